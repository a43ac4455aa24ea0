"""The Python entry point, in the reference's manner (ullm/llm.py:23-129):

    llm = LLM(EngineConfig(model=...))
    async for out in llm.generate(prompt_or_ids, SamplingParams(...)):
        ...                                   # one GenerateOutput per token
    llm.abort(sequence_id); await llm.shutdown()

plus a synchronous batch call for offline use, which needs no event loop and
no tokenizer:

    outs = llm.generate_batch([[1, 2, 3], [4, 5]], SamplingParams(max_new_tokens=8))

The reference hosts its engine in another process and feeds it over sockets;
here the engine lives in this process and `generate` drives `Engine.step`
from a background task.  A tokenizer is loaded only if the model folder has
one; token ids go in and out without it.
"""

from __future__ import annotations

import asyncio
import os
import uuid
from collections import deque
from typing import AsyncGenerator

from ..config.engine_config import EngineConfig
from ..sampling.params import EngineDeadError, FinishReason, GenerateOutput, RequestOutput, SamplingParams
from .engine import Engine


def init_tokenizer(model: str):
    """ullm/llm.py:12-20 (slow tokenizer, pad/unk default to eos); None when the
    folder has no tokenizer files."""
    names = ("tokenizer.json", "tokenizer_config.json", "vocab.json", "tokenizer.model")
    if not any(os.path.isfile(os.path.join(model, n)) for n in names):
        return None
    from transformers import AutoTokenizer

    tok = AutoTokenizer.from_pretrained(model, use_fast=False, trust_remote_code=True)
    if tok.pad_token is None:
        tok.pad_token = tok.eos_token
    if tok.unk_token is None:
        tok.unk_token = tok.eos_token
    return tok


class LLM:
    def __init__(self, config: EngineConfig):
        self.config = config
        self.engine = Engine(config)
        self.tokenizer = init_tokenizer(config.model)
        self.request_states: dict[str, asyncio.Queue] = {}
        self._loop_task: asyncio.Task | None = None
        self.is_dead = False  # set when a step raised: every later call raises EngineDeadError
        # Steps run in a worker thread while the event loop goes on taking requests and cancellations.  Those do
        # not touch the engine themselves: they are queued here and applied by the worker between two steps (the
        # reference sends them to its engine process over a socket, ullm/core/engine_client.py:299-326).
        self._commands: deque = deque()

    def _check_alive(self) -> None:
        if self.is_dead:
            raise EngineDeadError()

    def _apply_commands(self) -> list[tuple[str, Exception]]:
        """Queued additions and cancellations, in order; returns (sequence id, error) for those that failed."""
        errors = []
        while self._commands:
            cmd = self._commands.popleft()
            try:
                if cmd[0] == "add":
                    self.engine.add_sequence(*cmd[1:])
                else:
                    self.engine.abort_sequence(cmd[1])
            except Exception as e:
                errors.append((cmd[1], e))
        return errors

    def _step(self):
        """One step of the engine, after what was queued since the last (runs in the worker thread)."""
        errors = self._apply_commands()
        try:
            return self.engine.step(), errors
        except Exception:
            self.is_dead = True
            raise

    def _ensure_loop(self) -> None:
        if self._loop_task is None or self._loop_task.done():
            self._loop_task = asyncio.create_task(self._engine_loop())

    # -- text <-> ids ----------------------------------------------------------------
    def tokenize(self, texts: list[str]) -> list[list[int]]:
        if self.tokenizer is None:
            raise ValueError("the model folder has no tokenizer: pass token ids")
        return self.tokenizer(texts)["input_ids"]

    def detokenize(self, token_ids: list[list[int]]) -> list[str]:
        if self.tokenizer is None:
            return ["" for _ in token_ids]
        return self.tokenizer.batch_decode(token_ids, skip_special_tokens=True)

    def _params(self, params: SamplingParams | None) -> SamplingParams:
        from dataclasses import replace

        p = replace(params) if params is not None else self.config.get_default_sampling_params()
        if p.eos_token_id == -1:
            if self.tokenizer is not None and self.tokenizer.eos_token_id is not None:
                p.eos_token_id = self.tokenizer.eos_token_id
            elif self.engine.runner.spec.eos_token_id is not None:
                p.eos_token_id = self.engine.runner.spec.eos_token_id
        return p

    # -- streaming, as the reference ----------------------------------------------------
    async def _engine_loop(self) -> None:
        try:
            while self._commands or self.engine.has_unfinished_sequences():
                results, errors = await asyncio.to_thread(self._step)
                for sid, e in errors:
                    q = self.request_states.get(sid)
                    if q is not None:
                        q.put_nowait(e)
                for r in results:
                    q = self.request_states.get(r.seq_id)
                    if q is None:
                        continue
                    text = self.detokenize([[r.new_token_id]])[0] if r.new_token_id >= 0 else ""
                    if r.is_finished:
                        q.put_nowait(GenerateOutput(text, True, r.finish_reason, r.num_prompt_tokens,
                                                    r.num_generated_tokens, r.new_token_id))
                        q.put_nowait(None)
                    else:
                        q.put_nowait(GenerateOutput(text, False, None, 0, 0, r.new_token_id))
        except Exception as e:  # hand the failure to every waiting generator (ullm/llm.py:65-68)
            for q in self.request_states.values():
                q.put_nowait(e)

    async def generate(
        self,
        prompts: str | list[int],
        params: SamplingParams | None = None,
        sequence_id: str | None = None,
    ) -> AsyncGenerator[GenerateOutput, None]:
        self._check_alive()
        if sequence_id is None:
            sequence_id = uuid.uuid4().hex
        if sequence_id in self.request_states:  # (its queue would replace the live request's)
            raise ValueError(f"sequence {sequence_id!r} already exists")
        try:
            token_ids = prompts if isinstance(prompts, list) else self.tokenize([prompts])[0]
            q: asyncio.Queue = asyncio.Queue()
            sp = self._params(params)
            self.engine.check_prompt(token_ids)  # an empty prompt or an id outside the vocabulary raises here
            self.request_states[sequence_id] = q
            self._commands.append(("add", sequence_id, token_ids, sp))
            self._ensure_loop()
            while True:
                out = await q.get()
                if isinstance(out, Exception):
                    raise out
                if out is None:
                    break
                yield out
            self.request_states.pop(sequence_id, None)
        except (asyncio.CancelledError, GeneratorExit):
            self.abort(sequence_id)
            raise

    def abort(self, sequence_id: str) -> None:
        if self.is_dead:  # nothing to take back from an engine that is not stepped again
            self.request_states.pop(sequence_id, None)
            return
        if sequence_id in self.request_states:
            del self.request_states[sequence_id]
            self._commands.append(("abort", sequence_id))
            try:
                asyncio.get_running_loop()
                self._ensure_loop()  # (applies it even if nothing else is left to run)
            except RuntimeError:
                pass  # no event loop here: it is applied before the next step

    async def shutdown(self) -> None:
        if self._loop_task is not None:
            self._loop_task.cancel()
        self.engine.shutdown()

    async def profile(self, action: str) -> None:
        """"start" / "stop" the timing of steps and kernel groups; "stop" prints the tables and writes them
        to `profile_dir` (the reference starts and stops a torch profiler, ullm/core/engine.py:210-238)."""
        self._check_alive()
        self.engine.profile(action)

    # -- synchronous batch --------------------------------------------------------------
    def generate_batch(
        self,
        prompts: list[list[int] | str],
        params: SamplingParams | list[SamplingParams] | None = None,
        on_step=None,
    ) -> list[RequestOutput]:
        """Runs all prompts to completion under continuous batching and returns
        them in the order given."""
        self._check_alive()
        plist = params if isinstance(params, list) else [params] * len(prompts)
        ids_list, order = [], []
        for i, (pr, pa) in enumerate(zip(prompts, plist)):
            ids = pr if isinstance(pr, list) else self.tokenize([pr])[0]
            sid = f"batch-{uuid.uuid4().hex[:8]}-{i}"
            self.engine.add_sequence(sid, ids, self._params(pa))
            ids_list.append(list(ids)[-self.engine.context_len:])
            order.append(sid)
        got: dict[str, list[int]] = {sid: [] for sid in order}
        reason: dict[str, FinishReason | None] = {}
        while len(reason) < len(order) and self.engine.has_unfinished_sequences():
            for r in self._step()[0]:
                if r.seq_id not in got:
                    continue
                if r.new_token_id >= 0:
                    got[r.seq_id].append(r.new_token_id)
                if r.is_finished:
                    reason[r.seq_id] = r.finish_reason
            if on_step is not None:
                on_step(self.engine)
        outs = []
        for sid, ids in zip(order, ids_list):
            text = self.detokenize([got[sid]])[0] if self.tokenizer is not None else None
            outs.append(RequestOutput(sid, ids, got[sid], reason.get(sid), text))
        return outs
