"""The Python entry point's behaviour that needs no GPU: what happens after a step of the engine has failed."""

import asyncio
import threading
import time
from collections import deque
from types import SimpleNamespace

import pytest

import ullm_b200
from ullm_b200.engine.llm import LLM
from ullm_b200.sampling.params import EngineStepResult, SamplingParams


class _FailingEngine:
    """Stands in for the engine: hands out one token, then its step raises."""

    context_len = 64

    def __init__(self):
        from types import SimpleNamespace

        self.runner = SimpleNamespace(spec=SimpleNamespace(eos_token_id=None))
        self.live: list[str] = []
        self.steps = 0
        self.profile_steps = False

    def check_prompt(self, ids):
        if not ids:
            raise ValueError("empty prompt")
        return list(ids)

    def add_sequence(self, sid, ids, params):
        self.live.append(sid)

    def abort_sequence(self, sid):
        self.live.remove(sid)

    def has_unfinished_sequences(self):
        return bool(self.live)

    def step(self):
        self.steps += 1
        if self.steps > 1:
            raise RuntimeError("kernel status 6")
        return [EngineStepResult(s, 7, False, None, 0, 0) for s in self.live]

    def shutdown(self):
        pass


def _llm() -> LLM:
    llm = LLM.__new__(LLM)
    llm.config = SimpleNamespace(get_default_sampling_params=SamplingParams)
    llm.engine = _FailingEngine()
    llm.tokenizer = None
    llm.request_states = {}
    llm._loop_task = None
    llm.is_dead = False
    llm._commands = deque()
    return llm


def test_exports_follow_the_reference():
    """ullm/__init__.py:10-17."""
    for name in ("LLM", "EngineConfig", "SamplingParams", "FinishReason", "GenerateOutput", "EngineDeadError"):
        assert getattr(ullm_b200, name) is not None


def test_a_failed_step_reaches_the_caller_and_the_engine_takes_no_more_requests():
    llm = _llm()
    with pytest.raises(RuntimeError, match="kernel status 6"):
        llm.generate_batch([[1, 2, 3]], SamplingParams(max_new_tokens=4))
    assert llm.is_dead and llm.engine.steps == 2
    with pytest.raises(ullm_b200.EngineDeadError):
        llm.generate_batch([[1, 2, 3]], SamplingParams(max_new_tokens=4))
    assert llm.engine.steps == 2  # not stepped again


def test_streaming_generators_get_the_failure_and_later_calls_raise_engine_dead():
    llm = _llm()

    async def run():
        got = []
        with pytest.raises(RuntimeError, match="kernel status 6"):
            async for out in llm.generate([1, 2, 3], SamplingParams(max_new_tokens=4), "a"):
                got.append(out.token_id)
        assert got == [7]
        with pytest.raises(ullm_b200.EngineDeadError):
            async for _ in llm.generate([1, 2], None, "b"):
                pass
        with pytest.raises(ullm_b200.EngineDeadError):
            await llm.profile("start")
        llm.abort("a")  # harmless on a dead engine
        await llm.shutdown()

    asyncio.run(run())


class _SlowEngine:
    """Steps take a while and record whether a request was added or cancelled while one was running."""

    context_len = 64

    def __init__(self):
        self.runner = SimpleNamespace(spec=SimpleNamespace(eos_token_id=None))
        self.live: dict[str, int] = {}
        self.in_step = False
        self.touched_during_step = 0
        self.threads = set()
        self.aborted: list[str] = []
        self.profile_steps = False

    def check_prompt(self, ids):
        return list(ids)

    def _touch(self):
        self.threads.add(threading.get_ident())
        if self.in_step:
            self.touched_during_step += 1

    def add_sequence(self, sid, ids, params):
        self._touch()
        if sid in self.live:
            raise ValueError(f"sequence {sid!r} already exists")
        self.live[sid] = params.max_new_tokens

    def abort_sequence(self, sid):
        self._touch()
        self.aborted.append(sid)
        self.live.pop(sid, None)

    def has_unfinished_sequences(self):
        return bool(self.live)

    def step(self):
        self.in_step = True
        time.sleep(0.02)
        out = []
        for sid in list(self.live):
            self.live[sid] -= 1
            done = self.live[sid] == 0
            out.append(EngineStepResult(sid, 5, done, None, 0, 0))
            if done:
                del self.live[sid]
        self.in_step = False
        return out

    def shutdown(self):
        pass


def test_requests_and_cancellations_reach_the_engine_only_between_steps():
    """Steps run in a worker thread; `generate` and `abort` are called from the event loop while one runs.  They
    are queued and applied by the worker between two steps, never while the scheduler's lists are in use."""
    llm = _llm()
    eng = llm.engine = _SlowEngine()

    async def consume(sid, n, cancel_after=None):
        got = 0
        agen = llm.generate([1, 2, 3], SamplingParams(max_new_tokens=n), sid)
        async for _ in agen:
            got += 1
            if cancel_after is not None and got == cancel_after:
                await agen.aclose()  # the caller goes away: the generator cancels its request
                break
        return got

    async def run():
        first = asyncio.create_task(consume("a", 40))
        await asyncio.sleep(0.03)  # a step is running now
        second = asyncio.create_task(consume("b", 6))
        third = asyncio.create_task(consume("c", 30, cancel_after=2))
        await asyncio.sleep(0.01)
        with pytest.raises(ValueError, match="already exists"):
            await consume("a", 3)  # a duplicate id: the error comes back to its caller only
        assert await first == 40 and await second == 6 and await third == 2
        await llm.shutdown()

    asyncio.run(run())
    assert eng.touched_during_step == 0
    assert "c" in eng.aborted and not eng.live
    assert len(eng.threads) >= 1
