"""Engine: scheduler + step function + sampler, one `step()` at a time
(ullm/core/engine.py:24-200 is the reference's; its executor, worker processes
and batch queue collapse into direct calls here)."""

from __future__ import annotations

import logging
import time

import torch

from ..config.engine_config import EngineConfig
from ..sampling.params import EngineStepResult, FinishReason, SamplingParams
from ..sampling.sampler import Sampler
from .batch import StepEntry
from .runner import ModelRunner
from .scheduler import Scheduler, Sequence, SequenceStatus

logger = logging.getLogger("ullm_b200")


class Engine:
    def __init__(self, config: EngineConfig, runner: ModelRunner | None = None):
        self.config = config
        logging.basicConfig(level=getattr(logging, config.log_level.upper(), logging.INFO),
                            format="%(levelname)s %(asctime)s %(name)s: %(message)s")
        t0 = time.time()
        self.runner = runner or ModelRunner(
            config.model,
            dtype=config.dtype,
            device=config.device,
            page_size=config.page_size,
            num_pages=config.num_pages,
            gpu_memory_utilization=config.gpu_memory_utilization,
            max_requests=config.max_bs,
            max_context=config.context_len,
            max_step_tokens=config.max_num_batched_tokens,
            load_format=config.load_format,
            seed=config.seed,
            random_std=config.random_init_std,
            random_norm_std=config.random_init_norm_std,
            enable_prefix_cache=config.enable_prefix_caching,
        )
        cache = self.runner.cache
        logger.info("model ready in %.1f s; KV cache: %d pages of %d tokens (%d tokens)", time.time() - t0,
                    cache.num_pages, cache.page_size, cache.num_pages * cache.page_size)
        self.context_len = min(config.context_len, self.runner.max_context)
        self.scheduler = Scheduler(cache, config.max_bs, config.max_num_batched_tokens, self.context_len)
        self.sampler = Sampler(self.runner.device, max(config.max_bs, 1), self.runner.spec.vocab_size,
                               self.runner.last_tokens)
        self._cuda = self.runner.device.type == "cuda"
        self.async_decode = not config.disable_async_scheduling
        self._inflight = None
        self.decode_graphs = None
        if not config.enforce_eager and self.runner.device.type == "cuda":
            from .graph import DecodeGraphs

            self.decode_graphs = DecodeGraphs(self.runner, self.sampler, config.max_bs)
        self._seed_counter = 0
        from .profiler import StepProfiler

        self.profiler = StepProfiler(config.profile_dir, self._cuda)
        if config.warmup_graphs:
            n = self.warm_up_graphs()
            logger.info("recorded %d decode graphs", n)
        if config.profile:
            self.profile("start")

    # -- requests -------------------------------------------------------------------
    def add_sequence(self, sequence_id: str, prompt_token_ids: list[int], sampling_params: SamplingParams) -> None:
        """ullm/core/engine.py:72-90: a prompt longer than the context keeps its
        last `context_len` ids."""
        ids = self.check_prompt(prompt_token_ids)
        if len(ids) > self.context_len:
            ids = ids[-self.context_len:]
        seed = sampling_params.seed
        if seed is None:
            seed = (self.config.seed * 1000003 + self._seed_counter) & 0x7FFFFFFF
            self._seed_counter += 1
        seq = Sequence(sequence_id, ids, len(ids), sampling_params, seed=seed)
        self.scheduler.add_sequence(seq)
        logger.debug("Added sequence %s.", sequence_id)

    def check_prompt(self, prompt_token_ids) -> list[int]:
        """The prompt as a list of ints; ValueError if it is empty or holds an id outside the vocabulary."""
        ids = [int(t) for t in prompt_token_ids]
        if not ids:
            raise ValueError("empty prompt")
        V = self.runner.spec.vocab_size
        bad = [t for t in ids if not 0 <= t < V]
        if bad:
            raise ValueError(f"token id {bad[0]} is outside the vocabulary of {V}")
        return ids

    def abort_sequence(self, sequence_id: str) -> None:
        seq = self.scheduler.get_sequence(sequence_id)
        if seq:
            self.scheduler.finish_sequence(seq, FinishReason.ABORT)
        logger.debug("Aborted sequence %s.", sequence_id)

    def has_unfinished_sequences(self) -> bool:
        return self.scheduler.has_unfinished_sequences() or self._inflight is not None

    # -- one step ---------------------------------------------------------------------
    def step(self) -> list[EngineStepResult]:
        """Schedules a batch, runs it, samples, updates the sequences (ullm/core/engine.py:101-119).

        Decode steps are launched ahead: a step that holds one token per request is started before the
        tokens of the step before it have been read (each request's newest token stays on the device, the
        host passes -1 for it), and the results of the step before are read while this one runs.  What the
        reference calls asynchronous scheduling (ullm/core/engine.py:121-136) works the same way; as there, a
        request that stops on its eos token runs one more step whose output is dropped, while stops by length
        are known in advance and cost nothing.  `disable_async_scheduling` reads every step before the next.
        """
        results: list[EngineStepResult] = []
        if self._inflight is not None and self._must_read_first():
            results += self._collect(self._inflight)
            self._inflight = None
        sched = self.scheduler.schedule()
        results += [
            EngineStepResult(seq.seq_id, -1, True, reason, seq.num_prompt_tokens, seq.num_generated_tokens)
            for seq, reason in sched.finished
        ]
        if not sched.scheduled:
            if self._inflight is not None:
                results += self._collect(self._inflight)
                self._inflight = None
            return results
        rec = self.profiler.step_begin(sched.scheduled) if self.profiler.started else None
        sampling = [s for s in sched.scheduled if s.samples]
        params = [s.seq.sampling_params for s in sampling]
        seeds = [s.seq.seed for s in sampling]
        counters = [s.seq.num_generated_tokens for s in sampling]
        entries = [
            StepEntry(s.seq.seq_id, s.seq.token_ids[s.start:s.start + s.num_tokens],
                      [s.num_tokens - 1] if s.samples else [])
            for s in sched.scheduled
        ]
        decode_only = all(s.num_tokens == 1 and s.samples for s in sched.scheduled)
        if decode_only and self.decode_graphs is not None and self.decode_graphs.takes(len(entries)):
            handle = self.decode_graphs.launch(entries, params, seeds, counters)
        else:
            logits = self.runner.step(entries)
            handle = None
            if sampling:
                cache = self.runner.cache
                self.sampler.stage(params, seeds, counters, [cache.requests[s.seq.seq_id].slot for s in sampling])
                self.sampler.run(logits, len(sampling))
                from ..csrc import kernels

                handle = self.sampler.fetch_async(len(sampling), kernels().status if self._cuda else None)
        if rec is not None:
            self.profiler.step_launched(rec)
            if handle is None:
                self.profiler.step_read(rec)
        # bookkeeping that needs no token value: the portion is computed, the sampled token is a placeholder
        pending = []
        for s in sched.scheduled:
            self.scheduler.on_step_done(s)
            if s.samples:
                idx = self.scheduler.append_placeholder(s.seq)
                s.seq.will_finish = self._length_reached(s.seq, idx + 1)
                pending.append((s.seq, idx))
        this_step = (handle, pending, rec) if handle is not None else None
        if self._inflight is not None:  # read the step before while this one runs
            results += self._collect(self._inflight)
            self._inflight = None
        if this_step is not None:
            if self.async_decode and decode_only:
                self._inflight = this_step
            else:
                results += self._collect(this_step)
        return results

    def _must_read_first(self) -> bool:
        """The step in flight has to be read before the next is scheduled when scheduling may preempt (a
        preempted sequence is recomputed from its tokens, which must all be known).  It may when the running
        sequences TOGETHER want more pages for their next tokens than can be had: several of them can reach the
        end of a page in the same step."""
        cache = self.runner.cache
        need = [0] * len(cache.groups)
        for s in self.scheduler.running:
            if s.cache is None:
                continue
            if not cache.can_reserve(s.cache, 2):  # (also: a request at the most pages a request may hold)
                return True
            for g, k in enumerate(cache.pages_needed(s.cache, 2)):
                need[g] += max(int(k), 0)
        return any(need[g] > cache.num_available_pages(g) for g in range(len(need)))

    def _collect(self, step) -> list[EngineStepResult]:
        handle, pending, rec = step
        ids, status = self.sampler.wait(handle)
        if status:
            self.runner.check_device_status()
        results = []
        for (seq, idx), tok in zip(pending, ids):
            if seq.status != SequenceStatus.RUNNING:
                continue  # finished or aborted meanwhile: the token is dropped
            self.scheduler.fill_placeholder(seq, idx, tok)
            finished, reason = self._is_sequence_finished(seq, idx + 1, tok)
            if finished:
                del seq.token_ids[idx + 1:]  # a step launched ahead left a placeholder behind
                seq.num_inflight = 0
                self.scheduler.finish_sequence(seq, reason)
            results.append(EngineStepResult(seq.seq_id, tok, finished, reason, seq.num_prompt_tokens,
                                            idx + 1 - seq.num_prompt_tokens))
        if rec is not None:
            self.profiler.step_read(rec)
        return results

    def _length_reached(self, seq: Sequence, length: int) -> bool:
        p = seq.sampling_params
        return bool((p.max_tokens and length >= p.max_tokens)
                    or (p.max_new_tokens and length - seq.num_prompt_tokens >= p.max_new_tokens)
                    or length >= self.context_len)

    def _is_sequence_finished(self, seq: Sequence, length: int, token: int) -> tuple[bool, FinishReason | None]:
        """ullm/core/engine.py:175-200, same order: eos, max_tokens (total length), max_new_tokens, context
        length.  `length`: tokens of the sequence up to and including `token`."""
        p = seq.sampling_params
        if token == p.eos_token_id and not p.ignore_eos:
            return True, FinishReason.STOP
        if self._length_reached(seq, length):
            return True, FinishReason.LENGTH
        return False, None

    def warm_up_graphs(self) -> int:
        """Records the decode graphs of every padded batch size now, for even and for ragged batches, instead of
        at the first step of that size (the reference records its graphs while the engine starts,
        ullm/core/model_runner.py:428-500).  Each size runs one decode step of throw-away requests (one token of
        context each; for the ragged form one of them holds 33), which also times the library's products of
        that size; their pages and slots are given back.  Sizes the pool or the slots cannot hold are left for
        later.  Returns the number of graphs held afterwards."""
        from ..cache import OutOfPages

        dg = self.decode_graphs
        if dg is None or self.scheduler.running or self.scheduler.waiting or self._inflight is not None:
            return 0 if dg is None else len(dg.graphs)
        runner, greedy = self.runner, SamplingParams(temperature=0.0)
        # First the largest step there can be (a full token budget of prompt portions): the buffers that steps
        # work in grow to their final size, and a recorded graph is only good for the buffers it was recorded with.
        budget = self.scheduler.max_num_batched_tokens
        per = max(1, min(budget, self.context_len - 1))
        counts = [per] * (budget // per) + ([budget % per] if budget % per else [])
        admitted = []
        try:
            entries = []
            for i, n in enumerate(counts[: self.scheduler.max_bs]):
                rid = f"__warm_up_p{i}"
                if runner.add_request(rid) is None:
                    break
                admitted.append(rid)
                entries.append(StepEntry(rid, [0] * n, [n - 1]))
            if entries:
                runner.step(entries)
        except OutOfPages:
            pass
        finally:
            for rid in admitted:
                runner.end_request(rid)
        for size in dg.sizes:
            for ragged in ((False, True) if size > 1 else (False,)):
                ids = [f"__warm_up_{i}" for i in range(size)]
                admitted = []
                try:
                    for i, rid in enumerate(ids):
                        if runner.add_request(rid) is None:
                            raise OutOfPages("no request slot")
                        admitted.append(rid)
                        n = 33 if (ragged and i == 0) else 1
                        runner.step([StepEntry(rid, [0] * n, [])])
                    entries = [StepEntry(rid, [0], [0]) for rid in ids]
                    dg.run(entries, [greedy] * size, [0] * size, [0] * size)
                except OutOfPages:
                    pass
                finally:
                    for rid in admitted:
                        runner.end_request(rid)
        self.runner.check_device_status()
        return len(dg.graphs)

    def stats(self) -> dict:
        c = self.runner.cache
        d = dict(self.scheduler.stats)
        d.update(pages_total=c.num_pages, pages_free=c.num_free_pages(0),
                 pages_in_prefix_tree=c.tree.num_pages if c.tree is not None else 0,
                 steps_run=self.runner.steps_run)
        return d

    def profile(self, action: str) -> dict | None:
        """"start": steps are timed from now on (per step, and per kernel group for the steps that run
        eagerly).  "stop": the tables are printed and written as JSON into `profile_dir`; returns the report.
        The reference's engine starts and stops a torch profiler the same way (ullm/core/engine.py:210-238)."""
        if action == "start":
            self.profiler.start()
            return None
        if action == "stop":
            return self.profiler.stop()
        logger.warning("Unknown profiling action: %s, ignoring.", action)
        return None

    def shutdown(self) -> None:
        if self.profiler.started:
            self.profiler.stop()
        self.decode_graphs = None
