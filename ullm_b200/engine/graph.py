"""CUDA-graph replay of decode steps.

ullm/core/cuda_graph.py:9-97 and ullm/core/model_runner.py:428-500 capture the
model forward for batch sizes [1, 2, 4, 8, 16, 32, ...] and replay the smallest
one that fits, padding the batch.  Here the captured work is the whole device
side of a decode step: embedding to logits AND the sampling kernel.  The step's
integers and the sampling parameters live in fixed device buffers that are
refreshed by two small copies before each replay; block tables are on the
device already.  Graphs are captured on first use of a batch size, from the
live batch itself: that step runs eagerly, is recorded, and the recording is
replayed from the next step of that size on.
"""

from __future__ import annotations

import torch

from .batch import StepEntry


def graph_batch_sizes(max_bs: int, smallest: int = 1, skip: tuple = ()) -> list[int]:
    """ullm/core/model_runner.py:431-433: 1, 2, 4, 8, then steps of 16 up to max_bs.  `smallest` drops the sizes
    below it, `skip` leaves sizes out (their batches are padded to the next one).  Up to 8 rows a step's products
    are the weight-streaming kernel under dependent launch, whose cost grows with the rows (Qwen3-8B sizes, 8
    requests: 3.90 ms recorded at 8 rows, 4.26 at 16); with the library's products 8 requests were faster padded
    to 16 rows (4.05 against 4.19 ms)."""
    sizes = [b for b in (1, 2, 4, 8) if b <= max_bs and b not in skip] + list(range(16, max_bs + 1, 16))
    if max_bs not in sizes:
        sizes.append(max_bs)
    sizes = sorted(set(sizes))
    kept = [b for b in sizes if b >= min(smallest, sizes[-1])]
    return kept or sizes[-1:]


class DecodeGraphs:
    def __init__(self, runner, sampler, max_bs: int):
        self.runner = runner
        self.sampler = sampler
        import os

        skip = tuple(int(t) for t in os.environ.get("ULLM_B200_GRAPH_SKIP", "").split(",") if t.strip())
        self.sizes = graph_batch_sizes(max_bs, int(os.environ.get("ULLM_B200_MIN_GRAPH_BATCH", "1")), skip)
        # (size, the mixers' graph keys) -> (graph, signature, kernels recorded): a step is replayed from a graph
        # that was recorded with the kernels its mixers would choose for it (`Mixer.graph_key`)
        self.graphs: dict[tuple, tuple] = {}
        self.pool = None
        self.replays = 0

    def takes(self, batch: int) -> bool:
        return batch <= self.sizes[-1]

    def padded(self, batch: int) -> int:
        return next(s for s in self.sizes if s >= batch)

    def _signature(self) -> tuple:
        r = self.runner
        return (r.workspace.generation, r.decode_staging.dev.data_ptr(), self.sampler.dev.data_ptr())

    def run(self, entries: list[StepEntry], params, seeds, counters) -> list[int]:
        """One decode step for `entries` (one token each); returns their sampled ids."""
        ids, status = self.sampler.wait(self.launch(entries, params, seeds, counters))
        if status:
            from ..csrc import kernels

            kernels().raise_on_status()
        return ids

    def launch(self, entries: list[StepEntry], params, seeds, counters):
        """Starts one decode step and the copy of its sampled ids to the host; returns a handle for
        `sampler.wait`.  Nothing is waited for: the caller may prepare the next step meanwhile."""
        r = self.runner
        B = len(entries)
        Bp = self.padded(B)
        ctx = r.prepare(entries, pad_to=Bp, staging=r.decode_staging)
        self.sampler.stage(params, seeds, counters, [r.cache.requests[e.request_id].slot for e in entries])
        key = (Bp, r.model.graph_key(ctx))
        held = self.graphs.get(key)
        from ..csrc import kernels

        if held is None or held[1] != self._signature():
            # This step runs eagerly (which also sizes every workspace buffer) and is then recorded for the
            # steps to come.  The recording executes nothing, and the step is not replayed on top of its eager
            # run: with its input token taken from `last_tokens`, which the sampling kernel has just
            # overwritten, a second execution would be a different step.
            logits = r.run_model(ctx)
            self.sampler.run(logits, Bp)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            before = kernels().launches
            with torch.cuda.graph(g, pool=self.pool):
                logits = r.run_model(ctx)
                self.sampler.run(logits, Bp)
            captured = kernels().launches - before
            kernels().launches = before  # recording launched nothing
            if self.pool is None:
                self.pool = g.pool()
            self.graphs[key] = (g, self._signature(), captured)
        else:
            held[0].replay()
            self.replays += 1
            kernels().launches += held[2]
        _k = kernels
        handle = self.sampler.fetch_async(B, _k().status)
        r.commit(entries)
        return handle
