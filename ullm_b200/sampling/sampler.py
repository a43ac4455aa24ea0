"""Chooses the next token of each row of a batch of logits.

ullm/layers/sampler.py:20-56 is the reference: float32 logits / temperature,
top-k, top-p, min-p, softmax, one multinomial draw from torch's global
generator.  Here the filters and the draw are one CUDA kernel per row
(csrc/sampling.cu), greedy rows take its argmax branch, and the uniform number
of a row comes from a counter-based generator keyed by the request's seed and
its step count, so a request's tokens do not depend on its batch neighbours.
"""

from __future__ import annotations

import torch

from ..csrc import kernels
from .params import SamplingParams

_MASK64 = (1 << 64) - 1


def uniform_for(seed: int, step: int) -> float:
    """A number in [0, 1) from (seed, step): splitmix64 of a mixed key."""
    z = (seed * 0x9E3779B97F4A7C15 + (step + 1) * 0xBF58476D1CE4E5B9) & _MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
    z ^= z >> 31
    return (z >> 40) / float(1 << 24)


class Sampler:
    def __init__(self, device, max_rows: int, vocab_size: int, last_tokens: torch.Tensor | None = None):
        """`last_tokens` (int32 [request slots], on the device): if given, every sampled token is also stored
        under its request's slot, where a step launched before the host has read it finds it
        (ullm/core/model_runner.py:277-280 keeps `last_sampled_token` for the same purpose)."""
        self.device = torch.device(device)
        self.max_rows = max_rows
        self.vocab_size = vocab_size
        self.last_tokens = last_tokens
        pin = self.device.type == "cuda"
        # pinned blocks taken in turn: temperature, top_p, min_p, uniform (float32), top_k and request slot
        # (int32 bits).  A block is rewritten only after the copy that read it last has run (its event): with
        # steps launched ahead, the copy of step N may still be queued behind step N's forward when the host
        # stages step N + 1.
        self._hosts = [torch.zeros(6, max_rows, dtype=torch.float32, pin_memory=pin) for _ in range(4)]
        self._host_events = [torch.cuda.Event() if pin else None for _ in range(4)]
        self._host_next = 0
        self.host = self._hosts[0]
        self.dev = torch.zeros(6, max_rows, dtype=torch.float32, device=self.device)
        self.out = torch.zeros(max_rows, dtype=torch.int32, device=self.device)
        self.out_host = torch.zeros(max_rows, dtype=torch.int32, pin_memory=pin)
        # results that are read later (a step launched ahead): a few pinned buffers taken in turn
        self._ring = [torch.zeros(max_rows + 4, dtype=torch.int32, pin_memory=pin) for _ in range(4)]
        self._ring_events = [torch.cuda.Event() if pin else None for _ in range(4)]
        self._ring_next = 0

    def stage(self, params: list[SamplingParams], seeds: list[int], steps: list[int], slots=None) -> None:
        """Writes the rows' parameters (and request slots, -1 for none) into the pinned block and copies it."""
        R = len(params)
        if R > self.max_rows:
            raise ValueError(f"{R} rows to sample, room for {self.max_rows}")
        k = self._host_next
        self._host_next = (k + 1) % len(self._hosts)
        if self._host_events[k] is not None:
            self._host_events[k].synchronize()
        self.host = self._hosts[k]
        h = self.host.numpy()
        hk = self.host[4].view(torch.int32).numpy()
        hs = self.host[5].view(torch.int32).numpy()
        V = self.vocab_size
        hs[:] = -1
        for r, (p, seed, step) in enumerate(zip(params, seeds, steps)):
            h[0, r] = p.temperature if p.temperature > 0 else 0.0
            h[1, r] = p.top_p
            h[2, r] = p.min_p
            h[3, r] = uniform_for(seed, step) if p.temperature > 0 else 0.0
            hk[r] = V if p.top_k <= 0 else min(p.top_k, V)  # ullm/core/input_batch.py:163-171
        if slots is not None:
            hs[:R] = slots
        self.dev.copy_(self.host, non_blocking=True)
        if self._host_events[k] is not None:
            self._host_events[k].record()

    def run(self, logits: torch.Tensor, rows: int) -> torch.Tensor:
        """Samples rows 0..rows-1 of `logits` with the staged parameters; the
        ids stay on the device (int32 [rows])."""
        d = self.dev
        kernels().sample(logits[:rows], d[0], d[4].view(torch.int32), d[1], d[2], d[3], self.out,
                         row_slots=d[5].view(torch.int32) if self.last_tokens is not None else None,
                         last_tokens=self.last_tokens)
        return self.out[:rows]

    def fetch(self, rows: int) -> list[int]:
        self.out_host[:rows].copy_(self.out[:rows], non_blocking=False)
        return self.out_host[:rows].tolist()

    def fetch_async(self, rows: int, status: torch.Tensor | None = None):
        """Starts the copy of the sampled ids (and of the kernels' status word) to pinned memory and returns
        a handle for `wait`; the stream is not waited for."""
        k = self._ring_next
        self._ring_next = (k + 1) % len(self._ring)
        buf = self._ring[k]
        buf[:rows].copy_(self.out[:rows], non_blocking=True)
        if status is not None:
            buf[self.max_rows:self.max_rows + 4].copy_(status, non_blocking=True)
        else:
            buf[self.max_rows] = 0
        if self._ring_events[k] is not None:
            self._ring_events[k].record()
        return (k, rows)

    def wait(self, handle) -> tuple[list[int], int]:
        """(sampled ids, status code) of a `fetch_async` handle, once its copy has landed."""
        k, rows = handle
        if self._ring_events[k] is not None:
            self._ring_events[k].synchronize()
        buf = self._ring[k]
        return buf[:rows].tolist(), int(buf[self.max_rows])
