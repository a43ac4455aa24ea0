"""The scheduler: admits requests, cuts prompts into portions under a token
budget, decodes, finishes and frees.

The reference (ullm/core/scheduler.py:63-147) is first-come-first-served and
prefill-first: a step is either whole prompts of waiting requests or one token
for each running request; it has no token budget, and its handling of a full
cache loses the victim or never returns (its `preempt` runs after the victim
was popped).  Here:

* order is first-come-first-served; a step takes, in this order, one token
  for every running request that is decoding, then portions of running
  requests whose prompt is not through yet, then newly admitted requests, until
  `max_num_batched_tokens` tokens are in the step;
* a request is admitted while fewer than `max_bs` are live, a request slot is
  free and the pages for its first portion are there (after evicting
  unreferenced prefix pages); at admission full pages that already hold a prefix
  of it are taken over instead of recomputed (ullm/core/scheduler.py:74-75 does
  the match at scheduling time too);
* when a running request cannot get the page it needs, the most recently
  admitted running request (be it the one that asked) is preempted: its pages
  are given back (full pages stay findable in the prefix tree), it returns to
  the FRONT of the waiting queue (ullm/core/scheduler.py:169-183) and is later
  recomputed from its prompt plus what it had generated.  If the request that
  asked is the only one running, it cannot fit the pool at all and is finished
  with reason LENGTH;
* a prompt that can never fit the pool is finished at once instead of blocking
  the queue.

The scheduler never touches the device; it talks to the cache manager's host
side only.
"""

from __future__ import annotations

import enum
from collections import deque
from dataclasses import dataclass, field

from ..cache import CacheManager, RequestCache
from ..sampling.params import FinishReason, SamplingParams


class SequenceStatus(enum.Enum):
    WAITING = enum.auto()
    RUNNING = enum.auto()
    FINISHED = enum.auto()


@dataclass
class Sequence:
    """ullm/core/common.py:63-179 without the slot lists (pages live in the
    cache manager): prompt and generated ids, how many are computed."""

    seq_id: str
    token_ids: list[int]
    num_prompt_tokens: int
    sampling_params: SamplingParams
    status: SequenceStatus = SequenceStatus.WAITING
    num_computed: int = 0  # tokens whose keys/values are in the cache
    cache: RequestCache | None = None
    seed: int = 0
    finish_reason: FinishReason | None = None
    num_preemptions: int = 0
    num_cached_prompt_tokens: int = 0
    # Steps may be launched before the host has read the token of the step before (the device keeps it):
    # such a token is a placeholder (-1) at the end of token_ids until it is read
    # (ullm/core/common.py:79,168-179 keeps `num_placeholder_tokens` for the same purpose).
    num_inflight: int = 0
    will_finish: bool = False  # a length limit is reached by a token that is still in flight

    @property
    def num_known_tokens(self) -> int:
        return len(self.token_ids) - self.num_inflight

    @property
    def num_tokens(self) -> int:
        return len(self.token_ids)

    @property
    def num_generated_tokens(self) -> int:
        return len(self.token_ids) - self.num_prompt_tokens

    @property
    def num_pending(self) -> int:
        return len(self.token_ids) - self.num_computed


@dataclass
class ScheduledSequence:
    seq: Sequence
    start: int  # first token of the portion
    num_tokens: int
    samples: bool  # the portion ends at the last known token: its logits give the next one


@dataclass
class SchedulerOutput:
    scheduled: list[ScheduledSequence] = field(default_factory=list)
    preempted: list[str] = field(default_factory=list)
    finished: list[tuple[Sequence, FinishReason]] = field(default_factory=list)  # finished by the scheduler itself

    @property
    def num_tokens(self) -> int:
        return sum(s.num_tokens for s in self.scheduled)


class Scheduler:
    def __init__(self, cache: CacheManager, max_bs: int, max_num_batched_tokens: int, context_len: int):
        self.cache = cache
        self.max_bs = max_bs
        self.max_num_batched_tokens = max_num_batched_tokens
        self.context_len = context_len
        self.sequences: dict[str, Sequence] = {}
        self.waiting: deque[Sequence] = deque()
        self.running: list[Sequence] = []  # in order of admission
        self.stats = dict(preemptions=0, prefix_hit_tokens=0, scheduled_tokens=0, steps=0)

    # -- queues -------------------------------------------------------------------
    def add_sequence(self, seq: Sequence) -> None:
        if seq.seq_id in self.sequences:
            raise ValueError(f"sequence {seq.seq_id!r} already exists")
        if not seq.token_ids:
            raise ValueError("a request needs at least one prompt token")
        seq.status = SequenceStatus.WAITING
        self.sequences[seq.seq_id] = seq
        self.waiting.append(seq)

    def get_sequence(self, seq_id: str) -> Sequence | None:
        return self.sequences.get(seq_id)

    def has_unfinished_sequences(self) -> bool:
        return bool(self.waiting or self.running)

    # -- one step's choice ----------------------------------------------------------
    def schedule(self) -> SchedulerOutput:
        out = SchedulerOutput()
        budget = self.max_num_batched_tokens
        ps = self.cache.page_size
        chosen: dict[str, ScheduledSequence] = {}

        def take(seq: Sequence, n: int) -> None:
            nonlocal budget
            chosen[seq.seq_id] = ScheduledSequence(seq, seq.num_computed, n, seq.num_computed + n == seq.num_tokens)
            budget -= n

        # 1. running requests, decoding ones first, each in order of admission
        order = [s for s in self.running if s.num_pending == 1] + [s for s in self.running if s.num_pending > 1]
        order = [s for s in order if s.num_pending > 0]
        for seq in order:
            if seq.status != SequenceStatus.RUNNING or budget <= 0 or seq.will_finish:
                continue
            n = min(seq.num_pending, budget)
            while not self.cache.can_reserve(seq.cache, n):
                fits = self._tokens_that_fit(seq)
                if seq.num_pending > 1 and fits >= 1:
                    n = min(n, fits)  # a shorter portion fits
                    break
                victim = self.running[-1]
                if victim is seq and len(self.running) == 1:
                    # alone and still no room: this request cannot fit the pool
                    chosen.pop(seq.seq_id, None)
                    self.finish_sequence(seq, FinishReason.LENGTH)
                    out.finished.append((seq, FinishReason.LENGTH))
                    n = 0
                    break
                if victim.seq_id in chosen:
                    budget += chosen.pop(victim.seq_id).num_tokens
                self.preempt(victim)
                out.preempted.append(victim.seq_id)
                if victim is seq:
                    n = 0
                    break
            if n > 0 and seq.status == SequenceStatus.RUNNING:
                self.cache.reserve(seq.cache, n)
                take(seq, n)

        # 2. admissions, first come first served
        while self.waiting and budget > 0 and len(self.running) < self.max_bs:
            seq = self.waiting[0]
            if self._can_never_fit(seq):
                self.waiting.popleft()
                self._finish_unadmitted(seq, FinishReason.LENGTH)
                out.finished.append((seq, FinishReason.LENGTH))
                continue
            rc = self.cache.admit(seq.seq_id, seq.token_ids)
            if rc is None:
                break  # no request slot
            seq.num_computed = rc.num_tokens
            n = min(seq.num_pending, budget)
            # room for the portion, and for one more page so that its first decode step does not preempt at once
            extra = 1 if seq.num_computed + n == seq.num_tokens else 0
            if not self._can_reserve_with_headroom(rc, n, extra):
                self.cache.release(rc)
                seq.num_computed = 0
                if not self.running:
                    # nothing else holds pages and it still does not fit: shrink the portion, or give up
                    rc = self.cache.admit(seq.seq_id, seq.token_ids)
                    seq.num_computed = rc.num_tokens
                    fits = self._tokens_that_fit_rc(rc)
                    if fits < 1:
                        self.cache.release(rc)
                        self.waiting.popleft()
                        self._finish_unadmitted(seq, FinishReason.LENGTH)
                        out.finished.append((seq, FinishReason.LENGTH))
                        continue
                    n = min(n, fits)
                else:
                    break
            self.waiting.popleft()
            seq.cache = rc
            seq.status = SequenceStatus.RUNNING
            seq.num_cached_prompt_tokens = rc.num_cached_tokens
            self.stats["prefix_hit_tokens"] += rc.num_cached_tokens
            self.running.append(seq)
            self.cache.reserve(rc, n)
            take(seq, n)

        out.scheduled = [chosen[s.seq_id] for s in self.running if s.seq_id in chosen]
        self.stats["scheduled_tokens"] += out.num_tokens
        self.stats["steps"] += 1
        return out

    def _tokens_that_fit(self, seq: Sequence) -> int:
        return self._tokens_that_fit_rc(seq.cache)

    def _tokens_that_fit_rc(self, rc: RequestCache) -> int:
        """How many more tokens this request can write with the pages that are
        free or evictable now."""
        ps = self.cache.page_size
        room = min(len(rc.pages[g]) + self.cache.num_available_pages(g) for g in range(len(self.cache.groups)))
        room = min(room, self.cache.max_pages_per_request)
        return max(0, room * ps - rc.num_tokens)

    def _can_reserve_with_headroom(self, rc: RequestCache, n: int, extra_pages: int) -> bool:
        if not self.cache.can_reserve(rc, n):
            return False
        need = self.cache.pages_needed(rc, n)
        return all(need[g] + extra_pages <= self.cache.num_available_pages(g) or not self.running
                   for g in range(len(need)))

    def _can_never_fit(self, seq: Sequence) -> bool:
        pages = -(-seq.num_tokens // self.cache.page_size)
        return pages > self.cache.num_pages or pages > self.cache.max_pages_per_request

    # -- transitions ------------------------------------------------------------------
    def preempt(self, seq: Sequence) -> None:
        """Back to the front of the waiting queue; its pages are given back (full
        pages stay in the prefix tree), everything it generated is kept."""
        if seq.status != SequenceStatus.RUNNING:
            return
        if seq.num_inflight:
            raise RuntimeError("a sequence with a token in flight cannot be preempted: read its step first")
        self.running.remove(seq)
        self.cache.release(seq.cache, seq.token_ids[: seq.num_computed])
        seq.cache = None
        seq.num_computed = 0
        seq.status = SequenceStatus.WAITING
        seq.num_preemptions += 1
        self.stats["preemptions"] += 1
        self.waiting.appendleft(seq)

    def on_step_done(self, sched: ScheduledSequence) -> None:
        """The step wrote this portion's keys and values."""
        seq = sched.seq
        if seq.status != SequenceStatus.RUNNING:
            return
        seq.num_computed += sched.num_tokens
        if self.cache.tree is not None:
            self.cache.publish(seq.cache, seq.token_ids[: min(seq.num_computed, seq.num_known_tokens)])

    def append_token(self, seq: Sequence, token_id: int) -> None:
        """ullm/core/scheduler.py:191-202."""
        if seq.status == SequenceStatus.RUNNING:
            seq.token_ids.append(int(token_id))

    def append_placeholder(self, seq: Sequence) -> int:
        """The step that samples this sequence's next token has been launched; returns the token's index."""
        seq.token_ids.append(-1)
        seq.num_inflight += 1
        return len(seq.token_ids) - 1

    def fill_placeholder(self, seq: Sequence, index: int, token_id: int) -> None:
        seq.token_ids[index] = int(token_id)
        seq.num_inflight -= 1

    def finish_sequence(self, seq: Sequence, reason: FinishReason | None = None) -> None:
        """ullm/core/scheduler.py:204-222: out of the queues, pages to the prefix
        tree (full ones) or back to the pool, slot released."""
        if seq.status == SequenceStatus.FINISHED:
            return
        if seq.status == SequenceStatus.WAITING:
            self.waiting.remove(seq)
        elif seq.status == SequenceStatus.RUNNING:
            self.running.remove(seq)
            self.cache.release(seq.cache, seq.token_ids[: min(seq.num_computed, seq.num_known_tokens)])
            seq.cache = None
        seq.status = SequenceStatus.FINISHED
        seq.finish_reason = reason
        self.sequences.pop(seq.seq_id, None)

    def _finish_unadmitted(self, seq: Sequence, reason: FinishReason) -> None:
        seq.status = SequenceStatus.FINISHED
        seq.finish_reason = reason
        self.sequences.pop(seq.seq_id, None)
