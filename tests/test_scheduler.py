"""The scheduler's decisions, with the model replaced by a fake that 'samples'
a fixed token.  No GPU."""

import random

import pytest

from ullm_b200.cache import CacheManager
from ullm_b200.engine.scheduler import Scheduler, Sequence, SequenceStatus
from ullm_b200.parts import CacheNeed
from ullm_b200.sampling import FinishReason, SamplingParams

NEED = [(CacheNeed(2, 16, None), None, None)]


def setup(num_pages=16, page=4, max_bs=4, budget=8, context=64, prefix=True, needs=NEED):
    cache = CacheManager(needs, page, num_pages, max_bs, -(-context // page), device=None, enable_prefix_cache=prefix)
    return Scheduler(cache, max_bs, budget, context), cache


def seq(i, n, max_new=4, base=0):
    return Sequence(f"s{i}", [base + 1000 * i + j for j in range(n)], n, SamplingParams(max_new_tokens=max_new))


def run_step(s: Scheduler, cache, next_token=7, log=None):
    out = s.schedule()
    for x in out.scheduled:
        cache.reserve(x.seq.cache, x.num_tokens)  # what the runner's prepare does (no-op: already reserved)
        cache.commit(x.seq.cache, x.num_tokens)
        s.on_step_done(x)
        if x.samples:
            s.append_token(x.seq, next_token)
            p = x.seq.sampling_params
            if x.seq.num_generated_tokens >= p.max_new_tokens:
                s.finish_sequence(x.seq, FinishReason.LENGTH)
    cache.check_invariants()
    if log is not None:
        log.append(out)
    return out


def test_fcfs_decode_first_then_prompt_portions_under_the_budget():
    s, cache = setup(budget=8)
    a, b = seq(1, 5), seq(2, 13)
    s.add_sequence(a)
    s.add_sequence(b)
    o = run_step(s, cache)
    # a's whole prompt (5), then 3 tokens of b's prompt: 8 = the budget
    assert [(x.seq.seq_id, x.start, x.num_tokens, x.samples) for x in o.scheduled] == [("s1", 0, 5, True), ("s2", 0, 3, False)]
    o = run_step(s, cache)
    # a decodes first (1 token), b's next portion takes the rest of the budget
    assert [(x.seq.seq_id, x.start, x.num_tokens, x.samples) for x in o.scheduled] == [("s1", 5, 1, True), ("s2", 3, 7, False)]
    o = run_step(s, cache)
    assert [(x.seq.seq_id, x.start, x.num_tokens, x.samples) for x in o.scheduled] == [("s1", 6, 1, True), ("s2", 10, 3, True)]
    assert b.num_generated_tokens == 1


def test_max_bs_bounds_live_requests_and_order_is_arrival_order():
    s, cache = setup(max_bs=2, budget=64, num_pages=32)
    for i in range(4):
        s.add_sequence(seq(i, 3, max_new=2))
    o = run_step(s, cache)
    assert [x.seq.seq_id for x in o.scheduled] == ["s0", "s1"]
    assert len(s.running) == 2 and len(s.waiting) == 2
    run_step(s, cache)  # both finish (2 new tokens)
    o = run_step(s, cache)
    assert [x.seq.seq_id for x in o.scheduled] == ["s2", "s3"]


def test_one_token_prompt_and_finish_frees_everything():
    s, cache = setup(prefix=False)
    s.add_sequence(seq(1, 1, max_new=3))
    for _ in range(3):
        o = run_step(s, cache)
        assert len(o.scheduled) == 1 and o.scheduled[0].num_tokens == 1
    assert not s.has_unfinished_sequences()
    assert cache.num_free_pages() == 16 and cache.slots.num_free == 4


def test_decode_out_of_pages_preempts_the_newest_and_recomputes():
    # 5 pages of 4 tokens; two requests of 7 tokens take 2 pages each; at 8 tokens both need a third
    s, cache = setup(num_pages=5, page=4, budget=64, prefix=False)
    a, b = seq(1, 7, max_new=6), seq(2, 7, max_new=6)
    s.add_sequence(a)
    s.add_sequence(b)
    run_step(s, cache)  # both prompts; each holds 8 tokens' worth of ids, 7 computed
    assert len(s.running) == 2
    run_step(s, cache)  # token 8 of each still fits its second page
    o = run_step(s, cache)  # a takes the last page; b (the newest) finds none and is preempted
    assert o.preempted == ["s2"] and [x.seq.seq_id for x in o.scheduled] == ["s1"]
    assert b.status == SequenceStatus.WAITING and s.waiting[0] is b and b.num_preemptions == 1
    assert b.num_computed == 0 and b.num_generated_tokens == 2, "what it generated is kept for the recompute"
    steps = 0
    while s.has_unfinished_sequences():
        run_step(s, cache)
        steps += 1
        assert steps < 50
    assert a.num_generated_tokens == 6 and b.num_generated_tokens == 6
    assert cache.num_free_pages() == 5


def test_preempted_request_finds_its_pages_in_the_prefix_tree():
    s, cache = setup(num_pages=5, page=4, budget=64, prefix=True)
    a, b = seq(1, 7, max_new=6), seq(2, 7, max_new=6)
    s.add_sequence(a)
    s.add_sequence(b)
    run_step(s, cache)
    run_step(s, cache)
    o = run_step(s, cache)
    assert o.preempted == ["s2"]
    while s.has_unfinished_sequences():
        run_step(s, cache)
    assert s.stats["preemptions"] >= 1
    assert a.num_generated_tokens == 6 and b.num_generated_tokens == 6


def test_a_single_request_that_outgrows_the_pool_ends_with_length():
    s, cache = setup(num_pages=3, page=4, budget=64, context=64, prefix=False)
    a = seq(1, 10, max_new=50)
    s.add_sequence(a)
    outs = []
    for _ in range(10):
        outs.append(run_step(s, cache))
        if not s.has_unfinished_sequences():
            break
    assert a.status == SequenceStatus.FINISHED and a.finish_reason == FinishReason.LENGTH
    assert a.num_computed == 12 and a.num_tokens == 13, "it ran until the pool's 12 slots were full"
    assert any(o.finished for o in outs)
    assert cache.num_free_pages() == 3


def test_a_prompt_that_can_never_fit_does_not_block_the_queue():
    s, cache = setup(num_pages=3, page=4, budget=64, prefix=False)
    big, small = seq(1, 40), seq(2, 5, max_new=1)
    s.add_sequence(big)
    s.add_sequence(small)
    o = run_step(s, cache)
    assert [(q.seq_id, r) for q, r in o.finished] == [("s1", FinishReason.LENGTH)]
    assert [x.seq.seq_id for x in o.scheduled] == ["s2"]


def test_waiting_request_waits_for_pages_instead_of_failing():
    s, cache = setup(num_pages=4, page=4, budget=64, prefix=False)
    a, b = seq(1, 12, max_new=3), seq(2, 9, max_new=2)
    s.add_sequence(a)
    s.add_sequence(b)
    o = run_step(s, cache)
    assert [x.seq.seq_id for x in o.scheduled] == ["s1"], "b's prompt needs 3 pages, one is free"
    while a.status != SequenceStatus.FINISHED:
        o = run_step(s, cache)
        assert all(x.seq.seq_id == "s1" for x in o.scheduled)
    o = run_step(s, cache)
    assert [x.seq.seq_id for x in o.scheduled] == ["s2"]


def test_prefix_hit_at_admission_skips_cached_pages():
    s, cache = setup(num_pages=16, page=4, budget=64)
    a = seq(1, 13, max_new=1)
    s.add_sequence(a)
    run_step(s, cache)
    b = Sequence("b", a.token_ids[:12] + [5, 6, 7], 15, SamplingParams(max_new_tokens=1))
    s.add_sequence(b)
    o = run_step(s, cache)
    assert [(x.start, x.num_tokens) for x in o.scheduled] == [(12, 3)]
    assert b.num_cached_prompt_tokens == 12 and s.stats["prefix_hit_tokens"] == 12


def test_running_requests_publish_full_pages_for_later_arrivals():
    s, cache = setup(num_pages=16, page=4, budget=8, max_bs=2)
    a = seq(1, 13, max_new=8)
    s.add_sequence(a)
    run_step(s, cache)  # 8 tokens of a: two full pages are findable already
    b = Sequence("b", a.token_ids[:13] + [5], 14, SamplingParams(max_new_tokens=1))
    s.add_sequence(b)
    o = run_step(s, cache)  # a's last 5 prompt tokens, then b with the 3 tokens of budget left
    assert a.status == SequenceStatus.RUNNING
    assert b.num_cached_prompt_tokens == 8, "b takes over a's first pages while a is still running"
    assert b.cache.pages[0][:2] == a.cache.pages[0][:2]
    assert [(x.seq.seq_id, x.start, x.num_tokens) for x in o.scheduled] == [("s1", 8, 5), ("b", 8, 3)]
    while s.has_unfinished_sequences():
        run_step(s, cache)
    assert cache.num_free_pages() + cache.tree.num_evictable() == 16


def test_abort_and_finish_while_waiting():
    s, cache = setup()
    a, b = seq(1, 5), seq(2, 5)
    s.add_sequence(a)
    s.add_sequence(b)
    s.finish_sequence(b, FinishReason.ABORT)
    run_step(s, cache)
    s.finish_sequence(a, FinishReason.ABORT)
    assert not s.has_unfinished_sequences() and cache.slots.num_free == 4
    cache.check_invariants()


@pytest.mark.parametrize("seed", range(8))
def test_random_workloads_always_finish(seed):
    rng = random.Random(seed)
    page = rng.choice([1, 4, 16])
    context = 96
    num_pages = max(-(-context // page), rng.randint(8, 40))
    s, cache = setup(num_pages=num_pages, page=page, max_bs=rng.randint(1, 5), budget=rng.randint(1, 32), context=context,
                     prefix=rng.random() < 0.5)
    seqs = []
    pending = [Sequence(f"q{i}", [rng.randrange(6) for _ in range(rng.randint(1, 60))], 0,
                        SamplingParams(max_new_tokens=rng.randint(1, 30))) for i in range(20)]
    for q in pending:
        q.num_prompt_tokens = len(q.token_ids)
    steps = 0
    while pending or s.has_unfinished_sequences():
        if pending and rng.random() < 0.4:
            q = pending.pop()
            seqs.append(q)
            s.add_sequence(q)
        out = s.schedule()
        assert out.num_tokens <= s.max_num_batched_tokens
        assert len(s.running) <= s.max_bs
        for x in out.scheduled:
            cache.reserve(x.seq.cache, x.num_tokens)
            cache.commit(x.seq.cache, x.num_tokens)
            s.on_step_done(x)
            if x.samples:
                s.append_token(x.seq, rng.randrange(6))
                if (x.seq.num_generated_tokens >= x.seq.sampling_params.max_new_tokens
                        or x.seq.num_tokens >= context):
                    s.finish_sequence(x.seq, FinishReason.LENGTH)
        cache.check_invariants()
        steps += 1
        assert steps < 5000, "the scheduler must not loop"
    assert all(q.status == SequenceStatus.FINISHED for q in seqs)
    assert cache.slots.num_free == s.max_bs
    free = cache.num_free_pages() + (cache.tree.num_evictable() if cache.tree is not None else 0)
    assert free == num_pages


def test_decode_graph_sizes_and_padding():
    """ullm/core/model_runner.py:431-433 records 1, 2, 4, 8 and then steps of 16; the same here, sizes may be
    left out (their batches are padded to the next one), and the largest batch always has a graph of its own size."""
    from ullm_b200.engine.graph import graph_batch_sizes

    assert graph_batch_sizes(64) == [1, 2, 4, 8, 16, 32, 48, 64]
    assert graph_batch_sizes(64, skip=(8,)) == [1, 2, 4, 16, 32, 48, 64]
    assert graph_batch_sizes(50) == [1, 2, 4, 8, 16, 32, 48, 50]
    assert graph_batch_sizes(8) == [1, 2, 4, 8]
    assert graph_batch_sizes(3) == [1, 2, 3]
    assert graph_batch_sizes(1) == [1]
    assert graph_batch_sizes(64, smallest=16) == [16, 32, 48, 64]
    assert graph_batch_sizes(4, smallest=16) == [4]
    assert graph_batch_sizes(64, skip=()) == [1, 2, 4, 8, 16, 32, 48, 64]


def test_workspace_buffers_are_made_at_their_final_size():
    """A buffer with a row per token is made for the largest step at its first use, one with a row per request
    for all request slots; `generation` (which invalidates recorded graphs) only moves when a buffer is made or
    has to grow beyond that."""
    import torch

    from ullm_b200.engine.batch import Workspace

    ws = Workspace(torch.device("cpu"), max_tokens=64, max_requests=8)
    a = ws.tokens("x", 5, 16, torch.float32)
    assert a.shape == (5, 16) and ws.buffers[("x", 16, torch.float32)].shape == (64, 16) and ws.generation == 1
    b = ws.tokens("x", 64, 16, torch.float32)
    assert b.data_ptr() == a.data_ptr() and ws.generation == 1
    r = ws.requests("head", 2, 10, torch.float32)
    assert ws.buffers[("head", 10, torch.float32)].shape == (8, 10) and ws.generation == 2 and r.shape == (2, 10)
    ws.requests("head", 30, 10, torch.float32)  # a caller that wants logits at many places
    assert ws.buffers[("head", 10, torch.float32)].shape == (30, 10) and ws.generation == 3
    ws.get("scratch", 3, 4, torch.float32, reserve=100)
    assert ws.buffers[("scratch", 4, torch.float32)].shape == (100, 4)
    c = ws.tokens("x", 5, 32, torch.float32)  # another width under the same name: a buffer of its own
    assert ws.buffers[("x", 32, torch.float32)].shape == (64, 32) and ws.generation == 5
    # ... and the first one is still there: layers of two widths alternate without a new allocation
    assert ws.tokens("x", 7, 16, torch.float32).data_ptr() == a.data_ptr()
    assert ws.tokens("x", 7, 32, torch.float32).data_ptr() == c.data_ptr() and ws.generation == 5
