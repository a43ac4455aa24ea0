"""Generation through the Python entry point: greedy tokens against the plain
implementation, chunked prompts under a token budget, prefix sharing, CUDA-graph
decode against eager decode, preemption under a tiny pool, sampling that does
not depend on the batch."""

import asyncio

import pytest
import torch

import plain_model as pm
from conftest import device
from helpers import random_ids, weights_for, write_model_dir

pytestmark = pytest.mark.gpu


def make_llm(tmp_path, tag, dtype="float32", **kw):
    from ullm_b200 import LLM, EngineConfig

    cfg, w, page = weights_for(tag, dtype)
    d = write_model_dir(str(tmp_path / f"m{tag}{dtype}{len(kw)}"), cfg, w)
    args = dict(model=d, max_bs=4, context_len=cfg["max_position_embeddings"], page_size=page, num_pages=64,
                max_num_batched_tokens=64, dtype=dtype)
    args.update(kw)
    ec = EngineConfig(**args)
    if device() == "cpu":
        type(ec).device = property(lambda self: "cpu")
    return LLM(ec), cfg, {k: v.float() for k, v in w.items()}


def test_tiny_a_workload_greedy(tmp_path):
    """3 requests, prompts of 5, 11 and 17 ids, 8 greedy tokens each."""
    from ullm_b200 import SamplingParams

    llm, cfg, w = make_llm(tmp_path, "A")
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, 256, (n,), generator=g).tolist() for n in (5, 11, 17)]
    outs = llm.generate_batch(prompts, SamplingParams(temperature=0.0, max_new_tokens=8, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.token_ids == pm.greedy_generate(p, w, cfg, 8)
        assert o.finish_reason.name == "LENGTH" and o.num_prompt_tokens == len(p)
    llm.engine.runner.cache.check_invariants()


@pytest.mark.parametrize("eager", [True, False])
def test_tiny_b_workload_chunked_with_shared_prefix(tmp_path, eager):
    """5 requests (prompts 1, 7, 16, 33, 64), 12 new tokens, token budget 8,
    plus two requests that share a 32-token prefix."""
    from ullm_b200 import SamplingParams

    llm, cfg, w = make_llm(tmp_path, "B", max_num_batched_tokens=8, max_bs=3, enforce_eager=eager)
    prompts = [random_ids(331, n, 70 + n) for n in (1, 7, 16, 33, 64)]
    shared = random_ids(331, 32, 99)
    prompts += [shared + [5, 6, 7]]
    sp = SamplingParams(temperature=0.0, max_new_tokens=12, ignore_eos=True)
    outs = llm.generate_batch(prompts, sp)
    prompts += [shared + [9]]
    outs += llm.generate_batch(prompts[-1:], sp)
    for p, o in zip(prompts, outs):
        assert o.token_ids == pm.greedy_generate(p, w, cfg, 12), f"prompt of {len(p)}"
    st = llm.engine.stats()
    assert st["prefix_hit_tokens"] >= 32, "the second request with the shared prefix reuses its pages"
    if not eager and device() != "cpu":
        assert llm.engine.decode_graphs.replays > 0
    llm.engine.runner.cache.check_invariants()


def test_preemption_under_a_tiny_pool_keeps_the_tokens(tmp_path):
    from ullm_b200 import SamplingParams

    llm, cfg, w = make_llm(tmp_path, "B", num_pages=7, max_bs=3, max_num_batched_tokens=32)
    prompts = [random_ids(331, n, 80 + n) for n in (30, 20, 25)]
    outs = llm.generate_batch(prompts, SamplingParams(temperature=0.0, max_new_tokens=30, ignore_eos=True))
    assert llm.engine.stats()["preemptions"] >= 1, "7 pages of 16 cannot hold three requests of ~55 tokens"
    for p, o in zip(prompts, outs):
        assert o.token_ids == pm.greedy_generate(p, w, cfg, 30)
    llm.engine.runner.cache.check_invariants()


def test_requests_that_reach_a_page_end_in_the_same_step_with_too_few_pages_left(tmp_path):
    """Six requests of equal length decode side by side, steps launched ahead, and all need a new page in the
    same step while three are left: some are preempted (after the step in flight has been read: their tokens must
    be known to be recomputed), all finish with the tokens of the plain implementation."""
    from ullm_b200 import SamplingParams

    llm, cfg, w = make_llm(tmp_path, "B", num_pages=15, max_bs=6, max_num_batched_tokens=64)
    page = llm.engine.runner.cache.page_size
    n = 2 * page - 2
    prompts = [random_ids(331, n, 300 + i) for i in range(6)]
    outs = llm.generate_batch(prompts, SamplingParams(temperature=0.0, max_new_tokens=24, ignore_eos=True))
    assert llm.engine.stats()["preemptions"] >= 1
    for p, o in zip(prompts, outs):
        assert o.token_ids == pm.greedy_generate(p, w, cfg, 24)
    llm.engine.runner.cache.check_invariants()


@pytest.mark.needs_cuda
def test_graphs_recorded_at_start_up_are_the_ones_generation_replays(tmp_path):
    """`warmup_graphs`: every padded batch size is recorded (even and ragged form) before the first request, the
    throw-away requests leave nothing behind, and generation then only replays: same tokens as the plain
    implementation, no new graph."""
    from ullm_b200 import SamplingParams

    llm, cfg, w = make_llm(tmp_path, "D", dtype="bfloat16", max_bs=4, num_pages=64, warmup_graphs=True)
    dg = llm.engine.decode_graphs
    # per size one graph for even batches and (from two requests on) one for the attention mixer's "ragged" key
    assert set(dg.graphs) == {(s, (r,)) for s in dg.sizes for r in (((), ("ragged",)) if s > 1 else ((),))}
    cache = llm.engine.runner.cache
    assert not cache.requests and cache.num_free_pages(0) == 64
    cache.check_invariants()
    held = {k: v[0] for k, v in dg.graphs.items()}
    prompts = [random_ids(cfg["vocab_size"], n, 500 + n) for n in (9, 40, 3)]
    outs = llm.generate_batch(prompts, SamplingParams(temperature=0.0, max_new_tokens=12, ignore_eos=True))
    llm32, _, w32 = make_llm(tmp_path, "D", dtype="bfloat16", max_bs=4, num_pages=64, enforce_eager=True)
    ref = llm32.generate_batch(prompts, SamplingParams(temperature=0.0, max_new_tokens=12, ignore_eos=True))
    assert [o.token_ids for o in outs] == [o.token_ids for o in ref]
    assert dg.replays > 0 and all(dg.graphs[k][0] is g for k, g in held.items())


@pytest.mark.needs_cuda
def test_a_recorded_graph_survives_larger_steps_that_come_later(tmp_path):
    """Step buffers are made at their final size at first use (a row per token of the largest step, a row per
    request slot), so a decode graph recorded after a short prompt is still good after a prompt that fills the
    token budget and after a larger batch: it is the same graph object, and the workspace's generation stands."""
    from ullm_b200 import SamplingParams

    llm, cfg, w = make_llm(tmp_path, "D", dtype="bfloat16", max_bs=4, num_pages=64, max_num_batched_tokens=64)
    sp = SamplingParams(temperature=0.0, max_new_tokens=6, ignore_eos=True)
    llm.generate_batch([random_ids(cfg["vocab_size"], 5, 600)], sp)
    dg, ws = llm.engine.decode_graphs, llm.engine.runner.workspace
    held, gen = {k: v[0] for k, v in dg.graphs.items()}, ws.generation
    assert held
    prompts = [random_ids(cfg["vocab_size"], n, 601 + n) for n in (150, 64, 9, 31)]
    llm.generate_batch(prompts, sp)
    assert ws.generation == gen
    assert all(dg.graphs[k][0] is g for k, g in held.items())


def test_finish_rules(tmp_path):
    from ullm_b200 import SamplingParams

    llm, cfg, w = make_llm(tmp_path, "A", context_len=40)
    p = random_ids(256, 10, 5)
    ref = pm.greedy_generate(p, w, cfg, 30)
    # eos stops (and is emitted), unless ignored
    o = llm.generate_batch([p], SamplingParams(temperature=0.0, max_new_tokens=30, eos_token_id=ref[3]))[0]
    stop_at = ref.index(ref[3]) + 1
    assert o.token_ids == ref[:stop_at] and o.finish_reason.name == "STOP"
    # max_tokens bounds prompt + generated
    o = llm.generate_batch([p], SamplingParams(temperature=0.0, max_tokens=14, ignore_eos=True))[0]
    assert len(o.token_ids) == 4 and o.finish_reason.name == "LENGTH"
    # the context length bounds everything; a longer prompt keeps its last ids
    o = llm.generate_batch([p], SamplingParams(temperature=0.0, ignore_eos=True))[0]
    assert len(o.token_ids) == 30
    long = random_ids(256, 55, 6)
    o = llm.generate_batch([long], SamplingParams(temperature=0.0, max_new_tokens=2, ignore_eos=True))[0]
    assert o.prompt_token_ids == long[-40:] and len(o.token_ids) == 1


@pytest.mark.parametrize("eager", [True, False])
def test_steps_launched_ahead_give_the_same_tokens_as_steps_read_one_by_one(tmp_path, eager, monkeypatch):
    """Decode steps are launched before the tokens of the step before are read.  Requests that stop on an eos
    token at different times (their extra step is dropped), by length, and a request that arrives late must
    give what the synchronous engine gives, and every page comes back.  Graphs for batches of 1, 2 and 3 are
    recorded in mid-stream, from steps whose input token is still on the device only."""
    from ullm_b200 import SamplingParams

    monkeypatch.setenv("ULLM_B200_MIN_GRAPH_BATCH", "1")

    prompts = [random_ids(331, n, 40 + n) for n in (3, 18, 9, 30, 5)]
    outs = {}
    for sync in (True, False):
        llm, cfg, w = make_llm(tmp_path, "B", max_bs=3, max_num_batched_tokens=16, enforce_eager=eager,
                               disable_async_scheduling=sync)
        refs = [pm.greedy_generate(p, w, cfg, 20) for p in prompts]
        sps = [SamplingParams(temperature=0.0, max_new_tokens=20, eos_token_id=r[k])
               for r, k in zip(refs, (2, 19, 7, 11, 0))]
        sps[1] = SamplingParams(temperature=0.0, max_new_tokens=13, ignore_eos=True)
        got = llm.generate_batch(prompts, sps)
        for p, r, sp, o in zip(prompts, refs, sps, got):
            if sp.ignore_eos:
                want, reason = r[:13], "LENGTH"
            else:
                want, reason = r[:r.index(sp.eos_token_id) + 1], "STOP"
            assert o.token_ids == want and o.finish_reason.name == reason, f"prompt of {len(p)}, sync={sync}"
        assert llm.engine._inflight is None
        cache = llm.engine.runner.cache
        cache.check_invariants()
        assert not cache.requests, "every request gave its pages back"
        outs[sync] = [o.token_ids for o in got]
    assert outs[True] == outs[False]


def test_async_generate_streams_tokens(tmp_path):
    from ullm_b200 import SamplingParams

    llm, cfg, w = make_llm(tmp_path, "A")
    p1, p2 = random_ids(256, 9, 1), random_ids(256, 4, 2)

    async def consume(p):
        toks = []
        async for out in llm.generate(p, SamplingParams(temperature=0.0, max_new_tokens=6, ignore_eos=True)):
            toks.append(out.token_id)
            last = out
        assert last.is_finished and last.num_generated_tokens == 6 and last.num_prompt_tokens == len(p)
        return toks

    async def main():
        r = await asyncio.gather(consume(p1), consume(p2))
        await llm.shutdown()
        return r

    t1, t2 = asyncio.run(main())
    assert t1 == pm.greedy_generate(p1, w, cfg, 6) and t2 == pm.greedy_generate(p2, w, cfg, 6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sampled_tokens_do_not_depend_on_the_batch(tmp_path, dtype):
    from ullm_b200 import SamplingParams

    llm, cfg, w = make_llm(tmp_path, "B", dtype=dtype)
    prompts = [random_ids(331, n, 90 + n) for n in (7, 16, 33)]
    sp = [SamplingParams(temperature=0.7, top_k=20, top_p=0.95, max_new_tokens=12, ignore_eos=True, seed=4 + i)
          for i in range(3)]
    together = llm.generate_batch(prompts, sp)
    for p, s, o in zip(prompts, sp, together):
        alone = llm.generate_batch([p], s)[0]
        if dtype == "float32":
            assert alone.token_ids == o.token_ids
        assert len(o.token_ids) == 12
    # temperature sampling follows the filtered distribution of the plain implementation
    if dtype == "float32":
        p = prompts[1]
        o = together[1]
        ids = list(p)
        from ullm_b200.sampling import uniform_for

        for step, tok in enumerate(o.token_ids):
            lg = pm.forward_logits(ids, w, cfg)[-1]
            probs = pm.filtered_distribution(lg, 0.7, 20, 0.95, 0.0)
            assert probs[tok] > 0, f"step {step}: token {tok} is outside the top-k/top-p set"
            assert tok == pm.inverse_cdf_draw(probs, uniform_for(5, step))
            ids.append(tok)


def test_long_decoding_bf16_tracks_the_plain_logits(tmp_path):
    """120 greedy tokens in bfloat16; every chosen token's plain logit is within
    the bfloat16 tolerance of the plain maximum (teacher-forced on the engine's
    own tokens, so one near-tie cannot derail the comparison)."""
    from helpers import TOL
    from ullm_b200 import SamplingParams

    llm, cfg, w = make_llm(tmp_path, "C", dtype="bfloat16")
    p = random_ids(509, 20, 7)
    o = llm.generate_batch([p], SamplingParams(temperature=0.0, max_new_tokens=120, ignore_eos=True))[0]
    assert len(o.token_ids) == 120
    lg = pm.forward_logits(p + o.token_ids, w, cfg)
    scale = lg.abs().max().item()
    for i, tok in enumerate(o.token_ids):
        row = lg[len(p) - 1 + i]
        assert row.max().item() - row[tok].item() <= 2 * TOL["bfloat16"] * scale, f"token {i}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generation_with_head_size_64_through_decode_graphs(tmp_path, dtype):
    """Config D (head size 64): bfloat16 decode steps run the split tensor-core attention inside CUDA
    graphs, float32 the general kernel; both follow the plain implementation."""
    from helpers import TOL
    from ullm_b200 import SamplingParams

    llm, cfg, w = make_llm(tmp_path, "D", dtype=dtype, max_bs=5, max_num_batched_tokens=48)
    prompts = [random_ids(777, n, 30 + n) for n in (3, 50, 17, 130, 64)]
    outs = llm.generate_batch(prompts, SamplingParams(temperature=0.0, max_new_tokens=24, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert len(o.token_ids) == 24
        if dtype == "float32":
            assert o.token_ids == pm.greedy_generate(p, w, cfg, 24)
        else:
            lg = pm.forward_logits(p + o.token_ids, w, cfg)
            scale = lg.abs().max().item()
            for i, tok in enumerate(o.token_ids):
                row = lg[len(p) - 1 + i]
                assert row.max().item() - row[tok].item() <= 2 * TOL[dtype] * scale, f"token {i}"
    if device() != "cpu":
        assert llm.engine.decode_graphs.replays > 0


@pytest.mark.needs_cuda
def test_command_line_writes_a_random_model_and_generates_from_it(tmp_path):
    """`random-model` writes a folder from a config and a seed; `generate` loads it and prints one JSON line per
    prompt.  The greedy tokens are those of the plain implementation on the same weights."""
    import json
    import os
    import subprocess
    import sys

    from tiny_configs import TINY_A
    from ullm_b200.weights.safetensors_io import SafetensorsFile

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(TINY_A))
    model = tmp_path / "model"
    env = dict(os.environ, PYTHONPATH=root)
    r = subprocess.run([sys.executable, "-m", "ullm_b200.engine.cli", "random-model", "--out", str(model), "--config",
                        str(cfg_path), "--seed", "3", "--std", "0.05", "--norm-std", "0.1"],
                       capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert (model / "config.json").is_file() and (model / "model.safetensors").is_file()
    prompts = [random_ids(256, 9, 1), random_ids(256, 21, 2)]
    cmd = [sys.executable, "-m", "ullm_b200.engine.cli", "generate", "--model", str(model), "--max-bs", "2",
           "--context-len", "64", "--page-size", "4", "--num-pages", "40", "--temperature", "0", "--ignore-eos",
           "--max-new-tokens", "7"]
    for p in prompts:
        cmd += ["--prompt-ids", ",".join(map(str, p))]
    r = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 2
    f = SafetensorsFile(str(model / "model.safetensors"))
    w = {k: f.get(k).float().clone() for k in f.names()}
    f.close()
    for p, out in zip(prompts, lines):
        assert out["prompt_tokens"] == len(p) and out["finish_reason"] == "LENGTH"
        assert out["token_ids"] == pm.greedy_generate(p, w, TINY_A, 7)


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_random_workloads_through_the_engine_follow_the_plain_implementation(tmp_path, seed, monkeypatch):
    """Random prompts (some share a prefix), random lengths to generate, random arrival (a few requests are added
    while others decode), a small pool (preemption and page reuse), a small token budget (chunked prompts),
    decode graphs of every size recorded in mid-stream: every request's greedy tokens are those of the plain
    implementation, and every page comes back."""
    import random

    from ullm_b200 import SamplingParams

    monkeypatch.setenv("ULLM_B200_MIN_GRAPH_BATCH", "1")
    rng = random.Random(100 + seed)
    llm, cfg, w = make_llm(tmp_path, "B", max_bs=4, max_num_batched_tokens=rng.choice([8, 24, 64]),
                           num_pages=rng.choice([10, 14, 40]))
    V = cfg["vocab_size"]
    shared = random_ids(V, 33, 500 + seed)
    reqs = []
    for i in range(9):
        n = rng.choice([1, 2, 5, 16, 17, 31, 40, 64])
        p = random_ids(V, n, 600 + 10 * seed + i)
        if rng.random() < 0.3:
            p = shared + p[:8]
        reqs.append((p, rng.choice([1, 2, 7, 15, 24])))
    eng = llm.engine
    got = {}
    pending = list(enumerate(reqs))
    rng.shuffle(pending)
    live = 0
    steps = 0
    while pending or eng.has_unfinished_sequences():
        # a new arrival now and then, otherwise step
        if pending and (live == 0 or rng.random() < 0.25):
            i, (p, n_new) = pending.pop()
            eng.add_sequence(f"r{i}", p, SamplingParams(temperature=0.0, max_new_tokens=n_new, ignore_eos=True))
            got[i] = []
            live += 1
            continue
        for res in eng.step():
            i = int(res.seq_id[1:])
            if res.new_token_id >= 0:
                got[i].append(res.new_token_id)
            if res.is_finished:
                live -= 1
        steps += 1
        assert steps < 5000, "the engine does not finish"
    for i, (p, n_new) in enumerate(reqs):
        assert got[i] == pm.greedy_generate(p, w, cfg, n_new), f"request {i}: prompt of {len(p)}, {n_new} new tokens"
    cache = eng.runner.cache
    cache.check_invariants()
    assert not cache.requests


@pytest.mark.needs_cuda
def test_pool_sized_from_free_memory_when_no_page_count_is_given(tmp_path):
    """Without `num_pages` the pool comes from the free device memory times `gpu_memory_utilization`, capped at
    twice what `max_bs` requests of `context_len` tokens can hold; generation works on it."""
    from ullm_b200 import SamplingParams

    llm, cfg, w = make_llm(tmp_path, "A", num_pages=None, max_bs=3, context_len=64, gpu_memory_utilization=0.5)
    cache = llm.engine.runner.cache
    assert cache.num_pages == 3 * (64 // 4) * 2
    p = random_ids(256, 12, 3)
    o = llm.generate_batch([p], SamplingParams(temperature=0.0, max_new_tokens=6, ignore_eos=True))[0]
    assert o.token_ids == pm.greedy_generate(p, w, cfg, 6)
