"""Schedules and paths that the replay tests do not reach by themselves, each against the plain
implementation: a layer run twice and a layer that reads another execution's cache; a prefix hit whose first
portion starts in the middle of the context (bfloat16, tensor-core prompt kernels); very unequal decode batches
replayed from a CUDA graph; temperature sampling in bfloat16; the whole 28-layer model at the widths of
Qwen3-0.6B in 32-bit; two layers of different width decoding through one graph; steps launched ahead while the
GPU lags behind the host; the profiler's report; the kernels' bounded waits."""

import json
import os

import pytest
import torch

import plain_model as pm
from conftest import device
from helpers import TOL, assert_close, first_bad_row, plain_logits, random_ids, weights_for, write_model_dir
from test_gpu_replay import make_runner, run_cut

pytestmark = pytest.mark.gpu


# ---------------------------------------------------------------------------------------------------------
# a schedule that names a layer twice and lets an execution read an earlier execution's cache
# ---------------------------------------------------------------------------------------------------------
ENGINE_SCHEDULE = [(0, None), (1, None), (1, None), (2, None), (1, 2)]  # (layer, cache_of)


@pytest.fixture
def twice_architecture():
    from ullm_b200.config import ARCHITECTURES, Qwen3Config, ScheduleEntry, qwen3_model_spec, register_architecture

    def spec(cfg):
        s = qwen3_model_spec(cfg)
        s.architecture = "TwiceForCausalLM"
        s.schedule = [ScheduleEntry(l, c) for l, c in ENGINE_SCHEDULE]
        return s

    register_architecture("TwiceForCausalLM", Qwen3Config.from_dict, spec)
    yield "TwiceForCausalLM"
    ARCHITECTURES.pop("TwiceForCausalLM")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_repeated_layer_and_shared_cache_schedule(tmp_path, twice_architecture, dtype):
    """Tiny B with the schedule 0, 1, 1, 2, 1 where the last execution of layer 1 reads the keys and values that
    its second execution wrote: whole, last 32 one by one, and in portions, against the plain implementation
    run with the same schedule."""
    from ullm_b200.engine import ModelRunner

    cfg, w, page = weights_for("B", dtype)
    cfg = dict(cfg, architectures=[twice_architecture])
    d = write_model_dir(str(tmp_path / f"twice_{dtype}"), cfg, w)
    runner = ModelRunner(d, dtype=dtype, device=device(), page_size=page, num_pages=16, max_requests=2,
                         max_context=cfg["max_position_embeddings"], max_step_tokens=64, poison_cache=True)
    # four executions keep a cache of their own, the fifth reads the third's
    assert len(runner.cache.groups) == 1 and len(runner.cache.groups[0].executions) == 4
    n = 120
    ids = random_ids(cfg["vocab_size"], n, 31)
    ref = plain_logits(ids, w, cfg, schedule=ENGINE_SCHEDULE)
    assert not torch.allclose(ref, plain_logits(ids, w, cfg), atol=1e-3), "the schedule must matter"
    for cuts, what in (([n], "whole"), ([n - 32] + [1] * 32, "decode"), ([7, 2, 5, 3, 16, 2, 1, 9, 4, 17, 2, 33, 19], "portions")):
        got = run_cut(runner, f"r-{what}", ids, cuts)
        bad = first_bad_row(got, ref, dtype)
        assert bad is None, f"{what}: first wrong position {bad}"
        assert_close(got, ref, dtype, f"schedule {what}")
    runner.cache.check_invariants()


# ---------------------------------------------------------------------------------------------------------
# prefix hit: the first portion of the second request starts at a position > 0 (bf16 prompt kernels)
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.needs_cuda
@pytest.mark.parametrize("tag,shared", [("D", 32), ("D", 48), ("E", 32), ("E", 48)])
def test_prefix_hit_in_bfloat16_first_portion_starts_inside_the_context(tmp_path, tag, shared):
    """Two requests share their first 32 or 48 tokens.  The first one runs whole and ends; its full pages stay
    findable.  The second takes them over and runs only the rest, in one portion that starts at position 32 or
    48: head size 64 (D) takes the mma.sync prompt kernel, head size 128 (E, its window switched off so that
    prefix reuse applies) the tcgen05 one.  Every logit of the rest against the plain implementation."""
    from ullm_b200.csrc import kernels
    from ullm_b200.engine import ModelRunner, StepEntry

    cfg, w, page = weights_for(tag, "bfloat16")
    cfg = dict(cfg, use_sliding_window=False)
    d = write_model_dir(str(tmp_path / f"prefix_{tag}"), cfg, w)
    runner = ModelRunner(d, dtype="bfloat16", device=device(), page_size=page, num_pages=24, max_requests=2,
                         max_context=cfg["max_position_embeddings"], max_step_tokens=128, poison_cache=True,
                         enable_prefix_cache=True)
    V = cfg["vocab_size"]
    common = random_ids(V, shared, 5)
    a = common + random_ids(V, 40, 6)
    b = common + random_ids(V, 55, 7)
    runner.add_request("a", a)
    runner.step([StepEntry("a", a, [])])
    runner.end_request("a", a)
    rc = runner.add_request("b", b)
    assert rc.num_tokens == shared == rc.num_cached_tokens, "the shared full pages are taken over"
    rest = b[shared:]
    got = runner.step([StepEntry("b", rest, list(range(len(rest))))]).float().cpu()
    runner.check_device_status()
    assert kernels().attention_path == ("prefill_tcgen05" if tag == "E" and kernels().use_tcgen05_attention else "prefill")
    ref = plain_logits(b, w, cfg)[shared:]
    bad = first_bad_row(got, ref, "bfloat16")
    assert bad is None, f"first wrong position {shared + bad}"
    assert_close(got, ref, "bfloat16", f"{tag} prefix hit of {shared}")
    runner.end_request("b", b)
    runner.cache.check_invariants()


# ---------------------------------------------------------------------------------------------------------
# very unequal decode batches replayed from a CUDA graph, against the plain implementation
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.needs_cuda
@pytest.mark.parametrize("tag", ["D", "E"])
def test_ragged_decode_from_a_graph_tracks_the_plain_logits(tmp_path, tag):
    """One prompt of 300 tokens beside three short ones, 14 greedy tokens each with CUDA graphs on: the decode
    steps are replayed from the graph recorded for the attention mixer's "ragged" key, and every chosen token's
    plain logit is within the bfloat16 tolerance of the plain maximum (teacher-forced on the engine's tokens)."""
    from test_gpu_generate import make_llm
    from ullm_b200 import SamplingParams

    llm, cfg, w = make_llm(tmp_path, tag, dtype="bfloat16", max_bs=4, num_pages=64, max_num_batched_tokens=512)
    V = cfg["vocab_size"]
    prompts = [random_ids(V, n, 800 + n) for n in (300, 6, 11, 9)]
    outs = llm.generate_batch(prompts, SamplingParams(temperature=0.0, max_new_tokens=14, ignore_eos=True))
    dg = llm.engine.decode_graphs
    ragged_keys = [k for k in dg.graphs if any(k[1])]
    assert ragged_keys and dg.replays >= 8, (list(dg.graphs), dg.replays)
    for p, o in zip(prompts, outs):
        assert len(o.token_ids) == 14
        lg = pm.forward_logits(p + o.token_ids, w, cfg)
        scale = lg.abs().max().item()
        for i, tok in enumerate(o.token_ids):
            row = lg[len(p) - 1 + i]
            assert row.max().item() - row[tok].item() <= 2 * TOL["bfloat16"] * scale, f"prompt {len(p)}, token {i}"


# ---------------------------------------------------------------------------------------------------------
# temperature sampling in bfloat16: the chosen token lies in the plain implementation's filtered set
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("tag", ["B", "D"])
def test_bfloat16_temperature_sampling_stays_inside_the_plain_filtered_set(tmp_path, tag):
    """temperature 0.7, top_k 20, top_p 0.95: every sampled token, teacher-forced, has a plain logit no smaller
    than the smallest logit of the plain implementation's filtered set minus the bfloat16 tolerance (the two
    sides' logits differ by rounding, so the set's edge may move by that much and no more)."""
    from test_gpu_generate import make_llm
    from ullm_b200 import SamplingParams

    llm, cfg, w = make_llm(tmp_path, tag, dtype="bfloat16")
    V = cfg["vocab_size"]
    prompts = [random_ids(V, n, 90 + n) for n in (7, 16, 33)]
    sp = [SamplingParams(temperature=0.7, top_k=20, top_p=0.95, max_new_tokens=12, ignore_eos=True, seed=4 + i)
          for i in range(3)]
    outs = llm.generate_batch(prompts, sp)
    distinct = set()
    for p, o in zip(prompts, outs):
        assert len(o.token_ids) == 12
        lg = pm.forward_logits(p + o.token_ids, w, cfg)
        scale = lg.abs().max().item()
        for i, tok in enumerate(o.token_ids):
            row = lg[len(p) - 1 + i]
            probs = pm.filtered_distribution(row, 0.7, 20, 0.95, 0.0)
            edge = row[probs > 0].min().item()
            assert row[tok].item() >= edge - 2 * TOL["bfloat16"] * scale, f"prompt {len(p)}, token {i}: outside the set"
            distinct.add((i, tok == int(row.argmax())))
    assert any(not greedy for _, greedy in distinct), "with temperature 0.7 some token is not the most likely one"


# ---------------------------------------------------------------------------------------------------------
# the whole model at the widths and depth of Qwen3-0.6B in true 32-bit
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.needs_cuda
def test_float32_whole_model_at_qwen3_0_6b_shape(tmp_path):
    """All 28 layers at hidden 1024, 16 heads, 8 kv heads, head size 128, 3072 feed-forward, the 151,936-token
    vocabulary, tied head, in float32: a 16-token prompt and 4 tokens one by one against the plain implementation."""
    from ullm_b200.engine import ModelRunner

    cfg = {
        "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 28, "hidden_size": 1024, "num_attention_heads": 16,
        "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 3072, "vocab_size": 151936,
        "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "attention_bias": False, "tie_word_embeddings": True,
        "max_position_embeddings": 4096, "torch_dtype": "float32",
    }
    w = pm.random_weights(cfg, seed=23, std=0.02, norm_std=0.05)
    d = write_model_dir(str(tmp_path / "qwen3_0_6b_shape"), cfg, w)
    runner = ModelRunner(d, dtype="float32", device=device(), page_size=16, num_pages=4, max_requests=1,
                         max_context=64, max_step_tokens=32, poison_cache=True)
    ids = random_ids(cfg["vocab_size"], 20, 9)
    ref = plain_logits(ids, w, cfg)
    got = run_cut(runner, "a", ids, [16, 1, 1, 1, 1])
    assert_close(got, ref, "float32", "0.6B shape, 28 layers")
    assert torch.equal(got.argmax(-1), ref.argmax(-1))


# ---------------------------------------------------------------------------------------------------------
# two attention layers of different width decode through one recorded graph
# ---------------------------------------------------------------------------------------------------------
@pytest.fixture
def uneven_architecture():
    from dataclasses import replace

    from ullm_b200.config import ARCHITECTURES, Qwen3Config, qwen3_model_spec, register_architecture

    def spec(cfg):
        s = qwen3_model_spec(cfg)
        s.architecture = "UnevenForCausalLM"
        # the second layer has a third of the query heads and a narrower feed-forward
        l1 = s.layers[1]
        margs = dict(l1.mixer.args, num_heads=l1.mixer.args["num_kv_heads"])
        fargs = dict(l1.feed_forward.args, intermediate_size=l1.feed_forward.args["intermediate_size"] // 2)
        s.layers[1] = replace(l1, mixer=replace(l1.mixer, args=margs), feed_forward=replace(l1.feed_forward, args=fargs))
        return s

    register_architecture("UnevenForCausalLM", Qwen3Config.from_dict, spec)
    yield "UnevenForCausalLM"
    ARCHITECTURES.pop("UnevenForCausalLM")


@pytest.mark.needs_cuda
def test_layers_of_different_width_share_one_graph_without_recapture(tmp_path, uneven_architecture):
    """A model whose two layers differ in head count and feed-forward width (registered here, random weights):
    its step buffers are known by (name, width), so the layers do not reallocate each other's buffers, the
    workspace's generation stands still while decoding, the decode graph recorded first is the one replayed,
    and the tokens equal those of the eager engine."""
    from ullm_b200 import LLM, EngineConfig, SamplingParams
    from tiny_configs import ALL

    cfg = dict(ALL["D"][0], architectures=[uneven_architecture], torch_dtype="bfloat16")
    d = str(tmp_path / "uneven")
    os.makedirs(d)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    common = dict(model=d, max_bs=2, context_len=256, page_size=16, num_pages=32, max_num_batched_tokens=64,
                  dtype="bfloat16", load_format="random", seed=3, random_init_std=0.05)
    prompts = [random_ids(cfg["vocab_size"], n, 40 + n) for n in (9, 21)]
    sp = SamplingParams(temperature=0.0, max_new_tokens=10, ignore_eos=True)
    llm = LLM(EngineConfig(**common))
    m0, m1 = (b.mixer for b in llm.engine.runner.model.blocks)
    assert m0.num_heads != m1.num_heads
    outs = llm.generate_batch(prompts[:1], sp)  # records the graph of one request
    ws, dg = llm.engine.runner.workspace, llm.engine.decode_graphs
    gen, held, replays = ws.generation, dict(dg.graphs), dg.replays
    assert held and replays > 0
    outs = llm.generate_batch(prompts[:1], sp)
    assert ws.generation == gen and all(dg.graphs[k][0] is v[0] for k, v in held.items()) and dg.replays > replays
    assert {k[:2] for k in ws.buffers if k[0] == "attn.qkv"} == {
        ("attn.qkv", (m.num_heads + 2 * m.num_kv_heads) * m.head_dim) for m in (m0, m1)}
    both = llm.generate_batch(prompts, sp)
    eager = LLM(EngineConfig(**common, enforce_eager=True)).generate_batch(prompts, sp)
    assert [o.token_ids for o in both] == [o.token_ids for o in eager]
    assert outs[0].token_ids == eager[0].token_ids


# ---------------------------------------------------------------------------------------------------------
# steps launched ahead while the GPU lags behind the host
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.needs_cuda
@pytest.mark.parametrize("eager", [True, False])
def test_steps_launched_ahead_with_a_busy_stream_and_a_shrinking_batch(tmp_path, eager):
    """Four sampled requests of different lengths, so that the batch shrinks while steps are launched ahead,
    and after every step the stream is kept busy for about a millisecond, so that the host stages the next
    step's parameters while the copies of the one before have not run yet.  The tokens must equal those of the
    engine that reads every step before the next."""
    from test_gpu_generate import make_llm
    from ullm_b200 import SamplingParams

    prompts = [random_ids(331, n, 300 + n) for n in (5, 9, 14, 3)]
    sp = [SamplingParams(temperature=0.9, top_k=40, max_new_tokens=n, ignore_eos=True, seed=70 + i)
          for i, n in enumerate((4, 9, 6, 12))]
    ref_llm, cfg, w = make_llm(tmp_path, "B", enforce_eager=eager, disable_async_scheduling=True)
    ref = ref_llm.generate_batch(prompts, sp)
    llm, _, _ = make_llm(tmp_path, "B", enforce_eager=eager)
    assert llm.engine.async_decode
    outs = llm.generate_batch(prompts, sp, on_step=lambda eng: torch.cuda._sleep(2_000_000))
    assert [o.token_ids for o in outs] == [o.token_ids for o in ref]
    llm.engine.runner.cache.check_invariants()


# ---------------------------------------------------------------------------------------------------------
# the profiler's report
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.needs_cuda
def test_profile_reports_steps_and_kernel_groups(tmp_path, capsys):
    from test_gpu_generate import make_llm
    from ullm_b200 import SamplingParams

    pdir = str(tmp_path / "prof")
    llm, cfg, w = make_llm(tmp_path, "D", dtype="bfloat16", profile=True, profile_dir=pdir)
    prompts = [random_ids(cfg["vocab_size"], n, 60 + n) for n in (70, 12)]
    llm.generate_batch(prompts, SamplingParams(temperature=0.0, max_new_tokens=9, ignore_eos=True))
    report = llm.engine.profile("stop")
    kinds = {r["kind"] for r in report["by_kind"]}
    assert {"prefill", "decode"} <= kinds
    assert all(r["mean_device_ms"] and r["mean_device_ms"] > 0 for r in report["by_kind"])
    assert sum(r["tokens"] for r in report["by_kind"]) == 70 + 12 + 2 * 8
    groups = report["kernel_groups"]
    assert {"attention", "linear", "add_rmsnorm", "linear_head", "sampling"} <= set(groups)
    assert groups["linear"]["bytes"] > 0 and groups["linear"]["gb_per_s"] > 0
    with open(report["path"]) as f:
        assert json.load(f)["by_kind"] == report["by_kind"]
    assert "profile: steps by kind" in capsys.readouterr().out
    assert llm.engine.profile("stop") is None  # already stopped


# ---------------------------------------------------------------------------------------------------------
# the bounded waits of the tcgen05 / TMA kernels
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.needs_cuda
def test_a_wait_that_runs_out_is_reported_and_the_next_kernel_runs():
    """The give-up path that every tcgen05 / TMA kernel has, run on purpose by the library's self-test kernel: a
    barrier nobody arrives at, a few thousand polls, then the timeout lands in the status word, the tensor
    memory goes back, the kernel returns; the host raises, and the next ordinary kernels (tensor memory
    included) run and are right."""
    from ullm_b200.csrc import kernels
    from ullm_b200.csrc.ops import KernelError

    K = kernels()
    K.raise_on_status()
    assert K.wait_selftest(3000) == 1
    assert K.status.tolist()[:3] == [6, 90, 3000]
    with pytest.raises(KernelError, match="gave up waiting"):
        K.raise_on_status()
    assert K.status.tolist()[0] == 0
    x = torch.randn(5, 96, device="cuda")
    wt = torch.rand(96, device="cuda") + 0.5
    out = torch.empty_like(x)
    K.add_rmsnorm(x, None, wt, 1e-6, out)
    ref = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * wt
    assert torch.allclose(out, ref, atol=1e-5)
    # a kernel that allocates all 512 columns of tensor memory still gets them
    a = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(512, 512, device="cuda", dtype=torch.bfloat16)
    c = torch.empty(256, 512, device="cuda", dtype=torch.bfloat16)
    if K.large_linear(a, b, c):
        torch.cuda.synchronize()
        assert torch.allclose(c.float(), a.float() @ b.float().t(), atol=0.5, rtol=2e-2)
    K.raise_on_status()


# ---------------------------------------------------------------------------------------------------------
# norms folded between products: fewer kernels, the same logits
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.needs_cuda
def test_norms_folded_between_products_save_kernels_and_keep_the_logits(tmp_path, monkeypatch):
    """A three-layer bfloat16 model (head size 128) decoding three requests one token at a time, with the norms
    as kernels of their own (0), the feed-forward norm folded between o_proj and gate_up (1), and the next
    block's first norm folded behind down_proj as well (2): each level launches fewer kernels per step, and every
    level's logits are within the bfloat16 tolerance of the plain implementation."""
    import os

    from ullm_b200.csrc import kernels
    from ullm_b200.engine import ModelRunner, StepEntry

    cfg = {"architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 3, "hidden_size": 256,
           "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 640,
           "vocab_size": 523, "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "attention_bias": False,
           "tie_word_embeddings": True, "max_position_embeddings": 256, "torch_dtype": "bfloat16"}
    w = {n: t.to(torch.bfloat16) for n, t in pm.random_weights(cfg, seed=23, std=0.05, norm_std=0.2).items()}
    d = write_model_dir(str(tmp_path / "fold_model"), cfg, w)
    wf = {k: v.float() for k, v in w.items()}
    prompts = [random_ids(cfg["vocab_size"], n, 70 + n) for n in (33, 9, 20)]
    tails = [random_ids(cfg["vocab_size"], 6, 90 + i) for i in range(3)]
    want = [pm.forward_logits(p + t, wf, cfg) for p, t in zip(prompts, tails)]
    K = kernels()
    launches = {}
    try:
        for level in ("0", "1", "2"):
            monkeypatch.setenv("ULLM_B200_CHAIN_NORMS", level)
            K.apply_switches(os.environ)
            r = ModelRunner(d, dtype="bfloat16", device=device(), page_size=16, num_pages=32, max_requests=4,
                            max_context=256, max_step_tokens=64)
            for i, p in enumerate(prompts):
                r.add_request(f"q{i}")
                r.step([StepEntry(f"q{i}", p, [])])
            got = [[] for _ in prompts]
            l0 = K.launches
            for t in range(6):
                lg = r.step([StepEntry(f"q{i}", [tails[i][t]], [0]) for i in range(3)]).float().cpu()
                for i in range(3):
                    got[i].append(lg[i])
            launches[level] = (K.launches - l0) / 6
            r.check_device_status()
            for i in range(3):
                ref = want[i][len(prompts[i]):len(prompts[i]) + 6]
                assert_close(torch.stack(got[i]), ref, "bfloat16", f"fold level {level}, request {i}")
    finally:
        monkeypatch.undo()
        K.apply_switches(os.environ)
    # level 1 saves at least the feed-forward norm of every layer, level 2 also the first norm of every layer but
    # the first
    assert launches["0"] - launches["1"] >= cfg["num_hidden_layers"], launches
    assert launches["1"] - launches["2"] == cfg["num_hidden_layers"] - 1, launches


# ---------------------------------------------------------------------------------------------------------
# every environment switch: generation with it set still follows the plain implementation
# ---------------------------------------------------------------------------------------------------------
SWITCH_SETTINGS = [
    {"ULLM_B200_PDL": "1"}, {"ULLM_B200_SMALL_M_LINEAR": "0"}, {"ULLM_B200_SMALL_M_LINEAR": "stream"},
    {"ULLM_B200_SMALL_M_LINEAR": "skinny"}, {"ULLM_B200_SMALL_M_LINEAR": "tcgen05"},
    {"ULLM_B200_SMALL_M_LINEAR": "stream", "ULLM_B200_PDL": "1"}, {"ULLM_B200_STREAM_WEIGHT_MB": "0"},
    {"ULLM_B200_DECODE_TC": "1"}, {"ULLM_B200_DECODE_CLUSTER": "1"}, {"ULLM_B200_DECODE_CLUSTER": "0"},
    {"ULLM_B200_FUSE_DECODE_ROPE": "0"}, {"ULLM_B200_TC_ATTN": "0"}, {"ULLM_B200_TC_ATTN": "single"}, {"ULLM_B200_DECODE_BALANCED": "1"},
    {"ULLM_B200_DECODE_BALANCED": "0"}, {"ULLM_B200_MIXED_DECODE_ROWS": "0"}, {"ULLM_B200_LT_ROWS": "0"},
    {"ULLM_B200_FUSED_MLP_ROWS": "1"}, {"ULLM_B200_FUSED_TAIL_ROWS": "16"}, {"ULLM_B200_CHAIN_NORMS": "0"}, {"ULLM_B200_CHAIN_NORMS": "1"},
    {"ULLM_B200_STREAM_ALL_ROWS": "0"}, {"ULLM_B200_STREAM_ALL_ROWS": "32"}, {"ULLM_B200_GRAPH_SKIP": "2,8"},
    {"ULLM_B200_PDL": "0"}, {"ULLM_B200_SMALL_M_LINEAR": "0", "ULLM_B200_PDL": "1"}, {"ULLM_B200_DECODE_SPLIT_TARGET": "37"}, {"ULLM_B200_MIN_GRAPH_BATCH": "4"},
]


@pytest.mark.needs_cuda
@pytest.mark.parametrize("switches", SWITCH_SETTINGS, ids=lambda d: ",".join(f"{k[10:]}={v}" for k, v in d.items()))
def test_generation_under_each_switch_follows_the_plain_logits(tmp_path, monkeypatch, switches):
    """Every optional switch, set as the environment would set it: three requests (one much longer, so that even,
    ragged and mixed steps occur; prompts in portions of 64) on a two-layer bfloat16 model with head size 128,
    CUDA graphs on; every chosen token's plain logit is within the bfloat16 tolerance of the plain maximum."""
    import os

    from ullm_b200 import LLM, EngineConfig, SamplingParams
    from ullm_b200.csrc import kernels

    cfg = {"architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 256,
           "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 384,
           "vocab_size": 1031, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "attention_bias": False,
           "tie_word_embeddings": False, "max_position_embeddings": 512, "torch_dtype": "bfloat16"}
    w = {n: t.to(torch.bfloat16) for n, t in pm.random_weights(cfg, seed=19, std=0.04, norm_std=0.1).items()}
    d = write_model_dir(str(tmp_path / "switch_model"), cfg, w)
    for k, v in switches.items():
        monkeypatch.setenv(k, v)
    K = kernels()
    try:
        K.apply_switches(os.environ)
        llm = LLM(EngineConfig(model=d, max_bs=4, context_len=512, page_size=16, num_pages=64,
                               max_num_batched_tokens=64, dtype="bfloat16", log_level="warning"))
        prompts = [random_ids(cfg["vocab_size"], n, 50 + n) for n in (200, 40, 9, 70)]
        n_new = [6, 12, 12, 9]
        outs = llm.generate_batch(prompts, [SamplingParams(temperature=0.0, max_new_tokens=n, ignore_eos=True)
                                            for n in n_new])
        K.raise_on_status()
    finally:
        monkeypatch.undo()
        K.apply_switches(os.environ)
    wf = {k: v.float() for k, v in w.items()}
    for p, o, n in zip(prompts, outs, n_new):
        assert len(o.token_ids) == n
        lg = pm.forward_logits(p + o.token_ids, wf, cfg)
        scale = lg.abs().max().item()
        for i, tok in enumerate(o.token_ids):
            row = lg[len(p) - 1 + i]
            assert row.max().item() - row[tok].item() <= 2 * TOL["bfloat16"] * scale, f"prompt {len(p)}, token {i}"
