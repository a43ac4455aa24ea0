#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decode tokens per second (batch 8 by
default, also batch 1 and 64), prefill tokens per second at 2,048 tokens, and
the fraction of the roofline each reaches.  Qwen3-8B layer sizes, random
bfloat16 weights, synthetic token ids.

    python bench.py --gpus 1 --steps K --warmup W

prints ONE JSON line.  `value` times K decode steps with CUDA events around the
engine's own decode path (staging copy, graph replay, token read-back); `e2e`
times the same K steps through the public entry point (`Engine.step` under
`LLM`), host token ids in and out.  For more than one GPU it says so and
exits 2: this engine runs on one GPU.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# The benchmark configuration: Qwen3-8B layer sizes
QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"],
    "num_hidden_layers": 36,
    "hidden_size": 4096,
    "num_attention_heads": 32,
    "num_key_value_heads": 8,
    "head_dim": 128,
    "intermediate_size": 12288,
    "vocab_size": 151936,
    "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6,
    "attention_bias": False,
    "tie_word_embeddings": False,
    "use_sliding_window": False,
    "max_position_embeddings": 40960,
    "torch_dtype": "bfloat16",
}
# Qwen3-32B layer sizes (65.5 GB of bfloat16 weights): the memory-planning case
QWEN3_32B = dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, intermediate_size=25600)
# Qwen3-0.6B layer sizes, the model of the reference's own published benchmark (tied head)
QWEN3_0_6B = dict(QWEN3_8B, num_hidden_layers=28, hidden_size=1024, num_attention_heads=16, intermediate_size=3072,
                  tie_word_embeddings=True)
SHAPES = {"8b": ("Qwen3-8B shape", QWEN3_8B), "32b": ("Qwen3-32B shape", QWEN3_32B),
          "0.6b": ("Qwen3-0.6B shape", QWEN3_0_6B)}
CONTEXT_LEN = 4096
START_CONTEXT = 2048
PREFILL_TOKENS = 2048
PAGE_SIZE = 16
# the serving workload: 256 requests, prompt and output lengths uniform in 100..1024, seed 5, eos ignored
SERVE_REQUESTS, SERVE_MIN, SERVE_MAX, SERVE_SEED = 256, 100, 1024, 5


def metric_name(batch: int, label: str) -> str:
    """Both arms print this string, so that their values can be set side by side."""
    return f"decode tok/s at batch {batch}, {label}"


def common_config(label: str, cfg: dict, layers: int, batch: int) -> dict:
    """The keys both arms' `config` has (each arm adds `timing`, `cuda_graph`, `l2`, `peaks`, `kv_dtype`)."""
    return {
        "model": label, "global_batch": batch, "seq_len": CONTEXT_LEN, "parallelism": "single-gpu",
        "layers": layers, "layers_of_config": cfg["num_hidden_layers"], "hidden_size": cfg["hidden_size"],
        "num_attention_heads": cfg["num_attention_heads"], "num_key_value_heads": cfg["num_key_value_heads"],
        "head_dim": cfg["head_dim"], "intermediate_size": cfg["intermediate_size"],
        "vocab_size": cfg["vocab_size"], "start_context": START_CONTEXT, "page_size": PAGE_SIZE,
    }


def serve_workload(vocab: int):
    """(prompts, output lengths) of the serving workload, from its seed."""
    import random

    rng = random.Random(SERVE_SEED)
    prompts = [[rng.randrange(vocab) for _ in range(rng.randint(SERVE_MIN, SERVE_MAX))] for _ in range(SERVE_REQUESTS)]
    outs = [rng.randint(SERVE_MIN, SERVE_MAX) for _ in range(SERVE_REQUESTS)]
    return prompts, outs


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int = 0):
        self.rows: list[list[str]] = []
        self.proc = None
        self.device_index = device_index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.device_index), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        mhz = [int(r[0]) for r in self.rows if r and r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i].lower() == "active" for r in self.rows)]
        return {"sm_mhz": int(statistics.median(mhz)) if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(mhz)}


def model_numbers(cfg: dict, layers: int) -> dict:
    H, Hq, Hkv, D, I, V = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"],
                           cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"])
    per_layer = (Hq + 2 * Hkv) * D * H + H * Hq * D + 2 * I * H + H * I
    return {
        "layer_weight_elems": per_layer,
        "head_elems": V * H,
        "kv_bytes_per_token": layers * 2 * Hkv * D * 2,
        "weight_bytes_decode": (layers * per_layer + V * H) * 2,  # every matrix once; embedding rows are negligible
    }


def decode_bytes(nums: dict, batch: int, mean_ctx: float, hidden: int) -> float:
    return nums["weight_bytes_decode"] + batch * mean_ctx * nums["kv_bytes_per_token"] + batch * hidden * 2


def prefill_flops(cfg: dict, layers: int, T: int) -> float:
    n = model_numbers(cfg, layers)
    gemm = 2.0 * T * layers * n["layer_weight_elems"] + 2.0 * n["head_elems"]  # logits for the last token only
    attn = layers * 4.0 * cfg["num_attention_heads"] * cfg["head_dim"] * (T * (T + 1) / 2)
    return gemm + attn


def _make_llm(cfg: dict, layers: int, max_bs: int, num_pages, budget: int = 4096, context: int = CONTEXT_LEN,
              utilization: float = 0.9):
    from ullm_b200.config import EngineConfig
    from ullm_b200.engine.llm import LLM

    cfg = dict(cfg, num_hidden_layers=layers)
    tmp = tempfile.mkdtemp(prefix="ullm_b200_bench_")
    with open(os.path.join(tmp, "config.json"), "w") as f:
        json.dump(cfg, f)
    ec = EngineConfig(
        model=tmp, max_bs=max_bs, context_len=context, page_size=PAGE_SIZE, num_pages=num_pages,
        gpu_memory_utilization=utilization, max_num_batched_tokens=budget, dtype="bfloat16", load_format="random",
        seed=0, enable_prefix_caching=False, log_level="warning",
    )
    return LLM(ec), ec


def run_ours(args) -> dict:
    """Decode and prefill at the layer sizes of `--workload` (8b, the default line, or 32b)."""
    import torch

    from ullm_b200.csrc import kernels
    from ullm_b200.sampling import SamplingParams

    label, shape = SHAPES[args.workload]
    cfg = dict(shape)
    full_layers = cfg["num_hidden_layers"]
    layers = args.layers or full_layers
    cfg["num_hidden_layers"] = layers
    pk = peaks()
    nums = model_numbers(cfg, layers)
    K, W = args.steps, args.warmup
    KP = max(K, 64)  # steps of the points at batch 1 and 64
    max_bs = 64
    if args.workload == "8b":
        tokens_per_req = START_CONTEXT + 2 * (KP + W) + 64
        num_pages = max_bs * (-(-tokens_per_req // PAGE_SIZE)) + 64
    else:
        num_pages = None  # planned from the memory that is free once the weights are resident
    llm, ec = _make_llm(shape, layers, max_bs, num_pages)
    eng = llm.engine
    runner = eng.runner
    kern = kernels()
    g = torch.Generator().manual_seed(1)

    def prompt(n):
        return torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist()

    sp = SamplingParams(temperature=0.0, ignore_eos=True, max_new_tokens=10**9)

    def start_batch(B, tag):
        ids = [f"{tag}{i}" for i in range(B)]
        for sid in ids:
            eng.add_sequence(sid, prompt(START_CONTEXT), sp)
        while any(s.num_pending > 1 or s.status.name == "WAITING" for s in
                  [eng.scheduler.get_sequence(i) for i in ids]):
            eng.step()
        return ids

    def stop_batch(ids):
        for sid in ids:
            eng.abort_sequence(sid)
        while eng.has_unfinished_sequences():
            eng.step()

    def even_graph(B):
        dg = eng.decode_graphs
        if dg is None or not dg.takes(B):
            return None
        held = [v for k, v in dg.graphs.items() if k[0] == dg.padded(B) and not any(k[1])]
        return held[0][0] if held else None

    def replay_ms(graph, steps):
        """The device side alone: the captured step replayed back to back (it rewrites the same cache slots)."""
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    def time_decode(B, tag, steps, warmup, ablate=False):
        """Device-timed decode through Engine.step: (ms per step, wall seconds per step, launches per step,
        mean context, device-only ms, group times)."""
        ids = start_batch(B, tag)
        for _ in range(warmup):
            eng.step()
        torch.cuda.synchronize()
        l0 = kern.launches
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        for _ in range(steps):
            eng.step()
        e1.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        ms = e0.elapsed_time(e1) / steps
        launches = (kern.launches - l0) / steps
        ctx = START_CONTEXT + warmup + steps / 2.0
        graph = even_graph(B)
        graph_ms = replay_ms(graph, steps) if graph is not None else None
        groups = None
        if ablate and graph is not None:
            # What each group of kernels costs inside the step: the step recorded again without it (its results
            # are then meaningless), replayed back to back, and the difference to the whole step.
            groups = {}
            sets = {"products": ("linear", "linear_gate_up_act"), "attention": ("attention",),
                    "small": ("add_rmsnorm", "act_mul", "embedding", "gather_rows", "qk_norm_rope_store"),
                    "head": ("linear_head",), "sampling": ("sampling",)}
            dg = eng.decode_graphs
            try:
                for name, skip in sets.items():
                    kern.skip_groups = frozenset(skip)
                    dg.graphs.clear()
                    eng.step()  # runs eagerly and records
                    eng.step()
                    gr = even_graph(B)
                    if gr is not None:
                        groups[name] = max(graph_ms - replay_ms(gr, steps), 0.0)
            finally:
                kern.skip_groups = frozenset()
                dg.graphs.clear()
        stop_batch(ids)
        return ms, wall / steps, launches, ctx, graph_ms, groups

    # ---- prefill of 2,048 tokens ---------------------------------------------------
    pre_ms = []
    for i in range(max(3, min(W, 5)) + 5):
        sid = f"p{i}"
        eng.add_sequence(sid, prompt(PREFILL_TOKENS), SamplingParams(temperature=0.0, ignore_eos=True, max_new_tokens=1))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        eng.step()
        e1.record()
        torch.cuda.synchronize()
        pre_ms.append(e0.elapsed_time(e1))
    pre = statistics.median(pre_ms[3:])
    pflops = prefill_flops(cfg, layers, PREFILL_TOKENS)
    prefill = {"value": round(PREFILL_TOKENS / (pre / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(pre, 3),
               "frac": round(pflops / (pre / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
               "frac_of_sustained": round(pflops / (pre / 1e3) / (pk["bf16_tflops_sustained"] * 1e12), 4)}

    # ---- decode ----------------------------------------------------------------------
    B = args.batch
    with ClockSampler() as clk:
        ms, wall, launches, ctx, graph_ms, groups = time_decode(B, "d", K, W, ablate=not args.no_groups)
    clocks = clk.summary()
    value = B / (ms / 1e3)
    # End to end through the call a user makes: LLM.generate_batch, token ids in, token ids out.  Pairs of calls
    # on fresh prompts of the same lengths, WE and WE + K new tokens each: their prompt work is the same, the
    # difference of their wall times is K decode steps (each with its staging copy from pinned memory and the
    # read of its sampled ids) as the user sees them.  The median of five such differences.  (WE = at least 24
    # tokens: the first steps behind a burst of prompts run at the clocks the power cap left, as `value`'s own
    # warm-up steps do; the difference then covers steps like those `value` times.)
    def user_call(n_new):
        ps = [prompt(START_CONTEXT) for _ in range(B)]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = llm.generate_batch(ps, SamplingParams(temperature=0.0, ignore_eos=True, max_new_tokens=n_new))
        dt = time.perf_counter() - t0
        assert all(len(o.token_ids) == n_new for o in outs)
        return dt
    WE = max(W, 24)
    user_call(WE)  # warm
    KE = max(K, 64)  # (differences of fewer steps are a few percent of noise)
    diffs = []
    for _ in range(5):
        t_short = user_call(WE)
        diffs.append(user_call(WE + KE) - t_short)
    e2e_value = B * KE / max(statistics.median(diffs), 1e-9)
    e2e_steps_value = B / wall  # the same loop as `value`, by the wall clock
    dbytes = decode_bytes(nums, B, ctx, cfg["hidden_size"])
    achieved = dbytes / (ms / 1e3) / 1e9
    points = {f"decode_b{B}": round(value, 1)}
    for pb in (1, 8, 32, 64):
        if pb == B:
            pms, pctx, pgraph = ms, ctx, graph_ms
        else:
            pms, _pw, _pl, pctx, pgraph, _g = time_decode(pb, f"b{pb}_", KP, max(3, W))
        points[f"decode_b{pb}"] = round(pb / (pms / 1e3), 1)
        points[f"decode_b{pb}_ms"] = round(pms, 4)
        points[f"decode_b{pb}_frac"] = round(decode_bytes(nums, pb, pctx, cfg["hidden_size"]) / (pms / 1e3) / 1e9
                                             / pk["hbm_gbs"], 4)
        if pgraph:
            points[f"decode_b{pb}_device_only_ms"] = round(pgraph, 4)
    out_groups = None
    if groups:
        # milliseconds of the step that go to each group, and for the three that stream memory the fraction of
        # the copy bandwidth they reach on the bytes they have to read
        gbytes = {"products": layers * nums["layer_weight_elems"] * 2,
                  "attention": B * ctx * nums["kv_bytes_per_token"], "head": nums["head_elems"] * 2}
        out_groups = {"method": "difference to the step recorded without the group, device only"}
        for name, gms in groups.items():
            out_groups[f"{name}_ms"] = round(gms, 4)
            if name in gbytes and gms > 0:
                frac = gbytes[name] / (gms / 1e3) / 1e9 / pk["hbm_gbs"]
                if frac <= 1.05:  # (a difference smaller than the group can take alone says that the rest of the
                    out_groups[f"{name}_frac"] = round(frac, 4)  # step slowed down without it: no fraction then)
    st = runner.decode_staging
    h2d = st.layout(st.max_tokens, st.max_requests)["_end"][0] * 4 + eng.sampler.host.numel() * 4
    config = common_config(label, shape, layers, B)
    config.update({"kv_dtype": "bf16", "l2": "inputs>L2 (each step streams all weights)", "peaks": pk["source"],
                   "cuda_graph": not ec.enforce_eager, "timing": "CUDA events around Engine.step",
                   "num_pages": runner.cache.num_pages})
    out = {
        "metric": metric_name(B, label),
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights, uniform random token ids)",
        "config": config,
        "clocks": clocks,
        "e2e": {"value": round(e2e_value, 1), "unit": "tok/s", "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(B * 4), "api": "LLM.generate_batch", "steps": KE, "pairs": len(diffs),
                "engine_step_wall_value": round(e2e_steps_value, 1)},
        "gpu_launches": int(round(launches * K)),
        "device_only_ms_per_step": round(graph_ms, 4) if graph_ms else None,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
    }
    if out_groups:
        out["groups"] = out_groups
    return out


def run_serve(args) -> dict:
    """`--workload serve-0.6b`: the reference's own published workload (its bench.py: 256 requests, random prompt
    and output lengths, continuous batching) at Qwen3-0.6B layer sizes, through `LLM.generate_batch`: host token
    ids in, host token ids out, wall clock from the call to its return.  Each request generates exactly its
    output length (`max_new_tokens`; the reference's script passes `max_tokens`, which bounds the total length
    in its current tree)."""
    import torch

    from ullm_b200.csrc import kernels
    from ullm_b200.sampling import SamplingParams

    label, shape = SHAPES["0.6b"]
    layers = args.layers or shape["num_hidden_layers"]
    llm, ec = _make_llm(shape, layers, SERVE_REQUESTS, None, budget=8192, utilization=0.8)
    prompts, outs = serve_workload(shape["vocab_size"])
    sps = [SamplingParams(temperature=0.6, ignore_eos=True, max_new_tokens=n, seed=i) for i, n in enumerate(outs)]
    # warm-up: a short run over every batch size on the way down records the decode graphs and times the
    # library's products
    llm.generate_batch(prompts[:SERVE_REQUESTS], [SamplingParams(temperature=0.6, ignore_eos=True,
                                                                   max_new_tokens=4 + i % 3, seed=i)
                                                    for i in range(SERVE_REQUESTS)])
    kern = kernels()
    torch.cuda.synchronize()
    l0 = kern.launches
    with ClockSampler() as clk:
        t0 = time.perf_counter()
        res = llm.generate_batch(prompts, sps)
        dt = time.perf_counter() - t0
    assert [len(o.token_ids) for o in res] == outs
    gen, pro = sum(outs), sum(len(p) for p in prompts)
    st = llm.engine.stats()
    config = common_config(label, shape, layers, SERVE_REQUESTS)
    config.update({"requests": SERVE_REQUESTS, "prompt_tokens": pro, "generated_tokens": gen,
                   "lengths": f"uniform {SERVE_MIN}..{SERVE_MAX}, seed {SERVE_SEED}", "temperature": 0.6,
                   "timing": "wall clock around LLM.generate_batch"})
    config.pop("start_context")
    return {
        "metric": f"generated tok/s, {SERVE_REQUESTS} requests under continuous batching, {label}",
        "value": round(gen / dt, 1), "unit": "tok/s", "n_gpus": 1, "steps": int(st.get("steps_run", 0)), "warmup": 1,
        "ms_per_step": None, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (random weights, uniform random token ids)", "config": config,
        "clocks": clk.summary(), "seconds": round(dt, 3), "total_tok_s": round((gen + pro) / dt, 1),
        "e2e": {"value": round(gen / dt, 1), "unit": "tok/s", "api": "LLM.generate_batch"},
        "gpu_launches": int(kern.launches - l0), "preemptions": st.get("preemptions"),
    }


def run_long_context(args) -> dict:
    """`--workload 8b-long`: the same layer sizes at a context of 16,384 tokens: the prefill of one 16,384-token
    prompt (in portions of the engine's token budget, each behind the pages of the portions before it), and decode
    steps of 8 requests that each hold 16,384 tokens.  One line for `points`."""
    import torch

    from ullm_b200.csrc import kernels
    from ullm_b200.sampling import SamplingParams

    LONG, B, steps, warm = 16384, 8, 32, 4
    cfg = dict(QWEN3_8B)
    layers = args.layers or cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = layers
    pk = peaks()
    nums = model_numbers(cfg, layers)
    per_req = LONG + 2 * (steps + warm) + 64
    llm, _ = _make_llm(QWEN3_8B, layers, B, (B + 1) * (-(-per_req // PAGE_SIZE)) + 64, budget=4096, context=LONG + 1024)
    eng = llm.engine
    g = torch.Generator().manual_seed(2)

    def prompt(n):
        return torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist()

    def drain():
        while eng.has_unfinished_sequences():
            eng.step()

    pre_ms = []
    for i in range(4):
        eng.add_sequence(f"p{i}", prompt(LONG), SamplingParams(temperature=0.0, ignore_eos=True, max_new_tokens=1))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        drain()
        e1.record()
        torch.cuda.synchronize()
        pre_ms.append(e0.elapsed_time(e1))
    pre = statistics.median(pre_ms[1:])
    sp = SamplingParams(temperature=0.0, ignore_eos=True, max_new_tokens=10**9)
    ids = [f"d{i}" for i in range(B)]
    for sid in ids:
        eng.add_sequence(sid, prompt(LONG), sp)
    while any(s.num_pending > 1 or s.status.name == "WAITING" for s in [eng.scheduler.get_sequence(i) for i in ids]):
        eng.step()
    for _ in range(warm):
        eng.step()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        eng.step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    for sid in ids:
        eng.abort_sequence(sid)
    drain()
    kernels().raise_on_status()
    ctx = LONG + warm + steps / 2.0
    return {"workload": "8b-long", "context": LONG, "layers": layers,
            "prefill_tok_s": round(LONG / (pre / 1e3), 1), "prefill_ms": round(pre, 2),
            "prefill_frac": round(prefill_flops(cfg, layers, LONG) / (pre / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
            "decode_b8_ms": round(ms, 4), "decode_b8_tok_s": round(B / (ms / 1e3), 1),
            "decode_b8_frac": round(decode_bytes(nums, B, ctx, cfg["hidden_size"]) / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 4)}


def run_extra_shapes(args, impl: str) -> dict:
    """The two further workloads, each in a process of its own (the 32B shape needs the device to itself), as
    flat entries for `points`."""
    points = {}
    jobs = [("serve-0.6b", "qwen3_0_6b_serve")] + ([("32b", "qwen3_32b"), ("8b-long", "qwen3_8b_ctx16k")] if impl == "ours" else [])
    for workload, key in jobs:
        cmd = [sys.executable, os.path.abspath(__file__), "--workload", workload, "--impl", impl, "--steps",
               str(args.steps), "--warmup", str(args.warmup), "--no-groups"]
        try:
            r = subprocess.run(cmd, capture_output=True, text=True, timeout=1500)
            line = [l for l in r.stdout.splitlines() if l.startswith("{")][-1]
            d = json.loads(line)
        except Exception as e:  # noqa: BLE001 - a failed side run must not lose the main line
            points[f"{key}_error"] = f"{type(e).__name__}: {e}"[:200]
            continue
        if "unavailable" in d:
            points[f"{key}_unavailable"] = d["unavailable"][:200]
        elif workload == "8b-long":
            for k in ("prefill_tok_s", "prefill_frac", "decode_b8_ms", "decode_b8_tok_s", "decode_b8_frac"):
                points[f"{key}_{k}"] = d[k]
        elif workload == "32b":
            for k, v in d["points"].items():
                points[f"{key}_{k}"] = v
            points[f"{key}_prefill_tok_s"] = d["prefill"]["value"]
            points[f"{key}_prefill_frac"] = d["prefill"]["frac"]
        else:
            points[f"{key}_generated_tok_s"] = d["value"]
            points[f"{key}_total_tok_s"] = d.get("total_tok_s")
            points[f"{key}_seconds"] = d.get("seconds")
    return points


def run_probe(args) -> int:
    """A few eager steps at the benchmark's layer sizes, for profilers: `--probe decode` runs `--steps` decode
    steps of `--batch` requests that each hold `--context` tokens (the held context is reserved, not computed: a
    profile needs its size, not its content); `--probe prefill` runs `--steps` prompts of 2,048 tokens."""
    import torch

    from ullm_b200.engine import ModelRunner, StepEntry

    cfg = dict(QWEN3_8B)
    cfg["num_hidden_layers"] = args.layers or 2
    B, ctx = args.batch, args.context
    r = ModelRunner(config=cfg, dtype="bfloat16", page_size=PAGE_SIZE, num_pages=B * (ctx // PAGE_SIZE + 8) + 160,
                    max_requests=B + 1, max_context=CONTEXT_LEN, max_step_tokens=max(B, PREFILL_TOKENS),
                    load_format="random")
    ids = []
    for i in range(B):
        rc = r.add_request(f"r{i}")
        r.cache.reserve(rc, ctx)
        r.cache.commit(rc, ctx)
        ids.append(f"r{i}")
    if args.probe == "prefill":
        for s in range(args.steps):
            r.add_request(f"p{s}")
            r.step([StepEntry(f"p{s}", [1 + s] * PREFILL_TOKENS, [PREFILL_TOKENS - 1])])
            r.end_request(f"p{s}")
    else:
        for s in range(args.steps):
            r.step([StepEntry(i, [5 + s], [0]) for i in ids])
    torch.cuda.synchronize()
    r.check_device_status()
    print(f"probe {args.probe}: {args.steps} steps, {cfg['num_hidden_layers']} layers, batch {B}, context {ctx}")
    return 0


def run_linear_probe(args) -> int:
    """`--probe linear`: the decode step's five matrix products (Qwen3-8B sizes) alone, for `--batch` rows: the
    vendor library against this repo's two few-row kernels, each timed as 40 launches over rotating weight copies
    (more than L2 holds) inside one CUDA graph, so that no launch cost of the host is in the figure."""
    import torch

    from ullm_b200.csrc import kernels

    K = kernels()
    H, I, V = QWEN3_8B["hidden_size"], QWEN3_8B["intermediate_size"], QWEN3_8B["vocab_size"]
    qkv = (QWEN3_8B["num_attention_heads"] + 2 * QWEN3_8B["num_key_value_heads"]) * QWEN3_8B["head_dim"]
    shapes = {"qkv": (qkv, H), "o": (H, H), "gate_up": (2 * I, H), "down": (H, I), "head": (V, H)}
    M = args.batch
    pk = peaks()

    def timeit(fn, copies, iters=20):
        for i in range(copies):
            fn(i)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(iters):
                fn(i % copies)
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (2 * iters) * 1000.0

    if args.only and args.only != "tail":
        # one kernel on one shape, launched eagerly a few times: what a profiler is pointed at
        N, Kd = shapes[args.shape]
        ws = [torch.randn(N, Kd, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(2)]
        x = torch.randn(M, Kd, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        fn = {"stream": K.stream_linear, "skinny": K.skinny_linear, "tcgen05": K.small_m_linear,
              "library": lambda a, b, c: torch.mm(a, b.t(), out=c)}[args.only]
        for i in range(args.steps):
            fn(x, ws[i % 2], out)
        torch.cuda.synchronize()
        K.raise_on_status()
        print(f"probe linear: {args.only} on {args.shape} ({N} x {Kd}), {M} rows, {args.steps} launches")
        return 0
    print(f"rows {M}; microseconds per product (weights streamed at the copy peak: 'ideal')")
    if M <= 16:
        # the second half of a layer: output projection + residual, norm, gate_up + activation, down + residual
        QD = QWEN3_8B["num_attention_heads"] * QWEN3_8B["head_dim"]
        sets = [(torch.randn(H, QD, device="cuda", dtype=torch.bfloat16) * 0.02,
                 torch.randn(2 * I, H, device="cuda", dtype=torch.bfloat16) * 0.02,
                 torch.randn(H, I, device="cuda", dtype=torch.bfloat16) * 0.02) for _ in range(2)]
        attn = torch.randn(M, QD, device="cuda", dtype=torch.bfloat16)
        res = torch.randn(M, H, device="cuda", dtype=torch.bfloat16)
        nw = torch.ones(H, device="cuda")
        hbuf, o_out = torch.empty_like(res), torch.empty_like(res)
        gu = torch.empty(M, 2 * I, device="cuda", dtype=torch.bfloat16)
        act = torch.empty(M, I, device="cuda", dtype=torch.bfloat16)

        def separate(i):
            wo, wgu, wd = sets[i]
            K.linear(attn, wo, o_out)
            K.add_rmsnorm(o_out, res, nw, 1e-6, hbuf)
            K.linear_act_mul(hbuf, wgu, act, gu, 0)
            K.linear(act, wd, o_out)

        def fused(i):
            wo, wgu, wd = sets[i]
            K.fused_layer_tail(attn, res, act, wo, wgu, wd, nw, 1e-6, 0)

        nbytes = sum(t.numel() for t in sets[0]) * 2
        ts, tf = timeit(separate, 2), timeit(fused, 2)
        print(f"layer tail ({nbytes / 1e6:.0f} MB of weights, ideal {nbytes / (pk['hbm_gbs'] * 1e9) * 1e6:.1f} us): "
              f"separate kernels {ts:.1f} us, fused {tf:.1f} us ({nbytes / tf / 1e6:.2f} TB/s), grid "
              f"{K.lib.ullm_layer_tail_fused_last_grid()}")
        K.raise_on_status()
        if args.only == "tail":
            K.lib.ullm_layer_tail_fused_phase_mask.argtypes = [ctypes.c_int]
            for mask, what in ((0, "no product at all (launch, barriers, norm)"), (1, "output projection alone"), (2, "gate_up alone"), (4, "down alone"), (3, "o + gate_up"),
                               (6, "gate_up + down")):
                K.lib.ullm_layer_tail_fused_phase_mask(mask)
                print(f"   phases {what}: {timeit(fused, 2):.1f} us")
                K._tail_ws[H][1].zero_()
            K.lib.ullm_layer_tail_fused_phase_mask(7)
            return 0
    for name, (N, Kd) in shapes.items():
        nbytes = N * Kd * 2
        copies = max(2, int(300e6 // nbytes) + 1)
        ws = [torch.randn(N, Kd, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
        x = torch.randn(M, Kd, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        t = {"library": timeit(lambda i: torch.mm(x, ws[i].t(), out=out), copies)}
        if K.lt_linear(x, ws[0], out):  # times the library's candidates for this shape once
            ch = K.lt_last_choice()
            t[f"library, timed choice (#{ch['chosen']} of {ch['candidates']})"] = timeit(
                lambda i: K.lt_linear(x, ws[i], out, tune=False), copies)
        if M <= 64:
            t["tcgen05"] = timeit(lambda i: K.small_m_linear(x, ws[i], out), copies)
        else:
            t["tcgen05 128-row tiles"] = timeit(lambda i: K.large_linear(x, ws[i], out, None, None, 1), copies)
            t["256-row tiles"] = timeit(lambda i: K.large_linear(x, ws[i], out, None, None, 2), copies)
        if M <= 32:
            t["skinny"] = timeit(lambda i: K.skinny_linear(x, ws[i], out), copies)
            for ks in (1, 8):
                K.lib.ullm_linear_stream_ksplit_max(ks)
                t["stream" + (", no clusters" if ks == 1 else "")] = timeit(lambda i: K.stream_linear(x, ws[i], out), copies)
        line = "  ".join(f"{k} {v:.1f} ({nbytes / v / 1e6:4.2f})" for k, v in t.items())
        print(f"{name:8s} N={N:6d} K={Kd:5d}  ideal {nbytes / (pk['hbm_gbs'] * 1e9) * 1e6:.1f}  us (TB/s): {line}")
        if name == "gate_up":
            act = torch.empty(M, N // 2, device="cuda", dtype=torch.bfloat16)
            t = {"library+act_mul": timeit(lambda i: (torch.mm(x, ws[i].t(), out=out), K.act_mul(out, act, 0)), copies)}
            if M <= 64:
                t["tcgen05 fused"] = timeit(lambda i: K.small_m_linear(x, ws[i], act, None, 0), copies)
            else:
                t["tcgen05 fused 128-row tiles"] = timeit(lambda i: K.large_linear(x, ws[i], act, None, 0, 1), copies)
                t["256-row tiles"] = timeit(lambda i: K.large_linear(x, ws[i], act, None, 0, 2), copies)
            if M <= 32:
                t["skinny fused"] = timeit(lambda i: K.skinny_linear(x, ws[i], act, None, 0), copies)
                t["stream fused"] = timeit(lambda i: K.stream_linear(x, ws[i], act, None, 0), copies)
            print("         with the gate activation:  " + "  ".join(f"{k} {v:7.1f}" for k, v in t.items()))
        del ws
    K.raise_on_status()
    return 0


def run_decode_attention_probe(args) -> int:
    """`--probe decode-attention`: the two bfloat16 decode attention kernels alone (Qwen3-8B head sizes, pages of
    16 tokens) on batches of equal and of very unequal lengths; microseconds per call, launched eagerly (about
    10 us of launch cost are in every figure), L2 flushed before each call."""
    import random

    import torch

    from ullm_b200.csrc import kernels
    from ullm_b200.engine.batch import Workspace

    K = kernels()
    Hq, Hkv, D, page = (QWEN3_8B["num_attention_heads"], QWEN3_8B["num_key_value_heads"], QWEN3_8B["head_dim"],
                        args.page_size)
    pk = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    class Ctx:
        pass

    def case(name, lens):
        if args.case is not None and args.case != name:
            return
        B = len(lens)
        per = [-(-n // page) for n in lens]
        pages = sum(per) + 4
        kp = torch.randn(pages, page, Hkv, D, device="cuda", dtype=torch.bfloat16)
        vp = torch.randn(pages, page, Hkv, D, device="cuda", dtype=torch.bfloat16)
        bt = torch.full((B, max(per)), -1, dtype=torch.int32)
        o = 0
        for i, n in enumerate(per):
            bt[i, :n] = torch.arange(o, o + n, dtype=torch.int32)
            o += n
        bt = bt.cuda()
        qkv = torch.randn(B, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16)
        ctx = Ctx()
        ctx.decode_only, ctx.num_requests, ctx.max_q_len = True, B, 1
        ctx.workspace = Workspace(torch.device("cuda"))
        slots = torch.arange(B, dtype=torch.int32, device="cuda")
        cu = torch.arange(B + 1, dtype=torch.int32, device="cuda")
        kvl = torch.tensor(lens, dtype=torch.int32, device="cuda")
        res, outs = {}, []
        for mode in ("split", "balanced", "tcgen05"):
            K.use_balanced_decode, K.use_tcgen05_decode = mode == "balanced", mode == "tcgen05"
            out = torch.empty(B, Hq * D, device="cuda", dtype=torch.bfloat16)
            ts = []
            for _ in range(7):
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                K.paged_attention(qkv, out, kp, vp, bt, slots, cu, kvl, slots, Hq, Hkv, D, page, 0, D ** -0.5, ctx)
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1) * 1000)
            res[mode] = statistics.median(ts[2:])
            outs.append(out.float())
        mb = sum(lens) * Hkv * D * 2 * 2 / 1e6
        print(f"{name:28s} K+V {mb:7.1f} MB  at the copy peak {mb / pk['hbm_gbs'] * 1e3:6.1f} us   "
              f"per-request splits {res['split']:7.1f} us   batch-balanced {res['balanced']:7.1f} us   "
              f"tcgen05 {res['tcgen05']:7.1f} us   (largest differences of the outputs "
              f"{(outs[0] - outs[1]).abs().max().item():.1e}, {(outs[0] - outs[2]).abs().max().item():.1e})")

    random.seed(1)
    case("8 x 2048", [2048] * 8)
    case("16 x 2048", [2048] * 16)
    case("24 x 2048", [2048] * 24)
    case("32 x 2048", [2048] * 32)
    case("48 x 2048", [2048] * 48)
    case("64 x 2048", [2048] * 64)
    case("1 x 2048", [2048])
    case("4 x 8192", [8192] * 4)
    case("128 x 1024", [1024] * 128)
    case("1 x 16384 + 15 x 256", [16384] + [256] * 15)
    case("1 x 32768 + 63 x 512", [32768] + [512] * 63)
    case("64 x uniform(64..4096)", [random.randint(64, 4096) for _ in range(64)])
    case("32 x uniform(16..8192)", [random.randint(16, 8192) for _ in range(32)])
    K.raise_on_status()
    return 0


def run_prefill_attention_probe(args) -> int:
    """`--probe prefill-attention`: the bfloat16 prompt attention kernels alone (Qwen3-8B head sizes): whole
    prompts and portions that continue a context; microseconds per call (ten calls back to back in a CUDA graph,
    median of 5 replays after 2; `--steps 1`: one call per replay),
    TFLOP/s of the causal work, and the largest difference between the kernels' outputs."""
    import torch

    from ullm_b200.csrc import kernels

    K = kernels()
    Hq, Hkv, D, page = (QWEN3_8B["num_attention_heads"], QWEN3_8B["num_key_value_heads"], QWEN3_8B["head_dim"],
                        args.page_size)
    pk = peaks()

    class Ctx:
        pass

    def case(name, q_lens, kv_lens):
        B, T = len(q_lens), sum(q_lens)
        per = [-(-n // page) for n in kv_lens]
        pages = sum(per) + 4
        kp = torch.randn(pages, page, Hkv, D, device="cuda", dtype=torch.bfloat16)
        vp = torch.randn(pages, page, Hkv, D, device="cuda", dtype=torch.bfloat16)
        bt = torch.full((B, max(per)), -1, dtype=torch.int32)
        o = 0
        for i, n in enumerate(per):
            bt[i, :n] = torch.arange(o, o + n, dtype=torch.int32)
            o += n
        bt = bt.cuda()
        qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16)
        ctx = Ctx()
        ctx.decode_only, ctx.num_requests, ctx.max_q_len = False, B, max(q_lens)
        ctx.cu_q_host = None
        slots = torch.arange(B, dtype=torch.int32, device="cuda")
        cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device="cuda")
        kvl = torch.tensor(kv_lens, dtype=torch.int32, device="cuda")
        token_req = torch.cat([torch.full((n,), r, dtype=torch.int32) for r, n in enumerate(q_lens)]).cuda()
        res, outs = {}, []
        for mode in ("pair", "single", "0"):
            K.tc_attention_mode, K.use_tcgen05_attention = mode, mode != "0"
            out = torch.empty(T, Hq * D, device="cuda", dtype=torch.bfloat16)

            def call():
                K.paged_attention(qkv, out, kp, vp, bt, slots, cu, kvl, token_req, Hq, Hkv, D, page, 0, D ** -0.5, ctx)

            call()
            torch.cuda.synchronize()
            reps = 1 if args.steps == 1 else 10
            graph = torch.cuda.CUDAGraph()  # `reps` launches back to back: no host time between them
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    for _ in range(reps):
                        call()
            ts = []
            for _ in range(7):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                graph.replay()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1) * 1000 / reps)
            res[mode] = statistics.median(ts[2:])
            outs.append(out.float())
        K.raise_on_status()
        # causal work: row t of a request sees kv - q + t + 1 keys; 4 flops per (row, key, head, dim)
        keys = sum(q * (k - q) + q * (q + 1) // 2 for q, k in zip(q_lens, kv_lens))
        gf = 4.0 * keys * Hq * D / 1e9
        tf = {m: gf / res[m] * 1e3 for m in res}
        print(f"{name:34s} {gf:8.1f} GFLOP   two tiles per block {res['pair']:8.1f} us = {tf['pair']:6.0f} TFLOP/s "
              f"({tf['pair'] / pk['bf16_tflops']:.2f} of burst)   one tile {res['single']:8.1f} us = {tf['single']:6.0f}   "
              f"mma.sync {res['0']:8.1f} us = {tf['0']:6.0f}   (largest differences "
              f"{(outs[0] - outs[1]).abs().max().item():.1e}, {(outs[0] - outs[2]).abs().max().item():.1e})", flush=True)

    cases = [("1 x 2048", [2048], [2048]), ("1 x 512", [512], [512]), ("4 x 512", [512] * 4, [512] * 4),
             ("1 x 8192", [8192], [8192]), ("1 x 16384", [16384], [16384]),
             ("2048 behind 6144", [2048], [8192]), ("8 x 256 behind 1792", [256] * 8, [2048] * 8),
             ("64 + 37 + 300 + 1 (mixed)", [64, 37, 300, 1], [640, 37, 900, 77])]
    for c in cases:
        if args.case is None or args.case == c[0]:
            case(*c)
    K.apply_switches(os.environ)
    return 0


def run_mma_rate_probe(args) -> int:
    """`--probe mma-rate`: clocks per tcgen05.mma (bfloat16, M = 128, K = 16) issued back to back by one thread, on
    one block and on one block per SM (csrc/tcgen05_rate_probe.cu)."""
    import torch

    from ullm_b200.csrc import kernels

    K = kernels()
    lib = K.lib
    lib.ullm_tcgen05_mma_rate.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                                          ctypes.c_void_p]
    lib.ullm_tcgen05_mma_rate.restype = ctypes.c_int
    out = torch.zeros(2, dtype=torch.int64, device="cuda")
    names = ["A and B from shared memory, N = 128", "A and B from shared memory, N = 256",
             "A from tensor memory, B MN-major, N = 128", "A and B from shared memory, N = 64",
             "8 x (shared, N = 128) then 8 x (tensor memory, N = 128)"]
    for blocks in (1, K.sm_count):
        for mode, name in enumerate(names):
            for _ in range(2):
                n = lib.ullm_tcgen05_mma_rate(mode, 2000, blocks, out.data_ptr(), K.status.data_ptr(), None)
                torch.cuda.synchronize()
            K.raise_on_status()
            print(f"{blocks:4d} block(s)  {name:58s} {out[0].item() / n:6.1f} clocks per product", flush=True)
    return 0


def run_sampling_probe(args) -> int:
    """`--probe sampling`: the two sampling kernels alone on `--batch` rows of the benchmark's vocabulary, one
    parameter set for all rows; microseconds per call, 20 calls recorded in a CUDA graph (the logits stay in L2,
    as they do behind the output head's product)."""
    import torch

    from ullm_b200.csrc import kernels
    from ullm_b200.sampling.params import SamplingParams
    from ullm_b200.sampling.sampler import Sampler

    K = kernels()
    V, R = QWEN3_8B["vocab_size"], args.batch
    logits = torch.randn(R, V, device="cuda") * 3
    s = Sampler("cuda", R, V)
    cases = [("greedy", SamplingParams(temperature=0.0)), ("temperature", SamplingParams(temperature=0.8)),
             ("top_k 50", SamplingParams(temperature=0.8, top_k=50)), ("top_p 0.9", SamplingParams(temperature=0.8, top_p=0.9)),
             ("top_k 50 + top_p 0.9", SamplingParams(temperature=0.8, top_k=50, top_p=0.9)),
             ("min_p 0.05", SamplingParams(temperature=0.8, min_p=0.05))]
    print(f"rows {R}, vocabulary {V}; microseconds per call")
    for name, p in cases:
        s.stage([p] * R, list(range(R)), [3] * R)
        t = {}
        for label, one_block in (("one block per row", True), ("cluster of 8 blocks per row", False)):
            K.sample_force_one_block(one_block)
            try:
                s.run(logits, R)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    for _ in range(20):
                        s.run(logits, R)
                ts = []
                for _ in range(6):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    g.replay()
                    e1.record()
                    torch.cuda.synchronize()
                    ts.append(e0.elapsed_time(e1) * 1000 / 20)
                t[label] = statistics.median(ts[2:])
            finally:
                K.sample_force_one_block(False)
        print(f"{name:24s} " + "   ".join(f"{k} {v:8.1f}" for k, v in t.items()))
    K.raise_on_status()
    return 0


def write_synthetic_tokenizer(path: str, vocab_size: int) -> None:
    """Tokenizer files that know every id of a `vocab_size`-token vocabulary (byte-level alphabet first, then
    "tok0", "tok1", ...), and config.json's model_type: the reference's LLM loads a tokenizer unconditionally.
    Ids go in and out as integers; the tokenizer only has to exist."""
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    cs, n = bs[:], 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    vocab = {chr(c): i for i, c in enumerate(cs)}
    i = 0
    while len(vocab) < vocab_size:
        t = f"tok{i}"
        i += 1
        if t not in vocab:
            vocab[t] = len(vocab)
    with open(os.path.join(path, "vocab.json"), "w") as f:
        json.dump(vocab, f)
    with open(os.path.join(path, "merges.txt"), "w") as f:
        f.write("#version: 0.2\n")
    with open(os.path.join(path, "tokenizer_config.json"), "w") as f:
        json.dump({"tokenizer_class": "Qwen2Tokenizer", "eos_token": "tok0", "pad_token": "tok0",
                   "model_max_length": 40960}, f)
    with open(os.path.join(path, "config.json")) as f:
        c = json.load(f)
    c["model_type"] = "qwen3"
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(c, f)


def _write_reference_model(path: str, cfg: dict) -> None:
    """A model folder the reference can open: random weights (this repo's seeded writer) and the synthetic
    tokenizer."""
    from ullm_b200.weights import write_random_model

    write_random_model(path, cfg, seed=0, std=0.02, norm_std=0.0, dtype="bfloat16")
    write_synthetic_tokenizer(path, cfg["vocab_size"])


def _reference_available() -> str | None:
    """None when the reference can run here, else the reason it cannot."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "ullm", "core")):
        return "izmttk/ullm is not installed under baseline/_ref"
    import torch

    if not torch.cuda.is_available():
        return "no CUDA device here (the reference's engine process needs one)"
    if ref not in sys.path:
        sys.path.insert(0, ref)
    return None


class _StdoutToStderr:
    """The reference logs to standard output, from child processes too: descriptor 1 goes to standard error
    while it runs, so that this program's standard output holds the one JSON line only."""

    def __enter__(self):
        sys.stdout.flush()
        self.saved = os.dup(1)
        os.dup2(2, 1)

    def __exit__(self, *a):
        sys.stdout.flush()
        os.dup2(self.saved, 1)
        os.close(self.saved)


def run_reference(args) -> dict:
    """izmttk/ullm itself, unmodified, from baseline/_ref, through its own `LLM.generate`: the same metric
    (decode tokens per second at the given batch, requests holding 2,048 tokens) by the wall clock between
    streamed tokens.  Requests are started one after the other, each once the one before has its first token:
    the reference raises on a prefill step that holds several new requests (ullm/core/input_batch.py:185
    broadcasts [tokens] against [requests])."""
    import asyncio

    why = _reference_available()
    if why:
        return {"impl": "reference", "unavailable": why}
    label, shape = SHAPES[args.workload]
    cfg = dict(shape)
    full_layers = cfg["num_hidden_layers"]
    layers = args.layers or full_layers
    cfg["num_hidden_layers"] = layers
    K, W, B = args.steps, args.warmup, args.batch
    with _StdoutToStderr():
        try:
            import torch

            tmp = tempfile.mkdtemp(prefix="ullm_ref_model_")
            _write_reference_model(tmp, cfg)
            from ullm import LLM, EngineConfig, SamplingParams  # the reference's public API

            g = torch.Generator().manual_seed(1)
            prompts = [torch.randint(0, cfg["vocab_size"], (START_CONTEXT,), generator=g).tolist() for _ in range(B + 1)]
            stamps: list[list[float]] = [[] for _ in prompts]
            result: dict = {}

            async def main_async():
                llm = LLM(EngineConfig(model=tmp, gpu_memory_utilization=0.8, max_bs=max(B, 8), tp_size=1, pp_size=1,
                                       nccl_port=29533, device_ids=[0], context_len=CONTEXT_LEN))
                first = [asyncio.Event() for _ in prompts]

                async def run(i, n_new):
                    sp = SamplingParams(temperature=1.0, top_k=1, ignore_eos=True, max_new_tokens=n_new)
                    async for _out in llm.generate(prompts[i], sp):
                        stamps[i].append(time.perf_counter())
                        first[i].set()

                # prefill of one 2,048-token prompt: submit -> first token (after one untimed run, which also
                # pays for the attention library's just-in-time compilation)
                await run(B, 1)
                stamps[B].clear()
                t0 = time.perf_counter()
                await run(B, 1)
                result["prefill_s"] = stamps[B][0] - t0
                tasks = []
                for i in range(B):
                    tasks.append(asyncio.create_task(run(i, 2 * B + W + K + 8)))
                    await first[i].wait()
                await asyncio.gather(*tasks)
                await llm.shutdown()

            asyncio.run(main_async())
            # the window in which all B requests decode: from token (B + W) of the last-started request on
            start = max(s[-(K + 1)] for s in stamps[:B])
            end = max(s[-1] for s in stamps[:B])
            steps_ms = (end - start) / K * 1e3
            value = B * K / (end - start)
            config = common_config(label, shape, layers, B)
            config.update({"kv_dtype": "bf16", "l2": "inputs>L2 (each step streams all weights)", "peaks": "n/a",
                           "cuda_graph": True, "timing": "wall clock between streamed tokens", "num_pages": None})
            return {
                "impl": "reference", "metric": metric_name(B, label), "value": round(value, 1),
                "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": round(steps_ms, 4),
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
                "data": "synthetic (random weights, uniform random token ids)",
                "config": config,
                "e2e": {"value": round(value, 1), "unit": "tok/s", "api": "LLM.generate"},
                "prefill": {"value": round(PREFILL_TOKENS / result["prefill_s"], 1), "tokens": PREFILL_TOKENS,
                            "ms": round(result["prefill_s"] * 1e3, 3)},
                "points": {f"decode_b{B}": round(value, 1)},
            }
        except BaseException as e:  # the reference kills its process tree on errors; report, do not propagate
            msg = f"{type(e).__name__}: {e}".splitlines()[0][:300]
            return {"impl": "reference", "unavailable": f"izmttk/ullm failed to run here: {msg}"}


def run_reference_serve(args) -> dict:
    """The serving workload through the reference: the same prompts and output lengths as `run_serve`, streamed
    through its `LLM.generate`.  As in its own bench.py all requests are submitted from one task list, except
    that each is submitted once the one before has its first token (a prefill step that holds several new
    requests raises in its current tree, ullm/core/input_batch.py:185); decoding goes on meanwhile, so the
    batch grows as in continuous batching."""
    import asyncio

    why = _reference_available()
    if why:
        return {"impl": "reference", "unavailable": why}
    label, shape = SHAPES["0.6b"]
    cfg = dict(shape)
    layers = args.layers or cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = layers
    with _StdoutToStderr():
        try:
            tmp = tempfile.mkdtemp(prefix="ullm_ref_model_")
            # the reference never ties the head: its loader wants lm_head.weight in the file
            _write_reference_model(tmp, dict(cfg, tie_word_embeddings=False))
            from ullm import LLM, EngineConfig, SamplingParams

            prompts, outs = serve_workload(cfg["vocab_size"])
            done = [0] * len(prompts)
            result: dict = {}

            async def main_async():
                llm = LLM(EngineConfig(model=tmp, gpu_memory_utilization=0.8, max_bs=SERVE_REQUESTS, tp_size=1,
                                       pp_size=1, nccl_port=29534, device_ids=[0], context_len=CONTEXT_LEN))
                first = [asyncio.Event() for _ in prompts]

                async def run(i, n_new):
                    sp = SamplingParams(temperature=0.6, ignore_eos=True, max_new_tokens=n_new)
                    async for _out in llm.generate(prompts[i], sp):
                        done[i] += 1
                        first[i].set()

                await run(0, 8)  # untimed: the attention library compiles at its first call
                done[0] = 0
                first[0].clear()
                t0 = time.perf_counter()
                tasks = []
                for i, n in enumerate(outs):
                    tasks.append(asyncio.create_task(run(i, n)))
                    await first[i].wait()
                await asyncio.gather(*tasks)
                result["s"] = time.perf_counter() - t0
                await llm.shutdown()

            asyncio.run(main_async())
            # (the reference hands back one token fewer than max_new_tokens for most requests; what counts is what
            # came back)
            if any(d < n - 1 or d > n for d, n in zip(done, outs)):
                raise RuntimeError(f"{sum(done)} tokens came back, {sum(outs)} were asked for")
            gen, pro, dt = sum(done), sum(len(p) for p in prompts), result["s"]
            config = common_config(label, shape, layers, SERVE_REQUESTS)
            config.update({"requests": SERVE_REQUESTS, "prompt_tokens": pro, "generated_tokens": gen,
                           "lengths": f"uniform {SERVE_MIN}..{SERVE_MAX}, seed {SERVE_SEED}", "temperature": 0.6,
                           "timing": "wall clock around the generate tasks"})
            config.pop("start_context")
            return {
                "impl": "reference",
                "metric": f"generated tok/s, {SERVE_REQUESTS} requests under continuous batching, {label}",
                "value": round(gen / dt, 1), "unit": "tok/s", "n_gpus": 1, "steps": 0, "warmup": 1,
                "ms_per_step": None, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "bf16", "data": "synthetic (random weights, uniform random token ids)", "config": config,
                "seconds": round(dt, 3), "total_tok_s": round((gen + pro) / dt, 1),
                "e2e": {"value": round(gen / dt, 1), "unit": "tok/s", "api": "LLM.generate"},
            }
        except BaseException as e:
            msg = f"{type(e).__name__}: {e}".splitlines()[0][:300]
            return {"impl": "reference", "unavailable": f"izmttk/ullm failed to run here: {msg}"}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--workload", default="8b", choices=["8b", "32b", "serve-0.6b", "8b-long"],
                    help="8b: the default line (Qwen3-8B layer sizes); 32b: the same at Qwen3-32B layer sizes; "
                         "serve-0.6b: 256 requests under continuous batching at Qwen3-0.6B layer sizes; 8b-long: "
                         "prefill of 16,384 tokens and decode of 8 requests at that context")
    ap.add_argument("--no-extra-shapes", action="store_true",
                    help="the default line without the 32b and serve-0.6b runs that it adds to `points`")
    ap.add_argument("--no-groups", action="store_true", help="skip the per-kernel-group times of the decode step")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    ap.add_argument("--probe", default=None, choices=["decode", "prefill", "linear", "decode-attention", "prefill-attention", "mma-rate", "sampling"],
                    help="a few eager steps for a profiler; linear: the decode step's matrix products alone")
    ap.add_argument("--only", default=None, choices=["stream", "skinny", "tcgen05", "library", "tail"],
                    help="--probe linear: launch only this kernel, eagerly, --steps times (for a profiler)")
    ap.add_argument("--shape", default="gate_up", choices=["qkv", "o", "gate_up", "down", "head"],
                    help="--probe linear --only: which of the decode step's products")
    ap.add_argument("--case", default=None, help="run only the case of this name (--probe prefill-attention, decode-attention)")
    ap.add_argument("--context", type=int, default=START_CONTEXT, help="tokens each request holds (--probe)")
    ap.add_argument("--page-size", type=int, default=PAGE_SIZE, help="tokens of a page (--probe decode-attention)")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.probe == "linear":
        return run_linear_probe(args)
    if args.probe == "mma-rate":
        return run_mma_rate_probe(args)
    if args.probe == "prefill-attention":
        return run_prefill_attention_probe(args)
    if args.probe == "decode-attention":
        return run_decode_attention_probe(args)
    if args.probe == "sampling":
        return run_sampling_probe(args)
    if args.probe:
        return run_probe(args)
    extra = args.workload == "8b" and not args.no_extra_shapes and not args.layers
    if args.impl == "reference":
        out = run_reference_serve(args) if args.workload == "serve-0.6b" else run_reference(args)
        if extra and "unavailable" not in out:
            out.setdefault("points", {}).update(run_extra_shapes(args, "reference"))
        print(json.dumps(out))
        return 0
    import torch

    if not torch.cuda.is_available():
        print("bench.py: no CUDA device: this engine has no CPU path", file=sys.stderr)
        return 1
    if args.workload == "8b-long":
        print(json.dumps(run_long_context(args)))
        return 0
    out = run_serve(args) if args.workload == "serve-0.6b" else run_ours(args)
    if extra:
        import gc

        gc.collect()  # this run's engine goes first: the further shapes run in processes of their own
        torch.cuda.empty_cache()
        out["points"].update(run_extra_shapes(args, "ours"))
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
