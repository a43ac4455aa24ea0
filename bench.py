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

# BASELINE.json configs[2]: Qwen3-8B layer sizes
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
CONTEXT_LEN = 4096
START_CONTEXT = 2048
PREFILL_TOKENS = 2048
PAGE_SIZE = 16


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


def run_ours(args) -> dict:
    import torch

    from ullm_b200.config import EngineConfig
    from ullm_b200.csrc import kernels
    from ullm_b200.engine.llm import LLM
    from ullm_b200.sampling import SamplingParams

    cfg = dict(QWEN3_8B)
    full_layers = cfg["num_hidden_layers"]
    layers = args.layers or full_layers
    cfg["num_hidden_layers"] = layers
    pk = peaks()
    nums = model_numbers(cfg, layers)
    K, W = args.steps, args.warmup
    max_bs = 64
    tmp = tempfile.mkdtemp(prefix="ullm_b200_bench_")
    with open(os.path.join(tmp, "config.json"), "w") as f:
        json.dump(cfg, f)
    tokens_per_req = START_CONTEXT + 2 * (K + W) + 64
    num_pages = max_bs * (-(-tokens_per_req // PAGE_SIZE)) + 64
    ec = EngineConfig(
        model=tmp, max_bs=max_bs, context_len=CONTEXT_LEN, page_size=PAGE_SIZE, num_pages=num_pages,
        max_num_batched_tokens=4096, dtype="bfloat16", load_format="random", seed=0, enable_prefix_caching=False,
        log_level="warning",
    )
    llm = LLM(ec)
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

    def time_decode(B, tag, steps, warmup):
        """Device-timed decode through Engine.step: (ms per step, wall seconds per step, launches per step)."""
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
        # the device side alone: the captured step replayed back to back (it rewrites the same cache slots)
        graph_ms = None
        dg = eng.decode_graphs
        even = [v for k, v in (dg.graphs.items() if dg is not None else ()) if k[0] == dg.padded(B) and not any(k[1])]
        if dg is not None and dg.takes(B) and even:
            g0 = even[0][0]
            torch.cuda.synchronize()
            e0.record()
            for _ in range(steps):
                g0.replay()
            e1.record()
            torch.cuda.synchronize()
            graph_ms = e0.elapsed_time(e1) / steps
        stop_batch(ids)
        time_decode.graph_ms = graph_ms
        return ms, wall / steps, launches, ctx

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
               "frac": round(pflops / (pre / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}

    # ---- decode ----------------------------------------------------------------------
    B = args.batch
    with ClockSampler() as clk:
        ms, wall, launches, ctx = time_decode(B, "d", K, W)
    clocks = clk.summary()
    graph_ms = time_decode.graph_ms
    value = B / (ms / 1e3)
    # End to end through the call a user makes: LLM.generate_batch, token ids in, token ids out.  Two calls on
    # fresh prompts of the same lengths, W and W + K new tokens each: their prompt work is the same, the
    # difference of their wall times is K decode steps (each with its staging copy from pinned memory and the
    # read of its sampled ids) as the user sees them.
    def user_call(n_new):
        ps = [prompt(START_CONTEXT) for _ in range(B)]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        outs = llm.generate_batch(ps, SamplingParams(temperature=0.0, ignore_eos=True, max_new_tokens=n_new))
        dt = time.perf_counter() - t0
        assert all(len(o.token_ids) == n_new for o in outs)
        return dt
    user_call(W)  # warm
    t_short = min(user_call(W) for _ in range(2))
    t_long = min(user_call(W + K) for _ in range(2))
    e2e_value = B * K / max(t_long - t_short, 1e-9)
    e2e_steps_value = B / wall  # the same loop as `value`, by the wall clock
    dbytes = decode_bytes(nums, B, ctx, cfg["hidden_size"])
    achieved = dbytes / (ms / 1e3) / 1e9
    points = {}
    for pb in (1, 64):
        pms, _pw, _pl, _pc = time_decode(pb, f"b{pb}_", max(8, K // 2), max(3, W))
        points[f"decode_b{pb}"] = round(pb / (pms / 1e3), 1)
        if time_decode.graph_ms:
            points[f"decode_b{pb}_device_only_ms"] = round(time_decode.graph_ms, 4)
            points[f"decode_b{pb}_ms"] = round(pms, 4)
    st = runner.decode_staging
    h2d = st.layout(st.max_tokens, st.max_requests)["_end"][0] * 4 + eng.sampler.host.numel() * 4
    out = {
        "metric": "decode tok/s at batch 8, Qwen3-8B shape (also batch 1/64 and 2048-token prefill)",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights, uniform random token ids)",
        "config": {
            "model": "Qwen3-8B shape", "global_batch": B, "seq_len": CONTEXT_LEN, "parallelism": "single-gpu",
            "layers": layers, "layers_of_config": full_layers, "hidden_size": cfg["hidden_size"],
            "num_attention_heads": cfg["num_attention_heads"], "num_key_value_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate_size": cfg["intermediate_size"],
            "vocab_size": cfg["vocab_size"], "start_context": START_CONTEXT, "page_size": PAGE_SIZE,
            "kv_dtype": "bf16", "l2": "inputs>L2 (each step streams all weights)", "peaks": pk["source"],
            "cuda_graph": not ec.enforce_eager,
        },
        "clocks": clocks,
        "e2e": {"value": round(e2e_value, 1), "unit": "tok/s", "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(B * 4), "api": "LLM.generate_batch",
                "engine_step_wall_value": round(e2e_steps_value, 1)},
        "gpu_launches": int(round(launches * K)),
        "device_only_ms_per_step": round(graph_ms, 4) if graph_ms else None,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
    }
    return out


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

    print(f"rows {M}; microseconds per product (weights streamed at the copy peak: 'ideal')")
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
        line = "  ".join(f"{k} {v:7.1f} ({nbytes / v / 1e6:4.2f} TB/s)" for k, v in t.items())
        print(f"{name:8s} N={N:6d} K={Kd:5d}  {line}  ideal {nbytes / (pk['hbm_gbs'] * 1e9) * 1e6:6.1f}")
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


def run_reference(args) -> dict:
    """izmttk/ullm itself, unmodified, from baseline/_ref, through its own `LLM.generate`: the same metric
    (decode tokens per second at the given batch, requests holding 2,048 tokens) by the wall clock between
    streamed tokens.  Requests are started one after the other, each once the one before has its first token:
    the reference's default (asynchronous) scheduling raises on a prefill step that holds several requests
    (ullm/core/input_batch.py:185 broadcasts [tokens] against [requests])."""
    import asyncio

    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "ullm", "core")):
        return {"impl": "reference", "unavailable": "izmttk/ullm is not installed under baseline/_ref"}
    import torch

    if not torch.cuda.is_available():
        return {"impl": "reference", "unavailable": "no CUDA device here (the reference's engine process needs one)"}
    sys.path.insert(0, ref)
    cfg = dict(QWEN3_8B)
    full_layers = cfg["num_hidden_layers"]
    layers = args.layers or full_layers
    cfg["num_hidden_layers"] = layers
    K, W, B = args.steps, args.warmup, args.batch
    # the reference logs to standard output, from child processes too: send descriptor 1 to standard error
    # while it runs, so that this program's standard output holds the one JSON line only
    sys.stdout.flush()
    saved_stdout = os.dup(1)
    os.dup2(2, 1)
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
        return {
            "impl": "reference", "metric": "decode tok/s at batch 8, Qwen3-8B shape", "value": round(value, 1),
            "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": round(steps_ms, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (random weights, uniform random token ids)",
            "config": {"model": "Qwen3-8B shape", "global_batch": B, "seq_len": CONTEXT_LEN,
                       "parallelism": "single-gpu", "layers": layers, "layers_of_config": full_layers,
                       "start_context": START_CONTEXT, "timing": "wall clock between streamed tokens"},
            "e2e": {"value": round(value, 1), "unit": "tok/s"},
            "prefill": {"value": round(PREFILL_TOKENS / result["prefill_s"], 1), "tokens": PREFILL_TOKENS,
                        "ms": round(result["prefill_s"] * 1e3, 3)},
        }
    except BaseException as e:  # the reference kills its process tree on errors; report, do not propagate
        msg = f"{type(e).__name__}: {e}".splitlines()[0][:300]
        return {"impl": "reference", "unavailable": f"izmttk/ullm failed to run here: {msg}"}
    finally:
        sys.stdout.flush()
        os.dup2(saved_stdout, 1)
        os.close(saved_stdout)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    ap.add_argument("--probe", default=None, choices=["decode", "prefill", "linear", "decode-attention", "sampling"],
                    help="a few eager steps for a profiler; linear: the decode step's matrix products alone")
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
    if args.probe == "decode-attention":
        return run_decode_attention_probe(args)
    if args.probe == "sampling":
        return run_sampling_probe(args)
    if args.probe:
        return run_probe(args)
    if args.impl == "reference":
        print(json.dumps(run_reference(args)))
        return 0
    import torch

    if not torch.cuda.is_available():
        print("bench.py: no CUDA device: this engine has no CPU path", file=sys.stderr)
        return 1
    out = run_ours(args)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
