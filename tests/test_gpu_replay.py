"""The engine against the plain implementation under every way of cutting the
work: whole, last 32 tokens one by one, portions of changing size, mixed
batches with so few pages that they are used again.  float32 and bfloat16."""

import json
import os
import subprocess
import sys

import pytest
import torch

from helpers import SHARPEN, assert_close, first_bad_row, plain_logits, random_ids, weights_for, write_model_dir

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# float16 (the reference's default when config.json names no dtype) runs the plain kernels: three configurations
CASES = [(t, d) for d in ("float32", "bfloat16") for t in "ABCDE"] + [(t, "float16") for t in "ABD"]
LENGTHS = {"A": 100, "B": 200, "C": 180, "D": 300, "E": 230}


def make_runner(tmp_path, tag, dtype, num_pages, sharpen=1.0, max_requests=4, **kw):
    from ullm_b200.engine import ModelRunner

    cfg, w, page = weights_for(tag, dtype, sharpen)
    d = write_model_dir(str(tmp_path / f"model_{tag}_{dtype}"), cfg, w)
    from conftest import device

    r = ModelRunner(d, dtype=dtype, device=device(), page_size=page, num_pages=num_pages, max_requests=max_requests,
                    max_context=cfg["max_position_embeddings"], max_step_tokens=64, poison_cache=True, **kw)
    return r, cfg, w, page


def run_cut(runner, rid, ids, cuts, want_all=True):
    """Feeds ids in portions of the given sizes; returns logits at every position."""
    from ullm_b200.engine import StepEntry

    runner.add_request(rid)
    outs, i = [], 0
    for n in cuts:
        lg = runner.step([StepEntry(rid, ids[i:i + n], list(range(n)))])
        outs.append(lg.float().cpu().clone())
        i += n
    runner.check_device_status()
    runner.end_request(rid)
    assert i == len(ids)
    return torch.cat(outs)


@pytest.mark.parametrize("tag,dtype", CASES)
def test_whole_prompt(tmp_path, tag, dtype):
    n = LENGTHS[tag]
    runner, cfg, w, page = make_runner(tmp_path, tag, dtype, num_pages=-(-n // ALL_PAGE(tag)) + 1)
    ids = random_ids(cfg["vocab_size"], n, 11)
    ref = plain_logits(ids, w, cfg)
    got = run_cut(runner, "a", ids, [n])
    assert_close(got, ref, dtype, f"{tag} whole")
    runner.cache.check_invariants()


def ALL_PAGE(tag):
    from tiny_configs import ALL

    return ALL[tag][2]


@pytest.mark.parametrize("tag,dtype", CASES)
def test_last_32_one_by_one(tmp_path, tag, dtype):
    n = LENGTHS[tag]
    runner, cfg, w, page = make_runner(tmp_path, tag, dtype, num_pages=-(-n // ALL_PAGE(tag)) + 1)
    ids = random_ids(cfg["vocab_size"], n, 12)
    ref = plain_logits(ids, w, cfg)
    got = run_cut(runner, "a", ids, [n - 32] + [1] * 32)
    bad = first_bad_row(got, ref, dtype)
    assert bad is None, f"first wrong position {bad} (page size {page}, prefill {n - 32})"
    assert_close(got, ref, dtype, f"{tag} decode")


@pytest.mark.parametrize("tag,dtype", CASES)
def test_portions_of_changing_size(tmp_path, tag, dtype):
    n = LENGTHS[tag]
    runner, cfg, w, page = make_runner(tmp_path, tag, dtype, num_pages=-(-n // ALL_PAGE(tag)) + 1)
    ids = random_ids(cfg["vocab_size"], n, 13)
    ref = plain_logits(ids, w, cfg)
    pattern = [7, 2, 5, 3, 16, 2, 1, 9, 4, 17, 2, 33]
    cuts, left, i = [], n, 0
    while left > 0:
        c = min(pattern[i % len(pattern)], left)
        cuts.append(c)
        left -= c
        i += 1
    got = run_cut(runner, "a", ids, cuts)
    bad = first_bad_row(got, ref, dtype)
    assert bad is None, f"first wrong position {bad}; cuts {cuts}"
    assert_close(got, ref, dtype, f"{tag} portions")


@pytest.mark.parametrize("tag,dtype", CASES)
def test_mixed_batches_with_page_reuse(tmp_path, tag, dtype):
    """Eight requests, at most four live, portions of some beside decoded tokens
    of others; the pool is so small that finished requests' pages are used again."""
    from ullm_b200.engine import StepEntry

    page = ALL_PAGE(tag)
    lens = [37, 64, 21, 50, 33, 48, 10, 59]
    # room for the four longest requests at once, no more
    num_pages = sum(-(-L // page) for L in sorted(lens)[-4:])
    runner, cfg, w, page = make_runner(tmp_path, tag, dtype, num_pages=num_pages)
    prompts = [random_ids(cfg["vocab_size"], L, 20 + i) for i, L in enumerate(lens)]
    refs = [plain_logits(p, w, cfg) for p in prompts]
    # every request: a prefill in portions, then its last 8 tokens one by one
    plans = []
    for i, L in enumerate(lens):
        portions, left = [], L - 8
        sizes = [5 + 3 * i, 2, 11, 7, 30]
        k = 0
        while left > 0:
            c = min(sizes[k % len(sizes)], left)
            portions.append(c)
            left -= c
            k += 1
        plans.append(portions + [1] * 8)
    got = [[] for _ in lens]
    done_at = [0] * len(lens)
    waiting = list(range(len(lens)))
    live: list[int] = []
    page_owners: dict[tuple, set] = {}  # (group, page) -> requests that held it
    steps = 0
    while waiting or live:
        while waiting and len(live) < 4:
            i = waiting.pop(0)
            runner.add_request(f"r{i}")
            live.append(i)
        entries = []
        for i in live:
            n = plans[i].pop(0)
            entries.append(StepEntry(f"r{i}", prompts[i][done_at[i]:done_at[i] + n], list(range(n))))
        lg = runner.step(entries).float().cpu()
        row = 0
        for e, i in zip(entries, list(live)):
            n = len(e.tokens)
            got[i].append(lg[row:row + n].clone())
            row += n
            done_at[i] += n
            for g in range(len(runner.cache.groups)):
                for p in runner.cache.requests[f"r{i}"].pages[g]:
                    if p >= 0:
                        page_owners.setdefault((g, p), set()).add(i)
        for i in list(live):
            if not plans[i]:
                runner.end_request(f"r{i}")
                live.remove(i)
        runner.cache.check_invariants()
        steps += 1
    runner.check_device_status()
    assert sum(lens) > num_pages * page, "the pool must be too small to hold everything at once"
    assert any(len(o) > 1 for o in page_owners.values()), "no page was held by two requests in turn: nothing was reused"
    for i in range(len(lens)):
        g = torch.cat(got[i])
        bad = first_bad_row(g, refs[i], dtype)
        assert bad is None, f"request {i}: first wrong position {bad}"
        assert_close(g, refs[i], dtype, f"{tag} mixed r{i}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_far_key_and_window_edge_with_sharp_attention(tmp_path, dtype):
    """q_norm weights scaled up make the softmax peaky, so that a single wrong
    or missing key (a far one, one at the window's edge, one on a page edge)
    moves the logits far beyond the tolerance."""
    for tag, n in (("B", 250), ("C", 300), ("D", 400), ("E", 330)):
        runner, cfg, w, page = make_runner(tmp_path, tag, dtype, num_pages=-(-n // ALL_PAGE(tag)) + 1, sharpen=SHARPEN[dtype])
        ids = random_ids(cfg["vocab_size"], n, 31)
        ref = plain_logits(ids, w, cfg)
        got = run_cut(runner, "a", ids, [n - 40, 3, 5] + [1] * 32)
        bad = first_bad_row(got, ref, dtype)
        assert bad is None, f"{tag}: first wrong position {bad}"
        assert_close(got, ref, dtype, f"{tag} sharp")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(tmp_path, dtype):
    runner, cfg, w, page = make_runner(tmp_path, "B", dtype, num_pages=4)
    for n in (1, 2, 3):
        ids = random_ids(cfg["vocab_size"], n, 40 + n)
        ref = plain_logits(ids, w, cfg)
        got = run_cut(runner, f"s{n}", ids, [1] * n)
        assert_close(got, ref, dtype, f"first {n}")


@pytest.mark.needs_cuda
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tmp_path, dtype):
    """bin/trace_run as a user runs it: steps on stdin, <step>.f32 files out."""
    cfg, w, page = weights_for("B", dtype)
    d = write_model_dir(str(tmp_path / "m"), cfg, w)
    out = tmp_path / "out"
    a = random_ids(cfg["vocab_size"], 70, 51)
    b = random_ids(cfg["vocab_size"], 40, 52)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[30:32], "want": []}, {"id": "b", "tokens": b[:40], "want": [39]}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": a[32:69], "want": [36]}], "end": []},
        {"step": 3, "entries": [{"id": "a", "tokens": a[69:70], "want": [0]}], "end": ["a"]},
    ]
    p = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", str(out),
         "--max-tokens", "192"],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    ra, rb = plain_logits(a, w, cfg), plain_logits(b, w, cfg)
    V = cfg["vocab_size"]

    def read(i):
        return torch.frombuffer(bytearray((out / f"{i}.f32").read_bytes()), dtype=torch.float32).view(-1, V)

    assert_close(read(0), ra[[0, 29]], dtype, "step 0")
    assert_close(read(1), rb[[39]], dtype, "step 1")
    assert_close(read(2), ra[[68]], dtype, "step 2")
    assert_close(read(3), ra[[69]], dtype, "step 3")


@pytest.mark.needs_cuda
def test_bf16_engine_uses_the_tensor_core_attention_kernels(tmp_path):
    """With head sizes 64 and 128 in bfloat16 the engine's attention goes through the tensor-core kernels:
    the prefill kernel for portions, the split decode kernel for one-token steps."""
    from ullm_b200.csrc import kernels
    from ullm_b200.engine import StepEntry

    for tag in ("D", "E"):
        runner, cfg, w, page = make_runner(tmp_path, tag, "bfloat16", num_pages=8)
        ids = random_ids(cfg["vocab_size"], 40, 3)
        runner.add_request("a")
        runner.step([StepEntry("a", ids[:39], [38])])
        assert kernels().attention_path == ("prefill_tcgen05" if tag == "E" else "prefill")
        runner.step([StepEntry("a", ids[39:], [0])])
        # (ULLM_B200_DECODE_TC=1 sends head size 128 to the tcgen05 decode kernel instead)
        assert kernels().attention_path == ("decode_tcgen05" if kernels().use_tcgen05_decode and tag == "E" else "decode")
        runner, cfg, w, page = make_runner(tmp_path, tag, "float32", num_pages=8)
        runner.add_request("a")
        runner.step([StepEntry("a", ids[:39], [38])])
        assert kernels().attention_path == "generic"


@pytest.mark.needs_cuda
@pytest.mark.parametrize("tag", ["D", "E"])
def test_decode_batches_of_very_unequal_lengths_take_the_balanced_attention_kernel(tmp_path, tag):
    """One request of 300 tokens beside three of about ten: the step says so (`ragged`), the decode attention
    is the kernel that cuts the batch's keys evenly over the warps, and the logits of eight decode steps follow
    the plain implementation for every request (E has a sliding window on its last layer)."""
    from ullm_b200.csrc import kernels
    from ullm_b200.engine import StepEntry

    runner, cfg, w, page = make_runner(tmp_path, tag, "bfloat16", num_pages=40)
    V = cfg["vocab_size"]
    lens = {"long": 300, "s1": 5, "s2": 9, "s3": 14}
    ids = {r: random_ids(V, n + 8, 40 + n) for r, n in lens.items()}
    refs = {r: plain_logits(ids[r], w, cfg) for r in lens}
    for r, n in lens.items():
        runner.add_request(r)
        for at in range(0, n, 64):
            runner.step([StepEntry(r, ids[r][at:min(n, at + 64)], [])])
    for k in range(8):
        ctx_entries = [StepEntry(r, [ids[r][n + k]], [0]) for r, n in lens.items()]
        lg = runner.step(ctx_entries)
        assert kernels().attention_path == ("decode_tcgen05" if kernels().use_tcgen05_decode and tag == "E"
                                            else "decode_balanced")
        for row, (r, n) in enumerate(lens.items()):
            assert_close(lg[row:row + 1].float().cpu(), refs[r][[n + k]], "bfloat16", f"{r}, decode step {k}")
    runner.check_device_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_widths_two_layers(tmp_path, dtype):
    """Two layers at the widths of Qwen3-0.6B (hidden 1024, 16 heads, 8 kv heads, head size 128, 3072
    feed-forward, the 151,936-token vocabulary, tied head): a 48-token prompt, its last 8 tokens one by one."""
    from ullm_b200.engine import ModelRunner

    import plain_model as pm
    from conftest import device

    cfg = {
        "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 1024, "num_attention_heads": 16,
        "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 3072, "vocab_size": 151936,
        "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "attention_bias": False, "tie_word_embeddings": True,
        "max_position_embeddings": 4096, "torch_dtype": "float32",
    }
    w = pm.random_weights(cfg, seed=21, std=0.02, norm_std=0.05)
    if dtype == "bfloat16":
        w = {n: t.to(torch.bfloat16) for n, t in w.items()}
    d = write_model_dir(str(tmp_path / "wide"), cfg, w)
    runner = ModelRunner(d, dtype=dtype, device=device(), page_size=16, num_pages=8, max_requests=2, max_context=128,
                         max_step_tokens=64, poison_cache=True)
    ids = random_ids(cfg["vocab_size"], 48, 9)
    ref = plain_logits(ids, w, cfg)
    got = run_cut(runner, "a", ids, [40] + [1] * 8)
    assert_close(got, ref, dtype, "0.6B widths")


@pytest.mark.needs_cuda
def test_long_context_at_real_widths_prompt_portions_against_decode_steps():
    """Two layers at Qwen3-8B widths (hidden 4096, 32 heads, 8 kv heads, head size 128), bfloat16, random weights
    made on the device, 8,192 tokens of context.  The same history is built twice: request a by prompt portions
    of 2,048 tokens (the tcgen05 attention over pages), request b with its last tokens one by one (the split decode
    attention).  No plain implementation runs at this size: the two paths are compared with each other, at the
    tolerance they each have against the plain implementation."""
    from helpers import TOL, TOL_RMS
    from ullm_b200.engine import ModelRunner, StepEntry

    cfg = {
        "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 4096, "num_attention_heads": 32,
        "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936,
        "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "attention_bias": False, "tie_word_embeddings": False,
        "max_position_embeddings": 16384, "torch_dtype": "bfloat16",
    }
    N = 8192
    r = ModelRunner(config=cfg, dtype="bfloat16", page_size=16, num_pages=2 * (N // 16) + 8, max_requests=2,
                    max_context=N + 16, max_step_tokens=2048, load_format="random", seed=4, poison_cache=True)
    ids = random_ids(cfg["vocab_size"], N + 4, 77)
    r.add_request("a")
    for at in range(0, N, 2048):
        by_portions = r.step([StepEntry("a", ids[at:at + 2048], [2047])]).float().cpu().clone()
    r.add_request("b")
    for at in range(0, N - 2048, 2048):
        r.step([StepEntry("b", ids[at:at + 2048], [])])
    r.step([StepEntry("b", ids[N - 2048:N - 3], [])])
    for k in range(3):
        one_by_one = r.step([StepEntry("b", [ids[N - 3 + k]], [0])]).float().cpu().clone()
    r.check_device_status()
    scale = by_portions.abs().max().item()
    diff = (by_portions - one_by_one).abs()
    assert torch.isfinite(one_by_one).all() and scale > 0
    assert diff.max().item() <= TOL["bfloat16"] * scale, f"max {diff.max().item() / scale:.2e} of scale"
    assert diff.pow(2).mean().sqrt().item() <= TOL_RMS["bfloat16"] * scale
    assert int(by_portions.argmax()) == int(one_by_one.argmax())
    # both requests decode on, side by side: same history, same next token
    lg = r.step([StepEntry("a", [ids[N]], [0]), StepEntry("b", [ids[N]], [0])]).float().cpu()
    assert (lg[0] - lg[1]).abs().max().item() <= TOL["bfloat16"] * scale
    r.check_device_status()
    # at these widths the library's products went through the timed choice of algorithm (portions and decode steps)
    from ullm_b200.csrc import kernels

    if kernels().lt_rows > 0:
        tuned = kernels()._lt_tuned
        assert any(k[0] == 2048 for k in tuned) and any(k[0] <= 2 for k in tuned), sorted(tuned)


@pytest.mark.parametrize("seed", list(range(12)))
def test_random_configurations_follow_the_plain_implementation(tmp_path, seed):
    """Configurations drawn at random from what config.json allows (head sizes in steps of 16 up to 256, any
    number of heads and groups, widths and vocabularies that are no power of two, bias, tied head, windows, eps,
    rotation base, page size): a sequence whole, with its last tokens one by one, and in portions of changing
    size, in both dtypes, against the plain implementation."""
    import random

    import plain_model as pm
    from conftest import device
    from helpers import errors, TOL, TOL_RMS
    from ullm_b200.engine import ModelRunner, StepEntry

    rng = random.Random(1000 + seed)
    D = rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 144, 256])
    Hkv, G = rng.choice([1, 1, 2, 3, 5]), rng.choice([1, 2, 3, 4, 7, 8])
    window = rng.choice([None, None, 24, 50])
    cfg = {"architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": rng.choice([1, 2, 3]),
           "hidden_size": rng.choice([24, 40, 72, 100, 136, 200]), "num_attention_heads": Hkv * G,
           "num_key_value_heads": Hkv, "head_dim": D, "intermediate_size": rng.choice([24, 56, 136, 200, 328]),
           "vocab_size": rng.choice([97, 331, 517, 1000, 1031]), "rope_theta": rng.choice([10000.0, 1e6, 5e5]),
           "rms_norm_eps": rng.choice([1e-6, 1e-5, 3e-6]), "attention_bias": rng.random() < 0.4,
           "tie_word_embeddings": rng.random() < 0.5, "max_position_embeddings": 512, "torch_dtype": "float32"}
    if window is not None:
        cfg.update(use_sliding_window=True, sliding_window=window, max_window_layers=rng.choice([0, 1]))
    page, n = rng.choice([4, 8, 16, 32]), rng.choice([70, 130, 201])
    ids = random_ids(cfg["vocab_size"], n, seed)
    chunks, left = [], n
    while left:
        c = min(rng.choice([2, 3, 7, 16, 33, 5]), left)
        chunks.append(c)
        left -= c
    for dtype in ("float32", "bfloat16"):
        w = pm.random_weights(cfg, seed=seed, std=0.05, norm_std=0.1)
        if dtype == "bfloat16":
            w = {k: v.to(torch.bfloat16) for k, v in w.items()}
        d = write_model_dir(str(tmp_path / f"m{dtype}"), cfg, w)
        r = ModelRunner(d, dtype=dtype, device=device(), page_size=page, num_pages=2 * (-(-n // page)) + 2,
                        max_requests=3, max_context=512, max_step_tokens=64, poison_cache=True)
        ref = plain_logits(ids, w, cfg)
        for name, cuts in (("whole", [n]), ("decode", [n - 9] + [1] * 9), ("portions", chunks)):
            got = run_cut(r, name, ids, cuts)
            mx, rms = errors(got, ref)
            assert mx <= TOL[dtype] and rms <= TOL_RMS[dtype], (
                f"{dtype}, {name}: max {mx:.2e}, rms {rms:.2e} of scale; {cfg}, page {page}")
        r.cache.check_invariants()


@pytest.mark.needs_cuda
@pytest.mark.parametrize("tag", ["D", "E"])
def test_mixed_steps_send_their_decode_rows_to_the_decode_kernel(tmp_path, tag):
    """A step with one-token entries at its head and prompt portions behind them: the first go through the
    decode attention kernel, the rest through the prompt kernel, each with its slice of the per-request arrays;
    every row's logits follow the plain implementation (E has a sliding window on its last layer)."""
    from ullm_b200.csrc import kernels
    from ullm_b200.engine import StepEntry

    runner, cfg, w, page = make_runner(tmp_path, tag, "bfloat16", num_pages=60, max_requests=6)
    V = cfg["vocab_size"]
    lens = {"d0": 70, "d1": 9, "d2": 33, "p0": 50, "p1": 21}
    ids = {r: random_ids(V, n + 6, 700 + n) for r, n in lens.items()}
    refs = {r: plain_logits(ids[r], w, cfg) for r in lens}
    for r in ("d0", "d1", "d2"):
        runner.add_request(r)
        runner.step([StepEntry(r, ids[r][:lens[r]], [])])
    runner.add_request("p0")
    runner.add_request("p1")
    old = kernels().mixed_decode_rows
    kernels().mixed_decode_rows = 2
    try:
        done = {"p0": 0, "p1": 0}
        for k, (n0, n1) in enumerate([(17, 5), (2, 16), (31, 0), (6, 6)]):
            entries = [StepEntry(r, [ids[r][lens[r] + k]], [0]) for r in ("d0", "d1", "d2")]
            for r, n in (("p0", n0), ("p1", n1)):
                if n:
                    entries.append(StepEntry(r, ids[r][done[r]:done[r] + n], list(range(n))))
            lg = runner.step(entries).float().cpu()
            assert kernels().attention_path in ("prefill_tcgen05", "prefill")  # the last kernel of the step
            row = 0
            for e in entries:
                r, n = e.request_id, len(e.tokens)
                at = lens[r] + k if r.startswith("d") else done[r]
                assert_close(lg[row:row + n], refs[r][at:at + n], "bfloat16", f"{r}, step {k}")
                row += n
                if r.startswith("p"):
                    done[r] += n
    finally:
        kernels().mixed_decode_rows = old
    runner.check_device_status()
