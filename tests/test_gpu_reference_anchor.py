"""The attention core anchored on the reference itself, run on the GPU.

tests/golden/ pins the plain implementation on izmttk/ullm's model code run on the CPU, but there the attention
core (which query head reads which kv head, the causal mask) is a stand-in written for that script: the
reference's own is a GPU library call.  Here the reference runs whole, on the GPU, through its public API, in a
process of its own (tests/reference_greedy.py), on a random model with 16 query heads over 4 kv heads (a group
of 4, so a wrong head mapping shows) and an untied head; its greedy tokens are then checked, teacher-forced,
against the plain implementation's logits and against this engine's.  Skipped when baseline/_ref is absent.
"""

import json
import os
import subprocess
import sys

import pytest
import torch

import plain_model as pm
from conftest import ROOT, device
from helpers import TOL, random_ids, write_model_dir

pytestmark = [pytest.mark.gpu, pytest.mark.needs_cuda]

CFG = {
    "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 2, "hidden_size": 1024, "num_attention_heads": 16,
    "num_key_value_heads": 4, "head_dim": 128, "intermediate_size": 3072, "vocab_size": 151936,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "attention_bias": False, "tie_word_embeddings": False,
    "max_position_embeddings": 4096, "torch_dtype": "bfloat16",
}
NEW_TOKENS = 16


def _ids_from_strings(strings, vocab):
    """Token strings back to ids through the synthetic vocabulary; stops at the first string that is not one
    entry of it (a byte the tokenizer could not show, the end-of-sequence token shown as nothing)."""
    ids = []
    for s in strings:
        if s not in vocab:
            break
        ids.append(vocab[s])
    return ids


def _within_tolerance(logits_row, tok, scale) -> bool:
    return logits_row.max().item() - logits_row[tok].item() <= 2 * TOL["bfloat16"] * scale


def test_reference_greedy_tokens_follow_plain_and_engine_logits(tmp_path):
    if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "ullm", "core")):
        pytest.skip("izmttk/ullm is not installed under baseline/_ref")
    from bench import write_synthetic_tokenizer
    from ullm_b200.engine import ModelRunner, StepEntry

    w = pm.random_weights(CFG, seed=41, std=0.03, norm_std=0.1)
    w = {n: t.to(torch.bfloat16) for n, t in w.items()}
    d = write_model_dir(str(tmp_path / "anchor"), CFG, w)
    write_synthetic_tokenizer(d, CFG["vocab_size"])
    with open(os.path.join(d, "vocab.json")) as f:
        vocab = json.load(f)
    prompts = [random_ids(CFG["vocab_size"], n, 900 + n) for n in (5, 23, 64)]
    pfile = str(tmp_path / "prompts.json")
    with open(pfile, "w") as f:
        json.dump(prompts, f)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "reference_greedy.py"), d, pfile, str(NEW_TOKENS)],
                       capture_output=True, text=True, timeout=900, cwd=str(tmp_path))
    lines = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")]
    if r.returncode != 0 or not lines:
        pytest.skip(f"the reference did not run here (rc {r.returncode}): {r.stderr[-400:]}")
    strings = json.loads(lines[-1][len("RESULT "):])
    ref_tokens = [_ids_from_strings(s, vocab) for s in strings]
    assert sum(len(t) for t in ref_tokens) >= 2 * NEW_TOKENS, f"too few tokens could be mapped back: {strings}"

    wf = {n: t.float() for n, t in w.items()}
    # the same weights with the kv heads in reverse order: what a wrong head mapping would compute
    Hkv, D = CFG["num_key_value_heads"], CFG["head_dim"]
    wrong = dict(wf)
    for n in wf:
        if n.endswith(("k_proj.weight", "v_proj.weight")):
            wrong[n] = wf[n].view(Hkv, D, -1).flip(0).reshape(Hkv * D, -1)
    runner = ModelRunner(d, dtype="bfloat16", device=device(), page_size=16, num_pages=16, max_requests=1,
                         max_context=256, max_step_tokens=128, poison_cache=True)
    wrong_caught = 0
    for p, toks in zip(prompts, ref_tokens):
        if not toks:
            continue
        seq = p + toks
        plain = pm.forward_logits(seq, wf, CFG)
        scale = plain.abs().max().item()
        runner.add_request("r")
        got = runner.step([StepEntry("r", seq[:-1], list(range(len(p) - 1, len(seq) - 1)))]).float().cpu()
        runner.end_request("r")
        bad = pm.forward_logits(seq, wrong, CFG)
        for i, tok in enumerate(toks):
            assert _within_tolerance(plain[len(p) - 1 + i], tok, scale), (
                f"prompt of {len(p)}: the reference's token {i} ({tok}) is not the plain implementation's choice")
            assert _within_tolerance(got[i], tok, scale), (
                f"prompt of {len(p)}: the reference's token {i} ({tok}) is not this engine's choice")
            wrong_caught += not _within_tolerance(bad[len(p) - 1 + i], tok, scale)
    runner.check_device_status()
    assert wrong_caught > 0, "the check cannot tell a wrong head mapping from the right one"
