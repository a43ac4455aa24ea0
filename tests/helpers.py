"""Shared helpers of the tests: model folders made from the tiny configurations
(always in a temporary folder), runners, error measures, fixed tolerances."""

from __future__ import annotations

import json
import os

import torch

import plain_model as pm
from tiny_configs import ALL

# Largest allowed |engine - plain| relative to the largest |plain| logit of the
# compared block.  float32: both sides are 32-bit, only the order of additions
# differs.  bfloat16: weights are identical (rounded before both sides see
# them); activations are rounded to 8 bits of mantissa after every kernel.
# float16 keeps 11 bits where bfloat16 keeps 8: an eighth of its limits.
TOL = {"float32": 1e-4, "bfloat16": 4e-2, "float16": 5e-3}
TOL_RMS = {"float32": 2e-5, "bfloat16": 1e-2, "float16": 1.25e-3}
# How much the tests that sharpen attention scale q_norm: enough that one wrong
# key shows, little enough that bfloat16 rounding of q and k stays inside TOL.
SHARPEN = {"float32": 6.0, "bfloat16": 2.0, "float16": 3.0}


def weights_for(tag: str, dtype: str, sharpen: float = 1.0):
    cfg, init, page = ALL[tag]
    w = pm.random_weights(cfg, **init)
    if sharpen != 1.0:
        for n in w:
            if n.endswith("q_norm.weight"):
                w[n] = w[n] * sharpen
    if dtype in ("bfloat16", "float16"):
        w = {n: t.to(getattr(torch, dtype)) for n, t in w.items()}
    return cfg, w, page


def write_model_dir(path: str, cfg: dict, w: dict) -> str:
    from ullm_b200.weights import save_tensors

    os.makedirs(path, exist_ok=True)
    c = dict(cfg)
    c["torch_dtype"] = str(next(iter(w.values())).dtype).replace("torch.", "")
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(c, f)
    save_tensors(os.path.join(path, "model.safetensors"), w)
    return path


def plain_logits(ids, w, cfg, schedule=None):
    wf = {n: t.float() for n, t in w.items()}
    return pm.forward_logits(ids, wf, cfg, schedule)


def errors(got: torch.Tensor, ref: torch.Tensor) -> tuple[float, float]:
    """(max abs error, rms error), both relative to the largest |ref|."""
    got = got.detach().float().cpu()
    scale = max(ref.abs().max().item(), 1e-6)
    d = (got - ref).abs()
    return d.max().item() / scale, d.pow(2).mean().sqrt().item() / scale


def assert_close(got, ref, dtype: str, what: str = ""):
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} != {tuple(ref.shape)}"
    assert torch.isfinite(got.float()).all(), f"{what}: non-finite logits"
    mx, rms = errors(got, ref)
    assert mx <= TOL[dtype] and rms <= TOL_RMS[dtype], (
        f"{what}: max err {mx:.3e} (limit {TOL[dtype]:.0e}), rms {rms:.3e} (limit {TOL_RMS[dtype]:.0e}) of scale")


def first_bad_row(got, ref, dtype: str):
    got = got.detach().float().cpu()
    scale = max(ref.abs().max().item(), 1e-6)
    per_row = (got - ref).abs().max(dim=-1).values / scale
    bad = (per_row > TOL[dtype]).nonzero()
    return None if bad.numel() == 0 else int(bad[0])


def random_ids(vocab: int, n: int, seed: int) -> list[int]:
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()
