"""Random weights from a configuration and a seed.

Two ways, same distribution (matrices and biases N(0, std), norm weights
1 + N(0, norm_std)):

* `write_random_model` writes a model folder (config.json, model.safetensors)
  on the host.  Each tensor has a generator of its own, seeded from the seed
  and the tensor's name, so the values do not depend on the order of tensors or
  on which other tensors exist.
* `fill_random_` fills an allocated model in place on its device (used by
  benchmarks, where writing tens of GB to disk first would be pointless).

The reference has no such mode (ullm/model_loader.py loads files only).
"""

from __future__ import annotations

import hashlib
import json
import os

import torch

from ..config.registry import load_model_spec
from .safetensors_io import write_safetensors

_TORCH = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def random_tensor(seed: int, name: str, decl, std: float, norm_std: float, dtype: torch.dtype) -> torch.Tensor:
    g = torch.Generator().manual_seed(_tensor_seed(seed, name))
    t = torch.randn(decl.shape, generator=g, dtype=torch.float32)
    if decl.role == "norm":
        t = 1.0 + t * norm_std
    else:
        t = t * std
    return t.to(dtype)


def write_random_model(
    out_dir: str,
    config: dict,
    seed: int = 0,
    std: float = 0.02,
    norm_std: float = 0.0,
    dtype: str | None = None,
) -> str:
    """Writes `out_dir`/config.json and `out_dir`/model.safetensors.  `config`
    holds the architecture's own config.json keys; `dtype` (default: the
    config's) is the dtype the tensors are stored in."""
    from ..parts.model import DecoderModel

    cfg, spec = load_model_spec(config)
    store = _TORCH[dtype or spec.dtype]
    model = DecoderModel(spec)
    decls = model.all_decls()
    os.makedirs(out_dir, exist_ok=True)
    cfg_out = dict(config)
    cfg_out["torch_dtype"] = dtype or spec.dtype
    cfg_out.pop("dtype", None)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg_out, f, indent=1)
    listing = [(n, store, tuple(d.shape)) for n, d in decls.items()]

    def gen():
        for n, d in decls.items():
            yield n, random_tensor(seed, n, d, std, norm_std, store)

    write_safetensors(os.path.join(out_dir, "model.safetensors"), listing, gen(),
                      metadata={"format": "pt", "seed": str(seed)})
    return out_dir


def fill_random_(model, seed: int = 0, std: float = 0.02, norm_std: float = 0.0) -> None:
    """Fills an allocated model on its device.  Generator per tensor, seeded
    from (seed, name); values differ from `write_random_model`'s (another
    generator), the distribution is the same."""
    decls = model.all_decls()
    tensors = model.all_tensors()
    for n, d in decls.items():
        t = tensors[n]
        g = torch.Generator(device=t.device).manual_seed(_tensor_seed(seed, n))
        if t.is_contiguous():
            t.normal_(0.0, 1.0, generator=g)
            if d.role == "norm":
                t.mul_(norm_std).add_(1.0)
            else:
                t.mul_(std)
        else:
            tmp = torch.empty(t.shape, dtype=t.dtype, device=t.device).normal_(0.0, 1.0, generator=g)
            t.copy_(1.0 + tmp * norm_std if d.role == "norm" else tmp * std)
