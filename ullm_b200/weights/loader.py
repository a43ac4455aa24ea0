"""Weights by tensor name.

ullm/models/qwen3.py:300-336 walks the file's (name, tensor) pairs, maps
q_proj/k_proj/v_proj and gate_proj/up_proj into fused matrices and silently
skips names it does not know, and never notices a missing tensor.  Here the
model lists its tensors under the checkpoint's own names (fused matrices expose
their row ranges under the unfused names), the loader compares that list with
the files once, and raises ONE error naming every missing tensor, every
unexpected tensor and every wrong shape before anything is copied.

Precision: matrices and biases are kept in the engine's dtype (bfloat16 for
serving, float32 for the 32-bit path); norm weights are always kept in float32,
so a tensor the file stores in 32-bit stays so where the arithmetic is 32-bit.
Integer tensors, if a model declares any, are kept as int32.
"""

from __future__ import annotations

import torch

from .safetensors_io import open_model_files


class WeightError(ValueError):
    def __init__(self, missing, unexpected, wrong_shape, where: str):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        lines = [f"weights in {where} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n}: file {tuple(a)} != model {tuple(b)}" for n, a, b in self.wrong_shape))
        super().__init__("\n".join(lines))


def files_have(model_dir: str, name: str) -> bool:
    files = open_model_files(model_dir)
    try:
        return any(name in f.entries for f in files)
    finally:
        for f in files:
            f.close()


def load_weights(model, model_dir: str, progress=None) -> dict[str, str]:
    """Copies every tensor of the folder's *.safetensors into `model` (already
    allocated).  Returns {name: dtype in file}."""
    files = open_model_files(model_dir)
    try:
        where: dict[str, object] = {}
        for f in files:
            for n in f.names():
                where[n] = f
        targets = model.all_tensors()
        missing = [n for n in targets if n not in where]
        unexpected = [n for n in where if n not in targets]
        wrong = [(n, where[n].shape(n), tuple(targets[n].shape))
                 for n in targets if n in where and tuple(where[n].shape(n)) != tuple(targets[n].shape)]
        if missing or unexpected or wrong:
            raise WeightError(missing, unexpected, wrong, model_dir)
        seen = {}
        for i, (n, dst) in enumerate(targets.items()):
            src = where[n].get(n)
            seen[n] = str(src.dtype)
            if dst.dtype in (torch.int32, torch.int64):
                dst.copy_(src.to(torch.int32) if dst.dtype == torch.int32 else src)
            else:
                dst.copy_(src)  # converts on the way; float32 -> bfloat16 rounds to nearest even
            if progress is not None:
                progress(i + 1, len(targets), n)
        return seen
    finally:
        for f in files:
            f.close()
