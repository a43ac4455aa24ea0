"""RMSNorm, alone or fused with the residual sum.

ullm/layers/layernorm.py:20-34: everything in 32-bit; with a residual the sum
x + residual is normed unrounded and its rounded value becomes the new
residual; the weight multiplies before the cast back.
"""

from __future__ import annotations

from ..csrc import kernels
from .base import Norm, ParamDecl
from .registry import register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, size: int, eps: float):
        super().__init__()
        self.size = size
        self.eps = eps

    def param_decls(self):
        return {"weight": ParamDecl((self.size,), "norm")}

    def rms_params(self):
        return self.tensors["weight"], self.eps

    def forward(self, x, residual=None, out=None):
        """x [T, size].  residual (same shape), if given, is updated in place
        to x + residual.  Returns the normed rows (in `out` if given; `out`
        may be `x`)."""
        if out is None:
            out = x
        kernels().add_rmsnorm(x, residual, self.tensors["weight"], self.eps, out)
        return out
