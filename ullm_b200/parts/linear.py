"""y = x W^T (+ b), weight [out, in] as the checkpoint stores it
(ullm/layers/linear.py:165).  The product itself is the vendor library's
matrix product, as in the reference; in float32 it runs without any
reduced-precision mode."""

from __future__ import annotations

from ..csrc import kernels


def linear(x, weight, out, bias=None):
    return kernels().linear(x, weight, out, bias)
