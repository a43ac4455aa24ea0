"""The CUDA kernels (sm_100a) and their loader.

`kernels()` returns the one Kernels object of the process, compiling the
library on first use if no up-to-date build is found.  Tests that exercise the
host-side logic without a GPU install a stand-in with `set_kernels`.
"""

from __future__ import annotations

_KERNELS = None


def kernels():
    global _KERNELS
    if _KERNELS is None:
        from .ops import Kernels

        _KERNELS = Kernels()
    return _KERNELS


def set_kernels(obj) -> None:
    """Replaces the process-wide kernel object (None: load the real one on next use)."""
    global _KERNELS
    _KERNELS = obj


def check_attention_sizes(num_heads: int, num_kv_heads: int, head_dim: int, rotary_dim: int) -> None:
    from .ops import check_attention_sizes as f

    f(num_heads, num_kv_heads, head_dim, rotary_dim)
