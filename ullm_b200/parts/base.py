"""What every part is: an object built from sizes and constants alone, that
declares its parameters by name, receives tensors for them, and runs on a flat
batch of tokens.  No part knows which model it is in.

Interfaces (what a new part must have):

* every part: `param_decls() -> {name: ParamDecl}` and
  `materialize(make) -> None`, where `make(name, decl)` returns the tensor for a
  declared parameter; the part keeps what it needs and lists the tensors under
  their checkpoint names in `self.tensors`.
* Norm: `forward(x, residual=None, out=None) -> out`; with a residual the sum
  x + residual is formed in 32-bit, written back to `residual`, and normed.
* PositionEncoding: `tables() -> dict of device tensors` handed to the mixer's
  kernel, plus `rotary_dim`; or `transforms_qk() -> True` and `apply(q, k,
  positions)` for an encoding that is no rotation by tables.
* Mixer: `cache_need() -> CacheNeed | None`, `state_need() -> StateNeed | None`,
  `graph_key(ctx)` (what of a decode step changes its launches, default nothing),
  `forward(x[T, hidden], ctx, cache) -> [T, hidden]`; `cache` is the
  LayerCache of this execution (pages of its group + the group's step
  metadata, and its state rows if it asked for any).
* FeedForward: `forward(x[T, hidden], ctx) -> [T, hidden]`.
* Block: `forward(x, residual, ctx, cache) -> (x, residual)`.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch


@dataclass(frozen=True)
class ParamDecl:
    """A parameter as the checkpoint stores it.  `role` decides precision and
    random init: "matrix" (embedding and linear weights: engine dtype, N(0,
    std)), "bias" (engine dtype, N(0, std)), "norm" (always held in 32-bit,
    1 + N(0, norm_std))."""

    shape: tuple[int, ...]
    role: str = "matrix"


@dataclass(frozen=True)
class CacheNeed:
    """Keys and values this mixer keeps per token: `num_kv_heads` x `head_dim`
    for K and for V.  `window`: None keeps every token, w keeps the last w."""

    num_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size: one row of `shape` per live request."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


Maker = Callable[[str, ParamDecl], torch.Tensor]


class Part:
    def __init__(self) -> None:
        self.tensors: dict[str, torch.Tensor] = {}

    def param_decls(self) -> dict[str, ParamDecl]:
        return {}

    def materialize(self, make: Maker) -> None:
        for name, decl in self.param_decls().items():
            self.tensors[name] = make(name, decl)

    def subparts(self) -> dict[str, "Part"]:
        """Nested parts by tensor-name prefix."""
        return {}

    def activation_elems(self) -> int:
        """Elements per token that this part (with its sub-parts) keeps in the step's workspace while it
        runs; the engine sets that much memory aside before it sizes the cache pool.  A part that takes
        buffers from `ctx.workspace` says here how wide they are together."""
        return sum(p.activation_elems() for p in self.subparts().values())

    # -- walking a tree of parts ------------------------------------------
    def all_decls(self, prefix: str = "") -> dict[str, ParamDecl]:
        out = {prefix + n: d for n, d in self.param_decls().items()}
        for sub_prefix, sub in self.subparts().items():
            out.update(sub.all_decls(prefix + sub_prefix))
        return out

    def materialize_all(self, make: Maker, prefix: str = "") -> None:
        self.materialize(lambda n, d: make(prefix + n, d))
        for sub_prefix, sub in self.subparts().items():
            sub.materialize_all(make, prefix + sub_prefix)

    def all_tensors(self, prefix: str = "") -> dict[str, torch.Tensor]:
        out = {prefix + n: t for n, t in self.tensors.items()}
        for sub_prefix, sub in self.subparts().items():
            out.update(sub.all_tensors(prefix + sub_prefix))
        return out


class Norm(Part):
    def forward(self, x, residual=None, out=None):
        raise NotImplementedError

    def rms_params(self):
        """(weight, eps) if this norm is a plain RMSNorm over the whole row, which a block may then fold into a
        fused kernel; None otherwise."""
        return None


class PositionEncoding(Part):
    """Two kinds.  A rotation by per-position tables hands `tables()` (`cos` / `sin` rows of `rotary_dim / 2`
    floats per position) to the mixer's kernels, which rotate in 32-bit registers.  Any other encoding that acts
    on queries and keys answers True from `transforms_qk()` and does its work in `apply`, with device code of
    its own; the mixer then norms q and k first and stores the keys afterwards.  (An encoding that biases the
    SCORES by both positions would need an argument of the attention kernels; there is none yet.)"""

    rotary_dim: int = 0

    def build_tables(self, device) -> None:
        """Called once, when the mixer's parameters exist: put what the encoding needs on `device`."""

    def tables(self) -> dict[str, torch.Tensor]:
        return {}

    def transforms_qk(self) -> bool:
        return False

    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> None:
        """Changes this step's queries q [T, heads, head_dim] and keys k [T, kv heads, head_dim] in place
        (views of the projection's output); positions [T] int32 on the device."""
        raise NotImplementedError


class Mixer(Part):
    def cache_need(self) -> CacheNeed | None:
        return None

    def state_need(self) -> StateNeed | None:
        return None

    def graph_key(self, ctx):
        """What about a decode step, beyond its padded batch size, changes the kernels this mixer launches or
        their grids (a mixer that picks a kernel by how unequal the requests' lengths are, say).  A recorded
        CUDA graph is replayed only for steps with the same key.  Hashable; () when nothing does."""
        return ()

    def graph_key_group(self):
        """Mixers with equal groups give equal graph keys for the same step (one of them is asked)."""
        return type(self)

    def takes_input_norm(self) -> bool:
        """True when `forward(..., input_norm=(sq, cols, eps))` is understood: x is then r * w (the norm weight
        already applied) and the mixer's first product multiplies its sums by the rows' 1 / rms, computed from the
        sums of squares `sq` (see `Kernels.stream_linear`).  Only asked for in small decode steps."""
        return False

    def output_projection(self):
        """(weight [hidden, width], bias or None) if the mixer ends in a plain linear map and can also stop in
        front of it (`forward(..., project_output=False)` then returns its [T, width] input); None otherwise.
        A block may fold that product into a fused kernel."""
        return None

    def forward(self, x, ctx, cache):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x, ctx):
        raise NotImplementedError

    def gated_weights(self):
        """(w_gate_up [2 I, hidden], w_down [hidden, I], activation code) if this is a bias-free gated
        feed-forward down(act(gate(x)) * up(x)) that a block may fold into a fused kernel; None otherwise."""
        return None


class Block(Part):
    takes_next_norm = False  # True: `forward` has a `next_norm=` argument (see PreNormResidualBlock)

    def accepts_folded_norm(self) -> bool:
        return False

    def forward(self, x, residual, ctx, cache):
        raise NotImplementedError
