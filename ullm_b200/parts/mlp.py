"""Gated feed-forward: down(act(gate(x)) * up(x)), gate and up as one matrix
with rows gate | up (ullm/models/qwen3.py:23-46, ullm/layers/linear.py:490-491,
ullm/layers/activation.py:16-18)."""

from __future__ import annotations

from ..csrc import kernels
from .base import FeedForward, ParamDecl
from .linear import linear
from .registry import register_feed_forward

_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "silu"):
        super().__init__()
        if activation not in _ACTIVATIONS:
            raise ValueError(f"activation {activation!r} unknown (have {sorted(_ACTIVATIONS)})")
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.activation = activation

    def param_decls(self):
        H, I = self.hidden_size, self.intermediate_size
        return {
            "gate_proj.weight": ParamDecl((I, H)),
            "up_proj.weight": ParamDecl((I, H)),
            "down_proj.weight": ParamDecl((H, I)),
        }

    def materialize(self, make):
        H, I = self.hidden_size, self.intermediate_size
        self.w_gate_up = make("gate_up_proj.weight", ParamDecl((2 * I, H)))
        self.tensors["gate_proj.weight"] = self.w_gate_up[:I]
        self.tensors["up_proj.weight"] = self.w_gate_up[I:]
        self.tensors["down_proj.weight"] = make("down_proj.weight", ParamDecl((H, I)))

    def gated_weights(self):
        return self.w_gate_up, self.tensors["down_proj.weight"], _ACTIVATIONS[self.activation]

    def activation_elems(self):
        return 3 * self.intermediate_size + self.hidden_size  # gate | up, their product, the output

    def forward(self, x, ctx):
        T = x.shape[0]
        I = self.intermediate_size
        gu = ctx.workspace.tokens("mlp.gate_up", T, 2 * I, x.dtype)
        act = ctx.workspace.tokens("mlp.act", T, I, x.dtype)
        kernels().linear_act_mul(x, self.w_gate_up, act, gu, _ACTIVATIONS[self.activation])
        out = ctx.workspace.tokens("ffn.out", T, self.hidden_size, x.dtype)
        linear(act, self.tensors["down_proj.weight"], out)
        return out
