"""Arrangement of a layer: pre-norm, residual stream.

ullm/models/qwen3.py:160-178: the stream is carried as (x, residual).  The
first block takes residual = x; afterwards each norm is the fused form
"residual <- x + residual (32-bit sum, rounded on store); h = norm(sum)".
"""

from __future__ import annotations

import torch

from ..csrc import kernels
from .base import Block
from .registry import register_block


@register_block("prenorm_residual")
class PreNormResidualBlock(Block):
    def __init__(self, mixer, feed_forward, mixer_norm, feed_forward_norm, names=None):
        super().__init__()
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.mixer_norm = mixer_norm
        self.feed_forward_norm = feed_forward_norm
        n = names or {}
        self.names = {
            "mixer": n.get("mixer", "mixer."),
            "feed_forward": n.get("feed_forward", "feed_forward."),
            "mixer_norm": n.get("mixer_norm", "mixer_norm."),
            "feed_forward_norm": n.get("feed_forward_norm", "feed_forward_norm."),
        }

    def subparts(self):
        return {
            self.names["mixer_norm"]: self.mixer_norm,
            self.names["mixer"]: self.mixer,
            self.names["feed_forward_norm"]: self.feed_forward_norm,
            self.names["feed_forward"]: self.feed_forward,
        }

    def activation_elems(self):
        # the normed rows, and the wider of the two sub-layers (they run one after the other)
        size = getattr(self.mixer_norm, "size", 0)
        return size + max(self.mixer.activation_elems(), self.feed_forward.activation_elems())

    def forward(self, x, residual, ctx, cache):
        """x: the previous sub-layer's output that is still to be added to the stream (the embedding for the
        first block, with residual None; None when nothing is pending).  Returns (feed-forward output or None,
        residual); the caller's next norm adds them."""
        pending = x if x is not None else residual
        T = pending.shape[0]
        h = ctx.workspace.tokens("block.normed", T, pending.shape[1], pending.dtype)
        if residual is None:
            residual = x
            self.mixer_norm.forward(x, None, out=h)
        elif x is None:
            self.mixer_norm.forward(residual, None, out=h)
        else:
            self.mixer_norm.forward(x, residual, out=h)
        fused = self._fusable_tail(T, residual) if ctx.decode_only else None
        if fused is not None:
            # few rows (decode steps): output projection, residual, norm, gated feed-forward and residual in one
            # kernel; the stream then holds everything and nothing is pending
            w_o, norm_w, eps, w_gate_up, w_down, act = fused
            a = self.mixer.forward(h, ctx, cache, project_output=False)
            work = ctx.workspace.tokens("mlp.act", T, w_down.shape[1], residual.dtype)
            kernels().fused_layer_tail(a, residual, work, w_o, w_gate_up, w_down, norm_w, eps, act)
            return None, residual
        chain = self._fusable_chain(T, residual) if ctx.decode_only else None
        if chain is not None:
            # few rows, every product the weight-streaming kernel: the output projection adds the residual itself
            # and leaves r * w and the sums of squares for the norm, the gate / up product applies 1 / rms to its
            # sums, the down projection adds the residual: three kernels, no norm kernel, nothing pending
            K, (w_o, norm_w, eps, w_gate_up, w_down, act) = kernels(), chain
            a = self.mixer.forward(h, ctx, cache, project_output=False)
            H = residual.shape[1]
            sq = ctx.workspace.get("block.norm_sq", 1, K.stream_sq_floats(H), torch.float32)
            work = ctx.workspace.tokens("mlp.act", T, w_down.shape[1], residual.dtype)
            if (K.stream_linear(a, w_o, residual, None, None, residual, norm_behind=(norm_w, h, sq))
                    and K.stream_linear(h, w_gate_up, work, None, act, norm_in_front=(sq, H, eps))
                    and K.stream_linear(work, w_down, residual, None, None, residual)):
                return None, residual
            raise RuntimeError("the chained products were refused after the sizes had been accepted")
        a = self.mixer.forward(h, ctx, cache)
        self.feed_forward_norm.forward(a, residual, out=h)
        y = self.feed_forward.forward(h, ctx)
        return y, residual

    def _fusable_chain(self, rows: int, residual):
        """The same parts as `_fusable_tail` needs, when the step's products are all the stream kernel."""
        if not residual.is_cuda or not kernels().stream_chain_applies(rows, residual.dtype):
            return None
        proj, norm, ffn = self.mixer.output_projection(), self.feed_forward_norm.rms_params(), self.feed_forward.gated_weights()
        if proj is None or norm is None or ffn is None or proj[1] is not None:
            return None
        w_o, (norm_w, eps), (w_gate_up, w_down, act) = proj[0], norm, ffn
        K = kernels()
        H = residual.shape[1]
        if (w_o.dtype != torch.bfloat16 or H % 8 or w_o.shape[1] % 8 or w_down.shape[1] % 8
                or not K.lib.ullm_linear_stream_supported(rows, H, w_o.shape[1])):
            return None
        return w_o, norm_w, eps, w_gate_up, w_down, act

    def _fusable_tail(self, rows: int, residual):
        """What the fused kernel needs, if this block's parts offer it (a mixer that ends in a bias-free linear
        map, an RMSNorm, a bias-free gated feed-forward) and the kernel takes the sizes; else None."""
        proj, norm, ffn = self.mixer.output_projection(), self.feed_forward_norm.rms_params(), self.feed_forward.gated_weights()
        if proj is None or norm is None or ffn is None or proj[1] is not None or not residual.is_cuda:
            return None
        w_o, (norm_w, eps), (w_gate_up, w_down, act) = proj[0], norm, ffn
        if not kernels().layer_tail_applies(rows, residual.dtype, residual.shape[1], w_o.shape[1], w_down.shape[1]):
            return None
        return w_o, norm_w, eps, w_gate_up, w_down, act
