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

    takes_next_norm = True  # `forward` accepts the norm that the next block (or nobody) will apply first

    def accepts_folded_norm(self) -> bool:
        """True when this block can start from an operand r * w and the rows' sums of squares that the block
        before left (instead of norming r itself): an RMSNorm in front of a mixer whose first step is a product."""
        return self.mixer_norm.rms_params() is not None and self.mixer.takes_input_norm()

    def forward(self, x, residual, ctx, cache, next_norm=None):
        """x: the previous sub-layer's output that is still to be added to the stream (the embedding for the
        first block, with residual None; None when nothing is pending).  Returns (feed-forward output or None,
        residual); the caller's next norm adds them.  `next_norm`: the norm the next block will apply to the
        stream first, if that block `accepts_folded_norm()`; in small decode steps this block's last product then
        prepares it (`ctx.folded_norm`), and the next block's mixer starts from that."""
        pending = x if x is not None else residual
        T = pending.shape[0]
        folded, ctx.folded_norm = getattr(ctx, "folded_norm", None), None
        input_norm = None
        fused = chain = None
        if ctx.decode_only and residual is not None:
            fused = self._fusable_tail(T, residual)
            chain = self._fusable_chain(T, residual) if fused is None else None
        if (folded is not None and folded[0] is self.mixer_norm and x is None and residual is not None
                and chain is not None):
            # the block before left r * w and the sums of squares: the mixer's first product applies 1 / rms
            _norm, h, sq, eps = folded
            input_norm = (sq, residual.shape[1], eps)
        else:
            h = ctx.workspace.tokens("block.normed", T, pending.shape[1], pending.dtype)
            if residual is None:
                residual = x
                self.mixer_norm.forward(x, None, out=h)
            elif x is None:
                self.mixer_norm.forward(residual, None, out=h)
            else:
                self.mixer_norm.forward(x, residual, out=h)
        if fused is None and chain is None and ctx.decode_only:
            fused = self._fusable_tail(T, residual)  # the first block: the stream has only now got its rows
            chain = self._fusable_chain(T, residual) if fused is None else None
        if fused is not None:
            # few rows (decode steps): output projection, residual, norm, gated feed-forward and residual in one
            # kernel; the stream then holds everything and nothing is pending
            w_o, norm_w, eps, w_gate_up, w_down, act = fused
            a = self.mixer.forward(h, ctx, cache, project_output=False)
            work = ctx.workspace.tokens("mlp.act", T, w_down.shape[1], residual.dtype)
            kernels().fused_layer_tail(a, residual, work, w_o, w_gate_up, w_down, norm_w, eps, act)
            return None, residual
        if chain is not None:
            # few rows, every product the weight-streaming kernel: the output projection adds the residual itself
            # and leaves r * w and the sums of squares for the norm, the gate / up product applies 1 / rms to its
            # sums, the down projection adds the residual (and prepares the next block's norm the same way):
            # three kernels, no norm kernel, nothing pending
            K, (w_o, norm_w, eps, w_gate_up, w_down, act) = kernels(), chain
            if input_norm is not None:
                a = self.mixer.forward(h, ctx, cache, project_output=False, input_norm=input_norm)
            else:
                a = self.mixer.forward(h, ctx, cache, project_output=False)
            H = residual.shape[1]
            hn = ctx.workspace.tokens("block.normed", T, H, residual.dtype)
            sq = ctx.workspace.get("block.norm_sq", 1, K.stream_sq_floats(H), torch.float32)
            work = ctx.workspace.tokens("mlp.act", T, w_down.shape[1], residual.dtype)
            behind = None
            nxt = next_norm.rms_params() if next_norm is not None else None
            if nxt is not None and nxt[0].numel() == H and K.chain_norms >= 2:
                operand = ctx.workspace.tokens("block.next_operand", T, H, residual.dtype)
                sq2 = ctx.workspace.get("block.next_sq", 1, K.stream_sq_floats(H), torch.float32)
                behind = (nxt[0], operand, sq2)
            if (K.stream_linear(a, w_o, residual, None, None, residual, norm_behind=(norm_w, hn, sq))
                    and K.stream_linear(hn, w_gate_up, work, None, act, norm_in_front=(sq, H, eps))
                    and K.stream_linear(work, w_down, residual, None, None, residual, norm_behind=behind)):
                if behind is not None:
                    ctx.folded_norm = (next_norm, behind[1], behind[2], nxt[1])
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
