"""Grouped-query attention over a paged cache: qkv projection, optional
per-head q/k norm, position rotation, the write of this step's keys and values
into the pages, attention over the pages, output projection.

ullm/models/qwen3.py:113-130 gives the order (projection, q/k norm per head
over head_dim with one weight shared by all heads, rotation, attention, output
projection); ullm/models/qwen3.py:81 the scale; query head h reads kv head
h // (num_heads / num_kv_heads).  The three projections are one matrix with
rows q | k | v, as ullm/layers/linear.py:381-389 lays them out; the checkpoint's
q_proj / k_proj / v_proj tensors are row ranges of it.
"""

from __future__ import annotations

from ..csrc import check_attention_sizes, kernels
from .base import CacheNeed, Mixer, ParamDecl
from .linear import linear
from .registry import build_norm, build_position_encoding, register_mixer


def is_ragged(batch: int, max_kv: int, sum_kv: int) -> bool:
    """A decode batch whose longest request, times the batch, is more than 1.5 times all the keys there are:
    splitting every request alike would then leave most blocks waiting for the long one (measured: the
    batch-balanced attention kernel wins from about this ratio on, and loses about 5 % on even batches)."""
    return batch > 1 and 2 * batch * max_kv > 3 * sum_kv


@register_mixer("paged_attention")
class PagedAttention(Mixer):
    def __init__(
        self,
        hidden_size: int,
        num_heads: int,
        num_kv_heads: int,
        head_dim: int,
        qkv_bias: bool = False,
        qk_norm=None,
        position=None,
        window: int | None = None,
        scale: float | None = None,
    ):
        super().__init__()
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads={num_heads} is no multiple of num_kv_heads={num_kv_heads}")
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.qkv_bias = qkv_bias
        self.window = window
        self.scale = head_dim ** -0.5 if scale is None else scale
        self.q_size = num_heads * head_dim
        self.kv_size = num_kv_heads * head_dim
        self.q_norm = build_norm(qk_norm) if qk_norm is not None else None
        self.k_norm = build_norm(qk_norm) if qk_norm is not None else None
        self.position = build_position_encoding(position) if position is not None else None
        check_attention_sizes(num_heads, num_kv_heads, head_dim, self.position.rotary_dim if self.position else 0)

    # -- parameters -------------------------------------------------------
    def param_decls(self):
        H = self.hidden_size
        d = {
            "q_proj.weight": ParamDecl((self.q_size, H)),
            "k_proj.weight": ParamDecl((self.kv_size, H)),
            "v_proj.weight": ParamDecl((self.kv_size, H)),
            "o_proj.weight": ParamDecl((H, self.q_size)),
        }
        if self.qkv_bias:
            d["q_proj.bias"] = ParamDecl((self.q_size,), "bias")
            d["k_proj.bias"] = ParamDecl((self.kv_size,), "bias")
            d["v_proj.bias"] = ParamDecl((self.kv_size,), "bias")
        return d

    def subparts(self):
        s = {}
        if self.q_norm is not None:
            s["q_norm."] = self.q_norm
            s["k_norm."] = self.k_norm
        return s

    def materialize(self, make):
        H, q, kv = self.hidden_size, self.q_size, self.kv_size
        self.w_qkv = make("qkv_proj.weight", ParamDecl((q + 2 * kv, H)))
        self.tensors["q_proj.weight"] = self.w_qkv[:q]
        self.tensors["k_proj.weight"] = self.w_qkv[q:q + kv]
        self.tensors["v_proj.weight"] = self.w_qkv[q + kv:]
        self.tensors["o_proj.weight"] = make("o_proj.weight", ParamDecl((H, q)))
        self.b_qkv = None
        if self.qkv_bias:
            self.b_qkv = make("qkv_proj.bias", ParamDecl((q + 2 * kv,), "bias"))
            self.tensors["q_proj.bias"] = self.b_qkv[:q]
            self.tensors["k_proj.bias"] = self.b_qkv[q:q + kv]
            self.tensors["v_proj.bias"] = self.b_qkv[q + kv:]
        if self.position is not None:
            self.position.build_tables(self.w_qkv.device)

    # -- cache ------------------------------------------------------------
    def cache_need(self):
        return CacheNeed(self.num_kv_heads, self.head_dim, self.window)

    def activation_elems(self):
        # qkv, the attention's output, the projected output
        return self.q_size + 2 * self.kv_size + self.q_size + self.hidden_size

    # -- which kernels a decode step takes ---------------------------------
    def graph_key(self, ctx):
        return ("ragged",) if self._ragged(ctx) else ()

    def graph_key_group(self):
        return (type(self), self.num_heads, self.num_kv_heads, self.head_dim)

    @staticmethod
    def _ragged(ctx) -> bool:
        return bool(ctx.decode_only and is_ragged(ctx.num_live_requests, ctx.max_kv_len, ctx.sum_kv_len))

    def output_projection(self):
        return self.tensors["o_proj.weight"], None

    def takes_input_norm(self):
        return True

    # -- one step ---------------------------------------------------------
    def forward(self, x, ctx, cache, project_output: bool = True, input_norm=None):
        K = kernels()
        T = x.shape[0]
        ragged = self._ragged(ctx)
        qkv = ctx.workspace.tokens("attn.qkv", T, self.q_size + 2 * self.kv_size, x.dtype)
        if input_norm is not None:
            # x is r * w: the projection multiplies its sums by the rows' 1 / rms (a norm folded in front of it)
            if not K.stream_linear(x, self.w_qkv, qkv, self.b_qkv, norm_in_front=input_norm):
                raise RuntimeError("the projection with a folded norm was refused")
        else:
            linear(x, self.w_qkv, qkv, self.b_qkv)
        g = cache.group
        tables = self.position.tables() if self.position is not None else {}
        q_w = self.q_norm.tensors["weight"] if self.q_norm is not None else None
        k_w = self.k_norm.tensors["weight"] if self.k_norm is not None else None
        eps = self.q_norm.eps if self.q_norm is not None else 0.0
        rotary_dim = self.position.rotary_dim if self.position is not None else 0
        slot_mapping = g.slot_mapping if cache.writes else None
        fuse = None
        if self.position is not None and self.position.transforms_qk():
            # an encoding with code of its own: norm q and k, let it change them, then store the keys and values
            if q_w is not None or k_w is not None:
                K.qk_norm_in_place(qkv, self.num_heads, self.num_kv_heads, self.head_dim, q_w, k_w, eps)
            self.position.apply(qkv[:, :self.q_size].view(T, self.num_heads, self.head_dim),
                                qkv[:, self.q_size:self.q_size + self.kv_size].view(T, self.num_kv_heads, self.head_dim),
                                ctx.positions)
            if slot_mapping is not None:
                K.qk_norm_rope_store(qkv, self.num_heads, self.num_kv_heads, self.head_dim, None, None, 0.0, None, None, 0,
                                     ctx.positions, slot_mapping, cache.k_pages, cache.v_pages)
        elif K.decode_fusion_applies(ctx, qkv, self.num_heads, self.num_kv_heads, self.head_dim, g.page_size, rotary_dim,
                                     tables.get("cos"), ragged):
            # a decode step: the attention kernel norms and rotates q and k and writes k and v to their pages itself
            fuse = dict(q_w=q_w, k_w=k_w, eps=eps, cos=tables["cos"], sin=tables["sin"], positions=ctx.positions,
                        slot_mapping=slot_mapping)
        else:
            K.qk_norm_rope_store(
                qkv, self.num_heads, self.num_kv_heads, self.head_dim, q_w, k_w, eps, tables.get("cos"),
                tables.get("sin"), rotary_dim, ctx.positions, slot_mapping, cache.k_pages, cache.v_pages,
            )
        attn = ctx.workspace.tokens("attn.out", T, self.q_size, x.dtype)
        K.paged_attention(
            qkv, attn, cache.k_pages, cache.v_pages, g.block_table, g.req_slots, ctx.cu_q, g.kv_len,
            ctx.token_req,
            self.num_heads, self.num_kv_heads, self.head_dim, g.page_size,
            self.window or 0, self.scale, ctx, ragged=ragged, **({"fuse": fuse} if fuse is not None else {}),
        )
        if not project_output:
            return attn  # (the caller multiplies by `output_projection()` itself)
        out = ctx.workspace.tokens("mixer.out", T, self.hidden_size, x.dtype)
        linear(attn, self.tensors["o_proj.weight"], out)
        return out
