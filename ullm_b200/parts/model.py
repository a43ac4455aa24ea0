"""A decoder assembled from a ModelSpec: embedding, blocks run in the order the
schedule gives, final norm, output head.  ullm/models/qwen3.py:228-255 and
:284-286 are the reference's fixed version of this loop.

The model owns no cache and no batch logic: `forward` receives the step's
context and one LayerCache per schedule entry.
"""

from __future__ import annotations

import torch

from ..config.specs import ModelSpec
from ..csrc import kernels
from .base import Part
from .embedding import OutputHead, TokenEmbedding
from .registry import build_block, build_norm


class DecoderModel(Part):
    def __init__(self, spec: ModelSpec, untie_head: bool = False):
        super().__init__()
        spec.validate()
        self.spec = spec
        self.embedding = TokenEmbedding(spec.vocab_size, spec.hidden_size)
        self.blocks = [build_block(ls) for ls in spec.layers]
        self.final_norm = build_norm(spec.final_norm)
        tied = spec.tie_embeddings and not untie_head
        self.head = OutputHead(spec.vocab_size, spec.hidden_size, self.embedding if tied else None)
        self.schedule = list(spec.schedule)
        # one mixer of each group answers `graph_key` for all of its kind
        seen: dict = {}
        for e in self.schedule:
            m = self.blocks[e.layer].mixer
            seen.setdefault(m.graph_key_group(), m)
        self._graph_key_mixers = list(seen.values())
        self.dtype: torch.dtype | None = None
        self.device = None

    def subparts(self):
        s = {self.spec.embedding_name: self.embedding}
        for i, b in enumerate(self.blocks):
            s[self.spec.layer_name.format(i)] = b
        s[self.spec.final_norm_name] = self.final_norm
        s[self.spec.head_name] = self.head
        return s

    # -- what the cache manager needs to know ------------------------------
    def cache_needs(self):
        """Per schedule entry: (CacheNeed | None, StateNeed | None, cache_of)."""
        out = []
        for e in self.schedule:
            m = self.blocks[e.layer].mixer
            out.append((m.cache_need(), m.state_need(), e.cache_of))
        return out

    def graph_key(self, ctx) -> tuple:
        """What of a decode step, beyond its padded size, decides the kernels its mixers launch."""
        return tuple(m.graph_key(ctx) for m in self._graph_key_mixers)

    # -- allocation ---------------------------------------------------------
    def allocate(self, device, dtype: torch.dtype) -> None:
        """Gives every declared parameter a tensor on `device`: matrices and
        biases in `dtype`, norm weights in float32."""
        self.dtype = dtype
        self.device = torch.device(device)

        def make(name, decl):
            dt = torch.float32 if decl.role == "norm" else dtype
            return torch.empty(decl.shape, dtype=dt, device=self.device)

        self.materialize_all(make)

    # -- one step -----------------------------------------------------------
    def forward_hidden(self, ctx, caches):
        """Runs the blocks over the step's tokens.  Returns (y, residual): what the last block left to be added
        (or None) and the residual stream, before the final norm."""
        T = ctx.num_tokens
        x = ctx.workspace.tokens("model.hidden", T, self.spec.hidden_size, self.dtype)
        self.embedding.forward(ctx.token_ids, x, ctx)
        residual = None
        n = len(self.schedule)
        for i, e in enumerate(self.schedule):
            block = self.blocks[e.layer]
            if block.takes_next_norm:
                # the norm that the next block applies first, if that block can start from what this one prepares
                nxt = self.blocks[self.schedule[i + 1].layer] if i + 1 < n else None
                nxt_norm = nxt.mixer_norm if (nxt is not None and nxt.accepts_folded_norm()) else None
                x, residual = block.forward(x, residual, ctx, caches[i], next_norm=nxt_norm)
            else:
                x, residual = block.forward(x, residual, ctx, caches[i])
        ctx.folded_norm = None
        return x, residual

    def forward(self, ctx, caches):
        """Logits [len(ctx.logits_rows), vocab] float32 at the wanted rows."""
        y, residual = self.forward_hidden(ctx, caches)
        R = ctx.num_logits_rows
        if R == 0:
            return None
        K = kernels()
        H = self.spec.hidden_size
        ys = ctx.workspace.requests("head.y", R, H, self.dtype)
        if y is None or residual is None:
            # nothing is pending beside the stream (a block that adds its own output), or there is no stream
            K.gather_rows(y if residual is None else residual, ctx.logits_rows, ys)
            self.final_norm.forward(ys, None, out=ys)
        else:
            rs = ctx.workspace.requests("head.res", R, H, self.dtype)
            K.gather_rows(y, ctx.logits_rows, ys)
            K.gather_rows(residual, ctx.logits_rows, rs)
            self.final_norm.forward(ys, rs, out=ys)
        logits = ctx.workspace.requests("head.logits", R, self.spec.vocab_size, torch.float32)
        self.head.forward(ys, logits)
        return logits
