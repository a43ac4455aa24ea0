"""Token embedding (row gather, ullm/layers/vocab_parallel_embedding.py:117)
and the output head (ullm/layers/vocab_parallel_embedding.py:159-161).  No
vocabulary padding is kept: the kernels and the matrix product take any
vocabulary size.  A tied head reads the embedding table."""

from __future__ import annotations

from ..csrc import kernels
from .base import ParamDecl, Part


class TokenEmbedding(Part):
    def __init__(self, vocab_size: int, hidden_size: int):
        super().__init__()
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size

    def param_decls(self):
        return {"weight": ParamDecl((self.vocab_size, self.hidden_size))}

    def forward(self, token_ids, out, ctx=None):
        """An id of -1 stands for the token its request sampled last, when the step's context carries the
        device array that holds those (`ctx.last_tokens`)."""
        if ctx is not None and ctx.last_tokens is not None:
            kernels().embedding(token_ids, self.tensors["weight"], out, ctx.last_tokens, ctx.token_req, ctx.req_slots)
        else:
            kernels().embedding(token_ids, self.tensors["weight"], out)
        return out


class OutputHead(Part):
    """logits = h W^T in 32-bit output.  `tied_to`, when set, is the embedding
    part whose table is read and no tensor of its own is declared."""

    def __init__(self, vocab_size: int, hidden_size: int, tied_to: TokenEmbedding | None = None):
        super().__init__()
        self.vocab_size = vocab_size
        self.hidden_size = hidden_size
        self.tied_to = tied_to

    def param_decls(self):
        if self.tied_to is not None:
            return {}
        return {"weight": ParamDecl((self.vocab_size, self.hidden_size))}

    def weight(self):
        return self.tied_to.tensors["weight"] if self.tied_to is not None else self.tensors["weight"]

    def forward(self, h, out_f32):
        kernels().linear_f32_out(h, self.weight(), out_f32)
        return out_f32
