"""The two ends of a model: token ids into the residual stream, and the residual stream
into logits.

``token_embedding``: row ``id`` of the table, widened to float32
(src/l5_model.c:488-492 of AnonymoDGH/gguf2bin), times ``scale`` when the spec has one.
``lm_head``: logits = h . W^T in float32, W a matrix of its own or, when ``tied``, the
embedding's table (src/l5_model.c:600-605: without an output tensor the reference
multiplies by the token-embedding matrix).

Another architecture's ends (a scaled embedding, a logit scale or cap, a bias) are other
kinds of these two families; the model only walks parts.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from ..config.specs import ConfigError, PartSpec
from ..weights.loader import Expected
from .registry import register_embedding, register_head


class TokenEmbedding:
    graph_safe = True          # its step only launches kernels: may be replayed from a CUDA graph

    def __init__(self, spec: PartSpec, vocab_size: int, hidden_size: int, dtype: torch.dtype, device):
        self.name = spec["name"]
        self.vocab, self.hidden = int(vocab_size), int(hidden_size)
        self.scale = float(spec.get("scale") if spec.get("scale") is not None else 1.0)
        self.table: Optional[torch.Tensor] = None      # [vocab, hidden]; a tied head multiplies by it

    @classmethod
    def expected(cls, spec: PartSpec, vocab_size: int, hidden_size: int) -> dict:
        return {spec["name"]: Expected((int(vocab_size), int(hidden_size)))}

    def bind(self, tensors: dict) -> None:
        self.table = tensors[self.name].contiguous()

    def weights(self):
        return (self.table,)

    def forward(self, tok_ids: torch.Tensor, out32: torch.Tensor, ctx) -> None:
        """out32[t] = table[tok_ids[t]] * scale as float32; out32 is [T, hidden]."""
        kernels.embed_rows(self.table, tok_ids, out32, self.scale)


class LMHead:
    graph_safe = True

    def __init__(self, spec: PartSpec, vocab_size: int, hidden_size: int, dtype: torch.dtype, device):
        self.name = spec["name"]
        self.tied = bool(spec.get("tied") or False)
        self.vocab, self.hidden = int(vocab_size), int(hidden_size)
        self.dtype = dtype
        self.matrix: Optional[torch.Tensor] = None

    @classmethod
    def expected(cls, spec: PartSpec, vocab_size: int, hidden_size: int) -> dict:
        # beside tied embeddings a checkpoint may or may not carry the (equal) matrix
        return {spec["name"]: Expected((int(vocab_size), int(hidden_size)),
                                       optional=bool(spec.get("tied") or False))}

    def bind(self, tensors: dict, embedding) -> None:
        if self.tied:
            table = getattr(embedding, "table", None)
            if table is None or tuple(table.shape) != (self.vocab, self.hidden):
                raise ConfigError("lm_head: tied, but the embedding part offers no table of "
                                  f"[{self.vocab}, {self.hidden}]")
            self.matrix = table
        else:
            self.matrix = tensors[self.name].contiguous()

    def weights(self):
        return (self.matrix,)

    def notices(self) -> list:
        return kernels.product_notices("lm_head", self.matrix, self.dtype)

    def forward(self, h: torch.Tensor, logits32: torch.Tensor, ctx) -> None:
        """logits32 [n, vocab] float32 = h [n, hidden] . matrix^T."""
        kernels.linear(h, self.matrix, logits32)


class PairEmbedding:
    """``pair_embedding``: x_t = table[id_t] * scale + pairs[row_t], then an RMS norm with a weight.
    row_t = (id_{t-1} * mul_prev + id_t * mul_cur) mod buckets: a second, hashed table addressed by
    the previous and the current token; a sequence's first token takes the row behind the
    buckets (``pairs`` has ``buckets + 1`` rows).  The previous token of a step's first token is
    the embedding's own state: two places per slot, indexed by position parity."""
    graph_safe = True

    def __init__(self, spec: PartSpec, vocab_size: int, hidden_size: int, dtype: torch.dtype, device):
        self.name, self.pair_name, self.norm_name = spec["name"], spec["pair_name"], spec["norm_name"]
        self.vocab, self.hidden = int(vocab_size), int(hidden_size)
        self.scale, self.eps = float(spec["scale"]), float(spec["eps"])
        self.buckets = int(spec["buckets"])
        self.mul_prev, self.mul_cur = int(spec["mul_prev"]), int(spec["mul_cur"])
        if self.buckets <= 0:
            raise ConfigError("pair_embedding: buckets must be positive")
        self.table: Optional[torch.Tensor] = None
        self.pairs = self.norm_w = None

    @classmethod
    def expected(cls, spec: PartSpec, vocab_size: int, hidden_size: int) -> dict:
        return {spec["name"]: Expected((int(vocab_size), int(hidden_size))),
                spec["pair_name"]: Expected((int(spec["buckets"]) + 1, int(hidden_size))),
                spec["norm_name"]: Expected((int(hidden_size),), init="scale")}

    def bind(self, tensors: dict) -> None:
        self.table = tensors[self.name].contiguous()
        self.pairs = tensors[self.pair_name].to(self.table.dtype).contiguous()
        self.norm_w = tensors[self.norm_name].to(torch.float32).contiguous()

    def weights(self):
        return (self.table, self.pairs, self.norm_w)

    def cache_need(self):
        from ..cache.storage import StateNeed
        return StateNeed((2,), torch.int32, by_position=True)

    def forward(self, tok_ids: torch.Tensor, out32: torch.Tensor, ctx, view) -> None:
        kernels.embed_pair_norm(self.table, self.pairs, tok_ids, ctx, view.states, self.norm_w, self.eps,
                                self.scale, self.buckets, self.mul_prev, self.mul_cur, out32)


register_embedding("token_embedding", TokenEmbedding)
register_embedding("pair_embedding", PairEmbedding)
register_head("lm_head", LMHead)
