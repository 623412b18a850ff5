"""Sequence mixers.  ``gqa_attention``: causal grouped-query attention over the cache.

Order of operations (src/l5_model.c:497-583 of AnonymoDGH/gguf2bin): q, k, v projections
without bias; per-head RMSNorm of q and k (if the spec has ``qk_norm``); position
encoding of q and k; k (normed, rotated) and v (raw) written to the cache; scores
(q . k) * scale over the keys up to the token's own position (optionally only the last
``window`` of them); softmax; weighted values; output projection added to the residual.

With ``shared_kv`` the mixer has no k and v projections and writes nothing: it attends
over the keys and values that another layer stored (the schedule entry's ``cache_of``
names that layer, whose kv heads and head size it must share).

Further options, each a parameter of the spec and off by default:
``bias``: q, k and v are W h + b (names ``q_bias``, ``k_bias``, ``v_bias``);
``qk_norm_span`` = "projection": the RMS norm of q (and of k) runs over the WHOLE projection, all
heads at once, with a weight of that size, before the heads are split;
``v_dim``: a value head size other than the key head size (pages hold both at the larger size,
zero-filled);
``chunk``: a token sees only the keys of its own chunk of that many positions, counted from
position 0 of the sequence;
``sink`` = "zero": one more term exp(0) in the softmax's denominator, with no value;
``out_gate`` = "sigmoid": the concatenated heads times sigmoid(W_g h), element by element (name
``gate``), before the output projection;
``out_scale``: the mixer's result times a constant (applied to the gated heads in 32-bit);
``v_norm_eps``: every value head is divided by its root mean square (that eps inside the root, no
weight) before it is stored;
``pool`` (with a window): beside the window's tokens a query at position i sees one key and one value
for every block of ``pool`` positions that lies wholly before the window (block b, positions
b pool .. b pool + pool - 1, if b pool + pool - 1 <= i - window): the means of the block's keys and
values as the pages hold them, in the same softmax.  Tokens that have left the window and whose
block is not complete behind it are not seen.  The means are a second store beside the pages
(``KVNeed.rows``: a page keeps the blocks that start in it), written by the token that ends a block.
The first, second, third, sixth and the value norm take the prologue kernel that knows them
(``proj_norm_rope_cache``); its rotation is either pair layout of the position part.
"""
from __future__ import annotations

import math

import torch

from .. import kernels
from ..cache.storage import KVNeed, KVView
from ..config.specs import ConfigError, PartSpec
from ..weights.loader import Expected
from .fused import normed_linear
from .registry import norm_class, position_class, register_mixer


class GQAAttention:
    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device):
        self.nh = int(spec["n_heads"])
        self.nkv = int(spec["n_kv_heads"])
        self.hd = int(spec["head_dim"])
        self.hidden = int(hidden_size)
        self.window = int(spec.get("window") or 0)
        self.shared_kv = bool(spec.get("shared_kv") or False)
        scale = spec.get("scale")
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.hd)
        if self.nh <= 0 or self.nkv <= 0 or self.nh % self.nkv:
            raise ConfigError(f"gqa_attention: {self.nh} heads are not a multiple of "
                              f"{self.nkv} kv heads")
        if self.hd <= 0 or self.hd > 512:
            raise ConfigError(f"gqa_attention: head_dim {self.hd} outside 1..512")
        self.dtype, self.device = dtype, device
        self.names = dict(spec["names"])
        qk = spec.get("qk_norm")
        self.qk_eps = 0.0
        self.has_qk_norm = qk is not None
        if qk is not None:
            if qk.kind != "rmsnorm":
                raise ConfigError(f"gqa_attention: qk_norm of kind {qk.kind!r} is not supported")
            norm_class(qk)                            # must be registered
            self.qk_eps = float(qk["eps"])
        pos = spec.get("position") or PartSpec.make("none")
        self.position = position_class(pos)(pos, self.hd, device)
        self.w_qkv = self.w_o = self.q_norm_w = self.k_norm_w = None
        self.vd = int(spec.get("v_dim") or self.hd)
        self.has_bias = bool(spec.get("bias") or False)
        self.norm_span = spec.get("qk_norm_span") or "head"
        self.chunk = int(spec.get("chunk") or 0)
        self.out_gate = spec.get("out_gate")
        self.out_scale = float(spec.get("out_scale") if spec.get("out_scale") is not None else 1.0)
        sink = spec.get("sink")
        if self.norm_span not in ("head", "projection") or self.out_gate not in (None, "sigmoid") \
                or sink not in (None, "zero"):
            raise ConfigError("gqa_attention: qk_norm_span is 'head' or 'projection', out_gate None or "
                              "'sigmoid', sink None or 'zero'")
        if self.chunk < 0 or (self.chunk and self.window):
            raise ConfigError("gqa_attention: a chunk and a window exclude each other")
        self.v_norm_eps = float(spec.get("v_norm_eps") or 0.0)
        self.pool = int(spec.get("pool") or 0)
        if self.pool < 0 or (self.pool and (self.window <= 0 or sink is not None or self.out_gate)):
            raise ConfigError("gqa_attention: pooled blocks need a window and go with neither a sink nor a gate")
        self.sink = torch.zeros(self.nh, dtype=torch.float32, device=device) if sink == "zero" else None
        self.bias = None
        # the prologue that knows biases, a norm over the whole projection, unequal head sizes and
        # a gate's columns beside q, k and v
        self.wide = bool(self.has_bias or self.vd != self.hd or self.out_gate or self.v_norm_eps or self.pool
                         or getattr(self.position, "mult", 1.0) != 1.0
                         or (self.has_qk_norm and self.norm_span == "projection"))
        if self.wide:
            if self.shared_kv or (self.has_qk_norm and self.norm_span == "head"):
                raise ConfigError("gqa_attention: biases, a norm over the projection, a value size of its own "
                                  "and an output gate go with neither shared_kv nor a per-head norm")
            if not hasattr(self.position, "table_rotation"):
                raise ConfigError("gqa_attention: this position part offers no table rotation")
        self.cache_hd = max(self.hd, self.vd)

    # ---- weights -------------------------------------------------------------
    @classmethod
    def expected(cls, spec: PartSpec, hidden_size: int) -> dict:
        n = dict(spec["names"])
        vd = int(spec.get("v_dim") or spec["head_dim"])
        nq, nk = spec["n_heads"] * spec["head_dim"], spec["n_kv_heads"] * spec["head_dim"]
        nv, no = spec["n_kv_heads"] * vd, spec["n_heads"] * vd
        shared = bool(spec.get("shared_kv") or False)
        out = {n["q"]: Expected((nq, hidden_size)), n["o"]: Expected((hidden_size, no))}
        if not shared:
            out[n["k"]] = Expected((nk, hidden_size))
            out[n["v"]] = Expected((nv, hidden_size))
        if spec.get("qk_norm") is not None:
            whole = spec.get("qk_norm_span") == "projection"
            out[n["q_norm"]] = Expected((nq if whole else spec["head_dim"],), init="scale")
            if not shared:
                out[n["k_norm"]] = Expected((nk if whole else spec["head_dim"],), init="scale")
        if spec.get("bias"):
            out[n["q_bias"]], out[n["k_bias"]], out[n["v_bias"]] = Expected((nq,)), Expected((nk,)), Expected((nv,))
        if spec.get("out_gate"):
            out[n["gate"]] = Expected((no, hidden_size))
        return out

    def bind(self, tensors: dict) -> None:
        n = self.names
        parts = [tensors[n["q"]]] if self.shared_kv else \
            [tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]]
        if self.out_gate:
            parts.append(tensors[n["gate"]])          # reads the same input: one product
        if self.has_bias:
            self.bias = torch.cat([tensors[n[k]].to(torch.float32) for k in ("q_bias", "k_bias", "v_bias")]).contiguous()
        common = torch.float32 if any(p.dtype == torch.float32 for p in parts) else parts[0].dtype
        self.w_qkv = torch.cat([p.to(common) for p in parts], dim=0).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        if self.has_qk_norm:
            self.q_norm_w = tensors[n["q_norm"]].to(torch.float32).contiguous()
            if not self.shared_kv:
                self.k_norm_w = tensors[n["k_norm"]].to(torch.float32).contiguous()

    def weights(self):
        return [t for t in (self.w_qkv, self.w_o, self.q_norm_w, self.k_norm_w, self.bias) if t is not None]

    def absorb_norm_weight(self, norm) -> bool:
        """Takes the weight of the norm in front of this mixer into the columns of the q/k/v
        matrix, when that is what makes the decode step shorter: bfloat16 compute and a
        bfloat16 matrix (the product then normalises its own rows, see ``parts/fused.py``).
        The matrix is rounded to bfloat16 once more; the 32-bit path keeps the formula's order."""
        if self.dtype != torch.bfloat16 or self.w_qkv.dtype != torch.bfloat16 or not hasattr(norm, "give_up_weight"):
            return False
        w = norm.give_up_weight()
        self.w_qkv = (self.w_qkv.float() * w.to(self.w_qkv.device)[None, :]).to(torch.bfloat16).contiguous()
        return True

    def notices(self) -> list:
        from ..cache.storage import PAGE_SIZE
        return (kernels.product_notices("attention q/k/v", self.w_qkv, self.dtype)
                + kernels.product_notices("attention output", self.w_o, self.dtype)
                + kernels.attention_notices("attention", self.cache_hd, PAGE_SIZE, self.dtype))

    @property
    def graph_safe(self) -> bool:
        """Its own step only launches kernels; whether the whole of it may be replayed from a
        CUDA graph is then up to its position part."""
        return bool(getattr(self.position, "graph_safe", False))

    # ---- cache ---------------------------------------------------------------
    def cache_need(self):
        if self.shared_kv:
            return None
        need = KVNeed(self.nkv, self.cache_hd, self.window)
        if not self.pool:
            return need
        from ..cache.storage import PAGE_SIZE
        return {"kv": need, "pool": KVNeed(self.nkv, self.cache_hd, 0, rows=-(-PAGE_SIZE // self.pool))}

    # ---- step ----------------------------------------------------------------
    def forward(self, h: torch.Tensor, ctx, view: KVView, residual32: torch.Tensor) -> None:
        qkv = ctx.workspace.buffer("attn.qkv", (h.shape[0], self.w_qkv.shape[0]), self.dtype)
        kernels.linear(h, self.w_qkv, qkv)
        self._attend(qkv, ctx, view, residual32)

    def forward_store(self, h: torch.Tensor, ctx, view: KVView, out32: torch.Tensor) -> None:
        """Stores the result instead of adding it."""
        qkv = ctx.workspace.buffer("attn.qkv", (h.shape[0], self.w_qkv.shape[0]), self.dtype)
        kernels.linear(h, self.w_qkv, qkv)
        self._attend(qkv, ctx, view, out32, accumulate=False)

    def forward_from_stream(self, x32: torch.Tensor, norm, ctx, view: KVView,
                            residual32: torch.Tensor) -> None:
        """The same with the block's norm folded into the q/k/v product."""
        qkv = ctx.workspace.buffer("attn.qkv", (x32.shape[0], self.w_qkv.shape[0]), self.dtype)
        normed_linear(x32, norm, self.w_qkv, qkv, ctx)
        self._attend(qkv, ctx, view, residual32)

    def _attend_wide(self, qkv: torch.Tensor, ctx, view: KVView, residual32: torch.Tensor, accumulate: bool = True) -> None:
        """q, k, v (and the gate's columns) of one product; the prologue adds the biases, norms all
        of q and all of k, rotates and writes the pages; attention; gate; output product."""
        T, ws = qkv.shape[0], ctx.workspace
        hd, no = self.cache_hd, self.nh * self.vd
        pooled = None
        if self.pool:
            view, pooled = view["kv"], view["pool"].pages
        inv_freq, rot, interleaved = self.position.table_rotation()
        rope = ctx.rope_table(inv_freq, getattr(self.position, "mult", 1.0)) if inv_freq is not None else None
        q = ws.buffer("attn.q", (T, self.nh * hd), self.dtype)
        kernels.proj_norm_rope_cache(qkv, self.bias, self.nh, self.nkv, self.hd, self.vd, self.q_norm_w,
                                     self.k_norm_w, self.qk_eps, rope, rot, interleaved, ctx, view.pages,
                                     view.page_size, q, v_norm_eps=self.v_norm_eps)
        if self.pool:
            kernels.pool_update(view.pages, pooled, ctx, self.nkv, hd, view.page_size, self.pool)
        o = ws.buffer("attn.o", (T, self.nh * hd), self.dtype)
        kernels.attention(q, o, view.pages, ctx, self.nh, self.nkv, hd, view.page_size, self.window,
                          self.scale, sink=self.sink, chunk=self.chunk, pooled=pooled, pool=self.pool)
        if self.out_gate or hd != self.vd or self.out_scale != 1.0:
            gate = qkv[:, qkv.shape[1] - no:] if self.out_gate else None
            og = ws.buffer("attn.gated", (T, no), self.dtype)
            kernels.gate_mul(o, hd, gate, self.nh, self.vd, self.out_scale, og)
            o = og
        kernels.linear(o, self.w_o, residual32, accumulate=accumulate)

    def _attend(self, qkv: torch.Tensor, ctx, view: KVView, residual32: torch.Tensor, accumulate: bool = True) -> None:
        if self.wide:
            return self._attend_wide(qkv, ctx, view, residual32, accumulate)
        T = qkv.shape[0]
        nq = self.nh * self.hd
        nkv_own = 0 if self.shared_kv else self.nkv        # kv heads this layer projects
        nk = nkv_own * self.hd
        ws = ctx.workspace
        q = ws.buffer("attn.q", (T, nq), self.dtype)
        fused = self.position.fused_rotation()
        if fused is not None:
            inv_freq, rot = fused
            rope = ctx.rope_table(inv_freq) if inv_freq is not None else None
            kernels.qknorm_rope_cache(qkv, self.nh, nkv_own, self.hd, self.q_norm_w,
                                      self.k_norm_w, self.qk_eps, rope, rot, ctx.tok_pos,
                                      ctx.tok_seq, ctx.page_table, view.pages, view.page_size, q)
        else:
            k = ws.buffer("attn.k", (T, nk), self.dtype)
            v = ws.buffer("attn.v", (T, nk), self.dtype)
            kernels.qknorm_rope_cache(qkv, self.nh, nkv_own, self.hd, self.q_norm_w,
                                      self.k_norm_w, self.qk_eps, None, 0, ctx.tok_pos,
                                      ctx.tok_seq, None, None, view.page_size, q, k, v)
            self.position.apply(q, k, ctx)
            if nkv_own:
                kernels.cache_write(k, v, self.nkv, self.hd, ctx.tok_pos, ctx.tok_seq,
                                    ctx.page_table, view.pages, view.page_size)
        o = ws.buffer("attn.o", (T, nq), self.dtype)
        kernels.attention(q, o, view.pages, ctx, self.nh, self.nkv, self.hd, view.page_size,
                          self.window, self.scale, sink=self.sink, chunk=self.chunk)
        if self.out_scale != 1.0:
            og = ws.buffer("attn.gated", (T, nq), self.dtype)
            kernels.gate_mul(o, self.hd, None, self.nh, self.hd, self.out_scale, og)
            o = og
        kernels.linear(o, self.w_o, residual32, accumulate=accumulate)


register_mixer("gqa_attention", GQAAttention)
