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
``softcap``: a score s becomes softcap * tanh(s / softcap) after the scale;
``sink`` = "learned": the term in the denominator is exp(sink_h), one stored number per head (name ``sink``),
used as it is (neither scaled nor capped);
``keep_first`` (with a window): the keys at positions below it stay visible behind the window, at their
true positions;
``qk_unit_eps``: AFTER the rotation every head of q and of k is divided by its root mean square (that eps
inside the root, no weight);
``out_gate`` = "head_sigmoid": every head's output times sigmoid(W_g h)_h, one number per head (name ``gate``,
[heads, hidden]);
``one_pass_prologue``: norm, rotation and page writes in the one kernel below even where the narrower
kernels would do (a rotation of neighbouring pairs then costs one launch instead of four).
The first, second, third, sixth, the value norm, the unit norm and the gates take the prologue kernel that
knows them (``proj_norm_rope_cache``); its rotation is either pair layout of the position part, its norm
spans the projection or a head, and with ``shared_kv`` it prepares q alone.

``diff_attention``: two score maps per head over ONE set of values.  q has heads * 2 * head_dim rows and k
kv_heads * 2 * head_dim, head by head as [map 1, map 2]; every map is normed (per head and map, one weight of
head_dim shared by all), rotated, masked and softmaxed like an attention of its own; with a1, a2 the maps'
outputs, o = a1 - lambda a2 with lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff (four stored vectors of
head_dim, one number for the layer), then o / sqrt(mean(o^2) + eps) over the head's values, times (1 - diff),
and the output product.  It runs as 2 * heads query heads on 2 * kv_heads key heads whose value head is the
key head modulo kv_heads (the rows of W_q and W_k are put map by map when bound), so every attention
kernel option above applies to it.
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
        if self.norm_span not in ("head", "projection") or self.out_gate not in (None, "sigmoid", "head_sigmoid") \
                or sink not in (None, "zero", "learned"):
            raise ConfigError("gqa_attention: qk_norm_span is 'head' or 'projection', out_gate None, 'sigmoid' or "
                              "'head_sigmoid', sink None, 'zero' or 'learned'")
        self.softcap = float(spec.get("softcap") or 0.0)
        self.keep_first = int(spec.get("keep_first") or 0)
        self.unit_eps = float(spec.get("qk_unit_eps") or 0.0)
        self.learned_sink = sink == "learned"
        self.n_v_heads = self.nkv                      # value heads (fewer than key heads in ``diff_attention``)
        if self.softcap < 0 or self.keep_first < 0 or self.unit_eps < 0 or (self.keep_first and self.window <= 0):
            raise ConfigError("gqa_attention: softcap and qk_unit_eps are positive or absent; keep_first needs a window")
        if self.chunk < 0 or (self.chunk and self.window):
            raise ConfigError("gqa_attention: a chunk and a window exclude each other")
        self.v_norm_eps = float(spec.get("v_norm_eps") or 0.0)
        self.pool = int(spec.get("pool") or 0)
        if self.pool < 0 or (self.pool and (self.window <= 0 or sink is not None or self.out_gate)):
            raise ConfigError("gqa_attention: pooled blocks need a window and go with neither a sink nor a gate")
        if self.pool and (self.keep_first or self.softcap):
            raise ConfigError("gqa_attention: pooled blocks go with neither kept first tokens nor capped scores")
        self.sink = torch.zeros(self.nh, dtype=torch.float32, device=device) if sink == "zero" else None
        self.bias = None
        # the prologue that knows biases, a norm over the whole projection, unequal head sizes and
        # a gate's columns beside q, k and v
        self.wide = bool(self.has_bias or self.vd != self.hd or self.out_gate or self.v_norm_eps or self.pool
                         or getattr(self.position, "mult", 1.0) != 1.0 or self.unit_eps
                         or spec.get("one_pass_prologue")
                         or (self.has_qk_norm and self.norm_span == "projection"))
        if self.wide:
            if self.shared_kv and (self.has_bias or self.pool or self.v_norm_eps):
                raise ConfigError("gqa_attention: biases, pooled blocks and a value norm do not go with shared_kv")
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
            out[n["gate"]] = Expected((spec["n_heads"] if spec["out_gate"] == "head_sigmoid" else no, hidden_size))
        if spec.get("sink") == "learned":
            out[n["sink"]] = Expected((spec["n_heads"],))
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
        pad = -sum(p.shape[0] for p in parts) % 8 if self.wide else 0
        if pad:                                       # an output row then starts on 16 bytes in bfloat16
            parts.append(torch.zeros((pad, self.hidden), dtype=common, device=parts[0].device))
        self.w_qkv = torch.cat([p.to(common) for p in parts], dim=0).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        if self.learned_sink:
            self.sink = tensors[n["sink"]].to(torch.float32).contiguous()
        if self.has_qk_norm:
            self.q_norm_w = tensors[n["q_norm"]].to(torch.float32).contiguous()
            if not self.shared_kv:
                self.k_norm_w = tensors[n["k_norm"]].to(torch.float32).contiguous()

    def weights(self):
        return [t for t in (self.w_qkv, self.w_o, self.q_norm_w, self.k_norm_w, self.bias, self.sink) if t is not None]

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
        """q, k, v (and the gate's columns) of one product; the prologue adds the biases, norms q and k
        (all of each, or head by head), rotates, may divide every head by its root mean square, and writes
        the pages; attention; gate; output product."""
        T, ws = qkv.shape[0], ctx.workspace
        hd = self.cache_hd
        pooled = None
        if self.pool:
            view, pooled = view["kv"], view["pool"].pages
        nkv_own = 0 if self.shared_kv else self.nkv           # key and value heads this layer projects
        nv_own = 0 if self.shared_kv else self.n_v_heads
        inv_freq, rot, interleaved = self.position.table_rotation()
        rope = ctx.rope_table(inv_freq, getattr(self.position, "mult", 1.0)) if inv_freq is not None else None
        q = ws.buffer("attn.q", (T, self.nh * hd), self.dtype)
        kernels.proj_norm_rope_cache(qkv, self.bias, self.nh, nkv_own, self.hd, self.vd, self.q_norm_w,
                                     self.k_norm_w, self.qk_eps, rope, rot, interleaved, ctx,
                                     view.pages if nkv_own else None, view.page_size, q, v_norm_eps=self.v_norm_eps,
                                     norm_per_head=self.has_qk_norm and self.norm_span == "head",
                                     unit_eps=self.unit_eps, n_v_heads=nv_own)
        if self.pool:
            kernels.pool_update(view.pages, pooled, ctx, self.nkv, hd, view.page_size, self.pool)
        gate_at = self.nh * self.hd + nkv_own * self.hd + nv_own * self.vd       # the gate's first column
        head_gate = qkv[:, gate_at:gate_at + self.nh] if self.out_gate == "head_sigmoid" else None
        o = ws.buffer("attn.o", (T, self.nh * hd), self.dtype)
        kernels.attention(q, o, view.pages, ctx, self.nh, self.nkv, hd, view.page_size, self.window,
                          self.scale, sink=self.sink, gate=head_gate, chunk=self.chunk, pooled=pooled, pool=self.pool,
                          softcap=self.softcap, keep_first=self.keep_first,
                          v_heads=self.n_v_heads if self.n_v_heads != self.nkv else 0)
        self._project_out(o, qkv, gate_at, ctx, residual32, accumulate)

    def _project_out(self, o, qkv, gate_at: int, ctx, residual32, accumulate: bool) -> None:
        """What lies between the attention's output (heads padded to the pages' head size) and the stream."""
        T, hd, no = o.shape[0], self.cache_hd, self.nh * self.vd
        if self.out_gate == "sigmoid" or hd != self.vd or self.out_scale != 1.0:
            gate = qkv[:, gate_at:gate_at + no] if self.out_gate == "sigmoid" else None
            og = ctx.workspace.buffer("attn.gated", (T, no), self.dtype)
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
                          self.window, self.scale, sink=self.sink, chunk=self.chunk, softcap=self.softcap,
                          keep_first=self.keep_first)
        if self.out_scale != 1.0:
            og = ws.buffer("attn.gated", (T, nq), self.dtype)
            kernels.gate_mul(o, self.hd, None, self.nh, self.hd, self.out_scale, og)
            o = og
        kernels.linear(o, self.w_o, residual32, accumulate=accumulate)


class DiffAttention(GQAAttention):
    """Two score maps per head over one set of values, the second subtracted (see the module's text)."""

    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device):
        self.H, self.G = int(spec["n_heads"]), int(spec["n_kv_heads"])
        params = spec.as_dict()
        params.update(n_heads=2 * self.H, n_kv_heads=2 * self.G, one_pass_prologue=True)
        if spec.get("shared_kv") or spec.get("out_gate") or spec.get("pool"):
            raise ConfigError("diff_attention: neither shared_kv nor an output gate nor pooled blocks")
        super().__init__(PartSpec.make("gqa_attention", **params), hidden_size, dtype, device)
        self.n_v_heads = self.G
        self.diff = float(spec["diff"])
        self.out_eps = float(spec["out_norm_eps"])
        self.lam = None

    @classmethod
    def expected(cls, spec: PartSpec, hidden_size: int) -> dict:
        n = dict(spec["names"])
        H, G, D = int(spec["n_heads"]), int(spec["n_kv_heads"]), int(spec["head_dim"])
        V = int(spec.get("v_dim") or D)
        out = {n["q"]: Expected((2 * H * D, hidden_size)), n["k"]: Expected((2 * G * D, hidden_size)),
               n["v"]: Expected((G * V, hidden_size)), n["o"]: Expected((hidden_size, H * V))}
        if spec.get("qk_norm") is not None:
            out[n["q_norm"]], out[n["k_norm"]] = Expected((D,), init="scale"), Expected((D,), init="scale")
        for k in ("lq1", "lk1", "lq2", "lk2"):
            out[n[k]] = Expected((D,))
        if spec.get("sink") == "learned":
            out[n["sink"]] = Expected((2 * H,))
        return out

    def bind(self, tensors: dict) -> None:
        n, D = self.names, self.hd
        tensors = dict(tensors)
        for key, heads in (("q", self.H), ("k", self.G)):      # rows head by head [map 1, map 2] -> map by map
            w = tensors[n[key]]
            tensors[n[key]] = w.view(heads, 2, D, self.hidden).transpose(0, 1).reshape(2 * heads * D, self.hidden)
        super().bind(tensors)
        lq1, lk1, lq2, lk2 = (tensors[n[k]].to(torch.float64) for k in ("lq1", "lk1", "lq2", "lk2"))
        self.lam = math.exp(float(lq1 @ lk1)) - math.exp(float(lq2 @ lk2)) + self.diff

    def _project_out(self, o, qkv, gate_at: int, ctx, residual32, accumulate: bool) -> None:
        og = ctx.workspace.buffer("attn.gated", (o.shape[0], self.H * self.vd), self.dtype)
        kernels.diff_combine(o, self.H, self.cache_hd, self.vd, self.lam, self.out_eps, (1.0 - self.diff) * self.out_scale, og)
        kernels.linear(og, self.w_o, residual32, accumulate=accumulate)


register_mixer("gqa_attention", GQAAttention)
register_mixer("diff_attention", DiffAttention)
