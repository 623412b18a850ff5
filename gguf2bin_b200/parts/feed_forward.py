"""Feed-forwards.  ``swiglu``: down( silu(gate x) * (up x) ), no bias, dense
(src/l5_model.c:588-597, silu src/l3_math.c:57-62 of AnonymoDGH/gguf2bin).

The gate and up matrices are fused into one at bind time, rows alternating in blocks of
eight (eight gate rows, then the eight up rows of the same outputs), so one product
yields both and a kernel finds a gate and its up value sixteen columns apart at most.
A width that is no multiple of eight keeps the plain order (all gates, then all ups).
With ``limit`` the gate is capped from above and the up value from both sides, the gate's sigmoid
takes a slope and the up value an offset of one: g = min(gate x, limit), u = clamp(up x, -limit,
limit), down( g sigmoid(alpha g) (u + 1) ), ``alpha`` 1.702 unless the spec says otherwise.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..config.specs import ConfigError, PartSpec
from ..weights.loader import Expected
from .fused import normed_linear
from .registry import feed_forward_class, register_feed_forward


class SwiGLU:
    graph_safe = True          # its step only launches kernels: may be replayed from a CUDA graph

    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device):
        self.inter = int(spec["intermediate_size"])
        self.hidden = int(hidden_size)
        self.block = 8 if self.inter % 8 == 0 else self.inter
        self.dtype = dtype
        self.names = dict(spec["names"])
        self.w_gate_up = self.w_down = None
        self.limit = float(spec.get("limit") or 0.0)
        self.alpha = float(spec.get("alpha") if spec.get("alpha") is not None else 1.702)
        if self.limit < 0:
            raise ConfigError("swiglu: limit must be positive (or absent)")

    @classmethod
    def expected(cls, spec: PartSpec, hidden_size: int) -> dict:
        n, inter = dict(spec["names"]), spec["intermediate_size"]
        return {n["gate"]: Expected((inter, hidden_size)), n["up"]: Expected((inter, hidden_size)),
                n["down"]: Expected((hidden_size, inter))}

    def bind(self, tensors: dict) -> None:
        g, u = tensors[self.names["gate"]], tensors[self.names["up"]]
        if g.dtype != u.dtype:
            g, u = g.to(torch.float32), u.to(torch.float32)
        b = self.block
        fused = torch.stack([g.view(self.inter // b, b, self.hidden),
                             u.view(self.inter // b, b, self.hidden)], dim=1)
        self.w_gate_up = fused.reshape(2 * self.inter, self.hidden).contiguous()
        self.w_down = tensors[self.names["down"]].contiguous()

    def weights(self):
        return (self.w_gate_up, self.w_down)

    def absorb_norm_weight(self, norm) -> bool:
        """As ``GQAAttention.absorb_norm_weight``, into the columns of the gate/up matrix."""
        if self.dtype != torch.bfloat16 or self.w_gate_up.dtype != torch.bfloat16 or self.block != 8 \
                or not hasattr(norm, "give_up_weight") or self.limit:
            return False
        w = norm.give_up_weight()
        self.w_gate_up = (self.w_gate_up.float() * w.to(self.w_gate_up.device)[None, :]).to(torch.bfloat16).contiguous()
        return True

    def notices(self) -> list:
        return (kernels.product_notices("feed-forward gate/up", self.w_gate_up, self.dtype)
                + kernels.product_notices("feed-forward down", self.w_down, self.dtype))

    def forward(self, h: torch.Tensor, ctx, residual32: torch.Tensor) -> None:
        T = h.shape[0]
        ws = ctx.workspace
        mid = ws.buffer("ffn.mid", (T, self.inter), self.dtype)
        if self.limit or not kernels.gate_up_fused(h, self.w_gate_up, mid, self.block):
            gu = ws.buffer("ffn.gate_up", (T, 2 * self.inter), self.dtype)
            kernels.linear(h, self.w_gate_up, gu)
            kernels.swiglu(gu, mid, self.block, self.limit, self.alpha)
        kernels.linear(mid, self.w_down, residual32, accumulate=True)

    def forward_from_stream(self, x32: torch.Tensor, norm, ctx, residual32: torch.Tensor) -> None:
        """The same with the block's norm folded into the gate/up product."""
        if self.limit:                 # the fused epilogues know the plain SiLU gate only
            h = ctx.workspace.buffer("fused.normed", tuple(x32.shape), self.dtype)
            norm.forward(x32, h)
            return self.forward(h, ctx, residual32)
        mid = ctx.workspace.buffer("ffn.mid", (x32.shape[0], self.inter), self.dtype)
        normed_linear(x32, norm, self.w_gate_up, mid, ctx, gate_block=self.block)
        kernels.linear(mid, self.w_down, residual32, accumulate=True)


class ActMLP:
    """``act_mlp``: down( act(up x) ), two matrices and an elementwise activation.  Activations:
    ``xielu``, a z^2 + z/2 above zero and (1/2 + b)(exp(z) - 1 - z) + z/2 below, with a and b the
    softplus of two learned numbers (one tensor of two), computed in 32-bit; ``relu2``, max(z, 0)^2,
    which has no tensor of its own.

    A block may hand it one more matrix that reads the same input (``take_along``): its rows go
    under the up matrix, one product computes both, and the step leaves that matrix's output in
    ``side_out`` (a view of the product's output)."""
    graph_safe = True

    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device):
        self.inter, self.hidden = int(spec["intermediate_size"]), int(hidden_size)
        self.activation = spec.get("activation") or "xielu"
        if self.activation not in ("xielu", "relu2"):
            raise ConfigError(f"act_mlp: activation {self.activation!r} is not known (known: 'xielu', 'relu2')")
        self.dtype = dtype
        self.names = dict(spec["names"])
        self.w_up = self.w_down = self.act = None
        self.n_side = 0
        self.side_out = None

    @classmethod
    def expected(cls, spec: PartSpec, hidden_size: int) -> dict:
        n, inter = dict(spec["names"]), spec["intermediate_size"]
        out = {n["up"]: Expected((inter, hidden_size)), n["down"]: Expected((hidden_size, inter))}
        if (spec.get("activation") or "xielu") == "xielu":
            out[n["act"]] = Expected((2,))
        return out

    def bind(self, tensors: dict) -> None:
        self.w_up = tensors[self.names["up"]].contiguous()
        self.w_down = tensors[self.names["down"]].contiguous()
        if self.activation == "xielu":
            self.act = tensors[self.names["act"]].to(torch.float32).contiguous()

    def take_along(self, w_side: torch.Tensor) -> bool:
        """Puts ``w_side`` [n, hidden] under the up matrix; True when taken (equal dtypes, and an
        intermediate size that keeps the side output's rows on 16 bytes)."""
        if w_side.dtype != self.w_up.dtype or w_side.shape[1] != self.hidden or self.inter % 8 or self.n_side:
            return False
        pad = -(self.inter + w_side.shape[0]) % 8
        parts = [self.w_up, w_side]
        if pad:
            parts.append(torch.zeros((pad, self.hidden), dtype=self.w_up.dtype, device=self.w_up.device))
        self.w_up = torch.cat(parts, dim=0).contiguous()
        self.n_side = w_side.shape[0]
        return True

    def weights(self):
        return tuple(t for t in (self.w_up, self.w_down, self.act) if t is not None)

    def notices(self) -> list:
        return (kernels.product_notices("feed-forward up", self.w_up, self.dtype)
                + kernels.product_notices("feed-forward down", self.w_down, self.dtype))

    def forward(self, h: torch.Tensor, ctx, residual32: torch.Tensor) -> None:
        self._run(h, ctx, residual32, True)

    def forward_into(self, h: torch.Tensor, ctx, out32: torch.Tensor) -> None:
        """Stores the result instead of adding it."""
        self._run(h, ctx, out32, False)

    def _run(self, h, ctx, out32, accumulate: bool) -> None:
        T = h.shape[0]
        ws = ctx.workspace
        up = ws.buffer("mlp.up", (T, self.w_up.shape[0]), self.dtype)
        kernels.linear(h, self.w_up, up)
        self.side_out = up[:, self.inter:self.inter + self.n_side] if self.n_side else None
        mid = ws.buffer("mlp.mid", (T, self.inter), self.dtype)
        if self.activation == "relu2":
            kernels.relu2(up[:, :self.inter], mid)
        else:
            kernels.xielu(up[:, :self.inter], self.act, mid)
        kernels.linear(mid, self.w_down, out32, accumulate=accumulate)


class RoutedExperts:
    """``routed_experts``: ``n_experts`` small gated feed-forwards, down(silu(gate h) * (up h)) without
    biases, of which every token uses ``top``.  Router logits z = W_r h over ``n_experts + n_identity``
    outputs and their softmax are 32-bit; the ``top`` largest of score + ``correction`` (a stored
    vector that steers the choice and nothing else; optional) are chosen; a chosen expert's weight is
    its score as it is (``renormalise``: divided by the chosen scores' sum).  The last ``n_identity``
    router outputs stand for experts without matrices whose output is their input.  The result is
    the weighted sum of the chosen experts' outputs, added in the order of the choice.  ``scale``: every
    weight times that constant.  ``score`` = "sigmoid": the scores are the logits' sigmoids, each by itself,
    instead of a softmax.  ``groups`` with ``groups_kept``: the experts form that many equal groups of
    neighbours, a group counts as the sum of its two largest scores, and only experts of the best
    ``groups_kept`` groups can be chosen.  ``shared``: the spec of one more feed-forward (any registered kind)
    that runs for every token and is added.

    A step groups its (token, choice) pairs by expert on the device (``moe_plan``) and runs one
    grouped product for gate and up with the activation in its epilogue and one for down; nothing
    comes back to the host, so the step may be replayed from a CUDA graph."""
    graph_safe = True
    FEW_ROWS = 128            # (token, choice) pairs up to which every row streams its expert's matrices by itself
    MANY_ROWS = 48            # rows an expert on average from which its product runs on the tcgen05 kernel

    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device):
        self.E, self.I = int(spec["n_experts"]), int(spec.get("n_identity") or 0)
        self.top, self.inter = int(spec["top"]), int(spec["intermediate_size"])
        self.hidden, self.dtype, self.device = int(hidden_size), dtype, device
        self.renormalise = bool(spec.get("renormalise") or False)
        self.has_correction = bool(spec.get("correction") or False)
        if self.E < 0 or self.I < 0 or not (1 <= self.top <= self.E + self.I) or self.E > 1024:
            raise ConfigError(f"routed_experts: {self.top} choices among {self.E} + {self.I} experts")
        self.names = dict(spec["names"])
        self.w_router = self.correction = self.w_gate_up = self.w_down = None
        self.blocked = False
        self.scale = float(spec.get("scale") if spec.get("scale") is not None else 1.0)
        self.score = spec.get("score") or "softmax"
        self.groups = int(spec.get("groups") or 1)
        self.groups_kept = int(spec.get("groups_kept") or self.groups)
        n_all = self.E + self.I
        if self.score not in ("softmax", "sigmoid") or self.groups < 1 or n_all % self.groups \
                or not (1 <= self.groups_kept <= self.groups) or self.top > self.groups_kept * (n_all // self.groups):
            raise ConfigError(f"routed_experts: scores 'softmax' or 'sigmoid'; {n_all} experts in {self.groups} equal "
                              f"groups of which {self.groups_kept} are kept must hold {self.top} choices")
        shared = spec.get("shared")
        self.shared = feed_forward_class(shared)(shared, hidden_size, dtype, device) if shared is not None else None

    @classmethod
    def expected(cls, spec: PartSpec, hidden_size: int) -> dict:
        n, inter = dict(spec["names"]), spec["intermediate_size"]
        E, I = int(spec["n_experts"]), int(spec.get("n_identity") or 0)
        out = {n["router"]: Expected((E + I, hidden_size))}
        if spec.get("correction"):
            out[n["correction"]] = Expected((E + I,))
        for e in range(E):
            out[n["gate"].format(e)] = Expected((inter, hidden_size))
            out[n["up"].format(e)] = Expected((inter, hidden_size))
            out[n["down"].format(e)] = Expected((hidden_size, inter))
        if spec.get("shared") is not None:
            out.update(feed_forward_class(spec["shared"]).expected(spec["shared"], hidden_size))
        return out

    def bind(self, tensors: dict) -> None:
        n = self.names
        if self.shared is not None:
            self.shared.bind(tensors)
        self.w_router = tensors[n["router"]].contiguous()
        if self.has_correction:
            self.correction = tensors[n["correction"]].to(torch.float32).contiguous()
        if self.E:
            mats = [tensors[n[k].format(e)] for e in range(self.E) for k in ("gate", "up", "down")]
            common = torch.float32 if any(m.dtype == torch.float32 for m in mats) else mats[0].dtype
            # per expert: eight gate rows and the eight up rows of the same outputs in turn (the layout
            # whose neighbours the tensor-core epilogue combines); all gates, then all ups, where the
            # experts' size is no multiple of eight
            self.blocked = self.inter % 8 == 0
            b = 8 if self.blocked else self.inter

            def gate_up(e):
                g, u = tensors[n["gate"].format(e)].to(common), tensors[n["up"].format(e)].to(common)
                return torch.stack([g.view(self.inter // b, b, self.hidden), u.view(self.inter // b, b, self.hidden)],
                                   dim=1).reshape(2 * self.inter, self.hidden)
            self.w_gate_up = torch.stack([gate_up(e) for e in range(self.E)]).contiguous()
            self.w_down = torch.stack([tensors[n["down"].format(e)].to(common) for e in range(self.E)]).contiguous()

    def weights(self):
        own = tuple(t for t in (self.w_router, self.correction, self.w_gate_up, self.w_down) if t is not None)
        return own + (tuple(self.shared.weights()) if self.shared is not None else ())

    def notices(self) -> list:
        if self.w_gate_up is not None and self.dtype == torch.bfloat16 and \
                (self.w_gate_up.dtype != torch.bfloat16 or self.hidden % 8 or self.inter % 8):
            return ["routed experts: matrices kept in 32-bit, or sizes that are no multiple of 8: their "
                    "products run on the CUDA cores, not on the tensor cores"]
        return []

    def forward(self, h: torch.Tensor, ctx, residual32: torch.Tensor, x_self32: torch.Tensor = None) -> None:
        rows32, pair_row, weight = self._experts(h, ctx)
        if x_self32 is None and self.I:
            x_self32 = h if h.dtype == torch.float32 else h.float()
        kernels.moe_combine(rows32, pair_row, weight, x_self32 if self.I else rows32, self.top, residual32,
                            accumulate=True)
        if self.shared is not None:
            self.shared.forward(h, ctx, residual32)

    def forward_into(self, h: torch.Tensor, ctx, out32: torch.Tensor, x_self32: torch.Tensor = None) -> None:
        """Stores the result.  ``x_self32``: the input in 32-bit, for the experts whose output is their
        input (default: ``h`` widened)."""
        rows32, pair_row, weight = self._experts(h, ctx)
        if x_self32 is None and self.I:
            x_self32 = h if h.dtype == torch.float32 else h.float()
        kernels.moe_combine(rows32, pair_row, weight, x_self32 if self.I else rows32, self.top, out32)
        if self.shared is not None:
            self.shared.forward(h, ctx, out32)

    def forward_join(self, h: torch.Tensor, ctx, x32: torch.Tensor, norm_w, eps: float, cast_out) -> bool:
        """For a block that norms the feed-forward's output before it joins the stream ``x32`` (which is
        also the feed-forward's input in 32-bit): x += sum / sqrt(mean(sum^2) + eps) * norm_w in the
        pass that sums the experts.  False (nothing done) when the width is beyond that kernel."""
        if x32.shape[1] > 4096 or self.shared is not None:
            return False
        rows32, pair_row, weight = self._experts(h, ctx)
        return kernels.moe_combine_norm_add(rows32, pair_row, weight, x32, norm_w, eps, self.top, cast_out)

    def _experts(self, h: torch.Tensor, ctx):
        """Routing, plan and the experts' products: (rows, pair -> row, weights)."""
        T, ws, top, E = h.shape[0], ctx.workspace, self.top, self.E
        z = ws.buffer("moe.logits", (T, E + self.I), torch.float32)
        kernels.linear(h, self.w_router, z)
        idx = ws.buffer("moe.idx", (T, top), torch.int32)
        weight = ws.buffer("moe.weight", (T, top), torch.float32)
        kernels.moe_route(z, self.correction, top, self.renormalise, idx, weight, self.scale, self.score, self.groups,
                          self.groups_kept)
        n_pairs = T * top
        tile = kernels.moe_tile_rows()
        max_tiles = -(-n_pairs // tile) + E               # every expert's last tile may be part full
        plan = ws.buffer("moe.plan", (E + 2 + 3 * max_tiles,), torch.int32)
        row_pair = ws.buffer("moe.row_pair", (n_pairs,), torch.int32)
        pair_row = ws.buffer("moe.pair_row", (n_pairs,), torch.int32)
        kernels.moe_plan(idx, E, max_tiles, plan, row_pair, pair_row)
        rows32 = ws.buffer("moe.rows", (n_pairs, self.hidden), torch.float32)
        if E:
            wt = self.w_gate_up.dtype                     # matrices stored in 32-bit keep their products there
            mid = ws.buffer("moe.mid", (n_pairs, self.inter), wt)
            a = h if h.dtype == wt else h.to(wt)
            # few rows (decoding): every row streams its expert's matrices.  Many rows an expert (a prompt
            # step in bfloat16): the rows gathered side by side, then the tcgen05 kernel over each expert's
            # range.  Else tiles of rows per expert on mma.sync or the CUDA cores.
            few = n_pairs <= self.FEW_ROWS
            many = not few and wt == torch.bfloat16 and self.blocked and n_pairs >= self.MANY_ROWS * max(E, 1)
            done = False
            if few:
                done = kernels.moe_gemv(a, row_pair, top, True, idx, self.w_gate_up, self.inter, plan, E, n_pairs,
                                        True, mid, self.blocked)
            elif many and self.hidden % 8 == 0:
                rows = ws.buffer("moe.gathered", (n_pairs, self.hidden), wt)
                kernels.moe_gather(a, row_pair, top, plan, E, rows)
                done = kernels.moe_gemm_tc(rows, self.w_gate_up, self.inter, plan, E, max_tiles, True, mid)
            if not done:
                kernels.moe_gemm(a, row_pair, top, self.w_gate_up, self.inter, plan, E, max_tiles, True, mid,
                                 self.blocked)
            done = False
            if few:
                done = kernels.moe_gemv(mid, row_pair, top, False, idx, self.w_down, self.hidden, plan, E, n_pairs,
                                        False, rows32)
            elif many:
                done = kernels.moe_gemm_tc(mid, self.w_down, self.hidden, plan, E, max_tiles, False, rows32)
            if not done:
                kernels.moe_gemm(mid, None, 1, self.w_down, self.hidden, plan, E, max_tiles, False, rows32)
        return rows32, pair_row, weight


register_feed_forward("routed_experts", RoutedExperts)
register_feed_forward("swiglu", SwiGLU)
register_feed_forward("act_mlp", ActMLP)
