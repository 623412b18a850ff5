"""Mixers that keep a matrix state per head instead of keys, and a mixer made of several side by side.

``retention``: linear attention with a fixed decay per head and neither softmax nor denominator.
q = W_q h, k = W_k h (heads x qk_dim), v = W_v h (heads x v_dim); the position part turns q and k;
k times ``k_scale`` (default qk_dim^-1/2); per head S_t = a_h S_{t-1} + k_t v_t^T, o_t = S_t^T q_t;
each head's o divided by its root mean square (no weight); heads side by side times silu(W_g h);
output product.

``gated_delta``: the gated delta rule.  q = W_q h, k = W_k h (qk_heads x qk_dim), v = W_v h (heads x
v_dim); value head i reads query/key head i // (heads / qk_heads).  Each passes a short causal
convolution over time (``conv_taps`` taps per channel, the last the current token's) and SiLU; q and k
become unit vectors per head (x / sqrt(sum x^2 + unit_eps)), q times qk_dim^-1/2.  Per token and head
b = sigmoid(W_b h), g = exp(-exp(A_log) softplus(W_a h + dt_bias)); then S <- g S;
u = b (v - S^T k); S <- S + k u^T; o = S^T q, in this order.  Each head's o divided by its root mean
square, times a weight over v_dim shared by the heads, times silu(W_g h); output product.

``ssd``: a state-space mixer with one scalar decay per head and token (the state-space duality form).
One input product laid out as [z: inner | x: inner | B: groups*state | C: groups*state | dt: heads],
inner = heads * v_dim; x, B and C together pass a causal convolution per channel (``conv_taps`` taps,
the last the current token's, with a bias) and SiLU; dt = softplus(dt + dt_bias); per head (head h
reads group h // (heads / groups)) S = exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x; y times
silu(z), THEN divided by its root mean square in ``norm_groups`` equal parts, times a weight; output
product.  In the scan's words: q = C, k = B, v = x, decay and strength per token from ``scan_gates_step``.

``mlstm``: a matrix memory with exponential gates.  q = W_q h * qk_dim^-1/2, k = W_k h, v = W_v h; per
head and token a log input gate i = cap tanh((W_i h + b_i) / cap) and a log forget gate
f = logsigmoid(cap tanh((W_f h + b_f) / cap)); with a running maximum m (from 0): m' = max(f + m, i),
S = exp(f + m - m') S + exp(i - m') k v^T, n likewise with k alone, o = S^T q / (max(|n . q|, exp(-m')) + 1e-6);
each head's o divided by its root mean square, times a weight over all heads, times sigmoid(W_g h);
output product.  n rides in the scan as one more column of S whose value is always 1.

``selective_ssm``: a state-space mixer with a decay per channel AND state entry (the selective scan).
W_in h = [x: inner | z: inner]; x through a causal convolution per channel (``conv_taps`` taps with a bias,
the last the current token's) and SiLU; W_x x = [dt: dt_rank | B: state_dim | C: state_dim];
dt = softplus(W_dt dt + dt_bias), one per channel; A = -exp(A_log) [inner, state_dim]; per channel c and
entry n: S[c, n] = exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n, y_c = sum_n S[c, n] C_n + D_c x_c; y silu(z);
output product.  The state [inner, state_dim] is 32-bit and starts at zero; the convolution's last
inputs are a ring by position.  Step sizes, decays and the recurrence are 32-bit.

``parallel``: several mixers that read the same input; the result is the sum of theirs, each times
its ``out_scale``.  A branch is any registered mixer that takes ``out_scale``.

State: S in float32, [slots, heads, v_dim, qk_dim] (a column of S, everything that feeds one output
channel, is contiguous), and for the convolution a ring of ``conv_taps`` input rows per slot indexed
by position.  Decays, gates, step sizes, unit norms, rotation and the recurrence are 32-bit; the
products and the convolution's inputs and outputs are in the compute type.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.storage import StateNeed
from ..config.specs import ConfigError, PartSpec
from ..weights.loader import Expected
from .registry import mixer_class, position_class, register_mixer


def _common_dtype(parts):
    return torch.float32 if any(p.dtype == torch.float32 for p in parts) else parts[0].dtype


class RetentionMixer:
    graph_safe = True

    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device):
        self.H, self.D, self.V = int(spec["n_heads"]), int(spec["qk_dim"]), int(spec["v_dim"])
        self.hidden, self.dtype, self.device = int(hidden_size), dtype, device
        decay = tuple(float(a) for a in spec["decay"])
        if len(decay) != self.H:
            raise ConfigError(f"retention: {len(decay)} decays for {self.H} heads")
        if min(self.H, self.D, self.V) <= 0 or self.D > 512:
            raise ConfigError("retention: heads, qk_dim (at most 512) and v_dim must be positive")
        self.decay = torch.tensor(decay, dtype=torch.float32, device=device)
        k_scale = spec.get("k_scale")
        self.k_scale = float(k_scale) if k_scale is not None else self.D ** -0.5
        self.eps = float(spec["eps"])
        self.out_scale = float(spec.get("out_scale") if spec.get("out_scale") is not None else 1.0)
        pos = spec.get("position") or PartSpec.make("none")
        self.position = position_class(pos)(pos, self.D, device)
        if not hasattr(self.position, "table_rotation"):
            raise ConfigError("retention: this position part offers no table rotation")
        self.names = dict(spec["names"])
        self.w_in = self.w_o = None

    @classmethod
    def expected(cls, spec: PartSpec, hidden_size: int) -> dict:
        n = dict(spec["names"])
        nq, nv = spec["n_heads"] * spec["qk_dim"], spec["n_heads"] * spec["v_dim"]
        return {n["q"]: Expected((nq, hidden_size)), n["k"]: Expected((nq, hidden_size)),
                n["v"]: Expected((nv, hidden_size)), n["gate"]: Expected((nv, hidden_size)),
                n["o"]: Expected((hidden_size, nv))}

    def bind(self, tensors: dict) -> None:
        n = self.names
        parts = [tensors[n[k]] for k in ("q", "k", "v", "gate")]
        common = _common_dtype(parts)
        self.w_in = torch.cat([p.to(common) for p in parts], dim=0).contiguous()      # one product: q | k | v | gate
        self.w_o = tensors[n["o"]].contiguous()

    def weights(self):
        return (self.w_in, self.w_o)

    def notices(self) -> list:
        return (kernels.product_notices("retention input", self.w_in, self.dtype)
                + kernels.product_notices("retention output", self.w_o, self.dtype))

    def cache_need(self):
        return StateNeed((self.H, self.V, self.D), torch.float32)

    def forward(self, h: torch.Tensor, ctx, view, residual32: torch.Tensor) -> None:
        self._run(h, ctx, view, residual32, True)

    def forward_store(self, h: torch.Tensor, ctx, view, out32: torch.Tensor) -> None:
        """Stores the result instead of adding it."""
        self._run(h, ctx, view, out32, False)

    def _run(self, h, ctx, view, residual32, accumulate: bool) -> None:
        T, ws = h.shape[0], ctx.workspace
        nq, nv = self.H * self.D, self.H * self.V
        proj = ws.buffer("retention.in", (T, 2 * nq + 2 * nv), self.dtype)
        kernels.linear(h, self.w_in, proj)
        inv_freq, rot, interleaved = self.position.table_rotation()
        rope = ctx.rope_table(inv_freq) if inv_freq is not None else None
        o32 = ws.buffer("retention.o", (T, nv), torch.float32)
        kernels.state_scan(proj[:, :nq], proj[:, nq:2 * nq], proj[:, 2 * nq:2 * nq + nv], view.states, ctx, o32,
                           self.H, self.H, self.D, self.V, decay=self.decay, rope=rope, rotary_dim=rot,
                           interleaved=interleaved, k_scale=self.k_scale)
        og = ws.buffer("retention.gated", (T, nv), self.dtype)
        kernels.head_norm_gate(o32, self.H, self.V, None, self.eps, proj[:, 2 * nq + nv:], self.out_scale, og)
        kernels.linear(og, self.w_o, residual32, accumulate=accumulate)


class GatedDeltaMixer:
    graph_safe = True

    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device):
        self.H, self.G = int(spec["n_heads"]), int(spec["n_qk_heads"])
        self.D, self.V = int(spec["qk_dim"]), int(spec["v_dim"])
        self.taps = int(spec["conv_taps"])
        self.hidden, self.dtype, self.device = int(hidden_size), dtype, device
        if self.G <= 0 or self.H % self.G:
            raise ConfigError(f"gated_delta: {self.H} heads are not a multiple of {self.G} query/key heads")
        if min(self.D, self.V) <= 0 or self.D > 512 or not (1 <= self.taps <= 16):
            raise ConfigError("gated_delta: qk_dim in 1..512, v_dim positive, conv_taps in 1..16")
        self.eps = float(spec["eps"])
        self.unit_eps = float(spec.get("unit_eps") if spec.get("unit_eps") is not None else 1e-6)
        self.out_scale = float(spec.get("out_scale") if spec.get("out_scale") is not None else 1.0)
        self.names = dict(spec["names"])
        self.w_in = self.w_ab = self.w_conv = self.w_o = self.a_log = self.dt_bias = self.norm_w = None

    @property
    def channels(self) -> int:
        return 2 * self.G * self.D + self.H * self.V

    @classmethod
    def expected(cls, spec: PartSpec, hidden_size: int) -> dict:
        n = dict(spec["names"])
        H, G, D, V, taps = (spec[k] for k in ("n_heads", "n_qk_heads", "qk_dim", "v_dim", "conv_taps"))
        return {n["q"]: Expected((G * D, hidden_size)), n["k"]: Expected((G * D, hidden_size)),
                n["v"]: Expected((H * V, hidden_size)), n["gate"]: Expected((H * V, hidden_size)),
                n["q_conv"]: Expected((G * D, taps)), n["k_conv"]: Expected((G * D, taps)),
                n["v_conv"]: Expected((H * V, taps)), n["beta"]: Expected((H, hidden_size)),
                n["a"]: Expected((H, hidden_size)), n["a_log"]: Expected((H,)), n["dt_bias"]: Expected((H,)),
                n["norm"]: Expected((V,), init="scale"), n["o"]: Expected((hidden_size, H * V))}

    def bind(self, tensors: dict) -> None:
        n = self.names
        parts = [tensors[n[k]] for k in ("q", "k", "v", "gate")]
        common = _common_dtype(parts)
        self.w_in = torch.cat([p.to(common) for p in parts], dim=0).contiguous()       # q | k | v | gate
        ab = [tensors[n["a"]], tensors[n["beta"]]]
        self.w_ab = torch.cat([p.to(_common_dtype(ab)) for p in ab], dim=0).contiguous()       # decay input | write strength
        conv = torch.cat([tensors[n[k]].to(torch.float32) for k in ("q_conv", "k_conv", "v_conv")], dim=0)
        self.w_conv = conv.t().contiguous()               # [taps, channels]: a tap's weights side by side
        self.a_log = tensors[n["a_log"]].to(torch.float32).contiguous()
        self.dt_bias = tensors[n["dt_bias"]].to(torch.float32).contiguous()
        self.norm_w = tensors[n["norm"]].to(torch.float32).contiguous()
        self.w_o = tensors[n["o"]].contiguous()

    def weights(self):
        return (self.w_in, self.w_ab, self.w_conv, self.a_log, self.dt_bias, self.norm_w, self.w_o)

    def notices(self) -> list:
        return (kernels.product_notices("gated delta input", self.w_in, self.dtype)
                + kernels.product_notices("gated delta output", self.w_o, self.dtype))

    def cache_need(self):
        need = {"state": StateNeed((self.H, self.V, self.D), torch.float32)}
        if self.taps > 1:
            need["conv"] = StateNeed((self.taps, self.channels), self.dtype, by_position=True)
        return need

    def forward(self, h: torch.Tensor, ctx, view, residual32: torch.Tensor) -> None:
        self._run(h, ctx, view, residual32, True)

    def forward_store(self, h: torch.Tensor, ctx, view, out32: torch.Tensor) -> None:
        """Stores the result instead of adding it."""
        self._run(h, ctx, view, out32, False)

    def _run(self, h, ctx, view, residual32, accumulate: bool) -> None:
        T, ws = h.shape[0], ctx.workspace
        C, nq, nv = self.channels, self.G * self.D, self.H * self.V
        proj = ws.buffer("delta.in", (T, C + nv), self.dtype)
        kernels.linear(h, self.w_in, proj)
        ab = ws.buffer("delta.ab", (T, 2 * self.H), torch.float32)
        kernels.linear(h, self.w_ab, ab)
        mixed = ws.buffer("delta.conv", (T, C), self.dtype)
        ring = view["conv"].states if self.taps > 1 else None
        kernels.short_conv(proj[:, :C], self.w_conv, ring, ctx, mixed, act=True)
        o32 = ws.buffer("delta.o", (T, nv), torch.float32)
        kernels.state_scan(mixed[:, :nq], mixed[:, nq:2 * nq], mixed[:, 2 * nq:], view["state"].states, ctx, o32,
                           self.H, self.G, self.D, self.V, ab=ab, a_log=self.a_log, dt_bias=self.dt_bias,
                           q_scale=self.D ** -0.5, unit_eps=self.unit_eps)
        og = ws.buffer("delta.gated", (T, nv), self.dtype)
        kernels.head_norm_gate(o32, self.H, self.V, self.norm_w, self.eps, proj[:, C:], self.out_scale, og)
        kernels.linear(og, self.w_o, residual32, accumulate=accumulate)


def _padded_rows(parts, multiple: int = 8):
    """The matrices one under the other in a common type, with rows of zeros up to a multiple
    (an output row then starts on 16 bytes in bfloat16)."""
    common = _common_dtype(parts)
    rows = sum(p.shape[0] for p in parts)
    pad = -rows % multiple
    mats = [p.to(common) for p in parts]
    if pad:
        mats.append(torch.zeros((pad, parts[0].shape[1]), dtype=common, device=parts[0].device))
    return torch.cat(mats, dim=0).contiguous()


class SSDMixer:
    graph_safe = True

    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device):
        self.H, self.G = int(spec["n_heads"]), int(spec["n_groups"])
        self.N, self.V = int(spec["state_dim"]), int(spec["v_dim"])
        self.taps, self.norm_groups = int(spec["conv_taps"]), int(spec.get("norm_groups") or 1)
        self.hidden, self.dtype, self.device = int(hidden_size), dtype, device
        if self.G <= 0 or self.H % self.G:
            raise ConfigError(f"ssd: {self.H} heads are not a multiple of {self.G} groups")
        if min(self.N, self.V) <= 0 or self.N > 512 or not (1 <= self.taps <= 16):
            raise ConfigError("ssd: state_dim in 1..512, v_dim positive, conv_taps in 1..16")
        if self.norm_groups <= 0 or self.inner % self.norm_groups:
            raise ConfigError(f"ssd: {self.norm_groups} norm groups do not divide {self.inner} channels")
        self.eps = float(spec["eps"])
        self.names = dict(spec["names"])
        self.w_in = self.w_conv = self.b_conv = self.a_log = self.dt_bias = self.skip = self.norm_w = self.w_o = None

    @property
    def inner(self) -> int:
        return self.H * self.V

    @property
    def channels(self) -> int:
        return self.inner + 2 * self.G * self.N

    @classmethod
    def expected(cls, spec: PartSpec, hidden_size: int) -> dict:
        n = dict(spec["names"])
        H, G, N, V, taps = (int(spec[k]) for k in ("n_heads", "n_groups", "state_dim", "v_dim", "conv_taps"))
        inner, C = H * V, H * V + 2 * G * N
        return {n["in"]: Expected((2 * inner + 2 * G * N + H, hidden_size)), n["conv"]: Expected((C, taps)),
                n["conv_bias"]: Expected((C,)), n["dt_bias"]: Expected((H,)), n["a_log"]: Expected((H,)),
                n["skip"]: Expected((H,)), n["norm"]: Expected((inner,), init="scale"),
                n["o"]: Expected((hidden_size, inner))}

    def bind(self, tensors: dict) -> None:
        n = self.names
        self.w_in = _padded_rows([tensors[n["in"]]])             # z | x | B | C | dt (| zeros)
        self.w_conv = tensors[n["conv"]].to(torch.float32).t().contiguous()          # [taps, channels]
        self.b_conv = tensors[n["conv_bias"]].to(torch.float32).contiguous()
        self.a_log = tensors[n["a_log"]].to(torch.float32).contiguous()
        self.dt_bias = tensors[n["dt_bias"]].to(torch.float32).contiguous()
        self.skip = tensors[n["skip"]].to(torch.float32).contiguous()
        self.norm_w = tensors[n["norm"]].to(torch.float32).contiguous()
        self.w_o = tensors[n["o"]].contiguous()

    def weights(self):
        return (self.w_in, self.w_conv, self.b_conv, self.a_log, self.dt_bias, self.skip, self.norm_w, self.w_o)

    def notices(self) -> list:
        return (kernels.product_notices("state-space input", self.w_in, self.dtype)
                + kernels.product_notices("state-space output", self.w_o, self.dtype))

    def cache_need(self):
        need = {"state": StateNeed((self.H, self.V, self.N), torch.float32)}
        if self.taps > 1:
            need["conv"] = StateNeed((self.taps, self.channels), self.dtype, by_position=True)
        return need

    def forward(self, h: torch.Tensor, ctx, view, residual32: torch.Tensor) -> None:
        self._run(h, ctx, view, residual32, True)

    def forward_store(self, h: torch.Tensor, ctx, view, out32: torch.Tensor) -> None:
        """Stores the result instead of adding it."""
        self._run(h, ctx, view, out32, False)

    def _run(self, h, ctx, view, residual32, accumulate: bool) -> None:
        T, ws = h.shape[0], ctx.workspace
        inner, C, gn = self.inner, self.channels, self.G * self.N
        proj = ws.buffer("ssd.in", (T, self.w_in.shape[0]), self.dtype)
        kernels.linear(h, self.w_in, proj)
        mixed = ws.buffer("ssd.conv", (T, C), self.dtype)
        ring = view["conv"].states if self.taps > 1 else None
        kernels.short_conv(proj[:, inner:inner + C], self.w_conv, ring, ctx, mixed, act=True, bias=self.b_conv)
        gates = ws.buffer("ssd.gates", (T, 2 * self.H), torch.float32)
        kernels.scan_gates_step(proj[:, inner + C:inner + C + self.H], self.a_log, self.dt_bias, gates)
        o32 = ws.buffer("ssd.o", (T, inner), torch.float32)
        kernels.state_scan(mixed[:, inner + gn:], mixed[:, inner:inner + gn], mixed[:, :inner], view["state"].states,
                           ctx, o32, self.H, self.G, self.N, self.V, gates=gates)
        og = ws.buffer("ssd.gated", (T, inner), self.dtype)
        kernels.state_readout(o32, self.H, self.V, og, skip_x=mixed[:, :inner], skip_w=self.skip, gate=proj[:, :inner],
                              gate_act="silu", gate_first=True, group=inner // self.norm_groups, eps=self.eps,
                              w=self.norm_w)
        kernels.linear(og, self.w_o, residual32, accumulate=accumulate)


class SelectiveSSM:
    graph_safe = True

    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device):
        self.inner, self.N, self.R = int(spec["inner"]), int(spec["state_dim"]), int(spec["dt_rank"])
        self.taps = int(spec["conv_taps"])
        self.hidden, self.dtype, self.device = int(hidden_size), dtype, device
        if min(self.inner, self.R) <= 0 or not (1 <= self.N <= 256) or not (1 <= self.taps <= 16):
            raise ConfigError("selective_ssm: inner and dt_rank positive, state_dim in 1..256, conv_taps in 1..16")
        self.out_scale = float(spec.get("out_scale") if spec.get("out_scale") is not None else 1.0)
        self.names = dict(spec["names"])
        self.w_in = self.w_conv = self.b_conv = self.w_x = self.w_dt = self.dt_bias = self.a = self.skip = self.w_o = None

    @classmethod
    def expected(cls, spec: PartSpec, hidden_size: int) -> dict:
        n = dict(spec["names"])
        inner, N, R, taps = (int(spec[k]) for k in ("inner", "state_dim", "dt_rank", "conv_taps"))
        return {n["in"]: Expected((2 * inner, hidden_size)), n["conv"]: Expected((inner, taps)),
                n["conv_bias"]: Expected((inner,)), n["x"]: Expected((R + 2 * N, inner)), n["dt"]: Expected((inner, R)),
                n["dt_bias"]: Expected((inner,)), n["a_log"]: Expected((inner, N)), n["skip"]: Expected((inner,)),
                n["o"]: Expected((hidden_size, inner))}

    def bind(self, tensors: dict) -> None:
        n = self.names
        self.w_in = _padded_rows([tensors[n["in"]]])                  # x | z
        self.w_conv = tensors[n["conv"]].to(torch.float32).t().contiguous()          # [taps, channels]
        self.b_conv = tensors[n["conv_bias"]].to(torch.float32).contiguous()
        self.w_x = _padded_rows([tensors[n["x"]]])                    # dt | B | C (| zeros)
        self.w_dt = tensors[n["dt"]].contiguous()
        self.dt_bias = tensors[n["dt_bias"]].to(torch.float32).contiguous()
        self.a = (-torch.exp(tensors[n["a_log"]].to(torch.float32))).contiguous()    # the decay rates, 32-bit
        self.skip = tensors[n["skip"]].to(torch.float32).contiguous()
        self.w_o = tensors[n["o"]].contiguous()

    def weights(self):
        return (self.w_in, self.w_conv, self.b_conv, self.w_x, self.w_dt, self.dt_bias, self.a, self.skip, self.w_o)

    def notices(self) -> list:
        return (kernels.product_notices("state-space input", self.w_in, self.dtype)
                + kernels.product_notices("state-space step size", self.w_dt, self.dtype)
                + kernels.product_notices("state-space output", self.w_o, self.dtype))

    def cache_need(self):
        need = {"state": StateNeed((self.inner, self.N), torch.float32)}
        if self.taps > 1:
            need["conv"] = StateNeed((self.taps, self.inner), self.dtype, by_position=True)
        return need

    def forward(self, h: torch.Tensor, ctx, view, residual32: torch.Tensor) -> None:
        self._run(h, ctx, view, residual32, True)

    def forward_store(self, h: torch.Tensor, ctx, view, out32: torch.Tensor) -> None:
        """Stores the result instead of adding it."""
        self._run(h, ctx, view, out32, False)

    def _run(self, h, ctx, view, residual32, accumulate: bool) -> None:
        T, ws = h.shape[0], ctx.workspace
        inner, N, R = self.inner, self.N, self.R
        proj = ws.buffer("ssm.in", (T, self.w_in.shape[0]), self.dtype)
        kernels.linear(h, self.w_in, proj)
        x = ws.buffer("ssm.conv", (T, inner), self.dtype)
        ring = view["conv"].states if self.taps > 1 else None
        kernels.short_conv(proj[:, :inner], self.w_conv, ring, ctx, x, act=True, bias=self.b_conv)
        p = ws.buffer("ssm.x", (T, self.w_x.shape[0]), self.dtype)
        kernels.linear(x, self.w_x, p)
        dt = ws.buffer("ssm.dt", (T, inner), torch.float32)           # before bias and softplus, which the scan applies
        kernels.linear(p[:, :R], self.w_dt, dt)
        og = ws.buffer("ssm.gated", (T, inner), self.dtype)
        kernels.selective_scan(x, dt, self.dt_bias, p[:, R:R + 2 * N], self.a, self.skip, proj[:, inner:2 * inner],
                               view["state"].states, ctx, og, self.out_scale)
        kernels.linear(og, self.w_o, residual32, accumulate=accumulate)


class MLSTMMixer:
    graph_safe = True
    DEN_EPS = 1e-6            # added to the read-out's denominator

    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device):
        self.H, self.D, self.V = int(spec["n_heads"]), int(spec["qk_dim"]), int(spec["v_dim"])
        self.cap = float(spec["gate_cap"])
        self.hidden, self.dtype, self.device = int(hidden_size), dtype, device
        if min(self.H, self.D, self.V) <= 0 or self.D > 512:
            raise ConfigError("mlstm: heads, qk_dim (at most 512) and v_dim must be positive")
        if not self.cap > 0:
            raise ConfigError("mlstm: gate_cap must be positive")
        self.eps = float(spec["eps"])
        self.names = dict(spec["names"])
        self.w_in = self.w_o = self.b_i = self.b_f = self.norm_w = None

    @classmethod
    def expected(cls, spec: PartSpec, hidden_size: int) -> dict:
        n = dict(spec["names"])
        H, D, V = int(spec["n_heads"]), int(spec["qk_dim"]), int(spec["v_dim"])
        return {n["q"]: Expected((H * D, hidden_size)), n["k"]: Expected((H * D, hidden_size)),
                n["v"]: Expected((H * V, hidden_size)), n["gate"]: Expected((H * V, hidden_size)),
                n["i"]: Expected((H, hidden_size)), n["i_bias"]: Expected((H,)),
                n["f"]: Expected((H, hidden_size)), n["f_bias"]: Expected((H,)),
                n["norm"]: Expected((H * V,), init="scale"), n["o"]: Expected((hidden_size, H * V))}

    def bind(self, tensors: dict) -> None:
        n = self.names
        # one product: q | k | v | gate | i | f (| zeros)
        self.w_in = _padded_rows([tensors[n[k]] for k in ("q", "k", "v", "gate", "i", "f")])
        self.b_i = tensors[n["i_bias"]].to(torch.float32).contiguous()
        self.b_f = tensors[n["f_bias"]].to(torch.float32).contiguous()
        self.norm_w = tensors[n["norm"]].to(torch.float32).contiguous()
        self.w_o = tensors[n["o"]].contiguous()

    def weights(self):
        return (self.w_in, self.b_i, self.b_f, self.norm_w, self.w_o)

    def notices(self) -> list:
        return (kernels.product_notices("mlstm input", self.w_in, self.dtype)
                + kernels.product_notices("mlstm output", self.w_o, self.dtype))

    def cache_need(self):
        # S with the normaliser as its last column, and the running maximum
        return {"state": StateNeed((self.H, self.V + 1, self.D), torch.float32),
                "max": StateNeed((self.H,), torch.float32)}

    def forward(self, h: torch.Tensor, ctx, view, residual32: torch.Tensor) -> None:
        self._run(h, ctx, view, residual32, True)

    def forward_store(self, h: torch.Tensor, ctx, view, out32: torch.Tensor) -> None:
        """Stores the result instead of adding it."""
        self._run(h, ctx, view, out32, False)

    def _run(self, h, ctx, view, residual32, accumulate: bool) -> None:
        T, ws = h.shape[0], ctx.workspace
        H, nq, nv = self.H, self.H * self.D, self.H * self.V
        proj = ws.buffer("mlstm.in", (T, self.w_in.shape[0]), self.dtype)
        kernels.linear(h, self.w_in, proj)
        at = 2 * nq + 2 * nv
        gates = ws.buffer("mlstm.gates", (T, 2 * H), torch.float32)
        m = ws.buffer("mlstm.max", (T, H), torch.float32)
        kernels.scan_gates_max(proj[:, at:at + H], proj[:, at + H:at + 2 * H], self.b_i, self.b_f, self.cap,
                               view["max"].states, ctx, gates, m)
        o32 = ws.buffer("mlstm.o", (T, H * (self.V + 1)), torch.float32)
        kernels.state_scan(proj[:, :nq], proj[:, nq:2 * nq], proj[:, 2 * nq:2 * nq + nv], view["state"].states, ctx,
                           o32, H, H, self.D, self.V, gates=gates, q_scale=self.D ** -0.5, ones_column=True)
        og = ws.buffer("mlstm.gated", (T, nv), self.dtype)
        kernels.state_readout(o32, H, self.V, og, stored_cols=self.V + 1, m=m, den_eps=self.DEN_EPS,
                              gate=proj[:, 2 * nq + nv:at], gate_act="sigmoid", gate_first=False, group=self.V,
                              eps=self.eps, w=self.norm_w)
        kernels.linear(og, self.w_o, residual32, accumulate=accumulate)


class ParallelMixer:
    """Branches side by side on one input; what each stores is kept under ``<branch>.<name>``."""

    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device):
        branches = spec["branches"]                       # ((name, PartSpec), ...)
        if not branches:
            raise ConfigError("parallel: at least one branch")
        self.branches = [(name, mixer_class(s)(s, hidden_size, dtype, device)) for name, s in branches]

    @classmethod
    def expected(cls, spec: PartSpec, hidden_size: int) -> dict:
        out = {}
        for _, s in spec["branches"]:
            out.update(mixer_class(s).expected(s, hidden_size))
        return out

    def bind(self, tensors: dict) -> None:
        for _, m in self.branches:
            m.bind(tensors)

    def weights(self):
        for _, m in self.branches:
            yield from getattr(m, "weights", tuple)()

    def notices(self) -> list:
        return [line for _, m in self.branches for line in getattr(m, "notices", list)()]

    @property
    def graph_safe(self) -> bool:
        return all(getattr(m, "graph_safe", False) for _, m in self.branches)

    def cache_need(self):
        need = {}
        for name, m in self.branches:
            one = m.cache_need()
            if isinstance(one, dict):
                need.update({f"{name}.{k}": v for k, v in one.items() if v is not None})
            elif one is not None:
                need[name] = one
        return need or None

    def forward(self, h: torch.Tensor, ctx, view, residual32: torch.Tensor) -> None:
        self._run(h, ctx, view, residual32, True)

    def forward_store(self, h: torch.Tensor, ctx, view, out32: torch.Tensor) -> None:
        """Stores the result: the first branch stores (or adds into the cleared buffer), the others add."""
        self._run(h, ctx, view, out32, False)

    def _run(self, h, ctx, view, residual32, accumulate: bool) -> None:
        view = view or {}
        for i, (name, m) in enumerate(self.branches):
            own = view.get(name)
            if own is None:
                own = {k[len(name) + 1:]: v for k, v in view.items() if k.startswith(name + ".")} or None
            if i == 0 and not accumulate:
                if hasattr(m, "forward_store"):
                    m.forward_store(h, ctx, own, residual32)
                    continue
                residual32.zero_()
            m.forward(h, ctx, own, residual32)


register_mixer("retention", RetentionMixer)
register_mixer("gated_delta", GatedDeltaMixer)
register_mixer("parallel", ParallelMixer)
register_mixer("ssd", SSDMixer)
register_mixer("mlstm", MLSTMMixer)
register_mixer("selective_ssm", SelectiveSSM)
