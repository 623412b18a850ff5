"""Block arrangements.  ``prenorm``: x += mixer(norm(x)); x += feed_forward(norm(x)), the
residual stream kept in float32 (src/l5_model.c:494-597 of AnonymoDGH/gguf2bin).
``branch_norm``: x += norm(mixer(x)); x += norm(feed_forward(x)): the norm sits on each sublayer's
OUTPUT and the sublayers read the stream itself.
``gated_prenorm``: the same with each sublayer's result scaled by a learned gate, an optional
short convolution over time in front of the mixer, and an optional feed-forward.
``parallel_shift``: h = norm(x); x += mixer(shift(h)) + feed_forward(h): one norm, both sublayers read
it, and the mixer's copy is mixed with the token before, channel by channel.
``parallel_scaled``: h = norm(x); x += s1 * mixer(h) + s2 * feed_forward(h): one norm of any registered kind,
both sublayers read it, and each result is multiplied by a learned number per channel before the sum."""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.storage import StateNeed
from ..config.specs import ConfigError, LayerSpec
from ..weights.loader import Expected
from .feed_forward import RoutedExperts
from .norms import RMSNorm, TanhNorm, bind_norm
from .registry import (feed_forward_class, mixer_class, norm_class, register_block)


class PreNormBlock:
    def __init__(self, layer: LayerSpec, hidden_size: int, dtype: torch.dtype, device):
        self.names = dict(layer.block["names"])
        self.hidden, self.dtype = int(hidden_size), dtype
        ffn_norm = layer.ffn_norm or layer.norm
        self.mixer_norm = norm_class(layer.norm)(layer.norm, hidden_size, dtype, device)
        self.ffn_norm = norm_class(ffn_norm)(ffn_norm, hidden_size, dtype, device)
        self.mixer = mixer_class(layer.mixer)(layer.mixer, hidden_size, dtype, device)
        self.feed_forward = feed_forward_class(layer.feed_forward)(layer.feed_forward, hidden_size,
                                                                   dtype, device)

    @classmethod
    def expected(cls, layer: LayerSpec, hidden_size: int) -> dict:
        names = dict(layer.block["names"])
        ffn_norm = layer.ffn_norm or layer.norm
        out = {}
        out.update(norm_class(layer.norm).expected(layer.norm, hidden_size, names["mixer_norm"]))
        out.update(norm_class(ffn_norm).expected(ffn_norm, hidden_size, names["ffn_norm"]))
        out.update(mixer_class(layer.mixer).expected(layer.mixer, hidden_size))
        out.update(feed_forward_class(layer.feed_forward).expected(layer.feed_forward, hidden_size))
        return out

    def bind(self, tensors: dict) -> None:
        self.mixer_norm.bind(tensors[self.names["mixer_norm"]])
        self.ffn_norm.bind(tensors[self.names["ffn_norm"]])
        self.mixer.bind(tensors)
        self.feed_forward.bind(tensors)
        # a part that starts from the stream (``forward_from_stream``) may take the weight of
        # the norm in front of it into its first matrix; the norm is then a plain division
        for part, norm in ((self.mixer, self.mixer_norm), (self.feed_forward, self.ffn_norm)):
            if hasattr(part, "forward_from_stream") and hasattr(part, "absorb_norm_weight"):
                part.absorb_norm_weight(norm)

    def cache_need(self):
        return self.mixer.cache_need()

    def parts(self) -> tuple:
        return (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward)

    def weights(self):
        """Every tensor the block's parts hold (a part without ``weights()`` reports none)."""
        for part in self.parts():
            yield from getattr(part, "weights", tuple)()

    def notices(self) -> list:
        return [line for part in self.parts() for line in getattr(part, "notices", list)()]

    @property
    def graph_safe(self) -> bool:
        """Whether a step of this block may be captured in a CUDA graph and replayed: every part
        must say so itself (``graph_safe = True``: its step does nothing but launch kernels on
        the current stream, takes its scratch memory from the step's workspace, and neither reads
        results on the host nor keeps host-side state from step to step)."""
        return all(getattr(part, "graph_safe", False) for part in self.parts())

    def forward(self, x32: torch.Tensor, ctx, cache_view) -> None:
        # a part that offers ``forward_from_stream`` takes the stream and the norm and may
        # fold the norm into its first product; any other part gets normed activations
        T = x32.shape[0]
        if hasattr(self.mixer, "forward_from_stream"):
            self.mixer.forward_from_stream(x32, self.mixer_norm, ctx, cache_view, x32)
        else:
            h = ctx.workspace.buffer("block.normed", (T, self.hidden), self.dtype)
            self.mixer_norm.forward(x32, h)
            self.mixer.forward(h, ctx, cache_view, x32)
        if hasattr(self.feed_forward, "forward_from_stream"):
            self.feed_forward.forward_from_stream(x32, self.ffn_norm, ctx, x32)
        else:
            h = ctx.workspace.buffer("block.normed", (T, self.hidden), self.dtype)
            self.ffn_norm.forward(x32, h)
            self.feed_forward.forward(h, ctx, x32)


class BranchNormBlock:
    """``branch_norm``: x <- x + norm1(mixer(x)), then x <- x + norm2(feed_forward(x)).  The
    sublayers read the stream as it is (rounded to the compute type for their products); each
    sublayer's whole output is normed, in 32-bit, before it joins the stream.  A layer may have no
    feed-forward.  Any mixer or feed-forward of the library fits: a part adds into a cleared
    32-bit buffer, or stores there when it offers ``forward_store`` (mixers) or ``forward_into``
    (feed-forwards); routed experts sum, norm and join the stream in one pass (``forward_join``)."""

    def __init__(self, layer: LayerSpec, hidden_size: int, dtype: torch.dtype, device):
        self.names = dict(layer.block["names"])
        self.hidden, self.dtype = int(hidden_size), dtype
        ffn_norm = layer.ffn_norm or layer.norm
        self.mixer_norm = norm_class(layer.norm)(layer.norm, hidden_size, dtype, device)
        self.mixer = mixer_class(layer.mixer)(layer.mixer, hidden_size, dtype, device)
        self.feed_forward = self.ffn_norm = None
        if layer.feed_forward is not None:
            self.ffn_norm = norm_class(ffn_norm)(ffn_norm, hidden_size, dtype, device)
            self.feed_forward = feed_forward_class(layer.feed_forward)(layer.feed_forward, hidden_size,
                                                                       dtype, device)

    @classmethod
    def expected(cls, layer: LayerSpec, hidden_size: int) -> dict:
        names = dict(layer.block["names"])
        out = {}
        out.update(norm_class(layer.norm).expected(layer.norm, hidden_size, names["mixer_norm"]))
        out.update(mixer_class(layer.mixer).expected(layer.mixer, hidden_size))
        ffn_norm = layer.ffn_norm or layer.norm
        second = norm_class(ffn_norm).expected(ffn_norm, hidden_size, names["ffn_norm"])
        if layer.feed_forward is not None:
            out.update(second)
            out.update(feed_forward_class(layer.feed_forward).expected(layer.feed_forward, hidden_size))
        else:        # a checkpoint may carry the second norm all the same; it is unused
            out.update({k: Expected(e.shape, e.init, optional=True) for k, e in second.items()})
        return out

    def bind(self, tensors: dict) -> None:
        self.mixer_norm.bind(tensors[self.names["mixer_norm"]])
        self.mixer.bind(tensors)
        if self.feed_forward is not None:
            self.ffn_norm.bind(tensors[self.names["ffn_norm"]])
            self.feed_forward.bind(tensors)

    def cache_need(self):
        return self.mixer.cache_need()

    def parts(self) -> tuple:
        return tuple(p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward) if p is not None)

    def weights(self):
        for part in self.parts():
            yield from getattr(part, "weights", tuple)()

    def notices(self) -> list:
        return [line for part in self.parts() for line in getattr(part, "notices", list)()]

    @property
    def graph_safe(self) -> bool:
        return all(getattr(part, "graph_safe", False) for part in self.parts())

    def _join(self, x32, y, norm, h_next) -> None:
        """x += norm(y), and the new x rounded for the next reader."""
        w = getattr(norm, "weight", None)
        if isinstance(norm, RMSNorm):
            kernels.norm_add(x32, y, w, norm.eps, h_next)
            return
        normed = torch.empty_like(y)               # another kind of norm: its own kernel, then the sum
        norm.forward(y, normed)
        x32.add_(normed)
        if h_next is not None:
            h_next.copy_(x32)

    def forward(self, x32: torch.Tensor, ctx, cache_view) -> None:
        T, H, ws = x32.shape[0], self.hidden, ctx.workspace
        h = ctx.step_cache.pop(("branch_norm.rounded", x32.data_ptr()), None)
        if h is None:                              # the block in front left no rounded copy of the stream
            h = ws.buffer("branch.input", (T, H), self.dtype)
            kernels.norm_add(x32, None, None, 0.0, h)
        y = ws.buffer("branch.result", (T, H), torch.float32)
        if hasattr(self.mixer, "forward_store"):       # the mixer's last product stores: no cleared buffer
            self.mixer.forward_store(h, ctx, cache_view, y)
        else:
            y.zero_()
            self.mixer.forward(h, ctx, cache_view, y)
        last = self.feed_forward is None
        follows = isinstance(getattr(ctx, "next_block", None), BranchNormBlock)
        self._join(x32, y, self.mixer_norm, h if (not last or follows) else None)
        if not last:
            ff = self.feed_forward
            h_next = h if follows else None
            joined = False
            if isinstance(ff, RoutedExperts):
                if isinstance(self.ffn_norm, RMSNorm):       # the experts' sum, its norm and the addition in one pass
                    joined = ff.forward_join(h, ctx, x32, self.ffn_norm.weight, self.ffn_norm.eps, h_next)
                if not joined:
                    ff.forward_into(h, ctx, y, x32)
            elif hasattr(ff, "forward_into"):
                ff.forward_into(h, ctx, y)
            else:
                y.zero_()
                ff.forward(h, ctx, y)
            if not joined:
                self._join(x32, y, self.ffn_norm, h_next)
        if follows:
            ctx.step_cache[("branch_norm.rounded", x32.data_ptr())] = h


PENDING = "gated_prenorm.owed"        # key of a step's left-over gated addition in StepContext.step_cache


class GatedPreNormBlock:
    """``gated_prenorm``: h = norm(x); x += mixer(h + conv(h)) * sigmoid(G1 h + b1);
    h = norm(x); x += feed_forward(h) * sigmoid(G2 h + b2).

    Each sublayer's result is scaled, element by element, by a gate that is a linear function of
    the sublayer's normed input.  ``conv_taps`` > 0: what the mixer reads is its normed input plus
    a causal convolution of it over time, one filter of that many taps per channel (the gate
    still reads the input as normed).  The last ``conv_taps - 1`` normed rows of a sequence are
    the block's own state: a ring of ``conv_taps`` rows per slot, indexed by position.  A layer
    may have no feed-forward.  Mixers and feed-forwards that offer ``forward_into`` store their
    result for the gate; any other part of the library adds into a cleared buffer instead.
    """

    def __init__(self, layer: LayerSpec, hidden_size: int, dtype: torch.dtype, device):
        self.names = dict(layer.block["names"])
        self.hidden, self.dtype = int(hidden_size), dtype
        self.taps = int(layer.block.get("conv_taps") or 0)
        ffn_norm = layer.ffn_norm or layer.norm
        self.mixer_norm = norm_class(layer.norm)(layer.norm, hidden_size, dtype, device)
        self.mixer = mixer_class(layer.mixer)(layer.mixer, hidden_size, dtype, device)
        self.feed_forward = self.ffn_norm = None
        if layer.feed_forward is not None:
            self.ffn_norm = norm_class(ffn_norm)(ffn_norm, hidden_size, dtype, device)
            self.feed_forward = feed_forward_class(layer.feed_forward)(layer.feed_forward, hidden_size,
                                                                       dtype, device)
        self.w_conv = self.g1 = self.b1 = self.g2 = self.b2 = None
        self._g2_rides = False

    @classmethod
    def expected(cls, layer: LayerSpec, hidden_size: int) -> dict:
        names = dict(layer.block["names"])
        H = int(hidden_size)
        out = {}
        out.update(norm_class(layer.norm).expected(layer.norm, H, names["mixer_norm"]))
        out.update(mixer_class(layer.mixer).expected(layer.mixer, H))
        out[names["mixer_gate"]] = Expected((H, H))
        out[names["mixer_gate_bias"]] = Expected((H,))
        taps = int(layer.block.get("conv_taps") or 0)
        if taps:
            out[names["conv"]] = Expected((H, taps))
        if layer.feed_forward is not None:
            ffn_norm = layer.ffn_norm or layer.norm
            out.update(norm_class(ffn_norm).expected(ffn_norm, H, names["ffn_norm"]))
            out.update(feed_forward_class(layer.feed_forward).expected(layer.feed_forward, H))
            out[names["ffn_gate"]] = Expected((H, H))
            out[names["ffn_gate_bias"]] = Expected((H,))
        else:
            # a checkpoint may carry the second sublayer's norm and gate all the same; they are unused
            out.update({k: Expected(e.shape, e.init, optional=True) for k, e in
                        norm_class(layer.norm).expected(layer.norm, H, names["ffn_norm"]).items()})
            out[names["ffn_gate"]] = Expected((H, H), optional=True)
            out[names["ffn_gate_bias"]] = Expected((H,), optional=True)
        return out

    def bind(self, tensors: dict) -> None:
        n = self.names
        self.mixer_norm.bind(tensors[n["mixer_norm"]])
        self.mixer.bind(tensors)
        self.g1 = tensors[n["mixer_gate"]].contiguous()
        self.b1 = tensors[n["mixer_gate_bias"]].to(torch.float32).contiguous()
        if self.taps:
            # stored [width, taps]; the kernels want a tap's weights side by side: [taps, width]
            self.w_conv = tensors[n["conv"]].to(torch.float32).t().contiguous()
        if self.feed_forward is not None:
            self.ffn_norm.bind(tensors[n["ffn_norm"]])
            self.feed_forward.bind(tensors)
            self.g2 = tensors[n["ffn_gate"]].contiguous()
            self.b2 = tensors[n["ffn_gate_bias"]].to(torch.float32).contiguous()
            # the gate's matrix reads what the feed-forward's first matrix reads: one product
            take = getattr(self.feed_forward, "take_along", None)
            self._g2_rides = bool(take is not None and take(self.g2))

    def cache_need(self):
        need = {"mixer": self.mixer.cache_need()}
        if self.taps > 1:
            need["conv"] = StateNeed((self.taps, self.hidden), self.dtype, by_position=True)
        return need

    def parts(self) -> tuple:
        return tuple(p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward)
                     if p is not None)

    def weights(self):
        for part in self.parts():
            yield from getattr(part, "weights", tuple)()
        for t in (self.w_conv, self.g1, self.b1, self.b2) + (() if self._g2_rides else (self.g2,)):
            if t is not None:
                yield t

    def notices(self) -> list:
        out = [line for part in self.parts() for line in getattr(part, "notices", list)()]
        return out + kernels.product_notices("residual gate", self.g1, self.dtype)

    @property
    def graph_safe(self) -> bool:
        return all(getattr(part, "graph_safe", False) for part in self.parts())

    def forward(self, x32: torch.Tensor, ctx, cache_view) -> None:
        T, H, ws = x32.shape[0], self.hidden, ctx.workspace
        view = cache_view or {}
        h = ws.buffer("gated.normed", (T, H), self.dtype)
        u, keep = h, None
        w1 = getattr(self.mixer_norm, "weight", None)
        plain_norm = isinstance(self.mixer_norm, RMSNorm) and w1 is not None
        # the last gated addition of the block in front, when it left that to this block's first launch
        owed = ctx.step_cache.pop(PENDING, None)
        if self.taps and ctx.all_single and plain_norm:
            # one token per sequence: norm, convolution and the ring's update in one launch
            u = ws.buffer("gated.conv", (T, H), self.dtype)
            ring = view["conv"].states if self.taps > 1 else h
            kernels.norm_canon_single(x32, w1, self.mixer_norm.eps, self.w_conv, ring, ctx, h, u, add=owed)
            owed = None
        elif owed is not None and plain_norm:
            kernels.gated_add(x32, owed[0], owed[1], owed[2], w1, self.mixer_norm.eps, h)
        else:
            if owed is not None:
                kernels.gated_add(x32, *owed)
            self.mixer_norm.forward(x32, h)
        if self.taps and u is h:
            ring = view["conv"].states if self.taps > 1 else h      # one tap: nothing before the token
            u = ws.buffer("gated.conv", (T, H), self.dtype)
            kernels.canon_conv(h, self.w_conv, ring, ctx, u)
            if self.taps > 1:
                keep = (h, ring, self.taps)
        gate = ws.buffer("gated.gate", (T, H), self.dtype)
        kernels.linear(h, self.g1, gate)
        y = ws.buffer("gated.result", (T, H), torch.float32)
        if hasattr(self.mixer, "forward_into"):
            self.mixer.forward_into(u, ctx, view.get("mixer"), y, keep=keep)
        else:
            if keep is not None:
                kernels.latent_keep(None, None, 0.0, None, h, keep[1], self.taps, ctx)
            y.zero_()
            self.mixer.forward(u, ctx, view.get("mixer"), y)
        if self.feed_forward is None:
            self._add_or_leave(ctx, x32, y, gate, self.b1)
            return
        # the feed-forward's norm rides on the gated addition when it is a plain RMS norm
        eps = getattr(self.ffn_norm, "eps", None)
        w2 = getattr(self.ffn_norm, "weight", None)
        if isinstance(self.ffn_norm, RMSNorm) and w2 is not None:
            kernels.gated_add(x32, y, gate, self.b1, w2, eps, h)
        else:
            kernels.gated_add(x32, y, gate, self.b1)
            self.ffn_norm.forward(x32, h)
        ff = self.feed_forward
        if hasattr(ff, "forward_into"):
            ff.forward_into(h, ctx, y)
        else:
            y.zero_()
            ff.forward(h, ctx, y)
        if self._g2_rides:
            gate = ff.side_out
        else:
            kernels.linear(h, self.g2, gate)
        self._add_or_leave(ctx, x32, y, gate, self.b2)

    @staticmethod
    def _add_or_leave(ctx, x32, y, gate, bias) -> None:
        """The block's last gated addition: left to the first launch of the next block of the schedule
        when that is a block of this kind (``StepContext.next_block``, set by the model), which adds
        while it reads the stream for its norm anyway; done here otherwise."""
        if isinstance(getattr(ctx, "next_block", None), GatedPreNormBlock):
            ctx.step_cache[PENDING] = (y, gate, bias)
        else:
            kernels.gated_add(x32, y, gate, bias)


class ParallelShiftBlock:
    """``parallel_shift``: with h = norm(x), x <- x + mixer(hs) + feed_forward(h).  There is one norm;
    the feed-forward reads h as it is, the mixer reads hs_t = h_t + (h_{t-1} - h_t) * mu, mu one learned
    number per channel and h_{t-1} the UNshifted normed row of the token before (zeros in front of a
    sequence's first token).  The normed row of a sequence's latest token is the block's own state
    (one row per slot, 32-bit), whatever the mixer keeps.  A layer may have no feed-forward.  Any
    mixer and feed-forward of the library fit: both add into the stream."""

    def __init__(self, layer: LayerSpec, hidden_size: int, dtype: torch.dtype, device):
        self.names = dict(layer.block["names"])
        self.hidden, self.dtype = int(hidden_size), dtype
        self.norm = norm_class(layer.norm)(layer.norm, hidden_size, dtype, device)
        if not isinstance(self.norm, RMSNorm):
            raise ConfigError("parallel_shift: the norm in front of the token shift is an rmsnorm")
        self.mixer = mixer_class(layer.mixer)(layer.mixer, hidden_size, dtype, device)
        self.feed_forward = None
        if layer.feed_forward is not None:
            self.feed_forward = feed_forward_class(layer.feed_forward)(layer.feed_forward, hidden_size, dtype, device)
        self.mu = None

    @classmethod
    def expected(cls, layer: LayerSpec, hidden_size: int) -> dict:
        names = dict(layer.block["names"])
        out = {names["shift"]: Expected((int(hidden_size),))}
        out.update(norm_class(layer.norm).expected(layer.norm, hidden_size, names["norm"]))
        out.update(mixer_class(layer.mixer).expected(layer.mixer, hidden_size))
        if layer.feed_forward is not None:
            out.update(feed_forward_class(layer.feed_forward).expected(layer.feed_forward, hidden_size))
        return out

    def bind(self, tensors: dict) -> None:
        self.norm.bind(tensors[self.names["norm"]])
        self.mu = tensors[self.names["shift"]].to(torch.float32).contiguous()
        self.mixer.bind(tensors)
        if self.feed_forward is not None:
            self.feed_forward.bind(tensors)

    def cache_need(self):
        need = {"shift": StateNeed((self.hidden,), torch.float32)}
        own = self.mixer.cache_need()
        if isinstance(own, dict):
            need.update({f"mixer.{k}": v for k, v in own.items() if v is not None})
        elif own is not None:
            need["mixer"] = own
        return need

    def parts(self) -> tuple:
        return tuple(p for p in (self.norm, self.mixer, self.feed_forward) if p is not None)

    def weights(self):
        for part in self.parts():
            yield from getattr(part, "weights", tuple)()
        if self.mu is not None:
            yield self.mu

    def notices(self) -> list:
        return [line for part in self.parts() for line in getattr(part, "notices", list)()]

    @property
    def graph_safe(self) -> bool:
        return all(getattr(part, "graph_safe", False) for part in self.parts())

    def forward(self, x32: torch.Tensor, ctx, cache_view) -> None:
        T, H, ws = x32.shape[0], self.hidden, ctx.workspace
        view = cache_view or {}
        h = ws.buffer("shift.normed", (T, H), self.dtype)
        hs = ws.buffer("shift.shifted", (T, H), self.dtype)
        kernels.norm_shift(x32, self.norm.weight, self.mu, view["shift"].states, ctx, self.norm.eps, h, hs)
        own = view.get("mixer")
        if own is None:
            own = {k[len("mixer."):]: v for k, v in view.items() if k.startswith("mixer.")} or None
        self.mixer.forward(hs, ctx, own, x32)
        if self.feed_forward is not None:
            self.feed_forward.forward(h, ctx, x32)


class ParallelScaledBlock:
    """``parallel_scaled``: with h = norm(x), x <- x + (s1 * mixer(h) + s2 * feed_forward(h)); s1 and s2 are
    stored vectors of the model's width (names ``mixer_scale``, ``ffn_scale``), applied to each sublayer's
    whole result in 32-bit before the two are added and join the stream.  A layer may have no feed-forward.
    Any norm, mixer and feed-forward of the library fit: a sublayer stores into a 32-bit buffer of its own
    where it can (``forward_store``, ``forward_into``) and adds into a cleared one where it cannot.  When the
    block behind this one is of the same kind with a ``tanh_norm``, the launch that joins the results to the stream
    also writes that block's normed rows (``StepContext.step_cache`` hands them over)."""

    def __init__(self, layer: LayerSpec, hidden_size: int, dtype: torch.dtype, device):
        self.names = dict(layer.block["names"])
        self.hidden, self.dtype = int(hidden_size), dtype
        self.norm_spec = layer.norm
        self.norm = norm_class(layer.norm)(layer.norm, hidden_size, dtype, device)
        self.mixer = mixer_class(layer.mixer)(layer.mixer, hidden_size, dtype, device)
        self.feed_forward = None
        if layer.feed_forward is not None:
            self.feed_forward = feed_forward_class(layer.feed_forward)(layer.feed_forward, hidden_size, dtype, device)
        self.mixer_scale = self.ffn_scale = None

    @classmethod
    def expected(cls, layer: LayerSpec, hidden_size: int) -> dict:
        names = dict(layer.block["names"])
        out = {names["mixer_scale"]: Expected((int(hidden_size),), init="scale")}
        out.update(norm_class(layer.norm).expected(layer.norm, hidden_size, names["norm"]))
        out.update(mixer_class(layer.mixer).expected(layer.mixer, hidden_size))
        if layer.feed_forward is not None:
            out[names["ffn_scale"]] = Expected((int(hidden_size),), init="scale")
            out.update(feed_forward_class(layer.feed_forward).expected(layer.feed_forward, hidden_size))
        else:        # a checkpoint may carry the second vector all the same; it is unused
            out[names["ffn_scale"]] = Expected((int(hidden_size),), init="scale", optional=True)
        return out

    def bind(self, tensors: dict) -> None:
        bind_norm(self.norm, self.norm_spec, tensors, self.names["norm"])
        self.mixer_scale = tensors[self.names["mixer_scale"]].to(torch.float32).contiguous()
        self.mixer.bind(tensors)
        if self.feed_forward is not None:
            self.ffn_scale = tensors[self.names["ffn_scale"]].to(torch.float32).contiguous()
            self.feed_forward.bind(tensors)

    def cache_need(self):
        return self.mixer.cache_need()

    def parts(self) -> tuple:
        return tuple(p for p in (self.norm, self.mixer, self.feed_forward) if p is not None)

    def weights(self):
        for part in self.parts():
            yield from getattr(part, "weights", tuple)()
        for t in (self.mixer_scale, self.ffn_scale):
            if t is not None:
                yield t

    def notices(self) -> list:
        return [line for part in self.parts() for line in getattr(part, "notices", list)()]

    @property
    def graph_safe(self) -> bool:
        return all(getattr(part, "graph_safe", False) for part in self.parts())

    def forward(self, x32: torch.Tensor, ctx, cache_view) -> None:
        T, H, ws = x32.shape[0], self.hidden, ctx.workspace
        h = ctx.step_cache.pop(("pscaled.normed", x32.data_ptr()), None)
        if h is None:                              # the block in front left no normed rows
            h = ws.buffer("pscaled.normed", (T, H), self.dtype)
            self.norm.forward(x32, h)
        y1 = ws.buffer("pscaled.mixer", (T, H), torch.float32)
        if hasattr(self.mixer, "forward_store"):
            self.mixer.forward_store(h, ctx, cache_view, y1)
        else:
            y1.zero_()
            self.mixer.forward(h, ctx, cache_view, y1)
        y2, ff = None, self.feed_forward
        if ff is not None:
            y2 = ws.buffer("pscaled.ffn", (T, H), torch.float32)
            if hasattr(ff, "forward_into"):
                ff.forward_into(h, ctx, y2)
            else:
                y2.zero_()
                ff.forward(h, ctx, y2)
        nxt = getattr(ctx, "next_block", None)
        if isinstance(nxt, ParallelScaledBlock) and isinstance(nxt.norm, TanhNorm) and nxt.norm.weight is not None:
            # both sublayers have read h by now (stream order): the next block's normed rows take its place
            n = nxt.norm
            kernels.scaled_join(x32, y1, self.mixer_scale, y2, self.ffn_scale, norm=(n.alpha, n.weight, n.bias), normed_out=h)
            ctx.step_cache[("pscaled.normed", x32.data_ptr())] = h
        else:
            kernels.scaled_join(x32, y1, self.mixer_scale, y2, self.ffn_scale)


register_block("prenorm", PreNormBlock)
register_block("parallel_scaled", ParallelScaledBlock)
register_block("parallel_shift", ParallelShiftBlock)
register_block("gated_prenorm", GatedPreNormBlock)
register_block("branch_norm", BranchNormBlock)
