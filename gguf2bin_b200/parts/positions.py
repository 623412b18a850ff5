"""Position encodings applied to queries and keys before the keys are cached.

``rope_neox``: half-split rotation, pairs (j, j + r/2) of the first r = rotary_dim
dimensions of each head, angle = pos * theta^(-2j/r) in float32
(src/l3_math.c:84-102 of AnonymoDGH/gguf2bin; r = head_dim there).  The frequencies
are a table handed to the fused norm+rotation kernel, so another encoding that only
changes the frequencies needs no kernel of its own.
``rope_interleaved``: the same angles on neighbouring pairs (2j, 2j + 1).  No fused kernel takes
that layout, so a mixer runs it as a step of its own (``apply``) or hands ``table_rotation()`` to
a kernel that knows both layouts.
``rope_stretched``: the half-split rotation with its slow pairs slowed further, for sequences
longer than the ``original`` length: with pair(t) = r ln(original / (2 pi t)) / (2 ln theta) the pair
index that makes t turns over ``original`` positions, lo = max(floor(pair(fast)), 0),
hi = min(ceil(pair(slow)), r - 1) and ramp_j = clamp((j - lo) / max(hi - lo, 0.001), 0, 1), pair j
turns at f_j (1 - ramp_j) + (f_j / factor) ramp_j, and cos and sin are both multiplied by
0.1 ln(factor) + 1 (``mult``; the step's table carries it).  With ``interleaved`` the same frequencies
turn neighbouring pairs (2j, 2j + 1).
``none``: nothing is applied.
"""
from __future__ import annotations

import torch

from ..config.specs import ConfigError, PartSpec
from .registry import register_position


_INV_FREQ: dict = {}


class RopeNeox:
    graph_safe = True          # its step only launches kernels: may be replayed from a CUDA graph

    def __init__(self, spec: PartSpec, head_dim: int, device):
        self.theta = float(spec["theta"])
        self.head_dim = int(head_dim)
        self.rotary_dim = int(spec.get("rotary_dim") or head_dim)
        if self.rotary_dim % 2 or not (0 < self.rotary_dim <= head_dim):
            raise ConfigError(f"rope_neox: rotary_dim {self.rotary_dim} must be even and at most "
                              f"head_dim {head_dim}")
        # one table per (theta, rotary_dim, device): layers with equal frequencies share the tensor,
        # and with it the step's (cos, sin) table
        key = (self.theta, self.rotary_dim, str(device))
        if key not in _INV_FREQ:
            j = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
            _INV_FREQ[key] = (self.theta ** (-2.0 * j / self.rotary_dim)).to(torch.float32).to(device)
        self.inv_freq = _INV_FREQ[key]

    interleaved = False
    mult = 1.0                 # what cos and sin are multiplied by (the step's table carries it)

    def fused_rotation(self):
        return self.inv_freq, self.rotary_dim

    def table_rotation(self):
        """(inv_freq, rotary_dim, interleaved) for kernels that rotate from the step's (cos, sin)
        table in either pair layout."""
        return self.inv_freq, self.rotary_dim, self.interleaved

    def apply(self, q, k, ctx) -> None:
        """Rotates q [T, heads*head_dim] and k in place.  The library's own mixer never comes
        here (it hands ``fused_rotation()`` to its fused kernel); a mixer that runs its
        position part as a step of its own does.  The rotation is that same kernel's, asked
        for nothing but the rotation."""
        from .. import kernels
        rope = ctx.rope_table(self.inv_freq)
        for i, a in enumerate((q, k)):
            if a is None or a.numel() == 0:
                continue
            out = ctx.workspace.buffer(f"rope.apply.{i}", tuple(a.shape), a.dtype)
            kernels.qknorm_rope_cache(a, a.shape[1] // self.head_dim, 0, self.head_dim, None, None,
                                      0.0, rope, self.rotary_dim, ctx.tok_pos, ctx.tok_seq, None,
                                      None, ctx.page_size, out)
            a.copy_(out)


class RopeStretched(RopeNeox):
    """Half-split pairs whose frequencies are divided by ``factor`` along a ramp over the pair index."""

    def __init__(self, spec: PartSpec, head_dim: int, device):
        super().__init__(spec, head_dim, device)
        factor, original = float(spec["factor"]), float(spec["original"])
        fast, slow = float(spec["fast"]), float(spec["slow"])
        if not (factor > 0 and original > 0 and fast > 0 and slow > 0 and self.theta > 1.0):
            raise ConfigError("rope_stretched: factor, original, fast and slow must be positive, theta above 1")
        key = (self.theta, self.rotary_dim, str(device), factor, original, fast, slow)
        if key not in _INV_FREQ:
            import math
            r = self.rotary_dim

            def pair(turns):
                return r * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))
            lo, hi = max(math.floor(pair(fast)), 0), min(math.ceil(pair(slow)), r - 1)
            j = torch.arange(r // 2, dtype=torch.float64)
            f = self.theta ** (-2.0 * j / r)
            ramp = ((j - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
            _INV_FREQ[key] = (f / factor * ramp + f * (1.0 - ramp)).to(torch.float32).to(device)
        self.inv_freq = _INV_FREQ[key]
        import math
        self.mult = 0.1 * math.log(factor) + 1.0
        self.interleaved = bool(spec.get("interleaved") or False)

    def fused_rotation(self):
        if self.mult != 1.0 or self.interleaved:       # the fused kernel's table has no factor, its pairs are (j, j + r/2)
            return None
        return self.inv_freq, self.rotary_dim

    def apply(self, q, k, ctx) -> None:
        from .. import kernels
        rope = ctx.rope_table(self.inv_freq, self.mult)
        for a in (q, k):
            if a is not None and a.numel():
                kernels.rotate_heads(a, a.shape[1] // self.head_dim, self.head_dim, rope, self.rotary_dim,
                                     self.interleaved)


class RopeInterleaved(RopeNeox):
    """Pairs (2j, 2j + 1) of the first ``rotary_dim`` entries of each head."""
    interleaved = True

    def fused_rotation(self):
        return None                               # the fused norm + rotation kernel pairs (j, j + r/2)

    def apply(self, q, k, ctx) -> None:
        from .. import kernels
        rope = ctx.rope_table(self.inv_freq)
        for a in (q, k):
            if a is not None and a.numel():
                kernels.rotate_heads(a, a.shape[1] // self.head_dim, self.head_dim, rope, self.rotary_dim, True)


class NoPosition:
    graph_safe = True          # its step only launches kernels: may be replayed from a CUDA graph

    def __init__(self, spec: PartSpec, head_dim: int, device):
        pass

    def fused_rotation(self):
        return None, 0                           # fused path with no rotation

    def table_rotation(self):
        return None, 0, False

    def apply(self, q, k, ctx) -> None:
        pass


register_position("rope_neox", RopeNeox)
register_position("rope_interleaved", RopeInterleaved)
register_position("rope_stretched", RopeStretched)
register_position("none", NoPosition)
