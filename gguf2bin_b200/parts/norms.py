"""Norms.  ``rmsnorm``: o_j = (w_j * x_j) / sqrt(mean(x^2) + eps), statistics in float32,
the weight a plain multiplier (src/l3_math.c:21-51 of AnonymoDGH/gguf2bin).  With ``offset`` the
stored tensor is the weight's distance from that number (a checkpoint that keeps its norm
weights around zero has ``offset`` 1): the multiplier is ``offset + stored``, added once, in
32-bit, when the weights are bound.
``tanh_norm``: o_j = tanh(alpha * x_j) * w_j + b_j with one learned number alpha: no mean, no variance,
nothing summed over the row.  Its three tensors are ``<name>``, ``<name><bias_suffix>`` and
``<name><alpha_suffix>`` (suffixes ".b" and ".alpha" unless the spec says otherwise); a block binds it
through ``bind_norm``, which hands a norm with more than one tensor all of them."""
from __future__ import annotations

import torch

from .. import kernels
from ..config.specs import PartSpec
from ..weights.loader import Expected
from .registry import register_norm


class RMSNorm:
    graph_safe = True          # its step only launches kernels: may be replayed from a CUDA graph

    def __init__(self, spec: PartSpec, width: int, dtype: torch.dtype, device):
        self.eps = float(spec["eps"])
        self.width = int(width)
        self.offset = float(spec.get("offset") or 0.0)
        self.weight = None

    @classmethod
    def expected(cls, spec: PartSpec, width: int, name: str) -> dict:
        # a weight stored as a distance from ``offset`` is spread around zero
        return {name: Expected((int(width),), init="scale" if not spec.get("offset") else "matrix")}

    def bind(self, weight: torch.Tensor) -> None:
        self.weight = weight.to(torch.float32).contiguous()      # exact widening
        if self.offset:
            self.weight = (self.weight + self.offset).contiguous()

    def weights(self):
        return (self.weight,) if self.weight is not None else ()

    # ---- the weight moved into the matrix that follows ----------------------------------
    def give_up_weight(self) -> torch.Tensor:
        """Hands the per-channel weight to a part that multiplies it into the columns of its
        first matrix (W' = W . diag(w), so that W' . x/rms(x) = W . (w * x/rms(x))); from
        then on this norm only divides by the root mean square."""
        w, self.weight = self.weight, None
        return w

    def plain_rms_eps(self):
        """eps when this norm is x / sqrt(mean(x^2) + eps) and nothing else (its weight was
        given up), which is what the products that normalise their own input take; else None."""
        return self.eps if self.weight is None else None

    def forward(self, x32: torch.Tensor, out: torch.Tensor, rows=None) -> None:
        kernels.rmsnorm(x32, self.weight, self.eps, out, rows)


class TanhNorm:
    graph_safe = True

    def __init__(self, spec: PartSpec, width: int, dtype: torch.dtype, device):
        self.width = int(width)
        self.weight = self.bias = self.alpha = None

    @staticmethod
    def _names(spec: PartSpec, name: str):
        return name, name + (spec.get("bias_suffix") or ".b"), name + (spec.get("alpha_suffix") or ".alpha")

    @classmethod
    def expected(cls, spec: PartSpec, width: int, name: str) -> dict:
        w, b, a = cls._names(spec, name)
        return {w: Expected((int(width),), init="scale"), b: Expected((int(width),)), a: Expected((), init="scale")}

    def bind_named(self, spec: PartSpec, tensors: dict, name: str) -> None:
        w, b, a = self._names(spec, name)
        self.weight = tensors[w].to(torch.float32).contiguous()
        self.bias = tensors[b].to(torch.float32).contiguous()
        self.alpha = tensors[a].to(torch.float32).reshape(1).contiguous()      # stays on the device: read by the kernel

    def weights(self):
        return tuple(t for t in (self.weight, self.bias, self.alpha) if t is not None)

    def forward(self, x32: torch.Tensor, out: torch.Tensor, rows=None) -> None:
        kernels.tanh_norm(x32, self.alpha, self.weight, self.bias, out, rows)


def bind_norm(norm, spec: PartSpec, tensors: dict, name: str) -> None:
    """Hands a norm its tensors: the one called ``name``, or, for a norm that has several
    (``bind_named``), all that it listed under that name."""
    if hasattr(norm, "bind_named"):
        norm.bind_named(spec, tensors, name)
    else:
        norm.bind(tensors[name])


register_norm("rmsnorm", RMSNorm)
register_norm("tanh_norm", TanhNorm)
