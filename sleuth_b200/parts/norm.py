"""Normalisation parts. ``rmsnorm``: y = x * rsqrt(mean(x^2) + eps) * gain, float32 arithmetic on the
float32 stream, output in the run dtype (sleuth/forge/model/norm.py:34-50). ``layernorm``: y = (x - mean) /
sqrt(var + eps) * gain with var the mean of the squared deviations and no bias, the same way. A norm whose spec says
``gain="scalar"`` reads one number from the weight file and uses it for every channel."""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import BuildContext, ParamDecl, Part, register_norm
from .spec import NormSpec


def _gain_shape(spec: NormSpec) -> tuple:
    if spec.gain not in ("vector", "scalar"):
        raise ValueError(f"a norm's gain is 'vector' or 'scalar', not {spec.gain!r}")
    return () if spec.gain == "scalar" else (spec.dim,)


def _gain_vector(t: torch.Tensor, dim: int) -> torch.Tensor:
    """The gain as the kernels read it: one float32 value per channel (a scalar gain is repeated)."""
    return t.reshape(1).expand(dim).contiguous() if t.dim() == 0 or t.numel() == 1 and dim != 1 else t


class RMSNorm(Part):
    fusable = True      # a product kernel may apply this norm itself from ``weight`` and ``eps``

    def __init__(self, spec: NormSpec, ctx: BuildContext):
        self.dim, self.eps, self.dtype = spec.dim, spec.eps, ctx.dtype
        self.gain_shape = _gain_shape(spec)
        self.weight = None

    def declare(self):
        return {"weight": ParamDecl(self.gain_shape, "vector", init="gain")}

    def bind(self, tensors):
        self.weight = _gain_vector(tensors["weight"], self.dim)

    def fused_decode(self):
        return {"gain": self.weight, "eps": self.eps} if self.weight is not None else None

    def forward(self, x: torch.Tensor, out: torch.Tensor, rows: torch.Tensor | None = None, stream=None):
        """out[r] = norm(x[rows[r]]) (or x[r] without ``rows``); ``out`` has the run dtype."""
        ops.rmsnorm(x, self.weight, out, self.eps, rows, stream)
        return out


class LayerNorm(Part):
    """Layer norm with a gain and no bias. ``out`` may be float32 (and the stream itself: a row is read whole before it
    is written)."""
    fusable = False

    def __init__(self, spec: NormSpec, ctx: BuildContext):
        self.dim, self.eps, self.dtype = spec.dim, spec.eps, ctx.dtype
        self.gain_shape = _gain_shape(spec)
        self.weight = None

    def declare(self):
        return {"weight": ParamDecl(self.gain_shape, "vector", init="gain")}

    def bind(self, tensors):
        self.weight = _gain_vector(tensors["weight"], self.dim)

    def forward(self, x: torch.Tensor, out: torch.Tensor, rows: torch.Tensor | None = None, stream=None):
        ops.layernorm(x, self.weight, out, self.eps, rows, stream)
        return out

    def forward_with(self, other, x: torch.Tensor, out: torch.Tensor, out_other: torch.Tensor, stream=None) -> bool:
        """This norm and ``other`` of the same rows in one pass, when they differ in their gains only (mean and variance
        are then the same); False when they do not, and nothing has run."""
        if not (isinstance(other, LayerNorm) and other.eps == self.eps and other.dim == self.dim):
            return False
        ops.layernorm(x, self.weight, out, self.eps, None, stream, w2=other.weight, out2=out_other)
        return True


register_norm("rmsnorm", RMSNorm)
register_norm("layernorm", LayerNorm)
