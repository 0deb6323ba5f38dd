"""Position encodings of queries and keys.

``rotary``: pairs of channels turn by the angle position * theta^(-2i/rot) of pair i; which channels form pair i
(i and i + rot/2, or 2i and 2i + 1) is the spec's ``pairing``, which the kernels are told; the tables are the same. The cos and
sin tables ``[positions, rot/2]`` are built once, on the host, in float32, with the reference's own
order of operations (sleuth/forge/model/rope.py:30-38: ``1 / theta ** (arange(0, rot, 2) / rot)``,
``outer(positions, inv_freq)``), so the angles are the reference's to the bit. The kernels that
apply them live in ``csrc/qkv_post.cu``. With ``precise`` the angles and their cosines and sines are worked out in
64-bit and rounded to float32 once. ``scaling`` rescales the frequencies band by band (``rescale_bands``).
``none``: no tables, nothing is rotated.
"""

from __future__ import annotations

import torch

from .base import BuildContext, Part, register_position
from .spec import PositionSpec


class Rotary(Part):
    def __init__(self, spec: PositionSpec, ctx: BuildContext):
        self.rot_dim = spec.rotary_dim or spec.head_dim
        if self.rot_dim % 2 or self.rot_dim > spec.head_dim:
            raise ValueError(f"rotary_dim {self.rot_dim} must be even and at most head_dim {spec.head_dim}")
        if spec.pairing not in ("halves", "neighbours"):
            raise ValueError(f"rotary pairing {spec.pairing!r} is not 'halves' or 'neighbours'")
        self.neighbours = spec.pairing == "neighbours"
        work = torch.float64 if spec.precise else torch.float32
        inv_freq = 1.0 / (spec.theta ** (torch.arange(0, self.rot_dim, 2, dtype=work) / self.rot_dim))
        if spec.scaling:
            inv_freq = rescale_bands(inv_freq, *spec.scaling)
        pos = torch.arange(ctx.max_positions, dtype=work)
        ang = torch.outer(pos, inv_freq)                       # [positions, rot/2]
        self.cos = ang.cos().to(torch.float32).contiguous().to(ctx.device)
        self.sin = ang.sin().to(torch.float32).contiguous().to(ctx.device)

    def tables(self):
        return self.cos, self.sin


def rescale_bands(f: torch.Tensor, factor: float, low: float, high: float, original: float) -> torch.Tensor:
    """Frequencies rescaled band by band: with wavelength l = 2 pi / f, f stays where l < original / high, becomes
    f / factor where l > original / low, and between the two (1 - s) f / factor + s f, s = (original / l - low) / (high - low)."""
    if not (factor > 0 and high > low and original > 0):
        raise ValueError(f"frequency scaling: factor {factor}, low {low}, high {high}, original {original}")
    wavelength = 2.0 * torch.pi / f
    s = (original / wavelength - low) / (high - low)
    between = (1.0 - s) * f / factor + s * f
    return torch.where(wavelength < original / high, f, torch.where(wavelength > original / low, f / factor, between))


class NoPosition(Part):
    rot_dim = 0
    neighbours = False

    def __init__(self, spec, ctx: BuildContext):
        pass

    def tables(self):
        return None


register_position("rotary", Rotary)
register_position("none", NoPosition)
