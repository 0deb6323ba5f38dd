"""Tiny Fekitar configurations of the tests. They differ in every size and option: width, vocabulary, eps, the number of
copies of the stream (0 = a plain residual, 1, 3, 5) and the residual multiplier; 'parallel' layers with windows shorter
than a page, of exactly a page, of a page and one, of one token, and longer than any test sequence, convolutions of 2 to 5
taps (and a recurrence without one), 1 to 6 query heads on 1 to 3 key/value heads, key and value widths equal and unequal,
state sizes 8 to 72 (all register tilings of the recurrence kernel), one group or one a head, one to four norm groups;
'parallel_2' layers with whole and partial rotation, with and without band-wise frequency scaling, soft caps, decay ranks
and time constants; differential attention with and without convolution, whole, partial and no rotation, layers that
borrow keys and values (one owner lending to two layers); experts with top 1, 2, 3 and all, one expert, with and without
shared expert, and layers without feed-forward; every order of the three mixers."""

from __future__ import annotations


def att(heads, kv, dim, vdim, scale=None, conv=0, window=0, rot=None, softcap=0.0, diff=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if conv:
        m["conv"] = conv
    if window:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = rot
    if softcap:
        m["softcap"] = softcap
    if diff is not None:
        m["diff"] = diff
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def mamba(heads, vdim, state, groups=1, conv=4, norm_groups=1):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def gla(heads, dim, vdim, tau, rank):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}


def moe(experts, top, ff, limit=1.5, shared=None, shared_limit=2.0):
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared:
        out["shared"] = {"ff": shared, "limit": shared_limit}
    return out


def par(left, right, mlp):
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}


def par2(left, right, ls, rs, mlp):
    return {"type": "parallel_2", "mixer": {"left": left, "right": right, "left_scale": ls, "right_scale": rs}, "mlp": mlp}


def diff(m, mlp):
    return {"type": "attention", "mixer": m, "mlp": mlp}


SCALED = {"base": 500.0, "dims": 16, "scaling": {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 64}}

# odd sizes everywhere (the general kernels); three copies of the stream; a window shorter than a page; an owner of keys
# that lends to the last layer; a layer without feed-forward
R = {"architecture": "Fekitar", "vocab": 211, "width": 72, "norm": {"eps": 1e-5}, "residual_mult": 0.8, "streams": 3,
     "layers": [par(att(4, 2, 16, 24, conv=3, window=37), mamba(3, 16, 12, groups=1, conv=2, norm_groups=3), moe(5, 2, 36, shared=28)),
                par2(att(6, 3, 24, 16, scale=0.2, rot=SCALED, softcap=6.0), gla(3, 8, 20, 8.0, 5), 1.3, 0.6, moe(6, 1, 20)),
                diff(att(2, 1, 16, 40, conv=4, rot={"base": 100.0, "dims": 8}, diff=0.3), None),
                par(att(2, 1, 8, 8, conv=5, window=64), mamba(4, 8, 40, groups=4, conv=3, norm_groups=1), moe(4, 4, 16, limit=0.7, shared=24, shared_limit=1.1)),
                diff(att(2, 1, 16, 40, conv=2, rot={"base": 100.0, "dims": 8}, diff=0.3, kv_from=2), moe(3, 3, 12))]}

# no copies at all (a plain residual with a multiplier); widths that send bfloat16 prompts through the tensor-memory
# products and single tokens through the weight-streaming kernel; the differential attention first, lending to two layers;
# a window of a page and one; whole rotation without scaling; one key/value head a query head; both one-map attentions
# have keys and values of 64 channels, which in bfloat16 sends them through the tensor-core attention kernels
S = {"architecture": "Fekitar", "vocab": 320, "width": 256, "norm": {"eps": 1e-6}, "residual_mult": 1.0,
     "layers": [diff(att(4, 2, 32, 64, rot={"base": 10000.0, "dims": 32}, diff=0.5), moe(8, 2, 64, shared=128)),
                par2(att(4, 4, 64, 64, rot={"base": 10000.0, "dims": 64}, softcap=30.0), gla(2, 72, 32, 16.0, 8), 0.7, 1.4, moe(8, 3, 64, limit=3.0)),
                diff(att(4, 2, 32, 64, conv=3, rot={"base": 10000.0, "dims": 32}, diff=0.5, kv_from=0), None),
                par(att(4, 2, 64, 64, conv=4, window=65), mamba(4, 32, 72, groups=2, conv=4, norm_groups=2), moe(8, 2, 64, shared=64)),
                diff(att(4, 2, 32, 64, rot={"base": 10000.0, "dims": 32}, diff=0.5, kv_from=0), moe(1, 1, 40, shared=32))]}

# one copy of the stream with coefficients; a window of one token (a token sees itself alone) and one longer than any
# test sequence; a recurrence without convolution; differential attention without rotation; five copies in V below
U = {"architecture": "Fekitar", "vocab": 150, "width": 96, "norm": {"eps": 2e-5}, "residual_mult": 0.5, "streams": 1,
     "layers": [par(att(1, 1, 32, 16, conv=2, window=1), mamba(2, 24, 8, groups=2, conv=1, norm_groups=2), moe(4, 2, 24, shared=16)),
                diff(att(3, 3, 8, 16, conv=3, diff=0.0), moe(5, 3, 20, limit=1.0)),
                par(att(6, 3, 16, 16, conv=4, window=5000), mamba(6, 16, 17, groups=3, conv=5, norm_groups=4), None),
                par2(att(2, 1, 16, 48, scale=0.3), gla(1, 32, 96, 2.0, 3), 1.0, 1.0, moe(2, 1, 32, shared=48))]}

V = {"architecture": "Fekitar", "vocab": 97, "width": 64, "norm": {"eps": 1e-6}, "residual_mult": 1.2, "streams": 5,
     "layers": [par2(att(2, 2, 16, 16, rot={"base": 50.0, "dims": 16}, softcap=4.0), gla(4, 16, 16, 4.0, 16), 0.9, 1.1, None),
                par(att(2, 2, 16, 32, conv=2, window=63), mamba(1, 64, 33, groups=1, conv=4, norm_groups=1), moe(3, 2, 24, shared=8))]}

CONFIGS = {"R": R, "S": S, "U": U, "V": V}
SEEDS = {"R": 171, "S": 272, "U": 373, "V": 474}
STD = 0.08      # wide enough that attention is far from uniform and the experts' shares differ


def sharpen(folder, logit_std: float = 3.0) -> None:
    """Rewrite a written folder so that faults show: the routers' rows are scaled until their logits have about
    ``logit_std`` (the choice then changes from token to token and two scores seldom lie closer than a bfloat16 run's
    rounding); the copies' mixing matrices become the identity plus noise (a drawn matrix near zero would let the copies
    die out); the recurrences forget slowly (small step sizes, decays near one), so that a state that is lost, or starts
    from another sequence's, shows far behind the place where it happened; the differential attention's four vectors are
    large enough that its learned number is not just ``diff``."""
    from pathlib import Path

    import torch

    from plain.qwen3_plain import read_safetensors
    from sleuth_b200.weights.safetensors import write_safetensors
    path = Path(folder) / "model.safetensors"
    tensors = read_safetensors(path)
    for name, t in tensors.items():
        if name.endswith(".mlp.router"):
            tensors[name] = t * (logit_std / (float(t.float().std()) * t.shape[1] ** 0.5))
        elif name.endswith(".mix"):
            tensors[name] = torch.eye(t.shape[0], dtype=t.dtype) + 2.0 * t
        elif name.endswith(".dt_bias"):
            tensors[name] = t - 2.5
        elif name.endswith(".a2.b"):
            tensors[name] = t + 2.0
        elif name.endswith((".lq1", ".lk1", ".lq2", ".lk2")):
            tensors[name] = t * 2.0
        elif name.endswith(".shared.sg"):
            tensors[name] = t * 4.0
    write_safetensors(tensors, path, metadata={"format": "pt"})
