"""Tiny Movalorn configurations of the tests. They differ in every size and option: width, vocabulary, the pair table's
buckets and multipliers, embedding and logit scales, norm eps; attention layers with 1, 3, 5, 6 and 40 heads, key and
value widths equal and unequal, latent ranks that the tensor-core kernel takes (multiples of 16) and ranks it does not,
windows shorter than a page, of exactly a page, longer than a page, longer than any test sequence, and none; minGRU
layers narrower and wider than the model; dense, routed (top 1, 2, 3, all; one expert; with and without a shared expert) and absent
feed-forwards in different orders; the loop over the first layers three times, over two inner layers twice, over one
layer once, over four layers four times, and absent; recurrent layers only and attention layers only (windows of 1 and 2
tokens among them)."""

from __future__ import annotations


def attention(heads, dim, rot_dim, vdim, kv_rank, window, base=10000.0, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5, "rot": {"base": base, "dims": rot_dim}}
    if window:
        m["mask"] = {"size": window}
    return m


def gru(width):
    return {"width": width}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, scale=1.0, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def layer(kind, m, f):
    return {"type": kind, "mixer": m, "mlp": f}


A, G = "latent_attention", "mingru"

# attention first, odd sizes everywhere (the general kernels), a window shorter than a page, a layer without feed-forward
K = {"architecture": "Movalorn", "vocab": 301, "width": 72, "norm": {"eps": 1e-6}, "logit_scale": 0.5,
     "embedding": {"scale": 3.0, "bigram": {"buckets": 97, "mul_prev": 7, "mul_cur": 13}},
     "layers": [layer(A, attention(3, 16, 8, 24, 40, 37, base=500.0, scale=0.31), dense(100)),
                layer(G, gru(52), moe(5, 2, 36, scale=1.5, shared=28)),
                layer(A, attention(5, 8, 4, 12, 20, 0, base=50.0), None),
                layer(G, gru(100), moe(6, 1, 20, scale=0.7))],
     "loop": {"start": 1, "stop": 3, "times": 2}}

# the loop starts at layer 0 and runs three times; sizes the tensor-core latent kernel takes; a window of exactly a page
L = {"architecture": "Movalorn", "vocab": 257, "width": 128, "norm": {"eps": 2e-5}, "logit_scale": 2.0,
     "embedding": {"scale": 1.0, "bigram": {"buckets": 1031, "mul_prev": 1, "mul_cur": 257}},
     "layers": [layer(G, gru(192), moe(8, 3, 48, scale=2.5, shared=64)),
                layer(A, attention(6, 32, 16, 32, 64, 64, base=20000.0), dense(192))],
     "loop": {"start": 0, "stop": 2, "times": 3}}

# one head and forty heads (more than a block of the attention kernels takes at once); all experts chosen; no loop; a
# window longer than any sequence of the tests; no pair table
M = {"architecture": "Movalorn", "vocab": 203, "width": 64, "norm": {"eps": 1e-5},
     "embedding": {"scale": 0.5},
     "layers": [layer(A, attention(1, 16, 16, 8, 24, 5000), dense(48)),
                layer(A, attention(40, 8, 4, 8, 28, 9, base=100.0), moe(4, 4, 16, scale=0.25, shared=24)),
                layer(G, gru(64), None)]}

# sizes that send prompts of 128 tokens and more through the tensor-memory products, single tokens through the
# weight-streaming kernel and whole prompts through the per-head attention kernel; windows of 100 and 130 tokens (two
# cache groups); a loop over one layer, once
N = {"architecture": "Movalorn", "vocab": 640, "width": 384, "norm": {"eps": 1e-6}, "logit_scale": 0.125,
     "embedding": {"scale": 4.0, "bigram": {"buckets": 4099, "mul_prev": 641, "mul_cur": 3}},
     "layers": [layer(G, gru(256), dense(640)),
                layer(A, attention(4, 64, 32, 48, 128, 100), moe(8, 2, 128, scale=1.25, shared=192)),
                layer(G, gru(512), moe(8, 2, 128, scale=1.0)),
                layer(A, attention(6, 32, 32, 64, 96, 130, base=1000.0), dense(256))],
     "loop": {"start": 2, "stop": 3, "times": 1}}

# recurrent layers only (the cache holds no pages at all, only states), one of them without feed-forward, both in a loop
# that runs twice
P = {"architecture": "Movalorn", "vocab": 150, "width": 96, "norm": {"eps": 1e-5}, "logit_scale": 0.7,
     "embedding": {"scale": 2.0, "bigram": {"buckets": 53, "mul_prev": 5, "mul_cur": 11}},
     "layers": [layer(G, gru(64), dense(128)), layer(G, gru(160), None)],
     "loop": {"start": 0, "stop": 2, "times": 2}}

# attention layers only, with the smallest windows (1: a token sees itself alone; 2) beside windows of a page less one, a
# page and one, and two pages, four of the layers in a loop of four passes; one expert of which one is chosen; pair-table
# multipliers whose products do not fit 32 bits
Q = {"architecture": "Movalorn", "vocab": 150, "width": 96, "norm": {"eps": 1e-5},
     "embedding": {"scale": 1.0, "bigram": {"buckets": 200003, "mul_prev": 1000003, "mul_cur": 999983}},
     "layers": [layer(A, attention(4, 16, 8, 16, 32, 1), moe(1, 1, 40, scale=1.5, shared=24)),
                layer(A, attention(2, 32, 16, 24, 48, 2), None),
                layer(A, attention(4, 16, 16, 16, 32, 65), moe(4, 2, 32, scale=1.0, shared=32)),
                layer(A, attention(4, 16, 16, 16, 32, 63), None),
                layer(A, attention(4, 16, 16, 16, 32, 128), None)],
     "loop": {"start": 1, "stop": 5, "times": 4}}

CONFIGS = {"K": K, "L": L, "M": M, "N": N, "P": P, "Q": Q}
SEEDS = {"K": 151, "L": 252, "M": 353, "N": 454, "P": 555, "Q": 656}
STD = 0.08      # wide enough that attention is far from uniform and the experts' shares differ


def sharpen(folder, logit_std: float = 3.0) -> None:
    """Rewrite a written folder so that faults show: the routers' rows are scaled until their logits have about
    ``logit_std`` (the scores then differ clearly between experts and from token to token, so that the choice changes
    and two choice scores seldom lie closer than a bfloat16 run's rounding), the corrections become distinct multiples of
    0.04 in a shuffled order (two experts whose scores are both small are then told apart by a clear margin, and a
    correction that is left out or also enters the weights shows), and the recurrences' gate biases are pushed
    down a little so that a state remembers over dozens of tokens (a state that is lost, or starts from another
    sequence's, then shows far behind the place where it happened)."""
    from pathlib import Path

    from plain.qwen3_plain import read_safetensors
    from sleuth_b200.weights.safetensors import write_safetensors
    path = Path(folder) / "model.safetensors"
    tensors = read_safetensors(path)
    for name, t in tensors.items():
        if name.endswith(".mlp.router"):
            tensors[name] = t * (logit_std / (float(t.float().std()) * t.shape[1] ** 0.5))
        elif name.endswith(".mlp.correction"):
            import torch
            g = torch.Generator().manual_seed(t.numel())
            tensors[name] = (torch.randperm(t.numel(), generator=g).to(t.dtype) - (t.numel() - 1) / 2) * 0.04
        elif name.endswith(".mix.z.b"):
            tensors[name] = t - 2.0
    write_safetensors(tensors, path, metadata={"format": "pt"})
