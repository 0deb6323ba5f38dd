"""Plain Movalorn decoder: whole sequences, no cache, one function per mechanism.

Movalorn is a decoder whose embedding adds a row of a hashed table of token pairs to the token's own row; whose
layers put a norm in front of and behind each sublayer and multiply the sublayer's result by a sigmoid gate formed
from the sublayer's input; whose norms have one gain for all channels; whose mixers are either attention through a
low-rank latent with a sliding window, a rotated key part shared by all heads and a gate per head, or a minGRU (a
recurrence whose update gate and candidate come from the step's input alone); whose feed-forwards are a gated tanh-GELU layer or a
mixture of SiLU experts chosen by softmax scores plus a correction, with a shared expert; and in which a run of
layers may be applied several times, each pass entered through a matrix that mixes the stream with the embedding.

Everything runs on the CPU with ordinary tensor operations in the dtype ``work`` (float32 or float64). Nothing here is
imported by the product path and nothing of the product path is imported here. ``cfg`` is the parsed ``config.json``;
``w`` maps checkpoint names to tensors.
"""

from __future__ import annotations

import math

import torch


def rms(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def embedding(ids, w, e):
    """Token row times the scale, plus the row of the pair table that the previous and the current token hash to; a
    sequence's first token takes the table's last row."""
    x = w["embed"][ids] * e["scale"]
    bg = e.get("bigram")
    if bg:
        n = bg["buckets"]
        rows = torch.full_like(ids, n)
        rows[1:] = (ids[:-1] * bg["mul_prev"] + ids[1:] * bg["mul_cur"]) % n
        x = x + w["bigram"][rows]
    return x


def rotate_neighbours(v, positions, base, dims):
    """Turn the first ``dims`` channels of the last axis of ``v`` [tokens, ..., n]: channel 2i pairs with 2i + 1; the
    pair (a, b) at position p becomes (a cos t - b sin t, b cos t + a sin t), t = p * base^(-2i/dims)."""
    half = dims // 2
    i = torch.arange(half, dtype=v.dtype)
    ang = positions.to(v.dtype)[:, None] * (base ** (-2.0 * i / dims))[None, :]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [half]
    cos, sin = ang.cos().reshape(shape), ang.sin().reshape(shape)
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    turned = torch.stack([a * cos - b * sin, b * cos + a * sin], dim=-1).flatten(-2)
    return torch.cat([turned, v[..., dims:]], dim=-1)


def windowed_softmax_attention(q, k, v, scale, window):
    """q, k [tokens, heads, dk], v [tokens, heads, dv]: position i attends to j with 0 <= i - j < window (every j <= i
    when window is 0)."""
    T = q.shape[0]
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = (j <= i) & ((i - j < window) if window else torch.ones(T, T, dtype=torch.bool))
    p = torch.softmax(s.masked_fill(~seen, float("-inf")), dim=-1)
    return torch.einsum("hij,jhd->ihd", p, v)


def latent_attention(h, w, p, m, eps):
    """The attention mixer. ``m``: its sizes from config.json; ``p``: tensor-name prefix ('l3.mix.')."""
    T = h.shape[0]
    H, dn, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    q = (h @ w[p + "q"].T).reshape(T, H, dn + dr)
    dkv = h @ w[p + "dkv"].T
    c = rms(dkv[:, :r], eps) * w[p + "dkv.norm"]
    k_rot = dkv[:, r:r + dr]
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    q_rot = rotate_neighbours(q[..., dn:], pos, base, dims)
    k_rot = rotate_neighbours(k_rot[:, None, :], pos, base, dims).expand(T, H, dr)
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, dn)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    window = (m.get("mask") or {}).get("size", 0)
    o = windowed_softmax_attention(torch.cat([q[..., :dn], q_rot], -1), torch.cat([k_plain, k_rot], -1), v, m["scale"], window)
    o = o * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]          # one gate value per head
    return o.reshape(T, H * dv) @ w[p + "o"].T


def mingru(h, w, p):
    """S_t = (1 - z_t) S_(t-1) + z_t c_t from S = 0, z = sigmoid(W_z h + b_z), c = u + 1/2 where u >= 0 and sigmoid(u)
    below, u = W_x h + b_x; output W_o (S_t * silu(W_g h))."""
    z = torch.sigmoid(h @ w[p + "z"].T + w[p + "z.b"])
    u = h @ w[p + "x"].T + w[p + "x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    s = torch.zeros_like(z[0])
    states = []
    for t in range(h.shape[0]):
        s = (1.0 - z[t]) * s + z[t] * cand[t]
        states.append(s)
    return (torch.stack(states) * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def gated_mlp(h, w, p, act):
    return (act(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def expert_choice(h, w, p, f):
    """(indices [tokens, top], weights [tokens, top], margin [tokens]): the ``top`` experts by softmax score plus
    correction; weights are the uncorrected scores times the router's scale; ``margin`` is the gap between the last
    chosen and the first refused choice score."""
    top = f["router"]["top"]
    s = torch.softmax(h @ w[p + "router"].T, dim=-1)
    pick = s + w[p + "correction"]
    val, idx = torch.sort(pick, dim=-1, descending=True, stable=True)
    margin = val[:, top - 1] - val[:, top] if top < s.shape[-1] else torch.full_like(val[:, 0], float("inf"))
    idx = idx[:, :top]
    return idx, torch.gather(s, 1, idx) * f["router"].get("scale", 1.0), margin


def routed_experts(h, w, p, f, margins=None):
    idx, wt, margin = expert_choice(h, w, p, f)
    if margins is not None:
        margins.append(margin)
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for e in range(f["router"]["experts"]):
        share = (wt * (idx == e)).sum(dim=-1, keepdim=True)
        out = out + share * gated_mlp(h, w, p + f"e{e}.", silu)
    if f.get("shared"):
        out = out + gated_mlp(h, w, p + "shared.", silu)
    return out


def sublayer(x, fn, w, p, k, eps):
    """x + norm_kb(fn(h) * sigmoid(W_rg h + b)), h = norm_k(x); the norms have one gain each."""
    h = rms(x, eps) * w[p + f"norm{k}"]
    y = fn(h) * torch.sigmoid(h @ w[p + f"rg{k}"].T + w[p + f"rg{k}.b"])
    return x + rms(y, eps) * w[p + f"norm{k}b"]


def layer(x, w, i, L, eps, margins=None):
    p = f"l{i}."
    if L["type"] == "latent_attention":
        mix = lambda h: latent_attention(h, w, p + "mix.", L["mixer"], eps)
    elif L["type"] == "mingru":
        mix = lambda h: mingru(h, w, p + "mix.")
    else:
        raise ValueError(f"layer {i}: unknown mixer {L['type']!r}")
    x = sublayer(x, mix, w, p, 1, eps)
    f = L.get("mlp")
    if f is None:
        return x
    if f["kind"] == "dense":
        ff = lambda h: gated_mlp(h, w, p + "mlp.", gelu_tanh)
    elif f["kind"] == "moe":
        ff = lambda h: routed_experts(h, w, p + "mlp.", f, margins)
    else:
        raise ValueError(f"layer {i}: unknown feed-forward {f['kind']!r}")
    return sublayer(x, ff, w, p, 2, eps)


def layer_runs(cfg):
    """The order in which layers are applied: [(layer index, pass number or None, first of its pass)]."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or loop["stop"] <= loop["start"]:
        return [(i, None, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, None, False) for i in range(a)]
    for t in range(times):
        runs += [(i, t, i == a) for i in range(a, b)]
    runs += [(i, None, False) for i in range(b, n)]
    return runs


def forward(cfg, w, tokens, work=torch.float64, keep_stream=False, margins=None):
    """Logits [tokens, vocab] of one sequence (and, if asked, the stream after every layer application). ``margins``: a
    list that receives, for every run of a layer with experts, by how much each token's choice of experts was clear."""
    w = {k: (v.to(work) if v.is_floating_point() else v) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x0 = embedding(ids, w, cfg["embedding"])
    x = x0
    kept = []
    for i, t, first in layer_runs(cfg):
        if first:
            x = torch.cat([x, x0], dim=-1) @ w["loop.in"].T + w["loop.step"][t]
        x = layer(x, w, i, cfg["layers"][i], eps, margins)
        kept.append(x)
    logits = (rms(x, eps) * w["final.norm"]) @ w["head"].T * cfg.get("logit_scale", 1.0)
    return (logits, torch.stack(kept)) if keep_stream else logits


def greedy_generate(cfg, w, prompt, n, work=torch.float64):
    """The ``n`` tokens that always taking the largest logit gives after ``prompt`` (the whole sequence is run again
    for every token: slow and plain)."""
    seq, out = list(prompt), []
    for _ in range(n):
        tok = int(torch.argmax(forward(cfg, w, seq, work)[-1]))
        out.append(tok)
        seq.append(tok)
    return out
