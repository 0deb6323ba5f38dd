"""Plain Fekitar decoder: whole sequences, no cache, one function per mechanism.

Fekitar keeps several copies of the residual stream (hyper-connections): a sublayer reads a weighted sum of the copies,
and its result is handed back to every copy while the copies are mixed among themselves. Its mixers are pairs of an
attention and a recurrence that read the same input (a windowed attention with short convolutions, per-head norms and a
distance penalty beside a Mamba-2 state-space recurrence; a rotated, soft-capped, gated attention beside a gated linear
attention), or a differential attention (two softmax maps over the same values, subtracted) that may read the keys and
values of an earlier layer. Its feed-forward is a mixture of clamped-swish experts with a gated shared expert.

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


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def short_convolution(u, taps_w, bias=None):
    """u [tokens, channels], taps_w [channels, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    T, C = u.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + padded[j:j + T] * taps_w[:, j]
    return y if bias is None else y + bias


def rotary_frequencies(rot, work):
    """One frequency per pair: base^(-2i/dims), rescaled band by band when the configuration gives a scaling."""
    dims = rot["dims"]
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = rot["base"] ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if sc:
        factor, low, high, orig = sc["factor"], sc["low"], sc["high"], sc["original"]
        wavelength = 2 * math.pi / f
        s = (orig / wavelength - low) / (high - low)
        mid = (1 - s) * f / factor + s * f
        f = torch.where(wavelength < orig / high, f, torch.where(wavelength > orig / low, f / factor, mid))
    return f.to(work)


def rotate_halves(v, positions, rot):
    """v [tokens, units, n]: the first rot.dims channels turn, channel i paired with i + dims/2."""
    dims = rot["dims"]
    half = dims // 2
    ang = positions.to(v.dtype)[:, None] * rotary_frequencies(rot, v.dtype)[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = v[..., :half], v[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, v[..., dims:]], dim=-1)


def visible(T, window):
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = j <= i
    if window:
        seen = seen & (i - j < window)
    return seen


def softmax_attention(q, k, v, scale, window=0, slopes=None, softcap=0.0):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; query head h reads key/value head h // (H / G). With ``slopes`` the
    score loses slope_h * (i - j); with ``softcap`` c it becomes c tanh(score / c)."""
    T, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    kk, vv = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * scale
    if softcap:
        s = softcap * torch.tanh(s / softcap)
    if slopes is not None:
        dist = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).to(q.dtype)
        s = s - slopes[:, None, None] * dist[None]
    p = torch.softmax(s.masked_fill(~visible(T, window), float("-inf")), dim=-1)
    return torch.einsum("hij,jhd->ihd", p, vv)


def distance_slopes(H, work):
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=work)


def matrix_state_recurrence(a, k, v, q, S=None):
    """a [T, H, N] (or [T, H, 1]), k, q [T, H, N], v [T, H, P]: S_t = diag(a_t) S_(t-1) + k_t v_t^T from S (zeros when
    None), o_t = S_t^T q_t. Returns (o [T, H, P], the last S [H, N, P])."""
    T, H, N = k.shape
    S = torch.zeros(H, N, v.shape[2], dtype=k.dtype) if S is None else S.clone()
    out = []
    for t in range(T):
        S = a[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hnp,hn->hp", S, q[t]))
    return torch.stack(out), S


# ---------------------------------------------------------------- mixer 'parallel' ----

def windowed_conv_attention(h, w, p, m, eps):
    """Left half of 'parallel': projections, short convolutions, per-head norms of q and k, no rotation, a distance
    penalty, a sliding window."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ w[p + "q"].T, h @ w[p + "k"].T, h @ w[p + "v"].T
    if m.get("conv"):
        q, k, v = (short_convolution(t, w[p + n + ".conv"]) for t, n in ((q, "q"), (k, "k"), (v, "v")))
    q = rms(q.reshape(T, H, d), eps) * w[p + "q.norm"]
    k = rms(k.reshape(T, G, d), eps) * w[p + "k.norm"]
    window = m["mask"]["size"] if m.get("mask") else 0
    o = softmax_attention(q, k, v.reshape(T, G, dv), m["scale"], window, slopes=distance_slopes(H, h.dtype))
    return o.reshape(T, H * dv) @ w[p + "o"].T


def mamba2(h, w, p, m, eps):
    """Right half of 'parallel': the state-space recurrence, token by token."""
    T = h.shape[0]
    Hh, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = Hh * P
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_convolution(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, Hh, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N).repeat_interleave(Hh // G, dim=1)
    C = xbc[:, inner + G * N:].reshape(T, G, N).repeat_interleave(Hh // G, dim=1)
    dt = softplus(dt + w[p + "dt_bias"])
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * dt)                 # [T, heads]
    y, _ = matrix_state_recurrence(decay[:, :, None], B, dt[:, :, None] * x, C)
    y = (y + w[p + "D"][:, None] * x).reshape(T, inner) * silu(z)
    parts = m.get("norm_groups", 1)
    y = rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def mixer_parallel(h, w, p, m, eps):
    left = windowed_conv_attention(h, w, p + "left.", m["left"], eps)
    right = mamba2(h, w, p + "right.", m["right"], eps)
    return 0.5 * (rms(left, eps) * w[p + "left.out"] + rms(right, eps) * w[p + "right.out"])


# ---------------------------------------------------------------- mixer 'parallel_2' ----

def gated_rotary_attention(h, w, p, m):
    """Left half of 'parallel_2': rotated queries and keys, soft-capped scores, every key visible, an output gate per
    channel."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q, k, v = (h @ w[p + "q"].T).reshape(T, H, d), (h @ w[p + "k"].T).reshape(T, G, d), (h @ w[p + "v"].T).reshape(T, G, dv)
    if m.get("rot"):
        q, k = rotate_halves(q, pos, m["rot"]), rotate_halves(k, pos, m["rot"])
    o = softmax_attention(q, k, v, m["scale"], softcap=m.get("softcap", 0.0)).reshape(T, H * dv)
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def gated_linear_attention(h, w, p, m, eps):
    """Right half of 'parallel_2': a matrix state per head whose rows (key channels) decay by their own factor."""
    T = h.shape[0]
    Hh, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(T, Hh, d) * d ** -0.5
    k = (h @ w[p + "k"].T).reshape(T, Hh, d)
    v = (h @ w[p + "v"].T).reshape(T, Hh, dv)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = (torch.sigmoid(z) ** (1.0 / m["tau"])).reshape(T, Hh, d)
    o, _ = matrix_state_recurrence(alpha, k, v, q)
    o = rms(o, eps) * w[p + "norm"]
    return (o.reshape(T, Hh * dv) * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def mixer_parallel_2(h, w, p, m, eps):
    return (m["left_scale"] * gated_rotary_attention(h, w, p + "left.", m["left"])
            + m["right_scale"] * gated_linear_attention(h, w, p + "right.", m["right"], eps))


# ---------------------------------------------------------------- mixer 'attention' ----

def differential_keys_values(h, w, p, m):
    """Keys [T, G, 2, d] after convolution and rotation, values [T, G, dv] after convolution: what the layer's cache
    holds and what a later layer may borrow."""
    T = h.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    k, v = h @ w[p + "k"].T, h @ w[p + "v"].T
    if m.get("conv"):
        k, v = short_convolution(k, w[p + "k.conv"]), short_convolution(v, w[p + "v.conv"])
    k = k.reshape(T, G * 2, d)
    if m.get("rot"):
        k = rotate_halves(k, torch.arange(T), m["rot"])
    return k.reshape(T, G, 2, d), v.reshape(T, G, dv)


def differential_attention(h, w, p, m, eps, kv=None):
    """Two softmax maps a head over the same values; the second is subtracted, times one learned number of the layer."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = h @ w[p + "q"].T
    if m.get("conv"):
        q = short_convolution(q, w[p + "q.conv"])
    q = q.reshape(T, H * 2, d)
    if m.get("rot"):
        q = rotate_halves(q, torch.arange(T), m["rot"])
    q = q.reshape(T, H, 2, d)
    k, v = kv if kv is not None else differential_keys_values(h, w, p, m)
    a1 = softmax_attention(q[:, :, 0], k[:, :, 0], v, m["scale"])
    a2 = softmax_attention(q[:, :, 1], k[:, :, 1], v, m["scale"])
    lam = torch.exp((w[p + "lq1"] * w[p + "lk1"]).sum()) - torch.exp((w[p + "lq2"] * w[p + "lk2"]).sum()) + m["diff"]
    o = rms(a1 - lam * a2, eps) * (1.0 - m["diff"])
    o = o * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ w[p + "o"].T


# ---------------------------------------------------------------- feed-forward ----

def clamped_expert(h, w, p, limit):
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def router_scores(h, w, p):
    return torch.softmax((h.float() @ w[p + "router"].float().T), dim=-1)


def mixture(h, w, p, f, margins=None):
    """Softmax over all experts, the ``top`` largest chosen (lowest index first among equals), weights divided by their
    sum; a shared expert times sigmoid(W_sg h). ``margins``: a list that receives, per token, the gap between the
    logarithms of the last chosen and the first rejected score (the gap of their router logits)."""
    T = h.shape[0]
    E, top = f["router"]["experts"], f["router"]["top"]
    s = router_scores(h, w, p).to(h.dtype)
    order = torch.sort(s, dim=-1, descending=True, stable=True)
    idx, val = order.indices[:, :top], order.values[:, :top]
    if margins is not None:
        margins.extend((order.values[:, top - 1].log() - order.values[:, top].log()).tolist() if top < E else [1e9] * T)
    wt = val / (val.sum(dim=-1, keepdim=True) + 1e-20)
    out = torch.zeros(T, w[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(T):
        for c in range(top):
            e = int(idx[t, c])
            out[t] += wt[t, c] * clamped_expert(h[t:t + 1], w, f"{p}e{e}.", f["expert"]["limit"])[0]
    if f.get("shared"):
        gate = torch.sigmoid(h @ w[p + "shared.sg"].T)
        out = out + gate * clamped_expert(h, w, p + "shared.", f["shared"]["limit"])
    return out


# ---------------------------------------------------------------- layers ----

def hyper_read(xs, w, p):
    return torch.einsum("s,std->td", w[p + "in"], xs)


def hyper_write(xs, y, w, p, mult):
    return torch.einsum("sr,std->rtd", w[p + "mix"], xs) + mult * w[p + "out"][:, None, None] * y[None]


def forward(cfg, w, ids, work=torch.float64, margins=None):
    """ids [T] -> (logits [T, vocab], the summed stream after every layer [layers, T, width])."""
    w = {k: (v.to(work) if v.is_floating_point() else v) for k, v in w.items()}
    eps, mult, streams = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0), cfg.get("streams", 0)
    x = w["embed"][ids]
    xs = x[None].repeat(max(streams, 1), 1, 1)
    after, kvs = [], {}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]

        def sublayer(q, fn, xs):
            u = hyper_read(xs, w, f"{p}hc{q}.") if streams else xs[0]
            y = fn(rms(u, eps) * w[f"{p}norm{q}"])
            return hyper_write(xs, y, w, f"{p}hc{q}.", mult) if streams else (xs[0] + mult * y)[None]

        def mix(h):
            if L["type"] == "parallel":
                return mixer_parallel(h, w, p + "mix.", m, eps)
            if L["type"] == "parallel_2":
                return mixer_parallel_2(h, w, p + "mix.", m, eps)
            if "kv_from" in m:
                return differential_attention(h, w, p + "mix.", m, eps, kv=kvs[m["kv_from"]])
            kvs[i] = differential_keys_values(h, w, p + "mix.", m)
            return differential_attention(h, w, p + "mix.", m, eps, kv=kvs[i])

        xs = sublayer(1, mix, xs)
        if L.get("mlp"):
            xs = sublayer(2, lambda h: mixture(h, w, p + "mlp.", L["mlp"], margins), xs)
        after.append(xs.sum(dim=0))
    x = rms(xs.sum(dim=0), eps) * w["final.norm"]
    return x @ w["head"].T, torch.stack(after)


def greedy_generate(cfg, w, prompt, n, work=torch.float64):
    """The ``n`` tokens that always taking the largest logit gives after ``prompt`` (the whole sequence is run again for
    every token: slow and plain)."""
    seq, out = list(prompt), []
    for _ in range(n):
        tok = int(torch.argmax(forward(cfg, w, torch.tensor(seq), work)[0][-1]))
        out.append(tok)
        seq.append(tok)
    return out
