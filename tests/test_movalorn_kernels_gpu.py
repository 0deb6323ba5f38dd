"""Each Movalorn mechanism alone, its kernel against the plain implementation's function: the minGRU recurrence (one
pass and in chunks, states in scattered slots, unequal sequences, portions); the hashed pair table with the previous
token as state; the gated, normalised residual; the window over the latent cache (keys just inside and just outside it,
at page borders, in prompts, portions and single tokens, through the general, the tensor-core and the per-head kernel);
the gate per head; softmax routing with a choice correction; the tanh form of GELU alone and in the products'
epilogues; the loop's entry (two streams side by side) and the scaled logits."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from plain import lezepel_plain
from plain import movalorn_plain as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DT = {"fp32": torch.float32, "bf16": torch.bfloat16}
TOL = {"fp32": dict(rtol=2e-5, atol=2e-5), "bf16": dict(rtol=2e-2, atol=2e-2)}
# the window tests make one score stand out by a dozen or two: rounding a score of 20 to bfloat16 moves a softmax weight
# by a few per cent, while a window that is off by one key moves a row by about 1
WINDOW_TOL = {"fp32": dict(rtol=1e-4, atol=1e-4), "bf16": dict(rtol=5e-2, atol=5e-2)}


def window_close(got, want, dtype):
    """float32: every element inside the bound. bfloat16: where two loud scores compete, their rounding moves single
    elements by up to a tenth; so all but two in a thousand lie inside the bound and none is off by more than 0.3 (a
    window that is one key short or long moves a third of all rows by about 1)."""
    if dtype == "fp32":
        torch.testing.assert_close(got, want, **WINDOW_TOL[dtype])
        return
    t = WINDOW_TOL[dtype]
    off = (got - want).abs()
    outside = off > t["atol"] + t["rtol"] * want.abs()
    assert float(outside.double().mean()) <= 2e-3 and float(off.max()) < 0.3, (int(outside.sum()), float(off.max()))


def ops():
    from sleuth_b200.kernels import ops as o
    return o


def i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


# ---- the recurrence ----
def gru_weights(W, seed, slow=0.0):
    """Identity projections: the plain function then reads its gates straight from the columns of its input."""
    g = torch.Generator().manual_seed(seed)
    eye = torch.eye(3 * W, dtype=torch.float64)
    return {"z": eye[:W], "x": eye[W:2 * W], "g": eye[2 * W:], "o": torch.eye(W, dtype=torch.float64),
            "z.b": torch.randn(W, generator=g, dtype=torch.float64) - slow, "x.b": torch.randn(W, generator=g, dtype=torch.float64)}


def run_mingru(p_rows, w, state, slots, counts, dtype):
    o = ops()
    W = w["o"].shape[0]
    T = sum(counts)
    y = torch.empty(T, W, dtype=DT[dtype], device=DEV)
    starts = i32(np.concatenate([[0], np.cumsum(counts)]).tolist())
    need = o.mingru_scratch_floats(len(counts), max(counts), W)
    scratch = torch.empty(need, dtype=torch.float32, device=DEV) if need else None
    o.mingru(p_rows.float().to(DEV), w["z.b"].float().to(DEV), w["x.b"].float().to(DEV), state, i32(slots), starts, y, max(counts), scratch)
    return y.cpu().double()


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("W, counts", [(52, [1, 7, 64, 3]), (256, [65, 1, 200, 64, 129]), (130, [1]), (100, [640, 63, 128]),
                                       (33, [2100, 33, 17, 16, 700]), (160, [32, 48, 31])])
def test_the_recurrence_in_one_pass_and_in_chunks(W, counts, dtype):
    g = torch.Generator().manual_seed(W + len(counts))
    w = gru_weights(W, W, slow=2.0)                         # slow gates: the state remembers across chunks
    slots = [5, 0, 9, 2, 7][:len(counts)]
    state = torch.full((11, W), 3.0, dtype=torch.float32, device=DEV)      # other slots' states must stay as they are
    state[slots] = 0.0
    seqs = [torch.randn(c, 3 * W, generator=g, dtype=torch.float64) * 2.0 for c in counts]
    got = run_mingru(torch.cat(seqs), w, state, slots, counts, dtype)
    want = torch.cat([plain.mingru(s.float().double(), w, "") for s in seqs])
    torch.testing.assert_close(got, want, **TOL[dtype])
    others = [s for s in range(11) if s not in slots]
    assert bool((state[others] == 3.0).all()) and not bool((state[slots] == 0.0).all())
    # both branches of the candidate were taken
    u = torch.cat(seqs)[:, W:2 * W] + w["x.b"]
    assert bool((u >= 0).any()) and bool((u < 0).any())


@pytest.mark.parametrize("cuts", [[1, 1, 1, 197], [64, 64, 72], [2, 65, 130, 3], [199, 1]])
def test_the_state_carries_a_sequence_from_step_to_step(cuts):
    """A sequence fed in portions (single tokens, exactly a chunk, more than a chunk) ends where the whole sequence ends,
    beside another sequence whose steps have other lengths."""
    W = 72
    g = torch.Generator().manual_seed(sum(cuts))
    w = gru_weights(W, 3, slow=3.0)
    a, b = torch.randn(200, 3 * W, generator=g, dtype=torch.float64), torch.randn(200, 3 * W, generator=g, dtype=torch.float64)
    state = torch.zeros(4, W, dtype=torch.float32, device=DEV)
    other = list(reversed(cuts))
    got_a, got_b, at_a, at_b = [], [], 0, 0
    for ca, cb in zip(cuts, other):
        y = run_mingru(torch.cat([a[at_a:at_a + ca], b[at_b:at_b + cb]]), w, state, [3, 1], [ca, cb], "fp32")
        got_a.append(y[:ca]); got_b.append(y[ca:])
        at_a, at_b = at_a + ca, at_b + cb
    torch.testing.assert_close(torch.cat(got_a), plain.mingru(a.float().double(), w, ""), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(torch.cat(got_b), plain.mingru(b.float().double(), w, ""), rtol=1e-5, atol=1e-5)
    # the early tokens still count at the end: a sequence that lost its state would end elsewhere
    fresh = plain.mingru(a[150:].float().double(), w, "")
    assert float((fresh[-1] - torch.cat(got_a)[-1]).abs().max()) > 1e-3


# ---- the pair table ----
@pytest.mark.parametrize("one_pass", [False, True])
@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_pair_table_rows_and_the_previous_token_as_state(dtype, one_pass):
    o, dt = ops(), DT[dtype]
    vocab, d, buckets, mp, mc = 301, 40, 97, 7, 13
    g = torch.Generator().manual_seed(4)
    w = {"embed": torch.randn(vocab, d, generator=g).to(dt).double(), "bigram": torch.randn(buckets + 1, d, generator=g).to(dt).double()}
    e = {"scale": 3.0, "bigram": {"buckets": buckets, "mul_prev": mp, "mul_cur": mc}}
    rng = np.random.default_rng(0)
    seqs = [rng.integers(0, vocab, size=n).tolist() for n in (9, 1, 30)]
    seqs[2][4] = seqs[2][3] = 300                    # the largest products of the hash
    want = [plain.embedding(torch.tensor(s), w, e) for s in seqs]
    last = torch.full((6,), -1, dtype=torch.int32, device=DEV)          # a free slot holds no previous token
    slots = [4, 0, 2]
    table, pairs = w["embed"].to(dt).to(DEV), w["bigram"].to(dt).to(DEV)
    done, got = [0, 0, 0], [[], [], []]
    for counts in ([3, 1, 0], [1, 0, 1], [5, 0, 29]):        # portions, single tokens, a sequence that joins later
        live = [s for s in range(3) if counts[s]]
        ids = sum((seqs[s][done[s]:done[s] + counts[s]] for s in live), [])
        c = [counts[s] for s in live]
        tok_seq = i32(sum(([k] * n for k, n in enumerate(c)), []))
        tok_pos = i32(sum((list(range(done[s], done[s] + counts[s])) for s in live), []))
        x = torch.empty(len(ids), d, dtype=torch.float32, device=DEV)
        starts, now = i32(np.concatenate([[0], np.cumsum(c)]).tolist()), i32([slots[s] for s in live])
        if one_pass:        # the token's row and the pair's row in one kernel
            o.pair_embed(i32(ids), None, pairs, x, tok_seq, tok_pos, starts, now, last, vocab, buckets, mp, mc, table=table, scale=3.0)
        else:
            o.embed(i32(ids), table, x, 3.0)
            o.pair_embed(i32(ids), None, pairs, x, tok_seq, tok_pos, starts, now, last, vocab, buckets, mp, mc)
        at = 0
        for s in live:
            got[s].append(x[at:at + counts[s]].cpu().double())
            at += counts[s]
            done[s] += counts[s]
    for s in range(3):
        torch.testing.assert_close(torch.cat(got[s]), want[s], rtol=1e-6, atol=1e-6)
    assert last.cpu().tolist() == [seqs[1][-1], -1, seqs[2][-1], -1, seqs[0][-1], -1]


# ---- the gated, normalised residual ----
@pytest.mark.parametrize("d", [72, 75, 320, 1000, 2050, 4096, 6000])
def test_gated_normalised_residual(d):
    o = ops()
    g = torch.Generator().manual_seed(d)
    x, y = torch.randn(9, d, generator=g), 4.0 * torch.randn(9, d, generator=g)
    wide = 3.0 * torch.randn(9, d + 24, generator=g)        # the gate's values are a view of a wider product
    bias, gain, eps = torch.randn(d, generator=g), 1.7, 1e-3
    v = y.double() * torch.sigmoid(wide[:, 8:8 + d].double() + bias.double())
    want = x.double() + plain.rms(v, eps) * gain
    xd, wd = x.clone().to(DEV), wide.to(DEV)
    o.gated_norm_add(xd, y.clone().to(DEV), wd[:, 8:8 + d], bias.to(DEV), torch.full((d,), gain, device=DEV), eps)
    torch.testing.assert_close(xd.cpu().double(), want, rtol=1e-5, atol=1e-5)
    xd = x.clone().to(DEV)                                    # without a gate: the norm and the sum only
    o.gated_norm_add(xd, y.clone().to(DEV), None, None, torch.full((d,), gain, device=DEV), eps)
    torch.testing.assert_close(xd.cpu().double(), x.double() + plain.rms(y.double(), eps) * gain, rtol=1e-5, atol=1e-5)
    tiny = 1e-4 * y                                           # eps inside the root decides for small rows
    xd = torch.zeros(9, d, device=DEV)
    o.gated_norm_add(xd, tiny.clone().to(DEV), None, None, torch.ones(d, device=DEV), eps)
    torch.testing.assert_close(xd.cpu().double(), plain.rms(tiny.double(), eps), rtol=1e-5, atol=1e-7)
    assert float(xd.abs().max()) < 0.5


# ---- the window over the latent cache ----
def paged(rows_per_seq, width, dtype, seed):
    """A pool whose pages are handed out in a scrambled order, and the block table of the sequences."""
    n_pages = sum(-(-len(r) // 64) for r in rows_per_seq) + 3
    order = np.random.default_rng(seed).permutation(n_pages)
    pool = torch.full((n_pages, 64, width), 7.0, dtype=dtype, device=DEV)      # stale contents must never be read
    stride = max(-(-len(r) // 64) for r in rows_per_seq) + 1
    table = torch.full((len(rows_per_seq), stride), -1, dtype=torch.int32)
    k = 0
    for s, rows in enumerate(rows_per_seq):
        for p in range(-(-len(rows) // 64)):
            table[s, p] = int(order[k])
            part = rows[p * 64:(p + 1) * 64]
            pool[order[k], :len(part)] = part.to(dtype).to(DEV)
            k += 1
    return pool, table.to(DEV)


def rot_tables(positions, base, dims):
    i = torch.arange(dims // 2, dtype=torch.float32)
    ang = torch.outer(torch.arange(positions, dtype=torch.float32), base ** (-2.0 * i / dims))
    return ang.cos().to(DEV), ang.sin().to(DEV)


def window_case(H, dn, P, dv, R, pasts, counts, window, seed, dtype):
    """Random latents and queries. For every query of the step two keys are made loud in turn: even query positions
    point at the oldest key the window still holds (distance window - 1), odd ones at the newest key it has dropped
    (distance window), which must not count however loud it is."""
    g = torch.Generator().manual_seed(seed)
    dt = DT[dtype]
    w_uk = (torch.randn(H * dn, R, generator=g, dtype=torch.float64) / R ** 0.5).to(dt).double()
    w_uv = (torch.randn(H * dv, R, generator=g, dtype=torch.float64) / R ** 0.5).to(dt).double()
    seqs = []
    for p, c in zip(pasts, counts):
        n = p + c
        s = dict(c=torch.randn(n, R, generator=g, dtype=torch.float64), k_rot=0.3 * torch.randn(n, P, generator=g, dtype=torch.float64),
                 q=0.3 * torch.randn(n, H, dn + P, generator=g, dtype=torch.float64))
        for qi in range(p, n):
            ki = qi - (window - 1) - (qi % 2)
            if ki >= 0:
                k_plain = (s["c"][ki] @ w_uk.T).reshape(H, dn)
                s["q"][qi, :, :dn] = 30.0 * k_plain / k_plain.norm(dim=-1, keepdim=True)
        seqs.append({k: v.to(dt).double() for k, v in s.items()})
    return w_uk, w_uv, seqs


def window_want(seqs, w_uk, w_uv, H, dn, P, dv, pasts, counts, window, base, scale):
    want = []
    for s, p, c in zip(seqs, pasts, counts):
        n = p + c
        pos = torch.arange(n)
        q = torch.cat([s["q"][..., :dn], lezepel_plain.rotate_half_pairs(s["q"][..., dn:], pos, base, P)], -1)
        k = torch.cat([(s["c"] @ w_uk.T).reshape(n, H, dn),
                       lezepel_plain.rotate_half_pairs(s["k_rot"][:, None, :], pos, base, P).expand(n, H, P)], -1)
        v = (s["c"] @ w_uv.T).reshape(n, H, dv)
        want.append(plain.windowed_softmax_attention(q, k, v, scale, window)[p:])
    return torch.cat(want)


def run_window(H, dn, P, dv, R, pasts, counts, window, dtype, seed, splits=1, base=1000.0, scale=0.4):
    o, dt = ops(), DT[dtype]
    w_uk, w_uv, seqs = window_case(H, dn, P, dv, R, pasts, counts, window, seed, dtype)
    cos, sin = rot_tables(max(p + c for p, c in zip(pasts, counts)) + 1, base, P)
    rows = [torch.cat([s["c"], lezepel_plain.rotate_half_pairs(s["k_rot"][:, None, :], torch.arange(len(s["c"])), base, P)[:, 0]], -1)
            for s in seqs]
    pool, table = paged(rows, R + P, dt, seed)
    T = sum(counts)
    q_raw = torch.cat([s["q"][p:p + c] for s, p, c in zip(seqs, pasts, counts)]).reshape(T, H, dn + P)
    q_lat = torch.einsum("thd,hdr->htr", q_raw[..., :dn], w_uk.reshape(H, dn, R)).to(dt)
    out = torch.empty(H, T, R, dtype=dt, device=DEV)
    scratch = torch.empty(max(1, o.latent_scratch_floats(T, H, R, splits)), dtype=torch.float32, device=DEV)
    o.latent_attention(q_lat.to(DEV).contiguous(), q_raw.to(dt).to(DEV).contiguous(), pool, out, cos, sin,
                       i32(np.concatenate([[0], np.cumsum(counts)]).tolist()), i32(pasts), i32(counts), table, max(counts), H, R, P, dn,
                       P, window, scale, splits, scratch)
    got = torch.einsum("htr,hvr->thv", out.cpu().double(), w_uv.reshape(H, dv, R))
    return got, window_want(seqs, w_uk, w_uv, H, dn, P, dv, pasts, counts, window, base, scale), (seqs, w_uk, w_uv)


def loud_keys_decide(want, seqs, w_uv, pasts, counts, window, H, dv):
    """How many queries that point at the key just inside the window return about that key's value, and how many of
    those that point at the key just outside it do not: (inside hits, inside queries, outside misses, outside queries)."""
    at = 0
    hit = near = miss = far = 0
    for s, p, c in zip(seqs, pasts, counts):
        for qi in range(p, p + c):
            ki = qi - (window - 1) - (qi % 2)
            if ki >= 0:
                v = (s["c"][ki] @ w_uv.T).reshape(H, dv)
                d = float((want[at + qi - p] - v).abs().max())
                if qi % 2 == 0:
                    near, hit = near + 1, hit + (d < 0.25)
                else:
                    far, miss = far + 1, miss + (d > 0.25)
        at += c
    return hit, near, miss, far


@pytest.mark.parametrize("R, P", [(24, 8), (32, 16), (64, 16)])       # the last two go to the tensor-core kernel in bfloat16
@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("window", [1, 2, 37, 64, 65, 130])
def test_keys_just_inside_and_just_outside_the_window(window, dtype, R, P):
    """Whole prompts, a portion behind earlier tokens, a portion that starts at a page border, and single tokens (right
    behind the window's first fill, far behind it, at a page border), all in one step."""
    pasts, counts = [0, 100, 128, window - 1, window, 400, 191, 0], [150, 70, 64, 1, 1, 1, 1, 1]
    H, dn, dv = 3, 16, 12
    got, want, (seqs, w_uk, w_uv) = run_window(H, dn, P, dv, R, pasts, counts, window, dtype, seed=window + R)
    window_close(got, want, dtype)
    hit, near, miss, far = loud_keys_decide(want, seqs, w_uv, pasts, counts, window, H, dv)
    # the inputs do what they are made for: a window one key short changes a third of the rows and more, one key long most
    assert near > 50 and far > 50 and hit >= 0.3 * near and miss >= 0.8 * far


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("splits", [2, 5, 16])
@pytest.mark.parametrize("R, P, window", [(40, 8, 100), (48, 16, 64), (48, 16, 700)])
def test_single_tokens_with_the_keys_in_slices_keep_the_window(R, P, window, splits, dtype):
    pasts, counts = [1000, 70, 0, 511, 99, 100], [1, 1, 1, 1, 1, 1]
    got, want, _ = run_window(6, 16, P, 16, R, pasts, counts, window, dtype, seed=2, splits=splits)
    window_close(got, want, dtype)


@pytest.mark.parametrize("window", [1, 9, 64, 65, 100, 5000])
@pytest.mark.parametrize("H, dn, P, dv, R", [(3, 16, 16, 16, 40), (2, 64, 32, 48, 128), (5, 24, 8, 48, 24)])
def test_whole_prompts_with_per_head_keys_keep_the_window(H, dn, P, dv, R, window):
    o, dt = ops(), torch.bfloat16
    if not o.head_prompt_supported(dn, P, dv, dt):
        pytest.skip("these head sizes do not take the per-head prompt kernel")
    pasts, counts = [0, 0, 0, 0], [200, 64, 1, 131]
    base, scale = 500.0, 0.4
    w_uk, w_uv, seqs = window_case(H, dn, P, dv, R, pasts, counts, window, 5 + window, "bf16")
    T = sum(counts)
    cos, sin = rot_tables(max(counts) + 1, base, P)
    q = torch.cat([s["q"] for s in seqs]).to(dt).to(DEV).contiguous()
    c_all = torch.cat([s["c"] for s in seqs])
    kv = torch.cat([c_all @ w_uk.T, c_all @ w_uv.T], -1).to(dt)
    k_rot = torch.cat([lezepel_plain.rotate_half_pairs(s["k_rot"][:, None, :], torch.arange(len(s["c"])), base, P)[:, 0] for s in seqs]).to(dt)
    out = torch.empty(H, T, dv, dtype=dt, device=DEV)
    o.head_prompt_attention(q, kv.to(DEV).contiguous(), k_rot.to(DEV).contiguous(), out, cos, sin,
                            i32(np.concatenate([[0], np.cumsum(counts)]).tolist()), i32(counts), max(counts), H, dn, P, dv, P, window, scale)
    want = window_want(seqs, w_uk, w_uv, H, dn, P, dv, pasts, counts, window, base, scale)
    window_close(out.cpu().double().transpose(0, 1), want, "bf16")      # keys and values were rounded once more on the way
    if window < 200:
        hit, near, miss, far = loud_keys_decide(want, seqs, w_uv, pasts, counts, window, H, dv)
        assert hit >= 0.3 * near and miss >= 0.8 * far


# ---- the gate per head ----
@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("H, T, dv", [(5, 37, 24), (1, 1, 8), (40, 3, 80), (3, 130, 12), (7, 5, 7)])
def test_one_gate_value_per_head(H, T, dv, dtype):
    g = torch.Generator().manual_seed(H)
    val = torch.randn(H, T, dv, generator=g).to(DT[dtype])
    wide = 3 * torch.randn(T, 11 + H, generator=g)           # the gates ride in the last columns of a wider product
    y = torch.empty(T, H * dv, dtype=DT[dtype], device=DEV)
    ops().latent_head_gate(val.to(DEV), wide.to(DEV)[:, 11:], y)
    want = (val.double().transpose(0, 1) * torch.sigmoid(wide[:, 11:].double())[:, :, None]).reshape(T, H * dv)
    torch.testing.assert_close(y.cpu().double(), want, **TOL[dtype])


# ---- softmax routing with a choice correction ----
@pytest.mark.parametrize("T", [1, 7, 200])
@pytest.mark.parametrize("E, top, scale", [(5, 2, 1.5), (6, 1, 0.7), (4, 4, 0.25), (12, 2, 1.5), (70, 3, 1.0), (8, 3, 2.5)])
def test_softmax_scores_choose_with_the_correction_and_weigh_without_it(E, top, scale, T):
    o = ops()
    g = torch.Generator().manual_seed(E * 100 + T)
    d = 72
    h = torch.randn(T, d, generator=g)
    w = {"router": torch.randn(E, d, generator=g) * (3.0 / d ** 0.5),
         "correction": (torch.randperm(E, generator=g).double() - (E - 1) / 2) * (0.4 / E)}
    f = {"router": {"experts": E, "top": top, "scale": scale}}
    idx, wt, margin = plain.expert_choice(h.double(), {k: v.double() for k, v in w.items()}, "", f)
    n = T * top
    choice, rank, place, order = (torch.empty(n, dtype=torch.int32, device=DEV) for _ in range(4))
    counts = torch.empty(E, dtype=torch.int32, device=DEV)
    weight = torch.empty(n, dtype=torch.float32, device=DEV)
    logits = torch.empty(T, E, dtype=torch.float32, device=DEV)
    o.moe_route(h.to(DEV), w["router"].to(DEV), None, choice, weight, rank, counts, place, order, top, logits=logits,
                scoring="softmax", scale=scale, pick_bias=w["correction"].float().to(DEV))
    got_i, got_w = choice.cpu().view(T, top).long(), weight.cpu().view(T, top).double()
    sure = margin > 1e-5                                      # a choice that float32 cannot get wrong
    assert int(sure.sum()) >= 0.95 * T
    assert torch.equal(got_i[sure], idx[sure])
    torch.testing.assert_close(got_w[sure], wt[sure], rtol=1e-4, atol=1e-6)
    assert torch.equal(counts.cpu().long(), torch.bincount(got_i.flatten(), minlength=E))
    if top < E:
        # the correction decides some choices (without it other experts would be taken) and never enters a weight
        bare = torch.topk(torch.softmax(h.double() @ w["router"].double().T, -1), top, dim=-1).indices
        moved = (torch.sort(bare, -1).values != torch.sort(idx, -1).values).any(-1)
        assert T < 200 or bool(moved.any())
        assert float(got_w.sum(-1).max()) <= scale * (1 + 1e-5)


# ---- the tanh form of GELU ----
@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_gated_tanh_gelu(dtype):
    g = torch.Generator().manual_seed(6)
    ff = 40
    gu = (2.5 * torch.randn(9, 2 * ff, generator=g)).to(DT[dtype])
    act = torch.empty(9, ff, dtype=DT[dtype], device=DEV)
    ops().gated_act(gu.to(DEV), act, "gelu_tanh")
    want = plain.gelu_tanh(gu[:, :ff].double()) * gu[:, ff:].double()
    torch.testing.assert_close(act.cpu().double(), want, **TOL[dtype])
    exact = torch.nn.functional.gelu(gu[:, :ff].double()) * gu[:, ff:].double()       # the erf form is another function
    assert float((want - exact).abs().max()) > 1e-4


@pytest.mark.parametrize("T", [1, 8, 200])
def test_gated_products_apply_the_tanh_gelu_in_their_epilogue(T):
    o = ops()
    g = torch.Generator().manual_seed(T)
    d, ff = 256, 192
    h = torch.randn(T, d, generator=g).to(torch.bfloat16)
    w = {"gate": (torch.randn(ff, d, generator=g) * 0.15).to(torch.bfloat16).double(),
         "up": (torch.randn(ff, d, generator=g) * 0.15).to(torch.bfloat16).double(), "down": torch.eye(ff, dtype=torch.float64)}
    want = plain.gated_mlp(h.double(), w, "", plain.gelu_tanh)
    w_gu = torch.cat([w["gate"], w["up"]]).to(torch.bfloat16).to(DEV).contiguous()
    act = torch.empty(T, ff, dtype=torch.bfloat16, device=DEV)
    gate = ("gelu_tanh", 0.0, 1.0)
    if T <= 32:
        o.gemm_skinny(h.to(DEV), w_gu, act, "swiglu", gate=gate)
    else:
        o.gemm_tc(h.to(DEV), w_gu, act, "swiglu", gate=gate)
        o.gemm_tc_check(DEV)
    torch.testing.assert_close(act.cpu().double(), want, rtol=3e-2, atol=3e-2)
    silu = plain.gated_mlp(h.double(), w, "", plain.silu)
    assert float((want - silu).abs().max()) > 0.2             # another activation would show


# ---- the loop's entry and the scaled logits ----
@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_two_streams_side_by_side_and_scaled_rows(dtype):
    o = ops()
    g = torch.Generator().manual_seed(8)
    for d in (72, 75, 1030):                                   # whole pieces of four values and not
        a, b = torch.randn(13, d, generator=g), torch.randn(13, d, generator=g)
        both = torch.empty(13, 2 * d, dtype=DT[dtype], device=DEV)
        o.stream_pair(a.to(DEV), b.to(DEV), both)
        torch.testing.assert_close(both.cpu().float(), torch.cat([a, b], -1).to(DT[dtype]).float(), rtol=0, atol=0)
    v, row = torch.randn(13, 50, generator=g), torch.randn(50, generator=g)
    vd = v.clone().to(DEV)
    o.scale(vd, 0.25)
    torch.testing.assert_close(vd.cpu(), v * 0.25)
    wide = torch.randn(13, 80, generator=g).to(DEV)             # a view of a wider matrix, with a row added
    keep = wide.clone()
    o.scale(wide[:, 10:60], 2.0, add=row.to(DEV))
    torch.testing.assert_close(wide[:, 10:60].cpu(), keep[:, 10:60].cpu() * 2.0 + row)
    assert torch.equal(wide[:, :10], keep[:, :10]) and torch.equal(wide[:, 60:], keep[:, 60:])
