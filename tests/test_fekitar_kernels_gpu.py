"""Each kernel that came with the Fekitar design beside its plain function: short causal convolutions with a tail per
sequence, the recurrence with a matrix state (one decay a head and one a key channel), step sizes and decays, the gated
group norm in both orders, per-unit post-processing into the paged cache, attention with a distance penalty, a soft cap,
a window and two score maps (a loud key just inside and just outside every window, at page borders and far away), the
differential combination, the copies of the stream, the joins of two mixers, the gate of the shared expert, and the
routing rule whose weights are divided by their sum."""

from __future__ import annotations

import math

import pytest
import torch

from plain import fekitar_plain as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ops():
    from sleuth_b200.kernels import ops as o
    return o


def i32(v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


def batch_tables(counts, pasts=None):
    """tok_seq, tok_pos, seq_start for sequences that bring ``counts`` tokens behind ``pasts`` earlier ones."""
    pasts = pasts or [0] * len(counts)
    seq = [s for s, c in enumerate(counts) for _ in range(c)]
    pos = [p + i for c, p in zip(counts, pasts) for i in range(c)]
    start = [0]
    for c in counts:
        start.append(start[-1] + c)
    return i32(seq), i32(pos), i32(start)


# ---------------------------------------------------------------- short convolutions ----

@pytest.mark.parametrize("taps,C", [(2, 7), (4, 96), (5, 33), (16, 8)])
def test_convolution_in_one_step_and_in_portions(taps, C):
    o = ops()
    g = torch.Generator().manual_seed(taps * 100 + C)
    lengths = [1, taps - 1, 70, 3]
    us = [torch.randn(n, C + 5, generator=g) for n in lengths]          # rows wider than the channels: a view is convolved
    w, bias = torch.randn(C, taps, generator=g), torch.randn(C, generator=g)
    slots = [5, 0, 3, 6]
    for act, b in ((False, None), (True, bias)):
        want = [plain.short_convolution(u[:, :C].double(), w.double(), None if b is None else b.double()) for u in us]
        want = [plain.silu(y) if act else y for y in want]
        # one step with all sequences, then the same in portions of 1, 2 and the rest
        for cuts in ([None], [1, 2, None]):
            state = torch.full((8, taps - 1, C), 0.0, device=DEV)
            state[[1, 2, 4, 7]] = 9.0                                    # slots of other sequences
            done = [0] * len(us)
            got = [[] for _ in us]
            for cut in cuts:
                take = [len(u) - d if cut is None else min(cut, len(u) - d) for u, d in zip(us, done)]
                live = [i for i, t in enumerate(take) if t > 0]
                if not live:
                    continue
                rows = torch.cat([us[i][done[i]:done[i] + take[i]] for i in live]).to(DEV)
                tok_seq, _, start = batch_tables([take[i] for i in live])
                out = torch.empty(rows.shape[0], C, device=DEV)
                o.causal_conv(rows[:, :C], w.to(DEV), None if b is None else b.to(DEV), state, i32([slots[i] for i in live]), tok_seq, start, out, act)
                at = 0
                for i in live:
                    got[i].append(out[at:at + take[i]].cpu())
                    at += take[i]
                    done[i] += take[i]
            for i in range(len(us)):
                torch.testing.assert_close(torch.cat(got[i]).double(), want[i], rtol=1e-5, atol=1e-5)
                tail = torch.cat([torch.zeros(taps - 1, C), us[i][:, :C]])[-(taps - 1):]
                torch.testing.assert_close(state[slots[i]].cpu(), tail)
            assert bool((state[[1, 2, 4, 7]] == 9.0).all())


# ---------------------------------------------------------------- the recurrence ----

@pytest.mark.parametrize("H,G,N,P,per_channel", [(3, 1, 12, 16, False), (4, 4, 40, 8, False), (2, 2, 72, 33, True), (1, 1, 130, 5, True),
                                                 (6, 3, 17, 64, False), (2, 2, 8, 96, True)])
def test_recurrence_against_the_plain_loop_and_carried_through_steps(H, G, N, P, per_channel):
    o = ops()
    g = torch.Generator().manual_seed(H * 1000 + N)
    lengths = [1, 150, 7]           # the long one runs in chunks (from zero, chunk starts, from the starts), the others in one pass
    slots = [4, 1, 2]
    state = torch.zeros(6, H, N, P, device=DEV)
    state[[0, 3, 5]] = 3.0
    data = []
    for n in lengths:
        q, k = torch.randn(n, G * N + 3, generator=g), torch.randn(n, G * N, generator=g)
        v = torch.randn(n, H * P, generator=g)
        a = torch.rand(n, H * N if per_channel else H, generator=g) * 0.3 + 0.7
        vs = torch.rand(n, H, generator=g) + 0.5
        data.append((q, k, v, a, vs))
    want = []
    for q, k, v, a, vs in data:
        n = q.shape[0]
        rep = H // G
        qq = q[:, :G * N].reshape(n, G, N).repeat_interleave(rep, 1).double()
        kk = k.reshape(n, G, N).repeat_interleave(rep, 1).double()
        aa = a.reshape(n, H, N if per_channel else 1).double()
        vv = (v.reshape(n, H, P) * vs[:, :, None]).double()
        out, S = plain.matrix_state_recurrence(aa, kk, vv, qq)
        want.append((out.reshape(n, H * P) * 0.5, S))
    for cuts in ([None], [3, 1, None], [70, None], [49, 33, None]):
        state[slots] = 0.0
        done, got = [0] * 3, [[] for _ in range(3)]
        for cut in cuts:
            take = [n - d if cut is None else min(cut, n - d) for n, d in zip(lengths, done)]
            live = [i for i, t in enumerate(take) if t > 0]
            if not live:
                continue
            part = [torch.cat([data[i][j][done[i]:done[i] + take[i]] for i in live]).to(DEV) for j in range(5)]
            _, _, start = batch_tables([take[i] for i in live])
            out = torch.empty(part[0].shape[0], H * P, device=DEV)
            longest = max(take[i] for i in live)
            need = o.decay_scan_scratch_floats(len(live), longest, H, N, P, per_channel)
            assert (need > 0) == (longest > 48)
            scratch = torch.full((need,), float("nan"), device=DEV) if need else None
            o.decay_scan(part[0][:, :G * N], part[1], part[2], part[3], state, i32([slots[i] for i in live]), start, out, H, G, per_channel,
                         v_scale=part[4], q_scale=0.5, max_count=longest, scratch=scratch)
            at = 0
            for i in live:
                got[i].append(out[at:at + take[i]].cpu())
                at += take[i]
                done[i] += take[i]
        for i in range(3):
            torch.testing.assert_close(torch.cat(got[i]).double(), want[i][0], rtol=2e-4, atol=2e-4)
            torch.testing.assert_close(state[slots[i]].cpu().double(), want[i][1], rtol=2e-4, atol=2e-4)
        assert bool((state[[0, 3, 5]] == 3.0).all())


def test_step_sizes_decays_and_channel_decays():
    o = ops()
    g = torch.Generator().manual_seed(5)
    T, H = 37, 5
    raw = torch.randn(T, H + 3, generator=g) * 4
    bias, a_log = torch.randn(H, generator=g), torch.randn(H, generator=g)
    dt, decay = torch.empty(T, H, device=DEV), torch.empty(T, H, device=DEV)
    o.step_decay(raw.to(DEV)[:, 2:2 + H], bias.to(DEV), a_log.to(DEV), dt, decay)
    want_dt = plain.softplus(raw[:, 2:2 + H].double() + bias.double())
    torch.testing.assert_close(dt.cpu().double(), want_dt, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(decay.cpu().double(), torch.exp(-torch.exp(a_log.double()) * want_dt), rtol=1e-5, atol=1e-6)
    z, b = torch.randn(T, 24, generator=g) * 5, torch.randn(24, generator=g)
    zz = z.to(DEV).clone()
    o.channel_decay(zz, b.to(DEV), 16.0)
    torch.testing.assert_close(zz.cpu().double(), torch.sigmoid(z.double() + b.double()) ** (1 / 16.0), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inner,groups,gate_first", [(48, 3, True), (192, 2, True), (60, 3, False), (130, 1, False)])
def test_gated_group_norm_in_both_orders(inner, groups, gate_first, dtype):
    o = ops()
    g = torch.Generator().manual_seed(inner)
    T, eps = 9, 1e-5
    y, gate, skip = (torch.randn(T, inner + 4, generator=g) for _ in range(3))
    heads = groups if not gate_first else inner // 4
    width = inner // heads
    D = torch.randn(heads, generator=g)
    gain = torch.randn(inner if gate_first else width, generator=g) + 1
    out = torch.empty(T, inner, dtype=dtype, device=DEV)
    yy = y[:, :inner].contiguous()
    o.gated_group_norm(yy.to(DEV), gate.to(DEV)[:, 1:1 + inner], gain.to(DEV), out, groups, eps, gate_first,
                       skip=skip.to(DEV)[:, :inner] if gate_first else None, skip_gain=D.to(DEV) if gate_first else None, head_width=width)
    gt = gate[:, 1:1 + inner].double()
    v = yy.double()
    if gate_first:
        v = (v + D.double().repeat_interleave(width) * skip[:, :inner].double()) * plain.silu(gt)
        want = plain.rms(v.reshape(T, groups, -1), eps).reshape(T, inner) * gain.double()
    else:
        want = (plain.rms(v.reshape(T, groups, -1), eps) * gain.double()).reshape(T, inner) * plain.silu(gt)
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(out.cpu().double(), want, **tol)


# ---------------------------------------------------------------- attention ----

def attention_case(o, dtype, H, G, d, dv, maps, lengths, pasts, window, slopes, softcap, rot, norm, loud, flash=False, pad=0):
    """Write whole sequences into a paged cache through ``unit_post`` (in two steps: ``pasts`` tokens, then the rest) and
    attend from the second step's tokens. ``loud``: (distance) -> one key at that distance behind the LAST query of each
    sequence gets a large score."""
    g = torch.Generator().manual_seed(H * 31 + d + window)
    n = len(lengths)
    pages_per = [math.ceil(L / 64) for L in lengths]
    total = sum(pages_per) + 3
    order = torch.randperm(total, generator=g).tolist()                 # pages scattered over the pool
    table = torch.full((n, max(pages_per) + 1), -1, dtype=torch.int32)
    at = 0
    for s, k in enumerate(pages_per):
        table[s, :k] = torch.tensor(order[at:at + k], dtype=torch.int32)
        at += k
    k_pool = torch.full((total, G, 64, maps * d), 7.0, dtype=dtype, device=DEV)      # stale contents must never be read
    v_pool = torch.full((total, G, 64, dv), 7.0, dtype=dtype, device=DEV)
    if pad:         # rows widened to ``pad`` channels: the spare channels are zero from the start and nobody writes them
        k_pool, v_pool = (torch.zeros((total, G, 64, pad), dtype=dtype, device=DEV) for _ in range(2))
        k_pool[..., :maps * d] = 7.0
        v_pool[..., :dv] = 7.0
    width = H * maps * d + G * maps * d + G * dv
    rows = [torch.randn(L, width + 2, generator=g) for L in lengths]
    qg, kg = (torch.randn(d, generator=g) + 1 for _ in range(2))
    half = rot // 2
    cos = sin = None
    if rot:
        ang = torch.arange(max(lengths))[:, None] * (100.0 ** (-torch.arange(half) * 2.0 / rot))[None, :]
        cos, sin = ang.cos().float(), ang.sin().float()
    for r, L in zip(rows, lengths):
        if loud is not None and L - 1 - loud >= 0:         # the last query and the key at that distance point the same way
            qs = r[L - 1, :H * maps * d].reshape(H * maps, d)
            big = torch.ones(d) * 3.0
            qs[:] = big
            ks = r[L - 1 - loud, H * maps * d:H * maps * d + G * maps * d].reshape(G * maps, d)
            ks[:] = big * 3
    want, got = [], []
    for step in range(2):
        counts = [p if step == 0 else L - p for L, p in zip(lengths, pasts)]
        begin = [0 if step == 0 else p for p in pasts]
        live = [i for i, c in enumerate(counts) if c > 0]
        if not live:
            continue
        part = torch.cat([rows[i][begin[i]:begin[i] + counts[i]] for i in live]).to(DEV)
        tok_seq, tok_pos, _ = batch_tables([counts[i] for i in live], [begin[i] for i in live])
        tab = table[live].contiguous().to(DEV)
        T = part.shape[0]
        q = torch.full((T, H * maps, pad or d), 5.0, dtype=dtype, device=DEV)
        o.unit_post(part[:, :width], qg.to(DEV) if norm else None, kg.to(DEV) if norm else None, None if cos is None else cos.to(DEV),
                    None if sin is None else sin.to(DEV), q, k_pool, v_pool, tok_seq, tok_pos, tab, H, G, maps, d, dv, rot, 1e-6, pad=pad)
        if step == 0:
            continue
        if pad:         # 2 H query heads over rows of ``pad`` channels on the tensor-core kernels, float32 results
            counts_live = [counts[i] for i in live]
            _, _, start = batch_tables(counts_live)
            past_d, counts_d = i32([begin[i] for i in live]), i32(counts_live)
            wide = torch.empty(T, H * maps * pad, device=DEV)
            if max(counts_live) == 1:
                scratch = torch.empty(o.decode_scratch_floats(len(live), H * maps, pad, 2), device=DEV)
                o.attention_decode(q, k_pool, v_pool, wide, start, past_d, tab, H * maps, G, pad, window, 0.3, 2, scratch, out_f32=True)
            else:
                o.attention_prefill(q, k_pool, v_pool, wide, start, past_d, counts_d, tab, max(counts_live), H * maps, G, pad, window, 0.3,
                                    out_f32=True)
            at = 0
            for i in live:
                got.append(wide.view(T, H * maps, pad)[at:at + counts[i], :, :dv].float().cpu())
                at += counts[i]
            continue
        out = torch.empty(T, H * maps, dv, dtype=torch.float32 if maps > 1 else dtype, device=DEV)
        if flash:       # the tensor-core kernels: single tokens through the split-KV kernel, the rest through the prompt kernel
            counts_live = [counts[i] for i in live]
            _, _, start = batch_tables(counts_live)
            past_d, counts_d = i32([begin[i] for i in live]), i32(counts_live)
            sl = None if slopes is None else slopes.to(DEV)
            if flash == "tc" and max(counts_live) > 1:      # the tcgen05 kernels (one page a step and two pages a step in turn)
                o.attention_tc(q, k_pool, v_pool, out.view(T, -1), start, past_d, counts_d, tab, max(counts_live), H, G, d, window, 0.3,
                               wide=bool(len(lengths) % 2), max_keys=max(lengths), slopes=sl, softcap=softcap)
            elif max(counts_live) == 1:
                splits = 3
                scratch = torch.empty(o.decode_scratch_floats(len(live), H, d, splits), device=DEV)
                o.attention_decode(q, k_pool, v_pool, out.view(T, -1), start, past_d, tab, H, G, d, window, 0.3, splits, scratch,
                                   slopes=sl, softcap=softcap)
            else:
                o.attention_prefill(q, k_pool, v_pool, out.view(T, -1), start, past_d, counts_d, tab, max(counts_live), H, G, d, window, 0.3,
                                    slopes=sl, softcap=softcap)
        else:
            o.attention_scored(q, k_pool, v_pool, out.view(T, -1) if maps == 1 else out, tok_seq, tok_pos, tab, H, G, d, window, 0.3,
                               slopes=None if slopes is None else slopes.to(DEV), softcap=softcap, maps=maps, value_dim=dv)
        at = 0
        for i in live:
            got.append(out[at:at + counts[i]].float().cpu())
            at += counts[i]
    for r, L, p in zip(rows, lengths, pasts):
        if L - p <= 0:
            continue
        r = r.double()
        qq = r[:, :H * maps * d].reshape(L, H * maps, d)
        kk = r[:, H * maps * d:H * maps * d + G * maps * d].reshape(L, G * maps, d)
        vv = r[:, H * maps * d + G * maps * d:width].reshape(L, G, dv)
        if norm:
            qq, kk = plain.rms(qq, 1e-6) * qg.double(), plain.rms(kk, 1e-6) * kg.double()
        if rot:
            spec = {"base": 100.0, "dims": rot}
            qq, kk = plain.rotate_halves(qq, torch.arange(L), spec), plain.rotate_halves(kk, torch.arange(L), spec)
        if dtype == torch.bfloat16:      # the query buffer and the cache rows are rounded once, at their store
            qq, kk, vv = (t.to(torch.bfloat16).double() for t in (qq, kk, vv))
        outs = []
        for m in range(maps):
            outs.append(plain.softmax_attention(qq.reshape(L, H, maps, d)[:, :, m], kk.reshape(L, G, maps, d)[:, :, m], vv, 0.3, window,
                                                slopes=None if slopes is None else slopes.double(), softcap=softcap))
        want.append(torch.stack(outs, dim=2).reshape(L, H * maps, dv)[p:])
    return got, want


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [1, 2, 37, 64, 65, 130])
def test_a_loud_key_just_inside_and_just_outside_the_window(window, dtype):
    """For the last query of prompts and of single decoded tokens: the key at distance window - 1 is seen (the output is
    its value), the key at distance window is not."""
    o = ops()
    H, G, d, dv = 4, 2, 16, 24
    slopes = plain.distance_slopes(H, torch.float32)
    tol = dict(rtol=2e-4, atol=2e-4) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)
    for loud in (window - 1, window):
        for lengths, pasts in (([window + 70, 200, 3], [0, 0, 0]), ([window + 70, 200, 3], [window + 69, 199, 2])):
            got, want = attention_case(o, dtype, H, G, d, dv, 1, lengths, pasts, window, slopes, 0.0, 0, True, loud)
            for a, b in zip(got, want):
                torch.testing.assert_close(a.double(), b, **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,maps,rot,softcap", [(6, 3, 24, 16, 1, 16, 2.0), (2, 1, 16, 40, 2, 8, 0.0), (4, 4, 64, 64, 1, 64, 30.0),
                                                       (3, 3, 8, 16, 2, 0, 0.0), (4, 2, 32, 64, 2, 32, 0.0)])
def test_far_keys_soft_caps_rotation_and_two_maps(H, G, d, dv, maps, rot, softcap, dtype):
    """A loud key hundreds of tokens back, across several scattered pages, in prompts, portions and single tokens; with a
    soft cap the loud score is flattened, with two maps both maps come out side by side."""
    o = ops()
    tol = dict(rtol=2e-4, atol=2e-4) if dtype == torch.float32 else dict(rtol=3e-2, atol=3e-2)
    for lengths, pasts, loud in (([400, 66, 1], [0, 0, 0], 333), ([400, 129], [399, 64], 333), ([64, 65], [63, 2], 63)):
        got, want = attention_case(o, dtype, H, G, d, dv, maps, lengths, pasts, 0, None, softcap, rot, False, loud)
        for a, b in zip(got, want):
            torch.testing.assert_close(a.double(), b, **tol)


@pytest.mark.parametrize("path", [True, "tc"])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("window,softcap", [(0, 5.0), (37, 0.0), (64, 0.0), (130, 3.0), (0, 0.0)])
def test_the_tensor_core_kernels_know_the_penalty_and_the_cap(d, window, softcap, path):
    """The mma.sync prompt and single-token kernels and the two tcgen05 prompt kernels with a distance penalty a head, a soft
    cap and a window: a loud key just inside and just outside the window (or far back without one), in whole prompts,
    portions and single tokens."""
    o = ops()
    H, G = 8, 2
    slopes = plain.distance_slopes(H, torch.float32) if softcap != 5.0 else None
    tol = dict(rtol=3e-2, atol=3e-2)
    for loud in ((window - 1, window) if window else (300,)):
        for lengths, pasts in (([window + 270, 200, 3], [0, 0, 0]), ([window + 270, 200, 70], [window + 269, 199, 69]), ([window + 270, 150], [100, 64])):
            got, want = attention_case(o, torch.bfloat16, H, G, d, d, 1, lengths, pasts, window, slopes, softcap, d, True, loud, flash=path)
            for a, b in zip(got, want):
                torch.testing.assert_close(a.double(), b, **tol)
    o.gemm_tc_check(torch.device(DEV))          # no bounded wait inside a tensor-memory kernel gave up


@pytest.mark.parametrize("H,G,d,dv,rot,pad", [(2, 1, 16, 40, 8, 64), (4, 2, 32, 64, 32, 64), (4, 1, 48, 96, 48, 128), (3, 3, 8, 16, 0, 64),
                                              (8, 4, 64, 128, 64, 128)])
def test_two_maps_on_the_tensor_core_kernels(H, G, d, dv, rot, pad):
    """Differential attention's two maps as 2 H query heads over widened rows: a query is zero outside its map's channels,
    the cache's spare channels are zero, so the kernels' products over the whole row are the maps' own scores."""
    o = ops()
    tol = dict(rtol=3e-2, atol=3e-2)
    for lengths, pasts, loud in (([400, 66, 1], [0, 0, 0], 333), ([400, 129], [399, 128], 333), ([200, 65], [63, 2], 63)):
        got, want = attention_case(o, torch.bfloat16, H, G, d, dv, 2, lengths, pasts, 0, None, 0.0, rot, False, loud, pad=pad)
        for a, b in zip(got, want):
            torch.testing.assert_close(a.double(), b, **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_differential_combination(dtype):
    o = ops()
    g = torch.Generator().manual_seed(3)
    T, H, dv, lam, diff, eps = 11, 3, 40, 0.83, 0.3, 1e-5
    a = torch.randn(T, H * 2, dv, generator=g)
    gate = torch.randn(T, H + 2, generator=g)
    out = torch.empty(T, H * dv, dtype=dtype, device=DEV)
    o.diff_combine(a.to(DEV), gate.to(DEV)[:, 1:1 + H], out, H, dv, lam, 1 - diff, eps)
    aa = a.double().reshape(T, H, 2, dv)
    want = plain.rms(aa[:, :, 0] - lam * aa[:, :, 1], eps) * (1 - diff) * torch.sigmoid(gate[:, 1:1 + H].double())[:, :, None]
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(out.cpu().double().reshape(T, H, dv), want, **tol)


# ---------------------------------------------------------------- copies of the stream, joins, gates ----

@pytest.mark.parametrize("S,d", [(1, 40), (3, 72), (4, 320), (8, 33), (16, 64)])
def test_copies_of_the_stream(S, d):
    o = ops()
    g = torch.Generator().manual_seed(S * 7 + d)
    T, eps, mult = 6, 1e-5, 0.7
    x0 = torch.randn(T, d, generator=g)
    xs = torch.empty(T, S * d, device=DEV)
    o.streams_fill(x0.to(DEV), xs, S)
    assert torch.equal(xs.cpu().reshape(T, S, d), x0[:, None].expand(T, S, d))
    xs = torch.randn(T, S, d, generator=g)
    w = {"in": torch.randn(S, generator=g), "out": torch.randn(S, generator=g), "mix": torch.randn(S, S, generator=g)}
    gain = torch.randn(d, generator=g) + 1
    per_stream = xs.permute(1, 0, 2).double()
    h = torch.empty(T, d, device=DEV)
    o.hyper_read(xs.reshape(T, S * d).to(DEV), w["in"].to(DEV), gain.to(DEV), h, eps)
    want = plain.rms(plain.hyper_read(per_stream, {k: v.double() for k, v in w.items()}, ""), eps) * gain.double()
    torch.testing.assert_close(h.cpu().double(), want, rtol=1e-5, atol=1e-5)
    y = torch.randn(T, d, generator=g)
    dev = xs.reshape(T, S * d).to(DEV).clone()
    o.hyper_write(dev, y.to(DEV), w["mix"].to(DEV), w["out"].to(DEV), mult)
    want = plain.hyper_write(per_stream, y.double(), {k: v.double() for k, v in w.items()}, "", mult).permute(1, 0, 2)
    torch.testing.assert_close(dev.cpu().double().reshape(T, S, d), want, rtol=1e-5, atol=1e-5)
    total = torch.empty(T, d, device=DEV)
    o.streams_sum(dev, total)
    torch.testing.assert_close(total.cpu().double(), want.sum(dim=1), rtol=1e-5, atol=1e-5)
    # without coefficients: one copy, x <- x + mult * y
    one = x0.to(DEV).clone()
    o.hyper_write(one, y.to(DEV), None, None, mult)
    torch.testing.assert_close(one.cpu(), x0 + mult * y)


def test_joins_of_two_mixers_and_the_row_gate():
    o = ops()
    g = torch.Generator().manual_seed(11)
    T, d, eps = 7, 90, 1e-5
    a, b, base = (torch.randn(T, d, generator=g) for _ in range(3))
    ga, gb = (torch.randn(d, generator=g) + 1 for _ in range(2))
    want = 0.5 * (plain.rms(a.double(), eps) * ga.double() + plain.rms(b.double(), eps) * gb.double())
    for acc in (False, True):
        t = base.to(DEV).clone()
        o.pair_combine(a.to(DEV), b.to(DEV), t, ga.to(DEV), gb.to(DEV), 0.5, 0.5, eps, accumulate=acc)
        torch.testing.assert_close(t.cpu().double(), want + (base.double() if acc else 0), rtol=1e-5, atol=1e-5)
        t = base.to(DEV).clone()
        o.pair_combine(a.to(DEV), b.to(DEV), t, None, None, 1.2, 1.1, 0.0, accumulate=acc)
        torch.testing.assert_close(t.cpu().double(), 1.2 * a.double() + 1.1 * b.double() + (base.double() if acc else 0), rtol=1e-5, atol=1e-5)
    for dtype in (torch.float32, torch.bfloat16):
        h = torch.randn(T, 50, generator=g).to(dtype)
        w = torch.randn(50, generator=g)
        gate = torch.sigmoid(h.double() @ w.double())[:, None]
        for acc in (False, True):
            t = base.to(DEV).clone()
            o.row_gate(h.to(DEV), w.to(DEV), a.to(DEV), t, accumulate=acc)
            torch.testing.assert_close(t.cpu().double(), gate * a.double() + (base.double() if acc else 0), rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("E,top", [(5, 2), (16, 4), (3, 3), (1, 1), (40, 1)])
def test_routing_weights_are_divided_by_their_sum(E, top):
    o = ops()
    g = torch.Generator().manual_seed(E)
    T, d = 33, 48
    h = torch.randn(T, d, generator=g)
    wr = torch.randn(E, d, generator=g) * 0.5
    pairs = T * top
    choice, rank, place, order = (torch.zeros(pairs, dtype=torch.int32, device=DEV) for _ in range(4))
    counts = torch.zeros(E, dtype=torch.int32, device=DEV)
    weight = torch.zeros(pairs, device=DEV)
    logits = torch.zeros(T, E, device=DEV)
    o.moe_route(h.to(DEV), wr.to(DEV), None, choice, weight, rank, counts, place, order, top, None, logits, None, scoring="softmax_norm")
    s = plain.router_scores(h, {"router": wr}, "").double()
    srt = torch.sort(s, dim=-1, descending=True, stable=True)
    assert torch.equal(choice.cpu().reshape(T, top).long(), srt.indices[:, :top])
    want = srt.values[:, :top] / (srt.values[:, :top].sum(dim=-1, keepdim=True) + 1e-20)
    torch.testing.assert_close(weight.cpu().double().reshape(T, top), want, rtol=1e-4, atol=1e-6)
