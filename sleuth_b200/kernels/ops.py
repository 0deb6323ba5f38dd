"""Thin, checked Python fronts of the CUDA launchers.

Every function takes CUDA tensors, checks device, dtype, contiguity and the sizes that tie the
arguments together, and launches on the stream it is given (an integer handle, the current torch
stream by default). Nothing here computes with torch operations, with one exception that the
architecture's own engine makes too: the bfloat16 matrix product of more rows than the skinny
kernel takes is a library product (cuBLAS through ``torch.mm``), as the reference's ``nn.Linear``
is (sleuth/forge/model/attention.py:106-108,157; mlp.py:38-41; transformer.py:302).
"""

from __future__ import annotations

import ctypes
import os

import torch

from . import library

DT = {torch.float32: 0, torch.bfloat16: 1}
ACTIVATIONS = {"silu": 0, "relu": 1, "clamped_swish": 2, "gelu_tanh": 3}
ROUTE_SCORINGS = {"softmax_top": 0, "sigmoid": 1, "softmax": 2, "softmax_norm": 3}


def lib() -> library.KernelLibrary:
    return library.load()


def current_stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t):
    return None if t is None else t.data_ptr()


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise ValueError(msg)


def _cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not (t.is_cuda and t.is_contiguous()):
            _need(t.is_cuda, "the kernels of sleuth_b200 run on CUDA tensors only")
            _need(False, f"tensor of shape {tuple(t.shape)} must be contiguous")


def embed(ids: torch.Tensor, table: torch.Tensor, x: torch.Tensor, scale: float = 1.0, stream=None,
          ids_map: torch.Tensor | None = None) -> None:
    """x[t] = table[ids[t]] * scale, or table[ids[ids_map[t]]] with a map. Ids outside the table are clamped
    (the caller checks host ids; ids that a sampler left on the device lie inside by construction)."""
    _cuda(ids, table, x, ids_map)
    T, d = x.shape
    _need(ids.dtype == torch.int32 and (ids_map is not None or ids.numel() >= T), "embed: ids must be int32, one per row of x")
    _need(ids_map is None or (ids_map.dtype == torch.int32 and ids_map.numel() >= T), "embed: the map is int32, one per row")
    _need(table.shape[1] == d and x.dtype == torch.float32 and table.dtype in DT, "embed: shapes or dtypes disagree")
    lib().call("slb_embed", _p(ids), _p(ids_map), _p(table), DT[table.dtype], _p(x), T, d, table.shape[0], float(scale),
               stream if stream is not None else current_stream())


def rmsnorm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, eps: float, rows: torch.Tensor | None = None,
            stream=None) -> None:
    _cuda(x, w, out, rows)
    R, d = out.shape
    _need(x.dtype == torch.float32 and w.dtype == torch.float32 and out.dtype in DT, "rmsnorm: dtypes")
    _need(x.shape[1] == d and w.numel() == d, "rmsnorm: widths disagree")
    if rows is None:
        _need(x.shape[0] >= R, "rmsnorm: fewer input rows than output rows")
    else:
        _need(rows.dtype == torch.int32 and rows.numel() >= R, "rmsnorm: rows must be int32, one per output row")
    lib().call("slb_rmsnorm", _p(x), _p(w), _p(out), DT[out.dtype], _p(rows), R, d, float(eps),
               stream if stream is not None else current_stream())


def add(x: torch.Tensor, delta: torch.Tensor, stream=None) -> None:
    _cuda(x, delta)
    _need(x.dtype == torch.float32 and delta.dtype in DT and x.numel() == delta.numel(), "add: shapes or dtypes")
    lib().call("slb_add", _p(x), _p(delta), DT[delta.dtype], x.numel(),
               stream if stream is not None else current_stream())


def swiglu(gu: torch.Tensor, act: torch.Tensor, stream=None) -> None:
    _cuda(gu, act)
    T, inter = act.shape
    _need(gu.shape == (T, 2 * inter) and gu.dtype == act.dtype and act.dtype in DT, "swiglu: shapes or dtypes")
    lib().call("slb_swiglu", _p(gu), _p(act), DT[act.dtype], T, inter,
               stream if stream is not None else current_stream())


def gated_act(gu: torch.Tensor, act: torch.Tensor, kind: str = "silu", stream=None, limit: float = 0.0,
              alpha: float = 1.0) -> None:
    """act[t, j] = f(gu[t, j], gu[t, inter + j]): silu(g) u, relu(g) u, the clamped swish
    min(g, limit) sigmoid(alpha min(g, limit)) (clamp(u, -limit, limit) + 1), or the tanh form of gelu(g) u."""
    _cuda(gu, act)
    T, inter = act.shape
    _need(kind in ACTIVATIONS, f"gated_act: activation {kind!r} is not one of {sorted(ACTIVATIONS)}")
    _need(gu.shape == (T, 2 * inter) and gu.dtype == act.dtype and act.dtype in DT, "gated_act: shapes or dtypes")
    lib().call("slb_gated_act", _p(gu), _p(act), DT[act.dtype], T, inter, ACTIVATIONS[kind], float(limit), float(alpha),
               stream if stream is not None else current_stream())


def layernorm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, eps: float, rows: torch.Tensor | None = None,
              stream=None, w2: torch.Tensor | None = None, out2: torch.Tensor | None = None) -> None:
    """out[r] = (x[row] - mean) / sqrt(var + eps) * w (a gain, no bias); ``out`` may be ``x`` itself. With ``w2`` and
    ``out2``: the same rows once more with another gain, in the same pass (mean and variance are shared)."""
    _cuda(x, w, out, rows, w2, out2)
    R, d = out.shape
    _need(x.dtype == torch.float32 and w.dtype == torch.float32 and out.dtype in DT, "layernorm: dtypes")
    _need(x.shape[1] == d and w.numel() == d, "layernorm: widths disagree")
    _need((w2 is None) == (out2 is None), "layernorm: a second gain and a second output go together")
    if w2 is not None:
        _need(w2.dtype == torch.float32 and w2.numel() == d and out2.shape == out.shape and out2.dtype == out.dtype
              and out.data_ptr() != x.data_ptr(), "layernorm: the second gain and output")
    if rows is None:
        _need(x.shape[0] >= R, "layernorm: fewer input rows than output rows")
    else:
        _need(rows.dtype == torch.int32 and rows.numel() >= R, "layernorm: rows must be int32, one per output row")
    lib().call("slb_layernorm", _p(x), _p(w), _p(out), _p(w2), _p(out2), DT[out.dtype], _p(rows), R, d, float(eps),
               stream if stream is not None else current_stream())


def softcap(v: torch.Tensor, cap: float, stream=None) -> None:
    """v <- cap * tanh(v / cap) in place; v float32 [rows, cols] with unit column stride."""
    _need(v.is_cuda and v.dtype == torch.float32 and v.dim() == 2 and v.stride(1) == 1, "softcap: a float32 matrix")
    lib().call("slb_softcap", _p(v), v.stride(0) if v.shape[0] > 1 else v.shape[1], v.shape[0], v.shape[1], float(cap),
               stream if stream is not None else current_stream())


def stream_inject(x: torch.Tensor, again: torch.Tensor | None, row: torch.Tensor | None, stream=None) -> None:
    """x[t] += again[t] + row: ``again`` has the stream's shape, ``row`` one value per channel; either may be None."""
    _cuda(x, again, row)
    T, d = x.shape
    _need(x.dtype == torch.float32, "stream_inject: the stream is float32")
    _need(again is None or (again.dtype == torch.float32 and again.shape == x.shape), "stream_inject: the added rows")
    _need(row is None or (row.dtype == torch.float32 and row.numel() == d), "stream_inject: the added vector")
    lib().call("slb_stream_inject", _p(x), _p(again), _p(row), T, d, stream if stream is not None else current_stream())


def pair_embed(ids, ids_map, pairs, x, tok_seq, tok_pos, seq_start, slots, last, vocab: int, buckets: int, mul_prev: int,
               mul_cur: int, stream=None, table=None, scale: float = 1.0) -> None:
    """x[t] += pairs[(previous token * mul_prev + token * mul_cur) mod buckets], or pairs[buckets] for a sequence's first
    token. ``pairs`` [buckets + 1, dim]; ``last`` int32 [slots]: every sequence's last token so far, read for the first
    token of a step and left for the next step. With ``table`` [vocab, dim] (of ``pairs``' dtype) the token's own row comes
    in the same pass: x[t] = table[token] * scale + the pair's row."""
    _cuda(ids, ids_map, pairs, x, tok_seq, tok_pos, seq_start, slots, last, table)
    T, d = x.shape
    _need(x.dtype == torch.float32 and pairs.dtype in DT and tuple(pairs.shape) == (buckets + 1, d), "pair_embed: table or stream")
    _need(last.dtype == torch.int32 and last.dim() >= 1 and ids.dtype == torch.int32, "pair_embed: int32 ids and state")
    _need(ids_map is not None or ids.numel() >= T, "pair_embed: one id per row of x")
    _need(table is None or (table.dtype == pairs.dtype and tuple(table.shape) == (vocab, d)), "pair_embed: the token table")
    for t in (tok_seq, tok_pos, seq_start, slots):
        _need(t.dtype == torch.int32, "pair_embed: the batch tables are int32")
    lib().call("slb_pair_embed", _p(ids), _p(ids_map), _p(pairs), DT[pairs.dtype], _p(x), _p(tok_seq), _p(tok_pos), _p(seq_start),
               _p(slots), _p(last), T, d, int(vocab), int(buckets), int(mul_prev), int(mul_cur), _p(table), float(scale),
               stream if stream is not None else current_stream())


def gated_norm_add(x, y, g, bias, gain, eps: float, stream=None) -> None:
    """x += rmsnorm(y * sigmoid(g + bias)) * gain, row by row in float32; without ``g``: x += rmsnorm(y) * gain. ``y`` may be
    overwritten. ``g`` may be a view of a wider float32 matrix (unit column stride)."""
    _cuda(x, y, bias, gain)
    T, d = x.shape
    _need(x.dtype == torch.float32 and y.dtype == torch.float32 and y.shape == x.shape, "gated_norm_add: the stream and the sublayer's result are float32")
    _need(gain.dtype == torch.float32 and gain.numel() == d, "gated_norm_add: gain")
    stride = 0
    if g is not None:
        _need(g.is_cuda and g.dtype == torch.float32 and g.dim() == 2 and g.shape == x.shape and g.stride(1) == 1,
              "gated_norm_add: the gate's values are float32, one per element")
        stride = g.stride(0) if T > 1 else d
        _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == d), "gated_norm_add: bias")
    lib().call("slb_gated_norm_add", _p(x), _p(y), _p(g), stride, _p(bias) if g is not None else None, _p(gain), T, d, float(eps),
               stream if stream is not None else current_stream())


def stream_pair(a, b, out, stream=None) -> None:
    """out[t] = [a[t] | b[t]]: two float32 streams side by side in ``out``'s dtype."""
    _cuda(a, b, out)
    T, d = a.shape
    _need(a.dtype == torch.float32 and b.dtype == torch.float32 and b.shape == a.shape and out.shape == (T, 2 * d)
          and out.dtype in DT, "stream_pair: shapes or dtypes")
    lib().call("slb_stream_pair", _p(a), _p(b), _p(out), DT[out.dtype], T, d, stream if stream is not None else current_stream())


def scale(v: torch.Tensor, factor: float, stream=None, add: torch.Tensor | None = None) -> None:
    """v <- v * factor (+ add[column]) in place; v float32 [rows, cols] with unit column stride."""
    _need(v.is_cuda and v.dtype == torch.float32 and v.dim() == 2 and v.stride(1) == 1, "scale: a float32 matrix")
    _need(add is None or (add.is_cuda and add.dtype == torch.float32 and add.numel() == v.shape[1]), "scale: the added row")
    lib().call("slb_scale", _p(v), v.stride(0) if v.shape[0] > 1 else v.shape[1], v.shape[0], v.shape[1], float(factor), _p(add),
               stream if stream is not None else current_stream())


def mingru_scratch_floats(n_seqs: int, max_count: int, width: int) -> int:
    fn = lib().dll.slb_mingru_scratch_floats
    fn.argtypes, fn.restype = [ctypes.c_int] * 3, ctypes.c_longlong
    return int(fn(int(n_seqs), int(max_count), int(width)))


def mingru(p, bz, bu, state, slots, seq_start, y, max_count: int, scratch=None, stream=None) -> None:
    """The minGRU recurrence over each sequence's tokens of the step. p [T, 3 * W] float32: the stacked projections
    [z | u | g]; z = sigmoid(z + bz), u = u + bu, c = u + 1/2 where u >= 0 else sigmoid(u);
    S <- (1 - z) S + z c from state[slot]; y[t] = S * silu(g). ``state`` float32 [slots, W] is updated."""
    _cuda(bz, bu, state, slots, seq_start, y, scratch)
    _need(p.is_cuda, "mingru: the projections live on the device")
    T, W = y.shape
    n = slots.numel()
    _need(p.dtype == torch.float32 and p.shape == (T, 3 * W) and p.stride(1) == 1,
          "mingru: the projections are float32 [tokens, 3 * width] (possibly a view of a wider matrix)")
    _need(bz.dtype == torch.float32 and bu.dtype == torch.float32 and bz.numel() == W and bu.numel() == W, "mingru: biases")
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.shape[1] == W and y.dtype in DT, "mingru: state or output")
    _need(slots.dtype == torch.int32 and seq_start.dtype == torch.int32 and seq_start.numel() >= n + 1, "mingru: batch tables")
    need = mingru_scratch_floats(n, max_count, W)
    _need(need == 0 or (scratch is not None and scratch.dtype == torch.float32 and scratch.numel() >= need), "mingru: scratch")
    lib().call("slb_mingru", _p(p), p.stride(0) if T > 1 else 3 * W, _p(bz), _p(bu), _p(state), _p(slots), _p(seq_start), _p(y),
               _p(scratch), n, int(max_count), W, DT[y.dtype], stream if stream is not None else current_stream())


def qkv_post(qkv, bias, q_gain, k_gain, cos, sin, q_out, k_pool, v_pool, tok_seq, tok_pos, block_table,
             heads: int, kv_heads: int, head_dim: int, rot_dim: int, eps: float, stream=None) -> None:
    _cuda(qkv, bias, q_gain, k_gain, cos, sin, q_out, k_pool, v_pool, tok_seq, tok_pos, block_table)
    T = q_out.shape[0]
    rows = heads + 2 * kv_heads
    _need(qkv.shape == (T, rows * head_dim) and q_out.shape[1:] == (heads, head_dim), "qkv_post: shapes disagree")
    _need(qkv.dtype == q_out.dtype and qkv.dtype in DT, "qkv_post: dtypes")
    for v in (bias, q_gain, k_gain, cos, sin):
        _need(v is None or v.dtype == torch.float32, "qkv_post: gains, biases and tables are float32")
    _need(bias is None or bias.numel() == rows * head_dim, "qkv_post: bias length")
    _need(q_gain is None or (q_gain.numel() == head_dim and k_gain.numel() == head_dim), "qkv_post: gain length")
    if rot_dim:
        _need(cos is not None and cos.shape[1] == rot_dim // 2 and sin.shape == cos.shape, "qkv_post: rotation tables")
    stride = 0
    if kv_heads and k_pool is not None:
        _need(k_pool.dtype == qkv.dtype and k_pool.shape == v_pool.shape and
              tuple(k_pool.shape[1:]) == (kv_heads, 64, head_dim), "qkv_post: cache pool shape or dtype")
        _need(block_table.dtype == torch.int32 and block_table.dim() == 2, "qkv_post: block table")
        stride = block_table.shape[1]
    _need(tok_seq.dtype == torch.int32 and tok_pos.dtype == torch.int32, "qkv_post: token tables are int32")
    lib().call("slb_qkv_post", _p(qkv), _p(bias), _p(q_gain), _p(k_gain), _p(cos), _p(sin), _p(q_out), _p(k_pool),
               _p(v_pool), _p(tok_seq), _p(tok_pos), _p(block_table), stride, T, heads, kv_heads, head_dim, rot_dim,
               float(eps), DT[qkv.dtype], stream if stream is not None else current_stream())


def qkv_post_span(qkv, q_gain, k_gain, cos, sin, q_out, k_pool, v_pool, tok_seq, tok_pos, block_table, heads: int,
                  kv_heads: int, key_dim: int, value_dim: int, rot_dim: int, neighbours: bool, whole: bool, eps: float,
                  stream=None, norm_dim: int = 0) -> None:
    """What follows separate q, k and v projections whose float32 results lie side by side in ``qkv``
    [T, heads * key_dim + kv_heads * key_dim + kv_heads * value_dim]: RMS norm of q and k (``whole``: over the whole
    projection with gains of that length; else per head with gains [key_dim]; no gains: none), rotation of each head's
    first ``rot_dim`` channels (``neighbours``: pairs (2i, 2i + 1); else (i, i + rot_dim / 2)), q into ``q_out``
    [T, heads, key_dim], k and v into the token's cache row (pools [pages, kv_heads, 64, key_dim | value_dim]).
    ``norm_dim``: how many channels of a head count in the norms' means, when the heads end in zero channels that only
    pad them (0 = ``key_dim``)."""
    _cuda(qkv, q_gain, k_gain, cos, sin, q_out, k_pool, v_pool, tok_seq, tok_pos, block_table)
    T = q_out.shape[0]
    _need(qkv.dtype == torch.float32 and qkv.shape == (T, (heads + kv_heads) * key_dim + kv_heads * value_dim),
          "qkv_post_span: the projections' float32 rows")
    _need(q_out.shape[1:] == (heads, key_dim) and q_out.dtype in DT, "qkv_post_span: q_out")
    n_q, n_k = (heads * key_dim, kv_heads * key_dim) if whole else (key_dim, key_dim)
    for g, n in ((q_gain, n_q), (k_gain, n_k)):
        _need(g is None or (g.dtype == torch.float32 and g.numel() == n), "qkv_post_span: gains")
    if rot_dim:
        _need(cos is not None and cos.dtype == torch.float32 and cos.shape[1] == rot_dim // 2 and sin.shape == cos.shape,
              "qkv_post_span: rotation tables")
    stride = 0
    if k_pool is not None:
        _need(k_pool.dtype == v_pool.dtype == q_out.dtype and tuple(k_pool.shape[1:]) == (kv_heads, 64, key_dim)
              and tuple(v_pool.shape[1:]) == (kv_heads, 64, value_dim) and k_pool.shape[0] == v_pool.shape[0],
              "qkv_post_span: cache pool shape or dtype")
        _need(block_table.dtype == torch.int32 and block_table.dim() == 2, "qkv_post_span: block table")
        stride = block_table.shape[1]
    _need(tok_seq.dtype == torch.int32 and tok_pos.dtype == torch.int32, "qkv_post_span: token tables are int32")
    lib().call("slb_qkv_post_span", _p(qkv), _p(q_gain), _p(k_gain), _p(cos), _p(sin), _p(q_out), _p(k_pool), _p(v_pool),
               _p(tok_seq), _p(tok_pos), _p(block_table), stride, T, heads, kv_heads, key_dim, value_dim, rot_dim,
               1 if neighbours else 0, 1 if whole else 0, float(eps), int(norm_dim), DT[q_out.dtype],
               stream if stream is not None else current_stream())


def attention(q, k_pool, v_pool, out, tok_seq, tok_pos, block_table, heads: int, kv_heads: int, head_dim: int,
              window: int, scale: float, stream=None, sinks=None, value_dim: int = 0) -> None:
    """The general attention kernel. ``sinks`` [heads] float32: a learned score per head that joins the softmax
    denominator (unscaled, once, without a value). ``value_dim``: width of the value rows and of a head's output when it
    is not ``head_dim``."""
    _cuda(q, k_pool, v_pool, out, tok_seq, tok_pos, block_table, sinks)
    T = q.shape[0]
    vd = value_dim or head_dim
    _need(q.shape == (T, heads, head_dim) and out.shape == (T, heads * vd), "attention: shapes disagree")
    _need(q.dtype == out.dtype == k_pool.dtype == v_pool.dtype and q.dtype in DT, "attention: dtypes")
    _need(tuple(k_pool.shape[1:]) == (kv_heads, 64, head_dim) and tuple(v_pool.shape[1:]) == (kv_heads, 64, vd)
          and k_pool.shape[0] == v_pool.shape[0], "attention: pool shape")
    _need(block_table.dtype == torch.int32 and block_table.dim() == 2, "attention: block table")
    _need(sinks is None or (sinks.dtype == torch.float32 and sinks.numel() == heads), "attention: sinks are float32, one per head")
    lib().call("slb_attention_generic", _p(q), _p(k_pool), _p(v_pool), _p(out), _p(tok_seq), _p(tok_pos),
               _p(block_table), block_table.shape[1], T, heads, kv_heads, head_dim, int(window), float(scale),
               _p(sinks), vd, DT[q.dtype], stream if stream is not None else current_stream())


def flash_supported(head_dim: int, dtype: torch.dtype) -> bool:
    """Whether the tensor-core attention kernels take this head size and dtype."""
    return dtype == torch.bfloat16 and head_dim in (64, 128)


_SMS: dict = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the device, asked of the library once (148 on a B200). The launch choices made
    in Python count with the same number as those made in the launchers."""
    key = torch.cuda.current_device() if device is None else torch.device(device).index
    if key not in _SMS:
        fn = lib().dll.slb_sm_count
        fn.restype = ctypes.c_int
        with torch.cuda.device(key):
            _SMS[key] = int(fn())
    return _SMS[key]


def decode_splits(n_seqs: int, kv_heads: int, group: int, table_stride: int, sms: int | None = None) -> int:
    """Slices of the key range per (sequence, kv head) in a decode step: enough blocks to fill the
    GPU a few times over, never more than a sequence can have pages. It depends on the batch size
    only, not on the lengths, so a captured step stays valid as sequences grow. ``sms``: the device's
    multiprocessors (asked of the library when not given)."""
    if sms is None:
        sms = sm_count()
    blocks = max(1, n_seqs * kv_heads * ((group + 15) // 16))
    # Two blocks of this kernel fit an SM with its three page buffers (100 KB of shared memory at head size 128),
    # three with two buffers, which the launcher picks when that makes all blocks run at once: 2 or 3 per SM.
    # All slices should run in one wave.
    resident = sms * 2
    if blocks >= resident:
        return 1
    if 2 * blocks > resident and 2 * blocks <= sms * 3 and table_stride >= 8:
        return 2          # one slice each would leave half the GPU idle; two fit with two page buffers
    # merging the slices costs a few microseconds that grow with their number: a slice should hold at least
    # four pages of the longest sequence
    most = max(1, table_stride // 4)
    three_buffers = max(1, min(resident // blocks, 64, most))
    # with two page buffers three blocks fit an SM: more, shorter slices in the same single round (measured at
    # batch 8: 18.7 us with 6 slices against 19.5 us with 4 at 2,112 keys; 7 slices, a second round, take 24.2 us)
    two_buffers = max(1, min((sms * 3) // blocks, 64, most))
    # only where that is half as many slices again: batch 8, 6 for 4 slices, 0.982 against 1.010 ms a step; batch 16,
    # 3 for 2, 1.395 against 1.412 ms; batch 12, 4 for 3, is slower, 1.197 against 1.171 ms
    if 2 * two_buffers >= 3 * three_buffers and two_buffers * blocks > resident:
        return two_buffers
    return three_buffers


def _sinks_ok(sinks, heads: int) -> None:
    _need(sinks is None or (sinks.is_cuda and sinks.dtype == torch.float32 and sinks.numel() == heads and sinks.is_contiguous()),
          "attention: sinks are float32, one per head")


def attention_prefill(q, k_pool, v_pool, out, seq_start, past, counts, block_table, max_count: int, heads: int,
                      kv_heads: int, head_dim: int, window: int, scale: float, stream=None, sinks=None, slopes=None,
                      softcap: float = 0.0, out_f32: bool = False) -> None:
    """Tensor-core attention for a step in which sequences bring any number of tokens. ``sinks`` [heads]: a learned
    score per head in the softmax denominator (as in ``attention``). ``slopes`` [heads] float32 / ``softcap``: the score
    rules of ``attention_scored`` (not together with sinks). ``out_f32``: ``out`` is float32."""
    _cuda(q, k_pool, v_pool, out, seq_start, past, counts, block_table, slopes)
    _sinks_ok(sinks, heads)
    _slopes_ok(slopes, heads, sinks)
    T, n = q.shape[0], block_table.shape[0]
    _need(q.shape == (T, heads, head_dim) and out.shape == (T, heads * head_dim), "attention: shapes disagree")
    _need(q.dtype == k_pool.dtype == v_pool.dtype == torch.bfloat16 and out.dtype == (torch.float32 if out_f32 else torch.bfloat16),
          "attention (tensor cores): bfloat16 only")
    _need(tuple(k_pool.shape[1:]) == (kv_heads, 64, head_dim) and k_pool.shape == v_pool.shape, "attention: pool shape")
    _need(seq_start.numel() >= n + 1 and past.numel() >= n and counts.numel() >= n, "attention: per-sequence tables")
    _need(not out_f32 or sinks is None, "attention: a float32 result does not go with sinks")
    if slopes is not None or softcap or out_f32:
        lib().call("slb_attention_prefill_scored", _p(q), _p(k_pool), _p(v_pool), _p(out), _p(seq_start), _p(past), _p(counts),
                   _p(block_table), block_table.shape[1], n, int(max_count), heads, kv_heads, head_dim, int(window),
                   float(scale), _p(slopes), float(softcap), 1 if out_f32 else 0, stream if stream is not None else current_stream())
        return
    lib().call("slb_attention_prefill", _p(q), _p(k_pool), _p(v_pool), _p(out), _p(seq_start), _p(past), _p(counts),
               _p(block_table), block_table.shape[1], n, int(max_count), heads, kv_heads, head_dim, int(window),
               float(scale), _p(sinks), stream if stream is not None else current_stream())


def _slopes_ok(slopes, heads: int, sinks) -> None:
    _need(slopes is None or (slopes.dtype == torch.float32 and slopes.numel() == heads and sinks is None),
          "attention: slopes are float32, one per head, and do not go with sinks")


def attention_tc_supported(heads: int, kv_heads: int, head_dim: int, dtype: torch.dtype) -> bool:
    """Whether the tcgen05 attention kernel takes this shape (bfloat16, head size 64 or 128, group size dividing 128)."""
    if dtype != torch.bfloat16 or heads <= 0 or kv_heads <= 0 or heads % kv_heads:
        return False
    group = heads // kv_heads
    return head_dim in (64, 128) and group <= 128 and 128 % group == 0


def attention_tc_takes_two_pages(n_seqs: int, max_count: int, max_keys: int, heads: int, kv_heads: int, window: int = 0) -> bool:
    """Whether ``attention_tc``, left to choose, takes its kernel for long tiles (two pages a step, one block an SM)
    for a step of ``n_seqs`` sequences whose longest brings ``max_count`` tokens and then has ``max_keys`` keys."""
    fn = lib().dll.slb_attention_tc_wide_pays
    fn.argtypes = [ctypes.c_int] * 6
    fn.restype = ctypes.c_int
    return fn(int(n_seqs), int(max_count), int(max_keys), int(heads), int(kv_heads), int(window)) != 0


def attention_tc(q, k_pool, v_pool, out, seq_start, past, counts, block_table, max_count: int, heads: int,
                 kv_heads: int, head_dim: int, window: int, scale: float, stream=None, wide: bool | None = None,
                 max_keys: int = 0, sinks=None, slopes=None, softcap: float = 0.0) -> None:
    """Attention for a step in which sequences bring many tokens, on the tcgen05 tensor cores (same contract as
    ``attention_prefill``). A bounded wait that gave up inside the kernel shows in ``tc_check``. ``wide``: the
    kernel that walks two pages a step (True), one page a step (False), or the library's choice from the step's
    shape; ``max_keys`` (the most keys a sequence has after this step, 0 = not known) helps that choice. ``slopes`` /
    ``softcap``: the score rules of ``attention_scored`` (not together with sinks)."""
    _cuda(q, k_pool, v_pool, out, seq_start, past, counts, block_table, slopes)
    _sinks_ok(sinks, heads)
    _slopes_ok(slopes, heads, sinks)
    T, n = q.shape[0], block_table.shape[0]
    _need(q.shape == (T, heads, head_dim) and out.shape == (T, heads * head_dim), "attention: shapes disagree")
    _need(q.dtype == out.dtype == k_pool.dtype == v_pool.dtype == torch.bfloat16, "attention (tcgen05): bfloat16 only")
    _need(q.is_contiguous() and k_pool.is_contiguous() and v_pool.is_contiguous() and out.is_contiguous(),
          "attention (tcgen05): contiguous tensors")
    _need(tuple(k_pool.shape[1:]) == (kv_heads, 64, head_dim) and k_pool.shape == v_pool.shape, "attention: pool shape")
    _need(seq_start.numel() >= n + 1 and past.numel() >= n and counts.numel() >= n, "attention: per-sequence tables")
    if slopes is not None or softcap:
        lib().call("slb_attention_tc_scored", _p(q), _p(k_pool), _p(v_pool), _p(out), _p(seq_start), _p(past), _p(counts),
                   _p(block_table), block_table.shape[1], n, int(max_count), T, k_pool.shape[0], heads, kv_heads, head_dim,
                   int(window), float(scale), _p(_tc_status(q.device)), -1 if wide is None else int(bool(wide)),
                   int(max_keys), _p(slopes), float(softcap), stream if stream is not None else current_stream())
        return
    lib().call("slb_attention_tc", _p(q), _p(k_pool), _p(v_pool), _p(out), _p(seq_start), _p(past), _p(counts),
               _p(block_table), block_table.shape[1], n, int(max_count), T, k_pool.shape[0], heads, kv_heads, head_dim,
               int(window), float(scale), _p(_tc_status(q.device)), -1 if wide is None else int(bool(wide)),
               int(max_keys), _p(sinks), stream if stream is not None else current_stream())


def attention_decode(q, k_pool, v_pool, out, seq_start, past, block_table, heads: int, kv_heads: int, head_dim: int,
                     window: int, scale: float, splits: int, scratch, stream=None, qkv=None, qkv_kv_heads: int = 0,
                     bias=None, q_gain=None, k_gain=None, cos=None, sin=None, eps: float = 1e-6, next_read=None,
                     sinks=None, slopes=None, softcap: float = 0.0, out_f32: bool = False) -> None:
    """Tensor-core attention for a step in which every sequence brings one token (split-KV).

    With ``qkv`` (the raw fused projection ``[n, (heads + 2 * qkv_kv_heads) * head_dim]``) the kernel also does what
    ``qkv_post`` does for that token: bias, per-head QK-norm, rotation of the whole head, and, when
    ``qkv_kv_heads == kv_heads``, the write of its key and value into the cache; ``q`` is then not read.
    ``next_read``: a tensor that the kernel after this one reads and no kernel writes (a weight matrix); the blocks
    ask the L2 cache for it once their own pages are on their way. ``slopes`` / ``softcap``: the score rules of
    ``attention_scored``, with post-processed queries only."""
    _cuda(q, k_pool, v_pool, out, seq_start, past, block_table, scratch, qkv, bias, q_gain, k_gain, cos, sin, slopes)
    _sinks_ok(sinks, heads)
    _slopes_ok(slopes, heads, sinks)
    _need(not (slopes is not None or softcap) or qkv is None, "attention (decode): other score rules go with post-processed queries")
    n = block_table.shape[0]
    _need(out.shape == (n, heads * head_dim) and k_pool.dtype == v_pool.dtype == torch.bfloat16
          and out.dtype == (torch.float32 if out_f32 else torch.bfloat16), "attention (tensor cores): shapes disagree or not bfloat16")
    _need(not out_f32 or (sinks is None and qkv is None), "attention: a float32 result goes with post-processed queries and no sinks")
    _need(tuple(k_pool.shape[1:]) == (kv_heads, 64, head_dim) and k_pool.shape == v_pool.shape, "attention: pool shape")
    _need(scratch is None or scratch.dtype == torch.float32, "attention: scratch is float32")
    if qkv is None:
        _need(q is not None and q.shape == (n, heads, head_dim) and q.dtype == torch.bfloat16, "attention: q shape or dtype")
    else:
        _need(qkv.shape == (n, (heads + 2 * qkv_kv_heads) * head_dim) and qkv.dtype == torch.bfloat16, "attention: raw projection shape")
        for v in (bias, q_gain, k_gain, cos, sin):
            _need(v is None or v.dtype == torch.float32, "attention: gains, biases and tables are float32")
        _need(cos is None or (cos.shape[1] == head_dim // 2 and sin.shape == cos.shape), "attention: rotation tables")
    counters = _decode_counters(out.device, n * kv_heads * ((heads // kv_heads + 15) // 16)) if splits > 1 else None
    if slopes is not None or softcap or out_f32:
        lib().call("slb_attention_decode_scored", _p(q), _p(k_pool), _p(v_pool), _p(out), _p(seq_start), _p(past),
                   _p(block_table), block_table.shape[1], n, heads, kv_heads, head_dim, int(window), float(scale),
                   int(splits), _p(scratch), 0 if scratch is None else scratch.numel(), _p(counters),
                   0 if counters is None else counters.numel(), _p(next_read) if _nbytes(next_read) else None, _nbytes(next_read),
                   _p(slopes), float(softcap), 1 if out_f32 else 0, stream if stream is not None else current_stream())
        return
    lib().call("slb_attention_decode", _p(q), _p(k_pool), _p(v_pool), _p(out), _p(seq_start), _p(past),
               _p(block_table), block_table.shape[1], n, heads, kv_heads, head_dim, int(window), float(scale),
               int(splits), _p(scratch), 0 if scratch is None else scratch.numel(), _p(counters),
               0 if counters is None else counters.numel(), _p(qkv), int(qkv_kv_heads), _p(bias), _p(q_gain), _p(k_gain),
               _p(cos), _p(sin), float(eps), _p(next_read) if _nbytes(next_read) else None, _nbytes(next_read),
               _p(sinks), stream if stream is not None else current_stream())


_COUNTERS: dict = {}


def _decode_counters(device, n: int) -> torch.Tensor:
    """Ticket counters of the split-KV decode kernel: zero when a launch starts, left at zero when it ends."""
    key = str(device)
    t = _COUNTERS.get(key)
    if t is None or t.numel() < n:
        if t is not None:
            _RETIRED.append(t)          # a captured graph may still point at the smaller one
        t = torch.zeros(max(n, 4096), dtype=torch.int32, device=device)
        _COUNTERS[key] = t
    return t


_RETIRED: list = []


def decode_scratch_floats(n_seqs: int, heads: int, head_dim: int, splits: int) -> int:
    return 0 if splits <= 1 else n_seqs * heads * splits * (head_dim + 2)


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias=None, accumulate: bool = False,
             stream=None) -> None:
    """out[M, N] (+)= a[M, K] @ w[N, K]^T (+ bias), all float32, plain FMA."""
    _cuda(a, w, out, bias)
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (M, N), "gemm_f32: shapes disagree")
    _need(a.dtype == w.dtype == out.dtype == torch.float32, "gemm_f32: float32 only")
    lib().call("slb_gemm_f32", _p(a), _p(w), _p(bias), _p(out), M, N, K, K, K, N, int(accumulate),
               stream if stream is not None else current_stream())


SKINNY_MODES = {"bf16": 0, "f32": 1, "add": 2, "swiglu": 3}


def skinny_supported(M: int, N: int, K: int, norm: bool = False) -> bool:
    """Whether the few-rows bfloat16 product kernel takes this problem (with the norm fused in: up to 16 rows of
    at most 4,096 values, which it keeps normalised in shared memory)."""
    return 1 <= M <= (16 if norm else 64) and K >= 32 and K % 32 == 0 and N >= 1 and (not norm or K <= 4096)


# SLEUTH_B200_PREFETCH=0: kernels are not told what the kernel after them reads (for comparisons; measured on a
# B200 at batch 8: 1.055 ms a step with the hints, 1.073 ms without; no difference at batch 1).
PREFETCH = os.environ.get("SLEUTH_B200_PREFETCH", "1") != "0"
# No hint for a matrix of more than a quarter of the 126 MB L2: it would push out what it is meant to keep, and a
# product that large is bound by memory bandwidth, not by latency (hidden 4,096, one row: 1.40 ms a step with this
# limit, 1.57 ms without; hidden 2,048: 1.31 against 1.27 ms).
PREFETCH_MOST = 32 << 20


def _nbytes(t) -> int:
    """Bytes of a range handed to a kernel as its ``next_read``: 0 (no hint) unless it is one aligned piece of memory."""
    if t is None or not PREFETCH or not t.is_contiguous() or t.data_ptr() % 16:
        return 0
    n = t.numel() * t.element_size()
    return n if n <= PREFETCH_MOST else 0


class _NextPages(ctypes.Structure):
    _fields_ = [("k_pool", ctypes.c_void_p), ("v_pool", ctypes.c_void_p), ("block_table", ctypes.c_void_p),
                ("past", ctypes.c_void_p), ("page_bytes", ctypes.c_longlong), ("table_stride", ctypes.c_int),
                ("n_seqs", ctypes.c_int), ("splits", ctypes.c_int), ("depth", ctypes.c_int), ("window", ctypes.c_int)]


def next_pages(k_pool, v_pool, block_table, past, splits: int, window: int, depth: int = 2):
    """What a few-rows product hands its kernel as ``next_pages`` when ``attention_decode`` with these arguments
    follows it: the product's blocks then ask the L2 cache for the first ``depth`` pages of every slice."""
    if not PREFETCH:
        return None
    _cuda(k_pool, v_pool, block_table, past)
    page_bytes = k_pool[0].numel() * k_pool.element_size()
    if page_bytes > 32 * 32768 or page_bytes % 16:
        return None
    return _NextPages(k_pool.data_ptr(), v_pool.data_ptr(), block_table.data_ptr(), past.data_ptr(), page_bytes,
                      block_table.shape[1], block_table.shape[0], int(splits), int(depth), int(window))


def _pages_arg(pages):
    return None if pages is None else ctypes.addressof(pages)


def _gate_args(gate) -> tuple | None:
    """(kind number, limit, alpha) of a gated product's activation given as (name, limit, alpha); None = SiLU."""
    if gate is None or gate[0] == "silu":
        return None
    _need(gate[0] in ACTIVATIONS, f"gated product: activation {gate[0]!r} is not one of {sorted(ACTIVATIONS)}")
    return ACTIVATIONS[gate[0]], float(gate[1]), float(gate[2])


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: str, stream=None, next_read=None,
                next_pages=None, features: int = 0, gate=None) -> None:
    """out = x[M, K] @ w^T for M <= 16 (bfloat16 in, float32 accumulation). mode: "bf16" / "f32" store,
    "add" adds into a float32 ``out``, "swiglu" takes w = [gate rows; up rows] and stores silu(gate) * up.
    ``next_read``: a weight tensor that the kernel after this one reads; the blocks ask the L2 cache for it.
    ``features``: output features a block takes (8, 16, 32; 0 = the launcher's rule)."""
    _cuda(x, w, out)
    M, K = x.shape
    N = out.shape[1]
    _need(x.dtype == w.dtype == torch.bfloat16 and w.shape[1] == K and out.shape[0] == M, "gemm_skinny: shapes or dtypes")
    _need(w.shape[0] == (2 * N if mode == "swiglu" else N), "gemm_skinny: weight rows")
    _need(out.dtype == (torch.bfloat16 if mode in ("bf16", "swiglu") else torch.float32), "gemm_skinny: output dtype")
    g = _gate_args(gate) if mode == "swiglu" else None
    if g is not None:       # ``gate`` = (name, limit, alpha): the gated form with another activation than SiLU
        lib().call("slb_gemm_skinny_gated", _p(x), _p(w), _p(out), M, N, K, N, *g, _p(next_read) if _nbytes(next_read) else None,
                   _nbytes(next_read), _pages_arg(next_pages), int(features), stream if stream is not None else current_stream())
        return
    lib().call("slb_gemm_skinny", _p(x), _p(w), _p(out), M, N, K, N, SKINNY_MODES[mode], _p(next_read) if _nbytes(next_read) else None, _nbytes(next_read),
               _pages_arg(next_pages), int(features), stream if stream is not None else current_stream())


def gemm_skinny_norm(x: torch.Tensor, gain: torch.Tensor, eps: float, w: torch.Tensor, out: torch.Tensor, mode: str,
                     stream=None, next_read=None, next_pages=None, features: int = 0) -> None:
    """``gemm_skinny`` on rmsnorm(x; gain, eps): x is the float32 stream [M, K], normalised inside the kernel."""
    _cuda(x, gain, w, out)
    M, K = x.shape
    N = out.shape[1]
    _need(x.dtype == torch.float32 and gain.dtype == torch.float32 and gain.numel() == K, "gemm_skinny_norm: x and gain are float32")
    _need(w.dtype == torch.bfloat16 and w.shape[1] == K and out.shape[0] == M, "gemm_skinny_norm: shapes or dtypes")
    _need(w.shape[0] == (2 * N if mode == "swiglu" else N), "gemm_skinny_norm: weight rows")
    _need(out.dtype == (torch.bfloat16 if mode in ("bf16", "swiglu") else torch.float32), "gemm_skinny_norm: output dtype")
    lib().call("slb_gemm_skinny_norm", _p(x), _p(gain), float(eps), _p(w), _p(out), M, N, K, N, SKINNY_MODES[mode],
               _p(next_read) if _nbytes(next_read) else None, _nbytes(next_read), _pages_arg(next_pages), int(features),
               stream if stream is not None else current_stream())


def tc_supported(M: int, N: int, K: int) -> bool:
    """Whether the tcgen05/TMA product kernel takes this problem."""
    return M >= 1 and N >= 1 and K >= 8 and K % 8 == 0


_TC_STATUS: dict = {}


def _tc_status(device) -> torch.Tensor:
    st = _TC_STATUS.get(device)
    if st is None:
        st = _TC_STATUS.get(str(device))
        if st is None:
            st = torch.zeros(1, dtype=torch.int32, device=device)
            _TC_STATUS[str(device)] = st
        _TC_STATUS[device] = st
    return st


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: str, stream=None, gate=None) -> None:
    """out = x[M, K] @ w^T on the tcgen05 tensor cores (bfloat16 in, float32 accumulation in tensor memory).
    mode as for ``gemm_skinny``: "bf16" / "f32" store, "add" into a float32 ``out``, "swiglu" with w = [gate; up]."""
    _cuda(x, w, out)
    M, K = x.shape
    N = out.shape[1]
    _need(x.dtype == w.dtype == torch.bfloat16 and w.shape[1] == K and out.shape[0] == M, "gemm_tc: shapes or dtypes")
    _need(w.shape[0] == (2 * N if mode == "swiglu" else N), "gemm_tc: weight rows")
    _need(out.dtype == (torch.bfloat16 if mode in ("bf16", "swiglu") else torch.float32), "gemm_tc: output dtype")
    g = _gate_args(gate) if mode == "swiglu" else None
    if g is not None:       # ``gate`` = (name, limit, alpha): the gated form with another activation than SiLU
        lib().call("slb_gemm_tc_gated", _p(x), _p(w), _p(out), M, N, K, N, *g, _p(_tc_status(x.device)),
                   stream if stream is not None else current_stream())
        return
    lib().call("slb_gemm_tc", _p(x), _p(w), _p(out), M, N, K, N, SKINNY_MODES[mode], _p(_tc_status(x.device)),
               stream if stream is not None else current_stream())


def gemm_tc_qkv(x, w, heads: int, kv_heads: int, head_dim: int, bias, q_gain, k_gain, cos, sin, eps: float, q_out,
                k_pool, v_pool, tok_seq, tok_pos, block_table, stream=None) -> None:
    """The fused q/k/v projection of many tokens with everything ``qkv_post`` does in its epilogue, on the float32
    accumulators: bias, per-head RMSNorm of q and k, rotation of the whole head, q into ``q_out [T, H, hd]``, k and v
    into each token's cache page. ``kv_heads == 0``: ``w`` holds only q heads and nothing is written to the cache."""
    _cuda(x, w, bias, q_gain, k_gain, cos, sin, q_out, k_pool, v_pool, tok_seq, tok_pos, block_table)
    M, K = x.shape
    _need(x.dtype == w.dtype == q_out.dtype == torch.bfloat16, "gemm_tc_qkv: bfloat16 only")
    _need(w.shape == ((heads + 2 * kv_heads) * head_dim, K) and w.is_contiguous() and x.is_contiguous(), "gemm_tc_qkv: weight shape")
    _need(q_out.shape == (M, heads, head_dim) and q_out.is_contiguous(), "gemm_tc_qkv: q_out shape")
    for v in (bias, q_gain, k_gain, cos, sin):
        _need(v is None or (v.dtype == torch.float32 and v.is_contiguous()), "gemm_tc_qkv: gains, biases and tables are float32")
    _need(cos is None or (cos.shape[1] == head_dim // 2 and sin.shape == cos.shape), "gemm_tc_qkv: rotation tables [positions, hd / 2]")
    _need(tok_pos.numel() >= M and (kv_heads == 0 or tok_seq.numel() >= M), "gemm_tc_qkv: per-token tables")
    if kv_heads:
        _need(k_pool is not None and tuple(k_pool.shape[1:]) == (kv_heads, 64, head_dim) and k_pool.shape == v_pool.shape
              and k_pool.dtype == v_pool.dtype == torch.bfloat16, "gemm_tc_qkv: pool shape")
    lib().call("slb_gemm_tc_qkv", _p(x), _p(w), M, K, heads, kv_heads, head_dim, _p(bias), _p(q_gain), _p(k_gain), _p(cos),
               _p(sin), float(eps), _p(q_out), _p(k_pool) if kv_heads else None, _p(v_pool) if kv_heads else None,
               _p(tok_seq), _p(tok_pos), _p(block_table), 0 if block_table is None else block_table.shape[1],
               _p(_tc_status(x.device)), stream if stream is not None else current_stream())


def tc_wait_probe(device, polls: int = 1000, code: int = 99, stream=None) -> None:
    """Run the give-up path of the tensor-memory kernels on purpose and harmlessly: a one-block kernel takes tensor
    memory, waits ``polls`` times on a barrier that nothing completes, records ``code`` in the status word, frees its
    tensor memory and returns. ``gemm_tc_check`` then raises. For tests of that path; nothing faults or hangs."""
    with torch.cuda.device(torch.device(device)):
        lib().call("slb_tc_wait_probe", _p(_tc_status(torch.device(device))), int(polls), int(code),
                   stream if stream is not None else current_stream())


def tc_status(device):
    """The status word of the tcgen05 kernels on ``device`` (an int32 CUDA tensor), or None if none has run there."""
    return _TC_STATUS.get(str(torch.device(device)))


def gemm_tc_check(device) -> None:
    """Raise if a tcgen05 product kernel gave up one of its bounded waits since the last check (synchronises)."""
    st = _TC_STATUS.get(str(torch.device(device)))
    if st is None:
        return
    code = int(st.item())
    if code:
        st.zero_()
        raise RuntimeError(f"a wait inside a tcgen05 kernel gave up (code {code}; product: 1 = free stage, 2 = loaded "
                           f"stage, 3 = finished accumulator, 4 = drained accumulator; attention: 20 = shared memory "
                           f"misaligned, 21-27 = producer and MMA waits, 28-32 = softmax waits; persistent single-token kernel: 40 = grid "
                           f"barrier, 41 = a ring slot that did not fill, 42 = a ring slot that did not empty; 99 = the wait "
                           f"probe of the tests); "
                           f"its results are not valid")


# ---------------------------------------------------------------- the persistent single-token kernel ----
_VP, _LL, _CI, _CF = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_float
DL_MAX_PLANS, DL_MAX_ROWS, DL_MAX_UNITS, DL_MAX_GROUP, DL_MAX_COMBOS = 4, 16, 256, 8, 4


class _DlLayer(ctypes.Structure):          # mirrors DlLayer in csrc/decode_layers.cu
    _fields_ = [(n, _VP) for n in ("w_qkv", "w_o", "w_gu", "w_down", "norm1", "norm2", "bias", "q_gain", "k_gain", "cos_table",
                                   "sin_table", "k_pool", "v_pool")] + \
               [("k_row0", _LL), ("v_row0", _LL), ("eps1", _CF), ("eps2", _CF), ("qk_eps", _CF), ("scale_log2", _CF),
                ("heads", _CI), ("kv_heads", _CI), ("inter", _CI), ("window", _CI), ("group", _CI), ("plan", _CI),
                ("combo", _CI), ("pad1", _CI)]


class _DlArgs(ctypes.Structure):           # mirrors DlArgs
    _fields_ = [(n, _VP) for n in ("layers", "x", "qkv", "y", "act", "parts", "tickets", "barrier", "status", "past", "trace")] + \
               [("tables", _VP * 2), ("table_stride", _CI * 2), ("plan_window", _CI * DL_MAX_PLANS),
                ("plan_kv_heads", _CI * DL_MAX_PLANS), ("combo_plan", _CI * DL_MAX_COMBOS), ("combo_group", _CI * DL_MAX_COMBOS),
                ("n_plans", _CI), ("n_combos", _CI), ("n_layers", _CI), ("B", _CI), ("d", _CI), ("n_slots", _CI),
                ("stage_bytes", _CI), ("pad", _CI)]


class _DlHost(ctypes.Structure):           # mirrors DlHost
    _fields_ = [("args", _DlArgs), ("pool_base", _VP * 2), ("pool_rows", _LL * 2), ("head_dim", _CI), ("n_groups", _CI)]


class DecodeProgram:
    """A run of layers prepared for ``decode_layers``: the layers' descriptions in device memory and what is the same
    for every launch. Built by ``decode_program`` from what the layers' parts offer (``Part.fused_decode``)."""

    def __init__(self, layers_dev, n_layers, head_dim, hidden, kmax, max_qkv, max_heads, max_inter, plans, groups, combos, keep):
        self.layers_dev, self.n_layers, self.head_dim, self.hidden, self.kmax = layers_dev, n_layers, head_dim, hidden, kmax
        self.max_qkv, self.max_heads, self.max_inter = max_qkv, max_heads, max_inter
        self.plans, self.groups, self.combos, self.keep = plans, groups, combos, keep
        device = layers_dev.device
        self.tickets = torch.zeros(DL_MAX_UNITS, dtype=torch.int32, device=device)
        self.barrier = torch.zeros(4, dtype=torch.int32, device=device)
        self._slots: dict = {}

    def slots_for(self, rows: int) -> tuple[int, int]:
        """(ring slots, bytes of the staging area) for a step of ``rows`` sequences; fewer than 4 slots: do not fuse."""
        if rows not in self._slots:
            dll = lib().dll
            dll.slb_decode_layers_stage_bytes.restype = ctypes.c_int
            dll.slb_decode_layers_slots.restype = ctypes.c_int
            stage = int(dll.slb_decode_layers_stage_bytes(int(rows), int(self.kmax), int(self.head_dim)))
            self._slots[rows] = (int(dll.slb_decode_layers_slots(stage, int(rows))), stage)
        return self._slots[rows]


def decode_program(shares: list, views: list, pools: list) -> DecodeProgram | None:
    """Prepare a run of layers for the persistent single-token kernel. ``shares``: per layer what its parts offer
    (``PreNormLayer.fused_decode``); ``views``: per layer the ``KVView`` of its cache entry; ``pools``: the cache's
    pool tensor of each group. None when the run does not fit the kernel (mixed head sizes or widths, more than two
    cache groups or four page plans)."""
    if not shares:
        return None
    hd = shares[0]["mixer"]["head_dim"]
    d = shares[0]["mixer"]["hidden"]
    group_ids, plans, combos, keep = [], [], [], []
    arr = (_DlLayer * len(shares))()
    kmax = max_qkv = max_heads = max_inter = 0
    for i, (sh, view) in enumerate(zip(shares, views)):
        m, f = sh["mixer"], sh["ffn"]
        if m["head_dim"] != hd or m["hidden"] != d or view is None or not getattr(view, "writes", False):
            return None
        if view.group not in group_ids:
            group_ids.append(view.group)
        plan = (int(m["window"]), int(m["kv_heads"]))
        if plan not in plans:
            plans.append(plan)
        combo = (plans.index(plan), group_ids.index(view.group))
        if combo not in combos:
            combos.append(combo)
        if len(group_ids) > 2 or len(plans) > DL_MAX_PLANS or len(combos) > DL_MAX_COMBOS:
            return None
        pool = pools[view.group]
        L = arr[i]
        for name, t in (("w_qkv", m["w_qkv"]), ("w_o", m["w_o"]), ("w_gu", f["w_gu"]), ("w_down", f["w_down"]),
                        ("norm1", sh["norm1"]["gain"]), ("norm2", sh["norm2"]["gain"]), ("bias", m["bias"]),
                        ("q_gain", m["q_gain"]), ("k_gain", m["k_gain"]), ("cos_table", m["cos"]), ("sin_table", m["sin"]),
                        ("k_pool", view.k_pool), ("v_pool", view.v_pool)):
            if t is not None:
                _need(t.is_cuda and t.is_contiguous() and t.data_ptr() % 16 == 0, f"decode_program: {name} must be a contiguous, aligned CUDA tensor")
                keep.append(t)
            setattr(L, name, _p(t))
        for t in (m["w_qkv"], m["w_o"], f["w_gu"], f["w_down"], view.k_pool):
            _need(t.dtype == torch.bfloat16, "decode_program: matrices and the cache are bfloat16")
        for t in (sh["norm1"]["gain"], sh["norm2"]["gain"], m["bias"], m["q_gain"], m["k_gain"], m["cos"], m["sin"]):
            _need(t is None or t.dtype == torch.float32, "decode_program: gains, biases and tables are float32")
        row_bytes = hd * 2
        L.k_row0 = (view.k_pool.data_ptr() - pool.data_ptr()) // row_bytes
        L.v_row0 = (view.v_pool.data_ptr() - pool.data_ptr()) // row_bytes
        L.eps1, L.eps2, L.qk_eps = float(sh["norm1"]["eps"]), float(sh["norm2"]["eps"]), float(m["qk_eps"])
        L.scale_log2 = float(m["scale"]) * 1.4426950408889634
        L.heads, L.kv_heads, L.inter, L.window = int(m["heads"]), int(m["kv_heads"]), int(f["inter"]), int(m["window"])
        L.group, L.plan, L.combo = group_ids.index(view.group), plans.index(plan), combos.index(combo)
        n_qkv = (L.heads + 2 * L.kv_heads) * hd
        _need(tuple(m["w_qkv"].shape) == (n_qkv, d) and tuple(m["w_o"].shape) == (d, L.heads * hd) and
              tuple(f["w_gu"].shape) == (2 * L.inter, d) and tuple(f["w_down"].shape) == (d, L.inter),
              "decode_program: weight shapes disagree with the sizes")
        kmax = max(kmax, d, L.heads * hd, L.inter)
        max_qkv, max_heads, max_inter = max(max_qkv, n_qkv), max(max_heads, L.heads * hd), max(max_inter, L.inter)
    device = shares[0]["mixer"]["w_qkv"].device
    raw = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8).to(device)
    groups = [(pools[g], pools[g].numel() // hd) for g in group_ids]
    keep.extend(p for p, _ in groups)
    return DecodeProgram(raw, len(shares), hd, d, kmax, max_qkv, max_heads, max_inter, plans,
                         [(gid, *g) for gid, g in zip(group_ids, groups)], combos, keep)


def decode_layers_scratch_floats(prog: DecodeProgram, rows: int, blocks: int) -> int:
    return (blocks + DL_MAX_UNITS) * (DL_MAX_GROUP * prog.head_dim + 2 * DL_MAX_GROUP)


def decode_layers(prog: DecodeProgram, x: torch.Tensor, past: torch.Tensor, tables: list, qkv, y, act, parts, stream=None,
                  trace: torch.Tensor | None = None) -> None:
    """Run the program's layers on the float32 stream ``x [B, hidden]`` of a step in which each of the B sequences
    brings one token: ``past [B]`` their positions, ``tables`` the step's block table of every cache group
    (indexed as the cache indexes its groups). ``qkv``, ``y``, ``act`` (bfloat16) and ``parts`` (float32) are scratch.
    ``trace``: None, or an int64 tensor [blocks, layers, 24] that receives every block's nanosecond stamps at the phase
    boundaries of every layer (entries 0-14) and the clock cycles each phase waited for its data (15-19): a diagnostic."""
    _cuda(x, past, qkv, y, act, parts)
    B, d = x.shape
    _need(x.dtype == torch.float32 and d == prog.hidden and 1 <= B <= DL_MAX_ROWS, "decode_layers: x is float32 [1..16, hidden]")
    n_slots, stage = prog.slots_for(B)
    _need(n_slots >= 4, "decode_layers: the token rows leave no room for the ring in shared memory")
    blocks = sm_count(x.device)
    _need(qkv.numel() >= B * prog.max_qkv and y.numel() >= B * prog.max_heads and act.numel() >= B * prog.max_inter and
          parts.numel() >= decode_layers_scratch_floats(prog, B, blocks) and qkv.dtype == y.dtype == act.dtype == torch.bfloat16
          and parts.dtype == torch.float32, "decode_layers: scratch buffers are too small or of the wrong dtype")
    h = _DlHost()
    a = h.args
    a.layers, a.x, a.qkv, a.y, a.act, a.parts = prog.layers_dev.data_ptr(), x.data_ptr(), qkv.data_ptr(), y.data_ptr(), act.data_ptr(), parts.data_ptr()
    a.tickets, a.barrier, a.status, a.past = prog.tickets.data_ptr(), prog.barrier.data_ptr(), _tc_status(x.device).data_ptr(), past.data_ptr()
    if trace is not None:
        _need(trace.is_cuda and trace.dtype == torch.int64 and trace.numel() >= blocks * prog.n_layers * 24, "decode_layers: trace is int64 [blocks, layers, 24]")
    a.trace = _p(trace)
    for i, (gid, pool, rows) in enumerate(prog.groups):
        t = tables[gid]
        _need(t.dtype == torch.int32 and t.dim() == 2 and t.shape[0] >= B and t.is_contiguous(), "decode_layers: block tables are int32 [B, stride]")
        a.tables[i], a.table_stride[i] = t.data_ptr(), t.shape[1]
        h.pool_base[i], h.pool_rows[i] = pool.data_ptr(), rows
    for i, (window, kvh) in enumerate(prog.plans):
        a.plan_window[i], a.plan_kv_heads[i] = window, kvh
    for i, (plan, group) in enumerate(prog.combos):
        a.combo_plan[i], a.combo_group[i] = plan, group
    a.n_plans, a.n_combos, a.n_layers, a.B, a.d, a.n_slots, a.stage_bytes = len(prog.plans), len(prog.combos), prog.n_layers, B, d, n_slots, stage
    h.head_dim, h.n_groups = prog.head_dim, len(prog.groups)
    lib().call("slb_decode_layers", ctypes.addressof(h), stream if stream is not None else current_stream())


def penalize(logits, limit: int, recent, n_recent, penalty: float, banned, n_banned, stream=None) -> None:
    _cuda(logits, recent, n_recent, banned, n_banned)
    R = logits.shape[0]
    lib().call("slb_penalize", _p(logits), logits.stride(0), R, limit, _p(recent), _p(n_recent),
               0 if recent is None else recent.shape[1], float(penalty), _p(banned), _p(n_banned),
               0 if banned is None else banned.shape[1], stream if stream is not None else current_stream())


def argmax_scratch_words(rows: int) -> int:
    return 2 * rows * 64


def argmax(logits: torch.Tensor, limit: int, out: torch.Tensor, scratch: torch.Tensor, stream=None) -> None:
    """out[r] = first index of the largest of logits[r, :limit]. ``scratch``: int32, ``argmax_scratch_words(rows)`` long."""
    _need(logits.is_cuda and out.is_cuda and logits.dtype == torch.float32 and out.dtype == torch.int32, "argmax: dtypes")
    _need(logits.stride(1) == 1 and out.numel() >= logits.shape[0] and 0 < limit <= logits.shape[1], "argmax: shapes")
    _need(scratch.is_cuda and scratch.dtype == torch.int32, "argmax: scratch is an int32 CUDA tensor")
    lib().call("slb_argmax", _p(logits), logits.stride(0), logits.shape[0], limit, _p(out), _p(scratch), scratch.numel(),
               stream if stream is not None else current_stream())


def sample(logits: torch.Tensor, limit: int, temperature: float, top_k: int, top_p: float, min_p: float,
           uniform: torch.Tensor, out: torch.Tensor, stream=None) -> None:
    _need(logits.is_cuda and logits.dtype == torch.float32 and uniform.dtype == torch.float32 and
          out.dtype == torch.int32, "sample: dtypes")
    _need(logits.stride(1) == 1 and uniform.numel() >= logits.shape[0] and out.numel() >= logits.shape[0] and
          0 < limit <= logits.shape[1], "sample: shapes")
    lib().call("slb_sample", _p(logits), logits.stride(0), logits.shape[0], limit, float(temperature), int(top_k),
               float(top_p), float(min_p), _p(uniform), _p(out), stream if stream is not None else current_stream())


# ---- attention through low-rank latents (csrc/latent_attention.cu) ----
def latent_post(lat, q_gain, c_gain, cos, sin, cq, pool, tok_seq, tok_pos, block_table, q_rank: int, rank: int,
                rot_dim: int, rotated: int, eps: float, stream=None, c_out=None, k_out=None, dtype=None) -> None:
    """lat [T, q_rank + rank + rot_dim] float32 (the two down-projections' output): the normed query latent goes to
    ``cq`` [T, q_rank]; the normed latent and the rotated key part go to the token's row of ``pool``
    [pages, 64, rank + rot_dim] (``pool`` None: nothing is stored). ``rotated``: how many leading channels of the key
    part turn. ``c_out`` [T, rank] and ``k_out`` [T, rot_dim]: the same latent and key part once more, side by side in
    the order of the step's tokens (for a step that multiplies its own tokens' latents). ``lat`` may have more columns
    than the three parts (they are not read). With ``q_rank`` 0 there is no query latent: ``q_gain`` and ``cq`` are None
    and ``dtype`` names the dtype of what is stored."""
    _cuda(lat, q_gain, c_gain, cos, sin, cq, pool, tok_seq, tok_pos, block_table, c_out, k_out)
    _need((c_out is None) == (k_out is None), "latent_post: the two side-by-side outputs go together")
    T = lat.shape[0]
    dtype = cq.dtype if cq is not None else (dtype or (pool.dtype if pool is not None else c_out.dtype))
    if c_out is not None:
        _need(c_out.shape == (T, rank) and k_out.shape == (T, rot_dim) and c_out.dtype == k_out.dtype == dtype,
              "latent_post: side-by-side outputs")
    _need(lat.dtype == torch.float32 and lat.dim() == 2 and lat.shape[1] >= q_rank + rank + rot_dim, "latent_post: input shape or dtype")
    _need(dtype in DT and (q_rank == 0) == (cq is None), "latent_post: query latent")
    if cq is not None:
        _need(cq.shape == (T, q_rank) and q_gain.dtype == torch.float32 and q_gain.numel() == q_rank, "latent_post: query latent and its gain")
    _need(c_gain.dtype == torch.float32 and c_gain.numel() == rank, "latent_post: gains")
    if rotated:
        _need(cos is not None and cos.dtype == torch.float32 and cos.shape[1] == rotated // 2 and sin.shape == cos.shape,
              "latent_post: rotation tables")
    stride = 0
    if pool is not None:
        _need(pool.dtype == dtype and tuple(pool.shape[1:]) == (64, rank + rot_dim), "latent_post: pool shape or dtype")
        _need(block_table.dtype == torch.int32 and block_table.dim() == 2, "latent_post: block table")
        stride = block_table.shape[1]
    _need(tok_seq.dtype == torch.int32 and tok_pos.dtype == torch.int32, "latent_post: token tables are int32")
    lib().call("slb_latent_post", _p(lat), _p(q_gain), _p(c_gain), _p(cos), _p(sin), _p(cq), _p(pool), _p(tok_seq),
               _p(tok_pos), _p(block_table), stride, T, q_rank, rank, rot_dim, rotated, float(eps), DT[dtype],
               _p(c_out), _p(k_out), lat.shape[1], stream if stream is not None else current_stream())


def latent_attention_supported(rank: int, rot_dim: int) -> bool:
    fn = lib().dll.slb_latent_attention_supported
    fn.argtypes, fn.restype = [ctypes.c_int, ctypes.c_int], ctypes.c_int
    return bool(fn(int(rank), int(rot_dim)))


def latent_attention_general_only(on: bool) -> None:
    """Send bfloat16 steps through the general kernel too (tests compare it with the tensor-core kernel)."""
    lib().dll.slb_latent_attention_general_only(ctypes.c_int(1 if on else 0))


def latent_splits(n_seqs: int, heads: int, max_count: int, max_len: int, sms: int | None = None) -> int:
    """Into how many slices the keys of a step are cut: none while the step's own blocks fill the SMs, else as many
    as it takes to give every SM about two blocks, a slice being at least one page long."""
    sms = sms or sm_count()
    hb = min(heads, 64)
    blocks = n_seqs * -(-max_count // (64 // hb)) * -(-heads // hb)
    if blocks >= sms or max_len <= 128:
        return 1
    return int(max(1, min(2 * sms // max(blocks, 1), max_len // 64, 64)))


def latent_scratch_floats(tokens: int, heads: int, rank: int, splits: int) -> int:
    return 0 if splits <= 1 else splits * tokens * heads * (rank + 2)


def latent_attention(q_lat, q_raw, pool, out, cos, sin, seq_start, past, counts, block_table, max_count: int,
                     heads: int, rank: int, rot_dim: int, plain_dim: int, rotated: int, window: int, scale: float,
                     splits: int = 1, scratch=None, stream=None) -> None:
    """Causal softmax attention of every head over the latent cache rows. q_lat [heads, T, rank]: the queries' plain
    part carried into the latent space; q_raw [T, heads, plain_dim + rot_dim]: the up-projected queries, whose
    rotated part (from ``plain_dim`` on) is turned as it is read; out [heads, T, rank]."""
    _cuda(q_lat, q_raw, pool, out, cos, sin, seq_start, past, counts, block_table, scratch)
    T = q_raw.shape[0]
    _need(q_lat.shape == (heads, T, rank) and out.shape == (heads, T, rank), "latent_attention: latent query or output shape")
    _need(q_raw.shape == (T, heads, plain_dim + rot_dim), "latent_attention: query shape")
    _need(q_lat.dtype == q_raw.dtype == pool.dtype == out.dtype and out.dtype in DT, "latent_attention: dtypes")
    _need(tuple(pool.shape[1:]) == (64, rank + rot_dim), "latent_attention: pool shape")
    _need(block_table.dtype == torch.int32 and block_table.dim() == 2, "latent_attention: block table")
    if rotated:
        _need(cos is not None and cos.dtype == torch.float32 and cos.shape[1] == rotated // 2, "latent_attention: rotation tables")
    if splits > 1:
        _need(scratch is not None and scratch.dtype == torch.float32 and
              scratch.numel() >= latent_scratch_floats(T, heads, rank, splits), "latent_attention: scratch for the slices")
    n = past.numel()
    lib().call("slb_latent_attention", _p(q_lat), _p(q_raw), _p(pool), _p(out), _p(scratch), _p(cos), _p(sin),
               _p(seq_start), _p(past), _p(counts), _p(block_table), block_table.shape[1], n, int(max_count), T, heads,
               rank, rot_dim, plain_dim, rotated, int(window), float(scale), int(splits), DT[out.dtype],
               stream if stream is not None else current_stream())


def head_prompt_supported(plain_dim: int, rot_dim: int, value_dim: int, dtype: torch.dtype) -> bool:
    """Whether whole prompts of these head sizes can run as per-head attention (``head_prompt_attention``)."""
    if dtype != torch.bfloat16:
        return False
    fn = lib().dll.slb_head_prompt_supported
    fn.argtypes, fn.restype = [ctypes.c_int] * 3, ctypes.c_int
    return bool(fn(int(plain_dim), int(rot_dim), int(value_dim)))


def head_prompt_attention(q, kv, k_rot, out, cos, sin, seq_start, counts, max_count: int, heads: int, plain_dim: int,
                          rot_dim: int, value_dim: int, rotated: int, window: int, scale: float, stream=None) -> None:
    """Causal attention of whole prompts (every sequence starts at position 0) with per-head keys and values, bfloat16.
    q [T, heads, plain_dim + rot_dim] (rotated part turned as it is read); kv [T, heads * plain_dim + heads *
    value_dim]: every head's unrotated key values, then every head's values; k_rot [T, rot_dim] turned already;
    out [heads, T, value_dim]."""
    _cuda(q, kv, k_rot, out, cos, sin, seq_start, counts)
    T = q.shape[0]
    _need(q.shape == (T, heads, plain_dim + rot_dim) and kv.shape == (T, heads * (plain_dim + value_dim))
          and k_rot.shape == (T, rot_dim) and out.shape == (heads, T, value_dim), "head_prompt_attention: shapes")
    _need(q.dtype == kv.dtype == k_rot.dtype == out.dtype == torch.bfloat16, "head_prompt_attention: bfloat16 only")
    if rotated:
        _need(cos is not None and cos.dtype == torch.float32 and cos.shape[1] == rotated // 2, "head_prompt_attention: rotation tables")
    lib().call("slb_head_prompt_attention", _p(q), _p(kv), _p(k_rot), _p(out), _p(cos), _p(sin), _p(seq_start), _p(counts),
               counts.numel(), int(max_count), T, heads, plain_dim, rot_dim, value_dim, rotated, int(window), float(scale),
               stream if stream is not None else current_stream())


def latent_gate(val, g, y, stream=None) -> None:
    """y[t, h, :] = val[h, t, :] * sigmoid(g[t, h, :]); val [heads, T, width], g and y [T, heads * width]."""
    _cuda(val, g, y)
    H, T, dv = val.shape
    _need(g.shape == (T, H * dv) and y.shape == g.shape and val.dtype == g.dtype == y.dtype and y.dtype in DT,
          "latent_gate: shapes or dtypes")
    lib().call("slb_latent_gate", _p(val), _p(g), _p(y), T, H, dv, DT[y.dtype], stream if stream is not None else current_stream())


def latent_head_gate(val, g, y, stream=None) -> None:
    """y[t, h, :] = val[h, t, :] * sigmoid(g[t, h]): one gate value per head. val [heads, T, width], y [T, heads * width];
    g float32 [T, heads], possibly a view of a wider matrix (unit column stride)."""
    _cuda(val, y)
    H, T, dv = val.shape
    _need(y.shape == (T, H * dv) and val.dtype == y.dtype and y.dtype in DT, "latent_head_gate: shapes or dtypes")
    _need(g.is_cuda and g.dtype == torch.float32 and g.shape == (T, H) and g.stride(1) == 1, "latent_head_gate: the gates are float32 [tokens, heads]")
    lib().call("slb_latent_head_gate", _p(val), _p(g), g.stride(0) if T > 1 else H, _p(y), T, H, dv, DT[y.dtype],
               stream if stream is not None else current_stream())


# ---- routed experts (csrc/moe.cu) ----
def moe_tile_words(tokens: int, top: int, experts: int) -> int:
    """int32 words of the row-tile table that ``moe_route`` writes for ``moe_experts_tc``."""
    pairs = tokens * top
    return 1 + 3 * (pairs // 128 + min(pairs, experts))


MOE_FEW_PAIRS = 64      # up to this many (token, choice) pairs ``moe_experts`` runs a warp per output (csrc/moe.cu: kMoeFewPairs)


def moe_route(h, w_router, bias, choice, weight, rank, counts, place, order, top: int, stream=None, logits=None,
              tiles=None, layout: bool = True, scoring: str = "softmax_top", groups: int = 1, keep: int = 1,
              scale: float = 1.0, logits_ready: bool = False, pick_bias=None) -> None:
    """Router logits in float32, then the choice. ``scoring="softmax_top"``: the ``top`` largest logits, weights =
    softmax over those. ``scoring="sigmoid"``: scores = sigmoid(logits); the experts form ``groups`` equal groups of
    neighbours, a group scores the sum of its two largest scores, only experts of the ``keep`` best groups can be
    chosen; the ``top`` largest scores, weights = score / (their sum + 1e-20) * ``scale``. ``scoring="softmax"``:
    scores = softmax over all experts' logits; the ``top`` largest of score + ``pick_bias`` (a float32 correction per
    expert, or None) are chosen; weights = the chosen scores * ``scale`` as they are. ``scoring="softmax_norm"``: the
    same scores and choice; weights = score / (the chosen scores' sum + 1e-20) * ``scale``. Then the (token, choice)
    pairs are laid out expert by expert: counts [experts], place [T * top] (a pair's row in that order), order
    [T * top] (the pair at each row). choice, rank int32 [T * top]; weight float32 [T * top]. ``logits``: float32
    scratch [T, experts]; with it, steps of many tokens form their logits 32 tokens at a time (the same sums, k
    ascending). ``logits_ready``: ``logits`` holds the router's logits already (a product formed them; no bias).
    ``layout=False`` leaves counts, place and order unwritten: ``moe_experts`` with ``choice`` does not read
    them for steps of at most ``MOE_FEW_PAIRS`` pairs."""
    _cuda(h, w_router, bias, choice, weight, rank, counts, place, order, logits, tiles, pick_bias)
    T, d = h.shape
    E = w_router.shape[0]
    _need(h.dtype in DT and w_router.dtype == torch.float32 and w_router.shape == (E, d), "moe_route: input or router matrix")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == E), "moe_route: bias")
    _need(pick_bias is None or (pick_bias.dtype == torch.float32 and pick_bias.numel() == E and scoring in ("softmax", "softmax_norm")),
          "moe_route: the choice correction is float32, one per expert, and goes with the softmax scoring")
    _need(scoring in ROUTE_SCORINGS, f"moe_route: scoring {scoring!r} is not one of {sorted(ROUTE_SCORINGS)}")
    for t in (choice, rank, place, order):
        _need(t.dtype == torch.int32 and t.numel() >= T * top, "moe_route: int32 tables of tokens * top entries")
    _need(weight.dtype == torch.float32 and weight.numel() >= T * top and counts.dtype == torch.int32 and counts.numel() >= E,
          "moe_route: weights or counts")
    _need(logits is None or (logits.dtype == torch.float32 and logits.numel() >= T * E), "moe_route: scratch for the logits")
    _need(tiles is None or (tiles.dtype == torch.int32 and tiles.numel() >= moe_tile_words(T, top, E)), "moe_route: row-tile table")
    lib().call("slb_moe_route", _p(h), _p(w_router), _p(bias), _p(pick_bias), _p(choice), _p(weight), _p(rank), _p(counts), _p(place),
               _p(order), _p(logits), _p(tiles), 1 if layout else 0, T, d, E, int(top), ROUTE_SCORINGS[scoring], int(groups),
               int(keep), float(scale), 1 if logits_ready else 0, DT[h.dtype], stream if stream is not None else current_stream())


def moe_experts(h, w_gate_up, w_down, counts, order, weight, act, y, x, top: int, activation: str = "silu",
                stream=None, choice=None, place=None, limit: float = 0.0, alpha: float = 1.0) -> None:
    """x[t] += sum over the token's choices of weight * down_e(f(gate_e h) * (up_e h)). w_gate_up [experts, 2 * ff, d]
    (gate rows, then up rows), w_down [experts, d, ff]; act [T * top, ff] and y [T * top, d] float32 are scratch.
    With ``choice`` and ``place`` (from ``moe_route``) a step of few pairs runs a warp per output instead of tiles."""
    _cuda(h, w_gate_up, w_down, counts, order, weight, act, y, x, choice, place)
    for t in (choice, place):
        _need(t is None or (t.dtype == torch.int32 and t.numel() >= h.shape[0] * top), "moe_experts: choice and place tables")
    T, d = h.shape
    E, ff2, _ = w_gate_up.shape
    ff = ff2 // 2
    _need(w_gate_up.shape == (E, 2 * ff, d) and w_down.shape == (E, d, ff), "moe_experts: expert matrices")
    _need(h.dtype == w_gate_up.dtype == w_down.dtype == act.dtype and h.dtype in DT, "moe_experts: dtypes")
    _need(act.shape == (T * top, ff) and y.shape == (T * top, d) and y.dtype == torch.float32, "moe_experts: scratch")
    _need(x.shape == (T, d) and x.dtype == torch.float32, "moe_experts: the stream")
    _need(activation in ACTIVATIONS, f"moe_experts: activation {activation!r}")
    lib().call("slb_moe_experts", _p(h), _p(w_gate_up), _p(w_down), _p(counts), _p(order), _p(choice), _p(place), _p(weight), _p(act), _p(y),
               _p(x), T, d, ff, E, int(top), ACTIVATIONS[activation], float(limit), float(alpha), DT[h.dtype],
               stream if stream is not None else current_stream())


def moe_experts_tc(h, w_gate_up, w_down, order, place, weight, tiles, xs, act, y, x, top: int, stream=None,
                   activation: str = "silu", limit: float = 0.0, alpha: float = 1.0) -> None:
    """The same sum as ``moe_experts`` for steps of many pairs in bfloat16: the tokens' rows gathered into the
    expert order (``xs`` [T * top, d]) and both products as grouped tcgen05 products over the row tiles that
    ``moe_route`` wrote into ``tiles``; ``y`` [T * top, d] float32 comes out in the expert order."""
    _cuda(h, w_gate_up, w_down, order, place, weight, tiles, xs, act, y, x)
    T, d = h.shape
    E, ff2, _ = w_gate_up.shape
    ff = ff2 // 2
    _need(w_gate_up.shape == (E, 2 * ff, d) and w_down.shape == (E, d, ff), "moe_experts_tc: expert matrices")
    _need(h.dtype == w_gate_up.dtype == w_down.dtype == act.dtype == xs.dtype == torch.bfloat16, "moe_experts_tc: bfloat16 only")
    _need(d % 8 == 0 and ff % 8 == 0, "moe_experts_tc: inner sizes must be multiples of 8")
    _need(xs.shape == (T * top, d) and act.shape == (T * top, ff) and y.shape == (T * top, d) and y.dtype == torch.float32,
          "moe_experts_tc: scratch")
    _need(x.shape == (T, d) and x.dtype == torch.float32, "moe_experts_tc: the stream")
    _need(tiles.dtype == torch.int32 and tiles.numel() >= moe_tile_words(T, top, E), "moe_experts_tc: row-tile table")
    lib().call("slb_moe_experts_tc", _p(h), _p(w_gate_up), _p(w_down), _p(order), _p(place), _p(weight), _p(tiles), _p(xs),
               _p(act), _p(y), _p(x), T, d, ff, E, int(top), ACTIVATIONS[activation], float(limit), float(alpha),
               _p(_tc_status(h.device)), stream if stream is not None else current_stream())


# ---- other score rules, short convolutions, recurrences with a matrix state, several copies of the stream ----

def _st(stream):
    return stream if stream is not None else current_stream()


def _rows_f32(t, width: int, what: str) -> int:
    """``t`` is a float32 matrix (possibly a view of a wider one) whose rows hold at least ``width`` values; its row stride."""
    _need(t.is_cuda and t.dtype == torch.float32 and t.dim() == 2 and t.shape[1] >= width and (t.shape[1] == 0 or t.stride(1) == 1),
          f"{what}: float32 rows of at least {width} values (possibly a view of a wider matrix)")
    return t.stride(0) if t.shape[0] > 1 else max(t.shape[1], width)


def attention_scored(q, k_pool, v_pool, out, tok_seq, tok_pos, block_table, heads: int, kv_heads: int, head_dim: int,
                     window: int, scale: float, stream=None, slopes=None, softcap: float = 0.0, maps: int = 1, gate=None,
                     value_dim: int = 0) -> None:
    """The general attention kernel with other score rules. ``slopes`` [heads] float32: the score loses
    slopes[h] * (query position - key position). ``softcap`` c > 0: score <- c tanh(score / c) before that. ``maps`` m > 1:
    every head has m score maps over the same values; q is [T, heads * m, head_dim], a key row of the cache is m * head_dim
    wide, and ``out`` is float32 [T, heads * m, value_dim]. ``gate``: float32 [T, >= heads * value_dim] pre-activations;
    the result is multiplied by their sigmoid (one map only)."""
    _cuda(q, k_pool, v_pool, out, tok_seq, tok_pos, block_table, slopes)
    T = q.shape[0]
    vd = value_dim or head_dim
    _need(q.shape == (T, heads * maps, head_dim) and out.numel() == T * heads * maps * vd, "attention_scored: shapes disagree")
    _need(q.dtype == k_pool.dtype == v_pool.dtype and q.dtype in DT, "attention_scored: dtypes")
    _need(out.dtype == (torch.float32 if maps > 1 else q.dtype), "attention_scored: several maps give a float32 result")
    _need(tuple(k_pool.shape[1:]) == (kv_heads, 64, maps * head_dim) and tuple(v_pool.shape[1:]) == (kv_heads, 64, vd)
          and k_pool.shape[0] == v_pool.shape[0], "attention_scored: pool shape")
    _need(block_table.dtype == torch.int32 and block_table.dim() == 2, "attention_scored: block table")
    _need(slopes is None or (slopes.dtype == torch.float32 and slopes.numel() == heads), "attention_scored: slopes are float32, one per head")
    gs = 0
    if gate is not None:
        _need(maps == 1, "attention_scored: the gate goes with one map")
        gs = _rows_f32(gate, heads * vd, "attention_scored gate")
    lib().call("slb_attention_scored", _p(q), _p(k_pool), _p(v_pool), _p(out), _p(tok_seq), _p(tok_pos), _p(block_table),
               block_table.shape[1], T, heads, kv_heads, head_dim, int(window), float(scale), _p(slopes), float(softcap),
               int(maps), 1 if maps > 1 else 0, _p(gate), gs, vd, DT[q.dtype], _st(stream))


def causal_conv(u, weight, bias, state, slots, tok_seq, seq_start, out, act: bool = False, stream=None, max_count: int = 0) -> None:
    """out[t, c] = sum_j weight[c, j] * u_(t - taps + 1 + j)[c] (+ bias[c]; silu with ``act``) over each sequence's tokens
    of the step; inputs in front of the step come from ``state`` [slots, taps - 1, C] (the sequence's last inputs, zeros
    at its start), which is then brought up to date. ``u`` and ``out`` are float32 rows, possibly views of wider ones.
    ``max_count``: the step's longest portion when known; steps of up to four tokens a sequence run as one launch."""
    _cuda(weight, bias, state, slots, tok_seq, seq_start)
    C, taps = weight.shape
    T = u.shape[0]
    us, os_ = _rows_f32(u, C, "causal_conv input"), _rows_f32(out, C, "causal_conv output")
    _need(weight.dtype == torch.float32 and (bias is None or (bias.dtype == torch.float32 and bias.numel() == C)), "causal_conv: taps and bias are float32")
    _need(state.dtype == torch.float32 and tuple(state.shape[1:]) == (max(taps - 1, 0), C) or taps == 1, "causal_conv: state [slots, taps - 1, channels]")
    _need(out.shape[0] == T and slots.dtype == torch.int32 and tok_seq.dtype == torch.int32 and seq_start.dtype == torch.int32, "causal_conv: tables")
    lib().call("slb_causal_conv", _p(u), us, _p(weight), _p(bias), _p(state), _p(slots), _p(tok_seq), _p(seq_start), _p(out), os_,
               T, slots.numel(), C, taps, 1 if act else 0, int(max_count), _st(stream))


def decay_scan_scratch_floats(n_seqs: int, max_count: int, heads: int, N: int, P: int, per_channel: bool) -> int:
    """Scratch floats ``decay_scan`` needs for a step whose longest portion has ``max_count`` tokens (0: one pass)."""
    fn = lib().dll.slb_decay_scan_scratch_floats
    fn.argtypes, fn.restype = [ctypes.c_int] * 6, ctypes.c_longlong
    return int(fn(int(n_seqs), int(max_count), int(heads), int(N), int(P), 1 if per_channel else 0))


def decay_scan(q, k, v, a, state, slots, seq_start, out, heads: int, groups: int, per_channel: bool, v_scale=None,
               q_scale: float = 1.0, stream=None, max_count: int = 1, scratch=None) -> None:
    """Per head S_t = diag(a_t) S_(t-1) + k_t v_t^T and out_t = S_t^T q_t * ``q_scale`` over each sequence's tokens of the
    step, from and back into ``state`` float32 [slots, heads, N, P]. q, k: float32 rows of groups * N values (head h reads
    group h // (heads / groups)); v: rows of heads * P values, times ``v_scale`` [T, heads] when given; a: rows of
    heads * N decays (``per_channel``) or of one decay a head. out: float32 [T, heads * P]. ``max_count``: the longest
    portion of the step; long portions run in chunks (each from a zero state, then the chunks' start states in order, then
    each from its start state) and need ``scratch`` (``decay_scan_scratch_floats``)."""
    _cuda(state, slots, seq_start, out, scratch)
    _, H, N, P = state.shape
    T = out.shape[0]
    _need(H == heads and heads % groups == 0 and state.dtype == torch.float32 and out.dtype == torch.float32
          and out.shape == (T, heads * P), "decay_scan: state or output")
    qs, ks = _rows_f32(q, groups * N, "decay_scan q"), _rows_f32(k, groups * N, "decay_scan k")
    vs_ = _rows_f32(v, heads * P, "decay_scan v")
    as_ = _rows_f32(a, heads * N if per_channel else heads, "decay_scan a")
    ss = _rows_f32(v_scale, heads, "decay_scan v_scale") if v_scale is not None else 0
    _need(slots.dtype == torch.int32 and seq_start.dtype == torch.int32 and seq_start.numel() >= slots.numel() + 1, "decay_scan: tables")
    _need(scratch is None or scratch.dtype == torch.float32, "decay_scan: scratch is float32")
    lib().call("slb_decay_scan", _p(q), qs, _p(k), ks, _p(v), vs_, _p(a), as_, 1 if per_channel else 0, _p(v_scale), ss, _p(state),
               _p(slots), _p(seq_start), _p(out), slots.numel(), heads, groups, N, P, float(q_scale), int(max_count), _p(scratch),
               0 if scratch is None else scratch.numel(), _st(stream))


def step_decay(raw, dt_bias, a_log, dt, decay, stream=None) -> None:
    """dt = softplus(raw + dt_bias), decay = exp(-exp(a_log) * dt), per (token, head); raw: float32 rows of ``heads`` values."""
    _cuda(dt_bias, a_log, dt, decay)
    T, H = dt.shape
    rs = _rows_f32(raw, H, "step_decay")
    _need(dt.dtype == decay.dtype == dt_bias.dtype == a_log.dtype == torch.float32 and decay.shape == dt.shape and dt_bias.numel() == H
          and a_log.numel() == H and raw.shape[0] == T, "step_decay: float32 [tokens, heads]")
    lib().call("slb_step_decay", _p(raw), rs, _p(dt_bias), _p(a_log), _p(dt), _p(decay), T, H, _st(stream))


def channel_decay(z, bias, tau: float, stream=None) -> None:
    """z <- sigmoid(z + bias)^(1 / tau) in place; z float32 [T, C] contiguous."""
    _cuda(z, bias)
    T, C = z.shape
    _need(z.dtype == torch.float32 and (bias is None or (bias.dtype == torch.float32 and bias.numel() == C)), "channel_decay: float32")
    lib().call("slb_channel_decay", _p(z), _p(bias), T, C, float(tau), _st(stream))


def gated_group_norm(y, gate, gain, out, groups: int, eps: float, gate_first: bool, skip=None, skip_gain=None,
                     head_width: int = 1, stream=None) -> None:
    """Rows of ``y`` float32 [T, inner] in ``groups`` equal parts, each divided by its root mean square, times
    gain[c % len(gain)]; silu(gate) multiplies the row before the norm (``gate_first``) or after it. With ``skip``:
    skip_gain[c // head_width] * skip[t, c] is added to y first. ``out`` [T, inner] in the run dtype."""
    _cuda(y, gain, out, skip_gain)
    T, inner = y.shape
    gs = _rows_f32(gate, inner, "gated_group_norm gate")
    ks = _rows_f32(skip, inner, "gated_group_norm skip") if skip is not None else 0
    _need(y.dtype == torch.float32 and gain.dtype == torch.float32 and out.shape == (T, inner) and out.dtype in DT and inner % groups == 0,
          "gated_group_norm: shapes or dtypes")
    _need(skip is None or (skip_gain is not None and skip_gain.dtype == torch.float32 and skip_gain.numel() * head_width == inner),
          "gated_group_norm: the skip term's gains")
    lib().call("slb_gated_group_norm", _p(y), _p(skip), ks, _p(skip_gain), int(head_width), _p(gate), gs, _p(gain), gain.numel(),
               _p(out), T, inner, int(groups), 1 if gate_first else 0, float(eps), DT[out.dtype], _st(stream))


def unit_post(rows, q_gain, k_gain, cos, sin, q_out, k_pool, v_pool, tok_seq, tok_pos, block_table, heads: int, kv_heads: int,
              maps: int, dim: int, vdim: int, rot: int, eps: float, stream=None, pad: int = 0) -> None:
    """float32 rows [q units | k units | v units] -> q_out [T, heads * maps, dim] and the token's cache rows (keys
    [pages, kv_heads, 64, maps * dim], values [pages, kv_heads, 64, vdim]); without pools the rows hold q units only.
    q and k units: RMS norm with the gain when one is given, then the first ``rot`` channels turn in pairs (i, i + rot/2).
    ``pad`` W: q rows, key rows and value rows are all W wide; map m's channels sit at m * dim of a q row whose other
    channels are set to zero, and the cache's spare channels are left alone (they are zero from the start), so that a
    kernel that takes q . k over W channels forms the map's own score."""
    _cuda(q_gain, k_gain, cos, sin, q_out, k_pool, v_pool, tok_seq, tok_pos, block_table)
    T = q_out.shape[0]
    writes = k_pool is not None
    width = heads * maps * dim + (kv_heads * maps * dim + kv_heads * vdim if writes else 0)
    rs = _rows_f32(rows, width, "unit_post")
    qw, kw, vw = (pad, pad, pad) if pad else (dim, maps * dim, vdim)
    _need(q_out.shape == (T, heads * maps, qw) and q_out.dtype in DT and rows.shape[0] == T, "unit_post: the query buffer")
    for g in (q_gain, k_gain):
        _need(g is None or (g.dtype == torch.float32 and g.numel() == dim), "unit_post: gains are float32 [dim]")
    if rot:
        _need(cos is not None and cos.dtype == torch.float32 and cos.shape[1] == rot // 2 and sin.shape == cos.shape, "unit_post: rotation tables")
    stride = 0
    if writes:
        _need(k_pool.dtype == v_pool.dtype == q_out.dtype and tuple(k_pool.shape[1:]) == (kv_heads, 64, kw)
              and tuple(v_pool.shape[1:]) == (kv_heads, 64, vw), "unit_post: cache pools")
        _need(block_table.dtype == torch.int32 and block_table.dim() == 2, "unit_post: block table")
        stride = block_table.shape[1]
    lib().call("slb_unit_post", _p(rows), rs, _p(q_gain), _p(k_gain), _p(cos), _p(sin), _p(q_out), _p(k_pool), _p(v_pool),
               _p(tok_seq), _p(tok_pos), _p(block_table) if writes else None, stride, T, heads, kv_heads, maps, dim, vdim, int(rot),
               1 if writes else 0, float(eps), int(pad), DT[q_out.dtype], _st(stream))


def diff_combine(a, gate, out, heads: int, vdim: int, lam: float, post: float, eps: float, stream=None, row: int = 0) -> None:
    """out[t, h] = (a[t, h, 0] - lam * a[t, h, 1]) / rms * post * sigmoid(gate[t, h]); a float32 [T, heads * 2, row] of which
    the first vdim values of a row count (``row`` 0 = vdim)."""
    _cuda(a, out)
    T = out.shape[0]
    _need(a.dtype == torch.float32 and a.numel() == T * heads * 2 * (row or vdim) and out.shape == (T, heads * vdim) and out.dtype in DT, "diff_combine: shapes")
    gs = _rows_f32(gate, heads, "diff_combine gate") if gate is not None else 0
    lib().call("slb_diff_combine", _p(a), _p(gate), gs, _p(out), T, heads, vdim, float(lam), float(post), float(eps), int(row), DT[out.dtype], _st(stream))


def streams_fill(x0, xs, streams: int, stream=None) -> None:
    """xs [T, streams * d] <- every copy the row of x0 [T, d] (float32)."""
    _cuda(x0, xs)
    T, d = x0.shape
    _need(x0.dtype == xs.dtype == torch.float32 and xs.shape == (T, streams * d), "streams_fill: shapes")
    lib().call("slb_streams_fill", _p(x0), _p(xs), T, d, int(streams), _st(stream))


def hyper_read(xs, coef, gain, out, eps: float, stream=None) -> None:
    """out[t] = RMS norm of sum_s coef[s] xs[t, s] (ones without ``coef``), times gain, in the run dtype."""
    _cuda(xs, coef, gain, out)
    T, d = out.shape
    S = xs.shape[1] // d
    _need(xs.dtype == torch.float32 and xs.shape == (T, S * d) and gain.dtype == torch.float32 and gain.numel() == d and out.dtype in DT, "hyper_read: shapes")
    _need(coef is None or (coef.dtype == torch.float32 and coef.numel() == S), "hyper_read: one coefficient a copy")
    lib().call("slb_hyper_read", _p(xs), _p(coef), _p(gain), _p(out), T, d, S, float(eps), DT[out.dtype], _st(stream))


def hyper_write(xs, y, mix, out_coef, mult: float, stream=None) -> None:
    """xs[t, r] <- sum_s mix[s, r] xs[t, s] + mult * out_coef[r] * y[t], all copies from the old ones (identity and ones
    without ``mix`` / ``out_coef``)."""
    _cuda(xs, y, mix, out_coef)
    T, d = y.shape
    S = xs.shape[1] // d
    _need(xs.dtype == y.dtype == torch.float32 and xs.shape == (T, S * d), "hyper_write: shapes")
    _need(mix is None or (mix.dtype == torch.float32 and mix.shape == (S, S)), "hyper_write: the mixing matrix")
    _need(out_coef is None or (out_coef.dtype == torch.float32 and out_coef.numel() == S), "hyper_write: one coefficient a copy")
    lib().call("slb_hyper_write", _p(xs), _p(y), _p(mix), _p(out_coef), T, d, S, float(mult), _st(stream))


def streams_sum(xs, x, stream=None) -> None:
    _cuda(xs, x)
    T, d = x.shape
    S = xs.shape[1] // d
    _need(xs.dtype == x.dtype == torch.float32 and xs.shape == (T, S * d), "streams_sum: shapes")
    lib().call("slb_streams_sum", _p(xs), _p(x), T, d, S, _st(stream))


def pair_combine(a, b, target, gain_a=None, gain_b=None, scale_a: float = 1.0, scale_b: float = 1.0, eps: float = 0.0,
                 accumulate: bool = True, stream=None) -> None:
    """target (+)= scale_a * a + scale_b * b; with gains each row is first divided by its own root mean square and
    multiplied by its gain. All float32 [T, d]."""
    _cuda(a, b, target, gain_a, gain_b)
    T, d = a.shape
    _need(a.dtype == b.dtype == target.dtype == torch.float32 and b.shape == a.shape == target.shape, "pair_combine: shapes")
    for g in (gain_a, gain_b):
        _need(g is None or (g.dtype == torch.float32 and g.numel() == d), "pair_combine: gains")
    lib().call("slb_pair_combine", _p(a), _p(b), _p(gain_a), _p(gain_b), float(scale_a), float(scale_b), float(eps), _p(target), T, d,
               1 if accumulate else 0, _st(stream))


def row_gate(h, w, y, target, accumulate: bool = True, stream=None) -> None:
    """target[t] (+)= sigmoid(h[t] . w) * y[t]; h [T, k] in the run dtype, w float32 [k], y and target float32 [T, d]."""
    _cuda(h, w, y, target)
    T, k = h.shape
    d = y.shape[1]
    _need(h.dtype in DT and w.dtype == torch.float32 and w.numel() == k and y.dtype == target.dtype == torch.float32
          and y.shape == target.shape == (T, d), "row_gate: shapes")
    lib().call("slb_row_gate", _p(h), _p(w), _p(y), _p(target), T, k, d, 1 if accumulate else 0, DT[h.dtype], _st(stream))


def sigmoid_gate(y, gate, stream=None) -> None:
    """y[t, c] <- y[t, c] * sigmoid(gate[t, c]) in place; y [T, C] in the run dtype, gate float32 rows of at least C values."""
    _cuda(y)
    T, C = y.shape
    gs = _rows_f32(gate, C, "sigmoid_gate")
    _need(y.dtype in DT and gate.shape[0] == T, "sigmoid_gate: shapes")
    lib().call("slb_sigmoid_gate", _p(y), _p(gate), gs, T, C, DT[y.dtype], _st(stream))
