"""Causal grouped-query attention with other score rules, as a mixer part (``ScoredAttentionSpec``).

One stacked projection [q | k | v | gate] with a float32 result; then, as the spec asks: a short causal convolution over
time on the q, k and v channels (``ops.causal_conv``; a sequence's last taps - 1 projected values are state); per-unit RMS
norm, rotation and the cache write (``ops.unit_post``); attention over the paged cache by the general kernel with a soft
cap, a distance penalty per head, a window, and one or two score maps a head (``ops.attention_scored``); for two maps the
difference a1 - lambda a2 with its norm and the head gates (``ops.diff_combine``); the output projection into the stream. In bfloat16, one map with keys and values of 64 or 128 channels runs on the
tensor-core kernels instead (tcgen05 for steps that fill its 128-row tiles, mma.sync otherwise and for single tokens), and
two maps whose rows fit 128 channels run on the mma.sync kernels over rows widened with zero channels.

The entry keeps keys and values in pages (a key row is ``maps * head_dim`` wide, so both maps' keys of a position lie
together) and, with a convolution, the tails of the projected rows per sequence. A part that ``reads_shared_kv`` has no key
and value tensors: it reads the entry its schedule entry borrows and keeps only its own query tails.
"""

from __future__ import annotations

import math

import torch

from ..cache.paged import BundleRequest, KVRequest, StateRequest
from ..kernels import ops
from .attention import use_tc_attention
from .base import BuildContext, Normed, ParamDecl, Part, build_position, register_mixer, result_target
from .linear import Linear
from .spec import ScoredAttentionSpec


class ScoredAttention(Part):
    stores_result = True

    def __init__(self, spec: ScoredAttentionSpec, ctx: BuildContext):
        s = spec
        if s.heads % s.kv_heads:
            raise ValueError(f"heads ({s.heads}) must be a multiple of kv_heads ({s.kv_heads})")
        if s.head_dim % 2 or s.head_dim > 256 or s.value_dim > 256 or s.value_dim < 1:
            raise ValueError(f"scored attention: head_dim {s.head_dim} (even, at most 256), value_dim {s.value_dim} (at most 256)")
        if s.maps not in (1, 2):
            raise ValueError(f"scored attention: one score map a head or two (differential), not {s.maps}")
        if s.gate not in ("none", "channel", "head"):
            raise ValueError(f"scored attention: gate {s.gate!r} is not 'none', 'channel' or 'head'")
        if s.gate == "channel" and s.maps != 1 or s.gate == "head" and s.maps != 2:
            raise ValueError("scored attention: a gate per channel goes with one map, a gate per head with two")
        if not 0 <= s.conv_taps <= 16:
            raise ValueError(f"scored attention: conv_taps {s.conv_taps} (at most 16)")
        self.spec, self.ctx = spec, ctx
        self.position = build_position(s.position, ctx)
        self.scale = s.scale or 1.0 / math.sqrt(s.head_dim)
        self.nq = s.heads * s.maps * s.head_dim
        self.nk = 0 if s.reads_shared_kv else s.kv_heads * s.maps * s.head_dim
        self.nv = 0 if s.reads_shared_kv else s.kv_heads * s.value_dim
        self.ng = {"none": 0, "channel": s.heads * s.value_dim, "head": s.heads}[s.gate]
        self.slopes = None
        if s.slope_exponent > 0:
            self.slopes = torch.tensor([2.0 ** (-s.slope_exponent * (h + 1) / s.heads) for h in range(s.heads)],
                                       dtype=torch.float32, device=ctx.device)
        self.slopes_maps = self.slopes.repeat_interleave(s.maps).contiguous() if self.slopes is not None else None   # one a (head, map)
        self.qkvg = self.o = self.conv = self.q_gain = self.k_gain = None
        self.lam = 0.0
        # one map, bfloat16, keys and values of one width that the tensor-core kernels take: prompts and single tokens run
        # on the mma.sync kernels (which know the soft cap and the distance penalty); everything else on the general kernel
        self.flash = s.maps == 1 and s.value_dim == s.head_dim and ops.flash_supported(s.head_dim, ctx.dtype)
        # two maps in bfloat16 whose key row (both maps) and value row fit 128 channels: rows of 64 or 128 channels with zero
        # channels at the end. A query of map m is zero outside the map's own channels, so the same tensor-core kernels form
        # q_m . k_m as a product over the whole row, with 2 * heads query heads; their results come out in float32.
        self.pad = 0
        if s.maps == 2 and ctx.dtype == torch.bfloat16 and max(2 * s.head_dim, s.value_dim) <= 128 and (2 * s.heads) % s.kv_heads == 0:
            self.pad = 64 if max(2 * s.head_dim, s.value_dim) <= 64 else 128

    def _proj(self):
        return ["q"] if self.spec.reads_shared_kv else ["q", "k", "v"]

    def declare(self):
        s = self.spec
        d = {"q.weight": ParamDecl((self.nq, s.hidden)), "o.weight": ParamDecl((s.hidden, s.heads * s.value_dim))}
        if not s.reads_shared_kv:
            d["k.weight"] = ParamDecl((self.nk, s.hidden))
            d["v.weight"] = ParamDecl((self.nv, s.hidden))
        if s.conv_taps:
            for n, rows in (("q", self.nq), ("k", self.nk), ("v", self.nv)):
                if rows:
                    d[f"{n}.conv"] = ParamDecl((rows, s.conv_taps), "vector")
        if s.qk_norm:
            d["q_norm.weight"] = ParamDecl((s.head_dim,), "vector", init="gain")
            if not s.reads_shared_kv:
                d["k_norm.weight"] = ParamDecl((s.head_dim,), "vector", init="gain")
        if s.gate != "none":
            d["g.weight"] = ParamDecl((self.ng, s.hidden))
        if s.maps == 2:
            for n in ("lq1", "lk1", "lq2", "lk2"):
                d[n] = ParamDecl((s.head_dim,), "vector")
        return d

    def bind(self, t):
        s, dt = self.spec, self.ctx.dtype
        stack = [t[n + ".weight"] for n in self._proj()] + ([t["g.weight"]] if self.ng else [])
        self.qkvg = Linear(torch.cat(stack, dim=0), dt)
        self.o = Linear(t["o.weight"], dt)
        if s.conv_taps:
            self.conv = torch.cat([t[n + ".conv"] for n in self._proj()], dim=0).to(torch.float32).contiguous()
        if s.qk_norm:
            self.q_gain = t["q_norm.weight"].to(torch.float32).contiguous()
            self.k_gain = None if s.reads_shared_kv else t["k_norm.weight"].to(torch.float32).contiguous()
        if s.maps == 2:
            f = {n: t[n].to(torch.float32) for n in ("lq1", "lk1", "lq2", "lk2")}
            self.lam = float(torch.exp((f["lq1"] * f["lk1"]).sum()) - torch.exp((f["lq2"] * f["lk2"]).sum())) + s.diff

    def cache_request(self):
        s = self.spec
        parts = []
        if not s.reads_shared_kv:
            parts.append(("kv", KVRequest(s.kv_heads, self.pad, s.window) if self.pad else
                          KVRequest(s.kv_heads, s.maps * s.head_dim, s.window, s.value_dim)))
        if s.conv_taps > 1:
            parts.append(("tail", StateRequest((s.conv_taps - 1, self.nq + self.nk + self.nv), torch.float32)))
        return BundleRequest(tuple(parts)) if parts else None

    def lead_weight(self):
        return self.qkvg.weight if self.qkvg is not None else None

    def forward(self, h, x, b, view, ws):
        s, dt = self.spec, self.ctx.dtype
        if isinstance(h, Normed):
            h = h.tensor()
        T = h.shape[0]
        mark = ws.mark()
        kv = view["borrowed"]["kv"] if s.reads_shared_kv else view["kv"]
        writes = kv.writes and not s.reads_shared_kv
        table = b.tables[kv.group]
        p = self.qkvg.forward(h, ws=ws, stream=b.stream, out_dtype=torch.float32)
        nqkv = self.nq + self.nk + self.nv
        rows = p
        if self.conv is not None:
            rows = ws.take((T, nqkv), torch.float32)
            ops.causal_conv(p, self.conv, None, view["tail"].state, b.slots, b.tok_seq, b.seq_start, rows, False, b.stream, max_count=b.max_count)
        tables = self.position.tables()
        cos, sin = tables if tables is not None else (None, None)
        q = ws.take((T, s.heads * s.maps, self.pad or s.head_dim), dt)
        ops.unit_post(rows, self.q_gain, self.k_gain, cos, sin, q, kv.k_pool if writes else None, kv.v_pool if writes else None,
                      b.tok_seq, b.tok_pos, table, s.heads, s.kv_heads, s.maps, s.head_dim, s.value_dim,
                      self.position.rot_dim, s.eps, b.stream, pad=self.pad)
        gate = p[:, nqkv:] if self.ng else None
        y = ws.take((T, s.heads * s.value_dim), dt)
        if self.flash:
            if b.max_count == 1:
                splits = ops.decode_splits(b.n, s.kv_heads, s.heads // s.kv_heads, table.shape[1])
                floats = ops.decode_scratch_floats(b.n, s.heads, s.head_dim, splits)
                scratch = ws.take((floats,), torch.float32) if floats else None
                ops.attention_decode(q, kv.k_pool, kv.v_pool, y, b.seq_start, b.past, table, s.heads, s.kv_heads, s.head_dim,
                                     kv.window, self.scale, splits, scratch, b.stream, next_read=self.o.weight, slopes=self.slopes,
                                     softcap=s.softcap)
            elif use_tc_attention(s.heads, s.kv_heads, s.head_dim, dt, b.max_count, self.scale):
                ops.attention_tc(q, kv.k_pool, kv.v_pool, y, b.seq_start, b.past, b.counts, table, b.max_count, s.heads,
                                 s.kv_heads, s.head_dim, kv.window, self.scale, b.stream, max_keys=b.max_len, slopes=self.slopes,
                                 softcap=s.softcap)
            else:
                ops.attention_prefill(q, kv.k_pool, kv.v_pool, y, b.seq_start, b.past, b.counts, table, b.max_count, s.heads,
                                      s.kv_heads, s.head_dim, kv.window, self.scale, b.stream, slopes=self.slopes, softcap=s.softcap)
            if gate is not None:
                ops.sigmoid_gate(y, gate, b.stream)
        elif s.maps == 1:
            ops.attention_scored(q, kv.k_pool, kv.v_pool, y, b.tok_seq, b.tok_pos, table, s.heads, s.kv_heads, s.head_dim,
                                 kv.window, self.scale, b.stream, slopes=self.slopes, softcap=s.softcap, gate=gate,
                                 value_dim=s.value_dim)
        elif self.pad:
            W = self.pad
            a = ws.take((T, s.heads * 2 * W), torch.float32)
            if b.max_count == 1:
                splits = ops.decode_splits(b.n, s.kv_heads, 2 * s.heads // s.kv_heads, table.shape[1])
                floats = ops.decode_scratch_floats(b.n, 2 * s.heads, W, splits)
                scratch = ws.take((floats,), torch.float32) if floats else None
                ops.attention_decode(q, kv.k_pool, kv.v_pool, a, b.seq_start, b.past, table, 2 * s.heads, s.kv_heads, W, kv.window,
                                     self.scale, splits, scratch, b.stream, next_read=self.o.weight, slopes=self.slopes_maps,
                                     softcap=s.softcap, out_f32=True)
            else:
                ops.attention_prefill(q, kv.k_pool, kv.v_pool, a, b.seq_start, b.past, b.counts, table, b.max_count, 2 * s.heads,
                                      s.kv_heads, W, kv.window, self.scale, b.stream, slopes=self.slopes_maps, softcap=s.softcap,
                                      out_f32=True)
            ops.diff_combine(a, gate, y, s.heads, s.value_dim, self.lam, 1.0 - s.diff, s.eps, b.stream, row=W)
        else:
            a = ws.take((T, s.heads * 2, s.value_dim), torch.float32)
            ops.attention_scored(q, kv.k_pool, kv.v_pool, a, b.tok_seq, b.tok_pos, table, s.heads, s.kv_heads, s.head_dim,
                                 kv.window, self.scale, b.stream, slopes=self.slopes, softcap=s.softcap, maps=2,
                                 value_dim=s.value_dim)
            ops.diff_combine(a, gate, y, s.heads, s.value_dim, self.lam, 1.0 - s.diff, s.eps, b.stream)
        self.o.forward(y, ws=ws, stream=b.stream, next_read=getattr(b, "next_read", None), **result_target(b, x))
        ws.release(mark)


register_mixer("scored_attention", ScoredAttention)
