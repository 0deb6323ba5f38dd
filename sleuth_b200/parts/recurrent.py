"""Recurrent mixers: a float32 state per sequence instead of a cache of keys and values.

``mingru``: a recurrence whose update gate and candidate are functions of the step's input alone (neither sees the state), so a portion's gates are one product. With h the layer's normed input and
``width`` channels:

    z = sigmoid(W_z h + b_z)        u = W_x h + b_x        c = u + 1/2 where u >= 0, sigmoid(u) below
    S_t = (1 - z) S_(t-1) + z c     (S = 0 before a sequence's first token)
    output = W_o (S_t * silu(W_g h)),  added into the stream

The three projections are one stacked product with a float32 result (a layer's own rows may ride behind them, and
the layer's norm runs in that product's prologue where the kernel can); biases, gates, the candidate, the state and
its product with silu(g) are float32 (``csrc/recurrent.cu``), rounded once where the output projection reads them.
The state lives in the cache's per-sequence region (``StateRequest``): zero when a slot is taken, carried from step
to step, so prompts may arrive whole, in portions or token by token. Nothing depends on the host's view of the step,
so single-token steps replay as CUDA graphs.

``state_space`` (``StateSpaceSpec``) and ``gated_linear_attention`` (``GatedLinearAttentionSpec``) keep a matrix per head
and sequence, S_t = diag(a_t) S_(t-1) + k_t v_t^T with outputs S_t^T q_t, and share one recurrence kernel
(``ops.decay_scan``): the first reads one decay a head, exp(-exp(A_log) dt), keys B, queries C and values dt * x after
a short convolution with silu; the second a decay per key channel, sigmoid(.)^(1/tau), from a low-rank projection. Their
projections are stacked products with float32 results; decays, step sizes, the state, the skip term, the gates and the
group norms are float32 (``csrc/state_mixers.cu``), rounded once where the output projection reads them.
"""

from __future__ import annotations

import torch

from ..cache.paged import BundleRequest, StateRequest
from ..kernels import ops
from .base import BuildContext, Normed, ParamDecl, Part, register_mixer, result_target
from .linear import Linear
from .spec import GatedLinearAttentionSpec, MinGRUSpec, StateSpaceSpec


class MinGRU(Part):
    accepts_normed = True       # the stacked product normalises in its prologue where its kernel can
    stores_result = True
    accepts_rider = True

    def __init__(self, spec: MinGRUSpec, ctx: BuildContext):
        if spec.width < 1 or spec.hidden < 1:
            raise ValueError(f"mingru: width {spec.width}, hidden {spec.hidden}")
        self.spec, self.ctx = spec, ctx
        self.zxg = self.o = self.bz = self.bx = None

    def declare(self):
        s = self.spec
        return {"z.weight": ParamDecl((s.width, s.hidden)), "z.bias": ParamDecl((s.width,), "vector"),
                "x.weight": ParamDecl((s.width, s.hidden)), "x.bias": ParamDecl((s.width,), "vector"),
                "g.weight": ParamDecl((s.width, s.hidden)), "o.weight": ParamDecl((s.hidden, s.width))}

    def bind(self, t):
        dt = self.ctx.dtype
        stack = [t["z.weight"], t["x.weight"], t["g.weight"]]
        self.rider_rows = 0
        if t.get("rider.weight") is not None:       # the layer's rows ride behind the three projections
            stack.append(t["rider.weight"])
            self.rider_rows = t["rider.weight"].shape[0]
        self.zxg = Linear(torch.cat(stack, dim=0), dt)
        self.o = Linear(t["o.weight"], dt)
        self.bz, self.bx = t["z.bias"].contiguous(), t["x.bias"].contiguous()

    def cache_request(self):
        return StateRequest((self.spec.width,), torch.float32)

    def lead_weight(self):
        return self.zxg.weight if self.zxg is not None else None

    def forward(self, h, x, b, view, ws):
        W, T = self.spec.width, h.shape[0]
        mark = ws.mark()
        p = self.zxg.forward(h, ws=ws, stream=b.stream, out_dtype=torch.float32, next_read=self.o.weight)
        if self.rider_rows:
            b.rider = p[:, 3 * W:]
        y = ws.take((T, W), self.ctx.dtype)
        need = ops.mingru_scratch_floats(b.n, b.max_count, W)
        scratch = ws.take((need,), torch.float32) if need else None
        ops.mingru(p[:, :3 * W], self.bz, self.bx, view.state, b.slots, b.seq_start, y, b.max_count, scratch, b.stream)
        self.o.forward(y, ws=ws, stream=b.stream, next_read=getattr(b, "next_read", None), **result_target(b, x))
        ws.release(mark)


class StateSpace(Part):
    stores_result = True

    def __init__(self, spec: StateSpaceSpec, ctx: BuildContext):
        s = spec
        if s.heads % s.groups or s.state > 256 or not 1 <= s.conv_taps <= 16 or (s.heads * s.value_dim) % s.norm_groups:
            raise ValueError(f"state_space: heads {s.heads}, groups {s.groups}, state {s.state} (at most 256), conv_taps {s.conv_taps} "
                             f"(1 to 16), norm_groups {s.norm_groups}")
        self.spec, self.ctx = spec, ctx
        self.inner = s.heads * s.value_dim
        self.bc = s.groups * s.state
        self.proj = self.o = None

    def declare(self):
        s = self.spec
        conv = self.inner + 2 * self.bc
        return {"in.weight": ParamDecl((2 * self.inner + 2 * self.bc + s.heads, s.hidden)),
                "conv.weight": ParamDecl((conv, s.conv_taps), "vector"), "conv.bias": ParamDecl((conv,), "vector"),
                "dt_bias": ParamDecl((s.heads,), "vector"), "A_log": ParamDecl((s.heads,), "vector"),
                "D": ParamDecl((s.heads,), "vector", init="gain"), "norm.weight": ParamDecl((self.inner,), "vector", init="gain"),
                "o.weight": ParamDecl((s.hidden, self.inner))}

    def bind(self, t):
        dt = self.ctx.dtype
        self.proj, self.o = Linear(t["in.weight"], dt), Linear(t["o.weight"], dt)
        f = lambda n: t[n].to(torch.float32).contiguous()
        self.conv_w, self.conv_b, self.dt_bias, self.a_log, self.skip, self.gain = (
            f("conv.weight"), f("conv.bias"), f("dt_bias"), f("A_log"), f("D"), f("norm.weight"))

    def cache_request(self):
        s = self.spec
        parts = [("state", StateRequest((s.heads, s.state, s.value_dim), torch.float32))]
        if s.conv_taps > 1:
            parts.append(("tail", StateRequest((s.conv_taps - 1, self.inner + 2 * self.bc), torch.float32)))
        return BundleRequest(tuple(parts))

    def lead_weight(self):
        return self.proj.weight if self.proj is not None else None

    def forward(self, h, x, b, view, ws):
        s, inner, bc = self.spec, self.inner, self.bc
        if isinstance(h, Normed):
            h = h.tensor()
        T = h.shape[0]
        mark = ws.mark()
        p = self.proj.forward(h, ws=ws, stream=b.stream, out_dtype=torch.float32)      # [z | x B C | dt]
        xbc = ws.take((T, inner + 2 * bc), torch.float32)
        tail = view["tail"].state if s.conv_taps > 1 else p[:0]
        ops.causal_conv(p[:, inner:], self.conv_w, self.conv_b, tail, b.slots, b.tok_seq, b.seq_start, xbc, True, b.stream, max_count=b.max_count)
        dt, decay = ws.take((T, s.heads), torch.float32), ws.take((T, s.heads), torch.float32)
        ops.step_decay(p[:, 2 * inner + 2 * bc:], self.dt_bias, self.a_log, dt, decay, b.stream)
        y = ws.take((T, inner), torch.float32)
        need = ops.decay_scan_scratch_floats(b.n, b.max_count, s.heads, s.state, s.value_dim, False)
        scratch = ws.take((need,), torch.float32) if need else None
        ops.decay_scan(xbc[:, inner + bc:], xbc[:, inner:inner + bc], xbc[:, :inner], decay, view["state"].state, b.slots,
                       b.seq_start, y, s.heads, s.groups, False, v_scale=dt, stream=b.stream, max_count=b.max_count, scratch=scratch)
        g = ws.take((T, inner), self.ctx.dtype)
        ops.gated_group_norm(y, p[:, :inner], self.gain, g, s.norm_groups, s.eps, True, skip=xbc[:, :inner], skip_gain=self.skip,
                             head_width=s.value_dim, stream=b.stream)
        self.o.forward(g, ws=ws, stream=b.stream, next_read=getattr(b, "next_read", None), **result_target(b, x))
        ws.release(mark)


class GatedLinearAttention(Part):
    stores_result = True

    def __init__(self, spec: GatedLinearAttentionSpec, ctx: BuildContext):
        s = spec
        if s.head_dim > 256 or s.head_dim < 1 or s.decay_rank < 1 or not s.tau > 0:
            raise ValueError(f"gated_linear_attention: head_dim {s.head_dim} (at most 256), decay_rank {s.decay_rank}, tau {s.tau}")
        self.spec, self.ctx = spec, ctx
        self.nk, self.nv = s.heads * s.head_dim, s.heads * s.value_dim
        self.proj = self.a2 = self.o = None

    def declare(self):
        s = self.spec
        return {"q.weight": ParamDecl((self.nk, s.hidden)), "k.weight": ParamDecl((self.nk, s.hidden)),
                "v.weight": ParamDecl((self.nv, s.hidden)), "g.weight": ParamDecl((self.nv, s.hidden)),
                "a1.weight": ParamDecl((s.decay_rank, s.hidden)), "a2.weight": ParamDecl((self.nk, s.decay_rank)),
                "a2.bias": ParamDecl((self.nk,), "vector"), "norm.weight": ParamDecl((s.value_dim,), "vector", init="gain"),
                "o.weight": ParamDecl((s.hidden, self.nv))}

    def bind(self, t):
        dt = self.ctx.dtype
        self.proj = Linear(torch.cat([t[n + ".weight"] for n in ("q", "k", "v", "g", "a1")], dim=0), dt)
        self.a2, self.o = Linear(t["a2.weight"], dt), Linear(t["o.weight"], dt)
        self.a2_bias = t["a2.bias"].to(torch.float32).contiguous()
        self.gain = t["norm.weight"].to(torch.float32).contiguous()

    def cache_request(self):
        s = self.spec
        return BundleRequest((("state", StateRequest((s.heads, s.head_dim, s.value_dim), torch.float32)),))

    def lead_weight(self):
        return self.proj.weight if self.proj is not None else None

    def forward(self, h, x, b, view, ws):
        s, nk, nv = self.spec, self.nk, self.nv
        if isinstance(h, Normed):
            h = h.tensor()
        T = h.shape[0]
        mark = ws.mark()
        p = self.proj.forward(h, ws=ws, stream=b.stream, out_dtype=torch.float32)      # [q | k | v | g | a1]
        low = ws.take((T, s.decay_rank), self.ctx.dtype)
        low.copy_(p[:, 2 * nk + 2 * nv:])
        z = self.a2.forward(low, ws=ws, stream=b.stream, out_dtype=torch.float32)
        ops.channel_decay(z, self.a2_bias, s.tau, b.stream)
        y = ws.take((T, nv), torch.float32)
        need = ops.decay_scan_scratch_floats(b.n, b.max_count, s.heads, s.head_dim, s.value_dim, True)
        scratch = ws.take((need,), torch.float32) if need else None
        ops.decay_scan(p[:, :nk], p[:, nk:2 * nk], p[:, 2 * nk:2 * nk + nv], z, view["state"].state, b.slots, b.seq_start, y,
                       s.heads, s.heads, True, q_scale=s.head_dim ** -0.5, stream=b.stream, max_count=b.max_count, scratch=scratch)
        g = ws.take((T, nv), self.ctx.dtype)
        ops.gated_group_norm(y, p[:, 2 * nk + nv:2 * nk + 2 * nv], self.gain, g, s.heads, s.eps, False, stream=b.stream)
        self.o.forward(g, ws=ws, stream=b.stream, next_read=getattr(b, "next_read", None), **result_target(b, x))
        ws.release(mark)


register_mixer("mingru", MinGRU)
register_mixer("state_space", StateSpace)
register_mixer("gated_linear_attention", GatedLinearAttention)
