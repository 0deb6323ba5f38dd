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
"""

from __future__ import annotations

import torch

from ..cache.paged import StateRequest
from ..kernels import ops
from .base import BuildContext, Normed, ParamDecl, Part, register_mixer, result_target
from .linear import Linear
from .spec import MinGRUSpec


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


register_mixer("mingru", MinGRU)
