"""Routed experts as a feed-forward part.

Router logits z = W_r h + b in float32 (W_r and b are kept in float32; h is the layer's normed input in the run
dtype). A token uses the ``top`` experts with the largest logits, weighted by the softmax over those logits alone, or
(``scoring="sigmoid"``) those with the largest sigmoid scores among the best groups of neighbouring experts, weighted
by score / sum of the chosen scores, scaled, or (``scoring="softmax"``) those with the largest softmax score plus a
correction per expert, weighted by the uncorrected scores times a scale, without division by their sum; an expert is down(f(gate h, up h)) with one of the gated activations. The
part's output, the weighted sum (plus a shared expert that every token runs, when the spec names one), is added into
the stream.

The experts' matrices are stacked at load time ([experts, 2 * ff, hidden] for gate and up, [experts, hidden, ff]
for down). A step runs five kernels (``csrc/moe.cu``): router, the counts and the expert-ordered list of (token,
choice) pairs, gate/up with the activation, down scaled by the pair's weight, and the sum over a token's choices
in the order of the choices; bfloat16 steps of many pairs gather the tokens' rows into the expert order and run both
products as grouped tcgen05 products instead (``ops.moe_experts_tc``). None of them needs the host to know the counts, so the part can be recorded in a
CUDA graph like any other.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import BuildContext, Normed, ParamDecl, Part, build_ffn, register_ffn
from .linear import Linear
from .spec import RoutedExpertsSpec


# From this many (token, choice) pairs on a bfloat16 step runs its experts as grouped tcgen05 products (row tiles of 128
# pairs an expert); below, the warp-level kernels, whose tiles of 64 rows waste less on experts with few pairs.
TC_PAIRS = 1024


class RoutedExperts(Part):
    def __init__(self, spec: RoutedExpertsSpec, ctx: BuildContext):
        if spec.activation not in ops.ACTIVATIONS:
            raise ValueError(f"routed_experts: activation {spec.activation!r} is not supported ({sorted(ops.ACTIVATIONS)})")
        if not 0 < spec.top <= spec.experts:
            raise ValueError(f"routed_experts: top {spec.top} of {spec.experts} experts")
        if spec.scoring not in ops.ROUTE_SCORINGS:
            raise ValueError(f"routed_experts: scoring {spec.scoring!r} is not one of {sorted(ops.ROUTE_SCORINGS)}")
        if spec.groups < 1 or spec.experts % spec.groups or not 1 <= spec.keep_groups <= spec.groups:
            raise ValueError(f"routed_experts: {spec.experts} experts in {spec.groups} groups of which {spec.keep_groups} are kept")
        if spec.shared_gate and spec.shared is None:
            raise ValueError("routed_experts: a gate on the shared expert needs a shared expert")
        if spec.choice_bias and spec.scoring not in ("softmax", "softmax_norm"):
            raise ValueError("routed_experts: a choice correction goes with the softmax scoring over all experts")
        if spec.groups > 1 and spec.scoring != "sigmoid":
            raise ValueError("routed_experts: groups of experts go with the sigmoid scoring")
        if spec.keep_groups * (spec.experts // spec.groups) < spec.top:
            raise ValueError(f"routed_experts: {spec.keep_groups} groups of {spec.experts // spec.groups} experts cannot give {spec.top} choices")
        if spec.activation == "clamped_swish" and not spec.limit > 0:
            raise ValueError(f"routed_experts: the clamped swish needs a positive limit, got {spec.limit}")
        self.spec, self.ctx = spec, ctx
        self.w_router = self.bias = self.w_gate_up = self.w_down = self.router_product = self.pick_bias = None
        self.shared = build_ffn(spec.shared, ctx) if spec.shared is not None else None

    def lead_weight(self):
        return self.shared.lead_weight() if self.shared is not None else None

    def declare(self):
        s = self.spec
        d = {"router.weight": ParamDecl((s.experts, s.hidden), "vector")}
        if s.router_bias:
            d["router.bias"] = ParamDecl((s.experts,), "vector")
        if s.choice_bias:
            d["correction"] = ParamDecl((s.experts,), "vector")
        for e in range(s.experts):
            d[f"e{e}.gate.weight"] = ParamDecl((s.intermediate, s.hidden))
            d[f"e{e}.up.weight"] = ParamDecl((s.intermediate, s.hidden))
            d[f"e{e}.down.weight"] = ParamDecl((s.hidden, s.intermediate))
        if self.shared is not None:
            for name, decl in self.shared.declare().items():
                d["shared." + name] = decl
        if s.shared_gate:
            d["shared_gate"] = ParamDecl((1, s.hidden), "vector")
        return d

    def bind(self, t):
        s, dt = self.spec, self.ctx.dtype
        self.w_router = t["router.weight"].to(torch.float32).contiguous()
        self.bias = t["router.bias"].to(torch.float32).contiguous() if s.router_bias else None
        self.pick_bias = t["correction"].to(torch.float32).contiguous() if s.choice_bias else None
        self.w_gate_up = torch.stack([torch.cat([t[f"e{e}.gate.weight"], t[f"e{e}.up.weight"]], dim=0)
                                      for e in range(s.experts)]).to(dt).contiguous()
        self.w_down = torch.stack([t[f"e{e}.down.weight"] for e in range(s.experts)]).to(dt).contiguous()
        if self.shared is not None:
            self.shared.bind({k[len("shared."):]: v for k, v in t.items() if k.startswith("shared.")})
        self.w_shared_gate = t["shared_gate"].to(torch.float32).reshape(-1).contiguous() if s.shared_gate else None
        # A bfloat16 run whose router matrix is exactly representable in bfloat16 (a file that stores it so) forms the
        # logits as a product of its own: bfloat16 times bfloat16 is exact in float32 and the sums are float32, so these
        # are the float32 logits of the same inputs, from the tensor cores instead of a lane per token.
        self.router_product = None
        if (dt == torch.bfloat16 and self.bias is None and s.hidden % 32 == 0 and s.experts >= 8
                and torch.equal(self.w_router.to(torch.bfloat16).to(torch.float32), self.w_router)):
            self.router_product = Linear(self.w_router.to(torch.bfloat16), dt)

    @property
    def stores_result(self):
        """The shared expert's last product reaches ``x`` first (and may store); the chosen experts add to it."""
        return self.shared is not None

    def forward(self, h, x, b, ws):
        s, dt = self.spec, self.ctx.dtype
        if isinstance(h, Normed):
            h = h.tensor()
        mark = ws.mark()
        if self.shared is not None:       # the shared expert first: its weights are what the layer in front asked L2 for
            after = getattr(b, "next_read", None)
            b.next_read = None
            if self.w_shared_gate is None:
                self.shared.forward(h, x, b, ws)
            else:                         # its result times sigmoid(w . h), one number a token, joins the stream in one kernel
                store = bool(getattr(b, "store_first", False))
                own = ws.take(x.shape, torch.float32)
                if getattr(self.shared, "stores_result", False):
                    b.store_first = True
                else:
                    b.store_first = False
                    own.zero_()
                self.shared.forward(h, own, b, ws)
                ops.row_gate(h, self.w_shared_gate, own, x, accumulate=not store, stream=b.stream)
            b.next_read = after
        T = h.shape[0]
        pairs = T * s.top
        choice, rank, place, order = (ws.take((pairs,), torch.int32) for _ in range(4))
        counts = ws.take((s.experts,), torch.int32)
        weight = ws.take((pairs,), torch.float32)
        act = ws.take((pairs, s.intermediate), dt)
        y = ws.take((pairs, s.hidden), torch.float32)
        logits = ws.take((T, s.experts), torch.float32)
        # (Letting the choosing kernel form a single token's logits itself, one launch instead of two, was measured
        # slower: 0.461 against 0.374 ms a step at width 1,024 and batch 1, 0.708 against 0.425 ms at width 2,048: one
        # block walks all of the router's rows.)
        ready = self.router_product is not None
        if ready:
            self.router_product.forward(h, out=logits, ws=ws, stream=b.stream)
        # steps of many pairs: the tcgen05 grouped products (bfloat16, inner sizes that TMA takes)
        grouped = (dt == torch.bfloat16 and pairs >= TC_PAIRS and s.hidden % 8 == 0
                   and s.intermediate % 8 == 0)
        tiles = ws.take((ops.moe_tile_words(T, s.top, s.experts),), torch.int32) if grouped else None
        ops.moe_route(h, self.w_router, self.bias, choice, weight, rank, counts, place, order, s.top, b.stream, logits, tiles,
                      layout=pairs > ops.MOE_FEW_PAIRS, scoring=s.scoring, groups=s.groups, keep=s.keep_groups,
                      scale=s.route_scale, logits_ready=ready, pick_bias=self.pick_bias)
        if grouped:
            xs = ws.take((pairs, s.hidden), dt)
            ops.moe_experts_tc(h, self.w_gate_up, self.w_down, order, place, weight, tiles, xs, act, y, x, s.top, b.stream,
                               activation=s.activation, limit=s.limit, alpha=s.alpha)
        else:
            ops.moe_experts(h, self.w_gate_up, self.w_down, counts, order, weight, act, y, x, s.top, s.activation, b.stream,
                            choice, place, limit=s.limit, alpha=s.alpha)
        ws.release(mark)


register_ffn("routed_experts", RoutedExperts)
