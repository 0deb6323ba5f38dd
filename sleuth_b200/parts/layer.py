"""Arrangements of a mixer, a feed-forward and their norms in one layer.

``parallel``: x += mixer(norm1(x)) + ffn(norm2(x)), both sublayers reading the same x; with one norm
(``norm2`` absent) the feed-forward reads norm1's output too; the feed-forward may be absent.

``prenorm``: x += mixer(norm1(x)); x += ffn(norm2(x)) (sleuth/forge/model/transformer.py:78,87-88,96,99).
``sandwich``: a norm in front of and behind each sublayer, x += post1(mixer(norm1(x))), then x += post2(ffn(norm2(x)));
with ``gated`` each sublayer's result is multiplied by sigmoid(W h + b) of the sublayer's own input h before its norm.

The layer owns the residual arrangement only; the parts it is given decide everything else. The sum
itself is a float32 accumulation into the stream, done by the last product of the mixer or ffn.
"""

from __future__ import annotations

import os

import torch

from ..kernels import ops
from .base import BuildContext, Normed, ParamDecl, Part, build_ffn, build_mixer, build_norm, lead_weight_of, register_layer
from .linear import Linear
from .spec import LayerSpec

# A parallel layer's mixer and feed-forward read the same x and need nothing from each other. In a step that brings one
# token a sequence, where a layer is a dozen short kernels that each wait for the one before, the feed-forward runs on
# a second stream beside the mixer (into a sum of its own that one kernel adds to the stream at the end), so the layer
# takes as long as its longer branch. Recorded steps keep the fork and the join. SLEUTH_B200_BRANCH=0 turns it off.
BRANCH = os.environ.get("SLEUTH_B200_BRANCH", "1") != "0"
# A gated sandwich layer lets its mixer's first float32 product carry the gate's rows (``accepts_rider``).
# SLEUTH_B200_RIDE=0 keeps the gate a product of its own.
RIDE = os.environ.get("SLEUTH_B200_RIDE", "1") != "0"
_SIDE: dict = {}


def _side_stream(device) -> "torch.cuda.Stream":
    key = torch.device(device).index
    if key not in _SIDE:
        _SIDE[key] = torch.cuda.Stream(device=device)
    return _SIDE[key]


class PreNormLayer(Part):
    def __init__(self, spec: LayerSpec, ctx: BuildContext):
        self.ctx = ctx
        self.norm1 = build_norm(spec.norm1, ctx)
        self.mixer = build_mixer(spec.mixer, ctx)
        self.norm2 = build_norm(spec.norm2, ctx)
        self.ffn = build_ffn(spec.ffn, ctx)
        self.children = {"norm1": self.norm1, "mixer": self.mixer, "norm2": self.norm2, "ffn": self.ffn}
        self.capturable = all(getattr(p, "capturable", True) for p in self.children.values())

    def declare(self):
        out = {}
        for prefix, part in self.children.items():
            for name, decl in part.declare().items():
                out[f"{prefix}.{name}"] = decl
        return out

    def bind(self, tensors):
        for prefix, part in self.children.items():
            part.bind({k[len(prefix) + 1:]: v for k, v in tensors.items() if k.startswith(prefix + ".")})

    def cache_request(self):
        return self.mixer.cache_request()

    def lead_weight(self):
        return lead_weight_of(self.mixer)

    def fused_decode(self):
        """x += mixer(norm1(x)); x += ffn(norm2(x)) is what the persistent single-token kernel runs: offered when all
        four parts offer their share."""
        shares = {name: getattr(part, "fused_decode", lambda: None)() for name, part in self.children.items()}
        if any(v is None for v in shares.values()):
            return None
        if "w_qkv" not in shares["mixer"] or "w_gu" not in shares["ffn"] or "gain" not in shares["norm1"] or "gain" not in shares["norm2"]:
            return None
        return shares

    def forward(self, x, b, view, ws):
        mark = ws.mark()
        after = getattr(b, "next_read", None)    # what follows this layer
        b.next_read = lead_weight_of(self.ffn)
        self.mixer.forward(self._input(self.norm1, self.mixer, x, b, ws), x, b, view, ws)
        ws.release(mark)
        b.next_read = after
        self.ffn.forward(self._input(self.norm2, self.ffn, x, b, ws), x, b, ws)
        ws.release(mark)

    def _input(self, norm, part, x, b, ws):
        """What ``part`` reads: the normalised tensor, or, for a part that can normalise inside its first
        product, a ``Normed`` that runs the norm kernel only if asked for the tensor."""
        n = Normed(norm, x, ws, b.stream, self.ctx.dtype)
        return n if part.accepts_normed else n.tensor()


class ParallelLayer(Part):
    """x += mixer(norm1(x)) + ffn(norm2(x)): both sublayers read the same x and each adds its result into the float32
    stream, so both norms run before either sublayer does. With one norm (no ``norm2``) the feed-forward reads norm1's
    output. The feed-forward may be absent."""

    def __init__(self, spec: LayerSpec, ctx: BuildContext):
        self.ctx = ctx
        self.norm1 = build_norm(spec.norm1, ctx)
        self.mixer = build_mixer(spec.mixer, ctx)
        self.ffn = build_ffn(spec.ffn, ctx) if spec.ffn is not None else None
        self.norm2 = build_norm(spec.norm2, ctx) if (spec.norm2 is not None and self.ffn is not None) else None
        self.children = {"norm1": self.norm1, "mixer": self.mixer}
        if self.norm2 is not None:
            self.children["norm2"] = self.norm2
        if self.ffn is not None:
            self.children["ffn"] = self.ffn
        self.capturable = all(getattr(p, "capturable", True) for p in self.children.values())

    declare = PreNormLayer.declare
    bind = PreNormLayer.bind
    cache_request = PreNormLayer.cache_request
    lead_weight = PreNormLayer.lead_weight

    def forward(self, x, b, view, ws):
        mark = ws.mark()
        after = getattr(b, "next_read", None)
        # the feed-forward's input is formed before the mixer adds into the stream; two norms that can share a pass do
        together = getattr(self.norm1, "forward_with", None) if self.norm2 is not None else None
        h = h2 = None
        if together is not None:
            h, h2 = ws.take(x.shape, self.ctx.dtype), ws.take(x.shape, self.ctx.dtype)
            if not together(self.norm2, x, h, h2, stream=b.stream):
                h = h2 = None
        if h is None:
            h = Normed(self.norm1, x, ws, b.stream, self.ctx.dtype).tensor()
            h2 = Normed(self.norm2, x, ws, b.stream, self.ctx.dtype).tensor() if self.norm2 is not None else h
        if self.ffn is not None and BRANCH and b.max_count == 1:
            self._forward_branches(h, h2, x, b, view, ws, after)
            ws.release(mark)
            return
        b.next_read = lead_weight_of(self.ffn) if self.ffn is not None else after
        self.mixer.forward(h, x, b, view, ws)
        b.next_read = after
        if self.ffn is not None:
            self.ffn.forward(h2, x, b, ws)
        ws.release(mark)

    def _forward_branches(self, h, h2, x, b, view, ws, after):
        """The feed-forward on a second stream into a sum of its own, the mixer on this one into the stream, then
        x += that sum. The two branches' scratch memory must not overlap: the feed-forward's is taken first, and the
        mixer's begins above the highest address the feed-forward used."""
        main = torch.cuda.current_stream()
        side = _side_stream(x.device)
        x2 = ws.take(x.shape, torch.float32)
        seen, ws.high = ws.high, ws.top
        side.wait_stream(main)                  # the norms' outputs are ready
        b.next_read = None
        with torch.cuda.stream(side):
            b.stream = side.cuda_stream
            x2.zero_()
            self.ffn.forward(h2, x2, b, ws)
        b.stream = main.cuda_stream
        ws.top = max(ws.top, ws.high)
        ws.high = max(seen, ws.high)
        b.next_read = after
        self.mixer.forward(h, x, b, view, ws)
        main.wait_stream(side)
        ops.add(x, x2, stream=b.stream)


class SandwichLayer(Part):
    """x += post1(gate1 * mixer(norm1(x))); x += post2(gate2 * ffn(norm2(x))), gate_k = sigmoid(W_k h + b_k) of the
    sublayer's input h (only with ``spec.gated``). A sublayer adds its result into a zeroed float32 buffer of the
    stream's shape (its last product accumulates, as it would into the stream); one kernel then applies the gate,
    normalises the row and adds it to the stream. The gate's pre-activations are float32. The feed-forward may be absent.
    The closing norms must be RMS norms (their gain and eps are handed to that kernel)."""

    def __init__(self, spec: LayerSpec, ctx: BuildContext):
        self.ctx, self.gated = ctx, bool(spec.gated)
        self.hidden = spec.norm1.dim
        self.norm1 = build_norm(spec.norm1, ctx)
        self.mixer = build_mixer(spec.mixer, ctx)
        self.post1 = build_norm(spec.post1, ctx)
        self.ffn = build_ffn(spec.ffn, ctx) if spec.ffn is not None else None
        self.children = {"norm1": self.norm1, "mixer": self.mixer, "post1": self.post1}
        if self.ffn is not None:
            self.norm2, self.post2 = build_norm(spec.norm2, ctx), build_norm(spec.post2, ctx)
            self.children.update({"norm2": self.norm2, "ffn": self.ffn, "post2": self.post2})
        for name, part in self.children.items():
            if name.startswith("post") and not getattr(part, "fusable", False):
                raise ValueError("sandwich layer: the norm behind a sublayer must be an RMS norm")
        self.gate1 = self.gate2 = self.bias1 = self.bias2 = None
        self.capturable = all(getattr(p, "capturable", True) for p in self.children.values())

    def declare(self):
        out = PreNormLayer.declare(self)
        if self.gated:
            for k in ("1", "2") if self.ffn is not None else ("1",):
                out[f"gate{k}.weight"] = ParamDecl((self.hidden, self.hidden))
                out[f"gate{k}.bias"] = ParamDecl((self.hidden,), "vector")
        return out

    def bind(self, tensors):
        # a mixer that can carry extra rows in its first float32 product takes the gate's matrix along: one product less,
        # and the gate's pre-activations come out of the same pass over the normed rows
        self.rides = self.gated and getattr(self.mixer, "accepts_rider", False) and RIDE
        if self.rides:
            tensors = dict(tensors)
            tensors["mixer.rider.weight"] = tensors["gate1.weight"]
        PreNormLayer.bind(self, tensors)
        if self.gated:
            self.gate1 = None if self.rides else Linear(tensors["gate1.weight"], self.ctx.dtype)
            self.bias1 = tensors["gate1.bias"]
            if self.ffn is not None:
                self.gate2, self.bias2 = Linear(tensors["gate2.weight"], self.ctx.dtype), tensors["gate2.bias"]

    cache_request = PreNormLayer.cache_request

    def lead_weight(self):
        return lead_weight_of(self.mixer)

    def forward(self, x, b, view, ws):
        after = getattr(b, "next_read", None)
        self._sublayer(self.norm1, self.mixer, self.post1, self.gate1, self.bias1, x, b, ws, view,
                       lead_weight_of(self.ffn) if self.ffn is not None else after, self.rides)
        if self.ffn is not None:
            self._sublayer(self.norm2, self.ffn, self.post2, self.gate2, self.bias2, x, b, ws, None, after, False)
        b.next_read = after

    def _sublayer(self, norm, part, post, gate, bias, x, b, ws, view, after, rides):
        mark = ws.mark()
        y = ws.take(x.shape, torch.float32)
        n = Normed(norm, x, ws, b.stream, self.ctx.dtype)
        # the part alone reads the normed rows when the gate rides with it: it may then normalise inside its first product
        h = n if rides and part.accepts_normed else n.tensor()
        if getattr(part, "stores_result", False):
            b.store_first = True        # the part's first delivery into y is a store
        else:
            y.zero_()
        b.rider = None
        b.next_read = gate.weight if gate is not None else after
        if part is self.mixer:
            part.forward(h, y, b, view, ws)
        else:
            part.forward(h, y, b, ws)
        if getattr(b, "store_first", False):
            raise RuntimeError(f"{type(part).__name__} says it stores its result and did not")
        if rides:
            g = b.rider         # a view into the part's scratch memory: nothing takes scratch before the next kernel reads it
        else:
            g = gate.forward(n.tensor(), ws=ws, stream=b.stream, out_dtype=torch.float32, next_read=after) if gate is not None else None
        ops.gated_norm_add(x, y, g, bias if g is not None else None, post.weight, post.eps, b.stream)
        ws.release(mark)


class HyperLayer(Part):
    """Hyper-connections: the stream is ``streams`` copies [tokens, streams * hidden]. Sublayer q reads the copies' weighted
    sum through its norm (one kernel), delivers into an empty float32 buffer, and one kernel then rewrites all copies:
    x_r <- sum_s mix[s, r] x_s + mult * out[r] * y. With ``streams`` 0 there is one copy and no coefficients: the plain
    pre-norm layer with a multiplier on each sublayer's result. The norms must be RMS norms. The feed-forward may be absent."""

    def __init__(self, spec: LayerSpec, ctx: BuildContext):
        self.ctx, self.streams, self.mult = ctx, int(spec.streams), float(spec.residual_mult)
        self.hidden = spec.norm1.dim
        self.norm1 = build_norm(spec.norm1, ctx)
        self.mixer = build_mixer(spec.mixer, ctx)
        self.ffn = build_ffn(spec.ffn, ctx) if spec.ffn is not None else None
        self.children = {"norm1": self.norm1, "mixer": self.mixer}
        if self.ffn is not None:
            self.norm2 = build_norm(spec.norm2, ctx)
            self.children.update({"norm2": self.norm2, "ffn": self.ffn})
        for name, part in self.children.items():
            if name.startswith("norm") and not getattr(part, "fusable", False):
                raise ValueError("hyper layer: its norms must be RMS norms")
        if self.streams > 16:
            raise ValueError(f"hyper layer: at most 16 copies of the stream, got {self.streams}")
        self.coef = {}
        self.capturable = all(getattr(p, "capturable", True) for p in self.children.values())

    def declare(self):
        out = PreNormLayer.declare(self)
        if self.streams:
            for q in ("1", "2") if self.ffn is not None else ("1",):
                out[f"hc{q}.in"] = ParamDecl((self.streams,), "vector", init="gain")
                out[f"hc{q}.out"] = ParamDecl((self.streams,), "vector", init="gain")
                out[f"hc{q}.mix"] = ParamDecl((self.streams, self.streams), "vector")
        return out

    def bind(self, tensors):
        PreNormLayer.bind(self, tensors)
        self.coef = {k: v.to(torch.float32).contiguous() for k, v in tensors.items() if k.startswith("hc")}

    cache_request = PreNormLayer.cache_request

    def lead_weight(self):
        return lead_weight_of(self.mixer)

    def forward(self, x, b, view, ws):
        after = getattr(b, "next_read", None)
        self._sublayer("1", self.norm1, self.mixer, x, b, ws, view, lead_weight_of(self.ffn) if self.ffn is not None else after)
        if self.ffn is not None:
            self._sublayer("2", self.norm2, self.ffn, x, b, ws, None, after)
        b.next_read = after

    def _sublayer(self, q, norm, part, x, b, ws, view, after):
        mark = ws.mark()
        T = x.shape[0]
        h = ws.take((T, self.hidden), self.ctx.dtype)
        ops.hyper_read(x, self.coef.get(f"hc{q}.in"), norm.weight, h, norm.eps, b.stream)
        y = ws.take((T, self.hidden), torch.float32)
        if getattr(part, "stores_result", False):
            b.store_first = True
        else:
            y.zero_()
        b.next_read = after
        if part is self.mixer:
            part.forward(h, y, b, view, ws)
        else:
            part.forward(h, y, b, ws)
        if getattr(b, "store_first", False):
            raise RuntimeError(f"{type(part).__name__} says it stores its result and did not")
        ops.hyper_write(x, y, self.coef.get(f"hc{q}.mix"), self.coef.get(f"hc{q}.out"), self.mult, b.stream)
        ws.release(mark)


register_layer("hyper", HyperLayer)
register_layer("sandwich", SandwichLayer)
register_layer("prenorm", PreNormLayer)
register_layer("parallel", ParallelLayer)
