"""Two mixers side by side: both read the same normed input, each delivers into a float32 buffer of its own, and one
kernel joins the two results into the stream (``SideBySideSpec``): half the sum of the two after an RMS norm each with a
gain of its own, or a weighted sum. The pair's cache entry is a bundle of the two mixers' requests, so an attention's
pages and a recurrence's state of one layer are taken, freed and reused together.

The two mixers need nothing from each other. In a step that brings one token a sequence, where each is a chain of short
kernels that wait for one another, the right one runs on a second stream beside the left one (as a parallel layer's
feed-forward does, ``parts/layer.py``); recorded steps keep the fork and the join. SLEUTH_B200_BRANCH=0 turns it off.
"""

from __future__ import annotations

import torch

from ..cache.paged import BundleRequest
from ..kernels import ops
from .base import BuildContext, Normed, ParamDecl, Part, build_mixer, lead_weight_of, register_mixer
from .layer import BRANCH, _side_stream
from .spec import SideBySideSpec


class SideBySide(Part):
    stores_result = True

    def __init__(self, spec: SideBySideSpec, ctx: BuildContext):
        if spec.combine not in ("normed_mean", "scaled"):
            raise ValueError(f"side_by_side: combine {spec.combine!r} is not 'normed_mean' or 'scaled'")
        self.spec, self.ctx = spec, ctx
        self.left, self.right = build_mixer(spec.left, ctx), build_mixer(spec.right, ctx)
        self.children = {"left": self.left, "right": self.right}
        self.capturable = all(getattr(p, "capturable", True) for p in self.children.values())
        self.gain_left = self.gain_right = None

    def declare(self):
        out = {}
        for prefix, part in self.children.items():
            for name, decl in part.declare().items():
                out[f"{prefix}.{name}"] = decl
        if self.spec.combine == "normed_mean":
            out["left_out"] = ParamDecl((self.spec.hidden,), "vector", init="gain")
            out["right_out"] = ParamDecl((self.spec.hidden,), "vector", init="gain")
        return out

    def bind(self, t):
        for prefix, part in self.children.items():
            part.bind({k[len(prefix) + 1:]: v for k, v in t.items() if k.startswith(prefix + ".")})
        if self.spec.combine == "normed_mean":
            self.gain_left = t["left_out"].to(torch.float32).contiguous()
            self.gain_right = t["right_out"].to(torch.float32).contiguous()

    def cache_request(self):
        parts = tuple((n, r) for n, r in (("left", self.left.cache_request()), ("right", self.right.cache_request())) if r is not None)
        return BundleRequest(parts) if parts else None

    def lead_weight(self):
        return lead_weight_of(self.left)

    def forward(self, h, x, b, view, ws):
        s = self.spec
        if isinstance(h, Normed):
            h = h.tensor()
        store = bool(getattr(b, "store_first", False))
        b.store_first = False
        after = getattr(b, "next_read", None)
        mark = ws.mark()
        results = [ws.take(x.shape, torch.float32), ws.take(x.shape, torch.float32)]
        branch = BRANCH and b.max_count == 1 and x.is_cuda

        def run(i, name, part, following):
            y = results[i]
            if getattr(part, "stores_result", False):
                b.store_first = True
            else:
                y.zero_()
            b.next_read = following
            sub = view.get(name) if isinstance(view, dict) else None
            if isinstance(view, dict) and "borrowed" in view:
                sub = dict(sub) if isinstance(sub, dict) else {"own": sub}
                sub["borrowed"] = view["borrowed"].get(name) if isinstance(view["borrowed"], dict) else view["borrowed"]
            part.forward(h, y, b, sub, ws)
            if getattr(b, "store_first", False):
                raise RuntimeError(f"{type(part).__name__} says it stores its result and did not")

        if branch:
            # the right mixer on a second stream; its scratch memory is taken first, and the left one's begins above the
            # highest address it used, so the two never share a byte
            main, side = torch.cuda.current_stream(), _side_stream(x.device)
            seen, ws.high = ws.high, ws.top
            side.wait_stream(main)              # the normed input is ready
            with torch.cuda.stream(side):
                b.stream = side.cuda_stream
                run(1, "right", self.right, None)
            b.stream = main.cuda_stream
            ws.top = max(ws.top, ws.high)
            ws.high = max(seen, ws.high)
            run(0, "left", self.left, None)
            main.wait_stream(side)
        else:
            run(0, "left", self.left, lead_weight_of(self.right))
            run(1, "right", self.right, after)
        b.next_read = after
        if s.combine == "normed_mean":
            ops.pair_combine(results[0], results[1], x, self.gain_left, self.gain_right, 0.5, 0.5, s.eps, accumulate=not store,
                             stream=b.stream)
        else:
            ops.pair_combine(results[0], results[1], x, None, None, s.left_scale, s.right_scale, 0.0, accumulate=not store,
                             stream=b.stream)
        ws.release(mark)


register_mixer("side_by_side", SideBySide)
