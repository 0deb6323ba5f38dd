"""A model as the engine sees it: an embedding, layers built from a description, a schedule, a head.

``Model`` knows nothing about any architecture. It builds each layer from its ``LayerSpec`` through
the part registries, collects the tensors the parts declare under the names the description gives
them, asks the parts what their cache entries must hold, and runs ``ModelSpec.schedule``: a list of
layer applications that may name a layer twice (its weights are then shared and each application has
a cache entry of its own, as the reference's ``shared_layers``, sleuth/forge/model/config.py:80-86)
or let an application read the cache entry an earlier one wrote.

One forward pass is the reference's ``Transformer.forward`` (sleuth/forge/model/transformer.py:257-313)
for a ragged batch: embed, run the layers on the float32 stream, final norm and output matrix on the
rows whose logits are wanted only.
"""

from __future__ import annotations

import os

import torch

from ..parts import ends as _ends   # noqa: F401  (registers the token embedding and the output head)
from ..parts.base import BuildContext, ParamDecl, build_embedding, build_head, build_layer, lead_weight_of
from ..parts.spec import ModelSpec


# How a step in which every sequence brings one token runs: "fused" = runs of layers whose parts offer it go through
# the persistent kernel (csrc/decode_layers.cu), up to FUSED_DECODE_ROWS sequences; "kernels" = every layer launch
# by launch, as steps of many tokens always run.
DECODE_CHOICE = os.environ.get("SLEUTH_B200_DECODE", "kernels")
FUSED_DECODE_ROWS = 16
FUSED_DECODE_MIN_SLOTS = 5      # ring slots the kernel must have left beside the token rows in shared memory


class Model:
    def __init__(self, spec: ModelSpec, ctx: BuildContext):
        self.spec, self.ctx = spec, ctx
        self.embedding = build_embedding(spec.embedding, ctx)      # by ``spec.kind``, like every other part
        self.layers = [build_layer(ls, ctx) for ls in spec.layers]
        self.head = build_head(spec.head, ctx)
        self.hidden = spec.embedding.dim
        self.vocab = spec.head.vocab
        # single-token steps are recorded as CUDA graphs only if every layer allows it
        self.capturable = all(getattr(part, "capturable", True) for part in (self.embedding, *self.layers, self.head))
        # cache entries: the first application that names an entry owns it
        self.entry_owner: dict[int, int] = {}
        for i, e in enumerate(spec.schedule):
            self.entry_owner.setdefault(e.cache, i)
        self.cache_requests = [self.layers[spec.schedule[self.entry_owner[c]].layer].cache_request()
                               for c in range(len(self.entry_owner))]
        # an embedding that keeps something per sequence (the previous token, say) gets a cache entry behind the layers'
        self.embedding_entry = None
        request = getattr(self.embedding, "cache_request", lambda: None)()
        if request is not None:
            self.embedding_entry = len(self.cache_requests)
            self.cache_requests.append(request)
        self.pass_mix = None            # the product W [x; x0] of schedule entries that mix the embedding into the stream
        self._programs: dict = {}       # per cache: the runs of the schedule prepared for the persistent kernel
        self.pass_rows = None           # [rows, hidden] float32: vectors that schedule entries add to the stream
        self.keeps_embedding = any(e.add_embedding or e.mix_embedding for e in spec.schedule)
        self.observe = None             # callable(schedule index, stream) after every layer application, for inspection

    # ---- weights ----
    def _end_names(self, which: str) -> dict[str, str]:
        """Checkpoint names of the tensors an end part declares: ``weight`` (and ``norm.weight``, where the part has a
        norm) from the spec's own fields, anything else from the spec's ``names``."""
        spec = getattr(self.spec, which)
        part = getattr(self, which)
        given = dict(getattr(spec, "names", {}) or {})
        given.setdefault("weight", spec.name)
        if getattr(spec, "norm_name", None):
            given.setdefault("norm.weight", spec.norm_name)
        out = {}
        for local in part.declare():
            if local not in given:
                raise KeyError(f"{which}: its description gives no checkpoint name for tensor {local!r}")
            out[local] = given[local]
        return out

    def expected(self) -> dict[str, ParamDecl]:
        out = {}
        emb = self.embedding.declare()
        for local, name in self._end_names("embedding").items():
            out[name] = emb[local]
        for i, (layer, ls) in enumerate(zip(self.layers, self.spec.layers)):
            for local, decl in layer.declare().items():
                if local not in ls.names:
                    raise KeyError(f"layer {i}: its description gives no checkpoint name for tensor {local!r}")
                out[ls.names[local]] = decl
        hd = self.head.declare()
        for local, name in self._end_names("head").items():
            out[name] = hd[local]
        if self.spec.pass_rows:
            out[self.spec.pass_rows] = ParamDecl((self.spec.pass_rows_count, self.hidden), "vector")
        if self.spec.pass_mix:
            out[self.spec.pass_mix] = ParamDecl((self.hidden, 2 * self.hidden))
        return out

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.embedding.bind({local: tensors[name] for local, name in self._end_names("embedding").items() if name in tensors})
        for layer, ls in zip(self.layers, self.spec.layers):
            layer.bind({local: tensors[ls.names[local]] for local in layer.declare() if ls.names[local] in tensors})
        head = {local: tensors[name] for local, name in self._end_names("head").items() if name in tensors}
        self.head.bind(head, embedding_table=getattr(self.embedding, "table", None))
        if self.spec.pass_rows:
            self.pass_rows = tensors[self.spec.pass_rows].to(torch.float32).contiguous()
        if self.spec.pass_mix:
            from ..parts.linear import Linear
            self.pass_mix = Linear(tensors[self.spec.pass_mix], self.ctx.dtype)

    # ---- one step ----
    def forward(self, b, cache, ws, logits: torch.Tensor) -> torch.Tensor:
        """Run the tokens of batch ``b``; fill ``logits`` [len(b.rows), vocab] (float32)."""
        from ..kernels import ops
        b.stream = torch.cuda.current_stream().cuda_stream   # inside a graph capture this is the capture stream
        mark = ws.mark()
        x = ws.take((b.T, self.hidden), torch.float32)
        if self.embedding_entry is not None:
            self.embedding.forward(b, x, cache.view(self.embedding_entry, writes=True))
        else:
            self.embedding.forward(b, x)
        xs = None
        if self.spec.streams > 1:           # several copies of the stream: all start as the embedding's output
            from ..kernels import ops
            xs = ws.take((b.T, self.spec.streams * self.hidden), torch.float32)
            ops.streams_fill(x, xs, self.spec.streams, b.stream)
        x0 = None
        if self.keeps_embedding:        # some application adds the embedding's output again: keep a copy
            x0 = ws.take((b.T, self.hidden), torch.float32)
            x0.copy_(x)
        schedule = self.spec.schedule
        fused = self._fused_runs(b, cache)
        i = 0
        while i < len(schedule):
            if i in fused:
                i = self._run_fused(fused[i], x, b, ws)
                continue
            e = schedule[i]
            if e.mix_embedding:          # x <- W [x; x0]
                from ..kernels import ops
                m = ws.mark()
                both = ws.take((b.T, 2 * self.hidden), self.ctx.dtype)
                ops.stream_pair(x, x0, both, b.stream)
                self.pass_mix.forward(both, out=x, ws=ws, stream=b.stream)
                ws.release(m)
            if e.add_embedding or e.add_row >= 0:
                from ..kernels import ops
                ops.stream_inject(x, x0 if e.add_embedding else None,
                                  self.pass_rows[e.add_row] if e.add_row >= 0 else None, b.stream)
            view = cache.view(e.cache, writes=self.entry_owner[e.cache] == i)
            if e.borrow >= 0:               # the application also reads what an earlier one wrote
                view = dict(view) if isinstance(view, dict) else {"own": view}
                view["borrowed"] = cache.view(e.borrow, writes=False)
            following = self.layers[schedule[i + 1].layer] if i + 1 < len(schedule) and (i + 1) not in fused else None
            b.next_read = lead_weight_of(following)
            self.layers[e.layer].forward(x if xs is None else xs, b, view, ws)
            if self.observe is not None:
                if xs is not None:
                    ops.streams_sum(xs, x, b.stream)
                self.observe(i, x)
            i += 1
        b.next_read = None
        if xs is not None:                  # the copies' sum enters the final norm
            ops.streams_sum(xs, x, b.stream)
        if logits.shape[0]:
            self.head.forward(x, b, logits, ws)
        ws.release(mark)
        return logits

    # ---- single-token steps through the persistent kernel ----
    def _fused_runs(self, b, cache) -> dict:
        """{first schedule index: (index after the run, program)} for this step, or {} when it does not qualify: every
        sequence brings one token, at most FUSED_DECODE_ROWS of them, in bfloat16."""
        if (DECODE_CHOICE != "fused" or self.ctx.dtype != torch.bfloat16 or b.max_count != 1 or b.T != b.n
                or not 1 <= b.n <= FUSED_DECODE_ROWS):
            return {}
        runs = self._programs.get(id(cache))
        if runs is None:
            runs = self._programs[id(cache)] = self._prepare_runs(cache)
        return {start: (end, prog) for start, end, prog in runs if prog.slots_for(b.n)[0] >= FUSED_DECODE_MIN_SLOTS}

    def _prepare_runs(self, cache) -> list:
        """Maximal runs of consecutive layer applications whose layers offer ``fused_decode`` and own their cache entry."""
        from ..kernels import ops
        runs, cur = [], []
        schedule = self.spec.schedule

        def close():
            if cur:
                prog = ops.decode_program([s for _, s, _ in cur], [v for _, _, v in cur], cache.pools)
                if prog is not None:
                    runs.append((cur[0][0], cur[-1][0] + 1, prog))
                cur.clear()

        for i, e in enumerate(schedule):
            offer = getattr(self.layers[e.layer], "fused_decode", lambda: None)()
            view = cache.view(e.cache, writes=True) if offer is not None and self.entry_owner[e.cache] == i else None
            if offer is None or view is None or not hasattr(view, "k_pool"):
                close()
                continue
            if cur and (offer["mixer"]["head_dim"] != cur[0][1]["mixer"]["head_dim"]):
                close()
            cur.append((i, offer, view))
        close()
        return runs

    def _run_fused(self, run, x, b, ws) -> int:
        from ..kernels import ops
        end, prog = run
        mark = ws.mark()
        qkv = ws.take((b.n, prog.max_qkv), torch.bfloat16)
        y = ws.take((b.n, prog.max_heads), torch.bfloat16)
        act = ws.take((b.n, prog.max_inter), torch.bfloat16)
        parts = ws.take((ops.decode_layers_scratch_floats(prog, b.n, ops.sm_count(x.device)),), torch.float32)
        ops.decode_layers(prog, x, b.past, b.tables, qkv, y, act, parts, b.stream, trace=getattr(self, "decode_trace", None))
        ws.release(mark)
        return end

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for t in self._all_tensors():
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        return total

    def _all_tensors(self):
        """The tensors the parts hold: attributes that are tensors, or objects with a tensor ``weight`` (a product,
        a norm), looked for in the end parts and in each layer's ``children``."""
        parts = [self.embedding, self.head]
        for layer in self.layers:
            parts.append(layer)           # what the arrangement itself holds (a gate's matrix)
            parts.extend(getattr(layer, "children", {}).values())
        if self.pass_mix is not None:
            yield self.pass_mix.weight
        from ..parts.base import Part
        while parts:
            part = parts.pop()
            for v in vars(part).values():
                if isinstance(v, torch.Tensor):
                    yield v
                elif isinstance(getattr(v, "weight", None), torch.Tensor):
                    yield v.weight
                elif isinstance(v, Part) and not isinstance(v, type(part)):
                    parts.append(v)       # a part inside a part (a shared expert inside the routed experts)


def declare_model(spec: ModelSpec) -> dict[str, ParamDecl]:
    """The tensors a model description expects, found without a GPU."""
    ctx = BuildContext(device=torch.device("cpu"), dtype=torch.float32, max_positions=1)
    return Model(spec, ctx).expected()
