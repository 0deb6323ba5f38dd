"""The two ends of the model: token embedding and the output head."""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import BuildContext, ParamDecl, Part, build_norm, register_embedding, register_head
from .linear import Linear
from ..cache.paged import StateRequest
from .spec import EmbeddingSpec, HeadSpec, PairEmbeddingSpec


class TokenEmbedding(Part):
    """x[t] = table[ids[t]] * scale into the float32 stream (sleuth/forge/model/transformer.py:345-348); with
    ``spec.norm`` the rows are then normalised in place, in float32."""

    def __init__(self, spec: EmbeddingSpec, ctx: BuildContext):
        self.spec, self.ctx = spec, ctx
        self.table = None
        self.norm = build_norm(spec.norm, ctx) if spec.norm is not None else None

    def declare(self):
        d = {"weight": ParamDecl((self.spec.vocab, self.spec.dim))}
        if self.norm is not None:
            d["norm.weight"] = self.norm.declare()["weight"]
        return d

    def bind(self, t):
        self.table = t["weight"]
        if self.norm is not None:
            self.norm.bind({"weight": t["norm.weight"]})

    def forward(self, b, x):
        """``b``: the step's batch; its token ids sit in ``b.token_ids`` (read through ``b.ids_map`` in a step that
        takes its tokens from the device-side feed)."""
        ops.embed(b.token_ids, self.table, x, self.spec.scale, b.stream, b.ids_map)
        if self.norm is not None:
            self.norm.forward(x, x, stream=b.stream)


class PairEmbedding(Part):
    """x[t] = table[ids[t]] * scale + pairs[(previous token * mul_prev + token * mul_cur) mod buckets]; a sequence's
    first token takes the pair table's last row. The previous token of a step's first token is per-sequence state
    (one int32 per slot, asked for through ``cache_request`` like a mixer's state), so a prompt may arrive in
    portions and single-token steps find it without the host."""

    def __init__(self, spec: PairEmbeddingSpec, ctx: BuildContext):
        if spec.buckets < 1 or spec.mul_prev < 0 or spec.mul_cur < 0:
            raise ValueError(f"pair_embedding: buckets {spec.buckets}, multipliers {spec.mul_prev}, {spec.mul_cur}")
        self.spec, self.ctx = spec, ctx
        self.table = self.pairs = None

    def declare(self):
        s = self.spec
        return {"weight": ParamDecl((s.vocab, s.dim)), "pairs": ParamDecl((s.buckets + 1, s.dim))}

    def bind(self, t):
        self.table, self.pairs = t["weight"], t["pairs"]

    def cache_request(self):
        return StateRequest((1,), torch.int32)

    def forward(self, b, x, view):
        s = self.spec
        together = self.table.dtype == self.pairs.dtype        # one pass forms the sum of the two rows
        if not together:
            ops.embed(b.token_ids, self.table, x, s.scale, b.stream, b.ids_map)
        ops.pair_embed(b.token_ids, b.ids_map, self.pairs, x, b.tok_seq, b.tok_pos, b.seq_start, b.slots, view.state,
                       s.vocab, s.buckets, s.mul_prev, s.mul_cur, b.stream, self.table if together else None, s.scale)


class LMHead(Part):
    """Final norm on the chosen rows, then logits = h @ W^T in float32
    (sleuth/forge/model/transformer.py:301-302). A tied head uses the embedding table (:129-130). With
    ``spec.softcap`` = c the logits become c * tanh(logits / c); with ``spec.scale`` they are multiplied by it first."""

    def __init__(self, spec: HeadSpec, ctx: BuildContext):
        self.spec, self.ctx = spec, ctx
        self.norm = build_norm(spec.norm, ctx)
        self.proj = None

    def declare(self):
        d = {"norm.weight": self.norm.declare()["weight"]}
        if not self.spec.tied:
            d["weight"] = ParamDecl((self.spec.vocab, self.spec.dim))
        return d

    def bind(self, t, embedding_table: torch.Tensor | None = None):
        self.norm.bind({"weight": t["norm.weight"]})
        w = embedding_table if self.spec.tied else t["weight"]
        self.proj = Linear(w, self.ctx.dtype)

    def forward(self, x, b, logits, ws):
        """logits[r] = head(x[b.rows[r]]); ``logits`` is float32 [len(b.rows), vocab]."""
        mark = ws.mark()
        h = ws.take((logits.shape[0], self.spec.dim), self.ctx.dtype)
        self.norm.forward(x, h, b.rows, b.stream)
        self.proj.forward(h, out=logits, stream=b.stream)
        if self.spec.scale != 1.0:
            ops.scale(logits, self.spec.scale, b.stream)
        if self.spec.softcap > 0:
            ops.softcap(logits, self.spec.softcap, b.stream)
        ws.release(mark)


register_embedding("token_embedding", TokenEmbedding)
register_embedding("pair_embedding", PairEmbedding)
register_head("lm_head", LMHead)
