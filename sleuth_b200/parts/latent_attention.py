"""Causal attention through low-rank latents over the paged latent cache, as a mixer part.

With h the layer's normed input:

* queries: c_q = RMSNorm(W_dq h) (gain ``dq_norm``), q = W_uq c_q, laid out head by head as ``plain_dim``
  unrotated values followed by ``rot_dim`` rotated ones;
* keys and values: W_dkv h has ``kv_rank + rot_dim`` rows; the first ``kv_rank``, RMS-normed (gain ``dkv_norm``),
  are the token's latent c, the rest (not normed) is one rotated key part that all heads share. Head n's
  unrotated key is W_uk[n] c and its value W_uv[n] c;
* score = (q_plain . k_plain + q_rot . k_rot) * scale, causal softmax, the heads' outputs side by side, times
  sigmoid(W_g h), then W_o, added into the stream.

The cache keeps c and the rotated key part only (``LatentRequest``), and the per-head keys and values are never
formed: the key up-projection is applied to the query instead (q_lat[n] = W_uk[n]^T q_plain[n], so that
q_plain . (W_uk c) = q_lat . c), the softmax-weighted sum runs over the latents, and the value up-projection is
applied to that sum (value[n] = W_uv[n] sum_j p_j c_j). One kernel then serves prompts, single tokens and chunks
alike, and a token costs ``kv_rank + rot_dim`` cache values per layer whatever the number of heads.

A bfloat16 step in which every sequence starts at position 0 (whole prompts of 64 tokens and more) takes another
way to the same result: its keys are its own tokens, so one product forms every head's unrotated keys and values
from the step's latents and ``head_prompt_attention`` runs ordinary per-head attention, which multiplies
``plain_dim + rot_dim + value_dim`` values per head and pair of tokens instead of ``2 * kv_rank + rot_dim``. The cache
is written the same way, and later portions and single tokens read it through the latent form.

Options of the spec: ``q_rank`` 0 (the queries are W_q h, no query latent); ``window`` (a query sees the ``window`` most
recent tokens, its own included); ``gate_span="head"`` (W_g gives one gate value per head; its rows then ride in the
stacked down-projection and the gate is read from that product's float32 result); a position part that pairs
neighbouring channels (2i with 2i + 1): the rows of the query and key projections that produce the rotated parts are
reordered once at load time so that pair i sits at channels i and i + rot/2, which the kernels turn; a dot product
does not care about the order of its channels as long as query and key agree.

Launches of a step (latent form): the stacked down-projections (float32 result), the gate projection, ``latent_post`` (both
norms, the key part's rotation, the cache write), the query up-projection, the per-head carry into the latent
space (a batched library product), ``latent_attention`` (which turns the queries' rotated part as it loads them),
the per-head value up-projection (batched library product), ``latent_gate``, the output projection.
"""

from __future__ import annotations

import torch

from ..cache.paged import LatentRequest
from ..kernels import ops
from .base import BuildContext, Normed, ParamDecl, Part, build_position, register_mixer, result_target
from .linear import Linear
from .spec import LatentAttentionSpec


# From this many tokens of its longest sequence on, a bfloat16 step in which every sequence starts at position 0 (whole
# prompts) forms each head's keys and values from its own tokens' latents and runs ordinary per-head attention: that
# multiplies plain_dim + rot_dim + value_dim values per head and token pair instead of 2 * kv_rank + rot_dim.
PER_HEAD_PROMPT_TOKENS = 64


class LatentAttention(Part):
    stores_result = True
    accepts_rider = True        # a layer's own rows ride at the end of the stacked down-projection

    def __init__(self, spec: LatentAttentionSpec, ctx: BuildContext):
        if spec.rot_dim % 2:
            raise ValueError(f"rot_dim {spec.rot_dim} must be even")
        if spec.gate_span not in ("channel", "head"):
            raise ValueError(f"latent_attention: gate_span {spec.gate_span!r} is not 'channel' or 'head'")
        if spec.q_rank < 0 or spec.window < 0:
            raise ValueError(f"latent_attention: q_rank {spec.q_rank}, window {spec.window}")
        self.spec, self.ctx = spec, ctx
        self.head_gate = spec.output_gate and spec.gate_span == "head"
        self.position = build_position(spec.position, ctx)
        self.down = self.gate = self.uq = self.o = None
        self.w_uk = self.w_uv_t = self.q_gain = self.c_gain = None

    def declare(self):
        s = self.spec
        if s.q_rank:
            d = {"dq.weight": ParamDecl((s.q_rank, s.hidden)),
                 "dq_norm.weight": ParamDecl((s.q_rank,), "vector", init="gain"),
                 "uq.weight": ParamDecl((s.heads * (s.plain_dim + s.rot_dim), s.q_rank))}
        else:
            d = {"q.weight": ParamDecl((s.heads * (s.plain_dim + s.rot_dim), s.hidden))}
        d.update({
             "dkv.weight": ParamDecl((s.kv_rank + s.rot_dim, s.hidden)),
             "dkv_norm.weight": ParamDecl((s.kv_rank,), "vector", init="gain"),
             "uk.weight": ParamDecl((s.heads * s.plain_dim, s.kv_rank)),
             "uv.weight": ParamDecl((s.heads * s.value_dim, s.kv_rank)),
             "o.weight": ParamDecl((s.hidden, s.heads * s.value_dim))})
        if s.output_gate:
            d["g.weight"] = ParamDecl((s.heads if self.head_gate else s.heads * s.value_dim, s.hidden))
        return d

    def _paired_halves(self, w: torch.Tensor, first: int, step: int, count: int) -> torch.Tensor:
        """``w`` with the rows that produce rotated channels reordered from neighbouring pairs (2i, 2i + 1) to halves
        (i, i + rot/2): ``count`` runs of rotated channels, the first starting at row ``first``, ``step`` rows apart."""
        rot = self.position.rot_dim
        if not getattr(self.position, "neighbours", False) or rot < 4:
            return w
        order = torch.cat([torch.arange(0, rot, 2), torch.arange(1, rot, 2)]).to(w.device)
        rows = torch.arange(w.shape[0], device=w.device)
        for k in range(count):
            at = first + k * step
            rows[at:at + rot] = at + order
        return w[rows]

    def bind(self, t):
        s, dt = self.spec, self.ctx.dtype
        dn, P = s.plain_dim, s.rot_dim
        stack = ([t["dq.weight"]] if s.q_rank else []) + [self._paired_halves(t["dkv.weight"], s.kv_rank, 0, 1)]
        if self.head_gate:
            stack.append(t["g.weight"])         # a gate value per head: its few rows ride in the stacked product
        self.rider_rows = 0
        if t.get("rider.weight") is not None:
            stack.append(t["rider.weight"])
            self.rider_rows = t["rider.weight"].shape[0]
        self.down = Linear(torch.cat(stack, dim=0) if len(stack) > 1 else stack[0], dt)     # one product, float32 result
        self.gate = Linear(t["g.weight"], dt) if s.output_gate and not self.head_gate else None
        self.uq = Linear(self._paired_halves(t["uq.weight" if s.q_rank else "q.weight"], dn, dn + P, s.heads), dt)
        self.o = Linear(t["o.weight"], dt)
        self.ukv = Linear(torch.cat([t["uk.weight"], t["uv.weight"]], dim=0), dt)      # whole prompts: keys and values per head
        self.w_uk = t["uk.weight"].to(dt).view(s.heads, s.plain_dim, s.kv_rank).contiguous()
        self.w_uv_t = t["uv.weight"].to(dt).view(s.heads, s.value_dim, s.kv_rank).transpose(1, 2)   # [H, rank, value]
        self.q_gain, self.c_gain = t.get("dq_norm.weight"), t["dkv_norm.weight"]

    def cache_request(self):
        s = self.spec
        return LatentRequest(s.kv_rank + s.rot_dim, s.window)

    def lead_weight(self):
        return self.down.weight if self.down is not None else None

    def forward(self, h, x, b, view, ws):
        s, dt = self.spec, self.ctx.dtype
        if isinstance(h, Normed):
            h = h.tensor()
        T, H, R, P, dn, dv = h.shape[0], s.heads, s.kv_rank, s.rot_dim, s.plain_dim, s.value_dim
        table = b.tables[view.group]
        tables = self.position.tables()
        cos, sin = tables if tables is not None else (None, None)
        rotated = self.position.rot_dim
        mark = ws.mark()
        lat = self.down.forward(h, ws=ws, stream=b.stream, out_dtype=torch.float32)
        g = self.gate.forward(h, ws=ws, stream=b.stream) if self.gate is not None else None
        cq = ws.take((T, s.q_rank), dt) if s.q_rank else None
        if self.head_gate:
            g = lat[:, s.q_rank + R + P:s.q_rank + R + P + H]
        if self.rider_rows:
            b.rider = lat[:, lat.shape[1] - self.rider_rows:]
        per_head = (getattr(b, "fresh", False) and b.max_count >= PER_HEAD_PROMPT_TOKENS
                    and ops.head_prompt_supported(dn, P, dv, dt))
        c_out = ws.take((T, R), dt) if per_head else None
        k_out = ws.take((T, P), dt) if per_head else None
        ops.latent_post(lat, self.q_gain, self.c_gain, cos, sin, cq, view.pool if view.writes else None, b.tok_seq,
                        b.tok_pos, table, s.q_rank, R, P, rotated, s.norm_eps, b.stream, c_out, k_out, dtype=dt)
        q = self.uq.forward(cq if s.q_rank else h, ws=ws, stream=b.stream).view(T, H, dn + P)
        if per_head:
            kv = self.ukv.forward(c_out, ws=ws, stream=b.stream)
            val = ws.take((H, T, dv), dt)
            ops.head_prompt_attention(q, kv, k_out, val, cos, sin, b.seq_start, b.counts, b.max_count, H, dn, P, dv, rotated,
                                      view.window, s.scale, b.stream)
            self._gate_and_project(val, g, x, b, ws, T, H, dv, dt)
            ws.release(mark)
            return
        q_lat = ws.take((H, T, R), dt)
        torch.bmm(q[:, :, :dn].transpose(0, 1), self.w_uk, out=q_lat)
        o_lat = ws.take((H, T, R), dt)
        # the number of key slices follows the batch and the longest sequence allowed, never the lengths of the
        # moment: a recorded step stays valid as its sequences grow
        splits = ops.latent_splits(b.n, H, b.max_count, table.shape[1] * 64)
        floats = ops.latent_scratch_floats(T, H, R, splits)
        scratch = ws.take((floats,), torch.float32) if floats else None
        ops.latent_attention(q_lat, q, view.pool, o_lat, cos, sin, b.seq_start, b.past, b.counts, table, b.max_count,
                             H, R, P, dn, rotated, view.window, s.scale, splits, scratch, b.stream)
        val = ws.take((H, T, dv), dt)
        torch.bmm(o_lat, self.w_uv_t, out=val)
        self._gate_and_project(val, g, x, b, ws, T, H, dv, dt)
        ws.release(mark)

    def _gate_and_project(self, val, g, x, b, ws, T, H, dv, dt):
        y = ws.take((T, H * dv), dt)
        if g is not None and self.head_gate:
            ops.latent_head_gate(val, g, y, b.stream)
        elif g is not None:
            ops.latent_gate(val, g, y, b.stream)
        else:
            y.view(T, H, dv).copy_(val.transpose(0, 1))
        self.o.forward(y, ws=ws, stream=b.stream, next_read=getattr(b, "next_read", None), **result_target(b, x))


register_mixer("latent_attention", LatentAttention)
