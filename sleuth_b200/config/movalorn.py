"""The Movalorn decoder: its typed configuration and its model description.

A Movalorn ``config.json`` names the design in ``architecture`` and nests its sizes::

    {"architecture": "Movalorn", "vocab": V, "width": d, "norm": {"eps": e}, "logit_scale": c,
     "embedding": {"scale": s, "bigram": {"buckets": n, "mul_prev": a, "mul_cur": b}},
     "layers": [{"type": "latent_attention",
                 "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot": {"base", "dims"}, "mask": {"size"}},
                 "mlp": null | {"kind": "dense", "ff"}
                             | {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "scale"}, "shared": {"ff"}}},
                {"type": "mingru", "mixer": {"width"}, "mlp": ...}, ...],
     "loop": {"start", "stop", "times"}}

The model: x0 = E[token] * s + B[(previous token * a + token * b) mod n] (B's last row for a sequence's first token;
``parts/ends.py``). A layer is a *sandwich* (``parts/layer.py``): with h = norm(x), x += norm'(m(h) * sigmoid(W h + b))
for the mixer m and then the same for the feed-forward; every norm is an RMS norm with ONE gain for all channels. Mixers:
attention through a low-rank latent (``parts/latent_attention.py``: queries straight from h, a sliding window, rotation
of neighbouring channel pairs on the rotated parts, one output gate value per head) or a minGRU
(``parts/recurrent.py``). Feed-forwards: a gated layer with the tanh form of GELU, or experts with SiLU chosen by
softmax score plus a correction, weighted by the uncorrected score times the router's scale, plus a shared expert
(``parts/ffn.py``, ``parts/moe.py``), or none. Layers ``loop.start .. loop.stop - 1`` run ``loop.times`` times in a row
with the same weights and caches and states of their own; every pass (the first too) starts with x <- W_in [x; x0] and
then adds its row of ``loop.step``. Final norm, untied output matrix, logits times ``logit_scale``.

Tensor names: ``embed``, ``bigram``, ``loop.in``, ``loop.step``, ``l<i>.norm1|norm1b|norm2|norm2b`` (no axes),
``l<i>.rg1|rg1.b|rg2|rg2.b``, ``l<i>.mix.<q|dkv|dkv.norm|uk|uv|g|o>`` or ``l<i>.mix.<z|z.b|x|x.b|g|o>``,
``l<i>.mlp.<gate|up|down>`` or ``l<i>.mlp.<router|correction|e<k>.gate|e<k>.up|e<k>.down|shared.gate|shared.up|shared.down>``,
``final.norm`` (no axes), ``head``.
"""

from __future__ import annotations

from dataclasses import dataclass

from ..parts.spec import (GatedMLPSpec, HeadSpec, LatentAttentionSpec, LayerSpec, MinGRUSpec, ModelSpec, NormSpec,
                          PairEmbeddingSpec, EmbeddingSpec, PositionSpec, RoutedExpertsSpec, looped_schedule,
                          straight_schedule)
from .base import ConfigError, read_fields


@dataclass(frozen=True)
class _Rot:
    base: float
    dims: int


@dataclass(frozen=True)
class _Mask:
    size: int


@dataclass(frozen=True)
class _Attention:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot: dict
    mask: dict | None = None


@dataclass(frozen=True)
class _MinGRU:
    width: int


@dataclass(frozen=True)
class _Dense:
    kind: str
    ff: int


@dataclass(frozen=True)
class _Moe:
    kind: str
    expert: dict
    router: dict
    shared: dict | None = None


@dataclass(frozen=True)
class _ExpertSizes:
    ff: int


@dataclass(frozen=True)
class _Router:
    experts: int
    top: int
    scale: float = 1.0


@dataclass(frozen=True)
class _Layer:
    type: str
    mixer: dict
    mlp: dict | None = None


@dataclass(frozen=True)
class _Loop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class _Norm:
    eps: float


@dataclass(frozen=True)
class _Bigram:
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class _Embedding:
    scale: float = 1.0
    bigram: dict | None = None


MIXERS = ("latent_attention", "mingru")


def _strict(cls, d, where):
    """``read_fields`` that also refuses keys the class does not name: a key that nobody reads is a part of the model
    that would silently be left out."""
    obj, unread = read_fields(cls, d, where)
    if unread:
        raise ConfigError(f"{where}: unknown key(s) {unread}")
    return obj


@dataclass(frozen=True)
class MovalornConfig:
    vocab: int
    width: int
    layers: tuple[dict, ...]
    norm: dict
    embedding: dict | None = None
    loop: dict | None = None
    logit_scale: float = 1.0
    architecture: str = "Movalorn"
    max_positions: int = 1 << 20        # the design sets no limit; tables are built for what the engine is asked to hold
    eos_token_id: int | tuple[int, ...] | None = None

    def __post_init__(self):
        def need(cond, msg):
            if not cond:
                raise ConfigError("config.json: " + msg)

        need(self.vocab > 0 and self.width > 0, f"vocab ({self.vocab}) and width ({self.width}) must be positive")
        need(len(self.layers) > 0, "layers is empty")
        object.__setattr__(self, "eps", _strict(_Norm, self.norm, "config.json: norm").eps)
        need(self.eps > 0, f"norm.eps must be positive, got {self.eps}")
        emb = _strict(_Embedding, self.embedding, "config.json: embedding") if self.embedding is not None else _Embedding()
        bg = _strict(_Bigram, emb.bigram, "config.json: embedding.bigram") if emb.bigram is not None else None
        if bg is not None:
            need(bg.buckets > 0 and bg.mul_prev >= 0 and bg.mul_cur >= 0,
                 f"embedding.bigram: buckets {bg.buckets}, multipliers {bg.mul_prev}, {bg.mul_cur}")
        object.__setattr__(self, "embedding_scale", emb.scale)
        object.__setattr__(self, "bigram", bg)
        parsed = []
        for i, raw in enumerate(self.layers):
            where = f"config.json: layers[{i}]"
            L = _strict(_Layer, raw, where)
            need(L.type in MIXERS, f"layers[{i}].type {L.type!r} is not a known mixer {list(MIXERS)}")
            if L.type == "latent_attention":
                m = _strict(_Attention, L.mixer, where + ".mixer")
                rot = _strict(_Rot, m.rot, where + ".mixer.rot")
                mask = _strict(_Mask, m.mask, where + ".mixer.mask") if m.mask is not None else None
                for key in ("heads", "dim", "vdim", "kv_rank"):
                    need(getattr(m, key) > 0, f"layers[{i}].mixer.{key} must be positive, got {getattr(m, key)}")
                need(m.rot_dim >= 0 and 0 <= rot.dims <= m.rot_dim and rot.dims % 2 == 0 and m.rot_dim % 2 == 0,
                     f"layers[{i}].mixer: rot.dims ({rot.dims}) must be even and at most rot_dim ({m.rot_dim}, even)")
                need(rot.base > 0 and m.scale > 0, f"layers[{i}].mixer: rot.base and scale must be positive")
                need(mask is None or mask.size > 0, f"layers[{i}].mixer.mask.size must be positive")
                mixer = (m, rot, mask)
            else:
                mixer = _strict(_MinGRU, L.mixer, where + ".mixer")
                need(mixer.width > 0, f"layers[{i}].mixer.width must be positive, got {mixer.width}")
            f = None
            if L.mlp is not None:
                kind = L.mlp.get("kind") if isinstance(L.mlp, dict) else None
                if kind == "dense":
                    f = _strict(_Dense, L.mlp, where + ".mlp")
                    need(f.ff > 0, f"layers[{i}].mlp.ff must be positive")
                elif kind == "moe":
                    moe = _strict(_Moe, L.mlp, where + ".mlp")
                    ex = _strict(_ExpertSizes, moe.expert, where + ".mlp.expert")
                    ro = _strict(_Router, moe.router, where + ".mlp.router")
                    sh = _strict(_ExpertSizes, moe.shared, where + ".mlp.shared") if moe.shared is not None else None
                    need(ex.ff > 0 and 0 < ro.top <= ro.experts and (sh is None or sh.ff > 0),
                         f"layers[{i}].mlp: expert.ff {ex.ff}, router.experts {ro.experts}, router.top {ro.top}")
                    f = (ex, ro, sh)
                else:
                    raise ConfigError(f"{where}.mlp.kind {kind!r} is not 'dense' or 'moe'")
            parsed.append((L.type, mixer, f))
        object.__setattr__(self, "parsed_layers", tuple(parsed))
        lp = _strict(_Loop, self.loop, "config.json: loop") if self.loop is not None else None
        if lp is not None:
            need(0 <= lp.start <= lp.stop <= len(self.layers) and lp.times >= 1,
                 f"loop {self.loop} does not fit {len(self.layers)} layers")
        object.__setattr__(self, "parsed_loop", lp)

    @property
    def stop_ids(self) -> tuple[int, ...]:
        if self.eos_token_id is None:
            return ()
        return (self.eos_token_id,) if isinstance(self.eos_token_id, int) else tuple(self.eos_token_id)


def movalorn_model_spec(cfg: MovalornConfig, tensor_names=None) -> ModelSpec:
    d, eps = cfg.width, cfg.eps

    def one_gain():
        return NormSpec(d, eps, gain="scalar")

    layers = []
    for i, (kind, m, f) in enumerate(cfg.parsed_layers):
        p = f"l{i}."
        names = {"norm1.weight": p + "norm1", "post1.weight": p + "norm1b", "gate1.weight": p + "rg1", "gate1.bias": p + "rg1.b"}
        if kind == "latent_attention":
            m, rot, mask = m
            for local, theirs in (("q.weight", "q"), ("dkv.weight", "dkv"), ("dkv_norm.weight", "dkv.norm"),
                                  ("uk.weight", "uk"), ("uv.weight", "uv"), ("g.weight", "g"), ("o.weight", "o")):
                names["mixer." + local] = p + "mix." + theirs
            mixer = LatentAttentionSpec(
                hidden=d, heads=m.heads, plain_dim=m.dim, rot_dim=m.rot_dim, value_dim=m.vdim, q_rank=0, kv_rank=m.kv_rank,
                scale=m.scale, norm_eps=eps, window=mask.size if mask is not None else 0, gate_span="head",
                position=PositionSpec(head_dim=m.rot_dim, theta=rot.base, rotary_dim=rot.dims, pairing="neighbours",
                                      precise=True, kind="rotary" if rot.dims else "none"))
        else:
            for local, theirs in (("z.weight", "z"), ("z.bias", "z.b"), ("x.weight", "x"), ("x.bias", "x.b"),
                                  ("g.weight", "g"), ("o.weight", "o")):
                names["mixer." + local] = p + "mix." + theirs
            mixer = MinGRUSpec(hidden=d, width=m.width)
        if f is None:
            ffn = None
        else:
            names.update({"norm2.weight": p + "norm2", "post2.weight": p + "norm2b", "gate2.weight": p + "rg2",
                          "gate2.bias": p + "rg2.b"})
            if isinstance(f, _Dense):
                ffn = GatedMLPSpec(hidden=d, intermediate=f.ff, activation="gelu_tanh")
                for local in ("gate", "up", "down"):
                    names[f"ffn.{local}.weight"] = p + "mlp." + local
            else:
                ex, ro, sh = f
                shared = GatedMLPSpec(hidden=d, intermediate=sh.ff, activation="silu") if sh is not None else None
                ffn = RoutedExpertsSpec(hidden=d, intermediate=ex.ff, experts=ro.experts, top=ro.top, activation="silu",
                                        router_bias=False, scoring="softmax", route_scale=ro.scale, shared=shared,
                                        choice_bias=True)
                names["ffn.router.weight"] = p + "mlp.router"
                names["ffn.correction"] = p + "mlp.correction"
                for e in range(ro.experts):
                    for local in ("gate", "up", "down"):
                        names[f"ffn.e{e}.{local}.weight"] = p + f"mlp.e{e}.{local}"
                if sh is not None:
                    for local in ("gate", "up", "down"):
                        names[f"ffn.shared.{local}.weight"] = p + f"mlp.shared.{local}"
        layers.append(LayerSpec(mixer=mixer, ffn=ffn, norm1=one_gain(), norm2=one_gain() if ffn is not None else None,
                                post1=one_gain(), post2=one_gain() if ffn is not None else None, gated=True, names=names,
                                kind="sandwich"))
    lp = cfg.parsed_loop
    if lp is not None and lp.stop > lp.start:
        schedule = looped_schedule(len(layers), lp.start, lp.stop, lp.times, entry="mix")
        pass_rows, rows, pass_mix, ignored = "loop.step", lp.times, "loop.in", ()
    else:
        schedule, pass_rows, rows, pass_mix = straight_schedule(len(layers)), None, 0, None
        ignored = (r"loop\.step$", r"loop\.in$")
    bg = cfg.bigram
    if bg is not None:
        embedding = PairEmbeddingSpec(vocab=cfg.vocab, dim=d, buckets=bg.buckets, mul_prev=bg.mul_prev, mul_cur=bg.mul_cur,
                                      scale=cfg.embedding_scale, names={"weight": "embed", "pairs": "bigram"})
    else:
        embedding = EmbeddingSpec(vocab=cfg.vocab, dim=d, scale=cfg.embedding_scale, name="embed")
    return ModelSpec(
        embedding=embedding, layers=tuple(layers), schedule=schedule,
        head=HeadSpec(vocab=cfg.vocab, dim=d, norm=one_gain(), tied=False, norm_name="final.norm", name="head",
                      scale=cfg.logit_scale),
        max_positions=cfg.max_positions, pass_rows=pass_rows, pass_rows_count=rows, pass_mix=pass_mix,
        ignored_tensors=ignored)
