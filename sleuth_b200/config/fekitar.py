"""The Fekitar decoder: its typed configuration and its model description.

A Fekitar ``config.json`` names the design in ``architecture`` and nests its sizes::

    {"architecture": "Fekitar", "vocab": V, "width": d, "norm": {"eps": e}, "residual_mult": m, "streams": S,
     "layers": [{"type": "parallel",
                 "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "conv": taps, "mask": {"size"}},
                           "right": {"heads", "vdim", "state", "groups", "conv": taps, "norm_groups"}},
                 "mlp": null | {"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top"},
                                "shared": {"ff", "limit"}}},
                {"type": "parallel_2",
                 "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "softcap",
                                    "rot": {"base", "dims", "scaling": {"factor", "low", "high", "original"}}},
                           "right": {"heads", "dim", "vdim", "tau", "rank"?}, "left_scale", "right_scale"}, "mlp": ...},
                {"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "diff", "conv": taps, "rot": {"base", "dims"},
                           "kv_from": j}, "mlp": ...}]}

The model (``parts/layer.py`` ``HyperLayer``): ``streams`` copies of the stream, all equal to the embedding's row at the
start; sublayer q of a layer reads u = sum_s in_q[s] x_s, y = sublayer(RMSNorm_q(u)), and every copy becomes
x_r <- sum_s mix_q[s, r] x_s + m * out_q[r] * y; the copies' sum enters the final norm and the untied output matrix.
Mixers: ``parallel`` = a windowed attention (short convolutions on q, k and v, per-head norms, no rotation, a distance
penalty 2^(-8 (h + 1) / H) (i - j)) beside a Mamba-2 recurrence, each result RMS-normed over the width with its gain, half
their sum; ``parallel_2`` = an attention with rotated halves (frequencies rescaled band by band), soft-capped scores and
a sigmoid gate per channel beside a gated linear attention, joined with two scales; ``attention`` = differential
attention with head gates, which with ``kv_from`` reads layer j's keys and values instead of forming its own
(``parts/scored_attention.py``, ``parts/recurrent.py``, ``parts/side_by_side.py``). Feed-forward: clamped-swish experts
(alpha 1.702) chosen by softmax score over all experts, weights divided by their sum, plus a shared expert times
sigmoid(w . h) (``parts/moe.py``).

Tensor names: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.hc1|hc2.in|out|mix``, ``l<i>.mix.left.<q|k|v|o|g|q.norm|k.norm|
q.conv|k.conv|v.conv>``, ``l<i>.mix.right.<in|conv|conv.b|dt_bias|A_log|D|norm|o>`` or ``l<i>.mix.right.<q|k|v|g|o|norm|
a1|a2|a2.b>``, ``l<i>.mix.left.out|right.out``, ``l<i>.mix.<q|k|v|g|o|q.conv|k.conv|v.conv|lq1|lk1|lq2|lk2>``,
``l<i>.mlp.<router|e<k>.gate|e<k>.up|e<k>.down|shared.gate|shared.up|shared.down|shared.sg>``, ``final.norm``, ``head``.
"""

from __future__ import annotations

from dataclasses import dataclass

from ..parts.spec import (EmbeddingSpec, GatedLinearAttentionSpec, GatedMLPSpec, HeadSpec, LayerSpec, ModelSpec, NormSpec,
                          PositionSpec, RoutedExpertsSpec, ScheduleEntry, ScoredAttentionSpec, SideBySideSpec, StateSpaceSpec)
from .base import ConfigError, read_fields

SWISH_ALPHA = 1.702         # the experts' activation: g' sigmoid(1.702 g') (u' + 1)
SLOPE_EXPONENT = 8.0        # the distance penalty of head h: 2^(-8 (h + 1) / heads)


@dataclass(frozen=True)
class _Scaling:
    factor: float
    low: float
    high: float
    original: float


@dataclass(frozen=True)
class _Rot:
    base: float
    dims: int
    scaling: dict | None = None


@dataclass(frozen=True)
class _Mask:
    size: int


@dataclass(frozen=True)
class _Attention:
    """The keys an attention of any of the three mixers may carry."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv: int = 0
    mask: dict | None = None
    rot: dict | None = None
    softcap: float = 0.0
    diff: float | None = None
    kv_from: int | None = None


@dataclass(frozen=True)
class _Mamba:
    heads: int
    vdim: int
    state: int
    groups: int = 1
    conv: int = 1
    norm_groups: int = 1


@dataclass(frozen=True)
class _Linear:
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: int = 0           # rows of the decay's first matrix; a model file's own shape comes first


@dataclass(frozen=True)
class _Pair:
    left: dict
    right: dict
    left_scale: float = 1.0
    right_scale: float = 1.0


@dataclass(frozen=True)
class _Expert:
    ff: int
    limit: float


@dataclass(frozen=True)
class _Router:
    experts: int
    top: int


@dataclass(frozen=True)
class _Moe:
    kind: str
    expert: dict
    router: dict
    shared: dict | None = None


@dataclass(frozen=True)
class _Layer:
    type: str
    mixer: dict
    mlp: dict | None = None


@dataclass(frozen=True)
class _Norm:
    eps: float


MIXERS = ("parallel", "parallel_2", "attention")


def _strict(cls, d, where):
    obj, unread = read_fields(cls, d, where)
    if unread:
        raise ConfigError(f"{where}: unknown key(s) {unread}")
    return obj


@dataclass(frozen=True)
class FekitarConfig:
    vocab: int
    width: int
    layers: tuple[dict, ...]
    norm: dict
    residual_mult: float = 1.0
    streams: int = 0
    architecture: str = "Fekitar"
    max_positions: int = 1 << 20        # the design sets no limit; tables are built for what the engine is asked to hold
    eos_token_id: int | tuple[int, ...] | None = None

    def __post_init__(self):
        def need(cond, msg):
            if not cond:
                raise ConfigError("config.json: " + msg)

        need(self.vocab > 0 and self.width > 0, f"vocab ({self.vocab}) and width ({self.width}) must be positive")
        need(len(self.layers) > 0, "layers is empty")
        need(0 <= self.streams <= 16, f"streams must lie in 0..16, got {self.streams}")
        object.__setattr__(self, "eps", _strict(_Norm, self.norm, "config.json: norm").eps)
        need(self.eps > 0, f"norm.eps must be positive, got {self.eps}")
        parsed = []
        for i, raw in enumerate(self.layers):
            where = f"config.json: layers[{i}]"
            L = _strict(_Layer, raw, where)
            need(L.type in MIXERS, f"layers[{i}].type {L.type!r} is not a known mixer {list(MIXERS)}")

            def attention(d, w):
                a = _strict(_Attention, d, w)
                rot = _strict(_Rot, a.rot, w + ".rot") if a.rot is not None else None
                sc = _strict(_Scaling, rot.scaling, w + ".rot.scaling") if rot is not None and rot.scaling is not None else None
                mask = _strict(_Mask, a.mask, w + ".mask") if a.mask is not None else None
                need(a.heads > 0 and a.kv_heads > 0 and a.heads % a.kv_heads == 0, f"{w}: heads {a.heads}, kv_heads {a.kv_heads}")
                need(a.dim > 0 and a.dim % 2 == 0 and a.vdim > 0 and a.scale > 0, f"{w}: dim {a.dim} (even), vdim {a.vdim}, scale {a.scale}")
                need(rot is None or (0 <= rot.dims <= a.dim and rot.dims % 2 == 0 and rot.base > 0), f"{w}.rot: dims and base")
                need(mask is None or mask.size > 0, f"{w}.mask.size must be positive")
                need(a.conv >= 0 and a.softcap >= 0, f"{w}: conv {a.conv}, softcap {a.softcap}")
                return a, rot, sc, mask

            if L.type == "attention":
                a = attention(L.mixer, where + ".mixer")
                need(a[0].diff is not None and 0 <= a[0].diff < 1, f"layers[{i}].mixer.diff must lie in [0, 1)")
                j = a[0].kv_from
                if j is not None:
                    need(0 <= j < i and parsed[j][0] == "attention" and parsed[j][1][0].kv_from is None,
                         f"layers[{i}].mixer.kv_from {j} must name an earlier attention layer with keys and values of its own")
                    o = parsed[j][1][0]
                    need((o.kv_heads, o.dim, o.vdim) == (a[0].kv_heads, a[0].dim, a[0].vdim),
                         f"layers[{i}].mixer: its key/value heads and widths differ from layer {j}'s")
                mixer = a
            else:
                pair = _strict(_Pair, L.mixer, where + ".mixer")
                left = attention(pair.left, where + ".mixer.left")
                need(left[0].diff is None and left[0].kv_from is None, f"layers[{i}].mixer.left: diff and kv_from belong to 'attention'")
                if L.type == "parallel":
                    right = _strict(_Mamba, pair.right, where + ".mixer.right")
                    need(right.heads > 0 and right.vdim > 0 and 0 < right.state <= 256 and right.groups > 0 and right.heads % right.groups == 0
                         and right.conv >= 1 and right.norm_groups > 0 and (right.heads * right.vdim) % right.norm_groups == 0,
                         f"layers[{i}].mixer.right: {pair.right}")
                else:
                    right = _strict(_Linear, pair.right, where + ".mixer.right")
                    need(right.heads > 0 and 0 < right.dim <= 256 and right.vdim > 0 and right.tau > 0, f"layers[{i}].mixer.right: {pair.right}")
                mixer = (pair, left, right)
            f = None
            if L.mlp is not None:
                moe = _strict(_Moe, L.mlp, where + ".mlp")
                need(moe.kind == "moe", f"layers[{i}].mlp.kind {moe.kind!r} is not 'moe'")
                ex = _strict(_Expert, moe.expert, where + ".mlp.expert")
                ro = _strict(_Router, moe.router, where + ".mlp.router")
                sh = _strict(_Expert, moe.shared, where + ".mlp.shared") if moe.shared is not None else None
                need(ex.ff > 0 and ex.limit > 0 and 0 < ro.top <= ro.experts and (sh is None or (sh.ff > 0 and sh.limit > 0)),
                     f"layers[{i}].mlp: {L.mlp}")
                f = (ex, ro, sh)
            parsed.append((L.type, mixer, f))
        object.__setattr__(self, "parsed_layers", tuple(parsed))

    @property
    def stop_ids(self) -> tuple[int, ...]:
        if self.eos_token_id is None:
            return ()
        return (self.eos_token_id,) if isinstance(self.eos_token_id, int) else tuple(self.eos_token_id)


def _attention_spec(d, eps, a, rot, sc, mask, names, p, local, **more):
    """The ``ScoredAttentionSpec`` of one parsed attention and the checkpoint names of its tensors (``p``: their prefix in the
    files, ``local``: the part's prefix inside the layer)."""
    shared = a.kv_from is not None
    for n in ("q", "o") + (() if shared else ("k", "v")):
        names[f"{local}{n}.weight"] = f"{p}{n}"
    if a.conv:
        for n in ("q",) + (() if shared else ("k", "v")):
            names[f"{local}{n}.conv"] = f"{p}{n}.conv"
    position = PositionSpec(head_dim=a.dim, kind="none")
    if rot is not None and rot.dims:
        position = PositionSpec(head_dim=a.dim, theta=rot.base, rotary_dim=rot.dims, precise=True,
                                scaling=(sc.factor, sc.low, sc.high, sc.original) if sc is not None else ())
    return ScoredAttentionSpec(hidden=d, heads=a.heads, kv_heads=a.kv_heads, head_dim=a.dim, value_dim=a.vdim, position=position,
                               scale=a.scale, eps=eps, conv_taps=a.conv, softcap=a.softcap, window=mask.size if mask is not None else 0,
                               reads_shared_kv=shared, **more)


def fekitar_model_spec(cfg: FekitarConfig, tensor_names=None) -> ModelSpec:
    d, eps = cfg.width, cfg.eps
    layers, schedule = [], []
    for i, (kind, m, f) in enumerate(cfg.parsed_layers):
        p = f"l{i}."
        names = {"norm1.weight": p + "norm1"}
        borrow = -1
        if kind == "attention":
            a, rot, sc, mask = m
            mixer = _attention_spec(d, eps, a, rot, sc, mask, names, p + "mix.", "mixer.", maps=2, diff=a.diff, gate="head")
            names["mixer.g.weight"] = p + "mix.g"
            for n in ("lq1", "lk1", "lq2", "lk2"):
                names["mixer." + n] = p + "mix." + n
            if a.kv_from is not None:
                borrow = a.kv_from
        else:
            pair, (a, rot, sc, mask), right = m
            lp, rp = p + "mix.left.", p + "mix.right."
            if kind == "parallel":
                left = _attention_spec(d, eps, a, rot, sc, mask, names, lp, "mixer.left.", qk_norm=True, slope_exponent=SLOPE_EXPONENT)
                names["mixer.left.q_norm.weight"], names["mixer.left.k_norm.weight"] = lp + "q.norm", lp + "k.norm"
                rspec = StateSpaceSpec(hidden=d, heads=right.heads, value_dim=right.vdim, state=right.state, groups=right.groups,
                                       conv_taps=right.conv, norm_groups=right.norm_groups, eps=eps)
                for local, theirs in (("in.weight", "in"), ("conv.weight", "conv"), ("conv.bias", "conv.b"), ("dt_bias", "dt_bias"),
                                      ("A_log", "A_log"), ("D", "D"), ("norm.weight", "norm"), ("o.weight", "o")):
                    names["mixer.right." + local] = rp + theirs
                names["mixer.left_out"], names["mixer.right_out"] = lp + "out", rp + "out"
                mixer = SideBySideSpec(hidden=d, left=left, right=rspec, combine="normed_mean", eps=eps)
            else:
                left = _attention_spec(d, eps, a, rot, sc, mask, names, lp, "mixer.left.", gate="channel")
                names["mixer.left.g.weight"] = lp + "g"
                rspec = GatedLinearAttentionSpec(hidden=d, heads=right.heads, head_dim=right.dim, value_dim=right.vdim,
                                                 decay_rank=_decay_rank(tensor_names, rp, right), tau=right.tau, eps=eps)
                for local, theirs in (("q.weight", "q"), ("k.weight", "k"), ("v.weight", "v"), ("g.weight", "g"), ("a1.weight", "a1"),
                                      ("a2.weight", "a2"), ("a2.bias", "a2.b"), ("norm.weight", "norm"), ("o.weight", "o")):
                    names["mixer.right." + local] = rp + theirs
                mixer = SideBySideSpec(hidden=d, left=left, right=rspec, combine="scaled", left_scale=pair.left_scale,
                                       right_scale=pair.right_scale, eps=eps)
        ffn = None
        if f is not None:
            ex, ro, sh = f
            names["norm2.weight"] = p + "norm2"
            shared = (GatedMLPSpec(hidden=d, intermediate=sh.ff, activation="clamped_swish", limit=sh.limit, alpha=SWISH_ALPHA)
                      if sh is not None else None)
            ffn = RoutedExpertsSpec(hidden=d, intermediate=ex.ff, experts=ro.experts, top=ro.top, activation="clamped_swish",
                                    limit=ex.limit, alpha=SWISH_ALPHA, router_bias=False, scoring="softmax_norm", shared=shared,
                                    shared_gate=sh is not None)
            names["ffn.router.weight"] = p + "mlp.router"
            for e in range(ro.experts):
                for local in ("gate", "up", "down"):
                    names[f"ffn.e{e}.{local}.weight"] = p + f"mlp.e{e}.{local}"
            if sh is not None:
                for local in ("gate", "up", "down"):
                    names[f"ffn.shared.{local}.weight"] = p + f"mlp.shared.{local}"
                names["ffn.shared_gate"] = p + "mlp.shared.sg"
        if cfg.streams:
            for q in ("1", "2") if ffn is not None else ("1",):
                for n in ("in", "out", "mix"):
                    names[f"hc{q}.{n}"] = f"{p}hc{q}.{n}"
        layers.append(LayerSpec(mixer=mixer, ffn=ffn, norm1=NormSpec(d, eps), norm2=NormSpec(d, eps) if ffn is not None else None,
                                names=names, kind="hyper", streams=cfg.streams, residual_mult=cfg.residual_mult))
        schedule.append(ScheduleEntry(i, i, borrow=borrow))
    return ModelSpec(
        embedding=EmbeddingSpec(vocab=cfg.vocab, dim=d, name="embed"), layers=tuple(layers), schedule=tuple(schedule),
        head=HeadSpec(vocab=cfg.vocab, dim=d, norm=NormSpec(d, eps), tied=False, norm_name="final.norm", name="head"),
        max_positions=cfg.max_positions, streams=max(cfg.streams, 1))


# The rank of the decay's low-rank projection is the one size of a layer that config.json leaves to the tensors' shapes.
DEFAULT_DECAY_RANK = 16


def _decay_rank(tensor_names, prefix: str, right) -> int:
    """Rows of ``<prefix>a1`` when the caller knows the file's shapes (a mapping name -> shape), else the default."""
    if isinstance(tensor_names, dict):
        shape = tensor_names.get(prefix + "a1")
        if shape is not None:
            return int(shape[0])
    return right.rank or DEFAULT_DECAY_RANK
