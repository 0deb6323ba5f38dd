"""Descriptions of a model as data: which parts make up each layer, and in which order layers run.

An architecture turns its typed configuration into one ``ModelSpec``. Everything below the
architecture works from these descriptions alone: the part registries build a part from its spec
(``spec.kind`` names the class), the cache sizes its groups from what the parts ask for, and the
engine runs ``ModelSpec.schedule``. A spec carries every size and constant its part needs; no part
looks at a configuration or knows which model it sits in.

The reference composes its model the same way in spirit: ``make_norm(kind, dim, eps)``
(sleuth/forge/model/norm.py:53-58), ``make_mlp(cfg)`` (sleuth/forge/model/mlp.py:59-60), a per-layer
``attn_spec(i)`` (sleuth/forge/model/config.py:142-147) and ``shared_layers`` for a layer applied
more than once (sleuth/forge/model/config.py:80-86).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Mapping


@dataclass(frozen=True)
class NormSpec:
    """``kind="rmsnorm"``: x / sqrt(mean(x^2) + eps) * gain. ``kind="layernorm"``: (x - mean) / sqrt(var + eps) * gain,
    var the mean of the squared deviations, no bias. ``gain="scalar"``: the gain is one number for all channels (a
    tensor without axes in the weight file)."""
    dim: int
    eps: float
    kind: str = "rmsnorm"
    gain: str = "vector"


@dataclass(frozen=True)
class PositionSpec:
    """Position encoding applied to queries and keys. ``kind="rotary"``: the first ``rotary_dim`` channels of each
    head turn in pairs by the angle position * theta^(-2i/rotary_dim) of pair i; ``pairing="halves"`` pairs channel i
    with i + rotary_dim/2, ``pairing="neighbours"`` channel 2i with 2i + 1. ``kind="none"``: nothing.
    ``precise``: the tables are worked out in 64-bit and rounded once (otherwise in float32, operation by operation).
    ``scaling`` = (factor, low, high, original): frequencies are rescaled band by band. With wavelength l = 2 pi / f a
    frequency stays where l < original / high, becomes f / factor where l > original / low, and between the two
    (1 - s) f / factor + s f with s = (original / l - low) / (high - low)."""
    head_dim: int
    theta: float = 10000.0
    rotary_dim: int = 0          # 0 = all of head_dim
    kind: str = "rotary"
    pairing: str = "halves"
    precise: bool = False
    scaling: tuple = ()


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention over the key/value cache."""
    hidden: int                  # width of the input and of the output
    heads: int                   # query heads
    kv_heads: int                # key/value heads; divides ``heads``
    head_dim: int                # independent of ``hidden``
    position: PositionSpec
    qk_norm: bool = False        # per-head RMSNorm of q and k before the position encoding
    qk_norm_eps: float = 1e-6
    qkv_bias: bool = False
    window: int = 0              # 0 = every earlier key; n = the n most recent keys, the query's own included
    scale: float = 0.0           # 0 = 1/sqrt(head_dim)
    reads_shared_kv: bool = False  # no k/v projections: reads the cache another layer application wrote
    kind: str = "gqa_attention"
    value_dim: int = 0           # width of a head's values and output; 0 = head_dim
    qk_norm_span: str = "head"   # "head": one RMSNorm per head, gains [head_dim]; "projection": one over all heads of q
                                 # (and one over all heads of k) before they are split, gains of the projection's length
    sinks: bool = False          # a learned score per head joins the softmax denominator (no key, no value, unscaled)


@dataclass(frozen=True)
class ScoredAttentionSpec:
    """Causal grouped-query attention over the key/value cache with other score rules and other post-processing than
    ``AttentionSpec``'s. q = W_q h (``heads`` * ``maps`` units of ``head_dim``), k = W_k h (``kv_heads`` * ``maps`` units),
    v = W_v h (``kv_heads`` units of ``value_dim``); then, each optional and in this order: a short causal convolution over
    time on every channel of q, k and v (``conv_taps`` taps, tensors ``q.conv`` ...; the last taps - 1 projected values of a
    sequence are state); an RMS norm of every q and k unit with a gain of ``head_dim`` values (``qk_norm``); rotation of
    the first channels of every q and k unit (``position``). score = q . k * ``scale``; ``softcap`` c: c tanh(score / c);
    ``slope_exponent`` e > 0: the score loses 2^(-e (h + 1) / heads) * (i - j) for head h; ``window`` as for
    ``AttentionSpec``. ``maps`` = 2: differential attention, two softmax maps a head over the same values, o = a1 -
    lambda a2 with lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + ``diff`` (four tensors of ``head_dim`` values), then o
    divided by its root mean square over ``value_dim`` and multiplied by 1 - ``diff``. ``gate``: "channel" multiplies the
    concatenated heads by sigmoid(W_g h), "head" multiplies head h by sigmoid(W_g h)_h, "none" nothing.
    ``reads_shared_kv``: no key and value tensors; the application reads the cache entry that its schedule entry borrows."""
    hidden: int
    heads: int
    kv_heads: int
    head_dim: int
    value_dim: int
    position: PositionSpec
    scale: float
    eps: float = 1e-6
    conv_taps: int = 0
    qk_norm: bool = False
    softcap: float = 0.0
    slope_exponent: float = 0.0
    window: int = 0
    maps: int = 1
    diff: float = 0.0
    gate: str = "none"
    reads_shared_kv: bool = False
    kind: str = "scored_attention"


@dataclass(frozen=True)
class StateSpaceSpec:
    """The state-space-duality recurrence (Mamba-2). inner = ``heads`` * ``value_dim``; W_in h = [z: inner | x: inner |
    B: groups * state | C: groups * state | dt: heads]. x, B and C pass a causal convolution per channel (``conv_taps``
    taps with a bias) and silu. dt = softplus(dt + dt_bias); per head (head h reads group h // (heads / groups)) the
    ``state`` x ``value_dim`` matrix S_t = exp(-exp(A_log_h) dt) S_(t-1) + dt B_t x_t^T, y_t = S_t^T C_t + D_h x_t. y times
    silu(z), RMS-normed in ``norm_groups`` equal parts with a gain per channel, then W_o."""
    hidden: int
    heads: int
    value_dim: int
    state: int
    groups: int = 1
    conv_taps: int = 4
    norm_groups: int = 1
    eps: float = 1e-6
    kind: str = "state_space"


@dataclass(frozen=True)
class GatedLinearAttentionSpec:
    """Linear attention with a decay per key channel. q = W_q h * head_dim^(-1/2), k = W_k h (``heads`` x ``head_dim``),
    v = W_v h (``heads`` x ``value_dim``); alpha = sigmoid(W_a2 (W_a1 h) + b)^(1 / ``tau``), one factor per key channel.
    Per head S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; each head's o RMS-normed over ``value_dim`` with a
    gain shared by the heads, the heads times silu(W_g h), then W_o."""
    hidden: int
    heads: int
    head_dim: int
    value_dim: int
    decay_rank: int
    tau: float
    eps: float = 1e-6
    kind: str = "gated_linear_attention"


@dataclass(frozen=True)
class SideBySideSpec:
    """Two mixers that read the same input; tensors of the first under ``left.``, of the second under ``right.``.
    ``combine="normed_mean"``: half the sum of the two results, each first RMS-normed over the model width with a gain of
    its own (tensors ``left_out``, ``right_out``). ``combine="scaled"``: left_scale * left + right_scale * right."""
    hidden: int
    left: object
    right: object
    combine: str = "scaled"
    left_scale: float = 1.0
    right_scale: float = 1.0
    eps: float = 1e-6
    kind: str = "side_by_side"


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Causal attention through low-rank latents. Queries: a normed latent of ``q_rank`` values, up-projected to
    ``heads`` x (``plain_dim`` unrotated + ``rot_dim`` rotated) values. Keys and values: one normed latent of
    ``kv_rank`` values per token, from which each head's ``plain_dim`` key values and ``value_dim`` values are
    up-projected, plus one rotated key part of ``rot_dim`` values shared by all heads. The cache keeps the latent
    and the rotated part only. ``position`` rotates the ``rot_dim`` parts (its ``head_dim`` is ``rot_dim``).
    ``output_gate``: the heads' outputs are multiplied by sigmoid(W_g h) before the output matrix; ``gate_span`` says
    whether W_g gives one value per output channel ("channel") or one per head ("head").
    ``q_rank`` 0: the queries do not pass through a latent; q = W_q h with the tensor ``q.weight``.
    A position part with ``pairing="neighbours"`` turns channels 2i and 2i + 1 of the rotated parts together."""
    hidden: int
    heads: int
    plain_dim: int
    rot_dim: int
    value_dim: int
    q_rank: int
    kv_rank: int
    position: PositionSpec
    scale: float
    norm_eps: float = 1e-6
    window: int = 0              # 0 = every earlier token; n = the n most recent tokens, the query's own included
    output_gate: bool = True
    kind: str = "latent_attention"
    gate_span: str = "channel"


@dataclass(frozen=True)
class MinGRUSpec:
    """A recurrence whose update gate and candidate are functions of the step's input alone, ``width`` channels wide, with a float32 state per
    sequence: z = sigmoid(W_z h + b_z), u = W_x h + b_x, candidate c = u + 1/2 where u >= 0 and sigmoid(u) below,
    S_t = (1 - z) S_(t-1) + z c from S = 0, output W_o (S_t * silu(W_g h))."""
    hidden: int
    width: int
    kind: str = "mingru"


@dataclass(frozen=True)
class GatedMLPSpec:
    """down(f(gate(x), up(x))), no biases; ``activation``: "silu" (silu(g) u), "relu" (relu(g) u), "gelu_tanh"
    (0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))) u) or "clamped_swish"
    (g' = min(g, limit), u' = clamp(u, -limit, limit): g' sigmoid(alpha g') (u' + 1))."""
    hidden: int
    intermediate: int
    activation: str = "silu"
    kind: str = "gated_mlp"
    limit: float = 0.0
    alpha: float = 1.0


@dataclass(frozen=True)
class RoutedExpertsSpec:
    """``experts`` gated feed-forwards of ``intermediate`` channels, of which a token uses ``top``.
    ``scoring="softmax_top"``: those with the largest router logits (W_r h + b, float32), weighted by the softmax over
    those logits alone. ``scoring="sigmoid"``: scores = sigmoid(logits); the experts form ``groups`` equal groups of
    neighbours, a group scores the sum of its two largest scores, and only experts of the ``keep_groups`` best groups
    can be chosen; the ``top`` largest scores, weights = score / (their sum + 1e-20) * ``route_scale``.
    ``scoring="softmax"``: scores = softmax over all experts' logits; the ``top`` largest of score + correction are chosen
    (``choice_bias``: the tensor ``correction``, one value per expert, moves the choice and never the weights); weights = the chosen
    experts' scores * ``route_scale`` as they are (no division by their sum). ``scoring="softmax_norm"``: the same scores and
    choice; weights = score / (the chosen scores' sum + 1e-20) * ``route_scale``.
    ``activation``, ``limit``, ``alpha``: as for ``GatedMLPSpec``. ``shared``: a gated feed-forward (a ``GatedMLPSpec``)
    that every token runs and whose output is added, or None."""
    hidden: int
    intermediate: int
    experts: int
    top: int
    activation: str = "silu"
    router_bias: bool = True
    kind: str = "routed_experts"
    limit: float = 0.0
    alpha: float = 1.0
    scoring: str = "softmax_top"
    groups: int = 1
    keep_groups: int = 1
    route_scale: float = 1.0
    shared: object = None
    choice_bias: bool = False
    shared_gate: bool = False    # the shared expert's result is multiplied by sigmoid(w . h), one number a token (tensor ``shared_gate``)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (``kind``) of a mixer, a feed-forward and their norms. ``kind="parallel"``:
    x += mixer(norm1 x) + ffn(norm2 x), both of the same x; without ``norm2`` (None) the feed-forward reads norm1's
    output too; it may have no feed-forward (``ffn`` is None). ``kind="sandwich"``: a norm in front of and behind each
    sublayer, x += post1(mixer(norm1 x)), then x += post2(ffn(norm2 x)); with ``gated`` each sublayer's result is first
    multiplied by sigmoid(W h + b) of the sublayer's own input h (tensors ``gate1.weight``, ``gate1.bias``, ``gate2...``).

    ``kind="hyper"``: hyper-connections. The model keeps ``streams`` copies of the stream; sublayer q (1 the mixer, 2 the
    feed-forward) reads u = sum_s in_q[s] x_s, y = sublayer(norm_q(u)), and all copies change at once from the old ones:
    x_r <- sum_s mix_q[s, r] x_s + ``residual_mult`` * out_q[r] * y (tensors ``hc1.in`` [streams], ``hc1.out`` [streams],
    ``hc1.mix`` [streams, streams], ``hc2...``). With ``streams`` 0 there is one copy and no such tensors:
    x <- x + ``residual_mult`` * y.

    ``names`` maps each part-local tensor name ("norm1.weight", "mixer.q_proj.weight",
    "ffn.down.weight", ...) to its name in the weight files."""
    mixer: object
    ffn: object
    norm1: NormSpec
    norm2: NormSpec
    names: Mapping[str, str] = field(default_factory=dict)
    kind: str = "prenorm"
    post1: NormSpec | None = None
    post2: NormSpec | None = None
    gated: bool = False
    streams: int = 0
    residual_mult: float = 1.0


@dataclass(frozen=True)
class ScheduleEntry:
    """One application of a layer. ``cache`` numbers the cache entry it uses; the first application
    in schedule order that names an entry owns it (and writes it), later ones only read it.

    Right before the application the model may add to the stream: the embedding's output once more
    (``add_embedding``) and row ``add_row`` of the model's table of pass vectors (``ModelSpec.pass_rows``). With
    ``mix_embedding`` the stream is first replaced by W [x; x0], x0 being the embedding's output and W the model's
    ``[width, 2 * width]`` matrix ``ModelSpec.pass_mix``. ``borrow``: a cache entry of an earlier application whose
    keys and values this application reads beside its own entry (which still holds what it keeps for itself)."""
    layer: int
    cache: int
    add_embedding: bool = False
    add_row: int = -1
    mix_embedding: bool = False
    borrow: int = -1


@dataclass(frozen=True)
class EmbeddingSpec:
    """The part that fills the stream from token ids. ``name`` is the checkpoint name of its tensor ``weight``; a
    part of another ``kind`` that declares more tensors gives their checkpoint names in a field ``names``
    (local name -> checkpoint name) of its own spec class."""
    vocab: int
    dim: int
    scale: float = 1.0
    name: str = "model.embed_tokens.weight"
    kind: str = "token_embedding"
    norm: NormSpec | None = None          # a norm applied to the looked-up rows (its gain is the tensor ``norm.weight``)
    norm_name: str = "model.embed_norm.weight"


@dataclass(frozen=True)
class PairEmbeddingSpec:
    """Token rows times ``scale`` plus a row of a hashed table of token pairs: row (previous token * ``mul_prev`` + token
    * ``mul_cur``) mod ``buckets`` of the ``[buckets + 1, dim]`` tensor ``pairs``; a sequence's first token takes the
    last row. The previous token is kept per sequence between steps. ``names``: checkpoint names of ``weight`` and
    ``pairs``."""
    vocab: int
    dim: int
    buckets: int
    mul_prev: int
    mul_cur: int
    scale: float = 1.0
    names: Mapping[str, str] = field(default_factory=dict)
    name: str = ""
    kind: str = "pair_embedding"


@dataclass(frozen=True)
class HeadSpec:
    """Final norm and output matrix. ``tied``: the output matrix is the embedding table. ``norm_name`` and ``name``
    are the checkpoint names of the tensors ``norm.weight`` and ``weight``; more tensors of another ``kind`` are
    named by a field ``names`` (local name -> checkpoint name) of its own spec class."""
    vocab: int
    dim: int
    norm: NormSpec
    tied: bool
    norm_name: str = "model.norm.weight"
    name: str = "lm_head.weight"
    kind: str = "lm_head"
    softcap: float = 0.0         # c > 0: logits <- c * tanh(logits / c)
    scale: float = 1.0           # the logits are multiplied by this


@dataclass(frozen=True)
class ModelSpec:
    embedding: EmbeddingSpec
    layers: tuple
    schedule: tuple
    head: HeadSpec
    max_positions: int
    ignored_tensors: tuple = ()   # regular expressions of tensor names a checkpoint may hold and nobody reads
    pass_rows: str | None = None  # checkpoint name of a [rows, width] table whose rows schedule entries add to the stream
    pass_rows_count: int = 0
    pass_mix: str | None = None   # checkpoint name of the [width, 2 * width] matrix of entries with ``mix_embedding``
    streams: int = 1              # copies of the residual stream (hyper-connections): all start as the embedding's output,
                                  # layers of kind "hyper" read and write them, their sum enters the final norm

    def __post_init__(self):
        seen = set()
        for e in self.schedule:
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule names layer {e.layer}, the model has {len(self.layers)}")
            seen.add(e.cache)
            if e.add_row >= 0 and not (self.pass_rows and e.add_row < self.pass_rows_count):
                raise ValueError(f"schedule adds row {e.add_row} of a table of {self.pass_rows_count} pass vectors")
            if e.borrow >= 0 and e.borrow == e.cache:
                raise ValueError("a schedule entry borrows its own cache entry")
            if e.mix_embedding and not self.pass_mix:
                raise ValueError("a schedule entry mixes the embedding into the stream and the model names no matrix for it")
        if seen and seen != set(range(len(seen))):
            raise ValueError(f"cache entries must be numbered 0..{len(seen) - 1} without gaps, got {sorted(seen)}")


def looped_schedule(n_layers: int, start: int, stop: int, times: int, entry: str = "add") -> tuple:
    """Layers ``start .. stop - 1`` run ``times`` times in a row with the same weights, each pass with cache entries of
    its own; every pass begins by adding its row of the pass vectors. Before that, with ``entry="add"`` every pass but
    the first adds the embedding's output; with ``entry="mix"`` every pass (the first too) replaces the stream by the
    model's mixing matrix applied to [x; embedding output]. The other layers run once."""
    if entry not in ("add", "mix"):
        raise ValueError(f"a loop is entered by 'add' or 'mix', not {entry!r}")
    if not (0 <= start < stop <= n_layers and times >= 1):
        raise ValueError(f"a loop over layers {start}..{stop - 1}, {times} times, does not fit {n_layers} layers")
    out, cache = [], 0
    for i in range(start):
        out.append(ScheduleEntry(i, cache))
        cache += 1
    for t in range(times):
        for i in range(start, stop):
            first = i == start
            out.append(ScheduleEntry(i, cache, add_embedding=first and t > 0 and entry == "add", add_row=t if first else -1,
                                     mix_embedding=first and entry == "mix"))
            cache += 1
    for i in range(stop, n_layers):
        out.append(ScheduleEntry(i, cache))
        cache += 1
    return tuple(out)


def shared_weight_schedule(owners) -> tuple:
    """``owners[i]``: index (among the model's layers, which hold weights) of the layer whose weights application i uses.
    Every application has a cache entry of its own."""
    return tuple(ScheduleEntry(int(o), i) for i, o in enumerate(owners))


def straight_schedule(n_layers: int) -> tuple:
    """Every layer once, in order, each with a cache entry of its own."""
    return tuple(ScheduleEntry(i, i) for i in range(n_layers))
