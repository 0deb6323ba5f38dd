"""Movalorn without a GPU: its configuration, its model description, its tensors, refusals, and the plain
implementation's own consistency (the recurrence cut into chunks, the window, the rotation of neighbouring channels
against the rotation of halves on reordered channels, the pair table's rows, the order of layer runs)."""

from __future__ import annotations

import copy

import pytest
import torch

import tiny_movalorn as tm
from plain import lezepel_plain
from plain import movalorn_plain as plain
from plain.qwen3_plain import read_model
from sleuth_b200.config import ConfigError, parse_config
from sleuth_b200.engine.model import declare_model
from sleuth_b200.parts.spec import looped_schedule


def spec_of(cfg):
    arch, typed, unread = parse_config(cfg)
    assert arch.name == "Movalorn" and set(unread) <= {"torch_dtype"}      # the folder writer's own note
    return arch.model_spec(typed)


def test_every_size_and_constant_comes_from_the_configuration():
    spec = spec_of(tm.K)
    m = spec.layers[0].mixer
    assert (m.heads, m.plain_dim, m.rot_dim, m.value_dim, m.q_rank, m.kv_rank, m.window) == (3, 16, 8, 24, 0, 40, 37)
    assert m.scale == 0.31 and m.position.theta == 500.0 and m.position.rotary_dim == 8 and m.norm_eps == 1e-6
    assert m.position.pairing == "neighbours" and m.gate_span == "head" and m.output_gate
    assert spec.layers[2].mixer.window == 0 and spec.layers[2].mixer.heads == 5
    assert spec.layers[1].mixer.kind == "mingru" and spec.layers[1].mixer.width == 52 and spec.layers[3].mixer.width == 100
    e = spec.embedding
    assert (e.kind, e.vocab, e.dim, e.buckets, e.mul_prev, e.mul_cur, e.scale) == ("pair_embedding", 301, 72, 97, 7, 13, 3.0)
    assert spec.head.scale == 0.5 and spec.head.norm.eps == 1e-6 and spec.head.norm.gain == "scalar"
    kinds = [type(L.ffn).__name__ for L in spec.layers]
    assert kinds == ["GatedMLPSpec", "RoutedExpertsSpec", "NoneType", "RoutedExpertsSpec"]
    assert spec.layers[0].ffn.activation == "gelu_tanh" and spec.layers[0].ffn.intermediate == 100
    f = spec.layers[1].ffn
    assert (f.experts, f.top, f.intermediate, f.route_scale, f.scoring, f.choice_bias, f.router_bias) == (5, 2, 36, 1.5, "softmax", True, False)
    assert f.shared.intermediate == 28 and f.shared.activation == "silu" and f.activation == "silu"
    assert spec.layers[3].ffn.shared is None and spec.layers[3].ffn.top == 1 and spec.layers[3].ffn.route_scale == 0.7
    assert all(L.kind == "sandwich" and L.gated and L.norm1.gain == "scalar" and L.post1.gain == "scalar" for L in spec.layers)
    assert spec.layers[2].norm2 is None and spec.layers[2].post2 is None
    assert spec_of(tm.M).embedding.kind == "token_embedding" and spec_of(tm.M).head.scale == 1.0


def test_the_loop_becomes_a_schedule_with_caches_and_states_of_its_own():
    spec = spec_of(tm.K)
    got = [(e.layer, e.mix_embedding, e.add_row, e.add_embedding) for e in spec.schedule]
    assert got == [(0, False, -1, False), (1, True, 0, False), (2, False, -1, False), (1, True, 1, False), (2, False, -1, False),
                   (3, False, -1, False)]
    assert [e.cache for e in spec.schedule] == list(range(6)) and spec.pass_rows == "loop.step" and spec.pass_mix == "loop.in"
    first = [(e.layer, e.mix_embedding, e.add_row) for e in spec_of(tm.L).schedule]
    assert first == [(0, True, 0), (1, False, -1), (0, True, 1), (1, False, -1), (0, True, 2), (1, False, -1)]
    none = spec_of(tm.M)
    assert none.pass_rows is None and none.pass_mix is None and len(none.schedule) == 3
    once = [(e.layer, e.mix_embedding, e.add_row) for e in spec_of(tm.N).schedule]
    assert once == [(0, False, -1), (1, False, -1), (2, True, 0), (3, False, -1)]
    assert plain.layer_runs(tm.K) == [(0, None, False), (1, 0, True), (2, 0, False), (1, 1, True), (2, 1, False), (3, None, False)]
    with pytest.raises(ValueError):
        looped_schedule(3, 0, 2, 2, entry="replace")


def test_declared_tensors_carry_the_file_names_and_shapes():
    d = declare_model(spec_of(tm.K))
    assert d["embed"].shape == (301, 72) and d["bigram"].shape == (98, 72) and d["head"].shape == (301, 72)
    assert d["final.norm"].shape == () and d["final.norm"].role == "vector"
    assert d["loop.step"].shape == (2, 72) and d["loop.in"].shape == (72, 144) and d["loop.in"].role == "matrix"
    for n in ("norm1", "norm1b", "norm2", "norm2b"):
        assert d["l0." + n].shape == ()
    assert "l2.norm2" not in d and "l2.rg2" not in d and "l2.norm1b" in d
    assert d["l0.rg1"].shape == (72, 72) and d["l0.rg1.b"].shape == (72,) and d["l0.rg1.b"].role == "vector"
    assert d["l0.mix.q"].shape == (3 * 24, 72) and d["l0.mix.dkv"].shape == (48, 72) and d["l0.mix.dkv.norm"].shape == (40,)
    assert d["l0.mix.uk"].shape == (48, 40) and d["l0.mix.uv"].shape == (72, 40)
    assert d["l0.mix.g"].shape == (3, 72) and d["l0.mix.o"].shape == (72, 72)
    assert d["l1.mix.z"].shape == (52, 72) and d["l1.mix.z.b"].shape == (52,) and d["l1.mix.o"].shape == (72, 52)
    assert d["l0.mlp.gate"].shape == (100, 72) and d["l0.mlp.down"].shape == (72, 100)
    assert d["l1.mlp.router"].shape == (5, 72) and d["l1.mlp.correction"].shape == (5,)
    assert d["l1.mlp.e4.up"].shape == (36, 72) and d["l1.mlp.shared.down"].shape == (72, 28)
    assert "l3.mlp.shared.gate" not in d and "l1.mlp.router.b" not in d
    assert "bigram" not in declare_model(spec_of(tm.M))


@pytest.mark.parametrize("edit, word", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "known mixer"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("heads", 0), "positive"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("q_rank", 8), "unknown key"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 10), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("size", 0), "mask.size"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("width", -1), "width"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 9), "router.top"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "sparse"), "kind"),
    (lambda c: c["embedding"]["bigram"].__setitem__("buckets", 0), "buckets"),
    (lambda c: c["loop"].__setitem__("stop", 9), "loop"),
    (lambda c: c["norm"].__setitem__("eps", 0), "eps"),
    (lambda c: c.pop("width"), "width"),
])
def test_a_configuration_that_cannot_be_is_refused(edit, word):
    cfg = copy.deepcopy(tm.K)
    edit(cfg)
    with pytest.raises(ConfigError) as e:
        spec_of(cfg)
    assert word in str(e.value)


def test_random_folders_hold_the_declared_tensors(movalorn_folders):
    for name in tm.CONFIGS:
        cfg, w = read_model(movalorn_folders[name])
        d = declare_model(spec_of(cfg))
        assert set(w) == set(d)
        assert all(tuple(w[k].shape) == tuple(d[k].shape) for k in d)
        assert w["final.norm"].dim() == 0 and abs(float(w["final.norm"]) - 1.0) < 0.5


# ---- the plain implementation's own identities ----
def test_the_pair_table_rows():
    w = {"embed": torch.arange(12.0).reshape(6, 2), "bigram": torch.arange(100.0, 116.0).reshape(8, 2)}
    e = {"scale": 2.0, "bigram": {"buckets": 7, "mul_prev": 3, "mul_cur": 5}}
    ids = torch.tensor([4, 1, 1, 5])
    x = plain.embedding(ids, w, e)
    rows = [7, (4 * 3 + 1 * 5) % 7, (1 * 3 + 1 * 5) % 7, (1 * 3 + 5 * 5) % 7]
    assert torch.equal(x, w["embed"][ids] * 2.0 + w["bigram"][rows])


def test_neighbour_rotation_is_half_rotation_of_reordered_channels():
    torch.manual_seed(0)
    v = torch.randn(9, 3, 14, dtype=torch.float64)
    pos = torch.arange(9)
    a = plain.rotate_neighbours(v, pos, 300.0, 10)
    order = torch.cat([torch.arange(0, 10, 2), torch.arange(1, 10, 2), torch.arange(10, 14)])
    b = lezepel_plain.rotate_half_pairs(v[..., order], pos, 300.0, 10)
    torch.testing.assert_close(a[..., order], b)
    # a dot product of two turned vectors depends on the distance of their positions only
    q, k = torch.randn(1, 10, dtype=torch.float64), torch.randn(1, 10, dtype=torch.float64)
    d1 = (plain.rotate_neighbours(q, torch.tensor([7]), 50.0, 10) * plain.rotate_neighbours(k, torch.tensor([3]), 50.0, 10)).sum()
    d2 = (plain.rotate_neighbours(q, torch.tensor([24]), 50.0, 10) * plain.rotate_neighbours(k, torch.tensor([20]), 50.0, 10)).sum()
    torch.testing.assert_close(d1, d2)


def test_a_window_of_n_holds_the_query_and_the_n_minus_one_tokens_in_front():
    torch.manual_seed(1)
    q, k, v = (torch.randn(12, 2, 4, dtype=torch.float64) for _ in range(3))
    full = plain.windowed_softmax_attention(q, k, v, 0.5, 0)
    torch.testing.assert_close(plain.windowed_softmax_attention(q, k, v, 0.5, 12), full)
    torch.testing.assert_close(plain.windowed_softmax_attention(q, k, v, 0.5, 400), full)
    one = plain.windowed_softmax_attention(q, k, v, 0.5, 1)
    torch.testing.assert_close(one, v)                  # a window of one token is the token itself
    w3 = plain.windowed_softmax_attention(q, k, v, 0.5, 3)
    i = 9
    s = torch.einsum("hd,jhd->hj", q[i], k[i - 2:i + 1]) * 0.5
    torch.testing.assert_close(w3[i], torch.einsum("hj,jhd->hd", torch.softmax(s, -1), v[i - 2:i + 1]))


def test_the_recurrence_may_be_cut_anywhere():
    """S_end = A S_start + B over a chunk, A the product of the decays: what the two-pass kernel relies on."""
    torch.manual_seed(2)
    h = torch.randn(50, 6, dtype=torch.float64)
    w = {"z": torch.randn(4, 6, dtype=torch.float64), "z.b": torch.randn(4, dtype=torch.float64),
         "x": torch.randn(4, 6, dtype=torch.float64), "x.b": torch.randn(4, dtype=torch.float64),
         "g": torch.randn(4, 6, dtype=torch.float64), "o": torch.eye(4, dtype=torch.float64)}
    whole = plain.mingru(h, w, "")
    z = torch.sigmoid(h @ w["z"].T + w["z.b"])
    u = h @ w["x"].T + w["x.b"]
    c = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    S = torch.zeros(4, dtype=torch.float64)
    for a in range(0, 50, 16):
        A, B = torch.ones(4, dtype=torch.float64), torch.zeros(4, dtype=torch.float64)
        for t in range(a, min(50, a + 16)):
            A, B = A * (1 - z[t]), (1 - z[t]) * B + z[t] * c[t]
        S = A * S + B
    g = h[-1] @ w["g"].T
    torch.testing.assert_close(S * g * torch.sigmoid(g), whole[-1])
    assert float(c.min()) > 0 and torch.equal(c[u >= 0], u[u >= 0] + 0.5)


def test_the_chosen_experts_and_their_weights():
    h = torch.tensor([[1.0, 0.0], [0.0, 2.0]], dtype=torch.float64)
    w = {"router": torch.tensor([[1.0, 0.0], [0.0, 1.0], [0.5, 0.5]], dtype=torch.float64),
         "correction": torch.tensor([0.0, 0.0, 10.0], dtype=torch.float64)}
    f = {"router": {"experts": 3, "top": 2, "scale": 1.5}}
    idx, wt, margin = plain.expert_choice(h, w, "", f)
    s = torch.softmax(h @ w["router"].T, -1)
    assert idx.tolist() == [[2, 0], [2, 1]]            # the correction decides the choice ...
    torch.testing.assert_close(wt, torch.gather(s, 1, idx) * 1.5)      # ... and stays out of the weights
    assert float(wt.sum(-1).max()) < 1.5 and bool((margin > 0).all())


def test_whole_model_runs_and_greedy_generation_repeats(movalorn_folders):
    cfg, w = read_model(movalorn_folders["K"])
    ids = [5, 9, 200, 1, 1, 77, 300, 4]
    logits, stream = plain.forward(cfg, w, ids, torch.float64, keep_stream=True)
    assert logits.shape == (8, 301) and stream.shape == (6, 8, 72) and bool(torch.isfinite(logits).all())
    # causal: a longer sequence leaves the earlier rows alone
    again = plain.forward(cfg, w, ids + [3, 3], torch.float64)
    torch.testing.assert_close(again[:8], logits)
    out = plain.greedy_generate(cfg, w, ids[:3], 4)
    assert len(out) == 4 and out == plain.greedy_generate(cfg, w, ids[:3], 4)
