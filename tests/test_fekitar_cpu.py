"""Fekitar without a GPU: the configuration reader (nested keys, defaults, refusals), the model description (tensor names
and shapes, cache requests, the schedule's borrowed entries, a size that only a tensor's shape gives), and identities of the
plain implementation itself (a convolution cut anywhere with its tail, a recurrence cut anywhere with its state, window
membership, the band-wise frequency rescaling, routing weights that sum to one)."""

from __future__ import annotations

import copy

import pytest
import torch

import tiny_fekitar as tl
from plain import fekitar_plain as plain
from sleuth_b200.config import ConfigError, parse_config
from sleuth_b200.engine.model import declare_model


def spec_of(cfg, shapes=None):
    arch, c, unread = parse_config(cfg)
    assert arch.name == "Fekitar" and not unread
    return arch.model_spec(c, tensor_names=shapes)


@pytest.mark.parametrize("name", list(tl.CONFIGS))
def test_the_description_names_every_tensor_once(name):
    cfg = tl.CONFIGS[name]
    spec = spec_of(cfg)
    decl = declare_model(spec)
    d = cfg["width"]
    assert decl["embed"].shape == (cfg["vocab"], d) and decl["head"].shape == (cfg["vocab"], d) and decl["final.norm"].shape == (d,)
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        assert (p + "hc1.mix" in decl) == bool(cfg.get("streams"))
        assert (p + "hc2.mix" in decl) == bool(cfg.get("streams") and L["mlp"])
        assert (p + "norm2" in decl) == bool(L["mlp"])
        m = L["mixer"]
        if L["type"] == "attention":
            assert decl[p + "mix.q"].shape == (m["heads"] * 2 * m["dim"], d) and decl[p + "mix.g"].shape == (m["heads"], d)
            assert (p + "mix.k" in decl) == ("kv_from" not in m) and (p + "mix.q.conv" in decl) == bool(m.get("conv"))
            if "kv_from" not in m:
                assert decl[p + "mix.k"].shape == (m["kv_heads"] * 2 * m["dim"], d) and decl[p + "mix.v"].shape == (m["kv_heads"] * m["vdim"], d)
        elif L["type"] == "parallel":
            r = m["right"]
            inner = r["heads"] * r["vdim"]
            assert decl[p + "mix.right.in"].shape == (2 * inner + 2 * r["groups"] * r["state"] + r["heads"], d)
            assert decl[p + "mix.right.conv"].shape == (inner + 2 * r["groups"] * r["state"], r["conv"])
            assert decl[p + "mix.left.out"].shape == (d,) and decl[p + "mix.left.q.norm"].shape == (m["left"]["dim"],)
        else:
            r = m["right"]
            assert decl[p + "mix.right.a1"].shape == (r["rank"], d) and decl[p + "mix.right.a2"].shape == (r["heads"] * r["dim"], r["rank"])
            assert decl[p + "mix.left.g"].shape == (m["left"]["heads"] * m["left"]["vdim"], d)
        if L["mlp"]:
            f = L["mlp"]
            assert decl[p + "mlp.router"].shape == (f["router"]["experts"], d)
            assert (p + "mlp.shared.sg" in decl) == ("shared" in f)
    borrowed = [e.borrow for e in spec.schedule]
    assert borrowed == [L["mixer"].get("kv_from", -1) if L["type"] == "attention" else -1 for L in cfg["layers"]]
    assert spec.streams == max(cfg.get("streams", 0), 1)


def test_a_size_that_only_a_shape_gives_is_read_from_the_file():
    cfg = copy.deepcopy(tl.R)
    del cfg["layers"][1]["mixer"]["right"]["rank"]
    assert declare_model(spec_of(cfg, {"l1.mix.right.a1": (11, 72)}))["l1.mix.right.a2"].shape[1] == 11


def test_cache_requests_bundle_pages_states_and_tails():
    from sleuth_b200.cache.paged import BundleRequest, KVRequest, StateRequest, leaf_requests
    from sleuth_b200.engine.model import Model
    from sleuth_b200.parts.base import BuildContext
    model = Model(spec_of(tl.R), BuildContext(device=torch.device("cpu"), dtype=torch.float32, max_positions=64))
    reqs = model.cache_requests
    assert all(isinstance(r, BundleRequest) for r in reqs)
    leaves = [list(leaf_requests(r)) for r in reqs]
    assert leaves[0] == [KVRequest(2, 16, 37, 24), StateRequest((2, 4 * 16 + 2 * 16 + 2 * 24)), StateRequest((3, 12, 16)),
                         StateRequest((1, 48 + 24))]
    assert leaves[2] == [KVRequest(1, 32, 0, 40), StateRequest((3, 2 * 2 * 16 + 2 * 16 + 40))]
    assert leaves[4] == [StateRequest((1, 2 * 2 * 16))]           # the borrowing layer keeps its query tails only


def test_refusals():
    def broken(change):
        cfg = copy.deepcopy(tl.R)
        change(cfg)
        with pytest.raises(ConfigError):
            spec_of(cfg)
    broken(lambda c: c["layers"][0].update(type="serial"))
    broken(lambda c: c["layers"][0]["mixer"]["left"].update(heads=3))                 # 3 query heads on 2 key/value heads
    broken(lambda c: c["layers"][0]["mixer"]["left"].update(window=5))                # an unknown key
    broken(lambda c: c["layers"][4]["mixer"].update(kv_from=3))                       # layer 3 is no attention layer
    broken(lambda c: c["layers"][4]["mixer"].update(kv_from=4))                       # itself
    broken(lambda c: c["layers"][4]["mixer"].update(vdim=8))                          # other widths than its lender's
    broken(lambda c: c["layers"][2]["mixer"].pop("diff"))
    broken(lambda c: c["layers"][1]["mlp"]["router"].update(top=7))
    broken(lambda c: c.update(streams=17))
    broken(lambda c: c["layers"][0]["mixer"]["right"].update(groups=2))               # 3 heads in 2 groups


def test_a_convolution_cut_anywhere_with_its_tail():
    g = torch.Generator().manual_seed(0)
    u, w = torch.randn(40, 6, generator=g, dtype=torch.float64), torch.randn(6, 4, generator=g, dtype=torch.float64)
    whole = plain.short_convolution(u, w)
    for cut in (1, 2, 3, 17):
        tail = torch.cat([torch.zeros(3, 6, dtype=torch.float64), u[:cut]])[-3:]
        second = plain.short_convolution(torch.cat([tail, u[cut:]]), w)[3:]
        torch.testing.assert_close(second, whole[cut:])


def test_a_recurrence_cut_anywhere_with_its_state():
    g = torch.Generator().manual_seed(1)
    T, H, N, P = 30, 2, 5, 3
    a = torch.rand(T, H, N, generator=g, dtype=torch.float64)
    k, q = torch.randn(T, H, N, generator=g, dtype=torch.float64), torch.randn(T, H, N, generator=g, dtype=torch.float64)
    v = torch.randn(T, H, P, generator=g, dtype=torch.float64)
    whole, last = plain.matrix_state_recurrence(a, k, v, q)
    for cut in (1, 7, 29):
        _, S = plain.matrix_state_recurrence(a[:cut], k[:cut], v[:cut], q[:cut])
        rest, S2 = plain.matrix_state_recurrence(a[cut:], k[cut:], v[cut:], q[cut:], S)
        torch.testing.assert_close(rest, whole[cut:])
        torch.testing.assert_close(S2, last)


def test_window_membership_and_the_distance_penalty():
    seen = plain.visible(10, 3)
    assert seen[5].nonzero().flatten().tolist() == [3, 4, 5] and seen[1].nonzero().flatten().tolist() == [0, 1]
    assert plain.visible(4, 0)[3].all() and plain.visible(4, 1).sum() == 4
    s = plain.distance_slopes(4, torch.float64)
    assert s.tolist() == [2.0 ** -2, 2.0 ** -4, 2.0 ** -6, 2.0 ** -8]


def test_frequency_rescaling_band_by_band():
    from sleuth_b200.parts.position import rescale_bands
    rot = {"base": 10000.0, "dims": 64, "scaling": {"factor": 6.0, "low": 2.0, "high": 5.0, "original": 640}}
    plain_f = plain.rotary_frequencies(rot, torch.float64)
    base = 10000.0 ** (-torch.arange(32, dtype=torch.float64) * 2 / 64)
    torch.testing.assert_close(rescale_bands(base, 6.0, 2.0, 5.0, 640), plain_f)
    wavelength = 2 * torch.pi / base
    assert torch.equal(plain_f[wavelength < 128], base[wavelength < 128])
    assert torch.allclose(plain_f[wavelength > 320], base[wavelength > 320] / 6.0)
    between = (wavelength >= 128) & (wavelength <= 320)
    assert between.any() and bool(((plain_f[between] <= base[between]) & (plain_f[between] >= base[between] / 6.0)).all())


def test_routing_weights_sum_to_one_and_the_shared_expert_is_gated():
    g = torch.Generator().manual_seed(2)
    d, E = 16, 5
    w = {"router": torch.randn(E, d, generator=g), "shared.sg": torch.randn(1, d, generator=g)}
    for e in list(range(E)) + ["shared"]:
        p = f"e{e}." if e != "shared" else "shared."
        w[p + "gate"], w[p + "up"], w[p + "down"] = (torch.randn(8, d, generator=g), torch.randn(8, d, generator=g), torch.randn(d, 8, generator=g))
    w = {k: v.double() for k, v in w.items()}
    h = torch.randn(6, d, generator=g).double()
    f = {"router": {"experts": E, "top": E}, "expert": {"limit": 1.5}}
    every = sum(plain.router_scores(h, w, "").double()[:, e:e + 1] * plain.clamped_expert(h, w, f"e{e}.", 1.5) for e in range(E))
    torch.testing.assert_close(plain.mixture(h, w, "", f), every)           # all experts chosen: the softmax weights themselves
    f["shared"] = {"limit": 2.0}
    extra = plain.mixture(h, w, "", f) - every
    torch.testing.assert_close(extra, torch.sigmoid(h @ w["shared.sg"].T) * plain.clamped_expert(h, w, "shared.", 2.0))
