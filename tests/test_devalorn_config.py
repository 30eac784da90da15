"""Devalorn without a GPU: the configuration reader, the run order with its shared caches,
expected tensors, random models on disk, and the plain implementation's own consistency."""
import copy

import pytest
import torch

import plain_devalorn as P
from pretrained_rstr_b200.config.base import ConfigError
from pretrained_rstr_b200.config.registry import lookup, named_size, read_config
from pretrained_rstr_b200.weights import make_random_model

RAW = {"architecture": "Devalorn", "vocab": 90, "width": 32, "norm": {"eps": 1e-6},
       "layers": [
           {"type": "attention", "mlp": None,
            "mixer": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 10, "scale": 0.4,
                      "mask": {"size": 7}, "q_temp": {"coef": 0.25, "every": 3}}},
           {"type": "parallel", "mlp": {"kind": "moe", "router": {"experts": 3, "top": 2, "scale": 1.5},
                                        "expert": {"ff": 10}},
            "mixer": {"left": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 4, "scale": 0.3,
                               "mask": {"size": 5, "keep_first": 2}, "rot": {"base": 50.0, "dims": 4}},
                      "right": {"heads": 2, "dim": 12}, "left_scale": 0.5, "right_scale": 1.25}},
           {"type": "attention", "mlp": {"kind": "dense", "ff": 20},
            "mixer": {"heads": 2, "kv_heads": 2, "dim": 6, "vdim": 10, "scale": 0.5, "kv_from": 0,
                      "mask": {"size": 4}, "q_temp": {"coef": 1.0, "every": 2}}}]}


def test_registry_and_structure():
    arch = lookup(RAW)
    cfg = arch.config_class.from_dict(RAW)
    assert arch.name == "Devalorn" and cfg.to_dict()["layers"] == RAW["layers"]
    order = cfg.run_order()
    assert [e.layer for e in order] == [0, 1, 2]
    assert [e.cache_layer for e in order] == [0, 1, 0]              # layer 2 reads layer 0's cache
    assert [e.writes_cache for e in order] == [True, True, False]
    specs = cfg.layer_specs()
    assert [s.arrangement for s in specs] == ["parallel"] * 3
    assert [s.mixer.kind for s in specs] == ["window_attention", "side_by_side", "window_attention"]
    assert [s.feed_forward.kind for s in specs] == ["none", "gated_moe", "gated_mlp"]
    assert set(specs[0].norms) == {"mixer"} and set(specs[1].norms) == {"mixer", "feed_forward"}
    a0, a2 = specs[0].mixer.params, specs[2].mixer.params
    assert a0["window"] == 7 and a0["keep_first"] == 0 and a0["q_temp"] == (0.25, 3)
    assert a0["qk_norm"] and a0["slope_bits"] == 8.0 and not a0["shares_cache"]
    assert a2["shares_cache"] and set(a2["weights"]) == {"q", "out", "q_norm"}
    side = specs[1].mixer.params
    assert side["left_scale"] == 0.5 and side["right_scale"] == 1.25
    left = side["left"].params
    assert left["keep_first"] == 2 and left["rot_dims"] == 4 and left["head_gate"] and not left.get("qk_norm")
    moe = specs[1].feed_forward.params
    assert moe["score"] == "softmax" and moe["router_scale"] == 1.5 and not moe["renormalize"]
    exp = arch.expected_tensors(cfg)
    assert exp["l0.mix.q"].shape == (24, 32) and exp["l0.mix.k"].shape == (12, 32)
    assert exp["l0.mix.v"].shape == (20, 32) and exp["l0.mix.k.norm"].shape == (12,)
    assert exp["l1.mix.left.g"].shape == (2, 32) and exp["l1.mix.left.o"].shape == (32, 8)
    assert exp["l1.mix.right.u"].shape == (2, 12) and exp["l1.mix.right.mu.w"].shape == (32,)
    assert exp["l1.mix.right.w1"].free_dims == (0,) and exp["l1.mix.right.w2"].shape[0] == 24
    assert "l0.norm2" not in exp and "l2.mix.k" not in exp and "l2.mix.k.norm" not in exp
    assert "l2.mix.q.norm" in exp and "l1.mlp.e2.down" in exp and "l1.mlp.e3.up" not in exp


@pytest.mark.parametrize("change", [
    lambda r: r["layers"][0].__setitem__("type", "convolution"),
    lambda r: r["layers"][0]["mixer"].__setitem__("kv_heads", 3),
    lambda r: r["layers"][1]["mixer"]["left"]["rot"].__setitem__("dims", 5),
    lambda r: r["layers"][1]["mixer"]["left"]["rot"].__setitem__("dims", 10),
    lambda r: r["layers"][1]["mixer"].__delitem__("right_scale"),
    lambda r: r["layers"][1]["mlp"]["router"].__setitem__("top", 4),
    lambda r: r["layers"][1]["mlp"].__setitem__("kind", "sparse"),
    lambda r: r["layers"][2]["mixer"].__setitem__("kv_from", 2),
    lambda r: r["layers"][2]["mixer"].__setitem__("kv_from", 1),
    lambda r: r["layers"][2]["mixer"].__setitem__("vdim", 12),
    lambda r: r["layers"][0]["mixer"]["q_temp"].__setitem__("every", 0),
    lambda r: r.__delitem__("norm"),
    lambda r: r.__setitem__("layers", [])])
def test_bad_configurations_are_refused(change):
    raw = copy.deepcopy(RAW)
    change(raw)
    with pytest.raises(ConfigError):
        lookup(raw).config_class.from_dict(raw)


def test_random_folder_round_trip_and_plain_consistency(tmp_path):
    """A random model written by the package is read by the plain implementation's own reader;
    the plain model is causal, its windows hide what they should, and its state carries."""
    arch = lookup(RAW)
    cfg = arch.config_class.from_dict(RAW)
    folder = str(tmp_path / "m")
    make_random_model(folder, cfg, 3, torch.float32)
    assert read_config(folder)[1].to_dict() == cfg.to_dict()
    raw, tensors = P.read_folder(folder)
    assert set(tensors) == set(arch.expected_tensors(cfg))
    ids = [5, 17, 3, 80, 41, 2, 2, 9, 63, 30, 11, 7, 55]
    taps = []
    full = P.forward(ids, tensors, raw, taps=taps)
    assert full.shape == (len(ids), 90) and len(taps) == 3
    assert torch.allclose(P.forward(ids[:6], tensors, raw), full[:6], atol=1e-10)       # causal
    mask = P.window_mask(torch.arange(12), 12, 5, 2)
    assert bool(mask[5, 5]) and bool(mask[5, 1]) and bool(mask[9, 5]) and not bool(mask[10, 5])
    assert bool(mask[10, 1]) and not bool(mask[10, 2]) and not bool(mask[3, 4])
    assert float(P.query_temperature(torch.tensor([0, 1, 2, 5]), 0.5, 3, torch.float64)[1]) == 1.0
    assert float(P.query_temperature(torch.tensor([2]), 0.5, 3, torch.float64)[0]) == pytest.approx(1.0 + 0.5 * 0.6931471805599453)
    assert P.distance_slopes(4, torch.float64).tolist() == [0.25, 0.0625, 0.015625, 0.00390625]
    # the recurrence carries: a sequence cut in two gives the same rows
    g = torch.Generator().manual_seed(1)
    r, k, v = (torch.randn(6, 2, 4, generator=g).double() for _ in range(3))
    w, u = torch.rand(6, 2, 4, generator=g).double(), torch.randn(2, 4, generator=g).double()
    whole, _ = P.decayed_outer_states(r, k, v, w, u)
    _, mid = P.decayed_outer_states(r[:4], k[:4], v[:4], w[:4], u)
    rest, _ = P.decayed_outer_states(r[4:], k[4:], v[4:], w[4:], u, state=mid)
    assert torch.allclose(rest, whole[4:], atol=1e-12)
    # the first token's result is the bonus alone: (r . (u * k)) v
    first = (r[0] * u * k[0]).sum(-1, keepdim=True) * v[0]
    assert torch.allclose(whole[0], first, atol=1e-12)
    # time mixing and the windowed attention continue from what they carried
    h = torch.randn(9, 32, generator=g).double()
    mx = RAW["layers"][1]["mixer"]
    both, _ = P.time_mix(h, tensors, "l1.mix.right.", mx["right"], 1e-6)
    _, carried = P.time_mix(h[:5], tensors, "l1.mix.right.", mx["right"], 1e-6)
    tail, _ = P.time_mix(h[5:], tensors, "l1.mix.right.", mx["right"], 1e-6, carried=carried)
    assert torch.allclose(tail, both[5:], atol=1e-10)
    both, _ = P.gated_window_attention(h, tensors, "l1.mix.left.", mx["left"])
    _, kv = P.gated_window_attention(h[:5], tensors, "l1.mix.left.", mx["left"])
    tail, _ = P.gated_window_attention(h[5:], tensors, "l1.mix.left.", mx["left"], kv=kv)
    assert torch.allclose(tail, both[5:], atol=1e-10)
    # chosen experts weigh by their share of the softmax over all experts, times the constant
    out = P.softmax_routed_experts(h[:3], tensors, "l1.mlp.", RAW["layers"][1]["mlp"])
    s = torch.softmax(h[:3] @ tensors["l1.mlp.router"].double().T, dim=-1)
    for i in range(3):
        want = torch.zeros(32, dtype=torch.float64)
        for e in torch.topk(s[i], 2).indices.tolist():
            want += 1.5 * s[i, e] * P.gated_unit(h[i:i + 1], *(tensors[f"l1.mlp.e{e}.{n}"].double()
                                                              for n in ("gate", "up", "down")))[0]
        assert torch.allclose(out[i], want, atol=1e-10)


def test_named_sizes():
    for name in ("devalorn-tiny", "devalorn-small", "devalorn-wide"):
        arch, cfg = named_size(name)
        assert arch.name == "Devalorn" and len(cfg.run_order()) == len(cfg.layers)
        assert any(not e.writes_cache for e in cfg.run_order())
