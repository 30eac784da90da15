"""Vakilorn without a GPU: the configuration reader, the run order of layers that share
tensors, expected tensors, random models on disk, and the plain implementation's own
consistency (prefill against token-by-token states, the rotations' two layouts)."""
import copy

import pytest
import torch

import plain_vakilorn as P
from pretrained_rstr_b200.config.base import ConfigError
from pretrained_rstr_b200.config.registry import lookup, named_size
from pretrained_rstr_b200.weights import make_random_model

_REC = {"type": "parallel", "mlp": {"kind": "dense", "ff": 20, "limit": 2.5},
        "mixer": {"left": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 10, "scale": 0.4,
                           "rot": {"base": 50.0, "dims": 4}},
                  "right": {"width": 24, "blocks": 3, "conv": 2}, "left_scale": 0.5, "right_scale": 1.25}}
RAW = {"architecture": "Vakilorn", "vocab": 90, "width": 32, "norm": {"eps": 1e-6},
       "embedding": {"scale": 3.0, "bigram": {"buckets": 13, "mul_prev": 5, "mul_cur": 3}},
       "layers": [
           {**copy.deepcopy(_REC), "weights_of": 2},
           {"type": "latent_attention", "mlp": None,
            "mixer": {"heads": 2, "dim": 8, "rot_dim": 4, "vdim": 6, "kv_rank": 10, "scale": 0.3,
                      "mask": {"size": 5},
                      "rot": {"base": 100.0, "dims": 4,
                              "scaling": {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 1.0}}}},
           copy.deepcopy(_REC),
           {"type": "parallel_2", "mlp": {"kind": "dense", "ff": 12, "limit": 1.0},
            "mixer": {"left": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 4, "scale": 0.3,
                               "rot": {"base": 50.0, "dims": 8, "scaling": {"factor": 4.0}}},
                      "right": {"heads": 3, "dim": 4, "vdim": 6, "gate_cap": 9.0},
                      "left_scale": 1.5, "right_scale": 0.25}}]}


def test_registry_and_structure():
    arch = lookup(RAW)
    cfg = arch.config_class.from_dict(RAW)
    assert arch.name == "Vakilorn" and cfg.to_dict()["layers"] == RAW["layers"]
    order = cfg.run_order()
    assert [e.layer for e in order] == [1, 0, 1, 2]          # layer 0 runs layer 2's parts
    assert [e.cache_layer for e in order] == [0, 1, 2, 3] and all(e.writes_cache for e in order)
    specs = cfg.layer_specs()
    assert [s.arrangement for s in specs] == ["branch_norm"] * 3
    assert [s.mixer.kind for s in specs] == ["latent_attention", "side_by_side", "side_by_side"]
    assert [s.feed_forward.kind for s in specs] == ["none", "gated_mlp", "gated_mlp"]
    assert specs[1].prefix == "l2." and specs[1].norms["mixer"].params["offset"] == 1.0
    lat = specs[0].mixer.params
    assert lat["q_rank"] is None and lat["rot_layout"] == "interleaved" and lat["value_gate"]
    assert lat["window"] == 5 and lat["rot_scaling"]["original"] == 16
    rec = specs[1].mixer.params
    assert rec["left_scale"] == 0.5 and rec["right"].kind == "gated_linear_recurrence"
    left = rec["left"].params
    assert left["qk_norm"] == "head" and left["bias"] and left["sink"] and not left.get("value_gate")
    assert rec["right"].params["decay_constant"] == 8.0 and rec["right"].params["taps"] == 2
    mem = specs[2].mixer.params
    assert mem["left"].params["qk_norm"] == "head_after" and mem["left"].params["rot_factor"] == 4.0
    assert mem["left"].params["value_gate"] and mem["right"].params["gate_cap"] == 9.0
    ff = specs[2].feed_forward.params
    assert ff["limit"] == 1.0 and ff["act_alpha"] == 1.702 and ff["up_shift"] == 1.0
    assert cfg.embedding_spec().params["scale"] == 3.0 and cfg.head_spec().params["weights"] == "embed"
    exp = arch.expected_tensors(cfg)
    assert not any(k.startswith("l0.") for k in exp)
    assert exp["bigram"].shape == (14, 32) and exp["l1.mix.dkv"].shape == (14, 32)
    assert exp["l1.mix.q"].shape == (24, 32) and exp["l1.mix.g"].shape == (12, 32) and "l1.norm2" not in exp
    assert exp["l2.mix.left.q.norm"].shape == (6,) and exp["l2.mix.left.k.b"].shape == (12,)
    assert exp["l2.mix.right.ra"].shape == (3, 8, 8) and exp["l2.mix.right.conv"].shape == (24, 2)
    assert exp["l3.mix.left.g"].shape == (8, 32) and "l3.mix.left.q.b" not in exp
    assert exp["l3.mix.right.i"].shape == (3, 32) and exp["l3.mix.right.norm"].shape == (18,)


@pytest.mark.parametrize("change,where", [
    (lambda r: r["layers"][0].__setitem__("type", "attention"), "type"),
    (lambda r: r["layers"][0].__setitem__("weights_of", 0), "weights_of"),
    (lambda r: r["layers"][0].__setitem__("type", "parallel_2"), "another layer"),
    (lambda r: [r["layers"][i]["mixer"]["right"].__setitem__("blocks", 5) for i in (0, 2)], "blocks"),
    (lambda r: r["layers"][1]["mixer"]["rot"].__setitem__("dims", 6), "dims"),
    (lambda r: r["layers"][3]["mixer"]["left"]["rot"]["scaling"].__setitem__("original", 8), "scaling"),
    (lambda r: r["layers"][3]["mlp"].__setitem__("kind", "moe"), "kind"),
    (lambda r: r["embedding"].pop("scale"), "scale"),
    (lambda r: [r["layers"][i]["mixer"]["left"].__setitem__("kv_heads", 3) for i in (0, 2)], "kv_heads"),
])
def test_bad_configurations_are_named(change, where):
    raw = copy.deepcopy(RAW)
    change(raw)
    with pytest.raises(ConfigError) as err:
        lookup(raw).config_class.from_dict(raw)
    assert where in str(err.value)


def test_a_chain_of_shared_layers_leads_to_the_owner():
    raw = copy.deepcopy(RAW)
    raw["layers"].append({**copy.deepcopy(_REC), "weights_of": 0})      # 4 -> 0 -> 2
    cfg = lookup(raw).config_class.from_dict(raw)
    assert [e.layer for e in cfg.run_order()] == [1, 0, 1, 2, 1]
    assert [e.cache_layer for e in cfg.run_order()] == [0, 1, 2, 3, 4]
    raw["layers"][2]["weights_of"] = 4                                    # a circle
    with pytest.raises(ConfigError):
        lookup(raw).config_class.from_dict(raw)


def test_named_sizes_and_random_models(tmp_path):
    for name in ("vakilorn-tiny", "vakilorn-small", "vakilorn-wide"):
        arch, cfg = named_size(name)
        assert arch.name == "Vakilorn" and len(cfg.run_order()) == len(cfg.layers)
    arch, cfg = named_size("vakilorn-tiny")
    make_random_model(str(tmp_path), cfg, 3, torch.float32)
    raw, tensors = P.read_folder(str(tmp_path))
    assert set(tensors) == set(arch.expected_tensors(cfg))
    ids = [5, 17, 3, 3, 250, 0, 41, 9, 9, 9, 120]
    logits = P.forward(ids, tensors, raw)
    assert logits.shape == (len(ids), cfg.vocab) and bool(torch.isfinite(logits).all())
    # causal: a later token changes no earlier row
    other = P.forward(ids[:6] + [77] + ids[7:], tensors, raw)
    assert torch.allclose(logits[:6], other[:6], atol=1e-12) and not torch.allclose(logits[6:], other[6:])


def test_plain_mechanisms_are_consistent():
    g = torch.Generator().manual_seed(4)
    rn = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    # the matrix memory: the recurrent form against the sum over earlier tokens it stands for
    T, H, D, V = 9, 2, 4, 3
    q, k, v, i, f = rn(T, H, D), rn(T, H, D), rn(T, H, V), rn(T, H), -torch.rand(T, H, generator=g, dtype=torch.float64)
    o = P.matrix_memory_outputs(q, k, v, i, f)
    F = torch.cumsum(f, 0)
    for t in (0, 4, 8):
        logw = torch.stack([F[t] - F[s] + i[s] for s in range(t + 1)])          # [s, H]
        m = torch.maximum(logw.max(0).values, F[t])                               # the maximum starts at 0
        w = torch.exp(logw - m)
        num = torch.einsum("sh,shd,shv,hd->hv", w, k[:t + 1], v[:t + 1], q[t])
        den = torch.maximum(torch.einsum("sh,shd,hd->h", w, k[:t + 1], q[t]).abs(), torch.exp(-m)) + 1e-6
        assert torch.allclose(o[t], num / den[:, None], atol=1e-10)
    # the linear recurrence: unrolled
    u, r, gi, lam = rn(6, 5), torch.rand(6, 5, generator=g, dtype=torch.float64), torch.rand(6, 5, generator=g, dtype=torch.float64), rn(5)
    s = P.gated_recurrence_states(u, r, gi, lam)
    a = torch.exp(-8.0 * r * torch.nn.functional.softplus(lam))
    b = torch.sqrt(1 - a ** 2) * gi * u
    assert torch.allclose(s[2], a[2] * (a[1] * b[0] + b[1]) + b[2], atol=1e-12)
    # the convolution: the last tap is the current token's
    x, taps = rn(5, 2), rn(2, 3)
    y = P.causal_convolution(x, taps, torch.zeros(2, dtype=torch.float64))
    assert torch.allclose(y[0], taps[:, 2] * x[0]) and torch.allclose(y[3], taps[:, 0] * x[1] + taps[:, 1] * x[2] + taps[:, 2] * x[3])
    # a sink with a huge negative value changes nothing; scores are relative under rotation
    qq, kk, vv = rn(7, 2, 6), rn(7, 1, 6), rn(7, 1, 5)
    plain = P.masked_softmax_attention(qq, kk, vv, 0.5)
    assert torch.allclose(plain, P.masked_softmax_attention(qq, kk, vv, 0.5, sink=torch.tensor([-1e9, -1e9], dtype=torch.float64)))
    assert not torch.allclose(plain, P.masked_softmax_attention(qq, kk, vv, 0.5, sink=torch.zeros(2, dtype=torch.float64)))
    f8 = P.plain_frequencies(10.0, 6)
    for layout in ("half", "interleaved"):
        a0 = (P.turn(qq, torch.arange(7), f8, 6, layout)[5, 0] * P.turn(kk, torch.arange(7), f8, 6, layout)[2, 0]).sum()
        a1 = (P.turn(qq, torch.arange(7) + 11, f8, 6, layout)[5, 0] * P.turn(kk, torch.arange(7) + 11, f8, 6, layout)[2, 0]).sum()
        assert abs(float(a0 - a1)) < 1e-10
