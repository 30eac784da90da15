"""Devalorn as data for the engine: tensor names and shapes, random initialisation, named
sizes, registration.  The model is put together by
:func:`pretrained_rstr_b200.models.assembly.build_model` from the parts that
``DevalornConfig.layer_specs()`` names, in the order ``run_order()`` gives.

Tensor names: ``embed`` and ``head`` [vocab, width], ``final.norm`` [width] and per layer i
``l<i>.norm1``, ``l<i>.norm2`` [width] (the second only with a feed-forward), the mixer's
``l<i>.mix.*`` (``.left.*`` and ``.right.*`` in a parallel layer) and the feed-forward's
``l<i>.mlp.*``; matrices are [out, in].
"""
from __future__ import annotations

import math
from typing import Dict

import torch

from ..config.devalorn import DevalornConfig
from ..config.registry import Architecture, register_architecture
from ..weights.loader import TensorExpectation, normal

#: rows of the low-rank matrix inside the decay when a model is made from a named size (a
#: loaded model's rank is the shape of its tensor)
DECAY_RANK = 16


def _attention_tensors(exp, p: str, mx, d: int, rotary: bool) -> None:
    h, g, dim, vd = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    exp[p + "q"] = TensorExpectation((h * dim, d))
    exp[p + "o"] = TensorExpectation((d, h * vd))
    own = mx.get("kv_from") is None
    if own:
        exp[p + "k"] = TensorExpectation((g * dim, d))
        exp[p + "v"] = TensorExpectation((g * vd, d))
    if rotary:
        exp[p + "g"] = TensorExpectation((h, d))
    else:
        exp[p + "q.norm"] = TensorExpectation((h * dim,))
        if own:
            exp[p + "k.norm"] = TensorExpectation((g * dim,))


def expected_tensors(cfg: DevalornConfig, decay_rank=None) -> Dict[str, TensorExpectation]:
    """``decay_rank``: rows of ``w1`` (None: any number; the file's tensor decides)."""
    d = cfg.width
    exp: Dict[str, TensorExpectation] = {
        "embed": TensorExpectation((cfg.vocab, d)),
        "head": TensorExpectation((cfg.vocab, d)),
        "final.norm": TensorExpectation((d,)),
    }
    for i, entry in enumerate(cfg.layers):
        p = f"l{i}."
        mx, mlp = entry["mixer"], entry.get("mlp")
        exp[p + "norm1"] = TensorExpectation((d,))
        if entry["type"] == "parallel":
            _attention_tensors(exp, p + "mix.left.", mx["left"], d, rotary=True)
            r, h, dim = p + "mix.right.", mx["right"]["heads"], mx["right"]["dim"]
            for s in "rkvgw":
                exp[r + "mu." + s] = TensorExpectation((d,))
            for s in "rkvg":
                exp[r + s] = TensorExpectation((h * dim, d))
            rank = DECAY_RANK if decay_rank is None else decay_rank
            exp[r + "w1"] = TensorExpectation((rank, d), free_dims=(0,) if decay_rank is None else ())
            exp[r + "w2"] = TensorExpectation((h * dim, rank), free_dims=(1,) if decay_rank is None else ())
            exp[r + "w0"] = TensorExpectation((h * dim,))
            exp[r + "u"] = TensorExpectation((h, dim))
            exp[r + "norm"] = TensorExpectation((h * dim,))
            exp[r + "o"] = TensorExpectation((d, h * dim))
        else:
            _attention_tensors(exp, p + "mix.", mx, d, rotary=False)
        if mlp is None:
            continue
        exp[p + "norm2"] = TensorExpectation((d,))
        if mlp["kind"] == "dense":
            exp[p + "mlp.gate"] = TensorExpectation((mlp["ff"], d))
            exp[p + "mlp.up"] = TensorExpectation((mlp["ff"], d))
            exp[p + "mlp.down"] = TensorExpectation((d, mlp["ff"]))
        else:
            n, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            for e in range(n):
                exp[f"{p}mlp.e{e}.gate"] = TensorExpectation((ff, d))
                exp[f"{p}mlp.e{e}.up"] = TensorExpectation((ff, d))
                exp[f"{p}mlp.e{e}.down"] = TensorExpectation((d, ff))
            exp[p + "mlp.router"] = TensorExpectation((n, d))
    return exp


def random_tensors(cfg: DevalornConfig, seed: int) -> Dict[str, torch.Tensor]:
    """Seeded initialisation: matrices N(0, 1/in), the token table N(0, 1), norm weights 1 +
    N(0, 0.1), blend weights N(0.5, 0.2) kept inside [0, 1], decay offsets N(-1.5, 1) (decays
    between about 0.3 and 0.99), bonuses N(0, 0.5), routers N(0, 4/in) (scores that spread),
    head gates N(0, 4/in); every tensor from a generator of its own."""
    out: Dict[str, torch.Tensor] = {}
    for name, exp in expected_tensors(cfg, DECAY_RANK).items():
        last = name.rsplit(".", 1)[-1]
        if name == "embed":
            out[name] = normal(seed, name, exp.shape, 1.0)
        elif last in ("norm", "norm1", "norm2"):
            out[name] = normal(seed, name, exp.shape, 0.1, mean=1.0)
        elif ".mu." in name:
            out[name] = normal(seed, name, exp.shape, 0.2, mean=0.5).clamp_(0.0, 1.0)
        elif last == "w0":
            out[name] = normal(seed, name, exp.shape, 1.0, mean=-1.5)
        elif last == "u":
            out[name] = normal(seed, name, exp.shape, 0.5)
        elif last in ("router", "g") and exp.shape[0] < exp.shape[-1] and ".right." not in name:
            out[name] = normal(seed, name, exp.shape, 2.0 / math.sqrt(exp.shape[-1]))
        else:
            out[name] = normal(seed, name, exp.shape, 1.0 / math.sqrt(exp.shape[-1]))
    return out


def _left(heads, kv_heads, dim, vdim, window, keep_first, rot_dims=None, base=10000.0):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
            "scale": 1.0 / math.sqrt(dim), "mask": {"size": window, "keep_first": keep_first},
            "rot": {"base": base, "dims": dim if rot_dims is None else rot_dims}}


def _parallel(left, right_heads, right_dim, mlp, left_scale=0.7, right_scale=1.1):
    return {"type": "parallel",
            "mixer": {"left": left, "right": {"heads": right_heads, "dim": right_dim},
                      "left_scale": left_scale, "right_scale": right_scale},
            "mlp": mlp}


def _attention(heads, kv_heads, dim, vdim, window, mlp, coef=0.4, every=32, kv_from=None):
    mx = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
          "scale": 1.0 / math.sqrt(dim), "mask": {"size": window},
          "q_temp": {"coef": coef, "every": every}}
    if kv_from is not None:
        mx["kv_from"] = kv_from
    return {"type": "attention", "mixer": mx, "mlp": mlp}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff, scale=1.5):
    return {"kind": "moe", "router": {"experts": experts, "top": top, "scale": scale},
            "expert": {"ff": ff}}


def _sized(vocab, width, layers, eps=1e-6):
    return {"architecture": "Devalorn", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": layers}


#: Sizes a random-weight model can be asked for by name.  ``devalorn-small`` has the width, head
#: count, vocabulary and number of layers of GPT-2 small: parallel layers (12 attention heads of
#: 64 on 4 key/value heads over a window of 512 that keeps 16 first tokens, beside 12 time-mixing
#: heads of 64) with a gated feed-forward of 2,048 alternate with attention layers (window 1,024)
#: with 8 experts of 1,024 of which 2 run; every second attention layer shares the cache of the
#: one before.  ``devalorn-wide`` has GPT-2 XL's width with heads of 128.
NAMED_SIZES = {
    "devalorn-tiny": _sized(320, 64, [
        _parallel(_left(4, 2, 16, 24, 24, 5, rot_dims=8), 2, 16, _dense(96)),
        _attention(2, 1, 24, 16, 40, _moe(5, 2, 24), coef=0.3, every=8),
        _parallel(_left(2, 2, 24, 8, 12, 0), 4, 8, _moe(3, 1, 40), left_scale=1.2, right_scale=0.6),
        _attention(2, 1, 24, 16, 18, None, coef=0.6, every=5, kv_from=1)]),
    "devalorn-small": _sized(50257, 768, [
        layer for j in range(3) for layer in (
            _parallel(_left(12, 4, 64, 64, 512, 16), 12, 64, _dense(2048)),
            _attention(12, 4, 64, 64, 1024, _moe(8, 2, 1024)),
            _parallel(_left(12, 4, 64, 64, 512, 16), 12, 64, _dense(2048)),
            _attention(12, 4, 64, 64, 1024, _moe(8, 2, 1024), kv_from=4 * j + 1))]),
    "devalorn-wide": _sized(50257, 1600, [
        layer for j in range(3) for layer in (
            _parallel(_left(25, 5, 128, 128, 512, 16), 25, 64, _dense(4096)),
            _attention(25, 5, 128, 128, 1024, _moe(8, 2, 2048)),
            _parallel(_left(25, 5, 128, 128, 512, 16), 25, 64, _dense(4096)),
            _attention(25, 5, 128, 128, 1024, _moe(8, 2, 2048), kv_from=4 * j + 1))]),
}


def build(cfg: DevalornConfig, store, runtime):
    from .assembly import build_model
    return build_model(cfg, store, runtime)


ARCHITECTURE = Architecture(
    name="Devalorn",
    config_class=DevalornConfig,
    build=build,
    expected_tensors=expected_tensors,
    random_tensors=random_tensors,
    named_sizes=NAMED_SIZES,
)
register_architecture(DevalornConfig.identifiers, ARCHITECTURE)
