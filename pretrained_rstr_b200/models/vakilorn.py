"""Vakilorn as data for the engine: tensor names and shapes, random initialisation, named
sizes, registration.  The model is put together by
:func:`pretrained_rstr_b200.models.assembly.build_model` from the parts that
``VakilornConfig.layer_specs()`` names, in the order ``run_order()`` gives.

Tensor names: ``embed`` [vocab, width] (the head too), ``bigram`` [buckets + 1, width],
``final.norm`` [width] and, per layer i that has tensors of its own, ``l<i>.norm1``,
``l<i>.norm2`` [width] (the second only with a feed-forward), the mixer's ``l<i>.mix.*``
(``.left.*`` and ``.right.*`` in layers with two mixers) and the feed-forward's ``l<i>.mlp.*``;
matrices are [out, in], biases carry ``.b``.
"""
from __future__ import annotations

import math
from typing import Dict

import torch

from ..config.registry import Architecture, register_architecture
from ..config.vakilorn import VakilornConfig
from ..weights.loader import TensorExpectation, normal


def _left_tensors(exp, p: str, mx, d: int, second: bool) -> None:
    h, g, dim, vd = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    exp[p + "q"] = TensorExpectation((h * dim, d))
    exp[p + "k"] = TensorExpectation((g * dim, d))
    exp[p + "v"] = TensorExpectation((g * vd, d))
    exp[p + "sink"] = TensorExpectation((h,))
    exp[p + "o"] = TensorExpectation((d, h * vd))
    if second:
        exp[p + "g"] = TensorExpectation((h * vd, d))
    else:
        exp[p + "q.b"] = TensorExpectation((h * dim,))
        exp[p + "k.b"] = TensorExpectation((g * dim,))
        exp[p + "v.b"] = TensorExpectation((g * vd,))
        exp[p + "q.norm"] = TensorExpectation((dim,))
        exp[p + "k.norm"] = TensorExpectation((dim,))


def expected_tensors(cfg: VakilornConfig) -> Dict[str, TensorExpectation]:
    d = cfg.width
    exp: Dict[str, TensorExpectation] = {
        "embed": TensorExpectation((cfg.vocab, d)),
        "final.norm": TensorExpectation((d,)),
    }
    bg = cfg.embedding.get("bigram")
    if bg is not None:
        exp["bigram"] = TensorExpectation((bg["buckets"] + 1, d))
    for i in cfg.own_layers():
        entry = cfg.layers[i]
        p = f"l{i}."
        mx, mlp = entry["mixer"], entry.get("mlp")
        exp[p + "norm1"] = TensorExpectation((d,))
        if entry["type"] == "latent_attention":
            m = p + "mix."
            h, hd = mx["heads"], mx["dim"] + mx["rot_dim"]
            exp[m + "q"] = TensorExpectation((h * hd, d))
            exp[m + "dkv"] = TensorExpectation((mx["kv_rank"] + mx["rot_dim"], d))
            exp[m + "dkv.norm"] = TensorExpectation((mx["kv_rank"],))
            exp[m + "uk"] = TensorExpectation((h * mx["dim"], mx["kv_rank"]))
            exp[m + "uv"] = TensorExpectation((h * mx["vdim"], mx["kv_rank"]))
            exp[m + "g"] = TensorExpectation((h * mx["vdim"], d))
            exp[m + "o"] = TensorExpectation((d, h * mx["vdim"]))
        else:
            _left_tensors(exp, p + "mix.left.", mx["left"], d, entry["type"] == "parallel_2")
            r, right = p + "mix.right.", mx["right"]
            if entry["type"] == "parallel":
                w, b = right["width"], right["blocks"]
                for s in "yx":
                    exp[r + s] = TensorExpectation((w, d))
                    exp[r + s + ".b"] = TensorExpectation((w,))
                exp[r + "conv"] = TensorExpectation((w, right["conv"]))
                exp[r + "conv.b"] = TensorExpectation((w,))
                for s in ("ra", "ri"):
                    exp[r + s] = TensorExpectation((b, w // b, w // b))
                    exp[r + s + ".b"] = TensorExpectation((b, w // b))
                exp[r + "lam"] = TensorExpectation((w,))
                exp[r + "o"] = TensorExpectation((d, w))
            else:
                h, dim, vd = right["heads"], right["dim"], right["vdim"]
                exp[r + "q"] = TensorExpectation((h * dim, d))
                exp[r + "k"] = TensorExpectation((h * dim, d))
                exp[r + "v"] = TensorExpectation((h * vd, d))
                exp[r + "g"] = TensorExpectation((h * vd, d))
                exp[r + "o"] = TensorExpectation((d, h * vd))
                exp[r + "norm"] = TensorExpectation((h * vd,))
                for s in "if":
                    exp[r + s] = TensorExpectation((h, d))
                    exp[r + s + ".b"] = TensorExpectation((h,))
        if mlp is None:
            continue
        exp[p + "norm2"] = TensorExpectation((d,))
        exp[p + "mlp.gate"] = TensorExpectation((mlp["ff"], d))
        exp[p + "mlp.up"] = TensorExpectation((mlp["ff"], d))
        exp[p + "mlp.down"] = TensorExpectation((d, mlp["ff"]))
    return exp


def random_tensors(cfg: VakilornConfig, seed: int) -> Dict[str, torch.Tensor]:
    """Seeded initialisation: matrices N(0, 1/in), the token table N(0, 1/width) (the
    embedding's constant brings its rows to the stream's size), pair rows N(0, 1), the layers'
    norm weights N(0, 0.1) (they are stored around zero), the other norm weights 1 + N(0, 0.1),
    biases and sinks N(0, 0.5), convolution taps N(0, 0.5), the recurrence's lambda N(-3, 1)
    (decays between about 0.5 and 0.99), forget-gate biases N(3, 1); every tensor from a
    generator of its own."""
    out: Dict[str, torch.Tensor] = {}
    for name, exp in expected_tensors(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if name == "embed":
            out[name] = normal(seed, name, exp.shape, 1.0 / math.sqrt(cfg.width))
        elif name == "bigram":
            out[name] = normal(seed, name, exp.shape, 1.0)
        elif last in ("norm1", "norm2") or name == "final.norm":
            out[name] = normal(seed, name, exp.shape, 0.1)
        elif last == "norm":
            out[name] = normal(seed, name, exp.shape, 0.1, mean=1.0)
        elif last == "lam":
            out[name] = normal(seed, name, exp.shape, 1.0, mean=-3.0)
        elif name.endswith(".f.b"):
            out[name] = normal(seed, name, exp.shape, 1.0, mean=3.0)
        elif last in ("b", "sink", "conv"):
            out[name] = normal(seed, name, exp.shape, 0.5)
        else:
            out[name] = normal(seed, name, exp.shape, 1.0 / math.sqrt(exp.shape[-1]))
    return out


def _left(heads, kv_heads, dim, vdim, rot_dims=None, base=10000.0, factor=None):
    rot = {"base": base, "dims": dim if rot_dims is None else rot_dims}
    if factor is not None:
        rot["scaling"] = {"factor": factor}
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
            "scale": 1.0 / math.sqrt(dim), "rot": rot}


def _dense(ff, limit=7.0):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _recurrent(left, inner, blocks, taps, mlp, left_scale=0.8, right_scale=0.6):
    return {"type": "parallel",
            "mixer": {"left": left, "right": {"width": inner, "blocks": blocks, "conv": taps},
                      "left_scale": left_scale, "right_scale": right_scale},
            "mlp": mlp}


def _memory(left, heads, dim, vdim, mlp, cap=15.0, left_scale=1.1, right_scale=0.7):
    return {"type": "parallel_2",
            "mixer": {"left": left,
                      "right": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap},
                      "left_scale": left_scale, "right_scale": right_scale},
            "mlp": mlp}


def _latent(heads, dim, rot_dim, vdim, rank, window, mlp, base=10000.0, factor=8.0,
            original=256, fast=32.0, slow=1.0):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
                      "scale": 1.0 / math.sqrt(dim + rot_dim), "mask": {"size": window},
                      "rot": {"base": base, "dims": rot_dim,
                              "scaling": {"factor": factor, "original": original, "fast": fast,
                                          "slow": slow}}},
            "mlp": mlp}


def _shared(layer, src):
    return {**layer, "weights_of": src}


def _sized(vocab, width, layers, buckets, eps=1e-6):
    return {"architecture": "Vakilorn", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"scale": math.sqrt(width),
                          "bigram": {"buckets": buckets, "mul_prev": 31, "mul_cur": 5}},
            "layers": layers}


def _small_layers(width, heads, kv_heads, dim, ff, rank, depth):
    rec = _recurrent(_left(heads, kv_heads, dim, dim), width, 4 if width % 16 else 16, 4, _dense(ff))
    mem = _memory(_left(heads, kv_heads, dim, dim, factor=4.0), heads, dim, dim, _dense(ff))
    lat = _latent(heads, dim, dim // 2, dim, rank, 512, _dense(ff))
    return [layer for _ in range(depth // 4) for layer in (rec, lat, mem, lat)]


#: Sizes a random-weight model can be asked for by name.  ``vakilorn-small`` has the width, head
#: count, vocabulary and number of layers of GPT-2 small: a recurrent layer (12 attention heads
#: of 64 on 4 key/value heads beside a linear recurrence over 768 channels), a latent-attention
#: layer (heads of 64 + 32 over a latent of 256, window 512) and a matrix-memory layer (the same
#: attention with a gate, beside 12 memory heads of 64 x 64) take turns, every layer with a
#: gated feed-forward of 2,048.  ``vakilorn-wide`` has GPT-2 XL's width with heads of 128.
NAMED_SIZES = {
    "vakilorn-tiny": _sized(300, 64, [
        _recurrent(_left(4, 2, 16, 24, rot_dims=8), 48, 3, 3, _dense(96, 1.2)),
        _latent(2, 24, 8, 16, 40, 21, _dense(72, 0.9), original=64, factor=3.0, fast=16.0),
        _memory(_left(2, 1, 24, 8, factor=2.5), 3, 8, 24, None, cap=6.0),
        _shared(_recurrent(_left(4, 2, 16, 24, rot_dims=8), 48, 3, 3, _dense(96, 1.2)), 0)], 97),
    "vakilorn-small": _sized(50257, 768, _small_layers(768, 12, 4, 64, 2048, 256, 12), 8191),
    "vakilorn-wide": _sized(50257, 1600, _small_layers(1600, 25, 5, 128, 4096, 256, 12), 8191),
}


def build(cfg: VakilornConfig, store, runtime):
    from .assembly import build_model
    return build_model(cfg, store, runtime)


ARCHITECTURE = Architecture(
    name="Vakilorn",
    config_class=VakilornConfig,
    build=build,
    expected_tensors=expected_tensors,
    random_tensors=random_tensors,
    named_sizes=NAMED_SIZES,
)
register_architecture(VakilornConfig.identifiers, ARCHITECTURE)
