"""Devalorn configuration: a decoder whose layers are listed one by one in ``config.json``.

Keys read (nothing else exists in the design):

``vocab``, ``width``   sizes of the token table / head and of the residual stream
``norm.eps``           epsilon of every root-mean-square norm
``layers[i]``          ``type`` (``parallel`` or ``attention``), ``mixer`` (the mixer's sizes and
                       constants) and ``mlp`` (``kind`` dense or moe with its sizes, or null for
                       a layer without a feed-forward)

A layer is a block whose two branches read the same stream, each through a norm of its own:
x <- x + mixer(norm1 x) + mlp(norm2 x).  ``parallel`` layers have two mixers side by side,
``mixer.left`` (rotary softmax attention over a sliding window that keeps the first tokens
visible, with a gate per head) and ``mixer.right`` (time mixing over a running state), summed
with the constants ``left_scale`` and ``right_scale``.  ``attention`` layers have softmax
attention over a sliding window with a norm over the whole query and key projections, a query
temperature that grows with the position and a distance bias; with ``mixer.kv_from: j`` the
layer has no key/value tensors and attends over what layer j cached.

The design names no position limit; a loaded model's limit is what its page pool holds
(``position_limit`` caps it).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List

from .base import ConfigError, LayerSpec, ModelConfig, PartSpec, RunEntry

_TYPES = ("parallel", "attention")
#: the distance bias of ``attention`` layers: slope_h = 2^(-SLOPE_BITS * (h + 1) / heads)
SLOPE_BITS = 8.0


def _int(d, key: str, where: str, minimum: int = 1) -> int:
    v = d.get(key) if isinstance(d, dict) else None
    if isinstance(v, bool) or not isinstance(v, int) or v < minimum:
        raise ConfigError(f"config.json: {where}.{key} must be an integer >= {minimum}, got {v!r}")
    return v


def _num(d, key: str, where: str) -> float:
    v = d.get(key) if isinstance(d, dict) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}.{key} must be a number, got {v!r}")
    return float(v)


def _check_attention(mx, where: str, rotary: bool) -> None:
    if not isinstance(mx, dict):
        raise ConfigError(f"config.json: {where} must be an object")
    for key in ("heads", "kv_heads", "dim", "vdim"):
        _int(mx, key, where)
    if mx["heads"] % mx["kv_heads"]:
        raise ConfigError(f"config.json: {where}.heads is no multiple of kv_heads")
    _num(mx, "scale", where)
    mask = mx.get("mask")
    if mask is not None:
        _int(mask, "size", where + ".mask")
        if "keep_first" in mask:
            _int(mask, "keep_first", where + ".mask", 0)
    if rotary and mx.get("rot") is not None:
        dims = _int(mx["rot"], "dims", where + ".rot", 0)
        _num(mx["rot"], "base", where + ".rot")
        if dims % 2 or dims > mx["dim"]:
            raise ConfigError(f"config.json: {where}.rot.dims must be even and at most dim, got {dims}")
    if not rotary and mx.get("q_temp") is not None:
        _num(mx["q_temp"], "coef", where + ".q_temp")
        _int(mx["q_temp"], "every", where + ".q_temp")


@dataclass(frozen=True)
class DevalornConfig(ModelConfig):
    vocab: int
    width: int
    eps: float
    layers: tuple                           # the raw layer entries, validated
    position_limit: int = 1 << 20
    raw: Dict[str, Any] = field(default_factory=dict, compare=False, repr=False)

    identifiers = ("Devalorn",)

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "DevalornConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        cfg = cls(vocab=_int(raw, "vocab", "config"), width=_int(raw, "width", "config"),
                  eps=_num(raw.get("norm"), "eps", "norm"), layers=tuple(copy.deepcopy(layers)),
                  position_limit=int(raw.get("position_limit", 1 << 20)), raw=copy.deepcopy(raw))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.eps < 0.0:
            raise ConfigError("config.json: norm.eps must not be negative")
        for i, entry in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(entry, dict) or entry.get("type") not in _TYPES:
                raise ConfigError(f"config.json: {where}.type must be one of {list(_TYPES)}")
            mx = entry.get("mixer")
            if not isinstance(mx, dict):
                raise ConfigError(f"config.json: {where}.mixer must be an object")
            if entry["type"] == "parallel":
                _check_attention(mx.get("left"), where + ".mixer.left", rotary=True)
                right = mx.get("right")
                _int(right, "heads", where + ".mixer.right")
                _int(right, "dim", where + ".mixer.right")
                _num(mx, "left_scale", where + ".mixer")
                _num(mx, "right_scale", where + ".mixer")
            else:
                _check_attention(mx, where + ".mixer", rotary=False)
                src = mx.get("kv_from")
                if src is not None:
                    if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < i:
                        raise ConfigError(f"config.json: {where}.mixer.kv_from must name an earlier "
                                          f"layer, got {src!r}")
                    other = self.layers[src]
                    if other.get("type") != "attention" or other["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"config.json: {where}.mixer.kv_from names layer {src}, "
                                          f"which has no keys and values of its own kind")
                    if any(other["mixer"][k] != mx[k] for k in ("kv_heads", "dim", "vdim")):
                        raise ConfigError(f"config.json: {where}.mixer.kv_from: layer {src}'s "
                                          f"key/value heads differ from this layer's")
            mlp = entry.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                raise ConfigError(f"config.json: {where}.mlp.kind must be 'dense' or 'moe' (or mlp null)")
            if mlp["kind"] == "dense":
                _int(mlp, "ff", where + ".mlp")
            else:
                _int(mlp.get("expert"), "ff", where + ".mlp.expert")
                experts = _int(mlp.get("router"), "experts", where + ".mlp.router")
                if _int(mlp.get("router"), "top", where + ".mlp.router") > experts:
                    raise ConfigError(f"config.json: {where}.mlp.router.top exceeds experts")
                if mlp["router"].get("scale") is not None:
                    _num(mlp["router"], "scale", where + ".mlp.router")

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": "Devalorn", "vocab": self.vocab, "width": self.width,
                               "norm": {"eps": self.eps},
                               "layers": copy.deepcopy(list(self.layers))}
        if self.position_limit != 1 << 20:
            out["position_limit"] = self.position_limit
        return out

    # ---------------------------------------------------------------- structure
    def _attention_spec(self, mx, p: str, rotary: bool) -> PartSpec:
        mask, rot, temp = mx.get("mask") or {}, mx.get("rot") or {}, mx.get("q_temp")
        shares = mx.get("kv_from") is not None
        weights = {"q": p + "q", "out": p + "o"}
        if not shares:
            weights.update({"k": p + "k", "v": p + "v"})
        params = {"width": self.width, "heads": mx["heads"], "kv_heads": mx["kv_heads"],
                  "dim": mx["dim"], "vdim": mx["vdim"], "scale": float(mx["scale"]),
                  "eps": self.eps, "window": mask.get("size"),
                  "keep_first": mask.get("keep_first", 0), "shares_cache": shares,
                  "weights": weights}
        if rotary:
            params.update({"rot_dims": rot.get("dims", 0), "rot_base": float(rot.get("base", 10000.0)),
                           "head_gate": True})
            weights["gate"] = p + "g"
        else:
            params.update({"qk_norm": True, "slope_bits": SLOPE_BITS,
                           "q_temp": (float(temp["coef"]), int(temp["every"])) if temp else None})
            weights["q_norm"] = p + "q.norm"
            if not shares:
                weights["k_norm"] = p + "k.norm"
        return PartSpec("window_attention", params)

    def layer_specs(self) -> List[LayerSpec]:
        specs = []
        for i, entry in enumerate(self.layers):
            p = f"l{i}."
            mx, mlp = entry["mixer"], entry.get("mlp")
            if entry["type"] == "parallel":
                r = p + "mix.right."
                right = PartSpec("time_mix", {
                    "width": self.width, "heads": mx["right"]["heads"], "dim": mx["right"]["dim"],
                    "eps": self.eps,
                    "weights": {"r": r + "r", "k": r + "k", "v": r + "v", "g": r + "g",
                                "w1": r + "w1", "w2": r + "w2", "w0": r + "w0", "u": r + "u",
                                "norm": r + "norm", "out": r + "o",
                                **{"mu_" + s: r + "mu." + s for s in "rkvgw"}}})
                mixer = PartSpec("side_by_side", {
                    "left": self._attention_spec(mx["left"], p + "mix.left.", rotary=True),
                    "right": right, "left_scale": float(mx["left_scale"]),
                    "right_scale": float(mx["right_scale"])})
            else:
                mixer = self._attention_spec(mx, p + "mix.", rotary=False)
            norms = {"mixer": PartSpec("rms_norm", {"weight": p + "norm1", "eps": self.eps,
                                                    "size": self.width})}
            if mlp is None:
                ff = PartSpec("none", {})
            else:
                norms["feed_forward"] = PartSpec("rms_norm", {"weight": p + "norm2", "eps": self.eps,
                                                              "size": self.width})
                if mlp["kind"] == "dense":
                    ff = PartSpec("gated_mlp", {
                        "width": self.width, "inner": mlp["ff"],
                        "weights": {"gate": p + "mlp.gate", "up": p + "mlp.up",
                                    "down": p + "mlp.down"}})
                else:
                    ff = PartSpec("gated_moe", {
                        "prefix": p + "mlp.", "width": self.width,
                        "experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
                        "inner": mlp["expert"]["ff"], "limit": 0.0, "act_alpha": 1.0,
                        "up_shift": 0.0, "score": "softmax", "renormalize": False,
                        "router_scale": float(mlp["router"].get("scale", 1.0)),
                        "router_bias": False})
            specs.append(LayerSpec(prefix=p, arrangement="parallel", mixer=mixer, feed_forward=ff,
                                   norms=norms, width=self.width))
        return specs

    def run_order(self) -> List[RunEntry]:
        """Layers in order; a layer with ``kv_from`` reads the cache of the layer it names."""
        order = []
        for i, entry in enumerate(self.layers):
            src = entry["mixer"].get("kv_from") if entry["type"] == "attention" else None
            order.append(RunEntry(i, i) if src is None else RunEntry(i, src, writes_cache=False))
        return order

    def embedding_spec(self) -> PartSpec:
        return PartSpec("scaled_token_embedding", {"weights": "embed", "vocab": self.vocab,
                                                   "width": self.width, "scale": 1.0})

    def final_norm_spec(self) -> PartSpec:
        return PartSpec("rms_norm", {"weight": "final.norm", "eps": self.eps, "size": self.width})

    def head_spec(self) -> PartSpec:
        return PartSpec("linear_head", {"weights": "head", "vocab": self.vocab,
                                        "width": self.width})

    @property
    def max_positions(self) -> int:
        return self.position_limit
