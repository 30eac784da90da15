"""Vakilorn configuration: a decoder whose layers are listed one by one in ``config.json``.

Keys read (nothing else exists in the design):

``vocab``, ``width``   sizes of the token table (which is the head too) and of the residual stream
``norm.eps``           epsilon of every root-mean-square norm
``embedding``          ``scale`` (a constant on the token's row) and ``bigram`` (``buckets``,
                       ``mul_prev``, ``mul_cur``: a second table indexed by a hash of the
                       previous token and the token)
``layers[i]``          ``type`` (``parallel``, ``latent_attention`` or ``parallel_2``), ``mixer``
                       (the mixer's sizes and constants), ``mlp`` (``kind`` dense with ``ff`` and
                       ``limit``, or null for a layer without a feed-forward) and optionally
                       ``weights_of``: j, a layer that runs layer j's tensors with a cache and
                       state of its own

A layer norms each branch's RESULT: x <- x + norm1(mixer(x)), x <- x + norm2(mlp(x)); the
branches read the stream itself; the norms' weights are stored around zero (1 + w).
``parallel`` layers have two mixers side by side, ``mixer.left`` (causal softmax attention with
grouped key/value heads, biases, a norm per head on queries and keys before the rotation, and a
learned sink per head) and ``mixer.right`` (a gated linear recurrence per channel behind a short
convolution), summed with the constants ``left_scale`` and ``right_scale``.  ``parallel_2``
layers have attention without biases whose frequencies are divided by ``rot.scaling.factor``,
with a weightless norm per head after the rotation, a sink and a gate per value coordinate,
beside a matrix memory with exponential gates.  ``latent_attention`` layers attend over one
low-rank latent per token inside a sliding window, with interleaved rotary pairs, YaRN-scaled
frequencies and a gate per value coordinate.

The design names no position limit; a loaded model's limit is what its page pool holds
(``position_limit`` caps it).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError, LayerSpec, ModelConfig, PartSpec, RunEntry

_TYPES = ("parallel", "latent_attention", "parallel_2")
#: constants the design fixes
LRU_DECAY_CONSTANT = 8.0           # log a = -8 * r * softplus(lambda)
MLP_ACT_SLOPE = 1.702              # g * sigmoid(1.702 g)
MLP_UP_SHIFT = 1.0                 # ... * (u + 1)
NORM_OFFSET = 1.0                  # norms multiply by 1 + w


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


def _check_rot(rot, most: int, where: str, yarn: bool) -> None:
    dims = _int(rot, "dims", where, 0)
    _num(rot, "base", where)
    if dims % 2 or dims > most:
        raise ConfigError(f"config.json: {where}.dims must be even and at most {most}, got {dims}")
    sc = rot.get("scaling")
    if sc is None:
        return
    if _num(sc, "factor", where + ".scaling") <= 0.0:
        raise ConfigError(f"config.json: {where}.scaling.factor must be positive")
    if yarn:
        for key in ("original", "fast", "slow"):
            if _num(sc, key, where + ".scaling") <= 0.0:
                raise ConfigError(f"config.json: {where}.scaling.{key} must be positive")
    elif any(k in sc for k in ("original", "fast", "slow")):
        raise ConfigError(f"config.json: {where}.scaling: this attention divides its frequencies "
                          f"by a factor and has no other scaling")


def _check_left(mx, where: str) -> None:
    if not isinstance(mx, dict):
        raise ConfigError(f"config.json: {where} must be an object")
    for key in ("heads", "kv_heads", "dim", "vdim"):
        _int(mx, key, where)
    if mx["heads"] % mx["kv_heads"]:
        raise ConfigError(f"config.json: {where}.heads is no multiple of kv_heads")
    _num(mx, "scale", where)
    if mx.get("rot") is not None:
        _check_rot(mx["rot"], mx["dim"], where + ".rot", yarn=False)
    if mx.get("mask") is not None:
        _int(mx["mask"], "size", where + ".mask")


@dataclass(frozen=True)
class VakilornConfig(ModelConfig):
    vocab: int
    width: int
    eps: float
    embedding: Dict[str, Any]
    layers: tuple                           # the raw layer entries, validated
    position_limit: int = 1 << 20
    raw: Dict[str, Any] = field(default_factory=dict, compare=False, repr=False)

    identifiers = ("Vakilorn",)

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "VakilornConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        emb = raw.get("embedding")
        if not isinstance(emb, dict):
            raise ConfigError("config.json: 'embedding' must be an object")
        cfg = cls(vocab=_int(raw, "vocab", "config"), width=_int(raw, "width", "config"),
                  eps=_num(raw.get("norm"), "eps", "norm"), embedding=copy.deepcopy(emb),
                  layers=tuple(copy.deepcopy(layers)),
                  position_limit=int(raw.get("position_limit", 1 << 20)), raw=copy.deepcopy(raw))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.eps < 0.0:
            raise ConfigError("config.json: norm.eps must not be negative")
        _num(self.embedding, "scale", "embedding")
        bg = self.embedding.get("bigram")
        if bg is not None:
            _int(bg, "buckets", "embedding.bigram")
            _int(bg, "mul_prev", "embedding.bigram", 0)
            _int(bg, "mul_cur", "embedding.bigram", 0)
        for i, entry in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(entry, dict) or entry.get("type") not in _TYPES:
                raise ConfigError(f"config.json: {where}.type must be one of {list(_TYPES)}")
            src = entry.get("weights_of")
            mx = entry.get("mixer")
            if not isinstance(mx, dict) and src is None:
                raise ConfigError(f"config.json: {where}.mixer must be an object")
            if src is not None:
                if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < len(self.layers) \
                        or src == i:
                    raise ConfigError(f"config.json: {where}.weights_of must name another layer, "
                                      f"got {src!r}")
                seen = {i}
                while isinstance(self.layers[src], dict) and self.layers[src].get("weights_of") is not None:
                    seen.add(src)                 # (a layer that itself runs another's tensors)
                    src = self.layers[src]["weights_of"]
                    if isinstance(src, bool) or not isinstance(src, int) or \
                            not 0 <= src < len(self.layers) or src in seen:
                        raise ConfigError(f"config.json: {where}.weights_of leads to no layer with "
                                          f"tensors of its own")
                other = self.layers[src]
                if not isinstance(other, dict) or other.get("type") != entry.get("type"):
                    raise ConfigError(f"config.json: {where} uses layer {src}'s tensors but "
                                      f"describes another layer")
                continue            # (it runs layer src's parts, which are checked there)
            if entry["type"] in ("parallel", "parallel_2"):
                _check_left(mx.get("left"), where + ".mixer.left")
                right = mx.get("right")
                if entry["type"] == "parallel":
                    inner = _int(right, "width", where + ".mixer.right")
                    if inner % _int(right, "blocks", where + ".mixer.right"):
                        raise ConfigError(f"config.json: {where}.mixer.right.width is no multiple "
                                          f"of blocks")
                    _int(right, "conv", where + ".mixer.right")
                else:
                    for key in ("heads", "dim", "vdim"):
                        _int(right, key, where + ".mixer.right")
                    if _num(right, "gate_cap", where + ".mixer.right") <= 0.0:
                        raise ConfigError(f"config.json: {where}.mixer.right.gate_cap must be positive")
                _num(mx, "left_scale", where + ".mixer")
                _num(mx, "right_scale", where + ".mixer")
            else:
                for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank"):
                    _int(mx, key, where + ".mixer")
                _num(mx, "scale", where + ".mixer")
                if mx.get("rot") is not None:
                    _check_rot(mx["rot"], mx["rot_dim"], where + ".mixer.rot", yarn=True)
                if mx.get("mask") is not None:
                    _int(mx["mask"], "size", where + ".mixer.mask")
            mlp = entry.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                raise ConfigError(f"config.json: {where}.mlp.kind must be 'dense' (or mlp null)")
            _int(mlp, "ff", where + ".mlp")
            if _num(mlp, "limit", where + ".mlp") <= 0.0:
                raise ConfigError(f"config.json: {where}.mlp.limit must be positive")

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": "Vakilorn", "vocab": self.vocab, "width": self.width,
                               "norm": {"eps": self.eps},
                               "embedding": copy.deepcopy(self.embedding),
                               "layers": copy.deepcopy(list(self.layers))}
        if self.position_limit != 1 << 20:
            out["position_limit"] = self.position_limit
        return out

    # ---------------------------------------------------------------- structure
    def own_layers(self) -> List[int]:
        """Indices of the layers that have tensors of their own, in order."""
        return [i for i, e in enumerate(self.layers) if e.get("weights_of") is None]

    def _left_spec(self, mx, p: str, second: bool) -> PartSpec:
        rot, mask = mx.get("rot") or {}, mx.get("mask") or {}
        weights = {"q": p + "q", "k": p + "k", "v": p + "v", "out": p + "o", "sink": p + "sink"}
        params = {"width": self.width, "heads": mx["heads"], "kv_heads": mx["kv_heads"],
                  "dim": mx["dim"], "vdim": mx["vdim"], "scale": float(mx["scale"]),
                  "eps": self.eps, "window": mask.get("size"), "keep_first": 0,
                  "rot_dims": rot.get("dims", 0), "rot_base": float(rot.get("base", 10000.0)),
                  "rot_factor": float((rot.get("scaling") or {}).get("factor", 1.0)),
                  "sink": True, "weights": weights}
        if second:
            params.update({"qk_norm": "head_after", "value_gate": True})
            weights["gate"] = p + "g"
        else:
            params.update({"qk_norm": "head", "bias": True})
            weights.update({"q_norm": p + "q.norm", "k_norm": p + "k.norm", "q_bias": p + "q.b",
                            "k_bias": p + "k.b", "v_bias": p + "v.b"})
        return PartSpec("window_attention", params)

    def _mixer_spec(self, entry, p: str) -> PartSpec:
        mx = entry["mixer"]
        if entry["type"] == "latent_attention":
            rot = mx.get("rot") or {}
            m = p + "mix."
            return PartSpec("latent_attention", {
                "width": self.width, "heads": mx["heads"], "dim": mx["dim"],
                "rot_dim": mx["rot_dim"], "vdim": mx["vdim"], "kv_rank": mx["kv_rank"],
                "q_rank": None, "scale": float(mx["scale"]), "eps": self.eps,
                "rot_dims": rot.get("dims", mx["rot_dim"]) if rot else 0,
                "rot_base": float(rot.get("base", 10000.0)), "rot_layout": "interleaved",
                "rot_scaling": copy.deepcopy(rot.get("scaling")),
                "window": (mx.get("mask") or {}).get("size"), "value_gate": True,
                "weights": {"q": m + "q", "kv_down": m + "dkv", "kv_norm": m + "dkv.norm",
                            "k_up": m + "uk", "v_up": m + "uv", "gate": m + "g", "out": m + "o"}})
        r = p + "mix.right."
        right = mx["right"]
        if entry["type"] == "parallel":
            side = PartSpec("gated_linear_recurrence", {
                "width": self.width, "inner": right["width"], "blocks": right["blocks"],
                "taps": right["conv"], "decay_constant": LRU_DECAY_CONSTANT,
                "weights": {"y": r + "y", "y_bias": r + "y.b", "x": r + "x", "x_bias": r + "x.b",
                            "conv": r + "conv", "conv_bias": r + "conv.b", "gate_a": r + "ra",
                            "gate_a_bias": r + "ra.b", "gate_i": r + "ri", "gate_i_bias": r + "ri.b",
                            "lambda": r + "lam", "out": r + "o"}})
        else:
            side = PartSpec("matrix_memory", {
                "width": self.width, "heads": right["heads"], "dim": right["dim"],
                "vdim": right["vdim"], "gate_cap": float(right["gate_cap"]), "eps": self.eps,
                "weights": {"q": r + "q", "k": r + "k", "v": r + "v", "gate": r + "g",
                            "i": r + "i", "i_bias": r + "i.b", "f": r + "f", "f_bias": r + "f.b",
                            "norm": r + "norm", "out": r + "o"}})
        return PartSpec("side_by_side", {
            "left": self._left_spec(mx["left"], p + "mix.left.", entry["type"] == "parallel_2"),
            "right": side, "left_scale": float(mx["left_scale"]),
            "right_scale": float(mx["right_scale"])})

    def _norm_spec(self, name: str) -> PartSpec:
        return PartSpec("rms_norm", {"weight": name, "eps": self.eps, "size": self.width,
                                     "offset": NORM_OFFSET})

    def layer_specs(self) -> List[LayerSpec]:
        """One specification per layer that has tensors of its own (``run_order`` names them by
        their place in this list)."""
        specs = []
        for i in self.own_layers():
            entry = self.layers[i]
            p = f"l{i}."
            mlp = entry.get("mlp")
            norms = {"mixer": self._norm_spec(p + "norm1")}
            if mlp is None:
                ff = PartSpec("none", {})
            else:
                norms["feed_forward"] = self._norm_spec(p + "norm2")
                ff = PartSpec("gated_mlp", {
                    "width": self.width, "inner": mlp["ff"], "limit": float(mlp["limit"]),
                    "act_alpha": MLP_ACT_SLOPE, "up_shift": MLP_UP_SHIFT,
                    "weights": {"gate": p + "mlp.gate", "up": p + "mlp.up", "down": p + "mlp.down"}})
            specs.append(LayerSpec(prefix=p, arrangement="branch_norm",
                                   mixer=self._mixer_spec(entry, p), feed_forward=ff, norms=norms,
                                   width=self.width))
        return specs

    def run_order(self) -> List[RunEntry]:
        """Layers in order; a layer with ``weights_of`` runs the parts of the layer it names with
        a cache and state of its own (caches are numbered by the listed layer)."""
        place = {i: k for k, i in enumerate(self.own_layers())}
        return [RunEntry(place[self.tensors_of(i)], i) for i in range(len(self.layers))]

    def tensors_of(self, i: int) -> int:
        """The layer whose tensors layer i runs: itself, or where its ``weights_of`` leads."""
        while self.layers[i].get("weights_of") is not None:
            i = self.layers[i]["weights_of"]
        return i

    def layer_entry(self, i: int) -> Dict[str, Any]:
        """The entry whose sizes layer i runs with: its own, or, for a layer that runs another
        layer's tensors, that layer's (the tensors' shapes are that layer's)."""
        return self.layers[self.tensors_of(i)]

    def embedding_spec(self) -> PartSpec:
        bg = self.embedding.get("bigram")
        scale = float(self.embedding["scale"])
        if bg is None:
            return PartSpec("scaled_token_embedding", {"weights": "embed", "vocab": self.vocab,
                                                       "width": self.width, "scale": scale})
        return PartSpec("token_pair_embedding", {
            "table": "embed", "pairs": "bigram", "vocab": self.vocab, "width": self.width,
            "buckets": bg["buckets"], "mul_prev": bg["mul_prev"], "mul_cur": bg["mul_cur"],
            "scale": scale})

    def final_norm_spec(self) -> PartSpec:
        return self._norm_spec("final.norm")

    def head_spec(self) -> PartSpec:
        # the token table itself, without the embedding's constant
        return PartSpec("linear_head", {"weights": "embed", "vocab": self.vocab,
                                        "width": self.width})

    @property
    def max_positions(self) -> int:
        return self.position_limit
