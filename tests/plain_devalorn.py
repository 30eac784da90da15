"""A plain, slow Devalorn: whole sequences at once, no cache, no kernels, one function per
mechanism.  The oracle the engine is compared with; it shares no code with the package.

Notation: x is the residual stream [T, width]; ``tensors`` is a dict name -> torch tensor;
``cfg`` is the raw ``config.json`` dict.  Everything is computed in ``dtype`` (float64 by
default) from the tensors' stored values.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import List, Optional

import torch


# ------------------------------------------------------------------------------ reading
def read_folder(folder: str):
    """(cfg, tensors) of a model folder, with a reader of its own for the tensor file: eight
    bytes of header length, the JSON header, then the data."""
    with open(os.path.join(folder, "config.json"), "r", encoding="utf-8") as fh:
        cfg = json.load(fh)
    with open(os.path.join(folder, "model.safetensors"), "rb") as fh:
        blob = fh.read()
    (n,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + n].decode("utf-8"))
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16,
             "I32": torch.int32, "F64": torch.float64}
    tensors = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        raw = bytearray(blob[8 + n + lo:8 + n + hi])
        t = torch.frombuffer(raw, dtype=kinds[info["dtype"]]) if raw else \
            torch.empty(0, dtype=kinds[info["dtype"]])
        tensors[name] = t.reshape(info["shape"]).clone()
    return cfg, tensors


# ---------------------------------------------------------------------------- mechanisms
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def weighted_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * weight.to(x.dtype)


def rotate_half(v: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """Coordinate i < dims/2 of the last axis pairs with i + dims/2; the pair at position p
    turns by p * base^(-2i/dims); coordinates from ``dims`` on stay.  v: [T, heads, n]."""
    if dims == 0:
        return v
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=v.dtype)
    angle = positions.to(v.dtype)[:, None, None] * freq
    c, s = torch.cos(angle), torch.sin(angle)
    a, b = v[..., :half], v[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, v[..., dims:]], dim=-1)


def window_mask(positions: torch.Tensor, n_keys: int, size: Optional[int], keep_first: int = 0):
    """[len(positions), n_keys] bool: the query at position i sees key j <= i that is fewer
    than ``size`` back, or one of the first ``keep_first`` keys."""
    i = positions[:, None]
    j = torch.arange(n_keys)[None, :]
    near = (i - j < size) if size else torch.ones_like(i - j, dtype=torch.bool)
    return (j <= i) & (near | (j < keep_first))


def distance_slopes(heads: int, dtype) -> torch.Tensor:
    """Head h (from 0) loses 2^(-8 (h + 1) / heads) per token of distance."""
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=dtype)


def query_temperature(positions: torch.Tensor, coef: float, every: int, dtype) -> torch.Tensor:
    """1 + coef * ln(floor((p + 1) / every) + 1)."""
    return 1.0 + coef * torch.log(torch.div(positions + 1, every, rounding_mode="floor").to(dtype) + 1.0)


def masked_softmax_attention(q, k, v, mask, scale: float, positions=None, slopes=None):
    """q [T, H, d]; k [S, G, d]; v [S, G, dv]; mask [T, S]; key s stands at position s.  Head h
    reads key/value head h // (H / G).  With ``slopes`` a score loses slopes[h] * (position of
    the query - position of the key).  Returns [T, H, dv]."""
    t, heads, _ = q.shape
    per = heads // k.shape[1]
    out = []
    for h in range(heads):
        s = (q[:, h] @ k[:, h // per].T) * scale
        if slopes is not None:
            dist = positions[:, None] - torch.arange(k.shape[0])[None, :]
            s = s - slopes[h] * dist.to(s.dtype)
        s = s.masked_fill(~mask, float("-inf"))
        out.append(torch.softmax(s, dim=-1) @ v[:, h // per])
    return torch.stack(out, dim=1)


def gated_window_attention(h, tensors, prefix: str, mx: dict, positions=None, kv=None):
    """The left mixer of a parallel layer: rotary attention over a window that keeps the first
    tokens, each head times a sigmoid gate of the input, then the output matrix.  ``kv``: keys
    (rotated) and values of earlier tokens to go before this call's (for the tests of
    continuation); returns (result, (keys, values))."""
    dt = h.dtype
    t = h.shape[0]
    H, G, d, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    first = 0 if kv is None else kv[0].shape[0]
    pos = torch.arange(first, first + t) if positions is None else positions
    W = lambda n: tensors[prefix + n].to(dt)
    rot = mx.get("rot") or {"dims": 0, "base": 1.0}
    q = rotate_half((h @ W("q").T).reshape(t, H, d), pos, float(rot["base"]), int(rot["dims"]))
    k = rotate_half((h @ W("k").T).reshape(t, G, d), pos, float(rot["base"]), int(rot["dims"]))
    v = (h @ W("v").T).reshape(t, G, dv)
    if kv is not None:
        k, v = torch.cat([kv[0], k]), torch.cat([kv[1], v])
    mask_cfg = mx.get("mask") or {}
    mask = window_mask(pos, k.shape[0], mask_cfg.get("size"), mask_cfg.get("keep_first", 0))
    o = masked_softmax_attention(q, k, v, mask, float(mx["scale"]))
    gate = torch.sigmoid(h @ W("g").T)                       # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(t, H * dv) @ W("o").T, (k, v)


def biased_window_attention(h, tensors, prefix: str, mx: dict, eps: float, shared=None):
    """The mixer of an attention layer: norms over the whole query and key projections, a query
    temperature by position, a distance bias per head, a sliding window.  ``shared``: (keys,
    values) of the layer whose cache this one reads (it then has none of its own).  Returns
    (result, (keys, values))."""
    dt = h.dtype
    t = h.shape[0]
    H, G, d, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    pos = torch.arange(t)
    W = lambda n: tensors[prefix + n].to(dt)
    q = weighted_norm(h @ W("q").T, W("q.norm"), eps)
    temp = mx.get("q_temp")
    if temp:
        q = q * query_temperature(pos, float(temp["coef"]), int(temp["every"]), dt)[:, None]
    q = q.reshape(t, H, d)
    if shared is None:
        k = weighted_norm(h @ W("k").T, W("k.norm"), eps).reshape(t, G, d)
        v = (h @ W("v").T).reshape(t, G, dv)
    else:
        k, v = shared
    mask = window_mask(pos, t, (mx.get("mask") or {}).get("size"))
    o = masked_softmax_attention(q, k, v, mask, float(mx["scale"]), positions=pos,
                                 slopes=distance_slopes(H, dt))
    return o.reshape(t, H * dv) @ W("o").T, (k, v)


def shifted_blend(h: torch.Tensor, mu: torch.Tensor, before=None) -> torch.Tensor:
    """h_t + (h_(t-1) - h_t) * mu, the row before the first being ``before`` (zeros if None)."""
    first = torch.zeros_like(h[:1]) if before is None else before.reshape(1, -1).to(h.dtype)
    prev = torch.cat([first, h[:-1]])
    return h + (prev - h) * mu.to(h.dtype)


def decayed_outer_states(r, k, v, w, u, state=None, cancelled: Optional[list] = None):
    """r, k, w [T, H, d]; v [T, H, dv]; u [H, d].  Per head, S [d, dv] from zero (or ``state``):
    o_t = (S + diag(u) k_t v_t^T)^T r_t, then S <- diag(w_t) S + k_t v_t^T.  Returns (o [T, H,
    dv], last S [H, d, dv]).  ``cancelled`` receives, per token, the smallest ratio over the heads
    of |o_t| to the same sum of absolute terms: near zero, o_t is what large terms leave of one
    another, and its direction (all that a unit norm keeps) hangs on their last bits."""
    t, heads, d = r.shape
    S = torch.zeros(heads, d, v.shape[-1], dtype=r.dtype) if state is None else state.clone()
    out, ratios = [], []
    for i in range(t):
        kv = k[i][:, :, None] * v[i][:, None, :]
        M = S + u[:, :, None] * kv
        out.append(torch.einsum("hkv,hk->hv", M, r[i]))
        if cancelled is not None:
            bound = torch.einsum("hkv,hk->hv", M.abs(), r[i].abs())
            ratios.append((out[-1].norm(dim=-1) / bound.norm(dim=-1).clamp_min(1e-300)).min())
        S = w[i][:, :, None] * S + kv
    if cancelled is not None:
        cancelled.append(torch.stack(ratios))
    return torch.stack(out), S


def time_mix(h, tensors, prefix: str, mx: dict, eps: float, carried=None,
             cancelled: Optional[list] = None):
    """The right mixer of a parallel layer.  ``carried``: (last input row, state) of the tokens
    before; returns (result, (last input row, state))."""
    dt = h.dtype
    t = h.shape[0]
    H, d = mx["heads"], mx["dim"]
    W = lambda n: tensors[prefix + n].to(dt)
    before, state = (None, None) if carried is None else carried
    blend = {s: shifted_blend(h, W("mu." + s), before) for s in "rkvgw"}
    r = (blend["r"] @ W("r").T).reshape(t, H, d)
    k = (blend["k"] @ W("k").T).reshape(t, H, d)
    v = (blend["v"] @ W("v").T).reshape(t, H, d)
    z = blend["g"] @ W("g").T
    gate = z * torch.sigmoid(z)
    w = torch.exp(-torch.exp(torch.tanh(blend["w"] @ W("w1").T) @ W("w2").T + W("w0"))).reshape(t, H, d)
    o, state = decayed_outer_states(r, k, v, w, W("u"), state, cancelled)
    o = unit_rms(o, eps).reshape(t, H * d) * W("norm") * gate
    return o @ W("o").T, (h[-1].clone(), state)


def gated_unit(h, gate_w, up_w, down_w):
    z = h @ gate_w.T
    return ((z * torch.sigmoid(z)) * (h @ up_w.T)) @ down_w.T


def dense_feed_forward(h, tensors, prefix: str):
    dt = h.dtype
    return gated_unit(h, tensors[prefix + "gate"].to(dt), tensors[prefix + "up"].to(dt),
                      tensors[prefix + "down"].to(dt))


def softmax_routed_experts(h, tensors, prefix: str, mlp: dict, margins: Optional[list] = None):
    """Scores are the softmax of the router's logits over all experts; the ``top`` largest are
    chosen and weigh their experts by score times the router's constant, as they are.
    ``margins`` receives, per token, the gap between the last chosen logit and the next."""
    dt = h.dtype
    router = mlp["router"]
    n, top, factor = int(router["experts"]), int(router["top"]), float(router.get("scale", 1.0))
    z = h @ tensors[prefix + "router"].to(dt).T
    s = torch.softmax(z, dim=-1)
    order = torch.argsort(z, dim=-1, descending=True, stable=True)
    if margins is not None:
        zs = torch.gather(z, 1, order)
        margins.append((zs[:, top - 1] - zs[:, top]) if top < n else torch.full((h.shape[0],), math.inf, dtype=dt))
    out = torch.zeros_like(h)
    for i in range(h.shape[0]):
        for e in order[i, :top].tolist():
            p = f"{prefix}e{e}."
            out[i] += s[i, e] * factor * gated_unit(h[i:i + 1], tensors[p + "gate"].to(dt),
                                                    tensors[p + "up"].to(dt), tensors[p + "down"].to(dt))[0]
    return out


# --------------------------------------------------------------------------------- model
def forward(tokens: List[int], tensors, cfg: dict, dtype=torch.float64, taps: Optional[list] = None,
            margins: Optional[list] = None, cancelled: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence.  ``taps`` receives the stream after every layer;
    ``margins`` per routed layer the router's closest call per token; ``cancelled`` per time
    mixing how little of its terms each token's result keeps
    (:func:`decayed_outer_states`)."""
    eps = float(cfg["norm"]["eps"])
    x = tensors["embed"].to(dtype)[torch.tensor(tokens)]
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        mx, mlp = layer["mixer"], layer.get("mlp")
        h = weighted_norm(x, tensors[p + "norm1"], eps)
        if layer["type"] == "parallel":
            left, _ = gated_window_attention(h, tensors, p + "mix.left.", mx["left"])
            right, _ = time_mix(h, tensors, p + "mix.right.", mx["right"], eps, cancelled=cancelled)
            y = float(mx["left_scale"]) * left + float(mx["right_scale"]) * right
        else:
            src = mx.get("kv_from")
            y, kept[i] = biased_window_attention(h, tensors, p + "mix.", mx, eps,
                                                 shared=None if src is None else kept[src])
        if mlp is not None:
            h2 = weighted_norm(x, tensors[p + "norm2"], eps)
            if mlp["kind"] == "dense":
                y = y + dense_feed_forward(h2, tensors, p + "mlp.")
            else:
                y = y + softmax_routed_experts(h2, tensors, p + "mlp.", mlp, margins)
        x = x + y
        if taps is not None:
            taps.append(x.clone())
    return weighted_norm(x, tensors["final.norm"], eps) @ tensors["head"].to(dtype).T


def greedy(prompt: List[int], n_new: int, tensors, cfg: dict, dtype=torch.float64) -> List[int]:
    ids, out = list(prompt), []
    for _ in range(n_new):
        nxt = int(forward(ids, tensors, cfg, dtype)[-1].argmax())
        out.append(nxt)
        ids.append(nxt)
    return out
