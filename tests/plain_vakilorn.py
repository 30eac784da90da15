"""A plain, slow implementation of the Vakilorn design in float64 on the CPU: one function per
mechanism, written from the design's equations, with its own reader of model folders.  It
shares no code with the package; the GPU tests compare the engine with it.

Notation: T tokens of one sequence at positions 0..T-1; x the residual stream [T, width];
matrices are stored [out, in] and applied as ``h @ W.T``.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional

import numpy as np
import torch

F64 = torch.float64


# ----------------------------------------------------------------------- model folders
def read_folder(folder: str):
    """(config dict, {name: float64 / int32 tensor}) of a folder with config.json and
    model.safetensors (8-byte little-endian header length, a JSON header, the data)."""
    with open(os.path.join(folder, "config.json"), "r", encoding="utf-8") as fh:
        cfg = json.load(fh)
    with open(os.path.join(folder, "model.safetensors"), "rb") as fh:
        (n,) = struct.unpack("<Q", fh.read(8))
        header = json.loads(fh.read(n))
        blob = fh.read()
    tensors = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        raw = blob[lo:hi]
        kind = meta["dtype"]
        if kind == "BF16":
            bits = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            t = torch.from_numpy(bits.view(np.float32).copy()).to(F64)
        elif kind == "F32":
            t = torch.from_numpy(np.frombuffer(raw, dtype="<f4").copy()).to(F64)
        elif kind == "I32":
            t = torch.from_numpy(np.frombuffer(raw, dtype="<i4").copy())
        else:
            raise ValueError(f"{name}: element type {kind}")
        tensors[name] = t.reshape(meta["shape"])
    return cfg, tensors


# -------------------------------------------------------------------------- small pieces
def unit_rms(v: torch.Tensor, eps: float) -> torch.Tensor:
    """v / sqrt(mean(v^2) + eps) over the last axis."""
    return v / torch.sqrt(v.pow(2).mean(dim=-1, keepdim=True) + eps)


def offset_norm(v: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """A norm whose weight is stored around zero: unit_rms(v) * (1 + w)."""
    return unit_rms(v, eps) * (1.0 + w)


def tanh_gelu(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z.pow(3))))


# ----------------------------------------------------------------------------- rotations
def plain_frequencies(base: float, dims: int) -> torch.Tensor:
    return torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)


def yarn(base: float, dims: int, factor: float, original: float, fast: float, slow: float):
    """(frequencies, magnitude): pair i keeps its frequency where it turns fast and is
    interpolated (divided by ``factor``) where it turns slowly, with a linear ramp between."""
    def pair_of(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_of(fast)), 0)
    hi = min(math.ceil(pair_of(slow)), dims - 1)
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return torch.tensor(out, dtype=F64), 0.1 * math.log(factor) + 1.0


def turn(v: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor, dims: int, layout: str,
         magnitude: float = 1.0) -> torch.Tensor:
    """v [T, heads, n]: the first ``dims`` coordinates of every head turned by position x
    frequency; pairs (i, i + dims/2) in the "half" layout, (2i, 2i + 1) in "interleaved"."""
    if dims == 0:
        return v
    angle = positions.to(F64)[:, None, None] * freq[None, None, :]
    c, s = torch.cos(angle) * magnitude, torch.sin(angle) * magnitude
    out = v.clone()
    if layout == "half":
        a, b = v[..., :dims // 2], v[..., dims // 2:dims]
        out[..., :dims // 2] = a * c - b * s
        out[..., dims // 2:dims] = b * c + a * s
    else:
        a, b = v[..., 0:dims:2], v[..., 1:dims:2]
        out[..., 0:dims:2] = a * c - b * s
        out[..., 1:dims:2] = b * c + a * s
    return out


# ----------------------------------------------------------------------------- attention
def masked_softmax_attention(q, k, v, scale: float, sink: Optional[torch.Tensor] = None,
                             window: Optional[int] = None) -> torch.Tensor:
    """q [T, H, D], k [T, G, D], v [T, G, V] -> [T, H, V].  Query head h uses key/value head
    h // (H / G); position i sees j <= i (and i - j < window); exp(sink_h) joins the
    denominator once."""
    T, H, _ = q.shape
    G = k.shape[1]
    idx = torch.arange(T)
    seen = idx[None, :] <= idx[:, None]
    if window:
        seen = seen & ((idx[:, None] - idx[None, :]) < window)
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        score = (q[:, h] @ k[:, g].T) * scale
        score = score.masked_fill(~seen, -math.inf)
        top = score.max(dim=-1, keepdim=True).values
        if sink is not None:
            top = torch.maximum(top, sink[h].expand_as(top))
        w = torch.exp(score - top)
        total = w.sum(dim=-1, keepdim=True)
        if sink is not None:
            total = total + torch.exp(sink[h] - top)
        out[:, h] = (w / total) @ v[:, g]
    return out


def grouped_attention(W: Dict[str, torch.Tensor], p: str, mx: dict, h: torch.Tensor,
                      positions: torch.Tensor, eps: float, gated: bool) -> torch.Tensor:
    """The attention beside a recurrent mixer.  Ungated form: biases, a norm per head with a
    shared weight BEFORE the rotation.  Gated form: no biases, frequencies divided by a factor,
    a weightless norm per head AFTER the rotation, a gate per value coordinate."""
    H, G, D, V = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    T = h.shape[0]
    q, k, v = h @ W[p + "q"].T, h @ W[p + "k"].T, h @ W[p + "v"].T
    rot = mx.get("rot") or {"dims": 0, "base": 10000.0}
    dims = rot["dims"]
    freq = plain_frequencies(rot["base"], dims) if dims else None
    if not gated:
        q, k, v = q + W[p + "q.b"], k + W[p + "k.b"], v + W[p + "v.b"]
    q, k, v = q.reshape(T, H, D), k.reshape(T, G, D), v.reshape(T, G, V)
    if not gated:
        q = unit_rms(q, eps) * W[p + "q.norm"]
        k = unit_rms(k, eps) * W[p + "k.norm"]
        q, k = turn(q, positions, freq, dims, "half"), turn(k, positions, freq, dims, "half")
    else:
        if dims:
            freq = freq / float((rot.get("scaling") or {}).get("factor", 1.0))
        q, k = turn(q, positions, freq, dims, "half"), turn(k, positions, freq, dims, "half")
        q, k = unit_rms(q, eps), unit_rms(k, eps)
    o = masked_softmax_attention(q, k, v, mx["scale"], sink=W[p + "sink"],
                                 window=(mx.get("mask") or {}).get("size")).reshape(T, H * V)
    if gated:
        o = o * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def latent_attention(W, p: str, mx: dict, h, positions, eps: float) -> torch.Tensor:
    """Keys and values expanded from one normed latent per token, plus one rotated key part all
    heads share; a sliding window; an ordinary softmax; a gate per value coordinate."""
    T = h.shape[0]
    H, D, R, V, rank = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    q = (h @ W[p + "q"].T).reshape(T, H, D + R)
    down = h @ W[p + "dkv"].T
    c = unit_rms(down[:, :rank], eps) * W[p + "dkv.norm"]
    shared = down[:, rank:].reshape(T, 1, R)
    rot = mx.get("rot")
    if rot:
        sc = rot.get("scaling")
        if sc:
            freq, mag = yarn(rot["base"], rot["dims"], sc["factor"], sc["original"], sc["fast"], sc["slow"])
        else:
            freq, mag = plain_frequencies(rot["base"], rot["dims"]), 1.0
        q_rot = turn(q[..., D:], positions, freq, rot["dims"], "interleaved", mag)
        shared = turn(shared, positions, freq, rot["dims"], "interleaved", mag)
    else:
        q_rot = q[..., D:]
    keys = torch.cat([(c @ W[p + "uk"].T).reshape(T, H, D), shared.expand(T, H, R)], dim=-1)
    values = (c @ W[p + "uv"].T).reshape(T, H, V)
    queries = torch.cat([q[..., :D], q_rot], dim=-1)
    o = masked_softmax_attention(queries, keys, values, mx["scale"],
                                 window=(mx.get("mask") or {}).get("size")).reshape(T, H * V)
    return (o * torch.sigmoid(h @ W[p + "g"].T)) @ W[p + "o"].T


# ---------------------------------------------------------------------- recurrent mixers
def causal_convolution(x: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps [C, n] (the last column is the current token's), zeros before the start."""
    T, n = x.shape[0], taps.shape[1]
    out = bias.expand(T, -1).clone()
    for j in range(n):
        back = n - 1 - j
        if back < T:
            out[back:] += taps[:, j] * x[:T - back]
    return out


def gated_recurrence_states(u, r, i, lam, constant: float = 8.0) -> torch.Tensor:
    """S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t with log a_t = -constant r_t softplus(lam),
    from S = 0 (the first token is no special case); all [T, C] -> [T, C]."""
    a = torch.exp(-constant * r * torch.nn.functional.softplus(lam))
    state = torch.zeros(u.shape[1], dtype=F64)
    out = torch.zeros_like(u)
    for t in range(u.shape[0]):
        state = a[t] * state + torch.sqrt(1.0 - a[t] ** 2) * i[t] * u[t]
        out[t] = state
    return out


def linear_recurrence_mixer(W, p: str, mx: dict, h) -> torch.Tensor:
    T = h.shape[0]
    C, blocks = mx["width"], mx["blocks"]
    y = tanh_gelu(h @ W[p + "y"].T + W[p + "y.b"])
    u = causal_convolution(h @ W[p + "x"].T + W[p + "x.b"], W[p + "conv"], W[p + "conv.b"])
    ub = u.reshape(T, blocks, C // blocks)
    r = torch.sigmoid(torch.einsum("boi,tbi->tbo", W[p + "ra"], ub) + W[p + "ra.b"]).reshape(T, C)
    i = torch.sigmoid(torch.einsum("boi,tbi->tbo", W[p + "ri"], ub) + W[p + "ri.b"]).reshape(T, C)
    return (gated_recurrence_states(u, r, i, W[p + "lam"]) * y) @ W[p + "o"].T


def matrix_memory_outputs(q, k, v, i_gate, f_gate) -> torch.Tensor:
    """q, k [T, H, D], v [T, H, V], log gates [T, H] -> o [T, H, V] with a running maximum that
    starts at 0."""
    T, H, D = q.shape
    V = v.shape[-1]
    S = torch.zeros(H, D, V, dtype=F64)
    n = torch.zeros(H, D, dtype=F64)
    m = torch.zeros(H, dtype=F64)
    out = torch.zeros(T, H, V, dtype=F64)
    for t in range(T):
        m_next = torch.maximum(f_gate[t] + m, i_gate[t])
        keep = torch.exp(f_gate[t] + m - m_next)
        take = torch.exp(i_gate[t] - m_next)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        m = m_next
        below = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        out[t] = torch.einsum("hdv,hd->hv", S, q[t]) / below[:, None]
    return out


def matrix_memory_mixer(W, p: str, mx: dict, h, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, D, V, cap = mx["heads"], mx["dim"], mx["vdim"], mx["gate_cap"]
    q = (h @ W[p + "q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ W[p + "k"].T).reshape(T, H, D)
    v = (h @ W[p + "v"].T).reshape(T, H, V)
    i_gate = cap * torch.tanh((h @ W[p + "i"].T + W[p + "i.b"]) / cap)
    f_gate = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ W[p + "f"].T + W[p + "f.b"]) / cap))
    o = unit_rms(matrix_memory_outputs(q, k, v, i_gate, f_gate), eps).reshape(T, H * V)
    return (o * W[p + "norm"] * torch.sigmoid(h @ W[p + "g"].T)) @ W[p + "o"].T


# ------------------------------------------------------------------------- the rest
def clamped_gated_unit(W, p: str, mlp: dict, h) -> torch.Tensor:
    lim = mlp["limit"]
    g = (h @ W[p + "gate"].T).clamp(max=lim)
    u = (h @ W[p + "up"].T).clamp(-lim, lim)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def embed(W, cfg: dict, tokens: List[int]) -> torch.Tensor:
    emb = cfg["embedding"]
    x = W["embed"][tokens] * emb["scale"]
    bg = emb.get("bigram")
    if bg:
        rows = [bg["buckets"]] + [(tokens[t - 1] * bg["mul_prev"] + tokens[t] * bg["mul_cur"]) % bg["buckets"]
                                  for t in range(1, len(tokens))]
        x = x + W["bigram"][rows]
    return x


def forward(tokens: List[int], W: Dict[str, torch.Tensor], cfg: dict,
            taps: Optional[list] = None, rounded_stream: bool = False) -> torch.Tensor:
    """Logits [T, vocab] of one sequence; ``taps`` collects the stream after every layer.
    ``rounded_stream``: every branch reads the stream rounded to bfloat16 (what serving in
    bfloat16 does to a product's input at the least); the difference to the exact run says how
    far rounding alone moves a row."""
    eps = cfg["norm"]["eps"]
    positions = torch.arange(len(tokens))
    exact = embed(W, cfg, tokens)
    for i, layer in enumerate(cfg["layers"]):
        x = exact.to(torch.bfloat16).to(F64) if rounded_stream else exact
        j = layer["weights_of"] if layer.get("weights_of") is not None else i
        p = f"l{j}."
        mx = layer["mixer"]
        if layer["type"] == "latent_attention":
            y = latent_attention(W, p + "mix.", mx, x, positions, eps)
        else:
            gated = layer["type"] == "parallel_2"
            left = grouped_attention(W, p + "mix.left.", mx["left"], x, positions, eps, gated)
            right = matrix_memory_mixer(W, p + "mix.right.", mx["right"], x, eps) if gated \
                else linear_recurrence_mixer(W, p + "mix.right.", mx["right"], x)
            y = mx["left_scale"] * left + mx["right_scale"] * right
        exact = exact + offset_norm(y, W[p + "norm1"], eps)
        if layer.get("mlp"):
            x = exact.to(torch.bfloat16).to(F64) if rounded_stream else exact
            exact = exact + offset_norm(clamped_gated_unit(W, p + "mlp.", layer["mlp"], x), W[p + "norm2"], eps)
        if taps is not None:
            taps.append(exact.clone())
    return offset_norm(exact, W["final.norm"], eps) @ W["embed"].T


def greedy(prompt: List[int], n_new: int, W: Dict[str, torch.Tensor], cfg: dict) -> List[int]:
    """The ``n_new`` tokens greedy decoding appends (the whole sequence runs again per token)."""
    ids, out = list(prompt), []
    for _ in range(n_new):
        nxt = int(forward(ids, W, cfg)[-1].argmax())
        out.append(nxt)
        ids.append(nxt)
    return out
