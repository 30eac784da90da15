"""Softmax attention over the paged cache with the options of windowed designs, as a mixer.

Query head h uses key/value head h // (heads / kv_heads); keys have ``dim`` numbers a head,
values ``vdim``.  Every option is a parameter, and a design names the ones it has:

``window`` / ``keep_first``  position i sees j <= i with i - j < window, or j < keep_first (the
                      sequence's first tokens stay visible at their true positions); window
                      None or 0: every earlier key
``rot_dims`` / ``rot_base``  rotary positions on each head's first coordinates (rotate-half);
                      ``rot_factor``: every frequency is divided by it (linear scaling)
``qk_norm``           a root-mean-square norm over the whole query projection and over the
                      whole key projection before they are split into heads (weights
                      ``q_norm`` / ``k_norm``); "head": per head, before the rotation, with
                      weights of ``dim`` numbers that all heads share; "head_after": per head,
                      after the rotation, without weights
``bias``              q, k and v have biases (weights ``q_bias`` / ``k_bias`` / ``v_bias``)
``sink``              a learned number per head (weight ``sink``) whose exponential joins the
                      softmax's denominator once: it has no key and no value and is not scaled
``q_temp``            (coef, every): queries are multiplied by 1 + coef * ln(floor((p + 1) /
                      every) + 1) at position p
``slope_bits``        a distance bias slope_h * (i - j) is taken off the scores, slope_h =
                      2^(-slope_bits * (h + 1) / heads); None: no bias
``head_gate``         head h's result is multiplied by sigmoid(G x)_h (weight ``gate``, one
                      row a head; it rides in the first product)
``value_gate``        the concatenated heads are multiplied element by element by sigmoid(G x)
                      (weight ``gate``, heads * vdim rows; in the first product too)
``out_scale``         a constant on the result (a mixer that sums two mixers gives each one)
``shares_cache``      the layer has no key/value tensors: it attends over the cache rows
                      another layer wrote, with queries, mask and everything else of its own

The cache holds ONE row per (token, key/value head), [k | v] (a group with one pool per layer),
keys as the attention reads them (normed, rotated).  Q, K, V and the gate are one matrix
product whose 32-bit result is normed and rotated unrounded; scores, weights and sums are
32-bit.  Every key is kept: a window's pages are not given back, since kept first tokens and
layers that share a cache with another window may still read them.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .interfaces import KVSpec, LayerCache, Mixer
from .latent_attention import FusedInput
from .linear import padded_linear
from .positions_rotary import rotary_frequencies
from .registry import register_part


class WindowAttention(Mixer):
    graph_safe = True
    can_overwrite = True

    def __init__(self, p: dict, store, runtime):
        w = p["weights"]
        self.width, self.heads, self.kv_heads = int(p["width"]), int(p["heads"]), int(p["kv_heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.scale, self.eps = float(p["scale"]), float(p.get("eps", 0.0))
        self.window, self.keep_first = int(p.get("window") or 0), int(p.get("keep_first") or 0)
        self.rot_dims = int(p.get("rot_dims") or 0)
        self.out_scale = float(p.get("out_scale", 1.0))
        self.shares_cache = bool(p.get("shares_cache", False))
        temp = p.get("q_temp")
        self.temp_coef, self.temp_every = (float(temp[0]), int(temp[1])) if temp else (0.0, 0)
        self.runtime = runtime
        if self.heads % self.kv_heads:
            raise ValueError(f"window_attention: {self.heads} query heads are not a multiple of "
                             f"{self.kv_heads} key/value heads")
        if self.rot_dims % 2 or self.rot_dims > self.dim:
            raise ValueError(f"window_attention: {self.rot_dims} rotated coordinates of {self.dim}")
        if self.vdim > 512:
            raise ValueError("window_attention: value heads wider than 512 are not built")
        if temp and self.temp_every < 1:
            raise ValueError("window_attention: the query temperature's period must be positive")

        def need(name, shape):
            t = store.get(w[name])
            if tuple(t.shape) != tuple(shape):
                raise ValueError(f"{w[name]}: expected {list(shape)}, found {list(t.shape)}")
            return t

        dev = runtime.device
        self.input = FusedInput(self.width, runtime, "wattn_in")
        self.input.add("q", need("q", (self.heads * self.dim, self.width)))
        if not self.shares_cache:
            self.input.add("k", need("k", (self.kv_heads * self.dim, self.width)))
            self.input.add("v", need("v", (self.kv_heads * self.vdim, self.width)))
        self.value_gate = bool(p.get("value_gate"))
        self.gated = bool(p.get("head_gate")) or self.value_gate
        if self.gated:
            rows = self.heads * self.vdim if self.value_gate else self.heads
            self.input.add("gate", need("gate", (rows, self.width)))
        self.q_norm = self.k_norm = None
        mode = p.get("qk_norm")
        if mode not in (None, False, True, "whole", "head", "head_after"):
            raise ValueError(f"window_attention: unknown qk_norm {mode!r}")
        self.head_norm = {"head": "before", "head_after": "after"}.get(mode)
        if mode == "head":
            self.q_norm = need("q_norm", (self.dim,)).to(torch.float32).contiguous()
            if not self.shares_cache:
                self.k_norm = need("k_norm", (self.dim,)).to(torch.float32).contiguous()
        elif mode in (True, "whole"):
            self.q_norm = need("q_norm", (self.heads * self.dim,)).to(torch.float32).contiguous()
            if not self.shares_cache:
                self.k_norm = need("k_norm", (self.kv_heads * self.dim,)).to(torch.float32).contiguous()
        self.biases = None
        if p.get("bias"):
            f32 = lambda t: t.to(torch.float32).contiguous()
            self.biases = (f32(need("q_bias", (self.heads * self.dim,))),
                           None if self.shares_cache else f32(need("k_bias", (self.kv_heads * self.dim,))),
                           None if self.shares_cache else f32(need("v_bias", (self.kv_heads * self.vdim,))))
        self.sinks = need("sink", (self.heads,)).to(torch.float32).contiguous() if p.get("sink") else None
        self.out = padded_linear(need("out", (self.width, self.heads * self.vdim)), runtime)
        self.slopes = None
        if p.get("slope_bits") is not None:
            bits = float(p["slope_bits"])
            self.slopes = torch.tensor([2.0 ** (-bits * (h + 1) / self.heads)
                                        for h in range(self.heads)],
                                       dtype=torch.float64).to(torch.float32).to(dev)
        self.freq, self.freq_lo = rotary_frequencies(
            float(p.get("rot_base", 10000.0)), self.rot_dims, dev,
            divide_by=float(p.get("rot_factor") or 1.0), with_lo=True)
        gpu = torch.cuda.is_available()
        self.tile_rows = ops.wattn_tile_rows(self.heads, self.kv_heads, self.dim, self.vdim) if gpu else 0
        self.single_ok = gpu and ops.wattn_single_supports(self.heads, self.kv_heads, self.dim, self.vdim)

    def kv_spec(self) -> KVSpec:
        return KVSpec(self.kv_heads, self.dim + self.vdim, None, values=False)

    def step_bytes(self, context: int) -> int:
        """Cache bytes a single token at ``context`` tokens reads: the rows it sees."""
        seen = min(context, self.window + self.keep_first) if self.window else context
        return seen * self.kv_heads * (self.dim + self.vdim) * self.runtime.dtype.itemsize

    def fuse_input_rows(self, name: str, weight) -> str:
        return self.input.add(name, weight)

    def fused_rows(self, name: str):
        return self.input.view(self._proj, name)

    def fused_product(self):
        """(the fused product's 32-bit result of this step, first column by segment name): for a
        mixer beside this one whose projections ride in the product."""
        return self._proj, self.input.cols

    def forward(self, ctx, h, x, cache: LayerCache, accumulate: bool = True) -> None:
        if self.shares_cache == cache.writes:
            raise ValueError("window_attention: a layer without key/value tensors reads another "
                             "layer's cache, and only such a layer does")
        t = x.shape[0]
        cap = ctx.token_capacity
        group = ctx.groups[cache.group]
        proj = self._proj = self.input.run(ctx, h)
        cols = self.input.cols
        q = ctx.scratch("wattn_q", (cap, self.heads * self.dim), torch.float32)[:t]
        ops.wattn_prepare(q, cache.k, proj, cols["q"][0],
                          0 if self.shares_cache else cols["k"][0],
                          0 if self.shares_cache else cols["v"][0], self.q_norm, self.k_norm,
                          None if self.shares_cache else group.slots, ctx.positions, self.freq,
                          self.heads, self.kv_heads, self.dim, self.vdim, self.rot_dims, self.eps,
                          self.temp_coef, self.temp_every, ctx.status, head_norm=self.head_norm,
                          biases=self.biases, freq_lo=self.freq_lo)
        o = ctx.scratch_zero("wattn_out", (cap, self.out.n_in), self.runtime.dtype)[:t]
        # a step of single tokens: a CTA per (token, key/value head) whose warps share out the
        # key blocks (rows of different requests share no keys); sizes that kernel does not
        # take: the tiled kernel, a row a CTA
        single = ctx.max_q_len == 1 or ctx.layout.t_cap <= ctx.layout.b_cap
        ops.wattn(o, q, cache.k, group.block_table, ctx.seq_of_token, ctx.positions, self.heads,
                  self.dim, self.vdim, self.window, self.keep_first, self.scale,
                  gate=proj[:, cols["gate"][0]:] if self.gated else None, slopes=self.slopes,
                  out_scale=self.out_scale, status=ctx.status,
                  tile_rows=min(self.tile_rows, 1) if single else self.tile_rows,
                  single=single and self.single_ok, sinks=self.sinks,
                  gate_per_value=self.value_gate)
        self.out.forward(ctx, o, x, resid=x if accumulate else None)


register_part("mixer", "window_attention", lambda p, store, rt: WindowAttention(p, store, rt))
