"""Time mixing with a decay per channel that depends on the token (the recurrence of RWKV-style
layers), as a mixer over a running state instead of cached keys.

With x_t the mixer's input and x_(t-1) the previous token's (zeros at a sequence's start),
each of the five projections s in (r, k, v, g, w) reads its own blend

    b_s = x_t + (x_(t-1) - x_t) * mu_s

r, k (``dim`` numbers a head) and v (``vdim``) are matrices applied to their blends, the gate is
silu(G b_g), and the decay of head h's key channel c is

    w_t = exp(-exp(w0 + W2 tanh(W1 b_w)))            (W1: [rank, width], W2: [heads * dim, rank])

Per head, over a 32-bit state S [dim, vdim] that starts at zero,

    o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t        S_t = diag(w_t) S_(t-1) + k_t v_t^T

(the bonus u acts on the current token only); each head's o is brought to unit root-mean-square,
multiplied by a weight per channel and by the gate, and projected.  The state and the last
input row are per-request STATE of the cache manager (a slot per live request), so a prompt may
be cut anywhere and decoding is the same kernels with one token.  A projection of a blend is
linear in it, M b_s = M x_t + (M diag(mu_s)) (x_(t-1) - x_t): the five projections are ONE
product of the pair [x_t | x_(t-1) - x_t] with the rows [M | M diag(mu_s)] of all five (the
blend weights are folded into the matrices when the model is built), whose 32-bit result feeds
the recurrence unrounded; decays, their exponentials, the state and the unit norm are 32-bit.
Steps of few tokens run the recurrence with the finish in one launch; longer portions are cut
into segments that run side by side.  Sizes, eps and the constant on the result are parameters.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .interfaces import LayerCache, Mixer, StateSpec
from .latent_attention import FusedInput
from .linear import padded_linear
from .registry import register_part

_BLENDS = ("r", "k", "v", "g", "w")


def _pad8(n: int) -> int:
    return -(-n // 8) * 8


class TimeMix(Mixer):
    graph_safe = True
    can_overwrite = True

    def __init__(self, p: dict, store, runtime):
        w = p["weights"]
        self.width, self.heads = int(p["width"]), int(p["heads"])
        self.dim = int(p["dim"])
        self.vdim = int(p.get("vdim") or self.dim)
        self.eps = float(p["eps"])
        self.out_scale = float(p.get("out_scale", 1.0))
        self.runtime = runtime
        if torch.cuda.is_available() and ops.tmix_lanes(self.dim) == 0:
            raise ValueError(f"time_mix: a head size of {self.dim} is beyond the scan kernel's 512")

        def need(name, shape):
            t = store.get(w[name])
            if shape is not None and tuple(t.shape) != tuple(shape):
                raise ValueError(f"{w[name]}: expected {list(shape)}, found {list(t.shape)}")
            return t

        hk, hv = self.heads * self.dim, self.heads * self.vdim
        w1 = need("w1", None)
        if w1.dim() != 2 or w1.shape[1] != self.width:
            raise ValueError(f"{w['w1']}: expected [rank, {self.width}], found {list(w1.shape)}")
        self.rank = int(w1.shape[0])
        # one product for the five projections: rows [M | M diag(mu_s)] against [x | x' - x]
        mats = {"r": need("r", (hk, self.width)), "k": need("k", (hk, self.width)),
                "v": need("v", (hv, self.width)), "g": need("g", (hv, self.width)), "w": w1}
        f32 = lambda t: t.to(torch.float32).contiguous()
        self.input = FusedInput(2 * self.width, runtime, "tmix_proj")
        for s in _BLENDS:
            m, mu = f32(mats[s]), f32(need("mu_" + s, (self.width,)))
            self.input.add(s, torch.cat([m, m * mu[None, :]], dim=1))
        self.input.linear()
        self.cols = self.input.cols
        self.one_launch = torch.cuda.is_available() and ops.tmix_step_supports(self.dim, self.vdim)
        self.w2 = f32(need("w2", (hk, self.rank)))
        self.w0 = f32(need("w0", (hk,)))
        self.u = f32(need("u", (self.heads, self.dim)))
        self.norm = f32(need("norm", (hv,)))
        self.out = padded_linear(need("out", (self.width, hv)), runtime)

    def state_specs(self):
        return [StateSpec("time_mix", (self.heads, self.vdim, self.dim), torch.float32),
                StateSpec("time_mix_input", (self.width,), self.runtime.dtype)]

    def step_bytes(self, context: int) -> int:
        """State bytes a single token reads and writes back, whatever the context."""
        return 2 * (self.heads * self.vdim * self.dim * 4 + self.width * self.runtime.dtype.itemsize)

    def forward(self, ctx, h, x, cache: LayerCache, accumulate: bool = True) -> None:
        t = x.shape[0]
        cap = ctx.token_capacity
        state, prev = cache.state["time_mix"], cache.state["time_mix_input"]
        pair = ctx.scratch("tmix_pair", (cap, 2 * self.width), self.runtime.dtype)[:t]
        ops.tmix_shift(pair, h, prev, None, ctx.seq_of_token, ctx.positions, ctx.q_start,
                       ctx.state_slot, ctx.status)
        proj = self.input.run(ctx, pair)
        raw = ctx.scratch("tmix_raw", (cap, self.heads * self.vdim), torch.float32)[:t]
        gated = ctx.scratch_zero("tmix_gated", (cap, self.out.n_in), self.runtime.dtype)[:t]
        requests = ctx.layout.b_cap
        scan = lambda **kw: ops.tmix_scan(
            raw, proj, self.cols["r"][0], self.cols["k"][0], self.cols["v"][0], self.cols["w"][0],
            self.w2, self.w0, self.u, state, h, prev, ctx.q_start, ctx.state_slot, ctx.positions,
            requests, self.heads, self.dim, self.vdim, ctx.status, **kw)
        if ctx.layout.t_cap <= ops.tmix_segment():
            # a step of few tokens: a CTA per (head, request) from and to the slot, with the
            # finish inside where it holds all of the head's columns
            if self.one_launch:
                scan(finish=(gated, self.cols["g"][0], self.norm, self.eps, self.out_scale))
                self.out.forward(ctx, gated, x, resid=x if accumulate else None)
                return
            scan()
        else:
            # portions are cut into segments that run side by side (workspaces sized once, for
            # the largest step the runtime takes)
            n = ops.tmix_max_segments(max(ctx.runtime.max_batched_tokens, ctx.layout.t_cap),
                                      max(ctx.runtime.max_requests, requests))
            shape = (n, self.heads, self.vdim, self.dim)
            scan(segments=(ctx.scratch("tmix_seg_own", shape, torch.float32),
                           ctx.scratch("tmix_seg_start", shape, torch.float32),
                           ctx.scratch("tmix_seg_decay", (n, self.heads, self.dim), torch.float32)),
                 decays=ctx.scratch("tmix_decays", (cap, self.heads * self.dim), torch.float32)[:t])
        ops.tmix_finish(gated, raw, proj, self.cols["g"][0], self.norm, ctx.seq_of_token,
                        self.heads, self.vdim, self.eps, self.out_scale)
        self.out.forward(ctx, gated, x, resid=x if accumulate else None)


register_part("mixer", "time_mix", lambda p, store, rt: TimeMix(p, store, rt))
