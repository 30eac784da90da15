"""A matrix memory with exponential gates and a running maximum (the mLSTM cell of xLSTM), as
a mixer over a running state instead of cached keys.

Per head, with q = Wq h * ``q_scale``, k = Wk h (``dim`` numbers), v = Wv h (``vdim``) and two
gate inputs i' = Wi h + bi, f' = Wf h + bf (one number a head each),

    i = cap tanh(i' / cap)                 f = logsigmoid(cap tanh(f' / cap))      (``gate_cap``; 0: none)
    m_t = max(f + m_(t-1), i)                                                      (m_(-1) = 0)
    S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T                      (S_(-1) = 0)
    n_t = exp(f + m_(t-1) - m_t) n_(t-1) + exp(i - m_t) k
    o_t = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6)

Each head's o is brought to unit root-mean-square, multiplied by a weight per coordinate and
by sigmoid(Wg h), and projected.  S, n and m are per-request STATE of the cache manager (a
slot per live request, zero at position 0), so a prompt may be cut anywhere and decoding is
the same kernels with one token.  Steps of few tokens are one launch (a CTA per (head,
request) with the state in shared memory); longer portions compute the tokens' gate factors
first and then run the linear recurrence in segments of 64 tokens side by side.  All six projections are one product whose 32-bit result
feeds the cell unrounded; gates, exponentials, the state and the unit norm are 32-bit.  Sizes,
the cap, the query's factor, eps and the constant on the result are parameters.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .interfaces import LayerCache, Mixer, StateSpec
from .latent_attention import FusedInput
from .linear import padded_linear
from .registry import register_part


class MatrixMemory(Mixer):
    graph_safe = True
    can_overwrite = True

    def __init__(self, p: dict, store, runtime):
        w = p["weights"]
        self.width, self.heads = int(p["width"]), int(p["heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.cap, self.eps = float(p.get("gate_cap") or 0.0), float(p["eps"])
        self.q_scale = float(p.get("q_scale", self.dim ** -0.5))
        self.out_scale = float(p.get("out_scale", 1.0))
        self.runtime = runtime
        gpu = torch.cuda.is_available()
        # the one-launch kernel keeps a head's state in shared memory; the scan keeps a column
        # over up to 32 lanes of 16 numbers: either takes every step where the other cannot
        self.step_ok = gpu and ops.mmem_supports(self.dim, self.vdim)
        self.scan_ok = gpu and ops.mmem_scan_supports(self.dim)
        if gpu and not (self.step_ok or self.scan_ok):
            raise ValueError(f"matrix_memory: heads of {self.dim} x {self.vdim} are beyond both "
                             f"kernels (512 numbers a key, or a state of 200 KB)")

        def need(name, shape):
            t = store.get(w[name])
            if tuple(t.shape) != tuple(shape):
                raise ValueError(f"{w[name]}: expected {list(shape)}, found {list(t.shape)}")
            return t

        hk, hv = self.heads * self.dim, self.heads * self.vdim
        f32 = lambda t: t.to(torch.float32).contiguous()
        # the six projections: one product of the mixer's own, or rows in the product of a
        # mixer beside it that reads the same input (``input_host``)
        self.host = p.get("input_host")
        self.input = None if self.host is not None else FusedInput(self.width, runtime, "mmem_in")
        for name, rows in (("q", hk), ("k", hk), ("v", hv), ("gate", hv), ("i", self.heads),
                           ("f", self.heads)):
            if self.host is not None:
                self.host.fuse_input_rows("mmem_" + name, need(name, (rows, self.width)))
            else:
                self.input.add(name, need(name, (rows, self.width)))
        self.i_bias = f32(need("i_bias", (self.heads,))) if w.get("i_bias") else None
        self.f_bias = f32(need("f_bias", (self.heads,))) if w.get("f_bias") else None
        self.norm = f32(need("norm", (hv,)))
        self.out = padded_linear(need("out", (self.width, hv)), runtime)
        self.sm_count = ops.sm_count() if torch.cuda.is_available() else 148

    def state_specs(self):
        return [StateSpec("mmem_s", (self.heads, self.vdim, self.dim), torch.float32),
                StateSpec("mmem_n", (self.heads, self.dim), torch.float32),
                StateSpec("mmem_m", (self.heads,), torch.float32)]

    def step_bytes(self, context: int) -> int:
        """State bytes a single token reads and writes back, whatever the context."""
        return 2 * 4 * self.heads * (self.dim * self.vdim + self.dim + 1)

    takes_input_host = True

    def forward(self, ctx, h, x, cache: LayerCache, accumulate: bool = True) -> None:
        t = x.shape[0]
        cap = ctx.token_capacity
        if self.host is not None:
            proj, host_cols = self.host.fused_product()
            c = {name: host_cols["mmem_" + name] for name in ("q", "k", "v", "gate", "i", "f")}
        else:
            proj = self._proj = self.input.run(ctx, h)
            c = self.input.cols
        gated = ctx.scratch_zero("mmem_gated", (cap, self.out.n_in), self.runtime.dtype)[:t]
        columns = (c["q"][0], c["k"][0], c["v"][0], c["i"][0], c["f"][0], c["gate"][0])
        states = (cache.state["mmem_s"], cache.state["mmem_n"], cache.state["mmem_m"])
        requests = ctx.layout.b_cap
        few = ctx.layout.t_cap <= ops.mmem_segment()
        if (few and self.step_ok) or not self.scan_ok:
            # a step of few tokens: one launch, a CTA per (head, request)
            ops.mmem_step(gated, proj, columns, self.i_bias, self.f_bias, self.norm, *states,
                          ctx.q_start, ctx.state_slot, ctx.positions, requests, self.heads,
                          self.dim, self.vdim, self.cap, self.q_scale, self.eps,
                          out_scale=self.out_scale)
        else:
            # portions are cut into segments that run side by side (workspaces sized once, for
            # the largest step the runtime takes)
            n = ops.mmem_max_segments(max(ctx.runtime.max_batched_tokens, ctx.layout.t_cap),
                                      max(ctx.runtime.max_requests, requests))
            big, small = (n, self.heads, self.vdim, self.dim), (n, self.heads, self.dim)
            segments = None if few else (
                ctx.scratch("mmem_seg_own", big, torch.float32),
                ctx.scratch("mmem_seg_start", big, torch.float32),
                ctx.scratch("mmem_seg_own_n", small, torch.float32),
                ctx.scratch("mmem_seg_start_n", small, torch.float32),
                ctx.scratch("mmem_seg_keep", (n, self.heads), torch.float32))
            raw = ctx.scratch("mmem_raw", (cap, self.heads * self.vdim), torch.float32)[:t]
            gates = ctx.scratch("mmem_gates", (cap, self.heads, 4), torch.float32)[:t]
            cols = self.vdim           # value columns a CTA: halved while the GPU is not filled twice
            while cols > 8 and self.heads * n * -(-self.vdim // cols) < 2 * self.sm_count:
                cols = -(-cols // 2)
            ops.mmem_scan(gated, raw, gates, proj, columns, self.i_bias, self.f_bias, self.norm,
                          *states, ctx.q_start, ctx.state_slot, ctx.positions, ctx.seq_of_token,
                          requests, self.heads, self.dim, self.vdim, self.cap, self.q_scale,
                          self.eps, out_scale=self.out_scale, columns=cols, segments=segments)
        self.out.forward(ctx, gated, x, resid=x if accumulate else None)


register_part("mixer", "matrix_memory", lambda p, store, rt: MatrixMemory(p, store, rt))
