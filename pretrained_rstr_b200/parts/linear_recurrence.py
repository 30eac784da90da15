"""A gated linear recurrence per channel with a short convolution before it (the recurrent
block of Griffin-style layers), as a mixer over a running state instead of cached keys.

Two branches of ``inner`` channels read the mixer's input: y = gelu_tanh(Wy h + by) and
x = Wx h + bx.  x passes a causal convolution per channel (``taps`` long, the last tap on the
current token, zeros before the sequence's start, no activation): u.  The channels are cut
into ``blocks`` equal parts; in part b two square matrices give the gates

    r = sigmoid(A_b u_b + a_b)        i = sigmoid(B_b u_b + b_b)

and per channel, with ``decay_constant`` c (8 in Griffin) and a learned lambda,

    log a = -c * r * softplus(lambda)      S_t = a S_(t-1) + sqrt(1 - a^2) * i * u      (S_(-1) = 0)

The result is Wo (S * y).  The state S and the convolution's last ``taps - 1`` inputs are
per-request STATE of the cache manager (a slot per live request, zero at position 0), so a
prompt may be cut anywhere and decoding is the same kernels with one token.  Steps of few
tokens are one launch (a CTA per (request, block)); longer portions run the convolution, the
gates and then the recurrence in segments of 64 tokens side by side.  Wy and Wx are
one product whose 32-bit result feeds everything after it unrounded; the block matrices, the
gates, the decays, the recurrence and the state are 32-bit; a decay travels as a - 1 =
expm1(log a) and a step is S + (input + (a - 1) S), so that a decay close to one keeps its
precision.  Sizes, taps, blocks, the decay's
constant and the constant on the result are parameters.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .interfaces import LayerCache, Mixer, StateSpec
from .latent_attention import FusedInput
from .linear import padded_linear
from .registry import register_part


class GatedLinearRecurrence(Mixer):
    graph_safe = True
    can_overwrite = True

    def __init__(self, p: dict, store, runtime):
        w = p["weights"]
        self.width, self.inner = int(p["width"]), int(p["inner"])
        self.blocks, self.taps = int(p["blocks"]), int(p["taps"])
        self.out_scale = float(p.get("out_scale", 1.0))
        self.runtime = runtime
        if self.blocks < 1 or self.inner % self.blocks:
            raise ValueError(f"gated_linear_recurrence: {self.inner} channels do not split into "
                             f"{self.blocks} equal blocks")
        if self.taps < 1 or (torch.cuda.is_available() and self.taps > ops.lru_max_taps()):
            raise ValueError(f"gated_linear_recurrence: a convolution of {self.taps} taps is not built")
        bw = self.inner // self.blocks

        def need(name, shape):
            t = store.get(w[name])
            if tuple(t.shape) != tuple(shape):
                raise ValueError(f"{w[name]}: expected {list(shape)}, found {list(t.shape)}")
            return t

        f32 = lambda t: t.to(torch.float32).contiguous()
        # the two projections: one product of the mixer's own, or rows in the product of a
        # mixer beside it that reads the same input (``input_host``)
        self.host = p.get("input_host")
        self.input = None if self.host is not None else FusedInput(self.width, runtime, "lru_in")
        for name in ("y", "x"):
            rows = need(name, (self.inner, self.width))
            if self.host is not None:
                self.host.fuse_input_rows("lru_" + name, rows)
            else:
                self.input.add(name, rows)
        self.y_bias = f32(need("y_bias", (self.inner,))) if w.get("y_bias") else None
        self.x_bias = f32(need("x_bias", (self.inner,))) if w.get("x_bias") else None
        self.conv_w = f32(need("conv", (self.inner, self.taps)))
        self.conv_b = f32(need("conv_bias", (self.inner,))) if w.get("conv_bias") else None
        # the block matrices with the input axis outermost: a thread per output reads
        # neighbouring numbers
        self.wa_t = need("gate_a", (self.blocks, bw, bw)).to(runtime.dtype).transpose(1, 2).contiguous()
        self.wi_t = need("gate_i", (self.blocks, bw, bw)).to(runtime.dtype).transpose(1, 2).contiguous()
        self.ba = f32(need("gate_a_bias", (self.blocks, bw))).reshape(self.inner)
        self.bi = f32(need("gate_i_bias", (self.blocks, bw))).reshape(self.inner)
        # log a = decay * r with decay = -c * softplus(lambda), in 32-bit
        lam = f32(need("lambda", (self.inner,)))
        self.decay = (-float(p.get("decay_constant", 8.0)) * torch.nn.functional.softplus(lam)).contiguous()
        self.out = padded_linear(need("out", (self.width, self.inner)), runtime)
        self.one_launch = torch.cuda.is_available() and ops.lru_step_supports(bw)

    def state_specs(self):
        return [StateSpec("lru_state", (self.inner,), torch.float32),
                StateSpec("lru_inputs", (self.taps - 1, self.inner), torch.float32)]

    def step_bytes(self, context: int) -> int:
        """State bytes a single token reads and writes back, whatever the context."""
        return 2 * 4 * self.inner * self.taps

    takes_input_host = True

    def forward(self, ctx, h, x, cache: LayerCache, accumulate: bool = True) -> None:
        t = x.shape[0]
        cap = ctx.token_capacity
        state, inputs = cache.state["lru_state"], cache.state["lru_inputs"]
        if self.host is not None:
            proj, host_cols = self.host.fused_product()
            cols = {name: host_cols["lru_" + name] for name in ("y", "x")}
        else:
            proj = self._proj = self.input.run(ctx, h)
            cols = self.input.cols
        gated = ctx.scratch_zero("lru_gated", (cap, self.out.n_in), self.runtime.dtype)[:t]
        requests = ctx.layout.b_cap
        if ctx.layout.t_cap <= ops.lru_segment() and self.one_launch:
            # a step of few tokens: convolution, gates and recurrence in one launch
            ops.lru_step(gated, proj, cols["y"][0], cols["x"][0], self.y_bias, self.x_bias,
                         self.conv_w, self.conv_b, self.wa_t, self.wi_t, self.ba, self.bi,
                         self.decay, state, inputs, ctx.q_start, ctx.state_slot, ctx.positions,
                         requests, self.blocks, out_scale=self.out_scale)
            self.out.forward(ctx, gated, x, resid=x if accumulate else None)
            return
        u = ctx.scratch("lru_u", (cap, self.inner), torch.float32)[:t]
        a = ctx.scratch("lru_a", (cap, self.inner), torch.float32)[:t]
        ops.lru_conv(u, proj, cols["x"][0], self.x_bias, self.conv_w, self.conv_b, inputs,
                     ctx.seq_of_token, ctx.positions, ctx.q_start, ctx.state_slot)
        ops.lru_gates(a, u, self.wa_t, self.wi_t, self.ba, self.bi, self.decay, self.blocks)
        # portions are cut into segments that run side by side (workspaces sized once, for the
        # largest step the runtime takes)
        n = ops.lru_max_segments(max(ctx.runtime.max_batched_tokens, ctx.layout.t_cap),
                                 max(ctx.runtime.max_requests, requests))
        segments = (ctx.scratch("lru_seg_own", (n, self.inner), torch.float32),
                    ctx.scratch("lru_seg_keep", (n, self.inner), torch.float32))
        ops.lru_scan(gated, a, u, proj, cols["y"][0], cols["x"][0], self.y_bias, self.x_bias,
                     state, inputs, ctx.q_start, ctx.state_slot, ctx.positions, requests,
                     out_scale=self.out_scale, segments=segments)
        self.out.forward(ctx, gated, x, resid=x if accumulate else None)


register_part("mixer", "gated_linear_recurrence",
              lambda p, store, rt: GatedLinearRecurrence(p, store, rt))
