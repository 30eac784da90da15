"""Feed-forwards.  ``dense_mlp``: up -> activation -> down, added to the residual stream
(``dev/examples/gpt2.clj:160-166``).  Width, inner size (not tied to 4*width as in
``gpt2.clj:150``), activation and biases are parameters."""
from __future__ import annotations

import torch

from ..csrc import ops
from .interfaces import FeedForward
from .linear import Linear, padded_linear
from .registry import register_part


class DenseMLP(FeedForward):
    graph_safe = True
    accepts_lazy_norm = True      # the first matrix product may compute the norm itself
    can_overwrite = True
    def __init__(self, up: Linear, down: Linear, width: int, inner: int, activation: str, runtime):
        if activation not in ops.ACT_CODES:
            raise ValueError(f"dense_mlp: unknown activation {activation!r}")
        if (up.n_in, up.n_out) != (width, inner) or (down.n_in, down.n_out) != (inner, width):
            raise ValueError("dense_mlp: matrices have the wrong shape")
        self.up, self.down = up, down
        self.width, self.inner, self.activation = width, inner, activation
        self.runtime = runtime

    def forward(self, ctx, h, x, accumulate: bool = True) -> None:
        t = x.shape[0]
        u = ctx.scratch("mlp_inner", (ctx.token_capacity, self.inner), self.runtime.dtype)[:t]
        self.up.forward(ctx, h, u, act=self.activation)
        self.down.forward(ctx, u, x, resid=x if accumulate else None)


def _dense_mlp(p, store, rt) -> DenseMLP:
    layout = p.get("weight_layout", "out_in")
    up = Linear.from_store(store, p["weights"]["up"], layout, p["width"], p["inner"],
                           p.get("bias", False), rt)
    down = Linear.from_store(store, p["weights"]["down"], layout, p["inner"], p["width"],
                             p.get("bias", False), rt)
    return DenseMLP(up, down, p["width"], p["inner"], p["activation"], rt)


class NoFeedForward(FeedForward):
    """A layer without a feed-forward (``is_none``: arrangements skip the branch)."""
    graph_safe = True
    can_overwrite = True
    is_none = True

    def forward(self, ctx, h, x, accumulate: bool = True) -> None:
        if not accumulate:
            x.zero_()


class GatedMLP(FeedForward):
    """down(f(gate(h)) * (up(h) + up_shift)) with f(g) = g * sigmoid(act_alpha * g); with
    ``limit`` > 0 the gate's result is capped at ``limit`` and up's clamped to +-``limit``
    first.  (act_alpha 1, shift 0, no limit: the usual SiLU-gated feed-forward.)  Gate and up
    are one matrix product, in which rows of an arrangement may ride along
    (:meth:`fuse_input_rows`); its float32 result feeds the activation unrounded."""
    graph_safe = True
    can_overwrite = True
    accepts_lazy_norm = True      # the first matrix product may compute the norm itself

    def __init__(self, gate, up, down, width: int, inner: int, limit: float, act_alpha: float,
                 up_shift: float, runtime):
        from .latent_attention import FusedInput
        for name, t, shape in (("gate", gate, (inner, width)), ("up", up, (inner, width)),
                               ("down", down, (width, inner))):
            if tuple(t.shape) != shape:
                raise ValueError(f"gated_mlp: {name} is {list(t.shape)}, expected {list(shape)}")
        self.input = FusedInput(width, runtime, "gated_in")
        self.input.add("gate", gate)
        self.input.add("up", up)
        self.down = padded_linear(down, runtime)
        self.width, self.inner = width, inner
        self.limit, self.act_alpha, self.up_shift = float(limit), float(act_alpha), float(up_shift)
        self.runtime = runtime

    def fuse_input_rows(self, name: str, weight) -> str:
        return self.input.add(name, weight)

    def fused_rows(self, name: str):
        return self.input.view(self._proj, name)

    def forward(self, ctx, h, x, accumulate: bool = True) -> None:
        t = x.shape[0]
        proj = self._proj = self.input.run(ctx, h)
        cols = self.input.cols
        a = ctx.scratch_zero("gated_act", (ctx.token_capacity, self.down.n_in), self.runtime.dtype)[:t]
        ops.gated_pair(a, proj, cols["gate"][0], cols["up"][0], self.inner, limit=self.limit,
                       act_alpha=self.act_alpha, up_shift=self.up_shift)
        self.down.forward(ctx, a, x, resid=x if accumulate else None)


class GatedMoE(FeedForward):
    """A router chooses ``top`` of ``experts`` gated feed-forwards per token (logits in
    32-bit accumulators plus a bias, if the router has one); an optional shared expert runs for
    every token.  ``score`` says what the weights are: "softmax_chosen" (the default), the
    softmax over the chosen logits alone; "softmax", the chosen experts' shares of the softmax
    over ALL experts (``renormalize``: divided by their sum), times ``router_scale``.

    All experts' gate and up rows, the shared expert's, the router's and whatever an
    arrangement fuses in are ONE matrix product; the activations of experts a token did not
    choose are multiplied by zero and those it chose by their weight, and one product with all
    down matrices side by side sums the chosen experts (zeros add nothing).  Every token thus
    pays for every expert's arithmetic: right for any sizes, cheap while experts are small."""
    graph_safe = True
    can_overwrite = True
    accepts_lazy_norm = True      # the first matrix product may compute the norm itself

    def __init__(self, p: dict, store, runtime):
        from .latent_attention import FusedInput
        width, n, inner = p["width"], p["experts"], p["inner"]
        self.width, self.experts, self.top, self.inner = width, n, p["top"], inner
        self.shared_inner = int(p.get("shared_inner") or 0)
        self.limit, self.shared_limit = float(p["limit"]), float(p.get("shared_limit") or 0.0)
        self.act_alpha, self.up_shift = float(p["act_alpha"]), float(p["up_shift"])
        self.score = p.get("score", "softmax_chosen")
        self.renormalize = bool(p.get("renormalize", False))
        self.router_scale = float(p.get("router_scale", 1.0))
        if self.score not in ("softmax_chosen", "softmax"):
            raise ValueError(f"gated_moe: unknown score {self.score!r}")
        if not 1 <= self.top <= n:
            raise ValueError(f"gated_moe: top {self.top} of {n} experts")
        self.runtime = runtime
        pre = p["prefix"]

        def need(name, shape):
            t = store.get(pre + name)
            if tuple(t.shape) != tuple(shape):
                raise ValueError(f"{pre + name}: expected {list(shape)}, found {list(t.shape)}")
            return t

        self.input = FusedInput(width, runtime, "moe_in")
        self.input.add("gate", torch.cat([need(f"e{e}.gate", (inner, width)) for e in range(n)]))
        self.input.add("up", torch.cat([need(f"e{e}.up", (inner, width)) for e in range(n)]))
        downs = [need(f"e{e}.down", (width, inner)) for e in range(n)]
        if self.shared_inner:
            self.input.add("shared_gate", need("shared.gate", (self.shared_inner, width)))
            self.input.add("shared_up", need("shared.up", (self.shared_inner, width)))
            downs.append(need("shared.down", (width, self.shared_inner)))
        self.input.add("router", need("router", (n, width)))
        self.router_bias = need("router.b", (n,)).to(torch.float32).contiguous() \
            if p.get("router_bias", True) else None
        if self.score == "softmax" and self.router_bias is not None:
            raise ValueError("gated_moe: the softmax over all experts takes no router bias")
        self.down = padded_linear(torch.cat(downs, dim=1), runtime)

    def fuse_input_rows(self, name: str, weight) -> str:
        return self.input.add(name, weight)

    def fused_rows(self, name: str):
        return self.input.view(self._proj, name)

    def forward(self, ctx, h, x, accumulate: bool = True) -> None:
        t = x.shape[0]
        cap = ctx.token_capacity
        proj = self._proj = self.input.run(ctx, h)
        cols = self.input.cols
        scale = ctx.scratch("moe_scale", (cap, self.experts), torch.float32)[:t]
        chosen = ctx.scratch("moe_chosen", (cap, self.top), torch.int32)[:t]
        chosen_w = ctx.scratch("moe_chosen_w", (cap, self.top), torch.float32)[:t]
        if self.score == "softmax":
            ops.route_scores(scale, chosen, chosen_w, self.input.view(proj, "router"), None,
                             self.top, score="softmax", renormalize=self.renormalize,
                             factor=self.router_scale)
        else:
            ops.route(scale, chosen, chosen_w, self.input.view(proj, "router"), None,
                      self.router_bias, self.top)
        n_act = self.experts * self.inner
        a = ctx.scratch_zero("moe_act", (cap, self.down.n_in), self.runtime.dtype)[:t]
        ops.gated_pair(a, proj, cols["gate"][0], cols["up"][0], n_act, limit=self.limit,
                       act_alpha=self.act_alpha, up_shift=self.up_shift, scale=scale,
                       group=self.inner)
        if self.shared_inner:
            ops.gated_pair(a, proj, cols["shared_gate"][0], cols["shared_up"][0],
                           self.shared_inner, out_col=n_act, limit=self.shared_limit,
                           act_alpha=self.act_alpha, up_shift=self.up_shift)
        self.down.forward(ctx, a, x, resid=x if accumulate else None)


class RoutedExperts(FeedForward):
    """``experts`` small feed-forwards down(act(up(.))) without biases, of which a token uses
    the ``top`` with the largest scores s = sigmoid(router h) (``score``; router logits are
    32-bit accumulators).  The weights are the chosen scores themselves (``renormalize``:
    divided by their sum) and multiply the expert's INPUT (``weight_on`` "input": the result
    is the sum of expert(w h)) or its output.

    All experts' up rows and the router's are ONE matrix product (up is linear: up(w h) =
    w up(h), so the weight meets the 32-bit result inside the activation); activations of
    experts a token did not choose are zero, and one product with all down matrices side by
    side sums the chosen experts.  Every token pays for every expert's arithmetic: right at any
    sizes, cheap while experts are small."""
    graph_safe = True
    can_overwrite = True
    accepts_lazy_norm = True      # the first matrix product may compute the norm itself

    def __init__(self, p: dict, store, runtime):
        from .latent_attention import FusedInput
        width, n, inner = int(p["width"]), int(p["experts"]), int(p["inner"])
        self.width, self.experts, self.top, self.inner = width, n, int(p["top"]), inner
        self.activation = p.get("activation", "relu_squared")
        self.score = p.get("score", "sigmoid")
        self.renormalize = bool(p.get("renormalize", False))
        self.weight_on = p.get("weight_on", "input")
        if self.activation not in ops.ROUTED_ACT_CODES or self.score not in ops.SCORE_CODES or \
                self.weight_on not in ("input", "output"):
            raise ValueError("routed_experts: unknown activation, score or weight placement")
        if not 1 <= self.top <= n:
            raise ValueError(f"routed_experts: top {self.top} of {n} experts")
        self.runtime = runtime
        pre = p["prefix"]

        def need(name, shape):
            t = store.get(pre + name)
            if tuple(t.shape) != tuple(shape):
                raise ValueError(f"{pre + name}: expected {list(shape)}, found {list(t.shape)}")
            return t

        self.input = FusedInput(width, runtime, "routed_in")
        self.input.add("up", torch.cat([need(f"e{e}.up", (inner, width)) for e in range(n)]))
        self.input.add("router", need("router", (n, width)))
        self.down = padded_linear(
            torch.cat([need(f"e{e}.down", (width, inner)) for e in range(n)], dim=1), runtime)

    def fuse_input_rows(self, name: str, weight) -> str:
        return self.input.add(name, weight)

    def fused_rows(self, name: str):
        return self.input.view(self._proj, name)

    def forward(self, ctx, h, x, accumulate: bool = True) -> None:
        t = x.shape[0]
        cap = ctx.token_capacity
        proj = self._proj = self.input.run(ctx, h)
        # the router's scores, the choice and the activation with the chosen experts' weights:
        # one launch, a CTA per token
        a = ctx.scratch_zero("routed_act", (cap, self.down.n_in), self.runtime.dtype)[:t]
        ops.route_act(a, proj, self.input.cols["up"][0], self.input.cols["router"][0], self.experts,
                      self.top, self.inner, self.score, self.renormalize, self.activation,
                      self.weight_on)
        self.down.forward(ctx, a, x, resid=x if accumulate else None)


def _gated_mlp(p, store, rt) -> GatedMLP:
    w = p["weights"]
    return GatedMLP(store.get(w["gate"]), store.get(w["up"]), store.get(w["down"]), p["width"],
                    p["inner"], p.get("limit", 0.0), p.get("act_alpha", 1.0),
                    p.get("up_shift", 0.0), rt)


register_part("feed_forward", "dense_mlp", _dense_mlp)
register_part("feed_forward", "gated_mlp", _gated_mlp)
register_part("feed_forward", "gated_moe", lambda p, store, rt: GatedMoE(p, store, rt))
register_part("feed_forward", "routed_experts", lambda p, store, rt: RoutedExperts(p, store, rt))
register_part("feed_forward", "none", lambda p, store, rt: NoFeedForward())
