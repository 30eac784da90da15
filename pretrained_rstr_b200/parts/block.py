"""Arrangements of parts in a block.  ``pre_norm``:
x += mixer(norm_1(x)); x += feed_forward(norm_2(x))  (``dev/examples/gpt2.clj:149-166``).
The block knows its parts only through their interfaces."""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from .interfaces import Block, FeedForward, LayerCache, Mixer, Norm
from .linear import LazyNorm, Linear
from .registry import register_part


class PreNormBlock(Block):
    graph_safe = True
    def __init__(self, mixer: Mixer, feed_forward: FeedForward, norms: Dict[str, Norm],
                 width: int, runtime):
        # (a layer without a feed-forward has the mixer's norm alone)
        self.has_ff = not getattr(feed_forward, "is_none", False)
        wanted = {"mixer", "feed_forward"} if self.has_ff else {"mixer"}
        if set(norms) != wanted:
            raise ValueError(f"pre_norm wants the norms {sorted(wanted)}, got {sorted(norms)}")
        self.mixer, self.feed_forward = mixer, feed_forward
        self.norms = dict(norms)
        self.mixer_norm, self.feed_forward_norm = norms["mixer"], norms.get("feed_forward")
        self.width, self.runtime = width, runtime

    def forward(self, ctx, x, cache: LayerCache) -> None:
        t = x.shape[0]
        h = ctx.scratch("block_normed", (ctx.token_capacity, self.width), self.runtime.dtype)[:t]
        self.mixer.forward(ctx, self._normed(ctx, self.mixer, self.mixer_norm, x, h), x, cache)
        if not self.has_ff:
            return
        self.feed_forward.forward(
            ctx, self._normed(ctx, self.feed_forward, self.feed_forward_norm, x, h), x)

    @staticmethod
    def _normed(ctx, consumer, norm, x, out):
        """The consumer's input: a norm that has run, or, for consumers that say they take
        one (``accepts_lazy_norm``), a :class:`LazyNorm` they may fuse into their first
        matrix product."""
        lazy = LazyNorm(ctx, norm, x, out)
        return lazy if getattr(consumer, "accepts_lazy_norm", False) else lazy.tensor()


class PostNormGatedBlock(Block):
    """x <- norm_1(alpha x + g_1(x) * mixer(x)); x <- norm_2(alpha x + g_2(x) * feed_forward(x)):
    the branches read the stream itself, the norm comes after the sum, and a branch's result may
    be gated element by element by g(x) = sigmoid(W x + b) (``params["gates"]``: branch name ->
    tensor name of W, with ``.b``).  A layer without a feed-forward has the first half only
    (and, if its file still holds a second norm, ``params["norm_alone"]``, that norm of the
    scaled stream).

    The gate's matrix rides along in the branch's first matrix product where the part offers
    that (``fuse_input_rows``); sum, gate and norm are one kernel, which also leaves the
    stream's copy in the activation type for the next branch's product."""
    graph_safe = True

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, norms: Dict[str, Norm],
                 width: int, runtime, params=None, store=None):
        params = params or {}
        self.mixer, self.feed_forward = mixer, feed_forward
        self.norms = dict(norms)
        self.width, self.runtime = width, runtime
        self.alpha = float(params.get("alpha", 1.0))
        self.has_ff = not getattr(feed_forward, "is_none", False)
        wanted = {"mixer"} | ({"feed_forward"} if self.has_ff else set())
        if set(norms) != wanted:
            raise ValueError(f"post_norm_gated wants the norms {sorted(wanted)}, got {sorted(norms)}")
        for part in (mixer, feed_forward):
            if not getattr(part, "can_overwrite", False):
                raise ValueError(f"post_norm_gated: {type(part).__name__} cannot hand over its "
                                 f"result apart from the stream")
        for norm in norms.values():
            if not hasattr(norm, "joined"):
                raise ValueError("post_norm_gated needs norms that can join a branch to the stream")
        # a layer without a feed-forward whose file still holds the second norm: x <- norm(alpha x)
        self.norm_alone = None
        alone = params.get("norm_alone")
        if not self.has_ff and alone and store is not None and alone["gain"] in store:
            from .norms import RMSNorm
            self.norm_alone = RMSNorm(store.get(alone["gain"]), None, alone["eps"], width)
            self.norms["alone"] = self.norm_alone
        self.gates = {}
        for name, tensor in (params.get("gates") or {}).items():
            part = {"mixer": mixer, "feed_forward": feed_forward}[name]
            w, b = store.get(tensor), store.get(tensor + ".b")
            if tuple(w.shape) != (width, width) or b.numel() != width:
                raise ValueError(f"{tensor}: a gate of the stream is [{width}, {width}] with a bias")
            bias = b.to(torch.float32).contiguous()
            if hasattr(part, "fuse_input_rows"):
                self.gates[name] = (part.fuse_input_rows("branch_gate", w), None, bias)
            else:
                self.gates[name] = (None, Linear(w, None, runtime), bias)

    def forward(self, ctx, x, cache: LayerCache) -> None:
        t = x.shape[0]
        cap = ctx.token_capacity
        y = ctx.scratch("branch_result", (cap, self.width), torch.float32)[:t]
        serving = self.runtime.dtype != torch.float32
        copy = ctx.scratch("stream_copy", (cap, self.width), self.runtime.dtype)[:t] if serving else None
        # the stream in the products' type: the norm before left it, unless this is the model's
        # first branch or another kind of block has changed the stream since
        writer = getattr(ctx, "stream_copy_by", None)
        current = writer is not None and writer is getattr(ctx, "last_block", None)
        for name, part in (("mixer", self.mixer), ("feed_forward", self.feed_forward)):
            if name == "feed_forward" and not self.has_ff:
                break
            h = x
            if serving:
                if not current:
                    ops.bias_act(copy, x, None, None, None)
                h = copy
            if name == "mixer":
                part.forward(ctx, h, y, cache, accumulate=False)
            else:
                part.forward(ctx, h, y, accumulate=False)
            gate = bias = None
            if name in self.gates:
                fused, own, bias = self.gates[name]
                if fused is not None:
                    gate = part.fused_rows(fused)
                else:
                    gate = ctx.scratch("branch_gate", (cap, self.width), torch.float32)[:t]
                    own.forward(ctx, h, gate)
            self.norms[name].joined(ctx, x, y, self.alpha, gate=gate, gate_bias=bias, copy=copy)
            current = True
        if self.norm_alone is not None:
            self.norm_alone.joined(ctx, x, None, self.alpha, copy=copy)
        ctx.stream_copy_by = self


class ParallelBlock(Block):
    """x <- x + (mixer(norm_1(x)) + feed_forward(norm_2(x))): both branches read the stream as
    it was before the layer, each through a norm of its own, and their results join it in
    32-bit.  The mixer's norm runs first; the feed-forward then reads the untouched stream
    (its norm may ride in its first matrix product, see :class:`LazyNorm`) and adds its
    result, and the mixer, which works from its normed copy, adds its own after that.  A
    layer without a feed-forward has the mixer's norm alone."""
    graph_safe = True

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, norms: Dict[str, Norm],
                 width: int, runtime):
        self.has_ff = not getattr(feed_forward, "is_none", False)
        wanted = {"mixer", "feed_forward"} if self.has_ff else {"mixer"}
        if set(norms) != wanted:
            raise ValueError(f"parallel wants the norms {sorted(wanted)}, got {sorted(norms)}")
        self.mixer, self.feed_forward = mixer, feed_forward
        self.norms = dict(norms)
        self.width, self.runtime = width, runtime

    def forward(self, ctx, x, cache: LayerCache) -> None:
        t = x.shape[0]
        cap = ctx.token_capacity
        h1 = ctx.scratch("block_normed", (cap, self.width), self.runtime.dtype)[:t]
        self.norms["mixer"].forward(ctx, x, h1)
        if self.has_ff:
            h2 = ctx.scratch("block_normed_2", (cap, self.width), self.runtime.dtype)[:t]
            self.feed_forward.forward(
                ctx, PreNormBlock._normed(ctx, self.feed_forward, self.norms["feed_forward"], x, h2), x)
        self.mixer.forward(ctx, h1, x, cache)


class BranchNormBlock(Block):
    """x <- x + norm_1(mixer(x)); x <- x + norm_2(feed_forward(x)): the branches read the stream
    itself and each branch's RESULT is normed before it joins the stream.  A layer without a
    feed-forward has the first half only.  Norm and sum are one kernel, which also leaves the
    stream's copy in the activation type for the next branch's product."""
    graph_safe = True

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, norms: Dict[str, Norm],
                 width: int, runtime):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.norms = dict(norms)
        self.width, self.runtime = width, runtime
        self.has_ff = not getattr(feed_forward, "is_none", False)
        wanted = {"mixer"} | ({"feed_forward"} if self.has_ff else set())
        if set(norms) != wanted:
            raise ValueError(f"branch_norm wants the norms {sorted(wanted)}, got {sorted(norms)}")
        for part in (mixer, feed_forward):
            if not getattr(part, "can_overwrite", False):
                raise ValueError(f"branch_norm: {type(part).__name__} cannot hand over its result "
                                 f"apart from the stream")
        for norm in norms.values():
            if not hasattr(norm, "added"):
                raise ValueError("branch_norm needs norms that can add a normed branch to the stream")

    def forward(self, ctx, x, cache: LayerCache) -> None:
        t = x.shape[0]
        cap = ctx.token_capacity
        y = ctx.scratch("branch_result", (cap, self.width), torch.float32)[:t]
        serving = self.runtime.dtype != torch.float32
        copy = ctx.scratch("stream_copy", (cap, self.width), self.runtime.dtype)[:t] if serving else None
        # the stream in the products' type: the norm before left it, unless this is the model's
        # first branch or another kind of block has changed the stream since
        writer = getattr(ctx, "stream_copy_by", None)
        current = writer is not None and writer is getattr(ctx, "last_block", None)
        for name, part in (("mixer", self.mixer), ("feed_forward", self.feed_forward)):
            if name == "feed_forward" and not self.has_ff:
                break
            h = x
            if serving:
                if not current:
                    ops.bias_act(copy, x, None, None, None)
                h = copy
            if name == "mixer":
                part.forward(ctx, h, y, cache, accumulate=False)
            else:
                part.forward(ctx, h, y, accumulate=False)
            self.norms[name].added(ctx, x, y, copy=copy)
            current = True
        ctx.stream_copy_by = self


register_part("arrangement", "pre_norm", PreNormBlock)
register_part("arrangement", "branch_norm", BranchNormBlock)
register_part("arrangement", "post_norm_gated", PostNormGatedBlock)
register_part("arrangement", "parallel", ParallelBlock)
