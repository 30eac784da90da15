"""Norms.  ``layer_norm``: mean-centred, biased variance, gain and bias, statistics in
32-bit (call sites ``dev/examples/gpt2.clj:152,160,240``; formula
``src/pretrained/asr/moonshine.clj:87-104``).  Size and eps are parameters."""
from __future__ import annotations

import torch

from ..csrc import ops
from .interfaces import Norm
from .registry import register_part


class LayerNorm(Norm):
    graph_safe = True
    kind = "layer_norm"
    def __init__(self, gamma: torch.Tensor, beta, eps: float, size: int):
        if gamma.numel() != size or (beta is not None and beta.numel() != size):
            raise ValueError(f"layer_norm: gain/bias size differs from {size}")
        self.gamma = gamma.to(torch.float32).contiguous()
        self.beta = None if beta is None else beta.to(torch.float32).contiguous()
        self.eps = float(eps)
        self.size = size

    def forward(self, ctx, x, out, rows=None) -> None:
        ops.layernorm(out, x, self.gamma, self.beta, self.eps, rows=rows, status=ctx.status)


def _layer_norm(params, store, runtime) -> LayerNorm:
    name = params["weights"]
    beta = store.get(name + ".bias") if params.get("bias", True) else None
    return LayerNorm(store.get(name + ".weight"), beta, params["eps"], params["size"])


class RMSNorm(Norm):
    """x / sqrt(mean(x^2) + eps), times one learned number (``gain``) and/or a learned weight
    per coordinate; statistics in 32-bit.  ``joined`` is the same norm of a gated branch
    joined to the stream: x <- norm(alpha x + sigmoid(gate) * y), with an optional copy of the
    result in the activation type.  ``added`` is the norm of a branch alone with the stream
    joined after it: x <- x + norm(y)."""
    graph_safe = True
    kind = "rms_norm"

    def __init__(self, gain, weight, eps: float, size: int):
        if gain is not None and gain.numel() != 1:
            raise ValueError("rms_norm: the gain is one number")
        if weight is not None and weight.numel() != size:
            raise ValueError(f"rms_norm: weight size differs from {size}")
        self.gain = None if gain is None else gain.to(torch.float32).reshape(1).contiguous()
        self.weight = None if weight is None else weight.to(torch.float32).contiguous()
        self.eps, self.size = float(eps), size
        # what the decode-time product's fused prologue needs to compute this norm itself: the
        # layer norm's names, without a mean and a bias (only when a weight per coordinate is
        # the norm's one factor)
        self.gamma = self.weight if self.gain is None else None
        self.beta = None
        self.centred = False

    def forward(self, ctx, x, out, rows=None) -> None:
        ops.rms_norm(x, out=out, gain=self.gain, weight=self.weight, rows=rows, eps=self.eps,
                     status=ctx.status)

    def joined(self, ctx, x, y, alpha: float, gate=None, gate_bias=None, copy=None) -> None:
        ops.rms_norm(x, out=copy, x_out=x, y=y, gate=gate, gate_bias=gate_bias, gain=self.gain,
                     weight=self.weight, alpha=alpha, eps=self.eps, status=ctx.status)


    def added(self, ctx, x, y, copy=None) -> None:
        ops.rms_norm(x, out=copy, x_out=x, y=y, gain=self.gain, weight=self.weight, eps=self.eps,
                     status=ctx.status, branch_only=True)


def _rms_norm(params, store, runtime) -> RMSNorm:
    """``scale`` (optional): a constant the result is multiplied by (a head that scales its
    logits has the constant here, in the 32-bit weight, instead of a pass over the logits).
    ``offset`` (optional): the stored weight lies around zero and the norm multiplies by
    offset + weight (in 32-bit)."""
    gain = store.get(params["gain"]) if params.get("gain") else None
    weight = store.get(params["weight"]) if params.get("weight") else None
    offset = float(params.get("offset", 0.0))
    if offset != 0.0:
        if weight is None:
            raise ValueError("rms_norm: an offset belongs to a weight per coordinate")
        weight = weight.to(torch.float32) + offset
    scale = float(params.get("scale", 1.0))
    if scale != 1.0:
        weight = (torch.ones(params["size"], dtype=torch.float32, device=runtime.device)
                  if weight is None else weight.to(torch.float32)) * scale
    return RMSNorm(gain, weight, params["eps"], params["size"])


register_part("norm", "layer_norm", _layer_norm)
register_part("norm", "rms_norm", _rms_norm)
