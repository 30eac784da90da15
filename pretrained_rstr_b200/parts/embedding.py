"""Token embedding: x[t] = table[token[t]] + position row, gathered on the device from
token ids (the reference builds prompt embeddings on the host,
``src/pretrained/continuation/paged_decoder.clj:683-693``; here only ids cross)."""
from __future__ import annotations

import torch

from ..csrc import ops
from .interfaces import Embedding, StateSpec
from .registry import register_part


class TokenEmbedding(Embedding):
    graph_safe = True
    def __init__(self, table: torch.Tensor, vocab: int, width: int, runtime):
        if tuple(table.shape) != (vocab, width):
            raise ValueError(f"token_embedding: table is {list(table.shape)}, "
                             f"expected [{vocab}, {width}]")
        self.table = table.to(runtime.dtype).contiguous()
        self.vocab, self.width = vocab, width

    def forward(self, ctx, position, x) -> None:
        ops.embed(x, ctx.tokens, ctx.positions, self.table, position.table(), ctx.status)


class ScaledTokenEmbedding(Embedding):
    """x[t] = table[token[t]] * scale.  ``keeps_copy``: the rows can be left a second time in
    ``keep`` (for a run order that adds the embedding's output to the stream again)."""
    graph_safe = True
    keeps_copy = True

    def __init__(self, table: torch.Tensor, vocab: int, width: int, scale: float, runtime):
        if tuple(table.shape) != (vocab, width):
            raise ValueError(f"scaled_token_embedding: table is {list(table.shape)}, "
                             f"expected [{vocab}, {width}]")
        self.table = table.to(runtime.dtype).contiguous()
        self.vocab, self.width, self.scale = vocab, width, float(scale)

    def forward(self, ctx, position, x, keep=None) -> None:
        if position.table() is not None:
            raise ValueError("scaled_token_embedding adds no position table")
        ops.embed_scaled(x, ctx.tokens, self.table, self.scale, keep=keep, status=ctx.status)


class TokenPairEmbedding(Embedding):
    """x[t] = table[token] * scale + pairs[row]: a second table indexed by a hash of (previous token,
    token), row = (prev * mul_prev + token * mul_cur) mod buckets; a sequence's first token
    takes row ``buckets``.  The previous token of every request is state: one int32 per state
    slot on the device, read and brought up to date by the embedding kernel itself, so steps
    whose token ids are only known on the device work like any other."""
    graph_safe = True

    def __init__(self, table: torch.Tensor, pairs: torch.Tensor, vocab: int, width: int,
                 buckets: int, mul_prev: int, mul_cur: int, runtime, scale: float = 1.0):
        self.scale = float(scale)
        if tuple(table.shape) != (vocab, width) or tuple(pairs.shape) != (buckets + 1, width):
            raise ValueError(f"token_pair_embedding: tables are {list(table.shape)} and "
                             f"{list(pairs.shape)}, expected [{vocab}, {width}] and "
                             f"[{buckets + 1}, {width}]")
        self.table = table.to(runtime.dtype).contiguous()
        self.pairs = pairs.to(runtime.dtype).contiguous()
        self.vocab, self.width = vocab, width
        self.buckets, self.mul_prev, self.mul_cur = int(buckets), int(mul_prev), int(mul_cur)
        self.prev = None

    def state_specs(self):
        return [StateSpec("previous_token", (), torch.int32)]

    def bind_state(self, state) -> None:
        self.prev = state["previous_token"]

    def forward(self, ctx, position, x) -> None:
        if position.table() is not None:
            raise ValueError("token_pair_embedding adds no position table")
        ops.embed_pair(x, ctx.tokens, ctx.positions, ctx.seq_of_token, ctx.q_start, ctx.state_slot,
                       self.prev, self.table, self.pairs, self.buckets, self.mul_prev,
                       self.mul_cur, ctx.status, scale=self.scale)


register_part("embedding", "token_embedding",
              lambda p, store, rt: TokenEmbedding(
                  store.get(p["weights"] + p.get("suffix", ".weight"), rt.dtype),
                  p["vocab"], p["width"], rt))
register_part("embedding", "scaled_token_embedding",
              lambda p, store, rt: ScaledTokenEmbedding(
                  store.get(p["weights"], rt.dtype), p["vocab"], p["width"], p["scale"], rt))
register_part("embedding", "token_pair_embedding",
              lambda p, store, rt: TokenPairEmbedding(
                  store.get(p["table"], rt.dtype), store.get(p["pairs"], rt.dtype), p["vocab"],
                  p["width"], p["buckets"], p["mul_prev"], p["mul_cur"], rt,
                  scale=p.get("scale", 1.0)))
