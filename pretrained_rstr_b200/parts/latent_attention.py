"""Causal attention over one low-rank latent per token (``latent_attention``).

Per token the mixer keeps ONE row that all heads share: the normed latent c (``kv_rank``
numbers) from which a head's keys and values would be expanded, k_h = Uk_h c and
v_h = Uv_h c, and a rotated key part r (``rot_dim`` numbers) common to the heads.  Queries
pass a latent of their own, q = Uq norm(Dq h), or (``q_rank`` None) are one matrix, q = Wq h;
per head [``dim`` plain | ``rot_dim`` rotated].
The score of head h is (q_plain . k_h + q_rot . r) * scale; a learned sink per head may join
the softmax's denominator; a head's result may be gated by sigmoid(G h)_h (``head_gate``), or
the concatenated heads element by element by sigmoid(G h) (``value_gate``); the output
projection follows.  ``window``: position i sees j with 0 <= i - j < window.  The rotation
pairs coordinate i with i + rot_dims / 2 (``rot_layout`` "half") or 2i with 2i + 1
("interleaved": the rows of the rotated parts are reordered once, when the model is built,
which leaves every score as it is); ``rot_scaling`` (factor, original, fast, slow): YaRN's
frequencies, and its magnitude on cos and sin of both sides, which is one constant on the
cached rotated key part.

Nothing is expanded per key.  The query is folded through Uk once per token,
qa_h = [Uk_h^T q_plain | q_rot], so that the score is qa_h . [c | r] and the head's result
Uv_h (sum_j w_j c_j): the attention kernels read one row of ``kv_rank + rot_dim`` numbers per
key for all heads, which is what the cache holds (a group with one pool per layer and one
"head").  Sizes, the rotation's base and reach, the scale, the sink and the gate are
parameters.

Two ways through a step.  float32 (and bfloat16 sizes the tensor-core kernel does not take):
Uq, then per head the fold through Uk with the rotation, the 32-bit attention kernel, the
unfold through Uv with the gate, the output projection.  bfloat16 on tensor cores: Uk is
folded into Uq and Uv into the output projection when the model is built (in 32-bit, rounded
once), so a step is the folded query product, the attention kernel, which rotates the
queries as it loads them and leaves the gated sums in bfloat16, and the folded output
product: three kernels fewer, and the per-head matrices run at the products' speed.  With a
gate per value coordinate Uv cannot move into the output projection (the gate acts between
them): steps of few rows expand the values per head (``latent_unfold``), steps of many rows
as one product with all heads' Uv along the diagonal, followed by the gate.

The first matrix product carries Dq, Dkv and G in one, and whatever rows an arrangement
asks to ride along (:meth:`fuse_input_rows`); its float32 result feeds the norms unrounded.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..csrc import ops
from ..engine.batch import WorkPlanner
from .interfaces import KVSpec, LayerCache, Mixer
from .linear import Linear, padded_linear
from .registry import register_part


def _pad8(n: int) -> int:
    return -(-n // 8) * 8


class FusedInput:
    """One matrix product for several consumers of the same input: segments of rows, each
    starting at a multiple of 8 columns of the float32 result.  Segments are added while the
    model is built; the matrix is put together at the first use."""

    def __init__(self, width: int, runtime, key: str):
        self.width, self.runtime, self.key = width, runtime, key
        self._parts: List[Tuple[str, torch.Tensor]] = []
        self.cols: Dict[str, Tuple[int, int]] = {}          # name -> (first column, columns)
        self._linear: Optional[Linear] = None

    def add(self, name: str, weight: torch.Tensor) -> str:
        if self._linear is not None:
            raise RuntimeError("the fused product is built already")
        if weight.dim() != 2 or weight.shape[1] != self.width:
            raise ValueError(f"{name}: expected [rows, {self.width}], found {list(weight.shape)}")
        self._parts.append((name, weight))
        return name

    def linear(self) -> Linear:
        if self._linear is None:
            rows, at = [], 0
            for name, w in self._parts:
                self.cols[name] = (at, w.shape[0])
                rows.append(w.to(self.runtime.dtype))
                pad = _pad8(w.shape[0]) - w.shape[0]
                if pad:
                    rows.append(torch.zeros((pad, self.width), dtype=self.runtime.dtype,
                                            device=w.device))
                at += w.shape[0] + pad
            self._linear = Linear(torch.cat(rows, dim=0), None, self.runtime)
            self._parts = []
        return self._linear

    def run(self, ctx, h) -> torch.Tensor:
        lin = self.linear()
        t = h.shape[0]
        out = ctx.scratch(self.key, (ctx.token_capacity, lin.n_out), torch.float32)[:t]
        lin.forward(ctx, h, out)
        return out

    def view(self, out: torch.Tensor, name: str) -> torch.Tensor:
        at, n = self.cols[name]
        return out[:, at:at + n]


class LatentWork(WorkPlanner):
    """How the tensor-core kernel cuts a step.  A request that brings one token is a
    "single": an item of its own whose CTAs split the keys.  A portion of a prompt goes in
    "tiles" of consecutive tokens, as many as fit a CTA's 128 (token, head) rows: 128 // heads,
    so mixers with other head counts have lists of their own (``tile_row0_<tokens>``)."""

    key = "latent_attention"
    ROWS = 128

    def __init__(self):
        self.tile_tokens = set()           # tokens per tile of the mixers that use the lists

    def note_mixer(self, heads: int) -> int:
        tq = max(1, self.ROWS // int(heads))
        self.tile_tokens.add(tq)
        return tq

    def absorb(self, other: "LatentWork") -> None:
        self.tile_tokens |= other.tile_tokens

    @property
    def counters(self):
        return ("singles",) + tuple(f"tiles_{tq}" for tq in sorted(self.tile_tokens))

    def arrays(self, t_cap: int, b_cap: int):
        out = {"single_row0": (min(t_cap, b_cap), 0)}
        for tq in sorted(self.tile_tokens):
            cap = t_cap // tq + b_cap
            out[f"tile_row0_{tq}"] = (cap, 0)
            out[f"tile_tokens_{tq}"] = (cap, 0)
        return out

    def fill(self, arrays: Dict[str, np.ndarray], lengths: Sequence[int]) -> Dict[str, int]:
        counts = {name: 0 for name in self.counters}
        used = []
        if max(lengths) == 1:                   # a decode step
            n = len(lengths)
            arrays["single_row0"][:n] = np.arange(n, dtype=np.int32)
            counts["singles"] = n
            return {**counts, "_used": ["single_row0"]}
        t = 0
        sing = arrays["single_row0"]
        for n in lengths:
            if n == 1:
                sing[counts["singles"]] = t
                counts["singles"] += 1
            else:
                for tq in self.tile_tokens:
                    row0, toks = arrays[f"tile_row0_{tq}"], arrays[f"tile_tokens_{tq}"]
                    k = counts[f"tiles_{tq}"]
                    for r0 in range(0, n, tq):
                        row0[k] = t + r0
                        toks[k] = min(tq, n - r0)
                        k += 1
                    counts[f"tiles_{tq}"] = k
            t += n
        if counts["singles"]:
            used.append("single_row0")
        for tq in self.tile_tokens:
            if counts[f"tiles_{tq}"]:
                used += [f"tile_row0_{tq}", f"tile_tokens_{tq}"]
        return {**counts, "_used": used}


def key_splits(items: int, max_context: int, most: int, sm_count: int):
    """(keys per range, ranges) for a launch of ``items`` work items over contexts of up to
    ``max_context`` keys: about two CTAs per SM, ranges of whole 64-key blocks (measured, 8
    decoded tokens at 1,024 keys: 27.7 us in ranges of one block, 31.8 of two, 52 of eight; 64
    tokens: 46 us in ranges of four blocks, 58 of two)."""
    blocks = max(1, -(-max_context // 64))
    wanted = max(1, min(most, -(-2 * sm_count // max(1, items)), blocks))
    split_keys = -(-blocks // wanted) * 64
    return split_keys, -(-blocks * 64 // split_keys)


class LatentAttention(Mixer):
    graph_safe = True
    can_overwrite = True

    def __init__(self, p: dict, store, runtime):
        w = p["weights"]
        self.width, self.heads, self.dim = p["width"], p["heads"], p["dim"]
        self.rot_dim, self.vdim = p["rot_dim"], p["vdim"]
        self.rank, self.q_rank = p["kv_rank"], p.get("q_rank")
        self.scale, self.eps = float(p["scale"]), float(p["eps"])
        self.rot_dims, self.window = int(p.get("rot_dims", self.rot_dim)), p.get("window")
        self.runtime = runtime
        dtype, dev = runtime.dtype, runtime.device
        hd = self.dim + self.rot_dim

        def need(name, shape):
            t = store.get(w[name])
            if tuple(t.shape) != tuple(shape):
                raise ValueError(f"{w[name]}: expected {list(shape)}, found {list(t.shape)}")
            return t

        layout = p.get("rot_layout", "half")
        if layout not in ("half", "interleaved"):
            raise ValueError(f"latent_attention: unknown rot_layout {layout!r}")
        if self.rot_dims % 2 or self.rot_dims > self.rot_dim:
            raise ValueError(f"latent_attention: {self.rot_dims} rotated coordinates of {self.rot_dim}")
        # interleaved pairs (2i, 2i + 1) become (i, i + rot_dims / 2): the same reordering of
        # the rotated query rows and the rotated key rows leaves every dot product as it is
        order = list(range(self.rot_dim))
        if layout == "interleaved":
            order = list(range(0, self.rot_dims, 2)) + list(range(1, self.rot_dims, 2)) + \
                list(range(self.rot_dims, self.rot_dim))
        order = torch.tensor(order, dtype=torch.long)

        def reorder_q(m):          # [heads * hd, in]: the last rot_dim rows of every head
            m = m.reshape(self.heads, hd, m.shape[-1])
            return torch.cat([m[:, :self.dim], m[:, self.dim:][:, order.to(m.device)]], dim=1) \
                .reshape(self.heads * hd, -1)

        kv_down = need("kv_down", (self.rank + self.rot_dim, self.width))
        kv_down = torch.cat([kv_down[:self.rank], kv_down[self.rank:][order.to(kv_down.device)]], dim=0)
        self.input = FusedInput(self.width, runtime, "latent_in")
        self.tensor_cores = dtype == torch.bfloat16 and torch.cuda.is_available() and \
            ops.latent_mma_supports(self.heads, self.rank, self.rot_dim)
        if self.q_rank is not None:
            self.input.add("q", need("q_down", (self.q_rank, self.width)))
            self.q_norm = need("q_norm", (self.q_rank,)).to(torch.float32).contiguous()
            q_up = reorder_q(need("q_up", (self.heads * hd, self.q_rank)))
        else:
            self.q_norm = None
            q_up = reorder_q(need("q", (self.heads * hd, self.width)))
            if not self.tensor_cores:
                self.input.add("q", q_up)          # the query rides in the first product
        self.input.add("kv", kv_down)
        self.value_gate = bool(p.get("value_gate", False))
        self.head_gate = bool(p.get("head_gate", False)) or self.value_gate
        if self.head_gate:
            rows = self.heads * self.vdim if self.value_gate else self.heads
            self.input.add("gate", need("gate", (rows, self.width)))
        self.kv_norm = need("kv_norm", (self.rank,)).to(torch.float32).contiguous()
        self.sinks = need("sink", (self.heads,)).to(torch.float32).contiguous() \
            if p.get("sink", False) else None
        # bfloat16 serving: the tensor-core kernel where it takes the sizes, else (and in
        # float32) the 32-bit-arithmetic kernel
        q_in = self.q_rank if self.q_rank is not None else self.width
        k_up = need("k_up", (self.heads * self.dim, self.rank))
        v_up = need("v_up", (self.heads * self.vdim, self.rank))
        out = need("out", (self.width, self.heads * self.vdim))
        if self.tensor_cores:
            # Uk and Uv are folded into their neighbours once, in 32-bit: the query comes out
            # of ONE product as [Uk_h^T q_plain | q_rot] per head, and the output projection
            # takes the heads' gated latent sums as they leave the attention kernel
            uq = q_up.to(torch.float32).reshape(self.heads, hd, q_in)
            uk = k_up.to(torch.float32).reshape(self.heads, self.dim, self.rank)
            folded = torch.einsum("hdr,hdq->hrq", uk, uq[:, :self.dim])
            self.q_fold = padded_linear(
                torch.cat([folded, uq[:, self.dim:]], dim=1).reshape(
                    self.heads * (self.rank + self.rot_dim), q_in), runtime)
            uv = v_up.to(torch.float32).reshape(self.heads, self.vdim, self.rank)
            wo = out.to(torch.float32).reshape(self.width, self.heads, self.vdim)
            # (a gate per value coordinate acts between Uv and the output projection: they
            # stay two products then)
            self.out_fold = None if self.value_gate else padded_linear(
                torch.einsum("whv,hvr->whr", wo, uv).reshape(self.width, self.heads * self.rank),
                runtime)
        if not self.tensor_cores or self.value_gate:
            self.uvt = v_up.to(dtype).reshape(self.heads, self.vdim, self.rank) \
                .transpose(1, 2).contiguous()
            self.out = padded_linear(out, runtime)
        self.uv_blocks = None
        if self.tensor_cores and self.value_gate:
            # for steps of many rows: all heads' Uv as ONE product with the matrices along the
            # diagonal (heads times the needed arithmetic, on tensor cores, for a fraction of the
            # per-head kernel's time); steps of few rows keep the per-head kernel, which reads
            # the needed weights only
            uvb = torch.zeros((self.heads * self.vdim, self.heads * self.rank), dtype=torch.float32,
                              device=v_up.device)
            for hh in range(self.heads):
                uvb[hh * self.vdim:(hh + 1) * self.vdim, hh * self.rank:(hh + 1) * self.rank] = \
                    v_up[hh * self.vdim:(hh + 1) * self.vdim].to(torch.float32)
            self.uv_blocks = padded_linear(uvb, runtime)
        if not self.tensor_cores:
            self.q_up = padded_linear(q_up, runtime) if self.q_rank is not None else None
            self.uk = k_up.to(dtype).contiguous()
        half = self.rot_dims // 2
        base = float(p.get("rot_base", 10000.0))
        self.rot_scale = 1.0
        yarn = p.get("rot_scaling")
        if yarn:
            from .positions_rotary import yarn_frequencies
            (self.freq, self.freq_lo), mag = yarn_frequencies(
                base, self.rot_dims, float(yarn["factor"]), float(yarn["original"]),
                float(yarn["fast"]), float(yarn["slow"]), dev, with_lo=True)
            self.rot_scale = mag * mag         # both sides' magnitudes, on the cached key part
        else:
            from .positions_rotary import split_frequencies
            self.freq, self.freq_lo = split_frequencies(
                [base ** (-2.0 * i / self.rot_dims) for i in range(half)] or [0.0], dev)
        self.work_plan = LatentWork()
        self.tile_tokens = self.work_plan.note_mixer(self.heads)
        self.sm_count = ops.sm_count() if torch.cuda.is_available() else 148

    def work_planners(self):
        return [self.work_plan] if self.tensor_cores else []

    # ------------------------------------------------------------------ structure
    def kv_spec(self) -> KVSpec:
        return KVSpec(1, self.rank + self.rot_dim, self.window, values=False)

    def fuse_input_rows(self, name: str, weight: torch.Tensor) -> str:
        """Rows that read the mixer's input and ride along in its first product; their float32
        result is ``fused_rows(name)`` after :meth:`forward`."""
        return self.input.add(name, weight)

    def fused_rows(self, name: str) -> torch.Tensor:
        return self.input.view(self._proj, name)

    # -------------------------------------------------------------------- forward
    def forward(self, ctx, h, x, cache: LayerCache, accumulate: bool = True) -> None:
        t = x.shape[0]
        cap, dtype = ctx.token_capacity, self.runtime.dtype
        group = ctx.groups[cache.group]
        proj = self._proj = self.input.run(ctx, h)
        cols = self.input.cols
        first = self.q_fold if self.tensor_cores else self.q_up
        latent_q = self.q_rank is not None
        cq = ctx.scratch_zero("latent_cq", (cap, first.n_in), dtype)[:t] if latent_q else None
        ops.latent_prepare(cq, cache.k, proj, cols["q"][0] if latent_q else 0, cols["kv"][0],
                           self.q_norm, self.kv_norm, group.slots if cache.writes else None,
                           ctx.positions, self.freq, self.q_rank or 0, self.rank, self.rot_dim,
                           self.rot_dims, self.eps, ctx.status, rot_scale=self.rot_scale,
                           freq_lo=self.freq_lo)
        gate = self.input.view(proj, "gate") if self.head_gate else None
        width = self.rank + self.rot_dim
        if self.tensor_cores:
            # the folded query leaves its product in bfloat16; the attention kernel rotates
            # the rows' last parts as it loads them
            qa = ctx.scratch("latent_qa", (cap, self.heads, width), dtype)[:t]
            first.forward(ctx, cq if latent_q else h, qa.view(t, self.heads * width))
            if self.value_gate:
                o = ctx.scratch_zero("latent_o", (cap, self.out.n_in), dtype)[:t]
                if ctx.layout.t_cap > self.UNFOLD_ROWS:
                    sums = ctx.scratch("latent_gated", (cap, self.heads, self.rank), dtype)[:t]
                    self._attend_tensor_cores(ctx, sums, qa, cache, group, None)
                    val = ctx.scratch("latent_values", (cap, self.heads * self.vdim), torch.float32)[:t]
                    self.uv_blocks.forward(ctx, sums.view(t, self.heads * self.rank), val)
                    ops.gate_mul(o, val, gate)
                else:
                    lat = ctx.scratch("latent_sum", (cap, self.heads, self.rank), torch.float32)[:t]
                    self._attend_tensor_cores(ctx, lat, qa, cache, group, None)
                    ops.latent_unfold(o, lat, self.uvt, gate, self.heads, self.rank, self.vdim)
                self.out.forward(ctx, o, x, resid=x if accumulate else None)
                return
            gated = ctx.scratch("latent_gated", (cap, self.heads, self.rank), dtype)[:t]
            self._attend_tensor_cores(ctx, gated, qa, cache, group, gate)
            self.out_fold.forward(ctx, gated.view(t, self.heads * self.rank), x,
                                  resid=x if accumulate else None)
            return
        if latent_q:
            q = ctx.scratch("latent_q", (cap, first.n_out), torch.float32)[:t]
            first.forward(ctx, cq, q)
        else:
            q = self.input.view(proj, "q")
        qa = ctx.scratch("latent_qa", (cap, self.heads, width), torch.float32)[:t]
        ops.latent_fold(qa, q, self.uk, ctx.positions, self.freq, self.heads, self.dim,
                        self.rot_dim, self.rot_dims, self.rank, freq_lo=self.freq_lo)
        lat = ctx.scratch("latent_sum", (cap, self.heads, self.rank), torch.float32)[:t]
        attend_latent(ctx, lat, qa, cache, group, self.sinks, self.scale, self.window, self.rank)
        o = ctx.scratch_zero("latent_o", (cap, self.out.n_in), dtype)[:t]
        ops.latent_unfold(o, lat, self.uvt, gate, self.heads, self.rank, self.vdim)
        self.out.forward(ctx, o, x, resid=x if accumulate else None)


    #: most key ranges of a launch: single tokens, prompt tiles
    MAX_SPLITS = (32, 8)
    #: steps with room for more token rows than this expand the values of all heads as one
    #: product (a gate per value coordinate keeps Uv apart from the output projection)
    UNFOLD_ROWS = 64

    def _attend_tensor_cores(self, ctx, lat, qa, cache: LayerCache, group, gate=None) -> None:
        """Single tokens and prompt tiles as two launches (each only if the step has such
        work; a step that is replayed from a graph launches a list's capacity and lets the
        device-side count bound it)."""
        work = ctx.work[LatentWork.key]
        tq = self.tile_tokens
        lists = (("singles", "single_row0", None, ops.latent_mma_single_kw(self.heads), self.heads,
                  self.MAX_SPLITS[0]),
                 (f"tiles_{tq}", f"tile_row0_{tq}", f"tile_tokens_{tq}", 1, LatentWork.ROWS,
                  self.MAX_SPLITS[1]))
        for counter, rows_name, tokens_name, kw, ws_rows, most in lists:
            count = work.host_counts[counter]
            if count == 0:
                continue
            cap = work.caps[rows_name]
            n = cap if count is None else count
            most = max(1, min(most, 2 * self.sm_count // cap))     # (bounds the workspace too)
            split_keys, splits = key_splits(n, ctx.max_context, most, self.sm_count)
            slots = cap * ws_rows * most
            ws_o = ctx.scratch("latent_part_o", (slots * self.rank,), torch.float32)
            ws_ml = ctx.scratch("latent_part_ml", (slots * 2,), torch.float32)
            ops.latent_attention_mma(
                lat, qa, cache.k, group.block_table, ctx.seq_of_token, ctx.positions,
                work.arrays[rows_name], work.arrays[tokens_name] if tokens_name else None,
                work.counts[counter], n, self.sinks, ws_o, ws_ml, self.scale, self.window,
                self.rank, split_keys, splits, kw, ws_rows, ctx.status, gate=gate,
                rotate=(self.freq, self.rot_dims))


def attend_latent(ctx, lat, qa, cache: LayerCache, group, sinks, scale: float,
                  window: Optional[int], rank: int) -> None:
    """lat[t, h] = sum_j w_j c_j over the rows token t sees in its request's pages."""
    ops.latent_attention(lat, qa, cache.k, group.block_table, ctx.seq_of_token, ctx.positions,
                         sinks, scale, window, rank, ctx.status)


register_part("mixer", "latent_attention", lambda p, store, rt: LatentAttention(p, store, rt))
