"""Designs side by side: prefill and decode throughput of named sizes with random weights,
whatever their architecture, with what the rooflines allow, and the device time of every
kernel of one decode step and one prompt step.

A size is a name of ``config.registry.named_sizes()`` (``small`` and ``xl`` are GPT-2's;
``redisun-small``, ``redisun-small-moe`` and ``redisun-wide`` have the same width, depth,
head count and vocabulary with Redisun's parts).  Bytes and operations are counted from the
tensors a model holds and the cache rows its mixers declare, not from formulas per design."""
from __future__ import annotations

import shutil
import statistics
import tempfile
from typing import Dict, Optional, Sequence

from .roofline import peaks
from .workloads import timed_decode, timed_prefill


def load_size(name: str, layers: Optional[int] = None, max_lanes: int = 64,
              max_batched_tokens: int = 2048, maxpos: int = 1024):
    """(LM, raw config) of a named size with seeded random weights in bfloat16; with
    ``layers`` only that many of its layers (named in the record)."""
    import torch
    from .. import load_lm
    from ..config.registry import lookup, named_sizes
    from ..weights import make_random_model
    raw = dict(named_sizes()[name])
    if layers:
        if "n_layer" in raw:
            raw["n_layer"] = layers
        else:
            raw["layers"] = list(raw["layers"])[:layers]
    cfg = lookup(raw).config_class.from_dict(raw)
    tmp = tempfile.mkdtemp(prefix="prb200_design_")
    try:
        make_random_model(tmp, cfg, seed=2, dtype=torch.bfloat16)
        m = load_lm(tmp, gpu=True, dtype="bfloat16", max_lanes=max_lanes,
                    max_batched_tokens=max_batched_tokens, prefill_chunk=1024,
                    share_prefixes=False, maxpos=maxpos)
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    return m, raw


def weight_bytes(m) -> int:
    """Bytes of every matrix and table a decode step reads once (the token tables apart,
    of which a step reads a row per token; the head's matrix counts)."""
    from ..config.registry import lookup
    arch = lookup(m.config.to_dict())
    total = 0
    head = m.config.head_spec().params.get("weights")      # (a token table that is the head counts)
    for name, exp in arch.expected_tensors(m.config).items():
        n = 1
        for s in exp.shape:
            n *= s
        if name in ("wpe.weight", "embed", "bigram") and name != head:
            continue
        total += 2 * n
    return total


def matrix_flops_per_token(m) -> int:
    """Multiply-adds x 2 of every matrix a token passes (token tables apart; the head's once
    per wanted row is left out)."""
    from ..config.registry import lookup
    arch = lookup(m.config.to_dict())
    total = 0
    for name, exp in arch.expected_tensors(m.config).items():
        if len(exp.shape) == 2 and name not in ("wte.weight", "wpe.weight", "embed", "bigram", "head"):
            total += 2 * exp.shape[0] * exp.shape[1]
    return total


def cache_bytes_per_token(m) -> int:
    return sum(g.pools_per_layer * len(g.layers) * g.kv_heads * g.head_dim * 2
               for g in m.loaded.model.group_specs)


def _mixers(m):
    """Every mixer of the model's layer runs (the two of a pair side by side apart)."""
    for block in m.loaded.model.blocks:
        mixer = getattr(block, "mixer", None)
        if mixer is not None:
            yield from getattr(mixer, "children", [mixer])


def request_bytes(m, context: int) -> int:
    """Bytes a decode step reads (and, for running states, writes back) for ONE request that
    holds ``context`` tokens: mixers that say so themselves (``step_bytes(context)``: a window's
    keys, a layer that reads another's cache, a state) are asked; the others count every cache
    row of the context."""
    asked = [mx.step_bytes(context) for mx in _mixers(m) if hasattr(mx, "step_bytes")]
    if asked:
        return sum(asked)
    return context * cache_bytes_per_token(m)


def measure_size(name: str, batches: Sequence[int] = (1, 8, 64), context: int = 1000,
                 steps: int = 32, warmup: int = 4, layers: Optional[int] = None) -> Dict:
    m, raw = load_size(name, layers)
    pk = peaks()
    vocab = m.loaded.model.vocab
    wbytes, kvb, mflops = weight_bytes(m), cache_bytes_per_token(m), matrix_flops_per_token(m)
    out = {"layers": len(m.loaded.model.blocks), "weight_mb": round(wbytes / 1e6, 1),
           "cache_bytes_per_token": kvb, "request_bytes_at_context": request_bytes(m, context),
           "matrix_gflop_per_token": round(mflops / 1e9, 4)}
    pre = statistics.median(timed_prefill(m.loaded, 2, 1024, vocab))
    out["prefill_2x1024"] = {"ms": round(pre, 4), "tokens_per_s": round(2048 / (pre / 1e3)),
                             "matrix_frac_of_bf16_peak": round(
                                 2048 * mflops / (pre / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
    for b in batches:
        res = timed_decode(m.engine, b, context, steps, warmup, vocab, 1000 * b + context)
        ms = statistics.mean(res["ms"])
        nbytes = wbytes + b * request_bytes(m, int(res["mean_context"]))
        out[f"decode_b{b}"] = {"ms": round(ms, 4), "tokens_per_s": round(b / (ms / 1e3)),
                               "e2e_tokens_per_s": round(b * steps / res["wall_s"]),
                               "launches_per_step": round(res["launches"] / steps, 1),
                               "hbm_frac": round(nbytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 4)}
    return out


def kernel_table(name: str, batch: int = 8, context: int = 900, layers: Optional[int] = None,
                 rows: int = 14) -> Dict[str, list]:
    """Device time by kernel (torch profiler, kernels launched one by one) of four decode steps
    of ``batch`` requests at ``context`` tokens and of one step of 2 x 1,024 prompt tokens:
    name -> (calls, microseconds per call)."""
    import random
    import torch
    from torch.profiler import ProfilerActivity, profile
    from ..engine.batch import Entry
    m, raw = load_size(name, layers)
    e = m.engine
    e.runner.use_graphs = False
    vocab = m.loaded.model.vocab
    rng = random.Random(0)
    out = {}

    def table(prof):
        evs = sorted(prof.key_averages(), key=lambda ev: -ev.device_time_total)[:rows]
        return [(ev.key[:60], ev.count, round(ev.device_time_total / max(1, ev.count), 2))
                for ev in evs if ev.device_time_total > 0]

    for i in range(batch):
        e.submit(("k", i), [rng.randrange(vocab) for _ in range(context)], 64)
    while any(r.phase != "decode" for r in e.scheduler.running.values()) or e.scheduler.waiting:
        e.step()
    e.step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(4):
            e.step()
        torch.cuda.synchronize()
    out["decode"] = table(prof)
    for i in range(batch):
        e.cancel(("k", i))
    while e.scheduler.running:
        e.step()
    runner, cache = m.loaded.runner, m.loaded.cache

    def prompt_step(tag):
        entries = []
        for i in range(2):
            cache.open((tag, i))
            entries.append(Entry((tag, i), [rng.randrange(vocab) for _ in range(1024)], [1023]))
        runner.step(entries)
        torch.cuda.synchronize()
        for en in entries:
            cache.close(en.rid)

    prompt_step("warm")
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        prompt_step("timed")
    out["prefill"] = table(prof)
    return out
