"""Python face of the CUDA library: loads it (building it on first use) and wraps each
exported C function in a call that takes torch tensors.

There is no fallback: if the library cannot be built or loaded, or no CUDA device is
present, :func:`lib` raises :class:`ExtensionError`.  Wrappers check devices, element
types and contiguity, pass raw pointers and the current torch stream, and turn a
non-zero return code into an exception that names the refused argument.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_long, c_void_p
from typing import Optional

import torch

from . import build as _build

F32, BF16 = 0, 1
ACT_CODES = {None: 0, "none": 0, "gelu_new": 1, "gelu_pytorch_tanh": 1, "gelu": 2, "relu": 3}

_ERRORS = {
    -2: "unknown element type",
    -3: "a size this kernel does not take",
    -4: "a pointer or stride that is not aligned as the kernel requires",
    -5: "bad argument",
    -6: "the device or driver lacks a feature the kernel needs",
}
STATUS_TEXT = {
    1: "token id outside the vocabulary (token index, id, vocabulary size)",
    2: "position outside the position table or the cache (token index, position, limit)",
    3: "cache slot outside the pool (token index, slot, pages)",
    4: "block-table entry missing or outside the pool (token index, position, page)",
    5: "a bounded wait inside a kernel gave up (kernel id, block, stage)",
    6: "row index outside its tensor (row, index, rows)",
}


class ExtensionError(RuntimeError):
    pass


class KernelArgumentError(ValueError):
    pass


_LIB = None


def lib() -> ctypes.CDLL:
    """The loaded library; builds it at the first call."""
    global _LIB
    if _LIB is None:
        try:
            path = _build.build()
            handle = ctypes.CDLL(path)
        except (OSError, _build.BuildError) as exc:
            raise ExtensionError(
                f"the CUDA extension of pretrained_rstr_b200 is not available: {exc}") from exc
        _declare(handle)
        _LIB = handle
    return _LIB


def library_path() -> str:
    return _build.build()


def require_cuda() -> None:
    if not torch.cuda.is_available():
        raise ExtensionError("pretrained_rstr_b200 runs on a CUDA device only (sm_100a); "
                             "torch.cuda.is_available() is False and there is no CPU path")


def _declare(h: ctypes.CDLL) -> None:
    P, I, L, F = c_void_p, c_int, c_long, c_float
    h.prb_embed.argtypes = [P, P, P, P, P, I, I, I, I, I, P, P]
    h.prb_layernorm.argtypes = [P, P, P, P, P, I, I, I, F, I, P, P]
    h.prb_bias_act.argtypes = [P, P, P, P, I, I, I, I, I, P]
    h.prb_kv_append.argtypes = [P, P, P, P, L, P, I, I, I, I, I, I, P, P]
    h.prb_copy_pages.argtypes = [P, P, I, L, I, I, P, P]
    h.prb_resolve_tokens.argtypes = [P, I, P, I, P, P]
    h.prb_host_device_address.argtypes = [P]
    h.prb_host_device_address.restype = c_void_p
    h.prb_fetch_step.argtypes = [P, P, I, I, I, P, I, P, P]
    h.prb_publish_result.argtypes = [P, P, I, P]
    h.prb_gemm_f32.argtypes = [P, P, P, P, P, I, I, I, L, L, L, I, P]
    h.prb_gemm_bf16.argtypes = [P, P, P, P, P, I, I, I, L, L, L, I, I, I, P, P]
    h.prb_gemm_bf16_scatter.argtypes = [P, P, P, P, I, I, I, L, L, L, I, I, P, P, P, I, I, I, I, I,
                                        I, P, P]
    h.prb_gemm_midm.argtypes = [P, P, P, P, P, I, I, I, L, L, L, I, I, P, P]
    h.prb_gemm_midm_supports.argtypes = [I, I, I]
    h.prb_gemm_smallm.argtypes = [P, P, P, P, I, P, P, F, P, P, P, I, I, I, L, L, L, I, I,
                                  P, P, P, I, I, I, I, I, I, P, P]
    h.prb_gemm_smallm_max_rows.argtypes = []
    h.prb_gemm_smallm_max_norm_width.argtypes = []
    h.prb_attention_generic.argtypes = [P, L, P, L, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I,
                                        I, P, P]
    h.prb_attention_decode.argtypes = [P, L, P, L, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I,
                                       P, P, I, I, P, P]
    h.prb_attention_decode_ring.argtypes = [P, L, P, L, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F,
                                            I, I, P, P, L, P, P, I, I, P, P]
    h.prb_attention_decode_ring_tune.argtypes = [I, I]
    h.prb_attention_decode_ring_tune.restype = c_int
    h.prb_attention_decode_ring.restype = c_int
    h.prb_attention_decode_ring_supports.argtypes = [I, I]
    h.prb_attention_decode_ring_supports.restype = c_int
    h.prb_attention_decode_ring_prefers.argtypes = [I, I, I]
    h.prb_attention_decode_ring_prefers.restype = c_int
    h.prb_attention_decode_ring_max_list.argtypes = []
    h.prb_attention_decode_ring_max_list.restype = c_int
    h.prb_attention_decode_ring_workspace.argtypes = [I, I, I]
    h.prb_attention_decode_ring_workspace.restype = L
    h.prb_attention_prefill.argtypes = [P, L, P, L, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F,
                                        I, P, P]
    h.prb_attention_prefill_supports.argtypes = [I]
    h.prb_attention_prefill_tile.argtypes = []
    h.prb_attention_prefill_tc.argtypes = [P, L, P, L, I, P, P, P, P, P, P, P, P, I, I, I, I, I, I,
                                           I, F, I, I, I, P, P, P, P, P, P, P, P, I, P, P]
    h.prb_attention_prefill_tc_supports.argtypes = [I, I]
    h.prb_attention_prefill_tc_tile.argtypes = []
    h.prb_attention_decode_split.argtypes = []
    h.prb_attention_decode_max_split_pages.argtypes = []
    h.prb_attention_decode_max_split_pages.restype = c_int
    h.prb_device_sm_count.argtypes = []
    h.prb_device_sm_count.restype = c_int
    h.prb_attention_decode_set_stream.argtypes = [I]
    h.prb_attention_decode_set_stream.restype = None
    h.prb_set_pdl.argtypes = [I]
    h.prb_set_pdl.restype = None
    h.prb_sample.argtypes = [P, P, L, I, P, P, P, P, P, P, P, I, P, P, I, P, P]
    h.prb_sample_max_top_k.argtypes = []
    h.prb_sample_workspace_words.argtypes = []
    h.prb_sample_workspace_words.restype = c_int
    h.prb_embed_pair.argtypes = [P, P, P, P, P, P, P, P, P, I, I, I, L, L, L, I, I, I, F, P, P]
    h.prb_rms_norm.argtypes = [P, P, P, P, P, L, P, P, P, P, I, I, I, F, F, I, I, P, P]
    h.prb_gate_mul.argtypes = [P, L, P, L, P, L, I, I, I, P]
    h.prb_gate_mul.restype = c_int
    h.prb_gated_pair.argtypes = [P, L, I, P, L, I, I, I, I, F, F, F, P, L, I, I, P]
    h.prb_route.argtypes = [P, P, P, P, L, P, P, I, I, I, I, I, P]
    h.prb_latent_prepare.argtypes = [P, L, P, P, L, I, I, P, P, P, P, P, I, I, I, I, I, I, I, F,
                                     I, I, F, P, P, P]
    h.prb_latent_fold.argtypes = [P, P, L, P, P, P, P, I, I, I, I, I, I, I, I, P]
    h.prb_latent_attention_mma.argtypes = [P, P, P, L, P, P, P, P, P, P, P, P, I, P, P, P, I, I, I,
                                           I, I, I, F, I, I, I, I, I, P, I, P, P]
    h.prb_latent_mma_supports.argtypes = [I, I, I]
    h.prb_latent_mma_single_kw.argtypes = [I]
    h.prb_latent_mma_rows.argtypes = []
    h.prb_latent_attention.argtypes = [P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, I, P, P]
    h.prb_latent_unfold.argtypes = [P, L, P, P, P, L, I, I, I, I, I, I, I, P]
    h.prb_embed_scaled.argtypes = [P, P, P, P, I, I, I, F, I, P, P]
    h.prb_route_scores.argtypes = [P, P, P, P, L, P, I, I, I, I, I, I, F, I, I, P]
    h.prb_routed_act.argtypes = [P, L, P, L, I, I, I, P, L, I, I, I, I, P]
    h.prb_retention_lanes.argtypes = [I]
    h.prb_retention_scan.argtypes = [P, P, L, I, I, I, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I,
                                     P, P, I, P, P]
    h.prb_retention_segment.argtypes = []
    h.prb_retention_segment.restype = c_int
    h.prb_retention_max_segments.argtypes = [I, I]
    h.prb_retention_max_segments.restype = c_int
    h.prb_retention_finish.argtypes = [P, L, P, P, L, I, P, I, I, I, F, I, P]
    h.prb_diff_prepare.argtypes = [P, P, P, L, I, I, I, P, P, P, I, I, I, I, I, I, I, I, I, P, P]
    h.prb_diff_attention.argtypes = [P, L, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, F, F, F, I,
                                     I, P, P]
    h.prb_diff_attention_tile_rows.argtypes = [I, I, I, I]
    h.prb_diff_attention_tile_rows.restype = c_int
    h.prb_diff_attention_tile.argtypes = [P, L, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, F,
                                          F, F, I, I, P, P]
    h.prb_diff_attention_tile.restype = c_int
    h.prb_diff_attention_single_warps.argtypes = [I, I, I, I]
    h.prb_diff_attention_single_warps.restype = c_int
    h.prb_diff_attention_single.argtypes = [P, L, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, F, F,
                                            F, I, I, P, P]
    h.prb_diff_attention_single.restype = c_int
    h.prb_route_act.argtypes = [P, L, P, L, I, I, I, I, I, I, I, I, I, I, P, I, P]
    h.prb_route_act.restype = c_int
    h.prb_retention_step_supports.argtypes = [I, I]
    h.prb_retention_step_supports.restype = c_int
    h.prb_retention_step.argtypes = [P, L, P, L, I, I, I, I, P, P, P, P, P, P, I, I, I, I, I, I, I,
                                     F, F, I, P, P]
    h.prb_retention_step.restype = c_int
    h.prb_tmix_lanes.argtypes = [I]
    h.prb_tmix_shift.argtypes = [P, L, P, L, P, P, P, P, P, P, I, I, I, I, I, P, P]
    h.prb_tmix_scan.argtypes = [P, L, P, L, I, I, I, I, P, P, P, P, P, L, P, P, P, P, I, I, I, I,
                                I, I, I, I, P, P, L, I, P, F, F, P]
    h.prb_tmix_step_supports.argtypes = [I, I]
    h.prb_tmix_segment.argtypes = []
    h.prb_tmix_max_segments.argtypes = [I, I]
    h.prb_tmix_scan_segments.argtypes = [P, L, P, L, I, I, I, I, P, L, P, P, P, P, P, L, P, P, P, P,
                                         I, I, I, I, I, I, I, I, I, P, P, P, I, P, P]
    h.prb_tmix_finish.argtypes = [P, L, P, L, P, L, I, P, P, I, I, I, F, F, I, P]
    h.prb_wattn_prepare.argtypes = [P, P, P, L, I, I, I, P, P, P, P, P, I, I, I, I, I, I, F, F, I,
                                    I, I, I, I, P, P, P, P, P, P]
    h.prb_wattn.argtypes = [P, L, P, P, P, P, P, P, L, P, I, I, I, I, I, I, I, I, I, I, F, F, I, I,
                            P, I, P, P]
    h.prb_wattn_tile_rows.argtypes = [I, I, I, I]
    h.prb_wattn_single_supports.argtypes = [I, I, I, I]
    h.prb_wattn_single.argtypes = list(h.prb_wattn.argtypes)
    h.prb_wattn_tile.argtypes = [P, L, P, P, P, P, P, P, L, P, I, I, I, I, I, I, I, I, I, I, I, F,
                                 F, I, I, P, I, P, P]
    h.prb_lru_max_taps.argtypes = []
    h.prb_lru_conv.argtypes = [P, P, L, I, P, P, P, P, P, P, P, P, I, I, I, I, I, P]
    h.prb_lru_gates.argtypes = [P, P, P, P, P, P, P, I, I, I, I, P]
    h.prb_lru_scan.argtypes = [P, L, P, P, P, L, I, I, P, P, P, P, P, P, P, I, I, I, I, I, F, I, P]
    h.prb_mmem_supports.argtypes = [I, I]
    h.prb_mmem_step.argtypes = [P, L, P, L, I, I, I, I, I, I, P, P, P, P, P, P, P, P, P, I, I, I,
                                I, I, I, F, F, F, F, I, P]
    h.prb_lru_segment.argtypes = []
    h.prb_lru_max_segments.argtypes = [I, I]
    h.prb_lru_scan_segments.argtypes = [P, L, P, P, P, P, I, P, L, I, I, P, P, P, P, P, P, P, I, I,
                                        I, I, I, F, I, P]
    h.prb_lru_step_supports.argtypes = [I]
    h.prb_lru_step.argtypes = [P, L, P, L, I, I, P, P, P, P, P, P, P, P, P, P, P, P, P, P, I, I, I,
                               I, I, I, F, I, I, P]
    for name in ("prb_lru_segment", "prb_lru_max_segments", "prb_lru_scan_segments",
                 "prb_lru_step_supports", "prb_lru_step"):
        getattr(h, name).restype = c_int
    h.prb_mmem_segment.argtypes = []
    h.prb_mmem_max_segments.argtypes = [I, I]
    h.prb_mmem_scan_supports.argtypes = [I]
    h.prb_mmem_scan.argtypes = [P, L, P, P, P, L, I, I, I, I, I, I, P, P, P, P, P, P, P, P, P, P,
                                I, I, I, I, I, I, F, F, F, F, I, P, P, P, P, P, I, I, P]
    for name in ("prb_lru_max_taps", "prb_lru_conv", "prb_lru_gates", "prb_lru_scan",
                 "prb_mmem_supports", "prb_mmem_step", "prb_mmem_segment",
                 "prb_mmem_max_segments", "prb_mmem_scan_supports", "prb_mmem_scan"):
        getattr(h, name).restype = c_int
    for name in ("prb_tmix_lanes", "prb_tmix_shift", "prb_tmix_scan", "prb_tmix_finish",
                 "prb_tmix_step_supports", "prb_tmix_segment", "prb_tmix_max_segments",
                 "prb_tmix_scan_segments",
                 "prb_wattn_prepare", "prb_wattn", "prb_wattn_tile_rows", "prb_wattn_tile",
                 "prb_wattn_single_supports", "prb_wattn_single"):
        getattr(h, name).restype = c_int
    for name in ("prb_embed_scaled", "prb_route_scores", "prb_routed_act", "prb_retention_lanes",
                 "prb_retention_scan", "prb_retention_finish", "prb_diff_prepare",
                 "prb_diff_attention"):
        getattr(h, name).restype = c_int
    for name in ("prb_embed_pair", "prb_rms_norm", "prb_gated_pair", "prb_route",
                 "prb_latent_prepare", "prb_latent_fold", "prb_latent_attention",
                 "prb_latent_unfold", "prb_latent_attention_mma", "prb_latent_mma_supports",
                 "prb_latent_mma_single_kw", "prb_latent_mma_rows"):
        getattr(h, name).restype = c_int
    for name in ("prb_resolve_tokens", "prb_fetch_step", "prb_publish_result", "prb_embed", "prb_layernorm", "prb_bias_act", "prb_kv_append", "prb_copy_pages",
                 "prb_gemm_f32", "prb_gemm_bf16", "prb_gemm_bf16_scatter", "prb_gemm_midm",
                 "prb_gemm_midm_supports", "prb_gemm_smallm", "prb_gemm_smallm_max_rows",
                 "prb_gemm_smallm_max_norm_width", "prb_attention_generic", "prb_attention_decode",
                 "prb_attention_prefill", "prb_attention_prefill_supports",
                 "prb_attention_prefill_tile", "prb_attention_prefill_tc",
                 "prb_attention_prefill_tc_supports", "prb_attention_prefill_tc_tile",
                 "prb_attention_decode_split", "prb_sample", "prb_sample_max_top_k"):
        getattr(h, name).restype = c_int


# ------------------------------------------------------------------------- helpers
def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelArgumentError(f"element type {dtype} is not supported (float32 or bfloat16)")


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


_LAUNCHES = 0


def launch_count() -> int:
    """Kernels of this library launched so far through these wrappers."""
    return _LAUNCHES


def add_launches(n: int) -> None:
    """Account for kernels launched by replaying a CUDA graph that holds ``n`` of them."""
    global _LAUNCHES
    _LAUNCHES += int(n)


def _check(code: int, what: str) -> None:
    global _LAUNCHES
    if code == 0:
        _LAUNCHES += 1
        return
    if code < 0:
        raise KernelArgumentError(f"{what}: {_ERRORS.get(code, 'error')} (code {code})")
    raise ExtensionError(f"{what}: CUDA error {code} at launch")


def _need(t: torch.Tensor, dtype, name: str, what: str) -> None:
    if not t.is_cuda:
        raise KernelArgumentError(f"{what}: {name} is not on a CUDA device")
    if dtype is not None and t.dtype != dtype:
        raise KernelArgumentError(f"{what}: {name} must be {dtype}, is {t.dtype}")
    if not t.is_contiguous():
        raise KernelArgumentError(f"{what}: {name} must be contiguous")


_PDL = True


def set_pdl(on: bool) -> None:
    """Switch programmatic dependent launch of the decode-chain kernels on or off."""
    global _PDL
    _PDL = bool(on)
    lib().prb_set_pdl(1 if on else 0)


class plain_launch:
    """``with plain_launch(cond):`` kernels launched inside start only when their predecessor
    has ended (no programmatic dependent launch), if ``cond``; the setting outside is kept."""

    def __init__(self, cond: bool = True):
        self.cond = bool(cond) and _PDL

    def __enter__(self):
        if self.cond:
            lib().prb_set_pdl(0)
        return self

    def __exit__(self, *exc):
        if self.cond:
            lib().prb_set_pdl(1)
        return False


# ------------------------------------------------------------------------ kernels
def embed(out, tokens, positions, wte, wpe, status) -> None:
    """out[t,:] = wte[tokens[t],:] (+ wpe[positions[t],:]); out float32 [T, width]."""
    what = "embed"
    _need(out, torch.float32, "out", what)
    _need(tokens, torch.int32, "tokens", what)
    _need(positions, torch.int32, "positions", what)
    _need(wte, None, "wte", what)
    n, width = out.shape
    if wte.shape[1] != width or (wpe is not None and (wpe.shape[1] != width or wpe.dtype != wte.dtype)):
        raise KernelArgumentError(f"{what}: table widths or types differ from the output's")
    if tokens.numel() < n or positions.numel() < n:
        raise KernelArgumentError(f"{what}: fewer token ids or positions than output rows")
    _check(lib().prb_embed(_p(out), _p(tokens), _p(positions), _p(wte), _p(wpe), n, width,
                           wte.shape[0], 0 if wpe is None else wpe.shape[0],
                           dtype_code(wte.dtype), _p(status), _stream()), what)


def layernorm(out, x, gamma, beta, eps: float, rows=None, status=None) -> None:
    """out[r,:] = LayerNorm(x[rows[r],:] or x[r,:]); x float32, out float32 or bfloat16."""
    what = "layernorm"
    _need(x, torch.float32, "x", what)
    _need(out, None, "out", what)
    _need(gamma, torch.float32, "gamma", what)
    if beta is not None:
        _need(beta, torch.float32, "beta", what)
    n_rows, width = out.shape
    if x.shape[1] != width or gamma.numel() != width:
        raise KernelArgumentError(f"{what}: widths differ")
    if rows is None and x.shape[0] < n_rows:
        raise KernelArgumentError(f"{what}: fewer input rows than output rows")
    if rows is not None:
        _need(rows, torch.int32, "rows", what)
    _check(lib().prb_layernorm(_p(out), _p(x), _p(gamma), _p(beta), _p(rows), n_rows, x.shape[0],
                               width, float(eps), dtype_code(out.dtype), _p(status), _stream()),
           what)


def bias_act(out, inp, bias, resid, act) -> None:
    """out = act(inp + bias) (+ resid), sums in float32."""
    what = "bias_act"
    _need(out, None, "out", what)
    _need(inp, None, "inp", what)
    m, n = inp.shape
    if out.shape != inp.shape:
        raise KernelArgumentError(f"{what}: shapes differ")
    if bias is not None:
        _need(bias, torch.float32, "bias", what)
    if resid is not None:
        _need(resid, torch.float32, "resid", what)
    _check(lib().prb_bias_act(_p(out), _p(inp), _p(bias), _p(resid), m, n, ACT_CODES[act],
                              dtype_code(inp.dtype), dtype_code(out.dtype), _stream()), what)


def kv_append(k_pages, v_pages, k_src, v_src, slots, n_tokens, status) -> None:
    """Write the step's keys and values to their cache slots.  k_pages/v_pages:
    [pages, kv_heads, page_size, head_dim]; k_src/v_src: [T, kv_heads*head_dim] views that
    may be column slices of one wider row-major tensor."""
    what = "kv_append"
    num_pages, kv_heads, page_size, head_dim = k_pages.shape
    _need(k_pages, None, "k_pages", what)
    _need(v_pages, k_pages.dtype, "v_pages", what)
    _need(slots, torch.int32, "slots", what)
    for name, s in (("k_src", k_src), ("v_src", v_src)):
        if s.dtype != k_pages.dtype or s.stride(1) != 1 or s.shape[1] != kv_heads * head_dim:
            raise KernelArgumentError(f"{what}: {name} has the wrong type, width or inner stride")
    if k_src.stride(0) != v_src.stride(0):
        raise KernelArgumentError(f"{what}: k_src and v_src row strides differ")
    _check(lib().prb_kv_append(_p(k_pages), _p(v_pages), _p(k_src), _p(v_src), k_src.stride(0),
                               _p(slots), n_tokens, kv_heads, head_dim, page_size, num_pages,
                               dtype_code(k_pages.dtype), _p(status), _stream()), what)


def copy_pages(storage, pairs, n_pairs, status) -> None:
    """storage: [pools, pages, ...] contiguous; pairs int32 [n, 2] (source, destination)."""
    what = "copy_pages"
    _need(storage, None, "storage", what)
    _need(pairs, torch.int32, "pairs", what)
    pools, pages = storage.shape[0], storage.shape[1]
    page_bytes = storage[0, 0].numel() * storage.element_size()
    _check(lib().prb_copy_pages(_p(storage), _p(pairs), n_pairs, page_bytes, pools, pages,
                                _p(status), _stream()), what)


def gemm_f32(out, a, w, bias=None, resid=None, act=None) -> None:
    """out[M,N] = act(a[M,K] . w[N,K]^T + bias) (+ resid): true 32-bit FMA."""
    what = "gemm_f32"
    for name, t in (("out", out), ("a", a), ("w", w)):
        if not t.is_cuda or t.dtype != torch.float32 or t.stride(1) != 1:
            raise KernelArgumentError(f"{what}: {name} must be float32 on CUDA with unit inner stride")
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape[0] != m or out.shape[1] != n:
        raise KernelArgumentError(f"{what}: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    if bias is not None:
        _need(bias, torch.float32, "bias", what)
    if resid is not None:
        _need(resid, torch.float32, "resid", what)
        if resid.shape != out.shape or resid.stride(0) != out.stride(0):
            raise KernelArgumentError(f"{what}: resid must have the output's shape and stride")
    _check(lib().prb_gemm_f32(_p(out), _p(a), _p(w), _p(bias), _p(resid), m, n, k, a.stride(0),
                              w.stride(0), out.stride(0), ACT_CODES[act], _stream()), what)


def gemm_bf16(out, a, w, bias=None, resid=None, act=None, tile_n: int = 0, status=None,
              kv_scatter=None, split_k: int = 0, pair: bool = False) -> None:
    """out[M,N] = act(a[M,K] . w[N,K]^T + bias) (+ resid) on the tcgen05 tensor cores:
    bfloat16 operands, float32 accumulation in tensor memory, epilogue in float32; out is
    bfloat16 or float32.  K and the row pitches of a and w must be multiples of 8.
    ``kv_scatter`` = (k_pages, v_pages, slots, q_width[, only_cache]): the key and value
    columns of a fused QKV product also go to the paged cache (of the output's element type);
    with ``only_cache`` they need not reach ``out`` at all.  ``tile_n`` and
    ``split_k`` force a tile width and, for widths 64 and 128, a cluster of 2, 4 or 8 CTAs
    that share a tile's reduction; ``pair`` (widths 64, 128, 192, 256) forces pairs of CTAs on
    256-row tiles (``tcgen05.mma.cta_group::2``); left at 0 the kernel chooses."""
    what = "gemm_bf16"
    for name, t in (("a", a), ("w", w)):
        if not t.is_cuda or t.dtype != torch.bfloat16 or t.stride(1) != 1:
            raise KernelArgumentError(f"{what}: {name} must be bfloat16 on CUDA with unit inner stride")
    if not out.is_cuda or out.stride(1) != 1:
        raise KernelArgumentError(f"{what}: out must be on CUDA with unit inner stride")
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape[0] != m or out.shape[1] != n:
        raise KernelArgumentError(f"{what}: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    if bias is not None:
        _need(bias, torch.float32, "bias", what)
    if resid is not None:
        _need(resid, torch.float32, "resid", what)
        if resid.shape != out.shape or resid.stride(0) != out.stride(0):
            raise KernelArgumentError(f"{what}: resid must have the output's shape and stride")
    if kv_scatter is not None:
        k_pages, v_pages, slots, q_width = kv_scatter[:4]
        only_cache = bool(kv_scatter[4]) if len(kv_scatter) > 4 else False
        if resid is not None or tile_n or split_k or pair:
            raise KernelArgumentError(f"{what}: a product that scatters takes no residual or tile width")
        if k_pages.dtype != out.dtype or v_pages.dtype != out.dtype or not k_pages.is_contiguous() \
                or not v_pages.is_contiguous():
            raise KernelArgumentError(f"{what}: the cache must be contiguous and of the output's type")
        _need(slots, torch.int32, "slots", what)
        num_pages, kv_heads, page_size, head_dim = k_pages.shape
        _check(lib().prb_gemm_bf16_scatter(
            _p(out), _p(a), _p(w), _p(bias), m, n, k, a.stride(0), w.stride(0), out.stride(0),
            ACT_CODES[act], dtype_code(out.dtype), _p(k_pages), _p(v_pages), _p(slots), int(q_width),
            kv_heads * head_dim, head_dim, page_size, num_pages, int(only_cache), _p(status),
            _stream()), what)
        return
    _check(lib().prb_gemm_bf16(_p(out), _p(a), _p(w), _p(bias), _p(resid), m, n, k, a.stride(0),
                               w.stride(0), out.stride(0), ACT_CODES[act], dtype_code(out.dtype),
                               int(tile_n) | (int(split_k) << 16) | (int(bool(pair)) << 24),
                               _p(status), _stream()), what)


def midm_supports(m: int, n: int, k: int) -> bool:
    return bool(lib().prb_gemm_midm_supports(int(m), int(n), int(k)))


def gemm_midm(out, a, w, bias=None, resid=None, act=None, status=None) -> None:
    """out[M,N] = act(a[M,K] . w[N,K]^T + bias) (+ resid) for up to 64 rows, K a multiple of
    64: the reduction is split over a thread-block cluster (``csrc/gemm_bf16_midm.cu``)."""
    what = "gemm_midm"
    for name, t in (("a", a), ("w", w)):
        if not t.is_cuda or t.dtype != torch.bfloat16 or t.stride(1) != 1:
            raise KernelArgumentError(f"{what}: {name} must be bfloat16 on CUDA with unit inner stride")
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape[0] != m or out.shape[1] != n or out.stride(1) != 1:
        raise KernelArgumentError(f"{what}: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    if bias is not None:
        _need(bias, torch.float32, "bias", what)
    if resid is not None:
        _need(resid, torch.float32, "resid", what)
        if resid.shape != out.shape or resid.stride(0) != out.stride(0):
            raise KernelArgumentError(f"{what}: resid must have the output's shape and stride")
    _check(lib().prb_gemm_midm(_p(out), _p(a), _p(w), _p(bias), _p(resid), m, n, k, a.stride(0),
                               w.stride(0), out.stride(0), ACT_CODES[act], dtype_code(out.dtype),
                               _p(status), _stream()), what)


_SMALLM = None


def smallm_limits():
    """(most rows, widest fused norm) of the decode-time product kernel."""
    global _SMALLM
    if _SMALLM is None:
        _SMALLM = (lib().prb_gemm_smallm_max_rows(), lib().prb_gemm_smallm_max_norm_width())
    return _SMALLM


def gemm_smallm(out, w, a=None, norm_input=None, gamma=None, beta=None, eps=0.0, bias=None,
                resid=None, act=None, kv_scatter=None, status=None, norm_rows=None,
                centred: bool = True) -> None:
    """out[M,N] = act(X . w[N,K]^T + bias) (+ resid) for M <= 64 rows, weights streamed once.
    X is ``a`` (bfloat16 [M,K]) or LayerNorm(``norm_input``) (float32 [M,K]) with ``gamma``,
    ``beta`` and ``eps`` (``centred`` False: the mean is not taken off, i.e. x / sqrt(mean(x^2)
    + eps) * gamma, a root-mean-square norm), the norm fused into the kernel; with ``norm_rows`` (int32 [M]) row t
    of X is the norm of row norm_rows[t] of ``norm_input`` (an index outside it gives a zero
    row and is recorded in ``status``).  ``kv_scatter`` = (k_pages, v_pages,
    slots, q_width): the product is a fused QKV projection; its key and value columns are also
    written to the paged cache (same element type as ``out``) at each token's slot."""
    what = "gemm_smallm"
    if not w.is_cuda or w.dtype != torch.bfloat16 or w.stride(1) != 1:
        raise KernelArgumentError(f"{what}: w must be bfloat16 on CUDA with unit inner stride")
    n, k = w.shape
    if norm_input is not None:
        x = norm_input
        if x.dtype != torch.float32 or x.stride(1) != 1:
            raise KernelArgumentError(f"{what}: norm_input must be float32 with unit inner stride")
        _need(gamma, torch.float32, "gamma", what)
        if beta is not None:
            _need(beta, torch.float32, "beta", what)
    else:
        x = a
        if x is None or x.dtype != torch.bfloat16 or x.stride(1) != 1:
            raise KernelArgumentError(f"{what}: a must be bfloat16 with unit inner stride")
    m = out.shape[0]
    if norm_rows is not None:
        if norm_input is None:
            raise KernelArgumentError(f"{what}: norm_rows gathers rows of norm_input")
        _need(norm_rows, torch.int32, "norm_rows", what)
        if norm_rows.numel() < m:
            raise KernelArgumentError(f"{what}: {m} output rows, {norm_rows.numel()} row indices")
    if (norm_rows is None and x.shape[0] < m) or x.shape[1] != k or out.shape[1] != n or \
            out.stride(1) != 1:
        raise KernelArgumentError(f"{what}: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    if bias is not None:
        _need(bias, torch.float32, "bias", what)
    if resid is not None:
        if resid.dtype != torch.float32 or resid.shape != out.shape or resid.stride(0) != out.stride(0):
            raise KernelArgumentError(f"{what}: resid must be float32 with the output's shape and stride")
    kv = (None, None, None, 0, 0, 0, 0, 0)
    if kv_scatter is not None:
        k_pages, v_pages, slots, q_width = kv_scatter[:4]
        num_pages, kv_heads, page_size, head_dim = k_pages.shape
        if k_pages.dtype != out.dtype or v_pages.dtype != out.dtype or slots.dtype != torch.int32 \
                or q_width + 2 * kv_heads * head_dim != n:
            raise KernelArgumentError(f"{what}: cache type or widths do not fit the product")
        kv = (_p(k_pages), _p(v_pages), _p(slots), q_width, kv_heads * head_dim, head_dim,
              page_size, num_pages)
    _check(lib().prb_gemm_smallm(
        _p(out), None if norm_input is not None else _p(x),
        _p(x) if norm_input is not None else None, _p(norm_rows),
        x.shape[0] if norm_input is not None else 0, _p(gamma), _p(beta), float(eps), _p(w),
        _p(bias), _p(resid), m, n, k, x.stride(0), w.stride(0), out.stride(0), ACT_CODES[act],
        dtype_code(out.dtype), *kv, 0 if centred else 1, _p(status), _stream()), what)


def attention_generic(out, q, k_pages, v_pages, block_table, seq_of_token, positions, n_tokens,
                      n_heads, scale, window, max_context, status) -> None:
    """Attention of every token of the step over its request's cached keys; 32-bit
    arithmetic.  q: [T, n_heads*head_dim] (may be a column slice), out likewise."""
    what = "attention_generic"
    num_pages, kv_heads, page_size, head_dim = k_pages.shape
    for name, t in (("out", out), ("q", q)):
        if t.dtype != k_pages.dtype or t.stride(1) != 1 or t.shape[1] != n_heads * head_dim:
            raise KernelArgumentError(f"{what}: {name} has the wrong type, width or inner stride")
    _need(block_table, torch.int32, "block_table", what)
    _need(seq_of_token, torch.int32, "seq_of_token", what)
    _need(positions, torch.int32, "positions", what)
    _check(lib().prb_attention_generic(
        _p(out), out.stride(0), _p(q), q.stride(0), _p(k_pages), _p(v_pages), _p(block_table),
        _p(seq_of_token), _p(positions), n_tokens, n_heads, kv_heads, head_dim, page_size,
        block_table.shape[1], num_pages, max_context, float(scale), int(window or 0),
        dtype_code(k_pages.dtype), _p(status), _stream()), what)


_SM_COUNT = None


def sm_count() -> int:
    """Streaming multiprocessors of the current device."""
    global _SM_COUNT
    if _SM_COUNT is None:
        _SM_COUNT = max(1, int(lib().prb_device_sm_count()))
    return _SM_COUNT


def decode_max_split_pages() -> int:
    """Most pages one split of the decode attention kernel may span."""
    return lib().prb_attention_decode_max_split_pages()


def decode_split() -> int:
    """Keys per split of the decode attention kernel."""
    return lib().prb_attention_decode_split()


def decode_stream(mode: int) -> None:
    """Which key loop the decode attention kernel runs (for tests and measurements): -1 the
    kernel's own choice, 0 register batches always, 1 the shared-memory ring wherever it
    applies (no window, head size up to 128)."""
    lib().prb_attention_decode_set_stream(int(mode))


def prefill_supports(head_dim: int) -> bool:
    return bool(lib().prb_attention_prefill_supports(int(head_dim)))


def attention_decode(out, q, k_pages, v_pages, block_table, seq_of_token, positions, token_list,
                     token_count, n_list, n_heads, scale, window, workspace, counters, max_splits,
                     status, split_keys: Optional[int] = None) -> None:
    """bfloat16 attention of single tokens (those in ``token_list``, or all of the first
    ``n_list`` when it is None) over their requests' pages, keys split in ranges of
    ``split_keys`` positions (a multiple of ``decode_split()``, the default).  ``workspace`` float32 [n_list, heads, max_splits,
    head_dim + 4] and ``counters`` int32 [n_list * heads] (zero) are scratch."""
    what = "attention_decode"
    num_pages, kv_heads, page_size, head_dim = k_pages.shape
    for name, t in (("out", out), ("q", q)):
        if t.dtype != torch.bfloat16 or t.stride(1) != 1 or t.shape[1] != n_heads * head_dim:
            raise KernelArgumentError(f"{what}: {name} has the wrong type, width or inner stride")
    if k_pages.dtype != torch.bfloat16:
        raise KernelArgumentError(f"{what}: the cache must be bfloat16")
    split_keys = decode_split() if split_keys is None else int(split_keys)
    need = n_list * n_heads * max_splits * (head_dim + 4)
    if workspace.dtype != torch.float32 or workspace.numel() < need or \
            counters.dtype != torch.int32 or counters.numel() < n_list * n_heads:
        raise KernelArgumentError(f"{what}: scratch too small or of the wrong type")
    _check(lib().prb_attention_decode(
        _p(out), out.stride(0), _p(q), q.stride(0), _p(k_pages), _p(v_pages), _p(block_table),
        _p(seq_of_token), _p(positions), _p(token_list), _p(token_count), n_list, n_heads,
        kv_heads, head_dim, page_size, block_table.shape[1], num_pages, float(scale),
        int(window or 0), _p(workspace), _p(counters), max_splits, split_keys, _p(status),
        _stream()), what)


def decode_ring_supports(head_dim: int, page_size: int) -> bool:
    return bool(lib().prb_attention_decode_ring_supports(int(head_dim), int(page_size)))


def decode_ring_prefers(n_list: int, n_heads: int, max_context: int) -> bool:
    """Whether ``attention_decode_ring`` is the faster kernel for this launch (both are right)."""
    return bool(lib().prb_attention_decode_ring_prefers(int(n_list), int(n_heads), int(max_context)))


def decode_ring_max_list() -> int:
    """Most single tokens a launch of ``attention_decode_ring`` takes."""
    return int(lib().prb_attention_decode_ring_max_list())


def decode_ring_workspace(n_list: int, n_heads: int, head_dim: int) -> int:
    """float32 elements of workspace ``attention_decode_ring`` needs for up to ``n_list`` tokens."""
    return int(lib().prb_attention_decode_ring_workspace(int(n_list), int(n_heads), int(head_dim)))


def attention_decode_ring(out, q, k_pages, v_pages, block_table, seq_of_token, positions,
                          token_list, token_count, n_list, n_heads, scale, window, workspace,
                          counters, status, new_keys: int = 1, stages: int = 0,
                          max_context: int = 0, kv_new=None) -> None:
    """bfloat16 attention of single tokens over their requests' pages by persistent CTAs whose
    warps stream keys and values through rings of shared-memory buffers; what was cached before
    the step is requested before the kernel this one depends on has finished (head size 64).
    ``new_keys``: how many of a token's last visible positions the step itself may have
    written (at most 4).  ``kv_new`` = (k, v): the step's own keys and values, row t for token t
    ([T, kv_heads * head_dim], may be column slices of a wider tensor), as the product before
    this kernel left them; with them no part of the kernel waits for the cache rows the step
    appended.  ``workspace``: ``decode_ring_workspace`` floats; ``counters`` int32
    [n_list * heads], zero (left zero)."""
    what = "attention_decode_ring"
    num_pages, kv_heads, page_size, head_dim = k_pages.shape
    for name, t in (("out", out), ("q", q)):
        if t.dtype != torch.bfloat16 or t.stride(1) != 1 or t.shape[1] != n_heads * head_dim:
            raise KernelArgumentError(f"{what}: {name} has the wrong type, width or inner stride")
    if k_pages.dtype != torch.bfloat16 or not k_pages.is_contiguous() or not v_pages.is_contiguous():
        raise KernelArgumentError(f"{what}: the cache must be contiguous bfloat16")
    if workspace.dtype != torch.float32 or \
            workspace.numel() < decode_ring_workspace(n_list, n_heads, head_dim) or \
            counters.dtype != torch.int32 or counters.numel() < n_list * n_heads:
        raise KernelArgumentError(f"{what}: scratch too small or of the wrong type")
    k_new = v_new = None
    kv_stride = 0
    if kv_new is not None:
        k_new, v_new = kv_new
        for name, t in (("k_new", k_new), ("v_new", v_new)):
            if t.dtype != torch.bfloat16 or t.stride(1) != 1 or t.shape[1] != kv_heads * head_dim:
                raise KernelArgumentError(f"{what}: {name} has the wrong type, width or inner stride")
        if k_new.stride(0) != v_new.stride(0):
            raise KernelArgumentError(f"{what}: k_new and v_new row strides differ")
        kv_stride = k_new.stride(0)
    _check(lib().prb_attention_decode_ring(
        _p(out), out.stride(0), _p(q), q.stride(0), _p(k_pages), _p(v_pages), _p(block_table),
        _p(seq_of_token), _p(positions), _p(token_list), _p(token_count), n_list, n_heads,
        kv_heads, head_dim, page_size, block_table.shape[1], num_pages, float(scale),
        int(window or 0), int(new_keys), _p(k_new), _p(v_new), int(kv_stride), _p(workspace),
        _p(counters), int(stages), int(max_context), _p(status), _stream()), what)


def prefill_tile() -> int:
    """Rows per item of the work list the prompt attention kernels take."""
    return lib().prb_attention_prefill_tile()


def prefill_tc_supports(head_dim: int, page_size: int) -> bool:
    return bool(lib().prb_attention_prefill_tc_supports(int(head_dim), int(page_size)))


PREFILL_MAX_PARTS = 16


def attention_prefill_tc(out, q, k_pages, v_pages, block_table, positions, tile_req, tile_row0,
                         tile_rows, tile_count, n_tiles, n_heads, scale, window, status,
                         part_blocks: int = 0, max_parts: int = 1, parts=None, items=None) -> None:
    """bfloat16 causal attention of prompt portions on tcgen05 (head size 64, pages of a
    multiple of 64 positions): one CTA per work item of up to 128 queries and head, or, with
    ``part_blocks`` > 0, one per chunk of ``part_blocks`` * 64 keys of the item (at most
    ``max_parts`` chunks; ``parts`` = (float32 [n_tiles * n_heads * max_parts * 8192],
    float32 [n_tiles * n_heads * max_parts * 256], zeroed int32 [n_tiles * n_heads]) is the
    workspace through which the chunks of an item are merged).

    ``items`` = (item_tile, item_part, item_slot, item_count or None, part_blocks (device
    int32 [1]), n_items, n_slots): the CTAs' work as a list instead (item i is tile
    ``item_tile[i]`` as a whole when ``item_part[i]`` < 0, else that chunk of it, whose
    partial result goes to workspace slot ``item_slot[i]``; a tile's chunks have consecutive
    slots); ``parts`` then holds ``n_slots * n_heads`` slots and counters."""
    what = "attention_prefill_tc"
    num_pages, kv_heads, page_size, head_dim = k_pages.shape
    for name, t in (("out", out), ("q", q)):
        if t.dtype != torch.bfloat16 or t.stride(1) != 1 or t.shape[1] != n_heads * head_dim:
            raise KernelArgumentError(f"{what}: {name} has the wrong type, width or inner stride")
    if k_pages.dtype != torch.bfloat16 or not k_pages.is_contiguous() or not v_pages.is_contiguous():
        raise KernelArgumentError(f"{what}: the cache must be contiguous bfloat16")
    part_o = part_ml = part_count = None
    item_tile = item_part = item_slot = item_count = part_dev = None
    n_items = 0
    if items is not None:
        item_tile, item_part, item_slot, item_count, part_dev, n_items, n_slots = items
        if part_blocks or parts is None:
            raise KernelArgumentError(f"{what}: a work list brings its own chunk size and needs a workspace")
        for name, t in (("item_tile", item_tile), ("item_part", item_part), ("item_slot", item_slot),
                        ("part_blocks", part_dev)):
            _need(t, torch.int32, name, what)
        if min(item_tile.numel(), item_part.numel(), item_slot.numel()) < n_items:
            raise KernelArgumentError(f"{what}: the work list is shorter than {n_items} items")
        part_o, part_ml, part_count = parts
        _need(part_o, torch.float32, "parts[0]", what)
        _need(part_ml, torch.float32, "parts[1]", what)
        _need(part_count, torch.int32, "parts[2]", what)
        units = int(n_slots) * n_heads
        if part_o.numel() < units * 8192 or part_ml.numel() < units * 256 or part_count.numel() < units:
            raise KernelArgumentError(f"{what}: the workspace of the key parts is too small")
    if part_blocks:
        if parts is None or not 1 <= max_parts <= PREFILL_MAX_PARTS:
            raise KernelArgumentError(f"{what}: key parts need a workspace and 1 to "
                                      f"{PREFILL_MAX_PARTS} parts per item")
        part_o, part_ml, part_count = parts
        units = n_tiles * n_heads
        _need(part_o, torch.float32, "parts[0]", what)
        _need(part_ml, torch.float32, "parts[1]", what)
        _need(part_count, torch.int32, "parts[2]", what)
        if part_o.numel() < units * max_parts * 8192 or part_ml.numel() < units * max_parts * 256 \
                or part_count.numel() < units:
            raise KernelArgumentError(f"{what}: the workspace of the key parts is too small")
    _check(lib().prb_attention_prefill_tc(
        _p(out), out.stride(0), _p(q), q.stride(0), q.shape[0], _p(k_pages), _p(v_pages),
        _p(block_table), _p(positions), _p(tile_req), _p(tile_row0), _p(tile_rows), _p(tile_count),
        n_tiles, n_heads, kv_heads, head_dim, page_size, block_table.shape[1], num_pages,
        float(scale), int(window or 0), int(part_blocks), int(max_parts), _p(part_o), _p(part_ml),
        _p(part_count), _p(item_tile), _p(item_part), _p(item_slot), _p(item_count), _p(part_dev),
        int(n_items), _p(status), _stream()), what)


def attention_prefill(out, q, k_pages, v_pages, block_table, positions, tile_req, tile_row0,
                      tile_rows, tile_count, n_tiles, n_heads, scale, window, status) -> None:
    """bfloat16 causal attention of prompt portions (work items of up to 128 queries, two
    CTAs of 64 each) on mma.sync tensor-core instructions; any head size in steps of 16."""
    what = "attention_prefill"
    num_pages, kv_heads, page_size, head_dim = k_pages.shape
    for name, t in (("out", out), ("q", q)):
        if t.dtype != torch.bfloat16 or t.stride(1) != 1 or t.shape[1] != n_heads * head_dim:
            raise KernelArgumentError(f"{what}: {name} has the wrong type, width or inner stride")
    if k_pages.dtype != torch.bfloat16:
        raise KernelArgumentError(f"{what}: the cache must be bfloat16")
    _check(lib().prb_attention_prefill(
        _p(out), out.stride(0), _p(q), q.stride(0), _p(k_pages), _p(v_pages), _p(block_table),
        _p(positions), _p(tile_req), _p(tile_row0), _p(tile_rows), _p(tile_count), n_tiles,
        n_heads, kv_heads, head_dim, page_size, block_table.shape[1], num_pages, float(scale),
        int(window or 0), _p(status), _stream()), what)


def resolve_tokens(tokens, n, prev, status) -> None:
    """tokens[t] = prev[-tokens[t] - 1] wherever tokens[t] < 0 (t < n): ids that name a place
    among the tokens the sampling kernel chose last."""
    what = "resolve_tokens"
    _need(tokens, torch.int32, "tokens", what)
    _need(prev, torch.int32, "prev", what)
    _check(lib().prb_resolve_tokens(_p(tokens), int(n), _p(prev), prev.numel(), _p(status),
                                    _stream()), what)


def host_device_address(host: torch.Tensor) -> int:
    """The address under which kernels reach this pinned host tensor, or 0 if they cannot
    (the caller then copies with the copy engine)."""
    if host.is_cuda or not host.is_pinned():
        return 0
    return int(lib().prb_host_device_address(host.data_ptr()) or 0)


def fetch_step(dev, host_address: int, words: int, tokens_at: int = 0, n_tokens: int = 0,
               prev=None, status=None) -> None:
    """dev[:words] = the int32 words at ``host_address`` (from :func:`host_device_address`),
    read by a kernel; with ``prev``, token ids below zero among words
    [tokens_at, tokens_at + n_tokens) become prev[-id - 1] on the way."""
    what = "fetch_step"
    _need(dev, torch.int32, "dev", what)
    if not host_address or words > dev.numel():
        raise KernelArgumentError(f"{what}: no host address, or {words} words do not fit")
    if prev is not None:
        _need(prev, torch.int32, "prev", what)
    _check(lib().prb_fetch_step(_p(dev), host_address, int(words), int(tokens_at), int(n_tokens),
                                _p(prev), 0 if prev is None else prev.numel(), _p(status),
                                _stream()), what)


def publish_result(host_address: int, dev, words: int) -> None:
    """The int32 words dev[:words] written to pinned host memory at ``host_address`` by a
    kernel; the host sees them once an event recorded after this call has completed."""
    what = "publish_result"
    _need(dev, torch.int32, "dev", what)
    if not host_address or words > dev.numel():
        raise KernelArgumentError(f"{what}: no host address, or {words} words do not fit")
    _check(lib().prb_publish_result(host_address, _p(dev), int(words), _stream()), what)


def max_top_k() -> int:
    return lib().prb_sample_max_top_k()


def sample_workspace_words() -> int:
    return lib().prb_sample_workspace_words()


def sample(out, logits, n_rows, temperature=None, top_k=None, top_p=None, seeds=None, fresh=None,
           slots=None, rng_states=None, publish=None, workspace=None) -> None:
    """out[r] = chosen token of logits[r,:] (float32).  Without ``temperature`` every row
    is greedy; otherwise rows with temperature <= 0 are greedy and the rest sample.
    ``workspace``: :func:`sample_workspace_words` int32 words on the device, zero at first and
    then left to the kernels (one per stream of calls); with it a launch of up to 64 greedy
    rows gives every row to several CTAs.  ``publish`` = (host_address, src, words), with a
    workspace: the launch's last CTA also writes the int32 words src[:words] to pinned host
    memory at ``host_address`` (from :func:`host_device_address`)."""
    what = "sample"
    if workspace is not None:
        _need(workspace, torch.int32, "workspace", what)
        if workspace.numel() < sample_workspace_words() or not workspace.is_contiguous():
            raise KernelArgumentError(f"{what}: the workspace needs {sample_workspace_words()} "
                                      f"contiguous int32 words")
    pub = (None, None, 0)
    if publish is not None:
        address, src, words = publish
        _need(src, torch.int32, "publish source", what)
        if workspace is None or not address or words > src.numel():
            raise KernelArgumentError(f"{what}: publishing needs a workspace and a host address, "
                                      f"and {words} words the source holds")
        pub = (int(address), _p(src), int(words))
    _need(out, torch.int32, "out", what)
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelArgumentError(f"{what}: logits must be float32 with unit inner stride")
    if temperature is not None:
        _need(temperature, torch.float32, "temperature", what)
        _need(top_k, torch.int32, "top_k", what)
        _need(top_p, torch.float32, "top_p", what)
        _need(seeds, torch.int64, "seeds", what)
        _need(fresh, torch.int32, "fresh", what)
        _need(slots, torch.int32, "slots", what)
        _need(rng_states, torch.int64, "rng_states", what)
    _check(lib().prb_sample(_p(out), _p(logits), logits.stride(0), logits.shape[1],
                            _p(temperature), _p(top_k), _p(top_p), _p(seeds), _p(fresh), _p(slots),
                            _p(rng_states), n_rows, *pub, _p(workspace), _stream()), what)



# ------------------------------------------- gated branches, norms after the sum, routers
def embed_pair(out, tokens, positions, seq_of_token, q_start, state_slot, prev_state, table,
               pairs, buckets: int, mul_prev: int, mul_cur: int, status, scale: float = 1.0) -> None:
    """out[t,:] = table[tokens[t],:] * scale + pairs[row,:] with row = (prev * mul_prev + token *
    mul_cur) mod buckets, or row ``buckets`` for a sequence's first token; out float32
    [T, width].  ``prev_state`` (int32 [slots]) holds every request's last token between
    steps and is brought up to date by this call."""
    what = "embed_pair"
    _need(out, torch.float32, "out", what)
    for name, t in (("tokens", tokens), ("positions", positions), ("seq_of_token", seq_of_token),
                    ("q_start", q_start), ("state_slot", state_slot), ("prev_state", prev_state)):
        _need(t, torch.int32, name, what)
    _need(table, None, "table", what)
    _need(pairs, table.dtype, "pairs", what)
    n, width = out.shape
    buckets = int(buckets)
    if table.shape[1] != width or pairs.shape[1] != width or pairs.shape[0] != buckets + 1:
        raise KernelArgumentError(f"{what}: table widths differ from the output's, or the pair "
                                  f"table has not buckets + 1 rows")
    if min(tokens.numel(), positions.numel(), seq_of_token.numel()) < n:
        raise KernelArgumentError(f"{what}: fewer token ids, positions or requests than output rows")
    _check(lib().prb_embed_pair(_p(out), _p(tokens), _p(positions), _p(seq_of_token), _p(q_start),
                                _p(state_slot), _p(prev_state), _p(table), _p(pairs), n, width,
                                table.shape[0], buckets, int(mul_prev) % buckets,
                                int(mul_cur) % buckets, prev_state.numel(), state_slot.numel(),
                                dtype_code(table.dtype), float(scale), _p(status), _stream()), what)


def rms_norm(x, out=None, x_out=None, y=None, gate=None, gate_bias=None, gain=None, weight=None,
             rows=None, alpha: float = 1.0, eps: float = 0.0, status=None,
             branch_only: bool = False) -> None:
    """v = alpha * x (+ y, or + sigmoid(gate + gate_bias) * y); r = v / sqrt(mean(v^2) + eps)
    * gain (one number on the device) * weight (per coordinate).  ``branch_only``: the norm is
    the branch's alone and the stream joins after it, r = alpha * x + norm(y) (norm with gain
    and weight as before).  r goes to ``out`` (float32 or
    bfloat16) and/or ``x_out`` (float32; may be ``x`` itself); with ``rows`` row i of the result
    comes from row rows[i] of the inputs.  ``gate`` may be a column slice of a wider tensor."""
    what = "rms_norm"
    _need(x, torch.float32, "x", what)
    width = x.shape[1]
    n_rows = (out if out is not None else x_out).shape[0]
    for name, t in (("out", out), ("x_out", x_out)):
        if t is not None:
            _need(t, None if name == "out" else torch.float32, name, what)
            if t.shape[1] != width or t.shape[0] != n_rows:
                raise KernelArgumentError(f"{what}: {name} has the wrong shape")
    if y is not None:
        _need(y, torch.float32, "y", what)
        if y.shape != x.shape:
            raise KernelArgumentError(f"{what}: y must have x's shape")
    gate_ld = 0
    if gate is not None:
        if y is None or gate.dtype != torch.float32 or gate.stride(1) != 1 or \
                gate.shape[1] != width or gate.shape[0] < x.shape[0]:
            raise KernelArgumentError(f"{what}: gate must be float32 [rows, width] beside a branch y")
        gate_ld = gate.stride(0)
    for name, t, size in (("gate_bias", gate_bias, width), ("gain", gain, 1), ("weight", weight, width)):
        if t is not None:
            _need(t, torch.float32, name, what)
            if t.numel() != size:
                raise KernelArgumentError(f"{what}: {name} must hold {size} numbers")
    if rows is not None:
        _need(rows, torch.int32, "rows", what)
    elif x.shape[0] < n_rows:
        raise KernelArgumentError(f"{what}: fewer input rows than output rows")
    _check(lib().prb_rms_norm(_p(out), _p(x_out), _p(x), _p(y), _p(gate), gate_ld, _p(gate_bias),
                              _p(gain), _p(weight), _p(rows), n_rows, x.shape[0], width,
                              float(alpha), float(eps), 1 if branch_only else 0,
                              dtype_code(out.dtype) if out is not None else F32, _p(status),
                              _stream()), what)


def gate_mul(out, inp, gate) -> None:
    """out[t, i] = inp[t, i] * sigmoid(gate[t, i]) for the columns of ``inp``; inp and gate
    float32 (column slices of wider tensors are fine), out in the activation type with at least
    as many columns."""
    what = "gate_mul"
    for name, t in (("inp", inp), ("gate", gate)):
        if not t.is_cuda or t.dtype != torch.float32 or t.stride(1) != 1:
            raise KernelArgumentError(f"{what}: {name} must be float32 on CUDA with unit inner stride")
    n_rows, n = inp.shape
    if gate.shape[0] < n_rows or gate.shape[1] < n or out.stride(1) != 1 or out.shape[0] < n_rows or \
            out.shape[1] < n:
        raise KernelArgumentError(f"{what}: shapes do not fit")
    _check(lib().prb_gate_mul(_p(out), out.stride(0), _p(inp), inp.stride(0), _p(gate),
                              gate.stride(0), n_rows, n, dtype_code(out.dtype), _stream()), what)


def gated_pair(out, inp, gate_col: int, up_col: int, n: int, out_col: int = 0, limit: float = 0.0,
               act_alpha: float = 1.0, up_shift: float = 0.0, scale=None, group: int = 1) -> None:
    """out[t, out_col + i] = g * sigmoid(act_alpha * g) * (u + up_shift) (* scale[t, i // group])
    for i < n, with g = inp[t, gate_col + i] and u = inp[t, up_col + i] (float32), g capped at
    ``limit`` and u clamped to +-``limit`` when ``limit`` > 0."""
    what = "gated_pair"
    if not inp.is_cuda or inp.dtype != torch.float32 or inp.stride(1) != 1:
        raise KernelArgumentError(f"{what}: inp must be float32 on CUDA with unit inner stride")
    if not out.is_cuda or out.stride(1) != 1 or out.shape[0] < inp.shape[0] or \
            out_col + n > out.shape[1] or max(gate_col, up_col) + n > inp.shape[1]:
        raise KernelArgumentError(f"{what}: columns outside the tensors")
    if scale is not None:
        if scale.dtype != torch.float32 or scale.stride(1) != 1 or scale.shape[0] < inp.shape[0] \
                or scale.shape[1] * group < n:
            raise KernelArgumentError(f"{what}: scale must be float32 [rows, ceil(n / group)]")
    _check(lib().prb_gated_pair(_p(out), out.stride(0), int(out_col), _p(inp), inp.stride(0),
                                int(gate_col), int(up_col), int(n), inp.shape[0], float(limit),
                                float(act_alpha), float(up_shift), _p(scale),
                                0 if scale is None else scale.stride(0), int(group),
                                dtype_code(out.dtype), _stream()), what)


def route(scale, chosen, chosen_w, x, w, bias, top: int) -> None:
    """Router: z = x . w^T + bias in 32-bit (x float32 [T, width]; w [experts, width]), or,
    with ``w`` None, z = x + bias (x float32 [T, experts]: logits a product has made, possibly a
    column slice of a wider tensor); the ``top`` largest per row and the softmax over them.
    scale float32 [T, experts] (zero where not chosen), chosen int32 [T, top], chosen_w
    float32 [T, top]."""
    what = "route"
    if not x.is_cuda or x.dtype != torch.float32 or x.stride(1) != 1:
        raise KernelArgumentError(f"{what}: x must be float32 on CUDA with unit inner stride")
    _need(scale, torch.float32, "scale", what)
    _need(chosen, torch.int32, "chosen", what)
    _need(chosen_w, torch.float32, "chosen_w", what)
    n, width = x.shape
    experts = width if w is None else w.shape[0]
    if w is not None:
        _need(w, None, "w", what)
        if w.shape[1] != width:
            raise KernelArgumentError(f"{what}: shapes do not fit")
    if scale.shape != (n, experts) or chosen.shape != (n, top) or chosen_w.shape != (n, top):
        raise KernelArgumentError(f"{what}: shapes do not fit")
    if bias is not None:
        _need(bias, torch.float32, "bias", what)
    _check(lib().prb_route(_p(scale), _p(chosen), _p(chosen_w), _p(x), x.stride(0), _p(w), _p(bias),
                           n, width, experts, int(top), F32 if w is None else dtype_code(w.dtype),
                           _stream()), what)


# ----------------------------------------------------- attention over a shared latent
def latent_prepare(cq, cache, proj, q_col: int, kv_col: int, wq, wkv, slots, positions, freq,
                   q_rank: int, rank: int, rot_dim: int, rot_dims: int, eps: float, status,
                   rot_scale: float = 1.0, freq_lo=None) -> None:
    """Per token: the query latent proj[t, q_col : q_col + q_rank], unit-RMS-normed with weight
    ``wq``, goes to ``cq`` ([T, >= q_rank], activation type); the key/value latent
    proj[t, kv_col : kv_col + rank], normed with ``wkv``, and the ``rot_dim`` columns after it,
    rotated by the token's position (and multiplied by ``rot_scale`` where rotated), go to the
    token's cache row (``cache``: [pages, 1, page size, rank + rot_dim]).  ``proj`` is float32
    and may be a wider row-major tensor.  ``cq`` None: there is no query latent."""
    what = "latent_prepare"
    if proj.dtype != torch.float32 or proj.stride(1) != 1:
        raise KernelArgumentError(f"{what}: proj must be float32 with unit inner stride")
    _need(cache, None, "cache", what)
    num_pages, kv_heads, page_size, row = cache.shape
    if kv_heads != 1 or row != rank + rot_dim:
        raise KernelArgumentError(f"{what}: the cache must be [pages, 1, page size, {rank + rot_dim}]")
    if cq is not None and (cq.stride(1) != 1 or cq.shape[1] < q_rank or cq.shape[0] < proj.shape[0]):
        raise KernelArgumentError(f"{what}: cq has the wrong shape")
    for name, t in (("wq", wq), ("wkv", wkv), ("freq", freq)):
        if t is not None or name != "wq" or cq is not None:
            _need(t, torch.float32, name, what)
    if cq is None:
        q_rank = 0
    if (cq is not None and wq.numel() != q_rank) or wkv.numel() != rank or \
            freq.numel() < rot_dims // 2 or \
            max(q_col + q_rank, kv_col + rank + rot_dim) > proj.shape[1]:
        raise KernelArgumentError(f"{what}: weights or columns do not fit")
    if slots is not None:
        _need(slots, torch.int32, "slots", what)
    _need(positions, torch.int32, "positions", what)
    _check(lib().prb_latent_prepare(_p(cq), 0 if cq is None else cq.stride(0), _p(cache), _p(proj), proj.stride(0),
                                    int(q_col), int(kv_col), _p(wq), _p(wkv), _p(slots),
                                    _p(positions), _p(freq), proj.shape[0], q_rank, rank, rot_dim,
                                    rot_dims, page_size, num_pages, float(eps),
                                    dtype_code(cache.dtype),
                                    dtype_code(cache.dtype if cq is None else cq.dtype),
                                    float(rot_scale), _p(_freq_lo(freq_lo, rot_dims, what)),
                                    _p(status), _stream()), what)


def _freq_lo(freq_lo, rot_dims: int, what: str):
    """``freq_lo``: float32, one number per rotated pair: what each frequency's rounding to 32
    bits left out (the kernels add it to the frequency in 64-bit); None: nothing."""
    if freq_lo is not None:
        _need(freq_lo, torch.float32, "freq_lo", what)
        if freq_lo.numel() < rot_dims // 2:
            raise KernelArgumentError(f"{what}: {rot_dims // 2} low parts of frequencies wanted")
    return freq_lo


def latent_fold(qa, q, uk, positions, freq, heads: int, dim: int, rot_dim: int, rot_dims: int,
                rank: int, freq_lo=None) -> None:
    """qa[t, h, :rank] = Uk_h^T q[t, h, :dim]; qa[t, h, rank:] = q[t, h, dim:] rotated by the
    token's position.  q float32 [T, heads * (dim + rot_dim)]; uk [heads * dim, rank];
    qa [T, heads, rank + rot_dim], float32 or bfloat16."""
    what = "latent_fold"
    if q.dtype != torch.float32 or q.stride(1) != 1 or q.shape[1] != heads * (dim + rot_dim):
        raise KernelArgumentError(f"{what}: q must be float32 [T, heads * (dim + rot_dim)]")
    _need(qa, None, "qa", what)
    _need(uk, None, "uk", what)
    if tuple(uk.shape) != (heads * dim, rank) or tuple(qa.shape) != (q.shape[0], heads, rank + rot_dim):
        raise KernelArgumentError(f"{what}: shapes do not fit")
    _check(lib().prb_latent_fold(_p(qa), _p(q), q.stride(0), _p(uk), _p(positions), _p(freq),
                                 _p(_freq_lo(freq_lo, rot_dims, what)), q.shape[0], heads, dim, rot_dim, rot_dims, rank,
                                 dtype_code(uk.dtype), dtype_code(qa.dtype), _stream()), what)


def latent_attention(out, qa, cache, block_table, seq_of_token, positions, sinks, scale: float,
                     window, rank: int, status) -> None:
    """out[t, h, :] = sum_j w_j c_j over the keys token t sees, w = softmax of
    scale * qa[t, h] . [c_j | r_j] whose denominator also holds exp(sinks[h]) when ``sinks`` is
    given.  32-bit arithmetic, any sizes (rank up to 1,024)."""
    what = "latent_attention"
    _need(out, torch.float32, "out", what)
    _need(qa, torch.float32, "qa", what)
    _need(cache, None, "cache", what)
    num_pages, kv_heads, page_size, row = cache.shape
    n, heads, d = qa.shape
    if kv_heads != 1 or row != d or tuple(out.shape) != (n, heads, rank) or rank > d:
        raise KernelArgumentError(f"{what}: shapes do not fit")
    if sinks is not None:
        _need(sinks, torch.float32, "sinks", what)
        if sinks.numel() != heads:
            raise KernelArgumentError(f"{what}: one sink per head")
    _need(block_table, torch.int32, "block_table", what)
    _check(lib().prb_latent_attention(_p(out), _p(qa), _p(cache), _p(block_table),
                                      _p(seq_of_token), _p(positions), _p(sinks), n, heads, rank,
                                      d - rank, page_size, block_table.shape[1], num_pages,
                                      float(scale), int(window or 0), dtype_code(cache.dtype),
                                      _p(status), _stream()), what)


def latent_unfold(out, lat, uvt, gate, heads: int, rank: int, vdim: int) -> None:
    """out[t, h*vdim + v] = sigmoid(gate[t, h]) * sum_r uvt[h, r, v] * lat[t, h, r]; ``gate``
    float32 [T, heads] (may be a column slice), or [T, heads * vdim]: a gate per value
    coordinate, or None."""
    what = "latent_unfold"
    _need(lat, torch.float32, "lat", what)
    _need(uvt, None, "uvt", what)
    if tuple(uvt.shape) != (heads, rank, vdim) or tuple(lat.shape[1:]) != (heads, rank) or \
            out.stride(1) != 1 or out.shape[1] < heads * vdim or out.shape[0] < lat.shape[0]:
        raise KernelArgumentError(f"{what}: shapes do not fit")
    gate_ld, gate_per = 0, 1
    if gate is not None:
        if gate.dtype != torch.float32 or gate.stride(1) != 1 or \
                gate.shape[1] not in (heads, heads * vdim) or gate.shape[0] < lat.shape[0]:
            raise KernelArgumentError(f"{what}: gate must be float32 [T, heads] or [T, heads * vdim]")
        gate_ld = gate.stride(0)
        gate_per = vdim if gate.shape[1] == heads * vdim and vdim > 1 else 1
    _check(lib().prb_latent_unfold(_p(out), out.stride(0), _p(lat), _p(uvt), _p(gate), gate_ld,
                                   gate_per, lat.shape[0], heads, rank, vdim, dtype_code(uvt.dtype),
                                   dtype_code(out.dtype), _stream()), what)


def latent_mma_supports(heads: int, rank: int, rot_dim: int) -> bool:
    """Whether ``latent_attention_mma`` takes these sizes (up to 64 heads, rank a multiple of 16
    up to 256, rotated part a multiple of 16)."""
    return bool(lib().prb_latent_mma_supports(int(heads), int(rank), int(rot_dim)))


def latent_mma_single_kw(heads: int) -> int:
    """Into how many parts the warps of a CTA split a key block for single tokens."""
    return int(lib().prb_latent_mma_single_kw(int(heads)))


def latent_mma_rows() -> int:
    """Rows ((token, head) pairs) of a work item of ``latent_attention_mma``."""
    return int(lib().prb_latent_mma_rows())


def latent_attention_mma(out, qa, cache, block_table, seq_of_token, positions, item_row0,
                         item_tokens, item_count, n_items: int, sinks, ws_o, ws_ml, scale: float,
                         window, rank: int, split_keys: int, splits: int, kw: int, ws_rows: int,
                         status, gate=None, rotate=None) -> None:
    """The same as ``latent_attention`` on tensor cores for bfloat16 queries and cache.  Work
    items: item i is ``item_tokens[i]`` (1 if None) consecutive tokens of one request from
    token row ``item_row0[i]`` on, all heads (heads * tokens <= ``ws_rows`` <= 128); ``n_items``
    are launched, ``item_count`` (device int32, or None) bounds them.  Keys go in ``splits``
    ranges of ``split_keys`` positions (a multiple of 64) to a CTA each, whose warps split every
    block of 64 keys ``kw`` ways (1: prompt portions, items of up to 128 rows; 4 or 2: single
    tokens of up to 16 or 32 heads).  ``ws_o`` float32 [n_items * ws_rows * splits * rank] and
    ``ws_ml`` (the same without rank, times 2) hold the partial results of the key ranges,
    which a second kernel joins into ``out``.  ``out`` is float32 [T, heads, rank], or
    bfloat16 of that shape, and then every head's rows are multiplied by sigmoid(gate[t, h])
    when ``gate`` (float32 [T, heads], may be a column slice) is given.  ``rotate`` = (freq,
    rot_dims): the queries come unrotated and the kernel rotates the last part of every row by
    its position as it loads them."""
    what = "latent_attention_mma"
    freq, rot_dims = rotate if rotate is not None else (None, 0)
    if freq is not None:
        _need(freq, torch.float32, "freq", what)
        if freq.numel() < rot_dims // 2:
            raise KernelArgumentError(f"{what}: {rot_dims // 2} frequencies wanted")
    _need(out, None, "out", what)
    if out.dtype not in (torch.float32, torch.bfloat16) or (gate is not None and out.dtype != torch.bfloat16):
        raise KernelArgumentError(f"{what}: out is float32, or bfloat16 (which may take a gate)")
    gate_ld = 0
    if gate is not None:
        if gate.dtype != torch.float32 or gate.stride(1) != 1 or gate.shape[1] != qa.shape[1] or \
                gate.shape[0] < qa.shape[0]:
            raise KernelArgumentError(f"{what}: gate must be float32 [T, heads]")
        gate_ld = gate.stride(0)
    _need(qa, torch.bfloat16, "qa", what)
    _need(cache, torch.bfloat16, "cache", what)
    num_pages, kv_heads, page_size, row = cache.shape
    n, heads, d = qa.shape
    if kv_heads != 1 or row != d or tuple(out.shape) != (n, heads, rank) or rank > d:
        raise KernelArgumentError(f"{what}: shapes do not fit")
    _need(item_row0, torch.int32, "item_row0", what)
    if item_tokens is not None:
        _need(item_tokens, torch.int32, "item_tokens", what)
    if item_row0.numel() < n_items or (item_tokens is not None and item_tokens.numel() < n_items):
        raise KernelArgumentError(f"{what}: the work list is shorter than {n_items} items")
    parts = int(splits)
    _need(ws_o, torch.float32, "ws_o", what)
    _need(ws_ml, torch.float32, "ws_ml", what)
    if ws_o.numel() < n_items * ws_rows * parts * rank or ws_ml.numel() < n_items * ws_rows * parts * 2:
        raise KernelArgumentError(f"{what}: the workspace is too small")
    if sinks is not None:
        _need(sinks, torch.float32, "sinks", what)
    code = lib().prb_latent_attention_mma(
        _p(out) if out.dtype == torch.float32 else None,
        _p(out) if out.dtype == torch.bfloat16 else None, _p(gate), gate_ld, _p(qa), _p(cache), _p(block_table), _p(seq_of_token), _p(positions), _p(item_row0),
        _p(item_tokens), _p(item_count), int(n_items), _p(sinks), _p(ws_o), _p(ws_ml), heads, rank,
        d - rank, page_size, block_table.shape[1], num_pages, float(scale), int(window or 0),
        int(split_keys), int(splits), int(kw), int(ws_rows), _p(freq), int(rot_dims), _p(status),
        _stream())
    _check(code, what)
    if code == 0 and n_items > 0 and splits > 1:
        add_launches(1)                      # the kernel that joins the partial results


# ------------------------------------------------- scaled embedding, routing by scores
def embed_scaled(out, tokens, table, scale: float, keep=None, status=None) -> None:
    """out[t] = table[tokens[t]] * scale (float32 [T, width]); ``keep`` receives the same rows
    a second time (a stream that is joined by its own beginning again later)."""
    what = "embed_scaled"
    _need(out, torch.float32, "out", what)
    _need(tokens, torch.int32, "tokens", what)
    _need(table, None, "table", what)
    n, width = out.shape
    if table.shape[1] != width or tokens.numel() < n:
        raise KernelArgumentError(f"{what}: table width or token count does not fit the output")
    if keep is not None:
        _need(keep, torch.float32, "keep", what)
        if keep.shape[0] < n or keep.shape[1] != width:
            raise KernelArgumentError(f"{what}: keep has the wrong shape")
    _check(lib().prb_embed_scaled(_p(out), _p(keep), _p(tokens), _p(table), n, width,
                                  table.shape[0], float(scale), dtype_code(table.dtype),
                                  _p(status), _stream()), what)


SCORE_CODES = {"sigmoid": 0, "identity": 1, "softmax": 2}
ROUTED_ACT_CODES = {"relu_squared": 0, "relu": 1, "gelu_new": 2, "silu": 3}


def route_scores(weights, chosen, chosen_w, x, w, top: int, score: str = "sigmoid",
                 renormalize: bool = False, factor: float = 1.0) -> None:
    """Router by independent scores: z = x . w^T in 32-bit (x [T, width] float32 or bfloat16; w
    [experts, width]), or, with ``w`` None, x [T, experts] holds z already (possibly a column
    slice of a wider tensor); s = sigmoid(z), z, or softmax(z) over all experts; the ``top``
    largest; weights float32 [T, experts] hold the chosen scores (divided by their sum if
    ``renormalize``, then times ``factor``) and zero
    elsewhere; chosen int32 [T, top] and chosen_w float32 [T, top] list them by rank."""
    what = "route_scores"
    if not x.is_cuda or x.stride(1) != 1:
        raise KernelArgumentError(f"{what}: x must be on CUDA with unit inner stride")
    _need(weights, torch.float32, "weights", what)
    _need(chosen, torch.int32, "chosen", what)
    _need(chosen_w, torch.float32, "chosen_w", what)
    n, width = x.shape
    experts = width if w is None else w.shape[0]
    if w is not None:
        _need(w, None, "w", what)
        if w.shape[1] != width:
            raise KernelArgumentError(f"{what}: shapes do not fit")
    if weights.shape != (n, experts) or chosen.shape != (n, top) or chosen_w.shape != (n, top):
        raise KernelArgumentError(f"{what}: shapes do not fit")
    _check(lib().prb_route_scores(_p(weights), _p(chosen), _p(chosen_w), _p(x), x.stride(0), _p(w),
                                  n, width, experts, int(top), SCORE_CODES[score],
                                  1 if renormalize else 0, float(factor), dtype_code(x.dtype),
                                  F32 if w is None else dtype_code(w.dtype), _stream()), what)


def routed_act(out, inp, in_col: int, n: int, weights, group: int, act: str = "relu_squared",
               weight_on: str = "input") -> None:
    """out[t, i] = act(weights[t, i // group] * inp[t, in_col + i]) for i < n: the activation of
    routed experts whose weight multiplies the expert's input (inp float32: what the experts'
    first, linear product made of the unweighted input); ``weight_on`` "output": the weight
    times act(inp).  Zero where the weight is zero."""
    what = "routed_act"
    if not inp.is_cuda or inp.dtype != torch.float32 or inp.stride(1) != 1:
        raise KernelArgumentError(f"{what}: inp must be float32 on CUDA with unit inner stride")
    if not out.is_cuda or out.stride(1) != 1 or out.shape[0] < inp.shape[0] or n > out.shape[1] \
            or in_col + n > inp.shape[1]:
        raise KernelArgumentError(f"{what}: columns outside the tensors")
    if weights.dtype != torch.float32 or weights.stride(1) != 1 or weights.shape[0] < inp.shape[0] \
            or weights.shape[1] * group < n:
        raise KernelArgumentError(f"{what}: weights must be float32 [rows, ceil(n / group)]")
    _check(lib().prb_routed_act(_p(out), out.stride(0), _p(inp), inp.stride(0), int(in_col), int(n),
                                inp.shape[0], _p(weights), weights.stride(0), int(group),
                                ROUTED_ACT_CODES[act], 1 if weight_on == "output" else 0,
                                dtype_code(out.dtype), _stream()), what)


def route_act(out, inp, in_col: int, router_col: int, experts: int, top: int, group: int,
              score: str = "sigmoid", renormalize: bool = False, act: str = "relu_squared",
              weight_on: str = "input", weights_out=None) -> None:
    """:func:`route_scores` (of the logits at columns ``router_col`` .. of ``inp``) and
    :func:`routed_act` (of the ``experts * group`` columns from ``in_col`` on) in one launch, a
    CTA per row.  ``weights_out`` (optional, float32 [rows, experts]) receives the weights."""
    what = "route_act"
    if not inp.is_cuda or inp.dtype != torch.float32 or inp.stride(1) != 1:
        raise KernelArgumentError(f"{what}: inp must be float32 on CUDA with unit inner stride")
    n = experts * group
    if not out.is_cuda or out.stride(1) != 1 or out.shape[0] < inp.shape[0] or n > out.shape[1] \
            or in_col + n > inp.shape[1] or router_col + experts > inp.shape[1]:
        raise KernelArgumentError(f"{what}: columns outside the tensors")
    if weights_out is not None:
        _need(weights_out, torch.float32, "weights_out", what)
        if weights_out.shape != (inp.shape[0], experts):
            raise KernelArgumentError(f"{what}: weights_out must be [rows, experts]")
    _check(lib().prb_route_act(_p(out), out.stride(0), _p(inp), inp.stride(0), int(in_col),
                               int(router_col), inp.shape[0], int(experts), int(top),
                               SCORE_CODES[score], 1 if renormalize else 0, int(group),
                               ROUTED_ACT_CODES[act], 1 if weight_on == "output" else 0,
                               _p(weights_out), dtype_code(out.dtype), _stream()), what)


# ------------------------------------------------------------------------ retention
def retention_step_supports(dim: int, vdim: int) -> bool:
    """Whether the one-launch form of a retention step takes these sizes."""
    return bool(lib().prb_retention_step_supports(int(dim), int(vdim)))


def retention_step(out, proj, q_col: int, k_col: int, v_col: int, g_col: int, state, q_start,
                   state_slot, positions, decay, freq, n_requests: int, heads: int, dim: int,
                   vdim: int, rot_dims: int, k_scale: float, eps: float, status=None) -> None:
    """Rotation, recurrence and finish (:func:`retention_scan` and :func:`retention_finish`) of
    a step of few tokens in ONE launch, a CTA per (head, request); ``proj`` is not changed.
    ``g_col`` < 0: no gate.  out in the activation type, rows may be wider than heads * vdim."""
    what = "retention_step"
    _need(state, torch.float32, "state", what)
    _need(decay, torch.float32, "decay", what)
    _need(freq, torch.float32, "freq", what)
    for name, t in (("q_start", q_start), ("state_slot", state_slot), ("positions", positions)):
        _need(t, torch.int32, name, what)
    if not proj.is_cuda or proj.dtype != torch.float32 or proj.stride(1) != 1:
        raise KernelArgumentError(f"{what}: proj must be float32 on CUDA with unit inner stride")
    n = proj.shape[0]
    if not out.is_cuda or out.stride(1) != 1 or out.shape[0] < n or out.shape[1] < heads * vdim or \
            decay.numel() != heads or tuple(state.shape[1:]) != (heads, vdim, dim) or \
            q_start.numel() < n_requests + 1 or state_slot.numel() < n_requests or \
            freq.numel() < max(1, rot_dims // 2) or \
            max(q_col, k_col) + heads * dim > proj.shape[1] or \
            max(v_col, g_col) + heads * vdim > proj.shape[1]:
        raise KernelArgumentError(f"{what}: shapes do not fit")
    _check(lib().prb_retention_step(_p(out), out.stride(0), _p(proj), proj.stride(0), int(q_col),
                                    int(k_col), int(v_col), int(g_col), _p(state), _p(q_start),
                                    _p(state_slot), _p(positions), _p(decay), _p(freq), n,
                                    int(n_requests), state.shape[0], heads, dim, vdim,
                                    int(rot_dims), float(k_scale), float(eps),
                                    dtype_code(out.dtype), _p(status), _stream()), what)


def retention_lanes(dim: int) -> int:
    """Lanes the scan spreads a state column over (0: a head size it does not take)."""
    return int(lib().prb_retention_lanes(int(dim)))


def retention_segment() -> int:
    """Tokens of a segment of the segmented scan."""
    return int(lib().prb_retention_segment())


def retention_max_segments(t_cap: int, b_cap: int) -> int:
    """Most segments a step of ``t_cap`` token rows and ``b_cap`` requests can have."""
    return int(lib().prb_retention_max_segments(int(t_cap), int(b_cap)))


def retention_scan(o_raw, proj, q_col: int, k_col: int, v_col: int, state, q_start, state_slot,
                   positions, decay, freq, n_requests: int, heads: int, dim: int, vdim: int,
                   rot_dims: int, k_scale: float, cols: int, status=None, segments=None) -> None:
    """o_raw[t, h] = S_t^T q_t with S_t = decay_h S_(t-1) + k_t v_t^T per request and head, over
    the step's tokens in order, from and back to ``state`` [slots, heads, vdim, dim] float32
    (zero at position 0).  proj float32 [T, ld] holds q, k (heads * dim) and v (heads * vdim)
    at the given columns; q and k are first rotated IN PLACE in ``proj`` (rotate-half, the first
    ``rot_dims`` coordinates; one launch for all tokens) and k scaled by ``k_scale``.  ``cols``:
    value columns per CTA.  ``segments`` = (own, start): two float32 workspaces [n, heads, vdim,
    dim] with n >= retention_max_segments(rows of o_raw, n_requests): portions are cut into
    segments of retention_segment() tokens that run side by side (every segment's own sum, the
    states at the segments' starts one after the other, then the segments with outputs)."""
    what = "retention_scan"
    _need(o_raw, torch.float32, "o_raw", what)
    _need(state, torch.float32, "state", what)
    _need(decay, torch.float32, "decay", what)
    _need(freq, torch.float32, "freq", what)
    for name, t in (("q_start", q_start), ("state_slot", state_slot), ("positions", positions)):
        _need(t, torch.int32, name, what)
    if not proj.is_cuda or proj.dtype != torch.float32 or proj.stride(1) != 1:
        raise KernelArgumentError(f"{what}: proj must be float32 on CUDA with unit inner stride")
    n = o_raw.shape[0]
    if proj.shape[0] < n or o_raw.shape[1] != heads * vdim or decay.numel() != heads or \
            tuple(state.shape[1:]) != (heads, vdim, dim) or q_start.numel() < n_requests + 1 or \
            state_slot.numel() < n_requests or freq.numel() < max(1, rot_dims // 2) or \
            max(q_col, k_col) + heads * dim > proj.shape[1] or v_col + heads * vdim > proj.shape[1]:
        raise KernelArgumentError(f"{what}: shapes do not fit")
    seg_own = seg_start = None
    n_seg = 0
    if segments is not None:
        seg_own, seg_start = segments
        for name, t in (("segments[0]", seg_own), ("segments[1]", seg_start)):
            _need(t, torch.float32, name, what)
            if tuple(t.shape[1:]) != (heads, vdim, dim):
                raise KernelArgumentError(f"{what}: {name} must be [n, heads, vdim, dim]")
        n_seg = min(seg_own.shape[0], seg_start.shape[0])
    _check(lib().prb_retention_scan(_p(o_raw), _p(proj), proj.stride(0), int(q_col), int(k_col),
                                    int(v_col), _p(state), _p(q_start), _p(state_slot),
                                    _p(positions), _p(decay), _p(freq), n, int(n_requests),
                                    state.shape[0], heads, dim, vdim, int(rot_dims), float(k_scale),
                                    int(cols), _p(seg_own), _p(seg_start), n_seg, _p(status),
                                    _stream()), what)
    # (the rotation is a launch of its own; the segmented scan is three)
    add_launches((1 if rot_dims > 0 or float(k_scale) != 1.0 else 0) + (2 if n_seg else 0))


def retention_finish(out, o_raw, proj, g_col: int, seq_of_token, heads: int, vdim: int,
                     eps: float) -> None:
    """out[t, h] = o_raw[t, h] / sqrt(mean(o_raw[t, h]^2) + eps) * silu(proj[t, g_col + h * vdim
    ...]) per head; ``proj`` None: no gate.  out in the activation type, its rows may be wider
    than heads * vdim."""
    what = "retention_finish"
    _need(o_raw, torch.float32, "o_raw", what)
    _need(seq_of_token, torch.int32, "seq_of_token", what)
    n = o_raw.shape[0]
    if not out.is_cuda or out.stride(1) != 1 or out.shape[0] < n or out.shape[1] < heads * vdim:
        raise KernelArgumentError(f"{what}: out has the wrong shape")
    if proj is not None and (proj.dtype != torch.float32 or proj.stride(1) != 1 or
                             proj.shape[0] < n or g_col + heads * vdim > proj.shape[1]):
        raise KernelArgumentError(f"{what}: proj has the wrong shape or type")
    _check(lib().prb_retention_finish(_p(out), out.stride(0), _p(o_raw), _p(proj),
                                      0 if proj is None else proj.stride(0), int(g_col),
                                      _p(seq_of_token), n, heads, vdim, float(eps),
                                      dtype_code(out.dtype), _stream()), what)


# --------------------------------------------------------------- differential attention
def diff_prepare(q_out, cache, proj, q_col: int, k_col: int, v_col: int, slots, positions, freq,
                 heads: int, kv_heads: int, dim: int, vdim: int, rot_dims: int, status=None) -> None:
    """Rotate the two maps of every query and key head of the step (rotate-half, the first
    ``rot_dims`` coordinates); queries go to q_out float32 [T, heads * 2 * dim], keys and
    values to the tokens' cache rows [k map 1 | k map 2 | v] (cache: [pages, kv_heads, page
    size, 2 * dim + vdim]; ``slots`` None: nothing is cached)."""
    what = "diff_prepare"
    _need(q_out, torch.float32, "q_out", what)
    _need(cache, None, "cache", what)
    _need(positions, torch.int32, "positions", what)
    _need(freq, torch.float32, "freq", what)
    if not proj.is_cuda or proj.dtype != torch.float32 or proj.stride(1) != 1:
        raise KernelArgumentError(f"{what}: proj must be float32 on CUDA with unit inner stride")
    n = q_out.shape[0]
    pages, kvh, page_size, rowlen = cache.shape
    if kvh != kv_heads or rowlen != 2 * dim + vdim or q_out.shape[1] != heads * 2 * dim or \
            proj.shape[0] < n or q_col + heads * 2 * dim > proj.shape[1] or \
            k_col + kv_heads * 2 * dim > proj.shape[1] or v_col + kv_heads * vdim > proj.shape[1] \
            or freq.numel() < max(1, rot_dims // 2):
        raise KernelArgumentError(f"{what}: shapes do not fit")
    if slots is not None:
        _need(slots, torch.int32, "slots", what)
    _check(lib().prb_diff_prepare(_p(q_out), _p(cache), _p(proj), proj.stride(0), int(q_col),
                                  int(k_col), int(v_col), _p(slots), _p(positions), _p(freq), n,
                                  heads, kv_heads, dim, vdim, int(rot_dims), page_size, pages,
                                  dtype_code(cache.dtype), _p(status), _stream()), what)


def diff_attention_tile_rows(heads: int, kv_heads: int, dim: int, vdim: int) -> int:
    """Most token rows a CTA of the tiled kernel takes; 0: sizes only the kernel of a CTA per
    (token, head) takes (value heads wider than 128, more than 32 query heads a key head)."""
    return int(lib().prb_diff_attention_tile_rows(heads, kv_heads, dim, vdim))


def diff_attention_single_warps(heads: int, kv_heads: int, dim: int, vdim: int) -> int:
    """Warps of the single-token kernel at these sizes; 0: it does not take them (value heads
    wider than 128)."""
    return int(lib().prb_diff_attention_single_warps(heads, kv_heads, dim, vdim))


def diff_attention(out, q, cache, block_table, seq_of_token, positions, heads: int, dim: int,
                   vdim: int, block: int, scale: float, lam: float, eps: float, out_scale: float,
                   status=None, tile_rows: int = 0, single: bool = False) -> None:
    """Per (token, head): a1 - lam * a2 of two softmax attentions over the same values, then
    unit RMS over vdim times ``out_scale``.  A query at position p sees keys floor(p / block) *
    block .. p (``block`` 0: from 0).  32-bit arithmetic; out in the cache's type.
    ``tile_rows`` > 0: the tiled kernel, a CTA per (that many consecutive token rows, key/value
    head), keys staged in shared memory once for all of them; 0: a CTA per (token, head).
    ``single``: the kernel for steps of single tokens, a CTA per (token, key/value head) whose
    warps share the keys."""
    what = "diff_attention"
    _need(q, torch.float32, "q", what)
    _need(cache, None, "cache", what)
    _need(block_table, torch.int32, "block_table", what)
    _need(seq_of_token, torch.int32, "seq_of_token", what)
    _need(positions, torch.int32, "positions", what)
    n = q.shape[0]
    pages, kv_heads, page_size, rowlen = cache.shape
    if rowlen != 2 * dim + vdim or q.shape[1] != heads * 2 * dim or out.dtype != cache.dtype or \
            out.stride(1) != 1 or out.shape[0] < n or out.shape[1] < heads * vdim:
        raise KernelArgumentError(f"{what}: shapes or types do not fit")
    if single:
        _check(lib().prb_diff_attention_single(
            _p(out), out.stride(0), _p(q), _p(cache), _p(block_table), _p(seq_of_token),
            _p(positions), n, heads, kv_heads, dim, vdim, page_size, block_table.shape[1], pages,
            int(block or 0), float(scale), float(lam), float(eps), float(out_scale),
            dtype_code(cache.dtype), dtype_code(out.dtype), _p(status), _stream()), what)
        return
    if tile_rows > 0:
        _check(lib().prb_diff_attention_tile(
            _p(out), out.stride(0), _p(q), _p(cache), _p(block_table), _p(seq_of_token),
            _p(positions), n, heads, kv_heads, dim, vdim, page_size, block_table.shape[1], pages,
            int(block or 0), int(tile_rows), float(scale), float(lam), float(eps),
            float(out_scale), dtype_code(cache.dtype), dtype_code(out.dtype), _p(status),
            _stream()), what)
        return
    _check(lib().prb_diff_attention(_p(out), out.stride(0), _p(q), _p(cache), _p(block_table),
                                    _p(seq_of_token), _p(positions), n, heads, kv_heads, dim, vdim,
                                    page_size, block_table.shape[1], pages, int(block or 0),
                                    float(scale), float(lam), float(eps), float(out_scale),
                                    dtype_code(cache.dtype), dtype_code(out.dtype), _p(status),
                                    _stream()), what)


# ------------------------------------------------------------------------- time mixing
def tmix_lanes(dim: int) -> int:
    """Lanes a column of the time-mixing state is spread over (0: the head size is beyond the
    scan kernel)."""
    return int(lib().prb_tmix_lanes(int(dim)))


def tmix_shift(out, h, prev_state, mu, seq_of_token, positions, q_start, state_slot,
               status=None) -> None:
    """The blends of a token's input with the previous token's: out[t, s * width + i] =
    h[t, i] + (h[t - 1, i] - h[t, i]) * mu[s, i] for each of mu's rows s.  The row before a
    request's first token of the step is the request's row of ``prev_state`` [slots, width]
    (zeros at position 0).  ``mu`` None: out[t] = [h[t] | h[t - 1] - h[t]]."""
    what = "tmix_shift"
    if mu is not None:
        _need(mu, torch.float32, "mu", what)
    for name, t in (("seq_of_token", seq_of_token), ("positions", positions),
                    ("q_start", q_start), ("state_slot", state_slot)):
        _need(t, torch.int32, name, what)
    n, width = h.shape
    n_mix = 2 if mu is None else mu.shape[0]
    if not h.is_cuda or h.stride(1) != 1 or out.dtype != h.dtype or prev_state.dtype != h.dtype or \
            out.stride(1) != 1 or out.shape[0] < n or out.shape[1] < n_mix * width or \
            (mu is not None and mu.shape[1] != width) or prev_state.shape[1] != width or \
            not prev_state.is_contiguous():
        raise KernelArgumentError(f"{what}: shapes or types do not fit")
    _check(lib().prb_tmix_shift(_p(out), out.stride(0), _p(h), h.stride(0), _p(prev_state), _p(mu),
                                _p(seq_of_token), _p(positions), _p(q_start), _p(state_slot), n,
                                width, n_mix, prev_state.shape[0], dtype_code(h.dtype), _p(status),
                                _stream()), what)


def tmix_step_supports(dim: int, vdim: int) -> bool:
    """Whether :func:`tmix_scan` takes ``finish`` for these head sizes (a CTA then holds all of a
    head's value columns)."""
    return bool(lib().prb_tmix_step_supports(int(dim), int(vdim)))


def tmix_segment() -> int:
    """Tokens a segment of the segmented scan."""
    return int(lib().prb_tmix_segment())


def tmix_max_segments(t_cap: int, b_cap: int) -> int:
    """Segments a step of at most ``t_cap`` tokens in ``b_cap`` requests can have."""
    return int(lib().prb_tmix_max_segments(int(t_cap), int(b_cap)))


def tmix_scan(raw, proj, r_col: int, k_col: int, v_col: int, lr_col: int, w2, w0, u, state, h,
              prev_state, q_start, state_slot, positions, n_requests: int, heads: int, dim: int,
              vdim: int, status=None, segments=None, decays=None, finish=None) -> None:
    """The recurrence over the step's tokens, request by request: per head o_t = (S + diag(u)
    k_t v_t^T)^T r_t, then S <- diag(w_t) S + k_t v_t^T with w_t = exp(-exp(w0 + w2 tanh(lr_t)));
    r, k, v and lr are column ranges of ``proj`` (float32).  ``state`` [slots, heads, vdim, dim]
    float32 is read (zero at position 0) and written back; ``prev_state`` [slots, width]
    receives the request's last row of ``h``.  raw float32 [T, heads * vdim].

    ``segments`` (own, start, decay), workspaces [n, heads, vdim, dim] twice and [n, heads,
    dim] with n >= tmix_max_segments(T, n_requests): portions are cut into segments of
    tmix_segment() tokens that run side by side, and ``decays`` float32 [T, heads * dim]
    receives every token's decays.  ``finish`` (out, g_col, norm_w, eps, out_scale): the scan applies
    :func:`tmix_finish` itself and writes ``out`` instead of ``raw`` (sizes that
    :func:`tmix_step_supports` takes; not with ``segments``)."""
    what = "tmix_scan"
    for name, t in (("raw", raw), ("w2", w2), ("w0", w0), ("u", u), ("state", state)):
        _need(t, torch.float32, name, what)
    for name, t in (("q_start", q_start), ("state_slot", state_slot), ("positions", positions)):
        _need(t, torch.int32, name, what)
    if not proj.is_cuda or proj.dtype != torch.float32 or proj.stride(1) != 1:
        raise KernelArgumentError(f"{what}: proj must be float32 on CUDA with unit inner stride")
    rank = w2.shape[1]
    width = h.shape[1]
    if tuple(state.shape[1:]) != (heads, vdim, dim) or w2.shape[0] != heads * dim or \
            w0.numel() != heads * dim or u.numel() != heads * dim or \
            max(r_col, k_col) + heads * dim > proj.shape[1] or v_col + heads * vdim > proj.shape[1] \
            or lr_col + rank > proj.shape[1] or raw.shape[1] < heads * vdim or \
            prev_state.dtype != h.dtype or prev_state.shape != (state.shape[0], width) or \
            h.stride(1) != 1 or q_start.numel() < n_requests + 1:
        raise KernelArgumentError(f"{what}: shapes or types do not fit")
    if segments is not None:
        own, start, decay = segments
        n = own.shape[0]
        for name, t in (("segments' own sums", own), ("segments' starts", start),
                        ("segments' decays", decay)):
            _need(t, torch.float32, name, what)
        _need(decays, torch.float32, "decays", what)
        if finish is not None or decays.stride(1) != 1 or decays.shape[0] < proj.shape[0] or \
                decays.shape[1] < heads * dim or \
                tuple(own.shape) != (n, heads, vdim, dim) or tuple(start.shape) != tuple(own.shape) \
                or tuple(decay.shape) != (n, heads, dim) or \
                not (own.is_contiguous() and start.is_contiguous() and decay.is_contiguous()):
            raise KernelArgumentError(f"{what}: the segments' workspaces do not fit")
        _check(lib().prb_tmix_scan_segments(
            _p(raw), raw.stride(0), _p(proj), proj.stride(0), int(r_col), int(k_col), int(v_col),
            int(lr_col), _p(decays), decays.stride(0), _p(w2), _p(w0), _p(u), _p(state), _p(h),
            h.stride(0),
            _p(prev_state), _p(q_start), _p(state_slot), _p(positions), proj.shape[0],
            int(n_requests), heads, dim, vdim, rank, width, state.shape[0], dtype_code(h.dtype),
            _p(own), _p(start), _p(decay), n, _p(status), _stream()), what)
        return
    out, out_ld, g_col, norm_w, eps, out_scale = None, 0, 0, None, 0.0, 1.0
    if finish is not None:
        out, g_col, norm_w, eps, out_scale = finish
        _need(norm_w, torch.float32, "norm_w", what)
        if out.dtype != h.dtype or out.stride(1) != 1 or out.shape[0] < proj.shape[0] or \
                out.shape[1] < heads * vdim or g_col + heads * vdim > proj.shape[1] or \
                norm_w.numel() != heads * vdim:
            raise KernelArgumentError(f"{what}: the finish's tensors do not fit")
        out_ld = out.stride(0)
    _check(lib().prb_tmix_scan(_p(raw), raw.stride(0), _p(proj), proj.stride(0), int(r_col),
                               int(k_col), int(v_col), int(lr_col), _p(w2), _p(w0), _p(u), _p(state),
                               _p(h), h.stride(0), _p(prev_state), _p(q_start), _p(state_slot),
                               _p(positions), int(n_requests), heads, dim, vdim, rank, width,
                               state.shape[0], dtype_code(h.dtype), _p(status), _p(out), out_ld,
                               int(g_col), _p(norm_w), float(eps), float(out_scale), _stream()), what)


def tmix_finish(out, raw, proj, g_col: int, norm_w, seq_of_token, heads: int, vdim: int,
                eps: float, out_scale: float = 1.0) -> None:
    """out[t, h] = raw[t, h] / sqrt(mean(raw[t, h]^2) + eps) * norm_w[h] * silu(proj[t, g_col +
    h * vdim ...]) * out_scale per head; out in the activation type (rows may be wider)."""
    what = "tmix_finish"
    _need(raw, torch.float32, "raw", what)
    _need(norm_w, torch.float32, "norm_w", what)
    _need(seq_of_token, torch.int32, "seq_of_token", what)
    n = raw.shape[0]
    if not out.is_cuda or out.stride(1) != 1 or out.shape[0] < n or out.shape[1] < heads * vdim or \
            proj.dtype != torch.float32 or proj.stride(1) != 1 or proj.shape[0] < n or \
            g_col + heads * vdim > proj.shape[1] or norm_w.numel() != heads * vdim:
        raise KernelArgumentError(f"{what}: shapes or types do not fit")
    _check(lib().prb_tmix_finish(_p(out), out.stride(0), _p(raw), raw.stride(0), _p(proj),
                                 proj.stride(0), int(g_col), _p(norm_w), _p(seq_of_token), n, heads,
                                 vdim, float(eps), float(out_scale), dtype_code(out.dtype),
                                 _stream()), what)


# ------------------------------------------------------------------ windowed attention
def wattn_prepare(q_out, cache, proj, q_col: int, k_col: int, v_col: int, q_norm, k_norm, slots,
                  positions, freq, heads: int, kv_heads: int, dim: int, vdim: int, rot_dims: int,
                  eps: float, temp_coef: float, temp_every: int, status=None, head_norm=None,
                  biases=None, freq_lo=None) -> None:
    """Queries and keys of the step's tokens as the attention reads them: a root-mean-square
    norm over the whole projection (``q_norm`` / ``k_norm``: float32 weights, or None), or per
    head (``head_norm`` "before": before the rotation, ``q_norm`` / ``k_norm`` of ``dim`` numbers
    shared by the heads; "after": after the rotation, without weights), ``biases`` = (q, k, v)
    float32 vectors (or None each) that join the projection first, the
    query's temperature 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1) (``temp_every`` 0:
    none), the rotation of each head's first ``rot_dims`` coordinates (rotate-half).  Queries go
    to q_out float32 [T, heads * dim]; keys and values to the tokens' cache rows [k | v]
    (cache [pages, kv_heads, page size, dim + vdim]; ``slots`` None: nothing is cached)."""
    what = "wattn_prepare"
    _need(q_out, torch.float32, "q_out", what)
    _need(cache, None, "cache", what)
    _need(positions, torch.int32, "positions", what)
    _need(freq, torch.float32, "freq", what)
    if not proj.is_cuda or proj.dtype != torch.float32 or proj.stride(1) != 1:
        raise KernelArgumentError(f"{what}: proj must be float32 on CUDA with unit inner stride")
    n = q_out.shape[0]
    pages, kvh, page_size, rowlen = cache.shape
    if kvh != kv_heads or rowlen != dim + vdim or q_out.shape[1] != heads * dim or \
            proj.shape[0] < n or q_col + heads * dim > proj.shape[1] or \
            freq.numel() < max(1, rot_dims // 2):
        raise KernelArgumentError(f"{what}: shapes do not fit")
    if slots is not None:
        _need(slots, torch.int32, "slots", what)
        if k_col + kv_heads * dim > proj.shape[1] or v_col + kv_heads * vdim > proj.shape[1]:
            raise KernelArgumentError(f"{what}: key or value columns outside the projection")
    if head_norm not in (None, "before", "after"):
        raise KernelArgumentError(f"{what}: head_norm is None, 'before' or 'after'")
    mode = {None: 1 if q_norm is not None else 0, "before": 2, "after": 3}[head_norm]
    for name, t, size in (("q_norm", q_norm, dim if mode == 2 else heads * dim),
                          ("k_norm", k_norm, dim if mode == 2 else kv_heads * dim)):
        if t is not None:
            _need(t, torch.float32, name, what)
            if t.numel() != size:
                raise KernelArgumentError(f"{what}: {name} must hold {size} numbers")
    if mode == 2 and (q_norm is None or (slots is not None and k_norm is None)):
        raise KernelArgumentError(f"{what}: a norm per head before the rotation has weights")
    bq, bk, bv = biases if biases is not None else (None, None, None)
    for name, t, size in (("q bias", bq, heads * dim), ("k bias", bk, kv_heads * dim),
                          ("v bias", bv, kv_heads * vdim)):
        if t is not None:
            _need(t, torch.float32, name, what)
            if t.numel() != size:
                raise KernelArgumentError(f"{what}: the {name} must hold {size} numbers")
    _check(lib().prb_wattn_prepare(_p(q_out), _p(cache), _p(proj), proj.stride(0), int(q_col),
                                   int(k_col), int(v_col), _p(q_norm), _p(k_norm), _p(slots),
                                   _p(positions), _p(freq), n, heads, kv_heads, dim, vdim,
                                   int(rot_dims), float(eps), float(temp_coef), int(temp_every),
                                   page_size, pages, dtype_code(cache.dtype), mode, _p(bq),
                                   _p(bk), _p(bv), _p(_freq_lo(freq_lo, rot_dims, what)),
                                   _p(status), _stream()), what)


def wattn_tile_rows(heads: int, kv_heads: int, dim: int, vdim: int) -> int:
    """Most token rows a CTA of the tiled kernel takes; 0: sizes only the kernel of a CTA per
    (token, head) takes."""
    return int(lib().prb_wattn_tile_rows(heads, kv_heads, dim, vdim))


def wattn_single_supports(heads: int, kv_heads: int, dim: int, vdim: int) -> bool:
    """Whether the single-token kernel takes these sizes."""
    return bool(lib().prb_wattn_single_supports(heads, kv_heads, dim, vdim))


def wattn(out, q, cache, block_table, seq_of_token, positions, heads: int, dim: int, vdim: int,
          window: int, keep_first: int, scale: float, gate=None, slopes=None,
          out_scale: float = 1.0, status=None, tile_rows: int = 0, single: bool = False,
          sinks=None, gate_per_value: bool = False) -> None:
    """Softmax attention over cache rows [k | v]: a query at position i sees key j <= i with
    i - j < window (``window`` 0: all) or j < keep_first; score (q . k) * scale - slopes[h] * (i
    - j); ``sinks`` (float32 [heads]): exp(sinks[h]) joins the softmax's denominator once,
    without a key or a value; head h's result times sigmoid(gate[t, h]) (``gate``: float32, may
    be a column slice; ``gate_per_value``: [rows, heads * vdim], a gate per value coordinate) times
    ``out_scale``.  32-bit arithmetic; out in the cache's type.  ``tile_rows`` > 0: the
    tiled kernel (a CTA per that many consecutive token rows and key/value head).  ``single``:
    the kernel for steps of single tokens (a CTA per (token, key/value head) whose warps share
    out the key blocks; sizes that :func:`wattn_single_supports` takes)."""
    what = "wattn"
    _need(q, torch.float32, "q", what)
    _need(cache, None, "cache", what)
    _need(block_table, torch.int32, "block_table", what)
    _need(seq_of_token, torch.int32, "seq_of_token", what)
    _need(positions, torch.int32, "positions", what)
    n = q.shape[0]
    pages, kv_heads, page_size, rowlen = cache.shape
    if rowlen != dim + vdim or q.shape[1] != heads * dim or out.dtype != cache.dtype or \
            out.stride(1) != 1 or out.shape[0] < n or out.shape[1] < heads * vdim:
        raise KernelArgumentError(f"{what}: shapes or types do not fit")
    gate_ld = 0
    if gate is not None:
        if gate.dtype != torch.float32 or gate.stride(1) != 1 or gate.shape[0] < n or \
                gate.shape[1] < heads:
            raise KernelArgumentError(f"{what}: gate must be float32 [rows, heads]")
        gate_ld = gate.stride(0)
    gate_per = 1
    if gate_per_value:
        if gate is None or gate.shape[1] < heads * vdim:
            raise KernelArgumentError(f"{what}: a gate per value coordinate is [rows, heads * vdim]")
        gate_per = vdim
    if sinks is not None:
        _need(sinks, torch.float32, "sinks", what)
        if sinks.numel() != heads:
            raise KernelArgumentError(f"{what}: one sink per head")
    if slopes is not None:
        _need(slopes, torch.float32, "slopes", what)
        if slopes.numel() != heads:
            raise KernelArgumentError(f"{what}: one slope per head")
    common = (_p(out), out.stride(0), _p(q), _p(cache), _p(block_table), _p(seq_of_token),
              _p(positions), _p(gate), gate_ld, _p(slopes), n, heads, kv_heads, dim, vdim,
              page_size, block_table.shape[1], pages, int(window or 0), int(keep_first or 0))
    tail = (float(scale), float(out_scale), dtype_code(cache.dtype), dtype_code(out.dtype),
            _p(sinks), gate_per, _p(status), _stream())
    if single:
        _check(lib().prb_wattn_single(*common, *tail), what)
    elif tile_rows > 0:
        _check(lib().prb_wattn_tile(*common, int(tile_rows), *tail), what)
    else:
        _check(lib().prb_wattn(*common, *tail), what)


# ------------------------------------------------ recurrent units over a state per request
def lru_max_taps() -> int:
    """Most taps of the gated linear recurrence's convolution."""
    return int(lib().prb_lru_max_taps())


def lru_conv(u, proj, x_col: int, x_bias, conv_w, conv_b, conv_state, seq_of_token, positions,
             q_start, state_slot) -> None:
    """u[t, c] = conv_b[c] + sum_j conv_w[c, j] * x[t - (taps - 1 - j), c] with x = proj[:, x_col
    + c] + x_bias[c] (zeros before a sequence's start); the rows before a request's first
    token of the step come from ``conv_state`` [slots, taps - 1, width] (float32, the latest
    last).  u float32 [T, width]; ``proj`` float32, may be a wider row-major tensor."""
    what = "lru_conv"
    _need(u, torch.float32, "u", what)
    n, width = u.shape
    taps = conv_w.shape[1]
    if proj.dtype != torch.float32 or proj.stride(1) != 1 or proj.shape[0] < n or \
            x_col + width > proj.shape[1]:
        raise KernelArgumentError(f"{what}: proj must be float32 [T, >= x_col + width]")
    for name, t, size in (("x_bias", x_bias, width), ("conv_w", conv_w, width * taps),
                          ("conv_b", conv_b, width)):
        if t is not None:
            _need(t, torch.float32, name, what)
            if t.numel() != size:
                raise KernelArgumentError(f"{what}: {name} must hold {size} numbers")
    _need(conv_state, torch.float32, "conv_state", what)
    if tuple(conv_state.shape[1:]) != (max(taps - 1, 0), width):
        raise KernelArgumentError(f"{what}: conv_state must be [slots, taps - 1, width]")
    for name, t in (("seq_of_token", seq_of_token), ("positions", positions), ("q_start", q_start),
                    ("state_slot", state_slot)):
        _need(t, torch.int32, name, what)
    _check(lib().prb_lru_conv(_p(u), _p(proj), proj.stride(0), int(x_col), _p(x_bias), _p(conv_w),
                              _p(conv_b), _p(conv_state), _p(seq_of_token), _p(positions),
                              _p(q_start), _p(state_slot), n, width, taps, conv_state.shape[0],
                              state_slot.numel(), _stream()), what)


def lru_gates(a_out, u, wa_t, wi_t, ba, bi, decay, blocks: int) -> None:
    """Per token and block b of the channels: r = sigmoid(A_b u_b + ba), i = sigmoid(B_b u_b +
    bi) (``wa_t`` / ``wi_t``: [blocks, in, out], the block matrices transposed), a - 1 = expm1(decay
    * r) to ``a_out`` and sqrt(1 - a^2) * i * u in place of u; 32-bit arithmetic."""
    what = "lru_gates"
    _need(a_out, torch.float32, "a_out", what)
    _need(u, torch.float32, "u", what)
    n, width = u.shape
    bw = width // max(1, blocks)
    _need(wa_t, None, "wa_t", what)
    _need(wi_t, wa_t.dtype, "wi_t", what)
    if a_out.shape != u.shape or width % blocks or tuple(wa_t.shape) != (blocks, bw, bw) or \
            tuple(wi_t.shape) != (blocks, bw, bw):
        raise KernelArgumentError(f"{what}: shapes do not fit")
    for name, t in (("ba", ba), ("bi", bi), ("decay", decay)):
        _need(t, torch.float32, name, what)
        if t.numel() != width:
            raise KernelArgumentError(f"{what}: {name} must hold {width} numbers")
    _check(lib().prb_lru_gates(_p(a_out), _p(u), _p(wa_t), _p(wi_t), _p(ba), _p(bi), _p(decay), n,
                               width, int(blocks), dtype_code(wa_t.dtype), _stream()), what)


def lru_segment() -> int:
    """Tokens of a segment of the gated linear recurrence's scan."""
    return int(lib().prb_lru_segment())


def lru_max_segments(t_cap: int, b_cap: int) -> int:
    """Most segments a step of ``t_cap`` token rows and ``b_cap`` requests can have."""
    return int(lib().prb_lru_max_segments(int(t_cap), int(b_cap)))


def lru_step_supports(bw: int) -> bool:
    """Whether the one-launch form takes blocks of ``bw`` channels."""
    return bool(lib().prb_lru_step_supports(int(bw)))


def lru_step(out, proj, y_col: int, x_col: int, y_bias, x_bias, conv_w, conv_b, wa_t, wi_t, ba, bi,
             decay, state, conv_state, q_start, state_slot, positions, n_requests: int,
             blocks: int, out_scale: float = 1.0) -> None:
    """:func:`lru_conv`, :func:`lru_gates` and :func:`lru_scan` of a step of few tokens in one
    launch: a CTA per (request, block of channels)."""
    what = "lru_step"
    n = proj.shape[0]
    width, taps = conv_w.shape
    if proj.dtype != torch.float32 or proj.stride(1) != 1 or max(y_col, x_col) + width > proj.shape[1] \
            or out.stride(1) != 1 or out.shape[0] < n or out.shape[1] < width:
        raise KernelArgumentError(f"{what}: proj must be float32 [T, ld] and out [T, >= width]")
    bw = width // max(1, blocks)
    _need(wa_t, None, "wa_t", what)
    _need(wi_t, wa_t.dtype, "wi_t", what)
    if width % blocks or tuple(wa_t.shape) != (blocks, bw, bw) or tuple(wi_t.shape) != (blocks, bw, bw):
        raise KernelArgumentError(f"{what}: the block matrices must be [blocks, in, out]")
    for name, t, size in (("y_bias", y_bias, width), ("x_bias", x_bias, width), ("conv_w", conv_w, width * taps),
                          ("conv_b", conv_b, width), ("ba", ba, width), ("bi", bi, width), ("decay", decay, width)):
        if t is not None:
            _need(t, torch.float32, name, what)
            if t.numel() != size:
                raise KernelArgumentError(f"{what}: {name} must hold {size} numbers")
    _need(state, torch.float32, "state", what)
    _need(conv_state, torch.float32, "conv_state", what)
    if state.shape[1] != width or tuple(conv_state.shape[1:]) != (taps - 1, width) or \
            q_start.numel() < n_requests + 1:
        raise KernelArgumentError(f"{what}: the state tensors do not fit")
    _check(lib().prb_lru_step(_p(out), out.stride(0), _p(proj), proj.stride(0), int(y_col), int(x_col),
                              _p(y_bias), _p(x_bias), _p(conv_w), _p(conv_b), _p(wa_t), _p(wi_t),
                              _p(ba), _p(bi), _p(decay), _p(state), _p(conv_state), _p(q_start),
                              _p(state_slot), _p(positions), n, int(n_requests), state.shape[0],
                              width, int(blocks), taps, float(out_scale), dtype_code(wa_t.dtype),
                              dtype_code(out.dtype), _stream()), what)


def lru_scan(out, a_in, inp, proj, y_col: int, x_col: int, y_bias, x_bias, state, conv_state,
             q_start, state_slot, positions, n_requests: int, out_scale: float = 1.0,
             segments=None) -> None:
    """S_t = a_t S_(t-1) + inp_t per (request, channel), with ``a_in`` holding a_t - 1 (the
    step is taken as S + (inp + (a - 1) S), which keeps a decay close to one exact), from and to ``state`` [slots, width] (zero at position 0); out[t, c] = S_t * gelu_tanh(proj[t, y_col + c] + y_bias[c]) *
    out_scale; ``conv_state`` then holds the request's last taps - 1 inputs proj[:, x_col + c] +
    x_bias[c].  ``segments`` = (own, keep), two float32 workspaces [n, width] for n >=
    lru_max_segments: portions run in segments of 64 tokens side by side (two launches)."""
    what = "lru_scan"
    _need(a_in, torch.float32, "a_in", what)
    _need(inp, torch.float32, "inp", what)
    _need(state, torch.float32, "state", what)
    _need(conv_state, torch.float32, "conv_state", what)
    n, width = a_in.shape
    taps = conv_state.shape[1] + 1
    if inp.shape != a_in.shape or out.stride(1) != 1 or out.shape[0] < n or out.shape[1] < width or \
            state.shape[1] != width or conv_state.shape[2] != width or \
            proj.dtype != torch.float32 or proj.stride(1) != 1 or \
            max(y_col, x_col) + width > proj.shape[1] or q_start.numel() < n_requests + 1:
        raise KernelArgumentError(f"{what}: shapes do not fit")
    if segments is not None:
        own, keep = segments
        _need(own, torch.float32, "segments' own sums", what)
        _need(keep, torch.float32, "segments' products", what)
        if own.shape != keep.shape or own.shape[1] != width:
            raise KernelArgumentError(f"{what}: the segment workspaces must be [n, width]")
        code = lib().prb_lru_scan_segments(
            _p(out), out.stride(0), _p(a_in), _p(inp), _p(own), _p(keep), own.shape[0], _p(proj),
            proj.stride(0), int(y_col), int(x_col), _p(y_bias), _p(x_bias), _p(state),
            _p(conv_state), _p(q_start), _p(state_slot), _p(positions), n, int(n_requests),
            state.shape[0], width, taps, float(out_scale), dtype_code(out.dtype), _stream())
        _check(code, what)
        if code == 0 and n > 0:
            add_launches(1)
        return
    _check(lib().prb_lru_scan(_p(out), out.stride(0), _p(a_in), _p(inp), _p(proj), proj.stride(0),
                              int(y_col), int(x_col), _p(y_bias), _p(x_bias), _p(state),
                              _p(conv_state), _p(q_start), _p(state_slot), _p(positions), n,
                              int(n_requests), state.shape[0], width, taps, float(out_scale),
                              dtype_code(out.dtype), _stream()), what)


def mmem_supports(dim: int, vdim: int) -> bool:
    """Whether the matrix memory's kernel takes heads of these sizes."""
    return bool(lib().prb_mmem_supports(int(dim), int(vdim)))


def mmem_step(out, proj, cols, i_bias, f_bias, norm_w, state_s, state_n, state_m, q_start,
              state_slot, positions, n_requests: int, heads: int, dim: int, vdim: int, cap: float,
              q_scale: float, eps: float, out_scale: float = 1.0) -> None:
    """The matrix memory over the step's tokens, request by request from and to the state
    slots (``state_s`` [slots, heads, vdim, dim], ``state_n`` [slots, heads, dim], ``state_m``
    [slots, heads], float32, zero at position 0).  ``cols`` = first columns of (q, k, v, i, f,
    gate) in ``proj`` (float32 [T, ld]).  out[t, h * vdim + v] = o / rms(o) * norm_w * sigmoid(gate)
    * out_scale."""
    what = "mmem_step"
    if proj.dtype != torch.float32 or proj.stride(1) != 1 or not proj.is_cuda:
        raise KernelArgumentError(f"{what}: proj must be float32 on CUDA with unit inner stride")
    n = proj.shape[0]
    q_col, k_col, v_col, i_col, f_col, g_col = (int(c) for c in cols)
    if max(q_col + heads * dim, k_col + heads * dim, v_col + heads * vdim, i_col + heads,
           f_col + heads, g_col + heads * vdim) > proj.shape[1] or out.stride(1) != 1 or \
            out.shape[0] < n or out.shape[1] < heads * vdim:
        raise KernelArgumentError(f"{what}: columns outside the tensors")
    for name, t, shape in (("state_s", state_s, (heads, vdim, dim)), ("state_n", state_n, (heads, dim)),
                           ("state_m", state_m, (heads,))):
        _need(t, torch.float32, name, what)
        if tuple(t.shape[1:]) != shape:
            raise KernelArgumentError(f"{what}: {name} must be [slots, {', '.join(map(str, shape))}]")
    for name, t, size in (("i_bias", i_bias, heads), ("f_bias", f_bias, heads),
                          ("norm_w", norm_w, heads * vdim)):
        if t is not None:
            _need(t, torch.float32, name, what)
            if t.numel() != size:
                raise KernelArgumentError(f"{what}: {name} must hold {size} numbers")
    if norm_w is None or q_start.numel() < n_requests + 1:
        raise KernelArgumentError(f"{what}: norm_w or q_start missing")
    _check(lib().prb_mmem_step(_p(out), out.stride(0), _p(proj), proj.stride(0), q_col, k_col,
                               v_col, i_col, f_col, g_col, _p(i_bias), _p(f_bias), _p(norm_w),
                               _p(state_s), _p(state_n), _p(state_m), _p(q_start), _p(state_slot),
                               _p(positions), n, int(n_requests), state_s.shape[0], heads, dim,
                               vdim, float(cap), float(q_scale), float(eps), float(out_scale),
                               dtype_code(out.dtype), _stream()), what)


def mmem_segment() -> int:
    """Tokens of a segment of the matrix memory's scan."""
    return int(lib().prb_mmem_segment())


def mmem_max_segments(t_cap: int, b_cap: int) -> int:
    """Most segments a step of ``t_cap`` token rows and ``b_cap`` requests can have."""
    return int(lib().prb_mmem_max_segments(int(t_cap), int(b_cap)))


def mmem_scan_supports(dim: int) -> bool:
    """Whether the scan takes heads of ``dim`` numbers (up to 512)."""
    return bool(lib().prb_mmem_scan_supports(int(dim)))


def mmem_scan(out, raw, gates, proj, cols, i_bias, f_bias, norm_w, state_s, state_n, state_m,
              q_start, state_slot, positions, seq_of_token, n_requests: int, heads: int, dim: int,
              vdim: int, cap: float, q_scale: float, eps: float, out_scale: float = 1.0,
              columns: int = 0, segments=None) -> None:
    """The same as :func:`mmem_step` for long portions: the tokens' factors first (``gates``
    float32 [T, heads, 4]), then the linear recurrence with a column of S over neighbouring
    lanes (``raw`` float32 [T, heads * vdim]; ``columns`` value columns a CTA), then the finish.
    ``segments`` = (own_s, start_s, own_n, start_n, keep): workspaces of [n, heads, vdim, dim]
    (two), [n, heads, dim] (two) and [n, heads] for n >= mmem_max_segments segments; with them
    portions run in segments of 64 tokens side by side."""
    what = "mmem_scan"
    if proj.dtype != torch.float32 or proj.stride(1) != 1 or not proj.is_cuda:
        raise KernelArgumentError(f"{what}: proj must be float32 on CUDA with unit inner stride")
    n = proj.shape[0]
    q_col, k_col, v_col, i_col, f_col, g_col = (int(c) for c in cols)
    _need(raw, torch.float32, "raw", what)
    _need(gates, torch.float32, "gates", what)
    if max(q_col + heads * dim, k_col + heads * dim, v_col + heads * vdim, i_col + heads,
           f_col + heads, g_col + heads * vdim) > proj.shape[1] or out.stride(1) != 1 or \
            out.shape[0] < n or out.shape[1] < heads * vdim or raw.shape[0] < n or \
            raw.shape[1] != heads * vdim or gates.numel() < n * heads * 4:
        raise KernelArgumentError(f"{what}: shapes do not fit")
    for name, t, shape in (("state_s", state_s, (heads, vdim, dim)), ("state_n", state_n, (heads, dim)),
                           ("state_m", state_m, (heads,))):
        _need(t, torch.float32, name, what)
        if tuple(t.shape[1:]) != shape:
            raise KernelArgumentError(f"{what}: {name} must be [slots, {', '.join(map(str, shape))}]")
    _need(norm_w, torch.float32, "norm_w", what)
    segs, n_seg = (None,) * 5, 0
    if segments is not None:
        segs = tuple(segments)
        n_seg = segs[0].shape[0]
        for t, shape in zip(segs, ((heads, vdim, dim), (heads, vdim, dim), (heads, dim), (heads, dim), (heads,))):
            _need(t, torch.float32, "a segment workspace", what)
            if tuple(t.shape) != (n_seg,) + shape:
                raise KernelArgumentError(f"{what}: a segment workspace has the wrong shape")
    code = lib().prb_mmem_scan(_p(out), out.stride(0), _p(raw), _p(gates), _p(proj), proj.stride(0),
                               q_col, k_col, v_col, i_col, f_col, g_col, _p(i_bias), _p(f_bias),
                               _p(norm_w), _p(state_s), _p(state_n), _p(state_m), _p(q_start),
                               _p(state_slot), _p(positions), _p(seq_of_token), n, int(n_requests),
                               state_s.shape[0], heads, dim, vdim, float(cap), float(q_scale),
                               float(eps), float(out_scale), int(columns) or vdim,
                               *(_p(t) for t in segs), n_seg, dtype_code(out.dtype), _stream())
    _check(code, what)
    if code == 0 and n > 0:
        add_launches(4 if segments is not None else 2)
