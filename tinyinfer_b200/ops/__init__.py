"""Python face of the CUDA kernels: one function per kernel family.

Every function checks shapes and dtypes, allocates its output with torch, and calls an
``extern "C"`` launcher of ``tinyinfer_b200/csrc`` on the current CUDA stream. There is no CPU
path and no library attention or model code behind these names: a tensor that is not on a CUDA
device, or a library that cannot be built, raises.

Conventions: activations and matrices are bfloat16 or float32 (the model's compute dtype),
norm weights, biases and logits are float32, indices are int32, and everything is contiguous.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import library

c_int, c_float, c_void_p, c_ll = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong


class KernelError(RuntimeError):
    pass


_SIGNATURES = {
    "core": {
        "ti_embedding": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "ti_feed_tokens": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
        "ti_rmsnorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p],
        "ti_add": [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_void_p],
        "ti_qk_norm_rope_append": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float,
                                   c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                   c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p],
        "ti_attention_generic": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                 c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                 c_void_p, c_int, c_void_p],
        "ti_gemm_simt": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                         c_int, c_int, c_int, c_void_p],
        "ti_sample": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                      c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                      c_void_p, c_int, c_void_p],
        "ti_argmax": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
        "ti_token_nll": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
        "ti_sample_parts": [],
        "ti_sample_candidates": [],
    },
    # the parts of designs with a cached latent, gated recurrences and routed experts
    "latent": {
        "ti_embedding_scaled": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_int, c_void_p],
        "ti_norm_add": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int, c_void_p],
        "ti_rmsnorm_rows32": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p],
        "ti_relu_squared": [c_void_p, c_void_p, c_ll, c_int, c_void_p],
        "ti_gemm_batched": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_ll,
                            c_ll, c_ll, c_ll, c_int, c_int, c_void_p, c_ll, c_ll, c_int, c_void_p],
        "ti_latent_prepare": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float, c_int, c_int, c_int,
                              c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                              c_int, c_void_p, c_int, c_void_p],
        "ti_latent_query": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                            c_float, c_void_p, c_int, c_void_p],
        "ti_latent_attend": [c_void_p, c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                             c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_int, c_void_p],
        "ti_latent_merge": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "ti_latent_attend_mma_ok": [c_int, c_int],
        "ti_latent_attend_mma": [c_void_p, c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int,
                                 c_void_p, c_void_p],
        "ti_causal_conv": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                           c_int, c_int, c_int, c_int, c_void_p],
        "ti_gated_scan": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p,
                          c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
    },
    # routed experts
    "experts": {
        "ti_moe_route": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                         c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int,
                         c_int, c_void_p],
        "ti_moe_tile_rows": [],
        "ti_moe_gemm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                        c_void_p],
        "ti_moe_wide_tiles_ok": [c_int, c_int],
        "ti_moe_gather": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "ti_moe_silu_glu": [c_void_p, c_void_p, c_ll, c_int, c_void_p, c_int, c_void_p],
        "ti_moe_combine_norm_add": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                    c_int, c_float, c_int, c_void_p],
        "ti_moe_clamped_glu": [c_void_p, c_void_p, c_ll, c_int, c_float, c_float, c_int, c_void_p],
        "ti_moe_combine": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                           c_void_p],
    },
    # parts of designs with several residual streams, short convolutions, attention over [key | value] rows and
    # linear attention with a matrix state
    "hybrid": {
        "ti_streams_embed": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
        "ti_soft_cap": [c_void_p, c_ll, c_float, c_void_p],
        "ti_head_rotation": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p,
                             c_void_p, c_int, c_int, c_int, c_float, c_float, c_float, c_void_p, c_void_p, c_void_p, c_int, c_int,
                             c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p],
        "ti_delta_scan": [c_void_p, c_void_p, c_ll, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int,
                          c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_float, c_float, c_void_p,
                          c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_ll, c_int, c_void_p],
        "ti_streams_step": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int,
                            c_int, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p],
        "ti_gelu": [c_void_p, c_void_p, c_ll, c_int, c_int, c_void_p],
        "ti_scale": [c_void_p, c_ll, c_float, c_void_p],
        "ti_short_conv": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                          c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "ti_conv_state_update": [c_void_p, c_ll, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                 c_void_p],
        "ti_conv_qkv_append": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_ll, c_void_p, c_int, c_float, c_int, c_void_p,
                               c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                               c_int, c_int, c_void_p, c_int, c_void_p],
        "ti_attention_rows": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                              c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_float, c_void_p, c_void_p, c_int, c_int,
                              c_float, c_float, c_void_p, c_int, c_void_p],
        "ti_linear_scan": [c_void_p, c_void_p, c_ll, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int,
                           c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_float, c_void_p,
                           c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_ll, c_void_p, c_int, c_void_p],
        "ti_linear_scan_scratch_floats": [c_int, c_int, c_int, c_int, c_int, c_int],
        "ti_gated_group_norm": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_float,
                                c_int, c_float, c_int, c_int, c_void_p],
    },
}
_SIGNATURES["sm100"] = {
    "ti_gemm_bf16": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                     c_void_p, c_ll, c_void_p, c_int, c_void_p, c_void_p],
    "ti_gemm_bf16_linked": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                            c_void_p, c_ll, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p, c_void_p,
                            c_void_p, c_void_p, c_void_p, c_void_p],
}
_SIGNATURES["sm100"]["ti_gemm_set_pair_form"] = [c_int]
_SIGNATURES["sm100"]["ti_moe_gemm_tcgen05_ok"] = [c_int, c_int, c_int, c_int]
_SIGNATURES["sm100"]["ti_moe_tcgen05_tile_rows"] = []
_SIGNATURES["sm100"]["ti_moe_gemm_tcgen05"] = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                               c_int, c_void_p, c_void_p]
_SIGNATURES["sm100"]["ti_gemm_pair_bf16"] = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                             c_int, c_void_p, c_void_p]
NORM_LINK_MAX_TOKENS = 64   # up to here two products can share an RMSNorm between them (see linear)
PAIR_MIN_TOKENS = 1 << 30   # tests and measurements: from this many tokens on a product is sent to the pair form (two
                            # CTAs a 256 x 256 tile) whatever the library would choose; it chooses by itself from 512 on


def set_pair_form(allowed: bool) -> None:
    """Measurements: whether the library may run products of many tokens in the pair form (default: yes)."""
    _fn("sm100", "ti_gemm_set_pair_form")(1 if allowed else 0)
_SIGNATURES["sm100"]["ti_attention_decode_bf16"] = [
    c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
    c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p]
_SIGNATURES["sm100"]["ti_attention_decode_sink_bf16"] = [
    c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
    c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_float, c_float, c_void_p, c_void_p, c_int, c_int,
    c_float, c_void_p, c_void_p]
_SIGNATURES["sm100"]["ti_attention_prefill_pair_sink_bf16"] = [
    c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
    c_float, c_int, c_int, c_float, c_float, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p, c_void_p]
_SIGNATURES["sm100"]["ti_attention_prefill_tc_sink_bf16"] = [
    c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
    c_float, c_int, c_int, c_int, c_int, c_void_p, c_ll, c_int, c_float, c_float, c_void_p, c_void_p, c_int, c_int,
    c_float, c_void_p, c_void_p]
_SIGNATURES["sm100"]["ti_attention_decode_scratch_floats"] = [c_int, c_int, c_int, c_int, c_int, c_int]
_SIGNATURES["sm100"]["ti_attention_prefill_pair_bf16"] = [
    c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
    c_float, c_int, c_void_p, c_void_p]
_SIGNATURES["sm100"]["ti_attention_prefill_tc_bf16"] = [
    c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
    c_float, c_int, c_int, c_int, c_int, c_void_p, c_ll, c_void_p, c_void_p]
PREFILL_TILE = 256        # most query rows per CTA of the prefill attention kernels (two tiles of 128)
PAIR_MIN_CTAS = 148       # fewer CTAs than this of the two-tile kernel: its tiles run as halves, one a CTA
KEY_SPLIT_MAX_CTAS = 148  # at most half as many CTAs of the one-tile kernel: the keys are shared out over CTAs as well
_bound = {}
_status = {}


def status_words(device) -> torch.Tensor:
    """The two int32 device words through which kernels report what they could not do:
    [0] a bounded wait that ran out (the number of the wait), [1] a token or key whose request holds no
    page for it, or a context longer than the splits it was given. Zero means all is well."""
    key = torch.device(device)
    t = _status.get(key)
    if t is None:
        t = _status[key] = torch.zeros(2, dtype=torch.int32, device=key)
    return t


def kernel_status(device) -> torch.Tensor:
    """The word that kernels with bounded waits set when a wait runs out."""
    return status_words(device)[0:1]


def page_status(device) -> torch.Tensor:
    """The word that kernels set when they meet a token or a key without a page."""
    return status_words(device)[1:2]


def status_message(wait_code: int, page_code: int) -> Optional[str]:
    """What two status words say, or None if both are zero."""
    said = []
    if wait_code == 23:
        said.append("a decode step has more key tiles than its attention kernel counts (2^31: about 137 G keys); "
                    "the step's results are not to be used")
    elif wait_code:
        said.append(f"a kernel gave up waiting on a barrier (status {wait_code}); the step's results are not to be used")
    if page_code:
        said.append(f"a kernel met a token or key without a page (status {page_code})")
    return "; ".join(said) or None


def raise_on_status(device, wait_code: int, page_code: int) -> None:
    """Raises KernelError (and clears the words) if either code, read from ``device``, is set."""
    msg = status_message(wait_code, page_code)
    if msg is not None:
        status_words(device).zero_()
        raise KernelError(msg)


def check_kernel_status() -> None:
    """Raises if any kernel reported a wait that ran out or a missing page (synchronises)."""
    for device, t in list(_status.items()):
        wait_code, page_code = t.tolist()
        raise_on_status(device, wait_code, page_code)


_WORKSPACE_FLOATS = 12 * 1024 * 1024     # 48 MB of float32 partial tiles for the stream-k cuts of matrix products
_NUM_COUNTERS = 16384
_workspace = {}


def _gemm_scratch(device):
    """(partials, counters) shared by all tensor-core matrix products on this device; safe because
    they are ordered on one stream and every launch leaves the counters at zero."""
    key = torch.device(device)
    pair = _workspace.get(key)
    if pair is None:
        pair = _workspace[key] = (torch.empty(_WORKSPACE_FLOATS, dtype=torch.float32, device=key),
                                  torch.zeros(_NUM_COUNTERS, dtype=torch.int32, device=key))
    return pair


def _tensor_core_ok(x: torch.Tensor, w: torch.Tensor, *others) -> bool:
    """The tcgen05 kernels take bfloat16 operands whose rows start on 16-byte boundaries."""
    if x.dtype != torch.bfloat16 or x.shape[1] % 8:
        return False
    return all(t is None or t.data_ptr() % 16 == 0 for t in (x, w) + others)


def _fn(lib_name: str, name: str):
    key = (lib_name, name)
    fn = _bound.get(key)
    if fn is None:
        lib = library.load(lib_name)
        fn = getattr(lib, name)
        fn.argtypes = _SIGNATURES[lib_name][name]
        fn.restype = c_int
        _bound[key] = fn
    return fn


def _run(lib_name: str, name: str, *args) -> None:
    rc = _fn(lib_name, name)(*args)
    if rc != 0:
        msg = library.load(lib_name).ti_last_error().decode(errors="replace")
        raise KernelError(f"{name} failed ({rc}): {msg}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream's handle (the raw query is an order of magnitude cheaper than
    torch.cuda.current_stream(), and this runs once per kernel launch)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"compute dtype must be float32 or bfloat16, got {t.dtype}")


def _check(t: torch.Tensor, name: str, dtype=None, ndim: Optional[int] = None) -> torch.Tensor:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor: tinyinfer_b200 has no CPU path")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{name} must have {ndim} dimensions, got shape {tuple(t.shape)}")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    return t


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


# ---------------------------------------------------------------------- elementwise
def embedding(token_ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """rows of ``table`` [V, H] at ``token_ids`` int32 [T] -> [T, H]."""
    _check(token_ids, "token_ids", torch.int32, 1)
    _check(table, "table", None, 2)
    out = torch.empty((token_ids.shape[0], table.shape[1]), dtype=table.dtype, device=table.device)
    _run("core", "ti_embedding", out.data_ptr(), table.data_ptr(), token_ids.data_ptr(),
         token_ids.shape[0], table.shape[1], table.shape[0], _dtype_code(table), _stream())
    return out


def feed_tokens(token_ids: torch.Tensor, dst_rows: torch.Tensor, src_rows: torch.Tensor, src: torch.Tensor) -> None:
    """token_ids[dst_rows[i]] = src[src_rows[i]] wherever dst_rows[i] >= 0 (all int32, on the device): tokens
    that a step sampled become inputs of the next step without a trip to the host."""
    _check(token_ids, "token_ids", torch.int32, 1)
    _check(dst_rows, "dst_rows", torch.int32, 1)
    _check(src_rows, "src_rows", torch.int32, 1)
    _check(src, "src", torch.int32, 1)
    if src_rows.shape[0] != dst_rows.shape[0]:
        raise KernelError("feed_tokens: one source row per destination row")
    _run("core", "ti_feed_tokens", token_ids.data_ptr(), dst_rows.data_ptr(), src_rows.data_ptr(), src.data_ptr(),
         dst_rows.shape[0], _stream())


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float,
            rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """w * x * rsqrt(mean(x^2) + eps) over the last axis; ``rows`` int32 [N] picks input rows."""
    _check(x, "x")
    _check(weight, "weight", torch.float32, 1)
    size = x.shape[-1]
    if weight.shape[0] != size:
        raise KernelError(f"norm weight has {weight.shape[0]} entries, rows have {size}")
    if rows is None:
        out = torch.empty_like(x)
        n = x.numel() // size
    else:
        _check(rows, "rows", torch.int32, 1)
        if x.dim() != 2:
            raise KernelError("row selection needs a 2-D input")
        n = rows.shape[0]
        out = torch.empty((n, size), dtype=x.dtype, device=x.device)
    _run("core", "ti_rmsnorm", out.data_ptr(), x.data_ptr(), weight.data_ptr(), _ptr(rows), n, size,
         float(eps), _dtype_code(x), _stream())
    return out


def add(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a + b, summed in float32 and rounded once."""
    _check(a, "a")
    _check(b, "b", a.dtype)
    if a.shape != b.shape:
        raise KernelError(f"add: shapes differ {tuple(a.shape)} vs {tuple(b.shape)}")
    out = torch.empty_like(a)
    _run("core", "ti_add", out.data_ptr(), a.data_ptr(), b.data_ptr(), a.numel(), _dtype_code(a), _stream())
    return out


# ---------------------------------------------------------------------- matrix products
class NormLink:
    """What a product leaves for the RMSNorm behind it, when that norm is spread over the two products
    around it: ``scaled`` = x * g in x's dtype (x: the product's output as rounded, g: the norm's weight),
    ``sums`` float32 [parts, M]: per token, partial sums of squares of x; ``weight`` is g itself (kept to
    tell which norm the link was made for), ``size`` the length of a row of x."""

    def __init__(self, scaled, sums, parts, weight, size):
        self.scaled, self.sums, self.parts, self.weight, self.size = scaled, sums, parts, weight, size


def norm_link_ok(x: torch.Tensor) -> bool:
    """True if the products around an RMSNorm of ``x`` can share it (bfloat16 on the tensor cores, at
    most 64 rows): the norm kernel between them, a hop of a decode step, is then left out."""
    return x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[0] <= NORM_LINK_MAX_TOKENS


def _gemm_linked(out, x, w, bias, residual, m, n, k, gated, scale, emit_weight):
    ws, counters = _gemm_scratch(x.device)
    scaled = sums = None
    if emit_weight is not None:
        scaled = torch.empty((m, n), dtype=x.dtype, device=x.device)
        sums = torch.empty(((n + 127) // 128, m), dtype=torch.float32, device=x.device)
    written = ctypes.c_int(0)
    _run("sm100", "ti_gemm_bf16_linked", out.data_ptr(), x.data_ptr(), w.data_ptr(), _ptr(bias), _ptr(residual),
         m, n, k, gated, ws.data_ptr(), ws.numel(), counters.data_ptr(), counters.numel(),
         scale[0].sums.data_ptr() if scale else None, scale[0].parts if scale else 0,
         scale[0].size if scale else 0, float(scale[1]) if scale else 0.0,
         _ptr(emit_weight), _ptr(scaled), _ptr(sums), ctypes.addressof(written),
         kernel_status(x.device).data_ptr(), _stream())
    if emit_weight is None or written.value == 0:
        return None
    return NormLink(scaled, sums, written.value, emit_weight, n)


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
           residual: Optional[torch.Tensor] = None, out_float32: bool = False, *,
           link: Optional[NormLink] = None, link_eps: float = 0.0,
           next_norm_weight: Optional[torch.Tensor] = None):
    """x [M, K] . w [N, K]^T (+ bias [N]) (+ residual [M, N]), float32 accumulation.
    ``out_float32`` stores the accumulator unrounded (logits).

    An RMSNorm between two products of at most 64 tokens can be spread over them.
    ``next_norm_weight`` (float32 [N]): the weight of the norm that follows THIS product; the result is
    then (out, NormLink or None): the link, if the kernel could make it, holds out * weight and the
    sums of squares of out's rows. ``link`` (with ``link_eps``): x is ``link.scaled`` of the norm BEFORE
    this product, and every output row is multiplied by rsqrt(mean(x_before^2) + eps) here."""
    _check(x, "x", None, 2)
    _check(w, "w", x.dtype, 2)
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k:
        raise KernelError(f"linear: x has {k} columns, w has {w.shape[1]}")
    if bias is not None:
        _check(bias, "bias", torch.float32, 1)
    if residual is not None:
        _check(residual, "residual", x.dtype, 2)
        if tuple(residual.shape) != (m, n):
            raise KernelError("linear: residual shape differs from the output's")
    out = torch.empty((m, n), dtype=torch.float32 if out_float32 else x.dtype, device=x.device)
    wants_link = next_norm_weight is not None
    if link is not None or wants_link:
        if out_float32 or not (_tensor_core_ok(x, w) and norm_link_ok(x)):
            if link is not None:
                raise KernelError("linear: a norm link needs the tensor-core product of at most 64 rows")
        else:
            made = _gemm_linked(out, x, w, bias, residual, m, n, k, 0, (link, link_eps) if link else None,
                                next_norm_weight)
            return (out, made) if wants_link else out
    if _tensor_core_ok(x, w) and m >= PAIR_MIN_TOKENS and n >= 256:
        _run("sm100", "ti_gemm_pair_bf16", out.data_ptr(), x.data_ptr(), w.data_ptr(), _ptr(bias), _ptr(residual),
             m, n, k, 0, int(out_float32), kernel_status(x.device).data_ptr(), _stream())
        return (out, None) if wants_link else out
    if _tensor_core_ok(x, w):
        ws, counters = _gemm_scratch(x.device)
        _run("sm100", "ti_gemm_bf16", out.data_ptr(), x.data_ptr(), w.data_ptr(), _ptr(bias), _ptr(residual),
             m, n, k, 0, int(out_float32), ws.data_ptr(), ws.numel(), counters.data_ptr(), counters.numel(),
             kernel_status(x.device).data_ptr(), _stream())
        return (out, None) if wants_link else out
    _run("core", "ti_gemm_simt", out.data_ptr(), x.data_ptr(), w.data_ptr(), _ptr(bias), _ptr(residual),
         m, n, k, 0, int(out_float32 and x.dtype != torch.float32), _dtype_code(x), _stream())
    return (out, None) if wants_link else out


def gated_linear(x: torch.Tensor, w_gate_up: torch.Tensor, *, link: Optional[NormLink] = None,
                 link_eps: float = 0.0) -> torch.Tensor:
    """silu(x.Wg^T) * (x.Wu^T) with ``w_gate_up`` = [Wg; Wu] of shape [2I, K] -> [M, I]; the
    activation and the product act on the float32 accumulators, one rounding. ``link``: as in
    ``linear`` (both halves are scaled before the activation)."""
    _check(x, "x", None, 2)
    _check(w_gate_up, "w_gate_up", x.dtype, 2)
    m, k = x.shape
    if w_gate_up.shape[1] != k or w_gate_up.shape[0] % 2:
        raise KernelError("gated_linear: weight must be [2I, K]")
    inter = w_gate_up.shape[0] // 2
    out = torch.empty((m, inter), dtype=x.dtype, device=x.device)
    if link is not None:
        if not (_tensor_core_ok(x, w_gate_up) and norm_link_ok(x)):
            raise KernelError("gated_linear: a norm link needs the tensor-core product of at most 64 rows")
        _gemm_linked(out, x, w_gate_up, None, None, m, inter, k, 1, (link, link_eps), None)
        return out
    if _tensor_core_ok(x, w_gate_up) and m >= PAIR_MIN_TOKENS and inter >= 128:
        _run("sm100", "ti_gemm_pair_bf16", out.data_ptr(), x.data_ptr(), w_gate_up.data_ptr(), None, None,
             m, inter, k, 1, 0, kernel_status(x.device).data_ptr(), _stream())
        return out
    if _tensor_core_ok(x, w_gate_up):
        ws, counters = _gemm_scratch(x.device)
        _run("sm100", "ti_gemm_bf16", out.data_ptr(), x.data_ptr(), w_gate_up.data_ptr(), None, None,
             m, inter, k, 1, 0, ws.data_ptr(), ws.numel(), counters.data_ptr(), counters.numel(),
             kernel_status(x.device).data_ptr(), _stream())
        return out
    _run("core", "ti_gemm_simt", out.data_ptr(), x.data_ptr(), w_gate_up.data_ptr(), None, None,
         m, inter, k, 1, 0, _dtype_code(x), _stream())
    return out


# ---------------------------------------------------------------------- attention
class Rotation:
    """How a position turns the features of a head: what a position-encoding part hands to a mixer, which
    passes it on to ``qk_norm_rope_append`` unread. The first ``rotary_dim`` features of every head are
    rotated in pairs, (j, j + rotary_dim / 2) or, ``interleaved``, (2j, 2j + 1), pair j of position p by
    the angle p * inv_freq[j] (``inv_freq`` float32 [rotary_dim / 2]) or by the angle whose cosine and
    sine stand in ``cos_sin`` (float32 [positions, rotary_dim]: a row holds the rotary_dim / 2 cosines,
    then the sines; any encoding whose angles depend on the position alone). Exactly one of the two.
    ``factor`` multiplies every cosine and sine (an encoding that lengthens what it turns)."""

    def __init__(self, rotary_dim: int, inv_freq: Optional[torch.Tensor] = None,
                 cos_sin: Optional[torch.Tensor] = None, interleaved: bool = False, factor: float = 1.0):
        if (inv_freq is None) == (cos_sin is None):
            raise KernelError("a rotation needs inverse frequencies or a table of cosines and sines, one of them")
        if rotary_dim <= 0 or rotary_dim % 2:
            raise KernelError(f"rotary_dim must be positive and even, got {rotary_dim}")
        if inv_freq is not None:
            if inv_freq.dtype != torch.float32 or tuple(inv_freq.shape) != (rotary_dim // 2,):
                raise KernelError("inv_freq must be float32 with rotary_dim / 2 entries")
        elif cos_sin.dtype != torch.float32 or cos_sin.dim() != 2 or cos_sin.shape[1] != rotary_dim:
            raise KernelError("cos_sin must be float32 [positions, rotary_dim]")
        self.rotary_dim, self.inv_freq, self.cos_sin, self.interleaved = rotary_dim, inv_freq, cos_sin, bool(interleaved)
        self.factor = float(factor)


def qk_norm_rope_append(qkv: torch.Tensor, *, num_heads: int, num_kv_heads: int, head_dim: int,
                        q_norm_weight: Optional[torch.Tensor], k_norm_weight: Optional[torch.Tensor],
                        eps: float, positions: torch.Tensor, token_seq: torch.Tensor,
                        kv_cache: Optional[torch.Tensor], block_table: torch.Tensor,
                        rotation: Optional[Rotation] = None,
                        inv_freq: Optional[torch.Tensor] = None, rotary_dim: int = 0,
                        status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Splits ``qkv`` [T, (Hq + 2 Hkv) D] by heads; norms q and k per head, rotates them by
    their positions, returns q [T, Hq, D] and writes k and v into the pages of
    ``kv_cache`` [2, pages, Hkv, page, D] (None: the entry only reads the cache).
    ``rotation``: a ``Rotation`` or None (positions are not used); ``inv_freq`` with ``rotary_dim``
    is short for the half-split rotation by position * inv_freq."""
    _check(qkv, "qkv", None, 2)
    t = qkv.shape[0]
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise KernelError("qk_norm_rope_append: qkv width does not match the head counts")
    _check(positions, "positions", torch.int32, 1)
    _check(token_seq, "token_seq", torch.int32, 1)
    _check(block_table, "block_table", torch.int32, 2)
    for name, w in (("q_norm_weight", q_norm_weight), ("k_norm_weight", k_norm_weight)):
        if w is not None:
            _check(w, name, torch.float32, 1)
            if w.shape[0] != head_dim:
                raise KernelError(f"{name} must have head_dim entries")
    if rotation is None and inv_freq is not None:
        rotation = Rotation(rotary_dim, inv_freq=inv_freq)
    if rotation is not None:
        if rotation.rotary_dim > head_dim:
            raise KernelError(f"rotary_dim {rotation.rotary_dim} exceeds head_dim {head_dim}")
        if rotation.factor != 1.0:
            raise KernelError("qk_norm_rope_append turns without a factor; head_rotation takes one")
        _check(rotation.inv_freq if rotation.inv_freq is not None else rotation.cos_sin, "the rotation's tensor")
    page_size = num_pages = 1
    if kv_cache is not None:
        _check(kv_cache, "kv_cache", qkv.dtype, 5)
        if kv_cache.shape[0] != 2 or kv_cache.shape[2] != num_kv_heads or kv_cache.shape[4] != head_dim:
            raise KernelError(f"kv_cache shape {tuple(kv_cache.shape)} is not [2, pages, Hkv, page, D]")
        num_pages, page_size = kv_cache.shape[1], kv_cache.shape[3]
    q = torch.empty((t, num_heads, head_dim), dtype=qkv.dtype, device=qkv.device)
    rot = rotation
    _run("core", "ti_qk_norm_rope_append", q.data_ptr(), qkv.data_ptr(), _ptr(kv_cache),
         _ptr(q_norm_weight), _ptr(k_norm_weight), float(eps),
         _ptr(rot.inv_freq) if rot else None, _ptr(rot.cos_sin) if rot else None,
         rot.cos_sin.shape[0] if rot and rot.cos_sin is not None else 0, int(rot.interleaved) if rot else 0,
         rot.rotary_dim if rot else 0, positions.data_ptr(), token_seq.data_ptr(),
         block_table.data_ptr(), block_table.shape[1], t, num_heads, num_kv_heads, head_dim,
         page_size, num_pages, _ptr(status), _dtype_code(qkv), _stream())
    return q


def plan_attention(q_lens, starts):
    """Splits a step's entries into single decoded tokens and portions of prompts.
    Returns (decode_rows, tiles, num_pair_tiles): flat rows of entries that bring one token, and for the
    others tiles [entry, first flat row, rows, first position]. A portion is cut into tiles of
    PREFILL_TILE = 256 query rows for the kernel that runs two query tiles a CTA; what is left at its end,
    if it is at most 128 rows, is a tile for the kernel with one. The first ``num_pair_tiles`` tiles are
    the former, the rest the latter; each kind longest key range first."""
    decode_rows, pairs, singles = [], [], []
    row = 0
    for i, (n, start) in enumerate(zip(q_lens, starts)):
        if n == 1:
            decode_rows.append(row)
        else:
            off = 0
            while n - off > PREFILL_TILE // 2:
                rows = min(PREFILL_TILE, n - off)
                pairs.append((i, row + off, rows, start + off))
                off += rows
            if off < n:
                singles.append((i, row + off, n - off, start + off))
        row += n
    pairs.sort(key=lambda t: -(t[3] + t[2]))
    singles.sort(key=lambda t: -(t[3] + t[2]))
    return decode_rows, [x for t in pairs + singles for x in t], len(pairs)


def attention_tensor_cores_ok(q: torch.Tensor, kv_cache: torch.Tensor) -> bool:
    """The tensor-core attention kernels take bfloat16, head sizes 64 and 128, up to 16 query heads
    per kv head, and pages of 16, 32 or a multiple of 64 tokens."""
    _, hq, d = q.shape
    hkv, page = kv_cache.shape[2], kv_cache.shape[3]
    return (q.dtype == torch.bfloat16 and d in (64, 128) and hq % hkv == 0 and hq // hkv <= 16
            and (page in (16, 32) or page % 64 == 0))


_generic_warned = set()


def _warn_generic_attention(hq: int, hkv: int, d: int, page_size: int) -> None:
    """Says once per shape that a bfloat16 model runs its attention on the generic float32-arithmetic
    kernel: right, but many times slower than the tensor-core kernels."""
    key = (hq, hkv, d, page_size)
    if key in _generic_warned:
        return
    _generic_warned.add(key)
    import warnings
    warnings.warn(f"tinyinfer_b200: attention with {hq} query heads over {hkv} kv heads, head_dim {d}, pages of "
                  f"{page_size} runs on the generic kernel (the tensor-core kernels take head_dim 64 or 128, at most "
                  f"16 query heads per kv head, pages of 16, 32 or a multiple of 64): correct, but far slower",
                  RuntimeWarning, stacklevel=3)


_attn_scratch = {}
_attn_scratch_outgrown = []     # kept alive: captured graphs may still write their partials there


def _decode_scratch(device, floats: int) -> torch.Tensor:
    key = torch.device(device)
    t = _attn_scratch.get(key)
    if t is None or t.numel() < floats:
        if t is not None:
            _attn_scratch_outgrown.append(t)
        t = _attn_scratch[key] = torch.empty(max(floats, 1 << 20), dtype=torch.float32, device=key)
    return t


_scratch_floats = {}


def decode_scratch_floats(num_rows: int, hq: int, hkv: int, head_dim: int, max_context: int, window: int = 0) -> int:
    """Floats of scratch the decode attention kernel needs for this batch (a slot for every CTA's and every
    (request, kv head)'s partial result), as the library says. A function of its arguments alone."""
    key = (num_rows, hq, hkv, head_dim, max_context, window)
    n = _scratch_floats.get(key)
    if n is None:
        fn = _fn("sm100", "ti_attention_decode_scratch_floats")
        fn.restype = ctypes.c_longlong
        n = _scratch_floats[key] = int(fn(*key))
    return n


def release_scratch(device) -> None:
    """Drops the scratch buffers kept for ``device`` (they are made again when next needed). Only when no
    captured graph that uses them will be replayed again."""
    key = torch.device(device)
    _attn_scratch.pop(key, None)
    _attn_scratch_outgrown.clear()
    _workspace.pop(key, None)
    _argmax_scratch.pop(key, None)
    _sample_scratch.pop(key, None)


def paged_attention(q: torch.Tensor, kv_cache: torch.Tensor, *, positions: torch.Tensor,
                    token_seq: torch.Tensor, block_table: torch.Tensor, scale: float,
                    window: Optional[int] = None, step=None,
                    status: Optional[torch.Tensor] = None, sink: Optional[float] = None,
                    out_scale: float = 1.0, head_sinks: Optional[torch.Tensor] = None,
                    gate: Optional[torch.Tensor] = None, gate_offset: int = 0, softcap: float = 0.0) -> torch.Tensor:
    """Causal attention of q [T, Hq, D] over the pages of each token's own request.
    Token t sees keys max(0, pos - window + 1) .. pos of request ``token_seq[t]``.
    ``sink``: a logit whose exponential joins every softmax denominator without a value (0.0 adds one to the sum
    of exp(score)); ``head_sinks`` float32 [Hq]: such a logit per query head instead; ``gate`` [T, cols] of q's dtype:
    the output of (token, head) is multiplied by sigmoid(gate[token, gate_offset + head]); ``out_scale``: a factor on
    the output before its rounding; ``softcap`` > 0: a score s becomes softcap * tanh(s / softcap) before the softmax.
    Returns [T, Hq * D]. ``step`` (the StepContext of the batch) carries the split of the batch
    into decoded tokens and prompt portions; without it the split is derived here (a device read)."""
    _check(q, "q", None, 3)
    _check(kv_cache, "kv_cache", q.dtype, 5)
    _check(positions, "positions", torch.int32, 1)
    _check(token_seq, "token_seq", torch.int32, 1)
    _check(block_table, "block_table", torch.int32, 2)
    t, hq, d = q.shape
    _, num_pages, hkv, page_size, d2 = kv_cache.shape
    if d2 != d or kv_cache.shape[0] != 2:
        raise KernelError("paged_attention: kv_cache does not match q")
    out = torch.empty((t, hq * d), dtype=q.dtype, device=q.device)
    if t == 0:
        return out
    has_sink, sink_v = int(sink is not None), float(sink or 0.0)
    _check_head_extras(q, head_sinks, gate, gate_offset)
    extras = (_ptr(head_sinks), _ptr(gate), gate.shape[1] if gate is not None else 0, int(gate_offset), float(softcap or 0.0))
    if not attention_tensor_cores_ok(q, kv_cache):
        if q.dtype == torch.bfloat16:
            _warn_generic_attention(hq, hkv, d, page_size)
        if softcap or has_sink or out_scale != 1.0 or head_sinks is not None or gate is not None:
            return attention_rows(q, kv_cache, v_dim=d, positions=positions, token_seq=token_seq, block_table=block_table,
                                  scale=scale, sink=sink, window=window, out_scale=out_scale, status=status,
                                  head_sinks=head_sinks, gate=gate, gate_offset=gate_offset, softcap=softcap)
        _run("core", "ti_attention_generic", out.data_ptr(), q.data_ptr(), kv_cache.data_ptr(),
             positions.data_ptr(), token_seq.data_ptr(), block_table.data_ptr(), block_table.shape[1],
             t, hq, hkv, d, page_size, num_pages, float(scale), int(window or 0), _ptr(status),
             _dtype_code(q), _stream())
        return out
    if step is not None:
        decode_rows, num_decode = step.decode_rows, step.num_decode
        tiles, num_tiles, max_context = step.prefill_tiles, step.num_prefill_tiles, step.max_context
        num_pairs = step.num_pair_tiles
    else:
        pos_h, seq_h = positions.tolist(), token_seq.tolist()
        q_lens, starts = [], []
        for i, (p_, s_) in enumerate(zip(pos_h, seq_h)):
            if i and seq_h[i - 1] == s_ and pos_h[i - 1] + 1 == p_:
                q_lens[-1] += 1
            else:
                q_lens.append(1)
                starts.append(p_)
        # entries here are runs of consecutive positions; their request index comes from token_seq
        rows_l, tiles_l, num_pairs = plan_attention(q_lens, starts)
        firsts, r = [], 0
        for n in q_lens:
            firsts.append(seq_h[r])
            r += n
        for k in range(0, len(tiles_l), 4):
            tiles_l[k] = firsts[tiles_l[k]]
        decode_rows = torch.tensor(rows_l or [0], dtype=torch.int32, device=q.device)
        tiles = torch.tensor(tiles_l or [0, 0, 0, 0], dtype=torch.int32, device=q.device)
        num_decode, num_tiles, max_context = len(rows_l), len(tiles_l) // 4, max(pos_h) + 1
    kstatus = kernel_status(q.device).data_ptr()
    if num_decode:
        scratch = _decode_scratch(q.device, decode_scratch_floats(num_decode, hq, hkv, d, max_context, int(window or 0)))
        _run("sm100", "ti_attention_decode_sink_bf16", out.data_ptr(), q.data_ptr(), kv_cache.data_ptr(),
             scratch.data_ptr(), scratch.numel(), decode_rows.data_ptr(), num_decode, positions.data_ptr(),
             token_seq.data_ptr(), block_table.data_ptr(), block_table.shape[1], hq, hkv, d, page_size,
             num_pages, float(scale), int(window or 0), int(max_context), has_sink, sink_v, float(out_scale), *extras,
             kstatus, _stream())
    def one_tile_kernel(first: int, count: int, halves: int) -> None:
        # Few query tiles behind a long prefix: the keys are shared out over CTAs too (at least 1,024 to a CTA),
        # so that most SMs have a CTA; their partial results meet in a merge kernel.
        ctas = count * (2 if halves else 1) * hq
        splits = 1
        if ctas * 2 <= KEY_SPLIT_MAX_CTAS and max_context >= 2048:
            splits = max(1, min(KEY_SPLIT_MAX_CTAS // ctas, int(max_context) // 1024))
        split_keys = -(-(-(-int(max_context) // splits)) // 128) * 128 if splits > 1 else 0
        scratch_ptr, scratch_floats = None, 0
        if splits > 1:
            scratch = _decode_scratch(q.device, count * (2 if halves else 1) * splits * hq * 128 * (d + 2))
            scratch_ptr, scratch_floats = scratch.data_ptr(), scratch.numel()
        _run("sm100", "ti_attention_prefill_tc_sink_bf16", out.data_ptr(), q.data_ptr(), kv_cache.data_ptr(),
             tiles.data_ptr() + 16 * first, count, t, block_table.data_ptr(), block_table.shape[1], hq, hkv, d, page_size,
             num_pages, float(scale), int(window or 0), halves, splits, split_keys, scratch_ptr, scratch_floats, has_sink,
             sink_v, float(out_scale), *extras, kstatus, _stream())

    if num_pairs * hq >= PAIR_MIN_CTAS:             # two query tiles a CTA
        _run("sm100", "ti_attention_prefill_pair_sink_bf16", out.data_ptr(), q.data_ptr(), kv_cache.data_ptr(),
             tiles.data_ptr(), num_pairs, t, block_table.data_ptr(), block_table.shape[1], hq, hkv, d, page_size,
             num_pages, float(scale), int(window or 0), has_sink, sink_v, float(out_scale), *extras, kstatus, _stream())
    elif num_pairs:                                 # too few of them to fill the machine: one query tile a CTA
        one_tile_kernel(0, num_pairs, 1)
    if num_tiles > num_pairs:                       # ends of portions of at most 128 rows
        one_tile_kernel(num_pairs, num_tiles - num_pairs, 0)
    return out


# ---------------------------------------------------------------------- a float32 residual stream
def embedding_scaled(token_ids: torch.Tensor, table: torch.Tensor, scale: float):
    """(x32, copy): float32 rows ``table[token_ids] * scale`` and their rounding in the table's dtype
    (``copy`` is x32 itself for a float32 table)."""
    _check(token_ids, "token_ids", torch.int32, 1)
    _check(table, "table", None, 2)
    t, hidden = token_ids.shape[0], table.shape[1]
    x32 = torch.empty((t, hidden), dtype=torch.float32, device=table.device)
    copy = None if table.dtype == torch.float32 else torch.empty((t, hidden), dtype=table.dtype, device=table.device)
    _run("latent", "ti_embedding_scaled", x32.data_ptr(), _ptr(copy), table.data_ptr(), token_ids.data_ptr(), t, hidden,
         table.shape[0], float(scale), _dtype_code(table), _stream())
    return x32, (x32 if copy is None else copy)


def norm_add(x32: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float, copy_dtype: torch.dtype):
    """x32 += weight * y * rsqrt(mean(y^2) + eps) in place (float32 [T, size]); returns (x32, copy) with the
    rounding of the new rows in ``copy_dtype`` (x32 itself for float32). ``y``: float32 or ``copy_dtype``."""
    _check(x32, "x32", torch.float32, 2)
    _check(y, "y", None, 2)
    _check(weight, "weight", torch.float32, 1)
    if y.shape != x32.shape or weight.shape[0] != x32.shape[1]:
        raise KernelError("norm_add: shapes differ")
    if y.dtype not in (torch.float32, copy_dtype):
        raise KernelError(f"norm_add: y is {y.dtype}, the stream's copy {copy_dtype}")
    copy = None if copy_dtype == torch.float32 else torch.empty(x32.shape, dtype=copy_dtype, device=x32.device)
    _run("latent", "ti_norm_add", x32.data_ptr(), _ptr(copy), y.data_ptr(), weight.data_ptr(), x32.shape[0], x32.shape[1],
         float(eps), _dtype_code(y), 0 if copy is None else _dtype_code(copy), _stream())
    return x32, (x32 if copy is None else copy)


def rmsnorm_rows32(x32: torch.Tensor, weight: torch.Tensor, eps: float, rows: Optional[torch.Tensor],
                   out_dtype: torch.dtype) -> torch.Tensor:
    """RMSNorm of float32 rows (all, or those ``rows`` int32 [N] picks), stored in ``out_dtype``."""
    _check(x32, "x32", torch.float32, 2)
    _check(weight, "weight", torch.float32, 1)
    if rows is not None:
        _check(rows, "rows", torch.int32, 1)
    n = x32.shape[0] if rows is None else rows.shape[0]
    out = torch.empty((n, x32.shape[1]), dtype=out_dtype, device=x32.device)
    _run("latent", "ti_rmsnorm_rows32", out.data_ptr(), x32.data_ptr(), weight.data_ptr(), _ptr(rows), n, x32.shape[1],
         float(eps), _dtype_code(out), _stream())
    return out


def relu_squared(x: torch.Tensor) -> torch.Tensor:
    """max(x, 0)^2, one rounding."""
    _check(x, "x")
    out = torch.empty_like(x)
    _run("latent", "ti_relu_squared", out.data_ptr(), x.data_ptr(), x.numel(), _dtype_code(x), _stream())
    return out


def batched_linear(x: torch.Tensor, w: torch.Tensor, *, x_offset: int = 0, x_batch_stride: int, k: int,
                   out: Optional[torch.Tensor] = None, out_offset: int = 0, out_batch_stride: Optional[int] = None,
                   bias: Optional[torch.Tensor] = None, sigmoid: bool = False, out_float32: bool = False,
                   gate: Optional[torch.Tensor] = None, gate_offset: int = 0) -> torch.Tensor:
    """For every batch b of ``w`` [B, N, K]: out[:, b-th piece] = act(x[:, b-th piece] . w[b]^T + bias[b]).
    ``gate`` [M, cols] of x's dtype: batch b's result is also multiplied by sigmoid(gate[:, gate_offset + b * N + n]).
    ``x`` [M, row] holds the batches side by side in each row: piece b starts at column
    ``x_offset + b * x_batch_stride`` and has ``k`` columns; likewise ``out`` [M, row_out] (made here as
    [M, B * N] if not given) with ``out_offset`` and ``out_batch_stride`` (default N). float32 accumulation."""
    _check(x, "x", None, 2)
    _check(w, "w", x.dtype, 3)
    batch, n, kw = w.shape
    if kw != k:
        raise KernelError(f"batched_linear: w has {kw} columns, the pieces of x {k}")
    m = x.shape[0]
    if x_offset + (batch - 1) * x_batch_stride + k > x.shape[1]:
        raise KernelError("batched_linear: the pieces do not fit the rows of x")
    if out_batch_stride is None:
        out_batch_stride = n
    if out is None:
        out = torch.empty((m, out_offset + batch * out_batch_stride), device=x.device,
                          dtype=torch.float32 if out_float32 else x.dtype)
    _check(out, "out", None, 2)
    if out.dtype not in (torch.float32, x.dtype):
        raise KernelError(f"batched_linear: out must be float32 or {x.dtype}, got {out.dtype}")
    if out.shape[0] != m or out_offset + (batch - 1) * out_batch_stride + n > out.shape[1]:
        raise KernelError("batched_linear: the pieces do not fit the rows of out")
    if bias is not None:
        _check(bias, "bias", torch.float32, 2)
        if tuple(bias.shape) != (batch, n):
            raise KernelError("batched_linear: bias must be [B, N]")
    if gate is not None:
        _check(gate, "gate", x.dtype, 2)
        if gate.shape[0] != m or gate_offset < 0 or gate_offset + batch * n > gate.shape[1]:
            raise KernelError("batched_linear: the gate holds one column per output for every row")
    isz_x, isz_o = x.element_size(), out.element_size()
    _run("latent", "ti_gemm_batched", out.data_ptr() + out_offset * isz_o, x.data_ptr() + x_offset * isz_x, w.data_ptr(),
         _ptr(bias), batch, m, n, k, x.shape[1], x_batch_stride, k, n * k, out.shape[1], out_batch_stride, n,
         int(sigmoid), int(out.dtype == torch.float32 and x.dtype != torch.float32),
         gate.data_ptr() + gate_offset * isz_x if gate is not None else None, gate.shape[1] if gate is not None else 0, n,
         _dtype_code(x), _stream())
    return out


# ---------------------------------------------------------------------- attention over a cached latent
def _rotation_args(rot: Optional[Rotation]):
    if rot is None:
        return None, None, 0, 0, 0, 1.0
    _check(rot.inv_freq if rot.inv_freq is not None else rot.cos_sin, "the rotation's tensor")
    return (_ptr(rot.inv_freq), _ptr(rot.cos_sin), rot.cos_sin.shape[0] if rot.cos_sin is not None else 0,
            int(rot.interleaved), rot.rotary_dim, float(rot.factor))


def latent_prepare(down: torch.Tensor, *, q_rank: int, rank: int, rot: int, q_norm_weight: Optional[torch.Tensor],
                   kv_norm_weight: Optional[torch.Tensor], eps: float, rotation: Optional[Rotation],
                   positions: torch.Tensor, token_seq: torch.Tensor, cache: Optional[torch.Tensor],
                   block_table: torch.Tensor, dtype: torch.dtype, status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``down`` float32 [T, q_rank (+ rank + rot)]: a token's down projections [query latent | kv latent | keys to
    rotate]. Returns the normed query latent [T, q_rank] in ``dtype`` and, if ``cache`` ([1, pages, 1, page,
    rank + rot], ``dtype``) is given, writes the token's row [normed kv latent | rotated keys] there. ``q_rank`` 0: the
    queries have no latent of their own (nothing is returned)."""
    _check(down, "down", torch.float32, 2)
    if q_rank:
        _check(q_norm_weight, "q_norm_weight", torch.float32, 1)
    _check(positions, "positions", torch.int32, 1)
    _check(token_seq, "token_seq", torch.int32, 1)
    t = down.shape[0]
    need = q_rank + (rank + rot if cache is not None else 0)
    if down.shape[1] < need:
        raise KernelError(f"latent_prepare: rows of {down.shape[1]} features, {need} are needed")
    page_size = num_pages = 1
    max_blocks = 0
    if cache is not None:
        _check(cache, "cache", dtype, 5)
        _check(kv_norm_weight, "kv_norm_weight", torch.float32, 1)
        _check(block_table, "block_table", torch.int32, 2)
        if cache.shape[0] != 1 or cache.shape[2] != 1 or cache.shape[4] != rank + rot:
            raise KernelError(f"latent cache shape {tuple(cache.shape)} is not [1, pages, 1, page, {rank + rot}]")
        num_pages, page_size, max_blocks = cache.shape[1], cache.shape[3], block_table.shape[1]
    out = torch.empty((t, q_rank), dtype=dtype, device=down.device) if q_rank else None
    _run("latent", "ti_latent_prepare", _ptr(out), _ptr(cache), down.data_ptr(), down.shape[1],
         _ptr(q_norm_weight) if q_rank else None, _ptr(kv_norm_weight), float(eps), q_rank, rank, rot, *_rotation_args(rotation),
         positions.data_ptr(), token_seq.data_ptr(), _ptr(block_table) if cache is not None else None, max_blocks, t,
         page_size, num_pages, _ptr(status), 0 if dtype == torch.float32 else 1, _stream())
    return out


def latent_query_rotate(rows: torch.Tensor, q: torch.Tensor, *, heads: int, plain: int, rot: int, rank: int,
                        rotation: Optional[Rotation], positions: torch.Tensor) -> None:
    """Writes the rotated last ``rot`` features of every head of ``q`` [T, heads * (plain + rot) (+ columns not read)] into
    ``rows`` float32 [T, heads * (rank + rot)], behind each head's first ``rank`` features."""
    _check(rows, "rows", torch.float32, 2)
    _check(q, "q", None, 2)
    _check(positions, "positions", torch.int32, 1)
    if q.shape[1] < heads * (plain + rot) or rows.shape[1] != heads * (rank + rot) or rows.shape[0] != q.shape[0]:
        raise KernelError("latent_query_rotate: widths do not match the head sizes")
    _run("latent", "ti_latent_query", rows.data_ptr(), q.data_ptr(), q.shape[1], q.shape[0], heads, plain, rot, rank,
         *_rotation_args(rotation), positions.data_ptr(), _dtype_code(q), _stream())


LATENT_SPLIT_MIN_KEYS = 128     # a split of the keys over blocks gets at least this many
LATENT_TARGET_BLOCKS = 296      # enough blocks to have two on every SM


def latent_attention(q_rows: torch.Tensor, cache: torch.Tensor, *, heads: int, rank: int, rot: int, scale: float,
                     sink: Optional[torch.Tensor], positions: torch.Tensor, token_seq: torch.Tensor,
                     block_table: torch.Tensor, max_context: int, window: Optional[int] = None, step=None,
                     status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of query rows float32 [T, heads * (rank + rot)] over each token's own request's cached
    rows [c | k_rot] (``cache`` [1, pages, 1, page, rank + rot]); returns sum_j p_j c_j per head, [T, heads * rank]
    in the cache's dtype. ``sink`` float32 [heads]: exp(sink) joins every softmax denominator. ``max_context``
    (a host number, the longest context of the step) only decides over how many blocks the keys are shared.
    ``step`` (the StepContext): with it a bfloat16 cache whose rows are a multiple of 8 features runs on the
    tensor cores, prompt portions and decoded tokens in their own forms; without it, or in float32, the
    float32-arithmetic kernel runs. ``window``: a query sees only the last so many keys, itself included."""
    _check(q_rows, "q_rows", torch.float32, 2)
    _check(cache, "cache", None, 5)
    _check(positions, "positions", torch.int32, 1)
    _check(token_seq, "token_seq", torch.int32, 1)
    _check(block_table, "block_table", torch.int32, 2)
    if sink is not None:
        _check(sink, "sink", torch.float32, 1)
        if sink.shape[0] != heads:
            raise KernelError("latent_attention: one sink per head")
    t = q_rows.shape[0]
    if q_rows.shape[1] != heads * (rank + rot) or cache.shape[4] != rank + rot or cache.shape[0] != 1 or cache.shape[2] != 1:
        raise KernelError("latent_attention: the query rows or the cache do not match rank and rot")
    out = torch.empty((t, heads * rank), dtype=cache.dtype, device=cache.device)
    if t == 0:
        return out

    reach = min(int(max_context), int(window)) if window else int(max_context)     # keys a query can see at most

    def share_out(blocks: int, least: int = LATENT_SPLIT_MIN_KEYS) -> int:
        if blocks < LATENT_TARGET_BLOCKS and reach >= 2 * least:
            return max(1, min(-(-LATENT_TARGET_BLOCKS // blocks), reach // least, 64))
        return 1

    def scratch(splits: int):
        if splits == 1:
            return None, 0
        parts = _decode_scratch(cache.device, t * heads * splits * (rank + 2))
        return parts, parts.numel()

    if (step is not None and cache.dtype == torch.bfloat16
            and int(_fn("latent", "ti_latent_attend_mma_ok")(rank, rot))):
        decode = step.max_q_len == 1
        rows = 16 if decode else 32
        per_block = min(heads, rows)
        tokens_per_block = 1 if decode else max(1, rows // per_block)
        splits = share_out(-(-t // tokens_per_block) * -(-heads // per_block), 64 if decode else LATENT_SPLIT_MIN_KEYS)
        parts, parts_floats = scratch(splits)
        _run("latent", "ti_latent_attend_mma", out.data_ptr(), _ptr(parts), parts_floats, q_rows.data_ptr(), cache.data_ptr(),
             _ptr(sink), positions.data_ptr(), token_seq.data_ptr(), step.cu_seqlens.data_ptr(), block_table.data_ptr(),
             block_table.shape[1], step.num_seqs, t, heads, rank, rot, cache.shape[3], cache.shape[1], float(scale),
             int(window or 0), splits, int(decode), _ptr(status), _stream())
        if splits > 1:
            _run("latent", "ti_latent_merge", out.data_ptr(), parts.data_ptr(), _ptr(sink), t, heads, rank, splits,
                 _dtype_code(cache), _stream())
        return out
    splits = share_out(t * ((heads + 7) // 8))
    parts, parts_floats = scratch(splits)
    _run("latent", "ti_latent_attend", out.data_ptr(), _ptr(parts), parts_floats, q_rows.data_ptr(), cache.data_ptr(),
         _ptr(sink), positions.data_ptr(), token_seq.data_ptr(), block_table.data_ptr(), block_table.shape[1], t, heads,
         rank, rot, cache.shape[3], cache.shape[1], float(scale), int(window or 0), splits, _ptr(status),
         _dtype_code(cache), _stream())
    return out


# ---------------------------------------------------------------------- gated linear recurrence
def causal_conv(x: torch.Tensor, *, offset: int, width: int, state: torch.Tensor, weight: torch.Tensor,
                bias: Optional[torch.Tensor], token_seq: torch.Tensor, cu_seqlens: torch.Tensor,
                state_slots: torch.Tensor) -> torch.Tensor:
    """Per-channel causal convolution of columns [offset, offset + width) of ``x`` [T, row]: ``weight`` float32
    [width, taps], last column the current token's. Inputs from before the step come from ``state`` float32
    [slots, taps, width] (rows 1.. of a slot: the last taps - 1 inputs, oldest first). Returns [T, width]."""
    _check(x, "x", None, 2)
    _check(state, "state", torch.float32, 3)
    _check(weight, "weight", torch.float32, 2)
    taps = weight.shape[1]
    if weight.shape[0] != width or state.shape[1] != taps or state.shape[2] != width or offset + width > x.shape[1]:
        raise KernelError("causal_conv: shapes do not match")
    if bias is not None:
        _check(bias, "bias", torch.float32, 1)
    out = torch.empty((x.shape[0], width), dtype=x.dtype, device=x.device)
    _run("latent", "ti_causal_conv", out.data_ptr(), x.data_ptr(), x.shape[1], offset, state.data_ptr(), weight.data_ptr(),
         _ptr(bias), token_seq.data_ptr(), cu_seqlens.data_ptr(), state_slots.data_ptr(), x.shape[0], width, taps,
         _dtype_code(x), _stream())
    return out


def gated_scan(u: torch.Tensor, gates: torch.Tensor, yx: torch.Tensor, *, y_offset: int, x_offset: int,
               state: torch.Tensor, lam: torch.Tensor, block_width: int, decay: float, cu_seqlens: torch.Tensor,
               state_slots: torch.Tensor, num_seqs: int) -> torch.Tensor:
    """The recurrence S <- a S + sqrt(1 - a^2) (i u), a = exp(-decay r softplus(lam)), over every request's tokens
    of the step in order, from and back into ``state`` float32 [slots, taps, width] (row 0: S; the rows behind it
    take the convolution's newest inputs, columns [x_offset, +width) of ``yx``). ``gates`` float32 [T, 2 width],
    per block [r | i]. Returns S * gelu_tanh(y) with y = columns [y_offset, +width) of ``yx``, [T, width]."""
    _check(u, "u", None, 2)
    _check(gates, "gates", torch.float32, 2)
    _check(yx, "yx", u.dtype, 2)
    _check(state, "state", torch.float32, 3)
    _check(lam, "lam", torch.float32, 1)
    t, width = u.shape
    if gates.shape != (t, 2 * width) or yx.shape[0] != t or state.shape[2] != width or lam.shape[0] != width:
        raise KernelError("gated_scan: shapes do not match")
    out = torch.empty((t, width), dtype=u.dtype, device=u.device)
    _run("latent", "ti_gated_scan", out.data_ptr(), state.data_ptr(), u.data_ptr(), gates.data_ptr(), yx.data_ptr(),
         yx.shape[1], y_offset, x_offset, lam.data_ptr(), cu_seqlens.data_ptr(), state_slots.data_ptr(), num_seqs, t, width,
         block_width, state.shape[1], float(decay), _dtype_code(u), _stream())
    return out


# ---------------------------------------------------------------------- routed experts
class ExpertRouting:
    """Where a step's tokens go: ``chosen`` int32 [T, top], ``weight`` float32 [T, top], ``slot_of`` int32 [T, top]
    (row of each (token, choice) in the order sorted by expert), ``token_of`` int32 [T * top], and the row tiles
    ``tiles`` int32 [max_tiles, 3] = [expert, first row, rows] with their count ``num_tiles`` int32 [1] (on the
    device: the grouped products are launched for ``max_tiles`` and the surplus returns at once). ``slot_weight``
    float32 [T * top]: the weights in the sorted order (row ``slot_of[t, c]`` holds ``weight[t, c]``)."""

    def __init__(self, chosen, weight, slot_of, token_of, tiles, num_tiles, max_tiles, counts, tile_rows, slot_weight=None):
        self.chosen, self.weight, self.slot_of, self.token_of = chosen, weight, slot_of, token_of
        self.tiles, self.num_tiles, self.max_tiles, self.counts = tiles, num_tiles, max_tiles, counts
        self.tile_rows, self.slot_weight = tile_rows, slot_weight


def route_experts(x32: torch.Tensor, w_router: torch.Tensor, top: int, weight_eps: float,
                  wide_tiles: bool = False, tile_rows: int = 0, *, correction: Optional[torch.Tensor] = None,
                  renormalize: bool = True, real_experts: Optional[int] = None, scoring: str = "softmax") -> ExpertRouting:
    """Router of a mixture of experts: float32 logits from the rows ``x32`` [T, H] (float32, or the router's dtype)
    and ``w_router`` [E, H], softmax over all experts, the ``top`` largest (first index on ties), weights = their
    scores over their sum (+ ``weight_eps``). ``correction`` float32 [E]: the choice goes by score + correction, the
    weights stay the plain scores; ``renormalize`` False: the weights are the scores themselves; ``real_experts``:
    only the first so many router outputs are experts with weights, the rest stand for identity experts (rows, but
    no tiles in the plan). ``scoring`` 'sigmoid': an expert's score is the sigmoid of its own logit instead of the
    softmax over all. ``wide_tiles``: the row tiles of the plan hold 64 rows instead of 32 (for steps that bring
    an expert many rows; only the tensor-core grouped product takes them, see ``expert_tiles_may_be_wide``);
    ``tile_rows``: any other height the caller has settled with the grouped product (``expert_tile_rows``)."""
    _check(x32, "x32", None, 2)
    _check(w_router, "w_router", None, 2)
    if x32.dtype not in (torch.float32, w_router.dtype):
        raise KernelError("route_experts: the rows are float32 or of the router's dtype")
    t, hidden = x32.shape
    experts = w_router.shape[0]
    if w_router.shape[1] != hidden:
        raise KernelError("route_experts: the router's rows do not match the stream's")
    if correction is not None:
        _check(correction, "correction", torch.float32, 1)
        if correction.shape[0] != experts:
            raise KernelError("route_experts: one correction per router output")
    real = experts if real_experts is None else int(real_experts)
    if scoring not in ("softmax", "sigmoid"):
        raise KernelError(f"route_experts: unknown scoring {scoring!r}")
    dev = x32.device
    tile_rows = tile_rows or (64 if wide_tiles else int(_fn("experts", "ti_moe_tile_rows")()))
    max_tiles = (t * top + tile_rows - 1) // tile_rows + experts
    ints = torch.empty(t * top * 4 + experts + (experts + 1) + 3 * max_tiles + 1, dtype=torch.int32, device=dev)
    n = t * top
    chosen, rank, slot_of, token_of = (ints[i * n:(i + 1) * n] for i in range(4))
    o = 4 * n
    counts, starts = ints[o:o + experts], ints[o + experts:o + 2 * experts + 1]
    o += 2 * experts + 1
    tiles, num_tiles = ints[o:o + 3 * max_tiles], ints[o + 3 * max_tiles:o + 3 * max_tiles + 1]
    both = torch.empty((2, t, top), dtype=torch.float32, device=dev)
    weight, slot_weight = both[0], both[1].view(-1)
    _run("experts", "ti_moe_route", chosen.data_ptr(), weight.data_ptr(), rank.data_ptr(), counts.data_ptr(),
         starts.data_ptr(), tiles.data_ptr(), num_tiles.data_ptr(), slot_of.data_ptr(), token_of.data_ptr(),
         x32.data_ptr(), w_router.data_ptr(), t, hidden, experts, top, float(weight_eps), _ptr(correction),
         int(renormalize), real, tile_rows, max_tiles, int(scoring == "sigmoid"), slot_weight.data_ptr(), _dtype_code(x32),
         _dtype_code(w_router), _stream())
    return ExpertRouting(chosen.view(t, top), weight, slot_of.view(t, top), token_of, tiles.view(max_tiles, 3),
                         num_tiles, max_tiles, counts, tile_rows, slot_weight)


def expert_tiles_may_be_wide(x: torch.Tensor, *inner_sizes: int) -> bool:
    """True if the grouped products of ``x`` [T, K] (and of rows of the given other sizes) run on the tensor cores,
    which alone take row tiles of 64."""
    return all(int(_fn("experts", "ti_moe_wide_tiles_ok")(k, _dtype_code(x))) for k in (x.shape[1],) + inner_sizes)


EXPERT_TCGEN05_MIN_ROWS = 96     # rows an expert gets on average from which the tcgen05 grouped product is used


def expert_tile_rows(x: torch.Tensor, num_experts: int, top: int, *inner_sizes: int) -> int:
    """The height of the row tiles that the grouped products of a step should be planned with: 128 (tcgen05: many
    rows an expert, bfloat16, whole k blocks of 64), 64 or 32 (the warp-level tensor-core tiles; 32 also float32)."""
    t = x.shape[0]
    if x.dtype == torch.bfloat16 and t * top >= EXPERT_TCGEN05_MIN_ROWS * num_experts:
        ok = _fn("sm100", "ti_moe_gemm_tcgen05_ok")
        if all(int(ok(t * top, num_experts, n, k)) for n, k in ((inner_sizes[0], x.shape[1]), (x.shape[1], inner_sizes[0]))):
            return int(_fn("sm100", "ti_moe_tcgen05_tile_rows")())
    if t * top >= 48 * num_experts and expert_tiles_may_be_wide(x, *inner_sizes):
        return 64
    return int(_fn("experts", "ti_moe_tile_rows")())


def expert_linear(x: torch.Tensor, w: torch.Tensor, routing: ExpertRouting, *, up: bool, activation: bool = True) -> torch.Tensor:
    """Grouped product over the routing's row tiles with ``w`` [E, N, K]. ``up``: ``x`` [T, K] are the step's
    tokens, gathered per expert; the result [T * top, N] (sorted rows) has passed max(v, 0)^2 (``activation``
    False: it is stored as it is, for an activation that is a kernel of its own). Otherwise ``x``
    are sorted rows [T * top, K] and the result is float32 [T * top, N]."""
    _check(x, "x", None, 2)
    _check(w, "w", x.dtype, 3)
    _, n, k = w.shape
    if x.shape[1] != k:
        raise KernelError("expert_linear: x and w do not match")
    slots = routing.token_of.shape[0]
    out = torch.empty((slots, n), dtype=x.dtype if up else torch.float32, device=x.device)
    form = (1 if activation else 2) if up else 0
    if routing.tile_rows == 128:                 # tcgen05: tiled operand copies want the rows in expert order
        rows = x
        if up:
            rows = torch.empty((slots, k), dtype=x.dtype, device=x.device)
            _run("experts", "ti_moe_gather", rows.data_ptr(), x.data_ptr(), routing.token_of.data_ptr(), slots, k,
                 _dtype_code(x), _stream())
        _run("sm100", "ti_moe_gemm_tcgen05", out.data_ptr(), rows.data_ptr(), w.data_ptr(), routing.tiles.data_ptr(),
             routing.num_tiles.data_ptr(), slots, w.shape[0], n, k, routing.max_tiles, form,
             kernel_status(x.device).data_ptr(), _stream())
        return out
    _run("experts", "ti_moe_gemm", out.data_ptr(), x.data_ptr(), w.data_ptr(), routing.tiles.data_ptr(),
         routing.num_tiles.data_ptr(), routing.token_of.data_ptr(), n, k, routing.max_tiles, routing.tile_rows, form,
         _dtype_code(x), _stream())
    return out


def experts_combine_norm_add(x32: torch.Tensor, down: torch.Tensor, shared_out: Optional[torch.Tensor],
                             routing: ExpertRouting, norm_weight: torch.Tensor, eps: float, copy_dtype: torch.dtype):
    """y = sum_k weight_k * down[slot_k] (+ shared_out), then x32 += norm_weight * y * rsqrt(mean(y^2) + eps) in
    place; returns (x32, copy) as ``norm_add`` does."""
    _check(x32, "x32", torch.float32, 2)
    _check(down, "down", torch.float32, 2)
    _check(norm_weight, "norm_weight", torch.float32, 1)
    if shared_out is not None:
        _check(shared_out, "shared_out", copy_dtype, 2)
    t, size = x32.shape
    copy = None if copy_dtype == torch.float32 else torch.empty((t, size), dtype=copy_dtype, device=x32.device)
    _run("experts", "ti_moe_combine_norm_add", x32.data_ptr(), _ptr(copy), down.data_ptr(), _ptr(shared_out),
         routing.slot_of.data_ptr(), routing.weight.data_ptr(), norm_weight.data_ptr(), t, size,
         routing.chosen.shape[1], float(eps), 0 if copy is None else _dtype_code(copy), _stream())
    return x32, (x32 if copy is None else copy)


# ---------------------------------------------------------------------- several residual streams
def clamped_glu(gate_up: torch.Tensor, limit: float, alpha: float) -> torch.Tensor:
    """The gated activation of an expert on its stored product ``gate_up`` [rows, 2 F] = [gate | up]:
    g = min(gate, limit), u = clamp(up, -limit, limit), out = g * sigmoid(alpha * g) * (u + 1), [rows, F]; float32
    arithmetic, one rounding."""
    _check(gate_up, "gate_up", None, 2)
    rows, two_f = gate_up.shape
    if two_f % 2:
        raise KernelError("clamped_glu: a row holds a gate half and an up half")
    out = torch.empty((rows, two_f // 2), dtype=gate_up.dtype, device=gate_up.device)
    _run("experts", "ti_moe_clamped_glu", out.data_ptr(), gate_up.data_ptr(), rows, two_f // 2, float(limit), float(alpha),
         _dtype_code(gate_up), _stream())
    return out


def silu_glu(gate_up: torch.Tensor, row_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """silu(gate) * up on a stored product ``gate_up`` [rows, 2 F] = [gate | up] -> [rows, F]; float32 arithmetic, one
    rounding. ``row_scale`` float32 [rows]: both halves of a row are multiplied by its number first, silu(s gate) * (s up):
    for experts that are weighted at their input, since W (s h) = s (W h) (``ExpertRouting.slot_weight``)."""
    _check(gate_up, "gate_up", None, 2)
    rows, two_f = gate_up.shape
    if two_f % 2:
        raise KernelError("silu_glu: a row holds a gate half and an up half")
    if row_scale is not None:
        _check(row_scale, "row_scale", torch.float32, 1)
        if row_scale.shape[0] != rows:
            raise KernelError("silu_glu: one number per row")
    out = torch.empty((rows, two_f // 2), dtype=gate_up.dtype, device=gate_up.device)
    _run("experts", "ti_moe_silu_glu", out.data_ptr(), gate_up.data_ptr(), rows, two_f // 2, _ptr(row_scale),
         _dtype_code(gate_up), _stream())
    return out


def experts_combine(down: torch.Tensor, x: torch.Tensor, routing: ExpertRouting, real_experts: int,
                    weighted: bool = True) -> torch.Tensor:
    """out[t] = sum_c weight[t, c] * (down[slot_of[t, c]] if chosen[t, c] < real_experts else x[t]) in choice order:
    the weighted sum of the chosen experts' outputs (float32 sorted rows ``down``), an identity expert's output being
    the token's own row of ``x`` [T, H]. Float32 sums, one rounding to x's dtype. ``weighted`` False: every weight is
    one (the experts were weighted at their input)."""
    _check(down, "down", torch.float32, 2)
    _check(x, "x", None, 2)
    t, size = x.shape
    if down.shape[1] != size or routing.chosen.shape[0] != t:
        raise KernelError("experts_combine: the rows do not fit the routing")
    out = torch.empty_like(x)
    _run("experts", "ti_moe_combine", out.data_ptr(), down.data_ptr(), x.data_ptr(), routing.chosen.data_ptr(),
         routing.slot_of.data_ptr(), routing.weight.data_ptr() if weighted else None, t, size, routing.chosen.shape[1],
         int(real_experts), _dtype_code(x), _stream())
    return out


def streams_embed(token_ids: torch.Tensor, table: torch.Tensor, streams: int, scale: float = 1.0) -> torch.Tensor:
    """float32 [streams, T, width]: every stream starts as the rows ``table[token_ids]`` times ``scale``."""
    _check(token_ids, "token_ids", torch.int32, 1)
    _check(table, "table", None, 2)
    t, width = token_ids.shape[0], table.shape[1]
    out = torch.empty((streams, t, width), dtype=torch.float32, device=table.device)
    _run("hybrid", "ti_streams_embed", out.data_ptr(), table.data_ptr(), token_ids.data_ptr(), t, width, table.shape[0],
         streams, float(scale), _dtype_code(table), _stream())
    return out


class StreamUpdate:
    """What a sublayer leaves for the streams, applied by the next ``streams_step``:
    X[t] <- sum_s mix[s, t] X[s] + out[t] * y (``mix`` float32 [S, S] indexed [from, to], ``out`` float32 [S])."""

    def __init__(self, y: torch.Tensor, mix: torch.Tensor, out: torch.Tensor,
                 norm_weight: Optional[torch.Tensor] = None, norm_eps: float = 0.0):
        self.y, self.mix, self.out = y, mix, out
        # a norm on the sublayer's OUTPUT: y is replaced by norm_weight * y * rsqrt(mean(y^2) + norm_eps) as it is applied
        self.norm_weight, self.norm_eps = norm_weight, float(norm_eps)


def streams_step(x: torch.Tensor, pending: Optional[StreamUpdate], read_in: Optional[torch.Tensor],
                 norm_weight: Optional[torch.Tensor], eps: float, out_dtype: torch.dtype,
                 rows: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """One kernel between two sublayers of a model whose residual is several float32 streams ``x`` [S, T, W]:
    applies ``pending`` in place (if any), then returns h = norm_weight * u * rsqrt(mean(u^2) + eps) in ``out_dtype``
    with u = sum_s read_in[s] x[s] (if ``read_in`` is given; else None). ``rows`` int32 [N]: only these tokens are
    worked on (h then has N rows): for the rows whose logits are wanted, at the very end."""
    _check(x, "x", torch.float32, 3)
    s, t, width = x.shape
    y = None
    if pending is not None:
        y = _check(pending.y, "y", None, 2)
        _check(pending.mix, "mix", torch.float32, 2)
        _check(pending.out, "out", torch.float32, 1)
        if tuple(y.shape) != (t, width) or tuple(pending.mix.shape) != (s, s) or pending.out.shape[0] != s:
            raise KernelError("streams_step: the update does not fit the streams")
        if pending.norm_weight is not None:
            _check(pending.norm_weight, "the update's norm weight", torch.float32, 1)
            if pending.norm_weight.shape[0] != width:
                raise KernelError("streams_step: the update's norm does not fit the streams")
    h = None
    n = t if rows is None else _check(rows, "rows", torch.int32, 1).shape[0]
    if read_in is not None:
        _check(read_in, "read_in", torch.float32, 1)
        _check(norm_weight, "norm_weight", torch.float32, 1)
        if read_in.shape[0] != s or norm_weight.shape[0] != width:
            raise KernelError("streams_step: the read coefficients or the norm do not fit the streams")
        h = torch.empty((n, width), dtype=out_dtype, device=x.device)
    _run("hybrid", "ti_streams_step", x.data_ptr(), _ptr(y), _ptr(pending.mix) if pending else None,
         _ptr(pending.out) if pending else None, _ptr(read_in), _ptr(norm_weight), float(eps), _ptr(h), _ptr(rows), n, t,
         width, s, _dtype_code(y) if y is not None else 0, _dtype_code(h) if h is not None else 0,
         _ptr(pending.norm_weight) if pending else None, pending.norm_eps if pending else 0.0, _stream())
    return h


def gelu(x: torch.Tensor, tanh: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """0.5 z (1 + erf(z / sqrt 2)), or the tanh form; float32 arithmetic, one rounding. ``out`` may be ``x``."""
    _check(x, "x")
    if out is None:
        out = torch.empty_like(x)
    _run("hybrid", "ti_gelu", out.data_ptr(), x.data_ptr(), x.numel(), int(tanh), _dtype_code(x), _stream())
    return out


def scale_(x: torch.Tensor, factor: float) -> torch.Tensor:
    """x *= factor in place (float32)."""
    _check(x, "x", torch.float32)
    if factor != 1.0:
        _run("hybrid", "ti_scale", x.data_ptr(), x.numel(), float(factor), _stream())
    return x


def soft_cap_(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x <- cap * tanh(x / cap) in place (float32)."""
    _check(x, "x", torch.float32)
    if not cap > 0:
        raise KernelError("soft_cap_: the cap must be positive")
    _run("hybrid", "ti_soft_cap", x.data_ptr(), x.numel(), float(cap), _stream())
    return x


# ---------------------------------------------------------------------- short convolutions, attention over [k | v] rows
def _slot_stride(state: torch.Tensor, inner: int, name: str) -> int:
    """``state`` float32 [slots, ...]: a slice of the per-request state whose slots lie stride(0) floats apart
    and whose ``inner`` floats of a slot are contiguous."""
    if not isinstance(state, torch.Tensor) or not state.is_cuda or state.dtype != torch.float32:
        raise KernelError(f"{name} must be a float32 CUDA tensor")
    if state[0].numel() != inner or not state[0].is_contiguous():
        raise KernelError(f"{name}: a slot must hold {inner} contiguous floats, got shape {tuple(state.shape)}")
    return state.stride(0)


def short_conv(x: torch.Tensor, *, offset: int, width: int, history: torch.Tensor, weight: torch.Tensor,
               bias: Optional[torch.Tensor], silu: bool, token_seq: torch.Tensor, cu_seqlens: torch.Tensor,
               state_slots: torch.Tensor, shift_history: bool = False) -> torch.Tensor:
    """Causal per-channel convolution over time of columns [offset, offset + width) of ``x`` [T, row], ``weight``
    float32 [taps, width] (tap by tap; the last row meets the current token), then + bias and silu if asked. Inputs of earlier steps
    come from ``history`` float32 [slots, taps - 1, width] (oldest first), which ``conv_state_update`` keeps; in a
    step in which EVERY request brings one token, ``shift_history`` lets this kernel move the histories on itself."""
    _check(x, "x", None, 2)
    _check(weight, "weight", torch.float32, 2)
    taps = weight.shape[0]
    if weight.shape[1] != width or offset + width > x.shape[1]:
        raise KernelError("short_conv: shapes do not match")
    stride = _slot_stride(history, (taps - 1) * width, "history") if taps > 1 else 0
    if bias is not None:
        _check(bias, "bias", torch.float32, 1)
    out = torch.empty((x.shape[0], width), dtype=x.dtype, device=x.device)
    _run("hybrid", "ti_short_conv", out.data_ptr(), x.data_ptr(), x.shape[1], offset, history.data_ptr() if taps > 1 else None,
         stride, weight.data_ptr(), _ptr(bias), token_seq.data_ptr(), cu_seqlens.data_ptr(), state_slots.data_ptr(),
         x.shape[0], width, taps, int(silu), int(shift_history), _dtype_code(x), _stream())
    return out


def conv_state_update(history: torch.Tensor, x: torch.Tensor, *, offset: int, width: int, taps: int,
                      cu_seqlens: torch.Tensor, state_slots: torch.Tensor, num_seqs: int) -> None:
    """The last taps - 1 rows of every request's columns [offset, offset + width) of ``x`` become its ``history``
    (rows of a step shorter than that push the old ones up). Runs after the kernels that read the history."""
    if taps <= 1:
        return
    _check(x, "x", None, 2)
    stride = _slot_stride(history, (taps - 1) * width, "history")
    _run("hybrid", "ti_conv_state_update", history.data_ptr(), stride, x.data_ptr(), x.shape[1], offset,
         cu_seqlens.data_ptr(), state_slots.data_ptr(), num_seqs, width, taps, _dtype_code(x), _stream())


def _kv_planes(cache: torch.Tensor, num_kv_heads: int, head_dim: int, v_dim: int) -> int:
    """1 for a cache of rows [k | v], [1, pages, Hkv, page, d + dv]; 2 for planes [2, pages, Hkv, page, d] (d == dv)."""
    if cache.shape[2] == num_kv_heads:
        if cache.shape[0] == 1 and cache.shape[4] == head_dim + v_dim:
            return 1
        if cache.shape[0] == 2 and cache.shape[4] == head_dim == v_dim:
            return 2
    raise KernelError(f"cache shape {tuple(cache.shape)} is neither [1, pages, {num_kv_heads}, page, {head_dim + v_dim}] "
                      f"nor, for keys and values of one size, [2, pages, {num_kv_heads}, page, {head_dim}]")


def conv_qkv_append(qkv: torch.Tensor, *, num_heads: int, num_kv_heads: int, head_dim: int, v_dim: int,
                    conv_weight: Optional[torch.Tensor], history: Optional[torch.Tensor],
                    temperature: Optional[tuple], positions: torch.Tensor, token_seq: torch.Tensor,
                    cu_seqlens: torch.Tensor, state_slots: torch.Tensor, cache: Optional[torch.Tensor],
                    block_table: torch.Tensor, status: Optional[torch.Tensor] = None,
                    shift_history: bool = False, offset: int = 0) -> torch.Tensor:
    """Columns [offset, offset + Hq d + Hkv (d + dv)) of ``qkv`` [T, row], packed [q | k | v]: a short causal convolution per channel
    (``conv_weight`` float32 [taps, channels], tap by tap, with ``history`` float32 [slots, taps - 1, channels]; None: none),
    then q times its position's temperature 1 + coef * ln(floor((p + 1) / every) + 1) (``temperature`` =
    (coef, every) or None). Returns q [T, Hq, d]; k and v go to the token's row [k | v] of ``cache``
    [1, pages, Hkv, page, d + dv], or, where d == dv, to the planes of a cache [2, pages, Hkv, page, d].
    ``shift_history``: as in ``short_conv``."""
    _check(qkv, "qkv", None, 2)
    t = qkv.shape[0]
    width = num_heads * head_dim + num_kv_heads * (head_dim + v_dim)
    if offset < 0 or offset + width > qkv.shape[1]:
        raise KernelError("conv_qkv_append: the packed rows do not fit the rows they lie in")
    taps, stride = 1, 0
    if conv_weight is not None:
        _check(conv_weight, "conv_weight", torch.float32, 2)
        taps = conv_weight.shape[0]
        if conv_weight.shape[1] != width:
            raise KernelError("conv_qkv_append: every tap has a weight per packed channel")
        if taps > 1:
            stride = _slot_stride(history, (taps - 1) * width, "history")
    _check(positions, "positions", torch.int32, 1)
    _check(block_table, "block_table", torch.int32, 2)
    page_size = num_pages = planes = 1
    if cache is not None:
        _check(cache, "cache", qkv.dtype, 5)
        planes = _kv_planes(cache, num_kv_heads, head_dim, v_dim)
        num_pages, page_size = cache.shape[1], cache.shape[3]
    coef, every = (float(temperature[0]), int(temperature[1])) if temperature else (0.0, 0)
    q = torch.empty((t, num_heads, head_dim), dtype=qkv.dtype, device=qkv.device)
    _run("hybrid", "ti_conv_qkv_append", q.data_ptr(), _ptr(cache), qkv.data_ptr(), qkv.shape[1], offset,
         history.data_ptr() if taps > 1 else None,
         stride, _ptr(conv_weight), taps, coef, every, positions.data_ptr(), token_seq.data_ptr(), cu_seqlens.data_ptr(),
         state_slots.data_ptr(), block_table.data_ptr(), block_table.shape[1], t, num_heads, num_kv_heads, head_dim, v_dim,
         page_size, num_pages, planes, int(shift_history), _ptr(status), _dtype_code(qkv), _stream())
    return q


def _check_head_extras(q, head_sinks, gate, gate_offset) -> None:
    t, hq, _ = q.shape
    if head_sinks is not None:
        _check(head_sinks, "head_sinks", torch.float32, 1)
        if head_sinks.shape[0] != hq:
            raise KernelError("attention: one sink per query head")
    if gate is not None:
        _check(gate, "gate", q.dtype, 2)
        if gate.shape[0] != t or gate_offset < 0 or gate_offset + hq > gate.shape[1]:
            raise KernelError("attention: the gate holds one column per query head for every token")


def attention_rows(q: torch.Tensor, cache: torch.Tensor, *, v_dim: int, positions: torch.Tensor, token_seq: torch.Tensor,
                   block_table: torch.Tensor, scale: float, sink: Optional[float] = None, window: Optional[int] = None,
                   out_scale: float = 1.0, step=None, status: Optional[torch.Tensor] = None,
                   head_sinks: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                   gate_offset: int = 0, softcap: float = 0.0) -> torch.Tensor:
    """Causal attention of q [T, Hq, d] over pages whose rows are [k (d) | v (dv)] (``cache``
    [1, pages, Hkv, page, d + dv]; or planes [2, pages, Hkv, page, d] where d == dv), float32 arithmetic, any sizes. ``sink``: a logit whose exponential joins every softmax denominator without a
    value (0.0: one is added to the sum of exp(score)); ``head_sinks`` float32 [Hq]: such a logit per query head
    instead. ``gate`` [T, cols] of q's dtype: the output of (token, head) is also multiplied by
    sigmoid(gate[token, gate_offset + head]). ``softcap`` > 0: a score s becomes softcap * tanh(s / softcap) before the
    softmax. Returns [T, Hq * dv], multiplied by ``out_scale`` before its rounding."""
    _check(q, "q", None, 3)
    _check(cache, "cache", q.dtype, 5)
    _check(positions, "positions", torch.int32, 1)
    _check(token_seq, "token_seq", torch.int32, 1)
    _check(block_table, "block_table", torch.int32, 2)
    t, hq, d = q.shape
    _, num_pages, hkv, page_size, _row = cache.shape
    planes = _kv_planes(cache, hkv, d, v_dim)
    out = torch.empty((t, hq * v_dim), dtype=q.dtype, device=q.device)
    if t == 0:
        return out
    _check_head_extras(q, head_sinks, gate, gate_offset)
    _run("hybrid", "ti_attention_rows", out.data_ptr(), q.data_ptr(), cache.data_ptr(), positions.data_ptr(),
         token_seq.data_ptr(), block_table.data_ptr(), block_table.shape[1], t, hq, hkv, d, v_dim, page_size, num_pages,
         planes, float(scale), int(window or 0), int(sink is not None), float(sink or 0.0), _ptr(head_sinks), _ptr(gate),
         gate.shape[1] if gate is not None else 0, int(gate_offset), float(out_scale), float(softcap or 0.0), _ptr(status),
         _dtype_code(q), _stream())
    return out


# ---------------------------------------------------------------------- linear attention with a matrix state
class ScanGate:
    """How the decay of a linear-attention state is made from ``values`` (float32 [T, cols], read from column
    ``offset``). ``kind`` 'raw': the decay itself; 'sigmoid_power': sigmoid(v)^(1 / tau) per key channel;
    'step_size': dt = softplus(v + dt_bias[h]), decay exp(-exp(a_log[h]) dt) per head, and the keys are
    multiplied by dt; 'constant': ``values`` is one row [1, cols] of decays that every token uses (a fixed decay
    per head, as retention has). ``per_channel``: one value per (head, key channel) instead of one per head."""
    KINDS = {"raw": 0, "sigmoid_power": 1, "step_size": 2, "constant": 0}

    def __init__(self, kind: str, values: torch.Tensor, *, per_channel: bool, offset: int = 0, tau: float = 1.0,
                 a_log: Optional[torch.Tensor] = None, dt_bias: Optional[torch.Tensor] = None):
        if kind not in self.KINDS:
            raise KernelError(f"unknown gate {kind!r}; known: {sorted(self.KINDS)}")
        self.kind, self.values, self.per_channel, self.offset = kind, values, per_channel, offset
        self.tau, self.a_log, self.dt_bias = tau, a_log, dt_bias


SCAN_MIN_STRETCH = 32        # tokens a stretch of a long portion has at least
SCAN_TARGET_BLOCKS = 148 * 7  # what runs side by side at 72 registers a thread: more blocks would wait for a second round


def scan_stretches(max_q_len: int, num_seqs: int, heads: int, key_dim: int, value_dim: int) -> int:
    """Into how many stretches ``linear_scan`` cuts the requests' tokens: enough to have several blocks on every SM,
    none shorter than SCAN_MIN_STRETCH tokens; 1 for steps of short portions and decoded tokens."""
    if max_q_len < 2 * SCAN_MIN_STRETCH:
        return 1
    lanes = 1
    while lanes < 32 and -(-key_dim // lanes) > 16:
        lanes *= 2
    blocks = num_seqs * heads * -(-value_dim // (4 * (32 // lanes)))
    return max(1, min(SCAN_TARGET_BLOCKS // blocks, max_q_len // SCAN_MIN_STRETCH, 64))


def linear_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gate: ScanGate, *, state: torch.Tensor, heads: int,
                groups: int, key_dim: int, value_dim: int, q_offset: int = 0, k_offset: int = 0, v_offset: int = 0,
                q_scale: float = 1.0, skip: Optional[torch.Tensor] = None, cu_seqlens: torch.Tensor,
                state_slots: torch.Tensor, num_seqs: int, max_q_len: int = 0) -> torch.Tensor:
    """Per request and head, over the step's tokens in order: S <- diag(a) S + k v^T, o = S^T (q * q_scale)
    (+ skip[h] * v), from and back into ``state`` float32 [slots, heads, value_dim, key_dim] (S transposed).
    q and k: columns [offset, + groups * key_dim) of their tensors (head h reads group h // (heads / groups));
    v: columns [offset, + heads * value_dim). Returns o float32 [T, heads * value_dim]. ``max_q_len`` (a host
    number: the most tokens a request brings, 0: unknown) only decides into how many stretches long portions are cut
    to run side by side."""
    for name, ten in (("q", q), ("k", k), ("v", v)):
        _check(ten, name, q.dtype, 2)
    _check(gate.values, "gate", torch.float32, 2)
    t = q.shape[0]
    constant = gate.kind == "constant"          # the one row of decays is every token's: rows lie 0 floats apart
    if k.shape[0] != t or v.shape[0] != t or gate.values.shape[0] != (1 if constant else t):
        raise KernelError("linear_scan: one row per token in q, k, v and the gate (one row in all for a constant gate)")
    if (q_offset + groups * key_dim > q.shape[1] or k_offset + groups * key_dim > k.shape[1]
            or v_offset + heads * value_dim > v.shape[1]
            or gate.offset + heads * (key_dim if gate.per_channel else 1) > gate.values.shape[1]):
        raise KernelError("linear_scan: the columns do not fit the rows")
    stride = _slot_stride(state, heads * key_dim * value_dim, "state")
    for name, ten in (("a_log", gate.a_log), ("dt_bias", gate.dt_bias), ("skip", skip)):
        if ten is not None:
            _check(ten, name, torch.float32, 1)
            if ten.shape[0] != heads:
                raise KernelError(f"linear_scan: {name} has one entry per head")
    out = torch.empty((t, heads * value_dim), dtype=torch.float32, device=q.device)
    if t == 0:
        return out
    stretches, scratch = scan_stretches(max_q_len or t, num_seqs, heads, key_dim, value_dim), None
    if stretches > 1:
        fn = _fn("hybrid", "ti_linear_scan_scratch_floats")
        fn.restype = ctypes.c_longlong
        scratch = torch.empty(int(fn(num_seqs, t, heads, key_dim, value_dim, stretches)), dtype=torch.float32, device=q.device)
    made = None          # the decays (and the keys' factors) as the scan reads them, unless the gate holds them already
    if gate.kind not in ("raw", "constant") and stretches > 1:
        made = torch.empty(t * heads * (key_dim if gate.per_channel else 1) * (2 if gate.kind == "step_size" else 1),
                           dtype=torch.float32, device=q.device)
    _run("hybrid", "ti_linear_scan", out.data_ptr(), state.data_ptr(), stride, q.data_ptr(), q.shape[1], q_offset,
         k.data_ptr(), k.shape[1], k_offset, v.data_ptr(), v.shape[1], v_offset, gate.values.data_ptr(),
         0 if constant else gate.values.shape[1], gate.offset, ScanGate.KINDS[gate.kind], int(gate.per_channel), float(gate.tau),
         _ptr(gate.a_log), _ptr(gate.dt_bias), _ptr(skip), float(q_scale), cu_seqlens.data_ptr(), state_slots.data_ptr(),
         num_seqs, t, heads, groups, key_dim, value_dim, stretches, _ptr(scratch),
         scratch.numel() if scratch is not None else 0, _ptr(made), _dtype_code(q), _stream())
    return out


def head_rotation(rows: torch.Tensor, *, num_heads: int, num_kv_heads: int, head_dim: int, v_dim: int, has_kv: bool,
                  positions: torch.Tensor, token_seq: torch.Tensor, offset: int = 0,
                  q_norm_weight: Optional[torch.Tensor] = None, k_norm_weight: Optional[torch.Tensor] = None,
                  eps: float = 0.0, rotation: Optional[Rotation] = None, q_scale: float = 1.0, k_scale: float = 1.0,
                  cache: Optional[torch.Tensor] = None, block_table: Optional[torch.Tensor] = None,
                  out_float32: bool = False, status: Optional[torch.Tensor] = None,
                  norm_after: bool = False) -> torch.Tensor:
    """Per-head RMS norm (plain weights, optional), rotation and constant factors on the query heads, and with
    ``has_kv`` the key heads, that lie in columns [offset, ...) of ``rows`` [T, cols] as [q (Hq d) | k (Hkv d) |
    v (Hkv dv)]; values pass unchanged. With ``cache`` (planes [2, pages, Hkv, page, d] where d == dv, or rows
    [1, pages, Hkv, page, d + dv]) keys and values go to their token's place in the pages and q [T, Hq, d] is
    returned; without one, and with ``has_kv``, the result is the row [q | k | v] (for a recurrent mixer), float32
    if ``out_float32``. ``norm_after``: the norm of q and k comes after the rotation, with the weights or, without
    them, as a plain division by the root mean square. Float32 arithmetic, one rounding."""
    _check(rows, "rows", None, 2)
    _check(positions, "positions", torch.int32, 1)
    _check(token_seq, "token_seq", torch.int32, 1)
    t = rows.shape[0]
    nq, nk, nv = num_heads * head_dim, num_kv_heads * head_dim, num_kv_heads * v_dim
    if offset < 0 or offset + nq + ((nk + nv) if has_kv else 0) > rows.shape[1]:
        raise KernelError("head_rotation: the rows do not hold these heads")
    for name, w in (("q_norm_weight", q_norm_weight), ("k_norm_weight", k_norm_weight)):
        if w is not None:
            _check(w, name, torch.float32, 1)
            if w.shape[0] != head_dim:
                raise KernelError(f"head_rotation: {name} must have head_dim entries")
    if rotation is not None and rotation.rotary_dim > head_dim:
        raise KernelError(f"head_rotation: rotary_dim {rotation.rotary_dim} exceeds head_dim {head_dim}")
    planes = page_size = num_pages = 1
    max_blocks = 0
    if cache is not None:
        if not has_kv:
            raise KernelError("head_rotation: a cache is written with keys and values")
        _check(cache, "cache", rows.dtype, 5)
        _check(block_table, "block_table", torch.int32, 2)
        planes = _kv_planes(cache, num_kv_heads, head_dim, v_dim)
        num_pages, page_size, max_blocks = cache.shape[1], cache.shape[3], block_table.shape[1]
    to_row = has_kv and cache is None
    width = nq + nk + nv if to_row else nq
    out_dtype = torch.float32 if out_float32 else rows.dtype
    out = torch.empty((t, width), dtype=out_dtype, device=rows.device)
    if t:
        _run("hybrid", "ti_head_rotation", out.data_ptr(), width, _ptr(cache), planes, rows.data_ptr(), rows.shape[1],
             int(offset), _ptr(q_norm_weight), _ptr(k_norm_weight), float(eps), *_rotation_args(rotation), float(q_scale),
             float(k_scale), positions.data_ptr(), token_seq.data_ptr(), _ptr(block_table), max_blocks, t, num_heads,
             num_kv_heads, head_dim, v_dim, int(has_kv), page_size, num_pages, _ptr(status), int(out_float32),
             int(norm_after), _dtype_code(rows), _stream())
    return out if to_row else out.view(t, num_heads, head_dim)


def delta_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay_logits: torch.Tensor, beta_logits: torch.Tensor,
               *, a_log: torch.Tensor, dt_bias: Optional[torch.Tensor], state: torch.Tensor, heads: int, groups: int,
               key_dim: int, value_dim: int, q_offset: int = 0, k_offset: int = 0, v_offset: int = 0,
               decay_offset: int = 0, beta_offset: int = 0, q_scale: float = 1.0, unit_eps: float = 1e-6,
               cu_seqlens: torch.Tensor, state_slots: torch.Tensor, num_seqs: int) -> torch.Tensor:
    """The gated delta rule with a decay per head and key channel. Per request and head, over the step's tokens in
    order: S <- diag(g) S, u = beta (v - S^T k), S <- S + k u^T, o = S^T q, from and back into ``state`` float32
    [slots, heads, value_dim, key_dim] (S transposed). q and k (columns [offset, + groups * key_dim) of their tensors,
    head h reads group h // (heads / groups)) are made unit vectors, x / sqrt(sum x^2 + unit_eps), q also times
    ``q_scale``; g = exp(-exp(a_log[h]) * softplus(decay_logits[t, h, c] + dt_bias[h, c])) and
    beta = sigmoid(beta_logits[t, h]) from float32 rows. Returns o float32 [T, heads * value_dim]."""
    for name, ten in (("q", q), ("k", k), ("v", v)):
        _check(ten, name, q.dtype, 2)
    _check(decay_logits, "decay_logits", torch.float32, 2)
    _check(beta_logits, "beta_logits", torch.float32, 2)
    _check(a_log, "a_log", torch.float32, 1)
    if dt_bias is not None:
        _check(dt_bias, "dt_bias", torch.float32, 1)
    t = q.shape[0]
    if any(ten.shape[0] != t for ten in (k, v, decay_logits, beta_logits)):
        raise KernelError("delta_scan: one row per token in q, k, v and the gates")
    if (heads % groups or q_offset + groups * key_dim > q.shape[1] or k_offset + groups * key_dim > k.shape[1]
            or v_offset + heads * value_dim > v.shape[1] or decay_offset + heads * key_dim > decay_logits.shape[1]
            or beta_offset + heads > beta_logits.shape[1] or a_log.shape[0] != heads
            or (dt_bias is not None and dt_bias.shape[0] != heads * key_dim)):
        raise KernelError("delta_scan: the tensors do not hold these heads")
    stride = _slot_stride(state, heads * value_dim * key_dim, "state")
    out = torch.empty((t, heads * value_dim), dtype=torch.float32, device=q.device)
    if t:
        # what the recurrence reads of every token, made once: unit q and k, the decays, v, beta and k.q, float32
        work = torch.empty(t * (2 * groups * key_dim + heads * (key_dim + value_dim + 1) + groups) + 24,
                           dtype=torch.float32, device=q.device)
        _run("hybrid", "ti_delta_scan", out.data_ptr(), state.data_ptr(), stride, q.data_ptr(), q.shape[1], int(q_offset),
             k.data_ptr(), k.shape[1], int(k_offset), v.data_ptr(), v.shape[1], int(v_offset), decay_logits.data_ptr(),
             decay_logits.shape[1], int(decay_offset), beta_logits.data_ptr(), beta_logits.shape[1], int(beta_offset),
             a_log.data_ptr(), _ptr(dt_bias), float(q_scale), float(unit_eps), cu_seqlens.data_ptr(), state_slots.data_ptr(),
             int(num_seqs), t, heads, groups, key_dim, value_dim, work.data_ptr(), work.numel(), _dtype_code(q), _stream())
    return out


def gated_group_norm(y: torch.Tensor, gate: Optional[torch.Tensor], weight: torch.Tensor, *, group: int, eps: float,
                     gate_first: bool, out_dtype: torch.dtype, gate_offset: int = 0, out_scale: float = 1.0,
                     gate_activation: str = "silu") -> torch.Tensor:
    """Every ``group`` neighbouring features of y (float32 [T, C]) divided by their root mean square, times
    ``weight`` (float32, repeated along the row if shorter) and ``out_scale``; silu (or, ``gate_activation``
    'sigmoid', the sigmoid) of columns [gate_offset, + C) of ``gate`` multiplies y before the norm (``gate_first``)
    or the result after it. One rounding to ``out_dtype``."""
    if gate_activation not in ("silu", "sigmoid"):
        raise KernelError(f"gated_group_norm: unknown gate activation {gate_activation!r}")
    _check(y, "y", torch.float32, 2)
    _check(weight, "weight", torch.float32, 1)
    t, c = y.shape
    if c % group or c % weight.shape[0]:
        raise KernelError("gated_group_norm: the row does not split into these groups or weights")
    if gate is not None:
        _check(gate, "gate", out_dtype, 2)
        if gate.shape[0] != t or gate_offset + c > gate.shape[1]:
            raise KernelError("gated_group_norm: the gate does not fit")
    out = torch.empty((t, c), dtype=out_dtype, device=y.device)
    _run("hybrid", "ti_gated_group_norm", out.data_ptr(), y.data_ptr(), _ptr(gate), gate.shape[1] if gate is not None else 0,
         gate_offset, weight.data_ptr(), weight.shape[0], t, c, group, float(eps), int(gate_first), float(out_scale),
         int(gate_activation == "sigmoid"), _dtype_code(out), _stream())
    return out


# ---------------------------------------------------------------------- sampling
_ARGMAX_PARTS = 32
_argmax_scratch = {}
_sample_scratch = {}


def argmax(logits: torch.Tensor, extra: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Index of the largest logit of every row (first index on ties), int32 [N]. ``extra``: int32 device
    words (at most 32) that the kernel copies behind the tokens, so that one copy to the host brings both;
    the result then has N + len(extra) entries."""
    _check(logits, "logits", torch.float32, 2)
    n = logits.shape[0]
    num_extra = _check_extra(extra)
    out = torch.empty((n + num_extra,), dtype=torch.int32, device=logits.device)
    key = torch.device(logits.device)
    scratch = _argmax_scratch.get(key)
    if scratch is None or scratch[2].numel() < n:
        rows = max(256, n)
        scratch = _argmax_scratch[key] = (
            torch.empty(rows * _ARGMAX_PARTS, dtype=torch.float32, device=key),
            torch.empty(rows * _ARGMAX_PARTS, dtype=torch.int32, device=key),
            torch.zeros(rows, dtype=torch.int32, device=key))
    _run("core", "ti_argmax", out.data_ptr(), logits.data_ptr(), n, logits.shape[1], scratch[0].data_ptr(),
         scratch[1].data_ptr(), scratch[2].data_ptr(), _ptr(extra), num_extra, _stream())
    return out


def _check_extra(extra: Optional[torch.Tensor]) -> int:
    if extra is None:
        return 0
    _check(extra, "extra", torch.int32, 1)
    if extra.shape[0] > 32:
        raise KernelError("at most 32 extra words travel with the tokens")
    return extra.shape[0]


def sample(logits: torch.Tensor, temperature: torch.Tensor, topk: torch.Tensor, greedy: torch.Tensor,
           seed: torch.Tensor, stream_id: torch.Tensor, step: torch.Tensor,
           extra: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of float32 logits [N, V]. Per row: ``greedy`` (int32 0/1),
    ``temperature`` (float32 > 0), ``topk`` (int32, 0 = off), and the random stream
    (``seed`` int64, ``stream_id`` int32, ``step`` int32). ``extra``: as in ``argmax``."""
    _check(logits, "logits", torch.float32, 2)
    n = logits.shape[0]
    for name, t, dt in (("temperature", temperature, torch.float32), ("topk", topk, torch.int32),
                        ("greedy", greedy, torch.int32), ("seed", seed, torch.int64),
                        ("stream_id", stream_id, torch.int32), ("step", step, torch.int32)):
        _check(t, name, dt, 1)
        if t.shape[0] != n:
            raise KernelError(f"{name} must have one entry per row")
    num_extra = _check_extra(extra)
    out = torch.empty((n + num_extra,), dtype=torch.int32, device=logits.device)
    key = torch.device(logits.device)
    scratch = _sample_scratch.get(key)
    if scratch is None or scratch[5].numel() < n:
        # a row is shared out over several blocks: their best, and for top-k their candidates, meet here
        rows = max(64, n)
        parts = int(_fn("core", "ti_sample_parts")())
        cap = int(_fn("core", "ti_sample_candidates")())
        scratch = _sample_scratch[key] = (
            torch.empty(rows * parts, dtype=torch.float32, device=key),
            torch.empty(rows * parts, dtype=torch.int32, device=key),
            torch.empty(rows * parts * cap, dtype=torch.int32, device=key),
            torch.empty(rows * parts * cap, dtype=torch.int32, device=key),
            torch.empty(rows * parts, dtype=torch.int32, device=key),
            torch.zeros(rows, dtype=torch.int32, device=key))
    _run("core", "ti_sample", out.data_ptr(), logits.data_ptr(), n, logits.shape[1],
         temperature.data_ptr(), topk.data_ptr(), greedy.data_ptr(), seed.data_ptr(),
         stream_id.data_ptr(), step.data_ptr(), *(t.data_ptr() for t in scratch), _ptr(extra), num_extra, _stream())
    return out


def token_nll(logits: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """logsumexp(logits[row]) - logits[row, tokens[row]] in float32, [N]."""
    _check(logits, "logits", torch.float32, 2)
    _check(tokens, "tokens", torch.int32, 1)
    if tokens.shape[0] != logits.shape[0]:
        raise KernelError("token_nll: one token per row")
    out = torch.empty((logits.shape[0],), dtype=torch.float32, device=logits.device)
    _run("core", "ti_token_nll", out.data_ptr(), logits.data_ptr(), tokens.data_ptr(), logits.shape[0],
         logits.shape[1], _stream())
    return out


def launch_count() -> int:
    return library.launch_count()
