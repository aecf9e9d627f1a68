"""Python face of the CUDA kernel library: argument checks, dispatch, ctypes calls.

Every op runs a hand-written kernel on the current CUDA stream of ``torch``; torch itself
only owns the memory.  There is no CPU path and no library fallback: a missing library is
built on first use, and a failure to build or load it raises.

Dispatch rule for matrix products: the tensor-core kernel where its conditions hold
(bfloat16 operands, 16-byte aligned rows), else the general FP32-pipe kernel, which takes
every shape and dtype mix.  A kernel that cannot take a size refuses it with an error that
names the size; no op returns a wrong result for an odd size.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import build
from .plan import decode_splits

_c_int, _c_ll, _c_float, _c_ptr = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p

_SIGNATURES = {
    "hb_device_info": [_c_int, ctypes.POINTER(_c_int), ctypes.POINTER(_c_int), ctypes.POINTER(_c_int)],
    "hb_timeline_set": [_c_ptr, _c_ptr, _c_int, _c_int],
    "hb_embed": [_c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_float, _c_ptr, _c_ptr],
    "hb_rmsnorm": [_c_ptr, _c_ptr, _c_float, _c_float, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_ptr],
    "hb_silu_mul": [_c_ptr, _c_int, _c_ll, _c_ptr, _c_int, _c_ll, _c_int, _c_int, _c_ptr],
    "hb_rope_table": [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_float, _c_ptr],
    "hb_dyt": [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ll, _c_ptr, _c_int, _c_int, _c_ptr],
    "hb_short_conv": [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ll,
                      _c_int, _c_int, _c_int, _c_ptr],
    "hb_relu2": [_c_ptr, _c_int, _c_ll, _c_ptr, _c_int, _c_ll, _c_int, _c_int, _c_ptr],
    "hb_qkv_prepare": [_c_ptr, _c_int, _c_ll, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_float, _c_ptr,
                       _c_int, _c_ll, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_ptr,
                       _c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
    "hb_attention_sink": [_c_ptr, _c_int, _c_ll, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int,
                          _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_int, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr],
    "hb_head_mix": [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ll, _c_ptr],
    "hb_attention_heads": [_c_ptr, _c_int, _c_ll, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr,
                           _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_int, _c_ptr, _c_int, _c_int,
                           _c_int, _c_ptr, _c_ptr],
    "hb_attention_sink_prefill": [_c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int,
                                  _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr],
    "hb_head_mix_splits": [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ll, _c_ptr],
    "hb_mlstm_scan": [_c_ptr, _c_int, _c_ll, _c_ptr, _c_float, _c_float, _c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int,
                      _c_int, _c_int, _c_ptr],
    "hb_mlstm_chunks": [_c_ptr, _c_int, _c_ll, _c_ptr, _c_float, _c_float, _c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int,
                        _c_int, _c_int, _c_ptr],
    "hb_mlstm_output": [_c_ptr, _c_ptr, _c_int, _c_ll, _c_ptr, _c_float, _c_ptr, _c_int, _c_ll, _c_int, _c_int, _c_int, _c_ptr],
    "hb_rope_kv_append": [_c_ptr, _c_int, _c_ll, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_int,
                          _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
    "hb_gemm_general": [_c_ptr, _c_int, _c_ll, _c_ptr, _c_int, _c_ll, _c_ptr, _c_int, _c_ll, _c_int, _c_int, _c_int,
                        _c_int, _c_ptr],
    "hb_gemm_tc": [_c_ptr, _c_ll, _c_ptr, _c_ll, _c_ll, _c_ptr, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                   _c_ptr, _c_ll, _c_ptr, _c_ll, _c_ptr, _c_int, _c_ptr],
    "hb_gemm_tc_fold": [_c_ptr, _c_ll, _c_ptr, _c_ll, _c_ll, _c_ptr, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                        _c_ptr, _c_ll, _c_ptr, _c_ll, _c_ptr, _c_int, _c_ptr, _c_ptr],
    "hb_gemm_tc2": [_c_ptr, _c_ll, _c_ptr, _c_ll, _c_ll, _c_ptr, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_int,
                    _c_ptr],
    "hb_attention_general": [_c_ptr, _c_int, _c_ll, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr,
                             _c_int, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_ptr, _c_ptr],
    "hb_attention_decode": [_c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ll, _c_int, _c_int,
                            _c_int, _c_int, _c_float, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
    "hb_attention_decode_combined": [_c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ll, _c_int,
                                     _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
    "hb_attention_decode_fused": [_c_ptr, _c_ll, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr,
                                  _c_ll, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_int, _c_int, _c_int,
                                  _c_ptr, _c_ptr],
    "hb_attention_prefill": [_c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ll, _c_int, _c_int,
                             _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_ptr, _c_ptr],
    "hb_attention_prefill_tc": [_c_ptr, _c_ll, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ll, _c_int,
                                _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_ptr, _c_ptr],
    "hb_random_normal": [_c_ptr, _c_int, _c_ll, ctypes.c_ulonglong, _c_float, _c_float, _c_ptr],
    "hb_argmax": [_c_ptr, _c_ll, _c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr],
    "hb_sample": [_c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr],
    "hb_rmsnorm_add": [_c_ptr, _c_ll, _c_ptr, _c_float, _c_float, _c_ptr, _c_ll, _c_ptr, _c_float, _c_float, _c_ptr, _c_int, _c_ll, _c_int,
                       _c_int, _c_ptr],
    "hb_scaled_sum": [_c_ptr, _c_float, _c_ptr, _c_float, _c_ptr, _c_ll, _c_ptr],
    "hb_qk_norm_append": [_c_ptr, _c_ll, _c_ptr, _c_ptr, _c_float, _c_ptr, _c_int, _c_ll, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr,
                          _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
    "hb_pool_blocks": [_c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int,
                       _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
    "hb_attention_pool": [_c_ptr, _c_int, _c_ll, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int,
                          _c_int, _c_ptr, _c_ptr, _c_ll, _c_ptr, _c_int, _c_ll, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float,
                          _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
    "hb_attention_pool_prefill": [_c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ll, _c_ptr, _c_ll,
                                  _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_ptr, _c_ptr],
    "hb_decay_memory": [_c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr,
                        _c_int, _c_float, _c_ptr],
    "hb_gated_norm": [_c_ptr, _c_ll, _c_ptr, _c_ll, _c_ptr, _c_float, _c_float, _c_ptr, _c_int, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_ptr],
    "hb_layernorm": [_c_ptr, _c_ll, _c_ptr, _c_ptr, _c_float, _c_ptr, _c_int, _c_ll, _c_ptr, _c_int, _c_int, _c_ptr],
    "hb_layernorm_add": [_c_ptr, _c_ll, _c_ptr, _c_ll, _c_float, _c_float, _c_ptr, _c_ptr, _c_float, _c_ptr, _c_ll, _c_ptr, _c_int, _c_ll,
                         _c_int, _c_int, _c_ptr],
    "hb_convert": [_c_ptr, _c_ptr, _c_int, _c_ll, _c_ptr],
    "hb_latent_prepare": [_c_ptr, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_float, _c_ptr, _c_int, _c_ptr, _c_int, _c_ll,
                          _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
    "hb_latent_gather": [_c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr],
    "hb_latent_scatter": [_c_ptr, _c_ll, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                          _c_ptr, _c_ptr, _c_int, _c_ptr],
    "hb_head_linear": [_c_ptr, _c_ll, _c_ll, _c_ptr, _c_int, _c_ptr, _c_int, _c_ll, _c_ll, _c_ptr, _c_ll, _c_int, _c_int, _c_int, _c_int,
                       _c_ptr],
    "hb_conv_act": [_c_ptr, _c_ll, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ll, _c_int, _c_int, _c_int,
                    _c_int, _c_ptr],
    "hb_selective_scan": [_c_ptr, _c_int, _c_ll, _c_ptr, _c_ll, _c_ptr, _c_ll, _c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ll, _c_ptr,
                          _c_ptr, _c_ptr, _c_int, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ll, _c_ptr],
    "hb_moe_route": [_c_ptr, _c_int, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_ptr],
    "hb_moe_plan": [_c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr],
    "hb_moe_glu": [_c_ptr, _c_int, _c_ll, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr, _c_int, _c_ll, _c_int,
                   _c_int, _c_float, _c_float, _c_int, _c_ptr],
    "hb_moe_down": [_c_ptr, _c_int, _c_ll, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr, _c_ll, _c_int, _c_int, _c_int,
                    _c_ptr],
    "hb_moe_combine": [_c_ptr, _c_ll, _c_ptr, _c_int, _c_ptr, _c_ll, _c_int, _c_int, _c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_ll, _c_ptr],
    "hb_moe_route_scores": [_c_ptr, _c_int, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float,
                            _c_ptr],
    "hb_gelu_unit": [_c_ptr, _c_ll, _c_ptr, _c_int, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_ptr],
    "hb_embed_pair": [_c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_ll, _c_ll, _c_ptr, _c_ptr,
                      _c_ptr, _c_ptr, _c_ptr, _c_ll, _c_ptr, _c_ptr],
    "hb_scaled_add_norm": [_c_ptr, _c_ll, _c_float, _c_ptr, _c_ll, _c_ptr, _c_float, _c_float, _c_ptr, _c_int, _c_ll, _c_int, _c_int, _c_ptr],
    "hb_normed_sum": [_c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ll, _c_ptr, _c_float, _c_ptr, _c_ll, _c_int, _c_int, _c_int, _c_ptr],
    "hb_head_scan": [_c_ptr, _c_ll, _c_ptr, _c_ll, _c_ptr, _c_ll, _c_ptr, _c_ll, _c_ptr, _c_ll, _c_ptr, _c_ptr, _c_float, _c_ptr, _c_float,
                     _c_ptr, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ll, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                     _c_ptr, _c_ll, _c_ptr],
    "hb_glu_clamp": [_c_ptr, _c_ll, _c_ptr, _c_int, _c_ll, _c_int, _c_int, _c_float, _c_float, _c_ptr],
}

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}
_lib = None


class KernelError(RuntimeError):
    pass


def workspace_rows(workspace, rows: int) -> int:
    """Rows to ask a workspace for when a buffer's size follows a step's tokens: whole thousands, so that steps of similar
    sizes share one allocation."""
    return -(-int(rows) // 1024) * 1024


def load_library():
    """Loads (building first if needed) the kernel library; raises if that is impossible."""
    global _lib
    if _lib is None:
        path = build.library_path()
        lib = ctypes.CDLL(path)
        lib.hb_last_error.restype = ctypes.c_char_p
        lib.hb_last_error.argtypes = []
        for name, args in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = _c_int
        lib.hb_gemm_tc_token_tile.argtypes, lib.hb_gemm_tc_token_tile.restype = [_c_int], _c_int
        lib.hb_gemm_tc_scratch_floats.argtypes = [_c_int, _c_int, _c_int, _c_int, _c_int]
        lib.hb_gemm_tc_scratch_floats.restype = _c_ll
        lib.hb_gemm_tc_tiles.argtypes, lib.hb_gemm_tc_tiles.restype = [_c_int, _c_int, _c_int], _c_ll
        lib.hb_gemm_tc_resident_clusters.argtypes, lib.hb_gemm_tc_resident_clusters.restype = [_c_int, _c_int], _c_int
        lib.hb_gemm_tc2_wanted.argtypes, lib.hb_gemm_tc2_wanted.restype = [_c_int, _c_int, _c_int], _c_int
        lib.hb_gemm_tc2_resident_pairs.argtypes, lib.hb_gemm_tc2_resident_pairs.restype = [_c_int], _c_int
        for name in ("hb_attention_decode_supported", "hb_attention_prefill_supported", "hb_attention_prefill_tc_supported"):
            getattr(lib, name).argtypes, getattr(lib, name).restype = [_c_int, _c_int, _c_int], _c_int
        lib.hb_attention_sink_prefill_supported.argtypes, lib.hb_attention_sink_prefill_supported.restype = [_c_int] * 4, _c_int
        lib.hb_attention_heads_variant.argtypes, lib.hb_attention_heads_variant.restype = [_c_int] * 6, _c_int
        lib.hb_attention_heads_writes_output.argtypes, lib.hb_attention_heads_writes_output.restype = [_c_int] * 6, _c_int
        lib.hb_attention_pool_supported.argtypes, lib.hb_attention_pool_supported.restype = [_c_int] * 2, _c_int
        lib.hb_attention_pool_prefill_supported.argtypes, lib.hb_attention_pool_prefill_supported.restype = [_c_int] * 2, _c_int
        lib.hb_moe_max_tiles.argtypes, lib.hb_moe_max_tiles.restype = [_c_int] * 3, _c_int
        lib.hb_moe_tile_rows.argtypes, lib.hb_moe_tile_rows.restype = [_c_int], _c_int
        lib.hb_attention_decode_ctas_per_sm.argtypes, lib.hb_attention_decode_ctas_per_sm.restype = [_c_int], _c_int
        lib.hb_attention_decode_scratch_floats.argtypes = [_c_int, _c_int, _c_int, _c_int]
        lib.hb_attention_decode_scratch_floats.restype = _c_ll
        _lib = lib
    return _lib


def _code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not supported by the kernels") from None


def _rows(t: torch.Tensor, what: str) -> int:
    """Row stride of a 2-D tensor whose rows are contiguous."""
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise KernelError(f"{what}: expected a 2-D tensor with contiguous rows, got shape {tuple(t.shape)} "
                          f"strides {t.stride()}")
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


class _NormFold(ctypes.Structure):
    """HbNormFold of csrc/api.h."""
    _fields_ = [("prep_w", ctypes.c_void_p), ("prep_offset", ctypes.c_float), ("prep_out", ctypes.c_void_p),
                ("prep_ld", ctypes.c_longlong), ("prep_sumsq", ctypes.c_void_p), ("scale_sumsq", ctypes.c_void_p),
                ("scale_parts", ctypes.c_int), ("scale_inv_size", ctypes.c_float), ("scale_eps", ctypes.c_float),
                ("sumsq_ld", ctypes.c_int)]


class PreparedNorm:
    """A norm whose input the product in front has prepared: the buffer it was asked to fill
    holds ``x * (offset + weight)`` without the per-token factor ``rsqrt(mean(x^2) + eps)``, and
    ``sumsq[token, :parts]`` add up to the token's sum of squares.  The product that reads the
    buffer multiplies its rows by the factor (``Ops.linear(..., scale=...)``)."""

    def __init__(self, sumsq: torch.Tensor, parts: int, size: int, eps: float):
        self.sumsq, self.parts, self.size, self.eps = sumsq, int(parts), int(size), float(eps)


class PackedWeight:
    """A bfloat16 weight matrix ``[rows, cols]`` stored for the tensor-core products: every
    128-row x 64-column tile is one contiguous 16 KB piece, and the tiles of a 128-row band
    follow one another along the columns (``data`` has the shape ``[bands, column blocks, 128,
    64]``, zero beyond ``rows`` and ``cols``).  A CTA that walks along the columns of a band
    then reads one sequential range of memory instead of 128 rows a whole matrix row apart.

    ``gate_up_bands``: the matrix is ``[gate; up]`` with halves of a multiple of 64 rows, and band
    ``b`` holds the gate rows ``64 b .. 64 b + 63`` followed by the up rows of the same features:
    what one tile of the fused SwiGLU product needs is then ONE piece (one tile load per K block
    instead of two, which a many-token product's K loop feels: 0.41 against 0.46 us per block)."""

    def __init__(self, data: torch.Tensor, rows: int, cols: int, gate_up_bands: bool = False):
        self.data, self.rows, self.cols, self.gate_up_bands = data, int(rows), int(cols), bool(gate_up_bands)

    @classmethod
    def pack(cls, w: torch.Tensor, gate_up_bands: bool = False) -> "PackedWeight":
        rows, cols = w.shape
        if gate_up_bands:
            half = rows // 2
            if rows % 2 or half % 64:
                raise KernelError(f"gate/up bands need halves of a multiple of 64 rows, not {rows} rows")
            banded = torch.stack([w[:half].view(half // 64, 64, cols), w[half:].view(half // 64, 64, cols)], dim=1)
            packed = cls.pack(banded.reshape(rows, cols))
            packed.gate_up_bands = True
            return packed
        bands, blocks = -(-rows // 128), -(-cols // 64)
        if rows % 128 or cols % 64:
            full = torch.zeros(bands * 128, blocks * 64, dtype=w.dtype, device=w.device)
            full[:rows, :cols] = w
            w = full
        return cls(w.view(bands, 128, blocks, 64).permute(0, 2, 1, 3).contiguous(), rows, cols)

    def unpacked(self) -> torch.Tensor:
        bands, blocks = self.data.shape[0], self.data.shape[1]
        w = self.data.permute(0, 2, 1, 3).reshape(bands * 128, blocks * 64)[: self.rows, : self.cols]
        if self.gate_up_bands:
            w = w.reshape(self.rows // 128, 2, 64, self.cols).transpose(0, 1).reshape(self.rows, self.cols)
        return w.contiguous()

    def first_rows(self, n: int) -> "PackedWeight":
        """The matrix of the first ``n`` rows (shares the storage)."""
        if not 0 < n <= self.rows or self.gate_up_bands:
            raise KernelError(f"first_rows: {n} of {self.rows} rows" + (" of a [gate; up] matrix in bands" if self.gate_up_bands else ""))
        return PackedWeight(self.data, n, self.cols)

    @property
    def shape(self):
        return (self.rows, self.cols)

    @property
    def dtype(self):
        return self.data.dtype

    @property
    def device(self):
        return self.data.device

    def numel(self) -> int:
        return self.rows * self.cols

    def element_size(self) -> int:
        return self.data.element_size()

    def data_ptr(self) -> int:
        return self.data.data_ptr()


class Ops:
    """The kernels bound to one device."""

    def __init__(self, device):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise KernelError("the kernels run on a CUDA device only")
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device is available; the library has no CPU path")
        self.lib = load_library()
        self.call_log = None  # a list: the name of every library call is appended (diagnostics)
        major, minor, sms = _c_int(), _c_int(), _c_int()
        idx = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self._call("hb_device_info", idx, ctypes.byref(major), ctypes.byref(minor), ctypes.byref(sms))
        self.sm = (major.value, minor.value)
        self.sm_count = sms.value
        if major.value != 10:
            raise KernelError(f"the kernels are built for sm_100a; device {idx} is sm_{major.value}{minor.value}")
        self.launches = 0  # kernels launched through this object (a claim bench.py reports)
        self.use_tensor_cores = True   # tests switch this off to compare the two matrix-product kernels
        self.use_pair_gemm = True      # many-token products on CTA pairs (cta_group::2)
        # few-token steps: a norm between two products is folded into them (HILBERT_B200_FOLD_NORMS=0: norm kernels)
        self.fold_norms = os.environ.get("HILBERT_B200_FOLD_NORMS", "1") != "0"
        self._sumsq = None             # [FOLD_MAX_TOKENS, slots]: the partial sums of squares of a folded norm
        # weights as contiguous tiles (PackedWeight); HILBERT_B200_PACK=0 keeps them row-major
        self.use_packed_weights = os.environ.get("HILBERT_B200_PACK", "1") != "0"
        # device status words (csrc/common.cuh): a kernel that meets a fault notes the first one of
        # its kind and carries on with a safe value; the host reads the words where it waits anyway
        # (check_errors, or copied back beside a step's sampled tokens) and raises
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.error_flag = self.status[:1]      # word 0: a bounded wait of a tensor-core kernel ran out
        # split-K scratch: float32 partial tiles and one counter per output tile (kept zero)
        self._splitk_partials = torch.empty(8 << 20, dtype=torch.float32, device=self.device)
        self._splitk_counters = torch.zeros(1 << 16, dtype=torch.int32, device=self.device)
        # split-K decode attention scratch: partial outputs with their maxima and sums
        self._decode_scratch = torch.empty(4 << 20, dtype=torch.float32, device=self.device)
        self._decode_counters = torch.zeros(1 << 16, dtype=torch.int32, device=self.device)
        # greedy pick: (maximum, index) of each range of a row, and a counter per row (kept zero)
        self._argmax_scratch = torch.empty(2 * 1024 * self.ARGMAX_MAX_PARTS, dtype=torch.int32, device=self.device)
        self._argmax_counters = torch.zeros(1024, dtype=torch.int32, device=self.device)
        self._retired = []              # outgrown scratch, kept alive for graphs that captured it
        self._splits_cache = {}
        self.use_tcgen05_attention = True   # head size 128 prefill on tcgen05 (else the mma.sync kernel)
        self.use_fast_attention = True  # tests switch this off to compare with the general kernel
        # attention_heads: the weights-times-values product on the tensor cores (each 32-bit weight as two bfloat16
        # terms) where the sizes allow; tests switch it off to compare with the FP32-pipe variant
        self.use_mma_attention = True
        self.use_flash_sink_attention = True    # steps of many tokens: attention_sink_prefill where it is built
        self.use_mma_pool_attention = True      # steps of many tokens: attention_pool_prefill where it is built (tests compare both)
        # Decode attention that rotates the new queries and key and appends to the cache itself
        # (no rotation kernel in front; the new key and value go into the owning split's copy of
        # their page in shared memory).  Inside a replayed graph at batch 8 / 8192 tokens it takes
        # 43.2 us where rotation + attention take 3.4 + 41.0 us; alternating runs on one GPU, a step
        # of 8 layers: 1310 against 1312 us, at batch 1 1046 against 1047 us, 1B sizes 613 against
        # 616 us.  One launch less, the time of the hand-over between kernels stays.  Whether a
        # model's attention uses it is the part's choice (the mixer's `fuse_decode`, its position
        # encoding's `fusable`); this switch only takes the kernel away (tests compare both ways).
        self.fuse_decode_attention = True
        # Split-K decode attention whose last split combines the splits, instead of a second
        # kernel.  Off: at batch 8 / 8192 tokens a step of 8 layers takes 1319 us against 1313 us, at
        # batch 1 1079 against 1052 us (the last split's two round trips are longer than a kernel
        # that is already resident); with the rotation inside as well, 50.3 us per layer against
        # 43.2 + 3.5 us.  A single split always writes the result itself.
        self.combine_in_attention = False

    # ------------------------------------------------------------------ plumbing
    def _call(self, name: str, *args) -> None:
        rc = getattr(self.lib, name)(*args)
        if rc != 0:
            raise KernelError(self.lib.hb_last_error().decode("utf-8", "replace"))
        if self.call_log is not None:
            self.call_log.append(name)

    # ------------------------------------------------------------------ timeline
    def timeline_begin(self, capacity: int = 1 << 16, events: bool = False) -> None:
        """Switches the kernels' time marks on (library built with HILBERT_B200_TIMELINE=1 only):
        from now on every kernel notes when its first block reached its dependency wait and
        when that wait returned.  ``events`` also records the events inside the kernels that have
        some (the few-token matrix product); they cost those kernels a few microseconds."""
        self._tl_marks = torch.zeros(capacity, 2, dtype=torch.int64, device=self.device)
        self._tl_count = torch.zeros(1, dtype=torch.int32, device=self.device)
        torch.cuda.synchronize(self.device)
        self._call("hb_timeline_set", self._tl_marks.data_ptr(), self._tl_count.data_ptr(), capacity,
                   1 if events else 0)

    def timeline_end(self):
        """Switches the marks off; returns the marks ordered by their second field.  A kernel's
        mark is (resident_ns, predecessors_done_ns) of its first block; an event inside a kernel
        (the matrix product has some) is (code * 1000 + block, time_ns) with a first field
        below 10**9."""
        torch.cuda.synchronize(self.device)
        self._call("hb_timeline_set", None, None, 0, 0)
        n = min(int(self._tl_count.item()), self._tl_marks.shape[0])
        marks = self._tl_marks[:n].tolist()
        self._tl_marks = self._tl_count = None
        return sorted(((a, b) for a, b in marks), key=lambda m: m[1])

    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def _dev(self, *tensors) -> None:
        for t in tensors:
            if t is not None and t.device != self.device:
                raise KernelError(f"tensor on {t.device}, kernels bound to {self.device}")

    # ------------------------------------------------------------------ elementwise
    def embed(self, tokens, table, out, scale: float = 1.0) -> None:
        """``out[t] = table[tokens[t]] * scale`` in 32-bit; ``table`` row-major or a PackedWeight."""
        packed = isinstance(table, PackedWeight)
        self._dev(tokens, table.data if packed else table, out)
        if tokens.dtype != torch.int32 or out.dtype != torch.float32 or not out.is_contiguous() \
                or not (packed or table.is_contiguous()):
            raise KernelError("embed: tokens int32, contiguous table, contiguous float32 output expected")
        T, H = out.shape
        if table.shape[1] != H or tokens.numel() != T:
            raise KernelError("embed: shapes do not agree")
        self._call("hb_embed", tokens.data_ptr(), table.data_ptr(), _code(table), out.data_ptr(), T, H,
                   table.shape[0], 1 if packed else 0, float(scale), self.status.data_ptr(), self._stream())
        self.launches += 1

    def embed_pair(self, step, table, pairs, state, out, buckets: int, mul_prev: int, mul_cur: int, scale: float = 1.0) -> None:
        """``out[t] = table[token] * scale + pairs[row]`` in 32-bit with ``row = (previous * mul_prev + token * mul_cur) mod
        buckets``, and ``row = buckets`` (the last row of ``pairs``) for a sequence's first token.  ``state`` int32 ``[slots, 1]``:
        every sequence's last token, read by the step's first token and brought up to date."""
        packed = isinstance(table, PackedWeight)
        self._dev(step.tokens, table.data if packed else table, pairs, state, out)
        T, H = out.shape
        if out.dtype != torch.float32 or not out.is_contiguous() or not (packed or table.is_contiguous()) or not pairs.is_contiguous() \
                or table.shape[1] != H or tuple(pairs.shape) != (buckets + 1, H) or pairs.dtype != table.dtype or step.tokens.numel() != T:
            raise KernelError("embed_pair: contiguous tables of one dtype ([vocab, width], [buckets + 1, width]) and a float32 output expected")
        if state.dtype != torch.int32 or state.dim() != 2 or state.stride(1) != 1:
            raise KernelError("embed_pair: state must be int32 [slots, 1]")
        self._call("hb_embed_pair", step.tokens.data_ptr(), table.data_ptr(), _code(table), pairs.data_ptr(), out.data_ptr(), T, H,
                   table.shape[0], 1 if packed else 0, float(scale), int(buckets), int(mul_prev), int(mul_cur), step.positions.data_ptr(),
                   step.tok_seq.data_ptr(), step.seq_start.data_ptr(), step.state_slots.data_ptr(), state.data_ptr(), state.stride(0),
                   self.status.data_ptr(), self._stream())
        self.launches += 1

    def rmsnorm(self, x, weight, eps: float, offset: float, out, rows=None) -> None:
        self._dev(x, weight, out, rows)
        if x.dtype != torch.float32 or weight.dtype != torch.float32 or not x.is_contiguous() \
                or not out.is_contiguous() or not weight.is_contiguous():
            raise KernelError("rmsnorm: contiguous float32 input and weight, contiguous output expected")
        H = x.shape[1]
        n = out.shape[0]
        if out.shape[1] != H or weight.numel() != H:
            raise KernelError("rmsnorm: shapes do not agree")
        if rows is None:
            if n != x.shape[0]:
                raise KernelError("rmsnorm: output rows differ from input rows")
            rp = None
        else:
            if rows.dtype != torch.int32 or rows.numel() != n:
                raise KernelError("rmsnorm: rows must be int32, one per output row")
            rp = rows.data_ptr()
        self._call("hb_rmsnorm", x.data_ptr(), weight.data_ptr(), float(eps), float(offset), out.data_ptr(), _code(out),
                   rp, n, H, self._stream())
        self.launches += 1

    def silu_mul(self, gate_up, out) -> None:
        self._dev(gate_up, out)
        inter = out.shape[1]
        if gate_up.shape[1] != 2 * inter or gate_up.shape[0] != out.shape[0]:
            raise KernelError("silu_mul: input must be [rows, 2 * inter]")
        self._call("hb_silu_mul", gate_up.data_ptr(), _code(gate_up), _rows(gate_up, "silu_mul input"), out.data_ptr(),
                   _code(out), _rows(out, "silu_mul output"), out.shape[0], inter, self._stream())
        self.launches += 1

    def rope_table(self, positions, inv_freq, out, amplitude: float = 1.0) -> None:
        """``out[t, i] = amplitude * (cos, sin)(inv_freq[i] * positions[t])``."""
        self._dev(positions, inv_freq, out)
        T, half = out.shape[0], out.shape[1]
        if positions.dtype != torch.int32 or positions.numel() != T or inv_freq.dtype != torch.float32 \
                or inv_freq.numel() != half or out.dtype != torch.float32 or not out.is_contiguous() \
                or out.shape[2] != 2:
            raise KernelError("rope_table: shapes or dtypes do not agree")
        self._call("hb_rope_table", positions.data_ptr(), inv_freq.data_ptr(), out.data_ptr(), T, half, float(amplitude),
                   self._stream())
        self.launches += 1

    def rope_kv_append(self, qkv, table, rot: int, heads: int, kv_heads: int, head_dim: int, cache, step,
                       append: bool) -> None:
        self._dev(qkv, table, cache.k, cache.v)
        T = qkv.shape[0]
        need = (heads + (2 * kv_heads if append else 0)) * head_dim
        if qkv.shape[1] < need:
            raise KernelError("rope_kv_append: qkv rows are too short")
        pt = step.page_tables[cache.group]
        if rot and (table is None or table.shape[0] != T or table.shape[1] != rot // 2):
            raise KernelError("rope_kv_append: rotary table does not match the tokens")
        if cache.k.dtype != cache.v.dtype or not cache.k.is_contiguous() or not cache.v.is_contiguous():
            raise KernelError("rope_kv_append: cache layers must be contiguous and of one dtype")
        if tuple(cache.k.shape[1:]) != (kv_heads, 64, head_dim):
            raise KernelError(f"rope_kv_append: cache layer shape {tuple(cache.k.shape)} does not match "
                              f"{kv_heads} kv heads of size {head_dim}")
        self._call("hb_rope_kv_append", qkv.data_ptr(), _code(qkv), _rows(qkv, "qkv"),
                   table.data_ptr() if rot else None, rot, heads, kv_heads, head_dim, cache.k.data_ptr(),
                   cache.v.data_ptr(), _code(cache.k), pt.data_ptr(), pt.shape[1], step.tok_seq.data_ptr(),
                   step.positions.data_ptr(), T, 1 if append else 0, cache.k.shape[0], self.status.data_ptr(),
                   self._stream())
        self.launches += 1

    # ------------------------------------------------------------------ dynamic tanh, short convolution, squared ReLU
    @staticmethod
    def _f32_vec(t, n: int, what: str):
        if t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous():
            raise KernelError(f"{what}: a contiguous float32 tensor of {n} values expected")
        return t.data_ptr()

    def dyt(self, x, weight, bias, alpha, out, rows=None) -> None:
        """``out[r] = tanh(alpha * x[rows[r]]) * weight + bias`` (``rows`` None: every row)."""
        self._dev(x, weight, bias, alpha, out, rows)
        if x.dtype != torch.float32 or not x.is_contiguous():
            raise KernelError("dyt: contiguous float32 input expected")
        C, n = x.shape[1], out.shape[0]
        if out.shape[1] != C or (rows is None and n != x.shape[0]) or (rows is not None and (rows.dtype != torch.int32 or rows.numel() != n)):
            raise KernelError("dyt: shapes do not agree")
        self._call("hb_dyt", x.data_ptr(), self._f32_vec(weight, C, "dyt weight"), self._f32_vec(bias, C, "dyt bias"),
                   self._f32_vec(alpha, 1, "dyt alpha"), out.data_ptr(), _code(out), _rows(out, "dyt output"),
                   rows.data_ptr() if rows is not None else None, n, C, self._stream())
        self.launches += 1

    MAX_TAPS = 16

    def short_conv(self, x, conv_weight, state, step, out, norm=None) -> None:
        """``out = h + conv(h)`` over time per channel, ``conv(h)[t] = sum_j w[:, j] h[t - taps + 1 + j]``; ``state``
        ``[slots, (taps - 1) * C]`` float32 (a view with its own row stride) holds every sequence's last inputs and is
        brought up to date.  ``norm = (weight, bias, alpha)``: ``x`` is the residual stream and ``h = dyt(x)``."""
        self._dev(x, conv_weight, state, out)
        C = x.shape[1]
        taps = conv_weight.shape[1]
        if x.dtype != torch.float32 or not x.is_contiguous() or tuple(out.shape) != tuple(x.shape):
            raise KernelError("short_conv: contiguous float32 input and an output of its shape expected")
        if tuple(conv_weight.shape) != (C, taps) or conv_weight.dtype != torch.float32 or not conv_weight.is_contiguous():
            raise KernelError("short_conv: float32 taps [channels, taps] expected")
        if state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] != (taps - 1) * C or (taps > 1 and state.stride(1) != 1):
            raise KernelError("short_conv: state must be float32 [slots, (taps - 1) * channels]")
        nw = nb = na = None
        if norm is not None:
            nw, nb, na = (self._f32_vec(norm[0], C, "norm weight"), self._f32_vec(norm[1], C, "norm bias"),
                          self._f32_vec(norm[2], 1, "norm alpha"))
        self._call("hb_short_conv", x.data_ptr(), nw, nb, na, conv_weight.data_ptr(), taps, state.data_ptr(), state.stride(0),
                   step.state_slots.data_ptr(), step.seq_start.data_ptr(), out.data_ptr(), _code(out), _rows(out, "short_conv output"),
                   step.num_seqs, step.max_new, C, self._stream())
        self.launches += 1

    def relu2(self, x, out) -> None:
        """``out = max(x, 0)^2``."""
        self._dev(x, out)
        if tuple(x.shape) != tuple(out.shape):
            raise KernelError("relu2: shapes do not agree")
        self._call("hb_relu2", x.data_ptr(), _code(x), _rows(x, "relu2 input"), out.data_ptr(), _code(out), _rows(out, "relu2 output"),
                   x.shape[0], x.shape[1], self._stream())
        self.launches += 1

    # ------------------------------------------------------------------ attention with kept first tokens and mixed heads
    def qkv_prepare(self, proj, bias, table, rot: int, heads: int, kv_heads: int, head_dim: int, v_dim: int, unit_norm: bool,
                    eps: float, q_out, cache, step, append: bool, v_lambda=None, v_first=None, v_mode: int = 0,
                    norm_weights=None, interleaved: bool = False, v_from_k: bool = False) -> None:
        """From a step's projections ``[q | k | v]``: biases added, queries and keys turned by ``table`` and (``unit_norm``)
        divided by their root mean square per head; queries to ``q_out``, keys and values into the cache.  ``norm_weights``
        ``(wq, wk)`` (float32 ``[head_dim]`` each): instead, every head of q and of k is divided by its root mean square and
        multiplied by its weight BEFORE the rotation.  ``v_mode`` 1 also
        keeps the values in ``v_first`` (float32 ``[tokens, kv_heads * v_dim]``), 2 mixes them with it:
        ``v <- (1 - v_lambda) v + v_lambda v_first``.  ``interleaved``: the rotation turns the pairs ``(2i, 2i + 1)`` instead of
        ``(i, i + rot/2)``.  ``v_from_k``: there is no value projection; the values are the keys as projected (with their bias,
        before norm and rotation), and the projections' row is ``[q | k]``."""
        self._dev(proj, bias, table, q_out, cache.k, cache.v, v_lambda, v_first)
        T = proj.shape[0]
        if norm_weights is not None and unit_norm:
            raise KernelError("qkv_prepare: one norm of queries and keys at a time")
        width = heads * head_dim + kv_heads * (head_dim + (0 if v_from_k else v_dim))
        if proj.shape[1] < width or tuple(q_out.shape) != (T, heads * head_dim) or (v_from_k and (v_dim != head_dim or v_mode)):
            raise KernelError("qkv_prepare: shapes do not agree")
        if rot and (table is None or table.shape[0] != T or table.shape[1] != rot // 2):
            raise KernelError("qkv_prepare: rotary table does not match the tokens")
        if tuple(cache.k.shape[1:]) != (kv_heads, 64, head_dim) or tuple(cache.v.shape[1:]) != (kv_heads, 64, v_dim) \
                or not cache.k.is_contiguous() or not cache.v.is_contiguous() or cache.k.dtype != cache.v.dtype:
            raise KernelError("qkv_prepare: cache layer does not match the heads")
        if v_first is not None and (v_first.dtype != torch.float32 or not v_first.is_contiguous() or tuple(v_first.shape) != (T, kv_heads * v_dim)):
            raise KernelError("qkv_prepare: the first values must be contiguous float32 [tokens, kv_heads * v_dim]")
        pt = step.page_tables[cache.group]
        self._call("hb_qkv_prepare", proj.data_ptr(), _code(proj), _rows(proj, "projections"),
                   self._f32_vec(bias, width, "projection bias") if bias is not None else None,
                   table.data_ptr() if rot else None, rot, heads, kv_heads, head_dim, v_dim,
                   2 if norm_weights is not None else 1 if unit_norm else 0,
                   self._f32_vec(norm_weights[0], head_dim, "query norm weight") if norm_weights is not None else None,
                   self._f32_vec(norm_weights[1], head_dim, "key norm weight") if norm_weights is not None else None, float(eps),
                   q_out.data_ptr(), _code(q_out), _rows(q_out, "queries"), cache.k.data_ptr(), cache.v.data_ptr(), _code(cache.k),
                   pt.data_ptr(), pt.shape[1], step.tok_seq.data_ptr(), step.positions.data_ptr(), T, cache.k.shape[0],
                   1 if append else 0, self._f32_vec(v_lambda, 1, "value mix") if v_lambda is not None else None,
                   v_first.data_ptr() if v_first is not None else None, int(v_mode), 1 if interleaved else 0, 1 if v_from_k else 0,
                   self.status.data_ptr(), self._stream())
        self.launches += 1

    def attention_sink(self, q, heads: int, kv_heads: int, head_dim: int, v_dim: int, cache, step, partial, scale: float,
                       window: Optional[int], keep_first: int, all_values: bool, chunk: int = 0, sink=None) -> None:
        """Causal attention where a query at position p sees key s if ``p - s < window`` or ``s < keep_first``
        (``window`` None: every earlier key); with ``chunk`` instead, if s lies in p's own run of ``chunk`` positions (runs
        counted from the sequence's start).  ``sink`` float32 ``[heads]``: the softmax's sum holds ``exp(sink[h])`` once more.  ``partial`` float32 ``[tokens, heads, kv_heads if all_values else 1,
        v_dim]``: each head's softmax weights applied to the values of every key/value head, or of its own."""
        self._dev(q, cache.k, cache.v, partial)
        T = q.shape[0]
        n_val = kv_heads if all_values else 1
        if partial.dtype != torch.float32 or not partial.is_contiguous() or partial.numel() != T * heads * n_val * v_dim:
            raise KernelError("attention_sink: partial results must be contiguous float32 [tokens, heads, value heads, v_dim]")
        if tuple(cache.k.shape[1:]) != (kv_heads, 64, head_dim) or tuple(cache.v.shape[1:]) != (kv_heads, 64, v_dim):
            raise KernelError("attention_sink: cache layer does not match the heads")
        pt = step.page_tables[cache.group]
        self._call("hb_attention_sink", q.data_ptr(), _code(q), _rows(q, "queries"), cache.k.data_ptr(), cache.v.data_ptr(),
                   _code(cache.k), pt.data_ptr(), pt.shape[1], step.tok_seq.data_ptr(), step.positions.data_ptr(),
                   partial.data_ptr(), T, heads, kv_heads, head_dim, v_dim, float(scale), int(window) if window and not chunk else 0,
                   int(keep_first), int(chunk), self._f32_vec(sink, heads, "sink") if sink is not None else None,
                   1 if all_values else 0, cache.k.shape[0], self.status.data_ptr(), self._stream())
        self.launches += 1

    def _head_gate(self, gate, T: int, heads: int):
        """Pointer and row stride of a per-(token, head) gate, float32 ``[tokens, heads]`` with contiguous rows, or (None, 0)."""
        if gate is None:
            return None, 0
        if gate.dtype != torch.float32 or tuple(gate.shape) != (T, heads):
            raise KernelError("head gate: float32 [tokens, heads] expected")
        return gate.data_ptr(), _rows(gate, "head gate")

    def head_mix(self, partial, mix, out, heads: int, kv_heads: int, v_dim: int, n_val: int, ones: int = 0, gate=None) -> None:
        """``out[t, h] = sum_g mix[h, g] partial[t, g, kv(h)]`` (``mix`` None: the head's own); ``ones`` more columns
        (a one, then zeros) follow, through which the next product adds a bias stored as a column of its weight.  ``gate``
        float32 ``[tokens, heads]``: head h's result is multiplied by ``sigmoid(gate[t, h])``."""
        self._dev(partial, mix, out, gate)
        T = out.shape[0]
        if out.shape[1] != heads * v_dim + ones or partial.numel() != T * heads * n_val * v_dim:
            raise KernelError("head_mix: shapes do not agree")
        self._call("hb_head_mix", partial.data_ptr(), self._f32_vec(mix, heads * heads, "head mix") if mix is not None else None,
                   out.data_ptr(), _code(out), _rows(out, "head_mix output"), T, heads, kv_heads, v_dim, n_val, ones,
                   *self._head_gate(gate, T, heads), self._stream())
        self.launches += 1

    SINK_PREFILL_FROM = 16          # steps whose longest portion has at least so many tokens run the flash-style kernel

    def attention_sink_prefill_wanted(self, step, heads: int, kv_heads: int, head_dim: int, v_dim: int, dtype) -> bool:
        """Whether ``attention_sink_prefill`` takes this step: bfloat16, head sizes it is built for, a portion of
        ``SINK_PREFILL_FROM`` tokens or more (64 query tokens share a block; fewer tokens are better cut over the keys)."""
        return bool(self.use_flash_sink_attention and dtype == torch.bfloat16 and not step.is_decode
                    and step.max_new >= self.SINK_PREFILL_FROM
                    and self.lib.hb_attention_sink_prefill_supported(heads, kv_heads, head_dim, v_dim)
                    and sum((n + 63) // 64 for n in step.host_new) <= 65535)

    def attention_sink_prefill(self, q, heads: int, kv_heads: int, head_dim: int, v_dim: int, cache, step, partial, scale: float,
                               window: Optional[int], keep_first: int, all_values: bool, chunk: int = 0, sink=None) -> None:
        """``attention_sink`` on the tensor cores, 64 query tokens of a sequence per block: ``partial`` float32
        ``[tokens, heads, kv_heads if all_values else 1, v_dim]``, normalised."""
        self._dev(q, cache.k, cache.v, partial)
        T = q.shape[0]
        n_val = kv_heads if all_values else 1
        if q.dtype != torch.bfloat16 or cache.k.dtype != torch.bfloat16 or partial.dtype != torch.float32 or not partial.is_contiguous() \
                or partial.numel() != T * heads * n_val * v_dim:
            raise KernelError("attention_sink_prefill: bfloat16 queries and cache, float32 [tokens, heads, value heads, v_dim] expected")
        if tuple(cache.k.shape[1:]) != (kv_heads, 64, head_dim) or tuple(cache.v.shape[1:]) != (kv_heads, 64, v_dim):
            raise KernelError("attention_sink_prefill: cache layer does not match the heads")
        pt = step.page_tables[cache.group]
        q_blocks = sum((n + 63) // 64 for n in step.host_new)
        self._call("hb_attention_sink_prefill", q.data_ptr(), _rows(q, "queries"), cache.k.data_ptr(), cache.v.data_ptr(), pt.data_ptr(),
                   pt.shape[1], step.seq_start.data_ptr(), step.seq_pos0.data_ptr(), partial.data_ptr(), step.num_seqs, q_blocks,
                   heads, kv_heads, head_dim, v_dim, n_val, float(scale), int(window) if window and not chunk else 0, int(keep_first),
                   int(chunk), self._f32_vec(sink, heads, "sink") if sink is not None else None,
                   cache.k.shape[0], self.status.data_ptr(), self._stream())
        self.launches += 1

    ATTENTION_HEADS_MAX_ROWS = 512      # tokens x key splits of a step that has fewer tokens than the device has SMs

    def attention_heads_whole(self, heads: int, kv_heads: int, head_dim: int, v_dim: int, dtype) -> bool:
        """Whether a block of ``attention_heads`` holds every head of its value columns in one place (it can then mix the
        heads and write the output itself when the keys are not split)."""
        return bool(self.lib.hb_attention_heads_writes_output(heads, kv_heads, head_dim, v_dim, _DTYPE_CODE[dtype],
                                                              1 if self.use_mma_attention else 0))

    def attention_heads_plan(self, tokens: int, heads: int, kv_heads: int, head_dim: int, v_dim: int, dtype, longest: int):
        """How ``attention_heads`` would run a step, or None when its kernel is not built for these sizes:
        ``(splits, writes_output)``.  Few tokens are cut over the keys (``longest``: the most keys a token sees) so that
        the device is busy; a step of many tokens with every head of a value column in one thread writes the mixed
        output itself."""
        if not self.lib.hb_attention_heads_variant(heads, kv_heads, head_dim, v_dim, _DTYPE_CODE[dtype], 1 if self.use_mma_attention else 0):
            return None
        whole = self.attention_heads_whole(heads, kv_heads, head_dim, v_dim, dtype)
        # the kernel that combines the splits keeps [heads, splits + 32] floats in 48 KB of shared memory
        most = (48 * 1024 // 4 - heads * 32) // heads
        if most < 1 and not whole:
            return None
        splits = 1
        if tokens < self.sm_count:
            splits = max(1, min(-(-self.sm_count // tokens), longest // 64, 32, most))
        return splits, (splits == 1 and whole)

    def attention_heads(self, q, heads: int, kv_heads: int, head_dim: int, v_dim: int, cache, step, scale: float, window: Optional[int],
                        keep_first: int, splits: int, mix=None, out=None, ones: int = 0, partial=None, ml=None, chunk: int = 0,
                        sink=None) -> None:
        """The attention of ``attention_sink`` with one block per (token, key split) for all heads (each head's weights on
        the values of every key/value head).  With ``out`` (one split): the normalised, head-mixed output and ``ones``
        more columns (a one, then zeros).  Else ``partial`` float32 ``[tokens, heads, splits, kv_heads * v_dim]``
        unnormalised and ``ml`` ``[tokens, heads, splits, 2]`` (maximum, sum) for ``head_mix_splits``."""
        self._dev(q, cache.k, cache.v, out, partial, ml, mix)
        T = q.shape[0]
        if tuple(cache.k.shape[1:]) != (kv_heads, 64, head_dim) or tuple(cache.v.shape[1:]) != (kv_heads, 64, v_dim):
            raise KernelError("attention_heads: cache layer does not match the heads")
        if out is not None and (out.shape[0] != T or out.shape[1] != heads * v_dim + ones):
            raise KernelError("attention_heads: output shape does not match")
        if out is None and (partial is None or ml is None or partial.dtype != torch.float32 or ml.dtype != torch.float32
                            or partial.numel() < T * heads * splits * kv_heads * v_dim or ml.numel() < T * heads * splits * 2):
            raise KernelError("attention_heads: partial results need float32 [tokens, heads, splits, kv_heads * v_dim] and [.., 2]")
        pt = step.page_tables[cache.group]
        self._call("hb_attention_heads", q.data_ptr(), _code(q), _rows(q, "queries"), cache.k.data_ptr(), cache.v.data_ptr(),
                   _code(cache.k), pt.data_ptr(), pt.shape[1], step.tok_seq.data_ptr(), step.positions.data_ptr(),
                   partial.data_ptr() if partial is not None else None, ml.data_ptr() if ml is not None else None,
                   self._f32_vec(mix, heads * heads, "head mix") if mix is not None else None,
                   out.data_ptr() if out is not None else None, _rows(out, "attention output") if out is not None else 0, ones,
                   T, heads, kv_heads, head_dim, v_dim, float(scale), int(window) if window and not chunk else 0, int(keep_first),
                   int(chunk), self._f32_vec(sink, heads, "sink") if sink is not None else None, int(splits),
                   cache.k.shape[0], 1 if self.use_mma_attention else 0, self.status.data_ptr(), self._stream())
        self.launches += 1

    def head_mix_splits(self, partial, ml, mix, out, heads: int, kv_heads: int, v_dim: int, splits: int, ones: int = 0, gate=None) -> None:
        """Combines the key splits of ``attention_heads`` and mixes the heads (``mix`` None: each head its own).  ``ml`` None:
        one split, normalised already (``partial`` is then ``[tokens, heads, kv_heads, v_dim]``)."""
        self._dev(partial, ml, mix, out, gate)
        T = out.shape[0]
        if out.shape[1] != heads * v_dim + ones:
            raise KernelError("head_mix_splits: shapes do not agree")
        self._call("hb_head_mix_splits", partial.data_ptr(), ml.data_ptr() if ml is not None else None,
                   self._f32_vec(mix, heads * heads, "head mix") if mix is not None else None, out.data_ptr(), _code(out),
                   _rows(out, "head_mix output"), T, heads, kv_heads, v_dim, splits, ones, *self._head_gate(gate, T, heads), self._stream())
        self.launches += 1

    # ------------------------------------------------------------------ matrix memory (mLSTM)
    MLSTM_CHUNK_FROM = 8           # steps whose longest portion has at least so many tokens run the chunked kernel

    def mlstm_scan(self, proj, gate_bias, cap: float, q_scale: float, state, step, out, heads: int, d: int, dv: int,
                   chunked: Optional[bool] = None) -> None:
        """The matrix memory over a step's tokens, sequence by sequence (token by token, or with ``chunked``, default for
        steps that bring ``MLSTM_CHUNK_FROM`` tokens or more to a sequence, 32 tokens at a time): ``proj`` float32 rows
        ``[q | k | v | gate | z_i | z_f]``, ``state`` float32 ``[slots, heads*d*dv + heads*d + heads]`` (S, n, m),
        ``out`` float32 ``[tokens, heads * dv]``."""
        self._dev(proj, gate_bias, state, out)
        T = proj.shape[0]
        width = 2 * heads * d + 2 * heads * dv + 2 * heads
        if proj.dtype != torch.float32 or proj.shape[1] < width or out.dtype != torch.float32 or not out.is_contiguous() \
                or tuple(out.shape) != (T, heads * dv):
            raise KernelError("mlstm_scan: float32 projections [tokens, 2*heads*d + 2*heads*dv + 2*heads] and float32 output expected")
        if state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] != heads * d * dv + heads * d + heads or state.stride(1) != 1:
            raise KernelError("mlstm_scan: state must be float32 [slots, heads*d*dv + heads*d + heads]")
        if chunked is None:
            chunked = step.max_new >= self.MLSTM_CHUNK_FROM
        self._call("hb_mlstm_chunks" if chunked else "hb_mlstm_scan", proj.data_ptr(), _code(proj), _rows(proj, "projections"),
                   self._f32_vec(gate_bias, 2 * heads, "gate bias") if gate_bias is not None else None, float(cap), float(q_scale),
                   state.data_ptr(), state.stride(0), step.state_slots.data_ptr(), step.seq_start.data_ptr(), out.data_ptr(),
                   step.num_seqs, heads, d, dv, self._stream())
        self.launches += 1

    def mlstm_output(self, o, gate, weight, eps: float, out, heads: int, dv: int) -> None:
        """``out = o / rms(o per head) * weight * sigmoid(gate)``; ``gate`` a column view of the projections."""
        self._dev(o, gate, weight, out)
        T = o.shape[0]
        if o.dtype != torch.float32 or not o.is_contiguous() or tuple(gate.shape) != (T, heads * dv) or tuple(out.shape) != (T, heads * dv):
            raise KernelError("mlstm_output: shapes do not agree")
        self._call("hb_mlstm_output", o.data_ptr(), gate.data_ptr(), _code(gate), _rows(gate, "gate"),
                   self._f32_vec(weight, heads * dv, "mlstm norm weight"), float(eps), out.data_ptr(), _code(out),
                   _rows(out, "mlstm output"), T, heads, dv, self._stream())
        self.launches += 1

    STATUS_WORDS = 4

    @staticmethod
    def status_message(words) -> Optional[str]:
        """What the status words say, or None if all are zero."""
        w = [int(x) for x in words]
        if not any(w):
            return None
        parts = []
        if w[0]:
            parts.append(f"a tensor-core kernel gave up a bounded wait (code {w[0]}); its results are invalid")
        if w[1]:
            parts.append(f"non-finite logits at row {w[1] - 1} of a step (the reference fails such a row too)")
        if w[2]:
            parts.append(f"a page number outside the cache, or a missing page, for sequence {w[2] - 1} of a step: "
                         "the cache's bookkeeping is at fault")
        if w[3]:
            parts.append(f"a token id outside the vocabulary at row {w[3] - 1} of a step")
        return "; ".join(parts)

    def raise_on_status(self, words) -> None:
        """Raises ``KernelError`` for non-zero status words that were read already (a host copy),
        after clearing the device's words and the split-K counters a kernel that gave up may have
        left non-zero."""
        msg = self.status_message(words)
        if msg is not None:
            self.reset_status()
            raise KernelError(msg)

    def reset_status(self) -> None:
        self.status.zero_()
        self._splitk_counters.zero_()
        self._decode_counters.zero_()
        self._argmax_counters.zero_()

    def check_errors(self) -> None:
        """Reads the device status words (this synchronises) and raises if a kernel noted a fault."""
        self.raise_on_status(self.status.tolist())

    # ------------------------------------------------------------------ matrix products
    def pack_weight(self, w: torch.Tensor, swiglu: bool = False):
        """``w`` as a PackedWeight when the tensor-core products can read it that way (bfloat16
        on this device, rows of a multiple of 8 elements; a [gate; up] matrix needs halves of a
        multiple of 64 rows), else ``w`` itself."""
        if (not self.use_packed_weights or not isinstance(w, torch.Tensor) or w.dtype != torch.bfloat16 or w.dim() != 2
                or w.device != self.device or w.shape[1] % 8 or (swiglu and (w.shape[0] // 2) % 64)):
            return w
        return PackedWeight.pack(w, gate_up_bands=swiglu)

    def _tensor_core_operands(self, a, w) -> bool:
        if not (self.use_tensor_cores and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
                and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and _rows(a, "linear input") % 8 == 0):
            return False
        return isinstance(w, PackedWeight) or _rows(w, "linear weight") % 8 == 0

    SCHEDULES = {None: 0, "auto": 0, "tiles": 1, "stream_k": 2, "cut_first": 3}

    def _gemm_tc(self, a, w, out, mode: int, N: int, up_row0: int = 0, schedule=None, fold=None) -> None:
        M, K = a.shape
        packed = 1 if isinstance(w, PackedWeight) else 0
        ldw = 64 if packed else _rows(w, "linear weight")
        if fold is None and (schedule == "pairs" or (schedule is None and self.use_pair_gemm and self.lib.hb_gemm_tc2_wanted(M, N, K)
                                                     and not (mode == 3 and N % 8))):
            # many tokens: CTA pairs (cta_group::2) on 256 x 256 tiles
            self._call("hb_gemm_tc2", a.data_ptr(), _rows(a, "linear input"), w.data_ptr(), ldw, w.shape[0], out.data_ptr(),
                       _rows(out, "linear output"), M, N, K, mode, up_row0, self.error_flag.data_ptr(), packed, self._stream())
            self.launches += 1
            return
        sched = self.SCHEDULES[schedule]
        need = self.lib.hb_gemm_tc_scratch_floats(M, N, K, mode, sched)
        tiles = self.lib.hb_gemm_tc_tiles(M, N, mode)
        if need > self._splitk_partials.numel():
            self._retired.append(self._splitk_partials)     # a captured graph may still write there
            self._splitk_partials = torch.empty(need, dtype=torch.float32, device=self.device)
        if tiles > self._splitk_counters.numel():
            self._retired.append(self._splitk_counters)
            self._splitk_counters = torch.zeros(tiles, dtype=torch.int32, device=self.device)
        args = (a.data_ptr(), _rows(a, "linear input"), w.data_ptr(), ldw,
                w.shape[0], out.data_ptr(), _rows(out, "linear output"), M, N, K, mode, up_row0, sched,
                self._splitk_partials.data_ptr(), self._splitk_partials.numel(), self._splitk_counters.data_ptr(),
                self._splitk_counters.numel(), self.error_flag.data_ptr(), packed)
        if fold is None:
            self._call("hb_gemm_tc", *args, self._stream())
        else:
            self._call("hb_gemm_tc_fold", *args, ctypes.byref(fold), self._stream())    # the library copies the values
        self.launches += 1

    # ------------------------------------------------------------------ a norm folded into the products around it
    FOLD_MAX_TOKENS = 32           # TC_SCALE_ROWS of csrc/tcgen05.cuh: beyond, norm kernels are as fast or faster

    def can_fold_norm(self, tokens: int, size: int, dtype: torch.dtype) -> bool:
        """Whether a step of ``tokens`` tokens may fold a norm over vectors of ``size`` into the
        products around it: few tokens (the few-token tensor-core kernel), bfloat16 activations."""
        return bool(self.fold_norms and self.use_tensor_cores and dtype == torch.bfloat16 and 0 < tokens <= self.FOLD_MAX_TOKENS
                    and size % 8 == 0)

    def _sumsq_buffer(self, size: int) -> torch.Tensor:
        ld = (-(-size // 32) + 3) // 4 * 4
        if self._sumsq is None or self._sumsq.shape[1] < ld:
            if self._sumsq is not None:
                self._retired.append(self._sumsq)            # a captured graph may still write there
            self._sumsq = torch.zeros(self.FOLD_MAX_TOKENS, ld, dtype=torch.float32, device=self.device)
        return self._sumsq

    def _prepare_fold(self, out, prepare) -> Optional[_NormFold]:
        """The producer's half of HbNormFold, or None when this product cannot prepare the norm."""
        weight, offset, eps, h_out = prepare
        M, N = out.shape
        if not (self.can_fold_norm(M, N, h_out.dtype) and out.dtype == torch.float32 and out.data_ptr() % 16 == 0
                and _rows(out, "linear output") % 4 == 0 and weight.dtype == torch.float32 and weight.numel() == N
                and weight.data_ptr() % 16 == 0 and tuple(h_out.shape) == (M, N) and h_out.data_ptr() % 8 == 0
                and _rows(h_out, "norm output") % 4 == 0):
            return None
        sumsq = self._sumsq_buffer(N)
        fold = _NormFold()
        fold.prep_w, fold.prep_offset, fold.prep_out = weight.data_ptr(), float(offset), h_out.data_ptr()
        fold.prep_ld, fold.prep_sumsq, fold.sumsq_ld = _rows(h_out, "norm output"), sumsq.data_ptr(), sumsq.shape[1]
        return fold

    def _scale_fold(self, scale: PreparedNorm, tokens: int) -> _NormFold:
        if tokens > self.FOLD_MAX_TOKENS:
            raise KernelError(f"a prepared norm serves up to {self.FOLD_MAX_TOKENS} tokens, not {tokens}")
        fold = _NormFold()
        fold.scale_sumsq, fold.scale_parts, fold.sumsq_ld = scale.sumsq.data_ptr(), scale.parts, scale.sumsq.shape[1]
        fold.scale_inv_size, fold.scale_eps = 1.0 / scale.size, scale.eps
        return fold

    def linear(self, a, w, out, accumulate: bool = False, schedule=None, prepare=None, scale: Optional[PreparedNorm] = None):
        """``out[M,N] (+)= a[M,K] @ w[N,K]^T`` with float32 accumulation.  ``schedule`` forces
        the tensor-core kernel's work split ("tiles" or "stream_k"; default: by shape).

        A norm folded into the products around it (few tokens, bfloat16): with ``accumulate`` and
        ``prepare = (norm weight, offset, eps, buffer)`` the product also fills ``buffer`` with
        ``out * (offset + weight)`` and returns a ``PreparedNorm`` (None when it cannot: the
        caller then runs the norm).  ``scale``: ``a`` is such a buffer; the rows of the result are
        multiplied by the norm's per-token factor."""
        self._dev(a, w, out)
        M, K = a.shape
        N = w.shape[0]
        if w.shape[1] != K or tuple(out.shape) != (M, N):
            raise KernelError(f"linear: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} do not agree")
        if isinstance(w, PackedWeight) and w.gate_up_bands:
            raise KernelError("linear: a [gate; up] matrix stored in bands is an operand of linear_swiglu only")
        if self._tensor_core_operands(a, w) and (out.dtype == torch.float32 or not accumulate):
            mode = 2 if accumulate else (1 if out.dtype == torch.float32 else 0)
            fold = None
            if prepare is not None and accumulate and schedule != "pairs":
                fold = self._prepare_fold(out, prepare)
            if scale is not None:
                if accumulate:
                    raise KernelError("linear: the product that adds to the residual does not scale its rows")
                fold = self._scale_fold(scale, M)
            self._gemm_tc(a, w, out, mode, N, 0, schedule, fold=fold)
            if fold is not None and scale is None:
                return PreparedNorm(self._sumsq, -(-N // 32), N, prepare[2])
            return None
        if scale is not None:
            raise KernelError("linear: operands that the tensor-core product refuses cannot take a prepared norm")
        if isinstance(w, PackedWeight):
            w = w.unpacked()           # not a product path: only operands the tensor-core kernels refuse get here
        self._call("hb_gemm_general", a.data_ptr(), _code(a), _rows(a, "linear input"), w.data_ptr(), _code(w),
                   _rows(w, "linear weight"), out.data_ptr(), _code(out), _rows(out, "linear output"), M, N, K,
                   1 if accumulate else 0, self._stream())
        self.launches += 1

    def linear_swiglu(self, h, w_gate_up, act, workspace, cap: int, schedule=None, scale: Optional[PreparedNorm] = None) -> None:
        """``act = silu(h Wg^T) * (h Wu^T)`` with ``w_gate_up = [Wg; Wu]``; ``scale`` as in ``linear``."""
        T = h.shape[0]
        inter = act.shape[1]
        if w_gate_up.shape[0] != 2 * inter or act.shape[0] != T:
            raise KernelError("linear_swiglu: weight must be [2 * inter, hidden]")
        if (self._tensor_core_operands(h, w_gate_up) and act.dtype == torch.bfloat16 and act.data_ptr() % 16 == 0
                and _rows(act, "swiglu output") % 8 == 0):
            bands = isinstance(w_gate_up, PackedWeight) and w_gate_up.gate_up_bands
            self._gemm_tc(h, w_gate_up, act, 3, inter, up_row0=-1 if bands else inter, schedule=schedule,
                          fold=self._scale_fold(scale, T) if scale is not None else None)
            return
        if scale is not None:
            raise KernelError("linear_swiglu: operands that the tensor-core product refuses cannot take a prepared norm")
        if isinstance(w_gate_up, PackedWeight):
            w_gate_up = w_gate_up.unpacked()
        gu = workspace.buffer("swiglu.gate_up", (cap, 2 * inter), torch.float32 if act.dtype == torch.float32
                              else torch.bfloat16)[:T]
        self.linear(h, w_gate_up, gu)
        self.silu_mul(gu, act)

    # ------------------------------------------------------------------ attention
    def decode_splits_for(self, batch: int, kv_heads: int, max_pages: int, head_dim: int = 128) -> int:
        """Key splits of decode attention (``plan.decode_splits``) for this device: the CTAs it
        holds at once are the kernel's CTAs per SM (two at head size 128) times its SMs."""
        key = (batch, kv_heads, max_pages, head_dim)
        hit = self._splits_cache.get(key)
        if hit is None:
            slots = self.sm_count * max(1, self.lib.hb_attention_decode_ctas_per_sm(head_dim) or 2)
            hit = self._splits_cache[key] = decode_splits(batch, kv_heads, max_pages, slots)
        return hit

    def can_fuse_decode_attention(self, qkv, heads: int, kv_heads: int, head_dim: int, cache, step, out) -> bool:
        """Whether ``attention_decode_fused`` takes this step: one token per sequence,
        bfloat16 everywhere, a head size and group the tensor-core kernel is built for."""
        return bool(self.fuse_decode_attention and self.use_fast_attention and step.is_decode
                    and qkv.dtype == torch.bfloat16
                    and cache.k.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
                    and cache.k.is_contiguous() and cache.v.is_contiguous()
                    and step.num_tokens * kv_heads <= self._decode_counters.numel()
                    and self.lib.hb_attention_decode_supported(heads, kv_heads, head_dim))

    def attention_decode_fused(self, qkv, table, rot: int, heads: int, kv_heads: int, head_dim: int, cache, step, out,
                               scale: float, window: Optional[int], append: bool, splits: Optional[int] = None) -> None:
        """Rotation of the new tokens' queries and keys, cache append and split-K attention in
        one launch (decode steps only); the combination of the splits is a second kernel, or
        with ``combine_in_attention`` the work of the last split to finish.  ``qkv`` holds
        the projections before rotation and is not written."""
        self._dev(qkv, table, cache.k, cache.v, out)
        T = qkv.shape[0]
        pt = step.page_tables[cache.group]
        if out.shape[0] != T or out.shape[1] != heads * head_dim:
            raise KernelError("attention: output shape does not match")
        if rot and (table is None or table.shape[0] != T or table.shape[1] != rot // 2):
            raise KernelError("attention: rotary table does not match the tokens")
        if tuple(cache.k.shape[1:]) != (kv_heads, 64, head_dim):
            raise KernelError("attention: cache layer shape does not match the heads")
        max_pages = (step.max_len + 63) // 64
        n_splits = splits if splits is not None else self.decode_splits_for(T, kv_heads, max_pages, head_dim)
        n_splits = max(1, min(n_splits, max_pages))
        need = self.lib.hb_attention_decode_scratch_floats(T, heads, head_dim, n_splits)
        if need > self._decode_scratch.numel():
            self._retired.append(self._decode_scratch)
            self._decode_scratch = torch.empty(need, dtype=torch.float32, device=self.device)
        self._call("hb_attention_decode_fused", qkv.data_ptr(), _rows(qkv, "attention projections"),
                   table.data_ptr() if rot else None, rot, cache.k.data_ptr(), cache.v.data_ptr(), pt.data_ptr(),
                   pt.shape[1], step.positions.data_ptr(), self._decode_scratch.data_ptr(),
                   self._decode_counters.data_ptr() if self.combine_in_attention else None,
                   out.data_ptr(), _rows(out, "attention output"), T, heads, kv_heads,
                   head_dim, float(scale), int(window) if window else 0, n_splits, max_pages, cache.k.shape[0],
                   1 if append else 0, self.status.data_ptr(), self._stream())
        self.launches += 1 if (n_splits == 1 or self.combine_in_attention) else 2

    def attention(self, qkv, heads: int, kv_heads: int, head_dim: int, cache, step, out, scale: float,
                  window: Optional[int], splits: Optional[int] = None) -> None:
        """Causal attention of the step's tokens over the cache; queries are the first
        ``heads * head_dim`` columns of ``qkv``.  bfloat16 with head size 64 or 128 runs the
        tensor-core kernels (split-K for one token per sequence, flash-style otherwise);
        everything else runs the general kernel."""
        self._dev(qkv, cache.k, cache.v, out)
        T = qkv.shape[0]
        pt = step.page_tables[cache.group]
        if out.shape[0] != T or out.shape[1] != heads * head_dim:
            raise KernelError("attention: output shape does not match")
        win = int(window) if window else 0
        fast = (self.use_fast_attention and qkv.dtype == torch.bfloat16 and cache.k.dtype == torch.bfloat16
                and out.dtype == torch.bfloat16 and cache.k.is_contiguous() and cache.v.is_contiguous())
        if fast and step.is_decode and self.lib.hb_attention_decode_supported(heads, kv_heads, head_dim):
            max_pages = (step.max_len + 63) // 64
            n_splits = splits if splits is not None else self.decode_splits_for(T, kv_heads, max_pages, head_dim)
            n_splits = max(1, min(n_splits, max_pages))
            need = self.lib.hb_attention_decode_scratch_floats(T, heads, head_dim, n_splits)
            if need > self._decode_scratch.numel():
                self._retired.append(self._decode_scratch)
                self._decode_scratch = torch.empty(need, dtype=torch.float32, device=self.device)
            if ((n_splits == 1 or self.combine_in_attention) and n_splits <= 16
                    and T * kv_heads <= self._decode_counters.numel()):
                # one split writes the result itself; with more, the last split of a (sequence, kv
                # head) to finish can combine them (a switch: measured slower than the second kernel)
                self._call("hb_attention_decode_combined", qkv.data_ptr(), _rows(qkv, "attention queries"), cache.k.data_ptr(),
                           cache.v.data_ptr(), pt.data_ptr(), pt.shape[1], step.positions.data_ptr(),
                           self._decode_scratch.data_ptr(), self._decode_counters.data_ptr(), out.data_ptr(),
                           _rows(out, "attention output"), T, heads, kv_heads, head_dim, float(scale), win, n_splits, max_pages,
                           cache.k.shape[0], self.status.data_ptr(), self._stream())
                self.launches += 1
                return
            self._call("hb_attention_decode", qkv.data_ptr(), _rows(qkv, "attention queries"), cache.k.data_ptr(),
                       cache.v.data_ptr(), pt.data_ptr(), pt.shape[1], step.positions.data_ptr(),
                       self._decode_scratch.data_ptr(), out.data_ptr(), _rows(out, "attention output"), T, heads, kv_heads,
                       head_dim, float(scale), win, n_splits, max_pages, cache.k.shape[0], self.status.data_ptr(),
                       self._stream())
            self.launches += 2
            return
        if (fast and self.use_tcgen05_attention and self.lib.hb_attention_prefill_tc_supported(heads, kv_heads, head_dim)
                and qkv.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0 and _rows(qkv, "attention queries") % 8 == 0
                and _rows(out, "attention output") % 8 == 0
                and sum((n + 127) // 128 for n in step.host_new) <= 65535):
            q_blocks = sum((n + 127) // 128 for n in step.host_new)
            self._call("hb_attention_prefill_tc", qkv.data_ptr(), _rows(qkv, "attention queries"), T, cache.k.data_ptr(),
                       cache.v.data_ptr(), pt.data_ptr(), pt.shape[1], step.seq_start.data_ptr(), step.seq_pos0.data_ptr(),
                       out.data_ptr(), _rows(out, "attention output"), step.num_seqs, q_blocks, heads, kv_heads, head_dim,
                       float(scale), win, cache.k.shape[0], self.error_flag.data_ptr(), self._stream())
            self.launches += 1
            return
        if (fast and self.lib.hb_attention_prefill_supported(heads, kv_heads, head_dim)
                and sum((n + 63) // 64 for n in step.host_new) <= 65535):
            q_blocks = sum((n + 63) // 64 for n in step.host_new)
            self._call("hb_attention_prefill", qkv.data_ptr(), _rows(qkv, "attention queries"), cache.k.data_ptr(),
                       cache.v.data_ptr(), pt.data_ptr(), pt.shape[1], step.seq_start.data_ptr(), step.seq_pos0.data_ptr(),
                       out.data_ptr(), _rows(out, "attention output"), step.num_seqs, q_blocks, heads, kv_heads, head_dim,
                       float(scale), win, cache.k.shape[0], self.status.data_ptr(), self._stream())
            self.launches += 1
            return
        self._call("hb_attention_general", qkv.data_ptr(), _code(qkv), _rows(qkv, "attention queries"),
                   cache.k.data_ptr(), cache.v.data_ptr(), _code(cache.k), pt.data_ptr(), pt.shape[1],
                   step.tok_seq.data_ptr(), step.positions.data_ptr(), out.data_ptr(), _code(out),
                   _rows(out, "attention output"), T, heads, kv_heads, head_dim, float(scale), win, cache.k.shape[0],
                   self.status.data_ptr(), self._stream())
        self.launches += 1

    # ------------------------------------------------------------------ norms on a sublayer's output
    def rmsnorm_add(self, y, weight, eps: float, offset: float, x, then=None, then_out=None) -> None:
        """``x += y / sqrt(mean(y^2) + eps) * (offset + weight)`` row by row in 32-bit; with ``then = (weight2, eps2,
        offset2)`` and ``then_out`` also ``then_out = x / sqrt(mean(x^2) + eps2) * (offset2 + weight2)`` of the new rows."""
        self._dev(y, weight, x, then_out)
        T, n = x.shape
        if y.dtype != torch.float32 or x.dtype != torch.float32 or tuple(y.shape) != (T, n) or (then is None) != (then_out is None):
            raise KernelError("rmsnorm_add: float32 [tokens, width] input and residual expected")
        w2 = e2 = o2 = None
        if then is not None:
            w2, e2, o2 = then
            if tuple(then_out.shape) != (T, n):
                raise KernelError("rmsnorm_add: the second norm's output does not match")
        self._call("hb_rmsnorm_add", y.data_ptr(), _rows(y, "rmsnorm_add input"), self._f32_vec(weight, n, "norm weight"), float(eps),
                   float(offset), x.data_ptr(), _rows(x, "residual"), self._f32_vec(w2, n, "norm weight") if then is not None else None,
                   float(e2 or 0.0), float(o2 or 0.0), then_out.data_ptr() if then is not None else None,
                   _code(then_out) if then is not None else 0, _rows(then_out, "norm output") if then is not None else 0, T, n,
                   self._stream())
        self.launches += 1

    def scaled_sum(self, a, sa: float, b, sb: float, out) -> None:
        """``out = sa * a + sb * b`` over contiguous float32 tensors of one shape (``out`` may be ``a`` or ``b``)."""
        self._dev(a, b, out)
        if any(t.dtype != torch.float32 or not t.is_contiguous() or t.shape != out.shape for t in (a, b, out)):
            raise KernelError("scaled_sum: contiguous float32 tensors of one shape expected")
        self._call("hb_scaled_sum", a.data_ptr(), float(sa), b.data_ptr(), float(sb), out.data_ptr(), out.numel(), self._stream())
        self.launches += 1

    def scaled_add_norm(self, y, m: float, x, then=None, then_out=None) -> None:
        """``x += m * y`` row by row in 32-bit; with ``then = (weight, eps, offset)`` and ``then_out`` also ``then_out = x /
        sqrt(mean(x^2) + eps) * (offset + weight)`` of the new rows, in the same pass."""
        self._dev(y, x, then_out)
        T, n = x.shape
        if y.dtype != torch.float32 or x.dtype != torch.float32 or tuple(y.shape) != (T, n) or (then is None) != (then_out is None):
            raise KernelError("scaled_add_norm: float32 [tokens, width] input and residual expected")
        w2 = e2 = o2 = None
        if then is not None:
            w2, e2, o2 = then
            if tuple(then_out.shape) != (T, n):
                raise KernelError("scaled_add_norm: the norm's output does not match")
        self._call("hb_scaled_add_norm", y.data_ptr(), _rows(y, "sublayer result"), float(m), x.data_ptr(), _rows(x, "residual"),
                   self._f32_vec(w2, n, "norm weight") if then is not None else None, float(e2 or 0.0), float(o2 or 0.0),
                   then_out.data_ptr() if then is not None else None, _code(then_out) if then is not None else 0,
                   _rows(then_out, "norm output") if then is not None else 0, T, n, self._stream())
        self.launches += 1

    def normed_sum(self, a, wa, b, wb, eps: float, out, accumulate: bool = False) -> None:
        """``out (+)= a / sqrt(mean(a^2) + eps) * wa + b / sqrt(mean(b^2) + eps) * wb`` row by row, everything float32."""
        self._dev(a, wa, b, wb, out)
        T, n = out.shape
        if any(t.dtype != torch.float32 or tuple(t.shape) != (T, n) for t in (a, b, out)):
            raise KernelError("normed_sum: float32 [tokens, width] tensors expected")
        self._call("hb_normed_sum", a.data_ptr(), _rows(a, "first result"), self._f32_vec(wa, n, "norm weight"), b.data_ptr(),
                   _rows(b, "second result"), self._f32_vec(wb, n, "norm weight"), float(eps), out.data_ptr(), _rows(out, "sum"), T, n,
                   1 if accumulate else 0, self._stream())
        self.launches += 1

    # ------------------------------------------------------------------ window + pooled blocks, sigmoid weights
    def qk_norm_append(self, proj, q_weight, k_weight, eps: float, heads: int, kv_heads: int, head_dim: int, v_dim: int, q_out, cache,
                       step, append: bool) -> None:
        """From a step's float32 projections ``[q | k | v | ...]``: with weights, q and k are divided by the root mean square of
        the token's WHOLE query (key) projection and multiplied by them; queries to ``q_out``, keys and values into the cache."""
        self._dev(proj, q_weight, k_weight, q_out, cache.k, cache.v)
        T = proj.shape[0]
        if proj.dtype != torch.float32 or tuple(q_out.shape) != (T, heads * head_dim):
            raise KernelError("qk_norm_append: float32 projections and [tokens, heads * head_dim] queries expected")
        if tuple(cache.k.shape[1:]) != (kv_heads, 64, head_dim) or tuple(cache.v.shape[1:]) != (kv_heads, 64, v_dim) \
                or not cache.k.is_contiguous() or not cache.v.is_contiguous() or cache.k.dtype != cache.v.dtype:
            raise KernelError("qk_norm_append: cache layer does not match the heads")
        pt = step.page_tables[cache.group]
        self._call("hb_qk_norm_append", proj.data_ptr(), _rows(proj, "projections"),
                   self._f32_vec(q_weight, heads * head_dim, "query norm weight") if q_weight is not None else None,
                   self._f32_vec(k_weight, kv_heads * head_dim, "key norm weight") if k_weight is not None else None, float(eps),
                   q_out.data_ptr(), _code(q_out), _rows(q_out, "queries"), cache.k.data_ptr(), cache.v.data_ptr(), _code(cache.k),
                   pt.data_ptr(), pt.shape[1], step.tok_seq.data_ptr(), step.positions.data_ptr(), T, heads, kv_heads, head_dim, v_dim,
                   cache.k.shape[0], 1 if append else 0, self.status.data_ptr(), self._stream())
        self.launches += 1

    def pool_blocks(self, cache, pooled, step, pool: int, kv_heads: int, head_dim: int, v_dim: int) -> None:
        """The mean key and value of every block of ``pool`` tokens whose last token this step cached, from ``cache`` into
        ``pooled`` (float32 storage whose entry e is block e)."""
        self._dev(cache.k, cache.v, pooled.k, pooled.v)
        if pooled.k.dtype != torch.float32 or tuple(pooled.k.shape[1:]) != (kv_heads, 64, head_dim) \
                or tuple(pooled.v.shape[1:]) != (kv_heads, 64, v_dim) or not pooled.k.is_contiguous() or not pooled.v.is_contiguous():
            raise KernelError("pool_blocks: the pooled store must be contiguous float32 with the cache's heads")
        pt, pp = step.page_tables[cache.group], step.page_tables[pooled.group]
        if pt.shape[1] != pp.shape[1]:
            raise KernelError("pool_blocks: the two page tables differ in width")
        self._call("hb_pool_blocks", cache.k.data_ptr(), cache.v.data_ptr(), _code(cache.k), pooled.k.data_ptr(), pooled.v.data_ptr(),
                   pt.data_ptr(), pp.data_ptr(), pt.shape[1], step.seq_pos0.data_ptr(), step.seq_len.data_ptr(), step.num_seqs,
                   step.max_new, int(pool), kv_heads, head_dim, v_dim, cache.k.shape[0], pooled.k.shape[0], self.status.data_ptr(),
                   self._stream())
        self.launches += 1

    POOL_PREFILL_FROM = 16              # steps whose longest portion has at least so many tokens run the tensor-core kernel
    ATTENTION_POOL_TILE = 16            # query tokens of a sequence that share a block
    ATTENTION_POOL_MAX_SPLITS = 64

    def attention_pool_splits(self, step, heads: int, window: Optional[int], pool: int) -> int:
        """Key ranges a step is cut into: one unless the step's blocks are fewer than two per SM and a query sees
        enough keys (decode steps), then as many as give every SM two blocks, of 64 keys or more each."""
        tiles = sum(-(-n // self.ATTENTION_POOL_TILE) for n in step.host_new) * heads
        keys = step.max_len if not window else min(step.max_len, window + step.max_new) + (step.max_len // pool if pool else 0)
        if tiles >= 2 * self.sm_count or keys < 256:
            return 1
        return max(1, min(self.ATTENTION_POOL_MAX_SPLITS, -(-2 * self.sm_count // tiles), keys // 64))

    def attention_pool(self, q, cache, pooled, step, head_bias, gate, out, heads: int, kv_heads: int, head_dim: int, v_dim: int,
                       scale: float, window: Optional[int], pool: int, workspace=None) -> None:
        """Attention whose weights are ``sigmoid(q . k * scale + head_bias[head])``, not normalised: a query sees the last
        ``window`` tokens and, with ``pool``, one mean key and value (``pooled``) per block of ``pool`` tokens wholly before
        them; the result is multiplied by ``sigmoid(gate)`` (float32 ``[tokens, heads * v_dim]``, may be None)."""
        self._dev(q, cache.k, cache.v, head_bias, gate, out)
        T = q.shape[0]
        if tuple(out.shape) != (T, heads * v_dim) or tuple(q.shape) != (T, heads * head_dim):
            raise KernelError("attention_pool: shapes do not agree")
        if tuple(cache.k.shape[1:]) != (kv_heads, 64, head_dim) or tuple(cache.v.shape[1:]) != (kv_heads, 64, v_dim):
            raise KernelError("attention_pool: cache layer does not match the heads")
        if gate is not None and (gate.dtype != torch.float32 or tuple(gate.shape) != (T, heads * v_dim)):
            raise KernelError("attention_pool: the gate must be float32 [tokens, heads * v_dim]")
        if pool and (pooled is None or not window):
            raise KernelError("attention_pool: pooled blocks need their store and a window")
        pt = step.page_tables[cache.group]
        pp = step.page_tables[pooled.group] if pool else None
        bias_ptr = self._f32_vec(head_bias, heads, "head bias") if head_bias is not None else None
        common = (pooled.k.data_ptr() if pool else None, pooled.v.data_ptr() if pool else None, pt.data_ptr(),
                  pp.data_ptr() if pool else None, pt.shape[1], step.seq_start.data_ptr(), step.seq_pos0.data_ptr(), step.num_seqs)
        tiles = sum(-(-n // self.ATTENTION_POOL_TILE) for n in step.host_new)
        sizes = (T, heads, kv_heads, head_dim, v_dim, float(scale), int(window) if window else 0, int(pool) if pool else 0,
                 cache.k.shape[0], pooled.k.shape[0] if pool else 0)
        if (self.use_mma_pool_attention and q.dtype == torch.bfloat16 and cache.k.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
                and not step.is_decode and step.max_new >= self.POOL_PREFILL_FROM
                and self.lib.hb_attention_pool_prefill_supported(head_dim, v_dim) and _rows(q, "queries") % 2 == 0
                and _rows(out, "attention output") % 2 == 0 and sum(-(-n // 64) for n in step.host_new) <= 65535):
            # many tokens: the window on the tensor cores, 64 query tokens a block; the pooled blocks, few, by the FP32 kernel first
            share = None
            if pool:
                share = workspace.buffer("attention_pool.pooled_share", (workspace_rows(workspace, T), heads * v_dim), torch.float32)[:T]
                self._call("hb_attention_pool", q.data_ptr(), _code(q), _rows(q, "queries"), cache.k.data_ptr(), cache.v.data_ptr(),
                           _code(cache.k), *common, tiles, bias_ptr, None, 0, out.data_ptr(), _code(out), _rows(out, "attention output"),
                           share.data_ptr(), *sizes, 1, 1, 0, self.status.data_ptr(), self._stream())
                self.launches += 1
            self._call("hb_attention_pool_prefill", q.data_ptr(), _rows(q, "queries"), cache.k.data_ptr(), cache.v.data_ptr(), pt.data_ptr(),
                       pt.shape[1], step.seq_start.data_ptr(), step.seq_pos0.data_ptr(), bias_ptr,
                       share.data_ptr() if share is not None else None, gate.data_ptr() if gate is not None else None,
                       _rows(gate, "gate") if gate is not None else 0, out.data_ptr(), _rows(out, "attention output"), step.num_seqs,
                       sum(-(-n // 64) for n in step.host_new), heads, kv_heads, head_dim, v_dim, float(scale), int(window) if window else 0,
                       cache.k.shape[0], self.status.data_ptr(), self._stream())
            self.launches += 1
            return
        # one token per sequence: a block's rows are the query heads of a key/value head, which are then staged once per group
        grouped = 1 if (step.is_decode and heads // kv_heads <= self.ATTENTION_POOL_TILE) else 0
        splits = self.attention_pool_splits(step, kv_heads if grouped else heads, window, pool)
        partial = None
        if splits > 1:
            # the same buffer for every step of a shape: a captured graph holds its address
            partial = workspace.buffer(f"attention_pool.partial{step.tag}.{splits}", (splits, T, heads * v_dim), torch.float32)
        self._call("hb_attention_pool", q.data_ptr(), _code(q), _rows(q, "queries"), cache.k.data_ptr(), cache.v.data_ptr(),
                   _code(cache.k), *common, tiles, bias_ptr, gate.data_ptr() if gate is not None else None,
                   _rows(gate, "gate") if gate is not None else 0, out.data_ptr(), _code(out), _rows(out, "attention output"),
                   partial.data_ptr() if partial is not None else None, *sizes, splits, 0, grouped, self.status.data_ptr(), self._stream())
        self.launches += 1 if splits == 1 else 2

    # ------------------------------------------------------------------ matrix memory with a fixed decay
    ACTIVATIONS = {None: 0, "none": 0, "silu": 1}

    def decay_memory(self, proj, decay, state, step, out, heads: int, d: int, dv: int, activation="silu", table=None, rot: int = 0,
                     k_scale: float = 1.0) -> None:
        """``S <- decay[h] S + k v^T; o = S^T q`` per head over a step's tokens, sequence by sequence, with q, k, v the
        activation of the float32 projections ``[q | k | v | ...]``; ``state`` float32 ``[slots, heads * d * dv]``, ``out``
        float32 ``[tokens, heads * dv]``.  With ``table`` (``[tokens, rot / 2, 2]`` cosines and sines) the first ``rot``
        dimensions of every head of q and k are turned first; ``k_scale`` multiplies k after that."""
        self._dev(proj, decay, state, out, table)
        if rot and (table is None or table.dtype != torch.float32 or not table.is_contiguous() or tuple(table.shape[:2]) != (proj.shape[0], rot // 2)):
            raise KernelError("decay_memory: rotary table does not match the tokens")
        T = proj.shape[0]
        if proj.dtype != torch.float32 or out.dtype != torch.float32 or tuple(out.shape) != (T, heads * dv):
            raise KernelError("decay_memory: float32 projections and float32 [tokens, heads * dv] output expected")
        if state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] != heads * d * dv or state.stride(1) != 1:
            raise KernelError("decay_memory: state must be float32 [slots, heads * d * dv]")
        self._call("hb_decay_memory", proj.data_ptr(), _rows(proj, "projections"), self._f32_vec(decay, heads, "decay"), state.data_ptr(),
                   state.stride(0), step.state_slots.data_ptr(), step.seq_start.data_ptr(), out.data_ptr(), _rows(out, "output"),
                   step.num_seqs, heads, d, dv, self.ACTIVATIONS[activation], table.data_ptr() if rot else None, int(rot), float(k_scale),
                   self._stream())
        self.launches += 1

    GATES = {"sigmoid": 0, "silu": 1}

    def gated_norm(self, o, gate, weight, eps: float, out, out_scale: float = 1.0, group: Optional[int] = None, gate_kind: str = "sigmoid") -> None:
        """``out = o / sqrt(mean(o^2) + eps) * weight * f(gate) * out_scale``; the mean over whole rows, or with ``group`` over
        every run of that many values of a row; ``gate`` and ``weight`` may be None; f is sigmoid or silu."""
        self._dev(o, gate, weight, out)
        T, n = o.shape
        if gate_kind not in self.GATES:
            raise KernelError(f"gated_norm: gate {gate_kind!r} ({', '.join(self.GATES)})")
        if o.dtype != torch.float32 or tuple(out.shape) != (T, n) or (gate is not None and (gate.dtype != torch.float32 or tuple(gate.shape) != (T, n))):
            raise KernelError("gated_norm: float32 [tokens, n] input and gate expected")
        self._call("hb_gated_norm", o.data_ptr(), _rows(o, "gated_norm input"), gate.data_ptr() if gate is not None else None,
                   _rows(gate, "gate") if gate is not None else 0, self._f32_vec(weight, n, "norm weight") if weight is not None else None,
                   float(eps), float(out_scale), out.data_ptr(), _code(out), _rows(out, "gated_norm output"), T, n,
                   int(group) if group else n, self.GATES[gate_kind], self._stream())
        self.launches += 1

    # ------------------------------------------------------------------ layer norm (alone, and on a sublayer's output)
    def layernorm(self, x, weight, bias, eps: float, out, rows=None) -> None:
        """``out[i] = (x[r] - mean) / sqrt(var + eps) * weight + bias`` with ``r = rows[i]`` (``rows`` None: every row), 32-bit."""
        self._dev(x, weight, bias, out, rows)
        n = x.shape[1]
        if x.dtype != torch.float32 or out.shape[1] != n or (rows is None and out.shape[0] != x.shape[0]):
            raise KernelError("layernorm: float32 [rows, width] input and an output of the same width expected")
        if rows is not None and (rows.dtype != torch.int32 or rows.numel() != out.shape[0]):
            raise KernelError("layernorm: rows must be int32, one per output row")
        self._call("hb_layernorm", x.data_ptr(), _rows(x, "layernorm input"), self._f32_vec(weight, n, "norm weight"),
                   self._f32_vec(bias, n, "norm bias"), float(eps), out.data_ptr(), _code(out), _rows(out, "layernorm output"),
                   rows.data_ptr() if rows is not None else None, out.shape[0], n, self._stream())
        self.launches += 1

    def layernorm_add(self, y, weight, bias, eps: float, x, copy=None, y2=None, sa: float = 1.0, sb: float = 1.0) -> None:
        """``x += layernorm(y)`` row by row in 32-bit; with ``y2``: ``x += layernorm(sa * y + sb * y2)``; ``copy`` (same shape,
        any kernel dtype) also receives the new rows of ``x``."""
        self._dev(y, weight, bias, x, copy, y2)
        T, n = x.shape
        if x.dtype != torch.float32 or any(t is not None and (t.dtype != torch.float32 or tuple(t.shape) != (T, n)) for t in (y, y2)) \
                or (copy is not None and tuple(copy.shape) != (T, n)):
            raise KernelError("layernorm_add: float32 [tokens, width] inputs and residual expected")
        self._call("hb_layernorm_add", y.data_ptr(), _rows(y, "layernorm_add input"), y2.data_ptr() if y2 is not None else None,
                   _rows(y2, "layernorm_add input") if y2 is not None else 0, float(sa), float(sb), self._f32_vec(weight, n, "norm weight"),
                   self._f32_vec(bias, n, "norm bias"), float(eps), x.data_ptr(), _rows(x, "residual"),
                   copy.data_ptr() if copy is not None else None, _code(copy) if copy is not None else 0,
                   _rows(copy, "residual copy") if copy is not None else 0, T, n, self._stream())
        self.launches += 1

    def convert(self, x, out) -> None:
        """``out = x`` in ``out``'s dtype (``x`` float32, both contiguous)."""
        self._dev(x, out)
        if x.dtype != torch.float32 or not x.is_contiguous() or not out.is_contiguous() or x.shape != out.shape:
            raise KernelError("convert: contiguous float32 input and an output of the same shape expected")
        self._call("hb_convert", x.data_ptr(), out.data_ptr(), _code(out), x.numel(), self._stream())
        self.launches += 1

    # ------------------------------------------------------------------ attention over one cached latent per token
    def latent_prepare(self, proj, heads: int, d: int, dr: int, rank: int, down_at: int, c_weight, eps: float, table, rot: int,
                       q_out, cache, step, append: bool, whole_heads: int = 0) -> None:
        """From a step's float32 projections ``[q (heads x (d + dr)) | ... ]`` with the down projection ``[latent (rank) | shared
        key part (dr)]`` at column ``down_at``: the latent divided by its root mean square times ``c_weight`` and the key part
        turned by ``table`` (pairs ``(2i, 2i + 1)`` of its first ``rot`` dimensions) into the cache (key row ``[c | k_r]``, value
        row ``c``); every head's rotated query part turned into ``q_out[t, h, rank:]`` (``q_out`` ``[tokens, heads * (rank + dr)]``).
        With ``whole_heads`` = n: ``q_out`` is ``[tokens, heads * n]`` and receives every head's whole query, ``[unrotated (d) |
        rotated and turned (dr) | zeros]``."""
        self._dev(proj, c_weight, table, q_out, cache.k, cache.v)
        T = proj.shape[0]
        q_head = int(whole_heads) if whole_heads else rank + dr
        if proj.dtype != torch.float32 or tuple(q_out.shape) != (T, heads * q_head) or q_head < (d + dr if whole_heads else 0):
            raise KernelError("latent_prepare: float32 projections and queries [tokens, heads * (rank + dr)] expected")
        if rot and (table is None or table.dtype != torch.float32 or not table.is_contiguous() or tuple(table.shape[:2]) != (T, rot // 2)):
            raise KernelError("latent_prepare: rotary table does not match the tokens")
        if tuple(cache.k.shape[1:]) != (1, 64, rank + dr) or tuple(cache.v.shape[1:]) != (1, 64, rank) \
                or not cache.k.is_contiguous() or not cache.v.is_contiguous() or cache.k.dtype != cache.v.dtype:
            raise KernelError("latent_prepare: cache layer does not match the latent")
        pt = step.page_tables[cache.group]
        self._call("hb_latent_prepare", proj.data_ptr(), _rows(proj, "projections"), heads, d, dr, rank, int(down_at),
                   self._f32_vec(c_weight, rank, "latent norm weight"), float(eps), table.data_ptr() if rot else None, int(rot),
                   q_out.data_ptr(), _code(q_out), _rows(q_out, "queries"), q_head, d if whole_heads else rank, d if whole_heads else 0,
                   cache.k.data_ptr(), cache.v.data_ptr(), _code(cache.k),
                   pt.data_ptr(), pt.shape[1], step.tok_seq.data_ptr(), step.positions.data_ptr(), T, cache.k.shape[0],
                   1 if append else 0, self.status.data_ptr(), self._stream())
        self.launches += 1

    def latent_gather(self, cache, step, rank: int, rows, scratch_table) -> None:
        """The latents of the step's sequences, from their first token on, page by page: ``rows`` bfloat16 ``[pages * 64, rank]``
        (sequence b's pages follow those of the sequences in front of it; rows behind a sequence's end are zeros) and the page
        table of that layout, ``scratch_table`` int32 ``[sequences, width]``."""
        self._dev(cache.v, rows, scratch_table)
        pages = sum((n + 63) // 64 for n in step.host_len)
        if cache.v.dtype != torch.bfloat16 or rows.dtype != torch.bfloat16 or not rows.is_contiguous() or tuple(rows.shape) != (pages * 64, rank) \
                or tuple(cache.v.shape[1:]) != (1, 64, rank) or not cache.v.is_contiguous():
            raise KernelError("latent_gather: bfloat16 cache [pages, 1, 64, rank] and rows [step pages * 64, rank] expected")
        if scratch_table.dtype != torch.int32 or not scratch_table.is_contiguous() or scratch_table.shape[0] != step.num_seqs \
                or scratch_table.shape[1] < (step.max_len + 63) // 64:
            raise KernelError("latent_gather: the scratch page table must be int32 [sequences, pages of the longest]")
        pt = step.page_tables[cache.group]
        self._call("hb_latent_gather", cache.v.data_ptr(), pt.data_ptr(), pt.shape[1], step.seq_len.data_ptr(), step.num_seqs,
                   (step.max_len + 63) // 64, rank, rows.data_ptr(), scratch_table.data_ptr(), scratch_table.shape[1], cache.v.shape[0],
                   self.status.data_ptr(), self._stream())
        self.launches += 1

    def latent_scatter(self, kv, cache, step, heads: int, d: int, dr: int, dv: int, rank: int, k_out, v_out) -> None:
        """From ``kv`` bfloat16 ``[pages * 64, >= heads * (d + dv)]`` = ``[k_u (heads x d) | v (heads x dv)]`` per gathered row and the
        cached rotated key parts: ``k_out`` ``[pages, heads, 64, >= d + dr]`` = ``[k_u | k_r | zeros]`` and ``v_out`` ``[pages, heads, 64,
        >= dv]`` = ``[v | zeros]``, the paged layout of a cache with as many key/value heads as heads."""
        self._dev(kv, cache.k, k_out, v_out)
        pages = sum((n + 63) // 64 for n in step.host_len)
        if any(t.dtype != torch.bfloat16 for t in (kv, cache.k, k_out, v_out)) or kv.shape[0] != pages * 64 or kv.stride(1) != 1 \
                or not k_out.is_contiguous() or not v_out.is_contiguous() or tuple(k_out.shape[:3]) != (pages, heads, 64) \
                or tuple(v_out.shape[:3]) != (pages, heads, 64) or tuple(cache.k.shape[1:]) != (1, 64, rank + dr):
            raise KernelError("latent_scatter: bfloat16 rows [step pages * 64, ..] and outputs [step pages, heads, 64, ..] expected")
        pt = step.page_tables[cache.group]
        self._call("hb_latent_scatter", kv.data_ptr(), _rows(kv, "keys and values"), cache.k.data_ptr(), pt.data_ptr(), pt.shape[1],
                   step.seq_len.data_ptr(), step.num_seqs, (step.max_len + 63) // 64, heads, d, dr, dv, rank, k_out.shape[3], v_out.shape[3],
                   k_out.data_ptr(), v_out.data_ptr(), cache.k.shape[0], self._stream())
        self.launches += 1

    def head_linear(self, x, in_head: int, w, out, out_head: int, n_in: int, n_out: int, gate=None) -> None:
        """``out[t, h * out_head : + n_out] = W_h x[t, h * in_head : + n_in]`` for every head h, ``w`` ``[heads, n_in, n_out]``
        (``w[h, i, o] = W_h[o, i]``), ``x`` float32; with ``gate`` float32 ``[tokens, heads]`` times ``sigmoid(gate[t, h])``."""
        self._dev(x, w, out, gate)
        T, heads = x.shape[0], w.shape[0]
        if x.dtype != torch.float32 or w.dim() != 3 or tuple(w.shape[1:]) != (n_in, n_out) or not w.is_contiguous() or out.shape[0] != T:
            raise KernelError("head_linear: float32 input and weights [heads, n_in, n_out] expected")
        if x.shape[1] < (heads - 1) * in_head + n_in or out.shape[1] < (heads - 1) * out_head + n_out:
            raise KernelError("head_linear: rows are too short for the heads")
        gp, ldg = self._head_gate(gate, T, heads)
        self._call("hb_head_linear", x.data_ptr(), _rows(x, "head_linear input"), int(in_head), w.data_ptr(), _code(w), out.data_ptr(),
                   _code(out), _rows(out, "head_linear output"), int(out_head), gp, ldg, T, heads, n_in, n_out, self._stream())
        self.launches += 1

    # ------------------------------------------------------------------ selective state-space scan
    def conv_act(self, x, conv_weight, conv_bias, state, step, out, activation="silu") -> None:
        """``out[t] = act(bias + sum_j w[:, j] x[t - taps + 1 + j])`` per channel and sequence; ``x`` float32 (a column range
        of a wider matrix is fine), ``state`` float32 ``[slots, (taps - 1) * C]``: every sequence's last inputs, brought up to date."""
        self._dev(x, conv_weight, conv_bias, state, out)
        T, C = x.shape
        taps = conv_weight.shape[1]
        if x.dtype != torch.float32 or tuple(out.shape) != (T, C) or tuple(conv_weight.shape) != (C, taps) \
                or conv_weight.dtype != torch.float32 or not conv_weight.is_contiguous():
            raise KernelError("conv_act: float32 input, float32 taps [channels, taps] and an output of the input's shape expected")
        if state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] != (taps - 1) * C or (taps > 1 and state.stride(1) != 1):
            raise KernelError("conv_act: state must be float32 [slots, (taps - 1) * channels]")
        self._call("hb_conv_act", x.data_ptr(), _rows(x, "conv_act input"), conv_weight.data_ptr(),
                   self._f32_vec(conv_bias, C, "convolution bias") if conv_bias is not None else None, taps, state.data_ptr(),
                   state.stride(0), step.state_slots.data_ptr(), step.seq_start.data_ptr(), out.data_ptr(), _code(out),
                   _rows(out, "conv_act output"), step.num_seqs, step.max_new, C, self.ACTIVATIONS[activation], self._stream())
        self.launches += 1

    SCAN_CHUNK_FROM = 128           # steps whose longest portion has at least so many tokens run the scan in chunks side by side
    SCAN_CHUNK = 64

    def selective_scan(self, u, bc, z, dt_raw, b_dt, a_log, d_skip, state, step, out, n_state: int, workspace=None,
                       chunked: Optional[bool] = None) -> None:
        """The selective scan over a step's tokens, sequence by sequence: ``bc`` float32 rows ``[B | C]``, ``z`` float32 gate
        input, ``dt_raw`` float32 ``[tokens, inner]`` (the step sizes before bias and softplus), ``u`` and ``out`` in the
        activations' dtype ``[tokens, inner]``; ``state`` float32 ``[slots, inner * n_state]``.  ``chunked`` (default: steps that
        bring ``SCAN_CHUNK_FROM`` tokens or more to a sequence while channels and sequences are too few to fill the device, given
        a ``workspace``): the tokens of a sequence are cut into chunks that run side by side (three launches)."""
        self._dev(u, bc, z, dt_raw, b_dt, a_log, d_skip, state, out)
        T, inner = u.shape
        if any(t.dtype != torch.float32 for t in (bc, z, dt_raw)) or tuple(z.shape) != (T, inner) or tuple(dt_raw.shape) != (T, inner) \
                or tuple(out.shape) != (T, inner) or tuple(bc.shape) != (T, 2 * n_state) or u.dtype != out.dtype:
            raise KernelError("selective_scan: shapes or dtypes do not agree")
        if tuple(a_log.shape) != (inner, n_state) or a_log.dtype != torch.float32 or not a_log.is_contiguous():
            raise KernelError("selective_scan: float32 A_log [inner, state] expected")
        if state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] != inner * n_state or state.stride(1) != 1:
            raise KernelError("selective_scan: state must be float32 [slots, inner * state]")
        if chunked is None:
            # chunks pay (they walk every token twice) only while one block per group of channels and sequence leaves SMs idle
            chunked = (workspace is not None and not step.is_decode and step.max_new >= self.SCAN_CHUNK_FROM
                       and -(-inner // 8) * step.num_seqs < self.sm_count)
        chunk_len, max_chunks, carry = 0, 0, None
        if chunked:
            chunk_len = self.SCAN_CHUNK
            max_chunks = -(-step.max_new // chunk_len)
            carry = workspace.buffer("selective_scan.carry", (step.num_seqs * max_chunks * inner * (2 * n_state + 1),), torch.float32)
        self._call("hb_selective_scan", u.data_ptr(), _code(u), _rows(u, "scan input"), bc.data_ptr(), _rows(bc, "scan parameters"),
                   z.data_ptr(), _rows(z, "scan gate"), dt_raw.data_ptr(), _rows(dt_raw, "step sizes"),
                   self._f32_vec(b_dt, inner, "step-size bias"), a_log.data_ptr(), self._f32_vec(d_skip, inner, "skip weight"),
                   state.data_ptr(), state.stride(0), step.state_slots.data_ptr(), step.seq_start.data_ptr(), out.data_ptr(), _code(out),
                   _rows(out, "scan output"), step.num_seqs, inner, n_state, chunk_len, max_chunks,
                   carry.data_ptr() if carry is not None else None, carry.numel() if carry is not None else 0, self._stream())
        self.launches += 3 if chunked else 1

    HEAD_SCAN_CHUNK_FROM = 256      # steps whose longest portion has at least so many tokens may run the memory in chunks
    HEAD_SCAN_CHUNK = 128

    def head_scan(self, u, k, q, decay_raw, decay_bias, state, step, out, heads: int, groups: int, head_dim: int, n_state: int,
                  a_log=None, inv_tau: float = 1.0, skip=None, z=None, q_scale: float = 1.0, workspace=None,
                  chunked: Optional[bool] = None) -> None:
        """A recurrent memory per head whose decay depends on the token, over a step's tokens, sequence by sequence:
        ``S <- a S + s u k^T``, ``y = q_scale S^T q + skip u``, ``out = y silu(z)`` (``z`` None: no gate).  ``u`` float32
        ``[tokens, heads * head_dim]``, ``k`` and ``q`` float32 ``[tokens, groups * n_state]`` (heads share them in ``groups``
        runs).  With ``a_log`` (float32 ``[heads]``): ``decay_raw [tokens, heads]`` are step sizes before bias and softplus,
        ``a = exp(-exp(a_log) dt)`` and ``s = dt``.  Without: ``decay_raw [tokens, heads * n_state]``, ``a = sigmoid(decay_raw +
        decay_bias) ^ inv_tau`` per state index and ``s = 1``.  ``state`` float32 ``[slots, heads * head_dim * n_state]``.
        ``chunked`` (default: long portions while heads, channels and sequences are too few to fill the device, given a
        ``workspace``): the tokens of a sequence are cut into chunks that run side by side (three launches)."""
        self._dev(u, k, q, decay_raw, decay_bias, state, out, a_log, skip, z)
        T = u.shape[0]
        mode = 0 if a_log is not None else 1
        width = heads * head_dim
        if any(t.dtype != torch.float32 for t in (u, k, q, decay_raw)) or tuple(u.shape) != (T, width) or tuple(out.shape) != (T, width) \
                or tuple(k.shape) != (T, groups * n_state) or tuple(q.shape) != (T, groups * n_state) \
                or tuple(decay_raw.shape) != (T, heads * (n_state if mode else 1)) or (z is not None and (z.dtype != torch.float32 or tuple(z.shape) != (T, width))):
            raise KernelError("head_scan: shapes or dtypes do not agree")
        if state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] != width * n_state or state.stride(1) != 1:
            raise KernelError("head_scan: state must be float32 [slots, heads * head_dim * n_state]")
        if chunked is None:
            # chunks walk every token twice: they pay only while one block per 64 channels of a head and sequence (the shape in
            # which a thread holds the most state) would leave most SMs idle (measured, 2048 tokens of one sequence: 8 heads of
            # 256 channels and 64 state values 354 us in chunks against 843 us; 8 heads of 512 channels and 128 state values
            # 1168 against 1319 us; 64 heads of 64 channels 972 against 1001 us; 128 heads of 64 channels 1704 against 1418 us)
            chunked = (workspace is not None and not step.is_decode and step.max_new >= self.HEAD_SCAN_CHUNK_FROM
                       and -(-head_dim // 64) * heads * step.num_seqs < self.sm_count // 2)
        chunk_len, max_chunks, carry = 0, 0, None
        if chunked:
            chunk_len = self.HEAD_SCAN_CHUNK
            max_chunks = -(-step.max_new // chunk_len)
            carry = workspace.buffer("head_scan.carry", (step.num_seqs * max_chunks * heads * (2 * head_dim * n_state + (n_state if mode else 1)),),
                                     torch.float32)
        self._call("hb_head_scan", u.data_ptr(), _rows(u, "memory input"), k.data_ptr(), _rows(k, "memory keys"), q.data_ptr(),
                   _rows(q, "memory queries"), z.data_ptr() if z is not None else None, _rows(z, "memory gate") if z is not None else 0,
                   decay_raw.data_ptr(), _rows(decay_raw, "decay input"),
                   self._f32_vec(decay_bias, heads * (n_state if mode else 1), "decay bias"),
                   self._f32_vec(a_log, heads, "A_log") if a_log is not None else None, float(inv_tau),
                   self._f32_vec(skip, heads, "skip weight") if skip is not None else None, float(q_scale), state.data_ptr(),
                   state.stride(0), step.state_slots.data_ptr(), step.seq_start.data_ptr(), out.data_ptr(), _code(out),
                   _rows(out, "memory output"), step.num_seqs, heads, groups, head_dim, n_state, mode, chunk_len, max_chunks,
                   carry.data_ptr() if carry is not None else None, carry.numel() if carry is not None else 0, self._stream())
        self.launches += 3 if chunked else 1

    # ------------------------------------------------------------------ mixture of experts
    def moe_route_scores(self, h, w_router, correction, top: int, groups: int, keep: int, experts, weights, norm_eps: float = 1e-20) -> None:
        """Per token: scores = softmax over ALL router outputs (``w_router`` float32 ``[outputs, width]``, logits in 32-bit);
        the ``top`` outputs with the largest ``score + correction`` among the ``keep`` best of ``groups`` equal runs of
        neighbours (a run's score: its largest choice score) into ``experts``; their scores (without the correction) divided
        by their sum ``+ norm_eps`` into ``weights``."""
        self._dev(h, w_router, correction, experts, weights)
        T, W = h.shape
        E = w_router.shape[0]
        if w_router.dtype != torch.float32 or not w_router.is_contiguous() or w_router.shape[1] != W or experts.dtype != torch.int32 \
                or weights.dtype != torch.float32 or tuple(experts.shape) != (T, top) or tuple(weights.shape) != (T, top) \
                or not experts.is_contiguous() or not weights.is_contiguous():
            raise KernelError("moe_route_scores: float32 router [outputs, width], int32 experts and float32 weights [tokens, top] expected")
        self._call("hb_moe_route_scores", h.data_ptr(), _code(h), _rows(h, "router input"), w_router.data_ptr(),
                   self._f32_vec(correction, E, "router correction") if correction is not None else None, experts.data_ptr(),
                   weights.data_ptr(), T, W, E, int(top), int(groups), int(keep), float(norm_eps), self._stream())
        self.launches += 1

    def gelu_unit(self, x, out, kind: str, row_gate: Optional[int] = None) -> None:
        """``kind`` "tanh_gated": ``out = gelu_tanh(x[:, :F]) * x[:, F:2F]``; "erf": ``out = gelu_erf(x[:, :F])``, times
        ``sigmoid(x[:, row_gate])`` when a column of ``x`` is named as the row's gate.  ``x`` float32."""
        self._dev(x, out)
        T, F = out.shape
        code = {"tanh_gated": 0, "erf": 1}[kind]
        if x.dtype != torch.float32 or x.shape[0] != T or x.shape[1] < (2 * F if code == 0 else F) or (row_gate is not None and not 0 <= row_gate < x.shape[1]):
            raise KernelError("gelu_unit: float32 input rows that hold the unit's columns expected")
        self._call("hb_gelu_unit", x.data_ptr(), _rows(x, "gelu_unit input"), out.data_ptr(), _code(out), _rows(out, "gelu_unit output"), T, F,
                   code, -1 if row_gate is None else int(row_gate), self._stream())
        self.launches += 1

    def moe_route(self, h, w_router, top: int, experts, weights) -> None:
        """Per token the ``top`` experts with the largest router logits (``w_router`` float32 ``[experts, width]``, logits in
        32-bit) into ``experts`` int32 ``[tokens, top]`` and the softmax over those logits into ``weights`` float32."""
        self._dev(h, w_router, experts, weights)
        T, W = h.shape
        E = w_router.shape[0]
        if w_router.dtype != torch.float32 or not w_router.is_contiguous() or w_router.shape[1] != W or experts.dtype != torch.int32 \
                or weights.dtype != torch.float32 or tuple(experts.shape) != (T, top) or tuple(weights.shape) != (T, top) \
                or not experts.is_contiguous() or not weights.is_contiguous():
            raise KernelError("moe_route: float32 router [experts, width], int32 and float32 [tokens, top] outputs expected")
        self._call("hb_moe_route", h.data_ptr(), _code(h), _rows(h, "router input"), w_router.data_ptr(), experts.data_ptr(),
                   weights.data_ptr(), T, W, E, int(top), self._stream())
        self.launches += 1

    def moe_max_tiles(self, entries: int, n_experts: int, tile_rows: int) -> int:
        return int(self.lib.hb_moe_max_tiles(int(entries), int(n_experts), int(tile_rows)))

    def moe_experts(self, h, experts, weights, w_gate, w_up, w_down, limit: float, alpha: float, out, accumulate: bool, workspace,
                    cap: int, tag: str = "", identity: bool = False) -> None:
        """``out (+)= sum_k weights[t, k] * expert_{experts[t, k]}(h[t])`` with the experts' weights stacked ``[experts, ff,
        width]`` (gate, up) and ``[experts, width, ff]`` (down) in the activations' dtype and the clamped gated unit of
        ``glu_clamp`` between them.  Four launches: plan, gate/up with activation, down, weighted sum.  bfloat16 operands whose
        rows are multiples of 8 elements run the products on the tensor cores (``use_tensor_cores``), all others on the FP32 pipe.
        ``w_up`` None: experts of one matrix, ``act = gelu_erf(w_gate h)`` (``limit`` and ``alpha`` unused).  ``identity``: expert
        numbers from the stack's size on are identity experts, whose result is ``h[t]`` itself."""
        self._dev(h, experts, weights, w_gate, w_up, w_down, out)
        T, W = h.shape
        E, F = w_gate.shape[0], w_gate.shape[1]
        top = experts.shape[1]
        if tuple(w_gate.shape) != (E, F, W) or (w_up is not None and tuple(w_up.shape) != (E, F, W)) or tuple(w_down.shape) != (E, W, F) \
                or not (w_gate.is_contiguous() and (w_up is None or w_up.is_contiguous()) and w_down.is_contiguous()) \
                or not (w_gate.dtype == w_down.dtype == h.dtype) or (w_up is not None and w_up.dtype != h.dtype):
            raise KernelError("moe_experts: stacked contiguous expert weights in the activations' dtype expected")
        if out.dtype != torch.float32 or tuple(out.shape) != (T, W):
            raise KernelError("moe_experts: float32 [tokens, width] output expected")
        entries = T * top
        most = cap * top
        tc = 1 if (self.use_tensor_cores and h.dtype == torch.bfloat16 and W % 8 == 0 and F % 8 == 0 and _rows(h, "expert input") % 8 == 0
                   and h.data_ptr() % 16 == 0) else 0
        tile_rows = int(self.lib.hb_moe_tile_rows(tc))
        max_tiles = self.moe_max_tiles(entries, E, tile_rows)
        plan = workspace.buffer("moe.plan" + tag, (E + 1 + most + 1 + 2 * self.moe_max_tiles(most, E, 32),), torch.int32)
        offsets, order, tiles = plan[: E + 1], plan[E + 1: E + 1 + most], plan[E + 1 + most:]
        act = workspace.buffer("moe.act" + tag, (most, F), h.dtype)
        down = workspace.buffer("moe.down" + tag, (most, W), torch.float32)
        s = self._stream()
        self._call("hb_moe_plan", experts.data_ptr(), entries, E, tile_rows, offsets.data_ptr(), order.data_ptr(), tiles.data_ptr(), s)
        self._call("hb_moe_glu", h.data_ptr(), _code(h), _rows(h, "expert input"), w_gate.data_ptr(),
                   w_up.data_ptr() if w_up is not None else None, _code(w_gate),
                   offsets.data_ptr(), order.data_ptr(), tiles.data_ptr(), max_tiles, top, act.data_ptr(), _code(act), F, F, W,
                   float(limit), float(alpha), tc, s)
        self._call("hb_moe_down", act.data_ptr(), _code(act), F, w_down.data_ptr(), _code(w_down), offsets.data_ptr(), order.data_ptr(),
                   tiles.data_ptr(), max_tiles, top, down.data_ptr(), W, W, F, tc, s)
        self._call("hb_moe_combine", down.data_ptr(), W, weights.data_ptr(), top, out.data_ptr(), _rows(out, "expert output"), T, W,
                   1 if accumulate else 0, experts.data_ptr() if identity else None, E, h.data_ptr() if identity else None, _code(h),
                   _rows(h, "expert input"), s)
        self.launches += 4

    def glu_clamp(self, gate_up, out, limit: float, alpha: float) -> None:
        """``out = g' sigmoid(alpha g') (u' + 1)`` with ``g' = min(g, limit)``, ``u' = clamp(u, -limit, limit)`` from float32 ``[g | u]``."""
        self._dev(gate_up, out)
        T, F = out.shape
        if gate_up.dtype != torch.float32 or tuple(gate_up.shape) != (T, 2 * F):
            raise KernelError("glu_clamp: float32 [rows, 2 * ff] input expected")
        self._call("hb_glu_clamp", gate_up.data_ptr(), _rows(gate_up, "glu_clamp input"), out.data_ptr(), _code(out),
                   _rows(out, "glu_clamp output"), T, F, float(limit), float(alpha), self._stream())
        self.launches += 1

    # ------------------------------------------------------------------ random weights
    def random_normal(self, out, base: int, std: float, mean: float = 0.0) -> None:
        """``out.flat[i] = mean + std * N(0, 1)``, element ``i`` of the counter-based stream
        ``base`` (``weights.random_init.stream_base``): the values the CPU draws, bit for bit."""
        self._dev(out)
        if not out.is_contiguous():
            raise KernelError("random_normal: contiguous output expected")
        self._call("hb_random_normal", out.data_ptr(), _code(out), out.numel(), int(base) & ((1 << 64) - 1), float(std),
                   float(mean), self._stream())
        self.launches += 1

    # ------------------------------------------------------------------ sampling
    ARGMAX_MAX_PARTS = 16

    def argmax(self, logits, out) -> None:
        """``out[r]`` = index of the largest value of row r (the lowest index on ties).  A row is cut
        over several blocks when there are fewer rows than the device has room for."""
        self._dev(logits, out)
        n = logits.shape[0]
        if logits.dtype != torch.float32 or out.dtype != torch.int32 or out.numel() != n:
            raise KernelError("argmax: float32 logits and one int32 per row expected")
        parts = max(1, min(self.ARGMAX_MAX_PARTS, (2 * self.sm_count) // max(n, 1), logits.shape[1] // 4096))
        if n > self._argmax_counters.numel():
            self._retired += [self._argmax_counters, self._argmax_scratch]      # a captured graph may still use them
            self._argmax_counters = torch.zeros(n, dtype=torch.int32, device=self.device)
            self._argmax_scratch = torch.empty(2 * n * self.ARGMAX_MAX_PARTS, dtype=torch.int32, device=self.device)
        self._call("hb_argmax", logits.data_ptr(), _rows(logits, "logits"), out.data_ptr(), n, logits.shape[1], parts,
                   self._argmax_scratch.data_ptr(), self._argmax_counters.data_ptr(), self.status.data_ptr(), self._stream())
        self.launches += 1

    def sample(self, logits, temperature, seeds, request_ids, steps, out) -> None:
        self._dev(logits, temperature, seeds, request_ids, steps, out)
        n = logits.shape[0]
        if logits.dtype != torch.float32 or out.dtype != torch.int32 or temperature.dtype != torch.float32 \
                or any(t.dtype != torch.int64 for t in (seeds, request_ids, steps)) \
                or any(t.numel() != n for t in (temperature, seeds, request_ids, steps, out)):
            raise KernelError("sample: float32 logits/temperature, int64 seeds/requests/steps, int32 output, "
                              "one of each per row expected")
        self._call("hb_sample", logits.data_ptr(), _rows(logits, "logits"), temperature.data_ptr(), seeds.data_ptr(),
                   request_ids.data_ptr(), steps.data_ptr(), out.data_ptr(), n, logits.shape[1], self.status.data_ptr(),
                   self._stream())
        self.launches += 1
