"""ctypes binding of ``libentmaxkv_b200.so`` (the C ABI in ``include/entmaxkv_b200.h``).

There is no fallback: if the shared library is missing or a call fails, an
exception is raised.
"""

from __future__ import annotations

import ctypes as C
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libentmaxkv_b200.so")

EKV_F16, EKV_BF16, EKV_F32 = 0, 1, 2
TAU_NONE, TAU_EXACT, TAU_CORRECTED = 0, 1, 2
STATUS_PAGE_RANGE, STATUS_CAPACITY, STATUS_TOKENS, STATUS_PEER_TIMEOUT = 1, 2, 4, 8
XCH_SUM, XCH_MAX = 0, 1
EXCHANGE_MAX_RANKS, EXCHANGE_HANDLE_BYTES = 8, 64

_DTYPES = {torch.float16: EKV_F16, torch.bfloat16: EKV_BF16, torch.float32: EKV_F32}
_ERRORS = {-1: "unsupported dtype / head_dim (fp16, bf16, fp32 with head_dim 64 or 128)",
           -2: "bad argument (null pointer, size, stride or alignment)",
           -3: "workspace too small", -4: "alpha must be > 1",
           -5: "batch exceeds the built-in scratch of the allocation-free entry point"}


class CacheDesc(C.Structure):
    _fields_ = [
        ("k", C.c_void_p), ("v", C.c_void_p),
        ("k_min", C.c_void_p), ("k_max", C.c_void_p), ("k_mean", C.c_void_p), ("k_std", C.c_void_p),
        ("seq_lens", C.c_void_p),
        ("kv_stride_b", C.c_int64), ("kv_stride_h", C.c_int64),
        ("meta_stride_b", C.c_int64), ("meta_stride_h", C.c_int64),
        ("batch", C.c_int32), ("kv_heads", C.c_int32), ("head_dim", C.c_int32), ("page_size", C.c_int32),
        ("capacity", C.c_int32), ("page_capacity", C.c_int32), ("dtype", C.c_int32), ("reserved", C.c_int32),
        ("block_table", C.c_void_p), ("bt_stride", C.c_int64), ("kv_stride_block", C.c_int64),
        ("num_blocks", C.c_int32), ("reserved2", C.c_int32),
    ]


# name -> (restype, argtypes); mirrors include/entmaxkv_b200.h one to one
_P, _I, _L, _F, _Z = C.c_void_p, C.c_int32, C.c_int64, C.c_float, C.c_size_t
_D = C.POINTER(CacheDesc)
SIGNATURES = {
    "ekv_page_stats_init": (C.c_int, [_D, _I, _P]),
    "ekv_append": (C.c_int, [_D, _P, _P, _L, _L, _P, _P, _P]),
    "ekv_append_static": (C.c_int, [_D, _P, _P, _L, _L, _P, _P]),
    "ekv_topk_select": (C.c_int, [_D, _P, _L, _L, _I, _I, _I, _P, _L, _P, _L, _P, _P, _P, _L, _L, _P, _P]),
    "ekv_copy_timeouts": (C.c_int, [_P]),
    "ekv_topk_decode_stream_supported": (C.c_int, [_D, _I, _I, _I, _I]),
    "ekv_topk_decode_stream": (C.c_int, [_D, _P, _L, _L, _I, _I, _I, _F, _I, _P, _L, _P, _L, _P, _P, _P, _P,
                                         _L, _L, _P, _P, _Z, _P, _P]),
    "ekv_topk_decode_stream_scratch_bytes": (_Z, []),
    "ekv_stage_inputs": (C.c_int, [_P, _P, _Z, _P, _P, _Z, _P, _P, _Z, _P]),
    "ekv_topk_decode_fused_supported": (C.c_int, [_D, _I, _I, _I, _I]),
    "ekv_topk_decode_fused": (C.c_int, [_D, _P, _L, _L, _I, _I, _I, _F, _I, _P, _L, _P, _L, _P, _P, _P, _P,
                                        _L, _L, _P, _P]),
    "ekv_page_scores": (C.c_int, [_D, _P, _L, _L, _I, _I, _P, _L, _P]),
    "ekv_page_scores_alibi": (C.c_int, [_D, _P, _L, _L, _I, _I, _P, _L, _P, _P, _P]),
    "ekv_topk_pack": (C.c_int, [_D, _I, _I, _I, _P, _L, _P, _L, _P, _P, _P, _L, _L, _P, _P]),
    "ekv_gaussian_workspace_bytes": (_Z, [_I, _I, _I]),
    "ekv_gaussian_moments": (C.c_int, [_D, _P, _L, _L, _I, _I, _I, _F, _I, _P, _P, _L, _P, _P, _P, _Z, _P]),
    "ekv_gaussian_moments_alibi": (C.c_int, [_D, _P, _L, _L, _I, _I, _I, _F, _P, _P, _L, _P, _P, _P, _Z, _P, _P, _P]),
    "ekv_gaussian_finalize": (C.c_int, [_P, _P, _P, _I, _I, _F, _P, _P]),
    "ekv_gaussian_finalize_from_lengths": (C.c_int, [_P, _P, _I, _I, _I, _F, _P, _P]),
    "ekv_gaussian_select": (C.c_int, [_D, _I, _I, _I, _I, _F, _F, _F, _F, _F, _I, _P, _P, _P, _L, _P,
                                      _P, _L, _P, _P, _P, _P, _P, _P, _P, _P]),
    "ekv_tau_clamp": (C.c_int, [_P, _L, _P, _P, _I, _F, _F, _P, _P]),
    "ekv_decode_workspace_bytes": (_Z, [_I, _I, _I, _I]),
    "ekv_decode_workspace_reset": (C.c_int, [_P, _I, _I, _P]),
    "ekv_work_items_per_head": (C.c_int32, [_I]),
    "ekv_build_work_items": (C.c_int, [_P, _I, _I, _P, _P]),
    "ekv_decode_scores": (C.c_int, [_D, _P, _L, _L, _I, _P, _L, _P, _I, _F, _I, _I, _P, _P, _P, _I, _P, _P, _Z, _P]),
    "ekv_decode": (C.c_int, [_D, _P, _L, _L, _I, _P, _L, _P, _I, _F, _I, _I, _P, _P, _L, _L, _P, _I, _P, _P, _Z, _P, _P]),
    "ekv_decode_alibi": (C.c_int, [_D, _P, _L, _L, _I, _P, _L, _P, _I, _F, _I, _I, _P, _P, _L, _L, _P, _I, _P, _P, _Z, _P,
                                   _P, _P, _P]),
    "ekv_group_union": (C.c_int, [_D, _I, _P, _L, _P, _I, _P, _L, _P, _L, _P, _P, _I, _P, _P]),
    "ekv_decode_grouped": (C.c_int, [_D, _P, _L, _L, _I, _P, _L, _P, _I, _F, _I, _I, _P, _P, _L, _L, _P, _I, _P, _I,
                                     _P, _L, _P, _Z, _P, _P]),
    "ekv_halley_update": (C.c_int, [_P, _P, _I, _F, _P]),
    "ekv_decode_values": (C.c_int, [_D, _I, _P, _L, _P, _I, _F, _P, _P, _L, _L, _I, _P, _I, _P, _P, _Z, _P]),
    "ekv_exchange_create": (C.c_int, [_I, _I, _I, C.POINTER(C.c_void_p)]),
    "ekv_exchange_handle": (C.c_int, [_P, _P]),
    "ekv_exchange_connect": (C.c_int, [_P, _P]),
    "ekv_exchange_base": (C.c_void_p, [_P]),
    "ekv_exchange_connect_pointers": (C.c_int, [_P, C.POINTER(C.c_void_p)]),
    "ekv_exchange_set_spin_limit": (C.c_int, [_P, C.c_uint32]),
    "ekv_exchange_destroy": (C.c_int, [_P]),
    "ekv_exchange_allreduce": (C.c_int, [_P, _I, _P, _P, _I, _I, _P, _P]),
    "ekv_exchange_gaussian_finalize": (C.c_int, [_P, _P, _P, _I, _I, _I, _F, _P, _P, _P]),
    "ekv_exchange_gaussian_moments": (C.c_int, [_P, _D, _P, _L, _L, _I, _I, _I, _F, _P, _P, _P, _L, _P, _P, _P, _Z, _P, _P]),
    "ekv_exchange_gaussian_select": (C.c_int, [_P, _D, _I, _I, _I, _I, _F, _F, _F, _F, _F, _I, _P, _P, _P, _L, _P,
                                               _P, _L, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "ekv_exchange_tau_clamp": (C.c_int, [_P, _P, _P, _P, _I, _F, _F, _P, _P]),
    "ekv_exchange_halley_update": (C.c_int, [_P, _P, _P, _I, _F, _P, _P]),
    "ekv_exchange_decode": (C.c_int, [_P, _D, _P, _L, _L, _I, _P, _L, _P, _I, _F, _I, _P, _P, _P, _L, _L, _I,
                                      _P, _I, _P, _P, _Z, _P, _P]),
    "ekv_exchange_decode_grouped": (C.c_int, [_P, _D, _P, _L, _L, _I, _P, _L, _P, _I, _F, _I, _P, _P, _P, _L, _L, _I,
                                              _P, _I, _P, _I, _P, _L, _P, _Z, _P, _P]),
    "ekv_exchange_output": (C.c_int, [_P, _P, _I, _I, _P, _L, _I, _P, _P]),
    "ekv_decode_support_counts": (C.c_int, [_P, _Z, _I, _I, _I, _I, _P, _P]),
    "ekv_translate_pages": (C.c_int, [_D, _I, _P, _L, _P, _P, _L, _P]),
    "ekv_read_status": (C.c_int, [_P, C.POINTER(C.c_int32), _P]),
    "ekv_version": (C.c_int, []),
}

_lib = None


def load() -> C.CDLL:
    """Load the shared library (once). Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m entmaxkv_b200.build` "
                "(nvcc, sm_100a). There is no CPU or PyTorch fallback.")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(code: int, what: str) -> None:
    if code == 0:
        return
    if code < 0:
        raise ValueError(f"{what}: {_ERRORS.get(code, code)}")
    raise RuntimeError(f"{what}: CUDA error {code} at launch")


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPES[dt]
    except KeyError:
        raise ValueError(f"unsupported dtype {dt}; use float16, bfloat16 or float32") from None


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_ptr() -> int:
    """The current CUDA stream of the current device as a plain ``cudaStream_t`` value.  (Through torch's raw
    accessor when it exists: building a ``torch.cuda.Stream`` object costs ~6 us per call, a seventh of the host
    time of a whole eager decode step.)"""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("entmaxkv_b200 runs on CUDA tensors only (sm_100a); got a CPU tensor")
