"""ctypes binding of libytensor_cuda.so (the C ABI declared in include/ytcuda.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libytensor_cuda.so"

OK, INVALID_ARG, UNSUPPORTED, CUDA_ERROR, TIMEOUT, NOT_IMPLEMENTED = range(6)
F32, BF16, F16, F8_E5M2, F8_E4M3, F8_E8M0 = 0, 1, 2, 3, 4, 5

_i, _i64, _f, _vp, _u64 = C.c_int, C.c_int64, C.c_float, C.c_void_p, C.c_uint64

# name -> (restype, argtypes); one entry per declaration in include/ytcuda.h
SIGNATURES = {
    "ytcuda_last_error_string": (C.c_char_p, []),
    "ytcuda_malloc": (_i, [C.POINTER(_vp), _u64]),
    "ytcuda_free": (_i, [_vp]),
    "ytcuda_host_alloc": (_i, [C.POINTER(_vp), _u64]),
    "ytcuda_host_free": (_i, [_vp]),
    "ytcuda_memcpy_h2d": (_i, [_vp, _vp, _u64, _vp]),
    "ytcuda_memcpy_d2h": (_i, [_vp, _vp, _u64, _vp]),
    "ytcuda_memcpy_d2d": (_i, [_vp, _vp, _u64, _vp]),
    "ytcuda_pointer_is_device": (_i, [_vp]),
    "ytcuda_stream_sync": (_i, [_vp]),
    "ytcuda_device_status": (_i, [_vp]),
    "ytcuda_launch_count": (_u64, []),
    "ytcuda_copy_counts": (None, [_vp, _vp]),
    "ytcuda_set_wait_limit": (_i, [_i64]),
    "ytcuda_get_wait_limit": (_i64, []),
    "ytcuda_wait_probe": (_i, [_vp, _vp]),
    "ytcuda_gemm": (_i, [_i, _i, _vp, _vp, _vp, _i, _i, _i, _f, _f] + [_i64] * 6 + [_i64] * 4 + [_vp]),
    "ytcuda_gemm_masked": (_i, [_i, _i, _vp, _vp, _vp, _i, _i, _i] + [_i64] * 6 + [_i64] * 4 + [_vp, _i64, _f, _vp]),
    "ytcuda_gemm_masked_causal": (_i, [_i, _i, _vp, _vp, _vp, _i, _i, _i] + [_i64] * 6 + [_i64] * 4 + [_i, _f, _vp]),
    "ytcuda_gemm_set_path": (_i, [_i]),
    "ytcuda_gemm_set_f32_mode": (_i, [_i]),
    "ytcuda_gemm_set_tuning": (_i, [_i, _i]),
    "ytcuda_gemm_set_pair_mode": (_i, [_i]),
    "ytcuda_gemm_host": (_i, [_i, _i, _vp, _vp, _vp, _i, _i, _i, _f, _f] + [_i64] * 6 + [_i64] * 4),
    "ytcuda_softmax": (_i, [_i, _i, _vp, _vp, _vp, _vp, _vp, _i, _vp, _i, _vp]),
    "ytcuda_rmsnorm": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _i, _f, _vp]),
    "ytcuda_normalize": (_i, [_i, _i, _vp, _vp, _vp, _vp, _vp, _i, _vp, _i, _f, _f, _vp]),
    "ytcuda_layernorm": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _i, _f, _vp]),
    "ytcuda_reduce": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _vp, _i, _vp]),
    "ytcuda_reduce_noalloc": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _vp, _i, _vp]),
    "ytcuda_reduce_noalloc_set_limit": (_i, [_u64]),
    "ytcuda_rmsnorm_add_softmax_cast": (_i, [_i, _vp, _vp, _vp, _vp, _i64, _i64, _i, _i, _f, _vp]),
    "ytcuda_binary": (_i, [_i, _i, _i, _i, _vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp]),
    "ytcuda_unary": (_i, [_i, _i, _i, _vp, _vp, _i, _vp, _vp, _vp, _f, _vp]),
    "ytcuda_cast": (_i, [_i, _i, _vp, _vp, _i, _vp, _vp, _vp, _vp]),
    "ytcuda_swiglu": (_i, [_i, _i, _vp, _vp, _i64, _i, _i64, _i64, _vp]),
    "ytcuda_flash_attn_fwd": (_i, [_i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _vp, _vp, _vp, _vp, _i, _i,
                                   _vp, _i64, _vp, _i64, _i64, _vp]),
    "ytcuda_attn_set_path": (_i, [_i]),
    "ytcuda_rope_tables": (_i, [_i, _i, _f, _vp, _vp]),
    "ytcuda_embedding": (_i, [_vp, _vp, _vp, _i64, _i, _i, _vp]),
    "ytcuda_linear_w16": (_i, [_vp, _i64, _vp, _vp, _i64, _i64, _i, _i, _i, _vp, _vp]),
    "ytcuda_qwen3_qkv_post": (_i, [_vp] * 8 + [_i] * 8 + [_f, _vp]),
    "ytcuda_topk_sample": (_i, [_vp, _i64, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "ytcuda_qwen3_create": (_vp, [_i] * 7 + [_f, _f, _i, _i, _i, _i]),
    "ytcuda_qwen3_destroy": (None, [_vp]),
    "ytcuda_qwen3_set_weight": (_i, [_vp, C.c_char_p, _i, _vp]),
    "ytcuda_qwen3_set_allreduce": (_i, [_vp, _vp, _vp]),
    "ytcuda_qwen3_reset": (_i, [_vp]),
    "ytcuda_qwen3_cache_len": (_i, [_vp]),
    "ytcuda_qwen3_set_decode_path": (_i, [_vp, _i]),
    "ytcuda_qwen3_set_trace": (_i, [_vp, _vp, _i]),
    "ytcuda_qwen3_tp_export": (_i, [_vp, _vp]),
    "ytcuda_qwen3_tp_import": (_i, [_vp, _i, _vp]),
    "ytcuda_qwen3_tp_disconnect": (_i, [_vp]),
    "ytcuda_qwen3_tp_resync": (_i, [_vp]),
    "ytcuda_qwen3_forward": (_i, [_vp, _vp, _i, _vp, _vp]),
}


class YtCudaError(RuntimeError):
    def __init__(self, status: int, msg: str):
        super().__init__(f"ytcuda status {status}: {msg}")
        self.status = status


class YtCudaInvalidArgument(YtCudaError, ValueError):
    """Mirrors std::invalid_argument thrown by the reference's API layer."""


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m ytensor_b200.build` "
                "(there is no CPU fallback)")
        L = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def last_error() -> str:
    return lib().ytcuda_last_error_string().decode("utf-8", "replace")


def check(status: int) -> None:
    if status == OK:
        return
    msg = last_error()
    if status in (INVALID_ARG, UNSUPPORTED):
        raise YtCudaInvalidArgument(status, msg)
    raise YtCudaError(status, msg)
