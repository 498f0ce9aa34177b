"""ctypes bindings of the C ABI (include/esp_attention.h, include/esp_rnccl.h).

There is no fallback: if the CUDA library is missing this module raises, and every op raises
RuntimeError on a non-zero status.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# ESP_ATTENTION_LIB may point at another build of the same library (kernel tuning experiments)
ATTN_LIB = os.environ.get("ESP_ATTENTION_LIB") or os.path.join(HERE, "libesp_attention.so")
RNCCL_LIB = os.path.join(HERE, "libesp_rnccl.so")

ESP_DTYPE_F16, ESP_DTYPE_BF16, ESP_DTYPE_F32 = 0, 1, 2

_i32, _i64, _f32, _vp = C.c_int32, C.c_int64, C.c_float, C.c_void_p

# name -> argtypes, exactly as declared in include/esp_attention.h
ESP_ABI_VERSION = 4      # what esp_abi_version() of a matching library returns (see include/esp_attention.h)

ATTN_SIGNATURES = {
    "esp_abi_version": [],
    "esp_prefill_step": [_vp, _i64, _i64, _i64, _vp, _vp, _i64, _i64, _i64, _vp, _i64, _i64, _vp, _vp,
                         _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _f32, _vp],
    "esp_prefill_step_strided": [_vp, _i64, _i64, _i64, _vp, _vp, _i64, _i64, _i64, _vp, _i64, _i64, _vp, _vp,
                                 _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _f32, _vp],
    "esp_prefill_state_init": [_vp, _i64, _vp, _vp, _i64, _vp],
    "esp_prefill_lse": [_vp, _vp, _vp, _i64, _vp],
    "esp_device_status": [C.POINTER(_i32), _i32],
    "esp_set_wait_limit_cycles": [_i64],
    "esp_decode_stage1": [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _i64, _vp, _vp,
                          _i32, _i32, _i32, _i32, _i32, _i32, _i32, _f32, _i64, _vp],
    "esp_decode_merge": [_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp],
    "esp_decode_attention_noalloc": [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _i64, _vp, _vp,
                                     _i32, _i32, _i32, _i32, _i32, _i32, _i32, _f32, _i64, _vp],
    "esp_peer_buffer_create": [_i64, C.POINTER(_vp), C.POINTER(C.c_uint8)],
    "esp_peer_buffer_open": [C.POINTER(C.c_uint8), C.POINTER(_vp)],
    "esp_peer_buffer_close": [_vp],
    "esp_peer_buffer_destroy": [_vp],
    "esp_peer_push": [_vp, C.POINTER(_vp), C.POINTER(_vp), _i32, _i64, _i32, _vp, _vp],
    "esp_peer_signal": [_vp, _i32, _vp, _vp],
    "esp_flag_wait": [_vp, _i32, _vp, _i32, _i32, _vp],
    "esp_memcpy_async": [_vp, _vp, _i64, _vp],
    "esp_kv_device_status": [C.POINTER(_i32), _i32],
    "esp_decode_stage1_gated": [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _i64, _vp, _vp,
                                _i32, _i32, _i32, _i32, _i32, _i32, _i32, _f32, _i64, _vp, _i32, _vp, _vp],
    "esp_decode_merge_gated": [_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _i32, _i32, _vp, _vp],
    "esp_decode_device_status": [C.POINTER(_i32), _i32],
    "esp_kv_scatter": [_vp, _i64, _i64, _vp, _i64, _i64, _vp, _i32, _i64, _i32, _i32, _i32, _i64, _vp],
    "esp_kv_keep_range": [_vp, _vp, _vp, _i32, _i32, _vp, _vp, _vp, _vp],
    "esp_kv_scatter_register": [_i32, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _vp, _vp, _vp, _i32, _vp, _i64,
                                _i64, _vp, _i64, _vp, _i64, _i32, _i32, _i32, _i32, _i32, _i64, _vp],
    "esp_kv_index_register": [_vp, _i64, _vp, _vp, _vp, _i32, _i32, _vp],
    "esp_kv_index_init": [_vp, _i64, _vp, _vp, _vp, _i32, _i32, _i32, _vp],
    "esp_mig_gather": [_vp, _i64, _vp, _i64, _vp, _vp, _i64, _i64, _vp, _vp, _vp, _vp, _i32, _i32, _i32,
                       _i32, _i32, _i32, _i64, _vp],
    "esp_mig_scatter": [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _vp, _i32, _vp, _vp, _vp, _vp, _i32, _i32,
                        _i32, _i32, _i32, _i32, _i64, _vp],
    "esp_pool_create": [_i64, C.POINTER(_vp)],
    "esp_pool_destroy": [_vp],
    "esp_pool_alloc": [_vp, _i64, _vp],
    "esp_pool_alloc_contiguous": [_vp, _i64, C.POINTER(_i64)],
    "esp_pool_add_refs": [_vp, _vp, _i64],
    "esp_pool_decrease_refs": [_vp, _vp, _i64],
    "esp_pool_free_all": [_vp],
    "esp_pool_state": [_vp, _vp],
    "esp_memcpy_2d": [_vp, _i64, _vp, _i64, _i64, _i64, _i32, _vp],
    "esp_sched_minimize_prefill_iteration_time": [_i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64],
    "esp_sched_plan_prefill": [_i64, _vp, _i64, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _vp],
    "esp_rms_norm": [_vp, _vp, _vp, _i64, _i32, _f32, _i32, _vp],
    "esp_rotary_emb": [_vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _i32, _vp],
    "esp_silu_and_mul_inplace": [_vp, _i64, _i32, _i32, _vp],
}
ATTN_STRING_FUNCS = {"esp_strerror": [_i32], "esp_last_cuda_error": []}

RNCCL_SIGNATURES = {
    "esp_rnccl_unique_id": [C.POINTER(C.c_uint8)],
    "esp_rnccl_create": [C.POINTER(C.c_uint8), _i32, _i32, C.POINTER(_vp)],
    "esp_rnccl_destroy": [_vp],
    "esp_rnccl_group_start": [_vp],
    "esp_rnccl_group_end": [_vp],
    "esp_rnccl_send": [_vp, _vp, _i64, _i32],
    "esp_rnccl_recv": [_vp, _vp, _i64, _i32],
    "esp_rnccl_fence_in": [_vp, _vp],
    "esp_rnccl_fence_out": [_vp, _vp],
}

_attn = None
_rnccl = None


def attn():
    """The attention library, loaded once.  Raises if it has not been built."""
    global _attn
    if _attn is None:
        if not os.path.exists(ATTN_LIB):
            raise RuntimeError(f"{ATTN_LIB} is missing: run `python -m loongserve_b200.build` (no CPU fallback exists)")
        lib = C.CDLL(ATTN_LIB, mode=C.RTLD_GLOBAL)
        for name, args in ATTN_SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = _i32
        for name, args in ATTN_STRING_FUNCS.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = C.c_char_p
        lib.esp_pool_can_use.argtypes = [_vp]
        lib.esp_pool_can_use.restype = _i64
        _attn = lib
    return _attn


def rnccl():
    """The raw NCCL layer, loaded once (import torch first so that one NCCL copy serves the process)."""
    global _rnccl
    if _rnccl is None:
        if not os.path.exists(RNCCL_LIB):
            raise RuntimeError(f"{RNCCL_LIB} is missing: run `python -m loongserve_b200.build`")
        lib = C.CDLL(RNCCL_LIB, mode=C.RTLD_GLOBAL)
        for name, args in RNCCL_SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = _i32
        lib.esp_rnccl_stream.argtypes = [_vp]
        lib.esp_rnccl_stream.restype = _vp
        lib.esp_rnccl_last_error.argtypes = []
        lib.esp_rnccl_last_error.restype = C.c_char_p
        _rnccl = lib
    return _rnccl


def check(rc: int, what: str) -> None:
    if rc != 0:
        lib = attn()
        msg = lib.esp_strerror(rc).decode()
        detail = lib.esp_last_cuda_error().decode()
        raise RuntimeError(f"{what} failed: {msg} ({rc})" + (f": {detail}" if detail and rc == -3 else ""))


def check_rnccl(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed ({rc}): {rnccl().esp_rnccl_last_error().decode()}")
