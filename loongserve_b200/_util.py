from __future__ import annotations

import torch

from . import _lib

_DT = {torch.float16: _lib.ESP_DTYPE_F16, torch.bfloat16: _lib.ESP_DTYPE_BF16, torch.float32: _lib.ESP_DTYPE_F32}


def dtype_tag(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}") from None


def ptr(t):
    return 0 if t is None else t.data_ptr()


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("the ESP attention ops run on CUDA tensors only (there is no CPU path)")


def need_i32(*ts):
    for t in ts:
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise TypeError("metadata vectors must be contiguous int32")


def idx64_flag(t: torch.Tensor) -> int:
    if t.dtype == torch.int64:
        return 1
    if t.dtype == torch.int32:
        return 0
    raise TypeError("index tensors must be int32 or int64")
