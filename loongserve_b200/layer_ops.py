"""Element-wise layer ops with the reference's names (the pybind functions of ``longserve_cuda_kernels``,
longserve_cuda_kernels/src/entrypoints.cpp:15-101): ``rms_norm``, ``rotary_emb``, ``silu_and_mul_inplace`` and the
host-level fusion ``ffn_block``.  Matrix products are cuBLAS through ``torch.mm`` as in the reference."""
from __future__ import annotations

import torch

from . import _lib
from ._util import dtype_tag, need_cuda, ptr, stream_ptr


@torch.inference_mode()
def rms_norm(input: torch.Tensor, weight: torch.Tensor, eps: float, out=None) -> torch.Tensor:
    need_cuda(input, weight)
    assert input.dim() == 2 and weight.dim() == 1 and input.size(1) == weight.size(0)
    assert input.is_contiguous() and weight.is_contiguous() and weight.dtype == input.dtype
    output = torch.empty_like(input) if out is None else out
    rc = _lib.attn().esp_rms_norm(ptr(output), ptr(input), ptr(weight), input.size(0), input.size(1), float(eps),
                                  dtype_tag(input), stream_ptr())
    _lib.check(rc, "esp_rms_norm")
    return output


def _rotary_single(x, cos, sin):
    assert x.dim() == 3 and x.stride(2) == 1
    tokens, heads, head_dim = x.shape
    assert cos.shape == sin.shape == (tokens, head_dim // 2) and cos.is_contiguous() and sin.is_contiguous()
    assert cos.dtype == x.dtype and sin.dtype == x.dtype
    rc = _lib.attn().esp_rotary_emb(ptr(x), ptr(cos), ptr(sin), x.stride(0), x.stride(1), tokens, heads, head_dim,
                                    dtype_tag(x), stream_ptr())
    _lib.check(rc, "esp_rotary_emb")


@torch.inference_mode()
def rotary_emb(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> None:
    """In place on q and k (k may be the K half of a [tokens, 2*Hkv, D] cache view)."""
    need_cuda(q, k, cos, sin)
    _rotary_single(q, cos, sin)
    _rotary_single(k, cos, sin)


@torch.inference_mode()
def silu_and_mul_inplace(io: torch.Tensor) -> None:
    need_cuda(io)
    assert io.dim() == 2 and io.is_contiguous()
    rc = _lib.attn().esp_silu_and_mul_inplace(ptr(io), io.size(0), io.size(1) // 2, dtype_tag(io), stream_ptr())
    _lib.check(rc, "esp_silu_and_mul_inplace")


@torch.inference_mode()
def ffn_block(input_embds, norm_weight, norm_eps: float, gate_up_proj, down_proj) -> torch.Tensor:
    """rms_norm -> mm(gate_up) -> silu*mul -> mm(down), reusing the norm buffer as the output
    (entrypoints.cpp:89-101)."""
    input_normed = rms_norm(input_embds, norm_weight, norm_eps)
    up_gate_out = torch.mm(input_normed, gate_up_proj)
    silu_and_mul_inplace(up_gate_out)
    torch.mm(up_gate_out[:, : up_gate_out.size(-1) // 2], down_proj, out=input_normed)
    return input_normed
