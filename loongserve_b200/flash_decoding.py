"""Distributed flash-decoding ops with the reference's names and argument order.

``flash_decoding_stage1`` / ``flash_decoding_stage2`` correspond to the pybind functions of
``longserve_cuda_kernels`` (longserve_cuda_kernels/src/entrypoints.cpp:103-221); the
``longserve_*`` wrappers to loongserve/models/llama/triton_kernel/longserve_flash_decoding*.py.
"""
from __future__ import annotations

import torch

from . import _lib
from ._util import dtype_tag, need_cuda, need_i32, ptr, stream_ptr


@torch.inference_mode()
def flash_decoding_stage1(mid_o, mid_o_logexpsum, q, k, v, req_to_tokens, b_req_idx, b_seqlen,
                          max_len_in_batch: int, seq_block_size: int, sm_scale: float = 0.0):
    need_cuda(mid_o, mid_o_logexpsum, q, k, v, req_to_tokens, b_req_idx, b_seqlen)
    assert mid_o.is_contiguous() and mid_o_logexpsum.is_contiguous() and q.is_contiguous()
    assert k.stride(2) == 1 and v.stride(2) == 1 and req_to_tokens.is_contiguous()
    assert mid_o.dim() == 4 and mid_o_logexpsum.dim() == 3 and q.dim() == 3 and k.dim() == 3 and v.dim() == 3
    assert mid_o.dtype == torch.float32 and mid_o_logexpsum.dtype == torch.float32
    assert k.dtype == q.dtype and v.dtype == q.dtype and req_to_tokens.dtype == torch.int32
    need_i32(b_req_idx, b_seqlen)
    nblk = (int(max_len_in_batch) + int(seq_block_size) - 1) // int(seq_block_size)
    assert mid_o.shape[0] >= nblk and mid_o.shape[1] == q.shape[0] and mid_o.shape[2] == q.shape[1]
    rc = _lib.attn().esp_decode_stage1(
        ptr(mid_o), ptr(mid_o_logexpsum), ptr(q), ptr(k), ptr(v), k.stride(0), k.stride(1), v.stride(0),
        v.stride(1), ptr(req_to_tokens), req_to_tokens.stride(0), ptr(b_req_idx), ptr(b_seqlen),
        q.shape[0], q.shape[1], k.shape[1], q.shape[2], int(max_len_in_batch), int(seq_block_size),
        dtype_tag(q), float(sm_scale), min(k.shape[0], v.shape[0]), stream_ptr())
    _lib.check(rc, "esp_decode_stage1")


@torch.inference_mode()
def flash_decoding_stage2(o, out_logexpsum, b_seqlen, mid_o, mid_o_logexpsum, block_seq: int):
    need_cuda(o, out_logexpsum, b_seqlen, mid_o, mid_o_logexpsum)
    assert o.is_contiguous() and out_logexpsum.is_contiguous() and mid_o.is_contiguous() and mid_o_logexpsum.is_contiguous()
    assert o.dim() == 3 and out_logexpsum.dim() == 2 and mid_o.dim() == 4 and mid_o_logexpsum.dim() == 3
    assert out_logexpsum.dtype == torch.float32 and mid_o.dtype == torch.float32
    need_i32(b_seqlen)
    rc = _lib.attn().esp_decode_merge(ptr(o), ptr(out_logexpsum), ptr(b_seqlen), ptr(mid_o), ptr(mid_o_logexpsum),
                                      o.shape[0], o.shape[1], o.shape[2], mid_o.shape[0], int(block_seq),
                                      dtype_tag(o), stream_ptr())
    _lib.check(rc, "esp_decode_merge")


def longserve_flash_decode_stage1(q, k, v, Req_to_tokens, B_req_idx, B_Seqlen, max_len_in_batch, mid_out,
                                  mid_out_logsumexp, block_seq):
    """longserve_flash_decoding_stage1.py:78-88."""
    flash_decoding_stage1(mid_out, mid_out_logsumexp, q, k, v, Req_to_tokens, B_req_idx, B_Seqlen,
                          max_len_in_batch, block_seq)


def longserve_flash_decode_stage2(mid_out, mid_out_logexpsum, B_Seqlen, O, out_logexpsum, block_seq):
    """longserve_flash_decoding_stage2.py:53-61."""
    flash_decoding_stage2(O, out_logexpsum, B_Seqlen, mid_out, mid_out_logexpsum, block_seq)


def longserve_token_decode_attention_flash_decoding(q, req_to_token_indexs, b_req_idx, b_seq_len, mid_o,
                                                    mid_o_logexpsum, batch_size, max_len_in_batch, q_head_num,
                                                    head_dim, cache_k, cache_v, BLOCK_SEQ, out=None,
                                                    o_logexpsum=None):
    """Peer-side stage 1 + stage 2 for foreign queries -> (o fp32, lse fp32)
    (longserve_flash_decoding.py:3-28)."""
    shape = (-1, q_head_num, head_dim)
    o_tensor = torch.empty_like(q, dtype=torch.float32) if out is None else out
    out_lse = torch.empty([batch_size, q_head_num], dtype=torch.float32, device=q.device) if o_logexpsum is None else o_logexpsum
    longserve_flash_decode_stage1(q.view(shape), cache_k, cache_v, req_to_token_indexs, b_req_idx, b_seq_len,
                                  max_len_in_batch, mid_o, mid_o_logexpsum, BLOCK_SEQ)
    longserve_flash_decode_stage2(mid_o, mid_o_logexpsum, b_seq_len, o_tensor.view(shape), out_lse, BLOCK_SEQ)
    return o_tensor, out_lse


def device_status(clear: bool = True):
    """(code, block, which, value) of the decode kernels and flag waits on the current device: code 0, or
    ESP_ERR_DEVICE_TIMEOUT (-4) for a flag wait that ran out, or ESP_ERR_BAD_SLOT (-8) for a slot id outside the pool
    (that token was left out).  Synchronises the device."""
    import ctypes as C
    buf = (C.c_int32 * 4)()
    _lib.check(_lib.attn().esp_decode_device_status(buf, 1 if clear else 0), "esp_decode_device_status")
    return tuple(buf)


def set_wait_limit_cycles(cycles: int):
    """Limit of every bounded in-kernel wait on the current device, in SM cycles (default 2e9, about a second)."""
    _lib.check(_lib.attn().esp_set_wait_limit_cycles(int(cycles)), "esp_set_wait_limit_cycles")
