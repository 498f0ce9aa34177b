"""Token-granular KV pool ops with the reference's names and argument order.  All are bit-exact
copies / integer arithmetic executed by the CUDA library; outputs are written in place."""
from __future__ import annotations

import torch

from . import _lib
from ._util import idx64_flag, need_cuda, need_i32, ptr, stream_ptr


def _rows(t):
    assert t.dim() == 3 and t.stride(2) == 1, "expected [tokens, heads, head_dim] with contiguous head_dim"
    return t.shape[1], t.shape[2], t.element_size()


@torch.inference_mode()
def destindex_copy_kv(K, DestLoc, Out):
    """Out[DestLoc[i]] = K[i] (loongserve/common/basemodel/triton_kernel/destindex_copy_kv.py:32-51)."""
    need_cuda(K, DestLoc, Out)
    heads, dim, eb = _rows(K)
    assert Out.shape[1] == heads and Out.shape[2] == dim and Out.dtype == K.dtype and DestLoc.is_contiguous()
    rc = _lib.attn().esp_kv_scatter(ptr(K), K.stride(0), K.stride(1), ptr(Out), Out.stride(0), Out.stride(1),
                                    ptr(DestLoc), idx64_flag(DestLoc), DestLoc.shape[0], heads, dim, eb, Out.shape[0],
                                    stream_ptr())
    _lib.check(rc, "esp_kv_scatter")


@torch.inference_mode()
def pre_copy_and_register_kv(kv_cache_index_begin, kv_cache_index_end, kv_first_token_global_idx,
                             num_logical_sp_peers: int):
    """(kv_range_begin, kv_range_end, new_kv_cache_len)
    (loongserve/models/llama/triton_kernel/copy_and_register_kv.py:34-61)."""
    need_cuda(kv_cache_index_begin)
    need_i32(kv_cache_index_begin, kv_cache_index_end, kv_first_token_global_idx)
    rb = torch.empty_like(kv_cache_index_begin)
    re = torch.empty_like(kv_cache_index_begin)
    nl = torch.empty_like(kv_cache_index_begin)
    rc = _lib.attn().esp_kv_keep_range(ptr(kv_cache_index_begin), ptr(kv_cache_index_end),
                                       ptr(kv_first_token_global_idx), int(num_logical_sp_peers),
                                       kv_cache_index_begin.shape[0], ptr(rb), ptr(re), ptr(nl), stream_ptr())
    _lib.check(rc, "esp_kv_keep_range")
    return rb, re, nl


@torch.inference_mode()
def destindex_copy_and_register_kv(batch_size, new_kv_cache_len, kv_range_begin, kv_range_end, new_kv_cache_len_sum,
                                   kv, kv_b_start_loc, cur_kv_cache_index, mem_index, total_kv_cache,
                                   req_to_token_indexs, b_req_idx, num_used_mem_index: int, max_len_in_batch: int,
                                   should_register_kv: bool):
    """copy_and_register_kv.py:123-169."""
    need_cuda(kv, total_kv_cache, mem_index)
    need_i32(new_kv_cache_len, kv_range_begin, kv_range_end, kv_b_start_loc, cur_kv_cache_index, b_req_idx)
    assert new_kv_cache_len_sum.dtype == torch.int64 and new_kv_cache_len_sum.is_contiguous()
    heads, dim, eb = _rows(kv)
    assert total_kv_cache.shape[1] == heads and total_kv_cache.shape[2] == dim
    assert req_to_token_indexs.dtype == torch.int32 and req_to_token_indexs.stride(1) == 1 and mem_index.is_contiguous()
    rc = _lib.attn().esp_kv_scatter_register(
        int(batch_size), ptr(new_kv_cache_len), ptr(kv_range_begin), ptr(kv_range_end), ptr(new_kv_cache_len_sum),
        ptr(kv), kv.stride(0), kv.stride(1), ptr(kv_b_start_loc), ptr(cur_kv_cache_index), ptr(mem_index),
        idx64_flag(mem_index), ptr(total_kv_cache), total_kv_cache.stride(0), total_kv_cache.stride(1),
        ptr(req_to_token_indexs), req_to_token_indexs.stride(0), ptr(b_req_idx), int(num_used_mem_index),
        int(max_len_in_batch), 1 if should_register_kv else 0, heads, dim, eb, total_kv_cache.shape[0], stream_ptr())
    _lib.check(rc, "esp_kv_scatter_register")


@torch.inference_mode()
def copy_kv_index_to_req(req_to_token_indexs, b_req_idx, b_seq_len, memindex):
    """loongserve/common/basemodel/triton_kernel/copy_kv_index_to_req.py:22-38."""
    need_cuda(req_to_token_indexs, b_req_idx, b_seq_len, memindex)
    need_i32(b_req_idx, b_seq_len)
    assert b_seq_len.shape[0] == memindex.shape[0] and b_req_idx.shape[0] == b_seq_len.shape[0]
    assert req_to_token_indexs.dtype == torch.int32 and req_to_token_indexs.stride(1) == 1
    rc = _lib.attn().esp_kv_index_register(ptr(req_to_token_indexs), req_to_token_indexs.stride(0), ptr(b_req_idx),
                                           ptr(b_seq_len), ptr(memindex), idx64_flag(memindex), b_seq_len.shape[0],
                                           stream_ptr())
    _lib.check(rc, "esp_kv_index_register")


@torch.inference_mode()
def init_req_to_token_indexes(req_to_token_indexs, b_req_idx, b_seq_len, alloc_mem_index, max_len_in_batch=None):
    """loongserve/common/infer_utils.py:1-13, without the host loop and its device->host copies.
    ``max_len_in_batch`` bounds the per-request copy grid; it defaults to the table width."""
    need_cuda(req_to_token_indexs, b_req_idx, b_seq_len, alloc_mem_index)
    need_i32(b_req_idx, b_seq_len)
    assert req_to_token_indexs.dtype == torch.int32 and req_to_token_indexs.stride(1) == 1
    mx = int(max_len_in_batch) if max_len_in_batch is not None else req_to_token_indexs.shape[1]
    rc = _lib.attn().esp_kv_index_init(ptr(req_to_token_indexs), req_to_token_indexs.stride(0), ptr(b_req_idx),
                                       ptr(b_seq_len), ptr(alloc_mem_index), idx64_flag(alloc_mem_index),
                                       b_seq_len.shape[0], mx, stream_ptr())
    _lib.check(rc, "esp_kv_index_init")


def _mig_common(buf, kv_cache, num_tokens):
    assert kv_cache.dim() == 4 and kv_cache.stride(3) == 1 and kv_cache.stride(2) == kv_cache.shape[3]
    assert buf.is_contiguous() and buf.dim() == 4 and buf.shape[0] == kv_cache.shape[0]
    assert buf.shape[2:] == kv_cache.shape[2:] and buf.dtype == kv_cache.dtype
    cumsum = torch.cumsum(num_tokens, dim=0, dtype=torch.int64)
    return cumsum


@torch.inference_mode()
def decoding_stage_migration_sender_kernel(send_buf, req_to_token_indexes, mem_state, kv_cache, request_ids,
                                           num_tokens, b_seq_len, max_num_tokens=None):
    """loongserve/models/llama/triton_kernel/decoding_stage_migration.py:71-95.
    ``max_num_tokens`` (optional, host int >= max(num_tokens)) avoids the device->host read the
    reference performs; it defaults to send_buf.shape[1]."""
    need_cuda(send_buf, kv_cache, mem_state)
    need_i32(request_ids, num_tokens, b_seq_len)
    assert mem_state.dtype == torch.int32
    cumsum = _mig_common(send_buf, kv_cache, num_tokens)
    mx = int(max_num_tokens) if max_num_tokens is not None else send_buf.shape[1]
    rc = _lib.attn().esp_mig_gather(ptr(send_buf), send_buf.shape[1], ptr(req_to_token_indexes),
                                    req_to_token_indexes.stride(0), ptr(mem_state), ptr(kv_cache), kv_cache.stride(0),
                                    kv_cache.stride(1), ptr(request_ids), ptr(num_tokens), ptr(cumsum), ptr(b_seq_len),
                                    request_ids.shape[0], mx, kv_cache.shape[0], kv_cache.shape[2], kv_cache.shape[3],
                                    kv_cache.element_size(), kv_cache.shape[1], stream_ptr())
    _lib.check(rc, "esp_mig_gather")


@torch.inference_mode()
def decoding_stage_migration_receiver_kernel(recv_buf, req_to_token_indexes, kv_cache, alloc_mem, request_ids,
                                             num_tokens, b_seq_len, max_num_tokens=None):
    """decoding_stage_migration.py:160-184."""
    need_cuda(recv_buf, kv_cache, alloc_mem)
    need_i32(request_ids, num_tokens, b_seq_len)
    cumsum = _mig_common(recv_buf, kv_cache, num_tokens)
    mx = int(max_num_tokens) if max_num_tokens is not None else recv_buf.shape[1]
    rc = _lib.attn().esp_mig_scatter(ptr(recv_buf), recv_buf.shape[1], ptr(req_to_token_indexes),
                                     req_to_token_indexes.stride(0), ptr(kv_cache), kv_cache.stride(0),
                                     kv_cache.stride(1), ptr(alloc_mem), idx64_flag(alloc_mem), ptr(request_ids),
                                     ptr(num_tokens), ptr(cumsum), ptr(b_seq_len), request_ids.shape[0], mx,
                                     kv_cache.shape[0], kv_cache.shape[2], kv_cache.shape[3], kv_cache.element_size(),
                                     kv_cache.shape[1], stream_ptr())
    _lib.check(rc, "esp_mig_scatter")


def device_status(clear: bool = True):
    """(code, kernel, position, slot id) of the slot-id checks of the pool kernels on the current device; code 0 = every
    id seen so far was inside its pool.  Synchronises the device."""
    import ctypes as C
    buf = (C.c_int32 * 4)()
    _lib.check(_lib.attn().esp_kv_device_status(buf, 1 if clear else 0), "esp_kv_device_status")
    return tuple(buf)
