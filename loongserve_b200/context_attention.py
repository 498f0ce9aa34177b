"""Ring-prefill attention step; same signature and in-place semantics as the reference's
``context_attention_fwd`` (loongserve/models/llama/triton_kernel/ring_context_flashattention_nopad.py:191-284).
"""
from __future__ import annotations

import torch

from . import _lib
from ._util import dtype_tag, need_cuda, need_i32, ptr, stream_ptr


@torch.inference_mode()
def context_attention_fwd(q, k, v, o, q_b_start_loc, q_b_seq_len, q_first_token_global_idx,
                          kv_b_start_loc, kv_b_seq_len, kv_first_token_global_idx,
                          logical_sp_peers_num: int, max_q_b_seq_len: int, m, l, sm_scale: float = 0.0,
                          kv_pos_stride: int = None):
    """Attention between the local q and one local/remote KV block, merged into (o, m, l) in place.

    q, o: [num_q_tokens, num_q_heads, head_dim]; k, v: [num_kv_tokens, num_kv_heads, head_dim] (views
    with a contiguous last dimension are fine, e.g. the two halves of a [tokens, 2*Hkv, D] buffer);
    m, l: fp32 [num_q_tokens, num_q_heads]; the six metadata vectors are int32 [batch].
    ``o`` may be q's dtype (reference behaviour) or float32.  Before the first step of a ring pass
    set m = -inf and l = 0 (o need not be cleared).

    ``kv_pos_stride`` (default: ``logical_sp_peers_num``) is the position stride of consecutive keys when it differs from
    that of consecutive q rows (``logical_sp_peers_num``): 1 for a buffer that holds the other instances' rows in position order.
    """
    need_cuda(q, k, v, o, m, l, q_b_start_loc)
    need_i32(q_b_start_loc, q_b_seq_len, q_first_token_global_idx, kv_b_start_loc, kv_b_seq_len,
             kv_first_token_global_idx)
    Lq, Lk, Lv = q.shape[-1], k.shape[-1], v.shape[-1]
    assert Lq == Lk and Lk == Lv
    assert q.dim() == 3 and k.dim() == 3 and v.dim() == 3 and o.shape == q.shape
    assert q.stride(2) == 1 and k.stride(2) == 1 and v.stride(2) == 1 and o.stride(2) == 1
    assert k.dtype == q.dtype and v.dtype == q.dtype
    assert k.shape == v.shape and k.stride() == v.stride(), "k and v must share shape and strides"
    assert m.dtype == torch.float32 and l.dtype == torch.float32 and m.is_contiguous() and l.is_contiguous()
    assert m.shape == (q.shape[0], q.shape[1]) and l.shape == m.shape
    batch = q_b_seq_len.shape[0]
    rc = _lib.attn().esp_prefill_step_strided(
        ptr(q), q.stride(0), q.stride(1), q.shape[0],
        ptr(k), ptr(v), k.stride(0), k.stride(1), k.shape[0],
        ptr(o), o.stride(0), o.stride(1), ptr(m), ptr(l),
        ptr(q_b_start_loc), ptr(q_b_seq_len), ptr(q_first_token_global_idx),
        ptr(kv_b_start_loc), ptr(kv_b_seq_len), ptr(kv_first_token_global_idx),
        batch, q.shape[1], k.shape[1], Lq, int(logical_sp_peers_num),
        int(logical_sp_peers_num if kv_pos_stride is None else kv_pos_stride), int(max_q_b_seq_len),
        dtype_tag(q), dtype_tag(o), float(sm_scale), stream_ptr())
    _lib.check(rc, "esp_prefill_step_strided")


@torch.inference_mode()
def init_attention_state(o, m, l):
    """o = 0, m = -inf, l = 0 (what the reference does before the first ring step,
    longserve_transformer_layer_infer.py:123-126)."""
    need_cuda(o, m, l)
    assert m.is_contiguous() and l.is_contiguous() and m.dtype == torch.float32 and l.dtype == torch.float32
    o_bytes = o.numel() * o.element_size() if (o is not None and o.is_contiguous()) else 0
    if o is not None and not o.is_contiguous():
        o.zero_()
    rc = _lib.attn().esp_prefill_state_init(ptr(o) if o_bytes else 0, o_bytes, ptr(m), ptr(l), m.numel(), stream_ptr())
    _lib.check(rc, "esp_prefill_state_init")


@torch.inference_mode()
def attention_lse(m, l, out=None):
    """Natural-log log-sum-exp of the keys seen so far: ln2*m + ln(l)."""
    need_cuda(m, l)
    out = torch.empty_like(m) if out is None else out
    rc = _lib.attn().esp_prefill_lse(ptr(m), ptr(l), ptr(out), m.numel(), stream_ptr())
    _lib.check(rc, "esp_prefill_lse")
    return out


def device_status(clear: bool = True):
    """(code, block, wait id, detail) of the bounded in-kernel waits; code 0 means no wait expired."""
    import ctypes as C
    buf = (C.c_int32 * 4)()
    _lib.check(_lib.attn().esp_device_status(buf, 1 if clear else 0), "esp_device_status")
    return tuple(buf)
