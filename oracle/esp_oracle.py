"""CPU oracle for the elastic-sequence-parallel attention hot path.

THIS IS TEST INFRASTRUCTURE, NOT THE PRODUCT.  Only the test-suite, the smoke check and the
CPU-baseline leg of the benchmark may import it; the product path (the CUDA library behind
``loongserve_b200``) never does and has no CPU fallback.

It restates, in plain fp32 torch/numpy on the CPU, the algorithms of the reference
(paths relative to the reference project):

* one ring step of causal varlen attention with a running ``(o, m, l)`` state --
  ``loongserve/models/llama/triton_kernel/ring_context_flashattention_nopad.py:13-188``
  (visible range ``:78-85``, mask ``:156-161``, base-2 online softmax ``:134-140``, merge ``:175-188``);
* the ring loop itself -- ``loongserve/models/llama/layer_infer/longserve_transformer_layer_infer.py:104-178``;
* split-KV flash-decoding, stage 1 and stage 2 --
  ``longserve_cuda_kernels/src/flash_decoding_stage1.cu:25-143`` and ``flash_decoding_stage2.cu:15-58``;
* the token-granular KV scatter / registration / migration kernels --
  ``loongserve/models/llama/triton_kernel/copy_and_register_kv.py:7-31,64-120``,
  ``loongserve/common/basemodel/triton_kernel/destindex_copy_kv.py:8-28``,
  ``loongserve/common/basemodel/triton_kernel/copy_kv_index_to_req.py:8-18``,
  ``loongserve/common/infer_utils.py:1-13``,
  ``loongserve/models/llama/triton_kernel/decoding_stage_migration.py:6-69,98-158``;
* the slot allocator order -- ``loongserve/common/longserve_mem_manager.py:32-89``;
* the layer glue (RMSNorm, rotate-half RoPE, SiLU*mul, FFN block, one whole Llama layer) --
  ``longserve_cuda_kernels/src/rms_norm.cu``, ``rotary_emb.cu``, ``silu_and_mul.cu``, ``entrypoints.cpp:89-101``,
  ``loongserve/models/llama/layer_infer/longserve_transformer_layer_infer.py:70-96,372-456``;
* the prefill scheduling search -- ``longserve_c_scheduler/src/main.cpp:34-86``.

Parity status.  Pinned: the ring step, the full causal attention, every KV scatter / registration /
migration function and the allocator are checked against golden vectors produced by running the
reference's own code in this project's build container (``tests/golden/make_golden.py``: the Triton
kernels under Triton's CPU interpreter, ``torch_att`` and the Python managers directly); the scheduling
search is checked, bit for bit, against tables from the reference's own C++ module compiled by
``oracle/Makefile``.
Flash-decoding stage 1/2 exist in the reference only as CUDA and have no reference test:
their restatement is checked on a GPU against the reference kernels compiled by ``oracle/Makefile``;
on the CPU their parity is unpinned and rests on the algebraic identity with full softmax attention.

Known, deliberate divergence from the reference ring kernel: for a q block whose visible key range is
not a multiple of the 128-key tile, the reference starts its masked tail loop at ``loop_range - 128``
(``ring_context_flashattention_nopad.py:114,143``) and so counts the keys in
``[loop_range - 128, 128 * floor(loop_range / 128))`` twice.  The oracle (like the reference's own
``torch_att`` check) counts every visible key exactly once.
"""
from __future__ import annotations

import math

import numpy as np
import torch

LOG2E = 1.4426950408889634
LN2 = 0.6931471805599453
INT32_MAX = 2147483647


# ----------------------------------------------------------------------------------------------
# Prefill: full attention and one ring step
# ----------------------------------------------------------------------------------------------

def ceil_div(a: int, b: int) -> int:
    """Mathematical ceiling of a / b for b > 0 and any sign of a."""
    return -((-a) // b)


def full_causal_attention(q, k, v, lens, sm_scale=None):
    """Single-device causal attention over packed sequences; returns (o fp32, lse fp32 natural log).

    Same math as the reference's ``torch_att`` (ring_context_flashattention_nopad.py:287-321) but with a
    true -inf mask and the log-sum-exp as a second output.  q [T,Hq,D]; k, v [T,Hkv,D]; lens [B].
    """
    q = q.float(); k = k.float(); v = v.float()
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    g = Hq // Hkv
    scale = sm_scale if sm_scale is not None else 1.0 / math.sqrt(D)
    o = torch.empty_like(q)
    lse = torch.empty((T, Hq), dtype=torch.float32)
    start = 0
    for L in [int(x) for x in lens]:
        qs = q[start:start + L].permute(1, 0, 2)                              # [Hq, L, D]
        ks = k[start:start + L].repeat_interleave(g, dim=1).permute(1, 0, 2)
        vs = v[start:start + L].repeat_interleave(g, dim=1).permute(1, 0, 2)
        blk = 1024
        for r0 in range(0, L, blk):
            r1 = min(L, r0 + blk)
            s = (qs[:, r0:r1] @ ks[:, :r1].transpose(1, 2)) * scale           # [Hq, r, r1]
            rows = torch.arange(r0, r1).view(1, -1, 1)
            cols = torch.arange(0, r1).view(1, 1, -1)
            s = s.masked_fill(cols > rows, float("-inf"))
            ls = torch.logsumexp(s, dim=-1)                                   # [Hq, r]
            p = torch.exp(s - ls.unsqueeze(-1))
            o[start + r0:start + r1] = (p @ vs[:, :r1]).permute(1, 0, 2)
            lse[start + r0:start + r1] = ls.permute(1, 0)
        start += L
    return o, lse


def ring_step(q, k, v, o, m, l,
              q_b_start_loc, q_b_seq_len, q_first_token_global_idx,
              kv_b_start_loc, kv_b_seq_len, kv_first_token_global_idx,
              logical_sp_peers_num: int, sm_scale=None, round_acc_to=None, kv_pos_stride=None):
    """One ring step: attention of the local q rows against one (local or remote) KV block, merged
    in place into the running state.  Semantics of ``context_attention_fwd``
    (ring_context_flashattention_nopad.py:191-284):

    * key n of request b is visible to q row r iff
      ``q_first[b] + r*s >= kv_first[b] + n*s`` and ``n < kv_len[b]``  (:156-161);
    * scores are scaled by ``D**-0.5 * log2(e)`` and the softmax runs in base 2 (:252-256, :134-140);
    * ``m`` is the running base-2 maximum, ``l`` the matching sum, ``o`` is kept NORMALISED
      after every step; merge rule :175-188.
    * rows with no visible key in this call keep their state.

    ``o`` may be any float dtype (it is read and written in that dtype, like the reference does with
    the q dtype); m and l are fp32.  ``round_acc_to`` optionally rounds the step's unnormalised
    accumulator to a dtype before the merge, as the reference does with fp16 (:183).

    ``kv_pos_stride`` (not in the reference, whose keys and q rows always advance by the same stride): position stride of
    consecutive keys when it differs from that of q rows; the visibility rule becomes
    ``q_first[b] + r*s >= kv_first[b] + n*kv_pos_stride``.  Used to check attention over a buffer that holds several
    instances' blocks interleaved in position order.
    """
    Tq, Hq, D = q.shape
    Hkv = k.shape[1]
    g = Hq // Hkv
    s_ = int(logical_sp_peers_num)
    scale2 = (sm_scale if sm_scale is not None else 1.0 / math.sqrt(D)) * LOG2E
    B = len(q_b_seq_len)
    for b in range(B):
        qs, ql, qf = int(q_b_start_loc[b]), int(q_b_seq_len[b]), int(q_first_token_global_idx[b])
        ks, kl, kf = int(kv_b_start_loc[b]), int(kv_b_seq_len[b]), int(kv_first_token_global_idx[b])
        if ql <= 0 or kl <= 0:
            continue
        qq = q[qs:qs + ql].float().permute(1, 0, 2)                               # [Hq, ql, D]
        kk = k[ks:ks + kl].float().repeat_interleave(g, dim=1).permute(1, 0, 2)   # [Hq, kl, D]
        vv = v[ks:ks + kl].float().repeat_interleave(g, dim=1).permute(1, 0, 2)
        rows = (qf + torch.arange(ql, dtype=torch.int64) * s_).view(1, -1, 1)
        cols = (kf + torch.arange(kl, dtype=torch.int64) * (s_ if kv_pos_stride is None else int(kv_pos_stride))).view(1, 1, -1)
        blk = 1024
        for r0 in range(0, ql, blk):
            r1 = min(ql, r0 + blk)
            sc = (qq[:, r0:r1] @ kk.transpose(1, 2)) * scale2                     # [Hq, r, kl]
            sc = sc.masked_fill(~(rows[:, r0:r1] >= cols), float("-inf"))
            m_i = sc.amax(dim=-1)                                                 # [Hq, r]
            has = torch.isfinite(m_i)
            m_safe = torch.where(has, m_i, torch.zeros_like(m_i))
            p = torch.exp2(sc - m_safe.unsqueeze(-1))
            l_i = p.sum(dim=-1)
            acc = p @ vv                                                          # unnormalised
            if round_acc_to is not None:
                acc = acc.to(round_acc_to).float()
            m_old = m[qs + r0:qs + r1].permute(1, 0)
            l_old = l[qs + r0:qs + r1].permute(1, 0)
            o_old = o[qs + r0:qs + r1].float().permute(1, 0, 2)
            m_new = torch.maximum(m_i, m_old)
            m_new_safe = torch.where(torch.isfinite(m_new), m_new, torch.zeros_like(m_new))
            a_old = torch.exp2(m_old - m_new_safe)       # exp2(-inf) = 0 for untouched state
            a_new = torch.exp2(m_i - m_new_safe)
            l_new = l_old * a_old + l_i * a_new
            denom = torch.where(l_new > 0, l_new, torch.ones_like(l_new))
            o_new = (o_old * (l_old * a_old).unsqueeze(-1) + acc * a_new.unsqueeze(-1)) / denom.unsqueeze(-1)
            upd = has                                                            # rows that saw a key
            o_w = torch.where(upd.unsqueeze(-1), o_new, o_old).permute(1, 0, 2)
            o[qs + r0:qs + r1] = o_w.to(o.dtype)
            m[qs + r0:qs + r1] = torch.where(upd, m_new, m_old).permute(1, 0)
            l[qs + r0:qs + r1] = torch.where(upd, l_new, l_old).permute(1, 0)


def lse_from_state(m, l):
    """Natural-log lse of the rows seen so far from the base-2 running state: ln2*m + ln(l)."""
    return m * LN2 + torch.log(l)


def shard_request_lengths(lens, P: int, striped: bool):
    """Local token counts and first global index of every request on every logical rank.

    striped (reference placement, loongserve/longserve_server/io_struct.py:78-81): token t lives on
    rank t mod P; contiguous: rank r holds tokens [r*ceil(L/P), ...).  Returns (local_len[P][B],
    first_idx[P][B], stride)."""
    local_len, first = [], []
    for r in range(P):
        ll, ff = [], []
        for L in lens:
            L = int(L)
            if striped:
                ll.append(max(0, (L - r + P - 1) // P)); ff.append(r)
            else:
                per = (L + P - 1) // P
                b, e = min(L, r * per), min(L, (r + 1) * per)
                ll.append(e - b); ff.append(b)
        local_len.append(ll); first.append(ff)
    return local_len, first, (P if striped else 1)


def shard_tokens(x, lens, P: int, striped: bool):
    """Split a packed [T, H, D] tensor into the P per-rank packed tensors of that placement."""
    outs = [[] for _ in range(P)]
    start = 0
    for L in [int(v) for v in lens]:
        seq = x[start:start + L]
        for r in range(P):
            if striped:
                outs[r].append(seq[r::P])
            else:
                per = (L + P - 1) // P
                outs[r].append(seq[min(L, r * per):min(L, (r + 1) * per)])
        start += L
    return [torch.cat(o, dim=0) for o in outs]


def ring_prefill(q, k, v, lens, P: int, striped: bool, o_dtype=torch.float32, sm_scale=None):
    """The whole ring on one CPU: P logical ranks, P steps, block order rank, rank-1, ...
    (longserve_transformer_layer_infer.py:127-178).  Returns per-rank lists (o, m, l) plus the
    per-rank metadata used, so a test can feed the same shards to the CUDA path."""
    local_len, first, stride = shard_request_lengths(lens, P, striped)
    qs = shard_tokens(q, lens, P, striped)
    ks = shard_tokens(k, lens, P, striped)
    vs = shard_tokens(v, lens, P, striped)
    outs = []
    for r in range(P):
        Tq, Hq, D = qs[r].shape
        o = torch.zeros((Tq, Hq, D), dtype=o_dtype)
        m = torch.full((Tq, Hq), float("-inf"), dtype=torch.float32)
        l = torch.zeros((Tq, Hq), dtype=torch.float32)
        q_len = torch.tensor(local_len[r], dtype=torch.int32)
        q_start = torch.cumsum(q_len, 0, dtype=torch.int32) - q_len
        q_first = torch.tensor(first[r], dtype=torch.int32)
        for i in range(P):
            src = (r - i) % P
            kv_len = torch.tensor(local_len[src], dtype=torch.int32)
            kv_start = torch.cumsum(kv_len, 0, dtype=torch.int32) - kv_len
            kv_first = torch.tensor(first[src], dtype=torch.int32)
            ring_step(qs[r], ks[src], vs[src], o, m, l, q_start, q_len, q_first,
                      kv_start, kv_len, kv_first, stride, sm_scale)
        outs.append((o, m, l))
    meta = dict(local_len=local_len, first=first, stride=stride, q=qs, k=ks, v=vs)
    return outs, meta


def unshard_tokens(parts, lens, P: int, striped: bool):
    """Inverse of shard_tokens for per-row outputs ([T_local, ...] per rank -> packed [T, ...])."""
    T = int(sum(int(x) for x in lens))
    out = torch.empty((T,) + tuple(parts[0].shape[1:]), dtype=parts[0].dtype)
    offs = [0] * P
    start = 0
    for L in [int(v) for v in lens]:
        for r in range(P):
            if striped:
                n = max(0, (L - r + P - 1) // P)
                out[start + r:start + L:P] = parts[r][offs[r]:offs[r] + n]
            else:
                per = (L + P - 1) // P
                b, e = min(L, r * per), min(L, (r + 1) * per)
                n = e - b
                out[start + b:start + e] = parts[r][offs[r]:offs[r] + n]
            offs[r] += n
        start += L
    return out


# ----------------------------------------------------------------------------------------------
# Decode: split-KV stage 1, lse-merge stage 2
# ----------------------------------------------------------------------------------------------

def flash_decoding_stage1(mid_o, mid_lse, q, k, v, req_to_tokens, b_req_idx, b_seqlen,
                          max_len_in_batch: int, seq_block_size: int, sm_scale=None):
    """Partial attention per (request, head, block of ``seq_block_size`` tokens) over a token-indexed
    pool (flash_decoding_stage1.cu:50-57 block bounds, :70-76 slot gather, :85-116 scores + softmax,
    :126-142 weighted V sum).  mid_o [nblk,B,Hq,D] fp32 holds the block's NORMALISED output,
    mid_lse [nblk,B,Hq] its natural-log sum-exp.  Blocks past a request's length are left untouched."""
    B, Hq, D = q.shape
    Hkv = k.shape[1]
    g = Hq // Hkv
    scale = sm_scale if sm_scale is not None else 1.0 / math.sqrt(D)
    nblk = (int(max_len_in_batch) + seq_block_size - 1) // seq_block_size
    for b in range(B):
        L = int(b_seqlen[b]); rid = int(b_req_idx[b])
        for j in range(nblk):
            t0, t1 = j * seq_block_size, min((j + 1) * seq_block_size, L)
            if t1 <= t0:
                continue
            slots = req_to_tokens[rid, t0:t1].long()
            kk = k[slots].float().repeat_interleave(g, dim=1)          # [n, Hq, D]
            vv = v[slots].float().repeat_interleave(g, dim=1)
            s = torch.einsum("hd,nhd->hn", q[b].float(), kk) * scale   # [Hq, n]
            lse = torch.logsumexp(s, dim=-1)
            p = torch.exp(s - lse.unsqueeze(-1))
            mid_o[j, b] = torch.einsum("hn,nhd->hd", p, vv)
            mid_lse[j, b] = lse


def flash_decoding_stage2(o, out_lse, b_seqlen, mid_o, mid_lse, block_seq: int, zero_fill_empty=True):
    """Merge ceil(b_seqlen/block_seq) partials per (request, head) (flash_decoding_stage2.cu:30-57).
    The reference writes nothing for a request with zero partials; this build defines that case as
    o = 0, lse = -inf (``zero_fill_empty``)."""
    B = len(b_seqlen)
    for b in range(B):
        L = int(b_seqlen[b])
        n = 0 if L <= 0 else (L + block_seq - 1) // block_seq
        if n == 0:
            if zero_fill_empty:
                o[b] = 0
                out_lse[b] = float("-inf")
            continue
        lse_parts = mid_lse[:n, b].float()                              # [n, H]
        finite = torch.isfinite(lse_parts).any(dim=0)
        tot = torch.logsumexp(lse_parts, dim=0)                         # [H]
        w = torch.exp(lse_parts - torch.where(finite, tot, torch.zeros_like(tot)).unsqueeze(0))
        w = torch.where(torch.isfinite(lse_parts), w, torch.zeros_like(w))
        res = (w.unsqueeze(-1) * torch.nan_to_num(mid_o[:n, b].float())).sum(dim=0)
        o[b] = res.to(o.dtype)
        out_lse[b] = tot


def token_decode_attention(q, k, v, req_to_tokens, b_req_idx, b_seqlen, sm_scale=None):
    """Direct (unsplit) single-query attention over each request's pool slots: (o fp32, lse)."""
    B, Hq, D = q.shape
    Hkv = k.shape[1]
    g = Hq // Hkv
    scale = sm_scale if sm_scale is not None else 1.0 / math.sqrt(D)
    o = torch.zeros((B, Hq, D), dtype=torch.float32)
    lse = torch.full((B, Hq), float("-inf"), dtype=torch.float32)
    for b in range(B):
        L = int(b_seqlen[b])
        if L <= 0:
            continue
        slots = req_to_tokens[int(b_req_idx[b]), :L].long()
        kk = k[slots].float().repeat_interleave(g, dim=1)
        vv = v[slots].float().repeat_interleave(g, dim=1)
        s = torch.einsum("hd,nhd->hn", q[b].float(), kk) * scale
        lse[b] = torch.logsumexp(s, dim=-1)
        o[b] = torch.einsum("hn,nhd->hd", torch.exp(s - lse[b].unsqueeze(-1)), vv)
    return o, lse


# ----------------------------------------------------------------------------------------------
# KV pool: scatter, registration, migration  (bit-exact integer / byte work)
# ----------------------------------------------------------------------------------------------

def destindex_copy_kv(K, DestLoc, Out):
    """Out[DestLoc[i]] = K[i]  (destindex_copy_kv.py:8-28)."""
    Out[DestLoc.long()] = K[: DestLoc.shape[0]]


def pre_copy_and_register_kv(kv_cache_index_begin, kv_cache_index_end, kv_first_token_global_idx, P: int):
    """Local row range of a passing striped block that falls into [begin, end) of global positions
    (copy_and_register_kv.py:25-31): ceil((x - kv_first)/P).  The Triton source computes
    (x - kv_first + P - 1) // P with truncating division; both agree whenever x - kv_first >= -(P-1),
    which always holds because kv_first is in [0, P) and x >= 0."""
    cb = kv_cache_index_begin.to(torch.int64); ce = kv_cache_index_end.to(torch.int64)
    kf = kv_first_token_global_idx.to(torch.int64)
    rb = -((-(cb - kf)) // P)
    re = -((-(ce - kf)) // P)
    dt = kv_cache_index_begin.dtype
    return rb.to(dt), re.to(dt), (re - rb).to(dt)


def destindex_copy_and_register_kv(batch_size, new_kv_cache_len, kv_range_begin, kv_range_end,
                                   new_kv_cache_len_sum, kv, kv_b_start_loc, cur_kv_cache_index,
                                   mem_index, total_kv_cache, req_to_token_indexs, b_req_idx,
                                   num_used_mem_index: int, max_len_in_batch: int,
                                   should_register_kv: bool):
    """Copy the kept rows of a passing KV block into pool slots and (layer 0) record the slot ids
    (copy_and_register_kv.py:85-120).  Row n of request b goes to
    mem_index[num_used + cumsum_prev[b] + n]; at most ``max_len_in_batch`` rows (rounded up to the
    256-row program size) are handled per request, as in the reference grid (:146-148)."""
    BLOCK_N = 256
    cap = ((int(max_len_in_batch) + BLOCK_N - 1) // BLOCK_N) * BLOCK_N
    for b in range(int(batch_size)):
        n_new = int(new_kv_cache_len[b]); rb = int(kv_range_begin[b]); re = int(kv_range_end[b])
        if n_new <= 0 or rb < 0 or re < 0:
            continue
        base = (int(new_kv_cache_len_sum[b - 1]) if b > 0 else 0) + int(num_used_mem_index)
        src0 = int(kv_b_start_loc[b]) + rb
        n_do = min(n_new, cap)
        slots = mem_index[base:base + n_do].long()
        total_kv_cache[slots] = kv[src0:src0 + n_do]
        if should_register_kv:
            c0 = int(cur_kv_cache_index[b])
            req_to_token_indexs[int(b_req_idx[b]), c0:c0 + n_do] = slots.to(req_to_token_indexs.dtype)


def copy_kv_index_to_req(req_to_token_indexs, b_req_idx, b_seq_len, memindex):
    """req_to_token[req, seq_len-1] = slot  (copy_kv_index_to_req.py:8-18)."""
    for i in range(len(b_seq_len)):
        req_to_token_indexs[int(b_req_idx[i]), int(b_seq_len[i]) - 1] = int(memindex[i])


def init_req_to_token_indexes(req_to_token_indexs, b_req_idx, b_seq_len, alloc_mem_index):
    """Prefill registration: consecutive runs of the allocated slots, request by request
    (loongserve/common/infer_utils.py:1-13)."""
    start = 0
    for i in range(len(b_seq_len)):
        n = int(b_seq_len[i])
        req_to_token_indexs[int(b_req_idx[i]), 0:n] = alloc_mem_index[start:start + n].to(req_to_token_indexs.dtype)
        start += n


def decoding_stage_migration_sender(send_buf, req_to_token_indexes, mem_state, kv_cache,
                                    request_ids, num_tokens, b_seq_len):
    """Gather the last num_tokens[b] tokens of each request, all layers, into send_buf
    [L, sum(num_tokens), 2H, D] and zero their refcounts (decoding_stage_migration.py:41-69)."""
    off = 0
    for b in range(len(request_ids)):
        n = int(num_tokens[b]); L = int(b_seq_len[b]); rid = int(request_ids[b])
        slots = req_to_token_indexes[rid, L - n:L].long()
        mem_state[slots] = 0
        send_buf[:, off:off + n] = kv_cache[:, slots]
        off += n


def decoding_stage_migration_receiver(recv_buf, req_to_token_indexes, kv_cache, alloc_mem,
                                      request_ids, num_tokens, b_seq_len):
    """Scatter recv_buf into freshly allocated slots and append the slot ids at
    req_to_token[req, seq_len + i]  (decoding_stage_migration.py:132-158)."""
    off = 0
    for b in range(len(request_ids)):
        n = int(num_tokens[b]); L = int(b_seq_len[b]); rid = int(request_ids[b])
        slots = alloc_mem[off:off + n].long()
        req_to_token_indexes[rid, L:L + n] = slots.to(req_to_token_indexes.dtype)
        kv_cache[:, slots] = recv_buf[:, off:off + n]
        off += n


class OracleMemoryManager:
    """CPU restatement of the slot allocator's observable behaviour
    (loongserve/common/longserve_mem_manager.py:32-89): lowest free ids first, first free run for
    contiguous requests, int32 reference counts."""

    def __init__(self, size: int):
        self.size = size
        self.mem_state = np.zeros((size,), dtype=np.int32)
        self.can_use_mem_size = size

    def alloc(self, need: int):
        assert need <= self.can_use_mem_size
        idx = np.nonzero(self.mem_state == 0)[0][:need].astype(np.int64)
        self.add_refs(idx)
        return idx

    def alloc_contiguous(self, need: int):
        if need > self.can_use_mem_size:
            return None
        free = np.nonzero(self.mem_state == 0)[0]
        if len(free) < need:
            return None
        cand = free[: len(free) - need + 1][(free[need - 1:] - free[: len(free) - need + 1]) == need - 1]
        if len(cand) == 0:
            return None
        start = int(cand[0])
        idx = np.arange(start, start + need, dtype=np.int64)
        self.add_refs(idx)
        return idx, start, start + need

    def add_refs(self, idx):
        state = self.mem_state[idx]
        self.can_use_mem_size -= len(state) - int(np.count_nonzero(state))
        self.mem_state[idx] += 1

    def decrease_refs(self, idx):
        self.mem_state[idx] -= 1
        state = self.mem_state[idx]
        self.can_use_mem_size += len(state) - int(np.count_nonzero(state))

    def free(self, idx):
        self.decrease_refs(np.asarray(idx, dtype=np.int64))

    def free_all(self):
        self.mem_state[:] = 0
        self.can_use_mem_size = self.size


# ----------------------------------------------------------------------------------------------
# Layer glue around the attention path (element-wise ops, RoPE tables, one Llama layer)
# ----------------------------------------------------------------------------------------------

def rms_norm(x, weight, eps):
    """x * rsqrt(mean(x^2) + eps) * weight, fp32 (longserve_cuda_kernels/test/rms_norm.py:5-7,
    kernel longserve_cuda_kernels/src/rms_norm.cu:10-46)."""
    x = x.float()
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight.float()


def rotary_emb(x, cos, sin):
    """Rotate-half RoPE: first half / second half of head_dim (longserve_cuda_kernels/test/rotary_emb.py:5-14,
    kernel rotary_emb.cu:26-33)."""
    x = x.float()
    T, h, dim = x.shape
    x0, x1 = x[:, :, : dim // 2], x[:, :, dim // 2:]
    c = cos.float().view(T, 1, dim // 2); s = sin.float().view(T, 1, dim // 2)
    return torch.cat((x0 * c - x1 * s, x0 * s + x1 * c), dim=-1)


def silu_and_mul(io):
    """silu(io[:, :F]) * io[:, F:]  (longserve_cuda_kernels/test/silu_and_mul.py, kernel silu_and_mul.cu:17-34)."""
    io = io.float()
    F = io.shape[1] // 2
    return torch.nn.functional.silu(io[:, :F]) * io[:, F:]


def ffn_block(x, norm_weight, eps, gate_up_proj, down_proj, act_dtype=None):
    """norm -> mm(gate_up) -> silu*mul -> mm(down) (longserve_cuda_kernels/src/entrypoints.cpp:89-101).
    ``act_dtype`` rounds the intermediate activations like the 16-bit pipeline does."""
    r = (lambda t: t.to(act_dtype).float()) if act_dtype is not None else (lambda t: t)
    h = r(rms_norm(x, norm_weight, eps))
    gu = r(h @ gate_up_proj.float())
    a = r(silu_and_mul(gu))
    return r(a @ down_proj.float())


def rope_tables(positions, head_dim, base=10000.0):
    """cos/sin [len(positions), head_dim/2] of the rotate-half convention, fp32:
    angle = position * base^(-2i/head_dim) (loongserve/models/llama/longserve_model.py:264-275)."""
    inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    ang = torch.outer(positions.float(), inv_freq)
    return torch.cos(ang), torch.sin(ang)


def llama_layer(x, positions, lens, w, eps, Hq, Hkv, D, act_dtype=None):
    """One full-sequence Llama layer on packed sequences (prefill), fp32 math with optional 16-bit rounding of
    the activations: att_norm -> q / kv projections -> RoPE on q and k -> causal attention -> o projection ->
    residual -> ffn_block -> residual (longserve_transformer_layer_infer.py:70-96, 372-407).
    ``w`` holds att_norm, q, kv, o, ffn_norm, gate_up, down.  Returns (x_out, k, v)."""
    r = (lambda t: t.to(act_dtype).float()) if act_dtype is not None else (lambda t: t)
    x = x.float()
    h = r(rms_norm(x, w["att_norm"], eps))
    q = r(h @ w["q"].float()).view(-1, Hq, D)
    kv = r(h @ w["kv"].float()).view(-1, 2 * Hkv, D)
    cos, sin = rope_tables(positions, D)
    cos, sin = r(cos), r(sin)
    q = r(rotary_emb(q, cos, sin))
    k = r(rotary_emb(kv[:, :Hkv], cos, sin))
    v = kv[:, Hkv:]
    o, _ = full_causal_attention(q, k, v, lens)
    x = r(x + r(r(o).reshape(-1, Hq * D) @ w["o"].float()))
    x = r(x + ffn_block(x, w["ffn_norm"], eps, w["gate_up"], w["down"], act_dtype))
    return x, k, v


# ----------------------------------------------------------------------------------------------------------------------
# Prefill scheduling search (host logic): restatement of longserve_c_scheduler/src/main.cpp:34-86.

def minimize_prefill_iteration_time(num_new_req, num_instances, best, choice, tok_ps, sq_ps, inv_ps, room_ps, abc):
    """best [R+1, I+1] float64 (+inf), choice [R+1, I+1, 2] int32 (-1), both filled in place.  Pure-Python loops: small cases
    only.  Visit order, pruning bounds and the strict comparison follow main.cpp:36-84."""
    import numpy as _np

    def rng(ps, lo, hi):
        return ps[hi - 1] - (ps[lo - 1] if lo > 0 else 0)

    best[0, 0] = 0.0
    for n in range(1, num_new_req + 1):
        for m in range(1, num_instances + 1):
            b_hi = int(choice[n, m - 1, 0]) if choice[n, m - 1, 0] != -1 else n          # main.cpp:39-41
            u_lo = int(choice[n - 1, m, 1]) if choice[n - 1, m, 1] != -1 else 1          # main.cpp:45-47
            for b in range(1, b_hi + 1):
                for u in range(m, u_lo - 1, -1):
                    need = int(rng(tok_ps, n - b, n))
                    if need > int(rng(room_ps, m - u, m)):                               # main.cpp:61-63
                        break
                    need_sq = int(rng(sq_ps, n - b, n))
                    t = _np.float64(abc[u, 0]) + _np.float64(abc[u, 1]) * _np.float64(need) + _np.float64(abc[u, 2]) * _np.float64(need_sq)
                    total = t * _np.float64(rng(inv_ps, n - b, n)) + best[n - b, m - u]   # main.cpp:71-76
                    if total < best[n, m]:
                        best[n, m] = total
                        choice[n, m, 0] = b
                        choice[n, m, 1] = u
