"""Ring prefill loop and multi-master decode exchange: the orchestration around the kernels, following
loongserve/models/llama/layer_infer/longserve_transformer_layer_infer.py:104-222 (ring) and :224-370
(multi-master decode).  The communicator is duck-typed (``nccl_group_start/end``, ``nccl_send/recv``,
``wait_for_default_stream``, ``let_default_stream_wait``) so the same loop runs over
``loongserve_b200.rnccl.RNCCLComm`` on GPUs and over a gloo-backed stand-in in the CPU tests; the
attention / scatter callables are injected the same way.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import torch


def shard_lengths(lens: Sequence[int], P: int, striped: bool):
    """Per logical rank: local token count and first global index of every request.
    striped = reference placement (token t on rank t mod P, io_struct.py:78-81)."""
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


@dataclass
class BlockMeta:
    """start_loc / seq_len / first_token_global_idx of one rank's packed KV block (int32 [batch])."""
    start_loc: torch.Tensor
    seq_len: torch.Tensor
    first_idx: torch.Tensor

    @staticmethod
    def from_lengths(lens, first, device):
        sl = torch.tensor(lens, dtype=torch.int32)
        st = torch.cumsum(sl, 0, dtype=torch.int32) - sl
        return BlockMeta(st.to(device), sl.to(device), torch.tensor(first, dtype=torch.int32).to(device))


@dataclass
class KeepPlan:
    """Scale-down bookkeeping of one prefill (longserve_transformer_layer_infer.py:180-220): which
    global token range of every request this instance keeps, the slots to put them in, and the
    per-ring-step ranges computed at layer 0 and reused by the other layers."""
    kv_cache_index_begin: torch.Tensor
    kv_cache_index_end: torch.Tensor
    mem_index: torch.Tensor
    b_req_idx: torch.Tensor
    req_to_token_indexs: torch.Tensor
    cur_kv_cache_index: torch.Tensor
    cached: list = field(default_factory=list)


def ring_context_attention(q, local_kv, o, m, l, *, rank: int, peers: Sequence[int], metas: Sequence[BlockMeta],
                           stride: int, max_len_in_batch: int, num_kv_heads: int, comm, recv_buffers,
                           attention_fn: Callable, init_fn: Callable, overlap: bool = True,
                           keep: Optional[KeepPlan] = None, pool_layer=None, layer_idx: int = 0,
                           keep_fns=None, exchange=None):
    """One layer's ring pass on logical rank ``rank`` of the ring ``peers`` (SP ranks in ring order).

    q [Tq, Hq, D]; local_kv [max_token_num, 2*Hkv, D] (K heads then V heads); ``recv_buffers`` two
    buffers of local_kv's shape; ``metas[r]`` describes logical rank r's block (a pure function of the
    request lengths, so it is computed on the host instead of travelling with the block as in the
    reference, :162-178).  At step i the rank attends to the block of logical rank (rank - i) mod P,
    sends it on to rank+1 and receives the next one from rank-1 (:163,171).  With ``overlap`` the
    exchange of block i runs on the communicator's stream while block i is being attended to; without
    it the exchange is queued behind the kernel as in the reference's default mode (:464-465).

    ``exchange`` (a ``peer_ring.CopyEngineRing``) replaces the NCCL pair by a copy-engine transfer into the next
    instance's memory, synchronised by flags; the blocks then arrive in the exchange's own two buffers
    (``recv_buffers`` and ``comm`` are not used), in the same order and with the same buffer swap.
    """
    P = len(peers)
    init_fn(o, m, l)
    Hkv = num_kv_heads
    cur = local_kv
    nxt_rank = peers[(rank + 1) % P]
    prv_rank = peers[(rank - 1 + P) % P]
    num_used = 0
    if keep is not None:
        keep.cur_kv_cache_index.zero_()
    if exchange is not None and P > 1:
        recv_buffers = exchange.receive_buffers(local_kv)
        exchange.begin_pass(nxt_rank, prv_rank, P - 1)
        kv_bytes = local_kv.numel() * local_kv.element_size()
    else:
        exchange = None
    for i in range(P):
        src = (rank - i) % P
        meta = metas[src]
        recv = None
        if i != P - 1:
            recv = recv_buffers[i % 2]
            if exchange is not None:
                exchange.forward(i, cur.data_ptr(), kv_bytes)      # overlaps the attention over the same block
            elif overlap:
                comm.wait_for_default_stream()      # block i is ready, the receive buffer is no longer read
                comm.nccl_group_start()
                comm.nccl_recv(recv, prv_rank)
                comm.nccl_send(cur, nxt_rank)
                comm.nccl_group_end()
        attention_fn(q, cur[:, :Hkv, :], cur[:, Hkv:, :], o, metas[rank].start_loc, metas[rank].seq_len,
                     metas[rank].first_idx, meta.start_loc, meta.seq_len, meta.first_idx, stride,
                     max_len_in_batch, m, l)
        if i != P - 1 and not overlap and exchange is None:
            comm.wait_for_default_stream()
            comm.nccl_group_start()
            comm.nccl_recv(recv, prv_rank)
            comm.nccl_send(cur, nxt_rank)
            comm.nccl_group_end()
        if keep is not None:
            pre_fn, copy_fn = keep_fns
            if layer_idx == 0:
                rb, re, nl = pre_fn(keep.kv_cache_index_begin, keep.kv_cache_index_end, meta.first_idx, P)
                nls = torch.cumsum(nl, dim=0, dtype=torch.int64)
                keep.cached.append((rb, re, nl, nls, int(nls[-1].item())))
            rb, re, nl, nls, total = keep.cached[i]
            copy_fn(len(meta.seq_len), nl, rb, re, nls, cur, meta.start_loc, keep.cur_kv_cache_index,
                    keep.mem_index, pool_layer, keep.req_to_token_indexs, keep.b_req_idx, num_used,
                    max_len_in_batch + 1, layer_idx == 0)
            num_used += total
            if layer_idx == 0:
                keep.cur_kv_cache_index += nl
        if exchange is not None:
            if i > 0:
                exchange.release(i - 1)             # the buffer that held this step's block may be refilled
            if i != P - 1:
                exchange.wait_arrival(i)            # the next block has arrived before it is read
                cur = recv
        elif i != P - 1:
            comm.let_default_stream_wait()          # the next block has arrived before it is read
            cur = recv
    if exchange is not None:
        exchange.end_pass()
    return o


@dataclass
class GatherPlan:
    """Layout of one instance's gather buffer for a striped pass over ``P`` instances (``peer_ring.CopyEngineGather``):
    request b owns ``seq_len[b]`` rows from ``start_loc[b]``, holding the other instances' tokens of that request in
    position order (token n of the i-th other instance in row n*(P-1)+i).  Seen from there the local q row r of instance
    ``rank`` sits at position r*(P-1) + rank - 1 (``q_first``), keys at 0, 1, 2, ...

    With ``parts`` > 1 the rows of every request are cut into that many position ranges at multiples of P-1 rows (whole
    groups of positions), each delivered and announced on its own, so that the attention over an early range can run while
    the later ranges are still on their way: ``part_metas[k]`` describes range k as a block of its own (its keys start at
    position ``first_idx`` = the range's first row), ``part_groups[b]`` holds the group boundaries of request b."""
    meta: BlockMeta                   # start_loc / seq_len of the gathered rows, first_idx = 0
    q_first: torch.Tensor             # int32 [batch], rank - 1
    rows: int
    start_rows: List[int]             # start_loc on the host
    part_metas: List[BlockMeta] = field(default_factory=list)
    part_groups: List[List[int]] = field(default_factory=list)
    part_rows: List[int] = field(default_factory=list)

    @staticmethod
    def build(lens: Sequence[int], P: int, rank: int, device, parts: int = 1):
        local_len, _, _ = shard_lengths(lens, P, True)
        others = [int(L) - local_len[rank][b] for b, L in enumerate(lens)]
        meta = BlockMeta.from_lengths(others, [0] * len(lens), device)
        starts, acc = [], 0
        for n in others:
            starts.append(acc); acc += n
        plan = GatherPlan(meta, torch.full((len(lens),), rank - 1, dtype=torch.int32).to(device), acc, starts)
        w = max(P - 1, 1)
        for n in others:
            groups = (n + w - 1) // w
            plan.part_groups.append([groups * k // parts for k in range(parts + 1)])
        for k in range(parts):
            lo = [min(w * plan.part_groups[b][k], n) for b, n in enumerate(others)]
            hi = [min(w * plan.part_groups[b][k + 1], n) for b, n in enumerate(others)]
            i32 = lambda x: torch.tensor(x, dtype=torch.int32).to(device)
            plan.part_metas.append(BlockMeta(i32([starts[b] + lo[b] for b in range(len(lens))]),
                                             i32([hi[b] - lo[b] for b in range(len(lens))]), i32(lo)))
            plan.part_rows.append(sum(hi[b] - lo[b] for b in range(len(lens))))
        return plan


def gathered_context_attention(q, local_kv, o, m, l, *, rank: int, lens: Sequence[int], P: int, metas: Sequence[BlockMeta],
                               plans: Sequence[GatherPlan], max_len_in_batch: int, num_kv_heads: int,
                               attention_fn: Callable, init_fn: Callable, gather):
    """One layer's prefill pass on instance ``rank`` of a STRIPED ring of ``P`` in two launches instead of P: every
    instance sends its block to all others with copy-engine transfers while it attends to its own block, then attends to
    everything it was sent in one call (one call per position range when the plans were built with ``parts`` > 1).  Same
    result as ``ring_context_attention`` up to the order in which the partial softmaxes are merged
    (longserve_transformer_layer_infer.py:128-181 does it block by block).  ``plans[r]`` is instance r's ``GatherPlan`` (a
    pure function of the request lengths, so every instance can compute where its rows go in every other instance's
    buffer).  Costs (P-1)/P of the whole KV of the batch in memory per instance; for batches where that is too much, or
    scale-down bookkeeping is wanted (``keep``), use the ring."""
    Hkv = num_kv_heads
    init_fn(o, m, l)
    me = metas[rank]
    if P == 1:
        attention_fn(q, local_kv[:, :Hkv, :], local_kv[:, Hkv:, :], o, me.start_loc, me.seq_len, me.first_idx,
                     me.start_loc, me.seq_len, me.first_idx, 1, max_len_in_batch, m, l)
        return o
    row_bytes = local_kv[0].numel() * local_kv.element_size()
    local_len, _, _ = shard_lengths(lens, P, True)
    my_starts, acc = [], 0
    for n in local_len[rank]:
        my_starts.append(acc); acc += n
    parts = len(plans[rank].part_metas)
    assert parts == gather.parts, "the plans and the exchange were made for different numbers of position ranges"
    gather.begin_pass()
    for step in range(1, P):
        peer = (rank + step) % P
        i = rank if rank < peer else rank - 1           # this instance's place among the peer's other instances
        per_part = []
        for k in range(parts):
            copies = []
            for b, n in enumerate(local_len[rank]):
                n0, n1 = min(plans[peer].part_groups[b][k], n), min(plans[peer].part_groups[b][k + 1], n)
                if n1 > n0:
                    copies.append(((plans[peer].start_rows[b] + n0 * (P - 1) + i) * row_bytes, (P - 1) * row_bytes,
                                   local_kv.data_ptr() + (my_starts[b] + n0) * row_bytes, row_bytes, row_bytes, n1 - n0))
            per_part.append(copies)
        gather.push(peer, per_part)
    attention_fn(q, local_kv[:, :Hkv, :], local_kv[:, Hkv:, :], o, me.start_loc, me.seq_len, me.first_idx,
                 me.start_loc, me.seq_len, me.first_idx, P, max_len_in_batch, m, l)
    plan = plans[rank]
    g = gather.gathered(plan.rows, local_kv) if plan.rows > 0 else None
    for k in range(parts):
        gather.wait_part(k)
        if plan.part_rows[k] > 0:
            pm = plan.part_metas[k]
            attention_fn(q, g[:, :Hkv, :], g[:, Hkv:, :], o, me.start_loc, me.seq_len, plan.q_first,
                         pm.start_loc, pm.seq_len, pm.first_idx, P - 1, max_len_in_batch, m, l, kv_pos_stride=1)
    gather.end_pass()
    return o


@dataclass
class MasterPlan:
    """What a master instance needs for one multi-master decode step
    (longserve_model.py:505-533, longserve_transformer_layer_infer.py:268-281,312-367)."""
    peers: Sequence[int]              # SP ranks of all logical peers of this master's batch (incl. itself)
    b_req_idx: torch.Tensor
    b_seq_len: torch.Tensor           # local lengths on the master (new token included)
    max_len_in_batch: int
    block_seq: int
    global_mid_o: torch.Tensor        # [(P-1) + nblk, B, Hq, D] fp32
    global_mid_lse: torch.Tensor      # [(P-1) + nblk, B, Hq] fp32
    global_merge_len: torch.Tensor    # int32 [B] = (P-1) + ceil(len / block_seq)
    global_out_lse: torch.Tensor      # fp32 [B, Hq]


@dataclass
class PeerPlan:
    """What an instance needs to serve other masters' queries in the same step (pre_process.py:194-230)."""
    masters: Sequence[int]            # SP ranks of the other masters, logical order
    ranges: Sequence[tuple]           # slice of peer_query_buffer belonging to each of them
    peer_query_buffer: torch.Tensor   # [peer_bs, Hq, D]
    peer_b_req_idx: torch.Tensor
    peer_b_seq_len: torch.Tensor      # local token counts of the foreign requests
    peer_max_len_in_batch: int
    block_seq: int
    peer_mid_o: torch.Tensor
    peer_mid_lse: torch.Tensor
    peer_o: torch.Tensor              # fp32 [peer_bs, Hq, D]
    peer_lse: torch.Tensor            # fp32 [peer_bs, Hq]


def multi_master_decode_attention(q, pool_layer, req_to_token_indexs, num_kv_heads: int, comm, my_rank: int,
                                  master: Optional[MasterPlan], peer: Optional[PeerPlan], stage1_fn: Callable,
                                  stage2_fn: Callable, out=None):
    """One layer of multi-master distributed decode attention on one instance
    (longserve_transformer_layer_infer.py:224-370): queries travel to the instances holding the KV,
    partial (o fp32, lse) come back, the master merges them with its own split-KV partials."""
    Hkv = num_kv_heads
    k_cache, v_cache = pool_layer[:, :Hkv, :], pool_layer[:, Hkv:, :]
    if master is not None:
        comm.wait_for_default_stream()
    comm.nccl_group_start()
    if peer is not None:
        for mrank, (b0, b1) in zip(peer.masters, peer.ranges):
            comm.nccl_recv(peer.peer_query_buffer[b0:b1], mrank)
    if master is not None:
        for prank in master.peers:
            if prank != my_rank:
                comm.nccl_send(q, prank)
    comm.nccl_group_end()

    n_other = 0
    if master is not None:
        n_other = len(master.peers) - 1
        stage1_fn(master.global_mid_o[n_other:], master.global_mid_lse[n_other:], q, k_cache, v_cache,
                  req_to_token_indexs, master.b_req_idx, master.b_seq_len, master.max_len_in_batch, master.block_seq)
    if peer is not None:
        comm.let_default_stream_wait()
        stage1_fn(peer.peer_mid_o, peer.peer_mid_lse, peer.peer_query_buffer, k_cache, v_cache,
                  req_to_token_indexs, peer.peer_b_req_idx, peer.peer_b_seq_len, peer.peer_max_len_in_batch,
                  peer.block_seq)
        stage2_fn(peer.peer_o, peer.peer_lse, peer.peer_b_seq_len, peer.peer_mid_o, peer.peer_mid_lse, peer.block_seq)
        comm.wait_for_default_stream()

    if master is not None and peer is None:
        # start the (spinning) receive of the partials only once this instance's own stage 1 is done,
        # so that it does not hold SM slots while stage 1 runs; the peers finish at about the same time
        comm.wait_for_default_stream()
    comm.nccl_group_start()
    if master is not None:
        others = [r for r in master.peers if r != my_rank]
        for i, prank in enumerate(others):
            comm.nccl_recv(master.global_mid_o[i], prank)
            comm.nccl_recv(master.global_mid_lse[i], prank)
    if peer is not None:
        for mrank, (b0, b1) in zip(peer.masters, peer.ranges):
            comm.nccl_send(peer.peer_o[b0:b1], mrank)
            comm.nccl_send(peer.peer_lse[b0:b1], mrank)
    comm.nccl_group_end()

    o_tensor = None
    comm.let_default_stream_wait()
    if master is not None:
        o_tensor = torch.empty_like(q) if out is None else out
        stage2_fn(o_tensor, master.global_out_lse, master.global_merge_len, master.global_mid_o,
                  master.global_mid_lse, 1)
    return o_tensor
