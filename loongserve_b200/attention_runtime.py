"""Buffer contracts and call order of the attention path in the reference's model runtime, without the
rest of the model: what ``LongServeLlamaModel._prefill`` / ``_decode`` / ``decoding_stage_migration`` and the
attention part of ``LongServeTransformerLayerInfer`` do around the kernels
(loongserve/models/llama/longserve_model.py:324-436, :438-538, :563-622;
loongserve/models/llama/layer_infer/longserve_transformer_layer_infer.py:76-102, :104-222, :224-370).

The state object carries the reference's field names (loongserve/models/llama/longserve_infer_struct.py:18-133),
so code written against ``infer_state.q_b_seq_len`` etc. keeps working.  Projections, RoPE, FFN and sampling are
not here: the caller hands in q and the freshly computed K/V rows of each layer.
"""
from __future__ import annotations

from types import SimpleNamespace
from typing import List, Optional, Sequence

import torch

from . import context_attention as ca
from . import flash_decoding as fd
from . import kv_ops
from . import ring as ringmod
from .mem_manager import LongServeMemoryManager, LongServeReqManager


def next_power_of_2(n: int) -> int:
    return 1 << (max(int(n), 1) - 1).bit_length()


class LongServeLlamaInferStateInfo(SimpleNamespace):
    """Per-batch state; attribute names as in the reference's class of the same name."""


class ESPAttentionRuntime:
    """Owns the KV pool, the request table and the SP communicator of one instance (one GPU).

    ``sp_comm`` needs the RNCCLComm surface; it may be None when every batch runs on this instance alone.
    ``total_rank`` is this instance's SP rank.  ``dtype`` is the KV / activation dtype (fp16 or bf16)."""

    def __init__(self, *, layers_num: int, q_head_num: int, kv_head_num: int, head_dim: int, max_total_token_num: int,
                 max_req_num: int, max_seq_length: int, sp_world_size: int = 1, total_rank: int = 0, sp_comm=None,
                 dtype=torch.bfloat16, device="cuda", decode_block_seq: Optional[int] = None,
                 peer_memory_decode="auto", peer_memory_max_batch: Optional[int] = None, gathered_prefill: bool = False):
        self.layers_num = layers_num
        self.tp_q_head_num_ = q_head_num
        self.tp_k_head_num_ = kv_head_num
        self.tp_v_head_num_ = kv_head_num
        self.head_dim_ = head_dim
        self.total_rank_ = total_rank
        self.sp_world_size = sp_world_size
        self.sp_comm = sp_comm
        self.dtype = dtype
        self.device = torch.device(device)
        self.decode_block_seq = decode_block_seq
        # longserve_model.py:120-133: sp_world_size spare rows are appended to the pool and never handed out
        self.mem_manager = LongServeMemoryManager(max_total_token_num, dtype, kv_head_num, head_dim, layers_num,
                                                  num_idle_slots=sp_world_size, device=device)
        self.req_manager = LongServeReqManager(max_req_num, max_seq_length, self.mem_manager)
        self._fused_groups = {}
        # Striped prefill passes over all instances in two attention launches instead of sp_world_size (every block copied to
        # every instance by copy engines, ``ring.gathered_context_attention``): opt-in, for batches without scale-down
        # bookkeeping whose request lengths are known on the host.  The exchange buffer is made at the first such batch and
        # grown when a later one needs more (collective: all instances see the same batches).
        self.gathered_prefill = bool(gathered_prefill) and sp_world_size > 1
        self._gather = None
        # decode layer calls between two reads of the device status words (0 = never read them here)
        self.status_check_interval = 32 * 64
        self._decode_calls = 0
        # Multi-master decode exchanges queries and partials over peer memory (NVLink stores and flags inside the kernels)
        # whenever all instances sit in one node; the NCCL message exchange of the reference stays available
        # (peer_memory_decode=False) and is what batches that do not span every instance use.
        if peer_memory_decode == "auto":
            peer_memory_decode = (sp_comm is not None and sp_world_size > 1 and self.device.type == "cuda"
                                  and hasattr(sp_comm, "nccl_send") and torch.cuda.device_count() >= sp_world_size)
        if peer_memory_decode and sp_world_size > 1:
            mb = int(peer_memory_max_batch or min(max_req_num, 256))
            for master in range(sp_world_size):
                self.enable_peer_memory_decode(master, self._ring_all_gather_bytes, max_batch=mb)

    def enable_peer_memory_decode(self, master_rank: int, all_gather_bytes, max_batch: int):
        """Use NVLink stores and flags inside the kernels (``peer_decode.FusedDecodeGroup``) instead of NCCL messages
        for decode batches whose only master is ``master_rank`` and whose peers are all instances.  Collective:
        every instance must call it, with an ``all_gather_bytes`` that returns each rank's bytes in rank order."""
        from .peer_decode import FusedDecodeGroup
        if master_rank in self._fused_groups:
            self._fused_groups.pop(master_rank).close()
        self._fused_groups[master_rank] = FusedDecodeGroup(self.total_rank_, self.sp_world_size, master_rank, max_batch,
                                                           self.tp_q_head_num_, self.head_dim_, all_gather_bytes, self.dtype)

    def _ring_all_gather_bytes(self, mine: bytes) -> List[bytes]:
        """Every instance's 64 bytes in SP-rank order, passed round the ring of all instances over the communicator."""
        P, rank = self.sp_world_size, self.total_rank_
        assert len(mine) == 64
        got = [None] * P
        got[rank] = mine
        cur = torch.tensor(list(mine), dtype=torch.uint8, device=self.device)
        nxt, prv = (rank + 1) % P, (rank - 1 + P) % P
        for i in range(1, P):
            recv = torch.empty_like(cur)
            self.sp_comm.wait_for_default_stream()
            self.sp_comm.nccl_group_start()
            self.sp_comm.nccl_recv(recv, prv)
            self.sp_comm.nccl_send(cur, nxt)
            self.sp_comm.nccl_group_end()
            self.sp_comm.let_default_stream_wait()
            got[(rank - i) % P] = bytes(recv.cpu().tolist())
            cur = recv
        return got

    def close(self):
        for g in self._fused_groups.values():
            g.close()
        self._fused_groups = {}
        if self._gather is not None:
            self._gather.close()
            self._gather = None

    def _gather_exchange(self, nbytes: int):
        """The gather buffer of this instance, at least ``nbytes`` large (every instance computes the same size)."""
        if self._gather is None or self._gather.gathered_bytes < nbytes:
            from .peer_ring import CopyEngineGather
            if self._gather is not None:
                self._gather.close()
            self._gather = CopyEngineGather(self.total_rank_, self.sp_world_size, nbytes, self._ring_all_gather_bytes,
                                            device=self.device)
        return self._gather

    def check_device_status(self):
        """Raise if a bounded in-kernel wait ran out, or a kernel met a slot id outside the pool, on this device since
        the last check.  Synchronises the device: call it where the caller synchronises anyway (``token_attention`` does
        every ``status_check_interval`` decode layers calls).  After a timed-out wait the gated kernels of the device
        return at once and publish nothing until the status has been read here."""
        st = ca.device_status()
        dst = fd.device_status(clear=True)
        kst = kv_ops.device_status(clear=True)
        for name, v in (("prefill kernel", st), ("decode kernels / flag waits", dst), ("KV pool kernels", kst)):
            if v[0] != 0:
                raise RuntimeError(f"ESP attention device status, {name}: code {v[0]} ({tuple(v)})")

    # ------------------------------------------------------------------------------------------ prefill
    @torch.no_grad()
    def prepare_prefill(self, batch_size, total_token_num, max_token_num, max_len_in_batch, b_req_idx, b_start_loc,
                        b_seq_len, first_token_global_idx, logical_sp_peer_ranks: Sequence[int], logical_sp_rank: int,
                        need_context_migration: bool = False, kv_cache_index_begin=None, kv_cache_index_end=None,
                        request_lengths: Optional[Sequence[int]] = None, striped: bool = True):
        """longserve_model.py:324-436.  ``request_lengths`` (host list of the FULL request lengths) lets the
        metadata of every peer's block be computed on the host; without it the local metadata is used for a
        single-instance batch only."""
        st = LongServeLlamaInferStateInfo()
        st.is_prefill = True
        st.batch_size, st.total_token_num, st.max_token_num, st.max_len_in_batch = batch_size, total_token_num, max_token_num, max_len_in_batch
        assert b_req_idx.shape[0] == b_start_loc.shape[0] == b_seq_len.shape[0] == batch_size
        st.b_req_idx = b_req_idx
        st.q_b_start_loc, st.q_b_seq_len, st.q_first_token_global_idx = b_start_loc, b_seq_len, first_token_global_idx
        st.mem_manager, st.req_manager = self.mem_manager, self.req_manager
        st.logical_sp_peer_ranks, st.logical_sp_rank = list(logical_sp_peer_ranks), logical_sp_rank
        st.need_context_migration = bool(need_context_migration)
        P = len(st.logical_sp_peer_ranks)
        if need_context_migration:
            assert kv_cache_index_begin.shape[0] == kv_cache_index_end.shape[0] == batch_size
            st.kv_cache_index_begin, st.kv_cache_index_end = kv_cache_index_begin, kv_cache_index_end
            st.cur_kv_cache_index = torch.empty((batch_size,), dtype=torch.int32, device=self.device)
        alloc_mem = self.mem_manager.alloc_contiguous(total_token_num) if not need_context_migration else None
        if alloc_mem is not None:
            st.mem_is_contiguous = True
            st.mem_index, st.mem_start, st.mem_end = alloc_mem
        else:
            st.mem_is_contiguous = False
            n = total_token_num if not need_context_migration else int(torch.sum(kv_cache_index_end - kv_cache_index_begin).item())
            st.mem_index = self.mem_manager.alloc(n)
        H2 = self.tp_k_head_num_ + self.tp_v_head_num_
        st.kv_buffer = torch.empty((max_token_num, H2, self.head_dim_), dtype=self.dtype, device=self.device)
        st.peer_kv_buffer = torch.empty_like(st.kv_buffer) if P > 1 else None
        st.local_m = torch.empty((max_token_num, self.tp_q_head_num_), dtype=torch.float32, device=self.device)
        st.local_l = torch.empty_like(st.local_m)
        if not need_context_migration:
            kv_ops.init_req_to_token_indexes(self.req_manager.req_to_token_indexs, b_req_idx, b_seq_len, st.mem_index,
                                             max_len_in_batch)
        if request_lengths is not None:
            local_len, first, stride = ringmod.shard_lengths(request_lengths, P, striped)
            st.block_metas = [ringmod.BlockMeta.from_lengths(local_len[r], first[r], self.device) for r in range(P)]
            st.stride = stride
            if (self.gathered_prefill and striped and not need_context_migration and P == self.sp_world_size
                    and st.logical_sp_peer_ranks == list(range(P)) and logical_sp_rank == self.total_rank_):
                st.request_lengths = [int(x) for x in request_lengths]
                st.gather_plans = [ringmod.GatherPlan.build(st.request_lengths, P, r, self.device) for r in range(P)]
                row_bytes = H2 * self.head_dim_ * torch.empty((), dtype=self.dtype).element_size()
                self._gather_exchange(max(p.rows for p in st.gather_plans) * row_bytes)
        elif P == 1:
            st.block_metas = [ringmod.BlockMeta(b_start_loc, b_seq_len, first_token_global_idx)]
            st.stride = 1
        else:
            # no host knowledge of the other instances' shards: pass the metadata round the ring once per batch
            # (the reference sends it along with every KV block of every layer,
            # longserve_transformer_layer_infer.py:162-178)
            st.block_metas = self._exchange_block_metas(b_start_loc, b_seq_len, first_token_global_idx,
                                                        st.logical_sp_peer_ranks, logical_sp_rank)
            st.stride = P if striped else 1
        if need_context_migration:
            st.keep_plan = ringmod.KeepPlan(kv_cache_index_begin, kv_cache_index_end, st.mem_index, b_req_idx,
                                            self.req_manager.req_to_token_indexs, st.cur_kv_cache_index)
        return st

    def _exchange_block_metas(self, b_start_loc, b_seq_len, first_token_global_idx, peers, rank):
        P = len(peers)
        mine = torch.stack([b_start_loc, b_seq_len, first_token_global_idx]).to(torch.int32).contiguous()
        metas = [None] * P
        metas[rank] = mine
        cur = mine
        nxt, prv = peers[(rank + 1) % P], peers[(rank - 1 + P) % P]
        for i in range(1, P):
            recv = torch.empty_like(mine)
            self.sp_comm.wait_for_default_stream()
            self.sp_comm.nccl_group_start()
            self.sp_comm.nccl_recv(recv, prv)
            self.sp_comm.nccl_send(cur, nxt)
            self.sp_comm.nccl_group_end()
            self.sp_comm.let_default_stream_wait()
            metas[(rank - i) % P] = recv
            cur = recv
        return [ringmod.BlockMeta(m[0], m[1], m[2]) for m in metas]

    def migrate_chunked(self, is_receiver: bool, req_indices, migration_lens, seq_lens, peer_sp_rank: int, max_mig_len: int):
        """Decode-stage migration of a list of requests in chunks of at most ``max_mig_len`` tokens, in the order
        and with the bookkeeping of the reference's worker shell
        (loongserve/longserve_server/router/model_infer/model_rpc.py:178-217): requests are taken from the END of
        the lists; a request larger than the remaining buffer is split and its rest re-queued; the local length of a
        request grows (receiver) or shrinks (sender) by each chunk.  ``seq_lens`` is updated in place and returned."""
        req_indices, migration_lens, seq_lens = list(req_indices), list(migration_lens), list(seq_lens)
        lens_by_req = dict(zip(req_indices, seq_lens))
        pending = list(zip(req_indices, migration_lens))
        while pending:
            room = max_mig_len
            b_req, b_mig, b_len = [], [], []
            while pending and room > 0:
                rid, mig = pending.pop()
                cur = min(room, mig)
                room -= cur
                mig -= cur
                b_req.append(rid); b_mig.append(cur); b_len.append(lens_by_req[rid])
                lens_by_req[rid] += cur if is_receiver else -cur
                if room == 0:
                    if mig > 0:
                        pending.append((rid, mig))
                    break
            i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=self.device)
            self.decoding_stage_migration(is_receiver, i32(b_req), i32(b_mig), i32(b_len), peer_sp_rank,
                                          migration_len_sum=sum(b_mig), max_migration_len=max(b_mig))
        return [lens_by_req[r] for r in req_indices]

    def pre_cache_kv(self, st, layer_idx: int):
        """Buffer the layer's new K/V rows must be written into: the pool slice itself when the slots are
        contiguous, else the scratch block (longserve_transformer_layer_infer.py:76-84)."""
        if st.mem_is_contiguous:
            return self.mem_manager.kv_buffer[layer_idx][st.mem_start:st.mem_end, :, :]
        return st.kv_buffer

    @torch.inference_mode()
    def context_attention(self, q, st, layer_idx: int, out=None, overlap: bool = True):
        """One layer's attention of a prefill batch: pool write (when needed) + ring pass
        (longserve_transformer_layer_infer.py:98-222).  K/V of this layer must already be in
        ``pre_cache_kv(st, layer_idx)``."""
        P = len(st.logical_sp_peer_ranks)
        Hq, Hkv, D = self.tp_q_head_num_, self.tp_k_head_num_, self.head_dim_
        if st.mem_is_contiguous:
            kv = self.mem_manager.kv_buffer[layer_idx][st.mem_start:st.mem_start + st.max_token_num]
        else:
            kv = st.kv_buffer
            if not st.need_context_migration:
                kv_ops.destindex_copy_kv(kv[:st.total_token_num], st.mem_index, self.mem_manager.kv_buffer[layer_idx])
        o = torch.empty_like(q) if out is None else out
        if getattr(st, "gather_plans", None) is not None:
            ringmod.gathered_context_attention(
                q.view(-1, Hq, D), kv, o.view(-1, Hq, D), st.local_m[:q.shape[0]], st.local_l[:q.shape[0]],
                rank=st.logical_sp_rank, lens=st.request_lengths, P=P, metas=st.block_metas, plans=st.gather_plans,
                max_len_in_batch=st.max_len_in_batch, num_kv_heads=Hkv, attention_fn=ca.context_attention_fwd,
                init_fn=ca.init_attention_state, gather=self._gather)
            return o
        ringmod.ring_context_attention(
            q.view(-1, Hq, D), kv, o.view(-1, Hq, D), st.local_m[:q.shape[0]], st.local_l[:q.shape[0]],
            rank=st.logical_sp_rank, peers=st.logical_sp_peer_ranks, metas=st.block_metas, stride=st.stride,
            max_len_in_batch=st.max_len_in_batch, num_kv_heads=Hkv, comm=self.sp_comm,
            recv_buffers=[st.peer_kv_buffer, st.kv_buffer], attention_fn=ca.context_attention_fwd,
            init_fn=ca.init_attention_state, overlap=overlap,
            keep=st.keep_plan if st.need_context_migration else None,
            pool_layer=self.mem_manager.kv_buffer[layer_idx], layer_idx=layer_idx,
            keep_fns=(kv_ops.pre_copy_and_register_kv, kv_ops.destindex_copy_and_register_kv))
        return o

    # ------------------------------------------------------------------------------------------ decode
    @torch.no_grad()
    def prepare_decode(self, batch_size, total_token_num, max_len_in_batch, b_req_idx, b_seq_len, first_token_global_idx,
                       sp_master_rank, logical_sp_peer_ranks, logical_sp_rank, peer_sp_master_rank_list=None,
                       peer_query_buffer_range_list=None, peer_batch_size=0, peer_max_len_in_batch=0, peer_b_req_idx=None,
                       peer_b_seq_len=None):
        """longserve_model.py:438-538: slot for every new token on its master (registered at position len-1),
        split size, partial buffers for the master and peer roles."""
        st = LongServeLlamaInferStateInfo()
        is_master = sp_master_rank == self.total_rank_
        st.is_prefill = False
        st.batch_size, st.total_token_num, st.max_len_in_batch = batch_size, total_token_num, max_len_in_batch
        st.b_req_idx, st.q_b_seq_len, st.q_first_token_global_idx = b_req_idx, b_seq_len, first_token_global_idx
        st.mem_manager, st.req_manager = self.mem_manager, self.req_manager
        st.sp_master_rank, st.logical_sp_peer_ranks, st.logical_sp_rank = sp_master_rank, logical_sp_peer_ranks, logical_sp_rank
        Hq, D = self.tp_q_head_num_, self.head_dim_
        H2 = self.tp_k_head_num_ + self.tp_v_head_num_
        if is_master:
            assert b_req_idx.shape[0] == b_seq_len.shape[0] == batch_size == total_token_num and total_token_num > 0
            alloc_mem = self.mem_manager.alloc_contiguous(total_token_num)
            if alloc_mem is not None:
                st.mem_is_contiguous = True
                st.mem_index, st.mem_start, st.mem_end = alloc_mem
            else:
                st.mem_is_contiguous = False
                st.mem_index = self.mem_manager.alloc(total_token_num)
                st.kv_buffer = torch.empty((total_token_num, H2, D), dtype=self.dtype, device=self.device)
            kv_ops.copy_kv_index_to_req(self.req_manager.req_to_token_indexs, b_req_idx, b_seq_len, st.mem_index)
        if self.decode_block_seq is not None:
            st.BLOCK_SEQ = int(self.decode_block_seq)          # native callers may pick far larger splits
        else:
            st.BLOCK_SEQ = min(next_power_of_2(max(max_len_in_batch or 0, peer_max_len_in_batch or 0, 16)), 256)
        P = len(logical_sp_peer_ranks) if logical_sp_peer_ranks is not None else 1
        f32 = dict(dtype=torch.float32, device=self.device)
        st.master_plan = st.peer_plan = None
        if is_master:
            nblk = (max_len_in_batch + st.BLOCK_SEQ - 1) // st.BLOCK_SEQ
            st.num_seq_block = nblk
            st.global_mid_o = torch.empty((P - 1 + nblk, batch_size, Hq, D), **f32)
            st.global_mid_o_logexpsum = torch.empty((P - 1 + nblk, batch_size, Hq), **f32)
            st.global_merge_len = ((P - 1) + (b_seq_len + (st.BLOCK_SEQ - 1)) // st.BLOCK_SEQ).view((batch_size,)).to(torch.int32).contiguous().clone()
            st.global_out_logexpsum = torch.empty((batch_size, Hq), **f32)
            st.master_plan = ringmod.MasterPlan(peers=list(logical_sp_peer_ranks), b_req_idx=b_req_idx, b_seq_len=b_seq_len,
                                                max_len_in_batch=max_len_in_batch, block_seq=st.BLOCK_SEQ,
                                                global_mid_o=st.global_mid_o, global_mid_lse=st.global_mid_o_logexpsum,
                                                global_merge_len=st.global_merge_len, global_out_lse=st.global_out_logexpsum)
        if peer_sp_master_rank_list is not None:
            assert len(peer_sp_master_rank_list) == len(peer_query_buffer_range_list)
            assert peer_batch_size == peer_b_req_idx.shape[0] == peer_b_seq_len.shape[0] == peer_query_buffer_range_list[-1][1]
            st.peer_query_buffer = torch.empty((peer_batch_size, Hq, D), dtype=self.dtype, device=self.device)
            st.peer_sp_master_rank_list, st.peer_query_buffer_range_list = peer_sp_master_rank_list, peer_query_buffer_range_list
            st.peer_batch_size, st.peer_b_req_idx, st.peer_b_seq_len = peer_batch_size, peer_b_req_idx, peer_b_seq_len
            st.peer_max_len_in_batch = max(peer_max_len_in_batch, max_len_in_batch or 0)
            nblk = st.peer_max_len_in_batch // st.BLOCK_SEQ + 1
            st.peer_local_mid_o = torch.empty((nblk, peer_batch_size, Hq, D), **f32)
            st.peer_local_mid_o_logexpsum = torch.empty((nblk, peer_batch_size, Hq), **f32)
            st.peer_local_o = torch.empty((peer_batch_size, Hq, D), **f32)
            st.peer_local_out_logexpsum = torch.empty((peer_batch_size, Hq), **f32)
            st.peer_plan = ringmod.PeerPlan(masters=list(peer_sp_master_rank_list), ranges=list(peer_query_buffer_range_list),
                                            peer_query_buffer=st.peer_query_buffer, peer_b_req_idx=peer_b_req_idx,
                                            peer_b_seq_len=peer_b_seq_len, peer_max_len_in_batch=st.peer_max_len_in_batch,
                                            block_seq=st.BLOCK_SEQ, peer_mid_o=st.peer_local_mid_o,
                                            peer_mid_lse=st.peer_local_mid_o_logexpsum, peer_o=st.peer_local_o,
                                            peer_lse=st.peer_local_out_logexpsum)
        return st

    def decode_cache_kv(self, st, layer_idx: int):
        """Where the master writes the new tokens' K/V rows of this layer: the pool slice when contiguous, else
        the scratch rows that ``post_decode_cache_kv`` scatters (longserve_transformer_layer_infer.py:76-102)."""
        if st.mem_is_contiguous:
            return self.mem_manager.kv_buffer[layer_idx][st.mem_start:st.mem_end, :, :]
        return st.kv_buffer

    @torch.inference_mode()
    def post_decode_cache_kv(self, st, layer_idx: int):
        if not st.mem_is_contiguous:
            kv_ops.destindex_copy_kv(st.kv_buffer, st.mem_index, self.mem_manager.kv_buffer[layer_idx])

    @torch.inference_mode()
    def token_attention(self, q, st, layer_idx: int, out=None):
        """One layer's decode attention on this instance in its master and/or peer role
        (longserve_transformer_layer_infer.py:224-370).  Masters get the attention output, pure peers None."""
        pool_layer = self.mem_manager.kv_buffer[layer_idx]
        self._decode_calls += 1
        if (self.status_check_interval and self._decode_calls % self.status_check_interval == 0
                and not torch.cuda.is_current_stream_capturing()):
            self.check_device_status()
        single = st.peer_plan is None and (st.master_plan is None or len(st.master_plan.peers) == 1)
        if single and st.master_plan is not None:
            # the whole batch lives here: no exchange, stage 1 + merge only
            mp = st.master_plan
            Hkv = self.tp_k_head_num_
            qv = q.view(-1, self.tp_q_head_num_, self.head_dim_)
            fd.flash_decoding_stage1(mp.global_mid_o, mp.global_mid_lse, qv, pool_layer[:, :Hkv, :], pool_layer[:, Hkv:, :],
                                     self.req_manager.req_to_token_indexs, mp.b_req_idx, mp.b_seq_len, mp.max_len_in_batch,
                                     mp.block_seq)
            o = torch.empty_like(qv) if out is None else out
            fd.flash_decoding_stage2(o.view(-1, self.tp_q_head_num_, self.head_dim_), mp.global_out_lse, mp.b_seq_len,
                                     mp.global_mid_o, mp.global_mid_lse, mp.block_seq)
            return o
        qv = q.view(-1, self.tp_q_head_num_, self.head_dim_) if q is not None else None
        if self._fused_covers(st):
            return self._token_attention_peer_memory(qv, st, pool_layer, out)
        return ringmod.multi_master_decode_attention(qv, pool_layer, self.req_manager.req_to_token_indexs, self.tp_k_head_num_,
                                                     self.sp_comm, self.total_rank_, st.master_plan, st.peer_plan,
                                                     fd.flash_decoding_stage1, fd.flash_decoding_stage2, out=out)

    def _fused_covers(self, st) -> bool:
        """Whether this decode step goes over peer memory.  Decided from what EVERY instance of the batch knows -- the
        batch's instance list, the masters named in the plans, and the groups that exist -- so that a master and its
        peers always choose the same exchange: the batch must span all instances (the groups' layout assumes that) and
        every master in sight must have a group."""
        if not self._fused_groups:
            return False
        peers = getattr(st, "logical_sp_peer_ranks", None)
        if peers is None or sorted(peers) != list(range(self.sp_world_size)):
            return False
        masters = []          # (master rank, size of its mini-batch): both sides know both numbers
        if st.master_plan is not None:
            masters.append((self.total_rank_, int(st.master_plan.b_seq_len.shape[0])))
        if st.peer_plan is not None:
            masters += [(m, b - a) for m, (a, b) in zip(st.peer_plan.masters, st.peer_plan.ranges)]
        return bool(masters) and all(m in self._fused_groups and n <= self._fused_groups[m].B for m, n in masters)

    def _token_attention_peer_memory(self, qv, st, pool_layer, out):
        """The exchange of longserve_transformer_layer_infer.py:224-370 over peer memory: every master first pushes its
        queries (so no instance waits for one that is itself waiting), then serves the other masters' mini-batches in the
        order of ``peer_sp_master_rank_list``, then attends to its own tokens and merges."""
        rtt, Hkv = self.req_manager.req_to_token_indexs, self.tp_k_head_num_
        mp, pp = st.master_plan, st.peer_plan
        # a group's step counter advances only when the group is really used this step, on the master (which always
        # pushes) and on a peer (which serves unless the master's mini-batch is empty) alike: counters that drifted
        # apart would let a stale flag satisfy a later wait
        groups = ([self._fused_groups[self.total_rank_]] if mp is not None else []) + \
                 ([self._fused_groups[m] for m, (a, b) in zip(pp.masters, pp.ranges) if b > a] if pp is not None else [])
        for g in groups:
            g.next_step()
        if mp is not None:
            own = self._fused_groups[self.total_rank_]
            qv = qv.contiguous()
            own.master_push(qv)
        if pp is not None:
            Hq, D = self.tp_q_head_num_, self.head_dim_
            nblk = (pp.peer_max_len_in_batch + pp.block_seq - 1) // pp.block_seq
            for m, (a, b) in zip(pp.masters, pp.ranges):
                n = b - a
                if n == 0:
                    continue
                mid_o = pp.peer_mid_o.view(-1)[:nblk * n * Hq * D].view(nblk, n, Hq, D)        # scratch reused master after master
                mid_lse = pp.peer_mid_lse.view(-1)[:nblk * n * Hq].view(nblk, n, Hq)
                self._fused_groups[m].peer_serve(pool_layer, rtt, Hkv, pp.peer_b_req_idx[a:b], pp.peer_b_seq_len[a:b],
                                                 pp.peer_max_len_in_batch, pp.block_seq, mid_o, mid_lse)
        if mp is None:
            return None
        n_other = len(mp.peers) - 1
        o, _ = own.master_finish(qv, pool_layer, rtt, Hkv, mp.b_req_idx, mp.b_seq_len, mp.max_len_in_batch, mp.block_seq,
                                 mp.global_mid_o[n_other:], mp.global_mid_lse[n_other:], out=out, out_lse=mp.global_out_lse)
        return o

    # ------------------------------------------------------------------------------------------ migration
    @torch.inference_mode()
    def decoding_stage_migration(self, is_receiver: bool, b_req_idx, b_migration_len, b_seq_len, peer_sp_rank: int,
                                 migration_len_sum: Optional[int] = None, max_migration_len: Optional[int] = None):
        """longserve_model.py:563-622.  Assumes a reference count of one on the migrated slots, like the
        reference.  ``migration_len_sum`` / ``max_migration_len`` (host ints) avoid the two device->host reads."""
        total = int(migration_len_sum) if migration_len_sum is not None else int(torch.sum(b_migration_len).item())
        H2 = self.tp_k_head_num_ + self.tp_v_head_num_
        buf = torch.empty((self.layers_num, total, H2, self.head_dim_), dtype=self.dtype, device=self.device)
        if total == 0:
            return
        if is_receiver:
            # `buf` may be memory a kernel queued earlier on this stream still reads (the allocator hands a freed block
            # back at once): the communicator's stream must not write into it before that kernel has finished
            self.sp_comm.wait_for_default_stream()
            self.sp_comm.nccl_recv(buf, peer_sp_rank)
            alloc_mem = self.mem_manager.alloc(total)
            self.sp_comm.let_default_stream_wait()
            kv_ops.decoding_stage_migration_receiver_kernel(buf, self.req_manager.req_to_token_indexs, self.mem_manager.kv_buffer,
                                                            alloc_mem, b_req_idx, b_migration_len, b_seq_len, max_migration_len)
        else:
            kv_ops.decoding_stage_migration_sender_kernel(buf, self.req_manager.req_to_token_indexs, self.mem_manager.mem_state,
                                                          self.mem_manager.kv_buffer, b_req_idx, b_migration_len, b_seq_len,
                                                          max_migration_len)
            self.sp_comm.wait_for_default_stream()
            self.sp_comm.nccl_send(buf, peer_sp_rank)
            # `buf` goes back to the allocator when this function returns: whatever reuses it on this stream has to wait
            # for the send that still reads it (the reference fences here too, longserve_model.py:622)
            self.sp_comm.let_default_stream_wait()
            # the kernel zeroed the device reference counts; tell the host allocator which slots those were
            # (a device->host read, acceptable here: migration is not on the per-step path)
            rt_, ids = self.req_manager.req_to_token_indexs, []
            lens_h, mig_h, req_h = b_seq_len.tolist(), b_migration_len.tolist(), b_req_idx.tolist()
            for rid, n, L in zip(req_h, mig_h, lens_h):
                if n:
                    ids.append(rt_[rid, L - n:L])
            self.mem_manager.release_on_host(torch.cat(ids))
