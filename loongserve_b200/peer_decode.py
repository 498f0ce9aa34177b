"""Distributed decode attention over peer memory: the exchange of the multi-master decode step
(loongserve/models/llama/layer_infer/longserve_transformer_layer_infer.py:224-370) done with NVLink stores and
flags inside the kernels instead of NCCL messages.  A group has one master; a batch with several masters uses one group
per master (``ESPAttentionRuntime.enable_peer_memory_decode`` for each), every instance pushing its own queries first and
then serving the other masters.  The instances of a group make the same calls once per layer, in the same order.

Memory of one instance's shared region (created once, mapped by every other instance):
  [ q slot: B_max*Hq*D 16-bit | partial o: P*B_max*Hq*D fp32 | partial lse: P*B_max*Hq fp32 | flags: 64 int32 ]
flags[0] = "q of step s has arrived" (written by the master), flags[1+p] = "partial of peer p for step s has
arrived" (written by peer p into the master's region).
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, List, Optional, Sequence

import torch

from . import _lib
from ._util import dtype_tag, ptr, stream_ptr


class FusedDecodeGroup:
    def __init__(self, rank: int, world: int, master: int, max_batch: int, num_q_heads: int, head_dim: int,
                 all_gather_bytes: Callable[[bytes], List[bytes]], dtype=torch.bfloat16):
        """``all_gather_bytes(b)`` returns every rank's bytes in rank order (e.g. built on
        ``torch.distributed.all_gather_object``); it is used once, to exchange the 64-byte buffer handles."""
        assert 0 <= master < world and 0 <= rank < world
        self.rank, self.world, self.master, self.dtype = rank, world, master, dtype
        self.B, self.Hq, self.D = max_batch, num_q_heads, head_dim
        lib = _lib.attn()
        self._lib = lib
        es = 2
        self.q_bytes = max_batch * num_q_heads * head_dim * es
        self.off_o = (self.q_bytes + 255) // 256 * 256
        self.o_bytes = world * max_batch * num_q_heads * head_dim * 4
        self.off_lse = self.off_o + self.o_bytes
        self.lse_bytes = world * max_batch * num_q_heads * 4
        self.off_flags = (self.off_lse + self.lse_bytes + 255) // 256 * 256
        self.total = self.off_flags + 256
        base = C.c_void_p()
        handle = (C.c_uint8 * 64)()
        _lib.check(lib.esp_peer_buffer_create(self.total, C.byref(base), handle), "esp_peer_buffer_create")
        self.base = base.value
        handles = all_gather_bytes(bytes(handle))
        self.peer_base: List[Optional[int]] = [None] * world
        for r in range(world):
            if r == rank:
                self.peer_base[r] = self.base
            elif rank == master or r == master:          # only master <-> peer mappings are needed
                p = C.c_void_p()
                hb = (C.c_uint8 * 64)(*handles[r])
                _lib.check(lib.esp_peer_buffer_open(hb, C.byref(p)), "esp_peer_buffer_open")
                self.peer_base[r] = p.value
        self.step_id = 0
        self._ones = None
        self.peers = [r for r in range(world) if r != master]

    def close(self):
        for r, p in enumerate(self.peer_base):
            if p is not None and r != self.rank:
                self._lib.esp_peer_buffer_close(p)
        if self.base:
            self._lib.esp_peer_buffer_destroy(self.base)
            self.base = None

    def _values(self, step_value, value_base):
        if step_value is None:
            return self.step_id, None
        assert value_base is not None and value_base.dtype == torch.int32
        return int(step_value), ptr(value_base)

    def next_step(self) -> int:
        """Advance the group's own step counter: once per layer call, on every instance of the group alike."""
        self.step_id += 1
        return self.step_id

    @torch.inference_mode()
    def master_push(self, q, step_value=None, value_base=None):
        """Master, phase 1: copy q [batch, Hq, D] into every peer's q slot and raise their flags."""
        sid, vb = self._values(step_value, value_base)
        batch = q.shape[0]
        assert self.rank == self.master and q.is_contiguous() and q.shape == (batch, self.Hq, self.D) and 0 < batch <= self.B
        n = len(self.peers)
        if n:
            dsts = (C.c_void_p * n)(*[self.peer_base[r] for r in self.peers])
            flags = (C.c_void_p * n)(*[self.peer_base[r] + self.off_flags for r in self.peers])
            _lib.check(self._lib.esp_peer_push(ptr(q), dsts, flags, n, batch * self.Hq * self.D * 2, sid, vb, stream_ptr()), "esp_peer_push")

    @torch.inference_mode()
    def master_finish(self, q, pool_layer, req_to_token_indexs, num_kv_heads: int, b_req_idx, b_seq_len, max_len_in_batch: int,
                      block_seq: int, mid_o, mid_lse, out=None, out_lse=None, step_value=None, value_base=None):
        """Master, phase 2: attention over the local tokens, then the merge with the peers' partials (waits for their
        flags).  Returns (o in q's dtype, lse)."""
        lib, s = self._lib, stream_ptr()
        sid, vb = self._values(step_value, value_base)
        batch, Hq, D, Hkv = b_seq_len.shape[0], self.Hq, self.D, num_kv_heads
        k_cache, v_cache = pool_layer[:, :Hkv, :], pool_layer[:, Hkv:, :]
        nblk = (max_len_in_batch + block_seq - 1) // block_seq
        _lib.check(lib.esp_decode_stage1(ptr(mid_o), ptr(mid_lse), ptr(q), ptr(k_cache), ptr(v_cache), k_cache.stride(0),
                                         k_cache.stride(1), v_cache.stride(0), v_cache.stride(1), ptr(req_to_token_indexs),
                                         req_to_token_indexs.stride(0), ptr(b_req_idx), ptr(b_seq_len), batch, Hq, Hkv, D,
                                         max_len_in_batch, block_seq, dtype_tag(pool_layer), 0.0, pool_layer.shape[0], s),
                   "esp_decode_stage1")
        # merge own blocks into slot [master] of the partial region, then merge the P slots
        own_o = self.base + self.off_o + self.master * batch * Hq * D * 4
        own_lse = self.base + self.off_lse + self.master * batch * Hq * 4
        _lib.check(lib.esp_decode_merge(own_o, own_lse, ptr(b_seq_len), ptr(mid_o), ptr(mid_lse), batch, Hq, D, nblk,
                                        block_seq, _lib.ESP_DTYPE_F32, s), "esp_decode_merge")
        o = torch.empty_like(q) if out is None else out
        lse = torch.empty((batch, Hq), dtype=torch.float32, device=q.device) if out_lse is None else out_lse
        if self._ones is None or self._ones.shape[0] != batch:
            self._ones = torch.full((batch,), self.world, dtype=torch.int32, device=q.device)
        # the P slots are laid out [P, batch, Hq, D] for this step's batch: a merge over P one-token "blocks"
        _lib.check(lib.esp_decode_merge_gated(ptr(o), ptr(lse), ptr(self._ones), self.base + self.off_o,
                                              self.base + self.off_lse, batch, Hq, D, self.world, 1, dtype_tag(o),
                                              self.base + self.off_flags + 4, len(self.peers), sid, vb, s), "esp_decode_merge_gated")
        return o, lse

    @torch.inference_mode()
    def peer_serve(self, pool_layer, req_to_token_indexs, num_kv_heads: int, b_req_idx, b_seq_len, max_len_in_batch: int,
                   block_seq: int, mid_o, mid_lse, step_value=None, value_base=None):
        """Peer: wait for the master's q, attend to the master's requests as stored here, write the fp32 partial into the
        master's memory and raise this peer's flag there."""
        lib, s = self._lib, stream_ptr()
        sid, vb = self._values(step_value, value_base)
        assert self.rank != self.master
        batch, Hq, D, Hkv = b_seq_len.shape[0], self.Hq, self.D, num_kv_heads
        assert 0 < batch <= self.B, "batch exceeds the max_batch the shared region was sized for"
        k_cache, v_cache = pool_layer[:, :Hkv, :], pool_layer[:, Hkv:, :]
        nblk = (max_len_in_batch + block_seq - 1) // block_seq
        _lib.check(lib.esp_decode_stage1_gated(ptr(mid_o), ptr(mid_lse), self.base, ptr(k_cache), ptr(v_cache), k_cache.stride(0),
                                               k_cache.stride(1), v_cache.stride(0), v_cache.stride(1), ptr(req_to_token_indexs),
                                               req_to_token_indexs.stride(0), ptr(b_req_idx), ptr(b_seq_len), batch, Hq, Hkv, D,
                                               max_len_in_batch, block_seq, dtype_tag(pool_layer), 0.0, pool_layer.shape[0],
                                               self.base + self.off_flags, sid, vb, s), "esp_decode_stage1_gated")
        mbase = self.peer_base[self.master]
        slot = self.rank
        _lib.check(lib.esp_decode_merge(mbase + self.off_o + slot * batch * Hq * D * 4, mbase + self.off_lse + slot * batch * Hq * 4,
                                        ptr(b_seq_len), ptr(mid_o), ptr(mid_lse), batch, Hq, D, nblk, block_seq,
                                        _lib.ESP_DTYPE_F32, s), "esp_decode_merge (remote)")
        flag_idx = 1 + self.peers.index(self.rank)
        _lib.check(lib.esp_peer_signal(mbase + self.off_flags + 4 * flag_idx, sid, vb, s), "esp_peer_signal")

    @torch.inference_mode()
    def step(self, q, pool_layer, req_to_token_indexs, num_kv_heads: int, b_req_idx, b_seq_len, max_len_in_batch: int,
             block_seq: int, mid_o, mid_lse, out=None, out_lse=None, step_value: Optional[int] = None, value_base=None):
        """One layer's decode attention of a batch with this group's master as its only master.  On the master ``q`` is
        [batch, Hq, D] and the result (o in q's dtype, lse) is returned; on a peer ``q`` is None, (b_req_idx, b_seq_len)
        describe the master's requests as stored here, and None is returned.  mid_o / mid_lse: local scratch
        [nblk, batch, Hq, D] / [nblk, batch, Hq] fp32 (the peers' partials arrive in the shared region, so scratch only
        needs the local blocks).

        ``step_value`` / ``value_base`` are for callers that record steps into a CUDA graph: the flag value of this
        call becomes ``step_value + value_base[0]`` (an int32 device tensor read when the kernels run) instead of the
        group's own host-side counter; see ``advance``."""
        if step_value is None:
            self.next_step()
        if self.rank == self.master:
            self.master_push(q, step_value, value_base)
            return self.master_finish(q, pool_layer, req_to_token_indexs, num_kv_heads, b_req_idx, b_seq_len, max_len_in_batch,
                                      block_seq, mid_o, mid_lse, out, out_lse, step_value, value_base)
        self.peer_serve(pool_layer, req_to_token_indexs, num_kv_heads, b_req_idx, b_seq_len, max_len_in_batch, block_seq,
                        mid_o, mid_lse, step_value, value_base)
        return None

    def advance(self, n_steps: int):
        """Tell the group that ``n_steps`` steps ran outside its own counting (a graph replay), so that later calls
        without ``step_value`` keep using values above everything already stored in the flags."""
        self.step_id += int(n_steps)

    def device_status(self, clear: bool = True):
        """(code, block, which wait, value) of the bounded flag waits on this device; code 0 = none expired."""
        buf = (C.c_int32 * 4)()
        _lib.check(self._lib.esp_decode_device_status(buf, 1 if clear else 0), "esp_decode_device_status")
        return tuple(buf)
