"""Token-indexed KV pool: slot allocator and request table, with the attribute and method names the
reference's callers use (loongserve/common/longserve_mem_manager.py:7-113,
loongserve/common/longserve_req_manager.py:7-48)."""
from __future__ import annotations

import torch

INT32_MAX = 2147483647


class LongServeMemoryManager:
    """kv_buffer [layer, size + num_idle_slots, 2*head_num, head_dim] (K = heads [0, head_num),
    V = heads [head_num, 2*head_num) of the same slot row), int32 reference counts ``mem_state``,
    lowest-free-first allocation."""

    def __init__(self, size, dtype, head_num, head_dim, layer_num, num_idle_slots=0, always_copy=False,
                 device="cuda"):
        self.size = size
        self.dtype = dtype
        self.head_num = head_num
        self.head_dim = head_dim
        self.layer_num = layer_num
        self.num_idle_slots = num_idle_slots
        self.always_copy = always_copy
        self.device = torch.device(device)
        self.mem_state = torch.zeros((size,), dtype=torch.int32, device=self.device)
        self.indexes = torch.arange(0, size, dtype=torch.long, device=self.device)
        self.can_use_mem_size = size
        self._init_buffers(size, dtype, head_num, head_dim, layer_num, num_idle_slots)

    def _init_buffers(self, size, dtype, head_num, head_dim, layer_num, num_idle_slots):
        self.kv_buffer = torch.empty((layer_num, size + num_idle_slots, 2 * head_num, head_dim), dtype=dtype,
                                     device=self.device)

    def _free_buffers(self):
        self.kv_buffer = None

    @torch.inference_mode()
    def alloc(self, need_size):
        need_size = int(need_size)
        if need_size > self.can_use_mem_size:
            raise RuntimeError(f"not enough KV cache: need_size {need_size} left_size {self.can_use_mem_size}")
        can_use_index = torch.nonzero(self.mem_state == 0).view(-1)
        select_index = can_use_index[0:need_size]
        self.add_refs(select_index)
        return select_index

    @torch.inference_mode()
    def alloc_contiguous(self, need_size):
        need_size = int(need_size)
        if self.always_copy or need_size > self.can_use_mem_size:
            return None
        free = torch.nonzero(self.mem_state == 0).view(-1)
        n = len(free)
        if n < need_size or need_size <= 0:
            return None
        head = free[0:n - need_size + 1]
        head = head[(free[need_size - 1:] - head) == need_size - 1]
        if head.shape[0] == 0:
            return None
        start = int(head[0].item())
        end = start + need_size
        select_index = self.indexes[start:end]
        self.add_refs(select_index)
        return select_index, start, end

    @torch.inference_mode()
    def free(self, free_index):
        self.decrease_refs(free_index.long())

    @torch.inference_mode()
    def add_refs(self, token_index: torch.Tensor):
        state = self.mem_state[token_index]
        has_used_tokens = int(torch.count_nonzero(state).item())
        self.can_use_mem_size -= len(state) - has_used_tokens
        self.mem_state[token_index] += 1

    @torch.inference_mode()
    def decrease_refs(self, token_index: torch.Tensor):
        self.mem_state[token_index] -= 1
        state = self.mem_state[token_index]
        used_tokens = int(torch.count_nonzero(state).item())
        self.can_use_mem_size += len(state) - used_tokens

    @torch.inference_mode()
    def free_all(self):
        self.can_use_mem_size = len(self.mem_state)
        self.mem_state[:] = 0

    @torch.inference_mode()
    def resize_mem(self, new_size):
        self.size = new_size
        self.mem_state = torch.zeros((new_size,), dtype=torch.int32, device=self.device)
        self.indexes = torch.arange(0, new_size, dtype=torch.long, device=self.device)
        self.can_use_mem_size = new_size
        self._free_buffers()
        self._init_buffers(new_size, self.dtype, self.head_num, self.head_dim, self.layer_num, self.num_idle_slots)


class LongServeReqManager:
    """req_to_token_indexs [max_request_num, max_sequence_length] int32, filled with INT32_MAX."""

    def __init__(self, max_request_num, max_sequence_length, mem_manager: LongServeMemoryManager):
        dev = mem_manager.device
        self.req_state = torch.zeros((max_request_num,), dtype=torch.bool, device=dev)
        self.req_to_token_indexs = torch.full((max_request_num, max_sequence_length), fill_value=INT32_MAX,
                                              dtype=torch.int32, device=dev)
        self.can_use_req_size = max_request_num
        self.mem_manager = mem_manager

    def alloc(self, need_size):
        if need_size > self.can_use_req_size:
            return None
        select_index = torch.nonzero(self.req_state == 0).reshape(-1)[:need_size]
        self.req_state[select_index] = 1
        self.can_use_req_size -= len(select_index)
        return select_index

    def free(self, free_req_index, free_token_index):
        self.can_use_req_size += len(free_req_index)
        self.req_state[free_req_index] = 0
        if free_token_index is not None:
            self.mem_manager.free(free_token_index)

    def free_req(self, free_req_index):
        self.can_use_req_size += 1
        self.req_state[free_req_index] = 0

    def free_token(self, free_token_index):
        self.mem_manager.free(free_token_index)

    def free_all(self):
        self.can_use_req_size = len(self.req_state)
        self.req_state[:] = 0
