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


class HostSlotAllocator:
    """ctypes handle on the native host-side allocator (include/esp_attention.h, esp_pool_*): same allocation order
    and reference-count semantics as ``LongServeMemoryManager``, no device work."""

    def __init__(self, size: int):
        import ctypes as C
        from . import _lib
        self._C, self._lib_mod = C, _lib
        self._lib = _lib.attn()
        self.size = int(size)
        h = C.c_void_p()
        _lib.check(self._lib.esp_pool_create(self.size, C.byref(h)), "esp_pool_create")
        self._h = h

    def __del__(self):
        try:
            if getattr(self, "_h", None):
                self._lib.esp_pool_destroy(self._h)
                self._h = None
        except Exception:
            pass

    @property
    def can_use(self) -> int:
        return int(self._lib.esp_pool_can_use(self._h))

    def alloc(self, n: int) -> torch.Tensor:
        out = torch.empty((int(n),), dtype=torch.int64)
        rc = self._lib.esp_pool_alloc(self._h, int(n), out.data_ptr())
        if rc == -7:
            raise RuntimeError(f"not enough KV cache: need_size {n} left_size {self.can_use}")
        self._lib_mod.check(rc, "esp_pool_alloc")
        return out

    def alloc_contiguous(self, n: int):
        start = self._C.c_int64(-1)
        self._lib_mod.check(self._lib.esp_pool_alloc_contiguous(self._h, int(n), self._C.byref(start)), "esp_pool_alloc_contiguous")
        return None if start.value < 0 else int(start.value)

    def add_refs(self, ids: torch.Tensor):
        ids = ids.to(torch.int64).cpu().contiguous()
        self._lib_mod.check(self._lib.esp_pool_add_refs(self._h, ids.data_ptr(), ids.numel()), "esp_pool_add_refs")

    def decrease_refs(self, ids: torch.Tensor):
        ids = ids.to(torch.int64).cpu().contiguous()
        self._lib_mod.check(self._lib.esp_pool_decrease_refs(self._h, ids.data_ptr(), ids.numel()), "esp_pool_decrease_refs")

    def free_all(self):
        self._lib_mod.check(self._lib.esp_pool_free_all(self._h), "esp_pool_free_all")

    def state(self) -> torch.Tensor:
        out = torch.empty((self.size,), dtype=torch.int32)
        self._lib_mod.check(self._lib.esp_pool_state(self._h, out.data_ptr()), "esp_pool_state")
        return out


class SyncFreeMemoryManager(LongServeMemoryManager):
    """``LongServeMemoryManager`` whose allocation decisions are taken by the host-side allocator: ``alloc`` and
    ``alloc_contiguous`` return the same slot ids in the same order as the reference, but never read the device
    (the reference runs ``nonzero`` over the whole state and ``.item()`` on every call).  The device copy of
    ``mem_state`` is kept up to date with asynchronous updates for the kernels that touch it.  Callers that free
    slots pass host-resident (or host-copyable) index tensors."""

    def __init__(self, size, dtype, head_num, head_dim, layer_num, num_idle_slots=0, always_copy=False, device="cuda"):
        super().__init__(size, dtype, head_num, head_dim, layer_num, num_idle_slots, always_copy, device)
        self._host = HostSlotAllocator(size)

    def _to_device(self, ids_host: torch.Tensor) -> torch.Tensor:
        if self.device.type == "cuda":
            return ids_host.pin_memory().to(self.device, non_blocking=True)
        return ids_host

    @torch.inference_mode()
    def alloc(self, need_size):
        ids = self._host.alloc(int(need_size))
        self.can_use_mem_size = self._host.can_use
        dev_ids = self._to_device(ids)
        self.mem_state[dev_ids] += 1
        return dev_ids

    @torch.inference_mode()
    def alloc_contiguous(self, need_size):
        need_size = int(need_size)
        if self.always_copy or need_size <= 0:
            return None
        start = self._host.alloc_contiguous(need_size)
        if start is None:
            return None
        self.can_use_mem_size = self._host.can_use
        end = start + need_size
        self.mem_state[start:end] += 1
        return self.indexes[start:end], start, end

    @torch.inference_mode()
    def add_refs(self, token_index: torch.Tensor):
        self._host.add_refs(token_index)
        self.can_use_mem_size = self._host.can_use
        self.mem_state[token_index] += 1

    @torch.inference_mode()
    def decrease_refs(self, token_index: torch.Tensor):
        self._host.decrease_refs(token_index)
        self.can_use_mem_size = self._host.can_use
        self.mem_state[token_index] -= 1

    @torch.inference_mode()
    def free_all(self):
        self._host.free_all()
        super().free_all()
