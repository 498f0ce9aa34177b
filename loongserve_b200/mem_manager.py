"""Token-indexed KV pool: slot allocator and request table behind the attribute and method names the
reference's callers use (loongserve/common/longserve_mem_manager.py:7-113,
loongserve/common/longserve_req_manager.py:7-48).

Design.  Which slots are free, their reference counts and every allocation decision live on the HOST, in the
native bitmap allocator (``esp_pool_*``, csrc/pool_allocator.cpp): ``alloc`` hands out the lowest free slot ids,
``alloc_contiguous`` the first free run -- the order the reference's device-wide ``nonzero`` scan produces -- in a
few microseconds and without reading the device.  The device tensor ``mem_state`` is a mirror kept for the kernels
that look at reference counts (decode-stage migration); it is brought up to date with asynchronous index updates
queued on the current stream.  Freeing slots named by a DEVICE tensor costs one device-to-host copy of the ids;
callers that keep their ids on the host pay nothing.  The request table works the same way: a host-side set of free
request rows, a device mirror ``req_state``.
"""
from __future__ import annotations

import ctypes as C
import heapq

import torch

INT32_MAX = 2147483647


class HostSlotAllocator:
    """ctypes handle on the native host-side allocator (include/esp_attention.h, esp_pool_*)."""

    def __init__(self, size: int):
        from . import _lib
        self._lib_mod = _lib
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
        start = C.c_int64(-1)
        self._lib_mod.check(self._lib.esp_pool_alloc_contiguous(self._h, int(n), C.byref(start)), "esp_pool_alloc_contiguous")
        return None if start.value < 0 else int(start.value)

    @staticmethod
    def _host_ids(ids: torch.Tensor) -> torch.Tensor:
        # an index update on the device applies once per distinct slot, whatever the multiplicity in `ids`
        return torch.unique(ids.detach().to(torch.int64).cpu().reshape(-1)).contiguous()

    def add_refs(self, ids: torch.Tensor):
        ids = self._host_ids(ids)
        self._lib_mod.check(self._lib.esp_pool_add_refs(self._h, ids.data_ptr(), ids.numel()), "esp_pool_add_refs")

    def decrease_refs(self, ids: torch.Tensor):
        ids = self._host_ids(ids)
        self._lib_mod.check(self._lib.esp_pool_decrease_refs(self._h, ids.data_ptr(), ids.numel()), "esp_pool_decrease_refs")

    def free_all(self):
        self._lib_mod.check(self._lib.esp_pool_free_all(self._h), "esp_pool_free_all")

    def state(self) -> torch.Tensor:
        out = torch.empty((self.size,), dtype=torch.int32)
        self._lib_mod.check(self._lib.esp_pool_state(self._h, out.data_ptr()), "esp_pool_state")
        return out


class LongServeMemoryManager:
    """``kv_buffer [layer, size + num_idle_slots, 2*head_num, head_dim]`` (K = heads [0, head_num), V = heads
    [head_num, 2*head_num) of the same slot row), device reference counts ``mem_state`` (int32), ``indexes`` and
    ``can_use_mem_size`` as the reference's callers read them; decisions by the host-side allocator."""

    def __init__(self, size, dtype, head_num, head_dim, layer_num, num_idle_slots=0, always_copy=False, device="cuda"):
        self.dtype, self.head_num, self.head_dim, self.layer_num = dtype, head_num, head_dim, layer_num
        self.num_idle_slots, self.always_copy = num_idle_slots, always_copy
        self.device = torch.device(device)
        self._build(int(size))

    def _build(self, size: int):
        self.size = size
        self._slots = HostSlotAllocator(size)
        self.mem_state = torch.zeros((size,), dtype=torch.int32, device=self.device)
        self.indexes = torch.arange(0, size, dtype=torch.long, device=self.device)
        self.kv_buffer = torch.empty((self.layer_num, size + self.num_idle_slots, 2 * self.head_num, self.head_dim),
                                     dtype=self.dtype, device=self.device)

    @property
    def can_use_mem_size(self) -> int:
        return self._slots.can_use

    def _mirror(self, ids_host: torch.Tensor) -> torch.Tensor:
        """The ids on the pool's device (pinned staging + asynchronous copy when that is a GPU)."""
        if self.device.type == "cuda":
            return ids_host.pin_memory().to(self.device, non_blocking=True)
        return ids_host

    @torch.inference_mode()
    def alloc(self, need_size):
        ids = self._slots.alloc(int(need_size))        # raises RuntimeError when the pool cannot cover it
        dev_ids = self._mirror(ids)
        self.mem_state[dev_ids] = 1
        return dev_ids

    @torch.inference_mode()
    def alloc_contiguous(self, need_size):
        need_size = int(need_size)
        if self.always_copy or need_size <= 0:
            return None
        start = self._slots.alloc_contiguous(need_size)
        if start is None:
            return None
        end = start + need_size
        self.mem_state[start:end] = 1
        return self.indexes[start:end], start, end

    @torch.inference_mode()
    def free(self, free_index):
        self.decrease_refs(free_index)

    @torch.inference_mode()
    def add_refs(self, token_index: torch.Tensor):
        self._slots.add_refs(token_index)
        self.mem_state[token_index.long()] += 1

    @torch.inference_mode()
    def decrease_refs(self, token_index: torch.Tensor):
        self._slots.decrease_refs(token_index)
        self.mem_state[token_index.long()] -= 1

    def release_on_host(self, token_index: torch.Tensor):
        """Drop one reference of every slot in ``token_index`` in the host allocator only: for slots whose device
        counts a kernel has already lowered (the sender side of decode-stage migration)."""
        self._slots.decrease_refs(token_index)

    @torch.inference_mode()
    def free_all(self):
        self._slots.free_all()
        self.mem_state.zero_()

    @torch.inference_mode()
    def resize_mem(self, new_size):
        self.kv_buffer = None                     # let the old pool go before the new one is allocated
        self._build(int(new_size))


# earlier name of the host-decided manager, kept for callers written against it
SyncFreeMemoryManager = LongServeMemoryManager


class LongServeReqManager:
    """``req_to_token_indexs [max_request_num, max_sequence_length]`` int32 filled with 2147483647, the device mirror
    ``req_state`` and ``can_use_req_size``; free request rows are a host-side min-heap, so ``alloc`` returns the
    lowest free rows (the reference's order) without scanning the device."""

    def __init__(self, max_request_num, max_sequence_length, mem_manager: LongServeMemoryManager):
        dev = mem_manager.device
        self.device = dev
        self.mem_manager = mem_manager
        self.req_state = torch.zeros((max_request_num,), dtype=torch.bool, device=dev)
        self.req_to_token_indexs = torch.full((max_request_num, max_sequence_length), fill_value=INT32_MAX,
                                              dtype=torch.int32, device=dev)
        self._free_rows = list(range(max_request_num))       # a sorted list is a valid heap
        self._taken = set()

    @property
    def can_use_req_size(self) -> int:
        return len(self._free_rows)

    def alloc(self, need_size):
        need_size = int(need_size)
        if need_size > len(self._free_rows):
            return None
        rows = [heapq.heappop(self._free_rows) for _ in range(need_size)]
        self._taken.update(rows)
        select_index = torch.tensor(rows, dtype=torch.long).to(self.device)
        self.req_state[select_index] = True
        return select_index

    def _give_back(self, rows):
        for r in rows:
            r = int(r)
            if r in self._taken:
                self._taken.discard(r)
                heapq.heappush(self._free_rows, r)

    def free(self, free_req_index, free_token_index):
        rows = free_req_index.reshape(-1).tolist() if torch.is_tensor(free_req_index) else list(free_req_index)
        self._give_back(rows)
        self.req_state[torch.as_tensor(rows, dtype=torch.long, device=self.device)] = False
        if free_token_index is not None:
            self.mem_manager.free(free_token_index)

    def free_req(self, free_req_index):
        self._give_back([int(free_req_index)])
        self.req_state[int(free_req_index)] = False

    def free_token(self, free_token_index):
        self.mem_manager.free(free_token_index)

    def free_all(self):
        self._taken.clear()
        self._free_rows = list(range(self.req_state.shape[0]))
        self.req_state.zero_()
