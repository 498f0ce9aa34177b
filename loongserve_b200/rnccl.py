"""Raw NCCL point-to-point communicator with the reference module's surface
(rnccl/src/main.cpp:276-292): ``get_nccl_unique_id()`` and ``RNCCLComm`` with
``nccl_group_start/end``, ``nccl_send/recv``, ``wait_for_default_stream`` and
``let_default_stream_wait``.  The two fences act on torch's CURRENT stream (the reference fences
against the legacy default stream, which is what torch's current stream is in its workers)."""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib


def get_nccl_unique_id() -> list[int]:
    buf = (C.c_uint8 * 128)()
    _lib.check_rnccl(_lib.rnccl().esp_rnccl_unique_id(buf), "esp_rnccl_unique_id")
    return list(buf)


class RNCCLComm:
    def __init__(self, unique_id, world_size: int, total_rank: int):
        assert 0 <= total_rank < world_size
        assert len(unique_id) == 128
        self.world_size = world_size
        self.total_rank = total_rank
        self._lib = _lib.rnccl()
        buf = (C.c_uint8 * 128)(*[int(x) & 0xFF for x in unique_id])
        handle = C.c_void_p()
        _lib.check_rnccl(self._lib.esp_rnccl_create(buf, world_size, total_rank, C.byref(handle)), "esp_rnccl_create")
        self._h = handle
        self.stream = torch.cuda.ExternalStream(self._lib.esp_rnccl_stream(self._h))

    def close(self):
        if getattr(self, "_h", None):
            self._lib.esp_rnccl_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def nccl_group_start(self):
        _lib.check_rnccl(self._lib.esp_rnccl_group_start(self._h), "nccl_group_start")

    def nccl_group_end(self):
        _lib.check_rnccl(self._lib.esp_rnccl_group_end(self._h), "nccl_group_end")

    def nccl_send(self, data: torch.Tensor, peer: int):
        assert data.is_contiguous() and data.is_cuda
        assert 0 <= peer < self.world_size
        _lib.check_rnccl(self._lib.esp_rnccl_send(self._h, data.data_ptr(), data.numel() * data.element_size(), peer),
                         "nccl_send")

    def nccl_recv(self, data: torch.Tensor, peer: int):
        assert data.is_contiguous() and data.is_cuda
        assert 0 <= peer < self.world_size
        _lib.check_rnccl(self._lib.esp_rnccl_recv(self._h, data.data_ptr(), data.numel() * data.element_size(), peer),
                         "nccl_recv")

    def wait_for_default_stream(self):
        """The communicator's stream waits for everything queued so far on torch's current stream."""
        _lib.check_rnccl(self._lib.esp_rnccl_fence_in(self._h, torch.cuda.current_stream().cuda_stream), "fence_in")

    def let_default_stream_wait(self):
        """torch's current stream waits for everything queued so far on the communicator's stream."""
        _lib.check_rnccl(self._lib.esp_rnccl_fence_out(self._h, torch.cuda.current_stream().cuda_stream), "fence_out")
