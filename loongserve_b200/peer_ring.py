"""Ring exchange of KV blocks with copy-engine transfers into peer memory.

The reference rotates the KV block of every ring step with a grouped ncclSend / ncclRecv pair
(loongserve/models/llama/layer_infer/longserve_transformer_layer_infer.py:162-178); NCCL moves the bytes with SM
kernels, which take SMs (and shared memory) away from an attention kernel that wants one CTA on every SM.  Here the
sender copies its current block straight into the receiver's buffer with one ``cudaMemcpyAsync`` on a copy stream
(a DMA transfer over NVLink, no SM involved) and the two sides synchronise with two int32 counters per directed
pair, written with system-scope release stores by one-thread kernels and awaited by bounded one-thread kernels:

  arrived[s]  in the RECEIVER's region: number of blocks sender s has finished copying into the receiver's buffers;
  credit[r]   in the SENDER's region:   number of blocks receiver r has made room for.

A pass over a ring of P instances makes P-1 transfers per instance; transfer j goes into the receiver's buffer
j mod 2.  The receiver grants min(2, P-1) credits when the pass starts (both buffers are free then) and one more each
time it is done with a buffer that a later transfer of the pass will reuse -- done meaning attended to AND copied on
to the next instance.  Counters only grow, so nothing is reset between passes, layers or batches; the instances of
a ring must make the same passes in the same order (as with NCCL).

Every wait is bounded (``esp_flag_wait``); when one runs out the device status word says which, later signals are
withheld and ``check()`` raises.
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, List, Optional

import torch

from . import _lib

WAIT_CREDIT, WAIT_ARRIVAL = 16, 17          # wait ids reported in the device status word
_PATIENCE = 30                              # ring waits may last this many wait limits (ranks start passes at different times)


class _RawDeviceMemory:
    """Lets torch alias device memory it did not allocate."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class _CudaBackend:
    """Queues the exchange's operations on CUDA streams through the C ABI."""

    def __init__(self, device):
        self.lib = _lib.attn()
        self.device = device

    def flag_wait(self, stream, flag_addr: int, value: int, wait_id: int):
        _lib.check(self.lib.esp_flag_wait(flag_addr, value, None, wait_id, _PATIENCE, stream.cuda_stream), "esp_flag_wait")

    def signal(self, stream, flag_addr: int, value: int):
        _lib.check(self.lib.esp_peer_signal(flag_addr, value, None, stream.cuda_stream), "esp_peer_signal")

    def copy(self, stream, dst_addr: int, src_addr: int, nbytes: int):
        _lib.check(self.lib.esp_memcpy_async(dst_addr, src_addr, nbytes, stream.cuda_stream), "esp_memcpy_async")

    def copy2d(self, stream, dst_addr: int, dpitch: int, src_addr: int, spitch: int, width: int, rows: int):
        if dpitch == width and spitch == width:
            self.copy(stream, dst_addr, src_addr, width * rows)
        else:
            _lib.check(self.lib.esp_memcpy_2d(dst_addr, dpitch, src_addr, spitch, width, rows, 2, stream.cuda_stream), "esp_memcpy_2d")

    def record(self, stream):
        ev = torch.cuda.Event()
        ev.record(stream)
        return ev

    def wait(self, stream, ev):
        stream.wait_event(ev)

    def compute_stream(self):
        return torch.cuda.current_stream(self.device)


class CopyEngineRing:
    """One instance's end of the exchange.  ``all_gather_bytes(b)`` returns every rank's bytes in rank order; it is used
    once, to hand round the 64-byte buffer handles.  ``block_bytes`` is the largest KV block that will travel."""

    def __init__(self, rank: int, world: int, block_bytes: int, all_gather_bytes: Optional[Callable[[bytes], List[bytes]]],
                 device="cuda", backend=None, peer_bases: Optional[List[int]] = None, raw_buffers=None):
        assert 0 <= rank < world
        self.rank, self.world = rank, world
        self.block_bytes = (int(block_bytes) + 255) // 256 * 256
        self.off_flags = 2 * self.block_bytes
        self.total = self.off_flags + 256 * 2                      # arrived[world] then credit[world], 256 B each
        assert world <= 64
        self.device = torch.device(device)
        self.sent = [0] * world
        self.received = [0] * world
        self.granted = [0] * world
        self._pass = None
        self._last_copy_ev = None
        if backend is not None:
            # host-side tests: an injected backend that interprets the queued operations, regions in host memory
            self.backend, self.peer_base, self.base = backend, list(peer_bases), peer_bases[rank]
            self.copy_stream, self._lib, self._raw = "copy", None, list(raw_buffers)
            return
        self._lib = _lib.attn()
        self.backend = _CudaBackend(self.device)
        base = C.c_void_p()
        handle = (C.c_uint8 * 64)()
        _lib.check(self._lib.esp_peer_buffer_create(self.total, C.byref(base), handle), "esp_peer_buffer_create")
        self.base = base.value
        handles = all_gather_bytes(bytes(handle))
        self.peer_base = [None] * world
        for r in range(world):
            if r == rank:
                self.peer_base[r] = self.base
            else:
                p = C.c_void_p()
                _lib.check(self._lib.esp_peer_buffer_open((C.c_uint8 * 64)(*handles[r]), C.byref(p)), "esp_peer_buffer_open")
                self.peer_base[r] = p.value
        # transfers are issued ahead of the attention kernels that overlap them: highest priority
        self.copy_stream = torch.cuda.Stream(device=self.device, priority=-1)
        self._raw = [torch.as_tensor(_RawDeviceMemory(self.base + i * self.block_bytes, self.block_bytes), device=self.device)
                     for i in range(2)]

    def close(self):
        if self._lib is None or self.base is None:
            return
        torch.cuda.synchronize(self.device)
        self._raw = []
        for r, p in enumerate(self.peer_base):
            if p is not None and r != self.rank:
                self._lib.esp_peer_buffer_close(p)
        self._lib.esp_peer_buffer_destroy(self.base)
        self.base = None

    # ---------------------------------------------------------------------------------------------- buffers
    def receive_buffers(self, like: torch.Tensor) -> List[torch.Tensor]:
        """The two receive buffers viewed with ``like``'s shape and dtype (a KV block ``[tokens, 2*Hkv, D]``)."""
        n = like.numel() * like.element_size()
        assert like.is_contiguous() and n <= self.block_bytes, "KV block larger than the exchange was sized for"
        return [r[:n].view(like.dtype).view(like.shape) for r in self._raw]

    def _arrived_flag(self, owner: int, sender: int) -> int:
        return self.peer_base[owner] + self.off_flags + 4 * sender

    def _credit_flag(self, owner: int, receiver: int) -> int:
        return self.peer_base[owner] + self.off_flags + 256 + 4 * receiver

    # ---------------------------------------------------------------------------------------------- one pass
    def begin_pass(self, nxt: int, prv: int, transfers: int):
        """Start a pass that sends ``transfers`` blocks to ``nxt`` and receives as many from ``prv``."""
        assert self._pass is None, "the previous pass was not finished"
        be, S = self.backend, self.backend.compute_stream()
        self._pass = dict(nxt=nxt, prv=prv, n=transfers, fwd=[None] * transfers)
        if transfers <= 0:
            return
        if self._last_copy_ev is not None:          # the previous pass's last copy may still read a receive buffer
            be.wait(S, self._last_copy_ev)
        first = min(2, transfers)
        self.granted[prv] += first
        be.signal(S, self._credit_flag(prv, self.rank), self.granted[prv])

    def forward(self, j: int, src_addr: int, nbytes: int):
        """Transfer j of the pass: copy the block this instance attends to at step j on to the next instance.  Call
        it on the host BEFORE launching the attention over that block, so that the copy overlaps the kernel."""
        ps, be = self._pass, self.backend
        assert 0 <= j < ps["n"] and nbytes <= self.block_bytes
        S, Cs, nxt = be.compute_stream(), self.copy_stream, ps["nxt"]
        be.wait(Cs, be.record(S))                   # the block is complete (written, or arrived: S has waited for it)
        self.sent[nxt] += 1
        be.flag_wait(Cs, self._credit_flag(self.rank, nxt), self.sent[nxt], WAIT_CREDIT)
        be.copy(Cs, self.peer_base[nxt] + (j % 2) * self.block_bytes, src_addr, nbytes)
        be.signal(Cs, self._arrived_flag(nxt, self.rank), self.sent[nxt])
        ps["fwd"][j] = be.record(Cs)
        self._last_copy_ev = ps["fwd"][j]

    def wait_arrival(self, j: int) -> int:
        """The compute stream waits until transfer j has arrived; returns the index (0/1) of the buffer it is in."""
        ps, be = self._pass, self.backend
        prv = ps["prv"]
        self.received[prv] += 1
        be.flag_wait(be.compute_stream(), self._arrived_flag(self.rank, prv), self.received[prv], WAIT_ARRIVAL)
        return j % 2

    def release(self, j: int):
        """The block of transfer j has been attended to (kernel queued on the compute stream) and, unless it was the last
        one, forwarded (copy queued): when a later transfer of this pass reuses its buffer, give the sender a credit."""
        ps, be = self._pass, self.backend
        if j + 2 >= ps["n"]:
            return
        S, prv = be.compute_stream(), ps["prv"]
        be.wait(S, ps["fwd"][j + 1])                # the copy that reads this buffer has finished
        self.granted[prv] += 1
        be.signal(S, self._credit_flag(prv, self.rank), self.granted[prv])

    def end_pass(self):
        """Later work on the compute stream sees every copy of this pass finished (the local block may be overwritten)."""
        ps, be = self._pass, self.backend
        if ps["n"] > 0 and ps["fwd"][-1] is not None:
            be.wait(be.compute_stream(), ps["fwd"][-1])
        self._pass = None

    def check(self):
        """Raise if a wait of the exchange ran out on this device (synchronises the device)."""
        buf = (C.c_int32 * 4)()
        _lib.check(self._lib.esp_decode_device_status(buf, 0), "esp_decode_device_status")
        if buf[0] != 0:
            raise RuntimeError(f"ring exchange: device status {tuple(buf)} (code, block, wait id, awaited value)")


WAIT_GATHER_CREDIT, WAIT_GATHER_ARRIVAL = 18, 19


class CopyEngineGather:
    """The other way to feed a striped ring pass on parts with memory to spare: instead of passing blocks round the ring
    while P launches attend to them one by one, every instance copies its block into EVERY other instance's gather buffer
    (one strided copy-engine transfer per request and peer, all peers at once over NVSwitch) while the attention over the
    local block runs, and ONE more launch attends to everything gathered (``ring.gathered_context_attention``).  Rows are
    interleaved in position order -- token n of the i-th other instance lands in row n*(P-1)+i of its request -- so that the
    gathered buffer reads like one block whose keys advance by one position per row.

    Flags as in ``CopyEngineRing``: ``arrived[s]`` in the receiver's region counts the position ranges (``parts`` per pass)
    sender s has delivered, ``credit[r]`` in the sender's region the passes for which receiver r's buffer is free again.
    Every wait is bounded; ``check()`` reports an expired one."""

    def __init__(self, rank: int, world: int, gathered_bytes: int, all_gather_bytes: Optional[Callable[[bytes], List[bytes]]],
                 device="cuda", backend=None, peer_bases: Optional[List[int]] = None, raw_buffer=None, parts: int = 1):
        assert 0 <= rank < world <= 64 and parts >= 1
        self.rank, self.world, self.parts = rank, world, parts
        self.gathered_bytes = (int(gathered_bytes) + 255) // 256 * 256
        self.off_flags = self.gathered_bytes
        self.total = self.off_flags + 256 * 2
        self.device = torch.device(device)
        self.passes = 0
        self._events = []
        self._began = False
        if backend is not None:
            self.backend, self.peer_base, self.base = backend, list(peer_bases), peer_bases[rank]
            self._lib, self._raw = None, raw_buffer
            self.streams = {p: f"copy{p}" for p in range(world) if p != rank}
            return
        self._lib = _lib.attn()
        self.backend = _CudaBackend(self.device)
        base = C.c_void_p()
        handle = (C.c_uint8 * 64)()
        _lib.check(self._lib.esp_peer_buffer_create(self.total, C.byref(base), handle), "esp_peer_buffer_create")
        self.base = base.value
        handles = all_gather_bytes(bytes(handle))
        self.peer_base = [None] * world
        for r in range(world):
            if r == rank:
                self.peer_base[r] = self.base
            else:
                p = C.c_void_p()
                _lib.check(self._lib.esp_peer_buffer_open((C.c_uint8 * 64)(*handles[r]), C.byref(p)), "esp_peer_buffer_open")
                self.peer_base[r] = p.value
        self.streams = {p: torch.cuda.Stream(device=self.device, priority=-1) for p in range(world) if p != rank}
        self._raw = torch.as_tensor(_RawDeviceMemory(self.base, self.gathered_bytes), device=self.device)

    def close(self):
        if self._lib is None or self.base is None:
            return
        torch.cuda.synchronize(self.device)
        self._raw = None
        for r, p in enumerate(self.peer_base):
            if p is not None and r != self.rank:
                self._lib.esp_peer_buffer_close(p)
        self._lib.esp_peer_buffer_destroy(self.base)
        self.base = None

    def gathered(self, rows: int, like: torch.Tensor) -> torch.Tensor:
        """The gather buffer viewed as ``[rows, *like.shape[1:]]`` of ``like``'s dtype."""
        row_bytes = like[0].numel() * like.element_size()
        assert rows * row_bytes <= self.gathered_bytes, "gather buffer smaller than the pass needs"
        return self._raw[:rows * row_bytes].view(like.dtype).view(rows, *like.shape[1:])

    def _arrived_flag(self, owner: int, sender: int) -> int:
        return self.peer_base[owner] + self.off_flags + 4 * sender

    def _credit_flag(self, owner: int, receiver: int) -> int:
        return self.peer_base[owner] + self.off_flags + 256 + 4 * receiver

    def begin_pass(self):
        """This instance's gather buffer is free (stream order: the launch that read it last is queued before this call):
        tell every sender."""
        assert not self._began, "the previous pass was not finished"
        be, S = self.backend, self.backend.compute_stream()
        self.passes += 1
        self._began, self._events = True, []
        for p in self.streams:
            be.signal(S, self._credit_flag(p, self.rank), self.passes)

    def push(self, peer: int, copies_per_part):
        """Deliver this instance's block to ``peer``: for every position range, in order, a list of ``(dst_offset_bytes,
        dst_pitch, src_address, src_pitch, width_bytes, rows)`` strided copies into the peer's gather buffer, announced when
        they are done.  The local block must be complete on the compute stream when this is called."""
        assert len(copies_per_part) == self.parts
        be, Cs = self.backend, self.streams[peer]
        be.wait(Cs, be.record(be.compute_stream()))
        be.flag_wait(Cs, self._credit_flag(self.rank, peer), self.passes, WAIT_GATHER_CREDIT)
        for k, copies in enumerate(copies_per_part):
            for dst_off, dpitch, src, spitch, width, rows in copies:
                assert rows > 0 and dst_off + (rows - 1) * dpitch + width <= self.gathered_bytes
                be.copy2d(Cs, self.peer_base[peer] + dst_off, dpitch, src, spitch, width, rows)
            be.signal(Cs, self._arrived_flag(peer, self.rank), (self.passes - 1) * self.parts + k + 1)
        self._events.append(be.record(Cs))

    def wait_part(self, k: int):
        """The compute stream waits until position range k of this pass has arrived from every other instance."""
        assert 0 <= k < self.parts
        be, S = self.backend, self.backend.compute_stream()
        for p in self.streams:
            be.flag_wait(S, self._arrived_flag(self.rank, p), (self.passes - 1) * self.parts + k + 1, WAIT_GATHER_ARRIVAL)

    def end_pass(self):
        """Later work on the compute stream sees this instance's own copies finished (the local block may be overwritten)."""
        be, S = self.backend, self.backend.compute_stream()
        for ev in self._events:
            be.wait(S, ev)
        self._began = False

    def check(self):
        buf = (C.c_int32 * 4)()
        _lib.check(self._lib.esp_decode_device_status(buf, 0), "esp_decode_device_status")
        if buf[0] != 0:
            raise RuntimeError(f"gather exchange: device status {tuple(buf)} (code, block, wait id, awaited value)")
