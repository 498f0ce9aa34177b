"""Failure detection without faulting a GPU: host-side argument and capacity errors, a ring rank that never
sends (gloo, CPU, host-side timeout), and -- on a GPU -- a device-side wait that runs out and reports a status
while the context stays usable."""
import os
import socket
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def test_pool_exhaustion_and_bad_shapes_raise_instead_of_aborting():
    from loongserve_b200.mem_manager import LongServeMemoryManager
    mm = LongServeMemoryManager(16, torch.float16, 1, 8, 1, device="cpu")
    mm.alloc(10)
    with pytest.raises(RuntimeError, match="not enough KV cache"):
        mm.alloc(7)
    assert mm.alloc_contiguous(7) is None and mm.can_use_mem_size == 6
    from loongserve_b200 import _lib
    lib = _lib.attn()
    # head_dim the kernels do not support, misaligned strides, negative sizes: status codes, no launch
    assert lib.esp_decode_stage1(1, 1, 16, 16, 16, 8, 8, 8, 8, 16, 8, 16, 16, 1, 4, 4, 64, 10, 16, 1, 0.0, None) == -5
    assert lib.esp_decode_stage1(1, 1, 16, 16, 16, 7, 8, 8, 8, 16, 8, 16, 16, 1, 4, 4, 128, 10, 16, 1, 0.0, None) == -2
    assert lib.esp_kv_scatter(16, 8, 8, 16, 8, 8, 16, 0, -1, 1, 8, 2, None) == -1
    assert lib.esp_rms_norm(16, 16, 16, 4, 12, 1e-5, 1, None) == -2


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _silent_rank_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=3))
    res = "ok"
    if rank == 0:
        buf = torch.zeros(1024)
        try:
            dist.recv(buf, src=1)              # the peer never sends: the process-group timeout ends the wait
        except Exception as e:                  # noqa: BLE001
            res = "timeout:" + type(e).__name__
        open(os.path.join(out, "r0.txt"), "w").write(res)
    else:
        import time
        time.sleep(6)                           # stays alive, sends nothing
    try:
        dist.destroy_process_group()
    except Exception:                           # noqa: BLE001
        pass


def test_ring_peer_that_never_sends_times_out_on_the_host(tmp_path):
    mp.spawn(_silent_rank_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert open(os.path.join(str(tmp_path), "r0.txt")).read().startswith("timeout:")


@pytest.mark.gpu
def test_device_side_wait_runs_out_and_reports():
    from loongserve_b200 import _lib
    lib = _lib.attn()
    res = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.esp_selftest_bounded_wait(2_000_000, res.data_ptr(), torch.cuda.current_stream().cuda_stream)   # about a millisecond
    _lib.check(rc, "esp_selftest_bounded_wait")
    torch.cuda.synchronize()
    assert int(res.item()) == 1
    # the context is still usable afterwards
    x = torch.arange(8, device="cuda")
    assert int(x.sum().item()) == 28
    assert lib.esp_selftest_bounded_wait(0, res.data_ptr(), None) == -1
