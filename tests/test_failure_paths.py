"""Failure detection without faulting a GPU: host-side argument and capacity errors, a ring rank that never
sends (the product's ring loop over gloo on CPU, host-side timeout), and -- on a GPU -- device-side waits that run out by
design and report a status while the context stays usable, and slot ids outside the pool that are skipped and reported."""
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
    assert lib.esp_decode_stage1(1, 1, 16, 16, 16, 8, 8, 8, 8, 16, 8, 16, 16, 1, 4, 4, 64, 10, 16, 1, 0.0, 0, None) == -5
    assert lib.esp_decode_stage1(1, 1, 16, 16, 16, 7, 8, 8, 8, 16, 8, 16, 16, 1, 4, 4, 128, 10, 16, 1, 0.0, 0, None) == -2
    assert lib.esp_kv_scatter(16, 8, 8, 16, 8, 8, 16, 0, -1, 1, 8, 2, 0, None) == -1
    assert lib.esp_rms_norm(16, 16, 16, 4, 12, 1e-5, 1, None) == -2


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


class _GlooComm:
    """RNCCLComm's surface over gloo; ``drop_sends`` makes this rank's sends vanish (a peer that went silent)."""

    def __init__(self, drop_sends=False):
        self.ops, self.drop = [], drop_sends

    def nccl_group_start(self):
        self.ops = []

    def nccl_send(self, t, peer):
        if t.numel() and not self.drop:
            self.ops.append(dist.P2POp(dist.isend, t.contiguous(), peer))

    def nccl_recv(self, t, peer):
        if t.numel():
            self.ops.append(dist.P2POp(dist.irecv, t, peer))

    def nccl_group_end(self):
        if self.ops:
            for w in dist.batch_isend_irecv(self.ops):
                w.wait()
        self.ops = []

    def wait_for_default_stream(self):
        pass

    def let_default_stream_wait(self):
        pass


def _silent_rank_worker(rank, world, port, out):
    """Both ranks run the product's ring loop; rank 1 never sends its KV block on."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=3))
    from loongserve_b200 import ring
    from oracle import esp_oracle as O
    T, Hh, D = 64, 2, 128
    g = torch.Generator().manual_seed(rank)
    q = torch.randn(T, Hh, D, generator=g); kv = torch.randn(T, 2 * Hh, D, generator=g)
    local_len, first, stride = ring.shard_lengths([T * world], world, True)
    metas = [ring.BlockMeta.from_lengths(local_len[r], first[r], "cpu") for r in range(world)]
    o = torch.empty_like(q); m = torch.empty(T, Hh); l = torch.empty(T, Hh)

    def init_fn(o_, m_, l_):
        o_.zero_(); m_.fill_(float("-inf")); l_.zero_()

    def attn(q_, k_, v_, o_, qs_, ql_, qf_, ks_, kl_, kf_, s_, mx_, m_, l_):
        O.ring_step(q_, k_, v_, o_, m_, l_, qs_, ql_, qf_, ks_, kl_, kf_, s_)

    res = "ok"
    try:
        ring.ring_context_attention(q, kv, o, m, l, rank=rank, peers=list(range(world)), metas=metas, stride=stride,
                                    max_len_in_batch=T, num_kv_heads=Hh, comm=_GlooComm(drop_sends=(rank == 1)),
                                    recv_buffers=[torch.empty_like(kv), torch.empty_like(kv)], attention_fn=attn,
                                    init_fn=init_fn)
    except Exception as e:                      # noqa: BLE001
        res = "timeout:" + type(e).__name__
    open(os.path.join(out, f"r{rank}.txt"), "w").write(res)
    if rank == 1:
        import time
        time.sleep(5)                           # stays alive while rank 0's wait runs out
    try:
        dist.destroy_process_group()
    except Exception:                           # noqa: BLE001
        pass


def test_ring_peer_that_never_sends_times_out_on_the_host(tmp_path):
    mp.spawn(_silent_rank_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert open(os.path.join(str(tmp_path), "r0.txt")).read().startswith("timeout:")
    assert open(os.path.join(str(tmp_path), "r1.txt")).read() == "ok"      # the silent rank itself got its block


@pytest.mark.gpu
def test_device_side_wait_runs_out_and_reports(selftest_lib):
    """The bounded mbarrier wait every wait of the prefill kernel goes through, on a barrier nothing completes."""
    lib = selftest_lib
    res = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.esp_selftest_bounded_wait(2_000_000, res.data_ptr(), torch.cuda.current_stream().cuda_stream)   # about a millisecond
    assert rc == 0
    torch.cuda.synchronize()
    assert int(res.item()) == 1
    # the context is still usable afterwards
    x = torch.arange(8, device="cuda")
    assert int(x.sum().item()) == 28
    assert lib.esp_selftest_bounded_wait(0, res.data_ptr(), None) == -1


def _tiny_decode_inputs(dev="cuda"):
    g = torch.Generator().manual_seed(5)
    B, Hq, Hkv, D, pool = 2, 4, 2, 128, 96
    lens = [40, 17]
    kv = torch.randn(pool, 2 * Hkv, D, generator=g).to(torch.bfloat16).to(dev)
    q = torch.randn(B, Hq, D, generator=g).to(torch.bfloat16).to(dev)
    rt = torch.full((B, 64), 2147483647, dtype=torch.int32)
    perm = torch.randperm(pool, generator=g).to(torch.int32)
    rt[0, :40] = perm[:40]; rt[1, :17] = perm[40:57]
    return B, Hq, Hkv, D, lens, kv, q, rt.to(dev), torch.arange(B, dtype=torch.int32, device=dev), torch.tensor(lens, dtype=torch.int32, device=dev)


@pytest.mark.gpu
def test_gated_decode_kernels_give_up_on_a_flag_nobody_raises():
    """The product's own gated stage-1 and merge kernels with a flag that stays 0 and a limit of about a millisecond:
    they return, the status names the wait, later gated kernels drain at once, clearing the status restores normal
    calls, and the context stays usable.  Nothing faults or hangs: the wait is bounded by design."""
    import ctypes as C
    from loongserve_b200 import _lib
    from loongserve_b200 import flash_decoding as fd
    from loongserve_b200._util import dtype_tag, ptr
    lib = _lib.attn()
    B, Hq, Hkv, D, lens, kv, q, rt, b_req, b_len = _tiny_decode_inputs()
    k, v = kv[:, :Hkv], kv[:, Hkv:]
    bs, mx = 32, max(lens)
    nblk = (mx + bs - 1) // bs
    mid_o = torch.full((nblk, B, Hq, D), 7.0, device="cuda"); mid_l = torch.full((nblk, B, Hq), 7.0, device="cuda")
    o = torch.full((B, Hq, D), 7.0, device="cuda"); lse = torch.full((B, Hq), 7.0, device="cuda")
    flag = torch.zeros(4, dtype=torch.int32, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    fd.device_status(clear=True)
    fd.set_wait_limit_cycles(2_000_000)
    try:
        def stage1_gated():
            return lib.esp_decode_stage1_gated(ptr(mid_o), ptr(mid_l), ptr(q), ptr(k), ptr(v), k.stride(0), k.stride(1), v.stride(0),
                                               v.stride(1), ptr(rt), rt.stride(0), ptr(b_req), ptr(b_len), B, Hq, Hkv, D, mx, bs,
                                               dtype_tag(q), C.c_float(0.0), kv.shape[0], ptr(flag), 1, None, s)
        assert stage1_gated() == 0
        st = fd.device_status(clear=False)
        assert st[0] == -4 and st[2] == 1 and st[3] == 1, st          # timed out in the stage-1 gate, waiting for value 1
        assert bool((mid_o == 7.0).all())                              # nothing was written behind the failed wait
        # a later gated kernel on the device drains at once, the signal kernel publishes nothing
        t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        rc = lib.esp_decode_merge_gated(ptr(o), ptr(lse), ptr(b_len), ptr(mid_o), ptr(mid_l), B, Hq, D, nblk, bs, _lib.ESP_DTYPE_F32,
                                        ptr(flag), 1, 1, None, s)
        assert rc == 0
        assert lib.esp_peer_signal(flag.data_ptr() + 8, 5, None, s) == 0
        t1.record(); torch.cuda.synchronize()
        assert t0.elapsed_time(t1) < 0.5 and bool((o == 7.0).all()) and int(flag[2]) == 0
        # cleared: the merge gate itself now runs out (wait id 2), then the flag is raised and everything works
        fd.device_status(clear=True)
        assert lib.esp_decode_merge_gated(ptr(o), ptr(lse), ptr(b_len), ptr(mid_o), ptr(mid_l), B, Hq, D, nblk, bs, _lib.ESP_DTYPE_F32,
                                          ptr(flag), 1, 1, None, s) == 0
        st = fd.device_status(clear=True)
        assert st[0] == -4 and st[2] == 2, st
        flag.fill_(1)
        assert stage1_gated() == 0
        assert lib.esp_decode_merge_gated(ptr(o), ptr(lse), ptr(b_len), ptr(mid_o), ptr(mid_l), B, Hq, D, nblk, bs, _lib.ESP_DTYPE_F32,
                                          ptr(flag), 1, 1, None, s) == 0
        assert fd.device_status(clear=True)[0] == 0
    finally:
        fd.set_wait_limit_cycles(2_000_000_000)
    from oracle import esp_oracle as O
    ro, rl = O.token_decode_attention(q.cpu(), k.cpu(), v.cpu(), rt.cpu(), b_req.cpu(), b_len.cpu())
    assert torch.allclose(o.cpu(), ro, atol=2e-2, rtol=1e-2) and torch.allclose(lse.cpu(), rl, atol=1e-3, rtol=1e-3)


@pytest.mark.gpu
def test_slot_ids_outside_the_pool_are_skipped_and_reported():
    """The request table's filler value (2147483647) inside a request's range, and a scatter destination beyond the
    pool: neither is dereferenced; the row / token is skipped and the status words name the id."""
    from loongserve_b200 import flash_decoding as fd
    from loongserve_b200 import kv_ops
    from oracle import esp_oracle as O
    B, Hq, Hkv, D, lens, kv, q, rt, b_req, b_len = _tiny_decode_inputs()
    k, v = kv[:, :Hkv], kv[:, Hkv:]
    bs, mx = 32, max(lens)
    nblk = (mx + bs - 1) // bs
    fd.device_status(clear=True)
    rt_bad = rt.clone()
    rt_bad[0, 5] = 2147483647
    rt_bad[1, 16] = -3
    mid_o = torch.empty(nblk, B, Hq, D, device="cuda"); mid_l = torch.empty(nblk, B, Hq, device="cuda")
    o = torch.empty(B, Hq, D, device="cuda"); lse = torch.empty(B, Hq, device="cuda")
    fd.flash_decoding_stage1(mid_o, mid_l, q, k, v, rt_bad, b_req, b_len, mx, bs)
    fd.flash_decoding_stage2(o, lse, b_len, mid_o, mid_l, bs)
    st = fd.device_status(clear=True)
    assert st[0] == -8 and st[3] in (2147483647, -3), st
    # the answer is the attention over the remaining tokens
    keep0 = [i for i in range(40) if i != 5]
    rt_ref = torch.full_like(rt, 2147483647).cpu()
    rt_ref[0, :39] = rt[0, keep0].cpu(); rt_ref[1, :16] = rt[1, :16].cpu()
    ro, rl = O.token_decode_attention(q.cpu(), k.cpu(), v.cpu(), rt_ref, b_req.cpu(), torch.tensor([39, 16], dtype=torch.int32))
    assert torch.allclose(o.cpu(), ro, atol=2e-2, rtol=1e-2) and torch.allclose(lse.cpu(), rl, atol=1e-3, rtol=1e-3)
    # scatter: rows 1 and 3 name slots outside the 8-row pool
    kv_ops.device_status(clear=True)
    src = torch.arange(5 * 2 * 8, dtype=torch.float32, device="cuda").to(torch.bfloat16).view(5, 2, 8) + 1
    pool = torch.zeros(8, 2, 8, dtype=torch.bfloat16, device="cuda")
    dest = torch.tensor([6, 2147483647, 0, 8, 3], dtype=torch.int32, device="cuda")
    kv_ops.destindex_copy_kv(src, dest, pool)
    st = kv_ops.device_status(clear=True)
    assert st[0] == -8 and st[1] == 1 and (st[2], st[3]) in ((1, 2147483647), (3, 8)), st
    want = torch.zeros_like(pool); want[6] = src[0]; want[0] = src[2]; want[3] = src[4]
    assert torch.equal(pool.view(torch.int16), want.view(torch.int16))
    assert kv_ops.device_status()[0] == 0
