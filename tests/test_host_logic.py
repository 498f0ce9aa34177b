"""Host-side logic on CPU: the pool managers against the reference-generated golden trace, and the ring /
multi-master orchestration run as world_size-2 gloo processes with the CPU oracle standing in for the
kernels (the correctness configuration that needs no GPU: one 4096-token sequence, 2 contiguous shards of 2048,
32 q/kv heads x 128, fp32, seed 0)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import esp_oracle as O


def test_mem_manager_matches_reference_trace(golden_dir):
    from loongserve_b200.mem_manager import LongServeMemoryManager, LongServeReqManager
    g = np.load(os.path.join(golden_dir, "mem_manager.npz"))
    mm = LongServeMemoryManager(64, torch.float16, 2, 8, 1, device="cpu")
    a = mm.alloc(5)
    assert np.array_equal(a.numpy(), g["t0_alloc5"]) and mm.can_use_mem_size == int(g["t0_free"])
    b = mm.alloc_contiguous(7)
    assert np.array_equal(b[0].numpy(), g["t1_contig7"]) and mm.can_use_mem_size == int(g["t1_free"])
    mm.free(a[1:4])
    assert np.array_equal(mm.mem_state.numpy(), g["t2_free_a1_4"]) and mm.can_use_mem_size == int(g["t2_free"])
    c = mm.alloc(6)
    assert np.array_equal(c.numpy(), g["t3_alloc6"]) and mm.can_use_mem_size == int(g["t3_free"])
    d = mm.alloc_contiguous(4)
    assert np.array_equal(d[0].numpy(), g["t4_contig4"]) and mm.can_use_mem_size == int(g["t4_free"])
    mm.add_refs(c[:2])
    assert np.array_equal(mm.mem_state.numpy(), g["t5_addref"]) and mm.can_use_mem_size == int(g["t5_free"])
    mm.free(c)
    assert np.array_equal(mm.mem_state.numpy(), g["t6_free_c"]) and mm.can_use_mem_size == int(g["t6_free"])
    assert mm.alloc_contiguous(60) is None
    with pytest.raises(RuntimeError):
        mm.alloc(10_000)
    assert mm.kv_buffer.shape == (1, 64, 4, 8)
    rm = LongServeReqManager(4, 16, mm)
    assert int(rm.req_to_token_indexs[0, 0]) == 2147483647
    idx = rm.alloc(3)
    assert idx.tolist() == [0, 1, 2] and rm.can_use_req_size == 1 and rm.alloc(2) is None
    rm.free(idx[:1], None)
    assert rm.alloc(1).tolist() == [0]


class GlooComm:
    """CPU stand-in with RNCCLComm's surface: grouped point-to-point over gloo."""

    def __init__(self):
        self.ops = []

    def nccl_group_start(self):
        self.ops = []

    def nccl_send(self, t, peer):
        if t.numel():
            self.ops.append(dist.P2POp(dist.isend, t.contiguous(), peer))

    def nccl_recv(self, t, peer):
        if t.numel():
            assert t.is_contiguous()
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


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _ring_worker(rank, world, port, striped, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from loongserve_b200 import ring
    torch.manual_seed(0)
    T, Hh, D = 4096, 32, 128
    q = torch.randn(T, Hh, D); k = torch.randn(T, Hh, D); v = torch.randn(T, Hh, D)
    lens = [T]
    local_len, first, stride = ring.shard_lengths(lens, world, striped)
    qs = O.shard_tokens(q, lens, world, striped)[rank]
    kv = torch.cat([O.shard_tokens(k, lens, world, striped)[rank], O.shard_tokens(v, lens, world, striped)[rank]], dim=1)
    metas = [ring.BlockMeta.from_lengths(local_len[r], first[r], "cpu") for r in range(world)]
    o = torch.empty_like(qs); m = torch.empty(qs.shape[0], Hh); l = torch.empty(qs.shape[0], Hh)

    def init_fn(o_, m_, l_):
        o_.zero_(); m_.fill_(float("-inf")); l_.zero_()

    def attn(q_, k_, v_, o_, qs_, ql_, qf_, ks_, kl_, kf_, s_, mx_, m_, l_):
        O.ring_step(q_, k_, v_, o_, m_, l_, qs_, ql_, qf_, ks_, kl_, kf_, s_)

    ring.ring_context_attention(qs, kv, o, m, l, rank=rank, peers=list(range(world)), metas=metas, stride=stride,
                                max_len_in_batch=qs.shape[0], num_kv_heads=Hh, comm=GlooComm(),
                                recv_buffers=[torch.empty_like(kv), torch.empty_like(kv)], attention_fn=attn, init_fn=init_fn)
    torch.save((o, O.lse_from_state(m, l)), os.path.join(out, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("striped", [False, True])
def test_ring_world2_gloo_equals_full_attention(tmp_path, striped):
    world = 2
    mp.spawn(_ring_worker, args=(world, _free_port(), striped, str(tmp_path)), nprocs=world, join=True)
    torch.manual_seed(0)
    T, Hh, D = 4096, 32, 128
    q = torch.randn(T, Hh, D); k = torch.randn(T, Hh, D); v = torch.randn(T, Hh, D)
    ro, rlse = O.full_causal_attention(q, k, v, [T])
    parts = [torch.load(os.path.join(str(tmp_path), f"r{r}.pt")) for r in range(world)]
    o = O.unshard_tokens([p[0] for p in parts], [T], world, striped)
    lse = O.unshard_tokens([p[1] for p in parts], [T], world, striped)
    assert torch.allclose(o, ro, atol=1e-4, rtol=1e-4)
    assert torch.allclose(lse, rlse, atol=1e-4, rtol=1e-5)


def _decode_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from loongserve_b200 import ring
    g = torch.Generator().manual_seed(0)
    B, Hh, D, bs = 4, 8, 128, 64
    lens = [300, 41, 129, 64]
    total = sum(lens)
    kall = torch.randn(total, Hh, D, generator=g); vall = torch.randn(total, Hh, D, generator=g)
    q = torch.randn(B, Hh, D, generator=g)
    # token t of request b lives on instance (t mod world); instance 0 is the only master
    pool = torch.zeros(total, 2 * Hh, D); rt = torch.full((B, 400), O.INT32_MAX, dtype=torch.int32)
    loc_len = []
    off = 0; slot = 0
    for b, L in enumerate(lens):
        mine = list(range(rank, L, world))
        for j, t in enumerate(mine):
            pool[slot, :Hh] = kall[off + t]; pool[slot, Hh:] = vall[off + t]; rt[b, j] = slot; slot += 1
        loc_len.append(len(mine)); off += L
    b_req = torch.arange(B, dtype=torch.int32); b_len = torch.tensor(loc_len, dtype=torch.int32)
    mx = max(loc_len); nblk = (mx + bs - 1) // bs
    master = peer = None
    if rank == 0:
        master = ring.MasterPlan(peers=list(range(world)), b_req_idx=b_req, b_seq_len=b_len, max_len_in_batch=mx, block_seq=bs,
                                 global_mid_o=torch.zeros(world - 1 + nblk, B, Hh, D), global_mid_lse=torch.zeros(world - 1 + nblk, B, Hh),
                                 global_merge_len=(world - 1 + (b_len + bs - 1) // bs).to(torch.int32),
                                 global_out_lse=torch.zeros(B, Hh))
    else:
        peer = ring.PeerPlan(masters=[0], ranges=[(0, B)], peer_query_buffer=torch.zeros(B, Hh, D), peer_b_req_idx=b_req,
                             peer_b_seq_len=b_len, peer_max_len_in_batch=mx, block_seq=bs,
                             peer_mid_o=torch.zeros(nblk, B, Hh, D), peer_mid_lse=torch.zeros(nblk, B, Hh),
                             peer_o=torch.zeros(B, Hh, D), peer_lse=torch.zeros(B, Hh))

    def s1(mid_o, mid_l, q_, k_, v_, rt_, br_, bl_, mx_, bs_):
        O.flash_decoding_stage1(mid_o, mid_l, q_, k_, v_, rt_, br_, bl_, mx_, bs_)

    def s2(o_, lse_, bl_, mid_o, mid_l, bs_):
        O.flash_decoding_stage2(o_, lse_, bl_, mid_o, mid_l, bs_)

    o = ring.multi_master_decode_attention(q if rank == 0 else None, pool, rt, Hh, GlooComm(), rank, master, peer, s1, s2)
    if rank == 0:
        torch.save((o, master.global_out_lse), os.path.join(out, "dec.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_multi_master_decode_world2_gloo(tmp_path):
    world = 2
    mp.spawn(_decode_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    o, lse = torch.load(os.path.join(str(tmp_path), "dec.pt"))
    g = torch.Generator().manual_seed(0)
    B, Hh, D = 4, 8, 128
    lens = [300, 41, 129, 64]; total = sum(lens)
    kall = torch.randn(total, Hh, D, generator=g); vall = torch.randn(total, Hh, D, generator=g)
    q = torch.randn(B, Hh, D, generator=g)
    rt = torch.full((B, 400), O.INT32_MAX, dtype=torch.int32); off = 0
    for b, L in enumerate(lens):
        rt[b, :L] = torch.arange(off, off + L, dtype=torch.int32); off += L
    ro, rl = O.token_decode_attention(q, kall, vall, rt, torch.arange(B, dtype=torch.int32), torch.tensor(lens, dtype=torch.int32))
    assert torch.allclose(o, ro, atol=1e-5, rtol=1e-5) and torch.allclose(lse, rl, atol=1e-5, rtol=1e-5)


def test_host_side_allocator_matches_reference_trace_and_oracle(golden_dir):
    """The native host allocator reproduces the reference-generated golden trace and, over a random sequence of
    operations, the oracle's restatement of the reference allocator, slot for slot."""
    from loongserve_b200.mem_manager import HostSlotAllocator, LongServeMemoryManager
    g = np.load(os.path.join(golden_dir, "mem_manager.npz"))
    mm = LongServeMemoryManager(64, torch.float16, 2, 8, 1, device="cpu")
    a = mm.alloc(5)
    assert np.array_equal(a.numpy(), g["t0_alloc5"]) and mm.can_use_mem_size == int(g["t0_free"])
    b = mm.alloc_contiguous(7)
    assert np.array_equal(b[0].numpy(), g["t1_contig7"]) and mm.can_use_mem_size == int(g["t1_free"])
    mm.free(a[1:4])
    assert np.array_equal(mm.mem_state.numpy(), g["t2_free_a1_4"]) and mm.can_use_mem_size == int(g["t2_free"])
    c = mm.alloc(6)
    assert np.array_equal(c.numpy(), g["t3_alloc6"]) and mm.can_use_mem_size == int(g["t3_free"])
    d = mm.alloc_contiguous(4)
    assert np.array_equal(d[0].numpy(), g["t4_contig4"]) and mm.can_use_mem_size == int(g["t4_free"])
    mm.add_refs(c[:2])
    assert np.array_equal(mm.mem_state.numpy(), g["t5_addref"]) and mm.can_use_mem_size == int(g["t5_free"])
    mm.free(c)
    assert np.array_equal(mm.mem_state.numpy(), g["t6_free_c"]) and mm.can_use_mem_size == int(g["t6_free"])
    assert mm.alloc_contiguous(60) is None
    with pytest.raises(RuntimeError, match="not enough KV cache"):
        mm.alloc(10_000)
    assert np.array_equal(mm._slots.state().numpy(), mm.mem_state.numpy())
    # randomised comparison with the oracle
    rng = np.random.default_rng(0)
    size = 700
    host = HostSlotAllocator(size); ora = O.OracleMemoryManager(size)
    held = []
    for step in range(400):
        op = rng.integers(0, 4)
        if op == 0 and ora.can_use_mem_size > 0:
            n = int(rng.integers(1, min(40, ora.can_use_mem_size) + 1))
            x = host.alloc(n).numpy(); y = ora.alloc(n)
            assert np.array_equal(x, y); held.append(y)
        elif op == 1:
            n = int(rng.integers(1, 60))
            x = host.alloc_contiguous(n); y = ora.alloc_contiguous(n)
            assert (x is None) == (y is None)
            if y is not None:
                assert x == y[1]; held.append(y[0])
        elif op == 2 and held:
            ids = held.pop(int(rng.integers(0, len(held))))
            host.decrease_refs(torch.from_numpy(ids)); ora.decrease_refs(ids)
        elif op == 3 and held:
            ids = held[int(rng.integers(0, len(held)))][:3]
            host.add_refs(torch.from_numpy(ids)); ora.add_refs(ids)
            held.append(ids)
        assert host.can_use == ora.can_use_mem_size
        if step % 50 == 0:
            assert np.array_equal(host.state().numpy(), ora.mem_state)
    assert np.array_equal(host.state().numpy(), ora.mem_state)


def test_pool_manager_duplicates_resize_and_over_release():
    """Ids listed twice count once (an index update on the device applies once per distinct slot); resize_mem starts a
    fresh pool of the new size on the host and on the device alike; releasing a slot that holds no reference is an
    error and changes nothing."""
    from loongserve_b200.mem_manager import LongServeMemoryManager, LongServeReqManager
    mm = LongServeMemoryManager(32, torch.float16, 1, 8, 1, device="cpu")
    a = mm.alloc(4)
    mm.add_refs(torch.tensor([1, 1, 2]))
    assert mm.mem_state[:4].tolist() == [1, 2, 2, 1] and np.array_equal(mm._slots.state().numpy(), mm.mem_state.numpy())
    mm.free(torch.tensor([1, 1, 2], dtype=torch.int32))
    assert mm.mem_state[:4].tolist() == [1, 1, 1, 1] and mm.can_use_mem_size == 28
    with pytest.raises(RuntimeError):
        mm._slots.decrease_refs(torch.tensor([0, 9]))          # slot 9 holds nothing
    assert mm.can_use_mem_size == 28 and mm._slots.state()[0] == 1
    mm.resize_mem(48)
    assert mm.can_use_mem_size == 48 and mm.mem_state.shape[0] == 48 and mm.kv_buffer.shape[1] == 48
    assert mm.alloc(40).tolist() == list(range(40)) and mm.alloc_contiguous(8)[1:] == (40, 48)
    rm = LongServeReqManager(4, 16, mm)
    r = rm.alloc(3)
    assert r.tolist() == [0, 1, 2] and rm.can_use_req_size == 1 and rm.alloc(2) is None
    rm.free_req(1)
    rm.free(torch.tensor([0]), None)
    assert rm.can_use_req_size == 3 and rm.req_state.tolist() == [False, False, True, False]
    assert rm.alloc(2).tolist() == [0, 1]
    rm.free_all()
    assert rm.can_use_req_size == 4 and not rm.req_state.any()


def test_master_and_peers_choose_the_same_decode_exchange():
    """Peer-memory decode is chosen from data every instance of a batch has, so a master and its peers agree: a batch
    over a subset of the instances goes over NCCL on all of them, one over all instances over peer memory on all of them;
    and a peer advances the step counter of a master's group only when it really serves that master."""
    from types import SimpleNamespace as NS
    from loongserve_b200.attention_runtime import ESPAttentionRuntime

    def runtime(rank):
        rt = ESPAttentionRuntime(layers_num=1, q_head_num=2, kv_head_num=2, head_dim=128, max_total_token_num=16, max_req_num=2,
                                 max_seq_length=8, sp_world_size=4, total_rank=rank, dtype=torch.float16, device="cpu")
        rt._fused_groups = {0: NS(B=8), 2: NS(B=8)}
        return rt

    i32 = lambda n: torch.zeros(n, dtype=torch.int32)
    master_plan = NS(peers=[0, 1], b_seq_len=i32(3))
    peer_plan = NS(masters=[0], ranges=[(0, 3)])
    # batch on instances {0, 1} only: master 0 and peer 1 must both fall back to the NCCL exchange
    assert runtime(0)._fused_covers(NS(master_plan=master_plan, peer_plan=None, logical_sp_peer_ranks=[0, 1])) is False
    assert runtime(1)._fused_covers(NS(master_plan=None, peer_plan=peer_plan, logical_sp_peer_ranks=[0, 1])) is False
    # batch on all four instances, masters 0 and 2 both have groups
    full = [0, 1, 2, 3]
    assert runtime(0)._fused_covers(NS(master_plan=NS(peers=full, b_seq_len=i32(3)), peer_plan=NS(masters=[2], ranges=[(0, 1)]), logical_sp_peer_ranks=full))
    assert runtime(3)._fused_covers(NS(master_plan=None, peer_plan=NS(masters=[0, 2], ranges=[(0, 3), (3, 4)]), logical_sp_peer_ranks=full))
    # a master without a group: NCCL everywhere
    assert not runtime(3)._fused_covers(NS(master_plan=None, peer_plan=NS(masters=[0, 1], ranges=[(0, 3), (3, 4)]), logical_sp_peer_ranks=full))
    assert not runtime(1)._fused_covers(NS(master_plan=NS(peers=full, b_seq_len=i32(3)), peer_plan=None, logical_sp_peer_ranks=full))
    # a mini-batch larger than the group was sized for: NCCL on the master and on the peers alike
    assert not runtime(0)._fused_covers(NS(master_plan=NS(peers=full, b_seq_len=i32(9)), peer_plan=None, logical_sp_peer_ranks=full))
    assert not runtime(3)._fused_covers(NS(master_plan=None, peer_plan=NS(masters=[0], ranges=[(0, 9)]), logical_sp_peer_ranks=full))

    # step counters: the peer skips a master whose mini-batch is empty, as that master's own group does not advance either
    class G:
        def __init__(self): self.steps, self.served = 0, 0
        def next_step(self): self.steps += 1
        def peer_serve(self, *a, **k): self.served += 1
    rt = runtime(3)
    rt._fused_groups = {0: G(), 2: G()}
    pp = NS(masters=[0, 2], ranges=[(0, 2), (2, 2)], peer_max_len_in_batch=4, block_seq=4, peer_mid_o=torch.zeros(1, 2, 2, 128),
            peer_mid_lse=torch.zeros(1, 2, 2), peer_b_req_idx=torch.zeros(2, dtype=torch.int32), peer_b_seq_len=torch.ones(2, dtype=torch.int32))
    rt._token_attention_peer_memory(None, NS(master_plan=None, peer_plan=pp), rt.mem_manager.kv_buffer[0], None)
    assert (rt._fused_groups[0].steps, rt._fused_groups[0].served) == (1, 1)
    assert (rt._fused_groups[2].steps, rt._fused_groups[2].served) == (0, 0)


def test_migration_chunker_order_and_bookkeeping():
    """The chunker takes requests from the end of the lists, splits at the buffer size and re-queues the rest, and
    adjusts the local lengths, as the reference's worker shell does (model_rpc.py:178-217)."""
    from loongserve_b200.attention_runtime import ESPAttentionRuntime
    calls = []

    class Fake(ESPAttentionRuntime):
        def __init__(self):
            self.device = torch.device("cpu")

        def decoding_stage_migration(self, is_receiver, b_req_idx, b_migration_len, b_seq_len, peer, migration_len_sum=None,
                                     max_migration_len=None):
            calls.append((b_req_idx.tolist(), b_migration_len.tolist(), b_seq_len.tolist(), migration_len_sum, max_migration_len))

    rt = Fake()
    out = rt.migrate_chunked(False, [7, 3, 5], [10, 25, 4], [100, 200, 50], 1, max_mig_len=16)
    assert calls == [([5, 3], [4, 12], [50, 200], 16, 12), ([3, 7], [13, 3], [188, 100], 16, 13), ([7], [7], [97], 7, 7)]
    assert out == [90, 175, 46]
    calls.clear()
    out = rt.migrate_chunked(True, [1], [5], [9], 0, max_mig_len=100)
    assert calls == [([1], [5], [9], 5, 5)] and out == [14]


@pytest.mark.parametrize("P", [2, 3, 5, 8])
@pytest.mark.parametrize("parts", [1, 2, 3])
def test_gather_plan_layout_is_dense_ordered_and_partitioned(P, parts):
    """The layout of the gather buffer (ring.GatherPlan) and the copies ``gathered_context_attention`` derives from it, on
    integers: every row of every instance's buffer is written exactly once, row m of a request holds the m-th token of the
    other instances in position order, the position ranges partition the rows at whole groups of P-1, and the rows local q
    row r may see (m <= r*(P-1) + rank - 1) are exactly the other instances' tokens at positions up to its own."""
    from loongserve_b200 import ring
    rng = np.random.default_rng(100 * P + parts)
    lens = [int(x) for x in rng.integers(1, 90, size=5)] + [1, P, P + 1]
    local_len, first, stride = ring.shard_lengths(lens, P, True)
    plans = [ring.GatherPlan.build(lens, P, r, "cpu", parts=parts) for r in range(P)]
    for recv in range(P):
        plan = plans[recv]
        buf = np.full(plan.rows, -1, dtype=np.int64)           # global position of the token each row holds
        req = np.full(plan.rows, -1, dtype=np.int64)
        for send in range(P):
            if send == recv:
                continue
            i = send if send < recv else send - 1
            for b, n in enumerate(local_len[send]):
                for k in range(parts):
                    n0, n1 = min(plan.part_groups[b][k], n), min(plan.part_groups[b][k + 1], n)
                    for t in range(n0, n1):
                        row = plan.start_rows[b] + t * (P - 1) + i
                        assert buf[row] == -1, "a row written twice"
                        buf[row] = send + t * P
                        req[row] = b
                        # the copy lands inside the range it is announced with
                        pm = plan.part_metas[k]
                        assert int(pm.start_loc[b]) <= row < int(pm.start_loc[b]) + int(pm.seq_len[b])
        assert (buf >= 0).all(), "a row never written"
        for b, L in enumerate(lens):
            s0, n = plan.start_rows[b], int(plan.meta.seq_len[b])
            want = [p for p in range(L) if p % P != recv]
            assert n == len(want) and list(buf[s0:s0 + n]) == want and (req[s0:s0 + n] == b).all()
            # the ranges partition the request's rows, cut at whole groups
            lo = [int(plan.part_metas[k].first_idx[b]) for k in range(parts)]
            ln = [int(plan.part_metas[k].seq_len[b]) for k in range(parts)]
            assert lo[0] == 0 and all(lo[k] + ln[k] == (lo[k + 1] if k + 1 < parts else n) for k in range(parts))
            assert all(x % (P - 1) == 0 for x in lo)
            # visibility: local q row r (global position recv + r*P) sees exactly the rows up to r*(P-1) + recv - 1
            for r in range(local_len[recv][b]):
                limit = r * (P - 1) + int(plan.q_first[b])
                visible = [m for m in range(n) if m <= limit]
                assert [want[m] for m in visible] == [p for p in want if p <= recv + r * P]


def test_prefill_tile_arithmetic_covers_exactly_the_visible_keys():
    """The tile bookkeeping of the prefill kernels (csrc/prefill_attention.cu: vis_a, vis_c, n_tiles, masked, limit; for CTA
    pairs the tile count of a slot is that of the later CTA's rows), restated on integers and compared with the visibility
    rule itself, q_first + r*q_pos_stride >= kv_first + n*kv_pos_stride and n < kv_len, for ring steps (equal strides),
    the gathered form (key stride 1) and firsts of either sign: no visible key may fall outside the processed tiles, a tile
    taken without masking must be visible to all rows of the q tile, and the per-row limit must be the last visible key."""
    BM = BN = 128
    rng = np.random.default_rng(7)

    def floor_div(a, b):
        return a // b                                    # Python's // is the floor for either sign, like the kernel's formula

    cases = []
    for _ in range(300):
        sk = int(rng.choice([1, 1, 2, 3, 4, 8]))
        a = 1 if rng.random() < 0.5 else int(rng.integers(1, 8))
        sq = sk * a
        cases.append((sq, sk, int(rng.integers(-40, 2000)), int(rng.integers(-40, 2000)), int(rng.integers(1, 700)),
                      int(rng.integers(0, 3000))))
    cases += [(7, 1, -1, 0, 600, 2500), (7, 1, 6, 0, 513, 3591), (1, 1, 0, 0, 300, 300), (8, 8, 3, 5, 400, 400)]
    for sq, sk, q_first, kv_first, q_len, kv_len in cases:
        vis_a = sq // sk
        vis_c = floor_div(q_first - kv_first, sk)
        rows = np.arange(q_len)
        last_visible = np.minimum(floor_div(q_first + rows * sq - kv_first, sk), kv_len - 1)     # -1 or less: nothing visible
        assert (np.minimum(vis_a * rows + vis_c, kv_len - 1) == last_visible).all()
        for pairs in (False, True):
            block = 2 * BM * (2 if pairs else 1)
            for m0 in range(0, q_len, block):
                for t in range(2):
                    tile_rows = [m0 + c * 2 * BM + t * BM for c in ((0, 1) if pairs else (0,))]
                    cnt = 0
                    for r0 in tile_rows:
                        if r0 < q_len:
                            last_row = min(r0 + BM - 1, q_len - 1)
                            rng_keys = max(0, min(vis_a * last_row + vis_c + 1, kv_len))
                            cnt = max(cnt, (rng_keys + BN - 1) // BN)
                    for r0 in tile_rows:
                        if r0 >= q_len:
                            continue
                        rr = np.arange(r0, min(r0 + BM, q_len))
                        assert (last_visible[rr] < cnt * BN).all(), "a visible key outside the processed tiles"
                        for j in range(cnt):
                            n0 = j * BN
                            masked = (n0 + BN - 1 > vis_a * r0 + vis_c) or (n0 + BN > kv_len)
                            if not masked:
                                assert (last_visible[rr] >= n0 + BN - 1).all(), "an unmasked tile with an invisible key"
