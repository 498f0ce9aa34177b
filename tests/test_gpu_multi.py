"""Two-GPU runs of the ring prefill and of multi-master decode over the raw NCCL layer, one child process
per GPU, checked against the CPU oracle.  Skipped when fewer than two GPUs are visible."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from oracle import esp_oracle as O

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _setup(rank, world, port):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)       # host-side rendezvous only
    from loongserve_b200 import rnccl
    obj = [rnccl.get_nccl_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(obj, 0)
    return dist, rnccl.RNCCLComm(obj[0], world, rank)


def _gather_over(dist, world):
    def gather(b):
        lst = [None] * world
        dist.all_gather_object(lst, b)
        return lst
    return gather


def _ring_worker(rank, world, port, striped, overlap, out, exchange_kind="nccl"):
    dist, comm = _setup(rank, world, port)
    from loongserve_b200 import context_attention as ca
    from loongserve_b200 import kv_ops, ring
    dev = torch.device("cuda", rank)
    g = torch.Generator().manual_seed(0)
    lens = [3000, 77, 1025]
    T, Hq, Hkv, D = sum(lens), 8, 4, 128
    q = torch.randn(T, Hq, D, generator=g).to(torch.bfloat16)
    k = torch.randn(T, Hkv, D, generator=g).to(torch.bfloat16)
    v = torch.randn(T, Hkv, D, generator=g).to(torch.bfloat16)
    local_len, first, stride = ring.shard_lengths(lens, world, striped)
    max_tok = max(sum(x) for x in local_len)
    qs = O.shard_tokens(q, lens, world, striped)[rank].to(dev)
    kv = torch.full((max_tok, 2 * Hkv, D), float("nan"), dtype=torch.bfloat16)
    kr = O.shard_tokens(k, lens, world, striped)[rank]; vr = O.shard_tokens(v, lens, world, striped)[rank]
    kv[:kr.shape[0], :Hkv] = kr; kv[:vr.shape[0], Hkv:] = vr
    kv = kv.to(dev)
    metas = [ring.BlockMeta.from_lengths(local_len[r], first[r], dev) for r in range(world)]
    o = torch.empty_like(qs); m = torch.empty(qs.shape[0], Hq, device=dev); l = torch.empty(qs.shape[0], Hq, device=dev)
    # scale-down bookkeeping: rank 0 keeps the first half of every request, rank 1 the rest
    pool = torch.zeros(T + 16, 2 * Hkv, D, dtype=torch.bfloat16, device=dev)
    cb = torch.tensor([0 if rank == 0 else L // 2 for L in lens], dtype=torch.int32, device=dev)
    ce = torch.tensor([L // 2 if rank == 0 else L for L in lens], dtype=torch.int32, device=dev)
    n_keep = int((ce - cb).sum())
    gk = torch.Generator().manual_seed(5 + rank)
    keep = ring.KeepPlan(cb, ce, torch.randperm(T + 16, generator=gk)[:n_keep].to(dev), torch.arange(len(lens), dtype=torch.int32, device=dev),
                         torch.full((len(lens), 4000), O.INT32_MAX, dtype=torch.int32, device=dev),
                         torch.zeros(len(lens), dtype=torch.int32, device=dev))
    exchange = None
    if exchange_kind == "copy_engine":
        # KV blocks travel as copy-engine transfers into the next instance's memory; a first pass without the
        # bookkeeping leaves the flag counters at non-zero values for the pass that is checked
        from loongserve_b200.peer_ring import CopyEngineRing
        exchange = CopyEngineRing(rank, world, kv.numel() * kv.element_size(), _gather_over(dist, world), device=dev)
        ring.ring_context_attention(qs, kv, o, m, l, rank=rank, peers=list(range(world)), metas=metas, stride=stride,
                                    max_len_in_batch=max(local_len[rank]), num_kv_heads=Hkv, comm=None, recv_buffers=None,
                                    attention_fn=ca.context_attention_fwd, init_fn=ca.init_attention_state, exchange=exchange)
        o.fill_(float("nan"))
    ring.ring_context_attention(qs, kv, o, m, l, rank=rank, peers=list(range(world)), metas=metas, stride=stride,
                                max_len_in_batch=max(local_len[rank]), num_kv_heads=Hkv, comm=comm,
                                recv_buffers=[torch.empty_like(kv), torch.empty_like(kv)],
                                attention_fn=ca.context_attention_fwd, init_fn=ca.init_attention_state, overlap=overlap,
                                keep=keep if striped else None, pool_layer=pool, layer_idx=0,
                                keep_fns=(kv_ops.pre_copy_and_register_kv, kv_ops.destindex_copy_and_register_kv),
                                exchange=exchange)
    torch.cuda.synchronize()
    st = ca.device_status()
    if exchange is not None:
        exchange.check()                      # no flag wait ran out
        assert exchange.sent[(rank + 1) % world] == exchange.received[(rank - 1) % world] == 2 * (world - 1)
        dist.barrier()
        exchange.close()
    torch.save(dict(o=o.cpu(), lse=ca.attention_lse(m, l).cpu(), status=st, pool=pool.cpu(), rtt=keep.req_to_token_indexs.cpu(),
                    cb=cb.cpu(), ce=ce.cpu()), os.path.join(out, f"r{rank}.pt"))
    dist.barrier()
    comm.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("striped,overlap,exchange_kind", [(True, True, "nccl"), (False, True, "nccl"), (True, False, "nccl"),
                                                          (True, True, "copy_engine"), (False, True, "copy_engine")])
def test_ring_two_gpus(tmp_path, striped, overlap, exchange_kind):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world = 2
    mp.spawn(_ring_worker, args=(world, _free_port(), striped, overlap, str(tmp_path), exchange_kind), nprocs=world, join=True)
    g = torch.Generator().manual_seed(0)
    lens = [3000, 77, 1025]
    T, Hq, Hkv, D = sum(lens), 8, 4, 128
    q = torch.randn(T, Hq, D, generator=g).to(torch.bfloat16)
    k = torch.randn(T, Hkv, D, generator=g).to(torch.bfloat16)
    v = torch.randn(T, Hkv, D, generator=g).to(torch.bfloat16)
    ro, rlse = O.full_causal_attention(q, k, v, lens)
    parts = [torch.load(os.path.join(str(tmp_path), f"r{r}.pt")) for r in range(world)]
    assert all(p["status"][0] == 0 for p in parts)
    o = O.unshard_tokens([p["o"] for p in parts], lens, world, striped)
    lse = O.unshard_tokens([p["lse"] for p in parts], lens, world, striped)
    assert bool(((o.float() - ro).abs() <= 2e-2 + 1e-2 * ro.abs()).all())
    assert torch.allclose(lse, rlse, atol=1e-3, rtol=1e-3)
    if striped:
        # every instance kept exactly its assigned global range of every request, bit-exact
        kvfull = torch.cat([k, v], dim=1)
        starts = [0, lens[0], lens[0] + lens[1]]
        for r, p in enumerate(parts):
            for b, L in enumerate(lens):
                cb, ce = int(p["cb"][b]), int(p["ce"][b])
                slots = p["rtt"][b, :ce - cb].long()
                got = p["pool"][slots]
                want_set = kvfull[starts[b] + cb:starts[b] + ce]
                # slot order is grouped by ring step (source rank), not by position: compare as multisets of rows
                key = lambda t: sorted(map(bytes, t.reshape(t.shape[0], -1).view(torch.uint8).numpy()))
                assert key(got) == key(want_set), f"rank {r} request {b}"


def _decode_worker(rank, world, port, out):
    dist, comm = _setup(rank, world, port)
    from loongserve_b200 import flash_decoding as fd
    from loongserve_b200 import ring
    dev = torch.device("cuda", rank)
    g = torch.Generator().manual_seed(0)
    B, Hh, D, bs = 4, 8, 128, 256
    lens = [3000, 41, 1290, 640]
    total = sum(lens)
    kall = torch.randn(total, Hh, D, generator=g).to(torch.bfloat16); vall = torch.randn(total, Hh, D, generator=g).to(torch.bfloat16)
    q = torch.randn(B, Hh, D, generator=g).to(torch.bfloat16).to(dev)
    pool = torch.zeros(total, 2 * Hh, D, dtype=torch.bfloat16); rt = torch.full((B, 4000), O.INT32_MAX, dtype=torch.int32)
    loc_len = []
    off = 0; slot = 0
    for b, L in enumerate(lens):
        mine = list(range(rank, L, world))
        pool[slot:slot + len(mine), :Hh] = kall[off + rank:off + L:world]
        pool[slot:slot + len(mine), Hh:] = vall[off + rank:off + L:world]
        rt[b, :len(mine)] = torch.arange(slot, slot + len(mine), dtype=torch.int32)
        slot += len(mine); loc_len.append(len(mine)); off += L
    pool, rt = pool.to(dev), rt.to(dev)
    b_req = torch.arange(B, dtype=torch.int32, device=dev); b_len = torch.tensor(loc_len, dtype=torch.int32, device=dev)
    mx = max(loc_len); nblk = (mx + bs - 1) // bs
    master = peer = None
    f32 = dict(dtype=torch.float32, device=dev)
    if rank == 0:
        master = ring.MasterPlan(peers=list(range(world)), b_req_idx=b_req, b_seq_len=b_len, max_len_in_batch=mx, block_seq=bs,
                                 global_mid_o=torch.zeros(world - 1 + nblk, B, Hh, D, **f32), global_mid_lse=torch.zeros(world - 1 + nblk, B, Hh, **f32),
                                 global_merge_len=(world - 1 + (b_len + bs - 1) // bs).to(torch.int32), global_out_lse=torch.zeros(B, Hh, **f32))
    else:
        peer = ring.PeerPlan(masters=[0], ranges=[(0, B)], peer_query_buffer=torch.zeros(B, Hh, D, dtype=torch.bfloat16, device=dev),
                             peer_b_req_idx=b_req, peer_b_seq_len=b_len, peer_max_len_in_batch=mx, block_seq=bs,
                             peer_mid_o=torch.zeros(nblk, B, Hh, D, **f32), peer_mid_lse=torch.zeros(nblk, B, Hh, **f32),
                             peer_o=torch.zeros(B, Hh, D, **f32), peer_lse=torch.zeros(B, Hh, **f32))
    o = ring.multi_master_decode_attention(q if rank == 0 else None, pool, rt, Hh, comm, rank, master, peer,
                                           fd.flash_decoding_stage1, fd.flash_decoding_stage2)
    torch.cuda.synchronize()
    if rank == 0:
        torch.save((o.cpu(), master.global_out_lse.cpu()), os.path.join(out, "dec.pt"))
    dist.barrier()
    comm.close()
    dist.destroy_process_group()


def test_multi_master_decode_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world = 2
    mp.spawn(_decode_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    o, lse = torch.load(os.path.join(str(tmp_path), "dec.pt"))
    g = torch.Generator().manual_seed(0)
    B, Hh, D = 4, 8, 128
    lens = [3000, 41, 1290, 640]; total = sum(lens)
    kall = torch.randn(total, Hh, D, generator=g).to(torch.bfloat16); vall = torch.randn(total, Hh, D, generator=g).to(torch.bfloat16)
    q = torch.randn(B, Hh, D, generator=g).to(torch.bfloat16)
    rt = torch.full((B, 4000), O.INT32_MAX, dtype=torch.int32); off = 0
    for b, L in enumerate(lens):
        rt[b, :L] = torch.arange(off, off + L, dtype=torch.int32); off += L
    ro, rl = O.token_decode_attention(q, kall, vall, rt, torch.arange(B, dtype=torch.int32), torch.tensor(lens, dtype=torch.int32))
    assert torch.allclose(o.float(), ro, atol=2e-2, rtol=1e-2) and torch.allclose(lse, rl, atol=1e-3, rtol=1e-3)


def _runtime_worker(rank, world, port, out):
    dist, comm = _setup(rank, world, port)
    from loongserve_b200.attention_runtime import ESPAttentionRuntime
    dev = torch.device("cuda", rank)
    L, Hq, Hkv, D = 2, 8, 4, 128
    rt = ESPAttentionRuntime(layers_num=L, q_head_num=Hq, kv_head_num=Hkv, head_dim=D, max_total_token_num=4096, max_req_num=8,
                             max_seq_length=4096, sp_world_size=world, total_rank=rank, sp_comm=comm, dtype=torch.bfloat16,
                             device=dev, peer_memory_decode=False)
    g = torch.Generator().manual_seed(33)
    lens = [1500, 64, 777]
    B, T = len(lens), sum(lens)
    q = [torch.randn(T, Hq, D, generator=g).to(torch.bfloat16) for _ in range(L)]
    kv = [torch.randn(T, 2 * Hkv, D, generator=g).to(torch.bfloat16) for _ in range(L)]
    qd = [torch.randn(B, Hq, D, generator=g).to(torch.bfloat16) for _ in range(L)]       # decode queries
    local_len = [max(0, (n - rank + world - 1) // world) for n in lens]
    b_len = torch.tensor(local_len, dtype=torch.int32, device=dev)
    b_start = torch.cumsum(b_len, 0, dtype=torch.int32) - b_len
    b_req = torch.arange(B, dtype=torch.int32, device=dev)
    # scale-down plan: instance 0 keeps the first 60 % of every request, instance 1 the rest
    cb = torch.tensor([0 if rank == 0 else (6 * n) // 10 for n in lens], dtype=torch.int32, device=dev)
    ce = torch.tensor([(6 * n) // 10 if rank == 0 else n for n in lens], dtype=torch.int32, device=dev)
    max_tok = max(sum(max(0, (n - r + world - 1) // world) for n in lens) for r in range(world))
    st = rt.prepare_prefill(B, sum(local_len), max_tok, max(local_len), b_req, b_start, b_len,
                            torch.full((B,), rank, dtype=torch.int32, device=dev), list(range(world)), rank,
                            need_context_migration=True, kv_cache_index_begin=cb, kv_cache_index_end=ce,
                            request_lengths=lens, striped=True)
    outs = []
    for layer in range(L):
        mine = O.shard_tokens(kv[layer], lens, world, True)[rank]
        rt.pre_cache_kv(st, layer)[:mine.shape[0]].copy_(mine.to(dev))
        o = rt.context_attention(O.shard_tokens(q[layer], lens, world, True)[rank].to(dev), st, layer)
        outs.append(o.cpu())
    kept = [int(ce[b] - cb[b]) for b in range(B)]
    # ---- multi-master decode over the kept tokens (instance 0 is the master; no new token is added here)
    k_len = torch.tensor(kept, dtype=torch.int32, device=dev)
    f32 = dict(dtype=torch.float32, device=dev)
    from loongserve_b200 import ring
    bs = 256
    nblk = (max(kept) + bs - 1) // bs
    master = peer = None
    if rank == 0:
        master = ring.MasterPlan(peers=list(range(world)), b_req_idx=b_req, b_seq_len=k_len, max_len_in_batch=max(kept), block_seq=bs,
                                 global_mid_o=torch.empty(world - 1 + nblk, B, Hq, D, **f32), global_mid_lse=torch.empty(world - 1 + nblk, B, Hq, **f32),
                                 global_merge_len=(world - 1 + (k_len + bs - 1) // bs).to(torch.int32), global_out_lse=torch.empty(B, Hq, **f32))
    else:
        peer = ring.PeerPlan(masters=[0], ranges=[(0, B)], peer_query_buffer=torch.empty(B, Hq, D, dtype=torch.bfloat16, device=dev),
                             peer_b_req_idx=b_req, peer_b_seq_len=k_len, peer_max_len_in_batch=max(kept), block_seq=bs,
                             peer_mid_o=torch.empty(nblk, B, Hq, D, **f32), peer_mid_lse=torch.empty(nblk, B, Hq, **f32),
                             peer_o=torch.empty(B, Hq, D, **f32), peer_lse=torch.empty(B, Hq, **f32))
    dstate = LongServeState(master_plan=master, peer_plan=peer, logical_sp_peer_ranks=list(range(world)))
    dec1 = [rt.token_attention(qd[layer].to(dev) if rank == 0 else None, dstate, layer) for layer in range(L)]
    # ---- decode-stage migration: instance 1 hands the last 100 / 0 / 50 kept tokens of each request to instance 0
    mig = torch.tensor([100, 0, 50], dtype=torch.int32, device=dev)
    torch.cuda.synchronize(); dist.barrier()
    if rank == 0:
        rt.decoding_stage_migration(True, b_req, mig, k_len, 1, migration_len_sum=150, max_migration_len=100)
        new_len = k_len + mig
    else:
        rt.decoding_stage_migration(False, b_req, mig, k_len, 0, migration_len_sum=150, max_migration_len=100)
        new_len = k_len - mig
    if rank == 0:
        master.b_seq_len = new_len; master.max_len_in_batch = int(new_len.max())
        nb2 = (int(new_len.max()) + bs - 1) // bs
        master.global_mid_o = torch.empty(world - 1 + nb2, B, Hq, D, **f32); master.global_mid_lse = torch.empty(world - 1 + nb2, B, Hq, **f32)
        master.global_merge_len = (world - 1 + (new_len + bs - 1) // bs).to(torch.int32)
    else:
        peer.peer_b_seq_len = new_len
    dec2 = [rt.token_attention(qd[layer].to(dev) if rank == 0 else None, dstate, layer) for layer in range(L)]
    torch.cuda.synchronize()
    # ---- the same decode with the exchange done by NVLink stores and flags inside the kernels
    def gather(b):
        lst = [None] * world
        dist.all_gather_object(lst, b)
        return lst
    rt.enable_peer_memory_decode(0, gather, max_batch=B)
    dec3 = [rt.token_attention(qd[layer].to(dev) if rank == 0 else None, dstate, layer) for layer in range(L)]
    torch.cuda.synchronize()
    torch.save(dict(outs=outs, dec1=[x.cpu() if x is not None else None for x in dec1],
                    dec2=[x.cpu() if x is not None else None for x in dec2],
                    dec3=[x.cpu() if x is not None else None for x in dec3], free=rt.mem_manager.can_use_mem_size,
                    state_sum=int(rt.mem_manager.mem_state.sum()), kept=kept), os.path.join(out, f"rt{rank}.pt"))
    dist.barrier()
    rt.close()
    comm.close()
    dist.destroy_process_group()


def _runtime_gathered_worker(rank, world, port, out):
    """Prefill batches through the runtime with ``gathered_prefill=True``: two attention launches per layer instead of one per
    instance.  The second batch is larger than the first (the exchange buffer is remade, collectively), the third smaller."""
    dist, comm = _setup(rank, world, port)
    from loongserve_b200.attention_runtime import ESPAttentionRuntime
    dev = torch.device("cuda", rank)
    L, Hq, Hkv, D = 2, 8, 4, 128
    rt = ESPAttentionRuntime(layers_num=L, q_head_num=Hq, kv_head_num=Hkv, head_dim=D, max_total_token_num=8192, max_req_num=8,
                             max_seq_length=4096, sp_world_size=world, total_rank=rank, sp_comm=comm, dtype=torch.bfloat16,
                             device=dev, peer_memory_decode=False, gathered_prefill=True)
    res = []
    for bi, lens in enumerate(([300, 64], [1500, 3, 777], [129])):
        g = torch.Generator().manual_seed(50 + bi)
        B, T = len(lens), sum(lens)
        q = [torch.randn(T, Hq, D, generator=g).to(torch.bfloat16) for _ in range(L)]
        kv = [torch.randn(T, 2 * Hkv, D, generator=g).to(torch.bfloat16) for _ in range(L)]
        local_len = [max(0, (n - rank + world - 1) // world) for n in lens]
        b_len = torch.tensor(local_len, dtype=torch.int32, device=dev)
        b_start = torch.cumsum(b_len, 0, dtype=torch.int32) - b_len
        b_req = torch.arange(B, dtype=torch.int32, device=dev)
        max_tok = max(sum(max(0, (n - r + world - 1) // world) for n in lens) for r in range(world))
        st = rt.prepare_prefill(B, sum(local_len), max_tok, max(max(local_len), 1), b_req, b_start, b_len,
                                torch.full((B,), rank, dtype=torch.int32, device=dev), list(range(world)), rank,
                                request_lengths=lens, striped=True)
        assert getattr(st, "gather_plans", None) is not None
        outs = []
        for layer in range(L):
            mine = O.shard_tokens(kv[layer], lens, world, True)[rank]
            rt.pre_cache_kv(st, layer)[:mine.shape[0]].copy_(mine.to(dev))
            o = rt.context_attention(O.shard_tokens(q[layer], lens, world, True)[rank].to(dev), st, layer)
            outs.append(o.cpu())
        torch.cuda.synchronize()
        rt.check_device_status()
        res.append(outs)
        rt.mem_manager.free_all()
        rt.req_manager.free_all()
    torch.save(res, os.path.join(out, f"rg{rank}.pt"))
    dist.barrier()
    rt.close()
    comm.close()
    dist.destroy_process_group()


def test_runtime_gathered_prefill_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world = 2
    mp.spawn(_runtime_gathered_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    parts = [torch.load(os.path.join(str(tmp_path), f"rg{r}.pt")) for r in range(world)]
    L, Hq, Hkv, D = 2, 8, 4, 128
    for bi, lens in enumerate(([300, 64], [1500, 3, 777], [129])):
        g = torch.Generator().manual_seed(50 + bi)
        T = sum(lens)
        q = [torch.randn(T, Hq, D, generator=g).to(torch.bfloat16) for _ in range(L)]
        kv = [torch.randn(T, 2 * Hkv, D, generator=g).to(torch.bfloat16) for _ in range(L)]
        for layer in range(L):
            ro, _ = O.full_causal_attention(q[layer], kv[layer][:, :Hkv], kv[layer][:, Hkv:], lens)
            o = O.unshard_tokens([p[bi][layer] for p in parts], lens, world, True)
            assert bool(((o.float() - ro).abs() <= 2e-2 + 1e-2 * ro.abs()).all()), (bi, layer)


class LongServeState:
    def __init__(self, master_plan, peer_plan, logical_sp_peer_ranks=None):
        self.master_plan, self.peer_plan, self.logical_sp_peer_ranks = master_plan, peer_plan, logical_sp_peer_ranks


def test_runtime_prefill_keep_decode_migrate_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world = 2
    mp.spawn(_runtime_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    g = torch.Generator().manual_seed(33)
    L, Hq, Hkv, D = 2, 8, 4, 128
    lens = [1500, 64, 777]
    B, T = len(lens), sum(lens)
    q = [torch.randn(T, Hq, D, generator=g).to(torch.bfloat16) for _ in range(L)]
    kv = [torch.randn(T, 2 * Hkv, D, generator=g).to(torch.bfloat16) for _ in range(L)]
    qd = [torch.randn(B, Hq, D, generator=g).to(torch.bfloat16) for _ in range(L)]
    parts = [torch.load(os.path.join(str(tmp_path), f"rt{r}.pt")) for r in range(world)]
    rtab = torch.full((B, max(lens)), O.INT32_MAX, dtype=torch.int32); off = 0
    for b, n in enumerate(lens):
        rtab[b, :n] = torch.arange(off, off + n, dtype=torch.int32); off += n
    for layer in range(L):
        ro, _ = O.full_causal_attention(q[layer], kv[layer][:, :Hkv], kv[layer][:, Hkv:], lens)
        o = O.unshard_tokens([p["outs"][layer] for p in parts], lens, world, True)
        assert bool(((o.float() - ro).abs() <= 2e-2 + 1e-2 * ro.abs()).all())
        # decode over ALL tokens of every request (the two instances together hold each token exactly once),
        # identical before and after the migration
        rd, _ = O.token_decode_attention(qd[layer], kv[layer][:, :Hkv], kv[layer][:, Hkv:], rtab, torch.arange(B, dtype=torch.int32),
                                         torch.tensor(lens, dtype=torch.int32))
        for key in ("dec1", "dec2", "dec3"):
            got = parts[0][key][layer].float()
            assert bool(((got - rd).abs() <= 2e-2 + 1e-2 * rd.abs()).all()), key
    # slot accounting: kept tokens, then 150 tokens moved from instance 1 to instance 0
    assert parts[0]["free"] == 4096 - sum(parts[0]["kept"]) - 150 and parts[1]["free"] == 4096 - sum(parts[1]["kept"]) + 150
    assert parts[0]["state_sum"] == sum(parts[0]["kept"]) + 150 and parts[1]["state_sum"] == sum(parts[1]["kept"]) - 150


def _two_masters_worker(rank, world, port, out, peer_memory=False):
    """Both instances are masters of their own mini-batch and peers for the other's
    (the multi-master case: pre_process.py:194-230, longserve_transformer_layer_infer.py:247-265)."""
    dist, comm = _setup(rank, world, port)
    from loongserve_b200.attention_runtime import ESPAttentionRuntime
    dev = torch.device("cuda", rank)
    Hq, Hkv, D = 8, 2, 128
    rt = ESPAttentionRuntime(layers_num=1, q_head_num=Hq, kv_head_num=Hkv, head_dim=D, max_total_token_num=8192, max_req_num=16,
                             max_seq_length=4096, sp_world_size=world, total_rank=rank, sp_comm=comm, dtype=torch.float16, device=dev,
                             peer_memory_decode=False)
    if peer_memory:
        def gather(b):
            lst = [None] * world
            dist.all_gather_object(lst, b)
            return lst
        for master in range(world):                 # one group per master, created in the same order everywhere
            rt.enable_peer_memory_decode(master, gather, max_batch=4)
    g = torch.Generator().manual_seed(77)
    # requests 0..2 belong to master 0, requests 3..4 to master 1; lengths include the new token
    lens = [900, 33, 2000, 513, 1500]
    owner = [0, 0, 0, 1, 1]
    kv = [torch.randn(n, 2 * Hkv, D, generator=g).to(torch.float16) for n in lens]
    q = torch.randn(len(lens), Hq, D, generator=g).to(torch.float16)
    # existing tokens (all but the new one) are spread round-robin over the two instances; the new token's KV goes to its master
    slot = 0
    local_cnt = []
    for b, n in enumerate(lens):
        mine = [t for t in range(n - 1) if t % world == rank]
        rows = torch.tensor(mine, dtype=torch.long)
        rt.mem_manager.kv_buffer[0][slot:slot + len(mine)] = kv[b][rows].to(dev)
        rt.req_manager.req_to_token_indexs[b, :len(mine)] = torch.arange(slot, slot + len(mine), dtype=torch.int32, device=dev)
        slot += len(mine); local_cnt.append(len(mine))
    rt.mem_manager.add_refs(torch.arange(slot, device=dev))
    my_reqs = [b for b in range(len(lens)) if owner[b] == rank]
    other_reqs = [b for b in range(len(lens)) if owner[b] != rank]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    my_len = [local_cnt[b] + 1 for b in my_reqs]                      # + the new token
    st = rt.prepare_decode(len(my_reqs), len(my_reqs), max(my_len), i32(my_reqs), i32(my_len), i32([lens[b] - 1 for b in my_reqs]),
                           rank, list(range(world)), rank, peer_sp_master_rank_list=[1 - rank],
                           peer_query_buffer_range_list=[(0, len(other_reqs))], peer_batch_size=len(other_reqs),
                           peer_max_len_in_batch=max(local_cnt[b] for b in other_reqs), peer_b_req_idx=i32(other_reqs),
                           peer_b_seq_len=i32([local_cnt[b] for b in other_reqs]))
    new_rows = torch.stack([kv[b][lens[b] - 1] for b in my_reqs]).to(dev)
    rt.decode_cache_kv(st, 0).copy_(new_rows)
    rt.post_decode_cache_kv(st, 0)
    o = rt.token_attention(q[my_reqs].to(dev), st, 0)
    if peer_memory:
        o = rt.token_attention(q[my_reqs].to(dev), st, 0)        # a second layer call: flags and slots are reused
    torch.cuda.synchronize()
    status = rt._fused_groups[rank].device_status() if peer_memory else (0, 0, 0, 0)
    torch.save(dict(o=o.cpu(), lse=st.global_out_logexpsum.cpu(), reqs=my_reqs, status=status), os.path.join(out, f"mm{rank}.pt"))
    dist.barrier()
    rt.close()
    comm.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("peer_memory", [False, True], ids=["nccl", "peer_memory"])
def test_two_masters_two_gpus(tmp_path, peer_memory):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world = 2
    mp.spawn(_two_masters_worker, args=(world, _free_port(), str(tmp_path), peer_memory), nprocs=world, join=True)
    g = torch.Generator().manual_seed(77)
    Hq, Hkv, D = 8, 2, 128
    lens = [900, 33, 2000, 513, 1500]
    kv = [torch.randn(n, 2 * Hkv, D, generator=g).to(torch.float16) for n in lens]
    q = torch.randn(len(lens), Hq, D, generator=g).to(torch.float16)
    allkv = torch.cat(kv, 0)
    rtab = torch.full((len(lens), max(lens)), O.INT32_MAX, dtype=torch.int32); off = 0
    for b, n in enumerate(lens):
        rtab[b, :n] = torch.arange(off, off + n, dtype=torch.int32); off += n
    ro, rl = O.token_decode_attention(q, allkv[:, :Hkv], allkv[:, Hkv:], rtab, torch.arange(len(lens), dtype=torch.int32),
                                      torch.tensor(lens, dtype=torch.int32))
    for r in range(world):
        p = torch.load(os.path.join(str(tmp_path), f"mm{r}.pt"))
        got, want = p["o"].float(), ro[p["reqs"]]
        assert p["status"][0] == 0                                  # no flag wait ran out
        assert bool(((got - want).abs() <= 2e-2 + 1e-2 * want.abs()).all())
        assert torch.allclose(p["lse"], rl[p["reqs"]], atol=1e-3, rtol=1e-3)


def _fused_decode_worker(rank, world, port, out):
    dist, comm = _setup(rank, world, port)
    from loongserve_b200.peer_decode import FusedDecodeGroup
    dev = torch.device("cuda", rank)
    g = torch.Generator().manual_seed(0)
    B, Hh, D, bs = 4, 8, 128, 256
    lens = [3000, 41, 1290, 640]
    total = sum(lens)
    kall = torch.randn(total, Hh, D, generator=g).to(torch.bfloat16); vall = torch.randn(total, Hh, D, generator=g).to(torch.bfloat16)
    qs = [torch.randn(B, Hh, D, generator=g).to(torch.bfloat16) for _ in range(3)]
    pool = torch.zeros(total, 2 * Hh, D, dtype=torch.bfloat16); rt = torch.full((B, 4000), O.INT32_MAX, dtype=torch.int32)
    loc_len = []
    off = 0; slot = 0
    for b, L in enumerate(lens):
        n = len(range(rank, L, world))
        pool[slot:slot + n, :Hh] = kall[off + rank:off + L:world]; pool[slot:slot + n, Hh:] = vall[off + rank:off + L:world]
        rt[b, :n] = torch.arange(slot, slot + n, dtype=torch.int32)
        slot += n; loc_len.append(n); off += L
    pool, rt = pool.to(dev), rt.to(dev)
    b_req = torch.arange(B, dtype=torch.int32, device=dev); b_len = torch.tensor(loc_len, dtype=torch.int32, device=dev)
    mx = max(loc_len); nblk = (mx + bs - 1) // bs

    def gather(b):
        lst = [None] * world
        dist.all_gather_object(lst, b)
        return lst

    grp = FusedDecodeGroup(rank, world, 0, B + 3, Hh, D, gather)          # region sized for a larger batch than the one used
    mid_o = torch.empty(nblk, B, Hh, D, device=dev); mid_l = torch.empty(nblk, B, Hh, device=dev)
    res = []
    for q in qs:                                   # three steps in a row: the flags advance 1, 2, 3
        r = grp.step(q.to(dev) if rank == 0 else None, pool, rt, Hh, b_req, b_len, mx, bs, mid_o, mid_l)
        if rank == 0:
            res.append((r[0].cpu(), r[1].cpu()))
    torch.cuda.synchronize()
    st = grp.device_status()
    dist.barrier()
    if rank == 0:
        torch.save((res, st), os.path.join(out, "fused.pt"))
    grp.close()
    comm.close()
    dist.destroy_process_group()


def test_fused_peer_memory_decode_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world = 2
    mp.spawn(_fused_decode_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    res, st = torch.load(os.path.join(str(tmp_path), "fused.pt"))
    assert st[0] == 0, f"a bounded flag wait expired: {st}"
    g = torch.Generator().manual_seed(0)
    B, Hh, D = 4, 8, 128
    lens = [3000, 41, 1290, 640]; total = sum(lens)
    kall = torch.randn(total, Hh, D, generator=g).to(torch.bfloat16); vall = torch.randn(total, Hh, D, generator=g).to(torch.bfloat16)
    qs = [torch.randn(B, Hh, D, generator=g).to(torch.bfloat16) for _ in range(3)]
    rt = torch.full((B, 4000), O.INT32_MAX, dtype=torch.int32); off = 0
    for b, L in enumerate(lens):
        rt[b, :L] = torch.arange(off, off + L, dtype=torch.int32); off += L
    for q, (o, lse) in zip(qs, res):
        ro, rl = O.token_decode_attention(q, kall, vall, rt, torch.arange(B, dtype=torch.int32), torch.tensor(lens, dtype=torch.int32))
        assert torch.allclose(o.float(), ro, atol=2e-2, rtol=1e-2) and torch.allclose(lse, rl, atol=1e-3, rtol=1e-3)


def _forward_kwargs_worker(rank, world, port, out):
    """Drive the layer stack with exactly the keyword arguments the reference's worker builds
    (pre_process.py:95-121 for prefill, :232-258 for decode)."""
    dist, comm = _setup(rank, world, port)
    from loongserve_b200.attention_runtime import ESPAttentionRuntime
    from loongserve_b200.llama_stack import LlamaConfig, LlamaESPStack, LlamaWeights
    dev = torch.device("cuda", rank)
    cfg = LlamaConfig(num_layers=2, hidden=512, num_q_heads=4, num_kv_heads=4, head_dim=128, ffn=1024, vocab=1000)
    rt = ESPAttentionRuntime(layers_num=2, q_head_num=4, kv_head_num=4, head_dim=128, max_total_token_num=2048, max_req_num=8,
                             max_seq_length=2048, sp_world_size=world, total_rank=rank, sp_comm=comm, dtype=torch.bfloat16, device=dev)
    stack = LlamaESPStack(cfg, LlamaWeights(cfg, torch.bfloat16, dev, seed=3), rt)
    g = torch.Generator().manual_seed(9)
    full = [301, 64, 130]
    B = len(full)
    ids = torch.randint(0, cfg.vocab, (sum(full),), generator=g)
    pre = [n - 1 for n in full]
    starts = [0, full[0], full[0] + full[1]]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    local = [list(range(rank, n, world)) for n in pre]                      # striped placement of the prompt tokens
    from loongserve_b200 import pre_process as pp
    b_len = [len(l) for l in local]
    max_tok = max(sum(len(range(r, n, world)) for n in pre) for r in range(world))
    reqs = {f"req{b}": pp.InferReq(req_idx=b, prompt_len=pre[b], cur_kv_len=0) for b in range(B)}
    batch = pp.InferBatch(list(reqs), reqs)
    worker = pp.Worker(sp_rank=rank, device=dev)
    local_ids = [ids[s + torch.tensor(l, dtype=torch.long)].tolist() for s, l in zip(starts, local)]
    kwargs, run, not_run = pp.prepare_prefill_inputs(batch, (local_ids, max_tok, list(range(world)), rank, [True] * B, False, None, None), worker)
    assert len(run) == B and not not_run
    pre_logits = stack.forward(**kwargs)
    # decode: instance 0 is the master of all three requests; the router's records hold the tokens cached so far
    for b in range(B):
        reqs[f"req{b}"].cur_kv_len = reqs[f"req{b}"].prompt_len = b_len[b]
    new_ids = [int(ids[s + n - 1]) for s, n in zip(starts, full)]
    gk = (new_ids if rank == 0 else None, pre if rank == 0 else None, 1, [B], list(range(world)), rank)
    dk, run, peer_run, _ = pp.prepare_decode_inputs(batch, gk, worker)
    assert (len(run), len(peer_run)) == ((B, 0) if rank == 0 else (0, B))
    dec_logits = stack.forward(**dk)
    torch.cuda.synchronize()
    torch.save(dict(pre=pre_logits.cpu(), dec=None if dec_logits is None else dec_logits.cpu()), os.path.join(out, f"fw{rank}.pt"))
    rt.check_device_status()
    dist.barrier()
    rt.close()
    comm.close()
    dist.destroy_process_group()


def test_forward_with_reference_kwargs_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world = 2
    mp.spawn(_forward_kwargs_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    from loongserve_b200.llama_stack import LlamaConfig, LlamaWeights
    cfg = LlamaConfig(num_layers=2, hidden=512, num_q_heads=4, num_kv_heads=4, head_dim=128, ffn=1024, vocab=1000)
    w = LlamaWeights(cfg, torch.bfloat16, "cuda:0", seed=3)
    g = torch.Generator().manual_seed(9)
    full = [301, 64, 130]
    ids = torch.randint(0, cfg.vocab, (sum(full),), generator=g)
    pos = torch.cat([torch.arange(n) for n in full])
    x = w.embed.cpu()[ids.long()].float()
    for lw in w.layers:
        x, _, _ = O.llama_layer(x, pos, full, {k: v.cpu() for k, v in lw.items()}, cfg.rms_eps, 4, 4, 128, torch.bfloat16)
    starts = [0, full[0], full[0] + full[1]]
    new_rows = torch.tensor([s + n - 1 for s, n in zip(starts, full)])
    ref = O.rms_norm(x[new_rows], w.final_norm.cpu(), cfg.rms_eps).to(torch.bfloat16).float() @ w.lm_head.cpu().float()
    dec = torch.load(os.path.join(str(tmp_path), "fw0.pt"))["dec"]
    err = (dec - ref).abs()
    assert bool((err <= 5e-2 + 5e-2 * ref.abs()).all()), err.max()


def _graphed_decode_worker(rank, world, port, out):
    """The same prompt and the same fed tokens through two runtimes: decode steps issued kernel by kernel, and the
    step replayed as one CUDA graph per instance.  Both use the peer-memory exchange."""
    dist, comm = _setup(rank, world, port)
    from loongserve_b200.attention_runtime import ESPAttentionRuntime
    from loongserve_b200.llama_stack import GraphedDecode, LlamaConfig, LlamaESPStack, LlamaWeights
    dev = torch.device("cuda", rank)
    cfg = LlamaConfig(num_layers=3, hidden=512, num_q_heads=4, num_kv_heads=2, head_dim=128, ffn=1024, vocab=1000)
    weights = LlamaWeights(cfg, torch.bfloat16, dev, seed=4)

    def gather(b):
        lst = [None] * world
        dist.all_gather_object(lst, b)
        return lst

    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    lens = [700, 45]
    B, n_steps = len(lens), 4
    g = torch.Generator().manual_seed(21)
    ids = torch.randint(0, cfg.vocab, (sum(lens),), generator=g)
    fed = torch.randint(0, cfg.vocab, (n_steps, B), generator=g)
    starts = [0, lens[0]]
    local = [list(range(rank, n, world)) for n in lens]
    b_len = [len(l) for l in local]
    local_ids = torch.cat([ids[s + torch.tensor(l, dtype=torch.long)] for s, l in zip(starts, local)]).to(dev)
    pos = torch.cat([torch.tensor(l, dtype=torch.long) for l in local]).to(dev)
    max_tok = max(sum(len(range(r, n, world)) for n in lens) for r in range(world))
    results = {}
    for mode in ("eager", "graph"):
        rt = ESPAttentionRuntime(layers_num=cfg.num_layers, q_head_num=4, kv_head_num=2, head_dim=128, max_total_token_num=2048,
                                 max_req_num=8, max_seq_length=2048, sp_world_size=world, total_rank=rank, sp_comm=comm,
                                 dtype=torch.bfloat16, device=dev, decode_block_seq=256)
        rt.enable_peer_memory_decode(0, gather, max_batch=B)
        stack = LlamaESPStack(cfg, weights, rt)
        st = rt.prepare_prefill(B, sum(b_len), max_tok, max(b_len), i32([0, 1]), i32([0, b_len[0]]), i32(b_len), i32([rank] * B),
                                list(range(world)), rank, request_lengths=lens, striped=True)
        stack.prefill(local_ids, pos, st)
        logits = []
        cnt = list(b_len)
        if mode == "eager":
            for s_ in range(n_steps):
                if rank == 0:
                    cnt = [c + 1 for c in cnt]
                    d = rt.prepare_decode(B, B, max(cnt), i32([0, 1]), i32(cnt), i32([n + s_ for n in lens]), 0, list(range(world)), 0)
                    logits.append(stack.decode(fed[s_].to(dev), i32([n + s_ for n in lens]), d).cpu())
                else:
                    d = rt.prepare_decode(0, 0, 0, None, None, None, None, list(range(world)), rank, peer_sp_master_rank_list=[0],
                                          peer_query_buffer_range_list=[(0, B)], peer_batch_size=B, peer_max_len_in_batch=max(cnt),
                                          peer_b_req_idx=i32([0, 1]), peer_b_seq_len=i32(cnt))
                    stack.decode(None, None, d)
        else:
            gd = GraphedDecode(stack, rt._fused_groups[0], i32([0, 1]), i32(cnt), positions=i32(lens) if rank == 0 else None,
                               max_new_tokens=n_steps).capture()
            dist.barrier()
            for s_ in range(n_steps):
                lg = gd.step(fed[s_] if rank == 0 else None)
                if rank == 0:
                    logits.append(lg.cpu().clone())
        torch.cuda.synchronize()
        status = rt._fused_groups[0].device_status()
        results[mode] = dict(logits=logits, status=status, table=rt.req_manager.req_to_token_indexs[:2, :b_len[0] + n_steps].cpu(),
                             free=rt.mem_manager.can_use_mem_size)
        dist.barrier()
        rt.close()
    torch.save(results, os.path.join(out, f"gd{rank}.pt"))
    dist.barrier()
    comm.close()
    dist.destroy_process_group()


def test_graphed_decode_matches_kernel_by_kernel_decode_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world = 2
    mp.spawn(_graphed_decode_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        res = torch.load(os.path.join(str(tmp_path), f"gd{r}.pt"))
        assert res["eager"]["status"][0] == 0 and res["graph"]["status"][0] == 0        # no flag wait ran out
        assert torch.equal(res["eager"]["table"], res["graph"]["table"])                # same slots registered
        assert res["eager"]["free"] == res["graph"]["free"]
        if r == 0:
            assert len(res["graph"]["logits"]) == 4
            for a, b in zip(res["eager"]["logits"], res["graph"]["logits"]):
                assert bool(torch.isfinite(b).all())
                assert bool(((a - b).abs() <= 1e-3 + 1e-3 * a.abs()).all()), (a - b).abs().max()


def _gather_worker(rank, world, port, out, parts=1):
    """The two-launch form of a striped pass: blocks copied to every other instance by copy engines, flags in peer memory."""
    dist, comm = _setup(rank, world, port)
    from loongserve_b200 import context_attention as ca
    from loongserve_b200 import ring
    from loongserve_b200.peer_ring import CopyEngineGather
    dev = torch.device("cuda", rank)
    lens = [3000, 77, 1025, 1]
    T, Hq, Hkv, D = sum(lens), 8, 4, 128
    local_len, first, stride = ring.shard_lengths(lens, world, True)
    max_tok = max(sum(x) for x in local_len)
    metas = [ring.BlockMeta.from_lengths(local_len[r], first[r], dev) for r in range(world)]
    plans = [ring.GatherPlan.build(lens, world, r, dev, parts=parts) for r in range(world)]
    gather = CopyEngineGather(rank, world, max(p.rows for p in plans) * 2 * Hkv * D * 2, _gather_over(dist, world), device=dev,
                              parts=parts)
    res = {}
    for pass_no in range(2):                  # the second pass reuses the gather buffer: credits and counters at work
        g = torch.Generator().manual_seed(pass_no)
        q = torch.randn(T, Hq, D, generator=g).to(torch.bfloat16)
        k = torch.randn(T, Hkv, D, generator=g).to(torch.bfloat16)
        v = torch.randn(T, Hkv, D, generator=g).to(torch.bfloat16)
        qs = O.shard_tokens(q, lens, world, True)[rank].to(dev)
        kv = torch.full((max_tok, 2 * Hkv, D), float("nan"), dtype=torch.bfloat16)
        kr = O.shard_tokens(k, lens, world, True)[rank]; vr = O.shard_tokens(v, lens, world, True)[rank]
        kv[:kr.shape[0], :Hkv] = kr; kv[:vr.shape[0], Hkv:] = vr
        kv = kv.to(dev)
        o = torch.empty_like(qs); m = torch.empty(qs.shape[0], Hq, device=dev); l = torch.empty(qs.shape[0], Hq, device=dev)
        ring.gathered_context_attention(qs, kv, o, m, l, rank=rank, lens=lens, P=world, metas=metas, plans=plans,
                                        max_len_in_batch=max(local_len[rank]), num_kv_heads=Hkv,
                                        attention_fn=ca.context_attention_fwd, init_fn=ca.init_attention_state, gather=gather)
        kv.fill_(float("nan"))                # what the next layer would do to the local block right after the pass
        torch.cuda.synchronize()
        res[pass_no] = dict(o=o.cpu(), lse=ca.attention_lse(m, l).cpu())
    gather.check()
    res["status"] = ca.device_status()
    assert gather.passes == 2
    dist.barrier()
    gather.close()
    torch.save(res, os.path.join(out, f"g{rank}.pt"))
    dist.barrier()
    comm.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("parts", [1, 2])
def test_gathered_pass_two_gpus(tmp_path, parts):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world = min(torch.cuda.device_count(), 4)
    mp.spawn(_gather_worker, args=(world, _free_port(), str(tmp_path), parts), nprocs=world, join=True)
    lens = [3000, 77, 1025, 1]
    T, Hq, Hkv, D = sum(lens), 8, 4, 128
    parts = [torch.load(os.path.join(str(tmp_path), f"g{r}.pt")) for r in range(world)]
    assert all(p["status"][0] == 0 for p in parts)
    for pass_no in range(2):
        g = torch.Generator().manual_seed(pass_no)
        q = torch.randn(T, Hq, D, generator=g).to(torch.bfloat16)
        k = torch.randn(T, Hkv, D, generator=g).to(torch.bfloat16)
        v = torch.randn(T, Hkv, D, generator=g).to(torch.bfloat16)
        ro, rlse = O.full_causal_attention(q, k, v, lens)
        o = O.unshard_tokens([p[pass_no]["o"] for p in parts], lens, world, True)
        lse = O.unshard_tokens([p[pass_no]["lse"] for p in parts], lens, world, True)
        assert bool(((o.float() - ro).abs() <= 2e-2 + 1e-2 * ro.abs()).all())
        assert torch.allclose(lse, rlse, atol=1e-3, rtol=1e-3)


def _host_pipeline_worker(rank, world, port, out, exchange_kind="nccl"):
    """Ring prefill from pinned host buffers, pipelined over chunks of heads, against the plain device-resident ring."""
    dist, comm = _setup(rank, world, port)
    from loongserve_b200 import context_attention as ca
    from loongserve_b200 import ring
    from loongserve_b200.host_pipeline import HostPrefillPipeline
    dev = torch.device("cuda", rank)
    g = torch.Generator().manual_seed(3)
    lens = [1500, 130]
    T, Hq, Hkv, D = sum(lens), 8, 4, 128
    q = torch.randn(T, Hq, D, generator=g).to(torch.bfloat16)
    k = torch.randn(T, Hkv, D, generator=g).to(torch.bfloat16)
    v = torch.randn(T, Hkv, D, generator=g).to(torch.bfloat16)
    local_len, first, stride = ring.shard_lengths(lens, world, True)
    max_tok = max(sum(x) for x in local_len)
    hq = O.shard_tokens(q, lens, world, True)[rank].contiguous().pin_memory()
    hkv = torch.zeros(max_tok, 2 * Hkv, D, dtype=torch.bfloat16)
    kr = O.shard_tokens(k, lens, world, True)[rank]; vr = O.shard_tokens(v, lens, world, True)[rank]
    hkv[:kr.shape[0], :Hkv] = kr; hkv[:vr.shape[0], Hkv:] = vr
    hkv = hkv.pin_memory()
    ho = torch.zeros_like(hq).pin_memory()
    metas = [ring.BlockMeta.from_lengths(local_len[r], first[r], dev) for r in range(world)]
    exchange = None
    if exchange_kind == "copy_engine":
        from loongserve_b200.peer_ring import CopyEngineRing
        exchange = CopyEngineRing(rank, world, hkv.numel() * 2, _gather_over(dist, world), device=dev)
    gather = plans = None
    if exchange_kind == "gather":
        from loongserve_b200.peer_ring import CopyEngineGather
        plans = [ring.GatherPlan.build(lens, world, r, dev) for r in range(world)]
        gather = CopyEngineGather(rank, world, max(p.rows for p in plans) * Hkv * D * 2, _gather_over(dist, world), device=dev)
    pipe = HostPrefillPipeline(hq.shape[0], max_tok, Hq, Hkv, D, rank=rank, peers=list(range(world)), metas=metas, stride=stride,
                               max_len_in_batch=max(local_len[rank]), comm=comm, head_chunks=2, device=dev, exchange=exchange,
                               gather=gather, lens=lens)
    pipe.run(hq, hkv, ho).synchronize()
    ho.zero_()
    pipe.run(hq, hkv, ho).synchronize()
    dq, dkv = hq.to(dev), hkv.to(dev)
    o = torch.empty_like(dq); m = torch.empty(dq.shape[0], Hq, device=dev); l = torch.empty(dq.shape[0], Hq, device=dev)
    if gather is not None:
        # the device-resident run of the same form (all heads at once: its own, larger gather buffer)
        big = CopyEngineGather(rank, world, max(p.rows for p in plans) * 2 * Hkv * D * 2, _gather_over(dist, world), device=dev)
        ring.gathered_context_attention(dq, dkv, o, m, l, rank=rank, lens=lens, P=world, metas=metas, plans=plans,
                                        max_len_in_batch=max(local_len[rank]), num_kv_heads=Hkv,
                                        attention_fn=ca.context_attention_fwd,
                                        init_fn=lambda o_, m_, l_: ca.init_attention_state(None, m_, l_), gather=big)
        torch.cuda.synchronize()
        big.check()
        dist.barrier()
        big.close()
    else:
        ring.ring_context_attention(dq, dkv, o, m, l, rank=rank, peers=list(range(world)), metas=metas, stride=stride,
                                    max_len_in_batch=max(local_len[rank]), num_kv_heads=Hkv, comm=comm,
                                    recv_buffers=[torch.empty_like(dkv), torch.empty_like(dkv)], attention_fn=ca.context_attention_fwd,
                                    init_fn=lambda o_, m_, l_: ca.init_attention_state(None, m_, l_))
    torch.cuda.synchronize()
    torch.save(dict(same=bool(torch.equal(ho.view(torch.int16), o.cpu().view(torch.int16))), o=ho.clone(), status=ca.device_status()),
               os.path.join(out, f"hp{rank}.pt"))
    if exchange is not None or gather is not None:
        (exchange if exchange is not None else gather).check()
        dist.barrier()
        (exchange if exchange is not None else gather).close()
    dist.barrier()
    comm.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("exchange_kind", ["nccl", "copy_engine", "gather"])
def test_host_pipeline_ring_two_gpus(tmp_path, exchange_kind):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world = 2
    mp.spawn(_host_pipeline_worker, args=(world, _free_port(), str(tmp_path), exchange_kind), nprocs=world, join=True)
    g = torch.Generator().manual_seed(3)
    lens = [1500, 130]
    T, Hq, Hkv, D = sum(lens), 8, 4, 128
    q = torch.randn(T, Hq, D, generator=g).to(torch.bfloat16)
    k = torch.randn(T, Hkv, D, generator=g).to(torch.bfloat16)
    v = torch.randn(T, Hkv, D, generator=g).to(torch.bfloat16)
    ro, _ = O.full_causal_attention(q, k, v, lens)
    parts = [torch.load(os.path.join(str(tmp_path), f"hp{r}.pt")) for r in range(world)]
    assert all(p["same"] and p["status"][0] == 0 for p in parts)
    o = O.unshard_tokens([p["o"] for p in parts], lens, world, True)
    assert bool(((o.float() - ro).abs() <= 2e-2 + 1e-2 * ro.abs()).all())


def _migrate_chunked_worker(rank, world, port, out):
    """Instance 1 hands the tail of three requests to instance 0 in chunks of at most 700 tokens: five chunks of about
    3 MB each, back to back, every one through a freshly allocated staging buffer -- the allocator gives each chunk the
    block the previous one just released, so a missing fence between the exchange stream and the kernels shows up as
    corrupted rows."""
    dist, comm = _setup(rank, world, port)
    from loongserve_b200.attention_runtime import ESPAttentionRuntime
    dev = torch.device("cuda", rank)
    L, Hkv, D = 4, 4, 128
    rt = ESPAttentionRuntime(layers_num=L, q_head_num=4, kv_head_num=Hkv, head_dim=D, max_total_token_num=8192, max_req_num=8,
                             max_seq_length=8192, sp_world_size=world, total_rank=rank, sp_comm=comm, dtype=torch.bfloat16,
                             device=dev, peer_memory_decode=False)
    lens = [1800, 900, 1200]                      # tokens instance 1 holds of each request; instance 0 holds 5 of each
    mig = [1500, 700, 1000]
    g = torch.Generator().manual_seed(11)
    rows = [torch.randn(L, n, 2 * Hkv, D, generator=g).to(torch.bfloat16) for n in lens]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    have = lens if rank == 1 else [5, 5, 5]
    for b, n in enumerate(have):
        slots = rt.mem_manager.alloc(n)
        rt.req_manager.req_to_token_indexs[b, :n] = slots.to(torch.int32)
        if rank == 1:
            rt.mem_manager.kv_buffer[:, slots] = rows[b].to(dev)
    torch.cuda.synchronize(); dist.barrier()
    new_len = rt.migrate_chunked(rank == 0, [0, 1, 2], mig, have, 1 - rank, max_mig_len=700)
    torch.cuda.synchronize()
    res = dict(new_len=new_len, free=rt.mem_manager.can_use_mem_size, state_sum=int(rt.mem_manager.mem_state.sum()))
    if rank == 0:
        got = []
        for b in range(3):
            slots = rt.req_manager.req_to_token_indexs[b, 5:5 + mig[b]].long()
            got.append(rt.mem_manager.kv_buffer[:, slots].cpu())
        res["got"] = got
    torch.save(res, os.path.join(out, f"mc{rank}.pt"))
    rt.check_device_status()
    dist.barrier()
    rt.close()
    comm.close()
    dist.destroy_process_group()


def test_migrate_chunked_many_chunks_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    mp.spawn(_migrate_chunked_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    r0 = torch.load(os.path.join(str(tmp_path), "mc0.pt")); r1 = torch.load(os.path.join(str(tmp_path), "mc1.pt"))
    lens, mig, L, Hkv, D = [1800, 900, 1200], [1500, 700, 1000], 4, 4, 128
    g = torch.Generator().manual_seed(11)
    rows = [torch.randn(L, n, 2 * Hkv, D, generator=g).to(torch.bfloat16) for n in lens]
    assert r0["new_len"] == [5 + m for m in mig] and r1["new_len"] == [n - m for n, m in zip(lens, mig)]
    assert r0["free"] == 8192 - 15 - sum(mig) and r1["free"] == 8192 - sum(lens) + sum(mig)
    assert r0["state_sum"] == 15 + sum(mig) and r1["state_sum"] == sum(lens) - sum(mig)
    # the receiver appended every request's migrated rows in their original order, bit for bit; chunks were cut from the
    # END of the request list, and each chunk takes the LAST tokens still held by the sender
    for b in range(3):
        want = rows[b][:, lens[b] - mig[b]:]
        got = r0["got"][b]
        key = lambda t: sorted(map(bytes, t.permute(1, 0, 2, 3).reshape(t.shape[1], -1).contiguous().view(torch.uint8).numpy()))
        assert key(got) == key(want), f"request {b}: migrated rows differ from the sender's originals"
