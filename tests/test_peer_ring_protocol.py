"""The flag protocol of the copy-engine ring exchange (loongserve_b200/peer_ring.py), executed on the CPU.

Every instance's ring pass is queued through the product's own ``ring_context_attention`` and ``CopyEngineRing`` with a
backend that records the operations instead of handing them to CUDA: per instance a compute queue and a copy queue,
holding flag waits, flag stores, block copies, events and the attention steps (the CPU oracle's ring step).  The queues
of all instances are then executed in many random interleavings that respect only what the real machine guarantees:
order within a stream, event waits, and flag waits.  Whatever the interleaving, the result must equal full causal
attention, no queue may get stuck, and the flags must end at the number of transfers.  A missing or wrong dependency
(a buffer refilled before it was read or forwarded, a block read before it arrived) shows up as a wrong result."""
import collections
import ctypes
import random

import pytest
import torch

from loongserve_b200 import ring
from loongserve_b200.peer_ring import CopyEngineGather, CopyEngineRing
from oracle import esp_oracle as O


class Sim:
    def __init__(self, world):
        self.queues = collections.defaultdict(list)         # (rank, stream name) -> operations in stream order
        self.events_done = set()
        self.n_events = 0

    def run(self, rng):
        live = [k for k, q in self.queues.items() if q]
        heads = {k: 0 for k in self.queues}
        while True:
            runnable = []
            for k in live:
                if heads[k] < len(self.queues[k]):
                    ready, _ = self.queues[k][heads[k]]
                    if ready():
                        runnable.append(k)
            if not runnable:
                break
            k = rng.choice(runnable)
            self.queues[k][heads[k]][1]()
            heads[k] += 1
        stuck = {k: heads[k] for k in live if heads[k] < len(self.queues[k])}
        assert not stuck, f"queues stuck at {stuck}"


class Backend:
    def __init__(self, sim, rank):
        self.sim, self.rank = sim, rank
        self.dropped_flags = set()          # stores to these addresses vanish (a fault the harness must notice)

    def compute_stream(self):
        return "compute"

    def _push(self, stream, ready, run):
        self.sim.queues[(self.rank, stream)].append((ready, run))

    @staticmethod
    def _flag(addr):
        return ctypes.c_int32.from_address(addr)

    def flag_wait(self, stream, flag_addr, value, wait_id):
        self._push(stream, lambda: self._flag(flag_addr).value >= value, lambda: None)

    def signal(self, stream, flag_addr, value):
        def run():
            if flag_addr not in self.dropped_flags:
                self._flag(flag_addr).value = value
        self._push(stream, lambda: True, run)

    def copy(self, stream, dst_addr, src_addr, nbytes):
        self._push(stream, lambda: True, lambda: ctypes.memmove(dst_addr, src_addr, nbytes))

    def copy2d(self, stream, dst_addr, dpitch, src_addr, spitch, width, rows):
        def run():
            for i in range(rows):
                ctypes.memmove(dst_addr + i * dpitch, src_addr + i * spitch, width)
        self._push(stream, lambda: True, run)

    def record(self, stream):
        self.sim.n_events += 1
        ev = self.sim.n_events
        self._push(stream, lambda: True, lambda: self.sim.events_done.add(ev))
        return ev

    def wait(self, stream, ev):
        self._push(stream, lambda: ev in self.sim.events_done, lambda: None)


def _build(world, lens, striped, seed, passes=1, hook=None):
    g = torch.Generator().manual_seed(seed)
    T, Hh, D = sum(lens), 2, 16
    local_len, first, stride = ring.shard_lengths(lens, world, striped)
    max_tok = max(sum(x) for x in local_len)
    block_bytes = max_tok * 2 * Hh * D * 4
    sim = Sim(world)
    regions = [torch.zeros(((block_bytes + 255) // 256 * 256) * 2 + 512, dtype=torch.uint8) for _ in range(world)]
    bases = [r.data_ptr() for r in regions]
    outs = []
    for p in range(passes):
        q = torch.randn(T, Hh, D, generator=g); k = torch.randn(T, Hh, D, generator=g); v = torch.randn(T, Hh, D, generator=g)
        outs.append(dict(q=q, k=k, v=v, o=[None] * world, m=[None] * world, l=[None] * world))
    rings = []
    for rank in range(world):
        bb = (block_bytes + 255) // 256 * 256
        raw = [regions[rank][i * bb:(i + 1) * bb] for i in range(2)]
        rings.append(CopyEngineRing(rank, world, block_bytes, None, device="cpu", backend=Backend(sim, rank), peer_bases=bases,
                                    raw_buffers=raw))
    keep_alive = [regions]
    if hook is not None:
        hook(rings)
    for p in range(passes):
        d = outs[p]
        for rank in range(world):
            be = rings[rank].backend
            qs = O.shard_tokens(d["q"], lens, world, striped)[rank]
            kv = torch.zeros(max_tok, 2 * Hh, D)
            ks = O.shard_tokens(d["k"], lens, world, striped)[rank]; vs = O.shard_tokens(d["v"], lens, world, striped)[rank]
            kv[:ks.shape[0], :Hh] = ks; kv[:vs.shape[0], Hh:] = vs
            metas = [ring.BlockMeta.from_lengths(local_len[r], first[r], "cpu") for r in range(world)]
            o = torch.empty_like(qs); m = torch.empty(qs.shape[0], Hh); l = torch.empty(qs.shape[0], Hh)
            d["o"][rank], d["m"][rank], d["l"][rank] = o, m, l
            keep_alive.append((qs, kv))

            def init_fn(o_, m_, l_, be=be):
                def run():
                    o_.zero_(); m_.fill_(float("-inf")); l_.zero_()
                be._push("compute", lambda: True, run)

            def attn(q_, k_, v_, o_, qs_, ql_, qf_, ks_, kl_, kf_, s_, mx_, m_, l_, be=be):
                be._push("compute", lambda: True, lambda: O.ring_step(q_, k_, v_, o_, m_, l_, qs_, ql_, qf_, ks_, kl_, kf_, s_))

            ring.ring_context_attention(qs, kv, o, m, l, rank=rank, peers=list(range(world)), metas=metas, stride=stride,
                                        max_len_in_batch=max(local_len[rank]), num_kv_heads=Hh, comm=None, recv_buffers=None,
                                        attention_fn=attn, init_fn=init_fn, exchange=rings[rank])
    return sim, rings, outs, keep_alive, (lens, striped)


@pytest.mark.parametrize("world,striped", [(2, True), (3, True), (4, True), (4, False), (8, True)])
def test_every_interleaving_gives_full_attention(world, striped):
    lens = [37, 5, 64]
    for trial in range(6):
        sim, rings, outs, keep, _ = _build(world, lens, striped, seed=trial, passes=2)
        sim.run(random.Random(1000 * world + trial))
        for d in outs:
            ro, rlse = O.full_causal_attention(d["q"], d["k"], d["v"], lens)
            o = O.unshard_tokens(d["o"], lens, world, striped)
            lse = O.unshard_tokens([O.lse_from_state(m, l) for m, l in zip(d["m"], d["l"])], lens, world, striped)
            assert torch.allclose(o, ro, atol=1e-4, rtol=1e-4)
            assert torch.allclose(lse, rlse, atol=1e-4, rtol=1e-4)
        for r in rings:                      # two passes of world-1 transfers each, all acknowledged
            nxt, prv = (r.rank + 1) % world, (r.rank - 1) % world
            assert r.sent[nxt] == r.received[prv] == r.granted[prv] == 2 * (world - 1)


def test_a_missing_credit_is_detected_as_a_stuck_queue():
    """Sanity of the harness itself: if the receiver's credits never reach the sender, the run must be reported stuck."""
    def hook(rings):
        rings[1].backend.dropped_flags.add(rings[1]._credit_flag(0, 1))      # rank 1's credit word in rank 0's region

    sim, rings, outs, keep, _ = _build(2, [16], True, seed=0, hook=hook)
    with pytest.raises(AssertionError, match="stuck"):
        sim.run(random.Random(0))


# ------------------------------------------------------------------------------------------------ gather exchange
def _build_gather(world, lens, seed, passes=2, hook=None, parts=1):
    """The same harness around ``ring.gathered_context_attention`` and ``CopyEngineGather``: every instance sends its block
    to all others (one copy queue per peer) and attends to the local block and to the gathered rows."""
    g = torch.Generator().manual_seed(seed)
    T, Hh, D = sum(lens), 2, 16
    local_len, first, stride = ring.shard_lengths(lens, world, True)
    max_tok = max(sum(x) for x in local_len)
    row_bytes = 2 * Hh * D * 4
    plans = [ring.GatherPlan.build(lens, world, r, "cpu", parts=parts) for r in range(world)]
    gbytes = (max(p.rows for p in plans) * row_bytes + 255) // 256 * 256
    sim = Sim(world)
    regions = [torch.full((gbytes + 512,), 0, dtype=torch.uint8) for _ in range(world)]
    for reg in regions:
        reg[:gbytes].view(torch.float32).fill_(float("nan"))       # a row read before it arrived poisons the result
        reg[gbytes:].zero_()
    bases = [r.data_ptr() for r in regions]
    gathers = [CopyEngineGather(rank, world, gbytes, None, device="cpu", backend=Backend(sim, rank), peer_bases=bases,
                                raw_buffer=regions[rank][:gbytes], parts=parts) for rank in range(world)]
    if hook is not None:
        hook(gathers)
    outs, keep_alive = [], [regions]
    for p in range(passes):
        q = torch.randn(T, Hh, D, generator=g); k = torch.randn(T, Hh, D, generator=g); v = torch.randn(T, Hh, D, generator=g)
        d = dict(q=q, k=k, v=v, o=[None] * world, m=[None] * world, l=[None] * world)
        outs.append(d)
        for rank in range(world):
            be = gathers[rank].backend
            qs = O.shard_tokens(q, lens, world, True)[rank]
            kv = torch.zeros(max_tok, 2 * Hh, D)
            ks = O.shard_tokens(k, lens, world, True)[rank]; vs = O.shard_tokens(v, lens, world, True)[rank]
            kv[:ks.shape[0], :Hh] = ks; kv[:vs.shape[0], Hh:] = vs
            metas = [ring.BlockMeta.from_lengths(local_len[r], first[r], "cpu") for r in range(world)]
            o = torch.empty_like(qs); m = torch.empty(qs.shape[0], Hh); l = torch.empty(qs.shape[0], Hh)
            d["o"][rank], d["m"][rank], d["l"][rank] = o, m, l
            keep_alive.append((qs, kv))

            def init_fn(o_, m_, l_, be=be):
                def run():
                    o_.zero_(); m_.fill_(float("-inf")); l_.zero_()
                be._push("compute", lambda: True, run)

            def attn(q_, k_, v_, o_, qs_, ql_, qf_, ks_, kl_, kf_, s_, mx_, m_, l_, kv_pos_stride=None, be=be):
                be._push("compute", lambda: True,
                         lambda: O.ring_step(q_, k_, v_, o_, m_, l_, qs_, ql_, qf_, ks_, kl_, kf_, s_, kv_pos_stride=kv_pos_stride))

            ring.gathered_context_attention(qs, kv, o, m, l, rank=rank, lens=lens, P=world, metas=metas, plans=plans,
                                            max_len_in_batch=max(local_len[rank]), num_kv_heads=Hh, attention_fn=attn,
                                            init_fn=init_fn, gather=gathers[rank])
            # what a serving loop does next with the local block: overwrite it (the next layer's K/V).  Queued behind the
            # pass on the compute stream, so it must not reach a copy that is still reading the block.
            be._push("compute", lambda: True, lambda kv=kv: kv.fill_(float("nan")))
    return sim, gathers, outs, keep_alive


@pytest.mark.parametrize("world,parts", [(2, 1), (3, 1), (4, 1), (8, 1), (2, 2), (3, 2), (4, 3), (8, 2)])
def test_gather_every_interleaving_gives_full_attention(world, parts):
    lens = [37, 5, 64, 1]
    for trial in range(5):
        sim, gathers, outs, keep = _build_gather(world, lens, seed=trial, passes=2, parts=parts)
        sim.run(random.Random(77 * world + trial))
        for d in outs:
            ro, rlse = O.full_causal_attention(d["q"], d["k"], d["v"], lens)
            o = O.unshard_tokens(d["o"], lens, world, True)
            lse = O.unshard_tokens([O.lse_from_state(m, l) for m, l in zip(d["m"], d["l"])], lens, world, True)
            assert torch.allclose(o, ro, atol=1e-4, rtol=1e-4)
            assert torch.allclose(lse, rlse, atol=1e-4, rtol=1e-4)
        assert all(gt.passes == 2 for gt in gathers)


def test_gather_missing_credit_is_detected_as_a_stuck_queue():
    def hook(gathers):
        gathers[1].backend.dropped_flags.add(gathers[1]._credit_flag(0, 1))
    sim, gathers, outs, keep = _build_gather(3, [16, 7], seed=0, passes=1, hook=hook)
    with pytest.raises(AssertionError, match="stuck"):
        sim.run(random.Random(0))
