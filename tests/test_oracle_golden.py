"""The CPU oracle against golden vectors produced by the reference's own code
(tests/golden/make_golden.py).  No GPU needed."""
import os

import numpy as np
import pytest
import torch

from oracle import esp_oracle as O


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def _ring_meta(lens, P, striped):
    return O.shard_request_lengths(lens, P, striped)


@pytest.mark.parametrize("name", ["ring_ref_contig_p2.npz", "ring_ref_striped_p4.npz", "ring_ref_varlen_p8.npz"])
def test_ring_step_matches_reference_kernel(golden_dir, name):
    g = _load(golden_dir, name)
    lens = [int(x) for x in g["lens"]]
    P, striped = int(g["P"]), bool(g["striped"])
    q, k, v = (torch.from_numpy(g[x]) for x in ("q", "k", "v"))
    local_len, first, stride = _ring_meta(lens, P, striped)
    qs, ks, vs = (O.shard_tokens(x, lens, P, striped) for x in (q, k, v))
    for r in range(P):
        Tq, Hq, D = qs[r].shape
        o = torch.zeros((Tq, Hq, D), dtype=torch.float16)
        m = torch.full((Tq, Hq), float("-inf"))
        l = torch.zeros((Tq, Hq))
        q_len = torch.tensor(local_len[r], dtype=torch.int32)
        q_start = torch.cumsum(q_len, 0, dtype=torch.int32) - q_len
        for i in range(P):
            src = (r - i) % P
            kv_len = torch.tensor(local_len[src], dtype=torch.int32)
            kv_start = torch.cumsum(kv_len, 0, dtype=torch.int32) - kv_len
            O.ring_step(qs[r], ks[src], vs[src], o, m, l, q_start, q_len, torch.tensor(first[r]),
                        kv_start, kv_len, torch.tensor(first[src]), stride)
            ro = torch.from_numpy(g[f"o_r{r}_s{i}"]).float()
            rm = torch.from_numpy(g[f"m_r{r}_s{i}"])
            rl = torch.from_numpy(g[f"l_r{r}_s{i}"])
            # rows the reference kernel has given a finite state so far
            seen = torch.isfinite(rm) & (rm > -1e19)
            # reference tolerance rule (ring_context_flashattention_nopad.py:419): 1e-2 + 1e-2*|x|
            err = (o.float() - ro).abs()
            tol = 1e-2 + 1e-2 * torch.maximum(o.float().abs(), ro.abs())
            assert bool((err[seen] < tol[seen]).all()), f"{name} rank {r} step {i} o max err {err[seen].max()}"
            # the running state is in the base-2 domain: compare lse = ln2*m + ln l (tolerance 1e-3 rel+abs)
            lse_o = O.lse_from_state(m, l)[seen]
            lse_r = O.lse_from_state(rm, rl)[seen]
            assert torch.allclose(lse_o, lse_r, atol=2e-3, rtol=1e-3), f"{name} rank {r} step {i} lse"
            # rows never touched keep m = -inf, l = 0 in the oracle
            assert bool((l[~torch.isfinite(m)] == 0).all())


@pytest.mark.parametrize("name", ["torch_att_varlen.npz", "torch_att_selftest_dist.npz"])
def test_full_attention_matches_torch_att(golden_dir, name):
    g = _load(golden_dir, name)
    q, k, v = (torch.from_numpy(g[x]) for x in ("q", "k", "v"))
    o, lse = O.full_causal_attention(q, k, v, g["lens"])
    ref = torch.from_numpy(g["o"])
    assert torch.allclose(o, ref, atol=2e-5, rtol=1e-4)
    assert bool(torch.isfinite(lse).all())


@pytest.mark.parametrize("P,striped", [(1, False), (2, False), (3, True), (8, True)])
def test_ring_equals_full_attention(golden_dir, P, striped):
    g = _load(golden_dir, "torch_att_varlen.npz")
    q, k, v = (torch.from_numpy(g[x]).float() for x in ("q", "k", "v"))
    lens = g["lens"]
    outs, _ = O.ring_prefill(q, k, v, lens, P, striped)
    o = O.unshard_tokens([x[0] for x in outs], lens, P, striped)
    lse = O.unshard_tokens([O.lse_from_state(x[1], x[2]) for x in outs], lens, P, striped)
    ref = torch.from_numpy(g["o"])
    _, ref_lse = O.full_causal_attention(q, k, v, lens)
    assert torch.allclose(o, ref, atol=1e-4, rtol=1e-4)
    assert torch.allclose(lse, ref_lse, atol=1e-4, rtol=1e-5)


def test_kv_ops_match_reference_kernels(golden_dir):
    g = _load(golden_dir, "kv_ops.npz")
    t = lambda n: torch.from_numpy(g[n].copy())
    # destindex_copy_kv
    out = torch.zeros_like(t("dc_out"))
    O.destindex_copy_kv(t("dc_K"), t("dc_dest"), out)
    assert torch.equal(out, t("dc_out"))
    # keep-range + scatter-and-register over a ring pass
    P = int(g["cr_P"]); lens = [int(x) for x in g["cr_lens"]]
    pool = torch.zeros_like(t("cr_pool"))
    rt = torch.full_like(t("cr_req_to_tok"), O.INT32_MAX)
    cur = torch.zeros(len(lens), dtype=torch.int32)
    used = 0
    for r in range(P):
        llen = [max(0, (L - r + P - 1) // P) for L in lens]
        kv_len = torch.tensor(llen, dtype=torch.int32)
        kv_start = torch.cumsum(kv_len, 0, dtype=torch.int32) - kv_len
        rb, re, nl = O.pre_copy_and_register_kv(t("cr_cache_begin"), t("cr_cache_end"),
                                                torch.full((len(lens),), r, dtype=torch.int32), P)
        assert torch.equal(rb, t(f"cr_rb_{r}")) and torch.equal(re, t(f"cr_re_{r}")) and torch.equal(nl, t(f"cr_nl_{r}"))
        nls = torch.cumsum(nl, 0, dtype=torch.int64)
        O.destindex_copy_and_register_kv(len(lens), nl, rb, re, nls, t(f"cr_kv_{r}"), kv_start, cur,
                                         t("cr_mem_index"), pool, rt, t("cr_b_req_idx"), used, max(llen) + 1, True)
        used += int(nls[-1]); cur += nl
    assert torch.equal(pool, t("cr_pool"))
    assert torch.equal(rt, t("cr_req_to_tok"))
    assert torch.equal(cur, t("cr_cur_idx"))
    # decode registration
    rt = torch.full_like(t("ci_out"), O.INT32_MAX)
    O.copy_kv_index_to_req(rt, t("ci_b_req"), t("ci_b_len"), t("ci_memidx"))
    assert torch.equal(rt, t("ci_out"))
    # prefill registration
    rt = torch.full_like(t("ii_out"), O.INT32_MAX)
    O.init_req_to_token_indexes(rt, t("ii_b_req"), t("ii_b_len"), t("ii_alloc"))
    assert torch.equal(rt, t("ii_out"))
    # migration
    send = torch.zeros_like(t("mg_send")); ms = t("mg_mem_state_in")
    O.decoding_stage_migration_sender(send, t("mg_rt"), ms, t("mg_kvc"), t("mg_req_ids"), t("mg_ntok"), t("mg_b_len"))
    assert torch.equal(send, t("mg_send")) and torch.equal(ms, t("mg_mem_state_out"))
    kvc2 = torch.zeros_like(t("mg_kvc2")); rt2 = torch.full_like(t("mg_rt2"), O.INT32_MAX)
    O.decoding_stage_migration_receiver(send, rt2, kvc2, t("mg_alloc"), t("mg_req_ids"), t("mg_ntok"), t("mg_b_len2"))
    assert torch.equal(kvc2, t("mg_kvc2")) and torch.equal(rt2, t("mg_rt2"))


def test_allocator_order_matches_reference(golden_dir):
    g = _load(golden_dir, "mem_manager.npz")
    mm = O.OracleMemoryManager(64)
    a = mm.alloc(5)
    assert np.array_equal(a, g["t0_alloc5"]) and mm.can_use_mem_size == int(g["t0_free"])
    b = mm.alloc_contiguous(7)
    assert np.array_equal(b[0], g["t1_contig7"]) and mm.can_use_mem_size == int(g["t1_free"])
    mm.free(a[1:4])
    assert np.array_equal(mm.mem_state, g["t2_free_a1_4"]) and mm.can_use_mem_size == int(g["t2_free"])
    c = mm.alloc(6)
    assert np.array_equal(c, g["t3_alloc6"]) and mm.can_use_mem_size == int(g["t3_free"])
    d = mm.alloc_contiguous(4)
    assert np.array_equal(d[0], g["t4_contig4"]) and mm.can_use_mem_size == int(g["t4_free"])
    mm.add_refs(c[:2])
    assert np.array_equal(mm.mem_state, g["t5_addref"]) and mm.can_use_mem_size == int(g["t5_free"])
    mm.free(c)
    assert np.array_equal(mm.mem_state, g["t6_free_c"]) and mm.can_use_mem_size == int(g["t6_free"])
    assert mm.alloc_contiguous(60) is None and int(g["t7_contig60"][0]) == -1


def test_decode_split_merge_equals_direct():
    gen = torch.Generator().manual_seed(3)
    B, Hq, Hkv, D, pool = 5, 8, 2, 128, 700
    lens = torch.tensor([1, 130, 0, 257, 64], dtype=torch.int32)
    k = torch.randn(pool, Hkv, D, generator=gen); v = torch.randn(pool, Hkv, D, generator=gen)
    q = torch.randn(B, Hq, D, generator=gen)
    rt = torch.full((8, 300), O.INT32_MAX, dtype=torch.int32)
    perm = torch.randperm(pool, generator=gen).to(torch.int32)
    b_req = torch.tensor([4, 0, 7, 2, 5], dtype=torch.int32)
    off = 0
    for b in range(B):
        n = int(lens[b]); rt[int(b_req[b]), :n] = perm[off:off + n]; off += n
    for bs in (16, 64, 256):
        nblk = (int(lens.max()) + bs - 1) // bs
        mid_o = torch.full((nblk, B, Hq, D), float("nan")); mid_l = torch.full((nblk, B, Hq), float("nan"))
        O.flash_decoding_stage1(mid_o, mid_l, q, k, v, rt, b_req, lens, int(lens.max()), bs)
        o = torch.empty(B, Hq, D); lse = torch.empty(B, Hq)
        O.flash_decoding_stage2(o, lse, lens, mid_o, mid_l, bs)
        ro, rl = O.token_decode_attention(q, k, v, rt, b_req, lens)
        assert torch.allclose(o, ro, atol=1e-5, rtol=1e-5)
        assert torch.allclose(lse, rl, atol=1e-5, rtol=1e-5)
