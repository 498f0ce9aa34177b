"""GPU parity of the KV pool kernels (through the C ABI) against the CPU oracle and the golden vectors
from the reference's own Triton kernels.  Bit-exact."""
import os

import numpy as np
import pytest
import torch

from oracle import esp_oracle as O

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _kv():
    from loongserve_b200 import kv_ops
    return kv_ops


def test_golden_kv_ops(golden_dir):
    kv = _kv()
    g = np.load(os.path.join(golden_dir, "kv_ops.npz"))
    t = lambda n: torch.from_numpy(g[n].copy()).to(DEV)
    out = torch.zeros_like(t("dc_out"))
    kv.destindex_copy_kv(t("dc_K"), t("dc_dest"), out)
    assert torch.equal(out, t("dc_out"))
    P = int(g["cr_P"]); lens = [int(x) for x in g["cr_lens"]]
    pool = torch.zeros_like(t("cr_pool"))
    rt = torch.full_like(t("cr_req_to_tok"), O.INT32_MAX)
    cur = torch.zeros(len(lens), dtype=torch.int32, device=DEV)
    used = 0
    for r in range(P):
        llen = [max(0, (L - r + P - 1) // P) for L in lens]
        kv_len = torch.tensor(llen, dtype=torch.int32)
        kv_start = (torch.cumsum(kv_len, 0, dtype=torch.int32) - kv_len).to(DEV)
        rb, re, nl = kv.pre_copy_and_register_kv(t("cr_cache_begin"), t("cr_cache_end"),
                                                 torch.full((len(lens),), r, dtype=torch.int32, device=DEV), P)
        assert torch.equal(rb, t(f"cr_rb_{r}")) and torch.equal(re, t(f"cr_re_{r}")) and torch.equal(nl, t(f"cr_nl_{r}"))
        nls = torch.cumsum(nl, 0, dtype=torch.int64)
        kv.destindex_copy_and_register_kv(len(lens), nl, rb, re, nls, t(f"cr_kv_{r}"), kv_start, cur,
                                          t("cr_mem_index"), pool, rt, t("cr_b_req_idx"), used, max(llen) + 1, True)
        used += int(nls[-1]); cur += nl
    assert torch.equal(pool, t("cr_pool")) and torch.equal(rt, t("cr_req_to_tok")) and torch.equal(cur, t("cr_cur_idx"))
    rt = torch.full_like(t("ci_out"), O.INT32_MAX)
    kv.copy_kv_index_to_req(rt, t("ci_b_req"), t("ci_b_len"), t("ci_memidx"))
    assert torch.equal(rt, t("ci_out"))
    rt = torch.full_like(t("ii_out"), O.INT32_MAX)
    kv.init_req_to_token_indexes(rt, t("ii_b_req"), t("ii_b_len"), t("ii_alloc"))
    assert torch.equal(rt, t("ii_out"))
    send = torch.zeros_like(t("mg_send")); ms = t("mg_mem_state_in")
    kv.decoding_stage_migration_sender_kernel(send, t("mg_rt"), ms, t("mg_kvc"), t("mg_req_ids"), t("mg_ntok"), t("mg_b_len"))
    assert torch.equal(send, t("mg_send")) and torch.equal(ms, t("mg_mem_state_out"))
    kvc2 = torch.zeros_like(t("mg_kvc2")); rt2 = torch.full_like(t("mg_rt2"), O.INT32_MAX)
    kv.decoding_stage_migration_receiver_kernel(send, rt2, kvc2, t("mg_alloc"), t("mg_req_ids"), t("mg_ntok"), t("mg_b_len2"))
    assert torch.equal(kvc2, t("mg_kvc2")) and torch.equal(rt2, t("mg_rt2"))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("idx_dtype", [torch.int32, torch.int64])
def test_scatter_matches_oracle(dtype, idx_dtype):
    kv = _kv()
    g = torch.Generator().manual_seed(1)
    n, pool_sz, H2, D = 1000, 3000, 64, 128
    K = torch.randn(n, H2, D, generator=g).to(dtype)
    dest = torch.randperm(pool_sz, generator=g)[:n].to(idx_dtype)
    ref = torch.zeros(pool_sz, H2, D, dtype=dtype)
    O.destindex_copy_kv(K, dest, ref)
    out = torch.zeros(pool_sz, H2, D, dtype=dtype, device=DEV)
    kv.destindex_copy_kv(K.to(DEV), dest.to(DEV), out)
    assert torch.equal(out.cpu().view(torch.int16), ref.view(torch.int16))
    # strided source view (the K half of a [tokens, 2H, D] buffer) and empty input
    both = torch.randn(50, 2 * 8, D, generator=g).to(dtype).to(DEV)
    out2 = torch.zeros(80, 8, D, dtype=dtype, device=DEV)
    d2 = torch.randperm(80, generator=g)[:50].to(idx_dtype).to(DEV)
    kv.destindex_copy_kv(both[:, 8:, :], d2, out2)
    assert torch.equal(out2[d2.long()], both[:, 8:, :])
    kv.destindex_copy_kv(both[:0, 8:, :], d2[:0], out2)


def test_scatter_register_ring_pass_matches_oracle():
    """Config-4 style keep: several requests, every ring step of a striped pass, random keep ranges."""
    kv = _kv()
    g = torch.Generator().manual_seed(7)
    P, H2, D = 4, 8, 128
    lens = [1500, 37, 4, 2600, 1]
    B = len(lens)
    cb = torch.tensor([100, 0, 2, 1000, 0], dtype=torch.int32)
    ce = torch.tensor([1400, 37, 4, 2600, 0], dtype=torch.int32)
    n_keep = int((ce - cb).sum())
    mem_index = torch.randperm(6000, generator=g)[:n_keep].to(torch.int64)
    b_req = torch.tensor([3, 1, 0, 4, 2], dtype=torch.int32)
    pool_c = torch.zeros(6000, H2, D, dtype=torch.bfloat16); pool_g = pool_c.to(DEV)
    rt_c = torch.full((5, 3000), O.INT32_MAX, dtype=torch.int32); rt_g = rt_c.to(DEV)
    cur_c = torch.zeros(B, dtype=torch.int32); cur_g = cur_c.to(DEV)
    used = 0
    for r in range(P):
        llen = [max(0, (L - r + P - 1) // P) for L in lens]
        kvb = torch.randn(sum(llen) + 3, H2, D, generator=g).to(torch.bfloat16)
        kv_len = torch.tensor(llen, dtype=torch.int32)
        kv_start = torch.cumsum(kv_len, 0, dtype=torch.int32) - kv_len
        kvf = torch.full((B,), r, dtype=torch.int32)
        rb, re, nl = O.pre_copy_and_register_kv(cb, ce, kvf, P)
        grb, gre, gnl = kv.pre_copy_and_register_kv(cb.to(DEV), ce.to(DEV), kvf.to(DEV), P)
        assert torch.equal(grb.cpu(), rb) and torch.equal(gre.cpu(), re) and torch.equal(gnl.cpu(), nl)
        nls = torch.cumsum(nl, 0, dtype=torch.int64)
        O.destindex_copy_and_register_kv(B, nl, rb, re, nls, kvb, kv_start, cur_c, mem_index, pool_c, rt_c, b_req,
                                         used, max(llen) + 1, True)
        kv.destindex_copy_and_register_kv(B, gnl, grb, gre, nls.to(DEV), kvb.to(DEV), kv_start.to(DEV), cur_g,
                                          mem_index.to(DEV), pool_g, rt_g, b_req.to(DEV), used, max(llen) + 1, True)
        used += int(nls[-1]); cur_c += nl; cur_g += gnl
    assert used == n_keep
    assert torch.equal(pool_g.cpu().view(torch.int16), pool_c.view(torch.int16))
    assert torch.equal(rt_g.cpu(), rt_c)


def test_migration_roundtrip_full_rows():
    """gather -> scatter into a second pool reproduces the migrated tokens' rows of every layer
    (L x 16 KiB per token at the Llama-2-7B row size)."""
    kv = _kv()
    g = torch.Generator().manual_seed(9)
    L, S, H2, D = 4, 512, 64, 128
    kvc = torch.randn(L, S, H2, D, generator=g).to(torch.float16).to(DEV)
    lens = [100, 33, 250]
    rt = torch.full((4, 300), O.INT32_MAX, dtype=torch.int32)
    perm = torch.randperm(S, generator=g).to(torch.int32)
    off = 0
    for rid, n in zip([2, 0, 3], lens):
        rt[rid, :n] = perm[off:off + n]; off += n
    mem_state = torch.zeros(S, dtype=torch.int32); mem_state[perm[:off].long()] = 1
    req_ids = torch.tensor([2, 0, 3], dtype=torch.int32); ntok = torch.tensor([40, 0, 250], dtype=torch.int32)
    b_len = torch.tensor(lens, dtype=torch.int32)
    total = int(ntok.sum())
    send_c = torch.zeros(L, total, H2, D, dtype=torch.float16); ms_c = mem_state.clone()
    O.decoding_stage_migration_sender(send_c, rt, ms_c, kvc.cpu(), req_ids, ntok, b_len)
    send_g = torch.zeros(L, total, H2, D, dtype=torch.float16, device=DEV); ms_g = mem_state.to(DEV)
    kv.decoding_stage_migration_sender_kernel(send_g, rt.to(DEV), ms_g, kvc, req_ids.to(DEV), ntok.to(DEV), b_len.to(DEV),
                                              max_num_tokens=250)
    assert torch.equal(send_g.cpu(), send_c) and torch.equal(ms_g.cpu(), ms_c)
    kvc2 = torch.zeros(L, 400, H2, D, dtype=torch.float16, device=DEV)
    rt2 = torch.full((4, 600), O.INT32_MAX, dtype=torch.int32, device=DEV)
    alloc = torch.randperm(400, generator=g)[:total].to(torch.int64).to(DEV)
    b_len2 = torch.tensor([5, 9, 0], dtype=torch.int32, device=DEV)
    kv.decoding_stage_migration_receiver_kernel(send_g, rt2, kvc2, alloc, req_ids.to(DEV), ntok.to(DEV), b_len2)
    assert torch.equal(kvc2[:, alloc.long()], send_g)
    assert torch.equal(rt2[2, 5:45].long(), alloc[:40]) and torch.equal(rt2[3, 0:250].long(), alloc[40:])
