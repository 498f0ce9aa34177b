"""GPU parity of distributed flash-decoding (through the C ABI) against the CPU oracle, against the
reference's own CUDA kernels (compiled from the reference checkout into oracle/_ref, fp16 only) and,
at the full benchmark size, through the split-invariance property.
Tolerances: o within 2e-2 abs / 1e-2 rel, lse within 1e-3."""
import ctypes as C
import os

import pytest
import torch

from oracle import esp_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _close(o, ro, lse, rlse):
    assert torch.allclose(o.float().cpu(), ro.float().cpu(), atol=2e-2, rtol=1e-2), (o.float().cpu() - ro.float().cpu()).abs().max()
    fin = torch.isfinite(rlse.cpu())
    assert torch.equal(torch.isfinite(lse.cpu()), fin)
    assert torch.allclose(lse.cpu()[fin], rlse.cpu()[fin], atol=1e-3, rtol=1e-3), (lse.cpu()[fin] - rlse.cpu()[fin]).abs().max()


def _make(B, Hq, Hkv, D, lens, pool, dtype, seed, max_req=None, shuffled=True):
    g = torch.Generator().manual_seed(seed)
    kvbuf = torch.randn(pool, 2 * Hkv, D, generator=g).to(dtype)
    q = torch.randn(B, Hq, D, generator=g).to(dtype)
    max_req = max_req or B + 3
    rt = torch.full((max_req, max(int(max(lens)), 1) + 5), O.INT32_MAX, dtype=torch.int32)
    b_req = torch.randperm(max_req, generator=g)[:B].to(torch.int32)
    perm = (torch.randperm(pool, generator=g) if shuffled else torch.arange(pool)).to(torch.int32)
    off = 0
    for b in range(B):
        n = int(lens[b]); rt[int(b_req[b]), :n] = perm[off:off + n]; off += n
    return kvbuf, q, rt, b_req, torch.tensor(lens, dtype=torch.int32)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("Hq,Hkv", [(32, 32), (8, 2), (10, 2), (16, 2)])
@pytest.mark.parametrize("bs", [16, 256, 1000])
def test_stage1_stage2_match_oracle(dtype, Hq, Hkv, bs):
    from loongserve_b200 import flash_decoding as fd
    lens = [1, 300, 0, 257, 1025, 64]
    B, D = len(lens), 128
    kvbuf, q, rt, b_req, b_len = _make(B, Hq, Hkv, D, lens, 2000, dtype, 3)
    k, v = kvbuf[:, :Hkv], kvbuf[:, Hkv:]
    mx = max(lens); nblk = (mx + bs - 1) // bs
    mid_o = torch.zeros(nblk, B, Hq, D); mid_l = torch.zeros(nblk, B, Hq)
    O.flash_decoding_stage1(mid_o, mid_l, q, k, v, rt, b_req, b_len, mx, bs)
    g_mid_o = torch.full((nblk, B, Hq, D), float("nan"), device=DEV); g_mid_l = torch.full((nblk, B, Hq), float("nan"), device=DEV)
    kvg = kvbuf.to(DEV)
    fd.flash_decoding_stage1(g_mid_o, g_mid_l, q.to(DEV), kvg[:, :Hkv], kvg[:, Hkv:], rt.to(DEV), b_req.to(DEV),
                             b_len.to(DEV), mx, bs)
    for b in range(B):
        n = (lens[b] + bs - 1) // bs
        if n:
            _close(g_mid_o[:n, b], mid_o[:n, b], g_mid_l[:n, b], mid_l[:n, b])
        assert bool(torch.isnan(g_mid_l[n:, b]).all())          # blocks past the length are not written
    ro, rl = O.token_decode_attention(q, k, v, rt, b_req, b_len)
    for odt in (torch.float32, dtype):
        o = torch.full((B, Hq, D), 7.0, dtype=odt, device=DEV); lse = torch.full((B, Hq), 7.0, device=DEV)
        fd.flash_decoding_stage2(o, lse, b_len.to(DEV), g_mid_o, g_mid_l, bs)
        _close(o, ro, lse, rl)
        assert bool((o[2] == 0).all()) and bool(torch.isinf(lse[2]).all())   # zero-length request: (0, -inf)


def _ref_lib():
    path = os.path.join(ROOT, "oracle", "_ref", "libref_decode.so")
    if not os.path.exists(path):
        pytest.skip("reference decode kernels not built (make -C oracle)")
    return C.CDLL(path)


def test_against_reference_cuda_kernels_fp16():
    """Same inputs through the reference's flash_decoding_stage1/2 (fp16, BLOCK_SEQ <= 256) and ours."""
    from loongserve_b200 import flash_decoding as fd
    ref = _ref_lib()
    lens = [700, 1, 256, 513, 90]
    B, Hq, Hkv, D = len(lens), 16, 4, 128
    kvbuf, q, rt, b_req, b_len = _make(B, Hq, Hkv, D, lens, 2500, torch.float16, 5)
    kvg, qg, rtg, brg, blg = kvbuf.to(DEV), q.to(DEV), rt.to(DEV), b_req.to(DEV), b_len.to(DEV)
    k, v = kvg[:, :Hkv], kvg[:, Hkv:]
    mx = max(lens)
    i64, f32, vp = C.c_int64, C.c_float, C.c_void_p
    for bs in (64, 256):
        nblk = (mx + bs - 1) // bs
        r_mid_o = torch.zeros(nblk, B, Hq, D, device=DEV); r_mid_l = torch.zeros(nblk, B, Hq, device=DEV)
        torch.cuda.synchronize()
        ref.ref_flash_decoding_stage1(vp(r_mid_o.data_ptr()), vp(r_mid_l.data_ptr()), vp(qg.data_ptr()), vp(k.data_ptr()),
                                      vp(v.data_ptr()), i64(k.stride(0)), i64(k.stride(1)), i64(v.stride(0)), i64(v.stride(1)),
                                      f32(D ** -0.5), vp(rtg.data_ptr()), vp(brg.data_ptr()), vp(blg.data_ptr()), i64(B), i64(Hq),
                                      i64(Hkv), i64(nblk), i64(D), i64(rtg.shape[1]), i64(bs), i64(mx))
        r_o = torch.zeros(B, Hq, D, device=DEV); r_l = torch.zeros(B, Hq, device=DEV)
        ref.ref_flash_decoding_stage2_f32(vp(r_o.data_ptr()), vp(r_l.data_ptr()), vp(blg.data_ptr()), vp(r_mid_o.data_ptr()),
                                          vp(r_mid_l.data_ptr()), i64(B), i64(Hq), i64(nblk), i64(D), i64(bs))
        torch.cuda.synchronize()
        mid_o = torch.zeros(nblk, B, Hq, D, device=DEV); mid_l = torch.zeros(nblk, B, Hq, device=DEV)
        fd.flash_decoding_stage1(mid_o, mid_l, qg, k, v, rtg, brg, blg, mx, bs)
        o = torch.zeros(B, Hq, D, device=DEV); lse = torch.zeros(B, Hq, device=DEV)
        fd.flash_decoding_stage2(o, lse, blg, mid_o, mid_l, bs)
        for b in range(B):
            n = (lens[b] + bs - 1) // bs
            _close(mid_o[:n, b], r_mid_o[:n, b], mid_l[:n, b], r_mid_l[:n, b])
        _close(o, r_o, lse, r_l)


def test_full_size_split_invariance():
    """Benchmark-size decode (batch 64, 32 heads, bf16, lengths U[4096, 65536] scaled by 1/4 to bound
    test time and memory): the merged result does not depend on the split size, and a strided sample
    of requests matches the oracle."""
    from loongserve_b200 import flash_decoding as fd
    g = torch.Generator().manual_seed(0)
    B, H, D = 64, 32, 128
    lens = torch.randint(1024, 16385, (B,), generator=g).tolist()
    total = sum(lens)
    kvbuf = torch.randn(total + 8, 2 * H, D, generator=g, dtype=torch.float32).to(torch.bfloat16).to(DEV)
    q = torch.randn(B, H, D, generator=g).to(torch.bfloat16).to(DEV)
    rt = torch.full((B, max(lens)), O.INT32_MAX, dtype=torch.int32)
    perm = torch.randperm(total, generator=g).to(torch.int32)
    off = 0
    for b in range(B):
        rt[b, :lens[b]] = perm[off:off + lens[b]]; off += lens[b]
    rt = rt.to(DEV); b_req = torch.arange(B, dtype=torch.int32, device=DEV); b_len = torch.tensor(lens, dtype=torch.int32, device=DEV)
    k, v = kvbuf[:, :H], kvbuf[:, H:]
    outs = []
    for bs in (256, 2048, 16384):
        nblk = (max(lens) + bs - 1) // bs
        mid_o = torch.empty(nblk, B, H, D, device=DEV); mid_l = torch.empty(nblk, B, H, device=DEV)
        fd.flash_decoding_stage1(mid_o, mid_l, q, k, v, rt, b_req, b_len, max(lens), bs)
        o = torch.empty(B, H, D, device=DEV); lse = torch.empty(B, H, device=DEV)
        fd.flash_decoding_stage2(o, lse, b_len, mid_o, mid_l, bs)
        outs.append((o, lse))
    for o, lse in outs[1:]:
        assert torch.allclose(o, outs[0][0], atol=2e-3, rtol=1e-3) and torch.allclose(lse, outs[0][1], atol=1e-4, rtol=1e-5)
    sel = [0, 21, 63]
    ro, rl = O.token_decode_attention(q[sel].cpu(), k.cpu(), v.cpu(), rt.cpu(), b_req[sel].cpu(), b_len[sel].cpu())
    _close(outs[0][0][sel], ro, outs[0][1][sel], rl)
