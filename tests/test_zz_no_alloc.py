"""The allocation-free decode entry point, called through the C ABI, against the regular
stage-1 + merge entry points on the same inputs -- twice in a row with different inputs, so a result
that leaned on stale scratch contents from the previous call would show.

Who needs it: a serving worker that gave all of its device memory to the KV cache at start-up, or that
replays a fixed launch sequence, cannot call cudaMalloc for the partial (o, lse) buffers; this entry
point keeps them in a fixed array inside the library.  Collected last on purpose (file name), so that
a run stopping at the first failure has already run every other test."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _inputs(seed, B, Hq, Hkv, lens, pool, dtype):
    g = torch.Generator().manual_seed(seed)
    kv = torch.randn(pool, 2 * Hkv, 128, generator=g).to(dtype).to(DEV)
    q = torch.randn(B, Hq, 128, generator=g).to(dtype).to(DEV)
    rt = torch.full((B + 2, max(lens) + 3), 2147483647, dtype=torch.int32)
    perm = torch.randperm(pool, generator=g).to(torch.int32)
    b_req = torch.randperm(B + 2, generator=g)[:B].to(torch.int32)
    off = 0
    for b in range(B):
        rt[int(b_req[b]), :lens[b]] = perm[off:off + lens[b]]; off += lens[b]
    return kv, q, rt.to(DEV), b_req.to(DEV), torch.tensor(lens, dtype=torch.int32, device=DEV)


def _call_noalloc(lib, o, lse, q, k, v, rt, b_req, b_len, Hq, Hkv, max_len, dt, odt):
    return lib.esp_decode_attention_noalloc(
        o.data_ptr(), lse.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), k.stride(0), k.stride(1),
        v.stride(0), v.stride(1), rt.data_ptr(), rt.stride(0), b_req.data_ptr(), b_len.data_ptr(), q.shape[0], Hq,
        Hkv, 128, max_len, dt, odt, C.c_float(0.0), k.shape[0], torch.cuda.current_stream().cuda_stream)


def test_noalloc_matches_regular_entry_points_two_calls_in_a_row():
    from loongserve_b200 import _lib
    from loongserve_b200 import flash_decoding as fd
    lib = _lib.attn()
    cases = [(11, [3000, 1, 700, 0, 4097], 16, 4, torch.bfloat16), (12, [257, 5000, 64, 1024, 2], 8, 8, torch.float16)]
    for seed, lens, Hq, Hkv, dtype in cases:
        B = len(lens)
        kv, q, rt, b_req, b_len = _inputs(seed, B, Hq, Hkv, lens, sum(lens) + 50, dtype)
        k, v = kv[:, :Hkv], kv[:, Hkv:]
        mx = max(lens)
        bs = 256
        nblk = (mx + bs - 1) // bs
        mid_o = torch.empty(nblk, B, Hq, 128, device=DEV); mid_l = torch.empty(nblk, B, Hq, device=DEV)
        ref_o = torch.empty(B, Hq, 128, device=DEV); ref_l = torch.empty(B, Hq, device=DEV)
        fd.flash_decoding_stage1(mid_o, mid_l, q, k, v, rt, b_req, b_len, mx, bs)
        fd.flash_decoding_stage2(ref_o, ref_l, b_len, mid_o, mid_l, bs)
        o = torch.full((B, Hq, 128), float("nan"), device=DEV); lse = torch.full((B, Hq), float("nan"), device=DEV)
        free_before = torch.cuda.mem_get_info()[0]
        rc = _call_noalloc(lib, o, lse, q, k, v, rt, b_req, b_len, Hq, Hkv, mx, _lib.ESP_DTYPE_BF16 if dtype == torch.bfloat16 else _lib.ESP_DTYPE_F16, _lib.ESP_DTYPE_F32)
        _lib.check(rc, "esp_decode_attention_noalloc")
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] >= free_before - (1 << 20)     # no device memory was taken by the call
        assert torch.allclose(o, ref_o, atol=2e-2, rtol=1e-2), (o - ref_o).abs().max()
        fin = torch.isfinite(ref_l)
        assert torch.equal(torch.isfinite(lse), fin)
        assert torch.allclose(lse[fin], ref_l[fin], atol=1e-3, rtol=1e-3)


def test_noalloc_rejects_sizes_beyond_its_scratch():
    from loongserve_b200 import _lib
    lib = _lib.attn()
    t = torch.zeros(8, 4, 128, dtype=torch.bfloat16, device=DEV)
    f = torch.zeros(8, 4, 128, device=DEV)
    i = torch.zeros(8, dtype=torch.int32, device=DEV)
    # 4096 requests x 32 heads x 129 floats per split > 4 Mi floats: refused before anything is launched
    rc = lib.esp_decode_attention_noalloc(f.data_ptr(), f.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), 512, 128, 512, 128,
                                          i.data_ptr(), 8, i.data_ptr(), i.data_ptr(), 4096, 32, 32, 128, 100,
                                          _lib.ESP_DTYPE_BF16, _lib.ESP_DTYPE_F32, C.c_float(0.0), 8, None)
    assert rc == -7
    assert b"fixed capacity" in lib.esp_strerror(rc)
    # a negative length bound is an argument error, not a launch
    rc = lib.esp_decode_attention_noalloc(f.data_ptr(), f.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), 512, 128, 512, 128,
                                          i.data_ptr(), 8, i.data_ptr(), i.data_ptr(), 8, 4, 4, 128, -1,
                                          _lib.ESP_DTYPE_BF16, _lib.ESP_DTYPE_F32, C.c_float(0.0), 8, None)
    assert rc == -1


def test_noalloc_grows_the_split_when_the_fixed_scratch_is_small_for_the_batch():
    """Batch 64 x 32 heads leaves room for 15 splits only (4 Mi floats / (64*32*129)), so for a request of 8000 tokens
    the entry point has to use splits of 768 tokens instead of 256: the partials of all splits must still fit, and
    the result must match both the regular entry points and the CPU oracle.  Two calls in a row on different data."""
    from loongserve_b200 import _lib
    from loongserve_b200 import flash_decoding as fd
    from oracle import esp_oracle as O
    lib = _lib.attn()
    B, Hq, Hkv = 64, 32, 4
    for seed in (21, 22):
        g = torch.Generator().manual_seed(seed)
        lens = [8000] + [int(x) for x in torch.randint(1, 200, (B - 1,), generator=g)]
        lens[7] = 0
        kv, q, rt, b_req, b_len = _inputs(seed, B, Hq, Hkv, lens, sum(lens) + 9, torch.bfloat16)
        k, v = kv[:, :Hkv], kv[:, Hkv:]
        mx = max(lens)
        assert (4 * 1024 * 1024) // (B * Hq * 129) == 15 and (mx + 14) // 15 > 256       # the branch under test
        o = torch.full((B, Hq, 128), float("nan"), device=DEV); lse = torch.full((B, Hq), float("nan"), device=DEV)
        rc = _call_noalloc(lib, o, lse, q, k, v, rt, b_req, b_len, Hq, Hkv, mx, _lib.ESP_DTYPE_BF16, _lib.ESP_DTYPE_F32)
        _lib.check(rc, "esp_decode_attention_noalloc")
        bs = 768
        nblk = (mx + bs - 1) // bs
        mid_o = torch.empty(nblk, B, Hq, 128, device=DEV); mid_l = torch.empty(nblk, B, Hq, device=DEV)
        ref_o = torch.empty(B, Hq, 128, device=DEV); ref_l = torch.empty(B, Hq, device=DEV)
        fd.flash_decoding_stage1(mid_o, mid_l, q, k, v, rt, b_req, b_len, mx, bs)
        fd.flash_decoding_stage2(ref_o, ref_l, b_len, mid_o, mid_l, bs)
        torch.cuda.synchronize()
        assert torch.equal(o, ref_o) and torch.equal(lse, ref_l)           # same kernels, same split: bit-identical
        oo, ol = O.token_decode_attention(q.cpu(), k.cpu(), v.cpu(), rt.cpu(), b_req.cpu(), b_len.cpu())
        assert torch.allclose(o.cpu(), oo, atol=2e-2, rtol=1e-2)
        fin = torch.isfinite(ol)
        assert torch.equal(torch.isfinite(lse.cpu()), fin) and torch.allclose(lse.cpu()[fin], ol[fin], atol=1e-3, rtol=1e-3)
