"""Element-wise layer kernels and the Llama layer stack around the attention runtime, on one GPU: against the CPU
oracle (formulas of the reference's own op tests, tolerance rule 1e-2 + 1e-2*|x| from
longserve_cuda_kernels/test/common.py:13-29) and, in fp16, against the reference's CUDA kernels built into oracle/_ref."""
import ctypes as C
import os

import pytest
import torch

from oracle import esp_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _close(ans, std, tol=1e-2):
    ans = ans.float().cpu(); std = std.float().cpu()
    err = (ans - std).abs()
    assert bool((err <= tol + tol * torch.maximum(ans.abs(), std.abs())).all()), err.max()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_ops_match_oracle_at_the_reference_test_sizes(dtype):
    from loongserve_b200 import layer_ops as ops
    g = torch.Generator().manual_seed(0)
    # rms_norm: 105 x 1144 as in the reference's test
    x = torch.randn(105, 1144, generator=g).to(dtype); w = torch.randn(1144, generator=g).to(dtype)
    _close(ops.rms_norm(x.to(DEV), w.to(DEV), 1e-6), O.rms_norm(x, w, 1e-6), 2e-2 if dtype == torch.bfloat16 else 1e-2)
    big = torch.randn(3, 16384, generator=g).to(dtype); wb = torch.randn(16384, generator=g).to(dtype)      # beyond the register-cached row size
    _close(ops.rms_norm(big.to(DEV), wb.to(DEV), 1e-5), O.rms_norm(big, wb, 1e-5), 2e-2 if dtype == torch.bfloat16 else 1e-2)
    # rotary: value ranges of the reference's test; k is the strided K half of a [tokens, 2H, D] cache block
    T, H, D = 128, 32, 128
    q = (-2.3 + 0.5 * torch.randn(T, H, D, generator=g)).to(dtype)
    kv = (-2.3 + 0.5 * torch.randn(T, 2 * H, D, generator=g)).to(dtype)
    cos = (-1.2 + 0.5 * torch.randn(T, D // 2, generator=g)).to(dtype); sin = (-2.0 + 0.5 * torch.randn(T, D // 2, generator=g)).to(dtype)
    qg, kvg = q.to(DEV), kv.to(DEV)
    ops.rotary_emb(qg, kvg[:, :H], cos.to(DEV), sin.to(DEV))
    tol = 4e-2 if dtype == torch.bfloat16 else 1e-2
    _close(qg, O.rotary_emb(q, cos, sin), tol); _close(kvg[:, :H], O.rotary_emb(kv[:, :H], cos, sin), tol)
    assert torch.equal(kvg[:, H:].cpu(), kv[:, H:])                       # the V half is untouched
    # silu*mul
    io = torch.randn(105, 2 * 1144, generator=g).to(dtype)
    iog = io.to(DEV); ops.silu_and_mul_inplace(iog)
    _close(iog[:, :1144], O.silu_and_mul(io), 2e-2 if dtype == torch.bfloat16 else 1e-2)
    assert torch.equal(iog[:, 1144:].cpu(), io[:, 1144:])
    # ffn_block
    hid, F = 256, 512
    xe = torch.randn(37, hid, generator=g).to(dtype); nw = (1 + 0.1 * torch.randn(hid, generator=g)).to(dtype)
    gu = (0.05 * torch.randn(hid, 2 * F, generator=g)).to(dtype); dn = (0.05 * torch.randn(F, hid, generator=g)).to(dtype)
    _close(ops.ffn_block(xe.to(DEV), nw.to(DEV), 1e-5, gu.to(DEV), dn.to(DEV)), O.ffn_block(xe, nw, 1e-5, gu, dn, dtype), 3e-2)


def test_ops_match_reference_cuda_kernels_fp16():
    from loongserve_b200 import layer_ops as ops
    path = os.path.join(ROOT, "oracle", "_ref", "libref_decode.so")
    if not os.path.exists(path):
        pytest.skip("reference kernels not built (make -C oracle)")
    ref = C.CDLL(path)
    if not hasattr(ref, "ref_rms_norm"):
        pytest.skip("reference element-wise kernels not in this build of oracle/_ref")
    vp, i64, f32 = C.c_void_p, C.c_int64, C.c_float
    g = torch.Generator().manual_seed(1)
    x = torch.randn(105, 1144, generator=g).half().to(DEV); w = torch.randn(1144, generator=g).half().to(DEV)
    r = torch.empty_like(x); torch.cuda.synchronize()
    ref.ref_rms_norm(vp(r.data_ptr()), vp(x.data_ptr()), vp(w.data_ptr()), i64(105), i64(1144), f32(1e-6)); torch.cuda.synchronize()
    _close(ops.rms_norm(x, w, 1e-6), r)
    T, H, D = 64, 8, 128
    q = torch.randn(T, H, D, generator=g).half().to(DEV); cos = torch.rand(T, D // 2, generator=g).half().to(DEV); sin = torch.rand(T, D // 2, generator=g).half().to(DEV)
    r = q.clone(); torch.cuda.synchronize()
    ref.ref_rotary_emb(vp(r.data_ptr()), vp(cos.data_ptr()), vp(sin.data_ptr()), i64(r.stride(0)), i64(r.stride(1)), i64(r.stride(2)), i64(T), i64(H), i64(D))
    torch.cuda.synchronize()
    mine = q.clone(); ops.rotary_emb(mine, mine.clone(), cos, sin)
    _close(mine, r)
    io = torch.randn(50, 2 * 512, generator=g).half().to(DEV)
    r = io.clone(); torch.cuda.synchronize()
    ref.ref_silu_and_mul_inplace(vp(r.data_ptr()), i64(50), i64(512)); torch.cuda.synchronize()
    mine = io.clone(); ops.silu_and_mul_inplace(mine)
    _close(mine[:, :512], r[:, :512])


def _oracle_stack(cfg, w, ids, positions, lens, dtype):
    wl = [{k: v.cpu() for k, v in lw.items()} for lw in w.layers]
    x = w.embed.cpu()[ids.long()].float()
    for lw in wl:
        x, _, _ = O.llama_layer(x, positions, lens, lw, cfg.rms_eps, cfg.num_q_heads, cfg.num_kv_heads, cfg.head_dim, dtype)
    return x


def test_llama_stack_prefill_and_decode_single_instance():
    from loongserve_b200.attention_runtime import ESPAttentionRuntime
    from loongserve_b200.llama_stack import LlamaConfig, LlamaESPStack, LlamaWeights
    cfg = LlamaConfig(num_layers=2, hidden=512, num_q_heads=4, num_kv_heads=4, head_dim=128, ffn=1024, vocab=1000)
    dtype = torch.bfloat16
    w = LlamaWeights(cfg, dtype, DEV, seed=3)
    rt = ESPAttentionRuntime(layers_num=cfg.num_layers, q_head_num=4, kv_head_num=4, head_dim=128, max_total_token_num=2048,
                             max_req_num=8, max_seq_length=1024, dtype=dtype)
    stack = LlamaESPStack(cfg, w, rt)
    g = torch.Generator().manual_seed(5)
    full = [200, 33, 129]
    B = len(full)
    ids = torch.randint(0, cfg.vocab, (sum(full),), generator=g)
    pos = torch.cat([torch.arange(n) for n in full])
    starts = [0, full[0], full[0] + full[1]]
    pre = [n - 1 for n in full]
    pre_rows = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, pre)])
    new_rows = torch.tensor([s + n - 1 for s, n in zip(starts, full)])
    ref_x = _oracle_stack(cfg, w, ids, pos, full, dtype)
    b_req = rt.req_manager.alloc(B).to(torch.int32)
    b_len = torch.tensor(pre, dtype=torch.int32, device=DEV); b_start = torch.cumsum(b_len, 0, dtype=torch.int32) - b_len
    st = rt.prepare_prefill(B, sum(pre), sum(pre), max(pre), b_req, b_start, b_len, torch.zeros(B, dtype=torch.int32, device=DEV), [0], 0)
    x = stack.prefill(ids[pre_rows].to(DEV), pos[pre_rows].to(DEV), st)
    ref_pre = _oracle_stack(cfg, w, ids[pre_rows], pos[pre_rows], pre, dtype)
    _close(x, ref_pre, 5e-2)
    dst = rt.prepare_decode(B, B, max(full), b_req, torch.tensor(full, dtype=torch.int32, device=DEV),
                            torch.tensor(pre, dtype=torch.int32, device=DEV), 0, [0], 0)
    logits = stack.decode(ids[new_rows].to(DEV), pos[new_rows].to(DEV), dst)
    ref_h = O.rms_norm(ref_x[new_rows], w.final_norm.cpu(), cfg.rms_eps).to(dtype).float()
    ref_logits = ref_h @ w.lm_head.cpu().float()
    _close(logits, ref_logits, 5e-2)
