"""The runtime layer (pool slots, request table, per-layer call order) on one GPU: prefill of a varlen batch
through both slot-allocation paths, then a decode step whose new token attends to everything stored so far.
Checked against the CPU oracle's full attention."""
import pytest
import torch

from oracle import esp_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _check(o, ro):
    o = o.float().cpu(); ro = ro.float().cpu()
    assert bool(((o - ro).abs() <= 2e-2 + 1e-2 * ro.abs()).all()), (o - ro).abs().max()


@pytest.mark.parametrize("fragment_pool", [False, True])
def test_prefill_then_decode_single_instance(fragment_pool):
    from loongserve_b200.attention_runtime import ESPAttentionRuntime
    L, Hq, Hkv, D = 2, 8, 2, 128
    rt = ESPAttentionRuntime(layers_num=L, q_head_num=Hq, kv_head_num=Hkv, head_dim=D, max_total_token_num=2048,
                             max_req_num=8, max_seq_length=512, dtype=torch.bfloat16)
    if fragment_pool:
        # leave no contiguous run long enough: occupy every 64th slot
        hold = rt.mem_manager.alloc(2048)
        rt.mem_manager.free(hold[torch.arange(2048, device=DEV) % 64 != 0])
    g = torch.Generator().manual_seed(21)
    full = [301, 6, 130]                       # request lengths including the token decoded below
    pre = [n - 1 for n in full]
    B, T = len(full), sum(full)
    q = [torch.randn(T, Hq, D, generator=g).to(torch.bfloat16) for _ in range(L)]
    kv = [torch.randn(T, 2 * Hkv, D, generator=g).to(torch.bfloat16) for _ in range(L)]
    starts = [0, full[0], full[0] + full[1]]
    pre_rows = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, pre)])
    new_rows = torch.tensor([s + n - 1 for s, n in zip(starts, full)])
    b_req = rt.req_manager.alloc(B).to(torch.int32)
    b_len = torch.tensor(pre, dtype=torch.int32, device=DEV)
    b_start = (torch.cumsum(b_len, 0, dtype=torch.int32) - b_len)
    st = rt.prepare_prefill(B, sum(pre), sum(pre), max(pre), b_req, b_start, b_len, torch.zeros(B, dtype=torch.int32, device=DEV),
                            [0], 0)
    assert st.mem_is_contiguous == (not fragment_pool)
    for layer in range(L):
        rt.pre_cache_kv(st, layer)[:sum(pre)].copy_(kv[layer][pre_rows].to(DEV))
        o = rt.context_attention(q[layer][pre_rows].to(DEV), st, layer)
        ro, _ = O.full_causal_attention(q[layer][pre_rows], kv[layer][pre_rows, :Hkv], kv[layer][pre_rows, Hkv:], pre)
        _check(o, ro)
    # the request table lists exactly the allocated slots, request by request
    off = 0
    for b in range(B):
        assert torch.equal(rt.req_manager.req_to_token_indexs[int(b_req[b]), :pre[b]].long(), st.mem_index[off:off + pre[b]].long())
        off += pre[b]
    # ---- decode: one new token per request
    d_len = torch.tensor(full, dtype=torch.int32, device=DEV)
    dst = rt.prepare_decode(B, B, max(full), b_req, d_len, torch.tensor(pre, dtype=torch.int32, device=DEV), 0, [0], 0)
    assert dst.BLOCK_SEQ == 256 and dst.global_mid_o.shape == (2, B, Hq, D)
    for b in range(B):
        assert int(rt.req_manager.req_to_token_indexs[int(b_req[b]), full[b] - 1]) == int(dst.mem_index[b])
    for layer in range(L):
        rt.decode_cache_kv(dst, layer).copy_(kv[layer][new_rows].to(DEV))
        rt.post_decode_cache_kv(dst, layer)
        o = rt.token_attention(q[layer][new_rows].to(DEV), dst, layer)
        ro, rlse = O.full_causal_attention(q[layer], kv[layer][:, :Hkv], kv[layer][:, Hkv:], full)
        _check(o, ro[new_rows])
        assert torch.allclose(dst.global_out_logexpsum.cpu(), rlse[new_rows], atol=1e-3, rtol=1e-3)
    assert rt.mem_manager.can_use_mem_size == 2048 - T - (32 if fragment_pool else 0)
