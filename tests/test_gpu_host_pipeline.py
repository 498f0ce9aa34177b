"""Ring prefill with pinned host buffers, pipelined over chunks of heads, against the same call on device-resident
tensors (same kernel per head, so bit-identical) and against the CPU oracle."""
import pytest
import torch

from oracle import esp_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("chunks,Hq,Hkv", [(1, 4, 4), (2, 8, 4), (4, 4, 4)])
def test_host_pipeline_single_instance_matches_device_call(chunks, Hq, Hkv):
    from loongserve_b200 import context_attention as ca
    from loongserve_b200 import ring
    from loongserve_b200.host_pipeline import HostPrefillPipeline
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(chunks)
    lens = [700, 45, 300]
    T, D = sum(lens), 128
    hq = torch.randn(T, Hq, D, generator=g).to(torch.bfloat16).pin_memory()
    hkv = torch.randn(T, 2 * Hkv, D, generator=g).to(torch.bfloat16).pin_memory()
    ho = torch.zeros(T, Hq, D, dtype=torch.bfloat16).pin_memory()
    meta = ring.BlockMeta.from_lengths(lens, [0] * len(lens), dev)
    pipe = HostPrefillPipeline(T, T, Hq, Hkv, D, rank=0, peers=[0], metas=[meta], stride=1, max_len_in_batch=max(lens),
                               head_chunks=chunks, device=dev)
    for _ in range(2):                         # twice: buffers and events are reused across runs
        ho.zero_()
        pipe.run(hq, hkv, ho).synchronize()
        q, kv = hq.to(dev), hkv.to(dev)
        o = torch.empty_like(q); m = torch.empty(T, Hq, device=dev); l = torch.empty(T, Hq, device=dev)
        ca.init_attention_state(o, m, l)
        ca.context_attention_fwd(q, kv[:, :Hkv], kv[:, Hkv:], o, meta.start_loc, meta.seq_len, meta.first_idx, meta.start_loc,
                                 meta.seq_len, meta.first_idx, 1, max(lens), m, l)
        torch.cuda.synchronize()
        assert torch.equal(ho.view(torch.int16), o.cpu().view(torch.int16))
    ro, _ = O.full_causal_attention(hq, hkv[:, :Hkv], hkv[:, Hkv:], lens)
    assert bool(((ho.float() - ro).abs() <= 2e-2 + 1e-2 * ro.abs()).all())
    assert ca.device_status()[0] == 0


def test_memcpy_2d_rejects_bad_arguments():
    from loongserve_b200 import _lib
    lib = _lib.attn()
    t = torch.zeros(64, dtype=torch.uint8, device="cuda")
    assert lib.esp_memcpy_2d(t.data_ptr(), 8, t.data_ptr(), 4, 8, 2, 2, 0) == -1                                          # spitch < width
    assert lib.esp_memcpy_2d(t.data_ptr(), 8, t.data_ptr(), 8, 8, 2, 7, 0) == -1                                         # unknown kind
    assert lib.esp_memcpy_2d(0, 8, t.data_ptr(), 8, 0, 2, 2, 0) == 0                                                     # nothing to copy
