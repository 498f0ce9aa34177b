"""The three tcgen05.mma operand forms the prefill kernel relies on, each checked on one 128x128x128
product against fp32 matmul of the same 16-bit inputs."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("mode", [0, 1, 2])
def test_umma_forms(mode, dtype, selftest_lib):
    from loongserve_b200._util import dtype_tag
    g = torch.Generator().manual_seed(mode)
    a = torch.randn(128, 128, generator=g).to(dtype).cuda()
    b = torch.randn(128, 128, generator=g).to(dtype).cuda()
    d = torch.zeros(128, 128, device="cuda")
    rc = selftest_lib.esp_selftest_umma(a.data_ptr(), b.data_ptr(), d.data_ptr(), mode, dtype_tag(a),
                                        torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    ref = a.float() @ (b.float().t() if mode == 0 else b.float())
    assert not bool(torch.isnan(d).any()), "MMA chain timed out"
    assert torch.allclose(d, ref, atol=1e-2, rtol=1e-3), (d - ref).abs().max()
