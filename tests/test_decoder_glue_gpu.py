"""The decoder-layer glue kernels (fused residual add + RMSNorm, SwiGLU gate) against fp32 torch
arithmetic with the same rounding points."""
import pytest
import torch

from async_llm_b200.decoder_glue import add_rmsnorm, silu_mul

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,dim", [(1, 256), (32, 4096), (5, 16384), (3, 2056)])
@pytest.mark.parametrize("plus_one", [False, True])
def test_add_rmsnorm(cuda_device, n, dim, plus_one):
    g = torch.Generator().manual_seed(5)
    res = torch.randn(n, dim, generator=g).to(torch.bfloat16)
    delta = torch.randn(n, dim, generator=g).to(torch.bfloat16)
    w = (torch.randn(dim, generator=g) * 0.2 + (0.0 if plus_one else 1.0)).to(torch.bfloat16)
    eps = 1e-6
    total = res.float() + delta.float()
    want_res = total.to(torch.bfloat16)
    want = (total * torch.rsqrt(total.pow(2).mean(-1, keepdim=True) + eps) * (w.float() + (1.0 if plus_one else 0.0)))
    r = res.to(cuda_device)
    out = add_rmsnorm(r, delta.to(cuda_device), w.to(cuda_device), eps, plus_one)
    torch.cuda.synchronize()
    assert torch.equal(r.cpu(), want_res)                       # the residual stream is updated in place
    torch.testing.assert_close(out.float().cpu(), want, atol=2e-2, rtol=8e-3)   # one bf16 rounding
    # without a delta: a plain norm that leaves the residual alone
    r2 = res.to(cuda_device)
    out2 = add_rmsnorm(r2, None, w.to(cuda_device), eps, plus_one)
    x = res.float()
    want2 = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * (w.float() + (1.0 if plus_one else 0.0))
    assert torch.equal(r2.cpu(), res)
    torch.testing.assert_close(out2.float().cpu(), want2, atol=2e-2, rtol=8e-3)


@pytest.mark.parametrize("n,inter", [(1, 64), (32, 12288), (7, 520)])
def test_silu_mul(cuda_device, n, inter):
    g = torch.Generator().manual_seed(6)
    gu = (torch.randn(n, 2 * inter + 16, generator=g) * 2).to(torch.bfloat16)
    rows = gu[:, : 2 * inter]                                    # rows inside a wider buffer
    want = torch.nn.functional.silu(rows[:, :inter].float()) * rows[:, inter:].float()
    out = silu_mul(gu.to(cuda_device)[:, : 2 * inter])
    torch.cuda.synchronize()
    assert out.shape == (n, inter)
    torch.testing.assert_close(out.float().cpu(), want, atol=1e-2, rtol=8e-3)
