"""tcgen05 flash attention (forward, dQ, dK/dV) against the fp32 S x S formulation."""
import math

import pytest
import torch

from nanotitan_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,S,H,Dh", [(1, 128, 1, 32), (2, 256, 3, 32), (1, 768, 2, 32), (2, 200, 2, 64), (1, 1024, 2, 64), (3, 77, 1, 32)])
def test_flash_forward_backward(dtype, B, S, H, Dh):
    from nanotitan_b200.ops import flash
    from nanotitan_b200.ops.ext import get_ext

    torch.manual_seed(0)
    q, k, v = (torch.randn(B, S, H, Dh, device="cuda").to(dtype).requires_grad_() for _ in range(3))
    assert flash.supported(q, k, v)
    scale = 1.0 / math.sqrt(Dh)
    out = flash.flash_attention(q, k, v, scale)
    g = torch.randn_like(out)
    out.backward(g)
    code, kernel, detail, count = get_ext().read_status(True)
    assert code == 0, (code, kernel, detail, count)
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    want = ref.causal_attention(qf, kf, vf, scale)
    want.backward(g.float())
    tol = 2e-2 if dtype == torch.bfloat16 else 6e-3
    torch.testing.assert_close(out.float(), want, rtol=tol, atol=tol)
    for got, exp in ((q.grad, qf.grad), (k.grad, kf.grad), (v.grad, vf.grad)):
        torch.testing.assert_close(got.float(), exp, rtol=3 * tol, atol=3 * tol * exp.abs().max().item())


def test_flash_accepts_strided_qkv_views():
    """q, k, v as column slices of one [B, S, 3*H*Dh] buffer (how a fused QKV projection hands them over)."""
    from nanotitan_b200.ops import flash

    torch.manual_seed(1)
    B, S, H, Dh = 2, 256, 4, 32
    qkv = torch.randn(B, S, 3 * H * Dh, device="cuda").bfloat16()
    q, k, v = (qkv[..., i * H * Dh : (i + 1) * H * Dh].view(B, S, H, Dh) for i in range(3))
    from nanotitan_b200.ops.ext import get_ext

    out, _ = get_ext().flash_fwd(q, k, v, 1.0 / math.sqrt(Dh))
    want = ref.causal_attention(q.float(), k.float(), v.float())
    torch.testing.assert_close(out.float(), want, rtol=2e-2, atol=2e-2)


def test_flash_is_bitwise_reproducible():
    from nanotitan_b200.ops.ext import get_ext

    torch.manual_seed(2)
    q, k, v, g = (torch.randn(2, 384, 2, 32, device="cuda").bfloat16() for _ in range(4))
    runs = []
    for _ in range(2):
        out, lse = get_ext().flash_fwd(q, k, v, 0.2)
        runs.append((out, *get_ext().flash_bwd(g, q, k, v, out, lse, 0.2)))
    for a, b in zip(*runs):
        assert torch.equal(a, b)
