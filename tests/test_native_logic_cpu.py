"""Host-side bookkeeping of the fused unembed + cross-entropy op, checked on CPU with stand-ins for the two
kernels it calls (their contracts, restated in PyTorch): the row panels, the padded logits buffer, the 1 / rows
scale shared by all panels and the fp32 accumulation of the weight gradient across panels."""
import pytest
import torch


def _gemm_stand_in(a, a_mn, bs, b_mn, cs, *, accumulate=False, **_):
    """C = op(A) x op(B): A is [M, K] (or [K, M] when a_mn), B is [N, K] (or [K, N] when b_mn)."""
    left = a.t() if a_mn else a
    right = bs[0] if b_mn else bs[0].t()
    out = left.float() @ right.float()
    (c,) = cs
    c.copy_((c.float() + out if accumulate else out).to(c.dtype))


class _KernelStandIn:
    """cross_entropy_fwd_bwd(logits [R, ld], targets [R], vocab, scale, _): per-row loss; the first `vocab`
    columns are overwritten with scale * (softmax - onehot)."""

    def __init__(self):
        self.panels = []

    def cross_entropy_fwd_bwd(self, logits, targets, vocab, scale, _write_grad):
        self.panels.append(tuple(logits.shape))
        z = logits[:, :vocab].float()
        logp = torch.log_softmax(z, dim=1)
        rows = torch.arange(z.shape[0])
        loss = -logp[rows, targets]
        grad = logp.exp()
        grad[rows, targets] -= 1.0
        logits[:, :vocab] = (grad * scale).to(logits.dtype)
        return loss


@pytest.mark.parametrize("rows,chunk,want_panels", [(300, 0, [300]), (300, 128, [128, 128, 44]), (256, 128, [128, 128]),
                                                    (300, 100, [128, 128, 44]), (100, 4096, [100])])
def test_unembed_loss_panels_match_the_unfused_form(monkeypatch, rows, chunk, want_panels):
    from nanotitan_b200.ops import native

    kernels = _KernelStandIn()
    monkeypatch.setattr(native, "gemm_tc", _gemm_stand_in)
    monkeypatch.setattr(native, "get_ext", lambda: kernels)
    monkeypatch.setenv("NT_CE_CHUNK_ROWS", str(chunk))
    torch.manual_seed(0)
    vocab, d = 203, 24  # the vocabulary is not a multiple of the 64-column padding
    x = torch.randn(rows, d, requires_grad=True)
    w = (torch.randn(vocab, d) * 0.3).requires_grad_()
    targets = torch.randint(0, vocab, (rows,))
    loss = native._LinearCrossEntropy.apply(x, w, targets)
    (loss * 1.7).backward()  # a scale from above must reach both gradients

    x2, w2 = x.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    want = torch.nn.functional.cross_entropy(x2 @ w2.t(), targets)
    (want * 1.7).backward()
    assert [p[0] for p in kernels.panels] == want_panels and all(p[1] == 256 for p in kernels.panels)
    torch.testing.assert_close(loss, want, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(x.grad, x2.grad, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(w.grad, w2.grad, rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize("dtype,bound", [(torch.bfloat16, 2e-4), (torch.float16, 2e-5)])
def test_two_16_bit_products_recover_the_fp32_router_logits(monkeypatch, dtype, bound):
    """The router matrix is fp32; the tensor cores take 16-bit operands.  Head + remainder keeps the logits within
    ~2^-16 of the fp32 product (one rounded product is 100x worse), so top-k picks and probabilities follow the
    fp32 router."""
    from nanotitan_b200.ops import native

    monkeypatch.setattr(native, "gemm_tc", _gemm_stand_in)
    torch.manual_seed(1)
    tokens, experts, d = 512, 64, 256
    x = torch.randn(tokens, d).to(dtype)
    w = torch.randn(experts, d) / d**0.5
    head, rest = native.split_bf16(w, dtype)
    assert head.dtype == rest.dtype == dtype
    want = x.double() @ w.double().t()
    got = native.router_logits_tc(x, w).double()
    one = (x.float() @ head.float().t()).double()
    scale = want.abs().max()
    assert (got - want).abs().max() / scale < bound
    assert (one - want).abs().max() > 30 * (got - want).abs().max()
    assert torch.equal(got.topk(8, dim=1).indices, want.topk(8, dim=1).indices) or \
        (got.topk(8, dim=1).indices != want.topk(8, dim=1).indices).float().mean() < 1e-3


def test_router_path_switch(monkeypatch):
    from nanotitan_b200.ops import native

    x = torch.zeros(16, 64)
    w = torch.zeros(8, 64)
    monkeypatch.delenv("NT_ROUTER_GEMM", raising=False)
    assert not native._router_on_tensor_cores(x, w)
    monkeypatch.setenv("NT_ROUTER_GEMM", "1")
    assert not native._router_on_tensor_cores(x, w)  # not 16-bit tensors on a GPU: stays on the fused kernel
