"""tcgen05 GEMM against fp32 PyTorch references: every operand layout, the grouped modes,
the split sources / destinations and the fused SwiGLU epilogues."""
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = {torch.bfloat16: dict(rtol=2e-2, atol=2e-2), torch.float16: dict(rtol=1e-2, atol=1e-2)}


def _ext():
    from nanotitan_b200.ops.ext import get_ext

    return get_ext()


def _status_clean():
    code, kernel, detail, count = _ext().read_status(True)
    assert code == 0, f"device status: code={code} kernel={kernel} detail={detail} count={count}"


def _rand(*shape, dtype=torch.bfloat16, scale=1.0):
    return (torch.randn(*shape, device="cuda", dtype=torch.float32) * scale).to(dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K,bn", [(128, 256, 64, 0), (384, 512, 512, 0), (200, 328, 136, 0), (1000, 72, 264, 128), (136, 64, 64, 64)])
def test_dense_layouts(dtype, a_mn, b_mn, M, N, K, bn):
    from nanotitan_b200.ops import native

    torch.manual_seed(0)
    a = _rand(M, K, dtype=dtype)
    b = _rand(N, K, dtype=dtype)
    want = a.float() @ b.float().t()
    a_op = a.t().contiguous() if a_mn else a
    b_op = b.t().contiguous() if b_mn else b
    c = torch.full((M, N), float("nan"), device="cuda", dtype=dtype)
    native.gemm_tc(a_op, a_mn, [b_op], b_mn, [c], force_bn=bn)
    torch.cuda.synchronize()
    _status_clean()
    torch.testing.assert_close(c.float(), want, rtol=2e-2, atol=0.02 * K**0.5)


def test_fp32_output_accumulate_and_residual():
    from nanotitan_b200.ops import native

    torch.manual_seed(1)
    a, b = _rand(300, 256), _rand(192, 256)
    want = a.float() @ b.float().t()
    c32 = torch.ones(300, 192, device="cuda")
    native.gemm_tc(a, False, [b], False, [c32], accumulate=True)
    torch.testing.assert_close(c32, want + 1.0, rtol=1e-3, atol=0.05)
    res = _rand(300, 192)
    c = torch.empty(300, 192, device="cuda", dtype=torch.bfloat16)
    native.gemm_tc(a, False, [b], False, [c], aux=res)
    torch.testing.assert_close(c.float(), want + res.float(), rtol=2e-2, atol=0.3)
    _status_clean()


def test_padded_leading_dimensions_and_vocab_like_n():
    """N that is no multiple of anything (vocab 50257-like), C and A living in padded buffers."""
    from nanotitan_b200.ops import native

    torch.manual_seed(2)
    M, N, K = 256, 1001, 128
    ld = 1024
    a, w = _rand(M, K), _rand(N, K)
    buf = torch.zeros(M, ld, device="cuda", dtype=torch.bfloat16)
    native.gemm_tc(a, False, [w], False, [buf[:, :N]])
    want = a.float() @ w.float().t()
    torch.testing.assert_close(buf[:, :N].float(), want, rtol=2e-2, atol=0.25)
    assert buf[:, N:].abs().max().item() == 0
    # the padded buffer as the A operand of both gradient GEMMs
    logits = buf
    dx = torch.empty(M, K, device="cuda", dtype=torch.bfloat16)
    native.gemm_tc(logits[:, :N], False, [w], True, [dx])
    torch.testing.assert_close(dx.float(), logits[:, :N].float() @ w.float(), rtol=3e-2, atol=6.0)
    dw = torch.empty(N, K, device="cuda", dtype=torch.bfloat16)
    native.gemm_tc(logits[:, :N], True, [a], True, [dw])
    torch.testing.assert_close(dw.float(), logits[:, :N].float().t() @ a.float(), rtol=3e-2, atol=3.0)
    _status_clean()


def _offsets(counts):
    off = torch.zeros(len(counts) + 1, dtype=torch.int32)
    off[1:] = torch.cumsum(torch.tensor(counts), 0)
    return off.cuda()


@pytest.mark.parametrize("counts", [[128, 128], [3, 1, 4], [0, 300, 0, 77, 129], [513], [0], [0, 0]])
def test_grouped_forward_dgrad_wgrad(counts):
    ext = _ext()
    torch.manual_seed(3)
    E, K, N = len(counts), 64, 96
    rows = sum(counts)
    x, w, dout = _rand(rows, K), _rand(E, K, N, scale=0.2), _rand(rows, N)
    off = _offsets(counts)
    out = ext.grouped_gemm_kernel(x, off, w)
    dx = ext.bwd_grouped_gemm_dX_kernel(w, off, dout)
    dw = ext.bwd_grouped_gemm_dW_kernel(x, off, dout)
    torch.cuda.synchronize()
    _status_clean()
    lo = 0
    for e, c in enumerate(counts):
        xs, ds = x[lo : lo + c].float(), dout[lo : lo + c].float()
        torch.testing.assert_close(out[lo : lo + c].float(), xs @ w[e].float(), rtol=2e-2, atol=0.1)
        torch.testing.assert_close(dx[lo : lo + c].float(), ds @ w[e].float().t(), rtol=2e-2, atol=0.1)
        torch.testing.assert_close(dw[e].float(), xs.t() @ ds, rtol=2e-2, atol=0.02 * max(c, 1) ** 0.5 + 1e-3)
        lo += c


def test_expert_without_tokens_gets_zero_gradients():
    """A rank whose only local expert received no token this step: empty forward, zero weight gradients."""
    from nanotitan_b200.ops import native

    d, f = 128, 256
    x = torch.empty(0, d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    wg, wv = (_rand(1, d, f, scale=0.1).requires_grad_() for _ in range(2))
    wo = _rand(1, f, d, scale=0.1).requires_grad_()
    off = _offsets([0])
    y = native.swiglu_experts(x, wg, wv, wo, off)
    assert y.shape == (0, d)
    y.sum().backward()
    for w in (wg, wv, wo):
        assert w.grad is not None and torch.count_nonzero(w.grad) == 0
    _status_clean()


def test_split_sources_and_destinations():
    """QKV-style: three B sources side by side (N), stacked (K), and three C destinations."""
    from nanotitan_b200.ops import native

    torch.manual_seed(4)
    T, d, h = 384, 128, 128
    x = _rand(T, d)
    ws = [_rand(d, h, scale=0.1) for _ in range(3)]
    qkv = torch.empty(T, 3 * h, device="cuda", dtype=torch.bfloat16)
    native.gemm_tc(x, False, ws, True, [qkv], b_split=native.B_SPLIT_N)
    want = torch.cat([x.float() @ w.float() for w in ws], dim=1)
    torch.testing.assert_close(qkv.float(), want, rtol=2e-2, atol=0.1)
    dqkv = _rand(T, 3 * h)
    dx = torch.empty(T, d, device="cuda", dtype=torch.bfloat16)
    native.gemm_tc(dqkv, False, ws, False, [dx], b_split=native.B_SPLIT_K)
    want_dx = sum(dqkv[:, i * h : (i + 1) * h].float() @ ws[i].float().t() for i in range(3))
    torch.testing.assert_close(dx.float(), want_dx, rtol=2e-2, atol=0.15)
    dws = [torch.empty(d, h, device="cuda", dtype=torch.bfloat16) for _ in range(3)]
    native.gemm_tc(x, True, [dqkv], True, dws)
    for i in range(3):
        torch.testing.assert_close(dws[i].float(), x.float().t() @ dqkv[:, i * h : (i + 1) * h].float(), rtol=2e-2, atol=0.6)
    _status_clean()


@pytest.mark.parametrize("counts,d,f", [([256], 128, 256), ([100, 0, 301], 64, 192)])
def test_swiglu_experts_forward_backward(counts, d, f):
    from nanotitan_b200.ops import native
    from nanotitan_b200.ops import reference as ref

    torch.manual_seed(5)
    E, rows = len(counts), sum(counts)
    x = _rand(rows, d).requires_grad_()
    wg, wv = (_rand(E, d, f, scale=0.1).requires_grad_() for _ in range(2))
    wo = _rand(E, f, d, scale=0.1).requires_grad_()
    off = _offsets(counts)
    y = native.swiglu_experts(x, wg, wv, wo, off)
    dy = _rand(rows, d)
    y.backward(dy)
    _status_clean()
    xf, wgf, wvf, wof = (t.detach().float().requires_grad_() for t in (x, wg, wv, wo))
    yf = ref.swiglu_experts(xf, wgf, wvf, wof, off.cpu())
    yf.backward(dy.float())
    torch.testing.assert_close(y.float(), yf, rtol=3e-2, atol=0.05)
    for got, want in ((x.grad, xf.grad), (wg.grad, wgf.grad), (wv.grad, wvf.grad), (wo.grad, wof.grad)):
        torch.testing.assert_close(got.float(), want, rtol=5e-2, atol=0.05 * want.abs().max().item() + 1e-3)


def test_linear_autograd_matches_fp32():
    from nanotitan_b200.ops import native

    torch.manual_seed(6)
    x = _rand(4, 96, 256).requires_grad_()
    w = _rand(256, 320, scale=0.05).requires_grad_()
    res = _rand(4, 96, 320).requires_grad_()
    y = native.linear(x, w, res)
    g = _rand(4, 96, 320)
    y.backward(g)
    xf, wf, rf = (t.detach().float().requires_grad_() for t in (x, w, res))
    (xf @ wf + rf).backward(g.float())
    torch.testing.assert_close(y.float(), (xf @ wf + rf).detach(), rtol=2e-2, atol=0.05)
    torch.testing.assert_close(x.grad.float(), xf.grad, rtol=3e-2, atol=0.05)
    torch.testing.assert_close(w.grad.float(), wf.grad, rtol=3e-2, atol=0.3)
    torch.testing.assert_close(res.grad.float(), rf.grad)
    _status_clean()


def test_results_are_bitwise_reproducible():
    from nanotitan_b200.ops import native

    torch.manual_seed(7)
    a, b = _rand(777, 520), _rand(264, 520)
    outs = []
    for _ in range(2):
        c = torch.empty(777, 264, device="cuda", dtype=torch.bfloat16)
        native.gemm_tc(a, False, [b], False, [c])
        outs.append(c)
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (1024, 512, 512), (777, 1001, 264), (3000, 264, 136)])
def test_cta_pair_kernel_matches_reference(a_mn, b_mn, M, N, K):
    """The cta_group::2 kernel (256 x 256 tiles over two CTAs) on full and ragged tiles."""
    from nanotitan_b200.ops import native

    torch.manual_seed(8)
    pad = lambda n: (n + 7) // 8 * 8  # noqa: E731
    a = _rand(M, K)
    b = _rand(N, K, scale=0.1)
    a_op = a.t().contiguous() if a_mn else a
    if a_mn and M % 8:
        a_op = torch.zeros(K, pad(M), device="cuda", dtype=torch.bfloat16)
        a_op[:, :M] = a.t()
        a_op = a_op[:, :M]
    b_op = b
    if b_mn:
        b_op = torch.zeros(K, pad(N), device="cuda", dtype=torch.bfloat16)
        b_op[:, :N] = b.t()
        b_op = b_op[:, :N]
    outs = []
    for force in (512, -1):
        c = torch.full((M, pad(N)), float("nan"), device="cuda", dtype=torch.bfloat16)[:, :N]
        native.gemm_tc(a_op, a_mn, [b_op], b_mn, [c], force_bn=force)
        outs.append(c)
    _status_clean()
    want = a.float() @ b.float().t()
    torch.testing.assert_close(outs[0].float(), want, rtol=2e-2, atol=0.02 * K**0.5)
    assert torch.equal(outs[0], outs[1])  # same products, same accumulation order


def test_cta_pair_grouped_and_swiglu():
    from nanotitan_b200.ops import native

    torch.manual_seed(9)
    counts = [300, 0, 513, 129]
    E, d, f = len(counts), 256, 384
    rows = sum(counts)
    x = _rand(rows, d)
    wg, wv = _rand(E, d, f, scale=0.1), _rand(E, d, f, scale=0.1)
    off = _offsets(counts)
    res = []
    for force in (512, -1):
        gv = torch.zeros(rows, 2 * f, device="cuda", dtype=torch.bfloat16)
        h = torch.zeros(rows, f, device="cuda", dtype=torch.bfloat16)
        native.gemm_tc(x, False, [wg, wv], True, [gv], b_split=native.B_DUAL, mode=native.GROUPED_M, offsets=off,
                       epilogue=native.EPI_SWIGLU_FWD, aux_out=h, force_bn=force)
        dgv = torch.zeros_like(gv)
        torch.manual_seed(10)
        dy = _rand(rows, d)
        wo = _rand(E, f, d, scale=0.1)
        native.gemm_tc(dy, False, [wo], False, [dgv], mode=native.GROUPED_M, offsets=off, epilogue=native.EPI_SWIGLU_BWD,
                       aux=gv, force_bn=force)
        dx = torch.zeros(rows, d, device="cuda", dtype=torch.bfloat16)
        native.gemm_tc(dgv, False, [wg, wv], False, [dx], b_split=native.B_SPLIT_K, mode=native.GROUPED_M, offsets=off,
                       force_bn=force)
        res.append((gv, h, dgv, dx))
    _status_clean()
    for a, b in zip(*res):
        assert torch.equal(a, b)
    assert res[0][1].abs().max() > 0 and res[0][3].abs().max() > 0
