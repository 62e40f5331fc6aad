"""Memory-bound kernels and the reference-compatible entry points against PyTorch oracles."""
import pytest
import torch

from nanotitan_b200.ops import reference as ref

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.float16, torch.bfloat16]
TOL = {torch.float32: (1e-5, 1e-5), torch.float16: (1e-2, 1e-2), torch.bfloat16: (2e-2, 2e-2)}


def _ext():
    from nanotitan_b200.ops.ext import get_ext

    return get_ext()


def _close(got, want, dtype, scale=1.0):
    rtol, atol = TOL[dtype]
    torch.testing.assert_close(got.float(), want.float(), rtol=rtol, atol=atol * scale)


# ------------------------------------------------------------------ layer norm
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,d", [(7, 7), (33, 512), (5, 1000), (64, 1024)])
def test_layer_norm_forward_backward(dtype, rows, d):
    from nanotitan_b200.ops import native

    torch.manual_seed(0)
    x = (torch.randn(rows, d, device="cuda") * 2 + 0.5).to(dtype).requires_grad_()
    g = (torch.rand(d, device="cuda") + 0.5).to(dtype).requires_grad_()
    b = torch.randn(d, device="cuda").to(dtype).requires_grad_()
    y = native.layer_norm(x, g, b, 1e-8)
    dy = torch.randn(rows, d, device="cuda").to(dtype)
    y.backward(dy)
    xf, gf, bf = (t.detach().float().requires_grad_() for t in (x, g, b))
    yf = ref.layer_norm(xf, gf, bf, 1e-8)
    yf.backward(dy.float())
    _close(y, yf, dtype, 4)
    _close(x.grad, xf.grad, dtype, 8)
    _close(g.grad, gf.grad, dtype, 4 * rows**0.5)
    _close(b.grad, bf.grad, dtype, 4 * rows**0.5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,d", [(33, 512), (257, 100), (16, 2048)])
def test_layer_norm_residual_sums_both_gradients(dtype, rows, d):
    """(norm(x), x): the gradient of the pass-through output is added to dx inside the backward kernel."""
    from nanotitan_b200.ops import native

    torch.manual_seed(3)
    x = (torch.randn(rows, d, device="cuda") * 2 + 0.5).to(dtype).requires_grad_()
    g = (torch.rand(d, device="cuda") + 0.5).to(dtype).requires_grad_()
    b = torch.randn(d, device="cuda").to(dtype).requires_grad_()
    y, xp = native.layer_norm_residual(x, g, b, 1e-8)
    assert xp.data_ptr() == x.data_ptr()
    dy = torch.randn(rows, d, device="cuda").to(dtype)
    dp = torch.randn(rows, d, device="cuda").to(dtype)
    torch.autograd.backward([y, xp], [dy, dp])
    xf, gf, bf = (t.detach().float().requires_grad_() for t in (x, g, b))
    yf = ref.layer_norm(xf, gf, bf, 1e-8)
    torch.autograd.backward([yf, xf * 1.0], [dy.float(), dp.float()])
    _close(y, yf, dtype, 4)
    _close(x.grad, xf.grad, dtype, 8)
    _close(g.grad, gf.grad, dtype, 4 * rows**0.5)
    # only one of the two outputs used downstream
    x2 = x.detach().clone().requires_grad_()
    y2, xp2 = native.layer_norm_residual(x2, g.detach(), b.detach(), 1e-8)
    xp2.backward(dp)
    torch.testing.assert_close(x2.grad, dp)


# ------------------------------------------------------------------ cross entropy
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,vocab", [(5, 11), (64, 1000), (16, 50257)])
def test_cross_entropy_forward_backward(dtype, rows, vocab):
    from nanotitan_b200.ops import native

    torch.manual_seed(1)
    logits = (torch.randn(rows, vocab, device="cuda") * 3).to(dtype).requires_grad_()
    tgt = torch.randint(0, vocab, (rows,), device="cuda")
    loss = native.cross_entropy(logits, tgt)
    loss.backward()
    lf = logits.detach().float().requires_grad_()
    want = ref.cross_entropy(lf, tgt)
    want.backward()
    torch.testing.assert_close(loss, want, rtol=1e-4, atol=1e-4)
    rtol, atol = TOL[dtype]
    torch.testing.assert_close(logits.grad.float(), lf.grad, rtol=rtol, atol=atol / rows)


def test_linear_cross_entropy_matches_unfused(monkeypatch):
    from nanotitan_b200.ops import native

    monkeypatch.delenv("NT_CE_CHUNK_ROWS", raising=False)
    torch.manual_seed(2)
    rows, d, vocab = 300, 128, 1003
    x = (torch.randn(rows, d, device="cuda") * 0.5).bfloat16().requires_grad_()
    w = (torch.randn(vocab, d, device="cuda") * 0.1).bfloat16().requires_grad_()
    tgt = torch.randint(0, vocab, (rows,), device="cuda")
    loss = native.linear_cross_entropy(x, w, tgt)
    (loss * 0.5).backward()
    xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    want = ref.linear_cross_entropy(xf, wf, tgt)
    (want * 0.5).backward()
    torch.testing.assert_close(loss, want, rtol=5e-3, atol=5e-3)
    torch.testing.assert_close(x.grad.float(), xf.grad, rtol=5e-2, atol=2e-4)
    torch.testing.assert_close(w.grad.float(), wf.grad, rtol=5e-2, atol=2e-4)


# ------------------------------------------------------------------ AdamW
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fused_adamw_tracks_torch_adamw(dtype):
    from nanotitan_b200.ops.adamw import FusedAdamW

    torch.manual_seed(3)
    shapes = [(33, 7), (128,), (5, 5, 5)]
    mine = [torch.nn.Parameter(torch.randn(s, device="cuda").to(dtype)) for s in shapes]
    theirs = [torch.nn.Parameter(p.detach().float().clone()) for p in mine]
    opt_a = FusedAdamW(mine, lr=1e-2, weight_decay=0.1)
    opt_b = torch.optim.AdamW(theirs, lr=1e-2, weight_decay=0.1)
    for step in range(4):
        opt_a.zero_grad()
        for p, q in zip(mine, theirs):
            g = torch.randn_like(q)
            q.grad = g
            if p.grad is None:
                p.grad = g.to(dtype)
            else:
                p.grad.copy_(g.to(dtype))
        opt_a.step()
        opt_b.step()
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for p, q in zip(mine, theirs):
        torch.testing.assert_close(p.detach().float(), q.detach(), rtol=tol, atol=tol)


# ------------------------------------------------------------------ router / slots
@pytest.mark.parametrize("tokens,d,E,k", [(50, 32, 4, 2), (1000, 128, 8, 2), (37, 64, 64, 8), (9, 16, 1, 1)])
def test_router_topk_matches_torch(tokens, d, E, k):
    torch.manual_seed(4)
    x = torch.randn(tokens, d, device="cuda").bfloat16()
    w = torch.randn(E, d, device="cuda") * 0.3
    gates, idx, probs, counts, probs_mean = _ext().router_topk(x, w, k)
    g_ref, e_ref, p_ref = ref.router_topk(x, w, k)
    torch.testing.assert_close(probs, p_ref, rtol=1e-4, atol=1e-5)
    assert torch.equal(idx.long().sort(dim=1).values, e_ref.sort(dim=1).values)
    torch.testing.assert_close(gates.sum(1), torch.ones(tokens, device="cuda"), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(gates, g_ref, rtol=1e-4, atol=1e-5)
    assert torch.equal(counts.long(), ref.expert_counts(e_ref, E))
    torch.testing.assert_close(probs_mean, p_ref.mean(dim=0), rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize("tokens,d,E,k", [(1000, 128, 8, 2), (4096, 512, 64, 8), (37, 64, 64, 8)])
def test_router_from_gemm_logits_matches_the_fused_router(tokens, d, E, k, monkeypatch):
    """The other way to the same five outputs: logits from two thin tcgen05 products, routing kernel on the logits.
    Runs only when asked for (NT_TEST_ROUTER_GEMM=1): `router_from_logits_kernel` has not run on a GPU yet."""
    import os

    if os.environ.get("NT_TEST_ROUTER_GEMM") != "1":
        pytest.skip("set NT_TEST_ROUTER_GEMM=1 to run the tensor-core router path")
    from nanotitan_b200.ops import native

    torch.manual_seed(4)
    x = torch.randn(tokens, d, device="cuda").bfloat16()
    w = torch.randn(E, d, device="cuda") * 0.3
    fused = _ext().router_topk(x, w, k)
    monkeypatch.setenv("NT_ROUTER_GEMM", "1")
    assert native._router_on_tensor_cores(x, w)
    split = _ext().router_from_logits(native.router_logits_tc(x, w), k)
    torch.cuda.synchronize()
    assert _ext().read_status(True)[0] == 0
    for a, b, name in zip(fused, split, ("gates", "idx", "probs", "counts", "probs_mean")):
        if name in ("idx", "counts"):
            assert (a != b).float().mean() < 2e-3, name  # a near-tie may fall the other way
        else:
            torch.testing.assert_close(a, b, rtol=2e-3, atol=2e-5, msg=lambda m, n=name: f"{n}: {m}")


def test_slots_are_expert_major_in_token_order():
    torch.manual_seed(5)
    tokens, E, k = 5000, 8, 2
    idx = torch.stack([torch.randperm(E)[:k] for _ in range(tokens)]).int().cuda()
    counts = _ext().count_expert_kernel(idx, idx.new_empty(0), E, k)
    offsets, slot_of = _ext().assign_slots(idx, counts)
    want_slot, _, _, want_counts = ref.pack_plan(idx.long(), E)
    assert torch.equal(counts.long(), want_counts)
    assert torch.equal(offsets.long(), ref.offsets_from_counts(want_counts))
    assert torch.equal(slot_of.long(), want_slot)


def test_router_autograd_matches_torch():
    from nanotitan_b200.ops import native

    torch.manual_seed(6)
    x = torch.randn(64, 32, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(4, 32, device="cuda") * 0.3).requires_grad_()
    gates, idx, probs, _ = native.router_topk(x, w, 2)
    gg, gp = torch.randn_like(gates), torch.randn_like(probs)
    ((gates * gg).sum() + (probs * gp).sum()).backward()
    xf, wf = x.detach().float().requires_grad_(), w.detach().clone().requires_grad_()
    g_ref, _, _ = ref.router_topk(xf, wf, 2)
    _, _, p_ref = ref.router_topk(xf.detach(), wf, 2)  # the aux path sees detached tokens
    ((g_ref * gg).sum() + (p_ref * gp).sum()).backward()
    torch.testing.assert_close(x.grad.float(), xf.grad, rtol=5e-2, atol=5e-3)
    torch.testing.assert_close(w.grad, wf.grad, rtol=5e-2, atol=5e-2)


@pytest.mark.parametrize("tokens,E,k", [(64, 4, 2), (300, 8, 2), (33, 16, 4)])
def test_router_mean_probability_gradient(tokens, E, k):
    """The load-balancing path: gradient through the per-expert mean probability plus the gate path."""
    from nanotitan_b200.ops import native

    torch.manual_seed(7)
    x = torch.randn(tokens, 32, device="cuda").bfloat16().requires_grad_()
    w = (torch.randn(E, 32, device="cuda") * 0.3).requires_grad_()
    gates, idx, counts, pm = native.router_topk_mean(x, w, k)
    gg, gm = torch.randn_like(gates), torch.randn_like(pm) * 10
    ((gates * gg).sum() + (pm * gm).sum()).backward()
    xf, wf = x.detach().float().requires_grad_(), w.detach().clone().requires_grad_()
    g_ref, _, _ = ref.router_topk(xf, wf, k)
    _, _, p_ref = ref.router_topk(xf.detach(), wf, k)
    ((g_ref * gg).sum() + (p_ref.mean(dim=0) * gm).sum()).backward()
    torch.testing.assert_close(pm, p_ref.mean(dim=0), rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(x.grad.float(), xf.grad, rtol=5e-2, atol=5e-3)
    torch.testing.assert_close(w.grad, wf.grad, rtol=5e-2, atol=5e-2)


# ------------------------------------------------------------------ pack / combine (reference-style API)
@pytest.mark.parametrize("dtype", DTYPES)
def test_pack_tokens_kernel_small_case(dtype):
    ext = _ext()
    x = torch.arange(4 * 6, device="cuda").reshape(4, 6).to(dtype)
    e = torch.tensor([[0, 1], [2, 0], [1, 2], [0, 2]], device="cuda", dtype=torch.int32)
    w = torch.rand(4, 2, device="cuda")
    counts = torch.bincount(e.flatten().long(), minlength=3)
    offs = torch.zeros(4, device="cuda", dtype=torch.int32)
    offs[1:] = torch.cumsum(counts, 0)
    px, ptok, pexp, pw = ext.pack_tokens_kernel(x, w, e, offs.clone())
    assert px.shape == (8, 6) and ptok.dtype == torch.int32 and pw.dtype == torch.float32
    for a in range(8):
        assert torch.equal(px[a], x[ptok[a]])
        j = (e[ptok[a]] == pexp[a]).nonzero().item()
        assert pw[a] == w[ptok[a], j]
    for ex in range(3):
        assert (pexp[offs[ex] : offs[ex + 1]] == ex).all()
        assert (ptok[offs[ex] : offs[ex + 1]].diff() > 0).all()  # ascending token ids


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tokens,k,d", [(3, 2, 8), (5, 3, 7), (64, 2, 512)])
def test_pack_combine_autograd_matches_torch(dtype, tokens, k, d):
    from nanotitan_b200.models import moe_ops

    torch.manual_seed(7)
    E = 4
    x = torch.randn(tokens, d, device="cuda").to(dtype).requires_grad_()
    w = torch.rand(tokens, k, device="cuda").requires_grad_()
    e = torch.stack([torch.randperm(E)[:k] for _ in range(tokens)]).int().cuda()
    offs = torch.zeros(E + 1, device="cuda", dtype=torch.int32)
    px, ptok, pexp, pw = moe_ops.pack_tokens_fn(x, w, e, offs)
    out = moe_ops.combine_tokens_fn(px * 1.5, ptok, pw, tokens, d)
    g = torch.randn(tokens, d, device="cuda")
    out.float().backward(g)
    xf, wf = x.detach().float().requires_grad_(), w.detach().clone().requires_grad_()
    rx, rtok, _, rw, _ = ref.pack_tokens(xf, wf, e.long(), E)
    want = ref.combine_tokens(rx * 1.5, rtok, rw, tokens, torch.float32)
    want.backward(g)
    _close(out, want, dtype, 4)
    _close(x.grad, xf.grad, dtype, 8)
    torch.testing.assert_close(w.grad, wf.grad, rtol=TOL[dtype][0], atol=TOL[dtype][1] * d**0.5 * 4)


@pytest.mark.parametrize("dtype", DTYPES)
def test_combine_tokens_kernel_returns_fp32_and_matches_python(dtype):
    ext = _ext()
    torch.manual_seed(8)
    T, k, d = 6, 2, 10
    A = T * k
    y = torch.randn(A, d, device="cuda").to(dtype)
    tok = torch.arange(T, device="cuda", dtype=torch.int32).repeat_interleave(k)[torch.randperm(A, device="cuda")]
    w = torch.rand(A, device="cuda")
    out = ext.combine_tokens_kernel(y, tok, w, T, d)
    assert out.dtype == torch.float32
    want = torch.zeros(T, d, device="cuda")
    for a in range(A):
        want[tok[a]] += w[a] * y[a].float()
    torch.testing.assert_close(out, want, rtol=1e-5, atol=1e-5)
    dy, dw = ext.combine_kernel_backward(y, tok, w, torch.ones(T, d, device="cuda"), d)
    torch.testing.assert_close(dw, y.float().sum(1), rtol=1e-4, atol=1e-4)
    _close(dy, w[:, None].expand(A, d), dtype)


# ------------------------------------------------------------------ GEMM learning kernels, copies
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("impl", [None, "tiled", "naive"])
@pytest.mark.parametrize("shape", [(33, 17, 65), (1, 1, 1), (128, 64, 32)])
def test_gemm_kernel_matches_einsum(dtype, impl, shape):
    ext = _ext()
    M, K, N = shape
    torch.manual_seed(9)
    a, b = torch.randn(M, K, device="cuda").to(dtype), torch.randn(K, N, device="cuda").to(dtype)
    c = ext.gemm_kernel(a, b) if impl is None else ext.gemm_kernel(a, b, impl)
    want = a.float() @ b.float()
    rtol, atol = {torch.float32: (1e-4, 5e-4), torch.float16: (1e-2, 1e-1), torch.bfloat16: (2e-2, 3e-1)}[dtype]
    torch.testing.assert_close(c.float(), want, rtol=rtol, atol=atol)
    torch.testing.assert_close(ext.tiled_gemm_kernel(a, b), ext.naive_gemm_kernel(a, b), rtol=rtol, atol=atol)


def test_gemm_kernel_rejects_unknown_implementation():
    a = torch.randn(4, 4, device="cuda")
    with pytest.raises(RuntimeError, match="implementation must be either 'tiled' or 'naive'"):
        _ext().gemm_kernel(a, a, "fast")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_grouped_gemm_fallback_handles_fp32_odd_shapes(dtype):
    ext = _ext()
    torch.manual_seed(10)
    off = torch.tensor([0, 3, 4, 8], device="cuda", dtype=torch.int32)
    x, w, g = (torch.randn(8, 5, device="cuda", dtype=dtype), torch.randn(3, 5, 7, device="cuda", dtype=dtype),
               torch.randn(8, 7, device="cuda", dtype=dtype))
    out, dx, dw = ext.grouped_gemm_kernel(x, off, w), ext.bwd_grouped_gemm_dX_kernel(w, off, g), ext.bwd_grouped_gemm_dW_kernel(x, off, g)
    for e in range(3):
        lo, hi = off[e].item(), off[e + 1].item()
        torch.testing.assert_close(out[lo:hi], x[lo:hi] @ w[e], rtol=1e-4, atol=1e-4)
        torch.testing.assert_close(dx[lo:hi], g[lo:hi] @ w[e].t(), rtol=1e-4, atol=1e-4)
        torch.testing.assert_close(dw[e], x[lo:hi].t() @ g[lo:hi], rtol=1e-4, atol=1e-4)


def test_copy_kernels_and_toys():
    ext = _ext()
    src = torch.randn(1000003, device="cuda")
    dst = torch.zeros_like(src)
    ext.copy_scalar(src, dst, src.numel())
    assert torch.equal(src, dst)
    b = torch.randint(0, 255, (4099,), device="cuda", dtype=torch.uint8)
    out = torch.zeros_like(b)
    ext.copy_vector(b, out)
    assert torch.equal(b, out)
    z = ext.random_op(src, 5)
    assert z.shape == (5,) and z.dtype == src.dtype and z.abs().sum() == 0
    mask = torch.tensor([1, 0, 1], device="cuda", dtype=torch.int32)
    topk = torch.tensor([[0, 1], [1, 2], [2, 2]], device="cuda", dtype=torch.int32)
    assert ext.count_expert_kernel(topk, mask, 3, 2).tolist() == [1, 1, 2]


# ------------------------------------------------------------------ device-bounded copy, status word
def test_copy_rows_prefix_copies_only_the_counted_rows():
    ext = _ext()
    src = torch.randn(100, 64, device="cuda").bfloat16()
    for n in (0, 1, 37, 100, 250):  # a count past the buffers is clamped
        dst = torch.full((100, 64), -7.0, device="cuda", dtype=torch.bfloat16)
        ext.copy_rows_prefix(src, dst, torch.tensor([n], device="cuda", dtype=torch.int32))
        k = min(n, 100)
        assert torch.equal(dst[:k], src[:k])
        assert (dst[k:] == -7.0).all()


def test_status_word_tensor_reads_the_same_word_as_read_status():
    ext = _ext()
    word = ext.status_word_tensor()
    assert word.shape == (4,) and word.dtype == torch.int32 and word.is_cuda
    assert word.tolist() == list(ext.read_status(False))
