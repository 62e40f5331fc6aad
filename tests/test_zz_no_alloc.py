"""The allocation-free LayerNorm backward, called through its exported C symbol.

Some callers of this library cannot allocate GPU memory at the point of the call (stream
capture in progress, no allocator handle, no PyTorch at all).  `nt_layer_norm_bwd_noalloc`
serves them: outputs come from the caller, scratch from a fixed array inside the library.
The test calls it twice in a row through ctypes and checks both results against the regular
entry point, which allocates its outputs and scratch through PyTorch, and against an fp32 PyTorch
statement of LayerNorm differentiated by autograd.  It lives in a file that pytest collects last so
that a run stopping at the first failure has already run everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_D = 4096


def _lib():
    from nanotitan_b200.ops import ext

    path = ext.so_path()
    assert path is not None, "extension not built"
    lib = ctypes.CDLL(str(path))
    fn = lib.nt_layer_norm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 8 + [ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                                           ctypes.c_char_p, ctypes.c_int]
    return fn


def _call(fn, dy, x, gamma, mean, rstd, dtype_code):
    dx = torch.empty_like(x)
    dgamma = torch.empty(x.shape[-1], device=x.device, dtype=torch.float32)
    dbeta = torch.empty_like(dgamma)
    err = ctypes.create_string_buffer(256)
    rows = x.numel() // x.shape[-1]
    rc = fn(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
            dgamma.data_ptr(), dbeta.data_ptr(), rows, x.shape[-1], dtype_code,
            torch.cuda.current_stream().cuda_stream, err, len(err))
    assert rc == 0, err.value.decode()
    return dx, dgamma, dbeta


def _fp32_oracle(dy, x, gamma, eps=1e-8):
    """(dx, dgamma, dbeta) of y = (x - mean) * rsqrt(var + eps) * gamma + beta by autograd, in fp32."""
    xf = x.float().requires_grad_()
    gf = gamma.float().requires_grad_()
    bf = torch.zeros_like(gf).requires_grad_()
    mean = xf.mean(dim=-1, keepdim=True)
    var = xf.var(dim=-1, keepdim=True, correction=0)
    y = (xf - mean) * torch.rsqrt(var + eps) * gf + bf
    return torch.autograd.grad(y, (xf, gf, bf), dy.float())


@pytest.mark.parametrize("dtype,code,tol", [(torch.float32, 0, 1e-5), (torch.bfloat16, 2, 2e-2)])
def test_two_calls_in_a_row_match_the_allocating_entry_point(dtype, code, tol):
    from nanotitan_b200.ops.ext import get_ext

    ext = get_ext()
    fn = _lib()
    torch.manual_seed(0)
    # consecutive calls reuse (and must clear) the same scratch; (3, 64): fewer rows than one block
    # has warps; (70, 4096): the widest row the scratch takes
    for rows, d in ((300, 512), (37, 1000), (3, 64), (70, MAX_D)):
        x = (torch.randn(rows, d, device="cuda") * 2 + 0.3).to(dtype)
        dy = torch.randn(rows, d, device="cuda").to(dtype)
        gamma = (torch.rand(d, device="cuda") + 0.5).to(dtype)
        beta = torch.zeros(d, device="cuda").to(dtype)
        _, mean, rstd = ext.layer_norm_fwd(x, gamma, beta, 1e-8)
        want_dx, want_dg, want_db = ext.layer_norm_bwd(dy, x, gamma, mean, rstd)
        dx, dg, db = _call(fn, dy, x, gamma, mean, rstd, code)
        torch.cuda.synchronize()
        scale = rows**0.5 * 4
        for ref_dx, ref_dg, ref_db in ((want_dx, want_dg, want_db), _fp32_oracle(dy, x, gamma)):
            torch.testing.assert_close(dx.float(), ref_dx.float(), rtol=tol, atol=tol * 8)
            torch.testing.assert_close(dg, ref_dg.float(), rtol=max(tol, 1e-4), atol=max(tol, 1e-4) * scale)
            torch.testing.assert_close(db, ref_db.float(), rtol=max(tol, 1e-4), atol=max(tol, 1e-4) * scale)


def test_rows_wider_than_the_scratch_are_rejected_with_a_message():
    fn = _lib()
    d = MAX_D + 8
    x = torch.zeros(2, d, device="cuda")
    stat = torch.zeros(2, device="cuda")
    out = torch.zeros(d, device="cuda")
    err = ctypes.create_string_buffer(256)
    rc = fn(x.data_ptr(), x.data_ptr(), out.data_ptr(), stat.data_ptr(), stat.data_ptr(), x.data_ptr(), out.data_ptr(),
            out.data_ptr(), 2, d, 0, None, err, len(err))
    assert rc == -2
    assert b"exceeds" in err.value
