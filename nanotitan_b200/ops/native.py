"""Autograd Functions over the `nanotitan_cuda` kernels (GPU tensors only).

GEMM-shaped work goes to the tcgen05 kernel (`gemm_tc`) whenever its operands are
bf16/fp16 with 16-byte aligned rows; operands it cannot take (fp32, odd widths) go to
cuBLAS through torch, which only happens off the benchmarked path.
"""
from __future__ import annotations

import logging
import math
import os

import torch

from nanotitan_b200.ops.ext import get_ext

logger = logging.getLogger(__name__)
_FALLBACKS_SEEN: set = set()


def library_fallback(op: str, why: str) -> None:
    """Called whenever a GPU op leaves this library's kernels for a PyTorch / cuBLAS / cuDNN one
    (operands the tcgen05 kernels cannot take: fp32, rows that are not 16-byte multiples, head sizes
    other than 32 / 64).  Never silent: logged once per (op, reason) at WARNING, and an error when
    `NT_STRICT=1` - benchmarks and the multi-GPU tests run with the native kernels only."""
    if os.environ.get("NT_STRICT", "0") == "1":
        raise RuntimeError(f"{op}: would fall back to a library kernel ({why}) and NT_STRICT=1 forbids it")
    key = (op, why)
    if key not in _FALLBACKS_SEEN:
        _FALLBACKS_SEEN.add(key)
        logger.warning("%s runs on a library kernel, not on nanotitan_cuda: %s", op, why)


DENSE, GROUPED_M, GROUPED_K = 0, 1, 2
B_ONE, B_SPLIT_N, B_SPLIT_K, B_DUAL = 0, 1, 2, 3
EPI_STORE, EPI_SWIGLU_FWD, EPI_SWIGLU_BWD = 0, 1, 2


def tc_ok(*tensors: torch.Tensor) -> bool:
    """True when every tensor can be a TMA operand of the tcgen05 GEMM."""
    for t in tensors:
        if t.dtype not in (torch.bfloat16, torch.float16) or not t.is_cuda:
            return False
        if t.stride(-1) != 1 or t.size(-1) % 8 or t.stride(-2) % 8 or t.data_ptr() % 16:
            return False
        if t.dim() == 3 and t.stride(0) % 8:
            return False
    return True


def gemm_tc(a, a_mn, bs, b_mn, cs, *, b_split=B_ONE, mode=DENSE, offsets=None, epilogue=EPI_STORE,
            accumulate=False, aux=None, aux_out=None, force_bn=0):
    get_ext().gemm_tc(a, a_mn, list(bs), b_mn, b_split, list(cs), mode, offsets, epilogue, accumulate,
                      aux, aux_out, force_bn)


def grad_buffer(w: torch.Tensor) -> torch.Tensor:
    """Where to write w's gradient: its slot in the data-parallel gradient bucket when this is the
    step's first gradient for w (autograd then adopts the tensor as `w.grad` without a copy or an
    add), else a fresh tensor."""
    sink = getattr(w, "_nt_grad_sink", None)
    if sink is not None and w.grad is None:
        out = sink()
        if out.dtype == w.dtype and out.shape == w.shape:
            return out
    return torch.empty_like(w)


def _rows(t: torch.Tensor) -> torch.Tensor:
    """2-D row-major view/copy of the leading dims."""
    t2 = t.reshape(-1, t.shape[-1])
    return t2 if t2.stride(-1) == 1 and t2.stride(0) % 8 == 0 else t2.contiguous()


# ------------------------------------------------------------------------------- linear
class _Linear(torch.autograd.Function):
    """y = x @ w (+ residual), w stored [in, out]."""

    @staticmethod
    def forward(ctx, x, w, residual):
        x2 = _rows(x)
        y = torch.empty(x2.shape[0], w.shape[1], dtype=x.dtype, device=x.device)
        res = None if residual is None else _rows(residual)
        gemm_tc(x2, False, [w], True, [y], aux=res)
        ctx.save_for_backward(x2, w)
        ctx.has_res = residual is not None
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], w.shape[1])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = _rows(dy)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x2)
            gemm_tc(dy2, False, [w], False, [dx])  # w as [N_out = in, K = out]: K-major
            dx = dx.view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            dw = grad_buffer(w)
            wgrad(x2, dy2, [dw])  # x^T dy: both operands MN-major, split over the token dim
        return dx, dw, (dy if ctx.has_res else None)


_UNIT_OFFSETS: dict = {}


def whole_segment(rows: int, device) -> torch.Tensor:
    """Offsets [0, rows]: a dense weight-gradient GEMM run as a one-segment ragged reduction, which
    lets the kernel split the long reduction over the whole GPU."""
    key = (rows, str(device))
    if key not in _UNIT_OFFSETS:
        _UNIT_OFFSETS[key] = torch.tensor([0, rows], dtype=torch.int32, device=device)
    return _UNIT_OFFSETS[key]


def wgrad(x2, dy2, outs):
    """outs[i] = x2^T @ dy2[:, i-th column block]; reduction over the (long) row dim, split-K."""
    gemm_tc(x2, True, [dy2], True, [o.unsqueeze(0) for o in outs], mode=GROUPED_K,
            offsets=whole_segment(x2.shape[0], x2.device))


class _QKVProjection(torch.autograd.Function):
    """[q | k | v] = x @ [W_Q | W_K | W_V] as one GEMM over three weight tensors; backward is one
    dgrad GEMM with the three weights stacked along the reduction and one wgrad GEMM writing the
    three weight gradients."""

    @staticmethod
    def forward(ctx, x, wq, wk, wv):
        x2 = _rows(x)
        qkv = torch.empty(x2.shape[0], 3 * wq.shape[1], dtype=x.dtype, device=x.device)
        gemm_tc(x2, False, [wq, wk, wv], True, [qkv], b_split=B_SPLIT_N)
        ctx.save_for_backward(x2, wq, wk, wv)
        ctx.x_shape = x.shape
        return qkv.view(*x.shape[:-1], qkv.shape[1])

    @staticmethod
    def backward(ctx, dqkv):
        x2, wq, wk, wv = ctx.saved_tensors
        d2 = _rows(dqkv)
        dx = torch.empty_like(x2)
        gemm_tc(d2, False, [wq, wk, wv], False, [dx], b_split=B_SPLIT_K)
        dws = [grad_buffer(w) for w in (wq, wk, wv)]
        wgrad(x2, d2, dws)
        return dx.view(ctx.x_shape), dws[0], dws[1], dws[2]


def qkv_attention(x, wq, wk, wv, heads, d_head, scale):
    """x [B, S, d] -> attention context [B, S, H*Dh] (before the output projection)."""
    from nanotitan_b200.ops import flash

    inner = heads * d_head
    fused = (tc_ok(x.reshape(-1, x.shape[-1]), wq, wk, wv) and wq.shape == wk.shape == wv.shape
             and inner % 64 == 0 and d_head in (32, 64) and hasattr(get_ext(), "flash_fwd"))
    if fused:
        qkv = _QKVProjection.apply(x, wq, wk, wv)
        return flash.flash_attention_qkv(qkv, heads, d_head, scale).reshape(*x.shape[:-1], inner)
    library_fallback("qkv_attention", f"dtype {x.dtype}, head dim {d_head}, inner width {inner}: needs bf16/fp16, head dim 32 or 64")
    b, s, _ = x.shape
    q, k, v = (linear(x, w).view(b, s, heads, d_head) for w in (wq, wk, wv))
    return causal_attention(q, k, v, scale).reshape(b, s, inner)


def linear(x, w, residual=None):
    if tc_ok(x.reshape(-1, x.shape[-1]), w) and w.dim() == 2:
        return _Linear.apply(x, w, residual)
    library_fallback("linear", f"operands {tuple(x.shape)} {x.dtype} x {tuple(w.shape)} {w.dtype} are not TMA-addressable 16-bit matrices")
    y = x @ w
    return y if residual is None else y + residual


# ------------------------------------------------------------------------------- layer norm
def _ln_backward(ctx, dy, x, gamma, mean, rstd, dres):
    """(dx, dgamma, dbeta); the parameter gradients are folded straight into the parameters' dtype
    and, on a step's first gradient, into their slots of the gradient bucket."""
    gamma_p, beta_p = ctx.params
    dg, db = grad_buffer(gamma_p), grad_buffer(beta_p)
    if not (dg.is_contiguous() and db.is_contiguous()):
        dg, db = torch.empty_like(gamma_p), torch.empty_like(beta_p)
    dx, dg, db = get_ext().layer_norm_bwd(dy.contiguous(), x, gamma.contiguous(), mean, rstd, dres, dg, db)
    return dx, dg, db


class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, eps):
        xc = x.contiguous()
        y, mean, rstd = get_ext().layer_norm_fwd(xc, gamma.contiguous(), beta.contiguous(), eps)
        ctx.save_for_backward(xc, gamma, mean, rstd)
        ctx.params = (gamma, beta)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, gamma, mean, rstd = ctx.saved_tensors
        return (*_ln_backward(ctx, dy, x, gamma, mean, rstd, None), None)


def layer_norm(x, gamma, beta, eps=1e-8):
    if gamma.dtype != x.dtype:
        gamma, beta = gamma.to(x.dtype), beta.to(x.dtype)
    return _LayerNorm.apply(x, gamma, beta, eps)


class _LayerNormResidual(torch.autograd.Function):
    """(LayerNorm(x), x) for a pre-norm residual block `x + f(LayerNorm(x))`: the second output is x
    itself, routed through this node so that backward receives the residual path's gradient next
    to the normalised path's and writes their sum in the LayerNorm-backward kernel (autograd would
    otherwise add the two with a separate element-wise pass)."""

    @staticmethod
    def forward(ctx, x, gamma, beta, eps):
        xc = x.contiguous()
        y, mean, rstd = get_ext().layer_norm_fwd(xc, gamma.contiguous(), beta.contiguous(), eps)
        ctx.save_for_backward(xc, gamma, mean, rstd)
        ctx.params = (gamma, beta)
        return y, xc.view_as(xc)

    @staticmethod
    def backward(ctx, dy, dpass):
        x, gamma, mean, rstd = ctx.saved_tensors
        if dy is None:
            return dpass, None, None, None
        dres = None if dpass is None else dpass.contiguous()
        return (*_ln_backward(ctx, dy, x, gamma, mean, rstd, dres), None)


def layer_norm_residual(x, gamma, beta, eps=1e-8):
    if gamma.dtype != x.dtype:
        gamma, beta = gamma.to(x.dtype), beta.to(x.dtype)
    return _LayerNormResidual.apply(x, gamma, beta, eps)


# ------------------------------------------------------------------------------- attention
def causal_attention(q, k, v, scale=None):
    """[B, S, H, Dh] causal attention on the tcgen05 flash kernels."""
    from nanotitan_b200.ops import attention

    return attention.causal_attention(q, k, v, scale)


# ------------------------------------------------------------------------------- loss
class _CrossEntropy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets):
        rows = logits.reshape(-1, logits.shape[-1])
        work = rows.clone() if rows.stride(-1) == 1 else rows.contiguous()
        n = max(int(work.shape[0]), 1)
        row_loss = get_ext().cross_entropy_fwd_bwd(work, targets.reshape(-1).contiguous(), work.shape[1], 1.0 / n, True)
        ctx.save_for_backward(work)
        ctx.shape = logits.shape
        return row_loss.sum() / n

    @staticmethod
    def backward(ctx, g):
        (dlogits,) = ctx.saved_tensors
        return (dlogits * g.to(dlogits.dtype)).view(ctx.shape), None


def cross_entropy(logits, targets):
    return _CrossEntropy.apply(logits, targets)


def _ce_chunk_rows() -> int:
    """Rows per panel of the unembed + loss op (`NT_CE_CHUNK_ROWS`, 0 = one panel).  One panel is the
    fastest form and keeps a [rows, vocab] bf16 buffer alive for the duration of the op (3.1 GB at
    30720 x 50304); panels of e.g. 4096 rows bound that buffer (0.41 GB) at the price of accumulating
    the weight gradient in fp32 across panels."""
    try:
        return max(0, int(os.environ.get("NT_CE_CHUNK_ROWS", "0")))
    except ValueError:
        return 0


class _LinearCrossEntropy(torch.autograd.Function):
    """mean CE(x @ w^T, targets) with w [V, d].  The bf16 logits of a panel of rows live in one padded
    buffer that the loss kernel overwrites with their gradient; dx and dw are formed at once, so
    backward only scales them.  With several panels the buffer is reused and dw accumulates in fp32."""

    @staticmethod
    def forward(ctx, x, w, targets):
        ext = get_ext()
        rows, vocab = x.shape[0], w.shape[0]
        ld = (vocab + 63) // 64 * 64
        panel = _ce_chunk_rows()
        panel = rows if panel <= 0 or panel >= rows else (panel + 127) // 128 * 128
        targets = targets.contiguous()
        logits = torch.empty(min(panel, rows), ld, dtype=x.dtype, device=x.device)
        dx = torch.empty_like(x)
        inv_rows = 1.0 / max(rows, 1)
        if panel >= rows:
            view = logits[:, :vocab]
            gemm_tc(x, False, [w], False, [view])  # w [V, d]: K-major B
            row_loss = ext.cross_entropy_fwd_bwd(logits, targets, vocab, inv_rows, True)
            loss = row_loss.sum() * inv_rows
            gemm_tc(view, False, [w], True, [dx])  # reduction over V: w [V, d] is MN-major here
            dw = torch.empty_like(w)
            gemm_tc(view, True, [x], True, [dw])  # dlogits^T x
        else:
            dw32 = torch.empty(w.shape, dtype=torch.float32, device=x.device)
            loss_sum = torch.zeros((), dtype=torch.float32, device=x.device)
            for lo in range(0, rows, panel):
                hi = min(rows, lo + panel)
                view = logits[: hi - lo, :vocab]
                xs = x[lo:hi]
                gemm_tc(xs, False, [w], False, [view])
                loss_sum += ext.cross_entropy_fwd_bwd(logits[: hi - lo], targets[lo:hi], vocab, inv_rows, True).sum()
                gemm_tc(view, False, [w], True, [dx[lo:hi]])
                gemm_tc(view, True, [xs], True, [dw32], accumulate=lo > 0)
            loss = loss_sum * inv_rows
            dw = dw32.to(w.dtype)
        ctx.save_for_backward(dx, dw, w)
        return loss

    @staticmethod
    def backward(ctx, g):
        dx, dw, w = ctx.saved_tensors
        return dx * g.to(dx.dtype), torch.mul(dw, g.to(dw.dtype), out=grad_buffer(w)), None


def linear_cross_entropy(x, w_unembed, targets):
    x2 = _rows(x)
    if tc_ok(x2, w_unembed):
        return _LinearCrossEntropy.apply(x2, w_unembed, targets.reshape(-1))
    library_fallback("linear_cross_entropy", f"operands {tuple(x2.shape)} {x2.dtype} x {tuple(w_unembed.shape)} are not TMA-addressable 16-bit matrices")
    return cross_entropy(x2 @ w_unembed.t(), targets.reshape(-1))


# ------------------------------------------------------------------------------- MoE routing
def split_bf16(w: torch.Tensor, dtype: torch.dtype) -> tuple[torch.Tensor, torch.Tensor]:
    """w = head + remainder with both parts in a 16-bit `dtype`: the head is w rounded, the remainder what the
    rounding lost, rounded again.  Two 16-bit products then give x . w to about 2^-16 of |x||w| instead of the
    2^-8 (bf16) or 2^-11 (fp16) of one."""
    head = w.to(dtype)
    return head, (w.float() - head.float()).to(dtype)


def router_logits_tc(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """fp32 router logits x . w^T [T, E] on the tcgen05 GEMM from 16-bit tokens and the fp32 router matrix: two
    thin products (head and remainder of w) accumulated in fp32."""
    head, rest = split_bf16(w, x.dtype)
    logits = torch.empty(x.shape[0], w.shape[0], dtype=torch.float32, device=x.device)
    gemm_tc(x, False, [head], False, [logits])
    gemm_tc(x, False, [rest], False, [logits], accumulate=True)
    return logits


def _router_on_tensor_cores(x: torch.Tensor, w: torch.Tensor) -> bool:
    """`NT_ROUTER_GEMM=1`: form the router logits with the GEMM kernel instead of inside `router_topk`, which
    reads the router matrix once per group of four tokens - fine for 8 experts x 512, slow for 64 x 2048."""
    if os.environ.get("NT_ROUTER_GEMM", "0") != "1":
        return False
    return x.dim() == 2 and tc_ok(x) and w.dim() == 2 and w.shape[0] % 8 == 0 and w.shape[1] % 8 == 0 and x.shape[0] > 0


class _Router(torch.autograd.Function):
    """Fused fp32 router.  Outputs: gates [T,k] (grad -> x and w), ids [T,k], probs [T,E] and their
    column means [E], counts [E].  The gradient of the probabilities (the load-balancing loss) reaches
    w only when `aux_to_tokens` is false - the loss then sees detached tokens, as in the reference's
    CUDA backend (src/model/cuda_backend.py:39-41) - and also x when it is true, as in its torch
    backend (src/model/torch_backend.py:153-155)."""

    @staticmethod
    def forward(ctx, x, w, k, aux_to_tokens=False):
        if _router_on_tensor_cores(x, w):
            gates, idx, probs, counts, probs_mean = get_ext().router_from_logits(router_logits_tc(x, w), k)
        else:
            gates, idx, probs, counts, probs_mean = get_ext().router_topk(x.contiguous(), w.contiguous(), k)
        ctx.save_for_backward(x, w, gates, idx, probs)
        ctx.aux_to_tokens = aux_to_tokens
        ctx.mark_non_differentiable(idx, counts)
        return gates, idx, probs, counts, probs_mean

    @staticmethod
    def backward(ctx, dgates, _didx, dprobs, _dcounts, dprobs_mean):
        x, w, gates, idx, probs = ctx.saved_tensors

        def f32(t):
            return None if t is None else t.float().contiguous()

        # softmax / top-k / renormalise backward in one kernel, then two thin products on the tcgen05 GEMM
        dl_tok, dl_all = get_ext().router_bwd(gates, idx, probs, f32(dgates), f32(dprobs), f32(dprobs_mean), x)
        dl_x = dl_all if ctx.aux_to_tokens else dl_tok
        dx = dw = None
        thin = x.dim() == 2 and tc_ok(x, dl_x) and dl_x.shape[1] % 8 == 0
        if ctx.needs_input_grad[0]:
            w16 = w.to(x.dtype)
            if thin and tc_ok(w16):
                dx = torch.empty_like(x)
                gemm_tc(dl_x, False, [w16], True, [dx])  # [T, E] x [E, d]
            else:
                dx = dl_x @ w16
        if ctx.needs_input_grad[1]:
            if thin and w.dtype == torch.float32:
                dw = torch.empty_like(w)
                wgrad(dl_all, x, [dw])  # dl_all^T x: reduction over the tokens, fp32 result
            else:
                dw = (dl_all.t() @ x).to(w.dtype)
        return dx, dw, None, None


def router_topk(x, w, k):
    """-> gates, ids, probs, counts (see `_Router`)."""
    return _Router.apply(x, w, k)[:4]


def router_topk_mean(x, w, k, aux_to_tokens=False):
    """-> gates, ids, counts, mean router probability per expert [E] (what the load-balancing loss needs)."""
    gates, idx, _probs, counts, probs_mean = _Router.apply(x, w, k, aux_to_tokens)
    return gates, idx, counts, probs_mean


# ------------------------------------------------------------------------------- pack / combine
class _Pack(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gates, idx, counts):
        ext = get_ext()
        offsets, slot_of = ext.assign_slots(idx, counts)
        px, ptok, pexp, pgate = ext.pack_fwd(x.contiguous(), gates.contiguous(), idx, slot_of)
        ctx.save_for_backward(slot_of)
        ctx.tokens = x.shape[0]
        ctx.mark_non_differentiable(ptok, pexp, offsets, slot_of)
        return px, pgate, ptok, pexp, offsets, slot_of

    @staticmethod
    def backward(ctx, dpx, dpgate, *_):
        (slot_of,) = ctx.saved_tensors
        dx = get_ext().pack_bwd(dpx.contiguous(), slot_of.view(-1), None, ctx.tokens) if dpx is not None else None
        dgates = dpgate[slot_of.long()] if dpgate is not None else None
        return dx, dgates, None, None


def pack(x, gates, idx, counts):
    """-> packed_x, packed_gate, packed_token, packed_expert, offsets [E+1], slot_of [T,k]."""
    return _Pack.apply(x, gates, idx, counts)


def pack_tokens(x, gates, top_e, num_experts):
    idx = top_e.to(torch.int32).contiguous()
    counts = get_ext().count_expert_kernel(idx, idx.new_empty(0), num_experts, idx.shape[1])
    px, pgate, ptok, pexp, _, _ = pack(x, gates.float(), idx, counts)
    return px, ptok, pexp, pgate, counts


class _Combine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, gate, rows, row_start, token, num_tokens, residual):
        yc = y.contiguous()
        res = None if residual is None else residual.contiguous()
        out = get_ext().combine_fwd(yc, gate.contiguous(), rows, row_start, num_tokens, res, False)
        ctx.save_for_backward(yc, gate, token)
        ctx.has_res = residual is not None
        return out

    @staticmethod
    def backward(ctx, dout):
        y, gate, token = ctx.saved_tensors
        dy, dgate = get_ext().combine_bwd(y, token, gate.contiguous(), dout.contiguous())
        return dy, dgate, None, None, None, None, (dout if ctx.has_res else None)


def combine(y, packed_gate, packed_token, slot_of, num_tokens, residual=None):
    """Fixed fan-out combine: token t owns packed rows slot_of[t, :]."""
    return _Combine.apply(y, packed_gate, slot_of.view(-1), None, packed_token, num_tokens, residual)


def _csr(token: torch.Tensor, num_tokens: int):
    tok = token.long()
    order = torch.sort(tok, stable=True).indices.to(torch.int32)
    start = torch.zeros(num_tokens + 1, dtype=torch.int32, device=token.device)
    start[1:] = torch.cumsum(torch.bincount(tok, minlength=num_tokens), 0)
    return start, order


def combine_tokens(y, packed_token, packed_gate, num_tokens, residual=None, slot_of=None):
    tok = packed_token.to(torch.int32).contiguous()
    if slot_of is not None:
        return combine(y, packed_gate, tok, slot_of, num_tokens, residual)
    start, order = _csr(tok, num_tokens)
    return _Combine.apply(y, packed_gate.float(), order, start, tok, num_tokens, residual)


# ------------------------------------------------------------------------------- expert GEMMs
class _GroupedGemm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, offsets, w):
        ctx.save_for_backward(x, offsets, w)
        return get_ext().grouped_gemm_kernel(x, offsets, w)

    @staticmethod
    def backward(ctx, dout):
        x, offsets, w = ctx.saved_tensors
        ext = get_ext()
        dout = dout.contiguous()
        dx = ext.bwd_grouped_gemm_dX_kernel(w, offsets, dout) if ctx.needs_input_grad[0] else None
        dw = ext.bwd_grouped_gemm_dW_kernel(x, offsets, dout) if ctx.needs_input_grad[2] else None
        return dx, None, dw


def grouped_gemm(x, w, offsets):
    return _GroupedGemm.apply(x, offsets, w)


class _SwigluExperts(torch.autograd.Function):
    """Three grouped tcgen05 GEMMs forward (gate|value with the SwiGLU in the epilogue, then the
    down projection), four backward (dH with the SwiGLU derivative in the epilogue, dX over the
    stacked gate|value reduction, and the two weight-gradient GEMMs over ragged segments)."""

    @staticmethod
    def forward(ctx, x, w_gate, w_val, w_out, offsets, residual):
        rows, f, d = x.shape[0], w_gate.shape[2], w_out.shape[2]
        gv = torch.empty(rows, 2 * f, dtype=x.dtype, device=x.device)
        h = torch.empty(rows, f, dtype=x.dtype, device=x.device)
        gemm_tc(x, False, [w_gate, w_val], True, [gv], b_split=B_DUAL, mode=GROUPED_M, offsets=offsets,
                epilogue=EPI_SWIGLU_FWD, aux_out=h)
        y = torch.empty(rows, d, dtype=x.dtype, device=x.device)
        gemm_tc(h, False, [w_out], True, [y], mode=GROUPED_M, offsets=offsets, aux=residual)  # + residual in the epilogue
        ctx.save_for_backward(x, w_gate, w_val, w_out, offsets, gv, h)
        ctx.has_res = residual is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w_gate, w_val, w_out, offsets, gv, h = ctx.saved_tensors
        dy = dy.contiguous()
        dgv = torch.empty_like(gv)
        gemm_tc(dy, False, [w_out], False, [dgv], mode=GROUPED_M, offsets=offsets, epilogue=EPI_SWIGLU_BWD, aux=gv)
        dx = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x)
            gemm_tc(dgv, False, [w_gate, w_val], False, [dx], b_split=B_SPLIT_K, mode=GROUPED_M, offsets=offsets)
        d_out = grad_buffer(w_out)
        gemm_tc(h, True, [dy], True, [d_out], mode=GROUPED_K, offsets=offsets)
        d_gate, d_val = grad_buffer(w_gate), grad_buffer(w_val)
        gemm_tc(x, True, [dgv], True, [d_gate, d_val], mode=GROUPED_K, offsets=offsets)
        return dx, d_gate, d_val, d_out, None, (dy if ctx.has_res else None)


def swiglu_experts(x, w_gate, w_val, w_out, offsets, residual=None):
    """Expert SwiGLU FFN over expert-major rows; `residual` ([rows, d], row-aligned with x) is added
    in the down-projection's epilogue."""
    if offsets.dtype != torch.int32:
        offsets = offsets.to(torch.int32)
    f = w_gate.shape[2]
    if tc_ok(x, w_gate, w_val, w_out) and f % 64 == 0 and w_gate.shape[0] <= 256:
        res = None if residual is None else residual.contiguous()
        return _SwigluExperts.apply(x.contiguous(), w_gate, w_val, w_out, offsets.contiguous(), res)
    gate = grouped_gemm(x, w_gate, offsets)
    val = grouped_gemm(x, w_val, offsets)
    out = grouped_gemm(torch.nn.functional.silu(gate) * val, w_out, offsets)
    return out if residual is None else out + residual


def default_scale(d_head: int) -> float:
    return 1.0 / math.sqrt(d_head)
