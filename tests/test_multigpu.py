"""Multi-GPU paths (one process per GPU, NCCL): skipped unless the box has enough GPUs."""
import pytest
import torch

from tests.conftest import run_distributed

pytestmark = pytest.mark.gpu


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def _train_worker(rank, world, dp, pp, ep, experts, steps):
    from nanotitan_b200.metrics import reduce_metrics
    from nanotitan_b200.parallel_dims import ParallelDims
    from nanotitan_b200.train import build_training
    from nanotitan_b200.utils import seed_everything
    from tests.helpers import random_batch, tiny_app_cfg

    cfg = tiny_app_cfg(dp=dp, pp=pp, ep=ep, microbatches=2 if pp > 1 else 1, batch=4, vocab_size=503, d_model=128,
                       d_head=32, n_heads=4, n_layers=2, max_seq_len=128, ffn_in=256, num_experts=experts,
                       top_k=min(2, experts), moe_backend="cuda", dtype="bfloat16")
    seed_everything(11)
    dims = ParallelDims(cfg.runtime)
    model, _, step, opt = build_training(cfg, dims)
    losses = []
    for i in range(steps):
        m = step.train_step(model, random_batch(cfg, dims.data_rank), opt)  # same batch every step
        losses.append(reduce_metrics(m, torch.device("cuda", rank))["train/ce_loss"] / dims.data_world_size)
    from nanotitan_b200.ops.ext import get_ext

    assert get_ext().read_status(True)[0] == 0
    assert all(l == l for l in losses), losses
    assert losses[-1] < losses[0], losses
    # replicas of the shared parameters must stay identical
    flat = torch.cat([p.detach().float().reshape(-1) for p in model.parameter_sync_groups()["shared"]])
    ref = flat.clone()
    torch.distributed.all_reduce(ref, op=torch.distributed.ReduceOp.MAX, group=dims.shared_dp_group)
    torch.testing.assert_close(flat, ref, rtol=0, atol=0)


@pytest.mark.parametrize("dp,pp,ep,experts", [(2, 1, 1, 1), (1, 1, 2, 4), (1, 2, 1, 4)])
def test_two_gpu_training(dp, pp, ep, experts):
    _need(2)
    run_distributed(_train_worker, 2, dp, pp, ep, experts, 6, backend="nccl")


def test_four_gpu_three_d():
    _need(4)
    run_distributed(_train_worker, 4, 1, 2, 2, 4, 4, backend="nccl")


def _engine_worker(rank, world, multimem, heap="torch"):
    import os

    os.environ["NT_MULTIMEM"] = "1" if multimem else "0"
    os.environ["NT_SYMM_HEAP"] = heap
    os.environ["NT_COMM_WAIT_MS"] = "3000"
    import torch.distributed as dist
    import torch.nn as nn

    from nanotitan_b200.ops.adamw import FusedAdamW
    from nanotitan_b200.ops.ext import get_ext
    from nanotitan_b200.parallel import fused_allreduce
    from nanotitan_b200.parallel.reducer import ReducerV1

    dev = torch.device("cuda", rank)
    torch.manual_seed(5)  # same parameters on every rank
    shapes = [(257, 64), (1000,), (64, 96), (8,)]
    params = [nn.Parameter((torch.randn(s, device=dev) * 0.5).bfloat16()) for s in shapes]
    start = [p.detach().clone() for p in params]
    engine = fused_allreduce.make_engine(dist.group.WORLD, world, dev)
    assert engine is not None, "symmetric memory could not be set up"
    assert engine.symm.name == heap
    red = ReducerV1(params, world, dist.group.WORLD, bucket_size=1, engine=engine)

    def backward(seed):
        red.zero_grad()
        red.backward_grad_sync = True
        g = torch.Generator(device=dev).manual_seed(seed * 100 + rank)
        grads = [torch.randn(p.shape, device=dev, generator=g).bfloat16() for p in params]
        sum((p * gr).sum() for p, gr in zip(params, grads)).backward()
        red.prepare_missing_grad()
        red.finalize_backward()
        want = []
        for gr in grads:  # mean over ranks of the bf16 gradients, in fp32
            t = gr.float()
            dist.all_reduce(t)
            want.append(t / world)
        return want

    # ---- reduce-only mode: every rank ends with the mean gradient in its bucket views
    want = backward(1)
    torch.cuda.synchronize()
    assert get_ext().read_status(True)[0] == 0
    for p, w in zip(params, want):
        torch.testing.assert_close(p.grad.float(), w, rtol=8e-3, atol=8e-3)  # bf16 rounding of the mean

    # ---- optimizer mode: the kernel applies AdamW on the owner's slice and broadcasts parameters
    opt = FusedAdamW(params, lr=1e-2, weight_decay=0.1)
    opt.bind_reducers({"all": red})
    ref_params = [nn.Parameter(s.float().clone()) for s in start]
    ref_opt = torch.optim.AdamW(ref_params, lr=1e-2, weight_decay=0.1)
    for step in range(3):
        want = backward(10 + step)
        opt.step()
        for q, w in zip(ref_params, want):
            # the in-switch reduction returns the sum rounded to the bucket's dtype; peer loads sum in fp32
            q.grad = (w * world).bfloat16().float() / world if multimem else w
        ref_opt.step()
    torch.cuda.synchronize()
    assert get_ext().read_status(True)[0] == 0
    # Three steps at lr 1e-2 move every weight by about 3e-2.  The fp32 master weights of the slice this
    # rank owns must follow torch.optim.AdamW to 1e-5 on the peer-load path (fp32 sums).  The in-switch
    # reduction hands back a bf16 sum whose last bit need not match round-to-nearest of the fp32 sum; one
    # bf16 ulp of a gradient is 0.4 % of an update of 1e-2, hence 2e-4 there.
    tol = 2e-4 if multimem else 1e-5
    for c in opt._chunks:
        assert c.fused_by_engine
        ref_flat = torch.zeros(c.flat_param.numel(), device=dev)
        for p, (lo, hi) in zip(c.params, c.spans):
            ref_flat[lo:hi] = ref_params[[id(x) for x in params].index(id(p))].detach().reshape(-1)
        lo, hi = c.owned
        assert c.master.numel() == hi - lo
        mask = torch.zeros_like(ref_flat, dtype=torch.bool)
        for a, b in c.spans:
            mask[a:b] = True  # padding between parameters carries no weight
        got, want_slice = c.master[mask[lo:hi]], ref_flat[lo:hi][mask[lo:hi]]
        torch.testing.assert_close(got, want_slice, rtol=0, atol=tol)
    for p, q in zip(params, ref_params):  # stored bf16 parameters: the rounding of those masters
        torch.testing.assert_close(p.detach().float(), q.detach().bfloat16().float(), rtol=0, atol=2 ** -7 * 4 * 2)
    flat = torch.cat([p.detach().float().reshape(-1) for p in params])
    other = flat.clone()
    dist.all_reduce(other, op=dist.ReduceOp.MAX)
    assert torch.equal(flat, other), "replicas diverged"


@pytest.mark.parametrize("world", [2, 3, 4, 8])
@pytest.mark.parametrize("multimem", [False, True])
def test_fused_bucket_allreduce_and_adamw(multimem, world):
    """World 3 gives ragged slices (bucket lengths are multiples of 128, not of 8 * 3)."""
    _need(world)
    run_distributed(_engine_worker, world, multimem, backend="nccl")


@pytest.mark.parametrize("multimem", [False, True])
def test_native_symmetric_heap(multimem):
    """The fused all-reduce + AdamW on allocations of this library's own symmetric heap instead of torch's.
    Runs only when asked for (NT_TEST_NATIVE_HEAP=1): the heap's CUDA driver table has not run on a GPU yet,
    so it is not part of the default tier."""
    import os

    if os.environ.get("NT_TEST_NATIVE_HEAP") != "1":
        pytest.skip("set NT_TEST_NATIVE_HEAP=1 to run the native symmetric heap on GPUs")
    _need(2)
    run_distributed(_engine_worker, 2, multimem, "native", backend="nccl")


def _ep_compare_worker(rank, world, starve):
    import os

    os.environ["NT_COMM_WAIT_MS"] = "3000"
    import torch.distributed as dist

    from nanotitan_b200.config import ModelConfig
    from nanotitan_b200.models.feed_fwd import MoE
    from nanotitan_b200.models.utils import ModelShardSpec
    from nanotitan_b200.ops.ext import get_ext

    dev = torch.device("cuda", rank)
    cfg = ModelConfig(vocab_size=8, d_model=128, d_head=32, n_heads=4, n_layers=1, max_seq_len=64, ffn_in=256,
                      num_experts=8, top_k=2, router_alpha=0.01, moe_backend="cuda", dtype="bfloat16")
    per = cfg.num_experts // world
    spec = ModelShardSpec(0, 1, False, False, False, per, rank * per, (rank + 1) * per, ep_size=world, ep_group=dist.group.WORLD)
    torch.manual_seed(3)
    moe = MoE(cfg, spec).to(dev)
    with torch.no_grad():  # the router is replicated: same weights everywhere
        dist.broadcast(moe.router.weight, src=0)
        moe.router.weight.mul_(8.0)  # spread the routing
        if starve:  # expert 3 gets no row from rank 0 and a row of every token of the other ranks
            moe.router.weight[3].zero_()
            moe.router.weight[3, 0] = 60.0
    torch.manual_seed(100 + rank)
    x = torch.randn(3, 64, 128, device=dev).bfloat16()
    if starve:
        x[..., 0] = -1.0 if rank == 0 else 1.0
    g = torch.randn_like(x)
    results = []
    for fused in (True, False):
        xi = x.clone().requires_grad_()
        moe.zero_grad(set_to_none=True)
        if not fused:
            moe.moe_backend.fused_exchange = None  # fall back to the NCCL all-to-all path
        out, stats = moe(xi)
        if fused:
            assert moe.moe_backend.fused_exchange is not None, "symmetric memory could not be set up"
        (out * g).sum().backward()
        results.append([out.detach().clone(), xi.grad.clone()] + [p.grad.clone() for p in moe.experts.parameters()]
                       + [stats.tokens_per_expert.clone()])
    torch.cuda.synchronize()
    assert get_ext().read_status(True)[0] == 0
    for a, b in zip(*results):
        assert torch.equal(a, b)
    assert results[0][0].abs().max() > 0
    if starve:
        counts = results[0][-1]
        assert int(counts[3]) == (0 if rank == 0 else 3 * 64), counts


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("starve", [False, True])
def test_fused_ep_exchange_equals_nccl_path(world, starve):
    """Outputs, input gradients and expert weight gradients of the fused exchange are bitwise those of the
    NCCL all-to-all path, also when one source rank sends an expert nothing."""
    _need(world)
    run_distributed(_ep_compare_worker, world, starve, backend="nccl")


def _ep_overflow_worker(rank, world):
    """Every token of every rank picks experts 0 and 1 (both on rank 0): more rows than rank 0's bounded
    staging holds.  The kernel must drop the excess and say so in the status word, not write past the end."""
    import os

    os.environ["NT_COMM_WAIT_MS"] = "3000"
    os.environ["NT_EP_CAPACITY_FACTOR"] = "1.0"
    import torch.distributed as dist

    from nanotitan_b200.config import ModelConfig
    from nanotitan_b200.models.feed_fwd import MoE
    from nanotitan_b200.models.utils import ModelShardSpec
    from nanotitan_b200.ops.ext import get_ext

    dev = torch.device("cuda", rank)
    cfg = ModelConfig(vocab_size=8, d_model=128, d_head=32, n_heads=4, n_layers=1, max_seq_len=64, ffn_in=256,
                      num_experts=4, top_k=2, router_alpha=0.01, moe_backend="cuda", dtype="bfloat16")
    per = cfg.num_experts // world
    spec = ModelShardSpec(0, 1, False, False, False, per, rank * per, (rank + 1) * per, ep_size=world, ep_group=dist.group.WORLD)
    moe = MoE(cfg, spec).to(dev)
    with torch.no_grad():
        moe.router.weight.zero_()
        moe.router.weight[0, 0] = 40.0
        moe.router.weight[1, 0] = 39.0
    x = torch.ones(2, 64, 128, device=dev).bfloat16()
    with torch.no_grad():
        moe(x)
    torch.cuda.synchronize()
    code, kernel, _detail, count = get_ext().read_status(True)
    # rank 0's staging holds 256 rows; 512 were routed there (expert 1's rows from both ranks are the excess)
    assert code == 2 and kernel == 5 and count > 0, (code, kernel, count)
    dist.barrier()


def test_ep_capacity_overflow_is_reported_not_written():
    _need(2)
    run_distributed(_ep_overflow_worker, 2, backend="nccl")
