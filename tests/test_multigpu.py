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


def _engine_worker(rank, world, multimem):
    import os

    os.environ["NT_MULTIMEM"] = "1" if multimem else "0"
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
        torch.testing.assert_close(p.grad.float(), w, rtol=2e-2, atol=2e-2)

    # ---- optimizer mode: the kernel applies AdamW on the owner's slice and broadcasts parameters
    opt = FusedAdamW(params, lr=1e-2, weight_decay=0.1)
    opt.bind_reducers({"all": red})
    ref_params = [nn.Parameter(s.float().clone()) for s in start]
    ref_opt = torch.optim.AdamW(ref_params, lr=1e-2, weight_decay=0.1)
    for step in range(3):
        want = backward(10 + step)
        opt.step()
        for q, w in zip(ref_params, want):
            q.grad = w
        ref_opt.step()
    torch.cuda.synchronize()
    assert get_ext().read_status(True)[0] == 0
    for p, q in zip(params, ref_params):
        torch.testing.assert_close(p.detach().float(), q.detach(), rtol=3e-2, atol=3e-2)
    flat = torch.cat([p.detach().float().reshape(-1) for p in params])
    other = flat.clone()
    dist.all_reduce(other, op=dist.ReduceOp.MAX)
    assert torch.equal(flat, other), "replicas diverged"


@pytest.mark.parametrize("multimem", [False, True])
def test_fused_bucket_allreduce_and_adamw(multimem):
    _need(2)
    run_distributed(_engine_worker, 2, multimem, backend="nccl")


def _ep_compare_worker(rank, world):
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
    torch.manual_seed(100 + rank)
    x = torch.randn(3, 64, 128, device=dev).bfloat16()
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


def test_fused_ep_exchange_equals_nccl_path():
    _need(2)
    run_distributed(_ep_compare_worker, 2, backend="nccl")
