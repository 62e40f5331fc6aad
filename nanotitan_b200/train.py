"""Training entrypoint: ``torchrun ... -m nanotitan_b200.train @cfg.toml [--log.level L]``.

Same flow as the reference's `main()` (src/train.py:81-226): load the TOML, set up the
process group and the DP x PP x EP layout, build this rank's model shard, wrap it in
the data-parallel reducers and the GPipe step, then loop over the sharded loader
logging the reference's metric names.  It also runs as a single process with no
launcher, on CPU (gloo) as well as GPUs (NCCL), and adds `--resume`, periodic sharded
checkpoints, a per-step heartbeat, MFU and gradient-norm metrics.
"""
from __future__ import annotations

import argparse
import logging
import os

import torch

from nanotitan_b200.data.dataset import PackedTokenDataset, SyntheticTokenDataset
from nanotitan_b200.data.native_loader import skip_batches
from nanotitan_b200.dist_env import barrier, cleanup, get_world_size, init_distributed, local_device
from nanotitan_b200.metrics import MetricsLogger, ScalarMetric, reduce_metrics
from nanotitan_b200.models.model import NanoTitanModel
from nanotitan_b200.models.utils import get_model_shard_specs
from nanotitan_b200.optim import setup_optimizer
from nanotitan_b200.parallel import DataParallel, PipelineParallel
from nanotitan_b200.parallel_dims import get_parallel_dims
from nanotitan_b200.profiler import build_profiler
from nanotitan_b200.utils import load_run_config, reduce_scalars, seed_everything, setup_logging
from nanotitan_b200.utils.checkpoint import AsyncCheckpointer, latest_checkpoint, load_checkpoint, save_checkpoint
from nanotitan_b200.utils.heartbeat import Heartbeat, assert_peers_alive

logger = logging.getLogger(__name__)

__all__ = ["main", "parse_args", "reduce_metrics", "build_training", "model_flops_per_token"]


def parse_args(argv=None) -> argparse.Namespace:
    parser = argparse.ArgumentParser(description="Train a NanoTitan model from a TOML config.")
    parser.add_argument("--single_gpu", action="store_true",
                        help="Accepted for compatibility; a 1-process run needs no flag.")
    parser.add_argument("--log.level", default="INFO", dest="log_level",
                        help="Python logging level, e.g. DEBUG, INFO, WARNING.")
    parser.add_argument("--resume", default="", help="Checkpoint directory to resume from.")
    parser.add_argument("--synthetic-data", action="store_true",
                        help="Uniform-random token ids instead of the token file.")
    parser.add_argument("--init-from", default="",
                        help="File written by `python -m nanotitan_b200.utils.checkpoint consolidate [--with-optimizer]`: "
                             "start from those weights (and optimizer state, step and token count) on this run's layout.")
    parser.add_argument("--eval-batches", type=int, default=20,
                        help="Validation batches per rank and evaluation (trainer.eval_every_step != -1).")
    parser.add_argument("config", help="TOML config path, optionally prefixed with '@'.")
    return parser.parse_args(argv)


def model_flops_per_token(cfg, active_params: float) -> float:
    """6 * active matmul parameters + causal attention (fwd + bwd), per token."""
    m = cfg.model
    embed = m.vocab_size * m.d_model  # the lookup table does no matmul work
    attn = 6 * m.n_layers * m.max_seq_len * m.n_heads * m.d_head  # 12*S*H*Dh/2 (causal)
    return 6.0 * (active_params - embed) + attn


def build_training(cfg, dims):
    """Model shard + DP reducers + GPipe step + optimizer for this rank."""
    spec = get_model_shard_specs(dims, cfg)
    model = NanoTitanModel.from_specs(cfg.model, spec)
    dp = DataParallel(cfg, dims)
    dp.prepare_model(model)
    pp = PipelineParallel(cfg, dims, dp.get_reducers())
    optimizer = setup_optimizer(cfg.optim, model)
    if hasattr(optimizer, "bind_reducers"):
        optimizer.bind_reducers(dp.get_reducers())
    return model, dp, pp, optimizer


def main(argv=None) -> None:
    args = parse_args(argv)
    setup_logging(args.log_level)
    cfg = load_run_config(args.config)
    init_distributed(timeout_s=cfg.fault.pg_timeout_s)
    world_size = get_world_size()
    assert world_size == cfg.runtime.dp_size * cfg.runtime.pp_size * cfg.runtime.ep_size, (
        f"world size {world_size} != dp*pp*ep"
    )
    assert cfg.model.n_layers % cfg.runtime.pp_size == 0
    assert cfg.trainer.per_device_batch_size % cfg.runtime.num_microbatches == 0

    seed_everything(cfg.trainer.seed)
    dims = get_parallel_dims(cfg.runtime)
    logger.debug("rank %d: %r", dims.global_rank, dims)
    device = local_device()
    model, dp, pp, optimizer = build_training(cfg, dims)

    metrics_logger = MetricsLogger(cfg.run_name) if dims.local_rank == 0 else None
    if args.synthetic_data:
        n_seq = cfg.trainer.per_device_batch_size * dims.data_world_size * cfg.max_steps
        train_dataset = SyntheticTokenDataset(
            cfg.model.vocab_size, cfg.model.max_seq_len, n_seq, cfg.trainer.seed
        )
    else:
        train_dataset = PackedTokenDataset(cfg.data.train_tokens_path, cfg.model.max_seq_len)
    train_loader = dp.prepare_trainloader(train_dataset)
    val_loader = None
    if cfg.trainer.eval_every_step != -1:
        if args.synthetic_data:
            n_val = cfg.trainer.per_device_batch_size * dims.data_world_size * args.eval_batches
            val_dataset = SyntheticTokenDataset(cfg.model.vocab_size, cfg.model.max_seq_len, n_val, cfg.trainer.seed + 1)
        else:
            val_dataset = PackedTokenDataset(cfg.data.val_tokens_path, cfg.model.max_seq_len)
        val_loader = dp.prepare_valloader(val_dataset)

    counts = torch.tensor(
        [model.total_parameter_count(), float(model.active_parameter_count())],
        dtype=torch.float64, device=device,
    )
    reduce_scalars(counts, dims.pp_group)
    total_params, active_params = counts.tolist()
    if dims.global_rank == 0:
        logger.info("Number of parameters: %.2fM total, %.2fM active",
                    total_params / 1e6, active_params / 1e6)
        logger.info("Model parameters and activations will be in %s datatype", cfg.model.dtype)

    step = 0
    tokens_seen = 0
    epoch, batches_done = 0, 0  # loader position: batches of `epoch` already taken
    resume_dir = args.resume or (cfg.checkpoint.dir if cfg.checkpoint.resume else "")
    if resume_dir:
        found = latest_checkpoint(resume_dir)
        if found is not None:
            state = load_checkpoint(found, model, optimizer, dims)
            step, tokens_seen = state["step"], state["tokens_seen"]
            if state.get("data"):
                epoch, batches_done = state["data"]["epoch"], state["data"]["batches_done"]
            logger.info("resumed from %s at step %d", found, step)

    if args.init_from and step == 0:
        from nanotitan_b200.utils.checkpoint import load_full_optimizer, load_full_state

        full = torch.load(args.init_from, map_location="cpu", weights_only=False)
        if "model" in full and isinstance(full["model"], dict):
            load_full_state(model, full["model"])
            if full.get("optimizer") is not None:
                load_full_optimizer(model, optimizer, full["optimizer"])
            elif hasattr(optimizer, "set_master_weights"):
                optimizer.set_master_weights({id(p): p.detach() for p in model.parameters()})
            step, tokens_seen = int(full.get("step", 0)), int(full.get("tokens_seen", 0))
            if full.get("data") and full.get("data_world_size") == dims.data_world_size:
                epoch, batches_done = full["data"]["epoch"], full["data"]["batches_done"]
            elif step:
                logger.warning("the data is sharded over %d ranks now (%s when saved): the data order starts over",
                               dims.data_world_size, full.get("data_world_size"))
        else:  # a bare state dict
            load_full_state(model, full)
            if hasattr(optimizer, "set_master_weights"):
                optimizer.set_master_weights({id(p): p.detach() for p in model.parameters()})
        logger.info("initialised from %s at step %d", args.init_from, step)

    heartbeat = Heartbeat(cfg.fault.heartbeat_dir, dims.global_rank) if cfg.fault.heartbeat_dir else None
    if heartbeat is not None:
        heartbeat.beat(step)  # every rank is on record before anybody checks
        barrier()

    def check_peers() -> None:
        """A peer whose heartbeat went stale is found here, on the host, before the next launch
        (instead of after an in-kernel wait or a process-group timeout runs out)."""
        if heartbeat is not None:
            assert_peers_alive(cfg.fault.heartbeat_dir, world_size, cfg.fault.heartbeat_stale_s)

    inject = os.environ.get("NT_INJECT_EXIT", "")

    def inject_exit(at_step: int) -> None:
        """Host-side fault injection for restart tests: `NT_INJECT_EXIT=rank:step[:attempt]` makes that rank
        leave the job right before it would launch `step`, on the given launcher attempt (default: the first).
        The rank leaves between steps with nothing of its own in flight."""
        if not inject:
            return
        rank_s, step_s, *rest = inject.split(":")
        attempt = int(rest[0]) if rest else 0
        if (int(rank_s), int(step_s), attempt) != (dims.global_rank, at_step, int(os.environ.get("TORCHELASTIC_RESTART_COUNT", "0"))):
            return
        if device.type == "cuda":
            torch.cuda.synchronize(device)
        logger.error("NT_INJECT_EXIT: rank %d leaves before step %d", dims.global_rank, at_step)
        logging.shutdown()
        os._exit(17)

    profiler = build_profiler(cfg.run_name, cfg.profiler, dims)
    flops_per_token = model_flops_per_token(cfg, active_params)
    peak = cfg.hardware.peak_flops_tflops_per_gpu * 1e12
    # data is sharded over dp*ep ranks (the reference counts dp only, src/train.py:157)
    tokens_per_step = cfg.trainer.per_device_batch_size * dims.data_world_size * cfg.model.max_seq_len
    # Step metrics are reduced over a host-side (gloo) group: the values are already on the host when
    # they are reduced, and a collective on the compute stream would have to wait for the step that
    # was launched in the meantime.
    metrics_group = None
    if world_size > 1 and device.type == "cuda":
        import torch.distributed as dist

        metrics_group = dist.new_group(backend="gloo")

    def report(entry) -> None:
        """Collect, reduce and log the metrics of a step that was launched earlier."""
        index, seen, pending = entry
        metrics = pending.result()
        metrics["train/tokens_per_step"] = ScalarMetric(tokens_per_step, reduce="none")
        metrics["train/total_tokens_seen"] = ScalarMetric(seen, reduce="none")
        if hasattr(optimizer, "last_grad_norm"):
            metrics["train/grad_norm"] = ScalarMetric(optimizer.last_grad_norm(), reduce="max")
        metrics = reduce_metrics(metrics, torch.device("cpu") if metrics_group is not None else device, group=metrics_group)
        metrics["train/tokens_per_second"] = metrics["train/tokens_per_step"] / metrics["time/step_time"]
        metrics["train/ce_loss"] = metrics["train/ce_loss"] / dims.data_world_size
        metrics["train/lb_loss"] = metrics["train/lb_loss"] / dims.data_world_size
        if peak > 0:
            metrics["perf/mfu"] = metrics["train/tokens_per_second"] * flops_per_token / (peak * world_size)
        if dims.local_rank == 0:
            logger.info("step %d | ce %.4f | lb %.4f | %.0f tok/s | %.1f ms",
                        index, metrics["train/ce_loss"], metrics["train/lb_loss"],
                        metrics["train/tokens_per_second"], 1e3 * metrics["time/step_time"])
            metrics_logger.log(step=index, metrics=metrics)

    def evaluate(index: int) -> None:
        """Mean validation cross-entropy over at most `--eval-batches` full batches per rank, logged as
        `val/ce_loss` at step `index`.  Every rank runs the same number of batches (the sampler pads the
        shards to equal length), so the collectives inside the model line up."""
        total = torch.zeros(2, dtype=torch.float64, device=device)  # [sum of batch means, batches]
        for n, batch in enumerate(val_loader):
            if n >= args.eval_batches or batch[0].shape[0] != cfg.trainer.per_device_batch_size:
                break
            loss = pp.eval_step(model, batch)
            if loss is not None:
                total += torch.stack([loss.double(), torch.ones((), dtype=torch.float64, device=device)])
        reduce_scalars(total, None)  # over all ranks; only last pipeline stages contributed
        if total[1] > 0 and dims.local_rank == 0:
            value = float(total[0] / total[1])
            logger.info("step %d | val ce %.4f over %d batches", index, value, int(total[1]))
            metrics_logger.log(step=index, metrics={"val/ce_loss": value})

    logger.info("Attempting to begin training")
    def data_state() -> dict:
        return {"epoch": epoch, "batches_done": batches_done}

    background = AsyncCheckpointer(cfg.fault.pg_timeout_s) if cfg.checkpoint.async_save else None

    def save() -> None:
        check_peers()
        write = background.save if background is not None else save_checkpoint
        write(cfg.checkpoint.dir, step, tokens_seen, model, optimizer, dims, cfg, data_state(), cfg.checkpoint.portable_optimizer)

    try:
        # On GPUs the loop runs one step ahead of its own reporting: step i+1 is launched before the metrics
        # of step i are collected, so reading the losses never leaves the device idle.  On CPU a step's
        # collectives block the host, there is nothing to overlap, and every step is reported at once.
        run_ahead = os.environ.get("NT_RUN_AHEAD", "1" if device.type == "cuda" else "0") == "1"
        in_flight = None
        with profiler as prof:
            while step < cfg.max_steps:
                if hasattr(train_loader.sampler, "set_epoch"):
                    train_loader.sampler.set_epoch(epoch)
                progressed = batches_done > 0
                for batch in skip_batches(train_loader, batches_done):
                    progressed = True
                    check_peers()
                    inject_exit(step)
                    pending = pp.train_step(model, batch, optimizer, collect_metrics="deferred")
                    tokens_seen += tokens_per_step
                    batches_done += 1
                    if in_flight is not None:
                        report(in_flight)
                    in_flight = (step, tokens_seen, pending)
                    if not run_ahead:
                        report(in_flight)
                        in_flight = None
                    step += 1
                    prof.step()
                    if heartbeat is not None:
                        heartbeat.beat(step)
                    # -1: never, 0: after every step, n: after every n-th step (the rule of the reference's
                    # commented-out loop, src/train.py:187-190)
                    every_eval = cfg.trainer.eval_every_step
                    if val_loader is not None and (every_eval == 0 or step % every_eval == 0):
                        evaluate(step - 1)
                    every = cfg.checkpoint.every_steps
                    if cfg.checkpoint.dir and every and step % every == 0:
                        save()
                    if step >= cfg.max_steps:
                        break
                else:  # the epoch ran out (no break): the next one starts from its first batch
                    epoch, batches_done = epoch + 1, 0
                if not progressed:
                    raise RuntimeError("the training loader produced no batch (dataset too small)")
            if in_flight is not None:
                report(in_flight)
                in_flight = None
        if cfg.checkpoint.dir:
            save()
        if background is not None:
            background.wait()
            barrier()  # nobody leaves before rank 0 has seen every shard and written the manifest
    finally:
        if heartbeat is not None:
            heartbeat.leave(step)
        if metrics_logger is not None:
            metrics_logger.close()
        cleanup()


if __name__ == "__main__":
    main()
