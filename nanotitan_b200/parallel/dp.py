"""Data-parallel facade: device placement, initial parameter sync, reducers, loaders.

Surface of the reference (src/parallel/dp.py:14-107).  Shared (non-expert) parameters
are replicated over the dp*ep ranks of a pipeline stage, expert parameters over the dp
ranks that hold the same expert shard; each family gets its own bucketed reducer.
The initial sync broadcasts whole flat buckets (a handful of collectives) instead of
one broadcast per tensor.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.utils.data import DataLoader
from torch.utils.data.distributed import DistributedSampler

from nanotitan_b200.dist_env import local_device
from nanotitan_b200.parallel.reducer import ReducerV1


class DataParallel:
    def __init__(self, cfg, dims):
        self.cfg = cfg
        self.dims = dims
        self.device = local_device()
        self.shared_reducer: ReducerV1 | None = None
        self.expert_reducer: ReducerV1 | None = None

    def prepare_model(self, model: nn.Module):
        model.to(self.device)
        groups = model.parameter_sync_groups()
        self.broadcast_parameters(
            groups["shared"], self.dims.shared_dp_group_ranks[0], self.dims.shared_dp_group
        )
        self.broadcast_parameters(
            groups["expert"], self.dims.expert_dp_group_ranks[0], self.dims.expert_dp_group
        )
        bucket = self.cfg.runtime.bucket_size
        shared_engine = expert_engine = None
        if self.device.type == "cuda":
            from nanotitan_b200.parallel import fused_allreduce

            shared_engine = fused_allreduce.make_engine(
                self.dims.shared_dp_group, len(self.dims.shared_dp_group_ranks), self.device)
            expert_engine = fused_allreduce.make_engine(
                self.dims.expert_dp_group, len(self.dims.expert_dp_group_ranks), self.device)
        self.shared_reducer = ReducerV1(
            groups["shared"], len(self.dims.shared_dp_group_ranks), self.dims.shared_dp_group, bucket,
            engine=shared_engine,
        )
        self.expert_reducer = ReducerV1(
            groups["expert"], len(self.dims.expert_dp_group_ranks), self.dims.expert_dp_group, bucket,
            engine=expert_engine,
        )
        return model

    def broadcast_parameters(self, params, src_rank: int, group, async_op: bool = False) -> None:
        """Make every replica start from `src_rank`'s values (src is a global rank)."""
        params = list(params)
        if not params or group is None or dist.get_world_size(group) == 1:
            return
        with torch.no_grad():
            by_dtype: dict[torch.dtype, list[torch.Tensor]] = {}
            for p in params:
                by_dtype.setdefault(p.dtype, []).append(p)
            for tensors in by_dtype.values():
                flat = torch.cat([t.reshape(-1) for t in tensors])
                dist.broadcast(flat, src=src_rank, group=group, async_op=False)
                cursor = 0
                for t in tensors:
                    t.copy_(flat[cursor : cursor + t.numel()].view_as(t))
                    cursor += t.numel()

    def finalize_backward(self) -> None:
        self.shared_reducer.finalize_backward()
        self.expert_reducer.finalize_backward()

    def get_reducers(self) -> dict:
        return {"shared": self.shared_reducer, "expert": self.expert_reducer}

    def prepare_trainloader(self, train_dataset):
        """This rank's shuffled shard of the training set, in batches; packed token files are served by the C++
        loader (data/native_loader.py), anything else by a torch DataLoader."""
        from nanotitan_b200.data.native_loader import make_train_loader

        sampler = DistributedSampler(
            dataset=train_dataset,
            shuffle=True,
            num_replicas=self.dims.data_world_size,
            rank=self.dims.data_rank,
        )
        return make_train_loader(train_dataset, sampler, self.cfg.trainer.per_device_batch_size, self.device,
                                 self.cfg.data.num_workers)

    def prepare_valloader(self, val_dataset) -> DataLoader:
        sampler = DistributedSampler(
            dataset=val_dataset,
            shuffle=False,
            num_replicas=self.dims.data_world_size,
            rank=self.dims.data_rank,
        )
        return DataLoader(
            val_dataset,
            batch_size=self.cfg.trainer.per_device_batch_size,
            num_workers=self.cfg.data.num_workers,
            sampler=sampler,
            pin_memory=self.device.type == "cuda",
            drop_last=False,
        )
