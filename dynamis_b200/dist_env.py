"""``TorchDistEnv`` — the helper the reference's callers use to bring up torch.distributed and pick
the device (reference: dynamis_state/src/dynamis_state/state_wrapper.py:16-62).  Same attributes
(``device``, ``local_rank``, ``global_rank``, ``world_size``, ``num_nodes``, ``gpus_per_node``,
``is_distributed``), same ``dist_env`` property and ``barrier()``."""

from __future__ import annotations

import torch
import torch.distributed as dist

from .state import DistEnvironment


class TorchDistEnv:
    def __init__(self, is_distributed: bool = True, **kwargs) -> None:
        if is_distributed:
            if not dist.is_initialized():
                dist.init_process_group(backend="cuda:nccl,cpu:gloo", **kwargs)
            global_rank, world_size = dist.get_rank(), dist.get_world_size()
        else:
            global_rank, world_size = 0, 1
        num_gpus = torch.cuda.device_count()
        gpus_per_node = num_gpus if num_gpus > 0 else 1
        local_rank = global_rank % gpus_per_node
        if num_gpus > 0:
            torch.cuda.set_device(local_rank)
        self.device = torch.device(f"cuda:{local_rank}" if num_gpus > 0 else "cpu")
        self.local_rank, self.global_rank, self.world_size = local_rank, global_rank, world_size
        self.num_nodes = max(1, (world_size + gpus_per_node - 1) // gpus_per_node)
        self.gpus_per_node = gpus_per_node
        self.is_distributed = is_distributed

    @property
    def dist_env(self) -> DistEnvironment:
        env = DistEnvironment()
        env.global_rank, env.world_size = self.global_rank, self.world_size
        env.gpus_per_node, env.num_nodes, env.local_rank = self.gpus_per_node, self.num_nodes, self.local_rank
        return env

    def barrier(self) -> None:
        if self.is_distributed:
            dist.barrier()
