"""Distributed simulation state: repartition, halo-only rebuild, drift watchdog — host side.

Same interface as the reference's ``SimState`` (dynamis/src/dynamis/simulatorState.py:26-293):
``sync_and_repartition``, ``sync_positions_and_rebuild_halo``, ``snapshot_reference_positions``,
``write_local_drift_flag`` and the ``pos`` / ``vel`` / ``local_partition_info`` properties.

Differences in how, not in what:
  * every rank's (ids, positions, velocities) travel in two ``all_gather_into_tensor`` collectives of
    padded device tensors (the reference pickles them through ``all_gather_object``), and are put back
    into canonical atom order by one scatter kernel per array (no concatenate + argsort + gather);
  * the drift word is one kernel (``dynb_drift_flag``) instead of five reductions.
Partition and halo maps go through the partitioner, i.e. the CUDA library.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import _lib
from .partition import _stream, scratch
from .state import DistEnvironment, DynamisState, MolecularInfo, PartitionMessagePassingInfo, SimulationConfig

DRIFT_TRIP = 1
DRIFT_BREACH = 2


def scatter_rows(rows: torch.Tensor, idx: torch.Tensor, out: torch.Tensor) -> None:
    """``out[idx[i], :] = rows[i, :]`` for unique ``idx`` (device kernel)."""
    n = idx.numel()
    if n == 0:
        return
    rows = rows.contiguous()
    dev = rows.device
    row_bytes = rows[0].numel() * rows.element_size()
    with torch.cuda.device(dev):
        bad = scratch(dev, "bad", 256)
        bad.zero_()
        _lib.check(_lib.lib().dynb_scatter_rows(rows.data_ptr(), row_bytes, idx.data_ptr(), n, out.size(0), out.data_ptr(),
                                                bad.data_ptr(), _stream(dev)), "scatter_rows")


class SimState:
    def __init__(self, molecular_system: MolecularInfo, partitioner, simulation_config: SimulationConfig,
                 distributed_environment: DistEnvironment, device: Optional[torch.device] = None, process_group=None):
        self.dist_env_obj = distributed_environment
        self.local_rank = int(distributed_environment.local_rank)
        self.global_rank = int(distributed_environment.global_rank)
        self.world_size = int(distributed_environment.world_size)
        self.num_nodes = int(distributed_environment.num_nodes)
        self.gpus_per_node = int(distributed_environment.gpus_per_node)
        self.is_distributed = self.world_size > 1
        self.device = device if device is not None else torch.device(f"cuda:{self.local_rank}")
        self.process_group = process_group
        simulation_config.cell = simulation_config.cell.to(self.device)
        simulation_config.pbc = simulation_config.pbc.to(self.device)
        self.partitioner = partitioner
        info = partitioner.partition(molecular_system, self.dist_env_obj)
        partitioner.build_halo_maps(info, molecular_system, self.dist_env_obj, simulation_config)
        self.partition_info = info
        self.global_molecular_info = molecular_system
        self._state = DynamisState()
        self._state.dist_env = self.dist_env_obj
        self._state.sim_config = simulation_config
        self._state.global_molecular_info = molecular_system
        self._state.local_partition_info = info
        self._state.local_molecular_info = self.setup_mass_and_forces(info, molecular_system)
        self._ref_positions = None
        self._prev_velocities = None
        self._drift_state = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.snapshot_reference_positions()

    # ------------------------------------------------------------------ accessors
    @property
    def pos(self):
        return self._state.local_molecular_info.atom_positions

    @property
    def vel(self):
        return self._state.local_molecular_info.atom_velocities

    @property
    def sim_config(self):
        return self._state.sim_config

    @property
    def dist_env(self):
        return self._state.dist_env

    @property
    def local_state(self):
        return self._state.local_molecular_info

    @property
    def local_partition_info(self) -> PartitionMessagePassingInfo:
        return self._state.local_partition_info

    def setup_mass_and_forces(self, partition_info, molecular_system) -> MolecularInfo:
        loc = MolecularInfo()
        idx = partition_info.partition_indices
        loc.atom_positions = molecular_system.atom_positions[idx]
        loc.atom_velocities = molecular_system.atom_velocities[idx] if molecular_system.atom_velocities is not None else None
        loc.atom_types = molecular_system.atom_types[idx] if molecular_system.atom_types is not None else None
        loc.num_atoms = loc.atom_positions.shape[0]
        return loc

    # ------------------------------------------------------------------ gathers
    def _gather_rows(self, rows: torch.Tensor, ids: torch.Tensor, counts, out: torch.Tensor) -> None:
        """All ranks' ``rows`` (each [n_r, F], padded to the largest n_r) -> ``out[ids_r] = rows_r``."""
        import torch.distributed as dist

        W, m = self.world_size, max(counts)
        F = rows.shape[1]
        buf = rows.new_zeros((m, F))
        buf[: rows.shape[0]] = rows
        gathered = rows.new_empty((W * m, F))
        dist.all_gather_into_tensor(gathered, buf, group=self.process_group)
        for r in range(W):
            if counts[r]:
                scatter_rows(gathered[r * m: r * m + counts[r]], ids[r], out)

    def _ids_by_rank(self, info):
        """Global ids owned by each rank, ascending (the order of every rank's local arrays)."""
        from .partition import select_eq

        owner = info.partition_id
        counts = [int(c) for c in info.atom_counts.tolist()] if info.atom_counts is not None else \
            torch.bincount(owner, minlength=self.world_size).tolist()
        ids = [select_eq(owner, r) for r in range(self.world_size)]
        return ids, counts

    # ------------------------------------------------------------------ repartition
    def sync_and_repartition(self, paritioner=None, comm_backend: str = "nccl") -> None:
        info = self._state.local_partition_info
        loc = self._state.local_molecular_info
        glob = self._state.global_molecular_info
        N = glob.atom_positions.shape[0]
        if self.world_size == 1:
            scatter_rows(loc.atom_positions, info.partition_indices, glob.atom_positions)
            scatter_rows(loc.atom_velocities, info.partition_indices, glob.atom_velocities)
        else:
            ids, counts = self._ids_by_rank(info)
            both = torch.cat([loc.atom_positions, loc.atom_velocities], dim=1).contiguous()  # [n_local, 6]
            full = both.new_empty((N, 6))
            self._gather_rows(both, ids, counts, full)
            glob.atom_positions = full[:, :3].contiguous()
            glob.atom_velocities = full[:, 3:].contiguous()
        self.partitioner = paritioner if paritioner is not None else self.partitioner
        new_info = self.partitioner.partition(glob, self.dist_env)
        self.partitioner.build_halo_maps(new_info, glob, self.dist_env, self.sim_config)
        self._state.local_partition_info = new_info
        self._state.global_molecular_info = glob
        self.partition_info = new_info
        self._state.local_molecular_info = self.setup_mass_and_forces(new_info, glob)
        self.snapshot_reference_positions()

    def sync_positions_and_rebuild_halo(self) -> None:
        info = self._state.local_partition_info
        glob = self._state.global_molecular_info
        local_positions = self._state.local_molecular_info.atom_positions.detach()
        if self.world_size == 1:
            scatter_rows(local_positions, info.partition_indices, glob.atom_positions)
        else:
            ids, counts = self._ids_by_rank(info)
            if not torch.equal(ids[self.global_rank], info.partition_indices):
                raise AssertionError("partition_indices is not in ascending global-ID order")
            full = local_positions.new_empty((glob.atom_positions.shape[0], 3))
            self._gather_rows(local_positions.contiguous(), ids, counts, full)
            glob.atom_positions = full
        self.partitioner.build_halo_maps(info, glob, self.dist_env, self.sim_config)
        self.snapshot_reference_positions()

    # ------------------------------------------------------------------ drift watchdog
    def snapshot_reference_positions(self) -> None:
        loc = self._state.local_molecular_info
        self._ref_positions = loc.atom_positions.detach().clone()
        self._prev_velocities = loc.atom_velocities.detach().clone() if loc.atom_velocities is not None else None

    def write_local_drift_flag(self, flag: torch.Tensor, threshold: float, dt: float) -> None:
        """Writes this rank's 2-bit drift word into ``flag`` (int32 [1]); device only, one kernel."""
        loc = self._state.local_molecular_info
        cur = loc.atom_positions.detach()
        ref = self._ref_positions
        if ref is None or ref.shape != cur.shape:
            flag.fill_(DRIFT_TRIP)
            return
        if cur.shape[0] == 0:
            flag.zero_()
            return
        vel = loc.atom_velocities.detach()
        if cur.dtype != torch.float32:
            raise RuntimeError("write_local_drift_flag expects float32 positions")
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().dynb_drift_flag(cur.contiguous().data_ptr(), ref.data_ptr(), vel.contiguous().data_ptr(),
                                                  self._prev_velocities.data_ptr(), cur.shape[0], float(dt), float(threshold),
                                                  self._drift_state.data_ptr(), flag.data_ptr(), _stream(self.device)),
                       "drift_flag")
