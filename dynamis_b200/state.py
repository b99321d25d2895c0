"""Plain state structs with the reference's field names.

Mirrors the pybind classes of dynamis_state/src/dynamis_state_bindings.cpp:15-73 (structs in
dynamis_state/include/dynamis_state/dynamis_state.hpp:6-80): default-constructible, every field
readable and writable, an unset tensor field reads back as ``None``.
"""

from __future__ import annotations

from typing import Callable, Optional

import torch


class MolecularInfo:
    def __init__(self):
        self.num_atoms: int = 0
        self.atom_vertex_numbers: Optional[torch.Tensor] = None
        self.atom_types: Optional[torch.Tensor] = None
        self.atom_positions: Optional[torch.Tensor] = None
        self.atom_velocities: Optional[torch.Tensor] = None
        self.edge_counts: Optional[torch.Tensor] = None  # None = unweighted


class DistEnvironment:
    def __init__(self):
        self.global_rank: int = 0
        self.world_size: int = 0
        self.gpus_per_node: int = 0
        self.num_nodes: int = 0
        self.local_rank: int = 0


class SimulationConfig:
    def __init__(self):
        self.cutoff: float = 0.0
        self.ghost_cutoff_buffer: float = 0.0
        self.cell: Optional[torch.Tensor] = None
        self.pbc: Optional[torch.Tensor] = None


class PartitionMessagePassingInfo:
    """The halo plan passed from the partitioner to the exchangers.

    ``edge_index_halo`` (the full graph at cutoff + ghost buffer, which the reference stores for
    its tests) is produced on first access: the halo maps themselves are built without
    materialising that graph.
    """

    def __init__(self):
        self.partition_id: Optional[torch.Tensor] = None
        self.partition_indices: Optional[torch.Tensor] = None
        self.global_send_recv_matrix: Optional[torch.Tensor] = None
        self.send_offsets: Optional[torch.Tensor] = None
        self.send_local_indices: Optional[torch.Tensor] = None
        self.recv_offsets: Optional[torch.Tensor] = None
        self.recv_ghost_indices: Optional[torch.Tensor] = None
        self.interior_mask: Optional[torch.Tensor] = None
        self.edge_index: Optional[torch.Tensor] = None
        self.atom_counts: Optional[torch.Tensor] = None
        # extension (not in the reference struct): global ids of the ghost atoms, CSR order
        self.recv_atom_global: Optional[torch.Tensor] = None
        self._edge_index_halo: Optional[torch.Tensor] = None
        self._edge_index_halo_fn: Optional[Callable[[], torch.Tensor]] = None

    @property
    def edge_index_halo(self) -> Optional[torch.Tensor]:
        if self._edge_index_halo is None and self._edge_index_halo_fn is not None:
            self._edge_index_halo = self._edge_index_halo_fn()
            self._edge_index_halo_fn = None
        return self._edge_index_halo

    @edge_index_halo.setter
    def edge_index_halo(self, value):
        self._edge_index_halo = value
        self._edge_index_halo_fn = None


class DynamisState:
    def __init__(self):
        self.dist_env = DistEnvironment()
        self.sim_config = SimulationConfig()
        self.global_molecular_info = MolecularInfo()
        self.local_molecular_info = MolecularInfo()
        self.local_partition_info = PartitionMessagePassingInfo()
