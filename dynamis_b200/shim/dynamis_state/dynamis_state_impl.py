"""Stands where the reference's compiled module `dynamis_state.dynamis_state_impl` stands
(reference: dynamis_state/src/dynamis_state_bindings.cpp:13-264): same functions and classes."""

import enum

from dynamis_b200.graph import radius_graph_pbc, radius_graph_pbc_counts_ex, radius_graph_pbc_ex  # noqa: F401
from dynamis_b200.halo import extract_halo_info, filter_edges_to_radius  # noqa: F401
from dynamis_b200.partition import KDTreePartitioner, SFCCurveType, SFCPartitioner, SimpleSpatialPartitioner  # noqa: F401
from dynamis_b200.state import (  # noqa: F401
    DistEnvironment,
    DynamisState,
    MolecularInfo,
    PartitionMessagePassingInfo,
    SimulationConfig,
)

# ---- timing: outside the hot path; compiled out (TIMING_ENABLED False), every call is a no-op ----
TIMING_ENABLED = False


class TimerClass(enum.IntEnum):
    Compute = 0
    Comm = 1
    Wait = 2
    Other = 3
    Total = 4


class Where(enum.IntEnum):
    Host = 0
    Device = 1
    Both = 2


class Level(enum.IntEnum):
    Off = 0
    Basic = 1
    Detail = 2


class Timer:
    __slots__ = ()

    def start(self, key, cls, where=None, parent_id=0) -> None:
        pass

    def stop(self) -> None:
        pass

    @staticmethod
    def current_span_id() -> int:
        return 0

    @staticmethod
    def set_level(level) -> None:
        pass

    @staticmethod
    def enabled() -> bool:
        return False

    @staticmethod
    def set_step(step) -> None:
        pass


class TimingRegistry:
    _one = None

    @staticmethod
    def instance() -> "TimingRegistry":
        if TimingRegistry._one is None:
            TimingRegistry._one = TimingRegistry()
        return TimingRegistry._one

    def init(self, rank, local_rank, world_size, run_id, device_id, output_dir) -> None:
        pass

    def set_level(self, level) -> None:
        pass

    def enabled(self) -> bool:
        return False

    def set_step(self, step) -> None:
        pass

    def flush(self) -> None:
        pass

    def close(self) -> None:
        pass
