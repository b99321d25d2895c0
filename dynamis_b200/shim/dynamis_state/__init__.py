"""`dynamis_state` as the reference's callers import it (reference:
dynamis_state/src/dynamis_state/__init__.py:1-102), backed by dynamis_b200."""

import dynamis_state.dynamis_state_impl as dynamis_state_impl

MolecularInfo = dynamis_state_impl.MolecularInfo
DistEnvironment = dynamis_state_impl.DistEnvironment
SimulationConfig = dynamis_state_impl.SimulationConfig
PartitionMessagePassingInfo = dynamis_state_impl.PartitionMessagePassingInfo
DynamisState = dynamis_state_impl.DynamisState

SimpleSpatialPartitioner = dynamis_state_impl.SimpleSpatialPartitioner
KDTreePartitioner = dynamis_state_impl.KDTreePartitioner
SFCPartitioner = dynamis_state_impl.SFCPartitioner
SFCCurveType = dynamis_state_impl.SFCCurveType

from dynamis_state.radius_graph_pbc_cuda import radius_graph_pbc_cuda  # noqa: E402
from dynamis_state.state_wrapper import TorchDistEnv  # noqa: E402
from dynamis_state.dist_graph_builder import BuildMode, DistBuildGraphResult, DistGraphBuilder  # noqa: E402
from dynamis_state.io import TrajectoryReader, TrajectoryWriter, translate_dynamis_to_xyz  # noqa: E402
from dynamis_b200.sim_state import SimState  # noqa: E402

# Timing is outside the hot path: compiled out, as in a reference build with its timing option off.
TimingRegistry = dynamis_state_impl.TimingRegistry
TimerClass = dynamis_state_impl.TimerClass
Where = dynamis_state_impl.Where
Level = dynamis_state_impl.Level
TIMING_ENABLED = dynamis_state_impl.TIMING_ENABLED
Timer = dynamis_state_impl.Timer

__all__ = [
    "MolecularInfo", "DistEnvironment", "SimulationConfig", "PartitionMessagePassingInfo", "DynamisState",
    "SimpleSpatialPartitioner", "KDTreePartitioner", "SFCPartitioner", "SFCCurveType", "TrajectoryReader",
    "TrajectoryWriter", "translate_dynamis_to_xyz", "radius_graph_pbc_cuda", "TorchDistEnv", "DistGraphBuilder",
    "DistBuildGraphResult", "BuildMode", "SimState", "Timer", "TimingRegistry", "TimerClass", "Where", "Level",
    "TIMING_ENABLED",
]
