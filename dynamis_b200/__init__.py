"""dynamis_b200 — B200 (sm_100a) implementation of the Dynamis per-step data-parallel hot path.

Radius graph, space-filling-curve partition, halo maps and halo exchange behind the reference's
own Python-facing names.  The compute lives in ``libdynb.so`` (hand-written CUDA, C ABI in
``include/dynb.h``); there is no CPU or PyTorch fallback.
"""

from .graph import (  # noqa: F401
    launches_per_graph,
    owned_graph,
    plan_radius_graph,
    radius_graph_pbc,
    radius_graph_pbc_counts_ex,
    radius_graph_pbc_cuda,
    radius_graph_pbc_ex,
    radius_graph_pbc_with_dist,
)
from .exchange import (  # noqa: F401
    Exchanger,
    FeatureExchanger,
    FeaturePushToExchange,
    GPUDirectExchanger,
    IPCExchanger,
    PythonNCCLExchanger,
    drift_flags,
    push_buffer_create,
    supports_fabric_handles,
)
from .halo import extract_halo_info, filter_edges_to_radius  # noqa: F401
from .partition import (  # noqa: F401
    KDTreePartitioner,
    SFCCurveType,
    SFCPartitioner,
    SimpleSpatialPartitioner,
    kdtree_partition_labels,
    launches_per_partition,
    sfc_keys,
    sfc_partition_labels,
)
from .sim_state import DRIFT_BREACH, DRIFT_TRIP, SimState, scatter_rows  # noqa: F401
from .state import (  # noqa: F401
    DistEnvironment,
    DynamisState,
    MolecularInfo,
    PartitionMessagePassingInfo,
    SimulationConfig,
)

from . import integrators  # noqa: F401,E402
from .dist_env import TorchDistEnv  # noqa: F401,E402
from .migrate import DistributedSimState  # noqa: F401,E402


def install_shim() -> str:
    """Puts dynamis_b200/shim first on sys.path, so that ``import dynamis_state`` / ``import dynamis_model``
    resolve to this implementation for the reference's unchanged callers.  Returns the directory."""
    import os
    import sys

    d = os.path.join(os.path.dirname(os.path.abspath(__file__)), "shim")
    if d in sys.path:
        sys.path.remove(d)
    sys.path.insert(0, d)
    return d
