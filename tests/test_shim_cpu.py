"""The drop-in packages: with dynamis_b200/shim first on sys.path, ``dynamis_state`` and
``dynamis_model`` resolve to this implementation under the reference's own import names.

Where the reference tree is present (this container; not the GPU box) the reference's own
``comm/exchanger.py``, ``comm/feature_push.py``, ``potential.py`` and the LJ model are loaded BY PATH,
unmodified, on top of the shim: every name they import must exist, their exchanger classes must
construct over our FeatureExchanger, and the single-rank paths (identity pushes) must run.  The GPU
side of the same proof — a caller written like the reference's LJ model, through the shim's imports
— is tests/test_lj_caller_gpu.py."""

import importlib.util
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("DYNB_REFERENCE", "/root/reference")

_CHILD = r'''
import importlib.util, os, sys
root, ref = sys.argv[1], sys.argv[2]
sys.path.insert(0, root)
import dynamis_b200 as D
D.install_shim()
import torch, torch.distributed as dist
import dynamis_state, dynamis_model

# every name the reference's package exports exists here
for name in ["MolecularInfo", "DistEnvironment", "SimulationConfig", "PartitionMessagePassingInfo", "DynamisState",
             "SimpleSpatialPartitioner", "KDTreePartitioner", "SFCPartitioner", "SFCCurveType", "TrajectoryReader",
             "TrajectoryWriter", "translate_dynamis_to_xyz", "radius_graph_pbc_cuda", "TorchDistEnv", "DistGraphBuilder",
             "DistBuildGraphResult", "BuildMode", "SimState", "Timer", "TimingRegistry", "TimerClass", "Where", "Level",
             "TIMING_ENABLED"]:
    assert hasattr(dynamis_state, name), name
impl = dynamis_model.dynamis_model_impl
for name in ["push_buffer_create", "supports_fabric_handles", "IPCExchanger", "FeatureExchanger"]:
    assert hasattr(impl, name), name
for name in ["allocate_ipc_buffer", "export_ipc_handle", "setup", "push_forward", "push_backward", "create_and_export_sync_handle",
             "setup_sync", "record_push_complete", "wait_for_pushes", "set_watchdog_flags", "clear_watchdog_flags", "teardown",
             "is_setup", "use_fabric", "supports_fabric_handles"]:
    assert hasattr(impl.IPCExchanger, name), name
for name in ["feature_push_forward", "feature_push_backward", "supports_fabric_handles", "allocate_ipc_buffer", "export_ipc_handle",
             "setup_ipc", "create_and_export_sync_handle", "setup_sync", "record_push_complete", "wait_for_pushes",
             "set_watchdog_flags", "clear_watchdog_flags", "teardown", "is_ipc_setup", "use_fabric", "set_ce_threshold_bytes",
             "ce_threshold_bytes"]:
    assert hasattr(impl.FeatureExchanger, name), name
env = dynamis_state.TorchDistEnv(is_distributed=False)
assert env.world_size == 1 and env.dist_env.world_size == 1

if os.path.isdir(ref):
    def load(name, rel):
        spec = importlib.util.spec_from_file_location(name, os.path.join(ref, rel))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
        return mod
    # the reference's own Python, unmodified, over the shim's compiled-module stand-ins
    pot = load("dynamis_model.potential", "dynamis_model/src/dynamis_model/potential.py")
    rex = load("dynamis_model.comm.exchanger", "dynamis_model/src/dynamis_model/comm/exchanger.py")
    rfp = load("dynamis_model.comm.feature_push", "dynamis_model/src/dynamis_model/comm/feature_push.py")
    lj = load("ref_lj", "dynamis_model/src/dynamis_model/empirical/lj_potential_model.py")
    g = rex.GPUDirectExchanger()
    assert type(g.exchanger) is impl.FeatureExchanger
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:29533", rank=0, world_size=1)
    x = torch.arange(12.0).reshape(4, 3)
    st = dynamis_state.DynamisState()
    st.local_partition_info = dynamis_state.PartitionMessagePassingInfo()
    out = rfp.FeaturePushToExchange.apply(x.clone().requires_grad_(True), st, g)   # single rank: identity, no device work
    assert torch.equal(out, x)
    n = rex.PythonNCCLExchanger()
    assert torch.equal(n.feature_push_forward(x, st.local_partition_info), x)
    model = lj.LennardJonesPotentialModel(torch.ones(1), torch.ones(1))
    assert isinstance(model, pot.DynamisModel) and type(model.position_exchanger.exchanger) is impl.FeatureExchanger
    model.initialize_buffers(st.local_partition_info, torch.device("cpu"))          # single rank: nothing to map
    assert model.position_exchanger.is_ipc_setup
    from dynamis_model.comm import drift_flags
    assert drift_flags.get("cpu") is None
    dist.destroy_process_group()
    print("reference callers loaded")
print("shim ok")
'''


def test_shim_packages_resolve_and_reference_callers_load():
    r = subprocess.run([sys.executable, "-c", _CHILD, ROOT, REF], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "shim ok" in r.stdout
    if os.path.isdir(REF):
        assert "reference callers loaded" in r.stdout
