"""Process-wide drift-watchdog flags (reference: dynamis_model/src/dynamis_model/comm/drift_flags.py):
module-level ``enable`` / ``get`` / ``disable`` over the registry the exchangers of dynamis_b200 read."""

from dynamis_b200.exchange import DriftFlags, drift_flags as _registry  # noqa: F401

enable = _registry.enable
get = _registry.get
disable = _registry.disable
