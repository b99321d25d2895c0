"""Stands where the reference's compiled module `dynamis_model.dynamis_model_impl` stands
(reference: dynamis_model/src/dynamis_model_bindings.cpp:5-105)."""

from dynamis_b200.exchange import FeatureExchanger, IPCExchanger, push_buffer_create, supports_fabric_handles  # noqa: F401
