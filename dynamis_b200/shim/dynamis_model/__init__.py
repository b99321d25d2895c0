"""`dynamis_model` as the reference's callers import it (reference:
dynamis_model/src/dynamis_model/__init__.py:5-14), backed by dynamis_b200."""

from dynamis_model.potential import DynamisModel
import dynamis_model.dynamis_model_impl as dynamis_model_impl

FeatureExchanger = dynamis_model_impl.FeatureExchanger

__all__ = ["DynamisModel", "FeatureExchanger"]
