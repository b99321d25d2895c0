"""Base class of the model adapters (reference: dynamis_model/src/dynamis_model/potential.py): a
callable taking the distributed state and returning (energy, forces).  The reference wraps every
subclass's ``__call__`` in a timing span; timing is compiled out here, so the class is a plain ABC."""

from abc import ABC, abstractmethod
from typing import Any


class DynamisModel(ABC):
    def __init__(self) -> None:
        super().__init__()

    @abstractmethod
    def __call__(self, distributed_state, *args: Any, **kwds: Any):
        raise NotImplementedError

    def initialize_buffers(self, partition_info, device) -> None:
        """Called after every repartition; adapters set up their exchangers here."""
