"""Drop-in import name of the reference project: ``from uccl import Communicator``."""
from unified_ccl_b200 import Communicator, get_unique_id  # noqa: F401
from unified_ccl_b200 import __version__  # noqa: F401

__all__ = ["Communicator", "get_unique_id"]
