"""Blackwell-native unified collective communication library (Python side).

The native code lives in ``libuccl.so`` (host runtime + sm_100a kernels) and the pybind11
module ``_uccl_bindings`` next to this file; both are built in-tree by ``make`` (or
``python -c "import __graft_entry__ as g; g.build()"``).  Importing this package never
falls back to a pure-Python implementation: if the extension is missing the import fails
with the build command in the message.
"""
import os as _os

# The copy-engine transports keep one stream per peer (plus one for flags) busy next to the caller's
# stream, some of them parked on a memory value.  With the CUDA default of 8 hardware queues per
# context, streams share queues and a parked one holds up whatever was queued behind it.  The
# variable is read when the context is created, so it is set here unless the user chose a value.
_os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")

try:
    from . import _uccl_bindings as _C  # noqa: F401
except ImportError as _e:  # pragma: no cover - exercised only on a broken checkout
    raise ImportError(
        "unified_ccl_b200: native extension not built; run `make -j` in "
        f"{_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__)))} ({_e})"
    ) from _e

__version__ = "0.1.0"

from .communicator import Communicator, Window, get_unique_id  # noqa: E402,F401



def tuning_table(name: str = "b200_x8_nvswitch") -> str:
    """Path of a measured tuner table shipped with the package (written by ``benchmarks/sweep.py --tune``
    on the named machine); pass it to ``Communicator.load_tuning`` or set ``UCCL_TUNE_FILE``."""
    path = _os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "tuning", name + ".json")
    if not _os.path.exists(path):
        raise FileNotFoundError(path)
    return path


__all__ = ["Communicator", "Window", "get_unique_id", "tuning_table"]
