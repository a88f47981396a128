"""Model blocks built on the fused tensor-parallel operators."""
from .tp_mlp import TensorParallelMLP  # noqa: F401
