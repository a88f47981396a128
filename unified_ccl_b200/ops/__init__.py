"""Single-GPU compute ops backed by hand-written sm_100a kernels."""
from .gemm import gemm_bf16  # noqa: F401
