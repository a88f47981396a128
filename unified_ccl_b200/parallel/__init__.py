"""Tensor-parallel building blocks: collectives fused with the compute next to them."""
from .moe import MoeDispatcher, quantize_fp8_block128  # noqa: F401
from .tp import (allgather_gemm, allreduce_residual_rmsnorm, autotune_allreduce_residual_rmsnorm,  # noqa: F401
                 gemm_reduce_scatter)
