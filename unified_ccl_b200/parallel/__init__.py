"""Tensor-parallel building blocks: collectives fused with the compute next to them."""
from .moe import MoeDispatcher, quantize_fp8_block128  # noqa: F401
from .tp import allgather_gemm, allreduce_residual_rmsnorm, gemm_reduce_scatter  # noqa: F401
