"""Tensor-parallel building blocks: collectives fused with the compute next to them."""
from .tp import allgather_gemm, allreduce_residual_rmsnorm, gemm_reduce_scatter  # noqa: F401
