"""Comparators measured on the same box: NCCL collectives and NCCL + cuBLAS tensor-parallel MLP."""
