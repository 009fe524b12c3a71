"""Kernel-backed operators of ghost_flow_b200 (see ``gemm``, ``fused``, ``optim_kernels``)."""
from . import _lib  # noqa: F401
from .gemm import linear, matmul, matmul_nn, matmul_nt, matmul_tn, matmul_tt, gemm_raw  # noqa: F401
from .fused import (  # noqa: F401
    rms_norm, rms_norm_ref, layer_norm, rope, rope_ref, rope_tables, swiglu, unary, gelu, op_chain,
    cross_entropy, flash_attention, attention_ref, split_qkv,
)
