"""B200 (sm_100a) implementation of sme-gemm's weight-quantised matmul hot path.

The compute lives in the CUDA library built from sme_gemm_b200/csrc (C ABI in
include/smeg_api.h); this package is the host-side mirror of the reference's
API for that path.
"""
from ._lib import LIB_PATH, SmegError, lib  # noqa: F401
from .host import (  # noqa: F401
    Block, Epilogue, Gate, GatedLinear, Gemm, KvCache, Linear, Mlp, Norm, Packed, SelfAttention, Q1Weights, Q2Params, Q2Weights, Q2_BLOCK, Q2_TERNARY,
    Q4Params, Q4Weights, Q4_BLOCK, WeightLayout, device_info, interleave_gate_up, last_status, matmul_lowbit_debug,
    matmul_q1, matmul_q1_ep, matmul_q1_mopa, matmul_q1_mopa_ep, matmul_q2, matmul_q2_ep, matmul_q2_mopa,
    matmul_q2_mopa_ep, matmul_q4, matmul_q4_bf16, matmul_q4_bf16_ep, matmul_q4_ep, prepack_bf16, prepack_f16,
)
