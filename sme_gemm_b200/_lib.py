"""ctypes binding of the C ABI declared in include/smeg_api.h.

The library must have been built (python -m sme_gemm_b200.build).  There is no
fallback: a missing library raises, and every non-zero return code raises
SmegError.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libsmeg_b200.so")


class SmegError(RuntimeError):
    def __init__(self, fn: str, rc: int):
        self.rc = rc
        meaning = {-1: "bad block size", -2: "allocation / copy failed", -3: "form not supported by this build",
                   -4: "bad argument", -5: "no usable sm_100 device", -6: "launch failed",
                   -7: "a kernel abandoned a bounded wait"}.get(rc, "error")
        super().__init__(f"{fn} returned {rc} ({meaning})")


class EpNode(C.Structure):
    """EpNode, csrc/epilogue.h:214-229 of the reference (32 bytes)."""

    _fields_ = [("op", C.c_uint32), ("aux", C.c_uint32), ("scalar", C.c_float), ("ptr", C.c_void_p),
                ("ld", C.c_size_t)]


class EpDesc16(C.Structure):
    """ep_desc16, csrc/epilogue.h:233-236."""

    _fields_ = [("n_nodes", C.c_uint32), ("nodes", C.POINTER(EpNode))]


assert C.sizeof(EpNode) == 32 and EpNode.ptr.offset == 16 and EpNode.ld.offset == 24

_sz, _vp, _u32, _i = C.c_size_t, C.c_void_p, C.c_uint32, C.c_int
_pp = C.POINTER(C.c_void_p)
_epp = C.POINTER(EpDesc16)

# name -> (restype, argtypes); the same list the header declares
SIGNATURES = {
    "smeg_version": (C.c_char_p, []),
    "smeg_device_info": (_i, [C.POINTER(_i), C.POINTER(_sz)]),
    "smeg_last_status": (C.c_uint, []),
    "smeg_trace": (None, [_i]),
    "smeg_q4_create": (_i, [_vp, _vp, _vp, _sz, _sz, _sz, _pp]),
    "smeg_q4_quantize": (_i, [_vp, _i, _sz, _sz, _sz, _i, _pp]),
    "smeg_q4_from_band": (_i, [_vp, _vp, _vp, _sz, _sz, _sz, _pp]),
    "smeg_q4_destroy": (None, [_vp]),
    "smeg_q4_n": (_sz, [_vp]),
    "smeg_q4_k": (_sz, [_vp]),
    "smeg_q4_block": (_sz, [_vp]),
    "smeg_q4_unpack": (_i, [_vp, _vp, _vp]),
    "smeg_q4_device_bytes": (_sz, [_vp]),
    "smeg_q2_create": (_i, [_vp, _vp, _sz, _sz, _sz, _vp, _pp]),
    "smeg_q2_quantize": (_i, [_vp, _i, _sz, _sz, _sz, _vp, _pp]),
    "smeg_q1_create": (_i, [_vp, _vp, _i, _sz, _sz, _sz, _pp]),
    "smeg_q1_quantize": (_i, [_vp, _i, _sz, _sz, _sz, _pp]),
    "smeg_q2_from_band": (_i, [_vp, _vp, _sz, _sz, _sz, _vp, _pp]),
    "smeg_q1_from_band": (_i, [_vp, _vp, _sz, _sz, _sz, _pp]),
    "smeg_lowbit_destroy": (None, [_vp]),
    "smeg_lowbit_n": (_sz, [_vp]),
    "smeg_lowbit_k": (_sz, [_vp]),
    "smeg_lowbit_block": (_sz, [_vp]),
    "smeg_lowbit_bits": (_i, [_vp]),
    "smeg_lowbit_unpack": (_i, [_vp, _vp, _vp]),
    "smeg_lowbit_device_bytes": (_sz, [_vp]),
    "smeg_packed_code_bytes": (_sz, [_i, _sz, _sz]),
    "smeg_packed_scale_elems": (_sz, [_i, _sz, _sz, _sz]),
    "smeg_host_pack": (_i, [_i, _vp, _i, _vp, _sz, _sz, _sz, _vp, _vp]),
    "smeg_host_unpack": (_i, [_i, _vp, _vp, _sz, _sz, _sz, _vp, _vp]),
    "smeg_host_q4_quantize": (_i, [_vp, _i, _sz, _sz, _sz, _vp, _vp]),
    "smeg_host_q2_quantize": (_i, [_vp, _i, _sz, _sz, _sz, _vp, _vp, _vp]),
    "smeg_host_q1_quantize": (_i, [_vp, _i, _sz, _sz, _sz, _vp, _vp]),
    "smeg_matmul_q4_f16_dev": (_i, [_vp, _vp, _vp, _sz, _epp, _vp]),
    "smeg_matmul_q4_bf16_dev": (_i, [_vp, _vp, _vp, _sz, _epp, _vp]),
    "smeg_matmul_lowbit_dev": (_i, [_vp, _vp, _vp, _sz, _epp, _vp]),
    "smeg_lowbit_prepare_f16": (_i, [_vp]),
    "smeg_matmul_lowbit_f16_dev": (_i, [_vp, _vp, _vp, _sz, _epp, _vp]),
    "smeg_matmul_lowbit_static_dev": (_i, [_vp, _vp, _vp, _sz, _epp, _vp]),
    "smeg_matmul_lowbit_debug_dev": (_i, [_vp, _vp, _vp, _sz, _vp, _vp, _vp, _vp]),
    "smeg_glu_f16_dev": (_i, [_vp, _vp, _sz, _sz, _u32, _vp]),
    "smeg_add_f16_to_f32_dev": (_i, [_vp, _vp, _sz, _vp]),
    "smeg_act_f16_dev": (_i, [_vp, _vp, _sz, _u32, _vp]),
    "smeg_f32_to_f16_dev": (_i, [_vp, _vp, _sz, _vp]),
    "smeg_f16_to_f32_dev": (_i, [_vp, _vp, _sz, _vp]),
    "smeg_norm_rows_dev": (_i, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, C.c_float, _i, _vp]),
    "smeg_rms_scales_dev": (_i, [_vp, _vp, _sz, _sz, C.c_float, _vp]),
    "smeg_matmul_q4_f16": (_i, [_vp, _vp, _vp, _sz, _epp]),
    "smeg_matmul_q4_bf16": (_i, [_vp, _vp, _vp, _sz, _epp]),
    "smeg_matmul_lowbit": (_i, [_vp, _vp, _vp, _sz, _epp]),
    "smeg_matmul_lowbit_f16": (_i, [_vp, _vp, _vp, _sz, _epp]),
    "smeg_dense_create": (_i, [_vp, _sz, _sz, _i, _pp]),
    "smeg_dense_destroy": (None, [_vp]),
    "smeg_dense_n": (_sz, [_vp]),
    "smeg_dense_k": (_sz, [_vp]),
    "smeg_gemm_dense_dev": (_i, [_vp, _vp, _vp, _sz, C.c_uint16, _i, _epp, _vp]),
    "smeg_gemm_dense": (_i, [_vp, _vp, _vp, _sz, C.c_uint16, _i, _epp]),
    "smeg_mlp_create": (_i, [_vp, _vp, _u32, _pp]),
    "smeg_mlp_destroy": (None, [_vp]),
    "smeg_mlp_accumulate_dev": (_i, [_vp, _vp, _vp, _sz, _vp]),
    "smeg_mlp_accumulate": (_i, [_vp, _vp, _vp, _sz]),
    "smeg_mlp_partial_dev": (_i, [_vp, _vp, _vp, _sz, _vp]),
    "smeg_matmul_q4_partial_dev": (_i, [_vp, _vp, _vp, _sz, _vp]),
    "smeg_kv_append_dev": (_i, [_vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz, _vp]),
    "smeg_attn_kv_causal_dev": (_i, [_vp, _vp, _i, _sz, _vp, _vp, _sz, _sz, _sz, _sz, _sz, C.c_float, _vp]),
    "smeg_mlp_finish_dev": (_i, [_vp, _vp, _sz, _vp]),
    "smeg_mlp_reduce_finish_dev": (_i, [_vp, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), _i, _i, _sz, _u32, _i, _vp]),
    "smeg_mlp_partial_push_dev": (_i, [_vp, _vp, C.POINTER(C.c_uint64), _i, _i, _sz, _vp]),
    "smeg_mlp_reduce_finish_pushed_dev": (_i, [_vp, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), _i, _i, _sz, _sz, _u32, _vp]),
    "gemm_sme_f16f16_q4": (_i, [_sz, _sz, _sz, _vp, _vp, _vp, _vp, _vp, _sz, _epp]),
    "gemm_sme_b16b16_q4": (_i, [_sz, _sz, _sz, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _epp]),
    "gemm_sme_f16_q1": (_i, [_sz, _sz, _sz, _vp, _vp, _vp, _vp, _sz, _epp]),
    "gemm_sme_f16_q2": (_i, [_sz, _sz, _sz, _vp, _vp, _vp, _vp, _vp, _sz, _epp]),
    "gemm_sme_f16f16_q1": (_i, [_sz, _sz, _sz, _vp, _vp, _vp, _vp, _sz, _epp]),
    "gemm_sme_f16f16_q2": (_i, [_sz, _sz, _sz, _vp, _vp, _vp, _vp, _vp, _sz, _epp]),
    "neon_glu_f16": (None, [_vp, _vp, _sz, _sz, _u32]),
    "neon_add_f16_to_f32": (None, [_vp, _vp, _sz]),
    "neon_act_f16": (None, [_vp, _vp, _sz, _u32]),
    "neon_f32_to_f16": (None, [_vp, _vp, _sz]),
    "neon_f16_to_f32": (None, [_vp, _vp, _sz]),
    "smeg_forget": (None, [_vp]),
}

_lib = None


def lib() -> C.CDLL:
    """The loaded CUDA library.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m sme_gemm_b200.build` "
                               "(there is no CPU fallback)")
        _lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(_lib, name)
            fn.restype = res
            fn.argtypes = args
    return _lib


def check(fn: str, rc: int) -> None:
    if rc != 0:
        raise SmegError(fn, rc)
