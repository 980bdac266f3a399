"""ctypes binding of the C ABI declared in include/sglang_b200.h.

There is no fallback: if the CUDA library has not been built, importing this
module raises, and every op in the package fails with it.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
# SGLANG_B200_LIB names another build of the same C ABI (a library compiled with different tuning constants)
LIB_PATH = os.environ.get("SGLANG_B200_LIB") or os.path.join(_PKG, "lib", "libsglang_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python -m sglang_b200.build` "
        "(the sm_100a CUDA library is the only implementation; there is no CPU or Triton fallback)"
    )

lib = C.CDLL(LIB_PATH)

_vp, _i64, _i32, _f32 = C.c_void_p, C.c_int64, C.c_int, C.c_float

SIGNATURES = {
    "sglb200_last_error": (C.c_char_p, []),
    "sglb200_abi_version": (_i32, []),
    "sglb200_check_device": (_i32, [_i32]),
    "sglb200_per_token_group_quant_fp8": (_i32, [_vp, _i32, _vp, _vp, _i64, _i64, _i32, _f32, _f32, _f32, _i64, _i64, _vp]),
    "sglb200_silu_and_mul": (_i32, [_vp, _vp, _i32, _i64, _i64, _vp]),
    "sglb200_silu_and_mul_quant_fp8": (_i32, [_vp, _i32, _vp, _vp, _i64, _i64, _i32, _f32, _vp, _vp]),
    "sglb200_silu_and_mul_masked_quant_fp8": (_i32, [_vp, _i32, _vp, _vp, _i32, _i64, _i64, _i32, _f32, _vp, _vp]),
    "sglb200_moe_align_workspace_bytes": (_i64, [_i64, _i32]),
    "sglb200_moe_align_block_size": (_i32, [_vp, _i64, _i32, _i32, _vp, _vp, _vp, _vp, _i32, _vp, _i64, _vp]),
    "sglb200_moe_align_set_cooperative": (None, [_i32]),
    "sglb200_moe_align_block_size_noalloc": (_i32, [_vp, _i64, _i32, _i32, _vp, _vp, _vp, _i32, _vp]),
    "sglb200_moe_sum_reduce": (_i32, [_vp, _vp, _i32, _i64, _i64, _i64, _f32, _vp]),
    "sglb200_moe_sum_reduce_masked": (_i32, [_vp, _vp, _vp, _i32, _i64, _i64, _i64, _f32, _vp]),
    "sglb200_moe_align_drop_filtered": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _vp]),
    "sglb200_gather_sum_rows": (_i32, [_vp, _vp, _vp, _i32, _i64, _i32, _i64, _i64, _f32, _vp]),
    "sglb200_shuffle_mul_sum": (_i32, [_vp, _vp, _vp, _vp, _i32, _i64, _i32, _i64, _vp]),
    "sglb200_topk_softmax": (_i32, [_vp, _i32, _i64, _i32, _i32, _i32, _f32, _vp, _vp, _vp, _vp]),
    "sglb200_topk_sigmoid": (_i32, [_vp, _i32, _i64, _i32, _i32, _i32, _vp, _vp, _vp, _vp]),
    "sglb200_moe_fused_gate": (_i32, [_vp, _vp, _i32, _i64, _i32, _i32, _i32, _i32, _i32, _f32, _i32, _vp, _vp, _vp]),
    "sglb200_gather_rows_fp8": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _i64, _i64, _vp]),
    "sglb200_gemm_workspace_bytes": (_i64, [_i64, _i64, _i64]),
    "sglb200_fp8_blockwise_scaled_mm": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _vp, _i64, _vp]),
    "sglb200_fp8_blockwise_grouped_mm": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _i64, _i64, _i32, _i32, _vp]),
    "sglb200_gemm_status": (_i32, []),
    "sglb200_gemm_status_clear": (_i32, []),
    "sglb200_stream_status_clear": (_i32, []),
    "sglb200_comm_status_clear": (_i32, []),
    "sglb200_gemm_set_wait_probes": (None, [C.c_uint32]),
    "sglb200_stream_status": (_i32, []),
    "sglb200_stream_set_wait_probes": (None, [C.c_uint32]),
    "sglb200_comm_alloc": (_i32, [_i64, C.POINTER(_vp)]),
    "sglb200_comm_free": (_i32, [_vp]),
    "sglb200_comm_ipc_export": (_i32, [_vp, _vp]),
    "sglb200_comm_ipc_open": (_i32, [_vp, C.POINTER(_vp)]),
    "sglb200_comm_ipc_close": (_i32, [_vp]),
    "sglb200_comm_flag_bytes": (_i64, []),
    "sglb200_comm_status": (_i32, []),
    "sglb200_push_rows_per_owner": (_i64, [_i64, _i32]),
    "sglb200_fp8_blockwise_scaled_mm_push": (_i32, [_vp, _vp, _vp, _vp, C.POINTER(_vp), _i32, _i32, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _vp]),
    "sglb200_push_prepare": (_i32, [C.POINTER(_vp), _i32, _i64, _i64, _i32]),
    "sglb200_reduce_gather": (_i32, [_vp, C.POINTER(_vp), C.POINTER(_vp), _vp, _i32, _i32, _i64, _i64, _i32, _i32, _vp]),
    "sglb200_comm_set_wait_probes": (None, [C.c_uint32]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)  # AttributeError here = the .so is older than the header: rebuild
    _fn.restype = _res
    _fn.argtypes = _args


def check(rc: int) -> None:
    """Turn a non-zero return code of the C ABI into the exception the reference op would raise."""
    if rc != 0:
        msg = lib.sglb200_last_error().decode("utf-8", "replace")
        if rc == -2:
            raise NotImplementedError(msg)
        raise RuntimeError(msg)
