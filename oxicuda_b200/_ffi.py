"""ctypes binding of liboxq_b200.so (the C ABI declared in include/oxq.h).

There is no fallback: if the shared library is missing this module raises, and every launch on a
machine without an sm_100 GPU returns an error status from the library itself.
"""
from __future__ import annotations

import ctypes as C
import os

from . import _build

_i32, _i64, _sz, _vp, _int, _f32p = C.c_int32, C.c_int64, C.c_size_t, C.c_void_p, C.c_int, C.c_void_p

# symbol -> (restype, argtypes); mirrors include/oxq.h one to one
SIGNATURES = {
    "oxq_handle_create": (_i32, [_int, _vp, C.POINTER(_vp)]),
    "oxq_handle_destroy": (_i32, [_vp]),
    "oxq_set_stream": (_i32, [_vp, _vp]),
    "oxq_last_error_string": (C.c_char_p, [_vp]),
    "oxq_status_name": (C.c_char_p, [_i32]),
    "oxq_version": (_i32, []),
    "oxq_device_status": (_i32, [_vp, C.POINTER(_i32)]),
    "oxq_int8_quant_rows": (_i32, [_vp, _vp, _i64, _i64, _vp, _vp, _int]),
    "oxq_int8_dequant_rows": (_i32, [_vp, _vp, _vp, _i64, _i64, _vp]),
    "oxq_absmax": (_i32, [_vp, _vp, _int, _i64, _vp]),
    "oxq_fp8_quant": (_i32, [_vp, _vp, _int, _i64, _vp, _vp, _int]),
    "oxq_fp8_quant_dynamic": (_i32, [_vp, _vp, _int, _i64, _vp, _vp]),
    "oxq_fp8_dequant": (_i32, [_vp, _vp, _i64, _vp, _vp, _int, _int]),
    "oxq_int4g_quant_pack": (_i32, [_vp, _vp, _int, _i64, _i64, _int, _vp, _vp, _vp, _int]),
    "oxq_int4g_dequant": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _int, _vp, _int]),
    "oxq_int4g_quant_pack_f32": (_i32, [_vp, _vp, _i64, _i64, _int, _vp, _vp, _vp, _int]),
    "oxq_int4g_dequant_f32": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _int, _vp]),
    "oxq_fp4_microscale_quant": (_i32, [_vp, _vp, _i64, _i64, _vp, _vp]),
    "oxq_fp4_microscale_dequant": (_i32, [_vp, _vp, _vp, _i64, _i64, _vp]),
    "oxq_dnn_int4_quant": (_i32, [_vp, _vp, _i64, _i64, _int, _vp, _vp, _vp]),
    "oxq_dnn_int4_dequant": (_i32, [_vp, _vp, _vp, _i64, _i64, _int, _vp]),
    "oxq_dnn_block_scaled_quant": (_i32, [_vp, _vp, _int, _i64, _i64, _vp, _vp]),
    "oxq_dnn_fused_dequant_gemv": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int]),
    "oxq_swiglu_interleaved": (_i32, [_vp, _vp, _i64, _i64, _vp]),
    "oxq_sf_mma_bytes": (_sz, [_i64, _i64]),
    "oxq_mxfp8_quant": (_i32, [_vp, _vp, _int, _i64, _i64, _vp, _vp, _vp]),
    "oxq_mxfp8_dequant": (_i32, [_vp, _vp, _vp, _i64, _i64, _vp, _int]),
    "oxq_nvfp4_quant": (_i32, [_vp, _vp, _int, _i64, _i64, _vp, _vp, _vp, _vp]),
    "oxq_nvfp4_dequant": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _vp, _int]),
    "oxq_int8_quant_tensor": (_i32, [_vp, _vp, _int, _i64, _vp, _vp]),
    "oxq_int8_dequant_tensor": (_i32, [_vp, _vp, _vp, _i64, _vp, _int]),
    "oxq_int8_block_quant": (_i32, [_vp, _vp, _i64, _i64, _vp, _vp]),
    "oxq_int8_block_dequant": (_i32, [_vp, _vp, _vp, _i64, _i64, _vp]),
    "oxq_nf4_quant": (_i32, [_vp, _vp, _i64, _i64, _vp, _vp]),
    "oxq_nf4_dequant": (_i32, [_vp, _vp, _vp, _i64, _i64, _vp, _int]),
    "oxq_nf4_thresholds": (_i32, [_vp]),
    "oxq_gemm_nf4": (_i32, [_vp, _i64, _i64, _i64, _vp, _vp, _vp, _i64, _vp]),
    "oxq_rmsnorm_fp8_quant_rows": (_i32, [_vp, _vp, _int, _vp, _i64, _i64, C.c_float, _vp, _vp]),
    "oxq_silu_gate_fp8_quant": (_i32, [_vp, _vp, _vp, _int, _i64, _vp, _vp]),
    "oxq_rmsnorm_int8_quant_rows": (_i32, [_vp, _vp, _int, _vp, _i64, _i64, C.c_float, _vp, _vp, _vp]),
    "oxq_smooth_col_absmax": (_i32, [_vp, _vp, _i64, _i64, _vp]),
    "oxq_smooth_scales": (_i32, [_vp, _vp, _vp, _i64, C.c_float, _vp]),
    "oxq_smooth_apply": (_i32, [_vp, _vp, _i64, _i64, _vp, _int]),
    "oxq_bias_add_bf16": (_i32, [_vp, _vp, _i64, _vp, _i64, _i64]),
    "oxq_gemm_fp8": (_i32, [_vp, _i64, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _vp, _i64]),
    "oxq_gemm_fp8_ex": (_i32, [_vp, _i64, _i64, _i64, C.c_float, _vp, _i64, _vp, _i64, _vp, _vp, C.c_float, _vp, _i64]),
    "oxq_gemm_bf16_ex": (_i32, [_vp, _i64, _i64, _i64, C.c_float, _vp, _i64, _vp, _i64, C.c_float, _vp, _i64]),
    "oxq_gemm_fp8_op": (_i32, [_vp, _i64, _i64, _i64, C.c_float, _vp, _i64, _int, _vp, _i64, _int, _vp, _vp, C.c_float, _vp, _i64]),
    "oxq_gemm_bf16_op": (_i32, [_vp, _i64, _i64, _i64, C.c_float, _vp, _i64, _int, _vp, _i64, _int, C.c_float, _vp, _i64]),
    "oxq_gemm_fp8_swiglu": (_i32, [_vp, _i64, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _vp, _i64]),
    "oxq_gemm_bf16": (_i32, [_vp, _i64, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _i64]),
    "oxq_gemm_bf16_swiglu": (_i32, [_vp, _i64, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _i64]),
    "oxq_gemm_w8a8": (_i32, [_vp, _i64, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _vp, _i64]),
    "oxq_gemm_w8a32": (_i32, [_vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp]),
    "oxq_gptq_workspace_bytes": (_i32, [_i64, _i64, _vp]),
    "oxq_gptq_quantize_layer": (_i32, [_vp, _vp, _i64, _i64, _vp, _int, _int, C.c_double, _vp, _vp, _vp, _vp, _vp, _sz]),
    "oxq_gemm_w4a16_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "oxq_gemm_w4a16": (_i32, [_vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _int, _vp, _vp, _sz]),
    "oxq_gemm_w4a16_static": (_i32, [_vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _int, _vp]),
    "oxq_multimem_all_reduce_bf16": (_i32, [_vp, _vp, _i64, _int, _int]),
    "oxq_multimem_all_reduce_bf16_2d": (_i32, [_vp, _vp, _i64, _i64, _i64, _int, _int]),
    "oxq_multimem_all_reduce_bf16_2d_sync": (_i32, [_vp, _vp, _i64, _i64, _i64, _int, _int, _vp, _vp]),
    "oxq_gemm_fp8_all_reduce": (_i32, [_vp, _i64, _i64, _i64, _vp, _i64, _vp, _i64, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _i64, _int, _int]),
    "oxq_comm_unique_id": (_i32, [_vp]),
    "oxq_comm_init": (_i32, [_vp, _vp, _int, _int]),
    "oxq_comm_destroy": (_i32, [_vp]),
    "oxq_comm_info": (_i32, [_vp, _vp, _vp, _vp]),
    "oxq_all_reduce_bf16": (_i32, [_vp, _vp, _i64]),
    "oxq_all_gather_bf16": (_i32, [_vp, _vp, _i64, _vp]),
    "oxq_mlp_swiglu_tp_workspace_bytes": (_i32, [_int, _i64, _i64, _i64, _vp]),
    "oxq_mlp_swiglu_tp": (_i32, [_vp, _vp, _i64, _vp, _vp, _vp, _sz, _int]),
    "oxq_gemm_mxfp8": (_i32, [_vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _i64]),
    "oxq_gemm_nvfp4": (_i32, [_vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64]),
}

_lib = None


def lib_path() -> str:
    return _build.LIB_PATH


def load():
    """Load the library (never builds it implicitly on a GPU box: the prebuilt file travels with the tree)."""
    global _lib
    if _lib is None:
        path = lib_path()
        if not os.path.exists(path):
            raise ImportError(
                f"{path} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'`. "
                "oxicuda_b200 has no CPU or PyTorch fallback.")
        lib = C.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)          # AttributeError here means the header and the library disagree
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib
