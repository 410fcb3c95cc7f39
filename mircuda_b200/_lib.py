"""Loads ``libmircuda_b200.so`` and declares the C ABI of ``include/mircuda_b200.h``.

There is no fallback: if the library is missing or a symbol cannot be resolved the import
fails with an error that says how to build it.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

LIBRARY = Path(__file__).resolve().parent / "libmircuda_b200.so"

_vp = ctypes.c_void_p
_i = ctypes.c_int
_u32 = ctypes.c_uint32
_f = ctypes.c_float
_sz = ctypes.c_size_t
_vpp = ctypes.POINTER(ctypes.c_void_p)

# name -> (restype, argtypes); mirrors include/mircuda_b200.h one to one.
SIGNATURES = {
    "mircuda_b200_version": (_u32, []),
    "mircuda_cutlass_version": (_u32, []),
    "mircuda_b200_mxfp8_quantize_bf16": (_i, [_vp, _vp, _vp, _u32, _u32, _vp]),
    "mircuda_b200_mxfp8_quantize_bf16_blocks": (_i, [_vp, _vp, _vp, _u32, _u32, _u32, _vp]),
    "mircuda_b200_mxfp8_swizzle_scales": (_i, [_vp, _vp, _u32, _u32, _vp]),
    "mircuda_mxfp8_tc_create": (_i, [_i, _i, _i, _vp, _vpp]),
    "mircuda_mxfp8_tc_workspace_bytes": (_sz, [_vp]),
    "mircuda_mxfp8_tc_execute": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "mircuda_mxfp8_tc_destroy": (None, [_vp]),
    "mircuda_b200_mxfp8_tc_wait_probe": (_i, [_vp, _vp]),
    "mircuda_b200_mxfp8_bf16": (_i, [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _vp]),
    "mircuda_fp4_create": (_i, [_i, _i, _i, _vp, _vpp]),
    "mircuda_fp4_workspace_bytes": (_sz, [_vp]),
    "mircuda_fp4_execute": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _f]),
    "mircuda_fp4_destroy": (None, [_vp]),
    "mircuda_fp4_vector_create": (_i, [_i, _i, _vp, _vpp]),
    "mircuda_fp4_vector_execute": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _f]),
    "mircuda_fp4_vector_destroy": (None, [_vp]),
    "mircuda_b200_fp4_vector_execute_static": (_i, [_i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _f]),
    "mircuda_dense_vector_create": (_i, [_i, _i, _i, _vp, _vpp]),
    "mircuda_dense_vector_execute": (_i, [_vp, _vp, _vp, _vp, _vp, _f, _f]),
    "mircuda_dense_vector_destroy": (None, [_vp]),
    "mircuda_b200_nvfp4_vector_create": (_i, [_i, _i, _i, _vp, _vpp]),
    "mircuda_b200_nvfp4_vector_execute": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _f]),
    "mircuda_b200_nvfp4_vector_destroy": (None, [_vp]),
    "mircuda_b200_nvfp4_global_scale": (_i, [_vp, _sz, _vp, _vp]),
    "mircuda_b200_nvfp4_quantize_bf16": (_i, [_vp, _vp, _vp, _vp, _u32, _u32, _vp]),
    "mircuda_variable_grouped_bf16_create": (_i, [_i, _i, _i, _i, _vp, _vpp]),
    "mircuda_variable_grouped_bf16_execute": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _f]),
    "mircuda_variable_grouped_bf16_destroy": (None, [_vp]),
}

_b = ctypes.c_bool
SIGNATURES.update({
    "mircuda_marlin_nvfp4_repack": (_i, [_vp, _vp, _vp, _i, _i, _i]),
    "mircuda_marlin_nvfp4_repack_pair": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i]),
    "mircuda_marlin_mxfp4_repack": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _b]),
    "mircuda_marlin_mxfp4_prepare_scales": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _b]),
    "mircuda_marlin_nvfp4_prepare_scales": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i]),
    "mircuda_marlin_prepare_moe_routes": (_i, [_vp] * 8 + [_i, _i, _i]),
    "mircuda_marlin_nvfp4_dense_execute": (_i, [_vp] * 7 + [_i, _i, _i, _i, _vp, _b]),
    "mircuda_b200_mxfp8_tc_execute_gather": (_i, [_vp] * 6 + [_vpp, _i, _i, _i, _vp]),
    "mircuda_b200_column_gather_create": (_i, [_u32, _u32, _vpp]),
    "mircuda_b200_column_gather_send": (_i, [_vp, _vpp, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint64,
                                             ctypes.c_uint64, _vp]),
    "mircuda_b200_column_gather_join": (_i, [_vp, _vp]),
    "mircuda_b200_column_gather_destroy": (None, [_vp]),
    "mircuda_b200_variable_grouped_bf16_create_indexed": (_i, [_i, _i, _i, _i, _i, _vp, _vpp]),
    "mircuda_b200_variable_grouped_bf16_execute_indexed": (_i, [_vp] * 8 + [_f]),
    "mircuda_b200_moe_scatter_rows_bf16": (_i, [_vp, _vp, _vp, _vp, _u32, _u32, _vp]),
    "mircuda_b200_moe_swiglu_bf16": (_i, [_vp, _vp, _u32, _vp, _u32, _vp]),
    "mircuda_b200_moe_combine_rows_bf16": (_i, [_vp, _vp, _vp, _vp, _u32, _u32, _u32, _vp]),
    "mircuda_b200_moe_group_offsets": (_i, [_vp, _vp, _vp, _u32, _u32, _u32, _u32, _vp]),
    "mircuda_b200_moe_expert_layout": (_i, [_vp, _u32, _u32, _u32, _u32, _vp, _vp, _vp, _vp, _u32, _vp, _vp]),
    "mircuda_b200_nvfp4_quantize_rows_bf16": (_i, [_vp, _vp, _vp, _vp, _u32, _u32, _vp]),
    "mircuda_b200_moe_dispatch_rows_bf16": (_i, [_vp] * 5 + [_vpp, _u32, _vp, _u32, _u32, _u32, _u32, _vp]),
    "mircuda_b200_moe_collect_rows_bf16": (_i, [_vpp, _u32, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _u32, _vp]),
    "mircuda_marlin_nvfp4_moe_execute": (_i, [_vp] * 11 + [_i, _b, _i, _i, _i, _i, _vp, _b]),
    "mircuda_marlin_mxfp4_moe_execute": (_i, [_vp] * 10 + [_i, _b, _i, _i, _i, _i, _vp, _b]),
    "mircuda_b200_mxfp8_bf16_gathered": (_i, [_vp] * 6 + [_u32] * 5 + [_vp]),
    "mircuda_b200_mxfp8_embedding_bf16": (_i, [_vp] * 4 + [_u32] * 4 + [_f, _vp]),
    "mircuda_fp8_vector_create": (_i, [_i, _i, _vp, _vpp]),
    "mircuda_fp8_vector_workspace_bytes": (_sz, [_vp]),
    "mircuda_fp8_vector_execute": (_i, [_vp] * 7),
    "mircuda_fp8_vector_destroy": (None, [_vp]),
    "mircuda_scaled_fp8_create": (_i, [_i] * 7 + [_vp, _vpp]),
    "mircuda_scaled_fp8_workspace_bytes": (_sz, [_vp]),
    "mircuda_scaled_fp8_execute": (_i, [_vp] * 8),
    "mircuda_scaled_fp8_destroy": (None, [_vp]),
    "mircuda_dense_create": (_i, [_i, _i, _i, _i, _i, _vp, _vpp]),
    "mircuda_dense_workspace_bytes": (_sz, [_vp]),
    "mircuda_dense_execute": (_i, [_vp, _vp, _vp, _vp, _vp, _f, _f]),
    "mircuda_dense_destroy": (None, [_vp]),
    "mircuda_b200_w4a16_create": (_i, [_i, _i, _i, _vp, _vpp]),
    "mircuda_b200_w4a16_workspace_bytes": (_sz, [_vp]),
    "mircuda_b200_w4a16_execute": (_i, [_vp] * 6),
    "mircuda_b200_w4a16_destroy": (None, [_vp]),
    "mircuda_b200_moe_scale_atoms": (_i, [_vp, _vp, _u32, _vp, _u32, _vp]),
    "mircuda_b200_moe_swiglu_nvfp4": (_i, [_vp, _vp, _vp, _vp, _u32, _vp, _u32, _vp]),
    "mircuda_variable_grouped_fp4_create": (_i, [_i, _i, _i, _i, _i, _vp, _vpp]),
    "mircuda_variable_grouped_fp4_execute": (_i, [_vp] * 12),
    "mircuda_b200_variable_grouped_fp4_execute_swiglu": (_i, [_vp] * 14),
    "mircuda_variable_grouped_fp4_destroy": (None, [_vp]),
    "mircuda_paired_variable_grouped_fp4_create": (_i, [_i, _i, _i, _i, _i, _vp, _vpp]),
    "mircuda_paired_variable_grouped_fp4_execute": (_i, [_vp] * 18),
    "mircuda_paired_variable_grouped_fp4_destroy": (None, [_vp]),
    "mircuda_grouped_fp4_create": (_i, [_i, _i, _i, _i, _i, _b, _vp, _vpp]),
    "mircuda_grouped_fp4_execute": (_i, [_vp] * 9),
    "mircuda_grouped_fp4_destroy": (None, [_vp]),
})

_handle = None


def load() -> ctypes.CDLL:
    global _handle
    if _handle is not None:
        return _handle
    if not LIBRARY.exists():
        raise ImportError(
            f"{LIBRARY} is missing. Build it with `python -m mircuda_b200.build` "
            "(needs nvcc; cross-compiles for sm_100a without a GPU). There is no CPU fallback."
        )
    handle = ctypes.CDLL(str(LIBRARY))
    for name, (restype, argtypes) in SIGNATURES.items():
        try:
            function = getattr(handle, name)
        except AttributeError as error:
            raise ImportError(f"{LIBRARY} does not export {name}; rebuild it") from error
        function.restype = restype
        function.argtypes = argtypes
    _handle = handle
    return handle
