"""ctypes binding of libishizuki_cuda.so: one Python signature per declaration in
include/ishizuki_cuda.h. Loading fails loudly when the library is missing; there is no other
implementation behind these names."""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_void_p

from . import build as _build

OK, E_INVALID, E_SHAPE, E_UNSUPPORTED, E_CUDA, E_TIMEOUT, E_NOMEM, E_TOO_LARGE, E_NCCL = range(9)
GROUP_ID_BYTES = 128
GGML_Q4_K, GGML_Q6_K, GGML_IQ2_XS = 12, 14, 17
GGML_TYPE_SIZE = {10: 84, 12: 144, 14: 210, 16: 66, 17: 74, 18: 98, 19: 50, 21: 110, 22: 82, 23: 136, 29: 56}
KIND_AFFINE, KIND_GGML = 0, 1
DT_F16, DT_BF16, DT_F32 = 0, 1, 2
ROUTE_AUTO, ROUTE_GEMV, ROUTE_MMA = 0, 1, 2
EXL3_3INST, EXL3_MCG, EXL3_MUL1 = 0, 1, 2
OUT_TRANSPOSED = 1
EXCHANGE_HANDLE_BYTES = 128


class GGUFTensorInfo(ctypes.Structure):
    _fields_ = [("name", c_char_p), ("rank", c_int32), ("shape", c_int64 * 4), ("ggml_type", c_int32),
                ("offset", c_int64), ("byte_count", c_int64)]


class WeightDesc(ctypes.Structure):
    _fields_ = [
        ("kind", c_int32), ("ggml_type", c_int32), ("bits", c_int32), ("group_size", c_int32),
        ("scale_dtype", c_int32), ("hadamard_block", c_int32),
        ("n", c_int64), ("k", c_int64),
        ("weight_dev", c_void_p), ("weight_bytes", c_int64),
        ("scales_dev", c_void_p), ("biases_dev", c_void_p), ("signs_dev", c_void_p),
    ]


class EXL3Desc(ctypes.Structure):
    _fields_ = [
        ("trellis_dev", c_void_p), ("k", c_int64), ("n", c_int64),
        ("words_per_tile", c_int32), ("codebook", c_int32),
        ("input_scales_dev", c_void_p), ("output_scales_dev", c_void_p),
    ]


# name -> (restype, argtypes); every symbol the header declares
SIGNATURES = {
    "ishi_ctx_create": (c_int, [c_int, POINTER(c_void_p)]),
    "ishi_ctx_destroy": (None, [c_void_p]),
    "ishi_status_string": (c_char_p, [c_int]),
    "ishi_last_error": (c_char_p, [c_void_p]),
    "ishi_ctx_poll": (c_int, [c_void_p]),
    "ishi_ctx_set_route": (c_int, [c_void_p, c_int, c_int]),
    "ishi_projection_create": (c_int, [c_void_p, POINTER(WeightDesc), POINTER(c_void_p)]),
    "ishi_projection_create_fused": (c_int, [c_void_p, POINTER(WeightDesc), c_int, POINTER(c_void_p)]),
    "ishi_projection_create_gated": (c_int, [c_void_p, POINTER(WeightDesc), POINTER(WeightDesc), POINTER(c_void_p)]),
    "ishi_rms_norm": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int64, c_void_p, c_int, ctypes.c_float, c_void_p, c_void_p]),
    "ishi_exl3_dequantize": (c_int, [c_void_p, POINTER(EXL3Desc), c_int, c_void_p, c_void_p]),
    "ishi_exl3_rotate": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_int64, c_void_p, c_int, c_void_p, c_int, c_void_p]),
    "ishi_exl3_matvec": (c_int, [c_void_p, POINTER(EXL3Desc), c_void_p, c_int, c_void_p, c_void_p]),
    "ishi_exl3_apply": (c_int, [c_void_p, POINTER(EXL3Desc), c_void_p, c_int, c_void_p, c_void_p]),
    "ishi_projection_destroy": (None, [c_void_p]),
    "ishi_projection_input_dim": (c_int64, [c_void_p]),
    "ishi_projection_output_dim": (c_int64, [c_void_p]),
    "ishi_projection_weight_bytes": (c_int64, [c_void_p]),
    "ishi_projection_crossover_rows": (c_int, [c_void_p]),
    "ishi_projection_plan": (c_int, [c_void_p, ctypes.POINTER(c_int)]),
    "ishi_projection_set_plan": (c_int, [c_void_p, ctypes.POINTER(c_int)]),
    "ishi_projection_apply": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int, c_void_p]),
    "ishi_projection_apply_argmax": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "ishi_projection_rotate": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "ishi_projection_apply_rotated": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int, c_void_p]),
    "ishi_projection_apply_host": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "ishi_projection_apply_host_async": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "ishi_projection_apply_host_batch": (c_int, [POINTER(c_void_p), POINTER(c_void_p), c_int, POINTER(c_void_p), c_int, c_void_p]),
    "ishi_ggml_matvec": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int, c_int64, c_int64, c_void_p, c_void_p]),
    "ishi_ggml_matmul_few": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int, c_int64, c_int64, c_void_p, c_void_p]),
    "ishi_ggml_dequantize": (c_int, [c_void_p, c_int, c_void_p, c_int64, c_void_p, c_int, c_void_p]),
    "ishi_ggml_gather": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int64, c_int64, c_void_p, c_int, c_void_p]),
    "ishi_verify_matmul": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "ishi_affine_dequantize": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_int64, c_void_p, c_void_p]),
    "ishi_hadamard_rotate": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p]),
    "ishi_reference_minimum_rows": (c_int, [c_int64]),
    "ishi_ggml_block_size": (c_int, [c_int]),
    "ishi_ggml_type_size": (c_int, [c_int]),
    "ishi_q4k_matmul_few_static": (c_int, [c_void_p, c_int, c_void_p, c_int64, c_int64, c_int64, c_void_p, c_void_p]),
    "ishi_gguf_open": (c_int, [c_char_p, POINTER(c_void_p), c_char_p, ctypes.c_size_t]),
    "ishi_gguf_close": (None, [c_void_p]),
    "ishi_gguf_last_error": (c_char_p, [c_void_p]),
    "ishi_gguf_version": (ctypes.c_uint32, [c_void_p]),
    "ishi_gguf_data_offset": (c_int64, [c_void_p]),
    "ishi_gguf_alignment": (c_int64, [c_void_p]),
    "ishi_gguf_tensor_count": (c_int64, [c_void_p]),
    "ishi_gguf_find_tensor": (c_int64, [c_void_p, c_char_p]),
    "ishi_gguf_tensor": (c_int, [c_void_p, c_int64, POINTER(GGUFTensorInfo)]),
    "ishi_gguf_type_block_size": (c_int, [c_int]),
    "ishi_gguf_type_size": (c_int, [c_int]),
    "ishi_gguf_type_name": (c_char_p, [c_int]),
    "ishi_gguf_metadata_count": (c_int64, [c_void_p]),
    "ishi_gguf_metadata_key": (c_char_p, [c_void_p, c_int64]),
    "ishi_gguf_metadata_kind": (c_int, [c_void_p, c_char_p]),
    "ishi_gguf_metadata_int": (c_int, [c_void_p, c_char_p, POINTER(c_int64)]),
    "ishi_gguf_metadata_float": (c_int, [c_void_p, c_char_p, POINTER(ctypes.c_double)]),
    "ishi_gguf_metadata_string": (c_char_p, [c_void_p, c_char_p]),
    "ishi_gguf_metadata_array_length": (c_int64, [c_void_p, c_char_p]),
    "ishi_gguf_metadata_array_int": (c_int, [c_void_p, c_char_p, c_int64, POINTER(c_int64)]),
    "ishi_gguf_metadata_array_string": (c_char_p, [c_void_p, c_char_p, c_int64]),
    "ishi_gguf_read_tensor": (c_int, [c_void_p, c_int64, c_void_p, c_int64]),
    "ishi_gguf_upload_tensor": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_void_p]),
    "ishi_group_unique_id": (c_int, [c_void_p]),
    "ishi_group_create": (c_int, [c_void_p, c_int, c_int, c_int, POINTER(c_void_p)]),
    "ishi_group_last_error": (c_char_p, [c_void_p]),
    "ishi_projection_apply_sharded": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "ishi_group_destroy": (None, [c_void_p]),
    "ishi_group_debug_set_api": (c_int, [c_void_p]),
    "ishi_exchange_create": (c_int, [c_void_p, c_int, c_int, c_int64, POINTER(c_void_p)]),
    "ishi_exchange_export": (c_int, [c_void_p, c_void_p]),
    "ishi_exchange_connect": (c_int, [c_void_p, c_void_p]),
    "ishi_exchange_buffer": (c_void_p, [c_void_p]),
    "ishi_exchange_apply": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int, c_void_p]),
    "ishi_exchange_wait": (c_int, [c_void_p, c_void_p]),
    "ishi_exchange_debug_expect": (c_int, [c_void_p, ctypes.c_uint]),
    "ishi_exchange_disconnect": (c_int, [c_void_p]),
    "ishi_exchange_destroy": (None, [c_void_p]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Loads (building first if the sources are newer) and types the C-ABI library."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB
    if _build.stale():
        try:
            path = _build.build()
        except RuntimeError:
            if not path.exists():
                raise
    lib = ctypes.CDLL(str(path))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means header and library disagree
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
