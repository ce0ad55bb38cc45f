"""ctypes declarations for every symbol in include/fortai_cuda_backend_b200.h.

The library is built in-tree on first use (nvcc, sm_100a).  If it cannot be
built or loaded this module raises: the package never computes on the CPU.
"""
from __future__ import annotations

import ctypes
from ctypes import (POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint64,
                    c_void_p)

from . import build as _build

OK = 0
INVALID = 1
RUNTIME_ERROR = 2

_P = c_void_p
_PP = POINTER(c_void_p)
_F = POINTER(c_float)

# name -> (restype, argtypes); the order follows the header
SIGNATURES = {
    # ---- reference interface
    "fortai_cuda_q8_context_create": (c_int, [c_int, _PP]),
    "fortai_cuda_q8_context_destroy": (c_int, [_P]),
    "fortai_cuda_q8_context_set_position": (c_int, [_P, c_int]),
    "fortai_cuda_q8_context_capture_begin": (c_int, [_P]),
    "fortai_cuda_q8_context_capture_end": (c_int, [_P]),
    "fortai_cuda_q8_context_graph_launch": (c_int, [_P]),
    "fortai_cuda_q8_weights_upload": (c_int, [_P, _P, c_size_t, c_int, c_int, _PP]),
    "fortai_cuda_q8_weights_destroy": (c_int, [_P]),
    "fortai_cuda_q8_device_buffer_create": (c_int, [_P, c_size_t, _PP]),
    "fortai_cuda_q8_device_buffer_destroy": (c_int, [_P, _P]),
    "fortai_cuda_q8_device_buffer_upload": (c_int, [_P, _P, _P, c_size_t]),
    "fortai_cuda_q8_device_buffer_upload_ptr": (c_int, [_P, _P, _P, c_size_t]),
    "fortai_cuda_q8_device_buffer_download": (c_int, [_P, _P, _P, c_size_t]),
    "fortai_cuda_q8_matvec_resident": (c_int, [_P, _P, _P, _P, _F]),
    "fortai_cuda_q8_matvec_device_f32": (c_int, [_P, _P, _P, c_size_t, _P, c_size_t]),
    "fortai_cuda_qwen35_embedding_device": (c_int, [_P, _P, c_int64, _P, c_size_t]),
    "fortai_cuda_qwen35_copy_device": (c_int, [_P, _P, _P, c_size_t]),
    "fortai_cuda_qwen35_add_device": (c_int, [_P, _P, _P, _P, c_size_t]),
    "fortai_cuda_qwen35_rms_norm_device": (c_int, [_P, _P, _P, _P, c_size_t, c_float]),
    "fortai_cuda_q8_matvec_host": (c_int, [_P, _P, _P, c_size_t, _P, c_size_t, _F]),
    "fortai_cuda_q8_matvec_host_pair": (c_int, [_P, _P, _P, _P, c_size_t, _P, c_size_t, _P,
                                                c_size_t, _F]),
    "fortai_cuda_q8_matvec_host_triplet": (c_int, [_P, _P, _P, _P, _P, c_size_t, _P, c_size_t, _P,
                                                   c_size_t, _P, c_size_t, _F]),
    "fortai_cuda_q8_matvec_host_triplet_contiguous": (c_int, [_P, _P, _P, _P, _P, c_size_t, _P,
                                                              c_size_t, _F]),
    "fortai_cuda_q8_ffn_host": (c_int, [_P, _P, _P, _P, _P, c_size_t, _P, c_size_t, _F]),
    "fortai_cuda_q8_ffn_device": (c_int, [_P, _P, _P, _P, _P, c_size_t, _P, c_size_t]),
    "fortai_cuda_qwen35_recurrent_create": (c_int, [_P, _P, _P, _P, _P, _P, _P, c_size_t, c_int,
                                                    c_int, _P, c_size_t, _P, c_size_t, _P,
                                                    c_size_t, c_int, c_int, c_int, c_int, c_int,
                                                    c_float, _PP]),
    "fortai_cuda_qwen35_recurrent_destroy": (c_int, [_P]),
    "fortai_cuda_qwen35_recurrent_reset": (c_int, [_P]),
    "fortai_cuda_qwen35_recurrent_run": (c_int, [_P, _P, c_size_t, _P, c_size_t, _F]),
    "fortai_cuda_qwen35_recurrent_run_device": (c_int, [_P, _P, c_size_t, _P, c_size_t]),
    "fortai_cuda_qwen35_attention_create": (c_int, [_P, _P, _P, _P, _P, _P, c_size_t, _P,
                                                    c_size_t, c_int, c_int, c_int, c_int, c_int,
                                                    c_int, c_float, c_float, _PP]),
    "fortai_cuda_qwen35_attention_destroy": (c_int, [_P]),
    "fortai_cuda_qwen35_attention_reset": (c_int, [_P]),
    "fortai_cuda_qwen35_attention_run_device": (c_int, [_P, _P, c_size_t, c_int, _P, c_size_t]),
    "fortai_cuda_q8_last_error": (c_char_p, [_P]),
    # ---- extensions
    "fortai_cuda_q8_context_create_on_stream": (c_int, [c_int, _P, _PP]),
    "fortai_cuda_q8_context_stream": (c_void_p, [_P]),
    "fortai_cuda_q8_context_launch_count": (c_uint64, [_P]),
    "fortai_cuda_q8_context_synchronize": (c_int, [_P]),
    "fortai_cuda_q8_context_set_option": (c_int, [_P, c_char_p, c_int]),
    "fortai_cuda_q8_weights_shape": (c_int, [_P, POINTER(c_int), POINTER(c_int)]),
    "fortai_cuda_q8_weights_upload_columns": (c_int, [_P, _P, c_size_t, c_int, c_int, c_int,
                                                      c_int, _PP]),
    "fortai_cuda_q8_quantize_device": (c_int, [_P, _P, c_size_t, _P, c_size_t]),
    "fortai_cuda_q8_block_dots_device": (c_int, [_P, _P, _P, _P, c_size_t]),
    "fortai_cuda_q8_matvec_host_f32": (c_int, [_P, _P, _P, c_size_t, _P, c_size_t, _F]),
    "fortai_cuda_q8_matmul_device_f32": (c_int, [_P, _P, _P, c_int, _P, c_size_t]),
    "fortai_cuda_q8_matmul_resident": (c_int, [_P, _P, _P, c_int, _P, _F]),
    "fortai_cuda_q8_matmul_host_f32": (c_int, [_P, _P, _P, c_int, _P, c_size_t, _F]),
    "fortai_cuda_q8_matmul_block_dots_device": (c_int, [_P, _P, _P, c_int, _P, c_size_t]),
    "fortai_cuda_q8_matvec_device_f32_peers": (c_int, [_P, _P, _P, c_size_t, _PP, c_int,
                                                       c_size_t, c_size_t]),
    "fortai_cuda_q8_matvec_device_f32_allgather": (c_int, [_P, _P, _P, c_size_t, _PP, _PP, c_int,
                                                           c_int, c_size_t, c_size_t]),
    "fortai_cuda_q8_matvec_device_f32_allgather_ll": (c_int, [_P, _P, _P, c_size_t, _PP, c_int, c_int,
                                                              c_size_t, _P, c_size_t]),
    "fortai_cuda_q8_ffn_device_allreduce": (c_int, [_P, _P, _P, _P, _P, c_size_t, _PP, c_int,
                                                    c_int, _P, c_size_t]),
    "fortai_cuda_q8_ffn_device_noalloc": (c_int, [_P, _P, _P, _P, _P, c_size_t, _P, c_size_t]),
    "fortai_cuda_q8_ffn_batch_device": (c_int, [_P, _P, _P, _P, _P, c_int, _P, c_size_t]),
    "fortai_cuda_tensor_peak": (c_int, [_P, c_int, c_int, _F, _F]),
    "fortai_cuda_q8_matvec_device_q8": (c_int, [_P, _P, _P, _P, c_size_t]),
    "fortai_cuda_q8_group_create": (c_int, [POINTER(c_int), c_int, _PP]),
    "fortai_cuda_q8_group_destroy": (c_int, [_P]),
    "fortai_cuda_q8_group_device_count": (c_int, [_P]),
    "fortai_cuda_q8_group_last_error": (c_char_p, [_P]),
    "fortai_cuda_q8_group_weights_upload": (c_int, [_P, _P, c_size_t, c_int, c_int, c_int, _PP]),
    "fortai_cuda_q8_group_weights_destroy": (c_int, [_P]),
    "fortai_cuda_q8_group_matvec_f32": (c_int, [_P, _P, _P, c_size_t, _P, c_size_t, _F]),
    "fortai_cuda_q8_group_ffn_f32": (c_int, [_P, _P, _P, _P, _P, c_size_t, _P, c_size_t, _F]),
    "fortai_cuda_qwen35_recurrent_step_device": (c_int, [_P, _P, c_size_t, _P, c_float]),
    "fortai_cuda_qwen35_attention_step_device": (c_int, [_P, _P, c_size_t, c_int, _P, c_float]),
    "fortai_cuda_q8_ffn_step_device": (c_int, [_P, _P, _P, _P, _P, c_size_t, _P, c_float]),
    "fortai_cuda_q8_matvec_norm_device_f32": (c_int, [_P, _P, _P, c_size_t, _P, c_float, _P,
                                                      c_size_t]),
}

REFERENCE_SYMBOLS = [name for name in SIGNATURES][:35]

# include/fortai_gguf_b200.h
_I64P = POINTER(c_int64)
GGUF_SIGNATURES = {
    "fortai_gguf_open": (c_int, [c_char_p, _PP, c_char_p, c_size_t]),
    "fortai_gguf_close": (None, [_P]),
    "fortai_gguf_version": (c_int32, [_P]),
    "fortai_gguf_tensor_count": (c_int64, [_P]),
    "fortai_gguf_metadata_count": (c_int64, [_P]),
    "fortai_gguf_alignment": (c_int64, [_P]),
    "fortai_gguf_data_start": (c_int64, [_P]),
    "fortai_gguf_find_meta": (c_int64, [_P, c_char_p]),
    "fortai_gguf_find_tensor": (c_int64, [_P, c_char_p]),
    "fortai_gguf_meta_key": (c_char_p, [_P, c_int64]),
    "fortai_gguf_meta_type": (c_int32, [_P, c_int64]),
    "fortai_gguf_meta_int": (c_int64, [_P, c_char_p, c_int64]),
    "fortai_gguf_meta_real": (c_float, [_P, c_char_p, c_float]),
    "fortai_gguf_meta_string": (c_void_p, [_P, c_char_p, _I64P]),
    "fortai_gguf_meta_bool": (c_int, [_P, c_char_p, c_int]),
    "fortai_gguf_meta_int_array": (c_int64, [_P, c_char_p, _I64P, c_int64]),
    "fortai_gguf_tensor_info": (c_int, [_P, c_int64, POINTER(c_char_p), POINTER(c_int32),
                                        POINTER(c_int32), _I64P, _I64P, _I64P]),
    "fortai_gguf_tensor_data": (c_void_p, [_P, c_int64]),
    "fortai_gguf_tensor_value": (c_float, [_P, c_int64, c_int64]),
    "fortai_gguf_tensor_get_row": (c_int, [_P, c_int64, c_int64, _F, c_int64]),
    "fortai_gguf_upload_q8": (c_int, [_P, c_int64, _P, c_int64, c_int64, _PP]),
}

_LIB = None


def library_path() -> str:
    return _build.LIB_PATH


def load() -> ctypes.CDLL:
    """Build if needed, load, and type every symbol.  Raises on any failure."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = _build.build()
    lib = ctypes.CDLL(path)
    for name, (restype, argtypes) in {**SIGNATURES, **GGUF_SIGNATURES}.items():
        fn = getattr(lib, name)      # AttributeError if the symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    _LIB = lib
    return lib
