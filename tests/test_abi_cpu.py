"""The C-ABI library without a GPU: it builds, loads, exports every declared symbol,
and rejects bad arguments before touching CUDA."""
import ctypes
import os
import re
from ctypes import byref, c_float, c_int, c_void_p

import numpy as np

from conftest import ROOT


def header_symbols():
    text = open(os.path.join(ROOT, "include", "fortai_cuda_backend_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fortai_cuda_\w+)\s*\(", text)))


def gguf_header_symbols():
    text = open(os.path.join(ROOT, "include", "fortai_gguf_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fortai_gguf_\w+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    from fortai_b200 import abi
    lib = abi.load()
    names = header_symbols()
    assert len(names) >= 35
    assert set(names) == set(abi.SIGNATURES)
    gguf_names = gguf_header_symbols()
    assert set(gguf_names) == set(abi.GGUF_SIGNATURES)
    for name in names + gguf_names:
        assert getattr(lib, name) is not None


def test_reference_symbol_set_is_complete():
    # the 35 functions of the reference header (backend/cuda/fortai_cuda_backend.h:22-156)
    from fortai_b200 import abi
    expected = {
        "fortai_cuda_q8_context_create", "fortai_cuda_q8_context_destroy",
        "fortai_cuda_q8_context_set_position", "fortai_cuda_q8_context_capture_begin",
        "fortai_cuda_q8_context_capture_end", "fortai_cuda_q8_context_graph_launch",
        "fortai_cuda_q8_weights_upload", "fortai_cuda_q8_weights_destroy",
        "fortai_cuda_q8_device_buffer_create", "fortai_cuda_q8_device_buffer_destroy",
        "fortai_cuda_q8_device_buffer_upload", "fortai_cuda_q8_device_buffer_upload_ptr",
        "fortai_cuda_q8_device_buffer_download", "fortai_cuda_q8_matvec_resident",
        "fortai_cuda_q8_matvec_device_f32", "fortai_cuda_qwen35_embedding_device",
        "fortai_cuda_qwen35_copy_device", "fortai_cuda_qwen35_add_device",
        "fortai_cuda_qwen35_rms_norm_device", "fortai_cuda_q8_matvec_host",
        "fortai_cuda_q8_matvec_host_pair", "fortai_cuda_q8_matvec_host_triplet",
        "fortai_cuda_q8_matvec_host_triplet_contiguous", "fortai_cuda_q8_ffn_host",
        "fortai_cuda_q8_ffn_device", "fortai_cuda_qwen35_recurrent_create",
        "fortai_cuda_qwen35_recurrent_destroy", "fortai_cuda_qwen35_recurrent_reset",
        "fortai_cuda_qwen35_recurrent_run", "fortai_cuda_qwen35_recurrent_run_device",
        "fortai_cuda_qwen35_attention_create", "fortai_cuda_qwen35_attention_destroy",
        "fortai_cuda_qwen35_attention_reset", "fortai_cuda_qwen35_attention_run_device",
        "fortai_cuda_q8_last_error",
    }
    assert set(abi.REFERENCE_SYMBOLS) == expected


def test_null_and_bad_arguments_are_invalid_before_any_cuda_call():
    from fortai_b200 import abi
    lib = abi.load()
    out = c_void_p()
    ms = c_float(0)
    buf = np.zeros(64, np.int8)
    p = buf.ctypes.data_as(c_void_p)
    assert lib.fortai_cuda_q8_context_create(-1, byref(out)) == abi.INVALID
    assert lib.fortai_cuda_q8_context_create(0, None) == abi.INVALID
    assert lib.fortai_cuda_q8_context_destroy(None) == abi.OK          # destroy(NULL) is OK
    assert lib.fortai_cuda_q8_weights_destroy(None) == abi.OK
    assert lib.fortai_cuda_q8_weights_upload(None, p, 64, 1, 32, byref(out)) == abi.INVALID
    assert lib.fortai_cuda_q8_context_set_position(None, 0) == abi.INVALID
    assert lib.fortai_cuda_q8_context_capture_begin(None) == abi.INVALID
    assert lib.fortai_cuda_q8_context_graph_launch(None) == abi.INVALID
    assert lib.fortai_cuda_q8_device_buffer_create(None, 16, byref(out)) == abi.INVALID
    assert lib.fortai_cuda_q8_matvec_resident(None, None, p, p, byref(ms)) == abi.INVALID
    assert lib.fortai_cuda_q8_matvec_device_f32(None, None, p, 32, p, 1) == abi.INVALID
    assert lib.fortai_cuda_q8_matvec_host(None, None, p, 34, p, 4, byref(ms)) == abi.INVALID
    assert lib.fortai_cuda_q8_matvec_host_pair(None, None, None, p, 34, p, 4, p, 4,
                                               byref(ms)) == abi.INVALID
    assert lib.fortai_cuda_q8_matvec_host_triplet_contiguous(None, None, None, None, p, 34, p, 12,
                                                             byref(ms)) == abi.INVALID
    assert lib.fortai_cuda_q8_ffn_host(None, None, None, None, p, 34, p, 4,
                                       byref(ms)) == abi.INVALID
    assert lib.fortai_cuda_q8_ffn_device(None, None, None, None, p, 32, p, 1) == abi.INVALID
    assert lib.fortai_cuda_q8_matmul_device_f32(None, None, p, 4, p, 4) == abi.INVALID
    assert lib.fortai_cuda_q8_quantize_device(None, p, 32, p, 34) == abi.INVALID
    assert lib.fortai_cuda_q8_context_set_option(None, b"gemv_variant", 1) == abi.INVALID
    assert lib.fortai_cuda_q8_last_error(None) == b"invalid CUDA Q8 context"


def test_wrapper_reports_invalid_like_the_fortran_module():
    # unassociated handles are caught in the wrapper (fortai_backend_cuda.f90:786-790)
    from fortai_b200 import backend_cuda as b
    ctx = b.cuda_q8_context_t()
    w = b.cuda_q8_weights_t()
    act = np.zeros(34, np.int8)
    out = np.zeros(1, np.float32)
    ms, stat = b.cuda_q8_matvec_host(ctx, w, act, 34, out, 4)
    assert not stat.is_ok() and stat.code == b.FORTAI_INVALID
    assert stat.message == "invalid CUDA Q8 host matvec" and ms == 0.0
    stat = w.upload(ctx, act, 34, 1, 32)
    assert stat.code == b.FORTAI_INVALID and stat.message == "invalid CUDA Q8 weight upload"
    stat = ctx.set_position(3)
    assert stat.code == b.FORTAI_INVALID and stat.message == "invalid CUDA device position"
    assert ctx.destroy().is_ok() and w.destroy().is_ok()
    stat = b.cuda_q8_ffn_device(ctx, w, w, w, 0, 32, 0, 1)
    assert stat.code == b.FORTAI_INVALID


def test_layout_helpers_match_the_documented_row_stride():
    # row-planar device rows: round_up(34 * blocks, 32) bytes
    for blocks, stride in ((32, 1088), (80, 2720), (68, 2336), (1, 64), (544, 18496)):
        assert (blocks * 34 + 31) // 32 * 32 == stride
