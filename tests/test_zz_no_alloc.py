"""The allocation-free FFN entry point against the ordinary one (GPU required).

`fortai_cuda_q8_ffn_device_noalloc` exists for hosts that cannot let the library
call cudaMalloc/cudaFree while they run (their pools own all free HBM, or a
device-wide stall in the middle of a decode step is not acceptable).  It keeps its
two intermediates in a fixed array inside the library image instead of the
context's grow-on-demand scratch.  This file is collected last on purpose.
"""
from ctypes import byref, c_void_p

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _upload(lib, ctx, host, rows, width):
    out = c_void_p()
    assert lib.fortai_cuda_q8_weights_upload(ctx, host.ctypes.data_as(c_void_p), host.size, rows,
                                             width, byref(out)) == 0
    return out


def _buffer(lib, ctx, nbytes):
    out = c_void_p()
    assert lib.fortai_cuda_q8_device_buffer_create(ctx, nbytes, byref(out)) == 0
    return out


def test_noalloc_ffn_matches_the_allocating_entry_point_twice_in_a_row(oracle):
    from fortai_b200 import abi
    lib = abi.load()
    ctx = c_void_p()
    assert lib.fortai_cuda_q8_context_create(0, byref(ctx)) == 0
    hidden, inner = 2560, 9728
    gate = _upload(lib, ctx, oracle.make_weights(inner, hidden, seed=11), inner, hidden)
    up = _upload(lib, ctx, oracle.make_weights(inner, hidden, seed=12), inner, hidden)
    down = _upload(lib, ctx, oracle.make_weights(hidden, inner, seed=13), hidden, inner)
    d_in = _buffer(lib, ctx, 4 * hidden)
    d_ref = _buffer(lib, ctx, 4 * hidden)
    d_new = _buffer(lib, ctx, 4 * hidden)
    ref = np.zeros(hidden, np.float32)
    new = np.zeros(hidden, np.float32)
    # The point of the entry point: it must not allocate.  The inner size (9728) is one for
    # which the ordinary FFN would grow its prepared-activation buffer.  A throw-away context
    # runs the call once first, so that the driver has loaded the kernels' code (lazy module
    # loading takes device memory at a kernel's first launch in the process); then free device
    # memory is compared around the first call on a context that has not grown any scratch.
    import torch
    x0 = oracle.normal(hidden, seed=19)
    warm = c_void_p()
    assert lib.fortai_cuda_q8_context_create(0, byref(warm)) == 0
    warm_w = [_upload(lib, warm, oracle.make_weights(r, k, seed=1), r, k)
              for r, k in ((inner, hidden), (inner, hidden), (hidden, inner))]
    warm_in, warm_out = _buffer(lib, warm, 4 * hidden), _buffer(lib, warm, 4 * hidden)
    assert lib.fortai_cuda_q8_device_buffer_upload(warm, warm_in, x0.ctypes.data_as(c_void_p),
                                                   x0.nbytes) == 0
    assert lib.fortai_cuda_q8_ffn_device_noalloc(warm, warm_w[0], warm_w[1], warm_w[2], warm_in,
                                                 hidden, warm_out, hidden) == 0
    assert lib.fortai_cuda_q8_context_synchronize(warm) == 0
    for w in warm_w:
        lib.fortai_cuda_q8_weights_destroy(w)
    for b in (warm_in, warm_out):
        lib.fortai_cuda_q8_device_buffer_destroy(warm, b)
    lib.fortai_cuda_q8_context_destroy(warm)

    assert lib.fortai_cuda_q8_device_buffer_upload(ctx, d_in, x0.ctypes.data_as(c_void_p),
                                                   x0.nbytes) == 0
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info(0)[0]
    code = lib.fortai_cuda_q8_ffn_device_noalloc(ctx, gate, up, down, d_in, hidden, d_new, hidden)
    assert code == 0, lib.fortai_cuda_q8_last_error(ctx)
    assert lib.fortai_cuda_q8_context_synchronize(ctx) == 0
    assert torch.cuda.mem_get_info(0)[0] == free_before
    for call in range(2):          # the second call reuses whatever the first one left behind
        x = oracle.normal(hidden, seed=20 + call)
        assert lib.fortai_cuda_q8_device_buffer_upload(ctx, d_in, x.ctypes.data_as(c_void_p),
                                                       x.nbytes) == 0
        assert lib.fortai_cuda_q8_ffn_device(ctx, gate, up, down, d_in, hidden, d_ref, hidden) == 0
        code = lib.fortai_cuda_q8_ffn_device_noalloc(ctx, gate, up, down, d_in, hidden, d_new,
                                                     hidden)
        assert code == 0, lib.fortai_cuda_q8_last_error(ctx)
        assert lib.fortai_cuda_q8_device_buffer_download(ctx, ref.ctypes.data_as(c_void_p), d_ref,
                                                         ref.nbytes) == 0
        assert lib.fortai_cuda_q8_device_buffer_download(ctx, new.ctypes.data_as(c_void_p), d_new,
                                                         new.nbytes) == 0
        tolerance = 1e-5 * float(np.linalg.norm(ref.astype(np.float64)))
        assert float(np.abs(new - ref).max()) <= tolerance
        expected = oracle.ffn(oracle.make_weights(inner, hidden, seed=11),
                              oracle.make_weights(inner, hidden, seed=12),
                              oracle.make_weights(hidden, inner, seed=13), inner, hidden, hidden, x)
        assert float(np.abs(new - expected).max()) <= 2e-5 * float(np.linalg.norm(expected))
    # sizes beyond the fixed array are refused with a message, nothing is enqueued
    big_inner = 32768 + 32
    big_gate = _upload(lib, ctx, np.zeros(big_inner * 34, np.int8), big_inner, 32)
    big_down = _upload(lib, ctx, np.zeros((big_inner // 32) * 34, np.int8), 1, big_inner)
    code = lib.fortai_cuda_q8_ffn_device_noalloc(ctx, big_gate, big_gate, big_down, d_in, 32,
                                                 d_new, 1)
    assert code == abi.INVALID
    assert b"at most 32768" in lib.fortai_cuda_q8_last_error(ctx)
    for w in (gate, up, down, big_gate, big_down):
        lib.fortai_cuda_q8_weights_destroy(w)
    for b in (d_in, d_ref, d_new):
        lib.fortai_cuda_q8_device_buffer_destroy(ctx, b)
    lib.fortai_cuda_q8_context_destroy(ctx)
