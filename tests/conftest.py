import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def golden(name):
    path = os.path.join(GOLDEN, name)
    return np.load(path, allow_pickle=False)


@pytest.fixture(scope="session")
def oracle():
    from oracle import q8_oracle
    q8_oracle.lib()
    return q8_oracle


@pytest.fixture(scope="session")
def reference(oracle):
    """The reference's own compiled arithmetic, when oracle/_ref has been built."""
    if not oracle.Reference.available():
        pytest.skip("oracle/_ref not built (needs the reference checkout)")
    return oracle.Reference()


@pytest.fixture(scope="session")
def backend():
    from fortai_b200 import backend_cuda
    return backend_cuda


@pytest.fixture()
def context(backend):
    """A fresh context on cuda:0 (GPU tests only)."""
    ctx = backend.cuda_q8_context_t()
    stat = ctx.create(0)
    assert stat.is_ok(), stat
    yield ctx
    ctx.destroy()


class DeviceHelper:
    """Small conveniences for GPU tests, all through the C ABI."""

    def __init__(self, backend, context):
        self.b = backend
        self.c = context
        self._buffers = []
        self._weights = []

    def weights(self, host_bytes, rows, width):
        w = self.b.cuda_q8_weights_t()
        stat = w.upload(self.c, host_bytes, host_bytes.size, rows, width)
        assert stat.is_ok(), stat
        self._weights.append(w)
        return w

    def buffer(self, nbytes):
        ptr, stat = self.c.allocate_buffer(nbytes)
        assert stat.is_ok(), stat
        self._buffers.append(ptr)
        return ptr

    def to_device(self, array):
        a = np.ascontiguousarray(array)
        ptr = self.buffer(max(a.nbytes, 4))
        assert self.c.upload(ptr, a).is_ok()
        return ptr

    def floats(self, ptr, n):
        out, stat = self.c.download_real(ptr, n)
        assert stat.is_ok(), stat
        return out.copy()

    def int32s(self, ptr, n):
        out, stat = self.c.download(ptr, 4 * n)
        assert stat.is_ok(), stat
        return out.view(np.int32).copy()

    def bytes(self, ptr, n):
        out, stat = self.c.download(ptr, n)
        assert stat.is_ok(), stat
        return out.copy()

    def close(self):
        for w in self._weights:
            w.destroy()
        for p in self._buffers:
            self.c.free_buffer(p)


@pytest.fixture()
def dev(backend, context):
    helper = DeviceHelper(backend, context)
    yield helper
    helper.close()


def l2_tolerance(expected, factor=1e-5):
    """The fp32 bound of the task statement: max |gpu - cpu| <= 1e-5 * ||cpu||_2."""
    return factor * float(np.linalg.norm(expected.astype(np.float64)))


def reference_gate(actual, expected):
    """The reference's own per-element gate (tools/cuda_backend_smoke.cu:102-104):
    abs <= 2e-3 and abs / max(1, |expected|) <= 1e-4."""
    err = np.abs(actual.astype(np.float64) - expected.astype(np.float64))
    rel = err / np.maximum(1.0, np.abs(expected.astype(np.float64)))
    return float(err.max()) <= 2e-3 and float(rel.max()) <= 1e-4


def ffn_error_beyond_quant_flips(actual, expected, oracle, gate, up, down, inner, hidden, x):
    """Compare an FFN output with the oracle's, allowing for flipped quants of the hidden vector.

    The FFN re-quantizes h = silu(gate.x) * (up.x) to Q8_0 between its halves.  A last-bit
    difference in h (another summation order, the IEEE exponential instead of the reference's
    polynomial) now and then moves one element across a rounding boundary of the quantizer.
    One flipped quant i changes the output by exactly d_h[block(i)] * W_down[:, i], which is
    far above the fp32 bound for small layers.  This helper finds the flips that explain the
    difference (projection of the error on every such column), and returns
    (number of flips, largest |flip|, max |error| left after removing them).
    """
    g, u = oracle.matvec_pair(gate, up, inner, hidden, x)[:2]
    h = oracle.silu_product(g, u)
    scales = oracle.quantize(h)[1]
    rows = expected.size
    raw = np.ascontiguousarray(down).view(np.uint8).reshape(rows, inner // 32, 34)
    d = raw[:, :, :2].copy().view(np.float16).astype(np.float64).reshape(rows, inner // 32)
    q = raw[:, :, 2:].view(np.int8).astype(np.float64)
    columns = (q * d[:, :, None]).reshape(rows, inner) * np.repeat(scales.astype(np.float64), 32)
    error = actual.astype(np.float64) - expected.astype(np.float64)
    norms = (columns * columns).sum(axis=0)
    projection = np.where(norms > 0, (columns.T @ error) / np.maximum(norms, 1e-300), 0.0)
    flips = np.where(np.abs(projection) > 0.5, np.rint(projection), 0.0)
    left = error - columns @ flips
    return int(np.count_nonzero(flips)), float(np.abs(flips).max()), float(np.abs(left).max())
