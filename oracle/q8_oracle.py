"""ctypes/numpy front end of the CPU checker.  TEST INFRASTRUCTURE ONLY.

Loads ``oracle/libq8oracle.so`` (the scalar-C restatement in ``q8_oracle.c``)
and, when present, ``oracle/_ref/libfortai_ref_q8.so`` (the reference's own C
arithmetic, compiled from its checkout by ``oracle/Makefile``).  Nothing in the
shipped package imports this module: it is used by the test-suite, by the smoke
check, and by the CPU-baseline leg of the benchmark.

Every helper names the reference code it stands for; see ``q8_oracle.c`` for the
line-by-line citations.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import POINTER, c_double, c_float, c_int, c_int8, c_int32, c_int64, c_uint8, c_uint16, c_uint32, c_uint64, c_void_p

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
BLOCK_ELEMS = 32
BLOCK_BYTES = 34


def reference_checkout() -> str:
    """Where the reference's sources lie: FORTAI_REFERENCE, else a checkout named
    `reference` beside this repository; empty when there is neither."""
    given = os.environ.get("FORTAI_REFERENCE", "")
    if given:
        return given
    sibling = os.path.normpath(os.path.join(HERE, "..", "..", "reference"))
    return sibling if os.path.isdir(sibling) else ""


def build(force: bool = False) -> None:
    """Compile the restatement and (if the reference checkout is here) oracle/_ref."""
    target = os.path.join(HERE, "libq8oracle.so")
    if force or not os.path.exists(target) or (
            os.path.getmtime(target) < os.path.getmtime(os.path.join(HERE, "q8_oracle.c"))):
        subprocess.run(["make", "-C", HERE, "all", f"REFERENCE={reference_checkout()}"],
                       check=True, capture_output=True)
    elif os.path.isdir(reference_checkout()) and not os.path.exists(
            os.path.join(HERE, "_ref", "libfortai_ref_q8.so")):
        subprocess.run(["make", "-C", HERE, "ref", f"REFERENCE={reference_checkout()}"],
                       check=True, capture_output=True)


def _ptr(array: np.ndarray):
    return array.ctypes.data_as(c_void_p)


class _Lib:
    def __init__(self):
        build()
        self.lib = ctypes.CDLL(os.path.join(HERE, "libq8oracle.so"))
        L = self.lib
        L.oracle_float_to_half.restype = c_uint16
        L.oracle_float_to_half.argtypes = [c_float]
        L.oracle_half_to_float.restype = c_float
        L.oracle_half_to_float.argtypes = [c_uint16]
        L.oracle_q8_quantize.argtypes = [c_void_p, c_void_p, c_void_p, c_int64]
        L.oracle_q8_quantize_ties_away.argtypes = [c_void_p, c_void_p, c_void_p, c_int64]
        L.oracle_q8_dot.restype = c_float
        L.oracle_q8_dot.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64]
        L.oracle_q8_dot_blockwise.restype = c_float
        L.oracle_q8_dot_blockwise.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64]
        L.oracle_q8_block_dots.argtypes = [c_void_p, c_void_p, c_int64, c_int64, c_void_p]
        L.oracle_q8_dequantize_row.argtypes = [c_void_p, c_void_p, c_int64]
        L.oracle_matvec_q8.restype = c_int
        L.oracle_matvec_q8.argtypes = [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_void_p,
                                       c_int64, c_void_p, c_int64, c_void_p, c_int64]
        L.oracle_matvec_pair_q8.restype = c_int
        L.oracle_matvec_pair_q8.argtypes = [c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
                                            c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                                            c_void_p, c_int64, c_void_p, c_int64]
        L.oracle_matvec_triplet_q8.restype = c_int
        L.oracle_matvec_triplet_q8.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                               c_int64, c_int64, c_int64, c_int64, c_void_p,
                                               c_int64, c_void_p, c_int64, c_void_p, c_int64,
                                               c_void_p, c_int64, c_void_p, c_int64, c_void_p,
                                               c_int64]
        L.oracle_matvec_q8_prequantized.restype = c_int
        L.oracle_matvec_q8_prequantized.argtypes = [c_void_p, c_int64, c_int64, c_void_p, c_void_p]
        L.oracle_matmul_q8.restype = c_int
        L.oracle_matmul_q8.argtypes = [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_void_p,
                                       c_void_p, c_void_p]
        L.oracle_silu_product.argtypes = [c_void_p, c_void_p, c_int64, c_int]
        L.oracle_ffn_q8.restype = c_int
        L.oracle_ffn_q8.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                    c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_int]
        L.oracle_fill_normal.argtypes = [c_void_p, c_int64, c_int64, c_uint64, c_float]
        L.oracle_make_weights.argtypes = [c_void_p, c_int64, c_int64, c_int64, c_uint64, c_float]
        L.oracle_fixture_fill_q8.argtypes = [c_void_p, c_int, c_int, c_uint32, c_int]
        L.oracle_fixture_matvec.argtypes = [c_void_p, c_void_p, c_int, c_int, c_void_p]
        L.oracle_thread_count.restype = c_int
        L.oracle_set_threads.argtypes = [c_int]


_LIB = None


def lib():
    global _LIB
    if _LIB is None:
        _LIB = _Lib().lib
    return _LIB


# --------------------------------------------------------------------------- conversions
def float_to_half(value: float) -> int:
    return int(lib().oracle_float_to_half(c_float(value)))


def half_to_float(bits: int) -> float:
    return float(lib().oracle_half_to_float(c_uint16(bits)))


# --------------------------------------------------------------------------- quantizer
def quantize(values: np.ndarray, ties_away: bool = False):
    """fortai_q8_quantize: returns (Q8_0 bytes as int8[K + K/16], scales float32[K/32])."""
    x = np.ascontiguousarray(values, dtype=np.float32).reshape(-1)
    count = x.size
    blocks = count // BLOCK_ELEMS
    out = np.zeros(blocks * BLOCK_BYTES, dtype=np.int8)
    scales = np.zeros(blocks, dtype=np.float32)
    fn = lib().oracle_q8_quantize_ties_away if ties_away else lib().oracle_q8_quantize
    fn(_ptr(x), _ptr(out), _ptr(scales), count)
    return out, scales


def activation_scales(q8: np.ndarray) -> np.ndarray:
    """Float value of each block's fp16 scale."""
    raw = np.ascontiguousarray(q8).view(np.uint8).reshape(-1, BLOCK_BYTES)
    return raw[:, :2].copy().view(np.float16).astype(np.float32).reshape(-1)


def quants(q8: np.ndarray) -> np.ndarray:
    raw = np.ascontiguousarray(q8).view(np.int8).reshape(-1, BLOCK_BYTES)
    return raw[:, 2:].copy()


# --------------------------------------------------------------------------- dots
def dot(weights: np.ndarray, quantized: np.ndarray, scales: np.ndarray, row: int,
        blocks: int, blockwise: bool = False) -> float:
    fn = lib().oracle_q8_dot_blockwise if blockwise else lib().oracle_q8_dot
    return float(fn(_ptr(weights), _ptr(quantized), _ptr(scales), row, blocks))


def block_dots(weights: np.ndarray, quantized: np.ndarray, rows: int, blocks: int) -> np.ndarray:
    out = np.zeros((rows, blocks), dtype=np.int32)
    lib().oracle_q8_block_dots(_ptr(weights), _ptr(quantized), rows, blocks, _ptr(out))
    return out


def dequantize_row(weights: np.ndarray, row: int, blocks: int) -> np.ndarray:
    raw = np.ascontiguousarray(weights).view(np.int8).reshape(-1)
    out = np.zeros(blocks * BLOCK_ELEMS, dtype=np.float32)
    lib().oracle_q8_dequantize_row(_ptr(raw[row * blocks * BLOCK_BYTES:]), _ptr(out), blocks)
    return out


# --------------------------------------------------------------------------- drivers
def matvec(weights: np.ndarray, rows: int, width: int, vector: np.ndarray):
    """gguf_tensor_matvec_q8: returns (values, quantized, scales)."""
    v = np.ascontiguousarray(vector, dtype=np.float32)
    values = np.zeros(rows, dtype=np.float32)
    quantized = np.zeros(width + width // 16, dtype=np.int8)
    scales = np.zeros(width // 32, dtype=np.float32)
    code = lib().oracle_matvec_q8(_ptr(weights), rows, width, _ptr(v), v.size, _ptr(values),
                                  values.size, _ptr(quantized), quantized.size, _ptr(scales),
                                  scales.size)
    if code != 0:
        raise ValueError("activation Q8 matvec dimensions do not agree")
    return values, quantized, scales


def matvec_pair(first, second, rows, width, vector, second_rows=None, second_width=None):
    v = np.ascontiguousarray(vector, dtype=np.float32)
    second_rows = rows if second_rows is None else second_rows
    second_width = width if second_width is None else second_width
    a = np.zeros(rows, dtype=np.float32)
    b = np.zeros(second_rows, dtype=np.float32)
    quantized = np.zeros(v.size + v.size // 16 + 2, dtype=np.int8)
    scales = np.zeros(v.size // 32 + 1, dtype=np.float32)
    code = lib().oracle_matvec_pair_q8(_ptr(first), _ptr(second), rows, width, second_rows,
                                       second_width, _ptr(v), v.size, _ptr(a), a.size, _ptr(b),
                                       b.size, _ptr(quantized), quantized.size, _ptr(scales),
                                       scales.size)
    if code != 0:
        raise ValueError("paired activation matvec dimensions do not agree")
    return a, b


def matvec_triplet(first, second, third, rows3, width, vector, widths=None):
    v = np.ascontiguousarray(vector, dtype=np.float32)
    widths = widths or (width, width, width)
    outs = [np.zeros(r, dtype=np.float32) for r in rows3]
    quantized = np.zeros(v.size + v.size // 16 + 2, dtype=np.int8)
    scales = np.zeros(v.size // 32 + 1, dtype=np.float32)
    code = lib().oracle_matvec_triplet_q8(_ptr(first), _ptr(second), _ptr(third), rows3[0],
                                          rows3[1], rows3[2], widths[0], widths[1], widths[2],
                                          _ptr(v), v.size, _ptr(outs[0]), outs[0].size,
                                          _ptr(outs[1]), outs[1].size, _ptr(outs[2]),
                                          outs[2].size, _ptr(quantized), quantized.size,
                                          _ptr(scales), scales.size)
    if code != 0:
        raise ValueError("triplet matvec dimensions do not agree")
    return outs


def matvec_prequantized(weights, rows, blocks, activation) -> np.ndarray:
    values = np.zeros(rows, dtype=np.float32)
    code = lib().oracle_matvec_q8_prequantized(_ptr(weights), rows, blocks, _ptr(activation),
                                               _ptr(values))
    if code != 0:
        raise ValueError("bad shape")
    return values


def matmul(weights, rows, width, matrix):
    """`tokens` independent matvecs: returns (values[tokens, rows], quantized, scales)."""
    m = np.ascontiguousarray(matrix, dtype=np.float32).reshape(-1, width)
    tokens = m.shape[0]
    blocks = width // 32
    values = np.zeros((tokens, rows), dtype=np.float32)
    quantized = np.zeros(tokens * blocks * BLOCK_BYTES, dtype=np.int8)
    scales = np.zeros(tokens * blocks, dtype=np.float32)
    code = lib().oracle_matmul_q8(_ptr(weights), rows, width, _ptr(m), tokens, _ptr(values),
                                  _ptr(quantized), _ptr(scales))
    if code != 0:
        raise ValueError("bad shape")
    return values, quantized, scales


def silu_product(left, right, contract: bool = True) -> np.ndarray:
    out = np.ascontiguousarray(left, dtype=np.float32).copy()
    r = np.ascontiguousarray(right, dtype=np.float32)
    lib().oracle_silu_product(_ptr(out), _ptr(r), out.size, int(contract))
    return out


def ffn(gate, up, down, inner, hidden, hidden_out, vector, contract: bool = True) -> np.ndarray:
    v = np.ascontiguousarray(vector, dtype=np.float32)
    out = np.zeros(hidden_out, dtype=np.float32)
    wg = np.zeros(inner, dtype=np.float32)
    wu = np.zeros(inner, dtype=np.float32)
    qmax = max(inner, hidden)
    quantized = np.zeros(qmax + qmax // 16, dtype=np.int8)
    scales = np.zeros(qmax // 32, dtype=np.float32)
    code = lib().oracle_ffn_q8(_ptr(gate), _ptr(up), _ptr(down), inner, hidden, hidden_out,
                               _ptr(v), _ptr(out), _ptr(wg), _ptr(wu), _ptr(quantized),
                               _ptr(scales), int(contract))
    if code != 0:
        raise ValueError("bad shape")
    return out


# --------------------------------------------------------------------------- inputs
def normal(count: int, seed: int, sigma: float = 1.0, first: int = 0) -> np.ndarray:
    out = np.zeros(count, dtype=np.float32)
    lib().oracle_fill_normal(_ptr(out), first, count, seed, c_float(sigma))
    return out


def make_weights(rows: int, width: int, seed: int = 0, sigma: float = 0.02,
                 first_row: int = 0) -> np.ndarray:
    """rows x width ~N(0, sigma) quantized to Q8_0 (GGUF layout), as int8 bytes."""
    out = np.zeros(rows * (width // 32) * BLOCK_BYTES, dtype=np.int8)
    lib().oracle_make_weights(_ptr(out), first_row, rows, width, seed, c_float(sigma))
    return out


def fixture_fill_q8(rows: int, blocks: int, seed: int, per_row: bool) -> np.ndarray:
    data = np.zeros((rows if per_row else 1) * blocks * BLOCK_BYTES, dtype=np.uint8)
    lib().oracle_fixture_fill_q8(_ptr(data), rows, blocks, seed & 0xffffffff, int(per_row))
    return data


def fixture_matvec(weights, activation, rows, blocks) -> np.ndarray:
    out = np.zeros(rows, dtype=np.float32)
    lib().oracle_fixture_matvec(_ptr(weights), _ptr(activation), rows, blocks, _ptr(out))
    return out


def thread_count() -> int:
    return int(lib().oracle_thread_count())


def host_threads() -> int:
    """Cores this process may run on: the reference's own thread policy is all of them
    (tools/build_native.sh:7-9)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except (AttributeError, OSError):
        return max(1, os.cpu_count() or 1)


def set_threads(threads: int) -> None:
    lib().oracle_set_threads(int(threads))


# --------------------------------------------------------------------------- reference build
class Reference:
    """The reference's own C arithmetic (oracle/_ref).  `fast=True` loads the build
    with the reference's native-profile flags, used only for timing."""

    def __init__(self, fast: bool = False):
        name = "libfortai_ref_q8_fast.so" if fast else "libfortai_ref_q8.so"
        path = os.path.join(HERE, "_ref", name)
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        L = self.lib = ctypes.CDLL(path)
        L.fortai_q8_quantize.argtypes = [c_void_p, c_void_p, c_void_p, c_int64]
        L.fortai_q8_dot.restype = c_float
        L.fortai_q8_dot.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64]
        L.fortai_q8_dequantize_row.argtypes = [c_void_p, c_void_p, c_int64]
        L.fortai_float_to_half.restype = c_uint16
        L.fortai_float_to_half.argtypes = [c_float]
        L.fortai_silu_product.argtypes = [c_void_p, c_void_p, c_int64]
        L.ref_matvec_q8.argtypes = [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p,
                                    c_void_p]
        L.ref_rows_q8.argtypes = [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p]
        L.ref_matmul_q8.argtypes = [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_void_p,
                                    c_void_p, c_void_p]
        L.ref_matvec_q8_repeat.restype = c_double
        L.ref_matvec_q8_repeat.argtypes = [c_void_p, c_int64, c_int64, c_void_p, c_void_p,
                                           c_void_p, c_void_p, c_int]
        L.ref_thread_count.restype = c_int
        L.ref_set_threads.argtypes = [c_int]
        L.ref_uses_avx2.restype = c_int
        L.fortai_gdn_step.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_float,
                                      c_int64, c_float, c_void_p]
        L.fortai_silu.argtypes = [c_void_p, c_int64]

    @staticmethod
    def available(fast: bool = False) -> bool:
        name = "libfortai_ref_q8_fast.so" if fast else "libfortai_ref_q8.so"
        return os.path.exists(os.path.join(HERE, "_ref", name))

    def quantize(self, values):
        x = np.ascontiguousarray(values, dtype=np.float32).reshape(-1)
        blocks = x.size // BLOCK_ELEMS
        out = np.zeros(blocks * BLOCK_BYTES, dtype=np.int8)
        scales = np.zeros(blocks, dtype=np.float32)
        self.lib.fortai_q8_quantize(_ptr(x), _ptr(out), _ptr(scales), x.size)
        return out, scales

    def dot(self, weights, quantized, scales, row, blocks) -> float:
        return float(self.lib.fortai_q8_dot(_ptr(weights), _ptr(quantized), _ptr(scales), row,
                                            blocks))

    def matvec(self, weights, rows, width, vector):
        v = np.ascontiguousarray(vector, dtype=np.float32)
        values = np.zeros(rows, dtype=np.float32)
        quantized = np.zeros(width + width // 16, dtype=np.int8)
        scales = np.zeros(width // 32, dtype=np.float32)
        self.lib.ref_matvec_q8(_ptr(weights), rows, width, _ptr(v), _ptr(values), _ptr(quantized),
                               _ptr(scales))
        return values, quantized, scales

    def rows(self, weights, rows, blocks, quantized, scales):
        values = np.zeros(rows, dtype=np.float32)
        self.lib.ref_rows_q8(_ptr(weights), rows, blocks, _ptr(quantized), _ptr(scales),
                             _ptr(values))
        return values

    def matvec_repeat(self, weights, rows, width, vector, repeats):
        v = np.ascontiguousarray(vector, dtype=np.float32)
        values = np.zeros(rows, dtype=np.float32)
        quantized = np.zeros(width + width // 16, dtype=np.int8)
        scales = np.zeros(width // 32, dtype=np.float32)
        checksum = self.lib.ref_matvec_q8_repeat(_ptr(weights), rows, width, _ptr(v), _ptr(values),
                                                 _ptr(quantized), _ptr(scales), repeats)
        return float(checksum), values

    def silu_product(self, left, right):
        out = np.ascontiguousarray(left, dtype=np.float32).copy()
        r = np.ascontiguousarray(right, dtype=np.float32)
        self.lib.fortai_silu_product(_ptr(out), _ptr(r), out.size)
        return out

    def gdn_step(self, state, key, value, query, decay, beta, output_scale):
        """fortai_gdn_step: `state` (head_size x head_size, float32) is updated in place."""
        hs = key.size
        out = np.zeros(hs, dtype=np.float32)
        self.lib.fortai_gdn_step(_ptr(state), _ptr(np.ascontiguousarray(key, np.float32)),
                                 _ptr(np.ascontiguousarray(value, np.float32)),
                                 _ptr(np.ascontiguousarray(query, np.float32)), c_float(decay),
                                 c_float(beta), hs, c_float(output_scale), _ptr(out))
        return out

    def silu(self, values):
        out = np.ascontiguousarray(values, dtype=np.float32).copy()
        self.lib.fortai_silu(_ptr(out), out.size)
        return out

    def dequantize_row(self, weights, row, blocks):
        raw = np.ascontiguousarray(weights).view(np.int8).reshape(-1)
        out = np.zeros(blocks * BLOCK_ELEMS, dtype=np.float32)
        self.lib.fortai_q8_dequantize_row(_ptr(raw[row * blocks * BLOCK_BYTES:]), _ptr(out), blocks)
        return out

    def float_to_half(self, value: float) -> int:
        return int(self.lib.fortai_float_to_half(c_float(value)))

    def thread_count(self) -> int:
        return int(self.lib.ref_thread_count())

    def set_threads(self, threads: int) -> None:
        self.lib.ref_set_threads(int(threads))

    def uses_avx2(self) -> bool:
        return bool(self.lib.ref_uses_avx2())
