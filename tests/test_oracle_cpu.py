"""The CPU oracle against the reference's golden vectors and compiled C code."""
import hashlib
import json
import os

import numpy as np
import pytest

from conftest import GOLDEN, golden, l2_tolerance


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def test_known_answers_of_reference_test_program(oracle):
    # test/test_fortai_smoke.f90:221-265
    kat = json.load(open(os.path.join(GOLDEN, "known_answers.json")))
    w1 = np.zeros(34, np.int8); w1[1] = 0x3c; w1[2:] = np.arange(1, 33)
    ones = np.ones(32, np.float32)
    values, quantized, scales = oracle.matvec(w1, 1, 32, ones)
    assert float(values[0]) == 527.9677734375 == kat["single"]
    assert float(scales[0]) == kat["activation_scale"]
    assert np.array_equal(oracle.dequantize_row(w1, 0, 1), np.arange(1, 33, dtype=np.float32))
    w2 = np.zeros(68, np.int8)
    for r in range(2):
        w2[r * 34 + 1] = 0x3c
        w2[r * 34 + 2:r * 34 + 34] = (r + 1) * np.arange(1, 33)
    w3 = np.zeros(34, np.int8); w3[1] = 0x3c; w3[2:] = 3 * np.arange(1, 33)
    a, b, c = oracle.matvec_triplet(w1, w2, w3, (1, 2, 1), 32, ones)
    got = [float(a[0]), float(b[0]), float(b[1]), float(c[0])]
    assert got == kat["expected_in_reference_test"] == kat["triplet"]


def test_quantizer_matches_golden_bytes(oracle):
    g = golden("quantize_cases.npz")
    out, scales = oracle.quantize(g["input"])
    assert np.array_equal(out, g["bytes"])
    assert np.array_equal(scales.view(np.uint32), g["scales"].view(np.uint32))


def test_quantizer_rejects_ragged_and_empty(oracle):
    # fortai_q8_dot.c:204-205: nothing is written
    out = np.full(68, 77, np.int8)
    scales = np.full(2, 9.0, np.float32)
    x = np.ones(40, np.float32)
    oracle.lib().oracle_q8_quantize(x.ctypes.data, out.ctypes.data, scales.ctypes.data, 40)
    oracle.lib().oracle_q8_quantize(x.ctypes.data, out.ctypes.data, scales.ctypes.data, 0)
    assert (out == 77).all() and (scales == 9.0).all()


@pytest.mark.parametrize("key", ["r3_k64", "r127_k96", "r128_k256", "r130_k1024"])
def test_matvec_matches_golden_bit_for_bit(oracle, key):
    g = golden("matvec_cases.npz")
    rows, width = (int(s[1:]) for s in key.split("_"))
    values, quantized, scales = oracle.matvec(g[key + "_weights"], rows, width, g[key + "_x"])
    assert np.array_equal(quantized, g[key + "_quantized"])
    assert np.array_equal(values.view(np.uint32), g[key + "_values"].view(np.uint32))
    dots = oracle.block_dots(g[key + "_weights"], quantized, rows, width // 32)
    assert np.array_equal(dots, g[key + "_blockdots"])
    # the block-wise (scalar-path) summation differs only in rounding
    blockwise = np.array([oracle.dot(g[key + "_weights"], quantized, scales, r, width // 32, True)
                          for r in range(rows)], np.float32)
    assert np.abs(blockwise - values).max() <= l2_tolerance(values)


def test_silu_product_matches_golden(oracle):
    g = golden("silu_cases.npz")
    got = oracle.silu_product(g["left"], g["right"], contract=True)
    assert np.array_equal(got.view(np.uint32), g["product"].view(np.uint32))
    plain = oracle.silu_product(g["left"], g["right"], contract=False)
    assert np.abs(plain - g["product"]).max() <= 2e-5          # test_fortai_smoke.f90:296
    x = g["left"].astype(np.float64)
    exact = x / (1.0 + np.exp(-x)) * g["right"].astype(np.float64)
    inside = np.abs(x) <= 20
    assert np.abs(got[inside] - exact[inside]).max() <= 2e-5


def test_smoke_fixture_generator_and_oracle(oracle):
    # tools/cuda_backend_smoke.cu:33-49 + fortai_q8_bench_spec.h:68-101
    g = golden("smoke_fixture.npz")
    for rows, width in ((64, 256), (4096, 4096)):
        blocks = width // 32
        w = oracle.fixture_fill_q8(rows, blocks, 0x6f727461, True)
        a = oracle.fixture_fill_q8(1, blocks, 0x6f727461 ^ 0x9e3779b9, False)
        a2 = a.reshape(blocks, 34)
        a2[:, 2] = 127
        a2[:, 3] = np.uint8(256 - 127)
        assert sha(w) == str(g[f"{rows}x{width}_weights_sha256"])
        assert np.array_equal(a, g[f"{rows}x{width}_activation"])
        out = oracle.fixture_matvec(w, a, rows, blocks)
        assert np.array_equal(out.view(np.uint32), g[f"{rows}x{width}_oracle"].view(np.uint32))


def test_config0_inputs_and_outputs(oracle):
    g = golden("config0_3072x1024.npz")
    w = oracle.make_weights(3072, 1024, seed=0, sigma=0.02)
    assert sha(w) == str(g["weights_sha256"])
    x = oracle.normal(1024, seed=1)
    assert np.array_equal(x, g["x"])
    values, quantized, _ = oracle.matvec(w, 3072, 1024, x)
    assert np.array_equal(quantized, g["quantized"])
    assert np.array_equal(values.view(np.uint32), g["values"].view(np.uint32))
    assert sha(oracle.block_dots(w, quantized, 3072, 32)) == str(g["blockdots_sha256"])


def test_row_shards_regenerate_the_same_matrix(oracle):
    full = oracle.make_weights(64, 256, seed=3).reshape(64, -1)
    part = oracle.make_weights(16, 256, seed=3, first_row=32).reshape(16, -1)
    assert np.array_equal(full[32:48], part)


def test_drivers_validate_shapes(oracle):
    w = oracle.make_weights(4, 64, seed=1)
    with pytest.raises(ValueError):
        oracle.matvec(w, 4, 64, np.ones(32, np.float32))
    with pytest.raises(ValueError):
        oracle.matvec_pair(w, w, 4, 64, np.ones(64, np.float32), second_rows=3)
    with pytest.raises(ValueError):
        oracle.matvec_triplet(w, w, w, (4, 4, 4), 64, np.ones(64, np.float32), widths=(64, 32, 64))


def test_matmul_is_independent_matvecs(oracle):
    w = oracle.make_weights(40, 128, seed=5)
    x = oracle.normal(3 * 128, seed=6).reshape(3, 128)
    values, quantized, scales = oracle.matmul(w, 40, 128, x)
    for t in range(3):
        assert np.array_equal(values[t], oracle.matvec(w, 40, 128, x[t])[0])


def test_ffn_composition(oracle):
    hidden, inner = 64, 96
    gate = oracle.make_weights(inner, hidden, seed=1)
    up = oracle.make_weights(inner, hidden, seed=2)
    down = oracle.make_weights(hidden, inner, seed=3)
    x = oracle.normal(hidden, seed=4)
    out = oracle.ffn(gate, up, down, inner, hidden, hidden, x)
    g, u = oracle.matvec_pair(gate, up, inner, hidden, x)
    h = oracle.silu_product(g, u)
    assert np.array_equal(out, oracle.matvec(down, hidden, inner, h)[0])


# ---- against the reference's own compiled C code (skipped without oracle/_ref)
def test_restatement_equals_compiled_reference(oracle, reference):
    rng = np.random.default_rng(11)
    for scale in (1e-9, 1e-3, 1.0, 300.0, 1e5):
        x = (rng.standard_normal(32 * 64) * scale).astype(np.float32)
        a, b = oracle.quantize(x), reference.quantize(x)
        assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    rows, width = 257, 2560
    w = oracle.make_weights(rows, width, seed=9)
    x = oracle.normal(width, seed=10)
    mine = oracle.matvec(w, rows, width, x)
    theirs = reference.matvec(w, rows, width, x)
    assert np.array_equal(mine[1], theirs[1])
    assert np.array_equal(mine[0].view(np.uint32), theirs[0].view(np.uint32))
    left = np.linspace(-30, 30, 1003).astype(np.float32)
    right = rng.standard_normal(1003).astype(np.float32)
    assert np.array_equal(oracle.silu_product(left, right).view(np.uint32),
                          reference.silu_product(left, right).view(np.uint32))
    assert np.array_equal(oracle.dequantize_row(w, 5, width // 32),
                          reference.dequantize_row(w, 5, width // 32))
