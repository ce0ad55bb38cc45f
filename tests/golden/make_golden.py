"""Regenerates the golden fixtures in this directory FROM THE REFERENCE ITSELF.

Needs the reference checkout (path in FORTAI_REFERENCE): its C arithmetic is
compiled in place by oracle/Makefile into oracle/_ref, and its bench-spec header
is compiled into a helper under oracle/_ref.  Nothing from the restated oracle
(oracle/q8_oracle.c) is used to produce an expected value here, with one
documented exception: the seeded N(0, sigma) sample generator, which has no
counterpart in the reference and only produces INPUTS.

    python tests/golden/make_golden.py
"""
from __future__ import annotations

import hashlib
import json
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import q8_oracle as o  # noqa: E402

REFERENCE = os.environ.get("FORTAI_REFERENCE") or os.path.normpath(
    os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "..", "reference"))


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def exact_block_dots(weights: np.ndarray, act: np.ndarray, rows: int, blocks: int) -> np.ndarray:
    w = weights.view(np.int8).reshape(rows, blocks, 34)[:, :, 2:].astype(np.int64)
    a = act.view(np.int8).reshape(blocks, 34)[:, 2:].astype(np.int64)
    return (w * a[None]).sum(-1).astype(np.int32)


def main() -> None:
    subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), "ref"], check=True)
    ref = o.Reference()
    assert ref.uses_avx2(), "the golden vectors pin the AVX2 path of the reference"
    rng = np.random.default_rng(20240607)

    # 1. known answers spelled out in the reference's own test program
    #    (test/test_fortai_smoke.f90:221-265), recomputed through its C code
    w1 = np.zeros(34, np.int8); w1[1] = 0x3c; w1[2:] = np.arange(1, 33)
    w2 = np.zeros(68, np.int8)
    for r in range(2):
        w2[r * 34 + 1] = 0x3c
        w2[r * 34 + 2:r * 34 + 34] = (r + 1) * np.arange(1, 33)
    w3 = np.zeros(34, np.int8); w3[1] = 0x3c; w3[2:] = 3 * np.arange(1, 33)
    ones = np.ones(32, np.float32)
    kat = {
        "single": float(ref.matvec(w1, 1, 32, ones)[0][0]),
        "triplet": [float(ref.matvec(w1, 1, 32, ones)[0][0]),
                    *[float(v) for v in ref.matvec(w2, 2, 32, ones)[0]],
                    float(ref.matvec(w3, 1, 32, ones)[0][0])],
        "expected_in_reference_test": [527.9677734375, 527.9677734375, 1055.935546875,
                                       1583.9033203125],
        "activation_scale": float(ref.quantize(ones)[1][0]),
        "dequantized_row": [float(v) for v in ref.dequantize_row(w1, 0, 1)],
    }
    with open(os.path.join(HERE, "known_answers.json"), "w") as f:
        json.dump(kat, f, indent=1)

    # 2. quantizer: edge cases + random blocks
    blocks = []
    blocks.append(np.zeros(32, np.float32))                                   # all-zero block
    blocks.append(np.full(32, -3.5, np.float32))                              # all equal, negative
    blocks.append(np.linspace(-1, 1, 32).astype(np.float32))
    b = np.zeros(32, np.float32); b[0] = 127.0; b[1:] = np.arange(31) + 0.5   # exact .5 ties
    blocks.append(b)
    b = np.zeros(32, np.float32); b[0] = -254.0; b[1:] = (np.arange(31) - 15) * 1.0 + 1.0
    blocks.append(b)                                                          # ties after scaling by 0.5
    blocks.append((rng.standard_normal(32) * 1e-7).astype(np.float32))        # fp16-subnormal scale
    blocks.append((rng.standard_normal(32) * 1e-12).astype(np.float32))       # scale underflows to 0
    blocks.append((rng.standard_normal(32) * 3e6).astype(np.float32))         # scale > 65504/127 -> inf region
    blocks.append((rng.standard_normal(32) * 1e4).astype(np.float32))
    for s in (0.02, 1.0, 17.0):
        blocks.append((rng.standard_normal(32 * 40) * s).astype(np.float32))
    qin = np.concatenate(blocks)
    qout, qscales = ref.quantize(qin)
    np.savez_compressed(os.path.join(HERE, "quantize_cases.npz"), input=qin, bytes=qout,
                        scales=qscales)

    # 3. matvec: small shapes around the serial/parallel switch, with exact block dots
    cases = {}
    for rows, width in ((3, 64), (127, 96), (128, 256), (130, 1024)):
        wts = ref.quantize((rng.standard_normal(rows * width) * 0.02).astype(np.float32))[0]
        x = rng.standard_normal(width).astype(np.float32)
        values, quantized, scales = ref.matvec(wts, rows, width, x)
        key = f"r{rows}_k{width}"
        cases[key + "_weights"] = wts
        cases[key + "_x"] = x
        cases[key + "_values"] = values
        cases[key + "_quantized"] = quantized
        cases[key + "_scales"] = scales
        cases[key + "_blockdots"] = exact_block_dots(wts, quantized, rows, width // 32)
    np.savez_compressed(os.path.join(HERE, "matvec_cases.npz"), **cases)

    # 4. SiLU product, the points of the reference's own test plus the clamps
    left = np.concatenate([np.linspace(-20, 20, 256), [-25, -20.5, 20.5, 30, 0, 1e-8, -1e-8, 5]]
                          ).astype(np.float32)
    right = (1.0 + 0.25 * np.sin(np.arange(1, left.size + 1))).astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "silu_cases.npz"), left=left, right=right,
                        product=ref.silu_product(left, right))

    # 5. the reference's ABI-smoke fixture (xorshift32) and its scalar oracle
    helper = os.path.join(ROOT, "oracle", "_ref", "fixture_from_reference")
    subprocess.run(["g++", "-O2", "-std=c++17", "-I", os.path.join(REFERENCE, "backend", "cuda"),
                    "-o", helper, os.path.join(HERE, "fixture_from_reference.cpp")], check=True)
    smoke = {}
    for rows, width in ((4096, 4096), (64, 256)):
        prefix = os.path.join(ROOT, "oracle", "_ref", f"fixture_{rows}x{width}")
        subprocess.run([helper, str(rows), str(width), prefix], check=True)
        wts = np.fromfile(prefix + ".weights.bin", dtype=np.uint8)
        act = np.fromfile(prefix + ".activation.bin", dtype=np.uint8)
        orc = np.fromfile(prefix + ".oracle.bin", dtype=np.float32)
        smoke[f"{rows}x{width}_weights_sha256"] = np.array(sha(wts))
        smoke[f"{rows}x{width}_activation"] = act
        smoke[f"{rows}x{width}_oracle"] = orc
        for suffix in (".weights.bin", ".activation.bin", ".oracle.bin"):
            os.remove(prefix + suffix)
    np.savez_compressed(os.path.join(HERE, "smoke_fixture.npz"), **smoke)

    # 6. the CPU-bench configuration: 3072 x 1024, seed 0 (inputs from the seeded
    #    generator, outputs from the reference's C code)
    rows, width = 3072, 1024
    wts = o.make_weights(rows, width, seed=0, sigma=0.02)
    wts_ref = ref.quantize(o.normal(rows * width, seed=0, sigma=0.02))[0]
    assert np.array_equal(wts, wts_ref)
    x = o.normal(width, seed=1, sigma=1.0)
    values, quantized, scales = ref.matvec(wts, rows, width, x)
    np.savez_compressed(os.path.join(HERE, "config0_3072x1024.npz"),
                        weights_sha256=np.array(sha(wts)), x=x, values=values,
                        quantized=quantized,
                        blockdots_sha256=np.array(sha(exact_block_dots(wts, quantized, rows,
                                                                        width // 32))))
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
