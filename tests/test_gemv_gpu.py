"""Parity of the CUDA path with the CPU oracle, through the C ABI (GPU required)."""
import os
import subprocess

import numpy as np
import pytest

from conftest import ROOT, golden, l2_tolerance, reference_gate

pytestmark = pytest.mark.gpu

VARIANTS = [0, 1]   # 0 = automatic choice (slice / register-pipelined / half-block), 1 = always half-block per lane


def check_vector(actual, expected):
    err = float(np.abs(actual.astype(np.float64) - expected.astype(np.float64)).max())
    assert err <= l2_tolerance(expected), (err, l2_tolerance(expected))
    assert reference_gate(actual, expected)


# --------------------------------------------------------------------------- quantizer
def test_quantize_device_is_byte_exact_on_golden_cases(backend, context, dev):
    g = golden("quantize_cases.npz")
    x = g["input"]
    src = dev.to_device(x)
    nbytes = x.size // 32 * 34
    dst = dev.buffer(nbytes)
    assert backend.cuda_q8_quantize_device(context, src, x.size, dst, nbytes).is_ok()
    assert np.array_equal(dev.bytes(dst, nbytes), g["bytes"])


def test_quantize_device_is_byte_exact_on_random_blocks(backend, context, dev, oracle):
    rng = np.random.default_rng(5)
    x = (rng.standard_normal(32 * 4096) * np.repeat(10.0 ** rng.uniform(-6, 4, 4096), 32)
         ).astype(np.float32)
    src = dev.to_device(x)
    nbytes = x.size // 32 * 34
    dst = dev.buffer(nbytes)
    assert backend.cuda_q8_quantize_device(context, src, x.size, dst, nbytes).is_ok()
    assert np.array_equal(dev.bytes(dst, nbytes), oracle.quantize(x)[0])
    # ragged / empty inputs are refused
    assert not backend.cuda_q8_quantize_device(context, src, 40, dst, nbytes).is_ok()
    assert not backend.cuda_q8_quantize_device(context, src, 64, dst, 34).is_ok()


# --------------------------------------------------------------------------- matvec
@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("key", ["r3_k64", "r127_k96", "r128_k256", "r130_k1024"])
def test_matvec_host_on_golden_cases(backend, context, dev, key, variant):
    g = golden("matvec_cases.npz")
    rows, width = (int(s[1:]) for s in key.split("_"))
    context.set_option("gemv_variant", variant)
    w = dev.weights(g[key + "_weights"], rows, width)
    act = g[key + "_quantized"]
    out = np.zeros(rows, np.float32)
    ms, stat = backend.cuda_q8_matvec_host(context, w, act, act.size, out, out.nbytes)
    assert stat.is_ok(), stat
    check_vector(out, g[key + "_values"])
    # exact int32 block dots
    dact = dev.to_device(act)
    ddots = dev.buffer(4 * rows * (width // 32))
    assert backend.cuda_q8_block_dots_device(context, w, dact, ddots, rows * (width // 32)).is_ok()
    assert np.array_equal(dev.int32s(ddots, rows * (width // 32)).reshape(rows, -1),
                          g[key + "_blockdots"])


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("width", [32, 64, 256, 1024, 3840])
@pytest.mark.parametrize("rows", [1, 2, 127, 128, 129])
def test_matvec_edge_shapes(backend, context, dev, oracle, rows, width, variant):
    context.set_option("gemv_variant", variant)
    weights = oracle.make_weights(rows, width, seed=rows * 7 + width)
    x = oracle.normal(width, seed=3)
    expected, quantized, _ = oracle.matvec(weights, rows, width, x)
    w = dev.weights(weights, rows, width)
    out = np.zeros(rows, np.float32)
    _, stat = backend.cuda_q8_matvec_host(context, w, quantized, quantized.size, out, out.nbytes)
    assert stat.is_ok(), stat
    check_vector(out, expected)
    # fp32 activation, quantized on the device in the kernel prologue
    dx = dev.to_device(x)
    dout = dev.buffer(4 * rows)
    assert backend.cuda_q8_matvec_device_f32(context, w, dx, width, dout, rows).is_ok()
    assert np.array_equal(dev.floats(dout, rows), out)   # same kernel arithmetic either way


def decode_shapes():
    shapes = []
    for hidden in (1024, 2048, 2560):
        inner = int(round(3.8 * hidden / 256.0)) * 256
        shapes += [(3 * hidden, hidden), (hidden, hidden), (inner, hidden), (hidden, inner)]
    return shapes


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("rows,width", [(3072, 1024)] + decode_shapes())
def test_decode_projection_sweep(backend, context, dev, oracle, rows, width, variant):
    """Every named decode-step projection at batch 1."""
    context.set_option("gemv_variant", variant)
    weights = oracle.make_weights(rows, width, seed=0)
    x = oracle.normal(width, seed=1)
    expected, quantized, _ = oracle.matvec(weights, rows, width, x)
    w = dev.weights(weights, rows, width)
    dx = dev.to_device(x)
    dout = dev.buffer(4 * rows)
    assert backend.cuda_q8_matvec_device_f32(context, w, dx, width, dout, rows).is_ok()
    check_vector(dev.floats(dout, rows), expected)
    dact = dev.to_device(quantized)
    ddots = dev.buffer(4 * rows * (width // 32))
    assert backend.cuda_q8_block_dots_device(context, w, dact, ddots, rows * (width // 32)).is_ok()
    assert np.array_equal(dev.int32s(ddots, rows * (width // 32)).reshape(rows, -1),
                          oracle.block_dots(weights, quantized, rows, width // 32))


# --------------------------------------------------------------------------- few long rows
@pytest.mark.parametrize("split", [0, 4, 8])
@pytest.mark.parametrize("rows,width", [(5, 8192), (130, 9728), (64, 17408), (9, 2048), (257, 4608),
                                        (33, 18432)])
def test_slice_kernel_on_long_rows(backend, context, dev, oracle, rows, width, split):
    """K-slices of a row on 4 or 8 warps: granule counts that the warps share evenly (16, 36),
    unevenly (19, 34, 9) and barely (4), from Q8_0 and from fp32 activations, against the
    oracle and against the half-block kernel (same block arithmetic, other summation order)."""
    context.set_option("gemv_split", split)
    weights = oracle.make_weights(rows, width, seed=rows + width)
    x = oracle.normal(width, seed=2)
    expected, quantized, _ = oracle.matvec(weights, rows, width, x)
    w = dev.weights(weights, rows, width)
    out = np.zeros(rows, np.float32)
    _, stat = backend.cuda_q8_matvec_host(context, w, quantized, quantized.size, out, out.nbytes)
    assert stat.is_ok(), stat
    check_vector(out, expected)
    dx = dev.to_device(x)
    dout = dev.buffer(4 * rows)
    assert backend.cuda_q8_matvec_device_f32(context, w, dx, width, dout, rows).is_ok()
    sliced = dev.floats(dout, rows)
    assert np.array_equal(sliced, out)           # Q8_0 input and fp32 input: same arithmetic
    again = dev.buffer(4 * rows)
    assert backend.cuda_q8_matvec_device_f32(context, w, dx, width, again, rows).is_ok()
    assert np.array_equal(dev.floats(again, rows), sliced)   # fixed summation order
    context.set_option("gemv_variant", 1)
    assert backend.cuda_q8_matvec_device_f32(context, w, dx, width, again, rows).is_ok()
    check_vector(dev.floats(again, rows), sliced)


def test_config0_against_golden(backend, context, dev, oracle):
    g = golden("config0_3072x1024.npz")
    weights = oracle.make_weights(3072, 1024, seed=0)
    w = dev.weights(weights, 3072, 1024)
    out = np.zeros(3072, np.float32)
    ms, stat = backend.cuda_q8_matvec_host_f32(context, w, g["x"], out)
    assert stat.is_ok(), stat
    check_vector(out, g["values"])


@pytest.mark.parametrize("variant", VARIANTS)
def test_lm_head_full_size(backend, context, dev, oracle, variant):
    """The lm_head at full size: 151936 x 2560, every row against the oracle."""
    rows, width = 151936, 2560
    context.set_option("gemv_variant", variant)
    weights = oracle.make_weights(rows, width, seed=0)
    x = oracle.normal(width, seed=1)
    expected, quantized, _ = oracle.matvec(weights, rows, width, x)
    w = dev.weights(weights, rows, width)
    out = np.zeros(rows, np.float32)
    _, stat = backend.cuda_q8_matvec_host_f32(context, w, x, out)
    assert stat.is_ok(), stat
    check_vector(out, expected)
    assert int(np.argmax(out)) == int(np.argmax(expected))
    dact = dev.to_device(quantized)
    dres = dev.buffer(4 * rows)
    kernel_ms, stat = backend.cuda_q8_matvec_resident(context, w, dact, dres)
    assert stat.is_ok() and kernel_ms > 0
    assert np.array_equal(dev.floats(dres, rows), out)


# --------------------------------------------------------------------------- grouped
def test_reference_smoke_fixture(backend, context, dev, oracle):
    """The reference's own ABI smoke test (tools/cuda_backend_smoke.cu), case for case."""
    g = golden("smoke_fixture.npz")
    rows = width = 4096
    blocks = width // 32
    weights = oracle.fixture_fill_q8(rows, blocks, 0x6f727461, True)
    act = g["4096x4096_activation"]
    expected = g["4096x4096_oracle"]
    w = dev.weights(weights, rows, width)
    outs = [np.zeros(rows, np.float32) for _ in range(7)]
    _, stat = backend.cuda_q8_matvec_host(context, w, act, act.size, outs[0], outs[0].nbytes)
    assert stat.is_ok(), stat
    _, stat = backend.cuda_q8_matvec_host_pair(context, w, w, act, act.size, outs[1],
                                               outs[1].nbytes, outs[2], outs[2].nbytes)
    assert stat.is_ok(), stat
    _, stat = backend.cuda_q8_matvec_host_triplet(context, w, w, w, act, act.size, outs[3],
                                                  outs[3].nbytes, outs[4], outs[4].nbytes,
                                                  outs[5], outs[5].nbytes)
    assert stat.is_ok(), stat
    dact = dev.to_device(act)
    dout = dev.buffer(4 * rows)
    _, stat = backend.cuda_q8_matvec_resident(context, w, dact, dout)
    assert stat.is_ok(), stat
    outs[6] = dev.floats(dout, rows)
    for out in outs:
        assert reference_gate(out, expected)
    # 128 blocks per row: the reference refuses the contiguous form here
    # (backend/cuda/fortai_cuda_backend.cu:257-258) and so does this backend
    big = np.zeros(3 * rows, np.float32)
    _, stat = backend.cuda_q8_matvec_host_triplet_contiguous(context, w, w, w, act, act.size, big,
                                                             big.nbytes)
    assert not stat.is_ok() and stat.code == backend.FORTAI_UNSUPPORTED


def test_compiled_reference_smoke_program():
    """tools/cuda_backend_smoke.cu compiled unchanged and linked to this backend."""
    exe = os.path.join(ROOT, "oracle", "_ref", "cuda_backend_smoke")
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref/cuda_backend_smoke not built")
    result = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert result.returncode == 0, result.stdout + result.stderr
    assert '"correct":true' in result.stdout


def test_pair_and_triplet_with_different_row_counts(backend, context, dev, oracle):
    width = 1024
    rows3 = (96, 200, 33)
    mats = [oracle.make_weights(r, width, seed=20 + i) for i, r in enumerate(rows3)]
    x = oracle.normal(width, seed=8)
    expected = oracle.matvec_triplet(mats[0], mats[1], mats[2], rows3, width, x)
    quantized = oracle.quantize(x)[0]
    ws = [dev.weights(m, r, width) for m, r in zip(mats, rows3)]
    outs = [np.zeros(r, np.float32) for r in rows3]
    _, stat = backend.cuda_q8_matvec_host_triplet(context, ws[0], ws[1], ws[2], quantized,
                                                  quantized.size, outs[0], outs[0].nbytes, outs[1],
                                                  outs[1].nbytes, outs[2], outs[2].nbytes)
    assert stat.is_ok(), stat
    for out, exp in zip(outs, expected):
        check_vector(out, exp)
    combined = np.zeros(sum(rows3), np.float32)
    _, stat = backend.cuda_q8_matvec_host_triplet_contiguous(context, ws[0], ws[1], ws[2],
                                                             quantized, quantized.size, combined,
                                                             combined.nbytes)
    assert stat.is_ok(), stat
    assert np.array_equal(combined, np.concatenate(outs))
    # mismatched widths are refused (backend.cu:262)
    other = dev.weights(oracle.make_weights(8, 512, seed=1), 8, 512)
    o8 = np.zeros(8, np.float32)
    _, stat = backend.cuda_q8_matvec_host_pair(context, ws[0], other, quantized, quantized.size,
                                               outs[0], outs[0].nbytes, o8, o8.nbytes)
    assert not stat.is_ok()


# --------------------------------------------------------------------------- FFN
@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("hidden,inner", [(1024, 3840), (2560, 9728), (5120, 17408)])
def test_ffn_host_and_device(backend, context, dev, oracle, hidden, inner, variant):
    context.set_option("gemv_variant", variant)
    gate = oracle.make_weights(inner, hidden, seed=1)
    up = oracle.make_weights(inner, hidden, seed=2)
    down = oracle.make_weights(hidden, inner, seed=3)
    x = oracle.normal(hidden, seed=4)
    expected = oracle.ffn(gate, up, down, inner, hidden, hidden, x)
    wg, wu, wd = dev.weights(gate, inner, hidden), dev.weights(up, inner, hidden), \
        dev.weights(down, hidden, inner)
    quantized = oracle.quantize(x)[0]
    out = np.zeros(hidden, np.float32)
    _, stat = backend.cuda_q8_ffn_host(context, wg, wu, wd, quantized, quantized.size, out,
                                       out.nbytes)
    assert stat.is_ok(), stat
    # the hidden vector is re-quantized between the two halves; a one-ulp difference
    # in silu can move a quant by one step, hence twice the plain matvec bound
    err = float(np.abs(out.astype(np.float64) - expected).max())
    assert err <= 2 * l2_tolerance(expected), (err, l2_tolerance(expected))
    dx = dev.to_device(x)
    dout = dev.buffer(4 * hidden)
    assert backend.cuda_q8_ffn_device(context, wg, wu, wd, dx, hidden, dout, hidden).is_ok()
    assert np.array_equal(dev.floats(dout, hidden), out)
    # shape rule of the reference (backend.cu:1257-1262)
    assert not backend.cuda_q8_ffn_device(context, wg, wu, wg, dx, hidden, dout, hidden).is_ok()


def test_dependent_launch_settings_give_identical_results(backend, context, dev, oracle):
    """Where a GEMV lets its successor be scheduled (after its row loop / at its first
    instruction / at once when its grid fills the machine) and whether launches overlap at
    all are scheduling choices: a chain of calls in which each reads what the one before
    wrote must give the same bits under every setting, and its first link the oracle's."""
    hidden, inner = 1024, 3840
    up = oracle.make_weights(inner, hidden, seed=21)
    down = oracle.make_weights(hidden, inner, seed=22)
    wu, wd = dev.weights(up, inner, hidden), dev.weights(down, hidden, inner)
    x = oracle.normal(hidden, seed=23)
    first_link = oracle.matvec(up, inner, hidden, x)[0]
    assert not context.set_option("gemv_early_trigger", 4).is_ok()
    results = []
    for overlap in (0, 1):
        for trigger in (0, 1, 2, 3):
            assert context.set_option("gemv_overlap", overlap).is_ok()
            assert context.set_option("gemv_early_trigger", trigger).is_ok()
            dx, dmid = dev.to_device(x), dev.buffer(4 * inner)
            for link in range(4):   # wide -> narrow -> wide ...: many- and few-CTA successors
                dout = dev.buffer(4 * hidden)
                assert backend.cuda_q8_matvec_device_f32(context, wu, dx, hidden, dmid,
                                                         inner).is_ok()
                if link == 0:
                    check_vector(dev.floats(dmid, inner), first_link)
                assert backend.cuda_q8_matvec_device_f32(context, wd, dmid, inner, dout,
                                                         hidden).is_ok()
                dx = dout
            results.append(dev.floats(dx, hidden).copy())
    assert np.abs(results[0]).max() > 0
    for other in results[1:]:
        assert np.array_equal(results[0], other)


# --------------------------------------------------------------------------- ABI behaviour
def test_argument_validation_and_ownership(backend, context, dev, oracle):
    rows, width = 64, 256
    weights = oracle.make_weights(rows, width, seed=1)
    w = dev.weights(weights, rows, width)
    act = oracle.quantize(oracle.normal(width, seed=2))[0]
    out = np.zeros(rows, np.float32)
    # short activation / short output -> INVALID, nothing written
    _, stat = backend.cuda_q8_matvec_host(context, w, act, act.size - 1, out, out.nbytes)
    assert not stat.is_ok()
    _, stat = backend.cuda_q8_matvec_host(context, w, act, act.size, out, out.nbytes - 4)
    assert not stat.is_ok()
    assert (out == 0).all()
    # weights belong to the context that uploaded them (backend.cu:995)
    other = backend.cuda_q8_context_t()
    assert other.create(0).is_ok()
    _, stat = backend.cuda_q8_matvec_host(other, w, act, act.size, out, out.nbytes)
    assert not stat.is_ok()
    other.destroy()
    # width must be a multiple of 32, byte count must cover the matrix
    bad = backend.cuda_q8_weights_t()
    assert not bad.upload(context, weights, weights.size, rows, 250).is_ok()
    assert not bad.upload(context, weights, weights.size - 1, rows, width).is_ok()
    dx = dev.to_device(oracle.normal(width, seed=2))
    dout = dev.buffer(4 * rows)
    assert not backend.cuda_q8_matvec_device_f32(context, w, dx, width - 32, dout, rows).is_ok()
    assert not backend.cuda_q8_matvec_device_f32(context, w, dx, width, dout, rows - 1).is_ok()


def test_launch_counter_and_stream_handle(backend, context, dev, oracle):
    rows, width = 256, 512
    w = dev.weights(oracle.make_weights(rows, width, seed=1), rows, width)
    before = context.launch_count()
    dx = dev.to_device(oracle.normal(width, seed=2))
    dout = dev.buffer(4 * rows)
    assert backend.cuda_q8_matvec_device_f32(context, w, dx, width, dout, rows).is_ok()
    assert context.launch_count() == before + 1
    assert context.stream() != 0
    assert context.synchronize().is_ok()


def test_graph_capture_replays_the_matvec(backend, context, dev, oracle):
    rows, width = 512, 1024
    weights = oracle.make_weights(rows, width, seed=1)
    w = dev.weights(weights, rows, width)
    x = oracle.normal(width, seed=2)
    dx = dev.to_device(x)
    dout = dev.buffer(4 * rows)
    assert backend.cuda_q8_matvec_device_f32(context, w, dx, width, dout, rows).is_ok()
    first = dev.floats(dout, rows)
    assert context.capture_begin().is_ok()
    assert backend.cuda_q8_matvec_device_f32(context, w, dx, width, dout, rows).is_ok()
    assert context.capture_end().is_ok()
    x2 = oracle.normal(width, seed=3)
    assert context.upload_real(dx, x2).is_ok()
    assert context.graph_launch().is_ok()
    second = dev.floats(dout, rows)
    check_vector(second, oracle.matvec(weights, rows, width, x2)[0])
    assert not np.array_equal(first, second)


def test_small_device_ops(backend, context, dev, oracle):
    rows, width = 40, 256
    weights = oracle.make_weights(rows, width, seed=1)
    w = dev.weights(weights, rows, width)
    dout = dev.buffer(4 * width)
    assert backend.cuda_qwen35_embedding_device(context, w, 17, dout, width).is_ok()
    assert np.array_equal(dev.floats(dout, width), oracle.dequantize_row(weights, 17, width // 32))
    assert not backend.cuda_qwen35_embedding_device(context, w, rows, dout, width).is_ok()
    a = oracle.normal(width, seed=5)
    b = oracle.normal(width, seed=6)
    da, db = dev.to_device(a), dev.to_device(b)
    assert backend.cuda_qwen35_add_device(context, da, db, dout, width).is_ok()
    assert np.array_equal(dev.floats(dout, width), a + b)
    assert backend.cuda_qwen35_rms_norm_device(context, da, db, dout, width, 1e-6).is_ok()
    inv = 1.0 / np.sqrt(np.float32(np.mean(a.astype(np.float64) ** 2)) + np.float32(1e-6))
    assert np.allclose(dev.floats(dout, width), a * np.float32(inv) * b, rtol=2e-6, atol=1e-7)
    assert backend.cuda_qwen35_copy_device(context, da, dout, 4 * width).is_ok()
    assert np.array_equal(dev.floats(dout, width), a)


def test_host_f32_stores_straight_into_page_locked_output(backend, context, dev, oracle):
    """With a page-locked (device-mapped) output buffer the GEMV writes the results to host
    memory itself; with pageable memory they come back through a copy.  Same bits."""
    import torch
    rows, width = 5000, 2560
    weights = oracle.make_weights(rows, width, seed=21)
    x = oracle.normal(width, seed=22)
    expected = oracle.matvec(weights, rows, width, x)[0]
    w = dev.weights(weights, rows, width)
    pageable = np.zeros(rows, np.float32)
    _, stat = backend.cuda_q8_matvec_host_f32(context, w, x, pageable)
    assert stat.is_ok(), stat
    assert np.abs(pageable - expected).max() <= l2_tolerance(expected)
    locked = torch.zeros(rows + 3, dtype=torch.float32).pin_memory()
    before = context.launch_count()
    ms, stat = backend.cuda_q8_matvec_host_f32(context, w, x, locked.numpy()[:rows])
    assert stat.is_ok(), stat
    assert context.launch_count() - before == 1
    assert np.array_equal(locked.numpy()[:rows], pageable)
    assert float(locked[rows:].abs().max()) == 0.0        # nothing past the last row
    # switched off: back to the copy
    assert context.set_option("host_direct_output", 0).is_ok()
    again = torch.zeros(rows, dtype=torch.float32).pin_memory()
    _, stat = backend.cuda_q8_matvec_host_f32(context, w, x, again.numpy())
    assert stat.is_ok(), stat
    assert np.array_equal(again.numpy(), pageable)


def test_reference_host_call_into_page_locked_output(backend, context, dev, oracle):
    """fortai_cuda_q8_matvec_host (Q8_0 activation from the host) with a page-locked output."""
    import torch
    rows, width = 3000, 1024
    weights = oracle.make_weights(rows, width, seed=31)
    x = oracle.normal(width, seed=32)
    expected, quantized, _ = oracle.matvec(weights, rows, width, x)
    w = dev.weights(weights, rows, width)
    pageable = np.zeros(rows, np.float32)
    _, stat = backend.cuda_q8_matvec_host(context, w, quantized, quantized.size, pageable,
                                          pageable.nbytes)
    assert stat.is_ok(), stat
    locked = torch.zeros(rows, dtype=torch.float32).pin_memory()
    _, stat = backend.cuda_q8_matvec_host(context, w, quantized, quantized.size, locked.numpy(),
                                          locked.numpy().nbytes)
    assert stat.is_ok(), stat
    assert np.array_equal(locked.numpy(), pageable)
    assert np.abs(pageable - expected).max() <= l2_tolerance(expected)


def test_known_answers_of_the_reference_test_program_through_cuda(backend, context, dev, oracle):
    """test/test_fortai_smoke.f90:221-265: one 32-wide row with scale 1.0 and quants 1..32
    against a vector of ones gives 527.9677734375; the triplet of that row, two rows of
    1x and 2x, and one of 3x gives [527.97, 527.97, 1055.94, 1583.90].  The same bytes
    through the CUDA entry points (fp32 vector in, and pre-quantized)."""
    w1 = np.zeros(34, np.int8); w1[1] = 0x3c; w1[2:] = np.arange(1, 33)
    w2 = np.zeros(68, np.int8)
    for r in range(2):
        w2[r * 34 + 1] = 0x3c
        w2[r * 34 + 2:r * 34 + 34] = (r + 1) * np.arange(1, 33)
    w3 = np.zeros(34, np.int8); w3[1] = 0x3c; w3[2:] = 3 * np.arange(1, 33)
    ones = np.ones(32, np.float32)
    h1, h2, h3 = dev.weights(w1, 1, 32), dev.weights(w2, 2, 32), dev.weights(w3, 1, 32)
    out = np.zeros(1, np.float32)
    _, stat = backend.cuda_q8_matvec_host_f32(context, h1, ones, out)
    assert stat.is_ok(), stat
    assert abs(float(out[0]) - 527.9677734375) < 1.0e-4     # the reference test's own bound
    assert float(out[0]) == 527.9677734375                  # and in fact exact
    quantized = oracle.quantize(ones)[0]
    a, b, c = np.zeros(1, np.float32), np.zeros(2, np.float32), np.zeros(1, np.float32)
    _, stat = backend.cuda_q8_matvec_host_triplet(context, h1, h2, h3, quantized, quantized.size,
                                                  a, a.nbytes, b, b.nbytes, c, c.nbytes)
    assert stat.is_ok(), stat
    got = np.array([a[0], b[0], b[1], c[0]], np.float64)
    expected = np.array([527.9677734375, 527.9677734375, 1055.935546875, 1583.9033203125])
    assert np.abs(got - expected).max() < 1.0e-4
    # the exact int32 block dot of the row: sum(1..32) * 127
    dq = dev.to_device(quantized)
    ddots = dev.buffer(4)
    assert backend.cuda_q8_block_dots_device(context, h1, dq, ddots, 1).is_ok()
    assert int(dev.int32s(ddots, 1)[0]) == 127 * 528
