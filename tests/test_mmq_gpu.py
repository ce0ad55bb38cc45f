"""Batched (prefill) product against `tokens` independent oracle matvecs (GPU required)."""
import numpy as np
import pytest

from conftest import l2_tolerance

pytestmark = pytest.mark.gpu


def exact_dots(weights, quantized, tokens, rows, blocks):
    w = weights.view(np.int8).reshape(rows, blocks, 34)[:, :, 2:].astype(np.int32)
    a = quantized.view(np.int8).reshape(tokens, blocks, 34)[:, :, 2:].astype(np.int32)
    return np.einsum("rbi,tbi->trb", w, a).astype(np.int32)


def check_rows(actual, expected):
    for t in range(expected.shape[0]):
        err = float(np.abs(actual[t].astype(np.float64) - expected[t]).max())
        assert err <= l2_tolerance(expected[t]), (t, err, l2_tolerance(expected[t]))


@pytest.mark.parametrize("tokens,tensor_from", [(16, 0), (64, 0), (64, 33), (128, 0), (512, 0)])
def test_prefill_config_shapes(backend, context, dev, oracle, tokens, tensor_from):
    """The prefill configuration: M in {16, 64, 128, 512} x K=2560 x N=9728; 64 tokens through
    the few-token kernel (the default up to 64) and through the tcgen05 kernel's 64-token tile."""
    rows, width = 9728, 2560
    context.set_option("mmq_min_tokens", tensor_from)
    weights = oracle.make_weights(rows, width, seed=2)
    x = oracle.normal(tokens * width, seed=3).reshape(tokens, width)
    expected = oracle.matmul(weights, rows, width, x)[0]
    w = dev.weights(weights, rows, width)
    out = np.zeros((tokens, rows), np.float32)
    ms, stat = backend.cuda_q8_matmul_host_f32(context, w, x, tokens, out)
    assert stat.is_ok(), stat
    check_rows(out, expected)


@pytest.mark.parametrize("force_tensor", [True, False])
@pytest.mark.parametrize("tokens,rows,width", [(1, 130, 128), (33, 130, 384), (100, 257, 256),
                                               (128, 128, 128), (200, 512, 1024)])
def test_ragged_shapes_and_block_dots(backend, context, dev, oracle, tokens, rows, width,
                                      force_tensor):
    context.set_option("mmq_min_tokens", 1 if force_tensor else 100000)
    blocks = width // 32
    weights = oracle.make_weights(rows, width, seed=rows + width)
    x = oracle.normal(tokens * width, seed=tokens).reshape(tokens, width)
    expected, quantized, _ = oracle.matmul(weights, rows, width, x)
    w = dev.weights(weights, rows, width)
    dx = dev.to_device(x)
    dout = dev.buffer(4 * tokens * rows)
    assert backend.cuda_q8_matmul_device_f32(context, w, dx, tokens, dout, tokens * rows).is_ok()
    check_rows(dev.floats(dout, tokens * rows).reshape(tokens, rows), expected)
    # pre-quantized activation: same result, and exact int32 block dots
    dq = dev.to_device(quantized)
    dres = dev.buffer(4 * tokens * rows)
    ms, stat = backend.cuda_q8_matmul_resident(context, w, dq, tokens, dres)
    assert stat.is_ok(), stat
    # a tile shared by two CTAs is completed with fp32 atomic adds, so two runs may differ
    # in the last bit; both must meet the bound against the oracle
    check_rows(dev.floats(dres, tokens * rows).reshape(tokens, rows), expected)
    ddots = dev.buffer(4 * tokens * rows * blocks)
    assert backend.cuda_q8_matmul_block_dots_device(context, w, dq, tokens, ddots,
                                                    tokens * rows * blocks).is_ok()
    got = dev.int32s(ddots, tokens * rows * blocks).reshape(tokens, rows, blocks)
    assert np.array_equal(got, exact_dots(weights, quantized, tokens, rows, blocks))


def test_prefill_matches_the_batch1_kernel_closely(backend, context, dev, oracle):
    """Token t of the batched product and a batch-1 matvec of the same vector see the
    same int32 dots and scales; only the fp32 summation order differs."""
    rows, width, tokens = 1024, 2560, 64
    weights = oracle.make_weights(rows, width, seed=1)
    x = oracle.normal(tokens * width, seed=2).reshape(tokens, width)
    w = dev.weights(weights, rows, width)
    out = np.zeros((tokens, rows), np.float32)
    _, stat = backend.cuda_q8_matmul_host_f32(context, w, x, tokens, out)
    assert stat.is_ok(), stat
    single = np.zeros(rows, np.float32)
    _, stat = backend.cuda_q8_matvec_host_f32(context, w, np.ascontiguousarray(x[5]), single)
    assert stat.is_ok(), stat
    assert np.abs(out[5] - single).max() <= l2_tolerance(single)


def test_prefill_argument_validation(backend, context, dev, oracle):
    rows, width = 128, 128
    w = dev.weights(oracle.make_weights(rows, width, seed=1), rows, width)
    dx = dev.to_device(oracle.normal(4 * width, seed=1))
    dout = dev.buffer(4 * 4 * rows)
    assert not backend.cuda_q8_matmul_device_f32(context, w, dx, 0, dout, 4 * rows).is_ok()
    assert not backend.cuda_q8_matmul_device_f32(context, w, dx, 4, dout, 4 * rows - 1).is_ok()
