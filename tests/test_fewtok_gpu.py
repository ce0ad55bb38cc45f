"""The few-token product (2..32 tokens, warp-level int8 MMA) against independent oracle
matvecs, through the C ABI (GPU required)."""
import numpy as np
import pytest

from conftest import ffn_error_beyond_quant_flips, l2_tolerance
from test_mmq_gpu import check_rows, exact_dots

pytestmark = pytest.mark.gpu

SHAPES = [
    # tokens, rows, width
    (2, 16, 64),          # one row group, one step
    (3, 130, 192),        # ragged last group, width a multiple of 64 only
    (8, 257, 2560),       # full token tile
    (9, 1000, 1024),      # two token tiles, second almost empty
    (16, 3072, 1024),
    (17, 515, 512),       # four token tiles
    (31, 64, 4096),
    (8, 520, 17408),      # long rows: the activation image is split into K ranges
    (16, 96, 17408),
]


@pytest.mark.parametrize("tokens,rows,width", SHAPES)
def test_few_tokens_match_independent_matvecs(backend, context, dev, oracle, tokens, rows, width):
    blocks = width // 32
    weights = oracle.make_weights(rows, width, seed=rows + tokens)
    x = oracle.normal(tokens * width, seed=width + tokens).reshape(tokens, width)
    expected, quantized, _ = oracle.matmul(weights, rows, width, x)
    w = dev.weights(weights, rows, width)
    dx = dev.to_device(x)
    dout = dev.buffer(4 * tokens * rows)
    launches = context.launch_count()
    assert backend.cuda_q8_matmul_device_f32(context, w, dx, tokens, dout, tokens * rows).is_ok()
    # image + product (the output is zeroed by a memset, not a kernel): not one launch per token
    assert context.launch_count() - launches == 2
    check_rows(dev.floats(dout, tokens * rows).reshape(tokens, rows), expected)
    # pre-quantized activation, twice over the same buffers (stale sums must not survive)
    dq = dev.to_device(quantized)
    for _ in range(2):
        ms, stat = backend.cuda_q8_matmul_resident(context, w, dq, tokens, dout)
        assert stat.is_ok(), stat
        check_rows(dev.floats(dout, tokens * rows).reshape(tokens, rows), expected)
    # exact int32 block dots
    ddots = dev.buffer(4 * tokens * rows * blocks)
    assert backend.cuda_q8_matmul_block_dots_device(context, w, dq, tokens, ddots,
                                                    tokens * rows * blocks).is_ok()
    got = dev.int32s(ddots, tokens * rows * blocks).reshape(tokens, rows, blocks)
    assert np.array_equal(got, exact_dots(weights, quantized, tokens, rows, blocks))


@pytest.mark.parametrize("splits", [1, 2, 5])
def test_k_range_split_option(backend, context, dev, oracle, splits):
    tokens, rows, width = 8, 333, 2560          # 80 blocks: 1, 2 and 5 ranges divide them evenly
    assert context.set_option("fewtok_splits", splits).is_ok()
    weights = oracle.make_weights(rows, width, seed=5)
    x = oracle.normal(tokens * width, seed=6).reshape(tokens, width)
    expected = oracle.matmul(weights, rows, width, x)[0]
    w = dev.weights(weights, rows, width)
    out = np.zeros((tokens, rows), np.float32)
    _, stat = backend.cuda_q8_matmul_host_f32(context, w, x, tokens, out)
    assert stat.is_ok(), stat
    check_rows(out, expected)


def test_widths_the_kernel_does_not_take_fall_back_to_one_matvec_per_token(backend, context, dev,
                                                                           oracle):
    tokens, rows, width = 4, 70, 96             # 3 blocks: not a multiple of 64
    weights = oracle.make_weights(rows, width, seed=8)
    x = oracle.normal(tokens * width, seed=9).reshape(tokens, width)
    expected = oracle.matmul(weights, rows, width, x)[0]
    w = dev.weights(weights, rows, width)
    dx = dev.to_device(x)
    dout = dev.buffer(4 * tokens * rows)
    launches = context.launch_count()
    assert backend.cuda_q8_matmul_device_f32(context, w, dx, tokens, dout, tokens * rows).is_ok()
    assert context.launch_count() - launches == tokens
    check_rows(dev.floats(dout, tokens * rows).reshape(tokens, rows), expected)


def test_few_tokens_agree_with_the_batch1_kernel(backend, context, dev, oracle):
    rows, width, tokens = 2048, 2560, 8
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


@pytest.mark.parametrize("tokens,hidden,inner", [(8, 1024, 3840), (3, 256, 512), (40, 512, 1024),
                                                 (8, 5120, 17408)])   # the last: 27B class, batch 8
def test_batched_ffn_equals_the_single_token_ffn(backend, context, dev, oracle, tokens, hidden,
                                                 inner):
    gate = oracle.make_weights(inner, hidden, seed=1)
    up = oracle.make_weights(inner, hidden, seed=2)
    down = oracle.make_weights(hidden, inner, seed=3)
    x = oracle.normal(tokens * hidden, seed=4).reshape(tokens, hidden)
    wg, wu, wd = dev.weights(gate, inner, hidden), dev.weights(up, inner, hidden), \
        dev.weights(down, hidden, inner)
    dx = dev.to_device(x)
    dout = dev.buffer(4 * tokens * hidden)
    stat = backend.cuda_q8_ffn_batch_device(context, wg, wu, wd, dx, tokens, dout, tokens * hidden)
    assert stat.is_ok(), stat
    got = dev.floats(dout, tokens * hidden).reshape(tokens, hidden)
    flipped = 0
    # (the 27B-class case checks its first and last token: the comparison itself is a
    # 5120 x 17408 float64 projection per token)
    checked = range(tokens) if inner < 10000 else (0, tokens - 1)
    for t in checked:
        expected = oracle.ffn(gate, up, down, inner, hidden, hidden, x[t])
        # the hidden vector is re-quantized between the halves: what is left of the error
        # after removing single-step quant flips must meet the single-token FFN's bound
        count, largest, left = ffn_error_beyond_quant_flips(got[t], expected, oracle, gate, up,
                                                            down, inner, hidden, x[t])
        assert largest <= 1 and left <= 2 * l2_tolerance(expected), (t, count, largest, left)
        flipped += count
    assert flipped <= max(2, len(checked) * inner // 2000), flipped
    # the shape rule of the single-token entry point, and the output size
    assert not backend.cuda_q8_ffn_batch_device(context, wg, wu, wg, dx, tokens, dout,
                                                tokens * hidden).is_ok()
    assert not backend.cuda_q8_ffn_batch_device(context, wg, wu, wd, dx, tokens, dout,
                                                tokens * hidden - 1).is_ok()
