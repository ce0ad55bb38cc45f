"""The recurrent (gated-delta-net) and attention layer objects of the C ABI against the CPU
restatement of the reference's model code (oracle/qwen35_layers_oracle.py).

Tolerance.  Both layers quantize an fp32 intermediate to Q8_0 before their output
projection, and the attention layer also rounds keys and values to binary16.  The fp32
intermediates agree with the CPU's to a few ulps (other sum orders, other exp/sin/cos
implementations); now and then that moves one value across a rounding boundary of the
binary16 cache or of the Q8_0 quantizer.  One flipped quant is one step (1/127 of the
block maximum) on one input of the output projection, so it shows up on EVERY output row
at about 1e-4 of the output scale.  The checks are therefore
    max|gpu - cpu|  <= 2e-3 * max|cpu|     and     ||gpu - cpu||_2 <= 1e-3 * ||cpu||_2,
three orders of magnitude below what a wrong index, head mapping or rotation produces.
"""
import numpy as np
import pytest

from oracle import qwen35_layers_oracle as lo

pytestmark = pytest.mark.gpu


def layer_close(actual, expected):
    scale = float(np.abs(expected).max())
    error = np.abs(actual - expected)
    assert np.isfinite(actual).all()
    assert error.max() <= 2e-3 * scale, (error.max(), scale)
    norm = float(np.linalg.norm(expected.astype(np.float64)))
    assert float(np.linalg.norm(error.astype(np.float64))) <= 1e-3 * norm


RECURRENT_SHAPES = [
    # hidden, key_heads, value_heads, head_size, conv_kernel, steps
    (512, 2, 4, 64, 4, 6),
    (256, 1, 1, 32, 2, 4),
    (2048, 16, 32, 128, 4, 3),
]


def make_recurrent(oracle, backend, context, dev, shape, seed):
    hidden, key_heads, value_heads, head_size, conv_kernel, _ = shape
    state_size = head_size
    conv_size = 2 * state_size * key_heads + value_heads * head_size
    inner = value_heads * head_size
    rng = np.random.default_rng(seed)
    host = dict(qkv=oracle.make_weights(conv_size, hidden, seed=seed + 1, sigma=0.05),
                gate=oracle.make_weights(inner, hidden, seed=seed + 2, sigma=0.05),
                alpha=oracle.make_weights(value_heads, hidden, seed=seed + 3, sigma=0.05),
                beta=oracle.make_weights(value_heads, hidden, seed=seed + 4, sigma=0.05),
                out=oracle.make_weights(hidden, inner, seed=seed + 5, sigma=0.05))
    rows = dict(qkv=conv_size, gate=inner, alpha=value_heads, beta=value_heads, out=hidden)
    width = dict(qkv=hidden, gate=hidden, alpha=hidden, beta=hidden, out=inner)
    device = {name: dev.weights(host[name], rows[name], width[name]) for name in host}
    conv_weights = (rng.standard_normal((conv_size, conv_kernel)) * 0.5).astype(np.float32)
    ssm_a = -np.exp(rng.standard_normal(value_heads)).astype(np.float32)
    ssm_dt = rng.standard_normal(value_heads).astype(np.float32)
    ssm_norm = (1.0 + 0.1 * rng.standard_normal(head_size)).astype(np.float32)
    epsilon = 1e-6
    layer = backend.cuda_qwen35_recurrent_t()
    stat = layer.create(context, device["qkv"], device["gate"], device["alpha"], device["beta"],
                        device["out"], conv_weights, conv_size, conv_kernel, ssm_a, ssm_dt,
                        ssm_norm, state_size, key_heads, value_heads, head_size, inner, epsilon)
    assert stat.is_ok(), stat.message
    cpu = lo.Recurrent(host["qkv"], host["gate"], host["alpha"], host["beta"], host["out"],
                       hidden, conv_weights, conv_kernel, ssm_a, ssm_dt, ssm_norm, state_size,
                       key_heads, value_heads, head_size, np.float32(epsilon))
    return layer, cpu, device


@pytest.mark.parametrize("shape", RECURRENT_SHAPES)
def test_recurrent_steps_match_the_cpu_model(oracle, backend, context, dev, shape):
    hidden, steps = shape[0], shape[-1]
    layer, cpu, _ = make_recurrent(oracle, backend, context, dev, shape, seed=40)
    out_dev = dev.buffer(hidden * 4)
    history = []
    for step in range(steps):
        x = oracle.normal(hidden, seed=900 + step, sigma=1.0)
        history.append(x)
        x_dev = dev.to_device(x)
        assert layer.run_device(x_dev, hidden, out_dev, hidden).is_ok()
        context.synchronize()
        layer_close(dev.floats(out_dev, hidden), cpu.run(x))
    # reset clears both the convolution window and the delta-rule state
    assert layer.reset().is_ok()
    cpu.reset()
    for x in history[:2]:
        assert layer.run_device(dev.to_device(x), hidden, out_dev, hidden).is_ok()
        context.synchronize()
        layer_close(dev.floats(out_dev, hidden), cpu.run(x))
    assert layer.destroy().is_ok()


def test_recurrent_host_run_takes_q8_activation(oracle, backend, context, dev):
    shape = RECURRENT_SHAPES[0]
    hidden = shape[0]
    layer, cpu, _ = make_recurrent(oracle, backend, context, dev, shape, seed=70)
    for step in range(3):
        x = oracle.normal(hidden, seed=300 + step, sigma=1.0)
        q8, _ = oracle.quantize(x)
        out = np.zeros(hidden, np.float32)
        ms, stat = layer.run(q8, q8.nbytes, out, out.nbytes)
        assert stat.is_ok(), stat.message
        assert ms >= 0.0
        layer_close(out, cpu.run(x))
    assert layer.destroy().is_ok()


def test_recurrent_rejects_bad_arguments(oracle, backend, context, dev):
    shape = RECURRENT_SHAPES[1]
    hidden = shape[0]
    layer, _, device = make_recurrent(oracle, backend, context, dev, shape, seed=10)
    out_dev = dev.buffer(hidden * 4)
    x_dev = dev.to_device(oracle.normal(hidden, seed=1, sigma=1.0))
    assert not layer.run_device(x_dev, hidden - 32, out_dev, hidden).is_ok()
    assert not layer.run_device(x_dev, hidden, out_dev, hidden - 1).is_ok()
    assert not layer.run_device(0, hidden, out_dev, hidden).is_ok()
    assert layer.destroy().is_ok()
    # geometry that does not add up is refused at creation
    bad = backend.cuda_qwen35_recurrent_t()
    stat = bad.create(context, device["qkv"], device["gate"], device["alpha"], device["beta"],
                      device["out"], np.zeros(8, np.float32), 96, 2, np.zeros(1, np.float32),
                      np.zeros(1, np.float32), np.zeros(32, np.float32), 32, 1, 1, 32, 32, 1e-6)
    assert not stat.is_ok()


ATTENTION_SHAPES = [
    # hidden, heads, kv_heads, head_size, value_size, max_context, rope_dimension, positions
    (512, 4, 2, 64, 64, 64, 32, 9),
    (256, 2, 2, 32, 32, 16, 0, 4),
    (2048, 16, 4, 256, 256, 300, 64, 5),
]


def make_attention(oracle, backend, context, dev, shape, seed):
    hidden, heads, kv_heads, head_size, value_size, max_context, rope_dimension, _ = shape
    rng = np.random.default_rng(seed)
    rows = dict(q=heads * 2 * head_size, k=kv_heads * head_size, v=kv_heads * value_size,
                out=hidden)
    width = dict(q=hidden, k=hidden, v=hidden, out=heads * value_size)
    host = {name: oracle.make_weights(rows[name], width[name], seed=seed + i, sigma=0.05)
            for i, name in enumerate(rows)}
    device = {name: dev.weights(host[name], rows[name], width[name]) for name in host}
    q_norm = (1.0 + 0.1 * rng.standard_normal(head_size)).astype(np.float32)
    k_norm = (1.0 + 0.1 * rng.standard_normal(head_size)).astype(np.float32)
    rope_base, epsilon = 1.0e7, 1e-6
    layer = backend.cuda_qwen35_attention_t()
    stat = layer.create(context, device["q"], device["k"], device["v"], device["out"], q_norm,
                        k_norm, heads, kv_heads, head_size, value_size, max_context,
                        rope_dimension, rope_base, epsilon)
    assert stat.is_ok(), stat.message
    cpu = lo.Attention(host["q"], host["k"], host["v"], host["out"], hidden, q_norm, k_norm,
                       heads, kv_heads, head_size, value_size, max_context, rope_dimension,
                       np.float32(rope_base), np.float32(epsilon))
    return layer, cpu


@pytest.mark.parametrize("shape", ATTENTION_SHAPES)
def test_attention_positions_match_the_cpu_model(oracle, backend, context, dev, shape):
    hidden, max_context, positions = shape[0], shape[5], shape[-1]
    layer, cpu = make_attention(oracle, backend, context, dev, shape, seed=20)
    out_dev = dev.buffer(hidden * 4)
    for position in range(positions):
        x = oracle.normal(hidden, seed=500 + position, sigma=1.0)
        assert context.set_position(position).is_ok()
        assert layer.run_device(dev.to_device(x), hidden, position, out_dev, hidden).is_ok()
        context.synchronize()
        layer_close(dev.floats(out_dev, hidden), cpu.run(x, position))
    # a position outside the cache is refused on the host, before any launch
    x_dev = dev.to_device(oracle.normal(hidden, seed=1, sigma=1.0))
    assert not layer.run_device(x_dev, hidden, max_context, out_dev, hidden).is_ok()
    assert not layer.run_device(x_dev, hidden, -1, out_dev, hidden).is_ok()
    assert not layer.run_device(x_dev, hidden + 32, 0, out_dev, hidden).is_ok()
    # after a reset position 0 sees only itself again
    assert layer.reset().is_ok()
    cpu.reset()
    x = oracle.normal(hidden, seed=777, sigma=1.0)
    assert context.set_position(0).is_ok()
    assert layer.run_device(dev.to_device(x), hidden, 0, out_dev, hidden).is_ok()
    context.synchronize()
    layer_close(dev.floats(out_dev, hidden), cpu.run(x, 0))
    assert layer.destroy().is_ok()


def test_attention_position_word_outside_the_cache_is_reported_not_used(oracle, backend, context,
                                                                        dev):
    """The kernels read the position from a device word that the host argument only bounds: a
    word outside the caches (a replayed graph, a set_position the caller did not bound) must
    not become an index.  The guarded kernels record a status and skip their work; nothing
    faults, and the next blocking call says what happened."""
    shape = (256, 2, 1, 64, 64, 12, 64, 3)
    hidden, max_context = shape[0], shape[5]
    layer, cpu = make_attention(oracle, backend, context, dev, shape, seed=91)
    out_dev = dev.buffer(hidden * 4)
    x = oracle.normal(hidden, seed=51, sigma=1.0)
    x_dev = dev.to_device(x)
    assert context.set_position(0).is_ok()
    assert layer.run_device(x_dev, hidden, 0, out_dev, hidden).is_ok()
    assert context.synchronize().is_ok()
    layer_close(dev.floats(out_dev, hidden), cpu.run(x, 0))
    # device word beyond the cache, host argument in range
    assert context.set_position(max_context + 5).is_ok()
    assert layer.run_device(x_dev, hidden, 1, out_dev, hidden).is_ok()      # enqueue only
    stat = context.synchronize()
    assert not stat.is_ok()
    assert "attention position outside" in context.last_error()
    # the layer is still usable: position 1 as if the bad call had not happened
    x1 = oracle.normal(hidden, seed=52, sigma=1.0)
    assert context.set_position(1).is_ok()
    assert layer.run_device(dev.to_device(x1), hidden, 1, out_dev, hidden).is_ok()
    assert context.synchronize().is_ok()
    layer_close(dev.floats(out_dev, hidden), cpu.run(x1, 1))
    assert layer.destroy().is_ok()


def test_attention_last_cache_slot(oracle, backend, context, dev):
    """Fill every slot of a small cache; the last position reads all of them."""
    shape = (256, 2, 1, 64, 64, 12, 64, 12)
    hidden = shape[0]
    layer, cpu = make_attention(oracle, backend, context, dev, shape, seed=90)
    out_dev = dev.buffer(hidden * 4)
    for position in range(12):
        x = oracle.normal(hidden, seed=50 + position, sigma=1.0)
        assert context.set_position(position).is_ok()
        assert layer.run_device(dev.to_device(x), hidden, position, out_dev, hidden).is_ok()
        expected = cpu.run(x, position)
    context.synchronize()
    layer_close(dev.floats(out_dev, hidden), expected)
    assert layer.destroy().is_ok()


def test_recurrent_with_the_convolution_as_its_own_kernel(oracle, backend, context, dev):
    """The convolution normally rides in the input projection's epilogue; as a separate
    kernel it gives the same bits."""
    shape = RECURRENT_SHAPES[0]
    hidden = shape[0]
    fused_layer, _, _ = make_recurrent(oracle, backend, context, dev, shape, seed=40)
    out_a, out_b = dev.buffer(hidden * 4), dev.buffer(hidden * 4)
    results = []
    for separate in (0, 1):
        assert context.set_option("gdn_conv_in_gemv", 1 - separate).is_ok()
        layer = fused_layer if separate == 0 else make_recurrent(oracle, backend, context, dev,
                                                                 shape, seed=40)[0]
        outs = []
        for step in range(4):
            x = oracle.normal(hidden, seed=900 + step, sigma=1.0)
            before = context.launch_count()
            assert layer.run_device(dev.to_device(x), hidden, out_a, hidden).is_ok()
            assert context.launch_count() - before == 3 + separate
            context.synchronize()
            outs.append(dev.floats(out_a, hidden))
        results.append(outs)
    for a, b in zip(*results):
        assert np.array_equal(a, b)


def test_attention_over_several_hundred_positions(oracle, backend, context, dev):
    """Longer than the warp count and than one pass of the softmax loops: every warp gets
    many positions in the score and in the value passes."""
    shape = (256, 4, 2, 64, 64, 700, 32, 0)
    hidden = shape[0]
    layer, cpu = make_attention(oracle, backend, context, dev, shape, seed=123)
    out_dev = dev.buffer(hidden * 4)
    for position in range(640):
        x = oracle.normal(hidden, seed=10000 + position, sigma=1.0)
        assert context.set_position(position).is_ok()
        assert layer.run_device(dev.to_device(x), hidden, position, out_dev, hidden).is_ok()
        expected = cpu.run(x, position)
        if position % 127 == 0 or position == 639:
            context.synchronize()
            layer_close(dev.floats(out_dev, hidden), expected)
    assert layer.destroy().is_ok()
