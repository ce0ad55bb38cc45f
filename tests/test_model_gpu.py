"""The device pipeline of the reference's model object (embedding -> layers -> lm_head, all
on the device through the C ABI) against the CPU restatement of the same decode step."""
import numpy as np
import pytest

from oracle import qwen35_model_oracle as mo

pytestmark = pytest.mark.gpu


def make_spec(oracle, **kwargs):
    from fortai_b200.qwen35_device import synthetic_model
    return synthetic_model(lambda rows, width, seed, sigma: oracle.make_weights(rows, width, seed=seed,
                                                                               sigma=sigma), **kwargs)


def close_enough(actual, expected):
    # a model step chains four layers, each of which re-quantizes intermediates (see
    # tests/test_layers_gpu.py for what one flipped quant does): bounds are per step, on logits
    error = np.abs(actual - expected)
    norm = float(np.linalg.norm(expected.astype(np.float64)))
    assert np.isfinite(actual).all()
    assert float(np.linalg.norm(error.astype(np.float64))) <= 5e-3 * norm, \
        float(np.linalg.norm(error.astype(np.float64))) / norm
    assert error.max() <= 1e-2 * float(np.abs(expected).max())


def test_decode_steps_match_the_cpu_model_and_the_graph_replays_them(oracle):
    from fortai_b200.qwen35_device import qwen35_device_model_t
    spec = make_spec(oracle, hidden=256, inner=512, vocabulary=1024, layer_count=4, max_context=16)
    cpu = mo.Model(spec)
    eager, graphed = qwen35_device_model_t(), qwen35_device_model_t()
    assert eager.open(spec).is_ok()
    assert graphed.open(spec, cuda_graph=True).is_ok()
    token = 17
    for position in range(6):
        logits, stat = eager.forward(token, position)
        assert stat.is_ok(), stat
        close_enough(logits, cpu.forward(token, position))
        replayed, stat = graphed.forward(token, position)
        assert stat.is_ok(), stat
        # same kernels, same order: the graph replay gives the same bits as eager launches
        assert np.array_equal(replayed, logits)
        token = int(np.argmax(logits))
    assert graphed.cuda_graph_ready
    # 3 kernels per recurrent layer object, 4 per attention layer object, 2 per FFN (inner
    # sizes up to 4096 are quantized inside the down projection, else 3), 2 norms
    # and 2 adds per layer (the copies are memcpy nodes), embedding + norm + lm_head per step:
    # 40 for this model, where the reference's scheme needs about 17 per layer plus 4
    before = eager.cuda.launch_count()
    eager.forward(token, 6)
    per_step = eager.cuda.launch_count() - before
    assert per_step == 3 * (3 + 2 + 4) + (4 + 2 + 4) + 3, per_step
    # argument checks of qwen35_cpu_forward
    assert not eager.forward(-1, 0)[1].is_ok()
    assert not eager.forward(1024, 0)[1].is_ok()
    assert not eager.forward(0, 16)[1].is_ok()
    # reset: position 0 again gives the first step's logits
    assert eager.reset().is_ok()
    again, stat = eager.forward(17, 0)
    cpu2 = mo.Model(spec)
    close_enough(again, cpu2.forward(17, 0))
    eager.close()
    graphed.close()


def test_fused_residual_steps_match_the_unfused_pipeline(oracle):
    """x <- x + f(rms_norm(x)) inside the GEMVs: same logits as the call-by-call pipeline up
    to the rounding of the norm sum (another summation order in double), fewer launches."""
    from fortai_b200.qwen35_device import qwen35_device_model_t
    spec = make_spec(oracle, hidden=512, inner=1024, vocabulary=2048, layer_count=4, max_context=16)
    cpu = mo.Model(spec)
    plain, fused = qwen35_device_model_t(), qwen35_device_model_t()
    assert plain.open(spec).is_ok()
    assert fused.open(spec, cuda_graph=True, fused=True).is_ok()
    token = 5
    for position in range(5):
        expected, stat = plain.forward(token, position)
        assert stat.is_ok(), stat
        logits, stat = fused.forward(token, position)
        assert stat.is_ok(), stat
        close_enough(logits, cpu.forward(token, position))
        close_enough(logits, expected)
        token = int(np.argmax(expected))
    eager_fused = qwen35_device_model_t()
    assert eager_fused.open(spec, fused=True).is_ok()
    eager_fused.forward(1, 0)
    before = eager_fused.cuda.launch_count()
    eager_fused.forward(1, 1)
    # 3 or 4 kernels per layer object, 2 per FFN, embedding and the output head
    assert eager_fused.cuda.launch_count() - before == 3 * (3 + 2) + (4 + 2) + 2
    # argument checks
    c = eager_fused.cuda
    layer = eager_fused._layers[0]
    from fortai_b200 import backend_cuda as b
    assert not layer["mixer"].step_device(eager_fused.cuda_x, 512 + 32, layer["attn_norm"], 1e-6).is_ok()
    assert not layer["mixer"].step_device(eager_fused.cuda_x, 512, layer["attn_norm"], 0.0).is_ok()
    assert not b.cuda_q8_ffn_step_device(c, layer["ffn_gate"], layer["ffn_up"], layer["ffn_gate"],
                                         eager_fused.cuda_x, 512, layer["post_norm"], 1e-6).is_ok()
    for model in (plain, fused, eager_fused):
        model.close()
