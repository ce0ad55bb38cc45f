"""Device groups through the C ABI: one host thread, G contexts (GPU required).  With one GPU
the group has one member (the fused all-gather then runs against its own flag word); with
more, the sharded paths run across real devices."""
import numpy as np
import pytest

from conftest import l2_tolerance

pytestmark = pytest.mark.gpu


def group_sizes():
    import torch
    count = torch.cuda.device_count()
    return [g for g in (1, 2, 4, 8) if g <= count]


@pytest.fixture(params=[1, 2, 4, 8])
def group(request, backend):
    import torch
    size = request.param
    if size > torch.cuda.device_count():
        pytest.skip(f"needs {size} GPUs")
    g = backend.cuda_q8_group_t()
    stat = g.create(list(range(size)))
    assert stat.is_ok(), stat
    assert g.device_count() == size
    yield g
    g.destroy()


def test_group_row_sharded_matvec_equals_the_oracle(group, backend, oracle):
    rows, width = 4099, 2560            # a row count that no device count divides
    weights = oracle.make_weights(rows, width, seed=1)
    handle, stat = group.upload(weights, rows, width, 0)
    assert stat.is_ok(), stat
    for seed in (2, 3, 4):              # consecutive calls reuse the flag arrays
        x = oracle.normal(width, seed=seed)
        expected = oracle.matvec(weights, rows, width, x)[0]
        out = np.zeros(rows, np.float32)
        ms, stat = group.matvec_f32(handle, x, out)
        assert stat.is_ok(), stat
        assert ms > 0.0
        assert float(np.abs(out - expected).max()) <= l2_tolerance(expected)
    group.destroy_weights(handle)


def test_group_matvec_is_bit_identical_to_one_device(group, backend, context, dev, oracle):
    rows, width = 2048, 1024
    weights = oracle.make_weights(rows, width, seed=5)
    x = oracle.normal(width, seed=6)
    single = np.zeros(rows, np.float32)
    _, stat = backend.cuda_q8_matvec_host_f32(context, dev.weights(weights, rows, width), x, single)
    assert stat.is_ok(), stat
    handle, stat = group.upload(weights, rows, width, 0)
    assert stat.is_ok(), stat
    out = np.zeros(rows, np.float32)
    _, stat = group.matvec_f32(handle, x, out)
    assert stat.is_ok(), stat
    assert np.array_equal(out, single)
    group.destroy_weights(handle)


def test_group_ffn_equals_the_oracle(group, backend, oracle):
    hidden, inner = 1024, 3840
    gate = oracle.make_weights(inner, hidden, seed=7)
    up = oracle.make_weights(inner, hidden, seed=8)
    down = oracle.make_weights(hidden, inner, seed=9)
    hg, stat = group.upload(gate, inner, hidden, 0)
    assert stat.is_ok(), stat
    hu, stat = group.upload(up, inner, hidden, 0)
    assert stat.is_ok(), stat
    hd, stat = group.upload(down, hidden, inner, 1)
    assert stat.is_ok(), stat
    for seed in (10, 11):
        x = oracle.normal(hidden, seed=seed)
        expected = oracle.ffn(gate, up, down, inner, hidden, hidden, x)
        out = np.zeros(hidden, np.float32)
        _, stat = group.ffn_f32(hg, hu, hd, x, out)
        assert stat.is_ok(), stat
        assert float(np.abs(out - expected).max()) <= 2 * l2_tolerance(expected)
    # shards that do not line up are refused: down uploaded by rows
    wrong, stat = group.upload(down, hidden, inner, 0)
    assert stat.is_ok(), stat
    _, stat = group.ffn_f32(hg, hu, wrong, oracle.normal(hidden, seed=1), np.zeros(hidden, np.float32))
    assert not stat.is_ok()
    for h in (hg, hu, hd, wrong):
        group.destroy_weights(h)


def test_group_argument_validation(backend, oracle):
    g = backend.cuda_q8_group_t()
    assert not g.create([]).is_ok()
    assert not g.create([0, 0]).is_ok()
    assert not g.create([-1]).is_ok()
    assert not g.create([4096]).is_ok()
    assert g.create([0]).is_ok()
    weights = oracle.make_weights(64, 64, seed=1)
    handle, stat = g.upload(weights, 64, 64, 2)
    assert not stat.is_ok() and handle is None
    handle, stat = g.upload(weights, 64, 64, 0)
    assert stat.is_ok(), stat
    short = np.zeros(32, np.float32)
    _, stat = g.matvec_f32(handle, short, np.zeros(64, np.float32))
    assert not stat.is_ok()
    g.destroy_weights(handle)
    g.destroy()
