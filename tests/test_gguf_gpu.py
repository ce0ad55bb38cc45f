"""A Q8_0 tensor goes from a GGUF file to the device through the reader's upload call and
gives the same matvec as the oracle on the file's bytes (GPU required)."""
import numpy as np
import pytest

import gguf_writer as gw
from conftest import l2_tolerance
from fortai_b200 import gguf_runtime as rt

pytestmark = pytest.mark.gpu


def test_gguf_tensor_to_matvec_whole_and_row_shard(tmp_path, backend, context, dev, oracle):
    rows, width = 300, 1024
    q8 = oracle.make_weights(rows, width, seed=11)
    path = str(tmp_path / "model.gguf")
    gw.write_gguf(path, [("general.alignment", gw.U32, 64)],
                  [("pad", 0, [3], np.zeros(3, np.float32).tobytes()),
                   ("output.weight", rt.GGML_TYPE_Q8_0, [width, rows], q8.tobytes())], alignment=64)
    f = rt.gguf_file_t()
    assert f.open(path).is_ok()
    tensor = f.tensors[f.find_tensor("output.weight")]
    x = oracle.normal(width, seed=5)
    expected = oracle.matvec(q8, rows, width, x)[0]
    dx = dev.to_device(x)

    weights, stat = tensor.upload_q8(context)
    assert stat.is_ok(), stat
    dout = dev.buffer(4 * rows)
    assert backend.cuda_q8_matvec_device_f32(context, weights, dx, width, dout, rows).is_ok()
    got = dev.floats(dout, rows)
    assert np.abs(got - expected).max() <= l2_tolerance(expected)
    weights.destroy()

    # rows 100..219 only: a row shard is a byte range of the file
    shard, stat = tensor.upload_q8(context, first_row=100, row_count=120)
    assert stat.is_ok(), stat
    assert backend.cuda_q8_matvec_device_f32(context, shard, dx, width, dout, 120).is_ok()
    assert np.array_equal(dev.floats(dout, 120), got[100:220])
    shard.destroy()

    # not a Q8_0 matrix, rows out of range
    assert not f.tensors[0].upload_q8(context)[1].is_ok()
    assert not tensor.upload_q8(context, first_row=rows)[1].is_ok()
    assert not tensor.upload_q8(context, first_row=200, row_count=101)[1].is_ok()
    f.close()
