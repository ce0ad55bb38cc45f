"""The GGUF v3 reader (C ABI + its Python mirror) on files written by tests/gguf_writer.py.
Behaviour and messages follow the reference module (src/fortai_gguf_runtime.f90:106-197,
230-349, 739-789)."""
import numpy as np
import pytest

import gguf_writer as gw
from fortai_b200 import gguf_runtime as rt


def q8_matrix(oracle, rows, width, seed):
    return oracle.make_weights(rows, width, seed=seed)


def test_header_metadata_and_tensor_index(tmp_path, oracle):
    rows, width = 6, 64
    q8 = q8_matrix(oracle, rows, width, seed=3)
    f32 = np.arange(12, dtype=np.float32).reshape(3, 4) * 0.5 - 1.0
    f16 = np.array([0.0, 1.0, -2.5, 65504.0, 6.1e-5, 5.96e-8], np.float16)
    metadata = [
        ("general.architecture", gw.STRING, "qwen35"),
        ("a.u8", gw.U8, 200), ("a.i8", gw.I8, -5), ("a.u16", gw.U16, 60000), ("a.i16", gw.I16, -300),
        ("a.u32", gw.U32, 4000000000), ("a.i32", gw.I32, -7), ("a.u64", gw.U64, 1 << 40),
        ("a.i64", gw.I64, -(1 << 40)), ("a.f32", gw.F32, 1.5), ("a.f64", gw.F64, 2.25),
        ("a.flag", gw.BOOL, 1),
        ("a.ints", gw.ARRAY, (gw.I32, [1, -2, 3])), ("a.longs", gw.ARRAY, (gw.U64, [7, 1 << 33])),
        ("a.names", gw.ARRAY, (gw.STRING, ["x", "yy", ""])),     # skipped, as in the reference
        ("a.floats", gw.ARRAY, (gw.F32, [1.0, 2.0])),
    ]
    tensors = [("blk.0.w", rt.GGML_TYPE_Q8_0, [width, rows], q8.tobytes()),
               ("norm", rt.GGML_TYPE_F32, [4, 3], f32.tobytes()),
               ("half", rt.GGML_TYPE_F16, [6], f16.tobytes())]
    path = str(tmp_path / "model.gguf")
    data_start = gw.write_gguf(path, metadata, tensors)

    f = rt.gguf_file_t()
    stat = f.open(path)
    assert stat.is_ok(), stat
    assert (f.version, f.tensor_count, f.metadata_count) == (3, 3, len(metadata))
    assert f.alignment == 32 and f.data_start == data_start
    assert f.meta_keys() == [m[0] for m in metadata]
    assert f.meta_string("general.architecture") == "qwen35"
    assert f.meta_int("a.u8", 0) == 200 and f.meta_int("a.i8", 0) == -5
    assert f.meta_int("a.u16", 0) == 60000 and f.meta_int("a.i16", 0) == -300
    assert f.meta_int("a.u32", 0) == 4000000000 and f.meta_int("a.i32", 0) == -7
    assert f.meta_int("a.u64", 0) == 1 << 40 and f.meta_int("a.i64", 0) == -(1 << 40)
    # meta_int answers only for integer kinds, meta_real only for real kinds
    assert f.meta_int("a.f32", 42) == 42 and f.meta_int("missing", -1) == -1
    assert f.meta_real("a.f32", 0.0) == 1.5 and f.meta_real("a.f64", 0.0) == 2.25
    assert f.meta_real("a.u8", 9.0) == 9.0
    assert f.meta_bool("a.flag", False) is True and f.meta_bool("missing", False) is False
    assert f.meta_int_array("a.ints") == [1, -2, 3]
    assert f.meta_int_array("a.longs") == [7, 1 << 33]
    assert f.meta_int_array("a.names") is None and f.meta_int_array("a.floats") is None
    assert f.meta_type("a.names") == gw.ARRAY
    assert f.find_meta("a.i32") == 6 and f.find_meta("nope") == -1

    assert f.find_tensor("norm") == 1 and f.find_tensor("nope") == -1
    w, n, h = f.tensors
    assert (w.name, w.value_type, w.shape, w.byte_count) == ("blk.0.w", 8, [width, rows], q8.size)
    assert np.array_equal(w.bytes, q8.view(np.uint8))
    assert (n.shape, n.byte_count, h.byte_count) == ([4, 3], 48, 12)
    # element decode: F32, F16 (subnormals included), Q8_0 = scale * quant
    assert [n.value(i) for i in range(12)] == list(f32.reshape(-1))
    assert [h.value(i) for i in range(6)] == [float(v) for v in f16]
    assert n.value(12) == 0.0 and n.value(-1) == 0.0
    for row in range(rows):
        values, stat = w.get_row(row)
        assert stat.is_ok()
        assert np.array_equal(values, oracle.dequantize_row(q8, row, width // 32))
    values, stat = n.get_row(2)
    assert stat.is_ok() and np.array_equal(values, f32[2])
    assert not w.get_row(rows)[1].is_ok() and not h.get_row(0)[1].is_ok()
    f.close()
    assert f.handle == 0 and f.tensors == []


def test_alignment_key_moves_the_data_area(tmp_path):
    data = np.arange(8, dtype=np.float32)
    path = str(tmp_path / "aligned.gguf")
    start = gw.write_gguf(path, [("general.alignment", gw.U32, 256)],
                          [("a", 0, [8], data.tobytes()), ("b", 0, [8], (data * 2).tobytes())],
                          alignment=256)
    f = rt.gguf_file_t()
    assert f.open(path).is_ok()
    assert f.alignment == 256 and f.data_start == start and start % 256 == 0
    assert f.tensors[1].file_offset == 256
    assert [f.tensors[1].value(i) for i in range(8)] == list(data * 2)
    f.close()


def test_half_exponent_31_decodes_to_the_largest_float(tmp_path):
    # the reference's decoder maps infinities and NaNs of binary16 to +-huge(1.0)
    raw = np.array([0x7c00, 0xfc00, 0x7e01], np.uint16)
    path = str(tmp_path / "inf.gguf")
    gw.write_gguf(path, [], [("h", 1, [3], raw.tobytes())])
    f = rt.gguf_file_t()
    assert f.open(path).is_ok()
    big = float(np.finfo(np.float32).max)
    assert [f.tensors[0].value(i) for i in range(3)] == [big, -big, big]
    f.close()


@pytest.mark.parametrize("kwargs,code,text", [
    (dict(magic=b"GGML"), 1, "unsupported or malformed GGUF header"),
    (dict(version=2), 1, "unsupported or malformed GGUF header"),
    (dict(tensor_count=-1), 1, "GGUF counts cannot be negative"),
    (dict(metadata_count=5), 3, "could not read GGUF metadata"),
    (dict(truncate_to=20), 1, "unsupported or malformed GGUF header"),
])
def test_malformed_headers(tmp_path, kwargs, code, text):
    path = str(tmp_path / "bad.gguf")
    # an overstated metadata count runs off the end of a file that has nothing after it
    tensors = [] if "metadata_count" in kwargs else \
        [("t", 0, [4], np.zeros(4, np.float32).tobytes())]
    gw.write_gguf(path, [("k", gw.U32, 1)], tensors, **kwargs)
    stat = rt.gguf_file_t().open(path)
    assert (stat.code, stat.message) == (code, text)


def test_bad_tensor_entries(tmp_path):
    f = rt.gguf_file_t()
    cases = [
        ([("t", 8, [48, 2], b"\0" * 102)], 1, "Q8_0 tensor width is not a multiple of 32"),
        ([("t", 2, [32, 2], b"\0" * 36)], 2, "GGUF tensor quantization is not supported"),
        ([("t", 0, [2, 2, 2, 2, 2], b"\0" * 128)], 1, "invalid GGUF tensor rank"),
        ([("t", 0, [], b"")], 1, "invalid GGUF tensor rank"),
        # shapes whose element or byte count wraps 64 bits must not pass the range check
        ([("t", 8, [32, 2 ** 59 + 1], b"\0" * 68)], 1, "GGUF tensor shape overflows"),
        ([("t", 0, [2 ** 31, 2 ** 31, 2 ** 31, 4], b"\0" * 64)], 1, "GGUF tensor shape overflows"),
        ([("t", 0, [2 ** 61, 2], b"\0" * 64)], 1, "GGUF tensor shape overflows"),
    ]
    for index, (tensors, code, text) in enumerate(cases):
        path = str(tmp_path / f"bad{index}.gguf")
        gw.write_gguf(path, [], tensors)
        stat = f.open(path)
        assert (stat.code, stat.message) == (code, text)
    # data cut short
    path = str(tmp_path / "short.gguf")
    start = gw.write_gguf(path, [], [("t", 0, [64], np.zeros(64, np.float32).tobytes())])
    gw.write_gguf(path, [], [("t", 0, [64], np.zeros(64, np.float32).tobytes())],
                  truncate_to=start + 100)
    stat = f.open(path)
    assert (stat.code, stat.message) == (3, "could not read GGUF tensor data")
    stat = f.open(str(tmp_path / "missing.gguf"))
    assert (stat.code, stat.message) == (3, "could not open GGUF model")
    # an alignment that is no power of two, or absurdly large, is refused
    for index, value in enumerate((48, 2 ** 30)):
        path = str(tmp_path / f"align{index}.gguf")
        gw.write_gguf(path, [("general.alignment", gw.U32, value)],
                      [("t", 0, [4], np.zeros(4, np.float32).tobytes())])
        stat = f.open(path)
        assert (stat.code, stat.message) == (1, "invalid GGUF alignment")


def test_null_handles_are_harmless():
    from fortai_b200 import abi
    lib = abi.load()
    lib.fortai_gguf_close(None)
    assert lib.fortai_gguf_tensor_count(None) == 0
    assert lib.fortai_gguf_find_tensor(None, b"x") == -1
    assert lib.fortai_gguf_tensor_data(None, 0) is None
    assert lib.fortai_gguf_upload_q8(None, 0, None, 0, 0, None) == 1
