"""Host-side mirror of the reference's GGUF module for the parts the Q8_0 path needs
(src/fortai_gguf_runtime.f90: gguf_file_t :89-101, gguf_tensor_t :68-87), over the C ABI of
include/fortai_gguf_b200.h.  Same names, same status codes and messages; indices are
zero-based here where the Fortran module is one-based.
"""
from __future__ import annotations

import ctypes
from ctypes import byref, c_char_p, c_int32, c_int64, c_void_p, create_string_buffer

import numpy as np

from . import abi
from .backend_cuda import FORTAI_INVALID, FORTAI_UNSUPPORTED, cuda_q8_weights_t, status_t

FORTAI_IO_ERROR = 3
GGML_TYPE_F32 = 0
GGML_TYPE_F16 = 1
GGML_TYPE_Q8_0 = 8


class gguf_tensor_t:
    """One entry of the tensor index; `bytes` is a read-only view into the file mapping."""

    def __init__(self, owner, index, name, value_type, shape, file_offset, byte_count):
        self._owner = owner
        self.index = index
        self.name = name
        self.value_type = value_type
        self.shape = shape
        self.file_offset = file_offset
        self.byte_count = byte_count

    @property
    def bytes(self) -> np.ndarray:
        ptr = abi.load().fortai_gguf_tensor_data(self._owner.handle, self.index)
        raw = (ctypes.c_uint8 * self.byte_count).from_address(ptr)
        view = np.frombuffer(raw, dtype=np.uint8)
        view.flags.writeable = False
        return view

    def value(self, index: int) -> float:
        return float(abi.load().fortai_gguf_tensor_value(self._owner.handle, self.index, index))

    def get_row(self, row: int):
        stat = status_t()
        if len(self.shape) != 2:
            stat.set(FORTAI_INVALID, "GGUF tensor is not a matrix")
            return None, stat
        values = np.zeros(self.shape[0], np.float32)
        code = abi.load().fortai_gguf_tensor_get_row(
            self._owner.handle, self.index, row,
            values.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), values.size)
        if code != 0:
            stat.set(FORTAI_INVALID, "GGUF tensor row has the wrong shape")
            return None, stat
        return values, stat

    def upload_q8(self, context, first_row: int = 0, row_count: int = 0):
        """Rows [first_row, first_row + row_count) of a Q8_0 matrix as a weights handle."""
        stat = status_t()
        weights = cuda_q8_weights_t()
        out = c_void_p()
        code = abi.load().fortai_gguf_upload_q8(self._owner.handle, self.index, context.handle,
                                                first_row, row_count, byref(out))
        if code == FORTAI_INVALID:
            stat.set(FORTAI_INVALID, "GGUF tensor is not a Q8_0 matrix or the rows are out of range")
        elif code != 0:
            stat.set(FORTAI_UNSUPPORTED, "CUDA Q8 weight upload failed", context.last_error())
        else:
            rows = self.shape[1] - first_row if row_count == 0 else row_count
            weights.handle = out.value
            weights.rows, weights.width = rows, self.shape[0]
        return weights, stat


class gguf_file_t:
    def __init__(self):
        self.handle = 0
        self.version = 0
        self.tensor_count = 0
        self.metadata_count = 0
        self.data_start = 0
        self.alignment = 32
        self.tensors = []

    def open(self, path: str) -> status_t:
        self.close()
        stat = status_t()
        lib = abi.load()
        out = c_void_p()
        message = create_string_buffer(160)
        code = lib.fortai_gguf_open(path.encode(), byref(out), message, len(message))
        if code != 0:
            stat.set(code, message.value.decode(errors="replace"))
            return stat
        self.handle = out.value
        self.version = lib.fortai_gguf_version(self.handle)
        self.tensor_count = lib.fortai_gguf_tensor_count(self.handle)
        self.metadata_count = lib.fortai_gguf_metadata_count(self.handle)
        self.data_start = lib.fortai_gguf_data_start(self.handle)
        self.alignment = lib.fortai_gguf_alignment(self.handle)
        for i in range(self.tensor_count):
            name, vtype, rank = c_char_p(), c_int32(), c_int32()
            shape = (c_int64 * 4)()
            offset, count = c_int64(), c_int64()
            lib.fortai_gguf_tensor_info(self.handle, i, byref(name), byref(vtype), byref(rank),
                                        shape, byref(offset), byref(count))
            self.tensors.append(gguf_tensor_t(self, i, name.value.decode(), vtype.value,
                                              [int(shape[j]) for j in range(rank.value)],
                                              offset.value, count.value))
        return stat

    def close(self):
        if self.handle:
            abi.load().fortai_gguf_close(self.handle)
        self.__init__()

    def find_meta(self, key: str) -> int:
        return int(abi.load().fortai_gguf_find_meta(self.handle, key.encode())) if self.handle else -1

    def find_tensor(self, name: str) -> int:
        return int(abi.load().fortai_gguf_find_tensor(self.handle, name.encode())) if self.handle else -1

    def meta_keys(self):
        lib = abi.load()
        return [lib.fortai_gguf_meta_key(self.handle, i).decode() for i in range(self.metadata_count)]

    def meta_type(self, key: str) -> int:
        index = self.find_meta(key)
        return int(abi.load().fortai_gguf_meta_type(self.handle, index)) if index >= 0 else -1

    def meta_int(self, key: str, default: int) -> int:
        return int(abi.load().fortai_gguf_meta_int(self.handle, key.encode(), default))

    def meta_real(self, key: str, default: float) -> float:
        return float(abi.load().fortai_gguf_meta_real(self.handle, key.encode(), default))

    def meta_bool(self, key: str, default: bool) -> bool:
        return bool(abi.load().fortai_gguf_meta_bool(self.handle, key.encode(), int(default)))

    def meta_string(self, key: str):
        length = c_int64()
        ptr = abi.load().fortai_gguf_meta_string(self.handle, key.encode(), byref(length))
        return ctypes.string_at(ptr, length.value).decode(errors="replace") if ptr else None

    def meta_int_array(self, key: str):
        lib = abi.load()
        count = lib.fortai_gguf_meta_int_array(self.handle, key.encode(), None, 0)
        if count < 0:
            return None
        values = (c_int64 * max(count, 1))()
        lib.fortai_gguf_meta_int_array(self.handle, key.encode(), values, count)
        return [int(values[i]) for i in range(count)]
