"""Writes small GGUF v3 files for the reader tests (layout of the GGUF specification:
header, metadata key/value pairs, tensor index, padding to `general.alignment`, data)."""
import struct

import numpy as np

U8, I8, U16, I16, U32, I32, F32, BOOL, STRING, ARRAY, U64, I64, F64 = range(13)
_SCALAR = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", F32: "<f", BOOL: "<B",
           U64: "<Q", I64: "<q", F64: "<d"}


def _string(text) -> bytes:
    raw = text if isinstance(text, bytes) else text.encode()
    return struct.pack("<q", len(raw)) + raw


def _value(kind, value) -> bytes:
    if kind == STRING:
        return _string(value)
    if kind == ARRAY:
        element_kind, items = value
        out = struct.pack("<iq", element_kind, len(items))
        for item in items:
            out += _value(element_kind, item)
        return out
    return struct.pack(_SCALAR[kind], value)


def write_gguf(path, metadata, tensors, alignment=32, version=3, magic=b"GGUF",
               tensor_count=None, metadata_count=None, truncate_to=None):
    """metadata: list of (key, kind, value); tensors: list of (name, ggml_type, shape, bytes),
    shape[0] being the contiguous dimension.  Returns the offset of the data area."""
    head = magic + struct.pack("<iqq", version,
                               len(tensors) if tensor_count is None else tensor_count,
                               len(metadata) if metadata_count is None else metadata_count)
    for key, kind, value in metadata:
        head += _string(key) + struct.pack("<i", kind) + _value(kind, value)
    offsets, cursor = [], 0
    for _, _, _, data in tensors:
        offsets.append(cursor)
        cursor += (len(data) + alignment - 1) // alignment * alignment
    for (name, ggml_type, shape, _), offset in zip(tensors, offsets):
        head += _string(name) + struct.pack("<i", len(shape))
        head += b"".join(struct.pack("<q", d) for d in shape)
        head += struct.pack("<iq", ggml_type, offset)
    data_start = (len(head) + alignment - 1) // alignment * alignment
    blob = head + b"\0" * (data_start - len(head))
    for (_, _, _, data), offset in zip(tensors, offsets):
        blob += b"\0" * (data_start + offset - len(blob)) + bytes(data)
    if truncate_to is not None:
        blob = blob[:truncate_to]
    with open(path, "wb") as handle:
        handle.write(blob)
    return data_start


def half_bits(values) -> bytes:
    return np.asarray(values, dtype=np.float16).tobytes()
