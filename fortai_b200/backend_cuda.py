"""Host-side mirror of the reference's Fortran wrapper module `fortai_backend_cuda`
(src/backend/cuda/fortai_backend_cuda.f90) over the C ABI.

The image has no Fortran compiler, so the wrapper's types and free procedures are
restated here with the same names, argument meaning and error behaviour:

* `cuda_q8_context_t`, `cuda_q8_weights_t` hold an opaque handle (`.handle`,
  0 when unassociated), as the Fortran derived types hold a `c_ptr`
  (fortai_backend_cuda.f90:10-33);
* every procedure reports through a `status_t` (src/fortai_status.f90): argument
  problems caught before the C call give `FORTAI_INVALID` with the wrapper's
  message; any non-zero code from the C side collapses to `FORTAI_UNSUPPORTED`
  with the wrapper's fixed message (e.g. fortai_backend_cuda.f90:427-430,
  :775-797).  `status_t.detail` additionally carries `fortai_cuda_q8_last_error`.
* Fortran `intent(out)` arguments become return values: procedures return
  `(outputs..., stat)` or just `stat`.

Host arrays are numpy arrays (int8 for Q8_0 bytes, float32 for vectors); device
buffers are integer addresses, as Fortran holds them in `type(c_ptr)`.
"""
from __future__ import annotations

import ctypes
from ctypes import byref, c_float, c_int, c_void_p

import numpy as np

from . import abi

FORTAI_OK = 0
FORTAI_INVALID = 1
FORTAI_UNSUPPORTED = 2
FORTAI_CUDA_OK = 0

Q8_BLOCK_ELEMS = 32
Q8_BLOCK_BYTES = 34


class status_t:
    """src/fortai_status.f90:13-20"""

    def __init__(self):
        self.code = FORTAI_OK
        self.message = ""
        self.detail = ""

    def clear(self):
        self.code = FORTAI_OK
        self.message = ""
        self.detail = ""

    def is_ok(self) -> bool:
        return self.code == FORTAI_OK

    def set(self, code: int, message: str = "", detail: str = ""):
        self.code = code
        self.message = message
        self.detail = detail

    def __repr__(self):
        return f"status_t(code={self.code}, message={self.message!r}, detail={self.detail!r})"


def _lib():
    return abi.load()


def _host_ptr(array: np.ndarray) -> int:
    # (the plain address: building a ctypes pointer object costs a microsecond more per call)
    return array.ctypes.data


def pointer_array(pointers):
    """A C array of `void *` from a sequence of addresses.  Callers on a hot path build it once
    and pass it in place of the list: the wrappers take either."""
    if isinstance(pointers, ctypes.Array):
        return pointers
    return (c_void_p * len(pointers))(*[int(p) for p in pointers])


def _as_bytes(array) -> np.ndarray:
    a = np.ascontiguousarray(array)
    return a.view(np.int8).reshape(-1)


def _failed(stat: status_t, context, message: str) -> status_t:
    detail = ""
    if context is not None and context.handle:
        raw = _lib().fortai_cuda_q8_last_error(context.handle)
        detail = raw.decode(errors="replace") if raw else ""
    stat.set(FORTAI_UNSUPPORTED, message, detail)
    return stat


class cuda_q8_context_t:
    """fortai_backend_cuda.f90:10-26"""

    def __init__(self):
        self.handle = 0

    # -- lifetime
    def create(self, device: int, stream: int | None = None) -> status_t:
        """`stream` (a cudaStream_t address) is an extension: the context then
        borrows that stream instead of creating its own."""
        stat = status_t()
        if self.handle:
            self.destroy()
        out = c_void_p()
        if stream is None:
            code = _lib().fortai_cuda_q8_context_create(int(device), byref(out))
        else:
            code = _lib().fortai_cuda_q8_context_create_on_stream(int(device), c_void_p(stream),
                                                                 byref(out))
        if code != FORTAI_CUDA_OK:
            self.handle = 0
            stat.set(FORTAI_UNSUPPORTED, "CUDA Q8 context creation failed")
        else:
            self.handle = out.value
        return stat

    def destroy(self) -> status_t:
        stat = status_t()
        if not self.handle:
            return stat
        code = _lib().fortai_cuda_q8_context_destroy(self.handle)
        self.handle = 0
        if code != FORTAI_CUDA_OK:
            stat.set(FORTAI_UNSUPPORTED, "CUDA Q8 context destruction failed")
        return stat

    # -- position / graphs
    def set_position(self, position: int) -> status_t:
        stat = status_t()
        if not self.handle or position < 0:
            stat.set(FORTAI_INVALID, "invalid CUDA device position")
            return stat
        if _lib().fortai_cuda_q8_context_set_position(self.handle, int(position)) != FORTAI_CUDA_OK:
            return _failed(stat, self, "CUDA device position update failed")
        return stat

    def _graph(self, fn, message) -> status_t:
        stat = status_t()
        if not self.handle:
            stat.set(FORTAI_INVALID, "invalid CUDA graph context")
            return stat
        if fn(self.handle) != FORTAI_CUDA_OK:
            return _failed(stat, self, message)
        return stat

    def capture_begin(self) -> status_t:
        return self._graph(_lib().fortai_cuda_q8_context_capture_begin,
                           "CUDA graph capture begin failed")

    def capture_end(self) -> status_t:
        return self._graph(_lib().fortai_cuda_q8_context_capture_end,
                           "CUDA graph capture end failed")

    def graph_launch(self) -> status_t:
        return self._graph(_lib().fortai_cuda_q8_context_graph_launch, "CUDA graph launch failed")

    # -- device buffers
    def allocate_buffer(self, nbytes: int):
        stat = status_t()
        if not self.handle or nbytes <= 0:
            stat.set(FORTAI_INVALID, "invalid CUDA device buffer allocation")
            return 0, stat
        out = c_void_p()
        if _lib().fortai_cuda_q8_device_buffer_create(self.handle, nbytes, byref(out)) != FORTAI_CUDA_OK:
            return 0, _failed(stat, self, "CUDA device buffer allocation failed")
        return out.value, stat

    def free_buffer(self, device_buffer: int) -> status_t:
        stat = status_t()
        if not self.handle or not device_buffer:
            return stat
        if _lib().fortai_cuda_q8_device_buffer_destroy(self.handle, device_buffer) != FORTAI_CUDA_OK:
            return _failed(stat, self, "CUDA device buffer free failed")
        return stat

    def upload(self, device_buffer: int, host_data: np.ndarray, nbytes: int | None = None) -> status_t:
        stat = status_t()
        data = _as_bytes(host_data)
        nbytes = data.size if nbytes is None else nbytes
        if not self.handle or not device_buffer or data.size <= 0 or nbytes <= 0 or nbytes > data.size:
            stat.set(FORTAI_INVALID, "invalid CUDA device upload")
            return stat
        if _lib().fortai_cuda_q8_device_buffer_upload(self.handle, device_buffer, _host_ptr(data),
                                                     nbytes) != FORTAI_CUDA_OK:
            return _failed(stat, self, "CUDA device upload failed")
        return stat

    def upload_real(self, device_buffer: int, host_data: np.ndarray) -> status_t:
        return self.upload(device_buffer, np.ascontiguousarray(host_data, dtype=np.float32))

    def download(self, device_buffer: int, nbytes: int):
        stat = status_t()
        out = np.zeros(max(nbytes, 0), dtype=np.int8)
        if not self.handle or not device_buffer or nbytes <= 0:
            stat.set(FORTAI_INVALID, "invalid CUDA device download")
            return out, stat
        if _lib().fortai_cuda_q8_device_buffer_download(self.handle, _host_ptr(out), device_buffer,
                                                       nbytes) != FORTAI_CUDA_OK:
            return out, _failed(stat, self, "CUDA device download failed")
        return out, stat

    def download_real(self, device_buffer: int, elements: int):
        raw, stat = self.download(device_buffer, elements * 4)
        return raw.view(np.float32), stat

    def last_error(self) -> str:
        raw = _lib().fortai_cuda_q8_last_error(self.handle if self.handle else None)
        return raw.decode(errors="replace") if raw else ""

    # -- extensions
    def stream(self) -> int:
        return int(_lib().fortai_cuda_q8_context_stream(self.handle) or 0)

    def launch_count(self) -> int:
        return int(_lib().fortai_cuda_q8_context_launch_count(self.handle))

    def synchronize(self) -> status_t:
        stat = status_t()
        if not self.handle:
            stat.set(FORTAI_INVALID, "invalid CUDA Q8 context")
            return stat
        if _lib().fortai_cuda_q8_context_synchronize(self.handle) != FORTAI_CUDA_OK:
            return _failed(stat, self, "CUDA synchronize failed")
        return stat

    def set_option(self, name: str, value: int) -> status_t:
        stat = status_t()
        if not self.handle or _lib().fortai_cuda_q8_context_set_option(
                self.handle, name.encode(), int(value)) != FORTAI_CUDA_OK:
            stat.set(FORTAI_INVALID, "invalid CUDA Q8 option")
        return stat


class cuda_q8_weights_t:
    """fortai_backend_cuda.f90:28-33"""

    def __init__(self):
        self.handle = 0
        self.rows = 0
        self.width = 0

    def upload(self, context: cuda_q8_context_t, host_weights: np.ndarray, weight_bytes: int,
               rows: int, width: int) -> status_t:
        stat = status_t()
        data = _as_bytes(host_weights)
        if not context.handle or data.size <= 0 or rows <= 0 or width <= 0:
            stat.set(FORTAI_INVALID, "invalid CUDA Q8 weight upload")
            return stat
        if self.handle:
            self.destroy()
        out = c_void_p()
        code = _lib().fortai_cuda_q8_weights_upload(context.handle, _host_ptr(data), weight_bytes,
                                                    int(rows), int(width), byref(out))
        if code != FORTAI_CUDA_OK:
            self.handle = 0
            return _failed(stat, context, "CUDA Q8 weight upload failed")
        self.handle, self.rows, self.width = out.value, rows, width
        return stat

    def upload_columns(self, context: cuda_q8_context_t, host_weights: np.ndarray, rows: int,
                       width: int, first_block: int, block_count: int) -> status_t:
        """Extension: keep only a K-slice of every row (column-sharded projections)."""
        stat = status_t()
        data = _as_bytes(host_weights)
        if not context.handle or data.size <= 0 or rows <= 0 or width <= 0:
            stat.set(FORTAI_INVALID, "invalid CUDA Q8 weight upload")
            return stat
        if self.handle:
            self.destroy()
        out = c_void_p()
        code = _lib().fortai_cuda_q8_weights_upload_columns(
            context.handle, _host_ptr(data), data.size, int(rows), int(width), int(first_block),
            int(block_count), byref(out))
        if code != FORTAI_CUDA_OK:
            self.handle = 0
            return _failed(stat, context, "CUDA Q8 weight upload failed")
        self.handle, self.rows, self.width = out.value, rows, block_count * Q8_BLOCK_ELEMS
        return stat

    def destroy(self) -> status_t:
        stat = status_t()
        if not self.handle:
            return stat
        code = _lib().fortai_cuda_q8_weights_destroy(self.handle)
        self.handle = 0
        if code != FORTAI_CUDA_OK:
            stat.set(FORTAI_UNSUPPORTED, "CUDA Q8 weight destruction failed")
        return stat


def _f32_out(elements: int) -> np.ndarray:
    return np.zeros(max(int(elements), 0), dtype=np.float32)


# --------------------------------------------------------------------------- host calls
def cuda_q8_matvec_host(context, weights, activation, activation_bytes, output, output_bytes):
    """fortai_backend_cuda.f90:775-797.  Returns (elapsed_ms, stat); `output` is filled."""
    stat = status_t()
    act = _as_bytes(activation)
    if not context.handle or not weights.handle or act.size <= 0 or output.size <= 0:
        stat.set(FORTAI_INVALID, "invalid CUDA Q8 host matvec")
        return 0.0, stat
    ms = c_float(0.0)
    code = _lib().fortai_cuda_q8_matvec_host(context.handle, weights.handle, _host_ptr(act),
                                             activation_bytes, _host_ptr(output), output_bytes,
                                             byref(ms))
    if code != FORTAI_CUDA_OK:
        return 0.0, _failed(stat, context, "CUDA Q8 host matvec failed")
    return ms.value, stat


def cuda_q8_matvec_host_pair(context, first_weights, second_weights, activation, activation_bytes,
                             first_output, first_output_bytes, second_output, second_output_bytes):
    """fortai_backend_cuda.f90:799-825"""
    stat = status_t()
    act = _as_bytes(activation)
    if (not context.handle or not first_weights.handle or not second_weights.handle or
            act.size <= 0 or first_output.size <= 0 or second_output.size <= 0):
        stat.set(FORTAI_INVALID, "invalid CUDA Q8 host matvec pair")
        return 0.0, stat
    ms = c_float(0.0)
    code = _lib().fortai_cuda_q8_matvec_host_pair(
        context.handle, first_weights.handle, second_weights.handle, _host_ptr(act),
        activation_bytes, _host_ptr(first_output), first_output_bytes, _host_ptr(second_output),
        second_output_bytes, byref(ms))
    if code != FORTAI_CUDA_OK:
        return 0.0, _failed(stat, context, "CUDA Q8 host matvec pair failed")
    return ms.value, stat


def cuda_q8_matvec_host_triplet(context, first_weights, second_weights, third_weights, activation,
                                activation_bytes, first_output, first_output_bytes, second_output,
                                second_output_bytes, third_output, third_output_bytes):
    """fortai_backend_cuda.f90:827-858"""
    stat = status_t()
    act = _as_bytes(activation)
    if (not context.handle or not first_weights.handle or not second_weights.handle or
            not third_weights.handle or act.size <= 0 or first_output.size <= 0 or
            second_output.size <= 0 or third_output.size <= 0):
        stat.set(FORTAI_INVALID, "invalid CUDA Q8 host matvec triplet")
        return 0.0, stat
    ms = c_float(0.0)
    code = _lib().fortai_cuda_q8_matvec_host_triplet(
        context.handle, first_weights.handle, second_weights.handle, third_weights.handle,
        _host_ptr(act), activation_bytes, _host_ptr(first_output), first_output_bytes,
        _host_ptr(second_output), second_output_bytes, _host_ptr(third_output),
        third_output_bytes, byref(ms))
    if code != FORTAI_CUDA_OK:
        return 0.0, _failed(stat, context, "CUDA Q8 host matvec triplet failed")
    return ms.value, stat


def cuda_q8_matvec_host_triplet_contiguous(context, first_weights, second_weights, third_weights,
                                           activation, activation_bytes, output, output_bytes):
    """fortai_backend_cuda.f90:860-888"""
    stat = status_t()
    act = _as_bytes(activation)
    if (not context.handle or not first_weights.handle or not second_weights.handle or
            not third_weights.handle or act.size <= 0 or output.size <= 0):
        stat.set(FORTAI_INVALID, "invalid CUDA Q8 host matvec triplet")
        return 0.0, stat
    ms = c_float(0.0)
    code = _lib().fortai_cuda_q8_matvec_host_triplet_contiguous(
        context.handle, first_weights.handle, second_weights.handle, third_weights.handle,
        _host_ptr(act), activation_bytes, _host_ptr(output), output_bytes, byref(ms))
    if code != FORTAI_CUDA_OK:
        return 0.0, _failed(stat, context, "CUDA Q8 host matvec triplet failed")
    return ms.value, stat


def cuda_q8_ffn_host(context, gate_weights, up_weights, down_weights, activation, activation_bytes,
                     output, output_bytes):
    """fortai_backend_cuda.f90:890-918"""
    stat = status_t()
    act = _as_bytes(activation)
    if (not context.handle or not gate_weights.handle or not up_weights.handle or
            not down_weights.handle or act.size <= 0 or output.size <= 0):
        stat.set(FORTAI_INVALID, "invalid CUDA Q8 FFN")
        return 0.0, stat
    ms = c_float(0.0)
    code = _lib().fortai_cuda_q8_ffn_host(context.handle, gate_weights.handle, up_weights.handle,
                                          down_weights.handle, _host_ptr(act), activation_bytes,
                                          _host_ptr(output), output_bytes, byref(ms))
    if code != FORTAI_CUDA_OK:
        return 0.0, _failed(stat, context, "CUDA Q8 FFN failed")
    return ms.value, stat


# --------------------------------------------------------------------------- device calls
def cuda_q8_ffn_device(context, gate_weights, up_weights, down_weights, device_activation,
                       activation_elements, device_output, output_elements) -> status_t:
    """fortai_backend_cuda.f90:920-946"""
    stat = status_t()
    if (not context.handle or not gate_weights.handle or not up_weights.handle or
            not down_weights.handle or not device_activation or not device_output or
            activation_elements <= 0 or output_elements <= 0):
        stat.set(FORTAI_INVALID, "invalid CUDA Q8 device FFN")
        return stat
    code = _lib().fortai_cuda_q8_ffn_device(context.handle, gate_weights.handle, up_weights.handle,
                                            down_weights.handle, device_activation,
                                            activation_elements, device_output, output_elements)
    if code != FORTAI_CUDA_OK:
        return _failed(stat, context, "CUDA Q8 device FFN failed")
    return stat


def cuda_q8_matvec_resident(context, weights, device_activation, device_output):
    """fortai_backend_cuda.f90:1014-1036.  Returns (kernel_ms, stat)."""
    stat = status_t()
    if not context.handle or not weights.handle or not device_activation or not device_output:
        stat.set(FORTAI_INVALID, "invalid CUDA Q8 resident matvec")
        return 0.0, stat
    ms = c_float(0.0)
    code = _lib().fortai_cuda_q8_matvec_resident(context.handle, weights.handle, device_activation,
                                                 device_output, byref(ms))
    if code != FORTAI_CUDA_OK:
        return 0.0, _failed(stat, context, "CUDA Q8 resident matvec failed")
    return ms.value, stat


def cuda_q8_matvec_device_q8(context, weights, device_activation, device_output,
                             output_elements) -> status_t:
    """The resident matvec as an enqueue-only call (pre-quantized device activation)."""
    stat = status_t()
    if (not context.handle or not weights.handle or not device_activation or not device_output or
            output_elements <= 0):
        stat.set(FORTAI_INVALID, "invalid CUDA Q8 device matvec")
        return stat
    code = _lib().fortai_cuda_q8_matvec_device_q8(context.handle, weights.handle,
                                                  device_activation, device_output,
                                                  output_elements)
    if code != FORTAI_CUDA_OK:
        return _failed(stat, context, "CUDA Q8 device matvec failed")
    return stat


def cuda_q8_matvec_device_f32(context, weights, device_activation, activation_elements,
                              device_output, output_elements) -> status_t:
    """fortai_backend_cuda.f90:1038-1062"""
    stat = status_t()
    if (not context.handle or not weights.handle or not device_activation or not device_output or
            activation_elements <= 0 or output_elements <= 0):
        stat.set(FORTAI_INVALID, "invalid CUDA Q8 device F32 matvec")
        return stat
    code = _lib().fortai_cuda_q8_matvec_device_f32(context.handle, weights.handle,
                                                   device_activation, activation_elements,
                                                   device_output, output_elements)
    if code != FORTAI_CUDA_OK:
        return _failed(stat, context, "CUDA Q8 device F32 matvec failed")
    return stat


def cuda_qwen35_embedding_device(context, weights, token_id, device_output, output_elements):
    """fortai_backend_cuda.f90:1064-1086"""
    stat = status_t()
    if not context.handle or not weights.handle or not device_output or output_elements <= 0:
        stat.set(FORTAI_INVALID, "invalid CUDA device embedding")
        return stat
    code = _lib().fortai_cuda_qwen35_embedding_device(context.handle, weights.handle,
                                                      int(token_id), device_output,
                                                      output_elements)
    if code != FORTAI_CUDA_OK:
        return _failed(stat, context, "CUDA device embedding failed")
    return stat


def cuda_qwen35_copy_device(context, device_input, device_output, nbytes) -> status_t:
    """fortai_backend_cuda.f90:720-738"""
    stat = status_t()
    if not context.handle or not device_input or not device_output or nbytes <= 0:
        stat.set(FORTAI_INVALID, "invalid CUDA device copy")
        return stat
    if _lib().fortai_cuda_qwen35_copy_device(context.handle, device_input, device_output,
                                             nbytes) != FORTAI_CUDA_OK:
        return _failed(stat, context, "CUDA device copy failed")
    return stat


def cuda_qwen35_add_device(context, device_left, device_right, device_output, elements) -> status_t:
    """fortai_backend_cuda.f90:740-758"""
    stat = status_t()
    if (not context.handle or not device_left or not device_right or not device_output or
            elements <= 0):
        stat.set(FORTAI_INVALID, "invalid CUDA device add")
        return stat
    if _lib().fortai_cuda_qwen35_add_device(context.handle, device_left, device_right,
                                            device_output, elements) != FORTAI_CUDA_OK:
        return _failed(stat, context, "CUDA device add failed")
    return stat


def cuda_qwen35_rms_norm_device(context, device_input, device_weights, device_output, elements,
                                epsilon) -> status_t:
    """fortai_backend_cuda.f90:760-773"""
    stat = status_t()
    if (not context.handle or not device_input or not device_weights or not device_output or
            elements <= 0 or epsilon <= 0.0):
        stat.set(FORTAI_INVALID, "invalid CUDA device RMS norm")
        return stat
    if _lib().fortai_cuda_qwen35_rms_norm_device(context.handle, device_input, device_weights,
                                                 device_output, elements,
                                                 c_float(epsilon)) != FORTAI_CUDA_OK:
        return _failed(stat, context, "CUDA device RMS norm failed")
    return stat


# --------------------------------------------------------------------------- extensions
def cuda_q8_quantize_device(context, device_input, elements, device_output, output_bytes) -> status_t:
    stat = status_t()
    if not context.handle or not device_input or not device_output or elements <= 0:
        stat.set(FORTAI_INVALID, "invalid CUDA Q8 device quantize")
        return stat
    if _lib().fortai_cuda_q8_quantize_device(context.handle, device_input, elements, device_output,
                                             output_bytes) != FORTAI_CUDA_OK:
        return _failed(stat, context, "CUDA Q8 device quantize failed")
    return stat


def cuda_q8_block_dots_device(context, weights, device_activation, device_output,
                              output_elements) -> status_t:
    stat = status_t()
    if not context.handle or not weights.handle or not device_activation or not device_output:
        stat.set(FORTAI_INVALID, "invalid CUDA Q8 block dots")
        return stat
    if _lib().fortai_cuda_q8_block_dots_device(context.handle, weights.handle, device_activation,
                                               device_output, output_elements) != FORTAI_CUDA_OK:
        return _failed(stat, context, "CUDA Q8 block dots failed")
    return stat


def cuda_q8_matvec_host_f32(context, weights, activation, output):
    """Host fp32 vector in, host fp32 vector out.  Returns (elapsed_ms, stat)."""
    stat = status_t()
    if (not context.handle or not weights.handle or activation.size <= 0 or output.size <= 0 or
            activation.dtype != np.float32 or output.dtype != np.float32):
        stat.set(FORTAI_INVALID, "invalid CUDA Q8 host F32 matvec")
        return 0.0, stat
    ms = c_float(0.0)
    code = _lib().fortai_cuda_q8_matvec_host_f32(context.handle, weights.handle,
                                                 _host_ptr(activation), activation.size,
                                                 _host_ptr(output), output.nbytes, byref(ms))
    if code != FORTAI_CUDA_OK:
        return 0.0, _failed(stat, context, "CUDA Q8 host F32 matvec failed")
    return ms.value, stat


def cuda_q8_matmul_device_f32(context, weights, device_activation, tokens, device_output,
                              output_elements) -> status_t:
    stat = status_t()
    if (not context.handle or not weights.handle or not device_activation or not device_output or
            tokens <= 0):
        stat.set(FORTAI_INVALID, "invalid CUDA Q8 device matmul")
        return stat
    if _lib().fortai_cuda_q8_matmul_device_f32(context.handle, weights.handle, device_activation,
                                               int(tokens), device_output,
                                               output_elements) != FORTAI_CUDA_OK:
        return _failed(stat, context, "CUDA Q8 device matmul failed")
    return stat


def cuda_q8_matmul_resident(context, weights, device_activation, tokens, device_output):
    stat = status_t()
    if (not context.handle or not weights.handle or not device_activation or not device_output or
            tokens <= 0):
        stat.set(FORTAI_INVALID, "invalid CUDA Q8 resident matmul")
        return 0.0, stat
    ms = c_float(0.0)
    code = _lib().fortai_cuda_q8_matmul_resident(context.handle, weights.handle, device_activation,
                                                 int(tokens), device_output, byref(ms))
    if code != FORTAI_CUDA_OK:
        return 0.0, _failed(stat, context, "CUDA Q8 resident matmul failed")
    return ms.value, stat


def cuda_q8_matmul_host_f32(context, weights, activation, tokens, output):
    stat = status_t()
    if (not context.handle or not weights.handle or activation.size <= 0 or output.size <= 0 or
            tokens <= 0 or activation.dtype != np.float32 or output.dtype != np.float32):
        stat.set(FORTAI_INVALID, "invalid CUDA Q8 host matmul")
        return 0.0, stat
    ms = c_float(0.0)
    code = _lib().fortai_cuda_q8_matmul_host_f32(context.handle, weights.handle,
                                                 _host_ptr(activation), int(tokens),
                                                 _host_ptr(output), output.nbytes, byref(ms))
    if code != FORTAI_CUDA_OK:
        return 0.0, _failed(stat, context, "CUDA Q8 host matmul failed")
    return ms.value, stat


def cuda_tensor_peak(context, kind: int, iterations: int = 4000):
    """Measured tensor-core peak (bare tcgen05.mma loop on every SM): kind 0 = int8 TOPS,
    1 = binary16 TFLOPS.  Returns (tera-ops per second, elapsed ms, status)."""
    stat = status_t()
    if not context.handle or kind not in (0, 1) or iterations < 2:
        stat.set(FORTAI_INVALID, "invalid CUDA tensor peak probe")
        return 0.0, 0.0, stat
    tops, ms = c_float(0.0), c_float(0.0)
    code = _lib().fortai_cuda_tensor_peak(context.handle, int(kind), int(iterations), byref(tops),
                                          byref(ms))
    if code != FORTAI_CUDA_OK:
        return 0.0, 0.0, _failed(stat, context, "CUDA tensor peak probe failed")
    return tops.value, ms.value, stat


def cuda_q8_matmul_block_dots_device(context, weights, device_activation, tokens, device_output,
                                     output_elements) -> status_t:
    stat = status_t()
    if (not context.handle or not weights.handle or not device_activation or not device_output or
            tokens <= 0):
        stat.set(FORTAI_INVALID, "invalid CUDA Q8 matmul block dots")
        return stat
    if _lib().fortai_cuda_q8_matmul_block_dots_device(
            context.handle, weights.handle, device_activation, int(tokens), device_output,
            output_elements) != FORTAI_CUDA_OK:
        return _failed(stat, context, "CUDA Q8 matmul block dots failed")
    return stat


def cuda_q8_ffn_batch_device(context, gate_weights, up_weights, down_weights, device_activation,
                             tokens, device_output, output_elements) -> status_t:
    """Extension: the FFN of `tokens` activations in one call (token-major fp32)."""
    stat = status_t()
    if (not context.handle or not gate_weights.handle or not up_weights.handle
            or not down_weights.handle or not device_activation or not device_output
            or tokens <= 0):
        stat.set(FORTAI_INVALID, "invalid CUDA Q8 batched FFN")
        return stat
    code = _lib().fortai_cuda_q8_ffn_batch_device(context.handle, gate_weights.handle,
                                                  up_weights.handle, down_weights.handle,
                                                  device_activation, int(tokens), device_output,
                                                  output_elements)
    if code != FORTAI_CUDA_OK:
        return _failed(stat, context, "CUDA Q8 batched FFN failed")
    return stat


def cuda_q8_ffn_step_device(context, gate_weights, up_weights, down_weights, device_x, elements,
                            device_norm_weights, epsilon) -> status_t:
    """Extension: x <- x + FFN(rms_norm(x) * norm_weights), in place on the residual stream."""
    stat = status_t()
    if (not context.handle or not gate_weights.handle or not up_weights.handle
            or not down_weights.handle or not device_x or not device_norm_weights):
        stat.set(FORTAI_INVALID, "invalid CUDA Q8 FFN step")
        return stat
    code = _lib().fortai_cuda_q8_ffn_step_device(context.handle, gate_weights.handle,
                                                 up_weights.handle, down_weights.handle, device_x,
                                                 elements, device_norm_weights, c_float(epsilon))
    if code != FORTAI_CUDA_OK:
        return _failed(stat, context, "CUDA Q8 FFN step failed")
    return stat


def cuda_q8_matvec_norm_device_f32(context, weights, device_x, elements, device_norm_weights,
                                   epsilon, device_output, output_elements) -> status_t:
    """Extension: output = weights . Q8(rms_norm(x) * norm_weights) in one launch."""
    stat = status_t()
    if not context.handle or not weights.handle or not device_x or not device_output:
        stat.set(FORTAI_INVALID, "invalid CUDA Q8 normalised matvec")
        return stat
    code = _lib().fortai_cuda_q8_matvec_norm_device_f32(context.handle, weights.handle, device_x,
                                                        elements, device_norm_weights,
                                                        c_float(epsilon), device_output,
                                                        output_elements)
    if code != FORTAI_CUDA_OK:
        return _failed(stat, context, "CUDA Q8 normalised matvec failed")
    return stat


def cuda_q8_matvec_device_f32_peers(context, weights, device_activation, activation_elements,
                                    peer_outputs, first_row, output_elements) -> status_t:
    stat = status_t()
    if (not context.handle or not weights.handle or not device_activation or not peer_outputs):
        stat.set(FORTAI_INVALID, "invalid CUDA Q8 peer matvec")
        return stat
    array = pointer_array(peer_outputs)
    code = _lib().fortai_cuda_q8_matvec_device_f32_peers(
        context.handle, weights.handle, device_activation, activation_elements, array,
        len(peer_outputs), int(first_row), int(output_elements))
    if code != FORTAI_CUDA_OK:
        return _failed(stat, context, "CUDA Q8 peer matvec failed")
    return stat


def cuda_q8_matvec_device_f32_allgather(context, weights, device_activation, activation_elements,
                                        peer_outputs, peer_flags, my_rank, first_row,
                                        output_elements) -> status_t:
    """Row shard + all-gather in one kernel (flag words in every rank's memory)."""
    stat = status_t()
    if (not context.handle or not weights.handle or not device_activation or not peer_outputs or
            len(peer_outputs) != len(peer_flags)):
        stat.set(FORTAI_INVALID, "invalid CUDA Q8 all-gather matvec")
        return stat
    outs = pointer_array(peer_outputs)
    flags = pointer_array(peer_flags)
    code = _lib().fortai_cuda_q8_matvec_device_f32_allgather(
        context.handle, weights.handle, device_activation, activation_elements, outs, flags,
        len(peer_outputs), int(my_rank), int(first_row), int(output_elements))
    if code != FORTAI_CUDA_OK:
        return _failed(stat, context, "CUDA Q8 all-gather matvec failed")
    return stat


def cuda_q8_matvec_device_f32_allgather_ll(context, weights, device_activation,
                                           activation_elements, peer_pairs, my_rank, first_row,
                                           device_output, output_elements) -> status_t:
    """Row shard + all-gather in one kernel, the data carrying its own flag: results travel as
    (value, call number) pairs into every rank's pair array and are collected into
    `device_output` (output_elements floats on this rank)."""
    stat = status_t()
    if (not context.handle or not weights.handle or not device_activation or not peer_pairs or
            not device_output):
        stat.set(FORTAI_INVALID, "invalid CUDA Q8 all-gather matvec (pairs)")
        return stat
    pairs = pointer_array(peer_pairs)
    code = _lib().fortai_cuda_q8_matvec_device_f32_allgather_ll(
        context.handle, weights.handle, device_activation, activation_elements, pairs,
        len(peer_pairs), int(my_rank), int(first_row), device_output, int(output_elements))
    if code != FORTAI_CUDA_OK:
        return _failed(stat, context, "CUDA Q8 all-gather matvec (pairs) failed")
    return stat


def cuda_q8_ffn_device_allreduce(context, gate, up, down, device_activation, activation_elements,
                                 peer_pairs, my_rank, device_output, output_elements) -> status_t:
    """Sharded FFN with the sum over ranks inside the call: the down GEMV stores this rank's
    partial vector as (value, call number) pairs into every rank's pair array and adds the
    slots in rank order as they arrive.  peer_pairs[p]: 2 * world * hidden pairs of 8 bytes in
    rank p's memory, zeroed once."""
    stat = status_t()
    if (not context.handle or not gate.handle or not up.handle or not down.handle or
            not device_activation or not device_output or not peer_pairs):
        stat.set(FORTAI_INVALID, "invalid CUDA Q8 all-reduce FFN")
        return stat
    pairs = pointer_array(peer_pairs)
    code = _lib().fortai_cuda_q8_ffn_device_allreduce(
        context.handle, gate.handle, up.handle, down.handle, device_activation,
        int(activation_elements), pairs, len(peer_pairs), int(my_rank), device_output,
        int(output_elements))
    if code != FORTAI_CUDA_OK:
        return _failed(stat, context, "CUDA Q8 all-reduce FFN failed")
    return stat


# --------------------------------------------------------------------------- layer objects
class cuda_qwen35_recurrent_t:
    """fortai_backend_cuda.f90:35-43 (gated-delta-net layer; state lives on the device)."""

    def __init__(self):
        self.handle = 0
        self.context = None

    def create(self, context, qkv, gate, alpha, beta, output, conv_weights, conv_size,
               conv_kernel, ssm_a, ssm_dt, ssm_norm, state_size, key_heads, value_heads,
               head_size, inner_size, norm_epsilon) -> status_t:
        stat = status_t()
        handles = (qkv, gate, alpha, beta, output)
        if not context.handle or any(not w.handle for w in handles):
            stat.set(FORTAI_INVALID, "invalid CUDA Qwen recurrent layer")
            return stat
        arrays = [np.ascontiguousarray(a, dtype=np.float32)
                  for a in (conv_weights, ssm_a, ssm_dt, ssm_norm)]
        out = c_void_p()
        code = _lib().fortai_cuda_qwen35_recurrent_create(
            context.handle, qkv.handle, gate.handle, alpha.handle, beta.handle, output.handle,
            _host_ptr(arrays[0]), arrays[0].nbytes, int(conv_size), int(conv_kernel),
            _host_ptr(arrays[1]), arrays[1].nbytes, _host_ptr(arrays[2]), arrays[2].nbytes,
            _host_ptr(arrays[3]), arrays[3].nbytes, int(state_size), int(key_heads),
            int(value_heads), int(head_size), int(inner_size), c_float(norm_epsilon), byref(out))
        if code != FORTAI_CUDA_OK:
            return _failed(stat, context, "CUDA Qwen recurrent layer creation failed")
        self.handle, self.context = out.value, context
        return stat

    def destroy(self) -> status_t:
        stat = status_t()
        if self.handle:
            _lib().fortai_cuda_qwen35_recurrent_destroy(self.handle)
            self.handle = 0
        return stat

    def reset(self) -> status_t:
        stat = status_t()
        if not self.handle:
            stat.set(FORTAI_INVALID, "invalid CUDA Qwen recurrent layer")
        elif _lib().fortai_cuda_qwen35_recurrent_reset(self.handle) != FORTAI_CUDA_OK:
            return _failed(stat, self.context, "CUDA Qwen recurrent reset failed")
        return stat

    def run(self, activation, activation_bytes, output, output_bytes):
        stat = status_t()
        act = _as_bytes(activation)
        if not self.handle or act.size <= 0 or output.size <= 0:
            stat.set(FORTAI_INVALID, "invalid CUDA Qwen recurrent run")
            return 0.0, stat
        ms = c_float(0.0)
        code = _lib().fortai_cuda_qwen35_recurrent_run(self.handle, _host_ptr(act),
                                                       activation_bytes, _host_ptr(output),
                                                       output_bytes, byref(ms))
        if code != FORTAI_CUDA_OK:
            return 0.0, _failed(stat, self.context, "CUDA Qwen recurrent run failed")
        return ms.value, stat

    def run_device(self, device_activation, activation_elements, device_output,
                   output_elements) -> status_t:
        stat = status_t()
        if not self.handle or not device_activation or not device_output:
            stat.set(FORTAI_INVALID, "invalid CUDA Qwen recurrent device run")
            return stat
        code = _lib().fortai_cuda_qwen35_recurrent_run_device(
            self.handle, device_activation, activation_elements, device_output, output_elements)
        if code != FORTAI_CUDA_OK:
            return _failed(stat, self.context, "CUDA Qwen recurrent device run failed")
        return stat


def _step(self, call, message, *args) -> status_t:
    stat = status_t()
    if not self.handle or not args[0]:
        stat.set(FORTAI_INVALID, "invalid " + message)
        return stat
    if call(self.handle, *args) != FORTAI_CUDA_OK:
        return _failed(stat, self.context, message + " failed")
    return stat


def _recurrent_step_device(self, device_x, elements, device_norm_weights, epsilon) -> status_t:
    """Extension: x <- x + layer(rms_norm(x) * norm_weights), in place."""
    return _step(self, _lib().fortai_cuda_qwen35_recurrent_step_device,
                 "CUDA Qwen recurrent step", device_x, elements, device_norm_weights,
                 c_float(epsilon))


cuda_qwen35_recurrent_t.step_device = _recurrent_step_device


class cuda_qwen35_attention_t:
    """fortai_backend_cuda.f90:45-52 (gated attention layer; binary16 KV cache on the device)."""

    def __init__(self):
        self.handle = 0
        self.context = None

    def create(self, context, query, key, value, output, query_norm, key_norm, heads,
               key_value_heads, head_size, value_size, max_context, rope_dimension, rope_base,
               norm_epsilon) -> status_t:
        stat = status_t()
        if not context.handle or any(not w.handle for w in (query, key, value, output)):
            stat.set(FORTAI_INVALID, "invalid CUDA Qwen attention layer")
            return stat
        qn = np.ascontiguousarray(query_norm, dtype=np.float32)
        kn = np.ascontiguousarray(key_norm, dtype=np.float32)
        out = c_void_p()
        code = _lib().fortai_cuda_qwen35_attention_create(
            context.handle, query.handle, key.handle, value.handle, output.handle, _host_ptr(qn),
            qn.nbytes, _host_ptr(kn), kn.nbytes, int(heads), int(key_value_heads), int(head_size),
            int(value_size), int(max_context), int(rope_dimension), c_float(rope_base),
            c_float(norm_epsilon), byref(out))
        if code != FORTAI_CUDA_OK:
            return _failed(stat, context, "CUDA Qwen attention layer creation failed")
        self.handle, self.context = out.value, context
        return stat

    def destroy(self) -> status_t:
        stat = status_t()
        if self.handle:
            _lib().fortai_cuda_qwen35_attention_destroy(self.handle)
            self.handle = 0
        return stat

    def reset(self) -> status_t:
        stat = status_t()
        if not self.handle:
            stat.set(FORTAI_INVALID, "invalid CUDA Qwen attention layer")
        elif _lib().fortai_cuda_qwen35_attention_reset(self.handle) != FORTAI_CUDA_OK:
            return _failed(stat, self.context, "CUDA Qwen attention reset failed")
        return stat

    def run_device(self, device_activation, activation_elements, position, device_output,
                   output_elements) -> status_t:
        stat = status_t()
        if not self.handle or not device_activation or not device_output:
            stat.set(FORTAI_INVALID, "invalid CUDA Qwen attention device run")
            return stat
        code = _lib().fortai_cuda_qwen35_attention_run_device(
            self.handle, device_activation, activation_elements, int(position), device_output,
            output_elements)
        if code != FORTAI_CUDA_OK:
            return _failed(stat, self.context, "CUDA Qwen attention device run failed")
        return stat


def _attention_step_device(self, device_x, elements, position, device_norm_weights,
                           epsilon) -> status_t:
    """Extension: x <- x + layer(rms_norm(x) * norm_weights), in place."""
    return _step(self, _lib().fortai_cuda_qwen35_attention_step_device,
                 "CUDA Qwen attention step", device_x, elements, int(position),
                 device_norm_weights, c_float(epsilon))


cuda_qwen35_attention_t.step_device = _attention_step_device


# --------------------------------------------------------------------------- device groups
class cuda_q8_group_t:
    """Several GPUs of one box driven from one host thread through the C ABI: row- and
    column-sharded projections without torch.distributed (what a Fortran host would call)."""

    def __init__(self):
        self.handle = None

    def create(self, devices) -> status_t:
        stat = status_t()
        ids = (ctypes.c_int * len(devices))(*[int(d) for d in devices])
        out = c_void_p()
        code = _lib().fortai_cuda_q8_group_create(ids, len(devices), byref(out))
        if code != FORTAI_CUDA_OK:
            stat.set(FORTAI_UNSUPPORTED if code == 2 else FORTAI_INVALID,
                     "CUDA Q8 device group creation failed")
            return stat
        self.handle = out
        return stat

    def destroy(self):
        if self.handle:
            _lib().fortai_cuda_q8_group_destroy(self.handle)
            self.handle = None

    def device_count(self) -> int:
        return int(_lib().fortai_cuda_q8_group_device_count(self.handle)) if self.handle else 0

    def last_error(self) -> str:
        raw = _lib().fortai_cuda_q8_group_last_error(self.handle if self.handle else None)
        return raw.decode(errors="replace") if raw else ""

    def upload(self, host_weights, rows: int, width: int, shard_mode: int):
        """shard_mode 0: row ranges; 1: block (K) ranges of every row.  Returns (handle, stat)."""
        stat = status_t()
        data = _as_bytes(host_weights)
        out = c_void_p()
        code = _lib().fortai_cuda_q8_group_weights_upload(self.handle, _host_ptr(data), data.size,
                                                          int(rows), int(width), int(shard_mode),
                                                          byref(out))
        if code != FORTAI_CUDA_OK:
            stat.set(FORTAI_INVALID if code == 1 else FORTAI_UNSUPPORTED,
                     "CUDA Q8 group weights upload failed: " + self.last_error())
            return None, stat
        return out, stat

    @staticmethod
    def destroy_weights(weights):
        if weights:
            _lib().fortai_cuda_q8_group_weights_destroy(weights)

    def matvec_f32(self, weights, activation, output):
        stat = status_t()
        ms = c_float(0.0)
        code = _lib().fortai_cuda_q8_group_matvec_f32(self.handle, weights, _host_ptr(activation),
                                                      activation.size, _host_ptr(output),
                                                      output.nbytes, byref(ms))
        if code != FORTAI_CUDA_OK:
            stat.set(FORTAI_INVALID if code == 1 else FORTAI_UNSUPPORTED,
                     "CUDA Q8 group matvec failed: " + self.last_error())
        return ms.value, stat

    def ffn_f32(self, gate, up, down, activation, output):
        stat = status_t()
        ms = c_float(0.0)
        code = _lib().fortai_cuda_q8_group_ffn_f32(self.handle, gate, up, down,
                                                   _host_ptr(activation), activation.size,
                                                   _host_ptr(output), output.nbytes, byref(ms))
        if code != FORTAI_CUDA_OK:
            stat.set(FORTAI_INVALID if code == 1 else FORTAI_UNSUPPORTED,
                     "CUDA Q8 group FFN failed: " + self.last_error())
        return ms.value, stat
