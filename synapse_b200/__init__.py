"""Host-side mirror of the reference's operator surface for the quantized matrix-product path.

The product is ``libsynapse_b200.so`` (hand-written sm_100a CUDA behind a C ABI, ``include/synapse_b200.h``).
This package is the thin host layer above it, shaped like the reference's C# types so that callers and
tests read the same way:

* :class:`NativeB200Library` — loader with ABI check and status mapping, the sibling of ``NativeQ8Kernel`` /
  ``NativeGpuLibrary`` (src/Synapse.Runtime/Features/CpuKernels/NativeQ8Kernel.cs:45-71,
  src/Synapse.Runtime/Features/GpuKernels/NativeGpuLibrary.cs:49-75,130-145).
* :class:`QuantizedMatrix` — a loaded weight matrix, the sibling of ``Q8Matrix`` + ``Q8MatrixKernel.Multiply``
  (src/Synapse.Runtime/Features/CpuKernels/Q8Matrix.cs:6-55, Q8MatrixKernel.cs:11-48).
* :func:`quantize_row` / :class:`Q8ActivationBuffer` — ``Q8ActivationQuantizer.QuantizeRow`` and its buffer
  (Q8ActivationQuantizer.cs:15-57, Q8ActivationBuffer.cs:7-54).

There is no CPU fallback: if the library is missing or no B200 is present every call raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, byref, c_char, c_float, c_int8, c_int32, c_size_t, c_uint8, c_uint32, c_uint64, c_void_p

import numpy as np

Q8_0, Q4_K, Q6_K = 8, 12, 14
REPACK = 1
MODE_XQ8, MODE_XF32 = 0, 1
EPILOGUE_STORE, EPILOGUE_ACCUMULATE = 0, 1
GEMM_F16, GEMM_F16X2 = 0, 1
EXPECTED_ABI_VERSION = 1
BLOCK_VALUES = {Q8_0: 32, Q4_K: 256, Q6_K: 256}
BLOCK_BYTES = {Q8_0: 34, Q4_K: 144, Q6_K: 210}
LIBRARY_FILE_NAME = "libsynapse_b200.so"

_STATUS_NAMES = {1: "NULL_POINTER", 2: "INVALID_ARGUMENT", 3: "UNAVAILABLE", 4: "DEVICE_ERROR", 5: "OUT_OF_MEMORY", 6: "INTERNAL"}


class BackendUnavailableError(RuntimeError):
    """Status 3, or the library cannot be loaded (the C# side raises NotSupportedException)."""


class DeviceMemoryError(MemoryError):
    """Status 5 (InsufficientMemoryException on the C# side)."""


class KernelError(RuntimeError):
    """Every other non-zero status (InvalidOperationException on the C# side)."""

    def __init__(self, status: int, message: str):
        super().__init__(f"synapse_b200 returned status {status} ({_STATUS_NAMES.get(status, '?')}): {message}")
        self.status = status


class Epilogue(ctypes.Structure):
    """``syn_b200_epilogue``: v = dot (+ bias[r]); v = silu(gate[t][r]) * v; y = accumulate ? y + v : v (device pointers)."""

    _fields_ = [("bias", c_void_p), ("gate", c_void_p), ("gate_stride", c_uint64), ("accumulate", c_uint32), ("reserved", c_uint32)]


class Segment(ctypes.Structure):
    """``syn_b200_segment``: one row range of a product that multiplies several matrices in one launch (the reference's
    ``MatmulSegment``, native/synapse-gpu/src/Features/GpuKernels/params.rs:42-61)."""

    _fields_ = [("matrix", c_void_p), ("row_start", c_uint64), ("row_count", c_uint64), ("bias", c_void_p), ("out_column", c_uint64)]


class Gather(ctypes.Structure):
    """``syn_b200_gather``: the other GPUs' copies of a row-sharded product's output and its completion signal."""

    _fields_ = [("peer_outputs", POINTER(c_void_p)), ("peer_count", c_uint32), ("reserved", c_uint32), ("signals", POINTER(c_void_p)),
                ("arrivals", c_void_p)]


def _gather(peer_ptrs, signal_ptrs=(), arrivals_ptr=0):
    """A ``Gather`` (with the arrays it points to kept alive on it), or None for a product on one GPU without a signal."""
    if not peer_ptrs and not signal_ptrs:
        return None
    gather = Gather()
    gather._peers = (c_void_p * max(len(peer_ptrs), 1))(*peer_ptrs)
    gather.peer_outputs = ctypes.cast(gather._peers, POINTER(c_void_p))
    gather.peer_count = len(peer_ptrs)
    if signal_ptrs:
        if len(signal_ptrs) != len(peer_ptrs) + 1:
            raise ValueError("a completion signal needs one word per peer plus this GPU's own")
        gather._signals = (c_void_p * len(signal_ptrs))(*signal_ptrs)
        gather.signals = ctypes.cast(gather._signals, POINTER(c_void_p))
        gather.arrivals = arrivals_ptr
    return gather


class GgufTensor(ctypes.Structure):
    """``syn_b200_gguf_tensor``: one entry of a GGUF file's tensor table (the reference's ``GgufTensorInfo``)."""

    _fields_ = [("name", c_char * 128), ("ggml_type", c_uint32), ("rank", c_uint32), ("dimensions", c_uint64 * 8), ("offset", c_uint64),
                ("bytes", c_uint64)]


class DeviceInfo(ctypes.Structure):
    _fields_ = [("name", c_char * 128), ("total_memory_bytes", c_uint64), ("max_buffer_bytes", c_uint64),
                ("compute_capability", c_uint32), ("multiprocessors", c_uint32)]


_EXPORTS = {
    "syn_b200_abi_version": (c_uint32, []),
    "syn_b200_probe": (c_int32, [POINTER(DeviceInfo)]),
    "syn_b200_last_error": (c_size_t, [c_void_p, c_size_t]),
    "syn_b200_matrix_create": (c_int32, [c_void_p, c_uint32, c_uint64, c_uint64, c_uint32, POINTER(c_void_p)]),
    "syn_b200_matrix_create_from_device": (c_int32, [c_void_p, c_uint32, c_uint64, c_uint64, c_uint32, c_void_p, POINTER(c_void_p)]),
    "syn_b200_matrix_destroy": (None, [c_void_p]),
    "syn_b200_matrix_info": (c_int32, [c_void_p, POINTER(c_uint32), POINTER(c_uint64), POINTER(c_uint64), POINTER(c_uint32), POINTER(c_uint64)]),
    "syn_b200_quantize_q8": (c_int32, [c_void_p, c_uint64, c_uint64, c_uint64, c_void_p, c_void_p]),
    "syn_b200_matmul_q8": (c_int32, [c_void_p, c_uint64, c_uint64, c_void_p, c_void_p, c_uint64, c_void_p, c_uint64]),
    "syn_b200_matvec": (c_int32, [c_void_p, c_uint64, c_uint64, c_void_p, c_uint64, c_uint64, c_void_p, c_uint64, c_uint32, c_uint32]),
    "syn_b200_gemm": (c_int32, [c_void_p, c_void_p, c_uint64, c_uint64, c_void_p, c_uint64, c_uint32]),
    "syn_b200_block_dots": (c_int32, [c_void_p, c_uint64, c_uint64, c_void_p, c_uint64, c_void_p]),
    "syn_b200_activation_scratch_bytes": (c_uint64, [c_uint64, c_uint64]),
    "syn_b200_quantize_q8_dev": (c_int32, [c_void_p, c_uint64, c_uint64, c_uint64, c_void_p, c_uint64, c_void_p]),
    "syn_b200_matmul_q8_dev": (c_int32, [c_void_p, c_uint64, c_uint64, c_void_p, c_uint64, c_void_p, c_uint64, c_uint32, c_void_p]),
    "syn_b200_matvec_dev": (c_int32, [c_void_p, c_uint64, c_uint64, c_void_p, c_uint64, c_uint64, c_void_p, c_uint64, c_uint32, c_uint32, c_void_p, c_uint64, c_void_p]),
    "syn_b200_shared_buffer_create": (c_int32, [c_uint64, POINTER(c_void_p), POINTER(c_uint8)]),
    "syn_b200_shared_buffer_open": (c_int32, [POINTER(c_uint8), POINTER(c_void_p)]),
    "syn_b200_shared_buffer_close": (None, [c_void_p]),
    "syn_b200_shared_buffer_destroy": (None, [c_void_p]),
    "syn_b200_enable_peer_access": (c_int32, [c_int32]),
    "syn_b200_matmul_q8_gather_dev": (c_int32, [c_void_p, c_uint64, c_uint64, c_void_p, c_uint64, c_void_p, c_uint64, POINTER(Gather), c_void_p]),
    "syn_b200_gather_wait_dev": (c_int32, [c_void_p, c_uint32, c_void_p, c_uint32, c_void_p]),
    "syn_b200_matmul_q8_ex_dev": (c_int32, [c_void_p, c_uint64, c_uint64, c_void_p, c_uint64, c_void_p, c_uint64, POINTER(Epilogue), c_void_p]),
    "syn_b200_matmul_q8_segments_dev": (c_int32, [POINTER(Segment), c_uint32, c_void_p, c_uint64, c_void_p, c_uint64, c_uint32, POINTER(Gather), c_void_p]),
    "syn_b200_matmul_q8_swiglu_dev": (c_int32, [c_void_p, c_void_p, c_uint64, c_uint64, c_void_p, c_uint64, c_void_p, c_uint64, c_void_p, POINTER(Gather),
                                                c_void_p]),
    "syn_b200_matvec_ex_dev": (c_int32, [c_void_p, c_uint64, c_uint64, c_void_p, c_uint64, c_uint64, c_void_p, c_uint64, c_uint32, POINTER(Epilogue), c_void_p, c_uint64, c_void_p]),
    "syn_b200_matvec_static": (c_int32, [c_void_p, c_uint64, c_uint64, c_void_p, c_uint64, c_uint64, c_void_p, c_uint64, c_uint32, c_void_p]),
    "syn_b200_matvec_static_capacity": (c_uint64, []),
    "syn_b200_gemm_scratch_bytes": (c_uint64, [c_uint64, c_uint64]),
    "syn_b200_gemm_dev": (c_int32, [c_void_p, c_void_p, c_uint64, c_uint64, c_void_p, c_uint64, c_uint32, c_void_p, c_uint64, c_void_p]),
    "syn_b200_decoder_create": (c_int32, [c_void_p, POINTER(c_void_p)]),
    "syn_b200_decoder_forward": (c_int32, [c_void_p, c_void_p, c_uint64, c_void_p, c_uint64]),
    "syn_b200_decoder_forward_argmax": (c_int32, [c_void_p, c_void_p, c_uint64, c_void_p]),
    "syn_b200_decoder_destroy": (None, [c_void_p]),
    "syn_b200_decoder_kv_bytes": (c_uint64, [c_void_p]),
    "syn_b200_gguf_open": (c_int32, [ctypes.c_char_p, POINTER(c_void_p)]),
    "syn_b200_gguf_close": (None, [c_void_p]),
    "syn_b200_gguf_tensor_count": (c_uint64, [c_void_p]),
    "syn_b200_gguf_tensor_at": (c_int32, [c_void_p, c_uint64, POINTER(GgufTensor)]),
    "syn_b200_gguf_find": (c_int32, [c_void_p, ctypes.c_char_p, POINTER(GgufTensor)]),
    "syn_b200_gguf_mapping": (c_void_p, [c_void_p, POINTER(c_uint64), POINTER(c_uint64)]),
    "syn_b200_gguf_load_matrix": (c_int32, [c_void_p, ctypes.c_char_p, c_uint32, ctypes.c_char_p, POINTER(c_void_p)]),
    "syn_b200_launch_count": (c_uint64, [c_uint32]),
    "syn_b200_device_faults": (c_uint32, [c_uint32]),
}


def exported_symbols():
    """Names every loader expects to find, one per declaration of include/synapse_b200.h."""
    return sorted(_EXPORTS)


class NativeB200Library:
    """Loads ``libsynapse_b200.so`` from an explicit directory, checks the ABI version before anything else,
    and turns status codes into exceptions. Nothing is searched on the system path and nothing falls back."""

    def __init__(self, path: str, handle: ctypes.CDLL):
        self.library_path = path
        self._h = handle
        for name, (restype, argtypes) in _EXPORTS.items():
            try:
                fn = getattr(handle, name)
            except AttributeError as error:
                raise BackendUnavailableError(f"The B200 kernel backend is unavailable because it does not export '{name}': '{path}'.") from error
            fn.restype = restype
            fn.argtypes = argtypes
        self.abi_version = int(handle.syn_b200_abi_version())
        if self.abi_version != EXPECTED_ABI_VERSION:
            raise BackendUnavailableError(
                f"The B200 kernel backend is unavailable because its ABI version {self.abi_version} differs from the required "
                f"{EXPECTED_ABI_VERSION}: '{path}'.")

    @staticmethod
    def load(directory: str) -> "NativeB200Library":
        if not directory or not directory.strip():
            raise ValueError("directory must be a non-empty path")
        path = os.path.join(os.path.abspath(directory), LIBRARY_FILE_NAME)
        if not os.path.exists(path):
            raise BackendUnavailableError(
                f"The B200 kernel backend is unavailable because the library file is missing: '{path}'. "
                "Build it with `python -m synapse_b200.build`.")
        try:
            handle = ctypes.CDLL(path)
        except OSError as error:
            raise BackendUnavailableError(f"The B200 kernel backend is unavailable because the operating system could not load it: '{path}' ({error}).") from error
        return NativeB200Library(path, handle)

    @staticmethod
    def load_from_package_directory() -> "NativeB200Library":
        return NativeB200Library.load(os.path.dirname(os.path.abspath(__file__)))

    def last_error(self) -> str:
        length = self._h.syn_b200_last_error(None, 0)
        buffer = ctypes.create_string_buffer(length or 1)
        self._h.syn_b200_last_error(ctypes.cast(buffer, c_void_p), length)
        return buffer.raw[:length].decode("utf-8", "replace")

    def check(self, status: int) -> None:
        if status == 0:
            return
        message = self.last_error()
        if status == 3:
            raise BackendUnavailableError(message)
        if status == 5:
            raise DeviceMemoryError(message)
        raise KernelError(status, message)

    def probe(self) -> DeviceInfo:
        info = DeviceInfo()
        self.check(self._h.syn_b200_probe(byref(info)))
        return info

    def shared_buffer_create(self, size: int) -> tuple[int, bytes]:
        """(device pointer, 64-byte handle) of a zero-filled buffer on the current device that other processes can map."""
        pointer, handle = c_void_p(), (c_uint8 * 64)()
        self.check(self._h.syn_b200_shared_buffer_create(size, byref(pointer), handle))
        return int(pointer.value), bytes(handle)

    def shared_buffer_open(self, handle: bytes) -> int:
        """Maps another process's shared buffer for the kernels of the current device; returns the device pointer."""
        pointer, raw = c_void_p(), (c_uint8 * 64).from_buffer_copy(handle)
        self.check(self._h.syn_b200_shared_buffer_open(raw, byref(pointer)))
        return int(pointer.value)

    def shared_buffer_close(self, pointer: int) -> None:
        self._h.syn_b200_shared_buffer_close(pointer)

    def shared_buffer_destroy(self, pointer: int) -> None:
        self._h.syn_b200_shared_buffer_destroy(pointer)

    def enable_peer_access(self, peer_device: int) -> None:
        """Lets kernels of the current device store into memory of ``peer_device`` (needed before mapped peer buffers are
        passed to ``matmul_q8_gather_device``)."""
        self.check(self._h.syn_b200_enable_peer_access(peer_device))

    def launch_count(self, reset: bool = False) -> int:
        return int(self._h.syn_b200_launch_count(1 if reset else 0))

    def device_faults(self, reset: bool = False) -> int:
        """Bounded device-side waits that gave up since the last reset; 0 in a healthy run."""
        return int(self._h.syn_b200_device_faults(1 if reset else 0))

    def activation_scratch_bytes(self, tokens: int, columns: int) -> int:
        return int(self._h.syn_b200_activation_scratch_bytes(tokens, columns))

    def gemm_scratch_bytes(self, tokens: int, columns: int) -> int:
        return int(self._h.syn_b200_gemm_scratch_bytes(tokens, columns))

    @property
    def raw(self) -> ctypes.CDLL:
        return self._h


_default_library = None


def library() -> NativeB200Library:
    """The library built beside this package; raises :class:`BackendUnavailableError` if it is not there."""
    global _default_library
    if _default_library is None:
        _default_library = NativeB200Library.load_from_package_directory()
    return _default_library


def _addr(array: np.ndarray) -> int:
    return array.ctypes.data


def quantize_row(x: np.ndarray, lib: NativeB200Library | None = None):
    """``Q8ActivationQuantizer.QuantizeRow`` on the device. ``x``: float32 [tokens, columns] or [columns].

    Returns (codes int8 with x's shape, scales float32 [..., columns/32])."""
    lib = lib or library()
    x = np.ascontiguousarray(x, np.float32)
    flat = x.reshape(-1, x.shape[-1])
    tokens, columns = flat.shape
    if columns == 0 or columns % 32:
        raise ValueError(f"Q8_0 activation rows need a positive multiple of 32 values; got {columns}.")
    codes = np.empty((tokens, columns), np.int8)
    scales = np.empty((tokens, columns // 32), np.float32)
    lib.check(lib.raw.syn_b200_quantize_q8(_addr(flat), tokens, columns, columns, _addr(codes), _addr(scales)))
    return codes.reshape(x.shape), scales.reshape(x.shape[:-1] + (columns // 32,))


class Q8ActivationBuffer:
    """Token-major Q8_0 activations: ``capacity`` rows of ``columns`` int8 codes and ``columns/32`` scales."""

    def __init__(self, columns: int, capacity: int = 1):
        if columns <= 0 or columns % 32 or capacity <= 0:
            raise ValueError(f"Activation buffers need a positive multiple of 32 columns and a positive capacity; got {columns}, {capacity}.")
        self.columns = columns
        self.capacity = capacity
        self.blocks_per_row = columns // 32
        self.quants = np.zeros((capacity, columns), np.int8)
        self.scales = np.zeros((capacity, self.blocks_per_row), np.float32)

    def quantize(self, token: int, x: np.ndarray, lib: NativeB200Library | None = None) -> None:
        if not 0 <= token < self.capacity:
            raise IndexError(f"Token {token} is outside activation capacity {self.capacity}.")
        codes, scales = quantize_row(np.asarray(x, np.float32).reshape(self.columns), lib)
        self.quants[token] = codes
        self.scales[token] = scales


class QuantizedMatrix:
    """A row-major [rows][columns] matrix of GGUF Q8_0 / Q4_K / Q6_K blocks resident on the current device."""

    def __init__(self, blocks: np.ndarray, ggml_type: int, rows: int, columns: int, repack: bool = True,
                 lib: NativeB200Library | None = None):
        self._lib = lib or library()
        self._handle = c_void_p()
        blocks = np.ascontiguousarray(blocks, np.uint8).reshape(-1)
        values = BLOCK_VALUES.get(ggml_type)
        if values and columns > 0 and columns % values == 0 and rows > 0:
            expected = rows * (columns // values) * BLOCK_BYTES[ggml_type]
            if blocks.size < expected:
                raise ValueError(f"A {rows}x{columns} matrix of type {ggml_type} needs {expected} bytes; got {blocks.size}.")
        self._lib.check(self._lib.raw.syn_b200_matrix_create(_addr(blocks), ggml_type, rows, columns, REPACK if repack else 0,
                                                            byref(self._handle)))
        self.ggml_type, self.rows, self.columns, self.repacked = ggml_type, rows, columns, repack
        self.row_bytes = columns // values * BLOCK_BYTES[ggml_type]
        self.source_bytes = rows * self.row_bytes

    @classmethod
    def from_device(cls, device_pointer: int, ggml_type: int, rows: int, columns: int, repack: bool = True, stream: int = 0,
                    lib: NativeB200Library | None = None) -> "QuantizedMatrix":
        self = cls.__new__(cls)
        self._lib = lib or library()
        self._handle = c_void_p()
        self._lib.check(self._lib.raw.syn_b200_matrix_create_from_device(device_pointer, ggml_type, rows, columns,
                                                                        REPACK if repack else 0, stream, byref(self._handle)))
        self.ggml_type, self.rows, self.columns, self.repacked = ggml_type, rows, columns, repack
        self.row_bytes = columns // BLOCK_VALUES[ggml_type] * BLOCK_BYTES[ggml_type]
        self.source_bytes = rows * self.row_bytes
        return self

    @property
    def handle(self) -> c_void_p:
        if not self._handle:
            raise ValueError("the matrix has been closed")
        return self._handle

    def close(self) -> None:
        if getattr(self, "_handle", None):
            self._lib.raw.syn_b200_matrix_destroy(self._handle)
            self._handle = c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *_):
        self.close()

    # ---- host-buffer operators ------------------------------------------------------------------------

    def multiply(self, row_start: int, row_count: int, activations: Q8ActivationBuffer, token_count: int,
                 output: np.ndarray | None = None, output_stride: int | None = None) -> np.ndarray:
        """``Q8MatrixKernel.Multiply``: ``output[t*stride + (r-row_start)] = dot(W[r], A[t])``."""
        if activations is None:
            raise ValueError("activations must not be None")
        if row_start < 0 or row_count <= 0 or row_start > self.rows - row_count:
            raise IndexError(f"Rows [{row_start}, {row_start + row_count}) exceed matrix rows {self.rows}.")
        if token_count <= 0 or token_count > activations.capacity:
            raise IndexError(f"Token count {token_count} is outside activation capacity {activations.capacity}.")
        if activations.columns != self.columns:
            raise ValueError(f"Activation width {activations.columns} does not match matrix width {self.columns}.")
        stride = row_count if output_stride is None else output_stride
        if token_count > 1 and stride < row_count:
            raise IndexError("output_stride")
        floats = (token_count - 1) * stride + row_count
        if output is None:
            output = np.zeros(floats, np.float32)
        if output.dtype != np.float32 or not output.flags.c_contiguous or output.size < floats:
            raise ValueError(f"output must be contiguous float32 with at least {floats} values")
        self._lib.check(self._lib.raw.syn_b200_matmul_q8(self.handle, row_start, row_count, _addr(activations.quants),
                                                        _addr(activations.scales), token_count, _addr(output), stride))
        return output

    def matvec(self, x: np.ndarray, mode: int = MODE_XQ8, row_start: int = 0, row_count: int | None = None,
               epilogue: int = EPILOGUE_STORE, output: np.ndarray | None = None, output_stride: int | None = None) -> np.ndarray:
        """FP32 activations [tokens, columns] -> [tokens, row_count] (or the caller's strided ``output``)."""
        x = np.ascontiguousarray(x, np.float32).reshape(-1, x.shape[-1])
        tokens = x.shape[0]
        row_count = self.rows - row_start if row_count is None else row_count
        stride = row_count if output_stride is None else output_stride
        if output is None:
            output = np.zeros((tokens, stride), np.float32)
        self._lib.check(self._lib.raw.syn_b200_matvec(self.handle, row_start, row_count, _addr(x), tokens, x.shape[1],
                                                     _addr(output), stride, mode, epilogue))
        return output

    def gemm(self, x: np.ndarray, precision: int = GEMM_F16) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float32).reshape(-1, x.shape[-1])
        y = np.zeros((x.shape[0], self.rows), np.float32)
        self._lib.check(self._lib.raw.syn_b200_gemm(self.handle, _addr(x), x.shape[0], x.shape[1], _addr(y), self.rows, precision))
        return y

    def block_dots(self, codes: np.ndarray, row_start: int = 0, row_count: int | None = None) -> np.ndarray:
        """Exact integer sub-block dots [tokens, row_count, groups] of the quantised-activation contract."""
        codes = np.ascontiguousarray(codes, np.int8).reshape(-1, self.columns)
        row_count = self.rows - row_start if row_count is None else row_count
        groups = self.columns // (16 if self.ggml_type == Q6_K else 32)
        out = np.zeros((codes.shape[0], row_count, groups), np.int32)
        self._lib.check(self._lib.raw.syn_b200_block_dots(self.handle, row_start, row_count, _addr(codes), codes.shape[0], _addr(out)))
        return out

    # ---- device-buffer operators (raw device addresses, e.g. torch.Tensor.data_ptr()) --------------------

    def matvec_device(self, x_ptr: int, tokens: int, in_stride: int, y_ptr: int, out_stride: int, mode: int = MODE_XQ8,
                      epilogue: int = EPILOGUE_STORE, scratch_ptr: int = 0, scratch_bytes: int = 0, stream: int = 0,
                      row_start: int = 0, row_count: int | None = None) -> None:
        row_count = self.rows - row_start if row_count is None else row_count
        self._lib.check(self._lib.raw.syn_b200_matvec_dev(self.handle, row_start, row_count, x_ptr, tokens, in_stride, y_ptr,
                                                         out_stride, mode, epilogue, scratch_ptr, scratch_bytes, stream))

    def matvec_fused_device(self, x_ptr: int, tokens: int, in_stride: int, y_ptr: int, out_stride: int, mode: int = MODE_XQ8,
                            bias_ptr: int = 0, gate_ptr: int = 0, gate_stride: int = 0, accumulate: bool = False, scratch_ptr: int = 0,
                            scratch_bytes: int = 0, stream: int = 0, row_start: int = 0, row_count: int | None = None) -> None:
        """Device product with the fused epilogue of the reference's projection regions (bias, SwiGLU gate, residual)."""
        row_count = self.rows - row_start if row_count is None else row_count
        epilogue = Epilogue(bias_ptr or None, gate_ptr or None, gate_stride, 1 if accumulate else 0, 0)
        self._lib.check(self._lib.raw.syn_b200_matvec_ex_dev(self.handle, row_start, row_count, x_ptr, tokens, in_stride, y_ptr, out_stride,
                                                            mode, byref(epilogue), scratch_ptr, scratch_bytes, stream))

    def matmul_q8_fused_device(self, scratch_ptr: int, tokens: int, y_ptr: int, out_stride: int, bias_ptr: int = 0, gate_ptr: int = 0,
                               gate_stride: int = 0, accumulate: bool = False, stream: int = 0, row_start: int = 0,
                               row_count: int | None = None) -> None:
        row_count = self.rows - row_start if row_count is None else row_count
        epilogue = Epilogue(bias_ptr or None, gate_ptr or None, gate_stride, 1 if accumulate else 0, 0)
        self._lib.check(self._lib.raw.syn_b200_matmul_q8_ex_dev(self.handle, row_start, row_count, scratch_ptr, tokens, y_ptr, out_stride,
                                                               byref(epilogue), stream))

    def matmul_q8_gather_device(self, scratch_ptr: int, tokens: int, y_ptr: int, out_stride: int, peer_ptrs, stream: int = 0,
                                row_start: int = 0, row_count: int | None = None, signal_ptrs=(), arrivals_ptr: int = 0) -> None:
        """The product of a row shard whose kernel also stores every result into the other GPUs' copies of the output
        (``peer_ptrs``: device pointers mapped into this process, offset to the shard's first row like ``y_ptr``) and, when
        ``signal_ptrs`` (this GPU's word first, then each peer's) and ``arrivals_ptr`` are given, signals completion."""
        row_count = self.rows - row_start if row_count is None else row_count
        gather = _gather(peer_ptrs, signal_ptrs, arrivals_ptr)
        self._lib.check(self._lib.raw.syn_b200_matmul_q8_gather_dev(self.handle, row_start, row_count, scratch_ptr, tokens, y_ptr, out_stride,
                                                                   byref(gather) if gather is not None else None, stream))

    def matvec_static(self, x_ptr: int, tokens: int, in_stride: int, y_ptr: int, out_stride: int, epilogue: int = EPILOGUE_STORE,
                      stream: int = 0, row_start: int = 0, row_count: int | None = None) -> None:
        """The quantised-activation product for callers that cannot allocate device memory: the scratch is a fixed
        array inside the library (at most ``syn_b200_matvec_static_capacity()`` activation values per call; calls that
        overlap on the GPU race on it)."""
        row_count = self.rows - row_start if row_count is None else row_count
        self._lib.check(self._lib.raw.syn_b200_matvec_static(self.handle, row_start, row_count, x_ptr, tokens, in_stride, y_ptr, out_stride,
                                                            epilogue, stream))

    def matmul_q8_device(self, scratch_ptr: int, tokens: int, y_ptr: int, out_stride: int, epilogue: int = EPILOGUE_STORE,
                         stream: int = 0, row_start: int = 0, row_count: int | None = None) -> None:
        row_count = self.rows - row_start if row_count is None else row_count
        self._lib.check(self._lib.raw.syn_b200_matmul_q8_dev(self.handle, row_start, row_count, scratch_ptr, tokens, y_ptr,
                                                            out_stride, epilogue, stream))

    def gemm_device(self, x_ptr: int, tokens: int, in_stride: int, y_ptr: int, out_stride: int, scratch_ptr: int,
                    scratch_bytes: int, precision: int = GEMM_F16, stream: int = 0) -> None:
        self._lib.check(self._lib.raw.syn_b200_gemm_dev(self.handle, x_ptr, tokens, in_stride, y_ptr, out_stride, precision,
                                                       scratch_ptr, scratch_bytes, stream))


class GgufFile:
    """A mapped GGUF file and its tensor table, parsed by the native library (the sibling of ``GgufFile`` /
    ``GgufHeaderReader``, src/Synapse.Runtime/Features/ModelLoading/Gguf/GgufFile.cs:57-98, GgufHeaderReader.cs:20-154)."""

    def __init__(self, path: str, lib: NativeB200Library | None = None):
        self._lib = lib or library()
        self._handle = c_void_p()
        self._lib.check(self._lib.raw.syn_b200_gguf_open(os.fsencode(path), byref(self._handle)))

    def close(self) -> None:
        if getattr(self, "_handle", None):
            self._lib.raw.syn_b200_gguf_close(self._handle)
            self._handle = c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *_):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def tensors(self) -> list[GgufTensor]:
        out = []
        for index in range(int(self._lib.raw.syn_b200_gguf_tensor_count(self._handle))):
            entry = GgufTensor()
            self._lib.check(self._lib.raw.syn_b200_gguf_tensor_at(self._handle, index, byref(entry)))
            out.append(entry)
        return out

    def find(self, name: str) -> GgufTensor:
        entry = GgufTensor()
        self._lib.check(self._lib.raw.syn_b200_gguf_find(self._handle, name.encode(), byref(entry)))
        return entry

    def data_offset(self) -> int:
        length, offset = c_uint64(), c_uint64()
        self._lib.raw.syn_b200_gguf_mapping(self._handle, byref(length), byref(offset))
        return int(offset.value)

    def load_matrix(self, name: str, repack: bool = True, cache_directory: str | None = None) -> "QuantizedMatrix":
        """The tensor as a device-resident matrix; with ``cache_directory`` its repacked image is persisted and reused."""
        entry = self.find(name)
        handle = c_void_p()
        self._lib.check(self._lib.raw.syn_b200_gguf_load_matrix(self._handle, name.encode(), REPACK if repack else 0,
                                                                os.fsencode(cache_directory) if cache_directory else None, byref(handle)))
        matrix = QuantizedMatrix.__new__(QuantizedMatrix)
        matrix._lib, matrix._handle = self._lib, handle
        matrix.ggml_type, matrix.rows, matrix.columns, matrix.repacked = int(entry.ggml_type), int(entry.dimensions[1]), int(entry.dimensions[0]), repack
        matrix.row_bytes = matrix.columns // BLOCK_VALUES[matrix.ggml_type] * BLOCK_BYTES[matrix.ggml_type]
        matrix.source_bytes = matrix.rows * matrix.row_bytes
        return matrix


def matmul_q8_segments_device(segments, scratch_ptr: int, tokens: int, y_ptr: int, out_stride: int, accumulate: bool = False, peer_ptrs=(),
                              stream: int = 0, signal_ptrs=(), arrivals_ptr: int = 0, lib: NativeB200Library | None = None) -> None:
    """Up to three row ranges against the same quantised activations in one launch (Q | K | V): ``segments`` is a list of
    ``(matrix, row_start, row_count, bias_ptr, out_column)``; results of a range go to ``y[t * out_stride + out_column + r]``."""
    lib = lib or library()
    packed = (Segment * max(len(segments), 1))()
    for i, (matrix, row_start, row_count, bias_ptr, out_column) in enumerate(segments):
        packed[i] = Segment(matrix.handle, row_start, matrix.rows - row_start if row_count is None else row_count, bias_ptr or None, out_column)
    gather = _gather(peer_ptrs, signal_ptrs, arrivals_ptr)
    lib.check(lib.raw.syn_b200_matmul_q8_segments_dev(packed, len(segments), scratch_ptr, tokens, y_ptr, out_stride, 1 if accumulate else 0,
                                                      byref(gather) if gather is not None else None, stream))


def matmul_q8_swiglu_device(gate: "QuantizedMatrix", up: "QuantizedMatrix", scratch_ptr: int, tokens: int, y_ptr: int, out_stride: int,
                            gate_values_ptr: int = 0, peer_ptrs=(), stream: int = 0, row_start: int = 0, row_count: int | None = None,
                            signal_ptrs=(), arrivals_ptr: int = 0, lib: NativeB200Library | None = None) -> None:
    """``y = silu(gate . x) * (up . x)`` for the same rows of a gate and an up matrix in one launch (the gate/up region)."""
    lib = lib or library()
    row_count = gate.rows - row_start if row_count is None else row_count
    gather = _gather(peer_ptrs, signal_ptrs, arrivals_ptr)
    lib.check(lib.raw.syn_b200_matmul_q8_swiglu_dev(gate.handle, up.handle, row_start, row_count, scratch_ptr, tokens, y_ptr, out_stride,
                                                    gate_values_ptr or None, byref(gather) if gather is not None else None, stream))


def gather_wait_device(signals_ptr: int, count: int, epoch_ptr: int, timeout_us: int = 1_000_000, stream: int = 0,
                       lib: NativeB200Library | None = None) -> None:
    """Queues the bounded wait for the next complete gathered vector (``syn_b200_gather_wait_dev``)."""
    lib = lib or library()
    lib.check(lib.raw.syn_b200_gather_wait_dev(signals_ptr, count, epoch_ptr, timeout_us, stream))


def quantize_device(x_ptr: int, tokens: int, columns: int, in_stride: int, scratch_ptr: int, scratch_bytes: int, stream: int = 0,
                    lib: NativeB200Library | None = None) -> None:
    lib = lib or library()
    lib.check(lib.raw.syn_b200_quantize_q8_dev(x_ptr, tokens, columns, in_stride, scratch_ptr, scratch_bytes, stream))
