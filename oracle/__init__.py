"""ctypes front end of the CPU oracle (TEST INFRASTRUCTURE ONLY).

The oracle restates the reference's CPU arithmetic for the quantized matrix-product path in plain C
(``synapse_oracle.c``). Only tests, the smoke check and the benchmark's CPU-baseline leg import this
module; the product package never does. Arrays are numpy; every function returns fresh arrays.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import POINTER, c_double, c_float, c_int, c_int8, c_int16, c_int32, c_size_t, c_uint8, c_uint16, c_uint32, c_uint64, c_void_p

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libsynapse_oracle.so")
_lib = None

Q8_0, Q4_K, Q6_K = 8, 12, 14
BLOCK_VALUES = {Q8_0: 32, Q4_K: 256, Q6_K: 256}
BLOCK_BYTES = {Q8_0: 34, Q4_K: 144, Q6_K: 210}
GROUPS_PER_BLOCK = {Q8_0: 1, Q4_K: 8, Q6_K: 16}


def build(force: bool = False) -> str:
    """Compiles the oracle with gcc (``make`` in this folder) and returns the library path."""
    source = os.path.join(_HERE, "synapse_oracle.c")
    stale = not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(source)
    if force or stale:
        subprocess.run(["make", "-B", "-C", _HERE, "libsynapse_oracle.so"], check=True, capture_output=True)
    return _LIB_PATH


def _ptr(array: np.ndarray, ctype):
    return array.ctypes.data_as(POINTER(ctype))


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        handle = ctypes.CDLL(_LIB_PATH)
        handle.orc_fp16_to_f32.restype = c_float
        handle.orc_fp16_to_f32.argtypes = [c_uint16]
        handle.orc_f32_to_fp16.restype = c_uint16
        handle.orc_f32_to_fp16.argtypes = [c_float]
        handle.orc_q8_quantize_row.restype = c_int
        handle.orc_q8_quantize_row.argtypes = [c_void_p, c_size_t, c_void_p, c_void_p]
        handle.orc_q8_group_sums.restype = None
        handle.orc_q8_group_sums.argtypes = [c_void_p, c_size_t, c_void_p]
        handle.orc_q8q8_matmul.restype = c_int
        handle.orc_q8q8_matmul.argtypes = [c_void_p, c_size_t, c_size_t, c_size_t, c_void_p, c_void_p, c_size_t, c_void_p, c_size_t]
        handle.orc_q8q8_block_dots.restype = None
        handle.orc_q8q8_block_dots.argtypes = [c_void_p, c_size_t, c_size_t, c_void_p, c_size_t, c_void_p]
        handle.orc_q8q8_exact.restype = None
        handle.orc_q8q8_exact.argtypes = [c_void_p, c_size_t, c_size_t, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]
        handle.orc_have_avx2.restype = c_int
        handle.orc_row_bytes.restype = c_size_t
        handle.orc_row_bytes.argtypes = [c_uint32, c_size_t]
        handle.orc_decode_row.restype = c_int
        handle.orc_decode_row.argtypes = [c_uint32, c_void_p, c_size_t, c_void_p]
        handle.orc_f32_matmul.restype = c_int
        handle.orc_f32_matmul.argtypes = [c_uint32, c_void_p, c_size_t, c_size_t, c_void_p, c_size_t, c_size_t, c_void_p, c_size_t]
        handle.orc_f32_exact.restype = c_int
        handle.orc_f32_exact.argtypes = [c_uint32, c_void_p, c_size_t, c_size_t, c_void_p, c_size_t, c_size_t, c_void_p, c_void_p]
        handle.orc_int_dots.restype = c_size_t
        handle.orc_int_dots.argtypes = [c_uint32, c_void_p, c_size_t, c_size_t, c_void_p, c_size_t, c_void_p]
        handle.orc_kq_q8_matmul.restype = c_int
        handle.orc_kq_q8_matmul.argtypes = [c_uint32, c_void_p, c_size_t, c_size_t, c_void_p, c_void_p, c_size_t, c_void_p, c_size_t]
        handle.orc_kq_q8_exact.restype = c_int
        handle.orc_kq_q8_exact.argtypes = [c_uint32, c_void_p, c_size_t, c_size_t, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]
        handle.orc_chunk_rows.restype = c_size_t
        handle.orc_chunk_rows.argtypes = [c_size_t, c_size_t]
        handle.orc_q8q8_matmul_threads.restype = c_int
        handle.orc_q8q8_matmul_threads.argtypes = [c_void_p, c_size_t, c_size_t, c_void_p, c_void_p, c_size_t, c_void_p, c_size_t, c_size_t]
        handle.orc_f32_matmul_threads.restype = c_int
        handle.orc_f32_matmul_threads.argtypes = [c_uint32, c_void_p, c_size_t, c_size_t, c_void_p, c_size_t, c_size_t, c_void_p, c_size_t, c_size_t]
        handle.orc_lcg_case.restype = None
        handle.orc_lcg_case.argtypes = [c_uint64, c_size_t, c_size_t, c_size_t, c_void_p, c_void_p, c_void_p]
        handle.orc_decoder_create.restype = c_void_p
        handle.orc_decoder_create.argtypes = [c_void_p, c_size_t]
        handle.orc_decoder_destroy.restype = None
        handle.orc_decoder_destroy.argtypes = [c_void_p]
        handle.orc_decoder_forward.restype = c_int
        handle.orc_decoder_forward.argtypes = [c_void_p, c_int32, c_int32, c_int32, c_void_p]
        for name, argtypes in (("orc_rms_norm", [c_void_p, c_void_p, ctypes.c_float, c_size_t, c_void_p]),
                               ("orc_rotate_neox", [c_void_p, c_size_t, c_void_p, c_void_p]),
                               ("orc_swiglu", [c_void_p, c_void_p, c_size_t, c_void_p]),
                               ("orc_softmax", [c_void_p, c_size_t])):
            getattr(handle, name).restype = None
            getattr(handle, name).argtypes = argtypes
        handle.orc_argmax.restype = c_int32
        handle.orc_argmax.argtypes = [c_void_p, c_size_t]
        _lib = handle
    return _lib


def _c(array, dtype):
    return np.ascontiguousarray(array, dtype=dtype)


def _addr(array: np.ndarray) -> int:
    return array.ctypes.data


def rms_norm(x, weight, epsilon):
    """RMSNorm with the FP64 sum of squares of the optimized CPU executor."""
    x, weight = _c(x, np.float32), _c(weight, np.float32)
    out = np.empty_like(x)
    lib().orc_rms_norm(_addr(x), _addr(weight), np.float32(epsilon), x.size, _addr(out))
    return out


def rotate_neox(x, cosines, sines):
    """NeoX rotation of one head (first half against second half)."""
    out = _c(x, np.float32).copy()
    cosines, sines = _c(cosines, np.float32), _c(sines, np.float32)
    lib().orc_rotate_neox(_addr(out), out.size, _addr(cosines), _addr(sines))
    return out


def swiglu(gate, up):
    gate, up = _c(gate, np.float32), _c(up, np.float32)
    out = np.empty_like(gate)
    lib().orc_swiglu(_addr(gate), _addr(up), gate.size, _addr(out))
    return out


def softmax(scores):
    out = _c(scores, np.float32).copy()
    lib().orc_softmax(_addr(out), out.size)
    return out


def fp16_to_f32(bits: int) -> float:
    return float(lib().orc_fp16_to_f32(bits))


def f32_to_fp16(value: float) -> int:
    return int(lib().orc_f32_to_fp16(np.float32(value)))


def row_bytes(ggml_type: int, columns: int) -> int:
    """Bytes of one row, 0 for an unknown type or a width that is not a whole number of blocks."""
    return int(lib().orc_row_bytes(ggml_type, columns))


def quantize(x):
    """Q8_0 activation quantiser. ``x`` is [tokens, columns] (or [columns]) float32.

    Returns (codes int8 like x, scales float32 [tokens, columns/32])."""
    x = _c(x, np.float32)
    flat = x.reshape(-1, x.shape[-1])
    tokens, columns = flat.shape
    codes = np.empty((tokens, columns), np.int8)
    scales = np.empty((tokens, max(columns // 32, 0)), np.float32)
    for t in range(tokens):
        status = lib().orc_q8_quantize_row(_addr(flat[t]), columns, _addr(codes[t]), _addr(scales[t]))
        if status != 0:
            raise ValueError(f"Q8_0 activation rows need a positive multiple of 32 values; got {columns}")
    return codes.reshape(x.shape), scales.reshape(x.shape[:-1] + (columns // 32,))


def group_sums(codes):
    codes = _c(codes, np.int8)
    sums = np.empty(codes.size // 16, np.int16)
    lib().orc_q8_group_sums(_addr(codes), codes.size, _addr(sums))
    return sums.reshape(codes.shape[:-1] + (codes.shape[-1] // 16,))


def q8q8_matmul(weights, rows, blocks, quants, scales, tokens, stride=None, fill=0.0, row_bytes_arg=None):
    """The reference's Q8_0 x Q8_0 scalar kernel. Returns (status, output[(tokens-1)*stride + rows])."""
    weights = _c(weights, np.uint8)
    quants = _c(quants, np.int8)
    scales = _c(scales, np.float32)
    stride = rows if stride is None else stride
    output = np.full(max((tokens - 1) * stride + rows, 1), fill, np.float32)
    status = lib().orc_q8q8_matmul(_addr(weights), blocks * 34 if row_bytes_arg is None else row_bytes_arg, rows, blocks,
                                   _addr(quants), _addr(scales), tokens, _addr(output), stride)
    return status, output


def q8q8_block_dots(weights, rows, blocks, quants, tokens):
    weights = _c(weights, np.uint8)
    quants = _c(quants, np.int8)
    dots = np.empty((tokens, rows, blocks), np.int32)
    lib().orc_q8q8_block_dots(_addr(weights), rows, blocks, _addr(quants), tokens, _addr(dots))
    return dots


def q8q8_exact(weights, rows, blocks, quants, scales, tokens):
    weights = _c(weights, np.uint8)
    quants = _c(quants, np.int8)
    scales = _c(scales, np.float32)
    value = np.empty((tokens, rows), np.float64)
    magnitude = np.empty((tokens, rows), np.float64)
    lib().orc_q8q8_exact(_addr(weights), rows, blocks, _addr(quants), _addr(scales), tokens, _addr(value), _addr(magnitude))
    return value, magnitude


def decode(ggml_type, data, columns):
    """Decodes rows of ``columns`` values from raw GGUF blocks. Returns float32 [rows, columns]."""
    data = _c(data, np.uint8).reshape(-1)
    rb = row_bytes(ggml_type, columns)
    if rb == 0 or data.size % rb != 0:
        raise ValueError(f"{columns} values of type {ggml_type} do not form whole blocks in {data.size} bytes")
    rows = data.size // rb
    out = np.empty((rows, columns), np.float32)
    for r in range(rows):
        lib().orc_decode_row(ggml_type, _addr(data) + r * rb, columns, _addr(out[r]))
    return out


def f32_matmul(ggml_type, weights, rows, columns, x):
    """The reference backend's FP32-activation product. ``x`` [tokens, columns]; returns [tokens, rows]."""
    weights = _c(weights, np.uint8)
    x = _c(x, np.float32).reshape(-1, columns)
    y = np.empty((x.shape[0], rows), np.float32)
    status = lib().orc_f32_matmul(ggml_type, _addr(weights), rows, columns, _addr(x), x.shape[0], columns, _addr(y), rows)
    if status != 0:
        raise ValueError(f"oracle f32 matmul rejected the shape (status {status})")
    return y


def f32_exact(ggml_type, weights, rows, columns, x):
    weights = _c(weights, np.uint8)
    x = _c(x, np.float32).reshape(-1, columns)
    value = np.empty((x.shape[0], rows), np.float64)
    magnitude = np.empty((x.shape[0], rows), np.float64)
    lib().orc_f32_exact(ggml_type, _addr(weights), rows, columns, _addr(x), x.shape[0], columns, _addr(value), _addr(magnitude))
    return value, magnitude


def int_dots(ggml_type, weights, rows, columns, quants):
    """Exact integer sub-block dots: [tokens, rows, groups] int32 (1, 8 or 16 groups per block)."""
    weights = _c(weights, np.uint8)
    quants = _c(quants, np.int8).reshape(-1, columns)
    groups = columns // BLOCK_VALUES[ggml_type] * GROUPS_PER_BLOCK[ggml_type]
    out = np.empty((quants.shape[0], rows, groups), np.int32)
    got = lib().orc_int_dots(ggml_type, _addr(weights), rows, columns, _addr(quants), quants.shape[0], _addr(out))
    if got != groups:
        raise ValueError("oracle int dots rejected the shape")
    return out


def kq_q8_matmul(ggml_type, weights, rows, columns, quants, scales):
    """Quantised weights x Q8_0-quantised activations (any of the three encodings): [tokens, rows]."""
    weights = _c(weights, np.uint8)
    quants = _c(quants, np.int8).reshape(-1, columns)
    scales = _c(scales, np.float32).reshape(-1, columns // 32)
    y = np.empty((quants.shape[0], rows), np.float32)
    status = lib().orc_kq_q8_matmul(ggml_type, _addr(weights), rows, columns, _addr(quants), _addr(scales), quants.shape[0], _addr(y), rows)
    if status != 0:
        raise ValueError(f"oracle kq matmul rejected the shape (status {status})")
    return y


def kq_q8_exact(ggml_type, weights, rows, columns, quants, scales):
    weights = _c(weights, np.uint8)
    quants = _c(quants, np.int8).reshape(-1, columns)
    scales = _c(scales, np.float32).reshape(-1, columns // 32)
    value = np.empty((quants.shape[0], rows), np.float64)
    magnitude = np.empty((quants.shape[0], rows), np.float64)
    lib().orc_kq_q8_exact(ggml_type, _addr(weights), rows, columns, _addr(quants), _addr(scales), quants.shape[0], _addr(value), _addr(magnitude))
    return value, magnitude


def chunk_rows(rows: int, threads: int) -> int:
    return int(lib().orc_chunk_rows(rows, threads))


def q8q8_matmul_threads(weights, rows, blocks, quants, scales, tokens, threads, output=None):
    weights = _c(weights, np.uint8)
    quants = _c(quants, np.int8)
    scales = _c(scales, np.float32)
    if output is None:
        output = np.empty((tokens, rows), np.float32)
    status = lib().orc_q8q8_matmul_threads(_addr(weights), rows, blocks, _addr(quants), _addr(scales), tokens, _addr(output), rows, threads)
    if status != 0:
        raise ValueError(f"oracle q8q8 threads rejected the shape (status {status})")
    return output


def f32_matmul_threads(ggml_type, weights, rows, columns, x, threads, output=None):
    weights = _c(weights, np.uint8)
    x = _c(x, np.float32).reshape(-1, columns)
    if output is None:
        output = np.empty((x.shape[0], rows), np.float32)
    status = lib().orc_f32_matmul_threads(ggml_type, _addr(weights), rows, columns, _addr(x), x.shape[0], columns, _addr(output), rows, threads)
    if status != 0:
        raise ValueError(f"oracle f32 threads rejected the shape (status {status})")
    return output


def lcg_case(seed, rows, blocks, tokens):
    """The seeded Q8_0 x Q8_0 case of the reference's Rust kernel tests."""
    weights = np.empty(rows * blocks * 34, np.uint8)
    quants = np.empty(tokens * blocks * 32, np.int8)
    scales = np.empty(tokens * blocks, np.float32)
    lib().orc_lcg_case(seed, rows, blocks, tokens, _addr(weights), _addr(quants), _addr(scales))
    return weights, quants, scales


class Decoder:
    """The reference's optimized CPU executor, one token at a time (O8). ``desc`` is a ctypes structure with the layout of
    the reference's DecoderDesc; it and the buffers it points to must outlive the decoder."""

    def __init__(self, desc, vocabulary: int, threads: int | None = None):
        self._desc = desc
        self.vocabulary = vocabulary
        self._handle = lib().orc_decoder_create(ctypes.addressof(desc), threads or (os.cpu_count() or 1))
        if not self._handle:
            raise MemoryError("oracle decoder allocation failed")

    def decode(self, token: int, position: int, slot: int = 0) -> np.ndarray:
        logits = np.empty(self.vocabulary, np.float32)
        status = lib().orc_decoder_forward(self._handle, slot, token, position, _addr(logits))
        if status != 0:
            raise ValueError(f"oracle decoder rejected the token (status {status})")
        return logits

    @staticmethod
    def argmax(logits: np.ndarray) -> int:
        logits = _c(logits, np.float32)
        return int(lib().orc_argmax(_addr(logits), logits.size))

    def close(self):
        if self._handle:
            lib().orc_decoder_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
