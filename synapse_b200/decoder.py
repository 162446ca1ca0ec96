"""Host mirror of the reference's GPU decoder executor for the B200 backend, plus seeded random-init model images.

``Decoder`` is the sibling of ``GpuDecoderExecutor`` (src/Synapse.Runtime/Features/GpuKernels/GpuDecoderExecutor.cs:23-95):
it fills the same description structs (``DecoderDesc`` 136 B, ``DecoderLayerOffsets`` 120 B, ``BatchToken`` 16 B,
native/synapse-gpu/src/Features/GpuKernels/decoder.rs:61-141) and calls create / forward / destroy.
``ModelImage`` stands in for the mapped GGUF file: one byte buffer holding every tensor at an offset, random-init
with the block value distributions of the benchmark configs (no model file is needed or read).
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, byref, c_float, c_int32, c_uint8, c_uint32, c_uint64, c_void_p

import numpy as np

from . import synth

NO_TENSOR = 0xFFFFFFFFFFFFFFFF


class LayerOffsets(ctypes.Structure):
    _fields_ = [(name, c_uint64) for name in (
        "attention_norm", "query", "key", "value", "query_bias", "key_bias", "value_bias", "query_norm", "key_norm",
        "attention_output", "feed_forward_norm", "gate", "up", "down", "encodings")]


class DecoderDesc(ctypes.Structure):
    _fields_ = [("weights", c_void_p), ("weights_length", c_uint64), ("layers", POINTER(LayerOffsets)),
                ("rope_cosines", POINTER(c_float)), ("rope_sines", POINTER(c_float)),
                ("token_embedding", c_uint64), ("output_norm", c_uint64), ("output", c_uint64),
                ("layer_count", c_uint32), ("hidden", c_uint32), ("feed_forward", c_uint32), ("heads", c_uint32),
                ("kv_heads", c_uint32), ("head_dim", c_uint32), ("vocabulary", c_uint32), ("context", c_uint32),
                ("session_slots", c_uint32), ("step_tokens", c_uint32), ("logits_rows", c_uint32), ("rms_epsilon", c_float),
                ("embedding_encoding", c_uint32), ("rope_layout", c_uint32), ("activation", c_uint32), ("kv_precision", c_uint32),
                ("kv_growth_positions", c_uint32), ("output_encoding", c_uint32)]


class BatchToken(ctypes.Structure):
    _fields_ = [("slot", c_int32), ("token", c_int32), ("position", c_int32), ("logits_row", c_int32)]


assert ctypes.sizeof(LayerOffsets) == 120 and ctypes.sizeof(DecoderDesc) == 136 and ctypes.sizeof(BatchToken) == 16


def rope_tables(head_dim: int, context: int, theta: float = 1_000_000.0):
    """Unscaled rotary tables, ``position / theta ** (2i/d)`` evaluated in FP32
    (src/Synapse.Runtime/Features/TextGeneration/RopeFrequencies.cs:55-78). Returns (cosines, sines) [context, d/2]."""
    half = head_dim // 2
    index = np.arange(half, dtype=np.float32)
    exponent = (np.float32(2.0) * index / np.float32(head_dim)).astype(np.float32)
    divisor = np.power(np.float32(theta), exponent).astype(np.float32)
    angles = (np.arange(context, dtype=np.float32)[:, None] / divisor[None, :]).astype(np.float32)
    return np.cos(angles).astype(np.float32), np.sin(angles).astype(np.float32)


class ModelImage:
    """A random-init Qwen2-shaped model laid out like a mapped weight file."""

    def __init__(self, *, layers, hidden, feed_forward, heads, kv_heads, vocabulary, context, matrix_types, embedding_type=synth.Q8_0,
                 output_type=synth.Q8_0, seed=0, bias=True, session_slots=1, step_tokens=1, rms_epsilon=1e-6, rope_theta=1_000_000.0):
        """``matrix_types``: GGML type ids of (q, k, v, o, gate, up, down)."""
        self.shape = dict(layer_count=layers, hidden=hidden, feed_forward=feed_forward, heads=heads, kv_heads=kv_heads, head_dim=hidden // heads,
                          vocabulary=vocabulary, context=context, session_slots=session_slots, step_tokens=step_tokens, logits_rows=step_tokens,
                          rms_epsilon=rms_epsilon)
        head_dim = hidden // heads
        kv_width = kv_heads * head_dim
        chunks, self._cursor = [], 0

        def put(array):
            data = np.ascontiguousarray(array).view(np.uint8).reshape(-1)
            pad = (-self._cursor) % 32
            if pad:
                chunks.append(np.zeros(pad, np.uint8))
                self._cursor += pad
            offset = self._cursor
            chunks.append(data)
            self._cursor += data.size
            return offset

        rng = synth.rng_for(seed, "decoder")
        norm = lambda: (1.0 + 0.1 * rng.standard_normal(hidden)).astype(np.float32)
        self.embedding_type, self.output_type = embedding_type, output_type
        self.token_embedding = put(synth.matrix(embedding_type, vocabulary, hidden, seed, "token_embd"))
        self.output_norm = put(norm())
        self.output = put(synth.matrix(output_type, vocabulary, hidden, seed, "output"))
        self.layers = (LayerOffsets * layers)()
        shapes = [(hidden, hidden), (kv_width, hidden), (kv_width, hidden), (hidden, hidden), (feed_forward, hidden), (feed_forward, hidden),
                  (hidden, feed_forward)]
        names = ["query", "key", "value", "attention_output", "gate", "up", "down"]
        for l in range(layers):
            entry = self.layers[l]
            entry.attention_norm = put(norm())
            entry.feed_forward_norm = put(norm())
            for name, ggml_type, (rows, columns) in zip(names, matrix_types, shapes):
                setattr(entry, name, put(synth.matrix(ggml_type, rows, columns, seed, f"blk.{l}.{name}")))
            if bias:
                entry.query_bias = put((0.1 * rng.standard_normal(hidden)).astype(np.float32))
                entry.key_bias = put((0.1 * rng.standard_normal(kv_width)).astype(np.float32))
                entry.value_bias = put((0.1 * rng.standard_normal(kv_width)).astype(np.float32))
            else:
                entry.query_bias = entry.key_bias = entry.value_bias = NO_TENSOR
            entry.query_norm = entry.key_norm = NO_TENSOR
            entry.encodings = sum(int(t) << (4 * i) for i, t in enumerate(matrix_types))
        self.weights = np.concatenate(chunks)
        self.cosines, self.sines = rope_tables(head_dim, context, rope_theta)
        self.matrix_bytes = sum(rows * synth.row_bytes(t, cols) for t, (rows, cols) in zip(matrix_types, shapes)) * layers + \
            vocabulary * synth.row_bytes(output_type, hidden)

    def desc(self) -> DecoderDesc:
        d = DecoderDesc()
        d.weights = self.weights.ctypes.data
        d.weights_length = self.weights.size
        d.layers = ctypes.cast(self.layers, POINTER(LayerOffsets))
        d.rope_cosines = self.cosines.ctypes.data_as(POINTER(c_float))
        d.rope_sines = self.sines.ctypes.data_as(POINTER(c_float))
        d.token_embedding, d.output_norm, d.output = self.token_embedding, self.output_norm, self.output
        for key, value in self.shape.items():
            setattr(d, key, value)
        d.embedding_encoding, d.output_encoding = self.embedding_type, self.output_type
        d.rope_layout = d.activation = 0
        d.kv_precision = getattr(self, "kv_precision", 0)  # 0 = FP32 cache, 1 = FP16 (KvPrecision of the reference)
        d.kv_growth_positions = 1024
        return d


class Decoder:
    """Create / forward / destroy of the whole decode step on the current device."""

    def __init__(self, image: ModelImage, lib=None):
        from . import library

        self._lib = lib or library()
        raw = self._lib.raw
        raw.syn_b200_decoder_create.restype = c_int32
        raw.syn_b200_decoder_create.argtypes = [POINTER(DecoderDesc), POINTER(c_void_p)]
        raw.syn_b200_decoder_forward.restype = c_int32
        raw.syn_b200_decoder_forward.argtypes = [c_void_p, POINTER(BatchToken), c_uint64, c_void_p, c_uint64]
        raw.syn_b200_decoder_forward_argmax.restype = c_int32
        raw.syn_b200_decoder_forward_argmax.argtypes = [c_void_p, POINTER(BatchToken), c_uint64, c_void_p]
        raw.syn_b200_decoder_destroy.restype = None
        raw.syn_b200_decoder_destroy.argtypes = [c_void_p]
        raw.syn_b200_decoder_kv_bytes.restype = c_uint64
        raw.syn_b200_decoder_kv_bytes.argtypes = [c_void_p]
        self.image = image
        self._handle = c_void_p()
        desc = image.desc()
        self._lib.check(raw.syn_b200_decoder_create(byref(desc), byref(self._handle)))
        self.vocabulary = image.shape["vocabulary"]

    def close(self):
        if getattr(self, "_handle", None):
            self._lib.raw.syn_b200_decoder_destroy(self._handle)
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

    @staticmethod
    def _batch(tokens):
        batch = (BatchToken * len(tokens))()
        for i, (slot, token, position, logits_row) in enumerate(tokens):
            batch[i] = BatchToken(slot, token, position, logits_row)
        return batch

    def forward(self, tokens) -> np.ndarray:
        """``tokens``: (slot, token, position, logits_row) tuples. Returns [logits rows, vocabulary] FP32."""
        rows = sum(1 for t in tokens if t[3] >= 0)
        logits = np.empty((max(rows, 1), self.vocabulary), np.float32)
        self._lib.check(self._lib.raw.syn_b200_decoder_forward(self._handle, self._batch(tokens), len(tokens), logits.ctypes.data, logits.size))
        return logits[:rows]

    def forward_argmax(self, tokens) -> list[int]:
        rows = sum(1 for t in tokens if t[3] >= 0)
        out = np.zeros(max(rows, 1), np.int32)
        self._lib.check(self._lib.raw.syn_b200_decoder_forward_argmax(self._handle, self._batch(tokens), len(tokens), out.ctypes.data))
        return out[:rows].tolist()

    def decode(self, token: int, position: int, slot: int = 0) -> np.ndarray:
        """One token at one position, logits back (``IDecoderExecutor.Decode``)."""
        return self.forward([(slot, token, position, 0)])[0]

    def kv_bytes(self) -> int:
        return int(self._lib.raw.syn_b200_decoder_kv_bytes(self._handle))


# Shapes of the benchmark configs.
QWEN25_05B = dict(layers=24, hidden=896, feed_forward=4864, heads=14, kv_heads=2, vocabulary=151936)
QWEN25_7B = dict(layers=28, hidden=3584, feed_forward=18944, heads=28, kv_heads=4, vocabulary=152064)
Q8_TYPES = (synth.Q8_0,) * 7
Q4KM_TYPES = (synth.Q4_K, synth.Q4_K, synth.Q6_K, synth.Q4_K, synth.Q4_K, synth.Q4_K, synth.Q6_K)
