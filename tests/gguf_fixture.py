"""Writes small GGUF files for the loader tests: the public container format (magic, version, counts, metadata key/values,
tensor infos, aligned data section) with seeded synthetic blocks as tensor data. No model file is read or needed."""
import struct

import numpy as np

from synapse_b200 import synth


def _string(text):
    raw = text.encode()
    return struct.pack("<Q", len(raw)) + raw


def write_gguf(path, tensors, version=3, alignment=None, metadata=()):
    """``tensors``: list of (name, ggml_type, dimensions (row length first), bytes). Returns {name: absolute offset}."""
    entries = [("general.architecture", 8, "qwen2"), ("qwen2.block_count", 4, 2)] + list(metadata)
    if alignment is not None:
        entries.append(("general.alignment", 4, alignment))
    # an array of strings and an array of integers, as tokenizer metadata has
    body = struct.pack("<IIQQ", 0x46554747, version, len(tensors), len(entries) + 2)
    for key, kind, value in entries:
        body += _string(key) + struct.pack("<I", kind)
        body += _string(value) if kind == 8 else struct.pack({4: "<I", 5: "<i", 10: "<Q", 6: "<f"}[kind], value)
    body += _string("tokenizer.ggml.tokens") + struct.pack("<IIQ", 9, 8, 3) + b"".join(_string(t) for t in ("a", "bc", "def"))
    body += _string("tokenizer.ggml.token_type") + struct.pack("<IIQ", 9, 5, 4) + struct.pack("<4i", 1, 2, 3, 4)
    align = alignment or 32
    relative, offsets = 0, []
    for name, ggml_type, dimensions, data in tensors:
        body += _string(name) + struct.pack("<I", len(dimensions)) + b"".join(struct.pack("<Q", d) for d in dimensions)
        body += struct.pack("<IQ", ggml_type, relative)
        offsets.append(relative)
        relative += (len(data) + align - 1) // align * align
    data_offset = (len(body) + align - 1) // align * align
    blob = bytearray(body) + bytearray(data_offset - len(body))
    absolute = {}
    for (name, _, _, data), offset in zip(tensors, offsets):
        blob += bytearray(data_offset + offset - len(blob))
        absolute[name] = len(blob)
        blob += bytes(data)
    with open(path, "wb") as handle:
        handle.write(blob)
    return absolute, data_offset


def sample_tensors():
    """A handful of tensors shaped like a model file's: FP32 norms and matrices of every accepted encoding."""
    out = [("blk.0.attn_norm.weight", 0, [256], np.arange(256, dtype=np.float32).tobytes())]
    for name, ggml_type, rows, columns in (("blk.0.attn_q.weight", synth.Q4_K, 48, 512), ("blk.0.attn_v.weight", synth.Q6_K, 40, 256),
                                           ("blk.0.ffn_down.weight", synth.Q8_0, 33, 96), ("output.weight", synth.Q6_K, 130, 768)):
        out.append((name, ggml_type, [columns, rows], synth.matrix(ggml_type, rows, columns, seed=11, name=name).tobytes()))
    return out
