"""Matrices loaded tensor by tensor from a GGUF file by the native loader, with and without the persisted repack."""
import os

import numpy as np
import pytest

import synapse_b200 as sb
from synapse_b200 import synth
from gguf_fixture import sample_tensors, write_gguf

pytestmark = pytest.mark.gpu


def test_matrices_loaded_from_a_file_equal_matrices_built_from_the_same_bytes(tmp_path, oracle):
    path = str(tmp_path / "model.gguf")
    tensors = sample_tensors()
    write_gguf(path, tensors)
    cache = tmp_path / "cache"
    cache.mkdir()
    with sb.GgufFile(path) as file:
        for name, ggml_type, dimensions, data in tensors[1:]:
            columns, rows = dimensions
            x = synth.activations(2, columns, seed=5)
            blocks = np.frombuffer(bytes(data), np.uint8)
            with sb.QuantizedMatrix(blocks, ggml_type, rows, columns) as direct:
                want = direct.matvec(x, sb.MODE_XQ8)
            codes, scales = oracle.quantize(x)
            assert np.allclose(want, oracle.kq_q8_matmul(ggml_type, blocks, rows, columns, codes, scales), rtol=1e-3, atol=1e-4)
            for round_trip in range(2):  # the first load writes the cache entry of a repacked matrix, the second reads it
                with file.load_matrix(name, cache_directory=str(cache)) as loaded:
                    assert (loaded.rows, loaded.columns, loaded.ggml_type) == (rows, columns, ggml_type)
                    assert loaded.matvec(x, sb.MODE_XQ8).tobytes() == want.tobytes()
            # the file layout walks a row in other units than the planar one, so only the values agree, not the bits
            with file.load_matrix(name, repack=False) as natural, sb.QuantizedMatrix(blocks, ggml_type, rows, columns, repack=False) as reference:
                assert natural.matvec(x, sb.MODE_XQ8).tobytes() == reference.matvec(x, sb.MODE_XQ8).tobytes()
                assert np.allclose(natural.matvec(x, sb.MODE_XQ8), want, rtol=1e-3, atol=1e-4)
        entries = sorted(os.listdir(cache))
        assert len(entries) == 3 and all(e.endswith(".synb200") for e in entries)  # Q6_K, Q8_0, Q6_K: Q4_K keeps its file layout
        # a cache entry of another file (same name, other bytes) is not taken: the digest covers the header and the length
        other = str(tmp_path / "other.gguf")
        changed = [(n, t, d, bytes(reversed(bytes(b))) if n == "output.weight" else b) for n, t, d, b in tensors] + [("extra", 0, [4], bytes(16))]
        write_gguf(other, changed)
        with sb.GgufFile(other) as second:
            with second.load_matrix("blk.0.attn_v.weight", cache_directory=str(cache)) as loaded:
                assert loaded.rows == 40
        assert len(os.listdir(cache)) == 4
        with pytest.raises(sb.KernelError, match="not a two-dimensional"):
            file.load_matrix("blk.0.attn_norm.weight")
    assert sb.library().device_faults() == 0
