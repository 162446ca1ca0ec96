"""The native GGUF tensor-table reader against files written by the test (no GPU): same table, same failure rules as
the reference's header reader (src/Synapse.Runtime/Features/ModelLoading/Gguf/GgufHeaderReader.cs:20-154; its tests:
tests/Synapse.IntegrationTests/Features/ModelLoading)."""
import os
import struct

import numpy as np
import pytest

import synapse_b200 as sb
from gguf_fixture import sample_tensors, write_gguf


@pytest.fixture(scope="module")
def lib():
    from synapse_b200 import build

    build.build()
    return sb.NativeB200Library.load_from_package_directory()


@pytest.mark.parametrize("version,alignment", [(3, None), (2, 64), (3, 4096)])
def test_tensor_table_matches_what_was_written(lib, tmp_path, version, alignment):
    path = str(tmp_path / "model.gguf")
    tensors = sample_tensors()
    absolute, data_offset = write_gguf(path, tensors, version=version, alignment=alignment)
    with sb.GgufFile(path, lib) as file:
        table = file.tensors()
        assert [t.name.decode() for t in table] == [t[0] for t in tensors]
        assert file.data_offset() == data_offset and data_offset % (alignment or 32) == 0
        for entry, (name, ggml_type, dimensions, data) in zip(table, tensors):
            assert (entry.ggml_type, entry.rank, list(entry.dimensions)[:entry.rank]) == (ggml_type, len(dimensions), dimensions)
            assert entry.offset == absolute[name] and entry.bytes == len(data)
            assert open(path, "rb").read()[entry.offset:entry.offset + entry.bytes] == bytes(data)
        assert file.find("output.weight").bytes == 130 * 3 * 210
        with pytest.raises(sb.KernelError, match="has no tensor"):
            file.find("missing.weight")
    # an independent reader of the same container agrees on the table
    gguf = pytest.importorskip("gguf")
    reader = gguf.GGUFReader(path)
    assert [t.name for t in reader.tensors] == [t[0] for t in tensors]
    assert [int(t.data_offset) for t in reader.tensors] == [absolute[t[0]] for t in tensors]


def _expect(lib, path, status, text):
    handle = __import__("ctypes").c_void_p()
    assert lib.raw.syn_b200_gguf_open(os.fsencode(path), __import__("ctypes").byref(handle)) == status
    assert text in lib.last_error(), lib.last_error()
    assert not handle.value


def test_malformed_files_are_refused_like_the_reference_does(lib, tmp_path):
    good = str(tmp_path / "good.gguf")
    tensors = sample_tensors()
    write_gguf(good, tensors)
    blob = bytearray(open(good, "rb").read())

    def variant(name, edit):
        data = bytearray(blob)
        edit(data)
        path = str(tmp_path / name)
        open(path, "wb").write(data)
        return path

    _expect(lib, variant("magic.gguf", lambda d: d.__setitem__(slice(0, 4), b"GGML")), 2, "not a GGUF model")
    _expect(lib, variant("version.gguf", lambda d: d.__setitem__(slice(4, 8), struct.pack("<I", 1))), 2, "version 1 is not supported")
    _expect(lib, variant("count.gguf", lambda d: d.__setitem__(slice(8, 16), struct.pack("<Q", 2_000_000))), 2, "exceeds the limit")
    _expect(lib, variant("short.gguf", lambda d: d.__delitem__(slice(200, len(d)))), 2, "truncated")
    _expect(lib, variant("tail.gguf", lambda d: d.__delitem__(slice(len(d) - 100, len(d)))), 2, "outside the GGUF file")
    _expect(lib, str(tmp_path / "absent.gguf"), 2, "cannot open")
    write_gguf(str(tmp_path / "alignment.gguf"), tensors, alignment=48)
    _expect(lib, str(tmp_path / "alignment.gguf"), 2, "alignment 48 is invalid")
    write_gguf(str(tmp_path / "type.gguf"), [("w", 2, [32, 4], bytes(4 * 18))])  # Q4_0: a GGML type the backend does not execute
    _expect(lib, str(tmp_path / "type.gguf"), 3, "unsupported GGML type 2")
    write_gguf(str(tmp_path / "rank.gguf"), [("w", 0, [], bytes(4))])
    _expect(lib, str(tmp_path / "rank.gguf"), 2, "invalid rank 0")
    write_gguf(str(tmp_path / "ragged.gguf"), [("w", 12, [100, 4], bytes(1000))])
    _expect(lib, str(tmp_path / "ragged.gguf"), 3, "unsupported GGML type 12")  # 400 values are not whole Q4_K blocks: the reference's switch falls through
    assert lib.raw.syn_b200_gguf_open(None, None) == 1
    lib.raw.syn_b200_gguf_close(None)
