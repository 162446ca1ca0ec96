"""The C-ABI library loads, exports every declared symbol and validates arguments before touching a device."""
import ctypes
import os
import re

import numpy as np
import pytest

import synapse_b200 as sb

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from synapse_b200 import build

    build.build()
    return sb.NativeB200Library.load_from_package_directory()


def test_every_declared_symbol_is_exported(lib):
    header = open(os.path.join(ROOT, "include", "synapse_b200.h")).read()
    declared = sorted(set(re.findall(r"\b(syn_b200_[a-z0-9_]+)\s*\(", header)))
    assert declared == sb.exported_symbols()
    for name in declared:
        assert hasattr(lib.raw, name), name


def test_abi_version_is_checked_first(lib):
    assert lib.abi_version == sb.EXPECTED_ABI_VERSION == 1


def test_missing_library_is_reported_as_unavailable(tmp_path):
    with pytest.raises(sb.BackendUnavailableError, match="library file is missing"):
        sb.NativeB200Library.load(str(tmp_path))
    with pytest.raises(ValueError):
        sb.NativeB200Library.load("  ")


def test_device_info_struct_matches_the_reference_size():
    assert ctypes.sizeof(sb.DeviceInfo) == 152


def test_null_pointers_return_status_1_and_a_message(lib):
    raw = lib.raw
    assert raw.syn_b200_probe(None) == 1
    assert "null pointer" in lib.last_error()
    handle = ctypes.c_void_p()
    assert raw.syn_b200_matrix_create(None, 8, 4, 32, 0, ctypes.byref(handle)) == 1
    assert raw.syn_b200_matvec(None, 0, 1, None, 1, 32, None, 1, 0, 0) == 1
    assert raw.syn_b200_matmul_q8(None, 0, 1, None, None, 1, None, 1) == 1
    assert raw.syn_b200_quantize_q8(None, 1, 32, 32, None, None) == 1
    raw.syn_b200_matrix_destroy(None)  # ignored


def test_last_error_reports_full_length_and_truncates(lib):
    lib.raw.syn_b200_probe(None)
    full = lib.raw.syn_b200_last_error(None, 0)
    assert full > 4
    buffer = ctypes.create_string_buffer(4)
    assert lib.raw.syn_b200_last_error(ctypes.cast(buffer, ctypes.c_void_p), 4) == full
    assert buffer.raw == lib.last_error().encode()[:4]


def test_shapes_are_validated_before_any_device_work(lib):
    blocks = np.zeros(34 * 8, np.uint8)
    handle = ctypes.c_void_p()
    create = lib.raw.syn_b200_matrix_create
    assert create(blocks.ctypes.data, 99, 4, 32, 0, ctypes.byref(handle)) == 2  # unknown type
    assert create(blocks.ctypes.data, 8, 0, 32, 0, ctypes.byref(handle)) == 2  # zero rows
    assert create(blocks.ctypes.data, 8, 4, 32, 2, ctypes.byref(handle)) == 2  # unknown flag
    assert create(blocks.ctypes.data, 8, 2**63, 2**40, 0, ctypes.byref(handle)) == 2  # overflow
    # ragged width: the reference reports such tensors as unavailable (decoder/checks.rs:185-190)
    assert create(blocks.ctypes.data, 12, 4, 300, 0, ctypes.byref(handle)) == 3
    assert "multiple of its 256-value blocks" in lib.last_error()
    assert not handle.value
    x = np.zeros(33, np.float32)
    assert lib.raw.syn_b200_quantize_q8(x.ctypes.data, 1, 33, 33, x.ctypes.data, x.ctypes.data) == 2


@pytest.mark.parametrize("ggml_type,block_bytes,offsets", [(8, 34, (0,)), (12, 144, (0, 2)), (14, 210, (208,))])
def test_blocks_with_a_non_finite_scale_are_refused_at_load(lib, ggml_type, block_bytes, offsets):
    """BlockSourceDecoder.Decode (src/Synapse.Runtime/Features/ModelPackages/SourceFormats/SourceTensorDecoders.cs:134-146,
    161-172) validates every block's fp16 fields before decoding; the loader does the same before any device work and
    names the first offending block."""
    from synapse_b200 import synth

    rows, columns = 3, 512
    good = synth.matrix(ggml_type, rows, columns, seed=9)
    blocks_per_row = columns // sb.BLOCK_VALUES[ggml_type]
    handle = ctypes.c_void_p()
    for offset in offsets:
        for bits in (0x7C00, 0xFC00, 0x7E01):  # +inf, -inf, a NaN
            bad = good.copy()
            block = blocks_per_row + 1  # second block of the second row
            bad[block * block_bytes + offset] = bits & 0xFF
            bad[block * block_bytes + offset + 1] = bits >> 8
            assert lib.raw.syn_b200_matrix_create(bad.ctypes.data, ggml_type, rows, columns, 0, ctypes.byref(handle)) == 2
            assert f"block {block} fails validation: InvalidScale" in lib.last_error()
            assert not handle.value
    # the largest finite half is fine: the call gets as far as looking for a device
    edge = good.copy()
    edge[offsets[0]], edge[offsets[0] + 1] = 0xFF, 0x7B
    status = lib.raw.syn_b200_matrix_create(edge.ctypes.data, ggml_type, rows, columns, 0, ctypes.byref(handle))
    assert status in (0, 3)
    if status == 0:
        lib.raw.syn_b200_matrix_destroy(handle)


def test_host_wrappers_reject_bad_arguments_without_a_device():
    with pytest.raises(ValueError):
        sb.Q8ActivationBuffer(33)
    with pytest.raises(ValueError):
        sb.quantize_row(np.zeros(48, np.float32))


def test_without_a_b200_calls_fail_loudly_not_silently(lib):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    with pytest.raises(sb.BackendUnavailableError):
        lib.probe()
    with pytest.raises(sb.BackendUnavailableError):
        sb.QuantizedMatrix(np.zeros(34 * 4, np.uint8), sb.Q8_0, 4, 32)
    with pytest.raises(sb.BackendUnavailableError):
        sb.quantize_row(np.zeros(32, np.float32))


def test_scratch_sizes_are_plain_arithmetic(lib):
    """The scratch queries need no device: the activation scratch of the quantised products (codes, scales, sums per 16, each
    rounded up to 256 bytes) and the tensor-core product's scratch (two sets of 16-bit activation tiles of 128 tokens x 64
    values, plus the fixed room in which small products split along k)."""
    assert lib.activation_scratch_bytes(1, 3584) == 4608  # codes at 0 (3584), 112 scales at 3584 (448), 224 sums at 4096 (448), end rounded up
    tiles = lambda tokens, columns: 2 * (-(-tokens // 128) * (columns // 64) * 16384)
    split_room = lib.gemm_scratch_bytes(1, 64) - tiles(1, 64)
    assert split_room == 160 * 2 * 128 * 128 * 4 + 4 * 80
    for tokens, columns in ((128, 3584), (129, 3584), (4096, 18944)):
        assert lib.gemm_scratch_bytes(tokens, columns) == tiles(tokens, columns) + split_room
