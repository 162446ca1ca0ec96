"""The allocation-free entry point, checked against the ordinary device entry point.

Some callers of this library cannot call cudaMalloc at the moment they need a product: a decode thread that may not
block on the allocator, a plugin living inside a fixed memory budget, code that runs in a CUDA context it does not
own. syn_b200_matvec_static serves them from a scratch array built into the library. This test calls it through the
C ABI twice in a row on the same buffers and expects both results to equal syn_b200_matvec_dev's (same kernels, same
arithmetic, so the usual parity tolerance 1e-3 relative / 1e-5 absolute is far from being needed). The file sorts
last so that a run that stops at the first failure has already run everything else.
"""
import numpy as np
import pytest

import synapse_b200 as sb
from synapse_b200 import synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("ggml_type,rows,columns,tokens", [(sb.Q4_K, 512, 3584, 1), (sb.Q6_K, 300, 1024, 2), (sb.Q8_0, 128, 896, 5)])
def test_static_scratch_entry_point_matches_the_ordinary_one(ggml_type, rows, columns, tokens):
    import torch

    lib = sb.library()
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    weights = synth.matrix(ggml_type, rows, columns, seed=71)
    x = torch.from_numpy(synth.activations(tokens, columns, seed=72)).to(device)
    scratch_bytes = lib.activation_scratch_bytes(tokens, columns)
    scratch = torch.empty(scratch_bytes + 256, dtype=torch.uint8, device=device)
    scratch_ptr = (scratch.data_ptr() + 255) // 256 * 256
    want = torch.zeros(tokens, rows, dtype=torch.float32, device=device)
    with sb.QuantizedMatrix(weights, ggml_type, rows, columns) as matrix:
        matrix.matvec_device(x.data_ptr(), tokens, columns, want.data_ptr(), rows, sb.MODE_XQ8, scratch_ptr=scratch_ptr, scratch_bytes=scratch_bytes)
        torch.cuda.synchronize()
        expected = want.cpu().numpy()
        assert np.abs(expected).max() > 0
        for call in range(2):
            got = torch.full((tokens, rows), float("nan"), dtype=torch.float32, device=device)
            matrix.matvec_static(x.data_ptr(), tokens, columns, got.data_ptr(), rows)
            torch.cuda.synchronize()
            result = got.cpu().numpy()
            assert np.all(np.abs(result - expected) <= 1e-5 + 1e-3 * np.abs(expected)), f"call {call}: max difference {np.abs(result - expected).max()}"
        # a second input through the same array: the previous contents must not leak into the result
        x2 = torch.from_numpy(synth.activations(tokens, columns, seed=73)).to(device)
        matrix.matvec_device(x2.data_ptr(), tokens, columns, want.data_ptr(), rows, sb.MODE_XQ8, scratch_ptr=scratch_ptr, scratch_bytes=scratch_bytes)
        got = torch.zeros(tokens, rows, dtype=torch.float32, device=device)
        matrix.matvec_static(x2.data_ptr(), tokens, columns, got.data_ptr(), rows)
        torch.cuda.synchronize()
        expected2, result2 = want.cpu().numpy(), got.cpu().numpy()
        assert np.all(np.abs(result2 - expected2) <= 1e-5 + 1e-3 * np.abs(expected2))
        assert lib.device_faults() == 0


def test_static_scratch_entry_point_rejects_what_does_not_fit():
    import torch

    lib = sb.library()
    torch.cuda.set_device(0)
    capacity = int(lib.raw.syn_b200_matvec_static_capacity())
    assert capacity == 8 * 32768
    columns = 8192
    tokens = capacity // columns + 1
    weights = synth.matrix(sb.Q4_K, 16, columns, seed=74)
    x = torch.zeros(tokens, columns, dtype=torch.float32, device="cuda")
    y = torch.zeros(tokens, 16, dtype=torch.float32, device="cuda")
    with sb.QuantizedMatrix(weights, sb.Q4_K, 16, columns) as matrix:
        status = lib.raw.syn_b200_matvec_static(matrix.handle, 0, 16, x.data_ptr(), tokens, columns, y.data_ptr(), 16, 0, None)
        assert status == 2 and "exceed the built-in scratch" in lib.last_error()
        assert lib.raw.syn_b200_matvec_static(matrix.handle, 0, 16, x.data_ptr(), tokens - 1, columns, y.data_ptr(), 16, 0, None) == 0
        assert lib.raw.syn_b200_matvec_static(None, 0, 16, x.data_ptr(), 1, columns, y.data_ptr(), 16, 0, None) == 1
        torch.cuda.synchronize()
