"""The allocation-free entry point, checked against the CPU oracle and against the ordinary device entry point.

Some callers of this library cannot call cudaMalloc at the moment they need a product: a decode thread that may not
block on the allocator, a plugin living inside a fixed memory budget, code that runs in a CUDA context it does not
own. syn_b200_matvec_static serves them from a scratch array built into the library. This test calls it through the
C ABI twice in a row on the same buffers and expects both results to match the quantised-activation oracle within the
usual parity gate (1e-3 relative / 1e-5 absolute, see parity.py) and to equal syn_b200_matvec_dev's bit for bit (same
kernels, same arithmetic); it then repeats the comparison on a row range with the residual-add epilogue and on a call
that fills the array to its last value. The file sorts last so that a run that stops at the first failure has already
run everything else.
"""
import numpy as np
import pytest

import synapse_b200 as sb
from synapse_b200 import synth
from parity import assert_parity

pytestmark = pytest.mark.gpu


def _scratch(lib, tokens, columns, device):
    import torch

    size = lib.activation_scratch_bytes(tokens, columns)
    buffer = torch.empty(size + 256, dtype=torch.uint8, device=device)
    return buffer, (buffer.data_ptr() + 255) // 256 * 256, size


@pytest.mark.parametrize("ggml_type,rows,columns,tokens", [(sb.Q4_K, 512, 3584, 1), (sb.Q6_K, 300, 1024, 2), (sb.Q8_0, 128, 896, 5)])
def test_static_scratch_entry_point_matches_the_oracle_and_the_ordinary_entry_point(oracle, ggml_type, rows, columns, tokens):
    import torch

    lib = sb.library()
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    weights = synth.matrix(ggml_type, rows, columns, seed=71)
    with sb.QuantizedMatrix(weights, ggml_type, rows, columns) as matrix:
        for seed in (72, 73):  # a second input through the same array: the previous contents must not leak into the result
            x_host = synth.activations(tokens, columns, seed=seed)
            codes, scales = oracle.quantize(x_host)
            want = oracle.kq_q8_matmul(ggml_type, weights, rows, columns, codes, scales)
            exact, magnitude = oracle.kq_q8_exact(ggml_type, weights, rows, columns, codes, scales)
            x = torch.from_numpy(x_host).to(device)
            keep, scratch_ptr, scratch_bytes = _scratch(lib, tokens, columns, device)
            ordinary = torch.zeros(tokens, rows, dtype=torch.float32, device=device)
            matrix.matvec_device(x.data_ptr(), tokens, columns, ordinary.data_ptr(), rows, sb.MODE_XQ8, scratch_ptr=scratch_ptr,
                                 scratch_bytes=scratch_bytes)
            for call in range(2):
                got = torch.full((tokens, rows), float("nan"), dtype=torch.float32, device=device)
                matrix.matvec_static(x.data_ptr(), tokens, columns, got.data_ptr(), rows)
                torch.cuda.synchronize()
                assert_parity(got.cpu().numpy(), want, exact, magnitude, f"input {seed}, call {call}")
                assert torch.equal(got, ordinary), f"input {seed}, call {call}: differs from syn_b200_matvec_dev"
        # a row range with the residual-add epilogue
        first, count = 17, min(rows - 17, 100)
        residual = synth.activations(tokens, count, seed=74)
        got = torch.from_numpy(residual.copy()).to(device)
        matrix.matvec_static(x.data_ptr(), tokens, columns, got.data_ptr(), count, epilogue=sb.EPILOGUE_ACCUMULATE, row_start=first, row_count=count)
        torch.cuda.synchronize()
        assert np.array_equal(got.cpu().numpy(), residual + ordinary.cpu().numpy()[:, first:first + count])
        assert lib.device_faults() == 0


def test_static_scratch_entry_point_at_and_beyond_its_capacity(oracle):
    import torch

    lib = sb.library()
    torch.cuda.set_device(0)
    capacity = int(lib.raw.syn_b200_matvec_static_capacity())
    assert capacity == 8 * 32768
    columns, rows = 8192, 16
    tokens = capacity // columns  # fills the array to its last value
    weights = synth.matrix(sb.Q4_K, rows, columns, seed=75)
    x_host = synth.activations(tokens + 1, columns, seed=76)
    x = torch.from_numpy(x_host).cuda()
    y = torch.zeros(tokens + 1, rows, dtype=torch.float32, device="cuda")
    with sb.QuantizedMatrix(weights, sb.Q4_K, rows, columns) as matrix:
        status = lib.raw.syn_b200_matvec_static(matrix.handle, 0, rows, x.data_ptr(), tokens + 1, columns, y.data_ptr(), rows, 0, None)
        assert status == 2 and "exceed the built-in scratch" in lib.last_error()
        assert lib.raw.syn_b200_matvec_static(matrix.handle, 0, rows, x.data_ptr(), tokens, columns, y.data_ptr(), rows, 0, None) == 0
        assert lib.raw.syn_b200_matvec_static(None, 0, rows, x.data_ptr(), 1, columns, y.data_ptr(), rows, 0, None) == 1
        torch.cuda.synchronize()
        codes, scales = oracle.quantize(x_host[:tokens])
        want = oracle.kq_q8_matmul(sb.Q4_K, weights, rows, columns, codes, scales)
        exact, magnitude = oracle.kq_q8_exact(sb.Q4_K, weights, rows, columns, codes, scales)
        assert_parity(y.cpu().numpy()[:tokens], want, exact, magnitude, "at capacity")
        assert not y.cpu().numpy()[tokens].any(), "the rejected call wrote output"
    assert lib.device_faults() == 0
