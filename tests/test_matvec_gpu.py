"""GPU parity of the decode matrix-vector path, through the C ABI, against the CPU oracle and the golden vectors."""
import os

import numpy as np
import pytest

import synapse_b200 as sb
from synapse_b200 import synth
from parity import assert_parity

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "matvec_cases.npz")
CASE_NAMES = ["q8_0_a", "q8_0_b", "q4_k_a", "q4_k_b", "q6_k_a", "q6_k_b"]
SENTINEL = np.float32(12345.0)


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


def _buffer(codes, scales):
    tokens, columns = codes.shape
    buffer = sb.Q8ActivationBuffer(columns, tokens)
    buffer.quants[:] = codes
    buffer.scales[:] = scales
    return buffer


@pytest.mark.parametrize("name", CASE_NAMES)
@pytest.mark.parametrize("repack", [True, False])
def test_golden_vectors(golden, oracle, name, repack):
    ggml_type, rows, columns, tokens = (int(v) for v in golden[f"{name}.meta"])
    weights, x = golden[f"{name}.weights"], golden[f"{name}.x"]
    codes, scales = golden[f"{name}.codes"], golden[f"{name}.scales"]
    with sb.QuantizedMatrix(weights, ggml_type, rows, columns, repack=repack) as matrix:
        # the activation quantiser is bit-exact
        got_codes, got_scales = sb.quantize_row(x)
        assert np.array_equal(got_codes, codes)
        assert got_scales.tobytes() == scales.tobytes()
        # integer sub-block dots are bit-exact
        assert np.array_equal(matrix.block_dots(codes), golden[f"{name}.dots"])
        # quantised-activation product, pre-quantised and quantised in the library
        exact, magnitude = oracle.kq_q8_exact(ggml_type, weights, rows, columns, codes, scales)
        y = matrix.multiply(0, rows, _buffer(codes, scales), tokens).reshape(tokens, rows)
        assert_parity(y, golden[f"{name}.y_xq8"], exact, magnitude, f"{name} xq8")
        y2 = matrix.matvec(x, sb.MODE_XQ8)
        assert y2.tobytes() == y.tobytes()
        # FP32-activation product (the reference backend's contract)
        exact, magnitude = oracle.f32_exact(ggml_type, weights, rows, columns, x)
        assert_parity(matrix.matvec(x, sb.MODE_XF32), golden[f"{name}.y_xf32"], exact, magnitude, f"{name} xf32")


LCG_CASES = [(37, 28, 1, 37, 1), (16, 152, 3, 20, 2), (5, 64, 2, 9, 3), (8, 63, 4, 11, 4)]


@pytest.mark.parametrize("rows,blocks,tokens,stride,seed", LCG_CASES)
@pytest.mark.parametrize("repack", [True, False])
def test_reference_kernel_cases(oracle, rows, blocks, tokens, stride, seed, repack):
    # native/synapse-kernels/tests/Features/CpuKernels/q8_0_tests.rs:133-166: same seeds, tolerance and sentinel check
    weights, quants, scales = oracle.lcg_case(seed, rows, blocks, tokens)
    buffer = _buffer(quants.reshape(tokens, -1), scales.reshape(tokens, -1))
    output = np.full((tokens - 1) * stride + rows, SENTINEL, np.float32)
    with sb.QuantizedMatrix(weights, sb.Q8_0, rows, blocks * 32, repack=repack) as matrix:
        matrix.multiply(0, rows, buffer, tokens, output, stride)
        dots = matrix.block_dots(quants)
    exact, magnitude = oracle.q8q8_exact(weights, rows, blocks, quants, scales, tokens)
    for t in range(tokens):
        got = output[t * stride: t * stride + rows].astype(np.float64)
        assert np.all(np.abs(got - exact[t]) <= 2e-5 * magnitude[t] + 1e-12)
        if t + 1 < tokens:
            assert np.all(output[t * stride + rows: (t + 1) * stride].view(np.uint32) == SENTINEL.view(np.uint32)), "stride gap was written"
    assert np.array_equal(dots, oracle.q8q8_block_dots(weights, rows, blocks, quants, tokens))


SHAPES = [  # type, rows, columns: the benchmark configs' shapes at sizes the oracle finishes in seconds
    (sb.Q8_0, 4864, 896), (sb.Q8_0, 896, 4864), (sb.Q8_0, 128, 896),
    (sb.Q4_K, 3584, 3584), (sb.Q4_K, 512, 3584), (sb.Q4_K, 1024, 8192), (sb.Q4_K, 300, 28672),
    (sb.Q6_K, 512, 3584), (sb.Q6_K, 640, 18944), (sb.Q6_K, 3, 256), (sb.Q4_K, 1, 256), (sb.Q8_0, 1, 32),
]


@pytest.mark.parametrize("ggml_type,rows,columns", SHAPES)
@pytest.mark.parametrize("tokens", [1, 2, 3, 4, 8])
def test_config_shapes_against_the_oracle(oracle, ggml_type, rows, columns, tokens):
    weights = synth.matrix(ggml_type, rows, columns, seed=7)
    x = synth.activations(tokens, columns, seed=8)
    codes, scales = oracle.quantize(x)
    with sb.QuantizedMatrix(weights, ggml_type, rows, columns) as matrix:
        y = matrix.matvec(x, sb.MODE_XQ8)
        exact, magnitude = oracle.kq_q8_exact(ggml_type, weights, rows, columns, codes, scales)
        assert_parity(y, oracle.kq_q8_matmul(ggml_type, weights, rows, columns, codes, scales), exact, magnitude, "xq8")
        if tokens <= 4:  # the token counts the FP32-activation matrix-vector kernels take (step/projection.rs:51-72)
            yf = matrix.matvec(x, sb.MODE_XF32)
            exact, magnitude = oracle.f32_exact(ggml_type, weights, rows, columns, x)
            assert_parity(yf, oracle.f32_matmul_threads(ggml_type, weights, rows, columns, x, 8), exact, magnitude, "xf32")
        if rows <= 512:
            assert np.array_equal(matrix.block_dots(codes[:1]), oracle.int_dots(ggml_type, weights, rows, columns, codes[:1]))


@pytest.mark.parametrize("ggml_type", [sb.Q8_0, sb.Q4_K, sb.Q6_K])
def test_row_ranges_strides_and_accumulate(oracle, ggml_type):
    rows, columns, tokens = 100, 768 if ggml_type != sb.Q8_0 else 96, 3
    weights = synth.matrix(ggml_type, rows, columns, seed=21)
    x = synth.activations(tokens, columns, seed=22)
    codes, scales = oracle.quantize(x)
    want = oracle.kq_q8_matmul(ggml_type, weights, rows, columns, codes, scales)
    with sb.QuantizedMatrix(weights, ggml_type, rows, columns) as matrix:
        full = matrix.matvec(x, sb.MODE_XQ8)
        part = matrix.matvec(x, sb.MODE_XQ8, row_start=17, row_count=30)
        assert part.tobytes() == np.ascontiguousarray(full[:, 17:47]).tobytes()  # row chunks do not change a row's value
        strided = np.full((tokens, 40), SENTINEL, np.float32)
        matrix.matvec(x, sb.MODE_XQ8, row_start=17, row_count=30, output=strided, output_stride=40)
        assert strided[:, :30].tobytes() == part.tobytes() and np.all(strided[:, 30:] == SENTINEL)
        residual = synth.activations(tokens, rows, seed=23).copy()
        accumulated = residual.copy()
        matrix.matvec(x, sb.MODE_XQ8, epilogue=sb.EPILOGUE_ACCUMULATE, output=accumulated)
        assert np.array_equal(accumulated, residual + full)
        assert np.allclose(full, want, rtol=1e-3, atol=1e-4)


def test_tokens_are_batch_invariant(oracle):
    # tests/Synapse.IntegrationTests/Features/CpuKernels/OptimizedQwen2Tests.cs:41-54: a token's result does not
    # depend on how many tokens share the weight pass.
    rows, columns = 256, 1024
    weights = synth.matrix(sb.Q4_K, rows, columns, seed=31)
    x = synth.activations(8, columns, seed=32)
    with sb.QuantizedMatrix(weights, sb.Q4_K, rows, columns) as matrix:
        together = matrix.matvec(x, sb.MODE_XQ8)
        for t in range(8):
            assert matrix.matvec(x[t:t + 1], sb.MODE_XQ8).tobytes() == together[t:t + 1].tobytes()


# type, rows, columns. Q4_K: one-warp teams (28 units), ragged rows, two / five / seven team warps (the last ones partly
# filled), the shortest row there is, and row lengths whose activations fit shared memory only for four or two tokens at
# a time. Q6_K: one and two units per lane, second steps that are partly filled (3584: 24 of 32 lanes; 2304: 4; 18944:
# five team warps, the last with 32 + 8 units).
TENSOR_CORE_SHAPES = [(sb.Q4_K, 3584, 3584), (sb.Q4_K, 45, 3584), (sb.Q4_K, 130, 8192), (sb.Q4_K, 77, 18944), (sb.Q4_K, 33, 28672),
                      (sb.Q4_K, 20, 256), (sb.Q4_K, 19, 4096), (sb.Q4_K, 64, 4352),
                      (sb.Q6_K, 512, 3584), (sb.Q6_K, 45, 3584), (sb.Q6_K, 3584, 18944), (sb.Q6_K, 21, 256), (sb.Q6_K, 50, 2048),
                      (sb.Q6_K, 18, 2304), (sb.Q6_K, 130, 8192), (sb.Q6_K, 33, 28672)]


@pytest.mark.parametrize("ggml_type,rows,columns", TENSOR_CORE_SHAPES)
@pytest.mark.parametrize("tokens", [2, 3, 5, 8, 9, 17])
def test_kquant_token_groups_on_tensor_cores_equal_single_token_products(oracle, ggml_type, rows, columns, tokens):
    """Q4_K and (planar) Q6_K with several tokens run on the integer tensor cores. Every token's row must carry the bits
    of a launch of its own (OptimizedQwen2Tests.cs:41-54: a token's result does not depend on what shares its weight
    pass), for every team shape, with accumulation, row ranges and strides, and the values must be the oracle's."""
    if rows * columns > 20_000_000 and tokens not in (2, 8):
        pytest.skip("the large shapes run at two and eight tokens")
    weights = synth.matrix(ggml_type, rows, columns, seed=61 + rows)
    x = synth.activations(tokens, columns, seed=62)
    with sb.QuantizedMatrix(weights, ggml_type, rows, columns) as matrix:
        together = matrix.matvec(x, sb.MODE_XQ8)
        alone = np.concatenate([matrix.matvec(x[t:t + 1], sb.MODE_XQ8) for t in range(tokens)])
        assert together.tobytes() == alone.tobytes()
        first, count = rows // 3, rows - rows // 3 - 1
        strided = np.full((tokens, count + 5), SENTINEL, np.float32)
        matrix.matvec(x, sb.MODE_XQ8, row_start=first, row_count=count, output=strided, output_stride=count + 5)
        assert strided[:, :count].tobytes() == np.ascontiguousarray(together[:, first:first + count]).tobytes()
        assert np.all(strided[:, count:] == SENTINEL)
        residual = synth.activations(tokens, rows, seed=64).copy()
        accumulated = residual.copy()
        matrix.matvec(x, sb.MODE_XQ8, epilogue=sb.EPILOGUE_ACCUMULATE, output=accumulated)
        assert np.array_equal(accumulated, residual + together)
        assert sb.library().device_faults() == 0
    if rows * columns <= 20_000_000:
        codes, scales = oracle.quantize(x)
        exact, magnitude = oracle.kq_q8_exact(ggml_type, weights, rows, columns, codes, scales)
        assert_parity(together, oracle.kq_q8_matmul(ggml_type, weights, rows, columns, codes, scales), exact, magnitude, "tensor-core token groups")


def test_invalid_calls_fail_with_a_status_and_leave_outputs_untouched():
    weights = synth.matrix(sb.Q8_0, 4, 64, seed=41)
    with sb.QuantizedMatrix(weights, sb.Q8_0, 4, 64) as matrix:
        buffer = sb.Q8ActivationBuffer(64, 2)
        output = np.full(8, SENTINEL, np.float32)
        with pytest.raises(IndexError):
            matrix.multiply(0, 4, buffer, 2, output, 3)
        with pytest.raises(IndexError):
            matrix.multiply(2, 3, buffer, 1, output)
        raw = matrix._lib.raw
        assert raw.syn_b200_matmul_q8(matrix.handle, 0, 4, buffer.quants.ctypes.data, buffer.scales.ctypes.data, 2, output.ctypes.data, 3) == 2
        assert raw.syn_b200_matmul_q8(matrix.handle, 3, 2, buffer.quants.ctypes.data, buffer.scales.ctypes.data, 1, output.ctypes.data, 4) == 2
        assert raw.syn_b200_matvec(matrix.handle, 0, 4, buffer.scales.ctypes.data, 1, 32, output.ctypes.data, 4, 0, 0) == 2
        assert raw.syn_b200_matvec(matrix.handle, 0, 4, buffer.scales.ctypes.data, 1, 64, output.ctypes.data, 4, 7, 0) == 2
        assert np.all(output == SENTINEL)
    info = sb.library().probe()
    assert info.compute_capability // 10 == 10 and b"sm_100" in info.name
