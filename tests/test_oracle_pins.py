"""Pins the CPU oracle to the known-answer vectors of the reference's own tests (no GPU needed)."""
import numpy as np
import pytest

from synapse_b200 import synth

Q8_0, Q4_K, Q6_K = 8, 12, 14


def test_fp16_widening_is_exact_for_every_finite_half(oracle):
    # native/synapse-kernels/tests/Features/CpuKernels/q8_0_tests.rs:223-247
    bits = np.arange(65536, dtype=np.uint16)
    finite = ((bits >> 10) & 0x1F) != 0x1F
    expected = bits.view(np.float16).astype(np.float64)
    for b in bits[finite][:: 1]:
        assert np.float64(oracle.fp16_to_f32(int(b))).tobytes() == expected[b].tobytes(), hex(b)


def test_fp16_narrowing_matches_numpy_round_to_nearest_even(oracle):
    rng = np.random.default_rng(7)
    values = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 5, 20000).astype(np.float32),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e-8, 2.0 ** -25, 2.0 ** -24, 3 * 2.0 ** -25, 6.1e-5, 6.0975552e-05], np.float32),
    ]).astype(np.float32)
    with np.errstate(over="ignore"):
        expected = values.astype(np.float16).view(np.uint16)
    for value, want in zip(values, expected):
        assert oracle.f32_to_fp16(float(value)) == int(want), float(value)


def test_quantiser_rounds_ties_to_even(oracle):
    # tests/Synapse.IntegrationTests/Features/CpuKernels/ActivationQuantizerTests.cs:28-45
    x = np.zeros(32, np.float32)
    x[:6] = [127.0, 2.5, 3.5, -2.5, -0.5, 0.5]
    codes, scales = oracle.quantize(x)
    assert scales[0] == np.float32(1.0)
    assert codes[:6].tolist() == [127, 2, 4, -2, 0, 0]


def test_zero_block_stores_zero_scale_and_codes(oracle):
    # ActivationQuantizerTests.cs:47-61
    x = np.zeros(64, np.float32)
    x[40] = -3.0
    codes, scales = oracle.quantize(x)
    assert scales[0] == 0.0 and not codes[:32].any()
    assert codes[40] == -127
    assert scales[1] == np.float32(np.float16(np.float32(3.0) / np.float32(127.0)))


def test_quantiser_rejects_misaligned_rows(oracle):
    # ActivationQuantizerTests.cs:63-70
    with pytest.raises(ValueError):
        oracle.quantize(np.zeros(33, np.float32))


@pytest.mark.parametrize("columns", [32, 896, 4864])
def test_quantiser_matches_the_scalar_contract(oracle, columns):
    # ActivationQuantizerTests.cs:8-26,72-95: same formula written independently with numpy float32 ops.
    rng = np.random.default_rng(20260928 + columns)
    x = ((rng.random(columns) * 8 - 4).astype(np.float32) * rng.random(columns).astype(np.float32)).astype(np.float32)
    codes, scales = oracle.quantize(x)
    blocks = x.reshape(-1, 32)
    amax = np.abs(blocks).max(axis=1)
    scale = (amax / np.float32(127.0)).astype(np.float32)
    inverse = np.where(scale == 0, np.float32(0), np.float32(1.0) / np.where(scale == 0, np.float32(1), scale)).astype(np.float32)
    want = np.rint((blocks * inverse[:, None]).astype(np.float32)).astype(np.int8)
    assert np.array_equal(codes.reshape(-1, 32), want)
    assert np.array_equal(scales, scale.astype(np.float16).astype(np.float32))


def test_q8_0_golden_block_decodes(oracle):
    # tests/Synapse.IntegrationTests/Features/ModelPackages/SourceTensorDecoderTests.cs:56-70
    block = np.zeros(34, np.uint8)
    block[0:2] = [0x00, 0x34]
    block[2:5] = [0x7F, 0x81, 0x80]
    values = oracle.decode(Q8_0, block, 32)[0]
    assert values[:4].tolist() == [31.75, -31.75, -32.0, 0.0]


def test_k_quant_block_lengths_are_exact(oracle):
    # SourceTensorDecoderTests.cs:165-173
    assert oracle.row_bytes(Q4_K, 512) == 288
    assert oracle.row_bytes(Q4_K, 300) == 0
    assert oracle.row_bytes(Q6_K, 256) == 210
    assert oracle.row_bytes(Q8_0, 896) == 28 * 34
    with pytest.raises(ValueError):
        oracle.decode(Q4_K, np.zeros(144, np.uint8), 512)


def _python_lcg(seed, count):
    state, out = seed, []
    for _ in range(count):
        state = (state * 6364136223846793005 + 1442695040888963407) & (2**64 - 1)
        out.append(state >> 33)
    return out


def test_lcg_generator_matches_a_plain_python_restatement(oracle):
    # q8_0_tests.rs:9-23,36-62
    weights, quants, scales = oracle.lcg_case(5, 1, 1, 1)
    stream = _python_lcg(5, 1 + 32 + 32 + 1)
    assert int(weights[0]) | (int(weights[1]) << 8) == 0x1000 + stream[0] % 0x1400
    assert weights[2:].view(np.int8).tolist() == [v % 255 - 127 for v in stream[1:33]]
    assert quants.tolist() == [v % 255 - 127 for v in stream[33:65]]
    assert scales[0] == np.array([0x2000 + stream[65] % 0x1000], np.uint16).view(np.float16).astype(np.float32)[0]


LCG_CASES = [(37, 28, 1, 37, 1), (16, 152, 3, 20, 2), (5, 64, 2, 9, 3), (8, 63, 4, 11, 4)]
SENTINEL = np.float32(12345.0)


@pytest.mark.parametrize("rows,blocks,tokens,stride,seed", LCG_CASES)
def test_scalar_kernel_matches_the_f64_oracle_on_the_reference_cases(oracle, rows, blocks, tokens, stride, seed):
    # q8_0_tests.rs:110-131,133-166: |actual - exact| <= 2e-5 * sum|term| + 1e-12, stride gap untouched.
    weights, quants, scales = oracle.lcg_case(seed, rows, blocks, tokens)
    status, output = oracle.q8q8_matmul(weights, rows, blocks, quants, scales, tokens, stride, fill=SENTINEL)
    assert status == 0
    exact, magnitude = oracle.q8q8_exact(weights, rows, blocks, quants, scales, tokens)
    for t in range(tokens):
        got = output[t * stride: t * stride + rows].astype(np.float64)
        assert np.all(np.abs(got - exact[t]) <= 2e-5 * magnitude[t] + 1e-12)
        if t + 1 < tokens:
            assert np.all(output[t * stride + rows: (t + 1) * stride].view(np.uint32) == SENTINEL.view(np.uint32))
    threaded = oracle.q8q8_matmul_threads(weights, rows, blocks, quants, scales, tokens, 3)
    assert np.all(np.abs(threaded.astype(np.float64) - exact) <= 2e-5 * magnitude + 1e-12)


def test_invalid_shapes_are_rejected_before_reading(oracle):
    # q8_0_tests.rs:169-205 and 259-291
    weights, quants, scales = oracle.lcg_case(9, 4, 2, 2)
    assert oracle.q8q8_matmul(weights, 0, 2, quants, scales, 2, 4)[0] == 2
    status, output = oracle.q8q8_matmul(weights, 4, 2, quants, scales, 2, 3, fill=SENTINEL)
    assert status == 2 and np.all(output == SENTINEL)
    lib = oracle.lib()
    big = 2**64 - 1
    assert lib.orc_q8q8_matmul(weights.ctypes.data, 68, big, 2, quants.ctypes.data, scales.ctypes.data, 2, output.ctypes.data, big) == 3
    assert np.all(output == SENTINEL)
    assert oracle.q8q8_matmul(weights, 4, 2, quants, scales, 1, 4, row_bytes_arg=67)[0] == 2
    assert lib.orc_q8q8_matmul(None, 68, 4, 2, quants.ctypes.data, scales.ctypes.data, 1, output.ctypes.data, 4) == 1


def test_block_dots_are_the_exact_integer_sums(oracle):
    weights, quants, scales = oracle.lcg_case(21, 6, 5, 2)
    dots = oracle.q8q8_block_dots(weights, 6, 5, quants, 2)
    w = weights.reshape(6, 5, 34)[:, :, 2:].view(np.int8).astype(np.int64)
    a = quants.reshape(2, 5, 32).astype(np.int64)
    assert np.array_equal(dots, np.einsum("rbi,tbi->trb", w, a).astype(np.int32))
    assert np.array_equal(dots, oracle.int_dots(Q8_0, weights, 6, 160, quants))


@pytest.mark.parametrize("ggml_type,name", [(Q8_0, "Q8_0"), (Q4_K, "Q4_K"), (Q6_K, "Q6_K")])
def test_decoders_agree_with_an_independent_implementation(oracle, ggml_type, name):
    # Same purpose as tests/Synapse.IntegrationTests/Features/ModelPackages/GgmlReferenceDecoderTests.cs:30-49:
    # exact for Q8_0 / Q6_K, within 2^-20 * max|value| for the affine Q4_K.
    quants = pytest.importorskip("gguf.quants")
    gguf = pytest.importorskip("gguf")
    data = synth.matrix(ggml_type, 16, 256, seed=3)
    ours = oracle.decode(ggml_type, data, 256)
    theirs = quants.dequantize(data.reshape(16, -1), getattr(gguf.GGMLQuantizationType, name)).astype(np.float32)
    if ggml_type == Q4_K:
        assert np.max(np.abs(ours - theirs)) <= 2.0 ** -20 * np.max(np.abs(theirs))
    else:
        assert np.array_equal(ours, theirs)


@pytest.mark.parametrize("ggml_type", [Q4_K, Q6_K])
def test_k_quant_reference_equals_an_f32_model_holding_the_decoded_values_bitwise(oracle, ggml_type):
    # tests/Synapse.IntegrationTests/Features/Quantization/KQuantWeightTests.cs:26-47
    rows, columns = 12, 768
    data = synth.matrix(ggml_type, rows, columns, seed=11)
    x = synth.activations(2, columns, seed=12)
    decoded = oracle.decode(ggml_type, data, columns)
    want = np.zeros((2, rows), np.float32)
    for t in range(2):
        for r in range(rows):
            s = np.float32(0)
            for i in range(columns):
                s = np.float32(s + np.float32(decoded[r, i] * x[t, i]))
            want[t, r] = s
    got = oracle.f32_matmul(ggml_type, data, rows, columns, x)
    assert got.tobytes() == want.tobytes()
    assert oracle.f32_matmul_threads(ggml_type, data, rows, columns, x, 4).tobytes() == want.tobytes()


def test_q8_0_reference_backend_order(oracle):
    # src/Synapse.Runtime/Features/GraphExecution/Q8Operators.cs:75-96
    rows, columns = 5, 96
    data = synth.matrix(Q8_0, rows, columns, seed=13)
    x = synth.activations(1, columns, seed=14)
    blocks = data.reshape(rows, 3, 34)
    want = np.zeros(rows, np.float32)
    for r in range(rows):
        s = np.float32(0)
        for b in range(3):
            scale = blocks[r, b, :2].copy().view(np.float16).astype(np.float32)[0]
            bs = np.float32(0)
            for i in range(32):
                bs = np.float32(bs + np.float32(np.float32(blocks[r, b, 2 + i].view(np.int8)) * x[0, b * 32 + i]))
            s = np.float32(s + np.float32(scale * bs))
        want[r] = s
    assert oracle.f32_matmul(Q8_0, data, rows, columns, x)[0].tobytes() == want.tobytes()


def _tiny_q4k(values):
    """A simple valid Q4_K encoder, written after the reference tests' generator
    (tests/Synapse.IntegrationTests/Features/GpuKernels/TinyKQuantEncoder.cs:38-82)."""
    out = np.zeros((values.size // 256, 144), np.uint8)
    for bi, x in enumerate(values.reshape(-1, 256)):
        sub = x.reshape(8, 32)
        low = np.minimum(0, sub.min(axis=1))
        steps = (sub.max(axis=1) - low) / np.float32(15)
        offsets = -low
        d = np.float32(np.float16(steps.max() / np.float32(63)))
        dmin = np.float32(np.float16(offsets.max() / np.float32(63)))
        scale = np.zeros(8, np.int64) if d == 0 else np.clip(np.rint(steps / d), 0, 63).astype(np.int64)
        minimum = np.zeros(8, np.int64) if dmin == 0 else np.clip(np.rint(offsets / dmin), 0, 63).astype(np.int64)
        block = out[bi]
        block[0:2] = np.array([d], np.float16).view(np.uint8)
        block[2:4] = np.array([dmin], np.float16).view(np.uint8)
        for k in range(4):
            block[4 + k] = (scale[k] & 63) | ((scale[k + 4] >> 4) << 6)
            block[8 + k] = (minimum[k] & 63) | ((minimum[k + 4] >> 4) << 6)
            block[12 + k] = (scale[k + 4] & 0xF) | ((minimum[k + 4] & 0xF) << 4)
        for s in range(8):
            step, bias = d * scale[s], dmin * minimum[s]
            q = np.zeros(32, np.int64) if step == 0 else np.clip(np.rint((sub[s] + bias) / step), 0, 15).astype(np.int64)
            block[16 + (s // 2) * 32: 16 + (s // 2) * 32 + 32] |= (q if s % 2 == 0 else q << 4).astype(np.uint8)
    return out.reshape(-1)


def _tiny_q6k(values):
    """A simple valid Q6_K encoder (TinyKQuantEncoder.cs:84-109)."""
    out = np.zeros((values.size // 256, 210), np.uint8)
    for bi, x in enumerate(values.reshape(-1, 256)):
        steps = np.abs(x.reshape(16, 16)).max(axis=1) / np.float32(31)
        d = np.float32(np.float16(steps.max() / np.float32(127)))
        block = out[bi]
        block[208:210] = np.array([d], np.float16).view(np.uint8)
        sc = np.ones(16, np.int64) if d == 0 else np.clip(np.rint(steps / d), 1, 127).astype(np.int64)
        block[192:208] = sc.astype(np.uint8)
        for index in range(256):
            half, rest = divmod(index, 128)
            quarter, l = divmod(rest, 32)
            step = d * sc[index // 16]
            q = (0 if step == 0 else int(np.clip(np.rint(x[index] / step), -32, 31))) + 32
            low = half * 64 + (l if quarter % 2 == 0 else l + 32)
            block[low] |= (q & 0xF) if quarter < 2 else ((q & 0xF) << 4)
            block[128 + half * 32 + l] |= ((q >> 4) & 3) << (2 * quarter)
    return out.reshape(-1)


def test_tiny_k_quant_encoders_round_trip_through_the_decoders(oracle):
    rng = np.random.default_rng(5)
    x = (rng.uniform(-1, 1, 1024) * 1.5 / np.sqrt(1024)).astype(np.float32)
    y4 = oracle.decode(Q4_K, _tiny_q4k(x), 1024)[0]
    y6 = oracle.decode(Q6_K, _tiny_q6k(x), 1024)[0]
    span = float(x.max() - x.min())
    assert np.max(np.abs(y4 - x)) <= span / 15 * 0.75
    assert np.max(np.abs(y6 - x)) <= float(np.abs(x).max()) / 31 * 0.75


@pytest.mark.parametrize("rows,threads,expected", [(1, 8, 16), (4864, 8, 304), (151936, 8, 4096), (896, 2, 224), (17, 3, 16), (150, 1, 76)])
def test_row_chunk_rule(oracle, rows, threads, expected):
    # src/Synapse.Runtime/Features/CpuKernels/ChunkedRowWork.cs:41-64
    assert oracle.chunk_rows(rows, threads) == expected


@pytest.mark.parametrize("ggml_type", [Q8_0, Q4_K, Q6_K])
def test_quantised_activation_contract_is_consistent(oracle, ggml_type):
    """The integer sub-block dots recombine to the FP64 value of decoded weights x dequantised codes."""
    rows, columns = 9, 512
    data = synth.matrix(ggml_type, rows, columns, seed=17)
    x = synth.activations(3, columns, seed=18)
    codes, scales = oracle.quantize(x)
    got = oracle.kq_q8_matmul(ggml_type, data, rows, columns, codes, scales)
    exact, magnitude = oracle.kq_q8_exact(ggml_type, data, rows, columns, codes, scales)
    assert np.all(np.abs(got - exact) <= 2e-5 * magnitude + 1e-12)
    dots = oracle.int_dots(ggml_type, data, rows, columns, codes)
    assert dots.shape == (3, rows, columns // synth.BLOCK_VALUES[ggml_type] * oracle.GROUPS_PER_BLOCK[ggml_type])
    # and it tracks the FP32-activation reference to within the activation quantisation error
    reference, ref_mag = oracle.f32_exact(ggml_type, data, rows, columns, x)
    assert np.all(np.abs(got - reference) <= 1e-2 * ref_mag / np.sqrt(columns) * 4 + 1e-9)
