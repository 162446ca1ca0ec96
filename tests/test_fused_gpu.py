"""Fused projection epilogues (bias, residual, SwiGLU) and the matvec/GEMM selection rule, on device buffers.

The reference fuses these in its CPU executor's projection regions (Qwen2ProjectionWork.cs:7-131: Q/K/V + bias,
output/down + residual add, gate/up + SwiGLU) and selects matvec or GEMM by token count (step/projection.rs:51-72).
"""
import numpy as np
import pytest

import synapse_b200 as sb
from synapse_b200 import synth
from parity import rows_in_parallel

pytestmark = pytest.mark.gpu


def _device(array):
    import torch

    return torch.from_numpy(np.ascontiguousarray(array)).cuda()


@pytest.mark.parametrize("ggml_type,columns", [(sb.Q8_0, 896), (sb.Q4_K, 1024), (sb.Q6_K, 768)])
@pytest.mark.parametrize("tokens", [1, 2, 5])
def test_bias_residual_and_swiglu_epilogues(oracle, ggml_type, columns, tokens):
    import torch

    lib = sb.library()
    rows = 320
    gate_w = synth.matrix(ggml_type, rows, columns, seed=91, name="gate")
    up_w = synth.matrix(ggml_type, rows, columns, seed=92, name="up")
    x = synth.activations(tokens, columns, seed=93)
    bias = synth.activations(1, rows, seed=94)[0]
    residual = synth.activations(tokens, rows, seed=95)
    codes, scales = oracle.quantize(x)
    gate_want = oracle.kq_q8_matmul(ggml_type, gate_w, rows, columns, codes, scales)
    up_want = oracle.kq_q8_matmul(ggml_type, up_w, rows, columns, codes, scales)
    scratch_bytes = lib.activation_scratch_bytes(tokens, columns)
    scratch = torch.empty(scratch_bytes + 256, dtype=torch.uint8, device="cuda")
    scratch_ptr = (scratch.data_ptr() + 255) // 256 * 256
    dx, dbias = _device(x), _device(bias)
    with sb.QuantizedMatrix(gate_w, ggml_type, rows, columns) as gate, sb.QuantizedMatrix(up_w, ggml_type, rows, columns) as up:
        # bias (the Q/K/V region)
        y = torch.zeros(tokens, rows, device="cuda")
        gate.matvec_fused_device(dx.data_ptr(), tokens, columns, y.data_ptr(), rows, bias_ptr=dbias.data_ptr(), scratch_ptr=scratch_ptr,
                                 scratch_bytes=scratch_bytes)
        assert np.allclose(y.cpu().numpy(), gate_want + bias, rtol=1e-3, atol=1e-4)
        # residual add (the output / down region) on a row range
        hidden = _device(residual)
        up.matvec_fused_device(dx.data_ptr(), tokens, columns, hidden.data_ptr() + 4 * 64, rows, accumulate=True, scratch_ptr=scratch_ptr,
                               scratch_bytes=scratch_bytes, row_start=64, row_count=128)
        want = residual.copy()
        want[:, 64:192] += up_want[:, 64:192]
        assert np.allclose(hidden.cpu().numpy(), want, rtol=1e-3, atol=1e-4)
        # SwiGLU (the gate/up region): shared quantised activations, up's epilogue multiplies by silu(gate)
        sb.quantize_device(dx.data_ptr(), tokens, columns, columns, scratch_ptr, scratch_bytes)
        g = torch.zeros(tokens, rows, device="cuda")
        gate.matmul_q8_device(scratch_ptr, tokens, g.data_ptr(), rows)
        ff = torch.zeros(tokens, rows, device="cuda")
        up.matmul_q8_fused_device(scratch_ptr, tokens, ff.data_ptr(), rows, gate_ptr=g.data_ptr(), gate_stride=rows)
        torch.cuda.synchronize()
        swiglu = gate_want / (1.0 + np.exp(-gate_want.astype(np.float64))) * up_want
        assert np.allclose(ff.cpu().numpy(), swiglu, rtol=1e-3, atol=1e-4)
        bad = sb.Epilogue(None, None, 0, 2, 0)
        assert lib.raw.syn_b200_matmul_q8_ex_dev(up.handle, 0, rows, scratch_ptr, tokens, ff.data_ptr(), rows, bad, None) == 2
    assert lib.device_faults() == 0


def test_prompt_runs_above_four_tokens_take_the_tensor_core_path(oracle):
    import torch

    lib = sb.library()
    rows, columns, tokens = 512, 1024, 9
    weights = synth.matrix(sb.Q4_K, rows, columns, seed=96)
    x = _device(synth.activations(tokens, columns, seed=97))
    scratch_bytes = max(lib.gemm_scratch_bytes(tokens, columns), lib.activation_scratch_bytes(tokens, columns))
    scratch = torch.empty(scratch_bytes + 256, dtype=torch.uint8, device="cuda")
    scratch_ptr = (scratch.data_ptr() + 255) // 256 * 256
    with sb.QuantizedMatrix(weights, sb.Q4_K, rows, columns) as matrix:
        routed = torch.zeros(tokens, rows, device="cuda")
        launches = lib.launch_count(reset=True)
        matrix.matvec_fused_device(x.data_ptr(), tokens, columns, routed.data_ptr(), rows, mode=sb.MODE_XF32, scratch_ptr=scratch_ptr,
                                   scratch_bytes=scratch_bytes)
        direct = torch.zeros(tokens, rows, device="cuda")
        matrix.gemm_device(x.data_ptr(), tokens, columns, direct.data_ptr(), rows, scratch_ptr, scratch_bytes)
        few = torch.zeros(4, rows, device="cuda")
        matrix.matvec_fused_device(x.data_ptr(), 4, columns, few.data_ptr(), rows, mode=sb.MODE_XF32, scratch_ptr=scratch_ptr,
                                   scratch_bytes=scratch_bytes)
        torch.cuda.synchronize()
        assert torch.equal(routed, direct)  # same kernel, same result
        want = oracle.f32_matmul(sb.Q4_K, weights, rows, columns, x[:4].cpu().numpy())
        assert np.allclose(few.cpu().numpy(), want, rtol=1e-3, atol=1e-4)  # four tokens stay on the FP32 matvec
        assert not torch.equal(few, routed[:4])
        # which path an entry point takes is a matter of what the caller passes, never of chance: without the tensor-core
        # scratch every token count stays on the FP32-activation kernels, and so does the host-buffer entry point
        small = lib.activation_scratch_bytes(tokens, columns)
        assert small < lib.gemm_scratch_bytes(tokens, columns)
        plain = torch.zeros(tokens, rows, device="cuda")
        matrix.matvec_fused_device(x.data_ptr(), tokens, columns, plain.data_ptr(), rows, mode=sb.MODE_XF32, scratch_ptr=scratch_ptr, scratch_bytes=small)
        torch.cuda.synchronize()
        assert torch.equal(plain[:4], few) and not torch.equal(plain, routed)
        host = matrix.matvec(x.cpu().numpy(), sb.MODE_XF32)
        assert np.array_equal(host, plain.cpu().numpy())
        many = _device(synth.activations(129, columns, seed=98))
        need = lib.gemm_scratch_bytes(129, columns)
        work = torch.empty(need + 256, dtype=torch.uint8, device="cuda")
        work_ptr = (work.data_ptr() + 255) // 256 * 256
        a, b = torch.zeros(129, rows, device="cuda"), torch.zeros(129, rows, device="cuda")
        matrix.matvec_fused_device(many.data_ptr(), 129, columns, a.data_ptr(), rows, mode=sb.MODE_XF32, scratch_ptr=work_ptr, scratch_bytes=need)
        matrix.gemm_device(many.data_ptr(), 129, columns, b.data_ptr(), rows, work_ptr, need)
        torch.cuda.synchronize()
        assert torch.equal(a, b)


@pytest.mark.parametrize("ggml_type", [sb.Q8_0, sb.Q4_K, sb.Q6_K])
@pytest.mark.parametrize("tokens", [1, 8, 11])
def test_gather_entry_stores_every_result_into_all_copies(ggml_type, tokens):
    """syn_b200_matmul_q8_gather_dev on one GPU, the "peers" being further buffers of the same device: every copy ends up
    holding what the plain product writes, shard by shard, and nothing outside the shard's rows is touched. One token takes
    the pipelined kernel's storing variant, several tokens the tensor-core token groups' (Q4_K, Q6_K) or the direct-load
    kernels' (Q8_0)."""
    import torch

    rows, columns, world = 768, 1024, 3
    weights = synth.matrix(ggml_type, rows, columns, seed=21)
    x = torch.from_numpy(synth.activations(tokens, columns, seed=22)).cuda()
    lib = sb.library()
    need = lib.activation_scratch_bytes(tokens, columns)
    scratch = torch.empty(need + 256, dtype=torch.uint8, device="cuda")
    scratch_ptr = (scratch.data_ptr() + 255) // 256 * 256
    sb.quantize_device(x.data_ptr(), tokens, columns, columns, scratch_ptr, need, 0)
    with sb.QuantizedMatrix(weights, ggml_type, rows, columns) as matrix:
        want = torch.zeros(tokens, rows, device="cuda")
        matrix.matmul_q8_device(scratch_ptr, tokens, want.data_ptr(), rows)
        copies = [torch.full((tokens, rows), -7.0, device="cuda") for _ in range(world)]
        share = rows // world
        for rank in (1,):  # only the middle shard is computed: the others must keep their sentinel
            first = rank * share
            own = copies[rank].data_ptr() + 4 * first
            others = [copies[r].data_ptr() + 4 * first for r in range(world) if r != rank]
            matrix.matmul_q8_gather_device(scratch_ptr, tokens, own, rows, others, row_start=first, row_count=share)
        torch.cuda.synchronize()
        for copy in copies:
            assert torch.equal(copy[:, share:2 * share], want[:, share:2 * share])
            assert bool((copy[:, :share] == -7.0).all()) and bool((copy[:, 2 * share:] == -7.0).all())
        with pytest.raises(sb.KernelError):
            matrix.matmul_q8_gather_device(scratch_ptr, tokens, copies[0].data_ptr(), rows, [copies[1].data_ptr()] * 8)
    assert lib.device_faults() == 0


def test_shared_buffer_and_peer_access_entry_points():
    """The buffer that other processes map: created zero-filled, usable as an output of the product, and the error
    paths of the mapping calls (a process cannot map its own export; peer access to oneself is a no-op, to a device
    that does not exist an error)."""
    import torch

    lib = sb.library()
    pointer, handle = lib.shared_buffer_create(4096)
    try:
        assert len(handle) == 64 and pointer % 256 == 0
        with pytest.raises(sb.BackendUnavailableError):
            lib.shared_buffer_open(handle)
        lib.enable_peer_access(torch.cuda.current_device())
        with pytest.raises(sb.KernelError):
            lib.enable_peer_access(4096)
        with pytest.raises(sb.KernelError):
            lib.shared_buffer_create(0)
    finally:
        lib.shared_buffer_destroy(pointer)


SEGMENT_CASES = [  # type, columns, rows of the three segments
    (sb.Q4_K, 3584, (3584, 512, 512)),   # q | k | v of the 7B shape in one encoding: one-warp teams
    (sb.Q4_K, 8192, (300, 37, 64)),      # two-warp teams, ragged row counts
    (sb.Q6_K, 1024, (130, 70, 1)),
    (sb.Q8_0, 896, (896, 128, 128)),     # q | k | v of the 0.5B shape
]


@pytest.mark.parametrize("ggml_type,columns,row_counts", SEGMENT_CASES)
@pytest.mark.parametrize("tokens", [1, 3])
def test_segments_in_one_launch_equal_separate_products(oracle, ggml_type, columns, row_counts, tokens):
    """Q | K | V as one dispatch (MatmulArgs with three segments, native/synapse-gpu/.../step/layers.rs:71-94): every row
    keeps the summation order it has in a launch of its own, so the results are bit-identical to three products, and they
    match the oracle. One token takes the one-launch kernel, several tokens the per-segment launches behind the same call."""
    import torch

    lib = sb.library()
    weights = [synth.matrix(ggml_type, rows, columns, seed=401 + i, name=f"segment{i}") for i, rows in enumerate(row_counts)]
    biases = [synth.activations(1, rows, seed=411 + i)[0] for i, rows in enumerate(row_counts)]
    x = synth.activations(tokens, columns, seed=421)
    codes, scales = oracle.quantize(x)
    need = lib.activation_scratch_bytes(tokens, columns)
    scratch = torch.empty(need + 256, dtype=torch.uint8, device="cuda")
    scratch_ptr = (scratch.data_ptr() + 255) // 256 * 256
    dx = _device(x)
    sb.quantize_device(dx.data_ptr(), tokens, columns, columns, scratch_ptr, need)
    matrices = [sb.QuantizedMatrix(w, ggml_type, rows, columns) for w, rows in zip(weights, row_counts)]
    dbias = [_device(b) for b in biases]
    total = sum(row_counts) + 5  # a gap of five floats before the last segment and the stride
    columns_out = [0, row_counts[0], row_counts[0] + row_counts[1] + 5]
    try:
        separate = torch.full((tokens, total), -3.0, device="cuda")
        for m, b, rows, column in zip(matrices, dbias, row_counts, columns_out):
            m.matmul_q8_fused_device(scratch_ptr, tokens, separate.data_ptr() + 4 * column, total, bias_ptr=b.data_ptr())
        launches = lib.launch_count(reset=True)
        together = torch.full((tokens, total), -3.0, device="cuda")
        sb.matmul_q8_segments_device([(m, 0, None, b.data_ptr(), column) for m, b, column in zip(matrices, dbias, columns_out)], scratch_ptr, tokens,
                                     together.data_ptr(), total)
        torch.cuda.synchronize()
        assert lib.launch_count(reset=True) == (1 if tokens == 1 else 3)
        assert torch.equal(together, separate)
        got = together.cpu().numpy()
        for w, b, rows, column in zip(weights, biases, row_counts, columns_out):
            want = oracle.kq_q8_matmul(ggml_type, w, rows, columns, codes, scales) + b
            assert np.allclose(got[:, column:column + rows], want, rtol=1e-3, atol=1e-4)
        assert np.all(got[:, columns_out[2] - 5:columns_out[2]] == -3.0), "the gap between segments was written"
        # residual form on a row range of the first segment only
        base = torch.from_numpy(synth.activations(tokens, 40, seed=431)).cuda()
        result = base.clone()
        sb.matmul_q8_segments_device([(matrices[0], 3, 40, 0, 0)], scratch_ptr, tokens, result.data_ptr(), 40, accumulate=True)
        torch.cuda.synchronize()
        plain = torch.zeros(tokens, 40, device="cuda")
        matrices[0].matmul_q8_device(scratch_ptr, tokens, plain.data_ptr(), 40, row_start=3, row_count=40)
        torch.cuda.synchronize()
        assert torch.equal(result, base + plain)
        bad = [(matrices[0], 0, None, 0, 0)] * 4
        with pytest.raises(sb.KernelError):
            sb.matmul_q8_segments_device(bad, scratch_ptr, tokens, together.data_ptr(), total)
    finally:
        for m in matrices:
            m.close()
    assert lib.device_faults() == 0


@pytest.mark.parametrize("ggml_type,rows,columns", [(sb.Q4_K, 18944, 3584), (sb.Q4_K, 333, 8192), (sb.Q6_K, 150, 2048), (sb.Q8_0, 4864, 896)])
@pytest.mark.parametrize("tokens", [1, 2])
def test_gate_up_pair_in_one_launch_equals_the_two_launch_form(oracle, ggml_type, rows, columns, tokens):
    """The gate/up region (Qwen2GateUpWork, Qwen2ProjectionWork.cs:91-131) as one launch whose warps hold gate row r and up
    row r side by side: bit-identical to gate product -> memory -> up product with the SwiGLU epilogue, and equal to the
    oracle's silu(gate) * up. Includes the 7B feed-forward shape the benchmark's roofline figure is quoted on."""
    import torch

    lib = sb.library()
    gate_w = synth.matrix(ggml_type, rows, columns, seed=441, name="gate")
    up_w = synth.matrix(ggml_type, rows, columns, seed=442, name="up")
    x = synth.activations(tokens, columns, seed=443)
    codes, scales = oracle.quantize(x)
    need = lib.activation_scratch_bytes(tokens, columns)
    scratch = torch.empty(need + 256, dtype=torch.uint8, device="cuda")
    scratch_ptr = (scratch.data_ptr() + 255) // 256 * 256
    dx = _device(x)
    sb.quantize_device(dx.data_ptr(), tokens, columns, columns, scratch_ptr, need)
    with sb.QuantizedMatrix(gate_w, ggml_type, rows, columns) as gate, sb.QuantizedMatrix(up_w, ggml_type, rows, columns) as up:
        g = torch.zeros(tokens, rows, device="cuda")
        gate.matmul_q8_device(scratch_ptr, tokens, g.data_ptr(), rows)
        two = torch.zeros(tokens, rows, device="cuda")
        up.matmul_q8_fused_device(scratch_ptr, tokens, two.data_ptr(), rows, gate_ptr=g.data_ptr(), gate_stride=rows)
        lib.launch_count(reset=True)
        one = torch.full((tokens, rows), -3.0, device="cuda")
        spare = torch.zeros(tokens, rows, device="cuda")
        sb.matmul_q8_swiglu_device(gate, up, scratch_ptr, tokens, one.data_ptr(), rows, gate_values_ptr=spare.data_ptr())
        torch.cuda.synchronize()
        assert lib.launch_count(reset=True) == (1 if tokens == 1 else 2)
        assert torch.equal(one, two)
        if tokens == 1:
            assert not bool(spare.any()), "the gate values went to memory"
        # a row range in the middle
        first, count = rows // 3, min(100, rows - rows // 3)
        part = torch.zeros(tokens, count, device="cuda")
        sb.matmul_q8_swiglu_device(gate, up, scratch_ptr, tokens, part.data_ptr(), count, gate_values_ptr=spare.data_ptr(), row_start=first, row_count=count)
        torch.cuda.synchronize()
        assert torch.equal(part, two[:, first:first + count])
        if tokens > 1:
            with pytest.raises(sb.KernelError, match="gate_values"):
                sb.matmul_q8_swiglu_device(gate, up, scratch_ptr, tokens, one.data_ptr(), rows)
    gate_want = rows_in_parallel(oracle.kq_q8_matmul, ggml_type, gate_w, rows, columns, codes, scales).astype(np.float64)
    up_want = rows_in_parallel(oracle.kq_q8_matmul, ggml_type, up_w, rows, columns, codes, scales)
    want = gate_want / (1.0 + np.exp(-gate_want)) * up_want
    assert np.allclose(one.cpu().numpy(), want, rtol=1e-3, atol=1e-4 * max(1.0, float(np.abs(want).max())))
    assert lib.device_faults() == 0


@pytest.mark.parametrize("tokens", [1, 8])
def test_completion_signal_and_bounded_wait_on_one_gpu(tokens):
    """The exchange step's completion signal, with the "ranks" emulated on one GPU (three buffers of the same device):
    each rank's product writes its slice into all three copies and then its sequence number into its word of every copy's
    signal array; a wait on a copy succeeds once all three words show the sequence number. With one rank's product
    withheld the wait's limit runs out: the kernel returns, the fault count goes up by one, nothing is left waiting and
    the device stays usable. The ranks run one after the other on one stream, so no kernel ever waits for a later one.
    One token signals from the pipelined kernel, eight from the tensor-core token groups."""
    import torch

    lib = sb.library()
    rows, columns, world = 768, 1024, 3
    share = rows // world
    weights = synth.matrix(sb.Q4_K, rows, columns, seed=451)
    x = torch.from_numpy(synth.activations(tokens, columns, seed=452)).cuda()
    need = lib.activation_scratch_bytes(tokens, columns)
    scratch = torch.empty(need + 256, dtype=torch.uint8, device="cuda")
    scratch_ptr = (scratch.data_ptr() + 255) // 256 * 256
    sb.quantize_device(x.data_ptr(), tokens, columns, columns, scratch_ptr, need, 0)
    copies = [torch.full((tokens, rows), -7.0, device="cuda") for _ in range(world)]
    control = [torch.zeros(32, dtype=torch.int32, device="cuda") for _ in range(world)]  # per "GPU": signal words 0..2, arrivals 16/17, epoch 24
    assert lib.device_faults(reset=True) == 0
    with sb.QuantizedMatrix(weights, sb.Q4_K, rows, columns) as matrix:
        want = torch.zeros(tokens, rows, device="cuda")
        matrix.matmul_q8_device(scratch_ptr, tokens, want.data_ptr(), rows)

        def product(rank):
            first = rank * share
            own = copies[rank].data_ptr() + 4 * first
            others = [copies[r].data_ptr() + 4 * first for r in range(world) if r != rank]
            words = [control[rank].data_ptr() + 4 * rank] + [control[r].data_ptr() + 4 * rank for r in range(world) if r != rank]
            matrix.matmul_q8_gather_device(scratch_ptr, tokens, own, rows, others, row_start=first, row_count=share, signal_ptrs=words,
                                           arrivals_ptr=control[rank].data_ptr() + 4 * 16)

        def wait(rank, limit_us):
            sb.gather_wait_device(control[rank].data_ptr(), world, control[rank].data_ptr() + 4 * 24, limit_us)

        for step in (1, 2):  # two rounds: the sequence numbers count up, the arrival counters start over
            for rank in range(world):
                product(rank)
            for rank in range(world):
                wait(rank, 1_000_000)
            torch.cuda.synchronize()
            assert lib.device_faults() == 0
            for rank in range(world):
                assert torch.equal(copies[rank], want)
                assert control[rank][:world].tolist() == [step] * world and int(control[rank][24]) == step
                assert int(control[rank][16]) == 0 and int(control[rank][17]) == step
        # round three with rank 1 withheld: the others' words move on, rank 1's does not, the wait gives up after 20 ms
        product(0)
        product(2)
        wait(0, 20_000)
        torch.cuda.synchronize()
        assert control[0][:world].tolist() == [3, 2, 3]
        assert lib.device_faults(reset=True) == 1
        # the device is still usable and a later complete round is seen as such
        product(1)
        torch.cuda.synchronize()
        assert control[0][:world].tolist() == [3, 3, 3]
        with pytest.raises(sb.KernelError):
            sb.gather_wait_device(control[0].data_ptr(), 9, control[0].data_ptr() + 4 * 24)
    assert lib.device_faults() == 0
