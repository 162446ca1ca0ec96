"""Fused projection epilogues (bias, residual, SwiGLU) and the matvec/GEMM selection rule, on device buffers.

The reference fuses these in its CPU executor's projection regions (Qwen2ProjectionWork.cs:7-131: Q/K/V + bias,
output/down + residual add, gate/up + SwiGLU) and selects matvec or GEMM by token count (step/projection.rs:51-72).
"""
import numpy as np
import pytest

import synapse_b200 as sb
from synapse_b200 import synth

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


@pytest.mark.parametrize("ggml_type", [sb.Q8_0, sb.Q4_K, sb.Q6_K])
def test_gather_entry_stores_every_result_into_all_copies(ggml_type):
    """syn_b200_matmul_q8_gather_dev on one GPU, the "peers" being further buffers of the same device: every copy ends up
    holding what the plain product writes, shard by shard, and nothing outside the shard's rows is touched."""
    import torch

    rows, columns, world = 768, 1024, 3
    weights = synth.matrix(ggml_type, rows, columns, seed=21)
    x = torch.from_numpy(synth.activations(1, columns, seed=22)).cuda()
    lib = sb.library()
    need = lib.activation_scratch_bytes(1, columns)
    scratch = torch.empty(need + 256, dtype=torch.uint8, device="cuda")
    scratch_ptr = (scratch.data_ptr() + 255) // 256 * 256
    sb.quantize_device(x.data_ptr(), 1, columns, columns, scratch_ptr, need, 0)
    with sb.QuantizedMatrix(weights, ggml_type, rows, columns) as matrix:
        want = torch.zeros(rows, device="cuda")
        matrix.matmul_q8_device(scratch_ptr, 1, want.data_ptr(), rows)
        copies = [torch.full((rows,), -7.0, device="cuda") for _ in range(world)]
        share = rows // world
        for rank in (1,):  # only the middle shard is computed: the others must keep their sentinel
            first = rank * share
            own = copies[rank].data_ptr() + 4 * first
            others = [copies[r].data_ptr() + 4 * first for r in range(world) if r != rank]
            matrix.matmul_q8_gather_device(scratch_ptr, 1, own, share, others, row_start=first, row_count=share)
        torch.cuda.synchronize()
        for copy in copies:
            assert torch.equal(copy[share:2 * share], want[share:2 * share])
            assert bool((copy[:share] == -7.0).all()) and bool((copy[2 * share:] == -7.0).all())
        with pytest.raises(sb.KernelError):
            matrix.matmul_q8_gather_device(scratch_ptr, 1, copies[0].data_ptr(), share, [copies[1].data_ptr()] * 8)


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
