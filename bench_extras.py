"""Secondary measurements of bench.py (its `extras`): the prefill sweep, the row-sharded sweep of the 70B-class shapes,
FP32-activation matvec rates, the parity summary and the AVX2 CPU figures. Everything here runs after the headline
numbers have been taken; nothing here feeds `value`, `roofline` or `e2e`.
"""
from __future__ import annotations

import math
import os
import time

import numpy as np

from synapse_b200 import sharding, synth

SUSTAINED_TFLOPS_FALLBACK = 1400.0


def measured_tensor_peak(root):
    import json

    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as handle:
            return float(json.load(handle)["bf16_tflops_sustained"]), "measured"
    except (OSError, KeyError, ValueError):
        return SUSTAINED_TFLOPS_FALLBACK, "fallback"


def _aligned_scratch(torch, device, size):
    buffer = torch.empty(size + 256, dtype=torch.uint8, device=device)
    return buffer, (buffer.data_ptr() + 255) // 256 * 256


def _time_graph(torch, stream, body, launches_per_replay, replays=10, warmup=3):
    """Microseconds per launch of `body(stream)` replayed as a CUDA graph, CUDA events on the launch stream."""
    with torch.cuda.stream(stream):
        body(stream)
        stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        body(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(warmup):
            graph.replay()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record(stream)
        for _ in range(replays):
            graph.replay()
        end.record(stream)
        stream.synchronize()
    del graph
    return begin.elapsed_time(end) * 1e3 / (replays * launches_per_replay)


def prefill_sweep(sb, lib, torch, device, stream, root):
    """Config 3: the tensor-core product at 128 / 512 / 2048 / 4096 tokens on the 7B gate (Q4_K), down (Q6_K), attention
    output (Q4_K) and vocabulary (Q4_K) matrices, per precision. TFLOP/s counts 2 * tokens * rows * columns; the activation
    conversion is included. Consecutive launches take different device copies of the matrix (together larger than L2), so
    no launch finds its weights in L2."""
    peak, kind = measured_tensor_peak(root)
    out = {"peak_tflops": peak, "peak_kind": f"sustained bf16 matmul, of {kind}", "points": {}}
    shapes = [("q4_k 18944x3584", synth.Q4_K, 18944, 3584), ("q6_k 3584x18944", synth.Q6_K, 3584, 18944),
              ("q4_k 3584x3584", synth.Q4_K, 3584, 3584), ("q4_k 152064x3584", synth.Q4_K, 152064, 3584)]
    precisions = [("f16", sb.GEMM_F16)] + ([("f16x2", sb.GEMM_F16X2)] if hasattr(sb, "GEMM_F16X2") else [])
    for label, ggml_type, rows, columns in shapes:
        weights = synth.matrix(ggml_type, rows, columns, seed=501, name="prefill")
        copies = max(1, -(-160_000_000 // weights.nbytes))  # 160 MB of weights between two uses of the same copy
        matrices = [sb.QuantizedMatrix(weights, ggml_type, rows, columns) for _ in range(copies)]
        del weights
        try:
            for tokens in (128, 512, 2048, 4096):
                xs = torch.randn(tokens, columns, device=device)
                ys = torch.empty(tokens, rows, device=device)
                need = lib.gemm_scratch_bytes(tokens, columns)
                keep, work = _aligned_scratch(torch, device, need)
                for name, precision in precisions:
                    if name != "f16" and (tokens not in (512, 2048) or rows > 20000):
                        continue  # the second precision is quoted on two points per layer matrix
                    reps = max(copies, 10 if tokens * rows < 3e8 else 4)

                    def body(s):
                        for i in range(reps):
                            matrices[i % copies].gemm_device(xs.data_ptr(), tokens, columns, ys.data_ptr(), rows, work, need, precision=precision,
                                                             stream=s.cuda_stream)

                    microseconds = _time_graph(torch, stream, body, reps, replays=3, warmup=1)
                    tflops = 2.0 * tokens * rows * columns / microseconds / 1e6
                    out["points"][f"{label} x {tokens} tokens, {name}"] = {"us": microseconds, "tflops": tflops, "frac_of_tensor_peak": tflops / peak}
                del xs, ys, keep
        finally:
            for matrix in matrices:
                matrix.close()
    return out


def xf32_rates(sb, lib, torch, device, stream, peak):
    """The FP32-activation contract (the only one the reference defines for K-quants) on the two big 7B layer shapes."""
    out = {}
    for label, ggml_type, rows, columns, copies in (("q4_k 18944x3584", synth.Q4_K, 18944, 3584, 4), ("q6_k 3584x18944", synth.Q6_K, 3584, 18944, 3)):
        hold = [sb.QuantizedMatrix(synth.matrix(ggml_type, rows, columns, seed=520 + c, name="xf32"), ggml_type, rows, columns) for c in range(copies)]
        xs = torch.from_numpy(synth.activations(1, columns, seed=7)).to(device)
        ys = torch.zeros(rows, dtype=torch.float32, device=device)

        def body(s):
            for _ in range(4):
                for matrix in hold:
                    matrix.matvec_device(xs.data_ptr(), 1, columns, ys.data_ptr(), rows, sb.MODE_XF32, stream=s.cuda_stream)

        microseconds = _time_graph(torch, stream, body, 4 * copies)
        size = rows * synth.row_bytes(ggml_type, columns)
        out[label] = {"us": microseconds, "weight_gbs": size / microseconds / 1e3, "frac_of_hbm_peak": size / microseconds / 1e3 / peak}
        for matrix in hold:
            matrix.close()
    return out


def config4_sweep(sb, lib, torch, dist, device, stream, world, rank, peak, use_peers):
    """Config 4: Q4_K 28672x8192, 8192x28672 and 152064x3584 at 1, 8 and 64 activation columns, every matrix sharded by
    output rows over the ranks. Per point: the product alone (at N > 1 it also stores each result into every GPU's copy),
    the product followed by the wait for every rank's completion signal, and the product followed by an NCCL all-gather
    of the slices; at 64 columns also the tensor-core product. Figures are microseconds per product, the slowest rank's,
    and whole-job GB/s of GGUF bytes. Shards are rotated so that a launch never finds its weights in L2."""
    out = {}
    shapes = [("q4_k 28672x8192", synth.Q4_K, 28672, 8192), ("q4_k 8192x28672", synth.Q4_K, 8192, 28672), ("q4_k 152064x3584", synth.Q4_K, 152064, 3584)]

    def slowest(value):
        if world == 1:
            return value
        box = torch.tensor([value], dtype=torch.float64, device=device)
        dist.all_reduce(box, op=dist.ReduceOp.MAX)
        return float(box.item())

    for label, ggml_type, rows, columns in shapes:
        first, count = sharding.shard_rows(rows, world, rank)
        shard_bytes = count * synth.row_bytes(ggml_type, columns)
        whole_bytes = rows * synth.row_bytes(ggml_type, columns)
        copies = max(2, min(6, math.ceil(256e6 / shard_bytes)))
        hold = [sb.QuantizedMatrix(synth.matrix(ggml_type, count, columns, seed=540 + c, name=f"c4.{rank}"), ggml_type, count, columns) for c in range(copies)]
        peers = None
        if world > 1 and use_peers:
            peers = sharding.PeerOutputs({"y": 64 * rows}, device)
            dist.barrier()
        full = peers.view("y") if peers is not None else torch.zeros(64 * rows, dtype=torch.float32, device=device)
        local = torch.zeros(64 * count, dtype=torch.float32, device=device)
        staged = torch.zeros(world * 64 * count, dtype=torch.float32, device=device) if world > 1 else None
        for batch in (1, 8, 64):
            xs = torch.from_numpy(synth.activations(batch, columns, seed=8)).to(device)
            need = max(lib.activation_scratch_bytes(batch, columns), lib.gemm_scratch_bytes(batch, columns))
            keep, work = _aligned_scratch(torch, device, need)
            sb.quantize_device(xs.data_ptr(), batch, columns, columns, work, need, stream.cuda_stream)
            stream.synchronize()
            point = {}

            def store(matrix, s, signal):
                if peers is not None:
                    own, others = peers.pointers("y", first)
                    words, arrivals = peers.signals("y") if signal else ((), 0)
                    matrix.matmul_q8_gather_device(work, batch, own, rows, others, stream=s.cuda_stream, signal_ptrs=words, arrivals_ptr=arrivals)
                else:
                    matrix.matmul_q8_device(work, batch, full.data_ptr() + 4 * first, rows, stream=s.cuda_stream)

            def kernel_only(s):
                for matrix in hold:
                    store(matrix, s, False)

            point["kernel_us"] = slowest(_time_graph(torch, stream, kernel_only, copies))
            if peers is not None:
                def with_signal(s):
                    for matrix in hold:
                        store(matrix, s, True)
                        sb.gather_wait_device(*peers.wait_arguments("y"), timeout_us=2_000_000, stream=s.cuda_stream)

                dist.barrier()
                point["with_exchange_us"] = slowest(_time_graph(torch, stream, with_signal, copies))
            if world > 1:
                # NCCL form, launched from the host: product into this rank's slice, all-gather, and for several columns the
                # reordering of the rank-major result into token-major rows
                def nccl_round():
                    for matrix in hold:
                        matrix.matmul_q8_device(work, batch, local.data_ptr(), count, stream=stream.cuda_stream)
                        if batch == 1:
                            dist.all_gather_into_tensor(full[:rows], local[:count])
                        else:
                            dist.all_gather_into_tensor(staged[:world * batch * count], local[:batch * count])
                            full[:batch * rows].view(batch, world, count).copy_(staged[:world * batch * count].view(world, batch, count).permute(1, 0, 2))

                dist.barrier()
                with torch.cuda.stream(stream):
                    nccl_round()
                    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    begin.record(stream)
                    for _ in range(5):
                        nccl_round()
                    end.record(stream)
                    stream.synchronize()
                point["nccl_all_gather_us"] = slowest(begin.elapsed_time(end) * 1e3 / (5 * copies))
            if batch == 64:
                xf = torch.randn(batch, columns, device=device)

                def tensor_cores(s):
                    for matrix in hold:
                        matrix.gemm_device(xf.data_ptr(), batch, columns, full.data_ptr() + 4 * first, rows, work, need, stream=s.cuda_stream)

                point["tensor_core_f16_us"] = slowest(_time_graph(torch, stream, tensor_cores, copies))
            for key in list(point):
                point[key.replace("_us", "_gbs")] = whole_bytes / point[key] / 1e3
            point["kernel_frac_of_hbm_peak_per_gpu"] = whole_bytes / world / point["kernel_us"] / 1e3 / peak
            out[f"{label}, batch {batch}"] = point
            del xs, keep
        if world > 1:
            dist.barrier()
        if peers is not None:
            peers.close()
        for matrix in hold:
            matrix.close()
        del full, local, staged
    return out


def batched_decode(dec, image):
    """The decoder on several tokens per step: 2 / 4 / 8 sessions decoding together (one token each per step, greedy pick
    on the device) and prompt runs of 64 and 512 tokens of one session in chunks of 64 (``syn_b200_decoder_forward_argmax``,
    host tokens in, token ids out). Same model image as the single-session `e2e`; only the slot and step sizes of the descriptor differ."""
    import copy

    wide = copy.copy(image)
    wide.shape = dict(image.shape, session_slots=8, step_tokens=64, logits_rows=8)
    out = {}
    with dec.Decoder(wide) as model:
        for sessions in (2, 4, 8):
            tokens = [11 + s for s in range(sessions)]
            for position in range(3):
                tokens = model.forward_argmax([(s, tokens[s], position, s) for s in range(sessions)])
            steps = 10
            start = time.perf_counter()
            for position in range(3, 3 + steps):
                tokens = model.forward_argmax([(s, tokens[s], position, s) for s in range(sessions)])
            seconds = time.perf_counter() - start
            out[f"{sessions} sessions"] = {"ms_per_step": seconds / steps * 1e3, "tokens_per_s": sessions * steps / seconds}

        def prompt(length):
            # chunks of 64 tokens (the reference's prefill chunk); only the last token asks for logits
            for first in range(0, length, 64):
                chunk = [(0, 100 + p, p, 0 if p == length - 1 else -1) for p in range(first, min(first + 64, length))]
                last = model.forward_argmax(chunk)
            return last

        for length in (64, min(512, image.shape["context"])):
            prompt(length)
            runs = 3 if length == 64 else 2
            start = time.perf_counter()
            for _ in range(runs):
                prompt(length)
            seconds = time.perf_counter() - start
            out[f"{length}-token prompt run"] = {"ms_per_run": seconds / runs * 1e3, "tokens_per_s": length * runs / seconds}
    return out


def parity_summary(sb, torch):
    """Counts for the record (the assertions live in tests/): how many outputs of the benchmark's dominant shape pass on
    the summation-order gate instead of the 1e-3 relative one, and which share of tensor-core outputs is inside 1e-3."""
    import oracle

    oracle.build()
    out = {}
    rows, columns = 18944, 3584
    weights = synth.matrix(synth.Q4_K, rows, columns, seed=301)
    x = synth.activations(8, columns, seed=302)
    codes, scales = oracle.quantize(x)
    chunk = 1184
    want = np.concatenate([oracle.kq_q8_matmul(synth.Q4_K, weights[r * 2016:(r + chunk) * 2016], chunk, columns, codes, scales) for r in range(0, rows, chunk)], axis=1)
    with sb.QuantizedMatrix(weights, synth.Q4_K, rows, columns) as matrix:
        for tokens in (1, 8):
            got = matrix.matvec(x[:tokens], sb.MODE_XQ8)
            outside = np.abs(got - want[:tokens]) > 1e-5 + 1e-3 * np.abs(want[:tokens])
            out[f"q4_k 18944x3584, {tokens} token(s), xq8 vs oracle"] = {"outside_rel_gate": int(outside.sum()), "count": int(outside.size),
                                                                        "max_abs_error": float(np.abs(got - want[:tokens]).max())}
    rows, tokens = 2048, 128
    weights = synth.matrix(synth.Q4_K, rows, columns, seed=51)
    x = synth.activations(tokens, columns, seed=52)
    want = oracle.f32_matmul_threads(synth.Q4_K, weights, rows, columns, x, os.cpu_count() or 1)
    with sb.QuantizedMatrix(weights, synth.Q4_K, rows, columns) as matrix:
        for name, precision in [("f16", sb.GEMM_F16)] + ([("f16x2", sb.GEMM_F16X2)] if hasattr(sb, "GEMM_F16X2") else []):
            got = matrix.gemm(x, precision)
            inside = np.abs(got - want) <= 1e-5 + 1e-3 * np.abs(want)
            out[f"q4_k 2048x3584 x 128 tokens, tensor cores {name} vs FP32-activation oracle"] = {
                "inside_1e-3_rel_1e-5_abs": float(inside.mean()), "max_error_of_output_range": float(np.abs(got - want).max() / (want.max() - want.min()))}
    return out


def cpu_avx2_baseline(budget_seconds=4.0):
    """The reference's AVX2 Q8_0 x Q8_0 kernel (restated in the oracle, rows chunked over all host threads like its worker
    pool) on config 0's matrix and on one layer + vocabulary projection of config 1."""
    import oracle

    oracle.build()
    threads = os.cpu_count() or 1
    out = {"threads": threads, "kernel": "AVX2 maddubs/madd + FMA (native/synapse-kernels/.../avx2.rs:19-157), restated in oracle/"}
    cases = [("config 0: q8_0 4864x896", [(4864, 896)]),
             ("config 1: one 0.5B layer + vocabulary projection, q8_0", [(896, 896), (128, 896), (128, 896), (896, 896), (4864, 896), (4864, 896), (896, 4864), (151936, 896)])]
    for label, shapes in cases:
        work = []
        for index, (rows, columns) in enumerate(shapes):
            weights = synth.matrix(synth.Q8_0, rows, columns, seed=560 + index, name="cpu")
            codes, scales = oracle.quantize(synth.activations(1, columns, seed=9))
            work.append((weights, rows, columns // 32, codes.reshape(-1), scales.reshape(-1), np.empty((1, rows), np.float32)))
        size = sum(rows * (columns // 32) * 34 for rows, columns in shapes)

        def once():
            for weights, rows, blocks, codes, scales, output in work:
                oracle.q8q8_matmul_threads(weights, rows, blocks, codes, scales, 1, threads, output)

        once()
        passes, start = 0, time.perf_counter()
        while True:
            once()
            passes += 1
            elapsed = time.perf_counter() - start
            if elapsed >= budget_seconds or passes >= 2000:
                break
        out[label] = {"weight_gbs": size * passes / elapsed / 1e9, "us_per_pass": elapsed / passes * 1e6, "bytes_per_pass": size, "passes": passes}
    return out
