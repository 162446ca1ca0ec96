#!/usr/bin/env python
"""Benchmark of the quantized matrix-product hot path on B200.

Workload (``config.workload``): the Qwen2.5-7B-shaped Q4_K_M decode matvec set at batch 1 -- per layer q/o
3584x3584, k 512x3584 (Q4_K), v 512x3584 (Q6_K), gate/up 18944x3584 (Q4_K), down 3584x18944 (Q6_K), 28 layers,
plus the 152064x3584 Q4_K LM head: 4,480,401,408 bytes of GGUF blocks per step. A step is one pass over every
matrix with seeded N(0,1) FP32 activations, quantised on the device exactly as the reference's activation
quantiser does. The metric is weight GB/s (source GGUF block bytes / time). Weights exceed L2 (126 MB) by 35x,
so no flush is needed between iterations.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One step launches one kernel per fused region of a layer, as the reference's executors do: q | k as two segments of one
launch with v (another encoding) beside it, o, gate | up with SwiGLU applied in registers, down; `--separate` launches
every matrix on its own. With N > 1 (launched under torchrun, one rank per GPU) every matrix is sharded by output rows
across the ranks; by default the product kernels store each result into every GPU's copy of the output vector over
NVLink (`--gather peer`), `--gather nccl` all-gathers the slices with NCCL after each product instead. The same total
work is split, so scaling is "strong". Before timing, every rank compares the gathered vectors with whole-matrix
products computed locally (`gather_verified`).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import bench_extras  # noqa: E402
from synapse_b200 import sharding, synth  # noqa: E402

METRIC = "k-quant decode matvec weight bandwidth (Qwen2.5-7B Q4_K_M set, batch 1)"
UNIT = "GB/s"
WORKLOAD = "qwen2.5-7b q4_k_m decode matvec set, batch 1 (config 2)"


def parse_args():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--layers", type=int, default=28, help="layers of the model shape (28 = the full config)")
    parser.add_argument("--no-graph", action="store_true", help="launch every kernel from the host instead of replaying a CUDA graph")
    parser.add_argument("--separate", action="store_true",
                        help="one launch per matrix (q | k | v and gate | up on parallel graph branches) instead of one launch per fused region")
    parser.add_argument("--no-e2e", action="store_true")
    parser.add_argument("--gather", default="peer", choices=["peer", "nccl"],
                        help="N > 1: output slices are stored into every GPU's copy by the product kernel itself (peer), or "
                             "all-gathered by NCCL after each product")
    parser.add_argument("--no-cpu", action="store_true")
    return parser.parse_args()


def model_matrices(layers):
    """(name, type, rows, columns) of every matrix of one step, in execution order."""
    out = []
    per_layer = [m for m in synth.QWEN25_7B_Q4KM if m[0] != "lm_head"]
    for layer in range(layers):
        for name, ggml_type, rows, columns, _ in per_layer:
            out.append((f"blk.{layer}.{name}", ggml_type, rows, columns))
    name, ggml_type, rows, columns, _ = [m for m in synth.QWEN25_7B_Q4KM if m[0] == "lm_head"][0]
    out.append((name, ggml_type, rows, columns))
    return out


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.device_index = device_index
        self.lines = []
        self.process = None
        self.thread = None

    def start(self):
        try:
            self.process = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                                             "-i", str(self.device_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.process = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.process.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, start_time, end_time):
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.process.terminate()
        try:
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        rows = [line.split(", ") for stamp, line in self.lines if start_time - 0.05 <= stamp <= end_time + 0.15]
        if not rows:
            rows = [line.split(", ") for _, line in self.lines[-3:]]
        clocks, max_clocks, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for row in rows:
            if len(row) < 9:
                continue
            try:
                clocks.append(float(row[1]))
                max_clocks.append(float(row[2]))
                power.append(float(row[3]))
            except ValueError:
                continue
            for name, value in zip(names, row[5:9]):
                if value.strip().lower() == "active":
                    reasons.add(name)
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": float(np.median(clocks)), "sm_max_mhz": float(max(max_clocks)), "power_w_max": float(max(power)),
                "samples": len(clocks), "reasons": sorted(reasons)}


def measured_peak_hbm():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as handle:
            return float(json.load(handle)["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        return 6650.0, "fallback"


def profile_traffic(bytes_per_launch):
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch of the roofline kernel, from the tracked ncu summary whose
    `traffic_bytes_per_launch` line was captured on a launch of exactly this many algorithmic bytes; None otherwise."""
    import glob
    import re

    for path in sorted(glob.glob(os.path.join(ROOT, "profiles", "*.md"))):
        try:
            text = open(path).read()
        except OSError:
            continue
        match = re.search(r"traffic_bytes_per_launch:\s*(\d+)\s+algorithmic_bytes_per_launch:\s*(\d+)", text)
        if match and int(match.group(2)) == bytes_per_launch:
            return int(match.group(1))
    return None


# ------------------------------------------------------------------------------------------------------------
# CPU arm: the reference's own CPU path (restated in oracle/), timed on this host's cores
# ------------------------------------------------------------------------------------------------------------

def cpu_reference_pass(oracle, sample, xs, threads):
    """One pass of the reference backend's K-quant product (decode the row, FP32 dot) over the sample."""
    for (name, ggml_type, rows, columns), weights in sample:
        oracle.f32_matmul_threads(ggml_type, weights, rows, columns, xs[columns], threads)


def cpu_sample(layers=1):
    """One transformer layer of the workload (149 MB of blocks): a bounded sample of the same matrices."""
    sample = []
    for name, ggml_type, rows, columns in model_matrices(layers)[:-1]:
        sample.append(((name, ggml_type, rows, columns), synth.matrix(ggml_type, rows, columns, seed=1, name=name)))
    xs = {3584: synth.activations(1, 3584, seed=2), 18944: synth.activations(1, 18944, seed=2)}
    sample_bytes = sum(rows * synth.row_bytes(t, cols) for (_, t, rows, cols), _ in sample)
    return sample, xs, sample_bytes


def run_cpu_baseline(budget_seconds=12.0):
    import oracle

    oracle.build()
    threads = os.cpu_count() or 1
    sample, xs, sample_bytes = cpu_sample(1)
    cpu_reference_pass(oracle, sample, xs, threads)  # warm-up
    passes, start = 0, time.perf_counter()
    while True:
        cpu_reference_pass(oracle, sample, xs, threads)
        passes += 1
        elapsed = time.perf_counter() - start
        if elapsed >= budget_seconds or passes >= 200:
            break
    return {"value": sample_bytes * passes / elapsed / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{passes} passes over one layer of the workload ({sample_bytes} bytes of Q4_K/Q6_K blocks): decode row + FP32 dot "
                      f"(the reference backend's K-quant path), rows chunked over {threads} threads"}


def run_reference_arm(args):
    """`--impl reference`: the reference's CPU implementation of the path on the host cores, on a bounded sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle

    oracle.build()
    threads = os.cpu_count() or 1
    sample, xs, sample_bytes = cpu_sample(1)
    for _ in range(max(args.warmup, 1)):
        cpu_reference_pass(oracle, sample, xs, threads)
    start = time.perf_counter()
    for _ in range(args.steps):
        cpu_reference_pass(oracle, sample, xs, threads)
    elapsed = time.perf_counter() - start
    value = sample_bytes * args.steps / elapsed / 1e9
    sample_text = (f"each step = one layer of the workload ({sample_bytes} bytes of Q4_K/Q6_K blocks), decode row + FP32 dot "
                   f"(reference backend K-quant path), {threads} threads")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": elapsed / args.steps * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "sample": sample_text},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample_text},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------------------

def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return

    # Libraries print to standard output (NCCL its version line): the one JSON line must be alone there, so everything
    # else goes to standard error and the line is written to the saved descriptor at the end.
    sys.stdout.flush()
    result_fd = os.dup(1)
    os.dup2(2, 1)

    import torch
    import torch.distributed as dist

    import synapse_b200 as sb

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    lib = sb.library()
    lib.probe()

    # ---- weights: one random-init model image (the stand-in for the mapped GGUF file); every rank holds rows
    # [rank*R/world, (rank+1)*R/world) of every projection matrix ------------------------------------------------
    from synapse_b200 import decoder as dec

    shape = dict(dec.QWEN25_7B, layers=args.layers)
    image = dec.ModelImage(**shape, context=512, matrix_types=dec.Q4KM_TYPES, embedding_type=synth.Q4_K, output_type=synth.Q4_K, seed=100,
                           bias=True)
    leaf_fields = {"attn_q": "query", "attn_k": "key", "attn_v": "value", "attn_o": "attention_output", "ffn_gate": "gate", "ffn_up": "up",
                   "ffn_down": "down"}

    def image_bytes(name, rows, columns, ggml_type, first_row, row_count):
        leaf = name.split(".")[-1]
        base = image.output if leaf == "lm_head" else getattr(image.layers[int(name.split(".")[1])], leaf_fields[leaf])
        row_bytes = synth.row_bytes(ggml_type, columns)
        return image.weights[base + first_row * row_bytes:base + (first_row + row_count) * row_bytes]

    matrices = []
    total_bytes = 0
    for name, ggml_type, rows, columns in model_matrices(args.layers):
        first_row, shard_rows = sharding.shard_rows(rows, world, rank)
        shard = image_bytes(name, rows, columns, ggml_type, first_row, shard_rows)
        matrices.append((name, ggml_type, rows, columns, shard_rows, sb.QuantizedMatrix(shard, ggml_type, shard_rows, columns)))
        total_bytes += rows * synth.row_bytes(ggml_type, columns)
    by_name = {m[0]: m for m in matrices}

    # ---- activations (resident) and outputs -----------------------------------------------------------------
    # Output vectors of a step, full length on every rank: q | k | v share one vector (the row space of the reference's
    # QKV region), gate and up produce the feed-forward vector silu(gate) * up.
    hidden, ffn, kvw, vocabulary = shape["hidden"], shape["feed_forward"], shape["kv_heads"] * (shape["hidden"] // shape["heads"]), shape["vocabulary"]
    vectors = {"qkv": hidden + 2 * kvw, "attn_o": hidden, "ffn": ffn, "gate": ffn, "up": ffn, "ffn_down": hidden, "lm_head": vocabulary}
    x_host = {hidden: synth.activations(1, hidden, seed=5), ffn: synth.activations(1, ffn, seed=6)}
    x_dev = {k: torch.from_numpy(v).to(device) for k, v in x_host.items()}
    scratch = {k: torch.empty(lib.activation_scratch_bytes(1, k) + 256, dtype=torch.uint8, device=device) for k in x_host}
    peers = None
    if world > 1 and args.gather == "peer":
        # every rank's full output vectors live in one buffer that all other ranks map: the kernels gather by storing
        try:
            peers = sharding.PeerOutputs(vectors, device)
        except Exception as error:
            sys.stderr.write(f"rank {rank}: peer mapping failed ({error}); gathering with NCCL\n")
            peers = None
        agreed = torch.tensor([1 if peers is not None else 0], device=device)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        if int(agreed.item()) == 0 and peers is not None:
            peers.close()
            peers = None
    if peers is not None:
        out_full = {name: peers.view(name) for name in vectors}
    else:
        out_full = {name: torch.zeros(length, dtype=torch.float32, device=device) for name, length in vectors.items()}
    out_shard = {m[0].split(".")[-1]: torch.zeros(m[4], dtype=torch.float32, device=device) for m in matrices}
    # one launch per fused region (q | k, gate | up) unless told otherwise; NCCL gathers work per matrix
    fused_regions = not args.separate and (world == 1 or peers is not None)

    def aligned(tensor):
        return (tensor.data_ptr() + 255) // 256 * 256

    side = [torch.cuda.Stream(device), torch.cuda.Stream(device)]

    def destination(vector, column):
        """(own pointer, peer pointers) of element `column` of this rank's copy of `vector` and of every other rank's."""
        if peers is not None:
            return peers.pointers(vector, column)
        return out_full[vector].data_ptr() + 4 * column, []

    def product(entry, vector, column, stream, signal=False):
        """One matrix (this rank's rows of it) into `vector` at `column` + the rank's first row; with `signal` the launch
        also writes its sequence number into this rank's word of every GPU's signal array of the vector."""
        name, ggml_type, rows, columns, shard_rows, matrix = entry
        first_row, _ = sharding.shard_rows(rows, world, rank)
        if world > 1 and peers is None:
            target = out_shard[name.split(".")[-1]]
            matrix.matmul_q8_device(aligned(scratch[columns]), 1, target.data_ptr(), shard_rows, stream=stream.cuda_stream)
            with torch.cuda.stream(stream):
                sharding.gather_outputs(target, out_full[vector][column:column + rows])
            return
        own, others = destination(vector, column + first_row)
        if others:
            words, arrivals = peers.signals(vector) if signal else ((), 0)
            matrix.matmul_q8_gather_device(aligned(scratch[columns]), 1, own, shard_rows, others, stream=stream.cuda_stream, signal_ptrs=words,
                                           arrivals_ptr=arrivals)
        else:
            matrix.matmul_q8_device(aligned(scratch[columns]), 1, own, shard_rows, stream=stream.cuda_stream)

    def segments(entries, vector, columns_out, stream):
        """Several matrices of one encoding against the same activations in ONE launch (Q | K)."""
        parts, peer_lists = [], None
        for entry, column in zip(entries, columns_out):
            name, ggml_type, rows, columns, shard_rows, matrix = entry
            first_row, _ = sharding.shard_rows(rows, world, rank)
            parts.append((matrix, 0, shard_rows, 0, column + first_row))
        own, others = destination(vector, 0)
        sb.matmul_q8_segments_device(parts, aligned(scratch[entries[0][3]]), 1, own, vectors[vector], peer_ptrs=others, stream=stream.cuda_stream)

    def gate_up(gate_entry, up_entry, stream):
        """silu(gate . x) * (up . x) for this rank's rows in ONE launch."""
        name, ggml_type, rows, columns, shard_rows, gate_matrix = gate_entry
        first_row, _ = sharding.shard_rows(rows, world, rank)
        own, others = destination("ffn", first_row)
        sb.matmul_q8_swiglu_device(gate_matrix, up_entry[5], aligned(scratch[columns]), 1, own, shard_rows, peer_ptrs=others, stream=stream.cuda_stream)

    def quantize(columns, stream):
        sb.quantize_device(x_dev[columns].data_ptr(), 1, columns, columns, aligned(scratch[columns]),
                           lib.activation_scratch_bytes(1, columns), stream.cuda_stream)

    def parallel(calls, main):
        """Independent launches that read the same activations: the first on the main stream, the others on side streams
        (parallel branches of the captured graph)."""
        if (world > 1 and peers is None) or len(calls) == 1:
            for call in calls:
                call(main)
            return
        fork = torch.cuda.Event()
        fork.record(main)
        for call, stream in zip(calls[1:], side):
            stream.wait_event(fork)
            call(stream)
        calls[0](main)
        for _, stream in zip(calls[1:], side):
            join = torch.cuda.Event()
            join.record(stream)
            main.wait_event(join)

    def step(main):
        """One pass. Activations are quantised once per distinct input of a layer, as the reference's executor does
        (Qwen2CpuExecutor.cs:165-185). Q | K run as one launch of two segments with V (Q6_K, another encoding) beside it
        on a parallel branch, gate | up as one launch that applies SwiGLU in registers; `--separate` launches every matrix
        on its own (q | k | v and gate | up on parallel branches), the form earlier figures were measured in."""
        for layer in range(args.layers):
            get = lambda leaf: by_name[f"blk.{layer}.{leaf}"]
            quantize(hidden, main)
            if fused_regions:
                parallel([lambda s: segments([get("attn_q"), get("attn_k")], "qkv", [0, hidden], s),
                          lambda s: product(get("attn_v"), "qkv", hidden + kvw, s)], main)
            else:
                parallel([lambda s: product(get("attn_q"), "qkv", 0, s), lambda s: product(get("attn_k"), "qkv", hidden, s),
                          lambda s: product(get("attn_v"), "qkv", hidden + kvw, s)], main)
            quantize(hidden, main)
            product(get("attn_o"), "attn_o", 0, main)
            quantize(hidden, main)
            if fused_regions:
                gate_up(get("ffn_gate"), get("ffn_up"), main)
            else:
                parallel([lambda s: product(get("ffn_gate"), "gate", 0, s), lambda s: product(get("ffn_up"), "up", 0, s)], main)
            quantize(ffn, main)
            product(get("ffn_down"), "ffn_down", 0, main)
        quantize(hidden, main)
        product(by_name["lm_head"], "lm_head", 0, main, signal=True)
        if peers is not None:
            # The step's completion on this rank: every rank's last product has signalled, and a rank's products are
            # stream-ordered, so all slices of all vectors of the step have landed in this GPU's copies.
            sb.gather_wait_device(*peers.wait_arguments("lm_head"), timeout_us=2_000_000, stream=main.cuda_stream)

    stream = torch.cuda.Stream(device)
    graph = None
    lib.launch_count(reset=True)
    with torch.cuda.stream(stream):
        step(stream)
    torch.cuda.synchronize()
    launches_per_step = lib.launch_count(reset=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- N > 1: before anything is timed, every rank checks the vectors the step has just gathered against the same
    # products of the WHOLE matrices computed locally (the last layer's, whose results the vectors hold, and the
    # vocabulary projection): they must be equal bit for bit, since a row's value does not depend on its shard.
    gather_verified = None
    if world > 1:
        barrier()  # every rank's stores (or gathers) of the first step have landed
        last = args.layers - 1
        checks, mismatches = 0, 0

        def whole(name):
            _, ggml_type, rows, columns, _, _ = by_name[name]
            return sb.QuantizedMatrix(image_bytes(name, rows, columns, ggml_type, 0, rows), ggml_type, rows, columns)

        with torch.cuda.stream(stream):
            expected = {name: torch.zeros(length, dtype=torch.float32, device=device) for name, length in vectors.items()}
            for columns in (hidden, ffn):
                quantize(columns, stream)
            plan = [("qkv", 0, f"blk.{last}.attn_q"), ("qkv", hidden, f"blk.{last}.attn_k"), ("qkv", hidden + kvw, f"blk.{last}.attn_v"),
                    ("attn_o", 0, f"blk.{last}.attn_o"), ("ffn_down", 0, f"blk.{last}.ffn_down"), ("lm_head", 0, "lm_head")]
            for vector, column, name in plan:
                with whole(name) as matrix:
                    matrix.matmul_q8_device(aligned(scratch[matrix.columns]), 1, expected[vector].data_ptr() + 4 * column, matrix.rows, stream=stream.cuda_stream)
                    stream.synchronize()
            with whole(f"blk.{last}.ffn_gate") as gate_whole, whole(f"blk.{last}.ffn_up") as up_whole:
                if fused_regions:
                    sb.matmul_q8_swiglu_device(gate_whole, up_whole, aligned(scratch[hidden]), 1, expected["ffn"].data_ptr(), ffn, stream=stream.cuda_stream)
                else:
                    gate_whole.matmul_q8_device(aligned(scratch[hidden]), 1, expected["gate"].data_ptr(), ffn, stream=stream.cuda_stream)
                    up_whole.matmul_q8_device(aligned(scratch[hidden]), 1, expected["up"].data_ptr(), ffn, stream=stream.cuda_stream)
                stream.synchronize()
        for name in vectors:
            if name in (("gate", "up") if fused_regions else ("ffn",)):
                continue  # vectors this form of the step does not produce
            checks += 1
            if not torch.equal(out_full[name], expected[name]):
                mismatches += 1
                sys.stderr.write(f"rank {rank}: gathered vector {name} differs from the whole-matrix product\n")
        mismatch_total = torch.tensor([mismatches], device=device)
        dist.all_reduce(mismatch_total)
        gather_verified = {"ok": int(mismatch_total.item()) == 0, "vectors_per_rank": checks, "ranks": world,
                           "how": "bitwise equal to the whole-matrix products computed on every rank"}
        del expected

    use_graph = not args.no_graph
    if use_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                step(torch.cuda.current_stream())
        except Exception as error:  # a collective that cannot be captured: replay from the host instead
            if world == 1:
                raise
            sys.stderr.write(f"rank {rank}: graph capture failed ({error}); launching from the host\n")
            graph = None
            use_graph = False
            torch.cuda.synchronize()

    def run_step():
        if graph is not None:
            graph.replay()
        else:
            step(stream)

    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            run_step()
        barrier()
        sampler = ClockSampler(local_rank)
        sampler.start()
        time.sleep(0.25)
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        wall_start = time.time()
        begin.record(stream)
        for _ in range(args.steps):
            run_step()
        end.record(stream)
        barrier()
        wall_end = time.time()
    elapsed_ms = begin.elapsed_time(end)
    if world > 1:
        slowest = torch.tensor([elapsed_ms], dtype=torch.float64, device=device)
        dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
        elapsed_ms = float(slowest.item())
    clocks = sampler.stop(wall_start, wall_end)
    ms_per_step = elapsed_ms / args.steps
    value = total_bytes / (ms_per_step * 1e-3) / 1e9

    # ---- roofline of the dominant kernel: the gate | up launch (two Q4_K matrices of 38 MB, one launch) --------
    gates = [m for m in matrices if m[0].endswith("ffn_gate")]
    ups = [m for m in matrices if m[0].endswith("ffn_up")]
    per_matrix_bytes = gates[0][4] * synth.row_bytes(gates[0][1], gates[0][3])
    per_launch_bytes = (2 if fused_regions else 1) * per_matrix_bytes
    # Every gate/up pair once per pass (28 x 76 MB, no L2 reuse), launches back to back in stream order; timed with
    # CUDA events on the launch stream around whole passes, so the figure includes the gaps between launches.
    def roofline_pass(main):
        for gate_entry, up_entry in zip(gates, ups):
            if fused_regions:
                gate_up(gate_entry, up_entry, main)
            else:
                product(gate_entry, "gate", 0, main)
                product(up_entry, "up", 0, main)

    with torch.cuda.stream(stream):
        roofline_pass(stream)
        stream.synchronize()
    roofline_graph = None
    if use_graph:
        roofline_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(roofline_graph, stream=stream):
            roofline_pass(torch.cuda.current_stream())
    passes = 5
    with torch.cuda.stream(stream):
        roofline_graph.replay() if roofline_graph is not None else roofline_pass(stream)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(passes):
            roofline_graph.replay() if roofline_graph is not None else roofline_pass(stream)
        e1.record(stream)
        stream.synchronize()
    launches_timed = passes * len(gates) * (1 if fused_regions else 2)
    kernel_ms = e0.elapsed_time(e1) / launches_timed
    peak, peak_kind = measured_peak_hbm()
    achieved = per_launch_bytes / (kernel_ms * 1e-3) / 1e9
    kernel_name = ("matvec_xq8_pipe_kernel<Q4KXq8, T=1, W=1, UPL=1, R=2, CW=8, kPair> on ffn_gate | ffn_up (2 x 18944x3584, SwiGLU in registers)"
                   if fused_regions else "matvec_xq8_pipe_kernel<Q4KXq8, T=1, W=1, UPL=1, R=2, CW=8> on ffn_gate / ffn_up (18944x3584)")
    roofline = {"bound": "hbm", "kernel": kernel_name, "achieved": achieved, "peak": peak, "peak_kind": f"of {peak_kind}", "unit": "GB/s",
                "frac": achieved / peak, "traffic": profile_traffic(per_launch_bytes) if world == 1 else None,
                "bytes_per_launch": per_launch_bytes, "us_per_launch": kernel_ms * 1e3, "launches_timed": launches_timed}

    # ---- end to end, host buffers in and out ----------------------------------------------------------------------
    e2e = None
    per_matrix = None
    if not args.no_e2e and world > 1:
        # N > 1: the row-sharded step through the device entry points with the exchange inside: every step copies the
        # activations from pinned host memory, runs the gathered step (whose last kernel waits, bounded, until every
        # rank's slices of the vocabulary vector have landed), meets the other ranks so that nobody's next step stores
        # into a vector that is still being copied, and reads the gathered vocabulary vector back to the host.
        host_x = {k: torch.from_numpy(v).pin_memory() for k, v in x_host.items()}
        host_logits = torch.zeros(vocabulary, dtype=torch.float32).pin_memory()

        def e2e_step():
            with torch.cuda.stream(stream):
                for columns, tensor in x_dev.items():
                    tensor.copy_(host_x[columns].view_as(tensor), non_blocking=True)
                run_step()
            barrier()
            with torch.cuda.stream(stream):
                host_logits.copy_(out_full["lm_head"], non_blocking=True)
                stream.synchronize()

        e2e_steps = max(3, min(args.steps, 20))
        for _ in range(3):
            e2e_step()
        barrier()
        start = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        e2e_seconds = time.perf_counter() - start
        slowest = torch.tensor([e2e_seconds], dtype=torch.float64, device=device)
        dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
        e2e_seconds = float(slowest.item())
        e2e = {"value": total_bytes * e2e_steps / e2e_seconds / 1e9, "unit": UNIT, "h2d_bytes_per_step": 4 * (hidden + ffn),
               "d2h_bytes_per_step": 4 * vocabulary, "ms_per_step": e2e_seconds / e2e_steps * 1e3, "steps": e2e_steps,
               "api": "row-sharded step through the device entry points (" + ("syn_b200_matmul_q8_segments_dev / _swiglu_dev / _gather_dev storing "
                      "into every GPU's copy" if peers is not None else "syn_b200_matmul_q8_dev + NCCL all-gather per product") +
                      "): pinned host activations in; the step ends with the bounded device-side wait for every rank's completion word of the vocabulary "
                      "vector, a barrier across the ranks keeps the next step's stores out of the vector while it is copied, gathered vector out"}
    if not args.no_e2e and world == 1:
        # (a) the per-projection boundary: one host call per matrix, pinned host x in, host y out
        host_x = {k: torch.from_numpy(v).pin_memory() for k, v in x_host.items()}
        host_y = {m[4]: torch.zeros(m[4], dtype=torch.float32).pin_memory() for m in matrices}
        torch.cuda.synchronize()
        h2d = sum(4 * m[3] for m in matrices)
        d2h = sum(4 * m[4] for m in matrices)

        def e2e_step():
            for name, ggml_type, rows, columns, shard_rows, matrix in matrices:
                lib.check(lib.raw.syn_b200_matvec(matrix.handle, 0, shard_rows, host_x[columns].data_ptr(), 1, columns,
                                                  host_y[shard_rows].data_ptr(), shard_rows, sb.MODE_XQ8, sb.EPILOGUE_STORE))

        e2e_steps = max(3, min(args.steps, 10))
        for _ in range(3):
            e2e_step()
        barrier()
        start = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        barrier()
        e2e_seconds = time.perf_counter() - start
        per_matrix = {"value": total_bytes * e2e_steps / e2e_seconds / 1e9, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                      "ms_per_step": e2e_seconds / e2e_steps * 1e3, "steps": e2e_steps,
                      "api": "syn_b200_matvec (host FP32 activations in, host FP32 outputs out, one call per matrix)"}
        e2e = per_matrix
        if world == 1:
            # (b) the per-step boundary a generation loop uses: syn_b200_decoder_forward, host tokens in, host logits out.
            # The step runs the same 197 projections plus the kernels between them (norms, rotary, attention, SwiGLU).
            for entry in matrices:
                entry[5].close()
            with dec.Decoder(image) as model:
                token = 11
                for position in range(3):
                    token = int(np.argmax(model.decode(token, position)))
                torch.cuda.synchronize()
                decode_steps = max(3, min(args.steps, 20))
                start = time.perf_counter()
                for position in range(3, 3 + decode_steps):
                    token = int(np.argmax(model.decode(token, position)))
                decode_seconds = time.perf_counter() - start
                # the same step with the greedy pick on the device (4 bytes back instead of the logits)
                start = time.perf_counter()
                for position in range(3 + decode_steps, 3 + 2 * decode_steps):
                    token = model.forward_argmax([(0, token, position, 0)])[0]
                argmax_seconds = time.perf_counter() - start
            e2e = {"value": total_bytes * decode_steps / decode_seconds / 1e9, "unit": UNIT, "h2d_bytes_per_step": 16,
                   "d2h_bytes_per_step": 4 * shape["vocabulary"], "ms_per_step": decode_seconds / decode_steps * 1e3, "steps": decode_steps,
                   "tokens_per_s": decode_steps / decode_seconds,
                   "api": "syn_b200_decoder_forward (one call per decoded token: host BatchToken in, host logits out, greedy pick on the "
                          "host); the step is a replayed CUDA graph of one kernel per fused region"}
            e2e["argmax_api_tokens_per_s"] = decode_steps / argmax_seconds

    extras = None
    if world == 1 and not args.no_e2e:
        extras = {}
        # the same model through the decoder with several tokens per step (projections on the integer tensor cores)
        extras["qwen2.5-7b_q4_k_m_batched_decode"] = bench_extras.batched_decode(dec, image)
        # config 3: the tensor-core product over the token counts and matrices the baseline names
        extras["prefill"] = bench_extras.prefill_sweep(sb, lib, torch, device, stream, ROOT)
        # config 1: the Qwen2.5-0.5B-shaped all-Q8_0 decode step through the decoder, greedy pick on the device
        small = dec.ModelImage(**dec.QWEN25_05B, context=64, matrix_types=dec.Q8_TYPES, seed=101)
        with dec.Decoder(small) as model:
            token = 11
            for position in range(3):
                token = model.forward_argmax([(0, token, position, 0)])[0]
            start = time.perf_counter()
            for position in range(3, 35):
                token = model.forward_argmax([(0, token, position, 0)])[0]
            seconds = time.perf_counter() - start
        extras["qwen2.5-0.5b_q8_0_decode"] = {"tokens_per_s": 32 / seconds, "weight_gbs": small.matrix_bytes * 32 / seconds / 1e9,
                                               "api": "syn_b200_decoder_forward_argmax, one call per token"}

    if extras is not None:
        # single-kernel figures on the other shapes the baseline names: config 0 (Q8_0 4864x896), config 4's matrices at
        # batch 1 on one GPU, and the vocabulary projection in both encodings a Q4_K_M file may use for it
        def kernel_rate(ggml_type, rows, columns, copies, tokens=1):
            hold = [sb.QuantizedMatrix(synth.matrix(ggml_type, rows, columns, seed=200 + c, name="shape"), ggml_type, rows, columns)
                    for c in range(copies)]
            xs = torch.from_numpy(synth.activations(tokens, columns, seed=7)).to(device)
            need = lib.activation_scratch_bytes(tokens, columns)
            work = torch.empty(need + 256, dtype=torch.uint8, device=device)
            work_ptr = (work.data_ptr() + 255) // 256 * 256
            ys = torch.zeros(tokens * rows, dtype=torch.float32, device=device)
            sb.quantize_device(xs.data_ptr(), tokens, columns, columns, work_ptr, need, stream.cuda_stream)

            def once(s):
                for _ in range(4):
                    for matrix in hold:
                        matrix.matmul_q8_device(work_ptr, tokens, ys.data_ptr(), rows, stream=s.cuda_stream)

            with torch.cuda.stream(stream):
                once(stream)
                stream.synchronize()
            replay = torch.cuda.CUDAGraph()
            with torch.cuda.graph(replay, stream=stream):
                once(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                for _ in range(3):
                    replay.replay()
                t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0.record(stream)
                for _ in range(10):
                    replay.replay()
                t1.record(stream)
                stream.synchronize()
            microseconds = t0.elapsed_time(t1) * 1e3 / (10 * 4 * copies)
            size = rows * synth.row_bytes(ggml_type, columns)
            del replay
            for matrix in hold:
                matrix.close()
            return {"us": microseconds, "weight_gbs": size / microseconds / 1e3, "frac_of_hbm_peak": size / microseconds / 1e3 / peak}

        extras["matvec_shapes_batch1"] = {
            "q8_0 4864x896 (config 0; 40 copies rotate, 185 MB)": kernel_rate(synth.Q8_0, 4864, 896, 40),
            "q8_0 18944x3584": kernel_rate(synth.Q8_0, 18944, 3584, 3),
            "q4_k 28672x8192 (config 4)": kernel_rate(synth.Q4_K, 28672, 8192, 2),
            "q4_k 8192x28672 (config 4)": kernel_rate(synth.Q4_K, 8192, 28672, 2),
            "q4_k 152064x3584 (vocabulary projection)": kernel_rate(synth.Q4_K, 152064, 3584, 1),
            "q6_k 152064x3584 (vocabulary projection as Q6_K)": kernel_rate(synth.Q6_K, 152064, 3584, 1),
        }
        # several tokens per launch (batched decode, speculative verification): every weight is read once per launch
        extras["matvec_q4_k_18944x3584_tokens"] = {str(t): kernel_rate(synth.Q4_K, 18944, 3584, 4, tokens=t) for t in (2, 4, 8)}
        extras["matvec_q6_k_3584x18944_tokens"] = {str(t): kernel_rate(synth.Q6_K, 3584, 18944, 3, tokens=t) for t in (2, 4, 8)}
        # the FP32-activation contract of the reference backend on the two big layer shapes
        extras["matvec_xf32_batch1"] = bench_extras.xf32_rates(sb, lib, torch, device, stream, peak)

    # config 4 at this N: the 70B-class shapes and the vocabulary projection, row-sharded, at 1 / 8 / 64 columns
    stored_by_kernel = peers is not None
    if not args.no_e2e:
        if world > 1:
            for entry in matrices:
                entry[5].close()
            dist.barrier()  # nobody stores into a peer's buffer any more
            if peers is not None:
                out_full = None
                peers.close()
                peers = None
            dist.barrier()
        sweep = bench_extras.config4_sweep(sb, lib, torch, dist, device, stream, world, rank, peak, args.gather == "peer")
        if extras is None:
            extras = {}
        extras["config4_row_sharded_sweep"] = sweep

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = run_cpu_baseline()
        if extras is not None:
            # the oracle as the checker (counts for the record; the assertions are in tests/) and the reference's AVX2
            # Q8_0 x Q8_0 kernel on the host cores for configs 0 and 1
            extras["parity"] = bench_extras.parity_summary(sb, torch)
            extras["cpu_avx2_q8_0"] = bench_extras.cpu_avx2_baseline()

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
                "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "i8 dot / f32 accumulate",
                "data": "synthetic",
                "config": {"workload": WORKLOAD, "layers": args.layers, "matrices": len(matrices), "bytes_per_step": total_bytes,
                           "activation_contract": "xq8 (Q8_0 activation quantiser reproduced on device)",
                           "layout": "Q4_K file layout; Q6_K repacked to planes at load", "cuda_graph": bool(graph is not None),
                           "launches": ("one per fused region: q|k (two segments) with v beside it, o, gate|up with SwiGLU in registers, down" if fused_regions
                                        else "one per matrix, q|k|v and gate|up on parallel graph branches"),
                           "projection_launches_per_step": (5 if fused_regions else 7) * args.layers + 1,
                           "l2": "weights per step exceed L2 35x, no flush", "parallelism": (f"row-shard x{world}, " + ("slices stored into every GPU's copy by the product kernel; every step ends with a bounded wait for all ranks' completion signals" if stored_by_kernel
                                                                     else "NCCL all-gather per product")) if world > 1 else "single gpu",
                           "tokens_per_s": 1e3 / ms_per_step},
                "gather_verified": gather_verified, "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "e2e_per_matrix_calls": per_matrix, "extras": extras, "clocks": clocks,
                "gpu_launches": int(launches_per_step * args.steps)}
        sys.stdout.flush()
        os.write(result_fd, (json.dumps(line) + "\n").encode())
    if world > 1:
        # Captured collectives keep the communicator busy at teardown on some NCCL builds: release the graphs first and
        # do not let a stuck destroy hold the job (the result line is already printed).
        sys.stdout.flush()
        graph = None
        roofline_graph = None
        torch.cuda.synchronize()
        watchdog = threading.Timer(20.0, lambda: os._exit(0))
        watchdog.daemon = True
        watchdog.start()
        dist.barrier()
        dist.destroy_process_group()
        watchdog.cancel()


if __name__ == "__main__":
    main()
