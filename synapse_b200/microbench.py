"""Times one product kernel of the library on a seeded synthetic matrix.

    python -m synapse_b200.microbench --type q4_k --rows 18944 --cols 3584 --tokens 1 --copies 8 --mode xq8

``--copies`` distinct matrices are rotated so that consecutive launches never find their weights in L2
(8 x 38 MB > 126 MB). Prints one JSON line: microseconds per launch (CUDA events on the launch stream) and
GB/s of source GGUF block bytes. Small enough to run under a profiler: ``--reps 1 --warmup 0`` with ``--cycles 1`` gives
exactly ``copies`` launches of the kernel.
"""
from __future__ import annotations

import argparse
import json

import numpy as np


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--type", default="q4_k", choices=["q8_0", "q4_k", "q6_k"])
    parser.add_argument("--rows", type=int, default=18944)
    parser.add_argument("--cols", type=int, default=3584)
    parser.add_argument("--tokens", type=int, default=1)
    parser.add_argument("--copies", type=int, default=8)
    parser.add_argument("--cycles", type=int, default=4, help="times every copy is launched inside one graph (amortises the graph launch)")
    parser.add_argument("--reps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--mode", default="xq8", choices=["xq8", "xf32", "gemm", "decode", "pair"],
                        help="pair: consecutive copies are the gate and up matrix of one launch that stores silu(gate . x) * (up . x)")
    parser.add_argument("--layers", type=int, default=4, help="decode mode: layers of the Qwen2.5-7B-shaped Q4_K_M model")
    parser.add_argument("--context", type=int, default=64, help="decode mode: positions of the KV cache")
    parser.add_argument("--position", type=int, default=0, help="decode mode: position of the first step (the cache before it holds zeros)")
    parser.add_argument("--kv-fp16", action="store_true", help="decode mode: FP16 KV cache (kv_precision 1)")
    parser.add_argument("--no-repack", action="store_true")
    parser.add_argument("--fused-quantize", action="store_true", help="time quantise + product together (xq8)")
    parser.add_argument("--no-graph", action="store_true", help="launch from the host each time instead of replaying one CUDA graph")
    args = parser.parse_args()

    import torch

    import synapse_b200 as sb
    from synapse_b200 import synth

    if args.mode == "decode":
        return decode(args)

    ggml_type = {"q8_0": sb.Q8_0, "q4_k": sb.Q4_K, "q6_k": sb.Q6_K}[args.type]
    lib = sb.library()
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    matrices = []
    for copy in range(args.copies):
        blocks = synth.matrix(ggml_type, args.rows, args.cols, seed=copy, name="microbench")
        matrices.append(sb.QuantizedMatrix(blocks, ggml_type, args.rows, args.cols, repack=not args.no_repack))
    x = torch.from_numpy(synth.activations(args.tokens, args.cols, seed=99)).to(device)
    y = torch.zeros(args.tokens, args.rows, dtype=torch.float32, device=device)
    scratch_bytes = max(lib.activation_scratch_bytes(args.tokens, args.cols), lib.gemm_scratch_bytes(args.tokens, args.cols))
    scratch = torch.empty(scratch_bytes + 256, dtype=torch.uint8, device=device)
    scratch_ptr = (scratch.data_ptr() + 255) // 256 * 256
    stream = torch.cuda.Stream(device)
    sb.quantize_device(x.data_ptr(), args.tokens, args.cols, args.cols, scratch_ptr, scratch_bytes, stream.cuda_stream)

    def launch(matrix, stream_ptr):
        if args.mode == "gemm":
            matrix.gemm_device(x.data_ptr(), args.tokens, args.cols, y.data_ptr(), args.rows, scratch_ptr, scratch_bytes, stream=stream_ptr)
        elif args.mode == "xf32":
            matrix.matvec_device(x.data_ptr(), args.tokens, args.cols, y.data_ptr(), args.rows, sb.MODE_XF32, stream=stream_ptr)
        elif args.fused_quantize:
            matrix.matvec_device(x.data_ptr(), args.tokens, args.cols, y.data_ptr(), args.rows, sb.MODE_XQ8, scratch_ptr=scratch_ptr,
                                 scratch_bytes=scratch_bytes, stream=stream_ptr)
        else:
            matrix.matmul_q8_device(scratch_ptr, args.tokens, y.data_ptr(), args.rows, stream=stream_ptr)

    def one_round(stream_ptr):
        for _ in range(args.cycles):
            if args.mode == "pair":
                for gate, up in zip(matrices[0::2], matrices[1::2]):
                    sb.matmul_q8_swiglu_device(gate, up, scratch_ptr, args.tokens, y.data_ptr(), args.rows, stream=stream_ptr)
                continue
            for matrix in matrices:
                launch(matrix, stream_ptr)

    graph = None
    with torch.cuda.stream(stream):
        one_round(stream.cuda_stream)
        stream.synchronize()
    if not args.no_graph:
        # One graph holds a full round (every copy once): replaying it removes the host's launch cost from the timing.
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            one_round(torch.cuda.current_stream().cuda_stream)
    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            graph.replay() if graph is not None else one_round(stream.cuda_stream)
        stream.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record(stream)
        for _ in range(args.reps):
            graph.replay() if graph is not None else one_round(stream.cuda_stream)
        end.record(stream)
        stream.synchronize()
    per_launch = 2 if args.mode == "pair" else 1
    launches = args.reps * (args.copies // per_launch) * args.cycles
    microseconds = begin.elapsed_time(end) * 1e3 / launches
    source_bytes = matrices[0].source_bytes * per_launch
    print(json.dumps({"type": args.type, "rows": args.rows, "cols": args.cols, "tokens": args.tokens, "mode": args.mode,
                      "repack": not args.no_repack, "copies": args.copies, "cycles": args.cycles, "graph": graph is not None, "us_per_launch": microseconds,
                      "weight_gbs": source_bytes / microseconds / 1e3,
                      "tflops": 2.0 * args.rows * args.cols * args.tokens / microseconds / 1e6,
                      "checksum": float(y.double().sum().item())}))


def decode(args):
    """Whole single-token decode steps of a Qwen2.5-7B-shaped Q4_K_M model with ``--layers`` layers (a few layers keep
    the device footprint small enough for a profiler): ``--warmup`` + ``--reps`` steps, one kernel launch each."""
    import time

    import synapse_b200 as sb
    from synapse_b200 import decoder as dec
    from synapse_b200 import synth

    image = dec.ModelImage(**dict(dec.QWEN25_7B, layers=args.layers), context=args.context, matrix_types=dec.Q4KM_TYPES, embedding_type=synth.Q4_K,
                           output_type=synth.Q4_K, seed=100)
    image.kv_precision = 1 if args.kv_fp16 else 0
    with dec.Decoder(image) as model:
        token, position = 5, args.position
        for _ in range(args.warmup):
            token = model.forward_argmax([(0, token, position, 0)])[0]
            position += 1
        start = time.perf_counter()
        for _ in range(args.reps):
            token = model.forward_argmax([(0, token, position, 0)])[0]
            position += 1
        seconds = time.perf_counter() - start
    print(json.dumps({"mode": "decode", "layers": args.layers, "steps": args.reps, "first_position": args.position, "kv": "fp16" if args.kv_fp16 else "fp32",
                      "ms_per_step": seconds / args.reps * 1e3,
                      "weight_gbs": image.matrix_bytes * args.reps / seconds / 1e9, "last_token": token,
                      "device_faults": sb.library().device_faults()}))


if __name__ == "__main__":
    main()
