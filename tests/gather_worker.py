"""Worker of test_gather_multi_gpu.py, one process per GPU (launched by torch.distributed.run): every rank multiplies its
row shard of a small matrix with the gather entry point, storing into all ranks' copies of the output; afterwards every
copy must equal the product of the whole matrix computed locally."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import synapse_b200 as sb  # noqa: E402
from synapse_b200 import sharding, synth  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    lib = sb.library()
    failures = 0
    for ggml_type, rows, columns in ((sb.Q4_K, 512, 1024), (sb.Q8_0, 768, 896), (sb.Q6_K, 256, 2048)):
        weights = synth.matrix(ggml_type, rows, columns, seed=31)
        x = torch.from_numpy(synth.activations(1, columns, seed=32)).to(device)
        need = lib.activation_scratch_bytes(1, columns)
        scratch = torch.empty(need + 256, dtype=torch.uint8, device=device)
        scratch_ptr = (scratch.data_ptr() + 255) // 256 * 256
        sb.quantize_device(x.data_ptr(), 1, columns, columns, scratch_ptr, need, 0)
        peers = sharding.PeerOutputs({"y": rows}, device)
        dist.barrier()  # every rank has mapped every buffer
        first, count = sharding.shard_rows(rows, world, rank)
        offset, size = sharding.shard_bytes(ggml_type, rows, columns, world, rank)
        with sb.QuantizedMatrix(weights, ggml_type, rows, columns) as whole, \
                sb.QuantizedMatrix(weights[offset:offset + size], ggml_type, count, columns) as shard:
            want = torch.zeros(rows, device=device)
            whole.matmul_q8_device(scratch_ptr, 1, want.data_ptr(), rows)
            own, others = peers.pointers("y", first)
            words, arrivals = peers.signals("y")
            shard.matmul_q8_gather_device(scratch_ptr, 1, own, count, others, signal_ptrs=words, arrivals_ptr=arrivals)
            # no barrier: the wait returns when every rank's slice has landed in this GPU's copy (or after one second)
            sb.gather_wait_device(*peers.wait_arguments("y"), timeout_us=1_000_000)
            torch.cuda.synchronize()
            if not torch.equal(peers.view("y"), want):
                failures += 1
                print(f"rank {rank}: type {ggml_type} differs, max {float((peers.view('y') - want).abs().max())}", flush=True)
        dist.barrier()
        peers.close()
    total = torch.tensor([failures], device=device)
    dist.all_reduce(total)
    if rank == 0:
        print("GATHER_OK" if int(total.item()) == 0 and lib.device_faults() == 0 else "GATHER_FAILED", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
