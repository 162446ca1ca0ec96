"""Row sharding and the output gather, on two gloo ranks (no GPU): the gathered result equals the unsharded one bitwise."""
import os
import socket
import sys

import numpy as np
import pytest

from synapse_b200 import sharding, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_arithmetic():
    assert sharding.shard_rows(28672, 8, 3) == (3 * 3584, 3584)
    assert sharding.shard_rows(152064, 8, 7) == (7 * 19008, 19008)
    assert sharding.shard_bytes(synth.Q4_K, 8192, 28672, 4, 1) == (2048 * 16128, 2048 * 16128)
    with pytest.raises(ValueError):
        sharding.shard_rows(10, 4, 0)
    with pytest.raises(ValueError):
        sharding.shard_rows(8, 2, 2)
    covered = [sharding.shard_rows(3584, 4, r) for r in range(4)]
    assert covered[0][0] == 0 and all(a[0] + a[1] == b[0] for a, b in zip(covered, covered[1:])) and sum(c for _, c in covered) == 3584


def _worker(rank, world, port, tokens, out_path):
    import torch
    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    import oracle

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rows, columns = 64, 512
        weights = synth.matrix(synth.Q4_K, rows, columns, seed=81)
        x = synth.activations(tokens, columns, seed=82)
        codes, scales = oracle.quantize(x)
        offset, count = sharding.shard_bytes(synth.Q4_K, rows, columns, world, rank)
        first, shard = sharding.shard_rows(rows, world, rank)
        local = oracle.kq_q8_matmul(synth.Q4_K, weights[offset:offset + count], shard, columns, codes, scales)
        full = torch.zeros(tokens, rows) if tokens > 1 else torch.zeros(rows)
        sharding.gather_outputs(torch.from_numpy(local if tokens > 1 else local[0]), full)
        if rank == 0:
            want = oracle.kq_q8_matmul(synth.Q4_K, weights, rows, columns, codes, scales)
            got = full.numpy().reshape(tokens, rows)
            np.save(out_path, np.array([float(got.tobytes() == want.tobytes())]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("tokens", [1, 3])
def test_gathered_slices_equal_the_unsharded_product(tmp_path, tokens):
    import torch.multiprocessing as mp

    import oracle

    oracle.build()
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    out_path = str(tmp_path / "result.npy")
    mp.spawn(_worker, args=(2, port, tokens, out_path), nprocs=2, join=True)
    assert np.load(out_path)[0] == 1.0
