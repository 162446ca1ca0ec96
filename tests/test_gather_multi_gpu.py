"""The gather that the product kernel performs itself, across real GPUs (needs at least two; skipped otherwise)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


def test_row_shards_store_into_every_gpus_copy():
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "gather_worker.py")
    command = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
               "--master-port", "29533", worker]
    result = subprocess.run(command, capture_output=True, text=True, timeout=240)
    assert "GATHER_OK" in result.stdout, result.stdout[-2000:] + result.stderr[-2000:]


def test_one_process_drives_two_devices(oracle):
    """A process that has run every kind of product on cuda:0 runs the same shapes on cuda:1 (kernel attributes such as
    the dynamic shared-memory limit are per device): one token, eight tokens, the tensor-core product, the decoder.
    Local loads only, no peer memory."""
    import numpy as np
    import torch

    import synapse_b200 as sb
    from synapse_b200 import decoder as dec
    from synapse_b200 import synth

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    results = []
    image = dec.ModelImage(layers=2, hidden=256, feed_forward=512, heads=4, kv_heads=2, vocabulary=512, context=16, matrix_types=dec.Q4KM_TYPES,
                           embedding_type=synth.Q4_K, output_type=synth.Q6_K, seed=3)
    for device in (0, 1):
        torch.cuda.set_device(device)
        per_device = []
        for ggml_type, rows, columns in ((sb.Q4_K, 2048, 3584), (sb.Q6_K, 512, 18944), (sb.Q8_0, 4864, 896)):
            weights = synth.matrix(ggml_type, rows, columns, seed=61)
            x = synth.activations(8, columns, seed=62)
            with sb.QuantizedMatrix(weights, ggml_type, rows, columns) as matrix:
                per_device.append(matrix.matvec(x[:1], sb.MODE_XQ8))
                per_device.append(matrix.matvec(x, sb.MODE_XQ8))
                per_device.append(matrix.matvec(x[:2], sb.MODE_XF32))
                if columns % 64 == 0:
                    per_device.append(matrix.gemm(x))
                    per_device.append(matrix.gemm(x, sb.GEMM_F16X2))
        with dec.Decoder(image) as model:
            per_device.append(model.decode(7, 0))
            per_device.append(model.decode(9, 1))
        results.append(per_device)
    torch.cuda.set_device(0)
    for a, b in zip(*results):
        assert a.tobytes() == b.tobytes()
    assert sb.library().device_faults() == 0
