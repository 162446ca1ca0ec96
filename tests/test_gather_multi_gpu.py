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
