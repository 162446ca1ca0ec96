"""Row sharding of a quantised matrix across the GPUs of one box, and the gather of the output slices.

Every output row is an independent dot product (the reference already partitions rows across CPU threads with no
cross-chunk communication, src/Synapse.Runtime/Features/CpuKernels/ChunkedRowWork.cs:25-38), and a row-major block
layout makes a row range a contiguous byte range, so sharding needs no re-encoding: rank g of G holds rows
[g*R/G, (g+1)*R/G). Activations are replicated; the one exchange step is an all-gather of the FP32 output slices.
"""
from __future__ import annotations

from . import synth


def shard_rows(rows: int, world: int, rank: int) -> tuple[int, int]:
    """(first row, row count) of ``rank``'s shard. Rows must split evenly so that every gathered slice has one size."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} is outside a world of {world}")
    if rows % world:
        raise ValueError(f"{rows} rows do not split evenly over {world} ranks")
    count = rows // world
    return rank * count, count


def shard_bytes(ggml_type: int, rows: int, columns: int, world: int, rank: int) -> tuple[int, int]:
    """(byte offset, byte count) of the shard inside the row-major block array."""
    first, count = shard_rows(rows, world, rank)
    row_bytes = synth.row_bytes(ggml_type, columns)
    return first * row_bytes, count * row_bytes


def gather_outputs(local, full, group=None):
    """All-gathers per-rank output slices into the full output.

    ``local`` is this rank's [tokens, rows/G] (or [rows/G]) tensor, ``full`` the [tokens, rows] (or [rows]) result on
    every rank. One token: the slices are concatenated in place. Several tokens: slices are gathered rank-major and
    then laid out token-major."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    if local.dim() == 1 or local.shape[0] == 1:
        dist.all_gather_into_tensor(full.view(-1), local.contiguous().view(-1), group=group)
        return full
    tokens, count = local.shape
    staged = torch.empty((world, tokens, count), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(staged.view(-1), local.contiguous().view(-1), group=group)
    full.copy_(staged.permute(1, 0, 2).reshape(tokens, world * count))
    return full
