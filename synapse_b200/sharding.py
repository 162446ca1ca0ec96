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


class _DeviceArray:
    """Lets torch wrap a raw device pointer (the CUDA array interface)."""

    def __init__(self, pointer: int, count: int):
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": "<f4", "data": (pointer, False), "version": 3}


class PeerOutputs:
    """One flat FP32 device buffer per rank, each mapped into every other rank's process (CUDA IPC, through
    ``syn_b200_shared_buffer_*``), for the gather that the product kernel performs itself
    (``syn_b200_matmul_q8_gather_dev``): a rank stores its slice of an output vector into its own buffer and into all
    peers' buffers at the same offset.

    ``layout`` maps a name to the length of that output vector; all ranks must pass the same layout. The ranks of the
    group must be GPUs of one box with peer access to each other; every rank must have its own GPU current. Raises
    ``BackendUnavailableError`` when a buffer cannot be created or mapped; because one rank may fail where another does
    not, the ranks must then agree (one all-reduce) before they rely on it, and synchronise once before the first
    product so that nobody stores into a buffer that is not mapped yet."""

    def __init__(self, layout: dict, device, group=None):
        import torch
        import torch.distributed as dist

        from . import BackendUnavailableError, library

        self.offsets, total = {}, 0
        for name, length in layout.items():
            self.offsets[name] = (total, int(length))
            total += (int(length) + 63) // 64 * 64  # 256-byte aligned vectors
        # Behind the vectors, 32 words (128 bytes) per vector: words 0..world-1 are this GPU's signal array of the vector
        # (rank r's products write word r, here and in every peer's buffer), words 16 and 17 the local arrival words of
        # this rank's products, word 24 the local sequence number of this rank's waits.
        self.control = {}
        for name in layout:
            self.control[name] = total
            total += 32
        total = max(total, 64)
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        torch.cuda.set_device(device)
        self._lib = library()
        self._own, self._opened, self.bases = 0, [], []
        # Collectives are reached by every rank whatever fails locally, and a failure anywhere fails all ranks alike:
        # a rank that left early would leave the others waiting in the exchange.
        handle, problem = None, None
        try:
            self._own, handle = self._lib.shared_buffer_create(4 * total)
        except Exception as error:  # reported after the exchange
            problem = error
        handles = [None] * self.world
        dist.all_gather_object(handles, handle, group=group)
        if any(h is None for h in handles):
            self.close()
            raise BackendUnavailableError(f"a rank could not create its shared output buffer ({problem or 'another rank'})")
        for r in range(self.world):
            if r == self.rank:
                self.bases.append(self._own)
                continue
            try:
                mapped = self._lib.shared_buffer_open(handles[r])
            except Exception as error:
                problem = problem or error
                mapped = 0
            if mapped:
                self._opened.append(mapped)
            self.bases.append(mapped)
        if problem is not None:
            # no collective follows in here: the caller agrees with the other ranks on whether everyone got this far
            self.close()
            raise BackendUnavailableError(f"a peer's output buffer could not be mapped ({problem})")
        self.local = torch.as_tensor(_DeviceArray(self._own, total), device=device)

    def close(self):
        for mapped in self._opened:
            self._lib.shared_buffer_close(mapped)
        self._opened = []
        if self._own:
            self._lib.shared_buffer_destroy(self._own)
            self._own = 0

    def view(self, name):
        """This rank's copy of the full output vector ``name``."""
        offset, length = self.offsets[name]
        return self.local[offset:offset + length]

    def signals(self, name):
        """(signal word pointers, arrivals pointer) for this rank's products into vector ``name``: this rank's word of the
        vector's signal array in its own buffer first, then the same word in every peer's buffer."""
        at = 4 * (self.control[name] + self.rank)
        words = [self.bases[self.rank] + at] + [self.bases[r] + at for r in range(self.world) if r != self.rank]
        return words, self.bases[self.rank] + 4 * (self.control[name] + 16)

    def wait_arguments(self, name):
        """(signal array pointer, word count, sequence word pointer) for ``gather_wait_device`` on vector ``name``."""
        base = self.bases[self.rank] + 4 * self.control[name]
        return base, self.world, base + 4 * 24

    def pointers(self, name, first_row: int):
        """(own pointer, [peer pointers]) of element ``first_row`` of vector ``name``."""
        offset, _ = self.offsets[name]
        at = 4 * (offset + first_row)
        return self.bases[self.rank] + at, [self.bases[r] + at for r in range(self.world) if r != self.rank]
