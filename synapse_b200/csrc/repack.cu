// Load-time repack of GGUF blocks into planar layouts whose fields can be read with aligned 128-bit loads.
// The byte count does not grow: every source byte lands in exactly one plane.
//   Q8_0 (34 B blocks, 2-byte aligned in the file): codes int8 [rows][K] | scales half [rows][K/32]
//   Q6_K (210 B blocks, 2-byte aligned):            ql [rows][K/2] | qh [rows][K/4] | scales int8 [rows][K/16] | d half [rows][K/256]
//   Q4_K (144 B blocks) is 16-byte aligned already and stays in its file layout.
// Block layouts: native/synapse-gpu/src/Features/GpuKernels/cuda/kernels/common.cuh:13-16 (Q8_0),
// src/Synapse.Runtime/Features/ModelPackages/SourceFormats/GgufKQuantBlocks.cs:155-177 (Q6_K).
#include "common.cuh"

namespace syn {

uint64_t planar_bytes(uint32_t type, uint64_t rows, uint64_t columns, PlaneOffsets *planes)
{
    PlaneOffsets p;
    uint64_t total = 0;
    if (type == kQ8_0) {
        p.p0 = 0;
        p.p1 = align_up(rows * columns, 256);
        total = p.p1 + rows * (columns / 32) * 2;
    } else if (type == kQ6_K) {
        p.p0 = 0;
        p.p1 = align_up(rows * columns / 2, 256);
        p.p2 = align_up(p.p1 + rows * columns / 4, 256);
        p.p3 = align_up(p.p2 + rows * columns / 16, 256);
        total = p.p3 + rows * (columns / 256) * 2;
    }
    if (planes) {
        *planes = p;
    }
    return align_up(total, 256);
}

namespace {

__global__ void repack_q8_0_kernel(const uint8_t *__restrict__ natural, uint64_t blocks, int8_t *__restrict__ codes,
                                   uint16_t *__restrict__ scales)
{
    // One thread per 16-bit word of a block: word 0 is the scale, words 1..16 are code pairs.
    uint64_t index = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    const uint16_t *words = reinterpret_cast<const uint16_t *>(natural);
    for (; index < blocks * 17; index += stride) {
        const uint64_t block = index / 17;
        const uint32_t word = (uint32_t)(index - block * 17);
        const uint16_t value = words[index];
        if (word == 0) {
            scales[block] = value;
        } else {
            reinterpret_cast<uint16_t *>(codes)[block * 16 + (word - 1)] = value;
        }
    }
}

__global__ void repack_q6_k_kernel(const uint8_t *__restrict__ natural, uint64_t blocks, uint16_t *__restrict__ ql,
                                   uint16_t *__restrict__ qh, uint16_t *__restrict__ sc, uint16_t *__restrict__ d)
{
    // One thread per 16-bit word of a 210-byte block (105 words): 64 ql, 32 qh, 8 scales, 1 d.
    uint64_t index = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    const uint16_t *words = reinterpret_cast<const uint16_t *>(natural);
    for (; index < blocks * 105; index += stride) {
        const uint64_t block = index / 105;
        const uint32_t word = (uint32_t)(index - block * 105);
        const uint16_t value = words[index];
        if (word < 64) {
            ql[block * 64 + word] = value;
        } else if (word < 96) {
            qh[block * 32 + (word - 64)] = value;
        } else if (word < 104) {
            sc[block * 8 + (word - 96)] = value;
        } else {
            d[block] = value;
        }
    }
}

}  // namespace

cudaError_t launch_repack(uint32_t type, const uint8_t *natural, uint64_t rows, uint64_t columns, uint8_t *planar,
                          const PlaneOffsets &planes, cudaStream_t stream)
{
    const uint64_t blocks = rows * (columns / block_values(type));
    const uint64_t words = blocks * (type == kQ8_0 ? 17 : 105);
    uint64_t grid = (words + 255) / 256;
    if (grid > 148 * 16) {
        grid = 148 * 16;
    }
    if (type == kQ8_0) {
        repack_q8_0_kernel<<<(unsigned)grid, 256, 0, stream>>>(natural, blocks, reinterpret_cast<int8_t *>(planar + planes.p0),
                                                             reinterpret_cast<uint16_t *>(planar + planes.p1));
    } else if (type == kQ6_K) {
        repack_q6_k_kernel<<<(unsigned)grid, 256, 0, stream>>>(
            natural, blocks, reinterpret_cast<uint16_t *>(planar + planes.p0), reinterpret_cast<uint16_t *>(planar + planes.p1),
            reinterpret_cast<uint16_t *>(planar + planes.p2), reinterpret_cast<uint16_t *>(planar + planes.p3));
    } else {
        return cudaErrorInvalidValue;
    }
    count_launch();
    return cudaGetLastError();
}


// ---- block validation at load (BlockSourceDecoder.Decode, ModelPackages/SourceFormats/SourceTensorDecoders.cs:134-146,
// 161-172): every fp16 field of every block must be finite. Offsets of the fp16 fields inside a block: Q8_0 d at 0;
// Q4_K d at 0 and dmin at 2; Q6_K d at 208. -----------------------------------------------------------------

namespace {

__host__ __device__ inline bool half_bits_finite(uint32_t bits) { return (bits & 0x7C00u) != 0x7C00u; }
__host__ __device__ inline bool block_scales_finite(uint32_t type, const uint8_t *block)
{
    if (type == kQ6_K) {
        return half_bits_finite(block[208] | (block[209] << 8));
    }
    const bool d = half_bits_finite(block[0] | (block[1] << 8));
    return type == kQ4_K ? d && half_bits_finite(block[2] | (block[3] << 8)) : d;
}

__global__ void validate_blocks_kernel(const uint8_t *__restrict__ data, uint32_t type, uint32_t block_bytes, uint64_t blocks,
                                       unsigned long long *__restrict__ first_bad)
{
    uint64_t block = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (; block < blocks; block += stride) {
        if (!block_scales_finite(type, data + block * block_bytes)) {
            atomicMin(first_bad, (unsigned long long)block);
        }
    }
}

}  // namespace

uint64_t first_invalid_block_host(uint32_t type, const uint8_t *data, uint64_t blocks)
{
    const uint64_t bytes = block_bytes(type);
    for (uint64_t block = 0; block < blocks; ++block) {
        if (!block_scales_finite(type, data + block * bytes)) {
            return block;
        }
    }
    return UINT64_MAX;
}

cudaError_t launch_validate_blocks(uint32_t type, const uint8_t *data, uint64_t blocks, uint64_t *first_bad_device, cudaStream_t stream)
{
    cudaError_t error = cudaMemsetAsync(first_bad_device, 0xFF, sizeof(uint64_t), stream);
    if (error != cudaSuccess) {
        return error;
    }
    uint64_t grid = (blocks + 255) / 256;
    int device = 0;
    cudaGetDevice(&device);
    const uint64_t cap = (uint64_t)sm_count(device) * 8;
    if (grid > cap) {
        grid = cap;
    }
    validate_blocks_kernel<<<(unsigned)grid, 256, 0, stream>>>(data, type, (uint32_t)block_bytes(type), blocks,
                                                              reinterpret_cast<unsigned long long *>(first_bad_device));
    count_launch();
    return cudaGetLastError();
}

}  // namespace syn
