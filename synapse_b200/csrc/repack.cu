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

}  // namespace syn
