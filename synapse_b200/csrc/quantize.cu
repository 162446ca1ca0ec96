// Q8_0 activation quantiser on the device. Reproduces Q8ActivationQuantizer.QuantizeBlock
// (src/Synapse.Runtime/Features/CpuKernels/Q8ActivationQuantizer.cs:34-57) bit for bit: per 32 values
// scale = max|x| / 127 (IEEE division), inverse = scale == 0 ? 0 : 1 / scale, code = round-half-even(x * inverse)
// with the UNROUNDED scale, stored scale = the scale rounded through fp16. Also emits the sum of the codes of
// every 16 values, which the K-quant kernels need for their offset terms.
#include "common.cuh"

namespace syn {

namespace {

constexpr int kWarpsPerCta = 8;

int current_sm_count()
{
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) {
        cudaGetLastError();
    }
    return sm_count(device);
}

// One warp per 32-value block, one lane per value.
__global__ void __launch_bounds__(kWarpsPerCta * 32)
quantize_q8_kernel(const float *__restrict__ x, uint64_t blocks_per_row, uint64_t total_blocks, uint64_t in_stride,
                   int8_t *__restrict__ codes, float *__restrict__ scales, int16_t *__restrict__ sums)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t lane = threadIdx.x & 31;
    uint64_t block = (uint64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
    const uint64_t stride = (uint64_t)gridDim.x * kWarpsPerCta;
    for (; block < total_blocks; block += stride) {
        const uint64_t token = block / blocks_per_row;
        const uint64_t in_row = block - token * blocks_per_row;
        const float value = x[token * in_stride + in_row * 32 + lane];
        float amax = fabsf(value);
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, offset));
        }
        const float scale = __fdiv_rn(amax, 127.0f);
        const float inverse = scale == 0.0f ? 0.0f : __fdiv_rn(1.0f, scale);
        const int code = __float2int_rn(__fmul_rn(value, inverse));
        codes[block * 32 + lane] = (int8_t)code;
        int sum = code;
#pragma unroll
        for (int offset = 8; offset > 0; offset >>= 1) {
            sum += __shfl_xor_sync(0xffffffffu, sum, offset);
        }
        if ((lane & 15) == 0) {
            sums[block * 2 + (lane >> 4)] = (int16_t)sum;
        }
        if (lane == 0) {
            scales[block] = __half2float(__float2half_rn(scale));
        }
    }
}

// Sums of 16 codes for activations that arrive already quantised.
__global__ void group_sums_kernel(const int8_t *__restrict__ codes, uint64_t count16, int16_t *__restrict__ sums)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    uint64_t g = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (; g < count16; g += stride) {
        const int4 v = reinterpret_cast<const int4 *>(codes)[g];
        int s = __dp4a(v.x, 0x01010101, 0);
        s = __dp4a(v.y, 0x01010101, s);
        s = __dp4a(v.z, 0x01010101, s);
        s = __dp4a(v.w, 0x01010101, s);
        sums[g] = (int16_t)s;
    }
}

// One warp; lane i watches word i of the signal array. Every wait is bounded by the nanosecond timer.
__global__ void gather_wait_kernel(const uint32_t *signals, uint32_t count, uint32_t *epoch, uint64_t timeout_ns, uint32_t *fault)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t lane = threadIdx.x;
    const uint32_t expected = *epoch + 1;
    __syncwarp();
    bool reached = true;
    if (lane < count) {
        uint64_t start;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(start));
        reached = false;
        while (true) {
            uint32_t value;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(value) : "l"(signals + lane) : "memory");
            if ((int32_t)(value - expected) >= 0) {
                reached = true;
                break;
            }
            uint64_t now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (now - start > timeout_ns) {
                break;
            }
        }
    }
    const bool all = __all_sync(0xffffffffu, reached);
    if (lane == 0) {
        *epoch = expected;
        if (!all && fault) {
            atomicAdd(fault, 1u);
        }
    }
}

}  // namespace

cudaError_t launch_gather_wait(const uint32_t *signals, uint32_t count, uint32_t *epoch, uint32_t timeout_us, cudaStream_t stream)
{
    return launch_kernel(gather_wait_kernel, dim3(1), dim3(32), 0, stream, signals, count, epoch, (uint64_t)timeout_us * 1000ull, fault_word_device());
}

cudaError_t launch_quantize(const float *x, uint64_t tokens, uint64_t columns, uint64_t in_stride, int8_t *codes,
                            float *scales, int16_t *sums, cudaStream_t stream)
{
    const uint64_t blocks_per_row = columns / 32;
    const uint64_t total = tokens * blocks_per_row;
    uint64_t grid = (total + kWarpsPerCta - 1) / kWarpsPerCta;
    const uint64_t cap = (uint64_t)current_sm_count() * 8;
    if (grid > cap) {
        grid = cap;
    }
    return launch_kernel(quantize_q8_kernel, dim3((unsigned)grid), dim3(kWarpsPerCta * 32), 0, stream, x, blocks_per_row, total, in_stride,
                         codes, scales, sums);
}

cudaError_t launch_group_sums(const int8_t *codes, uint64_t count16, int16_t *sums, cudaStream_t stream)
{
    uint64_t grid = (count16 + 255) / 256;
    const uint64_t cap = (uint64_t)current_sm_count() * 8;
    if (grid > cap) {
        grid = cap;
    }
    return launch_kernel(group_sums_kernel, dim3((unsigned)grid), dim3(256), 0, stream, codes, count16, sums);
}

}  // namespace syn
