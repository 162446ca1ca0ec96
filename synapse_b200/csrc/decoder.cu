// The decode step around the matrix products: a whole-decoder create / forward / destroy behind the same structs as
// the reference's GPU ABI (DecoderDesc, DecoderLayerOffsets, BatchToken: native/synapse-gpu/src/Features/GpuKernels/
// decoder.rs:61-141, ffi.rs:113-271), with the numeric contract of the reference's optimized CPU executor
// (Qwen2/Qwen2CpuExecutor.cs:105-244): every projection multiplies Q8_0-quantised activations.
//
// One step = embedding rows, then per layer {RMSNorm + quantise, Q/K/V with bias, NeoX RoPE + KV append, softmax
// attention over the slot's cache, quantise, output projection + residual, RMSNorm + quantise, gate, up with the
// SwiGLU epilogue, quantise, down + residual}, output norm + quantise, vocabulary projection. Token, position and
// slot are read by the kernels from a small device array, so the launch sequence of a step does not depend on
// them: it is captured once per token count into a CUDA graph and replayed.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <type_traits>
#include <vector>

#include "common.cuh"
#include "decode_program.cuh"

namespace syn {

namespace {

constexpr uint64_t kNoTensor = 0xFFFFFFFFFFFFFFFFull;
// Tokens of one step: decode tokens of several sessions and prompt runs (the reference's prefill chunks hold up to 64
// tokens, src/Synapse.Runtime/Features/ModelLoading/ModelLoadOptions.cs:57). Steps of up to kMaxGraphTokens tokens are
// captured into a CUDA graph per token count.
constexpr uint32_t kMaxStepTokens = 64;
constexpr uint32_t kMaxGraphTokens = 8;

using prog::BatchToken;
using prog::decode_element;

// ---- small kernels ------------------------------------------------------------------------------------

// hidden[t] = embedding row of tokens[t].token (Qwen2CpuExecutor.cs:110-117).
__global__ void embed_kernel(const BatchToken *__restrict__ tokens, const uint8_t *__restrict__ table, uint32_t type, uint64_t row_bytes,
                             uint32_t hidden, float *__restrict__ out)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint8_t *row = table + (uint64_t)tokens[blockIdx.y].token * row_bytes;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < hidden; i += gridDim.x * blockDim.x) {
        out[(uint64_t)blockIdx.y * hidden + i] = decode_element(type, row, i);
    }
}

// RMSNorm with an FP64 sum of squares (Q8Operators.cs:101-123) fused with the Q8_0 activation quantiser
// (Q8ActivationQuantizer.cs:34-57), one CTA of 32 warps per token. Every value is loaded once and stays in registers: a
// lane takes four consecutive values, eight lanes one 32-value block, a warp one 128-value piece per round (rows of up
// to 32768 values take eight rounds). The sum of squares is formed per piece and the pieces are added in index order,
// the order every normalising kernel of the library uses, so all of them produce the same bits. With `by_logits_row` the
// token's activations go to row tokens[t].logits_row and tokens without a logits row are skipped
// (Qwen2CpuExecutor.cs:202-222).
constexpr int kNormWarps = 32, kNormRounds = 8;
__global__ void __launch_bounds__(kNormWarps * 32)
rmsnorm_quantize_kernel(const BatchToken *__restrict__ tokens, const float *__restrict__ x, const float *__restrict__ weight, float epsilon,
                        uint32_t n, uint32_t rows, uint32_t by_logits_row, int8_t *__restrict__ codes, float *__restrict__ scales,
                        int16_t *__restrict__ sums)
{
    __shared__ double quad_sums[kNormWarps * kNormRounds];  // rows of up to 32768 values
    __shared__ float shared_scale;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int target = (int)t;
    if (by_logits_row) {
        target = tokens[t].logits_row;
        if (target < 0 || (uint32_t)target >= rows) {
            return;
        }
    }
    const float *row = x + (uint64_t)t * n;
    const uint32_t quads = (n + 127) / 128;
    float4 v[kNormRounds];
#pragma unroll
    for (int i = 0; i < kNormRounds; ++i) {
        const uint32_t first = (warp + i * kNormWarps) * 128 + lane * 4;
        v[i] = first < n ? *reinterpret_cast<const float4 *>(row + first) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
#pragma unroll
    for (int i = 0; i < kNormRounds; ++i) {
        const uint32_t quad = warp + i * kNormWarps;
        if (quad < quads) {  // the same for the whole warp
            const double s = prog::quad_square_sum(v[i]);
            if (lane == 0) {
                quad_sums[quad] = s;
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        shared_scale = prog::norm_scale_from(quad_sums, quads, n, epsilon);
    }
    __syncthreads();
    const float scale = shared_scale;
    const uint32_t blocks = n / 32;
#pragma unroll
    for (int i = 0; i < kNormRounds; ++i) {
        const uint32_t first = (warp + i * kNormWarps) * 128 + lane * 4;
        if (warp + i * kNormWarps >= quads) {
            break;  // the same for the whole warp
        }
        const float4 w = first < n ? __ldg(reinterpret_cast<const float4 *>(weight + first)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        const float a = __fmul_rn(__fmul_rn(v[i].x, scale), w.x), b = __fmul_rn(__fmul_rn(v[i].y, scale), w.y);
        const float c = __fmul_rn(__fmul_rn(v[i].z, scale), w.z), e = __fmul_rn(__fmul_rn(v[i].w, scale), w.w);
        float amax = fmaxf(fmaxf(fabsf(a), fabsf(b)), fmaxf(fabsf(c), fabsf(e)));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
        const float d = __fdiv_rn(amax, 127.0f);
        const float inverse = d == 0.0f ? 0.0f : __fdiv_rn(1.0f, d);
        const int c0 = __float2int_rn(__fmul_rn(a, inverse)), c1 = __float2int_rn(__fmul_rn(b, inverse));
        const int c2 = __float2int_rn(__fmul_rn(c, inverse)), c3 = __float2int_rn(__fmul_rn(e, inverse));
        int group = (c0 + c1) + (c2 + c3);
        group += __shfl_xor_sync(0xffffffffu, group, 1);
        group += __shfl_xor_sync(0xffffffffu, group, 2);
        if (first < n) {
            const uint32_t packed = (uint32_t)(c0 & 0xff) | ((uint32_t)(c1 & 0xff) << 8) | ((uint32_t)(c2 & 0xff) << 16) | ((uint32_t)c3 << 24);
            *reinterpret_cast<uint32_t *>(codes + (uint64_t)target * n + first) = packed;
            if ((lane & 3) == 0) {
                sums[(uint64_t)target * (n / 16) + first / 16] = (int16_t)group;
            }
            if ((lane & 7) == 0) {
                scales[(uint64_t)target * blocks + first / 32] = __half2float(__float2half_rn(d));
            }
        }
    }
}

// NeoX rotation of every query and key head (first half against second half, Qwen2CpuState.cs:85-105) and the
// append of the rotated key and the value to the slot's cache. Grid (heads + kv_heads, tokens), head_dim/2 threads.
// What a value becomes in the cache: itself, or the nearest fp16 number (KvPrecision::F16,
// native/synapse-gpu/src/Features/GpuKernels/decoder.rs:43-58).
__device__ __forceinline__ void cache_store(float *p, float v) { *p = v; }
__device__ __forceinline__ void cache_store(__half *p, float v) { *p = __float2half_rn(v); }
__device__ __forceinline__ float cache_rounded(const float *, float v) { return v; }
__device__ __forceinline__ float cache_rounded(const __half *, float v) { return __half2float(__float2half_rn(v)); }

template <class KV>
__global__ void rope_store_kernel(const BatchToken *__restrict__ tokens, float *__restrict__ q, float *__restrict__ k,
                                  const float *__restrict__ v, const float *__restrict__ cosines, const float *__restrict__ sines,
                                  KV *__restrict__ keys, KV *__restrict__ values, uint32_t heads, uint32_t kv_heads, uint32_t head_dim,
                                  uint32_t layer, uint32_t layers, uint32_t context)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t t = blockIdx.y, head = blockIdx.x, half = head_dim / 2, i = threadIdx.x;
    const BatchToken token = tokens[t];
    const float c = cosines[(uint64_t)token.position * half + i], s = sines[(uint64_t)token.position * half + i];
    float *x = head < heads ? q + ((uint64_t)t * heads + head) * head_dim : k + ((uint64_t)t * kv_heads + (head - heads)) * head_dim;
    const float a = x[i], b = x[i + half];
    const float first = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s)), second = __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c));
    x[i] = first;
    x[i + half] = second;
    if (head >= heads) {
        const uint32_t kh = head - heads;
        const uint64_t at = ((((uint64_t)token.slot * layers + layer) * kv_heads + kh) * context + token.position) * head_dim;
        cache_store(keys + at + i, first);
        cache_store(keys + at + i + half, second);
        const float *vs = v + ((uint64_t)t * kv_heads + kh) * head_dim;
        cache_store(values + at + i, vs[i]);
        cache_store(values + at + i + half, vs[i + half]);
    }
}

// Softmax attention of one token's query head over positions 0..position of its slot (Qwen2CpuAttention.cs:82-173).
// Grid (heads, tokens), kAttentionWarps warps; each warp walks every kAttentionWarps-th position with an online softmax, the partial
// results are merged in shared memory. Head dimensions up to 256.
// ROTATE (single-token steps): the kernel also does the work of rope_store_kernel for its head -- it rotates its query
// head and the key head it reads, the first query head of every key head appends key and value to the cache -- and
// attends to the current position out of shared memory. Same arithmetic, one launch less per layer. Steps with several
// tokens keep the separate rotation kernel: a prompt run's later tokens read the cache entries of its earlier ones.
// KV: the cache's element type. With fp16 the current position is attended to with the values the cache holds for it
// (rounded), as every later step will see them.
// Caches of 1024 positions and more: gridDim.z CTAs share a head's positions (CTA z takes the streams z * 48 .. z * 48 + 47
// of 48 * gridDim.z); each leaves its unnormalised sum, maximum and weight sum in `split_partial`, and the CTA that counts
// itself in last (an arrival counter per token and head, reset for the next launch; no CTA waits for another) adds them
// in split order and quantises. One CTA per head otherwise (split_partial null).
// E4: 16-byte pieces of FP32 per lane the walk is built for (1, 2, 4, 8 for heads of up to 32, 64, 128, 256 values);
// SPLIT: whether several CTAs share a head. Both are template parameters so that a kernel holds one walk and nothing it
// does not use: these CTAs live for a few microseconds, and a kernel that carried all four walks and the split code
// spent a measurable part of that fetching instructions (1.5 us per layer at short contexts).
// Two of these CTAs must fit an SM's registers (heads of up to 128 values): the kernel is launched as a programmatic
// dependent of the q | k | v products, and only a CTA that fits beside theirs starts early; at 156 registers per thread
// it did not, which cost a decode step 1.5 us per layer.
template <bool ROTATE, class KV, int E4, bool SPLIT>
__global__ void __launch_bounds__(32 * prog::kAttentionWarps, E4 <= 4 ? 2 : 1)
attention_kernel(const BatchToken *__restrict__ tokens, const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                 const float *__restrict__ cosines, const float *__restrict__ sines, KV *__restrict__ keys, KV *__restrict__ values,
                 uint32_t heads, uint32_t kv_heads, uint32_t head_dim, uint32_t layer, uint32_t layers, uint32_t context, float scale,
                 int8_t *__restrict__ codes, float *__restrict__ scales, int16_t *__restrict__ sums, float *__restrict__ split_partial,
                 uint32_t *__restrict__ split_arrivals)
{
    __shared__ __align__(16) float merged[prog::kAttentionWarps][256 + 4];  // a warp's unnormalised sum, [256] its maximum, [257] its weight sum
    __shared__ bool last_split;
    __shared__ __align__(16) float rotated_query[ROTATE ? 256 : 4], current_key[ROTATE ? 256 : 4], current_value[ROTATE ? 256 : 4];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t t = blockIdx.y, head = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const BatchToken token = tokens[t];
    const uint32_t group = heads / kv_heads, kh = head / group, half = head_dim / 2;
    const float *query = q + ((uint64_t)t * heads + head) * head_dim;
    const uint64_t base = (((uint64_t)token.slot * layers + layer) * kv_heads + kh) * context * head_dim;
    if (ROTATE) {
        if (threadIdx.x < half) {
            const uint32_t i = threadIdx.x;
            const float c = cosines[(uint64_t)token.position * half + i], s = sines[(uint64_t)token.position * half + i];
            {
                const float a = query[i], b = query[i + half];
                rotated_query[i] = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
                rotated_query[i + half] = __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c));
            }
            const float *x = k + ((uint64_t)t * kv_heads + kh) * head_dim;
            const float a = x[i], b = x[i + half];
            const float first = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s)), second = __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c));
            const float *vs = v + ((uint64_t)t * kv_heads + kh) * head_dim;
            const float v0 = vs[i], v1 = vs[i + half];
            current_key[i] = cache_rounded(keys, first);
            current_key[i + half] = cache_rounded(keys, second);
            current_value[i] = cache_rounded(values, v0);
            current_value[i + half] = cache_rounded(values, v1);
            if (head % group == 0 && (!SPLIT || blockIdx.z == 0)) {
                const uint64_t at = base + (uint64_t)token.position * head_dim;
                cache_store(keys + at + i, first);
                cache_store(keys + at + i + half, second);
                cache_store(values + at + i, v0);
                cache_store(values + at + i + half, v1);
            }
        }
        __syncthreads();
        query = rotated_query;
    }
    constexpr int kStreams = 4 * prog::kAttentionWarps, kBatch = E4 == 1 ? 4 : E4 == 2 ? 2 : 1;  // 32 registers of keys and of values in flight
    prog::attend_streams<KV, E4, kBatch>(query, lane, warp, token.position, head_dim, scale, (const KV *)keys + base, (const KV *)values + base,
                                         ROTATE ? current_key : nullptr, ROTATE ? current_value : nullptr, merged[warp],
                                         SPLIT ? (int)blockIdx.z * kStreams : 0, SPLIT ? (int)gridDim.z * kStreams : kStreams);
    __syncthreads();
    float total_max = -INFINITY;
    for (int w = 0; w < prog::kAttentionWarps; ++w) {
        total_max = fmaxf(total_max, merged[w][256]);
    }
    float total_sum = 0.0f;
    for (int w = 0; w < prog::kAttentionWarps; ++w) {
        // an idle warp has sum 0 and max -inf: exp(-inf) = 0 (a CTA of a split that has no position at all: every warp is idle)
        total_sum += merged[w][256] == -INFINITY ? 0.0f : merged[w][257] * expf(merged[w][256] - total_max);
    }
    if constexpr (SPLIT) {
        // this CTA's share: element i unnormalised, then maximum and weight sum
        const uint32_t splits = gridDim.z, width = head_dim + 4;
        float *const mine = split_partial + (((uint64_t)t * heads + head) * splits + blockIdx.z) * width;
        if (threadIdx.x < head_dim) {
            float value = 0.0f;
            for (int w = 0; w < prog::kAttentionWarps; ++w) {
                value += merged[w][256] == -INFINITY ? 0.0f : merged[w][threadIdx.x] * expf(merged[w][256] - total_max);
            }
            mine[threadIdx.x] = value;
        }
        if (threadIdx.x == 0) {
            mine[head_dim] = total_max;
            mine[head_dim + 1] = total_sum;
        }
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            const uint32_t before = atomicAdd(split_arrivals + (uint64_t)t * heads + head, 1u);
            last_split = before + 1 == splits;
            if (last_split) {
                split_arrivals[(uint64_t)t * heads + head] = 0;  // for the next launch
            }
        }
        __syncthreads();
        if (!last_split) {
            return;
        }
        __threadfence();
        // The last CTA in: the splits' shares in split order, into merged[0] as one "warp" so that the code below serves both forms.
        const float *const shares = split_partial + ((uint64_t)t * heads + head) * splits * width;
        float joint = -INFINITY;
        for (uint32_t z = 0; z < splits; ++z) {
            joint = fmaxf(joint, __ldcg(shares + z * width + head_dim));
        }
        float sum = 0.0f;
        for (uint32_t z = 0; z < splits; ++z) {
            const float m = __ldcg(shares + z * width + head_dim);
            sum += m == -INFINITY ? 0.0f : __ldcg(shares + z * width + head_dim + 1) * expf(m - joint);
        }
        if (threadIdx.x < head_dim) {
            float value = 0.0f;
            for (uint32_t z = 0; z < splits; ++z) {
                const float m = __ldcg(shares + z * width + head_dim);
                value += m == -INFINITY ? 0.0f : __ldcg(shares + z * width + threadIdx.x) * expf(m - joint);
            }
            merged[0][threadIdx.x] = value;
        }
        __syncthreads();
        total_max = joint;
        total_sum = sum;
    }
    constexpr bool joined = SPLIT;  // merged[0] already holds the head's unnormalised sum
    // The head's output is head_dim/32 whole Q8_0 blocks of the attention row: quantise them here (one warp per
    // block, same arithmetic as the activation quantiser) instead of storing FP32 and launching the quantiser.
    const uint32_t hidden = heads * head_dim;
    for (uint32_t block = warp; block < head_dim / 32; block += prog::kAttentionWarps) {
        const uint32_t i = block * 32 + lane;
        float value = 0.0f;
        if (joined) {
            value = merged[0][i];
        } else {
            for (int w = 0; w < prog::kAttentionWarps; ++w) {
                value += merged[w][256] == -INFINITY ? 0.0f : merged[w][i] * expf(merged[w][256] - total_max);  // (an idle warp leaves its row unwritten)
            }
        }
        value = value / total_sum;
        float amax = fabsf(value);
        for (int offset = 16; offset > 0; offset >>= 1) {
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, offset));
        }
        const float d = __fdiv_rn(amax, 127.0f);
        const float inverse = d == 0.0f ? 0.0f : __fdiv_rn(1.0f, d);
        const int code = __float2int_rn(__fmul_rn(value, inverse));
        const uint64_t column = (uint64_t)head * head_dim + i;
        codes[(uint64_t)t * hidden + column] = (int8_t)code;
        int group = code;
        for (int offset = 8; offset > 0; offset >>= 1) {
            group += __shfl_xor_sync(0xffffffffu, group, offset);
        }
        if ((lane & 15) == 0) {
            sums[(uint64_t)t * (hidden / 16) + column / 16] = (int16_t)group;
        }
        if (lane == 0) {
            scales[(uint64_t)t * (hidden / 32) + column / 32] = __half2float(__float2half_rn(d));
        }
    }
}

// First maximum of each logits row (Q8Operators.cs:152-173): larger value wins, equal values keep the lower index.
// Grid (kArgmaxSlices, logits rows): every CTA reduces one slice of the row and leaves its best in `partial`; the CTA
// that finishes last (an arrival counter per row, reset for the next step) reduces the slices.
constexpr uint32_t kArgmaxSlices = 64;
__global__ void __launch_bounds__(256) argmax_kernel(const float *__restrict__ logits, uint32_t vocabulary, float *__restrict__ partial_value,
                                                     int32_t *__restrict__ partial_index, uint32_t *__restrict__ arrivals, int32_t *__restrict__ out)
{
    __shared__ float best_value[8];
    __shared__ int best_index[8];
    __shared__ bool last;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const float *row = logits + (uint64_t)blockIdx.y * vocabulary;
    const uint32_t slice = (vocabulary + kArgmaxSlices - 1) / kArgmaxSlices;
    const uint32_t begin = blockIdx.x * slice, end = min(vocabulary, begin + slice);
    float value = -INFINITY;
    int index = 0x7fffffff;
    auto better = [](float v, int i, float value, int index) { return v > value || (v == value && i < index); };
    for (uint32_t i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const float v = row[i];
        if (better(v, (int)i, value, index)) {
            value = v;
            index = (int)i;
        }
    }
    auto reduce_cta = [&]() {
        for (int offset = 16; offset > 0; offset >>= 1) {
            const float other_value = __shfl_xor_sync(0xffffffffu, value, offset);
            const int other_index = __shfl_xor_sync(0xffffffffu, index, offset);
            if (better(other_value, other_index, value, index)) {
                value = other_value;
                index = other_index;
            }
        }
        if ((threadIdx.x & 31) == 0) {
            best_value[threadIdx.x >> 5] = value;
            best_index[threadIdx.x >> 5] = index;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < (int)(blockDim.x >> 5); ++w) {
                if (better(best_value[w], best_index[w], value, index)) {
                    value = best_value[w];
                    index = best_index[w];
                }
            }
        }
    };
    reduce_cta();
    if (threadIdx.x == 0) {
        partial_value[blockIdx.y * kArgmaxSlices + blockIdx.x] = value;
        partial_index[blockIdx.y * kArgmaxSlices + blockIdx.x] = index;
        __threadfence();
        last = atomicAdd(arrivals + blockIdx.y, 1u) + 1 == gridDim.x;
    }
    __syncthreads();
    if (!last) {
        return;
    }
    __threadfence();
    value = -INFINITY;
    index = 0x7fffffff;
    if (threadIdx.x < kArgmaxSlices) {
        value = __ldcg(partial_value + blockIdx.y * kArgmaxSlices + threadIdx.x);
        index = __ldcg(partial_index + blockIdx.y * kArgmaxSlices + threadIdx.x);
    }
    __syncthreads();
    reduce_cta();
    if (threadIdx.x == 0) {
        out[blockIdx.y] = index;
        arrivals[blockIdx.y] = 0;
    }
}

struct Layer {
    syn_b200_matrix *query = nullptr, *key = nullptr, *value = nullptr, *output = nullptr, *gate = nullptr, *up = nullptr, *down = nullptr;
    float *attention_norm = nullptr, *feed_forward_norm = nullptr, *query_bias = nullptr, *key_bias = nullptr, *value_bias = nullptr;
};

}  // namespace

}  // namespace syn

using namespace syn;

struct syn_b200_decoder {
    syn_b200_decoder_desc shape{};  // scalars only; the pointers inside are not kept
    int device = 0;
    cudaStream_t stream = nullptr;
    cudaStream_t side[2] = {};      // the key and value projections run beside the query projection
    cudaEvent_t fork = nullptr, join[2] = {};
    std::vector<Layer> layers;
    syn_b200_matrix *embedding = nullptr, *output = nullptr;
    float *output_norm = nullptr, *cosines = nullptr, *sines = nullptr;
    std::vector<void *> owned;  // every cudaMalloc'd block, for destroy
    float *hidden = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *attention = nullptr, *gate = nullptr, *ff = nullptr, *logits = nullptr;
    void *act_hidden = nullptr, *act_ffn = nullptr;
    float *keys = nullptr, *values = nullptr;
    // attention of long caches: CTAs per head, their shares and arrival counters (null with one CTA per head)
    uint32_t attention_splits = 1;
    float *split_partial = nullptr;
    uint32_t *split_arrivals = nullptr;
    syn::BatchToken *device_tokens = nullptr, *host_tokens = nullptr;
    int32_t *device_argmax = nullptr, *host_argmax = nullptr;
    float *argmax_value = nullptr;       // per logits row and slice: the slice's best value and its index
    int32_t *argmax_index = nullptr;
    uint32_t *argmax_arrivals = nullptr;  // per logits row: slices done (zero between steps)
    float *host_logits = nullptr;  // pinned staging for the logits: a copy into pageable caller memory is slower than this plus a memcpy
    cudaGraphExec_t graphs[kMaxGraphTokens + 1] = {};
    uint64_t launches_per_step[kMaxGraphTokens + 1] = {};
    uint32_t steps_seen[kMaxGraphTokens + 1] = {};  // the first step of a token count runs uncaptured (one-time kernel set-up)
    // Single-token steps run as one persistent kernel when the model fits it (decode_program.cuh).
    bool program_ready = false;
    syn::prog::Op *program_ops = nullptr;
    uint32_t *program_sync = nullptr;
    syn::prog::Params program{};
    uint32_t program_grid = 0, program_shared = 0;
    uint64_t *program_timeline = nullptr;  // only with SYN_B200_PROGRAM_TIMELINE set: per-operation timestamps of CTA 0
    std::vector<uint32_t> program_kinds;
};

namespace syn {
namespace {

template <class T>
int32_t device_alloc(syn_b200_decoder *d, T **out, uint64_t count)
{
    void *p = nullptr;
    cudaError_t error = cudaMalloc(&p, count * sizeof(T) + 256);
    if (error != cudaSuccess) {
        cudaGetLastError();
        return cuda_fail(error, "allocating decoder buffers");
    }
    d->owned.push_back(p);
    *out = static_cast<T *>(p);
    return SYN_B200_OK;
}

int32_t upload_floats(syn_b200_decoder *d, const syn_b200_decoder_desc &desc, uint64_t offset, uint64_t count, const char *name, float **out)
{
    if (offset == kNoTensor) {
        *out = nullptr;
        return SYN_B200_OK;
    }
    if (offset % 4 != 0 || offset > desc.weights_length || count * 4 > desc.weights_length - offset) {
        return fail(SYN_B200_INVALID_ARGUMENT, std::string("tensor ") + name + " lies outside the weights or is misaligned");
    }
    int32_t status = device_alloc(d, out, count);
    if (status != SYN_B200_OK) {
        return status;
    }
    cudaError_t error = cudaMemcpy(*out, desc.weights + offset, count * 4, cudaMemcpyHostToDevice);
    return error == cudaSuccess ? SYN_B200_OK : cuda_fail(error, "uploading a decoder tensor");
}

int32_t upload_matrix(const syn_b200_decoder_desc &desc, uint64_t offset, uint32_t type, uint64_t rows, uint64_t columns, uint32_t flags,
                      const char *name, syn_b200_matrix **out)
{
    const uint64_t values = block_values(type);
    if (values == 0) {
        return fail(SYN_B200_UNAVAILABLE, std::string("tensor ") + name + " uses GGML type " + std::to_string(type) + ", which is not implemented");
    }
    if (columns % values != 0) {
        return fail(SYN_B200_UNAVAILABLE, std::string("tensor ") + name + " has " + std::to_string(columns) + " columns, not a multiple of its " +
                                              std::to_string(values) + "-value blocks");
    }
    const uint64_t bytes = rows * (columns / values) * block_bytes(type);
    if (offset % 2 != 0 || offset > desc.weights_length || bytes > desc.weights_length - offset) {
        return fail(SYN_B200_INVALID_ARGUMENT, std::string("tensor ") + name + " lies outside the weights");
    }
    return syn_b200_matrix_create(desc.weights + offset, type, rows, columns, flags, out);
}

cudaError_t product(syn_b200_decoder *d, const syn_b200_matrix *m, const void *act, uint32_t tokens, float *y, uint64_t out_stride,
                    const Epilogue &epilogue, cudaStream_t stream = nullptr)
{
    MatvecArgs args{};
    args.matrix = m;
    args.row_start = 0;
    args.row_count = m->rows;
    args.tokens = tokens;
    args.act = act_view(act, tokens, m->columns);
    args.act_ready = true;
    args.y = y;
    args.out_stride = out_stride;
    args.mode = SYN_B200_MODE_XQ8;
    args.epilogue = SYN_B200_EPILOGUE_STORE;
    args.fused = epilogue;
    return launch_matvec(args, stream ? stream : d->stream);
}

cudaError_t quantize(syn_b200_decoder *d, const float *x, uint32_t tokens, uint64_t columns, void *act)
{
    const ActLayout layout = act_layout(tokens, columns);
    uint8_t *base = static_cast<uint8_t *>(act);
    return launch_quantize(x, tokens, columns, columns, reinterpret_cast<int8_t *>(base + layout.codes),
                           reinterpret_cast<float *>(base + layout.scales), reinterpret_cast<int16_t *>(base + layout.sums), d->stream);
}

cudaError_t norm_quantize(syn_b200_decoder *d, const float *x, const float *weight, uint32_t tokens, uint32_t rows, bool by_logits_row, void *act)
{
    const uint32_t n = d->shape.hidden;
    const ActLayout layout = act_layout(rows, n);
    uint8_t *base = static_cast<uint8_t *>(act);
    return launch_kernel(rmsnorm_quantize_kernel, dim3(tokens), dim3(kNormWarps * 32), 0, d->stream, (const BatchToken *)d->device_tokens, x, weight,
                         d->shape.rms_epsilon, n, rows, by_logits_row ? 1u : 0u, reinterpret_cast<int8_t *>(base + layout.codes),
                         reinterpret_cast<float *>(base + layout.scales), reinterpret_cast<int16_t *>(base + layout.sums));
}

#define SYN_TRY(expression)                \
    do {                                   \
        cudaError_t syn_error = (expression); \
        if (syn_error != cudaSuccess) {    \
            return syn_error;              \
        }                                  \
    } while (0)

// Queues one step for `count` tokens (already in device_tokens) on the decoder's stream.
cudaError_t enqueue_step(syn_b200_decoder *d, uint32_t count, uint32_t logits_rows)
{
    const syn_b200_decoder_desc &s = d->shape;
    const uint32_t hidden = s.hidden, kvw = s.kv_heads * s.head_dim, ffn = s.feed_forward;
    SYN_TRY(launch_kernel(embed_kernel, dim3((hidden + 255) / 256, count), dim3(256), 0, d->stream, d->device_tokens,
                          (const uint8_t *)d->embedding->data, d->embedding->type, d->embedding->row_bytes, hidden, d->hidden));
    for (uint32_t l = 0; l < s.layer_count; ++l) {
        const Layer &L = d->layers[l];
        SYN_TRY(norm_quantize(d, d->hidden, L.attention_norm, count, count, false, d->act_hidden));
        // q | k | v read the same activations and write disjoint outputs. Matrices of one encoding share a launch (the
        // reference's three-segment dispatch, step/layers.rs:71-94); the others fork onto side streams (parallel
        // branches of the captured graph) and join before the rotation.
        {
            const syn_b200_matrix *members[3] = {L.query, L.key, L.value};
            float *outputs[3] = {d->q, d->k, d->v};
            const float *biases[3] = {L.query_bias, L.key_bias, L.value_bias};
            const uint64_t strides[3] = {hidden, kvw, kvw};
            bool done[3] = {false, false, false};
            if (count == 1) {
                // one token: q, k and v are three vectors of one buffer only by convention; out_column is relative to d->q
                MatvecArgs args{};
                args.form = 1;
                for (int i = 0; i < 3; ++i) {
                    if (members[i]->type == L.query->type && members[i]->layout == L.query->layout) {
                        MatvecSegment &segment = args.segments[args.segment_count++];
                        segment.matrix = members[i];
                        segment.row_count = members[i]->rows;
                        segment.bias = biases[i];
                        segment.out_column = (uint64_t)(outputs[i] - d->q);
                        args.row_count += members[i]->rows;
                        done[i] = true;
                    }
                }
                cudaError_t error = cudaErrorNotSupported;
                if (args.segment_count > 1) {
                    args.matrix = L.query;
                    args.tokens = 1;
                    args.act = act_view(d->act_hidden, 1, hidden);
                    args.act_ready = true;
                    args.y = d->q;
                    args.out_stride = hidden;
                    args.mode = SYN_B200_MODE_XQ8;
                    error = launch_matvec(args, d->stream);
                }
                if (error == cudaErrorNotSupported) {
                    done[0] = done[1] = done[2] = false;
                } else if (error != cudaSuccess) {
                    return error;
                }
            }
            int branch = 0;
            SYN_TRY(cudaEventRecord(d->fork, d->stream));
            for (int i = 1; i < 3; ++i) {
                if (!done[i]) {
                    Epilogue bias;
                    bias.bias = biases[i];
                    SYN_TRY(cudaStreamWaitEvent(d->side[branch], d->fork, 0));
                    SYN_TRY(product(d, members[i], d->act_hidden, count, outputs[i], strides[i], bias, d->side[branch]));
                    SYN_TRY(cudaEventRecord(d->join[branch], d->side[branch]));
                    ++branch;
                }
            }
            if (!done[0]) {
                Epilogue bias;
                bias.bias = biases[0];
                SYN_TRY(product(d, members[0], d->act_hidden, count, outputs[0], strides[0], bias));
            }
            for (int i = 0; i < branch; ++i) {
                SYN_TRY(cudaStreamWaitEvent(d->stream, d->join[i], 0));
            }
        }
        {
            // the attention output replaces the normalised activations of this layer in the same scratch
            const ActLayout layout = act_layout(count, hidden);
            uint8_t *base = static_cast<uint8_t *>(d->act_hidden);
            const float scale = 1.0f / sqrtf((float)s.head_dim);
            auto attend = [&](auto *cache_keys, auto *cache_values) -> cudaError_t {
                using KV = std::remove_pointer_t<decltype(cache_keys)>;
                int8_t *const codes = reinterpret_cast<int8_t *>(base + layout.codes);
                float *const scales = reinterpret_cast<float *>(base + layout.scales);
                int16_t *const sums = reinterpret_cast<int16_t *>(base + layout.sums);
                auto launch = [&](auto kernel) -> cudaError_t {
                    return launch_kernel(kernel, dim3(s.heads, count, d->attention_splits), dim3(32 * prog::kAttentionWarps), 0, d->stream,
                                         (const BatchToken *)d->device_tokens, (const float *)d->q, (const float *)d->k, (const float *)d->v,
                                         (const float *)d->cosines, (const float *)d->sines, cache_keys, cache_values, s.heads, s.kv_heads, s.head_dim, l,
                                         s.layer_count, s.context, scale, codes, scales, sums, d->split_partial, d->split_arrivals);
                };
                // the kernel built for this head width, step form and number of CTAs per head
                auto pick = [&](auto rotate, auto split) -> cudaError_t {
                    constexpr bool kRotate = decltype(rotate)::value, kSplit = decltype(split)::value;
                    if (s.head_dim <= 32) return launch(attention_kernel<kRotate, KV, 1, kSplit>);
                    if (s.head_dim <= 64) return launch(attention_kernel<kRotate, KV, 2, kSplit>);
                    if (s.head_dim <= 128) return launch(attention_kernel<kRotate, KV, 4, kSplit>);
                    return launch(attention_kernel<kRotate, KV, 8, kSplit>);
                };
                const bool split = d->attention_splits > 1;
                if (count == 1) {
                    return split ? pick(std::true_type{}, std::true_type{}) : pick(std::true_type{}, std::false_type{});
                }
                SYN_TRY(launch_kernel(rope_store_kernel<KV>, dim3(s.heads + s.kv_heads, count), dim3(s.head_dim / 2), 0, d->stream,
                                      (const BatchToken *)d->device_tokens, d->q, d->k, (const float *)d->v, (const float *)d->cosines,
                                      (const float *)d->sines, cache_keys, cache_values, s.heads, s.kv_heads, s.head_dim, l, s.layer_count, s.context));
                return split ? pick(std::false_type{}, std::true_type{}) : pick(std::false_type{}, std::false_type{});
            };
            if (s.kv_precision == 1) {
                SYN_TRY(attend(reinterpret_cast<__half *>(d->keys), reinterpret_cast<__half *>(d->values)));
            } else {
                SYN_TRY(attend(d->keys, d->values));
            }
        }
        Epilogue residual;
        residual.accumulate = 1;
        SYN_TRY(product(d, L.output, d->act_hidden, count, d->hidden, hidden, residual));
        SYN_TRY(norm_quantize(d, d->hidden, L.feed_forward_norm, count, count, false, d->act_hidden));
        {
            // gate | up: one launch whose warps hold gate row r and up row r and apply SwiGLU in registers (single-token
            // steps of matching encodings); otherwise the gate values go through memory into the up product's epilogue
            cudaError_t error = cudaErrorNotSupported;
            if (count == 1 && L.gate->type == L.up->type && L.gate->layout == L.up->layout) {
                MatvecArgs args{};
                args.form = 2;
                args.segment_count = 2;
                args.segments[0].matrix = L.gate;
                args.segments[1].matrix = L.up;
                args.segments[0].row_count = args.segments[1].row_count = ffn;
                args.matrix = L.gate;
                args.row_count = ffn;
                args.tokens = 1;
                args.act = act_view(d->act_hidden, 1, hidden);
                args.act_ready = true;
                args.y = d->ff;
                args.out_stride = ffn;
                args.mode = SYN_B200_MODE_XQ8;
                error = launch_matvec(args, d->stream);
            }
            if (error == cudaErrorNotSupported) {
                SYN_TRY(product(d, L.gate, d->act_hidden, count, d->gate, ffn, Epilogue{}));
                Epilogue swiglu;
                swiglu.gate = d->gate;
                swiglu.gate_stride = ffn;
                SYN_TRY(product(d, L.up, d->act_hidden, count, d->ff, ffn, swiglu));
            } else if (error != cudaSuccess) {
                return error;
            }
        }
        SYN_TRY(quantize(d, d->ff, count, ffn, d->act_ffn));
        SYN_TRY(product(d, L.down, d->act_ffn, count, d->hidden, hidden, residual));
    }
    if (logits_rows > 0) {
        SYN_TRY(norm_quantize(d, d->hidden, d->output_norm, count, logits_rows, true, d->act_hidden));
        SYN_TRY(product(d, d->output, d->act_hidden, logits_rows, d->logits, s.vocabulary, Epilogue{}));
        SYN_TRY(launch_kernel(argmax_kernel, dim3(kArgmaxSlices, logits_rows), dim3(256), 0, d->stream, (const float *)d->logits, s.vocabulary,
                              d->argmax_value, d->argmax_index, d->argmax_arrivals, d->device_argmax));
    }
    return cudaSuccess;
}

// ---- the single-token step as one persistent kernel ------------------------------------------------------

// Describes `m` as a projection of the program; false when its encoding or layout has no in-kernel consumer.
bool program_matvec(const syn_b200_matrix *m, float *y, const float *bias, const float *gate, bool accumulate, prog::Op &op)
{
    using namespace prog;
    const uint64_t K = m->columns;
    uint32_t units = 0, U = 1;
    op = Op{};
    op.kind = kOpMatvec;
    if (m->type == kQ8_0 && m->layout == Layout::Planar) {
        op.format = kFormatQ8Planar;
        units = (uint32_t)(K / 16);
        U = mv::Q8PlanarXq8::kMaxUpl;
        op.planes = mv::Q8PlanarXq8::kPlanes;
        mv::Q8PlanarXq8::plane_row_bytes(K, m->row_bytes, op.plane_row_bytes);
        op.plane[0] = m->data + m->planes.p0;
        op.plane[1] = m->data + m->planes.p1;
    } else if (m->type == kQ4_K && m->layout == Layout::Natural) {
        op.format = kFormatQ4K;
        units = (uint32_t)(K / 128);
        U = mv::Q4KXq8::kMaxUpl;
        op.planes = mv::Q4KXq8::kPlanes;
        mv::Q4KXq8::plane_row_bytes(K, m->row_bytes, op.plane_row_bytes);
        op.plane[0] = m->data;
    } else if (m->type == kQ6_K && m->layout == Layout::Planar) {
        op.format = kFormatQ6KPlanar;
        units = (uint32_t)(K / 64);
        U = mv::Q6KPlanarXq8::kMaxUpl;
        op.planes = mv::Q6KPlanarXq8::kPlanes;
        mv::Q6KPlanarXq8::plane_row_bytes(K, m->row_bytes, op.plane_row_bytes);
        op.plane[0] = m->data + m->planes.p0;
        op.plane[1] = m->data + m->planes.p1;
        op.plane[2] = m->data + m->planes.p2;
        op.plane[3] = m->data + m->planes.p3;
    } else {
        return false;
    }
    // The team shape of launch_format: it depends on the row length only.
    if (units <= 32) {
        op.team = 1;
        op.upl = 1;
        op.one_pass = 1;
    } else {
        const uint32_t teams = (units + 32 * U - 1) / (32 * U);
        if (teams > 8) {
            return false;  // rows that need several passes of an eight-warp team stay with the per-operation kernels
        }
        op.team = teams;
        op.upl = U;
        op.one_pass = 1;
    }
    op.rows = (uint32_t)m->rows;
    op.columns = (uint32_t)K;
    op.group_rows = prog::kConsumerWarps / op.team;
    uint64_t offset = 0;
    for (uint32_t k = 0; k < op.planes; ++k) {
        op.plane_offset[k] = (uint32_t)offset;
        offset += align_up((uint64_t)op.group_rows * op.plane_row_bytes[k] + 16, 128);
    }
    op.stage_bytes = (uint32_t)offset;
    op.teams = op.group_rows;
    op.groups = (op.rows + op.teams - 1) / op.teams;
    op.units = units;
    op.scales_offset = mv::shared_act_codes_bytes(1, (uint32_t)K);
    op.sums_offset = op.scales_offset + mv::shared_act_side_bytes(1, (uint32_t)K);
    for (uint32_t warp = 0; warp < (uint32_t)prog::kConsumerWarps; ++warp) {
        const bool active = warp < op.teams * op.team;
        op.team_of_warp |= (uint64_t)(active ? warp / op.team : 0) << (4 * warp);
        op.index_in_team |= (uint64_t)(warp % op.team) << (4 * warp);
    }
    op.y = y;
    op.bias = bias;
    op.gate = gate;
    op.accumulate = accumulate ? 1u : 0u;
    return true;
}

// Builds the program of a one-token step. Leaves d->program_ready false (the per-operation kernels are used)
// when the model does not fit: an encoding without an in-kernel consumer, more heads than CTAs, no room for the ring.
cudaError_t build_program(syn_b200_decoder *d)
{
    using namespace prog;
    const syn_b200_decoder_desc &s = d->shape;
    // The single-kernel form of the step is built on request only (SYN_B200_DECODE_PROGRAM=1): since the per-operation
    // kernels launch one kernel per fused region and overlap through programmatic dependent launch, the replayed graph
    // of them is the faster form on every shape measured (7B Q4_K_M: 1.6 ms per token against 1.8 ms; 0.5B Q8_0: 0.65
    // against 1.0 ms). The program stays as the reference point for that comparison and is kept bit-identical by the tests.
    const char *choice = getenv("SYN_B200_DECODE_PROGRAM");
    if (!choice || choice[0] != '1' || s.kv_precision != 0) {
        return cudaSuccess;  // (the program reads an FP32 cache)
    }
    int cooperative = 0;
    cudaDeviceGetAttribute(&cooperative, cudaDevAttrCooperativeLaunch, d->device);
    const uint32_t grid = (uint32_t)sm_count(d->device);
    if (!cooperative || s.heads > grid || s.head_dim > 256) {
        return cudaSuccess;
    }
    // the in-kernel quantiser holds a whole vector in the registers of one CTA
    if (s.hidden > (uint32_t)kNormDepth * kConsumerWarps * 128 || s.feed_forward > (uint32_t)kPlainDepth * kConsumerWarps * 128) {
        return cudaSuccess;
    }
    std::vector<Op> ops;
    uint32_t cursor = 0;
    bool supported = true;
    auto matvec = [&](const syn_b200_matrix *m, float *y, const float *bias, const float *gate, bool accumulate) -> Op * {
        Op op;
        if (!program_matvec(m, y, bias, gate, accumulate, op)) {
            supported = false;
            return nullptr;
        }
        op.first_cta = cursor % grid;
        cursor = (cursor + op.groups) % grid;
        ops.push_back(op);
        return &ops.back();
    };
    auto quantize = [&](const float *x, const float *norm, uint32_t n) {
        Op op;
        op.kind = kOpQuantize;
        op.barrier = 1;  // x was written by other CTAs, and every warp must be done with the previous activations
        op.x = x;
        op.norm_weight = norm;
        op.epsilon = s.rms_epsilon;
        op.columns = n;
        ops.push_back(op);
    };
    {
        Op op;
        op.kind = kOpEmbed;
        op.format = d->embedding->type;
        op.plane[0] = d->embedding->data;
        op.row_bytes = d->embedding->row_bytes;
        op.columns = s.hidden;
        op.y = d->hidden;
        ops.push_back(op);
    }
    if (d->embedding->layout != Layout::Natural) {
        supported = false;
    }
    for (uint32_t l = 0; l < s.layer_count && supported; ++l) {
        const Layer &L = d->layers[l];
        quantize(d->hidden, L.attention_norm, s.hidden);
        matvec(L.query, d->q, L.query_bias, nullptr, false);
        matvec(L.key, d->k, L.key_bias, nullptr, false);
        matvec(L.value, d->v, L.value_bias, nullptr, false);
        {
            Op op;
            op.kind = kOpAttention;
            op.barrier = 1;
            op.layer = l;
            ops.push_back(op);
        }
        quantize(d->attention, nullptr, s.hidden);
        matvec(L.output, d->hidden, nullptr, nullptr, true);
        quantize(d->hidden, L.feed_forward_norm, s.hidden);
        const uint32_t gate_cta = cursor;
        Op *gate = matvec(L.gate, d->gate, nullptr, nullptr, false);
        const Op gate_copy = gate ? *gate : Op{};
        const uint32_t after_gate = cursor;
        cursor = gate_cta;  // the up projection reads each gate value in the thread that wrote it: same row-to-CTA map
        Op *up = matvec(L.up, d->ff, nullptr, d->gate, false);
        if (gate && up) {
            if (up->format != gate_copy.format || up->team != gate_copy.team || up->upl != gate_copy.upl || up->rows != gate_copy.rows) {
                up->barrier = 1;  // different team shapes: the gate values come from other threads, through global memory
            } else if ((up->groups + grid - 1) / grid <= kStashIterations) {
                up->gate_stash = 2;
                (up - 1)->gate_stash = 1;  // the gate projection is the operation before
            }
        }
        cursor = (after_gate + (cursor + grid - gate_cta) % grid) % grid;
        quantize(d->ff, nullptr, s.feed_forward);
        matvec(L.down, d->hidden, nullptr, nullptr, true);
    }
    if (supported) {
        quantize(d->hidden, d->output_norm, s.hidden);
        if (Op *head = matvec(d->output, d->logits, nullptr, nullptr, false)) {
            head->track_argmax = 1;
        }
        Op op;
        op.kind = kOpArgmax;
        op.barrier = 1;
        ops.push_back(op);
    }
    if (!supported) {
        return cudaSuccess;
    }
    uint32_t largest = 0, longest = s.hidden > s.feed_forward ? s.hidden : s.feed_forward;
    for (const Op &op : ops) {
        if (op.kind == kOpMatvec && op.stage_bytes > largest) {
            largest = op.stage_bytes;
        }
    }
    const uint32_t act_bytes = (uint32_t)align_up(mv::shared_act_bytes(1, longest), 128);
    // the ring must hold at least two of the largest stages, or the producer could never run ahead
    if (largest == 0 || act_bytes + 2 * (uint64_t)largest > kDynamicSharedBudget) {
        return cudaSuccess;
    }
    const uint32_t ring_bytes = (kDynamicSharedBudget - act_bytes) / 128 * 128;
    const uint32_t dynamic = act_bytes + ring_bytes;
    cudaError_t error = cudaFuncSetAttribute(decode_program_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dynamic);
    int resident = 0;
    if (error == cudaSuccess) {
        error = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, decode_program_kernel, kThreads, dynamic);
    }
    if (error != cudaSuccess) {
        return error;
    }
    if (resident < 1) {
        return cudaSuccess;
    }
    void *p = nullptr;
    error = cudaMalloc(&p, ops.size() * sizeof(Op));
    if (error != cudaSuccess) {
        return error;
    }
    d->owned.push_back(p);
    d->program_ops = static_cast<Op *>(p);
    error = cudaMemcpy(d->program_ops, ops.data(), ops.size() * sizeof(Op), cudaMemcpyHostToDevice);
    if (error != cudaSuccess) {
        return error;
    }
    std::vector<ProducerOp> streams;
    for (const Op &op : ops) {
        if (op.kind == kOpMatvec) {
            ProducerOp stream;
            for (int k = 0; k < 4; ++k) {
                stream.plane[k] = op.plane[k];
                stream.plane_row_bytes[k] = op.plane_row_bytes[k];
                stream.plane_offset[k] = op.plane_offset[k];
            }
            stream.rows = op.rows;
            stream.group_rows = op.group_rows;
            stream.first_cta = op.first_cta;
            stream.planes = op.planes;
            stream.stage_bytes = op.stage_bytes;
            stream.groups = op.groups;
            streams.push_back(stream);
        }
    }
    error = cudaMalloc(&p, streams.size() * sizeof(ProducerOp));
    if (error != cudaSuccess) {
        return error;
    }
    d->owned.push_back(p);
    error = cudaMemcpy(p, streams.data(), streams.size() * sizeof(ProducerOp), cudaMemcpyHostToDevice);
    if (error != cudaSuccess) {
        return error;
    }
    const ProducerOp *producer_ops = static_cast<const ProducerOp *>(p);
    error = cudaMalloc(&p, 256);
    if (error != cudaSuccess) {
        return error;
    }
    d->owned.push_back(p);
    d->program_sync = static_cast<uint32_t *>(p);
    Params &P = d->program;
    P.ops = d->program_ops;
    P.op_count = (uint32_t)ops.size();
    P.producer_ops = producer_ops;
    P.producer_count = (uint32_t)streams.size();
    P.token = d->device_tokens;
    P.sync = d->program_sync;
    P.fault = fault_word_device();
    P.ring_bytes = ring_bytes;
    P.act_bytes = act_bytes;
    P.q = d->q;
    P.k = d->k;
    P.v = d->v;
    P.attention = d->attention;
    P.keys = d->keys;
    P.values = d->values;
    P.cosines = d->cosines;
    P.sines = d->sines;
    P.heads = s.heads;
    P.kv_heads = s.kv_heads;
    P.head_dim = s.head_dim;
    P.layers = s.layer_count;
    P.context = s.context;
    P.attention_scale = 1.0f / sqrtf((float)s.head_dim);
    error = cudaMalloc(&p, 2 * grid * sizeof(float));
    if (error != cudaSuccess) {
        return error;
    }
    d->owned.push_back(p);
    P.best_value = static_cast<float *>(p);
    P.best_index = reinterpret_cast<int32_t *>(P.best_value + grid);
    P.argmax = d->device_argmax;
    P.timeline = nullptr;
    if (getenv("SYN_B200_PROGRAM_TIMELINE")) {
        error = cudaMalloc(&p, (2 * ops.size() + 1) * sizeof(uint64_t));
        if (error == cudaSuccess) {
            error = cudaMemset(p, 0, (2 * ops.size() + 1) * sizeof(uint64_t));
        }
        if (error != cudaSuccess) {
            return error;
        }
        d->owned.push_back(p);
        d->program_timeline = P.timeline = static_cast<uint64_t *>(p);
        for (const Op &op : ops) {
            d->program_kinds.push_back(op.kind);
        }
    }
    d->program_grid = grid;
    d->program_shared = dynamic;
    d->program_ready = true;
    return cudaSuccess;
}

// Queues a one-token step (token already in host_tokens) as the persistent kernel.
cudaError_t enqueue_program(syn_b200_decoder *d)
{
    cudaError_t error = cudaMemcpyAsync(d->device_tokens, d->host_tokens, sizeof(BatchToken), cudaMemcpyHostToDevice, d->stream);
    if (error == cudaSuccess) {
        error = cudaMemsetAsync(d->program_sync, 0, 8, d->stream);
    }
    if (error != cudaSuccess) {
        return error;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(d->program_grid);
    config.blockDim = dim3(prog::kThreads);
    config.dynamicSmemBytes = d->program_shared;
    config.stream = d->stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeCooperative;  // all CTAs resident at once, or the launch fails
    attribute[0].val.cooperative = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    count_launch();
    error = cudaLaunchKernelEx(&config, prog::decode_program_kernel, d->program);
    if (error == cudaSuccess && d->program_timeline) {
        // Profiling aid: nanoseconds CTA 0 spent per kind of operation, and waiting in the grid barriers.
        std::vector<uint64_t> t(2 * d->program_kinds.size() + 1);
        error = cudaStreamSynchronize(d->stream);
        if (error == cudaSuccess) {
            error = cudaMemcpy(t.data(), d->program_timeline, t.size() * sizeof(uint64_t), cudaMemcpyDeviceToHost);
        }
        if (error == cudaSuccess) {
            uint64_t by_kind[5] = {0, 0, 0, 0, 0}, barriers = 0;
            for (size_t i = 0; i < d->program_kinds.size(); ++i) {
                barriers += t[2 * i + 1] - t[2 * i];
                by_kind[d->program_kinds[i]] += t[2 * i + 2] - t[2 * i + 1];
            }
            const char *detail = getenv("SYN_B200_PROGRAM_TIMELINE");
            if (detail && detail[0] == '2') {
                for (size_t i = 0; i < d->program_kinds.size(); ++i) {
                    if (i >= 32 && i + 4 < d->program_kinds.size()) {
                        continue;
                    }
                    fprintf(stderr, "  op %zu kind %u at %llu: barrier %llu ns, body %llu ns\n", i, d->program_kinds[i],
                            (unsigned long long)(t[2 * i] - t[0]), (unsigned long long)(t[2 * i + 1] - t[2 * i]),
                            (unsigned long long)(t[2 * i + 2] - t[2 * i + 1]));
                }
            }
            fprintf(stderr, "decode program: total %llu ns; barriers %llu, embed %llu, quantize %llu, matvec %llu, attention %llu, argmax %llu\n",
                    (unsigned long long)(t[2 * d->program_kinds.size()] - t[0]), (unsigned long long)barriers, (unsigned long long)by_kind[0],
                    (unsigned long long)by_kind[1], (unsigned long long)by_kind[2], (unsigned long long)by_kind[3], (unsigned long long)by_kind[4]);
        }
    }
    return error;
}

// Validates a step like Qwen2CpuExecutor.Validate (Qwen2CpuExecutor.cs:141-163) and returns its logits rows.
int32_t validate_step(const syn_b200_decoder *d, const syn_b200_batch_token *tokens, uint64_t count, uint32_t *logits_rows)
{
    const syn_b200_decoder_desc &s = d->shape;
    if (count == 0 || count > s.step_tokens) {
        return fail(SYN_B200_INVALID_ARGUMENT, "a step holds 1.." + std::to_string(s.step_tokens) + " tokens, not " + std::to_string(count));
    }
    uint32_t rows = 0;
    for (uint64_t i = 0; i < count; ++i) {
        const syn_b200_batch_token &t = tokens[i];
        if (t.slot < 0 || (uint32_t)t.slot >= s.session_slots || t.token < 0 || (uint32_t)t.token >= s.vocabulary || t.position < 0 ||
            (uint32_t)t.position >= s.context || t.logits_row >= (int32_t)s.logits_rows) {
            return fail(SYN_B200_INVALID_ARGUMENT, "invalid batch token " + std::to_string(i));
        }
        if (t.logits_row >= 0) {
            if ((uint32_t)t.logits_row != rows) {
                return fail(SYN_B200_INVALID_ARGUMENT, "logits rows must be numbered 0, 1, ... in token order");
            }
            ++rows;
        }
    }
    *logits_rows = rows;
    return SYN_B200_OK;
}

int32_t run_step(syn_b200_decoder *d, const syn_b200_batch_token *tokens, uint64_t count, uint32_t *rows_out)
{
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device != d->device) {
        cudaGetLastError();
        return fail(SYN_B200_INVALID_ARGUMENT, "the decoder lives on device " + std::to_string(d->device) + ", which is not the calling thread's current device");
    }
    uint32_t rows = 0;
    int32_t status = validate_step(d, tokens, count, &rows);
    if (status != SYN_B200_OK) {
        return status;
    }
    *rows_out = rows;
    for (uint64_t i = 0; i < count; ++i) {
        d->host_tokens[i] = syn::BatchToken{tokens[i].slot, tokens[i].token, tokens[i].position, tokens[i].logits_row};
    }
    // Steps in which every token asks for logits (plain decoding) replay a graph captured on their second occurrence;
    // anything else is enqueued kernel by kernel.
    const bool graphable = true;
    cudaError_t error = cudaSuccess;
    if (d->program_ready && count == 1 && rows == 1) {
        error = enqueue_program(d);
    } else if (graphable && rows == count && count <= kMaxGraphTokens && d->steps_seen[count]++ > 0) {
        if (!d->graphs[count]) {
            fault_word_device();
            const uint64_t before = syn_b200_launch_count(0);
            cudaGraph_t graph = nullptr;
            error = cudaStreamBeginCapture(d->stream, cudaStreamCaptureModeThreadLocal);
            if (error == cudaSuccess) {
                error = cudaMemcpyAsync(d->device_tokens, d->host_tokens, count * sizeof(syn::BatchToken), cudaMemcpyHostToDevice, d->stream);
                if (error == cudaSuccess) {
                    error = enqueue_step(d, (uint32_t)count, rows);
                }
                cudaError_t end = cudaStreamEndCapture(d->stream, &graph);
                if (error == cudaSuccess) {
                    error = end;
                }
            }
            if (error == cudaSuccess) {
                error = cudaGraphInstantiate(&d->graphs[count], graph, 0);
            }
            if (graph) {
                cudaGraphDestroy(graph);
            }
            if (error != cudaSuccess) {
                cudaGetLastError();
                return cuda_fail(error, "capturing the decode step");
            }
            d->launches_per_step[count] = syn_b200_launch_count(0) - before;
        } else {
            for (uint64_t i = 0; i < d->launches_per_step[count]; ++i) {
                count_launch();
            }
        }
        error = cudaGraphLaunch(d->graphs[count], d->stream);
    } else {
        error = cudaMemcpyAsync(d->device_tokens, d->host_tokens, count * sizeof(syn::BatchToken), cudaMemcpyHostToDevice, d->stream);
        if (error == cudaSuccess) {
            error = enqueue_step(d, (uint32_t)count, rows);
        }
    }
    if (error != cudaSuccess) {
        cudaGetLastError();
        return cuda_fail(error, "running the decode step");
    }
    return SYN_B200_OK;
}

}  // namespace
}  // namespace syn

extern "C" {

int32_t syn_b200_decoder_create(const syn_b200_decoder_desc *desc, syn_b200_decoder **out)
{
    if (!desc || !out) {
        return fail(SYN_B200_NULL_POINTER, "model description or output");
    }
    *out = nullptr;
    if (!desc->weights || !desc->layers || !desc->rope_cosines || !desc->rope_sines) {
        return fail(SYN_B200_NULL_POINTER, "model description");
    }
    try {
        const syn_b200_decoder_desc &s = *desc;
        if (s.layer_count == 0 || s.hidden == 0 || s.feed_forward == 0 || s.heads == 0 || s.kv_heads == 0 || s.head_dim == 0 ||
            s.vocabulary == 0 || s.context == 0 || s.session_slots == 0 || s.step_tokens == 0 || s.logits_rows == 0) {
            return fail(SYN_B200_INVALID_ARGUMENT, "every decoder dimension must be positive");
        }
        if (s.heads % s.kv_heads != 0 || s.heads * s.head_dim != s.hidden || s.head_dim % 32 != 0 || s.head_dim > 256 || s.hidden % 32 != 0 || s.hidden > 32768 ||
            s.feed_forward % 32 != 0) {
            return fail(SYN_B200_UNAVAILABLE, "unsupported head geometry: heads * head_dim must equal hidden, head_dim a multiple of 32 up to 256");
        }
        if (s.step_tokens > kMaxStepTokens || s.logits_rows > s.step_tokens) {
            return fail(SYN_B200_UNAVAILABLE, "a step holds at most " + std::to_string(kMaxStepTokens) + " tokens on this backend");
        }
        if (s.kv_precision > 1) {
            // decoder_tests.rs:211-230: an unknown precision is an invalid argument, not a missing feature
            return fail(SYN_B200_INVALID_ARGUMENT, "unknown KV precision " + std::to_string(s.kv_precision) + " (0 = FP32, 1 = FP16)");
        }
        if (s.kv_precision == 1 && s.head_dim % 64 != 0) {
            return fail(SYN_B200_UNAVAILABLE, "the FP16 KV cache needs a head_dim that is a multiple of 64");
        }
        if (s.rope_layout != 0 || s.activation != 0) {
            return fail(SYN_B200_UNAVAILABLE, "only the NeoX rotary layout and SwiGLU are implemented");
        }
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess) {
            cudaGetLastError();
            return fail(SYN_B200_UNAVAILABLE, "no usable CUDA device");
        }
        syn_b200_decoder *d = new syn_b200_decoder();
        d->shape = s;
        d->shape.weights = nullptr;
        d->shape.layers = nullptr;
        d->shape.rope_cosines = d->shape.rope_sines = nullptr;
        d->device = device;
        int32_t status = SYN_B200_OK;
        auto fail_out = [&](int32_t code) {
            syn_b200_decoder_destroy(d);
            return code;
        };
        const uint32_t kvw = s.kv_heads * s.head_dim, half = s.head_dim / 2;
        // the embedding is read row by row in its file layout; the projections take the load-time repack
        status = upload_matrix(s, s.token_embedding, s.embedding_encoding, s.vocabulary, s.hidden, 0, "token_embd", &d->embedding);
        if (status == SYN_B200_OK) status = upload_matrix(s, s.output, s.output_encoding, s.vocabulary, s.hidden, SYN_B200_REPACK, "output", &d->output);
        if (status == SYN_B200_OK) status = upload_floats(d, s, s.output_norm, s.hidden, "output_norm", &d->output_norm);
        if (status != SYN_B200_OK) return fail_out(status);
        d->layers.resize(s.layer_count);
        for (uint32_t l = 0; l < s.layer_count; ++l) {
            const syn_b200_layer_offsets &o = s.layers[l];
            Layer &L = d->layers[l];
            auto type = [&](int index) { return (uint32_t)((o.encodings >> (4 * index)) & 0xF); };
            if (o.query_norm != kNoTensor || o.key_norm != kNoTensor) {
                return fail_out(fail(SYN_B200_UNAVAILABLE, "per-head query/key norms are not implemented"));
            }
            status = upload_floats(d, s, o.attention_norm, s.hidden, "attn_norm", &L.attention_norm);
            if (status == SYN_B200_OK) status = upload_floats(d, s, o.feed_forward_norm, s.hidden, "ffn_norm", &L.feed_forward_norm);
            if (status == SYN_B200_OK) status = upload_floats(d, s, o.query_bias, s.hidden, "attn_q.bias", &L.query_bias);
            if (status == SYN_B200_OK) status = upload_floats(d, s, o.key_bias, kvw, "attn_k.bias", &L.key_bias);
            if (status == SYN_B200_OK) status = upload_floats(d, s, o.value_bias, kvw, "attn_v.bias", &L.value_bias);
            if (status == SYN_B200_OK) status = upload_matrix(s, o.query, type(0), s.hidden, s.hidden, SYN_B200_REPACK, "attn_q", &L.query);
            if (status == SYN_B200_OK) status = upload_matrix(s, o.key, type(1), kvw, s.hidden, SYN_B200_REPACK, "attn_k", &L.key);
            if (status == SYN_B200_OK) status = upload_matrix(s, o.value, type(2), kvw, s.hidden, SYN_B200_REPACK, "attn_v", &L.value);
            if (status == SYN_B200_OK) status = upload_matrix(s, o.attention_output, type(3), s.hidden, s.hidden, SYN_B200_REPACK, "attn_output", &L.output);
            if (status == SYN_B200_OK) status = upload_matrix(s, o.gate, type(4), s.feed_forward, s.hidden, SYN_B200_REPACK, "ffn_gate", &L.gate);
            if (status == SYN_B200_OK) status = upload_matrix(s, o.up, type(5), s.feed_forward, s.hidden, SYN_B200_REPACK, "ffn_up", &L.up);
            if (status == SYN_B200_OK) status = upload_matrix(s, o.down, type(6), s.hidden, s.feed_forward, SYN_B200_REPACK, "ffn_down", &L.down);
            if (status != SYN_B200_OK) return fail_out(status);
        }
        const uint64_t T = s.step_tokens;
        const uint64_t cache = (uint64_t)s.session_slots * s.layer_count * s.kv_heads * s.context * s.head_dim;
        uint8_t *act_hidden = nullptr, *act_ffn = nullptr;
        status = device_alloc(d, &d->cosines, (uint64_t)s.context * half);
        if (status == SYN_B200_OK) status = device_alloc(d, &d->sines, (uint64_t)s.context * half);
        if (status == SYN_B200_OK) status = device_alloc(d, &d->hidden, T * s.hidden);
        // q, k and v live in one block, in this order: a launch that computes all three addresses k and v relative to q
        if (status == SYN_B200_OK) status = device_alloc(d, &d->q, T * (s.hidden + 2ull * kvw));
        if (status == SYN_B200_OK) {
            d->k = d->q + T * s.hidden;
            d->v = d->k + T * kvw;
        }
        if (status == SYN_B200_OK) status = device_alloc(d, &d->attention, T * s.hidden);
        if (status == SYN_B200_OK) status = device_alloc(d, &d->gate, T * s.feed_forward);
        if (status == SYN_B200_OK) status = device_alloc(d, &d->ff, T * s.feed_forward);
        if (status == SYN_B200_OK) status = device_alloc(d, &d->logits, (uint64_t)s.logits_rows * s.vocabulary);
        if (status == SYN_B200_OK) status = device_alloc(d, &act_hidden, act_layout(T, s.hidden).total);
        if (status == SYN_B200_OK) status = device_alloc(d, &act_ffn, act_layout(T, s.feed_forward).total);
        // the cache: `cache` elements each of keys and values, 4 or 2 bytes wide (held through float pointers either way)
        const uint64_t cache_floats = s.kv_precision == 1 ? (cache + 1) / 2 : cache;
        if (status == SYN_B200_OK) status = device_alloc(d, &d->keys, cache_floats);
        if (status == SYN_B200_OK) status = device_alloc(d, &d->values, cache_floats);
        // caches of 1024 positions and more: several CTAs per head (4, or 8 from 4096 positions on)
        d->attention_splits = s.context >= 4096 ? 8 : s.context >= 1024 ? 4 : 1;
        if (d->attention_splits > 1) {
            if (status == SYN_B200_OK) status = device_alloc(d, &d->split_partial, T * s.heads * d->attention_splits * (s.head_dim + 4ull));
            if (status == SYN_B200_OK) status = device_alloc(d, &d->split_arrivals, T * s.heads);
        }
        if (status == SYN_B200_OK) status = device_alloc(d, &d->device_tokens, T);
        if (status == SYN_B200_OK) status = device_alloc(d, &d->device_argmax, T);
        if (status == SYN_B200_OK) status = device_alloc(d, &d->argmax_value, T * kArgmaxSlices);
        if (status == SYN_B200_OK) status = device_alloc(d, &d->argmax_index, T * kArgmaxSlices);
        if (status == SYN_B200_OK) status = device_alloc(d, &d->argmax_arrivals, T);
        if (status != SYN_B200_OK) return fail_out(status);
        d->act_hidden = act_hidden;
        d->act_ffn = act_ffn;
        cudaError_t error = cudaMemcpy(d->cosines, s.rope_cosines, (uint64_t)s.context * half * 4, cudaMemcpyHostToDevice);
        if (error == cudaSuccess) error = cudaMemcpy(d->sines, s.rope_sines, (uint64_t)s.context * half * 4, cudaMemcpyHostToDevice);
        if (error == cudaSuccess) error = cudaMemset(d->argmax_arrivals, 0, T * sizeof(uint32_t));
        if (error == cudaSuccess && d->split_arrivals) error = cudaMemset(d->split_arrivals, 0, T * s.heads * sizeof(uint32_t));
        if (error == cudaSuccess) error = cudaMemset(d->keys, 0, cache_floats * 4);
        if (error == cudaSuccess) error = cudaMemset(d->values, 0, cache_floats * 4);
        if (error == cudaSuccess) error = cudaHostAlloc(reinterpret_cast<void **>(&d->host_tokens), T * sizeof(syn::BatchToken), cudaHostAllocDefault);
        if (error == cudaSuccess) error = cudaHostAlloc(reinterpret_cast<void **>(&d->host_argmax), T * sizeof(int32_t), cudaHostAllocDefault);
        if (error == cudaSuccess) {
            error = cudaHostAlloc(reinterpret_cast<void **>(&d->host_logits), (uint64_t)s.logits_rows * s.vocabulary * sizeof(float), cudaHostAllocDefault);
        }
        if (error == cudaSuccess) error = cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking);
        for (int i = 0; i < 2; ++i) {
            if (error == cudaSuccess) error = cudaStreamCreateWithFlags(&d->side[i], cudaStreamNonBlocking);
            if (error == cudaSuccess) error = cudaEventCreateWithFlags(&d->join[i], cudaEventDisableTiming);
        }
        if (error == cudaSuccess) error = cudaEventCreateWithFlags(&d->fork, cudaEventDisableTiming);
        if (error == cudaSuccess) error = build_program(d);
        if (error != cudaSuccess) {
            cudaGetLastError();
            return fail_out(cuda_fail(error, "setting up the decoder"));
        }
        *out = d;
        return SYN_B200_OK;
    } catch (...) {
        return fail(SYN_B200_INTERNAL, "exception at the ABI");
    }
}

void syn_b200_decoder_destroy(syn_b200_decoder *d)
{
    if (!d) {
        return;
    }
    if (d->stream) {
        cudaStreamSynchronize(d->stream);
    }
    for (cudaGraphExec_t graph : d->graphs) {
        if (graph) {
            cudaGraphExecDestroy(graph);
        }
    }
    for (Layer &L : d->layers) {
        syn_b200_matrix_destroy(L.query);
        syn_b200_matrix_destroy(L.key);
        syn_b200_matrix_destroy(L.value);
        syn_b200_matrix_destroy(L.output);
        syn_b200_matrix_destroy(L.gate);
        syn_b200_matrix_destroy(L.up);
        syn_b200_matrix_destroy(L.down);
    }
    syn_b200_matrix_destroy(d->embedding);
    syn_b200_matrix_destroy(d->output);
    for (void *p : d->owned) {
        cudaFree(p);
    }
    if (d->host_tokens) cudaFreeHost(d->host_tokens);
    if (d->host_argmax) cudaFreeHost(d->host_argmax);
    if (d->host_logits) cudaFreeHost(d->host_logits);
    for (int i = 0; i < 2; ++i) {
        if (d->side[i]) cudaStreamDestroy(d->side[i]);
        if (d->join[i]) cudaEventDestroy(d->join[i]);
    }
    if (d->fork) cudaEventDestroy(d->fork);
    if (d->stream) cudaStreamDestroy(d->stream);
    delete d;
}

int32_t syn_b200_decoder_forward(syn_b200_decoder *d, const syn_b200_batch_token *tokens, uint64_t count, float *logits, uint64_t logits_capacity)
{
    if (!d || !tokens || !logits) {
        return fail(SYN_B200_NULL_POINTER, "model, tokens, or logits");
    }
    try {
        uint32_t rows = 0;
        int32_t status = run_step(d, tokens, count, &rows);
        if (status != SYN_B200_OK) {
            return status;
        }
        if ((uint64_t)rows * d->shape.vocabulary > logits_capacity) {
            cudaStreamSynchronize(d->stream);
            return fail(SYN_B200_INVALID_ARGUMENT, "the logits buffer holds " + std::to_string(logits_capacity) + " floats, the step needs " +
                                                       std::to_string((uint64_t)rows * d->shape.vocabulary));
        }
        cudaError_t error = cudaSuccess;
        if (rows > 0) {
            error = cudaMemcpyAsync(d->host_logits, d->logits, (uint64_t)rows * d->shape.vocabulary * 4, cudaMemcpyDeviceToHost, d->stream);
        }
        if (error == cudaSuccess) {
            error = cudaStreamSynchronize(d->stream);
        }
        if (error != cudaSuccess) {
            cudaGetLastError();
            return cuda_fail(error, "reading the logits");
        }
        memcpy(logits, d->host_logits, (uint64_t)rows * d->shape.vocabulary * 4);
        return SYN_B200_OK;
    } catch (...) {
        return fail(SYN_B200_INTERNAL, "exception at the ABI");
    }
}

int32_t syn_b200_decoder_forward_argmax(syn_b200_decoder *d, const syn_b200_batch_token *tokens, uint64_t count, int32_t *argmax)
{
    if (!d || !tokens || !argmax) {
        return fail(SYN_B200_NULL_POINTER, "model, tokens, or argmax");
    }
    try {
        uint32_t rows = 0;
        int32_t status = run_step(d, tokens, count, &rows);
        if (status != SYN_B200_OK) {
            return status;
        }
        cudaError_t error = cudaSuccess;
        if (rows > 0) {
            error = cudaMemcpyAsync(d->host_argmax, d->device_argmax, rows * sizeof(int32_t), cudaMemcpyDeviceToHost, d->stream);
        }
        if (error == cudaSuccess) {
            error = cudaStreamSynchronize(d->stream);
        }
        if (error != cudaSuccess) {
            cudaGetLastError();
            return cuda_fail(error, "reading the argmax");
        }
        for (uint32_t r = 0; r < rows; ++r) {
            argmax[r] = d->host_argmax[r];
        }
        return SYN_B200_OK;
    } catch (...) {
        return fail(SYN_B200_INTERNAL, "exception at the ABI");
    }
}

uint64_t syn_b200_decoder_kv_bytes(const syn_b200_decoder *d)
{
    if (!d) {
        return 0;
    }
    const syn_b200_decoder_desc &s = d->shape;
    return 2ull * s.session_slots * s.layer_count * s.kv_heads * s.context * s.head_dim * (s.kv_precision == 1 ? 2 : 4);
}

}  // extern "C"
