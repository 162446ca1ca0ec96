// Prompt-run product on the 5th-generation tensor cores: Y[t][r] = sum_k W[r][k] * X[t][k] for quantised W and
// many tokens. Replaces synapse_q8_gemm (cuda/kernels/matmul.cu:147-189) and the Metal K-quant GEMMs
// (metal/shaders/matmul_kquant.metal:227-291), which dequantise into shared memory and multiply with FP32 FMAs.
//
// One persistent CTA per SM, warp-specialised:
//   warps 0-3   epilogue  tcgen05.ld the FP32 accumulator out of tensor memory, scale, store Y
//   warps 4-11  dequant   read GGUF blocks (L2, one k step ahead), unpack to fp16 with packed-half arithmetic, write
//                         the B operand tile into shared memory in the 128-byte-swizzled K-major layout the MMA reads
//   warp  12    loader    bulk-copies the A operand tile (activations, converted and pre-swizzled by a pre-pass)
//   warp  13    MMA       one lane issues tcgen05.mma (M=128 tokens, N=256 or 128 weight rows, K=16) and commits
// Tokens are the MMA's M so that the expensive operand to move, the 16-bit activations, is read once per 256 weight
// rows, and with two token tiles per CTA tile a weight tile is dequantised once per 256 tokens. The 512 columns of
// tensor memory hold two 128 x 256 FP32 accumulators: the two token tiles of a tile, or (one token tile) two
// buffers so that the epilogue of one tile overlaps the MMAs of the next. Operands are fp16 (weights carry a 2^8 prescale so that
// small block scales stay out of the fp16 subnormal range; the epilogue removes it exactly).
//
// Every mbarrier wait is bounded: when one gives up the kernel bumps the host-mapped fault word and carries on to
// completion (with wrong results) instead of hanging, and the tensor memory it holds is always released.
#include <cuda_fp16.h>

#include <atomic>

#include "common.cuh"

namespace syn {

namespace {

constexpr int kTileTokens = 128;  // MMA M
constexpr int kMaxTileRows = 256; // MMA N: 256, or 128 when that is needed to give every SM a tile
constexpr int kTileK = 64;        // one 128-byte swizzle row of fp16
constexpr int kMaxStages = 4;
constexpr uint32_t kTileABytes = kTileTokens * kTileK * 2;     // 16 KB
constexpr uint32_t kTileBBytes = kMaxTileRows * kTileK * 2;    // 32 KB
// A CTA tile covers TT token tiles (TT activation tiles per stage, TT accumulators) against one weight tile, so a
// weight tile is dequantised once per TT * 128 tokens. TT = 1: four 48 KB stages, two accumulator buffers.
// TT = 2: three 64 KB stages, both accumulators in use at once.
constexpr uint32_t stage_bytes(int tt) { return tt * kTileABytes + kTileBBytes; }
constexpr uint32_t stage_count(int tt) { return tt == 1 ? 4 : 3; }
constexpr uint32_t kDequantWarps = 8;
constexpr uint32_t kLoaderWarp = 4 + kDequantWarps, kMmaWarp = kLoaderWarp + 1;
constexpr uint32_t kGemmThreads = (kMmaWarp + 1) * 32;
constexpr uint32_t kSpinLimit = 1u << 22;
constexpr float kPrescale = 256.0f;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity)
                 : "memory");
    return ok != 0;
}
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, uint32_t *fault)
{
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) {
            return;
        }
    }
    if (fault) {
        atomicAdd(fault, 1u);
    }
}
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes),
                 "r"(bar)
                 : "memory");
}

// Shared-memory matrix descriptor of a K-major tile with 128-byte rows, 128-byte swizzle: 8-row groups are 1024
// bytes apart (stride byte offset), the leading byte offset is the canonical 1, descriptor version 1 (Blackwell).
__device__ __forceinline__ uint64_t smem_desc(uint32_t address)
{
    return (uint64_t)((address & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// kind::f16 instruction descriptor: FP32 accumulator, fp16 A and B, both K-major, N weight rows, M = 128 tokens.
constexpr uint32_t instr_desc(int n) { return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kTileTokens >> 4) << 24); }

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_load32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Position of 16-byte chunk `c` of row `r` inside a 128-byte-swizzled tile.
__device__ __forceinline__ uint32_t swizzled(uint32_t r, uint32_t c) { return r * 128u + ((c ^ (r & 7u)) << 4); }

// ------------------------------------------------------------------------------------------------------
// Pre-pass: FP32 activations -> fp16 A-operand tiles, [token tile][k tile][128 tokens][64 values], each tile stored
// exactly as it will sit in shared memory (128-byte swizzle). Inside every group of four values the order is
// (0, 2, 1, 3): that is the order in which the dequantiser's packed-half unpacking produces weights, and the MMA
// only needs A and B to agree on the order of k. Tokens past the end are zero.
// ------------------------------------------------------------------------------------------------------

__global__ void convert_activations_kernel(const float *__restrict__ x, uint64_t tokens, uint64_t in_stride, uint32_t k_tiles,
                                           uint32_t token_tiles, uint8_t *__restrict__ tiles, uint8_t *__restrict__ low_tiles,
                                           uint32_t *__restrict__ arrivals, uint32_t arrival_words)
{
    // (the product that follows counts the CTAs of a tile that have finished their part of k: zero before it starts)
    if (blockIdx.x == 0) {
        for (uint32_t i = threadIdx.x; i < arrival_words; i += blockDim.x) {
            arrivals[i] = 0;
        }
    }
    // `low_tiles` (null for plain fp16 operands) receives fp16(x - fp16(x)): with it an activation carries 22 bits.
    const uint64_t chunks = (uint64_t)token_tiles * k_tiles * kTileTokens * 8;
    for (uint64_t index = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; index < chunks; index += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t c = (uint32_t)(index & 7);
        const uint32_t n = (uint32_t)((index >> 3) & (kTileTokens - 1));
        const uint64_t tile = index >> 10;  // 128 tokens * 8 chunks
        const uint32_t kt = (uint32_t)(tile % k_tiles);
        const uint64_t tt = tile / k_tiles;
        const uint64_t token = tt * kTileTokens + n;
        uint4 out = make_uint4(0, 0, 0, 0), low = make_uint4(0, 0, 0, 0);
        if (token < tokens) {
            const float *source = x + token * in_stride + (uint64_t)kt * kTileK + c * 8;
            const float4 lo = __ldg(reinterpret_cast<const float4 *>(source));
            const float4 hi = __ldg(reinterpret_cast<const float4 *>(source + 4));
            const __half2 h0 = __floats2half2_rn(lo.x, lo.z), h1 = __floats2half2_rn(lo.y, lo.w);
            const __half2 h2 = __floats2half2_rn(hi.x, hi.z), h3 = __floats2half2_rn(hi.y, hi.w);
            out = make_uint4(*reinterpret_cast<const uint32_t *>(&h0), *reinterpret_cast<const uint32_t *>(&h1),
                             *reinterpret_cast<const uint32_t *>(&h2), *reinterpret_cast<const uint32_t *>(&h3));
            if (low_tiles) {
                const float2 f0 = __half22float2(h0), f1 = __half22float2(h1), f2 = __half22float2(h2), f3 = __half22float2(h3);
                const __half2 l0 = __floats2half2_rn(lo.x - f0.x, lo.z - f0.y), l1 = __floats2half2_rn(lo.y - f1.x, lo.w - f1.y);
                const __half2 l2 = __floats2half2_rn(hi.x - f2.x, hi.z - f2.y), l3 = __floats2half2_rn(hi.y - f3.x, hi.w - f3.y);
                low = make_uint4(*reinterpret_cast<const uint32_t *>(&l0), *reinterpret_cast<const uint32_t *>(&l1),
                                 *reinterpret_cast<const uint32_t *>(&l2), *reinterpret_cast<const uint32_t *>(&l3));
            }
        }
        *reinterpret_cast<uint4 *>(tiles + tile * kTileABytes + swizzled(n, c)) = out;
        if (low_tiles) {
            *reinterpret_cast<uint4 *>(low_tiles + tile * kTileABytes + swizzled(n, c)) = low;
        }
    }
}

// ------------------------------------------------------------------------------------------------------
// Dequantisers: one thread turns 64 consecutive weights of one row (one k tile) into eight 16-byte chunks of fp16,
// in the (0, 2, 1, 3) order, times the 2^8 prescale.
// ------------------------------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t h2_bits(__half2 v) { return *reinterpret_cast<uint32_t *>(&v); }
__device__ __forceinline__ __half2 bits_h2(uint32_t v) { return *reinterpret_cast<__half2 *>(&v); }

// 6-bit scale and min of sub-block j of a Q4_K super-block (ScaleMinK4, GgufKQuantBlocks.cs:149-153).
__device__ __forceinline__ void q4k_scale_min(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t j, uint32_t &sc, uint32_t &mn)
{
    const uint32_t shift = 8 * (j & 3);
    if (j < 4) {
        sc = (w0 >> shift) & 63;
        mn = (w1 >> shift) & 63;
    } else {
        sc = ((w2 >> shift) & 0xF) | (((w0 >> shift) >> 2) & 0x30);
        mn = (((w2 >> shift) >> 4) & 0xF) | (((w1 >> shift) >> 2) & 0x30);
    }
}

struct GemmArgs;

// 16 bytes through 128-bit loads when the address is 16-byte aligned by construction, through eight 16-bit loads for
// the file layouts whose blocks are only 2-byte aligned.
template <bool ALIGNED>
__device__ __forceinline__ uint4 load16(const uint8_t *p)
{
    if (ALIGNED) {
        return __ldg(reinterpret_cast<const uint4 *>(p));
    }
    uint32_t h[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        h[i] = __ldg(reinterpret_cast<const unsigned short *>(p + 2 * i));
    }
    return make_uint4(h[0] | (h[1] << 16), h[2] | (h[3] << 16), h[4] | (h[5] << 16), h[6] | (h[7] << 16));
}
__device__ __forceinline__ uint32_t load_u16(const uint8_t *p) { return __ldg(reinterpret_cast<const unsigned short *>(p)); }

// Splits eight FP32 weights (times the prescale) into fp16 high and low parts, packed in the (0, 2, 1, 3) order of a chunk.
__device__ __forceinline__ void split_chunk(const float *w, uint4 &high, uint4 &low)
{
    uint32_t h[4], l[4];
#pragma unroll
    for (int pair = 0; pair < 4; ++pair) {
        // values (0, 2), (1, 3), (4, 6), (5, 7)
        const int first = (pair & 1) + 4 * (pair >> 1);
        const float a = w[first] * kPrescale, b = w[first + 2] * kPrescale;
        const __half2 hi = __floats2half2_rn(a, b);
        const float2 back = __half22float2(hi);
        h[pair] = h2_bits(hi);
        l[pair] = h2_bits(__floats2half2_rn(a - back.x, b - back.y));
    }
    high = make_uint4(h[0], h[1], h[2], h[3]);
    low = make_uint4(l[0], l[1], l[2], l[3]);
}

// 128-row tiles give every weight row two dequant threads (`part` 0 and 1), neighbours in a warp. PAIRED loads fetch
// each byte of the row once between the two -- a load instruction of the warp then touches 16 rows' lines instead of
// 32, and the L1 pipeline, not DRAM, is what bounds these thread-per-row loads -- and `share` hands the partner the
// pieces both need (executed by every lane of the warp).
__device__ __forceinline__ uint4 from_partner(uint4 v)
{
    return make_uint4(__shfl_xor_sync(0xffffffffu, v.x, 1), __shfl_xor_sync(0xffffffffu, v.y, 1), __shfl_xor_sync(0xffffffffu, v.z, 1),
                      __shfl_xor_sync(0xffffffffu, v.w, 1));
}

struct DequantQ4K {
    static constexpr int kAhead = 3;  // k steps of raw blocks a dequant thread keeps in flight (12 registers each)
    static constexpr int kStepsPerRaw = 1;
    struct Raw {
        uint4 header, q0, q1;
    };
    struct Row {
        const uint8_t *base;  // the row's first super-block
    };
    static __device__ __forceinline__ Row row_of(const GemmArgs &a, uint64_t row);
    // k tile `kt` is chunk kt%4 of super-block kt/4.
    template <bool PAIRED>
    static __device__ __forceinline__ void load(const Row &r, uint32_t kt, uint32_t part, Raw &raw)
    {
        const uint8_t *block = r.base + (uint64_t)(kt >> 2) * 144;
        raw.header = __ldg(reinterpret_cast<const uint4 *>(block));
        if (PAIRED) {  // both threads expand the same 32 bytes (low and high nibbles): each fetches one half of them
            raw.q0 = __ldg(reinterpret_cast<const uint4 *>(block + 16 + (kt & 3) * 32 + 16 * part));
        } else {
            raw.q0 = __ldg(reinterpret_cast<const uint4 *>(block + 16 + (kt & 3) * 32));
            raw.q1 = __ldg(reinterpret_cast<const uint4 *>(block + 32 + (kt & 3) * 32));
        }
    }
    static __device__ __forceinline__ void share(Raw &raw, uint32_t part)
    {
        const uint4 mine = raw.q0, other = from_partner(raw.q0);
        raw.q0 = part ? other : mine;
        raw.q1 = part ? mine : other;
    }
    // 128-row tiles, fp16 operands: a fetch brings a whole block (four k steps) -- the header and this thread's half of each
    // of the four 32-byte pieces. One burst of 144 contiguous bytes per row and four steps instead of a 48-byte visit per
    // step: with some 19,000 rows being walked at once, every visit finds its DRAM page closed again.
    static constexpr bool kHasWide = true;
    struct WideRaw {
        uint4 header, q[4];
    };
    struct WideFull {
        uint4 header, q[8];  // q[2c], q[2c + 1]: the 32 bytes of k step c
    };
    static __device__ __forceinline__ void load_wide(const Row &r, uint32_t kt, uint32_t part, WideRaw &raw)
    {
        const uint8_t *block = r.base + (uint64_t)(kt >> 2) * 144;
        raw.header = __ldg(reinterpret_cast<const uint4 *>(block));
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            raw.q[c] = __ldg(reinterpret_cast<const uint4 *>(block + 16 + c * 32 + 16 * part));
        }
    }
    static __device__ __forceinline__ void complete_wide(const WideRaw &raw, uint32_t part, WideFull &full)
    {
        full.header = raw.header;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const uint4 other = from_partner(raw.q[c]);
            full.q[2 * c] = part ? other : raw.q[c];
            full.q[2 * c + 1] = part ? raw.q[c] : other;
        }
    }
    // k step `step` (0..3) of the block
    static __device__ __forceinline__ void expand_wide(const WideFull &full, int step, uint32_t half, uint4 (&out)[4])
    {
        Raw one;
        one.header = full.header;
        one.q0 = full.q[2 * step];
        one.q1 = full.q[2 * step + 1];
        expand<true>(one, (uint32_t)step, half, out);
    }
    // Chunks 4*half .. 4*half+3 of the k tile: half 0 = the low nibbles (sub-block 2c), half 1 = the high nibbles
    // (sub-block 2c+1), where c = kt%4.
    template <bool PAIRED>
    static __device__ __forceinline__ void expand(const Raw &raw, uint32_t kt, uint32_t half, uint4 (&out)[4])
    {
        const float d = __half2float(__ushort_as_half((unsigned short)(raw.header.x & 0xffff))) * kPrescale;
        const float dmin = __half2float(__ushort_as_half((unsigned short)(raw.header.x >> 16))) * kPrescale;
        uint32_t sc, mn;
        q4k_scale_min(raw.header.y, raw.header.z, raw.header.w, 2 * (kt & 3) + half, sc, mn);
        // value = (d*sc) * q - dmin*m; the high nibbles are used in place as 16*q, so their scale is divided by 16
        const __half2 a = __float2half2_rn(d * (float)sc * (half ? 0.0625f : 1.0f)), b = __float2half2_rn(-dmin * (float)mn);
        const __half2 k1024 = __float2half2_rn(1024.0f);
        const uint32_t mask = half ? 0x00F000F0u : 0x000F000Fu;
        const uint32_t words[8] = {raw.q0.x, raw.q0.y, raw.q0.z, raw.q0.w, raw.q1.x, raw.q1.y, raw.q1.z, raw.q1.w};
        uint32_t v[16];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            // 0x6400 | n is the fp16 number 1024 + n: exact integers without a conversion instruction
            v[2 * j] = h2_bits(__hfma2(__hsub2(bits_h2((words[j] & mask) | 0x64006400u), k1024), a, b));
            v[2 * j + 1] = h2_bits(__hfma2(__hsub2(bits_h2(((words[j] >> 8) & mask) | 0x64006400u), k1024), a, b));
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            out[c] = make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
        }
    }
    // The same 32 weights in FP32, exactly as the reference decodes them: (d * sc) * q - dmin * m (GgufKQuantBlocks.cs:99-121).
    template <bool PAIRED>
    static __device__ __forceinline__ void expand_f32(const Raw &raw, uint32_t kt, uint32_t half, float (&w)[32])
    {
        const float d = __half2float(__ushort_as_half((unsigned short)(raw.header.x & 0xffff)));
        const float dmin = __half2float(__ushort_as_half((unsigned short)(raw.header.x >> 16)));
        uint32_t sc, mn;
        q4k_scale_min(raw.header.y, raw.header.z, raw.header.w, 2 * (kt & 3) + half, sc, mn);
        const float d1 = __fmul_rn(d, (float)sc), m1 = __fmul_rn(dmin, (float)mn);
        const uint32_t words[8] = {raw.q0.x, raw.q0.y, raw.q0.z, raw.q0.w, raw.q1.x, raw.q1.y, raw.q1.z, raw.q1.w};
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const uint32_t q = (words[i / 4] >> (8 * (i & 3) + 4 * half)) & 0xF;
            w[i] = __fsub_rn(__fmul_rn(d1, (float)q), m1);
        }
    }
};

// Q6_K: k tile kt is quarter kt%4 of super-block kt/4: half h = (kt%4)/2 of the block, nibble g = kt%2 of its 64 ql
// bytes; tile values 0..31 pair ql[l] with bits (4g, 4g+1) of qh[l], values 32..63 pair ql[l+32] with bits (4g+2, 4g+3)
// (GgufKQuantBlocks.cs:155-177). value = d * sc[8h + 4g + i/16] * (q - 32).
template <bool PLANAR>
struct DequantQ6K {
    static constexpr int kAhead = 2;  // 27 registers per fetch
    // The two k tiles of a half block (nibble g = 0, 1) are cut from the same 64 + 32 bytes: one fetch serves both steps,
    // so two fetches in flight are four k steps of lookahead.
    static constexpr int kStepsPerRaw = 2;
    static constexpr bool kHasWide = true;
    struct Raw {
        uint4 ql[4], qh[2];
        uint2 scales;  // the four int8 scales of k tile g = 0, then those of g = 1
        uint32_t d;    // fp16 bits
    };
    struct Row {
        const uint8_t *ql, *qh, *sc, *d;  // planar: per-plane row starts; file layout: all inside one block stream
    };
    static __device__ __forceinline__ Row row_of(const GemmArgs &a, uint64_t row);
    template <bool PAIRED>
    static __device__ __forceinline__ void load(const Row &r, uint32_t kt, uint32_t part, Raw &raw)
    {
        const uint32_t sb = kt >> 2, h = (kt >> 1) & 1;  // (kt is even: the first step of the pair)
        const uint8_t *ql, *qh, *sc, *d;
        if (PLANAR) {
            ql = r.ql + (uint64_t)sb * 128 + h * 64;
            qh = r.qh + (uint64_t)sb * 64 + h * 32;
            sc = r.sc + (uint64_t)sb * 16 + h * 8;
            d = r.d + (uint64_t)sb * 2;
        } else {
            const uint8_t *block = r.ql + (uint64_t)sb * 210;
            ql = block + h * 64;
            qh = block + 128 + h * 32;
            sc = block + 192 + h * 8;
            d = block + 208;
        }
        if (PAIRED) {  // ql[0..1]: the thread's own 32 bytes; qh[0]: its half of the 32 bytes both threads need
            raw.ql[0] = load16<PLANAR>(ql + 32 * part);
            raw.ql[1] = load16<PLANAR>(ql + 32 * part + 16);
            raw.qh[0] = load16<PLANAR>(qh + 16 * part);
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                raw.ql[i] = load16<PLANAR>(ql + 16 * i);
            }
            raw.qh[0] = load16<PLANAR>(qh);
            raw.qh[1] = load16<PLANAR>(qh + 16);
        }
        raw.scales = PLANAR ? __ldg(reinterpret_cast<const uint2 *>(sc))
                            : make_uint2(load_u16(sc) | (load_u16(sc + 2) << 16), load_u16(sc + 4) | (load_u16(sc + 6) << 16));
        raw.d = load_u16(d);
    }
    static __device__ __forceinline__ void share(Raw &raw, uint32_t part)
    {
        const uint4 mine = raw.qh[0], other = from_partner(raw.qh[0]);
        raw.qh[0] = part ? other : mine;
        raw.qh[1] = part ? mine : other;
    }
    // 128-row tiles, fp16 operands: a fetch brings the thread's share of a whole block (four k steps): of each half its own
    // 32 bytes of low nibbles and one 16-byte piece of the high bits, the sixteen scales and d.
    struct WideRaw {
        uint4 ql[4], qh[2], scales;  // ql[2h], ql[2h + 1] and qh[h]: half h
        uint32_t d;
    };
    struct WideFull {
        uint4 ql[4], qh[4], scales;  // qh[2h], qh[2h + 1]: the 32 bytes of half h
        uint32_t d;
    };
    static __device__ __forceinline__ void load_wide(const Row &r, uint32_t kt, uint32_t part, WideRaw &raw)
    {
        const uint32_t sb = kt >> 2;
        const uint8_t *ql, *qh, *sc, *d;
        if (PLANAR) {
            ql = r.ql + (uint64_t)sb * 128;
            qh = r.qh + (uint64_t)sb * 64;
            sc = r.sc + (uint64_t)sb * 16;
            d = r.d + (uint64_t)sb * 2;
        } else {
            const uint8_t *block = r.ql + (uint64_t)sb * 210;
            ql = block;
            qh = block + 128;
            sc = block + 192;
            d = block + 208;
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            raw.ql[2 * h] = load16<PLANAR>(ql + 64 * h + 32 * part);
            raw.ql[2 * h + 1] = load16<PLANAR>(ql + 64 * h + 32 * part + 16);
            raw.qh[h] = load16<PLANAR>(qh + 32 * h + 16 * part);
        }
        raw.scales = load16<PLANAR>(sc);
        raw.d = load_u16(d);
    }
    static __device__ __forceinline__ void complete_wide(const WideRaw &raw, uint32_t part, WideFull &full)
    {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            full.ql[i] = raw.ql[i];
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint4 other = from_partner(raw.qh[h]);
            full.qh[2 * h] = part ? other : raw.qh[h];
            full.qh[2 * h + 1] = part ? raw.qh[h] : other;
        }
        full.scales = raw.scales;
        full.d = raw.d;
    }
    // k step `step` (0..3) of the block: half step / 2, nibble step % 2
    static __device__ __forceinline__ void expand_wide(const WideFull &full, int step, uint32_t part, uint4 (&out)[4])
    {
        const int h = step >> 1;
        Raw one;
        one.ql[0] = full.ql[2 * h];
        one.ql[1] = full.ql[2 * h + 1];
        one.qh[0] = full.qh[2 * h];
        one.qh[1] = full.qh[2 * h + 1];
        one.scales = h ? make_uint2(full.scales.z, full.scales.w) : make_uint2(full.scales.x, full.scales.y);
        one.d = full.d;
        expand<true>(one, (uint32_t)step, part, out);
    }
    // part 0: tile values 0..31 (chunks 0..3), part 1: values 32..63 (chunks 4..7)
    template <bool PAIRED>
    static __device__ __forceinline__ void expand(const Raw &raw, uint32_t kt, uint32_t part, uint4 (&out)[4])
    {
        const uint32_t g = kt & 1;
        const float d = __half2float(__ushort_as_half((unsigned short)raw.d)) * kPrescale;
        const __half2 k1056 = __float2half2_rn(1056.0f);  // 1024 from the exponent trick + the code offset 32
        const uint4 first = PAIRED || !part ? raw.ql[0] : raw.ql[2], second = PAIRED || !part ? raw.ql[1] : raw.ql[3];
        const uint32_t ql[8] = {first.x, first.y, first.z, first.w, second.x, second.y, second.z, second.w};
        const uint32_t qh[8] = {raw.qh[0].x, raw.qh[0].y, raw.qh[0].z, raw.qh[0].w, raw.qh[1].x, raw.qh[1].y, raw.qh[1].z, raw.qh[1].w};
        const uint32_t high_shift = 4 * g + 2 * part;
        uint32_t v[16];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int scale = (int)(signed char)(((g ? raw.scales.y : raw.scales.x) >> (8 * (2 * part + j / 4))) & 0xff);
            const __half2 a = __float2half2_rn(d * (float)scale);
            const uint32_t nibbles = (g ? (ql[j] >> 4) : ql[j]) & 0x0F0F0F0Fu;
            const uint32_t codes = nibbles | (((qh[j] >> high_shift) & 0x03030303u) << 4);
            v[2 * j] = h2_bits(__hmul2(__hsub2(bits_h2((codes & 0x00FF00FFu) | 0x64006400u), k1056), a));
            v[2 * j + 1] = h2_bits(__hmul2(__hsub2(bits_h2(((codes >> 8) & 0x00FF00FFu) | 0x64006400u), k1056), a));
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            out[c] = make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
        }
    }
    // The same 32 weights in FP32 as the reference decodes them: (d * sc) * (q - 32) (GgufKQuantBlocks.cs:155-177).
    template <bool PAIRED>
    static __device__ __forceinline__ void expand_f32(const Raw &raw, uint32_t kt, uint32_t part, float (&w)[32])
    {
        const uint32_t g = kt & 1;
        const float d = __half2float(__ushort_as_half((unsigned short)raw.d));
        const uint4 first = PAIRED || !part ? raw.ql[0] : raw.ql[2], second = PAIRED || !part ? raw.ql[1] : raw.ql[3];
        const uint32_t ql[8] = {first.x, first.y, first.z, first.w, second.x, second.y, second.z, second.w};
        const uint32_t qh[8] = {raw.qh[0].x, raw.qh[0].y, raw.qh[0].z, raw.qh[0].w, raw.qh[1].x, raw.qh[1].y, raw.qh[1].z, raw.qh[1].w};
        const uint32_t high_shift = 4 * g + 2 * part;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const int scale = (int)(signed char)(((g ? raw.scales.y : raw.scales.x) >> (8 * (2 * part + i / 16))) & 0xff);
            const uint32_t byte = (ql[i / 4] >> (8 * (i & 3))) & 0xff;
            const uint32_t nibble = g ? byte >> 4 : byte & 0xF;
            const uint32_t high = (qh[i / 4] >> (8 * (i & 3) + high_shift)) & 3;
            w[i] = __fmul_rn(__fmul_rn(d, (float)scale), (float)((int)(nibble | (high << 4)) - 32));
        }
    }
};

// Q8_0: k tile kt is blocks 2kt and 2kt+1 of the row; value = d * code (GgufLegacyBlocks.cs:85-92).
template <bool PLANAR>
struct DequantQ8 {
    static constexpr int kAhead = 3;
    static constexpr int kStepsPerRaw = 1;
    static constexpr bool kHasWide = false;
    struct Raw {
        uint4 codes[4];
        uint32_t d0, d1;  // fp16 bits of the two block scales
    };
    struct Row {
        const uint8_t *codes, *scales;
    };
    static __device__ __forceinline__ Row row_of(const GemmArgs &a, uint64_t row);
    // (every thread fetches the whole k tile: the file layout's blocks are only 2-byte aligned, and the planar
    // layout's two threads of a row share nothing but the scale word)
    template <bool PAIRED>
    static __device__ __forceinline__ void load(const Row &r, uint32_t kt, uint32_t, Raw &raw)
    {
        if (PLANAR) {
            const uint8_t *codes = r.codes + (uint64_t)kt * 64;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                raw.codes[i] = load16<true>(codes + 16 * i);
            }
            const uint32_t scales = __ldg(reinterpret_cast<const uint32_t *>(r.scales + (uint64_t)kt * 4));
            raw.d0 = scales & 0xffff;
            raw.d1 = scales >> 16;
        } else {
            const uint8_t *block = r.codes + (uint64_t)kt * 68;
            raw.d0 = load_u16(block);
            raw.codes[0] = load16<false>(block + 2);
            raw.codes[1] = load16<false>(block + 18);
            raw.d1 = load_u16(block + 34);
            raw.codes[2] = load16<false>(block + 36);
            raw.codes[3] = load16<false>(block + 52);
        }
    }
    static __device__ __forceinline__ void share(Raw &, uint32_t) {}
    // part 0: the first block (chunks 0..3), part 1: the second (chunks 4..7)
    template <bool PAIRED>
    static __device__ __forceinline__ void expand(const Raw &raw, uint32_t, uint32_t part, uint4 (&out)[4])
    {
        const float d = __half2float(__ushort_as_half((unsigned short)(part ? raw.d1 : raw.d0))) * kPrescale;
        const __half2 a = __float2half2_rn(d);
        const __half2 k1152 = __float2half2_rn(1152.0f);  // 1024 from the exponent trick + the 128 that makes the byte unsigned
        const uint4 lo = part ? raw.codes[2] : raw.codes[0], hi = part ? raw.codes[3] : raw.codes[1];
        const uint32_t words[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        uint32_t v[16];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t biased = words[j] ^ 0x80808080u;
            v[2 * j] = h2_bits(__hmul2(__hsub2(bits_h2((biased & 0x00FF00FFu) | 0x64006400u), k1152), a));
            v[2 * j + 1] = h2_bits(__hmul2(__hsub2(bits_h2(((biased >> 8) & 0x00FF00FFu) | 0x64006400u), k1152), a));
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            out[c] = make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
        }
    }
    // The same 32 weights in FP32: d * code (GgufLegacyBlocks.cs:85-92).
    template <bool PAIRED>
    static __device__ __forceinline__ void expand_f32(const Raw &raw, uint32_t, uint32_t part, float (&w)[32])
    {
        const float d = __half2float(__ushort_as_half((unsigned short)(part ? raw.d1 : raw.d0)));
        const uint4 lo = part ? raw.codes[2] : raw.codes[0], hi = part ? raw.codes[3] : raw.codes[1];
        const uint32_t words[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            w[i] = __fmul_rn(d, (float)(int)(signed char)((words[i / 4] >> (8 * (i & 3))) & 0xff));
        }
    }
};

// ------------------------------------------------------------------------------------------------------
// The GEMM kernel
// ------------------------------------------------------------------------------------------------------

struct GemmArgs {
    const uint8_t *weights;  // file-layout rows, or plane 0 of the planar layout
    const uint8_t *plane1, *plane2, *plane3;
    uint64_t row_bytes;      // of the file layout
    uint64_t columns;
    uint64_t rows, tokens;
    uint32_t k_tiles, row_tiles, token_tiles;
    const uint8_t *x_tiles;      // converted activations
    const uint8_t *x_tiles_low;  // their low parts (two-part fp16 operands), or null
    float *y;
    uint64_t out_stride;
    uint32_t *fault;
    // Products with fewer tiles than half the SMs: the k steps of a tile are dealt to `k_parts` CTAs (`k_per_part` steps
    // each); every CTA leaves its share in `partials`, and the CTA that counts itself in last (`arrivals`, one word per
    // tile, zero before the launch) adds the shares in part order and stores the tile. k_parts = 1: none of that.
    uint32_t k_parts, k_per_part;
    float *partials;
    uint32_t *arrivals;
};

__device__ __forceinline__ DequantQ4K::Row DequantQ4K::row_of(const GemmArgs &a, uint64_t row) { return Row{a.weights + row * a.row_bytes}; }
template <bool PLANAR>
__device__ __forceinline__ typename DequantQ6K<PLANAR>::Row DequantQ6K<PLANAR>::row_of(const GemmArgs &a, uint64_t row)
{
    if (PLANAR) {
        return Row{a.weights + row * (a.columns / 2), a.plane1 + row * (a.columns / 4), a.plane2 + row * (a.columns / 16),
                   a.plane3 + row * (a.columns / 128)};
    }
    return Row{a.weights + row * a.row_bytes, nullptr, nullptr, nullptr};
}
template <bool PLANAR>
__device__ __forceinline__ typename DequantQ8<PLANAR>::Row DequantQ8<PLANAR>::row_of(const GemmArgs &a, uint64_t row)
{
    if (PLANAR) {
        return Row{a.weights + row * a.columns, a.plane1 + row * (a.columns / 16)};
    }
    return Row{a.weights + row * a.row_bytes, nullptr};
}

// SPLIT: both operands are carried as fp16 high + low parts (22 bits) and a k step issues three MMAs, high x high,
// low x high and high x low, into the same accumulator: the result then differs from the FP32-activation product of the
// reference by FP32 accumulation order only. A stage holds A high, A low, B high, B low (16 KB each, N = 128, one token tile).
template <class Dequant, int N, int TT, bool SPLIT = false>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_tc_kernel(GemmArgs a)
{
    static_assert(N == 128 || N == 256, "the weight-row tile is 128 or 256");
    static_assert(TT == 1 || TT == 2, "one or two token tiles per CTA tile");
    static_assert(!SPLIT || (N == 128 && TT == 1), "two-part operands use 128-row tiles and one token tile");
    constexpr uint32_t kTileRows = N;
    constexpr uint32_t kStages = SPLIT ? 3 : stage_count(TT), kStageBytes = SPLIT ? 4 * kTileABytes : stage_bytes(TT);
    constexpr uint32_t kTileBOffset = SPLIT ? 2 * kTileABytes : TT * kTileABytes;  // where the weight tile starts inside a stage
    constexpr uint32_t kBuffers = TT == 1 ? 2 : 1;  // accumulator sets that can be in flight
    extern __shared__ __align__(1024) uint8_t shared_raw[];
    // the dynamic window is only guaranteed 16-byte alignment; the swizzle needs 1024
    uint8_t *stages = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(shared_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t barriers[2 * kMaxStages + 4];  // full[s], empty[s], acc_full[2], acc_empty[2]
    __shared__ uint32_t tmem_slot;
    __shared__ int last_tile;  // the tile whose shares this CTA adds at its end (it was the last to arrive), or -1
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full0 = smem_u32(&barriers[0]), empty0 = smem_u32(&barriers[kMaxStages]);
    const uint32_t acc_full0 = smem_u32(&barriers[2 * kMaxStages]), acc_empty0 = smem_u32(&barriers[2 * kMaxStages + 2]);
    if (threadIdx.x == 0) {
        last_tile = -1;
        for (uint32_t s = 0; s < kStages; ++s) {
            mbar_init(full0 + 8 * s, 1 + kDequantWarps);  // the loader's expect_tx arrival + one arrival per dequant warp
            mbar_init(empty0 + 8 * s, 1);     // tcgen05.commit
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full0 + 8 * b, 1);   // tcgen05.commit
            mbar_init(acc_empty0 + 8 * b, 4);  // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(&tmem_slot)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    const uint32_t token_groups = (a.token_tiles + TT - 1) / TT;  // CTA tiles along the tokens
    const uint32_t tiles = a.row_tiles * token_groups;
    const uint32_t items = tiles * a.k_parts;  // item = part * tiles + tile: k steps [part * k_per_part, + k_per_part) of the tile
    auto first_step = [&](uint32_t item) { return (item / tiles) * a.k_per_part; };
    auto end_step = [&](uint32_t item) { return min(a.k_tiles, (item / tiles + 1) * a.k_per_part); };

    if (warp == kLoaderWarp) {
        // ---- loader: the activation tile of every (tile, k step) --------------------------------------
        if (lane == 0) {
            uint32_t s = 0, round = 0;
            for (uint32_t item = blockIdx.x; item < items; item += gridDim.x) {
                const uint32_t tile = item % tiles;
                const uint64_t tt0 = (tile / a.row_tiles) * TT;
                const uint32_t live = min((uint32_t)TT, a.token_tiles - (uint32_t)tt0);  // token tiles that exist
                for (uint32_t kt = first_step(item), k_end = end_step(item); kt < k_end; ++kt) {
                    if (round > 0) {
                        mbar_wait(empty0 + 8 * s, (round - 1) & 1, a.fault);
                    }
                    mbar_expect_tx(full0 + 8 * s, (SPLIT ? 2 : live) * kTileABytes);
                    for (uint32_t i = 0; i < live; ++i) {
                        bulk_copy(smem_u32(stages + s * kStageBytes + i * kTileABytes), a.x_tiles + ((tt0 + i) * a.k_tiles + kt) * kTileABytes,
                                  kTileABytes, full0 + 8 * s);
                    }
                    if (SPLIT) {
                        bulk_copy(smem_u32(stages + s * kStageBytes + kTileABytes), a.x_tiles_low + (tt0 * a.k_tiles + kt) * kTileABytes, kTileABytes,
                                  full0 + 8 * s);
                    }
                    if (++s == kStages) {
                        s = 0;
                        ++round;
                    }
                }
            }
        }
    } else if (warp == kMmaWarp) {
        // ---- MMA issuer -----------------------------------------------------------------------------------
        if (lane == 0) {
            uint32_t s = 0, phase = 0, local = 0;
            for (uint32_t item = blockIdx.x; item < items; item += gridDim.x, ++local) {
                const uint32_t tile = item % tiles;
                const uint32_t acc = local % kBuffers, use = local / kBuffers;
                const uint32_t live = min((uint32_t)TT, a.token_tiles - (uint32_t)((tile / a.row_tiles) * TT));
                const uint32_t k_begin = first_step(item), k_end = end_step(item);
                if (use >= 1) {
                    mbar_wait(acc_empty0 + 8 * acc, (use - 1) & 1, a.fault);
                }
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + acc * kMaxTileRows;  // token tile i of a TT = 2 tile sits at + i * 256 columns
                for (uint32_t kt = k_begin; kt < k_end; ++kt) {
                    mbar_wait(full0 + 8 * s, phase, a.fault);
                    tc_fence_after();
                    const uint32_t stage = smem_u32(stages + s * kStageBytes);
                    const uint64_t desc_b = smem_desc(stage + kTileBOffset);
                    if (SPLIT) {
                        const uint64_t a_high = smem_desc(stage), a_low = smem_desc(stage + kTileABytes), b_low = smem_desc(stage + kTileBOffset + kTileABytes);
#pragma unroll
                        for (uint32_t k = 0; k < kTileK / 16; ++k) {
                            umma_f16(tmem_d, a_high + 2 * k, desc_b + 2 * k, instr_desc(N), (kt != k_begin || k != 0) ? 1u : 0u);
                            umma_f16(tmem_d, a_low + 2 * k, desc_b + 2 * k, instr_desc(N), 1u);
                            umma_f16(tmem_d, a_high + 2 * k, b_low + 2 * k, instr_desc(N), 1u);
                        }
                    }
#pragma unroll
                    for (uint32_t i = 0; i < (SPLIT ? 0u : (uint32_t)TT); ++i) {
                        if (i < live) {
                            const uint64_t desc_a = smem_desc(stage + i * kTileABytes);
#pragma unroll
                            for (uint32_t k = 0; k < kTileK / 16; ++k) {
                                // 16 fp16 = 32 bytes further along the swizzled row: +2 in the descriptor's 16-byte units
                                umma_f16(tmem_d + i * kMaxTileRows, desc_a + 2 * k, desc_b + 2 * k, instr_desc(N), (kt != k_begin || k != 0) ? 1u : 0u);
                            }
                        }
                    }
                    umma_commit(empty0 + 8 * s);  // the stage is free once these MMAs have read it
                    if (++s == kStages) {
                        s = 0;
                        phase ^= 1;
                    }
                }
                umma_commit(acc_full0 + 8 * acc);  // the accumulator is complete once every MMA above has finished
            }
        }
    } else if (warp >= 4) {
        // ---- dequant warps: 256 threads over the tile's N rows; with N = 128 two threads share a row, one nibble
        // half (four of the eight 16-byte chunks) each. Raw blocks are fetched ahead of their expansion, so the memory
        // latency is off the critical path. Two loops: K-quants with 128-row tiles and fp16 operands fetch a whole
        // block (four k steps) at a time; every other variant fetches one or two k steps at a time, one to three
        // fetches ahead.
        const uint32_t dq = threadIdx.x - 128;
        constexpr uint32_t kParts = 256 / kTileRows;  // threads per row: neighbours in a warp
        constexpr bool kPaired = kParts == 2;
        const uint32_t r = dq / kParts, part = dq % kParts;  // part is 0 when N = 256
        uint32_t s = 0, round = 0;
        // Hands one k step's share of the weight tile (128-row tiles, fp16 operands: chunks 4 * part .. + 3 of row r) to the MMA.
        auto hand_over = [&](const uint4 (&chunks)[4]) {
            if (round > 0) {
                mbar_wait(empty0 + 8 * s, (round - 1) & 1, a.fault);
            }
            uint8_t *tile_b = stages + s * kStageBytes + kTileBOffset;
#pragma unroll
            for (uint32_t c = 0; c < 4; ++c) {
                *reinterpret_cast<uint4 *>(tile_b + swizzled(r, 4 * part + c)) = chunks[c];
            }
            // make the generic-proxy stores visible to the tensor core's (async proxy) reads
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(full0 + 8 * s);
            }
            if (++s == kStages) {
                s = 0;
                ++round;
            }
        };
        if constexpr (Dequant::kHasWide && kPaired && !SPLIT) {
            // ---- whole blocks per fetch (four k steps), one fetch in flight: issued when the block before it is taken up
            uint32_t fetches = 0;
            for (uint32_t item = blockIdx.x; item < items; item += gridDim.x) {
                fetches += (end_step(item) - first_step(item)) / 4;  // (first step and step count of an item are multiples of 4)
            }
            typename Dequant::WideRaw next;
            uint32_t fetch_item = blockIdx.x, fetch_kt = first_step(fetch_item), fetch_end = end_step(fetch_item);
            bool fetch_new_row = true;
            typename Dequant::Row fetch_row{};
            auto fetch = [&]() {
                if (fetch_new_row) {
                    fetch_row = Dequant::row_of(a, min((uint64_t)(((fetch_item % tiles) % a.row_tiles) * kTileRows + r), a.rows - 1));
                    fetch_new_row = false;
                }
                Dequant::load_wide(fetch_row, fetch_kt, part, next);
                fetch_kt += 4;
                if (fetch_kt == fetch_end) {
                    fetch_item += gridDim.x;
                    fetch_kt = first_step(fetch_item);
                    fetch_end = end_step(fetch_item);
                    fetch_new_row = true;
                }
            };
            if (fetches > 0) {
                fetch();
            }
            for (uint32_t n = 0; n < fetches; ++n) {
                const typename Dequant::WideRaw taken = next;
                if (n + 1 < fetches) {
                    fetch();
                }
                typename Dequant::WideFull block;
                Dequant::complete_wide(taken, part, block);
#pragma unroll
                for (int step = 0; step < 4; step += 2) {
                    uint4 both[2][4];  // two independent chains of arithmetic before either is handed over
                    Dequant::expand_wide(block, step, part, both[0]);
                    Dequant::expand_wide(block, step + 1, part, both[1]);
                    hand_over(both[0]);
                    hand_over(both[1]);
                }
            }
        } else {
        // fetches in flight (two-part operands expand to FP32 and have no registers to spare: one fetch of two steps)
        constexpr int kAhead = (SPLIT || N == 256) && Dequant::kStepsPerRaw == 2 ? 1 : Dequant::kAhead;
        constexpr uint32_t kSpan = Dequant::kStepsPerRaw;  // k steps one fetch serves (an item's first step and its step count are multiples of it)
        uint32_t fetches = 0;  // over all of this CTA's items
        for (uint32_t item = blockIdx.x; item < items; item += gridDim.x) {
            fetches += (end_step(item) - first_step(item)) / kSpan;
        }
        // The raw blocks of the next kAhead k steps (across tile boundaries) are fetched before the current ones are
        // expanded: with one token tile a k step is shorter than an L2 round trip, and one step of lookahead left the
        // dequantisers waiting for memory on every step.
        typename Dequant::Raw ahead[kAhead];
        uint32_t fetch_item = blockIdx.x;
        uint32_t fetch_kt = first_step(fetch_item), fetch_end = end_step(fetch_item);
        bool fetch_new_row = true;
        uint32_t fetched = 0;
        typename Dequant::Row fetch_row{};
        auto fetch = [&](typename Dequant::Raw &destination) {
            if (fetch_new_row) {
                fetch_row = Dequant::row_of(a, min((uint64_t)(((fetch_item % tiles) % a.row_tiles) * kTileRows + r), a.rows - 1));
                fetch_new_row = false;
            }
            Dequant::template load<kPaired>(fetch_row, fetch_kt, part, destination);
            fetch_kt += kSpan;
            if (fetch_kt == fetch_end) {
                fetch_item += gridDim.x;
                fetch_kt = first_step(fetch_item);
                fetch_end = end_step(fetch_item);
                fetch_new_row = true;
            }
            ++fetched;
        };
#pragma unroll
        for (int d = 0; d < kAhead; ++d) {
            if (fetched < fetches) {
                fetch(ahead[d]);
            }
        }
        uint32_t item = blockIdx.x;
        uint32_t kt = first_step(item), kt_end = end_step(item);
        for (uint32_t fetch0 = 0; fetch0 < fetches; fetch0 += kAhead) {
#pragma unroll
            for (int d = 0; d < kAhead; ++d) {
                if (fetch0 + d >= fetches) {
                    break;
                }
                typename Dequant::Raw raw = ahead[d];
                if (fetched < fetches) {
                    fetch(ahead[d]);
                }
                if (kPaired) {
                    Dequant::share(raw, part);
                }
                if constexpr (kSpan == 2 && kPaired && !SPLIT) {
                    // Both steps of the fetch are expanded before either is handed over: two independent chains of
                    // arithmetic for a warp that shares its scheduler with one other dequant warp.
                    uint4 both[2][4];
                    Dequant::template expand<true>(raw, kt, part, both[0]);
                    Dequant::template expand<true>(raw, kt + 1, part, both[1]);
                    hand_over(both[0]);
                    hand_over(both[1]);
                    kt += 2;
                } else
#pragma unroll 1
                for (uint32_t span = 0; span < kSpan; ++span) {
                    uint4 v[2][4];
                    if (SPLIT) {
                        float w[32];
                        Dequant::template expand_f32<kPaired>(raw, kt, part, w);
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            split_chunk(w + 8 * c, v[0][c], v[1][c]);
                        }
                    } else if (kParts == 1) {
                        Dequant::template expand<kPaired>(raw, kt, 0, v[0]);
                        Dequant::template expand<kPaired>(raw, kt, 1, v[1]);
                    } else {
                        Dequant::template expand<kPaired>(raw, kt, part, v[0]);
                    }
                    if (round > 0) {
                        mbar_wait(empty0 + 8 * s, (round - 1) & 1, a.fault);
                    }
                    uint8_t *tile_b = stages + s * kStageBytes + kTileBOffset;
#pragma unroll
                    for (uint32_t c = 0; c < 4; ++c) {
                        if (SPLIT) {
                            *reinterpret_cast<uint4 *>(tile_b + swizzled(r, 4 * part + c)) = v[0][c];
                            *reinterpret_cast<uint4 *>(tile_b + kTileABytes + swizzled(r, 4 * part + c)) = v[1][c];
                        } else if (kParts == 1) {
                            *reinterpret_cast<uint4 *>(tile_b + swizzled(r, c)) = v[0][c];
                            *reinterpret_cast<uint4 *>(tile_b + swizzled(r, 4 + c)) = v[1][c];
                        } else {
                            *reinterpret_cast<uint4 *>(tile_b + swizzled(r, 4 * part + c)) = v[0][c];
                        }
                    }
                    // make the generic-proxy stores visible to the tensor core's (async proxy) reads
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(full0 + 8 * s);
                    }
                    if (++s == kStages) {
                        s = 0;
                        ++round;
                    }
                    ++kt;
                }
                if (kt == kt_end) {
                    item += gridDim.x;
                    kt = first_step(item);
                    kt_end = end_step(item);
                }
            }
        }
        }
    } else {
        // ---- epilogue warps: warp q owns accumulator lanes (tokens) 32q .. 32q+31 ----------------------
        uint32_t local = 0;
        const bool whole = a.k_parts == 1;  // the accumulator is the result (else: this CTA's share of it)
        for (uint32_t item = blockIdx.x; item < items; item += gridDim.x, ++local) {
            const uint32_t tile = item % tiles;
            const uint32_t acc = local % kBuffers, use = local / kBuffers;
            const uint64_t row0 = (tile % a.row_tiles) * kTileRows;
            const uint64_t tt0 = (tile / a.row_tiles) * TT;
            const uint32_t live = min((uint32_t)TT, a.token_tiles - (uint32_t)tt0);
            mbar_wait(acc_full0 + 8 * acc, use & 1, a.fault);
            tc_fence_after();
            for (uint32_t i = 0; i < live; ++i) {
                const uint64_t token = (tt0 + i) * kTileTokens + warp * 32 + lane;
                float *destination = whole ? a.y + token * a.out_stride + row0
                                           : a.partials + ((item * TT + i) * kTileTokens + warp * 32 + lane) * kTileRows;
#pragma unroll 1
                for (uint32_t c = 0; c < kTileRows / 32; ++c) {
                    uint32_t v[32];
                    tmem_load32(tmem_base + ((warp * 32) << 16) + (acc + i) * kMaxTileRows + c * 32, v);
                    if (!whole || (token < a.tokens && row0 + c * 32 + 32 <= a.rows && ((reinterpret_cast<uintptr_t>(destination) & 15) == 0))) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            reinterpret_cast<float4 *>(destination + c * 32)[j] =
                                make_float4(__uint_as_float(v[4 * j]) * (1.0f / kPrescale), __uint_as_float(v[4 * j + 1]) * (1.0f / kPrescale),
                                            __uint_as_float(v[4 * j + 2]) * (1.0f / kPrescale), __uint_as_float(v[4 * j + 3]) * (1.0f / kPrescale));
                        }
                    } else if (token < a.tokens) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            if (row0 + c * 32 + j < a.rows) {
                                destination[c * 32 + j] = __uint_as_float(v[j]) * (1.0f / kPrescale);
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(acc_empty0 + 8 * acc);
            }
            if (!whole) {
                // The tile's parts meet through a counter: the CTA that arrives last adds all shares (below, with all of its
                // warps) and stores the tile. Nobody waits for anybody. (A split product gives every CTA exactly one item.)
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (threadIdx.x == 0 && atomicAdd(a.arrivals + tile, 1u) + 1 == a.k_parts) {
                    last_tile = (int)tile;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
    }
    if (a.k_parts > 1 && last_tile >= 0) {
        // The shares of the tile, part 0 first. Every thread of the CTA takes outputs (of 4 floats) eight at a time and two
        // shares per round of loads: what bounds this is the number of L2 round trips in a row, not the bytes.
        __threadfence();
        const uint32_t tile = (uint32_t)last_tile;
        const uint64_t row0 = (uint64_t)(tile % a.row_tiles) * kTileRows;
        const uint64_t tt0 = (uint64_t)(tile / a.row_tiles) * TT;
        const uint32_t live = min((uint32_t)TT, a.token_tiles - (uint32_t)tt0);
        constexpr uint32_t kShareFloats = TT * kTileTokens * kTileRows;
        constexpr uint32_t kBatch = 8;
        const uint32_t quads = live * kTileTokens * kTileRows / 4;
        for (uint32_t f0 = threadIdx.x; f0 < quads; f0 += kGemmThreads * kBatch) {
            float4 sum[kBatch];
#pragma unroll
            for (uint32_t j = 0; j < kBatch; ++j) {
                const uint32_t f = min(f0 + kGemmThreads * j, quads - 1);
                sum[j] = __ldcg(reinterpret_cast<const float4 *>(a.partials + tile * kShareFloats) + f);
            }
#pragma unroll 2
            for (uint32_t part = 1; part < a.k_parts; ++part) {
                const float4 *share = reinterpret_cast<const float4 *>(a.partials + (part * tiles + tile) * kShareFloats);
                float4 v[kBatch];
#pragma unroll
                for (uint32_t j = 0; j < kBatch; ++j) {
                    v[j] = __ldcg(share + min(f0 + kGemmThreads * j, quads - 1));
                }
#pragma unroll
                for (uint32_t j = 0; j < kBatch; ++j) {
                    sum[j].x += v[j].x;
                    sum[j].y += v[j].y;
                    sum[j].z += v[j].z;
                    sum[j].w += v[j].w;
                }
            }
#pragma unroll
            for (uint32_t j = 0; j < kBatch; ++j) {
                const uint32_t f = f0 + kGemmThreads * j;
                const uint32_t column = (4 * f) % kTileRows;
                const uint64_t token = tt0 * kTileTokens + (4 * f) / kTileRows;
                if (f < quads && token < a.tokens) {
                    float *out = a.y + token * a.out_stride + row0 + column;
                    if (row0 + column + 4 <= a.rows && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
                        *reinterpret_cast<float4 *>(out) = sum[j];
                    } else {
                        const float values[4] = {sum[j].x, sum[j].y, sum[j].z, sum[j].w};
                        for (int e = 0; e < 4; ++e) {
                            if (row0 + column + e < a.rows) {
                                out[e] = values[e];
                            }
                        }
                    }
                }
            }
        }
    }
}

constexpr uint32_t kGemmSharedBytes = 4 * stage_bytes(1) + 1024;  // = 3 * stage_bytes(2) + 1024
static_assert(4 * stage_bytes(1) == 3 * stage_bytes(2), "both tile shapes use the same shared-memory budget");

template <class Dequant, int N, int TT, bool SPLIT = false>
cudaError_t run_gemm_shape(const GemmArgs &a, uint64_t ctas, cudaStream_t stream)
{
    // the shared-memory limit of a kernel is a per-device attribute: set it once on every device the library meets
    static std::atomic<uint64_t> configured{0};
    int device = 0;
    cudaGetDevice(&device);
    const uint64_t bit = 1ull << (device & 63);
    if ((configured.load() & bit) == 0) {
        cudaError_t error = cudaFuncSetAttribute(gemm_tc_kernel<Dequant, N, TT, SPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGemmSharedBytes);
        if (error != cudaSuccess) {
            return error;
        }
        configured.fetch_or(bit);
    }
    gemm_tc_kernel<Dequant, N, TT, SPLIT><<<(unsigned)ctas, kGemmThreads, kGemmSharedBytes, stream>>>(a);
    return cudaGetLastError();
}

template <class Dequant>
cudaError_t run_gemm(const GemmArgs &a, int n, int tt, uint64_t ctas, cudaStream_t stream)
{
    if (a.x_tiles_low) {
        return run_gemm_shape<Dequant, 128, 1, true>(a, ctas, stream);
    }
    if (tt == 2) {
        return n == 256 ? run_gemm_shape<Dequant, 256, 2>(a, ctas, stream) : run_gemm_shape<Dequant, 128, 2>(a, ctas, stream);
    }
    return n == 256 ? run_gemm_shape<Dequant, 256, 1>(a, ctas, stream) : run_gemm_shape<Dequant, 128, 1>(a, ctas, stream);
}

}  // namespace

// Scratch of a product whose k steps are dealt to several CTAs: at most kMaxShares shares of a 128-row tile with up to two
// token tiles (one per CTA, and there are no more CTAs than SMs), then one arrival counter per tile.
constexpr uint64_t kMaxShares = 160;
constexpr uint64_t kShareBytes = 2ull * kTileTokens * 128 * sizeof(float);
constexpr uint64_t kArrivalWords = kMaxShares / 2;
constexpr uint64_t kPartsBytes = kMaxShares * kShareBytes + 4 * kArrivalWords;

static uint64_t activation_tile_bytes(uint64_t tokens, uint64_t columns)
{
    const uint64_t token_tiles = (tokens + kTileTokens - 1) / kTileTokens;
    const uint64_t k_tiles = (columns + kTileK - 1) / kTileK;
    return 2 * align_up(token_tiles * k_tiles * kTileABytes, 256);  // room for the low parts of two-part operands
}

uint64_t gemm_scratch_bytes(uint64_t tokens, uint64_t columns)
{
    return activation_tile_bytes(tokens, columns) + kPartsBytes;
}

int32_t launch_gemm(const syn_b200_matrix *m, const float *x, uint64_t tokens, uint64_t in_stride, float *y, uint64_t out_stride,
                    uint32_t precision, void *scratch, uint64_t scratch_bytes, cudaStream_t stream)
{
    if (precision != SYN_B200_GEMM_F16 && precision != SYN_B200_GEMM_F16X2) {
        return fail(SYN_B200_INVALID_ARGUMENT, "unknown tensor-core precision " + std::to_string(precision));
    }
    const bool split = precision == SYN_B200_GEMM_F16X2;
    if (in_stride < m->columns || in_stride % 4 != 0 || (reinterpret_cast<uintptr_t>(x) & 15)) {
        return fail(SYN_B200_INVALID_ARGUMENT, "device activations must be 16-byte aligned with a stride that covers the row and is a multiple of 4 floats");
    }
    if (m->columns % kTileK != 0) {
        return fail(SYN_B200_UNAVAILABLE, "the tensor-core product needs a row length that is a multiple of 64; this matrix has " + std::to_string(m->columns));
    }
    // (a caller that brings the activation tiles' room only gets the product without the split along k)
    const uint64_t need = activation_tile_bytes(tokens, m->columns);
    if (!scratch || scratch_bytes < need || (reinterpret_cast<uintptr_t>(scratch) & 255)) {
        return fail(SYN_B200_INVALID_ARGUMENT, "tensor-core scratch must be 256-byte aligned and hold " + std::to_string(need) + " bytes (" +
                                                   std::to_string(need + kPartsBytes) + " for products that split along k)");
    }
    GemmArgs a{};
    const bool planar = m->layout == Layout::Planar;
    a.weights = m->data + (planar ? m->planes.p0 : 0);
    a.plane1 = m->data + m->planes.p1;
    a.plane2 = m->data + m->planes.p2;
    a.plane3 = m->data + m->planes.p3;
    a.row_bytes = m->row_bytes;
    a.columns = m->columns;
    a.rows = m->rows;
    a.tokens = tokens;
    a.k_tiles = (uint32_t)(m->columns / kTileK);
    a.token_tiles = (uint32_t)((tokens + kTileTokens - 1) / kTileTokens);
    // Two token tiles per CTA tile when there are at least two (a weight tile is then dequantised once per 256
    // tokens); 256-row tiles unless that leaves SMs without a tile and 128-row tiles would not.
    const uint64_t sms = (uint64_t)sm_count(m->device);
    const int tt = a.token_tiles >= 2 && !split ? 2 : 1;
    const uint64_t token_groups = (a.token_tiles + tt - 1) / tt;
    // 256-row tiles when they give every SM work, and also when they fill fewer SMs but in fewer waves: a k step of a
    // 256-row tile takes about 1.7 times that of a 128-row tile (112 tiles of 256 rows in one wave beat 224 of 128 in two).
    const uint64_t tiles256 = ((m->rows + 255) / 256) * token_groups, tiles128 = ((m->rows + 127) / 128) * token_groups;
    const uint64_t waves256 = (tiles256 + sms - 1) / sms, waves128 = (tiles128 + sms - 1) / sms;
    const int n = !split && (tiles256 >= sms || 17 * waves256 < 10 * waves128) ? 256 : 128;
    a.row_tiles = (uint32_t)((m->rows + n - 1) / n);
    a.x_tiles = static_cast<const uint8_t *>(scratch);
    a.x_tiles_low = split ? a.x_tiles + need / 2 : nullptr;
    a.y = y;
    a.out_stride = out_stride;
    a.fault = fault_word_device();
    // Fewer tiles than half the SMs (few weight rows, few tokens): deal every tile's k steps to as many CTAs as there are
    // SMs per tile, no fewer than eight steps each. The shares are added in part order, so the result does not depend on
    // which CTA finishes when.
    const uint64_t tiles = (uint64_t)a.row_tiles * token_groups;
    a.k_parts = 1;
    a.k_per_part = a.k_tiles;
    if (n == 128 && 2 * tiles <= sms && sms <= kMaxShares && tiles <= kArrivalWords && scratch_bytes >= need + kPartsBytes) {
        uint64_t parts = sms / tiles;
        if (parts > a.k_tiles / 8) {
            parts = a.k_tiles / 8;
        }
        if (parts >= 2) {
            a.k_per_part = (uint32_t)((a.k_tiles + parts - 1) / parts + 3) & ~3u;  // whole Q6_K half blocks (pairs of steps share a fetch)
            a.k_parts = (a.k_tiles + a.k_per_part - 1) / a.k_per_part;  // (no empty parts)
            a.partials = reinterpret_cast<float *>(static_cast<uint8_t *>(scratch) + need);
            a.arrivals = reinterpret_cast<uint32_t *>(static_cast<uint8_t *>(scratch) + need + kMaxShares * kShareBytes);
        }
    }

    const uint64_t chunks = (uint64_t)a.token_tiles * a.k_tiles * kTileTokens * 8;
    uint64_t blocks = (chunks + 255) / 256;
    if (blocks > sms * 16) {
        blocks = sms * 16;
    }
    convert_activations_kernel<<<(unsigned)blocks, 256, 0, stream>>>(x, tokens, in_stride, a.k_tiles, a.token_tiles, static_cast<uint8_t *>(scratch),
                                                                   split ? static_cast<uint8_t *>(scratch) + need / 2 : nullptr, a.arrivals,
                                                                   a.k_parts > 1 ? (uint32_t)kArrivalWords : 0u);
    count_launch();
    cudaError_t error = cudaGetLastError();
    if (error != cudaSuccess) {
        return cuda_fail(error, "launching the activation conversion");
    }
    uint64_t ctas = tiles * a.k_parts;
    if (ctas > sms) {
        ctas = sms;
    }
    if (m->type == kQ4_K) {
        error = run_gemm<DequantQ4K>(a, n, tt, ctas, stream);
    } else if (m->type == kQ6_K) {
        error = planar ? run_gemm<DequantQ6K<true>>(a, n, tt, ctas, stream) : run_gemm<DequantQ6K<false>>(a, n, tt, ctas, stream);
    } else {
        error = planar ? run_gemm<DequantQ8<true>>(a, n, tt, ctas, stream) : run_gemm<DequantQ8<false>>(a, n, tt, ctas, stream);
    }
    if (error != cudaSuccess) {
        return cuda_fail(error, "configuring or launching the tensor-core kernel");
    }
    count_launch();
    return SYN_B200_OK;
}

}  // namespace syn
