// Decode matrix-vector kernels for Q8_0, Q4_K and Q6_K weights (sm_100a). These are HBM-bound: every
// weight byte is read once with 128-bit loads, unpacked in registers and reduced with warp shuffles.
//
// Geometry shared by all kernels: a warp owns R consecutive output rows and walks the row in "units"
// (16 or 64 weights per lane per step, chosen so one lane reads whole 16-byte pieces); the T tokens of a
// launch group share every weight load (the reference's matvec_{1,2,4,8}, cuda/kernels/matmul.cu:79-115).
// The grid is persistent: a multiple of the SM count, each warp striding over row groups.
//
// Contracts:
//   XQ8  - activations already quantised to Q8_0 codes (+ per-32 scale, + per-16 code sums). Block dots are
//          exact integers (dp4a); scale products and the cross-block sum are FP32, as in
//          native/synapse-kernels/src/Features/CpuKernels/scalar.rs:29-47 for Q8_0. For Q4_K / Q6_K the
//          sub-block sums are sum(q*a) and sum(a) per 32, resp. sum((q-32)*a) per 16.
//   XF32 - FP32 activations times exactly dequantised weights, the `reference` backend's result
//          (GraphExecution/Q8Operators.cs:75-96, GraphExecution/DecodedRowOperators.cs:29-40) up to FP32
//          summation order.
#pragma once
#include "common.cuh"

namespace syn {
namespace mv {

constexpr int kWarps = 8;  // consumer warps of the ordinary CTA
constexpr unsigned kFull = 0xffffffffu;

__device__ __forceinline__ uint4 ld_stream(const void *p)
{
    // Weights are read exactly once: keep them out of L1 so the activations stay resident there.
    uint4 v;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 ld_cached(const void *p) { return __ldg(reinterpret_cast<const uint4 *>(p)); }
__device__ __forceinline__ uint32_t ld_u16(const void *p) { return __ldg(reinterpret_cast<const unsigned short *>(p)); }
__device__ __forceinline__ float half_bits_to_float(uint32_t bits) { return __half2float(__ushort_as_half((unsigned short)bits)); }

// Where a kernel reads its weights from: global memory directly, or a shared-memory stage filled by bulk copies.
// Where byte `offset` of the quantised activation codes lives in shared memory. Piece p (16 bytes) of line l (128
// bytes) is stored at piece p ^ g(l), g(l) = 2 * (l % 4) + (l / 4) % 2: a permutation of the eight pieces for any eight
// consecutive lines (Q4_K: lane u reads piece i of line u) that also separates the piece pairs {2q, 2q+1} of four
// consecutive lines (Q6_K: lanes 2m, 2m+1 read pieces 2q, 2q+1 of line m). The code array must start on a 128-byte
// boundary.
__host__ __device__ __forceinline__ uint32_t swizzled_code_offset(uint32_t offset)
{
    const uint32_t line = offset >> 7;
    const uint32_t g = ((line & 3u) << 1) | ((line >> 2) & 1u);
    return offset ^ (g << 4);
}

template <class P>
struct WeightViewT;
struct GlobalMem {
    using View = WeightViewT<const uint8_t *>;
    using pointer = const uint8_t *;
    using index = uint64_t;
    static __device__ __forceinline__ uint4 v4(const void *p) { return ld_stream(p); }
    static __device__ __forceinline__ uint4 v4c(const void *p) { return ld_cached(p); }
    // 16 activation codes at byte `offset` of the code array (a multiple of 16)
    static __device__ __forceinline__ uint4 code16(const uint8_t *codes, uint64_t offset) { return ld_cached(codes + offset); }
    static __device__ __forceinline__ uint2 v2(const void *p) { return __ldg(reinterpret_cast<const uint2 *>(p)); }
    static __device__ __forceinline__ uint32_t u16(const void *p) { return ld_u16(p); }
    static __device__ __forceinline__ float f1(const void *p) { return __ldg(reinterpret_cast<const float *>(p)); }
    static __device__ __forceinline__ float2 f2(const void *p) { return __ldg(reinterpret_cast<const float2 *>(p)); }
    static __device__ __forceinline__ float4 f4(const void *p) { return __ldg(reinterpret_cast<const float4 *>(p)); }
};
struct SharedMem {
    using View = WeightViewT<uint32_t>;
    using pointer = uint32_t;  // address inside the shared-memory window
    using index = uint32_t;
    static __device__ __forceinline__ uint4 v4(uint32_t p)
    {
        uint4 v;
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(p));
        return v;
    }
    static __device__ __forceinline__ uint4 v4c(uint32_t p) { return v4(p); }
    // Activation codes in shared memory are stored with the 16-byte pieces of every 128-byte line permuted (see
    // swizzled_code_offset): a lane reads pieces 128 bytes (Q4_K) or 32 bytes (Q6_K) apart from its neighbours, which
    // would otherwise all fall into the same banks (an eight-way conflict on every load).
    static __device__ __forceinline__ uint4 code16(uint32_t codes, uint32_t offset) { return v4(codes + swizzled_code_offset(offset)); }
    static __device__ __forceinline__ uint2 v2(uint32_t p)
    {
        uint2 v;
        asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(p));
        return v;
    }
    static __device__ __forceinline__ uint32_t u16(uint32_t p)
    {
        unsigned short v;
        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(p));
        return v;
    }
    static __device__ __forceinline__ float f1(uint32_t p)
    {
        float v;
        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(p));
        return v;
    }
    static __device__ __forceinline__ float2 f2(uint32_t p)
    {
        float2 v;
        asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(p));
        return v;
    }
    static __device__ __forceinline__ float4 f4(uint32_t p)
    {
        float4 v;
        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(p));
        return v;
    }
};

// Quantised activations as byte addresses in the memory space M reads from:
// codes int8 [T][K], scales float [T][K/32], 16-value code sums int16 [T][K/16].
template <class P>
struct ActPtrT {
    P codes, scales, sums;
};
using ActGlobal = ActPtrT<const uint8_t *>;
using ActShared = ActPtrT<uint32_t>;
__device__ __forceinline__ ActGlobal act_global(const ActView &a)
{
    return ActGlobal{reinterpret_cast<const uint8_t *>(a.codes), reinterpret_cast<const uint8_t *>(a.scales),
                     reinterpret_cast<const uint8_t *>(a.sums)};
}

// 16 bytes from an address that is only 2-byte aligned (file-layout Q8_0 and Q6_K blocks).
template <class M>
__device__ __forceinline__ uint4 ld_unaligned16(typename M::pointer p)
{
    uint32_t h[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        h[i] = M::u16(p + 2 * i);
    }
    return make_uint4(h[0] | (h[1] << 16), h[2] | (h[3] << 16), h[4] | (h[5] << 16), h[6] | (h[7] << 16));
}

__device__ __forceinline__ int dot16(const uint4 &w, const uint4 &a, int acc)
{
    acc = __dp4a((int)w.x, (int)a.x, acc);
    acc = __dp4a((int)w.y, (int)a.y, acc);
    acc = __dp4a((int)w.z, (int)a.z, acc);
    acc = __dp4a((int)w.w, (int)a.w, acc);
    return acc;
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        v += __shfl_xor_sync(kFull, v, offset);
    }
    return v;
}

// 6-bit (scale, min) of sub-blocks 2p and 2p+1 of a Q4_K super-block from its 12 packed bytes (three words).
// Same bit selection as ScaleMinK4 (ModelPackages/SourceFormats/GgufKQuantBlocks.cs:149-153).
__device__ __forceinline__ void q4k_scales(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t p, uint32_t &sc0,
                                           uint32_t &m0, uint32_t &sc1, uint32_t &m1)
{
    const uint32_t shift = 16 * (p & 1);
    const uint32_t t0 = w0 >> shift, t1 = w1 >> shift, t2 = w2 >> shift;
    if (p < 2) {
        sc0 = t0 & 63;
        sc1 = (t0 >> 8) & 63;
        m0 = t1 & 63;
        m1 = (t1 >> 8) & 63;
    } else {
        sc0 = (t2 & 0xF) | ((t0 >> 2) & 0x30);
        sc1 = ((t2 >> 8) & 0xF) | ((t0 >> 10) & 0x30);
        m0 = ((t2 >> 4) & 0xF) | ((t1 >> 2) & 0x30);
        m1 = ((t2 >> 12) & 0xF) | ((t1 >> 10) & 0x30);
    }
}

// Four 6-bit code words (values 0..63, one per byte) from 4 bytes of ql (A, B = ql[l], ql[l+32]) and qh (H):
// the four value groups of GgufKQuantBlocks.cs:166-173 before the -32 offset.
__device__ __forceinline__ void q6k_codes(uint32_t a, uint32_t b, uint32_t h, uint32_t &v1, uint32_t &v2, uint32_t &v3,
                                          uint32_t &v4)
{
    v1 = (a & 0x0F0F0F0Fu) | ((h << 4) & 0x30303030u);
    v2 = (b & 0x0F0F0F0Fu) | ((h << 2) & 0x30303030u);
    v3 = ((a >> 4) & 0x0F0F0F0Fu) | (h & 0x30303030u);
    v4 = ((b >> 4) & 0x0F0F0F0Fu) | ((h >> 2) & 0x30303030u);
}

// Applies the epilogue to one finished dot product and stores it.
// GATHER: also store the result into the peer copies of the output (row-sharded products). It is a template
// parameter because even a never-taken peer branch in the epilogue cost the single-GPU kernels 2-4 %.
template <bool GATHER = false>
__device__ __forceinline__ void store_result(const Epilogue &e, float *__restrict__ y, uint64_t token, uint64_t out_stride, uint64_t row, float v)
{
    if (e.bias) {
        v += __ldg(e.bias + row);
    }
    if (e.gate) {
        const float g = __ldg(e.gate + token * e.gate_stride + row);
        v = g / (1.0f + expf(-g)) * v;
    }
    float *destination = y + token * out_stride + row;
    v = e.accumulate ? *destination + v : v;
    *destination = v;
    // plain stores over NVLink into the peers' copies; constant indices, so the epilogue stays in the parameter bank
    if (GATHER) {
#pragma unroll
        for (int peer = 0; peer < 7; ++peer) {
            if ((uint32_t)peer < e.peer_count) {
                e.peers[peer][token * out_stride + row] = v;
            }
        }
    }
}

// Called by ONE thread of every CTA of a row-sharded product after a CTA barrier behind the CTA's last store. The
// thread publishes the CTA's stores (its own and, through the barrier, its CTA's; the fence is cumulative) and counts the
// CTA in; the thread that counts the last CTA of the grid in has thereby observed every other CTA's count, so after one
// more fence its writes of the launch's sequence number to the signal words are ordered behind ALL stores of the launch,
// at system scope: whoever acquires a signal word sees the whole slice.
__device__ __forceinline__ void signal_completion(const Epilogue &e)
{
    if (e.signal_count == 0) {
        return;
    }
    __threadfence_system();
    const uint32_t total = gridDim.x * gridDim.y;
    if (atomicAdd(e.arrivals, 1u) + 1 == total) {
        atomicExch(e.arrivals, 0u);  // ready for the next launch (launches that share these words are stream-ordered)
        const uint32_t sequence = atomicAdd(e.arrivals + 1, 1u) + 1;
        __threadfence_system();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if ((uint32_t)i < e.signal_count) {
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(e.signals[i]), "r"(sequence) : "memory");
            }
        }
    }
}

__device__ __forceinline__ uint32_t word_of(const uint4 &v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

// Exact integer-to-float conversions on the FMA pipe (a PRMT or IADD plus one FADD) instead of I2F, which runs on the
// quarter-rate XU pipe: 2^23 + n is exactly representable for 0 <= n < 2^23, and 1.5 * 2^23 + n for |n| < 2^22.
__device__ __forceinline__ float byte_to_float(uint32_t word, int index)
{
    return __int_as_float((int)__byte_perm(word, 0x4B000000u, 0x7650 + index)) - 8388608.0f;
}
__device__ __forceinline__ float small_int_to_float(int n)  // |n| < 2^22
{
    return __int_as_float(0x4B400000 + n) - 12582912.0f;
}

// ------------------------------------------------------------------------------------------------------
// Weight views
// ------------------------------------------------------------------------------------------------------

template <class P>
struct WeightViewT {
    P p0, p1, p2, p3;    // plane (or file-layout) bases, already offset to the first row of the call
    uint32_t row_bytes;  // of the file layout
};
using WeightView = WeightViewT<const uint8_t *>;  // global memory
using SharedView = WeightViewT<uint32_t>;         // shared-memory window addresses

// ------------------------------------------------------------------------------------------------------
// XQ8 formats. Each provides: units(K); struct Act; struct W; load_act; load_w; dot (updates acc, optionally
// writes the integer sub-block sums of the unit to `dump`, which points at this (token,row)'s group array).
// ------------------------------------------------------------------------------------------------------

struct Q8PlanarXq8 {
    struct Act { uint4 c; float d; };
    struct W { uint4 c; float d; };
    static constexpr int kPlanes = 2;
    // Several tokens: the 16-weight units make a team per token no faster than the direct-load kernels (measured on
    // 18944x3584: 74 against 52 us at eight tokens), which therefore keep these launches.
    static constexpr bool kTokenTeams = false;
    static void plane_row_bytes(uint64_t K, uint64_t, uint32_t *out) { out[0] = (uint32_t)K; out[1] = (uint32_t)(K / 16); }
    static constexpr int kMaxUpl = 2, kRows = 2, kCtasPerSm = 2;
    static constexpr int min_ctas(int) { return 2; }
    static constexpr int ctas_per_sm(int) { return kCtasPerSm; }
    static __device__ __forceinline__ uint64_t units(uint64_t K) { return K / 16; }
    template <class M>
    static __device__ __forceinline__ void load_act(const ActPtrT<typename M::pointer> &a, uint64_t K_, uint64_t t_, uint64_t u_, Act &out)
    {
        using I = typename M::index;
        const I K = (I)K_, t = (I)t_, u = (I)u_;
        out.c = M::code16(a.codes, t * K + u * 16);
        out.d = M::f1(a.scales + (t * (K / 32) + (u >> 1)) * 4);
    }
    template <class M>
    static __device__ __forceinline__ void load_w(const typename M::View &w, uint64_t K_, uint64_t row_, uint64_t u_, uint32_t, W &out)
    {
        using I = typename M::index;
        const I K = (I)K_, row = (I)row_, u = (I)u_;
        (void)K;
        out.c = M::v4(w.p0 + row * K + u * 16);
        out.d = half_bits_to_float(M::u16(w.p1 + (row * (K / 32) + (u >> 1)) * 2));
    }
    template <bool DUMP>
    static __device__ __forceinline__ void dot(const W &w, const Act &a, bool valid, uint64_t u, uint32_t lane, float &acc, int32_t *dump)
    {
        int d = valid ? dot16(w.c, a.c, 0) : 0;
        if (DUMP) {
            // A block is split over two lanes; its exact integer dot is the sum of the halves.
            const int full = d + __shfl_xor_sync(kFull, d, 1);
            if (valid && !(lane & 1)) {
                dump[u >> 1] = full;
            }
        }
        if (valid) {
            acc = fmaf(small_int_to_float(d), w.d * a.d, acc);  // |d| <= 32 * 127 * 127
        }
    }
};

struct Q8NaturalXq8 {
    struct Act { uint4 c0, c1; float d; };
    struct W { uint4 c0, c1; float d; };
    static constexpr int kPlanes = 1;
    static constexpr bool kTokenTeams = false;  // as the planar layout
    static constexpr int kMaxUpl = 2, kRows = 2, kCtasPerSm = 2;
    static constexpr int min_ctas(int) { return 2; }
    static constexpr int ctas_per_sm(int) { return kCtasPerSm; }
    static void plane_row_bytes(uint64_t, uint64_t row_bytes, uint32_t *out) { out[0] = (uint32_t)row_bytes; }
    static __device__ __forceinline__ uint64_t units(uint64_t K) { return K / 32; }
    template <class M>
    static __device__ __forceinline__ void load_act(const ActPtrT<typename M::pointer> &a, uint64_t K_, uint64_t t_, uint64_t u_, Act &out)
    {
        using I = typename M::index;
        const I K = (I)K_, t = (I)t_, u = (I)u_;
        out.c0 = M::code16(a.codes, t * K + u * 32);
        out.c1 = M::code16(a.codes, t * K + u * 32 + 16);
        out.d = M::f1(a.scales + (t * (K / 32) + u) * 4);
    }
    template <class M>
    static __device__ __forceinline__ void load_w(const typename M::View &w, uint64_t K_, uint64_t row_, uint64_t u_, uint32_t, W &out)
    {
        using I = typename M::index;
        const I K = (I)K_, row = (I)row_, u = (I)u_;
        (void)K;
        const typename M::pointer block = w.p0 + row * w.row_bytes + u * 34;
        out.d = half_bits_to_float(M::u16(block));
        out.c0 = ld_unaligned16<M>(block + 2);
        out.c1 = ld_unaligned16<M>(block + 18);
    }
    template <bool DUMP>
    static __device__ __forceinline__ void dot(const W &w, const Act &a, bool valid, uint64_t u, uint32_t, float &acc, int32_t *dump)
    {
        if (valid) {
            const int d = dot16(w.c1, a.c1, dot16(w.c0, a.c0, 0));
            if (DUMP) {
                dump[u] = d;
            }
            acc = fmaf(small_int_to_float(d), w.d * a.d, acc);  // |d| <= 32 * 127 * 127
        }
    }
};

__device__ __forceinline__ int dp4a_us(uint32_t a_unsigned, uint32_t b_signed, int c)
{
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_unsigned), "r"(b_signed), "r"(c));
    return d;
}
// Q4_K in its file layout (144-byte blocks are 16-byte aligned). Unit = half a super-block: 64 nibble bytes = the
// four sub-blocks 4h..4h+3 (h = u%2) of super-block u/2. Taking four sub-blocks at once lets the 6-bit scales and
// mins be unpacked four at a time with a handful of word operations, and the high nibbles are used in place
// (q & 0xF0 = 16 * code, exact), so a weight word costs two masks and two dp4a.
struct Q4KXq8 {
    struct Act {
        uint4 c[8];   // 128 activation codes
        float d[4];   // block scales of the four sub-blocks
        float ds[4];  // block scale * sum of the block's codes (for the min term)
    };
    struct W { uint4 hdr, q[4]; };
    static constexpr int kPlanes = 1;
    static constexpr bool kTokenTeams = true;  // several tokens: one warp team per token (matvec_xq8_tokens_kernel)
    // One CTA per SM is launched, but the kernel is built so that two fit: the second slot is for the next kernel.
    static constexpr int kMaxUpl = 1, kRows = 2, kCtasPerSm = 1;
    static constexpr int min_ctas(int) { return 2; }
    static constexpr int ctas_per_sm(int) { return kCtasPerSm; }
    static void plane_row_bytes(uint64_t, uint64_t row_bytes, uint32_t *out) { out[0] = (uint32_t)row_bytes; }
    static __device__ __forceinline__ uint64_t units(uint64_t K) { return K / 128; }
    template <class M>
    static __device__ __forceinline__ void load_act(const ActPtrT<typename M::pointer> &a, uint64_t K_, uint64_t t_, uint64_t u_, Act &out)
    {
        using I = typename M::index;
        const I K = (I)K_, t = (I)t_, u = (I)u_;
        const I codes = t * K + u * 128;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            out.c[i] = M::code16(a.codes, codes + 16 * i);
        }
        const float4 d = M::f4(a.scales + (t * (K / 32) + u * 4) * 4);
        const uint4 s = M::v4c(a.sums + (t * (K / 16) + u * 8) * 2);
        out.d[0] = d.x;
        out.d[1] = d.y;
        out.d[2] = d.z;
        out.d[3] = d.w;
        out.ds[0] = d.x * (float)((int)(short)(s.x & 0xffff) + (int)(short)(s.x >> 16));
        out.ds[1] = d.y * (float)((int)(short)(s.y & 0xffff) + (int)(short)(s.y >> 16));
        out.ds[2] = d.z * (float)((int)(short)(s.z & 0xffff) + (int)(short)(s.z >> 16));
        out.ds[3] = d.w * (float)((int)(short)(s.w & 0xffff) + (int)(short)(s.w >> 16));
    }
    template <class M>
    static __device__ __forceinline__ void load_w(const typename M::View &w, uint64_t K_, uint64_t row_, uint64_t u_, uint32_t, W &out)
    {
        using I = typename M::index;
        const I K = (I)K_, row = (I)row_, u = (I)u_;
        (void)K;
        const typename M::pointer block = w.p0 + row * w.row_bytes + (u >> 1) * 144;
        out.hdr = M::v4c(block);
        const typename M::pointer q = block + 16 + (u & 1) * 64;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            out.q[i] = M::v4(q + 16 * i);
        }
    }
    template <bool DUMP>
    static __device__ __forceinline__ void dot(const W &w, const Act &a, bool valid, uint64_t u, uint32_t, float &acc, int32_t *dump)
    {
        if (!valid) {
            return;
        }
        // sub-block j = 2*pair + nibble: pair p uses nibble bytes q[2p], q[2p+1]; codes of sub-block j are c[2j], c[2j+1]
        int lo[2] = {0, 0}, hi16[2] = {0, 0};
#pragma unroll
        for (int p = 0; p < 2; ++p) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint32_t q = word_of(w.q[2 * p + i], k);
                    lo[p] = dp4a_us(q & 0x0F0F0F0Fu, word_of(a.c[4 * p + i], k), lo[p]);
                    hi16[p] = dp4a_us(q & 0xF0F0F0F0u, word_of(a.c[4 * p + 2 + i], k), hi16[p]);
                }
            }
        }
        if (DUMP) {
            int32_t *target = dump + u * 4;
            target[0] = lo[0];
            target[1] = hi16[0] >> 4;
            target[2] = lo[1];
            target[3] = hi16[1] >> 4;
        }
        // 6-bit scales and mins of sub-blocks 4h..4h+3, one per byte (ScaleMinK4, GgufKQuantBlocks.cs:149-153)
        uint32_t sc, mn;
        if ((u & 1) == 0) {
            sc = w.hdr.y & 0x3f3f3f3fu;
            mn = w.hdr.z & 0x3f3f3f3fu;
        } else {
            sc = (w.hdr.w & 0x0f0f0f0fu) | ((w.hdr.y >> 2) & 0x30303030u);
            mn = ((w.hdr.w >> 4) & 0x0f0f0f0fu) | ((w.hdr.z >> 2) & 0x30303030u);
        }
        // |lo| <= 32 * 15 * 127 and |hi16| <= 16 times that: both below 2^22
        float f_lo = (byte_to_float(sc, 0) * small_int_to_float(lo[0])) * a.d[0];
        f_lo = fmaf(byte_to_float(sc, 2) * small_int_to_float(lo[1]), a.d[2], f_lo);
        float f_hi = (byte_to_float(sc, 1) * small_int_to_float(hi16[0])) * a.d[1];
        f_hi = fmaf(byte_to_float(sc, 3) * small_int_to_float(hi16[1]), a.d[3], f_hi);
        float g = byte_to_float(mn, 0) * a.ds[0];
        g = fmaf(byte_to_float(mn, 1), a.ds[1], g);
        g = fmaf(byte_to_float(mn, 2), a.ds[2], g);
        g = fmaf(byte_to_float(mn, 3), a.ds[3], g);
        const float d = half_bits_to_float(w.hdr.x & 0xffff), dmin = half_bits_to_float(w.hdr.x >> 16);
        acc = fmaf(d, fmaf(f_hi, 0.0625f, f_lo), acc);
        acc = fmaf(-dmin, g, acc);
    }
};

// Q6_K. Unit = 64 values of super-block u/4: half h = (u/2)%2, byte range l = 16i..16i+15 with i = u%2; they are
// the four 16-value groups g = 8h + 2q + i (q = 0..3), each with its own int8 scale, living in activation
// block 8*sb + 4h + q.
struct Q6KAct {
    uint4 c[4];
    float d[4];
    int s[4];
};
template <class M>
__device__ __forceinline__ void q6k_load_act(const ActPtrT<typename M::pointer> &a, uint64_t K_, uint64_t t_, uint64_t u_, Q6KAct &out)
{
    using I = typename M::index;
    const I K = (I)K_, t = (I)t_, u = (I)u_;
    const I sb = u >> 2;
    const I h = (u >> 1) & 1, i = u & 1;
    const I codes = t * K + sb * 256 + h * 128 + i * 16;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        out.c[q] = M::code16(a.codes, codes + 32 * q);
    }
    const float4 d = M::f4(a.scales + (t * (K / 32) + sb * 8 + h * 4) * 4);
    out.d[0] = d.x;
    out.d[1] = d.y;
    out.d[2] = d.z;
    out.d[3] = d.w;
    const uint4 s = M::v4c(a.sums + (t * (K / 16) + sb * 16 + h * 8) * 2);
    const uint32_t shift = 16 * (uint32_t)i;
    out.s[0] = (int)(short)((s.x >> shift) & 0xffff);
    out.s[1] = (int)(short)((s.y >> shift) & 0xffff);
    out.s[2] = (int)(short)((s.z >> shift) & 0xffff);
    out.s[3] = (int)(short)((s.w >> shift) & 0xffff);
}

struct Q6KW {
    uint4 a, b, h;
    uint32_t sc_lo, sc_hi;  // the 8 int8 scales of the half
    float d;
};

template <bool DUMP>
__device__ __forceinline__ void q6k_dot(const Q6KW &w, const Q6KAct &a, bool valid, uint64_t u, float &acc, int32_t *dump)
{
    if (!valid) {
        return;
    }
    int dots[4] = {0, 0, 0, 0};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        uint32_t v1, v2, v3, v4;
        q6k_codes(word_of(w.a, k), word_of(w.b, k), word_of(w.h, k), v1, v2, v3, v4);
        dots[0] = __dp4a((int)v1, (int)word_of(a.c[0], k), dots[0]);
        dots[1] = __dp4a((int)v2, (int)word_of(a.c[1], k), dots[1]);
        dots[2] = __dp4a((int)v3, (int)word_of(a.c[2], k), dots[2]);
        dots[3] = __dp4a((int)v4, (int)word_of(a.c[3], k), dots[3]);
    }
    const uint32_t i = u & 1, h = (u >> 1) & 1;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int dot = dots[q] - 32 * a.s[q];
        // scale byte index inside the half: 2q + i
        const uint32_t word = q < 2 ? w.sc_lo : w.sc_hi;
        const int sc = (int)(signed char)((word >> (8 * (2 * (q & 1) + i))) & 0xff);
        if (DUMP) {
            dump[(u >> 2) * 16 + h * 8 + 2 * q + i] = dot;
        }
        acc = fmaf((w.d * small_int_to_float(sc)) * a.d[q], small_int_to_float(dot), acc);  // |dot| <= 16 * (63 + 32) * 127
    }
}

struct Q6KPlanarXq8 {
    using Act = Q6KAct;
    using W = Q6KW;
    static constexpr int kPlanes = 4;
    static constexpr bool kTokenTeams = true;  // as Q4_K
    static constexpr int kMaxUpl = 2, kRows = 2;
    // Single-warp teams (short rows): uncapped registers, one CTA per SM. Wider teams: two CTAs per SM.
    static constexpr int min_ctas(int W) { return W == 1 ? 1 : 2; }
    static constexpr int ctas_per_sm(int W) { return W == 1 ? 1 : 2; }
    static void plane_row_bytes(uint64_t K, uint64_t, uint32_t *out)
    {
        out[0] = (uint32_t)(K / 2);
        out[1] = (uint32_t)(K / 4);
        out[2] = (uint32_t)(K / 16);
        out[3] = (uint32_t)(K / 128);
    }
    static __device__ __forceinline__ uint64_t units(uint64_t K) { return K / 64; }
    template <class M>
    static __device__ __forceinline__ void load_act(const ActPtrT<typename M::pointer> &a, uint64_t K, uint64_t t, uint64_t u, Act &out)
    {
        q6k_load_act<M>(a, K, t, u, out);
    }
    template <class M>
    static __device__ __forceinline__ void load_w(const typename M::View &w, uint64_t K_, uint64_t row_, uint64_t u_, uint32_t, W &out)
    {
        using I = typename M::index;
        const I K = (I)K_, row = (I)row_, u = (I)u_;
        (void)K;
        const I sb = u >> 2;
        const I h = (u >> 1) & 1, i = u & 1;
        const typename M::pointer ql = w.p0 + row * (K / 2) + sb * 128 + h * 64 + i * 16;
        out.a = M::v4(ql);
        out.b = M::v4(ql + 32);
        out.h = M::v4(w.p1 + row * (K / 4) + sb * 64 + h * 32 + i * 16);
        const uint2 sc = M::v2(w.p2 + row * (K / 16) + sb * 16 + h * 8);
        out.sc_lo = sc.x;
        out.sc_hi = sc.y;
        out.d = half_bits_to_float(M::u16(w.p3 + (row * (K / 256) + sb) * 2));
    }
    template <bool DUMP>
    static __device__ __forceinline__ void dot(const W &w, const Act &a, bool valid, uint64_t u, uint32_t, float &acc, int32_t *dump)
    {
        q6k_dot<DUMP>(w, a, valid, u, acc, dump);
    }
};

struct Q6KNaturalXq8 {
    using Act = Q6KAct;
    using W = Q6KW;
    static constexpr int kPlanes = 1;
    static constexpr bool kTokenTeams = true;  // as Q4_K
    static constexpr int kMaxUpl = 2, kRows = 2, kCtasPerSm = 2;
    static constexpr int min_ctas(int) { return 2; }
    static constexpr int ctas_per_sm(int) { return kCtasPerSm; }
    static void plane_row_bytes(uint64_t, uint64_t row_bytes, uint32_t *out) { out[0] = (uint32_t)row_bytes; }
    static __device__ __forceinline__ uint64_t units(uint64_t K) { return K / 64; }
    template <class M>
    static __device__ __forceinline__ void load_act(const ActPtrT<typename M::pointer> &a, uint64_t K, uint64_t t, uint64_t u, Act &out)
    {
        q6k_load_act<M>(a, K, t, u, out);
    }
    template <class M>
    static __device__ __forceinline__ void load_w(const typename M::View &w, uint64_t K_, uint64_t row_, uint64_t u_, uint32_t, W &out)
    {
        using I = typename M::index;
        const I K = (I)K_, row = (I)row_, u = (I)u_;
        (void)K;
        const typename M::pointer block = w.p0 + row * w.row_bytes + (u >> 2) * 210;
        const I h = (u >> 1) & 1, i = u & 1;
        out.a = ld_unaligned16<M>(block + h * 64 + i * 16);
        out.b = ld_unaligned16<M>(block + h * 64 + i * 16 + 32);
        out.h = ld_unaligned16<M>(block + 128 + h * 32 + i * 16);
        const typename M::pointer sc = block + 192 + h * 8;
        out.sc_lo = M::u16(sc) | (M::u16(sc + 2) << 16);
        out.sc_hi = M::u16(sc + 4) | (M::u16(sc + 6) << 16);
        out.d = half_bits_to_float(M::u16(block + 208));
    }
    template <bool DUMP>
    static __device__ __forceinline__ void dot(const W &w, const Act &a, bool valid, uint64_t u, uint32_t, float &acc, int32_t *dump)
    {
        q6k_dot<DUMP>(w, a, valid, u, acc, dump);
    }
};

}  // namespace mv
}  // namespace syn
