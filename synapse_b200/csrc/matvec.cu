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
#include "common.cuh"

namespace syn {

namespace {

constexpr int kWarps = 8;
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

// 16 bytes from an address that is only 2-byte aligned (file-layout Q8_0 and Q6_K blocks).
__device__ __forceinline__ uint4 ld_unaligned16(const uint8_t *p)
{
    uint32_t h[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        h[i] = ld_u16(p + 2 * i);
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

__device__ __forceinline__ uint32_t word_of(const uint4 &v, int i) { return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w; }

// ------------------------------------------------------------------------------------------------------
// Weight views
// ------------------------------------------------------------------------------------------------------

struct WeightView {
    const uint8_t *p0, *p1, *p2, *p3;  // plane (or file-layout) bases, already offset to the first row of the call
    uint64_t row_bytes;                // of the file layout
};

// ------------------------------------------------------------------------------------------------------
// XQ8 formats. Each provides: units(K); struct Act; struct W; load_act; load_w; dot (updates acc, optionally
// writes the integer sub-block sums of the unit to `dump`, which points at this (token,row)'s group array).
// ------------------------------------------------------------------------------------------------------

struct Q8PlanarXq8 {
    struct Act { uint4 c; float d; };
    struct W { uint4 c; float d; };
    static __device__ __forceinline__ uint64_t units(uint64_t K) { return K / 16; }
    static __device__ __forceinline__ void load_act(const ActView &a, uint64_t K, uint64_t t, uint64_t u, Act &out)
    {
        out.c = ld_cached(a.codes + t * K + u * 16);
        out.d = __ldg(a.scales + t * (K / 32) + (u >> 1));
    }
    static __device__ __forceinline__ void load_w(const WeightView &w, uint64_t K, uint64_t row, uint64_t u, uint32_t, W &out)
    {
        out.c = ld_stream(w.p0 + row * K + u * 16);
        out.d = half_bits_to_float(ld_u16(w.p1 + (row * (K / 32) + (u >> 1)) * 2));
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
            acc = fmaf((float)d, w.d * a.d, acc);
        }
    }
};

struct Q8NaturalXq8 {
    struct Act { uint4 c0, c1; float d; };
    struct W { uint4 c0, c1; float d; };
    static __device__ __forceinline__ uint64_t units(uint64_t K) { return K / 32; }
    static __device__ __forceinline__ void load_act(const ActView &a, uint64_t K, uint64_t t, uint64_t u, Act &out)
    {
        out.c0 = ld_cached(a.codes + t * K + u * 32);
        out.c1 = ld_cached(a.codes + t * K + u * 32 + 16);
        out.d = __ldg(a.scales + t * (K / 32) + u);
    }
    static __device__ __forceinline__ void load_w(const WeightView &w, uint64_t, uint64_t row, uint64_t u, uint32_t, W &out)
    {
        const uint8_t *block = w.p0 + row * w.row_bytes + u * 34;
        out.d = half_bits_to_float(ld_u16(block));
        out.c0 = ld_unaligned16(block + 2);
        out.c1 = ld_unaligned16(block + 18);
    }
    template <bool DUMP>
    static __device__ __forceinline__ void dot(const W &w, const Act &a, bool valid, uint64_t u, uint32_t, float &acc, int32_t *dump)
    {
        if (valid) {
            const int d = dot16(w.c1, a.c1, dot16(w.c0, a.c0, 0));
            if (DUMP) {
                dump[u] = d;
            }
            acc = fmaf((float)d, w.d * a.d, acc);
        }
    }
};

// Q4_K in its file layout (144-byte blocks are 16-byte aligned). Unit = one 32-byte nibble chunk: sub-blocks
// 2p (low nibbles) and 2p+1 (high nibbles) of super-block u/4, p = u%4.
struct Q4KXq8 {
    struct Act { uint4 c[4]; float d0, d1; int s0, s1; };
    struct W { uint4 hdr, q0, q1; };
    static __device__ __forceinline__ uint64_t units(uint64_t K) { return K / 64; }
    static __device__ __forceinline__ void load_act(const ActView &a, uint64_t K, uint64_t t, uint64_t u, Act &out)
    {
        const int8_t *codes = a.codes + t * K + u * 64;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            out.c[i] = ld_cached(codes + 16 * i);
        }
        const float2 d = __ldg(reinterpret_cast<const float2 *>(a.scales + t * (K / 32) + u * 2));
        out.d0 = d.x;
        out.d1 = d.y;
        const uint2 s = __ldg(reinterpret_cast<const uint2 *>(a.sums + t * (K / 16) + u * 4));
        out.s0 = (int)(short)(s.x & 0xffff) + (int)(short)(s.x >> 16);
        out.s1 = (int)(short)(s.y & 0xffff) + (int)(short)(s.y >> 16);
    }
    static __device__ __forceinline__ void load_w(const WeightView &w, uint64_t, uint64_t row, uint64_t u, uint32_t, W &out)
    {
        const uint8_t *block = w.p0 + row * w.row_bytes + (u >> 2) * 144;
        out.hdr = ld_cached(block);
        out.q0 = ld_stream(block + 16 + (u & 3) * 32);
        out.q1 = ld_stream(block + 32 + (u & 3) * 32);
    }
    template <bool DUMP>
    static __device__ __forceinline__ void dot(const W &w, const Act &a, bool valid, uint64_t u, uint32_t, float &acc, int32_t *dump)
    {
        if (!valid) {
            return;
        }
        int lo = 0, hi = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t q = word_of(w.q0, i);
            lo = __dp4a((int)(q & 0x0F0F0F0Fu), (int)word_of(a.c[0], i), lo);
            hi = __dp4a((int)((q >> 4) & 0x0F0F0F0Fu), (int)word_of(a.c[2], i), hi);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t q = word_of(w.q1, i);
            lo = __dp4a((int)(q & 0x0F0F0F0Fu), (int)word_of(a.c[1], i), lo);
            hi = __dp4a((int)((q >> 4) & 0x0F0F0F0Fu), (int)word_of(a.c[3], i), hi);
        }
        if (DUMP) {
            dump[u * 2] = lo;
            dump[u * 2 + 1] = hi;
        }
        uint32_t sc0, m0, sc1, m1;
        q4k_scales(w.hdr.y, w.hdr.z, w.hdr.w, (uint32_t)(u & 3), sc0, m0, sc1, m1);
        const float d = half_bits_to_float(w.hdr.x & 0xffff), dmin = half_bits_to_float(w.hdr.x >> 16);
        acc = fmaf((d * (float)sc0) * a.d0, (float)lo, acc);
        acc = fmaf(-((dmin * (float)m0) * a.d0), (float)a.s0, acc);
        acc = fmaf((d * (float)sc1) * a.d1, (float)hi, acc);
        acc = fmaf(-((dmin * (float)m1) * a.d1), (float)a.s1, acc);
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
__device__ __forceinline__ void q6k_load_act(const ActView &a, uint64_t K, uint64_t t, uint64_t u, Q6KAct &out)
{
    const uint64_t sb = u >> 2;
    const uint32_t h = (u >> 1) & 1, i = u & 1;
    const int8_t *codes = a.codes + t * K + sb * 256 + h * 128 + i * 16;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        out.c[q] = ld_cached(codes + 32 * q);
    }
    const float4 d = __ldg(reinterpret_cast<const float4 *>(a.scales + t * (K / 32) + sb * 8 + h * 4));
    out.d[0] = d.x;
    out.d[1] = d.y;
    out.d[2] = d.z;
    out.d[3] = d.w;
    const uint4 s = ld_cached(a.sums + t * (K / 16) + sb * 16 + h * 8);
    const uint32_t shift = 16 * i;
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
        acc = fmaf((w.d * (float)sc) * a.d[q], (float)dot, acc);
    }
}

struct Q6KPlanarXq8 {
    using Act = Q6KAct;
    using W = Q6KW;
    static __device__ __forceinline__ uint64_t units(uint64_t K) { return K / 64; }
    static __device__ __forceinline__ void load_act(const ActView &a, uint64_t K, uint64_t t, uint64_t u, Act &out) { q6k_load_act(a, K, t, u, out); }
    static __device__ __forceinline__ void load_w(const WeightView &w, uint64_t K, uint64_t row, uint64_t u, uint32_t, W &out)
    {
        const uint64_t sb = u >> 2;
        const uint32_t h = (u >> 1) & 1, i = u & 1;
        const uint8_t *ql = w.p0 + row * (K / 2) + sb * 128 + h * 64 + i * 16;
        out.a = ld_stream(ql);
        out.b = ld_stream(ql + 32);
        out.h = ld_stream(w.p1 + row * (K / 4) + sb * 64 + h * 32 + i * 16);
        const uint2 sc = __ldg(reinterpret_cast<const uint2 *>(w.p2 + row * (K / 16) + sb * 16 + h * 8));
        out.sc_lo = sc.x;
        out.sc_hi = sc.y;
        out.d = half_bits_to_float(ld_u16(w.p3 + (row * (K / 256) + sb) * 2));
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
    static __device__ __forceinline__ uint64_t units(uint64_t K) { return K / 64; }
    static __device__ __forceinline__ void load_act(const ActView &a, uint64_t K, uint64_t t, uint64_t u, Act &out) { q6k_load_act(a, K, t, u, out); }
    static __device__ __forceinline__ void load_w(const WeightView &w, uint64_t, uint64_t row, uint64_t u, uint32_t, W &out)
    {
        const uint8_t *block = w.p0 + row * w.row_bytes + (u >> 2) * 210;
        const uint32_t h = (u >> 1) & 1, i = u & 1;
        out.a = ld_unaligned16(block + h * 64 + i * 16);
        out.b = ld_unaligned16(block + h * 64 + i * 16 + 32);
        out.h = ld_unaligned16(block + 128 + h * 32 + i * 16);
        const uint8_t *sc = block + 192 + h * 8;
        out.sc_lo = ld_u16(sc) | (ld_u16(sc + 2) << 16);
        out.sc_hi = ld_u16(sc + 4) | (ld_u16(sc + 6) << 16);
        out.d = half_bits_to_float(ld_u16(block + 208));
    }
    template <bool DUMP>
    static __device__ __forceinline__ void dot(const W &w, const Act &a, bool valid, uint64_t u, uint32_t, float &acc, int32_t *dump)
    {
        q6k_dot<DUMP>(w, a, valid, u, acc, dump);
    }
};

// ------------------------------------------------------------------------------------------------------
// XQ8 kernel
// ------------------------------------------------------------------------------------------------------

template <class F, int T, int R, bool DUMP>
__global__ void __launch_bounds__(kWarps * 32)
matvec_xq8_kernel(WeightView w, ActView act, uint64_t K, uint64_t rows, uint32_t tokens, float *__restrict__ y,
                  uint64_t out_stride, uint32_t accumulate, int32_t *__restrict__ dump, uint64_t dump_groups)
{
    const uint32_t lane = threadIdx.x & 31;
    const uint64_t warp = (uint64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
    const uint64_t warps = (uint64_t)gridDim.x * kWarps;
    const uint64_t token0 = (uint64_t)blockIdx.y * T;
    const uint32_t live = min((uint32_t)T, tokens - (uint32_t)token0);
    const uint64_t units = F::units(K);
    for (uint64_t row0 = warp * R; row0 < rows; row0 += warps * R) {
        float acc[R][T];
#pragma unroll
        for (int r = 0; r < R; ++r) {
#pragma unroll
            for (int t = 0; t < T; ++t) {
                acc[r][t] = 0.0f;
            }
        }
        for (uint64_t base = 0; base < units; base += 32) {
            const bool valid = base + lane < units;
            const uint64_t u = valid ? base + lane : units - 1;
            typename F::W wr[R];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                F::load_w(w, K, min(row0 + r, rows - 1), u, lane, wr[r]);
            }
#pragma unroll
            for (int t = 0; t < T; ++t) {
                typename F::Act a;
                F::load_act(act, K, token0 + min((uint32_t)t, live - 1), u, a);
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    int32_t *target = DUMP ? dump + ((token0 + t) * rows + min(row0 + r, rows - 1)) * dump_groups : nullptr;
                    F::template dot<DUMP>(wr[r], a, valid, u, lane, acc[r][t], target);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
#pragma unroll
            for (int t = 0; t < T; ++t) {
                const float total = warp_sum(acc[r][t]);
                if (lane == 0 && row0 + r < rows && (uint32_t)t < live) {
                    float *destination = y + (token0 + t) * out_stride + row0 + r;
                    *destination = accumulate ? *destination + total : total;
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------------
// XF32 kernels: same lane geometry, FP32 activations read through L1.
// ------------------------------------------------------------------------------------------------------

__device__ __forceinline__ float4 ldx4(const float *p) { return __ldg(reinterpret_cast<const float4 *>(p)); }

// sum over 4 bytes of word `q` (each 0..255, or signed when SIGNED) times x.
template <bool SIGNED>
__device__ __forceinline__ void fma4(uint32_t q, const float4 &x, float &s)
{
    if (SIGNED) {
        s = fmaf((float)(int)(signed char)(q & 0xff), x.x, s);
        s = fmaf((float)(int)(signed char)((q >> 8) & 0xff), x.y, s);
        s = fmaf((float)(int)(signed char)((q >> 16) & 0xff), x.z, s);
        s = fmaf((float)(int)(signed char)(q >> 24), x.w, s);
    } else {
        s = fmaf((float)(q & 0xff), x.x, s);
        s = fmaf((float)((q >> 8) & 0xff), x.y, s);
        s = fmaf((float)((q >> 16) & 0xff), x.z, s);
        s = fmaf((float)(q >> 24), x.w, s);
    }
}

struct Q8PlanarXf32 {
    using W = Q8PlanarXq8::W;
    static __device__ __forceinline__ uint64_t units(uint64_t K) { return K / 16; }
    static __device__ __forceinline__ void load_w(const WeightView &w, uint64_t K, uint64_t row, uint64_t u, W &out) { Q8PlanarXq8::load_w(w, K, row, u, 0, out); }
    static __device__ __forceinline__ void dot(const W &w, const float *x, uint64_t u, float &acc)
    {
        const float *xu = x + u * 16;
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            fma4<true>(word_of(w.c, i), ldx4(xu + 4 * i), s);
        }
        acc = fmaf(w.d, s, acc);
    }
};

struct Q8NaturalXf32 {
    using W = Q8NaturalXq8::W;
    static __device__ __forceinline__ uint64_t units(uint64_t K) { return K / 32; }
    static __device__ __forceinline__ void load_w(const WeightView &w, uint64_t K, uint64_t row, uint64_t u, W &out) { Q8NaturalXq8::load_w(w, K, row, u, 0, out); }
    static __device__ __forceinline__ void dot(const W &w, const float *x, uint64_t u, float &acc)
    {
        const float *xu = x + u * 32;
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            fma4<true>(word_of(w.c0, i), ldx4(xu + 4 * i), s);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            fma4<true>(word_of(w.c1, i), ldx4(xu + 16 + 4 * i), s);
        }
        acc = fmaf(w.d, s, acc);
    }
};

struct Q4KXf32 {
    using W = Q4KXq8::W;
    static __device__ __forceinline__ uint64_t units(uint64_t K) { return K / 64; }
    static __device__ __forceinline__ void load_w(const WeightView &w, uint64_t K, uint64_t row, uint64_t u, W &out) { Q4KXq8::load_w(w, K, row, u, 0, out); }
    static __device__ __forceinline__ void dot(const W &w, const float *x, uint64_t u, float &acc)
    {
        const float *xu = x + u * 64;
        float lo = 0.0f, hi = 0.0f, xlo = 0.0f, xhi = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t q = i < 4 ? word_of(w.q0, i) : word_of(w.q1, i - 4);
            const float4 a = ldx4(xu + 4 * i), b = ldx4(xu + 32 + 4 * i);
            fma4<false>(q & 0x0F0F0F0Fu, a, lo);
            fma4<false>((q >> 4) & 0x0F0F0F0Fu, b, hi);
            xlo += (a.x + a.y) + (a.z + a.w);
            xhi += (b.x + b.y) + (b.z + b.w);
        }
        uint32_t sc0, m0, sc1, m1;
        q4k_scales(w.hdr.y, w.hdr.z, w.hdr.w, (uint32_t)(u & 3), sc0, m0, sc1, m1);
        const float d = half_bits_to_float(w.hdr.x & 0xffff), dmin = half_bits_to_float(w.hdr.x >> 16);
        acc = fmaf(d * (float)sc0, lo, acc);
        acc = fmaf(-(dmin * (float)m0), xlo, acc);
        acc = fmaf(d * (float)sc1, hi, acc);
        acc = fmaf(-(dmin * (float)m1), xhi, acc);
    }
};

__device__ __forceinline__ void q6k_dot_f32(const Q6KW &w, const float *x, uint64_t u, float &acc)
{
    const uint64_t sb = u >> 2;
    const uint32_t h = (u >> 1) & 1, i = u & 1;
    const float *xu = x + sb * 256 + h * 128 + i * 16;
    float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        uint32_t v[4];
        q6k_codes(word_of(w.a, k), word_of(w.b, k), word_of(w.h, k), v[0], v[1], v[2], v[3]);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float4 xv = ldx4(xu + 32 * q + 4 * k);
            s[q] = fmaf((float)((int)(v[q] & 0xff) - 32), xv.x, s[q]);
            s[q] = fmaf((float)((int)((v[q] >> 8) & 0xff) - 32), xv.y, s[q]);
            s[q] = fmaf((float)((int)((v[q] >> 16) & 0xff) - 32), xv.z, s[q]);
            s[q] = fmaf((float)((int)(v[q] >> 24) - 32), xv.w, s[q]);
        }
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const uint32_t word = q < 2 ? w.sc_lo : w.sc_hi;
        const int sc = (int)(signed char)((word >> (8 * (2 * (q & 1) + i))) & 0xff);
        acc = fmaf(w.d * (float)sc, s[q], acc);
    }
}

struct Q6KPlanarXf32 {
    using W = Q6KW;
    static __device__ __forceinline__ uint64_t units(uint64_t K) { return K / 64; }
    static __device__ __forceinline__ void load_w(const WeightView &w, uint64_t K, uint64_t row, uint64_t u, W &out) { Q6KPlanarXq8::load_w(w, K, row, u, 0, out); }
    static __device__ __forceinline__ void dot(const W &w, const float *x, uint64_t u, float &acc) { q6k_dot_f32(w, x, u, acc); }
};
struct Q6KNaturalXf32 {
    using W = Q6KW;
    static __device__ __forceinline__ uint64_t units(uint64_t K) { return K / 64; }
    static __device__ __forceinline__ void load_w(const WeightView &w, uint64_t K, uint64_t row, uint64_t u, W &out) { Q6KNaturalXq8::load_w(w, K, row, u, 0, out); }
    static __device__ __forceinline__ void dot(const W &w, const float *x, uint64_t u, float &acc) { q6k_dot_f32(w, x, u, acc); }
};

template <class F, int T, int R>
__global__ void __launch_bounds__(kWarps * 32)
matvec_xf32_kernel(WeightView w, const float *__restrict__ x, uint64_t in_stride, uint64_t K, uint64_t rows, uint32_t tokens,
                   float *__restrict__ y, uint64_t out_stride, uint32_t accumulate)
{
    const uint32_t lane = threadIdx.x & 31;
    const uint64_t warp = (uint64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
    const uint64_t warps = (uint64_t)gridDim.x * kWarps;
    const uint64_t token0 = (uint64_t)blockIdx.y * T;
    const uint32_t live = min((uint32_t)T, tokens - (uint32_t)token0);
    const uint64_t units = F::units(K);
    for (uint64_t row0 = warp * R; row0 < rows; row0 += warps * R) {
        float acc[R][T];
#pragma unroll
        for (int r = 0; r < R; ++r) {
#pragma unroll
            for (int t = 0; t < T; ++t) {
                acc[r][t] = 0.0f;
            }
        }
        for (uint64_t u = lane; u < units; u += 32) {
            typename F::W wr[R];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                F::load_w(w, K, min(row0 + r, rows - 1), u, wr[r]);
            }
#pragma unroll
            for (int t = 0; t < T; ++t) {
                const float *xt = x + (token0 + min((uint32_t)t, live - 1)) * in_stride;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    F::dot(wr[r], xt, u, acc[r][t]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
#pragma unroll
            for (int t = 0; t < T; ++t) {
                const float total = warp_sum(acc[r][t]);
                if (lane == 0 && row0 + r < rows && (uint32_t)t < live) {
                    float *destination = y + (token0 + t) * out_stride + row0 + r;
                    *destination = accumulate ? *destination + total : total;
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------------
// Launch
// ------------------------------------------------------------------------------------------------------

struct Geometry {
    unsigned grid_x, grid_y;
};

Geometry geometry(const syn_b200_matrix *m, uint64_t rows, uint64_t tokens, int T, int R)
{
    const uint64_t row_groups = (rows + R - 1) / R;
    uint64_t ctas = (row_groups + kWarps - 1) / kWarps;
    const uint64_t cap = (uint64_t)sm_count(m->device) * 8;  // 8 CTAs of 256 threads fill an SM
    if (ctas > cap) {
        ctas = cap;
    }
    return Geometry{(unsigned)ctas, (unsigned)((tokens + T - 1) / T)};
}

WeightView view_of(const syn_b200_matrix *m, uint64_t row_start)
{
    WeightView v{};
    v.row_bytes = m->row_bytes;
    const uint64_t K = m->columns;
    if (m->layout == Layout::Natural) {
        v.p0 = m->data + row_start * m->row_bytes;
    } else if (m->type == kQ8_0) {
        v.p0 = m->data + m->planes.p0 + row_start * K;
        v.p1 = m->data + m->planes.p1 + row_start * (K / 32) * 2;
    } else {
        v.p0 = m->data + m->planes.p0 + row_start * (K / 2);
        v.p1 = m->data + m->planes.p1 + row_start * (K / 4);
        v.p2 = m->data + m->planes.p2 + row_start * (K / 16);
        v.p3 = m->data + m->planes.p3 + row_start * (K / 256) * 2;
    }
    return v;
}

template <class F, int T, int R>
cudaError_t run_xq8(const MatvecArgs &a, cudaStream_t stream)
{
    const Geometry g = geometry(a.matrix, a.row_count, a.tokens, T, R);
    matvec_xq8_kernel<F, T, R, false><<<dim3(g.grid_x, g.grid_y), kWarps * 32, 0, stream>>>(
        view_of(a.matrix, a.row_start), a.act, a.matrix->columns, a.row_count, (uint32_t)a.tokens, a.y, a.out_stride,
        a.epilogue == SYN_B200_EPILOGUE_ACCUMULATE, nullptr, 0);
    count_launch();
    return cudaGetLastError();
}

template <class F>
cudaError_t run_xq8_dump(const MatvecArgs &a, uint64_t groups, cudaStream_t stream)
{
    const Geometry g = geometry(a.matrix, a.row_count, a.tokens, 1, 1);
    matvec_xq8_kernel<F, 1, 1, true><<<dim3(g.grid_x, g.grid_y), kWarps * 32, 0, stream>>>(
        view_of(a.matrix, a.row_start), a.act, a.matrix->columns, a.row_count, (uint32_t)a.tokens, a.y, a.out_stride, 0,
        a.dump, groups);
    count_launch();
    return cudaGetLastError();
}

template <class F, int T, int R>
cudaError_t run_xf32(const MatvecArgs &a, cudaStream_t stream)
{
    const Geometry g = geometry(a.matrix, a.row_count, a.tokens, T, R);
    matvec_xf32_kernel<F, T, R><<<dim3(g.grid_x, g.grid_y), kWarps * 32, 0, stream>>>(
        view_of(a.matrix, a.row_start), a.x, a.in_stride, a.matrix->columns, a.row_count, (uint32_t)a.tokens, a.y,
        a.out_stride, a.epilogue == SYN_B200_EPILOGUE_ACCUMULATE);
    count_launch();
    return cudaGetLastError();
}

// Token group size: the smallest of 1, 2, 4, 8 that holds the tokens (step/projection.rs:82-87).
int group_size(uint64_t tokens) { return tokens <= 1 ? 1 : tokens == 2 ? 2 : tokens <= 4 ? 4 : 8; }

template <class F>
cudaError_t dispatch_xq8(const MatvecArgs &a, cudaStream_t stream)
{
    // Rows per warp: two while there are enough row groups to fill the machine, one otherwise.
    const bool wide = a.row_count >= (uint64_t)sm_count(a.matrix->device) * kWarps * 4;
    switch (group_size(a.tokens)) {
    case 1: return wide ? run_xq8<F, 1, 2>(a, stream) : run_xq8<F, 1, 1>(a, stream);
    case 2: return wide ? run_xq8<F, 2, 2>(a, stream) : run_xq8<F, 2, 1>(a, stream);
    case 4: return run_xq8<F, 4, 1>(a, stream);
    default: return run_xq8<F, 8, 1>(a, stream);
    }
}

template <class F>
cudaError_t dispatch_xf32(const MatvecArgs &a, cudaStream_t stream)
{
    switch (group_size(a.tokens)) {
    case 1: return run_xf32<F, 1, 2>(a, stream);
    case 2: return run_xf32<F, 2, 2>(a, stream);
    default: return run_xf32<F, 4, 1>(a, stream);
    }
}

}  // namespace

cudaError_t launch_matvec(const MatvecArgs &a, cudaStream_t stream)
{
    const syn_b200_matrix *m = a.matrix;
    const bool planar = m->layout == Layout::Planar;
    if (a.dump) {
        const uint64_t K = m->columns;
        if (m->type == kQ8_0) {
            return planar ? run_xq8_dump<Q8PlanarXq8>(a, K / 32, stream) : run_xq8_dump<Q8NaturalXq8>(a, K / 32, stream);
        }
        if (m->type == kQ4_K) {
            return run_xq8_dump<Q4KXq8>(a, K / 32, stream);
        }
        return planar ? run_xq8_dump<Q6KPlanarXq8>(a, K / 16, stream) : run_xq8_dump<Q6KNaturalXq8>(a, K / 16, stream);
    }
    if (a.mode == SYN_B200_MODE_XQ8) {
        if (m->type == kQ8_0) {
            return planar ? dispatch_xq8<Q8PlanarXq8>(a, stream) : dispatch_xq8<Q8NaturalXq8>(a, stream);
        }
        if (m->type == kQ4_K) {
            return dispatch_xq8<Q4KXq8>(a, stream);
        }
        return planar ? dispatch_xq8<Q6KPlanarXq8>(a, stream) : dispatch_xq8<Q6KNaturalXq8>(a, stream);
    }
    if (m->type == kQ8_0) {
        return planar ? dispatch_xf32<Q8PlanarXf32>(a, stream) : dispatch_xf32<Q8NaturalXf32>(a, stream);
    }
    if (m->type == kQ4_K) {
        return dispatch_xf32<Q4KXf32>(a, stream);
    }
    return planar ? dispatch_xf32<Q6KPlanarXf32>(a, stream) : dispatch_xf32<Q6KNaturalXf32>(a, stream);
}

}  // namespace syn
