// Dispatch of the decode matrix-vector products, and the FP32-activation (XF32) kernels.
//
// XF32 reproduces the `reference` backend: FP32 activations times exactly dequantised weights
// (GraphExecution/Q8Operators.cs:75-96, GraphExecution/DecodedRowOperators.cs:29-40) up to FP32 summation order.
// A warp owns R rows and strides over the row's units; activations are read through L1.
#include "matvec_formats.cuh"

namespace syn {
namespace mv {

cudaError_t launch_xq8_q8_0(const MatvecArgs &a, const WeightView *views, cudaStream_t stream);
cudaError_t launch_xq8_q4_k(const MatvecArgs &a, const WeightView *views, cudaStream_t stream);
cudaError_t launch_xq8_q6_k(const MatvecArgs &a, const WeightView *views, cudaStream_t stream);

namespace {

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
    static __device__ __forceinline__ void load_w(const WeightView &w, uint64_t K, uint64_t row, uint64_t u, W &out) { Q8PlanarXq8::load_w<GlobalMem>(w, K, row, u, 0, out); }
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
    static __device__ __forceinline__ void load_w(const WeightView &w, uint64_t K, uint64_t row, uint64_t u, W &out) { Q8NaturalXq8::load_w<GlobalMem>(w, K, row, u, 0, out); }
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

// Q4_K in its file layout, unit = one 32-byte nibble chunk: sub-blocks 2p (low nibbles) and 2p+1 (high nibbles) of
// super-block u/4, p = u%4.
struct Q4KXf32 {
    struct W { uint4 hdr, q0, q1; };
    static __device__ __forceinline__ uint64_t units(uint64_t K) { return K / 64; }
    static __device__ __forceinline__ void load_w(const WeightView &w, uint64_t, uint64_t row, uint64_t u, W &out)
    {
        const uint8_t *block = w.p0 + row * w.row_bytes + (u >> 2) * 144;
        out.hdr = ld_cached(block);
        out.q0 = ld_stream(block + 16 + (u & 3) * 32);
        out.q1 = ld_stream(block + 32 + (u & 3) * 32);
    }
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
    static __device__ __forceinline__ void load_w(const WeightView &w, uint64_t K, uint64_t row, uint64_t u, W &out) { Q6KPlanarXq8::load_w<GlobalMem>(w, K, row, u, 0, out); }
    static __device__ __forceinline__ void dot(const W &w, const float *x, uint64_t u, float &acc) { q6k_dot_f32(w, x, u, acc); }
};
struct Q6KNaturalXf32 {
    using W = Q6KW;
    static __device__ __forceinline__ uint64_t units(uint64_t K) { return K / 64; }
    static __device__ __forceinline__ void load_w(const WeightView &w, uint64_t K, uint64_t row, uint64_t u, W &out) { Q6KNaturalXq8::load_w<GlobalMem>(w, K, row, u, 0, out); }
    static __device__ __forceinline__ void dot(const W &w, const float *x, uint64_t u, float &acc) { q6k_dot_f32(w, x, u, acc); }
};

template <class F, int T, int R>
__global__ void __launch_bounds__(kWarps * 32)
matvec_xf32_kernel(WeightView w, const float *__restrict__ x, uint64_t in_stride, uint64_t K, uint64_t rows, uint32_t tokens,
                   float *__restrict__ y, uint64_t out_stride, Epilogue epilogue)
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
                    store_result(epilogue, y, token0 + t, out_stride, row0 + r, total);
                }
            }
        }
    }
}


WeightView view_of(const syn_b200_matrix *m, uint64_t row_start)
{
    WeightView v{};
    v.row_bytes = (uint32_t)m->row_bytes;
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
cudaError_t run_xf32(const MatvecArgs &a, cudaStream_t stream)
{
    const uint64_t row_groups = (a.row_count + R - 1) / R;
    uint64_t ctas = (row_groups + kWarps - 1) / kWarps;
    const uint64_t cap = (uint64_t)sm_count(a.matrix->device) * 8;
    if (ctas > cap) {
        ctas = cap;
    }
    const dim3 grid((unsigned)ctas, (unsigned)((a.tokens + T - 1) / T));
    matvec_xf32_kernel<F, T, R><<<grid, kWarps * 32, 0, stream>>>(view_of(a.matrix, a.row_start), a.x, a.in_stride, a.matrix->columns,
                                                                 a.row_count, (uint32_t)a.tokens, a.y, a.out_stride, a.fused);
    count_launch();
    return cudaGetLastError();
}

template <class F>
cudaError_t dispatch_xf32(const MatvecArgs &a, cudaStream_t stream)
{
    if (a.tokens <= 1) {
        return run_xf32<F, 1, 2>(a, stream);
    }
    if (a.tokens == 2) {
        return run_xf32<F, 2, 2>(a, stream);
    }
    return run_xf32<F, 4, 1>(a, stream);
}

}  // namespace
}  // namespace mv

cudaError_t launch_matvec(const MatvecArgs &args, cudaStream_t stream)
{
    using namespace mv;
    MatvecArgs a = args;
    a.fused.accumulate = (a.epilogue == SYN_B200_EPILOGUE_ACCUMULATE || args.fused.accumulate) ? 1u : 0u;
    const syn_b200_matrix *m = a.matrix;
    const bool planar = m->layout == Layout::Planar;
    if (a.dump || a.mode == SYN_B200_MODE_XQ8) {
        WeightView views[3] = {view_of(m, a.row_start), WeightView{}, WeightView{}};
        for (uint32_t i = 0; a.form != 0 && i < a.segment_count && i < 3; ++i) {
            views[i] = view_of(a.segments[i].matrix, a.segments[i].row_start);
        }
        return m->type == kQ8_0 ? launch_xq8_q8_0(a, views, stream)
               : m->type == kQ4_K ? launch_xq8_q4_k(a, views, stream)
                                  : launch_xq8_q6_k(a, views, stream);
    }
    if (a.form != 0) {
        return cudaErrorNotSupported;
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
