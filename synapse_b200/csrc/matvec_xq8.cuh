// The quantised-activation (XQ8) matrix-vector kernel and its launcher, instantiated once per weight format in
// matvec_q8_0.cu / matvec_q4_k.cu / matvec_q6_k.cu.
//
// Work split. A row is cut into "units" (the 16 or 64 weights one lane reads per step). A team of W warps covers
// the row: warp w of the team owns units [(i*W + w)*UPL*32, +UPL*32) for i = 0.., lane l takes unit +j*32 + l.
// W and UPL depend only on the row length, never on the number of rows or tokens, so a row's FP32 summation
// order -- lane chain, xor-shuffle tree, then the team's warps in index order -- is the same for every row range
// and token count (the reference's kernels are batch-invariant in the same way, cuda/kernels/matmul.cu:1-2).
// When one pass of the team covers the row and a single token is multiplied, each lane keeps its slice of the
// quantised activations in registers for the whole launch, and the loop body is weight loads + dp4a only.
// The grid is persistent (a multiple of the SM count); every CTA runs the same number of iterations so the
// team reduction can use one CTA barrier per iteration with double-buffered partial sums.
#pragma once
#include <atomic>
#include <type_traits>

#include "matvec_formats.cuh"

namespace syn {
namespace mv {

// Programmatic dependent launch: `pdl_launch_dependents` lets the next kernel of the stream start its prologue
// as soon as every CTA of this grid has passed this point; `pdl_wait` blocks until the kernel before this one has
// finished and its writes are visible. A kernel must not read anything an earlier kernel may have written, nor
// write global memory at all, before `pdl_wait`. Both are no-ops in an ordinary launch.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Shared-memory layout of in-kernel quantised activations for T tokens of K values.
__host__ __device__ inline uint32_t shared_act_codes_bytes(uint32_t tokens, uint32_t K) { return (tokens * K + 127u) & ~127u; }
__host__ __device__ inline uint32_t shared_act_side_bytes(uint32_t tokens, uint32_t K) { return (tokens * (K / 8) + 127u) & ~127u; }
__host__ __device__ inline uint32_t shared_act_bytes(uint32_t tokens, uint32_t K)
{
    return shared_act_codes_bytes(tokens, K) + 2 * shared_act_side_bytes(tokens, K);
}

// The Q8_0 activation quantiser (same arithmetic as quantize.cu, bit for bit) run by the `warps` calling warps of a
// CTA straight into shared memory. A lane reads four consecutive values (one 128-bit load), so a warp covers four
// 32-value blocks per load with eight lanes per block; eight loads per lane are in flight to cover the L2 latency.
template <int T>
__device__ __forceinline__ void quantize_to_shared(const float *__restrict__ x, uint64_t in_stride, uint32_t K, uint32_t live, uint32_t warp,
                                                   uint32_t warps, uint32_t lane, const ActShared &dst)
{
    constexpr int kDepth = 8;
    const uint32_t quads = (K + 127) / 128;  // groups of four blocks
#pragma unroll
    for (int t = 0; t < T; ++t) {
        const float *xt = x + (uint64_t)min((uint32_t)t, live - 1) * in_stride;
        for (uint32_t q0 = warp; q0 < quads; q0 += warps * kDepth) {
            float4 v[kDepth];
#pragma unroll
            for (int i = 0; i < kDepth; ++i) {
                const uint32_t first = (q0 + i * warps) * 128 + lane * 4;
                v[i] = first < K ? __ldg(reinterpret_cast<const float4 *>(xt + first)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
#pragma unroll
            for (int i = 0; i < kDepth; ++i) {
                const uint32_t first = (q0 + i * warps) * 128 + lane * 4;
                float amax = fmaxf(fmaxf(fabsf(v[i].x), fabsf(v[i].y)), fmaxf(fabsf(v[i].z), fabsf(v[i].w)));
                amax = fmaxf(amax, __shfl_xor_sync(kFull, amax, 1));
                amax = fmaxf(amax, __shfl_xor_sync(kFull, amax, 2));
                amax = fmaxf(amax, __shfl_xor_sync(kFull, amax, 4));
                const float scale = __fdiv_rn(amax, 127.0f);
                const float inverse = scale == 0.0f ? 0.0f : __fdiv_rn(1.0f, scale);
                const int c0 = __float2int_rn(__fmul_rn(v[i].x, inverse)), c1 = __float2int_rn(__fmul_rn(v[i].y, inverse));
                const int c2 = __float2int_rn(__fmul_rn(v[i].z, inverse)), c3 = __float2int_rn(__fmul_rn(v[i].w, inverse));
                int sum = (c0 + c1) + (c2 + c3);
                sum += __shfl_xor_sync(kFull, sum, 1);
                sum += __shfl_xor_sync(kFull, sum, 2);
                if (first < K) {
                    const uint32_t packed = (uint32_t)(c0 & 0xff) | ((uint32_t)(c1 & 0xff) << 8) | ((uint32_t)(c2 & 0xff) << 16) | ((uint32_t)c3 << 24);
                    asm volatile("st.shared.u32 [%0], %1;" ::"r"(dst.codes + swizzled_code_offset(t * K + first)), "r"(packed) : "memory");
                    if ((lane & 3) == 0) {
                        asm volatile("st.shared.u16 [%0], %1;" ::"r"(dst.sums + (t * (K / 16) + first / 16) * 2), "h"((short)sum) : "memory");
                    }
                    if ((lane & 7) == 0) {
                        asm volatile("st.shared.f32 [%0], %1;" ::"r"(dst.scales + (t * (K / 32) + first / 32) * 4), "f"(__half2float(__float2half_rn(scale)))
                                     : "memory");
                    }
                }
            }
        }
    }
}

// Consumer warps of a CTA for a team of W warps: as many whole teams as fit in eight warps.
__host__ __device__ constexpr int team_warps(int W) { return (kWarps / W) * W; }

template <class F, int T, int W, int UPL, int R, bool REGS, bool DUMP>
__global__ void __launch_bounds__(team_warps(W) * 32)
matvec_xq8_team_kernel(WeightView w, ActView act, uint64_t K, uint64_t rows, uint32_t tokens, float *__restrict__ y,
                       uint64_t out_stride, Epilogue epilogue, int32_t *__restrict__ dump, uint64_t dump_groups)
{
    static_assert(!REGS || T == 1, "register-resident activations are for single-token launches");
    constexpr int kTeams = kWarps / W;
    constexpr int kConsumers = team_warps(W);
    __shared__ float partial[2][kConsumers][R * T];
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t warp_in_cta = threadIdx.x >> 5;
    const uint32_t team_in_cta = warp_in_cta / W;
    const uint32_t warp_in_team = warp_in_cta % W;
    const uint64_t team = (uint64_t)blockIdx.x * kTeams + team_in_cta;
    const uint64_t teams = (uint64_t)gridDim.x * kTeams;
    const uint64_t token0 = (uint64_t)blockIdx.y * T;
    const uint32_t live = min((uint32_t)T, tokens - (uint32_t)token0);
    const uint64_t units = F::units(K);
    const uint64_t passes = (units + (uint64_t)W * UPL * 32 - 1) / ((uint64_t)W * UPL * 32);
    const uint64_t iterations = (rows + teams * R - 1) / (teams * R);
    pdl_launch_dependents();
    pdl_wait();

    typename F::Act held[REGS ? UPL : 1];
    if (REGS) {
#pragma unroll
        for (int j = 0; j < UPL; ++j) {
            const uint64_t u = ((uint64_t)warp_in_team * UPL + j) * 32 + lane;
            F::template load_act<GlobalMem>(act_global(act), K, token0, u < units ? u : units - 1, held[j]);
        }
    }

    for (uint64_t it = 0; it < iterations; ++it) {
        const uint64_t row0 = (it * teams + team) * R;
        float acc[R][T];
#pragma unroll
        for (int r = 0; r < R; ++r) {
#pragma unroll
            for (int t = 0; t < T; ++t) {
                acc[r][t] = 0.0f;
            }
        }
        for (uint64_t pass = 0; pass < passes; ++pass) {
            typename F::W wr[R][UPL];
            uint64_t u[UPL];
            bool valid[UPL];
#pragma unroll
            for (int j = 0; j < UPL; ++j) {
                const uint64_t unit = ((pass * W + warp_in_team) * UPL + j) * 32 + lane;
                valid[j] = unit < units;
                u[j] = valid[j] ? unit : units - 1;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    F::template load_w<GlobalMem>(w, K, min(row0 + r, rows - 1), u[j], lane, wr[r][j]);
                }
            }
#pragma unroll
            for (int j = 0; j < UPL; ++j) {
#pragma unroll
                for (int t = 0; t < T; ++t) {
                    typename F::Act loaded;
                    if (!REGS) {
                        F::template load_act<GlobalMem>(act_global(act), K, token0 + min((uint32_t)t, live - 1), u[j], loaded);
                    }
                    const typename F::Act &a = REGS ? held[j] : loaded;
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        int32_t *target = DUMP ? dump + ((token0 + t) * rows + min(row0 + r, rows - 1)) * dump_groups : nullptr;
                        F::template dot<DUMP>(wr[r][j], a, valid[j], u[j], lane, acc[r][t], target);
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
#pragma unroll
            for (int t = 0; t < T; ++t) {
                acc[r][t] = warp_sum(acc[r][t]);
            }
        }
        if (W == 1) {
            if (lane == 0) {
#pragma unroll
                for (int r = 0; r < R; ++r) {
#pragma unroll
                    for (int t = 0; t < T; ++t) {
                        if (row0 + r < rows && (uint32_t)t < live) {
                            store_result<true>(epilogue, y, token0 + t, out_stride, row0 + r, acc[r][t]);
                        }
                    }
                }
            }
        } else {
            const uint32_t buffer = (uint32_t)(it & 1);
            if (lane == 0) {
#pragma unroll
                for (int r = 0; r < R; ++r) {
#pragma unroll
                    for (int t = 0; t < T; ++t) {
                        partial[buffer][warp_in_cta][r * T + t] = acc[r][t];
                    }
                }
            }
            __syncthreads();
            if (warp_in_team == 0 && lane < R * T) {
                const uint32_t r = lane / T, t = lane % T;
                float total = partial[buffer][team_in_cta * W][lane];
#pragma unroll
                for (int k = 1; k < W; ++k) {
                    total += partial[buffer][team_in_cta * W + k][lane];
                }
                if (row0 + r < rows && t < live) {
                    store_result<true>(epilogue, y, token0 + t, out_stride, row0 + r, total);
                }
            }
        }
    }
    if (epilogue.signal_count != 0) {
        __syncthreads();
        if (threadIdx.x == 0) {
            signal_completion(epilogue);
        }
    }
}


template <class F, int T, int W, int UPL, int R, bool REGS, bool DUMP>
cudaError_t launch_team(const MatvecArgs &a, const WeightView &view, uint64_t dump_groups, cudaStream_t stream)
{
    constexpr int kTeams = kWarps / W;
    const uint64_t row_groups = (a.row_count + R - 1) / R;
    uint64_t ctas = (row_groups + kTeams - 1) / kTeams;
    // Persistent grid: exactly as many CTAs as the SMs can hold at once for this instantiation.
    // (the occupancy of an instantiation is the same on every device the library runs on: they are all sm_100)
    static std::atomic<int> resident{0};
    int blocks = resident.load(std::memory_order_relaxed);
    if (blocks == 0) {
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, matvec_xq8_team_kernel<F, T, W, UPL, R, REGS, DUMP>, team_warps(W) * 32, 0) !=
                cudaSuccess || blocks <= 0) {
            cudaGetLastError();
            blocks = 2;
        }
        resident.store(blocks, std::memory_order_relaxed);
    }
    const uint64_t cap = (uint64_t)sm_count(a.matrix->device) * blocks;
    if (ctas > cap) {
        ctas = cap;
    }
    const dim3 grid((unsigned)ctas, (unsigned)((a.tokens + T - 1) / T));
    return launch_kernel(matvec_xq8_team_kernel<F, T, W, UPL, R, REGS, DUMP>, grid, dim3(team_warps(W) * 32), 0, stream, view, a.act,
                         a.matrix->columns, a.row_count, (uint32_t)a.tokens, a.y, a.out_stride, a.fused, a.dump, dump_groups);
}

// ------------------------------------------------------------------------------------------------------
// Pipelined variant: the same team geometry and arithmetic, but the weights of a row group reach the CTA through
// a ring of shared-memory stages filled by bulk asynchronous copies (cp.async.bulk, completion on an mbarrier).
// One extra warp issues the copies; the eight consumer warps wait for a stage, pull their units into registers,
// hand the stage back, and compute. The copy engine keeps `stages` groups in flight per CTA whatever the
// consumers are doing, which is what an HBM-bound kernel needs. Every wait is bounded: when it gives up the
// kernel bumps the host-mapped fault word, stops waiting and still runs to completion (with wrong results).
// ------------------------------------------------------------------------------------------------------

constexpr int kMaxStages = 8;
constexpr uint64_t kWideBytes = 96ull << 20;  // matrices from this size on get the sixteen-warp CTA
constexpr uint32_t kSpinLimit = 1u << 22;
constexpr uint32_t kStageBudget = 100 * 1024;  // dynamic shared memory per CTA, so that two CTAs fit one SM

struct PipeSegment {
    WeightView global;     // plane bases at the first row of the segment
    const float *bias;     // by row of the segment, or null
    uint32_t rows;
    uint32_t first_group;  // index of the segment's first row group among the launch's
    uint64_t out_column;   // a result of row r goes to y[token * out_stride + out_column + r]
};

struct PipeArgs {
    WeightView global;            // plane bases at the first row of the call
    uint32_t plane_row_bytes[4];  // bytes of one row in each plane
    uint32_t plane_offset[4];     // offset of each plane inside a stage
    uint32_t planes, stages, stage_bytes;
    uint32_t act_bytes;           // shared memory reserved for in-kernel quantised activations (0 when not fused)
    // kSegments: the row ranges of the launch and their number, `groups` row groups in all. kPair: segments[0] is the
    // gate matrix, segments[1] the up matrix, whose rows sit pair_offset[k] behind the gate's in plane k of a stage.
    uint32_t segment_count, groups;
    uint32_t pair_offset[4];
    PipeSegment segments[3];
    // integer-dot hook: exact sub-block sums of row r go to dump[r * dump_groups ..]
    int32_t *dump;
    uint64_t dump_groups;
};

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait; false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity)
{
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) {
            return true;
        }
    }
    return false;
}
// Weights are read once per launch: mark their lines evict-first so activations and outputs stay in L2.
__device__ __forceinline__ uint64_t l2_evict_first_policy()
{
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar, uint64_t policy)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar), "l"(policy)
                 : "memory");
}
template <int THREADS>
__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(THREADS) : "memory"); }

// The sixteen-warp CTA has the SM to itself (no register cap).
__host__ __device__ constexpr bool roomy(int, int CW, bool) { return CW > kWarps; }
__host__ __device__ constexpr uint32_t stage_budget(int, bool) { return kStageBudget; }

// What one launch multiplies:
//   kSingle   - a row range of one matrix;
//   kSegments - up to three row ranges of matrices with the same encoding and width, each with its own bias and output
//               column (Q | K | V in one dispatch: MatmulArgs / MatmulSegment of the reference,
//               native/synapse-gpu/src/Features/GpuKernels/cuda/kernels/common.cuh:52-69, step/layers.rs:71-94);
//   kPair     - the same rows of a gate and an up matrix: a warp holds gate row r and up row r side by side and stores
//               silu(gate . x) * (up . x), so the gate values never go to memory (Qwen2GateUpWork,
//               src/Synapse.Runtime/Features/TextGeneration/Qwen2/Qwen2ProjectionWork.cs:91-131).
// Every row keeps the team shape and lane assignment it has in a launch of its own, so results are bit-identical.
enum : int { kSingle = 0, kSegments = 1, kPair = 2 };

__device__ __forceinline__ const PipeSegment &segment_at(const PipeArgs &p, uint32_t index)
{
    return index == 0 ? p.segments[0] : index == 1 ? p.segments[1] : p.segments[2];
}
// The segment that holds row group `group` of a kSegments launch.
__device__ __forceinline__ uint32_t segment_of(const PipeArgs &p, uint32_t group)
{
    return (p.segment_count > 1 && group >= p.segments[1].first_group ? 1u : 0u) + (p.segment_count > 2 && group >= p.segments[2].first_group ? 1u : 0u);
}

// CW = consumer warps the CTA is built for: 8 (two such CTAs fit one SM, so the next kernel of the stream can start
// copying while this one runs) or 16 (one CTA per SM: twice the rows in flight, which is what large matrices need to
// keep up with HBM).
template <class F, int T, int W, int UPL, int R, bool REGS, bool FUSED, int CW = kWarps, bool GATHER = false, int MODE = kSingle, bool DUMP = false>
__global__ void __launch_bounds__((CW / W) * W * 32 + 32, roomy(T, CW, FUSED) ? 1 : F::min_ctas(W))
matvec_xq8_pipe_kernel(PipeArgs p, ActView act, const float *__restrict__ x, uint64_t in_stride, uint64_t K, uint64_t rows, uint32_t tokens,
                       float *__restrict__ y, uint64_t out_stride, Epilogue epilogue, uint32_t *fault)
{
    static_assert(!REGS || T == 1, "register-resident activations are for single-token launches");
    static_assert(MODE != kPair || R == 2, "a pair launch holds one gate row and one up row per warp");
    static_assert(!DUMP || (T == 1 && MODE == kSingle), "the integer-dot hook is a single-token, single-matrix launch");
    constexpr int kTeams = CW / W;
    constexpr int kConsumers = kTeams * W;
    constexpr uint64_t G = MODE == kPair ? (uint64_t)kTeams : (uint64_t)kTeams * R;  // rows of one matrix per stage
    extern __shared__ __align__(128) uint8_t stage_memory[];
    __shared__ float partial[2][kConsumers][R * T];
    __shared__ __align__(8) uint64_t barriers[2 * kMaxStages];  // full[s] then empty[s]
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t warp_in_cta = threadIdx.x >> 5;
    const uint64_t groups = MODE == kSegments ? (uint64_t)p.groups : (rows + G - 1) / G;
    const uint64_t my_groups = groups > blockIdx.x ? (groups - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const uint32_t full0 = smem_u32(&barriers[0]), empty0 = smem_u32(&barriers[kMaxStages]);
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < p.stages; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, kConsumers);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_launch_dependents();
    // With in-kernel quantisation the first p.act_bytes of dynamic shared memory hold the activations.
    uint8_t *const ring = stage_memory + (FUSED ? p.act_bytes : 0);

    if (warp_in_cta == kConsumers) {
        // Producer warp: one lane streams this CTA's row groups into the ring.
        if (lane == 0) {
            const uint64_t policy = l2_evict_first_policy();
            // Calls `visit(source, bytes, offset inside the stage)` for every piece of row group `group`: one piece per
            // plane (two in a pair launch), cut out on 16-byte boundaries; returns the bytes of the group.
            auto pieces = [&](uint32_t group, auto visit) -> uint32_t {
                uint32_t total = 0;
                constexpr int kSources = MODE == kPair ? 2 : 1;
#pragma unroll
                for (int m = 0; m < kSources; ++m) {
                    uint32_t local = group;
                    uint64_t limit = rows;
                    const uint8_t *bases[4] = {p.global.p0, p.global.p1, p.global.p2, p.global.p3};
                    if (MODE != kSingle) {
                        const uint32_t index = MODE == kPair ? (uint32_t)m : segment_of(p, group);
                        const PipeSegment &segment = segment_at(p, index);
                        bases[0] = segment.global.p0;
                        bases[1] = segment.global.p1;
                        bases[2] = segment.global.p2;
                        bases[3] = segment.global.p3;
                        if (MODE == kSegments) {
                            local = group - segment.first_group;
                            limit = segment.rows;
                        }
                    }
                    const uint64_t row0 = (uint64_t)local * G;
                    const uint64_t n = min(G, limit - row0);
#pragma unroll
                    for (int k = 0; k < F::kPlanes; ++k) {
                        const uint8_t *source = bases[k] + row0 * p.plane_row_bytes[k];
                        const uint32_t shift = (uint32_t)(reinterpret_cast<uintptr_t>(source) & 15);
                        const uint32_t bytes = (uint32_t)((shift + n * p.plane_row_bytes[k] + 15) & ~(uint64_t)15);
                        visit(source - shift, bytes, p.plane_offset[k] + (uint32_t)m * p.pair_offset[k]);
                        total += bytes;
                    }
                }
                return total;
            };
            uint32_t s = 0, round = 0;  // ring slot and how many times the ring has wrapped
            for (uint32_t it = 0; it < my_groups; ++it) {
                if (round > 0 && !mbar_wait(empty0 + 8 * s, (round - 1) & 1) && fault) {
                    atomicAdd(fault, 1u);
                }
                const uint32_t group = blockIdx.x + it * gridDim.x;
                const uint32_t total = pieces(group, [](const uint8_t *, uint32_t, uint32_t) {});
                mbar_expect_tx(full0 + 8 * s, total);
                const uint32_t stage = smem_u32(ring) + s * p.stage_bytes;
                pieces(group, [&](const uint8_t *source, uint32_t bytes, uint32_t offset) { bulk_copy(stage + offset, source, bytes, full0 + 8 * s, policy); });
                if (++s == p.stages) {
                    s = 0;
                    ++round;
                }
            }
        }
        return;
    }

    const uint32_t team_in_cta = warp_in_cta / W;
    const uint32_t warp_in_team = warp_in_cta % W;
    const uint64_t token0 = (uint64_t)blockIdx.y * T;
    const uint32_t live = min((uint32_t)T, tokens - (uint32_t)token0);
    const uint64_t units = F::units(K);
    // Register-resident activations imply a single pass over the row (the launcher guarantees it).
    const uint32_t passes = REGS ? 1u : (uint32_t)((units + (uint64_t)W * UPL * 32 - 1) / ((uint64_t)W * UPL * 32));

    // Weights do not depend on earlier kernels (the producer is already copying them); activations and outputs do.
    pdl_wait();
    ActShared shared_act;
    if (FUSED) {
        const uint32_t base = smem_u32(stage_memory);
        shared_act.codes = base;
        shared_act.scales = base + shared_act_codes_bytes(T, (uint32_t)K);
        shared_act.sums = shared_act.scales + shared_act_side_bytes(T, (uint32_t)K);
        quantize_to_shared<T>(x + token0 * in_stride, in_stride, (uint32_t)K, live, warp_in_cta, kConsumers, lane, shared_act);
        consumer_barrier<kConsumers * 32>();
    }
    typename F::Act held[REGS ? UPL : 1];
    if (REGS) {
#pragma unroll
        for (int j = 0; j < UPL; ++j) {
            const uint64_t u = ((uint64_t)warp_in_team * UPL + j) * 32 + lane;
            if (FUSED) {
                F::template load_act<SharedMem>(shared_act, K, 0, u < units ? u : units - 1, held[j]);
            } else {
                F::template load_act<GlobalMem>(act_global(act), K, token0, u < units ? u : units - 1, held[j]);
            }
        }
    }

    uint32_t s = 0, phase = 0;
    for (uint32_t it = 0; it < my_groups; ++it) {
        // Where this group's rows come from, how many there are, and where their results go.
        uint32_t local = blockIdx.x + it * gridDim.x;
        uint64_t limit = rows, column = 0;
        const uint8_t *bases[2][4] = {{p.global.p0, p.global.p1, p.global.p2, p.global.p3}, {nullptr, nullptr, nullptr, nullptr}};
        Epilogue e = epilogue;
        if (MODE == kSegments) {
            const PipeSegment &segment = segment_at(p, segment_of(p, local));
            local -= segment.first_group;
            limit = segment.rows;
            column = segment.out_column;
            bases[0][0] = segment.global.p0;
            bases[0][1] = segment.global.p1;
            bases[0][2] = segment.global.p2;
            bases[0][3] = segment.global.p3;
            e.bias = segment.bias ? segment.bias - column : nullptr;  // store_result indexes the bias with the output column
        } else if (MODE == kPair) {
#pragma unroll
            for (int m = 0; m < 2; ++m) {
                bases[m][0] = p.segments[m].global.p0;
                bases[m][1] = p.segments[m].global.p1;
                bases[m][2] = p.segments[m].global.p2;
                bases[m][3] = p.segments[m].global.p3;
            }
        }
        const uint64_t group_row0 = (uint64_t)local * G;
        // first row of this team: R consecutive rows, or in a pair launch the same row of both matrices
        const uint64_t row0 = group_row0 + (uint64_t)team_in_cta * (MODE == kPair ? 1 : R);
        if (!mbar_wait(full0 + 8 * s, phase) && fault && lane == 0) {
            atomicAdd(fault, 1u);
        }
        // The stage holds rows [group_row0, +G) of every plane with the plane's own row pitch; a plane whose rows
        // are not 16-byte multiples starts `shift` bytes into its slot. A pair launch has two such sets of rows.
        SharedView views[MODE == kPair ? 2 : 1];
        {
            const uint32_t stage = smem_u32(ring) + s * p.stage_bytes;
#pragma unroll
            for (int m = 0; m < (MODE == kPair ? 2 : 1); ++m) {
                uint32_t local_base[4] = {0, 0, 0, 0};
#pragma unroll
                for (int k = 0; k < F::kPlanes; ++k) {
                    const uint32_t shift = (uint32_t)(reinterpret_cast<uintptr_t>(bases[m][k] + group_row0 * p.plane_row_bytes[k]) & 15);
                    local_base[k] = stage + p.plane_offset[k] + (uint32_t)m * p.pair_offset[k] + shift;
                }
                views[m].row_bytes = p.plane_row_bytes[0];
                views[m].p0 = local_base[0];
                views[m].p1 = local_base[1];
                views[m].p2 = local_base[2];
                views[m].p3 = local_base[3];
            }
        }
        float acc[R][T];
#pragma unroll
        for (int r = 0; r < R; ++r) {
#pragma unroll
            for (int t = 0; t < T; ++t) {
                acc[r][t] = 0.0f;
            }
        }
        uint32_t release_slot = 0;
        for (uint32_t pass = 0; pass < passes; ++pass) {
            typename F::W wr[R][UPL];
            uint64_t u[UPL];
            bool valid[UPL];
#pragma unroll
            for (int j = 0; j < UPL; ++j) {
                const uint64_t unit = (((uint64_t)pass * W + warp_in_team) * UPL + j) * 32 + lane;
                valid[j] = unit < units;
                u[j] = valid[j] ? unit : units - 1;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    if (MODE == kPair) {
                        F::template load_w<SharedMem>(views[MODE == kPair ? r : 0], K, (uint64_t)team_in_cta, u[j], lane, wr[r][j]);
                    } else {
                        F::template load_w<SharedMem>(views[0], K, (uint64_t)team_in_cta * R + r, u[j], lane, wr[r][j]);
                    }
                }
            }
            if (pass + 1 == passes) {
                // Every unit of this warp is in registers (or on its way there): the stage is released below.
                release_slot = s;
                if (++s == p.stages) {
                    s = 0;
                    phase ^= 1;
                }
            }
#pragma unroll
            for (int j = 0; j < UPL; ++j) {
#pragma unroll
                for (int t = 0; t < T; ++t) {
                    typename F::Act loaded;
                    if (!REGS) {
                        if (FUSED) {
                            F::template load_act<SharedMem>(shared_act, K, (uint32_t)t, u[j], loaded);
                        } else {
                            F::template load_act<GlobalMem>(act_global(act), K, token0 + min((uint32_t)t, live - 1), u[j], loaded);
                        }
                    }
                    const typename F::Act &a = REGS ? held[j] : loaded;
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        // rows past the end of the matrix hold whatever the stage held before: they are computed and
                        // dropped, but must not reach the integer-dot hook
                        int32_t *target = DUMP ? p.dump + min(row0 + r, rows - 1) * p.dump_groups : nullptr;
                        F::template dot<DUMP>(wr[r][j], a, valid[j] && (!DUMP || row0 + r < limit), u[j], lane, acc[r][t], target);
                    }
                }
            }
        }
        // Give the stage back to the producer. The bulk copy that refills it writes through the asynchronous proxy, the
        // loads above read through the generic one: the proxy fence orders the two (without it nothing says that a
        // load still in flight is performed before the refill lands). Doing this after the dot products, when the loaded
        // registers have been consumed, makes the fence free; releasing right after the loads was measured no faster.
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
            mbar_arrive(empty0 + 8 * release_slot);
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
#pragma unroll
            for (int t = 0; t < T; ++t) {
                acc[r][t] = warp_sum(acc[r][t]);
            }
        }
        if (W == 1) {
            if (lane == 0) {
                if (MODE == kPair) {
#pragma unroll
                    for (int t = 0; t < T; ++t) {
                        if (row0 < limit && (uint32_t)t < live) {
                            const float g = acc[0][t];
                            store_result<GATHER>(e, y, token0 + t, out_stride, row0, g / (1.0f + expf(-g)) * acc[1][t]);
                        }
                    }
                } else {
#pragma unroll
                    for (int r = 0; r < R; ++r) {
#pragma unroll
                        for (int t = 0; t < T; ++t) {
                            if (row0 + r < limit && (uint32_t)t < live) {
                                store_result<GATHER>(e, y, token0 + t, out_stride, column + row0 + r, acc[r][t]);
                            }
                        }
                    }
                }
            }
        } else {
            const uint32_t buffer = it & 1;
            if (lane == 0) {
#pragma unroll
                for (int r = 0; r < R; ++r) {
#pragma unroll
                    for (int t = 0; t < T; ++t) {
                        partial[buffer][warp_in_cta][r * T + t] = acc[r][t];
                    }
                }
            }
            consumer_barrier<kConsumers * 32>();
            if (MODE == kPair) {
                if (warp_in_team == 0 && lane < T) {
                    float g = partial[buffer][team_in_cta * W][lane], up = partial[buffer][team_in_cta * W][T + lane];
#pragma unroll
                    for (int k = 1; k < W; ++k) {
                        g += partial[buffer][team_in_cta * W + k][lane];
                        up += partial[buffer][team_in_cta * W + k][T + lane];
                    }
                    if (row0 < limit && lane < live) {
                        store_result<GATHER>(e, y, token0 + lane, out_stride, row0, g / (1.0f + expf(-g)) * up);
                    }
                }
            } else if (warp_in_team == 0 && lane < R * T) {
                const uint32_t r = lane / T, t = lane % T;
                float total = partial[buffer][team_in_cta * W][lane];
#pragma unroll
                for (int k = 1; k < W; ++k) {
                    total += partial[buffer][team_in_cta * W + k][lane];
                }
                if (row0 + r < limit && t < live) {
                    store_result<GATHER>(e, y, token0 + t, out_stride, column + row0 + r, total);
                }
            }
        }
    }
    if (GATHER) {
        // every consumer warp of the CTA has stored its last result (the producer warp left long ago)
        consumer_barrier<kConsumers * 32>();
        if (threadIdx.x == 0) {
            signal_completion(epilogue);
        }
    }
}

// ------------------------------------------------------------------------------------------------------
// Several tokens per launch (batched decode, speculative verification, short prompt runs): the tokens of a group are
// spread over the warp teams of the CTA instead of being looped over inside a warp. A team keeps ITS token's slice of
// the quantised activations in registers for the whole launch -- exactly as the single-token kernel does -- and walks
// the rows of every weight stage: a row costs five shared-memory loads and the dot products, nothing is re-unpacked or
// re-loaded per token, and every weight byte still crosses HBM once per token group. With `tp` tokens in the group and
// kTeams teams, kTeams / tp teams share a token and split the rows of a stage between them. A row's summation order is
// that of a launch of its own (it depends on W and UPL only), so batched results are bit-identical to single-token ones.
// ------------------------------------------------------------------------------------------------------
constexpr int kTokenWarps = 16;       // consumer warps of these CTAs (one CTA per SM)
constexpr uint32_t kTokenStageRows = 16;

template <class F, int W, int UPL, bool GATHER>
__global__ void __launch_bounds__((kTokenWarps / W) * W * 32 + 32, 1)
matvec_xq8_tokens_kernel(PipeArgs p, ActView act, uint64_t K, uint64_t rows, uint32_t tokens, uint32_t tp, float *__restrict__ y, uint64_t out_stride,
                         Epilogue epilogue, uint32_t *fault)
{
    constexpr int kTeams = kTokenWarps / W;
    constexpr int kConsumers = kTeams * W;
    constexpr uint32_t G = kTokenStageRows;
    extern __shared__ __align__(128) uint8_t stage_memory[];
    __shared__ float partial[2][G][kConsumers];
    __shared__ __align__(8) uint64_t barriers[2 * kMaxStages];  // full[s] then empty[s]
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t warp_in_cta = threadIdx.x >> 5;
    const uint64_t groups = (rows + G - 1) / G;
    const uint64_t my_groups = groups > blockIdx.x ? (groups - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const uint32_t full0 = smem_u32(&barriers[0]), empty0 = smem_u32(&barriers[kMaxStages]);
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < p.stages; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, kConsumers);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_launch_dependents();
    const uint8_t *const bases[4] = {p.global.p0, p.global.p1, p.global.p2, p.global.p3};

    if (warp_in_cta == kConsumers) {
        if (lane == 0) {
            const uint64_t policy = l2_evict_first_policy();
            uint32_t s = 0, round = 0;
            for (uint32_t it = 0; it < my_groups; ++it) {
                if (round > 0 && !mbar_wait(empty0 + 8 * s, (round - 1) & 1) && fault) {
                    atomicAdd(fault, 1u);
                }
                const uint64_t row0 = ((uint64_t)blockIdx.x + (uint64_t)it * gridDim.x) * G;
                const uint64_t n = min((uint64_t)G, rows - row0);
                uint32_t total = 0, bytes[4];
                const uint8_t *sources[4];
#pragma unroll
                for (int k = 0; k < F::kPlanes; ++k) {
                    const uint8_t *source = bases[k] + row0 * p.plane_row_bytes[k];
                    const uint32_t shift = (uint32_t)(reinterpret_cast<uintptr_t>(source) & 15);
                    sources[k] = source - shift;
                    bytes[k] = (uint32_t)((shift + n * p.plane_row_bytes[k] + 15) & ~(uint64_t)15);
                    total += bytes[k];
                }
                mbar_expect_tx(full0 + 8 * s, total);
                const uint32_t stage = smem_u32(stage_memory) + s * p.stage_bytes;
#pragma unroll
                for (int k = 0; k < F::kPlanes; ++k) {
                    bulk_copy(stage + p.plane_offset[k], sources[k], bytes[k], full0 + 8 * s, policy);
                }
                if (++s == p.stages) {
                    s = 0;
                    ++round;
                }
            }
        }
        return;
    }

    const uint32_t team_in_cta = warp_in_cta / W;
    const uint32_t warp_in_team = warp_in_cta % W;
    const uint32_t sharers = kTeams / tp;                 // teams that share a token (tp <= kTeams)
    const uint32_t token_slot = team_in_cta % tp;         // which token of the group this team multiplies
    const uint32_t row_lane = team_in_cta / tp;           // which share of a stage's rows it takes
    const uint64_t token0 = (uint64_t)blockIdx.y * tp;
    const uint32_t live = min(tp, tokens - (uint32_t)token0);
    const bool working = row_lane < sharers && token_slot < live;
    const uint64_t token = token0 + min(token_slot, live - 1);
    const uint64_t units = F::units(K);

    pdl_wait();
    typename F::Act held[UPL];
    uint64_t u[UPL];
    bool valid[UPL];
#pragma unroll
    for (int j = 0; j < UPL; ++j) {
        const uint64_t unit = ((uint64_t)warp_in_team * UPL + j) * 32 + lane;
        valid[j] = unit < units;
        u[j] = valid[j] ? unit : units - 1;
        F::template load_act<GlobalMem>(act_global(act), K, token, u[j], held[j]);
    }

    uint32_t s = 0, phase = 0;
    for (uint32_t it = 0; it < my_groups; ++it) {
        const uint64_t group_row0 = ((uint64_t)blockIdx.x + (uint64_t)it * gridDim.x) * G;
        if (!mbar_wait(full0 + 8 * s, phase) && fault && lane == 0) {
            atomicAdd(fault, 1u);
        }
        SharedView view;
        view.row_bytes = p.plane_row_bytes[0];
        {
            const uint32_t stage = smem_u32(stage_memory) + s * p.stage_bytes;
            uint32_t local[4] = {0, 0, 0, 0};
#pragma unroll
            for (int k = 0; k < F::kPlanes; ++k) {
                const uint32_t shift = (uint32_t)(reinterpret_cast<uintptr_t>(bases[k] + group_row0 * p.plane_row_bytes[k]) & 15);
                local[k] = stage + p.plane_offset[k] + shift;
            }
            view.p0 = local[0];
            view.p1 = local[1];
            view.p2 = local[2];
            view.p3 = local[3];
        }
        const uint32_t buffer = it & 1;
        if (working) {
            for (uint32_t row = row_lane; row < G; row += sharers) {
                if (group_row0 + row >= rows) {
                    break;  // rows past the end of the matrix: the stage holds nothing for them
                }
                typename F::W wr[UPL];
#pragma unroll
                for (int j = 0; j < UPL; ++j) {
                    F::template load_w<SharedMem>(view, K, (uint64_t)row, u[j], lane, wr[j]);
                }
                float acc = 0.0f;
#pragma unroll
                for (int j = 0; j < UPL; ++j) {
                    F::template dot<false>(wr[j], held[j], valid[j], u[j], lane, acc, nullptr);
                }
                acc = warp_sum(acc);
                if (W == 1) {
                    if (lane == 0) {
                        store_result<GATHER>(epilogue, y, token, out_stride, group_row0 + row, acc);
                    }
                } else if (lane == 0) {
                    partial[buffer][row][warp_in_cta] = acc;
                }
            }
        }
        // Give the stage back (see the single-token kernel for the fence).
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
            mbar_arrive(empty0 + 8 * s);
        }
        if (++s == p.stages) {
            s = 0;
            phase ^= 1;
        }
        if (W > 1) {
            // the team's warps in index order, as in every other kernel; one thread per (row, token) of the stage
            consumer_barrier<kConsumers * 32>();
            const uint32_t pairs = G * live;
            for (uint32_t index = threadIdx.x; index < pairs; index += kConsumers * 32) {
                const uint32_t row = index / live, slot = index % live;
                if (group_row0 + row < rows) {
                    // the team that computed (row, slot): its row lane is row % sharers
                    const uint32_t team = (row % sharers) * tp + slot;
                    float total = partial[buffer][row][team * W];
#pragma unroll
                    for (int k = 1; k < W; ++k) {
                        total += partial[buffer][row][team * W + k];
                    }
                    store_result<GATHER>(epilogue, y, token0 + slot, out_stride, group_row0 + row, total);
                }
            }
        }
    }
    if (GATHER) {
        consumer_barrier<kConsumers * 32>();
        if (threadIdx.x == 0) {
            signal_completion(epilogue);
        }
    }
}

// Lays out a stage for this format and row length; false when a group of rows does not fit the stage budget.
// `views` holds one view per segment of the launch (one for a plain product).
template <class F, int W, int R, int CW = kWarps>
bool plan_pipe(const MatvecArgs &a, const WeightView *views, uint32_t act_bytes, PipeArgs &p, uint32_t budget = kStageBudget, int mode = kSingle)
{
    constexpr uint64_t kTeams = CW / W;
    const uint64_t G = mode == kPair ? kTeams : kTeams * R;  // rows of one matrix per stage
    p = PipeArgs{};
    p.global = views[0];
    p.planes = F::kPlanes;
    F::plane_row_bytes(a.matrix->columns, a.matrix->row_bytes, p.plane_row_bytes);
    uint64_t offset = 0;
    for (int k = 0; k < F::kPlanes; ++k) {
        p.plane_offset[k] = (uint32_t)offset;
        const uint64_t slot = align_up(G * p.plane_row_bytes[k] + 16, 128);
        p.pair_offset[k] = mode == kPair ? (uint32_t)slot : 0u;
        offset += mode == kPair ? 2 * slot : slot;
    }
    for (int k = F::kPlanes; k < 4; ++k) {
        p.plane_offset[k] = 0;
        p.plane_row_bytes[k] = 0;
    }
    if (act_bytes >= budget || offset > (budget - act_bytes) / 2) {
        return false;
    }
    p.act_bytes = act_bytes;
    p.stage_bytes = (uint32_t)offset;
    uint64_t stages = (budget - act_bytes) / offset;
    p.stages = (uint32_t)(stages > kMaxStages ? kMaxStages : stages);
    p.groups = (uint32_t)((a.row_count + G - 1) / G);
    if (mode != kSingle) {
        p.segment_count = a.segment_count;
        uint64_t groups = 0;
        for (uint32_t i = 0; i < a.segment_count; ++i) {
            PipeSegment &segment = p.segments[i];
            segment.global = views[i];
            segment.bias = a.segments[i].bias;
            segment.rows = (uint32_t)a.segments[i].row_count;
            segment.out_column = a.segments[i].out_column;
            segment.first_group = (uint32_t)groups;
            groups += (a.segments[i].row_count + G - 1) / G;
        }
        if (mode == kSegments) {
            p.groups = (uint32_t)groups;
        }
    }
    p.dump = a.dump;
    return true;
}

// Device attributes of a kernel (its dynamic shared-memory limit) are per device: `first_use` is true once per
// device for the object it is called on, from whichever thread gets there first.
struct PerDevice {
    std::atomic<uint64_t> seen{0};
    bool first_use(int device)
    {
        const uint64_t bit = 1ull << (device & 63);
        return (seen.fetch_or(bit) & bit) == 0;
    }
    void forget(int device) { seen.fetch_and(~(1ull << (device & 63))); }
};

template <class F, int T, int W, int UPL, int R, bool REGS, bool FUSED, int CW = kWarps, bool GATHER = false, int MODE = kSingle, bool DUMP = false>
cudaError_t launch_pipe(const MatvecArgs &a, const PipeArgs &p, cudaStream_t stream)
{
    auto kernel = matvec_xq8_pipe_kernel<F, T, W, UPL, R, REGS, FUSED, CW, GATHER, MODE, DUMP>;
    const uint32_t dynamic = p.act_bytes + p.stages * p.stage_bytes;
    static PerDevice configured;
    if (configured.first_use(a.matrix->device)) {
        cudaError_t error = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)stage_budget(T, FUSED));
        if (error != cudaSuccess) {
            configured.forget(a.matrix->device);
            return error;
        }
    }
    // F::kCtasPerSm CTAs per SM. Where that is one, the kernel is still built so that two fit (registers and
    // shared memory): the second slot is for the next kernel of the stream, which starts copying its first stages
    // while this one is still running.
    uint64_t ctas = p.groups;
    // A launch of several row ranges, or of a gate/up pair, fills both CTA slots of every SM: it stands for the two or three
    // launches that otherwise run side by side on parallel branches (measured on the 2 x 38 MB gate | up pair: 15.9 us with
    // two CTAs per SM, 17.2 us with one).
    // So does a matrix small enough that two CTAs per SM leave every CTA a single row group (7 MB projections: one
    // stage per CTA instead of two one after the other).
    const uint64_t sms = (uint64_t)sm_count(a.matrix->device);
    const uint64_t cap = sms * (roomy(T, CW, FUSED) ? 1 : (MODE != kSingle || p.groups <= 2 * sms) ? 2 : F::ctas_per_sm(W));
    if (ctas > cap) {
        ctas = cap;
    }
    const dim3 grid((unsigned)ctas, (unsigned)((a.tokens + T - 1) / T));
    return launch_kernel(kernel, grid, dim3((CW / W) * W * 32 + 32), dynamic, stream, p, a.act, a.x, a.in_stride, a.matrix->columns, a.row_count,
                         (uint32_t)a.tokens, a.y, a.out_stride, a.fused, fault_word_device());
}

// The token-parallel kernel on `a.tokens` >= 2 ready-made activations; cudaErrorNotSupported when a stage of
// kTokenStageRows rows does not fit.
template <class F, int W, int UPL, bool GATHER>
cudaError_t launch_token_teams(const MatvecArgs &a, const WeightView &view, cudaStream_t stream)
{
    constexpr uint32_t kTeams = kTokenWarps / W;
    constexpr uint32_t kBudget = 200u * 1024u;
    PipeArgs p{};
    p.global = view;
    p.planes = F::kPlanes;
    F::plane_row_bytes(a.matrix->columns, a.matrix->row_bytes, p.plane_row_bytes);
    uint64_t offset = 0;
    for (int k = 0; k < F::kPlanes; ++k) {
        p.plane_offset[k] = (uint32_t)offset;
        offset += align_up((uint64_t)kTokenStageRows * p.plane_row_bytes[k] + 16, 128);
    }
    if (offset > kBudget / 2) {
        return cudaErrorNotSupported;
    }
    p.stage_bytes = (uint32_t)offset;
    const uint64_t stages = kBudget / offset;
    p.stages = (uint32_t)(stages > kMaxStages ? kMaxStages : stages);
    auto kernel = matvec_xq8_tokens_kernel<F, W, UPL, GATHER>;
    static PerDevice configured;
    if (configured.first_use(a.matrix->device)) {
        cudaError_t error = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kBudget);
        if (error != cudaSuccess) {
            configured.forget(a.matrix->device);
            return error;
        }
    }
    // Tokens per group: as many as there are teams at most; fewer tokens leave several teams per token, which split the rows.
    const uint32_t tp = (uint32_t)(a.tokens < kTeams ? a.tokens : kTeams);
    uint64_t ctas = (a.row_count + kTokenStageRows - 1) / kTokenStageRows;
    const uint64_t cap = (uint64_t)sm_count(a.matrix->device);
    if (ctas > cap) {
        ctas = cap;
    }
    const dim3 grid((unsigned)ctas, (unsigned)((a.tokens + tp - 1) / tp));
    return launch_kernel(kernel, grid, dim3(kTeams * W * 32 + 32), (size_t)p.stages * p.stage_bytes, stream, p, a.act, a.matrix->columns, a.row_count,
                         (uint32_t)a.tokens, tp, a.y, a.out_stride, a.fused, fault_word_device());
}

// Q4_K and planar Q6_K with 2..8 tokens on the integer tensor cores (matvec_mma.cuh); cudaErrorNotSupported for the
// other formats and when the row is too long for two tokens' activations and two stages to fit shared memory.
template <class F, bool GATHER>
cudaError_t launch_tensor_core_tokens(const MatvecArgs &a, const WeightView &view, uint32_t upl, cudaStream_t stream);

template <class F, int W, int UPL>
cudaError_t launch_tokens(const MatvecArgs &a, const WeightView *views, bool one_pass, uint64_t dump_groups, cudaStream_t stream)
{
    constexpr int R = F::kRows;
    const WeightView &view = views[0];
    PipeArgs pipe;
    if (a.dump) {
        // The integer-dot hook: token by token through the very kernel variant a single-token product of this matrix
        // takes (built with the hook compiled in), so that the sums come out of the code that is timed.
        const uint64_t K = a.matrix->columns;
        for (uint64_t t = 0; t < a.tokens; ++t) {
            MatvecArgs one = a;
            one.tokens = 1;
            one.act.codes = a.act.codes + t * K;
            one.act.scales = a.act.scales + t * (K / 32);
            one.act.sums = a.act.sums + t * (K / 16);
            one.y = a.y + t * a.out_stride;
            one.dump = a.dump + t * a.row_count * dump_groups;
            cudaError_t error;
            if (one_pass && a.row_count * a.matrix->row_bytes >= kWideBytes && plan_pipe<F, W, 1, 2 * kWarps>(one, views, 0, pipe)) {
                pipe.dump_groups = dump_groups;
                error = launch_pipe<F, 1, W, UPL, 1, true, false, 2 * kWarps, false, kSingle, true>(one, pipe, stream);
            } else if (one_pass && plan_pipe<F, W, R>(one, views, 0, pipe)) {
                pipe.dump_groups = dump_groups;
                error = launch_pipe<F, 1, W, UPL, R, true, false, kWarps, false, kSingle, true>(one, pipe, stream);
            } else {
                error = launch_team<F, 1, W, UPL, 1, false, true>(one, view, dump_groups, stream);
            }
            if (error != cudaSuccess) {
                return error;
            }
        }
        return cudaSuccess;
    }
    const uint32_t K32 = (uint32_t)a.matrix->columns;
    const bool gather = a.fused.peer_count != 0 || a.fused.signal_count != 0;
    if (a.form != kSingle) {
        // Several row ranges, or a gate/up pair, in one launch: single-token products on ready-made activations whose
        // rows one pass of the team covers. Anything else is refused here and runs as separate launches.
        if (a.tokens != 1 || !one_pass || !a.act_ready || !plan_pipe<F, W, R>(a, views, 0, pipe, kStageBudget, (int)a.form)) {
            return cudaErrorNotSupported;
        }
        if constexpr (R == 2) {
            if (a.form == kPair) {
                return gather ? launch_pipe<F, 1, W, UPL, R, true, false, kWarps, true, kPair>(a, pipe, stream)
                              : launch_pipe<F, 1, W, UPL, R, true, false, kWarps, false, kPair>(a, pipe, stream);
            }
        }
        if (a.form == kSegments) {
            return gather ? launch_pipe<F, 1, W, UPL, R, true, false, kWarps, true, kSegments>(a, pipe, stream)
                          : launch_pipe<F, 1, W, UPL, R, true, false, kWarps, false, kSegments>(a, pipe, stream);
        }
        return cudaErrorNotSupported;
    }
    // Products that also store into peer copies of the output: one pipelined variant (single token, one pass, ready
    // activations); every other shape takes the direct-load kernel below, whose epilogue handles peers at run time.
    if (gather && a.tokens <= 1 && one_pass && a.act_ready && a.row_count * a.matrix->row_bytes >= kWideBytes &&
        plan_pipe<F, W, 1, 2 * kWarps>(a, views, 0, pipe)) {
        return launch_pipe<F, 1, W, UPL, 1, true, false, 2 * kWarps, true>(a, pipe, stream);  // shards of 96 MB and more
    }
    if (gather && a.tokens <= 1 && one_pass && a.act_ready && plan_pipe<F, W, R>(a, views, 0, pipe)) {
        return launch_pipe<F, 1, W, UPL, R, true, false, kWarps, true>(a, pipe, stream);
    }
    if (!gather && a.tokens <= 1 && !a.act_ready && plan_pipe<F, W, R>(a, views, shared_act_bytes(1, K32), pipe)) {
        // FP32 activations in: the kernel quantises them itself.
        return one_pass ? launch_pipe<F, 1, W, UPL, R, true, true>(a, pipe, stream) : launch_pipe<F, 1, W, UPL, R, false, true>(a, pipe, stream);
    }
    if (!a.act_ready) {
        // Shapes the pipelined kernel does not quantise for: quantise into the caller's scratch first.
        cudaError_t error = launch_quantize(a.x, a.tokens, a.matrix->columns, a.in_stride, const_cast<int8_t *>(a.act.codes),
                                            const_cast<float *>(a.act.scales), const_cast<int16_t *>(a.act.sums), stream);
        if (error != cudaSuccess) {
            return error;
        }
    }
    if (std::is_same<F, Q6KPlanarXq8>::value && a.tokens == 2 && one_pass && !gather && W >= 3) {
        // Two tokens of long Q6_K rows: the tensor-core kernel's time does not depend on the token count (34 us for
        // 3584 x 18944 at 2 to 8 tokens), the single-token kernel runs at the memory rate (12 us): two of those are
        // cheaper, and the bits are the same either way.
        for (uint64_t t = 0; t < 2; ++t) {
            MatvecArgs one = a;
            one.tokens = 1;
            one.act_ready = true;
            one.act.codes = a.act.codes + t * a.matrix->columns;
            one.act.scales = a.act.scales + t * (a.matrix->columns / 32);
            one.act.sums = a.act.sums + t * (a.matrix->columns / 16);
            one.x = a.x ? a.x + t * a.in_stride : nullptr;
            one.y = a.y + t * a.out_stride;
            one.fused.gate = a.fused.gate ? a.fused.gate + t * a.fused.gate_stride : nullptr;
            const cudaError_t error = launch_tokens<F, W, UPL>(one, views, one_pass, dump_groups, stream);
            if (error != cudaSuccess) {
                return error;
            }
        }
        return cudaSuccess;
    }
    if (a.tokens >= 2 && one_pass) {
        // Several tokens of a K-quant: exact integer dots of 16 rows x 8 tokens per tensor-core instruction.
        const cudaError_t error = gather ? launch_tensor_core_tokens<F, true>(a, view, UPL, stream) : launch_tensor_core_tokens<F, false>(a, view, UPL, stream);
        if (error != cudaErrorNotSupported) {
            return error;
        }
    }
    // (rows so long that the sixteen warps form fewer teams than there are tokens would need several passes over the
    // weights: those keep the direct-load kernels, which loop over the tokens inside a warp)
    if (F::kTokenTeams && a.tokens >= 2 && one_pass && (uint64_t)(kTokenWarps / W) >= (a.tokens < 8 ? a.tokens : 8)) {
        // Several tokens: one team of warps per token, every team with its token's activations in registers.
        const cudaError_t error = gather ? launch_token_teams<F, W, UPL, true>(a, view, stream) : launch_token_teams<F, W, UPL, false>(a, view, stream);
        if (error != cudaErrorNotSupported) {
            return error;
        }
    }
    // Very large matrices (the vocabulary projection): sixteen consumer warps, one row each (the same summation order:
    // it depends on W and UPL only). Measured on Q4_K: 306 MB in 47.2 against 52.7 us, 153 MB in 25.4 against 30.7 us.
    // A 38 MB projection gains 4 % alone but loses more inside a decode step, where the eight-warp CTAs of two
    // kernels share an SM (parallel branches, and the next kernel's first copies).
    if (!gather && a.tokens <= 1 && one_pass && a.row_count * a.matrix->row_bytes >= kWideBytes && plan_pipe<F, W, 1, 2 * kWarps>(a, views, 0, pipe)) {
        return launch_pipe<F, 1, W, UPL, 1, true, false, 2 * kWarps>(a, pipe, stream);
    }
    if (!gather && a.tokens <= 1 && plan_pipe<F, W, R>(a, views, 0, pipe)) {
        return one_pass ? launch_pipe<F, 1, W, UPL, R, true, false>(a, pipe, stream) : launch_pipe<F, 1, W, UPL, R, false, false>(a, pipe, stream);
    }
    // Token group size: the smallest of 1, 2, 4, 8 that holds the tokens (step/projection.rs:82-87).
    if (a.tokens <= 1) {
        return one_pass ? launch_team<F, 1, W, UPL, R, true, false>(a, view, 0, stream)
                        : launch_team<F, 1, W, UPL, R, false, false>(a, view, 0, stream);
    }
    if (a.tokens == 2) {
        return launch_team<F, 2, W, UPL, R, false, false>(a, view, 0, stream);
    }
    if (a.tokens <= 4) {
        return launch_team<F, 4, W, UPL, R, false, false>(a, view, 0, stream);
    }
    return launch_team<F, 8, W, UPL, 1, false, false>(a, view, 0, stream);
}

// Team shape from the row length alone: the fewest warps that cover the row in one pass with F::kMaxUpl units per
// lane (one unit per lane when the row is short enough); eight warps making several passes for very long rows.
template <class F>
cudaError_t launch_format(const MatvecArgs &a, const WeightView *views, uint64_t units, uint64_t dump_groups, cudaStream_t stream)
{
    constexpr int U = F::kMaxUpl;
    if (units <= 32) {
        return launch_tokens<F, 1, 1>(a, views, true, dump_groups, stream);
    }
    switch ((units + 32 * U - 1) / (32 * U)) {
    case 1: return launch_tokens<F, 1, U>(a, views, true, dump_groups, stream);
    case 2: return launch_tokens<F, 2, U>(a, views, true, dump_groups, stream);
    case 3: return launch_tokens<F, 3, U>(a, views, true, dump_groups, stream);
    case 4: return launch_tokens<F, 4, U>(a, views, true, dump_groups, stream);
    case 5: return launch_tokens<F, 5, U>(a, views, true, dump_groups, stream);
    case 6: return launch_tokens<F, 6, U>(a, views, true, dump_groups, stream);
    case 7: return launch_tokens<F, 7, U>(a, views, true, dump_groups, stream);
    case 8: return launch_tokens<F, 8, U>(a, views, true, dump_groups, stream);
    default: return launch_tokens<F, 8, U>(a, views, false, dump_groups, stream);
    }
}

}  // namespace mv
}  // namespace syn

#include "matvec_mma.cuh"
