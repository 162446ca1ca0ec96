// A single-token decode step as ONE persistent kernel.
//
// Launching a kernel per operation leaves the memory system idle around every launch: a 38 MB projection streams in
// about 5 us but costs 9 us as its own kernel. Here one cooperative grid (one CTA per SM) walks a list of operations
// ("the program") built once per model:
//
//   * the producer warp of each CTA streams the CTA's share of EVERY projection's weights, in program order, through
//     a shared-memory ring with bulk copies. Weights depend on nothing, so the producer never waits for an operation
//     to finish, only for ring space: while the consumers sit in a grid barrier or run the attention, the ring fills
//     with the next projection's rows and HBM stays busy.
//   * fifteen consumer warps execute the operations: quantise an FP32 vector (optionally RMS-normalised) into the
//     CTA's own shared memory, multiply it with the rows the producer delivers, attention for one head, argmax.
//     Every CTA quantises the whole activation vector redundantly (it is at most 76 KB from L2), which removes the
//     separate quantise kernels and their grid-wide dependencies.
//   * operations whose inputs were written by other CTAs start with a grid barrier (an arrival counter in global
//     memory; five per layer). All waits are bounded: a wait that gives up raises the fault word and the abort
//     flag, after which no warp waits for anything any more and the grid drains.
//
// The arithmetic is that of the per-operation kernels, in the same order (same team shape per row length, same
// quantiser, same attention split), so both routes give bit-identical logits.
#pragma once
#include "matvec_xq8.cuh"

namespace syn {
namespace prog {

using namespace mv;

struct BatchToken {
    int32_t slot, token, position, logits_row;
};

// Exact ggml-order decode of element i of a row (GgufLegacyBlocks.cs:85-92, GgufKQuantBlocks.cs:99-177).
__device__ inline float decode_element(uint32_t type, const uint8_t *row, uint32_t i)
{
    if (type == kQ8_0) {
        const uint8_t *block = row + (uint64_t)(i / 32) * 34;
        const float d = __half2float(__ushort_as_half((unsigned short)(block[0] | (block[1] << 8))));
        return d * (float)(signed char)block[2 + (i & 31)];
    }
    if (type == kQ4_K) {
        const uint8_t *block = row + (uint64_t)(i / 256) * 144;
        const uint32_t within = i & 255, chunk = within / 64, l = within & 31, high = (within >> 5) & 1;
        const float d = __half2float(__ushort_as_half((unsigned short)(block[0] | (block[1] << 8))));
        const float dmin = __half2float(__ushort_as_half((unsigned short)(block[2] | (block[3] << 8))));
        const uint8_t *s = block + 4;
        const uint32_t j = chunk * 2 + high;
        uint32_t sc, mn;
        if (j < 4) {
            sc = s[j] & 63;
            mn = s[j + 4] & 63;
        } else {
            sc = (s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4);
            mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
        }
        const uint32_t q = high ? (block[16 + chunk * 32 + l] >> 4) : (block[16 + chunk * 32 + l] & 0x0F);
        return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(dmin, (float)mn));
    }
    const uint8_t *block = row + (uint64_t)(i / 256) * 210;
    const uint32_t within = i & 255, half = within / 128, rest = within & 127, quarter = rest / 32, l = rest & 31;
    const uint8_t *ql = block + half * 64, *qh = block + 128 + half * 32;
    const float d = __half2float(__ushort_as_half((unsigned short)(block[208] | (block[209] << 8))));
    const int scale = (int)(signed char)block[192 + half * 8 + l / 16 + 2 * quarter];
    const uint32_t low = (quarter & 1) ? ql[l + 32] : ql[l];
    const uint32_t nibble = quarter < 2 ? (low & 0x0F) : (low >> 4);
    const int q = (int)(nibble | (((qh[l] >> (2 * quarter)) & 3) << 4)) - 32;
    return __fmul_rn(__fmul_rn(d, (float)scale), (float)q);
}

constexpr int kConsumerWarps = 15;  // with the producer warp 512 threads: up to 128 registers each
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;
constexpr uint32_t kRingStagesMax = 16;
// Warps that share one head's attention: warp w walks positions w, w + kAttentionWarps, ...; the partial results are
// merged in warp order. Both forms of the step use the same split, so their results agree bit for bit.
constexpr int kAttentionWarps = 12;
constexpr uint32_t kStashIterations = 48;  // row groups per CTA of a gate projection whose results stay in shared memory
constexpr int kNormDepth = 5, kPlainDepth = 10;  // 128-value pieces per warp held in registers while quantising
constexpr uint32_t kNormQuadsMax = kNormDepth * 15;
constexpr uint32_t kGridSpinLimit = 1u << 21;        // polls of the arrival counter (a fraction of a second)
// Activations + ring. With the kernel's static shared memory this stays inside the 196 KB shared-memory carve-out, which
// leaves 60 KB of L1: a ring that fills the whole 227 KB was measured slower (the step has more in flight than the
// memory system needs, and every small load queues behind it).
constexpr uint32_t kDynamicSharedBudget = 168 * 1024;

enum : uint32_t { kOpEmbed = 0, kOpQuantize = 1, kOpMatvec = 2, kOpAttention = 3, kOpArgmax = 4 };
enum : uint32_t { kFormatQ8Planar = 0, kFormatQ4K = 1, kFormatQ6KPlanar = 2 };

// One operation of the program (device memory, read-only while the kernel runs).
struct Op {
    uint32_t kind = 0;
    uint32_t barrier = 0;  // the consumers of the whole grid meet before this operation starts
    // kOpMatvec: y[row] = epilogue(weights[row] . activations in shared memory)
    uint32_t format = 0, team = 1, upl = 1, one_pass = 1;
    uint32_t rows = 0, columns = 0;  // columns is also the length of the vector of kOpQuantize
    uint32_t group_rows = 0;         // rows per ring stage
    uint32_t first_cta = 0;          // row group g belongs to CTA (g + first_cta) % grid
    uint32_t planes = 0, stage_bytes = 0;
    uint32_t plane_offset[4] = {0, 0, 0, 0}, plane_row_bytes[4] = {0, 0, 0, 0};
    const uint8_t *plane[4] = {nullptr, nullptr, nullptr, nullptr};
    float *y = nullptr;
    const float *bias = nullptr, *gate = nullptr;
    uint32_t accumulate = 0;
    // kOpQuantize: shared activations = Q8_0(x) or Q8_0(rmsnorm(x) * norm_weight)
    float epsilon = 0.0f;
    const float *x = nullptr, *norm_weight = nullptr;
    // kOpAttention
    uint32_t layer = 0;
    // kOpMatvec on the vocabulary projection: every CTA also keeps the first maximum of the rows it wrote
    uint32_t track_argmax = 0;
    // kOpMatvec, worked out on the host so that the start of a projection is a few loads instead of a chain of
    // integer divisions: teams per CTA, row groups, units per row, offsets of the activation scales and code sums
    // behind the codes, and per consumer warp (four bits each) its team and its index inside the team.
    uint32_t teams = 0, groups = 0, units = 0, scales_offset = 0, sums_offset = 0;
    // 1: the gate projection keeps its results in shared memory for the up projection; 2: the up projection reads them
    uint32_t gate_stash = 0;
    uint64_t team_of_warp = 0, index_in_team = 0;
    // kOpEmbed: plane[0] = table, format = GGML type, y = hidden
    uint64_t row_bytes = 0;
};
static_assert(sizeof(Op) % 4 == 0, "operations are copied word by word");
constexpr uint32_t kOpWords = sizeof(Op) / 4;
constexpr uint32_t kWindowOps = 8;  // operations staged in shared memory at a time

// What the producer warp needs of a projection (the kOpMatvec operations in program order).
struct ProducerOp {
    const uint8_t *plane[4] = {nullptr, nullptr, nullptr, nullptr};
    uint32_t plane_row_bytes[4] = {0, 0, 0, 0}, plane_offset[4] = {0, 0, 0, 0};
    uint32_t rows = 0, group_rows = 0, first_cta = 0, planes = 0, stage_bytes = 0, groups = 0, pad[2] = {0, 0};
};
constexpr uint32_t kProducerOpWords = sizeof(ProducerOp) / 4;
constexpr uint32_t kProducerWindowOps = 8;
static_assert(kProducerOpWords * kProducerWindowOps % 32 == 0, "a window is copied by the 32 lanes of the producer warp");
constexpr uint32_t kProducerWordsPerLane = kProducerOpWords * kProducerWindowOps / 32;

struct Params {
    const Op *ops;
    uint32_t op_count;
    const ProducerOp *producer_ops;
    uint32_t producer_count;
    const BatchToken *token;
    uint32_t *sync;   // [0] barrier arrivals of this launch, [1] abort flag; zeroed before every launch
    uint32_t *fault;  // host-mapped fault word (may be null)
    uint32_t ring_bytes, act_bytes;  // dynamic shared memory: quantised activations, then the weight ring
    float *q, *k, *v, *attention, *keys, *values;
    const float *cosines, *sines;
    uint32_t heads, kv_heads, head_dim, layers, context;
    float attention_scale;
    float *best_value;  // [grid] per-CTA maxima of the vocabulary projection
    int32_t *best_index;
    int32_t *argmax;
    uint64_t *timeline;  // profiling aid, normally null: CTA 0 records the nanosecond timer before each operation and at the end
};

__device__ __forceinline__ uint32_t load_acquire(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint64_t global_timer()
{
    // SM cycle counter scaled to nanoseconds at the 1965 MHz the part runs at under this load: cheap to read, and all
    // marks come from one SM
    uint64_t t;
    asm volatile("mov.u64 %0, %%clock64;" : "=l"(t));
    return t * 1000 / 1965;
}
__device__ __forceinline__ float load_l2(const float *p) { return __ldcg(p); }
__device__ __forceinline__ float4 load_l2(const float4 *p) { return __ldcg(p); }

// Shared state of one CTA.
struct Shared {
    uint64_t barriers[2 * kRingStagesMax];  // full[s] then empty[s]
    float partial[2][kConsumerWarps];
    double square_sums[8];
    float norm_scale;
    int abort;  // set once a wait gave up: nobody waits any more
    // (rows of a multiple of four floats and 16-byte aligned vectors: the attention walk moves them four values at a time)
    alignas(16) float merged[kAttentionWarps][256 + 4];  // a warp's unnormalised sum, [256] its maximum, [257] its weight sum
    alignas(16) float query[256], key[256], value[256];
    float best_value[kConsumerWarps];
    int best_index[kConsumerWarps];
    double quad_sums[kNormQuadsMax];                 // sums of squares of 128-value pieces of the vector being normalised
    float gate_stash[kStashIterations][kConsumerWarps];  // gate projection results of this CTA's rows, by iteration and warp
    uint32_t stage_begin[kRingStagesMax];  // producer's record of where each stage in flight starts
    uint32_t window[2][kWindowOps * kOpWords];
    uint32_t producer_window[2][kProducerWindowOps * kProducerOpWords];  // the operations being executed and the next ones, copied from global memory
};

__device__ __forceinline__ void consumer_sync() { consumer_barrier<kConsumerThreads>(); }

__device__ __forceinline__ void raise_fault(const Params &P, Shared &sh)
{
    if (P.fault) {
        atomicAdd(P.fault, 1u);
    }
    atomicExch(P.sync + 1, 1u);
    *(volatile int *)&sh.abort = 1;
}
__device__ __forceinline__ bool aborted(const Shared &sh) { return *(const volatile int *)&sh.abort != 0; }

// Bounded wait on an mbarrier phase; gives up at once when the CTA is in abort mode. The common case (the phase has
// completed) is a single inlined test; the polling loop stays out of line, out of the hot code.
__device__ __noinline__ void wait_phase_slow(const Params &P, Shared &sh, uint32_t bar, uint32_t parity, bool report)
{
    if (aborted(sh)) {
        return;
    }
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) {
            return;
        }
        if ((i & 1023u) == 1023u && aborted(sh)) {
            return;
        }
    }
    if (report) {
        raise_fault(P, sh);
    }
}
__device__ __forceinline__ void wait_phase(const Params &P, Shared &sh, uint32_t bar, uint32_t parity, bool report)
{
    if (!mbar_try_wait(bar, parity)) {
        wait_phase_slow(P, sh, bar, parity, report);
    }
}

// All consumer warps of the grid meet. `epoch` counts the barriers this CTA has passed.
__device__ __noinline__ void grid_sync(const Params &P, Shared &sh, uint32_t &epoch)
{
    consumer_sync();
    if (threadIdx.x == 0 && !aborted(sh)) {
        // release: everything the CTA wrote before the barrier above is visible to whoever acquires the counter
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(P.sync) : "memory");
        const uint32_t target = (epoch + 1) * gridDim.x;
        bool met = false;
        for (uint32_t i = 0; i < kGridSpinLimit; ++i) {
            if (load_acquire(P.sync) >= target) {
                met = true;
                break;
            }
            if ((i & 63u) == 63u && load_acquire(P.sync + 1) != 0) {
                break;
            }
        }
        if (!met) {
            raise_fault(P, sh);
        }
    }
    consumer_sync();
    ++epoch;
}

// The first row group of a projection that this CTA owns; it then takes every gridDim.x-th. Interleaving keeps all
// CTAs inside one narrow window of the matrix, which spreads the reads evenly over the memory channels (contiguous
// runs per CTA were measured 35 % slower). CTAs are numbered from `first_cta` on so that the surplus groups of one
// projection and the next do not land on the same CTAs.
__device__ __forceinline__ uint32_t first_group(uint32_t first_cta)  // first_cta < gridDim.x
{
    const uint32_t v = blockIdx.x + gridDim.x - first_cta;
    return v >= gridDim.x ? v - gridDim.x : v;
}

// The weight ring is a circular byte buffer: stage j of a CTA (counted over all its projections) takes the next
// `stage_bytes` of it, starting over at 0 when it would run past the end, and uses barrier pair j % kRingStagesMax
// with phase parity (j / kRingStagesMax) & 1. Producer and consumers compute the same offsets independently.
struct Ring {
    uint32_t head = 0;      // where the next stage starts
    uint32_t sequence = 0;  // j
    uint32_t iteration = 0;
    __device__ __forceinline__ uint32_t take(uint32_t bytes, uint32_t capacity)
    {
        if (head + bytes > capacity) {
            head = 0;
        }
        const uint32_t offset = head;
        head += bytes;
        return offset;
    }
};

// The global operands of a row's epilogue (bias, the value to accumulate onto). They are fetched two iterations ahead:
// a load from L2 takes over a microsecond while the weight stream saturates the memory system, an iteration half of that.
struct EpilogueOperands {
    float bias = 0.0f, previous = 0.0f;
};
__device__ __forceinline__ EpilogueOperands fetch_epilogue(const Epilogue &e, const float *y, uint32_t row, bool wanted)
{
    EpilogueOperands o;
    if (wanted && e.bias) {
        o.bias = __ldg(e.bias + row);
    }
    if (wanted && e.accumulate) {
        o.previous = load_l2(y + row);
    }
    return o;
}
// Same arithmetic as store_result of the per-operation kernels.
__device__ __forceinline__ float store_epilogue(const Epilogue &e, const EpilogueOperands &o, float gate, float *y, uint32_t row, float v)
{
    if (e.bias) {
        v += o.bias;
    }
    if (e.gate) {
        v = gate / (1.0f + expf(-gate)) * v;
    }
    v = e.accumulate ? o.previous + v : v;
    y[row] = v;
    return v;
}

// The rows of one projection that this CTA owns, against the activations in shared memory. Same lane assignment and
// summation order as matvec_xq8_pipe_kernel with one token and one row per team iteration; the team width W (warps
// per row, 1..8, from the row length) is a run-time value here, so that there is ONE copy of this code per weight
// format: a step switches projections twelve times per layer, and code that is not in the instruction cache costs
// more than a microsecond to fetch while the weight stream saturates the memory system.
// Each lane keeps its slice of the activations in registers (the program is only built for rows that one pass of the
// team covers). A row shorter than 32 * UPL units leaves the upper units of a lane invalid, which adds nothing.
template <class F>
__device__ __noinline__ Ring consume_matvec(const Op *op, const Params &P, Shared &sh, uint32_t act_base, uint32_t ring_base, Ring ring)
{
    constexpr int UPL = F::kMaxUpl;
    const uint32_t W = op->team;
    const uint32_t teams = op->teams;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const bool active = warp < teams * W;
    const uint32_t team_in_cta = (uint32_t)(op->team_of_warp >> (4 * warp)) & 15u;  // 0 for a warp without a team
    const uint32_t warp_in_team = (uint32_t)(op->index_in_team >> (4 * warp)) & 15u;
    const uint32_t K = op->columns, rows = op->rows;
    const uint32_t units = op->units;
    const uint32_t full0 = smem_u32(&sh.barriers[0]), empty0 = smem_u32(&sh.barriers[kRingStagesMax]);
    ActShared act;
    act.codes = act_base;
    act.scales = act_base + op->scales_offset;
    act.sums = act_base + op->sums_offset;
    Epilogue epilogue;
    epilogue.bias = op->bias;
    epilogue.gate = op->gate;
    epilogue.accumulate = op->accumulate;
    float *const y = op->y;
    const uint32_t stage_bytes = op->stage_bytes;
    uint32_t plane_offset[4], plane_row_bytes[4], plane_low[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        plane_offset[k] = op->plane_offset[k];
        plane_row_bytes[k] = op->plane_row_bytes[k];
        plane_low[k] = (uint32_t)(reinterpret_cast<uintptr_t>(op->plane[k]) & 15);
    }

    const uint32_t groups = op->groups;
    const bool writer = active && warp_in_team == 0 && lane == 0;
    const uint32_t g0 = first_group(op->first_cta);
    EpilogueOperands operands0, operands1;
    {
        const uint32_t row0 = g0 * teams + team_in_cta, row1 = (g0 + gridDim.x) * teams + team_in_cta;
        operands0 = fetch_epilogue(epilogue, y, row0, writer && g0 < groups && row0 < rows);
        operands1 = fetch_epilogue(epilogue, y, row1, writer && row1 < rows);
    }

    typename F::Act held[UPL];
    uint32_t u[UPL];
    bool valid[UPL];
#pragma unroll
    for (int j = 0; j < UPL; ++j) {
        // with UPL == 1 in the per-operation kernel (rows of at most 32 units) unit j = 1 does not exist either
        const uint32_t unit = (warp_in_team * (op->upl == 1 ? 1 : UPL) + j) * 32 + lane;
        valid[j] = unit < units && (uint32_t)j < op->upl;
        u[j] = valid[j] ? unit : units - 1;
        F::template load_act<SharedMem>(act, K, 0, u[j], held[j]);
    }

    const bool track = op->track_argmax != 0;
    float best = -INFINITY;
    int best_row = 0x7fffffff;
    const uint32_t stash = op->gate_stash;
    uint32_t iteration = 0;
    for (uint32_t g = g0; g < groups; g += gridDim.x, ++iteration) {
        const uint32_t group_row0 = g * teams;
        const uint32_t row = group_row0 + team_in_cta;
        const EpilogueOperands operands = operands0;
        operands0 = operands1;
        {
            const uint32_t ahead = (g + 2 * gridDim.x) * teams + team_in_cta;
            operands1 = fetch_epilogue(epilogue, y, ahead, writer && ahead < rows);
        }
        float gate = 0.0f;
        if (epilogue.gate && writer && row < rows) {
            // the gate value of this row was computed by this same thread in the projection before
            gate = stash == 2 ? sh.gate_stash[iteration][warp] : load_l2(epilogue.gate + row);
        }
        const uint32_t stage = ring_base + ring.take(stage_bytes, P.ring_bytes);
        const uint32_t pair = ring.sequence % kRingStagesMax, parity = (ring.sequence / kRingStagesMax) & 1;
        ++ring.sequence;
        wait_phase(P, sh, full0 + 8 * pair, parity, lane == 0);
        // The stage holds rows [group_row0, +teams) of every plane with the plane's own row pitch; a plane whose rows
        // are not 16-byte multiples starts `shift` bytes into its slot.
        SharedView view;
        view.row_bytes = plane_row_bytes[0];
        {
            uint32_t local[4] = {0, 0, 0, 0};
#pragma unroll
            for (int k = 0; k < F::kPlanes; ++k) {
                const uint32_t shift = (plane_low[k] + group_row0 * plane_row_bytes[k]) & 15;
                local[k] = stage + plane_offset[k] + shift;
            }
            view.p0 = local[0];
            view.p1 = local[1];
            view.p2 = local[2];
            view.p3 = local[3];
        }
        float acc = 0.0f;
        if (active) {
            typename F::W wr[UPL];
#pragma unroll
            for (int j = 0; j < UPL; ++j) {
                F::template load_w<SharedMem>(view, K, team_in_cta, u[j], lane, wr[j]);
            }
#pragma unroll
            for (int j = 0; j < UPL; ++j) {
                F::template dot<false>(wr[j], held[j], valid[j], u[j], lane, acc, nullptr);
            }
            // Every unit of this warp has been consumed: give the stage back to the producer. The refill is written by the
            // asynchronous proxy, the loads above went through the generic one: the proxy fence orders them.
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(empty0 + 8 * pair);
            }
        } else if (lane == 0) {
            mbar_arrive(empty0 + 8 * pair);
        }
        acc = warp_sum(acc);
        if (W == 1) {
            if (lane == 0 && row < rows) {
                const float v = store_epilogue(epilogue, operands, gate, y, row, acc);
                if (stash == 1) {
                    sh.gate_stash[iteration][warp] = v;
                }
                if (track && v > best) {  // rows ascend within a warp: a later equal value never replaces an earlier one
                    best = v;
                    best_row = (int)row;
                }
            }
        } else {
            const uint32_t buffer = ring.iteration & 1;
            if (lane == 0) {
                sh.partial[buffer][warp] = acc;
            }
            consumer_sync();
            if (writer) {
                float total = sh.partial[buffer][team_in_cta * W];
                for (uint32_t k = 1; k < W; ++k) {
                    total += sh.partial[buffer][team_in_cta * W + k];
                }
                if (row < rows) {
                    const float v = store_epilogue(epilogue, operands, gate, y, row, total);
                    if (stash == 1) {
                        sh.gate_stash[iteration][warp] = v;
                    }
                    if (track && v > best) {
                        best = v;
                        best_row = (int)row;
                    }
                }
            }
        }
        ++ring.iteration;
    }
    if (track) {
        // first maximum over the rows this CTA wrote (larger value wins, equal values keep the lower row)
        if (lane == 0) {
            sh.best_value[warp] = writer ? best : -INFINITY;
            sh.best_index[warp] = writer ? best_row : 0x7fffffff;
        }
        consumer_sync();
        if (threadIdx.x == 0) {
            float value = sh.best_value[0];
            int index = sh.best_index[0];
            for (int w = 1; w < kConsumerWarps; ++w) {
                if (sh.best_value[w] > value || (sh.best_value[w] == value && sh.best_index[w] < index)) {
                    value = sh.best_value[w];
                    index = sh.best_index[w];
                }
            }
            P.best_value[blockIdx.x] = value;
            P.best_index[blockIdx.x] = index;
        }
    }
    return ring;
}

// Sum of squares of a 128-value piece: each lane adds the squares of its four values in order, then an xor tree
// over the warp. All in FP64 with explicit roundings, so that every kernel that normalises gets the same bits.
__device__ __forceinline__ double quad_square_sum(const float4 &v)
{
    double s = __dmul_rn((double)v.x, (double)v.x);
    s = __fma_rn((double)v.y, (double)v.y, s);
    s = __fma_rn((double)v.z, (double)v.z, s);
    s = __fma_rn((double)v.w, (double)v.w, s);
    for (int offset = 16; offset > 0; offset >>= 1) {
        s = __dadd_rn(s, __shfl_xor_sync(kFull, s, offset));
    }
    return s;
}
// 1 / sqrt(mean square + epsilon) from the per-piece sums, added in index order (Q8Operators.cs:101-123 sums in FP64).
__device__ __forceinline__ float norm_scale_from(const double *quad_sums, uint32_t quads, uint32_t n, float epsilon)
{
    double total = 0.0;
    for (uint32_t q = 0; q < quads; ++q) {
        total = __dadd_rn(total, quad_sums[q]);
    }
    return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn((float)__ddiv_rn(total, (double)n), epsilon)));
}

// Q8_0 quantisation of x[0..n), optionally RMS-normalised first, into the CTA's shared activations. Every value is
// loaded once and stays in registers: a lane takes four consecutive values, eight lanes one 32-value block, a warp
// DEPTH pieces of 128 values. Bit for bit the arithmetic of the stand-alone quantiser kernels.
template <int DEPTH, bool NORM>
__device__ __noinline__ void quantize_local(const Op *op, Shared &sh, uint32_t act_base)
{
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t n = op->columns;
    const float *const x = op->x;
    const uint32_t quads = (n + 127) / 128;
    float4 v[DEPTH];
#pragma unroll
    for (int i = 0; i < DEPTH; ++i) {
        const uint32_t first = (warp + i * kConsumerWarps) * 128 + lane * 4;
        v[i] = first < n ? load_l2(reinterpret_cast<const float4 *>(x + first)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    if (NORM) {
        const float *const weight = op->norm_weight;
        float4 w[DEPTH];
#pragma unroll
        for (int i = 0; i < DEPTH; ++i) {
            const uint32_t first = (warp + i * kConsumerWarps) * 128 + lane * 4;
            w[i] = first < n ? __ldg(reinterpret_cast<const float4 *>(weight + first)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
#pragma unroll
        for (int i = 0; i < DEPTH; ++i) {
            const uint32_t quad = warp + i * kConsumerWarps;
            if (quad < quads) {  // the same for the whole warp
                const double s = quad_square_sum(v[i]);
                if (lane == 0) {
                    sh.quad_sums[quad] = s;
                }
            }
        }
        consumer_sync();
        const float scale = norm_scale_from(sh.quad_sums, quads, n, op->epsilon);
#pragma unroll
        for (int i = 0; i < DEPTH; ++i) {
            if (warp + i * kConsumerWarps >= quads) {
                break;
            }
            v[i].x = __fmul_rn(__fmul_rn(v[i].x, scale), w[i].x);
            v[i].y = __fmul_rn(__fmul_rn(v[i].y, scale), w[i].y);
            v[i].z = __fmul_rn(__fmul_rn(v[i].z, scale), w[i].z);
            v[i].w = __fmul_rn(__fmul_rn(v[i].w, scale), w[i].w);
        }
    }
    const uint32_t codes = act_base, scales = act_base + shared_act_codes_bytes(1, n), sums = scales + shared_act_side_bytes(1, n);
#pragma unroll
    for (int i = 0; i < DEPTH; ++i) {
        if (warp + i * kConsumerWarps >= quads) {
            break;  // pieces past the end of the vector: the same for the whole warp
        }
        const uint32_t first = (warp + i * kConsumerWarps) * 128 + lane * 4;
        float amax = fmaxf(fmaxf(fabsf(v[i].x), fabsf(v[i].y)), fmaxf(fabsf(v[i].z), fabsf(v[i].w)));
        amax = fmaxf(amax, __shfl_xor_sync(kFull, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(kFull, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(kFull, amax, 4));
        const float d = __fdiv_rn(amax, 127.0f);
        const float inverse = d == 0.0f ? 0.0f : __fdiv_rn(1.0f, d);
        const int c0 = __float2int_rn(__fmul_rn(v[i].x, inverse)), c1 = __float2int_rn(__fmul_rn(v[i].y, inverse));
        const int c2 = __float2int_rn(__fmul_rn(v[i].z, inverse)), c3 = __float2int_rn(__fmul_rn(v[i].w, inverse));
        int sum = (c0 + c1) + (c2 + c3);
        sum += __shfl_xor_sync(kFull, sum, 1);
        sum += __shfl_xor_sync(kFull, sum, 2);
        if (first < n) {
            const uint32_t packed = (uint32_t)(c0 & 0xff) | ((uint32_t)(c1 & 0xff) << 8) | ((uint32_t)(c2 & 0xff) << 16) | ((uint32_t)c3 << 24);
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(codes + swizzled_code_offset(first)), "r"(packed) : "memory");
            if ((lane & 3) == 0) {
                asm volatile("st.shared.u16 [%0], %1;" ::"r"(sums + (first / 16) * 2), "h"((short)sum) : "memory");
            }
            if ((lane & 7) == 0) {
                asm volatile("st.shared.f32 [%0], %1;" ::"r"(scales + (first / 32) * 4), "f"(__half2float(__float2half_rn(d))) : "memory");
            }
        }
    }
    consumer_sync();
}

// One warp's share of a head's attention (Qwen2CpuAttention.cs:82-173, as a running softmax). Lane 8 g + e owns elements
// [e * E, (e + 1) * E) of the head, E = head_dim / 8, in position stream 4 * warp + g: the warp walks four positions at
// once, a position's dot product is reduced over eight lanes (three shuffles instead of five per position) and every
// lane's loads are whole 16-byte pieces. A stream takes positions stream, stream + 4 * kAttentionWarps, ...; BATCH of them
// are loaded at a time so that their latencies overlap, and enter the running softmax together: the batch's maximum
// first, then one rescale of what has been accumulated and the batch's weights side by side. `current_key/value` (may
// be null) replace the cache entry of `position`. The four streams of the warp are merged at the end; the warp leaves
// its unnormalised sum in merged_row[0 .. head_dim), its maximum in [256] and its weight sum in [257].
// KV is the cache's element type: float, or __half (DecoderDesc.kv_precision = 1, KvPrecision::F16 of the reference,
// native/synapse-gpu/src/Features/GpuKernels/decoder.rs:43-58), whose values widen exactly; head_dim is then a multiple
// of 64, so that a lane's E values are whole 16-byte pieces too.
// `first_stream` / `streams`: the CTA's share when several CTAs split a head's positions (0 and 4 * kAttentionWarps for one).
template <class KV, int E4, int BATCH>
__device__ __forceinline__ void attend_streams(const float *query, uint32_t lane, uint32_t warp, int position, uint32_t head_dim, float scale,
                                               const KV *keys, const KV *values, const float *current_key, const float *current_value,
                                               float *merged_row, int first_stream, int streams)
{
    constexpr bool kHalf = sizeof(KV) == 2;
    const uint32_t group = lane >> 3, part = lane & 7;
    const uint32_t e4 = head_dim / 32;           // 16-byte pieces of FP32 per lane
    const uint32_t first_element = part * (head_dim / 8);
    float4 q[E4], acc[E4];
#pragma unroll
    for (int i = 0; i < E4; ++i) {
        q[i] = (uint32_t)i < e4 ? *reinterpret_cast<const float4 *>(query + first_element + 4 * i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        acc[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    float running_max = -INFINITY, running_sum = 0.0f;
    const int stride = streams;
    // The loop count must be the same for all lanes of the warp (the shuffles below name all of them): it runs over the
    // warp's first stream, and a stream that has run out of positions takes part with weights of zero.
    for (int base = first_stream + (int)(4 * warp); base <= position; base += stride * BATCH) {
        const int p0 = base + (int)group;
        float4 k[BATCH][E4], v[BATCH][E4];
        // FP16 cache: the loaded pieces stay as they are until every load of the batch has been issued (a conversion right
        // behind its load would hold the warp, and with it the next load, for the load's whole latency)
        uint4 k_raw[kHalf ? BATCH : 1][kHalf ? (E4 + 1) / 2 : 1], v_raw[kHalf ? BATCH : 1][kHalf ? (E4 + 1) / 2 : 1];
#pragma unroll
        for (int b = 0; b < BATCH; ++b) {
            const int p = p0 + stride * b;
            const bool live = p <= position;
            const bool current = current_key && p == position;
            const uint64_t row = (uint64_t)(live ? p : position) * head_dim + first_element;
            if (current) {
#pragma unroll
                for (int i = 0; i < E4; ++i) {
                    const uint32_t at = first_element + 4 * ((uint32_t)i < e4 ? i : 0);
                    k[b][i] = *reinterpret_cast<const float4 *>(current_key + at);
                    v[b][i] = *reinterpret_cast<const float4 *>(current_value + at);
                }
            } else if constexpr (kHalf) {
#pragma unroll
                for (int i = 0; i < (E4 + 1) / 2; ++i) {
                    const uint32_t at = 8 * ((uint32_t)(2 * i) < e4 ? i : 0);  // unconditional loads; unused pieces are zeroed below
                    k_raw[b][i] = *reinterpret_cast<const uint4 *>(keys + row + at);
                    v_raw[b][i] = *reinterpret_cast<const uint4 *>(values + row + at);
                }
            } else {
#pragma unroll
                for (int i = 0; i < E4; ++i) {
                    const uint32_t at = 4 * ((uint32_t)i < e4 ? i : 0);
                    k[b][i] = *reinterpret_cast<const float4 *>(keys + row + at);
                    v[b][i] = *reinterpret_cast<const float4 *>(values + row + at);
                }
            }
        }
        if constexpr (kHalf) {
#pragma unroll
            for (int b = 0; b < BATCH; ++b) {
                if (!(current_key && p0 + stride * b == position)) {
#pragma unroll
                    for (int i = 0; i < (E4 + 1) / 2; ++i) {
                        const __half2 *kh = reinterpret_cast<const __half2 *>(&k_raw[b][i]), *vh = reinterpret_cast<const __half2 *>(&v_raw[b][i]);
                        const float2 k0 = __half22float2(kh[0]), k1 = __half22float2(kh[1]), k2 = __half22float2(kh[2]), k3 = __half22float2(kh[3]);
                        const float2 v0 = __half22float2(vh[0]), v1 = __half22float2(vh[1]), v2 = __half22float2(vh[2]), v3 = __half22float2(vh[3]);
                        k[b][2 * i] = make_float4(k0.x, k0.y, k1.x, k1.y);
                        v[b][2 * i] = make_float4(v0.x, v0.y, v1.x, v1.y);
                        if (2 * i + 1 < E4) {
                            k[b][2 * i + 1] = make_float4(k2.x, k2.y, k3.x, k3.y);
                            v[b][2 * i + 1] = make_float4(v2.x, v2.y, v3.x, v3.y);
                        }
                    }
                }
            }
        }
        float scores[BATCH], batch_max = running_max;
#pragma unroll
        for (int b = 0; b < BATCH; ++b) {
            float dot = 0.0f;
#pragma unroll
            for (int i = 0; i < E4; ++i) {
                if ((uint32_t)i < e4) {
                    dot = fmaf(q[i].x, k[b][i].x, dot);
                    dot = fmaf(q[i].y, k[b][i].y, dot);
                    dot = fmaf(q[i].z, k[b][i].z, dot);
                    dot = fmaf(q[i].w, k[b][i].w, dot);
                }
            }
            dot += __shfl_xor_sync(kFull, dot, 1);
            dot += __shfl_xor_sync(kFull, dot, 2);
            dot += __shfl_xor_sync(kFull, dot, 4);
            scores[b] = p0 + stride * b <= position ? dot * scale : -INFINITY;
            batch_max = fmaxf(batch_max, scores[b]);
        }
        // (a stream with no live position yet has running_max = batch_max = -inf: nothing to rescale, all weights zero;
        // exp(-inf) = 0 covers the first live batch and the dead positions of a live one)
        const float rescale = running_max == batch_max ? 1.0f : expf(running_max - batch_max);
        float weights[BATCH], total = 0.0f;
#pragma unroll
        for (int b = 0; b < BATCH; ++b) {
            weights[b] = scores[b] == -INFINITY ? 0.0f : expf(scores[b] - batch_max);
            total += weights[b];
        }
#pragma unroll
        for (int i = 0; i < E4; ++i) {
            if ((uint32_t)i < e4) {
                float4 a = make_float4(acc[i].x * rescale, acc[i].y * rescale, acc[i].z * rescale, acc[i].w * rescale);
#pragma unroll
                for (int b = 0; b < BATCH; ++b) {
                    a.x = fmaf(weights[b], v[b][i].x, a.x);
                    a.y = fmaf(weights[b], v[b][i].y, a.y);
                    a.z = fmaf(weights[b], v[b][i].z, a.z);
                    a.w = fmaf(weights[b], v[b][i].w, a.w);
                }
                acc[i] = a;
            }
        }
        running_sum = running_sum * rescale + total;
        running_max = batch_max;
    }
    if (first_stream + (int)(4 * warp) > position) {  // (same for all lanes) the warp had no position at all
        if (lane == 0) {
            merged_row[256] = -INFINITY;
            merged_row[257] = 0.0f;
        }
        return;
    }
    // The warp's four streams into one (a stream without positions has maximum -inf and weight sum 0). Each step halves
    // what a lane carries on: of the elements it still holds it keeps one half, hands the other half to its partner and
    // takes the partner's share of the half it keeps, so that the four lanes of a part end with a quarter of its elements each.
    float *const a = reinterpret_cast<float *>(acc);
    uint32_t kept = 0;  // first element (of the part's 4 * E4) this lane still holds
#pragma unroll
    for (int step = 0; step < 2; ++step) {
        const uint32_t offset = 8u << step;
        const int count = (4 * E4) >> (step + 1);  // elements kept
        const bool upper = lane & offset;
        const float other_max = __shfl_xor_sync(kFull, running_max, offset), other_sum = __shfl_xor_sync(kFull, running_sum, offset);
        const float joint = fmaxf(running_max, other_max);
        const float mine = running_max == -INFINITY ? 0.0f : expf(running_max - joint), theirs = other_max == -INFINITY ? 0.0f : expf(other_max - joint);
#pragma unroll
        for (int j = 0; j < count; ++j) {
            const float keep = upper ? a[count + j] : a[j], give = upper ? a[j] : a[count + j];
            const float taken = __shfl_xor_sync(kFull, give, offset);
            a[j] = __fmaf_rn(keep, mine, __fmul_rn(taken, theirs));
        }
        kept += upper ? count : 0;
        running_sum = __fmaf_rn(running_sum, mine, __fmul_rn(other_sum, theirs));
        running_max = joint;
    }
    if constexpr (E4 % 4 == 0) {
#pragma unroll
        for (int j = 0; j < E4; j += 4) {
            if (kept + j < 4 * e4) {
                *reinterpret_cast<float4 *>(merged_row + first_element + kept + j) = make_float4(a[j], a[j + 1], a[j + 2], a[j + 3]);
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < E4; ++j) {
            if (kept + j < 4 * e4) {
                merged_row[first_element + kept + j] = a[j];
            }
        }
    }
    if (lane == 0) {
        merged_row[256] = running_max;
        merged_row[257] = running_sum;
    }
}

// Heads of up to 32 / 64 / 128 / 256 values: the wider the head, the fewer positions a stream keeps in flight (the loaded
// keys and values live in registers).
template <class KV>
__device__ __forceinline__ void attend_head(const float *query, uint32_t lane, uint32_t warp, int position, uint32_t head_dim, float scale,
                                            const KV *keys, const KV *values, const float *current_key, const float *current_value,
                                            float *merged_row, int first_stream = 0, int streams = 4 * kAttentionWarps)
{
    if (head_dim <= 32) {
        attend_streams<KV, 1, 4>(query, lane, warp, position, head_dim, scale, keys, values, current_key, current_value, merged_row, first_stream, streams);
    } else if (head_dim <= 64) {
        attend_streams<KV, 2, 2>(query, lane, warp, position, head_dim, scale, keys, values, current_key, current_value, merged_row, first_stream, streams);
    } else if (head_dim <= 128) {
        attend_streams<KV, 4, 1>(query, lane, warp, position, head_dim, scale, keys, values, current_key, current_value, merged_row, first_stream, streams);
    } else {
        attend_streams<KV, 8, 1>(query, lane, warp, position, head_dim, scale, keys, values, current_key, current_value, merged_row, first_stream, streams);
    }
}

// One query head of the token: NeoX rotation of the head's query and of its key head (Qwen2CpuState.cs:85-105),
// append of key and value to the slot's cache (by the first query head of each key head), softmax attention over
// positions 0..position (Qwen2CpuAttention.cs:82-173) with the warp split of attention_kernel.
__device__ __noinline__ void attention_local(const Op *op, const Params &P, Shared &sh)
{
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t head = blockIdx.x, head_dim = P.head_dim, half = head_dim / 2;
    const uint32_t group = P.heads / P.kv_heads, kh = head / group;
    const BatchToken token = *P.token;
    const uint64_t base = (((uint64_t)token.slot * P.layers + op->layer) * P.kv_heads + kh) * P.context * head_dim;
    if (threadIdx.x < half) {
        const uint32_t i = threadIdx.x;
        const float c = P.cosines[(uint64_t)token.position * half + i], s = P.sines[(uint64_t)token.position * half + i];
        {
            const float *x = P.q + (uint64_t)head * head_dim;
            const float a = load_l2(x + i), b = load_l2(x + i + half);
            sh.query[i] = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
            sh.query[i + half] = __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c));
        }
        const float *x = P.k + (uint64_t)kh * head_dim;
        const float a = load_l2(x + i), b = load_l2(x + i + half);
        const float first = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s)), second = __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c));
        const float *vs = P.v + (uint64_t)kh * head_dim;
        const float v0 = load_l2(vs + i), v1 = load_l2(vs + i + half);
        sh.key[i] = first;
        sh.key[i + half] = second;
        sh.value[i] = v0;
        sh.value[i + half] = v1;
        if (head % group == 0) {
            const uint64_t at = base + (uint64_t)token.position * head_dim;
            P.keys[at + i] = first;
            P.keys[at + i + half] = second;
            P.values[at + i] = v0;
            P.values[at + i + half] = v1;
        }
    }
    consumer_sync();
    if (warp < (uint32_t)kAttentionWarps) {
        attend_head(sh.query, lane, warp, token.position, head_dim, P.attention_scale, P.keys + base, P.values + base, sh.key, sh.value, sh.merged[warp]);
    }
    consumer_sync();
    if (threadIdx.x < head_dim) {
        float total_max = -INFINITY;
        for (int w = 0; w < kAttentionWarps; ++w) {
            total_max = fmaxf(total_max, sh.merged[w][256]);
        }
        float total_sum = 0.0f;
        for (int w = 0; w < kAttentionWarps; ++w) {
            total_sum += sh.merged[w][256] == -INFINITY ? 0.0f : sh.merged[w][257] * expf(sh.merged[w][256] - total_max);
        }
        float value = 0.0f;
        for (int w = 0; w < kAttentionWarps; ++w) {
            value += sh.merged[w][256] == -INFINITY ? 0.0f : sh.merged[w][threadIdx.x] * expf(sh.merged[w][256] - total_max);  // (an idle warp leaves its row unwritten)
        }
        P.attention[(uint64_t)head * head_dim + threadIdx.x] = value / total_sum;
    }
}

// First maximum of the logits row (Q8Operators.cs:152-173: larger value wins, equal values keep the lower index)
// from the per-CTA maxima the vocabulary projection left behind. One warp.
__device__ __forceinline__ void argmax_local(const Params &P)
{
    if (threadIdx.x >= 32) {
        return;
    }
    float value = -INFINITY;
    int index = 0x7fffffff;
    for (uint32_t i = threadIdx.x; i < gridDim.x; i += 32) {
        const float v = load_l2(P.best_value + i);
        const int at = __ldcg(P.best_index + i);
        if (v > value || (v == value && at < index)) {
            value = v;
            index = at;
        }
    }
    for (int offset = 16; offset > 0; offset >>= 1) {
        const float other_value = __shfl_xor_sync(kFull, value, offset);
        const int other_index = __shfl_xor_sync(kFull, index, offset);
        if (other_value > value || (other_value == value && other_index < index)) {
            value = other_value;
            index = other_index;
        }
    }
    if (threadIdx.x == 0) {
        P.argmax[0] = index;
    }
}

// The producer warp. Lane 0 streams this CTA's row groups of every projection, in program order, into the ring; all
// 32 lanes keep a window of projection descriptors in shared memory one window ahead, so that lane 0 never waits for
// a descriptor (a dependent global load takes over a microsecond while the weight stream saturates the memory system).
__device__ __forceinline__ void produce(const Params &P, Shared &sh, uint32_t ring_base, uint32_t lane)
{
    const uint32_t full0 = smem_u32(&sh.barriers[0]), empty0 = smem_u32(&sh.barriers[kRingStagesMax]);
    const uint64_t policy = l2_evict_first_policy();
    const uint32_t *const words = reinterpret_cast<const uint32_t *>(P.producer_ops);
    const uint32_t total_words = P.producer_count * kProducerOpWords;
#pragma unroll
    for (uint32_t k = 0; k < kProducerWordsPerLane; ++k) {
        const uint32_t w = lane + 32 * k;
        sh.producer_window[0][w] = w < total_words ? __ldg(words + w) : 0u;
    }
    __syncwarp();
    Ring ring;
    uint32_t released = 0;  // stages 0..released-1 are known to have been read by every consumer warp
    uint32_t tail = 0;      // where the oldest stage not known to be read starts
    uint32_t issued = 0;
    for (uint32_t window0 = 0; window0 < P.producer_count; window0 += kProducerWindowOps) {
        const uint32_t buffer = (window0 / kProducerWindowOps) & 1;
        uint32_t next[kProducerWordsPerLane];
#pragma unroll
        for (uint32_t k = 0; k < kProducerWordsPerLane; ++k) {
            const uint32_t w = (window0 + kProducerWindowOps) * kProducerOpWords + lane + 32 * k;
            next[k] = w < total_words ? __ldg(words + w) : 0u;
        }
        const uint32_t window_end = min(P.producer_count, window0 + kProducerWindowOps);
        for (uint32_t index = window0; index < window_end && lane == 0; ++index) {
            const ProducerOp *op = reinterpret_cast<const ProducerOp *>(&sh.producer_window[buffer][(index - window0) * kProducerOpWords]);
            const uint32_t G = op->group_rows, rows = op->rows, planes = op->planes, stage_bytes = op->stage_bytes;
            const uint32_t groups = op->groups;
            const uint32_t group_begin = first_group(op->first_cta);
            uint32_t plane_offset[4], plane_row_bytes[4];
            const uint8_t *plane[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                plane_offset[k] = op->plane_offset[k];
                plane_row_bytes[k] = op->plane_row_bytes[k];
                plane[k] = op->plane[k];
            }
            for (uint32_t g = group_begin; g < groups; g += gridDim.x) {
                const uint32_t previous_head = ring.head;
                const uint32_t offset = ring.take(stage_bytes, P.ring_bytes);
                const uint32_t j = ring.sequence++;
                const uint32_t pair = j % kRingStagesMax;
                // Stage j needs its barrier pair (stage j - kRingStagesMax read by every consumer warp) and its bytes.
                // Stages are read in order, so the bytes in use run from the start of the oldest unread stage (tail)
                // forward to previous_head, possibly through the end of the ring.
                while (released < j) {
                    bool fits;
                    if (released + kRingStagesMax <= j) {
                        fits = false;
                    } else if (previous_head > tail) {
                        fits = offset >= previous_head || (offset == 0 && stage_bytes <= tail);
                    } else {
                        fits = offset == previous_head && previous_head + stage_bytes <= tail;
                    }
                    if (fits) {
                        break;
                    }
                    wait_phase(P, sh, empty0 + 8 * (released % kRingStagesMax), (released / kRingStagesMax) & 1, true);
                    ++released;
                    tail = sh.stage_begin[released % kRingStagesMax];  // meaningful while released < j
                }
                if (released == j) {
                    tail = offset;  // nothing else in flight: this stage is the oldest
                }
                if (aborted(sh)) {
                    continue;  // nobody will read further stages: issue nothing more
                }
                sh.stage_begin[pair] = offset;
                const uint32_t row0 = g * G;
                const uint32_t n = min(G, rows - row0);
                uint32_t total = 0, bytes[4] = {0, 0, 0, 0};
                const uint8_t *sources[4] = {nullptr, nullptr, nullptr, nullptr};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if ((uint32_t)k < planes) {
                        const uint8_t *source = plane[k] + (uint64_t)row0 * plane_row_bytes[k];
                        const uint32_t shift = (uint32_t)(reinterpret_cast<uintptr_t>(source) & 15);
                        sources[k] = source - shift;
                        bytes[k] = (shift + n * plane_row_bytes[k] + 15) & ~15u;
                        total += bytes[k];
                    }
                }
                mbar_expect_tx(full0 + 8 * pair, total);
                const uint32_t stage = ring_base + offset;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if ((uint32_t)k < planes) {
                        bulk_copy(stage + plane_offset[k], sources[k], bytes[k], full0 + 8 * pair, policy);
                    }
                }
                issued = j + 1;
            }
        }
        __syncwarp();
#pragma unroll
        for (uint32_t k = 0; k < kProducerWordsPerLane; ++k) {
            sh.producer_window[buffer ^ 1][lane + 32 * k] = next[k];
        }
        __syncwarp();
    }
    // Every copy lane 0 issued must have landed before the CTA may retire (bounded; normally they all have). After an
    // abort `issued` is the last stage actually copied; stages are issued in order, so only the newest can be pending.
    if (lane == 0) {
        for (uint32_t i = issued > kRingStagesMax ? issued - kRingStagesMax : 0; i < issued; ++i) {
            const uint32_t bar = full0 + 8 * (i % kRingStagesMax), parity = (i / kRingStagesMax) & 1;
            for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
                if (mbar_try_wait(bar, parity)) {
                    break;
                }
            }
        }
    }
}

__global__ void __launch_bounds__(kThreads, 1) decode_program_kernel(const __grid_constant__ Params P)
{
    extern __shared__ __align__(128) uint8_t dynamic_memory[];
    __shared__ Shared sh;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t full0 = smem_u32(&sh.barriers[0]), empty0 = smem_u32(&sh.barriers[kRingStagesMax]);
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kRingStagesMax; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, kConsumerWarps);
        }
        sh.abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const uint32_t act_base = smem_u32(dynamic_memory);
    const uint32_t ring_base = act_base + P.act_bytes;
    if (warp == kConsumerWarps) {
        produce(P, sh, ring_base, lane);
        return;
    }
    Ring ring;
    uint32_t epoch = 0;
    // Operations are executed from shared memory: while one window of them runs, the next is on its way.
    const uint32_t *const words = reinterpret_cast<const uint32_t *>(P.ops);
    const uint32_t total_words = P.op_count * kOpWords;
    for (uint32_t i = threadIdx.x; i < kWindowOps * kOpWords; i += kConsumerThreads) {
        sh.window[0][i] = i < total_words ? __ldg(words + i) : 0u;
    }
    consumer_sync();
    for (uint32_t window0 = 0; window0 < P.op_count; window0 += kWindowOps) {
        const uint32_t buffer = (window0 / kWindowOps) & 1;
        static_assert(kWindowOps * kOpWords <= kConsumerThreads, "one word of the next window per thread");
        const uint32_t next_word = (window0 + kWindowOps) * kOpWords + threadIdx.x;
        const uint32_t next = (threadIdx.x < kWindowOps * kOpWords && next_word < total_words) ? __ldg(words + next_word) : 0u;
        const uint32_t window_end = min(P.op_count, window0 + kWindowOps);
        for (uint32_t index = window0; index < window_end; ++index) {
            const Op *op = reinterpret_cast<const Op *>(&sh.window[buffer][(index - window0) * kOpWords]);
            if (P.timeline && blockIdx.x == 0 && threadIdx.x == 0) {
                P.timeline[2 * index] = global_timer();
            }
            if (op->barrier) {
                grid_sync(P, sh, epoch);
            }
            if (P.timeline && blockIdx.x == 0 && threadIdx.x == 0) {
                P.timeline[2 * index + 1] = global_timer();
            }
            switch (op->kind) {
            case kOpEmbed: {
                const uint8_t *row = op->plane[0] + (uint64_t)P.token->token * op->row_bytes;
                for (uint32_t i = blockIdx.x * kConsumerThreads + threadIdx.x; i < op->columns; i += gridDim.x * kConsumerThreads) {
                    op->y[i] = decode_element(op->format, row, i);
                }
                break;
            }
            case kOpQuantize:
                if (op->norm_weight) {
                    quantize_local<kNormDepth, true>(op, sh, act_base);
                } else {
                    quantize_local<kPlainDepth, false>(op, sh, act_base);
                }
                break;
            case kOpMatvec:
                if (op->format == kFormatQ8Planar) {
                    ring = consume_matvec<Q8PlanarXq8>(op, P, sh, act_base, ring_base, ring);
                } else if (op->format == kFormatQ4K) {
                    ring = consume_matvec<Q4KXq8>(op, P, sh, act_base, ring_base, ring);
                } else {
                    ring = consume_matvec<Q6KPlanarXq8>(op, P, sh, act_base, ring_base, ring);
                }
                break;
            case kOpAttention:
                if (blockIdx.x < P.heads) {
                    attention_local(op, P, sh);
                }
                break;
            default:
                if (blockIdx.x == 0) {
                    argmax_local(P);
                }
                break;
            }
        }
        if (threadIdx.x < kWindowOps * kOpWords) {
            sh.window[buffer ^ 1][threadIdx.x] = next;
        }
        consumer_sync();
    }
    if (P.timeline && blockIdx.x == 0 && threadIdx.x == 0) {
        P.timeline[2 * P.op_count] = global_timer();
    }
}

}  // namespace prog
}  // namespace syn
