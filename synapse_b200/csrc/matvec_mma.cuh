// Q4_K and Q6_K x Q8_0-quantised activations for 2..8 tokens per launch on the integer tensor-core path (mma.sync,
// 8-bit operands, 32-bit accumulators): the batched-decode and short-prompt shape of synapse_q8_matvec_{2,4,8}
// (native/synapse-gpu/src/Features/GpuKernels/cuda/kernels/matmul.cu:79-145). Included at the end of matvec_xq8.cuh.
//
// Why: with dp4a every (row, token) pair costs its own unpack and dot instructions (about 200 warp instructions per
// row and token), so eight tokens take seven times the one-token time although the weights cross HBM once. One MMA
// takes the exact integer dots of a group of weights for 16 rows x 8 tokens at once; what is left per (row, token) is
// the FP32 combination of a unit's groups.
//
// Bit-identical to the one-token kernels. Those give lane l of team warp w the units (w * UPL + j) * 32 + l, j < UPL,
// evaluate F::dot for them one after the other on one accumulator, sum the 32 lanes with the xor butterfly (offsets 16,
// 8, 4, 2, 1) and then the team's warps in index order. Here a stage of the ring holds the units (w * UPL + j) * 32 ..
// + 31 of 16 rows; consumer warp i plays lanes i and i + 16: it evaluates their units with the same FP32 expression
// from the same integers, carries their accumulators from j to j + 1, and adds the two (the butterfly's first level).
// 128 threads, one per (row, token), then add the sixteen partial sums in the butterfly's tree order
// ((p0 + p8) + (p4 + p12)) + ... and the team's warps (the chunks w) in index order. Floating-point addition is
// commutative, so the tree is all that matters.
#pragma once

namespace syn {
namespace mv {

constexpr int kMmaWarps = 16;                  // multiplying warps
constexpr int kMmaCombineWarps = 4;            // 128 threads, one per (row, token) of a tile, that add the warps' partial sums
constexpr uint32_t kMmaSlots = 4;              // sets of partial sums in flight between the two, at most
constexpr uint32_t kMmaRows = 16;              // rows of a tile: M of the MMA
constexpr uint32_t kMmaTokens = 8;             // tokens of a group: N of the MMA
constexpr uint32_t kMmaChunkValues = 4096;     // the values one warp of a one-token team covers (32 lanes x UPL units)
constexpr uint32_t kMmaShared = 226u * 1024u;  // dynamic shared memory of the kernel (the CTA has the SM to itself)

// Shared memory: [activation buffer 0][activation buffer 1 (rows longer than a chunk)][ring of partial sums][running sums][stages].
// An activation buffer holds, for the eight tokens of the group, the part of the quantised activations that goes with
// one team warp's units (a chunk of at most 4096 values): codes | block scales | block sums. The CTA walks the chunks in
// the outer loop and its row tiles in the inner one, so a chunk's activations are fetched once per CTA and the next
// chunk's arrive (cp.async) while the current one is multiplied; the sums of a tile's finished chunks wait in the
// running area.
struct MmaArgs {
    WeightView weights;      // plane bases at the first row of the call
    uint64_t rows;
    uint64_t row_first;      // the call's first row inside the matrix (tensor maps describe whole planes)
    uint32_t row_bytes;      // Q4_K: bytes of a row
    uint32_t K;
    uint32_t units;          // values / Codec::kUnitValues
    uint32_t upl;            // units per lane of the one-token team
    uint32_t chunks;         // warps of the one-token team: ceil(units / (32 * upl))
    uint32_t tokens;
    uint32_t row_stride;     // bytes between the rows of a stage, chosen so that a warp's loads do not meet in a bank
    uint32_t code_stride;    // bytes between the tokens' activation codes in a buffer (chunk length plus the same kind of padding)
    uint32_t scale_stride;   // 32-bit words between the tokens' block scales, and between their block sums
    uint32_t buffer_bytes;   // one activation buffer
    uint32_t offset_scales, offset_sums;  // inside an activation buffer
    uint32_t offset_partial, offset_running, offset_stages;  // inside the dynamic shared memory
    uint32_t offset_tail;    // Q6_K: where, inside a stage, the tile's super-block scales (the d plane) start
    uint32_t stage_bytes, stages;
    uint32_t slots;          // sets of partial sums in the ring (kMmaSlots, or two when that buys a third stage)
};

// The tensor maps of a planar Q6_K matrix, passed to the kernel by value (the tiled bulk copy wants them in parameter,
// constant or global memory).
struct alignas(64) MmaMaps {
    unsigned char bytes[3][128];
};

// Tiled bulk copy of one box of a 3-D tensor map into shared memory; completion on an mbarrier, like bulk_copy.
__device__ __forceinline__ void tensor_copy(uint32_t dst, const void *map, int x, int y, int z, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
                 "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void mma_u8s8_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %11, %12, %13};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
}
__device__ __forceinline__ void mma_u8s8_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0)
{
    asm("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0, %1, %2, %3}, {%4, %5}, {%6}, {%7, %8, %9, %10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(0), "r"(0), "r"(0), "r"(0));
}

// Shared-memory loads by 32-bit shared address with a constant byte offset. (Plain C++ loads through pointers kept in a
// struct cost 64-bit address arithmetic per access: a third of this kernel's instructions before these were used.)
// volatile: they must stay behind the wait for the stage and ahead of its hand-back.
template <int OFFSET = 0>
__device__ __forceinline__ uint4 lds128(uint32_t a)
{
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4+%5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a), "n"(OFFSET));
    return v;
}
template <int OFFSET = 0>
__device__ __forceinline__ float4 lds128f(uint32_t a)
{
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4+%5];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a), "n"(OFFSET));
    return v;
}
template <int OFFSET = 0>
__device__ __forceinline__ uint2 lds64(uint32_t a)
{
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(a), "n"(OFFSET));
    return v;
}
template <int OFFSET = 0>
__device__ __forceinline__ uint32_t lds32(uint32_t a)
{
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(a), "n"(OFFSET));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t a)
{
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
    return v;
}

// What a multiplying thread knows about its place: byte offsets and 32-bit shared addresses, set once per chunk.
struct MmaContext {
    uint32_t g, tig;        // the MMA's group (lane / 4) and thread-in-group (lane % 4): B column g, C columns 2 tig, 2 tig + 1
    uint32_t row0, row8;    // offset of row g inside a stage, and the distance to row g + 8
    uint32_t codes;         // the chunk's activation codes of token g, at this thread's k positions
    uint32_t scales, sums;  // the chunk's block scales and block sums of token 2 tig
    uint32_t token_step;    // distance to token 2 tig + 1 in both
    uint32_t tail;          // Q6_K: offset of row g's super-block scales inside a stage (the tile's shift included)
};

// ------------------------------------------------------------------------------------------------------
// Q4_K (file layout). Unit = half a super-block = sub-blocks 4h .. 4h+3; a stage holds 32 units = 16 super-blocks of
// every row, rows row_stride apart. One m16n8k32 per sub-block; the high nibbles are multiplied in place (sixteen times
// the dot, as Q4KXq8::dot has it).
// ------------------------------------------------------------------------------------------------------
struct Q4KMma {
    using Format = Q4KXq8;
    static constexpr uint32_t kUnitValues = 128;
    static void layout(MmaArgs &m)
    {
        const uint32_t piece = (m.units < 32 ? m.units : 32) * 72;
        m.row_stride = (uint32_t)align_up(piece, 128) + 32;  // 8-byte loads of rows g = 0..3 and tig = 0..3 cover the 32 banks
        m.offset_tail = 0;
        m.stage_bytes = kMmaRows * m.row_stride;
        m.code_stride = (m.K < kMmaChunkValues ? m.K : kMmaChunkValues) + 32;
    }

    static __device__ __forceinline__ void produce(const MmaArgs &m, const MmaMaps &, uint32_t stage, uint64_t row0, uint32_t n, uint32_t w, uint32_t j,
                                                   uint32_t lane, uint32_t bar, uint64_t policy)
    {
        const uint32_t first = (w * m.upl + j) * 32;                // first unit of the stage
        const uint32_t piece = min(32u, m.units - first) * 72u;  // a multiple of 144: rows hold whole super-blocks
        if (lane == 0) {
            mbar_expect_tx(bar, n * piece);
        }
        __syncwarp();
        if (lane < n) {
            bulk_copy(stage + lane * m.row_stride, m.weights.p0 + (row0 + lane) * m.row_bytes + (uint64_t)first * 72, piece, bar, policy);
        }
    }
    // The block sums arrive as the quantiser's pairs of 16-code sums; the min term wants scale * (sum of the block's
    // codes), computed as Q4KXq8::load_act computes it, in place.
    static __device__ __forceinline__ void finish_sums(const MmaArgs &m, uint8_t *buffer, uint32_t blocks, uint32_t thread, uint32_t threads)
    {
        const float *const scales = reinterpret_cast<const float *>(buffer + m.offset_scales);
        uint32_t *const sums = reinterpret_cast<uint32_t *>(buffer + m.offset_sums);
        for (uint32_t i = thread; i < kMmaTokens * blocks; i += threads) {
            const uint32_t index = (i / blocks) * m.scale_stride + i % blocks;
            const uint32_t pair = sums[index];
            sums[index] = __float_as_uint(scales[index] * (float)((int)(short)(pair & 0xffff) + (int)(short)(pair >> 16)));
        }
    }

    static __device__ __forceinline__ void place(const MmaArgs &m, MmaContext &c, uint32_t buffer)
    {
        c.row0 = c.g * m.row_stride;
        c.row8 = 8 * m.row_stride;
        c.codes = buffer + c.g * m.code_stride + 8 * c.tig;
        c.scales = buffer + m.offset_scales + 2 * c.tig * m.scale_stride * 4;
        c.sums = buffer + m.offset_sums + 2 * c.tig * m.scale_stride * 4;
        c.token_step = m.scale_stride * 4;
    }
    static __device__ __forceinline__ void place_tile(const MmaArgs &, MmaContext &, uint64_t) {}

    // Adds unit `u` (lane `local` of team warp w at step j; unit `ur` of the chunk) to the accumulators of this thread's
    // four (row, token) pairs. `stage` is the stage's shared address.
    static __device__ __forceinline__ void unit(const MmaArgs &, const MmaContext &c, uint32_t stage, uint32_t local, uint32_t ur, uint32_t, float (&acc)[4])
    {
        const uint32_t block = stage + c.row0 + (local >> 1) * 144;
        const uint4 h0 = lds128(block), h1 = lds128(block + c.row8);
        // this thread's eight bytes of each 32-byte nibble run: k positions (tig, byte) of the MMA, and the same eight
        // positions of the activation codes below
        const uint32_t q = block + 16 + (local & 1) * 64 + 8 * c.tig;
        const uint2 a00 = lds64<0>(q), a01 = lds64<32>(q), a10 = lds64<0>(q + c.row8), a11 = lds64<32>(q + c.row8);
        const uint32_t b = c.codes + ur * 128;
        const uint2 b0 = lds64<0>(b), b1 = lds64<32>(b), b2 = lds64<64>(b), b3 = lds64<96>(b);
        int lo0[4], hi0[4], lo1[4], hi1[4];
        constexpr uint32_t kLow = 0x0F0F0F0Fu, kHigh = 0xF0F0F0F0u;
        mma_u8s8_k32(lo0, a00.x & kLow, a10.x & kLow, a00.y & kLow, a10.y & kLow, b0.x, b0.y);
        mma_u8s8_k32(hi0, a00.x & kHigh, a10.x & kHigh, a00.y & kHigh, a10.y & kHigh, b1.x, b1.y);
        mma_u8s8_k32(lo1, a01.x & kLow, a11.x & kLow, a01.y & kLow, a11.y & kLow, b2.x, b2.y);
        mma_u8s8_k32(hi1, a01.x & kHigh, a11.x & kHigh, a01.y & kHigh, a11.y & kHigh, b3.x, b3.y);
        // 6-bit scales and mins of the unit's four sub-blocks, one per byte (as in Q4KXq8::dot)
        uint32_t sc[2], mn[2];
        if ((local & 1) == 0) {
            sc[0] = h0.y & 0x3f3f3f3fu;
            mn[0] = h0.z & 0x3f3f3f3fu;
            sc[1] = h1.y & 0x3f3f3f3fu;
            mn[1] = h1.z & 0x3f3f3f3fu;
        } else {
            sc[0] = (h0.w & 0x0f0f0f0fu) | ((h0.y >> 2) & 0x30303030u);
            mn[0] = ((h0.w >> 4) & 0x0f0f0f0fu) | ((h0.z >> 2) & 0x30303030u);
            sc[1] = (h1.w & 0x0f0f0f0fu) | ((h1.y >> 2) & 0x30303030u);
            mn[1] = ((h1.w >> 4) & 0x0f0f0f0fu) | ((h1.z >> 2) & 0x30303030u);
        }
        const float d[2] = {half_bits_to_float(h0.x & 0xffff), half_bits_to_float(h1.x & 0xffff)};
        const float dmin[2] = {half_bits_to_float(h0.x >> 16), half_bits_to_float(h1.x >> 16)};
        const float4 ad[2] = {lds128f(c.scales + ur * 16), lds128f(c.scales + c.token_step + ur * 16)};
        const float4 as[2] = {lds128f(c.sums + ur * 16), lds128f(c.sums + c.token_step + ur * 16)};
        // accumulator [2 * row + token]: row g / g + 8, token 2 tig / 2 tig + 1 -- the MMA's C fragment order
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const int row = p >> 1, token = p & 1;
            // the expression of Q4KXq8::dot
            float f_lo = (byte_to_float(sc[row], 0) * small_int_to_float(lo0[p])) * ad[token].x;
            f_lo = fmaf(byte_to_float(sc[row], 2) * small_int_to_float(lo1[p]), ad[token].z, f_lo);
            float f_hi = (byte_to_float(sc[row], 1) * small_int_to_float(hi0[p])) * ad[token].y;
            f_hi = fmaf(byte_to_float(sc[row], 3) * small_int_to_float(hi1[p]), ad[token].w, f_hi);
            float gm = byte_to_float(mn[row], 0) * as[token].x;
            gm = fmaf(byte_to_float(mn[row], 1), as[token].y, gm);
            gm = fmaf(byte_to_float(mn[row], 2), as[token].z, gm);
            gm = fmaf(byte_to_float(mn[row], 3), as[token].w, gm);
            acc[p] = fmaf(d[row], fmaf(f_hi, 0.0625f, f_lo), acc[p]);
            acc[p] = fmaf(-dmin[row], gm, acc[p]);
        }
    }
};

// ------------------------------------------------------------------------------------------------------
// Q6_K (planes: ql | qh | int8 scales | fp16 super-block scales). Unit = 64 values: bytes l = 16 i .. 16 i + 15 of half h
// of super-block u / 4, four groups of 16 values with their own scales. A stage holds 32 units = 8 super-blocks of every
// row and, behind them, the tile's part of the d plane. One m16n8k16 per group of 16 values.
// TILED: the three big planes arrive as one tiled bulk copy each (a box of 16 rows), laid out [segment of 128 bytes][row]
// with the 128-byte swizzle, whose key is the row: 16-byte piece p of a row's segment sits at piece p ^ (row % 8), so the
// eight rows a warp reads at one column are in different banks. A stage is ql 8 x 16 x 128 | qh 4 x 16 x 128 | scales
// 1 x 16 x 128 | d. Otherwise (no tensor maps to be had): one plain bulk copy per row and plane (49 per stage, which is
// what the multiplying warps then wait for a third of the time), rows row_stride apart (ql 1024, qh 512, scales 128 bytes).
// ------------------------------------------------------------------------------------------------------
template <bool TILED>
struct Q6KMmaT {
    using Format = Q6KPlanarXq8;
    static constexpr uint32_t kUnitValues = 64;
    static constexpr uint32_t kQh = 8 * 16 * 128, kScales = kQh + 4 * 16 * 128, kBoxBytes = kScales + 16 * 128;  // inside a tiled stage
    static void layout(MmaArgs &m)
    {
        const uint32_t sbs = m.units < 32 ? m.units / 4 : 8;  // super-blocks of a stage
        if (TILED) {
            m.row_stride = 128;
            m.offset_tail = kBoxBytes;
        } else {
            // 4-byte loads of rows g = 0..7 and tig = 0..3 cover the 32 banks when the stride is 16 more than a multiple of 128
            m.row_stride = (uint32_t)align_up(sbs * (128 + 64 + 16), 128) + 16;
            m.offset_tail = kMmaRows * m.row_stride;
        }
        // the 16 rows' super-block scales are contiguous in their plane: one copy from the 16-byte boundary below them
        // (stages are multiples of 1024 bytes: the swizzle's period)
        m.stage_bytes = (uint32_t)align_up(m.offset_tail + kMmaRows * (m.K / 128) + 32, 1024);
        m.code_stride = (m.K < kMmaChunkValues ? m.K : kMmaChunkValues) + 16;
    }

    static __device__ __forceinline__ void produce(const MmaArgs &m, const MmaMaps &maps, uint32_t stage, uint64_t row0, uint32_t n, uint32_t w, uint32_t j,
                                                   uint32_t lane, uint32_t bar, uint64_t policy)
    {
        const uint32_t first = (w * m.upl + j) * 32;            // first unit of the stage
        const uint32_t sb0 = first / 4, sbs = min(32u, m.units - first) / 4;
        const uint8_t *const tail = m.weights.p3 + row0 * (m.K / 128);
        const uint32_t shift = (uint32_t)(reinterpret_cast<uintptr_t>(tail) & 15);
        const uint32_t tail_bytes = (shift + n * (m.K / 128) + 15) & ~15u;
        if (TILED) {
            // Boxes are always whole: rows past the matrix read as zero, segments past the row's end are never looked at.
            // Coordinates: byte 0 of the segment (a multiple of 16, as a tiled copy needs), the row, the segment.
            if (lane == 0) {
                const int row = (int)(m.row_first + row0);
                mbar_expect_tx(bar, kBoxBytes + tail_bytes);
                tensor_copy(stage, maps.bytes[0], 0, row, (int)sb0, bar);
                tensor_copy(stage + kQh, maps.bytes[1], 0, row, (int)(sb0 / 2), bar);
                tensor_copy(stage + kScales, maps.bytes[2], 0, row, (int)(sb0 / 8), bar);
                bulk_copy(stage + m.offset_tail, tail - shift, tail_bytes, bar, policy);
            }
            return;
        }
        if (lane == 0) {
            mbar_expect_tx(bar, n * sbs * (128 + 64 + 16) + tail_bytes);
            bulk_copy(stage + m.offset_tail, tail - shift, tail_bytes, bar, policy);
        }
        __syncwarp();
        if (lane < n) {
            const uint64_t row = row0 + lane;
            const uint32_t base = stage + lane * m.row_stride;
            bulk_copy(base, m.weights.p0 + row * (m.K / 2) + (uint64_t)sb0 * 128, sbs * 128, bar, policy);
            bulk_copy(base + sbs * 128, m.weights.p1 + row * (m.K / 4) + (uint64_t)sb0 * 64, sbs * 64, bar, policy);
            bulk_copy(base + sbs * 192, m.weights.p2 + row * (m.K / 16) + (uint64_t)sb0 * 16, sbs * 16, bar, policy);
        }
    }
    // the quantiser's sums of every 16 codes are used as they are
    static __device__ __forceinline__ void finish_sums(const MmaArgs &, uint8_t *, uint32_t, uint32_t, uint32_t) {}

    static __device__ __forceinline__ void place(const MmaArgs &m, MmaContext &c, uint32_t buffer)
    {
        c.row0 = c.g * m.row_stride;
        c.row8 = 8 * m.row_stride;
        c.codes = buffer + c.g * m.code_stride + 4 * c.tig;
        c.scales = buffer + m.offset_scales + 2 * c.tig * m.scale_stride * 4;
        c.sums = buffer + m.offset_sums + 2 * c.tig * m.scale_stride * 4;
        c.token_step = m.scale_stride * 4;
    }
    // the tile's part of the d plane was copied from the 16-byte boundary below its first byte
    static __device__ __forceinline__ void place_tile(const MmaArgs &m, MmaContext &c, uint64_t row0)
    {
        c.tail = m.offset_tail + (uint32_t)(reinterpret_cast<uintptr_t>(m.weights.p3 + row0 * (m.K / 128)) & 15) + c.g * (m.K / 128);
    }

    static __device__ __forceinline__ void unit(const MmaArgs &m, const MmaContext &c, uint32_t stage, uint32_t local, uint32_t ur, uint32_t u, float (&acc)[4])
    {
        const uint32_t sbs = min(32u, m.units - (u - local)) / 4;  // super-blocks the stage holds
        const uint32_t sb = local >> 2, h = (local >> 1) & 1, i = local & 1;
        const uint32_t row = stage + c.row0;
        uint32_t a0, b0, h0, a1, b1, h1;
        if (TILED) {
            // segment of ql = the super-block; of qh = a pair of them; 16-byte piece p of the row's segment is at p ^ g
            // (rows g and g + 8 have the same key)
            const uint32_t ql = row + sb * 2048 + 4 * c.tig, qh = row + kQh + (sb >> 1) * 2048 + 4 * c.tig;
            const uint32_t pa = ((h * 4 + i) ^ c.g) << 4, pb = ((h * 4 + i + 2) ^ c.g) << 4, ph = (((sb & 1) * 4 + h * 2 + i) ^ c.g) << 4;
            a0 = lds32<0>(ql + pa), b0 = lds32<0>(ql + pb), h0 = lds32<0>(qh + ph);
            a1 = lds32<1024>(ql + pa), b1 = lds32<1024>(ql + pb), h1 = lds32<1024>(qh + ph);
        } else {
            const uint32_t ql = row + sb * 128 + h * 64 + i * 16 + 4 * c.tig, qh = row + sbs * 128 + sb * 64 + h * 32 + i * 16 + 4 * c.tig;
            a0 = lds32<0>(ql), b0 = lds32<32>(ql), h0 = lds32<0>(qh);
            a1 = lds32<0>(ql + c.row8), b1 = lds32<32>(ql + c.row8), h1 = lds32<0>(qh + c.row8);
        }
        uint32_t v0[4], v1[4];
        q6k_codes(a0, b0, h0, v0[0], v0[1], v0[2], v0[3]);
        q6k_codes(a1, b1, h1, v1[0], v1[1], v1[2], v1[3]);
        // activation codes of group q: 16 codes at sb * 256 + h * 128 + i * 16 + 32 q of the chunk; this thread's four
        const uint32_t b = c.codes + (ur >> 2) * 256 + h * 128 + i * 16;
        const uint32_t codes[4] = {lds32<0>(b), lds32<32>(b), lds32<64>(b), lds32<96>(b)};
        int dots[4][4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            mma_u8s8_k16(dots[q], v0[q], v1[q], codes[q]);
        }
        // the eight int8 scales of the half, and the super-block scale
        const uint32_t sc = TILED ? row + kScales + ((sb ^ c.g) << 4) + h * 8 : row + sbs * 192 + sb * 16 + h * 8;
        const uint2 s0 = lds64<0>(sc), s1 = lds64<0>(sc + c.row8);
        const uint32_t tail = stage + c.tail + (u >> 2) * 2;
        const float d[2] = {half_bits_to_float(lds16(tail)), half_bits_to_float(lds16(tail + 8 * (m.K / 128)))};
        const float4 ad[2] = {lds128f(c.scales + (ur >> 1) * 16), lds128f(c.scales + c.token_step + (ur >> 1) * 16)};
        // the sums of the eight 16-code groups of the half, two per word: group q of this unit is half i of word q
        const uint4 as[2] = {lds128(c.sums + (ur >> 1) * 16), lds128(c.sums + c.token_step + (ur >> 1) * 16)};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint32_t word0 = q < 2 ? s0.x : s0.y, word1 = q < 2 ? s1.x : s1.y;
            const int scale[2] = {(int)(signed char)((word0 >> (8 * (2 * (q & 1) + i))) & 0xff), (int)(signed char)((word1 >> (8 * (2 * (q & 1) + i))) & 0xff)};
            const float adq[2] = {q == 0 ? ad[0].x : q == 1 ? ad[0].y : q == 2 ? ad[0].z : ad[0].w, q == 0 ? ad[1].x : q == 1 ? ad[1].y : q == 2 ? ad[1].z : ad[1].w};
            const uint32_t pair0 = q == 0 ? as[0].x : q == 1 ? as[0].y : q == 2 ? as[0].z : as[0].w;
            const uint32_t pair1 = q == 0 ? as[1].x : q == 1 ? as[1].y : q == 2 ? as[1].z : as[1].w;
            const int asq[2] = {(int)(short)(i ? pair0 >> 16 : pair0 & 0xffff), (int)(short)(i ? pair1 >> 16 : pair1 & 0xffff)};
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                const int row_index = p >> 1, token = p & 1;
                // the expression of q6k_dot
                const int dot = dots[q][p] - 32 * asq[token];
                acc[p] = fmaf((d[row_index] * small_int_to_float(scale[row_index])) * adq[token], small_int_to_float(dot), acc[p]);
            }
        }
    }
};
using Q6KMma = Q6KMmaT<false>;
using Q6KTiledMma = Q6KMmaT<true>;

__device__ __forceinline__ void copy16_async(void *shared, const void *global)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(shared)), "l"(global) : "memory");
}
__device__ __forceinline__ void copies_async_wait() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// Starts the copy of chunk w's activations (the group's tokens token0 .. token0 + live - 1; the others read as zero)
// into `buffer`: 16-byte pieces, asynchronous where they come from memory.
__device__ __forceinline__ void fetch_chunk(const MmaArgs &m, const ActView &act, uint64_t token0, uint32_t live, uint32_t w, uint8_t *buffer, uint32_t thread,
                                            uint32_t threads)
{
    const uint32_t value0 = w * kMmaChunkValues, values = min(kMmaChunkValues, m.K - value0);
    const uint32_t code_pieces = values / 16, word_pieces = values / 128;  // 16-byte pieces per token: codes; scales and sums (4 bytes per 32 values)
    const uint32_t per_token = code_pieces + 2 * word_pieces;
    for (uint32_t i = thread; i < kMmaTokens * per_token; i += threads) {
        const uint32_t t = i / per_token, piece = i % per_token;
        uint8_t *destination;
        const uint8_t *source;
        if (piece < code_pieces) {
            destination = buffer + t * m.code_stride + piece * 16;
            source = reinterpret_cast<const uint8_t *>(act.codes) + (token0 + t) * m.K + value0 + piece * 16;
        } else if (piece < code_pieces + word_pieces) {
            destination = buffer + m.offset_scales + t * m.scale_stride * 4 + (piece - code_pieces) * 16;
            source = reinterpret_cast<const uint8_t *>(act.scales) + ((token0 + t) * (m.K / 32) + value0 / 32) * 4 + (piece - code_pieces) * 16;
        } else {
            destination = buffer + m.offset_sums + t * m.scale_stride * 4 + (piece - code_pieces - word_pieces) * 16;
            source = reinterpret_cast<const uint8_t *>(act.sums) + ((token0 + t) * (m.K / 16) + value0 / 16) * 2 + (piece - code_pieces - word_pieces) * 16;
        }
        if (t < live) {
            copy16_async(destination, source);
        } else {
            *reinterpret_cast<uint4 *>(destination) = make_uint4(0, 0, 0, 0);
        }
    }
}

template <class Codec, bool GATHER>
__global__ void __launch_bounds__((kMmaWarps + 1 + kMmaCombineWarps) * 32, 1)
matvec_mma_kernel(MmaArgs m, const __grid_constant__ MmaMaps maps, ActView act, float *__restrict__ y, uint64_t out_stride, Epilogue epilogue,
                  uint32_t *fault)
{
    extern __shared__ __align__(128) uint8_t mma_memory[];
    __shared__ __align__(8) uint64_t barriers[2 * kMaxStages + 2 * kMmaSlots];  // full[s], empty[s]; sums_full[k], sums_empty[k]
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint64_t tiles = (m.rows + kMmaRows - 1) / kMmaRows;
    const uint32_t my_tiles = tiles > blockIdx.x ? (uint32_t)((tiles - blockIdx.x + gridDim.x - 1) / gridDim.x) : 0;
    const uint32_t full0 = smem_u32(&barriers[0]), empty0 = smem_u32(&barriers[kMaxStages]);
    const uint32_t sums_full0 = smem_u32(&barriers[2 * kMaxStages]), sums_empty0 = smem_u32(&barriers[2 * kMaxStages + kMmaSlots]);
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < m.stages; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, kMmaWarps);
        }
        for (uint32_t k = 0; k < m.slots; ++k) {
            mbar_init(sums_full0 + 8 * k, kMmaWarps);
            mbar_init(sums_empty0 + 8 * k, kMmaCombineWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == kMmaWarps) {
        // ---- producer: one stage per (team warp w, tile, step j), one bulk copy per row and plane ----
        const uint64_t policy = l2_evict_first_policy();
        const uint32_t stage0 = (smem_u32(mma_memory) + m.offset_stages + 1023) & ~1023u;  // the swizzle's period
        uint32_t s = 0, round = 0;
        for (uint32_t w = 0; w < m.chunks; ++w) {
            for (uint32_t it = 0; it < my_tiles; ++it) {
                const uint64_t row0 = ((uint64_t)blockIdx.x + (uint64_t)it * gridDim.x) * kMmaRows;
                const uint32_t n = (uint32_t)min((uint64_t)kMmaRows, m.rows - row0);
                for (uint32_t j = 0; j < m.upl; ++j) {
                    if ((w * m.upl + j) * 32 >= m.units) {
                        break;  // the last team warp's lanes have no unit at this step
                    }
                    if (round > 0 && !mbar_wait(empty0 + 8 * s, (round - 1) & 1) && fault && lane == 0) {
                        atomicAdd(fault, 1u);
                    }
                    Codec::produce(m, maps, stage0 + s * m.stage_bytes, row0, n, w, j, lane, full0 + 8 * s, policy);
                    if (++s == m.stages) {
                        s = 0;
                        ++round;
                    }
                }
            }
        }
        return;
    }

    constexpr uint32_t kThreads = kMmaWarps * 32;
    const uint64_t token0 = (uint64_t)blockIdx.y * kMmaTokens;
    const uint32_t live = min(kMmaTokens, m.tokens - (uint32_t)token0);
    float *const partial = reinterpret_cast<float *>(mma_memory + m.offset_partial);  // [kMmaSlots][kMmaWarps][128]
    float *const running = reinterpret_cast<float *>(mma_memory + m.offset_running);  // [my_tiles][128] when the team has several warps

    if (warp > kMmaWarps) {
        // ---- combining warps: thread p owns (row p / 8, token p % 8) of every tile. They take the multiplying warps'
        // partial sums through a ring of kMmaSlots sets (mbarriers, no CTA-wide barrier), so the multiplying warps
        // never wait for the additions and drift apart instead of running every stage in lockstep.
        const uint32_t pair = threadIdx.x - (kMmaWarps + 1) * 32;
        const uint32_t out_row = pair >> 3, out_token = pair & 7;
        pdl_wait();
        uint32_t slot = 0, slot_phase = 0;
        for (uint32_t w = 0; w < m.chunks; ++w) {
            for (uint32_t it = 0; it < my_tiles; ++it) {
                const uint64_t row0 = ((uint64_t)blockIdx.x + (uint64_t)it * gridDim.x) * kMmaRows;
                if (!mbar_wait(sums_full0 + 8 * slot, slot_phase) && fault && lane == 0) {
                    atomicAdd(fault, 1u);
                }
                const float *const p = partial + slot * kMmaWarps * 128 + pair;
                float level[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    level[i] = p[i * 128] + p[(i + 8) * 128];  // offset 8
                }
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(sums_empty0 + 8 * slot);  // the values are in registers
                }
                if (++slot == m.slots) {
                    slot = 0;
                    slot_phase ^= 1;
                }
                const float c0 = level[0] + level[4], c1 = level[1] + level[5], c2 = level[2] + level[6], c3 = level[3] + level[7];  // offset 4
                const float e = (c0 + c2) + (c1 + c3);  // offsets 2 and 1
                // the team's warps in index order
                const float total = w == 0 ? e : running[it * 128 + pair] + e;
                if (w + 1 < m.chunks) {
                    running[it * 128 + pair] = total;
                } else if (row0 + out_row < m.rows && out_token < live) {
                    store_result<GATHER>(epilogue, y, token0 + out_token, out_stride, row0 + out_row, total);
                }
            }
        }
        if (GATHER) {
            asm volatile("bar.sync 2, %0;" ::"n"(kMmaCombineWarps * 32) : "memory");
            if (pair == 0) {
                signal_completion(epilogue);
            }
        }
        return;
    }

    // ---- multiplying warps ------------------------------------------------------------------------------
    pdl_wait();
    fetch_chunk(m, act, token0, live, 0, mma_memory, threadIdx.x, kThreads);
    copies_async_wait();
    consumer_barrier<kThreads>();
    Codec::finish_sums(m, mma_memory, min(kMmaChunkValues, m.K) / 32, threadIdx.x, kThreads);
    consumer_barrier<kThreads>();

    MmaContext c{};
    c.g = lane >> 2;
    c.tig = lane & 3;
    uint32_t s = 0, phase = 0, slot = 0, slot_round = 0;
    for (uint32_t w = 0; w < m.chunks; ++w) {
        uint8_t *const acts = mma_memory + (w & 1) * m.buffer_bytes;
        if (w + 1 < m.chunks) {
            // the other buffer was last read in chunk w - 1, which every warp has left (the barrier that ended it)
            fetch_chunk(m, act, token0, live, w + 1, mma_memory + ((w + 1) & 1) * m.buffer_bytes, threadIdx.x, kThreads);
        }
        Codec::place(m, c, smem_u32(acts));
        const uint32_t chunk_unit = w * m.upl * 32;
        for (uint32_t it = 0; it < my_tiles; ++it) {
            const uint64_t row0 = ((uint64_t)blockIdx.x + (uint64_t)it * gridDim.x) * kMmaRows;
            Codec::place_tile(m, c, row0);
            float acc[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};  // lanes warp and warp + 16 of team warp w
            for (uint32_t j = 0; j < m.upl; ++j) {
                const uint32_t first = (w * m.upl + j) * 32;
                if (first >= m.units) {
                    break;
                }
                if (!mbar_wait(full0 + 8 * s, phase) && fault && lane == 0) {
                    atomicAdd(fault, 1u);
                }
                const uint32_t stage = ((smem_u32(mma_memory) + m.offset_stages + 1023) & ~1023u) + s * m.stage_bytes;
                const uint32_t ur = first - chunk_unit + warp;  // place in the chunk of the unit of lane `warp`
                if (first + warp + 16 < m.units) {
                    // both lanes have a unit (the usual case): one straight run of code, so that the two independent
                    // chains of loads, MMAs and FP32 operations can be interleaved
                    Codec::unit(m, c, stage, warp, ur, first + warp, acc[0]);
                    Codec::unit(m, c, stage, warp + 16, ur + 16, first + warp + 16, acc[1]);
                } else if (first + warp < m.units) {
                    Codec::unit(m, c, stage, warp, ur, first + warp, acc[0]);
                }
                // Give the stage back: the shared-memory reads above have retired (their values were used), the fence
                // orders them before the producer's next bulk copy into the stage.
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(empty0 + 8 * s);
                }
                if (++s == m.stages) {
                    s = 0;
                    phase ^= 1;
                }
            }
            // first level of the butterfly: lane i + lane i + 16; the set goes to the combining warps
            if (slot_round > 0 && !mbar_wait(sums_empty0 + 8 * slot, (slot_round - 1) & 1) && fault && lane == 0) {
                atomicAdd(fault, 1u);
            }
            float *const mine = partial + (slot * kMmaWarps + warp) * 128;
            *reinterpret_cast<float2 *>(mine + c.g * 8 + 2 * c.tig) = make_float2(acc[0][0] + acc[1][0], acc[0][1] + acc[1][1]);
            *reinterpret_cast<float2 *>(mine + (c.g + 8) * 8 + 2 * c.tig) = make_float2(acc[0][2] + acc[1][2], acc[0][3] + acc[1][3]);
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(sums_full0 + 8 * slot);  // release: the warp's stores above are visible to who sees the phase complete
            }
            if (++slot == m.slots) {
                slot = 0;
                ++slot_round;
            }
        }
        if (w + 1 < m.chunks) {
            copies_async_wait();
            consumer_barrier<kThreads>();
            Codec::finish_sums(m, mma_memory + ((w + 1) & 1) * m.buffer_bytes, min(kMmaChunkValues, m.K - (w + 1) * kMmaChunkValues) / 32, threadIdx.x, kThreads);
            consumer_barrier<kThreads>();
        }
    }
}

// Lays the shared memory out for `a` and launches; cudaErrorNotSupported when two stages and the running sums of the
// CTA's tiles do not fit beside the activation buffers, so that the caller falls back to the dp4a kernels.
template <class Codec, bool GATHER>
cudaError_t launch_mma(const MatvecArgs &a, const WeightView &view, uint32_t upl, const unsigned char (*tensor_maps)[128], cudaStream_t stream)
{
    MmaArgs m{};
    m.weights = view;
    m.rows = a.row_count;
    m.row_first = a.row_start;
    m.row_bytes = (uint32_t)a.matrix->row_bytes;
    m.K = (uint32_t)a.matrix->columns;
    m.units = m.K / Codec::kUnitValues;  // (F::units is device code)
    m.upl = upl;
    m.chunks = (m.units + 32 * upl - 1) / (32 * upl);
    m.tokens = (uint32_t)a.tokens;
    if (m.chunks > 1 && upl * 32 * Codec::kUnitValues != kMmaChunkValues) {
        return cudaErrorNotSupported;  // a team warp always covers 4096 values when the team has several
    }
    Codec::layout(m);
    const uint32_t chunk_values = m.K < kMmaChunkValues ? m.K : kMmaChunkValues;
    m.scale_stride = chunk_values / 32 + 4;
    m.offset_scales = (uint32_t)align_up((uint64_t)kMmaTokens * m.code_stride, 128);
    m.offset_sums = m.offset_scales + (uint32_t)align_up((uint64_t)kMmaTokens * m.scale_stride * 4, 128);
    m.buffer_bytes = m.offset_sums + (uint32_t)align_up((uint64_t)kMmaTokens * m.scale_stride * 4, 128);
    uint64_t ctas = (a.row_count + kMmaRows - 1) / kMmaRows;
    const uint64_t cap = (uint64_t)sm_count(a.matrix->device);
    const uint64_t tiles_per_cta = ctas > cap ? (ctas + cap - 1) / cap : 1;
    if (ctas > cap) {
        ctas = cap;
    }
    m.offset_partial = (m.chunks > 1 ? 2 : 1) * m.buffer_bytes;
    // stages matter more than sets of partial sums: four sets only where they do not cost a stage
    auto lay = [&](uint32_t slots) {
        m.slots = slots;
        m.offset_running = m.offset_partial + slots * kMmaWarps * 128 * 4;  // behind the ring of partial sums
        m.offset_stages = m.offset_running + (m.chunks > 1 ? (uint32_t)tiles_per_cta * 128 * 4 : 0);
        // (up to 1023 bytes go into starting the stages on a multiple of 1024)
        const uint32_t stages = m.offset_stages + 1024 < kMmaShared ? (kMmaShared - 1024 - m.offset_stages) / m.stage_bytes : 0;
        m.stages = stages > (uint32_t)kMaxStages ? (uint32_t)kMaxStages : stages;
    };
    lay(2);
    const uint32_t with_two = m.stages;
    lay(kMmaSlots);
    if (m.stages < with_two) {
        lay(2);
    }
    if (m.stages < 2) {
        return cudaErrorNotSupported;
    }
    auto kernel = matvec_mma_kernel<Codec, GATHER>;
    static PerDevice configured;
    if (configured.first_use(a.matrix->device)) {
        cudaError_t error = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMmaShared);
        if (error != cudaSuccess) {
            configured.forget(a.matrix->device);
            return error;
        }
    }
    const dim3 grid((unsigned)ctas, (unsigned)((a.tokens + kMmaTokens - 1) / kMmaTokens));
    MmaMaps maps{};
    if (tensor_maps) {
        memcpy(maps.bytes, tensor_maps, sizeof(maps.bytes));
    }
    return launch_kernel(kernel, grid, dim3((kMmaWarps + 1 + kMmaCombineWarps) * 32), (size_t)kMmaShared, stream, m, maps, a.act, a.y, a.out_stride, a.fused,
                         fault_word_device());
}

template <class F, bool GATHER>
cudaError_t launch_tensor_core_tokens(const MatvecArgs &a, const WeightView &view, uint32_t upl, cudaStream_t stream)
{
    if constexpr (std::is_same<F, Q4KXq8>::value) {
        return launch_mma<Q4KMma, GATHER>(a, view, upl, nullptr, stream);
    } else if constexpr (std::is_same<F, Q6KPlanarXq8>::value) {
        const unsigned char(*tensor_maps)[128] = q6k_tensor_maps(a.matrix);
        return tensor_maps ? launch_mma<Q6KTiledMma, GATHER>(a, view, upl, tensor_maps, stream) : launch_mma<Q6KMma, GATHER>(a, view, upl, nullptr, stream);
    } else {
        return cudaErrorNotSupported;
    }
}

}  // namespace mv
}  // namespace syn
