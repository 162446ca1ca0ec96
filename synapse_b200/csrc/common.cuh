// Internal declarations shared by the translation units of libsynapse_b200.so (sm_100a only).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <exception>
#include <new>
#include <string>

#include "../../include/synapse_b200.h"

namespace syn {

constexpr uint32_t kQ8_0 = SYN_B200_TYPE_Q8_0;
constexpr uint32_t kQ4_K = SYN_B200_TYPE_Q4_K;
constexpr uint32_t kQ6_K = SYN_B200_TYPE_Q6_K;

constexpr int kMaxMatvecTokens = 8;  // tokens one matrix-vector launch group handles (cuda/kernels/matmul.cu:112-115)

inline uint64_t block_values(uint32_t type) { return type == kQ8_0 ? 32 : (type == kQ4_K || type == kQ6_K) ? 256 : 0; }
inline uint64_t block_bytes(uint32_t type) { return type == kQ8_0 ? 34 : type == kQ4_K ? 144 : type == kQ6_K ? 210 : 0; }
inline uint64_t align_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

// Device-resident weights. `layout` says how `data` is organised.
enum class Layout : uint32_t {
    Natural = 0,  // GGUF blocks exactly as in the file, rows contiguous
    Planar = 1,   // per-field planes, each plane row-major and 16-byte friendly (see repack.cu)
};

struct PlaneOffsets {
    // Byte offsets of the planes inside `data` (Planar only).
    // Q8_0: codes int8 [rows][K], scales half [rows][K/32].
    // Q6_K: ql [rows][K/2], qh [rows][K/4], scales int8 [rows][K/16], d half [rows][K/256].
    uint64_t p0 = 0, p1 = 0, p2 = 0, p3 = 0;
};

}  // namespace syn

struct syn_b200_matrix {
    uint32_t type = 0;
    uint32_t flags = 0;
    uint64_t rows = 0, columns = 0;
    uint64_t row_bytes = 0;  // of the GGUF encoding
    int device = 0;
    syn::Layout layout = syn::Layout::Natural;
    syn::PlaneOffsets planes;
    uint8_t *data = nullptr;  // device
    uint64_t data_bytes = 0;
    // Staging for the host-pointer entry points, grown on demand, owned by the handle.
    void *stage = nullptr;
    uint64_t stage_bytes = 0;
    // Tensor maps of the three big planes of a planar Q6_K matrix (ql, qh, scales), for tiled bulk copies of 16-row
    // boxes; built on first use (syn::q6k_tensor_maps). State: 0 not built yet, 1 ready, -1 cannot be built.
    alignas(64) unsigned char tensor_maps[3][128] = {};
    int tensor_maps_state = 0;
};

namespace syn {

// Quantised activations in device scratch: codes int8 [T][K], scales float [T][K/32], sums int16 [T][K/16].
struct ActLayout {
    uint64_t codes = 0, scales = 0, sums = 0, total = 0;
};
inline ActLayout act_layout(uint64_t tokens, uint64_t columns)
{
    ActLayout l;
    l.codes = 0;
    l.scales = align_up(tokens * columns, 256);
    l.sums = align_up(l.scales + tokens * (columns / 32) * 4, 256);
    l.total = align_up(l.sums + tokens * (columns / 16) * 2, 256);
    return l;
}

struct ActView {
    const int8_t *codes;
    const float *scales;
    const int16_t *sums;
};
inline ActView act_view(const void *scratch, uint64_t tokens, uint64_t columns)
{
    ActLayout l = act_layout(tokens, columns);
    const uint8_t *base = static_cast<const uint8_t *>(scratch);
    return ActView{reinterpret_cast<const int8_t *>(base + l.codes), reinterpret_cast<const float *>(base + l.scales),
                   reinterpret_cast<const int16_t *>(base + l.sums)};
}

struct Error {
    int32_t status;
    std::string message;
};

// Records the message for syn_b200_last_error and returns the status.
int32_t fail(int32_t status, const std::string &message);
int32_t cuda_fail(cudaError_t error, const char *what);
// Row range, token count and output size checks shared by every product (Q8MatrixKernel.cs:21-44); `out_floats`
// (optional) receives the floats the output spans.
int32_t check_product(const syn_b200_matrix *m, uint64_t row_start, uint64_t row_count, uint64_t tokens, uint64_t out_stride,
                      uint64_t *out_floats);
// The matrix must live on the calling thread's current device.
int32_t check_device(const syn_b200_matrix *m);
// Runs `body` and turns any C++ exception into SYN_B200_INTERNAL: nothing is thrown across the ABI (the reference's
// catch_unwind, native/synapse-gpu/src/Features/GpuKernels/ffi.rs:18-44).
template <class Body>
int32_t guarded(Body body)
{
    try {
        return body();
    } catch (const std::bad_alloc &) {
        return fail(SYN_B200_INTERNAL, "host allocation failed");
    } catch (const std::exception &e) {
        return fail(SYN_B200_INTERNAL, e.what());
    } catch (...) {
        return fail(SYN_B200_INTERNAL, "unknown exception at the ABI");
    }
}
void count_launch();
int sm_count(int device);
// The three tensor maps of a planar Q6_K matrix (3 x 128 bytes, 64-byte aligned), or null when they cannot be had.
const unsigned char (*q6k_tensor_maps(const syn_b200_matrix *matrix))[128];

// Launches `kernel` on `stream` with programmatic stream serialization: its prologue and first weight copies overlap
// the tail of the kernel before it. Every kernel launched this way executes griddepcontrol.wait before it reads
// anything an earlier kernel wrote, and before its first global write.
template <class... Params, class... Args>
cudaError_t launch_kernel(void (*kernel)(Params...), dim3 grid, dim3 block, size_t shared_bytes, cudaStream_t stream, Args... args)
{
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = shared_bytes;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    count_launch();
    return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}
// A host-mapped word that kernels bump when a bounded wait gives up (device pointer; null if it cannot be mapped).
uint32_t *fault_word_device();
uint32_t fault_word_read(bool reset);

// quantize.cu
cudaError_t launch_quantize(const float *x, uint64_t tokens, uint64_t columns, uint64_t in_stride, int8_t *codes,
                            float *scales, int16_t *sums, cudaStream_t stream);
cudaError_t launch_group_sums(const int8_t *codes, uint64_t count16, int16_t *sums, cudaStream_t stream);

// repack.cu
uint64_t planar_bytes(uint32_t type, uint64_t rows, uint64_t columns, PlaneOffsets *planes);
cudaError_t launch_repack(uint32_t type, const uint8_t *natural, uint64_t rows, uint64_t columns, uint8_t *planar,
                          const PlaneOffsets &planes, cudaStream_t stream);

// Index of the first block with a non-finite fp16 scale field, or UINT64_MAX (host scan of host blocks; the device
// variant writes the index, or UINT64_MAX, to `first_bad_device`).
uint64_t first_invalid_block_host(uint32_t type, const uint8_t *data, uint64_t blocks);
cudaError_t launch_validate_blocks(uint32_t type, const uint8_t *data, uint64_t blocks, uint64_t *first_bad_device, cudaStream_t stream);

// What happens to a finished dot product before it is stored (the fused regions of the reference's CPU executor,
// Qwen2/Qwen2ProjectionWork.cs:7-131, and `accumulate` of cuda/kernels/common.cuh:52-69):
//   v = dot (+ bias[row]);  v = silu(gate[token][row]) * v when gate is set;  y = accumulate ? y + v : v
struct Epilogue {
    const float *bias = nullptr;  // indexed by row relative to the first row of the call
    const float *gate = nullptr;  // gate projection results, [token][row] with gate_stride, same row origin
    uint64_t gate_stride = 0;
    uint32_t accumulate = 0;
    // Row-sharded products: every result is also stored at the same position of these vectors (the other GPUs' copies
    // of the output, peer-mapped), so the gather of the slices happens inside the product.
    uint32_t peer_count = 0;
    float *peers[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    // Completion signal of a row-sharded product: the last CTA of the launch to finish its stores writes the launch's
    // sequence number into signals[0..signal_count): this rank's word of the product's signal array in its own memory
    // and in every peer's. arrivals[0] counts the CTAs of the running launch, arrivals[1] the launches (both local).
    uint32_t signal_count = 0;
    uint32_t *signals[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    uint32_t *arrivals = nullptr;
};

// One of up to three row ranges that a single launch multiplies with the same activations (MatmulSegment of the
// reference, native/synapse-gpu/src/Features/GpuKernels/params.rs:42-61): results of row r of the range go to
// y[token * out_stride + out_column + r], with bias[r] added when a bias is given.
struct MatvecSegment {
    const syn_b200_matrix *matrix = nullptr;
    uint64_t row_start = 0, row_count = 0;
    const float *bias = nullptr;
    uint64_t out_column = 0;
};

// Waits (bounded) until every word of a signal array has reached the next sequence number; see syn_b200_gather_wait_dev.
cudaError_t launch_gather_wait(const uint32_t *signals, uint32_t count, uint32_t *epoch, uint32_t timeout_us, cudaStream_t stream);

// matvec.cu
struct MatvecArgs {
    // What the launch multiplies: 0 one row range of `matrix`; 1 the row ranges in `segments` (same encoding, layout and
    // width; `matrix` = segments[0].matrix, row_count = all rows together); 2 rows [row_start, +row_count) of
    // segments[0] (gate) and segments[1] (up) with y = silu(gate . x) * (up . x). Forms 1 and 2 are single-token
    // products on ready-made activations; launch_matvec returns cudaErrorNotSupported for shapes they do not take.
    uint32_t form = 0;
    uint32_t segment_count = 0;
    MatvecSegment segments[3];
    const syn_b200_matrix *matrix;
    uint64_t row_start, row_count;
    uint64_t tokens;
    // XF32: FP32 activations x with in_stride. XQ8: either ready-made quantised activations in `act`
    // (act_ready), or FP32 x that the kernel quantises itself; `act` is then scratch for the cases where it cannot.
    ActView act;
    bool act_ready;
    const float *x;
    uint64_t in_stride;
    float *y;
    uint64_t out_stride;
    uint32_t mode;
    uint32_t epilogue;  // SYN_B200_EPILOGUE_*; folded into `fused.accumulate` by launch_matvec
    Epilogue fused;
    int32_t *dump;  // test hook: integer sub-block dots, or null
};
cudaError_t launch_matvec(const MatvecArgs &args, cudaStream_t stream);

// gemm_tc.cu
uint64_t gemm_scratch_bytes(uint64_t tokens, uint64_t columns);
int32_t launch_gemm(const syn_b200_matrix *matrix, const float *x, uint64_t tokens, uint64_t in_stride, float *y,
                    uint64_t out_stride, uint32_t precision, void *scratch, uint64_t scratch_bytes, cudaStream_t stream);

}  // namespace syn
