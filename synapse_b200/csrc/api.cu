// The C ABI of libsynapse_b200.so: argument validation, matrix handles, host staging, error reporting.
// Conventions follow the reference's native libraries (status codes and thread-local last error:
// native/synapse-gpu/src/Features/GpuKernels/ffi.rs:18-44,89-104; validation before any read:
// native/synapse-kernels/src/Features/CpuKernels/q8_0.rs:212-246).
#include <cstdlib>
#include <exception>
#include <cstring>
#include <mutex>
#include <new>
#include <string>

#include <cuda.h>

#include "common.cuh"

namespace syn {

namespace {
thread_local std::string g_last_error;
thread_local uint64_t g_launches = 0;
}  // namespace

int32_t fail(int32_t status, const std::string &message)
{
    static const char *names[] = {"ok", "null pointer", "invalid argument", "unavailable", "device error",
                                  "out of device memory", "internal error"};
    g_last_error = std::string(names[status >= 0 && status <= 6 ? status : 6]) + ": " + message;
    return status;
}

int32_t cuda_fail(cudaError_t error, const char *what)
{
    const int32_t status = error == cudaErrorMemoryAllocation ? SYN_B200_OUT_OF_MEMORY
                           : (error == cudaErrorNoDevice || error == cudaErrorInsufficientDriver ||
                              error == cudaErrorNoKernelImageForDevice)
                               ? SYN_B200_UNAVAILABLE
                               : SYN_B200_DEVICE_ERROR;
    return fail(status, std::string(what) + ": " + cudaGetErrorString(error));
}

void count_launch() { ++g_launches; }

namespace {
uint32_t *g_fault_host = nullptr;
uint32_t *g_fault_device = nullptr;
std::once_flag g_fault_once;
}  // namespace

uint32_t *fault_word_device()
{
    std::call_once(g_fault_once, [] {
        void *host = nullptr;
        if (cudaHostAlloc(&host, 64, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
            cudaGetLastError();
            return;
        }
        *static_cast<volatile uint32_t *>(host) = 0;
        void *device = nullptr;
        if (cudaHostGetDevicePointer(&device, host, 0) != cudaSuccess) {
            cudaGetLastError();
            cudaFreeHost(host);
            return;
        }
        g_fault_host = static_cast<uint32_t *>(host);
        g_fault_device = static_cast<uint32_t *>(device);
    });
    return g_fault_device;
}

uint32_t fault_word_read(bool reset)
{
    if (!g_fault_host) {
        return 0;
    }
    volatile uint32_t *word = g_fault_host;
    const uint32_t value = *word;
    if (reset) {
        *word = 0;
    }
    return value;
}

// Tensor maps for tiled bulk copies (cp.async.bulk.tensor) of 16-row boxes out of the ql, qh and scale planes of a planar
// Q6_K matrix. A plane [rows][row_bytes] is described as bytes [segment][row][128] (strides 128 and row_bytes), so that a
// box of S segments x 16 rows x 128 bytes lands in shared memory segment by segment with the 128-byte swizzle keyed by
// the row: the eight rows a warp reads at one column then sit in different banks. The encoder is a driver entry point
// taken through the runtime (the library does not link libcuda). A last segment may reach past the row's end into the
// next row or, for the last row, into the plane behind it, which is inside the allocation; nothing reads those bytes.
const unsigned char (*q6k_tensor_maps(const syn_b200_matrix *matrix))[128]
{
    static std::mutex guard;
    std::lock_guard<std::mutex> lock(guard);
    syn_b200_matrix *m = const_cast<syn_b200_matrix *>(matrix);
    if (m->tensor_maps_state == 0) {
        m->tensor_maps_state = -1;
        using Encode = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                    const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
        void *entry = nullptr;
        cudaDriverEntryPointQueryResult found = cudaDriverEntryPointSymbolNotFound;
        if (m->type == kQ6_K && m->layout == Layout::Planar && m->rows > 0 &&
            cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &found) == cudaSuccess && entry &&
            found == cudaDriverEntryPointSuccess) {
            const uint64_t row_bytes[3] = {m->columns / 2, m->columns / 4, m->columns / 16};
            const uint64_t offsets[3] = {m->planes.p0, m->planes.p1, m->planes.p2};
            const uint32_t segments[3] = {8, 4, 1};  // of a box: eight super-blocks of a row
            bool ok = true;
            for (int k = 0; k < 3 && ok; ++k) {
                const cuuint64_t dims[3] = {128, m->rows, (row_bytes[k] + 127) / 128};
                const cuuint64_t strides[2] = {row_bytes[k], 128};
                const cuuint32_t box[3] = {128, 16, segments[k]};
                const cuuint32_t steps[3] = {1, 1, 1};
                ok = row_bytes[k] % 16 == 0 &&
                     reinterpret_cast<Encode>(entry)(reinterpret_cast<CUtensorMap *>(m->tensor_maps[k]), CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, m->data + offsets[k],
                                                     dims, strides, box, steps, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                                     CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
            }
            if (ok) {
                m->tensor_maps_state = 1;
            }
        } else {
            cudaGetLastError();
        }
    }
    return m->tensor_maps_state == 1 ? m->tensor_maps : nullptr;
}

int sm_count(int device)
{
    static int cached[64] = {0};
    if (device < 0 || device >= 64) {
        return 148;
    }
    if (cached[device] == 0) {
        int value = 0;
        if (cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || value <= 0) {
            value = 148;
        }
        cached[device] = value;
    }
    return cached[device];
}

// Row range and token checks shared by every product (Q8MatrixKernel.cs:21-44).
int32_t check_product(const syn_b200_matrix *m, uint64_t row_start, uint64_t row_count, uint64_t tokens,
                      uint64_t out_stride, uint64_t *out_floats)
{
    if (row_count == 0 || row_start > m->rows || row_count > m->rows - row_start) {
        return fail(SYN_B200_INVALID_ARGUMENT, "rows [" + std::to_string(row_start) + ", +" + std::to_string(row_count) +
                                                   ") exceed matrix rows " + std::to_string(m->rows));
    }
    if (tokens == 0) {
        return fail(SYN_B200_INVALID_ARGUMENT, "token count is zero");
    }
    if (tokens > 1 && out_stride < row_count) {
        return fail(SYN_B200_INVALID_ARGUMENT, "output stride " + std::to_string(out_stride) + " is below the row count " +
                                                   std::to_string(row_count));
    }
    uint64_t floats = 0;
    if (__builtin_mul_overflow(tokens - 1, out_stride, &floats) || __builtin_add_overflow(floats, row_count, &floats) ||
        floats > (UINT64_MAX >> 3)) {
        return fail(SYN_B200_INVALID_ARGUMENT, "output size overflows");
    }
    if (out_floats) {
        *out_floats = floats;
    }
    return SYN_B200_OK;
}

int32_t check_device(const syn_b200_matrix *m)
{
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device != m->device) {
        cudaGetLastError();
        return fail(SYN_B200_INVALID_ARGUMENT, "the matrix lives on device " + std::to_string(m->device) +
                                                   ", which is not the calling thread's current device");
    }
    return SYN_B200_OK;
}

namespace {

// The library only carries sm_100a code: any other device cannot run it.
int32_t require_device(int *device_out)
{
    int device = 0;
    cudaError_t error = cudaGetDevice(&device);
    if (error != cudaSuccess) {
        cudaGetLastError();
        return fail(SYN_B200_UNAVAILABLE, std::string("no usable CUDA device: ") + cudaGetErrorString(error));
    }
    static int checked[64] = {0};  // 0 unknown, 1 ok, -1 wrong architecture
    if (device >= 0 && device < 64 && checked[device] == 0) {
        int major = 0;
        error = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
        if (error != cudaSuccess) {
            cudaGetLastError();
            return fail(SYN_B200_UNAVAILABLE, std::string("cannot query the CUDA device: ") + cudaGetErrorString(error));
        }
        checked[device] = major == 10 ? 1 : -1;
    }
    if (device >= 0 && device < 64 && checked[device] < 0) {
        return fail(SYN_B200_UNAVAILABLE, "the device is not compute capability 10.x (B200, sm_100a)");
    }
    if (device_out) {
        *device_out = device;
    }
    return SYN_B200_OK;
}

bool mul_ok(uint64_t a, uint64_t b, uint64_t *out) { return !__builtin_mul_overflow(a, b, out); }

int32_t ensure_stage(syn_b200_matrix *m, uint64_t bytes)
{
    if (m->stage_bytes >= bytes) {
        return SYN_B200_OK;
    }
    if (m->stage) {
        cudaFree(m->stage);
        m->stage = nullptr;
        m->stage_bytes = 0;
    }
    const uint64_t want = align_up(bytes, 1 << 20);
    cudaError_t error = cudaMalloc(&m->stage, want);
    if (error != cudaSuccess) {
        cudaGetLastError();
        return cuda_fail(error, "allocating the staging buffer");
    }
    m->stage_bytes = want;
    return SYN_B200_OK;
}

int32_t create_matrix(const void *blocks_pointer, bool from_device, uint32_t type, uint64_t rows, uint64_t columns, uint32_t flags,
                      cudaStream_t stream, syn_b200_matrix **out)
{
    if (!blocks_pointer || !out) {
        return fail(SYN_B200_NULL_POINTER, "blocks or output handle");
    }
    *out = nullptr;
    const uint64_t values = block_values(type);
    if (values == 0) {
        return fail(SYN_B200_INVALID_ARGUMENT, "unsupported GGML tensor type " + std::to_string(type));
    }
    if (flags & ~SYN_B200_REPACK) {
        return fail(SYN_B200_INVALID_ARGUMENT, "unknown flag bits " + std::to_string(flags));
    }
    if (rows == 0 || columns == 0) {
        return fail(SYN_B200_INVALID_ARGUMENT, "a matrix needs at least one row and one column");
    }
    if (columns % values != 0) {
        return fail(SYN_B200_UNAVAILABLE, "the matrix has " + std::to_string(columns) + " columns, not a multiple of its " +
                                              std::to_string(values) + "-value blocks");
    }
    uint64_t row_bytes = 0, total = 0;
    if (!mul_ok(columns / values, block_bytes(type), &row_bytes) || !mul_ok(rows, row_bytes, &total) ||
        rows > (1ull << 31) || columns > (1ull << 31)) {
        return fail(SYN_B200_INVALID_ARGUMENT, "matrix size overflows");
    }
    const uint64_t blocks = rows * (columns / values);
    const std::string type_name = type == kQ8_0 ? "q8_0" : type == kQ4_K ? "q4_k" : "q6_k";
    if (!from_device) {
        // The reference refuses a tensor whose blocks hold a non-finite fp16 scale before it decodes anything
        // (BlockSourceDecoder.Decode, ModelPackages/SourceFormats/SourceTensorDecoders.cs:134-146,161-172).
        const uint64_t bad = first_invalid_block_host(type, static_cast<const uint8_t *>(blocks_pointer), blocks);
        if (bad != UINT64_MAX) {
            return fail(SYN_B200_INVALID_ARGUMENT, type_name + " block " + std::to_string(bad) + " fails validation: InvalidScale");
        }
    }
    int device = 0;
    int32_t status = require_device(&device);
    if (status != SYN_B200_OK) {
        return status;
    }
    fault_word_device();  // mapped once here, never during a stream capture
    syn_b200_matrix *m = new syn_b200_matrix();
    m->type = type;
    m->flags = flags;
    m->rows = rows;
    m->columns = columns;
    m->row_bytes = row_bytes;
    m->device = device;
    const bool repack = (flags & SYN_B200_REPACK) && type != kQ4_K;  // Q4_K blocks are 16-byte aligned as they are
    uint8_t *natural = nullptr;
    // 64 spare bytes so that 16-byte reads of the last, clamped unit never leave the allocation.
    cudaError_t error = cudaMalloc(&natural, align_up(total, 256) + 64);
    if (error != cudaSuccess) {
        cudaGetLastError();
        delete m;
        return cuda_fail(error, "allocating the weight buffer");
    }
    error = cudaMemcpyAsync(natural, blocks_pointer, total, from_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, stream);
    uint64_t *first_bad = nullptr;
    if (error == cudaSuccess && from_device) {
        // blocks that never were in host memory are validated on the device, before the repack reads them
        error = cudaMalloc(&first_bad, sizeof(uint64_t));
        if (error == cudaSuccess) {
            error = launch_validate_blocks(type, natural, blocks, first_bad, stream);
        }
    }
    if (error == cudaSuccess && repack) {
        m->data_bytes = planar_bytes(type, rows, columns, &m->planes);
        error = cudaMalloc(&m->data, m->data_bytes + 64);
        if (error == cudaSuccess) {
            m->layout = Layout::Planar;
            error = launch_repack(type, natural, rows, columns, m->data, m->planes, stream);
        }
    } else if (error == cudaSuccess) {
        m->data = natural;
        m->data_bytes = total;
        natural = nullptr;
    }
    if (error == cudaSuccess) {
        error = cudaStreamSynchronize(stream);
    }
    uint64_t bad = UINT64_MAX;
    if (error == cudaSuccess && first_bad) {
        error = cudaMemcpy(&bad, first_bad, sizeof(bad), cudaMemcpyDeviceToHost);
    }
    if (first_bad) {
        cudaFree(first_bad);
    }
    if (natural) {
        cudaFree(natural);
    }
    if (error != cudaSuccess || bad != UINT64_MAX) {
        cudaGetLastError();
        if (m->data) {
            cudaFree(m->data);
        }
        delete m;
        return error != cudaSuccess ? cuda_fail(error, "uploading the weights")
                                    : fail(SYN_B200_INVALID_ARGUMENT, type_name + " block " + std::to_string(bad) + " fails validation: InvalidScale");
    }
    *out = m;
    return SYN_B200_OK;
}

// Queues quantise (or upload of ready codes) + product on `stream` with device x / y.
// Prompt runs longer than this leave the matrix-vector kernels for the tensor cores (GEMM_MINIMUM_TOKENS,
// native/synapse-gpu/src/Features/GpuKernels/step/projection.rs:14).
constexpr uint64_t kGemmMinimumTokens = 4;

int32_t convert_epilogue(const syn_b200_epilogue *in, Epilogue &out)
{
    out = Epilogue{};
    if (!in) {
        return SYN_B200_OK;
    }
    if (in->reserved != 0 || in->accumulate > 1) {
        return fail(SYN_B200_INVALID_ARGUMENT, "epilogue flags must be 0 or 1 and the reserved field 0");
    }
    out.bias = in->bias;
    out.gate = in->gate;
    out.gate_stride = in->gate_stride;
    out.accumulate = in->accumulate;
    return SYN_B200_OK;
}

// Peer copies of the output and the completion signal of a row-sharded product; null = a product on one GPU.
int32_t convert_gather(const syn_b200_gather *in, Epilogue &out)
{
    out.peer_count = 0;
    out.signal_count = 0;
    out.arrivals = nullptr;
    if (!in) {
        return SYN_B200_OK;
    }
    if (in->peer_count > 7 || in->reserved != 0) {
        return fail(SYN_B200_INVALID_ARGUMENT, "at most 7 peer outputs (got " + std::to_string(in->peer_count) + ") and the reserved field 0");
    }
    if (in->peer_count > 0 && !in->peer_outputs) {
        return fail(SYN_B200_NULL_POINTER, "peer outputs");
    }
    for (uint32_t i = 0; i < in->peer_count; ++i) {
        if (!in->peer_outputs[i]) {
            return fail(SYN_B200_NULL_POINTER, "peer output " + std::to_string(i));
        }
        out.peers[i] = in->peer_outputs[i];
    }
    out.peer_count = in->peer_count;
    if (in->signals) {
        if (!in->arrivals) {
            return fail(SYN_B200_NULL_POINTER, "a completion signal needs the two local arrival words");
        }
        for (uint32_t i = 0; i <= in->peer_count; ++i) {
            if (!in->signals[i] || (reinterpret_cast<uintptr_t>(in->signals[i]) & 3)) {
                return fail(SYN_B200_NULL_POINTER, "signal word " + std::to_string(i));
            }
            out.signals[i] = in->signals[i];
        }
        out.signal_count = in->peer_count + 1;
        out.arrivals = in->arrivals;
    }
    return SYN_B200_OK;
}

int32_t product_dev(const syn_b200_matrix *m, uint64_t row_start, uint64_t row_count, const float *x, uint64_t tokens,
                    uint64_t in_stride, float *y, uint64_t out_stride, uint32_t mode, uint32_t epilogue, void *scratch,
                    uint64_t scratch_bytes, cudaStream_t stream, const Epilogue &fused = Epilogue{})
{
    if (mode != SYN_B200_MODE_XQ8 && mode != SYN_B200_MODE_XF32) {
        return fail(SYN_B200_INVALID_ARGUMENT, "unknown activation mode " + std::to_string(mode));
    }
    if (epilogue > SYN_B200_EPILOGUE_ACCUMULATE) {
        return fail(SYN_B200_INVALID_ARGUMENT, "unknown epilogue " + std::to_string(epilogue));
    }
    if (in_stride < m->columns) {
        return fail(SYN_B200_INVALID_ARGUMENT, "input stride " + std::to_string(in_stride) + " is below the matrix width " +
                                                   std::to_string(m->columns));
    }
    if (in_stride % 4 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0) {
        return fail(SYN_B200_INVALID_ARGUMENT, "device activations must be 16-byte aligned with a stride that is a multiple of 4 floats");
    }
    const bool plain = epilogue == SYN_B200_EPILOGUE_STORE && !fused.bias && !fused.gate && !fused.accumulate;
    if (mode == SYN_B200_MODE_XF32 && tokens > kGemmMinimumTokens && plain && row_start == 0 && row_count == m->rows &&
        m->columns % 64 == 0 && scratch && scratch_bytes >= gemm_scratch_bytes(tokens, m->columns) &&
        (reinterpret_cast<uintptr_t>(scratch) & 255) == 0) {
        return launch_gemm(m, x, tokens, in_stride, y, out_stride, SYN_B200_GEMM_F16, scratch, scratch_bytes, stream);
    }
    MatvecArgs args{};
    args.matrix = m;
    args.row_start = row_start;
    args.row_count = row_count;
    args.tokens = tokens;
    args.y = y;
    args.out_stride = out_stride;
    args.mode = mode;
    args.epilogue = epilogue;
    args.fused = fused;
    if (mode == SYN_B200_MODE_XQ8) {
        const ActLayout layout = act_layout(tokens, m->columns);
        if (!scratch || scratch_bytes < layout.total) {
            return fail(SYN_B200_INVALID_ARGUMENT, "activation scratch is missing or smaller than " + std::to_string(layout.total) + " bytes");
        }
        if (reinterpret_cast<uintptr_t>(scratch) & 255) {
            return fail(SYN_B200_INVALID_ARGUMENT, "activation scratch must be 256-byte aligned");
        }
        // The kernel quantises x itself where it can; the scratch serves the shapes where it cannot.
        args.act = act_view(scratch, tokens, m->columns);
        args.act_ready = false;
        args.x = x;
        args.in_stride = in_stride;
    } else {
        args.x = x;
        args.in_stride = in_stride;
    }
    cudaError_t error = launch_matvec(args, stream);
    if (error != cudaSuccess) {
        return cuda_fail(error, "launching the matrix-vector kernel");
    }
    return SYN_B200_OK;
}

}  // namespace

}  // namespace syn

using namespace syn;

extern "C" {

uint32_t syn_b200_abi_version(void) { return SYN_B200_ABI_VERSION; }

size_t syn_b200_last_error(uint8_t *buffer, size_t capacity)
{
    const std::string &message = g_last_error;
    if (buffer) {
        const size_t length = message.size() < capacity ? message.size() : capacity;
        for (size_t i = 0; i < length; ++i) {
            buffer[i] = (uint8_t)message[i];
        }
    }
    return message.size();
}

uint32_t syn_b200_device_faults(uint32_t reset) { return fault_word_read(reset != 0); }

uint64_t syn_b200_launch_count(uint32_t reset)
{
    const uint64_t value = g_launches;
    if (reset) {
        g_launches = 0;
    }
    return value;
}

int32_t syn_b200_probe(syn_b200_device_info *out)
{
    if (!out) {
        return fail(SYN_B200_NULL_POINTER, "device info");
    }
    return guarded([&]() -> int32_t {
        int device = 0;
        int32_t status = require_device(&device);
        if (status != SYN_B200_OK) {
            return status;
        }
        cudaDeviceProp prop;
        cudaError_t error = cudaGetDeviceProperties(&prop, device);
        if (error != cudaSuccess) {
            cudaGetLastError();
            return cuda_fail(error, "reading device properties");
        }
        syn_b200_device_info info{};
        std::string name = std::string(prop.name) + " (sm_" + std::to_string(prop.major) + std::to_string(prop.minor) + ")";
        name.copy(info.name, sizeof(info.name) - 1);
        info.total_memory_bytes = prop.totalGlobalMem;
        info.max_buffer_bytes = prop.totalGlobalMem;
        info.compute_capability = (uint32_t)(prop.major * 10 + prop.minor);
        info.multiprocessors = (uint32_t)prop.multiProcessorCount;
        *out = info;
        return SYN_B200_OK;
    });
}

int32_t syn_b200_matrix_create(const void *host_blocks, uint32_t ggml_type, uint64_t rows, uint64_t columns, uint32_t flags,
                               syn_b200_matrix **out)
{
    return guarded([&]() { return create_matrix(host_blocks, false, ggml_type, rows, columns, flags, nullptr, out); });
}

int32_t syn_b200_matrix_create_from_device(const void *device_blocks, uint32_t ggml_type, uint64_t rows, uint64_t columns,
                                           uint32_t flags, void *stream, syn_b200_matrix **out)
{
    return guarded([&]() {
        return create_matrix(device_blocks, true, ggml_type, rows, columns, flags, static_cast<cudaStream_t>(stream), out);
    });
}

void syn_b200_matrix_destroy(syn_b200_matrix *matrix)
{
    if (!matrix) {
        return;
    }
    if (matrix->data) {
        cudaFree(matrix->data);
    }
    if (matrix->stage) {
        cudaFree(matrix->stage);
    }
    delete matrix;
}

int32_t syn_b200_matrix_info(const syn_b200_matrix *matrix, uint32_t *ggml_type, uint64_t *rows, uint64_t *columns,
                             uint32_t *flags, uint64_t *source_bytes)
{
    if (!matrix) {
        return fail(SYN_B200_NULL_POINTER, "matrix");
    }
    if (ggml_type) *ggml_type = matrix->type;
    if (rows) *rows = matrix->rows;
    if (columns) *columns = matrix->columns;
    if (flags) *flags = matrix->flags;
    if (source_bytes) *source_bytes = matrix->rows * matrix->row_bytes;
    return SYN_B200_OK;
}

uint64_t syn_b200_activation_scratch_bytes(uint64_t tokens, uint64_t columns) { return act_layout(tokens, columns).total; }

int32_t syn_b200_quantize_q8_dev(const float *x, uint64_t tokens, uint64_t columns, uint64_t in_stride, void *scratch,
                                 uint64_t scratch_bytes, void *stream)
{
    if (!x || !scratch) {
        return fail(SYN_B200_NULL_POINTER, "activations or scratch");
    }
    return guarded([&]() -> int32_t {
        if (tokens == 0 || columns == 0 || columns % 32 != 0 || in_stride < columns) {
            return fail(SYN_B200_INVALID_ARGUMENT, "Q8_0 activation rows need a positive multiple of 32 values and a stride that covers them");
        }
        int32_t status = require_device(nullptr);
        if (status != SYN_B200_OK) {
            return status;
        }
        const ActLayout layout = act_layout(tokens, columns);
        if (scratch_bytes < layout.total || (reinterpret_cast<uintptr_t>(scratch) & 255)) {
            return fail(SYN_B200_INVALID_ARGUMENT, "activation scratch must be 256-byte aligned and hold " + std::to_string(layout.total) + " bytes");
        }
        uint8_t *base = static_cast<uint8_t *>(scratch);
        cudaError_t error = launch_quantize(x, tokens, columns, in_stride, reinterpret_cast<int8_t *>(base + layout.codes),
                                            reinterpret_cast<float *>(base + layout.scales),
                                            reinterpret_cast<int16_t *>(base + layout.sums), static_cast<cudaStream_t>(stream));
        return error == cudaSuccess ? SYN_B200_OK : cuda_fail(error, "launching the activation quantiser");
    });
}

int32_t syn_b200_quantize_q8(const float *x, uint64_t tokens, uint64_t columns, uint64_t in_stride, int8_t *codes, float *scales)
{
    if (!x || !codes || !scales) {
        return fail(SYN_B200_NULL_POINTER, "activations, codes or scales");
    }
    return guarded([&]() -> int32_t {
        if (tokens == 0 || columns == 0 || columns % 32 != 0 || in_stride < columns) {
            return fail(SYN_B200_INVALID_ARGUMENT, "Q8_0 activation rows need a positive multiple of 32 values and a stride that covers them");
        }
        uint64_t count = 0;
        if (!mul_ok(tokens, columns, &count) || count > (1ull << 40)) {
            return fail(SYN_B200_INVALID_ARGUMENT, "activation size overflows");
        }
        int32_t status = require_device(nullptr);
        if (status != SYN_B200_OK) {
            return status;
        }
        const ActLayout layout = act_layout(tokens, columns);
        const uint64_t x_bytes = align_up(count * 4, 256);
        uint8_t *device = nullptr;
        cudaError_t error = cudaMalloc(&device, x_bytes + layout.total);
        if (error != cudaSuccess) {
            cudaGetLastError();
            return cuda_fail(error, "allocating quantiser buffers");
        }
        float *dx = reinterpret_cast<float *>(device);
        uint8_t *base = device + x_bytes;
        error = cudaMemcpy2D(dx, columns * 4, x, in_stride * 4, columns * 4, tokens, cudaMemcpyHostToDevice);
        if (error == cudaSuccess) {
            error = launch_quantize(dx, tokens, columns, columns, reinterpret_cast<int8_t *>(base + layout.codes),
                                    reinterpret_cast<float *>(base + layout.scales), reinterpret_cast<int16_t *>(base + layout.sums), nullptr);
        }
        if (error == cudaSuccess) {
            error = cudaMemcpy(codes, base + layout.codes, count, cudaMemcpyDeviceToHost);
        }
        if (error == cudaSuccess) {
            error = cudaMemcpy(scales, base + layout.scales, count / 32 * 4, cudaMemcpyDeviceToHost);
        }
        cudaFree(device);
        if (error != cudaSuccess) {
            cudaGetLastError();
            return cuda_fail(error, "running the activation quantiser");
        }
        return SYN_B200_OK;
    });
}

int32_t syn_b200_matmul_q8_dev(const syn_b200_matrix *matrix, uint64_t row_start, uint64_t row_count, const void *scratch,
                               uint64_t tokens, float *y, uint64_t out_stride, uint32_t epilogue, void *stream)
{
    if (!matrix || !scratch || !y) {
        return fail(SYN_B200_NULL_POINTER, "matrix, scratch or output");
    }
    return guarded([&]() -> int32_t {
        int32_t status = check_product(matrix, row_start, row_count, tokens, out_stride, nullptr);
        if (status == SYN_B200_OK) status = check_device(matrix);
        if (status != SYN_B200_OK) {
            return status;
        }
        if (epilogue > SYN_B200_EPILOGUE_ACCUMULATE) {
            return fail(SYN_B200_INVALID_ARGUMENT, "unknown epilogue " + std::to_string(epilogue));
        }
        if (reinterpret_cast<uintptr_t>(scratch) & 255) {
            return fail(SYN_B200_INVALID_ARGUMENT, "activation scratch must be 256-byte aligned");
        }
        MatvecArgs args{};
        args.matrix = matrix;
        args.row_start = row_start;
        args.row_count = row_count;
        args.tokens = tokens;
        args.act = act_view(scratch, tokens, matrix->columns);
        args.act_ready = true;
        args.y = y;
        args.out_stride = out_stride;
        args.mode = SYN_B200_MODE_XQ8;
        args.epilogue = epilogue;
        cudaError_t error = launch_matvec(args, static_cast<cudaStream_t>(stream));
        return error == cudaSuccess ? SYN_B200_OK : cuda_fail(error, "launching the matrix-vector kernel");
    });
}

int32_t syn_b200_matvec_dev(const syn_b200_matrix *matrix, uint64_t row_start, uint64_t row_count, const float *x,
                            uint64_t tokens, uint64_t in_stride, float *y, uint64_t out_stride, uint32_t mode,
                            uint32_t epilogue, void *scratch, uint64_t scratch_bytes, void *stream)
{
    if (!matrix || !x || !y) {
        return fail(SYN_B200_NULL_POINTER, "matrix, activations or output");
    }
    return guarded([&]() -> int32_t {
        int32_t status = check_product(matrix, row_start, row_count, tokens, out_stride, nullptr);
        if (status == SYN_B200_OK) status = check_device(matrix);
        if (status != SYN_B200_OK) {
            return status;
        }
        return product_dev(matrix, row_start, row_count, x, tokens, in_stride, y, out_stride, mode, epilogue, scratch,
                           scratch_bytes, static_cast<cudaStream_t>(stream));
    });
}

int32_t syn_b200_matvec_ex_dev(const syn_b200_matrix *matrix, uint64_t row_start, uint64_t row_count, const float *x,
                               uint64_t tokens, uint64_t in_stride, float *y, uint64_t out_stride, uint32_t mode,
                               const syn_b200_epilogue *epilogue, void *scratch, uint64_t scratch_bytes, void *stream)
{
    if (!matrix || !x || !y) {
        return fail(SYN_B200_NULL_POINTER, "matrix, activations or output");
    }
    return guarded([&]() -> int32_t {
        int32_t status = check_product(matrix, row_start, row_count, tokens, out_stride, nullptr);
        if (status == SYN_B200_OK) status = check_device(matrix);
        Epilogue fused;
        if (status == SYN_B200_OK) status = convert_epilogue(epilogue, fused);
        if (status != SYN_B200_OK) {
            return status;
        }
        return product_dev(matrix, row_start, row_count, x, tokens, in_stride, y, out_stride, mode, SYN_B200_EPILOGUE_STORE, scratch,
                           scratch_bytes, static_cast<cudaStream_t>(stream), fused);
    });
}

int32_t syn_b200_matmul_q8_ex_dev(const syn_b200_matrix *matrix, uint64_t row_start, uint64_t row_count, const void *scratch,
                                  uint64_t tokens, float *y, uint64_t out_stride, const syn_b200_epilogue *epilogue, void *stream)
{
    if (!matrix || !scratch || !y) {
        return fail(SYN_B200_NULL_POINTER, "matrix, scratch or output");
    }
    return guarded([&]() -> int32_t {
        int32_t status = check_product(matrix, row_start, row_count, tokens, out_stride, nullptr);
        if (status == SYN_B200_OK) status = check_device(matrix);
        Epilogue fused;
        if (status == SYN_B200_OK) status = convert_epilogue(epilogue, fused);
        if (status != SYN_B200_OK) {
            return status;
        }
        if (reinterpret_cast<uintptr_t>(scratch) & 255) {
            return fail(SYN_B200_INVALID_ARGUMENT, "activation scratch must be 256-byte aligned");
        }
        MatvecArgs args{};
        args.matrix = matrix;
        args.row_start = row_start;
        args.row_count = row_count;
        args.tokens = tokens;
        args.act = act_view(scratch, tokens, matrix->columns);
        args.act_ready = true;
        args.y = y;
        args.out_stride = out_stride;
        args.mode = SYN_B200_MODE_XQ8;
        args.epilogue = SYN_B200_EPILOGUE_STORE;
        args.fused = fused;
        cudaError_t error = launch_matvec(args, static_cast<cudaStream_t>(stream));
        return error == cudaSuccess ? SYN_B200_OK : cuda_fail(error, "launching the matrix-vector kernel");
    });
}

int32_t syn_b200_shared_buffer_create(uint64_t bytes, void **device_ptr, uint8_t handle[64])
{
    if (!device_ptr || !handle) {
        return fail(SYN_B200_NULL_POINTER, "buffer or handle output");
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is passed as 64 bytes");
    return guarded([&]() -> int32_t {
        if (bytes == 0) {
            return fail(SYN_B200_INVALID_ARGUMENT, "a shared buffer needs at least one byte");
        }
        void *p = nullptr;
        cudaError_t error = cudaMalloc(&p, bytes);
        if (error != cudaSuccess) {
            cudaGetLastError();
            return error == cudaErrorMemoryAllocation ? fail(SYN_B200_OUT_OF_MEMORY, "allocating the shared buffer")
                                                      : cuda_fail(error, "allocating the shared buffer");
        }
        error = cudaMemset(p, 0, bytes);
        cudaIpcMemHandle_t ipc;
        if (error == cudaSuccess) {
            error = cudaIpcGetMemHandle(&ipc, p);
        }
        if (error != cudaSuccess) {
            cudaGetLastError();
            cudaFree(p);
            return cuda_fail(error, "exporting the shared buffer");
        }
        memcpy(handle, &ipc, sizeof(ipc));
        *device_ptr = p;
        return SYN_B200_OK;
    });
}

int32_t syn_b200_shared_buffer_open(const uint8_t handle[64], void **device_ptr)
{
    if (!device_ptr || !handle) {
        return fail(SYN_B200_NULL_POINTER, "handle or buffer output");
    }
    return guarded([&]() -> int32_t {
        cudaIpcMemHandle_t ipc;
        memcpy(&ipc, handle, sizeof(ipc));
        void *p = nullptr;
        // with the CALLER's device current: the mapping is made for this device's kernels, peer access included
        cudaError_t error = cudaIpcOpenMemHandle(&p, ipc, cudaIpcMemLazyEnablePeerAccess);
        if (error != cudaSuccess) {
            cudaGetLastError();
            return fail(SYN_B200_UNAVAILABLE, std::string("the shared buffer cannot be mapped: ") + cudaGetErrorString(error));
        }
        // prove the mapping before any kernel stores through it
        cudaPointerAttributes attributes{};
        uint32_t probe = 0;
        error = cudaPointerGetAttributes(&attributes, p);
        if (error == cudaSuccess && attributes.type != cudaMemoryTypeDevice) {
            error = cudaErrorInvalidDevicePointer;
        }
        if (error == cudaSuccess) {
            error = cudaMemcpy(&probe, p, sizeof(probe), cudaMemcpyDeviceToHost);
        }
        if (error != cudaSuccess) {
            cudaGetLastError();
            cudaIpcCloseMemHandle(p);
            return fail(SYN_B200_UNAVAILABLE, std::string("the mapped shared buffer is not usable from this device: ") + cudaGetErrorString(error));
        }
        *device_ptr = p;
        return SYN_B200_OK;
    });
}

void syn_b200_shared_buffer_close(void *device_ptr)
{
    if (device_ptr) {
        cudaIpcCloseMemHandle(device_ptr);
    }
}

void syn_b200_shared_buffer_destroy(void *device_ptr)
{
    if (device_ptr) {
        cudaFree(device_ptr);
    }
}

int32_t syn_b200_enable_peer_access(int32_t peer_device)
{
    return guarded([&]() -> int32_t {
        int device = 0, count = 0;
        if (cudaGetDevice(&device) != cudaSuccess || cudaGetDeviceCount(&count) != cudaSuccess) {
            cudaGetLastError();
            return fail(SYN_B200_UNAVAILABLE, "no usable CUDA device");
        }
        if (peer_device < 0 || peer_device >= count) {
            return fail(SYN_B200_INVALID_ARGUMENT, "device " + std::to_string(peer_device) + " does not exist");
        }
        if (peer_device == device) {
            return SYN_B200_OK;
        }
        int can = 0;
        cudaError_t error = cudaDeviceCanAccessPeer(&can, device, peer_device);
        if (error != cudaSuccess || !can) {
            cudaGetLastError();
            return fail(SYN_B200_UNAVAILABLE, "device " + std::to_string(device) + " has no peer path to device " + std::to_string(peer_device));
        }
        error = cudaDeviceEnablePeerAccess(peer_device, 0);
        if (error == cudaErrorPeerAccessAlreadyEnabled) {
            cudaGetLastError();
            return SYN_B200_OK;
        }
        return error == cudaSuccess ? SYN_B200_OK : cuda_fail(error, "enabling peer access");
    });
}

int32_t syn_b200_matmul_q8_gather_dev(const syn_b200_matrix *matrix, uint64_t row_start, uint64_t row_count, const void *scratch,
                                      uint64_t tokens, float *y, uint64_t out_stride, const syn_b200_gather *gather, void *stream)
{
    if (!matrix || !scratch || !y) {
        return fail(SYN_B200_NULL_POINTER, "matrix, scratch or output");
    }
    return guarded([&]() -> int32_t {
        int32_t status = check_product(matrix, row_start, row_count, tokens, out_stride, nullptr);
        if (status == SYN_B200_OK) status = check_device(matrix);
        Epilogue fused;
        if (status == SYN_B200_OK) status = convert_gather(gather, fused);
        if (status != SYN_B200_OK) {
            return status;
        }
        if (reinterpret_cast<uintptr_t>(scratch) & 255) {
            return fail(SYN_B200_INVALID_ARGUMENT, "activation scratch must be 256-byte aligned");
        }
        MatvecArgs args{};
        args.matrix = matrix;
        args.row_start = row_start;
        args.row_count = row_count;
        args.tokens = tokens;
        args.act = act_view(scratch, tokens, matrix->columns);
        args.act_ready = true;
        args.y = y;
        args.out_stride = out_stride;
        args.mode = SYN_B200_MODE_XQ8;
        args.epilogue = SYN_B200_EPILOGUE_STORE;
        args.fused = fused;
        cudaError_t error = launch_matvec(args, static_cast<cudaStream_t>(stream));
        return error == cudaSuccess ? SYN_B200_OK : cuda_fail(error, "launching the matrix-vector kernel");
    });
}

int32_t syn_b200_gather_wait_dev(const uint32_t *signals, uint32_t count, uint32_t *epoch, uint32_t timeout_us, void *stream)
{
    if (!signals || !epoch) {
        return fail(SYN_B200_NULL_POINTER, "signal array or epoch word");
    }
    return guarded([&]() -> int32_t {
        if (count == 0 || count > 8 || timeout_us == 0) {
            return fail(SYN_B200_INVALID_ARGUMENT, "a signal array holds 1 to 8 words and the wait needs a positive limit");
        }
        int32_t status = require_device(nullptr);
        if (status != SYN_B200_OK) {
            return status;
        }
        cudaError_t error = launch_gather_wait(signals, count, epoch, timeout_us, static_cast<cudaStream_t>(stream));
        return error == cudaSuccess ? SYN_B200_OK : cuda_fail(error, "launching the completion wait");
    });
}

int32_t syn_b200_matmul_q8_segments_dev(const syn_b200_segment *segments, uint32_t count, const void *scratch, uint64_t tokens, float *y,
                                        uint64_t out_stride, uint32_t accumulate, const syn_b200_gather *gather, void *stream)
{
    if (!segments || !scratch || !y) {
        return fail(SYN_B200_NULL_POINTER, "segments, scratch or output");
    }
    return guarded([&]() -> int32_t {
        if (count == 0 || count > 3) {
            return fail(SYN_B200_INVALID_ARGUMENT, "a product takes 1 to 3 segments, got " + std::to_string(count));
        }
        if (accumulate > 1) {
            return fail(SYN_B200_INVALID_ARGUMENT, "accumulate must be 0 or 1");
        }
        if (reinterpret_cast<uintptr_t>(scratch) & 255) {
            return fail(SYN_B200_INVALID_ARGUMENT, "activation scratch must be 256-byte aligned");
        }
        MatvecArgs args{};
        uint64_t total_rows = 0;
        for (uint32_t i = 0; i < count; ++i) {
            const syn_b200_segment &segment = segments[i];
            if (!segment.matrix) {
                return fail(SYN_B200_NULL_POINTER, "matrix of segment " + std::to_string(i));
            }
            const syn_b200_matrix *first = segments[0].matrix;
            if (segment.matrix->type != first->type || segment.matrix->layout != first->layout || segment.matrix->columns != first->columns) {
                // the reference shares a dispatch only between projections of one encoding (step/layers.rs:71-94)
                return fail(SYN_B200_INVALID_ARGUMENT, "the segments of one product must share encoding, layout and width");
            }
            uint64_t end = 0;
            if (__builtin_add_overflow(segment.out_column, segment.row_count, &end) || (tokens > 1 && end > out_stride)) {
                return fail(SYN_B200_INVALID_ARGUMENT, "segment " + std::to_string(i) + " does not fit the output stride");
            }
            int32_t status = check_product(segment.matrix, segment.row_start, segment.row_count, tokens, out_stride, nullptr);
            if (status == SYN_B200_OK) status = check_device(segment.matrix);
            if (status != SYN_B200_OK) {
                return status;
            }
            args.segments[i].matrix = segment.matrix;
            args.segments[i].row_start = segment.row_start;
            args.segments[i].row_count = segment.row_count;
            args.segments[i].bias = segment.bias;
            args.segments[i].out_column = segment.out_column;
            total_rows += segment.row_count;
        }
        Epilogue fused;
        if (int32_t status = convert_gather(gather, fused)) {
            return status;
        }
        fused.accumulate = accumulate;
        const uint32_t peer_count = fused.peer_count;
        const syn_b200_matrix *m = segments[0].matrix;
        args.form = 1;
        args.segment_count = count;
        args.matrix = m;
        args.row_start = segments[0].row_start;
        args.row_count = total_rows;
        args.tokens = tokens;
        args.act = act_view(scratch, tokens, m->columns);
        args.act_ready = true;
        args.y = y;
        args.out_stride = out_stride;
        args.mode = SYN_B200_MODE_XQ8;
        args.epilogue = SYN_B200_EPILOGUE_STORE;
        args.fused = fused;
        cudaError_t error = count > 1 ? launch_matvec(args, static_cast<cudaStream_t>(stream)) : cudaErrorNotSupported;
        if (error == cudaErrorNotSupported) {
            // shapes the one-launch form does not take (several tokens, rows longer than one pass of a team): one
            // launch per segment, same results
            error = cudaSuccess;
            for (uint32_t i = 0; i < count && error == cudaSuccess; ++i) {
                MatvecArgs one = args;
                one.form = 0;
                one.matrix = args.segments[i].matrix;
                one.row_start = args.segments[i].row_start;
                one.row_count = args.segments[i].row_count;
                one.y = y + args.segments[i].out_column;
                one.fused.bias = args.segments[i].bias;
                for (uint32_t k = 0; k < peer_count; ++k) {
                    one.fused.peers[k] = fused.peers[k] + args.segments[i].out_column;
                }
                if (i + 1 < count) {
                    one.fused.signal_count = 0;  // the launches are stream-ordered: the last one signals for all of them
                }
                error = launch_matvec(one, static_cast<cudaStream_t>(stream));
            }
        }
        return error == cudaSuccess ? SYN_B200_OK : cuda_fail(error, "launching the matrix-vector kernel");
    });
}

int32_t syn_b200_matmul_q8_swiglu_dev(const syn_b200_matrix *gate, const syn_b200_matrix *up, uint64_t row_start, uint64_t row_count,
                                      const void *scratch, uint64_t tokens, float *y, uint64_t out_stride, float *gate_values,
                                      const syn_b200_gather *gather, void *stream)
{
    if (!gate || !up || !scratch || !y) {
        return fail(SYN_B200_NULL_POINTER, "gate, up, scratch or output");
    }
    return guarded([&]() -> int32_t {
        if (gate->type != up->type || gate->layout != up->layout || gate->columns != up->columns || gate->rows != up->rows) {
            return fail(SYN_B200_INVALID_ARGUMENT, "the gate and up matrices must share encoding, layout and shape");
        }
        int32_t status = check_product(gate, row_start, row_count, tokens, out_stride, nullptr);
        if (status == SYN_B200_OK) status = check_device(gate);
        if (status == SYN_B200_OK) status = check_device(up);
        if (status != SYN_B200_OK) {
            return status;
        }
        if (reinterpret_cast<uintptr_t>(scratch) & 255) {
            return fail(SYN_B200_INVALID_ARGUMENT, "activation scratch must be 256-byte aligned");
        }
        Epilogue fused;
        status = convert_gather(gather, fused);
        if (status != SYN_B200_OK) {
            return status;
        }
        MatvecArgs args{};
        args.form = 2;
        args.segment_count = 2;
        args.segments[0].matrix = gate;
        args.segments[1].matrix = up;
        args.segments[0].row_start = args.segments[1].row_start = row_start;
        args.segments[0].row_count = args.segments[1].row_count = row_count;
        args.matrix = gate;
        args.row_start = row_start;
        args.row_count = row_count;
        args.tokens = tokens;
        args.act = act_view(scratch, tokens, gate->columns);
        args.act_ready = true;
        args.y = y;
        args.out_stride = out_stride;
        args.mode = SYN_B200_MODE_XQ8;
        args.epilogue = SYN_B200_EPILOGUE_STORE;
        args.fused = fused;
        cudaError_t error = launch_matvec(args, static_cast<cudaStream_t>(stream));
        if (error == cudaErrorNotSupported) {
            // several tokens, or rows longer than one pass of a team: the gate projection goes to memory after all
            if (!gate_values) {
                return fail(SYN_B200_INVALID_ARGUMENT, "this shape runs as two launches and needs gate_values (tokens x out_stride floats)");
            }
            MatvecArgs one = args;
            one.form = 0;
            one.fused = Epilogue{};
            one.y = gate_values;
            error = launch_matvec(one, static_cast<cudaStream_t>(stream));
            if (error == cudaSuccess) {
                one.matrix = up;
                one.y = y;
                one.fused = fused;
                one.fused.gate = gate_values;
                one.fused.gate_stride = out_stride;
                error = launch_matvec(one, static_cast<cudaStream_t>(stream));
            }
        }
        return error == cudaSuccess ? SYN_B200_OK : cuda_fail(error, "launching the matrix-vector kernel");
    });
}

int32_t syn_b200_matvec(const syn_b200_matrix *matrix, uint64_t row_start, uint64_t row_count, const float *x, uint64_t tokens,
                        uint64_t in_stride, float *y, uint64_t out_stride, uint32_t mode, uint32_t epilogue)
{
    if (!matrix || !x || !y) {
        return fail(SYN_B200_NULL_POINTER, "matrix, activations or output");
    }
    return guarded([&]() -> int32_t {
        uint64_t out_floats = 0;
        int32_t status = check_product(matrix, row_start, row_count, tokens, out_stride, &out_floats);
        if (status == SYN_B200_OK) status = check_device(matrix);
        if (status != SYN_B200_OK) {
            return status;
        }
        if (in_stride < matrix->columns) {
            return fail(SYN_B200_INVALID_ARGUMENT, "input stride " + std::to_string(in_stride) + " is below the matrix width " +
                                                       std::to_string(matrix->columns));
        }
        if (mode > SYN_B200_MODE_XF32 || epilogue > SYN_B200_EPILOGUE_ACCUMULATE) {
            return fail(SYN_B200_INVALID_ARGUMENT, "unknown activation mode or epilogue");
        }
        syn_b200_matrix *m = const_cast<syn_b200_matrix *>(matrix);
        const uint64_t K = m->columns;
        const uint64_t x_bytes = align_up(tokens * K * 4, 256);
        const uint64_t y_bytes = align_up(out_floats * 4, 256);
        const ActLayout layout = act_layout(tokens, K);
        status = ensure_stage(m, x_bytes + y_bytes + layout.total);
        if (status != SYN_B200_OK) {
            return status;
        }
        uint8_t *stage = static_cast<uint8_t *>(m->stage);
        float *dx = reinterpret_cast<float *>(stage);
        float *dy = reinterpret_cast<float *>(stage + x_bytes);
        void *scratch = stage + x_bytes + y_bytes;
        cudaError_t error = cudaMemcpy2DAsync(dx, K * 4, x, in_stride * 4, K * 4, tokens, cudaMemcpyHostToDevice, nullptr);
        if (error == cudaSuccess && (epilogue == SYN_B200_EPILOGUE_ACCUMULATE || (tokens > 1 && out_stride != row_count))) {
            // keep the caller's bytes in the stride gaps and, for accumulate, the values to add to
            error = cudaMemcpyAsync(dy, y, out_floats * 4, cudaMemcpyHostToDevice, nullptr);
        }
        if (error != cudaSuccess) {
            cudaGetLastError();
            return cuda_fail(error, "copying activations to the device");
        }
        status = product_dev(m, row_start, row_count, dx, tokens, K, dy, out_stride, mode, epilogue, scratch, layout.total, nullptr);
        if (status != SYN_B200_OK) {
            return status;
        }
        error = cudaMemcpyAsync(y, dy, out_floats * 4, cudaMemcpyDeviceToHost, nullptr);
        if (error == cudaSuccess) {
            error = cudaStreamSynchronize(nullptr);
        }
        if (error != cudaSuccess) {
            cudaGetLastError();
            return cuda_fail(error, "running the product");
        }
        return SYN_B200_OK;
    });
}

int32_t syn_b200_matmul_q8(const syn_b200_matrix *matrix, uint64_t row_start, uint64_t row_count, const int8_t *codes,
                           const float *scales, uint64_t tokens, float *output, uint64_t output_stride)
{
    if (!matrix || !codes || !scales || !output) {
        return fail(SYN_B200_NULL_POINTER, "matrix, codes, scales or output");
    }
    return guarded([&]() -> int32_t {
        uint64_t out_floats = 0;
        int32_t status = check_product(matrix, row_start, row_count, tokens, output_stride, &out_floats);
        if (status == SYN_B200_OK) status = check_device(matrix);
        if (status != SYN_B200_OK) {
            return status;
        }
        syn_b200_matrix *m = const_cast<syn_b200_matrix *>(matrix);
        const uint64_t K = m->columns;
        const ActLayout layout = act_layout(tokens, K);
        const uint64_t y_bytes = align_up(out_floats * 4, 256);
        status = ensure_stage(m, layout.total + y_bytes);
        if (status != SYN_B200_OK) {
            return status;
        }
        uint8_t *stage = static_cast<uint8_t *>(m->stage);
        float *dy = reinterpret_cast<float *>(stage + layout.total);
        cudaError_t error = cudaMemcpyAsync(stage + layout.codes, codes, tokens * K, cudaMemcpyHostToDevice, nullptr);
        if (error == cudaSuccess) {
            error = cudaMemcpyAsync(stage + layout.scales, scales, tokens * (K / 32) * 4, cudaMemcpyHostToDevice, nullptr);
        }
        if (error == cudaSuccess && tokens > 1 && output_stride != row_count) {
            error = cudaMemcpyAsync(dy, output, out_floats * 4, cudaMemcpyHostToDevice, nullptr);
        }
        if (error == cudaSuccess) {
            error = launch_group_sums(reinterpret_cast<const int8_t *>(stage + layout.codes), tokens * K / 16,
                                      reinterpret_cast<int16_t *>(stage + layout.sums), nullptr);
        }
        if (error != cudaSuccess) {
            cudaGetLastError();
            return cuda_fail(error, "copying quantised activations to the device");
        }
        MatvecArgs args{};
        args.matrix = m;
        args.row_start = row_start;
        args.row_count = row_count;
        args.tokens = tokens;
        args.act = act_view(stage, tokens, K);
        args.act_ready = true;
        args.y = dy;
        args.out_stride = output_stride;
        args.mode = SYN_B200_MODE_XQ8;
        args.epilogue = SYN_B200_EPILOGUE_STORE;
        error = launch_matvec(args, nullptr);
        if (error == cudaSuccess) {
            error = cudaMemcpyAsync(output, dy, out_floats * 4, cudaMemcpyDeviceToHost, nullptr);
        }
        if (error == cudaSuccess) {
            error = cudaStreamSynchronize(nullptr);
        }
        if (error != cudaSuccess) {
            cudaGetLastError();
            return cuda_fail(error, "running the product");
        }
        return SYN_B200_OK;
    });
}

int32_t syn_b200_block_dots(const syn_b200_matrix *matrix, uint64_t row_start, uint64_t row_count, const int8_t *codes,
                            uint64_t tokens, int32_t *out)
{
    if (!matrix || !codes || !out) {
        return fail(SYN_B200_NULL_POINTER, "matrix, codes or output");
    }
    return guarded([&]() -> int32_t {
        int32_t status = check_product(matrix, row_start, row_count, tokens, row_count, nullptr);
        if (status == SYN_B200_OK) status = check_device(matrix);
        if (status != SYN_B200_OK) {
            return status;
        }
        syn_b200_matrix *m = const_cast<syn_b200_matrix *>(matrix);
        const uint64_t K = m->columns;
        const uint64_t groups = m->type == kQ6_K ? K / 16 : K / 32;
        const ActLayout layout = act_layout(tokens, K);
        const uint64_t dump_bytes = align_up(tokens * row_count * groups * 4, 256);
        const uint64_t y_bytes = align_up(tokens * row_count * 4, 256);
        status = ensure_stage(m, layout.total + dump_bytes + y_bytes);
        if (status != SYN_B200_OK) {
            return status;
        }
        uint8_t *stage = static_cast<uint8_t *>(m->stage);
        cudaError_t error = cudaMemcpyAsync(stage + layout.codes, codes, tokens * K, cudaMemcpyHostToDevice, nullptr);
        if (error == cudaSuccess) {
            error = cudaMemsetAsync(stage + layout.scales, 0, tokens * (K / 32) * 4, nullptr);
        }
        if (error == cudaSuccess) {
            error = launch_group_sums(reinterpret_cast<const int8_t *>(stage + layout.codes), tokens * K / 16,
                                      reinterpret_cast<int16_t *>(stage + layout.sums), nullptr);
        }
        MatvecArgs args{};
        args.matrix = m;
        args.row_start = row_start;
        args.row_count = row_count;
        args.tokens = tokens;
        args.act = act_view(stage, tokens, K);
        args.act_ready = true;
        args.y = reinterpret_cast<float *>(stage + layout.total + dump_bytes);
        args.out_stride = row_count;
        args.mode = SYN_B200_MODE_XQ8;
        args.dump = reinterpret_cast<int32_t *>(stage + layout.total);
        if (error == cudaSuccess) {
            error = launch_matvec(args, nullptr);
        }
        if (error == cudaSuccess) {
            error = cudaMemcpyAsync(out, args.dump, tokens * row_count * groups * 4, cudaMemcpyDeviceToHost, nullptr);
        }
        if (error == cudaSuccess) {
            error = cudaStreamSynchronize(nullptr);
        }
        if (error != cudaSuccess) {
            cudaGetLastError();
            return cuda_fail(error, "running the block-dot hook");
        }
        return SYN_B200_OK;
    });
}

uint64_t syn_b200_gemm_scratch_bytes(uint64_t tokens, uint64_t columns) { return gemm_scratch_bytes(tokens, columns); }

int32_t syn_b200_gemm_dev(const syn_b200_matrix *matrix, const float *x, uint64_t tokens, uint64_t in_stride, float *y,
                          uint64_t out_stride, uint32_t precision, void *scratch, uint64_t scratch_bytes, void *stream)
{
    if (!matrix || !x || !y || !scratch) {
        return fail(SYN_B200_NULL_POINTER, "matrix, activations, output or scratch");
    }
    return guarded([&]() -> int32_t {
        int32_t status = check_product(matrix, 0, matrix->rows, tokens, out_stride, nullptr);
        if (status == SYN_B200_OK) status = check_device(matrix);
        if (status != SYN_B200_OK) {
            return status;
        }
        return launch_gemm(matrix, x, tokens, in_stride, y, out_stride, precision, scratch, scratch_bytes,
                           static_cast<cudaStream_t>(stream));
    });
}

int32_t syn_b200_gemm(const syn_b200_matrix *matrix, const float *x, uint64_t tokens, uint64_t in_stride, float *y,
                      uint64_t out_stride, uint32_t precision)
{
    if (!matrix || !x || !y) {
        return fail(SYN_B200_NULL_POINTER, "matrix, activations or output");
    }
    return guarded([&]() -> int32_t {
        uint64_t out_floats = 0;
        int32_t status = check_product(matrix, 0, matrix->rows, tokens, out_stride, &out_floats);
        if (status == SYN_B200_OK) status = check_device(matrix);
        if (status != SYN_B200_OK) {
            return status;
        }
        if (in_stride < matrix->columns) {
            return fail(SYN_B200_INVALID_ARGUMENT, "input stride is below the matrix width");
        }
        syn_b200_matrix *m = const_cast<syn_b200_matrix *>(matrix);
        const uint64_t K = m->columns;
        const uint64_t x_bytes = align_up(tokens * K * 4, 256);
        const uint64_t y_bytes = align_up(out_floats * 4, 256);
        const uint64_t scratch_bytes = gemm_scratch_bytes(tokens, K);
        status = ensure_stage(m, x_bytes + y_bytes + scratch_bytes);
        if (status != SYN_B200_OK) {
            return status;
        }
        uint8_t *stage = static_cast<uint8_t *>(m->stage);
        float *dx = reinterpret_cast<float *>(stage);
        float *dy = reinterpret_cast<float *>(stage + x_bytes);
        cudaError_t error = cudaMemcpy2DAsync(dx, K * 4, x, in_stride * 4, K * 4, tokens, cudaMemcpyHostToDevice, nullptr);
        if (error == cudaSuccess && out_stride != m->rows) {
            error = cudaMemcpyAsync(dy, y, out_floats * 4, cudaMemcpyHostToDevice, nullptr);
        }
        if (error != cudaSuccess) {
            cudaGetLastError();
            return cuda_fail(error, "copying activations to the device");
        }
        status = launch_gemm(m, dx, tokens, K, dy, out_stride, precision, stage + x_bytes + y_bytes, scratch_bytes, nullptr);
        if (status != SYN_B200_OK) {
            return status;
        }
        error = cudaMemcpyAsync(y, dy, out_floats * 4, cudaMemcpyDeviceToHost, nullptr);
        if (error == cudaSuccess) {
            error = cudaStreamSynchronize(nullptr);
        }
        if (error != cudaSuccess) {
            cudaGetLastError();
            return cuda_fail(error, "running the tensor-core product");
        }
        return SYN_B200_OK;
    });
}

}  // extern "C"
