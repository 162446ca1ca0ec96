// syn_b200_matvec_static: the quantised-activation product for callers that must not allocate device memory.
//
// Who needs it: code that runs where cudaMalloc is off the table -- a host thread inside a latency-critical decode
// loop that may not take the allocator's lock, a plugin that was handed a fixed memory budget by its embedder, a
// process whose CUDA context is shared and whose owner forbids new allocations after start-up. The ordinary
// device entry point (syn_b200_matvec_dev) makes such a caller bring its own scratch for the quantised
// activations; this one keeps that scratch inside the library image instead, in a fixed array that every device
// loading the library holds until the process exits.
//
// What it costs: kStaticActivationValues activation values at most per call (tokens x columns), one shared array
// per device -- two calls that overlap on the GPU (different streams, or a graph with parallel branches) race on
// it -- and the array keeps the previous call's contents (every element a call reads is rewritten by that call's
// own quantiser first, so nothing has to be cleared).
#include "common.cuh"

namespace syn {

namespace {

// tokens x columns a call may quantise: 8 tokens of a 32768-wide layer, or one token of 262144 values.
constexpr uint64_t kStaticActivationValues = 8ull * 32768ull;
// codes (1 B/value) + block scales (4 B per 32) + 16-value sums (2 B per 16) + the three 256-byte roundings
constexpr uint64_t kStaticScratchBytes = kStaticActivationValues + kStaticActivationValues / 8 + kStaticActivationValues / 8 + 3 * 256;

static __device__ __align__(256) uint8_t g_static_scratch[kStaticScratchBytes];

// Device address of g_static_scratch on each device, resolved once per device with that device current.
// In host code the array's name is only a handle for the runtime: it is never passed to a kernel.
void *g_static_address[64] = {nullptr};

int32_t static_scratch(int device, void **out)
{
    if (device < 0 || device >= 64) {
        return fail(SYN_B200_INVALID_ARGUMENT, "device index " + std::to_string(device) + " is outside the supported range");
    }
    if (!g_static_address[device]) {
        void *address = nullptr;
        cudaError_t error = cudaGetSymbolAddress(&address, g_static_scratch);
        if (error != cudaSuccess || !address) {
            cudaGetLastError();
            return cuda_fail(error, "resolving the built-in activation scratch");
        }
        g_static_address[device] = address;
    }
    *out = g_static_address[device];
    return SYN_B200_OK;
}

}  // namespace

}  // namespace syn

using namespace syn;

extern "C" uint64_t syn_b200_matvec_static_capacity(void) { return kStaticActivationValues; }

extern "C" int32_t syn_b200_matvec_static(const syn_b200_matrix *matrix, uint64_t row_start, uint64_t row_count, const float *x,
                                          uint64_t tokens, uint64_t in_stride, float *y, uint64_t out_stride, uint32_t epilogue,
                                          void *stream)
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
        if (epilogue > SYN_B200_EPILOGUE_ACCUMULATE) {
            return fail(SYN_B200_INVALID_ARGUMENT, "unknown epilogue " + std::to_string(epilogue));
        }
        const uint64_t K = matrix->columns;
        if (tokens > kStaticActivationValues / K) {
            return fail(SYN_B200_INVALID_ARGUMENT, std::to_string(tokens) + " tokens of " + std::to_string(K) + " values exceed the built-in scratch of " +
                                                       std::to_string(kStaticActivationValues) + " activation values; use syn_b200_matvec_dev with caller scratch");
        }
        if (in_stride < K || in_stride % 4 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0) {
            return fail(SYN_B200_INVALID_ARGUMENT, "device activations must be 16-byte aligned with a stride that covers the row and is a multiple of 4 floats");
        }
        void *scratch = nullptr;
        status = static_scratch(matrix->device, &scratch);
        if (status != SYN_B200_OK) {
            return status;
        }
        if (act_layout(tokens, K).total > kStaticScratchBytes) {
            return fail(SYN_B200_INVALID_ARGUMENT, "the activation layout does not fit the built-in scratch");
        }
        // Exactly what syn_b200_matvec_dev queues in its quantised-activation mode, with the built-in array as the
        // scratch: the kernel quantises x itself where it can (one token: a single launch), and the shapes where it
        // cannot get a quantiser launch into the array first.
        MatvecArgs args{};
        args.matrix = matrix;
        args.row_start = row_start;
        args.row_count = row_count;
        args.tokens = tokens;
        args.act = act_view(scratch, tokens, K);
        args.act_ready = false;
        args.x = x;
        args.in_stride = in_stride;
        args.y = y;
        args.out_stride = out_stride;
        args.mode = SYN_B200_MODE_XQ8;
        args.epilogue = epilogue;
        const cudaError_t error = launch_matvec(args, static_cast<cudaStream_t>(stream));
        return error == cudaSuccess ? SYN_B200_OK : cuda_fail(error, "launching the matrix-vector kernel");
    });
}
