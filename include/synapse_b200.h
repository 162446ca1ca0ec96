/*
 * synapse_b200 — C ABI of the B200 (sm_100a) CUDA backend for Synapse's quantized matrix products.
 *
 * The library stands beside the reference's two native libraries and keeps their conventions
 * (native/synapse-kernels/src/Features/CpuKernels/ffi.rs, native/synapse-gpu/src/Features/GpuKernels/ffi.rs):
 *   - every entry point returns an int32 status (0 = OK) and never throws or aborts across the ABI;
 *   - the caller owns every buffer for the duration of the call, the callee never frees caller memory;
 *   - a thread-local message describing the last failure is read with syn_b200_last_error;
 *   - the loader checks syn_b200_abi_version before any other call;
 *   - a matrix handle must not be used by two threads at once (the reference serialises model calls,
 *     src/Synapse.Runtime/Features/TextGeneration/Qwen2/Qwen2Model.cs:164);
 *   - nothing falls back to a CPU path: without a usable sm_100 device calls fail with SYN_B200_UNAVAILABLE.
 *
 * Weight blocks are plain GGUF, row-major [rows][columns], accepted unmodified:
 *   Q8_0 (type 8): 34 B / 32 values; Q4_K (type 12): 144 B / 256 values; Q6_K (type 14): 210 B / 256 values
 *   (native/synapse-gpu/src/Features/GpuKernels/decoder/encoding.rs:6-10,41-56).
 */
#ifndef SYNAPSE_B200_H
#define SYNAPSE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define SYN_B200_API __attribute__((visibility("default")))
#else
#define SYN_B200_API
#endif

#define SYN_B200_ABI_VERSION 1u

/* Status codes: the reference GPU ABI's (native/synapse-gpu/src/Features/GpuKernels/error.rs:3-16).
 * The C# side maps 3 to NotSupportedException, 5 to InsufficientMemoryException, the rest to
 * InvalidOperationException (src/Synapse.Runtime/Features/GpuKernels/NativeGpuLibrary.cs:130-145). */
#define SYN_B200_OK 0
#define SYN_B200_NULL_POINTER 1
#define SYN_B200_INVALID_ARGUMENT 2
#define SYN_B200_UNAVAILABLE 3
#define SYN_B200_DEVICE_ERROR 4
#define SYN_B200_OUT_OF_MEMORY 5
#define SYN_B200_INTERNAL 6 /* a C++ exception was caught at the ABI (the reference's STATUS_PANIC) */

/* GGML tensor type ids of the accepted encodings. */
#define SYN_B200_TYPE_Q8_0 8u
#define SYN_B200_TYPE_Q4_K 12u
#define SYN_B200_TYPE_Q6_K 14u

/* syn_b200_matrix_create flags. */
#define SYN_B200_REPACK 1u /* load-time repack into the coalesced planar layout (same byte count) */

/* Activation contract of a product (the reference has three numeric contracts,
 * docs/ADR/ADR-006-cpu-kernel-backends-and-native-boundary.md:20-24). */
#define SYN_B200_MODE_XQ8 0u /* activations Q8_0-quantised per 32 exactly as Q8ActivationQuantizer does; integer block dots */
#define SYN_B200_MODE_XF32 1u /* FP32 activations x exactly dequantised weights (the `reference` backend's contract) */

/* Epilogue of a product (the fused regions of Qwen2ProjectionWork.cs:7-88 and `accumulate` of
 * native/synapse-gpu/.../cuda/kernels/common.cuh:52-69). */
#define SYN_B200_EPILOGUE_STORE 0u      /* y = W x */
#define SYN_B200_EPILOGUE_ACCUMULATE 1u /* y += W x (residual add) */

/* Operand precision of the tensor-core product. */
#define SYN_B200_GEMM_F16 0u   /* weights and activations rounded to fp16, FP32 accumulation */
#define SYN_B200_GEMM_F16X2 1u /* both operands carried as fp16 high + low parts (22 bits), three MMAs per k step: the FP32-activation
                                  product of the reference up to FP32 accumulation order, at about a third of the F16 rate */

/* Mirrors GpuDeviceInfo (native/synapse-gpu/src/Features/GpuKernels/mod.rs:20-31), 152 bytes. */
typedef struct syn_b200_device_info {
    char name[128];                /* NUL-terminated, e.g. "NVIDIA B200 (sm_100)" */
    uint64_t total_memory_bytes;   /* device memory */
    uint64_t max_buffer_bytes;     /* largest single allocation the library will try */
    uint32_t compute_capability;   /* major * 10 + minor */
    uint32_t multiprocessors;
} syn_b200_device_info;

typedef struct syn_b200_matrix syn_b200_matrix;

/* Fused epilogue of a device product: v = dot (+ bias[r]); v = silu(gate[t][r]) * v when gate is set;
 * y = accumulate ? y + v : v. Mirrors the fused regions of the reference's CPU executor -- Q/K/V bias add, residual
 * add, gate/up SwiGLU (src/Synapse.Runtime/Features/TextGeneration/Qwen2/Qwen2ProjectionWork.cs:7-131) -- and the
 * bias / accumulate fields of MatmulArgs (native/synapse-gpu/.../cuda/kernels/common.cuh:52-69). Rows are counted from
 * the first row of the call. All pointers are DEVICE memory; null switches the term off. */
typedef struct syn_b200_epilogue {
    const float *bias;    /* row_count floats */
    const float *gate;    /* tokens rows of gate_stride floats: results of the gate projection for the same rows */
    uint64_t gate_stride;
    uint32_t accumulate;  /* 1: add to y (residual) */
    uint32_t reserved;    /* must be 0 */
} syn_b200_epilogue;

/* Replaces synapse_kernels_abi_version / synapse_gpu_abi_version (ffi.rs:22 / ffi.rs:55-59). */
SYN_B200_API uint32_t syn_b200_abi_version(void);

/* Replaces synapse_gpu_probe (native/synapse-gpu/.../ffi.rs:61-77): describes the current CUDA device.
 * SYN_B200_UNAVAILABLE when there is no device or it is not compute capability 10.x. */
SYN_B200_API int32_t syn_b200_probe(syn_b200_device_info *out);

/* Replaces synapse_gpu_last_error (ffi.rs:89-104): copies the calling thread's last error message (UTF-8,
 * not terminated) and returns its full length. `buffer` may be null. */
SYN_B200_API size_t syn_b200_last_error(uint8_t *buffer, size_t capacity);

/* Loads a row-major matrix of GGUF blocks from HOST memory onto the current device. Replaces the weight
 * upload of the reference CUDA backend (native/synapse-gpu/.../cuda/decoder.rs:59-60) and the view type
 * Q8Matrix (src/Synapse.Runtime/Features/CpuKernels/Q8Matrix.cs:6-55). The host bytes are not referenced
 * after the call. `columns` must be a whole number of blocks (decoder/checks.rs:185-190 -> UNAVAILABLE). */
SYN_B200_API int32_t syn_b200_matrix_create(const void *host_blocks, uint32_t ggml_type, uint64_t rows, uint64_t columns,
                               uint32_t flags, syn_b200_matrix **out);

/* Same, from blocks that already sit in DEVICE memory (copied device-to-device on `stream`, then repacked). */
SYN_B200_API int32_t syn_b200_matrix_create_from_device(const void *device_blocks, uint32_t ggml_type, uint64_t rows,
                                           uint64_t columns, uint32_t flags, void *stream, syn_b200_matrix **out);

/* Releases a matrix; null is ignored (ffi.rs:262-271). */
SYN_B200_API void syn_b200_matrix_destroy(syn_b200_matrix *matrix);

/* Shape query: any out pointer may be null. `source_bytes` = rows * row bytes of the GGUF encoding. */
SYN_B200_API int32_t syn_b200_matrix_info(const syn_b200_matrix *matrix, uint32_t *ggml_type, uint64_t *rows,
                             uint64_t *columns, uint32_t *flags, uint64_t *source_bytes);

/* Q8_0 activation quantiser, HOST buffers. Replaces Q8ActivationQuantizer.QuantizeRow
 * (src/Synapse.Runtime/Features/CpuKernels/Q8ActivationQuantizer.cs:15-57): per 32 values
 * scale = max|x|/127, code = round_half_even(x * (1/scale)) with the unrounded scale, stored scale rounded
 * through fp16. x: tokens rows of in_stride floats; codes: tokens*columns; scales: tokens*columns/32. */
SYN_B200_API int32_t syn_b200_quantize_q8(const float *x, uint64_t tokens, uint64_t columns, uint64_t in_stride,
                             int8_t *codes, float *scales);

/* Q8_0-quantised activations x matrix rows, HOST buffers. Replaces synapse_q8_0_matmul
 * (native/synapse-kernels/src/Features/CpuKernels/ffi.rs:44-54) and Q8MatrixKernel.Multiply
 * (src/Synapse.Runtime/Features/CpuKernels/Q8MatrixKernel.cs:11-48):
 *   output[t * output_stride + (r - row_start)] = dot(W[r], A[t]),  r in [row_start, row_start + row_count).
 * codes: tokens*columns int8; scales: tokens*columns/32 floats; output holds (tokens-1)*stride + row_count
 * floats and must not alias the inputs. Works for Q8_0, Q4_K and Q6_K matrices. */
SYN_B200_API int32_t syn_b200_matmul_q8(const syn_b200_matrix *matrix, uint64_t row_start, uint64_t row_count,
                           const int8_t *codes, const float *scales, uint64_t tokens, float *output,
                           uint64_t output_stride);

/* FP32 activations x matrix rows, HOST buffers; quantises in-library when mode is XQ8. Replaces one
 * projection of the reference GPU step (native/synapse-gpu/.../step/projection.rs:51-72; kernels
 * cuda/kernels/matmul.cu:79-189) and, in XF32 mode, Q8Operators.Multiply / DecodedRowOperators.Multiply
 * (src/Synapse.Runtime/Features/GraphExecution/Q8Operators.cs:46-98, DecodedRowOperators.cs:20-41).
 * Every token count runs on the matrix-vector kernels here (results do not depend on the token count of a call); the
 * tensor-core product is syn_b200_gemm. */
SYN_B200_API int32_t syn_b200_matvec(const syn_b200_matrix *matrix, uint64_t row_start, uint64_t row_count, const float *x,
                        uint64_t tokens, uint64_t in_stride, float *y, uint64_t out_stride, uint32_t mode,
                        uint32_t epilogue);

/* Prompt-run product on the tensor cores, HOST buffers: Y[t * out_stride + r] = sum_k W[r][k] X[t][k].
 * Replaces synapse_q8_gemm (cuda/kernels/matmul.cu:147-189) and the Metal K-quant GEMMs
 * (metal/shaders/matmul_kquant.metal:227-291). */
SYN_B200_API int32_t syn_b200_gemm(const syn_b200_matrix *matrix, const float *x, uint64_t tokens, uint64_t in_stride,
                      float *y, uint64_t out_stride, uint32_t precision);

/* Test hook: the exact integer sub-block dots of the XQ8 contract, HOST buffers.
 * out[(t*row_count + r) * groups + g]; groups per row = columns/32 (Q8_0), columns/32 (Q4_K, one per
 * sub-block), columns/16 (Q6_K). The sums come, token by token, out of the kernel variant that a single-token product of
 * the same rows takes (the pipelined kernel, also its sixteen-warp form for the largest matrices), built with this hook
 * compiled in. */
SYN_B200_API int32_t syn_b200_block_dots(const syn_b200_matrix *matrix, uint64_t row_start, uint64_t row_count,
                            const int8_t *codes, uint64_t tokens, int32_t *out);

/* ---- GGUF files: the tensor table and per-tensor loading on the native side. Replaces the header reader and tensor
 * table of the reference's runtime (src/Synapse.Runtime/Features/ModelLoading/Gguf/GgufHeaderReader.cs:20-154,
 * GgufTensorInfo.cs) for callers that hand the library a file instead of block pointers, and the whole-file device copy
 * of the reference's CUDA backend (native/synapse-gpu/src/Features/GpuKernels/cuda/decoder.rs:59-60): tensors are
 * uploaded one by one from the mapped file. Same rules as the reference: GGUF version 2 or 3; at most 1,000,000 tensors
 * and metadata entries; rank 1 to 8; general.alignment a power of two (default 32); F32, Q8_0, Q4_K and Q6_K tensors
 * (anything else: SYN_B200_UNAVAILABLE); a tensor outside the file or a truncated header: SYN_B200_INVALID_ARGUMENT. ---- */

typedef struct syn_b200_gguf syn_b200_gguf;

/* One entry of the tensor table (GgufTensorInfo): `dimensions[0]` is the row length, `offset` is absolute in the file. */
typedef struct syn_b200_gguf_tensor {
    char name[128]; /* NUL-terminated (longer names are cut) */
    uint32_t ggml_type;
    uint32_t rank;
    uint64_t dimensions[8]; /* unused entries are 1 */
    uint64_t offset;
    uint64_t bytes;
} syn_b200_gguf_tensor;

SYN_B200_API int32_t syn_b200_gguf_open(const char *path, syn_b200_gguf **out); /* maps the file read-only and parses its header */
SYN_B200_API void syn_b200_gguf_close(syn_b200_gguf *gguf);                     /* null is ignored */
SYN_B200_API uint64_t syn_b200_gguf_tensor_count(const syn_b200_gguf *gguf);
SYN_B200_API int32_t syn_b200_gguf_tensor_at(const syn_b200_gguf *gguf, uint64_t index, syn_b200_gguf_tensor *out);
SYN_B200_API int32_t syn_b200_gguf_find(const syn_b200_gguf *gguf, const char *name, syn_b200_gguf_tensor *out);
/* The mapped file (valid until close), its length and the offset of its data section: what syn_b200_decoder_desc.weights
 * and the tensor offsets refer to when a decoder is created from a file. */
SYN_B200_API const uint8_t *syn_b200_gguf_mapping(const syn_b200_gguf *gguf, uint64_t *length, uint64_t *data_offset);
/* syn_b200_matrix_create for the two-dimensional tensor `name` (rows = dimensions[1], columns = dimensions[0], as
 * src/Synapse.Runtime/Features/CpuKernels/Q8Matrix.cs:51-54). With `cache_directory` (may be null) a repacked device image is
 * written there after the first load and read back instead of repacking on later loads; entries are keyed by a digest of
 * the file's header and length and by the tensor's name and offset, and a cache that cannot be read or written is ignored. */
SYN_B200_API int32_t syn_b200_gguf_load_matrix(const syn_b200_gguf *gguf, const char *name, uint32_t flags, const char *cache_directory,
                                               syn_b200_matrix **out);

/* ---- Device-resident variants: every pointer is DEVICE memory on the matrix's device; work is queued on
 * `stream` (a cudaStream_t, null = default stream) and not synchronised. These are what a resident decode
 * loop calls; they replace the launches of step/projection.rs without the per-step host copies of
 * cuda/decoder.rs:106-145. ---- */

/* Bytes of device scratch syn_b200_matvec_dev needs in XQ8 mode for `tokens` x `columns` activations
 * (codes, block scales and 16-value code sums). */
SYN_B200_API uint64_t syn_b200_activation_scratch_bytes(uint64_t tokens, uint64_t columns);

/* Quantises FP32 device activations into a scratch area laid out by the library. */
SYN_B200_API int32_t syn_b200_quantize_q8_dev(const float *x, uint64_t tokens, uint64_t columns, uint64_t in_stride,
                                 void *scratch, uint64_t scratch_bytes, void *stream);

/* y (+)= W[row_start : row_start+row_count] * act, activations taken from a scratch area filled by
 * syn_b200_quantize_q8_dev with the same tokens/columns. */
SYN_B200_API int32_t syn_b200_matmul_q8_dev(const syn_b200_matrix *matrix, uint64_t row_start, uint64_t row_count,
                               const void *scratch, uint64_t tokens, float *y, uint64_t out_stride,
                               uint32_t epilogue, void *stream);

/* syn_b200_matmul_q8_dev with a fused epilogue (null = plain store). */
SYN_B200_API int32_t syn_b200_matmul_q8_ex_dev(const syn_b200_matrix *matrix, uint64_t row_start, uint64_t row_count,
                                               const void *scratch, uint64_t tokens, float *y, uint64_t out_stride,
                                               const syn_b200_epilogue *epilogue, void *stream);

/* Where a row-sharded product puts its results besides `y`, and how it tells the other GPUs that they are there.
 * `peer_outputs`: `peer_count` (at most 7) DEVICE pointers, the other GPUs' copies of the output mapped into this process
 * (syn_b200_shared_buffer_open), offset like `y` to the shard's first row; `peer_outputs` itself is a host array.
 * `signals` (host array, may be null): peer_count + 1 DEVICE pointers to 32-bit words, this rank's word of the product's
 * signal array in this GPU's memory first, then in each peer's. `arrivals`: two zero-initialised words in THIS GPU's memory
 * that belong to this product alone. When the last CTA of the launch has stored its results it writes the launch's
 * sequence number (1, 2, ... per product, counted in arrivals[1]) to every signal word, ordered behind all stores of the
 * launch at system scope. A GPU whose signal array shows sequence number n in every word holds the n-th gathered vector
 * complete (syn_b200_gather_wait_dev). Launches that share signal words must be ordered on one stream. */
typedef struct syn_b200_gather {
    float *const *peer_outputs;
    uint32_t peer_count;
    uint32_t reserved; /* must be 0 */
    uint32_t *const *signals;
    uint32_t *arrivals;
} syn_b200_gather;

/* syn_b200_matmul_q8_dev for a row shard of a matrix that is split over several GPUs: the kernel stores every result
 * into `y` AND at the same position of the peers' copies of the output -- plain stores over NVLink from the lane that
 * holds the result, so the gather of the output slices happens inside the product instead of in an all-gather after
 * it -- and signals completion as `gather` describes. The reference has no multi-GPU path
 * (native/synapse-gpu/src/Features/GpuKernels/ffi.rs:113-271 drives one device); this is the exchange step of the
 * row-sharded configuration. */
SYN_B200_API int32_t syn_b200_matmul_q8_gather_dev(const syn_b200_matrix *matrix, uint64_t row_start, uint64_t row_count,
                                                   const void *scratch, uint64_t tokens, float *y, uint64_t out_stride,
                                                   const syn_b200_gather *gather, void *stream);

/* Queues a one-warp kernel that waits until each of the `count` (1..8) words of this GPU's signal array `signals` has
 * reached the next sequence number, *epoch + 1, and then stores that number to *epoch (a zero-initialised DEVICE word
 * owned by the waiter, so the call can sit in a replayed CUDA graph). Kernels queued behind it on `stream` see the
 * complete gathered vector. The wait is bounded: after `timeout_us` microseconds without the signal the kernel gives
 * up, adds one to the fault count (syn_b200_device_faults) and returns; nothing is left waiting and the context stays
 * usable. Reusing an output vector for the next product before every rank has read it is the caller's protocol (two
 * vectors in turn, or a signal back). No reference counterpart (single-device ABI). */
SYN_B200_API int32_t syn_b200_gather_wait_dev(const uint32_t *signals, uint32_t count, uint32_t *epoch, uint32_t timeout_us,
                                              void *stream);

/* One row range of a product that multiplies several matrices with the same activations in ONE launch. Mirrors
 * MatmulSegment (native/synapse-gpu/src/Features/GpuKernels/params.rs:42-61; cuda/kernels/common.cuh:52-69): a result of
 * row r of the range goes to y[token * out_stride + out_column + r], plus bias[r] when `bias` (DEVICE memory) is set. */
typedef struct syn_b200_segment {
    const syn_b200_matrix *matrix;
    uint64_t row_start, row_count;
    const float *bias;
    uint64_t out_column;
} syn_b200_segment;

/* y[t][out_column_s + r] (+)= W_s[row_start_s + r] . act[t] (+ bias_s[r]) for up to three segments s in one launch:
 * the Q | K | V dispatch of the reference's GPU step (MatmulArgs with three segments, step/layers.rs:71-94) and the row
 * space of Qwen2QkvWork (src/Synapse.Runtime/Features/TextGeneration/Qwen2/Qwen2ProjectionWork.cs:7-53). The segments'
 * matrices must share encoding, layout and width, as in the reference. `accumulate` = 1 adds to y. `gather` as in
 * syn_b200_matmul_q8_gather_dev (null on one GPU; the peer pointers address column 0 like `y`). Every row is computed
 * exactly as in a launch of its own, so results are bit-identical to separate products. */
SYN_B200_API int32_t syn_b200_matmul_q8_segments_dev(const syn_b200_segment *segments, uint32_t count, const void *scratch,
                                                     uint64_t tokens, float *y, uint64_t out_stride, uint32_t accumulate,
                                                     const syn_b200_gather *gather, void *stream);

/* y[t][r] = silu(gate[row_start + r] . act[t]) * (up[row_start + r] . act[t]) in one launch: the gate/up region of the
 * reference's CPU executor (Qwen2GateUpWork, Qwen2ProjectionWork.cs:91-131) and its gate | up dispatch followed by
 * synapse_swiglu (step/layers.rs:159-177, cuda/kernels/elementwise.cu:100-110). The warp that holds gate row r holds up
 * row r too, so for single-token products the gate values never go to memory. Several tokens, or rows longer than one
 * pass of a warp team, run as two launches through `gate_values` (DEVICE, tokens * out_stride floats), which may be null
 * otherwise. `gather` as in syn_b200_matmul_q8_gather_dev (null on one GPU). Bit-identical to the two-launch form. */
SYN_B200_API int32_t syn_b200_matmul_q8_swiglu_dev(const syn_b200_matrix *gate, const syn_b200_matrix *up, uint64_t row_start,
                                                   uint64_t row_count, const void *scratch, uint64_t tokens, float *y,
                                                   uint64_t out_stride, float *gate_values, const syn_b200_gather *gather,
                                                   void *stream);

/* A zero-filled device buffer that other processes on the same box can map (CUDA IPC), for the output vectors of
 * row-sharded products: create it on the owning GPU, hand the 64-byte handle to the other ranks by any means, and let
 * each of them open it WITH ITS OWN GPU CURRENT, which maps the memory for that GPU's kernels over NVLink (peer access is
 * enabled as part of the open). `open` verifies the mapping with a 4-byte copy before it returns; status 3 when the
 * devices have no peer path or the handle cannot be mapped. `close` takes what `open` returned, `destroy` what `create`
 * returned. No reference counterpart (single-device ABI). */
SYN_B200_API int32_t syn_b200_shared_buffer_create(uint64_t bytes, void **device_ptr, uint8_t handle[64]);
SYN_B200_API int32_t syn_b200_shared_buffer_open(const uint8_t handle[64], void **device_ptr);
SYN_B200_API void syn_b200_shared_buffer_close(void *device_ptr);
SYN_B200_API void syn_b200_shared_buffer_destroy(void *device_ptr);

/* Lets kernels of the calling thread's current device read and write memory of `peer_device` (cudaDeviceEnablePeerAccess;
 * already enabled is not an error). A process that maps another GPU's buffer (CUDA IPC) must call this for that GPU before
 * it passes a pointer mapped for ANOTHER device to a gathering product (syn_b200_shared_buffer_open maps for the
 * current device and needs no further call).
 * Status 3 when the two devices have no peer path. No reference counterpart (single-device ABI). */
SYN_B200_API int32_t syn_b200_enable_peer_access(int32_t peer_device);

/* FP32 device activations x matrix rows. XQ8 mode quantises into `scratch` first (required, at least
 * syn_b200_activation_scratch_bytes). XF32 mode needs no scratch; a caller that passes one of at least
 * syn_b200_gemm_scratch_bytes thereby opts into the reference's projection rule (step/projection.rs:14,51-72): whole-matrix
 * products of more than 4 tokens with a plain store then run on the tensor cores with fp16 operands (SYN_B200_GEMM_F16),
 * everything else on the FP32-activation matrix-vector kernels.
 * XQ8 mode with several tokens (the reference's matvec_{2,4,8}, cuda/kernels/matmul.cu:79-145): Q4_K and repacked Q6_K
 * take the exact integer block dots on the tensor cores (mma.sync, u8 x s8), eight tokens per weight pass; a token's
 * result carries the bits of a single-token call whatever shares its pass. */
SYN_B200_API int32_t syn_b200_matvec_dev(const syn_b200_matrix *matrix, uint64_t row_start, uint64_t row_count,
                            const float *x, uint64_t tokens, uint64_t in_stride, float *y, uint64_t out_stride,
                            uint32_t mode, uint32_t epilogue, void *scratch, uint64_t scratch_bytes,
                            void *stream);

/* Same product as syn_b200_matvec_dev in XQ8 mode, for callers that cannot allocate device memory (a decode thread
 * that must not take the allocator's lock, a plugin with a fixed memory budget, a guest in someone else's CUDA
 * context): the scratch for the quantised activations is a fixed array inside the library image, so the call needs
 * nothing beyond the caller's x and y and calls neither cudaMalloc nor cudaFree nor any allocating library routine.
 * Limits: tokens * columns must not exceed syn_b200_matvec_static_capacity() (262144 values, e.g. 8 tokens of 32768),
 * else SYN_B200_INVALID_ARGUMENT; every call on a device shares the one array (about 328 KB per device, held until the
 * process exits), so two calls that overlap on the GPU race and must be ordered by the caller; the array keeps the last
 * call's contents, which is harmless because each call rewrites what it reads. The first call on a device resolves
 * the array's device address (cudaGetSymbolAddress), and the first launch of each kernel variant makes the CUDA runtime
 * load that kernel and raise its shared-memory limit, which the runtime may back with memory of its own: make one
 * warm-up call per matrix shape and device before the region that must not allocate, and outside any stream capture.
 * Results and launches are those of syn_b200_matvec_dev (one token: a single kernel that quantises x itself).
 * No counterpart in the reference. */
SYN_B200_API int32_t syn_b200_matvec_static(const syn_b200_matrix *matrix, uint64_t row_start, uint64_t row_count,
                                            const float *x, uint64_t tokens, uint64_t in_stride, float *y,
                                            uint64_t out_stride, uint32_t epilogue, void *stream);

/* Largest tokens * columns syn_b200_matvec_static accepts. */
SYN_B200_API uint64_t syn_b200_matvec_static_capacity(void);

/* syn_b200_matvec_dev with a fused epilogue (null = plain store). In XF32 mode prompt runs of more than 4 tokens go
 * to the tensor-core product, as the reference's project() does (step/projection.rs:14,51-72); scratch must then hold
 * syn_b200_gemm_scratch_bytes and the epilogue must be null. */
SYN_B200_API int32_t syn_b200_matvec_ex_dev(const syn_b200_matrix *matrix, uint64_t row_start, uint64_t row_count,
                                            const float *x, uint64_t tokens, uint64_t in_stride, float *y,
                                            uint64_t out_stride, uint32_t mode, const syn_b200_epilogue *epilogue,
                                            void *scratch, uint64_t scratch_bytes, void *stream);

/* Bytes of device scratch syn_b200_gemm_dev needs for `tokens` x `columns` activations: the 16-bit operand tiles plus a
 * fixed 21 MB in which products with fewer tiles than half the SMs (few weight rows, few tokens) leave the shares of the
 * CTAs a tile's k range is dealt to; the shares are added in a fixed order, so results do not depend on timing. */
SYN_B200_API uint64_t syn_b200_gemm_scratch_bytes(uint64_t tokens, uint64_t columns);

/* Tensor-core product with device buffers. */
SYN_B200_API int32_t syn_b200_gemm_dev(const syn_b200_matrix *matrix, const float *x, uint64_t tokens, uint64_t in_stride,
                          float *y, uint64_t out_stride, uint32_t precision, void *scratch,
                          uint64_t scratch_bytes, void *stream);

/* ---- Whole decode step (the surround of the matrix products). Same structs as the reference's GPU ABI, so that
 * GpuDecoderExecutor (src/Synapse.Runtime/Features/GpuKernels/GpuDecoderExecutor.cs:135-180) can fill them unchanged;
 * numerics are those of the reference's optimized CPU executor (Q8_0-quantised activations in every projection,
 * src/Synapse.Runtime/Features/TextGeneration/Qwen2/Qwen2CpuExecutor.cs:105-244). ---- */

#define SYN_B200_NO_TENSOR 0xFFFFFFFFFFFFFFFFull

/* DecoderLayerOffsets (native/synapse-gpu/src/Features/GpuKernels/decoder.rs:61-93), 120 bytes: byte offsets of one
 * block's tensors inside `weights`; optional tensors use SYN_B200_NO_TENSOR. `encodings`: GGML type ids of Q, K, V, O,
 * gate, up, down, four bits each from the lowest. Norm weights and biases are FP32. */
typedef struct syn_b200_layer_offsets {
    uint64_t attention_norm, query, key, value, query_bias, key_bias, value_bias, query_norm, key_norm;
    uint64_t attention_output, feed_forward_norm, gate, up, down, encodings;
} syn_b200_layer_offsets;

/* DecoderDesc (decoder.rs:96-131), 136 bytes. `weights` is HOST memory (the mapped model file) and is not referenced
 * after create; rope tables hold context * head_dim/2 floats each (computed by the host, RopeFrequencies.cs:55-78). */
typedef struct syn_b200_decoder_desc {
    const uint8_t *weights;
    uint64_t weights_length;
    const syn_b200_layer_offsets *layers;
    const float *rope_cosines;
    const float *rope_sines;
    uint64_t token_embedding, output_norm, output;
    uint32_t layer_count, hidden, feed_forward, heads, kv_heads, head_dim, vocabulary, context, session_slots;
    uint32_t step_tokens, logits_rows;
    float rms_epsilon;
    uint32_t embedding_encoding, rope_layout, activation, kv_precision, kv_growth_positions, output_encoding;
} syn_b200_decoder_desc;

/* BatchToken (decoder.rs:134-141), 16 bytes: KV slot, token id, position, logits row or -1. */
typedef struct syn_b200_batch_token {
    int32_t slot, token, position, logits_row;
} syn_b200_batch_token;

typedef struct syn_b200_decoder syn_b200_decoder;

/* Replaces synapse_gpu_decoder_create (ffi.rs:113-172). Up to 64 tokens per step (decode tokens of several sessions and
 * prompt runs: tokens of one slot at consecutive positions, the reference's prefill chunks); KV cache of `context`
 * positions per slot, FP32 (kv_precision 0) or FP16 (1: KvPrecision::F16, decoder.rs:43-58 -- keys and values are rounded
 * to the nearest fp16 number on their way in; any other value is status 2); NeoX rotary layout; SwiGLU. A token's logits do not depend on what else shares its step. */
SYN_B200_API int32_t syn_b200_decoder_create(const syn_b200_decoder_desc *desc, syn_b200_decoder **out);

/* Replaces synapse_gpu_decoder_forward (ffi.rs:181-203): one batched step; writes k * vocabulary logits for its k
 * logits rows (numbered 0..k-1 in token order) to HOST memory. */
SYN_B200_API int32_t syn_b200_decoder_forward(syn_b200_decoder *decoder, const syn_b200_batch_token *tokens, uint64_t count,
                                              float *logits, uint64_t logits_capacity);

/* Same step, but only the greedy choice of every logits row comes back (first maximum, as Q8Operators.ArgMax,
 * src/Synapse.Runtime/Features/GraphExecution/Q8Operators.cs:152-173). No counterpart in the reference's ABI. */
SYN_B200_API int32_t syn_b200_decoder_forward_argmax(syn_b200_decoder *decoder, const syn_b200_batch_token *tokens, uint64_t count,
                                                     int32_t *argmax);

/* Replaces synapse_gpu_decoder_destroy (ffi.rs:205-216); null is ignored. */
SYN_B200_API void syn_b200_decoder_destroy(syn_b200_decoder *decoder);

/* Replaces synapse_gpu_decoder_kv_bytes (ffi.rs:218-232). */
SYN_B200_API uint64_t syn_b200_decoder_kv_bytes(const syn_b200_decoder *decoder);

/* Number of bounded device-side waits that gave up since the last reset (0 in a healthy run). A kernel whose
 * wait on one of its own asynchronous copies runs out of patience records it here and still terminates; the
 * results of that launch are then undefined. No counterpart in the reference. */
SYN_B200_API uint32_t syn_b200_device_faults(uint32_t reset);

/* Number of kernel launches the library has queued from the calling thread since the last reset
 * (benchmark bookkeeping). Passing a non-zero `reset` clears the counter after reading it. */
SYN_B200_API uint64_t syn_b200_launch_count(uint32_t reset);

#ifdef __cplusplus
}
#endif
#endif /* SYNAPSE_B200_H */
