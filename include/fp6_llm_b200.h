/*
 * C interface of libfp6_b200.so: the FPx (FP6 e3m2 / FP5 e2m2) x FP16 linear layer for NVIDIA B200.
 *
 * Every entry point takes plain pointers and sizes and returns a cudaError_t value as int
 * (0 = success); nothing here allocates on behalf of the caller except the *_host helpers, which
 * stage through a private, grow-only device buffer.  Each declaration names the function of the
 * reference project (usyd-fsalab/fp6_llm, paths relative to its tree) that it stands in for.
 *
 * Matrix convention (same as the reference): M = output channels (rows of the weight matrix),
 * K = input channels, N = tokens.  Out[N][M] (fp16, row-major) = Act[N][K] * dequant(W)[M][K]^T.
 * Constraints (same as the reference, fp6_llm/csrc/fp6_linear.cu:56-58): M % 256 == 0,
 * K % 64 == 0, N > 0, (e_bits, m_bits) in {(3,2), (2,2)}.
 * Packed weights are the reference's layout, int32 [M][K/32*(1+e_bits+m_bits)] viewed as one flat
 * buffer [1-bit region][2-bit region][4-bit region]
 * (fp6_llm/csrc/utils/weight_prepacking.h:126-133).
 */
#ifndef FP6_LLM_B200_H_
#define FP6_LLM_B200_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Library interface version (bumped on any signature change). */
int fp6b200_version(void);

/* Text for a code returned by any function below. */
const char* fp6b200_error_string(int code);

/*
 * The linear layer on device buffers, asynchronous on `stream` (a cudaStream_t).
 * Stands in for fp_eXmY_linear_kernel (fp6_llm/csrc/fp6_linear.cuh:20-32; with e_bits=3, m_bits=2
 * also for fp6_linear_kernel, :8-18).  `workspace` holds split_k*M*N floats and is only touched
 * when split_k > 1.  split_k == 0 lets the library decompose the work itself (whole waves of output tiles,
 * then the K blocks of the remaining tiles dealt out evenly over the SMs and summed by a fix-up kernel);
 * size the workspace with fp6b200_workspace_bytes(M, N, K, 0) in that case.
 * Unsupported shapes/formats return cudaErrorInvalidValue instead of asserting or exiting.
 */
int fp6b200_linear(int e_bits, int m_bits, void* stream, const void* weight_packed, const void* scales,
                   const void* act, void* out, size_t M, size_t N, size_t K, float* workspace, int split_k);

/*
 * The layer with a fused epilogue (no counterpart in the reference, whose epilogue only converts and stores:
 * fp6_llm/csrc/include/utils_core.cuh:105-130, kernel_matmul.cuh:183-190; inference engines add bias and the MLP's gating
 * in separate kernels).  Between the fp32 accumulator (times the row scale) and the fp16 store:
 *   bias        fp16 [M] device pointer, added in fp32, or NULL;
 *   activation  FP6B200_ACT_NONE, or FP6B200_ACT_SILU_MUL: the weight rows come in pairs, row 2c = gate channel c and
 *               row 2c+1 = up channel c (scales and bias in the same order), and the output is out[N][M/2] with
 *               out[n][c] = silu(gate) * up - the gate+up projection of a LLaMA MLP in one launch.
 * Everything else as fp6b200_linear.
 */
#define FP6B200_ACT_NONE 0
#define FP6B200_ACT_SILU_MUL 1
int fp6b200_linear_ex(int e_bits, int m_bits, void* stream, const void* weight_packed, const void* scales, const void* act,
                      void* out, size_t M, size_t N, size_t K, float* workspace, int split_k, const void* bias, int activation);

/*
 * The layer on the tensor cores' own six-bit inputs, for batches of up to 64 tokens (no
 * counterpart in the reference, whose kernel - like fp6b200_linear - rebuilds an fp16 pattern of every weight with integer
 * instructions before the MMA: fp6_llm/csrc/include/utils_parallel_dequant.cuh:24-63).  sm_100's tensor cores multiply
 * e3m2 / e2m3 operands directly, and a tensor copy expands densely packed 6-bit codes on the way into shared memory, so
 * no thread touches a weight and the layer streams its weights near the memory roofline.  The activations go in as four
 * exact e5m2 planes (x = p0 + p1/4 + p2/32 + p3/256, written by a small kernel inside the call); every product is exact
 * and accumulated in fp32, as in fp6b200_linear.
 * Formats: e3m2 and e2m3 as they are; e2m2, e3m1 and e2m1 are widened to the six-bit format with the same exponent
 * field when the weights are re-laid (exact: their values are a subset), so every format occupies 6 bits per weight here.
 *   fp6b200_native_supported       1 if format and shape (M % 256 == 0, K % 64 == 0, 1 <= N <= 64) are taken;
 *   fp6b200_native_weight_bytes    bytes of the re-laid weights (tiles of 128 rows x 128 K, 12 KB each);
 *   fp6b200_native_repack          once per weight tensor: prepacked weights (the output of fp6b200_prepack, i.e. of the
 *                                  reference's weight_matrix_prepacking) -> the tile layout; device pointers, 16-byte aligned;
 *   fp6b200_native_workspace_bytes scratch one call needs (activation planes + stream-K partials), 256-byte aligned;
 *                                  calls that share a scratch buffer must be ordered on one stream;
 *   fp6b200_linear_native          the layer; arguments as fp6b200_linear_ex, the library's own work decomposition.
 */
int fp6b200_native_supported(int e_bits, int m_bits, size_t M, size_t N, size_t K);
/* 1 where fp6b200_linear_native measured faster than fp6b200_linear (at most 32 tokens): what
 * the module, the sharded layer and the batched host entry use to choose between the two. */
int fp6b200_native_preferred(int e_bits, int m_bits, size_t M, size_t N, size_t K);
size_t fp6b200_native_weight_bytes(size_t M, size_t K);
size_t fp6b200_native_workspace_bytes(size_t N, size_t K);
int fp6b200_native_repack(int e_bits, int m_bits, void* stream, const void* weight_packed, void* weight_native, size_t M,
                          size_t K);
int fp6b200_linear_native(int e_bits, int m_bits, void* stream, const void* weight_native, const void* scales, const void* act,
                          void* out, size_t M, size_t N, size_t K, void* workspace, const void* bias, int activation);
/* fp6b200_linear_gather (below) on the native path: the rank's shard in the tile layout, scratch as fp6b200_linear_native. */
int fp6b200_linear_native_gather(int e_bits, int m_bits, void* stream, const void* weight_native_shard, const void* scales_shard,
                                 const void* act, void* const* out_peers, void* const* flag_peers, void* epoch_counter,
                                 int world, int rank, size_t out_rows, size_t row0, size_t M, size_t N, size_t K,
                                 void* workspace);
/* Kernels one fp6b200_linear_native call launches (0 for an unsupported shape). */
int fp6b200_native_kernel_launches(size_t M, size_t N, size_t K);

/*
 * Same layer with HOST activations and output: copies act to the device, runs the layer, copies the
 * result back and synchronises.  Weights and scales stay resident on the device (they are parameters).
 * Stands in for the torch-level call fp_eXmY_linear_forward_cuda (fp6_llm/csrc/fp6_linear.cu:269-313)
 * when the caller's tensors live in host memory.
 */
int fp6b200_linear_host_io(int e_bits, int m_bits, const void* weight_packed_dev, const void* scales_dev,
                           const void* act_host, void* out_host, size_t M, size_t N, size_t K, int split_k);

/*
 * Several such layers as ONE pipelined batch: the activations of call i+1 are copied to the device and the result of
 * call i-1 is copied back while call i computes (three internal streams chained by events, one copy per buffer, one
 * synchronisation at the end; the calls compute in array order).  Host buffers should be pinned, or the copies do not
 * overlap.  Stands in for a sequence of fp_eXmY_linear_forward_cuda calls (fp6_llm/csrc/fp6_linear.cu:269-313) made
 * on host tensors; the reference has no batched form.  Returns the first error; no call's output is valid then.
 */
typedef struct fp6b200_host_call {
    int e_bits, m_bits;
    const void* weight_packed_dev;
    const void* scales_dev;
    const void* act_host;   /* fp16 [N][K] */
    void* out_host;         /* fp16 [N][M] */
    size_t M, N, K;
    int split_k;            /* as for fp6b200_linear; 0 = library decomposition */
    const void* weight_native_dev;   /* NULL, or the same weights in the layout of fp6b200_native_repack: calls with
                                        split_k == 0 for which fp6b200_native_preferred says so then run on
                                        fp6b200_linear_native */
} fp6b200_host_call;
int fp6b200_linear_host_io_batch(const fp6b200_host_call* calls, int n_calls);

/* Bytes of split-K workspace fp6b200_linear needs (split_k == 0: for the library's own choice). */
size_t fp6b200_workspace_bytes(size_t M, size_t N, size_t K, int split_k);

/* Number of kernels fp6b200_linear launches for this shape on the current device: the GEMM, plus the split-K reduction
 * or the fix-up of split tiles when the decomposition needs one (no counterpart in the reference; used to count launches). */
int fp6b200_kernel_launches(size_t M, size_t N, size_t K, int split_k);

/*
 * Split count for callers that keep the reference's explicit split-K scheme: the best split_k >= 1 for this
 * kernel on a GPU with `num_sms` SMs (148 on B200), given its 128-row tiles, one CTA per SM and the K blocks
 * available.  The reference's own heuristic (HeuristicFuntion_SplitK, fp6_llm/__init__.py:13-23) is kept
 * separately, unchanged, in Python.  Passing split_k = 0 to fp6b200_linear is usually faster than either.
 */
int fp6b200_choose_split_k(size_t M, size_t N, size_t K, int num_sms);

/*
 * fp16 weights [M][K] and fp16 row scales -> prepacked FPx weights in one pass on the device (the step before
 * prepacking when a checkpoint is loaded).  The reference has no working counterpart: its quantiser
 * (fp6_llm/csrc/utils/weight_quant.h:9-104) truncates and is not bound to Python; the output layout is the packer's
 * (fp6_llm/csrc/utils/weight_prepacking.h:118-196).  A weight becomes the code whose magnitude is nearest to
 * |w / scale| (fp32 division), ties to the even code, saturating at the largest magnitude, sign of the quotient.
 * Needs M % 64 == 0 and K % 64 == 0.
 */
int fp6b200_quantize_prepack(int e_bits, int m_bits, void* stream, const void* weights_fp16_dev, const void* scales_dev,
                             void* packed_dev, size_t M, size_t K);

/*
 * Weight prepacking on device buffers (in != out), asynchronous on `stream`.
 * GPU counterpart of weight_matrix_prepacking_fp_eXmY (fp6_llm/csrc/utils/weight_prepacking.h:204-211);
 * the output is bit-identical.  Needs M % 64 == 0 and K % 64 == 0 (:121-122).
 */
int fp6b200_prepack(int e_bits, int m_bits, void* stream, const void* unpacked_dev, void* packed_dev, size_t M,
                    size_t K);

/*
 * Same with host buffers (in == out allowed), synchronous.  Drop-in for
 * weight_matrix_prepacking_fp_eXmY(E, M, packed, unpacked, M, K) and weight_matrix_prepacking
 * (fp6_llm/csrc/fp6_linear.cuh:37-38).
 */
int fp6b200_prepack_host(int e_bits, int m_bits, int* packed_host, const int* unpacked_host, size_t M, size_t K);

/*
 * UNPACKED weights + per-row fp16 scales -> fp16 [M][K], device buffers.
 * GPU counterpart of dequant_matrix_fp_eXmY_to_fp16 (fp6_llm/csrc/utils/weight_dequant.h:54-61); bit-identical.
 */
int fp6b200_dequant(int e_bits, int m_bits, void* stream, const void* unpacked_dev, const void* scales_dev,
                    void* out_dev, size_t M, size_t K);

/* Same with host buffers, synchronous.  Drop-in for dequant_matrix_fp_eXmY_to_fp16 and
 * DeQuantMatrix_FP6_To_FP16 (fp6_llm/csrc/fp6_linear.cuh:42-43). */
int fp6b200_dequant_host(int e_bits, int m_bits, void* out_host, const void* unpacked_host, size_t M, size_t K,
                         const void* scales_host);

/*
 * PREPACKED weights + scales -> fp16 [M][K], device buffers: what the GEMM multiplies by, element for
 * element.  The reference has no such function; its GPU dequantiser is fused in the GEMM
 * (fp6_llm/csrc/include/utils_parallel_dequant.cuh:44-99), which is the code this mirrors.
 */
int fp6b200_dequant_packed(int e_bits, int m_bits, void* stream, const void* packed_dev, const void* scales_dev,
                           void* out_dev, size_t M, size_t K);

/* out[i] = rn_half(sum_s partials[s*elems + i]), ascending s, fp32.  Stands in for SplitK_Reduction
 * (fp6_llm/csrc/include/kernel_reduction.cuh:28-47).  elems % 4 == 0. */
int fp6b200_splitk_reduce(void* stream, void* out_dev, const float* partials_dev, size_t elems, int split_k);

/*
 * The linear layer for callers that cannot allocate and cannot pass a workspace (no counterpart in the reference,
 * whose torch wrapper allocates a workspace on every call).  Same arguments and result as fp6b200_linear with
 * split_k = 0, but the fp32 scratch is a fixed array of fp6b200_static_scratch_bytes() bytes inside the library:
 * every GPU that loads the library holds it until the process exits.  Returns cudaErrorInvalidValue (and says why on
 * stderr) when fp6b200_workspace_bytes(M, N, K, 0) exceeds that size (batch sizes above 64 on a 148-SM GPU).
 * Makes no cudaMalloc/cudaFree or other allocating call.  The first call on a device looks the array's address up
 * (cudaGetSymbolAddress), and with lazy module loading (the CUDA default) that first touch is also when the driver
 * places the library's device code and this array in device memory: a host that hands all free memory to its own pool
 * must make one call (any supported shape) - or otherwise force the module to load - BEFORE it reserves the rest.
 * All calls on a device share the array: calls whose kernels can overlap on the GPU race; order them on one stream.
 */
int fp6b200_linear_static_scratch(int e_bits, int m_bits, void* stream, const void* weight_packed, const void* scales,
                                  const void* act, void* out, size_t M, size_t N, size_t K);

/* Size in bytes of the built-in scratch array used by fp6b200_linear_static_scratch. */
size_t fp6b200_static_scratch_bytes(void);

/*
 * One rank's part of an OC-sharded linear layer with the exchange fused in (no counterpart in the reference, which
 * is single-GPU: fp6_llm/csrc/fp6_linear.cu:104-139 computes the whole layer on one device).  This rank holds the
 * packed shard of M output channels (rows row0 .. row0 + M of the layer's out_rows channels) and the matching scales;
 * act is the full [N][K] activation.  The kernel stores its [N][M] result straight into rows row0.. of EVERY rank's
 * output buffer [N][out_rows] (out_peers[r] = rank r's buffer as mapped into this process, peer-to-peer over
 * NVLink; out_peers[rank] is the local one), then tells every peer that its rows are there and waits for theirs:
 * flag_peers[r] = rank r's array of `world` 32-bit words, zeroed once before the first call; epoch_counter = a 32-bit
 * word in this rank's own memory, zeroed once, advanced by each call on the device.  When the call has completed on
 * the stream, out_peers[rank] holds the whole [N][out_rows] result.  Every rank must make the same sequence of calls.
 * A rank may be one call ahead of a peer, so successive calls must alternate between two output buffers.
 * split_k: 0 (library decomposition) or 1.  workspace as for fp6b200_linear.  A peer that does not arrive within two
 * seconds ends the wait; fp6b200_device_status then reports code 10 and the output is incomplete.
 */
int fp6b200_linear_gather(int e_bits, int m_bits, void* stream, const void* weight_shard, const void* scales_shard,
                          const void* act, void* const* out_peers, void* const* flag_peers, void* epoch_counter, int world,
                          int rank, size_t out_rows, size_t row0, size_t M, size_t N, size_t K, float* workspace,
                          int split_k);

/*
 * Process-wide options (no counterpart in the reference).
 * FP6B200_OPTION_STATIC_WEIGHTS (default 0): set to 1 to promise that no packed-weight buffer handed to fp6b200_linear*
 * is written by work that is still in flight on the same stream when the call is made (weights prepacked at load time
 * and then only read).  The GEMM is launched programmatically: its CTAs start while the previous kernel of the stream
 * is finishing, and with this option they already request the first weight stages and unpack them then; activations,
 * scales, outputs and workspace are touched only after the previous kernel has completed, option or not.
 * With the option on, a prepack (or any write of the weights) must be followed by a synchronisation or an event wait
 * before the first GEMM that reads them.  fp6b200_set_option returns cudaErrorInvalidValue for an unknown option;
 * fp6b200_get_option returns the value, or -1.
 * FP6B200_OPTION_PROGRAMMATIC_LAUNCH (default 1): the GEMM is launched with programmatic stream serialisation, so that
 * it starts and sets itself up while the previous kernel of the stream is finishing (it still waits for that kernel
 * to complete before it touches memory the kernel may have written).  0 restores plain stream order between a GEMM
 * and whatever precedes it.
 * FP6B200_OPTION_PAIR_TILES (default 0): layers of more than 128 tokens run as pairs of CTAs on neighbouring SMs that share
 * one 256-row tile and each load half of its activation tile (tcgen05 cta_group::2); 1 = when the layer has a tile for
 * every pair, 2 = always.  Same results; off by default because it measured slower than one CTA per tile.
 */
#define FP6B200_OPTION_STATIC_WEIGHTS 1
#define FP6B200_OPTION_PROGRAMMATIC_LAUNCH 2
#define FP6B200_OPTION_PAIR_TILES 3
int fp6b200_set_option(int option, int value);
int fp6b200_get_option(int option);

/*
 * Synchronises the current device, returns in *code the first time-out code a GEMM CTA recorded
 * since the last call (0 = none) and clears it.  A non-zero code means a bounded wait inside the
 * kernel gave up and the output of that launch is invalid.
 */
int fp6b200_device_status(int* code);

#ifdef __cplusplus
}
#endif
#endif /* FP6_LLM_B200_H_ */
