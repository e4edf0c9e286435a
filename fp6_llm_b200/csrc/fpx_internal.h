// Declarations shared by the translation units of the library (not part of the public interface).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace fpx {

// The reference's launcher knows e3m2 (FP6) and e2m2 (FP5) only (fp6_llm/csrc/fp6_linear.cu:133-138), but its packer and
// dequantiser are templates over any code narrower than 8 bits (fp6_llm/csrc/utils/weight_prepacking.h:118-128,
// fp6_llm/csrc/utils/weight_dequant.h:10-48).  Here: those two plus e2m1 (4-bit), e3m1 (5-bit) and e2m3 (6-bit).
inline bool format_supported(int e_bits, int m_bits) {
    return (m_bits == 2 && (e_bits == 3 || e_bits == 2)) || (m_bits == 1 && (e_bits == 2 || e_bits == 3)) || (m_bits == 3 && e_bits == 2);
}
// Runs CALL with the format as the compile-time constants kE and kM.
#define FPX_DISPATCH_FORMAT(e_bits, m_bits, CALL)                                   \
    do {                                                                            \
        if ((e_bits) == 3 && (m_bits) == 2) { constexpr int kE = 3, kM = 2; CALL; }   \
        else if ((e_bits) == 2 && (m_bits) == 2) { constexpr int kE = 2, kM = 2; CALL; } \
        else if ((e_bits) == 2 && (m_bits) == 1) { constexpr int kE = 2, kM = 1; CALL; } \
        else if ((e_bits) == 3 && (m_bits) == 1) { constexpr int kE = 3, kM = 1; CALL; } \
        else { constexpr int kE = 2, kM = 3; CALL; }                                  \
    } while (0)

// Status codes a kernel's bounded wait records in the device status word when it gives up.
enum : int {
    kErrStageEmpty = 1, kErrStageFull = 2, kErrAEmpty = 3, kErrAFull = 6, kErrAccFull = 7, kErrSmemAlign = 8,
    kErrAccEmpty = 9, kErrPeerWait = 10   // 10: a peer GPU did not arrive at the end of a sharded layer
};

// Where the fp16 result goes.  One target with ld == M and row0 == 0 is the plain layer.  Several targets are the
// output buffers [N][ld] of the ranks of an OC-sharded layer (this GPU's and its peers', as mapped into this
// process): the M rows computed here are stored at rows row0 .. row0 + M of every target.
constexpr int kMaxOutTargets = 8;
struct OutTargets {
    __half* ptr[kMaxOutTargets];
    uint32_t count;
    uint32_t ld;
    uint32_t row0;
};

// What happens to an output element between the fp32 accumulator and the fp16 store (after the row scale):
//   bias        per-row fp16 addend [M], or nullptr;
//   activation  kActNone, or kActSiluMul: rows come in pairs (2c = gate, 2c+1 = up) and the layer's output channel c is
//               silu(gate) * up, so the output is [N][M / 2].
enum : int { kActNone = 0, kActSiluMul = 1 };
struct Epilogue {
    const __half* bias;
    int activation;
};

// GEMM (+ split-K reduction when split_k > 1).  All pointers are device pointers.  targets == nullptr: the result
// goes to out[N][M] (out[N][M / 2] with kActSiluMul); otherwise out is ignored (split_k must then be 0 or 1, and no
// activation).  epilogue == nullptr: plain layer.
cudaError_t launch_gemm(int e_bits, int m_bits, cudaStream_t stream, const void* weight, const __half* scales,
                        const __half* act, __half* out, size_t M, size_t N, size_t K, float* workspace, int split_k,
                        int* status, const OutTargets* targets = nullptr, const Epilogue* epilogue = nullptr);
// Work decomposition of one call over `sms` CTAs (see WorkPlan): M rows in 128-row tiles, K in 64-wide blocks;
// split_k == 0 is the library's own (waves of whole tiles, then the K blocks of the remaining tiles dealt out evenly),
// split_k >= 1 the caller's.  Returns the effective split.
struct WorkPlan;
int make_plan(size_t M, size_t n_tiles, size_t K, int split_k, int sms, WorkPlan* out);
// tile_rows: height of the plan's row tiles (128, or 256 when CTA pairs computed them)
cudaError_t launch_streamk_fixup(cudaStream_t stream, const OutTargets& where, const float* workspace, size_t N,
                                 int n_tile, const WorkPlan& plan, const Epilogue* epilogue, int tile_rows = 128);
// Cross-GPU arrival barrier that ends a sharded layer: tells every peer that this rank's stores into its output
// buffer are complete and waits (bounded) for the same word from every peer.  flag_peers[r] = rank r's flag array
// (one 32-bit word per rank) as mapped here; epoch_counter = this rank's own call counter in device memory.
cudaError_t launch_gather_barrier(cudaStream_t stream, uint32_t* const* flag_peers, int world, int rank,
                                  uint32_t* epoch_counter, int* status);
// out[n][m] = rn_half(epilogue(sum over splits of partials[s][n][m])); rows = M (needed for the bias and the pairing).
cudaError_t launch_splitk_reduce(cudaStream_t stream, __half* out, const float* partials, size_t elems, int split_k,
                                 bool after_gemm = false, size_t rows = 0, const Epilogue* epilogue = nullptr);
// Process-wide promise that packed weights are never written by work still in flight on the stream of a GEMM that
// reads them; the GEMM then requests them before the previous kernel of its stream has completed.  Off by default.
void set_weights_static(int on);
int weights_static();
// Whether a GEMM may start while the previous kernel of its stream is finishing (programmatic dependent launch) and
// whether the fix-up kernel lets the kernel after it do the same.  On by default.
void set_programmatic_launch(int on);
int programmatic_launch();
// Whether layers of more than 128 tokens run as pairs of CTAs on 256-row tiles (tcgen05 cta_group::2): 0 no (default: it
// measured slower), 1 when the layer has a tile for every pair, 2 always.
void set_pair_tiles(int on);
int pair_tiles();
int gemm_n_tile(size_t N);
// Kernels one GEMM call launches on the current device (0 for an invalid shape).
int gemm_kernel_launches(size_t M, size_t N, size_t K, int split_k);
int device_sm_count();
// Workspace the GEMM needs when it picks its own decomposition (split_k == 0).
size_t gemm_auto_workspace_bytes(size_t N);

// The tensor cores' own six-bit inputs (fpx_native.cu): e3m2 and e2m3 weights re-laid into 128 x 128 tiles that a tensor
// copy expands in flight, activations split into four exact e5m2 planes; batches of up to native_max_tokens() tokens.
bool native_format(int e_bits, int m_bits);
int native_max_tokens();
size_t native_weight_bytes(size_t M, size_t K);
size_t native_workspace_bytes(size_t N, size_t K);
cudaError_t launch_native_repack(int e_bits, int m_bits, cudaStream_t stream, const void* packed, void* native, size_t M,
                                 size_t K);
// workspace: native_workspace_bytes(N, K) bytes, 256-byte aligned (activation planes, then the stream-K slots)
cudaError_t launch_native_gemm(int e_bits, int m_bits, cudaStream_t stream, const void* weight_native, const __half* scales,
                               const __half* act, __half* out, size_t M, size_t N, size_t K, void* workspace, int* status,
                               const OutTargets* targets = nullptr, const Epilogue* epilogue = nullptr);
int native_kernel_launches(size_t M, size_t N, size_t K);

// Device address (current device) of the word in which a GEMM CTA records a time-out; nullptr on failure.
int* gemm_status_word();

// Weight format kernels.  All pointers are device pointers; in != out.
cudaError_t launch_prepack(int e_bits, int m_bits, cudaStream_t stream, const void* unpacked, void* packed, size_t M,
                           size_t K);
// fp16 weights [M][K] + fp16 row scales -> prepacked FPx (round to nearest, ties to the even code, saturating).
cudaError_t launch_quantize_prepack(int e_bits, int m_bits, cudaStream_t stream, const __half* weights,
                                    const __half* scales, void* packed, size_t M, size_t K);
cudaError_t launch_dequant_unpacked(int e_bits, int m_bits, cudaStream_t stream, const void* unpacked,
                                    const __half* scales, __half* out, size_t M, size_t K);
cudaError_t launch_dequant_packed(int e_bits, int m_bits, cudaStream_t stream, const void* packed,
                                  const __half* scales, __half* out, size_t M, size_t K);

}  // namespace fpx
