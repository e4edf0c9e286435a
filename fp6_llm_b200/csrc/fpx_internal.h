// Declarations shared by the translation units of the library (not part of the public interface).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace fpx {

// Only e3m2 (FP6) and e2m2 (FP5) exist in the reference (fp6_llm/csrc/fp6_linear.cu:133-138).
inline bool format_supported(int e_bits, int m_bits) { return m_bits == 2 && (e_bits == 3 || e_bits == 2); }

// GEMM (+ split-K reduction when split_k > 1).  All pointers are device pointers.
cudaError_t launch_gemm(int e_bits, int m_bits, cudaStream_t stream, const void* weight, const __half* scales,
                        const __half* act, __half* out, size_t M, size_t N, size_t K, float* workspace, int split_k,
                        int* status);
cudaError_t launch_splitk_reduce(cudaStream_t stream, __half* out, const float* partials, size_t elems, int split_k,
                                 bool after_gemm = false);
int gemm_n_tile(size_t N);
int device_sm_count();
// Workspace the GEMM needs when it picks its own decomposition (split_k == 0).
size_t gemm_auto_workspace_bytes(size_t N);

// Device address (current device) of the word in which a GEMM CTA records a time-out; nullptr on failure.
int* gemm_status_word();

// Weight format kernels.  All pointers are device pointers; in != out.
cudaError_t launch_prepack(int e_bits, int m_bits, cudaStream_t stream, const void* unpacked, void* packed, size_t M,
                           size_t K);
cudaError_t launch_dequant_unpacked(int e_bits, int m_bits, cudaStream_t stream, const void* unpacked,
                                    const __half* scales, __half* out, size_t M, size_t K);
cudaError_t launch_dequant_packed(int e_bits, int m_bits, cudaStream_t stream, const void* packed,
                                  const __half* scales, __half* out, size_t M, size_t K);

}  // namespace fpx
