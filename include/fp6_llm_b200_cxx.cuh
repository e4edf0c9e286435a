// C++ interface with the reference's names and signatures (fp6_llm/csrc/fp6_linear.cuh:8-43), so code
// written against the reference's libfp6.so (e.g. its tests/cpp) links against libfp6_b200.so unchanged.
// Differences in behaviour: shape/format violations return cudaErrorInvalidValue (the GEMM) or are
// reported on stderr and leave the output untouched (the void functions) instead of assert/exit; the
// prepacking and dequantisation run on the GPU and return after a synchronise.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

cudaError_t fp6_linear_kernel(cudaStream_t stream, const uint4* Weight, const half* Scales, const half* B, half* C,
                              const size_t M_Global, const size_t N_Global, const size_t K_Global,
                              float* Reduction_Workspace, int Split_K);

cudaError_t fp_eXmY_linear_kernel(const int EXPONENT, const int MANTISSA, cudaStream_t stream, const uint4* Weight,
                                  const half* Scales, const half* B, half* C, const size_t M_Global,
                                  const size_t N_Global, const size_t K_Global, float* Reduction_Workspace,
                                  int Split_K);

void weight_matrix_prepacking(int* packed_weights, int* FP6Weights, size_t M, size_t K);
void weight_matrix_prepacking_fp_eXmY(const int EXPONENT, const int MANTISSA, int* packed_weights, int* FPxWeights,
                                      size_t M, size_t K);

void DeQuantMatrix_FP6_To_FP16(half* A_16bit_h, unsigned char* A_6bit_h, size_t M, size_t K, half* scale);
void dequant_matrix_fp_eXmY_to_fp16(const int EXPONENT, const int MANTISSA, half* A_16bit_h, unsigned char* A_6bit_h,
                                    size_t M, size_t K, half* scale);
