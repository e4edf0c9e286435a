// TEST / BENCHMARK INFRASTRUCTURE ONLY.  C-linkage wrapper around the reference's own GPU launcher
// (fp6_llm/csrc/fp6_linear.cuh:20-32, fp_eXmY_linear_kernel), compiled together with the reference's fp6_linear.cu from
// the sources where they lie (see oracle/Makefile, target refgpu; built with -DNO_PYTORCH as the reference's own
// Makefile builds libfp6.so, fp6_llm/Makefile:15).  The reference ships this kernel for sm_80 (mma.sync, ldmatrix,
// cp.async); recompiled for sm_100a it is the same-box GPU comparison of the benchmark, never a parity oracle and
// never part of the library.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include "fp6_linear.cuh"

extern "C" int ref_gpu_linear(int e_bits, int m_bits, void* stream, const void* weight, const void* scales, const void* act,
                              void* out, size_t M, size_t N, size_t K, float* workspace, int split_k) {
    return (int)fp_eXmY_linear_kernel(e_bits, m_bits, static_cast<cudaStream_t>(stream), static_cast<const uint4*>(weight),
                                      static_cast<const half*>(scales), static_cast<const half*>(act), static_cast<half*>(out),
                                      M, N, K, workspace, split_k);
}
