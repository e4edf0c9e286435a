// fp6b200_linear_static_scratch: the linear layer for callers that can neither hand over a workspace nor let the
// library allocate one.
//
// Who that is: a serving process that reserves all device memory for its own pools at start-up (a cudaMalloc made
// later simply fails), or a
// component whose memory budget is fixed by contract and audited.  Such callers still pass inputs and the output
// buffer; what they cannot provide is the fp32 scratch the kernel uses when it deals the K range of a tile out over
// several SMs.  Here that scratch is a fixed array inside the library image.
//
// Cost and limits: every GPU that loads the library carries kScratchBytes of device memory until the process exits,
// used or not.  Problems whose scratch need (fp6b200_workspace_bytes(M, N, K, 0)) is larger are refused.  All calls
// on one device share the one array, so two calls whose kernels may overlap on the GPU (different streams, no
// ordering between them) corrupt each other; order them on one stream or with events.  The array keeps whatever the
// previous call left in it; the kernel never reads a slot it has not written in the same launch, so nothing has to be
// cleared between calls.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdio.h>

#include <mutex>

#include "../../include/fp6_llm_b200.h"
#include "fpx_internal.h"

namespace {

constexpr size_t kScratchBytes = 10u << 20;   // 10 MiB: covers batch sizes up to 64 on a 148-SM GPU

// The name below is only a handle on the host side.  It must never be passed to a kernel as a pointer: the device
// address is obtained once per device with cudaGetSymbolAddress (see scratch_for_current_device).
static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;

// Device address of the scratch array on the CURRENT device, resolved on the first call for that device.
cudaError_t scratch_for_current_device(float** out) {
    static float* ptrs[kMaxDevices] = {};
    static std::mutex mu;
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(mu);
    if (!ptrs[dev]) {
        void* p = nullptr;
        err = cudaGetSymbolAddress(&p, g_static_scratch);
        if (err != cudaSuccess) return err;
        ptrs[dev] = static_cast<float*>(p);
    }
    *out = ptrs[dev];
    return cudaSuccess;
}

}  // namespace

extern "C" {

size_t fp6b200_static_scratch_bytes(void) { return kScratchBytes; }

int fp6b200_linear_static_scratch(int e_bits, int m_bits, void* stream, const void* weight_packed, const void* scales,
                                  const void* act, void* out, size_t M, size_t N, size_t K) {
    const size_t need = fp6b200_workspace_bytes(M, N, K, 0);
    if (need > kScratchBytes) {
        fprintf(stderr,
                "fp6b200_linear_static_scratch: M=%zu N=%zu K=%zu needs %zu bytes of scratch, the built-in array holds "
                "%zu; use fp6b200_linear with a caller-owned workspace\n",
                M, N, K, need, kScratchBytes);
        return cudaErrorInvalidValue;
    }
    float* scratch = nullptr;
    cudaError_t err = scratch_for_current_device(&scratch);
    if (err != cudaSuccess) return err;
    int* status = fpx::gemm_status_word();
    if (!status) return cudaErrorInitializationError;
    // split_k = 0: the library's own decomposition, the one the scratch is sized for
    return fpx::launch_gemm(e_bits, m_bits, static_cast<cudaStream_t>(stream), weight_packed,
                            static_cast<const __half*>(scales), static_cast<const __half*>(act),
                            static_cast<__half*>(out), M, N, K, scratch, 0, status);
}

}  // extern "C"
