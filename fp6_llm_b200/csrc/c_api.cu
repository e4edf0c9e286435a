// C interface (include/fp6_llm_b200.h) and the C++ interface with the reference's names
// (include/fp6_llm_b200_cxx.cuh) of libfp6_b200.so.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include <mutex>

#include "../../include/fp6_llm_b200.h"
#include "../../include/fp6_llm_b200_cxx.cuh"
#include "fpx_internal.h"

namespace {

// First time-out code recorded by a GEMM CTA (0 = none); one word per device that loads the library.
__device__ int g_gemm_status = 0;

constexpr int kMaxDevices = 64;

int* status_ptr() {
    static int* ptrs[kMaxDevices] = {};
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!ptrs[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_gemm_status) != cudaSuccess) return nullptr;
        ptrs[dev] = static_cast<int*>(p);
    }
    return ptrs[dev];
}

// Grow-only device staging buffer for the *_host entry points (one per device, calls are serialised).
struct Staging {
    std::mutex mu;
    void* buf[kMaxDevices] = {};
    size_t cap[kMaxDevices] = {};
    cudaStream_t stream[kMaxDevices] = {};
};
Staging& staging() {
    static Staging s;
    return s;
}
cudaError_t staging_get(size_t bytes, void** out, cudaStream_t* stream) {
    Staging& s = staging();
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    if (!s.stream[dev]) {
        err = cudaStreamCreateWithFlags(&s.stream[dev], cudaStreamNonBlocking);
        if (err != cudaSuccess) return err;
    }
    if (s.cap[dev] < bytes) {
        if (s.buf[dev]) cudaFree(s.buf[dev]);
        s.buf[dev] = nullptr;
        s.cap[dev] = 0;
        const size_t want = bytes + bytes / 4;
        err = cudaMalloc(&s.buf[dev], want);
        if (err != cudaSuccess) return err;
        s.cap[dev] = want;
    }
    *out = s.buf[dev];
    *stream = s.stream[dev];
    return cudaSuccess;
}
inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Split count for callers that want the reference's explicit split-K scheme on this kernel: one CTA per SM,
// 128-row tiles, items = tiles * split dealt round-robin.  Picks the split that minimises
// ceil(items / SMs) * (K blocks per item + fixed cost per item), preferring small splits on ties.
int choose_split_k(size_t M, size_t N, size_t K, int num_sms) {
    if (M == 0 || N == 0 || K < 64 || num_sms <= 0) return 1;
    const int n_tile = fpx::gemm_n_tile(N);
    const double tiles = (double)(M / 128) * (double)((N + n_tile - 1) / n_tile);
    const size_t kblocks = K / 64;
    const double item_overhead = 6.0;    // pipeline fill + epilogue, in K-block units
    int best = 1;
    double best_cost = 1e300;
    const size_t max_split = kblocks < 32 ? kblocks : 32;
    for (size_t k = 1; k <= max_split; k++) {
        const double rounds = ceil(tiles * (double)k / (double)num_sms);
        const double cost = rounds * (ceil((double)kblocks / (double)k) + item_overhead) + (k > 1 ? 8.0 : 0.0);
        if (cost < best_cost * 0.97) {
            best_cost = cost;
            best = (int)k;
        }
    }
    return best;
}

}  // namespace

namespace fpx {
int* gemm_status_word() { return status_ptr(); }
}  // namespace fpx

extern "C" {

int fp6b200_version(void) { return 2; }

const char* fp6b200_error_string(int code) { return cudaGetErrorString(static_cast<cudaError_t>(code)); }

int fp6b200_set_option(int option, int value) {
    if (option == FP6B200_OPTION_STATIC_WEIGHTS) fpx::set_weights_static(value);
    else if (option == FP6B200_OPTION_PROGRAMMATIC_LAUNCH) fpx::set_programmatic_launch(value);
    else if (option == FP6B200_OPTION_PAIR_TILES) fpx::set_pair_tiles(value);
    else return cudaErrorInvalidValue;
    return cudaSuccess;
}

int fp6b200_get_option(int option) {
    if (option == FP6B200_OPTION_STATIC_WEIGHTS) return fpx::weights_static();
    if (option == FP6B200_OPTION_PROGRAMMATIC_LAUNCH) return fpx::programmatic_launch();
    if (option == FP6B200_OPTION_PAIR_TILES) return fpx::pair_tiles();
    return -1;
}

int fp6b200_choose_split_k(size_t M, size_t N, size_t K, int num_sms) { return choose_split_k(M, N, K, num_sms); }

size_t fp6b200_workspace_bytes(size_t M, size_t N, size_t K, int split_k) {
    (void)K;
    if (split_k == 0) return fpx::gemm_auto_workspace_bytes(N);
    return split_k > 1 ? (size_t)split_k * M * N * sizeof(float) : 0;
}

int fp6b200_kernel_launches(size_t M, size_t N, size_t K, int split_k) { return fpx::gemm_kernel_launches(M, N, K, split_k); }

int fp6b200_linear(int e_bits, int m_bits, void* stream, const void* weight_packed, const void* scales,
                   const void* act, void* out, size_t M, size_t N, size_t K, float* workspace, int split_k) {
    int* status = status_ptr();
    if (!status) return cudaErrorInitializationError;
    return fpx::launch_gemm(e_bits, m_bits, static_cast<cudaStream_t>(stream), weight_packed,
                            static_cast<const __half*>(scales), static_cast<const __half*>(act),
                            static_cast<__half*>(out), M, N, K, workspace, split_k, status);
}

int fp6b200_linear_ex(int e_bits, int m_bits, void* stream, const void* weight_packed, const void* scales, const void* act,
                      void* out, size_t M, size_t N, size_t K, float* workspace, int split_k, const void* bias, int activation) {
    int* status = status_ptr();
    if (!status) return cudaErrorInitializationError;
    fpx::Epilogue epi;
    epi.bias = static_cast<const __half*>(bias);
    epi.activation = activation;
    return fpx::launch_gemm(e_bits, m_bits, static_cast<cudaStream_t>(stream), weight_packed,
                            static_cast<const __half*>(scales), static_cast<const __half*>(act),
                            static_cast<__half*>(out), M, N, K, workspace, split_k, status, nullptr, &epi);
}

int fp6b200_native_supported(int e_bits, int m_bits, size_t M, size_t N, size_t K) {
    return fpx::native_format(e_bits, m_bits) && M > 0 && M % 256 == 0 && K > 0 && K % 64 == 0 && N > 0 &&
           N <= (size_t)fpx::native_max_tokens();
}

int fp6b200_native_preferred(int e_bits, int m_bits, size_t M, size_t N, size_t K) {
    // measured on the LLaMA-2 7B / 13B / 70B layer sets: up to 32 tokens the tensor-core path makes the step faster (a rule
    // that kept layers of 4096 output channels on the other kernel from 5 tokens on, as their isolated timings suggested,
    // made the 7B step 4 % slower); from 33 tokens on four activation planes at the 8-bit rate cost more than unpacking
    return fp6b200_native_supported(e_bits, m_bits, M, N, K) && N <= 32;
}

size_t fp6b200_native_weight_bytes(size_t M, size_t K) { return fpx::native_weight_bytes(M, K); }

size_t fp6b200_native_workspace_bytes(size_t N, size_t K) { return fpx::native_workspace_bytes(N, K); }

int fp6b200_native_repack(int e_bits, int m_bits, void* stream, const void* weight_packed, void* weight_native, size_t M,
                          size_t K) {
    return fpx::launch_native_repack(e_bits, m_bits, static_cast<cudaStream_t>(stream), weight_packed, weight_native, M, K);
}

int fp6b200_linear_native(int e_bits, int m_bits, void* stream, const void* weight_native, const void* scales, const void* act,
                          void* out, size_t M, size_t N, size_t K, void* workspace, const void* bias, int activation) {
    int* status = status_ptr();
    if (!status) return cudaErrorInitializationError;
    fpx::Epilogue epi;
    epi.bias = static_cast<const __half*>(bias);
    epi.activation = activation;
    return fpx::launch_native_gemm(e_bits, m_bits, static_cast<cudaStream_t>(stream), weight_native,
                                   static_cast<const __half*>(scales), static_cast<const __half*>(act),
                                   static_cast<__half*>(out), M, N, K, workspace, status, nullptr, &epi);
}

int fp6b200_linear_native_gather(int e_bits, int m_bits, void* stream, const void* weight_native_shard, const void* scales_shard,
                                 const void* act, void* const* out_peers, void* const* flag_peers, void* epoch_counter,
                                 int world, int rank, size_t out_rows, size_t row0, size_t M, size_t N, size_t K,
                                 void* workspace) {
    int* status = status_ptr();
    if (!status) return cudaErrorInitializationError;
    if (!out_peers || !flag_peers || world < 1 || world > fpx::kMaxOutTargets || rank < 0 || rank >= world)
        return cudaErrorInvalidValue;
    if (out_rows > 0x7fffffffull || row0 > 0x7fffffffull || row0 + M > out_rows || out_rows % 4 != 0 || row0 % 4 != 0)
        return cudaErrorInvalidValue;
    fpx::OutTargets targets = {};
    uint32_t* flags[fpx::kMaxOutTargets] = {};
    for (int r = 0; r < world; r++) {
        targets.ptr[r] = static_cast<__half*>(out_peers[r]);
        flags[r] = static_cast<uint32_t*>(flag_peers[r]);
    }
    targets.count = (uint32_t)world;
    targets.ld = (uint32_t)out_rows;
    targets.row0 = (uint32_t)row0;
    cudaError_t err = fpx::launch_native_gemm(e_bits, m_bits, static_cast<cudaStream_t>(stream), weight_native_shard,
                                              static_cast<const __half*>(scales_shard), static_cast<const __half*>(act),
                                              nullptr, M, N, K, workspace, status, &targets);
    if (err != cudaSuccess) return err;
    return fpx::launch_gather_barrier(static_cast<cudaStream_t>(stream), flags, world, rank,
                                      static_cast<uint32_t*>(epoch_counter), status);
}

int fp6b200_native_kernel_launches(size_t M, size_t N, size_t K) { return fpx::native_kernel_launches(M, N, K); }

int fp6b200_linear_gather(int e_bits, int m_bits, void* stream, const void* weight_shard, const void* scales_shard,
                          const void* act, void* const* out_peers, void* const* flag_peers, void* epoch_counter, int world,
                          int rank, size_t out_rows, size_t row0, size_t M, size_t N, size_t K, float* workspace,
                          int split_k) {
    int* status = status_ptr();
    if (!status) return cudaErrorInitializationError;
    if (!out_peers || !flag_peers || world < 1 || world > fpx::kMaxOutTargets || rank < 0 || rank >= world)
        return cudaErrorInvalidValue;
    if (out_rows > 0x7fffffffull || row0 > 0x7fffffffull || row0 + M > out_rows || out_rows % 4 != 0 || row0 % 4 != 0)
        return cudaErrorInvalidValue;
    if (split_k != 0 && split_k != 1) return cudaErrorInvalidValue;
    fpx::OutTargets targets = {};
    uint32_t* flags[fpx::kMaxOutTargets] = {};
    for (int r = 0; r < world; r++) {
        targets.ptr[r] = static_cast<__half*>(out_peers[r]);
        flags[r] = static_cast<uint32_t*>(flag_peers[r]);
    }
    targets.count = (uint32_t)world;
    targets.ld = (uint32_t)out_rows;
    targets.row0 = (uint32_t)row0;
    cudaError_t err = fpx::launch_gemm(e_bits, m_bits, static_cast<cudaStream_t>(stream), weight_shard,
                                       static_cast<const __half*>(scales_shard), static_cast<const __half*>(act), nullptr,
                                       M, N, K, workspace, split_k, status, &targets);
    if (err != cudaSuccess) return err;
    return fpx::launch_gather_barrier(static_cast<cudaStream_t>(stream), flags, world, rank,
                                      static_cast<uint32_t*>(epoch_counter), status);
}

int fp6b200_linear_host_io(int e_bits, int m_bits, const void* weight_packed_dev, const void* scales_dev,
                           const void* act_host, void* out_host, size_t M, size_t N, size_t K, int split_k) {
    if (!act_host || !out_host || split_k < 0) return cudaErrorInvalidValue;
    const size_t act_bytes = align_up(N * K * sizeof(__half), 256), out_bytes = align_up(N * M * sizeof(__half), 256);
    const size_t ws_bytes = fp6b200_workspace_bytes(M, N, K, split_k);
    std::lock_guard<std::mutex> lock(staging().mu);
    void* base = nullptr;
    cudaStream_t stream = nullptr;
    cudaError_t err = staging_get(act_bytes + out_bytes + ws_bytes, &base, &stream);
    if (err != cudaSuccess) return err;
    char* p = static_cast<char*>(base);
    __half* act = reinterpret_cast<__half*>(p);
    __half* out = reinterpret_cast<__half*>(p + act_bytes);
    float* ws = ws_bytes ? reinterpret_cast<float*>(p + act_bytes + out_bytes) : nullptr;
    err = cudaMemcpyAsync(act, act_host, N * K * sizeof(__half), cudaMemcpyHostToDevice, stream);
    if (err != cudaSuccess) return err;
    int* status = status_ptr();
    if (!status) return cudaErrorInitializationError;
    err = fpx::launch_gemm(e_bits, m_bits, stream, weight_packed_dev, static_cast<const __half*>(scales_dev), act, out,
                           M, N, K, ws, split_k, status);
    if (err != cudaSuccess) return err;
    err = cudaMemcpyAsync(out_host, out, N * M * sizeof(__half), cudaMemcpyDeviceToHost, stream);
    if (err != cudaSuccess) return err;
    return cudaStreamSynchronize(stream);
}

// Several layers with host activations/outputs as one pipelined batch: call i+1's activations travel to the device
// and call i-1's result travels back while call i computes.  Three streams (copy in, compute, copy out) chained by
// events, one cudaMemcpyAsync per copy, one synchronisation at the end.
namespace {
struct BatchContext {
    cudaStream_t in = nullptr, compute = nullptr, out = nullptr;
    cudaEvent_t* events = nullptr;
    int n_events = 0;
};
BatchContext g_batch[kMaxDevices];

cudaError_t batch_context(int n_calls, BatchContext** ctx) {
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    BatchContext& c = g_batch[dev];
    if (!c.in) {
        if ((err = cudaStreamCreateWithFlags(&c.in, cudaStreamNonBlocking)) != cudaSuccess) return err;
        if ((err = cudaStreamCreateWithFlags(&c.compute, cudaStreamNonBlocking)) != cudaSuccess) return err;
        if ((err = cudaStreamCreateWithFlags(&c.out, cudaStreamNonBlocking)) != cudaSuccess) return err;
    }
    if (c.n_events < 2 * n_calls) {
        cudaEvent_t* grown = static_cast<cudaEvent_t*>(realloc(c.events, sizeof(cudaEvent_t) * 2 * (size_t)n_calls));
        if (!grown) return cudaErrorMemoryAllocation;
        c.events = grown;
        for (int i = c.n_events; i < 2 * n_calls; i++) {
            if ((err = cudaEventCreateWithFlags(&c.events[i], cudaEventDisableTiming)) != cudaSuccess) return err;
            c.n_events = i + 1;
        }
    }
    *ctx = &c;
    return cudaSuccess;
}
}  // namespace

// whether a call of a host batch runs on the tensor cores' own six-bit inputs
static bool host_call_native(const fp6b200_host_call& c) {
    return c.weight_native_dev && c.split_k == 0 && fp6b200_native_preferred(c.e_bits, c.m_bits, c.M, c.N, c.K);
}

int fp6b200_linear_host_io_batch(const fp6b200_host_call* calls, int n_calls) {
    if (!calls || n_calls <= 0) return cudaErrorInvalidValue;
    size_t total = 0, ws_bytes = 0;
    for (int i = 0; i < n_calls; i++) {
        const fp6b200_host_call& c = calls[i];
        if (!c.act_host || !c.out_host || !c.weight_packed_dev || !c.scales_dev || c.split_k < 0) return cudaErrorInvalidValue;
        total += align_up(c.N * c.K * sizeof(__half), 256) + align_up(c.N * c.M * sizeof(__half), 256);
        const size_t ws = host_call_native(c) ? fpx::native_workspace_bytes(c.N, c.K) : fp6b200_workspace_bytes(c.M, c.N, c.K, c.split_k);
        ws_bytes = ws > ws_bytes ? ws : ws_bytes;
    }
    std::lock_guard<std::mutex> lock(staging().mu);
    void* base = nullptr;
    cudaStream_t unused = nullptr;
    cudaError_t err = staging_get(total + align_up(ws_bytes, 256), &base, &unused);
    if (err != cudaSuccess) return err;
    BatchContext* ctx = nullptr;
    if ((err = batch_context(n_calls, &ctx)) != cudaSuccess) return err;
    int* status = status_ptr();
    if (!status) return cudaErrorInitializationError;
    char* p = static_cast<char*>(base);
    float* ws = ws_bytes ? reinterpret_cast<float*>(p + total) : nullptr;   // one workspace: the layers run in order on one stream
    for (int i = 0; i < n_calls && err == cudaSuccess; i++) {
        const fp6b200_host_call& c = calls[i];
        const size_t act_bytes = c.N * c.K * sizeof(__half), out_bytes = c.N * c.M * sizeof(__half);
        __half* act = reinterpret_cast<__half*>(p);
        __half* out = reinterpret_cast<__half*>(p + align_up(act_bytes, 256));
        p += align_up(act_bytes, 256) + align_up(out_bytes, 256);
        cudaEvent_t landed = ctx->events[2 * i], done = ctx->events[2 * i + 1];
        if ((err = cudaMemcpyAsync(act, c.act_host, act_bytes, cudaMemcpyHostToDevice, ctx->in)) != cudaSuccess) break;
        if ((err = cudaEventRecord(landed, ctx->in)) != cudaSuccess) break;
        if ((err = cudaStreamWaitEvent(ctx->compute, landed, 0)) != cudaSuccess) break;
        if (host_call_native(c))
            err = fpx::launch_native_gemm(c.e_bits, c.m_bits, ctx->compute, c.weight_native_dev, static_cast<const __half*>(c.scales_dev),
                                          act, out, c.M, c.N, c.K, ws, status);
        else
            err = fpx::launch_gemm(c.e_bits, c.m_bits, ctx->compute, c.weight_packed_dev, static_cast<const __half*>(c.scales_dev),
                                   act, out, c.M, c.N, c.K, ws, c.split_k, status);
        if (err != cudaSuccess) break;
        if ((err = cudaEventRecord(done, ctx->compute)) != cudaSuccess) break;
        if ((err = cudaStreamWaitEvent(ctx->out, done, 0)) != cudaSuccess) break;
        err = cudaMemcpyAsync(c.out_host, out, out_bytes, cudaMemcpyDeviceToHost, ctx->out);
    }
    // whatever was queued must finish before the staging buffer may be reused, error or not
    const cudaError_t e1 = cudaStreamSynchronize(ctx->in), e2 = cudaStreamSynchronize(ctx->compute), e3 = cudaStreamSynchronize(ctx->out);
    if (err != cudaSuccess) return err;
    return e1 != cudaSuccess ? e1 : (e2 != cudaSuccess ? e2 : e3);
}

int fp6b200_prepack(int e_bits, int m_bits, void* stream, const void* unpacked_dev, void* packed_dev, size_t M,
                    size_t K) {
    return fpx::launch_prepack(e_bits, m_bits, static_cast<cudaStream_t>(stream), unpacked_dev, packed_dev, M, K);
}

int fp6b200_quantize_prepack(int e_bits, int m_bits, void* stream, const void* weights_fp16_dev, const void* scales_dev,
                             void* packed_dev, size_t M, size_t K) {
    return fpx::launch_quantize_prepack(e_bits, m_bits, static_cast<cudaStream_t>(stream),
                                        static_cast<const __half*>(weights_fp16_dev), static_cast<const __half*>(scales_dev),
                                        packed_dev, M, K);
}

int fp6b200_prepack_host(int e_bits, int m_bits, int* packed_host, const int* unpacked_host, size_t M, size_t K) {
    if (!fpx::format_supported(e_bits, m_bits) || !packed_host || !unpacked_host || M % 64 || K % 64 || !M || !K)
        return cudaErrorInvalidValue;
    const size_t bytes = M * K * (size_t)(1 + e_bits + m_bits) / 8, padded = align_up(bytes, 256);
    std::lock_guard<std::mutex> lock(staging().mu);
    void* base = nullptr;
    cudaStream_t stream = nullptr;
    cudaError_t err = staging_get(2 * padded, &base, &stream);
    if (err != cudaSuccess) return err;
    char* in = static_cast<char*>(base);
    char* out = in + padded;
    err = cudaMemcpyAsync(in, unpacked_host, bytes, cudaMemcpyHostToDevice, stream);
    if (err != cudaSuccess) return err;
    err = fpx::launch_prepack(e_bits, m_bits, stream, in, out, M, K);
    if (err != cudaSuccess) return err;
    err = cudaMemcpyAsync(packed_host, out, bytes, cudaMemcpyDeviceToHost, stream);
    if (err != cudaSuccess) return err;
    return cudaStreamSynchronize(stream);
}

int fp6b200_dequant(int e_bits, int m_bits, void* stream, const void* unpacked_dev, const void* scales_dev,
                    void* out_dev, size_t M, size_t K) {
    return fpx::launch_dequant_unpacked(e_bits, m_bits, static_cast<cudaStream_t>(stream), unpacked_dev,
                                        static_cast<const __half*>(scales_dev), static_cast<__half*>(out_dev), M, K);
}

int fp6b200_dequant_host(int e_bits, int m_bits, void* out_host, const void* unpacked_host, size_t M, size_t K,
                         const void* scales_host) {
    if (!fpx::format_supported(e_bits, m_bits) || !out_host || !unpacked_host || !scales_host || M % 64 || K % 64 ||
        !M || !K)
        return cudaErrorInvalidValue;
    const size_t in_bytes = M * K * (size_t)(1 + e_bits + m_bits) / 8, in_pad = align_up(in_bytes, 256);
    const size_t sc_pad = align_up(M * sizeof(__half), 256), out_bytes = M * K * sizeof(__half);
    std::lock_guard<std::mutex> lock(staging().mu);
    void* base = nullptr;
    cudaStream_t stream = nullptr;
    cudaError_t err = staging_get(in_pad + sc_pad + out_bytes, &base, &stream);
    if (err != cudaSuccess) return err;
    char* in = static_cast<char*>(base);
    __half* sc = reinterpret_cast<__half*>(in + in_pad);
    __half* out = reinterpret_cast<__half*>(in + in_pad + sc_pad);
    err = cudaMemcpyAsync(in, unpacked_host, in_bytes, cudaMemcpyHostToDevice, stream);
    if (err != cudaSuccess) return err;
    err = cudaMemcpyAsync(sc, scales_host, M * sizeof(__half), cudaMemcpyHostToDevice, stream);
    if (err != cudaSuccess) return err;
    err = fpx::launch_dequant_unpacked(e_bits, m_bits, stream, in, sc, out, M, K);
    if (err != cudaSuccess) return err;
    err = cudaMemcpyAsync(out_host, out, out_bytes, cudaMemcpyDeviceToHost, stream);
    if (err != cudaSuccess) return err;
    return cudaStreamSynchronize(stream);
}

int fp6b200_dequant_packed(int e_bits, int m_bits, void* stream, const void* packed_dev, const void* scales_dev,
                           void* out_dev, size_t M, size_t K) {
    return fpx::launch_dequant_packed(e_bits, m_bits, static_cast<cudaStream_t>(stream), packed_dev,
                                      static_cast<const __half*>(scales_dev), static_cast<__half*>(out_dev), M, K);
}

int fp6b200_splitk_reduce(void* stream, void* out_dev, const float* partials_dev, size_t elems, int split_k) {
    if (!out_dev || !partials_dev || elems == 0 || elems % 4 || split_k < 1) return cudaErrorInvalidValue;
    return fpx::launch_splitk_reduce(static_cast<cudaStream_t>(stream), static_cast<__half*>(out_dev), partials_dev,
                                     elems, split_k, false, 0, nullptr);
}

int fp6b200_device_status(int* code) {
    if (!code) return cudaErrorInvalidValue;
    cudaError_t err = cudaDeviceSynchronize();
    if (err != cudaSuccess) return err;
    err = cudaMemcpyFromSymbol(code, g_gemm_status, sizeof(int));
    if (err != cudaSuccess) return err;
    if (*code != 0) {
        const int zero = 0;
        err = cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(int));
    }
    return err;
}

}  // extern "C"

// ------------------------------------------------------------------ C++ names of the reference
cudaError_t fp6_linear_kernel(cudaStream_t stream, const uint4* Weight, const half* Scales, const half* B, half* C,
                              const size_t M_Global, const size_t N_Global, const size_t K_Global,
                              float* Reduction_Workspace, int Split_K) {
    return static_cast<cudaError_t>(
        fp6b200_linear(3, 2, stream, Weight, Scales, B, C, M_Global, N_Global, K_Global, Reduction_Workspace, Split_K));
}

cudaError_t fp_eXmY_linear_kernel(const int EXPONENT, const int MANTISSA, cudaStream_t stream, const uint4* Weight,
                                  const half* Scales, const half* B, half* C, const size_t M_Global,
                                  const size_t N_Global, const size_t K_Global, float* Reduction_Workspace,
                                  int Split_K) {
    return static_cast<cudaError_t>(fp6b200_linear(EXPONENT, MANTISSA, stream, Weight, Scales, B, C, M_Global, N_Global,
                                                   K_Global, Reduction_Workspace, Split_K));
}

void weight_matrix_prepacking_fp_eXmY(const int EXPONENT, const int MANTISSA, int* packed_weights, int* FPxWeights,
                                      size_t M, size_t K) {
    const int rc = fp6b200_prepack_host(EXPONENT, MANTISSA, packed_weights, FPxWeights, M, K);
    if (rc != 0)
        fprintf(stderr, "fp6_llm_b200: weight prepacking failed (e%dm%d, %zux%zu): %s\n", EXPONENT, MANTISSA, M, K,
                fp6b200_error_string(rc));
}

void weight_matrix_prepacking(int* packed_weights, int* FP6Weights, size_t M, size_t K) {
    weight_matrix_prepacking_fp_eXmY(3, 2, packed_weights, FP6Weights, M, K);
}

void dequant_matrix_fp_eXmY_to_fp16(const int EXPONENT, const int MANTISSA, half* A_16bit_h, unsigned char* A_6bit_h,
                                    size_t M, size_t K, half* scale) {
    const int rc = fp6b200_dequant_host(EXPONENT, MANTISSA, A_16bit_h, A_6bit_h, M, K, scale);
    if (rc != 0)
        fprintf(stderr, "fp6_llm_b200: weight dequantisation failed (e%dm%d, %zux%zu): %s\n", EXPONENT, MANTISSA, M, K,
                fp6b200_error_string(rc));
}

void DeQuantMatrix_FP6_To_FP16(half* A_16bit_h, unsigned char* A_6bit_h, size_t M, size_t K, half* scale) {
    dequant_matrix_fp_eXmY_to_fp16(3, 2, A_16bit_h, A_6bit_h, M, K, scale);
}
