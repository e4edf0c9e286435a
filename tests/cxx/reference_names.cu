// Calls the library through the C++ names and signatures of the reference's header (fp6_llm/csrc/fp6_linear.cuh:8-43),
// the way the reference's own tests/cpp programs do: in-place weight prepacking, CPU-side dequantisation, the GEMM.
// Reads the unpacked weights, scales and activations from files, writes what the three calls produce; the Python test
// compares the files with the oracle.
//   usage: reference_names <dir> <M> <N> <K> <split_k>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "fp6_llm_b200_cxx.cuh"

static bool read_file(const std::string& path, void* dst, size_t bytes) {
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) return false;
    const size_t n = fread(dst, 1, bytes, f);
    fclose(f);
    return n == bytes;
}
static bool write_file(const std::string& path, const void* src, size_t bytes) {
    FILE* f = fopen(path.c_str(), "wb");
    if (!f) return false;
    const size_t n = fwrite(src, 1, bytes, f);
    fclose(f);
    return n == bytes;
}

int main(int argc, char** argv) {
    if (argc != 6) return 2;
    const std::string dir = argv[1];
    const size_t M = strtoull(argv[2], nullptr, 10), N = strtoull(argv[3], nullptr, 10), K = strtoull(argv[4], nullptr, 10);
    const int split_k = atoi(argv[5]);
    const size_t w_bytes = M * K * 6 / 8;
    std::vector<int> weights(w_bytes / 4);
    std::vector<half> scales(M), act(N * K), out(N * M), dequant(M * K);
    if (!read_file(dir + "/weights.bin", weights.data(), w_bytes) || !read_file(dir + "/scales.bin", scales.data(), M * 2) ||
        !read_file(dir + "/act.bin", act.data(), N * K * 2))
        return 3;
    // 1. CPU-side dequantisation of the UNPACKED weights (the reference tests' ground truth)
    DeQuantMatrix_FP6_To_FP16(dequant.data(), reinterpret_cast<unsigned char*>(weights.data()), M, K, scales.data());
    // 2. prepacking IN PLACE, as tests/cpp/kernel_test_fp6.cu does
    weight_matrix_prepacking(weights.data(), weights.data(), M, K);
    // 3. the GEMM on device buffers
    uint4* d_w = nullptr; half *d_s = nullptr, *d_x = nullptr, *d_y = nullptr; float* d_ws = nullptr;
    if (cudaMalloc(&d_w, w_bytes) || cudaMalloc(&d_s, M * 2) || cudaMalloc(&d_x, N * K * 2) || cudaMalloc(&d_y, N * M * 2) ||
        cudaMalloc(&d_ws, sizeof(float) * M * N * (split_k > 0 ? split_k : 1)))
        return 4;
    cudaMemcpy(d_w, weights.data(), w_bytes, cudaMemcpyHostToDevice);
    cudaMemcpy(d_s, scales.data(), M * 2, cudaMemcpyHostToDevice);
    cudaMemcpy(d_x, act.data(), N * K * 2, cudaMemcpyHostToDevice);
    const cudaError_t err = fp6_linear_kernel(0, d_w, d_s, d_x, d_y, M, N, K, d_ws, split_k);
    if (err != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) { fprintf(stderr, "fp6_linear_kernel: %s\n", cudaGetErrorString(err)); return 5; }
    cudaMemcpy(out.data(), d_y, N * M * 2, cudaMemcpyDeviceToHost);
    // the same through the eXmY name
    cudaMemset(d_y, 0, N * M * 2);
    if (fp_eXmY_linear_kernel(3, 2, 0, d_w, d_s, d_x, d_y, M, N, K, d_ws, split_k) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) return 6;
    std::vector<half> out2(N * M);
    cudaMemcpy(out2.data(), d_y, N * M * 2, cudaMemcpyDeviceToHost);
    if (!write_file(dir + "/packed.bin", weights.data(), w_bytes) || !write_file(dir + "/dequant.bin", dequant.data(), M * K * 2) ||
        !write_file(dir + "/out.bin", out.data(), N * M * 2) || !write_file(dir + "/out_exmy.bin", out2.data(), N * M * 2))
        return 7;
    printf("ok\n");
    return 0;
}
