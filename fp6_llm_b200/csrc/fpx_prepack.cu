// Weight-format kernels for sm_100a:
//   * prepack:            unpacked MSB-first code streams -> the reference's bit-interleaved
//                         [1-bit | 2-bit | 4-bit] region layout, bit-exact with the CPU packer
//                         (fp6_llm/csrc/utils/weight_prepacking.h:118-196);
//   * dequant (unpacked): the reference's CPU dequantiser on the GPU
//                         (fp6_llm/csrc/utils/weight_dequant.h:10-48);
//   * dequant (packed):   prepacked weights -> fp16 [M, K] with exactly the unpack code of the GEMM,
//                         for fp16 GEMM comparisons and for checking the packed format end to end.
// All three are byte shuffles bounded by HBM traffic (bytes in + bytes out).
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "fpx_internal.h"
#include "fpx_layout.h"

namespace fpx {

namespace {

constexpr int kPrepackThreads = 256;
constexpr int kChunkKBlocks = 4;   // a CTA repacks 64 rows x (up to) 256 columns

// One CTA: stage 64 rows x chunk columns of the unpacked stream in shared memory (coalesced 4-byte
// reads), then build every output word of that chunk; each word gathers 32/w segments.
template <int BW>
__global__ void __launch_bounds__(kPrepackThreads)
prepack_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, uint32_t M, uint32_t K) {
    constexpr uint32_t kMaxChunkBytes = kChunkKBlocks * kKBlock * BW / 8;
    constexpr uint32_t kPitch = kMaxChunkBytes + 4;
    __shared__ __align__(16) uint8_t tile[kRowsPerBlock * kPitch];

    const uint32_t kblocks = K / kKBlock;
    const uint32_t chunks_per_row = (kblocks + kChunkKBlocks - 1) / kChunkKBlocks;
    const uint32_t i = blockIdx.x / chunks_per_row;            // 64-row block
    const uint32_t kb0 = (blockIdx.x % chunks_per_row) * kChunkKBlocks;
    const uint32_t nkb = min((uint32_t)kChunkKBlocks, kblocks - kb0);
    const uint32_t chunk_bytes = nkb * kKBlock * BW / 8;       // multiple of 8
    const uint32_t col0 = kb0 * kKBlock;
    const size_t row_bytes = (size_t)K * BW / 8;

    const uint32_t words_per_row = chunk_bytes / 4;
    for (uint32_t x = threadIdx.x; x < kRowsPerBlock * words_per_row; x += kPrepackThreads) {
        const uint32_t r = x / words_per_row, wd = x % words_per_row;
        const uint32_t v = *reinterpret_cast<const uint32_t*>(in + (size_t)(i * kRowsPerBlock + r) * row_bytes +
                                                              (size_t)col0 * BW / 8 + wd * 4);
        *reinterpret_cast<uint32_t*>(tile + r * kPitch + wd * 4) = v;
    }
    if (threadIdx.x < kRowsPerBlock) tile[threadIdx.x * kPitch + chunk_bytes] = 0;   // read_code may peek one byte past
    __syncthreads();

#pragma unroll
    for (int w = 1; w <= 4; w <<= 1) {
        if (!has_seg(BW, w)) continue;
        const int shift = seg_shift(BW, w);
        const uint32_t words_per_tile = 4u * w * 32u;           // uint32 words of one 64x64 tile in this region
        uint32_t* region = reinterpret_cast<uint32_t*>(out + region_offset(BW, w, M, K));
        for (uint32_t x = threadIdx.x; x < nkb * words_per_tile; x += kPrepackThreads) {
            const uint32_t kb = kb0 + x / words_per_tile;
            const uint32_t in_tile = x % words_per_tile;
            const int lane = in_tile & 31;
            const uint64_t word_in_lane = ((uint64_t)i * kblocks + kb) * (4u * w) + (in_tile >> 5);
            uint32_t word = 0;
#pragma unroll 8
            for (int p = 0; p < 32 / w; p++) {
                const FieldSource s = field_source(w, word_in_lane, lane, p, K);
                const uint32_t code = read_code(tile + (s.row - i * kRowsPerBlock) * kPitch, s.col - col0, BW);
                word |= ((code >> shift) & ((1u << w) - 1u)) << (32 - (p + 1) * w);
            }
            region[word_in_lane * 32 + lane] = word;
        }
    }
}

// Round-to-nearest quantiser fused with the packer: fp16 weights [M, K] and fp16 row scales in, prepacked FPx out,
// without the unpacked tensor in between.  (The reference ships no working quantiser: fp6_llm/csrc/utils/
// weight_quant.h:9-104 truncates and is not bound; the layout it would feed is the packer's above.)
// Code of a weight = nearest representable magnitude of |w / scale| (the division in fp32, round to nearest);
// ties go to the even code; beyond the largest magnitude it saturates; the sign bit is the sign of the quotient.
template <int E_BITS, int M_BITS>
__global__ void __launch_bounds__(kPrepackThreads)
quantize_prepack_kernel(const __half* __restrict__ w, const __half* __restrict__ scales, uint8_t* __restrict__ out,
                        uint32_t M, uint32_t K) {
    constexpr int BW = 1 + E_BITS + M_BITS;
    constexpr uint32_t kCols = kChunkKBlocks * kKBlock;
    constexpr uint32_t kPitch = kCols + 4;
    __shared__ __align__(16) uint8_t codes[kRowsPerBlock * kPitch];

    const uint32_t kblocks = K / kKBlock;
    const uint32_t chunks_per_row = (kblocks + kChunkKBlocks - 1) / kChunkKBlocks;
    const uint32_t i = blockIdx.x / chunks_per_row;            // 64-row block
    const uint32_t kb0 = (blockIdx.x % chunks_per_row) * kChunkKBlocks;
    const uint32_t nkb = min((uint32_t)kChunkKBlocks, kblocks - kb0);
    const uint32_t ncols = nkb * kKBlock;
    const uint32_t col0 = kb0 * kKBlock;

    for (uint32_t x = threadIdx.x; x < kRowsPerBlock * (ncols / 2); x += kPrepackThreads) {   // two weights per thread and round
        const uint32_t r = x / (ncols / 2), c = (x % (ncols / 2)) * 2;
        const uint32_t row = i * kRowsPerBlock + r;
        const __half2 pair = *reinterpret_cast<const __half2*>(w + (size_t)row * K + col0 + c);
        const float sc = __half2float(scales[row]);
        codes[r * kPitch + c] = (uint8_t)quantize_rtn_code(E_BITS, M_BITS, __fdiv_rn(__low2float(pair), sc));
        codes[r * kPitch + c + 1] = (uint8_t)quantize_rtn_code(E_BITS, M_BITS, __fdiv_rn(__high2float(pair), sc));
    }
    __syncthreads();

#pragma unroll
    for (int wd = 1; wd <= 4; wd <<= 1) {
        if (!has_seg(BW, wd)) continue;
        const int shift = seg_shift(BW, wd);
        const uint32_t words_per_tile = 4u * wd * 32u;
        uint32_t* region = reinterpret_cast<uint32_t*>(out + region_offset(BW, wd, M, K));
        for (uint32_t x = threadIdx.x; x < nkb * words_per_tile; x += kPrepackThreads) {
            const uint32_t kb = kb0 + x / words_per_tile;
            const uint32_t in_tile = x % words_per_tile;
            const int lane = in_tile & 31;
            const uint64_t word_in_lane = ((uint64_t)i * kblocks + kb) * (4u * wd) + (in_tile >> 5);
            uint32_t word = 0;
#pragma unroll 8
            for (int pos = 0; pos < 32 / wd; pos++) {
                const FieldSource src = field_source(wd, word_in_lane, lane, pos, K);
                const uint32_t code = codes[(src.row - i * kRowsPerBlock) * kPitch + (src.col - col0)];
                word |= ((code >> shift) & ((1u << wd) - 1u)) << (32 - (pos + 1) * wd);
            }
            region[word_in_lane * 32 + lane] = word;
        }
    }
}

// Thread = 8 consecutive codes of one row (BW bytes in, 16 bytes out).
template <int E_BITS, int M_BITS>
__global__ void __launch_bounds__(256)
dequant_unpacked_kernel(const uint8_t* __restrict__ in, const __half* __restrict__ scales, __half* __restrict__ out,
                        uint32_t M, uint32_t K) {
    constexpr int BW = 1 + E_BITS + M_BITS;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;   // group of 8 codes
    const size_t groups_per_row = K / 8;
    if (idx >= (size_t)M * groups_per_row) return;
    const size_t row = idx / groups_per_row;
    const uint8_t* src = in + idx * BW;
    uint8_t bytes[BW + 1];
#pragma unroll
    for (int b = 0; b < BW; b++) bytes[b] = src[b];
    bytes[BW] = 0;
    const float s = __half2float(scales[row]);
    const float bias = (float)(1u << (16 - (1 << (E_BITS - 1))));
    __align__(16) __half vals[8];
#pragma unroll
    for (int c = 0; c < 8; c++) {
        const uint32_t code = read_code(bytes, c, BW);
        const uint32_t left = code << (16 - BW);   // code left-aligned in 16 bits
        const uint16_t h = (uint16_t)((left & 0x8000u) | ((left & 0x7fffu) >> (5 - E_BITS)));
        vals[c] = __float2half_rn(__half2float(__ushort_as_half(h)) * bias * s);
    }
    *reinterpret_cast<uint4*>(out + idx * 8) = *reinterpret_cast<const uint4*>(vals);
}

// Warp = 32 rows x 64 columns, the unit one unpack warp of the GEMM handles per pipeline stage.
template <int E_BITS, int M_BITS>
__global__ void __launch_bounds__(128)
dequant_packed_kernel(const uint8_t* __restrict__ packed, const __half* __restrict__ scales, __half* __restrict__ out,
                      uint32_t M, uint32_t K) {
    constexpr int BW = 1 + E_BITS + M_BITS;
    const uint32_t kblocks = K / kKBlock;
    const uint32_t unit = blockIdx.x * 4 + (threadIdx.x >> 5);     // (64-row block, k-block, half)
    if (unit >= (M / kRowsPerBlock) * kblocks * 2) return;
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int h = unit & 1;
    const uint32_t kb = (unit >> 1) % kblocks, i = (unit >> 1) / kblocks;
    const uint64_t tile = (uint64_t)i * kblocks + kb;
    const uint32_t* r1 = reinterpret_cast<const uint32_t*>(packed + region_offset(BW, 1, M, K) + tile * tile_bytes(1));
    const uint32_t* r2 = reinterpret_cast<const uint32_t*>(packed + region_offset(BW, 2, M, K) + tile * tile_bytes(2));
    const uint32_t* r4 = reinterpret_cast<const uint32_t*>(packed + region_offset(BW, 4, M, K) + tile * tile_bytes(4));
    const __half bias_h = __ushort_as_half(bias_half_bits(E_BITS));
    const uint32_t row_base = i * kRowsPerBlock + 32 * h;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const uint32_t w4a = r4[(j * 4 + 2 * h + 0) * 32 + lane], w4b = r4[(j * 4 + 2 * h + 1) * 32 + lane];
        const uint32_t w2 = has_seg(BW, 2) ? r2[(j * 2 + h) * 32 + lane] : 0u;
        const uint32_t w1 = has_seg(BW, 1) ? r1[j * 32 + lane] : 0u;
        uint32_t pat[8];
        unpack16_any<E_BITS, M_BITS>(w4a, w4b, w2, w1, h, pat);
#pragma unroll
        for (int kk = 0; kk < 2; kk++)
#pragma unroll
            for (int a = 0; a < 4; a++) {
                const uint32_t row = row_base + 16 * kk + 8 * (a & 1) + g;
                const uint32_t col = kb * kKBlock + 16 * j + 8 * (a >> 1) + 2 * t;
                const __half s = scales[row];
                __half2 v = *reinterpret_cast<__half2*>(&pat[4 * kk + a]);
                v = __hmul2(__hmul2(v, __half2half2(bias_h)), __half2half2(s));   // first product is exact
                *reinterpret_cast<__half2*>(out + (size_t)row * K + col) = v;
            }
    }
}

bool shape_ok(int e_bits, int m_bits, size_t M, size_t K) {
    // the packer itself needs 64-row / 64-column granularity (weight_prepacking.h:121-122)
    return format_supported(e_bits, m_bits) && M > 0 && K > 0 && M % 64 == 0 && K % 64 == 0 && M <= 0xffffffffull &&
           K <= 0x7fffffffull;
}

}  // namespace

cudaError_t launch_prepack(int e_bits, int m_bits, cudaStream_t stream, const void* unpacked, void* packed, size_t M,
                           size_t K) {
    if (!shape_ok(e_bits, m_bits, M, K) || !unpacked || !packed || unpacked == packed) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(unpacked) & 3) || (reinterpret_cast<uintptr_t>(packed) & 3))
        return cudaErrorMisalignedAddress;
    const size_t kblocks = K / kKBlock;
    const size_t blocks = (M / kRowsPerBlock) * ((kblocks + kChunkKBlocks - 1) / kChunkKBlocks);
    if (blocks > 0x7fffffffull) return cudaErrorInvalidValue;
    const uint8_t* in = static_cast<const uint8_t*>(unpacked);
    uint8_t* out = static_cast<uint8_t*>(packed);
    switch (1 + e_bits + m_bits) {
        case 4:  prepack_kernel<4><<<(unsigned)blocks, kPrepackThreads, 0, stream>>>(in, out, (uint32_t)M, (uint32_t)K); break;
        case 5:  prepack_kernel<5><<<(unsigned)blocks, kPrepackThreads, 0, stream>>>(in, out, (uint32_t)M, (uint32_t)K); break;
        default: prepack_kernel<6><<<(unsigned)blocks, kPrepackThreads, 0, stream>>>(in, out, (uint32_t)M, (uint32_t)K); break;
    }
    return cudaGetLastError();
}

cudaError_t launch_quantize_prepack(int e_bits, int m_bits, cudaStream_t stream, const __half* weights,
                                    const __half* scales, void* packed, size_t M, size_t K) {
    if (!shape_ok(e_bits, m_bits, M, K) || !weights || !scales || !packed) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(weights) & 3) || (reinterpret_cast<uintptr_t>(packed) & 3))
        return cudaErrorMisalignedAddress;
    const size_t kblocks = K / kKBlock;
    const size_t blocks = (M / kRowsPerBlock) * ((kblocks + kChunkKBlocks - 1) / kChunkKBlocks);
    if (blocks > 0x7fffffffull) return cudaErrorInvalidValue;
    uint8_t* out = static_cast<uint8_t*>(packed);
    FPX_DISPATCH_FORMAT(e_bits, m_bits, (quantize_prepack_kernel<kE, kM><<<(unsigned)blocks, kPrepackThreads, 0, stream>>>(weights, scales, out, (uint32_t)M, (uint32_t)K)));
    return cudaGetLastError();
}

cudaError_t launch_dequant_unpacked(int e_bits, int m_bits, cudaStream_t stream, const void* unpacked,
                                    const __half* scales, __half* out, size_t M, size_t K) {
    if (!shape_ok(e_bits, m_bits, M, K) || !unpacked || !scales || !out) return cudaErrorInvalidValue;
    if (reinterpret_cast<uintptr_t>(out) & 15) return cudaErrorMisalignedAddress;
    const size_t groups = M * (K / 8);
    const size_t blocks = (groups + 255) / 256;
    if (blocks > 0x7fffffffull) return cudaErrorInvalidValue;
    const uint8_t* in = static_cast<const uint8_t*>(unpacked);
    FPX_DISPATCH_FORMAT(e_bits, m_bits, (dequant_unpacked_kernel<kE, kM><<<(unsigned)blocks, 256, 0, stream>>>(in, scales, out, (uint32_t)M, (uint32_t)K)));
    return cudaGetLastError();
}

cudaError_t launch_dequant_packed(int e_bits, int m_bits, cudaStream_t stream, const void* packed,
                                  const __half* scales, __half* out, size_t M, size_t K) {
    if (!shape_ok(e_bits, m_bits, M, K) || !packed || !scales || !out) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(packed) & 15) || (reinterpret_cast<uintptr_t>(out) & 3))
        return cudaErrorMisalignedAddress;
    const size_t units = (M / kRowsPerBlock) * (K / kKBlock) * 2;
    const size_t blocks = (units + 3) / 4;
    if (blocks > 0x7fffffffull) return cudaErrorInvalidValue;
    const uint8_t* in = static_cast<const uint8_t*>(packed);
    FPX_DISPATCH_FORMAT(e_bits, m_bits, (dequant_packed_kernel<kE, kM><<<(unsigned)blocks, 128, 0, stream>>>(in, scales, out, (uint32_t)M, (uint32_t)K)));
    return cudaGetLastError();
}

}  // namespace fpx
