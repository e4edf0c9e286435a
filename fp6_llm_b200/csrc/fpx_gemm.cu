// FPx (e3m2 / e2m2) x fp16 linear layer for sm_100a:  Out[N, M] = Act[N, K] * dequant(W)[M, K]^T.
//
// Replaces the reference's QUANT_GEMM_Kernel + launcher
// (fp6_llm/csrc/include/kernel_matmul.cuh:29-191, fp6_llm/csrc/fp6_linear.cu:11-102) with a design
// built around Blackwell's tensor memory:
//
//   warp 0      streams the packed weight segments of one (128 rows x 64 K) stage with 1-D bulk
//               copies into an 8-deep shared-memory ring (the packed layout keeps all of K
//               contiguous per 64-row block and segment, so no tensor map is needed);
//   warp 1      streams the activation tile [N_TILE x 64] with a 2-D TMA tensor copy (128-byte
//               swizzle, rows past N zero-filled);
//   warps 3-10  unpack the segments with shift/LOP3/PRMT sequences, apply 2^bias * scale[row] in
//               fp16 and write the fp16 weights STRAIGHT INTO TENSOR MEMORY with
//               tcgen05.st.16x128b: the reference's packed format hands every lane exactly the
//               registers of an m16k16 A fragment, which is the register pattern of that store,
//               so the dequantised weights never touch shared memory;
//   warp 2      issues tcgen05.mma.kind::f16 with A from tensor memory and B from shared memory,
//               accumulating fp32 in tensor memory;
//   warps 3-10  finally read the accumulator with tcgen05.ld and store fp16 (or fp32 split-K
//               partials) to global memory.
//
// Every mbarrier wait is bounded; on a time-out the CTA records a code in a status word, drains its
// own copies, frees its tensor memory and returns.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "fpx_internal.h"
#include "fpx_layout.h"
#include "ptx_sm100.cuh"

namespace fpx {

namespace {

constexpr int kTileM = 128;
constexpr int kRawStages = 8;
constexpr int kAStages = 4;
constexpr int kAColsPerStage = 32;                       // 64 fp16 along K per tensor-memory lane
constexpr int kAccColBase = kAStages * kAColsPerStage;   // accumulator columns follow the A ring
constexpr int kFirstDequantWarp = 3;
constexpr int kDequantWarps = 8;
constexpr int kWarps = kFirstDequantWarp + kDequantWarps;
constexpr int kThreads = kWarps * 32;

// status codes written by a wait that gave up
enum : int {
    kErrRawEmpty = 1, kErrRawFull = 2, kErrBEmpty = 3, kErrBFull = 4, kErrAEmpty = 5, kErrAFull = 6, kErrAccFull = 7
};

template <int BW>
struct RawStage {
    static constexpr uint32_t seg1 = (BW & 1) ? tile_bytes(1) : 0u;
    static constexpr uint32_t seg2 = (BW & 2) ? tile_bytes(2) : 0u;
    static constexpr uint32_t seg4 = (BW & 4) ? tile_bytes(4) : 0u;
    // stage layout: [1-bit: row block 0, 1][2-bit: row block 0, 1][4-bit: row block 0, 1]
    static constexpr uint32_t off1 = 0u;
    static constexpr uint32_t off2 = 2u * seg1;
    static constexpr uint32_t off4 = 2u * seg1 + 2u * seg2;
    static constexpr uint32_t bytes = 2u * (seg1 + seg2 + seg4);
};

template <int N_TILE>
struct BStage {
    static constexpr uint32_t bytes = (uint32_t)N_TILE * 128u;
    static constexpr int stages = N_TILE <= 32 ? 8 : (N_TILE <= 64 ? 6 : 4);
};

template <int BW, int N_TILE>
struct Budget {
    static constexpr uint32_t tmem_cols = (kAccColBase + N_TILE) <= 256 ? 256u : 512u;
    static constexpr uint32_t smem_bytes =
        1024u /* alignment slack */ + BStage<N_TILE>::stages * BStage<N_TILE>::bytes + kRawStages * RawStage<BW>::bytes +
        (2 * kRawStages + 2 * BStage<N_TILE>::stages + 2 * kAStages + 1) * 8u + 16u;
};

__device__ __forceinline__ uint32_t scale_pair(uint32_t pat, __half2 c) {
    __half2 v = *reinterpret_cast<__half2*>(&pat);
    v = __hmul2(v, c);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int BW, int N_TILE, bool PARTIAL>
__global__ void __launch_bounds__(kThreads, (N_TILE <= 64) ? 2 : 1)
fpx_gemm_kernel(const __grid_constant__ CUtensorMap act_map, const uint8_t* __restrict__ weight,
                const __half* __restrict__ scales, void* __restrict__ out, uint32_t M, uint32_t N, uint32_t K,
                uint32_t split_k, int* __restrict__ status) {
    constexpr int E_BITS = BW - 3;   // both supported formats have a 2-bit mantissa
    using Raw = RawStage<BW>;
    using BS = BStage<N_TILE>;
    constexpr int SB = BS::stages;
    constexpr int R = kRawStages;
    constexpr int SA = kAStages;

    extern __shared__ uint8_t smem_dyn[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
    uint8_t* b_ring = smem;
    uint8_t* raw_ring = b_ring + SB * BS::bytes;
    uint64_t* raw_full = reinterpret_cast<uint64_t*>(raw_ring + R * Raw::bytes);
    uint64_t* raw_empty = raw_full + R;
    uint64_t* b_full = raw_empty + R;
    uint64_t* b_empty = b_full + SB;
    uint64_t* a_full = b_empty + SB;
    uint64_t* a_empty = a_full + SA;
    uint64_t* acc_full = a_empty + SA;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_full + 1);
    volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_holder + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t m_tile = blockIdx.x, n_tile = blockIdx.y, z = blockIdx.z;
    uint32_t kb_begin, nkb;
    split_range(K / kKBlock, split_k, z, &kb_begin, &nkb);

    if (threadIdx.x == 0) {
        for (int i = 0; i < R; i++) { ptx::mbar_init(&raw_full[i], 1); ptx::mbar_init(&raw_empty[i], 4); }
        for (int i = 0; i < SB; i++) { ptx::mbar_init(&b_full[i], 1); ptx::mbar_init(&b_empty[i], 1); }
        for (int i = 0; i < SA; i++) { ptx::mbar_init(&a_full[i], 4); ptx::mbar_init(&a_empty[i], 1); }
        ptx::mbar_init(acc_full, 1);
        *abort_word = 0;
        ptx::fence_barrier_init();
    }
    if (warp == 2) {
        ptx::tmem_alloc(tmem_holder, Budget<BW, N_TILE>::tmem_cols);
        ptx::tmem_relinquish();
    }
    if (warp == 1 && lane == 0) ptx::prefetch_tensormap(&act_map);
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;

    if (warp == 0) {
        // ------------------------------------------------------------ packed-weight producer
        if (lane == 0) {
            const uint64_t policy = ptx::policy_evict_first();
            const uint64_t kblocks = K / kKBlock;
            const uint64_t rb0 = (uint64_t)m_tile * 2;   // first 64-row block of this tile
            const uint8_t* reg1 = weight + region_offset(BW, 1, M, K);
            const uint8_t* reg2 = weight + region_offset(BW, 2, M, K);
            const uint8_t* reg4 = weight + region_offset(BW, 4, M, K);
            uint32_t issued = 0;
            for (uint32_t it = 0; it < nkb; it++) {
                const uint32_t r = it % R;
                if (!ptx::mbar_wait(&raw_empty[r], ((it / R) & 1u) ^ 1u, abort_word, kErrRawEmpty)) break;
                ptx::mbar_arrive_expect_tx(&raw_full[r], Raw::bytes);
                uint8_t* dst = raw_ring + r * Raw::bytes;
                const uint64_t kb = kb_begin + it;
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    const uint64_t tile = (rb0 + i) * kblocks + kb;
                    if (Raw::seg1) ptx::bulk_g2s(dst + Raw::off1 + i * Raw::seg1, reg1 + tile * Raw::seg1, Raw::seg1, &raw_full[r], policy);
                    if (Raw::seg2) ptx::bulk_g2s(dst + Raw::off2 + i * Raw::seg2, reg2 + tile * Raw::seg2, Raw::seg2, &raw_full[r], policy);
                    if (Raw::seg4) ptx::bulk_g2s(dst + Raw::off4 + i * Raw::seg4, reg4 + tile * Raw::seg4, Raw::seg4, &raw_full[r], policy);
                }
                issued = it + 1;
            }
            if (*abort_word != 0) {   // gave up somewhere: let this thread's own copies land before leaving
                const uint32_t first = issued > (uint32_t)R ? issued - R : 0u;
                for (uint32_t it = first; it < issued; it++)
                    ptx::mbar_wait(&raw_full[it % R], (it / R) & 1u, abort_word, kErrRawFull, 50000000ull);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ activation producer
        if (lane == 0) {
            const uint64_t policy = ptx::policy_evict_last();
            uint32_t issued = 0;
            for (uint32_t it = 0; it < nkb; it++) {
                const uint32_t s = it % SB;
                if (!ptx::mbar_wait(&b_empty[s], ((it / SB) & 1u) ^ 1u, abort_word, kErrBEmpty)) break;
                ptx::mbar_arrive_expect_tx(&b_full[s], BS::bytes);
                ptx::tma_load_2d(b_ring + s * BS::bytes, &act_map, (int32_t)((kb_begin + it) * kKBlock),
                                 (int32_t)(n_tile * N_TILE), &b_full[s], policy);
                issued = it + 1;
            }
            if (*abort_word != 0) {
                const uint32_t first = issued > (uint32_t)SB ? issued - SB : 0u;
                for (uint32_t it = first; it < issued; it++)
                    ptx::mbar_wait(&b_full[it % SB], (it / SB) & 1u, abort_word, kErrBFull, 50000000ull);
            }
        }
    } else if (warp == 2) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = ptx::idesc_f16_f32(kTileM, N_TILE);
            const uint32_t d_tmem = tmem_base + kAccColBase;
            for (uint32_t it = 0; it < nkb; it++) {
                const uint32_t sa = it % SA, sb = it % SB;
                if (!ptx::mbar_wait(&a_full[sa], (it / SA) & 1u, abort_word, kErrAFull)) break;
                if (!ptx::mbar_wait(&b_full[sb], (it / SB) & 1u, abort_word, kErrBFull)) break;
                ptx::tc_fence_after_sync();
                const uint64_t b_desc = ptx::smem_desc_k_sw128(ptx::smem_u32(b_ring + sb * BS::bytes));
                const uint32_t a_tmem = tmem_base + sa * kAColsPerStage;
#pragma unroll
                for (uint32_t kk = 0; kk < 4; kk++)   // four K=16 steps; B advances 32 bytes inside the swizzle row
                    ptx::mma_f16_ts(d_tmem, a_tmem + kk * 8, b_desc + kk * 2, idesc, (it | kk) != 0u ? 1u : 0u);
                ptx::tc_commit(&a_empty[sa]);
                ptx::tc_commit(&b_empty[sb]);
            }
            ptx::tc_commit(acc_full);
            if (*abort_word != 0)   // nobody will consume the accumulator: wait here so dealloc follows the MMAs
                ptx::mbar_wait(acc_full, 0, abort_word, kErrAccFull, 50000000ull);
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ unpack warps, then epilogue
        const int q = warp & 3;                          // tensor-memory lane quadrant this warp may touch
        const int pair = (warp - kFirstDequantWarp) >> 2;   // 0/1: which of the two warps of the quadrant
        const int h = q & 1;                             // sub-blocks 2h, 2h+1 of the 64-row block
        const int rb = q >> 1;                           // 64-row block inside the 128-row tile
        const int g = lane >> 2;
        const uint32_t row0 = m_tile * kTileM + 32u * q;

        // per-row constant 2^bias * scale (exact in fp16 unless it overflows; then multiply in two steps,
        // like the reference's MultScale, utils_parallel_dequant.cuh:30-42)
        const __half bias_h = __ushort_as_half(bias_half_bits(E_BITS));
        __half sc[2][2];
        bool overflow = false;
#pragma unroll
        for (int kk = 0; kk < 2; kk++)
#pragma unroll
            for (int hr = 0; hr < 2; hr++) {
                const __half s = scales[row0 + 16 * kk + 8 * hr + g];
                const __half c = __hmul(s, bias_h);
                overflow |= __hisinf(c) || __hisnan(c);
                sc[kk][hr] = c;
            }
        const bool two_step = __any_sync(0xffffffffu, overflow);
        __half2 c2[2][2];
        if (two_step) {
#pragma unroll
            for (int kk = 0; kk < 2; kk++)
#pragma unroll
                for (int hr = 0; hr < 2; hr++) c2[kk][hr] = __half2half2(scales[row0 + 16 * kk + 8 * hr + g]);
        } else {
#pragma unroll
            for (int kk = 0; kk < 2; kk++)
#pragma unroll
                for (int hr = 0; hr < 2; hr++) c2[kk][hr] = __half2half2(sc[kk][hr]);
        }
        const __half2 bias2 = __half2half2(bias_h);

        bool ok = true;
        for (uint32_t it = pair; it < nkb; it += 2) {
            const uint32_t r = it % R;
            if (!ptx::mbar_wait(&raw_full[r], (it / R) & 1u, abort_word, kErrRawFull)) { ok = false; break; }
            const uint32_t* raw = reinterpret_cast<const uint32_t*>(raw_ring + r * Raw::bytes);
            uint32_t w4[4][2], w2[4], w1[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                w4[j][0] = raw[Raw::off4 / 4 + rb * (Raw::seg4 / 4) + (j * 4 + 2 * h + 0) * 32 + lane];
                w4[j][1] = raw[Raw::off4 / 4 + rb * (Raw::seg4 / 4) + (j * 4 + 2 * h + 1) * 32 + lane];
                w2[j] = Raw::seg2 ? raw[Raw::off2 / 4 + rb * (Raw::seg2 / 4) + (j * 2 + h) * 32 + lane] : 0u;
                w1[j] = Raw::seg1 ? raw[Raw::off1 / 4 + rb * (Raw::seg1 / 4) + j * 32 + lane] : 0u;
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&raw_empty[r]);   // the slot can be refilled while we compute

            uint32_t v[2][16];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                uint32_t pat[8];
                unpack16<E_BITS>(w4[j][0], w4[j][1], w2[j], w1[j], h, pat);
#pragma unroll
                for (int kk = 0; kk < 2; kk++)
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        uint32_t x = pat[4 * kk + i];
                        if (two_step) x = scale_pair(x, bias2);
                        v[kk][4 * j + i] = scale_pair(x, c2[kk][i & 1]);   // a0,a2: row g; a1,a3: row g+8
                    }
            }
            const uint32_t sa = it % SA;
            if (!ptx::mbar_wait(&a_empty[sa], ((it / SA) & 1u) ^ 1u, abort_word, kErrAEmpty)) { ok = false; break; }
            ptx::tc_fence_after_sync();
            const uint32_t a_addr = tmem_base + ((uint32_t)(32 * q) << 16) + sa * kAColsPerStage;
            ptx::tmem_st_16x128b_x8(a_addr, v[0]);
            ptx::tmem_st_16x128b_x8(a_addr + (16u << 16), v[1]);
            ptx::tc_wait_st();
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&a_full[sa]);
        }

        // -------- epilogue: tensor-memory lane = output channel, column = token
        if (ok && nkb > 0) ok = ptx::mbar_wait(acc_full, 0, abort_word, kErrAccFull);
        ptx::tc_fence_after_sync();
        if (ok && *abort_word == 0) {
            const uint32_t row = row0 + lane;
            constexpr int kColsPerWarp = N_TILE / 2;
#pragma unroll 1
            for (int c0 = pair * kColsPerWarp; c0 < (pair + 1) * kColsPerWarp; c0 += 8) {
                const uint32_t n0 = n_tile * N_TILE + c0;
                if (n0 >= N) break;
                uint32_t acc[8];
                if (nkb > 0) {
                    ptx::tmem_ld_32x32b_x8(tmem_base + ((uint32_t)(32 * q) << 16) + kAccColBase + c0, acc);
                    ptx::tc_wait_ld();
                } else {
#pragma unroll
                    for (int u = 0; u < 8; u++) acc[u] = 0u;
                }
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const uint32_t n = n0 + u;
                    if (n < N) {
                        const float f = __uint_as_float(acc[u]);
                        if (PARTIAL)
                            reinterpret_cast<float*>(out)[((size_t)z * N + n) * M + row] = f;
                        else
                            reinterpret_cast<__half*>(out)[(size_t)n * M + row] = __float2half_rn(f);
                    }
                }
            }
        }
    }

    // ------------------------------------------------------------ teardown
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 2) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, Budget<BW, N_TILE>::tmem_cols);
    }
    if (threadIdx.x == 0 && *abort_word != 0) atomicCAS(status, 0, *abort_word);
}

// ------------------------------------------------------------------------------------------------
// Split-K reduction: out[i] = rn_half(sum over splits, ascending, fp32), the semantics of the
// reference's SplitK_Reduction (fp6_llm/csrc/include/kernel_reduction.cuh:28-47).
__global__ void __launch_bounds__(256) splitk_reduce_kernel(__half* __restrict__ out, const float* __restrict__ partials,
                                                            size_t elems, int split_k) {
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= elems) return;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < split_k; s++) {
        const float4 p = *reinterpret_cast<const float4*>(partials + (size_t)s * elems + i);
        acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
    }
    __half2 lo = __floats2half2_rn(acc.x, acc.y), hi = __floats2half2_rn(acc.z, acc.w);
    uint2 packed;
    packed.x = *reinterpret_cast<uint32_t*>(&lo);
    packed.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(out + i) = packed;
}

// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// Tensor map over the activations [N rows][K fp16], box = 64 K x n_tile rows, 128-byte swizzle.
cudaError_t make_act_map(CUtensorMap* map, const __half* act, size_t N, size_t K, int n_tile) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return cudaErrorNotSupported;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)N};
    cuuint64_t strides[1] = {(cuuint64_t)K * sizeof(__half)};
    cuuint32_t box[2] = {(cuuint32_t)kKBlock, (cuuint32_t)n_tile};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(act), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

template <int BW, int N_TILE, bool PARTIAL>
cudaError_t launch_one(cudaStream_t stream, const CUtensorMap& map, const uint8_t* weight, const __half* scales,
                       void* out, size_t M, size_t N, size_t K, int split_k, int* status) {
    auto kernel = fpx_gemm_kernel<BW, N_TILE, PARTIAL>;
    constexpr uint32_t smem = Budget<BW, N_TILE>::smem_bytes;
    static bool configured[64] = {};
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return err;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    dim3 grid((unsigned)(M / kTileM), (unsigned)((N + N_TILE - 1) / N_TILE), (unsigned)split_k);
    kernel<<<grid, kThreads, smem, stream>>>(map, weight, scales, out, (uint32_t)M, (uint32_t)N, (uint32_t)K,
                                             (uint32_t)split_k, status);
    return cudaGetLastError();
}

template <int BW, bool PARTIAL>
cudaError_t launch_by_n(int n_tile, cudaStream_t stream, const CUtensorMap& map, const uint8_t* weight,
                        const __half* scales, void* out, size_t M, size_t N, size_t K, int split_k, int* status) {
    switch (n_tile) {
        case 16:  return launch_one<BW, 16, PARTIAL>(stream, map, weight, scales, out, M, N, K, split_k, status);
        case 32:  return launch_one<BW, 32, PARTIAL>(stream, map, weight, scales, out, M, N, K, split_k, status);
        case 64:  return launch_one<BW, 64, PARTIAL>(stream, map, weight, scales, out, M, N, K, split_k, status);
        case 128: return launch_one<BW, 128, PARTIAL>(stream, map, weight, scales, out, M, N, K, split_k, status);
        default:  return launch_one<BW, 256, PARTIAL>(stream, map, weight, scales, out, M, N, K, split_k, status);
    }
}

}  // namespace

int gemm_n_tile(size_t N) { return N <= 16 ? 16 : (N <= 32 ? 32 : (N <= 64 ? 64 : (N <= 128 ? 128 : 256))); }

int gemm_ctas_per_sm(int n_tile) { return n_tile <= 64 ? 2 : 1; }

cudaError_t launch_splitk_reduce(cudaStream_t stream, __half* out, const float* partials, size_t elems, int split_k) {
    const size_t threads = (elems + 3) / 4;
    splitk_reduce_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(out, partials, elems, split_k);
    return cudaGetLastError();
}

cudaError_t launch_gemm(int e_bits, int m_bits, cudaStream_t stream, const void* weight, const __half* scales,
                        const __half* act, __half* out, size_t M, size_t N, size_t K, float* workspace, int split_k,
                        int* status) {
    if (!format_supported(e_bits, m_bits)) return cudaErrorInvalidValue;
    if (M == 0 || M % 256 != 0 || K == 0 || K % 64 != 0 || N == 0 || split_k < 1 || split_k > 65535)
        return cudaErrorInvalidValue;
    if (!weight || !scales || !act || !out || (split_k > 1 && !workspace)) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(weight) & 15) || (reinterpret_cast<uintptr_t>(act) & 15) ||
        (reinterpret_cast<uintptr_t>(out) & 7) || (reinterpret_cast<uintptr_t>(workspace) & 15))
        return cudaErrorMisalignedAddress;
    if (M > 0xffffffffull || N > 0x7fffffffull || K > 0x7fffffffull) return cudaErrorInvalidValue;
    const int n_tile = gemm_n_tile(N);
    if ((N + n_tile - 1) / n_tile > 65535) return cudaErrorInvalidValue;
    CUtensorMap map;
    cudaError_t err = make_act_map(&map, act, N, K, n_tile);
    if (err != cudaSuccess) return err;
    const uint8_t* w = static_cast<const uint8_t*>(weight);
    const int bw = 1 + e_bits + m_bits;
    if (split_k == 1) {
        return bw == 6 ? launch_by_n<6, false>(n_tile, stream, map, w, scales, out, M, N, K, 1, status)
                       : launch_by_n<5, false>(n_tile, stream, map, w, scales, out, M, N, K, 1, status);
    }
    err = bw == 6 ? launch_by_n<6, true>(n_tile, stream, map, w, scales, workspace, M, N, K, split_k, status)
                  : launch_by_n<5, true>(n_tile, stream, map, w, scales, workspace, M, N, K, split_k, status);
    if (err != cudaSuccess) return err;
    return launch_splitk_reduce(stream, out, workspace, M * N, split_k);
}

}  // namespace fpx
