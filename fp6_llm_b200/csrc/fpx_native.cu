// Weights on the tensor cores' own FP6 inputs (sm_100a): Out[N, M] = Act[N, K] * dequant(W)[M, K]^T for batches of up to 64
// tokens, the decode regime in which the layer is bound by streaming the weights.  e3m2 and e2m3 codes go in as they are;
// the narrower formats (e2m2, e3m1, e2m1) are widened to the six-bit format with the same exponent field when the weights
// are re-laid (their values are a subset of its values), so they stream 6 bits per weight here.
//
// The path of fpx_gemm.cu turns every weight into an fp16 pattern with integer instructions before the MMA
// (as the reference does, fp6_llm/csrc/include/utils_parallel_dequant.cuh:24-63), and those instructions bound it
// below the memory roofline.  Blackwell's tcgen05.mma.kind::f8f6f4 multiplies e3m2 / e2m3 operands directly, and a
// tensor copy of element type "16 x 6 bit" expands densely packed 6-bit codes into the layout that instruction reads
// from shared memory (every 16 codes = 12 bytes, padded to 16).  So here the weights are never touched by a thread:
//
//   weights      re-laid once (native_repack_kernel) from the reference's packed format into tiles of 128 rows x 128 K,
//                each 12 KB contiguous, codes in little-endian bit order; one tensor copy per tile and pipeline stage;
//   activations  the tensor cores need an 8-bit (or narrower) partner, so every fp16 activation goes in as the EXACT sum of
//                four e5m2 numbers, x = p0 + p1/4 + p2/32 + p3/256 (three significant bits each, truncated, the remainder
//                carried on), i.e. as four byte planes.  The planes are the columns of one MMA (N = 4 x tokens), so the four
//                partial products land in four column groups of the accumulator and the epilogue adds them with their
//                weights in fp32.  Every product e3m2 x e5m2 is exact and the sum is accumulated in fp32, as in the fp16
//                path.  Up to 4 tokens the planes are made inside the kernel: converter warps read the fp16
//                activations of a stage [tokens x 128 K] from global memory (one visit ahead, into registers), split them
//                with packed-half arithmetic and write the planes into the stage in the swizzled layout the MMA reads
//                (no kernel before the GEMM); for 5..64 tokens split_activations_kernel writes the
//                planes [4 * tokens][K] beforehand and a tensor copy brings them in;
//   kernel       persistent, one CTA per SM: warp 0 copies weight tiles, warp 1 the activations, warps 2-5 issue
//                the MMAs (four K = 32 steps per stage; up to four warps take the stages in turn, each into its own
//                accumulator; copies and MMAs are issued by whole converged warps with one elected lane, which keeps
//                addresses and descriptors warp-uniform: ~64 cycles for four MMAs and a commit, ~230 from a lone lane),
//                warps 6-9 are the epilogue (two accumulator buffers per issuer, so the epilogue of one segment runs
//                under the main loop of the next), warps 10.. the converters.  Work plan, stream-K partials, fix-up kernel, output targets and
//                fused epilogues are those of fpx_gemm.cu.
//
// Every mbarrier wait is bounded; on a time-out the CTA records a code in the status word, frees its tensor memory
// and returns.
#include <cuda.h>
#include <atomic>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "fpx_internal.h"
#include "fpx_layout.h"
#include "ptx_sm100.cuh"

namespace fpx {

namespace {

constexpr int kNatTileM = 128;                  // rows of a weight tile = M of the MMA
constexpr int kNatTileK = 128;                  // K of a weight tile = one 128-byte swizzle row of shared memory
constexpr int kNatRowBytes = kNatTileK * 6 / 8;        // 96 bytes of HBM per tile row
constexpr int kNatTileBytes = kNatTileM * kNatRowBytes;   // 12 KB of HBM per tile
constexpr uint32_t kNatTileSmem = kNatTileM * 128;     // 16 KB of shared memory per tile (16 codes -> 16 bytes)
constexpr int kPieces = 4;
// Optional milestones of every CTA (build with -DFPX_PROFILE): global-timer stamps read back with
// fp6b200_debug_read_native_stamps.
#ifdef FPX_PROFILE
__device__ unsigned long long g_nat_stamp[160][8];
#define NAT_STAMP(slot) do { if (blockIdx.x < 160) g_nat_stamp[blockIdx.x][slot] = ptx::global_timer_ns(); } while (0)
#else
#define NAT_STAMP(slot) do { } while (0)
#endif
constexpr int kNatFirstIssuer = 2;             // warps 2..5: MMA issue (the first `issuers` of them, one elected lane each)
constexpr int kNatMaxIssuers = 4;
constexpr int kNatFirstEpilogue = kNatFirstIssuer + kNatMaxIssuers;   // warps 6..9: one per tensor-memory lane quadrant
constexpr int kNatFirstConverter = kNatFirstEpilogue + 4;   // warps 10..: split the fp16 activations (fused variant only)
constexpr int kNatMaxTokens = 64;               // 4 x 64 = 256 MMA columns

template <int N_TILE>
struct NatCfg {
    static_assert(N_TILE == 16 || N_TILE == 32 || N_TILE == 64 || N_TILE == 128 || N_TILE == 256, "MMA width");
    static constexpr int tokens = N_TILE / kPieces;
    static constexpr uint32_t b_bytes = N_TILE * 128;
    static constexpr uint32_t stage_bytes = kNatTileSmem + b_bytes;
    // Up to 4 tokens the kernel splits the activations itself: conv_groups converter warps, warp g on the stages g,
    // g + conv_groups, ... (a stage's conversion is a chain of dependent steps, so several stages must be in work at once;
    // all warps on one stage measured 50 % slower than the separate kernel).  With more tokens the separate kernel
    // measured faster (gate_up 57344 x 8192: 64.9 us against 65.7 us at 8 tokens, 66 us against 72 us at 16), whatever the
    // number of converter warps; measured again with the MMAs issued by elected lanes: equal at 8 tokens (57.5 against
    // 58.8 us there, 15.3 against 14.9 us on 10240 x 8192), 3-6 % slower at 16.
    static constexpr bool fused = N_TILE <= 16;
    static constexpr int conv_groups = fused ? 4 : 0;
    static constexpr int conv_width = 1;
    static constexpr int conv_warps = conv_groups * conv_width;
    static constexpr int warps = kNatFirstConverter + conv_warps;
    static constexpr int threads = 32 * warps;
    // issuer i takes the stages i, i + issuers, ... of the CTA's running count and owns two accumulators; three issuers and
    // rings of 12 / 9 stages measured 1-4 % faster than four issuers and 8 stages (more weight bytes in flight)
    static constexpr int issuers = N_TILE <= 16 ? 4 : (N_TILE <= 64 ? 3 : (N_TILE <= 128 ? 2 : 1));
    static constexpr uint32_t ring_budget = 222 * 1024;
    static constexpr int fit = (int)(ring_budget / stage_bytes) < 12 ? (int)(ring_budget / stage_bytes) : 12;
    static constexpr int stages = fit / issuers * issuers;
    static constexpr uint32_t acc_stride = 2 * N_TILE;                        // columns per issuer
    static constexpr uint32_t pow2_at_least(uint32_t x) { uint32_t p = 32; while (p < x) p *= 2; return p; }
    static constexpr uint32_t tmem_cols = pow2_at_least(issuers * acc_stride);
    // an mbarrier wait sees only the parity of the phase: an issuer must meet a slot again on the slot's very next use
    static_assert(stages % issuers == 0, "ring depth must be a multiple of the issuers' stride");
    static_assert(!fused || stages % conv_groups == 0, "ring depth must be a multiple of the converter groups' stride");
    static_assert(tmem_cols <= 512 && (tmem_cols & (tmem_cols - 1)) == 0, "tensor memory");
    static constexpr uint32_t num_barriers = 2 * stages + 4;
    static constexpr uint32_t smem_bytes = stages * stage_bytes + 8 * num_barriers + 16;
    static_assert(stage_bytes % 1024 == 0, "swizzled tiles start on 1024-byte boundaries");
    static_assert(smem_bytes <= 227 * 1024, "shared memory");
};

struct NatParams {
    const __half* scales;
    OutTargets out;
    uint32_t weights_static;
    const __half* bias;
    uint32_t activation;
    float* workspace;           // stream-K partial slots [slot][tokens][128] fp32
    const __half* act;          // fp16 activations [N][K] (read by the converter warps of the fused variant)
    uint32_t M, N, K;           // output channels, tokens, input channels
    uint32_t ktiles;            // ceil(K / 128)
    uint32_t a_format;          // operand format code of the weights (ptx::kFmtE3M2 / kFmtE2M3)
    WorkPlan plan;
    int* status;
};

__device__ __forceinline__ float silu_mul_f(float gate, float up) { return gate / (1.0f + __expf(-gate)) * up; }

template <int N_TILE>
__global__ void __launch_bounds__(NatCfg<N_TILE>::threads, 1)
fpx_native_kernel(const __grid_constant__ CUtensorMap w_map, const __grid_constant__ CUtensorMap x_map,
                  const __grid_constant__ NatParams p) {
    using Cfg = NatCfg<N_TILE>;
    constexpr int S = Cfg::stages;
    constexpr int T = Cfg::tokens;
    constexpr int NI = Cfg::issuers;
    extern __shared__ __align__(1024) uint8_t smem_dyn[];
    const uint32_t ring = ptx::smem_u32(smem_dyn);
    constexpr bool kFused = Cfg::fused;
    constexpr int CW = Cfg::conv_warps;
    const uint32_t full = ring + S * Cfg::stage_bytes;   // per stage: weights and activation planes are in place
    const uint32_t empty = full + 8 * S;                 // per stage: the MMAs that read it are done
    const uint32_t acc_full = empty + 8 * S;             // per accumulator buffer
    const uint32_t acc_empty = acc_full + 16;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem_dyn + S * Cfg::stage_bytes + 8 * Cfg::num_barriers);
    volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_holder + 1);

    // through a shuffle, so that the compiler knows the index to be the same in every lane: the copy and MMA roles are
    // executed by whole warps with one elected lane issuing, which keeps their addresses and descriptors warp-uniform
    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31;
    const uint32_t cta = blockIdx.x;
    const WorkPlan& plan = p.plan;

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the fix-up kernel may become resident
    if (threadIdx.x == 0) NAT_STAMP(0);   // entry
    if ((ring & 1023u) != 0u) {
        if (threadIdx.x == 0) atomicCAS(p.status, 0, kErrSmemAlign);
        return;
    }
    if (warp == 0) {
        for (int i = lane; i < S; i += 32) {
            ptx::mbar_init(full + 8 * i, kFused ? 1 + Cfg::conv_width : 2);   // the weight copy + the stage's converter warps (or the plane copy)
            ptx::mbar_init(empty + 8 * i, 1);
        }
        if (lane < 2) {
            ptx::mbar_init(acc_full + 8 * lane, Cfg::issuers);
            ptx::mbar_init(acc_empty + 8 * lane, 4);
        }
        if (lane == 0) *abort_word = 0;
        ptx::fence_barrier_init();
        if (lane == 0) { ptx::prefetch_tensormap(&w_map); ptx::prefetch_tensormap(&x_map); }
    }
    if (warp == kNatFirstIssuer) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_holder), Cfg::tmem_cols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;
    if (threadIdx.x == 0) NAT_STAMP(1);   // set-up done

    if (warp < 2) {
        // ------------------------------------------------------------ copy producers (a warp each, one elected lane issues)
        // Warp 0: weight tiles; weights declared static are requested before griddepcontrol.wait, i.e. while the
        // previous kernel of the stream may still be running.  (Asking L2 at that point for the 20 tiles that follow the ring's
        // as well - cp.async.bulk.prefetch.L2, 35 MB over the GPU - measured slower, 12.1 -> 12.5 us on 8192 x 8192 at one
        // token and 32.8 -> 36.1 us on 8192 x 28672 at 16: the memory system is already busy filling the rings and
        // finishing the previous layer in that window.)  Warp 1: the activation planes, which the split
        // kernel just before this one writes, always after the wait.
        {
            const bool acts = warp == 1;
            const uint64_t pol = acts ? ptx::policy_evict_last() : ptx::policy_evict_first();
            bool waited = !acts && p.weights_static != 0;
            ptx::RingPos<S> pos;
            pos.set(0);
            uint32_t issued = 0;
            bool ok = !(kFused && acts);     // the fused variant has no activation copies: its converter warps read them
            SegmentIter iter;
            Segment seg;
            plan_start(plan, cta, &iter);
            while (ok && plan_next(plan, cta, &iter, &seg)) {
                uint32_t kt = plan_first_stage(plan, cta, seg.nkb);
                for (uint32_t i = 0; i < seg.nkb; i++) {
                    const uint32_t k_tile = seg.kb_begin + kt;
                    kt = kt + 1 == seg.nkb ? 0u : kt + 1;
                    if (!ptx::mbar_wait_warp(empty + 8 * pos.idx, pos.lap ^ 1u, abort_word, kErrStageEmpty, 100)) { ok = false; break; }
                    if (!waited) {
                        asm volatile("griddepcontrol.wait;" ::: "memory");
                        waited = true;
                    }
                    const uint32_t bar = full + 8 * pos.idx;
                    const uint32_t dst = ring + pos.idx * Cfg::stage_bytes;
                    const int32_t w_row = (int32_t)((seg.tile * p.ktiles + k_tile) * kNatTileM);
                    if (ptx::elect_one()) {
                        if (acts) {
                            ptx::mbar_arrive_expect_tx(bar, Cfg::b_bytes);
                            ptx::tma_load_2d(dst + kNatTileSmem, &x_map, (int32_t)(k_tile * kNatTileK), 0, bar, pol);
                        } else {
                            // the transaction count of a 6-bit copy is the bytes read from global memory
                            ptx::mbar_arrive_expect_tx(bar, (uint32_t)kNatTileBytes);
                            ptx::tma_load_2d(dst, &w_map, 0, w_row, bar, pol);
                        }
                    }
                    __syncwarp();
                    pos.advance(1);
                    issued++;
                }
            }
            if (*abort_word != 0) {   // gave up somewhere: let the copies in flight land before leaving
                const uint32_t first = issued > (uint32_t)S ? issued - S : 0u;
                for (uint32_t t = first; t < issued; t++)
                    ptx::mbar_wait_warp(full + 8 * (t % S), (t / S) & 1u, abort_word, kErrStageFull, 100, 50000000ull);
            }
        }
        __syncwarp();
    } else if (warp < kNatFirstEpilogue) {
        // ------------------------------------------------------------ MMA issue
        const uint32_t me = (uint32_t)(warp - kNatFirstIssuer);
        if (me < (uint32_t)NI) {   // the whole warp, converged
            const uint32_t idesc = ptx::idesc_f8f6f4_f32(p.a_format, ptx::kFmtE5M2, kNatTileM, N_TILE);
            const uint64_t desc0 = ptx::smem_desc_k_sw128(ring);
            uint32_t j0 = 0, nseg = 0;   // stages before this segment, segments so far
            bool ok = true;
            SegmentIter iter;
            Segment seg;
            plan_start(plan, cta, &iter);
            while (ok && plan_next(plan, cta, &iter, &seg)) {
                const uint32_t buf = nseg & 1u;
                if (!ptx::mbar_wait_warp(acc_empty + 8 * buf, ((nseg >> 1) & 1u) ^ 1u, abort_word, kErrAccEmpty)) { ok = false; break; }
                ptx::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + me * Cfg::acc_stride + buf * N_TILE;
                uint32_t accumulate = 0u;
                uint32_t t = (me + NI - (j0 % NI)) % NI;     // my first stage of the segment
                ptx::RingPos<S> pos;
                pos.set(j0 + t);
                for (; t < seg.nkb; t += NI) {
                    if (!ptx::mbar_wait_warp(full + 8 * pos.idx, pos.lap, abort_word, kErrStageFull)) { ok = false; break; }
                    if (me == 0 && lane == 0 && nseg == 0 && accumulate == 0u) NAT_STAMP(2);   // first stage in place
                    ptx::tc_fence_after_sync();
                    const uint64_t a_desc = desc0 + (uint64_t)(pos.idx * (Cfg::stage_bytes >> 4));
                    const uint64_t b_desc = a_desc + (kNatTileSmem >> 4);
#pragma unroll
                    for (uint32_t kk = 0; kk < 4; kk++) {   // four K = 32 steps: 32 bytes further inside the swizzle row
                        ptx::mma_f8f6f4_ss_elect(d_tmem, a_desc + kk * 2, b_desc + kk * 2, idesc, accumulate);
                        accumulate = 1u;
                    }
                    ptx::tc_commit_elect(empty + 8 * pos.idx);
                    pos.advance(NI);
                }
                if (!ok) break;
                ptx::tc_commit_elect(acc_full + 8 * buf);   // arrives once this issuer's MMAs (if any) are done
                if (me == 0 && lane == 0) NAT_STAMP(3);   // last commit of a segment issued
                j0 += seg.nkb;
                nseg++;
            }
        }
        __syncwarp();
    } else if (warp >= kNatFirstConverter) {
        // ------------------------------------------------------------ converters (fused variant): fp16 tile -> four e5m2 planes
        // Every converter warp works on every stage: a thread takes chunks of 8 consecutive K of one token (16 bytes of the
        // fp16 tile).  p0 = x with the mantissa cut to two bits (the upper byte of the pattern); the remainder x - p0 is
        // exact in fp16, and so is 4 x it; the same step gives p1, p2 and p3 (scales 4, 8, 8), after which nothing is
        // left: 11 significant bits fit into 3 + 3 + 3 + 3.  Bytes go to row piece * tokens + token of the stage's
        // activation tile, 128 bytes per row with the 16-byte units of a row XOR-swizzled by the row (the 128-byte
        // swizzle the MMA descriptor names).  Tokens past N arrive as zeros from the copy and give zero planes.
        if constexpr (kFused) {
            constexpr uint32_t CG = Cfg::conv_groups, WD = Cfg::conv_width;
            const uint32_t grp = (uint32_t)(warp - kNatFirstConverter) / WD, sub = (uint32_t)(warp - kNatFirstConverter) % WD;
            constexpr uint32_t kChunks = T * 16;                       // 16-byte chunks of a stage's activations
            constexpr uint32_t kPerLane = (kChunks + WD * 32 - 1) / (WD * 32);
            const __half2 four = __float2half2_rn(4.0f), eight = __float2half2_rn(8.0f);
            const uint64_t keep = ptx::policy_evict_last();
            // The group's stages in the CTA's running count are grp, grp + CG, ...  A cursor walks the plan to the K tile
            // of each; the activations of the NEXT visit are requested before those of this visit are converted.
            SegmentIter iter;
            Segment seg;
            plan_start(plan, cta, &iter);
            bool have = plan_next(plan, cta, &iter, &seg);
            uint32_t in_seg = grp;                                      // index of the cursor's stage inside its segment
            auto settle = [&]() {                                       // move the cursor into the segment that holds its stage
                while (have && in_seg >= seg.nkb) {
                    in_seg -= seg.nkb;
                    have = plan_next(plan, cta, &iter, &seg);
                }
            };
            auto request = [&](uint4 (&dst)[kPerLane]) {                // loads of the cursor's stage
                uint32_t kt = plan_first_stage(plan, cta, seg.nkb) + in_seg;
                if (kt >= seg.nkb) kt -= seg.nkb;
                const uint32_t k0 = (seg.kb_begin + kt) * kNatTileK;
#pragma unroll
                for (uint32_t c = 0; c < kPerLane; c++) {
                    const uint32_t chunk = (c * WD + sub) * 32 + lane;
                    const uint32_t token = chunk >> 4, k = k0 + (chunk & 15u) * 8;
                    dst[c] = make_uint4(0u, 0u, 0u, 0u);
                    if (chunk < kChunks && token < p.N && k < p.K)      // K is a multiple of 8: a chunk is inside or outside
                        asm volatile("ld.global.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;"   // keep them in L2 under the weight stream
                                     : "=r"(dst[c].x), "=r"(dst[c].y), "=r"(dst[c].z), "=r"(dst[c].w)
                                     : "l"(p.act + (size_t)token * p.K + k), "l"(keep));
                }
            };
            uint4 cur[kPerLane], nxt[kPerLane];
            asm volatile("griddepcontrol.wait;" ::: "memory");          // the activations may come from the previous kernel
            settle();
            if (have) request(nxt);
            uint32_t j = grp;                                           // running stage index of the visit
            bool ok = true;
            bool visit = have;                                          // the cursor's stage exists and its loads are in nxt
            while (ok && visit) {
#pragma unroll
                for (uint32_t c = 0; c < kPerLane; c++) cur[c] = nxt[c];
                in_seg += CG;
                settle();
                const bool more = have;
                if (more) request(nxt);
                // convert first (into registers), then wait for the stage: in the steady state every stage of the ring is in
                // flight and a stage is handed back only every ~300 ns, so whatever follows that wait delays the stage
                uint32_t plane[kPerLane][kPieces][2];
#pragma unroll
                for (uint32_t c = 0; c < kPerLane; c++) {
                    const uint32_t h[4] = {cur[c].x, cur[c].y, cur[c].z, cur[c].w};
                    uint32_t pc[kPieces][4];
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        uint32_t x = h[e];
                        pc[0][e] = x;
#pragma unroll
                        for (int s = 1; s < kPieces; s++) {
                            const uint32_t top = x & 0xff00ff00u;
                            __half2 r = __hsub2(*reinterpret_cast<__half2*>(&x), *reinterpret_cast<const __half2*>(&top));
                            r = __hmul2(r, s == 1 ? four : eight);
                            x = *reinterpret_cast<uint32_t*>(&r);
                            pc[s][e] = x;
                        }
                    }
#pragma unroll
                    for (int s = 0; s < kPieces; s++) {   // the upper bytes of the eight values, in K order
                        plane[c][s][0] = __byte_perm(pc[s][0], pc[s][1], 0x7531);
                        plane[c][s][1] = __byte_perm(pc[s][2], pc[s][3], 0x7531);
                    }
                }
                ptx::RingPos<S> pos;
                pos.set(j);
                if (!ptx::mbar_wait_warp(empty + 8 * pos.idx, pos.lap ^ 1u, abort_word, kErrStageEmpty, 40)) { ok = false; break; }
                const uint32_t b_tile = ring + pos.idx * Cfg::stage_bytes + kNatTileSmem;
#pragma unroll
                for (uint32_t c = 0; c < kPerLane; c++) {
                    const uint32_t chunk = (c * WD + sub) * 32 + lane;
                    if (chunk >= kChunks) continue;
                    const uint32_t token = chunk >> 4, k8 = chunk & 15u;       // K = 8 * k8 .. 8 * k8 + 7 of the stage
#pragma unroll
                    for (int s = 0; s < kPieces; s++) {
                        const uint32_t row = (uint32_t)s * T + token;
                        const uint32_t addr = b_tile + row * 128 + (((k8 >> 1) ^ (row & 7u)) << 4) + ((k8 & 1u) << 3);
                        asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(addr), "r"(plane[c][s][0]), "r"(plane[c][s][1]) : "memory");
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the MMA reads shared memory through the async proxy
                __syncwarp();
                ptx::mbar_arrive_elected(full + 8 * pos.idx);
                j += CG;
                visit = more;
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue: one warp per tensor-memory lane quadrant
        const int q = warp & 3;
        asm volatile("griddepcontrol.wait;" ::: "memory");   // before the scales are read and anything is stored
        uint32_t nseg = 0, j0 = 0;
        bool ok = true;
        SegmentIter iter;
        Segment seg;
        plan_start(plan, cta, &iter);
        // weights of the four planes: x = p0 + p1 / 4 + p2 / 32 + p3 / 256
        constexpr float kW1 = 0.25f, kW2 = 0.03125f, kW3 = 0.00390625f;
        while (ok && plan_next(plan, cta, &iter, &seg)) {
            const uint32_t buf = nseg & 1u;
            const uint32_t row_in_tile = 32u * q + lane;
            const uint32_t row = seg.tile * kNatTileM + row_in_tile;
            // the hardware reads e3m2 with exponent bias 3 and e2m3 with bias 1, which are the values the reference gives the codes
            // (pattern * 2^(16 - 2^(E-1)), fp6_llm/csrc/utils/weight_dequant.h:30-43): no factor besides the row scale
            const float row_scale = __half2float(p.scales[row]);
            const float row_bias = p.bias ? __half2float(p.bias[row]) : 0.0f;
            if (!ptx::mbar_wait_warp(acc_full + 8 * buf, (nseg >> 1) & 1u, abort_word, kErrAccFull)) { ok = false; break; }
            ptx::tc_fence_after_sync();
            const uint32_t acc = tmem_base + ((uint32_t)(32 * q) << 16) + buf * N_TILE;
            // issuers that took at least one stage of this segment (the others' accumulators hold nothing of it)
            uint32_t has_data = 0;
#pragma unroll
            for (uint32_t i = 0; i < (uint32_t)NI; i++)
                has_data |= ((i + NI - (j0 % NI)) % NI < seg.nkb ? 1u : 0u) << i;
            j0 += seg.nkb;
            constexpr int CH = T < 16 ? T : 16;   // tokens handled per round
#pragma unroll 1
            for (int t0 = 0; t0 < T; t0 += CH) {
                if ((uint32_t)t0 >= p.N) break;
                float f[CH];
#pragma unroll
                for (int u = 0; u < CH; u++) f[u] = 0.0f;
#pragma unroll
                for (uint32_t i = 0; i < (uint32_t)NI; i++) {
                    if (!((has_data >> i) & 1u)) continue;
                    const uint32_t a = acc + i * Cfg::acc_stride;
                    if constexpr (N_TILE == 16) {
                        uint32_t v[16];
                        ptx::tmem_ld_cols<16>(a, v);
                        ptx::tc_wait_ld();
#pragma unroll
                        for (int u = 0; u < 4; u++)
                            f[u] += __uint_as_float(v[u]) + kW1 * __uint_as_float(v[4 + u]) + kW2 * __uint_as_float(v[8 + u]) +
                                    kW3 * __uint_as_float(v[12 + u]);
                    } else if constexpr (N_TILE == 32) {
                        uint32_t va[16], vb[16];
                        ptx::tmem_ld_cols<16>(a, va);
                        ptx::tmem_ld_cols<16>(a + 16, vb);
                        ptx::tc_wait_ld();
#pragma unroll
                        for (int u = 0; u < 8; u++)
                            f[u] += __uint_as_float(va[u]) + kW1 * __uint_as_float(va[8 + u]) + kW2 * __uint_as_float(vb[u]) +
                                    kW3 * __uint_as_float(vb[8 + u]);
                    } else {
                        uint32_t v[16];
                        ptx::tmem_ld_cols<16>(a + t0, v);
                        ptx::tc_wait_ld();
#pragma unroll
                        for (int u = 0; u < 16; u++) f[u] += __uint_as_float(v[u]);
                        ptx::tmem_ld_cols<16>(a + T + t0, v);
                        ptx::tc_wait_ld();
#pragma unroll
                        for (int u = 0; u < 16; u++) f[u] += kW1 * __uint_as_float(v[u]);
                        ptx::tmem_ld_cols<16>(a + 2 * T + t0, v);
                        ptx::tc_wait_ld();
#pragma unroll
                        for (int u = 0; u < 16; u++) f[u] += kW2 * __uint_as_float(v[u]);
                        ptx::tmem_ld_cols<16>(a + 3 * T + t0, v);
                        ptx::tc_wait_ld();
#pragma unroll
                        for (int u = 0; u < 16; u++) f[u] += kW3 * __uint_as_float(v[u]);
                    }
                }
                const uint32_t n0 = (uint32_t)t0;
                if (seg.out_kind == kOutDirect) {
#pragma unroll
                    for (int u = 0; u < CH; u++) f[u] = f[u] * row_scale + row_bias;
                    if (p.activation == kActSiluMul) {
                        // rows 2c (gate) and 2c+1 (up) sit in neighbouring lanes: the even lane stores channel c
#pragma unroll
                        for (int u = 0; u < CH; u++) {
                            const float up = __shfl_xor_sync(0xffffffffu, f[u], 1);
                            f[u] = silu_mul_f(f[u], up);
                        }
                        if ((lane & 1) == 0) {
                            __half* dst = p.out.ptr[0] + (size_t)n0 * p.out.ld + p.out.row0 + (row >> 1);
#pragma unroll
                            for (int u = 0; u < CH; u++)
                                if (n0 + u < p.N) dst[(size_t)u * p.out.ld] = __float2half_rn(f[u]);
                        }
                    } else {
                        const size_t first = (size_t)n0 * p.out.ld + p.out.row0 + row;
#pragma unroll 1
                        for (uint32_t r = 0; r < p.out.count; r++) {   // one target, or the buffer of every rank
                            __half* dst = p.out.ptr[r] + first;
#pragma unroll
                            for (int u = 0; u < CH; u++)
                                if (n0 + u < p.N) dst[(size_t)u * p.out.ld] = __float2half_rn(f[u]);
                        }
                    }
                } else {   // part of a tile: fp32, scaled, into this CTA's slot [tokens][128]
                    float* dst = p.workspace + ((size_t)seg.out_index * T + t0) * kNatTileM + row_in_tile;
#pragma unroll
                    for (int u = 0; u < CH; u++)
                        if (n0 + u < p.N) dst[u * kNatTileM] = f[u] * row_scale;
                }
            }
            ptx::tc_fence_before_sync();
            __syncwarp();
            ptx::mbar_arrive_elected(acc_empty + 8 * buf);
            if (warp == kNatFirstEpilogue && lane == 0) NAT_STAMP(4);   // epilogue of a segment done
            nseg++;
        }
    }

    // ------------------------------------------------------------ teardown
    if (threadIdx.x == 0) NAT_STAMP(5);   // roles done
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == kNatFirstIssuer) {
        if (*abort_word != 0 && lane == 0) {   // gave up: let MMAs that may still be in flight finish before freeing
            const uint64_t t0 = ptx::global_timer_ns();
            while (ptx::global_timer_ns() - t0 < 2000000ull) { }
        }
        __syncwarp();
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, Cfg::tmem_cols);
    }
    if (threadIdx.x == 0 && *abort_word != 0) atomicCAS(p.status, 0, *abort_word);
    if (threadIdx.x == 0) NAT_STAMP(6);   // exit
}

// ------------------------------------------------------------------------------------------------
// fp16 activations [N][K] -> four planes of e5m2 bytes, row (piece * tokens + n) of [4 * tokens][kpad]:
// x = p0 + p1 / 4 + p2 / 32 + p3 / 256 exactly.  p0 is x truncated to three significant bits (the upper byte of the
// fp16 pattern); each further plane is the remainder, scaled, truncated the same way.  Eleven significant bits fit
// into 3 + 3 + 3 + 3; the scales keep every remainder inside the range of fp16 (and of e5m2, whose exponent range is
// the same), subnormals included.  Rows past N and columns past K are zero.  An infinite or NaN activation makes all
// four planes NaN or infinite, and the output NaN.
__global__ void __launch_bounds__(256) split_activations_kernel(const __half* __restrict__ act, uint8_t* __restrict__ planes,
                                                                uint32_t N, uint32_t K, uint32_t tokens, uint32_t kpad) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t chunks = kpad / 8;
    const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= tokens * chunks) return;
    const uint32_t n = idx / chunks, k0 = (idx - n * chunks) * 8;
    asm volatile("griddepcontrol.wait;" ::: "memory");   // the activations may come from the previous kernel
    uint32_t raw[4] = {0u, 0u, 0u, 0u};
    if (n < N && k0 < K) {   // K is a multiple of 8
        const uint4 v = *reinterpret_cast<const uint4*>(act + (size_t)n * K + k0);
        raw[0] = v.x; raw[1] = v.y; raw[2] = v.z; raw[3] = v.w;
    }
    uint32_t out[kPieces][2] = {{0u, 0u}, {0u, 0u}, {0u, 0u}, {0u, 0u}};
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const uint32_t h = (raw[i >> 1] >> (16 * (i & 1))) & 0xffffu;
        const float x = __half2float(__ushort_as_half((unsigned short)h));
        const uint32_t b0 = h >> 8;
        const float r1 = (x - __half2float(__ushort_as_half((unsigned short)(h & 0xff00u)))) * 4.0f;
        const uint32_t h1 = __half_as_ushort(__float2half_rn(r1));
        const float r2 = (r1 - __half2float(__ushort_as_half((unsigned short)(h1 & 0xff00u)))) * 8.0f;
        const uint32_t h2 = __half_as_ushort(__float2half_rn(r2));
        const float r3 = (r2 - __half2float(__ushort_as_half((unsigned short)(h2 & 0xff00u)))) * 8.0f;
        const uint32_t h3 = __half_as_ushort(__float2half_rn(r3));
        const int sh = 8 * (i & 3);
        out[0][i >> 2] |= b0 << sh;
        out[1][i >> 2] |= (h1 >> 8) << sh;
        out[2][i >> 2] |= (h2 >> 8) << sh;
        out[3][i >> 2] |= (h3 >> 8) << sh;
    }
#pragma unroll
    for (int pc = 0; pc < kPieces; pc++)
        *reinterpret_cast<uint2*>(planes + (size_t)(pc * tokens + n) * kpad + k0) = make_uint2(out[pc][0], out[pc][1]);
}

// ------------------------------------------------------------------------------------------------
// Reference-packed weights -> native tiles.  A warp takes the 32 rows x 64 columns one unpack warp of the fp16 path
// handles (same words, same unpack sequence), recovers the codes from the fp16 patterns (widened to six bits), gathers
// them in shared memory and writes every 16 codes of a row as 12 bytes, code i at bits 6 i .. 6 i + 5.
template <int E_BITS, int M_BITS>
__global__ void __launch_bounds__(128) native_repack_kernel(const uint8_t* __restrict__ packed, uint8_t* __restrict__ native,
                                                            uint32_t M, uint32_t K, uint32_t ktiles) {
    constexpr int BW = 1 + E_BITS + M_BITS;
    static_assert(BW <= 6, "codes of at most six bits");
    __shared__ uint8_t codes[4][32][64 + 4];
    const uint32_t kblocks = K / kKBlock;
    const int w = threadIdx.x >> 5;
    const uint32_t unit = blockIdx.x * 4 + w;     // (64-row block, k-block, half)
    const bool live = unit < (M / kRowsPerBlock) * kblocks * 2;
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int h = unit & 1;
    const uint32_t kb = (unit >> 1) % kblocks, i = (unit >> 1) / kblocks;
    if (live) {
        const uint64_t tile = (uint64_t)i * kblocks + kb;
        const uint32_t* r1 = reinterpret_cast<const uint32_t*>(packed + region_offset(BW, 1, M, K) + tile * tile_bytes(1));
        const uint32_t* r2 = reinterpret_cast<const uint32_t*>(packed + region_offset(BW, 2, M, K) + tile * tile_bytes(2));
        const uint32_t* r4 = reinterpret_cast<const uint32_t*>(packed + region_offset(BW, 4, M, K) + tile * tile_bytes(4));
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
                    const int row = 16 * kk + 8 * (a & 1) + g;
                    const int col = 16 * j + 8 * (a >> 1) + 2 * t;
                    const uint32_t v = pat[4 * kk + a];
                    // pattern = sign | (exponent, mantissa) >> (5 - E): exponent and mantissa are the E + M bits from bit
                    // 10 - M up.  The six-bit code of the same value in the hardware format with E exponent bits (e3m2
                    // or e2m3) has the same fields with the mantissa extended by zeros: shift left by 5 - E - M.
                    constexpr int sh = 10 - M_BITS, ext = 5 - E_BITS - M_BITS;
                    constexpr uint32_t mask = (1u << (E_BITS + M_BITS)) - 1u;
                    codes[w][row][col] = (uint8_t)(((v >> 10) & 0x20u) | (((v >> sh) & mask) << ext));
                    codes[w][row][col + 1] = (uint8_t)(((v >> 26) & 0x20u) | (((v >> (16 + sh)) & mask) << ext));
                }
        }
    }
    __syncwarp();
    if (live) {
        // 32 rows x 4 groups of 16 codes: four groups per lane
#pragma unroll
        for (int s = 0; s < 4; s++) {
            const int grp = s * 32 + lane;
            const int row = grp >> 2, c0 = (grp & 3) * 16;
            uint32_t words[3] = {0u, 0u, 0u};
#pragma unroll
            for (int c = 0; c < 16; c++) {
                const uint32_t code = codes[w][row][c0 + c];
                const int bit = 6 * c;
                words[bit >> 5] |= code << (bit & 31);
                if ((bit & 31) > 26) words[(bit >> 5) + 1] |= code >> (32 - (bit & 31));
            }
            const uint32_t grow = i * kRowsPerBlock + 32 * h + row;       // global row
            const uint32_t gcol = kb * kKBlock + c0;                      // global column
            const size_t tile = (size_t)(grow / kNatTileM) * ktiles + gcol / kNatTileK;
            uint8_t* dst = native + (tile * kNatTileM + grow % kNatTileM) * kNatRowBytes + (gcol % kNatTileK) * 6 / 8;
            uint32_t* d32 = reinterpret_cast<uint32_t*>(dst);
            d32[0] = words[0]; d32[1] = words[1]; d32[2] = words[2];
        }
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn native_encode_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<EncodeTiledFn>(ptr);
    }();
    return fn;
}

template <int N_TILE>
cudaError_t launch_native_one(cudaStream_t stream, const CUtensorMap& w_map, const CUtensorMap& x_map, const NatParams& prm) {
    auto kernel = fpx_native_kernel<N_TILE>;
    constexpr uint32_t smem = NatCfg<N_TILE>::smem_bytes;
    static std::atomic<bool> configured[64];
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 0 || dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
        err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return err;
        if (dev >= 0 && dev < 64) configured[dev].store(true, std::memory_order_release);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(prm.plan.grid);
    cfg.blockDim = dim3(NatCfg<N_TILE>::threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = programmatic_launch() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, w_map, x_map, prm);
}

}  // namespace

// Every format the library takes has its values among those of a six-bit tensor-core format with the same exponent width
// and bias: e3m2 and e2m3 as they are, e3m1 inside e3m2, e2m2 and e2m1 inside e2m3 (mantissa extended by zero bits).
bool native_format(int e_bits, int m_bits) { return format_supported(e_bits, m_bits); }
int native_max_tokens() { return kNatMaxTokens; }
int native_n_tile(size_t N) { return N <= 4 ? 16 : (N <= 8 ? 32 : (N <= 16 ? 64 : (N <= 32 ? 128 : 256))); }
static size_t native_ktiles(size_t K) { return (K + kNatTileK - 1) / kNatTileK; }

size_t native_weight_bytes(size_t M, size_t K) { return (M / kNatTileM) * native_ktiles(K) * (size_t)kNatTileBytes; }

// planes [4 * tokens][kpad] bytes (rounded up to 256), then the stream-K slots: two per CTA of [tokens][128] fp32
static size_t native_planes_bytes(size_t N, size_t K) {
    const size_t b = (size_t)native_n_tile(N) * native_ktiles(K) * kNatTileK;
    return (b + 255) & ~(size_t)255;
}
size_t native_workspace_bytes(size_t N, size_t K) {
    const size_t ctas = device_sm_count() < 256 ? device_sm_count() : 256;
    return native_planes_bytes(N, K) + 2 * ctas * kNatTileM * (native_n_tile(N) / kPieces) * sizeof(float);
}

cudaError_t launch_native_repack(int e_bits, int m_bits, cudaStream_t stream, const void* packed, void* native, size_t M, size_t K) {
    if (!native_format(e_bits, m_bits) || !packed || !native || packed == native) return cudaErrorInvalidValue;
    if (M == 0 || M % 256 != 0 || K == 0 || K % 64 != 0 || M > 0x7fffffffull || K > 0x7fffffffull) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(packed) & 3) || (reinterpret_cast<uintptr_t>(native) & 15)) return cudaErrorMisalignedAddress;
    const size_t ktiles = native_ktiles(K);
    if (K % kNatTileK != 0) {   // the last K tile is half empty: code 0 is +0
        cudaError_t err = cudaMemsetAsync(native, 0, native_weight_bytes(M, K), stream);
        if (err != cudaSuccess) return err;
    }
    const size_t units = (M / kRowsPerBlock) * (K / kKBlock) * 2;
    const size_t blocks = (units + 3) / 4;
    if (blocks > 0x7fffffffull) return cudaErrorInvalidValue;
    const uint8_t* in = static_cast<const uint8_t*>(packed);
    uint8_t* out = static_cast<uint8_t*>(native);
    FPX_DISPATCH_FORMAT(e_bits, m_bits, (native_repack_kernel<kE, kM><<<(unsigned)blocks, 128, 0, stream>>>(in, out, (uint32_t)M, (uint32_t)K, (uint32_t)ktiles)));
    return cudaGetLastError();
}

cudaError_t launch_native_gemm(int e_bits, int m_bits, cudaStream_t stream, const void* weight_native, const __half* scales,
                               const __half* act, __half* out, size_t M, size_t N, size_t K, void* workspace, int* status,
                               const OutTargets* targets, const Epilogue* epilogue) {
    if (!native_format(e_bits, m_bits)) return cudaErrorInvalidValue;
    const __half* bias = epilogue ? epilogue->bias : nullptr;
    const int activation = epilogue ? epilogue->activation : kActNone;
    if (activation != kActNone && activation != kActSiluMul) return cudaErrorInvalidValue;
    if (activation != kActNone && targets) return cudaErrorInvalidValue;
    if (bias && (reinterpret_cast<uintptr_t>(bias) & 1)) return cudaErrorMisalignedAddress;
    if (M == 0 || M % 256 != 0 || K == 0 || K % 64 != 0 || N == 0 || N > (size_t)kNatMaxTokens) return cudaErrorInvalidValue;
    if (M > 0x7fffffffull || K > 0x7fffffffull) return cudaErrorInvalidValue;
    OutTargets where;
    if (targets) {
        where = *targets;
        if (where.count == 0 || where.count > (uint32_t)kMaxOutTargets) return cudaErrorInvalidValue;
        if (where.ld % 4 != 0 || where.row0 % 4 != 0 || (size_t)where.row0 + M > where.ld) return cudaErrorInvalidValue;
        for (uint32_t t = 0; t < where.count; t++) {
            if (!where.ptr[t]) return cudaErrorInvalidValue;
            if (reinterpret_cast<uintptr_t>(where.ptr[t]) & 7) return cudaErrorMisalignedAddress;
        }
        out = where.ptr[0];
    } else {
        where.ptr[0] = out;
        where.count = 1;
        where.ld = (uint32_t)(activation == kActSiluMul ? M / 2 : M);
        where.row0 = 0;
    }
    if (!weight_native || !scales || !act || !out || !workspace) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(weight_native) & 15) || (reinterpret_cast<uintptr_t>(act) & 15) ||
        (reinterpret_cast<uintptr_t>(out) & 7) || (reinterpret_cast<uintptr_t>(workspace) & 255))
        return cudaErrorMisalignedAddress;
    EncodeTiledFn enc = native_encode_fn();
    if (!enc) return cudaErrorNotSupported;

    const int n_tile = native_n_tile(N);
    const int tokens = n_tile / kPieces;
    const bool fused = n_tile <= 16;      // NatCfg<n_tile>::fused: the kernel splits the activations itself
    const size_t ktiles = native_ktiles(K);
    const size_t kpad = ktiles * kNatTileK;
    uint8_t* planes = static_cast<uint8_t*>(workspace);
    float* slots = reinterpret_cast<float*>(planes + native_planes_bytes(N, K));

    CUtensorMap w_map, x_map;
    {
        // the tiles as one tall matrix of 128 codes per row: a box of 128 x 128 is one tile, 12 KB contiguous
        cuuint64_t dims[2] = {(cuuint64_t)kNatTileK, (cuuint64_t)((M / kNatTileM) * ktiles * kNatTileM)};
        cuuint64_t strides[1] = {(cuuint64_t)kNatRowBytes};
        cuuint32_t box[2] = {(cuuint32_t)kNatTileK, (cuuint32_t)kNatTileM};
        cuuint32_t es[2] = {1, 1};
        if (dims[1] > 0xffffffffull) return cudaErrorInvalidValue;
        CUresult r = enc(&w_map, CU_TENSOR_MAP_DATA_TYPE_16U6_ALIGN16B, 2, const_cast<void*>(weight_native), dims, strides, box, es,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
        if (fused) {
            x_map = w_map;   // not used: the converter warps read the activations themselves
        } else {
            cuuint64_t xdims[2] = {(cuuint64_t)kpad, (cuuint64_t)n_tile};
            cuuint64_t xstrides[1] = {(cuuint64_t)kpad};
            cuuint32_t xbox[2] = {(cuuint32_t)kNatTileK, (cuuint32_t)n_tile};
            r = enc(&x_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, planes, xdims, xstrides, xbox, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        }
        if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    }
    // 1. the activation planes
    if (!fused) {
        const size_t threads = (size_t)tokens * (kpad / 8);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)((threads + 255) / 256));
        cfg.blockDim = dim3(256);
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = programmatic_launch() ? 1 : 0;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cudaError_t err = cudaLaunchKernelEx(&cfg, split_activations_kernel, act, planes, (uint32_t)N, (uint32_t)K, (uint32_t)tokens,
                                             (uint32_t)kpad);
        if (err != cudaSuccess) return err;
    }
    // 2. the GEMM
    const int sms = device_sm_count() < 256 ? device_sm_count() : 256;
    NatParams prm;
    prm.scales = scales;
    prm.out = where;
    prm.weights_static = (uint32_t)weights_static();
    prm.bias = bias;
    prm.activation = (uint32_t)activation;
    prm.workspace = slots;
    prm.act = act;
    prm.M = (uint32_t)M;
    prm.N = (uint32_t)N;
    prm.K = (uint32_t)K;
    prm.ktiles = (uint32_t)ktiles;
    prm.a_format = e_bits == 3 ? ptx::kFmtE3M2 : ptx::kFmtE2M3;
    prm.status = status;
    make_plan(M, 1, ktiles * kKBlock, 0, sms, &prm.plan);   // units of the plan = K tiles
    cudaError_t err;
    switch (n_tile) {
        case 16:  err = launch_native_one<16>(stream, w_map, x_map, prm); break;
        case 32:  err = launch_native_one<32>(stream, w_map, x_map, prm); break;
        case 64:  err = launch_native_one<64>(stream, w_map, x_map, prm); break;
        case 128: err = launch_native_one<128>(stream, w_map, x_map, prm); break;
        default:  err = launch_native_one<256>(stream, w_map, x_map, prm); break;
    }
    if (err != cudaSuccess) return err;
    // 3. the sum of the split tiles
    return launch_streamk_fixup(stream, where, slots, N, tokens, prm.plan, epilogue);
}

int native_kernel_launches(size_t M, size_t N, size_t K) {
    if (M == 0 || M % 256 != 0 || K == 0 || K % 64 != 0 || N == 0 || N > (size_t)kNatMaxTokens) return 0;
    const int sms = device_sm_count() < 256 ? device_sm_count() : 256;
    WorkPlan plan;
    make_plan(M, 1, native_ktiles(K) * kKBlock, 0, sms, &plan);
    return (native_n_tile(N) <= 16 ? 1 : 2) + (plan_rem_tiles(plan) ? 1 : 0);
}

}  // namespace fpx

#ifdef FPX_PROFILE
extern "C" int fp6b200_debug_read_native_stamps(unsigned long long* host_out) {
    return cudaMemcpyFromSymbol(host_out, fpx::g_nat_stamp, sizeof(fpx::g_nat_stamp));
}
#endif
