// FPx x fp16 linear layer for sm_100a:  Out[N, M] = Act[N, K] * dequant(W)[M, K]^T, for every format the library takes
// (e3m2, e2m2, e2m1, e3m1, e2m3) and any batch size, on weights in the reference's packed layout.
//
// Replaces the reference's QUANT_GEMM_Kernel + launcher
// (fp6_llm/csrc/include/kernel_matmul.cuh:29-191, fp6_llm/csrc/fp6_linear.cu:11-102) with a persistent,
// warp-specialised kernel built around Blackwell's tensor memory.  One CTA per SM walks a list of
// segments (output tile 128 x N_TILE, range of 64-wide K blocks; see WorkPlan in fpx_layout.h):
//
//   warps 4-5   fill a shared-memory ring with the packed weight segments, one stage = 128 rows x 256 K (128 K / 64 K
//               for the 128- / 256-wide tile): warp 4 the tile's first 64-row block, warp 5 the second, 1-D bulk
//               copies (the packed layout keeps all of K contiguous per 64-row block and segment, so no tensor
//               map is needed and one copy per segment and row block covers the whole stage);
//   warp 22     brings the stage's activation tile [N_TILE x 64 per K block] with one 3-D TMA tensor copy (128-byte
//               swizzle, rows past N and K blocks past K zero-filled) onto a barrier of its own;
//   warps 6-21  unpack the segments into fp16 bit patterns (code value / 2^bias, exact) and write them STRAIGHT INTO
//               TENSOR MEMORY with tcgen05.st.16x128b: the reference's packed format hands every lane exactly the
//               registers of an m16k16 A fragment, which is the register pattern of that store, so the dequantised
//               weights never touch shared memory.  The 16 warps are four groups of four (one warp per tensor-memory
//               lane quadrant); the tensor-memory A operand is a ring of POSITIONS (one or two K blocks each), and
//               group g takes the positions g, g + 4, ... of the CTA's running count: per visit it waits for the
//               stage's weights, unpacks (for e3m2 / e2m2 with a sequence whose shifts are multiplications by
//               kernel parameters, so that they issue on the FMA pipe beside the logic pipe: unpack16_mul), waits for
//               the position's slot, stores, and hands the slot to the issuing warp;
//   warps 0-3   issue tcgen05.mma.kind::f16 with A from tensor memory and B from shared memory, accumulating
//               fp32 in tensor memory; issuer i takes the positions i, i + issuers, ... (up to four issuers, each with
//               its own accumulator).  An issuer is a WHOLE warp, converged, with one elected lane issuing: the warp
//               index comes through a shuffle, so addresses and descriptors stay warp-uniform, and a round of four
//               MMAs and a commit costs ~64 cycles where a branch taken by one lane alone pays ~230, plus ~200 for
//               every barrier wait whose result it consumes (the copy producers issue the same way).  At the end
//               of a segment the same four warps (one per tensor-memory lane quadrant) read the accumulators
//               with tcgen05.ld, add them, multiply by 2^bias * scale[row] in fp32 (the per-row scale is
//               applied here, once per output, not once per weight), add the bias, apply the fused activation and
//               store fp16 output - to this GPU's buffer or to every rank's - or fp32 partials.
//
// Six-bit weights and at most 64 tokens have a second path that does without the unpack warps altogether
// (fpx_native.cu); this kernel is the general one.
//
// The kernel is launched programmatically: it starts while the previous kernel of the stream is finishing and every
// role executes griddepcontrol.wait before it first touches global memory (weights that the caller declared
// static are requested before that).  Ring depths are multiples of the stride of every role that visits only every
// n-th position (see Config).
//
// Every mbarrier wait is bounded; on a time-out the CTA records a code in a status word, drains its
// own copies, frees its tensor memory and returns.
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

// K blocks (64 wide) per shared-memory pipeline stage for a given tile width
constexpr int gemm_ks(int n_tile) { return n_tile <= 64 ? 4 : (n_tile <= 128 ? 2 : 1); }

constexpr int kTileM = 128;
constexpr int kAColsPerKBlock = 32;      // 64 fp16 along K per tensor-memory lane
constexpr int kMaxIssuers = 4;           // warps 0..3: MMA issuers (whole warps, one elected lane) and, one per lane quadrant, the epilogue
constexpr int kProducerWarp = 4;         // warps 4,5: the weights' copy producers (whole warps, one elected lane)
constexpr int kProducerWarps = 2;
constexpr int kFirstDequantWarp = kProducerWarp + kProducerWarps;
constexpr int kDequantGroups = 4;        // a group = 4 consecutive warps, one per tensor-memory lane quadrant
constexpr int kDequantWarps = 4 * kDequantGroups;
constexpr int kEpilogueWarps = 4;        // = warps 0..3
constexpr int kActProducerWarp = kFirstDequantWarp + kDequantWarps;   // the last warp: activation copies (one thread)
constexpr int kWarps = kActProducerWarp + 1;
constexpr int kThreads = kWarps * 32;
constexpr uint32_t kTmemCols = 512;      // the whole tensor memory: one CTA per SM



// Sleep between two polls of a barrier (ns).  Each failed poll costs issue slots the unpack warps need, so with the
// long stages of the narrow tiles the copy producers (which run stages ahead of their consumers) and the issuing warps
// (which get a new position only every few hundred nanoseconds) poll slowly; the wide tiles have stages of ~250 ns and
// poll quickly.
constexpr uint32_t kPollProducerNarrow = 200, kPollIssuerNarrow = 40, kPollWide = 20, kPollUnpackWide = 100;

// Packed bytes of one (64 rows x 64 K) block per segment width.
template <int BW>
struct RawBlock {
    static constexpr uint32_t seg1 = (BW & 1) ? tile_bytes(1) : 0u;
    static constexpr uint32_t seg2 = (BW & 2) ? tile_bytes(2) : 0u;
    static constexpr uint32_t seg4 = (BW & 4) ? tile_bytes(4) : 0u;
    static constexpr uint32_t bytes128 = 2u * (seg1 + seg2 + seg4);   // 128 rows x 64 K
};

// A shared-memory pipeline stage covers KS K blocks (64 wide each) of one 128-row tile:
//   [activations: KS x (N_TILE x 128 B, 128-byte swizzled)]
//   [weights, per segment width: row block 0: KS blocks, row block 1: KS blocks]
// Tensor memory holds a ring of `a_slots` slots of `kpw` K blocks each (32 columns = 64 fp16 along K per K block and
// lane) and behind it the accumulators of the issuing warps.
//
// Positions.  A position is `kpw` consecutive K blocks of a stage: what one unpack warp turns into fp16 per visit and
// what is handed to an issuing warp at once.  Every stage contributes ks / kpw positions to one running count p
// (positions past the end of a tile's K range exist too: they take part in the hand-shakes and are unpacked from
// whatever the stage holds, but get no MMA).  Position p lives in ring slot p % a_slots.  Unpack group g (four warps,
// one per tensor-memory lane quadrant) takes the positions p = g (mod 4); issuing warp i takes p = i (mod issuers).
// PAIR: two CTAs on neighbouring SMs (a cluster of two) work on one 256-row tile: each unpacks its own 128 rows into its
// own tensor memory and loads HALF of the activation tile (N_TILE / 2 token rows); the first CTA issues
// tcgen05.mma.cta_group::2 for both (M = 256), whose B operand is read from both shared memories.  The activation tile,
// which a wide tile otherwise re-reads from L2 for every 128 output channels, is read once per 256.
// Correct (tests) but NOT the default: on the 57344 x 8192 layer at 1024 tokens it takes 0.73 ms against 0.66 ms.
// Measured: the pair's MMAs run at the full rate in isolation (128 cycles per M256 x N256 x K16, with multicast commits
// and concurrent tensor-memory stores), the L2 -> SM traffic does fall (7.5 -> 5.2 GB); in the kernel every role waits
// for completed MMAs, which take ~180 cycles each.  FP6B200_OPTION_PAIR_TILES turns it on.
template <int BW, int N_TILE, bool PAIR = false>
struct Config {
    using Raw = RawBlock<BW>;
    static constexpr bool pair = PAIR;
    static constexpr int n_local = PAIR ? N_TILE / 2 : N_TILE;   // token rows of the activation tile in this CTA's shared memory
    static constexpr int ks = gemm_ks(N_TILE);
    static constexpr int kpw = N_TILE <= 128 ? 2 : 1;
    // A pair signals across two SMs (stored slots and landed activations go to the first CTA's barriers, completed MMAs come
    // back by a multicast commit), so its rings are twice as deep - which the halved activation tile and the 128
    // tensor-memory columns the widest tile leaves free pay for.
    static constexpr int stages = PAIR ? 8 : (ks == 4 ? (N_TILE <= 16 ? 6 : 4) : 4);
    static constexpr int a_slots = PAIR ? 8 : 4;   // one or two slots per unpack group: 64 columns of fp16 weights each, 32 for the widest tile
    // The activation blocks may have a ring of their own, deeper than the weights' (b_stages > stages).  Measured on the
    // widest tile (32 KB blocks, 57344 x 8192 at 1024 tokens): six blocks in flight instead of four change nothing
    // (0.713 against 0.721 ms): the copies are not what the tile waits for.  Per position the MMAs read 32 KB of shared
    // memory, the copies write 38 KB and the unpack warps read 6 KB: 76 KB at 128 B/clk = 594 cycles for 512 cycles of
    // tensor work, which is the 84 % tensor-pipe activity the profiler reports.  So the rings stay one.
    static constexpr int b_stages = stages;
    static constexpr bool split_rings = b_stages != stages;
    static constexpr int pos_per_stage = ks / kpw;
    // When every stage is one position and the two rings are equally deep, slot and stage coincide and ONE commit of the
    // issuing warp frees both the tensor-memory slot and the stage's activations (measured 6 % faster on the widest
    // tile than two commits; the weights of a stage are still handed back by the unpack warps as soon as they are read).
    static constexpr bool unified = (ks == kpw) && (a_slots == stages) && !split_rings;
    // A warp needs ~60 cycles for a barrier wait and ~64 for four MMAs and a commit, and the narrow MMAs occupy the
    // tensor pipe for ~40 cycles only, so narrow tiles are issued by several warps, each into an accumulator of its own
    // (the epilogue adds them up).
    static constexpr int issuers = N_TILE <= 64 ? 4 : (N_TILE <= 128 ? 2 : 1);
    static constexpr int stage_step = kDequantGroups / pos_per_stage;   // an unpack group visits every stage_step-th stage
    static constexpr int issuer_step = issuers > pos_per_stage ? issuers / pos_per_stage : 1;   // same for an issuing warp
    static constexpr int stage_issuers = issuers < pos_per_stage ? issuers : pos_per_stage;    // issuers that read one stage
    // An mbarrier wait sees only the parity of the phase, so a waiter must know that the phase BEFORE the one it
    // waits for is complete: it must meet a barrier again on that barrier's very next use.  Hence every ring depth
    // is a multiple of the stride of every role that strides over it.  (With a depth of 5 and a stride of 4 a warp
    // once took a copy that had not landed yet for done and unpacked the slot's previous contents.)
    static_assert(ks % kpw == 0 && kDequantGroups % pos_per_stage == 0, "positions per stage");
    static_assert(stages % stage_step == 0, "an unpack group must meet a shared-memory slot again on the slot's next use");
    static_assert(stages % issuer_step == 0, "an issuing warp must meet a shared-memory slot again on the slot's next use");
    static_assert(a_slots % kDequantGroups == 0, "a tensor-memory slot is always filled by the same unpack group");
    static_assert(a_slots % issuers == 0 && (issuers % pos_per_stage == 0 || pos_per_stage % issuers == 0),
                  "a slot is always consumed by the same issuing warp");
    static_assert(issuers <= kMaxIssuers, "issuing warps are the first warps of the CTA");
    static constexpr int readers = 4 * pos_per_stage;   // unpack warps that read a stage's weights
    static constexpr uint32_t poll_producer = N_TILE <= 64 ? kPollProducerNarrow : kPollWide;
    static constexpr uint32_t poll_issuer = N_TILE <= 64 ? kPollIssuerNarrow : kPollWide;
    // the unpack warps of a wide tile are ahead of the tensor pipe most of the time: every poll they save is power for it
    static constexpr uint32_t poll_unpack = N_TILE <= 128 ? ptx::kPollFast : kPollUnpackWide;
    static constexpr uint32_t b_block = (uint32_t)n_local * 128u;
    // shared memory: either `stages` stages of [activation blocks | weight segments], or (split_rings) the ring of
    // activation blocks followed by the ring of weight segments
    static constexpr uint32_t w_stage = ks * Raw::bytes128;
    static constexpr uint32_t b_stride = split_rings ? ks * b_block : ks * b_block + w_stage;   // from one stage's activations to the next
    static constexpr uint32_t w_stride = split_rings ? w_stage : ks * b_block + w_stage;        // from one stage's weights to the next
    static constexpr uint32_t w_off = split_rings ? b_stages * ks * b_block : ks * b_block;    // the weights of stage 0
    static constexpr uint32_t off1 = w_off;
    static constexpr uint32_t off2 = off1 + 2u * ks * Raw::seg1;
    static constexpr uint32_t off4 = off2 + 2u * ks * Raw::seg2;
    static constexpr uint32_t ring_bytes = b_stages * ks * b_block + stages * w_stage;
    static constexpr uint32_t slot_cols = kpw * kAColsPerKBlock;
    static constexpr uint32_t acc_col0 = a_slots * slot_cols;
    static constexpr uint32_t acc_stride = N_TILE < 32 ? 32u : (uint32_t)N_TILE;
    static_assert(b_stride % 1024 == 0, "activation blocks must stay 1024-byte aligned");
    static_assert(b_stages % issuer_step == 0, "an issuing warp must meet an activation slot again on the slot's next use");
    static_assert(acc_col0 + issuers * acc_stride <= kTmemCols, "tensor memory budget");
    // + for a pair: the peer's "activations landed" per stage, "slot stored" per slot and "accumulator read" words
    static constexpr int num_barriers = 2 * stages + 2 * b_stages + 2 * a_slots + 2 + (PAIR ? stages + a_slots + 1 : 0);
    static constexpr uint32_t used_bytes = ring_bytes + num_barriers * 8u + 32u;
    static constexpr uint32_t smem_bytes = used_bytes > 116u * 1024u ? used_bytes : 116u * 1024u;   // never two CTAs per SM
    static_assert(2u * smem_bytes > 228u * 1024u, "two CTAs must never share an SM: each takes all of tensor memory");
    static_assert(!PAIR || (issuers == 1 && N_TILE % 32 == 0), "a pair has one issuing thread");
    static_assert(smem_bytes <= 227u * 1024u, "shared memory budget");
};

// Optional per-role cycle counters (build with -DFPX_PROFILE): every role thread accumulates the cycles it
// spends in each of its waits and in total, and leaves them in g_prof[cta][warp][counter].
#ifdef FPX_PROFILE
__device__ unsigned long long g_prof[160][kWarps][8];
__device__ unsigned long long g_stamp[160][16];   // global-timer stamps (ns) of a CTA's milestones
#define PROF_STAMP(slot) do { if (blockIdx.x < 160) g_stamp[blockIdx.x][slot] = ptx::global_timer_ns(); } while (0)
#define PROF_DECL unsigned long long prof_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}; const long long prof_t0 = clock64();
#define PROF_WAIT(slot, expr) [&]() { const long long t_ = clock64(); const bool r_ = (expr); prof_acc[slot] += (unsigned long long)(clock64() - t_); return r_; }()
#define PROF_BEGIN(var) const long long var = clock64();
#define PROF_END(slot, var) prof_acc[slot] += (unsigned long long)(clock64() - var);
#define PROF_COUNT(slot) prof_acc[slot]++;
#define PROF_FLUSH() do { prof_acc[7] = (unsigned long long)(clock64() - prof_t0); if (lane == 0 && blockIdx.x < 160) for (int i_ = 0; i_ < 8; i_++) g_prof[blockIdx.x][warp][i_] = prof_acc[i_]; } while (0)
#else
#define PROF_STAMP(slot) do { } while (0)
#define PROF_DECL
#define PROF_WAIT(slot, expr) (expr)
#define PROF_BEGIN(var)
#define PROF_END(slot, var)
#define PROF_COUNT(slot)
#define PROF_FLUSH() do { } while (0)
#endif

// Optional timeline of the first CTA (build with -DFPX_TRACE): global-timer stamps of what each role sees and does for
// the ring positions kTraceFirst .. kTraceFirst + 63, read back with fp6b200_debug_read_trace.
#ifdef FPX_TRACE
#ifndef FPX_TRACE_FIRST
#define FPX_TRACE_FIRST 512
#endif
constexpr uint32_t kTraceFirst = FPX_TRACE_FIRST;
__device__ unsigned long long g_trace[12][64];
#define PROF_TRACE(role, pos) do { if (blockIdx.x == 0 && lane == 0 && (uint32_t)(pos) - kTraceFirst < 64u) g_trace[role][(uint32_t)(pos) - kTraceFirst] = ptx::global_timer_ns(); } while (0)
#else
#define PROF_TRACE(role, pos) do { } while (0)
#endif

constexpr uint32_t kMaxGrid = 256;   // CTAs the fix-up kernel's slot list can hold

// silu(gate) * up in fp32
__device__ __forceinline__ float silu_mul(float gate, float up) { return gate / (1.0f + __expf(-gate)) * up; }

struct Params {
    const uint8_t* weight;
    const uint8_t* region[3];   // start of the 1-bit, 2-bit and 4-bit regions of the packed weights
    const __half* scales;
    OutTargets out;             // where finished fp16 tiles go (this GPU's buffer, or every rank's)
    uint32_t weights_static;    // the packed weights are not written by earlier work of the stream: read them at once
    UnpackMul mul[2];           // unpack16_mul's multipliers for h = 0, 1 (parameters so that they stay multiplications)
    const __half* bias;         // per-row addend, or nullptr
    uint32_t activation;        // kActNone / kActSiluMul (rows in gate/up pairs)
    float* workspace;
    uint32_t M, N, K;
    WorkPlan plan;
    int* status;
};

template <int E_BITS, int M_BITS, int N_TILE, bool PAIR = false>
__global__ void __launch_bounds__(kThreads, 1)
fpx_gemm_kernel(const __grid_constant__ CUtensorMap act_map, const __grid_constant__ Params p) {
    constexpr int BW = 1 + E_BITS + M_BITS;
    constexpr bool kShortUnpack = M_BITS == 2 && (E_BITS == 3 || E_BITS == 2);   // e3m2, e2m2: the multiply-based sequence
    using Cfg = Config<BW, N_TILE, PAIR>;
    using Raw = typename Cfg::Raw;
    constexpr int KS = Cfg::ks;
    constexpr int R = Cfg::stages;
    constexpr int RB = Cfg::b_stages;
    constexpr int SA = Cfg::a_slots;
    constexpr int NI = Cfg::issuers;

    // 128-byte-swizzled tiles need a 1024-byte aligned base; the dynamic window starts at offset 0 of the
    // CTA's shared memory (no static shared memory in this kernel), which is checked below.
    extern __shared__ __align__(1024) uint8_t smem_dyn[];
    // everything in shared memory is addressed by 32-bit shared-space addresses
    const uint32_t ring = ptx::smem_u32(smem_dyn);
    const uint32_t w_full = ring + Cfg::ring_bytes;      // barrier arrays, 8 bytes per barrier: the stage's weights have landed
    const uint32_t b_full = w_full + 8 * R;              // the stage's activations have landed
    const uint32_t w_empty = b_full + 8 * RB;            // the unpack warps have read the weights of the stage
    const uint32_t b_empty = w_empty + 8 * R;            // the MMAs that read the activations of the stage are done
    const uint32_t a_full = b_empty + 8 * RB;            // per tensor-memory slot: the K block's fp16 weights are stored
    const uint32_t a_empty = a_full + 8 * SA;            // per slot: the MMAs that read it are done
    const uint32_t acc_full = a_empty + 8 * SA;
    const uint32_t acc_empty = acc_full + 8;
    // pair only, used in the first CTA: what the second CTA reports when slot and stage do not share a barrier (its unpack
    // warps have stored the slot) and that its epilogue warps have read the accumulator.  In the configuration that exists
    // (slot = stage) the second CTA's copies and unpack warps arrive on the first CTA's b_full directly and b_peer is unused.
    const uint32_t b_peer = acc_empty + 8;
    const uint32_t a_peer = b_peer + 8 * R;
    const uint32_t acc_peer = a_peer + 8 * SA;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem_dyn + Cfg::ring_bytes + 8 * Cfg::num_barriers);
    volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_holder + 1);

    // the warp's index, taken through a shuffle so that the compiler knows it to be the same in every lane: the roles that
    // a whole warp executes (MMA issue) then keep their addresses and descriptors warp-uniform
    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
    const int lane = threadIdx.x & 31;
    // a pair shares one entry of the work plan; `half_id` is the CTA's place in it (its 128 of the tile's 256 rows)
    const uint32_t half_id = PAIR ? ptx::cluster_ctarank() : 0u;
    const uint32_t cta = PAIR ? blockIdx.x >> 1 : blockIdx.x;
    const WorkPlan& plan = p.plan;   // stays in the parameter space (it carries a table indexed by CTA)

    // The reduction / fix-up kernel that may follow is launched with programmatic stream serialisation: let it
    // become resident now; it waits for this grid to finish before it reads anything.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (threadIdx.x == 0) PROF_STAMP(0);
    if ((ring & 1023u) != 0u) {   // uniform over the CTA: nothing has been set up yet
        if (threadIdx.x == 0) atomicCAS(p.status, 0, kErrSmemAlign);
        return;
    }
    // Set-up.  The first producer warp initialises every barrier; the producer warps then meet on a barrier of
    // their own and start copying at once, while the rest of the CTA waits for the tensor-memory allocation too.
    if (warp == kProducerWarp) {   // one barrier per lane and round
        for (int i = lane; i < R; i += 32) {
            ptx::mbar_init(w_full + 8 * i, kProducerWarps);
            ptx::mbar_init(w_empty + 8 * i, Cfg::readers);
        }
        for (int i = lane; i < RB; i += 32) {
            // unified: "activations landed" and "slot stored" share the barrier (the copy's arrival + four unpack warps),
            // so that the issuing warp waits once per position; the second CTA of a pair reports both to the first
            ptx::mbar_init(b_full + 8 * i, Cfg::unified && half_id == 0u ? (PAIR ? 9 : 5) : 1);
            ptx::mbar_init(b_empty + 8 * i, Cfg::stage_issuers);
        }
        for (int i = lane; i < SA; i += 32) { ptx::mbar_init(a_full + 8 * i, 4); ptx::mbar_init(a_empty + 8 * i, 1); }
        if (lane == 0) { ptx::mbar_init(acc_full, NI); ptx::mbar_init(acc_empty, kEpilogueWarps); }
        if constexpr (PAIR) {
            for (int i = lane; i < SA; i += 32) ptx::mbar_init(a_peer + 8 * i, 4);
            if (lane == 0) ptx::mbar_init(acc_peer, kEpilogueWarps);
        }
        if (lane == 0) *abort_word = 0;
        ptx::fence_barrier_init();
        if (lane == 0) ptx::prefetch_tensormap(&act_map);
    }
    if (warp == 0) {
        if constexpr (PAIR) {
            ptx::tmem_alloc_pair(ptx::smem_u32(tmem_holder), kTmemCols);
            ptx::tmem_relinquish_pair();
        } else {
            ptx::tmem_alloc(ptx::smem_u32(tmem_holder), kTmemCols);
            ptx::tmem_relinquish();
        }
    }
    const bool is_producer = (warp >= kProducerWarp && warp < kProducerWarp + kProducerWarps) || warp == kActProducerWarp;
    if (is_producer) {
        __threadfence_block();
        asm volatile("bar.sync 1, %0;" ::"n"(32 * (kProducerWarps + 1)) : "memory");   // producers: the barriers exist
        asm volatile("bar.arrive 2, %0;" ::"n"(kThreads) : "memory");            // tell the others, do not wait
    } else {
        ptx::tc_fence_before_sync();
        asm volatile("bar.sync 2, %0;" ::"n"(kThreads) : "memory");
        ptx::tc_fence_after_sync();
    }
    if constexpr (PAIR) ptx::cluster_sync_all();   // both CTAs' barriers exist before either signals the other's
    if (threadIdx.x == 0) PROF_STAMP(1);
    const uint32_t tmem_base = *tmem_holder;   // valid for every warp but the producers, which never use it

    if (is_producer) {
        // ------------------------------------------------------------ producers (a warp each, one elected lane issues): warps 4 and 5 copy the
        // weight segments of the tile's first / second 64-row block, the last warp the activations (one 3-D TMA box per
        // stage).  Weights declared static are requested before griddepcontrol.wait, i.e. while the previous kernel
        // of the stream may still be running; everything else waits for it.
        {
            const bool acts = warp == kActProducerWarp;
            const uint32_t half = acts ? 0u : (uint32_t)(warp - kProducerWarp);
            if (warp == kProducerWarp && lane == 0) PROF_STAMP(13);
            const uint64_t pol = acts ? ptx::policy_evict_last() : ptx::policy_evict_first();
            const uint64_t kblocks = plan.kblocks;
            const uint8_t* reg1 = p.region[0];
            const uint8_t* reg2 = p.region[1];
            const uint8_t* reg4 = p.region[2];
            const uint32_t my_full = acts ? b_full : w_full;
            const uint32_t my_empty = acts ? (Cfg::unified ? a_empty : b_empty) : w_empty;
            bool waited = !acts && p.weights_static != 0;   // nothing to wait for before static weights are read
            // the ring this warp fills: activation blocks or weight segments (two rings of different depth for the widest tile)
            const uint32_t ring_n = acts ? (uint32_t)RB : (uint32_t)R;
            const uint32_t ring_stride = acts ? Cfg::b_stride : Cfg::w_stride;
            struct { uint32_t idx, lap; } pos = {0u, 0u};
            uint32_t issued = 0;
            bool ok = true;
            SegmentIter iter;
            Segment seg;
            PROF_DECL
            plan_start(plan, cta, &iter);
            while (ok && plan_next(plan, cta, &iter, &seg)) {
                const uint32_t p_tile = plan.n_tiles == 1 ? seg.tile : seg.tile / plan.n_tiles;   // row tile of the plan (256 rows for a pair)
                const uint32_t m_tile = PAIR ? 2u * p_tile + half_id : p_tile;                        // this CTA's 128 rows
                const uint64_t blk0 = ((uint64_t)m_tile * 2 + half) * kblocks + seg.kb_begin;   // my row block, first K block
                // a pair splits the tile's token rows: this CTA copies its half
                const int32_t n0 = (int32_t)((seg.tile - p_tile * plan.n_tiles) * N_TILE + half_id * Cfg::n_local);
                const uint32_t nstages = (seg.nkb + KS - 1) / KS;
                uint32_t sidx = plan_first_stage(plan, cta, nstages);   // stage of the segment's K range handled next
                if (warp == kProducerWarp && lane == 0 && issued == 0) PROF_STAMP(14);
                for (uint32_t i = 0; i < nstages; i++) {
                    const uint32_t kb_off = sidx * KS;
                    const uint32_t cnt = seg.nkb - kb_off < (uint32_t)KS ? seg.nkb - kb_off : (uint32_t)KS;
                    sidx = sidx + 1 == nstages ? 0u : sidx + 1;
                    if (!PROF_WAIT(0, ptx::mbar_wait_warp(my_empty + 8 * pos.idx, pos.lap ^ 1u, abort_word, kErrStageEmpty, Cfg::poll_producer))) { ok = false; break; }
                    PROF_COUNT(6)
                    PROF_TRACE(acts ? 0 : 8 + 2 * half, issued);
                    if (!waited) {
                        asm volatile("griddepcontrol.wait;" ::: "memory");   // first read of memory the previous kernel may write
                        waited = true;
                    }
                    if (warp == kProducerWarp && lane == 0 && issued == 0) PROF_STAMP(15);
                    PROF_BEGIN(t_issue)
                    const uint32_t bar = my_full + 8 * pos.idx;
                    const uint32_t dst = ring + pos.idx * ring_stride;
                    const uint64_t b0 = blk0 + kb_off;
                    if (ptx::elect_one()) {
                        if (acts && PAIR) {
                            // both halves of the activation tile are counted on the FIRST CTA's barrier, which expects the
                            // bytes of both: the issuing warp there waits once, and nothing has to pass the news on
                            if (half_id == 0u) ptx::mbar_arrive_expect_tx(bar, 2u * KS * Cfg::b_block);
                            ptx::tma_load_3d_pair(dst, &act_map, 0, n0, (int32_t)(seg.kb_begin + kb_off), ptx::mapa(bar, 0u), pol);
                        } else if (acts) {
                            // always KS blocks: blocks past the end of K are zero-filled by the copy
                            ptx::mbar_arrive_expect_tx(bar, KS * Cfg::b_block);
                            ptx::tma_load_3d(dst, &act_map, 0, n0, (int32_t)(seg.kb_begin + kb_off), bar, pol);
                        } else {
                            ptx::mbar_arrive_expect_tx(bar, cnt * (Raw::bytes128 / 2));
                            if (Raw::seg1) ptx::bulk_g2s(dst + Cfg::off1 + half * KS * Raw::seg1, reg1 + b0 * Raw::seg1, cnt * Raw::seg1, bar, pol);
                            if (Raw::seg2) ptx::bulk_g2s(dst + Cfg::off2 + half * KS * Raw::seg2, reg2 + b0 * Raw::seg2, cnt * Raw::seg2, bar, pol);
                            if (Raw::seg4) ptx::bulk_g2s(dst + Cfg::off4 + half * KS * Raw::seg4, reg4 + b0 * Raw::seg4, cnt * Raw::seg4, bar, pol);
                        }
                    }
                    __syncwarp();
                    PROF_END(3, t_issue)
                    PROF_TRACE(acts ? 1 : 9 + 2 * half, issued);
                    if (++pos.idx == ring_n) { pos.idx = 0; pos.lap ^= 1u; }
                    if (warp == kProducerWarp && lane == 0) { if (issued == 0) PROF_STAMP(2); PROF_STAMP(3); }
                    issued++;
                }
            }
            PROF_FLUSH();
            if (*abort_word != 0 && PAIR && acts && half_id != 0u) {   // this CTA's copies are counted in the other CTA: just give them time
                const uint64_t t0 = ptx::global_timer_ns();
                while (ptx::global_timer_ns() - t0 < 1000000ull) { }
            } else if (*abort_word != 0) {   // gave up somewhere: let the copies in flight land before leaving
                const uint32_t first = issued > ring_n ? issued - ring_n : 0u;
                for (uint32_t t = first; t < issued; t++)
                    ptx::mbar_wait_warp(my_full + 8 * (t % ring_n), (t / ring_n) & 1u, abort_word, kErrStageFull, Cfg::poll_producer, 50000000ull);
            }
        }
        __syncwarp();
    } else if (warp < kMaxIssuers) {
        // ------------------------------------------------------------ MMA issue + epilogue
        // Per segment: the first NI warps issue the MMAs, each converged with one elected lane (issuer i takes the K blocks i, i + NI, ... of every
        // stage, each as soon as its slot of the tensor-memory ring is full, and accumulates them in its own
        // accumulator); then all four warps, one per tensor-memory lane quadrant, read the accumulators, add them and
        // store the tile (lane = output channel, column = token).
        constexpr uint32_t idesc = ptx::idesc_f16_f32(PAIR ? 2 * kTileM : kTileM, N_TILE);
        // In a pair the first CTA issues for both.  The second CTA's issuing warp has nothing to do in the main loop: its
        // activation copies are counted on the first CTA's barrier (a copy may name a barrier of either CTA of the pair) and
        // its unpack warps arrive there too.  (An earlier form had this warp wait for its own copies and pass the news on
        // with a remote arrive: with the .release.cluster arrive that cost ~1300 cycles per stage and bounded the pair at
        // 1.37 ms on 57344 x 8192 at 1024 tokens; without the relay 0.78 ms, with plain remote arrives 0.73 ms, against
        // 0.66 ms for one CTA per tile.)
        const bool relay = PAIR && half_id != 0u;
        const uint32_t me = (uint32_t)warp;
        const int q = warp & 3;
        const uint64_t b_desc0 = ptx::smem_desc_k_sw128(ring);
        asm volatile("griddepcontrol.wait;" ::: "memory");   // before the scales are read and anything is stored
        uint32_t j0 = 0, nseg = 0;
        bool ok = true;
        SegmentIter iter;
        Segment seg;
        PROF_DECL
        plan_start(plan, cta, &iter);
        while (ok && plan_next(plan, cta, &iter, &seg)) {
            const uint32_t nstages = (seg.nkb + KS - 1) / KS;
            if (me < (uint32_t)NI) {   // the whole warp, converged; one elected lane issues
                if (!relay) {
                    if (!PROF_WAIT(2, ptx::mbar_wait_warp(acc_empty, (nseg & 1u) ^ 1u, abort_word, kErrAccEmpty))) ok = false;
                    if constexpr (PAIR)
                        if (ok && !ptx::mbar_wait_warp(acc_peer, (nseg & 1u) ^ 1u, abort_word, kErrAccEmpty)) ok = false;
                }
                ptx::tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + Cfg::acc_col0 + me * Cfg::acc_stride;
                constexpr uint32_t PPS = (uint32_t)Cfg::pos_per_stage, IST = (uint32_t)Cfg::issuer_step, KPW = (uint32_t)Cfg::kpw;
                // positions p = me (mod NI): K blocks [sub * KPW, (sub + 1) * KPW) of the stages j = first (mod IST)
                const uint32_t sub0 = me % PPS;                                  // first position of mine inside a stage
                const uint32_t cls_i = (me / PPS) % IST;
                uint32_t t = (cls_i + IST - (j0 % IST)) % IST;                    // my first stage of the segment
                ptx::RingPos<RB> rp;
                ptx::RingPos<SA> ap;
                rp.set(j0 + t);
                ap.set((j0 + t) * PPS + sub0);
                uint32_t sidx = plan_first_stage(plan, cta, nstages) + t;              // stage of the segment's K range handled next
                uint32_t accumulate = 0u;                                        // 0 only for this issuer's first MMA of the segment
                // (the second CTA of a pair issues nothing: its copies and its unpack warps report to the first CTA's barriers)
                for (; ok && !relay && t < nstages; t += IST) {
                    while (sidx >= nstages) sidx -= nstages;
                    const uint32_t cnt = seg.nkb - sidx * KS < (uint32_t)KS ? seg.nkb - sidx * KS : (uint32_t)KS;
                    sidx += IST;
                    if (!PROF_WAIT(1, ptx::mbar_wait_warp(b_full + 8 * rp.idx, rp.lap, abort_word, kErrStageFull))) { ok = false; break; }
                    PROF_COUNT(6)
                    PROF_TRACE(2, j0 + t);
                    const uint64_t b_desc = b_desc0 + (uint64_t)(rp.idx * (Cfg::b_stride >> 4));
#pragma unroll
                    for (uint32_t sub = sub0; sub < PPS; sub += (uint32_t)NI) {
                        if constexpr (!Cfg::unified) {   // unified: the stage's barrier has covered the slot too
                            if (!PROF_WAIT(0, ptx::mbar_wait_warp(a_full + 8 * ap.idx, ap.lap, abort_word, kErrAFull, Cfg::poll_issuer))) { ok = false; break; }
                            if constexpr (PAIR)
                                if (!PROF_WAIT(4, ptx::mbar_wait_warp(a_peer + 8 * ap.idx, ap.lap, abort_word, kErrAFull, Cfg::poll_issuer))) { ok = false; break; }
                        }
                        if (me == 0 && lane == 0 && nseg == 0 && t == 0) PROF_STAMP(5);
                        PROF_TRACE(3, j0 + t);
                        PROF_BEGIN(t_issue)
                        ptx::tc_fence_after_sync();
                        const uint32_t a_tmem = tmem_base + ap.idx * Cfg::slot_cols;
#pragma unroll
                        for (uint32_t b = 0; b < KPW; b++) {
                            const uint32_t kbi = sub * KPW + b;
                            if (kbi < cnt) {
#pragma unroll
                                for (uint32_t kk = 0; kk < 4; kk++) {   // four K=16 steps; B advances 32 bytes inside the swizzle row
                                    if constexpr (PAIR)
                                        ptx::mma_f16_ts_pair_elect(d_tmem, a_tmem + b * kAColsPerKBlock + kk * 8,
                                                                   b_desc + kbi * (Cfg::b_block >> 4) + kk * 2, idesc, accumulate);
                                    else
                                        ptx::mma_f16_ts_elect(d_tmem, a_tmem + b * kAColsPerKBlock + kk * 8,
                                                              b_desc + kbi * (Cfg::b_block >> 4) + kk * 2, idesc, accumulate);
                                    accumulate = 1u;
                                }
                            }
                        }
                        PROF_END(3, t_issue)
                        PROF_BEGIN(t_commit)
                        if constexpr (PAIR) ptx::tc_commit_pair_elect(a_empty + 8 * ap.idx);
                        else ptx::tc_commit_elect(a_empty + 8 * ap.idx);
                        PROF_END(4, t_commit)
                        PROF_TRACE(4, j0 + t);
                        ap.advance(NI);
                    }
                    if (!ok) break;
                    if (!Cfg::unified) {
                        if constexpr (PAIR) ptx::tc_commit_pair_elect(b_empty + 8 * rp.idx);
                        else ptx::tc_commit_elect(b_empty + 8 * rp.idx);
                    }
                    if (me == 0 && lane == 0) PROF_STAMP(6);
                    rp.advance(IST);
                }
                if (ok && !relay) {   // arrives once this issuer's MMAs (if any) are done
                    if constexpr (PAIR) ptx::tc_commit_pair_elect(acc_full);
                    else ptx::tc_commit_elect(acc_full);
                }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            // Which issuers hold a sum for this segment: issuer i visited the stages t = t_first (mod issuer_step); with two
            // or more visits one of them was a full stage, with one visit its first position must hold a K block.
            uint32_t has_data = 0;
            {
                constexpr uint32_t PPS = (uint32_t)Cfg::pos_per_stage, IST = (uint32_t)Cfg::issuer_step;
                const uint32_t first_stage = plan_first_stage(plan, cta, nstages);
#pragma unroll
                for (uint32_t i = 0; i < (uint32_t)NI; i++) {
                    const uint32_t t_first = ((i / PPS) % IST + IST - (j0 % IST)) % IST;
                    bool has = t_first < nstages;
                    if (has && t_first + IST >= nstages) {
                        uint32_t only = first_stage + t_first;
                        if (only >= nstages) only -= nstages;
                        const uint32_t cnt = seg.nkb - only * KS;   // >= KS for every stage but the last of the K range
                        has = (i % PPS) * (uint32_t)Cfg::kpw < cnt;
                    }
                    has_data |= (has ? 1u : 0u) << i;
                }
            }
            j0 += nstages;

            const uint32_t p_tile = plan.n_tiles == 1 ? seg.tile : seg.tile / plan.n_tiles, n_tile = seg.tile - p_tile * plan.n_tiles;
            const uint32_t m_tile = PAIR ? 2u * p_tile + half_id : p_tile;   // this CTA's 128 rows of the plan's row tile
            const uint32_t row_in_tile = 32u * q + lane;
            const uint32_t row = m_tile * kTileM + row_in_tile;
            // the accumulator holds sum(x * pattern); pattern = code value / 2^bias, so scale by 2^bias * scale[row] here, in fp32
            const float row_scale = __half2float(p.scales[row]) * (float)(1u << (16 - (1 << (E_BITS - 1))));
            const float row_bias = p.bias ? __half2float(p.bias[row]) : 0.0f;   // added where a tile is finished: here, or in the fix-up / reduction
            if (!PROF_WAIT(5, ptx::mbar_wait_warp(acc_full, nseg & 1u, abort_word, kErrAccFull))) { ok = false; break; }
            if (threadIdx.x == 0) PROF_STAMP(7);
            ptx::tc_fence_after_sync();
            const uint32_t acc = tmem_base + ((uint32_t)(32 * q) << 16) + Cfg::acc_col0;
            // issuers that contributed: the fullest stage of the segment holds min(KS, nkb) K blocks, dealt to the issuers in turn
            constexpr int CH = 16;   // columns handled per round
#pragma unroll 1
            for (int c0 = 0; c0 < N_TILE; c0 += CH) {
                const uint32_t n0 = n_tile * N_TILE + c0;
                if (n0 >= p.N) break;
                uint32_t v[CH];
                float f[CH];
#pragma unroll
                for (int u = 0; u < CH; u++) f[u] = 0.0f;
#pragma unroll
                for (uint32_t i = 0; i < (uint32_t)NI; i++)
                    if ((has_data >> i) & 1u) {
                        ptx::tmem_ld_cols<CH>(acc + i * Cfg::acc_stride + c0, v);
                        ptx::tc_wait_ld();
#pragma unroll
                        for (int u = 0; u < CH; u++) f[u] += __uint_as_float(v[u]);
                    }
                if (seg.out_kind == kOutDirect) {
#pragma unroll
                    for (int u = 0; u < CH; u++) f[u] = f[u] * row_scale + row_bias;
                    if (p.activation == kActSiluMul) {
                        // rows 2c (gate) and 2c+1 (up) sit in neighbouring lanes: the even lane computes and stores channel c
#pragma unroll
                        for (int u = 0; u < CH; u++) {
                            const float up = __shfl_xor_sync(0xffffffffu, f[u], 1);
                            f[u] = silu_mul(f[u], up);
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
                } else if (seg.out_kind == kOutSplitPartial) {
                    float* dst = p.workspace + ((size_t)seg.out_index * p.N + n0) * p.M + row;
#pragma unroll
                    for (int u = 0; u < CH; u++)
                        if (n0 + u < p.N) dst[(size_t)u * p.M] = f[u] * row_scale;
                } else {   // a pair's slot holds the 256 rows of the plan's tile: each CTA its half
                    constexpr uint32_t kSlotRows = PAIR ? 2u * kTileM : (uint32_t)kTileM;
                    float* dst = p.workspace + ((size_t)seg.out_index * N_TILE + c0) * kSlotRows + half_id * kTileM + row_in_tile;
#pragma unroll
                    for (int u = 0; u < CH; u++)
                        if (n0 + u < p.N) dst[u * kSlotRows] = f[u] * row_scale;
                }
            }
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (PAIR && half_id != 0u) ptx::mbar_arrive_remote_elected(ptx::mapa(acc_peer, 0u));   // tell the issuing CTA
            else ptx::mbar_arrive_elected(acc_empty);
            if (threadIdx.x == 0) PROF_STAMP(8);
            nseg++;
        }
        PROF_FLUSH();
    } else if (warp >= kFirstDequantWarp && warp < kActProducerWarp) {
        // ------------------------------------------------------------ unpack warps
        // Group g (four warps, one per lane quadrant) takes the K-block positions c = g (mod 4) of the CTA's running
        // count: K block g % KS of every stage_step-th stage.  Per position: wait for the stage's weights, read the
        // lane's words, hand the shared-memory stage back, unpack, wait for the position's tensor-memory slot, store,
        // tell the issuing warp.
        const int q = warp & 3;                                   // tensor-memory lane quadrant this warp may touch
        const uint32_t group = (uint32_t)(warp - kFirstDequantWarp) >> 2;
        constexpr uint32_t ST = Cfg::stage_step, PPS = Cfg::pos_per_stage;
        constexpr int KPW = Cfg::kpw;
        const uint32_t cls = (group / PPS) % ST;                  // it takes the stages j with j % ST == cls
        const uint32_t kb0 = (group % PPS) * KPW;                 // and these K blocks of them
        const int h = q & 1;                                      // sub-blocks 2h, 2h+1 of the 64-row block
        const int rb = q >> 1;                                    // 64-row block inside the 128-row tile
        const uint32_t lane_base = ring + 4u * lane;
        const uint32_t o4 = Cfg::off4 + (rb * KS + kb0) * Raw::seg4 + 2 * h * 128;
        const uint32_t o2 = Cfg::off2 + (rb * KS + kb0) * Raw::seg2 + h * 128;
        const uint32_t o1 = Cfg::off1 + (rb * KS + kb0) * Raw::seg1;
        const uint32_t a_lane = tmem_base + ((uint32_t)(32 * q) << 16);
        const UnpackMul km = p.mul[h];
        // Per visit: wait for the stage's weights, then K block by K block read the lane's words, unpack them and store
        // the fp16 patterns into the position's tensor-memory slot (the words of the next K block are requested before
        // the stores of this one go out); hand the shared-memory stage back as soon as the last words are read, and the
        // slot to the issuing warp once the stores have completed.  (Handing the slot over only at the start of the
        // next visit, to hide the wait for the stores, measured 6 % slower: the MMAs then finish too late for the
        // group's next visit, which needs the same slot.)  Positions past the end of a K range are unpacked like any
        // other (from whatever the stage holds): they get no MMA.
        uint32_t j0 = 0;            // running stage index at the start of the segment
        uint32_t slot = 0, slot_lap = 0, slot_primed = 0;
        uint32_t pending_bar = 0;   // a_full barrier of the position whose stores are in flight
        bool ok = true;
        SegmentIter iter;
        Segment seg;
        PROF_DECL
        plan_start(plan, cta, &iter);
        uint32_t w4[4][2], w2[4], w1[4];
        auto load_words = [&](uint32_t raw, int b) {
#pragma unroll
            for (int jj = 0; jj < 4; jj++) {
                w4[jj][0] = ptx::lds_u32(raw + o4 + b * Raw::seg4 + (jj * 4 + 0) * 128);
                w4[jj][1] = ptx::lds_u32(raw + o4 + b * Raw::seg4 + (jj * 4 + 1) * 128);
                w2[jj] = Raw::seg2 ? ptx::lds_u32(raw + o2 + b * Raw::seg2 + (jj * 2) * 128) : 0u;
                w1[jj] = Raw::seg1 ? ptx::lds_u32(raw + o1 + b * Raw::seg1 + jj * 128) : 0u;
            }
        };
        // the stores of a position have completed: tell the issuing warp
        auto hand_over = [&]() {
            ptx::tc_wait_st();
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (PAIR && half_id != 0u) ptx::mbar_arrive_remote_elected(pending_bar);   // a barrier of the issuing CTA
            else ptx::mbar_arrive_elected(pending_bar);
            pending_bar = 0;
        };
        while (ok && plan_next(plan, cta, &iter, &seg)) {
            const uint32_t nstages = (seg.nkb + KS - 1) / KS;
            uint32_t t = (cls + ST - (j0 % ST)) % ST;     // this group's first stage of the segment
            ptx::RingPos<R> rp;
            rp.set(j0 + t);
            if (!slot_primed && t < nstages) {            // the group's first position of all: p = (j0 + t) * PPS + group % PPS
                ptx::RingPos<SA> ap;
                ap.set((j0 + t) * PPS + group % PPS);
                slot = ap.idx; slot_lap = ap.lap; slot_primed = 1;
            }
            for (; t < nstages; t += ST) {
                if (!PROF_WAIT(0, ptx::mbar_wait_warp(w_full + 8 * rp.idx, rp.lap, abort_word, kErrStageFull, Cfg::poll_unpack))) { ok = false; break; }
                if (warp == kFirstDequantWarp && lane == 0 && j0 == 0 && t == cls) PROF_STAMP(4);
                PROF_COUNT(6)
                if (q == 0) PROF_TRACE(5, j0 + t);
                const uint32_t raw = lane_base + rp.idx * Cfg::w_stride;   // shared-space byte address of this lane's words
                load_words(raw, 0);
                const uint32_t a_addr = a_lane + slot * Cfg::slot_cols;
#pragma unroll
                for (int b = 0; b < KPW; b++) {
                    PROF_BEGIN(t_math)
                    uint32_t v[2][16];
#pragma unroll
                    for (int jj = 0; jj < 4; jj++) {
                        uint32_t pat[8];
                        if constexpr (kShortUnpack) unpack16_mul<E_BITS>(w4[jj][0], w4[jj][1], w2[jj], w1[jj], km, pat);
                        else unpack16_generic<E_BITS, M_BITS>(w4[jj][0], w4[jj][1], w2[jj], w1[jj], h, pat);
#pragma unroll
                        for (int kk = 0; kk < 2; kk++)
#pragma unroll
                            for (int i = 0; i < 4; i++) v[kk][4 * jj + i] = pat[4 * kk + i];
                    }
                    PROF_END(1, t_math)
                    if (b + 1 < KPW) {
                        load_words(raw, b + 1);
                    } else {
                        __syncwarp();
                        ptx::mbar_arrive_elected(w_empty + 8 * rp.idx);   // the weights can be refilled
                    }
                    if (b == 0) {
                        if (!PROF_WAIT(2, ptx::mbar_wait_warp(a_empty + 8 * slot, slot_lap ^ 1u, abort_word, kErrAEmpty, Cfg::poll_unpack))) { ok = false; break; }
                        ptx::tc_fence_after_sync();
                        if (q == 0) PROF_TRACE(6, j0 + t);
                    }
                    ptx::tmem_st_16x128b_x8(a_addr + b * kAColsPerKBlock, v[0]);
                    ptx::tmem_st_16x128b_x8(a_addr + b * kAColsPerKBlock + (16u << 16), v[1]);
                }
                if (!ok) break;
                {
                    const uint32_t mine = Cfg::unified ? b_full : a_full, peers = Cfg::unified ? b_full : a_peer;
                    pending_bar = (PAIR && half_id != 0u) ? ptx::mapa(peers + 8 * slot, 0u) : mine + 8 * slot;
                }
                hand_over();
                if (q == 0) PROF_TRACE(7, j0 + t);
                slot += kDequantGroups;
                if (slot >= (uint32_t)SA) { slot -= SA; slot_lap ^= 1u; }
                rp.advance(ST);
            }
            j0 += nstages;
        }
        PROF_FLUSH();
    }

    // ------------------------------------------------------------ teardown
    ptx::tc_fence_before_sync();
    __syncthreads();
    if constexpr (PAIR) ptx::cluster_sync_all();   // neither CTA leaves while the other may still signal its barriers
    if (warp == 0) {
        if (*abort_word != 0 && lane == 0) {   // gave up: let MMAs that may still be in flight finish before freeing
            const uint64_t t0 = ptx::global_timer_ns();
            while (ptx::global_timer_ns() - t0 < 2000000ull) { }
        }
        __syncwarp();
        ptx::tc_fence_after_sync();
        if constexpr (PAIR) ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
        else ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
    if (threadIdx.x == 0 && *abort_word != 0) atomicCAS(p.status, 0, *abort_word);
    if (threadIdx.x == 0) PROF_STAMP(9);
}

// ------------------------------------------------------------------------------------------------
// Split-K reduction: out[i] = rn_half(sum over splits, ascending, fp32), the semantics of the
// reference's SplitK_Reduction (fp6_llm/csrc/include/kernel_reduction.cuh:28-47).
__global__ void __launch_bounds__(256) splitk_reduce_kernel(__half* __restrict__ out, const float* __restrict__ partials,
                                                            size_t elems, int split_k, uint32_t rows,
                                                            const __half* __restrict__ bias, int activation) {
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    asm volatile("griddepcontrol.wait;" ::: "memory");   // no-op unless launched with programmatic serialisation
    if (i >= elems) return;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < split_k; s++) {
        const float4 v = *reinterpret_cast<const float4*>(partials + (size_t)s * elems + i);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (bias) {   // four consecutive rows of one token (rows is a multiple of 4)
        const uint32_t m = (uint32_t)(i % rows);
        acc.x += __half2float(bias[m]); acc.y += __half2float(bias[m + 1]);
        acc.z += __half2float(bias[m + 2]); acc.w += __half2float(bias[m + 3]);
    }
    if (activation == kActSiluMul) {   // two gate/up pairs -> two output channels of out[N][rows / 2]
        const __half2 r = __floats2half2_rn(silu_mul(acc.x, acc.y), silu_mul(acc.z, acc.w));
        *reinterpret_cast<__half2*>(out + i / 2) = r;
        return;
    }
    __half2 lo = __floats2half2_rn(acc.x, acc.y), hi = __floats2half2_rn(acc.z, acc.w);
    uint2 packed;
    packed.x = *reinterpret_cast<uint32_t*>(&lo);
    packed.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(out + i) = packed;
}

// Fix-up of the stream-K remainder: CTA of 512 threads = (remainder tile, 16 / groups token columns) x groups; 32 threads
// per column and group: a thread owns four consecutive output channels and every groups-th of the tile's partial slots
// (fp32, float4 loads, all in flight at once: a tile of a large layer has ~40 parts, and summing them one thread after the
// other cost ~6 us of load latency); the groups' sums are then added in group order, so the result does not depend on
// timing.  The host picks groups (1..16) from the parts per tile, keeping the grid within about two CTAs per SM: the
// CTAs are resident early and wait for the GEMM, and those that do not fit would run only after it.
// Tiles that one CTA computed alone were stored directly and are skipped.
// (Summing inside the GEMM by the CTA that delivers a tile's last part was measured slower: its dependent global
// round trips cost more than this launch, and wide tiles are then summed by one SM instead of all.)
constexpr int kFixupThreads = 512;   // 16 (column, group) pairs of 32 threads
constexpr uint64_t kEvenGridMinPercent = 85;
constexpr uint64_t kFixupCostUnits = 20;   // the fix-up launch and its dependency cost about as much as 20 K blocks on one CTA
constexpr uint64_t kMinUnitsPerCta = 8;   // a CTA is not started for fewer 64-K blocks than this (two 256-K stages)
__global__ void __launch_bounds__(kFixupThreads) streamk_fixup_kernel(const __grid_constant__ OutTargets out, const float* __restrict__ slots,
                                                                         uint32_t N, int n_tile_size, const __grid_constant__ WorkPlan plan,
                                                                         int early_trigger, const __half* __restrict__ bias, int activation, uint32_t groups,
                                                                         uint32_t tile_rows) {
    __shared__ uint32_t cand_slot[kMaxGrid];   // per candidate CTA: its slot, or ~0u when it holds nothing
    __shared__ uint32_t part_slot[kMaxGrid];   // slots that hold a part of this tile, in CTA order
    __shared__ uint32_t part_count;
    const uint32_t r = blockIdx.x;
    if (early_trigger) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // a GEMM that follows may set itself up meanwhile
    if (threadIdx.x == 0 && blockIdx.y == 0) PROF_STAMP(10);
    uint32_t first, last;
    plan_tile_owners(plan, r, &first, &last);
    if (first == last) {   // one CTA computed the whole tile and stored it; still do not finish before the GEMM has
        asm volatile("griddepcontrol.wait;" ::: "memory");
        return;
    }
    const uint32_t tile = plan_full_waves(plan) * plan.grid + r;
    const uint32_t m_tile = tile / plan.n_tiles, n_tile = tile % plan.n_tiles;
    const uint32_t span = last - first + 1 < kMaxGrid ? last - first + 1 : kMaxGrid;
    for (uint32_t i = threadIdx.x; i < span; i += blockDim.x) {   // one candidate CTA per thread
        const uint32_t cta = first + i;
        const bool holds = plan_rem_begin(plan, cta) != plan_rem_begin(plan, cta + 1);
        cand_slot[i] = holds ? plan_tile_slot(plan, r, cta) : ~0u;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t cnt = 0;
        for (uint32_t i = 0; i < span; i++)
            if (cand_slot[i] != ~0u) part_slot[cnt++] = cand_slot[i];
        part_count = cnt;
    }
    __syncthreads();
    const uint32_t count = part_count;
    const uint32_t row4 = (threadIdx.x & 31u) * 4u;          // first of this thread's four output channels
    // the plan's row tiles are tile_rows high (256 when CTA pairs computed them); blockIdx.z picks the 128 rows of this CTA
    const size_t slot_stride = (size_t)n_tile_size * tile_rows;
    const uint32_t row_off = blockIdx.z * kTileM + row4;
    asm volatile("griddepcontrol.wait;" ::: "memory");       // the GEMM grid has completed and its stores are visible
    if (threadIdx.x == 0 && blockIdx.y == 0) PROF_STAMP(11);
    __shared__ float4 group_sum[16][32];                      // [group * cols + column][lane]
    const uint32_t cols = 16u / groups;
    const uint32_t col = (threadIdx.x >> 5) % cols, grp = (threadIdx.x >> 5) / cols;
    const uint32_t c = blockIdx.y * cols + col;
    const uint32_t n = n_tile * n_tile_size + c;
    const bool live = c < (uint32_t)n_tile_size && n < N;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live) {
        const float* base = slots + (size_t)c * tile_rows + row_off;
#pragma unroll 8
        for (uint32_t i = grp; i < count; i += groups) {
            const float4 v = *reinterpret_cast<const float4*>(base + part_slot[i] * slot_stride);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
    }
    group_sum[threadIdx.x >> 5][threadIdx.x & 31u] = acc;
    __syncthreads();
    if (live && grp == 0) {
        for (uint32_t g = 1; g < groups; g++) {
            const float4 v = group_sum[g * cols + col][threadIdx.x & 31u];
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        const uint32_t m0 = m_tile * tile_rows + row_off;
        if (bias) {
            acc.x += __half2float(bias[m0]); acc.y += __half2float(bias[m0 + 1]);
            acc.z += __half2float(bias[m0 + 2]); acc.w += __half2float(bias[m0 + 3]);
        }
        if (activation == kActSiluMul) {   // two gate/up pairs -> two output channels
            const __half2 r2 = __floats2half2_rn(silu_mul(acc.x, acc.y), silu_mul(acc.z, acc.w));
            *reinterpret_cast<__half2*>(out.ptr[0] + (size_t)n * out.ld + out.row0 + (m0 >> 1)) = r2;
        } else {
            __half2 lo = __floats2half2_rn(acc.x, acc.y), hi = __floats2half2_rn(acc.z, acc.w);
            uint2 packed;
            packed.x = *reinterpret_cast<uint32_t*>(&lo);
            packed.y = *reinterpret_cast<uint32_t*>(&hi);
            const size_t at = (size_t)n * out.ld + out.row0 + m0;
            for (uint32_t t = 0; t < out.count; t++) *reinterpret_cast<uint2*>(out.ptr[t] + at) = packed;
        }
    }
    if (threadIdx.x == 0 && blockIdx.y == 0) PROF_STAMP(12);
}

// Arrival barrier between the GPUs of an OC-sharded layer.  Thread r tells rank r "the rows of rank `rank` are in
// your buffer" (a release store of this call's number to word `rank` of r's flag array) and then waits until rank r
// has said the same here (word r of the own array).  The call number lives in device memory and is advanced by the
// kernel itself, so a replayed CUDA graph keeps counting.  The kernels before it on the stream have completed when
// it runs (stream order, or griddepcontrol.wait under programmatic launch), which is what makes this rank's stores
// to the peers complete.  The wait is bounded: after kPeerWaitNs the kernel records kErrPeerWait and returns.
// (Running this in the last CTA of the fix-up kernel instead, behind a system-scope fence and a counter of finished
// CTAs, was measured 6 us slower per layer on two GPUs than this separate one-warp launch.)
struct PeerFlags {
    uint32_t* ptr[kMaxOutTargets];
};
constexpr unsigned long long kPeerWaitNs = 2000000000ull;
__global__ void __launch_bounds__(32) gather_barrier_kernel(const __grid_constant__ PeerFlags flags, int world, int rank,
                                                            uint32_t* epoch_counter, int* status) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int r = (int)threadIdx.x;
    const uint32_t epoch = *epoch_counter + 1u;
    __syncwarp();
    if (r == 0) *epoch_counter = epoch;
    if (r >= world) return;
    // The release is cumulative: this rank's stores into the peers' buffers were made by the grids that this kernel waited
    // for above, so they are ordered before the flag at system scope by the release itself (a separate system-scope fence
    // before it would cost a second round trip).
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags.ptr[r] + rank), "r"(epoch) : "memory");
    const uint32_t* mine = flags.ptr[rank] + r;
    const unsigned long long t0 = ptx::global_timer_ns();
    for (uint32_t polls = 0;; polls++) {
        uint32_t seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
        if ((int32_t)(seen - epoch) >= 0) break;
        if ((polls & 63u) == 63u && ptx::global_timer_ns() - t0 > kPeerWaitNs) {
            atomicCAS(status, 0, kErrPeerWait);
            break;
        }
    }
}

// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
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

// Tensor map over the activations [N rows][K fp16] seen as (64 K, N rows, K/64 blocks): one copy of box
// (64, n_tile, ks) lands ks consecutive [n_tile x 128 B] blocks, each 128-byte swizzled, rows past N and blocks
// past K zero-filled.
cudaError_t make_act_map(CUtensorMap* map, const __half* act, size_t N, size_t K, int n_tile, int ks) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return cudaErrorNotSupported;
    cuuint64_t dims[3] = {(cuuint64_t)kKBlock, (cuuint64_t)N, (cuuint64_t)(K / kKBlock)};
    cuuint64_t strides[2] = {(cuuint64_t)K * sizeof(__half), (cuuint64_t)kKBlock * sizeof(__half)};
    cuuint32_t box[3] = {(cuuint32_t)kKBlock, (cuuint32_t)n_tile, (cuuint32_t)ks};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<__half*>(act), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

}  // namespace

// The work decomposition of one call (see WorkPlan): split_k == 0 is the library's own (data-parallel waves of tiles,
// then the K blocks of the remaining tiles dealt out evenly), split_k >= 1 the caller's.  Returns the effective split.
int make_plan(size_t M, size_t n_tiles, size_t K, int split_k, int sms, WorkPlan* out) {
    WorkPlan& plan = *out;
    plan.m_tiles = (uint32_t)(M / kTileM);
    plan.n_tiles = (uint32_t)n_tiles;
    plan.kblocks = (uint32_t)(K / kKBlock);
    const uint64_t tiles = (uint64_t)plan.m_tiles * plan.n_tiles;
    int eff_split = 1;
    if (split_k == 0) {
        plan.mode = kStreamK;
        plan.split_k = 1;
        const uint64_t units = tiles * plan.kblocks;
        // Fewer tiles than SMs: one CTA per whole tile (no tile is split, so no fix-up kernel follows) when that costs no
        // more than dealing the K blocks out evenly plus the fix-up, which is worth about kFixupCostUnits K blocks.
        if (tiles <= (uint64_t)sms && plan.kblocks <= units / (uint64_t)sms + kFixupCostUnits) {
            plan.grid = (uint32_t)tiles;
            plan_finalize(&plan);
            return eff_split;
        }
        uint64_t cap = units / kMinUnitsPerCta;     // CTAs that still get kMinUnitsPerCta blocks each, at least one per tile
        if (cap < tiles) cap = tiles;
        if (cap > (uint64_t)sms) cap = (uint64_t)sms;
        plan.grid = (uint32_t)cap;
        // Fewer tiles than SMs: a grid that is a multiple of the tile count gives every tile the same number of
        // CTAs and no CTA a second tile (one epilogue per CTA); taken when it still fills most of the SMs.
        if (tiles < cap) {
            const uint64_t even = tiles * (cap / tiles);
            if (even * 100 >= cap * kEvenGridMinPercent) plan.grid = (uint32_t)even;
        }
    } else {              // the caller's split: splits beyond the number of K blocks would be empty
        plan.mode = kClassic;
        eff_split = split_k < (int)plan.kblocks ? split_k : (int)plan.kblocks;
        plan.split_k = (uint32_t)eff_split;
        const uint64_t items = tiles * eff_split;
        plan.grid = (uint32_t)(items < (uint64_t)sms ? items : (uint64_t)sms);
    }
    plan_finalize(&plan);
    return eff_split;
}

namespace {

template <int E_BITS, int M_BITS, int N_TILE, bool PAIR = false>
cudaError_t launch_one(cudaStream_t stream, const CUtensorMap& map, const Params& prm) {
    auto kernel = fpx_gemm_kernel<E_BITS, M_BITS, N_TILE, PAIR>;
    constexpr uint32_t smem = Config<1 + E_BITS + M_BITS, N_TILE, PAIR>::smem_bytes;
    static std::atomic<bool> configured[64];   // zero-initialised; several host threads may launch at once
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 0 || dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
        err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return err;
        if (dev >= 0 && dev < 64) configured[dev].store(true, std::memory_order_release);
    }
    // Programmatic launch: the CTAs may start, set up and find their work while the previous kernel of the stream is
    // still finishing; every role waits (griddepcontrol.wait) before it first touches global memory.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(PAIR ? 2 * prm.plan.grid : prm.plan.grid);   // a pair of CTAs (a cluster of two) per entry of the plan
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = programmatic_launch() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (PAIR) {
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = 2;
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = 1;
        cfg.numAttrs = 2;
    }
    return cudaLaunchKernelEx(&cfg, kernel, map, prm);
}

template <int E_BITS, int M_BITS>
cudaError_t launch_by_n(int n_tile, bool pair, cudaStream_t stream, const CUtensorMap& map, const Params& prm) {
    if (pair) return launch_one<E_BITS, M_BITS, 256, true>(stream, map, prm);
    switch (n_tile) {
        case 16:  return launch_one<E_BITS, M_BITS, 16>(stream, map, prm);
        case 32:  return launch_one<E_BITS, M_BITS, 32>(stream, map, prm);
        case 64:  return launch_one<E_BITS, M_BITS, 64>(stream, map, prm);
        case 128: return launch_one<E_BITS, M_BITS, 128>(stream, map, prm);
        default:  return launch_one<E_BITS, M_BITS, 256>(stream, map, prm);
    }
}

}  // namespace

#ifdef FPX_TRACE
extern "C" int fp6b200_debug_read_trace(unsigned long long* host_out) {
    return cudaMemcpyFromSymbol(host_out, g_trace, sizeof(g_trace));
}
#endif
#ifdef FPX_PROFILE
extern "C" int fp6b200_debug_read_profile(unsigned long long* host_out) {
    return cudaMemcpyFromSymbol(host_out, g_prof, sizeof(g_prof));
}
extern "C" int fp6b200_debug_read_stamps(unsigned long long* host_out) {
    return cudaMemcpyFromSymbol(host_out, g_stamp, sizeof(g_stamp));
}
#endif

int device_sm_count() {
    static std::atomic<int> counts[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int n = counts[dev].load(std::memory_order_relaxed);
    if (!n) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        counts[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

static std::atomic<int> g_pair_tiles{0};   // off: measured 0.6 of the single-CTA speed (see Config)
void set_pair_tiles(int on) { g_pair_tiles.store(on < 0 ? 0 : (on > 2 ? 2 : on)); }   // 2: also for layers too small to occupy every pair
int pair_tiles() { return g_pair_tiles.load(); }

// Whether a call runs as CTA pairs on 256-row tiles (the widest tile only, the library's own decomposition, enough row
// tiles to occupy the pairs), and its plan: for a pair the plan's row tiles are 256 rows and its "CTAs" are pairs.
static int plan_call(size_t M, size_t N, size_t K, int split_k, bool has_targets, WorkPlan* plan, bool* pair) {
    const int n_tile = gemm_n_tile(N);
    const size_t n_tiles = (N + n_tile - 1) / n_tile;
    const int sms = device_sm_count() < (int)kMaxGrid ? device_sm_count() : (int)kMaxGrid;
    *pair = pair_tiles() && n_tile == 256 && split_k == 0 && !has_targets && sms >= 2 &&
            (pair_tiles() == 2 || (M / 256) * n_tiles >= (size_t)(sms / 2));
    if (*pair) return make_plan(M / 2, n_tiles, K, split_k, sms / 2, plan);   // M / 2 rows in 128-row tiles = M in 256-row tiles
    return make_plan(M, n_tiles, K, split_k, sms, plan);
}

int gemm_kernel_launches(size_t M, size_t N, size_t K, int split_k) {
    if (M == 0 || M % 256 != 0 || K == 0 || K % 64 != 0 || N == 0 || split_k < 0) return 0;
    WorkPlan plan;
    bool pair = false;
    const int eff_split = plan_call(M, N, K, split_k, false, &plan, &pair);
    if (plan.mode == kStreamK) return plan_rem_tiles(plan) ? 2 : 1;   // GEMM (+ fix-up of the split tiles)
    return eff_split > 1 ? 2 : 1;                                     // GEMM (+ split-K reduction)
}

int gemm_n_tile(size_t N) { return N <= 16 ? 16 : (N <= 32 ? 32 : (N <= 64 ? 64 : (N <= 128 ? 128 : 256))); }

size_t gemm_auto_workspace_bytes(size_t N) {
    // stream-K: two partial slots of 128 x n_tile fp32 per CTA
    const size_t ctas = device_sm_count() < (int)kMaxGrid ? device_sm_count() : kMaxGrid;
    return 2 * ctas * kTileM * gemm_n_tile(N) * sizeof(float);
}

cudaError_t launch_splitk_reduce(cudaStream_t stream, __half* out, const float* partials, size_t elems, int split_k,
                                 bool after_gemm, size_t rows, const Epilogue* epilogue) {
    const __half* bias = epilogue ? epilogue->bias : nullptr;
    const int activation = epilogue ? epilogue->activation : kActNone;
    if ((bias || activation != kActNone) && (rows == 0 || rows % 4 != 0 || elems % rows != 0)) return cudaErrorInvalidValue;
    const size_t threads = (elems + 3) / 4;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((threads + 255) / 256));
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = after_gemm ? 1 : 0;   // overlap the launch with the GEMM's tail
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, splitk_reduce_kernel, out, partials, elems, split_k, (uint32_t)rows, bias, activation);
}

static std::atomic<int> g_weights_static{0};
void set_weights_static(int on) { g_weights_static.store(on ? 1 : 0); }
int weights_static() { return g_weights_static.load(); }
static std::atomic<int> g_programmatic_launch{1};
void set_programmatic_launch(int on) { g_programmatic_launch.store(on ? 1 : 0); }
int programmatic_launch() { return g_programmatic_launch.load(); }

// Sums the partial tiles a stream-K GEMM left in its slots (launched programmatically after it).
cudaError_t launch_streamk_fixup(cudaStream_t stream, const OutTargets& where, const float* workspace, size_t N,
                                 int n_tile, const WorkPlan& plan, const Epilogue* epilogue, int tile_rows) {
    const uint32_t rem = plan_rem_tiles(plan);
    if (rem == 0) return cudaSuccess;
    // groups: as many as half the parts of a tile (about grid / rem CTAs share one), while the grid stays within ~2 CTAs per SM
    const uint32_t parts = (plan.grid + rem - 1) / rem + 1;
    uint32_t groups = 1;
    while (groups < 16 && groups * 2 <= parts / 2 &&
           (uint64_t)rem * ((n_tile + 16 / (groups * 2) - 1) / (16 / (groups * 2))) <= 2ull * (uint64_t)device_sm_count())
        groups *= 2;
    const uint32_t cols = 16 / groups;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(rem, (unsigned)((n_tile + cols - 1) / cols), (unsigned)(tile_rows / kTileM));
    cfg.blockDim = dim3(kFixupThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const int early = programmatic_launch() ? 1 : 0;
    const __half* bias = epilogue ? epilogue->bias : nullptr;
    const int activation = epilogue ? epilogue->activation : kActNone;
    return cudaLaunchKernelEx(&cfg, streamk_fixup_kernel, where, workspace, (uint32_t)N, n_tile, plan, early, bias, activation, groups,
                              (uint32_t)tile_rows);
}

cudaError_t launch_gemm(int e_bits, int m_bits, cudaStream_t stream, const void* weight, const __half* scales,
                        const __half* act, __half* out, size_t M, size_t N, size_t K, float* workspace, int split_k,
                        int* status, const OutTargets* targets, const Epilogue* epilogue) {
    if (!format_supported(e_bits, m_bits)) return cudaErrorInvalidValue;
    const __half* bias = epilogue ? epilogue->bias : nullptr;
    const int activation = epilogue ? epilogue->activation : kActNone;
    if (activation != kActNone && activation != kActSiluMul) return cudaErrorInvalidValue;
    if (activation != kActNone && targets) return cudaErrorInvalidValue;   // the fused exchange stores plain rows only
    if (bias && (reinterpret_cast<uintptr_t>(bias) & 1)) return cudaErrorMisalignedAddress;
    OutTargets where;
    if (targets) {
        where = *targets;
        if (where.count == 0 || where.count > (uint32_t)kMaxOutTargets || split_k > 1) return cudaErrorInvalidValue;
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
    if (M == 0 || M % 256 != 0 || K == 0 || K % 64 != 0 || N == 0 || split_k < 0 || split_k > 65535)
        return cudaErrorInvalidValue;
    if (!weight || !scales || !act || !out || (split_k != 1 && !workspace)) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(weight) & 15) || (reinterpret_cast<uintptr_t>(act) & 15) ||
        (reinterpret_cast<uintptr_t>(out) & 7) || (reinterpret_cast<uintptr_t>(workspace) & 15))
        return cudaErrorMisalignedAddress;
    if (M > 0x7fffffffull || N > 0x7fffffffull || K > 0x7fffffffull) return cudaErrorInvalidValue;
    const int n_tile = gemm_n_tile(N);
    const size_t n_tiles = (N + n_tile - 1) / n_tile;
    if ((M / kTileM) * n_tiles > 0x3fffffffull) return cudaErrorInvalidValue;
    Params prm;
    WorkPlan& plan = prm.plan;
    bool pair = false;
    const int eff_split = plan_call(M, N, K, split_k, targets != nullptr, &plan, &pair);
    CUtensorMap map;
    cudaError_t err = make_act_map(&map, act, N, K, pair ? n_tile / 2 : n_tile, gemm_ks(n_tile));   // a pair's CTAs copy half a tile each
    if (err != cudaSuccess) return err;

    prm.weight = static_cast<const uint8_t*>(weight);
    {
        const int bw_ = 1 + e_bits + m_bits;
        prm.region[0] = prm.weight + region_offset(bw_, 1, M, K);
        prm.region[1] = prm.weight + region_offset(bw_, 2, M, K);
        prm.region[2] = prm.weight + region_offset(bw_, 4, M, K);
    }
    prm.scales = scales;
    prm.out = where;
    prm.workspace = workspace;
    prm.weights_static = (uint32_t)weights_static();
    prm.mul[0] = unpack_mul_values(0);
    prm.mul[1] = unpack_mul_values(1);
    prm.bias = bias;
    prm.activation = (uint32_t)activation;
    prm.M = (uint32_t)M;
    prm.N = (uint32_t)N;
    prm.K = (uint32_t)K;
    prm.status = status;
    FPX_DISPATCH_FORMAT(e_bits, m_bits, (err = launch_by_n<kE, kM>(n_tile, pair, stream, map, prm)));
    if (err != cudaSuccess) return err;
    if (plan.mode == kStreamK) {
        const uint32_t rem = plan_rem_tiles(plan);
        if (rem == 0) return cudaSuccess;
        return launch_streamk_fixup(stream, where, workspace, N, n_tile, plan, epilogue, pair ? 2 * kTileM : kTileM);
    }
    if (eff_split > 1) return launch_splitk_reduce(stream, out, workspace, M * N, eff_split, true, M, epilogue);
    return cudaSuccess;
}

cudaError_t launch_gather_barrier(cudaStream_t stream, uint32_t* const* flag_peers, int world, int rank,
                                  uint32_t* epoch_counter, int* status) {
    if (!flag_peers || world < 1 || world > kMaxOutTargets || rank < 0 || rank >= world || !epoch_counter || !status)
        return cudaErrorInvalidValue;
    PeerFlags flags = {};
    for (int r = 0; r < world; r++) {
        if (!flag_peers[r] || (reinterpret_cast<uintptr_t>(flag_peers[r]) & 3)) return cudaErrorInvalidValue;
        flags.ptr[r] = flag_peers[r];
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(32);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gather_barrier_kernel, flags, world, rank, epoch_counter, status);
}

}  // namespace fpx
