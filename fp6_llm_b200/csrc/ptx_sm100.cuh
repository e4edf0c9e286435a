// Thin inline-PTX wrappers for the sm_100a features the kernels use: mbarrier, bulk (TMA) copies,
// tensor memory (TMEM) management and tcgen05 MMA / load / store.  Device only.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ------------------------------------------------------------------ mbarrier
// Barriers are addressed by their 32-bit shared-space address (smem_u32 of the uint64_t).
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Polls the barrier inside one instruction sequence, without a branch the compiler has to reconverge: up to `tries`
// tests with a sleep of `sleep_ns` after each failed one.  A sleeping thread issues nothing, and every failed test costs
// five instructions, so roles that are far ahead of their partner (the copy producers) sleep long and only a role on
// the critical path polls quickly.
__device__ __forceinline__ bool mbar_spin(uint32_t bar, uint32_t parity, uint32_t tries, uint32_t sleep_ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        ".reg .u32 n;\n\t"
        "mov.u32 n, 0;\n"
        "FPX_SPIN:\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "@p bra FPX_DONE;\n\t"
        "nanosleep.u32 %3;\n\t"
        "add.u32 n, n, 1;\n\t"
        "setp.lt.u32 p, n, %4;\n\t"
        "@p bra FPX_SPIN;\n\t"
        "setp.ne.u32 p, n, n;\n"
        "FPX_DONE:\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(sleep_ns), "r"(tries)
        : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false when the CTA-wide abort word is (or becomes) non-zero: either another
// thread gave up, or this wait itself ran past `timeout_ns`, in which case it records `code` there.
// The clock and the abort word are only looked at between rounds of 1024 polls.
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_word, int code, uint32_t sleep_ns,
                                            uint64_t timeout_ns) {
    const uint64_t t0 = global_timer_ns();
    for (;;) {
        if (mbar_spin(bar, parity, 1024u, sleep_ns)) return true;
        if (*abort_word != 0) return false;
        if (global_timer_ns() - t0 > timeout_ns) {
            *abort_word = code;
            return false;
        }
    }
}
constexpr uint32_t kPollFast = 20;   // ns between polls of a role on the critical path
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_word, int code,
                                          uint32_t sleep_ns = kPollFast, uint64_t timeout_ns = 2000000000ull) {
    if (mbar_spin(bar, parity, 1024u, sleep_ns)) return true;
    return mbar_wait_slow(bar, parity, abort_word, code, sleep_ns, timeout_ns);
}

// The same wait for a whole warp, leaving it converged and with one verdict.  The lanes poll independently and can
// leave the loop in different rounds; warp-wide tcgen05 instructions (.sync.aligned loads, stores and waits)
// that follow a wait must be executed by all lanes together, so the lanes meet again here.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_word, int code,
                                               uint32_t sleep_ns = kPollFast, uint64_t timeout_ns = 2000000000ull) {
    bool ok = mbar_spin(bar, parity, 1024u, sleep_ns);
    if (!__all_sync(0xffffffffu, ok ? 1 : 0)) {
        if (!ok) ok = mbar_wait_slow(bar, parity, abort_word, code, sleep_ns, timeout_ns);
        ok = __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
    }
    return ok;
}

// True in exactly one lane of the (converged) warp.
__device__ __forceinline__ bool elect_one() {
    uint32_t e;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(e));
    return e != 0;
}

// One lane of the (converged) warp arrives for all of it.
__device__ __forceinline__ void mbar_arrive_elected(uint32_t bar) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "@p mbarrier.arrive.shared::cta.b64 _, [%0];\n\t"
        "}\n" ::"r"(bar)
        : "memory");
}

// Position in a ring of SIZE slots: slot index and the parity of the number of completed laps.
template <int SIZE>
struct RingPos {
    uint32_t idx, lap;
    __device__ __forceinline__ void set(uint32_t n) { idx = n % SIZE; lap = (n / SIZE) & 1u; }
    __device__ __forceinline__ void advance(uint32_t step) {
        idx += step;
        while (idx >= (uint32_t)SIZE) { idx -= SIZE; lap ^= 1u; }
    }
};

__device__ __forceinline__ uint32_t lds_u32(uint32_t smem_addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(smem_addr));
    return v;
}

// ------------------------------------------------------------------ L2 policies
__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}

// ------------------------------------------------------------------ bulk copies (TMA)
// 1-D bulk copy global -> shared.  dst/src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t smem_dst, const void* gmem_src, uint32_t bytes, uint32_t bar,
                                         uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(smem_dst), "l"(gmem_src), "r"(bytes), "r"(bar), "l"(policy)
        : "memory");
}
// 3-D tiled tensor copy global -> shared through a tensor map; x is the innermost coordinate.
__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const CUtensorMap* map, int32_t x, int32_t y, int32_t z,
                                            uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%2, %3, %4}], [%5], %6;"
        ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(bar), "l"(policy)
        : "memory");
}
// The same copy issued by a CTA of a pair (cluster of two): the data lands in the issuing CTA's shared memory, the
// transaction bytes are counted on `bar`, a shared::cluster address that may name a barrier of EITHER CTA of the pair
// (no multicast: one destination).
__device__ __forceinline__ void tma_load_3d_pair(uint32_t smem_dst, const CUtensorMap* map, int32_t x, int32_t y, int32_t z,
                                                 uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.cta_group::2.L2::cache_hint"
        " [%0], [%1, {%2, %3, %4}], [%5], %6;"
        ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(bar), "l"(policy)
        : "memory");
}
// 2-D tiled tensor copy global -> shared; x is the innermost coordinate.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, int32_t x, int32_t y, uint32_t bar,
                                            uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%2, %3}], [%4], %5;"
        ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ------------------------------------------------------------------ CTA pairs (clusters of two)
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// All threads of both CTAs.
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address, in the cluster's shared window, of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t mapa(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
// One lane of the (converged) warp arrives on a barrier of another CTA of the cluster (address from mapa).  Without
// the .release.cluster qualifiers: with them a warp spent ~1900 cycles per arrive (the cluster-scope release waits for
// everything the thread has in flight), and what the arrive announces here - tensor-memory stores already waited for
// with tcgen05.wait::st, an accumulator already read - is complete before it is issued.
__device__ __forceinline__ void mbar_arrive_remote_elected(uint32_t cluster_addr) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "@p mbarrier.arrive.shared::cluster.b64 _, [%0];\n\t"
        "}\n" ::"r"(cluster_addr)
        : "memory");
}

// ------------------------------------------------------------------ tensor memory
// Whole-warp calls.  `ncols` is a power of two >= 32; the base address is written to *smem_holder.
__device__ __forceinline__ void tmem_alloc(uint32_t smem_holder, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_holder), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// The same for a CTA pair: executed by the same warp of both CTAs, the columns are taken in both tensor memories.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_holder, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_holder), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// mbarrier arrives (count 1) when every tcgen05 operation this thread issued so far has completed.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// The same instructions for a role that a WHOLE warp executes, converged, with one elected lane issuing: addresses and
// descriptors then stay warp-uniform, and a round of four MMAs and a commit costs the warp ~64 cycles where a branch
// taken by one lane alone pays ~230 (and ~200 more for every barrier wait whose result it consumes).
__device__ __forceinline__ void mma_f16_ts_elect(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, e;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The MMA issued by the first CTA of a pair for both: M = 256 (rows 0..127 from this CTA's tensor memory, 128..255 from
// the peer's, at the same address), B's N rows split between the two CTAs' shared memories (same offset), each CTA's
// accumulator holds its own 128 rows.
__device__ __forceinline__ void mma_f16_ts_pair_elect(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                      uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, e;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "@e tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_commit_elect(uint32_t bar) {
    asm volatile(
        "{\n\t"
        ".reg .pred e;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
        "}\n" ::"r"(bar)
        : "memory");
}
// The commit for MMAs issued for a CTA pair: the barrier at this shared-memory offset arrives in both CTAs.
__device__ __forceinline__ void tc_commit_pair_elect(uint32_t bar) {
    asm volatile(
        "{\n\t"
        ".reg .pred e;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "@e tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n\t"
        "}\n" ::"r"(bar), "h"((uint16_t)3)
        : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[tmem] * B[smem descriptor]; fp16 inputs, fp32 accumulate; one thread issues it.
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[smem descriptor] * B[smem descriptor]; 8-, 6- or 4-bit floating-point inputs (each operand its own
// format, given in the instruction descriptor), fp32 accumulate, K = 32 per instruction; one thread issues it.
__device__ __forceinline__ void mma_f8f6f4_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The same for a whole converged warp with one elected lane issuing (see mma_f16_ts_elect).
__device__ __forceinline__ void mma_f8f6f4_ss_elect(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                    uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, e;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Shared-memory matrix descriptor of a K-major tile stored with the 128-byte swizzle: rows of
// 128 bytes (64 fp16), 8-row groups 1024 bytes apart, tile base 1024-byte aligned.
__device__ __forceinline__ uint64_t smem_desc_k_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);   // start address, 16-byte units
    d |= static_cast<uint64_t>(1) << 16;                        // leading byte offset (unused with swizzle)
    d |= static_cast<uint64_t>(1024 >> 4) << 32;                // stride byte offset: next 8-row group
    d |= static_cast<uint64_t>(1) << 46;                        // descriptor version of sm_100
    d |= static_cast<uint64_t>(2) << 61;                        // layout type: 128-byte swizzle
    return d;
}

// Instruction descriptor of kind::f16: fp16 A and B, both K-major, fp32 accumulator.
__device__ __host__ constexpr uint32_t idesc_f16_f32(uint32_t m, uint32_t n) {
    return (1u << 4)            // D format: fp32
           | (0u << 7)          // A format: fp16
           | (0u << 10)         // B format: fp16
           | (0u << 15)         // A K-major
           | (0u << 16)         // B K-major
           | ((n >> 3) << 17)   // N / 8
           | ((m >> 4) << 24);  // M / 16
}

// Instruction descriptor of kind::f8f6f4: operand formats 0 = e4m3, 1 = e5m2, 3 = e2m3, 4 = e3m2, 5 = e2m1; both
// operands K-major, fp32 accumulator.
constexpr uint32_t kFmtE4M3 = 0, kFmtE5M2 = 1, kFmtE2M3 = 3, kFmtE3M2 = 4, kFmtE2M1 = 5;
__device__ __host__ constexpr uint32_t idesc_f8f6f4_f32(uint32_t a_format, uint32_t b_format, uint32_t m, uint32_t n) {
    return (1u << 4) | (a_format << 7) | (b_format << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// One warp stores, for the 16 TMEM lanes starting at the lane of `taddr`, 32 consecutive 32-bit
// columns.  Thread 4g+t supplies v[2c+hr] for lane (g + 8*hr), column (t + 4c), c = 0..7.
__device__ __forceinline__ void tmem_st_16x128b_x8(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.16x128b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, "
        "%15, %16};" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
        "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}
// One warp loads, for its 32 TMEM lanes (thread i <-> lane base+i), 16 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, "
        "%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}

// CH consecutive columns for the warp's 32 lanes.
template <int CH>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&v)[CH]) {
    static_assert(CH == 16, "chunk width");
    tmem_ld_32x32b_x16(taddr, v);
}

}  // namespace ptx
