// Index arithmetic and bit manipulation of the FPx prepacked weight format, shared by the
// device kernels and by a host-compiled test harness (everything here is integer-only and
// host/device callable).
//
// The format is the one produced by the reference packer
// (fp6_llm/csrc/utils/weight_prepacking.h:118-196) and consumed by its GPU dequantiser
// (fp6_llm/csrc/include/utils_parallel_dequant.cuh:44-99):
//   * a bw-bit code [sign | E exponent bits | M mantissa bits] is cut, MSB first, into a 1-bit,
//     a 2-bit and a 4-bit segment (a segment exists iff that bit of bw is set);
//   * the packed buffer is [1-bit region][2-bit region][4-bit region] over the whole matrix;
//   * inside a region the unit is a 32-bit word owned by one of 32 "lanes"; lane 4g+t owns, in
//     every 16x16 block, rows {g, g+8} x cols {2t, 2t+1, 2t+8, 2t+9} (8 codes);
//   * blocks are ordered (64-row block i, 16-col block j, 16-row sub-block k); a word holds the
//     segments of 32/w codes, i.e. of 4/w... consecutive blocks, bit-interleaved so that masking
//     the top w bits of every byte and then shifting left by w walks the codes in use order.
#pragma once
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define FPX_HD __host__ __device__ __forceinline__
#else
#define FPX_HD inline
#endif

namespace fpx {

constexpr int kRowsPerBlock = 64;   // rows whose data is contiguous along K in every region
constexpr int kKBlock = 64;         // K extent of one pipeline stage (4 column blocks of 16)

FPX_HD constexpr int bit_width(int e_bits, int m_bits) { return 1 + e_bits + m_bits; }
FPX_HD constexpr bool has_seg(int bw, int w) { return (bw & w) != 0; }

// Byte offset of the region that stores the w-bit segments (w in {1,2,4}).
FPX_HD uint64_t region_offset(int bw, int w, uint64_t rows, uint64_t cols) {
    uint64_t off = 0;
    if (w > 1 && has_seg(bw, 1)) off += rows * cols / 8;
    if (w > 2 && has_seg(bw, 2)) off += rows * cols / 4;
    return off;
}

// Bytes of one (64-row block x 64-K block) tile in the w-bit region: 64*64*w/8.
FPX_HD constexpr uint32_t tile_bytes(int w) { return 512u * (uint32_t)w; }

// Number of low bits of the code that lie below the w-bit segment.
FPX_HD constexpr int seg_shift(int bw, int w) {
    // segments are taken MSB first in the order 1, 2, 4
    return w == 4 ? 0 : (w == 2 ? (has_seg(bw, 4) ? 4 : 0) : ((has_seg(bw, 2) ? 2 : 0) + (has_seg(bw, 4) ? 4 : 0)));
}

struct FieldSource {
    uint32_t row;   // absolute row of the code
    uint32_t col;   // absolute column of the code
};

// For the 32-bit word `word_in_lane` of lane `lane` in the w-bit region, the code whose
// segment sits in field p (field p occupies bits [32-(p+1)w, 32-pw) of the little-endian word).
FPX_HD FieldSource field_source(int w, uint64_t word_in_lane, int lane, int p, uint32_t cols) {
    const int fields_per_byte = 8 / w;
    const int byteidx = p / fields_per_byte;       // byte of the word, counted from the MSB
    const int n = p % fields_per_byte;             // dequant iteration that consumes this field
    // the dequantiser reads codes (4n+1, 4n+3, 4n, 4n+2) from the bytes (MSB .. LSB) of iteration n
    const int q = (byteidx == 0) ? 1 : (byteidx == 1) ? 3 : (byteidx == 2) ? 0 : 2;
    const int f = 4 * n + q;                       // code index inside the word, in use order
    const int e = f % 8;                           // index among the lane's 8 codes of one 16x16 block
    const uint64_t b = word_in_lane * (uint64_t)(4 / w) + (uint64_t)(f / 8);   // 16x16 block, packing order
    const uint32_t k = (uint32_t)(b % 4);
    const uint64_t ij = b / 4;
    const uint32_t i = (uint32_t)(ij / (cols / 16)), j = (uint32_t)(ij % (cols / 16));
    const uint32_t g = (uint32_t)lane / 4, t = (uint32_t)lane % 4;
    FieldSource s;
    s.row = 64 * i + 16 * k + 8 * (uint32_t)((e / 2) % 2) + g;
    s.col = 16 * j + 8 * (uint32_t)(e / 4) + 2 * t + (uint32_t)(e % 2);
    return s;
}

// The bw-bit code at column c of a row stored as an MSB-first bit stream.
FPX_HD uint32_t read_code(const uint8_t* row, uint32_t c, int bw) {
    const uint32_t bit = c * (uint32_t)bw;
    const uint32_t byte = bit >> 3, off = bit & 7;
    uint32_t two = (uint32_t)row[byte] << 8;
    if (off + (uint32_t)bw > 8) two |= row[byte + 1];
    return (two >> (16 - off - (uint32_t)bw)) & ((1u << bw) - 1u);
}

// ---------------------------------------------------------------------------------------------
// Dequantisation of four codes at a time, as raw fp16 bit patterns before any scaling.
//
// A code becomes the fp16 pattern  sign | (exponent,mantissa bits) >> (5 - E)  (the reference's
// FPx_FP16_Cast_4Way, utils_parallel_dequant.cuh:13-28), so for E=3,M=2 the high byte of the fp16
// is [s 0 0 e2 e1 e0 m1 m0] and for E=2,M=2 it is [s 0 0 0 e1 e0 m1 m0]; the low byte is zero.
// The value is then 2^-(16 - 2^(E-1)) times the FPx value.
//
// `hi4` holds in every byte the 4-bit segment of one code (already masked to the low nibble).
// For e3m2, `s_src` has the sign at bit 7 of every byte and `e_src` has e2 at bit 4 of every byte
// (other bits arbitrary).  For e2m2, `s_src` has the sign at bit 7 (e_src unused).
// Returns the four high bytes; out_lo/out_hi expand them into two half2 patterns:
//   out_lo = (byte1 -> low half, byte3 -> high half), out_hi = (byte0 -> low half, byte2 -> high half).
FPX_HD uint32_t stitch_e3m2(uint32_t s_src, uint32_t e_src, uint32_t nib) {
    return (s_src & 0x80808080u) | ((e_src & 0x10101010u) | nib);
}
FPX_HD uint32_t stitch_e2m2(uint32_t s_src, uint32_t nib) { return (s_src & 0x80808080u) | nib; }

FPX_HD uint32_t expand_13(uint32_t y) {   // bytes 3,1 -> high bytes of the two halves
#if defined(__CUDA_ARCH__)
    return __byte_perm(y, 0u, 0x3414);
#else
    return y & 0xff00ff00u;
#endif
}
FPX_HD uint32_t expand_02(uint32_t y) {   // bytes 2,0 -> high bytes of the two halves
#if defined(__CUDA_ARCH__)
    return __byte_perm(y, 0u, 0x2404);
#else
    return (y << 8) & 0xff00ff00u;
#endif
}

// Unpack the 16 codes that one lane owns in two vertically adjacent 16x16 blocks (sub-blocks
// 2h and 2h+1 of a 64-row block, same 16 columns) into eight half2 bit patterns
//   out[4*kk + 0..3] = A-fragment registers a0..a3 of sub-block 2h+kk:
//   a0 = (row g,   cols 2t,2t+1)   a1 = (row g+8, cols 2t,2t+1)
//   a2 = (row g,   cols 2t+8,2t+9) a3 = (row g+8, cols 2t+8,2t+9)
// w4a / w4b: the lane's 4-bit words of sub-blocks 2h and 2h+1.
// w2: the lane's 2-bit word that covers both sub-blocks (e3m2 only).
// w1: the lane's 1-bit word of the column block, which covers all four sub-blocks (e2m2 only);
//     h selects its upper (h=0) or lower (h=1) half of the iterations.
template <int E_BITS>
FPX_HD void unpack16(uint32_t w4a, uint32_t w4b, uint32_t w2, uint32_t w1, int h, uint32_t out[8]) {
    const uint32_t nib0 = (w4a >> 4) & 0x0f0f0f0fu, nib1 = w4a & 0x0f0f0f0fu;
    const uint32_t nib2 = (w4b >> 4) & 0x0f0f0f0fu, nib3 = w4b & 0x0f0f0f0fu;
    uint32_t y0, y1, y2, y3;
    if (E_BITS == 3) {
        // iteration n' (0..3) has the sign at bit 7-2n' and e2 at bit 6-2n' of every byte of w2
        y0 = stitch_e3m2(w2, w2 >> 2, nib0);
        y1 = stitch_e3m2(w2 << 2, w2, nib1);
        y2 = stitch_e3m2(w2 << 4, w2 << 2, nib2);
        y3 = stitch_e3m2(w2 << 6, w2 << 4, nib3);
    } else {
        // iteration i (0..7) of the column block has the sign at bit 7-i; this lane pair uses 4h..4h+3
        const uint32_t s = w1 << (4 * h);
        y0 = stitch_e2m2(s, nib0);
        y1 = stitch_e2m2(s << 1, nib1);
        y2 = stitch_e2m2(s << 2, nib2);
        y3 = stitch_e2m2(s << 3, nib3);
    }
    out[0] = expand_13(y0); out[1] = expand_02(y0); out[2] = expand_13(y1); out[3] = expand_02(y1);
    out[4] = expand_13(y2); out[5] = expand_02(y2); out[6] = expand_13(y3); out[7] = expand_02(y3);
}

// The general case: any format whose code is at most 6 bits wide (e2m1, e3m1, e2m3 besides the two above).  Every
// byte first receives its code left-aligned, [code | 0...], the way the reference's dequantiser assembles it
// (utils_parallel_dequant.cuh:63-86: the 1-, 2- and 4-bit segments are masked at the top of each byte and shifted
// right by the width of the segments above them); the bytes are then spread into 16-bit lanes and everything but
// the sign is shifted right by 5 - E (FPx_FP16_Cast_4Way, :13-28).  About twice the instructions of the two
// sequences above, which exist because e3m2 and e2m2 are the formats that matter.
template <int E_BITS, int M_BITS>
FPX_HD void unpack16_generic(uint32_t w4a, uint32_t w4b, uint32_t w2, uint32_t w1, int h, uint32_t out[8]) {
    constexpr int BW = 1 + E_BITS + M_BITS;
    static_assert(BW >= 4 && BW <= 6 && E_BITS >= 1 && E_BITS <= 5, "one or two segments: 4-bit, 1+4-bit or 2+4-bit codes");
    constexpr int kAbove4 = BW - 4;   // bits of the code above its 4-bit segment (0, 1 or 2)
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
    for (int n = 0; n < 4; n++) {
        const uint32_t w4 = n < 2 ? w4a : w4b;
        const uint32_t nib = ((n & 1) ? (w4 << 4) : w4) & 0xf0f0f0f0u;     // the 4-bit segment at the top of every byte
        uint32_t code = nib >> kAbove4;
        if (BW == 5) code |= (w1 << (4 * h + n)) & 0x80808080u;           // iteration 4h+n of the 1-bit word
        if (BW == 6) code |= (w2 << (2 * n)) & 0xc0c0c0c0u;               // iteration n of the 2-bit word
        // bytes 3,1 and bytes 2,0 as the high bytes of two 16-bit lanes each; sign stays, the rest moves down
        const uint32_t a = expand_13(code), b = expand_02(code);
        out[2 * n] = (a & 0x80008000u) | ((a & 0x7fff7fffu) >> (5 - E_BITS));
        out[2 * n + 1] = (b & 0x80008000u) | ((b & 0x7fff7fffu) >> (5 - E_BITS));
    }
}

// What the kernels call: the short sequences for e3m2 / e2m2, the general one otherwise.
template <int E_BITS, int M_BITS>
FPX_HD void unpack16_any(uint32_t w4a, uint32_t w4b, uint32_t w2, uint32_t w1, int h, uint32_t out[8]) {
    if (M_BITS == 2 && (E_BITS == 3 || E_BITS == 2)) unpack16<(M_BITS == 2 && E_BITS == 2) ? 2 : 3>(w4a, w4b, w2, w1, h, out);
    else unpack16_generic<E_BITS, M_BITS>(w4a, w4b, w2, w1, h, out);
}

// The same unpack for the GEMM's inner loop, in fewer instructions and with part of them moved off the logic pipe.
// On B200 the logic operations (LOP3, PRMT, funnel shifts) issue at 64 lanes per clock and SM, and integer
// multiply-adds issue at the same rate on the other (FMA) pipe; the sequence above keeps only the logic pipe busy.
// Here the sign and exponent bits are brought into one word once, the left shifts are multiplications, and the low
// nibbles are what is left of the word after the high ones (w - 16 * high).  The multipliers come in through `k`
// (kernel parameters on the device), so that the compiler cannot turn them back into shifts; the values are fixed:
//   m4 = 4, m16 = 16, mneg16 = -16, sign[i] = 1 << (4h + i)  (e2m2 only; h as above).
struct UnpackMul {
    uint32_t m4, m16, mneg16;
    uint32_t sign[4];
};
FPX_HD UnpackMul unpack_mul_values(int h) {
    UnpackMul k;
    k.m4 = 4u; k.m16 = 16u; k.mneg16 = 0u - 16u;
    for (int i = 0; i < 4; i++) k.sign[i] = 1u << (4 * h + i);
    return k;
}
FPX_HD uint32_t mul_add(uint32_t a, uint32_t b, uint32_t c) {
#if defined(__CUDA_ARCH__)
    uint32_t r;
    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
#else
    return a * b + c;
#endif
}
FPX_HD uint32_t rot_left(uint32_t x, int n) {
#if defined(__CUDA_ARCH__)
    return __funnelshift_l(x, x, n);
#else
    return (x << n) | (x >> (32 - n));
#endif
}
template <int E_BITS>
FPX_HD void unpack16_mul(uint32_t w4a, uint32_t w4b, uint32_t w2, uint32_t w1, const UnpackMul& k, uint32_t out[8]) {
    const uint32_t nib0 = (w4a >> 4) & 0x0f0f0f0fu, nib2 = (w4b >> 4) & 0x0f0f0f0fu;
    const uint32_t nib1 = mul_add(nib0, k.mneg16, w4a), nib3 = mul_add(nib2, k.mneg16, w4b);
    uint32_t y[4];
    if (E_BITS == 3) {
        // se: the sign of iteration n' at bit 7-2n' and its e2 three bits below (at bit 4-2n'; for n' = 3 that is bit 6 of
        // the byte below, and of the top byte for the lowest one), so one shift or rotation by 2n' puts both in place
        const uint32_t se = (w2 & 0xaaaaaaaau) | rot_left(w2 & 0x55555555u, 30);
        y[0] = (se & 0x90909090u) | nib0;
        y[1] = (mul_add(se, k.m4, 0u) & 0x90909090u) | nib1;
        y[2] = (mul_add(se, k.m16, 0u) & 0x90909090u) | nib2;
        y[3] = (rot_left(se, 6) & 0x90909090u) | nib3;
    } else {
        y[0] = (mul_add(w1, k.sign[0], 0u) & 0x80808080u) | nib0;
        y[1] = (mul_add(w1, k.sign[1], 0u) & 0x80808080u) | nib1;
        y[2] = (mul_add(w1, k.sign[2], 0u) & 0x80808080u) | nib2;
        y[3] = (mul_add(w1, k.sign[3], 0u) & 0x80808080u) | nib3;
    }
    out[0] = expand_13(y[0]); out[1] = expand_02(y[0]); out[2] = expand_13(y[1]); out[3] = expand_02(y[1]);
    out[4] = expand_13(y[2]); out[5] = expand_02(y[2]); out[6] = expand_13(y[3]); out[7] = expand_02(y[3]);
}

// Round-to-nearest quantiser.  Value of the non-negative code c = (e << M) | m: subnormals m / 2^M * 2^(1-bias),
// otherwise (1 + m / 2^M) * 2^(e-bias), bias = 2^(E-1) - 1 (28 is the largest e3m2 magnitude, 7 the largest e2m2 one).
FPX_HD float fpx_magnitude(int e_bits, int m_bits, int c) {
    const int bias = (1 << (e_bits - 1)) - 1;
    const int e = c >> m_bits, m = c & ((1 << m_bits) - 1);
    const int p = (e == 0 ? 1 : e) - bias - m_bits;          // the value is (e == 0 ? m : 2^M + m) * 2^p
    const float unit = p >= 0 ? (float)(1 << p) : 1.0f / (float)(1 << -p);
    return (float)(e == 0 ? m : (1 << m_bits) + m) * unit;
}
// Code (sign bit included) of the quotient q = w / scale: the nearest magnitude, ties to the even code, saturating;
// the sign bit is the sign bit of q (so -0 keeps its sign).
FPX_HD uint32_t quantize_rtn_code(int e_bits, int m_bits, float q) {
    const int codes = 1 << (e_bits + m_bits);
    const float a = q < 0.0f ? -q : q;
    int below = 0, not_above = 0;                            // midpoints < a, midpoints <= a
    for (int c = 0; c + 1 < codes; c++) {
        const float mid = 0.5f * (fpx_magnitude(e_bits, m_bits, c) + fpx_magnitude(e_bits, m_bits, c + 1));
        below += mid < a ? 1 : 0;
        not_above += mid <= a ? 1 : 0;
    }
    const uint32_t mag = (uint32_t)((below & 1) ? not_above : below);   // they differ only on an exact tie
    uint32_t bits;
#if defined(__CUDA_ARCH__)
    bits = __float_as_uint(q);
#else
    memcpy(&bits, &q, sizeof(bits));
#endif
    return mag | ((bits >> 31) ? (uint32_t)codes : 0u);
}

// 2^(16 - 2^(E-1)) as an fp16 bit pattern: 2^12 for E=3, 2^14 for E=2
// (the reference's BIAS, utils_parallel_dequant.cuh:32-33).
FPX_HD constexpr uint16_t bias_half_bits(int e_bits) {
    return (uint16_t)(((16 - (1 << (e_bits - 1))) + 15) << 10);
}

// Split-K: K is cut in 64-wide blocks; split z of `splits` gets base (+1 for the first `extra`)
// blocks, like the reference kernel (fp6_llm/csrc/include/kernel_matmul.cuh:60-70).
FPX_HD void split_range(uint32_t k_blocks, uint32_t splits, uint32_t z, uint32_t* begin, uint32_t* count) {
    const uint32_t base = k_blocks / splits, extra = k_blocks % splits;
    *count = base + (z < extra ? 1u : 0u);
    *begin = z * base + (z < extra ? z : extra);
}

// ---------------------------------------------------------------------------------------------
// Work decomposition of the persistent GEMM kernel.
//
// An output tile is 128 rows x n_tile columns; a *unit* is one 64-wide K block of one tile.  `grid`
// CTAs each walk a list of *segments* (tile, first K block, number of K blocks):
//   kClassic  the caller fixed split_k: item i = (tile i / split_k, split i % split_k), CTA c takes
//             items c, c + grid, ...; a split writes an fp32 partial [split][N][M] that a reduction
//             kernel sums (the reference's scheme, fp6_llm/csrc/fp6_linear.cu:81-99).
//   kStreamK  whole waves of tiles are taken data-parallel (CTA c takes tiles c, c + grid, ...), then
//             the units of the remaining tiles are dealt out evenly: CTA c gets units
//             [c*U/grid, (c+1)*U/grid) of the remainder.  A CTA's first and last remainder segment may
//             cover only part of a tile's K range; those go to partial slots 2c and 2c+1 and a fix-up
//             kernel sums the slots of every split tile in CTA order.
enum WorkMode : uint32_t { kClassic = 0, kStreamK = 1 };
constexpr uint32_t kPlanTableGrid = 256;   // largest grid for which a plan carries its table of remainder starts
enum OutKind : uint32_t { kOutDirect = 0, kOutSplitPartial = 1, kOutSlotPartial = 2 };

struct WorkPlan {
    uint32_t mode;
    uint32_t m_tiles;     // M / 128
    uint32_t n_tiles;     // ceil(N / n_tile)
    uint32_t kblocks;     // K / 64
    uint32_t split_k;     // kClassic only (1 <= split_k <= kblocks)
    uint32_t grid;        // number of CTAs
    // derived by plan_finalize (so that device code does not redo the divisions)
    uint32_t full_waves;  // tiles / grid
    uint32_t rem_tiles;   // tiles - full_waves * grid
    uint32_t rem_units32; // rem_tiles * kblocks when (rem_tiles * kblocks + 1) * grid fits 32 bits, else 0
    // kStreamK, grid <= kPlanTableGrid and kblocks < 65536: rem_start[c] = (remainder tile << 16) | K block at which
    // CTA c starts in the remainder (c == grid: the end), so that a CTA finds its work with two loads.
    uint32_t has_table;
    uint32_t rem_start[kPlanTableGrid + 1];
};

struct Segment {
    uint32_t tile;        // m_tile * n_tiles + n_tile
    uint32_t kb_begin;
    uint32_t nkb;         // > 0
    uint32_t out_kind;
    uint32_t out_index;   // split index (kOutSplitPartial) or slot (kOutSlotPartial)
};

FPX_HD uint32_t plan_tiles(const WorkPlan& p) { return p.m_tiles * p.n_tiles; }
FPX_HD uint64_t plan_rem_begin(const WorkPlan& p, uint32_t c);
FPX_HD void plan_finalize(WorkPlan* p) {
    p->full_waves = plan_tiles(*p) / p->grid;
    p->rem_tiles = plan_tiles(*p) - p->full_waves * p->grid;
    const uint64_t units = (uint64_t)p->rem_tiles * p->kblocks;
    p->rem_units32 = (units + 1) * p->grid <= 0xffffffffull ? (uint32_t)units : 0u;
    p->has_table = 0;
    if (p->mode == kStreamK && p->grid <= kPlanTableGrid && p->kblocks < 65536u) {
        for (uint32_t c = 0; c <= p->grid; c++) {
            const uint64_t u = plan_rem_begin(*p, c);
            p->rem_start[c] = ((uint32_t)(u / p->kblocks) << 16) | (uint32_t)(u % p->kblocks);
        }
        p->has_table = 1;
    }
}
FPX_HD uint32_t plan_full_waves(const WorkPlan& p) { return p.full_waves; }
FPX_HD uint32_t plan_rem_tiles(const WorkPlan& p) { return p.rem_tiles; }
// first remainder unit of CTA c (kStreamK); c == grid gives the total
FPX_HD uint64_t plan_rem_begin(const WorkPlan& p, uint32_t c) {
    if (p.rem_units32) return (uint64_t)(c * p.rem_units32 / p.grid);
    return (uint64_t)c * ((uint64_t)p.rem_tiles * p.kblocks) / p.grid;
}
// CTA that owns remainder unit u
FPX_HD uint32_t plan_rem_owner(const WorkPlan& p, uint64_t u) {
    if (p.rem_units32) return ((uint32_t)(u + 1) * p.grid - 1u) / p.rem_units32;
    const uint64_t total = (uint64_t)p.rem_tiles * p.kblocks;
    return (uint32_t)(((u + 1) * p.grid - 1) / total);
}

struct SegmentIter {
    uint32_t step;                 // segments handed out so far
    uint32_t cur_tile, cur_kb;     // kStreamK: next remainder unit to hand out, as (remainder tile, K block)
    uint32_t end_tile, end_kb;     // kStreamK: where this CTA's remainder units end
    uint32_t rem_first;            // 1 until the first remainder segment has been handed out
};

FPX_HD void plan_start(const WorkPlan& p, uint32_t cta, SegmentIter* it) {
    it->step = 0;
    it->rem_first = 1;
    it->cur_tile = it->cur_kb = it->end_tile = it->end_kb = 0;
    if (p.mode != kStreamK) return;
    if (p.has_table) {
        const uint32_t a = p.rem_start[cta], b = p.rem_start[cta + 1];
        it->cur_tile = a >> 16; it->cur_kb = a & 0xffffu;
        it->end_tile = b >> 16; it->end_kb = b & 0xffffu;
    } else {
        const uint64_t a = plan_rem_begin(p, cta), b = plan_rem_begin(p, cta + 1);
        it->cur_tile = (uint32_t)(a / p.kblocks); it->cur_kb = (uint32_t)(a % p.kblocks);
        it->end_tile = (uint32_t)(b / p.kblocks); it->end_kb = (uint32_t)(b % p.kblocks);
    }
}

// Next segment of CTA `cta`; false when the CTA is done.  Every role of the CTA calls this with its own
// iterator and sees the same sequence.
FPX_HD bool plan_next(const WorkPlan& p, uint32_t cta, SegmentIter* it, Segment* seg) {
    if (p.mode == kClassic) {
        const uint64_t item = (uint64_t)cta + (uint64_t)it->step * p.grid;
        if (item >= (uint64_t)plan_tiles(p) * p.split_k) return false;
        it->step++;
        seg->tile = (uint32_t)(item / p.split_k);
        seg->out_index = (uint32_t)(item % p.split_k);
        split_range(p.kblocks, p.split_k, seg->out_index, &seg->kb_begin, &seg->nkb);
        seg->out_kind = p.split_k > 1 ? kOutSplitPartial : kOutDirect;
        return true;
    }
    const uint32_t waves = plan_full_waves(p);
    if (it->step < waves) {
        seg->tile = cta + it->step * p.grid;
        seg->kb_begin = 0;
        seg->nkb = p.kblocks;
        seg->out_kind = kOutDirect;
        seg->out_index = 0;
        it->step++;
        return true;
    }
    if (it->cur_tile == it->end_tile && it->cur_kb >= it->end_kb) return false;
    if (it->cur_tile > it->end_tile) return false;
    const uint32_t kb = it->cur_kb;
    const uint32_t n = (it->cur_tile == it->end_tile ? it->end_kb : p.kblocks) - kb;
    seg->tile = waves * p.grid + it->cur_tile;
    seg->kb_begin = kb;
    seg->nkb = n;
    if (n == p.kblocks) {
        seg->out_kind = kOutDirect;
        seg->out_index = 0;
    } else {
        seg->out_kind = kOutSlotPartial;
        seg->out_index = 2 * cta + (it->rem_first ? 0u : 1u);
    }
    it->rem_first = 0;
    it->cur_kb = 0;
    if (kb + n == p.kblocks) it->cur_tile++;
    else it->cur_kb = kb + n;
    it->step++;
    return true;
}

// The order in which a CTA walks the K range of a segment: the i-th stage processed is stage (first + i) mod nstages
// (the order of the K blocks does not matter for the sum).  Every CTA starts at stage 0.  An earlier form started
// each CTA at a stage of its own ((cta * 7) mod nstages), so that the CTAs would not ask the same L2 lines for the same
// activation block at the same moment; measured, that is what they should do: with several token tiles (prefill) the
// activations are tens of MB, a K window of them stays in L2 where the whole matrix does not, and the weights fetched
// for one token tile are still there for the others (3-5 % faster on the 57344 x 8192 and 8192 x 28672 layers at
// 512-2048 tokens; 827 -> 670 us on 8192 x 28672 at 2048 tokens, whose 117 MB of activations otherwise thrash the L2);
// with one token tile (decode) the common start is 0-2 % faster too.  A loop of nothing but activation copies reaches
// 33 TB/s over the GPU when all CTAs ask for the same blocks and 23 TB/s when they are spread over K.
FPX_HD uint32_t plan_first_stage(const WorkPlan& p, uint32_t cta, uint32_t nstages) {
    (void)p; (void)cta; (void)nstages;
    return 0u;
}

// Fix-up side: for remainder tile r (0 <= r < plan_rem_tiles) the CTAs [*first, *last] hold its parts;
// *first == *last means one CTA computed the whole tile and stored it directly.
FPX_HD void plan_tile_owners(const WorkPlan& p, uint32_t r, uint32_t* first, uint32_t* last) {
    *first = plan_rem_owner(p, (uint64_t)r * p.kblocks);
    *last = plan_rem_owner(p, (uint64_t)(r + 1) * p.kblocks - 1);
}
// Slot in which CTA c left its part of remainder tile r (c in [first, last], first != last).  CTAs in
// that range whose unit range is empty (plan_rem_begin(c) == plan_rem_begin(c+1)) hold nothing.
FPX_HD uint32_t plan_tile_slot(const WorkPlan& p, uint32_t r, uint32_t c) {
    if (p.has_table) return ((p.rem_start[c] >> 16) == r) ? 2 * c : 2 * c + 1;
    const uint64_t begin = plan_rem_begin(p, c);
    return (begin / p.kblocks == r) ? 2 * c : 2 * c + 1;
}

}  // namespace fpx
