/*
 * TEST INFRASTRUCTURE ONLY.  CPU restatement of the FPx (e3m2 / e2m2) weight
 * prepacking and dequantisation algorithms of usyd-fsalab/fp6_llm, in plain C.
 * Nothing in the shipped library may link, import or call this file; it is the
 * checker that the CUDA path is compared against.
 *
 * Parity status: PINNED.  tests/test_oracle.py checks this file byte-for-byte
 * against (a) the reference's own CPU code compiled from its sources
 * (oracle/_ref, see oracle/Makefile), (b) the known-answer words in the
 * reference's tests (tests/python/kernel_test_fpx.py:92-107,114-131) and
 * (c) fixtures under tests/golden/ that were produced by the reference code.
 *
 * Reference functions restated here (paths relative to the reference tree):
 *   fp6_llm/csrc/utils/common.h:4-19            Extract_X_Bits_To_A_Byte
 *   fp6_llm/csrc/utils/weight_prepacking.h:23-35   Extract_segments_from_8_padded_fpx
 *   fp6_llm/csrc/utils/weight_prepacking.h:39-85   Assign_32_FPx_To_4_Thread
 *   fp6_llm/csrc/utils/weight_prepacking.h:87-116  BitInterleaving_x_bit
 *   fp6_llm/csrc/utils/weight_prepacking.h:118-196 weight_matrix_prepacking_x_bit
 *   fp6_llm/csrc/utils/weight_dequant.h:10-48      DeQuantMatrix_FPx_To_FP16
 *   fp6_llm/csrc/include/kernel_reduction.cuh:28-47 SplitK_Reduction (fp32 sum, one rn)
 */
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ---------- IEEE binary16 <-> binary32, round-to-nearest-even ---------- */

static float half_bits_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            man &= 0x3ffu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

static uint16_t float_to_half_bits_rn(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    uint32_t absx = x & 0x7fffffffu;
    if (absx >= 0x7f800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7c00u | ((absx > 0x7f800000u) ? 0x200u : 0));
    }
    if (absx >= 0x477ff000u) { /* >= 65520 rounds to inf */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (absx < 0x33000001u) { /* <= 2^-25: rounds to zero (tie at 2^-25 goes to even = 0) */
        return sign;
    }
    int32_t e = (int32_t)(absx >> 23) - 127;
    uint32_t m = (absx & 0x7fffffu) | 0x800000u; /* 24-bit significand */
    int shift;
    uint32_t hexp;
    if (e < -14) { /* subnormal result */
        shift = 13 + (-14 - e);
        hexp = 0;
    } else {
        shift = 13;
        hexp = (uint32_t)(e + 15);
    }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) q++;
    uint32_t res;
    if (hexp == 0) {
        res = q; /* may carry into exponent 1, which is correct */
    } else {
        res = ((hexp - 1) << 10) + q; /* q includes the hidden bit (0x400) */
    }
    return (uint16_t)(sign | res);
}

/* ---------- bit-field helpers ---------- */

/* common.h:4-19.  Reads the bw-bit code that starts `bit_off` bits into
 * bytes[byte_off] (MSB first) and returns it left-aligned in a byte.  Unlike
 * the reference this never touches bytes[byte_off+1] when the field does not
 * reach it, so it has no one-byte over-read at the end of the buffer. */
static uint8_t code_left_aligned(const uint8_t* bytes, size_t byte_off, int bit_off, int bw) {
    uint32_t two = (uint32_t)bytes[byte_off] << 8;
    if (bit_off + bw > 8) two |= bytes[byte_off + 1];
    uint32_t v = (two << bit_off) & 0xffffu;
    return (uint8_t)((v >> 8) & (0xffu << (8 - bw)));
}

/* weight_prepacking.h:23-35.  From 8 left-aligned codes take the `seg_w` bits
 * that start `seg_off` bits below the top, and pack them MSB-first. */
static void pack_segment(uint8_t* seg_out, const uint8_t codes[8], int seg_w, int seg_off) {
    for (int i = 0; i < seg_w; i++) seg_out[i] = 0;
    for (int i = 0; i < 8; i++) {
        uint32_t s = ((uint32_t)codes[i] << seg_off) & 0xffu;
        s &= (0xff00u >> seg_w) & 0xffu;
        int pos = i * seg_w;
        seg_out[pos / 8] |= (uint8_t)(s >> (pos % 8));
    }
}

/* weight_prepacking.h:87-116.  Re-orders the 32/seg_w fields of one 32-bit
 * word so that masking the top seg_w bits of every byte, then shifting left,
 * walks the fields in the order the GPU dequantiser needs them. */
static uint32_t interleave_word(uint32_t in, int seg_w) {
    static const int order1[32] = {2, 6, 10, 14, 18, 22, 26, 30, 4, 8, 12, 16, 20, 24, 28, 32,
                                   1, 5, 9, 13, 17, 21, 25, 29, 3, 7, 11, 15, 19, 23, 27, 31};
    static const int order2[16] = {2, 6, 10, 14, 4, 8, 12, 16, 1, 5, 9, 13, 3, 7, 11, 15};
    static const int order4[8] = {2, 6, 4, 8, 1, 5, 3, 7};
    const int* order = seg_w == 1 ? order1 : (seg_w == 2 ? order2 : order4);
    uint32_t top = ~0u << (32 - seg_w);
    uint32_t out = 0;
    for (int i = 0; i < 32 / seg_w; i++) {
        uint32_t field = (in << (seg_w * (order[i] - 1))) & top;
        out |= field >> (i * seg_w);
    }
    return out;
}

/* The reference's templates take any code narrower than 8 bits (weight_prepacking.h:124-128, weight_dequant.h:14-15);
 * its run-time dispatch knows e3m2 and e2m2.  Restated here for those two and for e2m1, e3m1 and e2m3. */
static int supported(int e, int m) {
    return (m == 2 && (e == 3 || e == 2)) || (m == 1 && (e == 2 || e == 3)) || (m == 3 && e == 2);
}

/*
 * weight_prepacking.h:118-196.  `in`: rows x (cols*bw/8) bytes, each row an
 * MSB-first stream of bw-bit codes.  `out`: same number of bytes, laid out as
 * [1-bit region][2-bit region][4-bit region] (a region exists iff that bit of
 * bw is set).  in == out is allowed (the input is copied first).
 * Returns 0, or -1 for an unsupported format / shape.
 */
int oracle_prepack(int e_bits, int m_bits, uint8_t* out, const uint8_t* in, size_t rows, size_t cols) {
    if (!supported(e_bits, m_bits) || rows % 64 || cols % 64) return -1;
    const int bw = 1 + e_bits + m_bits;
    const size_t total = rows * cols * bw / 8;
    uint8_t* src = (uint8_t*)malloc(total + 1);
    if (!src) return -1;
    memcpy(src, in, total);
    src[total] = 0;

    const int seg_ws[3] = {1, 2, 4};
    size_t region_off[3];
    size_t off = 0;
    for (int s = 0; s < 3; s++) {
        region_off[s] = off;
        if (bw & seg_ws[s]) off += rows * cols * seg_ws[s] / 8;
    }
    /* per-lane byte streams, one set per segment width (Pass-1 target) */
    uint8_t* lanes[3] = {0, 0, 0};
    size_t lane_bytes[3] = {0, 0, 0};
    for (int s = 0; s < 3; s++) {
        if (!(bw & seg_ws[s])) continue;
        lane_bytes[s] = rows * cols * seg_ws[s] / 8 / 32;
        lanes[s] = (uint8_t*)malloc(lane_bytes[s] * 32);
        if (!lanes[s]) {
            for (int t = 0; t < s; t++) free(lanes[t]);
            free(src);
            return -1;
        }
    }
    const size_t row_bytes = cols * bw / 8;
    /* Pass-1 (:141-157): walk 64-row blocks, 16-col blocks, 16-row sub-blocks;
     * in each 16x16 block, "thread" 4*l+t owns rows {l, l+8} x cols {2t,2t+1,2t+8,2t+9}. */
    size_t block_seq = 0;
    for (size_t i = 0; i < rows / 64; i++)
        for (size_t j = 0; j < cols / 16; j++)
            for (size_t k = 0; k < 4; k++, block_seq++) {
                const size_t r0 = i * 64 + k * 16, c0 = j * 16;
                for (int l = 0; l < 8; l++)
                    for (int t = 0; t < 4; t++) {
                        uint8_t codes[8];
                        for (int x = 0; x < 8; x++) {
                            /* x/2: 0 -> (row l, cols 0-7), 1 -> (row l+8, cols 0-7),
                             *      2 -> (row l, cols 8-15), 3 -> (row l+8, cols 8-15)  (:145-152) */
                            size_t r = r0 + (size_t)l + (((x / 2) & 1) ? 8 : 0);
                            size_t c = c0 + (((x / 2) & 2) ? 8 : 0) + (size_t)(t * 2 + x % 2);
                            size_t bit = c * bw;
                            codes[x] = code_left_aligned(src + r * row_bytes, bit / 8, (int)(bit % 8), bw);
                        }
                        int lane = l * 4 + t;
                        int seg_off = 0;
                        for (int s = 0; s < 3; s++) {
                            int w = seg_ws[s];
                            if (!(bw & w)) continue;
                            uint8_t seg[4];
                            pack_segment(seg, codes, w, seg_off); /* offsets bw&0, bw&1, bw&3 (:64-66) */
                            seg_off += w;
                            memcpy(lanes[s] + (size_t)lane * lane_bytes[s] + block_seq * w, seg, (size_t)w);
                        }
                    }
            }
    /* Pass-2 (:171-185): interleave the 32 lanes at 4-byte granularity, bytes reversed in each word.
     * Pass-3 (:187-195): bit interleave inside every 32-bit word. */
    for (int s = 0; s < 3; s++) {
        int w = seg_ws[s];
        if (!(bw & w)) continue;
        uint8_t* region = out + region_off[s];
        for (size_t word = 0; word < lane_bytes[s] / 4; word++)
            for (int t = 0; t < 32; t++) {
                const uint8_t* p = lanes[s] + (size_t)t * lane_bytes[s] + word * 4;
                /* byte b of the stream lands at byte (3-b) => the stream is the word, MSB first */
                uint32_t v = ((uint32_t)p[0] << 24) | ((uint32_t)p[1] << 16) | ((uint32_t)p[2] << 8) | p[3];
                v = interleave_word(v, w);
                uint8_t* q = region + word * 128 + (size_t)t * 4;
                q[0] = (uint8_t)v; q[1] = (uint8_t)(v >> 8); q[2] = (uint8_t)(v >> 16); q[3] = (uint8_t)(v >> 24);
            }
        free(lanes[s]);
    }
    free(src);
    return 0;
}

/*
 * weight_dequant.h:10-48.  `in` is the UNPACKED stream (before prepacking).
 * out[r*cols+c] = rn_half( float(h) * 2^bias * float(scale[r]) ) where h is the
 * code moved into fp16 bit positions: sign kept, the rest shifted right by 5-E
 * (:30-40), bias = 16 - 2^(E-1) (:34-35).  fp16 values are passed as raw bits.
 */
int oracle_dequant(int e_bits, int m_bits, uint16_t* out, const uint8_t* in, size_t rows, size_t cols,
                   const uint16_t* scale) {
    if (!supported(e_bits, m_bits) || rows % 64 || cols % 64) return -1;
    const int bw = 1 + e_bits + m_bits;
    const size_t row_bytes = cols * bw / 8;
    const float bias = (float)(1u << (16 - (1 << (e_bits - 1))));
    for (size_t r = 0; r < rows; r++) {
        const float s = half_bits_to_float(scale[r]);
        for (size_t c = 0; c < cols; c++) {
            size_t bit = c * bw;
            uint8_t code = code_left_aligned(in + r * row_bytes, bit / 8, (int)(bit % 8), bw);
            uint32_t v = (uint32_t)code << 8; /* code left-aligned in 16 bits */
            uint16_t h = (uint16_t)((v & 0x8000u) | ((v & 0x7fffu) >> (5 - e_bits)));
            float f = half_bits_to_float(h) * bias * s;
            out[r * cols + c] = float_to_half_bits_rn(f);
        }
    }
    return 0;
}

/* kernel_reduction.cuh:28-47: C[i] = rn_half(sum over splits, ascending, in fp32). */
void oracle_splitk_reduce(uint16_t* out, const float* partials, size_t elems, int split_k) {
    for (size_t i = 0; i < elems; i++) {
        float acc = 0.0f;
        for (int s = 0; s < split_k; s++) acc += partials[(size_t)s * elems + i];
        out[i] = float_to_half_bits_rn(acc);
    }
}

/* Exposed so the tests can pin the fp16 conversions against numpy. */
uint16_t oracle_float_to_half(float f) { return float_to_half_bits_rn(f); }
float oracle_half_to_float(uint16_t h) { return half_bits_to_float(h); }
