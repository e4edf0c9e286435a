// Host build of the integer-only layout/unpack code the CUDA kernels use (fp6_llm_b200/csrc/fpx_layout.h),
// so the index arithmetic can be checked against the CPU oracle without a GPU.  Test code only.
#include <cstdint>
#include <cstring>
#include <vector>

#include "../../fp6_llm_b200/csrc/fpx_layout.h"

using namespace fpx;

extern "C" {

// The prepack kernel's gather, word by word.
int harness_prepack(int e_bits, int m_bits, uint8_t* out, const uint8_t* in, uint32_t rows, uint32_t cols) {
    const int bw = 1 + e_bits + m_bits;
    const size_t row_bytes = (size_t)cols * bw / 8;
    std::vector<uint8_t> padded((size_t)rows * row_bytes + 1, 0);
    std::memcpy(padded.data(), in, (size_t)rows * row_bytes);
    for (int w = 1; w <= 4; w <<= 1) {
        if (!has_seg(bw, w)) continue;
        uint32_t* region = reinterpret_cast<uint32_t*>(out + region_offset(bw, w, rows, cols));
        const uint64_t words_per_lane = (uint64_t)rows * cols * w / 8 / 4 / 32;
        for (uint64_t wl = 0; wl < words_per_lane; wl++)
            for (int lane = 0; lane < 32; lane++) {
                uint32_t word = 0;
                for (int p = 0; p < 32 / w; p++) {
                    FieldSource s = field_source(w, wl, lane, p, cols);
                    uint32_t code = read_code(padded.data() + (size_t)s.row * row_bytes, s.col, bw);
                    word |= ((code >> seg_shift(bw, w)) & ((1u << w) - 1u)) << (32 - (p + 1) * w);
                }
                region[wl * 32 + lane] = word;
            }
    }
    return 0;
}

// The GEMM's unpack path: for every 128-row tile, 64-wide K block, tensor-memory quadrant q and lane, read
// the words the kernel reads (stage layout = [segment][row block][word]), run unpack16 and scatter the
// registers the way tcgen05.st.16x128b.x8 places them (thread 4g+t, register 2c+hr -> lane g+8hr, 32-bit
// column t+4c).  out_bits[row*cols+col] receives the unscaled fp16 pattern.
int harness_unpack(int e_bits, int m_bits, uint16_t* out_bits, const uint8_t* packed, uint32_t rows, uint32_t cols) {
    const int bw = 1 + e_bits + m_bits;
    if (rows % 128 || cols % 64) return -1;
    const uint32_t kblocks = cols / 64;
    for (uint32_t m_tile = 0; m_tile < rows / 128; m_tile++)
        for (uint32_t kb = 0; kb < kblocks; kb++)
            for (int q = 0; q < 4; q++)
                for (int lane = 0; lane < 32; lane++) {
                    const int h = q & 1, rb = q >> 1, g = lane >> 2, t = lane & 3;
                    const uint64_t tile = (uint64_t)(m_tile * 2 + rb) * kblocks + kb;
                    const uint32_t* r1 = reinterpret_cast<const uint32_t*>(packed + region_offset(bw, 1, rows, cols) + tile * tile_bytes(1));
                    const uint32_t* r2 = reinterpret_cast<const uint32_t*>(packed + region_offset(bw, 2, rows, cols) + tile * tile_bytes(2));
                    const uint32_t* r4 = reinterpret_cast<const uint32_t*>(packed + region_offset(bw, 4, rows, cols) + tile * tile_bytes(4));
                    uint32_t v[2][16];
                    for (int j = 0; j < 4; j++) {
                        uint32_t w4a = r4[(j * 4 + 2 * h + 0) * 32 + lane], w4b = r4[(j * 4 + 2 * h + 1) * 32 + lane];
                        uint32_t w2 = has_seg(bw, 2) ? r2[(j * 2 + h) * 32 + lane] : 0u;
                        uint32_t w1 = has_seg(bw, 1) ? r1[j * 32 + lane] : 0u;
                        uint32_t pat[8];
                        uint32_t pat2[8];
                        const UnpackMul km = unpack_mul_values(h);
                        if (m_bits == 2 && e_bits == 3) {
                            unpack16<3>(w4a, w4b, w2, w1, h, pat);
                            unpack16_mul<3>(w4a, w4b, w2, w1, km, pat2);      // the GEMM's multiply-based sequence: same registers
                            for (int i = 0; i < 8; i++) if (pat[i] != pat2[i]) return -2;
                            unpack16_generic<3, 2>(w4a, w4b, w2, w1, h, pat2);   // and so must the general sequence
                        } else if (m_bits == 2 && e_bits == 2) {
                            unpack16<2>(w4a, w4b, w2, w1, h, pat);
                            unpack16_mul<2>(w4a, w4b, w2, w1, km, pat2);
                            for (int i = 0; i < 8; i++) if (pat[i] != pat2[i]) return -2;
                            unpack16_generic<2, 2>(w4a, w4b, w2, w1, h, pat2);
                        } else if (e_bits == 2 && m_bits == 1) { unpack16_any<2, 1>(w4a, w4b, w2, w1, h, pat); unpack16_generic<2, 1>(w4a, w4b, w2, w1, h, pat2); }
                        else if (e_bits == 3 && m_bits == 1) { unpack16_any<3, 1>(w4a, w4b, w2, w1, h, pat); unpack16_generic<3, 1>(w4a, w4b, w2, w1, h, pat2); }
                        else { unpack16_any<2, 3>(w4a, w4b, w2, w1, h, pat); unpack16_generic<2, 3>(w4a, w4b, w2, w1, h, pat2); }
                        for (int i = 0; i < 8; i++) if (pat[i] != pat2[i]) return -3;
                        for (int kk = 0; kk < 2; kk++)
                            for (int i = 0; i < 4; i++) v[kk][4 * j + i] = pat[4 * kk + i];
                    }
                    for (int kk = 0; kk < 2; kk++)
                        for (int reg = 0; reg < 16; reg++) {
                            const int c = reg / 2, hr = reg % 2;
                            const uint32_t tm_lane = 32 * q + 16 * kk + g + 8 * hr;     // tensor-memory lane = tile row
                            const uint32_t col32 = t + 4 * c;                            // 32-bit column = K pair
                            const uint32_t row = m_tile * 128 + tm_lane;
                            const uint32_t col = kb * 64 + 2 * col32;
                            out_bits[(size_t)row * cols + col] = (uint16_t)(v[kk][reg] & 0xffffu);
                            out_bits[(size_t)row * cols + col + 1] = (uint16_t)(v[kk][reg] >> 16);
                        }
                }
    return 0;
}

void harness_split_range(uint32_t k_blocks, uint32_t splits, uint32_t z, uint32_t* begin, uint32_t* count) {
    split_range(k_blocks, splits, z, begin, count);
}

uint16_t harness_bias_bits(int e_bits) { return bias_half_bits(e_bits); }

// Walks the work plan of every CTA and checks it against the fix-up arithmetic:
//  * every unit (tile, K block) is covered exactly once;
//  * for every remainder tile, summing the slots the fix-up side computes covers exactly its K range.
// Returns 0 when consistent, else a small error code.
int harness_check_plan(uint32_t mode, uint32_t m_tiles, uint32_t n_tiles, uint32_t kblocks, uint32_t split_k,
                       uint32_t grid) {
    WorkPlan p{mode, m_tiles, n_tiles, kblocks, split_k, grid, 0, 0, 0};
    plan_finalize(&p);
    const uint32_t tiles = plan_tiles(p);
    std::vector<uint32_t> cover((size_t)tiles * kblocks, 0);
    std::vector<int64_t> slot_tile((size_t)2 * grid, -1);
    std::vector<uint32_t> slot_kb((size_t)2 * grid, 0);
    std::vector<uint32_t> direct(tiles, 0), split_seen((size_t)tiles * (split_k ? split_k : 1), 0);
    for (uint32_t c = 0; c < grid; c++) {
        SegmentIter it;
        plan_start(p, c, &it);
        Segment s;
        uint32_t count = 0;
        while (plan_next(p, c, &it, &s)) {
            if (s.nkb == 0 || s.tile >= tiles || s.kb_begin + s.nkb > kblocks) return 1;
            for (uint32_t k = 0; k < s.nkb; k++) cover[(size_t)s.tile * kblocks + s.kb_begin + k]++;
            if (s.out_kind == kOutDirect) {
                if (s.nkb != kblocks) return 2;
                direct[s.tile]++;
            } else if (s.out_kind == kOutSlotPartial) {
                if (mode != kStreamK || s.out_index >= 2 * grid || slot_tile[s.out_index] != -1) return 3;
                slot_tile[s.out_index] = s.tile;
                slot_kb[s.out_index] = s.nkb;
            } else {
                if (mode != kClassic || s.out_index >= split_k) return 4;
                split_seen[(size_t)s.tile * split_k + s.out_index]++;
            }
            if (++count > tiles * (split_k ? split_k : 1) + 4) return 5;
        }
    }
    for (uint32_t v : cover) if (v != 1) return 6;
    if (mode == kClassic) {
        if (split_k > 1) for (uint32_t v : split_seen) if (v != 1) return 7;
        return 0;
    }
    const uint32_t waves = plan_full_waves(p), rem = plan_rem_tiles(p);
    for (uint32_t r = 0; r < rem; r++) {
        const uint32_t tile = waves * grid + r;
        uint32_t first, last;
        plan_tile_owners(p, r, &first, &last);
        if (first > last || last >= grid) return 8;
        if (first == last) {
            if (direct[tile] != 1) return 9;
            continue;
        }
        if (direct[tile] != 0) return 10;
        uint32_t sum = 0;
        for (uint32_t c = first; c <= last; c++) {
            if (plan_rem_begin(p, c) == plan_rem_begin(p, c + 1)) continue;   // this CTA got no units
            const uint32_t slot = plan_tile_slot(p, r, c);
            if (slot_tile[slot] != (int64_t)tile) return 11;
            sum += slot_kb[slot];
            slot_tile[slot] = -2;   // consumed
        }
        if (sum != kblocks) return 12;
    }
    for (int64_t t : slot_tile) if (t >= 0) return 13;   // a partial nobody sums
    return 0;
}


// Codes of n quotients, as the fused quantise + pack kernel computes them.
void harness_quantize(int e_bits, int m_bits, const float* q, int n, unsigned char* codes) {
    for (int i = 0; i < n; i++) codes[i] = (unsigned char)fpx::quantize_rtn_code(e_bits, m_bits, q[i]);
}
}
