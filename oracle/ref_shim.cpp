// TEST INFRASTRUCTURE ONLY.  C-linkage wrappers around the reference's own CPU
// functions, compiled from the reference sources where they lie (the include
// path is given by oracle/Makefile; no reference source is copied here).
// Wraps: fp6_llm/csrc/utils/weight_prepacking.h:199-211 and fp6_llm/csrc/utils/weight_dequant.h:51-61 for the two
// formats those entry points dispatch, and the templates behind them (weight_prepacking.h:118-196,
// weight_dequant.h:10-48) instantiated for e2m1, e3m1 and e2m3.
#include <cstddef>
#include <cstring>
#include <vector>
#include <cuda_fp16.h>
#include "utils/weight_prepacking.h"
#include "utils/weight_dequant.h"

extern "C" {

// The reference reads one byte past the end of its input (common.h:10), so the
// input is copied into a buffer with one byte of padding first.
int ref_prepack(int e_bits, int m_bits, int* out, const int* in, size_t rows, size_t cols) {
    size_t bytes = rows * cols * (1 + e_bits + m_bits) / 8;
    std::vector<unsigned char> padded(bytes + 4, 0);
    std::memcpy(padded.data(), in, bytes);
    int* src = reinterpret_cast<int*>(padded.data());
    if ((e_bits == 3 || e_bits == 2) && m_bits == 2) weight_matrix_prepacking_fp_eXmY(e_bits, m_bits, out, src, rows, cols);
    else if (e_bits == 2 && m_bits == 1) weight_matrix_prepacking_x_bit<2, 1>(out, src, rows, cols);
    else if (e_bits == 3 && m_bits == 1) weight_matrix_prepacking_x_bit<3, 1>(out, src, rows, cols);
    else if (e_bits == 2 && m_bits == 3) weight_matrix_prepacking_x_bit<2, 3>(out, src, rows, cols);
    else return -1;
    return 0;
}

int ref_dequant(int e_bits, int m_bits, unsigned short* out, const unsigned char* in, size_t rows, size_t cols,
                const unsigned short* scale) {
    half* o = reinterpret_cast<half*>(out);
    half* sc = reinterpret_cast<half*>(const_cast<unsigned short*>(scale));
    // the reference reads one byte past the end of its input here too (common.h:10)
    size_t bytes = rows * cols * (1 + e_bits + m_bits) / 8;
    std::vector<unsigned char> padded(bytes + 4, 0);
    std::memcpy(padded.data(), in, bytes);
    unsigned char* src = padded.data();
    if ((e_bits == 3 || e_bits == 2) && m_bits == 2) dequant_matrix_fp_eXmY_to_fp16(e_bits, m_bits, o, src, rows, cols, sc);
    else if (e_bits == 2 && m_bits == 1) DeQuantMatrix_FPx_To_FP16<2, 1>(o, src, rows, cols, sc);
    else if (e_bits == 3 && m_bits == 1) DeQuantMatrix_FPx_To_FP16<3, 1>(o, src, rows, cols, sc);
    else if (e_bits == 2 && m_bits == 3) DeQuantMatrix_FPx_To_FP16<2, 3>(o, src, rows, cols, sc);
    else return -1;
    return 0;
}

}  // extern "C"
