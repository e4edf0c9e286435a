// TEST INFRASTRUCTURE ONLY.  C-linkage wrappers around the reference's own CPU
// functions, compiled from the reference sources where they lie (the include
// path is given by oracle/Makefile; no reference source is copied here).
// Wraps: fp6_llm/csrc/utils/weight_prepacking.h:199-211 and
//        fp6_llm/csrc/utils/weight_dequant.h:51-61.
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
    if (!((e_bits == 3 || e_bits == 2) && m_bits == 2)) return -1;
    size_t bytes = rows * cols * (1 + e_bits + m_bits) / 8;
    std::vector<unsigned char> padded(bytes + 4, 0);
    std::memcpy(padded.data(), in, bytes);
    weight_matrix_prepacking_fp_eXmY(e_bits, m_bits, out, reinterpret_cast<int*>(padded.data()), rows, cols);
    return 0;
}

int ref_dequant(int e_bits, int m_bits, unsigned short* out, const unsigned char* in, size_t rows, size_t cols,
                const unsigned short* scale) {
    if (!((e_bits == 3 || e_bits == 2) && m_bits == 2)) return -1;
    dequant_matrix_fp_eXmY_to_fp16(e_bits, m_bits, reinterpret_cast<half*>(out), const_cast<unsigned char*>(in), rows,
                                   cols, reinterpret_cast<half*>(const_cast<unsigned short*>(scale)));
    return 0;
}

}  // extern "C"
