// C-callable shim around the reference's own CPU GEMMs and im2row, for validating the oracle and as
// the "reference" CPU baseline.  TEST INFRASTRUCTURE ONLY.
//
// This file holds no reference code: build_ref.py extracts the four *GEMM_baseline functions from
// the reference's TAB_CPU.cpp (where it lies, outside this repository) into a temporary include file
// named by REF_GEMM_INC, and TAB_CPU.h is included from the reference's own directory.  The whole
// TAB_CPU.cpp cannot be compiled (it references undefined identifiers in its wrappers), its GEMMs can.
#define GCC
#include <cstdint>
#include <cstring>
#include <vector>
#include "TAB_CPU.h"
#include REF_GEMM_INC

extern "C" void ref_gemm(const int64_t* a, const int64_t* b, const int32_t* btn, int32_t* y,
                         int type, long M, int KN, int K, int NUM) {
    std::vector<int> r;
    int64_t* aa = const_cast<int64_t*>(a);
    int64_t* bb = const_cast<int64_t*>(b);
    switch (type) {
        case 0: r = TNNGEMM_baseline(aa, bb, (int)M, KN, K); break;
        case 1: r = TBNGEMM_baseline(aa, bb, (int)M, KN, K); break;
        case 2: r = BTNGEMM_baseline(aa, bb, const_cast<int*>(btn), (int)M, KN, K); break;
        default: r = BNNGEMM_baseline(aa, bb, (int)M, KN, K, NUM); break;
    }
    std::memcpy(y, r.data(), sizeof(int) * r.size());
}

// The reference's explicit im2row (TAB_CPU.h:27-63; written for 3x3, row-generic in KW*C).
extern "C" long ref_im2row_3x3(const int64_t* x, int64_t* y, int N, int C, int H, int W, int KH, int KW, int s1, int s2) {
    std::vector<int64_t> r = Parallel_Img2Row_NHWCB_3x3<int64_t>(const_cast<int64_t*>(x), N, C, H, W, KH, KW, s1, s2);
    std::memcpy(y, r.data(), sizeof(int64_t) * r.size());
    return (long)r.size();
}
