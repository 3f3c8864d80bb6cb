// The matvec kernel's instantiations, one translation unit per weight format so that they compile
// side by side (each holds 12 row counts x {plain, block-dot dump}).
#pragma once
#include "kernels.cuh"

namespace apk {

typedef void (*MvKernel)(const MvParams);

template <int TY, bool DUMP>
MvKernel pick_m(int m) {
    switch (m) {
        case 1: return matvec_streamk_kernel<TY, 1, DUMP>;
        case 2: return matvec_streamk_kernel<TY, 2, DUMP>;
        case 3: return matvec_streamk_kernel<TY, 3, DUMP>;
        case 4: return matvec_streamk_kernel<TY, 4, DUMP>;
        case 5: return matvec_streamk_kernel<TY, 5, DUMP>;
        case 6: return matvec_streamk_kernel<TY, 6, DUMP>;
        case 7: return matvec_streamk_kernel<TY, 7, DUMP>;
        case 8: return matvec_streamk_kernel<TY, 8, DUMP>;
        case 10: return matvec_streamk_kernel<TY, 10, DUMP>;
        case 12: return matvec_streamk_kernel<TY, 12, DUMP>;
        case 14: return matvec_streamk_kernel<TY, 14, DUMP>;
        case 16: return matvec_streamk_kernel<TY, 16, DUMP>;
        default: return nullptr;
    }
}

// defined in mv_q8_0.cu, mv_q5_0.cu, mv_q2_k.cu, mv_q4_k.cu, mv_q5_k.cu, mv_q6_k.cu
MvKernel mv_pick_q5_0(int m_eff, bool dump);
MvKernel mv_pick_q2_k(int m_eff, bool dump);
MvKernel mv_pick_q8_0(int m_eff, bool dump);
MvKernel mv_pick_q4_k(int m_eff, bool dump);
MvKernel mv_pick_q5_k(int m_eff, bool dump);
MvKernel mv_pick_q6_k(int m_eff, bool dump);

}  // namespace apk
