// matvec_streamk_kernel<TY_Q2_K, *, *>: see mv_pick.h.
#include "mv_pick.h"

namespace apk {
MvKernel mv_pick_q2_k(int m_eff, bool dump) { return dump ? pick_m<TY_Q2_K, true>(m_eff) : pick_m<TY_Q2_K, false>(m_eff); }
}  // namespace apk
