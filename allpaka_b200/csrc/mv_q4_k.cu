// matvec_streamk_kernel<TY_Q4_K, *, *>: see mv_pick.h.
#include "mv_pick.h"

namespace apk {
MvKernel mv_pick_q4_k(int m_eff, bool dump) { return dump ? pick_m<TY_Q4_K, true>(m_eff) : pick_m<TY_Q4_K, false>(m_eff); }
}  // namespace apk
