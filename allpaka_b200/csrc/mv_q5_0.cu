// matvec_streamk_kernel<TY_Q5_0, *, *>: see mv_pick.h.
#include "mv_pick.h"

namespace apk {
MvKernel mv_pick_q5_0(int m_eff, bool dump) { return dump ? pick_m<TY_Q5_0, true>(m_eff) : pick_m<TY_Q5_0, false>(m_eff); }
}  // namespace apk
