"""The split of RMSNorm + Q8 quantisation that the residual epilogue uses (CPU check against the oracle).

rmsnorm_into gives y = f32(f64(x) * scale) * gamma and Q8Acts::from_f32 quantises y per 32-element block.
The GPU path quantises u = x * gamma before the row-wide scale is known and multiplies the block scales by
f32(scale) afterwards.  The codes round(v / d) are invariant under a common positive factor up to f32 rounding;
this test pins how close "up to rounding" is on the benchmark's value distribution."""
import numpy as np

from allpaka_b200 import synth


def test_codes_do_not_depend_on_the_row_scale(orc):
    n = 5120
    rng = np.random.default_rng(77)
    x = (rng.standard_normal(n) * 3.0).astype(np.float32)
    gamma = synth.gamma(n, 78)
    eps = 1e-6
    y = orc.rmsnorm_into(x, gamma, eps)
    d_ref, _, q_ref = orc.q8acts(y)
    u = (x * gamma).astype(np.float32)
    d_u, _, q_u = orc.q8acts(u)
    scale = np.float32(1.0 / np.sqrt(orc.sum_sq_f64(x) / n + eps))
    d_split = (d_u * scale).astype(np.float32)
    # block scales agree to a few ulp, codes are identical except where v/d sits on a .5 boundary
    assert np.max(np.abs(d_split - d_ref) / d_ref) < 4e-7
    flips = np.count_nonzero(q_u != q_ref)
    assert flips <= 2, flips
    assert np.max(np.abs(q_u.astype(np.int32) - q_ref.astype(np.int32))) <= 1
    # and the dequantised rows agree to well below one code step
    yq_ref = q_ref.astype(np.float32) * np.repeat(d_ref, 32)
    yq_split = q_u.astype(np.float32) * np.repeat(d_split, 32)
    assert np.linalg.norm(yq_split - yq_ref) / np.linalg.norm(yq_ref) < 1e-3
