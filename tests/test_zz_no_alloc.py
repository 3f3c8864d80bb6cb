"""apk_matvec_noalloc: the matvec for callers that may not allocate device memory.

Some hosts of this library budget all of their VRAM at start-up, or call from a
latency-bounded decode loop that cannot afford an allocation's device-wide stall,
so cudaMalloc is not an option for them.  They pass their own input and output buffers and the kernel's
private scratch comes from a fixed array inside the library.  This test drives
that entry point through the C ABI, twice in a row (the array keeps the last
call's contents), and requires the same results as the ordinary apk_matvec.
It lives in the last-collected file so a run that stops at the first failure
has already run everything else.
"""
import numpy as np
import pytest

from allpaka_b200 import synth
from tests.util import Q4_K, Q8_0, Region, rel_l2

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    from allpaka_b200 import gpu as G

    g = G.Gpu(0)
    yield g
    g.close()


CASES = [
    (Q8_0, 3072, 1024, 1, 2),    # decode row: activations quantised inside the kernel
    (Q8_0, 700, 5120, 3, 0),     # batch: the separate quantiser writes into the built-in scratch
    (Q8_0, 256, 25600, 2, 1),    # f32-activation mode, long rows (records streamed)
    (Q4_K, 513, 2048, 1, 2),
    (Q4_K, 130, 1024, 4, 1),
    (Q8_0, 16384, 5120, 1, 2),
]


@pytest.mark.parametrize("ty,n_out,n_in,m,mode", CASES)
def test_noalloc_matches_the_allocating_entry_point_twice(gpu, orc, ty, n_out, n_in, m, mode):
    import torch

    w = synth.matrix(ty, n_out, n_in, 77)
    r = Region([w])
    assert gpu.attach(r.buf)
    x = synth.normal_f32((m, n_in), 78)
    # not resident yet: the entry point must refuse rather than upload (uploading allocates)
    xd = torch.from_numpy(x).cuda()
    yd = torch.full((m, n_out), float("nan"), device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    torch.cuda.synchronize()
    assert gpu.matvec_noalloc(ty, r.views[0], n_in, n_out, xd.data_ptr(), m, yd.data_ptr(), stream, mode) is False
    assert gpu.last_decline[0] == 6
    want = gpu.matvec(ty, r.views[0], n_in, n_out, x, m, mode)   # uploads the matrix; the reference result
    oracle = orc.matmul(ty, w, n_out, n_in, x, m, mode)
    assert rel_l2(want, oracle) <= 2e-3
    for rep in range(2):
        x2 = synth.normal_f32((m, n_in), 79 + rep)
        xd.copy_(torch.from_numpy(x2))
        yd.fill_(float("nan"))
        torch.cuda.synchronize()
        assert gpu.matvec_noalloc(ty, r.views[0], n_in, n_out, xd.data_ptr(), m, yd.data_ptr(), stream, mode)
        got = yd.cpu().numpy()
        ref = gpu.matvec(ty, r.views[0], n_in, n_out, x2, m, mode)
        assert np.array_equal(got, ref), rel_l2(got, ref)   # same kernel, same summation order
        assert rel_l2(got, orc.matmul(ty, w, n_out, n_in, x2, m, mode)) <= 2e-3
    gpu.detach(r.buf)


def test_noalloc_unwaited_call_then_another_and_no_allocation(gpu, orc):
    """wait=False leaves the call unobserved: the next call on the device clears the tagged partial
    sums first and is right all the same.  Neither call changes the amount of free device memory."""
    import torch

    n_out, n_in = 700, 5120
    w = synth.q8_0_matrix(n_out, n_in, 91)
    r = Region([w])
    assert gpu.attach(r.buf)
    assert gpu.register_matrix(r.views[0], Q8_0, n_out, n_in)
    x = synth.normal_f32((1, n_in), 92)
    xd = torch.from_numpy(x).cuda()
    yd = torch.zeros((1, n_out), device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert gpu.matvec_noalloc(Q8_0, r.views[0], n_in, n_out, xd.data_ptr(), 1, yd.data_ptr(), stream)  # symbol resolved
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    assert gpu.matvec_noalloc(Q8_0, r.views[0], n_in, n_out, xd.data_ptr(), 1, yd.data_ptr(), stream, wait=False)
    assert gpu.matvec_noalloc(Q8_0, r.views[0], n_in, n_out, xd.data_ptr(), 1, yd.data_ptr(), stream, wait=True)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0
    assert rel_l2(yd.cpu().numpy(), orc.matmul(Q8_0, w, n_out, n_in, x, 1)) <= 1e-5
    # a second context on the same device shares the one array and its state
    from allpaka_b200 import gpu as G

    g2 = G.Gpu(0)
    assert g2.attach(r.buf) and g2.register_matrix(r.views[0], Q8_0, n_out, n_in)
    yd.zero_()
    assert gpu.matvec_noalloc(Q8_0, r.views[0], n_in, n_out, xd.data_ptr(), 1, yd.data_ptr(), stream, wait=False)
    torch.cuda.synchronize()
    assert g2.matvec_noalloc(Q8_0, r.views[0], n_in, n_out, xd.data_ptr(), 1, yd.data_ptr(), stream)
    assert rel_l2(yd.cpu().numpy(), orc.matmul(Q8_0, w, n_out, n_in, x, 1)) <= 1e-5
    g2.detach(r.buf)
    g2.close()
    gpu.detach(r.buf)


def test_noalloc_rejects_sizes_beyond_its_scratch(gpu):
    w = synth.q8_0_matrix(4, 64, 1)
    r = Region([w])
    assert gpu.attach(r.buf)
    assert gpu.matvec_noalloc(Q8_0, r.views[0], 65536, 4, 1, 1, 1) is False
    assert gpu.last_decline[0] == 3 and "exceeds the built-in scratch" in gpu.last_decline[1]
    assert gpu.matvec_noalloc(Q8_0, r.views[0], 64, 600000, 1, 1, 1) is False
    assert gpu.last_decline[0] == 3
    gpu.detach(r.buf)
