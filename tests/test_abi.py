"""CPU-side checks of the C ABI: the library loads and exports every symbol the
header declares (no compute without a GPU), and the ctypes request structs match
the C layouts."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from allpaka_b200 import build, gpu

    build.build()
    return gpu.load_library()


def declared_symbols():
    hdr = open(os.path.join(ROOT, "include", "allpaka_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    return sorted(set(re.findall(r"\b(apk_[a-z0-9_]+)\s*\(", hdr)))


def test_header_and_binding_agree_on_the_entry_points(lib):
    from allpaka_b200 import gpu

    syms = declared_symbols()
    assert len(syms) >= 18
    assert sorted(gpu.EXPORTS) == syms
    for s in syms:
        assert hasattr(lib, s), f"libapk_b200.so does not export {s}"


def test_no_device_is_a_decline_not_a_crash(lib):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    rc = lib.apk_init(C.byref(h), 0)
    assert rc == 1  # APK_DECLINE_NO_DEVICE, DeclineReason::NoDevice
    assert b"no accelerator device" in lib.apk_last_error(None)
    from allpaka_b200 import gpu

    with pytest.raises(gpu.GpuError):
        gpu.Gpu(0)


def test_struct_sizes_against_the_compiler(tmp_path):
    """Compile a tiny C program against the header and compare sizeof()."""
    import subprocess

    from allpaka_b200 import gpu

    src = tmp_path / "sz.c"
    src.write_text(
        '#include "allpaka_b200.h"\n#include <stdio.h>\n'
        "int main(void){printf(\"%zu %zu %zu %zu %zu %zu %zu\\n\", sizeof(apk_matvec_req), sizeof(apk_ffn_req),"
        " sizeof(apk_mat), sizeof(apk_token_layer), sizeof(apk_attn_in_req), sizeof(apk_token_req),"
        " sizeof(apk_stats_t));return 0;}\n")
    exe = tmp_path / "sz"
    subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)])
    got = [int(v) for v in subprocess.check_output([str(exe)]).split()]
    want = [C.sizeof(t) for t in (gpu._MatvecReq, gpu._FfnReq, gpu._Mat, gpu._TokenLayer, gpu._AttnInReq,
                                  gpu._TokenReq, gpu._Stats)]
    assert got == want
