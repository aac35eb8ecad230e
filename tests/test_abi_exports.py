"""The C-ABI library loads without a GPU and exports every symbol the headers declare
(no compute calls here)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    names = []
    for fn in os.listdir(os.path.join(ROOT, "include")):
        if fn.endswith(".h"):
            text = open(os.path.join(ROOT, "include", fn)).read()
            names += re.findall(r"GSB_API\s+[\w\s\*]+?\b(gsb_\w+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    from glmserve_b200 import build
    from glmserve_b200._lib import LIB_PATH
    if not os.path.exists(LIB_PATH):
        build.build()
    lib = ctypes.CDLL(LIB_PATH)
    names = _declared()
    assert len(names) >= 25
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    lib.gsb_status_string.restype = ctypes.c_char_p
    assert lib.gsb_status_string(0) == b"ok"
    assert lib.gsb_status_string(2) == b"unsupported shape or format"


def test_pure_host_entry_points_validate_arguments():
    from glmserve_b200._lib import lib
    L = lib()
    assert L.gsb_prepack_bytes(1, 64, 1024) == 2 * 2 * 8448
    assert L.gsb_prepack_bytes(1, 64, 1000) == 0
    assert L.gsb_moe_layer_create(None, None) == 1
    assert L.gsb_moe_route_static_max_floats() == 65536
    # heap bytes the all-reduce reserves: staging of four areas plus two parities of world slots of the
    # flag-in-data words (8 bytes per float, at most 65536 floats) - it grows with the world size
    L.gsb_comm_allreduce_reserve_bytes.restype = ctypes.c_size_t
    rb = lambda w, n: L.gsb_comm_allreduce_reserve_bytes(w, ctypes.c_int64(n))
    assert rb(2, 6144) == 4 * (6144 + 64) * 4 + 2 * 2 * (6144 // 2) * 16
    assert rb(8, 256 * 6144) == 4 * (256 * 6144 + 64) * 4 + 2 * 8 * 32768 * 16
    assert rb(8, 1 << 20) > rb(4, 1 << 20) > rb(2, 1 << 20)
    assert rb(0, 16) == 0 and rb(2, -1) == 0


def test_shim_header_names_match_reference_surface():
    text = open(os.path.join(ROOT, "include", "glmserve_cuda_shim.cuh")).read()
    for name in ("moe_router", "moe_dispatch", "moe_expert_ffn", "moe_expert_ffn_w4a16", "gemm_w4a16",
                 "gemm_q", "gemm_q_i8", "quantize_act_q8", "qtype_has_i8", "moe_expert_ffn_q",
                 "moe_expert_ffn_q_i8"):
        assert re.search(r"inline\s+\w+\s+%s\s*\(" % name, text), name


def test_shim_compiles_and_links_against_the_library(tmp_path):
    """A translation unit written the way src/model_gpu.cpp calls the operators (namespace
    glmserve::cuda, default stream argument) compiles against the shim and links with the
    library - no GPU needed, nothing is run."""
    import shutil
    import subprocess
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not found")
    src = tmp_path / "caller.cu"
    src.write_text(
        '#include <cuda_runtime.h>\n'
        '#include "glmserve_b200.h"\n'
        '#include "glmserve_cuda_shim.cuh"\n'
        'int main() {\n'
        '    float* f = nullptr; int* i = nullptr; unsigned char* q = nullptr;\n'
        '    glmserve::cuda::moe_router(f, f, 0, 8, 2, true, 2.5f, i, f);\n'
        '    glmserve::cuda::moe_dispatch(i, 0, 2, 8, i, i, i);\n'
        '    glmserve::cuda::moe_expert_ffn_w4a16(f, i, f, q, f, q, f, q, f, 0, 2, 64, 64, 8, 32, f);\n'
        '    glmserve::cuda::gemm_w4a16(f, q, f, nullptr, f, 0, 64, 64, 32);\n'
        '    return glmserve::cuda::b200_last_status();\n'
        '}\n')
    exe = tmp_path / "caller"
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-I", os.path.join(ROOT, "include"),
           str(src), "-o", str(exe), "-L", os.path.join(ROOT, "glmserve_b200"), "-lglmserve_b200"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
