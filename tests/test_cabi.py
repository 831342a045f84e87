"""The C-ABI shared library: loads, exports every declared symbol, rejects bad arguments
on the host (no kernel is launched here, so this runs without a GPU)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from svoo_b200 import build
    build.build()
    from svoo_b200 import _lib
    return _lib


def declared_functions():
    text = open(os.path.join(ROOT, "include", "svoo_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(svoo_b200_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(lib):
    names = declared_functions()
    assert len(names) >= 12
    raw = ctypes.CDLL(lib._build.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), f"{n} declared in include/svoo_b200.h but not exported"
        assert n in lib.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(lib.SIGNATURES) == names


def test_version_and_error_strings(lib):
    assert lib.LIB.svoo_b200_version() == lib.VERSION
    assert lib.LIB.svoo_b200_error_string(0) == b"ok"
    assert b"128" in lib.LIB.svoo_b200_error_string(-3)
    with pytest.raises(ValueError):
        lib.check(-1, "x")
    with pytest.raises(lib.SvooB200Error):
        lib.check(700, "x")


def test_workspace_bytes(lib):
    out = ctypes.c_int64(0)
    assert lib.LIB.svoo_b200_workspace_bytes(40, 75600, 100, 500, ctypes.byref(out)) == 0
    big = out.value
    assert 50e6 < big < 2e9
    assert lib.LIB.svoo_b200_workspace_bytes(40, 75600, 500, 100, ctypes.byref(out)) == 0
    assert out.value == big                                   # symmetric in (QC, KC)
    assert lib.LIB.svoo_b200_workspace_bytes(40, 75600, 100, 2000, ctypes.byref(out)) == -6
    # the shipped HunyuanVideo setting: 256 / 1024 clusters plus the two text blocks
    assert lib.LIB.svoo_b200_workspace_bytes(24, 118800 + 256, 258, 1026, ctypes.byref(out)) == 0
    assert lib.LIB.svoo_b200_workspace_bytes(0, 75600, 100, 500, ctypes.byref(out)) == -2
    assert lib.LIB.svoo_b200_workspace_bytes(1, 10, 1, 1, None) == -1


def test_host_side_argument_checks(lib):
    L = lib.LIB
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.addressof(buf)
    p = (p + 255) // 256 * 256
    assert L.svoo_b200_permute(None, p, 1, 4, 128, 4, 4, p, None) == -1
    assert L.svoo_b200_permute(p, p, 1, 4, 64, 4, 4, p, None) == -3
    assert L.svoo_b200_permute(p + 2, p, 1, 4, 128, 4, 4, p, None) == -5
    assert L.svoo_b200_permute(p, p, 1, 4, 128, 2, 4, p, None) == -2
    assert L.svoo_b200_sort_labels(p, 1, 4, 4, p, p, p, 16, None) == -4
    assert L.svoo_b200_sparse_attn(p, p, p, p, p, p, 1, 4, 128, 2, 2000, 0.1, p, None, None, p, 1 << 30, None) == -6
    # the attention side takes the clusters plus two text blocks, the clustering does not
    assert L.svoo_b200_sparse_attn(p, p, p, p, p, p, 1, 4, 128, 258, 1026, 0.1, p, None, None, p, 16, None) == -4
    assert L.svoo_b200_sparse_attn(p, p, p, p, p, p, 1, 4, 128, 258, 1027, 0.1, p, None, None, p, 1 << 30, None) == -6
    assert L.svoo_b200_cocluster(p, p, p, p, 1, 4, 128, 2, 1025, 1, p, p, p, p, p, p, p, p, p, p, p, 1 << 30, None) == -6
    assert L.svoo_b200_cocluster(p, p, p, None, 1, 4, 128, 2, 2, 1, p, p, p, p, p, p, p, p, p, p, p, 1 << 30, None) == -1
    # BH * N must fit a 32-bit row index
    assert L.svoo_b200_permute(p, p, 200, 1 << 24, 128, 1 << 24, 1 << 24, p, None) == -2
    assert L.svoo_b200_sort_labels_static(p, 200, 1 << 24, 4, p, p, None) == -2
    assert L.svoo_b200_euclid_assign(p, p, 1, 4, 128, 2000, p, p, 1 << 30, None) == -6
    assert L.svoo_b200_qk_prep_heads(p, None, 1e-6, None, None, 64, 4, 128, 0, None, 64, 0, None) == -1
    assert L.svoo_b200_qk_prep_heads(p, None, 1e-6, None, None, 64, 4, 128, 65, p, 64, 0, None) == -2
    assert L.svoo_b200_qk_prep_heads(p, None, 1e-6, None, None, 64, 4, 128, 0, p, 64, 1, None) == -2
    # error-aware routing entries: argument checks run before any device work
    assert L.svoo_b200_ear_workspace_bytes(2, 4096, 32, 128, None, None) == -1
    assert L.svoo_b200_ear_value_centroids(None, p, 1, 64, 128, 4, 8, p, p, 1 << 30, None) == -1
    assert L.svoo_b200_ear_value_centroids(p, p, 1, 64, 64, 4, 8, p, p, 1 << 30, None) == -3
    assert L.svoo_b200_ear_block_scores(p, p, p, p, p, 1, 64, 128, 4, 2000, 1.0, p, p, p, 1 << 30, None) == -6
    assert L.svoo_b200_ear_block_scores(p, p, p, p, p, 1, 64, 128, 4, 8, 1.0, p, p, p, 16, None) == -4
    assert L.svoo_b200_ear_select_blocks(p, p, p, p, 1, 4, 8, 0.9, None, None, p, None) == -1
    assert L.svoo_b200_sparse_attn_ear(p, p, p, p, p, p, 1, 64, 128, 4, 8, 0.1, None, None, None, p, 1 << 30, None) == -1
    assert L.svoo_b200_sparse_attn_ear(p, p, p, p, p, p, 1, 64, 128, 4, 8, 0.1, p, None, None, p, 16, None) == -4
    assert L.svoo_b200_append_text_blocks(p, p, p, p, p, 1, 4, 2, 2, 4, 5, p, p, p, p, p, None) == -2
    out = ctypes.c_int64(0)
    assert L.svoo_b200_layer_scratch_bytes(2, 1000, 8, 16, 64, ctypes.byref(out)) == 0 and out.value > 3 * 2 * 1000 * 256
    assert L.svoo_b200_layer_scratch_bytes(2, 1000, 8, 16, 1000, ctypes.byref(out)) == -2
    assert L.svoo_b200_layer(p, p, p, p, p, 2, 1000, 128, 8, 16, 1, 0.9, p, p, 0.1, 64, 65, p, p, 1 << 40, p, 1 << 40, None) == -2
    assert L.svoo_b200_cocluster(p, p, p, p, 1, 4, 128, 2, 2, 0, p, p, p, p, p, p, p, p, p, p, p, 1 << 30, None) == -2


def test_tensor_core_kernels_do_not_spill():
    """tcgen05.ld fills registers asynchronously; a spill store scheduled between the load and
    its tcgen05.wait::ld would save garbage, so the code that issues tcgen05.ld must compile
    spill-free.  The attention kernel moves registers between warpgroups (setmaxnreg): its
    softmax warpgroups are checked at their real budget by compiling the service warpgroup with
    the launch allotment (a build that is never run); the product build may only spill a few
    words in the TMA producer / MMA issuer branch, which never issues tcgen05.ld."""
    import subprocess
    from svoo_b200 import build

    def spills(src, *extra):
        res = subprocess.run([build._nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-Xptxas", "-v",
                              *extra, "-c", os.path.join(build.CSRC, src), "-o", os.devnull], capture_output=True, text=True)
        assert res.returncode == 0, res.stderr
        blocks = re.findall(r"Function properties for (\S+)\n\s*(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads",
                            res.stderr)
        tc = [(n, int(st), int(ld)) for n, _, st, ld in blocks if "_tc_kernel" in n]
        assert tc, res.stderr
        return tc

    for name, st, ld in spills("assign_tc.cu") + spills("attn_tc.cu", "-DSVOO_REGS_SERVICE=168"):
        assert st == 0 and ld == 0, f"{name} spills {st}/{ld} bytes"
    for name, st, ld in spills("attn_tc.cu"):
        assert st <= 32, f"{name}: service branch spills {st} bytes"


def test_header_is_plain_c_and_links(tmp_path):
    """include/svoo_b200.h compiles as C99 (no C++ or torch types in the ABI) and a C program
    links against the shared library."""
    import shutil
    import subprocess
    from svoo_b200 import build
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    src = tmp_path / "t.c"
    src.write_text('#include "svoo_b200.h"\n#include <stdio.h>\n'
                   'int main(void) { long long b = 0; int rc = svoo_b200_workspace_bytes(2, 4096, 32, 128, (int64_t*)&b);\n'
                   '  printf("%d %d %lld\\n", svoo_b200_version(), rc, b); return rc; }\n')
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = tmp_path / "t"
    lib_dir = os.path.dirname(build.LIB_PATH)
    res = subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-I", os.path.join(root, "include"),
                          str(src), "-o", str(exe), "-L", lib_dir, "-l:libsvoo_b200.so", f"-Wl,-rpath,{lib_dir}"],
                         capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True)
    assert run.returncode == 0, run.stderr
    version, rc, nbytes = run.stdout.split()
    assert int(version) == 104 and int(rc) == 0 and int(nbytes) > 0
