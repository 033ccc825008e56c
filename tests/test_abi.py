"""The shared library loads without a GPU and exports every symbol include/drone_b200.h declares."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = []
    for fn in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if not fn.endswith(".h"):
            continue
        text = open(os.path.join(ROOT, "include", fn)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"\b(drone_[a-z0-9_]+|build_graph|addMasterRoute|addMirrorRoute|getLocalVertexSize|"
                            r"getGlobalVertexSize|loadOutDegree|PR_PEVal|PR_IncEVal)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    import drone_b200
    lib = drone_b200.lib()
    names = declared_symbols()
    assert "drone_spmm" in names and "drone_plan_create" in names
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, "declared in include/ but not exported: %s" % missing


def test_version_and_error_string():
    import drone_b200
    lib = drone_b200.lib()
    assert lib.drone_version() >= 1000
    # an invalid call fails with a code and a message, without touching a device
    rc = lib.drone_plan_create(None, 1, 1, None, None, None, None, None, 3, None)
    assert rc == -1
    assert b"out is NULL" in lib.drone_last_error()
    h = C.c_void_p(0)
    rc = lib.drone_plan_create(C.byref(h), -5, 0, None, None, None, None, None, 3, None)
    assert rc == -1 and b"negative" in lib.drone_last_error()
    rc = lib.drone_spmm(None, 0, 32, None, 32, None, 32, None)
    assert rc == -1 and b"plan is NULL" in lib.drone_last_error()


def test_missing_library_fails_loudly(monkeypatch):
    from drone_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libdrone_b200.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.lib()


def test_reference_shaped_shims_export_the_reference_symbols():
    import drone_b200
    drone_b200.lib()
    libdir = os.path.join(ROOT, "drone_b200", "lib")
    pr = C.CDLL(os.path.join(libdir, "libdrone_pr_compat.so"))
    header = open(os.path.join(ROOT, "drone_b200", "compat", "drone_pr_compat.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    names = re.findall(r"\b(build_graph|getLocalVertexSize|getGlobalVertexSize|addMasterRoute|addMirrorRoute|"
                       r"loadOutDegree|PR_PEVal|PR_IncEVal)\s*\(", header)
    assert len(set(names)) == 8
    for n in set(names):
        assert hasattr(pr, n), n
    gcn = C.CDLL(os.path.join(libdir, "libdrone_gcn_compat.so"))
    for n in ("create", "forward", "backward", "destroy"):
        assert hasattr(gcn, "drone_compat_graphsum_" + n)


def test_header_is_plain_c(tmp_path):
    """cgo (and any C host) compiles the header as C, not C++."""
    import shutil
    import subprocess
    gcc = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    src = tmp_path / "use_header.c"
    src.write_text('#include "drone_b200.h"\n'
                   "int main(void) { drone_pr_response r; drone_plan_stats s; (void)r; (void)s;\n"
                   "                 return DRONE_OK + DRONE_OP_A + DRONE_PLAN_BOTH * 0 + DRONE_MP_SSSP * 0; }\n")
    r = subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-fsyntax-only",
                        "-I", os.path.join(ROOT, "include"), str(src)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_compat_library_exports_the_cgo_interface():
    """The symbols DRONE/src/tools/cuda_convert.go binds, by the reference's names."""
    import drone_b200
    drone_b200.lib()
    path = os.path.join(ROOT, "drone_b200", "lib", "libdrone_pr_compat.so")
    if not os.path.exists(path):
        pytest.skip("compat library not built")
    lib = C.CDLL(path)
    for name in ("build_graph", "addMasterRoute", "addMirrorRoute", "getLocalVertexSize", "getGlobalVertexSize",
                 "loadOutDegree", "PR_PEVal", "PR_IncEVal", "CC_PEVal", "CC_IncEVal", "SSSP_PEVal", "SSSP_IncEVal"):
        assert hasattr(lib, name), name
