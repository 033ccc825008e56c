"""ctypes wrapper of baseline/cusparse_spmm.cu (built into baseline/_build/)."""
import ctypes as C
import os
import shutil
import subprocess

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libcusparse_baseline.so")
_SRC = os.path.join(_HERE, "cusparse_spmm.cu")


def build(force=False):
    if force or not os.path.exists(_SO) or os.path.getmtime(_SRC) > os.path.getmtime(_SO):
        os.makedirs(os.path.dirname(_SO), exist_ok=True)
        nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
        subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17", "-Xcompiler", "-fPIC",
                        "-shared", "-o", _SO, _SRC, "-lcusparse"], check=True)
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            raise RuntimeError("%s missing: run baseline.cusparse_ref.build()" % _SO)
        _lib = C.CDLL(_SO)
        _lib.ref_cusparse_spmm_create.argtypes = [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_int, C.c_void_p,
                                                  C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int,
                                                  C.c_void_p]
        _lib.ref_cusparse_spmm_run.argtypes = [C.c_void_p]
        _lib.ref_cusparse_spmm_destroy.argtypes = [C.c_void_p]
        _lib.ref_cusparse_spmm_buffer_bytes.argtypes = [C.c_void_p]
        _lib.ref_cusparse_spmm_buffer_bytes.restype = C.c_longlong
    return _lib


class CusparseSpmm:
    """Y = A·X with cuSPARSE, descriptors created once (as CUDAGraphSum's constructor does)."""

    def __init__(self, rowptr, col, val, x, y, alg=0):
        self.keep = (rowptr, col, val, x, y)
        self.h = C.c_void_p(0)
        n_rows = rowptr.numel() - 1
        rc = lib().ref_cusparse_spmm_create(C.byref(self.h), n_rows, x.shape[0], col.numel(), rowptr.data_ptr(),
                                            col.data_ptr(), val.data_ptr(), x.shape[1], x.data_ptr(), y.data_ptr(),
                                            alg, torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise RuntimeError("cusparse baseline set-up failed (%d)" % rc)

    def run(self):
        if lib().ref_cusparse_spmm_run(self.h) != 0:
            raise RuntimeError("cusparseSpMM failed")

    def buffer_bytes(self):
        return lib().ref_cusparse_spmm_buffer_bytes(self.h)

    def close(self):
        if self.h.value:
            lib().ref_cusparse_spmm_destroy(self.h)
            self.h = C.c_void_p(0)
