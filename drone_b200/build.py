"""In-tree build of the CUDA library (nvcc, sm_100a only).

    python -m drone_b200.build          # build if sources changed
    python -m drone_b200.build --force

The library lands in drone_b200/lib/libdrone_b200.so next to the sources, so
that a copy of the tree carries the binary with it.
"""
import glob
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIBDIR = os.path.join(PKG, "lib")
LIB = os.path.join(LIBDIR, "libdrone_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def nvcc_path():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the drone_b200 library cannot be built")


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force=False, verbose=False):
    """Compile every .cu under csrc/ into one shared library.  Returns its path."""
    deps = sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h")) + \
        [os.path.join(PKG, "..", "include", "drone_b200.h"), os.path.abspath(__file__)]
    if not force and not _stale(LIB, deps):
        return LIB
    os.makedirs(LIBDIR, exist_ok=True)
    objdir = os.path.join(LIBDIR, "obj")
    os.makedirs(objdir, exist_ok=True)
    nvcc = nvcc_path()
    objs = []
    procs = []
    for src in sources():
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if force or _stale(obj, deps):
            cmd = [nvcc, *NVCC_FLAGS, "-c", src, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(out)
        if p.returncode != 0:
            raise RuntimeError("nvcc failed on %s" % src)
    link = [nvcc, "-shared", "-o", LIB, *objs, "-lcudart", "-lnccl"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("link of %s failed" % LIB)
    return LIB


COMPAT = os.path.join(PKG, "compat")
COMPAT_LIBS = {
    "libdrone_pr_compat.so": ["pr_compat.cu"],
    "libdrone_gcn_compat.so": ["graphsum_module.cu"],
}


def build_compat(force=False):
    """The reference-shaped shims (exact symbol / class names of the reference) as separate libraries
    linked against libdrone_b200.so."""
    build_library(force=force)
    nvcc = nvcc_path()
    out = []
    for name, srcs in COMPAT_LIBS.items():
        target = os.path.join(LIBDIR, name)
        deps = [os.path.join(COMPAT, s) for s in srcs] + glob.glob(os.path.join(COMPAT, "*.h")) + \
            glob.glob(os.path.join(COMPAT, "*.cuh")) + [LIB]
        if force or _stale(target, deps):
            cmd = [nvcc, *NVCC_FLAGS, "-shared", "-o", target, *[os.path.join(COMPAT, s) for s in srcs],
                   "-L" + LIBDIR, "-ldrone_b200", "-lnccl", "-Xlinker", "-rpath=$ORIGIN"]
            r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            if r.returncode != 0:
                sys.stderr.write(r.stdout)
                raise RuntimeError("build of %s failed" % name)
        out.append(target)
    return out


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print("\n".join(build_compat(force="--force" in sys.argv)))
