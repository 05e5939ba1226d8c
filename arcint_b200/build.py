"""Compile the CUDA library in-tree for sm_100a: arcint_b200/lib/libb200q.so.

nvcc cross-compiles without a GPU. Objects are rebuilt only when a source or header is
newer; `python -m arcint_b200.build --force` rebuilds everything, `--verbose` adds
-Xptxas -v (registers, spills, shared memory per kernel).
"""
import argparse
import concurrent.futures
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
OBJDIR = os.path.join(HERE, "build")
LIB = os.path.join(LIBDIR, "libb200q.so")
EMUL = os.path.join(LIBDIR, "libb200q_emul.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr"]


def nvcc():
    p = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(p):
        raise RuntimeError("nvcc not found")
    return p


def _deps():
    return glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h")) + \
        [os.path.join(HERE, "..", "include", "b200q.h")]


def _stale(dst, srcs):
    return not os.path.exists(dst) or any(os.path.getmtime(s) > os.path.getmtime(dst) for s in srcs)


def _compile(src, obj, verbose):
    extra = os.environ.get("B200Q_NVCC_EXTRA", "").split()          # e.g. -DNAME for a one-off experiment build
    cmd = [nvcc()] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    return src, r.returncode, r.stdout + r.stderr


def build(force=False, verbose=False):
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(OBJDIR, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    deps = _deps()
    jobs, objs = [], []
    for s in srcs:
        o = os.path.join(OBJDIR, os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if force or verbose or _stale(o, [s] + deps):
            jobs.append((s, o))
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for src, rc, out in ex.map(lambda j: _compile(j[0], j[1], verbose), jobs):
            if verbose or rc:
                print(out)
            if rc:
                raise RuntimeError("nvcc failed on " + src)
    if jobs or not os.path.exists(LIB):
        cmd = [nvcc(), "-shared", "-o", LIB] + objs + ["-lcudart"] + _extra_link()
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            print(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    build_emul(force)
    return LIB


def _extra_link():
    return ["-ldl"]


def _sanitize():
    """B200Q_SANITIZE=1: the host-only libraries (the lane-code replay, the GGUF reader) are built with
    AddressSanitizer and UndefinedBehaviorSanitizer under names of their own; the process that loads them needs
    the ASan runtime preloaded (tests/test_sanitizers.py does that)."""
    return os.environ.get("B200Q_SANITIZE") == "1"


SAN_FLAGS = ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined", "-fno-omit-frame-pointer", "-g1", "-O0"]


def build_emul(force=False, define=None):
    """Host build of the kernels' per-lane text (device-free tests): g++ on emul.cpp. `define` names a
    red-case switch (e.g. "B200Q_RED_Q40"): the mutant is built beside the real library."""
    src = os.path.join(CSRC, "emul.cpp")
    if not os.path.exists(src):
        return None
    os.makedirs(LIBDIR, exist_ok=True)
    EMUL = os.path.join(LIBDIR, "libb200q_emul%s%s.so" % ("_" + define.lower() if define else "", "_san" if _sanitize() else ""))
    if not force and not _stale(EMUL, [src] + _deps()):
        return EMUL
    cuda_inc = os.path.join(os.path.dirname(os.path.dirname(nvcc())), "include")
    for cxx in ("/usr/bin/g++", os.environ.get("CXX", "g++"), "g++"):
        cxx = cxx if os.path.isabs(cxx) else shutil.which(cxx)
        if not cxx or not os.path.exists(cxx):
            continue
        cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-ffp-contract=off", "-I", cuda_inc, src, "-o", EMUL] + \
            (["-D" + define] if define else []) + (SAN_FLAGS if _sanitize() else [])
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode == 0:
            return EMUL
        err = r.stderr
    raise RuntimeError("emul build failed:\n" + err[-2000:])


def build_gguf(force=False):
    """The GGUF reader of adapters/gguf (plain C++, no CUDA): g++ into lib/libb200q_gguf.so."""
    src = os.path.join(HERE, "..", "adapters", "gguf", "b200q_gguf.cpp")
    hdr = os.path.join(HERE, "..", "adapters", "gguf", "b200q_gguf.h")
    if not os.path.exists(src):
        return None
    os.makedirs(LIBDIR, exist_ok=True)
    out = os.path.join(LIBDIR, "libb200q_gguf%s.so" % ("_san" if _sanitize() else ""))
    if not force and not _stale(out, [src, hdr, os.path.join(HERE, "..", "include", "b200q.h")]):
        return out
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else shutil.which(os.environ.get("CXX", "g++"))
    r = subprocess.run([cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", src, "-o", out] + (SAN_FLAGS if _sanitize() else []),
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("gguf reader build failed:\n" + r.stderr[-2000:])
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
    sys.exit(0)
