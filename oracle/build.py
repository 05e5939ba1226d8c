"""Build the CPU oracle (TEST INFRASTRUCTURE, never part of the product library).

  python oracle/build.py          -> oracle/liborc.so from b200q_oracle.c, and, when the
                                     reference tree is present, oracle/_ref/libkqref.so
                                     from the reference's own kq_i8_ops.inc.

kq_i8_ops.inc only exists as an added file inside a patch of the reference tree
(contrib/llama.cpp/patches/0000-09-moe-routing-gemm-tiles.patch), so its '+' lines are
extracted into a temporary directory, compiled together with ref_shim.cpp and deleted: only
the built library stays in oracle/_ref/ (git-ignored), no reference source is kept.

The reference tree is looked for in $B200Q_REFERENCE_ROOT, else in a directory named
`reference` beside the repository.
"""
import argparse
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
PATCH = "contrib/llama.cpp/patches/0000-09-moe-routing-gemm-tiles.patch"
TARGET = "ggml/src/ggml-opencl/kernels/kq_i8_ops.inc"
CFLAGS = ["-O3", "-mavx2", "-mfma", "-ffp-contract=off", "-fPIC", "-Wall", "-Wextra", "-std=c11", "-shared"]


def _compilers(names):
    seen = []
    for c in names:
        p = c if os.path.isabs(c) else shutil.which(c)
        if p and os.path.exists(p) and p not in seen:
            seen.append(p)
    return seen


def _newer(dst, srcs):
    return os.path.exists(dst) and all(os.path.getmtime(dst) >= os.path.getmtime(s) for s in srcs)


def build_oracle(force=False):
    """Compile liborc.so; OpenMP when a compiler that has it is found, else one thread."""
    src = os.path.join(HERE, "b200q_oracle.c")
    hdr = os.path.join(HERE, "b200q_oracle.h")
    so = os.path.join(HERE, "liborc.so")
    if not force and _newer(so, [src, hdr]):
        return so
    errs = []
    for cc in _compilers(["/usr/bin/gcc", os.environ.get("CC", "gcc"), "gcc", "cc"]):
        for omp in (["-fopenmp"], []):
            cmd = [cc] + CFLAGS + omp + ["-o", so, src, "-lm"]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode == 0:
                return so
            errs.append(" ".join(cmd) + "\n" + r.stderr[-400:])
    raise RuntimeError("could not build the oracle:\n" + "\n".join(errs))


def _extract(patch_path):
    out, grab, in_hunk = [], False, False
    with open(patch_path, "r", encoding="utf-8", errors="replace") as f:
        for line in f:
            if line.startswith("diff --git "):
                grab = line.rstrip().endswith("b/" + TARGET)
                in_hunk = False
                continue
            if not grab:
                continue
            if line.startswith("@@"):
                in_hunk = True
                continue
            if in_hunk and line.startswith("+"):
                out.append(line[1:])
    if not out:
        raise RuntimeError("kq_i8_ops.inc not found in " + patch_path)
    return "".join(out)


def default_ref_root():
    return os.environ.get("B200Q_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build_ref(ref_root=None):
    """Compile _ref/libkqref.so from the reference tree; None when the tree is absent."""
    patch = os.path.join(ref_root or default_ref_root(), PATCH)
    if not os.path.isfile(patch):
        return None
    dst = os.path.join(HERE, "_ref")
    os.makedirs(dst, exist_ok=True)
    stale = os.path.join(dst, "kq_i8_ops.inc")           # an earlier layout kept the extracted text here
    if os.path.exists(stale):
        os.remove(stale)
    so = os.path.join(dst, "libkqref.so")
    errs = []
    with tempfile.TemporaryDirectory() as tmp:
        with open(os.path.join(tmp, "kq_i8_ops.inc"), "w") as f:
            f.write(_extract(patch))
        for cxx in _compilers(["/usr/bin/g++", os.environ.get("CXX", "g++"), "g++"]):
            cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-I", tmp, os.path.join(HERE, "ref_shim.cpp"), "-o", so]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode == 0:
                return so
            errs.append(r.stderr[-400:])
    raise RuntimeError("could not build _ref:\n" + "\n".join(errs))


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=None)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(build_oracle(force=a.force))
    print(build_ref(a.ref) or "reference tree absent: _ref not rebuilt")
    sys.exit(0)
