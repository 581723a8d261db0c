"""Builds librapidh3_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m rapid_h3_b200._build [--force] [--verbose]

Objects go to rapid_h3_b200/build/, the library next to this file so that it travels with the
source tree. Sources are recompiled only when they (or a header) are newer than their object.
"""
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
OBJDIR = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "librapidh3_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
    "-I", INCLUDE, "-I", CSRC,
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: librapidh3_b200.so cannot be built")


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers_mtime():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    return max(os.path.getmtime(h) for h in hs)


def _compile(nvcc, src, obj, verbose):
    cmd = [nvcc, *NVCC_FLAGS, *os.environ.get("RH3_EXTRA_NVCC", "").split(), "-Xptxas", "-v" if verbose else "-warn-spills", "-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    return r.stderr


def build(force=False, verbose=False):
    """Compile every csrc/*.cu and link the shared library; returns its path."""
    nvcc = _nvcc()
    os.makedirs(OBJDIR, exist_ok=True)
    hm = _headers_mtime()
    jobs, objs = [], []
    for f in sources():
        src, obj = os.path.join(CSRC, f), os.path.join(OBJDIR, f[:-3] + ".o")
        objs.append(obj)
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hm):
            jobs.append((src, obj))
    with cf.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for (src, _), log in zip(jobs, ex.map(lambda j: _compile(nvcc, j[0], j[1], verbose), jobs)):
            if verbose and log:
                print(f"---- {os.path.basename(src)}\n{log}", file=sys.stderr)
    if jobs or not os.path.exists(LIB):
        cmd = [nvcc, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
