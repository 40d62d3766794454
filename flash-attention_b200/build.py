"""Builds libfa_b200.so (the C-ABI library with the sm_100a kernels) in-tree with nvcc.

Usage: python flash-attention_b200/build.py [--force] [--verbose]

The library links the CUDA runtime statically and resolves the one driver entry point it needs at
run time, so it can be dlopen'ed on a machine without a GPU driver (for symbol checks).
"""
import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "flash_attn_b200")
LIB_PATH = os.path.join(OUT_DIR, "libfa_b200.so")
OBJ_DIR = os.path.join(HERE, "build")

SOURCES = ["fa_api.cu", "fa_fwd_sm100.cu", "fa_bwd_sm100.cu", "fa_aux.cu", "fa_padding.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--use_fast_math",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
    "--expt-relaxed-constexpr",
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _digest(paths):
    h = hashlib.sha256()
    for p in sorted(paths):
        with open(p, "rb") as f:
            h.update(p.encode())
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(os.environ.get("FA_PROFILE", "").encode())
    h.update(os.environ.get("FA_DEFS", "").encode())
    return h.hexdigest()


def build(force=False, verbose=False):
    """Compile every .cu under csrc/ for sm_100a and link libfa_b200.so.  Returns the path."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    sources = [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(HERE, "..", "include", "fa_b200.h"))
    stamp = os.path.join(OBJ_DIR, "stamp.txt")
    digest = _digest(sources + headers)
    if (not force and os.path.exists(LIB_PATH) and os.path.exists(stamp)
            and open(stamp).read().strip() == digest):
        return LIB_PATH

    nvcc = _nvcc()
    extra = ["-DFA_PROFILE"] if os.environ.get("FA_PROFILE") else []
    extra += os.environ.get("FA_DEFS", "").split()  # extra -D switches of kernel variants

    def compile_one(src):
        obj = os.path.join(OBJ_DIR, os.path.basename(src).replace(".cu", ".o"))
        cmd = [nvcc] + NVCC_FLAGS + extra + ["-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        log = os.path.join(OBJ_DIR, os.path.basename(src) + ".log")
        with open(log, "w") as f:
            f.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s" % (src, r.stderr[-4000:]))
        if verbose:
            sys.stderr.write(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as ex:
        objs = list(ex.map(compile_one, sources))
    cmd = [nvcc, "-shared", "-o", LIB_PATH] + objs + ["-cudart", "static", "-Xcompiler", "-fPIC"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n" + r.stderr[-4000:])
    with open(stamp, "w") as f:
        f.write(digest)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
