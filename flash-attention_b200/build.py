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


BINDING_SRC = os.path.join(CSRC, "fa_torch_binding.cpp")
BINDING_NAME = "_fa_binding"
BINDING_PATH = os.path.join(OUT_DIR, BINDING_NAME + ".so")


def build_binding(force=False):
    """Compile the pybind11 / libtorch binding (csrc/fa_torch_binding.cpp) against libfa_b200.so with the
    host compiler.  Returns the path of flash_attn_b200/_fa_binding.so.  The Python package works
    without it (ctypes binding); with it a dense fwd / bwd call costs a few microseconds of host time."""
    import sysconfig
    import torch
    from torch.utils import cpp_extension as ce
    os.makedirs(OBJ_DIR, exist_ok=True)
    header = os.path.join(HERE, "..", "include", "fa_b200.h")
    stamp = os.path.join(OBJ_DIR, "binding_stamp.txt")
    h = hashlib.sha256()
    for path in (BINDING_SRC, header):
        with open(path, "rb") as f:
            h.update(f.read())
    h.update(torch.__version__.encode())
    digest = h.hexdigest()
    if (not force and os.path.exists(BINDING_PATH) and os.path.exists(stamp)
            and open(stamp).read().strip() == digest):
        return BINDING_PATH
    try:
        inc = ce.include_paths(device_type="cuda")
        libs = ce.library_paths(device_type="cuda")
    except TypeError:  # older signature
        inc = ce.include_paths(cuda=True)
        libs = ce.library_paths(cuda=True)
    cmd = ([os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden",
            "-DTORCH_EXTENSION_NAME=" + BINDING_NAME, "-DTORCH_API_INCLUDE_EXTENSION_H",
            "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)]
           + ["-I" + i for i in inc] + ["-I" + sysconfig.get_paths()["include"], "-I" + os.path.dirname(header)]
           + [BINDING_SRC, "-o", BINDING_PATH]
           + ["-L" + l for l in libs] + ["-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda"]
           + ["-L" + OUT_DIR, "-lfa_b200", "-Wl,-rpath,$ORIGIN"] + ["-Wl,-rpath," + l for l in libs])
    r = subprocess.run(cmd, capture_output=True, text=True)
    with open(os.path.join(OBJ_DIR, "fa_torch_binding.cpp.log"), "w") as f:
        f.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError("host compiler failed for %s:\n%s" % (BINDING_SRC, r.stderr[-4000:]))
    with open(stamp, "w") as f:
        f.write(digest)
    return BINDING_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
    if "--no-binding" not in sys.argv:
        print(build_binding(force="--force-binding" in sys.argv))
