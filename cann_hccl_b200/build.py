"""Build the native library in-tree: every .cc with g++, every .cu with nvcc for sm_100a, one shared object.

    python -m cann_hccl_b200.build [--force] [--verbose] [--sanitize=address|thread]

The shared library lands in cann_hccl_b200/lib/libhccl_b200.so.  Objects are rebuilt when their source or any
header is newer.  nvcc cross-compiles, so this works on machines without a GPU.

--sanitize builds a second library, lib/libhccl_b200_<kind>.so, whose host code is instrumented by the address or the
thread sanitizer (objects under build_<kind>/).  Run the CPU suite on it with

    LD_PRELOAD=$(gcc -print-file-name=libasan.so) ASAN_OPTIONS=detect_leaks=0 \
        HCCL_B200_LIB=cann_hccl_b200/lib/libhccl_b200_address.so python -m pytest tests -m "not gpu"

(libtsan.so and TSAN_OPTIONS for the thread sanitizer).
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
INC = os.path.join(PKG, "include")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "lib")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA, "bin", "nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CXXFLAGS = ["-O2", "-g", "-fPIC", "-std=c++17", "-Wall", "-Wno-unused-function", "-pthread",
            "-I" + INC, "-I" + CSRC, "-I" + os.path.join(CUDA, "include")]
NVCCFLAGS = ARCH + ["-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC", "-I" + INC, "-I" + CSRC,
                    "--expt-relaxed-constexpr", "-Xptxas", "-v" if os.environ.get("HCCL_PTXAS_V") else "-O3"]


def _sources():
    out = []
    for root, _, files in os.walk(CSRC):
        for f in sorted(files):
            if f.endswith((".cc", ".cu")):
                out.append(os.path.join(root, f))
    return sorted(out)


def _newest_header():
    newest = 0.0
    for base in (CSRC, INC):
        for root, _, files in os.walk(base):
            for f in files:
                if f.endswith((".h", ".cuh")):
                    newest = max(newest, os.path.getmtime(os.path.join(root, f)))
    return newest


def _compile(src, obj, verbose):
    os.makedirs(os.path.dirname(obj), exist_ok=True)
    if src.endswith(".cu"):
        cmd = [NVCC] + NVCCFLAGS + ["-c", src, "-o", obj]
    else:
        cmd = ["g++"] + CXXFLAGS + ["-c", src, "-o", obj]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("compile failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))
    if verbose and (r.stdout or r.stderr):
        print(r.stdout + r.stderr, flush=True)
    return obj


def lib_path(sanitize=None):
    return os.path.join(LIB, "libhccl_b200_%s.so" % sanitize if sanitize else "libhccl_b200.so")


def build(force=False, verbose=False, sanitize=None):
    global OBJ, CXXFLAGS, NVCCFLAGS
    san_link = []
    if sanitize:
        if sanitize not in ("address", "thread"):
            raise ValueError("--sanitize takes address or thread")
        flag = "-fsanitize=" + sanitize
        OBJ = os.path.join(PKG, "build_" + sanitize)
        CXXFLAGS = [f for f in CXXFLAGS if f != "-O2"] + ["-O1", "-fno-omit-frame-pointer", flag]
        NVCCFLAGS = NVCCFLAGS + ["-Xcompiler", flag + ",-fno-omit-frame-pointer"]
        san_link = ["-Xcompiler", flag]
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(LIB, exist_ok=True)
    hdr = _newest_header()
    jobs, objs = [], []
    for src in _sources():
        obj = os.path.join(OBJ, os.path.relpath(src, CSRC).replace(os.sep, "__") + ".o")
        objs.append(obj)
        stale = force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr)
        if stale:
            jobs.append((src, obj))
    with ThreadPoolExecutor(max_workers=max(1, os.cpu_count() or 4)) as ex:
        list(ex.map(lambda j: _compile(j[0], j[1], verbose), jobs))
    out = lib_path(sanitize)
    if jobs or not os.path.exists(out):
        cmd = [NVCC] + ARCH + ["-shared", "-o", out] + objs + san_link + ["-lpthread", "-ldl", "-lrt"]
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n%s\n%s" % (r.stdout, r.stderr))
    return out


if __name__ == "__main__":
    _san = [a.split("=", 1)[1] for a in sys.argv if a.startswith("--sanitize=")]
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv or "-v" in sys.argv, sanitize=_san[0] if _san else None))
