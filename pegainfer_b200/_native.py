"""Build and load ``libpegainfer_b200.so`` (hand-written sm_100a CUDA + C++ runtime).

The library is plain CUDA/C++ with a C API (``csrc/api.h``), compiled in-tree with
``nvcc -gencode arch=compute_100a,code=sm_100a`` and loaded through ``ctypes``; it does
not link against PyTorch.  A stamp file holds the hash of the sources so a stale
binary is rebuilt and an up-to-date one is loaded as is.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "csrc")
LIB_DIR = os.path.join(ROOT, "pegainfer_b200", "lib")
LIB_PATH = os.path.join(LIB_DIR, "libpegainfer_b200.so")
STAMP = os.path.join(LIB_DIR, "build.stamp")
NVCC = os.environ.get("PEGAINFER_NVCC", "/usr/local/cuda/bin/nvcc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-O3", "--expt-relaxed-constexpr"]

_lib = None


def _sources():
    out = []
    for dp, _, fns in os.walk(CSRC):
        for fn in sorted(fns):
            if fn.endswith((".cu", ".cpp")):
                out.append(os.path.join(dp, fn))
    return sorted(out)


def _headers():
    out = []
    for dp, _, fns in os.walk(CSRC):
        for fn in sorted(fns):
            if fn.endswith((".cuh", ".h", ".hpp")):
                out.append(os.path.join(dp, fn))
    return sorted(out)


def source_hash() -> str:
    h = hashlib.sha256()
    for p in _sources() + _headers():
        h.update(os.path.relpath(p, CSRC).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(ARCH_FLAGS + COMMON_FLAGS).encode())
    return h.hexdigest()


def is_current() -> bool:
    if not (os.path.exists(LIB_PATH) and os.path.exists(STAMP)):
        return False
    with open(STAMP) as f:
        return f.read().strip() == source_hash()


def build(force: bool = False, verbose: bool = False, jobs: int = 0) -> str:
    """Compile every translation unit for sm_100a and link the shared library."""
    if not force and is_current():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    obj_dir = os.path.join(LIB_DIR, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    srcs = _sources()
    hdr_hash = hashlib.sha256()
    for p in _headers():
        with open(p, "rb") as f:
            hdr_hash.update(f.read())
    hdr_hash.update(" ".join(ARCH_FLAGS + COMMON_FLAGS).encode())

    def compile_one(src):
        with open(src, "rb") as f:
            key = hashlib.sha256(f.read() + hdr_hash.digest()).hexdigest()[:16]
        base = os.path.relpath(src, CSRC).replace(os.sep, "_")
        obj = os.path.join(obj_dir, f"{base}.{key}.o")
        if os.path.exists(obj) and not force:
            return obj, ""
        for old in os.listdir(obj_dir):
            if old.startswith(base + "."):
                os.remove(os.path.join(obj_dir, old))
        cmd = [NVCC, *ARCH_FLAGS, *COMMON_FLAGS, "-I", CSRC, "-c", src, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        return obj, r.stderr

    with ThreadPoolExecutor(jobs or min(8, os.cpu_count() or 4)) as ex:
        results = list(ex.map(compile_one, srcs))
    objs = [o for o, _ in results]
    if verbose:
        for _, log in results:
            if log:
                sys.stderr.write(log)
    cmd = [NVCC, *ARCH_FLAGS, "-shared", "-o", LIB_PATH, *objs, "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    with open(STAMP, "w") as f:
        f.write(source_hash())
    return LIB_PATH


def load():
    """Load the library, building it first if the binary is missing or stale."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.environ.get("PEGAINFER_LIB_PATH") and not is_current():
        # several ranks of one box may get here together: one builds, the others wait on the lock
        import fcntl

        os.makedirs(LIB_DIR, exist_ok=True)
        with open(os.path.join(LIB_DIR, ".build.lock"), "w") as lk:
            fcntl.flock(lk, fcntl.LOCK_EX)
            try:
                if not is_current():
                    build()
            finally:
                fcntl.flock(lk, fcntl.LOCK_UN)
    # PEGAINFER_LIB_PATH loads another build of the library as is (A/B timing of kernel changes)
    _lib = ctypes.CDLL(os.environ.get("PEGAINFER_LIB_PATH") or LIB_PATH)
    _lib.pg_last_error.restype = ctypes.c_char_p
    for name in ("pg_gemm_fp8_ws_bytes", "pg_decode_chain_ws_bytes", "pg_argmax_scratch_bytes"):
        if hasattr(_lib, name):
            getattr(_lib, name).restype = ctypes.c_longlong
    return _lib


class NativeError(RuntimeError):
    pass


def check(rc: int) -> None:
    if rc != 0:
        msg = load().pg_last_error().decode(errors="replace")
        raise NativeError(f"libpegainfer_b200 error {rc}: {msg}")


def build_api_counter() -> str:
    """Compile the LD_PRELOAD CUDA API counter (utils/cuda_api_counter.c) next to the main library."""
    src = os.path.join(ROOT, "pegainfer_b200", "utils", "cuda_api_counter.c")
    out = os.path.join(LIB_DIR, "libcuda_api_counter.so")
    os.makedirs(LIB_DIR, exist_ok=True)
    if not os.path.exists(out) or os.path.getmtime(out) < os.path.getmtime(src):
        r = subprocess.run(["gcc", "-O2", "-shared", "-fPIC", "-o", out, src, "-ldl"], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"gcc failed for {src}:\n{r.stderr}")
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_api_counter())
