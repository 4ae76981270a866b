"""Builds the CUDA shared library in-tree with nvcc for sm_100a (cross-compiles without a GPU).

Every source is compiled to an object file on its own (in parallel) and the objects are
linked into kvax_b200/libkvax_b200.so.  Objects live in kvax_b200/_obj/ and are reused while
they are newer than their source and every header.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "_obj")
LIB = os.path.join(HERE, "libkvax_b200.so")
SOURCES = ["api.cu", "mask_build.cu", "permute.cu", "schedule.cu", "attn_fwd.cu", "attn_fwd_one.cu", "attn_bwd.cu", "attn_bwd_fused.cu",
           "wait_probe.cu", "peer_exchange.cu", "attn_merge.cu"]
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = [*ARCH_FLAGS, "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC"]
LINK_FLAGS = [*ARCH_FLAGS, "-shared", "-cudart", "static", "-Xcompiler", "-fPIC"]


def _headers() -> list[str]:
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    return hs + [os.path.join(HERE, "..", "include", "kvax_b200.h")]


def _newer(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    os.makedirs(OBJ, exist_ok=True)
    headers = _headers()
    logs: list[str] = []

    def compile_one(src: str) -> tuple[str, bool]:
        path = os.path.join(CSRC, src)
        obj = os.path.join(OBJ, src.replace(".cu", ".o"))
        if not force and _newer(obj, [path] + headers):
            return obj, False
        cmd = [nvcc, *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-c", path, "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError(f"nvcc failed on {src}")
        if verbose:
            logs.append(f"== {src}\n{res.stderr}")
        return obj, True

    with ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as pool:
        results = list(pool.map(compile_one, SOURCES))
    objs = [o for o, _ in results]
    if force or any(changed for _, changed in results) or not _newer(LIB, objs):
        res = subprocess.run([nvcc, *LINK_FLAGS, "-o", LIB, *objs], capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("nvcc failed linking libkvax_b200.so")
    if verbose:
        print("\n".join(logs))
    build_xla_ffi(verbose=verbose)
    return LIB


def xla_ffi_include_dir() -> str | None:
    """Directory that holds xla/ffi/api/ffi.h: XLA_FFI_INCLUDE_DIR, else jaxlib's copy, else None."""
    d = os.environ.get("XLA_FFI_INCLUDE_DIR")
    if d and os.path.exists(os.path.join(d, "xla", "ffi", "api", "ffi.h")):
        return d
    try:
        import jax.ffi
        d = jax.ffi.include_dir()
        return d if os.path.exists(os.path.join(d, "xla", "ffi", "api", "ffi.h")) else None
    except Exception:
        return None


def build_xla_ffi(verbose: bool = False) -> str | None:
    """Compiles csrc/ffi_xla.cc (the XLA FFI handlers over the C ABI) into libkvax_b200_xla_ffi.so when the XLA FFI
    headers are available; returns None (and says why when verbose) otherwise."""
    inc = xla_ffi_include_dir()
    if inc is None:
        if verbose:
            print("ffi_xla.cc not compiled: no xla/ffi/api/ffi.h (set XLA_FFI_INCLUDE_DIR or install jaxlib)")
        return None
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    out = os.path.join(HERE, "libkvax_b200_xla_ffi.so")
    cmd = [nvcc, "-std=c++17", "-O2", "-Xcompiler", "-fPIC", "-shared", "-I", inc, "-x", "cu", os.path.join(CSRC, "ffi_xla.cc"),
           "-o", out, "-L", HERE, "-l:libkvax_b200.so", "-Xlinker", "-rpath=$ORIGIN"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed building libkvax_b200_xla_ffi.so")
    return out


if __name__ == "__main__":
    print(build(force="-f" in sys.argv or "--force" in sys.argv, verbose="-v" in sys.argv))
