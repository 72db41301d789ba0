"""Builds libemelb.so (the C-ABI library of include/emelb.h) in-tree with nvcc for
sm_100a.  Run directly (`python emel.cpp_b200/build.py`) or through
`__graft_entry__.build()`.  Only out-of-date objects are recompiled."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libemelb.so")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

# per-file extra flags: the bit-exact kernels must not contract a*b+c into one fma
SOURCES = {
    "quantize.cu": ["-fmad=false"],
    "elementwise.cu": ["-fmad=false"],
    "gemv.cu": [],
    "gemv2.cu": [],
    "token_kernel.cu": ["-fmad=false"],
    "synth.cu": [],
    "attention.cu": ["-fmad=false"],
    "attention_bf16.cu": ["-fmad=false"],
    "prefill_attention.cu": [],
    "gemm_tc.cu": [],
    "gemm_q8_mma.cu": [],
    "gemm_q4k_mma.cu": [],
    "gemm_q6k_mma.cu": [],
    "llama.cu": [],
    "comm.cu": [],
    "noalloc.cu": [],
    "gguf.cu": [],
    "upload.cu": [],
    "window.cu": [],
    "api.cu": [],
}


def _nccl_paths():
    try:
        import nvidia.nccl as n  # torch's bundled NCCL (headers + libnccl.so.2)
        base = os.path.dirname(n.__file__) if getattr(n, "__file__", None) else list(n.__path__)[0]
        inc, lib = os.path.join(base, "include"), os.path.join(base, "lib")
        if os.path.exists(os.path.join(inc, "nccl.h")):
            return inc, lib
    except Exception:
        pass
    return None, None


def _newer(src_paths, target):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(p) > t for p in src_paths)


def build(verbose: bool = False, force: bool = False) -> str:
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(os.path.dirname(HERE), "include", "emelb.h"))
    headers.append(os.path.join(os.path.dirname(HERE), "include", "emelb_llama.h"))
    headers.append(os.path.join(os.path.dirname(HERE), "include", "emelb_gguf.h"))
    headers.append(os.path.join(os.path.dirname(HERE), "include", "emelb_window.h"))
    headers = [h for h in headers if os.path.exists(h)]
    nccl_inc, nccl_lib = _nccl_paths()
    objs = []
    for name, extra in SOURCES.items():
        src = os.path.join(CSRC, name)
        if not os.path.exists(src):
            continue
        obj = os.path.join(CSRC, name.replace(".cu", ".o"))
        objs.append(obj)
        if force or _newer([src] + headers, obj):
            cmd = [nvcc] + ARCH + COMMON + extra + (["-Xptxas", "-v"] if verbose else [])
            if nccl_inc:
                cmd += ["-I", nccl_inc, "-DEMELB_HAVE_NCCL=1"]
            cmd += ["-c", src, "-o", obj]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if verbose or r.returncode != 0:
                sys.stderr.write(r.stdout + r.stderr)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed for {name}")
    if force or _newer(objs, OUT):
        cmd = [nvcc] + ARCH + ["-shared", "-o", OUT] + objs
        if nccl_lib:
            # linked by soname; resolved at run time from the same wheel
            cmd += ["-L", nccl_lib, "-l:libnccl.so.2", "-Xlinker", f"-rpath={nccl_lib}"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return OUT


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
