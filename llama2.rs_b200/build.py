"""Builds libllama2_b200.so (the C-ABI library) in-tree for sm_100a with nvcc.

Usage: python build.py [--verbose]   (also importable: build.build())
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libllama2_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
HOST_CXX = "/usr/bin/g++"

CU_SOURCES = ["decode_kernels.cu", "gemv_kernels.cu", "token_kernel.cu", "gemm_tc.cu", "prefill_kernels.cu", "prefill.cu", "model.cu", "attention_noalloc.cu"]
CPP_SOURCES = ["layout.cpp", "synth.cpp", "repack.cpp", "tokenizer.cpp", "tp.cpp"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall", "-ccbin", HOST_CXX,
]


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build(verbose=False, force=False):
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(HERE, "..", "include", "llama2_b200.h"))
    objs, jobs = [], []
    for src in CU_SOURCES + CPP_SOURCES:
        path = os.path.join(CSRC, src)
        obj = os.path.join(HERE, "build", src + ".o")
        objs.append(obj)
        if force or _stale(obj, [path] + headers):
            # L2_TK_TRACE=1: compile the clock stamps of the token kernel in (a debugging build: they cost registers)
            trace = ["-DL2_TK_TRACE"] if os.environ.get("L2_TK_TRACE") else []
            cmd = [NVCC] + NVCC_FLAGS + trace + (["-Xptxas", "-v"] if verbose else []) + ["-c", path, "-o", obj]
            if not src.endswith(".cu"):
                cmd = [NVCC] + NVCC_FLAGS + ["-x", "cu", "-c", path, "-o", obj]
            jobs.append((src, cmd))
    # the translation units compile side by side (the token kernel alone takes most of a minute)
    from concurrent.futures import ThreadPoolExecutor
    with ThreadPoolExecutor(max_workers=max(1, min(8, os.cpu_count() or 1))) as pool:
        results = list(pool.map(lambda j: (j[0], subprocess.run(j[1], capture_output=True, text=True)), jobs))
    for src, r in results:
        if verbose or r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode:
            raise RuntimeError("nvcc failed on " + src)
    if force or _stale(OUT, objs):
        cmd = [NVCC, "-shared", "-o", OUT] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-ccbin", HOST_CXX, "-lpthread", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return OUT


if __name__ == "__main__":
    print(build(verbose="--verbose" in sys.argv, force="--force" in sys.argv))
