"""Builds libtorch_int_b200.so (the CUDA kernels plus the C ABI) for sm_100a.

Usage: python build.py [--force] [--verbose]
The library is written next to the Python package (torch_int/lib/) so that it
travels with the source tree; nothing is installed into site-packages.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(os.path.dirname(HERE), "torch_int", "lib")
OUT = os.path.join(OUT_DIR, "libtorch_int_b200.so")
SOURCES = ["gemm_i8_sm100.cu", "norm_quant.cu", "decode_attention.cu", "attention_prefill_sm100.cu", "abi.cu"]
HEADERS = ["gemm_i8.h", "norm_quant.h", "attention_prefill.h", "sm100_ptx.cuh", "grid_dependency.cuh",
           os.path.join("..", "..", "include", "torch_int_b200.h")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-diag-suppress", "177",
]


def _nvcc():
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def up_to_date():
    if not os.path.exists(OUT):
        return False
    t = os.path.getmtime(OUT)
    deps = [os.path.join(HERE, f) for f in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return all(os.path.getmtime(d) <= t for d in deps)


def build(force=False, verbose=False):
    if not force and up_to_date():
        return OUT
    os.makedirs(OUT_DIR, exist_ok=True)
    objs = []
    procs = []
    for src in SOURCES:
        obj = os.path.join(OUT_DIR, src.replace(".cu", ".o"))
        cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + \
              ["-c", os.path.join(HERE, src), "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for src, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(out)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
    # link next to the target and rename: a reader never sees a half-written library
    tmp = OUT + ".tmp"
    cmd = [_nvcc(), "-shared", "-Wno-deprecated-gpu-targets", "-o", tmp] + objs + ["-lcudart_static", "-ldl", "-lrt", "-lpthread"]
    subprocess.check_call(cmd)
    os.replace(tmp, OUT)
    for o in objs:
        os.remove(o)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
