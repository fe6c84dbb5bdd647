"""TEST INFRASTRUCTURE: builds oracle/_ref/ref_fused.so from the REFERENCE's own source.

The reference's dq_add_layernorm_q (torch_int/kernels/fused.cu) is plain libtorch code, so it
compiles with g++ on CPU and gives the oracle a real-reference check for that op.  Its GEMM/BMM
sources (linear.cu, bmm.cu) are CUTLASS template instantiations and CUTLASS is an empty,
un-vendored submodule of the reference tree: they cannot be built here.

Usage: python oracle/build_ref.py [/path/to/reference-checkout] [--force]
Default location: the directory `reference` next to this repository, or $TORCH_INT_REFERENCE.
The output is git-ignored; nothing is copied from the reference.
"""
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "ref_fused.so")
BINDING = os.path.join(HERE, "ref_fused_binding.cpp")


def reference_dir(path=None):
    cands = [path, os.environ.get("TORCH_INT_REFERENCE"),
             os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")]
    for c in cands:
        if c and os.path.isfile(os.path.join(c, "torch_int", "kernels", "fused.cu")):
            return c
    return None


def build(path=None, force=False):
    """Returns the path of the built module, or None when no reference checkout is available."""
    ref = reference_dir(path)
    if ref is None:
        return OUT if os.path.exists(OUT) else None
    src = os.path.join(ref, "torch_int", "kernels", "fused.cu")
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= max(os.path.getmtime(src), os.path.getmtime(BINDING)):
        return OUT
    import torch
    from torch.utils import cpp_extension as ce
    os.makedirs(OUT_DIR, exist_ok=True)
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")  # common.h includes cuda.h
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O1", "-std=c++17", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=ref_fused",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)]
    for inc in ce.include_paths() + [sysconfig.get_paths()["include"], cuda_inc, os.path.join(ref, "torch_int", "kernels")]:
        cmd += ["-I", inc]
    cmd += ["-x", "c++", src, BINDING, "-o", OUT, "-L", libdir, "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_python",
            "-Wl,-rpath," + libdir]
    subprocess.check_call(cmd)
    return OUT


def load():
    """The built module (imports oracle/_ref/ref_fused.so), or None if it has not been built."""
    if not os.path.exists(OUT):
        return None
    import importlib.util
    import torch  # noqa: F401  (libtorch must be loaded first)
    try:
        spec = importlib.util.spec_from_file_location("ref_fused", OUT)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    except (ImportError, OSError):  # built against another libtorch: treat as not built
        return None
    return mod


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    print(build(args[0] if args else None, force="--force" in sys.argv))
