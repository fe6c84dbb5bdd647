"""TEST INFRASTRUCTURE: builds oracle/_ref/ref_torch_int.so - the REFERENCE's own CUDA extension.

The reference's GEMM / BMM ops (torch_int/kernels/linear.cu, bmm.cu) are CUTLASS 2.x `device::Gemm`
instantiations.  The reference pins no CUTLASS version (its submodule is empty); this image carries CUTLASS
header trees inside Python packages (flashinfer, tilelang), and the 2.x device API the reference uses is
still part of them.  This recipe compiles the reference's four source files where they lie (nothing is
copied) with nvcc against those headers and this image's libtorch, as PTX for compute_80 (the reference's
Sm80 mma.sync path), which the driver translates for whatever GPU runs the tests.  The result is the
reference itself - with an unknown-to-the-reference CUTLASS version - and is used by tests/ to pin the last
bit of the GEMM epilogues on a GPU.  Outputs only into oracle/_ref/ (git-ignored).

Usage: python oracle/build_ref_gemm.py [/path/to/reference-checkout] [--force]
Takes several minutes.  Returns None (and builds nothing) when the reference checkout, nvcc or the CUTLASS
headers are not available.
"""
import glob
import os
import shutil
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "ref_torch_int.so")
SOURCES = ["linear.cu", "bmm.cu", "fused.cu", "bindings.cpp"]


def reference_dir(path=None):
    cands = [path, os.environ.get("TORCH_INT_REFERENCE"),
             os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")]
    for c in cands:
        if c and os.path.isfile(os.path.join(c, "torch_int", "kernels", "linear.cu")):
            return c
    return None


def cutlass_dir():
    """A CUTLASS tree with include/ and tools/util/include/ (the reference includes cutlass/util/host_tensor.h)."""
    site = sysconfig.get_paths()["purelib"]
    cands = [os.environ.get("CUTLASS_HOME"), "/opt/cutlass",
             os.path.join(site, "flashinfer", "data", "cutlass"),
             os.path.join(site, "tilelang", "3rdparty", "cutlass")]
    for c in cands:
        if c and os.path.isfile(os.path.join(c, "include", "cutlass", "gemm", "device", "gemm.h")) and \
                os.path.isfile(os.path.join(c, "tools", "util", "include", "cutlass", "util", "host_tensor.h")):
            return c
    return None


def build(path=None, force=False):
    ref, cut = reference_dir(path), cutlass_dir()
    nvcc = shutil.which("nvcc") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if ref is None or cut is None or not os.path.exists(nvcc):
        return OUT if os.path.exists(OUT) else None
    kdir = os.path.join(ref, "torch_int", "kernels")
    srcs = [os.path.join(kdir, s) for s in SOURCES]
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= max(os.path.getmtime(s) for s in srcs):
        return OUT
    import torch
    from torch.utils import cpp_extension as ce
    os.makedirs(OUT_DIR, exist_ok=True)
    incs = []
    for inc in ce.include_paths() + [sysconfig.get_paths()["include"], os.path.join(cut, "include"),
                                     os.path.join(cut, "tools", "util", "include"), kdir]:
        incs += ["-I", inc]
    common = [nvcc, "-O2", "-std=c++17", "-gencode", "arch=compute_80,code=compute_80", "-DCUDA_ARCH=800",
              "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__",
              "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
              "-DTORCH_EXTENSION_NAME=ref_torch_int", "-Xcompiler", "-fPIC"] + incs
    objs, procs = [], []
    for src in srcs:
        obj = os.path.join(OUT_DIR, os.path.basename(src) + ".o")
        lang = ["-x", "cu"] if src.endswith(".cu") else []
        procs.append(subprocess.Popen(common + lang + ["-c", src, "-o", obj]))
        objs.append(obj)
    if any(p.wait() != 0 for p in procs):
        raise RuntimeError("nvcc failed on the reference sources")
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    subprocess.check_call([nvcc, "-shared", "-o", OUT + ".tmp"] + objs +
                          ["-L", libdir, "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda", "-ltorch_python",
                           "-Xlinker", "-rpath=" + libdir])
    os.replace(OUT + ".tmp", OUT)
    for o in objs:
        os.remove(o)
    return OUT


def load():
    """The built module (the reference's `torch_int._CUDA` under the name ref_torch_int), or None."""
    if not os.path.exists(OUT):
        return None
    import importlib.util
    import torch  # noqa: F401  (libtorch must be loaded first)
    try:
        spec = importlib.util.spec_from_file_location("ref_torch_int", OUT)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    except (ImportError, OSError):  # built against another libtorch: treat as not built
        return None
    return mod


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    print(build(args[0] if args else None, force="--force" in sys.argv))
