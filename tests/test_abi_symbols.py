"""The C-ABI library loads without a GPU and exports every symbol its header declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "torch-int_b200", "torch_int", "lib", "libtorch_int_b200.so")
HEADER = os.path.join(ROOT, "include", "torch_int_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ti_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_reference_ops():
    # One entry point per callable of the reference's pybind module
    # (torch_int/kernels/bindings.cpp:5-20).
    names = declared_symbols()
    for op in ("linear_relu_a8_w8_b8_o8", "linear_a8_w8_b32_o32", "linear_a8_w8_bfp32_ofp32",
               "linear_a8_w8_b32_o32_with_scaling", "linear_a8_w8_b8_o8", "dq_add_layernorm_q",
               "bmm_s8t_s8n_s8t", "bmm_s8t_s8n_f32t", "bmm_s8t_s8n_s32t"):
        assert "ti_" + op in names


def test_library_exports_every_declared_symbol():
    assert os.path.exists(LIB), f"{LIB} is not built (python torch-int_b200/csrc/build.py)"
    lib = ctypes.CDLL(LIB)
    missing = [s for s in declared_symbols() if not hasattr(lib, s)]
    assert not missing, f"declared in the header but not exported: {missing}"
    lib.ti_abi_version.restype = ctypes.c_int
    assert lib.ti_abi_version() == 1
    lib.ti_last_error.restype = ctypes.c_char_p
    assert isinstance(lib.ti_last_error(), bytes)


def test_argument_validation_needs_no_gpu():
    """Shape / alignment errors are reported by the host code before any CUDA call."""
    lib = ctypes.CDLL(LIB)
    lib.ti_last_error.restype = ctypes.c_char_p
    i64, f32, p = ctypes.c_int64, ctypes.c_float, ctypes.c_void_p
    lib.ti_linear_a8_w8_b8_o8.argtypes = [p, p, p, p, i64, i64, i64, f32, f32, p]
    buf = ctypes.create_string_buffer(4096 + 64)
    base = (ctypes.addressof(buf) + 63) & ~63
    # K not a multiple of 16
    rc = lib.ti_linear_a8_w8_b8_o8(base, base, base, base, 4, 16, 24, 1.0, 1.0, None)
    assert rc == -1 and b"multiple of 16" in lib.ti_last_error()
    # N not a multiple of 16 for an int8 output
    rc = lib.ti_linear_a8_w8_b8_o8(base, base, base, base, 4, 20, 32, 1.0, 1.0, None)
    assert rc == -1 and b"N=20" in lib.ti_last_error()
    # misaligned pointer
    rc = lib.ti_linear_a8_w8_b8_o8(base + 1, base, base, base, 4, 16, 32, 1.0, 1.0, None)
    assert rc == -1 and b"aligned" in lib.ti_last_error()
    # null pointer
    rc = lib.ti_linear_a8_w8_b8_o8(None, base, base, base, 4, 16, 32, 1.0, 1.0, None)
    assert rc == -1
    # empty problem: accepted, nothing launched
    assert lib.ti_linear_a8_w8_b8_o8(base, base, base, base, 0, 16, 32, 1.0, 1.0, None) == 0


def test_attention_and_row_kernel_validation_needs_no_gpu():
    """The attention entry points and the row kernels check their arguments on the host as well."""
    lib = ctypes.CDLL(LIB)
    lib.ti_last_error.restype = ctypes.c_char_p
    i64, f32, p = ctypes.c_int64, ctypes.c_float, ctypes.c_void_p
    lib.ti_attention_prefill_s8.argtypes = [p, i64, i64, p, i64, i64, p, i64, p, i64, i64,
                                            i64, i64, i64, i64, i64, f32, f32, p]
    buf = ctypes.create_string_buffer(1 << 16)
    base = (ctypes.addressof(buf) + 63) & ~63

    def attn(q=base, ld_q=256, qbs=256 * 32, k=base, ld_k=256, kbs=256 * 32, vt=base, ld_vt=32, ctx=base, ld_ctx=256,
             cbs=256 * 32, batch=1, heads=2, d=128, t=32, s=32):
        return lib.ti_attention_prefill_s8(q, ld_q, qbs, k, ld_k, kbs, vt, ld_vt, ctx, ld_ctx, cbs, batch, heads, d,
                                           t, s, 1.0, 1.0, None)
    assert attn(d=96) == -1 and b"head_dim" in lib.ti_last_error()
    assert attn(t=40, s=32) == -1                                   # fewer keys than query rows
    assert attn(ld_q=250) == -1 and b"multiples of 16" in lib.ti_last_error()
    assert attn(q=base + 8) == -1
    assert attn(ld_k=128) == -1 and b"row stride" in lib.ti_last_error()   # narrower than heads * head_dim
    assert attn(ld_vt=16) == -1                                      # shorter than the key count
    assert attn(q=None) == -1
    assert attn(batch=0) == 0 and attn(t=0, s=0) == 0                # empty: accepted, nothing launched
    lib.ti_decode_attention_s8.argtypes = [p, i64, p, p, i64, i64, i64, i64, p, f32, f32, p, i64, p]
    rc = lib.ti_decode_attention_s8(base, 768, base, base, 1, 2, 96, 64, base, 1.0, 1.0, base, 256, None)
    assert rc == -1 and b"head_dim" in lib.ti_last_error()
    rc = lib.ti_decode_attention_s8(base, 768, base, base, 1, 2, 128, 60, base, 1.0, 1.0, base, 256, None)
    assert rc == -1                                                  # capacity not a multiple of 16
    assert lib.ti_decode_attention_s8(base, 768, base, base, 0, 2, 128, 64, base, 1.0, 1.0, base, 256, None) == 0
