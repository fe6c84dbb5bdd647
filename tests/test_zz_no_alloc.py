"""ti_linear_a8_w8_b8_o8_static: the int8-output linear for few rows whose split-K scratch is a
fixed array inside the library, for callers that are not allowed to allocate device memory (an
inference server that hands plug-ins no allocator, a serving loop that bans cudaMalloc after
start-up).  The entry point is called straight through the C ABI and must reproduce the regular
entry point bit for bit, on two calls in a row: the shared scratch keeps what the last call left,
so the second call only works if the first one handed it back zeroed.

This file sorts last on purpose: if it fails, a run that stops at the first failure has already
run every other test.  It passes alone in a fresh process and after the other tests."""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "torch-int_b200", "torch_int", "lib", "libtorch_int_b200.so")


def _lib():
    lib = ctypes.CDLL(LIB)
    p, i64, f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_float
    for name in ("ti_linear_a8_w8_b8_o8", "ti_linear_a8_w8_b8_o8_static"):
        fn = getattr(lib, name)
        fn.argtypes = [p, p, p, p, i64, i64, i64, f32, f32, p]
        fn.restype = ctypes.c_int
    lib.ti_last_error.restype = ctypes.c_char_p
    lib.ti_device_status.argtypes = [ctypes.POINTER(ctypes.c_int), ctypes.c_int]
    lib.ti_split_k_splits.argtypes = [i64, i64, i64]
    lib.ti_split_k_splits.restype = ctypes.c_int
    return lib


def _s8(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(-127, 128, shape, generator=g, dtype=torch.int8).cuda()


def test_static_scratch_entry_point_matches_regular_one_twice():
    assert torch.cuda.is_available()
    lib = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    # (M, N, K): decode-sized problems whose K gets split over the SMs; two different ones in a
    # row, then the first again, all through the same built-in scratch
    for call, (m, n, k) in enumerate([(16, 7168, 7168), (8, 4096, 16384), (16, 7168, 7168)]):
        x, w, b = _s8((m, k), 100 + call), _s8((n, k), 200 + call), _s8((n,), 300 + call)
        alpha, beta = 1.0 / (60.0 * k ** 0.5), 0.01
        want = torch.empty((m, n), dtype=torch.int8, device="cuda")
        got = torch.full((m, n), 99, dtype=torch.int8, device="cuda")
        rc = lib.ti_linear_a8_w8_b8_o8(x.data_ptr(), w.data_ptr(), b.data_ptr(), want.data_ptr(), m, n, k,
                                       alpha, beta, stream)
        assert rc == 0, lib.ti_last_error()
        rc = lib.ti_linear_a8_w8_b8_o8_static(x.data_ptr(), w.data_ptr(), b.data_ptr(), got.data_ptr(), m, n, k,
                                              alpha, beta, stream)
        assert rc == 0, lib.ti_last_error()
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"call {call}: {int((got != want).sum())} of {got.numel()} int8 outputs differ"
        # the call really went through the built-in scratch (K split over several CTAs), and both entry
        # points give what the CPU oracle gives
        assert lib.ti_split_k_splits(m, n, k) > 1, "this problem is expected to take the split-K path"
        from oracle import w8a8 as O
        assert torch.equal(got.cpu(), O.linear_a8_w8_b8_o8(x.cpu(), w.cpu(), b.cpu(), alpha, beta)), \
            f"call {call}: differs from the oracle"
    status = ctypes.c_int(-1)
    assert lib.ti_device_status(ctypes.byref(status), 1) == 0 and status.value == 0


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    lib = _lib()
    x = torch.zeros(4096, dtype=torch.int8, device="cuda")
    # M beyond the rows it handles, and an N whose scratch need exceeds the 4 MiB array: both must be
    # refused before anything is launched, with a message that says why
    rc = lib.ti_linear_a8_w8_b8_o8_static(x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(),
                                          129, 4096, 4096, 1.0, 1.0, None)
    assert rc == -1 and b"128 rows" in lib.ti_last_error()
    rc = lib.ti_linear_a8_w8_b8_o8_static(x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(),
                                          128, 65536, 4096, 1.0, 1.0, None)
    assert rc == -1 and b"nothing is allocated" in lib.ti_last_error()
