"""Pins the CPU oracle against the fixtures generated from the reference's own
code and test formulas (tests/golden/make_golden.py).  No GPU."""
import os

import numpy as np
import torch

from oracle import w8a8 as O


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def test_layernorm_q_matches_reference_python(golden_dir):
    # Outputs of the reference's LayerNormQ.forward (torch_int/nn/fused.py:13-18).
    z = _load(golden_dir, "layernorm_q.npz")
    for i in range(int(z["n"])):
        q = O.layernorm_q(torch.from_numpy(z[f"x{i}"]), torch.from_numpy(z[f"gamma{i}"]),
                          torch.from_numpy(z[f"beta{i}"]), float(z[f"eps{i}"]))
        assert torch.equal(q, torch.from_numpy(z[f"q{i}"])), f"case {i}"


def test_dq_add_layernorm_q_matches_reference_python(golden_dir):
    # Outputs of dq_add_layernorm_q_py (torch_int/functional/fused.py:5-12), whose
    # case 0 is the shape of the reference's tests/test_dq_add_ln_q.py:8.
    z = _load(golden_dir, "dq_add_layernorm_q.npz")
    for i in range(int(z["n"])):
        r, q = O.dq_add_layernorm_q(torch.from_numpy(z[f"in{i}"]), float(z[f"scale{i}"]),
                                    torch.from_numpy(z[f"res{i}"]), torch.from_numpy(z[f"gamma{i}"]),
                                    torch.from_numpy(z[f"beta{i}"]), float(z[f"eps{i}"]))
        assert torch.equal(r, torch.from_numpy(z[f"res_out{i}"])), f"residual, case {i}"
        assert torch.equal(q, torch.from_numpy(z[f"q{i}"])), f"q, case {i}"


def test_bmm_known_answer(golden_dir):
    # The hard-coded operands of the reference's tests/test_bmm.py:34-106.
    z = _load(golden_dir, "bmm_known_answer.npz")
    a = torch.from_numpy(z["a"])
    b_nk = torch.from_numpy(z["b_kn"]).transpose(1, 2).contiguous()  # the test transposes too (:103)
    c = O.bmm_s8t_s8n_s8t(a, b_nk, float(z["scale"]))
    want = torch.from_numpy(z["c"])
    # The test reports an MSE; its formula rounds the same fp32 product, so the
    # results agree except possibly at exact rounding ties.
    d = (c.int() - want.int()).abs()
    assert int(d.max()) <= 1 and float((d == 0).double().mean()) >= 0.99
    assert torch.equal(O.bmm_s8t_s8n_s32t(a, b_nk),
                       torch.bmm(a.double(), b_nk.double().transpose(1, 2)).to(torch.int32))


def test_linear_formulas_within_reference_tolerances(golden_dir):
    # Ground truths of tests/test_linear_kernels.py:7-84 with the tolerances of those tests.
    z = _load(golden_dir, "linear_formulas.npz")
    x, w = torch.from_numpy(z["x"]), torch.from_numpy(z["w"])
    b32, b8, bf = torch.from_numpy(z["b32"]), torch.from_numpy(z["b8"]), torch.from_numpy(z["bf"])
    ab, atol = z["alpha_beta"], z["atol"]
    # int32 + int32 bias: the float image of the exact result (wrap-around excluded:
    # the float ground truth cannot represent it, compare where no wrap occurred)
    y = O.linear_a8_w8_b32_o32(x, w, b32)
    exact = O.gemm_acc_numpy(x, w).long() + b32.long()
    nowrap = (exact >= -2 ** 31) & (exact < 2 ** 31)
    gt = torch.from_numpy(z["gt_b32_o32"])
    assert torch.equal(y.long()[nowrap], exact[nowrap])
    assert torch.allclose(gt[nowrap], y.float()[nowrap], atol=float(atol[0]), rtol=1e-6)
    y = O.linear_a8_w8_b32_o32_with_scaling(x, w, b32, *ab[1])
    assert torch.allclose(torch.from_numpy(z["gt_b32_o32_scaling"]), y.float(), atol=float(atol[1]), rtol=1e-6)
    y = O.linear_a8_w8_bfp32_ofp32(x, w, bf, *ab[2])
    assert torch.allclose(torch.from_numpy(z["gt_bfp32_ofp32"]), y, atol=float(atol[2]))
    y = O.linear_a8_w8_b8_o8(x, w, b8, *ab[3])
    assert torch.allclose(torch.from_numpy(z["gt_b8_o8"]), y.float(), atol=float(atol[3]))
    y = O.linear_relu_a8_w8_b8_o8(x, w, b8, *ab[4])
    assert torch.allclose(torch.from_numpy(z["gt_relu_b8_o8"]), y.float(), atol=float(atol[4]))


def test_bmm_formulas(golden_dir):
    # tests/test_bmm.py:7-16 (exact allclose), :20-30 (MSE), :112-120 (exact).
    z = _load(golden_dir, "bmm_formulas.npz")
    a, b, s = torch.from_numpy(z["a"]), torch.from_numpy(z["b"]), float(z["scale"])
    assert torch.equal(O.bmm_s8t_s8n_s32t(a, b), torch.from_numpy(z["gt_s32"]))
    d = (O.bmm_s8t_s8n_s8t(a, b, s).int() - torch.from_numpy(z["gt_s8"]).int()).abs()
    assert int(d.max()) <= 1 and float((d == 0).double().mean()) >= 0.999
    mse = torch.mean((O.bmm_s8t_s8n_f32t(a, b, s) - torch.from_numpy(z["gt_f32"])) ** 2)
    assert float(mse) < 1e-8


def test_quantize_absmax_matches_reference(golden_dir):
    # torch_int/functional/quantization.py:6-27, through the product's helpers
    # (pure torch, importable without a GPU build only via the functional module).
    import importlib.util
    import sys
    path = os.path.join(os.path.dirname(golden_dir), "..", "torch-int_b200", "torch_int", "functional",
                        "quantization.py")
    spec = importlib.util.spec_from_file_location("_quantization_under_test", os.path.abspath(path))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    z = _load(golden_dir, "quantize_absmax.npz")
    w = torch.from_numpy(z["w"])
    keep = w.clone()
    q, s = mod.quantize_per_tensor_absmax(w)
    assert torch.equal(q, torch.from_numpy(z["q_tensor"])) and float(s) == float(z["s_tensor"])
    qc, sc = mod.quantize_weight_per_channel_absmax(w)
    assert torch.equal(qc, torch.from_numpy(z["q_channel"]))
    assert torch.equal(sc, torch.from_numpy(z["s_channel"]))
    assert torch.equal(w, keep), "the source tensor must not be modified"
    del sys
