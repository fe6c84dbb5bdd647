"""Generates the golden fixtures of tests/golden/ from the REFERENCE's own code.

Run in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/reference-checkout [generator,generator,...]
(or set TORCH_INT_REFERENCE to that path; the optional list regenerates only those fixtures)

What comes from where:
  * layernorm_q.npz, dq_add_layernorm_q.npz, quantize_absmax.npz: outputs of the
    reference's importable Python (torch_int/nn/fused.py LayerNormQ.forward,
    torch_int/functional/fused.py dq_add_layernorm_q_py,
    torch_int/functional/quantization.py) executed here on CPU, with a stub in
    place of its CUDA extension module (which cannot be built without a GPU and
    without CUTLASS);
  * bmm_known_answer.npz: the hard-coded 16x16 operands of the reference's
    tests/test_bmm.py:34-106, read from that file as text, with the expected
    result computed by that test's own formula;
  * linear_formulas.npz / bmm_formulas.npz: seeded inputs at reduced sizes with
    the ground truths of the reference's kernel tests evaluated by THEIR
    formulas (tests/test_linear_kernels.py:7-84, tests/test_bmm.py:7-30,112-120):
    a float torch.nn.Linear / torch.bmm, then clamp / round as each test does.
    The tolerances of those tests are stored next to each ground truth.
  * from_float.npz: the conversion code of the reference's own modules (W8A8*Linear.from_float,
    BMM_*.from_scale, LayerNormQ.from_float) executed on seeded float modules.
The fixtures travel with the repository; nothing at test time reads the
reference checkout.
"""
import ast
import os
import re
import sys
import types

import numpy as np
import torch

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("TORCH_INT_REFERENCE", "")
if not REF or not os.path.isdir(os.path.join(REF, "torch_int")):
    raise SystemExit("usage: make_golden.py /path/to/reference-checkout (a directory holding torch_int/)")
OUT = os.path.dirname(os.path.abspath(__file__))


def import_reference():
    """Imports the reference's pure-Python modules with a stub _CUDA module."""
    for name in list(sys.modules):
        if name == "torch_int" or name.startswith("torch_int."):
            del sys.modules[name]
    sys.path.insert(0, REF)
    stub = types.ModuleType("torch_int._CUDA")

    def _unavailable(*a, **k):
        raise RuntimeError("the reference's CUDA extension is not built here")

    for n in ("linear_a8_w8_b32_o32", "linear_relu_a8_w8_b8_o8", "linear_a8_w8_b8_o8",
              "linear_a8_w8_b32_o32_with_scaling", "linear_a8_w8_bfp32_ofp32", "bmm_s8t_s8n_s8t",
              "bmm_s8t_s8n_s32t", "bmm_s8t_s8n_f32t", "dq_add_layernorm_q"):
        setattr(stub, n, _unavailable)
    sys.modules["torch_int._CUDA"] = stub
    import torch_int  # noqa: F401  (the reference's)
    assert os.path.realpath(torch_int.__file__).startswith(os.path.realpath(REF)), torch_int.__file__
    from torch_int.nn.fused import LayerNormQ
    from torch_int.functional.fused import dq_add_layernorm_q_py
    from torch_int.functional.quantization import (quantize_per_tensor_absmax,
                                                   quantize_weight_per_channel_absmax)
    return LayerNormQ, dq_add_layernorm_q_py, quantize_per_tensor_absmax, quantize_weight_per_channel_absmax


def save(name, **arrays):
    path = os.path.join(OUT, name)
    np.savez_compressed(path, **arrays)
    print(f"{name}: {os.path.getsize(path) / 1024:.1f} KiB")


def gen_layernorm(LayerNormQ):
    g = torch.Generator().manual_seed(1234)
    out = {}
    for i, (shape, scale) in enumerate([((2, 3, 4), 1.0), ((4, 16, 64), 8.0), ((3, 5, 768), 20.0),
                                        ((2, 4, 5120), 30.0)]):
        h = shape[-1]
        x = torch.randn(shape, generator=g) * 1.5
        m = LayerNormQ(h)
        m.weight = (1.0 + 0.1 * torch.randn(h, generator=g)) * scale
        m.bias = 0.1 * torch.randn(h, generator=g) * scale
        with torch.no_grad():
            q = m(x)
        out.update({f"x{i}": x.numpy(), f"gamma{i}": m.weight.numpy(), f"beta{i}": m.bias.numpy(),
                    f"eps{i}": np.float64(m.eps), f"q{i}": q.numpy()})
    save("layernorm_q.npz", n=np.int64(4), **out)


def gen_dq_add(dq_add_layernorm_q_py):
    g = torch.Generator().manual_seed(4321)
    out = {}
    # case 0 is the shape and value range of tests/test_dq_add_ln_q.py:8-15
    for i, (shape, scale, gs) in enumerate([((2, 3, 4), 0.01, 1.0), ((2, 8, 256), 0.001, 25.0),
                                            ((1, 6, 5120), 0.0005, 40.0)]):
        h = shape[-1]
        x = torch.randint(-65536, 65536, shape, generator=g, dtype=torch.int32)
        res = torch.randn(shape, generator=g)
        gamma = (1.0 + 0.1 * torch.randn(h, generator=g)) * gs
        beta = 0.1 * torch.randn(h, generator=g) * gs
        with torch.no_grad():
            r, q = dq_add_layernorm_q_py(x, scale, res, gamma, beta, 1e-5)
        out.update({f"in{i}": x.numpy(), f"scale{i}": np.float64(scale), f"res{i}": res.numpy(),
                    f"gamma{i}": gamma.numpy(), f"beta{i}": beta.numpy(), f"eps{i}": np.float64(1e-5),
                    f"res_out{i}": r.numpy(), f"q{i}": q.numpy()})
    save("dq_add_layernorm_q.npz", n=np.int64(3), **out)


def gen_quantize(qt, qc):
    g = torch.Generator().manual_seed(99)
    w = torch.randn(48, 80, generator=g)
    q, s = qt(w.clone())
    qcw, sc = qc(w.clone())
    save("quantize_absmax.npz", w=w.numpy(), q_tensor=q.numpy(), s_tensor=s.numpy(),
         q_channel=qcw.numpy(), s_channel=sc.numpy())


def gen_bmm_known():
    """Operands of test_bmm_s8t_s8n_s8t_2 (tests/test_bmm.py:34-106), taken from the file text."""
    src = open(os.path.join(REF, "tests", "test_bmm.py")).read()
    body = src[src.index("def test_bmm_s8t_s8n_s8t_2"):src.index("def test_bmm_s8t_s8n_s32t")]

    def literal(var):
        m = re.search(rf"\b{var} = torch\.tensor\((\[\[\[.*?\]\]\])", body, re.S)
        return np.array(ast.literal_eval(m.group(1)))

    a, b = literal("a"), literal("b")
    scale = float(re.search(r"scale = ([0-9.eE+-]+)", body).group(1))
    at, bt = torch.tensor(a), torch.tensor(b)
    # the test's formula (tests/test_bmm.py:100-101): A x B (B given [K,N]) * scale, round, clamp
    c = (torch.bmm(at.float(), bt.float()) * scale).round().clamp(-128, 127).to(torch.int8)
    save("bmm_known_answer.npz", a=a.astype(np.int8), b_kn=b.astype(np.int8),
         scale=np.float64(scale), c=c.numpy())


def gen_linear_formulas():
    g = torch.Generator().manual_seed(2024)
    rows, k, n = 48, 256, 96  # reduced from the tests' 128 x 512 x 1024
    w = torch.randint(-128, 127, (n, k), generator=g, dtype=torch.int8)
    x = torch.randint(-128, 127, (rows, k), generator=g, dtype=torch.int8)
    b32 = torch.randint(-2 ** 31, 2 ** 31 - 1, (n,), generator=g, dtype=torch.int32)
    b8 = torch.randint(-128, 127, (n,), generator=g, dtype=torch.int8)
    bf = torch.randn(n, generator=g)

    def lin(wf, bfv):
        layer = torch.nn.Linear(k, n, bias=True)
        layer.weight.data = wf
        layer.bias.data = bfv
        with torch.no_grad():
            return layer(x.float())

    out = dict(x=x.numpy(), w=w.numpy(), b32=b32.numpy(), b8=b8.numpy(), bf=bf.numpy())
    # tests/test_linear_kernels.py:7-18: exact int32 (atol 1e-3 on the float image)
    out["gt_b32_o32"] = lin(w.float(), b32.float()).numpy()
    # :22-35 alpha 0.01, beta 1e-4, atol 0.5
    out["gt_b32_o32_scaling"] = lin(w.float() * 0.01, b32.float() * 0.0001).numpy()
    # :39-51 alpha 0.001, beta 1, atol 0.5
    out["gt_bfp32_ofp32"] = lin(w.float() * 0.001, bf.float() * 1).numpy()
    # :55-67 alpha 0.001 beta 0.01, clamp(-128,127).round(), atol 1
    out["gt_b8_o8"] = lin(w.float() * 0.001, b8.float() * 0.01).clamp(-128, 127).round().numpy()
    # :71-84 relu: clamp(0,127).round(), atol 1
    out["gt_relu_b8_o8"] = lin(w.float() * 0.001, b8.float() * 0.01).clamp(0, 127).round().numpy()
    out["alpha_beta"] = np.array([[1, 1], [0.01, 0.0001], [0.001, 1], [0.001, 0.01], [0.001, 0.01]], dtype=np.float64)
    out["atol"] = np.array([1e-3, 0.5, 0.5, 1.0, 1.0])
    save("linear_formulas.npz", **out)


def gen_bmm_formulas():
    g = torch.Generator().manual_seed(77)
    bsz, m, k, n = 2, 64, 128, 32  # reduced from 1 x 512 x 512 x 32
    a = torch.randint(-128, 127, (bsz, m, k), generator=g, dtype=torch.int8)
    b = torch.randint(-128, 127, (bsz, n, k), generator=g, dtype=torch.int8)
    scale = 0.001
    f = torch.bmm(a.float(), b.float().transpose(1, 2))
    save("bmm_formulas.npz", a=a.numpy(), b=b.numpy(), scale=np.float64(scale),
         # tests/test_bmm.py:7-16 (allclose), :20-30 (MSE), :112-120 (allclose)
         gt_s8=(f * scale).clamp(-128, 127).round().to(torch.int8).numpy(),
         gt_f32=(f * scale).numpy(), gt_s32=f.round().to(torch.int32).numpy())


def gen_from_float():
    """The conversion code of the reference's own modules (torch_int/nn/linear.py:45-57,89-102,161-179,
    218-229; nn/bmm.py:17-24,39-46; nn/fused.py:20-27) executed on seeded float modules: quantised
    weights, biases and scale factors.  The float modules are rebuilt for every call because the
    reference quantises in place (functional/quantization.py:12)."""
    from torch_int.nn.bmm import BMM_S8T_S8N_F32T, BMM_S8T_S8N_S8T
    from torch_int.nn.fused import LayerNormQ
    from torch_int.nn.linear import (W8A8B8O8Linear, W8A8B8O8LinearReLU, W8A8B32O32Linear,
                                     W8A8BFP32OFP32Linear)

    def float_linear():
        g = torch.Generator().manual_seed(321)
        lin = torch.nn.Linear(48, 80)
        with torch.no_grad():
            lin.weight.copy_(torch.randn(80, 48, generator=g) * 0.2)
            lin.bias.copy_(torch.randn(80, generator=g) * 0.5)
        return lin

    out = {"w": float_linear().weight.detach().numpy().copy(), "b": float_linear().bias.detach().numpy().copy(),
           "input_scale": np.float64(0.037), "output_scale": np.float64(0.052)}
    with torch.no_grad():
        for tag, cls in (("b8o8", W8A8B8O8Linear), ("relu", W8A8B8O8LinearReLU), ("b32o32", W8A8B32O32Linear)):
            m = cls.from_float(float_linear(), 0.037, 0.052)
            out.update({f"{tag}_weight": m.weight.numpy(), f"{tag}_bias": m.bias.numpy(),
                        f"{tag}_a": np.float32(float(m.a)), f"{tag}_b": np.float32(float(m.b))})
        m = W8A8BFP32OFP32Linear.from_float(float_linear(), 0.037)
        out.update({"bfp32_weight": m.weight.numpy(), "bfp32_bias": m.bias.numpy(), "bfp32_a": np.float32(float(m.a))})
        out["bmm_s8t_a"] = np.float32(float(BMM_S8T_S8N_S8T.from_scale(1.0 / 127, 0.031, 0.044).a))
        out["bmm_f32t_a"] = np.float32(float(BMM_S8T_S8N_F32T.from_scale(0.021, 0.017).a))
        g = torch.Generator().manual_seed(322)
        ln = torch.nn.LayerNorm(96)
        ln.weight.copy_(torch.randn(96, generator=g) * 0.1 + 1)
        ln.bias.copy_(torch.randn(96, generator=g) * 0.1)
        out.update({"ln_w": ln.weight.detach().numpy().copy(), "ln_b": ln.bias.detach().numpy().copy()})
        q = LayerNormQ.from_float(ln, 0.061)
        out.update({"lnq_weight": q.weight.detach().numpy(), "lnq_bias": q.bias.detach().numpy(),
                    "ln_output_scale": np.float64(0.061), "ln_eps": np.float64(q.eps)})
    save("from_float.npz", **out)


GENERATORS = ("layernorm", "dq_add", "quantize", "bmm_known", "linear_formulas", "bmm_formulas", "from_float")

if __name__ == "__main__":
    # optional second argument: comma-separated subset of GENERATORS (default: all)
    only = set(sys.argv[2].split(",")) if len(sys.argv) > 2 else set(GENERATORS)
    assert only <= set(GENERATORS), f"unknown generator in {only}; choose from {GENERATORS}"
    LayerNormQ, dq_py, qt, qc = import_reference()
    if "layernorm" in only:
        gen_layernorm(LayerNormQ)
    if "dq_add" in only:
        gen_dq_add(dq_py)
    if "quantize" in only:
        gen_quantize(qt, qc)
    if "bmm_known" in only:
        gen_bmm_known()
    if "linear_formulas" in only:
        gen_linear_formulas()
    if "bmm_formulas" in only:
        gen_bmm_formulas()
    if "from_float" in only:
        gen_from_float()
