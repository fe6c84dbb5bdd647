// TEST INFRASTRUCTURE.  pybind11 binding around the REFERENCE's own C++ implementation of
// dq_add_layernorm_q (torch_int/kernels/fused.cu:7-25 of the reference checkout, five ATen
// calls that also run on CPU tensors, as the reference's tests/test_dq_add_ln_q.py does).
// oracle/build_ref.py compiles that source file where it lies, together with this binding, into
// oracle/_ref/ref_fused.so; no reference source is copied into this repository.
#include <torch/extension.h>

#include "include/fused.h"  // the reference's header, found through -I <reference>/torch_int/kernels

PYBIND11_MODULE(ref_fused, m) {
  m.def("dq_add_layernorm_q", &dq_add_layernorm_q,
        "the reference's dq_add_layernorm_q(input int32, input_scale, residual, gamma, beta, eps)");
}
