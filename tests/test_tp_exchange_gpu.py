"""The reduce + LayerNorm-quantise kernel of the tensor-parallel exchange with its synchronisation folded
in (ti_tp_exchange_reduce_layernorm_q), on ONE GPU: with a single rank the kernel signals and waits on
its own pad, so the whole protocol (arrival words, CTA counter, completion words, epochs) runs inside one
launch.  A second test lets a wait run out on purpose - a pad word that nothing sets - and checks that
the kernel ends, reports status 105 and leaves the context usable; nothing faults or hangs."""
import time

import pytest
import torch

from helpers import assert_bit_exact, assert_quant_close
from oracle import w8a8 as O

pytestmark = pytest.mark.gpu


def _inputs(rows, h, slabs, seed):
    g = torch.Generator().manual_seed(seed)
    stage = torch.randint(-60000, 60000, (slabs, rows, h), generator=g, dtype=torch.int32)
    res = torch.randn((rows, h), generator=g)
    bias = torch.randn(h, generator=g) * 0.1
    gamma, beta = torch.rand(h, generator=g) * 20 + 5, torch.randn(h, generator=g)
    return stage, res, bias, gamma, beta


@pytest.mark.parametrize("rows,h,slabs", [(5, 768, 2), (300, 5120, 4), (64, 12288, 8)])
def test_exchange_kernel_single_rank(cuda_ops, rows, h, slabs):
    C = cuda_ops
    stage, res, bias, gamma, beta = _inputs(rows, h, slabs, 3)
    want_res, want_q = O.dq_add_layernorm_q_bias(stage.sum(0, dtype=torch.int32), 2e-4, bias, res, gamma, beta, 1e-5)
    pad = torch.zeros(64, dtype=torch.int32, device="cuda")
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    q = torch.full((rows + 2, h), 99, dtype=torch.int8, device="cuda")
    sd, rd = stage.cuda(), res.cuda()
    for epoch in (1, 2, 3):     # consecutive exchanges reuse the pad and the counter
        out = C.tp_exchange_reduce_layernorm_q(sd, slabs, rows * h, 2e-4, bias.cuda(), rd, gamma.cuda(), beta.cuda(),
                                               1e-5, [q.data_ptr()], 1, [pad.data_ptr()], 0, epoch, counter,
                                               limit_ms=500)
        assert C.device_status() == 0
        assert_bit_exact(out, want_res, "residual rows")
        assert_quant_close(q[1:rows + 1], want_q, what="int8 rows")
        assert int(q[0].eq(99).all()) and int(q[rows + 1].eq(99).all()), "rows outside the offset range are untouched"
        assert int(counter.item()) == 0, "the CTA counter is back at zero"
        p = pad.cpu()
        assert int(p[0]) == epoch and int(p[8]) == epoch, "arrival and completion words carry the epoch"
    # same numbers as the kernel without the folded-in synchronisation
    q2 = torch.empty((rows, h), dtype=torch.int8, device="cuda")
    out2 = C.tp_reduce_layernorm_q(sd, slabs, rows * h, 2e-4, bias.cuda(), rd, gamma.cuda(), beta.cuda(), 1e-5,
                                   [q2.data_ptr()], 0)
    assert_bit_exact(out2, out) and assert_bit_exact(q2, q[1:rows + 1])


def test_a_wait_that_runs_out_is_reported_not_hung(cuda_ops):
    """Two ranks are declared but the second rank's words are never written: the arrival wait gives up
    after its limit, the status word becomes 105, later waits do not block, and after a reset the same
    buffers work again."""
    C = cuda_ops
    rows, h = 40, 1024
    stage, res, bias, gamma, beta = _inputs(rows, h, 2, 4)
    mine = torch.zeros(64, dtype=torch.int32, device="cuda")
    nobody = torch.zeros(64, dtype=torch.int32, device="cuda")   # stands in for a rank that never arrives
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    q = torch.zeros((rows, h), dtype=torch.int8, device="cuda")
    args = (stage.cuda(), 2, rows * h, 1e-4, bias.cuda(), res.cuda(), gamma.cuda(), beta.cuda(), 1e-5, [q.data_ptr()], 0)
    t0 = time.time()
    C.tp_exchange_reduce_layernorm_q(*args, [mine.data_ptr(), nobody.data_ptr()], 0, 1, counter, limit_ms=100)
    assert C.device_status(reset=False) == 105
    # no wait blocks while the status word is set: a second launch returns at once
    C.tp_exchange_reduce_layernorm_q(*args, [mine.data_ptr(), nobody.data_ptr()], 0, 2, counter, limit_ms=100)
    torch.cuda.synchronize()
    assert time.time() - t0 < 5.0
    assert C.device_status(reset=True) == 105 and C.device_status() == 0
    assert int(counter.item()) == 0
    # the context is intact: the single-rank form on the same buffers gives the right answer
    want_res, want_q = O.dq_add_layernorm_q_bias(stage.sum(0, dtype=torch.int32), 1e-4, bias, res, gamma, beta, 1e-5)
    out = C.tp_exchange_reduce_layernorm_q(*args, [mine.data_ptr()], 0, 3, counter, limit_ms=500)
    assert C.device_status() == 0
    assert_bit_exact(out, want_res) and assert_quant_close(q, want_q)
    # the stand-alone barrier kernel behaves the same way
    C.tp_barrier([mine.data_ptr() + 128, nobody.data_ptr() + 128], 0, 1, torch.device("cuda", 0), limit_ms=100)
    assert C.device_status(reset=True) == 105 and C.device_status() == 0
