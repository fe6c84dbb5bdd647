"""The ALGORITHM of the fused prefill attention kernel (csrc/attention_prefill_sm100.cu), emulated tile by
tile in numpy float32 and compared with the oracle chain scores -> softmax -> x127 -> round -> context
(torch_int/models/opt.py:131-181).  This pins the index arithmetic of the kernel (tile counts, causal limits
with a cached prefix, ragged last tiles) and the claim that accumulating the row sum tile by tile with a
running maximum (per column half, combined once) moves the int8 context by at most one unit; it says nothing
about the kernel's PTX."""
import numpy as np
import pytest
import torch

from helpers import rand_s8
from oracle import w8a8 as O

TILE = 128
F = np.float32
LOG2E = F(1.4426950408889634)


def emulate(q, k, vt, past, alpha_qk, alpha_pv):
    """q [T,D], k [S,D], vt [D,S] int8 (one sequence, one head) -> int8 [T,D], following the kernel:
    one CTA per 128 query rows, keys visited in tiles of 128 up to the last one any row of the CTA sees;
    the row sum is built from two per-thread partial sums (keys [0,64) and [64,128) of every tile) with
    2^(x log2 e) as the exponential, every probability from expf and an exact division."""
    t_len, d = q.shape
    s_len = k.shape[0]
    out = np.zeros((t_len, d), dtype=np.int8)
    fmin = F(-np.finfo(np.float32).max)
    for qt in range((t_len + TILE - 1) // TILE):
        t0 = qt * TILE
        kv_end = min(s_len, min(t0 + TILE, t_len) + past)
        nt = (kv_end + TILE - 1) // TILE
        rows = np.arange(t0, t0 + TILE)
        valid = rows < t_len
        lim = np.where(valid, rows + past, -1)
        qtile = np.zeros((TILE, d), dtype=np.int64)
        qtile[valid] = q[t0:t0 + int(valid.sum())]

        def scores(j):
            ktile = np.zeros((TILE, d), dtype=np.int64)          # rows past the end read as zero (TMA fill)
            n = max(0, min(TILE, s_len - j * TILE))
            ktile[:n] = k[j * TILE:j * TILE + n]
            acc = qtile @ ktile.T                                # int32 accumulators
            cols = j * TILE + np.arange(TILE)
            return (F(alpha_qk) * acc.astype(F)).astype(F), cols[None, :] <= lim[:, None]

        # pass 1: two threads per row, each with a running maximum and sum over ITS 64 keys of every tile
        mh = [np.full(TILE, fmin, dtype=F) for _ in range(2)]
        lh = [np.zeros(TILE, dtype=F) for _ in range(2)]
        for j in range(nt):
            s, vis = scores(j)
            for hf in range(2):
                sl = slice(64 * hf, 64 * hf + 64)
                sh, vh = s[:, sl], vis[:, sl]
                any_vis = vh.any(axis=1)
                tmax = np.where(vh, sh, fmin).max(axis=1).astype(F)
                mn = np.where(any_vis, np.maximum(mh[hf], tmax), mh[hf]).astype(F)
                with np.errstate(over="ignore", under="ignore"):
                    lh[hf] = (lh[hf] * np.exp2(((mh[hf] - mn).astype(F) * LOG2E).astype(F)).astype(F)).astype(F)
                    e = np.where(vh, np.exp2(((sh - mn[:, None]).astype(F) * LOG2E).astype(F)), F(0)).astype(F)
                lh[hf] = (lh[hf] + e.sum(axis=1, dtype=F)).astype(F)
                mh[hf] = mn
        m = np.maximum(mh[0], mh[1])
        with np.errstate(over="ignore", under="ignore", invalid="ignore"):
            l = ((lh[0] * np.exp((mh[0] - m).astype(F)).astype(F)).astype(F) +
                 (lh[1] * np.exp((mh[1] - m).astype(F)).astype(F)).astype(F)).astype(F)
        acc_o = np.zeros((TILE, d), dtype=np.int64)
        for j in range(nt):                                      # pass 2
            s, vis = scores(j)
            with np.errstate(invalid="ignore", divide="ignore", over="ignore"):   # rows past the end: masked below
                e = np.exp((s - m[:, None]).astype(F)).astype(F)
                p = np.rint((e / l[:, None]).astype(F) * F(127)).astype(np.int64)
            p = np.where(vis, np.minimum(p, 127), 0)
            vtile = np.zeros((d, TILE), dtype=np.int64)
            n = max(0, min(TILE, s_len - j * TILE))
            vtile[:, :n] = vt[:, j * TILE:j * TILE + n]
            acc_o += p @ vtile.T
        y = np.rint((F(alpha_pv) * acc_o.astype(F)).astype(F))
        o = np.clip(y, -128, 127).astype(np.int8)
        out[t0:t0 + int(valid.sum())] = o[valid]
    return out


@pytest.mark.parametrize("t,past,d", [(128, 0, 128), (200, 0, 64), (77, 51, 128), (300, 5, 64), (130, 126, 128)])
def test_tiled_two_pass_attention_matches_the_oracle_chain(t, past, d):
    s = past + t
    q, k, v = rand_s8((t, d), 11), rand_s8((s, d), 12), rand_s8((s, d), 13)
    vt = v.t().contiguous()
    alpha_qk, alpha_pv = 2.5 / (127 * 127 * d ** 0.5), 0.02
    scores = O.bmm_s8t_s8n_f32t(q.view(1, t, d), k.view(1, s, d), alpha_qk)
    probs = O.softmax_q(scores, O.causal_mask(1, t, s))
    want = O.bmm_s8t_s8n_s8t(probs, vt.view(1, d, s), alpha_pv)[0].numpy()
    got = emulate(q.numpy(), k.numpy(), vt.numpy(), past, alpha_qk, alpha_pv)
    diff = np.abs(got.astype(np.int32) - want.astype(np.int32))
    assert diff.max() <= 1, diff.max()
    assert (diff == 0).mean() >= 0.995, (diff == 0).mean()
    assert np.abs(want.astype(np.int32)).max() > 20
