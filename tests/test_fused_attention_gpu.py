"""Parity of the one-kernel causal prefill attention (ti_attention_prefill_s8) with the CPU oracle's
scores -> softmax -> x127 -> round -> context chain (torch_int/models/opt.py:131-181).

Tolerance: the context may differ by one unit where a probability sat on a rounding tie (the row sum
is accumulated in another order than torch's)."""
import pytest
import torch

from helpers import rand_s8, set_fused_attention
from oracle import w8a8 as O

pytestmark = pytest.mark.gpu


def oracle_attention(q, k, vt, alpha_qk, alpha_pv):
    """q [B,H,T,D], k [B,H,S,D], vt [B,H,D,S] int8 -> int8 context [B,T,H*D]."""
    b, h, t, d = q.shape
    s = k.shape[2]
    scores = O.bmm_s8t_s8n_f32t(q.reshape(b * h, t, d), k.reshape(b * h, s, d), alpha_qk)
    probs = O.softmax_q(scores, O.causal_mask(b, t, s))
    ctx = O.bmm_s8t_s8n_s8t(probs, vt.reshape(b * h, d, s), alpha_pv)          # [B*H, T, D]
    return ctx.view(b, h, t, d).permute(0, 2, 1, 3).reshape(b, t, h * d).contiguous()


@pytest.mark.parametrize("b,h,t,past,d", [
    (1, 1, 128, 0, 128),     # one full tile
    (2, 3, 200, 0, 128),     # ragged last query tile, two key tiles
    (1, 2, 384, 0, 64),      # head_dim 64, three tiles
    (2, 2, 77, 51, 128),     # cached prefix: row t sees 51 + t + 1 keys
    (1, 1, 640, 0, 128),     # five key tiles: the tile ring wraps
])
def test_fused_prefill_attention_matches_oracle(cuda_ops, b, h, t, past, d):
    C = cuda_ops
    s = past + t
    s_pad = (s + 15) // 16 * 16
    el = h * d
    q = rand_s8((b, t, el), 1)                       # query rows, heads side by side (as the q projection writes them)
    k = rand_s8((b, s, el), 2)
    v = rand_s8((b, s, el), 3)
    vt = torch.zeros((b, h, d, s_pad), dtype=torch.int8)
    vt[..., :s] = v.view(b, s, h, d).permute(0, 2, 3, 1)
    alpha_qk, alpha_pv = 2.5 / (127 * 127 * d ** 0.5), 0.02
    want = oracle_attention(q.view(b, t, h, d).transpose(1, 2), k.view(b, s, h, d).transpose(1, 2),
                            vt[..., :s].contiguous(), alpha_qk, alpha_pv)
    out = torch.full((b, t, el), 77, dtype=torch.int8, device="cuda")
    C.attention_prefill(q.cuda(), k.cuda(), vt.cuda(), out, batch=b, heads=h, head_dim=d, tgt_len=t, src_len=s,
                        ld_q=el, q_batch_stride=t * el, ld_k=el, k_batch_stride=s * el, ld_vt=s_pad,
                        alpha_qk=alpha_qk, alpha_pv=alpha_pv)
    assert C.device_status() == 0
    diff = (out.cpu().int() - want.int()).abs()
    assert int(diff.max()) <= 1, f"max |d| = {int(diff.max())}"
    assert float((diff == 0).double().mean()) >= 0.995
    assert want.int().abs().max() > 20           # the case exercises the value range


def test_fused_attention_in_the_model(cuda_ops):
    """The model with fused_attention on agrees with the three-kernel wiring (up to tie flips)."""
    from torch_int.models.opt import Int8OPTConfig
    from torch_int.models.random_init import random_int8_opt
    cfg = Int8OPTConfig(vocab_size=512, hidden_size=256, num_hidden_layers=2, ffn_dim=512, num_attention_heads=2,
                        max_position_embeddings=512)
    model = random_int8_opt(cfg, seed=5, device="cuda")
    ids = torch.randint(2, 512, (2, 300), generator=torch.Generator().manual_seed(6)).cuda()
    base = set_fused_attention(model, False)(ids).logits
    fused = set_fused_attention(model, True)(ids).logits
    assert cuda_ops.device_status() == 0
    assert float((fused.argmax(-1) == base.argmax(-1)).double().mean()) > 0.99
    assert float((fused - base).abs().max()) <= 0.05 * float(base.abs().max())
