"""Pre-allocated int8 key/value cache for the Int8 OPT decoder.

The reference grows its cache with ``torch.cat`` and re-transposes the values on
every call (torch_int/models/opt.py:113-116,180).  Here, per layer,
  keys    are kept as rows   [B, capacity, Hl*D]   (what k_proj writes), and
  values  are kept transposed [B, Hl, D, capacity]  (the K-major operand P.V needs),
with the capacity rounded up to a multiple of 16 so that the padded key length
satisfies the kernels' shape rules; positions beyond the current length are
masked by the softmax kernel and contribute nothing.
"""
import torch

from .. import _CUDA as C


class StaticInt8KVCache:
    def __init__(self, num_layers, batch_size, local_heads, head_dim, max_len, device):
        self.capacity = (max_len + 15) // 16 * 16
        self.batch_size = batch_size
        self.local_heads = local_heads
        self.head_dim = head_dim
        self.length = 0  # positions filled so far (same for every layer once a forward ends)
        el = local_heads * head_dim
        self.keys = [torch.zeros((batch_size, self.capacity, el), dtype=torch.int8, device=device)
                     for _ in range(num_layers)]
        self.values_t = [torch.zeros((batch_size, local_heads, head_dim, self.capacity), dtype=torch.int8,
                                     device=device) for _ in range(num_layers)]

    def reset(self):
        self.length = 0

    def append(self, layer_idx, k_proj, v_proj, x2d, bsz, tgt_len, past_len, b0=0):
        """Projects x2d [B*T, E] to keys and values and stores them at positions
        [past_len, past_len + T) of the sequences [b0, b0 + B).  The key GEMM writes
        straight into the cache.  Returns the (keys, transposed values) views of
        those sequences."""
        if b0 < 0 or b0 + bsz > self.batch_size:
            raise RuntimeError(f"cache was allocated for batch {self.batch_size}, got sequences [{b0}, {b0 + bsz})")
        if past_len + tgt_len > self.capacity:
            raise RuntimeError(f"cache capacity {self.capacity} exceeded ({past_len} + {tgt_len})")
        kc, vt = self.keys[layer_idx][b0:b0 + bsz], self.values_t[layer_idx][b0:b0 + bsz]
        el, e = kc.shape[2], x2d.shape[1]
        dst = kc[:, past_len:, :]  # view starting at the first new row of batch 0
        if tgt_len == 1:
            # one row per sequence: a single GEMM with the cache's batch stride as row stride
            C.gemm_i8_ex(x2d, k_proj.weight, dst, k_proj.bias, epilogue=C.EPI_S8_BIAS_S8, m=bsz, n=el, k=e,
                         lda=e, ldb=e, ldc=self.capacity * el, alpha=k_proj._scalar("a"), beta=k_proj._scalar("b"))
        else:
            C.gemm_i8_ex(x2d, k_proj.weight, dst, k_proj.bias, epilogue=C.EPI_S8_BIAS_S8, m=tgt_len, n=el, k=e,
                         batch=bsz, lda=e, ldb=e, ldc=el, stride_a=tgt_len * e, stride_b=0,
                         stride_c=self.capacity * el, alpha=k_proj._scalar("a"), beta=k_proj._scalar("b"))
        v = v_proj._op(x2d)
        C.transpose_values(v.view(bsz, tgt_len, self.local_heads, self.head_dim), vt, past_len)
        return kc, vt
