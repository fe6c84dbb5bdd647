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
        # the same count in device memory: the one-token attention kernel reads it there, so a decode
        # step has no per-step host parameters and can be replayed from a CUDA graph
        self.pos = torch.zeros(1, dtype=torch.int32, device=device)
        self.graph = None  # (CUDAGraph, static token buffer, static next-token buffer) of generate_greedy
        el = local_heads * head_dim
        self.keys = [torch.zeros((batch_size, self.capacity, el), dtype=torch.int8, device=device)
                     for _ in range(num_layers)]
        self.values_t = [torch.zeros((batch_size, local_heads, head_dim, self.capacity), dtype=torch.int8,
                                     device=device) for _ in range(num_layers)]

    def reset(self):
        self.length = 0
        self.pos.zero_()

    def set_length(self, n):
        self.length = int(n)
        self.pos.fill_(int(n))

    def store(self, layer_idx, k_view, v_view, bsz, tgt_len, past_len, b0=0):
        """Stores new keys and values at positions [past_len, past_len + T) of the sequences
        [b0, b0 + B).  k_view / v_view: int8 [B, T, Hl*D] views (tokens may be strided, e.g.
        column blocks of a fused q/k/v projection).  Returns the (keys, transposed values)
        views of those sequences."""
        if b0 < 0 or b0 + bsz > self.batch_size:
            raise RuntimeError(f"cache was allocated for batch {self.batch_size}, got sequences [{b0}, {b0 + bsz})")
        if past_len + tgt_len > self.capacity:
            raise RuntimeError(f"cache capacity {self.capacity} exceeded ({past_len} + {tgt_len})")
        kc, vt = self.keys[layer_idx][b0:b0 + bsz], self.values_t[layer_idx][b0:b0 + bsz]
        kc[:, past_len:past_len + tgt_len].copy_(k_view)
        C.transpose_values(v_view.as_strided((bsz, tgt_len, self.local_heads, self.head_dim),
                                             (v_view.stride(0), v_view.stride(1), self.head_dim, 1)),
                           vt, past_len)
        return kc, vt
