"""Batched int8 products as modules with one folded scale.
Reference: torch_int/nn/bmm.py:5-58."""
import torch

from .._CUDA import bmm_s8t_s8n_f32t, bmm_s8t_s8n_s32t, bmm_s8t_s8n_s8t


class _ScaledBMM(torch.nn.Module):
    def __init__(self, alpha):
        super().__init__()
        self.register_buffer("a", torch.tensor(alpha))
        self._cached = None

    def _alpha(self):
        # Cached Python float instead of a device read-back per call (nn/bmm.py:15,37).
        t = self.a
        c = self._cached
        if c is not None and c[0] is t and c[1] == t._version:
            return c[2]
        v = float(t.item())
        self._cached = (t, t._version, v)
        return v

    @classmethod
    def _with_alpha(cls, alpha):
        m = cls(1.0)
        m.a = alpha if torch.is_tensor(alpha) else torch.tensor(alpha)
        return m


class BMM_S8T_S8N_S8T(_ScaledBMM):
    """int8 [B,M,N] = sat_rne(a * A[b] . B[b]^T); A [B,M,K], B [B,N,K] int8 (P.V)."""

    @torch.no_grad()
    def forward(self, a, b):
        return bmm_s8t_s8n_s8t(a, b, self._alpha())

    @staticmethod
    def from_scale(a_scale, b_scale, output_scale):
        return BMM_S8T_S8N_S8T._with_alpha(a_scale * b_scale / output_scale)


class BMM_S8T_S8N_F32T(_ScaledBMM):
    """fp32 [B,M,N] = a * A[b] . B[b]^T (Q.K^T)."""

    @torch.no_grad()
    def forward(self, a, b):
        return bmm_s8t_s8n_f32t(a, b, self._alpha())

    @staticmethod
    def from_scale(a_scale, b_scale):
        return BMM_S8T_S8N_F32T._with_alpha(a_scale * b_scale)


class BMM_S8T_S8N_S32T(torch.nn.Module):
    """int32 [B,M,N] = A[b] . B[b]^T."""

    @torch.no_grad()
    def forward(self, a, b):
        return bmm_s8t_s8n_s32t(a, b)
