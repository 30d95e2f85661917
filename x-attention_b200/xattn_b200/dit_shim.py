"""Full (non-causal) self-attention of a video-diffusion block in the reference's "xattn" mode.

Reference: eval/HunyuanVideo/hyvideo/modules/attenion.py:132-166.  The sequence of a sample is
[valid image+text tokens | padded text tail]; the two segments attend only within themselves
(`cu_seqlens = [0, valid, total]`).  The valid segment goes through XAttention (non-causal; dense attention
instead when threshold >= 1, which the model uses during its warm-up steps, models.py:211), the tail is dense.
Both dense cases run through the block-sparse kernel with an all-ones block list, so no third-party attention
package is involved.
"""
from __future__ import annotations

import torch

from . import ops
from .api import Xattention_prefill


def _dense(q, k, v):
    B, H, Lq, _ = q.shape
    Lk = k.shape[2]
    qb, kb = (Lq + 127) // 128, (Lk + 127) // 128
    idx = torch.arange(kb, dtype=torch.int32, device=q.device).expand(B, H, qb, kb).contiguous()
    cnt = torch.full((B, H, qb), kb, dtype=torch.int32, device=q.device)
    return ops.block_sparse_attention(q.contiguous(), k.contiguous(), v.contiguous(), idx, cnt, causal=False)


def xattn_varlen_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens_q, cu_seqlens_kv,
                           threshold: float = 0.95, stride: int = 8) -> torch.Tensor:
    """q, k, v [1, heads, total, D]; cu_seqlens_* = [0, valid, total].  Returns [1, heads, total, D]."""
    v0q, v1q = int(cu_seqlens_q[1]), int(cu_seqlens_q[2])
    v0k, v1k = int(cu_seqlens_kv[1]), int(cu_seqlens_kv[2])
    q1, k1, v1 = q[:, :, :v0q], k[:, :, :v0k], v[:, :, :v0k]
    if threshold < 1:
        x1 = Xattention_prefill(q1.contiguous(), k1.contiguous(), v1.contiguous(), stride=stride, norm=1,
                                threshold=threshold, causal=False, kdb=1)
    else:
        x1 = _dense(q1, k1, v1)
    parts = [x1]
    if v1q > v0q:
        parts.append(_dense(q[:, :, v0q:v1q], k[:, :, v0k:v1k], v[:, :, v0k:v1k]))
    return torch.cat(parts, dim=2)
