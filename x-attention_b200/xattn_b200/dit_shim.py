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


def _dense(q, k, v, out):
    B, H, Lq, _ = q.shape
    Lk = k.shape[2]
    qb, kb = (Lq + 127) // 128, (Lk + 127) // 128
    idx = torch.arange(kb, dtype=torch.int32, device=q.device).expand(B, H, qb, kb).contiguous()
    cnt = torch.full((B, H, qb), kb, dtype=torch.int32, device=q.device)
    ops.block_sparse_attention(q, k, v, idx, cnt, causal=False, out=out)


def _xattn(q, k, v, out, threshold, stride):
    """Non-causal Xattention_prefill (xattn/src/Xattention.py:302-402) writing into `out`."""
    Lq, Lk = q.shape[2], k.shape[2]
    chunk = ops.default_chunk_size(Lk)
    g = ops.geometry(Lq, Lk, chunk, stride, 128)
    sums = ops.estimate_block_sums(q, k, stride, 128, chunk, 1.0, False)
    _, idx, cnt = ops.select_blocks(sums, g["bpc"], g["block_offset"], threshold, False, True, list_shape=(Lq, Lk),
                                    want_mask=False)
    ops.block_sparse_attention(q, k, v, idx, cnt, causal=False, out=out)


def xattn_varlen_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens_q, cu_seqlens_kv,
                           threshold: float = 0.95, stride: int = 8) -> torch.Tensor:
    """q, k, v [1, heads, total, D] (16 bit, any strides with unit stride on D); cu_seqlens_* = [0, valid, total].
    Returns [1, heads, total, D] (a view of [1, total, heads, D] storage).  The two segments are read through
    strided views and written straight into their rows of the result: no copy of q, k, v or of the outputs,
    whatever the segment lengths (the estimate stages only the tile that holds a ragged last stride group)."""
    v0q, v1q = int(cu_seqlens_q[1]), int(cu_seqlens_q[2])
    v0k, v1k = int(cu_seqlens_kv[1]), int(cu_seqlens_kv[2])
    B, H, _, D = q.shape
    res = torch.empty(B, v1q, H, D, dtype=q.dtype, device=q.device).transpose(1, 2)
    q1, k1, v1 = q[:, :, :v0q], k[:, :, :v0k], v[:, :, :v0k]
    if threshold < 1:
        _xattn(q1, k1, v1, res[:, :, :v0q], threshold, stride)
    else:
        _dense(q1, k1, v1, res[:, :, :v0q])
    if v1q > v0q:
        _dense(q[:, :, v0q:v1q], k[:, :, v0k:v1k], v[:, :, v0k:v1k], res[:, :, v0q:v1q])
    return res
