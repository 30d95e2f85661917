"""Attention core of the reference's Llama integration, with native GQA.

The reference patches `LlamaAttention.forward` (xattn/src/load_llama.py:80-220).  Around the projections,
RoPE and the cache update (which stay the model's business) its core is: repeat K/V to the query heads
(:158-160), then prefill -> `Xattention_prefill` with the layer's per-head threshold row (:173-177), decode
(q_len == 1 against a longer cache) -> a dense single-query attention from a third-party package (:188-197).
`attention_core` is that core for callers that hold q/k/v after RoPE: K/V are NOT repeated (the kernels read
kv head h // (Hq/Hkv)), prefill goes to the sm_100a XAttention path, decode and the "full" metric run dense
through the same block-sparse attention kernel with an all-ones block list.

`FastPrefillConfig` mirrors the reference's (xattn/src/load_llama.py:224-262).  The reference ships
per-(layer, head) threshold tables for Llama-3.1-8B (xattn/threshold/llama_threshold.py); they are model data,
not part of this package: pass your table as `threshold` ([layers, heads] tensor) or a scalar.
"""
from __future__ import annotations

from typing import Optional, Union

import torch

from . import ops
from .api import Xattention_prefill


class FastPrefillConfig(dict):
    def __init__(self, threshold: Union[None, float, torch.Tensor] = None, print_detail: bool = False, stride=16,
                 metric: str = "xattn", num_layers: int = 32, num_heads: int = 32, device="cuda"):
        super().__init__()
        if metric not in ("xattn", "full"):
            raise NotImplementedError(f"metric {metric!r}: only 'xattn' and 'full' are implemented")
        self.print_detail = print_detail
        self.metric = metric
        self.stride = stride
        if threshold is None:
            threshold = 0.9
        if isinstance(threshold, torch.Tensor):
            self.threshold = threshold.to(device=device, dtype=torch.float32)
        else:
            self.threshold = torch.ones((num_layers, num_heads), device=device) * float(threshold)


def _dense_lists(batch, heads, q_len, k_len, device):
    qb, kb = (q_len + 127) // 128, (k_len + 127) // 128
    idx = torch.arange(kb, dtype=torch.int32, device=device).expand(batch, heads, qb, kb).contiguous()
    cnt = torch.full((batch, heads, qb), kb, dtype=torch.int32, device=device)
    return idx, cnt


def attention_core(query_states: torch.Tensor, key_states: torch.Tensor, value_states: torch.Tensor,
                   layer_idx: int, config: FastPrefillConfig) -> torch.Tensor:
    """q [B,Hq,q_len,D], k/v [B,Hkv,k_len,D] (after RoPE and the cache update) -> [B,Hq,q_len,D]."""
    B, Hq, q_len, D = query_states.shape
    k_len = key_states.shape[2]
    decoding = q_len != k_len and q_len == 1                       # load_llama.py:156
    if not decoding and config.metric == "xattn":
        thr = config.threshold[layer_idx] if config.threshold.dim() == 2 else config.threshold
        return Xattention_prefill(query_states, key_states, value_states, config.stride, norm=1, threshold=thr,
                                  use_triton=True)
    # decode, or dense prefill: every key block that a row may see (token-level causal inside the kernel)
    idx, cnt = _dense_lists(B, Hq, q_len, k_len, query_states.device)
    return ops.block_sparse_attention(query_states, key_states, value_states, idx, cnt, causal=True)


def rope_and_attend(q_proj_out: torch.Tensor, k_proj_out: torch.Tensor, v_proj_out: torch.Tensor,
                    cos: torch.Tensor, sin: torch.Tensor, num_heads: int, num_key_value_heads: int,
                    layer_idx: int, config: FastPrefillConfig) -> torch.Tensor:
    """The steps either side of the attention core, without their copies (prefill, no earlier cache).

    The reference reshapes the projection outputs [B, L, H*D] to [B, H, L, D] views, applies the rotary embedding
    out of place (three full-size temporaries per tensor, xattn/src/load_llama.py:124-142), repeats K/V, and
    after attention makes `attn_output.transpose(1, 2).contiguous()` before `o_proj` (:211-213).  Here the rotary
    embedding is one in-place kernel on the projection outputs, the estimate and attention kernels read the
    [B, H, L, D] views through their strides, and the attention output is written as [B, L, H, D], so the
    returned [B, L, H*D] tensor is what `o_proj` consumes: no transposed copy on either side.
    `q_proj_out` and `k_proj_out` are overwritten with their rotated values (the key cache wants those)."""
    B, L, _ = q_proj_out.shape
    D = q_proj_out.shape[2] // num_heads
    q = q_proj_out.view(B, L, num_heads, D).transpose(1, 2)
    k = k_proj_out.view(B, L, num_key_value_heads, D).transpose(1, 2)
    v = v_proj_out.view(B, L, num_key_value_heads, D).transpose(1, 2)
    ops.apply_rotary_pos_emb_(q, k, cos, sin)
    out = attention_core(q, k, v, layer_idx, config)               # [B, Hq, L, D] view of [B, L, Hq, D] storage
    out_blhd = out.transpose(1, 2)
    if not out_blhd.is_contiguous():                               # never for this package's kernels
        out_blhd = out_blhd.contiguous()
    return out_blhd.reshape(B, L, num_heads * D)
