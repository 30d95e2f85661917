"""Attention core of the reference's Llama integration, with native GQA.

The reference patches `LlamaAttention.forward` (xattn/src/load_llama.py:80-220).  Around the projections,
RoPE and the cache update (which stay the model's business) its core is: repeat K/V to the query heads
(:158-160), then prefill -> `Xattention_prefill` with the layer's per-head threshold row (:173-177), decode
(q_len == 1 against a longer cache) -> a dense single-query attention from a third-party package (:188-197).
`attention_core` is that core for callers that hold q/k/v after RoPE: K/V are NOT repeated (the kernels read
kv head h // (Hq/Hkv)), prefill goes to the sm_100a XAttention path, decode and the "full" metric run dense
through the same block-sparse attention kernel with an all-ones block list.

`llama_attention_forward` / `patch_llama_attention` are the whole patch for Hugging Face's `LlamaAttention`
(projections, in-place RoPE on the projection outputs, cache update, prefill or decode core, `o_proj` fed
without a transposed copy).

`FastPrefillConfig` mirrors the reference's (xattn/src/load_llama.py:224-262), including its default: with no
threshold given, the per-(layer, head) table the reference ships for Llama-3.1-8B and the chosen stride
(xattn/threshold/llama_threshold.py, stored as data/llama_thresholds.npz).
"""
from __future__ import annotations

import os
import types
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
            # xattn/src/load_llama.py:253-261: the profiled Llama-3.1-8B table of the stride
            threshold = default_threshold_table(stride)
        if isinstance(threshold, torch.Tensor):
            self.threshold = threshold.to(device=device, dtype=torch.float32)
        else:
            self.threshold = torch.ones((num_layers, num_heads), device=device) * float(threshold)


def default_threshold_table(stride: int) -> torch.Tensor:
    """[32, 32] per-(layer, head) thresholds the reference profiled for Llama-3.1-8B-Instruct at stride 4, 8 or 16."""
    import numpy as np
    if stride not in (4, 8, 16):
        raise ValueError("the reference ships threshold tables for stride 4, 8 and 16 only")
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "data", "llama_thresholds.npz"))
    return torch.from_numpy(z[f"fuse_{stride}"].copy())


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


def llama_attention_forward(self, hidden_states: torch.Tensor, position_embeddings=None, attention_mask=None,
                            past_key_values=None, past_key_value=None, cache_position=None, **kwargs):
    """Replacement for `LlamaAttention.forward` (what the reference's `forward_eval` does,
    xattn/src/load_llama.py:80-220), for modules that carry a `fastprefillconfig`.  Prefill (q_len == k_len, or a
    chunk against a longer cache) goes through XAttention with the layer's thresholds, a single new token against
    the cache through dense attention.  The attention mask is not consulted: like the reference's path, the call
    is causal over one un-padded sequence per batch entry.  Returns (attn_output, None)."""
    cfg = self.fastprefillconfig
    cache = past_key_values if past_key_values is not None else past_key_value
    B, L, _ = hidden_states.shape
    D = self.head_dim
    q_out, k_out, v_out = self.q_proj(hidden_states), self.k_proj(hidden_states), self.v_proj(hidden_states)
    Hq, Hkv = q_out.shape[-1] // D, k_out.shape[-1] // D
    q = q_out.view(B, L, Hq, D).transpose(1, 2)
    k = k_out.view(B, L, Hkv, D).transpose(1, 2)
    v = v_out.view(B, L, Hkv, D).transpose(1, 2)
    if position_embeddings is None:
        raise ValueError("position_embeddings=(cos, sin) is required")
    cos, sin = position_embeddings
    if q.dtype in (torch.bfloat16, torch.float16) and q.is_cuda:
        ops.apply_rotary_pos_emb_(q, k, cos.to(q.dtype), sin.to(q.dtype))      # in place, on the projection outputs
    else:
        raise TypeError("llama_attention_forward needs 16-bit CUDA activations")
    if cache is not None:
        try:
            k, v = cache.update(k, v, self.layer_idx, {"sin": sin, "cos": cos, "cache_position": cache_position})
        except TypeError:
            k, v = cache.update(k, v, self.layer_idx)
        if cache_position is not None and type(cache).__name__ == "StaticCache":       # load_llama.py:147-149
            end = min(int(cache_position[-1]) + 1, k.shape[2])
            k, v = k[:, :, :end], v[:, :, :end]
    out = attention_core(q, k, v, self.layer_idx, cfg)                 # [B, Hq, L, D] view of [B, L, Hq, D] storage
    out = out.transpose(1, 2)
    if not out.is_contiguous():
        out = out.contiguous()
    return self.o_proj(out.reshape(B, L, Hq * D)), None


def patch_llama_attention(model: torch.nn.Module, config: Optional[FastPrefillConfig] = None) -> int:
    """Give every `LlamaAttention`-like module of `model` (one that has q_proj, k_proj, v_proj, o_proj, head_dim and
    layer_idx) the forward above and `config` as its `fastprefillconfig` (the reference assigns both in
    xattn/src/load_llama.py:265-300).  Returns the number of modules patched."""
    cfg = config if config is not None else FastPrefillConfig()
    n = 0
    for m in model.modules():
        if all(hasattr(m, a) for a in ("q_proj", "k_proj", "v_proj", "o_proj", "head_dim", "layer_idx")):
            m.fastprefillconfig = cfg
            m.forward = types.MethodType(llama_attention_forward, m)
            n += 1
    return n
