"""The reference's operator interface for the prefill hot path, backed by the sm_100a kernels.

Names, argument meaning, defaults and error behaviour follow xattn/src/Xattention.py
(`xattn_estimate` :13-299, `Xattention_prefill` :302-402), xattn/src/utils.py
(`find_blocks_chunked` :44-191) and the call-site contract of the third-party
`block_sparse_attn.block_sparse_attn_func` (xattn/src/Xattention.py:377-391).
"""
from __future__ import annotations

from typing import Optional, Union

import torch

from . import ops

Threshold = Union[float, torch.Tensor]


def _check_modes(softmax, select_mode, kdb):
    if not softmax:
        raise NotImplementedError("softmax=False is not used by Xattention_prefill and is not implemented")
    if select_mode not in ("inverse", ""):
        raise NotImplementedError(f"select_mode={select_mode!r}: only the antidiagonal ('inverse') mode is implemented")
    if kdb != 1:
        # the reference raises ValueError for kdb != 1 on its kernel path (Xattention.py:140-141)
        raise ValueError("use_triton and kdb cannot be used together")


def xattn_estimate(
    query_states: torch.Tensor,
    key_states: torch.Tensor,
    block_size,
    stride,
    norm=1,
    softmax=True,
    threshold=0.9,
    chunk_size=16384,
    select_mode="inverse",
    use_triton=True,
    causal=True,
    kdb: int = 1,
    keep_sink=False,
    keep_recent=False,
):
    """Returns (attn_sums, simple_masks), both [B, H, q_blocks_pad, k_blocks_pad]; attn_sums in the input
    dtype, simple_masks bool (Xattention.py:13-299).  `use_triton` is accepted and ignored: the CUDA path
    always runs; which of the reference's two estimate variants it reproduces is set by
    ops.set_estimate_semantics.  K/V with fewer heads than Q (GQA) are accepted."""
    _check_modes(softmax, select_mode, kdb)
    B, Hq, Lq, D = query_states.shape
    Lk = key_states.shape[2]
    assert Hq % key_states.shape[1] == 0
    g = ops.geometry(Lq, Lk, chunk_size, stride, block_size)
    sums = ops.estimate_block_sums(query_states, key_states, stride, block_size, chunk_size, float(norm),
                                   bool(causal))
    mask, _, _ = ops.select_blocks(sums, g["bpc"], g["block_offset"], threshold, bool(causal), True,
                                   bool(keep_sink), bool(keep_recent))
    return sums.to(query_states.dtype), mask


def find_blocks_chunked(input_tensor, current_index, threshold, num_to_choose, decoding: bool,
                        mode: str = "both", causal=True):
    """Prefill branch of the reference's selection for one chunk (utils.py:87-180).  input_tensor
    [B, H, chunk_blocks, k_blocks]; returns a bool mask of the same shape."""
    assert threshold is None or num_to_choose is None
    if threshold is None:
        raise NotImplementedError("block num chunk prefill not impleted")
    if mode == "prefill" and decoding:
        return torch.ones_like(input_tensor, dtype=torch.bool)
    if (mode == "decode" and not decoding) or decoding:
        raise NotImplementedError("only the prefill branch is implemented")
    R = input_tensor.shape[2]
    mask, _, _ = ops.select_blocks(input_tensor, R, int(current_index), threshold, bool(causal),
                                   diagonal_cleanup=False)
    return mask


def block_sparse_attn_func(q, k, v, cu_seqlens_q, cu_seqlens_k, head_mask_type, streaming_info,
                           base_blockmask, max_seqlen_q_, max_seqlen_k_, p_dropout=0.0, deterministic=False,
                           softmax_scale=None, is_causal=False, exact_streaming=False, return_attn_probs=False):
    """Single-sequence subset of block_sparse_attn.block_sparse_attn_func as Xattention_prefill uses it:
    q [Lq,H,D], k/v [Lk,Hkv,D], base_blockmask [1,H,qb,kb] bool, every head of mask type 1, no dropout."""
    if p_dropout != 0.0 or streaming_info is not None or return_attn_probs:
        raise NotImplementedError("dropout, streaming heads and attention probabilities are not implemented")
    Lq, H, D = q.shape
    Lk = k.shape[0]
    if cu_seqlens_q is not None and cu_seqlens_q.numel() != 2:
        raise NotImplementedError("one sequence per call")
    q4 = q.unsqueeze(0).transpose(1, 2)
    k4 = k.unsqueeze(0).transpose(1, 2)
    v4 = v.unsqueeze(0).transpose(1, 2)
    idx, cnt = ops.mask_to_lists(base_blockmask, Lq, Lk, bool(is_causal))
    out = ops.block_sparse_attention(q4, k4, v4, idx, cnt, bool(is_causal), softmax_scale)
    return out.transpose(1, 2).reshape(Lq, H, D)


def Xattention_prefill(
    query_states: torch.Tensor,
    key_states: torch.Tensor,
    value_states: torch.Tensor,
    stride,
    norm=1,
    threshold=0.8,
    block_size=128,
    use_triton=True,
    causal=True,
    kdb=1,
    chunk_size=None,
    keep_sink=False,
    keep_recent=False,
):
    """Estimate -> select -> block-sparse attention (Xattention.py:302-402).  Returns [B, H, Lq, D] in the
    input dtype (a transposed view of [B, Lq, H, D] storage, as in the reference)."""
    _check_modes(True, "inverse", kdb)
    B, Hq, Lq, D = query_states.shape
    Lk = key_states.shape[2]
    assert block_size == 128
    assert B == 1
    if chunk_size is None:
        chunk_size = ops.default_chunk_size(Lk)
    dev = query_states.device
    if key_states.device != dev:
        key_states = key_states.to(dev)
    if value_states.device != dev:
        value_states = value_states.to(dev)
    g = ops.geometry(Lq, Lk, chunk_size, stride, block_size)
    # un-padded causal keys under the torch branch: the sums outside a row's own chunk are zero and are not kept
    band = ops.band_applies(Lk, chunk_size, bool(causal))
    sums = ops.estimate_block_sums(query_states, key_states, stride, block_size, chunk_size, float(norm),
                                   bool(causal), band=band)
    _, idx, cnt = ops.select_blocks(sums, g["bpc"], g["block_offset"], threshold, bool(causal), True,
                                    bool(keep_sink), bool(keep_recent), list_shape=(Lq, Lk), want_mask=False,
                                    band_k_blocks=g["kb"] if band else None)
    return ops.block_sparse_attention(query_states, key_states, value_states, idx, cnt, bool(causal))
