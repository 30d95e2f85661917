"""Torch-facing operators over the C ABI: device memory, streams and argument checks only.

All compute happens in libxattn_b200.so.  Tensors must live on a CUDA device (sm_100); every op
launches on torch's current stream of that device and does not synchronise.
"""
from __future__ import annotations

import ctypes as C
import math
import os
from typing import Optional, Tuple, Union

import torch

from . import _lib

_DT = {torch.bfloat16: _lib.BF16, torch.float16: _lib.F16}
_SEM = {"torch": _lib.SEMANTICS_TORCH, "triton": _lib.SEMANTICS_TRITON}

# Which of the reference's two estimate code paths is reproduced.  The reference picks by GPU
# name (xattn/src/Xattention.py:57-63: Triton only when the name contains "100", i.e. A100/H100);
# on a B200 it therefore runs its torch branch, which is the default here.
_estimate_semantics = "torch"


def set_estimate_semantics(name: str) -> None:
    """'torch' (default; what the unmodified reference computes on a B200) or 'triton'
    (the reference's Triton kernels, which keep all earlier chunks visible to later query chunks)."""
    global _estimate_semantics
    if name not in _SEM:
        raise ValueError("semantics must be 'torch' or 'triton'")
    _estimate_semantics = name


def get_estimate_semantics() -> str:
    return _estimate_semantics


# ------------------------------------------------------------------------------ status word
_status_words = {}


def _status(device: torch.device) -> torch.Tensor:
    """One pinned, device-visible int32 per device that kernels write on a bounded-wait timeout."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    w = _status_words.get(key)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32).pin_memory()
        _status_words[key] = w
    return w


def check_device_status(device: Optional[torch.device] = None, synchronize: bool = True) -> None:
    """Raise if a kernel reported a timed-out wait.  With synchronize=False only work that has
    already finished is covered."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
    if synchronize:
        torch.cuda.synchronize(dev)
    w = _status(dev)
    code = int(w[0])
    if code != 0:
        w[0] = 0
        _lib.check(code, "device status")


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _require_cuda(*ts: torch.Tensor) -> None:
    for t in ts:
        if not t.is_cuda:
            raise _lib.XattnB200Error("xattn_b200 ops need CUDA tensors: there is no CPU path")


def _strides3(t: torch.Tensor) -> Tuple[int, int, int]:
    if t.stride(3) != 1:
        raise ValueError("head_dim must have unit stride")
    return t.stride(0), t.stride(1), t.stride(2)


def geometry(q_len: int, k_len: int, chunk_size: int, stride: int, block_size: int = 128) -> dict:
    out = (C.c_int * 8)()
    _lib.check(_lib.load().xattn_b200_estimate_geometry(q_len, k_len, chunk_size, stride, block_size, out),
               "estimate_geometry")
    keys = ("lq", "lk", "qb", "kb", "q_chunks", "k_chunks", "bpc", "block_offset")
    return dict(zip(keys, list(out)))


def default_chunk_size(k_len: int) -> int:
    return _lib.load().xattn_b200_default_chunk_size(k_len)


def _aligned16(x: torch.Tensor) -> torch.Tensor:
    ok = x.stride(3) == 1 and x.data_ptr() % 16 == 0 and all((s * x.element_size()) % 16 == 0 for s in x.stride()[:3])
    return x if ok else x.contiguous()


# ------------------------------------------------------------------------------ phase 1
def band_applies(k_len: int, chunk_size: int, causal: bool, semantics: Optional[str] = None) -> bool:
    """True when the estimate leaves every key block outside a row's own chunk at zero (the reference's torch
    branch on un-padded keys, xattn/src/Xattention.py:201), so that the sums can be kept as a chunk-wide band.
    (Block counts that are not multiples of four keep the dense layout.)"""
    return (bool(causal) and (semantics or _estimate_semantics) == "torch" and k_len % chunk_size == 0
            and (chunk_size // 128) % 4 == 0)


def estimate_block_sums(q: torch.Tensor, k: torch.Tensor, stride: int, block_size: int = 128,
                        chunk_size: int = 16384, norm: float = 1.0, causal: bool = True,
                        semantics: Optional[str] = None, band: bool = False) -> torch.Tensor:
    """fp32 attn_sums [B, Hq, q_blocks_pad, k_blocks_pad] of the antidiagonal estimate.

    band=True (see band_applies): only the key blocks of each row's own chunk are produced,
    [B, Hq, q_blocks_pad, chunk_size/block_size]; every other block has sum zero under the torch branch.

    q [B,Hq,Lq,D], k [B,Hkv,Lk,D] in bf16/fp16, or fp32 (split into three bf16 terms on the device so
    that the tensor-core product keeps fp32 accuracy)."""
    _require_cuda(q, k)
    lib = _lib.load()
    B, Hq, Lq, D = q.shape
    Hkv, Lk = k.shape[1], k.shape[2]
    sem = _SEM[semantics or _estimate_semantics]
    if band:
        if not band_applies(Lk, chunk_size, causal, semantics):
            raise ValueError("band layout needs the torch branch, causal, and k_len a multiple of chunk_size")
        sem = _lib.SEMANTICS_TORCH_BAND
    scale = 1.0 / math.sqrt(D) / stride / norm
    # lengths that are no multiple of the stride go to the library as they are (it stages the one ragged tile);
    # only the fp32 path rounds up, inside the split kernel that writes the widened rows anyway
    Lq_s, Lk_s = Lq, Lk
    g = geometry(Lq, Lk, chunk_size, stride, block_size)
    stream = _stream(q)
    if q.dtype == torch.float32:
        Lq_s, Lk_s = -(-Lq // stride) * stride, -(-Lk // stride) * stride
        q3 = torch.empty(B, Hq, Lq_s, 6 * D, dtype=torch.bfloat16, device=q.device)
        k3 = torch.empty(B, Hkv, Lk_s, 6 * D, dtype=torch.bfloat16, device=q.device)
        q = q if q.stride(3) == 1 else q.contiguous()
        k = k.float()
        k = k if k.stride(3) == 1 else k.contiguous()
        _lib.check(lib.xattn_b200_split_f32(q.data_ptr(), B, Hq, Lq_s, Lq, D, *_strides3(q), 0, q3.data_ptr(), stream),
                   "split_f32(q)")
        _lib.check(lib.xattn_b200_split_f32(k.data_ptr(), B, Hkv, Lk_s, Lk, D, *_strides3(k), 1, k3.data_ptr(), stream),
                   "split_f32(k)")
        q, k, D_eff, dt = q3, k3, 6 * D, _lib.BF16
    else:
        if q.dtype not in _DT or k.dtype != q.dtype:
            raise TypeError("q/k must both be bf16, fp16 or fp32")
        q, k, D_eff, dt = _aligned16(q), _aligned16(k), D, _DT[q.dtype]
        if D != 128 and (Lq % stride or Lk % stride):        # the staging tiles are sized for head_dim 128
            pad = lambda x: torch.nn.functional.pad(x, (0, 0, 0, (-x.shape[2]) % stride))  # noqa: E731
            q, k = pad(q), pad(k)
            Lq_s, Lk_s = q.shape[2], k.shape[2]
    ws_bytes = lib.xattn_b200_estimate_workspace_bytes_ex(B, Hq, Lq_s, Lk_s, stride, block_size, chunk_size,
                                                          int(causal), sem)
    if ws_bytes == 0:
        raise ValueError("unsupported estimate geometry (stride must be 4/8/16/32, block_size 128, "
                         "chunk_size a multiple of 128)")
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
    sums = torch.empty(B, Hq, g["qb"], g["bpc"] if band else g["kb"], dtype=torch.float32, device=q.device)
    st = _status(q.device)
    _lib.check(lib.xattn_b200_estimate(
        q.data_ptr(), k.data_ptr(), dt, B, Hq, Hkv, Lq_s, Lk_s, D_eff, *_strides3(q), *_strides3(k),
        stride, block_size, chunk_size, scale, int(causal), sem, sums.data_ptr(), ws.data_ptr(), ws_bytes,
        st.data_ptr(), stream), "estimate")
    return sums


# ------------------------------------------------------------------------------ phase 2
def select_blocks(sums: torch.Tensor, blocks_per_chunk: int, block_offset: int,
                  threshold: Union[float, torch.Tensor], causal: bool = True, diagonal_cleanup: bool = True,
                  keep_sink: bool = False, keep_recent: bool = False,
                  list_shape: Optional[Tuple[int, int]] = None, want_mask: bool = True,
                  band_k_blocks: Optional[int] = None):
    """Threshold selection over fp32 sums [B,H,qb,kb].  Returns (mask bool or None, block_idx, block_cnt);
    the lists are None unless list_shape=(q_len, k_len) is given.  band_k_blocks=kb: `sums` is the chunk band
    [B,H,qb,blocks_per_chunk] of estimate_block_sums(band=True) and kb the full number of key blocks."""
    _require_cuda(sums)
    lib = _lib.load()
    sums = sums.float().contiguous()
    B, H, QB, KB = sums.shape
    if band_k_blocks is not None:
        if KB != blocks_per_chunk:
            raise ValueError("band sums must have blocks_per_chunk columns")
        KB = int(band_k_blocks)
    thr_ptr, thr_val = 0, 0.0
    thr_t = None
    if isinstance(threshold, torch.Tensor):
        thr_t = threshold.detach().to(device=sums.device, dtype=torch.float32).reshape(-1).contiguous()
        if thr_t.numel() != H:
            raise ValueError("per-head threshold needs one entry per head")
        thr_ptr = thr_t.data_ptr()
    else:
        thr_val = float(threshold)
    mask = torch.empty(B, H, QB, KB, dtype=torch.uint8, device=sums.device) if want_mask else None
    idx = cnt = None
    lq = lk = lqb = lkb = 0
    if list_shape is not None:
        lq, lk = list_shape
        lqb, lkb = (lq + 127) // 128, (lk + 127) // 128
        idx = torch.empty(B, H, lqb, lkb, dtype=torch.int32, device=sums.device)
        cnt = torch.empty(B, H, lqb, dtype=torch.int32, device=sums.device)
    fn = lib.xattn_b200_select_band if band_k_blocks is not None else lib.xattn_b200_select
    _lib.check(fn(
        sums.data_ptr(), B, H, QB, KB, blocks_per_chunk, block_offset, int(causal), int(diagonal_cleanup),
        thr_val, thr_ptr, int(keep_sink), int(keep_recent),
        mask.data_ptr() if mask is not None else 0,
        idx.data_ptr() if idx is not None else 0, cnt.data_ptr() if cnt is not None else 0,
        lqb, lkb, lq, lk, _status(sums.device).data_ptr(), _stream(sums)), "select")
    return (mask.view(torch.bool) if mask is not None else None), idx, cnt


def apply_rotary_pos_emb_(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> None:
    """In-place rotary embedding of q [B,Hq,L,D] and k [B,Hkv,L,D] (any strides, unit stride on D) with
    cos/sin [B,L,D] (or [1,L,D]) of the same 16-bit dtype: bit-identical to the reference's
    `apply_rotary_pos_emb` (xattn/src/load_llama.py:41-65), one launch for both tensors."""
    _require_cuda(q, k, cos, sin)
    if q.dtype not in _DT or k.dtype != q.dtype or cos.dtype != q.dtype or sin.dtype != q.dtype:
        raise ValueError("apply_rotary_pos_emb_: q, k, cos, sin must share one 16-bit dtype (bf16 or fp16)")
    B, Hq, L, D = q.shape
    Hkv = k.shape[1]
    if k.shape != (B, Hkv, L, D):
        raise ValueError("apply_rotary_pos_emb_: q and k must share batch, length and head_dim")
    if cos.dim() != 3 or cos.shape[1:] != (L, D) or cos.shape[0] not in (1, B) or sin.shape != cos.shape:
        raise ValueError("apply_rotary_pos_emb_: cos/sin must be [batch or 1, len, head_dim]")
    if cos.stride(2) != 1 or sin.stride(2) != 1 or sin.stride() != cos.stride():
        cos, sin = cos.contiguous(), sin.contiguous()
    cs_b = cos.stride(0) if cos.shape[0] == B and B > 1 else 0
    lib = _lib.load()
    _lib.check(lib.xattn_b200_rope_qk(q.data_ptr(), k.data_ptr(), _DT[q.dtype], B, Hq, Hkv, L, D, *_strides3(q),
                                      *_strides3(k), cos.data_ptr(), sin.data_ptr(), cs_b, cos.stride(1),
                                      _stream(q)), "rope_qk")


def mask_to_lists(mask: torch.Tensor, q_len: int, k_len: int, causal: bool):
    _require_cuda(mask)
    lib = _lib.load()
    m = mask.contiguous()
    m = m.view(torch.uint8) if m.dtype == torch.bool else m.to(torch.uint8)
    B, H, MQ, MK = m.shape
    lqb, lkb = (q_len + 127) // 128, (k_len + 127) // 128
    idx = torch.empty(B, H, lqb, lkb, dtype=torch.int32, device=m.device)
    cnt = torch.empty(B, H, lqb, dtype=torch.int32, device=m.device)
    _lib.check(lib.xattn_b200_mask_to_lists(m.data_ptr(), B, H, MQ, MK, q_len, k_len, int(causal),
                                            idx.data_ptr(), cnt.data_ptr(), _stream(m)), "mask_to_lists")
    return idx, cnt


# ------------------------------------------------------------------------------ phase 3
# The split has fixed costs: the classify kernel (8 us) and the general kernel's pass over the rows the pair kernel
# leaves (a few items per SM, each a full latency chain), against 8-12 % of the call won when 95 % of the blocks
# qualify (Llama-3.1-8B at 128K tokens); and an attempt that the library declines costs 15-45 us (at 32K or 64K
# tokens it does decline: 66 % / 89 % qualify).  Measured on 1 / 2 / 4 / 8 kv heads of the 128K-token layer (4096 /
# 8192 / 16384 / 32768 items): general kernel alone 117 / 221 / 430 / 830 us, with the split 134 / 219 / 393 / 750.
# So the scratch memory is offered by default only for sequences of at least 96K tokens (PAIR_MIN_K_BLOCKS key
# blocks) and calls of at least PAIR_MIN_ITEMS (batch, query head, query block) items.
PAIR_MIN_K_BLOCKS = 768
PAIR_MIN_ITEMS = 12288
# Non-causal calls: sorting the items by list length is one launch of a few microseconds; with only a few items per
# SM there is nothing to balance.
ORDER_MIN_ITEMS = 16 * 148


def pair_split_share(percent: Optional[int] = None) -> int:
    """Share (per cent) of a call's listed blocks that must qualify for the pair kernel before the library splits
    the call between the two attention kernels (process-wide; 0: whenever anything qualifies, 101: never).
    Returns the previous value; without an argument only reads it."""
    return int(_lib.load().xattn_b200_block_sparse_attn_split_share(-1 if percent is None else int(percent)))


def block_sparse_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, block_idx: torch.Tensor,
                           block_cnt: torch.Tensor, causal: bool = True, scale: Optional[float] = None,
                           out: Optional[torch.Tensor] = None, use_workspace: Optional[bool] = None) -> torch.Tensor:
    """q [B,Hq,Lq,128], k/v [B,Hkv,Lk,128] (bf16/fp16; fp32 is computed in bf16) -> [B,Hq,Lq,128], returned
    as a transposed view of [B,Lq,Hq,128] storage, like the reference's output (Xattention.py:392-394).
    `out`, if given, is a [B,Hq,Lq,128] tensor of the compute dtype (any strides, unit stride on the last
    dimension, 16-byte aligned rows) that receives the result instead.  `use_workspace=True` hands the library
    scratch memory (xattn_b200_block_sparse_attn_ws).  Causal calls: it may then send the rows whose kv group shares a
    list of one or two blocks to the kernel that loads K/V once per group and treats both blocks in one softmax pass;
    the library takes that route only when those rows list at least `pair_split_share()` per cent of the blocks,
    which it finds out on the device, and a declined attempt costs 30-45 us, so by default (None) the memory is
    offered only for sequences of at least PAIR_MIN_K_BLOCKS key blocks and calls of at least PAIR_MIN_ITEMS items.  Non-causal calls: the work items are sorted
    by list length before they are dealt to the SMs (one small kernel); offered by default from ORDER_MIN_ITEMS
    items on.  False: the general kernel alone, items in their natural order."""
    _require_cuda(q, k, v, block_idx, block_cnt)
    lib = _lib.load()
    B, Hq, Lq, D = q.shape
    Hkv, Lk = k.shape[1], k.shape[2]
    if D != 128:
        raise ValueError("head_dim must be 128")
    in_dtype = q.dtype
    if in_dtype == torch.float32:
        q, k, v = q.bfloat16(), k.bfloat16(), v.bfloat16()
    if q.dtype not in _DT or k.dtype != q.dtype or v.dtype != q.dtype:
        raise TypeError("q/k/v must share one of bf16, fp16, fp32")
    q, k, v = _aligned16(q), _aligned16(k), _aligned16(v)
    scale = 1.0 / math.sqrt(D) if scale is None else float(scale)
    if out is None:
        out_view = torch.empty(B, Lq, Hq, D, dtype=q.dtype, device=q.device).transpose(1, 2)
    else:
        if tuple(out.shape) != (B, Hq, Lq, D) or out.dtype != q.dtype or out.stride(3) != 1 or not out.is_cuda:
            raise ValueError("out must be a CUDA tensor [B,Hq,Lq,D] of the compute dtype with unit inner stride")
        out_view = out
    lqb, lkb = (Lq + 127) // 128, (Lk + 127) // 128
    if tuple(block_idx.shape) != (B, Hq, lqb, lkb) or tuple(block_cnt.shape) != (B, Hq, lqb):
        raise ValueError("block lists have the wrong shape")
    if use_workspace is None:
        forced = os.environ.get("XATTN_B200_ATTN_WORKSPACE")         # "0" / "1": overrides the rule (for measurements)
        if forced in ("0", "1"):
            use_workspace = forced == "1"
        else:
            use_workspace = ((lkb >= PAIR_MIN_K_BLOCKS and B * Hq * lqb >= PAIR_MIN_ITEMS) if causal
                             else B * Hq * lqb >= ORDER_MIN_ITEMS)
    ws_bytes = lib.xattn_b200_block_sparse_attn_workspace_bytes(B, Hq, Hkv, Lq, Lk) if use_workspace else 0
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device) if ws_bytes else None
    _lib.check(lib.xattn_b200_block_sparse_attn_ws(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), _DT[q.dtype], B, Hq, Hkv, Lq, Lk, D,
        *_strides3(q), *_strides3(k), *_strides3(v), block_idx.contiguous().data_ptr(),
        block_cnt.contiguous().data_ptr(), int(causal), scale, out_view.data_ptr(),
        out_view.stride(0), out_view.stride(1), out_view.stride(2), ws.data_ptr() if ws is not None else 0, ws_bytes,
        _status(q.device).data_ptr(), _stream(q)), "block_sparse_attn")
    return out_view.to(in_dtype) if (in_dtype == torch.float32 and out is None) else out_view
