"""CPU oracle for the XAttention prefill hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, on the CPU in fp32/fp64 torch ops, what the reference project
(mit-han-lab/x-attention) computes for

  * the antidiagonal block-importance estimate      (xattn/src/Xattention.py:13-299,
                                                     torch branch :71-136, :174-252),
  * the threshold block selection                   (xattn/src/utils.py:44-191,
                                                     prefill branch :87-172),
  * the mask post-processing of ``xattn_estimate``  (xattn/src/Xattention.py:272-297),
  * block-sparse attention under a block mask       (call site xattn/src/Xattention.py:377-391;
                                                     the arithmetic lives in the third-party
                                                     package ``block_sparse_attn==0.0.1``,
                                                     requirements.txt:29, whose source is not
                                                     part of the reference tree; the in-tree
                                                     statement of the same math for the causal
                                                     case is xattn/src/Flexprefill.py:12-44).

  * the rotary embedding of the Llama patch          (xattn/src/load_llama.py:34-65; pinned against
                                                     the reference function, tests/golden/rope.npz).

Nothing in the shipped package may import this module: only ``tests/``, the smoke check and
the CPU-baseline leg of ``bench.py`` do, and only as the checker or as the timed baseline.

Parity pinning
--------------
* estimate + selection: pinned against the *unmodified reference code* imported on the CPU
  (``tests/golden/make_golden.py`` generates ``tests/golden/*.npz`` from the reference;
  ``tests/test_oracle_golden.py`` replays them through this module).
* block-sparse attention, causal: pinned against the reference's own in-tree statement of the operation,
  ``torch_block_wise_attention`` (xattn/src/Flexprefill.py:12-44), imported on the CPU and run in fp32 on
  seeded cases (``tests/golden/attention_blockwise.npz``; replayed by ``tests/test_oracle_golden.py``).
  Non-causal masks and queries shorter than the keys have no reference-held statement (the production
  kernel lives in ``block_sparse_attn==0.0.1``, whose source is not part of the reference tree): there the
  definition is dense fp32 softmax(QK^T/sqrt(D)) V restricted to kept 128x128 blocks, query end aligned to
  key end, checked against torch's scaled_dot_product_attention on all-ones masks.

Two estimate semantics are restated (they differ only for causal, un-padded K, see
``estimate_block_sums``):

  "torch"  : the reference's torch branch, which is what the unmodified reference executes
             on any GPU whose name lacks "100" (Xattention.py:57-63) -- a B200 included.
  "triton" : the reference's Triton kernels (xattn/src/kernels.py:5-156, :197-235).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple, Union

import torch

Threshold = Union[float, torch.Tensor]


# ----------------------------------------------------------------------------------------
# shapes
# ----------------------------------------------------------------------------------------
def default_chunk_size(k_len: int) -> int:
    """Default estimate chunk of ``Xattention_prefill`` (Xattention.py:322-331)."""
    p = 1 << (k_len - 1).bit_length()
    return int(max(min(max(2048, p), 128 * 1024 * 2048 // p), 2048))


def padded_geometry(q_len: int, k_len: int, chunk_size: int, block_size: int, stride: int):
    """Padded lengths and counts (Xattention.py:33-40, :65-70)."""
    k_pad = (-k_len) % chunk_size
    q_pad = (-q_len) % chunk_size
    g = dict(
        q_pad=q_pad, k_pad=k_pad, lq=q_len + q_pad, lk=k_len + k_pad,
        q_chunks=(q_len + q_pad) // chunk_size, k_chunks=(k_len + k_pad) // chunk_size,
        qb=(q_len + q_pad) // block_size, kb=(k_len + k_pad) // block_size,
        rcs=chunk_size // stride, rbs=block_size // stride,
        # reshaped pad counts use floor division in the reference (:67, :69)
        k_rpad=k_pad // stride, q_rpad=q_pad // stride,
    )
    g["bpc"] = g["rcs"] // g["rbs"]
    if g["k_chunks"] < g["q_chunks"]:
        raise AssertionError("k_chunk_num >= q_chunk_num is required (Xattention.py:39)")
    return g


# ----------------------------------------------------------------------------------------
# phase 1: estimate
# ----------------------------------------------------------------------------------------
def reshape_antidiagonal(q: torch.Tensor, k: torch.Tensor, stride: int):
    """Stride-reshaped operands of the "inverse" mode (Xattention.py:84-94).

    Qr[..., i, t*D + d] = Q[..., S*i + S-1-t, d]   and   Kr[..., j, t*D + d] = K[..., S*j + t, d]
    so that Qr @ Kr^T sums, per S x S cell of QK^T, its antidiagonal.
    """
    B, H, Lq, D = q.shape
    Lk = k.shape[2]
    S = stride
    qr = q.reshape(B, H, Lq // S, S, D).flip(3).reshape(B, H, Lq // S, S * D)
    kr = k.reshape(B, H, Lk // S, S, D).reshape(B, H, Lk // S, S * D)
    return qr, kr


def estimate_block_sums(
    q: torch.Tensor,
    k: torch.Tensor,
    block_size: int = 128,
    stride: int = 16,
    norm: float = 1.0,
    chunk_size: int = 16384,
    causal: bool = True,
    semantics: str = "torch",
) -> torch.Tensor:
    """fp32 block sums of the row-softmaxed antidiagonal scores, padded block counts.

    Follows Xattention.py:174-252 ("torch") or kernels.py:5-156 ("triton").  Returns
    ``[B, H, qb_pad, kb_pad]`` float32.
    """
    assert semantics in ("torch", "triton")
    B, H, Lq, D = q.shape
    Lk = k.shape[2]
    S = stride
    g = padded_geometry(Lq, Lk, chunk_size, block_size, S)
    q32 = torch.nn.functional.pad(q.float(), (0, 0, 0, g["q_pad"]))
    k32 = torch.nn.functional.pad(k.float(), (0, 0, 0, g["k_pad"]))
    qr, kr = reshape_antidiagonal(q32, k32, S)
    rcs, rbs, bpc = g["rcs"], g["rbs"], g["bpc"]
    n_cols = g["lk"] // S
    n_rows = g["lq"] // S
    off_chunks = g["k_chunks"] - g["q_chunks"]
    rows_valid = n_rows - g["q_rpad"]          # rows past this are zeroed (:237-238)
    cols_valid = n_cols - g["k_rpad"]          # causal only: pad columns are -inf (:201)
    col = torch.arange(n_cols)
    out = []
    for c in range(g["q_chunks"]):
        w = torch.matmul(qr[:, :, c * rcs:(c + 1) * rcs], kr.transpose(2, 3))
        w = w / math.sqrt(D) / S / norm
        if causal:
            chunk_start = (c + off_chunks) * rcs
            i_local = torch.arange(rcs)[:, None]
            hi = chunk_start + i_local                        # last visible column, per row
            if semantics == "torch":
                # Xattention.py:201 -- with k_rpad == 0 the slice [-0:] is the whole axis, so
                # every column left of the chunk is -inf as well.
                lo = chunk_start if g["k_rpad"] == 0 else 0
                visible = (col[None, :] >= lo) & (col[None, :] <= hi) & (col[None, :] < cols_valid)
            else:
                # kernels.py:56 -- global reshaped position of the row vs the column, nothing else.
                visible = col[None, :] <= hi
            w = w.masked_fill(~visible, float("-inf"))
        p = torch.softmax(w, dim=-1, dtype=torch.float32)
        p = torch.nan_to_num(p, nan=0.0)                      # rows with no visible column
        row_global = c * rcs + torch.arange(rcs)
        p = p * (row_global < rows_valid).float()[:, None]
        out.append(p.view(B, H, bpc, rbs, n_cols // rbs, rbs).sum(-1).sum(-2))
    return torch.cat(out, dim=-2)


# ----------------------------------------------------------------------------------------
# phase 2: selection
# ----------------------------------------------------------------------------------------
def _threshold_column(threshold: Threshold, H: int) -> torch.Tensor:
    if isinstance(threshold, torch.Tensor):
        t = threshold.detach().cpu().to(torch.float64).reshape(-1)
        assert t.numel() == H, "per-head threshold must have one entry per head"
        return t.view(1, H, 1, 1)
    return torch.full((1, H, 1, 1), float(threshold), dtype=torch.float64)


def select_blocks_chunk(
    x: torch.Tensor, current_index: int, threshold: Threshold, causal: bool = True
) -> torch.Tensor:
    """Block selection for one query chunk (utils.py:87-172 + :176-180), restated.

    Per row r with block scores x[0..N) in fp64 and ``req = sum(x) * threshold``:

    * causal: the diagonal block d = current_index + r is forced; block 0 is forced too unless
      ``current_index == 0`` (utils.py:100-106: the eye assignment over columns
      [current_index, current_index+R) overwrites the column-0 flag).  The other blocks are
      ranked by score, descending; the i-th of them (1-based) is taken iff c_i < req with
      c_i = forced + (sum of the first i-1-lag ranked scores), c_i = 0 when i-lag <= 0, and
      lag = 1 when only one block is forced (the bookkeeping at utils.py:115-139 always
      reserves two leading slots).
    * non-causal: nothing forced, c_i = sum of the first i-1 ranked scores.
    * block 0 is set whenever at least one rank position is *not* taken (utils.py:142, :164
      redirect those positions to index 0 before the scatter).
    * causal: columns >= current_index + R are cleared (utils.py:176-180).

    Ties are ranked lowest block index first (the reference's sort is unstable).
    """
    B, H, R, N = x.shape
    x64 = x.detach().cpu().to(torch.float64)
    req = x64.sum(-1, keepdim=True) * _threshold_column(threshold, H)
    forced = torch.zeros(R, N, dtype=torch.bool)
    if causal:
        rows = torch.arange(R)
        if current_index != 0:
            forced[:, 0] = True
        forced[rows, current_index + rows] = True
    n_forced = int(forced[0].sum()) if causal else 0
    lag = 1 if n_forced == 1 else 0
    fsum = (x64 * forced).sum(-1, keepdim=True)
    ranked = x64.masked_fill(forced.expand_as(x64), -1.0)      # forced blocks rank last
    v, order = torch.sort(ranked, dim=-1, descending=True, stable=True)
    n_others = N - n_forced
    v = v[..., :n_others].clamp_min(0.0)
    order = order[..., :n_others]
    prefix = torch.cat([torch.zeros_like(v[..., :1]), v.cumsum(-1)], dim=-1)   # prefix[m] = first m
    i = torch.arange(1, n_others + 1)
    take_from = (i - lag - 1).clamp_min(0)
    c = fsum + prefix[..., take_from]
    c = torch.where((i - lag) <= 0, torch.zeros_like(c), c)
    taken = c < req
    mask = forced.expand(B, H, R, N).clone()
    mask.scatter_(-1, order, mask.gather(-1, order) | taken)
    # rank positions of the reference: n_forced leading slots (taken iff 0 < req) + the others
    all_taken = taken.all(-1) & (req[..., 0] > 0) if n_others > 0 else (req[..., 0] > 0)
    mask[..., 0] |= ~all_taken
    if causal:
        mask[..., current_index + R:] = False
    return mask


def finish_masks(masks: torch.Tensor, qb: int, causal: bool, keep_sink: bool, keep_recent: bool):
    """Post-processing after the chunks are concatenated (Xattention.py:275-297)."""
    masks = masks.clone()
    tri = torch.tril(torch.ones(qb, qb, dtype=torch.bool))
    if causal:
        masks[:, :, -qb:, -qb:] &= tri
    if keep_sink:
        masks[:, :, 0, :] = True            # query-block ROW 0, as the reference writes it (:287)
    if keep_recent:
        masks[:, :, -qb:, -qb:] |= torch.eye(qb, dtype=torch.bool)
    return masks


def xattn_estimate_oracle(
    q: torch.Tensor,
    k: torch.Tensor,
    block_size: int = 128,
    stride: int = 16,
    norm: float = 1.0,
    threshold: Threshold = 0.9,
    chunk_size: int = 16384,
    causal: bool = True,
    keep_sink: bool = False,
    keep_recent: bool = False,
    semantics: str = "torch",
) -> Tuple[torch.Tensor, torch.Tensor]:
    """(attn_sums fp32, simple_masks bool), both ``[B, H, qb_pad, kb_pad]`` (Xattention.py:13-299)."""
    sums = estimate_block_sums(q, k, block_size, stride, norm, chunk_size, causal, semantics)
    g = padded_geometry(q.shape[2], k.shape[2], chunk_size, block_size, stride)
    bpc = g["bpc"]
    parts = []
    for c in range(g["q_chunks"]):
        cur = g["kb"] - g["qb"] + c * bpc
        parts.append(select_blocks_chunk(sums[:, :, c * bpc:(c + 1) * bpc], cur, threshold, causal))
    masks = finish_masks(torch.cat(parts, dim=-2), g["qb"], causal, keep_sink, keep_recent)
    return sums, masks


# ----------------------------------------------------------------------------------------
# margin exemption (which blocks may legitimately differ from the oracle mask)
# ----------------------------------------------------------------------------------------
def margin_exempt_chunk(
    x: torch.Tensor, current_index: int, threshold: Threshold, causal: bool, rel: float = 1e-4
) -> torch.Tensor:
    """Blocks whose take/skip decision sits within ``rel`` of the cut, for one chunk.

    A block is exempt iff its decision value c_i satisfies |c_i - req| < rel * max(req, tiny),
    or its score is within ``rel`` (relative) of the score of a ranked neighbour whose decision
    is the opposite one (a tie across the cut).  Block 0 is exempt when the "anything left
    un-taken" rule that sets it (utils.py:142) hinges on such a block.
    """
    B, H, R, N = x.shape
    x64 = x.detach().cpu().to(torch.float64)
    req = x64.sum(-1, keepdim=True) * _threshold_column(threshold, H)
    forced = torch.zeros(R, N, dtype=torch.bool)
    if causal:
        rows = torch.arange(R)
        if current_index != 0:
            forced[:, 0] = True
        forced[rows, current_index + rows] = True
    n_forced = int(forced[0].sum()) if causal else 0
    lag = 1 if n_forced == 1 else 0
    fsum = (x64 * forced).sum(-1, keepdim=True)
    ranked = x64.masked_fill(forced.expand_as(x64), -1.0)
    v, order = torch.sort(ranked, dim=-1, descending=True, stable=True)
    n_others = N - n_forced
    v = v[..., :n_others].clamp_min(0.0)
    order = order[..., :n_others]
    prefix = torch.cat([torch.zeros_like(v[..., :1]), v.cumsum(-1)], dim=-1)
    i = torch.arange(1, n_others + 1)
    c = fsum + prefix[..., (i - lag - 1).clamp_min(0)]
    c = torch.where((i - lag) <= 0, torch.zeros_like(c), c)
    taken = c < req
    tol = rel * req.clamp_min(1e-300)
    near = (c - req).abs() < tol
    # ties across the cut: neighbour in rank with (almost) the same score and the other decision
    same_next = torch.zeros_like(near)
    same_prev = torch.zeros_like(near)
    if n_others > 1:
        close = (v[..., :-1] - v[..., 1:]).abs() <= rel * v[..., :-1].abs().clamp_min(1e-30)
        flips = taken[..., :-1] != taken[..., 1:]
        same_next[..., :-1] = close & flips
        same_prev[..., 1:] = close & flips
    # propagate along runs of equal scores that contain the cut
    ex_rank = near | same_next | same_prev
    if n_others > 1:
        close_full = torch.zeros_like(near)
        close_full[..., 1:] = (v[..., :-1] - v[..., 1:]).abs() <= rel * v[..., :-1].abs().clamp_min(1e-30)
        for _ in range(8):   # a few sweeps spread the flag along short tie runs
            grow = ex_rank.clone()
            grow[..., 1:] |= ex_rank[..., :-1] & close_full[..., 1:]
            grow[..., :-1] |= ex_rank[..., 1:] & close_full[..., 1:]
            if torch.equal(grow, ex_rank):
                break
            ex_rank = grow
    exempt = torch.zeros(B, H, R, N, dtype=torch.bool)
    exempt.scatter_(-1, order, ex_rank)
    exempt &= ~forced
    # block 0 via the redirect rule: hinges on the last ranked block's decision
    if n_others > 0:
        exempt[..., 0] |= ex_rank[..., -1] & ~forced[:, 0]
    return exempt


def margin_exempt(
    sums: torch.Tensor, q_len: int, k_len: int, block_size: int, stride: int, chunk_size: int,
    threshold: Threshold, causal: bool, rel: float = 1e-4,
) -> torch.Tensor:
    g = padded_geometry(q_len, k_len, chunk_size, block_size, stride)
    bpc = g["bpc"]
    parts = []
    for c in range(g["q_chunks"]):
        cur = g["kb"] - g["qb"] + c * bpc
        parts.append(margin_exempt_chunk(sums[:, :, c * bpc:(c + 1) * bpc], cur, threshold, causal, rel))
    return torch.cat(parts, dim=-2)


# ----------------------------------------------------------------------------------------
# phase 3: block-sparse attention
# ----------------------------------------------------------------------------------------
def block_sparse_attention_oracle(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, block_mask: torch.Tensor,
    causal: bool = True, block_size: int = 128, scale: Optional[float] = None,
) -> torch.Tensor:
    """fp32 attention restricted to kept blocks (call-site contract, Xattention.py:377-391).

    q ``[B,Hq,Lq,D]``; k, v ``[B,Hkv,Lk,D]`` with Hq a multiple of Hkv; ``block_mask``
    ``[B,Hq,>=ceil(Lq/bs),>=ceil(Lk/bs)]`` bool.  Causal is token-level with the query end
    aligned to the key end.  Rows without any visible key give zeros.
    """
    B, Hq, Lq, D = q.shape
    Hkv, Lk = k.shape[1], k.shape[2]
    rep = Hq // Hkv
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    qb = (Lq + block_size - 1) // block_size
    kb = (Lk + block_size - 1) // block_size
    out = torch.zeros(B, Hq, Lq, D, dtype=torch.float32)
    kpos = torch.arange(Lk)
    for b in range(B):
        for h in range(Hq):
            kk = k[b, h // rep].float()
            vv = v[b, h // rep].float()
            for r in range(qb):
                r0, r1 = r * block_size, min((r + 1) * block_size, Lq)
                keep = block_mask[b, h, r, :kb].cpu().repeat_interleave(block_size)[:Lk]
                vis = keep[None, :].expand(r1 - r0, Lk)
                if causal:
                    qpos = torch.arange(r0, r1) + (Lk - Lq)
                    vis = vis & (kpos[None, :] <= qpos[:, None])
                s = (q[b, h, r0:r1].float() @ kk.T) * scale
                s = s.masked_fill(~vis, float("-inf"))
                p = torch.nan_to_num(torch.softmax(s, dim=-1), nan=0.0)
                out[b, h, r0:r1] = p @ vv
    return out


def apply_rotary_pos_emb_oracle(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
    """Rotary embedding as the reference's Llama patch applies it (xattn/src/load_llama.py:34-65): per head
    row x of width D, x' = x*cos + rot(x)*sin with rot(x)[i] = -x[i + D/2] for i < D/2, x[i - D/2] otherwise.
    The reference evaluates this as 16-bit tensor operations; each of them computes in fp32 and rounds to the
    storage type, which is restated here explicitly.  q [B,Hq,L,D], k [B,Hkv,L,D], cos/sin [B,L,D]."""
    def one(x):
        dt = x.dtype
        half = x.shape[-1] // 2
        xf = x.float()
        c, s = cos.float()[:, None], sin.float()[:, None]
        rot = torch.empty_like(xf)
        rot[..., :half] = -xf[..., half:]
        rot[..., half:] = xf[..., :half]
        a = (xf * c).to(dt).float()
        b = (rot * s).to(dt).float()
        return (a + b).to(dt)
    return one(q), one(k)
