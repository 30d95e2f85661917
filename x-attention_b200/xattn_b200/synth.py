"""Seeded synthetic Q/K/V generators with the shapes and value structure of the workloads the
reference is evaluated on (long-context Llama prefill, Qwen2-VL video prefill, HunyuanVideo
DiT self-attention).  They stand in for real model activations, which are not available
offline.  Everything is generated in fp32 from a ``torch.Generator`` so that a seed fully determines the
tensors: on the CPU by default (what the tests and fixtures use), or directly on a CUDA device
(``make_inputs(..., device=...)``; a different random stream, for benchmarks that need the long
sequences quickly).

Layout of every returned tensor: ``[1, H, L, D]`` contiguous.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import torch


def _ar1(noise: torch.Tensor, rho: float, dim: int) -> torch.Tensor:
    """Unit-variance stationary AR(1) filter along ``dim``: x_0 = e_0,
    x_t = rho x_{t-1} + sqrt(1-rho^2) e_t.  Computed blockwise in fp64 with the closed form
    x_{t0+u} = rho^u (x_{t0} + sum_{v<=u} rho^{-v} c e_{t0+v})."""
    x = noise.transpose(dim, -1).to(torch.float64)
    dev = x.device
    T = x.shape[-1]
    c = math.sqrt(1.0 - rho * rho)
    out = torch.empty_like(x)
    blk = 256
    prev = None
    for t0 in range(0, T, blk):
        e = x[..., t0:t0 + blk].clone()
        n = e.shape[-1]
        if prev is None:
            u = torch.arange(n, dtype=torch.float64, device=dev)
            e[..., 1:] *= c
            w = e * rho ** (-u)
            out[..., t0:t0 + n] = w.cumsum(-1) * rho ** u
        else:
            u = torch.arange(1, n + 1, dtype=torch.float64, device=dev)
            w = (e * c) * rho ** (-u)
            out[..., t0:t0 + n] = (prev[..., None] + w.cumsum(-1)) * rho ** u
        prev = out[..., t0 + n - 1]
    return out.transpose(dim, -1).to(torch.float32)


def _unit(gen: torch.Generator, *shape) -> torch.Tensor:
    u = torch.randn(*shape, generator=gen, device=gen.device)
    return u / u.norm(dim=-1, keepdim=True)


@dataclass
class Workload:
    name: str
    hq: int
    hkv: int
    seq_len: int
    stride: int
    threshold: float
    causal: bool
    chunk_size: Optional[int]
    dtype: torch.dtype
    head_dim: int = 128
    block_size: int = 128


def llama_like(gen: torch.Generator, hq: int, hkv: int, L: int, D: int = 128,
               rho: float = 0.99, local_std: float = 1.5, sink_tokens: int = 128,
               q_dir: float = 1.0, sink_dir: float = 3.0
               ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Long-context decoder activations: per kv head a unit direction u and an AR(1) local
    component s_t shared by q and k at position t (and by the q heads of the group);
    q_t = N(0,I) + s_t + q_dir u;  k_t = N(0,I) + s_t (+ sink_dir u for t < sink_tokens);
    v_t = N(0,I).  Returns q [1,hq,L,D], k, v [1,hkv,L,D]."""
    rep = hq // hkv
    u = _unit(gen, hkv, 1, D)
    s = _ar1(torch.randn(hkv, L, D, generator=gen, device=gen.device), rho, dim=1) * local_std
    k = torch.randn(hkv, L, D, generator=gen, device=gen.device) + s
    k[:, :sink_tokens] += sink_dir * u
    q = torch.randn(hq, L, D, generator=gen, device=gen.device)
    q += s.repeat_interleave(rep, dim=0)
    q += (q_dir * u).repeat_interleave(rep, dim=0)
    v = torch.randn(hkv, L, D, generator=gen, device=gen.device)
    return q[None], k[None], v[None]


def video_like(gen: torch.Generator, hq: int, hkv: int, text_pre: int = 512, frames: int = 240,
               frame_tokens: int = 256, text_post: int = 256, D: int = 128,
               rho: float = 0.95, frame_std: float = 0.5, sink_tokens: int = 128,
               sink_dir: float = 3.0, q_dir: float = 1.0):
    """Video-LLM prefill: text, then ``frames`` x ``frame_tokens`` visual tokens, then text.
    Visual tokens of frame j carry a frame mean f_j (AR(1) across frames) on q and k; text
    tokens are N(0,I) with the attention-sink rule on the first ``sink_tokens`` keys."""
    rep = hq // hkv
    L = text_pre + frames * frame_tokens + text_post
    u = _unit(gen, hkv, 1, D)
    f = _ar1(torch.randn(hkv, frames, D, generator=gen, device=gen.device), rho, dim=1) * frame_std
    k = torch.randn(hkv, L, D, generator=gen, device=gen.device)
    q = torch.randn(hq, L, D, generator=gen, device=gen.device)
    fm = f.repeat_interleave(frame_tokens, dim=1)
    k[:, text_pre:text_pre + frames * frame_tokens] += fm
    q[:, text_pre:text_pre + frames * frame_tokens] += fm.repeat_interleave(rep, dim=0)
    k[:, :sink_tokens] += sink_dir * u
    q[:, :text_pre] += (q_dir * u).repeat_interleave(rep, dim=0)
    q[:, L - text_post:] += (q_dir * u).repeat_interleave(rep, dim=0)
    v = torch.randn(hkv, L, D, generator=gen, device=gen.device)
    return q[None], k[None], v[None]


def dit_like(gen: torch.Generator, heads: int, frames: int = 33, rows: int = 45, cols: int = 80,
             text_tokens: int = 256, D: int = 128, rho: float = 0.9, local_std: float = 1.5,
             text_dir: float = 2.0, pad_to: int = 128):
    """Video-diffusion self-attention: a separable AR(1) field over (frame,row,col) shared by
    q and k of each spatial token, plus N(0,I); text tokens get +text_dir u.  The sequence is
    padded with N(0,I) tokens to a multiple of ``pad_to``."""
    n_img = frames * rows * cols
    L = n_img + text_tokens
    L = (L + pad_to - 1) // pad_to * pad_to
    field = torch.randn(heads, frames, rows, cols, D, generator=gen, device=gen.device)
    for ax in (1, 2, 3):
        field = _ar1(field, rho, dim=ax)
    field = field.reshape(heads, n_img, D) * local_std
    u = _unit(gen, heads, 1, D)
    q = torch.randn(heads, L, D, generator=gen, device=gen.device)
    k = torch.randn(heads, L, D, generator=gen, device=gen.device)
    q[:, :n_img] += field
    k[:, :n_img] += field
    q[:, n_img:n_img + text_tokens] += text_dir * u
    k[:, n_img:n_img + text_tokens] += text_dir * u
    v = torch.randn(heads, L, D, generator=gen, device=gen.device)
    return q[None], k[None], v[None]


WORKLOADS = {
    # fp32 reference-sized case
    "llama_mha_4k_fp32": Workload("llama_mha_4k_fp32", 32, 32, 4096, 16, 0.9, True, 2048, torch.float32),
    # Llama-3-8B attention layer shapes
    "llama3_8b_32k": Workload("llama3_8b_32k", 32, 8, 32768, 8, 0.9, True, 16384, torch.bfloat16),
    "llama3_8b_128k": Workload("llama3_8b_128k", 32, 8, 131072, 16, 0.9, True, None, torch.bfloat16),
    "llama3_8b_256k": Workload("llama3_8b_256k", 32, 8, 262144, 16, 0.9, True, None, torch.bfloat16),
    # Qwen2-VL-7B video prefill
    "qwen2vl_video_62k": Workload("qwen2vl_video_62k", 28, 4, 62208, 16, 0.9, True, None, torch.bfloat16),
    # HunyuanVideo DiT full attention
    "hunyuan_dit_119k": Workload("hunyuan_dit_119k", 24, 24, 119168, 8, 0.95, False, None, torch.bfloat16),
}


def make_inputs(name: str, seed: int = 0, heads_limit: Optional[int] = None,
                seq_len: Optional[int] = None, device=None):
    """Generate (q, k, v, workload) for a named workload.  ``heads_limit`` keeps only the first
    kv heads (and their q heads); ``seq_len`` overrides the length (decoder workloads only);
    ``device`` generates on that device (tensors stay there) instead of the CPU."""
    w = WORKLOADS[name]
    gen = (torch.Generator() if device is None else torch.Generator(device=device)).manual_seed(seed)
    hq, hkv = w.hq, w.hkv
    if heads_limit is not None:
        rep = hq // hkv
        hkv = min(hkv, heads_limit)
        hq = hkv * rep
    if name.startswith("llama"):
        q, k, v = llama_like(gen, hq, hkv, seq_len or w.seq_len)
    elif name.startswith("qwen2vl"):
        q, k, v = video_like(gen, hq, hkv)
    else:
        q, k, v = dit_like(gen, hq)
    if w.dtype != torch.float32:
        q, k, v = q.to(w.dtype), k.to(w.dtype), v.to(w.dtype)
    return q, k, v, w
