"""Generate tests/golden/*.npz from the UNMODIFIED reference code, imported on the CPU.

Run once, by hand, in a container that has the reference checked out:

    python tests/golden/make_golden.py --reference /path/to/x-attention

Nothing under tests/ reads the reference at test time: the tests replay these fixtures.

The reference needs two shims to import/run without a GPU (none of its files is changed):
  * a stub module ``block_sparse_attn`` (imported unconditionally at xattn/src/Xattention.py:10),
  * ``Tensor.to("cuda")`` made a no-op (hard-coded at xattn/src/Xattention.py:43,47,185,251).
The attention fixture comes from xattn/src/Flexprefill.py:12-44 (torch_block_wise_attention), the reference's own
statement of causal block-sparse attention; that module imports triton and flash_attn at load time, so both must
be importable where the script runs (no GPU needed).
For the Triton-semantics fixtures the reference's Triton kernels are run by Triton's CPU
interpreter (TRITON_INTERPRET=1) with ``torch.cuda.get_device_properties`` faked to a name
containing "100" (gate at xattn/src/Xattention.py:57-63).

Inputs are not stored: each case is (generator, seed, shape); a float64 checksum of the
inputs is stored so a drifting RNG is detected instead of silently failing parity.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def case_inputs(spec):
    """Deterministic (q, k) for a golden case; shared with the tests."""
    import torch
    sys.path.insert(0, os.path.join(ROOT, "x-attention_b200")) if os.path.join(
        ROOT, "x-attention_b200") not in sys.path else None
    from xattn_b200 import synth
    gen = torch.Generator().manual_seed(spec["seed"])
    H, Lq, Lk, D = spec["heads"], spec["q_len"], spec["k_len"], 128
    if spec["gen"] == "iid":
        q = torch.randn(1, H, Lq, D, generator=gen)
        k = torch.randn(1, H, Lk, D, generator=gen)
    elif spec["gen"] == "llama":
        q, k, _ = synth.llama_like(gen, H, H, Lk)
        q = q[:, :, Lk - Lq:].contiguous()
    else:
        raise ValueError(spec["gen"])
    if spec["dtype"] == "bf16":
        q, k = q.bfloat16(), k.bfloat16()
    return q, k


ESTIMATE_CASES = []


def _add(q_len, k_len, chunk, stride, causal, threshold, gen="iid", dtype="fp32", heads=2,
         keep_sink=False, keep_recent=False, seed=None):
    ESTIMATE_CASES.append(dict(
        q_len=q_len, k_len=k_len, chunk=chunk, stride=stride, causal=causal, threshold=threshold,
        gen=gen, dtype=dtype, heads=heads, keep_sink=keep_sink, keep_recent=keep_recent,
        seed=1000 + len(ESTIMATE_CASES) if seed is None else seed))


# un-padded multi-chunk causal (left-of-chunk columns blanked + first-chunk extra block)
for S in (4, 8, 16):
    _add(4096, 4096, 2048, S, True, 0.9)
_add(4096, 4096, 2048, 16, True, 0.9, gen="llama")
_add(4096, 4096, 1024, 8, True, 0.9, gen="llama")
# padded multi-chunk causal
for S in (8, 16):
    _add(4000, 4000, 2048, S, True, 0.9)
_add(4000, 4000, 2048, 16, True, 0.9, gen="llama")
# single chunk
_add(4096, 4096, 4096, 16, True, 0.9)
_add(4096, 4096, 4096, 8, True, 0.95, gen="llama")
# shorter than a chunk, not a multiple of 128
_add(1000, 1000, 2048, 16, True, 0.9)
_add(1000, 1000, 2048, 8, True, 0.5, gen="llama")
# non-causal padded / un-padded
_add(1920, 1920, 2048, 8, False, 0.95)
_add(1920, 1920, 2048, 16, False, 0.9, gen="llama")
_add(2048, 2048, 1024, 8, False, 0.9)
_add(2048, 2048, 1024, 16, False, 0.95, gen="llama")
# thresholds
for t in (0.0, 0.5, 1.0):
    _add(2048, 2048, 1024, 16, True, t, gen="llama")
    _add(2048, 2048, 1024, 16, False, t, gen="llama")
_add(4096, 4096, 2048, 16, True, [0.0, 0.5, 0.9, 0.99], heads=4, gen="llama")
# keep_sink / keep_recent
_add(4096, 4096, 2048, 16, True, 0.5, gen="llama", keep_sink=True, keep_recent=True)
_add(2048, 2048, 2048, 8, False, 0.5, gen="llama", keep_sink=True, keep_recent=True)
# q shorter than k (chunked prefill against a cache)
_add(2048, 6144, 2048, 16, True, 0.9, gen="llama")
_add(1024, 5000, 2048, 16, True, 0.9, gen="llama")
_add(2048, 6144, 2048, 8, False, 0.9, gen="llama")
# bf16 inputs (reference returns bf16 sums; the oracle is compared on the fp32 upcast run)
_add(4096, 4096, 2048, 16, True, 0.9, gen="llama", dtype="bf16")

TRITON_CASES = [
    dict(q_len=4096, k_len=4096, chunk=2048, stride=16, causal=True, threshold=0.9, gen="llama",
         dtype="fp32", heads=1, keep_sink=False, keep_recent=False, seed=7001),
    dict(q_len=2048, k_len=2048, chunk=1024, stride=8, causal=True, threshold=0.9, gen="iid",
         dtype="fp32", heads=1, keep_sink=False, keep_recent=False, seed=7002),
    dict(q_len=4096, k_len=4096, chunk=2048, stride=16, causal=False, threshold=0.9, gen="llama",
         dtype="fp32", heads=1, keep_sink=False, keep_recent=False, seed=7003),
]


# rotary embedding applied to the projection outputs (xattn/src/load_llama.py:34-65, call site :142)
ROPE_CASES = [
    dict(dtype="bf16", batch=1, hq=4, hkv=2, length=40, head_dim=128, seed=9001),
    dict(dtype="fp16", batch=2, hq=2, hkv=1, length=17, head_dim=128, seed=9002),
    dict(dtype="bf16", batch=1, hq=3, hkv=3, length=9, head_dim=64, seed=9003),
]


def rope_inputs(spec):
    """q [B,Hq,L,D], k [B,Hkv,L,D] (views of [B,L,H,D] storage, as the projections leave them) and cos/sin [B,L,D]
    built the way Llama's rotary module does (fp32 angles, cast to the model dtype)."""
    import torch
    dt = {"bf16": torch.bfloat16, "fp16": torch.float16}[spec["dtype"]]
    g = torch.Generator().manual_seed(spec["seed"])
    B, L, D = spec["batch"], spec["length"], spec["head_dim"]
    q = torch.randn(B, L, spec["hq"], D, generator=g).to(dt).transpose(1, 2)
    k = torch.randn(B, L, spec["hkv"], D, generator=g).to(dt).transpose(1, 2)
    pos = (torch.arange(L)[None, :] + torch.randint(0, 5000, (B, 1), generator=g)).float()
    inv_freq = 1.0 / (500000.0 ** (torch.arange(0, D, 2).float() / D))
    ang = pos[:, :, None] * inv_freq[None, None, :]
    emb = torch.cat((ang, ang), dim=-1)
    return q, k, emb.cos().to(dt), emb.sin().to(dt)


# block-sparse causal attention as the reference's own baseline file states it
# (xattn/src/Flexprefill.py:12-44, torch_block_wise_attention): MHA, q_len == k_len, causal
ATTENTION_CASES = [
    dict(length=512, heads=3, dtype="bf16", density=0.4, seed=8001),
    dict(length=1000, heads=2, dtype="bf16", density=0.3, seed=8002),      # ragged last block
    dict(length=1536, heads=2, dtype="bf16", density=0.25, seed=8003),
    dict(length=640, heads=2, dtype="fp16", density=0.5, seed=8004),
    dict(length=1280, heads=4, dtype="bf16", density=0.0, seed=8005),      # sink + diagonal only
]
ATTENTION_COL_STEP = 4        # every 4th output column is stored, plus the sum of each full output row


def attention_inputs(spec):
    """q, k, v [1,H,L,128] rounded to the case's 16-bit dtype, and a causal block mask [1,H,nb,nb] that keeps the
    sink block, the diagonal and a random `density` of the rest; shared with the tests."""
    import torch
    dt = {"bf16": torch.bfloat16, "fp16": torch.float16}[spec["dtype"]]
    g = torch.Generator().manual_seed(spec["seed"])
    H, L = spec["heads"], spec["length"]
    q = torch.randn(1, H, L, 128, generator=g).to(dt)
    k = torch.randn(1, H, L, 128, generator=g).to(dt)
    v = torch.randn(1, H, L, 128, generator=g).to(dt)
    nb = (L + 127) // 128
    m = torch.rand(1, H, nb, nb, generator=g) < spec["density"]
    m[..., 0] = True
    m |= torch.eye(nb, dtype=torch.bool)
    m &= torch.tril(torch.ones(nb, nb, dtype=torch.bool))
    return q, k, v, m


def make_attention_fixture(path):
    """Outputs of the reference's torch_block_wise_attention (fp32, on the fp32 upcast of the rounded inputs)."""
    import numpy as np
    import torch
    from xattn.src.Flexprefill import torch_block_wise_attention
    out = {}
    specs = []
    for i, spec in enumerate(ATTENTION_CASES):
        q, k, v, m = attention_inputs(spec)
        H, L = spec["heads"], spec["length"]
        nb = m.shape[-1]
        # the reference takes flat block indices row*nb+col, one list length for all heads: shorter lists are
        # filled up with repeats of block (0,0), which every list holds anyway
        flat = [(m[0, h].reshape(-1).nonzero().flatten()) for h in range(H)]
        width = max(int(f.numel()) for f in flat)
        block_idx = torch.zeros(1, H, width, dtype=torch.long)
        for h, f in enumerate(flat):
            block_idx[0, h, : f.numel()] = f
        o = torch_block_wise_attention(q.float().transpose(1, 2), k.float().transpose(1, 2),
                                       v.float().transpose(1, 2), block_idx, 128)       # [1,L,H,D]
        o = o.transpose(1, 2).contiguous()                                              # [1,H,L,D]
        chk = float(q.double().sum() + 3.0 * k.double().sum() + 5.0 * v.double().sum())
        out[f"out_{i}"] = o[..., ::ATTENTION_COL_STEP].contiguous().numpy()
        out[f"rowsum_{i}"] = o.double().sum(-1).numpy()
        out[f"mask_{i}"] = np.packbits(m.reshape(-1).numpy())
        specs.append(dict(spec, checksum=chk, mask_shape=list(m.shape), col_step=ATTENTION_COL_STEP))
        print("attention", i, spec, "blocks %d" % int(m.sum()))
    out["specs"] = np.array(json.dumps(specs))
    np.savez_compressed(path, **out)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rope-only", action="store_true", help="only (re)generate the rotary-embedding fixture")
    ap.add_argument("--attention-only", action="store_true", help="only (re)generate the attention fixture")
    ap.add_argument("--reference", default=os.environ.get("XATTN_REFERENCE"), required="XATTN_REFERENCE" not in os.environ,
                    help="checkout of mit-han-lab/x-attention (or set XATTN_REFERENCE)")
    ap.add_argument("--triton", action="store_true", help="also (re)generate the Triton-interpreter fixtures")
    args = ap.parse_args()
    if args.triton:
        os.environ["TRITON_INTERPRET"] = "1"

    import numpy as np
    import torch

    sys.path.insert(0, args.reference)
    stub = types.ModuleType("block_sparse_attn")
    stub.block_sparse_attn_func = None
    sys.modules["block_sparse_attn"] = stub
    _orig_to = torch.Tensor.to

    def _to(self, *a, **k):
        if a and isinstance(a[0], str) and a[0].startswith("cuda"):
            return self
        return _orig_to(self, *a, **k)

    torch.Tensor.to = _to
    from xattn.src.Xattention import xattn_estimate
    from xattn.src.utils import find_blocks_chunked

    make_attention_fixture(os.path.join(HERE, "attention_blockwise.npz"))
    if args.attention_only:
        return

    # rotary embedding: the reference's own function on the same inputs; 16-bit values stored as their bits
    from xattn.src.load_llama import apply_rotary_pos_emb
    out = {}
    for i, spec in enumerate(ROPE_CASES):
        q, k, cos, sin = rope_inputs(spec)
        qe, ke = apply_rotary_pos_emb(q, k, cos, sin)
        out[f"q_{i}"] = qe.contiguous().view(torch.int16).numpy()
        out[f"k_{i}"] = ke.contiguous().view(torch.int16).numpy()
    out["specs"] = np.array(json.dumps(ROPE_CASES))
    np.savez_compressed(os.path.join(HERE, "rope.npz"), **out)
    print("rope cases:", len(ROPE_CASES))
    if args.rope_only:
        return

    def run(spec, use_triton):
        q, k = case_inputs(spec)
        thr = spec["threshold"]
        thr_arg = torch.tensor(thr, dtype=torch.float32) if isinstance(thr, list) else thr
        qf, kf = q.float(), k.float()       # graded oracle = fp32 run on the (rounded) inputs
        sums, mask = xattn_estimate(
            qf, kf, block_size=128, stride=spec["stride"], threshold=thr_arg,
            chunk_size=spec["chunk"], use_triton=use_triton, causal=spec["causal"],
            keep_sink=spec["keep_sink"], keep_recent=spec["keep_recent"])
        chk = float(q.double().sum() + 3.0 * k.double().sum())
        return sums.float().numpy(), mask.numpy(), chk

    out = {}
    specs = []
    for i, spec in enumerate(ESTIMATE_CASES):
        sums, mask, chk = run(spec, use_triton=False)
        spec = dict(spec, checksum=chk, mask_shape=list(mask.shape))
        specs.append(spec)
        out[f"sums_{i}"] = sums
        out[f"mask_{i}"] = np.packbits(mask.reshape(-1))
        print(i, spec, "density %.3f" % mask.mean())
    out["specs"] = np.array(json.dumps(specs))
    np.savez_compressed(os.path.join(HERE, "estimate_torch_path.npz"), **out)

    # find_blocks_chunked alone, on random non-negative rows
    out = {}
    specs = []
    g = torch.Generator().manual_seed(4242)
    i = 0
    for causal in (True, False):
        for cur, R, N in ((0, 8, 8), (0, 16, 40), (4, 8, 12), (24, 16, 40), (12, 4, 16)):
            for thr in (0.0, 0.5, 0.9, 0.95, 1.0):
                x = torch.rand(1, 3, R, N, generator=g) ** 4
                if causal:   # future blocks carry no mass, as in the estimate
                    col = torch.arange(N)[None, :]
                    x = x * (col <= cur + torch.arange(R)[:, None]).float()
                m = find_blocks_chunked(x, cur, thr, None, decoding=False, mode="prefill", causal=causal)
                out[f"x_{i}"] = x.numpy()
                out[f"mask_{i}"] = m.numpy()
                specs.append(dict(current_index=cur, threshold=thr, causal=causal))
                i += 1
    # per-head tensor threshold
    x = torch.rand(1, 3, 8, 24, generator=g) ** 4
    thr = torch.tensor([0.3, 0.9, 0.6])
    m = find_blocks_chunked(x, 16, thr, None, decoding=False, mode="prefill", causal=True)
    out[f"x_{i}"] = x.numpy(); out[f"mask_{i}"] = m.numpy()
    specs.append(dict(current_index=16, threshold=thr.tolist(), causal=True))
    out["specs"] = np.array(json.dumps(specs))
    np.savez_compressed(os.path.join(HERE, "find_blocks_chunked.npz"), **out)
    print("find_blocks_chunked cases:", len(specs))

    if args.triton:
        class _P:
            name = "FAKE A100"
        torch.cuda.current_device = lambda: 0
        torch.cuda.get_device_properties = lambda *_a, **_k: _P()
        out = {}
        specs = []
        for i, spec in enumerate(TRITON_CASES):
            sums, mask, chk = run(spec, use_triton=True)
            # columns of skipped (future) GEMM tiles are uninitialised in the reference
            # (kernels.py:333 torch.empty); the softmax kernel writes zeros there, so sums are defined.
            spec = dict(spec, checksum=chk, mask_shape=list(mask.shape))
            specs.append(spec)
            out[f"sums_{i}"] = sums
            out[f"mask_{i}"] = np.packbits(mask.reshape(-1))
            print("triton", i, spec, "density %.3f" % mask.mean())
        out["specs"] = np.array(json.dumps(specs))
        np.savez_compressed(os.path.join(HERE, "estimate_triton_path.npz"), **out)


if __name__ == "__main__":
    main()
