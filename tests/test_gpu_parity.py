"""GPU parity: the sm_100a kernels, called through the C ABI, against the CPU oracle and against the
fixtures produced by the reference code.  Every test needs a B200."""
import json
import os

import numpy as np
import pytest
import torch

from make_golden import attention_inputs, case_inputs
from oracle import xattn_oracle as orc

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
DEV = "cuda"


def _assert_same_up_to_body_choice(a, b, msg=None):
    """Two ways of cutting the same prefill into kernel launches select the same blocks, but a CTA picks its
    attention body (whole blocks / half blocks) from the lists it happens to hold, and the two bodies add in
    a different order and round P against different running maxima: outputs agree to a few units of the last
    place of the 16-bit format (the bar against the oracle is 2e-2 max-abs)."""
    torch.testing.assert_close(a.float(), b.float(), rtol=2.0 ** -6, atol=2.0 ** -8, msg=msg)


def _load(name):
    z = np.load(os.path.join(GOLD, name))
    return z, json.loads(str(z["specs"]))


def _thr(spec):
    t = spec["threshold"]
    return torch.tensor(t, dtype=torch.float32) if isinstance(t, list) else t


def _unpack_mask(z, i, shape):
    return torch.from_numpy(np.unpackbits(z[f"mask_{i}"])[: int(np.prod(shape))].reshape(shape).astype(bool))


@pytest.fixture(autouse=True)
def _status_clean():
    import xattn_b200
    yield
    xattn_b200.check_device_status()


def _assert_masks(mask, ref_mask, ref_sums, spec):
    exempt = orc.margin_exempt(ref_sums, spec["q_len"], spec["k_len"], 128, spec["stride"], spec["chunk"],
                               _thr(spec), spec["causal"])
    diff = (mask != ref_mask) & ~exempt
    assert not diff.any(), f"{int(diff.sum())} non-exempt mask mismatches at {diff.nonzero()[:6].tolist()}"
    # exemptions must stay the exception
    assert int((mask != ref_mask).sum()) <= max(2, int(0.01 * mask.numel()))


# sums tolerance: block sums are O(1) sums of fp32 softmax probabilities; the tensor-core product of
# the (bf16 or split-fp32) inputs differs from the CPU fp32 product by ~1e-6 relative per score.
SUMS_RTOL, SUMS_ATOL = 2e-4, 2e-5

_zt, _st = _load("estimate_torch_path.npz")


@pytest.mark.parametrize("i", range(len(_st)))
def test_estimate_and_masks_vs_reference_fixtures(i):
    """fp32 inputs (split-precision GEMM) and bf16 inputs against the reference's torch branch."""
    import xattn_b200
    spec = _st[i]
    q, k = case_inputs(spec)
    xattn_b200.set_estimate_semantics("torch")
    sums, mask = xattn_b200.xattn_estimate(
        q.to(DEV), k.to(DEV), 128, spec["stride"], threshold=_thr(spec), chunk_size=spec["chunk"],
        causal=spec["causal"], keep_sink=spec["keep_sink"], keep_recent=spec["keep_recent"])
    ref_sums = torch.from_numpy(_zt[f"sums_{i}"])
    ref_mask = _unpack_mask(_zt, i, spec["mask_shape"])
    assert sums.dtype == q.dtype and mask.dtype == torch.bool
    assert tuple(mask.shape) == tuple(spec["mask_shape"])
    tol = dict(rtol=SUMS_RTOL, atol=SUMS_ATOL) if q.dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    assert torch.allclose(sums.float().cpu(), ref_sums, **tol), (sums.float().cpu() - ref_sums).abs().max()
    _assert_masks(mask.cpu(), ref_mask, ref_sums, spec)


def test_estimate_triton_semantics_vs_reference_fixtures():
    import xattn_b200
    z, specs = _load("estimate_triton_path.npz")
    try:
        xattn_b200.set_estimate_semantics("triton")
        for i, spec in enumerate(specs):
            q, k = case_inputs(spec)
            sums, mask = xattn_b200.xattn_estimate(q.to(DEV), k.to(DEV), 128, spec["stride"], threshold=_thr(spec),
                                                   chunk_size=spec["chunk"], causal=spec["causal"])
            ref_sums = torch.from_numpy(z[f"sums_{i}"])
            assert torch.allclose(sums.float().cpu(), ref_sums, rtol=SUMS_RTOL, atol=SUMS_ATOL)
            _assert_masks(mask.cpu(), _unpack_mask(z, i, spec["mask_shape"]), ref_sums, spec)
    finally:
        xattn_b200.set_estimate_semantics("torch")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("hq,hkv", [(4, 4), (8, 2)])
def test_estimate_16bit_inputs_vs_oracle(dtype, hq, hkv):
    """bf16/fp16 inputs, GQA included: fp32 sums against the oracle run on the same rounded values."""
    from xattn_b200 import ops, synth
    gen = torch.Generator().manual_seed(11)
    q, k, _ = synth.llama_like(gen, hq, hkv, 4096)
    q, k = q.to(dtype), k.to(dtype)
    for stride, chunk, causal, sem in ((16, 2048, True, "torch"), (8, 4096, True, "triton"), (8, 2048, False, "torch")):
        got = ops.estimate_block_sums(q.to(DEV), k.to(DEV), stride, 128, chunk, 1.0, causal, semantics=sem).cpu()
        want = orc.estimate_block_sums(q.float(), k.float().repeat_interleave(hq // hkv, 1), 128, stride, 1.0, chunk,
                                       causal, sem)
        assert torch.allclose(got, want, rtol=SUMS_RTOL, atol=SUMS_ATOL), (got - want).abs().max()


def test_estimate_strided_layout_and_ragged_length():
    """HF-style [B,L,H,D] storage viewed as [B,H,L,D], and a length that is not a multiple of the stride."""
    from xattn_b200 import ops
    g = torch.Generator().manual_seed(5)
    L = 1003
    q = torch.randn(1, L, 3, 128, generator=g).bfloat16().transpose(1, 2)
    k = torch.randn(1, L, 3, 128, generator=g).bfloat16().transpose(1, 2)
    dq = q.to(DEV).transpose(1, 2).contiguous().transpose(1, 2)
    dk = k.to(DEV).transpose(1, 2).contiguous().transpose(1, 2)
    got = ops.estimate_block_sums(dq, dk, 16, 128, 2048, 1.0, True).cpu()
    want = orc.estimate_block_sums(q.float(), k.float(), 128, 16, 1.0, 2048, True, "torch")
    assert torch.allclose(got, want, rtol=SUMS_RTOL, atol=SUMS_ATOL), (got - want).abs().max()
    # other strides, non-causal, and a longer ragged sequence whose last tile is not the first one
    for S, causal, sem in ((8, False, "torch"), (4, True, "triton")):
        got = ops.estimate_block_sums(dq, dk, S, 128, 2048, 1.0, causal, semantics=sem).cpu()
        want = orc.estimate_block_sums(q.float(), k.float(), 128, S, 1.0, 2048, causal, sem)
        assert torch.allclose(got, want, rtol=SUMS_RTOL, atol=SUMS_ATOL), (S, causal, (got - want).abs().max())


def test_ragged_lengths_are_not_padded_by_copying():
    """A length that is no multiple of the stride costs a staging copy of one tile per head, not a padded copy of
    q and k (HunyuanVideo's real calls have such lengths at 118K tokens)."""
    from xattn_b200 import ops
    g = torch.Generator().manual_seed(6)
    Lq, Lk, H = 40003, 40011, 2
    q = torch.randn(1, H, Lq, 128, generator=g).bfloat16()
    k = torch.randn(1, H, Lk, 128, generator=g).bfloat16()
    dq, dk = q.to(DEV), k.to(DEV)
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    got = ops.estimate_block_sums(dq, dk, 8, 128, 4096, 1.0, False)
    torch.cuda.synchronize()
    extra = torch.cuda.max_memory_allocated() - base
    want = orc.estimate_block_sums(q.float(), k.float(), 128, 8, 1.0, 4096, False, "torch")
    assert torch.allclose(got.cpu(), want, rtol=SUMS_RTOL, atol=SUMS_ATOL), (got.cpu() - want).abs().max()
    # scratch for the partial sums is inherent (rows x key blocks); a padded copy of q and k would add 20 MB more
    rows, kb = want.shape[2] * 16, want.shape[3]
    scratch = H * rows * (kb * 4 + 8 * ((kb + 15) // 16) + 8) + got.numel() * 4
    assert extra < scratch + 4 * 1024 * 1024, (extra, scratch)
    assert extra < scratch + (dq.numel() + dk.numel()) * 2 // 2


def test_select_vs_find_blocks_chunked_fixtures():
    """The selection kernel alone, on the reference's own inputs/outputs: bit-exact outside the margin."""
    import xattn_b200
    z, specs = _load("find_blocks_chunked.npz")
    for i, spec in enumerate(specs):
        x = torch.from_numpy(z[f"x_{i}"])
        ref = torch.from_numpy(z[f"mask_{i}"])
        thr = _thr(spec)
        got = xattn_b200.find_blocks_chunked(x.to(DEV), spec["current_index"], thr, None, decoding=False,
                                             mode="prefill", causal=spec["causal"]).cpu()
        ex = orc.margin_exempt_chunk(x, spec["current_index"], thr, spec["causal"])
        d = (got != ref) & ~ex
        assert not d.any(), (i, spec, d.nonzero()[:5].tolist())


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("N,bpc", [(512, 16), (1024, 64), (200, 8)])
def test_select_flat_rows_take_the_sort_route(causal, N, bpc):
    """Flat score rows keep hundreds of blocks, which exercises the warp-sort route of the kernel (peaked
    rows finish in the extraction loop); both must agree with the oracle outside the margin."""
    from xattn_b200 import ops
    g = torch.Generator().manual_seed(N + bpc)
    R = 2 * bpc
    off = N - R
    x = torch.rand(1, 3, R, N, generator=g) + 0.05
    x[:, 1] = x[:, 1] ** 8                       # one peaked head next to two flat ones
    if causal:
        x = x * (torch.arange(N)[None, :] <= off + torch.arange(R)[:, None]).float()
    for thr in (0.3, 0.9, 1.0):
        got, _, _ = ops.select_blocks(x.to(DEV), bpc, off, thr, causal, True)
        parts, exs = [], []
        for c in range(2):
            xc = x[:, :, c * bpc:(c + 1) * bpc]
            parts.append(orc.select_blocks_chunk(xc, off + c * bpc, thr, causal))
            exs.append(orc.margin_exempt_chunk(xc, off + c * bpc, thr, causal))
        want = orc.finish_masks(torch.cat(parts, -2), R, causal, False, False)
        dmask = (got.cpu() != want) & ~torch.cat(exs, -2)
        assert not dmask.any(), (thr, dmask.nonzero()[:5].tolist())
        assert int(want.sum()) > 24 * 3 * R * (0.5 if causal else 1.0) or thr < 0.9


def test_select_lists_match_mask():
    from xattn_b200 import ops
    g = torch.Generator().manual_seed(9)
    x = (torch.rand(1, 4, 32, 32, generator=g) ** 6) * torch.tril(torch.ones(32, 32))
    mask, idx, cnt = ops.select_blocks(x.to(DEV), 16, 0, 0.9, True, True, list_shape=(4096 - 50, 4096 - 50))
    mask, idx, cnt = mask.cpu(), idx.cpu(), cnt.cpu()
    for h in range(4):
        for r in range(32):
            want = mask[0, h, r].nonzero().flatten().tolist()
            assert idx[0, h, r, : cnt[0, h, r]].tolist() == want
    idx2, cnt2 = ops.mask_to_lists(mask.to(DEV), 4096 - 50, 4096 - 50, True)
    assert torch.equal(cnt2.cpu(), cnt)
    for h in range(4):
        for r in range(32):
            assert torch.equal(idx2.cpu()[0, h, r, : cnt[0, h, r]], idx[0, h, r, : cnt[0, h, r]])


def _random_block_mask(g, H, qb, kb, causal, density=0.35):
    m = torch.rand(1, H, qb, kb, generator=g) < density
    off = kb - qb
    for r in range(qb):
        m[:, :, r, min(off + r, kb - 1)] = True
        m[:, :, r, 0] = True
    if causal:
        m &= torch.tril(torch.ones(qb, kb, dtype=torch.bool), diagonal=off)
    return m


# output tolerance of the attention phase: bf16 against the fp32 oracle under the same mask
OUT_MAX_ABS, OUT_MEAN_ABS = 2e-2, 2e-3


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("hq,hkv,lq,lk", [(2, 2, 1024, 1024), (4, 1, 1000, 1000), (2, 2, 512, 1536), (2, 1, 300, 1100)])
def test_block_sparse_attention_vs_oracle(causal, dtype, hq, hkv, lq, lk):
    from xattn_b200 import ops
    g = torch.Generator().manual_seed(lq + lk + hq)
    q = torch.randn(1, hq, lq, 128, generator=g).to(dtype)
    k = torch.randn(1, hkv, lk, 128, generator=g).to(dtype)
    v = torch.randn(1, hkv, lk, 128, generator=g).to(dtype)
    qb, kb = (lq + 127) // 128, (lk + 127) // 128
    mask = _random_block_mask(g, hq, qb, kb, causal)
    idx, cnt = ops.mask_to_lists(mask.to(DEV), lq, lk, causal)
    out = ops.block_sparse_attention(q.to(DEV), k.to(DEV), v.to(DEV), idx, cnt, causal).float().cpu()
    ref = orc.block_sparse_attention_oracle(q, k, v, mask, causal)
    err = (out - ref).abs()
    assert err.max() < OUT_MAX_ABS and err.mean() < OUT_MEAN_ABS, (err.max(), err.mean())


def test_block_sparse_attention_vs_reference_blockwise_fixture():
    """The attention kernel against outputs of the reference's own torch_block_wise_attention
    (xattn/src/Flexprefill.py:12-44) stored in tests/golden/attention_blockwise.npz."""
    from xattn_b200 import ops
    z, specs = _load("attention_blockwise.npz")
    for i, spec in enumerate(specs):
        q, k, v, m = attention_inputs(spec)
        L = spec["length"]
        idx, cnt = ops.mask_to_lists(m.to(DEV), L, L, True)
        out = ops.block_sparse_attention(q.to(DEV), k.to(DEV), v.to(DEV), idx, cnt, True).float().cpu()
        err = (out[..., :: spec["col_step"]] - torch.from_numpy(z[f"out_{i}"])).abs()
        assert err.max() < OUT_MAX_ABS and err.mean() < OUT_MEAN_ABS, (spec, err.max(), err.mean())
        rs = (out.double().sum(-1) - torch.from_numpy(z[f"rowsum_{i}"])).abs()
        assert rs.max() < 128 * OUT_MEAN_ABS, (spec, rs.max())


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("dtype,hq,hkv,lq,lk", [(torch.bfloat16, 8, 2, 2048, 2048), (torch.float16, 4, 1, 1000, 1000),
                                                (torch.bfloat16, 2, 1, 640, 1664), (torch.bfloat16, 6, 1, 1300, 1300)])
def test_short_shared_lists_take_the_pair_kernel(causal, dtype, hq, hkv, lq, lk):
    """Rows whose kv group shares a list of one or two blocks (sink + diagonal) run through the kernel that loads
    K/V once per group; rows with longer lists, or lists that differ between the heads of a group, stay in the
    general kernel.  Both against the oracle, and against the general kernel alone."""
    from xattn_b200 import ops
    g = torch.Generator().manual_seed(lq + hq)
    q = torch.randn(1, hq, lq, 128, generator=g).to(dtype)
    k = torch.randn(1, hkv, lk, 128, generator=g).to(dtype)
    v = torch.randn(1, hkv, lk, 128, generator=g).to(dtype)
    qb, kb = (lq + 127) // 128, (lk + 127) // 128
    off = kb - qb
    mask = torch.zeros(1, hq, qb, kb, dtype=torch.bool)
    for r in range(qb):
        mask[:, :, r, 0] = True
        mask[:, :, r, min(off + r, kb - 1)] = True
    mask[0, 0, 3, 1] = True            # one head of a group lists a third block: the whole group item stays general
    mask[0, hq - 1, 2, 0] = False      # a list that differs inside a group
    if qb > 5:
        mask[0, :, 5, :] = False
        mask[0, :, 5, min(off + 5, kb - 1)] = True      # a one-block list shared by all heads
    idx, cnt = ops.mask_to_lists(mask.to(DEV), lq, lk, causal)
    # these small masks stay below the share of qualifying blocks at which the library splits a call by itself
    before = ops.pair_split_share(0)
    try:
        n0 = ops._lib.load().xattn_b200_launch_count()
        out = ops.block_sparse_attention(q.to(DEV), k.to(DEV), v.to(DEV), idx, cnt, causal,
                                         use_workspace=True).float().cpu()
        # causal: classify, pair kernel, general kernel; non-causal calls sort their items instead: order, general
        assert ops._lib.load().xattn_b200_launch_count() - n0 == (3 if causal else 2)
    finally:
        ops.pair_split_share(before)
    ref = orc.block_sparse_attention_oracle(q, k, v, mask, causal)
    err = (out - ref).abs()
    assert err.max() < OUT_MAX_ABS and err.mean() < OUT_MEAN_ABS, (err.max(), err.mean())
    gen = ops.block_sparse_attention(q.to(DEV), k.to(DEV), v.to(DEV), idx, cnt, causal, use_workspace=False)
    _assert_same_up_to_body_choice(out, gen.float().cpu())


@pytest.mark.parametrize("hq,hkv,L", [(4, 4, 6400), (3, 1, 2000), (6, 2, 128 * 75)])
def test_non_causal_items_sorted_by_list_length(hq, hkv, L):
    """With scratch memory a non-causal call deals its work items longest list first, in alternating direction over
    the SMs (more than one row of the deal for the first and last shape, a partial last row in all).  Every row must
    still be computed exactly once: against the oracle, and against the call without scratch memory, on a mask whose
    rows list between one block and all of them; the output buffer starts as NaN."""
    from xattn_b200 import ops
    g = torch.Generator().manual_seed(L + hq)
    q = torch.randn(1, hq, L, 128, generator=g).bfloat16()
    k = torch.randn(1, hkv, L, 128, generator=g).bfloat16()
    v = torch.randn(1, hkv, L, 128, generator=g).bfloat16()
    nb = (L + 127) // 128
    want = (torch.rand(1, hq, nb, 1, generator=g) ** 3 * nb).long().clamp(1, nb)       # skewed list lengths
    mask = torch.rand(1, hq, nb, nb, generator=g).argsort(-1).argsort(-1) < want
    mask[0, 0, 0, :] = True                                                            # one row lists every block
    mask[0, hq - 1, nb - 1, :] = False                                                 # and one lists none
    idx, cnt = ops.mask_to_lists(mask.to(DEV), L, L, False)
    outs = []
    for ws in (True, False):
        buf = torch.full((1, L, hq, 128), float("nan"), dtype=torch.bfloat16, device=DEV).transpose(1, 2)
        ops.block_sparse_attention(q.to(DEV), k.to(DEV), v.to(DEV), idx, cnt, False, out=buf, use_workspace=ws)
        outs.append(buf.float().cpu())
    assert not torch.isnan(outs[0]).any()
    ref = orc.block_sparse_attention_oracle(q, k, v, mask, False)
    err = (outs[0] - ref).abs()
    assert err.max() < OUT_MAX_ABS and err.mean() < OUT_MEAN_ABS, (err.max(), err.mean())
    _assert_same_up_to_body_choice(outs[0], outs[1])


def test_pair_kernel_is_declined_on_the_device_when_few_blocks_qualify():
    """With the library's own rule (92 % of the listed blocks must qualify) a mask whose rows mostly list three blocks
    is computed by the general kernel alone, although the pair kernel was offered its scratch memory: same output as
    without it, bit for bit; a sink + diagonal mask takes the split and matches up to summation order."""
    from xattn_b200 import ops
    assert ops.pair_split_share() == 92
    g = torch.Generator().manual_seed(5)
    hq, hkv, L = 8, 2, 4096
    q = torch.randn(1, hq, L, 128, generator=g).bfloat16().to(DEV)
    k = torch.randn(1, hkv, L, 128, generator=g).bfloat16().to(DEV)
    v = torch.randn(1, hkv, L, 128, generator=g).bfloat16().to(DEV)
    nb = L // 128
    eye = torch.eye(nb, dtype=torch.bool)
    two = eye.clone(); two[:, 0] = True
    three = two | torch.diag(torch.ones(nb - 1, dtype=torch.bool), -1)
    for base, split in ((three, False), (two, True)):
        mask = base[None, None].expand(1, hq, -1, -1).contiguous()
        idx, cnt = ops.mask_to_lists(mask.to(DEV), L, L, True)
        gen = ops.block_sparse_attention(q, k, v, idx, cnt, True, use_workspace=False).clone()
        both = ops.block_sparse_attention(q, k, v, idx, cnt, True, use_workspace=True)
        if split:
            assert not torch.equal(both, gen)                      # another summation order: the pair kernel ran
            _assert_same_up_to_body_choice(both.float().cpu(), gen.float().cpu())
        else:
            assert torch.equal(both, gen)


@pytest.mark.parametrize("causal,density,hq,hkv,L", [(True, 1.0, 2, 1, 4096), (False, 0.5, 2, 2, 3072), (True, 0.3, 4, 2, 5000)])
def test_long_lists_take_the_half_block_path(causal, density, hq, hkv, L):
    """Rows that list many blocks run through the half-block instantiation of the kernel (each 128-key block
    as two 64-key halves); short lists (the other tests) through the full-block one.  Same oracle, same bars."""
    from xattn_b200 import ops
    g = torch.Generator().manual_seed(L + hq)
    q = torch.randn(1, hq, L, 128, generator=g).bfloat16()
    k = torch.randn(1, hkv, L, 128, generator=g).bfloat16()
    v = torch.randn(1, hkv, L, 128, generator=g).bfloat16()
    qb = (L + 127) // 128
    mask = _random_block_mask(g, hq, qb, qb, causal, density)
    idx, cnt = ops.mask_to_lists(mask.to(DEV), L, L, causal)
    assert float(cnt.float().mean()) >= 5          # well above the kernel's switch-over point (3.5)
    out = ops.block_sparse_attention(q.to(DEV), k.to(DEV), v.to(DEV), idx, cnt, causal).float().cpu()
    ref = orc.block_sparse_attention_oracle(q, k, v, mask, causal)
    err = (out - ref).abs()
    assert err.max() < OUT_MAX_ABS and err.mean() < OUT_MEAN_ABS, (err.max(), err.mean())


def test_attention_rescale_path_long_list():
    """Growing key norms force repeated lazy rescales of O, here on a list long enough for the half-block path."""
    from xattn_b200 import ops
    g = torch.Generator().manual_seed(78)
    L = 2048
    q = torch.randn(1, 1, L, 128, generator=g)
    k = torch.randn(1, 1, L, 128, generator=g) * torch.linspace(6.0, 0.5, L)[None, None, :, None]   # early keys dominate
    v = torch.randn(1, 1, L, 128, generator=g)
    q, k, v = q.bfloat16(), k.bfloat16(), v.bfloat16()
    mask = torch.tril(torch.ones(16, 16, dtype=torch.bool))[None, None].clone()
    idx, cnt = ops.mask_to_lists(mask.to(DEV), L, L, True)
    out = ops.block_sparse_attention(q.to(DEV), k.to(DEV), v.to(DEV), idx, cnt, True).float().cpu()
    ref = orc.block_sparse_attention_oracle(q, k, v, mask, True)
    err = (out - ref).abs()
    assert torch.isfinite(out).all() and err.max() < 3e-2 and err.mean() < OUT_MEAN_ABS, (err.max(), err.mean())


def test_attention_rescale_path_and_empty_rows():
    """Scores that grow block after block force the lazy rescale of O; rows with an empty list give zeros."""
    from xattn_b200 import ops
    g = torch.Generator().manual_seed(77)
    L = 1024
    q = torch.randn(1, 1, L, 128, generator=g)
    k = torch.randn(1, 1, L, 128, generator=g)
    k = k * torch.linspace(0.5, 6.0, L)[None, None, :, None]        # later keys dominate more and more
    v = torch.randn(1, 1, L, 128, generator=g)
    q, k, v = q.bfloat16(), k.bfloat16(), v.bfloat16()
    mask = torch.tril(torch.ones(8, 8, dtype=torch.bool))[None, None].clone()
    mask[0, 0, 3] = False                                            # an empty row
    idx, cnt = ops.mask_to_lists(mask.to(DEV), L, L, True)
    out = ops.block_sparse_attention(q.to(DEV), k.to(DEV), v.to(DEV), idx, cnt, True).float().cpu()
    ref = orc.block_sparse_attention_oracle(q, k, v, mask, True)
    assert torch.isfinite(out).all()
    assert out[0, 0, 384:512].abs().max() == 0
    err = (out - ref).abs()
    assert err.max() < 3e-2 and err.mean() < OUT_MEAN_ABS, (err.max(), err.mean())


def test_block_sparse_attn_func_mirror():
    import xattn_b200
    g = torch.Generator().manual_seed(1)
    L, H = 640, 2
    q = torch.randn(L, H, 128, generator=g).bfloat16()
    k = torch.randn(L, H, 128, generator=g).bfloat16()
    v = torch.randn(L, H, 128, generator=g).bfloat16()
    mask = _random_block_mask(g, H, 5, 5, True)
    cu = torch.tensor([0, L], dtype=torch.int32, device=DEV)
    hm = torch.ones(H, dtype=torch.int32, device=DEV)
    out = xattn_b200.block_sparse_attn_func(q.to(DEV), k.to(DEV), v.to(DEV), cu, cu, hm, None, mask.to(DEV), L, L,
                                            p_dropout=0.0, deterministic=True, is_causal=True)
    ref = orc.block_sparse_attention_oracle(q.transpose(0, 1)[None], k.transpose(0, 1)[None],
                                            v.transpose(0, 1)[None], mask, True)
    err = (out.float().cpu().transpose(0, 1)[None] - ref).abs()
    assert err.max() < OUT_MAX_ABS and err.mean() < OUT_MEAN_ABS


@pytest.mark.parametrize("name,L,heads", [("llama3_8b_32k", 8192, 2), ("llama3_8b_128k", 4096, 1)])
def test_prefill_end_to_end_vs_oracle(name, L, heads):
    """Xattention_prefill on a cut-down Llama workload: mask parity with the oracle, then output parity with
    the oracle's attention under the mask the GPU produced."""
    import xattn_b200
    from xattn_b200 import ops, synth
    q, k, v, w = synth.make_inputs(name, seed=3, heads_limit=heads, seq_len=L)
    chunk = w.chunk_size or orc.default_chunk_size(L)
    chunk = min(chunk, 2048) if L <= 4096 else chunk
    rep = q.shape[1] // k.shape[1]
    sums, mask = xattn_b200.xattn_estimate(q.to(DEV), k.to(DEV), 128, w.stride, threshold=w.threshold,
                                           chunk_size=chunk, causal=True)
    osums, omask = orc.xattn_estimate_oracle(q.float(), k.float().repeat_interleave(rep, 1), 128, w.stride, 1.0,
                                             w.threshold, chunk, True)
    ex = orc.margin_exempt(osums, L, L, 128, w.stride, chunk, w.threshold, True)
    d = (mask.cpu() != omask) & ~ex
    assert not d.any(), d.nonzero()[:6].tolist()
    out = xattn_b200.Xattention_prefill(q.to(DEV), k.to(DEV), v.to(DEV), w.stride, threshold=w.threshold,
                                        chunk_size=chunk, causal=True)
    assert out.shape == q.shape and out.dtype == q.dtype
    ref = orc.block_sparse_attention_oracle(q, k, v, mask.cpu()[:, :, : L // 128, : L // 128], True)
    err = (out.float().cpu() - ref).abs()
    assert err.max() < OUT_MAX_ABS and err.mean() < OUT_MEAN_ABS, (err.max(), err.mean())


def _check_workload(q, k, v, stride, threshold, chunk, causal, sample_rows=None):
    """Mask parity with the oracle outside the margin, then output parity under the GPU's own mask."""
    import xattn_b200
    L = q.shape[2]
    rep = q.shape[1] // k.shape[1]
    dq, dk, dv = q.to(DEV), k.to(DEV), v.to(DEV)
    sums, mask = xattn_b200.xattn_estimate(dq, dk, 128, stride, threshold=threshold, chunk_size=chunk, causal=causal)
    osums, omask = orc.xattn_estimate_oracle(q.float(), k.float().repeat_interleave(rep, 1), 128, stride, 1.0,
                                             threshold, chunk, causal)
    assert torch.allclose(sums.float().cpu(), osums, rtol=2e-2, atol=2e-2)          # returned in bf16
    ex = orc.margin_exempt(osums, L, L, 128, stride, chunk, threshold, causal)
    d = (mask.cpu() != omask) & ~ex
    assert not d.any(), d.nonzero()[:6].tolist()
    assert int((mask.cpu() != omask).sum()) <= max(2, int(2e-3 * mask.numel()))
    out = xattn_b200.Xattention_prefill(dq, dk, dv, stride, threshold=threshold, chunk_size=chunk, causal=causal)
    qb = (L + 127) // 128
    m = mask.cpu()[:, :, :qb, :qb]
    if sample_rows is None:
        ref = orc.block_sparse_attention_oracle(q, k, v, m, causal)
        err = (out.float().cpu() - ref).abs()
    else:
        errs = []
        for r in sample_rows:
            r0, r1 = r * 128, min(L, (r + 1) * 128)
            kk = k[:, :, :r1] if causal else k
            vv = v[:, :, :r1] if causal else v
            mm = m[:, :, r:r + 1, : (kk.shape[2] + 127) // 128]
            ref = orc.block_sparse_attention_oracle(q[:, :, r0:r1], kk, vv, mm, causal)
            errs.append((out[:, :, r0:r1].float().cpu() - ref).abs())
        err = torch.cat(errs, dim=2)
    assert err.max() < OUT_MAX_ABS and err.mean() < OUT_MEAN_ABS, (err.max(), err.mean())
    return float(mask.float().mean())


def test_llama_32k_full_length_one_kv_group():
    """The llama3_8b_32k workload at its real length (32768, S=8, chunk 16384) on one kv group (4 query heads);
    outputs checked on 12 query blocks spread over the sequence."""
    from xattn_b200 import synth
    q, k, v, w = synth.make_inputs("llama3_8b_32k", seed=1, heads_limit=1)
    _check_workload(q, k, v, w.stride, w.threshold, w.chunk_size, True, sample_rows=[0, 1, 7, 31, 64, 100, 127, 128, 129, 200, 254, 255])


def test_llama_128k_full_length_two_query_heads():
    """The llama3_8b_128k workload at its real length (131072, S=16, default chunk 2048: 64 chunks, 1024 key
    blocks per row, the single-CTA streaming estimate and the chunk-band layout) on two query heads of one kv
    group: masks over all rows, outputs on 12 query blocks."""
    from xattn_b200 import synth
    q, k, v, w = synth.make_inputs("llama3_8b_128k", seed=2, heads_limit=1)
    assert q.shape[2] == 131072 and orc.default_chunk_size(131072) == 2048
    _check_workload(q[:, :2].contiguous(), k, v, w.stride, w.threshold, 2048, True,
                    sample_rows=[0, 1, 15, 16, 17, 100, 511, 512, 513, 800, 1022, 1023])


def test_video_62k_full_length_two_query_heads():
    """The qwen2vl_video_62k workload at its real length (62208 tokens, keys padded to 65536, default chunk
    4096, S=16) on two query heads of one kv group: masks over all rows, outputs on 12 query blocks."""
    from xattn_b200 import synth
    q, k, v, w = synth.make_inputs("qwen2vl_video_62k", seed=3, heads_limit=1)
    assert q.shape[2] == 62208 and orc.default_chunk_size(62208) == 4096
    _check_workload(q[:, :2].contiguous(), k, v, w.stride, w.threshold, 4096, True,
                    sample_rows=[0, 3, 4, 31, 32, 33, 200, 243, 300, 400, 484, 485])


def test_dit_119k_full_length_two_heads():
    """The hunyuan_dit_119k workload at its real length (119168 tokens, non-causal, S=8, threshold 0.95,
    default chunk 2048: keys zero-padded to 120832, and the padded keys take softmax mass as in the
    reference) on two heads: masks over all rows, outputs on 12 query blocks."""
    from xattn_b200 import synth
    g = torch.Generator().manual_seed(4)
    q, k, v = synth.dit_like(g, 2)
    q, k, v = q.bfloat16(), k.bfloat16(), v.bfloat16()
    assert q.shape[2] == 119168 and orc.default_chunk_size(119168) == 2048
    _check_workload(q, k, v, 8, 0.95, 2048, False,
                    sample_rows=[0, 1, 15, 16, 100, 300, 464, 465, 700, 900, 929, 930])


def test_llama_mha_4k_fp32_end_to_end():
    """The fp32 reference-sized case (32 MHA heads, 4096 tokens, S=16, chunk 2048) through Xattention_prefill
    on fp32 inputs.  Masks: against the fp32 oracle over all heads and rows.  Outputs: the attention phase
    computes fp32 inputs in bf16 (the reference's attention backend takes 16-bit inputs only), so they are
    checked against the oracle's attention on the bf16-rounded q/k/v under the GPU's mask."""
    import xattn_b200
    from xattn_b200 import synth
    q, k, v, w = synth.make_inputs("llama_mha_4k_fp32", seed=0)
    assert q.dtype == torch.float32 and q.shape == (1, 32, 4096, 128)
    L = 4096
    dq, dk, dv = q.to(DEV), k.to(DEV), v.to(DEV)
    sums, mask = xattn_b200.xattn_estimate(dq, dk, 128, w.stride, threshold=w.threshold, chunk_size=w.chunk_size)
    osums, omask = orc.xattn_estimate_oracle(q, k, 128, w.stride, 1.0, w.threshold, w.chunk_size, True)
    assert sums.dtype == torch.float32
    assert torch.allclose(sums.cpu(), osums, rtol=SUMS_RTOL, atol=SUMS_ATOL), (sums.cpu() - osums).abs().max()
    ex = orc.margin_exempt(osums, L, L, 128, w.stride, w.chunk_size, w.threshold, True)
    d = (mask.cpu() != omask) & ~ex
    assert not d.any(), d.nonzero()[:6].tolist()
    out = xattn_b200.Xattention_prefill(dq, dk, dv, w.stride, threshold=w.threshold, chunk_size=w.chunk_size)
    assert out.dtype == torch.float32 and out.shape == q.shape
    qr, kr, vr = q.bfloat16(), k.bfloat16(), v.bfloat16()
    errs = []
    for r in (0, 5, 15, 16, 17, 31):
        r0, r1 = r * 128, (r + 1) * 128
        ref = orc.block_sparse_attention_oracle(qr[:, :, r0:r1], kr[:, :, :r1], vr[:, :, :r1],
                                                mask.cpu()[:, :, r:r + 1, : r + 1], True)
        errs.append((out[:, :, r0:r1].cpu() - ref).abs())
    err = torch.cat(errs, dim=2)
    assert err.max() < OUT_MAX_ABS and err.mean() < OUT_MEAN_ABS, (err.max(), err.mean())


def test_video_prefill_like_workload_padded_causal():
    """Qwen2-VL-style sequence (text + frames + text), length not a multiple of the chunk (padded keys)."""
    from xattn_b200 import synth
    g = torch.Generator().manual_seed(4)
    q, k, v = synth.video_like(g, 7, 1, text_pre=512, frames=22, frame_tokens=256, text_post=256)
    q, k, v = q.bfloat16(), k.bfloat16(), v.bfloat16()
    assert q.shape[2] == 6400
    _check_workload(q, k, v, 16, 0.9, 4096, True)


def test_dit_like_workload_non_causal_padded():
    """HunyuanVideo-style full attention: non-causal, S=8, threshold 0.95, zero-padded keys take softmax mass
    as in the reference."""
    from xattn_b200 import synth
    g = torch.Generator().manual_seed(6)
    q, k, v = synth.dit_like(g, 3, frames=3, rows=20, cols=32, text_tokens=256)
    q, k, v = q.bfloat16(), k.bfloat16(), v.bfloat16()
    assert q.shape[2] == 2176
    _check_workload(q, k, v, 8, 0.95, 2048, False)


def test_prefill_dense_threshold_one_matches_sdpa():
    """threshold=1 keeps every causal block with mass: the op must equal dense causal attention
    (size-independent property, no oracle involved)."""
    import xattn_b200
    g = torch.Generator().manual_seed(2)
    L = 2048
    q = torch.randn(1, 2, L, 128, generator=g).bfloat16().to(DEV)
    k = torch.randn(1, 2, L, 128, generator=g).bfloat16().to(DEV)
    v = torch.randn(1, 2, L, 128, generator=g).bfloat16().to(DEV)
    xattn_b200.set_estimate_semantics("triton")      # every past block carries mass under these semantics
    try:
        out = xattn_b200.Xattention_prefill(q, k, v, 8, threshold=1.0, chunk_size=2048, causal=True)
    finally:
        xattn_b200.set_estimate_semantics("torch")
    ref = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float(), is_causal=True)
    err = (out.float() - ref).abs()
    assert err.max() < OUT_MAX_ABS and err.mean() < OUT_MEAN_ABS, (err.max(), err.mean())


def test_host_pipeline_equals_device_call():
    """Xattention_prefill_host (pinned host tensors, kv groups streamed over PCIe) gives the result of the
    device call."""
    import xattn_b200
    from xattn_b200 import synth
    q, k, v, w = synth.make_inputs("llama3_8b_32k", seed=5, heads_limit=3, seq_len=4096)
    ref = xattn_b200.Xattention_prefill(q.to(DEV), k.to(DEV), v.to(DEV), 8, threshold=0.9, chunk_size=2048)
    for gps in (1, 2):
        out = xattn_b200.Xattention_prefill_host(q.pin_memory(), k.pin_memory(), v.pin_memory(), 8, threshold=0.9,
                                                 chunk_size=2048, groups_per_step=gps)
        assert not out.is_cuda and out.shape == q.shape
        _assert_same_up_to_body_choice(out, ref.cpu())


def test_head_shards_concatenate_to_the_full_result():
    """Two ranks' head shards, computed one after the other on this GPU, equal the unsharded call."""
    import xattn_b200
    from xattn_b200 import synth
    from xattn_b200.sharding import prefill_sharded
    q, k, v, w = synth.make_inputs("llama3_8b_32k", seed=6, heads_limit=2, seq_len=4096)
    dq, dk, dv = q.to(DEV), k.to(DEV), v.to(DEV)
    thr = torch.linspace(0.6, 0.95, q.shape[1])
    full = xattn_b200.Xattention_prefill(dq, dk, dv, 8, threshold=thr, chunk_size=2048)
    for world in (2, 4):
        parts = [prefill_sharded(dq, dk, dv, xattn_b200.Xattention_prefill, world, r, threshold=thr, stride=8,
                                 chunk_size=2048) for r in range(world)]
        _assert_same_up_to_body_choice(torch.cat(parts, dim=1), full)


def test_query_chunk_shards_equal_the_full_call():
    """Causal prefill cut into query chunks (as dealt to ranks for very long sequences), each computed
    against the keys up to its own end, reproduces the single call."""
    import xattn_b200
    from xattn_b200 import synth
    from xattn_b200.sharding import prefill_query_chunk_sharded
    q, k, v, w = synth.make_inputs("llama3_8b_128k", seed=9, heads_limit=1, seq_len=8192)
    dq, dk, dv = q.to(DEV), k.to(DEV), v.to(DEV)
    full = xattn_b200.Xattention_prefill(dq, dk, dv, 16, threshold=0.9, chunk_size=2048)
    for world in (2, 4):
        for r in range(world):
            parts = prefill_query_chunk_sharded(dq, dk, dv, xattn_b200.Xattention_prefill, world, r, 2048,
                                                threshold=0.9, stride=16)
            for c, o in parts.items():
                _assert_same_up_to_body_choice(o, full[:, :, c * 2048:(c + 1) * 2048], msg=str((world, r, c)))
    # pieces of two estimate chunks each (fewer, larger launches per rank)
    for r in range(2):
        parts = prefill_query_chunk_sharded(dq, dk, dv, xattn_b200.Xattention_prefill, 2, r, 2048, threshold=0.9,
                                            shard_rows=4096, stride=16)
        assert sorted(parts) == [r]
        for c, o in parts.items():
            _assert_same_up_to_body_choice(o, full[:, :, c * 4096:(c + 1) * 4096], msg=str(("rows 4096", r, c)))


def test_prefill_against_a_longer_key_cache():
    """q shorter than k (chunked prefill against a cache): masks vs the oracle, outputs vs the oracle's
    attention under the GPU mask, queries aligned to the end of the keys."""
    import xattn_b200
    from xattn_b200 import synth
    g = torch.Generator().manual_seed(12)
    Lq, Lk = 2048, 6144
    q, k, v = synth.llama_like(g, 4, 2, Lk)
    q = q[:, :, Lk - Lq:].contiguous().bfloat16()
    k, v = k.bfloat16(), v.bfloat16()
    sums, mask = xattn_b200.xattn_estimate(q.to(DEV), k.to(DEV), 128, 16, threshold=0.9, chunk_size=2048, causal=True)
    osums, omask = orc.xattn_estimate_oracle(q.float(), k.float().repeat_interleave(2, 1), 128, 16, 1.0, 0.9, 2048, True)
    ex = orc.margin_exempt(osums, Lq, Lk, 128, 16, 2048, 0.9, True)
    d = (mask.cpu() != omask) & ~ex
    assert not d.any(), d.nonzero()[:6].tolist()
    out = xattn_b200.Xattention_prefill(q.to(DEV), k.to(DEV), v.to(DEV), 16, threshold=0.9, chunk_size=2048, causal=True)
    ref = orc.block_sparse_attention_oracle(q, k, v, mask.cpu()[:, :, : Lq // 128, : Lk // 128], True)
    err = (out.float().cpu() - ref).abs()
    assert err.max() < OUT_MAX_ABS and err.mean() < OUT_MEAN_ABS, (err.max(), err.mean())


def test_llama_attention_core_prefill_decode_and_gqa():
    """The Llama integration core: prefill equals Xattention_prefill on repeated K/V with the layer's per-head
    thresholds; decode (one query against the cache) and the dense metric equal SDPA."""
    import xattn_b200
    from xattn_b200 import synth
    from xattn_b200.llama_shim import FastPrefillConfig, attention_core
    q, k, v, w = synth.make_inputs("llama3_8b_32k", seed=13, heads_limit=2, seq_len=4096)
    dq, dk, dv = q.to(DEV), k.to(DEV), v.to(DEV)
    table = torch.rand(3, 8) * 0.4 + 0.55
    cfg = FastPrefillConfig(threshold=table, stride=8)
    got = attention_core(dq, dk, dv, 1, cfg)
    want = xattn_b200.Xattention_prefill(dq, dk.repeat_interleave(4, 1), dv.repeat_interleave(4, 1), 8,
                                         threshold=table[1].to(DEV))
    assert torch.equal(got, want)
    # decode step: the newest query against all keys
    o = attention_core(dq[:, :, -1:], dk, dv, 0, cfg)
    ref = torch.nn.functional.scaled_dot_product_attention(dq[:, :, -1:].float(), dk.float().repeat_interleave(4, 1),
                                                           dv.float().repeat_interleave(4, 1))
    assert (o.float() - ref).abs().max() < OUT_MAX_ABS
    full = attention_core(dq, dk, dv, 0, FastPrefillConfig(metric="full"))
    ref = torch.nn.functional.scaled_dot_product_attention(dq.float(), dk.float().repeat_interleave(4, 1),
                                                           dv.float().repeat_interleave(4, 1), is_causal=True)
    err = (full.float() - ref).abs()
    assert err.max() < OUT_MAX_ABS and err.mean() < OUT_MEAN_ABS


def test_llama_attention_patch_matches_the_unpatched_model_at_threshold_one():
    """A small random-weight Hugging Face Llama (2 layers, 4 query / 2 kv heads of 128) with every attention module
    patched (projections, in-place RoPE, cache update, XAttention prefill, dense decode, o_proj): at threshold 1
    the selection keeps every causal block, so prefill and a following decode step must reproduce the unpatched
    model (SDPA attention) up to 16-bit rounding."""
    transformers = pytest.importorskip("transformers")
    from transformers import LlamaConfig, LlamaModel
    from transformers.cache_utils import DynamicCache
    from xattn_b200.llama_shim import FastPrefillConfig, patch_llama_attention
    cfg = LlamaConfig(vocab_size=128, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_position_embeddings=4096,
                      rope_theta=500000.0, attn_implementation="sdpa")
    torch.manual_seed(0)
    model = LlamaModel(cfg).to(device=DEV, dtype=torch.bfloat16).eval()
    L = 1024
    ids = torch.randint(0, 128, (1, L + 1), device=DEV)
    with torch.no_grad():
        ref_cache = DynamicCache(config=cfg)
        ref_pre = model(input_ids=ids[:, :L], past_key_values=ref_cache, use_cache=True).last_hidden_state
        ref_dec = model(input_ids=ids[:, L:], past_key_values=ref_cache, use_cache=True).last_hidden_state
        n = patch_llama_attention(model, FastPrefillConfig(threshold=1.0, stride=8, num_layers=2, num_heads=4,
                                                           device=DEV))
        assert n == 2
        cache = DynamicCache(config=cfg)
        got_pre = model(input_ids=ids[:, :L], past_key_values=cache, use_cache=True).last_hidden_state
        got_dec = model(input_ids=ids[:, L:], past_key_values=cache, use_cache=True).last_hidden_state
    import xattn_b200
    xattn_b200.check_device_status()
    for got, ref in ((got_pre, ref_pre), (got_dec, ref_dec)):
        err = (got.float() - ref.float()).abs()
        scale = ref.float().abs().mean()
        assert err.mean() < 0.02 * scale and err.max() < 0.25 * ref.float().abs().max(), (err.mean(), err.max(), scale)


def test_dit_varlen_wrapper_ragged_lengths():
    """The video-diffusion call pattern: a valid segment whose length is no multiple of 128 (or of the stride)
    through non-causal XAttention, a padded text tail dense; threshold >= 1 switches the first to dense."""
    from xattn_b200 import synth
    from xattn_b200.dit_shim import xattn_varlen_attention
    g = torch.Generator().manual_seed(21)
    q, k, v = synth.dit_like(g, 2, frames=2, rows=20, cols=32, text_tokens=256, pad_to=1)
    valid = 1280 + 75                       # image tokens + 75 real text tokens
    q, k, v = q.bfloat16().to(DEV), k.bfloat16().to(DEV), v.bfloat16().to(DEV)
    total = q.shape[2]
    cu = torch.tensor([0, valid, total], dtype=torch.int32)
    dense = xattn_varlen_attention(q, k, v, cu, cu, threshold=1.0)
    ref = torch.cat([
        torch.nn.functional.scaled_dot_product_attention(q[:, :, :valid].float(), k[:, :, :valid].float(), v[:, :, :valid].float()),
        torch.nn.functional.scaled_dot_product_attention(q[:, :, valid:].float(), k[:, :, valid:].float(), v[:, :, valid:].float())], 2)
    err = (dense.float() - ref).abs()
    assert dense.shape == q.shape and err.max() < OUT_MAX_ABS and err.mean() < OUT_MEAN_ABS
    sparse = xattn_varlen_attention(q, k, v, cu, cu, threshold=0.95, stride=8)
    # the tail is dense in both; the valid part must equal the oracle's attention under the oracle-checked mask
    assert torch.equal(sparse[:, :, valid:], dense[:, :, valid:])
    qc, kc, vc = q[:, :, :valid].cpu(), k[:, :, :valid].cpu(), v[:, :, :valid].cpu()
    chunk = orc.default_chunk_size(valid)
    _, omask = orc.xattn_estimate_oracle(qc.float(), kc.float(), 128, 8, 1.0, 0.95, chunk, False)
    import xattn_b200
    _, gmask = xattn_b200.xattn_estimate(q[:, :, :valid].contiguous(), k[:, :, :valid].contiguous(), 128, 8,
                                         threshold=0.95, chunk_size=chunk, causal=False)
    assert int((gmask.cpu() != omask).sum()) <= max(2, int(5e-3 * omask.numel()))
    refs = orc.block_sparse_attention_oracle(qc, kc, vc, gmask.cpu(), False)
    err = (sparse[:, :, :valid].float().cpu() - refs).abs()
    assert err.max() < OUT_MAX_ABS and err.mean() < OUT_MEAN_ABS, (err.max(), err.mean())


def test_dit_varlen_wrapper_makes_no_copies_of_its_inputs():
    """At a length where copies would show (30K tokens, 4 heads: q, k, v 31 MB each): the peak device memory of
    the call stays below the result plus the estimate's own scratch; contiguous copies of the three segments and a
    concatenation of the outputs would add four times the size of q."""
    from xattn_b200.dit_shim import xattn_varlen_attention
    g = torch.Generator(device=DEV).manual_seed(3)
    total, valid, H = 30000 + 77, 30000 - 13, 4
    q, k, v = (torch.randn(1, H, total, 128, generator=g, device=DEV).bfloat16() for _ in range(3))
    q[:, :, :256] += 4.0                            # a few strong keys, so that the selection stays sparse
    k[:, :, :256] += 4.0
    cu = torch.tensor([0, valid, total], dtype=torch.int32)
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    out = xattn_varlen_attention(q, k, v, cu, cu, threshold=0.9, stride=8)
    torch.cuda.synchronize()
    qbytes = q.numel() * q.element_size()
    extra = torch.cuda.max_memory_allocated() - base
    # result (1x) + partial sums of the non-causal estimate (rows x key blocks, fp32: 4 heads x 4096 x 256 x 4 B =
    # 16 MB) + block sums, lists and the staged ragged tiles (a few MB)
    assert extra < qbytes + 16 * (1 << 20) + 12 * (1 << 20), (extra, qbytes)
    assert out.shape == q.shape and torch.isfinite(out.float()).all()
    ref = torch.nn.functional.scaled_dot_product_attention(q[:, :, valid:], k[:, :, valid:], v[:, :, valid:])
    assert (out[:, :, valid:].float() - ref.float()).abs().max() < OUT_MAX_ABS


def test_rotary_embedding_matches_reference_fixture_bit_for_bit():
    import xattn_b200
    from xattn_b200 import ops
    from make_golden import rope_inputs
    z, specs = _load("rope.npz")
    for i, spec in enumerate(specs):
        q, k, cos, sin = rope_inputs(spec)
        # device copies that keep the [B, L, H, D] storage behind the [B, H, L, D] views
        qd = q.transpose(1, 2).contiguous().to(DEV).transpose(1, 2)
        kd = k.transpose(1, 2).contiguous().to(DEV).transpose(1, 2)
        ops.apply_rotary_pos_emb_(qd, kd, cos.to(DEV), sin.to(DEV))
        xattn_b200.check_device_status()
        assert np.array_equal(qd.cpu().contiguous().view(torch.int16).numpy(), z[f"q_{i}"]), spec
        assert np.array_equal(kd.cpu().contiguous().view(torch.int16).numpy(), z[f"k_{i}"]), spec


def _rope_table(L, D, dtype):
    ang = torch.arange(L).float()[:, None] / (500000.0 ** (torch.arange(0, D, 2).float() / D))[None, :]
    emb = torch.cat((ang, ang), -1)[None]                                 # [1, L, D]: one table for the batch
    return emb.cos().to(dtype), emb.sin().to(dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_rotary_embedding_vs_oracle_larger_and_shared_table(dtype):
    from xattn_b200 import ops
    g = torch.Generator().manual_seed(77)
    B, Hq, Hkv, L, D = 2, 8, 2, 1000, 128
    q = torch.randn(B, L, Hq, D, generator=g).to(dtype).transpose(1, 2)
    k = torch.randn(B, L, Hkv, D, generator=g).to(dtype).transpose(1, 2)
    cos, sin = _rope_table(L, D, dtype)
    want_q, want_k = orc.apply_rotary_pos_emb_oracle(q, k, cos, sin)
    qd = q.transpose(1, 2).contiguous().to(DEV).transpose(1, 2)
    kd = k.transpose(1, 2).contiguous().to(DEV).transpose(1, 2)
    ops.apply_rotary_pos_emb_(qd, kd, cos.to(DEV), sin.to(DEV))
    assert torch.equal(qd.cpu(), want_q) and torch.equal(kd.cpu(), want_k)
    # contiguous [B, H, L, D] storage works as well
    qc, kc = q.contiguous().to(DEV), k.contiguous().to(DEV)
    ops.apply_rotary_pos_emb_(qc, kc, cos.to(DEV), sin.to(DEV))
    assert torch.equal(qc.cpu(), want_q) and torch.equal(kc.cpu(), want_k)


def test_llama_rope_and_attend_equals_the_composed_reference_steps():
    import xattn_b200
    from xattn_b200 import llama_shim, synth
    L = 2048
    q, k, v, w = synth.make_inputs("llama3_8b_32k", seed=5, heads_limit=2, seq_len=L)
    B, Hq, _, D = q.shape
    Hkv = k.shape[1]
    # projection outputs [B, L, H*D]
    qp = q.transpose(1, 2).reshape(B, L, Hq * D).contiguous().to(DEV)
    kp = k.transpose(1, 2).reshape(B, L, Hkv * D).contiguous().to(DEV)
    vp = v.transpose(1, 2).reshape(B, L, Hkv * D).contiguous().to(DEV)
    cos, sin = _rope_table(L, D, q.dtype)
    cfg = llama_shim.FastPrefillConfig(threshold=0.9, stride=8, num_layers=1, num_heads=Hq, device=DEV)
    # the reference's sequence of steps, each on its own tensors
    q_ref, k_ref = orc.apply_rotary_pos_emb_oracle(q, k, cos, sin)
    want = llama_shim.attention_core(q_ref.to(DEV), k_ref.to(DEV), v.to(DEV), 0, cfg)
    want = want.transpose(1, 2).contiguous().reshape(B, L, Hq * D)
    got = llama_shim.rope_and_attend(qp, kp, vp, cos.to(DEV), sin.to(DEV), Hq, Hkv, 0, cfg)
    xattn_b200.check_device_status()
    assert got.shape == (B, L, Hq * D) and got.is_contiguous()
    assert torch.equal(got, want)
    assert torch.equal(kp.view(B, L, Hkv, D).transpose(1, 2).cpu(), k_ref)     # rotated keys left for the cache


@pytest.mark.parametrize("name,L,Lq,chunk", [("llama3_8b_32k", 8192, 8192, 2048), ("llama3_8b_128k", 8192, 8192, 2048),
                                             ("llama3_8b_32k", 8192, 4096, 4096), ("llama3_8b_32k", 6144, 6144, 2048),
                                             ("llama3_8b_128k", 8192, 4096, 2048), ("llama3_8b_128k", 10240, 2048, 2048)])
def test_chunk_band_layout_equals_the_dense_one(name, L, Lq, chunk):
    """Un-padded causal keys under the torch branch: the sums kept as a chunk-wide band, and the selection run
    on the band, give the dense layout's sums, mask and block lists.  The sums are bit-identical except where a
    chunk is a single 128x128 tile (stride 16, chunk 2048): there the band layout's block sums are finished in the
    GEMM's epilogue, which adds the rows of a query block in another order (agreement to the last few bits)."""
    from xattn_b200 import ops, synth
    q, k, v, w = synth.make_inputs(name, seed=11, heads_limit=1, seq_len=L)
    q, k = q[:, :, L - Lq:].to(DEV), k.to(DEV)
    assert ops.band_applies(L, chunk, True)
    g = ops.geometry(Lq, L, chunk, w.stride)
    dense = ops.estimate_block_sums(q, k, w.stride, 128, chunk, 1.0, True)
    band = ops.estimate_block_sums(q, k, w.stride, 128, chunk, 1.0, True, band=True)
    assert band.shape == (1, q.shape[1], g["qb"], g["bpc"])
    rebuilt = torch.zeros_like(dense)
    for c in range(g["qb"] // g["bpc"]):
        cur = g["block_offset"] + c * g["bpc"]
        rows = slice(c * g["bpc"], (c + 1) * g["bpc"])
        rebuilt[:, :, rows, cur:cur + g["bpc"]] = band[:, :, rows]
    if chunk // w.stride == 128:
        torch.testing.assert_close(rebuilt, dense, rtol=2e-6, atol=0.0)
        assert torch.equal(rebuilt == 0, dense == 0)
        dense = rebuilt                      # the selection is compared on the same numbers in both layouts
    else:
        assert torch.equal(rebuilt, dense)
    for thr, sink, recent in ((0.9, False, False), (torch.linspace(0.5, 1.0, q.shape[1]), False, False),
                              (0.7, True, True), (0.0, False, True), (1.0, True, False)):
        m0, i0, c0 = ops.select_blocks(dense, g["bpc"], g["block_offset"], thr, True, True, sink, recent,
                                       list_shape=(Lq, L))
        m1, i1, c1 = ops.select_blocks(band, g["bpc"], g["block_offset"], thr, True, True, sink, recent,
                                       list_shape=(Lq, L), band_k_blocks=g["kb"])
        assert torch.equal(m0, m1) and torch.equal(c0, c1)
        valid = torch.arange(i0.shape[-1], device=DEV)[None, None, None, :] < c0[..., None]
        assert torch.equal(i0[valid], i1[valid])


def test_runs_are_bit_identical():
    """Same inputs, two runs: identical bits (no race between the roles of a CTA)."""
    import xattn_b200
    from xattn_b200 import synth
    q, k, v, w = synth.make_inputs("llama3_8b_32k", seed=8, heads_limit=1, seq_len=4096)
    a = xattn_b200.Xattention_prefill(q.to(DEV), k.to(DEV), v.to(DEV), 8, threshold=0.9, chunk_size=2048)
    b = xattn_b200.Xattention_prefill(q.to(DEV), k.to(DEV), v.to(DEV), 8, threshold=0.9, chunk_size=2048)
    assert torch.equal(a, b)


def test_bad_arguments_raise_before_launch():
    import xattn_b200
    from xattn_b200._lib import XattnB200Error
    q = torch.zeros(1, 2, 256, 128, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ValueError):
        xattn_b200.xattn_estimate(q, q, 128, 16, kdb=2)
    with pytest.raises(NotImplementedError):
        xattn_b200.xattn_estimate(q, q, 128, 16, select_mode="slash")
    with pytest.raises((XattnB200Error, ValueError)):
        xattn_b200.xattn_estimate(q, q, 128, 3)
    with pytest.raises(AssertionError):
        xattn_b200.Xattention_prefill(torch.cat([q, q]), torch.cat([q, q]), torch.cat([q, q]), 16)
