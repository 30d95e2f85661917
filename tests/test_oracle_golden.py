"""The CPU oracle replayed against fixtures produced by the unmodified reference code
(tests/golden/make_golden.py).  No GPU, no reference checkout needed."""
import json
import os

import numpy as np
import pytest
import torch

from make_golden import attention_inputs, case_inputs, rope_inputs
from oracle import xattn_oracle as orc

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _load(name):
    z = np.load(os.path.join(GOLD, name))
    return z, json.loads(str(z["specs"]))


def _threshold(spec):
    t = spec["threshold"]
    return torch.tensor(t, dtype=torch.float32) if isinstance(t, list) else t


def _check_estimate(z, specs, i, semantics):
    spec = specs[i]
    q, k = case_inputs(spec)
    chk = float(q.double().sum() + 3.0 * k.double().sum())
    assert abs(chk - spec["checksum"]) <= 1e-6 * max(1.0, abs(chk)), "input generator drifted"
    sums, mask = orc.xattn_estimate_oracle(
        q.float(), k.float(), 128, spec["stride"], 1.0, _threshold(spec), spec["chunk"],
        spec["causal"], spec["keep_sink"], spec["keep_recent"], semantics=semantics)
    ref_sums = torch.from_numpy(z[f"sums_{i}"])
    shape = spec["mask_shape"]
    ref_mask = torch.from_numpy(
        np.unpackbits(z[f"mask_{i}"])[: int(np.prod(shape))].reshape(shape).astype(bool))
    assert sums.shape == ref_sums.shape
    # fp32 softmax sums: a block sums at most rbs rows of probabilities
    assert torch.allclose(sums, ref_sums, rtol=2e-5, atol=2e-6), (sums - ref_sums).abs().max()
    exempt = orc.margin_exempt(ref_sums, spec["q_len"], spec["k_len"], 128, spec["stride"],
                               spec["chunk"], _threshold(spec), spec["causal"])
    diff = (mask != ref_mask) & ~exempt
    assert not diff.any(), f"{int(diff.sum())} non-exempt mask mismatches, e.g. {diff.nonzero()[:5].tolist()}"
    return int((mask != ref_mask).sum())


_z_t, _specs_t = _load("estimate_torch_path.npz")


@pytest.mark.parametrize("i", range(len(_specs_t)))
def test_estimate_matches_reference_torch_path(i):
    _check_estimate(_z_t, _specs_t, i, "torch")


def test_exemptions_are_rare_on_torch_path():
    total = sum(_check_estimate(_z_t, _specs_t, i, "torch") for i in range(len(_specs_t)))
    cells = sum(int(np.prod(s["mask_shape"])) for s in _specs_t)
    assert total <= 1e-3 * cells, (total, cells)


@pytest.mark.skipif(not os.path.exists(os.path.join(GOLD, "estimate_triton_path.npz")),
                    reason="triton-interpreter fixtures not generated")
def test_estimate_matches_reference_triton_path():
    z, specs = _load("estimate_triton_path.npz")
    for i in range(len(specs)):
        _check_estimate(z, specs, i, "triton")


def test_selection_matches_find_blocks_chunked():
    z, specs = _load("find_blocks_chunked.npz")
    bad = 0
    for i, spec in enumerate(specs):
        x = torch.from_numpy(z[f"x_{i}"])
        ref = torch.from_numpy(z[f"mask_{i}"])
        thr = _threshold(spec)
        got = orc.select_blocks_chunk(x, spec["current_index"], thr, spec["causal"])
        ex = orc.margin_exempt_chunk(x, spec["current_index"], thr, spec["causal"])
        d = (got != ref) & ~ex
        bad += int(d.sum())
        assert not d.any(), (i, spec, d.nonzero()[:5].tolist())
    assert bad == 0


def test_default_chunk_rule():
    # Xattention.py:322-331
    for L, want in ((1000, 2048), (4096, 4096), (8192, 8192), (16384, 16384), (32768, 8192),
                    (62208, 4096), (65536, 4096), (119056, 2048), (131072, 2048), (262144, 2048)):
        assert orc.default_chunk_size(L) == want


def test_attention_oracle_dense_equals_sdpa():
    g = torch.Generator().manual_seed(3)
    q = torch.randn(1, 4, 300, 128, generator=g)
    k = torch.randn(1, 2, 300, 128, generator=g)
    v = torch.randn(1, 2, 300, 128, generator=g)
    mask = torch.ones(1, 4, 3, 3, dtype=torch.bool)
    for causal in (True, False):
        o = orc.block_sparse_attention_oracle(q, k, v, mask, causal=causal)
        ref = torch.nn.functional.scaled_dot_product_attention(
            q, k.repeat_interleave(2, 1), v.repeat_interleave(2, 1), is_causal=causal)
        assert torch.allclose(o, ref, atol=2e-5, rtol=1e-4)


def test_attention_oracle_matches_the_reference_blockwise_attention():
    """The attention oracle against outputs of the reference's own statement of causal block-sparse attention
    (xattn/src/Flexprefill.py:12-44, torch_block_wise_attention), fp32 on both sides."""
    z, specs = _load("attention_blockwise.npz")
    assert len(specs) >= 4
    for i, spec in enumerate(specs):
        q, k, v, m = attention_inputs(spec)
        chk = float(q.double().sum() + 3.0 * k.double().sum() + 5.0 * v.double().sum())
        assert abs(chk - spec["checksum"]) <= 1e-6 * max(1.0, abs(chk)), "input generator drifted"
        shape = spec["mask_shape"]
        ref_m = np.unpackbits(z[f"mask_{i}"])[: int(np.prod(shape))].reshape(shape).astype(bool)
        assert np.array_equal(m.numpy(), ref_m)
        o = orc.block_sparse_attention_oracle(q, k, v, m, causal=True)
        ref = torch.from_numpy(z[f"out_{i}"])
        assert (o[..., :: spec["col_step"]] - ref).abs().max() <= 1e-5, spec
        assert (o.double().sum(-1) - torch.from_numpy(z[f"rowsum_{i}"])).abs().max() <= 1e-4, spec


def test_rotary_embedding_oracle_matches_the_reference_function_bit_for_bit():
    z, specs = _load("rope.npz")
    assert len(specs) >= 3
    for i, spec in enumerate(specs):
        q, k, cos, sin = rope_inputs(spec)
        qe, ke = orc.apply_rotary_pos_emb_oracle(q, k, cos, sin)
        assert np.array_equal(qe.contiguous().view(torch.int16).numpy(), z[f"q_{i}"]), spec
        assert np.array_equal(ke.contiguous().view(torch.int16).numpy(), z[f"k_{i}"]), spec
