"""xattn_b200_estimate_static -- the estimate for callers that may not allocate device memory.

Some users of the library cannot call cudaMalloc where they run the estimate (their GPU memory belongs
to a pool set up at start-up, or an allocation's implicit synchronisation is unacceptable there).  For
them the library carries a fixed scratch array of its own.  This test drives that entry point through
the C ABI exactly as such a caller would -- inputs and output only -- and checks it against the regular
entry point (which gets its workspace from the caller), twice in a row because the second call finds
the scratch full of the first call's data.  It is collected last on purpose and must pass both on its
own in a fresh process and after every other test.
"""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_static(lib, q, k, stride, chunk, causal, sums, status):
    B, H, L, D = q.shape
    return lib.xattn_b200_estimate_static(
        q.data_ptr(), k.data_ptr(), 0, B, H, k.shape[1], L, k.shape[2], D,
        q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
        stride, 128, chunk, 1.0 / math.sqrt(D) / stride, int(causal), 0,
        sums.data_ptr(), status.data_ptr(), torch.cuda.current_stream().cuda_stream)


def test_static_scratch_estimate_matches_regular_estimate_twice():
    from xattn_b200 import _lib, ops, synth
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    status = torch.zeros(1, dtype=torch.int32).pin_memory()
    cases = [(4096, 16, 2048, True, 11), (2048, 8, 1024, False, 12)]   # second call: other shape, other data
    for L, stride, chunk, causal, seed in cases:
        gen = torch.Generator().manual_seed(seed)
        q, k, _ = synth.llama_like(gen, 4, 2, L)
        q, k = q.bfloat16().to(dev), k.bfloat16().to(dev)
        want = ops.estimate_block_sums(q, k, stride, 128, chunk, 1.0, causal, semantics="torch")
        got = torch.full_like(want, float("nan"))
        rc = _call_static(lib, q, k, stride, chunk, causal, got, status)
        assert rc == 0, lib.xattn_b200_error_string(rc)
        torch.cuda.synchronize()
        assert int(status[0]) == 0
        # same kernels, same inputs, different scratch memory: identical within the sums tolerance
        assert torch.allclose(got, want, rtol=2e-4, atol=2e-5), (got - want).abs().max()


def test_static_scratch_estimate_refuses_oversized_problems():
    from xattn_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    # 32 heads x 128K tokens, non-causal (every row keeps partial sums for all 1024 key blocks), needs ~1 GiB of
    # scratch: far beyond the built-in array, and refused before any pointer is touched
    assert lib.xattn_b200_estimate_workspace_bytes_ex(1, 32, 131072, 131072, 16, 128, 2048, 0, 0) > (32 << 20)
    dummy = torch.zeros(16, device=dev)
    rc = lib.xattn_b200_estimate_static(
        dummy.data_ptr(), dummy.data_ptr(), 0, 1, 32, 8, 131072, 131072, 128,
        0, 131072 * 128, 128, 0, 131072 * 128, 128, 16, 128, 2048, 0.01, 0, 0,
        dummy.data_ptr(), 0, torch.cuda.current_stream().cuda_stream)
    assert rc == 5 and b"maximum" in lib.xattn_b200_error_string(rc)
