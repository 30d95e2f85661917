"""Head sharding across ranks, exercised as two gloo processes on the CPU: the shard plan covers every head
once, and running the path per shard (the CPU oracle stands in for the GPU op here) then gathering gives
exactly the unsharded result -- no collective is needed on the data path."""
import os
import sys

import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_plan_covers_all_heads_once():
    from xattn_b200.sharding import all_shards
    for hq, hkv in ((32, 8), (28, 4), (24, 24), (8, 8), (4, 1)):
        for world in (1, 2, 3, 4, 8):
            shards = all_shards(hq, hkv, world)
            cover = []
            rep = hq // hkv
            for q0, q1, k0, k1 in shards:
                cover += list(range(q0, q1))
                for h in range(q0, q1):
                    assert k0 <= h // rep < k1          # the kv head each local query head reads is local
            assert cover == list(range(hq)), (hq, hkv, world, shards)
            sizes = [s[1] - s[0] for s in shards]
            if world <= hkv:
                assert max(sizes) - min(sizes) <= rep   # whole groups, as even as possible


def test_host_pipeline_group_slices():
    from xattn_b200.host_pipeline import group_slices
    for hq, hkv, gps in ((32, 8, 1), (32, 8, 3), (28, 4, 2), (24, 24, 5)):
        sl = group_slices(hq, hkv, gps)
        assert [h for s in sl for h in range(s[0], s[1])] == list(range(hq))
        assert [h for s in sl for h in range(s[2], s[3])] == list(range(hkv))


def test_query_chunk_plan_is_balanced_and_complete():
    from xattn_b200.sharding import shard_query_chunks
    for n, world in ((128, 8), (64, 4), (7, 2), (5, 8)):
        owned = [shard_query_chunks(n, world, r) for r in range(world)]
        assert sorted(c for o in owned for c in o) == list(range(n))
        work = [sum(c + 1 for c in o) for o in owned]          # chunk c costs ~ c+1 key chunks
        if n % (2 * world) == 0:
            assert max(work) == min(work)


def _oracle_prefill(q, k, v, threshold, stride, chunk_size, causal):
    from oracle import xattn_oracle as orc
    rep = q.shape[1] // k.shape[1]
    _, mask = orc.xattn_estimate_oracle(q.float(), k.float().repeat_interleave(rep, 1), 128, stride, 1.0, threshold,
                                        chunk_size, causal)
    return orc.block_sparse_attention_oracle(q, k, v, mask, causal)


def _worker(rank, world, port, hq, hkv, ret):
    for p in (ROOT, os.path.join(ROOT, "x-attention_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch.distributed as dist
    from xattn_b200.sharding import prefill_sharded
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    g = torch.Generator().manual_seed(123)             # same full tensors on every rank
    L = 512
    q = torch.randn(1, hq, L, 128, generator=g)
    k = torch.randn(1, hkv, L, 128, generator=g)
    v = torch.randn(1, hkv, L, 128, generator=g)
    thr = torch.linspace(0.5, 0.95, hq)
    full = prefill_sharded(q, k, v, _oracle_prefill, world, rank, threshold=thr, gather=True,
                           stride=16, chunk_size=256, causal=True)
    want = _oracle_prefill(q, k, v, thr, 16, 256, True)
    ret[rank] = float((full - want).abs().max())
    dist.barrier()
    dist.destroy_process_group()


def _worker_qchunks(rank, world, port, ret):
    for p in (ROOT, os.path.join(ROOT, "x-attention_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch.distributed as dist
    from xattn_b200.sharding import prefill_query_chunk_sharded
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    g = torch.Generator().manual_seed(321)
    L, chunk = 1024, 256
    q = torch.randn(1, 2, L, 128, generator=g)             # every rank has its queries
    k = torch.randn(1, 2, L, 128, generator=g)
    v = torch.randn(1, 2, L, 128, generator=g)
    if rank != 0:                                          # K/V only exist on rank 0 until the broadcast
        k, v = torch.zeros_like(k), torch.zeros_like(v)
    parts = prefill_query_chunk_sharded(q, k, v, _oracle_prefill, world, rank, chunk, threshold=0.9,
                                        broadcast_kv_from=0, stride=16)
    g2 = torch.Generator().manual_seed(321)
    qf = torch.randn(1, 2, L, 128, generator=g2); kf = torch.randn(1, 2, L, 128, generator=g2); vf = torch.randn(1, 2, L, 128, generator=g2)
    want = _oracle_prefill(qf, kf, vf, 0.9, 16, chunk, True)
    err = 0.0
    for c, o in parts.items():
        err = max(err, float((o - want[:, :, c * chunk:(c + 1) * chunk]).abs().max()))
    ret[rank] = (sorted(parts), err)
    dist.barrier()
    dist.destroy_process_group()


def test_query_pieces_of_several_chunks_equal_the_full_call():
    """Pieces larger than one estimate chunk (shard_rows = 2 chunks): each piece, computed against the keys up to
    its own end, equals the rows of the single call (no process group needed: no broadcast is requested)."""
    from xattn_b200.sharding import prefill_query_chunk_sharded
    g = torch.Generator().manual_seed(55)
    L, chunk = 1024, 256
    q, k, v = (torch.randn(1, 2, L, 128, generator=g) for _ in range(3))
    want = _oracle_prefill(q, k, v, 0.9, 16, chunk, True)
    seen = []
    for rank in range(2):
        parts = prefill_query_chunk_sharded(q, k, v, _oracle_prefill, 2, rank, chunk, threshold=0.9,
                                            shard_rows=512, stride=16)
        for c, o in parts.items():
            seen.append(c)
            assert float((o - want[:, :, c * 512:(c + 1) * 512]).abs().max()) < 1e-5
    assert sorted(seen) == [0, 1]
    with pytest.raises(ValueError):
        prefill_query_chunk_sharded(q, k, v, _oracle_prefill, 2, 0, chunk, shard_rows=384, stride=16)


def test_query_chunk_sharding_with_kv_broadcast_gloo():
    port = 31500 + (os.getpid() % 2000)
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker_qchunks, args=(2, port, ret), nprocs=2, join=True)
    chunks = sorted(c for r in ret.values() for c in r[0])
    assert chunks == [0, 1, 2, 3]
    assert all(r[1] < 1e-5 for r in ret.values()), dict(ret)


@pytest.mark.parametrize("hq,hkv,world", [(8, 2, 2), (4, 1, 2)])
def test_sharded_equals_unsharded_gloo(hq, hkv, world):
    port = 29500 + (os.getpid() % 2000) + hq
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, hq, hkv, ret), nprocs=world, join=True)
    assert len(ret) == world
    assert all(err == 0.0 for err in ret.values()), dict(ret)


def test_host_pipeline_steps_keep_the_kv_head_mapping():
    """Every step of the host pipeline must map its local query heads to the right kv heads with the rule the
    kernels apply (local q head h -> local kv head h // (n_q / n_kv)), cover every head once, in order, and
    copy K/V exactly once per slice."""
    from xattn_b200.host_pipeline import plan_steps
    for hq, hkv in ((32, 8), (12, 3), (28, 4), (24, 24), (8, 1), (6, 2)):
        rep = hq // hkv
        for gps in (1, 2, 3):
            for splits, tail in ((0, 1), (1, 1), (2, 1), (4, 1), (1, 2), (1, 4), (2, 4)):
                steps = plan_steps(hq, hkv, gps, splits, tail)
                if tail > 1 and gps == 1 and rep % tail == 0:
                    # only the last slice is cut finer than the others
                    assert sum(1 for st in steps if st[2] == hkv - 1) == max(tail, splits if rep % max(splits, 1) == 0 else 1)
                seen = []
                firsts = 0
                for (q0, q1, k0, k1, first, last) in steps:
                    nq, nk = q1 - q0, k1 - k0
                    assert nq > 0 and nk > 0 and nq % nk == 0
                    for h in range(nq):
                        assert k0 + h // (nq // nk) == (q0 + h) // rep, (hq, hkv, gps, splits, tail, q0, h)
                    seen.extend(range(q0, q1))
                    firsts += int(first)
                assert seen == list(range(hq))
                assert firsts == (hkv + gps - 1) // gps


def test_default_thresholds_are_the_profiled_llama_tables():
    """FastPrefillConfig(threshold=None) takes the per-(layer, head) table of its stride, as the reference does
    (xattn/src/load_llama.py:253-261); the tables are data generated from xattn/threshold/llama_threshold.py."""
    from xattn_b200.llama_shim import FastPrefillConfig, default_threshold_table
    means = {4: 0.79205, 8: 0.76135, 16: 0.90738}
    for stride, mean in means.items():
        t = FastPrefillConfig(threshold=None, stride=stride, device="cpu").threshold
        assert t.shape == (32, 32) and t.dtype == torch.float32
        assert abs(float(t.mean()) - mean) < 1e-4 and 0.0 <= float(t.min()) and float(t.max()) <= 1.0
        assert torch.equal(t, default_threshold_table(stride))
    with pytest.raises(ValueError):
        default_threshold_table(32)
    assert float(FastPrefillConfig(threshold=0.9, device="cpu").threshold.mean()) == pytest.approx(0.9)
