"""Multi-GPU sharding of the prefill path: one process per GPU, no collective on the data path.

Every (batch, kv-head group) is independent in all three phases (estimate, selection, attention), so a
layer is split across ranks by whole kv-head groups: rank r owns a contiguous range of kv heads and the
query heads that read them, runs the unchanged single-GPU path on its slice and keeps its slice of the
output.  A collective (all_gather of the outputs) is only needed if the caller wants the full tensor on
every rank.  The reference has no multi-GPU code for this path; nothing here mirrors a reference file.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch


def shard_kv_groups(hq: int, hkv: int, world_size: int, rank: int) -> Tuple[int, int, int, int]:
    """(q_head_start, q_head_end, kv_head_start, kv_head_end) owned by `rank`.

    kv groups are dealt out as evenly as possible, the first `hkv % world_size` ranks get one more.  When
    there are more ranks than kv groups, a group's query heads are split over several ranks (each of them
    then needs that group's K/V) so that no rank idles while hq >= world_size."""
    if hq % hkv != 0:
        raise ValueError("hq must be a multiple of hkv")
    rep = hq // hkv
    if world_size <= hkv:
        base, extra = divmod(hkv, world_size)
        k0 = rank * base + min(rank, extra)
        k1 = k0 + base + (1 if rank < extra else 0)
        return k0 * rep, k1 * rep, k0, k1
    # more ranks than groups: split query heads, round-robin over groups
    base, extra = divmod(hq, world_size)
    q0 = rank * base + min(rank, extra)
    q1 = q0 + base + (1 if rank < extra else 0)
    if q1 <= q0:
        return q0, q0, 0, 0
    k0, k1 = q0 // rep, (q1 - 1) // rep + 1
    return q0, q1, k0, k1


def all_shards(hq: int, hkv: int, world_size: int) -> List[Tuple[int, int, int, int]]:
    return [shard_kv_groups(hq, hkv, world_size, r) for r in range(world_size)]


def prefill_sharded(query_states: torch.Tensor, key_states: torch.Tensor, value_states: torch.Tensor,
                    prefill_fn: Callable[..., torch.Tensor], world_size: int, rank: int,
                    threshold=0.8, gather: bool = False, group=None, **kwargs) -> torch.Tensor:
    """Run `prefill_fn(q, k, v, threshold=..., **kwargs)` on this rank's head slice of full tensors
    q [B,Hq,L,D], k/v [B,Hkv,L,D].  Returns the slice's output [B,hq_local,L,D]; with gather=True the full
    [B,Hq,L,D] is assembled on every rank with one all_gather per rank slice size class."""
    hq, hkv = query_states.shape[1], key_states.shape[1]
    rep = hq // hkv
    q0, q1, k0, k1 = shard_kv_groups(hq, hkv, world_size, rank)
    if q1 > q0:
        # K/V heads needed by the local query heads; when a group is split the local q heads still index
        # kv heads relative to k0, which needs hq_local to be a multiple of the local kv heads: repeat-free
        # only for whole groups, otherwise the few K/V heads are expanded to one per query head
        q = query_states[:, q0:q1]
        if (q1 - q0) % (k1 - k0) == 0 and q0 == k0 * rep and q1 == k1 * rep:
            k, v = key_states[:, k0:k1], value_states[:, k0:k1]
        else:
            idx = torch.arange(q0, q1, device=key_states.device) // rep
            k, v = key_states[:, idx], value_states[:, idx]
        thr = threshold[q0:q1] if isinstance(threshold, torch.Tensor) else threshold
        local = prefill_fn(q, k, v, threshold=thr, **kwargs)
    else:
        local = query_states[:, :0]
    if not gather:
        return local
    import torch.distributed as dist
    shards = all_shards(hq, hkv, world_size)
    width = max(s[1] - s[0] for s in shards)
    B, _, L, D = query_states.shape
    pad = torch.zeros(B, width, L, D, dtype=local.dtype, device=local.device)
    pad[:, : local.shape[1]] = local
    parts = [torch.empty_like(pad) for _ in range(world_size)]
    dist.all_gather(parts, pad.contiguous(), group=group)
    return torch.cat([p[:, : s[1] - s[0]] for p, s in zip(parts, shards)], dim=1)


# ----------------------------------------------------------------------------------------------------------
# Query-chunk sharding for sequences whose heads alone do not give enough parallelism (or whose K/V must be
# replicated anyway): causal prefill only.
# ----------------------------------------------------------------------------------------------------------
def shard_query_chunks(n_chunks: int, world_size: int, rank: int) -> List[int]:
    """Chunk indices owned by `rank`, dealt zig-zag (0,1,..,W-1,W-1,..,1,0,0,1,..) so that the causal work
    (chunk c attends to c+1 chunks of keys) is balanced across ranks."""
    out = []
    for c in range(n_chunks):
        lap, pos = divmod(c, world_size)
        owner = pos if lap % 2 == 0 else world_size - 1 - pos
        if owner == rank:
            out.append(c)
    return out


def prefill_query_chunk_sharded(query_states: torch.Tensor, key_states: torch.Tensor, value_states: torch.Tensor,
                                prefill_fn: Callable[..., torch.Tensor], world_size: int, rank: int, chunk_size: int,
                                threshold=0.8, broadcast_kv_from: Optional[int] = None, group=None,
                                shard_rows: Optional[int] = None, **kwargs):
    """Causal prefill with the QUERY axis cut into pieces that are dealt to the ranks; every rank needs all of
    K and V (one collective: `broadcast_kv_from` = source rank broadcasts them, NCCL over NVLink on GPUs),
    kernels then read local memory only.

    A piece is `shard_rows` query rows (a multiple of the estimate's `chunk_size`; default: one chunk).  Piece c
    is computed exactly by the unchanged single-GPU call on q[piece c] against k/v[: end of piece c] (queries
    aligned to the end of the keys, which is the layout the path already supports for prefill against a cache):
    same block offsets, same first-chunk rule, same normalisation as in the one-GPU run.  Larger pieces mean
    fewer, larger launches per rank.  Returns {piece index: output [B,Hq,rows,D]} for the local pieces.
    q_len must equal k_len and be a multiple of shard_rows."""
    if broadcast_kv_from is not None:
        import torch.distributed as dist
        dist.broadcast(key_states, src=broadcast_kv_from, group=group)
        dist.broadcast(value_states, src=broadcast_kv_from, group=group)
    rows = chunk_size if shard_rows is None else int(shard_rows)
    L = query_states.shape[2]
    if rows % chunk_size != 0:
        raise ValueError("shard_rows must be a multiple of chunk_size")
    if key_states.shape[2] != L or L % rows != 0:
        raise ValueError("query-chunk sharding needs q_len == k_len, a multiple of the piece length")
    out = {}
    for c in shard_query_chunks(L // rows, world_size, rank):
        r0, r1 = c * rows, (c + 1) * rows
        out[c] = prefill_fn(query_states[:, :, r0:r1], key_states[:, :, :r1], value_states[:, :, :r1],
                            threshold=threshold, chunk_size=chunk_size, causal=True, **kwargs)
    return out
