"""Xattention_prefill for inputs that live in (pinned) host memory.

Every (batch, kv-head group) of the path is independent, so the call is cut into kv-head groups and the
three engines of the GPU work at the same time: while group g is computed, the q/k/v of group g+1 come
in over PCIe and the output of group g-1 goes back (PCIe is full duplex).  Two device buffer sets rotate;
all ordering is by CUDA events, the host thread does not block until the final wait.

The reference has no counterpart (its callers hand over device tensors); this is the end-to-end path the
benchmark times with host buffers.
"""
from __future__ import annotations

from typing import Optional, Union

import torch

from . import ops

_copy_streams = {}


def bind_host_to_gpu(device: Union[int, str, torch.device]) -> Optional[list]:
    """Restrict the calling process to the CPU cores next to `device` (NVML's CPU affinity of that GPU), so that
    host buffers allocated and first touched afterwards sit on the GPU's NUMA node and copies over PCIe do not
    cross the socket interconnect.  One process per GPU should call this before it allocates pinned memory.
    Changes nothing on the GPU.  Returns the core list, or None when the affinity cannot be read."""
    import os
    dev = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)
    try:
        import pynvml
        pynvml.nvmlInit()
        uuid = str(torch.cuda.get_device_properties(dev).uuid)
        handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode() if not uuid.startswith("GPU-") else uuid.encode())
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        cpus = [64 * i + b for i, m in enumerate(mask) for b in range(64) if (int(m) >> b) & 1]
        allowed = sorted(set(cpus) & set(os.sched_getaffinity(0)))
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return allowed
    except Exception:                                   # no NVML, no such call, container without the cores
        return None


def _streams(device: torch.device):
    key = device.index
    s = _copy_streams.get(key)
    if s is None:
        s = (torch.cuda.Stream(device), torch.cuda.Stream(device))
        _copy_streams[key] = s
    return s


def group_slices(hq: int, hkv: int, groups_per_step: int = 1):
    """[(q_head_start, q_head_end, kv_head_start, kv_head_end)] covering all heads, kv groups kept whole."""
    rep = hq // hkv
    out = []
    for g0 in range(0, hkv, groups_per_step):
        g1 = min(hkv, g0 + groups_per_step)
        out.append((g0 * rep, g1 * rep, g0, g1))
    return out


def plan_steps(hq: int, hkv: int, groups_per_step: int = 1, q_splits: int = 1, tail_splits: int = 1):
    """Steps of the host pipeline: [(q0, q1, k0, k1, first_of_slice, last_of_slice)].  A slice is `groups_per_step`
    whole kv groups (its K/V are copied with its first step); the query heads of a slice that holds ONE kv head
    run in `q_splits` steps when that divides them, those of the LAST slice in `tail_splits` steps (what follows
    the last input copy -- the last step's kernels and its output copy -- overlaps with nothing, so that step
    should be small).  A slice with several kv heads is never split: the kernels map local query head h to local
    kv head h // (query heads / kv heads), which a partial slice would break."""
    steps = []
    slices = group_slices(hq, hkv, groups_per_step)
    for si, (q0, q1, k0, k1) in enumerate(slices):
        n = q1 - q0
        want = max(q_splits, tail_splits) if si == len(slices) - 1 else q_splits
        parts = want if (want > 0 and k1 - k0 == 1 and n % want == 0) else 1
        for j in range(parts):
            steps.append((q0 + j * (n // parts), q0 + (j + 1) * (n // parts), k0, k1, j == 0, j == parts - 1))
    return steps


def Xattention_prefill_host(query_states: torch.Tensor, key_states: torch.Tensor, value_states: torch.Tensor,
                            stride, norm=1, threshold: Union[float, torch.Tensor] = 0.8, block_size=128,
                            causal=True, chunk_size=None, keep_sink=False, keep_recent=False,
                            device: Optional[torch.device] = None, out: Optional[torch.Tensor] = None,
                            groups_per_step: int = 1, q_splits: int = 1, tail_splits: int = 4) -> torch.Tensor:
    """Same computation as Xattention_prefill (xattn/src/Xattention.py:302-402) for host tensors.

    query_states [1,Hq,L,D], key/value_states [1,Hkv,L,D] on the CPU (pin them: pageable memory makes the
    copies synchronous).  Returns a pinned CPU tensor [1,Hq,L,D] (contiguous), or fills `out`.  The call
    returns when the result is complete.  `groups_per_step` kv groups are resident at a time; the query heads of
    a group slice run in `q_splits` steps, those of the last slice in `tail_splits` steps (when that divides them)."""
    assert block_size == 128
    B, Hq, Lq, D = query_states.shape
    assert B == 1
    Hkv, Lk = key_states.shape[1], key_states.shape[2]
    if query_states.is_cuda or key_states.is_cuda or value_states.is_cuda:
        raise ValueError("Xattention_prefill_host takes host tensors; use Xattention_prefill for device tensors")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if chunk_size is None:
        chunk_size = ops.default_chunk_size(Lk)
    cdtype = torch.bfloat16 if query_states.dtype == torch.float32 else query_states.dtype
    if out is None:
        out = torch.empty(1, Hq, Lq, D, dtype=cdtype).pin_memory()
    g = ops.geometry(Lq, Lk, chunk_size, stride, block_size)
    band = ops.band_applies(Lk, chunk_size, bool(causal))
    # smaller steps shorten what cannot overlap (the first step's input copy, the last step's output copy) but make
    # more, shorter copies: on a PCIe 5 x16 link one kv group per step measured best (8.93 ms at 32K; two steps per
    # group 9.06, four 9.76, two groups per step 9.4); cutting only the last group into four takes its output copy
    # from 0.65 to 0.21 ms (8.77 ms; 128K tokens: 34.3 -> 33.4 ms).  The input copies themselves take 8.2-8.5 ms with
    # the output copies running beside them, against 7.26 ms alone.
    steps = plan_steps(Hq, Hkv, groups_per_step, q_splits, tail_splits)
    slices = []                                          # [(q0, q1, k0, k1, [steps of the slice])]
    for st in steps:
        if st[4]:
            slices.append([st[0], st[1], st[2], st[3], []])
        slices[-1][1] = st[1]
        slices[-1][4].append(st)
    nq = max(sl[1] - sl[0] for sl in slices)
    nk = max(sl[3] - sl[2] for sl in slices)
    parts = max(len(sl[4]) for sl in slices)
    with torch.cuda.device(dev):
        h2d, d2h = _streams(dev)
        compute = torch.cuda.current_stream(dev)
        # two buffer sets, one per slice in flight; a slice's steps work on sub-views of its set
        sets = []
        for _ in range(2):
            sets.append(dict(
                q=torch.empty(1, nq, Lq, D, dtype=query_states.dtype, device=dev),
                o=torch.empty(1, nq, Lq, D, dtype=cdtype, device=dev),
                k=torch.empty(1, nk, Lk, D, dtype=key_states.dtype, device=dev),
                v=torch.empty(1, nk, Lk, D, dtype=value_states.dtype, device=dev),
                loaded_q=[torch.cuda.Event() for _ in range(parts)],
                loaded_k=torch.cuda.Event(), loaded_v=torch.cuda.Event(),
                released=torch.cuda.Event(),             # the slice's last kernel has run: q, k, v may be overwritten
                stored=torch.cuda.Event(),               # the slice's last output copy has left: o may be overwritten
                used=False))
        h2d.wait_stream(compute)

        def enqueue_inputs(si):
            """All input copies of slice si, in the order the kernels need them: K, the query heads step by step,
            V (not needed by the estimate).  Enqueued one slice ahead of the kernels, so that the copy engine never
            waits for the host thread, however small the steps."""
            q0s, _, k0, k1, sl_steps = slices[si]
            c = sets[si & 1]
            with torch.cuda.stream(h2d):
                if c["used"]:
                    h2d.wait_event(c["released"])
                c["k"][:, :k1 - k0].copy_(key_states[:, k0:k1], non_blocking=True)
                c["loaded_k"].record(h2d)
                for j, (q0, q1, *_rest) in enumerate(sl_steps):
                    c["q"][:, q0 - q0s:q1 - q0s].copy_(query_states[:, q0:q1], non_blocking=True)
                    c["loaded_q"][j].record(h2d)
                    if j == 0:
                        c["v"][:, :k1 - k0].copy_(value_states[:, k0:k1], non_blocking=True)
                        c["loaded_v"].record(h2d)

        enqueue_inputs(0)
        for si, (q0s, _q1s, k0, k1, sl_steps) in enumerate(slices):
            if si + 1 < len(slices):
                enqueue_inputs(si + 1)
            c = sets[si & 1]
            hk_n = k1 - k0
            kd, vd = c["k"][:, :hk_n], c["v"][:, :hk_n]
            compute.wait_event(c["loaded_k"])
            if c["used"]:
                compute.wait_event(c["stored"])            # the set's output buffer (slice si - 2) has left the device
            for j, (q0, q1, *_rest) in enumerate(sl_steps):
                compute.wait_event(c["loaded_q"][j])
                thr = threshold[q0:q1] if isinstance(threshold, torch.Tensor) else threshold
                qd, od = c["q"][:, q0 - q0s:q1 - q0s], c["o"][:, q0 - q0s:q1 - q0s]
                sums = ops.estimate_block_sums(qd, kd, stride, block_size, chunk_size, float(norm), bool(causal),
                                               band=band)
                _, idx, cnt = ops.select_blocks(sums, g["bpc"], g["block_offset"], thr, bool(causal), True,
                                                bool(keep_sink), bool(keep_recent), list_shape=(Lq, Lk),
                                                want_mask=False, band_k_blocks=g["kb"] if band else None)
                if j == 0:
                    compute.wait_event(c["loaded_v"])
                ops.block_sparse_attention(qd, kd, vd, idx, cnt, bool(causal), out=od)
                computed = torch.cuda.Event()
                computed.record(compute)
                if j == len(sl_steps) - 1:
                    c["released"].record(compute)
                with torch.cuda.stream(d2h):
                    d2h.wait_event(computed)
                    out[:, q0:q1].copy_(od, non_blocking=True)
                    if j == len(sl_steps) - 1:
                        c["stored"].record(d2h)
            c["used"] = True
        compute.wait_stream(d2h)
        compute.wait_stream(h2d)
        compute.synchronize()
        ops.check_device_status(dev, synchronize=False)      # a kernel whose bounded wait ran out: raise, not garbage
    return out
