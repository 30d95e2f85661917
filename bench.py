#!/usr/bin/env python
"""Benchmark of the XAttention prefill hot path (estimate -> select -> block-sparse attention).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one `Xattention_prefill` call over one synthetic attention layer (the workload's Q/K/V for one
sequence).  The printed line:

* `value` / `ms_per_step`: dense-equivalent ("effective") TFLOP/s = 4*Lq*Lk*D*Hq (halved when causal) over the
  step time, inputs resident in HBM.  With N GPUs (torchrun, one rank per GPU) the (batch, kv-head group) units
  of N sequences are dealt to the ranks, one sequence each: the path needs no collective, per-GPU work is fixed
  ("weak" scaling) and `value` is the aggregate over ranks.
* `e2e`: the same metric through the public host-buffer call: q/k/v come from pinned host memory and the output
  returns to it inside the timed region; `e2e.pcie_floor_ms` is what plain pinned copies of the same bytes take
  with all N ranks copying at once.
* `roofline` / `phase_rooflines`: every phase against the measured dense bf16 peak AND the measured HBM copy
  bandwidth; `bound` names the tighter of the two.
* `workloads`: at N=1 the long-context workload (llama3_8b_128k) measured the same way.
* `cpu_baseline`, `--impl reference`: the reference's own torch code (staged under oracle/_ref by
  oracle/make_ref.py; the CPU restatement in oracle/ when no staged copy exists) on the host cores, on a bounded
  sample of the workload.  `reference_gpu`: the unmodified reference's estimate+selection on the GPU (its torch
  branch, and its Triton kernels with the device-name gate answered), plus a dense library attention for scale.
* N > 1 only: `strong_128k` (ONE 128K sequence, kv-head groups dealt to the ranks, no collective) and
  `qchunk_256k` (ONE 256K sequence, query pieces dealt to the ranks after one NCCL broadcast of K and V).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "x-attention_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch  # noqa: E402

METRIC = "prefill_attention_effective_tflops"
UNIT = "TFLOP/s (dense-equivalent, 4*Lq*Lk*D*Hq/2 causal)"
# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the attention kernel that does the bulk of the call,
# from ncu captures of this benchmark's own command line.  32K: block_sparse_attn_kernel on the full workload
# (405.4 MB read + 234.1 MB written).  128K: block_sparse_attn_pair_kernel, captured on two of the eight kv-head
# groups (--heads-limit 2: 421.3 MB + 219.8 MB) and multiplied by four -- every kv group reads and writes its own
# Q, K, V and O, so the traffic grows in proportion.
NCU_ATTENTION_TRAFFIC_BYTES = {"llama3_8b_32k": 639_545_088, "llama3_8b_128k": 4 * 641_088_000}
DEFAULT_WORKLOAD = "llama3_8b_32k"
LONG_WORKLOAD = "llama3_8b_128k"


def effective_flops(w, heads=None, q_rows=None) -> float:
    hq = w.hq if heads is None else heads
    lq = w.seq_len if q_rows is None else q_rows
    f = 4.0 * lq * w.seq_len * w.head_dim * hq
    return f * 0.5 if w.causal else f


def estimate_executed_flops(w, chunk, torch_branch=True, heads=None):
    """FLOPs of the estimate GEMM as executed: 2 * 128 * tile_n * (S*D) per visible tile (csrc/estimate.cu picks
    the visible column tiles of every 128-row tile of the stride-reshaped problem; same bounds here)."""
    S, D, L = w.stride, w.head_dim, w.seq_len
    lp = -(-L // chunk) * chunk
    rows = lp // S
    rcs = chunk // S
    k_pad = lp - L
    left_blank = w.causal and torch_branch and k_pad == 0
    tile_n = 128 if (left_blank and rcs <= 128) else 256
    rows_valid = rows - k_pad // S
    cols_valid = rows - k_pad // S
    tiles = 0
    for mt in range((rows + 127) // 128):
        i0, i1 = mt * 128, min((mt + 1) * 128, rows, rows_valid)
        if i1 <= i0:
            continue
        if not w.causal:
            lo, hi = 0, rows - 1
        else:
            lo = (i0 // rcs) * rcs if left_blank else 0
            hi = min(i1 - 1, cols_valid - 1)
        if hi >= lo:
            tiles += hi // tile_n - lo // tile_n + 1
    return 2.0 * 128 * tile_n * S * D * tiles * (w.hq if heads is None else heads)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(bf16=float(d["bf16_tflops"]), hbm=float(d["hbm_gbs"]), source="measured")
    return dict(bf16=1590.0, hbm=6650.0, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.proc.terminate()
        rows = [r for r in self.rows if len(r) >= 6 and r[0].isdigit()]
        if not rows:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["no samples"])
        sm = sorted(int(r[0]) for r in rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)]
        return dict(sm_mhz=sm[len(sm) // 2], sm_max_mhz=int(rows[0][1]), reasons=reasons, samples=len(rows))


def dist_setup(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        return rank, world, local, dist
    return 0, 1, 0, None


def max_over_ranks(x: float, dist, device) -> float:
    if dist is None:
        return x
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def sum_over_ranks(x: float, dist, device) -> float:
    if dist is None:
        return x
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t[0])


def _default_chunk(L):
    p = 1 << (L - 1).bit_length()
    return int(max(min(max(2048, p), 128 * 1024 * 2048 // p), 2048))


def _describe(w, chunk):
    return (f"{w.name}: causal={w.causal} bsz=1/GPU hq={w.hq} hkv={w.hkv} seq_len={w.seq_len} head_dim=128 "
            f"stride={w.stride} block=128 threshold={w.threshold} chunk={chunk}")


def _config(w, chunk, n):
    return dict(workload=_describe(w, chunk), global_batch=n, seq_len=w.seq_len,
                parallelism=f"dp{n}: the (batch, kv-head group) units of {n} sequence(s), one sequence per GPU, "
                            f"no collective on the data path",
                l2="inputs (Q+K+V >= 384 MB per step) exceed the 126 MB L2; no flush needed",
                estimate_semantics="reference torch branch (what the reference executes on a B200)")


# ------------------------------------------------------------------------------------ CPU arm
def _reference_estimate_fn():
    """(callable, kind): the staged reference's own xattn_estimate when oracle/_ref exists, else the oracle port."""
    from oracle import make_ref
    if make_ref.available():
        ref = make_ref.load()

        def run(q1, k1, w, chunk):
            make_ref.keep_on_cpu(True)
            try:
                return ref.xattn_estimate(q1, k1, block_size=128, stride=w.stride, threshold=w.threshold,
                                          chunk_size=chunk, use_triton=False, causal=w.causal)[1]
            finally:
                make_ref.keep_on_cpu(False)
        return run, "reference"
    from oracle import xattn_oracle as orc

    def run(q1, k1, w, chunk):
        return orc.xattn_estimate_oracle(q1, k1, 128, w.stride, 1.0, w.threshold, chunk, w.causal)[1]
    return run, "port"


def cpu_reference_sample(q, k, v, w, chunk, estimate_fn, q_blocks_sampled=64, head=0):
    """One bounded sample of the reference's CPU path on ONE query head: the full-length estimate and selection of
    that head (the reference's xattn_estimate, torch branch, fp32), then dense masked attention (the fp32
    statement of the attention phase; the reference's own attention backend is a CUDA-only third-party package)
    for `q_blocks_sampled` evenly spaced query blocks.  Returns (seconds per head, detail)."""
    from oracle import xattn_oracle as orc
    rep = q.shape[1] // k.shape[1]
    hk = head // rep
    q1, k1, v1 = q[:, head:head + 1].float(), k[:, hk:hk + 1].float(), v[:, hk:hk + 1].float()
    L = q.shape[2]
    t0 = time.perf_counter()
    mask = estimate_fn(q1, k1, w, chunk)
    t_est = time.perf_counter() - t0
    qb = (L + 127) // 128
    rows = sorted(set(int(round(i * (qb - 1) / max(1, q_blocks_sampled - 1))) for i in range(q_blocks_sampled)))
    t1 = time.perf_counter()
    covered = 0.0
    for r in rows:
        r0, r1 = r * 128, min(L, (r + 1) * 128)
        m = torch.zeros(1, 1, 1, mask.shape[-1], dtype=torch.bool)
        m[0, 0, 0] = mask[0, 0, r]
        qq = q1[:, :, r0:r1]
        kk = k1[:, :, : r1] if w.causal else k1
        vv = v1[:, :, : r1] if w.causal else v1
        mm = m[..., : (kk.shape[2] + 127) // 128]
        orc.block_sparse_attention_oracle(qq, kk, vv, mm, w.causal)
        covered += 4.0 * (r1 - r0) * L * w.head_dim * (0.5 if w.causal else 1.0)
    t_att = time.perf_counter() - t1
    t_head = t_est + t_att * (effective_flops(w, heads=1) / covered)
    return t_head, dict(t_estimate_s=t_est, t_attention_sample_s=t_att, q_blocks=len(rows))


def cpu_baseline_run(q, k, v, w, chunk, q_blocks, heads, reps):
    """Per-head time of the CPU path over `heads` sampled query heads: one untimed warm-up per head, then `reps`
    timed repetitions; the value uses the median of all timed samples, the spread is reported."""
    torch.set_num_threads(os.cpu_count() or 1)
    fn, kind = _reference_estimate_fn()
    samples, detail = [], None
    for hh in heads:
        cpu_reference_sample(q, k, v, w, chunk, fn, q_blocks, head=hh)            # warm-up
        for _ in range(reps):
            t_h, detail = cpu_reference_sample(q, k, v, w, chunk, fn, q_blocks, head=hh)
            samples.append(t_h)
    s = sorted(samples)
    t_head = s[len(s) // 2]
    value = effective_flops(w) / (t_head * w.hq) / 1e12
    sample = (f"{len(heads)} of {w.hq} query heads at full length, 1 warm-up + {reps} repetitions each: estimate + "
              f"selection in full ({'the reference xattn_estimate, torch branch' if kind == 'reference' else 'CPU restatement'}), "
              f"dense masked attention on {detail['q_blocks']} evenly spaced query blocks scaled to the head; "
              f"median per-head time x {w.hq} heads")
    return dict(value=value, unit=UNIT, cores=torch.get_num_threads(), kind=kind, sample=sample,
                host_cores=os.cpu_count(), per_head_s=dict(min=s[0], median=t_head, max=s[-1], n=len(s)),
                detail=detail), t_head


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from xattn_b200 import synth
    q, k, v, w = synth.make_inputs(args.workload, seed=0, heads_limit=1)
    chunk = w.chunk_size or _default_chunk(w.seq_len)
    rep = w.hq // w.hkv
    base, t_head = cpu_baseline_run(q, k, v, w, chunk, args.cpu_q_blocks, heads=list(range(min(rep, 2))),
                                    reps=max(3, args.steps))
    n = args.gpus
    step_s = t_head * w.hq * n            # whole job = N sequences x Hq heads at the measured per-head rate
    value = effective_flops(w) * n / step_s / 1e12
    base["value"] = value
    line = dict(
        impl="reference", metric=METRIC, value=value, unit=UNIT, n_gpus=n, steps=args.steps, warmup=args.warmup,
        ms_per_step=step_s * 1e3, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f32",
        data="synthetic", config=_config(w, chunk, n), cpu_baseline=base,
        e2e=dict(value=value, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0),
        gpu_launches=0,
        note="a step is extrapolated from the sampled heads (ms_per_step = median per-head time x heads x sequences)",
    )
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------ GPU arm
def _events(n):
    return [torch.cuda.Event(enable_timing=True) for _ in range(n)]


def _bounds(flops, nbytes, ms, peaks):
    """A phase against both rooflines; `bound` is the one whose floor time is larger."""
    tf = flops / (ms * 1e-3) / 1e12 if ms > 0 else 0.0
    gbs = nbytes / (ms * 1e-3) / 1e9 if ms > 0 else 0.0
    f_t, f_h = tf / peaks["bf16"], gbs / peaks["hbm"]
    return dict(bound="tensor" if f_t >= f_h else "hbm", executed_flops=flops, algorithmic_bytes=nbytes,
                tflops=tf, frac=f_t, gbs=gbs, hbm_frac=f_h, peak_tflops=peaks["bf16"], peak_gbs=peaks["hbm"],
                floor_ms=max(flops / peaks["bf16"] / 1e9, nbytes / peaks["hbm"] / 1e6))


def phase_profile(w, dq, dk, dv, chunk, reps, device, peaks):
    """Per-phase device times (median of `reps`) of the three calls Xattention_prefill makes, the executed
    attention work, and every phase against its rooflines."""
    from xattn_b200 import ops
    L, hq, hkv = dq.shape[2], dq.shape[1], dk.shape[1]
    g = ops.geometry(L, L, chunk, w.stride)
    ev = _events(4)
    samples = [[], [], []]
    n_sel, cnt = 0, None
    band = ops.band_applies(L, chunk, w.causal)                     # what Xattention_prefill does
    for it in range(reps + 1):
        ev[0].record()
        sums = ops.estimate_block_sums(dq, dk, w.stride, 128, chunk, 1.0, w.causal, band=band)
        ev[1].record()
        _, idx, cnt = ops.select_blocks(sums, g["bpc"], g["block_offset"], w.threshold, w.causal, True,
                                        list_shape=(L, L), want_mask=False,
                                        band_k_blocks=g["kb"] if band else None)
        ev[2].record()
        ops.block_sparse_attention(dq, dk, dv, idx, cnt, w.causal)
        ev[3].record()
        torch.cuda.synchronize(device)
        if it > 0:
            for i in range(3):
                samples[i].append(ev[i].elapsed_time(ev[i + 1]))
    n_sel = int(cnt.sum())
    ph = [sorted(x)[len(x) // 2] for x in samples]
    qb = (L + 127) // 128
    total_blocks = hq * (qb * (qb + 1) // 2 if w.causal else qb * qb)
    f_att = 4.0 * 128 * 128 * 128 * n_sel
    b_att = (2.0 * hq + 2.0 * hkv) * L * w.head_dim * 2             # Q+O, K+V once; 16-bit
    f_est = estimate_executed_flops(w, chunk, heads=hq)
    b_est = (hq + hkv) * L * w.head_dim * 2.0 + 4.0 * hq * g["qb"] * (g["bpc"] if band else g["kb"])
    b_sel = 4.0 * hq * g["qb"] * (g["bpc"] if band else g["kb"]) + 4.0 * n_sel + 4.0 * hq * qb
    rl = dict(estimate=_bounds(f_est, b_est, ph[0], peaks), attend=_bounds(f_att, b_att, ph[2], peaks))
    rl["select"] = dict(bound="hbm", algorithmic_bytes=b_sel, gbs=b_sel / (ph[1] * 1e-3) / 1e9,
                        hbm_frac=b_sel / (ph[1] * 1e-3) / 1e9 / peaks["hbm"], peak_gbs=peaks["hbm"],
                        note="tens of microseconds: launch latency and one dependent memory round trip per row")
    return dict(phases_ms=dict(estimate=ph[0], select=ph[1], attend=ph[2]), selected_blocks=n_sel,
                block_density=n_sel / total_blocks, blocks_per_row=n_sel / (hq * qb), rooflines=rl,
                cnt=cnt)


def attention_roofline(name, prof, peaks):
    a = prof["rooflines"]["attend"]
    from xattn_b200 import ops, synth
    w = synth.WORKLOADS[name]
    split = (w.seq_len // 128 >= ops.PAIR_MIN_K_BLOCKS and w.hq * (w.seq_len // 128) >= ops.PAIR_MIN_ITEMS
             and w.hq // w.hkv >= 2 and (w.hq // w.hkv) % 2 == 0)
    kernel = ("block_sparse_attn_pair_kernel (rows whose kv group shares a list of one or two blocks) + "
              "block_sparse_attn_kernel (the rest), one call") if split else "block_sparse_attn_kernel"
    return dict(bound=a["bound"], kernel=kernel, achieved=a["tflops"], peak=peaks["bf16"],
                unit="TFLOP/s", frac=a["frac"], hbm_achieved_gbs=a["gbs"], hbm_peak_gbs=peaks["hbm"],
                hbm_frac=a["hbm_frac"], traffic=NCU_ATTENTION_TRAFFIC_BYTES.get(name),
                traffic_unit="bytes per launch (ncu)", algorithmic_bytes=a["algorithmic_bytes"],
                peak_source=peaks["source"], executed_flops_per_launch=a["executed_flops"],
                selected_blocks=prof["selected_blocks"])


def pcie_floor(bytes_in, bytes_out, device, dist, reps=3):
    """Plain pinned copies of one step's bytes, both directions at once on two streams, all ranks together."""
    hin = torch.empty(bytes_in, dtype=torch.uint8).pin_memory()
    hout = torch.empty(bytes_out, dtype=torch.uint8).pin_memory()
    din = torch.empty(bytes_in, dtype=torch.uint8, device=device)
    dout = torch.empty(bytes_out, dtype=torch.uint8, device=device)
    s1, s2 = torch.cuda.Stream(device), torch.cuda.Stream(device)
    best = None
    for it in range(reps + 1):
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(device)
        e0, e1 = _events(2)
        e0.record()
        s1.wait_event(e0)
        s2.wait_event(e0)
        with torch.cuda.stream(s1):
            din.copy_(hin, non_blocking=True)
        with torch.cuda.stream(s2):
            hout.copy_(dout, non_blocking=True)
        torch.cuda.current_stream(device).wait_stream(s1)
        torch.cuda.current_stream(device).wait_stream(s2)
        e1.record()
        torch.cuda.synchronize(device)
        ms = max_over_ranks(e0.elapsed_time(e1), dist, device)
        if it > 0:
            best = ms if best is None else min(best, ms)
    return best


def measure_workload(name, args, rank, dist, device, peaks, steps, warmup, seed, with_clocks=False):
    """value/e2e/phase measurements of one workload on this rank's own sequence."""
    import xattn_b200
    from xattn_b200 import ops, synth
    dq, dk, dv, w = synth.make_inputs(name, seed=seed, device=device, heads_limit=args.heads_limit)
    if args.heads_limit is not None:             # a kv-group slice of the workload (small captures under a profiler)
        import dataclasses
        # the slice stands for the whole workload: it takes the attention kernels the whole workload would take
        ops.PAIR_MIN_ITEMS = ops.PAIR_MIN_ITEMS * dk.shape[1] // w.hkv
        w = dataclasses.replace(w, hq=dq.shape[1], hkv=dk.shape[1], name=f"{w.name}[{dk.shape[1]} kv group(s)]")
    chunk = w.chunk_size or ops.default_chunk_size(w.seq_len)
    q_pin, k_pin, v_pin = dq.cpu().pin_memory(), dk.cpu().pin_memory(), dv.cpu().pin_memory()
    out_host = torch.empty(1, w.hq, w.seq_len, w.head_dim, dtype=w.dtype).pin_memory()
    lib = xattn_b200._lib.load()

    def step():
        return xattn_b200.Xattention_prefill(dq, dk, dv, w.stride, threshold=w.threshold, chunk_size=chunk,
                                             causal=w.causal)

    def step_e2e():
        xattn_b200.Xattention_prefill_host(q_pin, k_pin, v_pin, w.stride, threshold=w.threshold, chunk_size=chunk,
                                           causal=w.causal, device=device, out=out_host)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(device)

    def timed(fn, n_steps, n_warm):
        for _ in range(n_warm):
            fn()
        barrier()
        c0 = lib.xattn_b200_launch_count()
        e0, e1 = _events(2)
        e0.record()
        for _ in range(n_steps):
            fn()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1), dist, device) / n_steps, lib.xattn_b200_launch_count() - c0

    sampler = ClockSampler(device.index) if (with_clocks and rank == 0) else None
    if sampler:
        sampler.start()
    ms, launches = timed(step, steps, warmup)
    clocks = sampler.stop() if sampler else None
    xattn_b200.check_device_status(device)
    ms_e2e, _ = timed(step_e2e, max(2, steps // 4), 2)
    xattn_b200.check_device_status(device)
    prof = phase_profile(w, dq, dk, dv, chunk, max(3, steps // 4), device, peaks)
    prof.pop("cnt")
    bi = (dq.numel() + dk.numel() + dv.numel()) * dq.element_size()
    bo = out_host.numel() * out_host.element_size()
    return dict(w=w, chunk=chunk, ms=ms, ms_e2e=ms_e2e, launches=launches, clocks=clocks, prof=prof, bi=bi, bo=bo,
                host=(q_pin, k_pin, v_pin))


def dense_mask_record(device, peaks):
    """The attention kernel on a dense causal mask (long block lists): what its inner loop sustains when the
    per-item prologue/epilogue no longer dominates."""
    from xattn_b200 import ops
    Ld, Hd = 16384, 16
    gd = torch.Generator(device=device).manual_seed(1)
    qd_, kd_, vd_ = (torch.randn(1, Hd, Ld, 128, generator=gd, device=device).to(torch.bfloat16) for _ in range(3))
    md = torch.tril(torch.ones(Ld // 128, Ld // 128, dtype=torch.bool, device=device))[None, None].expand(1, Hd, -1, -1)
    idx_d, cnt_d = ops.mask_to_lists(md.contiguous(), Ld, Ld, True)
    for _ in range(3):
        ops.block_sparse_attention(qd_, kd_, vd_, idx_d, cnt_d, True)
    d0, d1 = _events(2)
    d0.record()
    for _ in range(10):
        ops.block_sparse_attention(qd_, kd_, vd_, idx_d, cnt_d, True)
    d1.record()
    torch.cuda.synchronize(device)
    nb = int(cnt_d.sum())
    tf = 4.0 * 128 * 128 * 128 * nb / (d0.elapsed_time(d1) / 10 * 1e-3) / 1e12
    return dict(workload=f"dense causal mask, {Hd} heads x {Ld} tokens, {nb} blocks", achieved=tf, unit="TFLOP/s",
                peak=peaks["bf16"], frac=tf / peaks["bf16"])


def reference_gpu_record(names, device):
    """The unmodified reference's estimate + selection on this GPU (secondary figures, a few launches each):
    `torch_branch_ms` is what the reference executes on a B200 (its device-name gate sends every GPU whose name
    lacks "100" to the torch branch, xattn/src/Xattention.py:57-63); `triton_ms` is its Triton path
    (flat_group_gemm_fuse_reshape + softmax_fuse_block_sum + find_blocks_chunked) with that gate answered.  K is
    repeated to the query heads beforehand, as the reference requires.  `dense_sdpa_ms`: torch's library dense
    causal attention on the same tensors (the "full attention" bar of the reference's speed-up figures)."""
    from oracle import make_ref
    from xattn_b200 import ops, synth
    if not make_ref.available():
        return dict(unavailable="oracle/_ref is not staged (run oracle/make_ref.py where the reference is checked out)")
    try:
        ref = make_ref.load()
    except Exception as e:  # noqa: BLE001
        return dict(unavailable=f"staged reference failed to import: {type(e).__name__}: {e}"[:300])
    out = {}

    def timed(fn, reps):
        fn()
        torch.cuda.synchronize(device)
        ts = []
        for _ in range(reps):
            e0, e1 = _events(2)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize(device)
            ts.append(e0.elapsed_time(e1))
        return sorted(ts)[len(ts) // 2]

    real_props = torch.cuda.get_device_properties
    for name in names:
        rec = {}
        dq, dk, dv, w = synth.make_inputs(name, seed=0, device=device)
        chunk = w.chunk_size or ops.default_chunk_size(w.seq_len)
        kr = dk.repeat_interleave(w.hq // w.hkv, 1)

        def est(use_triton):
            return ref.xattn_estimate(dq, kr, block_size=128, stride=w.stride, threshold=w.threshold,
                                      chunk_size=chunk, use_triton=use_triton, causal=w.causal)
        try:
            rec["torch_branch_ms"] = timed(lambda: est(False), 3)
        except Exception as e:  # noqa: BLE001
            rec["torch_branch_ms"] = None
            rec["torch_branch_unavailable"] = f"{type(e).__name__}: {e}"[:300]
        try:
            class _Named:
                def __init__(self, p):
                    self._p = p
                    self.name = p.name + " (gate answered: 100)"

                def __getattr__(self, k):
                    return getattr(self._p, k)
            torch.cuda.get_device_properties = lambda *a, **k: _Named(real_props(*a, **k))
            rec["triton_ms"] = timed(lambda: est(True), 3)
        except Exception as e:  # noqa: BLE001
            rec["triton_ms"] = None
            rec["triton_unavailable"] = f"{type(e).__name__}: {e}"[:300]
        finally:
            torch.cuda.get_device_properties = real_props
        del kr
        try:
            from torch.nn.attention import SDPBackend, sdpa_kernel
            with sdpa_kernel([SDPBackend.FLASH_ATTENTION, SDPBackend.CUDNN_ATTENTION, SDPBackend.EFFICIENT_ATTENTION]):
                rec["dense_sdpa_ms"] = timed(lambda: torch.nn.functional.scaled_dot_product_attention(
                    dq, dk, dv, is_causal=w.causal, enable_gqa=True), 2)
        except Exception as e:  # noqa: BLE001
            rec["dense_sdpa_ms"] = None
            rec["dense_sdpa_unavailable"] = f"{type(e).__name__}: {e}"[:300]
        out[name] = rec
        del dq, dk, dv
        torch.cuda.empty_cache()
    return out


def strong_scaling_record(rank, world, dist, device, peaks, steps):
    """ONE llama3_8b_128k sequence, its kv-head groups dealt to the ranks (sharding.prefill_sharded), no collective
    on the data path.  t_N = max over ranks; t_1 = the whole sequence on rank 0 alone (the others wait)."""
    import xattn_b200
    from xattn_b200 import ops, sharding, synth
    dq, dk, dv, w = synth.make_inputs(LONG_WORKLOAD, seed=0, device=device)       # same tensors on every rank
    chunk = w.chunk_size or ops.default_chunk_size(w.seq_len)
    q0, q1, k0, k1 = sharding.shard_kv_groups(w.hq, w.hkv, world, rank)

    def run_shard():
        return sharding.prefill_sharded(dq, dk, dv, xattn_b200.Xattention_prefill, world, rank, threshold=w.threshold,
                                        stride=w.stride, chunk_size=chunk, causal=w.causal)

    def timed(fn, n, everyone=True):
        for _ in range(3):
            fn()
        dist.barrier()
        torch.cuda.synchronize(device)
        e0, e1 = _events(2)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize(device)
        ms = e0.elapsed_time(e1) / n
        return max_over_ranks(ms, dist, device) if everyone else ms

    t_n = timed(run_shard, steps)
    xattn_b200.check_device_status(device)
    # host-buffer leg: every rank moves only its slice
    qh, kh, vh = dq[:, q0:q1].cpu().pin_memory(), dk[:, k0:k1].cpu().pin_memory(), dv[:, k0:k1].cpu().pin_memory()
    oh = torch.empty(1, q1 - q0, w.seq_len, w.head_dim, dtype=w.dtype).pin_memory()
    t_e2e = timed(lambda: xattn_b200.Xattention_prefill_host(qh, kh, vh, w.stride, threshold=w.threshold,
                                                             chunk_size=chunk, causal=w.causal, device=device,
                                                             out=oh), max(2, steps // 4))
    bytes_rank = (qh.numel() + kh.numel() + vh.numel() + oh.numel()) * qh.element_size()
    # listed blocks of this rank's shard
    g = ops.geometry(w.seq_len, w.seq_len, chunk, w.stride)
    band = ops.band_applies(w.seq_len, chunk, w.causal)
    sums = ops.estimate_block_sums(dq[:, q0:q1], dk[:, k0:k1], w.stride, 128, chunk, 1.0, w.causal, band=band)
    _, _, cnt = ops.select_blocks(sums, g["bpc"], g["block_offset"], w.threshold, w.causal, True,
                                  list_shape=(w.seq_len, w.seq_len), want_mask=False,
                                  band_k_blocks=g["kb"] if band else None)
    mine = float(cnt.sum())
    tot, mx = sum_over_ranks(mine, dist, device), max_over_ranks(mine, dist, device)
    # the same sequence on one GPU (rank 0 alone)
    t_1 = 0.0
    if rank == 0:
        t_1 = timed(lambda: xattn_b200.Xattention_prefill(dq, dk, dv, w.stride, threshold=w.threshold,
                                                          chunk_size=chunk, causal=w.causal), steps, everyone=False)
    else:
        dist.barrier()
    t_1 = max_over_ranks(t_1, dist, device)
    flops = effective_flops(w)
    return dict(workload=_describe(w, chunk), parallelism=f"kv-head groups of ONE sequence over {world} GPUs "
                f"({w.hkv // world if world <= w.hkv else 1} group(s) per GPU), no collective", scaling="strong",
                ms_per_step=t_n, ms_per_step_1gpu=t_1, speedup=t_1 / t_n, efficiency=t_1 / t_n / world,
                effective_tflops=flops / (t_n * 1e-3) / 1e12, effective_tflops_1gpu=flops / (t_1 * 1e-3) / 1e12,
                e2e_ms_per_step=t_e2e, e2e_effective_tflops=flops / (t_e2e * 1e-3) / 1e12,
                e2e_bytes_per_rank_per_step=bytes_rank, load_imbalance=mx / (tot / world),
                selected_blocks=tot)


def qchunk_record(rank, world, dist, device, steps):
    """ONE llama3_8b_256k sequence: rank 0 holds K and V and broadcasts them once over NCCL, then every rank runs
    its query pieces (two per rank, dealt zig-zag) against local memory only."""
    import xattn_b200
    from xattn_b200 import ops, sharding, synth
    name = "llama3_8b_256k"
    dq, dk, dv, w = synth.make_inputs(name, seed=0, device=device)        # every rank has its queries
    chunk = w.chunk_size or ops.default_chunk_size(w.seq_len)
    L = w.seq_len
    k_src, v_src = dk, dv
    if rank != 0:                                                          # K/V exist on rank 0 only until the broadcast
        dk, dv = torch.empty_like(dk), torch.empty_like(dv)
    bc = []
    for it in range(3):
        dist.barrier()
        torch.cuda.synchronize(device)
        e0, e1 = _events(2)
        e0.record()
        dist.broadcast(dk, src=0)
        dist.broadcast(dv, src=0)
        e1.record()
        torch.cuda.synchronize(device)
        bc.append(max_over_ranks(e0.elapsed_time(e1), dist, device))
    kv_ok = bool(torch.equal(dk, k_src) and torch.equal(dv, v_src))        # same seed, same generator: same tensors
    rows = L // (2 * world)

    def run():
        return sharding.prefill_query_chunk_sharded(dq, dk, dv, xattn_b200.Xattention_prefill, world, rank, chunk,
                                                    threshold=w.threshold, shard_rows=rows, stride=w.stride)
    for _ in range(2):
        parts = run()
    dist.barrier()
    torch.cuda.synchronize(device)
    e0, e1 = _events(2)
    e0.record()
    for _ in range(steps):
        parts = run()
    e1.record()
    torch.cuda.synchronize(device)
    t_n = max_over_ranks(e0.elapsed_time(e1) / steps, dist, device)
    xattn_b200.check_device_status(device)
    # one GPU: the whole sequence (rank 0), and the difference of this rank's first piece against it
    full = xattn_b200.Xattention_prefill(dq, dk, dv, w.stride, threshold=w.threshold, chunk_size=chunk, causal=True)
    c = sorted(parts)[0]
    diff = float((parts[c].float() - full[:, :, c * rows:(c + 1) * rows].float()).abs().max())
    diff = max_over_ranks(diff, dist, device)
    e0, e1 = _events(2)
    torch.cuda.synchronize(device)
    e0.record()
    for _ in range(3):
        xattn_b200.Xattention_prefill(dq, dk, dv, w.stride, threshold=w.threshold, chunk_size=chunk, causal=True)
    e1.record()
    torch.cuda.synchronize(device)
    t_1 = max_over_ranks(e0.elapsed_time(e1) / 3, dist, device)
    flops = effective_flops(w)
    return dict(workload=_describe(w, chunk), parallelism=f"query pieces of {rows} rows dealt zig-zag over {world} "
                f"GPUs, all heads on every GPU, K and V broadcast once from rank 0 (NCCL)", scaling="strong",
                broadcast_ms=sorted(bc)[1], broadcast_bytes=2 * dk.numel() * dk.element_size(),
                broadcast_gbs=2 * dk.numel() * dk.element_size() / (sorted(bc)[1] * 1e-3) / 1e9,
                kv_identical_after_broadcast=kv_ok, ms_per_step=t_n, ms_per_step_1gpu=t_1, speedup=t_1 / t_n,
                efficiency=t_1 / t_n / world, effective_tflops=flops / (t_n * 1e-3) / 1e12,
                max_abs_diff_vs_1gpu=diff)


def run_gpu_arm(args):
    rank, world, local, dist = dist_setup(args.gpus)
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    n = max(world, 1)
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    import xattn_b200  # noqa: F401
    from xattn_b200 import host_pipeline

    numa_cores = host_pipeline.bind_host_to_gpu(device)
    peaks = measured_peaks()
    m = measure_workload(args.workload, args, rank, dist, device, peaks, args.steps, args.warmup, seed=rank,
                         with_clocks=True)
    w, chunk, prof = m["w"], m["chunk"], m["prof"]
    floor_ms = pcie_floor(m["bi"], m["bo"], device, dist)
    agg_flops = sum_over_ranks(effective_flops(w), dist, device)
    value = agg_flops / (m["ms"] * 1e-3) / 1e12
    e2e_value = agg_flops / (m["ms_e2e"] * 1e-3) / 1e12

    secondary = not args.no_secondary
    dense = dense_mask_record(device, peaks) if (rank == 0 and secondary) else None

    workloads = None
    if n == 1 and secondary and args.workload != LONG_WORKLOAD:
        m2 = measure_workload(LONG_WORKLOAD, args, rank, dist, device, peaks, max(5, args.steps // 2), 3, seed=0)
        w2, p2 = m2["w"], m2["prof"]
        f2 = effective_flops(w2)
        workloads = {LONG_WORKLOAD: dict(
            workload=_describe(w2, m2["chunk"]), ms_per_step=m2["ms"], value=f2 / (m2["ms"] * 1e-3) / 1e12, unit=UNIT,
            phases_ms=p2["phases_ms"], block_density=p2["block_density"], blocks_per_row=p2["blocks_per_row"],
            roofline=attention_roofline(LONG_WORKLOAD, p2, peaks), phase_rooflines=p2["rooflines"],
            gpu_launches_per_step=m2["launches"] / max(5, args.steps // 2),
            e2e=dict(value=f2 / (m2["ms_e2e"] * 1e-3) / 1e12, unit=UNIT, ms_per_step=m2["ms_e2e"],
                     h2d_bytes_per_step=m2["bi"], d2h_bytes_per_step=m2["bo"]))}
        del m2

    cpu_baseline = None
    if rank == 0 and n == 1 and not args.no_cpu_baseline:
        q_pin, k_pin, v_pin = m["host"]
        rep_ = w.hq // w.hkv
        cpu_baseline, _ = cpu_baseline_run(q_pin, k_pin, v_pin, w, chunk, args.cpu_q_blocks,
                                           heads=[0, rep_ * (w.hkv // 2)], reps=3)
    reference_gpu = None
    if rank == 0 and n == 1 and secondary:
        names = [args.workload] + ([LONG_WORKLOAD] if args.workload != LONG_WORKLOAD else [])
        reference_gpu = reference_gpu_record(names, device)

    strong = qchunk = None
    if n > 1 and secondary:
        strong = strong_scaling_record(rank, world, dist, device, peaks, max(5, args.steps // 2))
        qchunk = qchunk_record(rank, world, dist, device, max(3, args.steps // 4))

    if rank == 0:
        line = dict(
            metric=METRIC, value=value, unit=UNIT, n_gpus=n, steps=args.steps, warmup=args.warmup,
            ms_per_step=m["ms"], higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16",
            data="synthetic", config=_config(w, chunk, n), clocks=m["clocks"],
            e2e=dict(value=e2e_value, unit=UNIT, ms_per_step=m["ms_e2e"], h2d_bytes_per_step=m["bi"],
                     d2h_bytes_per_step=m["bo"], pcie_floor_ms=floor_ms,
                     pcie_floor_note=f"plain pinned copies of the same bytes, both directions at once, {n} rank(s) "
                                     f"copying together", host_cores_bound=len(numa_cores) if numa_cores else None),
            gpu_launches=m["launches"], gpu_launches_per_step=m["launches"] / args.steps,
            phases_ms=prof["phases_ms"], block_density=prof["block_density"], blocks_per_row=prof["blocks_per_row"],
            roofline=attention_roofline(args.workload, prof, peaks), phase_rooflines=prof["rooflines"],
            attention_dense_mask=dense, workloads=workloads, cpu_baseline=cpu_baseline, reference_gpu=reference_gpu,
            strong_128k=strong, qchunk_256k=qchunk,
        )
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true",
                    help="only the primary workload: no long-context record, reference-on-GPU figures or extra "
                         "multi-GPU legs (for profiling runs)")
    ap.add_argument("--cpu-q-blocks", type=int, default=64)
    ap.add_argument("--heads-limit", type=int, default=None,
                    help="keep only the first N kv-head groups of the workload (small cases for profiler captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
