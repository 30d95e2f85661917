#!/usr/bin/env python
"""Benchmark of the XAttention prefill hot path (estimate -> select -> block-sparse attention).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one `Xattention_prefill` call over one synthetic attention layer (the workload's Q/K/V for
one sequence).  With N GPUs (torchrun, one rank per GPU) every rank runs its own sequence of the
same shape -- the path shards by (batch, kv-head group) with no collective -- so per-GPU work is
fixed ("weak" scaling) and `value` is the aggregate over ranks.

`value` is dense-equivalent ("effective") TFLOP/s: 4*Lq*Lk*D*Hq (halved when causal) divided by the
step time, inputs already resident in HBM.  `e2e` is the same metric measured through the public
call with pinned HOST buffers: host->device copies of q/k/v and the device->host copy of the output
are inside the timed region.

`--impl reference` times the CPU restatement of the reference's torch path (oracle/) on the host
cores, on a bounded sample of the same workload.
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
# dram__bytes_read.sum + dram__bytes_write.sum of one block_sparse_attn_kernel launch, from the ncu capture that
# profiles/block_sparse_attn_kernel_llama3_8b_32k.md summarises (406.9 MB + 233.7 MB); other workloads: not captured
NCU_ATTENTION_TRAFFIC_BYTES = {"llama3_8b_32k": 640_664_576}
DEFAULT_WORKLOAD = "llama3_8b_32k"


def effective_flops(w, heads=None, q_rows=None) -> float:
    hq = w.hq if heads is None else heads
    lq = w.seq_len if q_rows is None else q_rows
    f = 4.0 * lq * w.seq_len * w.head_dim * hq
    return f * 0.5 if w.causal else f


def estimate_executed_flops(w, chunk, torch_branch=True):
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
    return 2.0 * 128 * tile_n * S * D * tiles * w.hq


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


# ------------------------------------------------------------------------------------ CPU arm
def cpu_reference_sample(q, k, v, w, chunk, q_blocks_sampled=64, head=0):
    """One bounded sample of the reference's CPU path on ONE query head: the full-length estimate and
    selection of that head (Xattention.py:13-299 restated in oracle/), then dense masked attention
    (the fp32 statement of the attention phase) for `q_blocks_sampled` evenly spaced query blocks.
    Returns (seconds per head, dense-equivalent FLOPs of a head, detail)."""
    from oracle import xattn_oracle as orc
    rep = q.shape[1] // k.shape[1]
    hk = head // rep
    q1, k1, v1 = q[:, head:head + 1].float(), k[:, hk:hk + 1].float(), v[:, hk:hk + 1].float()
    L = q.shape[2]
    t0 = time.perf_counter()
    _, mask = orc.xattn_estimate_oracle(q1, k1, 128, w.stride, 1.0, w.threshold, chunk, w.causal)
    t_est = time.perf_counter() - t0
    qb = (L + 127) // 128
    rows = sorted(set(int(round(i * (qb - 1) / max(1, q_blocks_sampled - 1))) for i in range(q_blocks_sampled)))
    t1 = time.perf_counter()
    covered = 0.0
    for r in rows:
        r0, r1 = r * 128, min(L, (r + 1) * 128)
        m = torch.zeros(1, 1, 1, mask.shape[-1], dtype=torch.bool)
        m[0, 0, 0] = mask[0, 0, r]
        # query rows r0:r1 against all keys, end-aligned like the full problem
        qq = q1[:, :, r0:r1]
        kk = k1[:, :, : r1] if w.causal else k1
        vv = v1[:, :, : r1] if w.causal else v1
        mm = m[..., : (kk.shape[2] + 127) // 128]
        orc.block_sparse_attention_oracle(qq, kk, vv, mm, w.causal)
        covered += 4.0 * (r1 - r0) * L * w.head_dim * (0.5 if w.causal else 1.0)
    t_att = time.perf_counter() - t1
    # scale the attention part to the whole head: time per dense-equivalent FLOP of the sampled rows
    full_head = effective_flops(w, heads=1)
    t_head = t_est + t_att * (full_head / covered)
    return t_head, full_head, dict(t_estimate_s=t_est, t_attention_sample_s=t_att, q_blocks=len(rows), rep=rep)


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from xattn_b200 import synth
    torch.set_num_threads(os.cpu_count() or 1)
    q, k, v, w = synth.make_inputs(args.workload, seed=0, heads_limit=1)
    chunk = w.chunk_size or _default_chunk(w.seq_len)
    times = []
    detail = None
    for i in range(args.warmup + args.steps):
        t_head, flops_head, detail = cpu_reference_sample(q, k, v, w, chunk, args.cpu_q_blocks)
        if i >= args.warmup:
            times.append(t_head)
    t = sum(times) / len(times)
    # whole job = N sequences x Hq heads, at the measured per-head rate on all host cores
    n = args.gpus
    step_s = t * w.hq * n
    value = effective_flops(w) * n / step_s / 1e12
    sample = (f"1 of {w.hq} query heads at full length: estimate+select in full, dense masked attention on "
              f"{detail['q_blocks']} evenly spaced query blocks scaled to the head; per-head time x {w.hq} heads")
    line = dict(
        impl="reference", metric=METRIC, value=value, unit=UNIT, n_gpus=n, steps=args.steps, warmup=args.warmup,
        ms_per_step=step_s * 1e3, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f32",
        data="synthetic", config=_config(w, chunk, n),
        cpu_baseline=dict(value=value, unit=UNIT, cores=torch.get_num_threads(), kind="port", sample=sample,
                          host_cores=os.cpu_count(), detail=detail),
        e2e=dict(value=value, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0),
        gpu_launches=0,
    )
    print(json.dumps(line), flush=True)


def _default_chunk(L):
    p = 1 << (L - 1).bit_length()
    return int(max(min(max(2048, p), 128 * 1024 * 2048 // p), 2048))


def _config(w, chunk, n):
    return dict(workload=f"{w.name}: causal={w.causal} bsz=1/GPU hq={w.hq} hkv={w.hkv} seq_len={w.seq_len} "
                         f"head_dim=128 stride={w.stride} block=128 threshold={w.threshold} chunk={chunk}",
                global_batch=n, seq_len=w.seq_len, parallelism=f"dp{n} (one sequence per GPU, no collective)",
                l2="inputs (Q+K+V >= 384 MB per step) exceed the 126 MB L2; no flush needed",
                estimate_semantics="reference torch branch (what the reference executes on a B200)")


# ------------------------------------------------------------------------------------ GPU arm
def run_gpu_arm(args):
    rank, world, local, dist = dist_setup(args.gpus)
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    n = max(world, 1)
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    import xattn_b200
    from xattn_b200 import host_pipeline, ops, synth

    # host buffers of this rank on the NUMA node of its GPU (matters for the host-buffer leg with several ranks)
    numa_cores = host_pipeline.bind_host_to_gpu(device)
    q, k, v, w = synth.make_inputs(args.workload, seed=rank)
    chunk = w.chunk_size or ops.default_chunk_size(w.seq_len)
    hq_pin, k_pin, v_pin = q.pin_memory(), k.pin_memory(), v.pin_memory()
    dq, dk, dv = hq_pin.to(device), k_pin.to(device), v_pin.to(device)

    def step():
        return xattn_b200.Xattention_prefill(dq, dk, dv, w.stride, threshold=w.threshold, chunk_size=chunk,
                                             causal=w.causal)

    out_host = torch.empty(1, w.hq, w.seq_len, w.head_dim, dtype=w.dtype).pin_memory()

    def step_e2e():
        # public host-buffer call: q/k/v come from pinned host memory and the output goes back to it, cut into
        # kv-head groups so that both PCIe directions and the kernels overlap
        xattn_b200.Xattention_prefill_host(hq_pin, k_pin, v_pin, w.stride, threshold=w.threshold,
                                           chunk_size=chunk, causal=w.causal, device=device, out=out_host)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(device)

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1), dist, device) / steps

    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    ms = timed(step, args.steps, args.warmup)
    clocks = sampler.stop() if sampler else None
    xattn_b200.check_device_status(device)
    ms_e2e = timed(step_e2e, max(2, args.steps // 2), 2)
    xattn_b200.check_device_status(device)

    # per-phase device times and the executed attention work (rank-local, explains `value`)
    g = ops.geometry(w.seq_len, w.seq_len, chunk, w.stride)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    samples = [[], [], []]
    reps = max(3, args.steps // 2)
    n_sel = 0
    for it in range(reps + 1):
        ev[0].record()
        band = ops.band_applies(w.seq_len, chunk, w.causal)          # what Xattention_prefill does
        sums = ops.estimate_block_sums(dq, dk, w.stride, 128, chunk, 1.0, w.causal, band=band)
        ev[1].record()
        mask, idx, cnt = ops.select_blocks(sums, g["bpc"], g["block_offset"], w.threshold, w.causal, True,
                                           list_shape=(w.seq_len, w.seq_len), want_mask=False,
                                           band_k_blocks=g["kb"] if band else None)
        ev[2].record()
        ops.block_sparse_attention(dq, dk, dv, idx, cnt, w.causal)
        ev[3].record()
        torch.cuda.synchronize(device)
        if it > 0:
            for i in range(3):
                samples[i].append(ev[i].elapsed_time(ev[i + 1]))
        n_sel = int(cnt.sum())
    ph = [sorted(x)[len(x) // 2] for x in samples]       # median over the repetitions
    qb = (w.seq_len + 127) // 128
    total_blocks = w.hq * (qb * (qb + 1) // 2 if w.causal else qb * qb)
    density = n_sel / total_blocks
    f_att = 4.0 * 128 * 128 * 128 * n_sel
    peaks = measured_peaks()
    att_tflops = f_att / (ph[2] * 1e-3) / 1e12 if ph[2] > 0 else 0.0
    roofline = dict(bound="tensor", kernel="block_sparse_attn_kernel", achieved=att_tflops, peak=peaks["bf16"],
                    unit="TFLOP/s", frac=att_tflops / peaks["bf16"],
                    traffic=NCU_ATTENTION_TRAFFIC_BYTES.get(args.workload), traffic_unit="bytes per launch (ncu)",
                    algorithmic_bytes=(2 * w.hq + 2 * w.hkv) * w.seq_len * w.head_dim * 2,   # Q+O, K+V once; 16-bit
                    peak_source=peaks["source"],
                    executed_flops_per_launch=f_att, selected_blocks=n_sel)

    # every phase against its roofline: the two tensor-core phases against the measured dense bf16 peak, the
    # selection against the measured HBM copy bandwidth (bytes: the block sums it reads + the lists it writes)
    band = ops.band_applies(w.seq_len, chunk, w.causal)
    f_est = estimate_executed_flops(w, chunk)
    sel_bytes = 4.0 * w.hq * g["qb"] * (g["bpc"] if band else g["kb"]) + 4.0 * n_sel + 4.0 * w.hq * qb
    phase_rooflines = dict(
        estimate=dict(bound="tensor", executed_flops=f_est, achieved=f_est / (ph[0] * 1e-3) / 1e12, unit="TFLOP/s",
                      peak=peaks["bf16"], frac=f_est / (ph[0] * 1e-3) / 1e12 / peaks["bf16"]),
        select=dict(bound="hbm", bytes=sel_bytes, achieved=sel_bytes / (ph[1] * 1e-3) / 1e9, unit="GB/s",
                    peak=peaks["hbm"], frac=sel_bytes / (ph[1] * 1e-3) / 1e9 / peaks["hbm"],
                    note="a 13-30 us phase: launch latency and one dependent memory round trip per row, not bandwidth"),
        attend=dict(bound="tensor", executed_flops=f_att, achieved=att_tflops, unit="TFLOP/s", peak=peaks["bf16"],
                    frac=att_tflops / peaks["bf16"]))

    # the same attention kernel on a dense causal mask (long block lists): what the inner loop sustains when the
    # per-item prologue/epilogue no longer dominates.  Rank 0 only, a few launches.
    dense = None
    if rank == 0:
        Ld, Hd = 16384, 16
        gd = torch.Generator().manual_seed(1)
        qd_, kd_, vd_ = (torch.randn(1, Hd, Ld, 128, generator=gd).to(torch.bfloat16).to(device) for _ in range(3))
        md = torch.tril(torch.ones(Ld // 128, Ld // 128, dtype=torch.bool, device=device))[None, None].expand(1, Hd, -1, -1)
        idx_d, cnt_d = ops.mask_to_lists(md.contiguous(), Ld, Ld, True)
        for _ in range(3):
            ops.block_sparse_attention(qd_, kd_, vd_, idx_d, cnt_d, True)
        d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        d0.record()
        for _ in range(10):
            ops.block_sparse_attention(qd_, kd_, vd_, idx_d, cnt_d, True)
        d1.record()
        torch.cuda.synchronize(device)
        nb = int(cnt_d.sum())
        tf = 4.0 * 128 * 128 * 128 * nb / (d0.elapsed_time(d1) / 10 * 1e-3) / 1e12
        dense = dict(workload=f"dense causal mask, {Hd} heads x {Ld} tokens, {nb} blocks", achieved=tf,
                     unit="TFLOP/s", peak=peaks["bf16"], frac=tf / peaks["bf16"])
        del qd_, kd_, vd_, idx_d, cnt_d, md

    agg_flops = sum_over_ranks(effective_flops(w), dist, device)
    value = agg_flops / (ms * 1e-3) / 1e12
    e2e_value = agg_flops / (ms_e2e * 1e-3) / 1e12
    bi = (q.numel() + k.numel() + v.numel()) * q.element_size()
    bo = out_host.numel() * out_host.element_size()

    cpu_baseline = None
    if rank == 0 and n == 1 and not args.no_cpu_baseline:
        torch.set_num_threads(os.cpu_count() or 1)
        rep_ = w.hq // w.hkv
        t_heads = []
        for hh in range(0, w.hq, rep_):          # one query head per kv group
            t_h, _, detail = cpu_reference_sample(q, k, v, w, chunk, args.cpu_q_blocks, head=hh)
            t_heads.append(t_h)
        t_head = sum(t_heads) / len(t_heads)
        detail["heads_sampled"] = len(t_heads)
        cpu_value = effective_flops(w) / (t_head * w.hq) / 1e12
        cpu_baseline = dict(
            value=cpu_value, unit=UNIT, cores=torch.get_num_threads(), kind="port",
            sample=(f"{detail['heads_sampled']} of {w.hq} query heads at full length: estimate+select in full, dense "
                    f"masked attention on {detail['q_blocks']} evenly spaced query blocks scaled to the head; "
                    f"mean per-head time x {w.hq} heads"),
            host_cores=os.cpu_count(), detail=detail)

    if rank == 0:
        line = dict(
            metric=METRIC, value=value, unit=UNIT, n_gpus=n, steps=args.steps, warmup=args.warmup, ms_per_step=ms,
            higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16", data="synthetic",
            config=_config(w, chunk, n), clocks=clocks,
            e2e=dict(value=e2e_value, unit=UNIT, ms_per_step=ms_e2e, h2d_bytes_per_step=bi, d2h_bytes_per_step=bo,
                     host_cores_bound=len(numa_cores) if numa_cores else None),
            # est_setup, est_gemm(_pair), [est_rowstat], est_blocksum, select, block_sparse_attn; the row statistics
            # are a launch of their own except where est_blocksum computes them (the 32K workload)
            gpu_launches=(5 if args.workload == "llama3_8b_32k" else 6) * args.steps,
            kernels_per_step=["est_setup_kernel", "est_gemm_pair_kernel | est_gemm_kernel",
                              "est_rowstat_kernel (not at 32K)", "est_blocksum_kernel",
                              "select_kernel", "block_sparse_attn_kernel"],
            phases_ms=dict(estimate=ph[0], select=ph[1], attend=ph[2]),
            block_density=density, roofline=roofline, phase_rooflines=phase_rooflines, attention_dense_mask=dense,
            cpu_baseline=cpu_baseline,
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
    ap.add_argument("--cpu-q-blocks", type=int, default=64)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
