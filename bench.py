#!/usr/bin/env python
"""Benchmark of the fp32 GEMM / im2col-convolution hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--workload NAME] [--mode strict|3xtf32|1xtf32|f16]
    python bench.py --impl reference ...     # the reference's CPU GEMM on the host cores

One "step" is one pass of the hot path over one batch of synthetic input.  Default workload:
BASELINE config 2, the fp32 GEMM M=8192 N=4096 K=2048 (3xTF32); with N>1 GPUs every rank
owns its own 8192 rows of A and C and a replica of B (weak scaling, no data-path collective).
Prints ONE JSON line on rank 0.  `value` is device-timed (CUDA events on the launch stream,
max over ranks) with operands resident in HBM; `e2e` runs the host-resident entry point
(pinned host buffers, H2D and D2H inside the timed region).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: kind, dims, sharding over ranks
    "cfg1": dict(kind="gemm", M=1024, N=1024, K=1024, scaling="weak",
                 desc="fp32 GEMM 1024x1024x1024 (BASELINE config 1)"),
    "cfg2": dict(kind="gemm", M=8192, N=4096, K=2048, scaling="weak",
                 desc="fp32 GEMM M=8192 N=4096 K=2048 per GPU (BASELINE config 2)"),
    "gemm16k": dict(kind="gemm", M=16384, N=16384, K=16384, scaling="weak",
                    desc="fp32 GEMM 16384^3 per GPU (north-star target shape)"),
    "cfg5": dict(kind="gemm", M=32768, N=32768, K=32768, scaling="strong",
                 desc="fp32 GEMM 32768^3, A/C row-blocks sharded over ranks, B replicated (BASELINE config 5)"),
    "cfg3": dict(kind="conv", W=224, H=224, C=64, kW=3, kH=3, F=64, batch=1, scaling="weak",
                 desc="im2col conv 224x224x64 -> 64 filters 3x3, zero border (BASELINE config 3)"),
    "cfg4": dict(kind="conv", W=56, H=56, C=256, kW=3, kH=3, F=256, batch=256, scaling="strong",
                 desc="im2col conv 256 x (56x56x256 -> 256 filters 3x3), batch sharded over ranks (BASELINE config 4)"),
}

# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the dominant kernel, from the ncu
# captures summarised under profiles/ (gemm_tf32_kernel_cfg2.md, im2col_pack_kernel_cfg3.md)
NCU_TRAFFIC_BYTES = {("cfg2", "3xtf32", "gemm"): 727.8e6, ("cfg2", "strict", "gemm"): 731.1e6, ("cfg3", "3xtf32", "pack"): 70.7e6,
                     ("cfg3", "strict", "pack"): 70.7e6,
                     ("cfg4", "strict", "gemm"): 2594e6, ("cfg4", "3xtf32", "gemm"): 2515e6}

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                    bf16_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), basis="measured")
    return dict(hbm_gbs=FALLBACK_HBM_GBS, bf16_tflops=FALLBACK_BF16_TFLOPS, bf16_sustained=1400.0, basis="fallback")


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples of one GPU while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(gpu_index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        # samples under load: the upper half of what was seen
        load = sorted(sm)[len(sm) // 2:] if sm else []
        return {"sm_mhz": statistics.median(load) if load else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# --------------------------------------------------------------------------------------------
# reference arm: the reference's own CPU GEMM (oracle/_ref/decx_ref_cpu) on the host cores
# --------------------------------------------------------------------------------------------
def run_reference(args, wl, name):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    from oracle import oracle as o

    base = {"impl": "reference", "metric": "fp32_gemm_conv_tflops", "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": wl["scaling"],
            "vs_baseline": None, "dtype": "f32", "data": "synthetic (seeded uniform [-1,1))",
            "config": {"workload": name, "desc": wl["desc"]}, "gpu_launches": 0}
    if not o.ref_cpu_available():
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/decx_ref_cpu is not built"}))
        return
    if wl["kind"] == "gemm":
        M, N, K = wl["M"], wl["N"], wl["K"]
    else:  # the reference has no CPU convolution: its GEMM on the convolution's column-matrix shape
        g = o.conv_geometry(wl["W"], wl["H"], wl["C"], wl["kW"], wl["kH"], 1)
        M, N, K = g[3], o.ceil4(wl["F"]), g[4]
    N = (N + 15) // 16 * 16
    # bounded sample: a row-block of the workload sized so that steps+warmup stay within ~2 minutes
    tx, ty = o.ref_cpu_threads(4096, N)
    probe_m = 128 * tx
    try:
        t_probe = o.ref_cpu_gemm(probe_m, N, K, reps=2, split=(tx, ty))["best_s"]
    except Exception as ex:
        print(json.dumps({"impl": "reference", "unavailable": f"reference CPU GEMM did not run: {str(ex)[:160]}"}))
        return
    budget_s = 120.0 / max(args.steps + args.warmup, 1)
    rows = int(min(M, max(probe_m, budget_s / max(t_probe, 1e-6) * probe_m)))
    rows = max(probe_m, rows // (32 * tx) * (32 * tx))
    if wl["kind"] == "conv":
        rows = min(rows, (M // (32 * tx)) * (32 * tx)) or probe_m
    try:
        r = o.ref_cpu_gemm(rows, N, K, reps=args.steps + args.warmup, split=(tx, ty), timeout=900)
    except Exception as ex:
        print(json.dumps({"impl": "reference", "unavailable": f"reference CPU GEMM did not run: {str(ex)[:160]}"}))
        return
    tx, ty = (int(v) for v in r["split"].split("x"))
    tflops = 2.0 * rows * N * K / r["median_s"] / 1e12
    sample = f"{rows} of {M} rows x N={N} x K={K}, decx::sgemm_caller<{tx},{ty}>, median of {args.steps + args.warmup} runs"
    base.update(value=tflops, ms_per_step=r["median_s"] * 1e3 * (M / rows),
                cpu_baseline={"value": tflops, "unit": "TFLOP/s", "cores": tx * ty, "kind": "reference", "sample": sample},
                e2e={"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0})
    print(json.dumps(base))


# --------------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS))
    ap.add_argument("--mode", default="strict", choices=["strict", "3xtf32", "1xtf32", "f16"],
                    help="strict = 3xTF32 with chunked IEEE accumulation (the default of the DECX-facing layer); "
                         "3xtf32 = tensor core accumulates over all of K; 1xtf32 = plain TF32; f16 = the fp16 overloads")
    ap.add_argument("--tile", type=int, default=0)
    ap.add_argument("--algo", default="implicit", choices=["explicit", "implicit"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--pack-variant", type=int, default=0, help="0 copy-engine pack, 1 staged, 2 direct (explicit convolution)")
    ap.add_argument("--batch", type=int, default=0, help="override the image count of a convolution workload")
    ap.add_argument("--gather", action="store_true", help="also all-gather the C row-blocks over NCCL (timed separately)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--e2e-steps", type=int, default=0, help="steps of the host-resident leg (default min(steps, 10))")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    wl = dict(WORKLOADS[args.workload])
    if args.batch > 0 and wl["kind"] == "conv":
        wl["batch"] = args.batch
        wl["desc"] += f" [batch overridden to {args.batch}]"
    if args.impl == "reference":
        return run_reference(args, wl, args.workload)

    import numpy as np  # noqa: F401
    import torch
    import torch.distributed as dist

    import backup_1_b200 as b
    from backup_1_b200 import shard

    rank, world, local = dist_env()
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    else:
        torch.cuda.set_device(local)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU fallback)")
    dev = torch.device(f"cuda:{local}")
    ctx = b.Context(local)
    ctx.set_pack_variant(args.pack_variant)
    mode = {"3xtf32": b.GEMM_3XTF32, "1xtf32": b.GEMM_1XTF32, "strict": b.GEMM_3XTF32_STRICT, "f16": b.GEMM_1XTF32}[args.mode]
    if args.mode == "f16" and wl["kind"] != "gemm":
        raise SystemExit("--mode f16 applies to the GEMM workloads")
    algo = b.CONV_EXPLICIT if args.algo == "explicit" else b.CONV_IMPLICIT
    ts = torch.cuda.Stream(device=dev)
    st = ts.cuda_stream
    peaks = load_peaks()

    # ---- operands resident in HBM -------------------------------------------------------------
    if wl["kind"] == "gemm":
        M, N, K = wl["M"], wl["N"], wl["K"]
        if wl["scaling"] == "strong":
            r0, r1 = shard.gemm_row_shard(M, world, rank)
            M_rank, row0 = r1 - r0, r0
        else:
            M_rank, row0 = M, rank * M
        dA = torch.empty((M_rank, K), device=dev); dB = torch.empty((K, N), device=dev); dD = torch.empty((M_rank, N), device=dev)
        ctx.fill_uniform(dA, M_rank, K, K, 1, first_index=row0 * K)
        ctx.fill_uniform(dB, K, N, N, 2)
        flops_rank = 2.0 * M_rank * N * K
        touched = (M_rank * K + K * N) * 4 * (3 if args.mode in ("3xtf32", "strict") else 2) + M_rank * N * 4

        def step():
            ctx.gemm(M_rank, N, K, dA, K, dB, N, dD, N, mode=mode, tile=args.tile, stream=st)

        if args.mode == "f16":          # the fp16 overloads: half operands and result, fp32 accumulation
            dA, dB, dD = dA.half(), dB.half(), dD.half()
            touched = ((M_rank * K + 2 * K * N) + M_rank * N) * 2

            def step():  # noqa: F811
                ctx.gemm_f16(M_rank, N, K, dA, K, dB, N, dD, N, stream=st)

        hA = torch.empty((M_rank, K), pin_memory=True, dtype=dA.dtype); hB = torch.empty((K, N), pin_memory=True, dtype=dA.dtype)
        hD = torch.empty((M_rank, N), pin_memory=True, dtype=dA.dtype)
        hA.copy_(dA); hB.copy_(dB)
        esz = dA.element_size()
        h2d, d2h = (M_rank * K + K * N) * esz, M_rank * N * esz

        def step_host():
            if args.mode == "f16":
                ctx.gemm_f16_host(M_rank, N, K, hA.data_ptr(), K, hB.data_ptr(), N, hD.data_ptr(), N)
            else:
                ctx.gemm_host(M_rank, N, K, hA.data_ptr(), K, hB.data_ptr(), N, hD.data_ptr(), N, mode=mode, tile=args.tile)
    else:
        W, H, C, kW, kH, F, batch = (wl[k] for k in ("W", "H", "C", "kW", "kH", "F", "batch"))
        if wl["scaling"] == "strong":
            b0, b1 = shard.conv_batch_shard(batch, world, rank)
            nb, img0 = b1 - b0, b0
        else:
            nb, img0 = batch, rank * batch
        g = b.conv_geometry(W, H, C, kW, kH, F, 1)
        dp, wp, kwp = (C + 3) // 4 * 4, (W + 3) // 4 * 4, (kW + 3) // 4 * 4
        # padded tensors; padding of a DECX tensor is zero: for these configs W, C, F are multiples of 4
        assert W % 4 == 0 and C % 4 == 0 and F % 4 == 0 and kW == 3
        dS = torch.empty((nb, H, wp, dp), device=dev)
        ctx.fill_uniform(dS, nb * H * wp, dp, dp, 4, first_index=img0 * H * wp * dp)
        dF = torch.zeros((F, kH, kwp, dp), device=dev)
        tmpF = torch.empty((F, kH, kW, dp), device=dev)
        ctx.fill_uniform(tmpF, F * kH * kW, dp, dp, 5)
        ctx.synchronize()
        dF[:, :, :kW, :] = tmpF
        dO = torch.empty((nb, g.out_h, g.eq_w, g.Np), device=dev)
        flops_rank = 2.0 * nb * (H * W) * (kW * kH * C) * F
        touched = dS.numel() * 4 + nb * g.M * g.Kp * 4 * (3 if args.mode in ("3xtf32", "strict") else 1) + dO.numel() * 4

        def step():
            ctx.conv2_im2col(dS, W, H, C, dF, kW, kH, F, dO, flag=1, batch=nb, mode=mode, algo=algo, stream=st)

        hS = torch.empty(dS.shape, pin_memory=True); hF = torch.empty(dF.shape, pin_memory=True)
        hO = torch.empty(dO.shape, pin_memory=True)
        hS.copy_(dS); hF.copy_(dF)
        h2d, d2h = (hS.numel() + hF.numel()) * 4, hO.numel() * 4

        def step_host():
            ctx.conv2_im2col_host(hS.data_ptr(), W, H, C, hF.data_ptr(), kW, kH, F, hO.data_ptr(), flag=1, batch=nb,
                                  mode=mode, algo=algo)
    ctx.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    # ---- device-resident leg -------------------------------------------------------------------
    for _ in range(args.warmup):
        step()
    ctx.synchronize()
    sampler = ClockSampler(local) if rank == 0 else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = ctx.launches()
    barrier()
    e0.record(ts)
    for _ in range(args.steps):
        step()
    e1.record(ts)
    barrier()
    ctx.synchronize()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    launches = int(sum_over_ranks(ctx.launches() - launches0))
    clocks = sampler.stop() if sampler else None
    total_flops = sum_over_ranks(flops_rank)
    value = total_flops * args.steps / (ms_total * 1e-3) / 1e12

    # ---- per-kernel times of the same steps (separate pass so the events do not sit in the timed region)
    ctx.profile_enable(True)
    for _ in range(args.steps):
        step()
    prof = ctx.profile_read()
    ctx.profile_enable(False)
    tot_ms = sum(v["ms"] for v in prof.values()) or 1.0
    dom = max(prof, key=lambda k: prof[k]["ms"])
    shares = {k: round(v["ms"] / tot_ms, 4) for k, v in prof.items() if v["launches"]}
    if dom == "gemm":
        avg_ms = prof["gemm"]["ms"] / prof["gemm"]["launches"]
        launches_per_step = prof["gemm"]["launches"] / args.steps
        ach = flops_rank / launches_per_step / (avg_ms * 1e-3) / 1e12
        tf32 = peaks["bf16_tflops"] / 2.0
        peak = {"3xtf32": tf32 / 3.0, "strict": tf32 / 3.0, "1xtf32": tf32, "f16": peaks["bf16_tflops"]}[args.mode]
        # DRAM traffic of one launch from the ncu capture of the same workload (profiles/); a rank of a strong-scaling
        # run launches on its share of the images, and the traffic of this kernel grows with the images
        traffic = NCU_TRAFFIC_BYTES.get((args.workload, args.mode, "gemm")) if args.tile == 0 else None
        if traffic is not None and wl["kind"] == "conv":
            traffic = traffic * nb / wl["batch"] if (algo == b.CONV_IMPLICIT and not args.batch) else None
        roofline = {"bound": "tensor", "kernel": "decxb_gemm_tf32_kernel", "achieved": ach, "peak": peak, "unit": "TFLOP/s",
                    "frac": ach / peak, "traffic": traffic,
                    "peak_basis": f"{peaks['basis']} bf16 dense burst {peaks['bf16_tflops']} TFLOP/s"
                                  + {"3xtf32": " / 2 (TF32) / 3 (3xTF32)", "strict": " / 2 (TF32) / 3 (3xTF32)", "1xtf32": " / 2 (TF32)",
                                     "f16": " (fp16 runs at the bf16 rate)"}[args.mode],
                    "avg_launch_ms": avg_ms, "time_shares": shares}
    else:
        # HBM-bound kernel: algorithmic bytes = what it must read plus what it must write
        k = prof[dom]
        avg_ms = k["ms"] / k["launches"]
        per_step = k["launches"] / args.steps
        if dom == "pack":
            packs = 2 if args.mode in ("3xtf32", "strict") else 1                    # hi and lo parts are packed separately
            alg = packs * (H * wp * dp + g.M * g.Kp) * 4 * nb / per_step   # read tensor, write column matrix
            kname = "decxb_im2col_pack_tma_kernel"
        elif wl["kind"] == "conv":
            alg = 3 * g.M * g.Kp * 4 * nb / per_step                      # read column matrix, write hi and lo
            kname = "decxb_split_rows_kernel"
        else:
            alg = 3 * (M_rank * K + K * N) * 4 / per_step                 # read A and B, write hi and lo of each
            kname = "decxb_split_rows_kernel + decxb_split_transpose_kernel"
        ach = alg / (avg_ms * 1e-3) / 1e9 if alg else None
        roofline = {"bound": "hbm", "kernel": kname, "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": ach / peaks["hbm_gbs"] if ach else None, "traffic": NCU_TRAFFIC_BYTES.get((args.workload, args.mode, dom)),
                    "peak_basis": f"{peaks['basis']} copy bandwidth", "avg_launch_ms": avg_ms, "time_shares": shares,
                    "per_class_ms_per_step": {c: round(v["ms"] / args.steps, 5) for c, v in prof.items() if v["launches"]}}

    # ---- host-resident leg (e2e) -----------------------------------------------------------------
    e2e_steps = args.e2e_steps or min(args.steps, 10)
    for _ in range(2):
        step_host()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        step_host()
    torch.cuda.synchronize()
    t_e2e = max_over_ranks(time.perf_counter() - t0)
    e2e_val = total_flops * e2e_steps / t_e2e / 1e12

    # ---- optional all-gather of the result row-blocks ----------------------------------------------
    gather = None
    if args.gather and world > 1:
        flat = (dD if wl["kind"] == "gemm" else dO).reshape(-1)
        full = torch.empty(flat.numel() * world, device=dev)
        for _ in range(2):
            dist.all_gather_into_tensor(full, flat)
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        dist.all_gather_into_tensor(full, flat)
        g1.record()
        torch.cuda.synchronize()
        gms = max_over_ranks(g0.elapsed_time(g1))
        gather = {"ms": gms, "bytes_per_rank": flat.numel() * 4,
                  "busbw_gbs": flat.numel() * 4 * (world - 1) / (gms * 1e-3) / 1e9}

    # ---- CPU baseline (rank 0, N = 1 only) ------------------------------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            from oracle import oracle as o

            if wl["kind"] == "gemm":
                cm, cn, ck = wl["M"], wl["N"], wl["K"]
            else:
                cm, cn, ck = g.M, (g.Np + 15) // 16 * 16, g.Kp
            if o.ref_cpu_available():
                tx, ty = o.ref_cpu_threads(4096, cn)
                probe = o.ref_cpu_gemm(128 * tx, cn, ck, reps=2, split=(tx, ty))["best_s"]
                rows = int(min(cm, max(128 * tx, 3.0 / max(probe, 1e-6) * 128 * tx)))
                rows = max(128 * tx, rows // (32 * tx) * (32 * tx))
                r = o.ref_cpu_gemm(rows, cn, ck, reps=5, split=(tx, ty), timeout=600)
                cpu = {"value": 2.0 * rows * cn * ck / r["best_s"] / 1e12, "unit": "TFLOP/s", "cores": tx * ty,
                       "kind": "reference",
                       "sample": f"decx::sgemm_caller<{tx},{ty}> on {rows} of {cm} rows x N={cn} x K={ck}, best of 5"}
            else:
                import numpy as np

                rows = 256
                A = o.fill_uniform(rows * ck, 1).reshape(rows, ck); B = o.fill_uniform(ck * cn, 2).reshape(ck, cn)
                t0 = time.perf_counter(); o.gemm_fmaf(A, B); dt = time.perf_counter() - t0
                cpu = {"value": 2.0 * rows * cn * ck / dt / 1e12, "unit": "TFLOP/s", "cores": o.lib().decxo_num_threads(),
                       "kind": "port", "sample": f"oracle fma chain on {rows} of {cm} rows"}
        except Exception as ex:  # the baseline is reported, never required
            cpu = {"value": None, "unit": "TFLOP/s", "cores": 0, "kind": "reference", "sample": f"failed: {ex}"}

    if rank == 0:
        line = {
            "metric": "fp32_gemm_conv_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_total / args.steps, "higher_is_better": True,
            "scaling": wl["scaling"], "vs_baseline": None, "dtype": {"3xtf32": "f32 (3xTF32 tensor-core split, fp32 accumulate)", "strict": "f32 (3xTF32, K chunks added in IEEE fp32)",
                      "1xtf32": "tf32", "f16": "f16 (fp32 accumulate)"}[args.mode], "data": "synthetic (seeded uniform [-1,1), generated on device)",
            "config": {"workload": args.workload, "desc": wl["desc"], "mode": args.mode, "tile": args.tile,
                       "algo": args.algo if wl["kind"] == "conv" else None,
                       "l2": (f"each step touches {touched / 1e6:.0f} MB (operands, split/column scratch, result) "
                              + ("> 126 MB L2, no flush needed" if touched > 126e6 else
                                 "< 126 MB L2: steps run back to back WITHOUT a flush")),
                       "parallelism": f"row/batch shards x{world}, no data-path collective"},
            "roofline": roofline, "cpu_baseline": cpu,
            "e2e": {"value": e2e_val, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "ms_per_step": t_e2e / e2e_steps * 1e3},
            "gpu_launches": launches, "clocks": clocks,
        }
        if gather:
            line["allgather"] = gather
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    ctx.close()


if __name__ == "__main__":
    main()
