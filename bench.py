#!/usr/bin/env python
"""Benchmark of the fp32 GEMM / im2col-convolution hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--workload NAME] [--mode strict|3xtf32|1xtf32|f16]
    python bench.py --impl reference ...     # the reference's CPU code on the host cores
    python bench.py --workload pcie ...      # pinned-copy bandwidth per rank, alone and all ranks together

One "step" is one pass of the hot path over one batch of synthetic input.  Default workload:
BASELINE config 5, the fp32 GEMM 32768^3 in the default (3xTF32, chunked IEEE accumulation) mode;
with N GPUs the rows of A and C are sharded over the ranks and B is replicated (strong scaling,
no data-path collective; the all-gather of C is timed separately and reported beside it).
Prints ONE JSON line on rank 0.  `value` is device-timed (CUDA events on the launch stream, max
over ranks) with operands resident in HBM; `e2e` runs the host-resident entry point (pinned host
buffers, H2D and D2H inside the timed region; with N GPUs on the sharded GEMM a rank uploads its
rows of A and its 1/N of B, and the ranks all-gather B on the device: `--no-host-gather` makes every
rank upload all of B instead); `also` carries the other BASELINE configurations measured in the
same process.
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
    "pcie": dict(kind="pcie", scaling="weak", desc="pinned host<->device copies of 128 MiB per rank"),
}
ALSO = [("gemm16k", 5), ("cfg2", 40), ("cfg4", 8), ("cfg3", 60), ("cfg1", 60)]   # (workload, timed steps)

# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the dominant kernel, from the ncu captures
# summarised under profiles/; the per-flop figure below is scaled to a launch by the launch's flops
NCU_TRAFFIC_BYTES = {("cfg2", "3xtf32", "gemm"): 727.8e6, ("cfg2", "strict", "gemm"): 737.8e6,
                     ("cfg3", "3xtf32", "pack"): 70.7e6, ("cfg3", "strict", "pack"): 70.7e6,
                     ("cfg4", "strict", "gemm"): 2530e6, ("cfg4", "3xtf32", "gemm"): 2515e6,
                     ("cfg2", "tf32bf16", "gemm"): 738.0e6,
                     # one launch of the whole 32768^3 product on one GPU (275.23 GB read + 4.44 GB written)
                     ("cfg5", "strict", "gemm"): 279.67e9}
# DRAM bytes per algorithmic flop of the 256 x 256-tile GEMM with the block pairs aligned, from the single-pass capture at
# 16384^3 in profiles/gemm_tf32_kernel_16384.md (35.44 GB read + 1.10 GB written per 2 * 16384^3 flop).  A wave of 74
# tiles reads 17.25 operand panels whatever K and N are, so the traffic of a larger product grows with its flops.
NCU_TRAFFIC_PER_FLOP = {("strict", "gemm"): (35.44e9 + 1.10e9) / (2.0 * 16384 ** 3)}

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
L2_BYTES = 126e6


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                    bf16_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), basis="measured")
    return dict(hbm_gbs=FALLBACK_HBM_GBS, bf16_tflops=FALLBACK_BF16_TFLOPS, bf16_sustained=1400.0, basis="fallback")


class ClockSampler:
    """nvidia-smi samples of one GPU while a timed region runs.  The clock under load is the
    median over the samples whose GPU utilisation is at least 50 % (under a power cap the loaded
    clock is the LOWER one, so the clock itself cannot select them)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,utilization.gpu,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_id: str, period_ms: int = 50):
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", str(period_ms), "-i", gpu_id],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.12)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        rows, mx, reasons = [], [], set()
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                rows.append((float(f[1]), float(f[3]), float(f[4])))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        load = [r for r in rows if r[2] >= 50.0]
        basis = "samples with utilization.gpu >= 50 %"
        if not load and rows:           # region shorter than the sampling period: take what there is, say so
            load, basis = rows, "all samples (none reached 50 % utilisation: region shorter than the sampling period)"
        return {"sm_mhz": statistics.median(r[0] for r in load) if load else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "power_w": round(statistics.median(r[1] for r in load), 1) if load else None,
                "samples": len(rows), "samples_under_load": len(load) if basis.startswith("samples") else 0, "selected": basis}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def touched_bytes(wl, mode, world):
    """Bytes one step touches per rank (operands, split/column scratch, result): decides whether L2 must be flushed."""
    parts = 3 if mode in ("3xtf32", "strict", "tf32bf16") else 2
    if wl["kind"] == "gemm":
        m = wl["M"] // world if wl["scaling"] == "strong" else wl["M"]
        esz = 2 if mode == "f16" else 4
        return (m * wl["K"] + wl["K"] * wl["N"]) * esz * parts + m * wl["N"] * esz
    nb = max(wl["batch"] // world, 1) if wl["scaling"] == "strong" else wl["batch"]
    return nb * wl["H"] * wl["W"] * (wl["C"] * 4 * parts + wl["F"] * 4) + wl["F"] * wl["kW"] * wl["kH"] * wl["C"] * 4 * parts


def config_for(args, wl, name, world):
    """The `config` object of the JSON line; both arms print the same one for the same command line."""
    if wl["kind"] == "pcie":
        return {"workload": name, "desc": wl["desc"]}
    t = touched_bytes(wl, args.mode, world)
    return {"workload": name, "desc": wl["desc"], "mode": args.mode, "tile": args.tile, "wave_align": args.wave_align,
            "algo": args.algo if wl["kind"] == "conv" else None,
            "l2": (f"each step touches {t / 1e6:.0f} MB per GPU (operands, split scratch, result): "
                   + ("larger than the 126 MB L2, steps run back to back" if t > 2 * L2_BYTES else
                      "not larger than twice the 126 MB L2: a 512 MB buffer is written between timed steps (L2 flush)")),
            "parallelism": (f"{'row' if wl['kind'] == 'gemm' else 'image'} shards x{world} (strong scaling), no data-path collective"
                            if wl["scaling"] == "strong" else f"one replica of the workload per GPU x{world} (weak scaling), no collective")}


# --------------------------------------------------------------------------------------------
# reference arm: the reference's own CPU code (oracle/_ref/decx_ref_cpu) on the host cores
# --------------------------------------------------------------------------------------------
def cpu_reference_measure(wl, budget_s, reps):
    """Times the reference's CPU GEMM (decx::sgemm_caller) on a bounded row-block of the workload; for a
    convolution workload also the im2col pack (the oracle's restatement of the reference's pack kernel, all
    host threads; the reference has no CPU pack) on the images that row-block covers, and reports the sum."""
    from oracle import oracle as o

    if wl["kind"] == "gemm":
        M, N, K = wl["M"], wl["N"], wl["K"]
    else:
        g = o.conv_geometry(wl["W"], wl["H"], wl["C"], wl["kW"], wl["kH"], 1)
        M, N, K = g[3], o.ceil4(wl["F"]), g[4]            # rows of ONE image's column matrix
    N16 = (N + 15) // 16 * 16
    tx, ty = o.ref_cpu_threads(4096, N16)
    probe_m = 128 * tx
    t_probe = o.ref_cpu_gemm(probe_m, N16, K, reps=2, split=(tx, ty))["best_s"]
    rows = int(min(M, max(probe_m, budget_s / max(t_probe, 1e-6) * probe_m)))
    rows = max(probe_m, rows // (32 * tx) * (32 * tx))
    r = o.ref_cpu_gemm(rows, N16, K, reps=reps, split=(tx, ty), timeout=900)
    tx, ty = (int(v) for v in r["split"].split("x"))
    t_gemm, t_best = r["median_s"], r["best_s"]
    flops = 2.0 * rows * N * K           # algorithmic flops of those rows (N as the workload has it)
    sample = f"decx::sgemm_caller<{tx},{ty}> on {rows} of {M} rows x N={N16} x K={K}, median of {reps}"
    t_pack = 0.0
    if wl["kind"] == "conv":
        src = o.make_tensor(wl["W"], wl["H"], wl["C"], 4)
        o.im2col_pack(src, wl["W"], wl["C"], wl["kW"], wl["kH"], 1)
        ts = []
        for _ in range(3):
            t0 = time.perf_counter()
            o.im2col_pack(src, wl["W"], wl["C"], wl["kW"], wl["kH"], 1)
            ts.append(time.perf_counter() - t0)
        t_pack = statistics.median(ts) * rows / M       # the share of the pack that those rows are
        flops = 2.0 * rows * wl["F"] * wl["kW"] * wl["kH"] * wl["C"] * (wl["W"] / o.ceil4(wl["W"]))
        sample += f" + im2col pack of that share of one image on {o.lib().decxo_num_threads()} threads ({t_pack * 1e3:.2f} ms)"
    total_units = M * (wl.get("batch", 1) if wl["kind"] == "conv" else 1)
    return {"tflops": flops / (t_gemm + t_pack) / 1e12, "tflops_best": flops / (t_best + t_pack) / 1e12,
            "step_s_extrapolated": (t_gemm + t_pack) * total_units / rows, "cores": tx * ty, "sample": sample}


def run_reference(args, wl, name):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    from oracle import oracle as o

    base = {"impl": "reference", "metric": "fp32_gemm_conv_tflops", "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": wl["scaling"],
            "vs_baseline": None, "dtype": "f32", "data": "synthetic (seeded uniform [-1,1))",
            "config": config_for(args, wl, name, max(args.gpus, 1)), "gpu_launches": 0}
    if not o.ref_cpu_available():
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/decx_ref_cpu is not built"}))
        return
    try:
        m = cpu_reference_measure(wl, 120.0 / max(args.steps + args.warmup, 1), args.steps + args.warmup)
    except Exception as ex:
        print(json.dumps({"impl": "reference", "unavailable": f"reference CPU GEMM did not run: {str(ex)[:160]}"}))
        return
    base.update(value=m["tflops"], ms_per_step=m["step_s_extrapolated"] * 1e3,
                cpu_baseline={"value": m["tflops"], "unit": "TFLOP/s", "cores": m["cores"], "kind": "reference", "sample": m["sample"]},
                e2e={"value": m["tflops"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0})
    print(json.dumps(base))


# --------------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------------
class Bench:
    def __init__(self, args):
        import torch
        import torch.distributed as dist

        import backup_1_b200 as b

        self.torch, self.dist, self.b, self.args = torch, dist, b, args
        self.rank, self.world, self.local = dist_env()
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device (no CPU fallback)")
        # every rank keeps to its own host cores, and allocates its pinned buffers after that
        try:
            cpus = sorted(os.sched_getaffinity(0))
            if self.world > 1 and len(cpus) >= 2 * self.world:
                per = len(cpus) // self.world
                os.sched_setaffinity(0, cpus[self.local * per:(self.local + 1) * per])
        except (AttributeError, OSError):
            pass
        torch.cuda.set_device(self.local)
        if self.world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=torch.device(f"cuda:{self.local}"))
        self.dev = torch.device(f"cuda:{self.local}")
        self.ctx = b.Context(self.local)
        self.ctx.set_pack_variant(args.pack_variant)
        self.ctx.set_wave_align(args.wave_align)
        self.ts = torch.cuda.Stream(device=self.dev)
        self.st = self.ts.cuda_stream
        self.peaks = load_peaks()
        self.flush_buf = None
        # nvidia-smi's name for this rank's GPU: its UUID (indices differ under CUDA_VISIBLE_DEVICES)
        self.gpu_id = str(self.local)
        try:
            uid = "GPU-" + str(torch.cuda.get_device_properties(self.local).uuid)
            if subprocess.run(["nvidia-smi", "-i", uid, "--query-gpu=index", "--format=csv,noheader"],
                              capture_output=True, timeout=20).returncode == 0:
                self.gpu_id = uid
        except Exception:
            pass

    # ---- plumbing ---------------------------------------------------------------------------
    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def _reduce(self, x: float, op) -> float:
        if self.world == 1:
            return x
        t = self.torch.tensor([x], device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=op)
        return float(t.item())

    def max_over_ranks(self, x):
        return self._reduce(x, self.dist.ReduceOp.MAX) if self.world > 1 else x

    def sum_over_ranks(self, x):
        return self._reduce(x, self.dist.ReduceOp.SUM) if self.world > 1 else x

    def per_rank(self, x: float):
        if self.world == 1:
            return [x]
        t = self.torch.zeros(self.world, device=self.dev, dtype=self.torch.float64)
        t[self.rank] = x if x is not None else -1.0
        self.dist.all_reduce(t)
        return [round(float(v), 4) for v in t.tolist()]

    def flush_l2(self):
        if self.flush_buf is None:
            self.flush_buf = self.torch.empty(512 << 20, dtype=self.torch.uint8, device=self.dev)
        with self.torch.cuda.stream(self.ts):
            self.flush_buf.fill_(1)

    # ---- a workload resident in HBM -------------------------------------------------------------
    def build(self, name, wl, mode_name, host_leg):
        torch, b, ctx, dev, world, rank = self.torch, self.b, self.ctx, self.dev, self.world, self.rank
        from backup_1_b200 import shard
        args = self.args
        mode = {"3xtf32": b.GEMM_3XTF32, "1xtf32": b.GEMM_1XTF32, "strict": b.GEMM_3XTF32_STRICT, "f16": b.GEMM_1XTF32,
                "tf32bf16": b.GEMM_TF32_2XBF16}[mode_name]
        algo = b.CONV_EXPLICIT if args.algo == "explicit" else b.CONV_IMPLICIT
        w = {"name": name, "wl": wl, "mode": mode_name}
        if wl["kind"] == "gemm":
            M, N, K = wl["M"], wl["N"], wl["K"]
            if wl["scaling"] == "strong":
                r0, r1 = shard.gemm_row_shard(M, world, rank)
                M_rank, row0 = r1 - r0, r0
            else:
                M_rank, row0 = M, rank * M
            dA = torch.empty((M_rank, K), device=dev); dB = torch.empty((K, N), device=dev)
            if wl["scaling"] == "strong" and world > 1 and mode_name != "f16":
                w["full"] = torch.empty((M, N), device=dev)          # the whole result: this rank's rows are computed in place
                dD = w["full"][row0:row0 + M_rank]
            else:
                dD = torch.empty((M_rank, N), device=dev)
            ctx.fill_uniform(dA, M_rank, K, K, 1, first_index=row0 * K)
            ctx.fill_uniform(dB, K, N, N, 2)
            w.update(flops=2.0 * M_rank * N * K, M_rank=M_rank, row0=row0, dA=dA, dB=dB, dD=dD, K_err=K)

            def step():
                ctx.gemm(M_rank, N, K, dA, K, dB, N, dD, N, mode=mode, tile=args.tile, stream=self.st)

            if mode_name == "f16":          # the fp16 overloads: half operands and result, fp32 accumulation
                dA, dB, dD = dA.half(), dB.half(), dD.half()
                w.update(dA=dA, dB=dB, dD=dD)

                def step():  # noqa: F811
                    ctx.gemm_f16(M_rank, N, K, dA, K, dB, N, dD, N, stream=self.st)
            w["step"] = step
            if mode_name not in ("f16", "tf32bf16"):
                def prepare():
                    w["pb"] = ctx.prepare_b(K, N, dB, N, mode=mode, stream=self.st)

                def step_prepared():
                    ctx.gemm_prepared(M_rank, dA, K, w["pb"], dD, N, tile=args.tile, stream=self.st)

                def release():
                    ctx.release_b(w.pop("pb"), stream=self.st)
                w.update(prepare=prepare, step_prepared=step_prepared, release=release)
            if host_leg:
                hA = torch.empty((M_rank, K), pin_memory=True, dtype=dA.dtype); hB = torch.empty((K, N), pin_memory=True, dtype=dA.dtype)
                hD = torch.empty((M_rank, N), pin_memory=True, dtype=dA.dtype)
                hA.copy_(dA); hB.copy_(dB)
                esz = dA.element_size()
                w.update(h2d=(M_rank * K + K * N) * esz, d2h=M_rank * N * esz, host=(hA, hB, hD))

                def step_host():
                    if mode_name == "f16":
                        ctx.gemm_f16_host(M_rank, N, K, hA.data_ptr(), K, hB.data_ptr(), N, hD.data_ptr(), N)
                    else:
                        # the host-resident entry does not take the bf16 cross-product mode: its leg runs the default mode
                        ctx.gemm_host(M_rank, N, K, hA.data_ptr(), K, hB.data_ptr(), N, hD.data_ptr(), N,
                                      mode=b.GEMM_3XTF32_STRICT if mode_name == "tf32bf16" else mode, tile=args.tile)
                w["step_host"] = step_host
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
            dS = torch.empty((max(nb, 1), H, wp, dp), device=dev)
            ctx.fill_uniform(dS, max(nb, 1) * H * wp, dp, dp, 4, first_index=img0 * H * wp * dp)
            dF = torch.zeros((F, kH, kwp, dp), device=dev)
            tmpF = torch.empty((F, kH, kW, dp), device=dev)
            ctx.fill_uniform(tmpF, F * kH * kW, dp, dp, 5)
            ctx.synchronize()
            dF[:, :, :kW, :] = tmpF
            if wl["scaling"] == "strong" and world > 1:
                w["full"] = torch.empty((batch, g.out_h, g.eq_w, g.Np), device=dev)
                dO = w["full"][img0:img0 + max(nb, 1)]
            else:
                dO = torch.empty((max(nb, 1), g.out_h, g.eq_w, g.Np), device=dev)
            w.update(flops=2.0 * nb * (H * W) * (kW * kH * C) * F, nb=nb, dS=dS, dF=dF, dO=dO, g=g, K_err=kW * kH * C,
                     dims=(W, H, C, kW, kH, F, dp, wp))

            def step():
                if nb:
                    ctx.conv2_im2col(dS, W, H, C, dF, kW, kH, F, dO, flag=1, batch=nb, mode=mode, algo=algo, stream=self.st)
            w["step"] = step

            def prepare():
                w["pf"] = ctx.conv_prepare_filters(dF, kW, kH, C, F, mode=mode, algo=algo, stream=self.st)

            def step_prepared():
                if nb:
                    ctx.conv2_im2col_prepared(dS, W, H, w["pf"], dO, flag=1, batch=nb, stream=self.st)

            def release():
                ctx.conv_release_filters(w.pop("pf"), stream=self.st)
            w.update(prepare=prepare, step_prepared=step_prepared, release=release)
            if host_leg:
                hS = torch.empty(dS.shape, pin_memory=True); hF = torch.empty(dF.shape, pin_memory=True)
                hO = torch.empty(dO.shape, pin_memory=True)
                hS.copy_(dS); hF.copy_(dF)
                w.update(h2d=(hS.numel() + hF.numel()) * 4, d2h=hO.numel() * 4, host=(hS, hF, hO))

                def step_host():
                    if nb:
                        ctx.conv2_im2col_host(hS.data_ptr(), W, H, C, hF.data_ptr(), kW, kH, F, hO.data_ptr(), flag=1, batch=nb,
                                              mode=mode, algo=algo)
                w["step_host"] = step_host
        ctx.synchronize()
        w["flush"] = touched_bytes(wl, mode_name, world) <= 2 * L2_BYTES
        return w

    def check(self, w):
        """max|D - D_ref| / (K max|a| max|b|) of sampled results of the last step against an fp64 product of the
        same device operands (computed here with torch in double precision: a checker, not the product path)."""
        torch = self.torch
        if w["mode"] == "f16":
            return None
        if w["wl"]["kind"] == "gemm":
            dA, dB, dD = w["dA"], w["dB"], w["dD"]
            M, N = dD.shape
            rows = torch.unique(torch.tensor([0, 1, M // 2, M // 2 + 129, M - 128, M - 1], device=self.dev).clamp_(0, M - 1))
            cols = torch.unique(torch.cat([torch.arange(0, min(256, N)), torch.arange(max(N - 256, 0), N)]).to(self.dev))
            ref = dA[rows].double() @ dB[:, cols].double()
            return float((dD[rows][:, cols].double() - ref).abs().max()) / w["K_err"]
        if not w["nb"]:
            return 0.0
        W, H, C, kW, kH, F, dp, wp = w["dims"]
        img = w["nb"] - 1
        x = w["dS"][img, :, :W, :C].permute(2, 0, 1).unsqueeze(0).double()                 # [1][C][H][W]
        k = w["dF"][:, :, :kW, :C].permute(0, 3, 1, 2).double()                              # [F][C][kH][kW]
        ref = torch.nn.functional.conv2d(x, k, padding=(kH // 2, kW // 2))[0]                # [F][H][W]
        got = w["dO"][img, :, :W, :F].permute(2, 0, 1).double()
        return float((got - ref).abs().max()) / w["K_err"]

    # ---- timing ---------------------------------------------------------------------------------
    def measure(self, w, steps, warmup, sample_clocks=True, profile_steps=None):
        torch, ctx = self.torch, self.ctx
        step = w["step"]
        for _ in range(warmup):
            step()
        ctx.synchronize()
        sampler = ClockSampler(self.gpu_id) if sample_clocks else None
        launches0 = ctx.launches()
        self.barrier()
        if w["flush"]:
            # small workload: L2 is flushed between the timed steps, every step has its own pair of events
            evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
            for e0, e1 in evs:
                self.flush_l2()
                e0.record(self.ts)
                step()
                e1.record(self.ts)
            self.barrier()
            ms_rank = sum(e0.elapsed_time(e1) for e0, e1 in evs)
        else:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(self.ts)
            for _ in range(steps):
                step()
            e1.record(self.ts)
            self.barrier()
            ms_rank = e0.elapsed_time(e1)
        ctx.synchronize()
        ms_total = self.max_over_ranks(ms_rank)
        launches = int(self.sum_over_ranks(ctx.launches() - launches0))
        clocks = sampler.stop() if sampler else None
        total_flops = self.sum_over_ranks(w["flops"])
        res = {"value": total_flops * steps / (ms_total * 1e-3) / 1e12, "ms_per_step": ms_total / steps, "launches": launches,
               "clocks": clocks, "total_flops": total_flops, "ms_rank_per_step": ms_rank / steps}
        # per-kernel times in a separate pass of the same steps, so that the events do not sit in the timed region
        psteps = profile_steps or steps
        ctx.profile_enable(True)
        for _ in range(psteps):
            if w["flush"]:
                self.flush_l2()
            step()
        prof = ctx.profile_read()
        ctx.profile_enable(False)
        res["prof"], res["prof_steps"] = prof, psteps
        return res

    def measure_prepared(self, w, steps):
        """The same step with the weights (B / the filter bank) prepared once outside the timed region
        (decxb_gemm_prepare_b / decxb_conv_prepare_filters).  Plain and prepared steps alternate, each between its own
        pair of events, so that both see the same clocks; returns (ms per prepared step, ms per plain step), max over ranks."""
        if "prepare" not in w:
            return None
        torch = self.torch
        w["prepare"]()
        for _ in range(2):
            w["step_prepared"](); w["step"]()
        self.ctx.synchronize()
        self.barrier()
        evs = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(steps)]
        for e in evs:
            if w["flush"]:
                self.flush_l2()
            e[0].record(self.ts); w["step"](); e[1].record(self.ts)
            if w["flush"]:
                self.flush_l2()
            e[2].record(self.ts); w["step_prepared"](); e[3].record(self.ts)
        self.barrier()
        plain = sum(e[0].elapsed_time(e[1]) for e in evs) / steps
        prepared = sum(e[2].elapsed_time(e[3]) for e in evs) / steps
        w["release"]()
        self.ctx.synchronize()
        return self.max_over_ranks(prepared), self.max_over_ranks(plain)

    def roofline(self, w, res):
        peaks, wl, mode, args = self.peaks, w["wl"], w["mode"], self.args
        prof, psteps = res["prof"], res["prof_steps"]
        tot_ms = sum(v["ms"] for v in prof.values()) or 1.0
        dom = max(prof, key=lambda k: prof[k]["ms"])
        shares = {k: round(v["ms"] / tot_ms, 4) for k, v in prof.items() if v["launches"]}
        if dom == "gemm":
            avg_ms = prof["gemm"]["ms"] / prof["gemm"]["launches"]
            per_step = prof["gemm"]["launches"] / psteps
            flops_launch = w["flops"] / per_step
            ach = flops_launch / (avg_ms * 1e-3) / 1e12
            div = {"3xtf32": 6.0, "strict": 6.0, "1xtf32": 2.0, "f16": 1.0, "tf32bf16": 4.0}[mode]
            long_step = avg_ms * per_step >= 100.0          # a kernel inside a seconds-long region runs under the power cap
            bf16 = peaks["bf16_sustained"] if long_step else peaks["bf16_tflops"]
            peak = bf16 / div
            traffic = NCU_TRAFFIC_BYTES.get((w["name"], mode, "gemm")) if args.tile == 0 else None
            if traffic is not None and wl["kind"] == "gemm" and (w["M_rank"] != wl["M"] or args.wave_align == 0):
                traffic = None                      # the capture is of the unsharded, aligned launch
            if traffic is not None and wl["kind"] == "conv":
                traffic = traffic * w["nb"] / wl["batch"] if (args.algo == "implicit" and not args.batch) else None
            traffic_note = None
            if (traffic is None and args.tile == 0 and args.wave_align != 0 and wl["kind"] == "gemm" and (mode, "gemm") in NCU_TRAFFIC_PER_FLOP
                    and w["M_rank"] >= 4096 and wl["N"] >= 4096 and wl["K"] >= 4096):
                traffic = NCU_TRAFFIC_PER_FLOP[(mode, "gemm")] * flops_launch
                traffic_note = "scaled by flops from the single-pass ncu capture of one 16384^3 launch (profiles/gemm_tf32_kernel_16384.md)"
            r = {"bound": "tensor", "kernel": "decxb_gemm_tf32_kernel", "achieved": ach, "peak": peak, "unit": "TFLOP/s",
                 "frac": ach / peak, "traffic": traffic,
                 "peak_basis": (f"{peaks['basis']} bf16 dense {'sustained' if long_step else 'burst'} {bf16} TFLOP/s"
                                + {"3xtf32": " / 2 (TF32) / 3 (3xTF32)", "strict": " / 2 (TF32) / 3 (3xTF32)", "1xtf32": " / 2 (TF32)",
                                   "f16": " (fp16 runs at the bf16 rate)",
                                   "tf32bf16": " / 4 (one TF32 product and two bf16 products at twice the TF32 rate = two TF32 products)"}[mode]
                                + (": steps of >= 100 ms run under the power cap" if long_step else ": a step is shorter than 100 ms")),
                 "frac_burst_basis": ach / (peaks["bf16_tflops"] / div), "frac_sustained_basis": ach / (peaks["bf16_sustained"] / div),
                 "avg_launch_ms": avg_ms, "time_shares": shares}
            if traffic_note:
                r["traffic_basis"] = traffic_note
            if r["frac"] > 1.0:
                r["note"] = ("frac > 1: the denominator is derived from a cuBLAS bf16 run, not a TF32 measurement; "
                             "frac_of_probe compares with this library's own tcgen05 kind::tf32 probe on the same GPU")
            return r
        # HBM-bound kernel: algorithmic bytes = what it must read plus what it must write
        k = prof[dom]
        avg_ms = k["ms"] / k["launches"]
        per_step = k["launches"] / psteps
        if dom == "pack":
            W, H, C, kW, kH, F, dp, wp = w["dims"]
            packs = 2 if mode in ("3xtf32", "strict") else 1                    # hi and lo parts are packed separately
            alg = packs * (H * wp * dp + w["g"].M * w["g"].Kp) * 4 * w["nb"] / per_step   # read tensor, write column matrix
            kname = "decxb_im2col_pack_tma_kernel"
        elif wl["kind"] == "conv":
            alg = 3 * w["g"].M * w["g"].Kp * 4 * w["nb"] / per_step
            kname = "decxb_split_rows_kernel"
        else:
            alg = 3 * (w["M_rank"] * wl["K"] + wl["K"] * wl["N"]) * 4 / per_step
            kname = "decxb_split_rows_kernel + decxb_split_transpose_kernel"
        ach = alg / (avg_ms * 1e-3) / 1e9 if alg else None
        return {"bound": "hbm", "kernel": kname, "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": ach / peaks["hbm_gbs"] if ach else None, "traffic": NCU_TRAFFIC_BYTES.get((w["name"], mode, dom)),
                "peak_basis": f"{peaks['basis']} copy bandwidth", "avg_launch_ms": avg_ms, "time_shares": shares}

    def probes(self):
        """This GPU's own tensor ceilings: the tcgen05 kind::tf32 issue peak and the ceiling of the 3xTF32 k-step,
        as a burst (about 60 ms) and sustained (about 1.5 s, under the power cap), with the SM clock seen."""
        out = {}
        for key, pattern in (("tf32_peak_probe", 0), ("x3_ceiling_probe", 1)):
            burst = self.ctx.probe_tensor_peak(pattern, 60.0)
            s = ClockSampler(self.gpu_id)
            sus = self.ctx.probe_tensor_peak(pattern, 1500.0)
            c = s.stop()
            mhz = c.get("sm_mhz")
            out[key] = {"burst_tflops": round(burst["algorithmic_tflops"], 1), "sustained_tflops": round(sus["algorithmic_tflops"], 1),
                        "sustained_sm_mhz": mhz, "sustained_power_w": c.get("power_w"), "reasons": c.get("reasons"),
                        "tensor_flop_per_clk_per_sm": round(sus["tensor_tflops"] * 1e12 / (mhz * 1e6 * sus["sms"]), 1) if mhz else None,
                        "unit": "TFLOP/s of algorithmic flops (tensor flops / MMAs per k-step)"}
        return out


def run_pcie(bench, args):
    """Pinned-copy bandwidth: every rank copies 128 MiB host->device and device->host, each direction alone, both
    together, and then all ranks at the same time."""
    torch = bench.torch
    n = 128 << 20
    h_up = torch.empty(n, dtype=torch.uint8, pin_memory=True); h_dn = torch.empty(n, dtype=torch.uint8, pin_memory=True)
    d_up = torch.empty(n, dtype=torch.uint8, device=bench.dev); d_dn = torch.empty(n, dtype=torch.uint8, device=bench.dev)
    s_up, s_dn = torch.cuda.Stream(device=bench.dev), torch.cuda.Stream(device=bench.dev)

    def run(up, dn, reps=8):
        e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        torch.cuda.synchronize()
        e[0].record(s_up); e[2].record(s_dn)
        for _ in range(reps):
            if up:
                with torch.cuda.stream(s_up):
                    d_up.copy_(h_up, non_blocking=True)
            if dn:
                with torch.cuda.stream(s_dn):
                    h_dn.copy_(d_dn, non_blocking=True)
        e[1].record(s_up); e[3].record(s_dn)
        torch.cuda.synchronize()
        return (n * reps / (e[0].elapsed_time(e[1]) * 1e-3) / 1e9 if up else None,
                n * reps / (e[2].elapsed_time(e[3]) * 1e-3) / 1e9 if dn else None)

    run(True, True, 2)
    res = {}
    for label in ("alone", "all_ranks"):
        if label == "alone":
            # one rank at a time
            vals = []
            for r in range(bench.world):
                bench.barrier()
                if r == bench.rank:
                    up, _ = run(True, False); _, dn = run(False, True); bu, bd = run(True, True)
                    vals = [up, dn, bu, bd]
                bench.barrier()
        else:
            bench.barrier()
            up, _ = run(True, False); bench.barrier()
            _, dn = run(False, True); bench.barrier()
            bu, bd = run(True, True); bench.barrier()
            vals = [up, dn, bu, bd]
        res[label] = {k: bench.per_rank(v) for k, v in zip(("h2d_gbs", "d2h_gbs", "both_h2d_gbs", "both_d2h_gbs"), vals)}
    if bench.rank == 0:
        agg = sum(res["all_ranks"]["both_h2d_gbs"]) + sum(res["all_ranks"]["both_d2h_gbs"])
        print(json.dumps({"metric": "pinned_copy_gbs", "value": agg, "unit": "GB/s", "n_gpus": bench.world, "steps": 8, "warmup": 2,
                          "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
                          "config": config_for(args, WORKLOADS["pcie"], "pcie", bench.world), "per_rank": res,
                          "note": "value = sum over ranks and both directions with every rank copying both ways at once"}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="cfg5", choices=sorted(WORKLOADS))
    ap.add_argument("--mode", default="strict", choices=["strict", "3xtf32", "1xtf32", "f16", "tf32bf16"],
                    help="strict = 3xTF32 with chunked IEEE accumulation (the default of the DECX-facing layer); "
                         "3xtf32 = tensor core accumulates over all of K; 1xtf32 = plain TF32; f16 = the fp16 overloads; "
                         "tf32bf16 = hi*hi in TF32 and the two cross products in bf16 (opt-in, GEMM workloads)")
    ap.add_argument("--tile", type=int, default=0)
    ap.add_argument("--algo", default="implicit", choices=["explicit", "implicit"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--pack-variant", type=int, default=0, help="0 copy-engine pack, 1 staged, 2 direct (explicit convolution)")
    ap.add_argument("--batch", type=int, default=0, help="override the image count of a convolution workload")
    ap.add_argument("--no-gather", action="store_true", help="skip the all-gather of the result blocks (N > 1)")
    ap.add_argument("--wave-align", type=int, default=1, choices=[0, 1, 2],
                    help="GEMM wave alignment: 1 cooperative launches (default), 2 plain launches (profilers; also beside a transfer), 0 off")
    ap.add_argument("--comm-ctas", type=int, default=0,
                    help="thread blocks per NCCL kernel for the transfers that overlap a GEMM (0 = the library's default, two per rank)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-also", action="store_true", help="skip the other BASELINE configurations")
    ap.add_argument("--no-probe", action="store_true", help="skip the tensor-ceiling probes")
    ap.add_argument("--no-host-gather", action="store_true",
                    help="N > 1: every rank uploads the whole B in the host-resident leg instead of a share that the ranks all-gather")
    ap.add_argument("--e2e-steps", type=int, default=0, help="steps of the host-resident leg (default min(steps, 3) for the large workloads)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    wl = dict(WORKLOADS[args.workload])
    if args.batch > 0 and wl["kind"] == "conv":
        wl["batch"] = args.batch
        wl["desc"] += f" [batch overridden to {args.batch}]"
    if args.impl == "reference":
        if wl["kind"] == "pcie":
            print(json.dumps({"impl": "reference", "unavailable": "the pcie workload measures this host's copies only"}))
            return
        return run_reference(args, wl, args.workload)
    if args.mode in ("f16", "tf32bf16") and wl["kind"] != "gemm":
        raise SystemExit(f"--mode {args.mode} applies to the GEMM workloads")

    bench = Bench(args)
    torch, dist, ctx, rank, world = bench.torch, bench.dist, bench.ctx, bench.rank, bench.world
    if wl["kind"] == "pcie":
        run_pcie(bench, args)
        if world > 1:
            dist.destroy_process_group()
        ctx.close()
        return

    # ---- headline workload: device-resident leg -----------------------------------------------------
    w = bench.build(args.workload, wl, args.mode, host_leg=True)
    big = w["flops"] >= 1e13
    res = bench.measure(w, args.steps, args.warmup, profile_steps=min(args.steps, 5) if big else None)
    roofline = bench.roofline(w, res)
    ms_prepared = bench.measure_prepared(w, min(args.steps, 5) if big else args.steps)
    err = bench.check(w)
    err = bench.max_over_ranks(err) if err is not None else None

    # ---- the NCCL layer (N > 1): B's shares in the host-resident leg, the result blocks after it ---------
    comm, comm_error = None, None
    if world > 1 and wl["scaling"] == "strong" and not (args.no_gather and args.no_host_gather):
        if args.comm_ctas > 0:
            os.environ["DECXB_COMM_MAX_CTAS"] = str(args.comm_ctas)
        # the layer loads NCCL at run time: if it cannot on this box, every rank goes on without it (said in the line)
        try:
            uid = [bench.b.Comm.unique_id() if rank == 0 else None]
        except Exception as ex:
            uid, comm_error = [None], str(ex)[:200]
        dist.broadcast_object_list(uid, src=0)
        if uid[0] is not None:
            try:
                comm = bench.b.Comm(ctx, world, rank, uid[0], timeout_ms=120000)
            except Exception as ex:
                comm_error = str(ex)[:200]
        if bench.max_over_ranks(0.0 if comm is not None else 1.0) > 0.0:
            if comm is not None:
                comm.close()
            comm = None
            comm_error = comm_error or "the communicator could not be created on another rank"

    # ---- host-resident leg (e2e) ---------------------------------------------------------------------
    e2e_how = ("decxb_gemm_f16_host" if args.mode == "f16" else "decxb_gemm_f32_host / decxb_conv2_im2col_f32_host" if world == 1 else
               "decxb_gemm_f32_host / decxb_conv2_im2col_f32_host per rank on its shard: every rank uploads all of the shared operand")
    if comm is not None and wl["kind"] == "gemm" and args.mode != "f16" and not args.no_host_gather:
        hA, hB, hD = w["host"]
        M, N, K = wl["M"], wl["N"], wl["K"]
        mode_h = {"3xtf32": bench.b.GEMM_3XTF32, "1xtf32": bench.b.GEMM_1XTF32, "strict": bench.b.GEMM_3XTF32_STRICT,
                  "tf32bf16": bench.b.GEMM_3XTF32_STRICT}[args.mode]
        w["step_host"] = lambda: comm.gemm_rowshard_host(M, N, K, hA.data_ptr(), K, hB.data_ptr(), N, hD.data_ptr(), N,
                                                         mode=mode_h, tile=args.tile)
        k0, k1 = bench.b.shard_range(K, world, rank)
        w["h2d"] = (w["M_rank"] * K + (k1 - k0) * N) * 4
        e2e_how = ("decxb_gemm_f32_rowshard_host: a rank uploads its rows of A and its 1/N of B's rows, the ranks all-gather B "
                   "on the device (NCCL over NVLink), then each multiplies its rows and sends them home")
    e2e_steps = args.e2e_steps or (min(args.steps, 3) if big else min(args.steps, 10))
    for _ in range(1 if big else 2):
        w["step_host"]()
    bench.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        w["step_host"]()
    torch.cuda.synchronize()
    t_e2e = bench.max_over_ranks(time.perf_counter() - t0)
    e2e_val = res["total_flops"] * e2e_steps / t_e2e / 1e12
    h2d, d2h = w["h2d"], w["d2h"]
    e2e_err = None
    if "rowshard_host" in e2e_how:
        # the rows that came home equal the rows the device-resident leg left in HBM (same mode and shapes: bit for bit)
        hD = w["host"][2]
        if args.mode != "tf32bf16" and w["M_rank"] > 0:
            same = all(torch.equal(hD[sl].to(bench.dev), w["dD"][sl]) for sl in (slice(0, 64), slice(-64, None)))
            e2e_err = bench.max_over_ranks(0.0 if same else 1.0)
    w.pop("host", None); w.pop("step_host", None)

    # ---- gathering the result blocks over NCCL (N > 1): after the step, and overlapped with it ------------
    gather = None
    if comm is not None and not args.no_gather and "full" in w:
        from backup_1_b200 import shard

        full = w["full"]
        total_units = wl["M"] if wl["kind"] == "gemm" else wl["batch"]
        unit_bytes = full[0].numel() * 4
        mine = (w["M_rank"] if wl["kind"] == "gemm" else w["nb"]) * unit_bytes

        def timed(fn, reps):
            fn(); comm.synchronize()
            bench.barrier()
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            g0.record(bench.ts)
            for _ in range(reps):
                fn()
            g1.record(bench.ts)
            comm.synchronize()
            bench.barrier()
            return bench.max_over_ranks(g0.elapsed_time(g1)) / reps

        gms = timed(lambda: comm.allgather_blocks(full, unit_bytes, total_units, stream=bench.st), 2)
        gather = {"ms": gms, "bytes_per_rank": mine, "busbw_gbs": mine * (world - 1) / (gms * 1e-3) / 1e9,
                  "nccl_thread_blocks": {"alone": 32, "beside_a_gemm": args.comm_ctas or min(16, max(4, 2 * world))},
                  "how": "decxb_comm_allgather_blocks (NCCL, in place in the whole-result array) after the step, timed alone"}
        if wl["kind"] == "gemm":
            mode = {"3xtf32": bench.b.GEMM_3XTF32, "1xtf32": bench.b.GEMM_1XTF32, "strict": bench.b.GEMM_3XTF32_STRICT,
                    "tf32bf16": bench.b.GEMM_3XTF32_STRICT}[args.mode]
            A_rows, Bm = w["dA"], w["dB"]
            for groups in (1, 3, 4, 6):
                ms = timed(lambda: comm.gemm_rowshard_gather(wl["M"], wl["N"], wl["K"], A_rows, wl["K"], Bm, wl["N"], full, groups=groups,
                                                             mode=mode, tile=args.tile, stream=bench.st), max(2, min(args.steps, 5)))
                gather[f"step_with_gather_ms_groups{groups}"] = ms
            # a peer's gathered rows equal what this rank computes for a sample of those rows itself (fp64 checker)
            peer = (rank + 1) % world
            p0, p1 = shard.gemm_row_shard(wl["M"], world, peer)
            rows = torch.tensor([p0, (p0 + p1) // 2, p1 - 1], device=bench.dev)
            a = torch.empty((3, wl["K"]), device=bench.dev)
            for i, r in enumerate(rows.tolist()):
                ctx.fill_uniform(a[i], 1, wl["K"], wl["K"], 1, first_index=r * wl["K"])
            ctx.synchronize()
            cols = torch.arange(0, 256, device=bench.dev)
            ref = a.double() @ Bm[:, cols].double()
            gather["gathered_rows_max_norm_err"] = bench.max_over_ranks(float((full[rows][:, cols].double() - ref).abs().max()) / wl["K"])
            best = min((gather[f"step_with_gather_ms_groups{g}"], g) for g in (3, 4, 6))
            gather["overlapped_groups"] = best[1]
            gather["step_with_overlapped_gather_ms"] = best[0]
            gather["how_overlapped"] = ("decxb_gemm_f32_rowshard_gather: the rank's rows in row-panel groups, each group sent to the peers "
                                        "(NCCL send/receive on a side stream) while the next is multiplied")
        full = None
    if comm is not None:
        comm.close()
    per_rank_ms = bench.per_rank(res["ms_rank_per_step"])
    per_rank_mhz = bench.per_rank(res["clocks"]["sm_mhz"] if res["clocks"] else None)

    # ---- this GPU's tensor ceilings --------------------------------------------------------------------
    probes = None
    if not args.no_probe and rank == 0:
        try:
            probes = bench.probes()
        except Exception as ex:  # reported, never required
            probes = {"failed": str(ex)[:200]}
    bench.barrier()
    if probes and "x3_ceiling_probe" in probes and roofline.get("bound") == "tensor" and args.mode in ("strict", "3xtf32"):
        long_step = roofline["avg_launch_ms"] >= 100.0
        den = probes["x3_ceiling_probe"]["sustained_tflops" if long_step else "burst_tflops"]
        roofline["frac_of_probe"] = roofline["achieved"] / den
        roofline["probe_basis"] = (f"this GPU's 3xTF32 k-step ceiling, {'sustained' if long_step else 'burst'} {den} TFLOP/s "
                                   "(decxb_probe_tensor_peak pattern 1: MMAs only, operands resident in shared memory)")
    if probes:
        roofline.update(probes)

    # ---- the other BASELINE configurations, same process ------------------------------------------------
    also = []
    del w
    torch.cuda.empty_cache(); ctx.release_cached()
    if not args.no_also and args.mode not in ("f16", "tf32bf16"):
        for name, steps in ALSO:
            if name == args.workload:
                continue
            wl2 = dict(WORKLOADS[name])
            try:
                w2 = bench.build(name, wl2, args.mode, host_leg=False)
                r2 = bench.measure(w2, steps, 3, sample_clocks=False)
                rf2 = bench.roofline(w2, r2)
                mp2 = bench.measure_prepared(w2, steps)
                e2 = bench.check(w2)
                also.append({"workload": name, "value": r2["value"], "ms_per_step": r2["ms_per_step"], "steps": steps,
                             "ms_per_step_prepared_weights": mp2[0] if mp2 else None,
                             "ms_per_step_plain_alternating": mp2[1] if mp2 else None,
                             "kernel": rf2["kernel"], "kernel_tflops_or_gbs": rf2["achieved"], "kernel_frac": rf2["frac"],
                             "kernel_avg_launch_ms": rf2["avg_launch_ms"], "time_shares": rf2["time_shares"],
                             "max_norm_err": bench.max_over_ranks(e2) if e2 is not None else None,
                             "scaling": wl2["scaling"], "l2_flushed_between_steps": w2["flush"]})
                del w2
            except Exception as ex:
                also.append({"workload": name, "failed": str(ex)[:200]})
            torch.cuda.empty_cache(); ctx.release_cached()

    if not args.no_also and args.mode == "strict":
        try:     # the opt-in TF32 + 2 x bf16 mode on the north-star shape, for the record
            w3 = bench.build("gemm16k", dict(WORKLOADS["gemm16k"]), "tf32bf16", host_leg=False)
            r3 = bench.measure(w3, 5, 3, sample_clocks=False)
            rf3 = bench.roofline(w3, r3)
            e3 = bench.check(w3)
            also.append({"workload": "gemm16k", "mode": "tf32bf16 (opt-in: TF32 hi*hi + two bf16 cross products)", "value": r3["value"],
                         "ms_per_step": r3["ms_per_step"], "steps": 5, "kernel_tflops_or_gbs": rf3["achieved"],
                         "kernel_avg_launch_ms": rf3["avg_launch_ms"], "time_shares": rf3["time_shares"],
                         "max_norm_err": bench.max_over_ranks(e3) if e3 is not None else None})
            del w3
        except Exception as ex:
            also.append({"workload": "gemm16k", "mode": "tf32bf16", "failed": str(ex)[:200]})
        torch.cuda.empty_cache(); ctx.release_cached()

    # ---- CPU baseline (rank 0, N = 1 only) ------------------------------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            from oracle import oracle as o

            if o.ref_cpu_available():
                m = cpu_reference_measure(wl, 4.0, 3)
                cpu = {"value": m["tflops"], "unit": "TFLOP/s", "cores": m["cores"], "kind": "reference", "sample": m["sample"]}
            else:
                rows, ck, cn = 256, (wl["K"] if wl["kind"] == "gemm" else 2304), (wl["N"] if wl["kind"] == "gemm" else 256)
                cn = min(cn, 4096)
                A = o.fill_uniform(rows * ck, 1).reshape(rows, ck); B = o.fill_uniform(ck * cn, 2).reshape(ck, cn)
                t0 = time.perf_counter(); o.gemm_fmaf(A, B); dt = time.perf_counter() - t0
                cpu = {"value": 2.0 * rows * cn * ck / dt / 1e12, "unit": "TFLOP/s", "cores": o.lib().decxo_num_threads(),
                       "kind": "port", "sample": f"oracle fma chain on {rows} rows x {cn} columns x K={ck}"}
        except Exception as ex:  # the baseline is reported, never required
            cpu = {"value": None, "unit": "TFLOP/s", "cores": 0, "kind": "reference", "sample": f"failed: {ex}"}

    if rank == 0:
        clocks = res["clocks"] or {}
        clocks.update(per_rank_sm_mhz=per_rank_mhz, ms_times_mhz=[round(a * b, 1) if b and b > 0 else None
                                                                  for a, b in zip(per_rank_ms, per_rank_mhz)])
        line = {
            "metric": "fp32_gemm_conv_tflops", "value": res["value"], "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True,
            "scaling": wl["scaling"], "vs_baseline": None,
            "dtype": {"3xtf32": "f32 (3xTF32 tensor-core split, fp32 accumulate)", "strict": "f32 (3xTF32, K chunks added in IEEE fp32)",
                      "1xtf32": "tf32", "f16": "f16 (fp32 accumulate)",
                      "tf32bf16": "f32 (TF32 hi*hi + two bf16 cross products, K chunks added in IEEE fp32)"}[args.mode],
            "data": "synthetic (seeded uniform [-1,1), generated on device)",
            "config": config_for(args, wl, args.workload, world),
            "max_norm_err": err, "max_norm_err_basis": "sampled results against an fp64 product of the same operands, / (K max|a| max|b|)",
            "roofline": roofline, "cpu_baseline": cpu,
            "e2e": {"value": e2e_val, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "ms_per_step": t_e2e / e2e_steps * 1e3, "how": e2e_how,
                    **({"rows_differing_from_device_leg": e2e_err} if e2e_err is not None else {})},
            "ms_per_step_prepared_weights": ms_prepared[0] if ms_prepared else None,
            "ms_per_step_plain_alternating": ms_prepared[1] if ms_prepared else None,
            "prepared_weights_note": ("the same step with B / the filter bank split and laid out once outside the timed region "
                                      "(decxb_gemm_prepare_b, decxb_conv_prepare_filters), alternating with plain steps so that both see "
                                      "the same clocks; `value` uses the plain entry, which prepares them on every call"),
            "gpu_launches": res["launches"], "clocks": clocks, "per_rank_ms_per_step": per_rank_ms, "also": also,
        }
        if comm_error:
            line["comm_unavailable"] = comm_error
        if gather:
            line["allgather"] = gather
            line["value_with_gather"] = res["total_flops"] / ((res["ms_per_step"] + gather["ms"]) * 1e-3) / 1e12
            if "step_with_overlapped_gather_ms" in gather:
                line["value_with_overlapped_gather"] = res["total_flops"] / (gather["step_with_overlapped_gather_ms"] * 1e-3) / 1e12
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    ctx.close()


if __name__ == "__main__":
    main()
