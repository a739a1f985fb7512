#!/usr/bin/env python3
"""Benchmark of the matmul_fw + matmul_bw hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (one "step" = one forward plus both backward products over the batch):
non-broadcast batched square GEMM, fp32 in 3xTF32 mode: A and B each
Shape({4096,4096}, batch 8) ~ N(0, 0.02), upstream gradient N(0,1), seeded
synthetic data.  With N GPUs every rank holds a full batch-8 shard of its own
(weak scaling; the products of different batch elements are independent, so the
data path has no collective).

Prints ONE JSON line on rank 0.  `value` is algorithmic GFLOP/s (2*m*n*k per product,
three products per batch element) over all ranks with operands resident in HBM;
`e2e` is the same metric through the host-buffer entry points of the C ABI with the
host<->device copies inside the timed region.

--impl reference times the reference's own CPU implementation of the path (its
Naive device compiled from its sources into oracle/_ref, else the C restatement
under oracle/) on a bounded sample of the same workload.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_DIM = 4096
BATCH = 8
METRIC = "matmul_fw_bw_gflops"
FLOPS_PER_STEP = 3 * 2 * N_DIM ** 3 * BATCH        # 3,298,534,883,328
# CPU sample: one batch element, restricted to the first 64 columns of b / gy
SAMPLE_DK = 64
SAMPLE_FLOPS = 3 * 2 * N_DIM * N_DIM * SAMPLE_DK


def set_batch(batch):
    global BATCH, FLOPS_PER_STEP
    BATCH = batch
    FLOPS_PER_STEP = 3 * 2 * N_DIM ** 3 * BATCH


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return dict(bf16_burst=d["bf16_tflops"], bf16_sustained=d["bf16_tflops_sustained"],
                    hbm=d["hbm_gbs"], source="measured")
    except Exception:
        return dict(bf16_burst=1590.0, bf16_sustained=1400.0, hbm=6650.0, source="fallback")


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.stop_flag = index, [], False

    def run(self):
        if self._run_nvml():
            return
        while not self.stop_flag:
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True,
                                     timeout=5).stdout.strip()
                if out:
                    self.samples.append([c.strip() for c in out.split(",")])
            except Exception:
                pass
            time.sleep(0.05)

    def _run_nvml(self):
        """Reads the same counters through NVML (read-only calls), every 20 ms."""
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            mx = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
            bits = [(pynvml.nvmlClocksEventReasonHwSlowdown, 2), (pynvml.nvmlClocksEventReasonHwThermalSlowdown, 3),
                    (pynvml.nvmlClocksEventReasonSwThermalSlowdown, 4), (pynvml.nvmlClocksEventReasonSwPowerCap, 5)]
        except Exception:
            return False
        while not self.stop_flag:
            try:
                row = [str(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)), str(mx), "", "", "", ""]
                r = pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)
                for bit, col in bits:
                    row[col] = "Active" if (r & bit) else "Not Active"
                self.samples.append(row)
            except Exception:
                pass
            time.sleep(0.02)
        return True

    def summary(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        mhz, reasons, mx = [], set(), None
        for s in self.samples:
            try:
                mhz.append(float(s[0]))
                mx = float(s[1])
            except Exception:
                continue
            for i, nm in enumerate(names):
                if len(s) > 2 + i and s[2 + i].lower().startswith("active"):
                    reasons.add(nm)
        mhz.sort()
        return dict(sm_mhz=(mhz[len(mhz) // 2] if mhz else None), sm_max_mhz=mx,
                    reasons=sorted(reasons), samples=len(mhz))


def cpu_sample():
    """Times fw + bw of the reference CPU path on the bounded sample.  Returns (seconds, kind, cores)."""
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as ol
    di, dj, dk = N_DIM, N_DIM, SAMPLE_DK
    rng = np.random.default_rng(0)
    a = (rng.standard_normal(di * dj) * 0.02).astype(np.float32)
    b = (rng.standard_normal(dj * dk) * 0.02).astype(np.float32)
    gy = rng.standard_normal(di * dk).astype(np.float32)
    ga0, gb0 = np.zeros(di * dj, np.float32), np.zeros(dj * dk, np.float32)
    if ol.have_ref():
        _, t_fw = ol.ref_fw(a, b, di, dj, dk, 1, 1)
        _, _, t_bw = ol.ref_bw(a, b, gy, ga0, gb0, di, dj, dk, 1, 1)
        return t_fw + t_bw, "reference", 1
    os.environ["OMP_NUM_THREADS"] = "1"   # the reference's CPU devices are single-threaded
    t0 = time.perf_counter()
    ol.fw_naive(a, b, di, dj, dk, 1, 1)
    ol.bw_naive(a, b, gy, ga0, gb0, di, dj, dk, 1, 1)
    return time.perf_counter() - t0, "port", 1


SAMPLE_TEXT = ("one batch element, first %d columns of b and gy: fw {4096,4096}.{4096,%d} plus both "
               "backward products, %d FLOP" % (SAMPLE_DK, SAMPLE_DK, SAMPLE_FLOPS))


def run_reference(args, rank):
    if rank != 0:
        return
    for _ in range(args.warmup):
        cpu_sample()
    total, kind, cores = 0.0, "port", 1
    for _ in range(args.steps):
        t, kind, cores = cpu_sample()
        total += t
    gflops = SAMPLE_FLOPS * args.steps / total / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": gflops, "unit": "GFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": gflops, "unit": "GFLOP/s", "cores": cores, "kind": kind, "sample": SAMPLE_TEXT},
        "e2e": {"value": gflops, "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus):
    return {"workload": "batched_square_gemm_4096x4096x4096_batch%d_fp32_3xtf32_fw_bw" % BATCH,
            "shape": [N_DIM, N_DIM, N_DIM], "batch_per_gpu": BATCH, "global_batch": BATCH * n_gpus,
            "mode": "3xTF32", "flops_per_step_per_gpu": FLOPS_PER_STEP,
            "l2": "every operand (512 MiB) is larger than L2 (126 MB); no flush needed",
            "parallelism": "batch-sharded x%d, no collective on the data path" % n_gpus}


def run_ours(args, rank, local_rank, world):
    import torch
    import primitiv_b200 as pb

    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = pb.Context(local_rank)
    mode = pb.MODE_FP32_3XTF32
    n, bs = N_DIM, BATCH
    g = torch.Generator(device="cuda")
    g.manual_seed(1234 + rank)
    a = torch.randn(n * n * bs, generator=g, device="cuda") * 0.02
    b = torch.randn(n * n * bs, generator=g, device="cuda") * 0.02
    gy = torch.randn(n * n * bs, generator=g, device="cuda")
    y = torch.empty(n * n * bs, device="cuda")
    ga = torch.zeros(n * n * bs, device="cuda")
    gb = torch.zeros(n * n * bs, device="cuda")
    P = lambda t: t.data_ptr()

    def step():
        ctx.matmul_fw(mode, P(a), P(b), P(y), n, n, n, bs, bs)
        ctx.matmul_bw(mode, P(a), P(b), P(gy), P(ga), P(gb), n, n, n, bs, bs)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    ctx.profile_read()
    ctx.profile_enable(True)
    launches0 = ctx.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    ctx.profile_enable(False)
    prof = ctx.profile_read()
    launches = ctx.launch_count() - launches0
    sampler.stop_flag = True
    sampler.join(timeout=3)
    assert ctx.status_poll() == 0, "a kernel reported a bounded-wait timeout"

    # ---- end to end through the host-buffer entry points (pinned host memory) ----
    e2e = None
    if not args.skip_e2e:
        e2e = run_e2e(args, ctx, mode, a, b, gy, barrier, dist, torch)
    if dist is not None:
        t = torch.tensor([ms, e2e["ms"] if e2e else 0.0], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
        if e2e:
            e2e["ms"] = float(t[1])
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    emit(args, world, ms, prof, launches, sampler, e2e)
    if dist is not None:
        dist.destroy_process_group()


def run_e2e(args, ctx, mode, a, b, gy, barrier, dist, torch):
    n, bs = N_DIM, BATCH
    P = lambda t: t.data_ptr()
    e2e_steps = max(1, min(args.steps, 3))
    hb = lambda src: src.cpu().pin_memory()
    ha, hbm, hgy = hb(a), hb(b), hb(gy)
    hy = torch.empty(n * n * bs).pin_memory()
    hga = torch.zeros(n * n * bs).pin_memory()
    hgb = torch.zeros(n * n * bs).pin_memory()

    def e2e_step():
        ctx.matmul_fw_host(mode, P(ha), P(hbm), P(hy), n, n, n, bs, bs)
        ctx.matmul_bw_host(mode, P(ha), P(hbm), P(hgy), P(hga), P(hgb), n, n, n, bs, bs)
        return float(hga[0])  # the step's result is read on the host

    e2e_step()
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(e2e_steps):
        e2e_step()
    f1.record()
    barrier()
    tensor_bytes = n * n * bs * 4
    return {"ms": f0.elapsed_time(f1), "steps": e2e_steps,
            "h2d": (2 + 5) * tensor_bytes,   # fw: a, b;  bw: a, b, gy, ga, gb (gradients hold the values added to)
            "d2h": (1 + 2) * tensor_bytes}   # y; ga, gb


def emit(args, world, ms, prof, launches, sampler, e2e):
    peaks = measured_peaks()
    ms_per_step = ms / args.steps
    value = FLOPS_PER_STEP * world / (ms_per_step * 1e-3) / 1e9
    tc_ms, tc_n = prof["gemm_tc"]
    issued_flops_per_launch = 3.0 * FLOPS_PER_STEP * args.steps / max(tc_n, 1)  # 3 TF32 passes per product
    tc_avg_ms = tc_ms / max(tc_n, 1)
    achieved = issued_flops_per_launch / (tc_avg_ms * 1e-3) / 1e12 if tc_n else 0.0
    tf32_peak = peaks["bf16_sustained"] / 2.0
    tf32_burst = peaks["bf16_burst"] / 2.0
    # DRAM bytes of one gemm_tc_kernel launch: ncu capture of the batch-2 case (1.64 GB, see profiles/),
    # scaled by the batch (independent products, traffic grows in proportion)
    traffic = 1.64e9 * BATCH / 2.0
    line = {
        "metric": METRIC, "value": value, "unit": "GFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "tf32x3 (fp32 storage, fp32 accumulate)", "data": "synthetic",
        "config": workload_config(world),
        "roofline": {
            "bound": "tensor", "kernel": "gemm_tc_kernel<chunked, cta pair>", "achieved": achieved,
            "peak": tf32_peak, "unit": "TFLOP/s", "frac": achieved / tf32_peak, "traffic": traffic,
            "frac_of_burst_peak": achieved / tf32_burst,
            "note": ("achieved = tensor-issued FLOP/s (3 TF32 passes x algorithmic 2mnk) / mean CUDA-event "
                     "duration of %d launches; peak = %s bf16 sustained / 2 (TF32 runs at half the 16-bit rate; "
                     "the timed region is a fraction of a second, so the burst figure / 2 = %.0f is given beside it); "
                     "traffic = ncu dram bytes of the batch-2 capture scaled to this batch"
                     % (tc_n, peaks["source"], tf32_burst)),
            "algorithmic_tflops_in_kernel": achieved / 3.0,
            "kernel_ms_per_step": tc_ms / args.steps, "pack_ms_per_step": prof["pack"][0] / args.steps,
        },
        "gpu_launches": int(launches),
        "clocks": sampler.summary(),
    }
    if e2e:
        per = e2e["ms"] / e2e["steps"]
        line["e2e"] = {"value": FLOPS_PER_STEP * world / (per * 1e-3) / 1e9, "unit": "GFLOP/s",
                       "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"],
                       "steps": e2e["steps"], "ms_per_step": per}
    if world == 1 and not args.skip_cpu:
        t, kind, cores = cpu_sample()
        line["cpu_baseline"] = {"value": SAMPLE_FLOPS / t / 1e9, "unit": "GFLOP/s", "cores": cores,
                                "kind": kind, "sample": SAMPLE_TEXT}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=BATCH,
                    help="batch elements per GPU (default 8 = the benchmark workload; smaller values are for "
                         "profiler captures and are marked in config.workload)")
    ap.add_argument("--skip-e2e", action="store_true", help="leave out the host-buffer leg (profiler captures)")
    ap.add_argument("--skip-cpu", action="store_true", help="leave out the CPU baseline leg (profiler captures)")
    args = ap.parse_args()
    set_batch(args.batch)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
    else:
        run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
