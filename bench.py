#!/usr/bin/env python3
"""Benchmark of the matmul_fw + matmul_bw hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Default workload (one "step" = one forward plus both backward products over the batch):
non-broadcast batched square GEMM, fp32 in 3xTF32 mode: A and B each
Shape({4096,4096}, batch 8) ~ N(0, 0.02), upstream gradient N(0,1), seeded synthetic
data.  With N GPUs every rank holds a full batch-8 shard of its own (weak scaling; the
products of different batch elements are independent, so the data path has no collective).

`--workload batched_square_3xfp16` runs the default shapes in the opt-in fp32-grade mode on the fp16
pipe.  `--workload lstm_steps` / `--workload mlp_step` run the graph-level programs of the other named
configurations (1 GPU).  `--workload batched_square_tf32` runs the same shapes in the single-pass TF32 fast mode, and
`--workload fp16_broadcast` runs the half-precision workload instead: A {8192,8192}
broadcast, B {8192,2048} x 32, fp32 accumulation, gA summed over the batch (and, with
N GPUs, all-reduced over NCCL: B, gy, y, gB are batch-sharded 32 per GPU, A is replicated).

Prints ONE JSON line on rank 0.  `value` is algorithmic GFLOP/s (2*m*n*k per product, three
products per step) over all ranks with operands resident in HBM; `e2e` is the same metric
through the host-buffer entry points of the C ABI with the host<->device copies inside the
timed region.

--impl reference times the reference's own CPU implementation of the path (its Naive
device compiled from its sources into oracle/_ref, else the C restatement under oracle/)
on a bounded sample of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "matmul_fw_bw_gflops"


class Workload:
    """Shapes in primitiv terms: a {di,dj} x ba, b {dj,dk} x bb; per-GPU batch sizes."""

    def __init__(self, name, batch):
        self.name = name
        if name == "batched_square":
            self.di = self.dj = self.dk = 4096
            self.ba = self.bb = batch if batch else 8
            self.mode_name, self.passes, self.half = "3xTF32", 3, False
            self.sa, self.sb, self.sgy = 0.02, 0.02, 1.0
            self.dtype = "tf32x3 (fp32 storage, fp32 accumulate)"
            self.sample_dk = 64
        elif name == "batched_square_tf32":
            # the same shapes in the single-pass TF32 fast mode (tolerance 2e-3 instead of 1e-5)
            self.di = self.dj = self.dk = 4096
            self.ba = self.bb = batch if batch else 8
            self.mode_name, self.passes, self.half = "TF32", 1, False
            self.sa, self.sb, self.sgy = 0.02, 0.02, 1.0
            self.dtype = "tf32 (fp32 storage, one tensor-core pass, fp32 accumulate)"
            self.sample_dk = 64
        elif name == "batched_square_3xfp16":
            # the same shapes and fp32-grade results on the fp16 pipe (row-scaled half planes, 3 passes)
            self.di = self.dj = self.dk = 4096
            self.ba = self.bb = batch if batch else 8
            self.mode_name, self.passes, self.half = "3xFP16", 3, False
            self.sa, self.sb, self.sgy = 0.02, 0.02, 1.0
            self.dtype = "f16x3 (fp32 storage, two scaled half planes per operand, fp32 accumulate)"
            self.sample_dk = 64
        elif name == "fp16_broadcast":
            self.di = self.dj = 8192
            self.dk = 2048
            self.ba, self.bb = 1, (batch if batch else 32)
            self.mode_name, self.passes, self.half = "FP16", 1, True
            self.sa, self.sb, self.sgy = 0.05, 0.05, 1.0
            self.dtype = "f16 (half storage, fp32 accumulate)"
            self.sample_dk = 16
        else:
            raise ValueError(name)
        self.bs = max(self.ba, self.bb)
        self.flops = 3 * 2 * self.di * self.dj * self.dk * self.bs
        self.sample_flops = 3 * 2 * self.di * self.dj * self.sample_dk
        self.elem = 2 if self.half else 4

    def label(self):
        if self.name == "batched_square":
            return "batched_square_gemm_4096x4096x4096_batch%d_fp32_3xtf32_fw_bw" % self.bs
        if self.name == "batched_square_3xfp16":
            return "batched_square_gemm_4096x4096x4096_batch%d_fp32_3xfp16_fw_bw" % self.bs
        if self.name == "batched_square_tf32":
            return "batched_square_gemm_4096x4096x4096_batch%d_fp32_tf32_fast_fw_bw" % self.bs
        return "fp16_a8192x8192_broadcast_b8192x2048_batch%d_fw_bw" % self.bs

    def sample_text(self):
        return ("one batch element, first %d columns of b and gy: fw {%d,%d}.{%d,%d} plus both backward "
                "products, %d FLOP" % (self.sample_dk, self.di, self.dj, self.dj, self.sample_dk, self.sample_flops))

    def config(self, n_gpus):
        collective = ("none: no broadcast operand" if self.ba == self.bb else
                      "all-reduce (sum) of the broadcast operand's gradient partial, NCCL")
        return {"workload": self.label(), "a": [self.di, self.dj, self.ba], "b": [self.dj, self.dk, self.bb],
                "batch_per_gpu": self.bs, "global_batch": self.bs * n_gpus, "mode": self.mode_name,
                "flops_per_step_per_gpu": self.flops,
                "l2": "every batched operand (>= 512 MiB) is larger than L2 (126 MB); no flush needed",
                "parallelism": "batch-sharded x%d" % n_gpus, "collective": collective}


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
    """Samples SM clock and throttle reasons of one GPU while the timed region runs (read-only)."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.stop_flag = index, [], False

    def _run_nvml(self):
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


def cpu_sample(wl):
    """Times fw + bw of the reference CPU path on the bounded sample.  Returns (seconds, kind, cores)."""
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as ol
    di, dj, dk = wl.di, wl.dj, wl.sample_dk
    rng = np.random.default_rng(0)
    a = (rng.standard_normal(di * dj) * wl.sa).astype(np.float32)
    b = (rng.standard_normal(dj * dk) * wl.sb).astype(np.float32)
    gy = (rng.standard_normal(di * dk) * wl.sgy).astype(np.float32)
    if wl.half:   # the CPU reference computes in fp32 on the half-rounded values
        a, b, gy = ol.round_to_half(a), ol.round_to_half(b), ol.round_to_half(gy)
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


def cpu_eigen_standin(wl):
    """The reference's Eigen device cannot be built here (Eigen3 is not in the image): as a labelled
    stand-in, the same three products of ONE batch element (forward, ga += gy.b^T, gb += a^T.gy) through
    the host BLAS behind torch's CPU matmul, on all host threads.  Context beside the Naive figure,
    never the baseline the speed-up is quoted against."""
    import torch
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(0)
    di, dj, dk = wl.di, wl.dj, wl.dk
    a = torch.randn(di, dj, generator=g) * wl.sa
    b = torch.randn(dj, dk, generator=g) * wl.sb
    gy = torch.randn(di, dk, generator=g) * wl.sgy
    if wl.half:
        a, b, gy = a.half().float(), b.half().float(), gy.half().float()
    ga, gb = torch.zeros(di, dj), torch.zeros(dj, dk)

    def products():
        y = a @ b
        ga.add_(gy @ b.t())
        gb.add_(a.t() @ gy)
        return y

    products()
    t0 = time.perf_counter()
    products()
    t = time.perf_counter() - t0
    return {"value": 3 * 2.0 * di * dj * dk / t / 1e9, "unit": "GFLOP/s", "cores": cores,
            "kind": "stand-in for the reference's Eigen device: host BLAS sgemm via torch CPU, fp32",
            "sample": "one batch element {%d,%d}.{%d,%d}, forward plus both backward products" % (di, dj, dj, dk)}


def run_reference(args, wl, rank):
    if rank != 0:
        return
    for _ in range(args.warmup):
        cpu_sample(wl)
    total, kind, cores = 0.0, "port", 1
    for _ in range(args.steps):
        t, kind, cores = cpu_sample(wl)
        total += t
    gflops = wl.sample_flops * args.steps / total / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": gflops, "unit": "GFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": wl.config(args.gpus),
        "cpu_baseline": {"value": gflops, "unit": "GFLOP/s", "cores": cores, "kind": kind,
                         "sample": wl.sample_text()},
        "e2e": {"value": gflops, "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args, wl, rank, local_rank, world):
    import torch
    import primitiv_b200 as pb
    from primitiv_b200.sharding import GpuBackend, ShardedMatmul, nccl_all_reduce

    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = pb.Context(local_rank)
    mode = {"FP16": pb.MODE_FP16, "TF32": pb.MODE_TF32, "3xFP16": pb.MODE_FP32_3XFP16}.get(wl.mode_name, pb.MODE_FP32_3XTF32)
    dt = torch.float16 if wl.half else torch.float32
    g = torch.Generator(device="cuda")
    g.manual_seed(1234 + rank)
    shared = torch.Generator(device="cuda")
    shared.manual_seed(99)            # a replicated operand is the same on every rank
    na, nb, ny = wl.di * wl.dj * wl.ba, wl.dj * wl.dk * wl.bb, wl.di * wl.dk * wl.bs
    a = (torch.randn(na, generator=(shared if wl.ba == 1 else g), device="cuda") * wl.sa).to(dt)
    b = (torch.randn(nb, generator=g, device="cuda") * wl.sb).to(dt)
    gy = (torch.randn(ny, generator=g, device="cuda") * wl.sgy).to(dt)
    y = torch.empty(ny, device="cuda", dtype=dt)
    ga = torch.zeros(na, device="cuda", dtype=dt)
    gb = torch.zeros(nb, device="cuda", dtype=dt)
    # global batch sizes as the sharded orchestration sees them (1 = replicated operand)
    gba = 1 if wl.ba == 1 else wl.ba * world
    gbb = 1 if wl.bb == 1 else wl.bb * world
    sm = ShardedMatmul(GpuBackend(ctx, mode), world, rank, nccl_all_reduce)

    def step():
        sm.forward(a, b, y, wl.di, wl.dj, wl.dk, gba, gbb)
        sm.backward(a, b, gy, ga, gb, wl.di, wl.dj, wl.dk, gba, gbb)

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
    coll0 = sm.collectives
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
    collectives = sm.collectives - coll0
    sampler.stop_flag = True
    sampler.join(timeout=3)
    assert ctx.status_poll() == 0, "a kernel reported a bounded-wait timeout"

    # ---- end to end through the host-buffer entry points (pinned host memory) ----
    e2e = None
    if not args.skip_e2e:
        e2e = run_e2e(args, wl, ctx, mode, a, b, gy, barrier, torch)
    if dist is not None:
        t = torch.tensor([ms, e2e["ms"] if e2e else 0.0], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
        if e2e:
            e2e["ms"] = float(t[1])
    if rank == 0:
        emit(args, wl, world, ms, prof, launches, sampler, e2e, collectives)
    if dist is not None:
        dist.destroy_process_group()


def run_e2e(args, wl, ctx, mode, a, b, gy, barrier, torch):
    """Each rank pushes its own shard through b200_matmul_{fw,bw}_host (no collective on this leg)."""
    P = lambda t: t.data_ptr()
    e2e_steps = max(1, min(args.steps, 3))
    hb = lambda src: src.cpu().pin_memory()
    ha, hbm, hgy = hb(a), hb(b), hb(gy)
    hy = torch.empty(gy.numel(), dtype=gy.dtype).pin_memory()
    hga = torch.zeros(a.numel(), dtype=a.dtype).pin_memory()
    hgb = torch.zeros(b.numel(), dtype=b.dtype).pin_memory()
    dims = (wl.di, wl.dj, wl.dk, wl.ba, wl.bb)

    def e2e_step():
        ctx.matmul_fw_host(mode, P(ha), P(hbm), P(hy), *dims)
        ctx.matmul_bw_host(mode, P(ha), P(hbm), P(hgy), P(hga), P(hgb), *dims)
        return float(hga[0])  # the step's result is read on the host

    e2e_step()
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(e2e_steps):
        e2e_step()
    f1.record()
    barrier()
    ba, bb_, by = a.numel() * wl.elem, b.numel() * wl.elem, gy.numel() * wl.elem
    return {"ms": f0.elapsed_time(f1), "steps": e2e_steps,
            "h2d": (ba + bb_) + (ba + bb_ + by + ba + bb_),   # fw: a, b;  bw: a, b, gy and the gradients added to
            "d2h": by + ba + bb_}                              # y; ga, gb


def emit(args, wl, world, ms, prof, launches, sampler, e2e, collectives):
    peaks = measured_peaks()
    ms_per_step = ms / args.steps
    value = wl.flops * world / (ms_per_step * 1e-3) / 1e9
    tc_ms, tc_n = prof["gemm_tc"]
    issued_flops_per_launch = float(wl.passes) * wl.flops * args.steps / max(tc_n, 1)
    tc_avg_ms = tc_ms / max(tc_n, 1)
    achieved = issued_flops_per_launch / (tc_avg_ms * 1e-3) / 1e12 if tc_n else 0.0
    div = 1.0 if (wl.half or wl.mode_name == "3xFP16") else 2.0     # TF32 runs at half the 16-bit rate
    peak, burst = peaks["bf16_sustained"] / div, peaks["bf16_burst"] / div
    # DRAM bytes of one gemm_tc_kernel launch: ncu capture of the batch-2 square case (1.48 GB, mean of
    # an overwriting and an accumulating launch, see profiles/), scaled by the batch (independent
    # products, traffic grows in proportion)
    traffic = 1.48e9 * wl.bs / 2.0 if wl.name == "batched_square" else None
    line = {
        "metric": METRIC, "value": value, "unit": "GFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic", "config": wl.config(world),
        "roofline": {
            "bound": "tensor", "kernel": "gemm_tc_kernel (tcgen05, cta pair)", "achieved": achieved,
            "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "traffic": traffic,
            "frac_of_burst_peak": achieved / burst,
            "note": ("achieved = tensor-issued FLOP/s (%d tensor-core pass(es) x algorithmic 2mnk) / mean "
                     "CUDA-event duration of %d launches; peak = %s bf16 sustained%s; the timed region is a "
                     "fraction of a second, so the burst figure %.0f is given beside it%s"
                     % (wl.passes, tc_n, peaks["source"],
                        "" if div == 1.0 else " / 2 (TF32 runs at half the 16-bit rate)", burst,
                        "; traffic = ncu dram bytes of the batch-2 capture scaled to this batch" if traffic else "")),
            "algorithmic_tflops_in_kernel": achieved / wl.passes,
            "kernel_ms_per_step": tc_ms / args.steps, "pack_ms_per_step": prof["pack"][0] / args.steps,
        },
        "gpu_launches": int(launches),
        "collectives_per_step": collectives / max(args.steps, 1),
        "clocks": sampler.summary(),
    }
    if e2e:
        per = e2e["ms"] / e2e["steps"]
        line["e2e"] = {"value": wl.flops * world / (per * 1e-3) / 1e9, "unit": "GFLOP/s",
                       "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"],
                       "steps": e2e["steps"], "ms_per_step": per}
    if world == 1 and not args.skip_cpu:
        t, kind, cores = cpu_sample(wl)
        line["cpu_baseline"] = {"value": wl.sample_flops / t / 1e9, "unit": "GFLOP/s", "cores": cores,
                                "kind": kind, "sample": wl.sample_text()}
        line["cpu_eigen_standin"] = cpu_eigen_standin(wl)
    print(json.dumps(line), flush=True)


GRAPH_PROGRAMS = {
    # workload -> (binary under primitiv_b200/device/_build, arguments before the repeat count, what it is)
    "lstm_steps": ("lstm_steps", ["tf32", "50"],
                   "50 LSTM steps (E 512, H 1024, batch 64) forward + backward through primitiv's Graph, TF32 fast mode"),
    "mlp_step": ("mlp_step", ["3xtf32", "65536"],
                 "one SGD step of 784-1024-1024-10 at batch 65536 through primitiv's Graph, 3xTF32"),
}


def run_graph_program(args):
    """The other named configurations are whole-graph programs on devices::B200 (C++, built where the
    primitiv headers are available).  This leg runs one and reports it in the same line format; the
    step is the program's own (one recurrent loop / one training step), timed by wall clock inside it
    because host work is part of what it measures."""
    import subprocess
    binary, pre, what = GRAPH_PROGRAMS[args.workload]
    path = os.path.join(ROOT, "primitiv_b200", "device", "_build", binary)
    if not os.path.exists(path):
        print(json.dumps({"workload": args.workload, "unavailable": "%s is not built (needs the primitiv headers)" % path}))
        return
    r = subprocess.run([path] + pre + [str(max(args.steps, 1)), "0"], capture_output=True, text=True, timeout=1800)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise SystemExit(r.returncode)
    out = json.loads(r.stdout.strip().splitlines()[-1])
    ms = out.get("ms_per_loop_mean", out.get("ms_per_step_mean"))
    dev = out.get("device_ms_per_loop", out.get("device_ms_per_step"))
    launches = out.get("launches_per_loop", out.get("launches_per_step"))
    passes = 3.0 if pre[0] == "3xtf32" else 1.0
    flops = out["matmul_gflops"] * 1e9 * ms * 1e-3   # algorithmic matmul FLOP of one step
    peaks = measured_peaks()
    peak = peaks["bf16_sustained"] / 2.0
    achieved = passes * flops / (dev["gemm_tc"] * 1e-3) / 1e12 if dev["gemm_tc"] else 0.0
    line = {
        "metric": METRIC, "value": out["matmul_gflops"], "unit": "GFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": 2, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "tf32x3" if passes == 3.0 else "tf32", "data": "synthetic",
        "config": {"workload": args.workload, "what": what, "timing": "wall clock inside the program, host work included"},
        "roofline": {"bound": "tensor", "kernel": "gemm_tc_kernel", "achieved": achieved, "peak": peak,
                     "unit": "TFLOP/s", "frac": achieved / peak, "traffic": None,
                     "note": "the step is launch-bound: tensor-issued FLOP / device time of the product launches only "
                             "(per-launch CUDA events of one extra, untimed step)",
                     "device_ms_per_step": dev, "launches_per_step": launches},
        "gpu_launches": int(sum(launches.values()) * args.steps),
        "e2e": {"value": out["matmul_gflops"], "unit": "GFLOP/s", "h2d_bytes_per_step": None, "d2h_bytes_per_step": None,
                "note": "value is already end to end: inputs start in host vectors"},
        "program_output": out,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="batched_square", choices=["batched_square", "batched_square_tf32", "batched_square_3xfp16", "fp16_broadcast", "lstm_steps",
                             "mlp_step"])
    ap.add_argument("--batch", type=int, default=0,
                    help="batch elements per GPU (default: the workload's own, 8 / 32; smaller values are for "
                         "profiler captures and show in config.workload)")
    ap.add_argument("--skip-e2e", action="store_true", help="leave out the host-buffer leg (profiler captures)")
    ap.add_argument("--skip-cpu", action="store_true", help="leave out the CPU baseline leg (profiler captures)")
    args = ap.parse_args()
    if args.workload in GRAPH_PROGRAMS:
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "workload": args.workload,
                              "unavailable": "the program times the reference's Naive device itself "
                                             "(naive_ms_per_step, on a prefix) when given a check size"}))
        elif int(os.environ.get("RANK", "0")) == 0:
            run_graph_program(args)
        return
    wl = Workload(args.workload, args.batch)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, wl, rank)
    else:
        run_ours(args, wl, rank, local_rank, world)


if __name__ == "__main__":
    main()
