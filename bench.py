#!/usr/bin/env python3
"""Benchmark of the matmul_fw + matmul_bw hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Default workload (one "step" = one forward plus both backward products over the batch):
non-broadcast batched square GEMM, fp32 in 3xTF32 mode: A and B each
Shape({4096,4096}, batch 8) ~ N(0, 0.02), upstream gradient N(0,1), seeded synthetic
data.  With N GPUs every rank holds a full batch-8 shard of its own (weak scaling; the
products of different batch elements are independent, so the data path has no collective).

Prints ONE JSON line on rank 0.  `value` is algorithmic GFLOP/s (2*m*n*k per product, three
products per step) over all ranks with operands resident in HBM; `e2e` is the same metric
through the fused host-buffer entry point of the C ABI (b200_matmul_fw_bw_host) with the
host<->device copies inside the timed region.

Beside the headline the same line carries, at every N:
  collective_check   untimed parity of the path's one exchange step: the plumbing workload
                     (W {256,256} broadcast, X {256,64} x 16, gradients pre-filled 0.5) cut over the
                     N ranks; y and gX gathered, gW all-reduced over NCCL, all compared with an fp64
                     product computed on the host, and gW compared bit for bit between the ranks;
  secondary          two timed legs whose backward has that exchange step: `fp16_broadcast`
                     (A {8192,8192} replicated, B {8192,2048} x 32 per GPU, half storage; the
                     128 MiB gA partial is all-reduced) and `mlp_products` (the nine products of a
                     784-1024-1024-10 perceptron step over 65536 items per GPU, 3xTF32; three
                     weight-gradient all-reduces);
  tf32_cublas_measured / l2_ingest_measured / gpu_comparator   context figures (rank 0): the TF32 rate
                     of the vendor GEMM on this GPU, the rate at which an SM takes operand tiles in
                     from L2 (the second ceiling of the tensor-core kernels), and the reference's own
                     CUDA / CUDA16 devices on the same
                     workloads when they have been built (own process, never linked here);
  graph_programs     (1 GPU) the recurrent step loop and one perceptron training step as whole
                     programs through primitiv's Graph on devices::B200, each beside the same model
                     code on the reference's devices::CUDA.

`--workload batched_square_3xfp16 | batched_square_tf32 | fp16_broadcast` make another workload the
headline; `--workload lstm_steps | mlp_step` run the graph-level programs of the other named
configurations (1 GPU).

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
# dram__bytes_read.sum + dram__bytes_write.sum of one gemm_tc_kernel launch on the batch-2 square case
# (profiles/gemm_tc_kernel_fp32_mix_batch2_ncu_full.md): 1.38 GB overwriting, 1.51 GB accumulating
NCU_DRAM_BYTES_PER_LAUNCH_BATCH2 = 1.47e9
# plane memory the library may keep between the forward and the backward call of a step
PLANE_CACHE_BYTES = 8 << 30


class Workload:
    """Shapes in primitiv terms: a {di,dj} x ba, b {dj,dk} x bb; per-GPU batch sizes."""

    def __init__(self, name, batch):
        self.name = name
        if name == "batched_square":
            self.di = self.dj = self.dk = 4096
            self.ba = self.bb = batch if batch else 8
            self.mode_name, self.passes, self.half = "3xTF32", 3, False
            self.sa, self.sb, self.sgy = 0.02, 0.02, 1.0
            self.dtype = "f32 via tf32 + 2 x bf16 correction passes (fp32 storage, fp32 accumulate)"
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
                "parallelism": "batch-sharded x%d" % n_gpus, "collective": collective,
                "operand_planes": "fp32 mode: the planes the forward call packs from a and b are reused by the backward "
                                  "call of the same step and dropped at the start of the next"}


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


class Rig:
    """What every leg needs: the context, the process group and the timing rules (barrier +
    synchronize on both sides, CUDA events on the launching stream, max over ranks)."""

    def __init__(self, rank, local_rank, world):
        import torch
        import primitiv_b200 as pb
        self.torch, self.pb = torch, pb
        self.rank, self.local_rank, self.world = rank, local_rank, world
        torch.cuda.set_device(local_rank)
        self.dist = None
        if world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
            self.dist = dist
        self.ctx = pb.Context(local_rank)

    def mode(self, name):
        pb = self.pb
        return {"FP16": pb.MODE_FP16, "TF32": pb.MODE_TF32, "3xFP16": pb.MODE_FP32_3XFP16}.get(name, pb.MODE_FP32_3XTF32)

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, values):
        if self.dist is None:
            return [float(v) for v in values]
        t = self.torch.tensor(values, device="cuda", dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t]

    def sharded(self, mode):
        from primitiv_b200.sharding import GpuBackend, ShardedMatmul, nccl_all_reduce
        return ShardedMatmul(GpuBackend(self.ctx, mode), self.world, self.rank, nccl_all_reduce)

    def timed(self, step, steps, warmup, sm):
        """W warm-up steps, then exactly K timed steps.  -> dict(ms, prof, launches, collectives, clocks)"""
        torch, ctx = self.torch, self.ctx
        for _ in range(warmup):
            step()
        self.barrier()
        sampler = ClockSampler(self.local_rank)
        sampler.start()
        ctx.profile_read()
        ctx.profile_enable(True)
        launches0, coll0 = ctx.launch_count(), sm.collectives
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        self.barrier()
        ms = e0.elapsed_time(e1)
        ctx.profile_enable(False)
        prof = ctx.profile_read()
        sampler.stop_flag = True
        sampler.join(timeout=3)
        assert ctx.status_poll() == 0, "a kernel reported a bounded-wait timeout"
        return {"ms": self.max_over_ranks([ms])[0], "prof": prof, "launches": ctx.launch_count() - launches0,
                "collectives": sm.collectives - coll0, "clocks": sampler.summary()}


def workload_tensors(rig, wl):
    """This rank's shard of the workload: seeded synthetic tensors, a replicated operand the same on every rank."""
    torch = rig.torch
    dt = torch.float16 if wl.half else torch.float32
    g = torch.Generator(device="cuda")
    g.manual_seed(1234 + rig.rank)
    shared = torch.Generator(device="cuda")
    shared.manual_seed(99)
    na, nb, ny = wl.di * wl.dj * wl.ba, wl.dj * wl.dk * wl.bb, wl.di * wl.dk * wl.bs
    a = (torch.randn(na, generator=(shared if wl.ba == 1 else g), device="cuda") * wl.sa).to(dt)
    b = (torch.randn(nb, generator=g, device="cuda") * wl.sb).to(dt)
    gy = (torch.randn(ny, generator=g, device="cuda") * wl.sgy).to(dt)
    y = torch.empty(ny, device="cuda", dtype=dt)
    ga = torch.zeros(na, device="cuda", dtype=dt)
    gb = torch.zeros(nb, device="cuda", dtype=dt)
    return a, b, gy, y, ga, gb


def run_workload(rig, wl, steps, warmup):
    """Device-resident leg of one Workload.  -> (result of Rig.timed, the operand tensors)"""
    a, b, gy, y, ga, gb = workload_tensors(rig, wl)
    # global batch sizes as the sharded orchestration sees them (1 = replicated operand)
    gba = 1 if wl.ba == 1 else wl.ba * rig.world
    gbb = 1 if wl.bb == 1 else wl.bb * rig.world
    sm = rig.sharded(rig.mode(wl.mode_name))
    rig.ctx.operand_cache_enable(PLANE_CACHE_BYTES)

    def step():
        # a step starts from operands the library has not seen (in training the weights have just been
        # updated and the minibatch is new): planes kept from the previous step are dropped.  Within
        # the step the backward call reuses the planes the forward call packed from the same a and b.
        rig.ctx.operand_cache_invalidate()
        sm.forward(a, b, y, wl.di, wl.dj, wl.dk, gba, gbb)
        sm.backward(a, b, gy, ga, gb, wl.di, wl.dj, wl.dk, gba, gbb)

    try:
        return rig.timed(step, steps, warmup, sm), (a, b, gy)
    finally:
        rig.ctx.operand_cache_enable(0)


def peak_divisor(mode_name, half):
    """Measured bf16 peak / this = the peak of the passes a mode issues.  Single-pass fp16 and 3xFP16
    run on the 16-bit pipe (1).  TF32 runs at half that rate (2).  The fp32 mode issues one TF32 pass
    and two bf16 correction passes of the same FLOP count: the least time for its 3F issued FLOP is
    F / (P/2) + 2F / P = 4F / P, so the peak of the mix is 3P/4 (divisor 4/3)."""
    if half or mode_name == "3xFP16":
        return 1.0
    return 4.0 / 3.0 if mode_name == "3xTF32" else 2.0


def tensor_roofline(wl, res, steps, peaks):
    tc_ms, tc_n = res["prof"]["gemm_tc"]
    issued_flops_per_launch = float(wl.passes) * wl.flops * steps / max(tc_n, 1)
    tc_avg_ms = tc_ms / max(tc_n, 1)
    achieved = issued_flops_per_launch / (tc_avg_ms * 1e-3) / 1e12 if tc_n else 0.0
    div = peak_divisor(wl.mode_name, wl.half)
    sustained, burst = peaks["bf16_sustained"] / div, peaks["bf16_burst"] / div
    return achieved, sustained, burst, tc_ms, tc_n, div


def collective_check(rig):
    """Untimed parity of the exchange step on the plumbing workload: W {256,256} broadcast, X {256,64} x 16
    U(-1,1), gy N(0,1), gradients pre-filled 0.5, the batch cut over the ranks.  The fp64 products are
    computed here with numpy (the check must not depend on where the test oracle is built)."""
    import numpy as np
    from primitiv_b200.sharding import shard_range
    torch, dist, world, rank = rig.torch, rig.dist, rig.world, rig.rank
    di, dj, dk, bb = 256, 256, 64, 16
    rng = np.random.default_rng(0)
    w = rng.uniform(-1, 1, di * dj).astype(np.float32)
    x = rng.uniform(-1, 1, dj * dk * bb).astype(np.float32)
    gy = rng.standard_normal(di * dk * bb).astype(np.float32)
    first, count = shard_range(bb, rank, world)
    cu = lambda v: torch.from_numpy(np.ascontiguousarray(v)).cuda()
    lw, lx, lgy = cu(w), cu(x[first * dj * dk:(first + count) * dj * dk]), cu(gy[first * di * dk:(first + count) * di * dk])
    y = torch.empty(di * dk * count, device="cuda")
    gw = torch.full((di * dj,), 0.5, device="cuda")
    gx = torch.full((dj * dk * count,), 0.5, device="cuda")
    sm = rig.sharded(rig.pb.MODE_FP32_3XTF32)
    rig.ctx.set_path_policy(2)            # the tensor-core kernel, although the problem is small
    try:
        sm.forward(lw, lx, y, di, dj, dk, 1, bb)
        sm.backward(lw, lx, lgy, gw, gx, di, dj, dk, 1, bb)
    finally:
        rig.ctx.set_path_policy(0)
    torch.cuda.synchronize()
    assert rig.ctx.status_poll() == 0

    def gather(t):
        if dist is None:
            return [t]
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t)
        return parts

    ys, gxs, gws = gather(y), gather(gx), gather(gw)
    if rank != 0:
        return None
    W = w.astype(np.float64).reshape(dj, di).T                      # column-major {di, dj}
    X = x.astype(np.float64).reshape(bb * dk, dj).T                 # {dj, dk*bb}: the batches are adjacent columns
    G = gy.astype(np.float64).reshape(bb * dk, di).T                # {di, dk*bb}
    flat = lambda m: np.ascontiguousarray(m.T).reshape(-1)
    rel = lambda got, ref: float(np.linalg.norm(got.astype(np.float64) - ref) / np.linalg.norm(ref))
    errs = {"y": rel(torch.cat(ys).cpu().numpy(), flat(W @ X)),
            "gW": rel(gws[0].cpu().numpy(), flat(0.5 + G @ X.T)),
            "gX": rel(torch.cat(gxs).cpu().numpy(), flat(0.5 + W.T @ G))}
    return {"workload": "W{256,256} broadcast . X{256,64} x 16, gradients pre-filled 0.5, 3xTF32, batch cut over the ranks",
            "nranks": world, "rel_err": max(errs.values()), "rel_err_by_tensor": errs, "tolerance": 1e-5,
            "collectives": sm.collectives,
            "replicas_bit_identical": all(bool(torch.equal(gws[0], g)) for g in gws[1:])}


def leg_fp16_broadcast(rig, steps, warmup, peaks):
    """Secondary leg: the half-precision workload with a replicated A (its gradient partial is all-reduced)."""
    wl = Workload("fp16_broadcast", 0)
    res, _ = run_workload(rig, wl, steps, warmup)
    rig.torch.cuda.empty_cache()
    ms = res["ms"] / steps
    achieved, sustained, burst, tc_ms, tc_n, _ = tensor_roofline(wl, res, steps, peaks)
    return {"workload": wl.label(), "value": wl.flops * rig.world / (ms * 1e-3) / 1e9, "unit": "GFLOP/s",
            "ms_per_step": ms, "steps": steps, "warmup": warmup, "dtype": wl.dtype, "mode": wl.mode_name,
            "batch_per_gpu": wl.bs, "scaling": "weak",
            "collectives_per_step": res["collectives"] / steps,
            "collective": "all-reduce (sum) of the 128 MiB gA partial over NCCL, started before and waited for "
                          "after the local gB product" if rig.world > 1 else "none at 1 GPU",
            "roofline": {"bound": "tensor", "kernel": "gemm_tc_kernel (kind::f16, cta pair)", "achieved": achieved,
                         "peak": burst, "unit": "TFLOP/s", "frac": achieved / burst,
                         "frac_of_sustained_peak": achieved / sustained, "traffic": None,
                         "note": "tensor-issued = algorithmic FLOP / mean CUDA-event duration of %d launches; peak = %s "
                                 "bf16 burst (the leg lasts a fraction of a second)" % (tc_n, peaks["source"]),
                         "kernel_ms_per_step": tc_ms / steps},
            "gpu_launches": int(res["launches"]), "clocks": res["clocks"]}


MLP_LAYERS = ((1024, 784), (1024, 1024), (10, 1024))     # (rows, cols) of W1, W2, W3
MLP_BATCH = 65536


def leg_mlp_products(rig, steps, warmup, peaks):
    """Secondary leg: the nine products of one 784-1024-1024-10 perceptron step (three forward, three
    weight gradients summed over the batch and all-reduced, three input gradients), 65536 items per
    GPU, fp32 via 3xTF32.  Weights Xavier-uniform and replicated, inputs U(0,1), upstream N(0,1)."""
    torch = rig.torch
    g = torch.Generator(device="cuda")
    g.manual_seed(4321 + rig.rank)
    shared = torch.Generator(device="cuda")
    shared.manual_seed(77)
    B = MLP_BATCH
    ws, gws, acts, gacts = [], [], [], []
    acts.append(torch.rand(MLP_LAYERS[0][1] * B, generator=g, device="cuda"))
    for rows, cols in MLP_LAYERS:
        lim = (6.0 / (rows + cols)) ** 0.5
        ws.append((torch.rand(rows * cols, generator=shared, device="cuda") * 2 - 1) * lim)
        gws.append(torch.zeros(rows * cols, device="cuda"))
        acts.append(torch.empty(rows * B, device="cuda"))
    gacts = [torch.zeros(a.numel(), device="cuda") for a in acts]
    gacts[-1] = torch.randn(MLP_LAYERS[-1][0] * B, generator=g, device="cuda")
    sm = rig.sharded(rig.pb.MODE_FP32_3XTF32)
    gb = B * rig.world

    def step():
        rig.ctx.operand_cache_invalidate()      # as in run_workload: nothing is carried from step to step
        for l, (rows, cols) in enumerate(MLP_LAYERS):
            sm.forward(ws[l], acts[l], acts[l + 1], rows, cols, 1, 1, gb)
        for l in range(len(MLP_LAYERS) - 1, -1, -1):
            rows, cols = MLP_LAYERS[l]
            sm.backward(ws[l], acts[l], gacts[l + 1], gws[l], gacts[l], rows, cols, 1, 1, gb)

    rig.ctx.operand_cache_enable(PLANE_CACHE_BYTES)
    try:
        res = rig.timed(step, steps, warmup, sm)
    finally:
        rig.ctx.operand_cache_enable(0)
    same = True
    if rig.dist is not None:      # replicas of a weight gradient hold the same bits on every rank
        parts = [torch.empty_like(gws[0]) for _ in range(rig.world)]
        rig.dist.all_gather(parts, gws[0])
        same = all(bool(torch.equal(parts[0], p)) for p in parts[1:])
    del ws, gws, acts, gacts
    torch.cuda.empty_cache()
    flops = 3 * sum(2 * r * c * B for r, c in MLP_LAYERS)
    tc_flops = 3 * sum(2 * r * c * B for r, c in MLP_LAYERS[:2])       # the 10-row layer runs on CUDA cores
    ms = res["ms"] / steps
    tc_ms, tc_n = res["prof"]["gemm_tc"]
    achieved = 3.0 * tc_flops * steps / (tc_ms * 1e-3) / 1e12 if tc_ms else 0.0
    burst = peaks["bf16_burst"] / peak_divisor("3xTF32", False)
    kinds = {k: {"ms_per_step": v[0] / steps, "launches_per_step": v[1] / steps} for k, v in res["prof"].items()}
    return {"workload": "mlp_784_1024_1024_10_batch%d_per_gpu_nine_products_fp32_3xtf32" % B, "value": flops * rig.world / (ms * 1e-3) / 1e9,
            "unit": "GFLOP/s", "ms_per_step": ms, "steps": steps, "warmup": warmup, "mode": "3xTF32",
            "dtype": "f32 via tf32 + 2 x bf16 correction passes (fp32 storage, fp32 accumulate)", "batch_per_gpu": B, "scaling": "weak",
            "collectives_per_step": res["collectives"] / steps,
            "collective": "all-reduce (sum) of gW1, gW2, gW3 partials (3.2 MB, 4.2 MB, 41 kB) over NCCL" if rig.world > 1 else "none at 1 GPU",
            "replicas_bit_identical": same,
            "roofline": {"bound": "tensor", "kernel": "gemm_tc_kernel (3xTF32) over the two 1024-row layers", "achieved": achieved,
                         "peak": burst, "unit": "TFLOP/s", "frac": achieved / burst, "traffic": None,
                         "note": "tensor-issued FLOP (3 passes) of the six tensor-core products / their summed CUDA-event "
                                 "time; the 10-row layer's three products are HBM-bound CUDA-core kernels (gemm_simt row)",
                         "device_ms_by_kernel_kind": kinds},
            "gpu_launches": int(res["launches"]), "clocks": res["clocks"]}


def tf32_cublas_measured(rig):
    """TF32 rate of the vendor GEMM on this GPU, measured the way MEASURED_PEAKS.json measures bf16
    (torch.matmul 8192^3, best of 10 = burst; back to back for a second = sustained).  A measurement
    aid beside the roofline, never on the product path."""
    torch = rig.torch
    n = 8192
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        a = torch.randn(n, n, device="cuda")
        b = torch.randn(n, n, device="cuda")
        c = torch.empty(n, n, device="cuda")
        for _ in range(3):
            torch.matmul(a, b, out=c)
        best = 1e9
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch.matmul(a, b, out=c)
            e1.record()
            e1.synchronize()
            best = min(best, e0.elapsed_time(e1))
        reps = max(10, int(1000.0 / best))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            torch.matmul(a, b, out=c)
        e1.record()
        e1.synchronize()
        sustained_ms = e0.elapsed_time(e1) / reps
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    del a, b, c
    torch.cuda.empty_cache()
    fl = 2.0 * n ** 3
    return {"burst_tflops": fl / (best * 1e-3) / 1e12, "sustained_tflops": fl / (sustained_ms * 1e-3) / 1e12,
            "how": "torch.matmul fp32 with TF32 allowed, 8192^3: best of 10 (burst), %d back to back (sustained)" % reps}


def gpu_comparator(wl_names):
    """The reference's own GPU devices (devices::CUDA: cublasSgemm / SgemmBatched, primitiv/devices/cuda/ops/
    matmul.cu:26-138; devices::CUDA16: cublasHgemm, cuda16/ops/matmul.cu:46-266) on the same workloads, timed
    with CUDA events in a process of their own.  Built by `make -C oracle ref_cuda` where the reference tree
    is mounted; the binary travels under baseline/_ref/ and is never linked into this library."""
    exe = os.path.join(ROOT, "baseline", "_ref", "cuda", "ref_cuda_matmul")
    if not os.path.exists(exe):
        return {"unavailable": "baseline/_ref/cuda/ref_cuda_matmul is not built (make -C oracle ref_cuda, needs the reference tree)"}
    out = {}
    for name in wl_names:
        try:
            r = subprocess.run([exe, name, "5", "2"], capture_output=True, text=True, timeout=600)
            if r.returncode != 0:
                out[name] = {"unavailable": "exit %d: %s" % (r.returncode, (r.stderr or r.stdout).strip()[-300:])}
            else:
                out[name] = json.loads(r.stdout.strip().splitlines()[-1])
        except Exception as e:      # noqa: BLE001 -- a comparator that cannot run is reported, not fatal
            out[name] = {"unavailable": repr(e)[:300]}
    return out


def graph_legs():
    """The two graph-level configurations (the recurrent step loop, one perceptron training step) as whole
    programs through primitiv's Graph: on devices::B200 (tests/cpp/_build, with a parity check against the
    reference's Naive device on a short prefix / small batch inside the program) and, beside each, the same
    model code on the reference's devices::CUDA (baseline/_ref/cuda/ref_cuda_graphs).  Wall clock inside the
    programs, host work included; each runs in a process of its own on GPU 0."""
    def run(cmd):
        if not os.path.exists(cmd[0]):
            return {"unavailable": "%s is not built (needs the reference tree at build time)" % os.path.relpath(cmd[0], ROOT)}
        try:
            r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
            if r.returncode != 0:
                return {"unavailable": "exit %d: %s" % (r.returncode, (r.stderr or r.stdout).strip()[-300:])}
            return json.loads(r.stdout.strip().splitlines()[-1])
        except Exception as e:      # noqa: BLE001 -- a leg that cannot run is reported, not fatal
            return {"unavailable": repr(e)[:300]}

    ours = os.path.join(ROOT, "tests", "cpp", "_build")
    ref = os.path.join(ROOT, "baseline", "_ref", "cuda", "ref_cuda_graphs")
    out = {}
    # devices::CUDA puts the batch index of its broadcasting elementwise kernels in gridDim.y
    # (primitiv/devices/cuda/ops/common.h:118-151), which ends at 65535: at the configuration's 65536 items
    # the bias additions are never launched and nothing reports it (the loss then differs in the second
    # digit).  The perceptron step is therefore compared at 32768 items as well, where the reference runs.
    for name, mine, theirs, key in (
            ("lstm_steps", ["tf32", "50", "5", "2"], ["lstm_steps", "50", "5"], "ms_per_loop_mean"),
            ("mlp_step", ["3xtf32", "65536", "3", "256"], ["mlp_step", "65536", "3"], "ms_per_step_mean"),
            ("mlp_step_batch32768", ["3xtf32", "32768", "3", "0"], ["mlp_step", "32768", "3"], "ms_per_step_mean")):
        program = name.split("_batch")[0]
        b200 = run([os.path.join(ours, program)] + mine)
        time.sleep(1.0)
        cuda = run([ref] + theirs)
        time.sleep(1.0)
        leg = {"what": GRAPH_PROGRAMS[program][2] if name == program else "the same step at 32768 items",
               "b200": b200, "reference_cuda": cuda}
        if key in b200 and key in cuda:
            leg["ms"] = {"b200": b200[key], "reference_cuda": cuda[key]}
            leg["speedup_vs_reference_cuda"] = cuda[key] / b200[key]
            if "ms_of_best" in b200 and "ms_of_best" in cuda:    # the part of the step that is device work
                leg["backward_update_ms"] = {"b200": b200["ms_of_best"]["backward_update"],
                                             "reference_cuda": cuda["ms_of_best"]["backward_update"]}
            if b200.get("loss") and cuda.get("loss"):
                diff = abs(b200["loss"] - cuda["loss"]) / abs(cuda["loss"])
                leg["loss_rel_diff_vs_reference_cuda"] = diff
                if diff > 1e-2:
                    leg["note"] = ("the reference device did not compute this configuration: its elementwise kernels "
                                   "index the batch with gridDim.y, which ends at 65535")
        out[name] = leg
    return out


def run_ours(args, wl, rank, local_rank, world):
    rig = Rig(rank, local_rank, world)
    peaks = measured_peaks()
    check = collective_check(rig)
    res, (a, b, gy) = run_workload(rig, wl, args.steps, args.warmup)

    # ---- end to end through the host-buffer entry point (pinned host memory) ----
    e2e = None
    if not args.skip_e2e:
        e2e = run_e2e(args, wl, rig, a, b, gy)
        e2e["ms"] = rig.max_over_ranks([e2e["ms"]])[0]
    del a, b, gy
    rig.torch.cuda.empty_cache()
    rig.ctx.pool_release_cached()

    secondary = {}
    if not args.skip_secondary:
        # a second of idling before each leg: every leg starts from the same power and clock state
        # instead of inheriting the cap the previous one ran into
        if wl.name != "fp16_broadcast":
            time.sleep(1.0)
            secondary["fp16_broadcast"] = leg_fp16_broadcast(rig, args.secondary_steps, 3, peaks)
            rig.ctx.pool_release_cached()
        time.sleep(1.0)
        secondary["mlp_products"] = leg_mlp_products(rig, args.secondary_steps, 3, peaks)
        rig.ctx.pool_release_cached()
    extras = {}
    if rank == 0 and not args.skip_cpu:
        extras["tf32_cublas_measured"] = tf32_cublas_measured(rig)
        per_clk, gbs = rig.ctx.measure_l2_ingest()
        extras["l2_ingest_measured"] = {
            "bytes_per_clk_per_sm": per_clk, "gb_per_s_per_sm": gbs,
            "needed_at_full_tensor_rate": 64.0,
            "note": "bulk copies L2 -> shared memory and nothing else, 128 KB in flight per SM, everything an L2 hit "
                    "(b200_measure_l2_ingest); the 256 x 256 pair tiles of the fp32, TF32 and half-precision kinds need "
                    "64 B per SM clock at full tensor rate and see a quarter of their sectors at HBM latency"}
    rig.barrier()
    if rank == 0 and world == 1 and not args.skip_cpu:
        extras["gpu_comparator"] = gpu_comparator(["batched_square", "fp16_broadcast"])
        if not args.skip_secondary:
            extras["graph_programs"] = graph_legs()
    if rank == 0:
        emit(args, wl, world, res, e2e, peaks, check, secondary, extras)
    if rig.dist is not None:
        rig.barrier()
        rig.dist.destroy_process_group()


def run_e2e(args, wl, rig, a, b, gy):
    """Each rank pushes its own shard through b200_matmul_fw_bw_host (no collective on this leg): a, b and
    gy go up once, y, ga and gb come down; the gradients start from zeros (the workload's definition), so
    the entry point is told so and does not upload them."""
    torch, ctx = rig.torch, rig.ctx
    mode = rig.mode(wl.mode_name)
    P = lambda t: t.data_ptr()
    e2e_steps = max(1, min(args.steps, 5))
    hb = lambda src: src.cpu().pin_memory()
    ha, hbm, hgy = hb(a), hb(b), hb(gy)
    hy = torch.empty(gy.numel(), dtype=gy.dtype).pin_memory()
    hga = torch.empty(a.numel(), dtype=a.dtype).pin_memory()
    hgb = torch.empty(b.numel(), dtype=b.dtype).pin_memory()
    dims = (wl.di, wl.dj, wl.dk, wl.ba, wl.bb)

    def e2e_step():
        ctx.matmul_fw_bw_host(mode, P(ha), P(hbm), P(hgy), P(hy), P(hga), P(hgb), *dims,
                              accumulate_a=False, accumulate_b=False)
        return float(hga[0]) + float(hy[0])  # the step's results are read on the host

    for _ in range(2):
        e2e_step()
    rig.barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(e2e_steps):
        e2e_step()
    f1.record()
    rig.barrier()
    ba, bb_, by = a.numel() * wl.elem, b.numel() * wl.elem, gy.numel() * wl.elem
    return {"ms": f0.elapsed_time(f1), "steps": e2e_steps,
            "h2d": ba + bb_ + by,       # a, b, gy: once each
            "d2h": by + ba + bb_}       # y; ga, gb


def emit(args, wl, world, res, e2e, peaks, check, secondary, extras):
    ms_per_step = res["ms"] / args.steps
    value = wl.flops * world / (ms_per_step * 1e-3) / 1e9
    achieved, sustained, burst, tc_ms, tc_n, div = tensor_roofline(wl, res, args.steps, peaks)
    # DRAM bytes of one gemm_tc_kernel launch: ncu capture of the batch-2 square case (see profiles/),
    # mean of an overwriting and an accumulating launch, scaled by the batch (independent products:
    # traffic grows in proportion)
    traffic = NCU_DRAM_BYTES_PER_LAUNCH_BATCH2 * wl.bs / 2.0 if wl.name == "batched_square" else None
    line = {
        "metric": METRIC, "value": value, "unit": "GFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic", "config": wl.config(world),
        "roofline": {
            "bound": "tensor", "kernel": "gemm_tc_kernel (tcgen05, cta pair)", "achieved": achieved,
            "peak": burst, "unit": "TFLOP/s", "frac": achieved / burst, "traffic": traffic,
            "frac_of_sustained_peak": achieved / sustained,
            "note": ("achieved = tensor-issued FLOP/s (%d tensor-core pass(es) x algorithmic 2mnk) / mean "
                     "CUDA-event duration of %d launches; peak = %s bf16 burst%s (the timed region is a "
                     "fraction of a second); the sustained figure is %.0f%s"
                     % (wl.passes, tc_n, peaks["source"],
                        "" if div == 1.0 else (" / 2 (TF32 runs at half the 16-bit rate)" if div == 2.0 else
                                               " x 3/4 (one TF32 pass at half the 16-bit rate plus two bf16 passes at the full rate)"),
                        sustained,
                        "; traffic = ncu dram bytes of the batch-2 capture scaled to this batch" if traffic else "")),
            "algorithmic_tflops_in_kernel": achieved / wl.passes,
            "kernel_ms_per_step": tc_ms / args.steps, "pack_ms_per_step": res["prof"]["pack"][0] / args.steps,
        },
        "gpu_launches": int(res["launches"]),
        "collectives_per_step": res["collectives"] / max(args.steps, 1),
        "clocks": res["clocks"],
    }
    if e2e:
        per = e2e["ms"] / e2e["steps"]
        line["e2e"] = {"value": wl.flops * world / (per * 1e-3) / 1e9, "unit": "GFLOP/s",
                       "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"],
                       "steps": e2e["steps"], "ms_per_step": per,
                       "entry_point": "b200_matmul_fw_bw_host (pinned host buffers; a, b, gy up once, y, ga, gb down)"}
    if check is not None:
        line["collective_check"] = check
    if secondary:
        line["secondary"] = secondary
    line.update(extras)
    if "tf32_cublas_measured" in extras and div == 2.0:
        line["roofline"]["frac_of_cublas_tf32_burst"] = achieved / extras["tf32_cublas_measured"]["burst_tflops"]
    if "tf32_cublas_measured" in extras and wl.mode_name != "FP16":
        # what one pass of the vendor's TF32 GEMM would deliver on these shapes, at a thousandth of the accuracy
        line["roofline"]["algorithmic_vs_cublas_tf32_single_pass"] = (achieved / wl.passes) / extras["tf32_cublas_measured"]["burst_tflops"]
    if world == 1 and not args.skip_cpu:
        t, kind, cores = cpu_sample(wl)
        line["cpu_baseline"] = {"value": wl.sample_flops / t / 1e9, "unit": "GFLOP/s", "cores": cores,
                                "kind": kind, "sample": wl.sample_text()}
        line["cpu_eigen_standin"] = cpu_eigen_standin(wl)
    print(json.dumps(line), flush=True)


GRAPH_PROGRAMS = {
    # workload -> (binary under tests/cpp/_build, arguments before the repeat count, what it is)
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
    path = os.path.join(ROOT, "tests", "cpp", "_build", binary)
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
    peak = peaks["bf16_sustained"] / peak_divisor("3xTF32" if passes == 3.0 else "TF32", False)
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
    ap.add_argument("--skip-secondary", action="store_true", help="leave out the secondary legs (profiler captures)")
    ap.add_argument("--secondary-steps", type=int, default=8, help="timed steps of each secondary leg")
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
