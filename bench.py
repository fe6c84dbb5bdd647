"""Benchmark of the W8A8 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Prints ONE JSON line (rank 0).  Workloads:
  gemm     the headline W8A8 GEMM, 4096 x 12288 x 12288, int8 output
           (linear_a8_w8_b8_o8); N GPUs run N independent replicas.
  opt30b   Int8OPTForCausalLM at the OPT-30B architecture, batch 8, 512-token
           prefill, one GPU.
  opt175b  the OPT-175B architecture, batch 16, 1024-token prefill, tensor
           parallel over N = 2/4/8 GPUs with two int32 all-reduces per layer.
The default is opt30b at N=1 and opt175b at N>1 once the model path is
available in this checkout, else gemm.

`--impl reference` times the reference semantics on the host CPU (the oracle's
C restatement, all host threads) on a bounded sample of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "torch-int_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

HG = (4096, 12288, 12288)  # M, N, K of the headline GEMM


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.thread.join(timeout=2)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def dist_env():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return world, rank, local


# ----------------------------------------------------------------------------- GEMM workload
class GemmWorkload:
    name = "w8a8_gemm_4096x12288x12288_int8out"
    metric = "w8a8_gemm_tops"
    unit = "TOP/s"
    dtype = "int8 x int8 -> int32, fp32 epilogue, int8 out"
    scaling = "weak"

    def __init__(self, device):
        from torch_int import _CUDA as C
        self.C = C
        m, n, k = HG
        g = torch.Generator().manual_seed(0)
        self.x_host = torch.randint(-127, 128, (m, k), generator=g, dtype=torch.int8).pin_memory()
        self.y_host = torch.empty((m, n), dtype=torch.int8).pin_memory()
        gd = torch.Generator(device=device).manual_seed(1)
        self.x = self.x_host.to(device)
        self.w = torch.randint(-127, 128, (n, k), generator=gd, dtype=torch.int8, device=device)
        self.b = torch.randint(-127, 128, (n,), generator=gd, dtype=torch.int8, device=device)
        self.alpha, self.beta = 1e-4, 0.01
        self.ops_per_step = 2.0 * m * n * k
        self.h2d = self.x_host.numel()
        self.d2h = self.y_host.numel()
        self.launches_per_step = 1

    def step(self):
        return self.C.linear_a8_w8_b8_o8(self.x, self.w, self.b, self.alpha, self.beta)

    def step_e2e(self):
        x = self.x_host.to(self.x.device, non_blocking=True)
        y = self.C.linear_a8_w8_b8_o8(x, self.w, self.b, self.alpha, self.beta)
        self.y_host.copy_(y, non_blocking=True)

    def units(self, n_gpus):
        return self.ops_per_step * n_gpus / 1e12  # tera-ops per step over all replicas

    def config(self, n_gpus):
        return {"workload": self.name, "M": HG[0], "N": HG[1], "K": HG[2], "alpha": self.alpha,
                "beta": self.beta, "replicas": n_gpus,
                "l2": "inputs (201 MB of int8 operands) exceed the 126 MB L2"}

    def roofline(self, ms, peaks):
        peak = 2.0 * peaks["bf16_tflops"]
        achieved = self.ops_per_step / (ms * 1e-3) / 1e12
        return {"bound": "tensor", "achieved": round(achieved, 1), "peak": round(peak, 1), "unit": "TOP/s",
                "frac": round(achieved / peak, 4), "traffic": None,
                "peak_source": f"2 x cuBLAS bf16 burst of MEASURED_PEAKS.json ({peaks['source']}): "
                               "kind::i8 issues at twice the kind::f16 rate",
                "kernel": "gemm_i8_kernel<256, EPI_S8_BIAS_S8, PAIR=true> (256x256 tiles on CTA pairs)",
                "frac_of_nominal_4500": round(achieved / 4500.0, 4)}

    def cpu_sample(self):
        """Bounded sample for the CPU arm: the first `rows` rows of the same GEMM."""
        from oracle import w8a8 as O
        rows = 128
        x = self.x_host[:rows].clone()
        w, b = self.w.cpu(), self.b.cpu()
        ops = 2.0 * rows * HG[1] * HG[2]

        def run():
            return O.linear_a8_w8_b8_o8(x, w, b, self.alpha, self.beta)
        return run, ops / 1e12, f"first {rows} of {HG[0]} rows of the headline GEMM (all of W)", O.num_threads()


def time_steps(fn, steps, warmup, world):
    import torch.distributed as dist
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms / steps


def cpu_baseline(wl, min_seconds=10.0, max_reps=50):
    run, units, sample, cores = wl.cpu_sample()
    run()  # warm-up (page in, spin up the thread pool)
    t0 = time.perf_counter()
    reps = 0
    while True:
        run()
        reps += 1
        dt = time.perf_counter() - t0
        if dt >= min_seconds or reps >= max_reps:
            break
    return {"value": round(units * reps / dt, 4), "unit": wl.unit, "cores": cores, "kind": "port",
            "sample": f"{sample}; {reps} repetitions in {dt:.1f} s"}


def pick_workload(name, world):
    if name in (None, "auto"):
        name = "gemm"
    if name == "gemm":
        return GemmWorkload
    raise SystemExit(f"unknown workload {name}")


def run_reference(args, world, rank):
    """CPU arm: the reference semantics on the host cores (the oracle's C port)."""
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    WL = pick_workload(args.workload, world)
    wl = WL.__new__(WL)
    # CPU-only construction of the sample
    m, n, k = HG
    g = torch.Generator().manual_seed(0)
    wl.x_host = torch.randint(-127, 128, (128, k), generator=g, dtype=torch.int8)
    g1 = torch.Generator().manual_seed(1)
    wl.w = torch.randint(-127, 128, (n, k), generator=g1, dtype=torch.int8)
    wl.b = torch.randint(-127, 128, (n,), generator=g1, dtype=torch.int8)
    wl.alpha, wl.beta = 1e-4, 0.01
    run, units, sample, cores = wl.cpu_sample()
    for _ in range(max(1, min(args.warmup, 2))):
        run()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run()
    dt = time.perf_counter() - t0
    value = units * args.steps / dt
    line = {"impl": "reference", "metric": WL.metric, "value": round(value, 4), "unit": WL.unit,
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(dt / args.steps * 1e3, 3), "higher_is_better": True, "scaling": WL.scaling,
            "vs_baseline": None, "dtype": WL.dtype, "data": "synthetic (seeded uniform int8 on [-127,127])",
            "config": {"workload": WL.name, "M": HG[0], "N": HG[1], "K": HG[2], "sample": sample},
            "cpu_baseline": {"value": round(value, 4), "unit": WL.unit, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": round(value, 4), "unit": WL.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="auto")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile", action="store_true",
                    help="kernel-only run for ncu: no end-to-end leg, no CPU baseline")
    args = ap.parse_args()
    world, rank, local = dist_env()
    if args.impl == "reference":
        run_reference(args, world, rank)
        return
    if args.warmup < 3:
        args.warmup = 3
    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU fallback"
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    WL = pick_workload(args.workload, world)
    wl = WL(device)
    peaks = measured_peaks()

    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    ms = time_steps(wl.step, args.steps, args.warmup, world)
    clocks = sampler.stop() if sampler else None
    ms_e2e = ms if args.profile else time_steps(wl.step_e2e, args.steps, args.warmup, world)
    from torch_int import _CUDA as C
    status = C.device_status()
    assert status == 0, f"a kernel reported wait timeout {status}"
    if rank == 0:
        units = wl.units(world)
        line = {"metric": wl.metric, "value": round(units / (ms * 1e-3), 2), "unit": wl.unit, "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4),
                "higher_is_better": True, "scaling": wl.scaling, "vs_baseline": None, "dtype": wl.dtype,
                "data": "synthetic (seeded uniform int8 on [-127,127])", "config": wl.config(world),
                "e2e": {"value": round(units / (ms_e2e * 1e-3), 2), "unit": wl.unit,
                        "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h,
                        "ms_per_step": round(ms_e2e, 4)},
                "gpu_launches": wl.launches_per_step * args.steps, "clocks": clocks,
                "roofline": wl.roofline(ms, peaks)}
        if world == 1 and not args.no_cpu_baseline and not args.profile:
            line["cpu_baseline"] = cpu_baseline(wl)
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
