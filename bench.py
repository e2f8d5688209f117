#!/usr/bin/env python
"""Benchmark of the CAKE SGEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--size S]

Workload (the headline configuration): dense FP32 C = A*B, M = K = N = 8192,
row-major, A and B uniform(-1, 1) from a fixed seed, computed by the tcgen05
3xTF32 kernel.  A "step" is one whole product: the operand-split pass plus the
contraction kernel.  At N > 1 GPUs (one process per GPU, launched by
torch.distributed.run) the same 8192^3 product is split by row blocks of M,
B replicated, no collective on the data path ("strong" scaling).

Prints ONE JSON line.  `value` is whole-job TFLOP/s with operands resident in
HBM; `e2e` is the same product through the public host-pointer API (pinned host
buffers, host->device and device->host copies inside the timed region);
`roofline` describes the contraction kernel alone; `cpu_baseline` is the
reference's own CPU cake_sgemm timed on this box's host cores.

`--impl reference` times only that CPU implementation (rank 0; other ranks exit).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "FP32 SGEMM TFLOP/s at 8192^3"
UNIT = "TFLOP/s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="cake_b200", choices=["cake_b200", "reference"])
    ap.add_argument("--size", type=int, default=8192, help="M = K = N (default: the headline 8192)")
    ap.add_argument("--kernel", default="tf32x3", choices=["tf32x3", "ffma"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    return ap.parse_args()


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d["hbm_gbs"], d["bf16_tflops"], d.get("bf16_tflops_sustained", d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.QUERY,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [float(r[1]) for r in self.rows if len(r) >= 8 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 8 and r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 8 and r[4 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ----------------------------------------------------------------- CPU arm

def cpu_threads_and_ctx(ref):
    ctx, info = ref.query_ctx()
    return ctx, info


def time_reference(size, steps, warmup, budget_s=150.0):
    """Reference CPU cake_sgemm (oracle/_ref) on a bounded row sample of the size^3 product."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import numpy as np
    from _oracle import NA, Oracle, Reference
    O = Oracle()
    K = N = size
    if Reference.available():
        R, kind = Reference(), "reference"
        ctx, info = R.query_ctx()
        cores = info["ncores"]

        def run(A, B):
            return R.sgemm(A, B, cores, NA, ctx=ctx)[1]
    else:
        kind, cores, info = "port", os.cpu_count() or 1, {}

        def run(A, B):
            t0 = time.perf_counter()
            O.sgemm(A, B, cores, NA)
            return time.perf_counter() - t0
    B = O.uniform((K, N), 2)
    probe_rows = min(size, 512)
    A = O.uniform((probe_rows, K), 1)
    t_probe = run(A, B)
    rate = 2.0 * probe_rows * K * N / max(t_probe, 1e-9)
    per_step_target = min(2.0, budget_s / max(steps + warmup, 1))
    rows = int(min(size, max(128, rate * per_step_target / (2.0 * K * N))))
    rows = max(128, rows // 128 * 128)
    A = O.uniform((rows, K), 1)
    for _ in range(warmup):
        run(A, B)
    times = [run(A, B) for _ in range(steps)]
    total = sum(times)
    tflops = 2.0 * rows * K * N * steps / total / 1e12
    return {"value": tflops, "unit": UNIT, "cores": cores, "kind": kind,
            "sample": "%d x %d x %d row block of the %d^3 product per step, %d steps (+%d warm-up); time = value "
                      "returned by cake_sgemm (packing included); host context %s" % (rows, K, N, size, steps, warmup, info),
            "ms_per_step": total / steps * 1e3}


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    r = time_reference(args.size, args.steps, args.warmup)
    line = {"impl": "reference", "metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "dense FP32 SGEMM M=K=N=%d, uniform(-1,1), seeded" % args.size, "kernel": "reference CPU cake_sgemm",
                       "step": "one cake_sgemm call on a row block of the product (see cpu_baseline.sample)"},
            "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


# ----------------------------------------------------------------- GPU arm

def gpu_arm(args):
    import torch
    import cake_on_cpu_b200 as cake
    from cake_on_cpu_b200 import build
    from cake_on_cpu_b200.partition import grid_block, grid_shape

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit("--gpus %d but WORLD_SIZE=%d" % (args.gpus, world))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if not os.path.exists(cake.library_path()):
        build.build()
    cake.lib()

    size = args.size
    M = K = N = size
    # rank (i, j) of a pr x pc grid owns C[r0:r1, c0:c1]; nothing is exchanged (pc = 1: plain row blocks, B replicated)
    pr, pc = grid_shape(M, N, K, world)
    r0, r1, c0, c1 = grid_block(M, N, K, world, rank)
    rows, cols = r1 - r0, c1 - c0
    kernel = cake.KERNEL_TF32X3 if args.kernel == "tf32x3" else cake.KERNEL_FFMA

    g = torch.Generator(device="cuda").manual_seed(1234)
    A = (torch.rand((M, K), device="cuda", generator=g) * 2 - 1)[r0:r1].contiguous()
    B = (torch.rand((K, N), device="cuda", generator=g) * 2 - 1)[:, c0:c1].contiguous()
    C = torch.empty((rows, cols), device="cuda")
    stream = torch.cuda.current_stream()

    def step():
        cake.cake_sgemm_async(A.data_ptr(), B.data_ptr(), C.data_ptr(), rows, cols, K, 0, cake.NA, kernel, stream.cuda_stream)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # first call allocates the scratch arena (blocking entry point), then warm up
    cake.cake_sgemm(A, B, C, kernel=kernel)
    launches_per_step = cake.last_stats()["launches"]
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    # per-kernel CUDA events inside the timed region (recorded on the launching stream, no synchronisation)
    cake.profile_begin()
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    barrier()
    prof_pre_ms, prof_kern_ms, prof_calls = cake.profile_end()
    ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    if dist is not None:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_total = float(ms.item())
    clocks = sampler.stop() if rank == 0 else None

    # the contraction kernel alone: average launch duration over the timed region itself
    # (only the first 256 steps carry events)
    calls = max(prof_calls, 1)
    kern = torch.tensor([prof_kern_ms / calls], device="cuda")
    pre = torch.tensor([prof_pre_ms / calls], device="cuda")
    if dist is not None:
        dist.all_reduce(kern, op=dist.ReduceOp.MAX)
    kern_ms_avg = float(kern.item())

    # end to end through the public API: pinned host operands, copies inside the timed region
    Ah = torch.empty((rows, K), pin_memory=True).copy_(A)
    Bh = torch.empty((K, cols), pin_memory=True).copy_(B)
    Ch = torch.empty((rows, cols), pin_memory=True)
    e2e_steps = max(3, min(args.steps, 10))
    cake.cake_sgemm(Ah.numpy(), Bh.numpy(), Ch.numpy(), kernel=kernel)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        cake.cake_sgemm(Ah.numpy(), Bh.numpy(), Ch.numpy(), kernel=kernel)
        _ = float(Ch[0, 0])
    barrier()
    e2e_s = torch.tensor([time.perf_counter() - t0], device="cuda")
    if dist is not None:
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
    e2e_stats = cake.last_stats()

    flops = 2.0 * M * N * K
    if rank == 0:
        hbm, bf16_burst, bf16_sust, which = measured_peaks()
        peak = bf16_burst / 2 / 3 if args.kernel == "tf32x3" else 148 * 128 * 2 * 1.965e9 / 1e12
        achieved = 2.0 * rows * cols * K / (kern_ms_avg * 1e-3) / 1e12
        # DRAM bytes of one contraction launch, from one ncu capture of the 8192^3 launch on one GPU
        # (dram__bytes_read.sum 5.22 GB + dram__bytes_write.sum 0.255 GB; summary under profiles/).  The
        # algorithmic bytes are 1.34 GB (four operand planes read once, C written once); the rest is A and B
        # panels read again by later waves of tiles once they have left the 126 MB L2.  A rank of a
        # multi-GPU run owns rows x cols of C and its traffic is scaled by that share.
        traffic = None
        if args.kernel == "tf32x3" and size == 8192:
            traffic = (5.22e9 + 0.25544e9) * (rows * cols) / float(M * N)
        line = {
            "metric": METRIC, "value": flops * args.steps / (ms_total * 1e-3) / 1e12, "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_total / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "dense FP32 SGEMM M=K=N=%d, uniform(-1,1), seeded" % size,
                       "kernel": args.kernel, "partition": ("row blocks of M over %d GPU(s), B replicated" % world) if pc == 1 else
                                    ("%d x %d grid of GPUs: row blocks of A x column blocks of B, no exchange" % (pr, pc)),
                       "l2": "operands (%.0f MB per GPU) exceed the 126 MB L2; no flush between steps" %
                             ((rows * K + K * cols + rows * cols) * 4 / 1e6),
                       "step": "operand split pass + contraction kernel"},
            "clocks": clocks,
            "e2e": {"value": flops * e2e_steps / float(e2e_s.item()) / 1e12, "unit": UNIT,
                    "h2d_bytes_per_step": (rows * K + K * cols) * 4, "d2h_bytes_per_step": rows * cols * 4,
                    "ms_h2d": e2e_stats["ms_h2d"], "ms_d2h": e2e_stats["ms_d2h"], "steps": e2e_steps},
            "gpu_launches": launches_per_step * args.steps,
            "roofline": {"bound": "tensor", "kernel": "sgemm_tf32x3_kernel" if args.kernel == "tf32x3" else "sgemm_ffma_kernel",
                         "achieved": achieved, "peak": peak, "unit": UNIT, "frac": achieved / peak,
                         "peak_source": ("bf16 burst %.1f TFLOP/s of %s / 2 (TF32 rate) / 3 (MMAs per product)" % (bf16_burst, which))
                         if args.kernel == "tf32x3" else "148 SMs x 128 lanes x 2 flop x 1.965 GHz",
                         "frac_of_sustained": achieved / (bf16_sust / 6) if args.kernel == "tf32x3" else None,
                         "kernel_ms": kern_ms_avg, "prepass_ms": float(pre.item()),
                         "traffic": traffic},
        }
        if world == 1 and not args.no_cpu_baseline:
            try:
                r = time_reference(size, 2, 1, budget_s=30.0)
                line["cpu_baseline"] = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}
            except Exception as exc:  # the bench line is still valid without it
                line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": 0, "kind": "reference",
                                        "sample": "failed: %r" % (exc,)}
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()
