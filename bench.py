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
    ap.add_argument("--no-bind", action="store_true", help="do not bind the process to the CPUs next to its GPU")
    ap.add_argument("--repeats", type=int, default=5, help="timed regions of --steps steps each; the median is reported")
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
                                          "--format=csv,noheader,nounits", "-lms", "20"],
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


def time_reference(size, steps, warmup, budget_s=200.0):
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
    # the whole product per step when the run then still ends within the budget, else a block of its rows
    per_step_target = budget_s / max(steps + warmup, 1)
    rows = int(min(size, max(128, rate * per_step_target / (2.0 * K * N))))
    rows = size if rows >= size else max(128, rows // 128 * 128)
    A = O.uniform((rows, K), 1)
    for _ in range(warmup):
        run(A, B)
    times = [run(A, B) for _ in range(steps)]
    total = sum(times)
    tflops = 2.0 * rows * K * N * steps / total / 1e12
    return {"value": tflops, "unit": UNIT, "cores": cores, "kind": kind,
            "sample": "%s per step, %d steps (+%d warm-up); time = value returned by cake_sgemm (packing included); "
                      "host context %s" % ("the whole %d^3 product" % size if rows == size else
                                           "%d x %d x %d row block of the %d^3 product" % (rows, K, N, size), steps, warmup, info),
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
                       "step": "one cake_sgemm call (see cpu_baseline.sample)"},
            "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


# ----------------------------------------------------------------- GPU arm

def sampled_parity(torch, A_rows, B_cols, C_block, seed, side=32):
    """Largest deviation of side x side entries of this rank's block of C from a float64 recomputation:
    (normalised by ||A[m,:]|| ||B[:,n]||, absolute, entries)."""
    import numpy as np
    rng = np.random.default_rng(seed)
    rows = torch.as_tensor(np.sort(rng.choice(C_block.shape[0], min(side, C_block.shape[0]), replace=False)), device="cuda")
    cols = torch.as_tensor(np.sort(rng.choice(C_block.shape[1], min(side, C_block.shape[1]), replace=False)), device="cuda")
    a, b = A_rows[rows].double(), B_cols[:, cols].double()
    d = (C_block[rows][:, cols].double() - a @ b).abs()
    den = a.norm(dim=1)[:, None] * b.norm(dim=0)[None, :]
    return (d / den.clamp_min(1e-30)).max().item(), d.max().item(), rows.numel() * cols.numel()


def gpu_arm(args):
    import numpy as np
    import torch
    import cake_on_cpu_b200 as cake
    from cake_on_cpu_b200 import build, distributed, seeded
    from cake_on_cpu_b200.partition import grid_block, grid_shape, k_block, row_block

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit("--gpus %d but WORLD_SIZE=%d" % (args.gpus, world))
    torch.cuda.set_device(local)
    near_cpus = None if args.no_bind else distributed.bind_near_gpu(local)  # pinned buffers next to this rank's GPU
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if not os.path.exists(cake.library_path()):
        build.build()
    cake.lib()

    def reduce_max(v):
        t = torch.tensor([float(v)], device="cuda", dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def reduce_sum(v):
        t = torch.tensor([float(v)], device="cuda", dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    size = args.size
    M = K = N = size
    # rank (i, j) of a pr x pc grid owns C[r0:r1, c0:c1]; nothing is exchanged (pc = 1: plain row blocks, B replicated)
    pr, pc = grid_shape(M, N, K, world)
    r0, r1, c0, c1 = grid_block(M, N, K, world, rank)
    rows, cols = r1 - r0, c1 - c0
    kernel = cake.KERNEL_TF32X3 if args.kernel == "tf32x3" else cake.KERNEL_FFMA

    # the seeded streams of the benchmark configurations: A = stream 1, B = stream 2, uniform(-1, 1)
    A_full = seeded.uniform((M, K), 1)
    B_full = seeded.uniform((K, N), 2)
    A = A_full[r0:r1].contiguous()
    B = B_full[:, c0:c1].contiguous()
    C = torch.full((rows, cols), float("nan"), device="cuda")
    stream = torch.cuda.current_stream()

    def step():
        cake.cake_sgemm_async(A.data_ptr(), B.data_ptr(), C.data_ptr(), rows, cols, K, 0, cake.NA, kernel, stream.cuda_stream)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # measured issue rate of the tensor pipe (outside every timed region)
    tf32_rate, tf32_ms = cake.tf32_peak(5.0) if args.kernel == "tf32x3" else (None, None)

    # first call allocates the scratch arena (blocking entry point), then warm up
    cake.cake_sgemm(A, B, C, kernel=kernel)
    launches_per_step = cake.last_stats()["launches"]
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()

    # K steps are timed as one region; the region is repeated so that the clock sampler sees the load for long
    # enough, and the median region is the one reported
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    regions = []
    for rep in range(max(args.repeats, 1)):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        cake.profile_begin()  # per-kernel CUDA events inside the timed region (launching stream, no synchronisation)
        e0.record(stream)
        for _ in range(args.steps):
            step()
        e1.record(stream)
        barrier()
        prof_pre_ms, prof_kern_ms, prof_calls = cake.profile_end()
        calls = max(prof_calls, 1)
        regions.append((reduce_max(e0.elapsed_time(e1)), reduce_max(prof_kern_ms / calls), reduce_max(prof_pre_ms / calls)))
    clocks = sampler.stop() if rank == 0 else None
    regions.sort()
    ms_total, kern_ms_avg, pre_ms_avg = regions[len(regions) // 2]

    # parity, outside the timed region: 1024 entries of this rank's block against float64, worst over ranks
    err_n, err_a, entries = sampled_parity(torch, A, B, C, 100 + rank)
    parity_n, parity_a = reduce_max(err_n), reduce_max(err_a)
    nan_blocks = reduce_sum(float(torch.isnan(C).any().item()))

    # end to end through the public API: pinned host operands, copies inside the timed region.  One GPU: the
    # reference's call, cake_sgemm on host pointers.  Several GPUs: row blocks of A and C, and every rank copies
    # only its own 1/N of the rows of B from the host; the slices are gathered over NVLink into local memory.
    er0, er1 = row_block(M, world, rank)
    k0, k1 = k_block(K, world, rank)
    Ah = torch.empty((er1 - er0, K), pin_memory=True).copy_(A_full[er0:er1])
    Bh = torch.empty((k1 - k0, N), pin_memory=True).copy_(B_full[k0:k1])
    Ch = torch.empty((er1 - er0, N), pin_memory=True)
    del A_full
    e2e_steps = max(3, min(args.steps, 10))

    def e2e_step():
        distributed.sharded_sgemm_host(Ah.numpy(), Bh.numpy(), Ch.numpy(), kernel=kernel)
        return float(Ch[0, 0])

    e2e_step()
    e2e_stats = cake.last_stats()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_s = reduce_max(time.perf_counter() - t0)
    e2e_n, e2e_a, _ = sampled_parity(torch, Ah.cuda(), B_full, Ch.cuda(), 200 + rank)
    e2e_parity = reduce_max(e2e_n)
    h2d = reduce_sum((Ah.numel() + Bh.numel()) * 4)
    d2h = reduce_sum(Ch.numel() * 4)

    flops = 2.0 * M * N * K
    ok = parity_n <= 1e-5 and e2e_parity <= 1e-5 and nan_blocks == 0
    if rank == 0:
        hbm, bf16_burst, bf16_sust, which = measured_peaks()
        peak = bf16_burst / 2 / 3 if args.kernel == "tf32x3" else 148 * 128 * 2 * 1.965e9 / 1e12
        achieved = 2.0 * rows * cols * K / (kern_ms_avg * 1e-3) / 1e12
        # DRAM bytes of one contraction launch, from one ncu capture of the 8192^3 launch on one GPU
        # (dram__bytes_read.sum 4.552 GB + dram__bytes_write.sum 0.520 GB; summary under profiles/).  The
        # algorithmic bytes are 1.34 GB (four operand planes read once, C written once); the rest is A and B
        # panels read again by later waves of tiles once they have left the 126 MB L2.  A rank of a
        # multi-GPU run owns rows x cols of C and its traffic is scaled by that share.
        traffic = None
        if args.kernel == "tf32x3" and size == 8192:
            traffic = (4.552e9 + 0.520e9) * (rows * cols) / float(M * N)
        roofline = {"bound": "tensor", "kernel": "sgemm_tf32x3_chunked_kernel<256, pair>" if args.kernel == "tf32x3" else "sgemm_ffma_kernel",
                    "achieved": achieved, "peak": peak, "unit": UNIT, "frac": achieved / peak,
                    "peak_source": ("bf16 burst %.1f TFLOP/s of %s / 2 (TF32 rate) / 3 (MMAs per product)" % (bf16_burst, which))
                    if args.kernel == "tf32x3" else "148 SMs x 128 lanes x 2 flop x 1.965 GHz",
                    "frac_of_sustained": achieved / (bf16_sust / 6) if args.kernel == "tf32x3" else None,
                    "kernel_ms": kern_ms_avg, "prepass_ms": pre_ms_avg, "traffic": traffic}
        if tf32_rate:
            # measured on this device just before the timed region: every SM issuing tcgen05.mma kind::tf32
            # 128 x 256 x 8 back to back on resident shared-memory tiles (cakeb200_tf32_peak), no memory traffic
            roofline["tf32_issue_rate"] = {"tflops": tf32_rate, "ms": tf32_ms, "third": tf32_rate / 3,
                                           "frac_of_third": achieved / (tf32_rate / 3),
                                           "how": "tcgen05.mma kind::tf32 128x256x8 issue-rate microbenchmark, measured"}
            # The microbenchmark lasts 5 ms and runs at the maximum SM clock (its 1113-1116 TFLOP/s are 99 % of
            # 148 SMs x 8192 flop/clock x 1.965 GHz, and ncu shows its tensor pipe 99.5 % active); the timed loop
            # runs for seconds under the power cap at the sampled clock.  Scaled to that clock the pipe could
            # have issued third x (sampled MHz / max MHz).
            if clocks and clocks.get("sm_mhz") and clocks.get("sm_max_mhz"):
                scale = clocks["sm_mhz"] / clocks["sm_max_mhz"]
                roofline["tf32_issue_rate"]["third_at_sampled_clock"] = tf32_rate / 3 * scale
                roofline["tf32_issue_rate"]["frac_at_sampled_clock"] = achieved / (tf32_rate / 3 * scale)
        line = {
            "metric": METRIC, "value": flops * args.steps / (ms_total * 1e-3) / 1e12, "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_total / args.steps,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "dense FP32 SGEMM M=K=N=%d, uniform(-1,1), seeded" % size,
                       "kernel": args.kernel, "partition": ("row blocks of M over %d GPU(s), B replicated" % world) if pc == 1 else
                                    ("%d x %d grid of GPUs: row blocks of A x column blocks of B, no exchange" % (pr, pc)),
                       "l2": "operands (%.0f MB per GPU) exceed the 126 MB L2; no flush between steps" %
                             ((rows * K + K * cols + rows * cols) * 4 / 1e6),
                       "step": "operand split pass + contraction kernel",
                       "timed_regions": "%d regions of %d steps, the median region is reported" % (len(regions), args.steps),
                       "inputs": "counter-based streams: A = stream 1, B = stream 2 (cake_on_cpu_b200/seeded.py)"},
            "clocks": clocks,
            "parity": {"norm_err": parity_n, "abs_err": parity_a, "entries_per_rank": entries, "against": "float64",
                       "e2e_norm_err": e2e_parity, "tolerance": 1e-5, "ok": ok},
            "e2e": {"value": flops * e2e_steps / e2e_s / 1e12, "unit": UNIT,
                    "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                    "ms_per_step": e2e_s / e2e_steps * 1e3, "steps": e2e_steps,
                    "ms_h2d_last_rank0": e2e_stats["ms_h2d"], "ms_d2h_last_rank0": e2e_stats["ms_d2h"],
                    "host_cpus_bound": (len(near_cpus) if near_cpus else 0),
                    "how": "cake_sgemm on pinned host operands" if world == 1 else
                           "distributed.sharded_sgemm_host: row blocks of A and C; each rank copies 1/%d of the rows of B from "
                           "the host, the slices are gathered over NVLink (NCCL all-gather) into local memory" % world},
            "gpu_launches": launches_per_step * args.steps,
            "roofline": roofline,
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
        distributed.release()
        dist.barrier()
        dist.destroy_process_group()
    if not ok:
        raise SystemExit("parity check failed: normalised error %.3e (device), %.3e (end to end), %d blocks with NaN"
                         % (parity_n, e2e_parity, int(nan_blocks)))


def main():
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()
