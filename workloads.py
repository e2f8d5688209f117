"""Times the benchmark configurations of the CAKE SGEMM path on one GPU.

    python workloads.py [--config NAME ...] [--reps R] [--list]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        workloads.py --distributed {square_8192,rect_m_first,rect_n_first,rect_k_first}

Each configuration prints one JSON line: device time of the whole library call
(CUDA events on the calling stream, operands resident in device memory, best of
R after one warm-up), the algorithmic work, and the rate against the bound that
applies (tensor pipe, FP32 pipe or HBM).  Inputs are synthetic and seeded:
uniform(-1, 1) operands, Bernoulli masks for the sparse operand, normal(0, 0.1)
for the convolution, as the configurations specify.

The headline number (8192^3 with its end-to-end and CPU-baseline legs) comes from
bench.py at the repository root; this module covers the other shapes: the square
sweep, the M-first / N-first / K-first rectangles, the batch of small products,
sparse A at several densities, the two convolutions and the packing routines.
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from cake_on_cpu_b200 import api  # noqa: E402

HBM_GBS = 6551.4          # measured copy bandwidth of this pool's B200s
TENSOR_3XTF32 = 274.5     # measured BF16 burst 1647.2 / 2 / 3, TFLOP/s
FP32_PIPE = 74.4          # 148 SMs x 128 lanes x 2 x 1.965 GHz, TFLOP/s


def _timed(fn, reps):
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    best = float("inf")
    for _ in range(reps):
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    return best


def _uniform(gen, *shape):
    return torch.rand(shape, device="cuda", generator=gen) * 2 - 1


def _dense(M, K, N, kernel):
    def run(reps):
        g = torch.Generator(device="cuda").manual_seed(1)
        A, B, C = _uniform(g, M, K), _uniform(g, K, N), torch.empty((M, N), device="cuda")
        ms = _timed(lambda: api.cake_sgemm(A, B, C, kernel=kernel), reps)
        st = api.last_stats()
        flops = 2.0 * M * N * K
        peak = TENSOR_3XTF32 if st["kernel"] == api.KERNEL_TF32X3 else FP32_PIPE
        return {"ms": ms, "flops": flops, "tflops": flops / ms / 1e9, "bound": "tensor" if peak == TENSOR_3XTF32 else "fp32",
                "frac": flops / ms / 1e9 / peak, "kernel_ms": st["ms_gemm"], "prepass_ms": st["ms_prepass"],
                "sched": ["KMN", "MKN", "NKM", "NA"][st["sched"]], "launches": st["launches"]}
    return run


def _dense_stream(n, graph):
    """Products enqueued back to back on one stream (no host synchronisation between them), eagerly or as a
    replayed CUDA graph of ten products: what a caller that keeps the GPU fed sees for a small product."""
    def run(reps):
        g = torch.Generator(device="cuda").manual_seed(1)
        A, B, C = _uniform(g, n, n), _uniform(g, n, n), torch.empty((n, n), device="cuda")
        s = torch.cuda.Stream()
        per = 10
        with torch.cuda.stream(s):
            def enqueue():
                for _ in range(per):
                    api.cake_sgemm_async(A.data_ptr(), B.data_ptr(), C.data_ptr(), n, n, n, 0, api.NA, api.KERNEL_TF32X3, s.cuda_stream)
            enqueue()
            s.synchronize()
            if graph:
                cg = torch.cuda.CUDAGraph()
                with torch.cuda.graph(cg, stream=s):
                    enqueue()
                enqueue = cg.replay
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            best = float("inf")
            for _ in range(max(reps, 1)):
                e0.record(s)
                for _ in range(10):
                    enqueue()
                e1.record(s)
                s.synchronize()
                best = min(best, e0.elapsed_time(e1) / (10 * per))
        flops = 2.0 * n ** 3
        return {"ms": best, "flops": flops, "tflops": flops / best / 1e9, "bound": "tensor", "frac": flops / best / 1e9 / TENSOR_3XTF32,
                "mode": "CUDA graph of 10 products" if graph else "asynchronous calls back to back"}
    return run


def _batched(batch, n, kernel=api.KERNEL_AUTO):
    def run(reps):
        g = torch.Generator(device="cuda").manual_seed(1)
        A, B = _uniform(g, batch, n, n), _uniform(g, batch, n, n)
        C = torch.empty((batch, n, n), device="cuda")
        ms = _timed(lambda: api.cake_sgemm_batched(A, B, C, kernel=kernel), reps)
        st = api.last_stats()
        flops, nbytes = 2.0 * batch * n ** 3, 3.0 * batch * n * n * 4
        return {"ms": ms, "flops": flops, "tflops": flops / ms / 1e9, "bytes": nbytes, "gbs": nbytes / ms / 1e6,
                "bound": "hbm", "frac": nbytes / ms / 1e6 / HBM_GBS, "kernel_ms": st["ms_gemm"],
                "ran": "tcgen05, operands split in shared memory" if st["kernel"] == api.KERNEL_TF32X3 else "ffma",
                "frac_fp32_pipe": flops / ms / 1e9 / FP32_PIPE}
    return run


def _sparse(n, density, kernel):
    def run(reps):
        g = torch.Generator(device="cuda").manual_seed(1)
        A = _uniform(g, n, n) * (torch.rand((n, n), device="cuda", generator=g) < density)
        B, C = _uniform(g, n, n), torch.empty((n, n), device="cuda")
        nnz = int((A != 0).sum().item())
        ms = _timed(lambda: api.cake_sp_sgemm(A, B, C, kernel=kernel), reps)
        st = api.last_stats()
        flops = 2.0 * nnz * n
        dense = st["kernel"] == api.KERNEL_TF32X3
        res = {"ms": ms, "nnz": nnz, "flops": flops, "tflops": flops / ms / 1e9,
               "ran": "dense tcgen05 on the operand as given" if dense else "zero skipping (compaction + gather)"}
        if dense:
            # every element is multiplied, zeros included: the tensor pipe bounds it
            rate = 2.0 * n ** 3 / ms / 1e9
            res.update({"bound": "tensor", "dense_tflops": rate, "frac": rate / TENSOR_3XTF32})
        else:
            # every nonzero of A pulls one row of B (N floats) through L2; no measured L2 peak to divide by
            gather = 4.0 * nnz * n
            res.update({"bound": "l2 gather", "gather_bytes": gather, "gbs": gather / ms / 1e6, "frac": None})
        return res
    return run


def _conv(b, cin, hw, cout):
    def run(reps):
        g = torch.Generator(device="cuda").manual_seed(4)
        x = torch.randn((b, cin, hw, hw), device="cuda", generator=g) * 0.1
        w = torch.randn((cout, cin, 3, 3), device="cuda", generator=g) * 0.1
        out = torch.empty((b, cout, hw, hw), device="cuda")
        ms = _timed(lambda: api.cake_conv2d(x, w, 1, 1, out), reps)
        flops = 2.0 * cout * cin * 9 * b * hw * hw
        nbytes = 4.0 * (x.numel() + w.numel() + out.numel())
        return {"ms": ms, "flops": flops, "tflops": flops / ms / 1e9, "bytes": nbytes, "gbs": nbytes / ms / 1e6,
                "bound": "tensor", "frac": flops / ms / 1e9 / TENSOR_3XTF32, "kernel_ms": api.last_stats()["ms_gemm"],
                "ran": ("ffma" if api.last_stats()["kernel"] != api.KERNEL_TF32X3 else
                        "tcgen05, implicit (patch operand built on chip)" if api.last_stats()["launches"] == 2 else
                        "tcgen05 on im2col planes")}
    return run


def _gemv(M, K, col_major):
    def run(reps):
        g = torch.Generator(device="cuda").manual_seed(1)
        A = _uniform(g, K, M) if col_major else _uniform(g, M, K)
        x, y = _uniform(g, K), torch.empty(M, device="cuda")
        ms = _timed(lambda: api.cake_sgemv(A, x, y, col_major=col_major), reps)
        nbytes = 4.0 * M * K
        return {"ms": ms, "kernel_ms": api.last_stats()["ms_gemm"], "bytes": nbytes, "gbs": nbytes / ms / 1e6, "bound": "hbm",
                "frac": nbytes / ms / 1e6 / HBM_GBS, "layout": "column-major" if col_major else "row-major"}
    return run


def _pack(n, which):
    def run(reps):
        g = torch.Generator(device="cuda").manual_seed(1)
        X = _uniform(g, n, n)
        cx = api.Cntx.make(49152, 2097152, 110100480, 8)  # CPU-style block sizes, as a caller of the reference has
        x = api.init_block_dims(n, n, n, 8, cx, api.KMN)
        if which == "A":
            P = torch.empty(api.cake_sgemm_packed_A_size(n, n, 8, x, cx, x.sch) // 4, device="cuda")
            ms = _timed(lambda: api.pack_A(X, n, n, 8, x, cx, P), reps)
        elif which == "B":
            P = torch.empty(api.cake_sgemm_packed_B_size(n, n, 8, x, cx) // 4, device="cuda")
            ms = _timed(lambda: api.pack_B(X, n, n, 8, x, cx, P), reps)
        else:
            P = torch.empty(api.cake_sgemm_packed_C_size(n, n, 8, x, cx, x.sch) // 4, device="cuda")
            api.pack_C(X, n, n, 8, x, cx, P)
            ms = _timed(lambda: api.unpack_C(P, n, n, 8, x, cx, X), reps)
        nbytes = 8.0 * n * n
        return {"ms": ms, "bytes": nbytes, "gbs": nbytes / ms / 1e6, "bound": "hbm", "frac": nbytes / ms / 1e6 / HBM_GBS}
    return run


CONFIGS = {}
for _n in (1024, 2048, 3000, 4096, 8192, 16384, 32768):
    CONFIGS["square_%d" % _n] = _dense(_n, _n, _n, api.KERNEL_AUTO)
for _n in (1024, 2048):
    CONFIGS["square_%d_stream" % _n] = _dense_stream(_n, False)
    CONFIGS["square_%d_graph" % _n] = _dense_stream(_n, True)
CONFIGS["square_8192_ffma"] = _dense(8192, 8192, 8192, api.KERNEL_FFMA)
CONFIGS["rect_m_first"] = _dense(65536, 1024, 1024, api.KERNEL_AUTO)
CONFIGS["rect_n_first"] = _dense(1024, 1024, 65536, api.KERNEL_AUTO)
CONFIGS["rect_k_first"] = _dense(1024, 262144, 1024, api.KERNEL_AUTO)
CONFIGS["small_batch"] = _batched(4096, 96)
CONFIGS["small_batch_ffma"] = _batched(4096, 96, api.KERNEL_FFMA)
for _d, _name in ((0.5, "50"), (0.1, "10"), (0.01, "1")):
    CONFIGS["sparse_%s" % _name] = _sparse(8192, _d, api.KERNEL_AUTO)
    CONFIGS["sparse_%s_zero_skipping" % _name] = _sparse(8192, _d, api.KERNEL_FFMA)
CONFIGS["conv_64x64x56"] = _conv(64, 64, 56, 64)
CONFIGS["conv_256x512x14"] = _conv(64, 256, 14, 512)
CONFIGS["gemv_16384_col_major"] = _gemv(16384, 16384, True)
CONFIGS["gemv_16384_row_major"] = _gemv(16384, 16384, False)
CONFIGS["gemv_1024x262144_col_major"] = _gemv(1024, 262144, True)
CONFIGS["pack_A_8192"] = _pack(8192, "A")
CONFIGS["pack_B_8192"] = _pack(8192, "B")
CONFIGS["unpack_C_8192"] = _pack(8192, "C")

DEFAULT = [k for k in CONFIGS if k not in ("square_32768", "sparse_50_zero_skipping", "sparse_10_zero_skipping")]


def _distributed(name, reps):
    """One product over all ranks of a torchrun launch (NCCL): every rank holds only its own share of the
    operands (row block, column block, grid block or K slice) before the timed region; the K split is timed twice,
    with the partial rows stored into the owners' memory by the summing kernel and with an NCCL reduce-scatter,
    either of which leaves every rank with its row block of C.  Device time, maximum over ranks."""
    import os
    import torch.distributed as dist
    from cake_on_cpu_b200 import distributed, partition
    shapes = {"square_8192": (8192, 8192, 8192), "rect_m_first": (65536, 1024, 1024), "rect_n_first": (1024, 1024, 65536),
              "rect_k_first": (1024, 262144, 1024)}
    M, K, N = shapes[name]
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    kind = partition.plan(M, N, K, world)
    g = torch.Generator(device="cuda").manual_seed(1)
    if kind == "k":
        k0, k1 = partition.k_block(K, world, rank)
        A, B = _uniform(g, M, k1 - k0), _uniform(g, k1 - k0, N)
        out = torch.empty((M // world, N), device="cuda") if M % world == 0 else None

        def step_nccl():
            partial = api.cake_sgemm(A, B)
            if out is not None:
                dist.reduce_scatter_tensor(out, partial)
            else:
                dist.all_reduce(partial)

        steps = [("reduce-scatter of the partial products (NCCL)", step_nccl)]
        shares = [partition.k_block(K, world, r) for r in range(world)]
        if world > 1 and all(api.kshard_supported(M, N, b - a) for a, b in shares):
            x = distributed._exchange(M, N, world, rank, None)
            mine = torch.empty((x.rows[1] - x.rows[0], N), device="cuda")

            def step_stores():
                x.partial(A, B)
                x.finish(mine)

            steps.insert(0, ("rows stored into the owners' memory while the tiles are summed, owners add the slots", step_stores))
    else:
        r0, r1, c0, c1 = (partition.grid_block(M, N, K, world, rank) if kind == "grid" else
                          partition.row_block(M, world, rank) + (0, N) if kind == "rows" else
                          (0, M) + partition.col_block(N, world, rank))
        A, B = _uniform(g, r1 - r0, K), _uniform(g, K, c1 - c0)
        C = torch.empty((r1 - r0, c1 - c0), device="cuda")

        def step():
            api.cake_sgemm(A, B, C)

        steps = [("none", step)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for exchange, step in steps:
        for _ in range(3):
            step()
        best = float("inf")
        for _ in range(max(reps, 3)):
            dist.barrier()
            torch.cuda.synchronize()
            e0.record()
            step()
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1)], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            best = min(best, float(t.item()))
        if rank == 0:
            flops = 2.0 * M * N * K
            print(json.dumps({"config": name, "ranks": world, "split": kind, "ms": round(best, 4), "flops": flops,
                              "tflops": round(flops / best / 1e9, 2), "exchange": exchange}), flush=True)
    distributed.release()
    dist.barrier()
    dist.destroy_process_group()


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", nargs="*", default=None)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--list", action="store_true")
    ap.add_argument("--distributed", default=None, help="time one dense shape over the ranks of a torchrun launch")
    args = ap.parse_args(argv)
    if args.distributed:
        api.lib()
        _distributed(args.distributed, args.reps)
        return 0
    if args.list:
        print("\n".join(CONFIGS))
        return 0
    api.lib()
    for name in (args.config or DEFAULT):
        if name not in CONFIGS:
            print(json.dumps({"config": name, "error": "unknown configuration"}))
            continue
        res = CONFIGS[name](args.reps)
        res = {k: (round(v, 4) if isinstance(v, float) else v) for k, v in res.items()}
        print(json.dumps(dict(config=name, **res)), flush=True)
        torch.cuda.empty_cache()
    return 0


if __name__ == "__main__":
    sys.exit(main())
