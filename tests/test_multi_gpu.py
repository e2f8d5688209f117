"""One process per GPU over NCCL: row split, column split, the 2 x 2 grid and the K split
(summed by stores into the owners' memory and, for comparison, by a reduce-scatter), each
checked against a float64 product.  Needs two (four) GPUs;
skipped on a single-GPU box (the host logic is covered on CPU by test_partition_gloo.py)."""
import os
import socket

import pytest

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


TWO_RANK_CASES = [(2048, 512, 768, "rows"), (256, 384, 4096, "cols"), (512, 16384, 256, "k"), (300, 20000, 130, "k")]
FOUR_RANK_CASES = [(4096, 512, 4096, "grid"), (3000, 700, 2900, "grid"), (8192, 256, 512, "rows"), (640, 32768, 256, "k")]


def _worker(rank, world, port, out, cases=TWO_RANK_CASES):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from cake_on_cpu_b200 import distributed
    results = []
    for (M, K, N, want) in cases:
        g = torch.Generator(device="cuda").manual_seed(5)
        A = torch.rand((M, K), device="cuda", generator=g) * 2 - 1
        B = torch.rand((K, N), device="cuda", generator=g) * 2 - 1
        kind, span, block = distributed.sharded_sgemm(A, B)
        full = A.double() @ B.double()
        den = A.double().norm(dim=1)[:, None] * B.double().norm(dim=0)[None, :]
        if kind == "grid":
            cut = lambda X: X[span[0]:span[1], span[2]:span[3]]
        elif kind == "cols":
            cut = lambda X: X[:, span[0]:span[1]]
        else:
            cut = lambda X: X[span[0]:span[1]]
        err = ((block.double() - cut(full)).abs() / cut(den)).max().item() if block.shape == cut(full).shape else float("inf")
        if kind == "k":
            # the same product summed by NCCL instead of by stores into the owners' memory
            _, span2, block2 = distributed.sharded_sgemm(A, B, exchange="nccl")
            err2 = ((block2.double() - full[span2[0]:span2[1]]).abs() / den[span2[0]:span2[1]]).max().item()
            err = max(err, err2)
        results.append((kind == want, err, span[0], span[1], block.numel()))
    # independent units: batch items, row blocks of a sparse operand, images of a convolution
    g = torch.Generator(device="cuda").manual_seed(6)
    Ab = torch.rand((37, 96, 64), device="cuda", generator=g) * 2 - 1
    Bb = torch.rand((37, 64, 80), device="cuda", generator=g) * 2 - 1
    (lo, hi), Cb = distributed.sharded_sgemm_batched(Ab, Bb)
    err_b = (Cb.double() - torch.bmm(Ab[lo:hi].double(), Bb[lo:hi].double())).abs().max().item()
    As = (torch.rand((700, 512), device="cuda", generator=g) * 2 - 1) * (torch.rand((700, 512), device="cuda", generator=g) < 0.02)
    Bs = torch.rand((512, 384), device="cuda", generator=g) * 2 - 1
    (r0, r1), Cs = distributed.sharded_sp_sgemm(As, Bs)
    err_s = (Cs.double() - As[r0:r1].double() @ Bs.double()).abs().max().item()
    x = torch.randn((9, 16, 12, 12), device="cuda", generator=g) * 0.1
    w = torch.randn((24, 16, 3, 3), device="cuda", generator=g) * 0.1
    (i0, i1), y = distributed.sharded_conv2d(x, w, 1, 1)
    err_c = (y.double() - torch.nn.functional.conv2d(x[i0:i1].double(), w.double(), padding=1)).abs().max().item()
    # host operands: row blocks of A and C, every rank copies only its slice of B, the rest arrives from the peers
    from cake_on_cpu_b200 import partition
    err_h = 0.0
    for (M, K, N) in ((2560, 1024, 1536), (2100, 1000, 520), (96, 64, 40)):  # even slices, ragged slices, tiny
        gh = torch.Generator(device="cuda").manual_seed(8)
        A = torch.rand((M, K), device="cuda", generator=gh) * 2 - 1
        B = torch.rand((K, N), device="cuda", generator=gh) * 2 - 1
        a0, a1 = partition.row_block(M, world, rank)
        b0, b1 = partition.k_block(K, world, rank)
        Ah = torch.empty((a1 - a0, K), pin_memory=True).copy_(A[a0:a1])
        Bh = torch.empty((b1 - b0, N), pin_memory=True).copy_(B[b0:b1])
        Ch = torch.full((a1 - a0, N), float("nan")).pin_memory()
        for _ in range(2):  # twice: the gathered B of the first call is overwritten by the second
            distributed.sharded_sgemm_host(Ah.numpy(), Bh.numpy(), Ch.numpy())
        if a1 > a0:
            exact = A[a0:a1].double() @ B.double()
            den = A[a0:a1].double().norm(dim=1)[:, None] * B.double().norm(dim=0)[None, :]
            err_h = max(err_h, ((Ch.cuda().double() - exact).abs() / den).max().item())
    units = (hi - lo, r1 - r0, i1 - i0, err_b, err_s, err_c, err_h)
    gathered = [None] * world
    dist.all_gather_object(gathered, (results, units))
    if rank == 0:
        out.put(gathered)
    distributed.release()
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_nccl(cake):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = out.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    units = [u for _, u in res]
    res = [r for r, _ in res]
    for per_rank in res:
        for ok_kind, err, lo, hi, _ in per_rank:
            assert ok_kind
            assert err <= 1e-5
    # the two ranks' blocks tile the matrix
    for case in range(len(res[0])):
        assert res[0][case][2] == 0 and res[0][case][3] == res[1][case][2]
    # batch items, sparse row blocks and images: every unit owned once, results right
    assert sum(u[0] for u in units) == 37 and sum(u[1] for u in units) == 700 and sum(u[2] for u in units) == 9
    assert all(u[3] <= 1e-3 and u[4] <= 1e-3 and u[5] <= 1e-4 for u in units), units
    assert all(u[6] <= 1e-5 for u in units), units


def test_four_ranks_nccl_grid(cake):
    """2 x 2 process grid (no exchange), a row split and a K split at world size 4."""
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 4:
        pytest.skip("needs four GPUs")
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 4, port, out, FOUR_RANK_CASES)) for r in range(4)]
    for p in procs:
        p.start()
    res = out.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert all(u[6] <= 1e-5 for _, u in res), [u for _, u in res]
    res = [r for r, _ in res]
    for per_rank in res:
        for ok_kind, err, lo, hi, _ in per_rank:
            assert ok_kind
            assert err <= 1e-5
    # every element of C is owned exactly once
    for case, (M, K, N, _) in enumerate(FOUR_RANK_CASES):
        assert sum(per_rank[case][4] for per_rank in res) == M * N


@pytest.mark.parametrize("shape", [(2304, 256, 640), (4100, 1111, 1300)])
def test_cpp_api_splits_rows_over_visible_gpus(cake, tmp_path, shape):
    """cake_sgemm(p > 1) with host pointers: one host thread per device inside the call; each device copies
    its own slice of B from the host and fetches the other slices from its peers (on one GPU: the plain call)."""
    import numpy as np
    import ctypes
    L = ctypes.CDLL(cake.library_path())
    rng = np.random.default_rng(3)
    M, K, N = shape
    A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    B = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    C = np.full((M, N), np.nan, np.float32)
    # C++ symbol of cake_sgemm(float*, float*, float*, int, int, int, int, cake_cntx_t*, char**, bool, bool, float, float, sched, int, int, int)
    fn = getattr(L, "_Z10cake_sgemmPfS_S_iiiiP11cake_cntx_tPPcbbff5schediii")
    fn.restype = ctypes.c_double
    fn.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int] * 4 + [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_bool, ctypes.c_bool,
                                                              ctypes.c_float, ctypes.c_float, ctypes.c_int, ctypes.c_int,
                                                              ctypes.c_int, ctypes.c_int]
    t = fn(A.ctypes.data, B.ctypes.data, C.ctypes.data, M, N, K, 8, None, None, False, False, 1.0, 0.0, 3, 0, 0, 0)
    assert t > 0
    ref = A.astype(np.float64) @ B.astype(np.float64)
    den = np.outer(np.linalg.norm(A, axis=1), np.linalg.norm(B, axis=0))
    assert (np.abs(C - ref) / den).max() <= 1e-5
