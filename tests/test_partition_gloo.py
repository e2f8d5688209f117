"""Host-side logic of the multi-GPU split, run as two CPU ranks over gloo: the
shares tile the matrix exactly, and the K split's reduce-scatter reassembles
the product.  (numpy matmul stands in for the local GPU product here; the GPU
product itself is covered by the gpu-marked tests.)"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cake_on_cpu_b200 import partition


def test_blocks_tile_the_range():
    for total in (1, 100, 128, 1000, 8192, 65536):
        for world in (1, 2, 3, 4, 8):
            for fn in (partition.row_block, partition.col_block, partition.k_block):
                cuts = [fn(total, world, r) for r in range(world)]
                assert cuts[0][0] == 0 and cuts[-1][1] == total
                for a, b in zip(cuts, cuts[1:]):
                    assert a[1] == b[0]
    assert partition.row_block(8192, 8, 3) == (3072, 4096)


def test_unit_blocks_tile_the_batch():
    for units in (1, 7, 64, 4096):
        for world in (1, 2, 3, 8):
            cuts = [partition.unit_block(units, world, r) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == units
            assert all(a[1] == b[0] for a, b in zip(cuts, cuts[1:]))
            assert max(hi - lo for lo, hi in cuts) - min(hi - lo for lo, hi in cuts) <= 1


def test_plan_follows_the_benchmark_shapes():
    assert partition.plan(8192, 8192, 8192, 2) == "rows"
    assert partition.plan(8192, 8192, 8192, 4) == "grid" and partition.grid_shape(8192, 8192, 8192, 4) == (2, 2)
    assert partition.plan(8192, 8192, 8192, 8) == "grid" and partition.grid_shape(8192, 8192, 8192, 8) == (4, 2)
    assert partition.plan(65536, 1024, 1024, 8) == "rows"
    assert partition.plan(1024, 65536, 1024, 8) == "cols"
    assert partition.plan(1024, 1024, 262144, 8) == "k"
    assert partition.plan(5, 5, 5, 1) == "rows"


def test_grid_blocks_tile_the_matrix():
    for (M, N, K) in [(8192, 8192, 8192), (3000, 3000, 3000), (16384, 4096, 512), (1000, 5000, 64)]:
        for world in (1, 2, 4, 6, 8):
            pr, pc = partition.grid_shape(M, N, K, world)
            assert pr * pc == world
            cover = np.zeros((M, N), np.int8)
            for r in range(world):
                r0, r1, c0, c1 = partition.grid_block(M, N, K, world, r)
                cover[r0:r1, c0:c1] += 1
            assert (cover == 1).all()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, shape, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    M, K, N = shape
    rng = np.random.default_rng(0)
    A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    B = rng.uniform(-1, 1, (K, N)).astype(np.float32)

    def reduce_scatter(partial, r0, r1):
        t = torch.from_numpy(partial.copy())
        dist.all_reduce(t)  # gloo has no reduce_scatter; the row block is cut from the sum
        return t.numpy()[r0:r1]

    kind, span, local = partition.sharded_sgemm(A, B, rank, world, lambda a, b: a @ b, reduce_scatter)
    full = A @ B
    if kind == "grid":
        want = full[span[0]:span[1], span[2]:span[3]]
        lo, hi = span[0] * N + span[2], span[1] * N + span[3]  # only reported
    else:
        lo, hi = span
        want = full[lo:hi] if kind in ("rows", "k") else full[:, lo:hi]
    ok = local.shape == want.shape and np.allclose(local, want, atol=1e-3)
    gathered = [None] * world
    dist.all_gather_object(gathered, (kind, lo, hi, bool(ok)))
    if rank == 0:
        out.put(gathered)
    dist.destroy_process_group()


@pytest.mark.parametrize("shape", [(1024, 64, 96), (64, 96, 2048), (96, 4096, 64)])
def test_two_ranks_reassemble_the_product(shape):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, shape, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    kinds = {r[0] for r in res}
    assert len(kinds) == 1
    assert all(r[3] for r in res)
    assert res[0][1] == 0 and res[0][2] == res[1][1]


def test_four_ranks_on_a_grid():
    """2 x 2 grid: every rank's block equals the matching block of the full product, nothing exchanged."""
    shape = (2048, 32, 2048)
    assert partition.plan(shape[0], shape[2], shape[1], 4) == "grid"
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 4, port, shape, out)) for r in range(4)]
    for p in procs:
        p.start()
    res = out.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert {r[0] for r in res} == {"grid"}
    assert all(r[3] for r in res)
