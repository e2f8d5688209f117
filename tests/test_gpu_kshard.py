"""The K-sharded product's exchange on ONE GPU: the ranks are objects of one process wired to each
other's buffers, every rank's first half (multiply its range of K, store the rows into the owners'
slots) runs before any rank's second half (wait for the flags, add the slots), so nothing ever waits
for a kernel that has not run.  The real thing, one process per GPU with the buffers mapped across
processes, is covered by test_multi_gpu.py where two GPUs are present."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
TOL = 1e-5


def _operands(M, K, N, seed):
    import torch
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.rand((M, K), device="cuda", generator=g) * 2 - 1, torch.rand((K, N), device="cuda", generator=g) * 2 - 1


def _norm_err(C, A, B, lo, hi):
    exact = A[lo:hi].double() @ B.double()
    den = A[lo:hi].double().norm(dim=1)[:, None] * B.double().norm(dim=0)[None, :]
    return ((C.double() - exact).abs() / den.clamp_min(1e-30)).max().item()


@pytest.mark.parametrize("world,M,K,N", [(1, 256, 4096, 256), (2, 512, 16384, 256), (4, 640, 32768, 256),
                                         (8, 1024, 32768, 1024), (2, 300, 20000, 130), (3, 129, 9000, 77)])
def test_emulated_ranks_sum_to_the_product(cake, world, M, K, N):
    import torch
    from cake_on_cpu_b200 import api, partition
    A, B = _operands(M, K, N, 21)
    ranks = [api.KShard(world, r, M, N) for r in range(world)]
    try:
        api.KShard.connect_local(ranks)
        for rep in range(3):  # three products: both buffer sets and their reuse
            if rep:
                A = A.roll(1, 0)
            for r, x in enumerate(ranks):
                k0, k1 = partition.k_block(K, world, r)
                assert api.kshard_supported(M, N, k1 - k0)
                x.partial(A[:, k0:k1], B[k0:k1])
            covered = 0
            for r, x in enumerate(ranks):
                lo, hi = x.rows
                assert (lo, hi) == partition.row_block(M, world, r)
                out = torch.full((hi - lo, N), float("nan"), device="cuda")
                x.finish(out)
                covered += hi - lo
                if hi > lo:
                    assert _norm_err(out, A, B, lo, hi) <= TOL, (world, r, rep)
            assert covered == M
    finally:
        for x in ranks:
            x.close()


def test_the_sum_is_in_rank_order_and_repeatable(cake):
    import torch
    from cake_on_cpu_b200 import api, partition
    world, M, K, N = 4, 512, 16384, 512
    A, B = _operands(M, K, N, 22)
    ranks = [api.KShard(world, r, M, N) for r in range(world)]
    try:
        api.KShard.connect_local(ranks)
        runs = []
        for order in (range(world), reversed(range(world))):  # the order in which the ranks store must not matter
            for r in order:
                k0, k1 = partition.k_block(K, world, r)
                ranks[r].partial(A[:, k0:k1], B[k0:k1])
            runs.append(torch.cat([x.finish() for x in ranks]))
        assert torch.equal(runs[0], runs[1])
        # the same partial products added in rank order by hand
        parts = [api.cake_sgemm(A[:, a:b].contiguous(), B[a:b].contiguous(), kernel=api.KERNEL_TF32X3)
                 for a, b in (partition.k_block(K, world, r) for r in range(world))]
        by_hand = parts[0].clone()
        for p in parts[1:]:
            by_hand += p
        assert torch.equal(runs[0], by_hand)
    finally:
        for x in ranks:
            x.close()


def test_a_missing_rank_is_reported_and_the_product_can_still_finish(cake):
    import torch
    from cake_on_cpu_b200 import api, partition
    world, M, K, N = 2, 256, 8192, 256
    A, B = _operands(M, K, N, 23)
    ranks = [api.KShard(world, r, M, N) for r in range(world)]
    try:
        api.KShard.connect_local(ranks)
        k0, k1 = partition.k_block(K, world, 0)
        ranks[0].partial(A[:, k0:k1], B[k0:k1])
        with pytest.raises(api.CakeError) as e:  # rank 1 has stored nothing: rank 0's wait runs out after 3 ms
            ranks[0].finish(wait_limit_us=3000)
        assert e.value.code == -4 and "where 910" in str(e.value) and "info 1" in str(e.value), str(e.value)
        # the context is intact and the late rank can still arrive
        k0, k1 = partition.k_block(K, world, 1)
        ranks[1].partial(A[:, k0:k1], B[k0:k1])
        for x in ranks:
            lo, hi = x.rows
            assert _norm_err(x.finish(), A, B, lo, hi) <= TOL
    finally:
        for x in ranks:
            x.close()


def test_shapes_the_exchange_does_not_take(cake):
    from cake_on_cpu_b200 import api
    assert not api.kshard_supported(8192, 8192, 1024)  # plenty of tiles: rows are split instead
    assert not api.kshard_supported(256, 256, 256)  # too shallow to cut
    x = api.KShard(1, 0, 8192, 8192)
    try:
        import torch
        A = torch.zeros((8192, 1024), device="cuda")
        B = torch.zeros((1024, 8192), device="cuda")
        with pytest.raises(api.CakeError):
            x.partial(A, B)
    finally:
        x.close()


def test_partial_and_finish_must_alternate(cake):
    """Misuse is refused on the host, before any launch: a second partial before the finish of the first (its
    slot set may still be read by an owner), a finish with nothing in flight, and a new partial after a finish
    that gave up waiting."""
    import torch
    from cake_on_cpu_b200 import api, partition
    world, M, K, N = 2, 256, 8192, 256
    A, B = _operands(M, K, N, 24)
    ranks = [api.KShard(world, r, M, N) for r in range(world)]
    try:
        api.KShard.connect_local(ranks)
        with pytest.raises(api.CakeError) as e:
            ranks[0].finish()
        assert e.value.code == -1
        k0, k1 = partition.k_block(K, world, 0)
        ranks[0].partial(A[:, k0:k1], B[k0:k1])
        with pytest.raises(api.CakeError) as e:
            ranks[0].partial(A[:, k0:k1], B[k0:k1])
        assert e.value.code == -1 and "finish" in str(e.value)
        with pytest.raises(api.CakeError) as e:  # rank 1 has not stored: the wait gives up after 2 ms
            ranks[0].finish(wait_limit_us=2000)
        assert e.value.code == -4
        with pytest.raises(api.CakeError) as e:  # still open: no new product
            ranks[0].partial(A[:, k0:k1], B[k0:k1])
        assert e.value.code == -1
        k0, k1 = partition.k_block(K, world, 1)
        ranks[1].partial(A[:, k0:k1], B[k0:k1])
        for x in ranks:
            lo, hi = x.rows
            assert _norm_err(x.finish(), A, B, lo, hi) <= TOL
        # and the next product runs as usual
        for r, x in enumerate(ranks):
            k0, k1 = partition.k_block(K, world, r)
            x.partial(A[:, k0:k1], B[k0:k1])
        for x in ranks:
            lo, hi = x.rows
            assert _norm_err(x.finish(), A, B, lo, hi) <= TOL
    finally:
        for x in ranks:
            x.close()
