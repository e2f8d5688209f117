"""Splitting one product over the GPUs of a box, one process per GPU.

Rows of C are independent, so rank g computes C[r0:r1, :] = A[r0:r1, :] @ B with
B replicated and nothing exchanged: the reference's K-first schedule hands each
core its own m_c-row slab of a CB block in the same way
(reference src/cake_sgemm_k_first.cpp:85-129); here the "cores" are GPUs.  The
N-first shape (few rows, very wide) splits columns of B and C instead.  Only a
product that is small in both M and N but very deep is split along K, and that
is the one case with an exchange: the partial products are summed with a
reduce-scatter over row blocks.

With four or more GPUs and a product that is large in both M and N the ranks
form a pr x pc grid: rank (i, j) owns rows block i of A and columns block j of
B.  Still nothing is exchanged, and every rank prepares (splits into TF32
planes) only 1/pr of A and 1/pc of B instead of 1/world of A and all of B,
which is what limits a pure row split at 8 GPUs.
"""

TILE_M = 128  # rows of one tensor-core tile; blocks are whole tiles except the last


def row_block(M, world, rank):
    """[r0, r1) of the rows owned by `rank`: whole 128-row tiles, balanced to within one tile."""
    tiles = (M + TILE_M - 1) // TILE_M
    lo = (tiles * rank) // world * TILE_M
    hi = (tiles * (rank + 1)) // world * TILE_M
    return min(lo, M), (M if rank == world - 1 else min(hi, M))


def col_block(N, world, rank, tile=256):
    tiles = (N + tile - 1) // tile
    lo = (tiles * rank) // world * tile
    hi = (tiles * (rank + 1)) // world * tile
    return min(lo, N), (N if rank == world - 1 else min(hi, N))


def k_block(K, world, rank, tile=32):
    tiles = (K + tile - 1) // tile
    lo = (tiles * rank) // world * tile
    hi = (tiles * (rank + 1)) // world * tile
    return min(lo, K), (K if rank == world - 1 else min(hi, K))


def unit_block(units, world, rank):
    """[lo, hi) of `units` independent items (products of a batch, images of a convolution) owned by
    `rank`, balanced to within one item."""
    return (units * rank) // world, (units * (rank + 1)) // world


def grid_shape(M, N, K, world):
    """(pr, pc), pr * pc == world: the process grid with the least time per rank.

    The model is the measured one of the library on a B200: the operand-split
    pass moves 12 bytes per operand element at about 5.4 TB/s and the contraction
    runs 128 x 256 tiles at about 250 TFLOP/s.  Ties go to the taller grid (more
    row blocks), so two GPUs split rows."""
    best, best_t = (world, 1), None
    for pr in range(world, 0, -1):
        if world % pr:
            continue
        pc = world // pr
        rows, cols = -(-M // pr), -(-N // pc)
        tiles = -(-rows // TILE_M) * -(-cols // 256)
        t = 12.0 * K * (rows + cols) / 5.4e12 + 2.0 * tiles * TILE_M * 256 * K / 250e12
        if best_t is None or t < best_t * 0.999:
            best, best_t = (pr, pc), t
    return best


def grid_block(M, N, K, world, rank):
    """(r0, r1, c0, c1) of rank's block of C on the grid_shape grid; ranks run along a grid row first."""
    pr, pc = grid_shape(M, N, K, world)
    i, j = divmod(rank, pc)
    return row_block(M, pr, i) + col_block(N, pc, j)


def plan(M, N, K, world):
    """'rows' | 'cols' | 'grid' | 'k' : how to split the product for `world` GPUs."""
    kind = _plan_1d(M, N, K, world)
    if kind != "k" and world > 1:
        pr, pc = grid_shape(M, N, K, world)
        if pr > 1 and pc > 1:
            return "grid"
        if kind == "rows" and pr == 1 and N >= world * 256:
            return "cols"
    return kind


def _plan_1d(M, N, K, world):
    if world <= 1:
        return "rows"
    tiles = ((M + TILE_M - 1) // TILE_M) * ((N + 255) // 256)
    # too few output tiles to occupy the box (a quarter of the 148 SMs per GPU) and a deep K
    if tiles < world * 37 and K >= world * 2048 and K >= 8 * max(M, N):
        return "k"
    if M >= N:
        return "rows" if M >= world * TILE_M or N < world * 256 else "cols"
    return "cols" if N >= world * 256 or M < world * TILE_M else "rows"


def sharded_sgemm(A, B, rank, world, sgemm, reduce_scatter=None):
    """Runs this rank's share.  `sgemm(a, b)` multiplies two local matrices;
    `reduce_scatter(partial, r0, r1)` (needed for the K split only) returns the
    sum over ranks of rows [r0, r1) of the partial products.  Returns
    (kind, span, local_result) with span = (lo, hi), or (r0, r1, c0, c1) for a grid."""
    M, K = A.shape
    N = B.shape[1]
    kind = plan(M, N, K, world)
    if kind == "rows":
        r0, r1 = row_block(M, world, rank)
        return kind, (r0, r1), sgemm(A[r0:r1], B)
    if kind == "cols":
        c0, c1 = col_block(N, world, rank)
        return kind, (c0, c1), sgemm(A, B[:, c0:c1])
    if kind == "grid":
        r0, r1, c0, c1 = grid_block(M, N, K, world, rank)
        return kind, (r0, r1, c0, c1), sgemm(A[r0:r1], B[:, c0:c1])
    k0, k1 = k_block(K, world, rank)
    partial = sgemm(A[:, k0:k1], B[k0:k1])
    r0, r1 = row_block(M, world, rank)
    if reduce_scatter is None:
        raise ValueError("a K split needs a reduce_scatter")
    return kind, (r0, r1), reduce_scatter(partial, r0, r1)
