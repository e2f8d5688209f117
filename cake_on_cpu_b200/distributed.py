"""One product over the GPUs of a box, one process per GPU (torch.distributed, NCCL).

The batched, sparse and convolution entry points shard by their independent units
(products of the batch, row blocks of the sparse operand, images): every rank
calls the library on its share and nothing is exchanged.

Rows (or columns) of C are independent, so each rank multiplies its block with
the library and nothing is exchanged.  Only the deep-K shape is different: K is
cut, every rank produces a full-size partial product, and the partials are
summed so that rank r ends up with its row block of C.  Where the library's
K-shard exchange takes the shape (few tiles, deep K: the case this split exists
for) the sum needs no collective: while a rank sums its tiles it stores the rows
straight into the owners' memory over NVLink and each owner adds the slots in
rank order (api.KShard).  Other shapes, and `exchange="nccl"`, use an NCCL
reduce-scatter.
The reference has no distributed layer; its K-first schedule splits a block of
rows over cores in the same way (reference src/cake_sgemm_k_first.cpp:85-129).
"""
import torch
import torch.distributed as dist

from . import api, partition


def _local(a, b, kernel):
    out = torch.empty((a.shape[0], b.shape[1]), dtype=torch.float32, device=a.device)
    return api.cake_sgemm(a.contiguous(), b.contiguous(), out, kernel=kernel)


_exchanges = {}


def _exchange(M, N, world, rank, group):
    """The K-shard exchange object of this shape, created and connected on first use (collective)."""
    key = (M, N, world, id(group))
    x = _exchanges.get(key)
    if x is None:
        x = api.KShard(world, rank, M, N)
        mine = torch.tensor(list(x.handle), dtype=torch.uint8, device="cuda")
        every = torch.empty(world * api.IPC_HANDLE_BYTES, dtype=torch.uint8, device="cuda")
        dist.all_gather_into_tensor(every, mine, group=group)
        x.connect(bytes(every.cpu().numpy().tobytes()))
        _exchanges[key] = x
    return x


def release(group=None):
    """Free the exchange buffers (collective: no rank may still be storing into another's)."""
    if dist.is_initialized() and _exchanges:
        torch.cuda.synchronize()
        dist.barrier(group)
    for x in _exchanges.values():
        x.close()
    _exchanges.clear()
    _gather_state.clear()


def sharded_sgemm(A, B, kernel=api.KERNEL_AUTO, group=None, exchange="auto"):
    """A (M x K) and B (K x N) are CUDA tensors present on every rank.  Returns
    (kind, span, block): kind 'rows' -> span (lo, hi), block = C[lo:hi, :]; 'cols' ->
    C[:, lo:hi]; 'grid' -> span (r0, r1, c0, c1), block = C[r0:r1, c0:c1]; 'k' ->
    C[lo:hi, :] after the partial products have been summed.  exchange: 'auto' (stores into
    the owners' memory where the library takes the shape, else NCCL), 'stores', 'nccl'."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    M, K = A.shape
    N = B.shape[1]

    def reduce_scatter(partial, r0, r1):
        if M % world == 0:
            out = torch.empty((M // world, N), dtype=torch.float32, device=partial.device)
            dist.reduce_scatter_tensor(out, partial, group=group)
            lo = rank * (M // world)
            return out, (lo, lo + M // world)
        dist.all_reduce(partial, group=group)  # ragged row blocks: sum everywhere, keep the own block
        return partial[r0:r1], (r0, r1)

    kind = partition.plan(M, N, K, world)
    if kind == "rows":
        r0, r1 = partition.row_block(M, world, rank)
        return kind, (r0, r1), _local(A[r0:r1], B, kernel)
    if kind == "cols":
        c0, c1 = partition.col_block(N, world, rank)
        return kind, (c0, c1), _local(A, B[:, c0:c1], kernel)
    if kind == "grid":
        r0, r1, c0, c1 = partition.grid_block(M, N, K, world, rank)
        # the column block of B is read where it lies (leading dimension N), no copy
        return kind, (r0, r1, c0, c1), api.cake_sgemm_ex(A[r0:r1], B[:, c0:c1], kernel=kernel)
    k0, k1 = partition.k_block(K, world, rank)
    if exchange not in ("auto", "stores", "nccl"):
        raise ValueError("exchange must be 'auto', 'stores' or 'nccl'")
    if exchange != "nccl" and world > 1 and kernel != api.KERNEL_FFMA:
        # every rank evaluates every rank's share, so all of them take the same route
        shares = [partition.k_block(K, world, r) for r in range(world)]
        if all(api.kshard_supported(M, N, b - a) for a, b in shares):
            x = _exchange(M, N, world, rank, group)
            x.partial(A[:, k0:k1], B[k0:k1])  # column range of A read where it lies (leading dimension K)
            return kind, x.rows, x.finish()
        if exchange == "stores":
            raise ValueError("the K-shard exchange does not take this shape")
    partial = _local(A[:, k0:k1], B[k0:k1], kernel)
    r0, r1 = partition.row_block(M, world, rank)
    block, span = reduce_scatter(partial, r0, r1)
    return kind, span, block


def bind_near_gpu(device_index):
    """Keep this process's host threads, and with them the pinned buffers it allocates from now on,
    on the CPUs next to GPU `device_index` (the affinity NVML reports for it), so that host-to-device
    copies do not cross the socket interconnect.  Reads settings only; returns the CPU set chosen, or
    None when NVML or the affinity call is not available or the set would be empty."""
    import os
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        near = {64 * w + b for w, word in enumerate(words) for b in range(64) if (int(word) >> b) & 1}
        allowed = os.sched_getaffinity(0)
        pick = near & allowed
        if not pick:
            return None
        os.sched_setaffinity(0, pick)
        return sorted(pick)
    except Exception:
        return None


_gather_state = {}


def sharded_sgemm_host(A_rows, B_rows, C_rows, kernel=api.KERNEL_AUTO, group=None):
    """One product C = A @ B whose operands live in HOST memory, spread over the ranks by rows.

    Rank r passes the rows of A and of C that it owns (``partition.row_block(M, world, r)``)
    and ITS slice of the rows of B (``partition.k_block(K, world, r)``), as float32 numpy
    arrays (pinned memory makes the copies asynchronous).  Every rank needs all of B, but each
    row of B crosses PCIe once: a rank copies only its slice to the device and the slices are
    gathered from the peers over NVLink into a B in the rank's own memory (NCCL all-gather on a
    side stream), which the kernels then read locally.  While that gather runs, the rank's rows
    of A are already arriving; the product is multiplied band by band as they land and the
    result rows leave band by band (cakeb200_sgemm_after).  Per step and rank the host link
    carries 4 * (rows * K + (K / world) * N) bytes in and 4 * rows * N bytes out; with B copied by
    every rank it would carry 4 * (rows * K + K * N) bytes in.

    The reference shares one packed B among all cores of a CB block in the same way
    (reference src/cake_sgemm_k_first.cpp:85-129).  Returns C_rows.
    """
    import numpy as np
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    rows, K = A_rows.shape
    N = B_rows.shape[1]
    k0, k1 = partition.k_block(K, world, rank)
    if B_rows.shape[0] != k1 - k0:
        raise ValueError("this rank's slice of B must have %d rows (partition.k_block), got %d" % (k1 - k0, B_rows.shape[0]))
    if tuple(C_rows.shape) != (rows, N):
        raise ValueError("C_rows has the wrong shape")
    if world == 1:
        return api.cake_sgemm(A_rows, B_rows, C_rows, kernel=kernel)
    key = (K, N, world, id(group))
    st = _gather_state.get(key)
    if st is None:
        st = {"B": torch.empty((K, N), dtype=torch.float32, device="cuda"), "side": torch.cuda.Stream(),
              "slice_in": torch.cuda.Event(), "ready": torch.cuda.Event()}
        _gather_state[key] = st
    Bd, side = st["B"], st["side"]
    main = torch.cuda.current_stream()
    Bd[k0:k1].copy_(torch.from_numpy(B_rows) if isinstance(B_rows, np.ndarray) else B_rows, non_blocking=True)
    st["slice_in"].record(main)
    shares = [partition.k_block(K, world, r) for r in range(world)]
    with torch.cuda.stream(side):
        side.wait_event(st["slice_in"])
        if all(b - a == k1 - k0 for a, b in shares):
            dist.all_gather_into_tensor(Bd, Bd[k0:k1], group=group)  # in place: this rank's slice already sits where it belongs
        else:
            for r, (a, b) in enumerate(shares):  # ragged slices: one broadcast per owner
                if b > a:
                    dist.broadcast(Bd[a:b], src=dist.get_global_rank(group, r) if group is not None else r, group=group)
        st["ready"].record(side)
    if rows > 0:
        api.cake_sgemm(A_rows, Bd, C_rows, kernel=kernel, stream=main.cuda_stream, b_ready=st["ready"])
    else:
        st["ready"].synchronize()
    return C_rows


def _rank_world(group):
    if dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


def sharded_sgemm_batched(A, B, kernel=api.KERNEL_AUTO, group=None):
    """A (batch x M x K), B (batch x K x N) present on every rank.  Returns ((lo, hi), C[lo:hi])."""
    rank, world = _rank_world(group)
    lo, hi = partition.unit_block(A.shape[0], world, rank)
    if hi == lo:
        return (lo, hi), torch.empty((0, A.shape[1], B.shape[2]), dtype=torch.float32, device=A.device)
    return (lo, hi), api.cake_sgemm_batched(A[lo:hi].contiguous(), B[lo:hi].contiguous(), kernel=kernel)


def sharded_sp_sgemm(A, B, kernel=api.KERNEL_AUTO, group=None):
    """Sparse A (M x K) and dense B present on every rank: row blocks of A.  Returns ((r0, r1), C[r0:r1])."""
    rank, world = _rank_world(group)
    r0, r1 = partition.row_block(A.shape[0], world, rank)
    if r1 == r0:
        return (r0, r1), torch.empty((0, B.shape[1]), dtype=torch.float32, device=A.device)
    return (r0, r1), api.cake_sp_sgemm(A[r0:r1].contiguous(), B.contiguous(), kernel=kernel)


def sharded_conv2d(x, w, stride=1, pad=0, kernel=api.KERNEL_AUTO, group=None):
    """Input x (batch x Cin x H x W) and filters present on every rank: images.  Returns ((lo, hi), out[lo:hi])."""
    rank, world = _rank_world(group)
    lo, hi = partition.unit_block(x.shape[0], world, rank)
    if hi == lo:
        return (lo, hi), None
    return (lo, hi), api.cake_conv2d(x[lo:hi].contiguous(), w.contiguous(), stride, pad, kernel=kernel)
