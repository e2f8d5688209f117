"""Regenerates tests/golden/reference_golden.npz from the UNMODIFIED reference
(oracle/_ref/libcake_ref.so, built by `make -C oracle ref` where the reference
tree is available).  Inputs are not stored: they come from the oracle's seeded
generator (oracle_fill_uniform), so only the reference's outputs are kept.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from _oracle import KMN, MKN, NKM, NA, Oracle, Reference  # noqa: E402

# (M, K, N, p): the reference's own edge sizes (src/util.cpp:12-13: 1, 10, 96, 111, 960, 2111)
SGEMM_CASES = [(1, 1, 1, 2), (10, 10, 10, 3), (96, 96, 96, 4), (111, 96, 77, 4), (96, 111, 10, 8),
               (10, 2111, 96, 5), (2111, 10, 7, 8), (111, 960, 33, 2), (37, 300, 211, 8)]
PACK_CASES = [(111, 96, 77, 4), (10, 960, 20, 5), (960, 10, 7, 8)]
# (M, K, N, nonzeros per thousand) for the sparse microkernel
GEMV_CASES = [(37, 53), (1000, 700), (96, 2111), (13, 9)]
SPARSE_CASES = [(37, 53, 29, 100), (100, 257, 130, 20), (111, 300, 211, 300), (96, 1030, 64, 10), (64, 96, 48, 0)]
# block-dimension cases: edge sizes plus every shape of the benchmark configurations
BLOCK_CASES = [(m, k, n, p) for m in (1, 10, 96, 111, 960, 2111) for k in (1, 96, 2111) for n in (10, 111, 960)
               for p in (2, 8)]
BLOCK_CASES += [(3000, 3000, 3000, 8), (1024, 1024, 1024, 8), (2048, 2048, 2048, 8), (4096, 4096, 4096, 8),
                (8192, 8192, 8192, 8), (16384, 16384, 16384, 8), (32768, 32768, 32768, 8),
                (65536, 1024, 1024, 8), (1024, 1024, 65536, 8), (1024, 262144, 1024, 8), (96, 96, 96, 8),
                (64, 576, 200704, 8), (512, 2304, 12544, 8), (8192, 8192, 8192, 10), (3000, 3000, 3000, 10)]


def main():
    O, R = Oracle(), Reference()
    out = {}
    for (M, K, N, p) in SGEMM_CASES:
        A, B = O.uniform((M, K), 1), O.uniform((K, N), 2)
        for sch in (KMN, MKN, NKM, NA):
            C, _ = R.sgemm(A, B, p, sch)
            out["sgemm_%d_%d_%d_%d_%d" % (M, K, N, p, sch)] = C
    for (M, K, N, p) in PACK_CASES:
        A, B, C = O.uniform((M, K), 1), O.uniform((K, N), 2), O.uniform((M, N), 3)
        for sch in (KMN, MKN, NKM):
            out["packA_%d_%d_%d_%d_%d" % (M, K, N, p, sch)] = R.pack(0, A, M, N, K, p, sch)
            if sch == KMN:  # the reference leaves M/N-first pad columns of B unwritten-from-source
                out["packB_%d_%d_%d_%d_%d" % (M, K, N, p, sch)] = R.pack(1, B, M, N, K, p, sch)
            if sch != NKM:  # the reference's N-first pack_C overruns its buffer on ragged shapes
                out["packC_%d_%d_%d_%d_%d" % (M, K, N, p, sch)] = R.pack(2, C, M, N, K, p, sch)
    rows = []
    for (M, K, N, p) in BLOCK_CASES:
        for sch in (KMN, MKN, NKM, NA):
            d = R.block_dims(M, N, K, p, sch)
            rows.append([M, K, N, p, sch] + [d[k] for k in sorted(d) if k != "alpha_n"] + [int(round(d["alpha_n"] * 1e9))])
    out["block_dims"] = np.array(rows, dtype=np.int64)
    out["block_dims_fields"] = np.array(sorted(k for k in R.block_dims(10, 10, 10, 2, 0) if k != "alpha_n"))
    sets = [[s, M, N, K, R.set_schedule(s, M, N, K)] for s in (KMN, NA) for M in (1, 100, 1000) for N in (1, 100, 1000)
            for K in (1, 100, 1000)]
    out["set_schedule"] = np.array(sets, dtype=np.int64)
    # the reference's sparse microkernel, tile by tile (oracle/ref_sparse_driver.cpp): A = sparse stream (1, mask 3)
    for (M, K, N, d) in SPARSE_CASES:
        A, B = O.sparse((M, K), 1, 3, d / 1000.0), O.uniform((K, N), 2)
        out["sparse_%d_%d_%d_%d" % (M, K, N, d)] = R.sp_sgemm(A, B)
    # the matrix-vector microkernel of examples/cake_gemv.cpp (oracle/ref_gemv_driver.cpp): A (K, M) = stream 1
    for (M, K) in GEMV_CASES:
        out["gemv_%d_%d" % (M, K)] = R.sgemv(O.uniform((K, M), 1), O.uniform((K,), 2), O.uniform((M,), 3))
    # rand_init(srand(1)) head, examples/cake_conv.cpp:924 seeds this way
    out["rand_init_seed1"] = R.rand_init(1, 4, 8)
    path = os.path.join(HERE, "reference_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
