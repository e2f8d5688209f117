"""Pins the CPU oracle to the unmodified reference, live, wherever the
reference library could be built (oracle/_ref/).  Everything is compared
bit for bit on the reference's own grid of awkward sizes
(src/util.cpp:12-13: 1, 10, 96, 111, 960, 2111)."""
import numpy as np
import pytest

from _oracle import KMN, MKN, NKM, NA

DIMS = (1, 10, 96, 111)
CASES = [(M, K, N) for M in DIMS for K in DIMS for N in DIMS]
CASES += [(960, 111, 96), (96, 960, 111), (111, 96, 960), (2111, 96, 111), (300, 2111, 50), (37, 53, 2111),
          (960, 960, 960)]


@pytest.mark.parametrize("p", [2, 3, 8])
def test_sgemm_blockdims_and_packers_bit_exact(oracle, reference, p):
    rng = np.random.default_rng(p)
    for (M, K, N) in CASES:
        A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
        B = rng.uniform(-1, 1, (K, N)).astype(np.float32)
        for sch in (KMN, MKN, NKM, NA):
            bo, br = oracle.block_dims(M, N, K, p, sch), reference.block_dims(M, N, K, p, sch)
            assert bo == br, (M, K, N, p, sch)
            Co, ran = oracle.sgemm(A, B, p, sch)
            Cr, _ = reference.sgemm(A, B, p, sch)
            assert np.array_equal(Co, Cr), (M, K, N, p, sch)
            assert ran == bo["sch"]
            assert oracle.packed_sizes(M, N, K, p, sch) == reference.packed_sizes(M, N, K, p, sch)
            # pack_A: every position, padding included
            assert np.array_equal(oracle.pack(0, A, M, N, K, p, sch), reference.pack(0, A, M, N, K, p, sch))
            # pack_B: the reference's M-/N-first packers copy whatever follows a row into the pad
            # columns instead of zero (src/pack_ob.cpp:126-138); compare the positions that hold data
            po, pr = oracle.pack(1, B, M, N, K, p, sch), reference.pack(1, B, M, N, K, p, sch)
            if bo["sch"] != KMN:
                keep = oracle.pack(1, np.ones_like(B), M, N, K, p, sch) != 0
                po, pr = po[keep], pr[keep]
            assert np.array_equal(po, pr), (M, K, N, p, sch)
            # pack_C / unpack_C: the reference's N-first pack_C is only defined for aligned shapes
            aligned = M % (p * bo["m_c"]) == 0 and N % bo["n_c"] == 0
            if bo["sch"] != NKM or aligned:
                Pc = reference.pack(2, Cr, M, N, K, p, sch)
                assert np.array_equal(oracle.pack(2, Cr, M, N, K, p, sch), Pc)
                assert np.array_equal(oracle.pack(3, Pc, M, N, K, p, sch), Cr)
                assert np.array_equal(reference.pack(3, Pc, M, N, K, p, sch), Cr)


def test_beta_flag_semantics(oracle, reference):
    rng = np.random.default_rng(7)
    M, K, N, p = 111, 96, 211, 4
    A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    B = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    C0 = rng.uniform(-1, 1, (M, N)).astype(np.float32)
    for sch in (KMN, MKN):
        Co, _ = oracle.sgemm(A, B, p, sch, beta=1.0, C=C0)
        Cr, _ = reference.sgemm(A, B, p, sch, beta=1.0, C=C0)
        assert np.array_equal(Co, Cr)
    plain, _ = reference.sgemm(A, B, p, KMN)
    kept, _ = reference.sgemm(A, B, p, KMN, beta=1.0, C=C0)
    assert np.array_equal(plain, kept)  # K-first ignores beta and overwrites


def test_user_block_sizes_and_other_drivers(oracle, reference):
    rng = np.random.default_rng(9)
    M, K, N, p = 300, 200, 260, 4
    A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    B = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    for sch in (KMN, MKN, NKM):
        Co, _ = oracle.sgemm(A, B, p, sch, blk=(24, 40, 64))
        Cr, _ = reference.sgemm(A, B, p, sch, blk=(24, 40, 64))
        assert np.array_equal(Co, Cr)
    # the online-packing and 2-D drivers of the reference agree with the float64 product
    ref64 = A.astype(np.float64) @ B.astype(np.float64)
    for variant in (1, 2):
        Cv, _ = reference.sgemm(A, B, p, KMN, variant=variant)
        assert np.abs(Cv - ref64).max() < 1e-3
    assert reference.checker(A, B, Cr) == 0


def test_rectangular_benchmark_shapes_scaled_down(oracle, reference):
    # 1/16-scale versions of the M-first / N-first / K-first benchmark shapes
    for (M, K, N) in [(4096, 64, 64), (64, 64, 4096), (64, 16384, 64)]:
        A, B = oracle.uniform((M, K), 1), oracle.uniform((K, N), 2)
        Co, so = oracle.sgemm(A, B, 8, NA)
        Cr, _ = reference.sgemm(A, B, 8, NA)
        assert np.array_equal(Co, Cr)


def test_sparse_restatement_equals_the_reference_microkernel(oracle, reference):
    """oracle_sp_sgemm against the reference's own sparse microkernel (cake_sp_sgemm_haswell_6x16, the one sparse
    routine the reference ships), driven tile by tile over whole matrices: bit for bit, at densities from empty to
    dense, with ragged M (not a multiple of 6), N (not a multiple of 16) and K (not a multiple of 4)."""
    if not reference.sparse_available():
        pytest.skip("oracle/_ref/libcake_ref_sparse.so not built")
    for (M, K, N, d) in [(6, 4, 16, 0.5), (37, 53, 29, 0.1), (100, 257, 130, 0.02), (13, 7, 5, 1.0), (64, 96, 48, 0.0),
                         (111, 300, 211, 0.3), (7, 1, 17, 0.9), (96, 1030, 64, 0.01)]:
        A = oracle.sparse((M, K), 1, 3, d) if d < 1.0 else oracle.uniform((M, K), 1)
        B = oracle.uniform((K, N), 2)
        assert np.array_equal(oracle.sp_sgemm(A, B), reference.sp_sgemm(A, B)), (M, K, N, d)


def test_matrix_vector_restatement_equals_the_reference_microkernel(oracle, reference):
    """oracle_sgemv against the microkernel of the reference's matrix-vector example (cake_sgemv_haswell_8x8_col),
    bit for bit: ragged M (not a multiple of 8), K not a multiple of the kernel's unrolling, y added to."""
    if not reference.gemv_available():
        pytest.skip("oracle/_ref/libcake_ref_gemv.so not built")
    for (M, K) in [(8, 8), (1, 1), (37, 53), (1000, 700), (96, 2111), (13, 9), (300, 4)]:
        A = oracle.uniform((K, M), 1)
        x = oracle.uniform((K,), 2)
        y0 = oracle.uniform((M,), 3)
        assert np.array_equal(oracle.sgemv(A, x, y0), reference.sgemv(A, x, y0)), (M, K)
        assert np.array_equal(oracle.sgemv(A, x), reference.sgemv(A, x)), (M, K)


def test_im2col_restatement_equals_the_reference(oracle, reference):
    """oracle_im2col against im_2_col of the reference's convolution example, for what the reference covers
    (one image, no padding, stride 1); batch and padding are this build's extensions and are checked against
    float64 convolutions elsewhere."""
    if not reference.im2col_available():
        pytest.skip("oracle/_ref/libcake_ref_im2col.so not built")
    for (cin, H, W, hf, wf) in [(3, 7, 6, 3, 3), (8, 33, 33, 3, 3), (5, 9, 12, 1, 1), (2, 10, 8, 5, 3), (16, 14, 14, 3, 3)]:
        x = oracle.normal((1, cin, H, W), 4, 0.1)
        assert np.array_equal(oracle.im2col(x, hf, wf, 1, 0), reference.im2col(x[0], hf, wf)), (cin, H, W, hf, wf)
