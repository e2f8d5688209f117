"""The CPU oracle against outputs of the unmodified reference (tests/golden/,
written by tests/golden/make_golden.py).  Bit-exact: the oracle keeps the
reference's floating-point operation order."""
import os

import numpy as np
import pytest

from _oracle import KMN, MKN, NKM, NA, BLK_FIELDS

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_golden.npz"))


def _cases(prefix):
    return sorted(k for k in GOLDEN.files if k.startswith(prefix + "_"))


@pytest.mark.parametrize("key", _cases("sgemm"))
def test_sgemm_bit_exact(oracle, key):
    M, K, N, p, sch = (int(v) for v in key.split("_")[1:])
    A, B = oracle.uniform((M, K), 1), oracle.uniform((K, N), 2)
    C, _ = oracle.sgemm(A, B, p, sch)
    assert np.array_equal(C, GOLDEN[key])


@pytest.mark.parametrize("key", _cases("packA") + _cases("packB") + _cases("packC"))
def test_pack_layout_exact(oracle, key):
    which = {"packA": 0, "packB": 1, "packC": 2}[key.split("_")[0]]
    M, K, N, p, sch = (int(v) for v in key.split("_")[1:])
    src = [oracle.uniform((M, K), 1), oracle.uniform((K, N), 2), oracle.uniform((M, N), 3)][which]
    got = oracle.pack(which, src, M, N, K, p, sch)
    assert np.array_equal(got, GOLDEN[key])


def test_unpack_inverts_pack(oracle):
    for key in _cases("packC"):
        M, K, N, p, sch = (int(v) for v in key.split("_")[1:])
        C = oracle.uniform((M, N), 3)
        assert np.array_equal(oracle.pack(3, GOLDEN[key], M, N, K, p, sch), C)


def test_block_dims(oracle):
    fields = [str(f) for f in GOLDEN["block_dims_fields"]]
    assert sorted(BLK_FIELDS) == fields
    for row in GOLDEN["block_dims"]:
        M, K, N, p, sch = (int(v) for v in row[:5])
        d = oracle.block_dims(M, N, K, p, sch)
        got = [d[f] for f in fields] + [int(round(d["alpha_n"] * 1e9))]
        assert got == [int(v) for v in row[5:]], (M, K, N, p, sch)


def test_set_schedule(oracle):
    for s, M, N, K, want in GOLDEN["set_schedule"]:
        assert oracle.set_schedule(int(s), int(M), int(N), int(K)) == int(want)


def test_benchmark_shapes_derive_expected_schedules(oracle):
    # schedules the reference derives on an 8-core host with these cache sizes for the benchmark shapes
    want = {(3000, 3000, 3000): MKN, (4096, 4096, 4096): KMN, (8192, 8192, 8192): KMN,
            (65536, 1024, 1024): MKN, (1024, 1024, 65536): NKM, (1024, 262144, 1024): KMN,
            (64, 576, 200704): KMN, (96, 96, 96): MKN}
    for (M, K, N), sch in want.items():
        assert oracle.block_dims(M, N, K, 8, NA)["sch"] == sch, (M, K, N)


@pytest.mark.parametrize("key", _cases("sparse"))
def test_sparse_bit_exact(oracle, key):
    """The row-skipping restatement against stored outputs of the reference's sparse microkernel."""
    M, K, N, d = (int(v) for v in key.split("_")[1:])
    A, B = oracle.sparse((M, K), 1, 3, d / 1000.0), oracle.uniform((K, N), 2)
    assert np.array_equal(oracle.sp_sgemm(A, B), GOLDEN[key])


@pytest.mark.parametrize("key", _cases("gemv"))
def test_matrix_vector_bit_exact(oracle, key):
    """The matrix-vector restatement against stored outputs of the reference example's microkernel."""
    M, K = (int(v) for v in key.split("_")[1:])
    got = oracle.sgemv(oracle.uniform((K, M), 1), oracle.uniform((K,), 2), oracle.uniform((M,), 3))
    assert np.array_equal(got, GOLDEN[key])


def test_sparse_restatement_equals_dense_chain(oracle):
    # zeros contribute no operation: skipping them leaves the FMA chain of the others unchanged
    A = oracle.sparse((37, 53), 1, 3, 0.1)
    B = oracle.uniform((53, 29), 2)
    C = oracle.sp_sgemm(A, B)
    ref = np.zeros((37, 29), np.float64)
    ref = A.astype(np.float64) @ B.astype(np.float64)
    assert np.abs(C - ref).max() < 1e-5
    assert (A == 0).mean() > 0.8


def test_conv_restatement_against_float64(oracle):
    x = oracle.normal((2, 3, 7, 6), 4, 0.1)
    w = oracle.normal((5, 3, 3, 3), 5, 0.1)
    out = oracle.conv2d(x, w, 1, 1, 4)
    ref = np.zeros(out.shape)
    xp = np.pad(x.astype(np.float64), ((0, 0), (0, 0), (1, 1), (1, 1)))
    for ho in range(7):
        for wo in range(6):
            ref[:, :, ho, wo] = np.einsum("bchw,ochw->bo", xp[:, :, ho:ho + 3, wo:wo + 3], w.astype(np.float64))
    assert np.abs(out - ref).max() < 1e-6
