"""The large-matrix kernel that runs one 256 x 256 tile on a pair of SMs (tcgen05 cta_group::2) against the
single-SM kernel and the oracle.  Both kernels issue the same three MMAs per 8 of K in the same order into
tensor memory, so their results are expected to be equal bit for bit; the oracle gate is the usual
max |C - C_ref| / (||A[m,:]|| ||B[:,n]||) <= 1e-5."""
import numpy as np
import pytest

from _oracle import KMN, MKN, NKM, rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-5
UNBROKEN = 1 << 20  # chunk length (slices of 32 of K) longer than any K here: one unbroken accumulation


@pytest.fixture
def pair_options(cake):
    yield cake
    cake.set_option("pair", 0)
    cake.set_option("chunk_kb", 0)


def _product(cake, A, B, pair, **kw):
    cake.set_option("pair", pair)
    cake.set_option("chunk_kb", UNBROKEN)
    C = np.full((A.shape[0], B.shape[1]), np.nan, np.float32)
    cake.cake_sgemm_ex(A, B, C, kernel=cake.KERNEL_TF32X3, **kw) if kw else cake.cake_sgemm(A, B, C, kernel=cake.KERNEL_TF32X3)
    return C


@pytest.mark.parametrize("shape", [(256, 64, 256), (512, 512, 512), (1000, 700, 900), (257, 33, 1030), (2111, 960, 2111)])
def test_pair_kernel_matches_single_sm_kernel_and_oracle(pair_options, oracle, shape):
    cake = pair_options
    M, K, N = shape
    A, B = oracle.uniform((M, K), 1), oracle.uniform((K, N), 2)
    ref, _ = oracle.sgemm(A, B, 8, KMN)
    pair = _product(cake, A, B, 1)
    single = _product(cake, A, B, 2)
    assert rel_err(pair, ref, A, B) <= TOL
    assert np.array_equal(pair, single)


@pytest.mark.parametrize("sch", [KMN, MKN, NKM])
def test_pair_kernel_every_schedule(pair_options, oracle, sch):
    cake = pair_options
    M, K, N = 1536, 320, 2304
    A, B = oracle.uniform((M, K), 3), oracle.uniform((K, N), 4)
    ref, _ = oracle.sgemm(A, B, 8, sch)
    cake.set_option("pair", 1)
    cake.set_option("chunk_kb", UNBROKEN)
    C = np.full((M, N), np.nan, np.float32)
    cake.cake_sgemm(A, B, C, p=8, sch=sch, kernel=cake.KERNEL_TF32X3)
    assert rel_err(C, ref, A, B) <= TOL


def test_pair_kernel_bias_and_accumulate(pair_options):
    import torch
    cake = pair_options
    M, K, N = 777, 515, 1030
    g = torch.Generator(device="cuda").manual_seed(5)
    A = torch.rand((M, K), device="cuda", generator=g) * 2 - 1
    B = torch.rand((K, N), device="cuda", generator=g) * 2 - 1
    bias = torch.rand((N,), device="cuda", generator=g)
    out = {}
    for pair in (1, 2):
        cake.set_option("pair", pair)
        cake.set_option("chunk_kb", UNBROKEN)
        C = torch.full((M, N), float("nan"), device="cuda")
        cake.cake_sgemm_ex(A, B, C, bias=bias, kernel=cake.KERNEL_TF32X3)
        cake.cake_sgemm_ex(A, B, C, accumulate=True, kernel=cake.KERNEL_TF32X3)
        out[pair] = C
    assert torch.equal(out[1], out[2])
    exact = 2 * (A.double() @ B.double()) + bias.double()[None, :]
    den = A.double().norm(dim=1)[:, None] * B.double().norm(dim=0)[None, :]
    assert ((out[1].double() - exact).abs() / den).max().item() <= 2 * TOL


def test_pair_kernel_full_size(pair_options):
    """8192^3, the headline product: sampled rows against float64, and the same bits as the single-SM kernel."""
    import torch
    cake = pair_options
    n = 8192
    g = torch.Generator(device="cuda").manual_seed(6)
    A = torch.rand((n, n), device="cuda", generator=g) * 2 - 1
    B = torch.rand((n, n), device="cuda", generator=g) * 2 - 1
    out = {}
    for pair in (1, 2):
        cake.set_option("pair", pair)
        C = torch.empty((n, n), device="cuda")
        cake.cake_sgemm(A, B, C, kernel=cake.KERNEL_TF32X3)
        out[pair] = C
    assert torch.equal(out[1], out[2])
    rows = torch.as_tensor(np.random.default_rng(0).integers(0, n, 48), device="cuda")
    exact = A[rows].double() @ B.double()
    den = A[rows].double().norm(dim=1)[:, None] * B.double().norm(dim=0)[None, :]
    assert ((out[1][rows].double() - exact).abs() / den).max().item() <= TOL
