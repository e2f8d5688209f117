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
    for name in ("pair", "chunk_kb", "k_pieces", "tile_n"):
        cake.set_option(name, 0)


def _product(cake, A, B, pair, chunk_kb=UNBROKEN, k_pieces=1, tile_n=0, **kw):
    cake.set_option("pair", pair)
    cake.set_option("chunk_kb", chunk_kb)
    cake.set_option("k_pieces", k_pieces)  # 1: whole tiles only, so that both forms add in the same order
    cake.set_option("tile_n", tile_n)
    C = np.full((A.shape[0], B.shape[1]), np.nan, np.float32)
    cake.cake_sgemm(A, B, C, kernel=cake.KERNEL_TF32X3)
    return C


SHAPES = [(256, 64, 256), (512, 512, 512), (1000, 700, 900), (257, 33, 1030), (2111, 960, 2111), (129, 100, 64)]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("chunk_kb", [UNBROKEN, 8])
@pytest.mark.parametrize("tile_n", [0, 128])
def test_pair_kernel_matches_single_sm_kernel_and_oracle(pair_options, oracle, shape, chunk_kb, tile_n):
    cake = pair_options
    M, K, N = shape
    A, B = oracle.uniform((M, K), 1), oracle.uniform((K, N), 2)
    ref, _ = oracle.sgemm(A, B, 8, KMN)
    pair = _product(cake, A, B, 1, chunk_kb, 1, tile_n)
    assert cake.last_stats()["tile_m"] == 256
    single = _product(cake, A, B, 2, chunk_kb, 1, tile_n)
    assert cake.last_stats()["tile_m"] == 128
    assert rel_err(pair, ref, A, B) <= TOL
    assert np.array_equal(pair, single)


@pytest.mark.parametrize("shape", [(2111, 960, 2111), (1024, 4100, 1024), (3000, 3000, 3000), (640, 2048, 5000)])
def test_pair_kernel_with_tiles_cut_along_k(pair_options, oracle, shape):
    """The ragged last wave is cut into K pieces whose partial tiles (two 128-row halves per pair) are summed
    by the reduction kernel; chunk length by the rule."""
    cake = pair_options
    M, K, N = shape
    A, B = oracle.uniform((M, K), 5), oracle.uniform((K, N), 6)
    exact = A.astype(np.float64) @ B.astype(np.float64)
    for pair in (1, 2):
        C = _product(cake, A, B, pair, 0, 0)
        assert rel_err(C, exact, A, B) <= TOL, (pair, shape)


def test_pair_kernel_with_an_empty_k_piece(pair_options):
    """Sixteen slices of K cut into five pieces of four leave the last piece empty: it still hands an accumulator
    over (zeros), in both CTAs of the pair."""
    import torch
    cake = pair_options
    M, K, N = 512, 512, 512
    g = torch.Generator(device="cuda").manual_seed(9)
    A = torch.rand((M, K), device="cuda", generator=g) * 2 - 1
    B = torch.rand((K, N), device="cuda", generator=g) * 2 - 1
    exact = A.double() @ B.double()
    den = A.double().norm(dim=1)[:, None] * B.double().norm(dim=0)[None, :]
    for pair in (1, 2):
        for tile_n in (128, 256):
            for name, v in (("pair", pair), ("chunk_kb", UNBROKEN), ("k_pieces", 5), ("tile_n", tile_n)):
                cake.set_option(name, v)
            C = torch.full((M, N), float("nan"), device="cuda")
            cake.cake_sgemm(A, B, C, kernel=cake.KERNEL_TF32X3)
            assert cake.last_stats()["launches"] == 4  # two splits, the product, the sum of the pieces
            assert ((C.double() - exact).abs() / den).max().item() <= TOL, (pair, tile_n)


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
        cake.set_option("k_pieces", 1)
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
        cake.set_option("k_pieces", 1)  # whole tiles in both forms: the same order of additions
        C = torch.empty((n, n), device="cuda")
        cake.cake_sgemm(A, B, C, kernel=cake.KERNEL_TF32X3)
        out[pair] = C
    assert torch.equal(out[1], out[2])
    rows = torch.as_tensor(np.random.default_rng(0).integers(0, n, 48), device="cuda")
    exact = A[rows].double() @ B.double()
    den = A[rows].double().norm(dim=1)[:, None] * B.double().norm(dim=0)[None, :]
    assert ((out[1][rows].double() - exact).abs() / den).max().item() <= TOL


def test_pair_kernel_stores_a_convolution_output(pair_options, oracle):
    """The im2col route of the convolution multiplies filters (rows = output channels) by the patch matrix and
    stores straight to NCHW from the epilogue; forced onto pairs of SMs it must agree with the implicit kernel."""
    cake = pair_options
    x, w = oracle.normal((3, 40, 12, 12), 4, 0.1), oracle.normal((300, 40, 3, 3), 5, 0.1)
    implicit = cake.cake_conv2d(x, w, 1, 1, kernel=cake.KERNEL_TF32X3)
    cake.set_option("conv_route", 1)
    cake.set_option("pair", 1)
    try:
        paired = cake.cake_conv2d(x, w, 1, 1, kernel=cake.KERNEL_TF32X3)
        cake.set_option("pair", 2)
        single = cake.cake_conv2d(x, w, 1, 1, kernel=cake.KERNEL_TF32X3)
    finally:
        cake.set_option("conv_route", 0)
    col = oracle.im2col(x, 3, 3, 1, 1)
    flat = lambda t: t.transpose(1, 0, 2, 3).reshape(300, -1)
    assert rel_err(flat(paired), flat(implicit), w.reshape(300, -1), col) <= TOL
    assert rel_err(flat(paired), flat(single), w.reshape(300, -1), col) <= TOL

