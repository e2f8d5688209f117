"""The benchmark configurations at their full sizes.  The CPU oracle would need
minutes to hours for these, so each result is checked through properties that do
not depend on size: float64 recomputation of sampled rows / entries (the same
normalised gate, 1e-5), agreement between the tensor-core and the exact-FP32
kernels, and agreement of the zero-skipping product with the dense one."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
TOL = 1e-5


def _sample_err(A, B, C, rows):
    import torch
    r = torch.as_tensor(rows, device="cuda")
    exact = A[r].double() @ B.double()
    den = A[r].double().norm(dim=1)[:, None] * B.double().norm(dim=0)[None, :]
    return ((C[r].double() - exact).abs() / den.clamp_min(1e-30)).max().item()


@pytest.mark.parametrize("shape,want", [((65536, 1024, 1024), "MKN"), ((1024, 1024, 65536), "NKM"),
                                        ((1024, 262144, 1024), "KMN"), ((3000, 3000, 3000), "MKN")])
def test_rectangular_and_reference_cpu_shapes(cake, shape, want):
    import torch
    M, K, N = shape
    g = torch.Generator(device="cuda").manual_seed(1)
    A = torch.rand((M, K), device="cuda", generator=g) * 2 - 1
    B = torch.rand((K, N), device="cuda", generator=g) * 2 - 1
    C = torch.empty((M, N), device="cuda")
    cake.cake_sgemm(A, B, C)
    st = cake.last_stats()
    assert st["kernel"] == cake.KERNEL_TF32X3
    assert ["KMN", "MKN", "NKM"][st["sched"]] == want  # the schedule the reference derives for this shape
    rows = np.random.default_rng(0).integers(0, M, 48)
    assert _sample_err(A, B, C, rows) <= TOL
    Cf = torch.empty((M, N), device="cuda")
    cake.cake_sgemm(A, B, Cf, kernel=cake.KERNEL_FFMA)
    assert _sample_err(A, B, Cf, rows) <= TOL
    den = A.double().norm(dim=1)[rows][:, None] * B.double().norm(dim=0)[None, :]
    assert ((C[rows] - Cf[rows]).double().abs() / den).max().item() <= TOL


def test_deep_product_runs_in_ranges_of_k(cake):
    """A product deeper than 16384 with several waves of tiles is issued as launches over ranges of K that add
    to C (with a bias added once and with accumulation on top of an existing C): float64 on sampled rows."""
    import torch
    M, K, N = 4096, 16416 + 7, 4864
    g = torch.Generator(device="cuda").manual_seed(2)
    A = torch.rand((M, K), device="cuda", generator=g) * 2 - 1
    B = torch.rand((K, N), device="cuda", generator=g) * 2 - 1
    bias = torch.rand((N,), device="cuda", generator=g)
    C = torch.full((M, N), float("nan"), device="cuda")
    cake.cake_sgemm_ex(A, B, C, bias=bias, kernel=cake.KERNEL_TF32X3)
    assert cake.last_stats()["launches"] == 2 + 3  # two split kernels, three ranges of K
    rows = np.random.default_rng(1).integers(0, M, 32)
    assert _sample_err(A, B, C - bias[None, :], rows) <= TOL
    cake.cake_sgemm_ex(A, B, C, accumulate=True, kernel=cake.KERNEL_TF32X3)
    assert _sample_err(A, B, (C - bias[None, :]) / 2, rows) <= TOL


def test_batch_of_4096_small_products(cake):
    import torch
    g = torch.Generator(device="cuda").manual_seed(1)
    A = torch.rand((4096, 96, 96), device="cuda", generator=g) * 2 - 1
    B = torch.rand((4096, 96, 96), device="cuda", generator=g) * 2 - 1
    C = cake.cake_sgemm_batched(A, B)
    exact = torch.bmm(A.double(), B.double())
    den = A.double().norm(dim=2)[:, :, None] * B.double().norm(dim=1)[:, None, :]
    assert ((C.double() - exact).abs() / den).max().item() <= TOL


@pytest.mark.parametrize("density", [0.5, 0.1, 0.01])
def test_sparse_8192(cake, density):
    import torch
    n = 8192
    g = torch.Generator(device="cuda").manual_seed(3)
    A = (torch.rand((n, n), device="cuda", generator=g) * 2 - 1) * (torch.rand((n, n), device="cuda", generator=g) < density)
    B = torch.rand((n, n), device="cuda", generator=g) * 2 - 1
    rows = np.random.default_rng(1).integers(0, n, 32)
    auto = cake.cake_sp_sgemm(A, B, kernel=cake.KERNEL_AUTO)
    picked = cake.last_stats()["kernel"]
    assert picked == (cake.KERNEL_TF32X3 if density > 0.035 else cake.KERNEL_FFMA)
    assert _sample_err(A, B, auto, rows) <= TOL
    dense = torch.empty((n, n), device="cuda")
    cake.cake_sgemm(A, B, dense)  # the dense path on the densified operand
    den = A.double().norm(dim=1)[rows][:, None] * B.double().norm(dim=0)[None, :]
    assert ((auto[rows] - dense[rows]).double().abs() / den.clamp_min(1e-30)).max().item() <= TOL
    if density <= 0.1:
        skip = cake.cake_sp_sgemm(A, B, kernel=cake.KERNEL_FFMA)
        assert _sample_err(A, B, skip, rows) <= TOL
        # zero skipping == exact-FP32 dense kernel on the same operand, bit for bit (zeros contribute no operation)
        exact_kernel = torch.empty((256, n), device="cuda")
        cake.cake_sgemm(A[:256].contiguous(), B, exact_kernel, kernel=cake.KERNEL_FFMA)
        assert torch.equal(skip[:256], exact_kernel)


@pytest.mark.parametrize("cfg", [(64, 64, 56, 64), (64, 256, 14, 512)])
def test_convolutions(cake, cfg):
    import torch
    b, cin, hw, cout = cfg
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn((b, cin, hw, hw), device="cuda", generator=g) * 0.1
    w = torch.randn((cout, cin, 3, 3), device="cuda", generator=g) * 0.1
    out = cake.cake_conv2d(x, w, 1, 1)
    assert cake.last_stats()["kernel"] == cake.KERNEL_TF32X3
    ref = torch.nn.functional.conv2d(x[:4].double(), w.double(), padding=1)
    # ||filter row|| * ||patch column|| bound, evaluated loosely through the largest norms
    wn = w.double().flatten(1).norm(dim=1).max().item()
    xn = torch.nn.functional.unfold(x[:4].double(), 3, padding=1).norm(dim=1).max().item()
    assert (out[:4].double() - ref).abs().max().item() <= TOL * wn * xn
    exact = cake.cake_conv2d(x[:4].contiguous(), w, 1, 1, kernel=cake.KERNEL_FFMA)
    assert (out[:4] - exact).double().abs().max().item() <= TOL * wn * xn


def test_run_tests_of_the_cpp_api(cake):
    """run_tests() of the reference (src/util.cpp:3-136): its own grid of awkward sizes through cake_sgemm
    with every schedule, checked by cake_sgemm_checker."""
    import ctypes
    L = ctypes.CDLL(cake.library_path())
    fn = getattr(L, "_Z9run_testsv")
    fn.restype = ctypes.c_int
    assert fn() == 0
