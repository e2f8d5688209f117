"""Seeded random shapes through every entry point of the path, each result against float64 with the
normalised gate of the parity tests (1e-5).  The fixed cases elsewhere are the reference's own edge list and
the benchmark shapes; this sweep is for the corners between them: odd leading dimensions, tails shorter than a
tile, products that fit one tile exactly, shapes on either side of the kernel-selection thresholds."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
TOL = 1e-5


def _norm_err(C, A, B):
    """max |C - A B| / (||A[m,:]|| ||B[:,n]||) with the product in float64 (torch tensors on the GPU)."""
    exact = A.double() @ B.double()
    den = A.double().norm(dim=1)[:, None] * B.double().norm(dim=0)[None, :]
    return ((C.double() - exact).abs() / den.clamp_min(1e-30)).max().item()


def _rand(gen, *shape):
    import torch
    return torch.rand(shape, device="cuda", generator=gen) * 2 - 1


def test_dense_products_of_random_shapes(cake):
    import torch
    rng = np.random.default_rng(2024)
    gen = torch.Generator(device="cuda").manual_seed(7)
    shapes = [(int(rng.integers(1, 700)), int(rng.integers(1, 900)), int(rng.integers(1, 700))) for _ in range(24)]
    shapes += [(128, 32, 256), (129, 33, 257), (256, 64, 256), (255, 63, 255), (1, 1, 1), (640, 2049, 384), (1537, 40, 771)]
    for (M, K, N) in shapes:
        A, B = _rand(gen, M, K), _rand(gen, K, N)
        for kernel in (cake.KERNEL_FFMA, cake.KERNEL_TF32X3, cake.KERNEL_AUTO):
            for sch in (cake.KMN, cake.MKN, cake.NKM, cake.NA):
                C = torch.full((M, N), float("nan"), device="cuda")
                cake.cake_sgemm(A, B, C, sch=sch, kernel=kernel)
                assert _norm_err(C, A, B) <= TOL, (M, K, N, kernel, sch)


def test_extended_product_of_random_shapes(cake):
    import torch
    rng = np.random.default_rng(11)
    gen = torch.Generator(device="cuda").manual_seed(8)
    for _ in range(16):
        M, K, N = (int(rng.integers(1, 600)) for _ in range(3))
        pa, pb, pc = (int(rng.integers(0, 7)) for _ in range(3))
        ta, tb = bool(rng.integers(0, 2)), bool(rng.integers(0, 2))
        A, B = _rand(gen, M, K), _rand(gen, K, N)
        bias = _rand(gen, N)
        store_a = (A.t().contiguous() if ta else A)
        store_b = (B.t().contiguous() if tb else B)
        wide_a = torch.zeros((store_a.shape[0], store_a.shape[1] + pa), device="cuda")
        wide_b = torch.zeros((store_b.shape[0], store_b.shape[1] + pb), device="cuda")
        wide_a[:, :store_a.shape[1]] = store_a
        wide_b[:, :store_b.shape[1]] = store_b
        Cw = torch.full((M, N + pc), float("nan"), device="cuda")
        for kernel in (cake.KERNEL_FFMA, cake.KERNEL_TF32X3):
            cake.cake_sgemm_ex(wide_a[:, :store_a.shape[1]], wide_b[:, :store_b.shape[1]], Cw[:, :N], trans_a=ta, trans_b=tb,
                               bias=bias, kernel=kernel)
            assert _norm_err(Cw[:, :N] - bias[None, :], A, B) <= TOL, (M, K, N, ta, tb, pa, pb, pc, kernel)
            assert pc == 0 or torch.isnan(Cw[:, N:]).all()


def test_batches_of_random_small_products(cake):
    import torch
    rng = np.random.default_rng(5)
    gen = torch.Generator(device="cuda").manual_seed(9)
    for _ in range(12):
        batch, M, K, N = int(rng.integers(1, 400)), int(rng.integers(1, 129)), int(rng.integers(1, 300)), int(rng.integers(1, 257))
        A, B = _rand(gen, batch, M, K), _rand(gen, batch, K, N)
        for kernel in (cake.KERNEL_FFMA, cake.KERNEL_TF32X3, cake.KERNEL_AUTO):
            C = torch.full((batch, M, N), float("nan"), device="cuda")
            cake.cake_sgemm_batched(A, B, C, kernel=kernel)
            exact = torch.bmm(A.double(), B.double())
            den = A.double().norm(dim=2)[:, :, None] * B.double().norm(dim=1)[:, None, :]
            assert ((C.double() - exact).abs() / den.clamp_min(1e-30)).max().item() <= TOL, (batch, M, K, N, kernel)


def test_random_convolutions(cake):
    import torch
    rng = np.random.default_rng(3)
    gen = torch.Generator(device="cuda").manual_seed(10)
    for _ in range(14):
        b, cin, cout = int(rng.integers(1, 6)), int(rng.integers(1, 70)), int(rng.integers(1, 150))
        H, W = int(rng.integers(3, 30)), int(rng.integers(3, 30))
        hf, wf = int(rng.integers(1, 4)), int(rng.integers(1, 4))
        stride, pad = int(rng.integers(1, 3)), int(rng.integers(0, 3))
        if H + 2 * pad < hf or W + 2 * pad < wf:
            continue
        x = torch.randn((b, cin, H, W), device="cuda", generator=gen) * 0.1
        w = torch.randn((cout, cin, hf, wf), device="cuda", generator=gen) * 0.1
        ref = torch.nn.functional.conv2d(x.double(), w.double(), stride=stride, padding=pad)
        # normalisation: the product behind the convolution has rows w[co] and columns = patches
        patches = torch.nn.functional.unfold(x.double(), (hf, wf), padding=pad, stride=stride)  # b x K x P
        den = w.double().reshape(cout, -1).norm(dim=1)[None, :, None] * patches.norm(dim=1)[:, None, :]
        for kernel in (cake.KERNEL_FFMA, cake.KERNEL_TF32X3, cake.KERNEL_AUTO):
            out = cake.cake_conv2d(x, w, stride, pad, kernel=kernel)
            err = ((out.double() - ref).reshape(b, cout, -1).abs() / den.clamp_min(1e-30)).max().item()
            assert err <= TOL, (b, cin, H, W, cout, hf, wf, stride, pad, kernel, err)


def test_random_matrix_vector_products_and_sparse(cake):
    import torch
    rng = np.random.default_rng(4)
    gen = torch.Generator(device="cuda").manual_seed(12)
    for _ in range(12):
        M, K = int(rng.integers(1, 5000)), int(rng.integers(1, 5000))
        A, x = _rand(gen, M, K), _rand(gen, K)
        exact = A.double() @ x.double()
        scale = A.double().norm(dim=1) * x.double().norm()
        y = cake.cake_sgemv(A, x)
        assert ((y.double() - exact).abs() / scale.clamp_min(1e-30)).max().item() <= TOL, (M, K)
        y = cake.cake_sgemv(A.t().contiguous(), x, col_major=True)
        assert ((y.double() - exact).abs() / scale.clamp_min(1e-30)).max().item() <= TOL, (M, K, "col")
    for _ in range(6):
        M, K, N = (int(rng.integers(1, 900)) for _ in range(3))
        density = float(rng.choice([0.002, 0.02, 0.3]))
        A = _rand(gen, M, K) * (torch.rand((M, K), device="cuda", generator=gen) < density)
        B = _rand(gen, K, N)
        for kernel in (cake.KERNEL_FFMA, cake.KERNEL_AUTO):
            C = cake.cake_sp_sgemm(A, B, kernel=kernel)
            exact = A.double() @ B.double()
            den = A.double().norm(dim=1)[:, None] * B.double().norm(dim=0)[None, :]
            assert ((C.double() - exact).abs() / den.clamp_min(1e-30)).max().item() <= TOL, (M, K, N, density, kernel)
