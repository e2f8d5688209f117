"""Parity of the CUDA path with the CPU oracle, through the C ABI.

Gate (both kernels): max |C - C_ref| / (||A[m,:]||_2 ||B[:,n]||_2) <= 1e-5, where
C_ref is the oracle's cake_sgemm (= the reference's result bit for bit).  Data
movement (pack / unpack / im2col) and the sparse product are compared bit-exactly.
"""
import os

import numpy as np
import pytest

from _oracle import KMN, MKN, NKM, NA, DEFAULT_CACHES, rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-5
GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_golden.npz"))

# the reference's own grid of awkward sizes (src/util.cpp:12-13)
EDGE = (1, 10, 96, 111, 960)
GRID = [(M, K, N) for M in EDGE for K in EDGE for N in EDGE if (M * K * N) <= 960 * 960 * 111]
GRID += [(2111, 96, 111), (111, 2111, 96), (96, 111, 2111), (960, 960, 960), (2111, 2111, 10)]


def _inputs(oracle, M, K, N):
    return oracle.uniform((M, K), 1), oracle.uniform((K, N), 2)


@pytest.mark.parametrize("kernel_name", ["ffma", "tf32x3"])
def test_dense_grid_all_schedules(cake, oracle, kernel_name):
    kernel = {"ffma": cake.KERNEL_FFMA, "tf32x3": cake.KERNEL_TF32X3}[kernel_name]
    worst = 0.0
    for i, (M, K, N) in enumerate(GRID):
        A, B = _inputs(oracle, M, K, N)
        scheds = (KMN, MKN, NKM, NA) if i % 4 == 0 else ((KMN, MKN, NKM, NA)[i % 4],)
        for sch in scheds:
            ref, _ = oracle.sgemm(A, B, 8, sch)
            C = np.full((M, N), np.nan, np.float32)
            cake.cake_sgemm(A, B, C, p=8, sch=sch, kernel=kernel)
            assert cake.last_stats()["kernel"] == kernel
            err = rel_err(C, ref, A, B)
            worst = max(worst, err)
            assert err <= TOL, (kernel_name, M, K, N, sch, err)
    print("worst normalised error (%s): %.3e" % (kernel_name, worst))


@pytest.mark.parametrize("key", sorted(k for k in GOLDEN.files if k.startswith("sgemm_")))
def test_dense_against_reference_golden(cake, oracle, key):
    M, K, N, p, sch = (int(v) for v in key.split("_")[1:])
    A, B = _inputs(oracle, M, K, N)
    for kernel in (cake.KERNEL_FFMA, cake.KERNEL_TF32X3):
        C = cake.cake_sgemm(A, B, sch=sch, kernel=kernel)
        assert rel_err(C, GOLDEN[key], A, B) <= TOL


def test_auto_kernel_and_device_pointers(cake, oracle):
    import torch
    M, K, N = 777, 515, 1030
    A, B = _inputs(oracle, M, K, N)
    ref, _ = oracle.sgemm(A, B, 8, NA)
    dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    for kernel in (cake.KERNEL_AUTO, cake.KERNEL_FFMA, cake.KERNEL_TF32X3):
        dC = torch.full((M, N), float("nan"), device="cuda")
        cake.cake_sgemm(dA, dB, dC, kernel=kernel)
        assert rel_err(dC.cpu().numpy(), ref, A, B) <= TOL
    assert cake.last_stats()["kernel"] == cake.KERNEL_TF32X3
    # AUTO picks the tensor-core kernel for this size and FFMA for a tiny one
    cake.cake_sgemm(dA, dB, dC, kernel=cake.KERNEL_AUTO)
    assert cake.last_stats()["kernel"] == cake.KERNEL_TF32X3
    cake.cake_sgemm(A[:8], B, kernel=cake.KERNEL_AUTO)
    assert cake.last_stats()["kernel"] == cake.KERNEL_FFMA


@pytest.mark.parametrize("kernel_name", ["ffma", "tf32x3"])
def test_transposed_operands_leading_dimensions_and_bias(cake, oracle, kernel_name):
    """cakeb200_sgemm_ex: op(A) op(B) + bias must equal the oracle's product of the
    explicitly transposed, densely copied operands (what reference src/linear.cpp:22,76-84
    feeds cake_sgemm) plus the bias added afterwards (:44-46)."""
    import torch
    kernel = {"ffma": cake.KERNEL_FFMA, "tf32x3": cake.KERNEL_TF32X3}[kernel_name]
    for (M, K, N) in [(300, 515, 260), (129, 96, 1031), (1000, 2111, 257)]:
        A, B = _inputs(oracle, M, K, N)
        bias = oracle.uniform((1, N), 7)[0]
        ref, _ = oracle.sgemm(A, B, 8, NA)
        dbias = torch.from_numpy(bias).cuda()
        # operands live inside wider allocations, so every leading dimension differs from the row length
        wide = lambda X: torch.from_numpy(np.pad(X, ((0, 0), (3, 5)))).cuda()[:, 3:3 + X.shape[1]]
        for ta in (False, True):
            for tb in (False, True):
                dA = wide(np.ascontiguousarray(A.T)) if ta else wide(A)
                dB = wide(np.ascontiguousarray(B.T)) if tb else wide(B)
                Cw = torch.full((M, N + 8), float("nan"), device="cuda")
                dC = Cw[:, 4:4 + N]
                cake.cake_sgemm_ex(dA, dB, dC, trans_a=ta, trans_b=tb, bias=dbias, kernel=kernel)
                assert cake.last_stats()["kernel"] == kernel
                got = dC.cpu().numpy()
                assert rel_err(got - bias[None, :], ref, A, B) <= TOL, (kernel_name, M, K, N, ta, tb)
                assert torch.isnan(Cw[:, :4]).all() and torch.isnan(Cw[:, 4 + N:]).all()  # nothing outside the view
                # accumulate on top of the previous result: C += A B + bias
                cake.cake_sgemm_ex(dA, dB, dC, trans_a=ta, trans_b=tb, bias=dbias, accumulate=True, kernel=kernel)
                assert rel_err((dC.cpu().numpy() - 2 * bias[None, :]) / 2, ref, A, B) <= TOL
    # a leading dimension shorter than a row is an argument error, not a launch
    import ctypes
    x = torch.zeros((64, 64), device="cuda")
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = cake.lib().cakeb200_sgemm_ex(vp(x), 32, 0, vp(x), 64, 0, vp(x), 64, 64, 64, 64, None, 0, NA, kernel, None)
    assert rc != 0 and b"leading dimension" in cake.lib().cakeb200_last_error()


def test_beta_flag_matches_reference_semantics(cake, oracle):
    M, K, N = 300, 200, 260
    A, B = _inputs(oracle, M, K, N)
    C0 = oracle.uniform((M, N), 3)
    for kernel in (cake.KERNEL_FFMA, cake.KERNEL_TF32X3):
        for sch in (MKN, NKM):
            ref, _ = oracle.sgemm(A, B, 8, sch, beta=1.0, C=C0)
            C = C0.copy()
            cake.cake_sgemm(A, B, C, beta=1.0, sch=sch, kernel=kernel)
            assert rel_err(C, ref, A, B) <= TOL
        ref, _ = oracle.sgemm(A, B, 8, KMN, beta=1.0, C=C0)  # K-first overwrites
        C = C0.copy()
        cake.cake_sgemm(A, B, C, beta=1.0, sch=KMN, kernel=kernel)
        assert rel_err(C, ref, A, B) <= TOL


def test_host_operands_banded_copy_compute_overlap(cake, oracle):
    """Host arrays with many rows take the banded path (copies overlapped with compute);
    it must give what the single-shot path gives for device operands."""
    import torch
    for (M, K, N) in [(2600, 300, 520), (1024, 64, 1000), (4099, 129, 257)]:
        A, B = _inputs(oracle, M, K, N)
        C0 = oracle.uniform((M, N), 3)
        ref, _ = oracle.sgemm(A, B, 8, NA)
        for kernel in (cake.KERNEL_FFMA, cake.KERNEL_TF32X3):
            C = cake.cake_sgemm(A, B, kernel=kernel)
            assert rel_err(C, ref, A, B) <= TOL, (M, K, N, kernel)
            dC = cake.cake_sgemm(torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda(), kernel=kernel)
            assert np.array_equal(C, dC.cpu().numpy()), (M, K, N, kernel)
            # host A and C, device B
            C2 = np.full((M, N), np.nan, np.float32)
            cake.cake_sgemm(A, torch.from_numpy(B).cuda(), C2, kernel=kernel)
            assert np.array_equal(C, C2), (M, K, N, kernel)
        refb, _ = oracle.sgemm(A, B, 8, MKN, beta=1.0, C=C0)
        Cb = C0.copy()
        cake.cake_sgemm(A, B, Cb, beta=1.0, sch=MKN, kernel=cake.KERNEL_TF32X3)
        assert rel_err(Cb, refb, A, B) <= TOL


def test_profile_events_of_async_products(cake):
    import torch
    n = 1024
    A, B, C = (torch.rand((n, n), device="cuda") for _ in range(3))
    s = torch.cuda.current_stream().cuda_stream
    cake.cake_sgemm(A, B, C, kernel=cake.KERNEL_TF32X3)
    cake.profile_begin()
    for _ in range(4):
        cake.cake_sgemm_async(A.data_ptr(), B.data_ptr(), C.data_ptr(), n, n, n, 0, cake.NA, cake.KERNEL_TF32X3, s)
    pre, ker, calls = cake.profile_end()
    assert calls == 4 and pre > 0 and ker > 0
    ref = A.double() @ B.double()
    assert (C.double() - ref).abs().max().item() < 1e-2


def test_async_products_capture_into_a_cuda_graph(cake, oracle):
    """After one ordinary call (which sizes the scratch arena and uploads the tile plan) the asynchronous entry
    point only enqueues kernels, so a stream capture records it; replaying the graph gives the same bits."""
    import torch
    for (M, K, N, kernel) in [(1024, 1024, 1024, cake.KERNEL_TF32X3), (300, 200, 260, cake.KERNEL_FFMA)]:
        A, B = _inputs(oracle, M, K, N)
        ref, _ = oracle.sgemm(A, B, 8, NA)
        dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
        dC = torch.zeros((M, N), device="cuda")
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            cake.cake_sgemm_async(dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), M, N, K, 0, NA, kernel, s.cuda_stream)
            s.synchronize()
            eager = dC.clone()
            dC.zero_()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=s):
                for _ in range(3):
                    cake.cake_sgemm_async(dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), M, N, K, 0, NA, kernel, s.cuda_stream)
            assert not dC.any()  # capturing ran nothing
            graph.replay()
            s.synchronize()
        assert torch.equal(dC, eager)
        assert rel_err(dC.cpu().numpy(), ref, A, B) <= TOL


def test_skinny_shapes_exercise_each_schedule_and_cut_tiles(cake, oracle):
    # 1/16-scale versions of the M-first, N-first and K-first benchmark shapes
    for (M, K, N, want) in [(4096, 64, 64, MKN), (64, 64, 4096, NKM), (256, 16384, 320, KMN)]:
        A, B = _inputs(oracle, M, K, N)
        ref, _ = oracle.sgemm(A, B, 8, NA)
        for kernel in (cake.KERNEL_FFMA, cake.KERNEL_TF32X3):
            C = cake.cake_sgemm(A, B, kernel=kernel)
            assert rel_err(C, ref, A, B) <= TOL, (M, K, N, kernel)
        assert cake.last_stats()["sched"] == want


def test_tf32x3_is_fp32_class_against_float64(cake, oracle):
    M, K, N = 512, 4096, 512
    A, B = _inputs(oracle, M, K, N)
    ref64 = A.astype(np.float64) @ B.astype(np.float64)
    bound = np.abs(A).astype(np.float64) @ np.abs(B).astype(np.float64)
    errs = {}
    for name, kernel in (("ffma", cake.KERNEL_FFMA), ("tf32x3", cake.KERNEL_TF32X3)):
        C = cake.cake_sgemm(A, B, kernel=kernel)
        errs[name] = float((np.abs(C - ref64) / bound).max())
    print("max |C - C64| / sum|a||b|:", errs)
    assert errs["ffma"] < 2e-6 and errs["tf32x3"] < 2e-6


def test_full_size_properties(cake, oracle):
    """8192^3 (the headline configuration): the oracle would take minutes, so
    check float64 recomputation of sampled entries, agreement of the two
    kernels, and linearity C(A, B) + C(A, B') = C(A, B + B') on a slab."""
    import torch
    n = 8192
    g = torch.Generator(device="cuda").manual_seed(1)
    A = torch.rand((n, n), device="cuda", generator=g) * 2 - 1
    B = torch.rand((n, n), device="cuda", generator=g) * 2 - 1
    C3 = torch.empty((n, n), device="cuda")
    cake.cake_sgemm(A, B, C3, kernel=cake.KERNEL_TF32X3)
    rng = np.random.default_rng(0)
    rows, cols = rng.integers(0, n, 2048), rng.integers(0, n, 2048)
    r_t, c_t = torch.from_numpy(rows).cuda(), torch.from_numpy(cols).cuda()
    exact = (A[r_t].double() * B[:, c_t].t().double()).sum(1)
    norm = A[r_t].double().norm(dim=1) * B[:, c_t].double().norm(dim=0)
    err = ((C3[r_t, c_t].double() - exact).abs() / norm).max().item()
    assert err <= TOL, err
    Cf = torch.empty((1024, n), device="cuda")
    cake.cake_sgemm(A[:1024].contiguous(), B, Cf, kernel=cake.KERNEL_FFMA)
    na, nb = A[:1024].double().norm(dim=1), B.double().norm(dim=0)
    diff = ((Cf - C3[:1024]).double().abs() / (na[:, None] * nb[None, :])).max().item()
    assert diff <= TOL, diff
    B2 = torch.rand((n, n), device="cuda", generator=g) * 2 - 1
    As = A[:1024].contiguous()
    C1, C2, C12 = (torch.empty((1024, n), device="cuda") for _ in range(3))
    cake.cake_sgemm(As, B, C1, kernel=cake.KERNEL_TF32X3)
    cake.cake_sgemm(As, B2, C2, kernel=cake.KERNEL_TF32X3)
    cake.cake_sgemm(As, B + B2, C12, kernel=cake.KERNEL_TF32X3)
    nb12 = (B.double().norm(dim=0) + B2.double().norm(dim=0))
    lin = ((C1 + C2 - C12).double().abs() / (na[:, None] * nb12[None, :])).max().item()
    assert lin <= TOL, lin


def test_pack_unpack_bit_exact(cake, oracle):
    for (M, K, N, p) in [(111, 96, 77, 4), (10, 960, 20, 5), (960, 10, 7, 8), (2111, 300, 500, 8), (96, 96, 96, 3)]:
        A, B, C = oracle.uniform((M, K), 1), oracle.uniform((K, N), 2), oracle.uniform((M, N), 3)
        for sch in (KMN, MKN, NKM, NA):
            cx = cake.Cntx.make(*DEFAULT_CACHES)
            x = cake.init_block_dims(M, N, K, p, cx, sch)
            Ap = cake.pack_A(A, M, K, p, x, cx)
            Bp = cake.pack_B(B, K, N, p, x, cx)
            Cp = cake.pack_C(C, M, N, p, x, cx)
            assert np.array_equal(Ap, oracle.pack(0, A, M, N, K, p, sch)), ("A", M, K, N, p, sch)
            assert np.array_equal(Bp, oracle.pack(1, B, M, N, K, p, sch)), ("B", M, K, N, p, sch)
            assert np.array_equal(Cp, oracle.pack(2, C, M, N, K, p, sch)), ("C", M, K, N, p, sch)
            assert np.array_equal(cake.unpack_C(Cp, M, N, p, x, cx), C)
            assert np.array_equal(cake.unpack_A(Ap, M, K, p, x, cx), A)
            assert np.array_equal(cake.unpack_B(Bp, K, N, p, x, cx), B)
            for which, got in ((0, Ap), (1, Bp), (2, Cp)):
                key = "pack%s_%d_%d_%d_%d_%d" % ("ABC"[which], M, K, N, p, x.sch)
                if sch != NA and key in GOLDEN.files:
                    assert np.array_equal(got, GOLDEN[key]), key


def test_pack_sixteen_byte_path_bit_exact(cake, oracle):
    """Shapes whose blocks allow 16-byte moves (A: four k at a time for the 6-row panels; B, C: four columns of
    a 16-wide panel): same bytes as the oracle and as the one-element-per-thread path."""
    wide = 0
    for (M, K, N, p) in [(960, 960, 960, 8), (1200, 512, 1024, 4), (1026, 516, 1040, 8), (3000, 3000, 3000, 8)]:
        A, B, C = oracle.uniform((M, K), 1), oracle.uniform((K, N), 2), oracle.uniform((M, N), 3)
        for sch in (KMN, MKN, NKM):
            cx = cake.Cntx.make(*DEFAULT_CACHES)
            x = cake.init_block_dims(M, N, K, p, cx, sch)
            got = {}
            for mode in ("vector", "scalar"):
                if mode == "scalar":
                    cake.set_option("pack_scalar", 1)
                try:
                    Ap = cake.pack_A(A, M, K, p, x, cx); wa = cake.last_stats()["tile_k"]
                    Bp = cake.pack_B(B, K, N, p, x, cx); wb = cake.last_stats()["tile_k"]
                    Cp = cake.pack_C(C, M, N, p, x, cx); wc = cake.last_stats()["tile_k"]
                    back = (cake.unpack_A(Ap, M, K, p, x, cx), cake.unpack_B(Bp, K, N, p, x, cx), cake.unpack_C(Cp, M, N, p, x, cx))
                finally:
                    cake.set_option("pack_scalar", 0)
                got[mode] = (Ap, Bp, Cp)
                if mode == "vector":
                    wide += (wa > 1) + (wb > 1) + (wc > 1)
                else:
                    assert (wa, wb, wc) == (1, 1, 1)
                assert np.array_equal(back[0], A) and np.array_equal(back[1], B) and np.array_equal(back[2], C)
            for i in range(3):
                assert np.array_equal(got["vector"][i], got["scalar"][i]), ("ABC"[i], M, K, N, p, sch)
            if M <= 1200:
                assert np.array_equal(got["vector"][0], oracle.pack(0, A, M, N, K, p, sch))
                assert np.array_equal(got["vector"][1], oracle.pack(1, B, M, N, K, p, sch))
                assert np.array_equal(got["vector"][2], oracle.pack(2, C, M, N, K, p, sch))
    assert wide >= 24, wide  # most of these calls must actually have taken a wide path


def test_pack_on_device_pointers(cake, oracle):
    import torch
    M, K, N, p = 500, 300, 700, 8
    A = oracle.uniform((M, K), 1)
    cx = cake.Cntx.make(*DEFAULT_CACHES)
    x = cake.init_block_dims(M, N, K, p, cx, KMN)
    Ap = cake.pack_A(torch.from_numpy(A).cuda(), M, K, p, x, cx)
    assert Ap.is_cuda
    assert np.array_equal(Ap.cpu().numpy(), oracle.pack(0, A, M, N, K, p, KMN))


def test_sparse_product_bit_exact_and_against_dense_reference(cake, oracle):
    # densities on both sides of the 3 % switch between the staged and the gathering multiply kernel,
    # aligned and ragged N, an all-zero operand
    for (M, K, N, d) in [(300, 257, 130, 0.5), (513, 1000, 260, 0.1), (1024, 2048, 515, 0.01), (7, 5, 3, 0.5),
                         (512, 1024, 640, 0.02), (130, 300, 1100, 0.005), (64, 64, 64, 0.0)]:
        A = oracle.sparse((M, K), 1, 3, d)
        B = oracle.uniform((K, N), 2)
        C = cake.cake_sp_sgemm(A, B, kernel=cake.KERNEL_FFMA)  # forced zero-skipping kernels
        assert cake.last_stats()["kernel"] == cake.KERNEL_FFMA
        assert np.array_equal(C, oracle.sp_sgemm(A, B)), (M, K, N, d)
        dense_ref, _ = oracle.sgemm(A, B, 8, NA)  # the reference's dense path on the densified operand
        assert rel_err(C, dense_ref, A, B) <= TOL
        for kernel in (cake.KERNEL_TF32X3, cake.KERNEL_AUTO):
            C3 = cake.cake_sp_sgemm(A, B, kernel=kernel)
            assert rel_err(C3, dense_ref, A, B) <= TOL
    # AUTO: dense tensor-core product once more than ~1 % is nonzero and the product is large, else zero skipping
    A, B = oracle.sparse((1024, 2048), 1, 3, 0.05), oracle.uniform((2048, 512), 2)
    cake.cake_sp_sgemm(A, B, kernel=cake.KERNEL_AUTO)
    assert cake.last_stats()["kernel"] == cake.KERNEL_TF32X3
    A = oracle.sparse((1024, 2048), 1, 3, 0.002)
    cake.cake_sp_sgemm(A, B, kernel=cake.KERNEL_AUTO)
    assert cake.last_stats()["kernel"] == cake.KERNEL_FFMA


def test_im2col_and_conv(cake, oracle):
    for (b, cin, H, W, cout, hf, stride, pad) in [(2, 3, 7, 6, 5, 3, 1, 1), (3, 8, 14, 14, 16, 3, 1, 1),
                                                 (1, 4, 9, 9, 6, 3, 2, 0), (2, 16, 12, 12, 32, 1, 1, 0),
                                                 (1, 64, 5, 300, 8, 3, 1, 1)]:  # last: rows too wide to stage in shared memory
        x = oracle.normal((b, cin, H, W), 4, 0.1)
        w = oracle.normal((cout, cin, hf, hf), 5, 0.1)
        assert np.array_equal(cake.im2col(x, hf, hf, stride, pad), oracle.im2col(x, hf, hf, stride, pad))
        ref = oracle.conv2d(x, w, stride, pad, 8)
        col = oracle.im2col(x, hf, hf, stride, pad)
        for kernel in (cake.KERNEL_FFMA, cake.KERNEL_TF32X3, cake.KERNEL_AUTO):
            out = cake.cake_conv2d(x, w, stride, pad, kernel=kernel)
            Ho, Wo = out.shape[2:]
            got = out.transpose(1, 0, 2, 3).reshape(cout, b * Ho * Wo)
            want = ref.transpose(1, 0, 2, 3).reshape(cout, b * Ho * Wo)
            assert rel_err(got, want, w.reshape(cout, -1), col) <= TOL, (b, cin, H, W, cout, kernel)


def test_conv_benchmark_shape_scaled_down(cake, oracle):
    """The second convolution configuration (256 -> 512 channels, 14 x 14, 3 x 3, pad 1) at batch 4:
    large enough for the tensor-core route, checked against float64."""
    import torch
    x = oracle.normal((4, 256, 14, 14), 4, 0.1)
    w = oracle.normal((512, 256, 3, 3), 5, 0.1)
    out = cake.cake_conv2d(x, w, 1, 1)
    assert cake.last_stats()["kernel"] == cake.KERNEL_TF32X3
    ref = torch.nn.functional.conv2d(torch.from_numpy(x).double(), torch.from_numpy(w).double(), padding=1).numpy()
    col = oracle.im2col(x, 3, 3, 1, 1)
    got = out.transpose(1, 0, 2, 3).reshape(512, -1)
    want = ref.transpose(1, 0, 2, 3).reshape(512, -1)
    assert rel_err(got, want, w.reshape(512, -1), col) <= TOL


def test_implicit_convolution_geometries(cake, oracle):
    """The stride-1 tensor-core convolution that builds its patch operand in shared memory: filter shapes,
    paddings, channel counts off the 32 / 16 grids, several channel tiles, tiles of one and of many rows, and
    the fallbacks (stride 2, image area not a multiple of 4 floats) - each against the oracle's im2col + GEMM
    where that is small and against a float64 convolution always."""
    import torch
    cases = [  # batch, cin, H, W, cout, hf, wf, pad, implicit route expected
        (3, 8, 14, 14, 16, 3, 3, 1, True), (2, 3, 8, 6, 5, 3, 3, 1, True), (2, 40, 12, 12, 130, 3, 3, 1, True),
        (2, 32, 10, 10, 64, 1, 1, 0, True), (1, 16, 9, 12, 24, 5, 3, 2, True), (2, 7, 6, 10, 9, 3, 5, 0, True),
        (5, 64, 56, 56, 64, 3, 3, 1, True), (2, 33, 16, 4, 17, 3, 3, 3, True), (1, 4, 30, 80, 8, 3, 3, 1, True),
        (4, 8, 10, 8, 16, 3, 3, 1, True), (7, 20, 12, 8, 140, 3, 3, 1, True),
        (1, 64, 5, 300, 8, 3, 3, 1, False), (2, 8, 7, 7, 16, 3, 3, 1, False)]
    for (b, cin, H, W, cout, hf, wf, pad, implicit) in cases:
        x = oracle.normal((b, cin, H, W), 4, 0.1)
        w = oracle.normal((cout, cin, hf, wf), 5, 0.1)
        out = cake.cake_conv2d(x, w, 1, pad, kernel=cake.KERNEL_TF32X3)
        st = cake.last_stats()
        assert st["kernel"] == cake.KERNEL_TF32X3
        assert (st["launches"] == 2) == implicit, (b, cin, H, W, cout, hf, wf, pad, st)
        # both tilings of the implicit kernel (whole rows of one image; runs of 128 positions across images)
        for force in (2, 3):  # "conv_route": 2 = whole rows of one image, 3 = runs of 128 positions
            cake.set_option("conv_route", force)
            try:
                other = cake.cake_conv2d(x, w, 1, pad, kernel=cake.KERNEL_TF32X3)
            finally:
                cake.set_option("conv_route", 0)
            assert np.abs(other - out).max() <= 1e-4 * max(1.0, np.abs(out).max()), (force, b, cin, H, W, cout)
        ref = torch.nn.functional.conv2d(torch.from_numpy(x).double(), torch.from_numpy(w).double(), padding=pad).numpy()
        assert out.shape == ref.shape
        col = oracle.im2col(x, hf, wf, 1, pad)
        Ho, Wo = out.shape[2:]
        got = out.transpose(1, 0, 2, 3).reshape(cout, b * Ho * Wo)
        want = ref.transpose(1, 0, 2, 3).reshape(cout, b * Ho * Wo)
        assert rel_err(got, want, w.reshape(cout, -1), col) <= TOL, (b, cin, H, W, cout, hf, wf, pad)
        if b * cin * H * W <= 20000:
            want = oracle.conv2d(x, w, 1, pad, 8).transpose(1, 0, 2, 3).reshape(cout, b * Ho * Wo)
            assert rel_err(got, want, w.reshape(cout, -1), col) <= TOL
    # the older route (im2col planes) must agree with the implicit one to the same tolerance
    x, w = oracle.normal((2, 40, 12, 12), 4, 0.1), oracle.normal((130, 40, 3, 3), 5, 0.1)
    a = cake.cake_conv2d(x, w, 1, 1, kernel=cake.KERNEL_TF32X3)
    cake.set_option("conv_route", 1)
    try:
        b2 = cake.cake_conv2d(x, w, 1, 1, kernel=cake.KERNEL_TF32X3)
        assert cake.last_stats()["launches"] == 3
    finally:
        cake.set_option("conv_route", 0)
    col = oracle.im2col(x, 3, 3, 1, 1)
    assert rel_err(a.transpose(1, 0, 2, 3).reshape(130, -1), b2.transpose(1, 0, 2, 3).reshape(130, -1), w.reshape(130, -1), col) <= TOL


def test_batched_small(cake, oracle):
    for (batch, M, K, N) in [(64, 96, 96, 96), (5, 33, 17, 70), (3, 130, 40, 129)]:
        A, B = oracle.uniform((batch, M, K), 1), oracle.uniform((batch, K, N), 2)
        C = cake.cake_sgemm_batched(A, B)
        ref = oracle.sgemm_batched(A, B, 8)
        for i in range(batch):
            assert rel_err(C[i], ref[i], A[i], B[i]) <= TOL


def test_batched_small_on_tensor_cores(cake, oracle):
    """The batched kernel that splits its operands in shared memory: full and ragged tiles, K not a multiple
    of the stage depth, N at the 256 limit, more products than SMs (several per CTA, both accumulators in use)."""
    shapes = [(300, 96, 96, 96), (7, 128, 64, 256), (333, 33, 17, 70), (40, 100, 200, 48), (2, 1, 1, 1), (150, 128, 37, 130),
              (1, 64, 100, 64), (200, 33, 64, 48), (37, 128, 96, 192), (300, 96, 96, 96), (300, 96, 96, 96)]
    for case, (batch, M, K, N) in enumerate(shapes):
        # the last case repeats the first with the producers reading global memory themselves instead of the TMA ring
        if case == len(shapes) - 1:
            cake.set_option("small_operands", 2)
        # ... and the one before it with the split A operand in shared memory instead of tensor memory
        if case == len(shapes) - 2:
            cake.set_option("small_operands", 1)
        A, B = oracle.uniform((batch, M, K), 1), oracle.uniform((batch, K, N), 2)
        C = np.full((batch, M, N), np.nan, np.float32)
        cake.cake_sgemm_batched(A, B, C, kernel=cake.KERNEL_TF32X3)
        assert cake.last_stats()["kernel"] == cake.KERNEL_TF32X3
        check = range(batch) if batch <= 8 else (0, 1, batch // 2, batch - 2, batch - 1)
        ref = oracle.sgemm_batched(np.ascontiguousarray(A[list(check)]), np.ascontiguousarray(B[list(check)]), 8)
        for j, i in enumerate(check):
            assert rel_err(C[i], ref[j], A[i], B[i]) <= TOL, (batch, M, K, N, i)
        # every item against float64 as well (cheap), so no item is skipped
        ref64 = np.einsum("bmk,bkn->bmn", A.astype(np.float64), B.astype(np.float64))
        den = np.linalg.norm(A, axis=2)[:, :, None] * np.linalg.norm(B, axis=1)[:, None, :]
        assert (np.abs(C - ref64) / np.maximum(den, 1e-30)).max() <= TOL
    cake.set_option("small_operands", 0)
    # AUTO takes the tensor-core kernel for a large batch of well-filled tiles, FFMA for a handful of tiny ones
    A, B = oracle.uniform((300, 96, 96), 1), oracle.uniform((300, 96, 96), 2)
    cake.cake_sgemm_batched(A, B)
    assert cake.last_stats()["kernel"] == cake.KERNEL_TF32X3
    cake.cake_sgemm_batched(A[:4], B[:4])
    assert cake.last_stats()["kernel"] == cake.KERNEL_FFMA
    with pytest.raises(cake.CakeError):
        cake.cake_sgemm_batched(oracle.uniform((2, 130, 8), 1), oracle.uniform((2, 8, 8), 2), kernel=cake.KERNEL_TF32X3)


def test_matrix_vector_product(cake, oracle):
    """cake_sgemv: the reference driver's column-major layout (accumulating into y, as its microkernel does) and
    the row-major N = 1 case, against the oracle's fused-multiply-add chain and float64.  Shapes cover one K
    slice and many, row counts off the 4- and 1024-grids, and rows that cannot be read 16 bytes at a time."""
    import torch
    for (M, K) in [(8, 8), (1000, 77), (4096, 4096), (17, 5000), (1022, 333), (20000, 130), (64, 100000)]:
        A = oracle.uniform((K, M), 1)   # column-major storage of the M x K matrix
        x = oracle.uniform((K,), 2)
        y0 = oracle.uniform((M,), 3)
        want = oracle.sgemv(A, x, y0)
        ref64 = y0.astype(np.float64) + A.astype(np.float64).T @ x.astype(np.float64)
        scale = np.linalg.norm(A, axis=0) * np.linalg.norm(x)
        y = y0.copy()
        cake.cake_sgemv(A, x, y, col_major=True, accumulate=True)
        assert (np.abs(y - want) / scale).max() <= TOL, (M, K)
        assert (np.abs(y - ref64) / scale).max() <= TOL
        # device pointers, no accumulation
        dy = cake.cake_sgemv(torch.from_numpy(A).cuda(), torch.from_numpy(x).cuda(), col_major=True).cpu().numpy()
        assert (np.abs(dy - (ref64 - y0)) / scale).max() <= TOL
        # row-major
        Ar = np.ascontiguousarray(A.T)
        yr = cake.cake_sgemv(Ar, x)
        assert (np.abs(yr - (ref64 - y0)) / scale).max() <= TOL
        yr2 = y0.copy()
        cake.cake_sgemv(Ar, x, yr2, accumulate=True)
        assert (np.abs(yr2 - ref64) / scale).max() <= TOL
    # cake_sgemm with one column or one row takes the same kernels
    dev = lambda X: torch.from_numpy(X).cuda()
    A, B = oracle.uniform((3000, 1500), 1), oracle.uniform((1500, 1), 2)
    ref, _ = oracle.sgemm(A, B, 8, NA)
    assert rel_err(cake.cake_sgemm(dev(A), dev(B)).cpu().numpy(), ref, A, B) <= TOL and cake.last_stats()["launches"] == 1
    assert rel_err(cake.cake_sgemm(A, B), ref, A, B) <= TOL  # host operands: row bands, same kernel
    A, B = oracle.uniform((1, 1500), 1), oracle.uniform((1500, 2000), 2)
    ref, _ = oracle.sgemm(A, B, 8, NA)
    assert rel_err(cake.cake_sgemm(dev(A), dev(B)).cpu().numpy(), ref, A, B) <= TOL and cake.last_stats()["launches"] == 2
    # twice the same call gives the same bits (fixed summation order)
    A, x = oracle.uniform((3000, 2000), 1), oracle.uniform((3000,), 2)
    assert np.array_equal(cake.cake_sgemv(A, x, col_major=True), cake.cake_sgemv(A, x, col_major=True))


def test_a_stalled_wait_gives_up_and_the_context_survives(cake, oracle):
    """The device-side waits are bounded.  The self-test kernel waits on a barrier nothing signals (limit 2 ms):
    the call must come back with the time-out status, and the next product must run as if nothing had happened."""
    import time
    cake.cake_sgemm(*_inputs(oracle, 64, 64, 64))  # the first call of a process creates the device state
    t0 = time.perf_counter()
    rc = cake.lib().cakeb200_selftest_bounded_wait(2000, None)
    waited = time.perf_counter() - t0
    assert rc == -4, rc  # CAKEB200_ERR_DEVICE_TIMEOUT
    assert b"where 900" in cake.lib().cakeb200_last_error()
    assert 0.0015 <= waited < 0.5, waited
    A, B = _inputs(oracle, 300, 200, 260)
    ref, _ = oracle.sgemm(A, B, 8, NA)
    for kernel in (cake.KERNEL_TF32X3, cake.KERNEL_FFMA):
        assert rel_err(cake.cake_sgemm(A, B, kernel=kernel), ref, A, B) <= TOL
    assert cake.lib().cakeb200_selftest_bounded_wait(0, None) == -1  # argument error, nothing launched
    # the same in a cluster of two CTAs: the leader waits for an arrival of its peer that never comes
    t0 = time.perf_counter()
    rc = cake.lib().cakeb200_selftest_bounded_wait_pair(2000, None)
    waited = time.perf_counter() - t0
    assert rc == -4, rc
    assert b"where 901" in cake.lib().cakeb200_last_error()
    assert 0.0015 <= waited < 0.5, waited
    big = oracle.uniform((512, 256), 3), oracle.uniform((256, 512), 4)
    ref, _ = oracle.sgemm(big[0], big[1], 8, NA)
    cake.set_option("pair", 1)
    try:
        assert rel_err(cake.cake_sgemm(*big, kernel=cake.KERNEL_TF32X3), ref, *big) <= TOL
    finally:
        cake.set_option("pair", 0)


def test_errors_are_status_codes(cake):
    A = np.zeros((4, 4), np.float32)
    with pytest.raises(ValueError):
        cake.cake_sgemm(A, np.zeros((5, 4), np.float32))
    with pytest.raises(cake.CakeError):
        cake.cake_sgemm(A, A, sch=9)
    with pytest.raises(cake.CakeError):
        cake.cake_sgemm(A, A, kernel=17)
    with pytest.raises(cake.CakeError):
        cake.cake_sgemm_async(0, 0, 0, 4, 4, 4)
    # the library is still usable afterwards
    C = cake.cake_sgemm(np.eye(4, dtype=np.float32), np.eye(4, dtype=np.float32))
    assert np.array_equal(C, np.eye(4, dtype=np.float32))


def test_operand_planes_kept_across_products(cake):
    """An operand split once (cakeb200_planes_create, what pack_A / pack_B keep behind packedA / packedB = 1) gives
    the same bits as the product that splits it on every call, with the operand's split kernel gone from the call."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(9)
    for (M, K, N) in [(1000, 515, 777), (2048, 1024, 512), (130, 36, 140)]:
        A = torch.rand((M, K), device="cuda", generator=g) * 2 - 1
        B = torch.rand((K, N), device="cuda", generator=g) * 2 - 1
        want = cake.cake_sgemm(A, B, kernel=cake.KERNEL_TF32X3)
        base = cake.last_stats()["launches"]
        pa, pb = cake.Planes(A), cake.Planes(B, is_b=True)
        try:
            assert torch.equal(cake.cake_sgemm_planes(pa, B), want) and cake.last_stats()["launches"] == base - 1
            assert torch.equal(cake.cake_sgemm_planes(A, pb), want) and cake.last_stats()["launches"] == base - 1
            C = torch.full((M, N), float("nan"), device="cuda")
            assert torch.equal(cake.cake_sgemm_planes(pa, pb, C), want) and cake.last_stats()["launches"] == base - 2
            # host matrices work too, and planes of the wrong operand or shape are refused
            assert np.array_equal(cake.cake_sgemm_planes(A.cpu().numpy(), pb), want.cpu().numpy())
            with pytest.raises(cake.CakeError):
                cake.cake_sgemm_planes(pb, B)
        finally:
            pa.close()
            pb.close()
