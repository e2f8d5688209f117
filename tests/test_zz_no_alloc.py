"""The entry point for callers that cannot allocate device memory
(cakeb200_sgemm_noalloc): called through the C ABI, twice in a row with
different operands, and compared with the regular entry point.

Collected last on purpose: a run that stops at the first failure has then
already run every other test.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
TOL = 1e-5  # max |C - C_ref| / (||A[m,:]|| ||B[:,n]||), the gate of the other GPU tests


def _norm_err(C, ref, A, B):
    den = A.double().norm(dim=1)[:, None] * B.double().norm(dim=0)[None, :]
    return ((C.double() - ref.double()).abs() / den.clamp_min(1e-30)).max().item()


def test_no_alloc_entry_point_matches_the_regular_one(cake):
    import torch
    torch.cuda.set_device(0)
    g = torch.Generator(device="cuda").manual_seed(7)
    shapes = [(1024, 1024, 1024), (777, 515, 1030)]  # second call: smaller, ragged, stale planes underneath
    outs = []
    for (M, K, N) in shapes:
        A = torch.rand((M, K), device="cuda", generator=g) * 2 - 1
        B = torch.rand((K, N), device="cuda", generator=g) * 2 - 1
        ref = torch.empty((M, N), device="cuda")
        cake.cake_sgemm(A, B, ref, kernel=cake.KERNEL_TF32X3)
        C = torch.full((M, N), float("nan"), device="cuda")
        torch.cuda.synchronize()
        before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
        cake.cake_sgemm_noalloc(A, B, C)
        assert torch.cuda.memory_allocated() == before
        assert torch.cuda.mem_get_info()[0] >= free_before  # the driver handed out no new device memory
        err = _norm_err(C, ref, A, B)
        assert err <= TOL, (M, K, N, err)
        exact = (A.double() @ B.double())
        assert _norm_err(C, exact, A, B) <= TOL
        outs.append(C)
    # repeating the first shape after the second gives the first result again, bit for bit
    M, K, N = shapes[0]
    g = torch.Generator(device="cuda").manual_seed(7)
    A = torch.rand((M, K), device="cuda", generator=g) * 2 - 1
    B = torch.rand((K, N), device="cuda", generator=g) * 2 - 1
    again = cake.cake_sgemm_noalloc(A, B, torch.empty((M, N), device="cuda"))
    assert torch.equal(again, outs[0])


def test_no_alloc_entry_point_rejects_what_it_cannot_hold(cake):
    import torch
    torch.cuda.set_device(0)
    A = torch.zeros((2048, 2048), device="cuda")
    with pytest.raises(cake.CakeError) as e:
        cake.cake_sgemm_noalloc(A, A, torch.empty((2048, 2048), device="cuda"))
    assert e.value.code == -5 and "scratch" in str(e.value)
    with pytest.raises(TypeError):
        cake.cake_sgemm_noalloc(np.zeros((4, 4), np.float32), np.zeros((4, 4), np.float32))
    # still usable afterwards
    I = torch.eye(64, device="cuda")
    assert torch.equal(cake.cake_sgemm_noalloc(I, I, torch.empty((64, 64), device="cuda")), I)
