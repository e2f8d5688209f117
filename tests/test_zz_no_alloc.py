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


def test_size_limit_follows_the_documented_formula(cake):
    """The header's examples, in the function's own (M, N, K) order: 2048 x 1024 x 512 fits the 17 MiB array,
    2048 x 512 x 1024 does not (A's planes alone take 16 MiB)."""
    import torch
    torch.cuda.set_device(0)
    M, N, K = 2048, 1024, 512
    A = torch.rand((M, K), device="cuda") * 2 - 1
    B = torch.rand((K, N), device="cuda") * 2 - 1
    C = cake.cake_sgemm_noalloc(A, B, torch.empty((M, N), device="cuda"))
    assert _norm_err(C, A.double() @ B.double(), A, B) <= TOL
    M, N, K = 2048, 512, 1024
    with pytest.raises(cake.CakeError) as e:
        cake.cake_sgemm_noalloc(torch.zeros((M, K), device="cuda"), torch.zeros((K, N), device="cuda"), torch.empty((M, N), device="cuda"))
    assert e.value.code == -5


def test_first_library_call_of_a_process_may_be_the_no_alloc_one(cake):
    """A fresh process whose very first call into the library is the no-allocation entry point: that first call
    is where the driver loads the library's module (and with it the built-in array) under CUDA's lazy loading,
    so it is the warm-up the header asks for; the second call must then leave the device's free memory alone
    and give the same bits."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = """
import torch, cake_on_cpu_b200 as cake
torch.cuda.set_device(0)
g = torch.Generator(device='cuda').manual_seed(11)
A = torch.rand((512, 384), device='cuda', generator=g) * 2 - 1
B = torch.rand((384, 640), device='cuda', generator=g) * 2 - 1
C1 = torch.empty((512, 640), device='cuda'); C2 = torch.empty((512, 640), device='cuda')
torch.cuda.synchronize()
cake.cake_sgemm_noalloc(A, B, C1)            # first call into the library in this process
free_before = torch.cuda.mem_get_info()[0]
cake.cake_sgemm_noalloc(A, B, C2)
free_after = torch.cuda.mem_get_info()[0]
exact = A.double() @ B.double()
den = A.double().norm(dim=1)[:, None] * B.double().norm(dim=0)[None, :]
err = ((C2.double() - exact).abs() / den).max().item()
print('RESULT', int(torch.equal(C1, C2)), int(free_after >= free_before), err)
"""
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300,
                       env=dict(os.environ, PYTHONPATH=root))
    line = [l for l in r.stdout.splitlines() if l.startswith("RESULT")]
    assert line, r.stderr[-2000:]
    same, no_new_memory, err = line[0].split()[1:]
    assert same == "1" and no_new_memory == "1" and float(err) <= TOL


def test_no_alloc_entry_point_on_pairs_of_sms(cake):
    """The same entry point with its tiles forced onto pairs of SMs (256-row tiles) and onto single SMs: the same
    bits, no allocation either way."""
    import torch
    M, K, N = 768, 512, 1024
    g = torch.Generator(device="cuda").manual_seed(8)
    A = torch.rand((M, K), device="cuda", generator=g) * 2 - 1
    B = torch.rand((K, N), device="cuda", generator=g) * 2 - 1
    out = {}
    try:
        for pair in (1, 2, 1):
            cake.set_option("pair", pair)
            C = torch.full((M, N), float("nan"), device="cuda")
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
            cake.cake_sgemm_noalloc(A, B, C)
            if pair in out:  # the first call of either form may load its kernels; the repeat may not take memory
                assert torch.cuda.mem_get_info()[0] >= free_before
            out[pair] = C
    finally:
        cake.set_option("pair", 0)
    assert torch.equal(out[1], out[2])
    assert _norm_err(out[1], A.double() @ B.double(), A, B) <= TOL
