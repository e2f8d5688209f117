"""CPU-only checks of the product's host side: the shared library loads and
exports every symbol include/cake_b200.h declares, and the host block-sizing
code agrees with the oracle (no GPU compute is called here)."""
import ctypes
import os
import re

import numpy as np
import pytest

from _oracle import KMN, MKN, NKM, NA, DEFAULT_CACHES, BLK_FIELDS

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(cake):
    header = open(os.path.join(ROOT, "include", "cake_b200.h")).read()
    declared = sorted(set(re.findall(r"\b(cakeb200_[a-zA-Z0-9_]+)\s*\(", header)))
    assert len(declared) >= 20
    L = ctypes.CDLL(cake.library_path())
    for name in declared:
        assert hasattr(L, name), name
    from cake_on_cpu_b200.api import EXPORTED_SYMBOLS
    assert set(EXPORTED_SYMBOLS) <= set(declared)


def test_cpp_api_symbols_present(cake):
    # the C++ API keeps the reference's (mangled) names: cake_sgemm, pack_A, init_block_dims, ...
    import subprocess
    out = subprocess.run(["nm", "-D", "--defined-only", "-C", cake.library_path()], capture_output=True, text=True).stdout
    for name in ["cake_sgemm(", "cake_sgemm_online(", "cake_sgemm_2d(", "schedule_KMN(", "schedule_MKN(", "schedule_NKM(",
                 "schedule(", "set_schedule(", "cake_query_cntx(", "cake_query_cntx_torch(", "update_mr_nr(",
                 "derive_schedule(", "get_cache_dims(", "init_block_dims(", "grid_dims_2d(", "pack_A(", "pack_B(",
                 "pack_C(", "unpack_C(", "cake_sgemm_packed_A_size(", "cake_sgemm_packed_B_size(",
                 "cake_sgemm_packed_C_size(", "rand_init(", "cake_sgemm_checker(", "mat_equals(", "run_tests(",
                 "cake_gemm_small(", "cake_sgemm_2d_small(", "cake_sgemm_test(", "schedule_KMN_online(",
                 "schedule_KMN_C_unpacked(", "schedule_KMN_2d(", "schedule_KMN_2d_small(", "schedule_KMN_small(",
                 "schedule_MKN_small(", "schedule_NKM_small(", "schedule_NKM_small_A_packed(",
                 "schedule_MKN_small_B_packed(", "schedule_KMN_small_C_packed(", "init_block_dims_2d(",
                 "init_block_dims_2d_small(",
                 # both overloads of cake_gemm_small (reference include/cake.h:52-53 and :71-72)
                 "cake_gemm_small(float*, float*, float*, int,", "cake_gemm_small(float*, float*, float*, float*, float*, float*,"]:
        assert name in out, name


def test_no_gpu_means_loud_failure(cake):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    A = np.zeros((8, 8), np.float32)
    with pytest.raises(cake.CakeError):
        cake.cake_sgemm(A, A)


@pytest.mark.parametrize("p", [1, 2, 5, 8, 10])
def test_block_dims_match_oracle(cake, oracle, p):
    dims = (1, 10, 96, 111, 960, 2111, 8192)
    for M in dims:
        for K in dims:
            for N in dims:
                for sch in (KMN, MKN, NKM, NA):
                    cx = cake.Cntx.make(*DEFAULT_CACHES)
                    x = cake.init_block_dims(M, N, K, p, cx, sch).as_dict()
                    want = oracle.block_dims(M, N, K, p, sch)
                    assert {k: x[k] for k in BLK_FIELDS} == {k: want[k] for k in BLK_FIELDS}, (M, K, N, p, sch)
                    assert cx.alpha_n == want["alpha_n"]
                    xs = cake.init_block_dims(M, N, K, p, cake.Cntx.make(*DEFAULT_CACHES), sch)
                    cx2 = cake.Cntx.make(*DEFAULT_CACHES)
                    got = (cake.cake_sgemm_packed_A_size(M, K, p, xs, cx2, xs.sch),
                           cake.cake_sgemm_packed_B_size(K, N, p, xs, cx2),
                           cake.cake_sgemm_packed_C_size(M, N, p, xs, cx2, xs.sch))
                    assert got == oracle.packed_sizes(M, N, K, p, sch)


def test_benchmark_shapes_and_user_blocks(cake, oracle):
    shapes = [(3000, 3000, 3000), (8192, 8192, 8192), (32768, 32768, 32768), (65536, 1024, 1024), (1024, 1024, 65536),
              (1024, 262144, 1024), (96, 96, 96), (64, 576, 200704), (512, 2304, 12544)]
    for (M, K, N) in shapes:
        for blk in ((0, 0, 0), (48, 64, 96)):
            x = cake.init_block_dims(M, N, K, 8, cake.Cntx.make(*DEFAULT_CACHES), NA, *blk).as_dict()
            want = oracle.block_dims(M, N, K, 8, NA, blk=blk)
            assert {k: x[k] for k in BLK_FIELDS} == {k: want[k] for k in BLK_FIELDS}


def test_schedule_helpers(cake, oracle):
    for M in (1, 100, 1000, 70000):
        for N in (1, 100, 1000, 70000):
            for K in (1, 100, 1000, 300000):
                assert cake.set_schedule(NA, M, N, K) == oracle.set_schedule(NA, M, N, K)
                assert cake.set_schedule(MKN, M, N, K) == MKN
                for mc in (6, 96, 492):
                    cx = cake.Cntx.make(*DEFAULT_CACHES)
                    cx.alpha_n = 0.84
                    assert cake.derive_schedule(M, N, K, 8, mc, cx) == oracle.derive_schedule(M, N, K, 8, mc, 0.84)


def test_bad_arguments_are_reported_not_fatal(cake):
    cx = cake.Cntx.make(*DEFAULT_CACHES)
    with pytest.raises(cake.CakeError):
        cake.init_block_dims(0, 10, 10, 2, cx, NA)
    with pytest.raises(cake.CakeError):
        cake.init_block_dims(10, 10, 10, 2, cx, 7)


def test_convolution_plan_routes_and_tilings():
    """Host logic of the tensor-core convolution (no device needed): which route a geometry takes and how the
    implicit kernel tiles it.  Shared memory must stay within the 227 KB a CTA may use."""
    import cake_on_cpu_b200 as cake
    first = cake.conv_plan(64, 64, 56, 56, 64, 3, 3, 1, 1)
    assert first["route"] == 0 and first["positions_tile"] == 112 and first["channel_tile"] == 64
    assert first["tiles"] == 64 * 28 and first["k_slices"] == 2 * 9
    second = cake.conv_plan(64, 256, 14, 14, 512, 3, 3, 1, 1)
    assert second["route"] == 1 and second["tiles"] == 98 * 4 and second["channel_tile"] == 128 and second["k_slices"] == 72
    assert cake.conv_plan(4, 16, 9, 9, 8, 3, 3, 2, 0)["route"] == 2      # stride 2
    assert cake.conv_plan(1, 64, 5, 300, 8, 3, 3, 1, 1)["route"] == 2    # rows wider than a tile
    assert cake.conv_plan(2, 8, 7, 7, 16, 3, 3, 1, 1)["route"] == 2      # 49 floats per channel: not 16-byte steps
    for geometry in [(3, 8, 14, 14, 16, 3, 3, 1, 1), (2, 40, 12, 12, 130, 3, 3, 1, 1), (1, 4, 30, 80, 8, 3, 3, 1, 1),
                     (7, 20, 12, 8, 140, 3, 3, 1, 1), (1, 3, 4, 4, 1, 1, 1, 1, 0)]:
        p = cake.conv_plan(*geometry)
        assert p["route"] in (0, 1) and 0 < p["smem_bytes"] <= 227 * 1024 and p["stages"] >= 2 and p["ring"] >= 2
        assert p["positions_tile"] <= 128 and p["channel_tile"] % 16 == 0 and p["channel_tile"] <= 128
    with pytest.raises(cake.CakeError):
        cake.conv_plan(1, 1, 2, 2, 1, 3, 3, 1, 0)  # filter larger than the padded image


def test_kshard_rows_match_the_partition_module_and_shape_query_needs_no_device():
    from cake_on_cpu_b200 import api, partition
    for M in (1, 127, 128, 129, 300, 1000, 1024, 5000):
        for world in (1, 2, 3, 4, 8):
            blocks = [api.kshard_rows(M, world, r) for r in range(world)]
            assert blocks == [partition.row_block(M, world, r) for r in range(world)]
            assert blocks[0][0] == 0 and blocks[-1][1] == M
            assert all(blocks[i][1] == blocks[i + 1][0] for i in range(world - 1))
    # few tiles and a deep K: taken; many tiles or a shallow K: not
    assert api.kshard_supported(1024, 1024, 32768, sm_count=148)
    assert api.kshard_supported(512, 256, 8192, sm_count=148)
    assert not api.kshard_supported(8192, 8192, 1024, sm_count=148)
    assert not api.kshard_supported(256, 256, 256, sm_count=148)
    with pytest.raises(api.CakeError):
        api.kshard_rows(100, 9, 0)  # more ranks than the exchange has slots for


def test_wrong_shaped_outputs_are_rejected_before_any_launch(cake):
    """The wrappers hand raw pointers to the kernels, so a caller-supplied array of the wrong
    shape must be refused on the host (ValueError), not discovered by the device."""
    A = np.zeros((16, 8), np.float32)
    B = np.zeros((8, 12), np.float32)
    small = np.zeros((16, 11), np.float32)
    with pytest.raises(ValueError):
        cake.cake_sgemm(A, B, small)
    with pytest.raises(ValueError):
        cake.cake_sp_sgemm(A, B, small)
    with pytest.raises(ValueError):
        cake.cake_sp_sgemm(A, np.zeros((9, 12), np.float32))
    with pytest.raises(ValueError):
        cake.cake_sgemv(A, np.zeros(8, np.float32), np.zeros(15, np.float32))
    with pytest.raises(ValueError):
        cake.cake_sgemv(A, np.zeros(9, np.float32))
    with pytest.raises(ValueError):
        cake.cake_sgemm_batched(np.zeros((3, 16, 8), np.float32), np.zeros((3, 8, 12), np.float32),
                                np.zeros((3, 16, 11), np.float32))
    with pytest.raises(ValueError):
        cake.cake_conv2d(np.zeros((1, 2, 8, 8), np.float32), np.zeros((4, 2, 3, 3), np.float32), pad=1,
                         out=np.zeros((1, 4, 8, 7), np.float32))
    cx = cake.Cntx.make(*DEFAULT_CACHES)
    x = cake.init_block_dims(16, 12, 8, 2, cx, KMN)
    with pytest.raises(ValueError):
        cake.pack_A(A, 16, 8, 2, x, cx, A_p=np.zeros(4, np.float32))
    with pytest.raises(ValueError):
        cake.pack_A(np.zeros((15, 8), np.float32), 16, 8, 2, x, cx)


def test_device_selection_for_host_pointer_calls(cake):
    """cakeb200_select_devices: current device first, then the other sm_100 devices in ordinal order,
    bounded by p, the CAKE_NGPU cap and 512 rows of C per device."""
    from cake_on_cpu_b200.api import select_devices
    all10 = [10] * 8
    assert select_devices(all10, 0, 8) == list(range(8))
    assert select_devices(all10, 3, 4) == [3, 0, 1, 2]
    assert select_devices(all10, 3, 8, cap=2) == [3, 0]
    assert select_devices(all10, 5, 1) == [5]
    assert select_devices(all10, 0, 8, M=1500) == [0, 1]
    assert select_devices(all10, 0, 8, M=100) == [0]
    # devices of another architecture are skipped, wherever they sit
    assert select_devices([9, 10, 10, 8, 10], 2, 8) == [2, 1, 4]
    assert select_devices([9, 10], 0, 2) == [1]
    assert select_devices([], 0, 2) == []
