"""B200 implementation of the CAKE SGEMM path (vnatesh/CAKE_on_CPU).

The arithmetic lives in hand-written sm_100a CUDA kernels inside
``libcake_b200.so`` (built in-tree by ``cake_on_cpu_b200.build``).  This module
binds the library's C ABI (``include/cake_b200.h``) with ctypes and exposes the
operator interface of the reference under the reference's own names:
``cake_sgemm`` with its ``sch`` / ``beta`` / ``p`` arguments
(reference include/cake.h:12-14), ``init_block_dims`` / ``derive_schedule`` /
``set_schedule`` (include/tiling.h), ``pack_A`` / ``pack_B`` / ``pack_C`` /
``unpack_C`` and the packed sizes (include/packing.h).

Matrices may be numpy float32 arrays (host memory), CPU torch tensors, or CUDA
torch tensors (device memory, used in place).  There is no CPU fallback: if the
shared library is missing, importing the operators raises.
"""
from .api import (  # noqa: F401
    KMN, MKN, NKM, NA, KERNEL_AUTO, KERNEL_TF32X3, KERNEL_FFMA,
    BlkDims, Cntx, CakeError, Stats,
    cake_sgemm, cake_sgemm_ex, cake_sgemv, cake_sgemm_async, cake_sgemm_batched, cake_sp_sgemm, cake_conv2d, conv_plan, im2col,
    cake_query_cntx, init_block_dims, derive_schedule, set_schedule,
    cake_sgemm_packed_A_size, cake_sgemm_packed_B_size, cake_sgemm_packed_C_size,
    pack_A, pack_B, pack_C, unpack_C, unpack_A, unpack_B,
    device_count, last_stats, lib, library_path, cake_sgemm_noalloc, NOALLOC_SCRATCH_BYTES, profile_begin, profile_end, tf32_peak, select_devices, set_option, get_option, Planes, cake_sgemm_planes, tune, tune_search, tune_search_shape, tune_put, tune_get, tune_clear, tune_save, tune_load,
)
