"""ctypes binding of include/cake_b200.h and the reference-shaped operators."""
import ctypes
import os

import numpy as np

KMN, MKN, NKM, NA = 0, 1, 2, 3
KERNEL_AUTO, KERNEL_TF32X3, KERNEL_FFMA = 0, 1, 2

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libcake_b200.so")
_lib = None

_fp = ctypes.POINTER(ctypes.c_float)
_i, _vp, _sz = ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t


class CakeError(RuntimeError):
    """A C-ABI call returned a negative status."""

    def __init__(self, code, text):
        super().__init__("cake_b200 status %d: %s" % (code, text))
        self.code = code


class Stats(ctypes.Structure):
    """cakeb200_stats: timings (ms, CUDA events) and choices of the last call."""
    _fields_ = [("ms_h2d", ctypes.c_float), ("ms_prepass", ctypes.c_float), ("ms_gemm", ctypes.c_float),
                ("ms_d2h", ctypes.c_float), ("kernel", _i), ("sched", _i), ("tile_m", _i), ("tile_n", _i),
                ("tile_k", _i), ("launches", _i)]

    def as_dict(self):
        return {k: getattr(self, k) for k, _ in self._fields_}


class ConvPlan(ctypes.Structure):
    """cakeb200_conv_plan: how a convolution is laid out on the tensor-core path."""
    _fields_ = [(n, _i) for n in ("route", "tiles", "channel_tile", "positions_tile", "k_slices", "stages", "ring", "smem_bytes")]

    def as_dict(self):
        return {k: getattr(self, k) for k, _ in self._fields_}


class Cntx(ctypes.Structure):
    """cakeb200_cntx: the fields of cake_cntx_t the block-sizing formulas read
    (reference include/common.h:138-151)."""
    _fields_ = [("alpha_n", ctypes.c_double), ("mr", _i), ("nr", _i), ("L1", _i), ("L2", _i), ("L3", _i),
                ("ncores", _i)]

    @classmethod
    def make(cls, L1, L2, L3, ncores, mr=6, nr=16):
        c = cls()
        c.alpha_n, c.mr, c.nr, c.L1, c.L2, c.L3, c.ncores = 1.0, mr, nr, L1, L2, L3, ncores
        return c


class BlkDims(ctypes.Structure):
    """cakeb200_blk_dims == blk_dims_t (reference include/common.h:108-135)."""
    _names = ["m_c", "k_c", "n_c", "m_c1", "k_c1", "n_c1", "m_c1_last_core", "n_c1_last_core", "k_c1_last_core",
              "mr_rem", "nr_rem", "k_rem", "p_l", "pm_l", "pn_l", "pm", "pn", "m_pad", "k_pad", "n_pad", "Mb", "Kb",
              "Nb", "M_padded", "N_padded", "sch"]
    _fields_ = [(n, _i) for n in _names]

    def as_dict(self):
        return {n: getattr(self, n) for n in self._names}


_SIGNATURES = {
    "cakeb200_last_error": (ctypes.c_char_p, []),
    "cakeb200_get_stats": (None, [ctypes.POINTER(Stats)]),
    "cakeb200_device_count": (_i, []),
    "cakeb200_query_cntx": (_i, [ctypes.POINTER(Cntx)]),
    "cakeb200_sgemm": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "cakeb200_sgemm_after": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp]),
    "cakeb200_sgemm_async": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "cakeb200_sgemm_batched": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "cakeb200_sp_sgemm": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "cakeb200_conv2d": (_i, [_vp, _vp, _vp] + [_i] * 10 + [_vp]),
    "cakeb200_im2col": (_i, [_vp, _vp] + [_i] * 8 + [_vp]),
    "cakeb200_init_block_dims": (_i, [_i, _i, _i, _i, ctypes.POINTER(BlkDims), ctypes.POINTER(Cntx), _i, _i, _i, _i]),
    "cakeb200_derive_schedule": (_i, [_i, _i, _i, _i, _i, ctypes.POINTER(Cntx)]),
    "cakeb200_set_schedule": (_i, [_i, _i, _i, _i]),
    "cakeb200_packed_A_size": (_sz, [_i, _i, _i, ctypes.POINTER(BlkDims), ctypes.POINTER(Cntx), _i]),
    "cakeb200_packed_B_size": (_sz, [_i, _i, _i, ctypes.POINTER(BlkDims), ctypes.POINTER(Cntx)]),
    "cakeb200_packed_C_size": (_sz, [_i, _i, _i, ctypes.POINTER(BlkDims), ctypes.POINTER(Cntx), _i]),
}
for _n in ("pack_A", "unpack_A", "pack_B", "unpack_B", "pack_C", "unpack_C"):
    _SIGNATURES["cakeb200_" + _n] = (_i, [_vp, _vp, _i, _i, _i, ctypes.POINTER(BlkDims), ctypes.POINTER(Cntx), _vp])

_SIGNATURES["cakeb200_profile_begin"] = (_i, [])
_SIGNATURES["cakeb200_profile_end"] = (_i, [ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_float), ctypes.POINTER(_i)])
_SIGNATURES["cakeb200_sgemm_ex"] = (_i, [_vp, _i, _i, _vp, _i, _i, _vp, _i, _i, _i, _i, _vp, _i, _i, _i, _vp])
_SIGNATURES["cakeb200_conv_plan_query"] = (_i, [_i] * 10 + [ctypes.POINTER(ConvPlan)])
_SIGNATURES["cakeb200_selftest_bounded_wait"] = (_i, [_i, _vp])
_SIGNATURES["cakeb200_selftest_bounded_wait_pair"] = (_i, [_i, _vp])
_pi = ctypes.POINTER(_i)
_SIGNATURES["cakeb200_kshard_rows"] = (_i, [_i, _i, _i, _pi, _pi])
_SIGNATURES["cakeb200_kshard_supported"] = (_i, [_i, _i, _i, _i])
_SIGNATURES["cakeb200_kshard_create"] = (_i, [_i, _i, _i, _i, ctypes.POINTER(_vp), _vp])
_SIGNATURES["cakeb200_kshard_connect_ipc"] = (_i, [_vp, _vp])
_SIGNATURES["cakeb200_kshard_connect_local"] = (_i, [_vp, ctypes.POINTER(_vp)])
_SIGNATURES["cakeb200_kshard_partial"] = (_i, [_vp, _vp, _i, _vp, _i, _i, _vp])
_SIGNATURES["cakeb200_kshard_finish"] = (_i, [_vp, _vp, _i, _vp])
_SIGNATURES["cakeb200_kshard_destroy"] = (_i, [_vp])
_SIGNATURES["cakeb200_sgemv"] = (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _vp])
_pf = ctypes.POINTER(ctypes.c_float)
_SIGNATURES["cakeb200_tf32_peak"] = (_i, [ctypes.c_float, _pf, _pf, _vp])
_SIGNATURES["cakeb200_planes_create"] = (_i, [_vp, _i, _i, _i, ctypes.POINTER(_vp), _vp])
_SIGNATURES["cakeb200_planes_destroy"] = (_i, [_vp])
_SIGNATURES["cakeb200_sgemm_planes"] = (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp])
TUNE_COST = ctypes.CFUNCTYPE(ctypes.c_double, _i, _i, _i, _vp)
TUNE_COST_SHAPE = ctypes.CFUNCTYPE(ctypes.c_double, _i, _i, _i, _i, _vp)
_SIGNATURES["cakeb200_tune"] = (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp])
_SIGNATURES["cakeb200_tune_search"] = (_i, [_i, _i, _i, _i, _i, ctypes.c_ulonglong, TUNE_COST, _vp, _pi, _pi, _pi, _pf, _pi])
_SIGNATURES["cakeb200_tune_put"] = (_i, [_i, _i, _i, _i, _i, _i, _i, ctypes.c_float])
_SIGNATURES["cakeb200_tune_get"] = (_i, [_i, _i, _i, _i, _pi, _pi, _pi, _pf])
_SIGNATURES["cakeb200_tune_search_shape"] = (_i, [_i, _i, _i, _i, _i, ctypes.c_ulonglong, TUNE_COST_SHAPE, _vp, _pi, _pi, _pi, _pi, _pf, _pi])
_SIGNATURES["cakeb200_tune_put_shape"] = (_i, [_i, _i, _i, _i, _i, _i, _i, _i, ctypes.c_float])
_SIGNATURES["cakeb200_tune_get_shape"] = (_i, [_i, _i, _i, _i, _pi, _pi, _pi, _pi, _pf])
_SIGNATURES["cakeb200_tune_clear"] = (_i, [])
_SIGNATURES["cakeb200_tune_save"] = (_i, [ctypes.c_char_p])
_SIGNATURES["cakeb200_tune_load"] = (_i, [ctypes.c_char_p])
_SIGNATURES["cakeb200_set_option"] = (_i, [ctypes.c_char_p, _i])
_SIGNATURES["cakeb200_get_option"] = (_i, [ctypes.c_char_p])
_SIGNATURES["cakeb200_select_devices"] = (_i, [_pi, _i, _i, _i, _i, _i, _pi])
_SIGNATURES["cakeb200_sgemm_noalloc"] = (_i, [_vp, _vp, _vp, _i, _i, _i, _vp])

EXPORTED_SYMBOLS = sorted(_SIGNATURES)


def library_path():
    return _LIB_PATH


def lib():
    """The loaded shared library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise RuntimeError("libcake_b200.so is missing: run `python -m cake_on_cpu_b200.build` "
                               "(there is no CPU fallback)")
        L = ctypes.CDLL(_LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def _check(rc):
    if rc != 0:
        raise CakeError(rc, lib().cakeb200_last_error().decode(errors="replace"))


def last_stats():
    s = Stats()
    lib().cakeb200_get_stats(ctypes.byref(s))
    return s.as_dict()


def device_count():
    return lib().cakeb200_device_count()


def select_devices(cc_major, current, p, cap=0, M=1 << 30):
    """Device ordinals a host-pointer product with p > 1 is spread over by the C++ API
    (cakeb200_select_devices; host logic, no device needed)."""
    n = len(cc_major)
    majors = (_i * n)(*cc_major)
    out = (_i * max(n, 1))()
    got = lib().cakeb200_select_devices(majors, n, current, p, cap, M, out)
    return [out[k] for k in range(got)]


def _is_torch(x):
    return type(x).__module__.startswith("torch")


def _ptr(x):
    """Raw address of a contiguous float32 numpy array or torch tensor."""
    if _is_torch(x):
        import torch
        if x.dtype != torch.float32 or not x.is_contiguous():
            raise TypeError("expected a contiguous float32 tensor")
        return ctypes.c_void_p(x.data_ptr())
    if not isinstance(x, np.ndarray) or x.dtype != np.float32 or not x.flags["C_CONTIGUOUS"]:
        raise TypeError("expected a C-contiguous float32 array")
    return ctypes.c_void_p(x.ctypes.data)


def _empty_like_kind(ref, shape):
    if _is_torch(ref):
        import torch
        return torch.empty(shape, dtype=torch.float32, device=ref.device)
    return np.empty(shape, np.float32)


def _need_shape(x, shape, what):
    """Raise before any launch when a caller-supplied array does not have the shape the
    kernels will read or write through its raw pointer."""
    if tuple(x.shape) != tuple(shape):
        raise ValueError("%s has shape %s, expected %s" % (what, tuple(x.shape), tuple(shape)))


def _stream_of(x, stream):
    if stream is not None:
        return ctypes.c_void_p(int(stream))
    if _is_torch(x) and x.is_cuda:
        import torch
        return ctypes.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)
    return None


# ------------------------------------------------------------------ the product

def cake_sgemm(A, B, C=None, p=1, cake_cntx=None, packedA=False, packedB=False, alpha=1.0, beta=0.0, sch=NA,
               kernel=KERNEL_AUTO, stream=None, b_ready=None):
    """C = A @ B through the reference's operator interface
    (cake_sgemm, reference include/cake.h:12-14, src/cake_sgemm.cpp:9-175).

    ``alpha`` is accepted and ignored and ``beta`` is a flag, exactly as in the
    reference: K-first overwrites C, M-first / N-first add A@B to C when
    ``beta != 0``.  ``sch`` picks the tile order (NA = derive from the shape).
    ``p`` and ``cake_cntx`` are accepted for signature parity; one process
    drives one GPU here.  ``b_ready`` (a ``torch.cuda.Event`` already recorded, or a
    raw cudaEvent_t) makes the kernels wait until B is complete, see
    cakeb200_sgemm_after.  Returns C.
    """
    if packedA or packedB:
        raise NotImplementedError("pre-packed operands go through the C++ API (include/cake.h)")
    M, K = A.shape
    K2, N = B.shape
    if K != K2:
        raise ValueError("inner dimensions differ")
    if C is None:
        C = _empty_like_kind(A, (M, N))
        beta = 0.0
    _need_shape(C, (M, N), "C")
    accumulate = 1 if (beta != 0 and sch in (MKN, NKM)) else 0
    if beta != 0 and sch == NA:
        # the schedule decides whether beta is honoured; resolve it the way the library will
        accumulate = 1 if last_schedule_for(M, N, K) != KMN else 0
    if stream is None and not (_is_torch(C) and C.is_cuda) and _is_torch(B) and B.is_cuda:
        stream = _stream_of(B, None).value  # host result, device B: run on the stream that produces B
    if b_ready is not None:
        ev = ctypes.c_void_p(b_ready.cuda_event if hasattr(b_ready, "cuda_event") else int(b_ready))
        _check(lib().cakeb200_sgemm_after(_ptr(A), _ptr(B), _ptr(C), M, N, K, accumulate, sch, kernel,
                                          _stream_of(C, stream), ev))
    else:
        _check(lib().cakeb200_sgemm(_ptr(A), _ptr(B), _ptr(C), M, N, K, accumulate, sch, kernel, _stream_of(C, stream)))
    return C


def cake_sgemm_ex(A, B, C=None, trans_a=False, trans_b=False, bias=None, accumulate=False, sch=NA,
                  kernel=KERNEL_AUTO, stream=None):
    """C (+)= op(A) @ op(B) (+ bias) on CUDA tensors, enqueued on the current stream.

    ``A`` and ``B`` are 2-D float32 tensors whose rows are contiguous (a row
    stride is allowed, so column slices work); ``trans_a`` / ``trans_b`` multiply
    the transpose of the tensor as stored.  ``bias`` has one entry per column of
    C and is added in the kernel's epilogue.  This is the product behind the
    linear layer (reference src/linear.cpp:12-102) without its transposed copies.
    """
    import torch
    for t in (A, B) + ((C,) if C is not None else ()) + ((bias,) if bias is not None else ()):
        if not (_is_torch(t) and t.is_cuda and t.dtype == torch.float32):
            raise TypeError("cake_sgemm_ex needs float32 CUDA tensors")
    for t in (A, B) + ((C,) if C is not None else ()):
        if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1) or (t.shape[0] > 1 and t.stride(0) < t.shape[1]):
            raise TypeError("operands must be 2-D with contiguous rows")
    M, K = (A.shape[1], A.shape[0]) if trans_a else A.shape
    K2, N = (B.shape[1], B.shape[0]) if trans_b else B.shape
    if K != K2:
        raise ValueError("inner dimensions differ")
    if C is None:
        C = torch.empty((M, N), dtype=torch.float32, device=A.device)
        accumulate = False
    if tuple(C.shape) != (M, N):
        raise ValueError("C has the wrong shape")
    if bias is not None and (bias.dim() != 1 or bias.shape[0] != N or not bias.is_contiguous()):
        raise ValueError("bias must be a contiguous vector with one entry per column of C")
    ld = lambda t: t.stride(0) if t.shape[0] > 1 else t.shape[1]
    _check(lib().cakeb200_sgemm_ex(ctypes.c_void_p(A.data_ptr()), ld(A), int(trans_a), ctypes.c_void_p(B.data_ptr()), ld(B),
                                   int(trans_b), ctypes.c_void_p(C.data_ptr()), ld(C), M, N, K,
                                   ctypes.c_void_p(bias.data_ptr()) if bias is not None else None,
                                   int(bool(accumulate)), sch, kernel, _stream_of(C, stream)))
    return C


def last_schedule_for(M, N, K):
    """Schedule the library derives for a shape on the current device."""
    c = cake_query_cntx()
    c.ncores = 1
    return init_block_dims(M, N, K, 1, c, NA).sch


def cake_sgemm_async(dA, dB, dC, M, N, K, accumulate=0, sch=NA, kernel=KERNEL_AUTO, stream=0):
    """Enqueue C = A @ B on ``stream`` for raw device addresses; no synchronisation."""
    _check(lib().cakeb200_sgemm_async(ctypes.c_void_p(dA), ctypes.c_void_p(dB), ctypes.c_void_p(dC), M, N, K,
                                      accumulate, sch, kernel, ctypes.c_void_p(stream)))


def cake_sgemm_batched(A, B, C=None, kernel=KERNEL_AUTO, stream=None):
    """Batch of independent products, A[b] @ B[b] (the reference's small-matrix
    path, reference include/cake.h:52-72, is one cake_sgemm per item)."""
    batch, M, K = A.shape
    _, _, N = B.shape
    _need_shape(B, (batch, K, N), "B")
    if C is None:
        C = _empty_like_kind(A, (batch, M, N))
    _need_shape(C, (batch, M, N), "C")
    _check(lib().cakeb200_sgemm_batched(_ptr(A), _ptr(B), _ptr(C), M, N, K, batch, kernel, _stream_of(C, stream)))
    return C


def cake_sgemv(A, x, y=None, col_major=False, accumulate=False, stream=None):
    """y (+)= A x (cake_sgemv of reference examples/cake_gemv.cpp:716-765).  ``col_major``: A is given as
    the (K, M) array whose element [k, m] is A[m, k], the reference driver's layout; otherwise A is (M, K)."""
    if col_major:
        K, M = A.shape
    else:
        M, K = A.shape
    if (x.numel() if _is_torch(x) else x.size) != K:
        raise ValueError("vector length differs from the matrix")
    if y is None:
        y = _empty_like_kind(A, (M,))
        accumulate = False
    if (y.numel() if _is_torch(y) else y.size) != M:
        raise ValueError("y has %d elements, expected %d" % ((y.numel() if _is_torch(y) else y.size), M))
    _check(lib().cakeb200_sgemv(_ptr(A), _ptr(x), _ptr(y), M, K, int(bool(col_major)), int(bool(accumulate)),
                                _stream_of(y, stream)))
    return y


def cake_sp_sgemm(A, B, C=None, kernel=KERNEL_FFMA, stream=None):
    """C = A @ B for a mostly-zero A (row-skipping product of the reference's
    sparse microkernel, reference src/kernels/haswell/sparse.cpp:7-131)."""
    M, K = A.shape
    K2, N = B.shape
    if K != K2:
        raise ValueError("inner dimensions differ")
    if C is None:
        C = _empty_like_kind(A, (M, N))
    _need_shape(C, (M, N), "C")
    _check(lib().cakeb200_sp_sgemm(_ptr(A), _ptr(B), _ptr(C), M, N, K, kernel, _stream_of(C, stream)))
    return C


def cake_conv2d(x, w, stride=1, pad=0, out=None, kernel=KERNEL_AUTO, stream=None):
    """NCHW convolution via im2col + SGEMM (reference examples/cake_conv.cpp:1007-1066)."""
    b, cin, H, W = x.shape
    cout, cin2, hf, wf = w.shape
    if cin != cin2:
        raise ValueError("channel mismatch")
    Ho, Wo = (H + 2 * pad - hf) // stride + 1, (W + 2 * pad - wf) // stride + 1
    if out is None:
        out = _empty_like_kind(x, (b, cout, Ho, Wo))
    _need_shape(out, (b, cout, Ho, Wo), "out")
    _check(lib().cakeb200_conv2d(_ptr(x), _ptr(w), _ptr(out), b, cin, H, W, cout, hf, wf, stride, pad, kernel,
                                 _stream_of(out, stream)))
    return out


def conv_plan(batch, cin, H, W, cout, hf, wf, stride=1, pad=0, sm_count=148):
    """Route and tiling cake_conv2d takes on the tensor-core path (host logic, no device needed)."""
    out = ConvPlan()
    _check(lib().cakeb200_conv_plan_query(batch, cin, H, W, cout, hf, wf, stride, pad, sm_count, ctypes.byref(out)))
    return out.as_dict()


def im2col(x, hf, wf, stride=1, pad=0, stream=None):
    """im_2_col (reference examples/cake_conv.cpp:1178-1213) with batch and padding."""
    b, cin, H, W = x.shape
    Ho, Wo = (H + 2 * pad - hf) // stride + 1, (W + 2 * pad - wf) // stride + 1
    col = _empty_like_kind(x, (cin * hf * wf, b * Ho * Wo))
    _check(lib().cakeb200_im2col(_ptr(x), _ptr(col), b, cin, H, W, hf, wf, stride, pad, _stream_of(col, stream)))
    return col


# ------------------------------------------------------- context and tiling

def cake_query_cntx():
    c = Cntx()
    _check(lib().cakeb200_query_cntx(ctypes.byref(c)))
    return c


def init_block_dims(M, N, K, p, cake_cntx, sch=NA, mcu=0, kcu=0, ncu=0):
    x = BlkDims()
    _check(lib().cakeb200_init_block_dims(M, N, K, p, ctypes.byref(x), ctypes.byref(cake_cntx), sch, mcu, kcu, ncu))
    return x


def derive_schedule(M, N, K, p, mc_ret, cake_cntx):
    return lib().cakeb200_derive_schedule(M, N, K, p, mc_ret, ctypes.byref(cake_cntx))


def set_schedule(sch, M, N, K):
    return lib().cakeb200_set_schedule(sch, M, N, K)


def cake_sgemm_packed_A_size(M, K, p, x, cake_cntx, sch):
    return lib().cakeb200_packed_A_size(M, K, p, ctypes.byref(x), ctypes.byref(cake_cntx), sch)


def cake_sgemm_packed_B_size(K, N, p, x, cake_cntx):
    return lib().cakeb200_packed_B_size(K, N, p, ctypes.byref(x), ctypes.byref(cake_cntx))


def cake_sgemm_packed_C_size(M, N, p, x, cake_cntx, sch):
    return lib().cakeb200_packed_C_size(M, N, p, ctypes.byref(x), ctypes.byref(cake_cntx), sch)


# ------------------------------------------------------------------ packing

def _pack(name, mat, packed, d0, d1, p, x, cake_cntx, stream):
    fn = getattr(lib(), "cakeb200_" + name)
    _need_shape(mat, (d0, d1), "matrix")
    kind = name[-1]
    want = (cake_sgemm_packed_A_size(d0, d1, p, x, cake_cntx, x.sch) if kind == "A" else
            cake_sgemm_packed_B_size(d0, d1, p, x, cake_cntx) if kind == "B" else
            cake_sgemm_packed_C_size(d0, d1, p, x, cake_cntx, x.sch)) // 4
    have = packed.numel() if _is_torch(packed) else packed.size
    if have < want:
        raise ValueError("packed buffer holds %d floats, the layout needs %d" % (have, want))
    _check(fn(_ptr(mat), _ptr(packed), d0, d1, p, ctypes.byref(x), ctypes.byref(cake_cntx), _stream_of(packed, stream)))


def pack_A(A, M, K, p, x, cake_cntx, A_p=None, stream=None):
    if A_p is None:
        A_p = _empty_like_kind(A, (cake_sgemm_packed_A_size(M, K, p, x, cake_cntx, x.sch) // 4,))
    _pack("pack_A", A, A_p, M, K, p, x, cake_cntx, stream)
    return A_p


def pack_B(B, K, N, p, x, cake_cntx, B_p=None, stream=None):
    if B_p is None:
        B_p = _empty_like_kind(B, (cake_sgemm_packed_B_size(K, N, p, x, cake_cntx) // 4,))
    _pack("pack_B", B, B_p, K, N, p, x, cake_cntx, stream)
    return B_p


def pack_C(C, M, N, p, x, cake_cntx, C_p=None, stream=None):
    if C_p is None:
        C_p = _empty_like_kind(C, (cake_sgemm_packed_C_size(M, N, p, x, cake_cntx, x.sch) // 4,))
    _pack("pack_C", C, C_p, M, N, p, x, cake_cntx, stream)
    return C_p


def unpack_C(C_p, M, N, p, x, cake_cntx, C=None, stream=None):
    if C is None:
        C = _empty_like_kind(C_p, (M, N))
    _pack("unpack_C", C, C_p, M, N, p, x, cake_cntx, stream)
    return C


def unpack_A(A_p, M, K, p, x, cake_cntx, A=None, stream=None):
    if A is None:
        A = _empty_like_kind(A_p, (M, K))
    _pack("unpack_A", A, A_p, M, K, p, x, cake_cntx, stream)
    return A


def unpack_B(B_p, K, N, p, x, cake_cntx, B=None, stream=None):
    if B is None:
        B = _empty_like_kind(B_p, (K, N))
    _pack("unpack_B", B, B_p, K, N, p, x, cake_cntx, stream)
    return B


NOALLOC_SCRATCH_BYTES = 17 << 20


def cake_sgemm_noalloc(A, B, C=None, stream=None):
    """C = A @ B for callers that must not allocate device memory (embedded in
    another framework's memory pool, fixed memory budget, plug-ins that are only
    handed buffers).  CUDA tensors only; the scratch is a fixed 17 MiB array in
    the library, so shapes are limited (1024 x 1024 x 1024 fits) and calls that
    overlap on the GPU race on it.  The first call on a device should happen
    outside any stream capture.  Pass ``C`` to keep the call itself free of
    allocations on the Python side as well."""
    if not (_is_torch(A) and A.is_cuda and _is_torch(B) and B.is_cuda):
        raise TypeError("cake_sgemm_noalloc takes CUDA tensors")
    M, K = A.shape
    K2, N = B.shape
    if K != K2:
        raise ValueError("inner dimensions differ")
    if C is None:
        C = _empty_like_kind(A, (M, N))
    if not (_is_torch(C) and C.is_cuda):
        raise TypeError("cake_sgemm_noalloc takes CUDA tensors")
    _need_shape(C, (M, N), "C")
    _check(lib().cakeb200_sgemm_noalloc(_ptr(A), _ptr(B), _ptr(C), M, N, K, _stream_of(C, stream)))
    return C


IPC_HANDLE_BYTES = 64


def kshard_rows(M, world, rank):
    """[lo, hi) of the rows of C that `rank` owns in a K-sharded product (whole 128-row tiles)."""
    lo, hi = _i(), _i()
    _check(lib().cakeb200_kshard_rows(M, world, rank, ctypes.byref(lo), ctypes.byref(hi)))
    return lo.value, hi.value


def kshard_supported(M, N, K_local, sm_count=0):
    """Whether the K-sharded exchange takes a product of this shape per rank (few tiles, deep K).
    sm_count > 0 answers without a device."""
    return bool(lib().cakeb200_kshard_supported(M, N, K_local, sm_count))


class KShard:
    """One rank's end of a product whose K is sharded over the GPUs of a box: this rank's
    partial rows go straight into the owners' memory while its tiles are summed, and the
    owner adds the slots of all ranks in rank order.  `handle` is what the other ranks
    need (64 bytes) for `connect`; `KShard.connect_local` wires objects of one process."""

    def __init__(self, world, rank, M, N):
        self.world, self.rank, self.M, self.N = world, rank, M, N
        self._h = _vp()
        buf = (ctypes.c_ubyte * IPC_HANDLE_BYTES)()
        _check(lib().cakeb200_kshard_create(world, rank, M, N, ctypes.byref(self._h), buf))
        self.handle = bytes(buf)
        self.rows = kshard_rows(M, world, rank)

    def connect(self, handles):
        """handles: the `handle` of every rank, in rank order (one bytes object of world x 64, or a list)."""
        blob = handles if isinstance(handles, (bytes, bytearray)) else b"".join(handles)
        if len(blob) != self.world * IPC_HANDLE_BYTES:
            raise ValueError("expected one 64-byte handle per rank")
        arr = (ctypes.c_ubyte * len(blob)).from_buffer_copy(blob)
        _check(lib().cakeb200_kshard_connect_ipc(self._h, arr))

    @staticmethod
    def connect_local(objects):
        arr = (_vp * len(objects))(*[o._h.value for o in objects])
        for o in objects:
            _check(lib().cakeb200_kshard_connect_local(o._h, arr))

    def partial(self, A_k, B_k, stream=None):
        """A_k: this rank's columns of A (M x Kr, rows may be strided), B_k: the same rows of B (Kr x N)."""
        if A_k.stride(1) != 1 or B_k.stride(1) != 1:
            raise TypeError("operands need unit stride along their rows")
        M, Kr = A_k.shape
        if (M, B_k.shape[0], B_k.shape[1]) != (self.M, Kr, self.N):
            raise ValueError("operand shapes do not match this product")
        _check(lib().cakeb200_kshard_partial(self._h, _vp(A_k.data_ptr()), A_k.stride(0), _vp(B_k.data_ptr()), B_k.stride(0),
                                             Kr, _stream_of(A_k, stream)))

    def finish(self, out=None, wait_limit_us=0, stream=None):
        """This rank's rows of C (rows[0]:rows[1]); blocks until they are complete."""
        import torch
        lo, hi = self.rows
        if out is None:
            out = torch.empty((hi - lo, self.N), dtype=torch.float32, device="cuda")
        if out.numel() != (hi - lo) * self.N:
            raise ValueError("out has %d elements, expected %d" % (out.numel(), (hi - lo) * self.N))
        _check(lib().cakeb200_kshard_finish(self._h, _ptr(out), wait_limit_us, _stream_of(out, stream)))
        return out

    def close(self):
        if self._h:
            lib().cakeb200_kshard_destroy(self._h)
            self._h = _vp()


def tf32_peak(ms_target=0.0, stream=None):
    """(TFLOP/s, ms): measured dense TF32 issue rate of the current device (cakeb200_tf32_peak)."""
    t, ms = ctypes.c_float(), ctypes.c_float()
    _check(lib().cakeb200_tf32_peak(ms_target, ctypes.byref(t), ctypes.byref(ms), ctypes.c_void_p(int(stream)) if stream else None))
    return t.value, ms.value


class Planes:
    """An operand split once into its TF32 hi / lo planes and kept on the device (cakeb200_planes_create):
    the counterpart of an operand packed once with pack_A / pack_B and passed with packedA / packedB = 1.
    ``Planes(A)`` for the left operand (M x K), ``Planes(B, is_b=True)`` for the right one (K x N)."""

    def __init__(self, mat, is_b=False, stream=None):
        r, c = mat.shape
        self.rows, self.K, self.is_b = (c, r, True) if is_b else (r, c, False)
        self._h = _vp()
        _check(lib().cakeb200_planes_create(_ptr(mat), self.rows, self.K, int(is_b), ctypes.byref(self._h), _stream_of(mat, stream)))

    def close(self):
        if self._h:
            lib().cakeb200_planes_destroy(self._h)
            self._h = _vp()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def cake_sgemm_planes(A, B, C=None, sch=NA, accumulate=False, stream=None):
    """C (+)= A @ B where A and / or B is a ``Planes`` object (the other a matrix): cakeb200_sgemm_planes."""
    pa, pb = isinstance(A, Planes), isinstance(B, Planes)
    if not (pa or pb):
        raise TypeError("at least one operand must be a Planes object")
    M, K = (A.rows, A.K) if pa else A.shape
    K2, N = (B.K, B.rows) if pb else B.shape
    if K != K2:
        raise ValueError("inner dimensions differ")
    if C is None:
        if pa and pb:
            raise ValueError("give C when both operands are planes")
        C = _empty_like_kind(B if pa else A, (M, N))
        accumulate = False
    _need_shape(C, (M, N), "C")
    _check(lib().cakeb200_sgemm_planes(A._h if pa else None, None if pa else _ptr(A), B._h if pb else None, None if pb else _ptr(B),
                                       _ptr(C), M, N, K, int(bool(accumulate)), sch, _stream_of(C, stream)))
    return C


def tune(A, B, C=None, sch=NA, trials=24, stream=None):
    """Search the tile shape of the large-matrix kernel for this product's shape on the device and
    remember the winner (cakeb200_tune).  Returns the winning entry as a dict."""
    M, K = A.shape
    K2, N = B.shape
    if K != K2:
        raise ValueError("inner dimensions differ")
    if C is None:
        C = _empty_like_kind(A, (M, N))
    _need_shape(C, (M, N), "C")
    _check(lib().cakeb200_tune(_ptr(A), _ptr(B), _ptr(C), M, N, K, sch, trials, _stream_of(C, stream)))
    st = last_stats()
    return dict(tune_get(M, N, K, st["sched"]), evaluated=st["launches"])


def tune_search(M, N, K, cost, sm_count=148, trials=24, seed=1):
    """The search alone with a Python cost function cost(tile_n, band, k_pieces) -> ms (<= 0: invalid point)."""
    cb = TUNE_COST(lambda w, b, p, _user: float(cost(w, b, p)))
    w, b, p, n, ms = _i(), _i(), _i(), _i(), ctypes.c_float()
    _check(lib().cakeb200_tune_search(M, N, K, sm_count, trials, seed, cb, None, ctypes.byref(w), ctypes.byref(b), ctypes.byref(p),
                                      ctypes.byref(ms), ctypes.byref(n)))
    return {"tile_n": w.value, "band": b.value, "k_pieces": p.value, "ms": ms.value, "evaluated": n.value}


def tune_search_shape(M, N, K, cost, sm_count=148, trials=24, seed=1):
    """The search over tile width, cluster shape, band and K pieces with a Python cost function
    cost(tile_n, cluster, band, k_pieces) -> ms (<= 0: invalid point); cluster 1 = pairs of SMs, 2 = single SMs."""
    cb = TUNE_COST_SHAPE(lambda w, c, b, p, _user: float(cost(w, c, b, p)))
    w, c, b, p, n, ms = _i(), _i(), _i(), _i(), _i(), ctypes.c_float()
    _check(lib().cakeb200_tune_search_shape(M, N, K, sm_count, trials, seed, cb, None, ctypes.byref(w), ctypes.byref(c), ctypes.byref(b),
                                            ctypes.byref(p), ctypes.byref(ms), ctypes.byref(n)))
    return {"tile_n": w.value, "cluster": c.value, "band": b.value, "k_pieces": p.value, "ms": ms.value, "evaluated": n.value}


def tune_put(M, N, K, sch, tile_n, band, k_pieces, ms=0.0, cluster=0):
    """Record a choice for a shape; ``cluster`` 0 = the rule, 1 = pairs of SMs, 2 = single SMs."""
    _check(lib().cakeb200_tune_put_shape(M, N, K, sch, tile_n, cluster, band, k_pieces, ms))


def tune_get(M, N, K, sch):
    w, c, b, p, ms = _i(), _i(), _i(), _i(), ctypes.c_float()
    if not lib().cakeb200_tune_get_shape(M, N, K, sch, ctypes.byref(w), ctypes.byref(c), ctypes.byref(b), ctypes.byref(p), ctypes.byref(ms)):
        return None
    return {"tile_n": w.value, "cluster": c.value, "band": b.value, "k_pieces": p.value, "ms": ms.value}


def tune_clear():
    _check(lib().cakeb200_tune_clear())


def tune_save(path):
    n = lib().cakeb200_tune_save(str(path).encode())
    if n < 0:
        _check(n)
    return n


def tune_load(path):
    n = lib().cakeb200_tune_load(str(path).encode())
    if n < 0:
        _check(n)
    return n


def set_option(name, value):
    """Override one choice of the large-matrix kernel (cakeb200_set_option); 0 restores the rule."""
    _check(lib().cakeb200_set_option(name.encode(), int(value)))


def get_option(name):
    return lib().cakeb200_get_option(name.encode())


def profile_begin():
    """Start device-side timing of the asynchronous products that follow (see cakeb200_profile_begin)."""
    _check(lib().cakeb200_profile_begin())


def profile_end():
    """(ms_prepass, ms_kernel, calls) summed over the products since profile_begin()."""
    pre, ker, n = ctypes.c_float(), ctypes.c_float(), ctypes.c_int()
    _check(lib().cakeb200_profile_end(ctypes.byref(pre), ctypes.byref(ker), ctypes.byref(n)))
    return pre.value, ker.value, n.value
