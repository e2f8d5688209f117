"""ctypes bindings for the CPU oracle (oracle/liboracle.so) and, when it was
built, the unmodified reference (oracle/_ref/libcake_ref.so).

Test infrastructure: imported by tests, the smoke check and the CPU-baseline
leg of the bench only; the product package never imports it.
"""
import ctypes
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
KMN, MKN, NKM, NA = 0, 1, 2, 3
SCHED_NAMES = {KMN: "KMN", MKN: "MKN", NKM: "NKM", NA: "NA"}
BLK_FIELDS = ["m_c", "k_c", "n_c", "m_c1", "k_c1", "n_c1", "m_c1_last_core", "n_c1_last_core",
              "k_c1_last_core", "mr_rem", "nr_rem", "k_rem", "p_l", "pm_l", "pn_l", "pm", "pn",
              "m_pad", "k_pad", "n_pad", "Mb", "Kb", "Nb", "M_padded", "N_padded", "sch"]

_fp = ctypes.POINTER(ctypes.c_float)
_ip = ctypes.POINTER(ctypes.c_int)
_c_int, _c_f, _vp, _sz = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t


def _f(a):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_fp)


class OracleCntx(ctypes.Structure):
    _fields_ = [("alpha_n", ctypes.c_double), ("mr", _c_int), ("nr", _c_int), ("L1", _c_int),
                ("L2", _c_int), ("L3", _c_int), ("ncores", _c_int)]


# cache sizes of an 8-core x86 host (L1 48 KiB, L2 2 MiB, L3 105 MiB); fixed so block sizes (and with them
# the summation order) are the same wherever the tests run
DEFAULT_CACHES = (49152, 2097152, 110100480, 8)


def build_oracle():
    """Compile oracle/liboracle.so (and _ref when the reference tree is here)."""
    subprocess.run(["make", "-C", ORACLE_DIR, "all", "ref"], check=True, capture_output=True)


class Oracle:
    """The plain-C restatement."""

    def __init__(self):
        path = os.path.join(ORACLE_DIR, "liboracle.so")
        if not os.path.exists(path):
            build_oracle()
        L = self.L = ctypes.CDLL(path)
        L.oracle_cake_sgemm.argtypes = [_fp, _fp, _fp, _c_int, _c_int, _c_int, _c_int,
                                        ctypes.POINTER(OracleCntx), _c_int, _c_f, _c_int, _c_int, _c_int]
        L.oracle_cake_sgemm.restype = _c_int
        L.oracle_block_dims_flat.argtypes = [_c_int] * 4 + [ctypes.POINTER(OracleCntx)] + [_c_int] * 4 + [_ip]
        L.oracle_derive_schedule.argtypes = [_c_int] * 5 + [ctypes.POINTER(OracleCntx)]
        L.oracle_set_schedule.argtypes = [_c_int] * 4
        L.oracle_pack.argtypes = [_c_int, _fp, _fp] + [_c_int] * 4 + [ctypes.POINTER(OracleCntx), _c_int]
        L.oracle_packed_sizes.argtypes = [_c_int] * 4 + [ctypes.POINTER(OracleCntx), _c_int, ctypes.POINTER(_sz)]
        L.oracle_im2col.argtypes = [_fp, _fp] + [_c_int] * 8
        L.oracle_conv2d.argtypes = [_fp, _fp, _fp] + [_c_int] * 10 + [ctypes.POINTER(OracleCntx)]
        L.oracle_sgemm_batched.argtypes = [_fp, _fp, _fp] + [_c_int] * 5 + [ctypes.POINTER(OracleCntx)]
        L.oracle_sp_sgemm.argtypes = [_fp, _fp, _fp] + [_c_int] * 3
        L.oracle_sgemv.argtypes = [_fp, _fp, _fp] + [_c_int] * 2
        L.oracle_fill_uniform.argtypes = [_fp, _sz, ctypes.c_ulonglong]
        L.oracle_fill_normal.argtypes = [_fp, _sz, ctypes.c_ulonglong, _c_f]
        L.oracle_fill_sparse.argtypes = [_fp, _sz, ctypes.c_ulonglong, ctypes.c_ulonglong, ctypes.c_double]

    def cntx(self, caches=DEFAULT_CACHES):
        c = OracleCntx()
        self.L.oracle_cntx_init(ctypes.byref(c), *caches)
        return c

    def sgemm(self, A, B, p, sch=NA, caches=DEFAULT_CACHES, beta=0.0, C=None, blk=(0, 0, 0)):
        M, K = A.shape
        N = B.shape[1]
        C = np.zeros((M, N), np.float32) if C is None else np.ascontiguousarray(C, np.float32).copy()
        c = self.cntx(caches)
        ran = self.L.oracle_cake_sgemm(_f(A), _f(B), _f(C), M, N, K, p, ctypes.byref(c), sch, beta, *blk)
        return C, ran

    def block_dims(self, M, N, K, p, sch=NA, caches=DEFAULT_CACHES, blk=(0, 0, 0)):
        out = (ctypes.c_int * 26)()
        c = self.cntx(caches)
        self.L.oracle_block_dims_flat(M, N, K, p, ctypes.byref(c), sch, *blk, out)
        d = dict(zip(BLK_FIELDS, list(out)))
        d["alpha_n"] = c.alpha_n
        return d

    def derive_schedule(self, M, N, K, p, mc_ret, alpha_n, caches=DEFAULT_CACHES):
        c = self.cntx(caches)
        c.alpha_n = alpha_n
        return self.L.oracle_derive_schedule(M, N, K, p, mc_ret, ctypes.byref(c))

    def set_schedule(self, sch, M, N, K):
        return self.L.oracle_set_schedule(sch, M, N, K)

    def packed_sizes(self, M, N, K, p, sch, caches=DEFAULT_CACHES):
        out = (_sz * 3)()
        c = self.cntx(caches)
        self.L.oracle_packed_sizes(M, N, K, p, ctypes.byref(c), sch, out)
        return tuple(int(v) for v in out)

    def pack(self, which, src, M, N, K, p, sch, caches=DEFAULT_CACHES, out_elems=None):
        """which: 0 A, 1 B, 2 C, 3 unpack C (src packed, returns M x N)."""
        sizes = self.packed_sizes(M, N, K, p, sch, caches)
        if which == 3:
            dst = np.zeros((M, N), np.float32)
        else:
            dst = np.zeros(sizes[which] // 4, np.float32)
        c = self.cntx(caches)
        self.L.oracle_pack(which, _f(np.ascontiguousarray(src, np.float32)), _f(dst), M, N, K, p, ctypes.byref(c), sch)
        return dst

    def im2col(self, x, hf, wf, stride, pad):
        b, cin, H, W = x.shape
        Ho, Wo = (H + 2 * pad - hf) // stride + 1, (W + 2 * pad - wf) // stride + 1
        col = np.zeros((cin * hf * wf, b * Ho * Wo), np.float32)
        self.L.oracle_im2col(_f(x), _f(col), b, cin, H, W, hf, wf, stride, pad)
        return col

    def conv2d(self, x, w, stride, pad, p, caches=DEFAULT_CACHES):
        b, cin, H, W = x.shape
        cout, _, hf, wf = w.shape
        Ho, Wo = (H + 2 * pad - hf) // stride + 1, (W + 2 * pad - wf) // stride + 1
        out = np.zeros((b, cout, Ho, Wo), np.float32)
        c = self.cntx(caches)
        self.L.oracle_conv2d(_f(x), _f(w), _f(out), b, cin, H, W, cout, hf, wf, stride, pad, p, ctypes.byref(c))
        return out

    def sgemm_batched(self, A, B, p, caches=DEFAULT_CACHES):
        batch, M, K = A.shape
        N = B.shape[2]
        C = np.zeros((batch, M, N), np.float32)
        c = self.cntx(caches)
        self.L.oracle_sgemm_batched(_f(A), _f(B), _f(C), M, N, K, batch, p, ctypes.byref(c))
        return C

    def sp_sgemm(self, A, B):
        M, K = A.shape
        N = B.shape[1]
        C = np.zeros((M, N), np.float32)
        self.L.oracle_sp_sgemm(_f(A), _f(B), _f(C), M, N, K)
        return C

    def sgemv(self, A_colmajor, x, y0=None):
        """y0 + A x with A stored column-major as a (K, M) array (reference examples/cake_gemv.cpp)."""
        K, M = A_colmajor.shape
        y = np.zeros(M, np.float32) if y0 is None else np.array(y0, np.float32)
        self.L.oracle_sgemv(_f(A_colmajor), _f(x), _f(y), M, K)
        return y

    def uniform(self, shape, seed):
        x = np.empty(shape, np.float32)
        self.L.oracle_fill_uniform(_f(x), x.size, seed)
        return x

    def normal(self, shape, seed, sigma):
        x = np.empty(shape, np.float32)
        self.L.oracle_fill_normal(_f(x), x.size, seed, sigma)
        return x

    def sparse(self, shape, seed, mask_seed, density):
        x = np.empty(shape, np.float32)
        self.L.oracle_fill_sparse(_f(x), x.size, seed, mask_seed, density)
        return x


class Reference:
    """The unmodified reference, compiled from its own sources (oracle/_ref)."""

    PATH = os.path.join(ORACLE_DIR, "_ref", "libcake_ref.so")

    @classmethod
    def available(cls):
        return os.path.exists(cls.PATH)

    def __init__(self):
        L = self.L = ctypes.CDLL(self.PATH)
        L.ref_ctx_make.restype = _vp
        L.ref_ctx_make.argtypes = [_c_int] * 4
        L.ref_ctx_query.restype = _vp
        L.ref_ctx_get.argtypes = [_vp, _ip, ctypes.POINTER(ctypes.c_double)]
        L.ref_ctx_free.argtypes = [_vp]
        L.ref_cake_sgemm.restype = ctypes.c_double
        L.ref_cake_sgemm.argtypes = [_fp, _fp, _fp] + [_c_int] * 4 + [_vp, _c_int, _c_f] + [_c_int] * 4
        L.ref_init_block_dims.argtypes = [_c_int] * 4 + [_vp] + [_c_int] * 4 + [_ip]
        L.ref_derive_schedule.argtypes = [_c_int] * 5 + [_vp]
        L.ref_set_schedule.argtypes = [_c_int] * 4
        L.ref_packed_sizes.argtypes = [_c_int] * 4 + [_vp, _c_int, ctypes.POINTER(_sz)]
        L.ref_pack.argtypes = [_c_int, _fp, _fp] + [_c_int] * 4 + [_vp, _c_int]
        L.ref_rand_init.argtypes = [ctypes.c_uint, _fp, _c_int, _c_int]
        L.ref_checker.argtypes = [_fp, _fp, _fp] + [_c_int] * 3

    def ctx(self, caches=DEFAULT_CACHES):
        return _vp(self.L.ref_ctx_make(*caches))

    def query_ctx(self):
        ctx = _vp(self.L.ref_ctx_query())
        out = (ctypes.c_int * 6)()
        a = ctypes.c_double()
        self.L.ref_ctx_get(ctx, out, ctypes.byref(a))
        info = dict(zip(["mr", "nr", "L1", "L2", "L3", "ncores"], list(out)))
        return ctx, info

    def sgemm(self, A, B, p, sch=NA, caches=DEFAULT_CACHES, beta=0.0, C=None, blk=(0, 0, 0), variant=0, ctx=None):
        M, K = A.shape
        N = B.shape[1]
        C = np.zeros((M, N), np.float32) if C is None else np.ascontiguousarray(C, np.float32).copy()
        own = ctx is None
        ctx = self.ctx(caches) if own else ctx
        t = self.L.ref_cake_sgemm(_f(A), _f(B), _f(C), M, N, K, p, ctx, sch, beta, *blk, variant)
        if own:
            self.L.ref_ctx_free(ctx)
        return C, t

    def block_dims(self, M, N, K, p, sch=NA, caches=DEFAULT_CACHES, blk=(0, 0, 0)):
        out = (ctypes.c_int * 26)()
        ctx = self.ctx(caches)
        self.L.ref_init_block_dims(M, N, K, p, ctx, sch, *blk, out)
        o6 = (ctypes.c_int * 6)()
        a = ctypes.c_double()
        self.L.ref_ctx_get(ctx, o6, ctypes.byref(a))
        self.L.ref_ctx_free(ctx)
        d = dict(zip(BLK_FIELDS, list(out)))
        d["alpha_n"] = a.value
        return d

    def set_schedule(self, sch, M, N, K):
        return self.L.ref_set_schedule(sch, M, N, K)

    def packed_sizes(self, M, N, K, p, sch, caches=DEFAULT_CACHES):
        out = (_sz * 3)()
        ctx = self.ctx(caches)
        self.L.ref_packed_sizes(M, N, K, p, ctx, sch, out)
        self.L.ref_ctx_free(ctx)
        return tuple(int(v) for v in out)

    def pack(self, which, src, M, N, K, p, sch, caches=DEFAULT_CACHES):
        sizes = self.packed_sizes(M, N, K, p, sch, caches)
        dst = np.zeros((M, N), np.float32) if which == 3 else np.zeros(sizes[which] // 4, np.float32)
        ctx = self.ctx(caches)
        self.L.ref_pack(which, _f(np.ascontiguousarray(src, np.float32)), _f(dst), M, N, K, p, ctx, sch)
        self.L.ref_ctx_free(ctx)
        return dst

    def rand_init(self, seed, r, c):
        x = np.empty((r, c), np.float32)
        self.L.ref_rand_init(seed, _f(x), r, c)
        return x

    def checker(self, A, B, C):
        M, K = A.shape
        N = B.shape[1]
        return self.L.ref_checker(_f(A), _f(B), _f(C), N, M, K)

    IM2COL_PATH = os.path.join(ORACLE_DIR, "_ref", "libcake_ref_im2col.so")

    @classmethod
    def im2col_available(cls):
        return os.path.exists(cls.IM2COL_PATH)

    def im2col(self, x, hf, wf):
        """im_2_col of the reference's convolution example (examples/cake_conv.cpp:1178-1213): one image
        (cin, H, W), no padding, stride 1."""
        if not hasattr(self, "_im2col"):
            self._im2col = ctypes.CDLL(self.IM2COL_PATH)
            self._im2col.ref_im_2_col.argtypes = [_fp, _fp] + [_c_int] * 5
        cin, H, W = x.shape
        col = np.full((cin * hf * wf, (H - hf + 1) * (W - wf + 1)), np.nan, np.float32)
        assert self._im2col.ref_im_2_col(_f(x), _f(col), cin, H, W, hf, wf) == 0
        return col

    GEMV_PATH = os.path.join(ORACLE_DIR, "_ref", "libcake_ref_gemv.so")

    @classmethod
    def gemv_available(cls):
        return os.path.exists(cls.GEMV_PATH)

    def sgemv(self, A_colmajor, x, y0=None):
        """y0 + A x through the reference's microkernel cake_sgemv_haswell_8x8_col (examples/cake_gemv.cpp:87-140),
        eight rows at a time (oracle/ref_gemv_driver.cpp); A is the (K, M) array with A[k, m]."""
        if not hasattr(self, "_gemv"):
            self._gemv = ctypes.CDLL(self.GEMV_PATH)
            self._gemv.ref_sgemv.argtypes = [_fp, _fp, _fp, _c_int, _c_int]
        K, M = A_colmajor.shape
        y = np.zeros(M, np.float32) if y0 is None else np.array(y0, np.float32)
        assert self._gemv.ref_sgemv(_f(A_colmajor), _f(x), _f(y), M, K) == 0
        return y

    SPARSE_PATH = os.path.join(ORACLE_DIR, "_ref", "libcake_ref_sparse.so")

    @classmethod
    def sparse_available(cls):
        return os.path.exists(cls.SPARSE_PATH)

    def sp_sgemm(self, A, B):
        """C = A @ B through the reference's sparse microkernel cake_sp_sgemm_haswell_6x16
        (src/kernels/haswell/sparse.cpp:7-126), one 6 x 16 tile at a time (oracle/ref_sparse_driver.cpp)."""
        if not hasattr(self, "_sparse"):
            self._sparse = ctypes.CDLL(self.SPARSE_PATH)
            self._sparse.ref_sp_sgemm.argtypes = [_fp, _fp, _fp, _c_int, _c_int, _c_int]
        M, K = A.shape
        N = B.shape[1]
        C = np.full((M, N), np.nan, np.float32)
        assert self._sparse.ref_sp_sgemm(_f(A), _f(B), _f(C), M, N, K) == 0
        return C


def rel_err(C, C_ref, A, B):
    """max |C - C_ref| / (||A[m,:]||_2 * ||B[:,n]||_2), the parity gate of the SGEMM path."""
    ra = np.linalg.norm(A.astype(np.float64), axis=1)
    cb = np.linalg.norm(B.astype(np.float64), axis=0)
    den = np.outer(ra, cb)
    den[den == 0] = 1.0
    return float((np.abs(C.astype(np.float64) - C_ref.astype(np.float64)) / den).max())
