"""ctypes binding of libvtlb200.so (the C ABI declared in include/vtlb.h).

This is the Python stand-in for the `fn C.vtlb_*` declarations a V build of vtl
would carry.  It adds nothing of its own: `Device` owns one `vtlb_ctx` and
forwards calls, turning non-zero return codes into `VtlbError`.  There is no
CPU path: if the library is missing or no B200 is present, creation fails.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libvtlb200.so")

OK, EINVAL, ECUDA, ENOMEM, ETIMEOUT, ENCCL, ESTATE = 0, -1, -2, -3, -4, -5, -6


class VtlbError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"vtlb error {code}: {msg}")
        self.code = code


class AdamTensor(C.Structure):
    _fields_ = [("d_grad", C.c_void_p), ("d_theta", C.c_void_p), ("d_m", C.c_void_p),
                ("d_v", C.c_void_p), ("n", C.c_size_t)]


_vp, _i, _sz, _d = C.c_void_p, C.c_int, C.c_size_t, C.c_double
_PROTOS = {
    "vtlb_device_count": [C.POINTER(C.c_int)],
    "vtlb_ctx_create": [_i, C.POINTER(_vp)],
    "vtlb_ctx_destroy": [_vp],
    "vtlb_sync": [_vp],
    "vtlb_check_status": [_vp, C.POINTER(C.c_uint32)],
    "vtlb_event_create": [_vp, C.POINTER(_vp)],
    "vtlb_event_record": [_vp, _vp],
    "vtlb_event_elapsed_ms": [_vp, _vp, _vp, C.POINTER(C.c_float)],
    "vtlb_event_destroy": [_vp, _vp],
    "vtlb_wait_probe": [_vp, C.c_uint64, _i],
    "vtlb_profile_gemm": [_vp, _i],
    "vtlb_profile_gemm_read": [_vp, C.POINTER(C.c_double), C.POINTER(C.c_uint64), C.POINTER(C.c_double)],
    "vtlb_profile_read_phase": [_vp, _i, C.POINTER(C.c_double), C.POINTER(C.c_uint64)],
    "vtlb_alloc": [_vp, _sz, C.POINTER(_vp)],
    "vtlb_free": [_vp, _vp],
    "vtlb_h2d": [_vp, _vp, _vp, _sz],
    "vtlb_d2h": [_vp, _vp, _vp, _sz],
    "vtlb_d2d": [_vp, _vp, _vp, _sz],
    "vtlb_memset0": [_vp, _vp, _sz],
    "vtlb_host_alloc": [_sz, C.POINTER(_vp)],
    "vtlb_host_free": [_vp],
    "vtlb_reserve_scratch": [_vp, _sz],
    "vtlb_set_small_gemm_limit": [_vp, _d],
    "vtlb_gemm_f32": [_vp, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _i],
    "vtlb_linear_fwd_f32": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "vtlb_plane_ld": [_i], "vtlb_f32_planes_worthwhile": [_vp, _i, _i, _i],
    "vtlb_split_planes_f32": [_vp, _vp, _i, _i, _vp, _vp],
    "vtlb_linear_fwd_f32_planes": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp],
    "vtlb_linear_bwd_f32_planes": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp],
    "vtlb_linear_bwd_f32": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i],
    "vtlb_bias_grad_f32_noalloc": [_vp, _vp, _i, _i, _vp],
    "vtlb_relu_fwd_f32": [_vp, _vp, _vp, _sz],
    "vtlb_relu_bwd_f32": [_vp, _vp, _vp, _vp, _sz],
    "vtlb_add_inplace_f32": [_vp, _vp, _vp, _sz],
    "vtlb_fill_f32": [_vp, _vp, C.c_float, _sz],
    "vtlb_init_uniform_f32": [_vp, _vp, _sz, C.c_float, C.c_float, C.c_uint64],
    "vtlb_init_normal_f32": [_vp, _vp, _sz, C.c_double, C.c_double, C.c_uint64],
    "vtlb_ckpt_encode_f32": [_vp, _vp, _sz, _vp],
    "vtlb_linear_i8_fwd_amax": [_vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
    "vtlb_copy_h2d_async": [_vp, _vp, _vp, _sz],
    "vtlb_sgd_step_f32": [_vp, _i, _vp, _d, _i],
    "vtlb_rmsprop_step_f32": [_vp, _i, _vp, _d, _d, _d, _d, _i],
    "vtlb_softmax_fwd_f32": [_vp, _vp, _sz, _sz, _vp],
    "vtlb_softmax_bwd_f32": [_vp, _vp, _vp, _sz, _sz, _vp],
    "vtlb_avgpool2d_fwd_f32": [_vp, _vp, _vp] + [_i] * 10,
    "vtlb_avgpool2d_bwd_f32": [_vp, _vp, _vp] + [_i] * 10,
    "vtlb_global_avgpool2d_fwd_f32": [_vp, _vp, _vp] + [_i] * 4,
    "vtlb_global_avgpool2d_bwd_f32": [_vp, _vp, _vp] + [_i] * 4,
    "vtlb_batchnorm1d_train_f32": [_vp, _vp, _i, _i, _vp, _vp, _d, _vp, _vp, _vp, _vp, _vp, _d],
    "vtlb_batchnorm1d_infer_f32": [_vp, _vp, _i, _i, _vp, _vp, _vp, _vp, _d, _vp],
    "vtlb_batchnorm1d_bwd_f32": [_vp, _vp, _vp, _i, _i, _vp, _vp, _vp, _d, _vp, _vp, _vp],
    "vtlb_copy_d2h_async": [_vp, _vp, _vp, _sz],
    "vtlb_copy_wait": [_vp, _i],
    "vtlb_gather_rows_f32": [_vp, _vp, _i, _sz, _vp, _i, _vp, _i],
    "vtlb_one_hot_f32": [_vp, _vp, _sz, _i, _vp, _i],
    "vtlb_ckpt_decode_f32": [_vp, _vp, _sz, _vp, _sz],
    "vtlb_conv2d_fwd_f32": [_vp, _vp, _vp, _vp, _vp] + [_i] * 12 + [_vp],
    "vtlb_conv2d_bwd_f32": [_vp, _vp, _vp, _vp, _vp, _vp, _vp] + [_i] * 11,
    "vtlb_conv2d_fwd_f32_dilated": [_vp, _vp, _vp, _vp, _vp] + [_i] * 14 + [_vp],
    "vtlb_conv2d_bwd_f32_dilated": [_vp, _vp, _vp, _vp, _vp, _vp, _vp] + [_i] * 13,
    "vtlb_maxpool2d_fwd_f32": [_vp, _vp, _vp, _vp] + [_i] * 10,
    "vtlb_maxpool2d_bwd_f32": [_vp, _vp, _vp, _vp, _sz, _sz],
    "vtlb_maxpool2x2_bwd_f32": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i],
    "vtlb_mse_fwd_bwd_f32": [_vp, _vp, _vp, _sz, _sz, _vp, _vp],
    "vtlb_softmax_ce_fwd_bwd_f32": [_vp, _vp, _vp, _i, _i, _i, _vp, _vp],
    "vtlb_adam_step_f32": [_vp, _i, C.POINTER(AdamTensor), _d, _d, _d, _d, _i],
    "vtlb_adamw_step_f32": [_vp, _i, C.POINTER(AdamTensor), _d, _d, _d, _d, _d, _i],
    "vtlb_i8_ld": [_i],
    "vtlb_quant_rows_i8": [_vp, _vp, _i, _i, _vp, _vp, _vp],
    "vtlb_row_absmax_f32": [_vp, _vp, _i, _i, _vp],
    "vtlb_gemm_i8_i32": [_vp, _vp, _vp, _i, _i, _i, _vp],
    "vtlb_linear_i8_fwd": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i],
    "vtlb_linear_i8_fwd_sharded_a": [_vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i],
    "vtlb_comm_unique_id": [_vp],
    "vtlb_comm_init_rank": [_vp, _i, _i, _vp],
    "vtlb_comm_destroy": [_vp],
    "vtlb_allreduce_sum_f32_async": [_vp, _vp, _sz],
    "vtlb_allreduce_max_f32_async": [_vp, _vp, _sz],
    "vtlb_allgather_async": [_vp, _vp, _vp, _sz],
    "vtlb_int8_issue_yardstick": [_vp, _i, C.POINTER(C.c_double)],
    "vtlb_comm_small_lane": [_vp],
    "vtlb_shared_alloc": [_vp, _sz, C.POINTER(_vp), _vp], "vtlb_shared_free": [_vp, _vp],
    "vtlb_shared_open": [_vp, _vp, C.POINTER(_vp)], "vtlb_shared_close": [_vp, _vp],
    "vtlb_allgather_push_async": [_vp, _vp, C.POINTER(_vp), _i, _sz],
    "vtlb_comm_wait": [_vp], "vtlb_comm_mark": [_vp, _i, _i], "vtlb_comm_wait_mark": [_vp, _i],
}

_lib = None


def load() -> C.CDLL:
    """Loads libvtlb200.so; raises if it has not been built (python -m vtl_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: run `python -m vtl_b200.build` "
                              "(there is no CPU fallback)")
        lib = C.CDLL(LIB_PATH)
        for name, args in _PROTOS.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = C.c_int
        lib.vtlb_last_error.argtypes = [_vp]
        lib.vtlb_last_error.restype = C.c_char_p
        lib.vtlb_launch_count.argtypes = [_vp]
        lib.vtlb_launch_count.restype = C.c_uint64
        lib.vtlb_stream.argtypes = [_vp]
        lib.vtlb_stream.restype = _vp
        lib.vtlb_ckpt_text_len.argtypes = [_sz]
        lib.vtlb_ckpt_text_len.restype = _sz
        _lib = lib
    return _lib


def device_count() -> int:
    n = C.c_int(0)
    load().vtlb_device_count(C.byref(n))
    return n.value


class _VtlbPlanes(C.Structure):
    _fields_ = [("hi", C.c_void_p), ("lo", C.c_void_p)]


class Planes:
    """TF32 hi / lo planes [rows, plane_ld(kdim)] of a matrix (vtlb_planes)."""

    def __init__(self, dev: "Device", rows: int, kdim: int):
        self.rows, self.kdim, self.ld = rows, kdim, dev.plane_ld(kdim)
        self.hi = dev.empty((rows, self.ld))
        self.lo = dev.empty((rows, self.ld))
        self.c = _VtlbPlanes(self.hi.ptr, self.lo.ptr)

    def numpy(self):
        """(hi, lo) without the padding columns."""
        return self.hi.numpy()[:, :self.kdim], self.lo.numpy()[:, :self.kdim]


def _pl(p):
    return C.byref(p.c) if p is not None else None


class DBuf:
    """A device allocation with a shape and dtype attached (host-side bookkeeping only)."""

    def __init__(self, dev: "Device", ptr: int, shape, dtype):
        self.dev, self.ptr, self.shape, self.dtype = dev, ptr, tuple(shape), np.dtype(dtype)

    @property
    def nbytes(self) -> int:
        return int(np.prod(self.shape, dtype=np.int64)) * self.dtype.itemsize

    @property
    def size(self) -> int:
        return int(np.prod(self.shape, dtype=np.int64))

    def numpy(self) -> np.ndarray:
        return self.dev.d2h(self)

    def free(self):
        if self.ptr:
            self.dev.free(self.ptr)
            self.ptr = 0


def _ptr(x):
    if x is None:
        return None
    if isinstance(x, DBuf):
        return x.ptr
    return x


class Device:
    """One vtlb_ctx (one GPU)."""

    def __init__(self, index: int = 0):
        self.lib = load()
        h = _vp()
        rc = self.lib.vtlb_ctx_create(index, C.byref(h))
        if rc != OK:
            raise VtlbError(rc, self.lib.vtlb_last_error(None).decode())
        self.h = h
        self.index = index

    # -- plumbing
    def _ck(self, rc: int):
        if rc != OK:
            raise VtlbError(rc, self.lib.vtlb_last_error(self.h).decode())

    def close(self):
        if getattr(self, "h", None):
            self.lib.vtlb_ctx_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def sync(self):
        self._ck(self.lib.vtlb_sync(self.h))

    def check_status(self) -> int:
        st = C.c_uint32(0)
        self._ck(self.lib.vtlb_check_status(self.h, C.byref(st)))
        return st.value

    def wait_probe(self, limit_ns: int, arrive: bool):
        self._ck(self.lib.vtlb_wait_probe(self.h, int(limit_ns), int(arrive)))

    def launch_count(self) -> int:
        return int(self.lib.vtlb_launch_count(self.h))

    def profile_gemm(self, enable: bool):
        self._ck(self.lib.vtlb_profile_gemm(self.h, int(enable)))

    def profile_gemm_read(self):
        """-> (summed GEMM kernel ms, launches, algorithmic operations) since the last read."""
        ms, n, ops = C.c_double(0), C.c_uint64(0), C.c_double(0)
        self._ck(self.lib.vtlb_profile_gemm_read(self.h, C.byref(ms), C.byref(n), C.byref(ops)))
        return ms.value, int(n.value), ops.value

    PHASES = ("gemm", "operand_split", "optimizer", "comm_wait", "elementwise")

    def profile_read_phases(self):
        """-> {phase: (summed ms, spans)} since the last profile_gemm_read (call before it)."""
        out = {}
        for i, name in enumerate(self.PHASES):
            ms, n = C.c_double(0), C.c_uint64(0)
            self._ck(self.lib.vtlb_profile_read_phase(self.h, i, C.byref(ms), C.byref(n)))
            out[name] = (ms.value, int(n.value))
        return out

    # -- events
    def event(self) -> int:
        ev = _vp()
        self._ck(self.lib.vtlb_event_create(self.h, C.byref(ev)))
        return ev.value

    def record(self, ev: int):
        self._ck(self.lib.vtlb_event_record(self.h, ev))

    def elapsed_ms(self, e0: int, e1: int) -> float:
        ms = C.c_float(0)
        self._ck(self.lib.vtlb_event_elapsed_ms(self.h, e0, e1, C.byref(ms)))
        return ms.value

    # -- memory
    def alloc(self, nbytes: int) -> int:
        p = _vp()
        self._ck(self.lib.vtlb_alloc(self.h, nbytes, C.byref(p)))
        return p.value or 0

    def free(self, ptr: int):
        self._ck(self.lib.vtlb_free(self.h, ptr))

    def empty(self, shape, dtype=np.float32) -> DBuf:
        shape = (shape,) if np.isscalar(shape) else tuple(shape)
        nbytes = int(np.prod(shape, dtype=np.int64)) * np.dtype(dtype).itemsize
        return DBuf(self, self.alloc(max(nbytes, 16)), shape, dtype)

    def zeros(self, shape, dtype=np.float32) -> DBuf:
        b = self.empty(shape, dtype)
        self._ck(self.lib.vtlb_memset0(self.h, b.ptr, max(b.nbytes, 16)))
        return b

    def to_device(self, a: np.ndarray) -> DBuf:
        a = np.ascontiguousarray(a)
        b = self.empty(a.shape, a.dtype)
        if a.nbytes:
            self._ck(self.lib.vtlb_h2d(self.h, b.ptr, a.ctypes.data, a.nbytes))
            self.sync()  # `a` may be a temporary
        return b

    def h2d_raw(self, dptr, hptr: int, nbytes: int):
        self._ck(self.lib.vtlb_h2d(self.h, _ptr(dptr), hptr, nbytes))

    def d2h_raw(self, hptr: int, dptr, nbytes: int):
        self._ck(self.lib.vtlb_d2h(self.h, hptr, _ptr(dptr), nbytes))

    def d2h(self, b: DBuf) -> np.ndarray:
        out = np.empty(b.shape, b.dtype)
        if out.nbytes:
            self._ck(self.lib.vtlb_d2h(self.h, out.ctypes.data, b.ptr, out.nbytes))
        return out

    def d2d(self, dst, src, nbytes: int):
        self._ck(self.lib.vtlb_d2d(self.h, _ptr(dst), _ptr(src), nbytes))

    def memset0(self, dst, nbytes: int):
        self._ck(self.lib.vtlb_memset0(self.h, _ptr(dst), nbytes))

    def reserve_scratch(self, nbytes: int):
        self._ck(self.lib.vtlb_reserve_scratch(self.h, nbytes))

    # -- f32
    def set_small_gemm_limit(self, max_flops: float):
        self._ck(self.lib.vtlb_set_small_gemm_limit(self.h, float(max_flops)))

    def gemm_f32(self, ta, tb, M, N, K, A, B, Cout, bias=None, relu=False):
        self._ck(self.lib.vtlb_gemm_f32(self.h, int(ta), int(tb), M, N, K, _ptr(A), _ptr(B),
                                        _ptr(Cout), _ptr(bias), int(relu)))

    def linear_fwd_f32(self, X, W, b, Y, M, N, K, relu=False, pre=None):
        self._ck(self.lib.vtlb_linear_fwd_f32(self.h, _ptr(X), _ptr(W), _ptr(b), _ptr(Y), M, N, K,
                                              int(relu), _ptr(pre)))

    def linear_bwd_f32(self, G, X, W, dX, dW, db, M, N, K):
        self._ck(self.lib.vtlb_linear_bwd_f32(self.h, _ptr(G), _ptr(X), _ptr(W), _ptr(dX),
                                              _ptr(dW), _ptr(db), M, N, K))

    # -- TF32 operand planes handed from producer to consumer (include/vtlb.h, vtlb_planes)
    def plane_ld(self, kdim: int) -> int:
        return int(self.lib.vtlb_plane_ld(int(kdim)))

    def planes(self, rows: int, kdim: int) -> "Planes":
        """Two uninitialised [rows, plane_ld(kdim)] f32 arrays (hi, lo) and their vtlb_planes struct."""
        return Planes(self, rows, kdim)

    def f32_planes_worthwhile(self, M, N, K) -> bool:
        return bool(self.lib.vtlb_f32_planes_worthwhile(self.h, M, N, K))

    def split_planes_f32(self, src, R, Ccols, rows=None, cols=None):
        self._ck(self.lib.vtlb_split_planes_f32(self.h, _ptr(src), R, Ccols, _pl(rows), _pl(cols)))

    def linear_fwd_f32_planes(self, X, W, b, Y, M, N, K, relu=False, pre=None, x_rows=None, y_rows=None, y_cols=None):
        self._ck(self.lib.vtlb_linear_fwd_f32_planes(self.h, _ptr(X), _ptr(W), _ptr(b), _ptr(Y), M, N, K, int(relu),
                                                     _ptr(pre), _pl(x_rows), _pl(y_rows), _pl(y_cols)))

    def linear_bwd_f32_planes(self, G, X, W, dX, dW, db, M, N, K, g_rows=None, g_cols=None, x_cols=None,
                              relu_mask_src=None, dx_rows=None, dx_cols=None):
        self._ck(self.lib.vtlb_linear_bwd_f32_planes(self.h, _ptr(G), _ptr(X), _ptr(W), _ptr(dX), _ptr(dW), _ptr(db),
                                                     M, N, K, _pl(g_rows), _pl(g_cols), _pl(x_cols),
                                                     _ptr(relu_mask_src), _pl(dx_rows), _pl(dx_cols)))

    def bias_grad_f32_noalloc(self, G, M, N, db):
        self._ck(self.lib.vtlb_bias_grad_f32_noalloc(self.h, _ptr(G), M, N, _ptr(db)))

    def relu_fwd_f32(self, x, y, n):
        self._ck(self.lib.vtlb_relu_fwd_f32(self.h, _ptr(x), _ptr(y), n))

    def relu_bwd_f32(self, g, cached, dx, n):
        self._ck(self.lib.vtlb_relu_bwd_f32(self.h, _ptr(g), _ptr(cached), _ptr(dx), n))

    def add_inplace_f32(self, dst, src, n):
        self._ck(self.lib.vtlb_add_inplace_f32(self.h, _ptr(dst), _ptr(src), n))

    def fill_f32(self, dst, value, n):
        self._ck(self.lib.vtlb_fill_f32(self.h, _ptr(dst), value, n))

    def init_uniform_f32(self, out, n, lo, hi, seed):
        self._ck(self.lib.vtlb_init_uniform_f32(self.h, _ptr(out), n, lo, hi, seed))

    def init_normal_f32(self, out, n, mu, sigma, seed):
        self._ck(self.lib.vtlb_init_normal_f32(self.h, _ptr(out), n, mu, sigma, seed))

    # -- input pipeline: copies on their own streams (host pointers as integers, pinned memory)
    COPY_IN_BEFORE_COMPUTE, COPY_OUT_BEFORE_COMPUTE, COPY_OUT_DONE = 1, 2, 4

    def copy_h2d_async(self, dst, hptr: int, nbytes: int):
        self._ck(self.lib.vtlb_copy_h2d_async(self.h, _ptr(dst), hptr, nbytes))

    def copy_d2h_async(self, hptr: int, src, nbytes: int):
        self._ck(self.lib.vtlb_copy_d2h_async(self.h, hptr, _ptr(src), nbytes))

    def copy_wait(self, what: int):
        self._ck(self.lib.vtlb_copy_wait(self.h, what))

    # -- batch assembly on the device (datasets/dataloader.v:41-143)
    def gather_rows_f32(self, src, src_rows, row_elems, indices, n_rows, dst, check=True):
        self._ck(self.lib.vtlb_gather_rows_f32(self.h, _ptr(src), src_rows, row_elems, _ptr(indices), n_rows,
                                               _ptr(dst), int(check)))

    def one_hot_f32(self, labels, n, classes, out, check=True):
        self._ck(self.lib.vtlb_one_hot_f32(self.h, _ptr(labels), n, classes, _ptr(out), int(check)))

    # -- checkpoint payloads (text of nn/models/serialization.v:421-473)
    def ckpt_text_len(self, n: int) -> int:
        return int(self.lib.vtlb_ckpt_text_len(n))

    def ckpt_encode_f32(self, src, n, text):
        self._ck(self.lib.vtlb_ckpt_encode_f32(self.h, _ptr(src), n, _ptr(text)))

    def ckpt_decode_f32(self, text, text_len, dst, n):
        self._ck(self.lib.vtlb_ckpt_decode_f32(self.h, _ptr(text), text_len, _ptr(dst), n))

    def conv2d_fwd_f32(self, x, w, bias, y, B, Cc, H, W, O, kh, kw, ph, pw, sh, sw, relu=False, pre=None, dil=None):
        if dil is not None:
            self._ck(self.lib.vtlb_conv2d_fwd_f32_dilated(self.h, _ptr(x), _ptr(w), _ptr(bias), _ptr(y), B, Cc, H, W, O,
                                                          kh, kw, ph, pw, sh, sw, dil[0], dil[1], int(relu), _ptr(pre)))
            return
        self._ck(self.lib.vtlb_conv2d_fwd_f32(self.h, _ptr(x), _ptr(w), _ptr(bias), _ptr(y), B, Cc, H, W, O,
                                              kh, kw, ph, pw, sh, sw, int(relu), _ptr(pre)))

    def conv2d_bwd_f32(self, g, x, w, dx, dw, db, B, Cc, H, W, O, kh, kw, ph, pw, sh, sw, dil=None):
        if dil is not None:
            self._ck(self.lib.vtlb_conv2d_bwd_f32_dilated(self.h, _ptr(g), _ptr(x), _ptr(w), _ptr(dx), _ptr(dw),
                                                          _ptr(db), B, Cc, H, W, O, kh, kw, ph, pw, sh, sw, dil[0],
                                                          dil[1]))
            return
        self._ck(self.lib.vtlb_conv2d_bwd_f32(self.h, _ptr(g), _ptr(x), _ptr(w), _ptr(dx), _ptr(dw), _ptr(db),
                                              B, Cc, H, W, O, kh, kw, ph, pw, sh, sw))

    def maxpool2d_fwd_f32(self, x, y, idx, B, Cc, H, W, kh, kw, ph, pw, sh, sw):
        self._ck(self.lib.vtlb_maxpool2d_fwd_f32(self.h, _ptr(x), _ptr(y), _ptr(idx), B, Cc, H, W, kh, kw,
                                                 ph, pw, sh, sw))

    def maxpool2x2_bwd_f32(self, g, idx, relu_cache, dx, B, Cc, H, W):
        """relu_cache: the pre-activation of a ReLU in front of the pool (its backward is fused) or None."""
        self._ck(self.lib.vtlb_maxpool2x2_bwd_f32(self.h, _ptr(g), _ptr(idx), _ptr(relu_cache), _ptr(dx), B, Cc, H, W))

    def maxpool2d_bwd_f32(self, g, idx, dx, n_out, n_in):
        self._ck(self.lib.vtlb_maxpool2d_bwd_f32(self.h, _ptr(g), _ptr(idx), _ptr(dx), n_out, n_in))

    def mse_fwd_bwd_f32(self, P, T, n, n_div, loss, dP=None):
        self._ck(self.lib.vtlb_mse_fwd_bwd_f32(self.h, _ptr(P), _ptr(T), n, n_div, _ptr(loss),
                                               _ptr(dP)))

    def softmax_ce_fwd_bwd_f32(self, X, T, B, Cc, batch_div, loss, dX=None):
        self._ck(self.lib.vtlb_softmax_ce_fwd_bwd_f32(self.h, _ptr(X), _ptr(T), B, Cc, batch_div,
                                                      _ptr(loss), _ptr(dX)))

    # -- optimizers
    @staticmethod
    def adam_table(tensors):
        arr = (AdamTensor * len(tensors))()
        for i, (g, th, m, v, n) in enumerate(tensors):
            arr[i] = AdamTensor(_ptr(g), _ptr(th), _ptr(m), _ptr(v), n)
        return arr

    def adam_step_f32(self, table, beta1, beta2, lr_t, eps, zero_grad=True):
        self._ck(self.lib.vtlb_adam_step_f32(self.h, len(table), table, beta1, beta2, lr_t, eps,
                                             int(zero_grad)))

    def adamw_step_f32(self, table, beta1, beta2, lr_t, eps, wd, zero_grad=True):
        self._ck(self.lib.vtlb_adamw_step_f32(self.h, len(table), table, beta1, beta2, lr_t, eps,
                                              wd, int(zero_grad)))

    def sgd_step_f32(self, table, lr, zero_grad=True):
        self._ck(self.lib.vtlb_sgd_step_f32(self.h, len(table), table, lr, int(zero_grad)))

    def rmsprop_step_f32(self, table, lr, alpha, eps, wd, zero_grad=True):
        self._ck(self.lib.vtlb_rmsprop_step_f32(self.h, len(table), table, lr, alpha, eps, wd, int(zero_grad)))

    # -- layers next to the GEMMs
    def softmax_fwd_f32(self, x, rows, n, y):
        self._ck(self.lib.vtlb_softmax_fwd_f32(self.h, _ptr(x), rows, n, _ptr(y)))

    def softmax_bwd_f32(self, g, x, rows, n, dx):
        self._ck(self.lib.vtlb_softmax_bwd_f32(self.h, _ptr(g), _ptr(x), rows, n, _ptr(dx)))

    def avgpool2d_fwd_f32(self, x, y, B, Cc, H, W, kh, kw, ph, pw, sh, sw):
        self._ck(self.lib.vtlb_avgpool2d_fwd_f32(self.h, _ptr(x), _ptr(y), B, Cc, H, W, kh, kw, ph, pw, sh, sw))

    def avgpool2d_bwd_f32(self, g, dx, B, Cc, H, W, kh, kw, ph, pw, sh, sw):
        self._ck(self.lib.vtlb_avgpool2d_bwd_f32(self.h, _ptr(g), _ptr(dx), B, Cc, H, W, kh, kw, ph, pw, sh, sw))

    def global_avgpool2d_fwd_f32(self, x, y, B, Cc, H, W):
        self._ck(self.lib.vtlb_global_avgpool2d_fwd_f32(self.h, _ptr(x), _ptr(y), B, Cc, H, W))

    def global_avgpool2d_bwd_f32(self, g, dx, B, Cc, H, W):
        self._ck(self.lib.vtlb_global_avgpool2d_bwd_f32(self.h, _ptr(g), _ptr(dx), B, Cc, H, W))

    def batchnorm1d_train_f32(self, x, B, F, gamma, beta, eps, y, mean, var, rmean=None, rvar=None, momentum=0.1):
        self._ck(self.lib.vtlb_batchnorm1d_train_f32(self.h, _ptr(x), B, F, _ptr(gamma), _ptr(beta), eps, _ptr(y),
                                                     _ptr(mean), _ptr(var), _ptr(rmean), _ptr(rvar), momentum))

    def batchnorm1d_infer_f32(self, x, B, F, gamma, beta, rmean, rvar, eps, y):
        self._ck(self.lib.vtlb_batchnorm1d_infer_f32(self.h, _ptr(x), B, F, _ptr(gamma), _ptr(beta), _ptr(rmean),
                                                     _ptr(rvar), eps, _ptr(y)))

    def batchnorm1d_bwd_f32(self, g, x, B, F, gamma, mean, var, eps, dx=None, dgamma=None, dbeta=None):
        self._ck(self.lib.vtlb_batchnorm1d_bwd_f32(self.h, _ptr(g), _ptr(x), B, F, _ptr(gamma), _ptr(mean), _ptr(var),
                                                   eps, _ptr(dx), _ptr(dgamma), _ptr(dbeta)))

    # -- int8
    def i8_ld(self, K: int) -> int:
        return int(self.lib.vtlb_i8_ld(K))

    def quant_rows_i8(self, A, M, K, Q, scale, amax_in=None):
        self._ck(self.lib.vtlb_quant_rows_i8(self.h, _ptr(A), M, K, _ptr(Q), _ptr(scale),
                                             _ptr(amax_in)))

    def row_absmax_f32(self, A, M, K, amax):
        self._ck(self.lib.vtlb_row_absmax_f32(self.h, _ptr(A), M, K, _ptr(amax)))

    def gemm_i8_i32(self, Aq, Wq, M, N, K, acc):
        self._ck(self.lib.vtlb_gemm_i8_i32(self.h, _ptr(Aq), _ptr(Wq), M, N, K, _ptr(acc)))

    def linear_i8_fwd(self, Aq, sa, Wq, sw, bias, Y, M, N, K, relu=False):
        self._ck(self.lib.vtlb_linear_i8_fwd(self.h, _ptr(Aq), _ptr(sa), _ptr(Wq), _ptr(sw),
                                             _ptr(bias), _ptr(Y), M, N, K, int(relu)))

    def linear_i8_fwd_sharded_a(self, Aq_shards, shards, sa, Wq, sw, bias, Y, M, N, K, relu=False):
        self._ck(self.lib.vtlb_linear_i8_fwd_sharded_a(self.h, _ptr(Aq_shards), shards, _ptr(sa), _ptr(Wq),
                                                       _ptr(sw), _ptr(bias), _ptr(Y), M, N, K, int(relu)))

    def linear_i8_fwd_amax(self, Aq_shards, shards, sa, Wq, sw, bias, Y, M, N, K, relu, row_amax):
        self._ck(self.lib.vtlb_linear_i8_fwd_amax(self.h, _ptr(Aq_shards), shards, _ptr(sa), _ptr(Wq), _ptr(sw),
                                                  _ptr(bias), _ptr(Y), M, N, K, int(relu), _ptr(row_amax)))

    def int8_issue_yardstick(self, mma_groups: int = 20000) -> float:
        """TOPS of back-to-back INT8 MMAs on shared-memory-resident operands (no loads)."""
        t = C.c_double(0)
        self._ck(self.lib.vtlb_int8_issue_yardstick(self.h, mma_groups, C.byref(t)))
        return t.value

    # -- collectives
    def comm_unique_id(self) -> bytes:
        buf = C.create_string_buffer(128)
        rc = self.lib.vtlb_comm_unique_id(buf)
        if rc != OK:
            raise VtlbError(rc, self.lib.vtlb_last_error(None).decode())
        return buf.raw

    def comm_init_rank(self, nranks: int, rank: int, uid: bytes):
        self._ck(self.lib.vtlb_comm_init_rank(self.h, nranks, rank, C.c_char_p(uid)))

    def allreduce_sum_f32_async(self, buf, n):
        self._ck(self.lib.vtlb_allreduce_sum_f32_async(self.h, _ptr(buf), n))

    def allreduce_max_f32_async(self, buf, n):
        self._ck(self.lib.vtlb_allreduce_max_f32_async(self.h, _ptr(buf), n))

    def allgather_async(self, send, recv, bytes_per_rank):
        self._ck(self.lib.vtlb_allgather_async(self.h, _ptr(send), _ptr(recv), bytes_per_rank))

    LANE_BULK, LANE_SMALL = 0, 1

    def comm_small_lane(self):
        """A communicator and stream of their own for the small collectives (every rank calls it)."""
        self._ck(self.lib.vtlb_comm_small_lane(self.h))

    # -- all-gather by copy engines: buffers that the other ranks' processes can write
    def shared_alloc(self, nbytes: int):
        """-> (device pointer, 64-byte IPC handle) of a zeroed buffer the peers may open."""
        p, h = _vp(), C.create_string_buffer(64)
        self._ck(self.lib.vtlb_shared_alloc(self.h, nbytes, C.byref(p), h))
        return p.value, h.raw

    def shared_free(self, ptr: int):
        self._ck(self.lib.vtlb_shared_free(self.h, ptr))

    def shared_open(self, handle: bytes) -> int:
        p = _vp()
        self._ck(self.lib.vtlb_shared_open(self.h, C.c_char_p(handle), C.byref(p)))
        return p.value

    def shared_close(self, ptr: int):
        self._ck(self.lib.vtlb_shared_close(self.h, ptr))

    def allgather_push_async(self, src, peer_dst, nbytes: int):
        """peer_dst: one device address per rank (None / 0 = skip, e.g. this rank itself)."""
        arr = (_vp * len(peer_dst))(*[_vp(p) if p else _vp(None) for p in peer_dst])
        self._ck(self.lib.vtlb_allgather_push_async(self.h, _ptr(src), arr, len(peer_dst), nbytes))

    def comm_mark(self, lane: int, slot: int):
        self._ck(self.lib.vtlb_comm_mark(self.h, lane, slot))

    def comm_wait_mark(self, slot: int):
        self._ck(self.lib.vtlb_comm_wait_mark(self.h, slot))

    def comm_wait(self):
        self._ck(self.lib.vtlb_comm_wait(self.h))
