"""ctypes binding of libvtl_host.so: the C++ mirror of vtl's Sequential / autograd /
optimizer API (vtl_b200/csrc/host).  A model is built the way a vtl program builds it:

    s = Session(0)
    m = Model(s)
    m.input([784]); m.linear(256); m.relu(); m.linear(10); m.mse_loss()
    m.adam(1e-3)
    loss = m.train_step(d_x, (64, 784), d_t, (64, 10))

Inputs and targets are device buffers (vtl_b200.capi.DBuf or raw device pointers)."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import capi

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libvtl_host.so")
_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        capi.load()  # libvtlb200.so first (the host library links against it)
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: run `python -m vtl_b200.build`")
        lib = C.CDLL(LIB_PATH)
        lib.vtlh_last_error.restype = C.c_char_p
        lib.vtlh_session_ctx.restype = C.c_void_p
        lib.vtlh_session_ctx.argtypes = [C.c_void_p]
        vp, i, d = C.c_void_p, C.c_int, C.c_double
        ip = C.POINTER(C.c_int)
        protos = {
            "vtlh_session_create": [i, C.POINTER(vp)], "vtlh_session_destroy": [vp],
            "vtlh_session_comm_init": [vp, i, i, vp],
            "vtlh_session_set_seed": [vp, C.c_ulonglong], "vtlh_session_set_pass_planes": [vp, i],
            "vtlh_session_set_plane_min_flops": [vp, d],
            "vtlh_compute_fans": [i, ip, C.POINTER(C.c_longlong), C.POINTER(C.c_longlong)],
            "vtlh_variance_scaled": [vp, i, ip, d, i, i, C.c_ulonglong, vp],
            "vtlh_model_create": [vp, C.POINTER(vp)], "vtlh_model_destroy": [vp],
            "vtlh_model_input": [vp, i, ip], "vtlh_model_linear": [vp, i], "vtlh_model_relu": [vp],
            "vtlh_model_flatten": [vp], "vtlh_model_conv2d": [vp] + [i] * 8,
            "vtlh_model_conv2d_dilated": [vp] + [i] * 10,
            "vtlh_model_maxpool2d": [vp] + [i] * 6, "vtlh_model_mse_loss": [vp],
            "vtlh_model_softmax_cross_entropy_loss": [vp], "vtlh_model_set_fuse_relu": [vp, i],
            "vtlh_model_adam": [vp, d, d, d, d], "vtlh_model_adamw": [vp, d, d, d, d, d],
            "vtlh_model_num_params": [vp], "vtlh_model_param_size": [vp, i, C.POINTER(C.c_size_t)],
            "vtlh_model_set_param": [vp, i, vp], "vtlh_model_get_param": [vp, i, vp],
            "vtlh_model_get_grad": [vp, i, vp], "vtlh_model_get_moment": [vp, i, i, vp],
            "vtlh_model_forward": [vp, vp, i, ip, vp],
            "vtlh_model_train_step": [vp, vp, i, ip, vp, i, ip, i, i, C.POINTER(C.c_float)],
            "vtlh_model_get_input_grad": [vp, vp], "vtlh_model_zero_grad": [vp],
            "vtlh_matmul_mse_backprop": [vp, vp, i, i, vp, i, vp, vp, vp, vp, vp],
            "vtlh_model_sgd": [vp, d], "vtlh_model_rmsprop": [vp, d, d, d, d],
            "vtlh_model_softmax": [vp], "vtlh_model_avgpool2d": [vp] + [i] * 6,
            "vtlh_model_global_avgpool2d": [vp], "vtlh_model_batchnorm1d": [vp, i, d, d],
            "vtlh_model_get_running_stat": [vp, i, i, vp], "vtlh_model_get_sq_avg": [vp, i, vp],
            "vtlh_model_save_checkpoint": [vp, C.c_char_p, i, d, i],
            "vtlh_model_load_weights": [vp, C.c_char_p, i],
            "vtlh_load_checkpoint": [C.c_char_p, ip, C.POINTER(d)],
            "vtlh_loader_create": [vp, vp, i, ip, vp, i, ip, i, i, i, C.c_ulonglong, C.POINTER(vp)],
            "vtlh_loader_destroy": [vp], "vtlh_loader_len": [vp], "vtlh_loader_total_samples": [vp],
            "vtlh_loader_reset": [vp], "vtlh_loader_indices": [vp, ip],
            "vtlh_loader_batch": [vp, i, vp, vp, ip],
            "vtlh_loader_split": [vp, d, C.POINTER(vp), C.POINTER(vp)],
        }
        for name, args in protos.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = C.c_int
        _lib = lib
    return _lib


def _ck(rc: int):
    if rc != 0:
        raise capi.VtlbError(rc, load().vtlh_last_error().decode())


def _shape(shape):
    arr = (C.c_int * len(shape))(*[int(x) for x in shape])
    return len(shape), arr


FAN_AVG, FAN_IN, FAN_OUT = 0, 1, 2   # internal.FanMode (nn/internal/init.v:7-12)
UNIFORM, NORMAL = 0, 1               # internal.Distribution (:14-18)


def compute_fans(shape):
    """internal.compute_fans as written (nn/internal/init.v:21-33): (shape[0]*prod(shape[1:]),
    shape[1]*prod(shape[1:]))."""
    f0, f1 = C.c_longlong(0), C.c_longlong(0)
    _ck(load().vtlh_compute_fans(*_shape(shape), C.byref(f0), C.byref(f1)))
    return f0.value, f1.value


class Session:
    """autograd_cuda.DeviceSession: owns the device context of one GPU."""

    def __init__(self, device: int = 0):
        self.lib = load()
        h = C.c_void_p()
        _ck(self.lib.vtlh_session_create(device, C.byref(h)))
        self.h = h
        # a capi.Device view of the same vtlb_ctx, for allocations and copies
        self.dev = capi.Device.__new__(capi.Device)
        self.dev.lib = capi.load()
        self.dev.h = C.c_void_p(self.lib.vtlh_session_ctx(h))
        self.dev.index = device
        self.dev.close = lambda: None  # the session owns the context

    def comm_init(self, nranks: int, rank: int, uid: bytes):
        _ck(self.lib.vtlh_session_comm_init(self.h, nranks, rank, C.c_char_p(uid)))

    def set_seed(self, seed: int):
        """Seed of the Kaiming-normal draws of the layers built after this call."""
        _ck(self.lib.vtlh_session_set_seed(self.h, int(seed)))

    def set_pass_planes(self, on: bool):
        """Producer-to-consumer hand-over of TF32 operand planes in large Linear layers (default on)."""
        _ck(self.lib.vtlh_session_set_pass_planes(self.h, int(on)))

    def set_plane_min_flops(self, flops: float):
        """Smallest product (2*M*N*K) whose planes are handed on (default 1e12)."""
        _ck(self.lib.vtlh_session_set_plane_min_flops(self.h, float(flops)))

    def variance_scaled(self, shape, scale, fan_mode, distribution, seed):
        """internal.variance_scaled (nn/internal/init.v:36-60) -> host array."""
        out = np.empty(shape, np.float32)
        _ck(self.lib.vtlh_variance_scaled(self.h, *_shape(shape), float(scale), int(fan_mode), int(distribution),
                                          int(seed), out.ctypes.data))
        return out

    def kaiming_uniform(self, shape, seed):
        return self.variance_scaled(shape, 2.0, FAN_IN, UNIFORM, seed)

    def kaiming_normal(self, shape, seed):
        return self.variance_scaled(shape, 2.0, FAN_IN, NORMAL, seed)

    def matmul_mse_backprop(self, d_A, M, K, d_B, N, d_T):
        """Variable.matmul + MSE loss + backprop on a fresh tape -> (loss, C, dA, dB) on the host."""
        loss = np.zeros(1, np.float32)
        Cm, dA, dB = np.empty((M, N), np.float32), np.empty((M, K), np.float32), np.empty((K, N), np.float32)
        _ck(self.lib.vtlh_matmul_mse_backprop(self.h, capi._ptr(d_A), M, K, capi._ptr(d_B), N, capi._ptr(d_T),
                                              loss.ctypes.data, Cm.ctypes.data, dA.ctypes.data, dB.ctypes.data))
        return float(loss[0]), Cm, dA, dB

    def close(self):
        if self.h:
            self.dev.h = None
            self.lib.vtlh_session_destroy(self.h)
            self.h = None


class Model:
    """nn/models/sequential.v Sequential plus its optimizer."""

    def __init__(self, session: Session):
        self.s, self.lib = session, session.lib
        h = C.c_void_p()
        _ck(self.lib.vtlh_model_create(session.h, C.byref(h)))
        self.h = h

    def close(self):
        if self.h:
            self.lib.vtlh_model_destroy(self.h)
            self.h = None

    # -- builder (same names as the reference)
    def input(self, shape):
        _ck(self.lib.vtlh_model_input(self.h, *_shape(shape)))

    def linear(self, n):
        _ck(self.lib.vtlh_model_linear(self.h, n))

    def relu(self):
        _ck(self.lib.vtlh_model_relu(self.h))

    def flatten(self):
        _ck(self.lib.vtlh_model_flatten(self.h))

    def conv2d(self, in_ch, out_ch, kernel, padding=(0, 0), stride=(1, 1), dilation=(1, 1)):
        _ck(self.lib.vtlh_model_conv2d_dilated(self.h, in_ch, out_ch, kernel[0], kernel[1], padding[0], padding[1],
                                               stride[0], stride[1], dilation[0], dilation[1]))

    def maxpool2d(self, kernel, padding, stride):
        _ck(self.lib.vtlh_model_maxpool2d(self.h, kernel[0], kernel[1], padding[0], padding[1], stride[0],
                                          stride[1]))

    def softmax(self):
        _ck(self.lib.vtlh_model_softmax(self.h))

    def avgpool2d(self, kernel, padding, stride):
        _ck(self.lib.vtlh_model_avgpool2d(self.h, kernel[0], kernel[1], padding[0], padding[1], stride[0],
                                          stride[1]))

    def global_avgpool2d(self):
        _ck(self.lib.vtlh_model_global_avgpool2d(self.h))

    def batchnorm1d(self, num_features, eps=1e-5, momentum=0.1):
        _ck(self.lib.vtlh_model_batchnorm1d(self.h, int(num_features), float(eps), float(momentum)))

    def running_stat(self, bn_index, num_features, variance=False):
        out = np.empty(num_features, np.float32)
        _ck(self.lib.vtlh_model_get_running_stat(self.h, bn_index, int(variance), out.ctypes.data))
        return out

    def sgd(self, lr=1e-3):
        _ck(self.lib.vtlh_model_sgd(self.h, lr))

    def rmsprop(self, lr=1e-3, alpha=0.99, eps=1e-8, weight_decay=0.0):
        _ck(self.lib.vtlh_model_rmsprop(self.h, lr, alpha, eps, weight_decay))

    def get_sq_avg(self, i):
        return self._get(self.lib.vtlh_model_get_sq_avg, i)

    def mse_loss(self):
        _ck(self.lib.vtlh_model_mse_loss(self.h))

    def softmax_cross_entropy_loss(self):
        _ck(self.lib.vtlh_model_softmax_cross_entropy_loss(self.h))

    def set_fuse_relu(self, on: bool):
        _ck(self.lib.vtlh_model_set_fuse_relu(self.h, int(on)))

    def adam(self, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8):
        _ck(self.lib.vtlh_model_adam(self.h, lr, beta1, beta2, eps))

    def adamw(self, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01):
        _ck(self.lib.vtlh_model_adamw(self.h, lr, beta1, beta2, eps, weight_decay))

    # -- parameters
    def num_params(self) -> int:
        return int(self.lib.vtlh_model_num_params(self.h))

    def param_size(self, i) -> int:
        n = C.c_size_t(0)
        _ck(self.lib.vtlh_model_param_size(self.h, i, C.byref(n)))
        return n.value

    def set_param(self, i, a):
        a = np.ascontiguousarray(a, np.float32)
        assert a.size == self.param_size(i), (a.size, self.param_size(i))
        _ck(self.lib.vtlh_model_set_param(self.h, i, a.ctypes.data))

    def _get(self, fn, i, *extra):
        out = np.empty(self.param_size(i), np.float32)
        _ck(fn(self.h, i, *extra, out.ctypes.data))
        return out

    def get_param(self, i):
        return self._get(self.lib.vtlh_model_get_param, i)

    def get_grad(self, i):
        return self._get(self.lib.vtlh_model_get_grad, i)

    def get_moment(self, i, second=False):
        return self._get(self.lib.vtlh_model_get_moment, i, int(second))

    # -- running
    def forward(self, d_x, xshape, d_y=None):
        _ck(self.lib.vtlh_model_forward(self.h, capi._ptr(d_x), *_shape(xshape), capi._ptr(d_y)))

    def train_step(self, d_x, xshape, d_t, tshape, global_rows=0, update=True, want_loss=True):
        loss = C.c_float(0)
        _ck(self.lib.vtlh_model_train_step(self.h, capi._ptr(d_x), *_shape(xshape), capi._ptr(d_t),
                                           *_shape(tshape), int(global_rows), int(update),
                                           C.byref(loss) if want_loss else None))
        return loss.value if want_loss else None

    def zero_grad(self):
        _ck(self.lib.vtlh_model_zero_grad(self.h))

    def input_grad(self, shape):
        out = np.empty(shape, np.float32)
        _ck(self.lib.vtlh_model_get_input_grad(self.h, out.ctypes.data))
        return out

    # -- checkpoints in the reference's format (nn/models/serialization.v)
    def save(self, path):
        """Sequential.save: weights only, epoch 0, loss 0 (serialization.v:102-104)."""
        self.save_checkpoint(path, 0, 0.0)

    def save_checkpoint(self, path, epoch=0, loss=0.0, with_optimizer=False):
        _ck(self.lib.vtlh_model_save_checkpoint(self.h, os.fsencode(path), int(epoch), float(loss),
                                                int(with_optimizer)))

    def load_weights(self, path, with_optimizer=False):
        _ck(self.lib.vtlh_model_load_weights(self.h, os.fsencode(path), int(with_optimizer)))


def load_checkpoint(path):
    """Sequential.load_checkpoint: (epoch, loss) stored in a checkpoint (serialization.v:266-276)."""
    epoch, loss = C.c_int(0), C.c_double(0.0)
    _ck(load().vtlh_load_checkpoint(os.fsencode(path), C.byref(epoch), C.byref(loss)))
    return epoch.value, loss.value


class DataLoader:
    """datasets.DataLoader (datasets/dataloader.v) over device-resident dataset / label buffers
    (capi.DBuf, f32, first dimension = samples).  batch(i) returns device buffers."""

    def __init__(self, session: Session, dataset, labels=None, batch_size=32, shuffle=True, drop_last=True,
                 seed=0, _handle=None):
        self.lib, self.session, self.dataset, self.labels = load(), session, dataset, labels
        self.batch_size = batch_size
        if _handle is not None:
            self.h = _handle
            return
        h = C.c_void_p()
        ln, ls = _shape(labels.shape) if labels is not None else (0, None)
        _ck(self.lib.vtlh_loader_create(session.h, capi._ptr(dataset), *_shape(dataset.shape),
                                        capi._ptr(labels), ln, ls, int(batch_size), int(shuffle),
                                        int(drop_last), int(seed), C.byref(h)))
        self.h = h

    def close(self):
        if getattr(self, "h", None):
            self.lib.vtlh_loader_destroy(self.h)
            self.h = None

    def __len__(self):
        return int(self.lib.vtlh_loader_len(self.h))

    def total_samples(self) -> int:
        return int(self.lib.vtlh_loader_total_samples(self.h))

    def reset(self):
        _ck(self.lib.vtlh_loader_reset(self.h))

    @property
    def indices(self):
        out = (C.c_int * max(self.total_samples(), 1))()
        _ck(self.lib.vtlh_loader_indices(self.h, out))
        return list(out[: self.total_samples()])

    def _batch(self, i, with_labels):
        dev = self.session.dev
        feat = dev.empty((self.batch_size,) + tuple(self.dataset.shape[1:]), np.float32)
        lab = dev.empty((self.batch_size,) + tuple(self.labels.shape[1:]), np.float32) if with_labels else None
        rows = C.c_int(0)
        _ck(self.lib.vtlh_loader_batch(self.h, int(i), feat.ptr, lab.ptr if lab else None, C.byref(rows)))
        if rows.value == 0:
            feat.free()
            if lab:
                lab.free()
            return None
        feat.shape = (rows.value,) + tuple(self.dataset.shape[1:])
        if lab:
            lab.shape = (rows.value,) + tuple(self.labels.shape[1:])
        return (feat, lab) if with_labels else feat

    def batch(self, i):
        return self._batch(i, False)

    def batch_with_labels(self, i):
        if self.labels is None:
            return None
        return self._batch(i, True)

    def split(self, val_fraction):
        t, v = C.c_void_p(), C.c_void_p()
        _ck(self.lib.vtlh_loader_split(self.h, float(val_fraction), C.byref(t), C.byref(v)))
        mk = lambda h: DataLoader(self.session, self.dataset, self.labels, self.batch_size, _handle=h)
        return mk(t), mk(v)
