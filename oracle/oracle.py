"""CPU oracle for the dense-contraction hot path (TEST INFRASTRUCTURE ONLY).

NumPy front end of ``oracle.c`` (loaded through ctypes) plus BLAS-level NumPy
restatements used where the plain C loops would take too long.  Nothing in the
product package imports this module; only the tests, the smoke check and the
CPU-baseline / reference legs of the benchmark do.

Every function names the reference code it follows (paths inside vlang/vtl).
The INT8 functions have no counterpart in the reference ("parity unpinned"):
their definition is the one in ``oracle.c``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle.so")


def build(force: bool = False) -> str:
    """Compile oracle.c -> liboracle.so with the Makefile next to it."""
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "liboracle.so"], stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = C.CDLL(_SO)
        _lib.orc_mse_f32.restype = C.c_float
        _lib.orc_mse_f64.restype = C.c_double
        _lib.orc_softmax_ce_f32.restype = C.c_float
        _lib.orc_adam_lr_t.restype = C.c_double
        _lib.orc_max_threads.restype = C.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _f64(a):
    return np.ascontiguousarray(a, dtype=np.float64)


def max_threads() -> int:
    return int(lib().orc_max_threads())


def set_threads(n: int) -> None:
    """Lets the OpenMP loops of the C oracle use n threads from now on."""
    lib().orc_set_threads(int(n))


# ---------------------------------------------------------------- matmul
def matmul_f32(A, B, ta=False, tb=False):
    """la.matmul[f32] (la/la.v:38-55): f64 multiply-accumulate, one final rounding."""
    A, B = _f32(A), _f32(B)
    M, K = (A.shape[1], A.shape[0]) if ta else A.shape
    N = B.shape[0] if tb else B.shape[1]
    out = np.empty((M, N), np.float32)
    lib().orc_matmul_f32(_p(A), _p(B), _p(out), M, N, K, int(ta), int(tb))
    return out


def matmul_f64(A, B, ta=False, tb=False):
    A, B = _f64(A), _f64(B)
    M, K = (A.shape[1], A.shape[0]) if ta else A.shape
    N = B.shape[0] if tb else B.shape[1]
    out = np.empty((M, N), np.float64)
    lib().orc_matmul_f64(_p(A), _p(B), _p(out), M, N, K, int(ta), int(tb))
    return out


def matmul_f32_blas(A, B, ta=False, tb=False):
    """Same recipe as matmul_f32 with NumPy's OpenBLAS dgemm doing the f64 GEMM
    (the class of backend VSL uses with -d cblas); for sizes the C loops cannot
    finish in seconds, and for the timed CPU baseline."""
    a = np.asarray(A, np.float32).astype(np.float64)
    b = np.asarray(B, np.float32).astype(np.float64)
    if ta:
        a = a.T
    if tb:
        b = b.T
    return (a @ b).astype(np.float32)


# ---------------------------------------------------------------- linear
def linear_fwd_f32(X, W, b=None, blas=False):
    """linear_forward_f32_cpu (nn/layers/linear_forward_f32.v:16-18): X.W^T + b."""
    X, W = _f32(X), _f32(W)
    if blas:
        Y = matmul_f32_blas(X, W, tb=True)
        return Y if b is None else (Y + _f32(b).reshape(1, -1)).astype(np.float32)
    M, K = X.shape
    N = W.shape[0]
    Y = np.empty((M, N), np.float32)
    bb = None if b is None else _f32(b).reshape(-1)
    lib().orc_linear_fwd_f32(_p(X), _p(W), _p(bb), _p(Y), M, N, K)
    return Y


def linear_bwd_f32(G, X, W, blas=False):
    """LinearGate.backward (nn/gates/layers/linear.v:69-79) -> (dX, dW, db[1,N])."""
    G, X, W = _f32(G), _f32(X), _f32(W)
    M, N = G.shape
    K = X.shape[1]
    if blas:
        dX = matmul_f32_blas(G, W)
        dW = matmul_f32_blas(G, X, ta=True)
        db = matmul_f32_blas(np.ones((1, M), np.float32), G)
        return dX, dW, db
    dX = np.empty((M, K), np.float32)
    dW = np.empty((N, K), np.float32)
    db = np.empty((1, N), np.float32)
    lib().orc_linear_bwd_f32(_p(G), _p(X), _p(W), _p(dX), _p(dW), _p(db), M, N, K)
    return dX, dW, db


def linear_fwd_f64(X, W, b):
    X, W, b = _f64(X), _f64(W), _f64(b).reshape(-1)
    M, K = X.shape
    N = W.shape[0]
    Y = np.empty((M, N), np.float64)
    lib().orc_linear_fwd_f64(_p(X), _p(W), _p(b), _p(Y), M, N, K)
    return Y


def linear_bwd_f64(G, X, W):
    G, X, W = _f64(G), _f64(X), _f64(W)
    M, N = G.shape
    K = X.shape[1]
    dX = np.empty((M, K))
    dW = np.empty((N, K))
    db = np.empty((1, N))
    lib().orc_linear_bwd_f64(_p(G), _p(X), _p(W), _p(dX), _p(dW), _p(db), M, N, K)
    return dX, dW, db


# ---------------------------------------------------------------- relu / losses
def relu_f32(x):
    """internal.relu (nn/internal/activation.v:63-70)."""
    x = _f32(x)
    y = np.empty_like(x)
    lib().orc_relu_f32(_p(x), _p(y), C.c_size_t(x.size))
    return y


def relu_bwd_f32(g, cached):
    """internal.deriv_relu (nn/internal/activation.v:78-87)."""
    g, cached = _f32(g), _f32(cached)
    dx = np.empty_like(g)
    lib().orc_relu_bwd_f32(_p(g), _p(cached), _p(dx), C.c_size_t(g.size))
    return dx


def mse_f32(p, t) -> np.float32:
    """internal.mse (nn/internal/activation.v:365-373)."""
    p, t = _f32(p), _f32(t)
    return np.float32(lib().orc_mse_f32(_p(p), _p(t), C.c_size_t(p.size)))


def mse_f64(p, t) -> float:
    p, t = _f64(p), _f64(t)
    return float(lib().orc_mse_f64(_p(p), _p(t), C.c_size_t(p.size)))


def mse_bwd_f32(p, t, g=1.0):
    """internal.mse_backward (nn/internal/loss.v:7-12), upstream g of size 1."""
    p, t = _f32(p), _f32(t)
    dp = np.empty_like(p)
    lib().orc_mse_bwd_f32(_p(p), _p(t), _p(dp), C.c_size_t(p.size), C.c_float(g))
    return dp


def softmax_ce_f32(x, t) -> np.float32:
    """internal.softmax_cross_entropy (nn/internal/activation.v:392-420)."""
    x, t = _f32(x), _f32(t)
    return np.float32(lib().orc_softmax_ce_f32(_p(x), _p(t), x.shape[0], x.shape[1]))


def softmax_ce_bwd_f32(x, t, upstream=1.0, batch_div=None):
    """softmax_cross_entropy_backward (nn/internal/loss.v:39-65)."""
    x, t = _f32(x), _f32(t)
    dx = np.empty_like(x)
    bd = x.shape[0] if batch_div is None else int(batch_div)
    lib().orc_softmax_ce_bwd_f32(_p(x), _p(t), _p(dx), x.shape[0], x.shape[1],
                                 C.c_double(upstream), bd)
    return dx


# ---------------------------------------------------------------- conv / pool
def conv_out_hw(H, W, kh, kw, ph, pw, sh, sw, dh=1, dw=1):
    return (H + 2 * ph - dh * (kh - 1) - 1) // sh + 1, (W + 2 * pw - dw * (kw - 1) - 1) // sw + 1


def conv2d_fwd_f32(x, w, bias, pad=(0, 0), stride=(1, 1), dil=(1, 1)):
    """conv2d_forward_cpu_f32 (nn/internal/conv2d_forward_cpu_f32.v:26-62)."""
    x, w = _f32(x), _f32(w)
    B, Ci, H, W = x.shape
    O, _, kh, kw = w.shape
    OH, OW = conv_out_hw(H, W, kh, kw, pad[0], pad[1], stride[0], stride[1], dil[0], dil[1])
    y = np.empty((B, O, OH, OW), np.float32)
    bb = None if bias is None else _f32(bias).reshape(-1)
    lib().orc_conv2d_fwd_f32(_p(x), _p(w), _p(bb), _p(y), B, Ci, H, W, O, kh, kw, pad[0], pad[1],
                             stride[0], stride[1], dil[0], dil[1])
    return y


def conv2d_bwd_f32(g, x, w, pad=(0, 0), stride=(1, 1), dil=(1, 1)):
    """conv2d_backward_cpu_f32 (nn/internal/conv2d_backward_cpu_f32.v:26-97) -> (dx, dw, db[1,O])."""
    g, x, w = _f32(g), _f32(x), _f32(w)
    B, Ci, H, W = x.shape
    O, _, kh, kw = w.shape
    dx = np.empty_like(x)
    dw = np.empty_like(w)
    db = np.empty((1, O), np.float32)
    lib().orc_conv2d_bwd_f32(_p(g), _p(x), _p(w), _p(dx), _p(dw), _p(db), B, Ci, H, W, O, kh, kw,
                             pad[0], pad[1], stride[0], stride[1], dil[0], dil[1])
    return dx, dw, db


def maxpool2d_fwd_f32(x, kernel=(2, 2), pad=(0, 0), stride=(2, 2)):
    """Window geometry of internal.maxpool2d (nn/internal/layers.v:21-66), standard
    max selection and whole-tensor flat indices (see oracle.c for why)."""
    x = _f32(x)
    B, Ci, H, W = x.shape
    OH = (H + 2 * pad[0] - kernel[0]) // stride[0] + 1
    OW = (W + 2 * pad[1] - kernel[1]) // stride[1] + 1
    y = np.empty((B, Ci, OH, OW), np.float32)
    idx = np.empty((B, Ci, OH, OW), np.int32)
    lib().orc_maxpool2d_fwd_f32(_p(x), _p(y), _p(idx), B, Ci, H, W, kernel[0], kernel[1], pad[0],
                                pad[1], stride[0], stride[1])
    return y, idx


def maxpool2d_bwd_f32(g, idx, in_shape):
    g = _f32(g)
    idx = np.ascontiguousarray(idx, np.int32)
    dx = np.empty(in_shape, np.float32)
    lib().orc_maxpool2d_bwd_f32(_p(g), _p(idx), _p(dx), C.c_size_t(g.size), C.c_size_t(dx.size))
    return dx


# ---------------------------------------------------------------- optimizers
def adam_lr_t(lr, beta1_t, beta2_t, beta1, beta2):
    """lr_t and advanced beta^t of AdamOptimizer.update (nn/optimizers/adam.v:88-91)."""
    b1 = C.c_double(beta1_t)
    b2 = C.c_double(beta2_t)
    lr_t = lib().orc_adam_lr_t(C.c_double(lr), C.byref(b1), C.byref(b2), C.c_double(beta1),
                               C.c_double(beta2))
    return float(lr_t), b1.value, b2.value


def adam_step_f32(grad, theta, m, v, beta1, beta2, lr_t, eps):
    """adam_step_f32_cpu (nn/optimizers/adam_step_f32.v:6-21); returns new (theta, m, v)."""
    grad = _f32(grad)
    theta, m, v = _f32(theta).copy(), _f32(m).copy(), _f32(v).copy()
    lib().orc_adam_step_f32(_p(grad), _p(theta), _p(m), _p(v), C.c_size_t(grad.size),
                            C.c_double(beta1), C.c_double(beta2), C.c_double(lr_t), C.c_double(eps))
    return theta, m, v


def adam_step_f64(grad, theta, m, v, beta1, beta2, lr_t, eps):
    """adam_step_f64_cpu (nn/optimizers/adam_step_f64.v:15-23)."""
    grad = _f64(grad)
    theta, m, v = _f64(theta).copy(), _f64(m).copy(), _f64(v).copy()
    lib().orc_adam_step_f64(_p(grad), _p(theta), _p(m), _p(v), C.c_size_t(grad.size),
                            C.c_double(beta1), C.c_double(beta2), C.c_double(lr_t), C.c_double(eps))
    return theta, m, v


def adamw_step_f32(grad, theta, m, v, beta1, beta2, lr_t, eps, wd):
    """AdamWOptimizer.update, T=f32 (nn/optimizers/adamw.v:78-106), moments in the textbook operand
    order (see the note on orc_adamw_step_f32 in oracle.c for the as-written difference)."""
    grad = _f32(grad)
    theta, m, v = _f32(theta).copy(), _f32(m).copy(), _f32(v).copy()
    lib().orc_adamw_step_f32(_p(grad), _p(theta), _p(m), _p(v), C.c_size_t(grad.size),
                             C.c_double(beta1), C.c_double(beta2), C.c_double(lr_t),
                             C.c_double(eps), C.c_double(wd))
    return theta, m, v


def adamw_step_f32_as_written(grad, theta, m, v, beta1, beta2, lr_t, eps, wd):
    """adamw.v:86-93 with the closures' operands exactly as Tensor.napply hands them over
    (m = b1*g + (1-b1)*m, v = b2*g + (1-b2)*v*v).  Forensic comparison only."""
    grad = _f32(grad)
    theta, m, v = _f32(theta).copy(), _f32(m).copy(), _f32(v).copy()
    lib().orc_adamw_step_f32_as_written(_p(grad), _p(theta), _p(m), _p(v), C.c_size_t(grad.size),
                                        C.c_double(beta1), C.c_double(beta2), C.c_double(lr_t),
                                        C.c_double(eps), C.c_double(wd))
    return theta, m, v


# ---------------------------------------------------------------- TF32 operand split of the device GEMMs
def tf32_rna(x):
    """cvt.rna.tf32.f32: round an f32 to 10 mantissa bits, to nearest with ties away from zero
    (finite inputs).  Not a reference function: the device products split every operand into
    hi = tf32(x), lo = tf32(x - hi), and the tests check the planes a product leaves for the next."""
    b = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((b + np.uint32(0x1000)) & np.uint32(0xFFFFE000)).view(np.float32)


def tf32_split(x):
    x = np.ascontiguousarray(x, np.float32)
    hi = tf32_rna(x)
    return hi, tf32_rna((x - hi).astype(np.float32))


# ---------------------------------------------------------------- initialisers (nn/internal/init.v)
def compute_fans(shape):
    """compute_fans as written (nn/internal/init.v:21-33): the product runs over shape[1..], so
    shape[1] enters both fans: (shape[0]*prod(shape[1:]), shape[1]*prod(shape[1:]))."""
    product = int(np.prod(shape[1:], dtype=np.int64))
    return int(shape[0]) * product, int(shape[1]) * product


def variance_scaled_std(shape, scale, fan_mode):
    """std of variance_scaled (nn/internal/init.v:36-50); fan_mode in {"fan_in", "fan_out", "fan_avg"}."""
    f0, f1 = compute_fans(shape)
    if fan_mode == "fan_in":
        return float(np.sqrt(scale / f0))
    if fan_mode == "fan_out":
        return float(np.sqrt(scale / f1))
    return float(np.sqrt(scale * 2.0 / (f0 + f1)))


def _splitmix64(seed, n):
    """The counter-based generator of the device fills: z_i = mix(seed + (i+1)*golden)."""
    with np.errstate(over="ignore"):
        z = np.uint64(seed) + (np.arange(1, n + 1, dtype=np.uint64) * np.uint64(0x9E3779B97F4A7C15))
        z ^= z >> np.uint64(30)
        z *= np.uint64(0xBF58476D1CE4E5B9)
        z ^= z >> np.uint64(27)
        z *= np.uint64(0x94D049BB133111EB)
        z ^= z >> np.uint64(31)
    return z


def init_uniform_f32(n, lo, hi, seed):
    """vtl.random(lo, hi, shape) (rand.v:70-79) on the counter-based stream: u = (z >> 40) * 2^-24,
    x = lo + u * (hi - lo) with each f32 operation rounded on its own."""
    z = _splitmix64(seed, n)
    u = (z >> np.uint64(40)).astype(np.float32) * np.float32(2.0 ** -24)
    lo, hi = np.float32(lo), np.float32(hi)
    return (lo + (u * np.float32(hi - lo)).astype(np.float32)).astype(np.float32)


def init_normal_f32(n, mu, sigma, seed):
    """vtl.normal(shape, mu, sigma) (rand.v:57-66) on the counter-based stream: Box-Muller in f64."""
    z = _splitmix64(seed, n)
    u1 = ((z >> np.uint64(32)).astype(np.float64) + 1.0) * 2.0 ** -32
    u2 = (z & np.uint64(0xFFFFFFFF)).astype(np.float64) * 2.0 ** -32
    r = np.sqrt(-2.0 * np.log(u1))
    return (mu + sigma * (r * np.cos(6.283185307179586476925286766559 * u2))).astype(np.float32)


# ---------------------------------------------------------------- layers and optimizers next to the GEMMs
def softmax_fwd_f32(x):
    """internal.softmax_forward over the last dimension (nn/internal/activation.v:423-457)."""
    x = _f32(x)
    n = x.shape[-1]
    y = np.empty_like(x)
    lib().orc_softmax_fwd_f32(_p(x), C.c_size_t(x.size // n), C.c_size_t(n), _p(y))
    return y


def softmax_bwd_f32(g, x):
    """internal.deriv_softmax (nn/internal/activation.v:285-332)."""
    g, x = _f32(g), _f32(x)
    n = x.shape[-1]
    dx = np.empty_like(x)
    lib().orc_softmax_bwd_f32(_p(g), _p(x), C.c_size_t(x.size // n), C.c_size_t(n), _p(dx))
    return dx


def avgpool2d_fwd_f32(x, kernel=(2, 2), pad=(0, 0), stride=(2, 2)):
    """internal.avgpool2d_forward (nn/internal/pool.v:6-45)."""
    x = _f32(x)
    B, Cc, H, W = x.shape
    OH = (H + 2 * pad[0] - kernel[0]) // stride[0] + 1
    OW = (W + 2 * pad[1] - kernel[1]) // stride[1] + 1
    y = np.empty((B, Cc, OH, OW), np.float32)
    lib().orc_avgpool2d_fwd_f32(_p(x), _p(y), B, Cc, H, W, kernel[0], kernel[1], pad[0], pad[1], stride[0], stride[1])
    return y


def avgpool2d_bwd_f32(g, in_shape, kernel=(2, 2), pad=(0, 0), stride=(2, 2)):
    """Standard average-pool backward (the reference's returns zeros of the wrong shape)."""
    g = _f32(g)
    B, Cc, H, W = in_shape
    dx = np.empty(in_shape, np.float32)
    lib().orc_avgpool2d_bwd_f32(_p(g), _p(dx), B, Cc, H, W, kernel[0], kernel[1], pad[0], pad[1], stride[0], stride[1])
    return dx


def global_avgpool2d_fwd_f32(x):
    x = _f32(x)
    B, Cc, H, W = x.shape
    y = np.empty((B, Cc, 1, 1), np.float32)
    lib().orc_global_avgpool2d_fwd_f32(_p(x), _p(y), B * Cc, H * W)
    return y


def global_avgpool2d_bwd_f32(g, in_shape):
    g = _f32(g)
    B, Cc, H, W = in_shape
    dx = np.empty(in_shape, np.float32)
    lib().orc_global_avgpool2d_bwd_f32(_p(g), _p(dx), B * Cc, H * W)
    return dx


def batchnorm1d_train_f32(x, gamma, beta, eps=1e-5, running_mean=None, running_var=None, momentum=0.1):
    """batchnorm1d_training + the layer's running-statistics update; returns
    (y, batch_mean, batch_var, running_mean, running_var)."""
    x, gamma, beta = _f32(x), _f32(gamma).reshape(-1), _f32(beta).reshape(-1)
    B, F = x.shape
    y, mean, var = np.empty_like(x), np.empty(F, np.float32), np.empty(F, np.float32)
    rm = _f32(running_mean).reshape(-1).copy() if running_mean is not None else None
    rv = _f32(running_var).reshape(-1).copy() if running_var is not None else None
    lib().orc_batchnorm1d_train_f32(_p(x), B, F, _p(gamma), _p(beta), C.c_double(eps), _p(y), _p(mean), _p(var),
                                    _p(rm), _p(rv), C.c_double(momentum))
    return y, mean, var, rm, rv


def batchnorm1d_infer_f32(x, gamma, beta, running_mean, running_var, eps=1e-5):
    x = _f32(x)
    B, F = x.shape
    y = np.empty_like(x)
    lib().orc_batchnorm1d_infer_f32(_p(x), B, F, _p(_f32(gamma).reshape(-1)), _p(_f32(beta).reshape(-1)),
                                    _p(_f32(running_mean).reshape(-1)), _p(_f32(running_var).reshape(-1)),
                                    C.c_double(eps), _p(y))
    return y


def batchnorm1d_bwd_f32(g, x, gamma, mean, var, eps=1e-5):
    g, x = _f32(g), _f32(x)
    B, F = x.shape
    dx, dgamma, dbeta = np.empty_like(x), np.empty(F, np.float32), np.empty(F, np.float32)
    lib().orc_batchnorm1d_bwd_f32(_p(g), _p(x), B, F, _p(_f32(gamma).reshape(-1)), _p(_f32(mean).reshape(-1)),
                                  _p(_f32(var).reshape(-1)), C.c_double(eps), _p(dx), _p(dgamma), _p(dbeta))
    return dx, dgamma, dbeta


def sgd_step_f32(grad, theta, lr):
    """internal.sgd_optimize (nn/internal/optimizers.v:6-13)."""
    grad, theta = _f32(grad), _f32(theta).copy()
    lib().orc_sgd_step_f32(_p(grad), _p(theta), C.c_size_t(grad.size), C.c_double(lr))
    return theta


def rmsprop_step_f32(grad, theta, sq_avg, lr, alpha=0.99, eps=1e-8, wd=0.0):
    """RMSPropOptimizer.update (nn/optimizers/rmsprop.v:70-91)."""
    grad, theta, sq = _f32(grad), _f32(theta).copy(), _f32(sq_avg).copy()
    lib().orc_rmsprop_step_f32(_p(grad), _p(theta), _p(sq), C.c_size_t(grad.size), C.c_double(lr),
                               C.c_double(alpha), C.c_double(eps), C.c_double(wd))
    return theta, sq


# ---------------------------------------------------------------- int8
def quant_rows_i8(A):
    """Symmetric per-row int8 quantisation -> (codes int8 [M,K], scale f32 [M])."""
    A = _f32(A)
    M, K = A.shape
    q = np.empty((M, K), np.int8)
    s = np.empty((M,), np.float32)
    lib().orc_quant_rows_i8(_p(A), _p(q), _p(s), M, K)
    return q, s


def quant_rows_i8_with_amax(A, amax):
    A, amax = _f32(A), _f32(amax)
    M, K = A.shape
    q = np.empty((M, K), np.int8)
    s = np.empty((M,), np.float32)
    lib().orc_quant_rows_i8_with_amax(_p(A), _p(amax), _p(q), _p(s), M, K)
    return q, s


def gemm_i8_i32(Aq, Wq):
    """acc[m,n] = sum_k Aq[m,k]*Wq[n,k], exact int32."""
    Aq = np.ascontiguousarray(Aq, np.int8)
    Wq = np.ascontiguousarray(Wq, np.int8)
    M, K = Aq.shape
    N = Wq.shape[0]
    acc = np.empty((M, N), np.int32)
    lib().orc_gemm_i8_i32(_p(Aq), _p(Wq), _p(acc), M, N, K)
    return acc


def dequant_bias_relu(acc, sa, sw, bias, relu):
    acc = np.ascontiguousarray(acc, np.int32)
    sa, sw = _f32(sa), _f32(sw)
    M, N = acc.shape
    Y = np.empty((M, N), np.float32)
    bb = None if bias is None else _f32(bias).reshape(-1)
    lib().orc_dequant_bias_relu(_p(acc), _p(sa), _p(sw), _p(bb), _p(Y), M, N, int(bool(relu)))
    return Y


def linear_i8_fwd(A, Wq, sw, bias, relu):
    """Quantise rows of A, int8 GEMM against pre-quantised W, dequant + bias (+ReLU)."""
    A = _f32(A)
    Wq = np.ascontiguousarray(Wq, np.int8)
    sw = _f32(sw)
    M, K = A.shape
    N = Wq.shape[0]
    Y = np.empty((M, N), np.float32)
    bb = None if bias is None else _f32(bias).reshape(-1)
    lib().orc_linear_i8_fwd(_p(A), _p(Wq), _p(sw), _p(bb), _p(Y), M, N, K, int(bool(relu)))
    return Y


# ---------------------------------------------------------------- training steps
class MLPOracle:
    """One f32 training step exactly as the reference CPU path computes it for a
    Sequential of Linear(+ReLU) layers with MSE loss and Adam or AdamW:
    Sequential.forward (nn/models/sequential.v:204-215), Variable.backprop
    (autograd/variable.v:87-109, gradients accumulate onto zeros in f32),
    AdamOptimizer.update (nn/optimizers/adam.v:87-145) or AdamWOptimizer.update
    (nn/optimizers/adamw.v:78-106).  ``relu_after[i]`` tells whether a ReLU layer
    follows Linear i.  ``blas`` switches the GEMMs to OpenBLAS dgemm."""

    def __init__(self, weights, biases, relu_after, lr, beta1=0.9, beta2=0.999, eps=1e-8,
                 weight_decay=None, blas=False):
        self.W = [_f32(w).copy() for w in weights]
        self.b = [_f32(b).reshape(1, -1).copy() for b in biases]
        self.relu_after = list(relu_after)
        self.lr, self.beta1, self.beta2, self.eps = lr, beta1, beta2, eps
        self.wd = weight_decay
        self.beta1_t, self.beta2_t = beta1, beta2
        self.blas = blas
        self.mW = [np.zeros_like(w) for w in self.W]
        self.vW = [np.zeros_like(w) for w in self.W]
        self.mb = [np.zeros_like(b) for b in self.b]
        self.vb = [np.zeros_like(b) for b in self.b]

    def forward(self, X):
        acts, pres = [_f32(X)], []
        h = acts[0]
        for W, b, r in zip(self.W, self.b, self.relu_after):
            pre = linear_fwd_f32(h, W, b, blas=self.blas)
            pres.append(pre)
            h = relu_f32(pre) if r else pre
            acts.append(h)
        return h, acts, pres

    def grads(self, X, T, grad_scale_rows=None):
        y, acts, pres = self.forward(X)
        loss = mse_f32(y, T)
        g = mse_bwd_f32(y, T)
        dWs, dbs = [None] * len(self.W), [None] * len(self.W)
        for i in reversed(range(len(self.W))):
            if self.relu_after[i]:
                g = relu_bwd_f32(g, pres[i])
            dX, dW, db = linear_bwd_f32(g, acts[i], self.W[i], blas=self.blas)
            dWs[i], dbs[i] = dW, db
            g = dX
        return loss, y, dWs, dbs, g

    def apply(self, dWs, dbs):
        lr_t, self.beta1_t, self.beta2_t = adam_lr_t(self.lr, self.beta1_t, self.beta2_t,
                                                      self.beta1, self.beta2)
        for i in range(len(self.W)):
            for (P, G, Mo, Vo) in ((self.W, dWs, self.mW, self.vW), (self.b, dbs, self.mb, self.vb)):
                shp = P[i].shape
                if self.wd is None:
                    th, m, v = adam_step_f32(G[i].ravel(), P[i].ravel(), Mo[i].ravel(),
                                             Vo[i].ravel(), self.beta1, self.beta2, lr_t, self.eps)
                else:
                    th, m, v = adamw_step_f32(G[i].ravel(), P[i].ravel(), Mo[i].ravel(),
                                              Vo[i].ravel(), self.beta1, self.beta2, lr_t,
                                              self.eps, self.wd)
                P[i], Mo[i], Vo[i] = th.reshape(shp), m.reshape(shp), v.reshape(shp)
        return lr_t

    def step(self, X, T):
        loss, y, dWs, dbs, _ = self.grads(X, T)
        self.apply(dWs, dbs)
        return loss


class SequentialOracle:
    """A Sequential of conv2d / relu / maxpool2d / flatten / linear layers with an MSE or
    softmax-cross-entropy loss and Adam, stepped exactly as the reference CPU path does
    (Sequential.forward nn/models/sequential.v:204-215; backprop autograd/variable.v:87-109;
    AdamOptimizer.update nn/optimizers/adam.v:87-145).  `spec` is a list of tuples:
    ("conv2d", W[O,C,kh,kw], b[O], pad, stride) | ("linear", W[N,K], b[N]) | ("relu",) |
    ("maxpool2d", kernel, pad, stride) | ("flatten",)."""

    def __init__(self, spec, loss="mse", lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, blas=False):
        self.spec = [list(s) for s in spec]
        self.loss_kind, self.lr, self.beta1, self.beta2, self.eps = loss, lr, beta1, beta2, eps
        self.beta1_t, self.beta2_t, self.blas = beta1, beta2, blas
        self.params = []  # (layer index, slot) in the order layers declare them (weight, bias)
        for li, s in enumerate(self.spec):
            if s[0] in ("conv2d", "linear"):
                s[1] = _f32(s[1]).copy()
                s[2] = _f32(s[2]).reshape(1, -1).copy()
                self.params += [(li, 1), (li, 2)]
        self.m = [np.zeros_like(self.spec[li][k]) for li, k in self.params]
        self.v = [np.zeros_like(self.spec[li][k]) for li, k in self.params]

    def param(self, i):
        li, k = self.params[i]
        return self.spec[li][k]

    def forward(self, x):
        caches = []
        h = _f32(x)
        for s in self.spec:
            if s[0] == "conv2d":
                caches.append(h)
                h = conv2d_fwd_f32(h, s[1], s[2], pad=s[3], stride=s[4])
            elif s[0] == "linear":
                caches.append(h)
                h = linear_fwd_f32(h, s[1], s[2], blas=self.blas)
            elif s[0] == "relu":
                caches.append(h)
                h = relu_f32(h)
            elif s[0] == "maxpool2d":
                y, idx = maxpool2d_fwd_f32(h, s[1], s[2], s[3])
                caches.append((idx, h.shape))
                h = y
            elif s[0] == "flatten":
                caches.append(h.shape)
                h = h.reshape(h.shape[0], -1)
        return h, caches

    def grads(self, x, t):
        y, caches = self.forward(x)
        if self.loss_kind == "mse":
            loss, g = mse_f32(y, t), mse_bwd_f32(y, t)
        else:
            loss, g = softmax_ce_f32(y, t), softmax_ce_bwd_f32(y, t)
        grads = {}
        for li in reversed(range(len(self.spec))):
            s, c = self.spec[li], caches[li]
            if s[0] == "conv2d":
                g, dw, db = conv2d_bwd_f32(g, c, s[1], pad=s[3], stride=s[4])
                grads[(li, 1)], grads[(li, 2)] = dw, db
            elif s[0] == "linear":
                g, dw, db = linear_bwd_f32(g, c, s[1], blas=self.blas)
                grads[(li, 1)], grads[(li, 2)] = dw, db
            elif s[0] == "relu":
                g = relu_bwd_f32(g, c)
            elif s[0] == "maxpool2d":
                g = maxpool2d_bwd_f32(g, c[0], c[1])
            elif s[0] == "flatten":
                g = g.reshape(c)
        return loss, y, [grads[p] for p in self.params], g

    def step(self, x, t):
        loss, _, grads, _ = self.grads(x, t)
        lr_t, self.beta1_t, self.beta2_t = adam_lr_t(self.lr, self.beta1_t, self.beta2_t, self.beta1,
                                                      self.beta2)
        for i, (li, k) in enumerate(self.params):
            shp = self.spec[li][k].shape
            th, m, v = adam_step_f32(grads[i].ravel(), self.spec[li][k].ravel(), self.m[i].ravel(),
                                     self.v[i].ravel(), self.beta1, self.beta2, lr_t, self.eps)
            self.spec[li][k], self.m[i], self.v[i] = th.reshape(shp), m.reshape(shp), v.reshape(shp)
        return loss
