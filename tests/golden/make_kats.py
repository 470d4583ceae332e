"""Writes reference_kats.json: the known-answer vectors the reference's own tests
hold for the dense-contraction path, read from its test files as text (the
reference is V code and cannot be executed here).  Inputs are copied verbatim
from the cited tests; where a test asserts a value it is recorded as asserted;
where a test only compares its GPU path with its CPU path, the expected output
is derived here with plain Python floats from the formula in the cited CPU
function -- independently of oracle/, which these vectors then pin.

    python tests/golden/make_kats.py
"""
import json
import math
import os

kats = {}

# la/la_test.v:30-37 -- matmul(I, B) == B
kats["matmul_identity"] = {
    "source": "la/la_test.v:30-37",
    "a": [[1.0, 0.0], [0.0, 1.0]], "b": [[4.0, 1.0], [2.0, 2.0]],
    "expected": [[4.0, 1.0], [2.0, 2.0]],
}

# autograd_cuda/device_session_test.v:25-48 -- Linear forward, y = x.W^T + b (f64, 1e-9)
x = [1.0, 2.0, 3.0]
w = [[0.1, 0.2, 0.3], [0.4, 0.5, 0.6]]
b = [0.01, 0.02]
y = [sum(xi * wi for xi, wi in zip(x, row)) + bi for row, bi in zip(w, b)]
kats["linear_forward_f64"] = {
    "source": "autograd_cuda/device_session_test.v:25-48; linear_forward_f64_cpu",
    "x": [x], "w": w, "b": b, "expected": [y], "tol": 1e-9,
}

# autograd_cuda/device_session_test.v:50-80 -- Linear backward (f64, 1e-6)
g = [1.0, 0.5]
dx = [sum(g[n] * w[n][k] for n in range(2)) for k in range(3)]
dw = [[g[n] * x[k] for k in range(3)] for n in range(2)]
db = [1.0 * g[0], 1.0 * g[1]]
kats["linear_backward_f64"] = {
    "source": "autograd_cuda/device_session_test.v:50-80; autograd_cuda/linear_backward_f64.v:7-18",
    "grad": [g], "x": [x], "w": w, "dx": [dx], "dw": dw, "db": [db], "tol": 1e-6,
}

# nn/loss/loss_test.v:20-51 -- asserted values
kats["mse"] = {
    "source": "nn/loss/loss_test.v:20-51",
    "cases": [
        {"pred": [1.0, 2.0, 3.0, 4.0], "target": [1.0, 2.0, 3.0, 4.0], "loss": 0.0, "tol": 1e-9},
        {"pred": [2.0, 2.0], "target": [0.0, 0.0], "loss": 4.0, "tol": 1e-6},
        {"pred": [3.0, 1.0], "target": [1.0, 1.0], "grad0": 2.0, "tol": 1e-6},
    ],
}

# nn/optimizers/adam_cuda_d_cuda_test.v:8-34 and :36-62 -- adam_step_f64_cpu (adam_step_f64.v:15-23)
def adam(grad, th, m, v, b1, b2, lr_t, eps):
    th, m, v = list(th), list(m), list(v)
    for i, gi in enumerate(grad):
        m[i] = b1 * m[i] + (1.0 - b1) * gi
        v[i] = b2 * v[i] + (1.0 - b2) * gi * gi
        th[i] -= lr_t * m[i] / (math.sqrt(v[i]) + eps)
    return th, m, v

p = dict(b1=0.9, b2=0.999, lr_t=0.01, eps=1e-8)
th, m, v = adam([1.0, 2.0, 0.5], [3.0, 4.0, 5.0], [0.1, 0.2, 0.3], [0.01, 0.02, 0.03], **p)
kats["adam_one_step_f64"] = {
    "source": "nn/optimizers/adam_cuda_d_cuda_test.v:8-34; nn/optimizers/adam_step_f64.v:15-23",
    "grad": [1.0, 2.0, 0.5], "theta": [3.0, 4.0, 5.0], "m": [0.1, 0.2, 0.3], "v": [0.01, 0.02, 0.03],
    "params": p, "theta_out": th, "m_out": m, "v_out": v, "tol": 1e-6,
}
th, m, v = [2.0, 3.0], [0.0, 0.0], [0.0, 0.0]
for _ in range(2):
    th, m, v = adam([0.5, -0.25], th, m, v, **p)
kats["adam_two_steps_f64"] = {
    "source": "nn/optimizers/adam_cuda_d_cuda_test.v:36-62",
    "grad": [0.5, -0.25], "theta": [2.0, 3.0], "params": p, "theta_out": th, "tol": 1e-5,
}

# nn/internal/conv2d_cuda_test.v:32-59, 85-122 -- 1x1x4x4 input 1..16, 3x3 kernel with ones at
# [0,0] and [1,2]... (flat index 0 and 5), pad 1, stride 1; expected from the loop nest of
# conv2d_forward_cpu_f64 / conv2d_backward_cpu_f64 written out below.
inp = [[float(r * 4 + c + 1) for c in range(4)] for r in range(4)]
ker = [[1.0, 0.0, 0.0], [0.0, 0.0, 1.0], [0.0, 0.0, 0.0]]
flat = [1.0, 0, 0, 0, 0, 1, 0, 0, 0]
ker = [flat[0:3], flat[3:6], flat[6:9]]

def conv_fwd(inp, ker):
    out = [[0.0] * 4 for _ in range(4)]
    for oh in range(4):
        for ow in range(4):
            s = 0.0
            for kh in range(3):
                for kw in range(3):
                    ih, iw = oh - 1 + kh, ow - 1 + kw
                    if 0 <= ih < 4 and 0 <= iw < 4:
                        s += inp[ih][iw] * ker[kh][kw]
            out[oh][ow] = s
    return out

gout = [[0.1 * (r * 4 + c + 1) for c in range(4)] for r in range(4)]
dinp = [[0.0] * 4 for _ in range(4)]
dker = [[0.0] * 3 for _ in range(3)]
for oh in range(4):
    for ow in range(4):
        for kh in range(3):
            for kw in range(3):
                ih, iw = oh - 1 + kh, ow - 1 + kw
                if 0 <= ih < 4 and 0 <= iw < 4:
                    dinp[ih][iw] += gout[oh][ow] * ker[kh][kw]
                    dker[kh][kw] += inp[ih][iw] * gout[oh][ow]
kats["conv2d_4x4"] = {
    "source": "nn/internal/conv2d_cuda_test.v:32-59,85-122; conv2d_forward_cpu_f32.v:26-62; conv2d_backward_cpu_f32.v:26-97",
    "input": inp, "weight": ker, "pad": [1, 1], "stride": [1, 1],
    "forward": conv_fwd(inp, ker), "grad_out": gout,
    "d_input": dinp, "d_weight": dker, "d_bias": sum(sum(r) for r in gout),
    "tol_fwd": 1e-5, "tol_bwd": 1e-4,
}

# nn/internal/conv2d_cuda_test.v:7-19 -- shape only: 4x4 input, 2x2 kernel, no pad -> [1,1,3,3]
kats["conv2d_shape"] = {"source": "nn/internal/conv2d_cuda_test.v:7-19",
                        "in": [1, 1, 4, 4], "kernel": [2, 2], "pad": [0, 0], "out": [1, 1, 3, 3]}

# nn/optimizers/adamw.v:78-106 -- no reference test holds an AdamW value; one step derived by hand
# from the update's closures, (a) in the textbook operand order this build implements and (b) with
# the operands as the closures receive them from Tensor.napply (fun.v:37-44: vals[0] is the receiver,
# i.e. the moment tensor; vals[1] the gradient).  State is f32, each closure computes in f64 and
# casts its result to f32 (vtl.cast[T]); f32() below rounds a Python float the same way.
import struct


def f32(x):
    return struct.unpack("f", struct.pack("f", x))[0]


aw = dict(b1=0.9, b2=0.999, lr_t=0.01, eps=1e-8, wd=0.01)
aw_g, aw_th, aw_m, aw_v = [1.0, 2.0, 0.5, -0.25], [3.0, 4.0, 5.0, -1.5], [0.125, 0.25, 0.375, 0.0], [0.015625, 0.03125, 0.0625, 0.0]


def adamw(order):
    th, m, v = list(aw_th), list(aw_m), list(aw_v)
    for i, g in enumerate(aw_g):
        if order == "textbook":
            m[i] = f32(aw["b1"] * m[i] + (1.0 - aw["b1"]) * g)
            v[i] = f32(aw["b2"] * v[i] + (1.0 - aw["b2"]) * g * g)
        else:  # adamw.v:86-93 literally: vals[0] = moment, vals[1] = gradient
            m[i] = f32(aw["b1"] * g + (1.0 - aw["b1"]) * m[i])
            v[i] = f32(aw["b2"] * g + (1.0 - aw["b2"]) * v[i] * v[i])
    for i in range(len(th)):
        if v[i] < 0.0:  # the as-written second moment goes negative with a negative gradient
            th[i] = float("nan")
            continue
        th[i] = f32(th[i] - aw["lr_t"] * (m[i] / (math.sqrt(v[i]) + aw["eps"]) + aw["wd"] * th[i]))
    return th, m, v


tb, aswr = adamw("textbook"), adamw("as_written")
kats["adamw_one_step_f32"] = {
    "source": "nn/optimizers/adamw.v:78-106 (no value asserted by any reference test); fun.v:37-44 for the "
              "operand order of napply",
    "grad": aw_g, "theta": aw_th, "m": aw_m, "v": aw_v, "params": aw,
    "textbook": {"theta_out": tb[0], "m_out": tb[1], "v_out": tb[2]},
    "as_written": {"theta_out": [None if t != t else t for t in aswr[0]], "m_out": aswr[1], "v_out": aswr[2]},
}

here = os.path.dirname(os.path.abspath(__file__))
with open(os.path.join(here, "reference_kats.json"), "w") as f:
    json.dump(kats, f, indent=1)
print("wrote", len(kats), "KAT groups")
