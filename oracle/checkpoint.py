"""CPU restatement of the reference's checkpoint format (TEST INFRASTRUCTURE ONLY: imported by
tests/, by the smoke test and by the benchmark's cpu_baseline leg, never by the product path).

Follows nn/models/serialization.v of the reference:
  * encode_tensor (:421-438): every element widened to f64, its bit pattern written most
    significant byte first, the byte string in standard base64 (V's encoding.base64: RFC 4648
    alphabet with '=' padding), prefixed by "<shape, comma separated>;<row_major|col_major>|".
  * decode_tensor (:441-473): the inverse; shape checked against the expected one; each f64
    converted to T with a plain cast.
  * save_checkpoint (:109-262): one JSON object {version, layers[{layer_type, in_shape, config}],
    layer_data[{weights{name: text}}], optimizer{optimizer_type, learning_rate, config, moments},
    metadata{epoch, loss, saved_at, version}}; layer configs as sequential_info.v:40-215 records
    them; the optimizer block is left empty by the reference.
  * load_weights (:279-373) and load_checkpoint (:266-276): version, layer count, layer type,
    weight presence and shape checks with the reference's error texts.
The optimizer moments ("moment_<i>", "second_moment_<i>", config beta1_t / beta2_t) follow the
key names of the reference's own, commented-out loader (:376-417).

Parity unpinned: the reference's tests (nn/models/serialization_test.v) check structure and
round trips only, there is no byte-level golden vector; the KATs in tests/ are derived from the
published definitions of IEEE-754 binary64 and RFC 4648.
"""
from __future__ import annotations

import base64
import json

import numpy as np

MODEL_VERSION = "1.0"  # serialization.v:11


def encode_payload(values) -> str:
    """The base64 text of a flat array (serialization.v:429-437)."""
    be = np.ascontiguousarray(np.asarray(values).reshape(-1).astype(np.float64)).astype(">f8")
    return base64.b64encode(be.tobytes()).decode("ascii")


def decode_payload(text: str, dtype=np.float32) -> np.ndarray:
    """serialization.v:462-471: 8 bytes per element, most significant first, then a plain cast."""
    raw = base64.b64decode(text, validate=True)
    return np.frombuffer(raw[: len(raw) // 8 * 8], dtype=">f8").astype(np.float64).astype(dtype)


def encode_tensor(t: np.ndarray) -> str:
    shape = ",".join(str(int(d)) for d in t.shape)
    return f"{shape};row_major|{encode_payload(t)}"


def decode_tensor(encoded: str, shape, dtype=np.float32) -> np.ndarray:
    parts = encoded.split("|")
    if len(parts) != 2:
        raise ValueError("Invalid tensor encoding: missing shape delimiter")
    shape_str = parts[0].split(";")[0]
    decoded_shape = [int(x) for x in shape_str.split(",")] if shape_str else []
    if list(decoded_shape) != [int(d) for d in shape]:
        raise ValueError(f"Shape mismatch: encoded {decoded_shape}, expected {list(shape)}")
    return decode_payload(parts[1], dtype).reshape(shape)


# ---------------------------------------------------------------- whole files
_WEIGHT_KEYS = {"LinearLayer": ("weight", "bias"), "Conv2DLayer": ("weight", "bias"),
                "BatchNorm1DLayer": ("gamma", "beta")}


def layer_defs(spec):
    """spec: the layer list of tests' SequentialOracle / the host mirror's builder calls:
    ("input", shape) | ("linear", out) | ("relu",) | ("flatten",) |
    ("conv2d", in_ch, out_ch, kh, kw, ph, pw, sh, sw) | ("maxpool2d", kh, kw, ph, pw, sh, sw) |
    ("avgpool2d", kh, kw, ph, pw, sh, sw) | ("global_avgpool2d",) | ("softmax",) | ("batchnorm1d", F).
    Returns [(layer_type, in_shape, config, [param shapes])] as save_checkpoint would see them."""
    out = []
    cur = []
    for item in spec:
        kind = item[0]
        in_shape = list(cur) if out else []
        if kind == "input":
            shape = [int(d) for d in item[1]]
            cfg = {f"shape_{i}": d for i, d in enumerate(shape)}
            out.append(("InputLayer", in_shape, cfg, []))
            cur = shape
        elif kind == "linear":
            fin, fout = int(cur[0]), int(item[1])
            out.append(("LinearLayer", in_shape, {"in_features": fin, "out_features": fout},
                        [[fout, fin], [1, fout]]))
            cur = [fout]
        elif kind == "relu":
            out.append(("ReLULayer", in_shape, {}, []))
        elif kind == "flatten":
            out.append(("FlattenLayer", in_shape, {}, []))
            cur = [int(np.prod(cur))]
        elif kind == "conv2d":
            _, cin, cout, kh, kw, ph, pw, sh, sw = item
            cin = int(cur[0]) if cur and cur[0] > 0 else int(cin)
            cfg = {"in_channels": cin, "out_channels": int(cout), "kernel_h": kh, "kernel_w": kw,
                   "padding_h": ph, "padding_w": pw, "stride_h": sh, "stride_w": sw,
                   "dilation_h": 1, "dilation_w": 1, "groups": 1}
            out.append(("Conv2DLayer", in_shape, cfg, [[int(cout), cin, kh, kw], [1, int(cout)]]))
            oh = (cur[1] + 2 * ph - (kh - 1) - 1) // sh + 1
            ow = (cur[2] + 2 * pw - (kw - 1) - 1) // sw + 1
            cur = [int(cout), oh, ow]
        elif kind == "maxpool2d":
            _, kh, kw, ph, pw, sh, sw = item
            cfg = {"kernel_h": kh, "kernel_w": kw, "padding_h": ph, "padding_w": pw, "stride_h": sh,
                   "stride_w": sw}
            out.append(("MaxPool2DLayer", in_shape, cfg, []))
            cur = [cur[0], (cur[1] + 2 * ph - kh) // sh + 1, (cur[2] + 2 * pw - kw) // sw + 1]
        elif kind == "avgpool2d":
            _, kh, kw, ph, pw, sh, sw = item
            cfg = {"kernel_h": kh, "kernel_w": kw, "padding_h": ph, "padding_w": pw, "stride_h": sh,
                   "stride_w": sw}
            out.append(("AvgPool2DLayer", in_shape, cfg, []))
            cur = [cur[0], (cur[1] + 2 * ph - kh) // sh + 1, (cur[2] + 2 * pw - kw) // sw + 1]
        elif kind == "global_avgpool2d":
            out.append(("GlobalAvgPool2DLayer", in_shape, {}, []))
            cur = [cur[0], 1, 1]
        elif kind == "softmax":
            out.append(("SoftmaxLayer", in_shape, {}, []))
            cur = []  # SoftmaxLayer.output_shape() is empty in the reference (nn/layers/softmax.v:36-38)
        elif kind == "batchnorm1d":
            f = int(item[1])
            out.append(("BatchNorm1DLayer", in_shape, {"num_features": f}, [[1, f], [1, f]]))
            cur = [f]
        else:
            raise ValueError(f"unknown layer {kind}")
    return out


def save_checkpoint(path, spec, params, epoch=0, loss=0.0, optimizer=None):
    """params: flat list of arrays in layer.variables() order.  optimizer (optional):
    {"optimizer_type", "learning_rate", "config": {...}, "first": [...], "second": [...]}."""
    defs = layer_defs(spec)
    layers, data = [], []
    it = iter(params)
    for ltype, in_shape, cfg, shapes in defs:
        weights = {}
        for key, shape in zip(_WEIGHT_KEYS.get(ltype, ()), shapes):
            weights[key] = encode_tensor(np.asarray(next(it), dtype=np.float32).reshape(shape))
        layers.append({"layer_type": ltype, "in_shape": in_shape, "config": cfg})
        data.append({"weights": weights})
    opt = {"optimizer_type": "", "learning_rate": 0.0, "config": {}, "moments": {}}
    if optimizer is not None:
        opt = {"optimizer_type": optimizer["optimizer_type"], "learning_rate": float(optimizer["learning_rate"]),
               "config": {k: float(v) for k, v in optimizer["config"].items()}, "moments": {}}
        for i, (m, v) in enumerate(zip(optimizer["first"], optimizer["second"])):
            opt["moments"][f"moment_{i}"] = encode_tensor(np.asarray(m, dtype=np.float32))
            opt["moments"][f"second_moment_{i}"] = encode_tensor(np.asarray(v, dtype=np.float32))
    model = {"version": MODEL_VERSION, "layers": layers, "layer_data": data, "optimizer": opt,
             "metadata": {"epoch": int(epoch), "loss": float(loss), "saved_at": "vtl_checkpoint",
                          "version": MODEL_VERSION}}
    with open(path, "w") as f:
        json.dump(model, f, separators=(",", ":"))
    return model


def load_checkpoint(path):
    """(epoch, loss) of a checkpoint (serialization.v:266-276)."""
    model = json.load(open(path))
    if model["version"] != MODEL_VERSION:
        raise ValueError(f"Model version mismatch: expected {MODEL_VERSION}, got {model['version']}")
    return int(model["metadata"]["epoch"]), float(model["metadata"]["loss"])


def load_weights(path, spec):
    """The parameter arrays of a checkpoint, checked against `spec` as load_weights checks them
    against the constructed model (serialization.v:279-373)."""
    model = json.load(open(path))
    if model["version"] != MODEL_VERSION:
        raise ValueError(f"Model version mismatch: expected {MODEL_VERSION}, got {model['version']}")
    defs = layer_defs(spec)
    if len(model["layers"]) != len(defs):
        raise ValueError(f"Layer count mismatch: model has {len(defs)}, checkpoint has {len(model['layers'])}")
    out = []
    for i, (ltype, _, _, shapes) in enumerate(defs):
        saved = model["layers"][i]["layer_type"]
        if saved != ltype:
            raise ValueError(f"Layer {i} type mismatch: expected {saved}, got {ltype}")
        weights = model["layer_data"][i]["weights"]
        for key, shape in zip(_WEIGHT_KEYS.get(ltype, ()), shapes):
            if key not in weights:
                raise ValueError(f"Missing weight {key} for layer {i}")
            out.append(decode_tensor(weights[key], shape))
    return out


def load_moments(path, shapes):
    """(optimizer block, first moments, second moments) of a checkpoint that carries them."""
    model = json.load(open(path))
    opt = model["optimizer"]
    first = [decode_tensor(opt["moments"][f"moment_{i}"], s) for i, s in enumerate(shapes)]
    second = [decode_tensor(opt["moments"][f"second_moment_{i}"], s) for i, s in enumerate(shapes)]
    return opt, first, second
