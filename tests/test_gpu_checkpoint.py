"""Checkpoint payloads encoded/decoded on the device, and whole checkpoint files written and read
by the host mirror, against the CPU restatement of the reference's format (byte-exact)."""
import json

import numpy as np
import pytest

from oracle import checkpoint as ock

pytestmark = pytest.mark.gpu


def device_encode(dev, a):
    n = a.size
    length = dev.ckpt_text_len(n)
    d_src = dev.to_device(a)
    d_text = dev.zeros((max(length, 1),), np.uint8)
    dev.ckpt_encode_f32(d_src, n, d_text)
    text = d_text.numpy()[:length].tobytes().decode("ascii")
    d_src.free(); d_text.free()
    return text


def device_decode(dev, text, n):
    raw = np.frombuffer(text.encode("ascii"), np.uint8)
    d_text = dev.to_device(raw if raw.size else np.zeros(1, np.uint8))
    d_dst = dev.zeros((max(n, 1),), np.float32)
    try:
        dev.ckpt_decode_f32(d_text, len(text), d_dst, n)
        return d_dst.numpy()[:n]
    finally:
        d_text.free(); d_dst.free()


@pytest.mark.parametrize("n", [1, 2, 3, 4, 5, 6, 100, 767, 768, 769, 4097, (1 << 20) + 1])
def test_payload_matches_oracle_bytes(dev, n):
    rng = np.random.default_rng(n)
    a = (rng.standard_normal(n) * 10.0 ** rng.integers(-30, 30, n)).astype(np.float32)
    special = np.array([0.0, -0.0, np.inf, -np.inf, 1e-45, -1.17549435e-38, 3.4028235e38], np.float32)
    a[: min(n, special.size)] = special[: min(n, special.size)]
    assert dev.ckpt_text_len(n) == len(ock.encode_payload(a))
    text = device_encode(dev, a)
    assert text == ock.encode_payload(a)
    back = device_decode(dev, text, n)
    assert np.array_equal(back.view(np.uint32), a.view(np.uint32))


def test_known_answers_on_device(dev):
    assert device_encode(dev, np.array([1.0], np.float32)) == "P/AAAAAAAAA="
    assert device_encode(dev, np.array([1.0, -2.5], np.float32)) == "P/AAAAAAAADABAAAAAAAAA=="
    assert dev.ckpt_text_len(0) == 0 and dev.ckpt_text_len(3) == 32 and dev.ckpt_text_len(4) == 44


def test_decode_rounds_f64_to_f32(dev):
    """decode_tensor casts each f64 with a plain conversion: values a checkpoint written from f64
    weights may hold round to the nearest f32."""
    vals = np.array([1.0 + 2.0 ** -30, np.pi, 1e-50, 1e300, -1e300], np.float64)
    text = ock.encode_payload(vals)
    with np.errstate(over="ignore"):
        want = vals.astype(np.float32)
    assert np.array_equal(device_decode(dev, text, vals.size).view(np.uint32), want.view(np.uint32))


def test_decode_rejects_bad_text(dev):
    from vtl_b200.capi import VtlbError
    good = ock.encode_payload(np.arange(5, dtype=np.float32))
    with pytest.raises(VtlbError, match="cannot hold"):
        device_decode(dev, good, 6)
    with pytest.raises(VtlbError, match="outside the base64 alphabet"):
        device_decode(dev, good[:3] + "*" + good[4:], 5)
    with pytest.raises(VtlbError, match="outside the base64 alphabet"):
        device_decode(dev, good[:40] + "?" + good[41:], 5)
    assert good.endswith("==")
    with pytest.raises(VtlbError, match="padding"):
        device_decode(dev, good[:-1] + "A", 5)
    assert dev.check_status() == 0


# ---------------------------------------------------------------- whole files
@pytest.fixture(scope="module")
def sess():
    from vtl_b200 import capi, host
    if capi.device_count() == 0:
        pytest.skip("no CUDA device")
    s = host.Session(0)
    yield s
    s.dev.sync()
    assert s.dev.check_status() == 0
    s.close()


CNN = [("input", [3, 8, 8]), ("conv2d", 3, 4, 3, 3, 1, 1, 1, 1), ("relu",), ("maxpool2d", 2, 2, 0, 0, 2, 2),
       ("flatten",), ("linear", 5)]
MLP = [("input", [6]), ("linear", 7), ("relu",), ("linear", 3)]
BNM = [("input", [2, 4, 4]), ("avgpool2d", 2, 2, 0, 0, 2, 2), ("flatten",), ("linear", 5), ("batchnorm1d", 5),
       ("relu",), ("linear", 3), ("softmax",)]


def build(sess, spec, loss="mse", opt="adam"):
    from vtl_b200 import host
    m = host.Model(sess)
    for item in spec:
        kind = item[0]
        if kind == "input":
            m.input(item[1])
        elif kind == "linear":
            m.linear(item[1])
        elif kind == "relu":
            m.relu()
        elif kind == "flatten":
            m.flatten()
        elif kind == "conv2d":
            m.conv2d(item[1], item[2], (item[3], item[4]), padding=(item[5], item[6]), stride=(item[7], item[8]))
        elif kind == "maxpool2d":
            m.maxpool2d((item[1], item[2]), (item[3], item[4]), (item[5], item[6]))
        elif kind == "avgpool2d":
            m.avgpool2d((item[1], item[2]), (item[3], item[4]), (item[5], item[6]))
        elif kind == "global_avgpool2d":
            m.global_avgpool2d()
        elif kind == "softmax":
            m.softmax()
        elif kind == "batchnorm1d":
            m.batchnorm1d(item[1])
    m.mse_loss() if loss == "mse" else m.softmax_cross_entropy_loss()
    m.adam(lr=1e-2) if opt == "adam" else m.adamw(lr=1e-2)
    return m


def random_params(m, rng):
    ps = [rng.standard_normal(m.param_size(i)).astype(np.float32) for i in range(m.num_params())]
    for i, p in enumerate(ps):
        m.set_param(i, p)
    return ps


@pytest.mark.parametrize("spec", [MLP, CNN, BNM], ids=["mlp", "cnn", "batchnorm"])
def test_saved_file_is_what_the_oracle_writes(sess, tmp_path, spec):
    rng = np.random.default_rng(11)
    m = build(sess, spec)
    ps = random_params(m, rng)
    ours, theirs = tmp_path / "ours.json", tmp_path / "oracle.json"
    m.save_checkpoint(ours, epoch=7, loss=0.25)
    ock.save_checkpoint(theirs, spec, ps, epoch=7, loss=0.25)
    a, b = json.load(open(ours)), json.load(open(theirs))
    assert a == b  # same structure, same configs, byte-identical payload strings
    assert list(a) == ["version", "layers", "layer_data", "optimizer", "metadata"]
    for got, want in zip(ock.load_weights(ours, spec), ps):
        assert np.array_equal(got.reshape(-1), want)
    m.close()


@pytest.mark.parametrize("spec", [MLP, CNN, BNM], ids=["mlp", "cnn", "batchnorm"])
def test_load_weights_from_an_oracle_file(sess, tmp_path, spec):
    from vtl_b200 import host
    rng = np.random.default_rng(12)
    m = build(sess, spec)
    shapes = [m.param_size(i) for i in range(m.num_params())]
    ps = [rng.standard_normal(n).astype(np.float32) for n in shapes]
    path = tmp_path / "oracle.json"
    ock.save_checkpoint(path, spec, ps, epoch=3, loss=1.5)
    m.load_weights(path)
    for i, want in enumerate(ps):
        assert np.array_equal(m.get_param(i).reshape(-1), want)
    assert host.load_checkpoint(path) == (3, 1.5)
    m.close()


def test_load_weights_refuses_what_the_reference_refuses(sess, tmp_path):
    """Error cases of nn/models/serialization_test.v: layer count, layer type, missing weight,
    shape, version."""
    from vtl_b200 import host
    from vtl_b200.capi import VtlbError
    rng = np.random.default_rng(13)
    m = build(sess, MLP)
    ps = random_params(m, rng)
    path = tmp_path / "m.json"

    ock.save_checkpoint(path, MLP[:-1], ps[:2])
    with pytest.raises(VtlbError, match="Layer count mismatch: model has 4, checkpoint has 3"):
        m.load_weights(path)

    other = [("input", [6]), ("linear", 7), ("linear", 7), ("linear", 3)]
    ock.save_checkpoint(path, other, [ps[0], ps[1], np.zeros((7, 7), np.float32), np.zeros((1, 7), np.float32),
                                      ps[2], ps[3]])
    with pytest.raises(VtlbError, match="Layer 2 type mismatch: expected LinearLayer, got ReLULayer"):
        m.load_weights(path)

    wide = [("input", [6]), ("linear", 9), ("relu",), ("linear", 3)]
    ock.save_checkpoint(path, wide, [np.zeros((9, 6), np.float32), np.zeros((1, 9), np.float32),
                                     np.zeros((3, 9), np.float32), ps[3]])
    with pytest.raises(VtlbError, match=r"Shape mismatch: encoded \[9, 6\], expected \[7, 6\]"):
        m.load_weights(path)

    model = ock.save_checkpoint(path, MLP, ps)
    del model["layer_data"][3]["weights"]["bias"]
    json.dump(model, open(path, "w"))
    with pytest.raises(VtlbError, match="Missing weight bias for layer 3"):
        m.load_weights(path)

    model = ock.save_checkpoint(path, MLP, ps)
    model["version"] = "0.1"
    json.dump(model, open(path, "w"))
    with pytest.raises(VtlbError, match="Model version mismatch"):
        m.load_weights(path)

    model = ock.save_checkpoint(path, MLP, ps)
    w = model["layer_data"][1]["weights"]["weight"]
    model["layer_data"][1]["weights"]["weight"] = w[:30] + "#" + w[31:]
    json.dump(model, open(path, "w"))
    with pytest.raises(VtlbError, match="outside the base64 alphabet"):
        m.load_weights(path)

    # numbers follow the JSON grammar: what strtod alone would also take is refused
    text = json.dumps(ock.save_checkpoint(path, MLP, ps))
    for bad in ("nan", "inf", "0x1p3", "-", "1.", "1e"):
        open(path, "w").write(text.replace('"loss": 0.0', f'"loss": {bad}'))
        assert f'"loss": {bad}' in open(path).read()
        with pytest.raises(VtlbError):
            host.load_checkpoint(path)
    m.close()


def test_save_replaces_the_file_only_when_complete(sess, tmp_path):
    """The checkpoint is written beside the target and renamed over it: no temporary file stays
    behind, and a target that cannot be written leaves the previous checkpoint as it was."""
    from vtl_b200 import host
    from vtl_b200.capi import VtlbError
    rng = np.random.default_rng(14)
    m = build(sess, MLP)
    random_params(m, rng)
    path = tmp_path / "m.json"
    m.save_checkpoint(path, epoch=1, loss=0.5)
    first = open(path, "rb").read()
    assert sorted(p.name for p in tmp_path.iterdir()) == ["m.json"]
    random_params(m, rng)
    m.save_checkpoint(path, epoch=2, loss=0.25)
    assert host.load_checkpoint(path) == (2, 0.25) and open(path, "rb").read() != first
    assert sorted(p.name for p in tmp_path.iterdir()) == ["m.json"]
    with pytest.raises(VtlbError):
        m.save_checkpoint(tmp_path / "no_such_dir" / "m.json", epoch=3, loss=0.1)
    assert host.load_checkpoint(path) == (2, 0.25)
    m.close()


@pytest.mark.parametrize("opt", ["adam", "adamw"])
def test_resume_with_optimizer_moments_is_bit_identical(sess, tmp_path, opt):
    """Train 3 steps, save with the optimizer's state, restore into a fresh model, train 2 more:
    the parameters equal those of 5 uninterrupted steps bit for bit."""
    rng = np.random.default_rng(14)
    X = rng.standard_normal((16, 6)).astype(np.float32)
    T = rng.standard_normal((16, 3)).astype(np.float32)
    dX, dT = sess.dev.to_device(X), sess.dev.to_device(T)
    a = build(sess, MLP, opt=opt)
    ps = random_params(a, rng)
    for _ in range(3):
        a.train_step(dX, X.shape, dT, T.shape)
    path = tmp_path / "ckpt.json"
    a.save_checkpoint(path, epoch=3, loss=0.5, with_optimizer=True)
    for _ in range(2):
        a.train_step(dX, X.shape, dT, T.shape)

    b = build(sess, MLP, opt=opt)
    b.load_weights(path, with_optimizer=True)
    stored = json.load(open(path))["optimizer"]
    assert stored["optimizer_type"] == ("AdamOptimizer" if opt == "adam" else "AdamWOptimizer")
    assert stored["config"]["beta1_t"] == pytest.approx(0.9 ** 4) and set(stored["moments"]) == {
        f"{k}_{i}" for i in range(4) for k in ("moment", "second_moment")}
    shapes = [[7, 6], [1, 7], [3, 7], [1, 3]]
    _, first, second = ock.load_moments(path, shapes)
    for i in range(4):
        assert np.array_equal(first[i].reshape(-1), b.get_moment(i).reshape(-1))
        assert np.array_equal(second[i].reshape(-1), b.get_moment(i, second=True).reshape(-1))
    for _ in range(2):
        b.train_step(dX, X.shape, dT, T.shape)
    for i in range(4):
        assert np.array_equal(a.get_param(i).view(np.uint32), b.get_param(i).view(np.uint32))

    c = build(sess, MLP, opt="adamw" if opt == "adam" else "adam")
    from vtl_b200.capi import VtlbError
    with pytest.raises(VtlbError, match="Optimizer type mismatch"):
        c.load_weights(path, with_optimizer=True)
    path2 = tmp_path / "weights_only.json"
    a.save(path2)
    with pytest.raises(VtlbError, match="no optimizer moments"):
        c.load_weights(path2, with_optimizer=True)
    for mdl in (a, b, c):
        mdl.close()
    dX.free(); dT.free()
