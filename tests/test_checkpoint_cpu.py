"""Checkpoint format on the CPU: the oracle against known answers worked out from the
definitions (IEEE-754 binary64, RFC 4648), and the host library's reader on oracle-written files
(no GPU involved: load_checkpoint only parses)."""
import json

import numpy as np
import pytest

from oracle import checkpoint as ock

MLP = [("input", [4]), ("linear", 3), ("relu",), ("linear", 2)]


def mlp_params(rng):
    return [rng.standard_normal((3, 4)).astype(np.float32), rng.standard_normal((1, 3)).astype(np.float32),
            rng.standard_normal((2, 3)).astype(np.float32), rng.standard_normal((1, 2)).astype(np.float32)]


def test_payload_known_answers():
    # 1.0 = 0x3FF0000000000000: 3F F0 00 | 00 00 00 | 00 00 -> "P/AA" "AAAA" "AAA="
    assert ock.encode_payload([1.0]) == "P/AAAAAAAAA="
    # -2.5 = 0xC004000000000000: C0 04 00 -> 110000 000000 010000 000000 = "wAQA"
    assert ock.encode_payload([-2.5]) == "wAQAAAAAAAA="
    # two values: 16 bytes -> 22 characters + "=="
    assert ock.encode_payload([1.0, -2.5]) == "P/AAAAAAAADABAAAAAAAAA=="
    # three values fill 24 bytes exactly: no padding
    three = ock.encode_payload([1.0, -2.5, 0.0])
    assert len(three) == 32 and "=" not in three and three.startswith("P/AAAAAAAADABAAAAAAAAA")
    assert ock.encode_payload([]) == ""


def test_tensor_header_and_round_trip():
    rng = np.random.default_rng(0)
    t = rng.standard_normal((2, 3)).astype(np.float32)
    enc = ock.encode_tensor(t)
    assert enc.startswith("2,3;row_major|")
    back = ock.decode_tensor(enc, [2, 3])
    assert back.dtype == np.float32 and np.array_equal(back.view(np.uint32), t.view(np.uint32))
    with pytest.raises(ValueError, match="Shape mismatch"):
        ock.decode_tensor(enc, [3, 2])
    with pytest.raises(ValueError, match="missing shape delimiter"):
        ock.decode_tensor("2,3;row_major", [2, 3])


def test_special_values_survive():
    vals = np.array([0.0, -0.0, np.inf, -np.inf, 1e-45, -1.17549435e-38, 3.4028235e38], np.float32)
    back = ock.decode_payload(ock.encode_payload(vals))
    assert np.array_equal(back.view(np.uint32), vals.view(np.uint32))


def test_file_structure_matches_the_reference_layout(tmp_path):
    """What nn/models/serialization_test.v checks on a saved file: version, layer types, weight
    names per layer, empty weights for activations, metadata."""
    rng = np.random.default_rng(1)
    path = tmp_path / "m.json"
    ock.save_checkpoint(path, MLP, mlp_params(rng), epoch=42, loss=0.123)
    model = json.load(open(path))
    assert list(model) == ["version", "layers", "layer_data", "optimizer", "metadata"]
    assert model["version"] == "1.0"
    assert [l["layer_type"] for l in model["layers"]] == ["InputLayer", "LinearLayer", "ReLULayer", "LinearLayer"]
    assert model["layers"][1]["config"] == {"in_features": 4, "out_features": 3}
    assert model["layers"][1]["in_shape"] == [4] and model["layers"][0]["in_shape"] == []
    assert set(model["layer_data"][1]["weights"]) == {"weight", "bias"}
    assert model["layer_data"][2]["weights"] == {}
    assert model["metadata"] == {"epoch": 42, "loss": 0.123, "saved_at": "vtl_checkpoint", "version": "1.0"}
    assert ock.load_checkpoint(path) == (42, 0.123)


def test_oracle_load_weights_checks(tmp_path):
    rng = np.random.default_rng(2)
    params = mlp_params(rng)
    path = tmp_path / "m.json"
    ock.save_checkpoint(path, MLP, params)
    for a, b in zip(ock.load_weights(path, MLP), params):
        assert np.array_equal(a, b)
    with pytest.raises(ValueError, match="Layer count mismatch"):
        ock.load_weights(path, MLP[:-1])
    with pytest.raises(ValueError, match="type mismatch"):
        ock.load_weights(path, [("input", [4]), ("linear", 3), ("linear", 3), ("linear", 2)])
    with pytest.raises(ValueError, match="Shape mismatch"):
        ock.load_weights(path, [("input", [4]), ("linear", 5), ("relu",), ("linear", 2)])
    model = json.load(open(path))
    model["version"] = "0.9"
    json.dump(model, open(path, "w"))
    with pytest.raises(ValueError, match="version mismatch"):
        ock.load_weights(path, MLP)


def test_host_library_reads_checkpoint_metadata(tmp_path):
    """The C++ reader (no device needed for the metadata) on an oracle-written file."""
    from vtl_b200 import capi, host
    rng = np.random.default_rng(3)
    path = tmp_path / "m.json"
    ock.save_checkpoint(path, MLP, mlp_params(rng), epoch=100, loss=0.00123)
    assert host.load_checkpoint(path) == (100, 0.00123)
    model = json.load(open(path))
    model["version"] = "2.0"
    json.dump(model, open(path, "w"))
    with pytest.raises(capi.VtlbError, match="Model version mismatch: expected 1.0, got 2.0"):
        host.load_checkpoint(path)
    open(path, "w").write('{"version": "1.0", "layers": [')
    with pytest.raises(capi.VtlbError, match="malformed JSON"):
        host.load_checkpoint(path)
    with pytest.raises(capi.VtlbError, match="cannot open"):
        host.load_checkpoint(tmp_path / "absent.json")
