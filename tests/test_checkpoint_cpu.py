"""Checkpoint files in the reference's JSON model layout (engine/src/serialization.rs): field names, byte
encoding, size and version checks, optimizer-state extension.  CPU only."""
import json

import numpy as np
import pytest
import torch

from minitensor_b200 import checkpoint as ck


def test_tensor_record_layout_and_round_trip(tmp_path):
    arrays = {
        "f32": np.array([[1.0, -2.5], [3.25, 4.0]], np.float32),
        "f64": np.array([1e-300, 2.0], np.float64),
        "i32": np.array([-7, 2**31 - 1], np.int32),
        "i64": np.array([[-(2**62)], [5]], np.int64),
        "flag": np.array([True, False, True]),
        "scalar": np.array(3.5, np.float32),
    }
    rec = ck.serialize_tensor(arrays["f32"])
    assert set(rec) == {"shape", "dtype", "device", "data", "requires_grad"}            # SerializedTensor's fields
    assert rec["shape"] == {"dims": [2, 2]} and rec["dtype"] == "Float32"
    assert rec["device"] == {"device_type": "Cpu", "device_id": None} and rec["requires_grad"] is False
    assert rec["data"][:4] == [0, 0, 128, 63]                                            # 1.0f little-endian
    assert ck.serialize_tensor(arrays["flag"])["data"] == [1, 0, 1]                      # one byte per bool
    path = tmp_path / "m.json"
    ck.save_checkpoint(str(path), {k: torch.from_numpy(v) for k, v in arrays.items() if k != "flag"},
                       {"flag": arrays["flag"]}, name="net", architecture="mlp", description="d",
                       optimizer_buffers={"exp_avg": arrays["f32"]}, optimizer_scalars={"step": 7, "lr": 1e-3})
    doc = json.loads(path.read_text())
    assert set(doc) == {"metadata", "state_dict", "architecture_config"}                 # SerializedModel
    assert set(doc["metadata"]) == {"name", "description", "version", "created_at", "platform", "architecture",
                                    "input_shapes", "output_shapes", "custom"}          # ModelMetadata
    assert set(doc["metadata"]["version"]) == {"major", "minor", "patch", "engine_version"}
    assert set(doc["state_dict"]) == {"parameters", "buffers"}
    params, buffers, opt_buffers, opt_scalars, meta = ck.load_checkpoint(str(path))
    for k, v in arrays.items():
        got = (buffers if k == "flag" else params)[k].numpy()
        assert got.dtype == v.dtype and got.shape == v.shape
        np.testing.assert_array_equal(got, v)
    np.testing.assert_array_equal(opt_buffers["exp_avg"].numpy(), arrays["f32"])
    assert opt_scalars == {"step": 7, "lr": 0.001} and meta["name"] == "net"


def test_loads_a_record_written_in_the_reference_layout(tmp_path):
    """A file assembled by hand from the reference's struct definitions (what serde_json writes for them)."""
    doc = {
        "metadata": {"name": "tiny", "description": None,
                     "version": {"major": 1, "minor": 0, "patch": 0, "engine_version": "0.1.0"},
                     "created_at": "2025-01-01T00:00:00+00:00", "platform": "linux-x86_64", "architecture": "dense",
                     "input_shapes": [{"dims": [1, 2]}], "output_shapes": [], "custom": {}},
        "state_dict": {"parameters": {"weight": {"shape": {"dims": [1, 2]}, "dtype": "Float32",
                                                 "device": {"device_type": "Cpu", "device_id": None},
                                                 "data": [0, 0, 128, 63, 0, 0, 0, 192], "requires_grad": True}},
                       "buffers": {}},
        "architecture_config": None,
    }
    path = tmp_path / "ref.json"
    path.write_text(json.dumps(doc, indent=2))                                           # to_writer_pretty
    params, buffers, opt_b, opt_s, _ = ck.load_checkpoint(str(path))
    np.testing.assert_array_equal(params["weight"].numpy(), np.array([[1.0, -2.0]], np.float32))
    assert not buffers and not opt_b and not opt_s


def test_size_and_version_checks(tmp_path):
    good = ck.serialize_tensor(np.zeros(3, np.float32))
    bad = dict(good, data=good["data"][:-1])
    with pytest.raises(ck.SerializationError, match="size mismatch"):
        ck.deserialize_tensor(bad)
    with pytest.raises(ck.SerializationError):
        ck.deserialize_tensor({"shape": {"dims": [1]}, "dtype": "Float16", "data": [0, 0]})
    path = tmp_path / "v2.json"
    ck.save_checkpoint(str(path), {"w": np.zeros(1, np.float32)})
    doc = json.loads(path.read_text())
    doc["metadata"]["version"]["major"] = 2
    path.write_text(json.dumps(doc))
    with pytest.raises(ck.SerializationError, match="not compatible"):
        ck.load_checkpoint(str(path))
    doc["metadata"]["version"] = {"major": 1, "minor": 9, "patch": 3, "engine_version": "x"}   # same major: accepted
    path.write_text(json.dumps(doc))
    ck.load_checkpoint(str(path))
    path.write_text("{not json")
    with pytest.raises(ck.SerializationError):
        ck.load_checkpoint(str(path))
