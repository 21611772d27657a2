"""Checkpoint files in the reference's model layouts (engine/src/serialization.rs) - JSON, bincode, MessagePack:
field names and order, byte encoding, size and version checks, optimizer-state extension.  CPU only."""
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
    assert rec["data"][:4].tolist() == [0, 0, 128, 63]                                   # 1.0f little-endian
    assert ck.serialize_tensor(arrays["flag"])["data"].tolist() == [1, 0, 1]             # one byte per bool
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


# ---------------------------------------------------------------------- binary formats (.bin = bincode 2, .msgpack = rmp-serde)
TINY = {
    "metadata": {"name": "t", "description": None,
                 "version": {"major": 1, "minor": 0, "patch": 0, "engine_version": "0.1.0"},
                 "created_at": "c", "platform": "p", "architecture": "a",
                 "input_shapes": [{"dims": [1, 300]}], "output_shapes": [], "custom": {"k": "v"}},
    "state_dict": {"parameters": {"w": {"shape": {"dims": [2]}, "dtype": "Int32",
                                        "device": {"device_type": "Cuda", "device_id": 3},
                                        "data": [1, 0, 0, 0, 200, 204, 127, 128], "requires_grad": True}},
                   "buffers": {}},
    "architecture_config": "cfg",
}

# bincode 2, standard configuration: fields in declaration order, varint lengths, enum variants by index
TINY_BINCODE = bytes(
    [1]) + b"t" + bytes([0]) + bytes([1, 0, 0]) + bytes([5]) + b"0.1.0" + bytes([1]) + b"c" + bytes([1]) + b"p" + bytes(
    [1]) + b"a" + bytes([1, 2, 1, 0xFB, 0x2C, 0x01]) + bytes([0]) + bytes([1, 1]) + b"k" + bytes([1]) + b"v" + bytes(
    [1, 1]) + b"w" + bytes([1, 2]) + bytes([2]) + bytes([1]) + bytes([1, 3]) + bytes(
    [8, 1, 0, 0, 0, 200, 204, 127, 128]) + bytes([1]) + bytes([0]) + bytes([1, 3]) + b"cfg"

# MessagePack as rmp-serde's default serializer writes it: structs as arrays, unit variants by name, Vec<u8> as an
# array of integers (0xcc before every byte of 128 or more)
TINY_MSGPACK = (b"\x93" + b"\x99" + b"\xa1t" + b"\xc0" + b"\x94\x01\x00\x00\xa50.1.0" + b"\xa1c\xa1p\xa1a" +
                b"\x91\x91\x92\x01\xcd\x01\x2c" + b"\x90" + b"\x81\xa1k\xa1v" +
                b"\x92" + b"\x81\xa1w" + b"\x95" + b"\x91\x91\x02" + b"\xa5Int32" + b"\x92\xa4Cuda\x03" +
                b"\x98\x01\x00\x00\x00\xcc\xc8\xcc\xcc\x7f\xcc\x80" + b"\xc3" + b"\x80" + b"\xa3cfg")


def _same_model(a, b):
    assert a["metadata"] == b["metadata"] and a["architecture_config"] == b["architecture_config"]
    for group in ("parameters", "buffers"):
        assert set(a["state_dict"][group]) == set(b["state_dict"][group])
        for k, t in a["state_dict"][group].items():
            u = b["state_dict"][group][k]
            assert {f: t[f] for f in t if f != "data"} == {f: u[f] for f in u if f != "data"}
            np.testing.assert_array_equal(np.asarray(t["data"], np.uint8), np.asarray(u["data"], np.uint8))


def test_binary_encoders_match_hand_assembled_bytes():
    from minitensor_b200 import serial_formats as sf
    assert sf.encode_bincode(TINY) == TINY_BINCODE
    assert sf.encode_msgpack(TINY) == TINY_MSGPACK
    _same_model(sf.decode_bincode(TINY_BINCODE), TINY)
    _same_model(sf.decode_msgpack(TINY_MSGPACK), TINY)
    # integers at the width boundaries of both encodings
    assert sf._bc_uint(250) == b"\xfa" and sf._bc_uint(251) == b"\xfb\xfb\x00" and sf._bc_uint(65536) == b"\xfc\x00\x00\x01\x00"
    assert sf._bc_uint(2 ** 32) == b"\xfd" + (2 ** 32).to_bytes(8, "little")
    assert sf._mp_uint(127) == b"\x7f" and sf._mp_uint(128) == b"\xcc\x80" and sf._mp_uint(256) == b"\xcd\x01\x00"
    assert sf._mp_uint(70000) == b"\xce\x00\x01\x11\x70" and sf._mp_str("x" * 40)[:2] == b"\xd9\x28"


@pytest.mark.parametrize("ext", ["bin", "msgpack", "json", "ckpt"])
def test_round_trip_in_every_format(tmp_path, ext):
    """Same content through every format the reference's save_auto / load_auto choose by extension (an unknown
    extension means binary), byte runs that stress the MessagePack integer array (runs of 0xcc) included."""
    rng = np.random.default_rng(3)
    arrays = {
        "w": rng.standard_normal((37, 19)).astype(np.float32),
        "d": rng.standard_normal(5),
        "i": np.array([-1, 0xCCCCCC, -0x33333334, 204], np.int32),      # bytes full of 0xcc
        "big": rng.integers(-2 ** 62, 2 ** 62, 70000, dtype=np.int64),  # > 65535 elements: 32-bit array header
        "empty": np.zeros((0, 3), np.float32),
    }
    path = str(tmp_path / f"m.{ext}")
    ck.save_checkpoint(path, {k: torch.from_numpy(v) for k, v in arrays.items()}, {"flag": np.array([True, False])},
                       name="net", architecture="mlp", description="with ünicode",
                       optimizer_buffers={"exp_avg": arrays["w"]}, optimizer_scalars={"step": 12},
                       architecture_config=json.dumps({"dims": [19, 37]}))
    assert ck.format_of(path) == {"bin": "binary", "ckpt": "binary"}.get(ext, ext)
    params, buffers, opt_buffers, opt_scalars, meta = ck.load_checkpoint(path)
    for k, v in arrays.items():
        got = params[k].numpy()
        assert got.dtype == v.dtype and got.shape == v.shape
        np.testing.assert_array_equal(got, v)
    np.testing.assert_array_equal(buffers["flag"].numpy(), [True, False])
    np.testing.assert_array_equal(opt_buffers["exp_avg"].numpy(), arrays["w"])
    assert opt_scalars == {"step": 12} and meta["description"] == "with ünicode" and meta["version"]["major"] == 1


@pytest.mark.parametrize("ext", ["bin", "msgpack"])
def test_damaged_binary_files_are_refused(tmp_path, ext):
    from minitensor_b200 import serial_formats as sf
    good = sf.encode_bincode(TINY) if ext == "bin" else sf.encode_msgpack(TINY)
    path = tmp_path / f"m.{ext}"
    for bad in (good[:-2], good[: len(good) // 2], good + b"\x00", b""):
        path.write_bytes(bad)
        with pytest.raises(ck.SerializationError):
            ck.load_checkpoint(str(path))
    # a tensor whose byte count disagrees with its shape (serialization.rs:192-280)
    model = json.loads(json.dumps(TINY))
    model["state_dict"]["parameters"]["w"]["data"] = [1, 2, 3]
    path.write_bytes(sf.encode_bincode(model) if ext == "bin" else sf.encode_msgpack(model))
    with pytest.raises(ck.SerializationError, match="size mismatch"):
        ck.load_checkpoint(str(path))
    # a file of another major version (serialization.rs:372-387)
    model = json.loads(json.dumps(TINY))
    model["metadata"]["version"]["major"] = 2
    path.write_bytes(sf.encode_bincode(model) if ext == "bin" else sf.encode_msgpack(model))
    with pytest.raises(ck.SerializationError, match="not compatible"):
        ck.load_checkpoint(str(path))
