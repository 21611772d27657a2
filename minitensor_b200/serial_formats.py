"""The two binary encodings of the reference's model file, written and read without the Rust crates.

``ModelSerializer::save`` (``engine/src/serialization.rs:393-446``) writes a ``SerializedModel`` with

* ``bincode::serde::encode_into_std_write(model, w, bincode::config::standard())`` for ``.bin`` - bincode 2.0
  (``engine/Cargo.toml:59``), standard configuration: little-endian, variable-length integers, no field names.
  A value is its fields in declaration order; ``u16/u32/u64/usize`` are varints (below 251 one byte, else a marker
  byte 251 / 252 / 253 followed by the 2 / 4 / 8 little-endian bytes); ``u8`` and ``bool`` one byte; a ``String``,
  a ``Vec`` and a ``HashMap`` start with their length as a varint; ``Option`` is a 0 byte, or a 1 byte and the value;
  a unit enum variant is its index as a ``u32`` varint.
* ``rmp_serde::encode::write(w, model)`` for ``.msgpack`` - rmp-serde 1.3 (``engine/Cargo.toml:60``), default
  serializer: a struct is a MessagePack ARRAY of its fields in declaration order, a map a MessagePack map, ``None``
  is nil, a unit enum variant is its NAME as a string, integers take the shortest encoding, and a ``Vec<u8>`` (no
  ``serde_bytes`` in the reference) is an array of integers, not a bin.

Both are restated from the crates' published format descriptions; no file written by the reference is available
here to compare with byte for byte ("parity unpinned"), so the tests pin the encoders to hand-assembled byte
strings of small values and to round trips.

The model is the same nested ``dict`` the JSON form uses (``checkpoint.py``), except that a tensor's ``data`` may be
a ``numpy`` ``uint8`` array instead of a list; decoding always returns arrays.
"""
from __future__ import annotations

import struct
from typing import Dict, List, Tuple

import numpy as np

DTYPES = ["Float32", "Float64", "Int32", "Int64", "Bool"]           # engine/src/tensor/dtype.rs:12-19
DEVICE_TYPES = ["Cpu", "Cuda", "Metal", "OpenCL"]                   # engine/src/device.rs:12-21


class FormatError(ValueError):
    pass


def _as_u8(data) -> np.ndarray:
    if isinstance(data, np.ndarray):
        if data.dtype != np.uint8:
            raise FormatError("tensor data must be uint8")
        return np.ascontiguousarray(data).reshape(-1)
    return np.asarray(data, dtype=np.uint8).reshape(-1)


# ====================================================================== bincode 2, standard configuration
def _bc_uint(v: int) -> bytes:
    if v < 0:
        raise FormatError("negative value for an unsigned field")
    if v < 251:
        return bytes([v])
    if v < 1 << 16:
        return b"\xfb" + struct.pack("<H", v)
    if v < 1 << 32:
        return b"\xfc" + struct.pack("<I", v)
    if v < 1 << 64:
        return b"\xfd" + struct.pack("<Q", v)
    raise FormatError("integer does not fit in 64 bits")


def _bc_str(s: str) -> bytes:
    b = s.encode("utf-8")
    return _bc_uint(len(b)) + b


def _bc_opt_str(s) -> bytes:
    return b"\x00" if s is None else b"\x01" + _bc_str(s)


def _bc_shape(shape: dict) -> bytes:
    dims = shape["dims"]
    return _bc_uint(len(dims)) + b"".join(_bc_uint(int(d)) for d in dims)


def _bc_tensor(t: dict) -> List[bytes]:
    data = _as_u8(t["data"])
    dev = t["device"]
    dev_id = dev.get("device_id")
    return [_bc_shape(t["shape"]), _bc_uint(DTYPES.index(t["dtype"])), _bc_uint(DEVICE_TYPES.index(dev["device_type"])),
            b"\x00" if dev_id is None else b"\x01" + _bc_uint(int(dev_id)),
            _bc_uint(data.size), data.tobytes(), b"\x01" if t["requires_grad"] else b"\x00"]


def encode_bincode(model: dict) -> bytes:
    m, v = model["metadata"], model["metadata"]["version"]
    out: List[bytes] = [
        _bc_str(m["name"]), _bc_opt_str(m.get("description")),
        _bc_uint(int(v["major"])), _bc_uint(int(v["minor"])), _bc_uint(int(v["patch"])), _bc_str(v["engine_version"]),
        _bc_str(m["created_at"]), _bc_str(m["platform"]), _bc_str(m["architecture"]),
    ]
    for key in ("input_shapes", "output_shapes"):
        shapes = m.get(key, [])
        out.append(_bc_uint(len(shapes)))
        out.extend(_bc_shape(s) for s in shapes)
    custom = m.get("custom", {})
    out.append(_bc_uint(len(custom)))
    for k, val in custom.items():
        out.append(_bc_str(k))
        out.append(_bc_str(val))
    for group in ("parameters", "buffers"):
        tensors = model["state_dict"].get(group, {})
        out.append(_bc_uint(len(tensors)))
        for k, t in tensors.items():
            out.append(_bc_str(k))
            out.extend(_bc_tensor(t))
    out.append(_bc_opt_str(model.get("architecture_config")))
    return b"".join(out)


class _Reader:
    def __init__(self, buf: bytes):
        self.buf = memoryview(buf)
        self.pos = 0

    def take(self, n: int) -> memoryview:
        if n < 0 or self.pos + n > len(self.buf):
            raise FormatError("unexpected end of data")
        v = self.buf[self.pos:self.pos + n]
        self.pos += n
        return v

    def byte(self) -> int:
        return self.take(1)[0]


def _bc_read_uint(r: _Reader) -> int:
    b = r.byte()
    if b < 251:
        return b
    if b == 251:
        return struct.unpack("<H", r.take(2))[0]
    if b == 252:
        return struct.unpack("<I", r.take(4))[0]
    if b == 253:
        return struct.unpack("<Q", r.take(8))[0]
    raise FormatError(f"unsupported integer marker {b}")


def _bc_read_str(r: _Reader) -> str:
    n = _bc_read_uint(r)
    try:
        return bytes(r.take(n)).decode("utf-8")
    except UnicodeDecodeError as exc:
        raise FormatError(f"invalid UTF-8 in a string: {exc}") from None


def _bc_read_bool(r: _Reader) -> bool:
    b = r.byte()
    if b > 1:
        raise FormatError(f"invalid bool / option tag {b}")
    return b == 1


def _bc_read_opt_str(r: _Reader):
    return _bc_read_str(r) if _bc_read_bool(r) else None


def _bc_read_shape(r: _Reader) -> dict:
    return {"dims": [_bc_read_uint(r) for _ in range(_bc_read_uint(r))]}


def _enum(names, idx: int) -> str:
    if idx >= len(names):
        raise FormatError(f"enum variant index {idx} out of range")
    return names[idx]


def _bc_read_tensor(r: _Reader) -> dict:
    shape = _bc_read_shape(r)
    dtype = _enum(DTYPES, _bc_read_uint(r))
    dev_type = _enum(DEVICE_TYPES, _bc_read_uint(r))
    dev_id = _bc_read_uint(r) if _bc_read_bool(r) else None
    n = _bc_read_uint(r)
    data = np.frombuffer(r.take(n), dtype=np.uint8).copy()
    return {"shape": shape, "dtype": dtype, "device": {"device_type": dev_type, "device_id": dev_id}, "data": data,
            "requires_grad": _bc_read_bool(r)}


def decode_bincode(buf: bytes) -> dict:
    r = _Reader(buf)
    meta = {"name": _bc_read_str(r), "description": _bc_read_opt_str(r)}
    meta["version"] = {"major": _bc_read_uint(r), "minor": _bc_read_uint(r), "patch": _bc_read_uint(r),
                       "engine_version": _bc_read_str(r)}
    meta["created_at"], meta["platform"], meta["architecture"] = _bc_read_str(r), _bc_read_str(r), _bc_read_str(r)
    for key in ("input_shapes", "output_shapes"):
        meta[key] = [_bc_read_shape(r) for _ in range(_bc_read_uint(r))]
    meta["custom"] = {}
    for _ in range(_bc_read_uint(r)):
        k = _bc_read_str(r)
        meta["custom"][k] = _bc_read_str(r)
    state: Dict[str, dict] = {}
    for group in ("parameters", "buffers"):
        state[group] = {}
        for _ in range(_bc_read_uint(r)):
            k = _bc_read_str(r)
            state[group][k] = _bc_read_tensor(r)
    cfg = _bc_read_opt_str(r)
    if r.pos != len(r.buf):
        raise FormatError(f"{len(r.buf) - r.pos} trailing bytes after the model")
    return {"metadata": meta, "state_dict": state, "architecture_config": cfg}


# ====================================================================== MessagePack as rmp-serde writes it
def _mp_uint(v: int) -> bytes:
    if v < 0:
        raise FormatError("negative value for an unsigned field")
    if v < 0x80:
        return bytes([v])
    if v < 1 << 8:
        return b"\xcc" + bytes([v])
    if v < 1 << 16:
        return b"\xcd" + struct.pack(">H", v)
    if v < 1 << 32:
        return b"\xce" + struct.pack(">I", v)
    return b"\xcf" + struct.pack(">Q", v)


def _mp_str(s: str) -> bytes:
    b = s.encode("utf-8")
    n = len(b)
    if n < 32:
        return bytes([0xa0 | n]) + b
    if n < 1 << 8:
        return b"\xd9" + bytes([n]) + b
    if n < 1 << 16:
        return b"\xda" + struct.pack(">H", n) + b
    return b"\xdb" + struct.pack(">I", n) + b


def _mp_array_header(n: int) -> bytes:
    if n < 16:
        return bytes([0x90 | n])
    if n < 1 << 16:
        return b"\xdc" + struct.pack(">H", n)
    return b"\xdd" + struct.pack(">I", n)


def _mp_map_header(n: int) -> bytes:
    if n < 16:
        return bytes([0x80 | n])
    if n < 1 << 16:
        return b"\xde" + struct.pack(">H", n)
    return b"\xdf" + struct.pack(">I", n)


def _mp_opt_str(s) -> bytes:
    return b"\xc0" if s is None else _mp_str(s)


def _mp_u8_array(data: np.ndarray) -> bytes:
    """An array of u8 values: below 128 one byte each, otherwise 0xcc and the byte."""
    n = data.size
    big = data >= 128
    start = np.arange(n, dtype=np.int64) + np.cumsum(big) - big       # first byte of every element
    out = np.empty(n + int(big.sum()), dtype=np.uint8)
    out[start[big]] = 0xCC
    out[start + big] = data
    return _mp_array_header(n) + out.tobytes()


def _mp_shape(shape: dict) -> bytes:
    dims = shape["dims"]
    return b"\x91" + _mp_array_header(len(dims)) + b"".join(_mp_uint(int(d)) for d in dims)   # struct Shape { dims }


def _mp_tensor(t: dict) -> List[bytes]:
    dev = t["device"]
    dev_id = dev.get("device_id")
    return [b"\x95", _mp_shape(t["shape"]), _mp_str(t["dtype"]),
            b"\x92" + _mp_str(dev["device_type"]) + (b"\xc0" if dev_id is None else _mp_uint(int(dev_id))),
            _mp_u8_array(_as_u8(t["data"])), b"\xc3" if t["requires_grad"] else b"\xc2"]


def encode_msgpack(model: dict) -> bytes:
    m, v = model["metadata"], model["metadata"]["version"]
    out: List[bytes] = [b"\x93",                                           # SerializedModel: 3 fields
                        b"\x99", _mp_str(m["name"]), _mp_opt_str(m.get("description")),
                        b"\x94", _mp_uint(int(v["major"])), _mp_uint(int(v["minor"])), _mp_uint(int(v["patch"])),
                        _mp_str(v["engine_version"]),
                        _mp_str(m["created_at"]), _mp_str(m["platform"]), _mp_str(m["architecture"])]
    for key in ("input_shapes", "output_shapes"):
        shapes = m.get(key, [])
        out.append(_mp_array_header(len(shapes)))
        out.extend(_mp_shape(s) for s in shapes)
    custom = m.get("custom", {})
    out.append(_mp_map_header(len(custom)))
    for k, val in custom.items():
        out.append(_mp_str(k))
        out.append(_mp_str(val))
    out.append(b"\x92")                                                    # StateDict: 2 fields
    for group in ("parameters", "buffers"):
        tensors = model["state_dict"].get(group, {})
        out.append(_mp_map_header(len(tensors)))
        for k, t in tensors.items():
            out.append(_mp_str(k))
            out.extend(_mp_tensor(t))
    out.append(_mp_opt_str(model.get("architecture_config")))
    return b"".join(out)


def _mp_read_uint(r: _Reader) -> int:
    b = r.byte()
    if b < 0x80:
        return b
    if b == 0xCC:
        return r.byte()
    if b == 0xCD:
        return struct.unpack(">H", r.take(2))[0]
    if b == 0xCE:
        return struct.unpack(">I", r.take(4))[0]
    if b == 0xCF:
        return struct.unpack(">Q", r.take(8))[0]
    raise FormatError(f"expected an unsigned integer, found marker 0x{b:02x}")


def _mp_read_len(r: _Reader, fix_base: int, fix_max: int, m16: int, m32: int, what: str) -> int:
    b = r.byte()
    if fix_base <= b <= fix_base + fix_max:
        return b - fix_base
    if b == m16:
        return struct.unpack(">H", r.take(2))[0]
    if b == m32:
        return struct.unpack(">I", r.take(4))[0]
    raise FormatError(f"expected {what}, found marker 0x{b:02x}")


def _mp_read_array(r: _Reader, expect=None) -> int:
    n = _mp_read_len(r, 0x90, 15, 0xDC, 0xDD, "an array")
    if expect is not None and n != expect:
        raise FormatError(f"expected an array of {expect} fields, found {n}")
    return n


def _mp_read_map(r: _Reader) -> int:
    return _mp_read_len(r, 0x80, 15, 0xDE, 0xDF, "a map")


def _mp_read_str(r: _Reader) -> str:
    b = r.byte()
    if 0xA0 <= b <= 0xBF:
        n = b - 0xA0
    elif b == 0xD9:
        n = r.byte()
    elif b == 0xDA:
        n = struct.unpack(">H", r.take(2))[0]
    elif b == 0xDB:
        n = struct.unpack(">I", r.take(4))[0]
    else:
        raise FormatError(f"expected a string, found marker 0x{b:02x}")
    try:
        return bytes(r.take(n)).decode("utf-8")
    except UnicodeDecodeError as exc:
        raise FormatError(f"invalid UTF-8 in a string: {exc}") from None


def _mp_read_opt_str(r: _Reader):
    if r.buf[r.pos] == 0xC0:
        r.pos += 1
        return None
    return _mp_read_str(r)


def _mp_read_bool(r: _Reader) -> bool:
    b = r.byte()
    if b not in (0xC2, 0xC3):
        raise FormatError(f"expected a bool, found marker 0x{b:02x}")
    return b == 0xC3


def _mp_read_u8_array(r: _Reader) -> np.ndarray:
    """n elements, each one byte below 128 or 0xcc + byte.  Element boundaries without a Python loop: a run of 0xcc
    bytes always starts at an element boundary, and inside it markers and values alternate."""
    n = _mp_read_array(r)
    if n == 0:
        return np.zeros(0, dtype=np.uint8)
    raw = np.frombuffer(r.buf[r.pos:r.pos + min(2 * n, len(r.buf) - r.pos)], dtype=np.uint8)
    is_cc = raw == 0xCC
    idx = np.arange(raw.size, dtype=np.int64)
    run_start = np.maximum.accumulate(np.where(is_cc, -1, idx))       # last non-0xcc position at or before i
    marker = is_cc & (((idx - run_start) & 1) == 1)                    # odd distance from it: a marker
    ends = np.cumsum(~marker)                                          # elements completed after byte i
    stop = int(np.searchsorted(ends, n))                               # byte that completes the n-th element
    if stop >= raw.size or ends[stop] != n or marker[stop]:
        raise FormatError("unexpected end of data inside a byte array")
    used = raw[:stop + 1]
    mk = marker[:stop + 1]
    values = used[~mk]
    # every value at or above 128 must have been introduced by a marker (an unmarked byte up there is another type)
    prev_marker = np.concatenate(([False], mk[:-1]))[~mk]
    if ((values >= 128) & ~prev_marker).any():
        raise FormatError("byte array holds something other than u8 values")
    r.pos += stop + 1
    return values.copy()


def _mp_read_shape(r: _Reader) -> dict:
    _mp_read_array(r, 1)
    return {"dims": [_mp_read_uint(r) for _ in range(_mp_read_array(r))]}


def _named(names, s: str) -> str:
    if s not in names:
        raise FormatError(f"unknown enum variant {s!r}")
    return s


def _mp_read_tensor(r: _Reader) -> dict:
    _mp_read_array(r, 5)
    shape = _mp_read_shape(r)
    dtype = _named(DTYPES, _mp_read_str(r))
    _mp_read_array(r, 2)
    dev_type = _named(DEVICE_TYPES, _mp_read_str(r))
    if r.buf[r.pos] == 0xC0:
        r.pos += 1
        dev_id = None
    else:
        dev_id = _mp_read_uint(r)
    data = _mp_read_u8_array(r)
    return {"shape": shape, "dtype": dtype, "device": {"device_type": dev_type, "device_id": dev_id}, "data": data,
            "requires_grad": _mp_read_bool(r)}


def decode_msgpack(buf: bytes) -> dict:
    r = _Reader(buf)
    try:
        _mp_read_array(r, 3)
        _mp_read_array(r, 9)
        meta = {"name": _mp_read_str(r), "description": _mp_read_opt_str(r)}
        _mp_read_array(r, 4)
        meta["version"] = {"major": _mp_read_uint(r), "minor": _mp_read_uint(r), "patch": _mp_read_uint(r),
                           "engine_version": _mp_read_str(r)}
        meta["created_at"], meta["platform"], meta["architecture"] = _mp_read_str(r), _mp_read_str(r), _mp_read_str(r)
        for key in ("input_shapes", "output_shapes"):
            meta[key] = [_mp_read_shape(r) for _ in range(_mp_read_array(r))]
        meta["custom"] = {}
        for _ in range(_mp_read_map(r)):
            k = _mp_read_str(r)
            meta["custom"][k] = _mp_read_str(r)
        _mp_read_array(r, 2)
        state: Dict[str, dict] = {}
        for group in ("parameters", "buffers"):
            state[group] = {}
            for _ in range(_mp_read_map(r)):
                k = _mp_read_str(r)
                state[group][k] = _mp_read_tensor(r)
        cfg = _mp_read_opt_str(r)
    except IndexError:
        raise FormatError("unexpected end of data") from None
    if r.pos != len(r.buf):
        raise FormatError(f"{len(r.buf) - r.pos} trailing bytes after the model")
    return {"metadata": meta, "state_dict": state, "architecture_config": cfg}
