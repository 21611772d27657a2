"""Checkpoints in the reference's model formats - JSON, bincode (``.bin``) and MessagePack (``.msgpack``) - read and
written from device buffers, with the optimizer state the reference leaves out.  The format follows the file
extension as ``ModelSerializer::save_auto`` / ``load_auto`` do (``engine/src/serialization.rs:490-520``: ``.json``,
``.msgpack``, anything else binary); the two binary encodings are in :mod:`minitensor_b200.serial_formats`.

The layout is what ``serde_json`` produces for ``SerializedModel`` (``engine/src/serialization.rs:345-357``):
``metadata`` (``ModelMetadata``, ``:64-105``, with ``version`` = ``ModelVersion`` ``:20-47``), ``state_dict`` with
``parameters`` and ``buffers`` maps of ``SerializedTensor`` (``:131-190``: ``shape`` = ``{"dims": [...]}``,
``dtype`` = ``"Float32" | "Float64" | "Int32" | "Int64" | "Bool"``, ``device`` = ``{"device_type": "Cpu" |
"Cuda", "device_id": null | n}``, ``data`` = the little-endian bytes as a list of integers, ``requires_grad``) and
``architecture_config``.  Loading checks the byte count of every tensor against its shape and dtype (``:192-280``) and
the major version (``:372-387``).

Optimizer state (absent in the reference): moment buffers are stored as additional entries of ``buffers`` under
``optimizer.<name>`` and scalar state (step count, hyper-parameters) as strings in ``metadata.custom`` - both places
the reference's own loader tolerates.

Parity note: no file written by the reference is available here (it cannot be built), so the field layout is pinned
to the reference's struct definitions and serde's documented conventions, not to a byte-for-byte sample.
"""
from __future__ import annotations

import datetime
import json
import platform
from typing import Dict, Mapping, Optional, Tuple

import numpy as np
import torch

from . import serial_formats

FORMAT_VERSION = (1, 0, 0)          # ModelVersion::current()
ENGINE_VERSION = "minitensor_b200"

_DTYPE_NAMES = {np.dtype(np.float32): "Float32", np.dtype(np.float64): "Float64", np.dtype(np.int32): "Int32",
                np.dtype(np.int64): "Int64", np.dtype(np.bool_): "Bool"}
_NAME_DTYPES = {v: k for k, v in _DTYPE_NAMES.items()}


class SerializationError(RuntimeError):
    """The counterpart of ``MinitensorError::serialization_error``."""


def _to_numpy(t) -> Tuple[np.ndarray, Optional[int], bool]:
    """(host array, CUDA ordinal or None, requires_grad) of a torch tensor, a mirror Tensor or an array."""
    requires_grad = bool(getattr(t, "requires_grad", False))
    buf = getattr(t, "_buf", t)
    if isinstance(buf, torch.Tensor):
        ordinal = buf.device.index if buf.is_cuda else None
        return buf.detach().cpu().contiguous().numpy(), ordinal, requires_grad
    return np.ascontiguousarray(buf), None, requires_grad


def serialize_tensor(t) -> dict:
    arr, ordinal, requires_grad = _to_numpy(t)
    if arr.dtype not in _DTYPE_NAMES:
        raise SerializationError(f"unsupported dtype {arr.dtype}")
    raw = arr.astype(arr.dtype.newbyteorder("<"), copy=False).tobytes()   # one byte per bool, as the reference writes
    return {
        "shape": {"dims": [int(d) for d in arr.shape]},
        "dtype": _DTYPE_NAMES[arr.dtype],
        "device": {"device_type": "Cpu" if ordinal is None else "Cuda", "device_id": ordinal},
        "data": np.frombuffer(raw, dtype=np.uint8),      # a list of integers once it is written as JSON
        "requires_grad": requires_grad,
    }


def deserialize_tensor(obj: Mapping, device: Optional[torch.device] = None) -> torch.Tensor:
    try:
        dims = [int(d) for d in obj["shape"]["dims"]]
        dtype = _NAME_DTYPES[obj["dtype"]]
        data = obj["data"]
    except (KeyError, TypeError) as exc:
        raise SerializationError(f"malformed tensor record: {exc}") from None
    numel = int(np.prod(dims, dtype=np.int64)) if dims else 1
    if len(data) != numel * dtype.itemsize:
        raise SerializationError(f"{obj['dtype']} data size mismatch: expected {numel * dtype.itemsize} bytes, "
                                 f"got {len(data)}")
    raw = np.asarray(data, dtype=np.uint8).tobytes()
    arr = np.frombuffer(raw, dtype=dtype.newbyteorder("<")).astype(dtype).reshape(dims)
    if dtype == np.bool_:
        arr = arr != 0
    t = torch.from_numpy(arr.copy())
    return t.to(device) if device is not None else t


def save_checkpoint(path: str, parameters: Mapping[str, object], buffers: Optional[Mapping[str, object]] = None, *,
                    name: str = "model", architecture: str = "custom", description: Optional[str] = None,
                    optimizer_buffers: Optional[Mapping[str, object]] = None,
                    optimizer_scalars: Optional[Mapping[str, object]] = None,
                    architecture_config: Optional[str] = None) -> None:
    """Write ``parameters`` / ``buffers`` (name -> tensor, device or host) as a ``SerializedModel`` JSON file."""
    all_buffers = {k: serialize_tensor(v) for k, v in (buffers or {}).items()}
    for k, v in (optimizer_buffers or {}).items():
        all_buffers["optimizer." + k] = serialize_tensor(v)
    custom = {"optimizer." + k: repr(v) for k, v in (optimizer_scalars or {}).items()}
    model = {
        "metadata": {
            "name": name,
            "description": description,
            "version": {"major": FORMAT_VERSION[0], "minor": FORMAT_VERSION[1], "patch": FORMAT_VERSION[2],
                        "engine_version": ENGINE_VERSION},
            "created_at": datetime.datetime.now(datetime.timezone.utc).isoformat(),
            "platform": f"{platform.system().lower()}-{platform.machine()}",
            "architecture": architecture,
            "input_shapes": [],
            "output_shapes": [],
            "custom": custom,
        },
        "state_dict": {"parameters": {k: serialize_tensor(v) for k, v in parameters.items()}, "buffers": all_buffers},
        "architecture_config": architecture_config,
    }
    write_model(path, model)


def format_of(path: str) -> str:
    """"json", "msgpack" or "binary" by file extension (``save_auto`` / ``load_auto``)."""
    ext = path.rsplit(".", 1)[-1].lower() if "." in path.rsplit("/", 1)[-1] else ""
    return {"json": "json", "msgpack": "msgpack"}.get(ext, "binary")


def write_model(path: str, model: dict) -> None:
    fmt = format_of(path)
    if fmt == "json":
        class _Enc(json.JSONEncoder):
            def default(self, o):
                if isinstance(o, np.ndarray):
                    return o.tolist()
                return super().default(o)
        with open(path, "w") as f:
            json.dump(model, f, cls=_Enc)
        return
    blob = serial_formats.encode_msgpack(model) if fmt == "msgpack" else serial_formats.encode_bincode(model)
    with open(path, "wb") as f:
        f.write(blob)


def read_model(path: str) -> dict:
    fmt = format_of(path)
    try:
        if fmt == "json":
            with open(path) as f:
                return json.load(f)
        with open(path, "rb") as f:
            blob = f.read()
        return serial_formats.decode_msgpack(blob) if fmt == "msgpack" else serial_formats.decode_bincode(blob)
    except json.JSONDecodeError as exc:
        raise SerializationError(f"JSON deserialization failed: {exc}") from None
    except serial_formats.FormatError as exc:
        kind = "MessagePack" if fmt == "msgpack" else "Binary"
        raise SerializationError(f"{kind} deserialization failed: {exc}") from None


def load_checkpoint(path: str, device: Optional[torch.device] = None):
    """Returns ``(parameters, buffers, optimizer_buffers, optimizer_scalars, metadata)``; tensors go to ``device``."""
    model = read_model(path)
    try:
        meta = model["metadata"]
        version = meta["version"]
        state = model["state_dict"]
    except (KeyError, TypeError) as exc:
        raise SerializationError(f"malformed model file: {exc}") from None
    if int(version["major"]) != FORMAT_VERSION[0]:
        raise SerializationError(
            f"Model version {version['major']}.{version['minor']}.{version['patch']} is not compatible with current "
            f"version {FORMAT_VERSION[0]}.{FORMAT_VERSION[1]}.{FORMAT_VERSION[2]}")
    params = {k: deserialize_tensor(v, device) for k, v in state.get("parameters", {}).items()}
    buffers, opt_buffers = {}, {}
    for k, v in state.get("buffers", {}).items():
        (opt_buffers if k.startswith("optimizer.") else buffers)[k[len("optimizer."):] if k.startswith("optimizer.") else k] = \
            deserialize_tensor(v, device)
    opt_scalars = {}
    for k, v in meta.get("custom", {}).items():
        if k.startswith("optimizer."):
            try:
                opt_scalars[k[len("optimizer."):]] = json.loads(v)
            except (json.JSONDecodeError, TypeError):
                opt_scalars[k[len("optimizer."):]] = v
    return params, buffers, opt_buffers, opt_scalars, meta


# ---------------------------------------------------------------------- the MLP trainer's state
def save_mlp_trainer(trainer, path: str) -> None:
    """Parameters ``layers.<l>.weight`` / ``.bias`` plus Adam's moments and step count."""
    params, opt = {}, {}
    for l in range(trainer.nl):
        params[f"layers.{l}.weight"] = trainer.W[l]
        params[f"layers.{l}.bias"] = trainer.b[l]
    opt["exp_avg"] = trainer.m
    opt["exp_avg_sq"] = trainer.v
    save_checkpoint(path, params, name="mlp", architecture="mlp", optimizer_buffers=opt,
                    optimizer_scalars={"step": trainer.step_count, "lr": trainer.lr, "beta1": trainer.beta1,
                                       "beta2": trainer.beta2, "eps": trainer.eps},
                    architecture_config=json.dumps({"dims": trainer.dims}))


def load_mlp_trainer(trainer, path: str) -> None:
    """Restores what :func:`save_mlp_trainer` wrote into an existing trainer of the same layer sizes."""
    dev = trainer.params.device
    params, _, opt, scalars, _ = load_checkpoint(path, dev)
    for l in range(trainer.nl):
        for kind, dst in (("weight", trainer.W[l]), ("bias", trainer.b[l])):
            src = params.get(f"layers.{l}.{kind}")
            if src is None:
                raise SerializationError(f"Parameter 'layers.{l}.{kind}' not found in state dict")
            if tuple(src.shape) != tuple(dst.shape) or src.dtype != dst.dtype:
                raise SerializationError(f"shape mismatch for layers.{l}.{kind}: {tuple(src.shape)} vs {tuple(dst.shape)}")
            dst.copy_(src)
    if "exp_avg" in opt and "exp_avg_sq" in opt:
        trainer.m.copy_(opt["exp_avg"].reshape(-1))
        trainer.v.copy_(opt["exp_avg_sq"].reshape(-1))
    trainer.step_count = int(scalars.get("step", trainer.step_count))
