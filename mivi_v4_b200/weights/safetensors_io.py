"""Reading and writing the safetensors container: an 8-byte little-endian
header length, a JSON header (tensor name -> dtype, shape, byte range), then
the raw little-endian data.

The reference parses its own container with bounds and overflow checks before
it touches any tensor (crates/mivi-model/src/gguf.rs:106-197, limits 12-18);
the same discipline is kept for this format: every offset is checked against
the file before a byte is read.
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

MAX_HEADER_BYTES = 100 * 1024 * 1024

DTYPES = {
    "F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2),
    "F64": (torch.float64, 8), "I32": (torch.int32, 4), "I64": (torch.int64, 8),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in DTYPES.items()}


class SafetensorsError(ValueError):
    """The file is not a well-formed safetensors container."""


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int          # byte range within the file
    end: int
    path: str


def read_header(path: str) -> Dict[str, TensorEntry]:
    try:
        size = os.path.getsize(path)
        f = open(path, "rb")
    except OSError as e:
        raise SafetensorsError(f"{path}: cannot be read ({e.strerror or e})") from None
    with f:
        head = f.read(8)
        if len(head) < 8:
            raise SafetensorsError(f"{path}: {size} bytes is too short for a safetensors file")
        (n,) = struct.unpack("<Q", head)
        if n > MAX_HEADER_BYTES or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} does not fit the file ({size} bytes)")
        try:
            meta = json.loads(f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
    if not isinstance(meta, dict):
        raise SafetensorsError(f"{path}: header is not a JSON object")
    base = 8 + n
    out: Dict[str, TensorEntry] = {}
    for name, info in meta.items():
        if name == "__metadata__":
            continue
        try:
            dtype, shape, (b, e) = info["dtype"], tuple(int(s) for s in info["shape"]), info["data_offsets"]
        except (KeyError, TypeError, ValueError):
            raise SafetensorsError(f"{path}: malformed entry for tensor {name!r}") from None
        if dtype not in DTYPES:
            raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dtype!r}")
        numel = 1
        for s in shape:
            if s < 0:
                raise SafetensorsError(f"{path}: tensor {name!r} has a negative size")
            numel *= s
        if not (0 <= b <= e) or base + e > size or e - b != numel * DTYPES[dtype][1]:
            raise SafetensorsError(
                f"{path}: tensor {name!r} ({dtype} {list(shape)}) claims bytes {b}..{e}, which do not fit "
                f"its size or the file")
        out[name] = TensorEntry(name, dtype, shape, base + b, base + e, path)
    return out


def read_tensor(entry: TensorEntry) -> torch.Tensor:
    """The tensor in its stored dtype, on the CPU, as a copy."""
    dtype, _ = DTYPES[entry.dtype]
    nbytes = entry.end - entry.begin
    if nbytes == 0:
        return torch.empty(entry.shape, dtype=dtype)
    buf = bytearray(nbytes)
    with open(entry.path, "rb") as f:
        f.seek(entry.begin)
        got = f.readinto(buf)
    if got != nbytes:
        raise SafetensorsError(f"{entry.path}: short read of tensor {entry.name!r}")
    return torch.frombuffer(buf, dtype=dtype).reshape(entry.shape)


def read_model_headers(model_dir: str) -> Dict[str, TensorEntry]:
    """Entries of every tensor of a model folder: ``model.safetensors``, or the
    shards that ``model.safetensors.index.json`` lists."""
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(single):
        return read_header(single)
    if os.path.isfile(index):
        with open(index) as f:
            try:
                weight_map = json.load(f)["weight_map"]
            except (json.JSONDecodeError, KeyError, TypeError):
                raise SafetensorsError(f"{index}: no weight_map") from None
        out: Dict[str, TensorEntry] = {}
        if not isinstance(weight_map, dict) or not all(isinstance(v, str) for v in weight_map.values()):
            raise SafetensorsError(f"{index}: weight_map must map tensor names to file names")
        for shard in sorted(set(weight_map.values())):
            path = os.path.join(model_dir, shard)
            if not os.path.isfile(path):
                raise SafetensorsError(f"{index} names the shard {shard!r}, which is not in the folder")
            out.update(read_header(path))
        return out
    raise SafetensorsError(f"{model_dir}: neither model.safetensors nor model.safetensors.index.json")


def write_file(path: str, tensors: Dict[str, torch.Tensor], metadata: Optional[Dict[str, str]] = None) -> None:
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store tensor {name!r} of dtype {t.dtype}")
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hjson += b" " * (-len(hjson) % 8)
    tmp = path + ".part"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for raw in blobs:
            f.write(raw)
    os.replace(tmp, path)
