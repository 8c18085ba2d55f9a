"""Reading and writing safetensors files, by tensor name, without any model library.

File layout: 8 bytes little-endian header length N, N bytes of JSON
``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}``, then the
raw little-endian tensor bytes. A folder holds ``model.safetensors``, or several shards named by
``model.safetensors.index.json`` (``weight_map``: tensor name -> file).

The reference reads one ``<name>.bin`` file per tensor (cpp/src/serialize.cpp:11-66) and checks
magic, sizes and trailing bytes there; the same checks are made here on the safetensors header.
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, List, Tuple

import numpy as np
import torch


class SafetensorsError(ValueError):
    pass


# safetensors dtype tag -> (numpy storage dtype, torch dtype, bytes per element)
_DTYPES = {
    "F64": (np.float64, torch.float64, 8),
    "F32": (np.float32, torch.float32, 4),
    "F16": (np.float16, torch.float16, 2),
    "BF16": (np.uint16, torch.bfloat16, 2),
    "I64": (np.int64, torch.int64, 8),
    "I32": (np.int32, torch.int32, 4),
    "I16": (np.int16, torch.int16, 2),
    "I8": (np.int8, torch.int8, 1),
    "U8": (np.uint8, torch.uint8, 1),
    "BOOL": (np.bool_, torch.bool, 1),
}
_TAG_OF_TORCH = {v[1]: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """One file, memory-mapped; tensors are materialised on request."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file ({size} bytes)")
        with open(path, "rb") as f:
            (n,) = struct.unpack("<Q", f.read(8))
            if n <= 0 or 8 + n > size:
                raise SafetensorsError(f"{path}: header length {n} does not fit the file ({size} bytes)")
            raw = f.read(n)
        try:
            header = json.loads(raw.decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON ({e})") from e
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self.metadata = header.pop("__metadata__", {}) or {}
        self.data_start = 8 + n
        self.data_size = size - self.data_start
        self.entries: Dict[str, dict] = {}
        for name, e in header.items():
            try:
                tag, shape, (b, end) = e["dtype"], tuple(int(x) for x in e["shape"]), e["data_offsets"]
            except (KeyError, TypeError, ValueError) as ex:
                raise SafetensorsError(f"{path}: malformed header entry for '{name}'") from ex
            if tag not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {tag}")
            if any(d < 0 for d in shape):
                raise SafetensorsError(f"{path}: tensor '{name}' has a negative dimension {shape}")
            count = int(np.prod(shape, dtype=np.int64)) if shape else 1
            if end - b != count * _DTYPES[tag][2]:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' {tag}{list(shape)} needs {count * _DTYPES[tag][2]} bytes, "
                    f"header gives {end - b}")
            if b < 0 or end > self.data_size:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' lies outside the file (truncated file?)")
            self.entries[name] = {"dtype": tag, "shape": shape, "begin": b, "end": end}
        self._mmap = None

    def names(self) -> List[str]:
        return list(self.entries)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.entries[name]["shape"]

    def dtype_tag(self, name: str) -> str:
        return self.entries[name]["dtype"]

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that owns its memory (a copy out of the mapped file)."""
        e = self.entries[name]
        if self._mmap is None:
            self._mmap = np.memmap(self.path, dtype=np.uint8, mode="r", offset=self.data_start,
                                   shape=(self.data_size,)) if self.data_size else np.zeros(0, np.uint8)
        np_dtype, torch_dtype, _ = _DTYPES[e["dtype"]]
        buf = np.array(self._mmap[e["begin"]:e["end"]])  # copy
        arr = buf.view(np_dtype).reshape(e["shape"])
        t = torch.from_numpy(arr)
        if e["dtype"] == "BF16":
            t = t.view(torch.bfloat16)
        return t


def open_model_files(model_dir: str) -> List[SafetensorsFile]:
    """The safetensors files of a model folder (single file, or the shards of its index)."""
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            weight_map = json.load(f).get("weight_map", {})
        files = sorted(set(weight_map.values()))
        if not files:
            raise SafetensorsError(f"{index}: empty weight_map")
        return [SafetensorsFile(os.path.join(model_dir, fn)) for fn in files]
    if os.path.isfile(single):
        return [SafetensorsFile(single)]
    shards = sorted(fn for fn in os.listdir(model_dir) if fn.endswith(".safetensors")) \
        if os.path.isdir(model_dir) else []
    if not shards:
        raise SafetensorsError(f"no model.safetensors in '{model_dir}'")
    return [SafetensorsFile(os.path.join(model_dir, fn)) for fn in shards]


def save_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] = None) -> None:
    """Write ``tensors`` (CPU, contiguous) to ``path`` in name order."""
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _TAG_OF_TORCH:
            raise SafetensorsError(f"cannot store tensor '{name}' of dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _TAG_OF_TORCH[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * ((8 - len(raw) % 8) % 8)
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            if t.dtype == torch.bfloat16:
                t = t.view(torch.int16)
            f.write(t.numpy().tobytes())
