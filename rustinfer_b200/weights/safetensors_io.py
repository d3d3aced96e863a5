"""Reading and writing the safetensors container.

The format: 8 bytes little-endian header length, a JSON header
{name: {dtype, shape, data_offsets}}, then the raw tensor bytes.  A folder holds either
one `model.safetensors` or a `*.safetensors.index.json` naming shards, as RustInfer's
reader accepts (crates/infer-worker/src/infrastructure/io/safetensors.rs:62-153).
Tensors are views of a memory map; nothing is copied until a tensor is moved to the
device.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Mapping, Tuple

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class _Shard:
    def __init__(self, path: str):
        self.path = path
        self._file = open(path, "rb")
        size = os.fstat(self._file.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        (hlen,) = struct.unpack("<Q", self._file.read(8))
        if 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} exceeds the file")
        try:
            header = json.loads(self._file.read(hlen))
        except json.JSONDecodeError as e:
            raise SafetensorsError(f"{path}: header is not JSON ({e})")
        header.pop("__metadata__", None)
        self.entries: Dict[str, dict] = header
        self._base = 8 + hlen
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ) if size else None
        for name, e in header.items():
            b, end = e["data_offsets"]
            if e["dtype"] not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {e['dtype']}")
            n = 1
            for s in e["shape"]:
                n *= s
            if end - b != n * torch.empty((), dtype=_DTYPES[e["dtype"]]).element_size():
                raise SafetensorsError(
                    f"{path}: tensor '{name}' has {end - b} bytes, shape {e['shape']} needs "
                    f"{n * torch.empty((), dtype=_DTYPES[e['dtype']]).element_size()}")
            if self._base + end > size:
                raise SafetensorsError(f"{path}: tensor '{name}' runs past the end of the file")

    def tensor(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        b, end = e["data_offsets"]
        dtype = _DTYPES[e["dtype"]]
        if end == b:
            return torch.empty(e["shape"], dtype=dtype)
        buf = memoryview(self._map)[self._base + b: self._base + end]
        # A read-only map: torch warns about non-writable buffers; the view is only read.
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            t = torch.frombuffer(buf, dtype=dtype)
        return t.view(e["shape"])


class SafetensorsReader:
    """name -> (dtype, shape) of every tensor of a folder, and the tensors themselves."""

    def __init__(self, folder_or_file: str):
        self._shards: List[_Shard] = []
        self._where: Dict[str, _Shard] = {}
        path = folder_or_file
        if os.path.isdir(path):
            single = os.path.join(path, "model.safetensors")
            index = [f for f in sorted(os.listdir(path)) if f.endswith(".safetensors.index.json")]
            if os.path.isfile(single):
                self._add(single)
            elif index:
                with open(os.path.join(path, index[0])) as f:
                    wm = json.load(f).get("weight_map", {})
                for shard in sorted(set(wm.values())):
                    self._add(os.path.join(path, shard), only={n for n, s in wm.items() if s == shard})
            else:
                files = [f for f in sorted(os.listdir(path)) if f.endswith(".safetensors")]
                if not files:
                    raise SafetensorsError(f"{path}: no .safetensors file in the model folder")
                for f in files:
                    self._add(os.path.join(path, f))
        else:
            self._add(path)

    def _add(self, path: str, only=None) -> None:
        if not os.path.isfile(path):
            raise SafetensorsError(f"{path}: file named by the index does not exist")
        sh = _Shard(path)
        self._shards.append(sh)
        for name in sh.entries:
            if only is None or name in only:
                self._where[name] = sh

    def names(self) -> List[str]:
        return sorted(self._where)

    def __contains__(self, name: str) -> bool:
        return name in self._where

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self._where[name].entries[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self._where[name].entries[name]["dtype"]]

    def tensor(self, name: str) -> torch.Tensor:
        if name not in self._where:
            raise SafetensorsError(f"tensor '{name}' not found")
        return self._where[name].tensor(name)


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor]) -> None:
    """Write `tensors` (CPU, contiguous or not) as one file, names sorted, 8-byte aligned header."""
    header: Dict[str, dict] = {}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor '{name}': dtype {t.dtype} cannot be stored")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + n]}
        offset += n
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-len(blob) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    os.replace(tmp, path)
