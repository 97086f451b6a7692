"""Reading and writing the safetensors container without a third-party package.

The format is: eight bytes (little-endian unsigned length ``n``), ``n`` bytes of JSON that
map each tensor name to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets are
relative to the end of the header), then the raw little-endian tensor bytes.  Files are
memory-mapped, so a tensor's bytes are touched only when that tensor is asked for.

The reference reads every ``*.safetensors`` file of the folder in sorted order into one
dict (src/mini_engine/engine.py:126-128 of YuvGev00/mini-engine); ``read_folder_index``
keeps that behaviour and additionally honours ``model.safetensors.index.json``.
"""

from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Iterable, Mapping

import torch

_DTYPES: dict[str, torch.dtype] = {
    "F64": torch.float64,
    "F32": torch.float32,
    "F16": torch.float16,
    "BF16": torch.bfloat16,
    "I64": torch.int64,
    "I32": torch.int32,
    "I16": torch.int16,
    "I8": torch.int8,
    "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """One memory-mapped file; ``entries`` maps a tensor name to (dtype, shape)."""

    def __init__(self, path: str | Path):
        self.path = Path(path)
        with open(self.path, "rb") as handle:
            head = handle.read(8)
            if len(head) != 8:
                raise ValueError(f"{self.path}: too short to be a safetensors file")
            (header_len,) = struct.unpack("<Q", head)
            header = json.loads(handle.read(header_len))
            self._map = mmap.mmap(handle.fileno(), 0, access=mmap.ACCESS_COPY)
        self._base = 8 + header_len
        self.metadata = header.pop("__metadata__", {})
        self._raw = header
        self.entries: dict[str, tuple[torch.dtype, tuple[int, ...]]] = {}
        for name, info in header.items():
            if info["dtype"] not in _DTYPES:
                raise ValueError(f"{self.path}: tensor {name!r} has unsupported dtype {info['dtype']}")
            self.entries[name] = (_DTYPES[info["dtype"]], tuple(info["shape"]))

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU view of the tensor's bytes in the file (private mapping: no copy until written)."""
        dtype, shape = self.entries[name]
        begin, end = self._raw[name]["data_offsets"]
        count = 1
        for extent in shape:
            count *= extent
        if count == 0:
            return torch.empty(shape, dtype=dtype)
        view = memoryview(self._map)[self._base + begin : self._base + end]
        return torch.frombuffer(view, dtype=dtype, count=count).view(shape)


def read_folder_index(folder: str | Path) -> dict[str, SafetensorsFile]:
    """Tensor name -> the file that holds it, over every safetensors file of a folder."""
    folder = Path(folder)
    index_file = folder / "model.safetensors.index.json"
    files: dict[str, SafetensorsFile] = {}
    where: dict[str, SafetensorsFile] = {}
    if index_file.is_file():
        weight_map = json.loads(index_file.read_text())["weight_map"]
        for name, file_name in weight_map.items():
            if file_name not in files:
                files[file_name] = SafetensorsFile(folder / file_name)
            where[name] = files[file_name]
        return where
    shards = sorted(folder.glob("*.safetensors"))
    if not shards:
        raise FileNotFoundError(f"{folder} holds no .safetensors file")
    for shard in shards:  # later files win, as dict.update does in the reference
        opened = SafetensorsFile(shard)
        for name in opened.entries:
            where[name] = opened
    return where


def write_safetensors(
    path: str | Path, tensors: Mapping[str, torch.Tensor] | Iterable[tuple[str, torch.Tensor]]
) -> None:
    """Write tensors (CPU, any listed dtype) in the order given."""
    items = list(tensors.items()) if isinstance(tensors, Mapping) else list(tensors)
    header: dict[str, dict] = {}
    offset = 0
    for name, tensor in items:
        if tensor.dtype not in _NAMES:
            raise ValueError(f"tensor {name!r} has dtype {tensor.dtype}, which safetensors cannot hold")
        size = tensor.numel() * tensor.element_size()
        header[name] = {
            "dtype": _NAMES[tensor.dtype],
            "shape": list(tensor.shape),
            "data_offsets": [offset, offset + size],
        }
        offset += size
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-len(blob) % 8)  # keep the data 8-byte aligned
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(blob)))
        handle.write(blob)
        for _, tensor in items:
            flat = tensor.detach().contiguous().cpu().reshape(-1)
            handle.write(flat.view(torch.uint8).numpy().tobytes())
