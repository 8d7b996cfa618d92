"""Reader and writer for the safetensors container.

Layout (the reference parses the same in src/safetensors.cpp:12-53): an
unsigned 64-bit little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [begin, end]}}`` (the entry
``__metadata__`` is skipped), then the raw little-endian tensor bytes, whose
offsets count from the end of the header.  All ``*.safetensors`` files of a
folder are read, in sorted order (safetensors.cpp:40-53).

Files are memory-mapped; a tensor's bytes are touched only when it is loaded.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass

import numpy as np
import torch

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: torch.dtype
    shape: tuple
    file_index: int
    begin: int      # absolute byte offsets in the file
    end: int


class SafetensorsFolder:
    """Index of every tensor in a model folder (or in one file)."""

    def __init__(self, path: str):
        if os.path.isdir(path):
            files = sorted(os.path.join(path, f) for f in os.listdir(path) if f.endswith(".safetensors"))
        else:
            files = [path]
        if not files:
            raise SafetensorsError(f"no *.safetensors file in {path}")
        self.files = files
        self._maps: list = [None] * len(files)
        self.tensors: dict[str, TensorInfo] = {}
        for i, fn in enumerate(files):
            self._read_header(i, fn)

    def _read_header(self, idx: int, fn: str) -> None:
        size = os.path.getsize(fn)
        with open(fn, "rb") as f:
            head = f.read(8)
            if len(head) != 8:
                raise SafetensorsError(f"{fn}: shorter than its 8-byte header length")
            (n,) = struct.unpack("<Q", head)
            if n <= 0 or 8 + n > size:
                raise SafetensorsError(f"{fn}: header length {n} does not fit the file ({size} bytes)")
            try:
                header = json.loads(f.read(n).decode("utf-8"))
            except (UnicodeDecodeError, json.JSONDecodeError) as e:
                raise SafetensorsError(f"{fn}: header is not valid JSON ({e})") from None
        base = 8 + n
        for name, ent in header.items():
            if name == "__metadata__":
                continue
            try:
                dt, item = _DTYPES[ent["dtype"]]
            except KeyError:
                raise SafetensorsError(f"{fn}: tensor {name!r} has unsupported dtype {ent.get('dtype')!r}") from None
            shape = tuple(int(s) for s in ent["shape"])
            b, e = (int(x) for x in ent["data_offsets"])
            count = int(np.prod(shape, dtype=np.int64)) if shape else 1
            if e - b != count * item or b < 0 or base + e > size:
                raise SafetensorsError(
                    f"{fn}: tensor {name!r} claims bytes [{b}, {e}) for shape {list(shape)} {ent['dtype']}; "
                    f"that does not fit ({count * item} bytes needed, {size - base} in the file)")
            if name in self.tensors:
                raise SafetensorsError(f"tensor {name!r} appears in more than one file")
            self.tensors[name] = TensorInfo(name, dt, shape, idx, base + b, base + e)

    def __contains__(self, name: str) -> bool:
        return name in self.tensors

    def names(self) -> list[str]:
        return list(self.tensors)

    def _map(self, idx: int):
        if self._maps[idx] is None:
            with open(self.files[idx], "rb") as f:
                self._maps[idx] = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        return self._maps[idx]

    def load(self, name: str) -> torch.Tensor:
        """The tensor in its stored dtype, as a CPU tensor that owns its memory."""
        info = self.tensors[name]
        mm = self._map(info.file_index)
        nbytes = info.end - info.begin
        if nbytes == 0:
            return torch.empty(info.shape, dtype=info.dtype)
        raw = np.frombuffer(mm, dtype=np.uint8, count=nbytes, offset=info.begin)
        t = torch.from_numpy(raw.copy()).view(info.dtype)
        return t.reshape(info.shape)

    def close(self) -> None:
        for m in self._maps:
            if m is not None:
                m.close()
        self._maps = [None] * len(self.files)


def save_safetensors(path: str, tensors: dict[str, torch.Tensor], metadata: dict | None = None) -> None:
    """Write one file; tensors are laid out in the order given, each aligned to 8 bytes."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        raw = t.view(torch.uint8).reshape(-1).numpy() if t.numel() else np.zeros(0, np.uint8)
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + raw.nbytes]}
        blobs.append(raw)
        off += raw.nbytes
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for raw in blobs:
            f.write(raw.tobytes())
    os.replace(tmp, path)
