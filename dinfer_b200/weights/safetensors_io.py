"""Reader and writer of the safetensors container.

Format (as the reference's own parser reads it, crates/layers/src/weights.rs:1-5,96-130):
8 bytes little-endian header length, a JSON header ``{name: {dtype, shape, data_offsets}}``
(``__metadata__`` is skipped), then the raw little-endian tensor bytes.  Several files in a
folder are read in sorted order.  Tensors are handed out as torch views over a memory map,
so a tensor is copied once, on its way to the device.
"""
from __future__ import annotations

import glob
import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Tuple

import torch

_DTYPES = {
    "F32": (torch.float32, 4),
    "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2),
    "F64": (torch.float64, 8),
    "I64": (torch.int64, 8),
    "I32": (torch.int32, 4),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str            # the container's dtype string, e.g. "BF16"
    shape: Tuple[int, ...]
    start: int            # byte offsets inside the file
    end: int
    file_index: int


class SafetensorsFiles:
    """All ``*.safetensors`` of a folder (or one file), indexed by tensor name."""

    def __init__(self, path: str):
        if os.path.isdir(path):
            files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
            if not files:
                raise SafetensorsError(f"{path}: no *.safetensors file")
        elif os.path.isfile(path):
            files = [path]
        else:
            raise SafetensorsError(f"{path}: no such file or folder")
        self.files: List[str] = files
        self._maps: List[mmap.mmap] = []
        self._handles = []
        self.entries: Dict[str, TensorEntry] = {}
        for i, fn in enumerate(files):
            self._open(i, fn)

    def _open(self, index: int, fn: str) -> None:
        size = os.path.getsize(fn)
        if size < 8:
            raise SafetensorsError(f"{fn}: shorter than its header length field")
        fh = open(fn, "rb")
        mm = mmap.mmap(fh.fileno(), 0, access=mmap.ACCESS_READ)
        self._handles.append(fh)
        self._maps.append(mm)
        (hlen,) = struct.unpack("<Q", mm[:8])
        if 8 + hlen > size:
            raise SafetensorsError(f"{fn}: header length {hlen} exceeds the file")
        try:
            header = json.loads(mm[8:8 + hlen].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{fn}: header is not valid JSON ({e})") from e
        base = 8 + hlen
        for name, info in header.items():
            if name == "__metadata__":
                continue
            dtype = info.get("dtype")
            if dtype not in _DTYPES:
                raise SafetensorsError(f"{fn}: tensor {name!r} has unsupported dtype {dtype!r}")
            shape = tuple(int(x) for x in info["shape"])
            lo, hi = (int(x) for x in info["data_offsets"])
            n = 1
            for s in shape:
                n *= s
            if lo > hi or base + hi > size or hi - lo != n * _DTYPES[dtype][1]:
                raise SafetensorsError(
                    f"{fn}: tensor {name!r} of shape {list(shape)} {dtype} does not fit its "
                    f"byte range [{lo}, {hi})")
            if name in self.entries:
                raise SafetensorsError(f"{fn}: tensor {name!r} appears in two files")
            self.entries[name] = TensorEntry(name, dtype, shape, base + lo, base + hi, index)

    def names(self) -> List[str]:
        return list(self.entries)

    def torch_dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name].dtype][0]

    def tensor(self, name: str) -> torch.Tensor:
        """A read-only CPU view of the tensor's bytes in the memory map."""
        e = self.entries[name]
        dt = _DTYPES[e.dtype][0]
        if e.end == e.start:
            return torch.empty(e.shape, dtype=dt)
        buf = memoryview(self._maps[e.file_index])[e.start:e.end]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")     # "buffer is not writable": it is never written
            t = torch.frombuffer(buf, dtype=dt)
        return t.reshape(e.shape)

    def close(self) -> None:
        for mm in self._maps:
            try:
                mm.close()
            except BufferError:
                pass                            # a view is still alive; freed with it
        for fh in self._handles:
            fh.close()
        self._maps, self._handles = [], []


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]],
                      metadata: Dict[str, str] | None = None) -> None:
    """Write ``(name, tensor)`` pairs as one safetensors file, data aligned to 8 bytes."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blobs: List[Tuple[torch.Tensor, int]] = []
    offset = 0
    for name, t in tensors:
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        t = t.detach().cpu().contiguous()
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        blobs.append((t, nbytes))
        offset += nbytes
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * ((8 - len(raw) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for t, nbytes in blobs:
            if nbytes:
                f.write(memoryview(t.reshape(-1).view(torch.uint8).numpy()))
    os.replace(tmp, path)
