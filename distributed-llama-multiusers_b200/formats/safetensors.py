"""Reader and writer of the safetensors container: an 8-byte little-endian header length, that many bytes of JSON
(name -> {"dtype", "shape", "data_offsets"}), then the tensor bytes.  Only what dense-weight models need: BF16, F32,
F16 and I32 tensors.  The reader maps the file and hands out torch tensors that view it (no copy until `.to()`)."""
from __future__ import annotations

import json
import mmap
import struct
from typing import Dict, Iterable, Tuple

import numpy as np
import torch

_DTYPES = {"BF16": (torch.bfloat16, 2), "F32": (torch.float32, 4), "F16": (torch.float16, 2), "I32": (torch.int32, 4)}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        head = self._f.read(8)
        if len(head) != 8:
            raise ValueError(f"{path}: not a safetensors file")
        (n,) = struct.unpack("<Q", head)
        if n > 100 << 20:
            raise ValueError(f"{path}: header of {n} bytes")
        self.meta = json.loads(self._f.read(n).decode("utf-8"))
        self.meta.pop("__metadata__", None)
        self._base = 8 + n
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        self._buf = np.frombuffer(self._map, dtype=np.uint8)

    def names(self) -> Iterable[str]:
        return self.meta.keys()

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self.meta[name]["shape"])

    def __contains__(self, name: str) -> bool:
        return name in self.meta

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor viewing the mapped file (read-only memory: copy or move it before writing)."""
        e = self.meta[name]
        if e["dtype"] not in _DTYPES:
            raise ValueError(f"{self.path}: tensor {name} has unsupported dtype {e['dtype']}")
        dt, size = _DTYPES[e["dtype"]]
        a, b = e["data_offsets"]
        n = int(np.prod(e["shape"])) if e["shape"] else 1
        if b - a != n * size:
            raise ValueError(f"{self.path}: tensor {name}: {b - a} bytes for shape {e['shape']}")
        raw = self._buf[self._base + a:self._base + b]
        return torch.from_numpy(raw.copy()).view(dt).reshape(e["shape"])

    def close(self):
        self._buf = None
        try:
            self._map.close()
        except BufferError:
            pass
        self._f.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor]):
    meta, off, blobs = {}, 0, []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise ValueError(f"tensor {name}: unsupported dtype {t.dtype}")
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""      # reshape: a tensor without dimensions too
        meta[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    head = json.dumps(meta, separators=(",", ":")).encode("utf-8")
    head += b" " * (-len(head) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for b in blobs:
            f.write(b)
