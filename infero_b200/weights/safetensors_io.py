"""Reader and writer for the safetensors container (no third-party reader on the path).

File = 8-byte little-endian header length, a JSON header mapping each tensor name to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the end of the
header), then the raw little-endian payload.  The checks mirror the reference's
(crates/safetensors/src/lib.rs:390-436): header inside the file, offsets inside the
payload, byte count == prod(shape) * element size; a name present in two shards is an
error (:477-514).
"""
from __future__ import annotations

import glob
import json
import mmap
import os
import struct
import warnings
from dataclasses import dataclass
from typing import Dict, Iterable, Iterator, List, Tuple

import torch

_DTYPES = {
    "F32": (torch.float32, 4),
    "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
    "U8": (torch.uint8, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    begin: int          # absolute byte offset in the file
    nbytes: int
    file: "SafetensorsFile"


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to hold a safetensors header")
        self._fh = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._fh.read(hlen).decode("utf-8"))
        except Exception as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from None
        self.metadata = header.pop("__metadata__", {}) or {}
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size else None
        payload = size - 8 - hlen
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            dt = info.get("dtype")
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unsupported dtype {dt!r}")
            tdtype, esize = _DTYPES[dt]
            shape = tuple(int(s) for s in info["shape"])
            b, e = (int(x) for x in info["data_offsets"])
            n = 1
            for s in shape:
                n *= s
            if b < 0 or e < b or e > payload:
                raise SafetensorsError(f"{path}: tensor '{name}' offsets [{b}, {e}) lie outside the payload")
            if e - b != n * esize:
                raise SafetensorsError(
                    f"{path}: tensor '{name}' holds {e - b} bytes but shape {list(shape)} of {dt} needs {n * esize}")
            self.entries[name] = TensorEntry(name, tdtype, shape, 8 + hlen + b, e - b, self)

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor over the mapped bytes (read-only view; copy before writing)."""
        ent = self.entries[name]
        n = 1
        for s in ent.shape:
            n *= s
        if n == 0:
            return torch.empty(ent.shape, dtype=ent.dtype)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)     # the mapping is read-only by design
            t = torch.frombuffer(self._mm, dtype=ent.dtype, count=n, offset=ent.begin)
        return t.view(ent.shape)

    def close(self):
        try:
            if self._mm is not None:
                self._mm.close()
        except BufferError:
            pass  # tensors still alias the mapping; the OS unmaps at exit
        self._fh.close()


class SafetensorsDir:
    """Every ``*.safetensors`` file of a model folder as one name -> tensor table."""

    def __init__(self, model_dir: str):
        paths = sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
        if not paths:
            raise SafetensorsError(f"{model_dir}: no .safetensors file found")
        self.files = [SafetensorsFile(p) for p in paths]
        self.entries: Dict[str, TensorEntry] = {}
        for f in self.files:
            for name, ent in f.entries.items():
                if name in self.entries:
                    raise SafetensorsError(
                        f"tensor '{name}' appears in both {self.entries[name].file.path} and {f.path}")
                self.entries[name] = ent

    def names(self) -> List[str]:
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        return self.entries[name].file.tensor(name)


def write_safetensors(path: str, decls: List[Tuple[str, torch.dtype, Tuple[int, ...]]],
                      produce, metadata: Dict[str, str] | None = None) -> None:
    """Write tensors one at a time: ``decls`` fixes names, dtypes and shapes (hence the
    header); ``produce(name)`` is then called in order and must return a CPU tensor of that
    dtype and shape.  Peak memory is one tensor."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    for name, dtype, shape in decls:
        n = 1
        for s in shape:
            n *= s
        nbytes = n * _DTYPES[_NAMES[dtype]][1]
        header[name] = {"dtype": _NAMES[dtype], "shape": list(shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name, dtype, shape in decls:
            t = produce(name)
            if tuple(t.shape) != tuple(shape) or t.dtype != dtype:
                raise SafetensorsError(
                    f"write: tensor '{name}' is {t.dtype}{list(t.shape)}, declared {dtype}{list(shape)}")
            t = t.contiguous().cpu()
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dtype != torch.uint8 else t.numpy().tobytes())
    os.replace(tmp, path)
