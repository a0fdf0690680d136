"""Reader and writer for the safetensors container (no third-party reader on the path).

File = 8-byte little-endian header length, a JSON header mapping each tensor name to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the end of the
header), then the raw little-endian payload.  The checks mirror the reference's
(crates/safetensors/src/lib.rs:390-436): header inside the file, offsets inside the
payload, byte count == prod(shape) * element size; a name present in two shards is an
error (:477-514).  Reading is native code (``csrc/host_safetensors.cpp``); writing (the
random-weights mode) is Python.
"""
from __future__ import annotations

import ctypes
import glob
import json
import os
import struct
import warnings
from dataclasses import dataclass
from typing import Dict, List, Tuple

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


def _lib():
    from ..kernels import lib
    L = lib()
    if not getattr(L, "_st_api_ready", False):
        L.infero_st_open.restype = ctypes.c_void_p
        L.infero_st_open.argtypes = [ctypes.c_char_p]
        for fn in ("infero_st_error", "infero_st_name"):
            getattr(L, fn).restype = ctypes.c_char_p
        for fn in ("infero_st_nbytes", "infero_st_offset"):
            getattr(L, fn).restype = ctypes.c_longlong
        L.infero_st_data.restype = ctypes.c_void_p
        for fn in ("infero_st_error", "infero_st_count", "infero_st_close"):
            getattr(L, fn).argtypes = [ctypes.c_void_p]
        for fn in ("infero_st_name", "infero_st_dtype", "infero_st_rank", "infero_st_nbytes", "infero_st_offset",
                   "infero_st_data"):
            getattr(L, fn).argtypes = [ctypes.c_void_p, ctypes.c_int]
        L.infero_st_shape.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_longlong)]
        L._st_api_ready = True
    return L


_DTYPE_ORDER = ("F32", "F16", "BF16", "I32", "I64", "U8")       # the reader's dtype numbers


class SafetensorsFile:
    """One file, mapped and checked by the native reader (``csrc/host_safetensors.cpp``, in the
    engine's shared library, no CUDA in it); tensors come back as views of the mapping."""

    def __init__(self, path: str):
        self.path = path
        self._L = _lib()
        self._h = ctypes.c_void_p(self._L.infero_st_open(os.fsencode(path)))
        if not self._h:
            raise MemoryError("safetensors reader")
        err = self._L.infero_st_error(self._h).decode("utf-8", "replace")
        if err:
            self._L.infero_st_close(self._h)
            self._h = None
            raise SafetensorsError(err)
        self.metadata: Dict[str, str] = {}
        self.entries: Dict[str, TensorEntry] = {}
        self._index: Dict[str, int] = {}
        for i in range(self._L.infero_st_count(self._h)):
            name = self._L.infero_st_name(self._h, i).decode("utf-8")
            rank = self._L.infero_st_rank(self._h, i)
            dims = (ctypes.c_longlong * max(1, rank))()
            self._L.infero_st_shape(self._h, i, dims)
            tdtype, _ = _DTYPES[_DTYPE_ORDER[self._L.infero_st_dtype(self._h, i)]]
            self.entries[name] = TensorEntry(name, tdtype, tuple(int(dims[k]) for k in range(rank)),
                                             int(self._L.infero_st_offset(self._h, i)),
                                             int(self._L.infero_st_nbytes(self._h, i)), self)
            self._index[name] = i

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor over the mapped bytes (read-only view; copy before writing).  The mapping
        stays for the life of the process once a tensor has been handed out."""
        ent = self.entries[name]
        n = 1
        for s in ent.shape:
            n *= s
        if n == 0:
            return torch.empty(ent.shape, dtype=ent.dtype)
        ptr = self._L.infero_st_data(self._h, self._index[name])
        buf = (ctypes.c_char * ent.nbytes).from_address(ptr)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)     # the mapping is read-only by design
            t = torch.frombuffer(buf, dtype=ent.dtype, count=n)
        return t.view(ent.shape)

    def close(self):
        h, self._h = self._h, None
        if h:
            self._L.infero_st_close(h)

    def __del__(self):
        try:
            self.close()
        except Exception:          # noqa: BLE001  (interpreter shutdown)
            pass


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
                f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.dtype != torch.uint8 else t.numpy().tobytes())
    os.replace(tmp, path)
