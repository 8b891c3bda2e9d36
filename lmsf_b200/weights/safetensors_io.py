"""A reader and a writer for the safetensors format, with no dependency but torch.

File layout: 8 bytes little-endian header length n, n bytes of JSON
{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}, then the raw
little-endian tensor data.  The reference mmaps such files through candle
(core/src/model_executor/models/model_factory.rs:133-139) and finds the shards of a model in
`model.safetensors.index.json` (model_factory.rs:58-77); a lone `model.safetensors` is accepted here too.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Callable, Dict, List, Tuple

import torch

DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
          "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
          "BOOL": torch.bool}
NAMES = {v: k for k, v in DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class TensorEntry:
    """One tensor of a file: its dtype and shape are known without reading the data."""
    __slots__ = ("name", "dtype", "shape", "_file", "_begin", "_end")

    def __init__(self, name, dtype, shape, file, begin, end):
        self.name, self.dtype, self.shape = name, dtype, tuple(shape)
        self._file, self._begin, self._end = file, begin, end

    def load(self) -> torch.Tensor:
        """A CPU tensor that shares memory with the mapped file (read it, do not write it)."""
        return self._file.tensor(self)


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        self._fh = open(path, "rb")
        size = os.fstat(self._fh.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        (n,) = struct.unpack("<Q", self._fh.read(8))
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._fh.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: the header is not valid JSON ({e})") from None
        self._data_start = 8 + n
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None
        self.entries: Dict[str, TensorEntry] = {}
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            dt = DTYPES.get(meta.get("dtype"))
            if dt is None:
                raise SafetensorsError(f"{path}: tensor {name!r} has the unsupported dtype {meta.get('dtype')!r}")
            b, e = meta["data_offsets"]
            numel = 1
            for s in meta["shape"]:
                numel *= int(s)
            if e - b != numel * torch.empty(0, dtype=dt).element_size() or self._data_start + e > size:
                raise SafetensorsError(f"{path}: tensor {name!r}: data range [{b}, {e}) does not match shape "
                                       f"{meta['shape']} of {meta['dtype']}")
            self.entries[name] = TensorEntry(name, dt, meta["shape"], self, b, e)

    def tensor(self, e: TensorEntry) -> torch.Tensor:
        if e._end == e._begin:
            return torch.empty(e.shape, dtype=e.dtype)
        buf = memoryview(self._map)[self._data_start + e._begin:self._data_start + e._end]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")   # the buffer is read-only; the tensor is only ever read
            t = torch.frombuffer(buf, dtype=e.dtype)
        return t.reshape(e.shape)


def open_model_tensors(model_dir: str) -> Dict[str, TensorEntry]:
    """All tensors of a model folder by name, from the shards of the index or from model.safetensors."""
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(index):
        with open(index) as f:
            shards = sorted(set(json.load(f)["weight_map"].values()))
    elif os.path.isfile(os.path.join(model_dir, "model.safetensors")):
        shards = ["model.safetensors"]
    else:
        raise SafetensorsError(f"{model_dir!r} holds neither model.safetensors.index.json nor model.safetensors")
    out: Dict[str, TensorEntry] = {}
    for s in shards:
        f = SafetensorsFile(os.path.join(model_dir, s))
        for name, e in f.entries.items():
            if name in out:
                raise SafetensorsError(f"tensor {name!r} appears in more than one shard")
            out[name] = e
    return out


def write_safetensors(path: str, specs: List[Tuple[str, torch.dtype, Tuple[int, ...]]],
                      make: Callable[[str], torch.Tensor], metadata: Dict[str, str] = None) -> None:
    """Writes tensors one at a time: `specs` lists (name, dtype, shape); `make(name)` returns the tensor when
    its turn comes, so a model larger than host memory could be written."""
    header, off = {}, 0
    for name, dt, shape in specs:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty(0, dtype=dt).element_size()
        header[name] = {"dtype": NAMES[dt], "shape": [int(s) for s in shape], "data_offsets": [off, off + nbytes]}
        off += nbytes
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name, dt, shape in specs:
            t = make(name)
            if t.dtype != dt or tuple(t.shape) != tuple(shape):
                raise SafetensorsError(f"{name}: made {tuple(t.shape)} of {t.dtype}, declared {tuple(shape)} of {dt}")
            t = t.contiguous().cpu()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
