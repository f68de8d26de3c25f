"""Reading and writing the safetensors container.

Format, as the reference reads it (src/safetensors.cpp:52-105): an 8-byte
little-endian header length, a JSON header mapping each tensor name to
``dtype``, ``shape`` and ``data_offsets`` relative to the end of the header,
then the raw little-endian data.  The same checks are made (header inside the
file, ``numel * itemsize == nbytes``, data inside the file); unlike the
reference's ``tensor()``, which aborts the process on a missing name
(src/safetensors.cpp:115-122), every failure here is a ``WeightsError``.

Shards: a folder holds ``model.safetensors`` or a
``model.safetensors.index.json`` whose ``weight_map`` names the shard of each
tensor (src/model.cpp:31-57).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from typing import Dict, Iterable, List, Tuple

import torch


class WeightsError(RuntimeError):
    """A checkpoint that cannot be read or does not fit the model."""


_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """One memory-mapped safetensors file."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._fh = open(path, "rb")
        except OSError as e:
            raise WeightsError(f"cannot open {path}: {e.strerror}")
        size = os.fstat(self._fh.fileno()).st_size
        if size < 8:
            raise WeightsError(f"truncated file {path}")
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        (n,) = struct.unpack("<Q", self._map[:8])
        if n + 8 > size:
            raise WeightsError(f"invalid safetensors header length in {path}")
        try:
            header = json.loads(self._map[8:8 + n].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightsError(f"bad safetensors header in {path}: {e}")
        if not isinstance(header, dict):
            raise WeightsError(f"bad safetensors header in {path}: not an object")
        self._data_start = 8 + n
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, t in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype_name = t["dtype"]
                shape = tuple(int(s) for s in t["shape"])
                begin, end = (int(x) for x in t["data_offsets"])
            except (KeyError, TypeError, ValueError):
                raise WeightsError(f"bad safetensors header entry for {name} in {path}")
            if dtype_name not in _DTYPES:
                raise WeightsError(f"unsupported dtype {dtype_name} for {name} in {path}")
            dtype = _DTYPES[dtype_name]
            numel = 1
            for s in shape:
                numel *= s
            nbytes = end - begin
            if begin < 0 or numel * dtype.itemsize != nbytes or self._data_start + end > size:
                raise WeightsError(f"inconsistent size for {name} in {path}")
            self.entries[name] = (dtype, shape, begin, nbytes)

    def names(self) -> List[str]:
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the mapped file (read-only memory: copy or
        move it to a device before writing to it)."""
        if name not in self.entries:
            raise WeightsError(f"missing tensor {name} in {self.path}")
        dtype, shape, begin, nbytes = self.entries[name]
        if nbytes == 0:
            return torch.empty(shape, dtype=dtype)
        numel = nbytes // dtype.itemsize
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)   # the mapping is read-only by design
            t = torch.frombuffer(self._map, dtype=dtype, count=numel, offset=self._data_start + begin)
        return t.reshape(shape)

    def close(self) -> None:
        # tensors handed out keep the mapping alive through the buffer protocol;
        # closing an exported mmap raises, so drop the references instead.
        self._map = None
        self._fh.close()


class TensorStore:
    """All shards of a model folder, addressed by tensor name."""

    def __init__(self, model_dir: str):
        if os.path.isfile(model_dir):
            model_dir = os.path.dirname(model_dir) or "."
        self.model_dir = model_dir
        single = os.path.join(model_dir, "model.safetensors")
        index = os.path.join(model_dir, "model.safetensors.index.json")
        shards: List[str] = []
        if os.path.exists(single):
            shards = [single]
        elif os.path.exists(index):
            try:
                with open(index, "r", encoding="utf-8") as f:
                    weight_map = json.load(f)["weight_map"]
                shards = sorted({os.path.join(model_dir, str(v)) for v in weight_map.values()})
            except (OSError, KeyError, TypeError, AttributeError, json.JSONDecodeError) as e:
                raise WeightsError(f"bad index {index}: {e}")
        else:
            raise WeightsError(f"no model.safetensors or model.safetensors.index.json in {model_dir}")
        self.files = [SafetensorsFile(s) for s in shards]
        self.where: Dict[str, SafetensorsFile] = {}
        for f in self.files:
            for n in f.names():
                self.where.setdefault(n, f)

    def names(self) -> List[str]:
        return list(self.where)

    def shape(self, name: str) -> Tuple[int, ...]:
        return self.where[name].entries[name][1]

    def dtype(self, name: str) -> torch.dtype:
        return self.where[name].entries[name][0]

    def tensor(self, name: str) -> torch.Tensor:
        if name not in self.where:
            raise WeightsError(f"missing tensor {name}")
        return self.where[name].tensor(name)

    def close(self) -> None:
        for f in self.files:
            f.close()


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]],
                      metadata: Dict[str, str] | None = None) -> None:
    """Writes tensors (CPU, any supported dtype) in the order given."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blobs: List[torch.Tensor] = []
    offset = 0
    for name, t in tensors:
        if t.dtype not in _NAMES:
            raise WeightsError(f"cannot write dtype {t.dtype} for {name}")
        if name in header:
            raise WeightsError(f"tensor {name} given twice")
        t = t.detach().to("cpu").contiguous()
        nbytes = t.numel() * t.dtype.itemsize
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
        blobs.append(t)
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * ((8 - len(raw) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for t in blobs:
            if t.numel():
                f.write(memoryview(t.reshape(-1).view(torch.uint8).numpy()))
    os.replace(tmp, path)
