"""Reader and writer of the safetensors container.

Layout: ``u64 little-endian header length``, a JSON header mapping each tensor
name to ``{dtype, shape, data_offsets}``, then the data.  The reader applies the
bounds rules of the reference's parser (src/model/safetensors.rs:40-45,
:248-402): header no longer than 100 MiB and than the file, rank at most 8,
sizes multiplied without overflow, offsets inside the data section, byte size
equal to elements times element size, no two tensors overlapping.  Every
violation is a ``WeightsError``; nothing is read outside the file.  Shards
listed by ``model.safetensors.index.json`` are opened together (:521-549); a
name in two shards and a shard path that leaves the folder are errors
(:552-565, :649-654).
"""
from __future__ import annotations

import json
import mmap
import os
import struct

import torch

from ..errors import WeightsError

MAX_HEADER_BYTES = 100 * 1024 * 1024
MAX_RANK = 8

DTYPES = {
    "F32": (torch.float32, 4),
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
}
_NAMES = {v[0]: k for k, v in DTYPES.items()}


class TensorEntry:
    __slots__ = ("name", "dtype_name", "shape", "begin", "end", "file")

    def __init__(self, name, dtype_name, shape, begin, end, file):
        self.name, self.dtype_name, self.shape = name, dtype_name, tuple(shape)
        self.begin, self.end, self.file = begin, end, file

    @property
    def nbytes(self):
        return self.end - self.begin


class SafeTensorsFile:
    """One mapped ``.safetensors`` file.  ``entries`` maps names to ``TensorEntry``."""

    def __init__(self, path):
        self.path = path
        try:
            size = os.path.getsize(path)
            self._fh = open(path, "rb")
        except OSError as e:
            raise WeightsError(f"{path}: cannot open: {e}") from None
        if size < 8:
            raise WeightsError(f"{path}: malformed safetensors: file shorter than its 8-byte length field")
        (header_len,) = struct.unpack("<Q", self._fh.read(8))
        if header_len > MAX_HEADER_BYTES:
            raise WeightsError(f"{path}: malformed safetensors: header of {header_len} bytes exceeds "
                               f"{MAX_HEADER_BYTES}")
        if header_len > size - 8:
            raise WeightsError(f"{path}: malformed safetensors: header of {header_len} bytes exceeds the file")
        raw = self._fh.read(header_len)
        try:
            header = json.loads(raw.decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightsError(f"{path}: malformed safetensors: header is not JSON: {e}") from None
        if not isinstance(header, dict):
            raise WeightsError(f"{path}: malformed safetensors: header is not a JSON object")
        self.data_start = 8 + header_len
        data_len = size - self.data_start
        self.metadata = header.pop("__metadata__", None) or {}
        self.entries = {}
        spans = []
        for name, info in header.items():
            if not isinstance(info, dict):
                raise WeightsError(f"{path}: malformed safetensors: entry '{name}' is not an object")
            dtype_name, shape, offs = info.get("dtype"), info.get("shape"), info.get("data_offsets")
            if dtype_name not in DTYPES:
                raise WeightsError(f"{path}: tensor '{name}' has unsupported dtype {dtype_name!r} "
                                   f"(supported: {', '.join(DTYPES)})")
            if (not isinstance(shape, list) or len(shape) > MAX_RANK
                    or any(isinstance(d, bool) or not isinstance(d, int) or d < 0 for d in shape)):
                raise WeightsError(f"{path}: malformed safetensors: tensor '{name}' has a bad shape {shape!r}")
            if (not isinstance(offs, list) or len(offs) != 2
                    or any(isinstance(o, bool) or not isinstance(o, int) or o < 0 for o in offs)):
                raise WeightsError(f"{path}: malformed safetensors: tensor '{name}' has bad data_offsets {offs!r}")
            begin, end = offs
            numel = 1
            for d in shape:
                numel *= d
                if numel >= 1 << 63:
                    raise WeightsError(f"{path}: malformed safetensors: tensor '{name}' shape overflows")
            if begin > end or end > data_len:
                raise WeightsError(f"{path}: malformed safetensors: tensor '{name}' offsets {offs} lie "
                                   f"outside the data section of {data_len} bytes")
            if end - begin != numel * DTYPES[dtype_name][1]:
                raise WeightsError(f"{path}: malformed safetensors: tensor '{name}' holds {end - begin} "
                                   f"bytes, its shape {shape} and dtype {dtype_name} need "
                                   f"{numel * DTYPES[dtype_name][1]}")
            self.entries[name] = TensorEntry(name, dtype_name, shape, begin, end, self)
            if end > begin:
                spans.append((begin, end, name))
        spans.sort()
        for (b0, e0, n0), (b1, e1, n1) in zip(spans, spans[1:]):
            if b1 < e0:
                raise WeightsError(f"{path}: malformed safetensors: tensors '{n0}' and '{n1}' overlap")
        self._map = None

    def _mapped(self):
        if self._map is None:
            # copy-on-write mapping: torch wants a writable buffer, the file is never written
            self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_COPY)
        return self._map

    def tensor(self, name):
        """The tensor as a torch view of the mapped file (host memory, stored dtype)."""
        e = self.entries[name]
        dtype, _ = DTYPES[e.dtype_name]
        numel = 1
        for d in e.shape:
            numel *= d
        if numel == 0:
            return torch.empty(e.shape, dtype=dtype)
        flat = torch.frombuffer(self._mapped(), dtype=dtype, count=numel, offset=self.data_start + e.begin)
        return flat.reshape(e.shape)

    def close(self):
        self._map = None  # views keep the mapping alive while they exist
        self._fh.close()


class SafeTensorsModel:
    """All weight files of a model folder behind one name -> tensor view."""

    def __init__(self, model_dir):
        self.model_dir = model_dir
        self.files = []
        self.entries = {}
        for path in self._shard_paths(model_dir):
            f = SafeTensorsFile(path)
            self.files.append(f)
            for name, entry in f.entries.items():
                if name in self.entries:
                    raise WeightsError(f"tensor '{name}' appears in both {self.entries[name].file.path} "
                                       f"and {path}")
                self.entries[name] = entry

    @staticmethod
    def _shard_paths(model_dir):
        if os.path.isfile(model_dir) and model_dir.endswith(".safetensors"):
            return [model_dir]
        single = os.path.join(model_dir, "model.safetensors")
        if os.path.isfile(single):
            return [single]
        index = os.path.join(model_dir, "model.safetensors.index.json")
        if os.path.isfile(index):
            try:
                with open(index, "r", encoding="utf-8") as f:
                    weight_map = json.load(f)["weight_map"]
                shards = sorted(set(weight_map.values()))
            except (OSError, ValueError, KeyError, TypeError, AttributeError) as e:
                raise WeightsError(f"{index}: invalid shard index: {e}") from None
            paths = []
            for s in shards:
                if not isinstance(s, str) or os.path.isabs(s) or ".." in s.replace("\\", "/").split("/"):
                    raise WeightsError(f"{index}: shard path {s!r} leaves the model folder")
                paths.append(os.path.join(model_dir, s))
            if paths:
                return paths
        found = sorted(p for p in (os.listdir(model_dir) if os.path.isdir(model_dir) else [])
                       if p.endswith(".safetensors"))
        if not found:
            raise WeightsError(f"{model_dir}: no .safetensors weights found")
        return [os.path.join(model_dir, p) for p in found]

    def names(self):
        return list(self.entries)

    def shape(self, name):
        return self.entries[name].shape

    def dtype_name(self, name):
        return self.entries[name].dtype_name

    def tensor(self, name):
        return self.entries[name].file.tensor(name)

    def close(self):
        for f in self.files:
            f.close()


def write_safetensors(path, tensors, metadata=None):
    """Write ``{name: torch tensor}`` as one safetensors file, names in sorted order, data
    8-byte aligned by padding the header with spaces."""
    header = {}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise WeightsError(f"cannot write tensor '{name}' of dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * (-(8 + len(raw)) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes())
