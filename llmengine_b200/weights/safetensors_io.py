"""Reading and writing the safetensors container, without any library.

Layout: an 8-byte little-endian header length, a JSON header that maps each
tensor name to `{"dtype", "shape", "data_offsets": [begin, end]}` (offsets are
relative to the first byte after the header), then the raw little-endian data.
The reference reads GGUF files instead (src/io/gguf_parser.cpp); what is kept
from it is the behaviour: tensors are found by name, and a file whose offsets
do not fit is refused before anything is copied
(src/io/gguf_weight_loader.cpp:106-113).
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, Iterable, List, Mapping, Tuple

import numpy as np
import torch


class SafetensorsError(IOError):
    pass


_DTYPES = {
    "F32": (torch.float32, np.dtype("<f4")),
    "F16": (torch.float16, np.dtype("<f2")),
    "BF16": (torch.bfloat16, np.dtype("<u2")),   # numpy has no bfloat16: carried as raw 16-bit words
    "I32": (torch.int32, np.dtype("<i4")),
    "I64": (torch.int64, np.dtype("<i8")),
    "U8": (torch.uint8, np.dtype("u1")),
    "BOOL": (torch.bool, np.dtype("u1")),
}
_NAMES = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16", torch.int32: "I32",
          torch.int64: "I64", torch.uint8: "U8"}


class SafetensorsFile:
    """One opened file: the parsed header and a memory map of the data."""

    def __init__(self, path: str):
        self.path = path
        try:
            size = os.path.getsize(path)
        except OSError as e:
            raise SafetensorsError(f"{path}: {e.strerror or e}") from None
        if size < 8:
            raise SafetensorsError(f"{path}: too short to hold a safetensors header")
        with open(path, "rb") as f:
            (hlen,) = struct.unpack("<Q", f.read(8))
            if hlen <= 0 or 8 + hlen > size:
                raise SafetensorsError(f"{path}: header length {hlen} does not fit a file of {size} bytes")
            try:
                header = json.loads(f.read(hlen).decode("utf-8"))
            except (UnicodeDecodeError, json.JSONDecodeError) as e:
                raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from None
        self.metadata = header.pop("__metadata__", {}) or {}
        self.data_start = 8 + hlen
        self.data_size = size - self.data_start
        self.entries: Dict[str, dict] = {}
        for name, e in header.items():
            try:
                dtype, shape, (b, en) = e["dtype"], [int(s) for s in e["shape"]], e["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed header entry for tensor {name!r}") from None
            if dtype not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dtype}")
            numel = int(np.prod(shape, dtype=np.int64)) if shape else 1
            nbytes = numel * _DTYPES[dtype][1].itemsize
            if b < 0 or en < b or en > self.data_size or en - b != nbytes:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} ({dtype}{shape}) has data offsets [{b}, {en}) that do not match "
                    f"its {nbytes} bytes or lie outside the file's {self.data_size} data bytes")
            self.entries[name] = {"dtype": dtype, "shape": shape, "begin": b, "end": en}
        self._map = None

    def names(self) -> List[str]:
        return list(self.entries)

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self.entries[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name]["dtype"]][0]

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the mapped file (copy it before the file goes away)."""
        e = self.entries[name]
        if self._map is None:
            self._map = np.memmap(self.path, dtype=np.uint8, mode="r", offset=self.data_start,
                                  shape=(self.data_size,)) if self.data_size else np.zeros(0, np.uint8)
        tdt, ndt = _DTYPES[e["dtype"]]
        raw = np.asarray(self._map[e["begin"]:e["end"]])
        arr = raw.view(ndt).reshape(e["shape"])
        with _quiet_nonwritable():
            t = torch.from_numpy(arr)
        if tdt == torch.bfloat16:
            t = t.view(torch.bfloat16)
        elif tdt == torch.bool:
            t = t.to(torch.bool)
        return t


class _quiet_nonwritable:
    """torch warns when wrapping a read-only array; the tensors are only read."""

    def __enter__(self):
        import warnings
        self._cm = warnings.catch_warnings()
        self._cm.__enter__()
        warnings.simplefilter("ignore")

    def __exit__(self, *a):
        return self._cm.__exit__(*a)


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] = None) -> None:
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store tensor {name!r} of dtype {t.dtype}")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + n]}
        offset += n
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.dtype == torch.bfloat16:
                t = t.view(torch.int16)
            f.write(t.numpy().tobytes())
    os.replace(tmp, path)


def open_model_files(model_dir: str) -> List[SafetensorsFile]:
    """The weight files of a model folder: `model.safetensors`, or the shards
    that `model.safetensors.index.json` names."""
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.exists(single):
        return [SafetensorsFile(single)]
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index, "r", encoding="utf-8") as f:
            files = sorted(set(json.load(f)["weight_map"].values()))
        return [SafetensorsFile(os.path.join(model_dir, fn)) for fn in files]
    raise SafetensorsError(f"{model_dir}: neither model.safetensors nor model.safetensors.index.json found")
