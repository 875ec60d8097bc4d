"""Reading and writing safetensors files by tensor name.

The format: 8 bytes little-endian header length, a JSON header ``{name: {dtype, shape, data_offsets}}``, then the
tensors' bytes. The reference reads it the same way where it reads such files (``kindi/dspine.py:79-119``: header
parse, all ``*.safetensors`` of a folder merged, BF16/F16/F32 accepted). This reader maps the file and hands out
torch tensors that view the mapping (no copy until the caller moves them to the device).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, List, Mapping, Tuple

import torch

_DTYPES = {
    "F32": (torch.float32, 4), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2), "F64": (torch.float64, 8),
    "I64": (torch.int64, 8), "I32": (torch.int32, 4), "I16": (torch.int16, 2), "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One mapped file: ``entries`` gives (dtype name, shape) by tensor name; ``tensor(name)`` views its bytes."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError("%s: too short to be a safetensors file (%d bytes)" % (path, size))
        self._f = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError("%s: header length %d does not fit the file (%d bytes)" % (path, hlen, size))
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError("%s: header is not valid JSON: %s" % (path, e))
        self.metadata = header.pop("__metadata__", None) or {}
        self._data0 = 8 + hlen
        self.entries: Dict[str, Tuple[str, Tuple[int, ...]]] = {}
        self._spans: Dict[str, Tuple[int, int]] = {}
        for name, e in header.items():
            dt, shape, (b, en) = e["dtype"], tuple(int(s) for s in e["shape"]), e["data_offsets"]
            if dt not in _DTYPES:
                raise SafetensorsError("%s: tensor %r has unsupported dtype %s" % (path, name, dt))
            n = 1
            for s in shape:
                n *= s
            if en - b != n * _DTYPES[dt][1]:
                raise SafetensorsError("%s: tensor %r: %d bytes stored for shape %s of %s"
                                       % (path, name, en - b, list(shape), dt))
            if self._data0 + en > size:
                raise SafetensorsError("%s: tensor %r ends at byte %d past the end of the file (%d): truncated"
                                       % (path, name, self._data0 + en, size))
            self.entries[name] = (dt, shape)
            self._spans[name] = (self._data0 + b, self._data0 + en)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def tensor(self, name: str) -> torch.Tensor:
        dt, shape = self.entries[name]
        b, e = self._spans[name]
        tdt = _DTYPES[dt][0]
        if e == b:
            return torch.empty(shape, dtype=tdt)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")        # the mapping is read-only; the tensors are never written
            raw = torch.frombuffer(self._mm, dtype=torch.uint8, count=e - b, offset=b)
        return raw.view(tdt).reshape(shape)

    def close(self):
        # tensors handed out keep the mapping alive through the buffer protocol; closing is best effort
        try:
            if self._mm is not None:
                self._mm.close()
        except BufferError:
            pass
        self._f.close()


def folder_files(model_dir: str) -> List[str]:
    """the safetensors files of a model folder: those the index names if there is one, else every *.safetensors"""
    idx = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(idx):
        with open(idx) as f:
            names = sorted(set(json.load(f)["weight_map"].values()))
        return [os.path.join(model_dir, n) for n in names]
    names = sorted(n for n in os.listdir(model_dir) if n.endswith(".safetensors"))
    return [os.path.join(model_dir, n) for n in names]


def write_file(path: str, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] = None) -> None:
    """write tensors (CPU, contiguous) in name order"""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError("tensor %r: dtype %s cannot be stored" % (name, t.dtype))
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + n]}
        off += n
    hj = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    os.replace(tmp, path)
