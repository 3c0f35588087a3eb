"""Reader and writer for the safetensors container, by tensor name.

Format: 8 bytes little-endian header length N, N bytes of JSON mapping each name to
{"dtype", "shape", "data_offsets": [begin, end)} relative to the end of the header, then raw
little-endian data. The reference's container is GGUF (gguf.go:524-684); like its loader, this one
maps the file read-only and checks every range before touching it (gguf.go:492-518).
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path

import torch

_DTYPES = {
    "F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2),
    "I32": (torch.int32, 4), "I64": (torch.int64, 8), "F64": (torch.float64, 8),
    "U8": (torch.uint8, 1), "I8": (torch.int8, 1), "I16": (torch.int16, 2), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """A mapped file: `entries` gives dtype, shape and byte range per name; `tensor(name)` a CPU
    tensor that views the mapping (copy it before the file object goes away)."""

    def __init__(self, path):
        self.path = str(path)
        size = Path(path).stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: too short to hold a safetensors header ({size} bytes)")
        self._fh = open(path, "rb")
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self._map[:8])
        if hlen > size - 8:
            raise SafetensorsError(f"{self.path}: header length {hlen} exceeds the file ({size} bytes)")
        try:
            header = json.loads(self._map[8:8 + hlen].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{self.path}: header is not valid JSON ({e})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{self.path}: header must be a JSON object")
        self.data_start = 8 + hlen
        data_len = size - self.data_start
        self.metadata = header.pop("__metadata__", None)
        self.entries: dict[str, tuple[torch.dtype, tuple[int, ...], int, int]] = {}
        ranges = []
        for name, meta in header.items():
            try:
                dt, shape, (b, e) = meta["dtype"], tuple(int(s) for s in meta["shape"]), meta["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{self.path}: entry {name!r} is malformed") from None
            if dt not in _DTYPES:
                raise SafetensorsError(f"{self.path}: tensor {name!r} has unsupported dtype {dt!r}")
            tdt, width = _DTYPES[dt]
            count = 1
            for s in shape:
                count *= s
            if not (0 <= b <= e <= data_len) or e - b != count * width:
                raise SafetensorsError(f"{self.path}: tensor {name!r} ({dt}, shape {list(shape)}) claims bytes "
                                       f"[{b}, {e}) of a data section of {data_len} bytes")
            self.entries[name] = (tdt, shape, b, e)
            ranges.append((b, e, name))
        ranges.sort()
        for (b0, e0, n0), (b1, e1, n1) in zip(ranges, ranges[1:]):
            if b1 < e0:
                raise SafetensorsError(f"{self.path}: tensors {n0!r} and {n1!r} overlap")

    def names(self):
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        tdt, shape, b, e = self.entries[name]
        if e == b:
            return torch.empty(shape, dtype=tdt)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")     # the mapping is read-only; the view is never written
            flat = torch.frombuffer(self._map, dtype=tdt, count=(e - b) // _DTYPES[_NAMES[tdt]][1],
                                    offset=self.data_start + b)
        return flat.view(shape)

    def close(self):
        try:
            self._map.close()
        except BufferError:
            pass                                 # a view is still alive; the mapping goes with it
        self._fh.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_safetensors(path, tensors: dict[str, torch.Tensor], metadata: dict | None = None) -> None:
    """Write CPU tensors under their names, in the given order, data 8-byte aligned."""
    header, offset, blobs = {}, 0, []
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name, t in tensors.items():
        t = t.detach().contiguous().cpu()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store tensor {name!r} of dtype {t.dtype}")
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hjson += b" " * (-len(hjson) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for raw in blobs:
            f.write(raw)
