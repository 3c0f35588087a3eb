"""Weights by tensor name, checked as a whole, kept in the precision they are stored in.

The reference reads each tensor by its (mapped) name and fails at the first that is missing or
misshapen (model_f32.go:137-206, gguf.go:744-751, :819-825). Here every expected tensor is checked
before anything is copied, and one error lists all that is missing, unexpected or of the wrong
shape.

Precision: bfloat16 stays bfloat16, float32 stays float32, integer tables become int32;
float16 is widened (to float32: exact). `compute_dtype=float32` widens bfloat16 too, which is
exact, so the 32-bit engine sees the very same numbers.
"""
from __future__ import annotations

from pathlib import Path
from typing import Iterable

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile
from .spec import TensorSpec

WEIGHTS_FILE = "model.safetensors"
INDEX_FILE = "model.safetensors.index.json"     # {"weight_map": {tensor name: file name}}: the tensors are spread over several files


class WeightError(ValueError):
    """The weight file does not hold what the model needs; `.missing`, `.unexpected`, `.misshapen`."""

    def __init__(self, path, missing, unexpected, misshapen, bad_dtype):
        self.missing, self.unexpected, self.misshapen, self.bad_dtype = missing, unexpected, misshapen, bad_dtype
        lines = [f"{path}: the weights do not fit the model"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if misshapen:
            lines.append(f"  wrong shapes ({len(misshapen)}): " + "; ".join(
                f"{n} is {list(found)}, expected {list(want)}" for n, found, want in misshapen))
        if bad_dtype:
            lines.append(f"  unsupported dtypes ({len(bad_dtype)}): " + "; ".join(f"{n} is {d}" for n, d in bad_dtype))
        super().__init__("\n".join(lines))


_FLOATS = (torch.float32, torch.bfloat16, torch.float16)
_INTS = (torch.int32, torch.int64, torch.int16, torch.int8, torch.uint8)


def stored_to_kept(t: torch.Tensor, compute_dtype: torch.dtype) -> torch.Tensor:
    if t.dtype in _INTS:
        return t.to(torch.int32)
    if t.dtype == torch.float16:
        return t.to(torch.float32)
    if compute_dtype == torch.float32:
        return t.to(torch.float32)
    return t


def load_weights(model_dir, specs: Iterable[TensorSpec], device, compute_dtype: torch.dtype,
                 ignore: Iterable[str] = ()) -> dict[str, torch.Tensor]:
    """Read the tensors named by `specs` from `model_dir`/model.safetensors (or, where that file is
    absent, from the files that model.safetensors.index.json names) onto `device`.

    `ignore`: names that may be present without being used (an output head beside a tied
    embedding). Raises WeightError listing every fault at once."""
    path = Path(model_dir) / WEIGHTS_FILE
    specs = list(specs)
    files = [path]
    if not path.is_file():
        index = Path(model_dir) / INDEX_FILE
        if not index.is_file():
            raise WeightError(path, [s.name for s in specs if not s.optional], [], [], [])
        path, files = index, _shards(index)
    ignore = set(ignore)
    opened = [SafetensorsFile(p) for p in files]
    try:
        entries, owner = {}, {}
        for f in opened:
            for n, e in f.entries.items():
                if n in entries:
                    raise SafetensorsError(f"{path}: tensor {n!r} is stored in two files")
                entries[n], owner[n] = e, f
        wanted = {s.name: s for s in specs}
        missing = [s.name for s in specs if s.name not in entries and not s.optional]
        unexpected = [n for n in entries if n not in wanted and n not in ignore]
        misshapen, bad_dtype = [], []
        for s in specs:
            if s.name in entries:
                tdt, shape, _, _ = entries[s.name]
                if tuple(shape) != tuple(s.shape):
                    misshapen.append((s.name, tuple(shape), tuple(s.shape)))
                if tdt not in _FLOATS + _INTS or (s.init != "integer_table" and tdt not in _FLOATS):
                    bad_dtype.append((s.name, str(tdt).replace("torch.", "")))
        if missing or unexpected or misshapen or bad_dtype:
            raise WeightError(path, missing, unexpected, misshapen, bad_dtype)
        out = {}
        for s in specs:
            if s.name not in entries:
                continue
            t = owner[s.name].tensor(s.name)
            # copy to the device first where that is lossless and smaller, then widen there
            out[s.name] = stored_to_kept(t.to(device, copy=True), compute_dtype).contiguous()
    finally:
        for f in opened:
            f.close()
    return out


def _shards(index: Path) -> list[Path]:
    """The files an index names, in the order of their first mention."""
    import json
    try:
        weight_map = json.loads(index.read_text())["weight_map"]
        names = list(dict.fromkeys(str(v) for v in weight_map.values()))
    except (ValueError, KeyError, AttributeError, TypeError) as e:
        raise SafetensorsError(f"{index}: not an index of weight files ({e})") from None
    files = [index.parent / n for n in names]
    for f in files:
        if not f.is_file() or f.parent.resolve() != index.parent.resolve():
            raise SafetensorsError(f"{index}: names the file {f.name!r}, which is not in the model folder")
    return files


__all__ = ["WeightError", "SafetensorsError", "load_weights", "stored_to_kept", "WEIGHTS_FILE"]
