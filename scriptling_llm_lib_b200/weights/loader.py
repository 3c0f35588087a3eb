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
    """Read the tensors named by `specs` from `model_dir`/model.safetensors onto `device`.

    `ignore`: names that may be present without being used (an output head beside a tied
    embedding). Raises WeightError listing every fault at once."""
    path = Path(model_dir) / WEIGHTS_FILE
    if not path.is_file():
        raise WeightError(path, [s.name for s in specs if not s.optional], [], [], [])
    specs = list(specs)
    ignore = set(ignore)
    with SafetensorsFile(path) as f:
        wanted = {s.name: s for s in specs}
        missing = [s.name for s in specs if s.name not in f.entries and not s.optional]
        unexpected = [n for n in f.entries if n not in wanted and n not in ignore]
        misshapen, bad_dtype = [], []
        for s in specs:
            if s.name in f.entries:
                tdt, shape, _, _ = f.entries[s.name]
                if tuple(shape) != tuple(s.shape):
                    misshapen.append((s.name, tuple(shape), tuple(s.shape)))
                if tdt not in _FLOATS + _INTS or (s.init != "integer_table" and tdt not in _FLOATS):
                    bad_dtype.append((s.name, str(tdt).replace("torch.", "")))
        if missing or unexpected or misshapen or bad_dtype:
            raise WeightError(path, missing, unexpected, misshapen, bad_dtype)
        out = {}
        for s in specs:
            if s.name not in f.entries:
                continue
            t = f.tensor(s.name)
            # copy to the device first where that is lossless and smaller, then widen there
            out[s.name] = stored_to_kept(t.to(device, copy=True), compute_dtype).contiguous()
    return out


__all__ = ["WeightError", "SafetensorsError", "load_weights", "stored_to_kept", "WEIGHTS_FILE"]
