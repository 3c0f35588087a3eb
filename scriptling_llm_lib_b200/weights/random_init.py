"""Random-weights mode: a model folder (config.json, model.safetensors) from a configuration and a
seed. The reference has no such mode (its only source of weights is a GGUF file); matrices are
drawn N(0, 0.02) and norm weights 1 + N(0, 0.02), each tensor from its own stream (seed, index in
the model's tensor list), so a tensor's values do not depend on the others' sizes."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Iterable

import torch

from .loader import WEIGHTS_FILE
from .safetensors_io import write_safetensors
from .spec import TensorSpec

MATRIX_STD = 0.02


def draw_tensor(spec: TensorSpec, seed: int, index: int, dtype: torch.dtype, device="cpu",
                norm_init: str = "one_plus") -> torch.Tensor:
    gen = torch.Generator(device=device)
    gen.manual_seed((int(seed) * 1_000_003 + index * 7919 + 17) % (2 ** 63 - 1))
    if spec.init == "integer_table":
        return torch.randint(0, 2 ** 15, spec.shape, generator=gen, device=device, dtype=torch.int32)
    t = torch.randn(spec.shape, generator=gen, device=device, dtype=torch.float32) * MATRIX_STD
    if spec.init == "norm_weight" and norm_init == "one_plus":
        t = t + 1.0
    return t.to(dtype)


def random_tensors(specs: Iterable[TensorSpec], seed: int, dtype: torch.dtype, device="cpu",
                   norm_init: str = "one_plus") -> dict[str, torch.Tensor]:
    return {s.name: draw_tensor(s, seed, i, dtype, device, norm_init) for i, s in enumerate(specs)}


def write_random_model(config, specs: Iterable[TensorSpec], seed: int, out_dir, dtype=torch.bfloat16,
                       norm_init: str = "one_plus") -> Path:
    """Write `out_dir`/config.json and `out_dir`/model.safetensors; returns out_dir."""
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    (out_dir / "config.json").write_text(json.dumps(config.to_json_dict(), indent=1))
    tensors = random_tensors(specs, seed, dtype, "cpu", norm_init)
    write_safetensors(out_dir / WEIGHTS_FILE, tensors, {"format": "pt", "seed": seed})
    return out_dir
