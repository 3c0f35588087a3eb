"""Random-weights mode: tensors from a configuration and a seed, on the device or into a model folder.

The reference has no such mode (its only source of weights is a GGUF file, model_f32.go:133-293).
Here every tensor is drawn from a counter-based generator, so that the device can fill a model in
place and a written folder holds the very same values:

  element e of tensor number i (its place in the model's tensor list) comes from Philox4x32-10
  with key (seed & 0xffffffff, i) and counter (e // 4 as two words, seed >> 32, 0); output words
  (0, 1) give elements 4c and 4c+1, words (2, 3) elements 4c+2 and 4c+3, as the cosine and sine
  branch of a Box-Muller pair: u1 = (a + 1/2) / 2^32, u2 = b / 2^32, r = sqrt(-2 ln u1),
  z = r cos(2 pi u2) | r sin(2 pi u2); value = mean + std * z in double, rounded to float32 and,
  for bfloat16 storage, once more.

Logarithm, sine and cosine are series of +, * and / in double with every operation rounded on
its own; this file states them in numpy, csrc/philox.cuh on the device, and the two give the same
bits. How a tensor is drawn is looked up by its spec's `init` name in INIT_LAWS ("matrix":
N(0, 0.02); "norm_weight": 1 + N(0, 0.02), or N(0, 0.02) with norm_init="plain";
"integer_table": uniform integers below 2^15); a part whose tensor needs another law registers it.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from pathlib import Path
from typing import Iterable

import numpy as np
import torch

from .loader import WEIGHTS_FILE
from .safetensors_io import write_safetensors
from .spec import TensorSpec

MATRIX_STD = 0.02
RANDOM_PREFIX = "random:"


@dataclass(frozen=True)
class Normal:
    mean: float
    std: float


@dataclass(frozen=True)
class UniformInteger:
    modulus: int            # values 0 .. modulus-1, stored as int32


INIT_LAWS: dict[str, Normal | UniformInteger] = {
    "matrix": Normal(0.0, MATRIX_STD),
    "norm_weight": Normal(1.0, MATRIX_STD),
    "integer_table": UniformInteger(2 ** 15),
}


def register_init(name: str, law: Normal | UniformInteger, replace: bool = False) -> None:
    if name in INIT_LAWS and not replace:
        raise ValueError(f"init law {name!r} is already registered")
    INIT_LAWS[name] = law


def law_for(spec: TensorSpec, norm_init: str = "one_plus"):
    try:
        law = INIT_LAWS[spec.init]
    except KeyError:
        raise ValueError(f"tensor {spec.name!r} asks for the unknown init law {spec.init!r}; "
                         f"registered: {', '.join(sorted(INIT_LAWS))}") from None
    if spec.init == "norm_weight" and norm_init == "plain":
        return Normal(0.0, law.std)
    return law


# --------------------------------------------------------------------------- the generator on the host
_M0, _M1, _W0, _W1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57), 0x9E3779B9, 0xBB67AE85
_MASK = np.uint64(0xFFFFFFFF)
_S32 = np.uint64(32)


def philox4x32_10(c0, c1, c2, c3, k0: int, k1: int):
    """Vectorised Philox4x32-10: counter words as uint64 arrays holding 32-bit values, key as ints."""
    c = [np.asarray(v, dtype=np.uint64) for v in (c0, c1, c2, c3)]
    for _ in range(10):
        p0, p1 = _M0 * c[0], _M1 * c[2]
        c = [(p1 >> _S32) ^ c[1] ^ np.uint64(k0), p1 & _MASK, (p0 >> _S32) ^ c[3] ^ np.uint64(k1), p0 & _MASK]
        k0, k1 = (k0 + _W0) & 0xFFFFFFFF, (k1 + _W1) & 0xFFFFFFFF
    return c


def _exact_log(u: np.ndarray) -> np.ndarray:
    m, e = np.frexp(u)
    low = m < 0.70710678118654752440
    m = np.where(low, m * 2.0, m)
    e = np.where(low, e - 1, e).astype(np.float64)
    s = (m + -1.0) / (m + 1.0)
    s2 = s * s
    p = np.full_like(s, 1.0 / 19.0)
    for k in range(17, 0, -2):
        p = p * s2 + 1.0 / float(k)
    return e * 0.693147180559945309417 + (2.0 * s) * p


def _exact_sincos_turn(b: np.ndarray):
    b = b.astype(np.uint64)
    q = (b >> np.uint64(30)).astype(np.int64)
    r = (b & np.uint64(0x3FFFFFFF)).astype(np.int64)
    swap = r > 0x20000000
    rr = np.where(swap, 0x40000000 - r, r).astype(np.float64)
    y = (rr * (1.0 / 1073741824.0)) * 1.57079632679489661923
    y2 = y * y
    ps = np.full_like(y, -1.0 / 1307674368000.0)
    for coef in (1.0 / 6227020800.0, -1.0 / 39916800.0, 1.0 / 362880.0, -1.0 / 5040.0, 1.0 / 120.0, -1.0 / 6.0, 1.0):
        ps = ps * y2 + coef
    sn = ps * y
    pc = np.full_like(y, 1.0 / 20922789888000.0)
    for coef in (-1.0 / 87178291200.0, 1.0 / 479001600.0, -1.0 / 3628800.0, 1.0 / 40320.0, -1.0 / 720.0, 1.0 / 24.0, -0.5):
        pc = pc * y2 + coef
    cs = pc * y2 + 1.0
    c1, s1 = np.where(swap, sn, cs), np.where(swap, cs, sn)
    c = np.select([q == 0, q == 1, q == 2], [c1, -s1, -c1], s1)
    s = np.select([q == 0, q == 1, q == 2], [s1, c1, -s1], -c1)
    return c, s


def _normal_pair(a: np.ndarray, b: np.ndarray):
    u1 = (a.astype(np.float64) + 0.5) * (1.0 / 4294967296.0)
    r = np.sqrt(-2.0 * _exact_log(u1))
    c, s = _exact_sincos_turn(b)
    return r * c, r * s


def _host_words(n: int, seed: int, index: int, first_counter: int, n_counters: int):
    c = np.arange(first_counter, first_counter + n_counters, dtype=np.uint64)
    zeros = np.zeros_like(c)
    return philox4x32_10(c & _MASK, c >> _S32, zeros + np.uint64((seed >> 32) & 0xFFFFFFFF), zeros,
                         seed & 0xFFFFFFFF, index & 0xFFFFFFFF)


_HOST_CHUNK = 1 << 15        # counters per pass: the working arrays of a pass stay in the cache
_HOST_THREADS = max(1, min(16, os.cpu_count() or 1))


def draw_host(spec: TensorSpec, seed: int, index: int, dtype: torch.dtype, norm_init: str = "one_plus") -> torch.Tensor:
    """Tensor `index` of a model drawn on the host (numpy; passes of 32 Ki counters spread over threads)."""
    law = law_for(spec, norm_init)
    n = int(np.prod(spec.shape)) if spec.shape else 1
    n_counters = (n + 3) // 4
    integer = isinstance(law, UniformInteger)
    out = np.empty(n_counters * 4, dtype=np.int32 if integer else np.float32)

    def one_pass(c0: int) -> None:
        nc = min(_HOST_CHUNK, n_counters - c0)
        w = _host_words(n, seed, index, c0, nc)
        view = out[c0 * 4:(c0 + nc) * 4].reshape(nc, 4)
        if integer:
            for j in range(4):
                view[:, j] = (w[j] % np.uint64(law.modulus)).astype(np.int32)
        else:
            z0, z1 = _normal_pair(w[0], w[1])
            z2, z3 = _normal_pair(w[2], w[3])
            for j, z in enumerate((z0, z1, z2, z3)):
                view[:, j] = (law.mean + law.std * z).astype(np.float32)

    starts = range(0, n_counters, _HOST_CHUNK)
    if len(starts) > 1 and _HOST_THREADS > 1:
        from concurrent.futures import ThreadPoolExecutor
        with ThreadPoolExecutor(_HOST_THREADS) as pool:
            list(pool.map(one_pass, starts))
    else:
        for c0 in starts:
            one_pass(c0)
    t = torch.from_numpy(out[:n].reshape(spec.shape))
    return t if integer else t.to(dtype)


def draw_device(spec: TensorSpec, seed: int, index: int, dtype: torch.dtype, device, norm_init: str = "one_plus") -> torch.Tensor:
    """The same tensor filled in place on a CUDA device by the fill kernels (csrc/lib_random.cu)."""
    from ..csrc.bindings import RandomKernels
    law = law_for(spec, norm_init)
    kernels = RandomKernels()
    if isinstance(law, UniformInteger):
        t = torch.empty(spec.shape, dtype=torch.int32, device=device)
        kernels.fill_integer(t, seed, index, law.modulus)
    else:
        t = torch.empty(spec.shape, dtype=dtype, device=device)
        kernels.fill_normal(t, seed, index, law.mean, law.std)
    return t


def random_tensors(specs: Iterable[TensorSpec], seed: int, dtype: torch.dtype, device="cpu",
                   norm_init: str = "one_plus") -> dict[str, torch.Tensor]:
    """Every tensor of `specs`, numbered in order, stored as `dtype` (float32 or bfloat16): on the
    host through numpy, on a CUDA device through the fill kernels; same values either way."""
    if dtype not in (torch.float32, torch.bfloat16):
        raise ValueError(f"random weights are stored as float32 or bfloat16, not {dtype}")
    dev = torch.device(device)
    if dev.type == "cuda":
        with torch.cuda.device(dev):
            return {s.name: draw_device(s, seed, i, dtype, dev, norm_init) for i, s in enumerate(specs)}
    return {s.name: draw_host(s, seed, i, dtype, norm_init) for i, s in enumerate(specs)}


def write_random_model(config, specs: Iterable[TensorSpec], seed: int, out_dir, dtype=torch.bfloat16,
                       norm_init: str = "one_plus", device="cpu") -> Path:
    """Write `out_dir`/config.json and `out_dir`/model.safetensors; returns out_dir. `device`: where
    the values are drawn (a CUDA device is much faster for large models; the file is the same)."""
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    (out_dir / "config.json").write_text(json.dumps(config.to_json_dict(), indent=1))
    tensors = {k: v.cpu() for k, v in random_tensors(specs, seed, dtype, device, norm_init).items()}
    write_safetensors(out_dir / WEIGHTS_FILE, tensors, {"format": "pt", "seed": seed})
    return out_dir


# --------------------------------------------------------------------------- "random:<config.json>[:seed[:dtype]]"
@dataclass(frozen=True)
class RandomSpec:
    config_path: str
    seed: int = 0
    dtype: torch.dtype = torch.bfloat16       # the precision the weights are "stored" in


def is_random_spec(model) -> bool:
    return isinstance(model, str) and model.startswith(RANDOM_PREFIX)


def parse_random_spec(text: str) -> RandomSpec:
    """`random:<config.json>[:seed[:bfloat16|float32]]`: a model that exists only as a configuration
    and a seed. Takes the place of a model folder wherever one is named."""
    if not is_random_spec(text):
        raise ValueError(f"{text!r} is not a random-model spec (random:<config.json>[:seed[:dtype]])")
    body = text[len(RANDOM_PREFIX):]
    parts = body.split(":")
    seed, dtype = 0, torch.bfloat16
    names = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "f32": torch.float32}
    if len(parts) >= 2 and parts[-1] in names and _is_int(parts[-2]):
        dtype, seed, parts = names[parts[-1]], int(parts[-2]), parts[:-2]
    elif len(parts) >= 2 and _is_int(parts[-1]):
        seed, parts = int(parts[-1]), parts[:-1]
    path = ":".join(parts)
    if not path:
        raise ValueError(f"{text!r} names no config.json")
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    return RandomSpec(path, seed, dtype)


def _is_int(s: str) -> bool:
    try:
        int(s)
        return True
    except ValueError:
        return False
