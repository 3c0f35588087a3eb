"""The Python entry point, in the manner of the reference's `llm.generate`.

Reference: `llm.generate(model_path, prompt, max_tokens=100, strategy="greedy", temperature=1.0,
top_k=50, top_p=0.9, repeat_penalty=1.15, repeat_last_n=64, ..., stats=False)` (model.go:853-977,
registered in llm.go:458-473). Same positions, names, meanings and defaults here; the model is a
folder (config.json + model.safetensors) and the prompt a list of token ids, or a list of such
lists for a batch of unequal prompts (tokenizer and chat template are not part of this library).
Models are loaded once per (folder, dtype) and kept, like the reference's global model cache
(model_f32.go:42-70).
"""
from __future__ import annotations

import os
import threading

from .cache.needs import PAGE
from .engine.generate import GenerationResult, Generator
from .engine.step import DTYPES, Engine
from .sampling.sampler import Sampler, SamplingOptions

VERSION = "0.1.0"

_models: dict[tuple[str, str, str], tuple[Engine, Sampler]] = {}
_models_lock = threading.Lock()
_run_locks: dict[int, threading.Lock] = {}      # one generation at a time per engine (its cache and graphs are shared)


def load(model_dir, dtype="bfloat16", device="cuda:0", max_tokens: int = 4096, max_seqs: int | None = None):
    """The cached (engine, sampler) of a model folder, or of `random:<config.json>[:seed[:dtype]]`."""
    key = (_model_key(model_dir), str(DTYPES[dtype]), str(device))
    with _models_lock:
        if key not in _models:
            eng = Engine.from_folder(model_dir, dtype, max_tokens, max_seqs, device)
            _models[key] = (eng, Sampler(eng.device))
        return _models[key]


def _model_key(model_dir) -> str:
    from .weights.random_init import is_random_spec
    return str(model_dir) if is_random_spec(model_dir) else os.path.realpath(str(model_dir))


def unload(model_dir=None) -> None:
    """Drop one cached model, or all of them."""
    with _models_lock:
        for key in [k for k in _models if model_dir is None or k[0] == _model_key(model_dir)]:
            _run_locks.pop(id(_models[key][0]), None)
            del _models[key]


def _fit_cache(eng: Engine, prompts, max_tokens, max_batch):
    """Grow the engine's cache so the requests run in as few batches as memory allows."""
    import torch
    pages = [(min(eng.layout.max_positions, len(p) + max_tokens - 1) + PAGE - 1) // PAGE for p in prompts]
    if max_batch:
        pages = sorted(pages, reverse=True)[:max_batch]
    want_pages, want_seqs = sum(pages), len(pages)
    if want_pages <= eng.cache.n_pages and want_seqs <= eng.cache.n_slots:
        return
    free, _ = torch.cuda.mem_get_info(eng.device)
    have = eng.cache.n_pages * eng.bytes_per_page()
    # what a prompt step's activations and the captured decode steps need stays free
    afford = max(0, int((free + have - eng.activation_reserve_bytes()) * 0.9)) // max(1, eng.bytes_per_page())
    n_pages = max(max(pages), min(want_pages, afford), eng.cache.n_pages)
    eng.resize_cache(n_pages * PAGE, max(want_seqs, eng.cache.n_slots))


def generate(model_dir, prompt_ids, max_tokens: int = 100, strategy: str = "greedy", *, temperature: float = 1.0,
             top_k: int = 50, top_p: float = 0.9, repeat_penalty: float = 1.15, repeat_last_n: int = 64,
             seed: int = 0, stop_ids=None, dtype: str = "bfloat16", device: str = "cuda:0", max_batch: int | None = None,
             stats: bool = False, on_step=None):
    """Generate from token ids.

    prompt_ids: a list of ids -> returns the list of generated ids; a list of lists (unequal
    lengths allowed) -> returns one list per prompt. `max_tokens` counts every sampled token,
    the first included; a stop token (config.json's eos ids unless `stop_ids` is given; pass an
    empty list for none) is kept in the output. `strategy` "greedy" ignores temperature and
    penalty; `temperature=0.0` means greedy. With `stats=True` returns (ids, stats) where stats
    holds prompt_tokens, generated_tokens, prefill_ms, decode_ms (lists when given a batch).
    """
    single = len(prompt_ids) > 0 and not isinstance(prompt_ids[0], (list, tuple))
    prompts = [list(prompt_ids)] if single else [list(p) for p in prompt_ids]
    options = SamplingOptions(strategy, float(temperature), int(top_k), float(top_p), float(repeat_penalty),
                              int(repeat_last_n))
    eng, sampler = load(model_dir, dtype, device)
    with _models_lock:
        run_lock = _run_locks.setdefault(id(eng), threading.Lock())
    with run_lock:      # concurrent callers of one model take turns (the reference gives each a clone; here they share a cache)
        _fit_cache(eng, prompts, max_tokens, max_batch)
        results = Generator(eng, sampler).generate(prompts, max_tokens, options, stop_ids, seed, max_batch, on_step)
    ids = [r.tokens for r in results]
    if not stats:
        return ids[0] if single else ids
    st = _stats(results)
    return (ids[0], {k: v[0] for k, v in st.items()}) if single else (ids, st)


def _stats(results: list[GenerationResult]) -> dict:
    return {"prompt_tokens": [r.prompt_tokens for r in results],
            "generated_tokens": [r.generated_tokens for r in results],
            "finish_reason": [r.finish_reason for r in results],
            "prefill_ms": [r.prefill_ms for r in results], "decode_ms": [r.decode_ms for r in results]}


def random_model(config, seed: int, out_dir, dtype: str = "bfloat16"):
    """Write a model folder (config.json, model.safetensors) with random weights drawn from `seed`
    for `config`: a dict of config.json keys or the path of such a file. Returns the folder, which
    `generate` and the command line then take like any other. Needs no GPU."""
    import json
    from pathlib import Path
    import torch
    from . import models  # noqa: F401  (registers the architectures)
    from .config.registry import architecture_for
    from .engine.model import DecoderModel
    from .weights.random_init import write_random_model
    where = "config"
    if not isinstance(config, dict):
        where = str(config)
        config = json.loads(Path(config).read_text())
    arch = architecture_for(config["architectures"][0] if config.get("architectures") else None)
    cfg = arch.config_class.from_dict(config, where)
    specs = DecoderModel(arch.layout(cfg)).tensor_specs()
    return write_random_model(cfg, specs, int(seed), Path(out_dir), {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype])
