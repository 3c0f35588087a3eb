"""Tiny configurations, random model folders and comparison helpers shared by the tests."""
from __future__ import annotations

import json
import sys
import os
from pathlib import Path

import numpy as np
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

import plain_llama as plain  # noqa: E402

# Two tiny configurations that differ in every size and option, and a third with a window and a
# head width that is no power of two.
TINY_A = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "intermediate_size": 176, "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": True, "max_position_embeddings": 128, "rope_pairing": "interleaved",
    "hidden_act": "silu", "eos_token_id": 7,
}
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32,
    "intermediate_size": 256, "vocab_size": 384, "rope_theta": 100000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": False, "max_position_embeddings": 256, "rope_pairing": "half",
    "partial_rotary_factor": 0.5,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
    "hidden_act": "silu", "eos_token_id": [11, 12],
}
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 144, "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 48,
    "intermediate_size": 200, "vocab_size": 1003, "rope_theta": 500000.0, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "max_position_embeddings": 512, "sliding_window": 24,
    "hidden_act": "silu",
}
TINY = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 2)}


def make_model_dir(tmp, raw_cfg: dict, seed: int, dtype=torch.bfloat16, norm_init="one_plus") -> Path:
    """Write a random-weights model folder with the library's own random mode."""
    from scriptling_llm_lib_b200 import models  # noqa: F401
    from scriptling_llm_lib_b200.config.registry import architecture_for
    from scriptling_llm_lib_b200.engine.model import DecoderModel
    from scriptling_llm_lib_b200.weights.random_init import write_random_model
    arch = architecture_for(raw_cfg["architectures"][0])
    cfg = arch.config_class.from_dict(raw_cfg, "test config")
    specs = DecoderModel(arch.layout(cfg)).tensor_specs()
    return write_random_model(cfg, specs, seed, Path(tmp), dtype, norm_init)


def plain_model(model_dir, act_round=None, schedule=None) -> "plain.PlainLlama":
    cfg, weights = plain.load_folder(model_dir)
    return plain.PlainLlama(cfg, weights, act_round=act_round, schedule=schedule)


def random_ids(n: int, vocab: int, seed: int) -> list[int]:
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()


def rel_err(got, want) -> float:
    """max |difference| over the row's largest |wanted value|, the largest over rows: the
    vector-scale measure the reference uses for kernel parity (q8q8_test.go:73-84)."""
    got = torch.as_tensor(np.asarray(got), dtype=torch.float64)
    want = torch.as_tensor(np.asarray(want), dtype=torch.float64)
    if got.shape != want.shape:
        raise AssertionError(f"shapes differ: {tuple(got.shape)} vs {tuple(want.shape)}")
    if got.dim() == 1:
        got, want = got[None], want[None]
    if not torch.isfinite(got).all():
        return float("inf")
    scale = want.abs().amax(dim=-1).clamp_min(1e-30)
    return float(((got - want).abs().amax(dim=-1) / scale).max())


# tolerances, fixed before any measurement: float32 arithmetic against the float64 plain
# implementation; bfloat16 against the plain implementation rounding activations where the engine
# stores them (8 mantissa bits: 2^-9 relative per rounding, a few dozen roundings deep)
TOL_F32 = 1e-4
TOL_BF16 = 3e-2
