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
# Two more with the head widths that the tensor-core kernels of the bfloat16 path take (64 and 128):
# grouped queries with a window that cuts long prompts, and one key/value head for six query heads (also windowed)
TINY_D = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 200, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 64,
    "intermediate_size": 328, "vocab_size": 515, "rope_theta": 20000.0, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": True, "max_position_embeddings": 512, "sliding_window": 150, "hidden_act": "silu",
}
TINY_E = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 264, "num_attention_heads": 6, "num_key_value_heads": 1, "head_dim": 128,
    "intermediate_size": 136, "vocab_size": 777, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": False, "max_position_embeddings": 512, "rope_pairing": "interleaved", "sliding_window": 200,
    "hidden_act": "silu",
}
TINY = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 2), "D": (TINY_D, 3), "E": (TINY_E, 4)}


def make_model_dir(tmp, raw_cfg: dict, seed: int, dtype=torch.bfloat16, norm_init="one_plus", device=None) -> Path:
    """Write a random-weights model folder with the library's own random mode (values drawn on the
    GPU where there is one: the same bits as on the host, which its own test shows, and faster)."""
    if device is None:
        device = "cuda:0" if torch.cuda.is_available() else "cpu"
    from scriptling_llm_lib_b200 import models  # noqa: F401
    from scriptling_llm_lib_b200.config.registry import architecture_for
    from scriptling_llm_lib_b200.engine.model import DecoderModel
    from scriptling_llm_lib_b200.weights.random_init import write_random_model
    arch = architecture_for(raw_cfg["architectures"][0])
    cfg = arch.config_class.from_dict(raw_cfg, "test config")
    specs = DecoderModel(arch.layout(cfg)).tensor_specs()
    return write_random_model(cfg, specs, seed, Path(tmp), dtype, norm_init, device)


def plain_model(model_dir, act_round=None, schedule=None) -> "plain.PlainLlama":
    cfg, weights = plain.load_folder(model_dir)
    return plain.PlainLlama(cfg, weights, act_round=act_round, schedule=schedule)


def plain_model_bf16(model_dir, schedule=None) -> "plain.PlainLlama":
    """The plain implementation rounding to bfloat16 where the engine's bfloat16 path writes an
    activation to memory: norm outputs, q, k, v before and after rotation, attention output, the
    gated activation, o and down outputs; gate and up are not rounded on their own (the gate is
    applied in the product's epilogue)."""
    return plain_model(model_dir, act_round=plain.bf16_activations(skip=("gate", "up")), schedule=schedule)


def check_logits(got, want, want16, dtype: str, what: str = "") -> None:
    """32-bit: against the plain implementation within TOL_F32. bfloat16: against the plain
    implementation with rounded activations within TOL_BF16_ROUNDED and against the unrounded one
    within TOL_BF16."""
    if dtype == "float32":
        e = rel_err(got, want)
        assert e < TOL_F32, f"{what}: {e:.3g}"
        return
    e16, e = rel_err(got, want16), rel_err(got, want)
    assert e16 < TOL_BF16_ROUNDED, f"{what} against the rounding plain implementation: {e16:.3g}"
    assert e < TOL_BF16, f"{what}: {e:.3g}"
    MEASURED.append((what, e16, e))


# --------------------------------------------------------------------------- the C++ statement
_CPP_BINARY = None


def cpp_plain_binary():
    """tests/plain_cpp/plain_llama.cpp compiled with g++ (no fused multiply-add, no fast-math); None
    where there is no compiler."""
    global _CPP_BINARY
    import shutil
    import subprocess
    import tempfile
    if _CPP_BINARY is None:
        gxx = shutil.which("g++")
        if gxx is None:
            return None
        src = Path(__file__).resolve().parent / "plain_cpp" / "plain_llama.cpp"
        out = Path(tempfile.mkdtemp(prefix="plain_cpp_")) / "plain_llama"
        subprocess.run([gxx, "-O2", "-std=c++17", "-ffp-contract=off", "-o", str(out), str(src)], check=True)
        _CPP_BINARY = out
    return _CPP_BINARY


def cpp_logits(model_dir, ids, tmp) -> np.ndarray:
    """Logits [S, vocab] of the C++ plain statement (the reference's float32 arithmetic) for a model
    folder: weights widened to float32 into one flat file, the configuration as numbers."""
    import subprocess
    cfg, w = plain.load_folder(model_dir)
    hd = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]
    sc = cfg.get("rope_scaling") or {}
    kind = {None: 0, "default": 0, "linear": 1, "llama3": 2}[sc.get("rope_type", sc.get("type"))]
    numbers = {
        "layers": cfg["num_hidden_layers"], "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
        "kv_heads": cfg.get("num_key_value_heads") or cfg["num_attention_heads"], "head_dim": hd,
        "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
        "rotary_dim": int(hd * cfg.get("partial_rotary_factor", 1.0)), "eps": cfg.get("rms_norm_eps", 1e-5),
        "theta": cfg.get("rope_theta", 10000.0), "interleaved": int(cfg.get("rope_pairing", "half") == "interleaved"),
        "tied": int(bool(cfg.get("tie_word_embeddings", False))), "window": cfg.get("sliding_window") or 0,
        "scaling_kind": kind, "factor": sc.get("factor", 1.0), "low": sc.get("low_freq_factor", 1.0),
        "high": sc.get("high_freq_factor", 4.0), "original": sc.get("original_max_position_embeddings", 8192),
    }
    tmp = Path(tmp)
    tmp.mkdir(parents=True, exist_ok=True)
    lines, off, chunks = [f"{k} {float(v)!r}" for k, v in numbers.items()], 0, []
    for name, t in w.items():
        a = t.to(torch.float32).numpy().ravel()
        lines.append(f"tensor {name} {off} {a.size}")
        chunks.append(a)
        off += a.size
    (tmp / "manifest.txt").write_text("\n".join(lines) + "\n")
    np.concatenate(chunks).astype("<f4").tofile(tmp / "weights.f32")
    np.asarray(ids, dtype="<i4").tofile(tmp / "tokens.i32")
    subprocess.run([str(cpp_plain_binary()), str(tmp / "manifest.txt"), str(tmp / "weights.f32"), str(tmp / "tokens.i32"),
                    str(tmp / "out.f32")], check=True)
    return np.fromfile(tmp / "out.f32", dtype="<f4").reshape(len(ids), cfg["vocab_size"])


MEASURED: list = []       # (what, error against the rounding oracle, against the unrounded): printed with -s


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
# bfloat16 against the plain implementation that rounds to bfloat16 where the engine stores
# activations (`plain_model_bf16`): what is left is the order of sums, the probabilities' rounding
# before P V and the products whose partial sums stay in 32-bit.
TOL_BF16_ROUNDED = 1.5e-2


# --------------------------------------------------------------------------- trace replay client
class Replay:
    """Drives bin/trace_run as a user would: one JSON line per step, waits for `done <step>`."""

    def __init__(self, model_dir, dtype: str, out_dir, max_tokens: int, vocab: int):
        import subprocess
        root = Path(__file__).resolve().parent.parent
        self.out_dir, self.vocab, self.step_no = Path(out_dir), vocab, 0
        self.proc = subprocess.Popen(
            [sys.executable, str(root / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype, "--out",
             str(out_dir), "--max-tokens", str(max_tokens)], stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)

    def step(self, entries: list[tuple[str, list[int], list[int]]], end=()) -> np.ndarray | None:
        """entries: (request id, tokens, want). Returns the logits rows written for this step."""
        rec = {"step": self.step_no, "entries": [{"id": i, "tokens": t, "want": w} for i, t, w in entries], "end": list(end)}
        self.proc.stdin.write(json.dumps(rec) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline().strip()
        if line != f"done {self.step_no}":
            raise AssertionError(f"trace_run answered {line!r} to step {self.step_no} (exit code {self.proc.poll()})")
        n_want = sum(len(w) for _, _, w in entries)
        path = self.out_dir / f"{self.step_no}.f32"
        self.step_no += 1
        if n_want == 0:
            assert not path.exists()
            return None
        return np.fromfile(path, dtype="<f4").reshape(n_want, self.vocab)

    def close(self) -> int:
        self.proc.stdin.close()
        return self.proc.wait(timeout=120)


def replay_whole(rp: Replay, rid: str, ids: list[int]) -> np.ndarray:
    return rp.step([(rid, ids, list(range(len(ids))))], end=[rid])


def replay_tail_stepwise(rp: Replay, rid: str, ids: list[int], tail: int = 32) -> np.ndarray:
    head = len(ids) - tail
    rows = []
    if head > 0:
        rows.append(rp.step([(rid, ids[:head], list(range(head)))]))
    for j in range(max(head, 0), len(ids)):
        rows.append(rp.step([(rid, [ids[j]], [0])], end=[rid] if j == len(ids) - 1 else []))
    return np.concatenate(rows)


def replay_batch(rp: Replay, reqs: dict[str, list[int]], prompt_lens: dict[str, int]) -> dict[str, np.ndarray]:
    """The requests start together with prompts of `prompt_lens`, then go on by one token each;
    shorter requests end earlier. Returns every request's logits at all its places."""
    got = {r: [] for r in reqs}
    order = list(reqs)
    ends = [r for r in order if prompt_lens[r] == len(reqs[r])]
    out = rp.step([(r, reqs[r][:prompt_lens[r]], list(range(prompt_lens[r]))) for r in order], end=ends)
    off = 0
    for r in order:
        got[r].append(out[off:off + prompt_lens[r]])
        off += prompt_lens[r]
    pos = dict(prompt_lens)
    live = [r for r in order if r not in ends]
    while live:
        ends = [r for r in live if pos[r] + 1 == len(reqs[r])]
        out = rp.step([(r, [reqs[r][pos[r]]], [0]) for r in live], end=ends)
        for i, r in enumerate(live):
            got[r].append(out[i:i + 1])
            pos[r] += 1
        live = [r for r in live if r not in ends]
    return {r: np.concatenate(v) for r, v in got.items()}
