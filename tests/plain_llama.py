"""Plain, slow statement of the Llama / SmolLM2 decoder, written from the reference's formulas.

This file rests on the formulas of martinsuchenak/scriptling-llm-lib (file:line cited at every
function); the reference itself is Go and cannot be compiled where these tests run, so nothing here
was checked against its binary.

Whole sequences only, no cache, one function per part, float64 throughout (the reference computes
in float32 with float64 islands; float64 everywhere is the same mathematics with less rounding).
It shares no code with the engine: it reads its own copy of config.json and its own safetensors
parse. Weights are used exactly as stored (bfloat16 and float32 both convert to float64 exactly).

`act_round(name, tensor)` lets a caller imitate an engine that stores activations in bfloat16
between kernels: it is called where such an engine may write an activation to memory, with the
name of that place ("norm", "q", "k", "v", "q_rot", "k_rot", "attn", "o", "gate", "up", "act",
"down", "final_norm"), and returns what the next part reads. With `act_round=None` nothing is
rounded.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

F64 = torch.float64


def round_bf16(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.float32).to(torch.bfloat16).to(F64)


def bf16_activations(skip=()):
    """An `act_round` that rounds to bfloat16 everywhere but at the places named in `skip`."""
    return lambda name, t: t if name in skip else round_bf16(t)


# --------------------------------------------------------------------------- files
_ST_DTYPES = {"F32": (np.float32, 4), "BF16": (np.uint16, 2), "F16": (np.float16, 2), "I32": (np.int32, 4)}


def read_safetensors(path) -> dict[str, torch.Tensor]:
    """Own minimal parse of a safetensors file: u64 header length, JSON header, raw data."""
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        npdt, _ = _ST_DTYPES[meta["dtype"]]
        b, e = meta["data_offsets"]
        arr = np.frombuffer(raw, dtype=npdt, count=(e - b) // np.dtype(npdt).itemsize, offset=8 + hlen + b)
        arr = arr.reshape(meta["shape"])
        if meta["dtype"] == "BF16":
            t = torch.from_numpy((arr.astype(np.uint32) << 16).view(np.float32).copy()).to(F64)
        else:
            t = torch.from_numpy(arr.copy()).to(F64)
        out[name] = t
    return out


def load_folder(model_dir):
    model_dir = Path(model_dir)
    cfg = json.loads((model_dir / "config.json").read_text())
    weights = read_safetensors(model_dir / "model.safetensors")
    return cfg, weights


# --------------------------------------------------------------------------- parts
def rms_norm(x, w, eps):
    """y = (x * 1/sqrt(mean(x^2) + eps)) * w, weight used as is.  float32_ops.go:159-172."""
    ss = (x * x).sum(dim=-1, keepdim=True)
    inv = 1.0 / torch.sqrt(ss / x.shape[-1] + eps)
    return (x * inv) * w


def rope_inv_freq(rot_dim, theta, scaling=None):
    """f_i = 1 / theta^(2i/rot_dim), i < rot_dim/2.  model_f32.go:252-260.

    The reference has no frequency rescaling; the llama3 rule (configs of the family carry it in
    config.json's rope_scaling) rewrites the table only: long wavelengths are divided by `factor`,
    short ones kept, the band between blended linearly in the frequency's period count.
    """
    i = torch.arange(rot_dim // 2, dtype=F64)
    f = 1.0 / (float(theta) ** (2.0 * i / rot_dim))
    if scaling is None:
        return f
    kind = scaling.get("rope_type", scaling.get("type"))
    if kind == "linear":
        return f / float(scaling["factor"])
    if kind != "llama3":
        raise ValueError(f"plain implementation knows no rope scaling {kind!r}")
    factor = float(scaling["factor"])
    lo = float(scaling["low_freq_factor"])
    hi = float(scaling["high_freq_factor"])
    orig = float(scaling["original_max_position_embeddings"])
    out = f.clone()
    for j in range(f.numel()):
        wavelen = 2.0 * math.pi / f[j].item()
        if wavelen > orig / lo:
            out[j] = f[j] / factor
        elif wavelen >= orig / hi:
            smooth = (orig / wavelen - lo) / (hi - lo)
            out[j] = (1.0 - smooth) * f[j] / factor + smooth * f[j]
    return out


def apply_rope(x, positions, inv_freq, pairing):
    """Rotate pairs of x[..., :rot_dim] by angle f_i * position; dims past rot_dim untouched.

    x: [S, heads, hd].  float32_ops.go:174-188 rotates adjacent pairs (2i, 2i+1) ("interleaved");
    the half-split pairing (i, i + rot_dim/2) is the same rotation under a permutation of the
    projection's rows and is what safetensors checkpoints of this family expect.
    """
    half = inv_freq.numel()
    ang = positions.to(F64)[:, None] * inv_freq[None, :]          # [S, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    if pairing == "interleaved":
        x0, x1 = x[..., 0:2 * half:2], x[..., 1:2 * half:2]
        out[..., 0:2 * half:2] = x0 * c - x1 * s
        out[..., 1:2 * half:2] = x0 * s + x1 * c
    elif pairing == "half":
        x0, x1 = x[..., :half], x[..., half:2 * half]
        out[..., :half] = x0 * c - x1 * s
        out[..., half:2 * half] = x0 * s + x1 * c
    else:
        raise ValueError(pairing)
    return out


def attention(q, k, v, q_positions, k_positions, window=None):
    """Causal grouped-query attention, one sequence.  float32_ops.go:190-235, :252-260.

    q: [S, H, hd]; k, v: [Sk, G, hd]; query head h reads key/value head h // (H/G).
    score = (q.k) * (1/sqrt(hd)); keys after the query's position are masked; max-subtracted
    softmax; out = sum p*v.  `window` (not in the reference) also masks keys at a distance of
    `window` or more behind the query.
    """
    S, H, hd = q.shape
    G = k.shape[1]
    n_rep = H // G
    scale = 1.0 / math.sqrt(hd)
    out = torch.zeros(S, H, hd, dtype=F64)
    qp = q_positions[:, None]
    kp = k_positions[None, :]
    masked = kp > qp
    if window is not None:
        masked = masked | (kp <= qp - window)
    for h in range(H):
        g = h // n_rep
        scores = (q[:, h, :] @ k[:, g, :].T) * scale
        scores = scores.masked_fill(masked, float("-inf"))
        m = scores.max(dim=-1, keepdim=True).values
        e = torch.exp(scores - m)
        p = e * (1.0 / e.sum(dim=-1, keepdim=True))
        out[:, h, :] = p @ v[:, g, :]
    return out


def swiglu(gate, up):
    """h = g * sigmoid(g) * u.  model_f32.go:484-490."""
    return gate * (1.0 / (1.0 + torch.exp(-gate))) * up


def linear(x, w):
    """y[r, j] = sum_l x[r, l] * W[j, l]; weights are [out, in].  float32_ops.go:462-482."""
    return x @ w.T


# --------------------------------------------------------------------------- model
class PlainLlama:
    """The whole decoder on one token list.  model_f32.go:359-527."""

    def __init__(self, cfg: dict, weights: dict, act_round=None, schedule=None):
        self.cfg = cfg
        self.w = weights
        self.rnd = act_round if act_round is not None else (lambda name, t: t)
        self.d = cfg["hidden_size"]
        self.H = cfg["num_attention_heads"]
        self.G = cfg.get("num_key_value_heads") or self.H
        self.hd = cfg.get("head_dim") or self.d // self.H
        self.L = cfg["num_hidden_layers"]
        self.eps = cfg.get("rms_norm_eps", 1e-5)
        self.pairing = cfg.get("rope_pairing", "half")
        rot = int(self.hd * cfg.get("partial_rotary_factor", 1.0))
        self.inv_freq = rope_inv_freq(rot, cfg.get("rope_theta", 10000.0), cfg.get("rope_scaling"))
        self.window = cfg.get("sliding_window")
        # order of execution: (layer, cache unit it reads, whether it writes that unit)
        self.schedule = schedule if schedule is not None else [(i, i, True) for i in range(self.L)]

    def block(self, i, x, positions, kv_store, unit, writes):
        """One pre-norm block: norm -> attention -> residual -> norm -> SwiGLU -> residual.
        model_f32.go:382-500."""
        w, p, rnd = self.w, f"model.layers.{i}.", self.rnd
        S = x.shape[0]
        n = rnd("norm", rms_norm(x, w[p + "input_layernorm.weight"], self.eps))
        q = rnd("q", linear(n, w[p + "self_attn.q_proj.weight"])).view(S, self.H, self.hd)
        q = rnd("q_rot", apply_rope(q, positions, self.inv_freq, self.pairing))
        if writes:
            k = rnd("k", linear(n, w[p + "self_attn.k_proj.weight"])).view(S, self.G, self.hd)
            v = rnd("v", linear(n, w[p + "self_attn.v_proj.weight"])).view(S, self.G, self.hd)
            k = rnd("k_rot", apply_rope(k, positions, self.inv_freq, self.pairing))
            kv_store[unit] = (k, v)
        k, v = kv_store[unit]
        a = rnd("attn", attention(q, k, v, positions, positions, self.window)).reshape(S, self.H * self.hd)
        x = x + rnd("o", linear(a, w[p + "self_attn.o_proj.weight"]))
        n2 = rnd("norm", rms_norm(x, w[p + "post_attention_layernorm.weight"], self.eps))
        g = rnd("gate", linear(n2, w[p + "mlp.gate_proj.weight"]))
        u = rnd("up", linear(n2, w[p + "mlp.up_proj.weight"]))
        h = rnd("act", swiglu(g, u))
        x = x + rnd("down", linear(h, w[p + "mlp.down_proj.weight"]))
        return x

    def hidden(self, ids):
        ids = torch.as_tensor(ids, dtype=torch.long)
        x = self.w["model.embed_tokens.weight"][ids]             # model_f32.go:363-369
        positions = torch.arange(len(ids))
        kv_store = {}
        for layer, unit, writes in self.schedule:
            x = self.block(layer, x, positions, kv_store, unit, writes)
        return x

    def logits(self, ids):
        """Logits at every position of `ids`: [S, V].  model_f32.go:502-527 (there: last row)."""
        x = self.hidden(ids)
        n = self.rnd("final_norm", rms_norm(x, self.w["model.norm.weight"], self.eps))
        head = self.w["model.embed_tokens.weight"] if self.cfg.get("tie_word_embeddings", False) \
            else self.w["lm_head.weight"]
        return linear(n, head)


# --------------------------------------------------------------------------- sampling
def argmax_first(logits):
    """First index of the maximum, strict '>'.  float32_ops.go:812-822."""
    best, best_v = 0, logits[0]
    for i in range(1, len(logits)):
        if logits[i] > best_v:
            best, best_v = i, logits[i]
    return best


def softmax_t(logits, temperature):
    """softmax(logits / T) with max subtraction.  model.go:805-826."""
    z = np.asarray(logits, dtype=np.float64) / temperature
    e = np.exp(z - z.max())
    return e * (1.0 / e.sum())


def weighted_pick(probs, u):
    """First i with u <= cumsum_i, else the last index.  model.go:828-838."""
    cum = 0.0
    for i, p in enumerate(probs):
        cum += p
        if u <= cum:
            return i
    return len(probs) - 1


def apply_repeat_penalty(logits, recent, penalty, last_n):
    """Each distinct in-range token of the last `last_n` of `recent`: positive logit /= penalty,
    else *= penalty.  sampling.go:314-336."""
    logits = np.array(logits, dtype=np.float64)
    seen = set()
    for t in list(recent)[max(0, len(recent) - last_n):]:
        if t < 0 or t >= len(logits) or t in seen:
            continue
        seen.add(t)
        logits[t] = logits[t] / penalty if logits[t] > 0 else logits[t] * penalty
    return logits


def sample(logits, strategy, temperature=1.0, top_k=50, top_p=0.9, u=0.0):
    """model.go:701-799 with the uniform draw `u` given by the caller."""
    logits = np.asarray(logits, dtype=np.float64)
    n = len(logits)
    if strategy == "greedy":
        return argmax_first(logits)
    if strategy == "temperature":
        return weighted_pick(softmax_t(logits, temperature), u)
    if strategy == "top_k":
        k = 50 if top_k <= 0 else min(top_k, n)
        # the k largest logits; the reference's quick-select leaves them in no defined order, so
        # the draw is defined here over ascending token index
        order = np.argsort(-logits, kind="stable")[:k]
        order = np.sort(order)
        return int(order[weighted_pick(softmax_t(logits[order], temperature), u)])
    if strategy == "top_p":
        probs = softmax_t(logits, temperature)
        order = np.argsort(-probs, kind="stable")               # insertion sort, descending: model.go:845-851
        cum, cutoff = 0.0, 0
        for i, idx in enumerate(order):
            cum += probs[idx]
            cutoff = i
            if cum >= top_p:
                break
        keep = np.sort(order[:cutoff + 1])
        kept = probs[keep]
        kept = kept * (1.0 / kept.sum())
        return int(keep[weighted_pick(kept, u)])
    raise ValueError(strategy)


# --------------------------------------------------------------------------- Philox4x32-10
def philox4x32(counter, key):
    """Philox4x32-10 (Salmon et al., 2011): 4 x u32 counter, 2 x u32 key -> 4 x u32."""
    M0, M1, W0, W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
    c = [int(v) & 0xFFFFFFFF for v in counter]
    k = [int(v) & 0xFFFFFFFF for v in key]
    for _ in range(10):
        p0, p1 = M0 * c[0], M1 * c[2]
        c = [(p1 >> 32) ^ c[1] ^ k[0], p1 & 0xFFFFFFFF, (p0 >> 32) ^ c[3] ^ k[1], p0 & 0xFFFFFFFF]
        c = [v & 0xFFFFFFFF for v in c]
        k = [(k[0] + W0) & 0xFFFFFFFF, (k[1] + W1) & 0xFFFFFFFF]
    return c


def uniform_for(seed, draw_index):
    """The engine's uniform in [0,1) for a sequence's `draw_index`-th sampled token: 53 bits from
    Philox4x32-10 keyed by the sequence's 64-bit seed, counter = draw index."""
    r = philox4x32([draw_index & 0xFFFFFFFF, (draw_index >> 32) & 0xFFFFFFFF, 0, 0],
                   [seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF])
    return (((r[0] << 32) | r[1]) >> 11) * (1.0 / 9007199254740992.0)


def generate(model: PlainLlama, prompt, max_tokens, strategy="greedy", temperature=1.0, top_k=50, top_p=0.9,
             repeat_penalty=0.0, repeat_last_n=64, stop_ids=(), seed=0):
    """Prefill, sample, feed back, until max_tokens sampled or a stop token (which is kept and
    counted).  model_f32.go:604-669.  Greedy ignores temperature and penalty (:610-615)."""
    ids = list(prompt)
    out = []
    for n in range(max_tokens):
        lg = model.logits(ids)[-1].numpy()
        if strategy == "greedy" or temperature == 0.0:
            t = argmax_first(lg)
        else:
            if repeat_penalty > 0:
                lg = apply_repeat_penalty(lg, ids, repeat_penalty, repeat_last_n)
            t = sample(lg, strategy, temperature, top_k, top_p, uniform_for(seed, n))
        out.append(int(t))
        ids.append(int(t))
        if t in stop_ids:
            break
    return out
