"""LlamaConfig: every size and constant of the Llama / SmolLM2 decoder, from config.json.

Field by field this is the reference's ModelConfig (gguf.go:50-61: VocabSize, DModel, NHeads,
NKVHeads, NLayers, MaxSeqLen, DFF, NormEps, RopeFreqBase, RopeDim) under the key names that a
safetensors model folder of this family uses, with the reference's defaults (gguf.go:587-599:
kv heads = heads, eps 1e-5, theta 10000, rotary width = head width). No size stands anywhere else.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field

from .base import ConfigError, KeyReader

ROPE_PAIRINGS = ("half", "interleaved")
ROPE_SCALING_TYPES = ("llama3", "linear", "default")


@dataclass(frozen=True)
class RopeScaling:
    """Rescaling of the rotary frequency table (absent in the reference, present in the family's
    config.json as `rope_scaling`)."""
    rope_type: str
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 8192


@dataclass(frozen=True)
class LlamaConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: RopeScaling | None
    rotary_dim: int
    rope_pairing: str
    max_position_embeddings: int
    tie_word_embeddings: bool
    sliding_window: int | None
    eos_token_ids: tuple[int, ...]
    bos_token_id: int | None
    torch_dtype: str | None
    unknown_keys: tuple[str, ...] = field(default=(), compare=False)

    # ------------------------------------------------------------------ derived
    @property
    def q_width(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def to_json_dict(self) -> dict:
        """The config.json that reads back as this record."""
        d = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "hidden_act": "silu",
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": dataclasses.asdict(self.rope_scaling) if self.rope_scaling else None,
            "partial_rotary_factor": self.rotary_dim / self.head_dim,
            "rope_pairing": self.rope_pairing,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "sliding_window": self.sliding_window,
            "attention_bias": False,
            "mlp_bias": False,
            "eos_token_id": list(self.eos_token_ids) if len(self.eos_token_ids) != 1 else self.eos_token_ids[0],
            "bos_token_id": self.bos_token_id,
            "torch_dtype": self.torch_dtype,
        }
        if not self.eos_token_ids:
            d["eos_token_id"] = None
        return d

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: dict, where: str = "config.json") -> "LlamaConfig":
        r = KeyReader(raw, where)
        archs = r.any("architectures")
        if not (isinstance(archs, list) and archs and isinstance(archs[0], str)):
            raise ConfigError(f"{where}: 'architectures' must be a list that names the model class")
        r.any("model_type")

        vocab = r.integer("vocab_size", minimum=1)
        hidden = r.integer("hidden_size", minimum=1)
        layers = r.integer("num_hidden_layers", minimum=1)
        heads = r.integer("num_attention_heads", minimum=1)
        kv_heads = r.integer("num_key_value_heads", default=heads, minimum=1)   # gguf.go:589-590
        if heads % kv_heads != 0:
            raise ConfigError(f"{where}: num_attention_heads ({heads}) must be a multiple of "
                              f"num_key_value_heads ({kv_heads})")
        head_dim = r.integer("head_dim", default=None, minimum=1)
        if head_dim is None:
            if hidden % heads != 0:
                raise ConfigError(f"{where}: hidden_size ({hidden}) is no multiple of num_attention_heads "
                                  f"({heads}) and no head_dim is given")
            head_dim = hidden // heads                                          # model_f32.go:249
        inter = r.integer("intermediate_size", minimum=1)
        eps = r.number("rms_norm_eps", default=1e-5, positive=True)             # gguf.go:594
        theta = r.number("rope_theta", default=10000.0, positive=True)          # gguf.go:595
        max_pos = r.integer("max_position_embeddings", minimum=1)
        tie = r.boolean("tie_word_embeddings", default=False)

        act = r.string("hidden_act", default="silu")
        if act != "silu":
            raise ConfigError(f"{where}: hidden_act {act!r} is not supported (this decoder's feed-forward is "
                              f"SiLU-gated)")
        for key in ("attention_bias", "mlp_bias"):
            if r.boolean(key, default=False):
                raise ConfigError(f"{where}: {key}=true is not supported (the Llama/SmolLM2 projections have no bias)")
        window = r.integer("sliding_window", default=None, minimum=1)

        factor = r.number("partial_rotary_factor", default=1.0, positive=True)  # gguf.go:596-599 (rope dim)
        rotary_dim = int(round(head_dim * factor))
        if rotary_dim < 2 or rotary_dim > head_dim or rotary_dim % 2:
            raise ConfigError(f"{where}: partial_rotary_factor {factor} gives a rotary width of {rotary_dim}; it must "
                              f"be even and between 2 and head_dim ({head_dim})")
        pairing = r.string("rope_pairing", default="half", choices=ROPE_PAIRINGS)

        scaling = None
        rs = r.any("rope_scaling")
        if rs is not None:
            sr = KeyReader(rs, where + ":rope_scaling")
            kind = sr.string("rope_type", default=None) or sr.string("type", default=None)
            if kind is None:
                raise ConfigError(f"{where}: rope_scaling needs a 'rope_type'")
            if kind not in ROPE_SCALING_TYPES:
                raise ConfigError(f"{where}: rope_scaling type {kind!r} is not supported; supported: "
                                  f"{', '.join(ROPE_SCALING_TYPES)}")
            if kind == "llama3":
                scaling = RopeScaling(
                    "llama3", sr.number("factor", positive=True),
                    sr.number("low_freq_factor", positive=True), sr.number("high_freq_factor", positive=True),
                    sr.integer("original_max_position_embeddings", minimum=1))
                if scaling.high_freq_factor <= scaling.low_freq_factor:
                    raise ConfigError(f"{where}: rope_scaling high_freq_factor must exceed low_freq_factor")
            elif kind == "linear":
                scaling = RopeScaling("linear", sr.number("factor", positive=True))

        eos = r.any("eos_token_id")
        if eos is None:
            eos_ids: tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, list) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError(f"{where}: eos_token_id must be an integer or a list of integers, found {eos!r}")
        for e in eos_ids:
            if not 0 <= e < vocab:
                raise ConfigError(f"{where}: eos_token_id {e} is outside the vocabulary (0..{vocab - 1})")
        bos = r.integer("bos_token_id", default=None)
        dtype = r.string("torch_dtype", default=None) or r.string("dtype", default=None)

        unknown = tuple(sorted(k for k in raw if k not in r.seen))
        return cls(archs[0], vocab, hidden, layers, heads, kv_heads, head_dim, inter, eps, theta, scaling,
                   rotary_dim, pairing, max_pos, tie, window, eos_ids, bos, dtype, unknown)
