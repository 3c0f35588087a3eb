"""Layout of the Llama / SmolLM2 decoder: which parts, with which numbers and tensor names.

Per layer: RMSNorm -> grouped-query attention with rotary positions -> residual -> RMSNorm ->
SiLU-gated feed-forward -> residual; then a final RMSNorm and the output head, tied to the
embedding when the configuration says so (model_f32.go:133-293, :382-527). Tensor names are those
of the family's safetensors checkpoints; the reference's own (GGUF) names map onto them one to one
(gguf.go:254-302: token_embd, blk.N.attn_{q,k,v,output}, blk.N.ffn_{gate,up,down}, blk.N.attn_norm,
blk.N.ffn_norm, output_norm, output).
"""
from __future__ import annotations

from ..config.llama import LlamaConfig
from ..config.registry import register_architecture
from ..engine.layout import ModelLayout, sequential_schedule
from ..parts.base import PartSpec
from ..parts.block import pre_norm_layer
from ..parts.embedding import linear_head, token_embedding


def llama_layout(cfg: LlamaConfig) -> ModelLayout:
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        position = PartSpec("rotary", dict(head_dim=cfg.head_dim, rotary_dim=cfg.rotary_dim, theta=cfg.rope_theta,
                                           scaling=cfg.rope_scaling, pairing=cfg.rope_pairing))
        mixer = PartSpec("attention", dict(
            hidden=cfg.hidden_size, n_heads=cfg.num_attention_heads, n_kv_heads=cfg.num_key_value_heads,
            head_dim=cfg.head_dim, position=position, window=cfg.sliding_window,
            q_name=p + "self_attn.q_proj.weight", k_name=p + "self_attn.k_proj.weight",
            v_name=p + "self_attn.v_proj.weight", o_name=p + "self_attn.o_proj.weight"))
        ffn = PartSpec("swiglu", dict(hidden=cfg.hidden_size, intermediate=cfg.intermediate_size,
                                      gate_name=p + "mlp.gate_proj.weight", up_name=p + "mlp.up_proj.weight",
                                      down_name=p + "mlp.down_proj.weight"))
        norm1 = PartSpec("rmsnorm", dict(width=cfg.hidden_size, eps=cfg.rms_norm_eps,
                                         weight_name=p + "input_layernorm.weight"))
        norm2 = PartSpec("rmsnorm", dict(width=cfg.hidden_size, eps=cfg.rms_norm_eps,
                                         weight_name=p + "post_attention_layernorm.weight"))
        layers.append(pre_norm_layer(mixer, ffn, norm1, norm2))
    return ModelLayout(
        vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, max_positions=cfg.max_position_embeddings,
        embedding=token_embedding(cfg.vocab_size, cfg.hidden_size, "model.embed_tokens.weight"), layers=tuple(layers),
        schedule=sequential_schedule(cfg.num_hidden_layers),
        final_norm=PartSpec("rmsnorm", dict(width=cfg.hidden_size, eps=cfg.rms_norm_eps, weight_name="model.norm.weight")),
        head=linear_head(cfg.vocab_size, cfg.hidden_size, "model.embed_tokens.weight", tied=True) if cfg.tie_word_embeddings
        else linear_head(cfg.vocab_size, cfg.hidden_size, "lm_head.weight"),
        stop_ids=cfg.eos_token_ids,
        ignorable_tensors=("lm_head.weight",) if cfg.tie_word_embeddings else ())


register_architecture("LlamaForCausalLM", LlamaConfig, llama_layout)
