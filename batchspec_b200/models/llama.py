"""Llama-3 dense decoder as a model description (the architecture run by the
reference's batchspec/models/standard_model.py:15-119): every layer is
RMSNorm -> GQA attention with rotary positions -> RMSNorm -> SwiGLU, pre-norm
residual; final RMSNorm; linear head, untied or tied to the embedding.

Checkpoint names are those the reference's converter consumes
(tools/prepare_model/convert_weights.py:29-43)."""
from __future__ import annotations

from ..config.model_config import LlamaConfig
from ..parts.base import PartSpec
from .spec import ModelSpec, RunEntry, prenorm_layer


def build_llama(cfg: LlamaConfig) -> ModelSpec:
    scaling = cfg.rope_scaling.to_json_dict() if cfg.rope_scaling else None
    position = PartSpec("rope", dict(head_dim=cfg.head_dim, theta=cfg.rope_theta, scaling=scaling))
    norm = PartSpec("rmsnorm", dict(dim=cfg.hidden_size, eps=cfg.rms_norm_eps))
    mixer = PartSpec("attention", dict(dim=cfg.hidden_size, n_heads=cfg.num_attention_heads,
                                       n_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim,
                                       position=position))
    ffn = PartSpec("swiglu", dict(dim=cfg.hidden_size, intermediate=cfg.intermediate_size))
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append(prenorm_layer(norm, mixer, norm, ffn, names={
            "norm1.weight": p + "input_layernorm.weight",
            "mixer.q": p + "self_attn.q_proj.weight", "mixer.k": p + "self_attn.k_proj.weight",
            "mixer.v": p + "self_attn.v_proj.weight", "mixer.o": p + "self_attn.o_proj.weight",
            "norm2.weight": p + "post_attention_layernorm.weight",
            "ffn.gate": p + "mlp.gate_proj.weight", "ffn.up": p + "mlp.up_proj.weight",
            "ffn.down": p + "mlp.down_proj.weight",
        }))
    return ModelSpec(
        vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, layers=layers,
        order=[RunEntry(i) for i in range(cfg.num_hidden_layers)],
        final_norm=norm, embed_name="model.embed_tokens.weight",
        final_norm_names={"weight": "model.norm.weight"},
        lm_head_name=None if cfg.tie_word_embeddings else "lm_head.weight",
        ignore_suffixes=("rotary_emb.inv_freq",),
        # a tied checkpoint may store the head a second time, but only as a copy of the embedding
        must_equal={"lm_head.weight": "model.embed_tokens.weight"} if cfg.tie_word_embeddings else {},
    )
