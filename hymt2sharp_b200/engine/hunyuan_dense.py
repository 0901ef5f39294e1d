"""Hunyuan dense ("HunYuanDenseV1ForCausalLM"): from its configuration to a ModelSpec.

Every layer is a pre-norm block of grouped-query attention (rotate-half rotary
encoding with the dynamic-NTK base, per-head q/k RMSNorm after the rotation when
use_qk_norm is set) and a SwiGLU feed-forward
(src/HyMT2Sharp/HunyuanDenseModel.Prefill.cs:14-89), between a token embedding and
a final RMSNorm with a tied or separate output head
(src/HyMT2Sharp/HunyuanDenseModel.cs:390-419).  Tensor names are those of the
architecture's checkpoints.
"""
from __future__ import annotations

from ..config.hunyuan_dense import ARCHITECTURE, HunyuanDenseConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from .spec import ModelSpec


def build_spec(cfg: HunyuanDenseConfig) -> ModelSpec:
    layers = []
    for l in range(cfg.num_hidden_layers):
        p = f"model.layers.{l}."
        position = PartSpec("neox_rope", dict(head_dim=cfg.head_dim, rope_dim=cfg.rope_dim, base=cfg.rope_base))
        mixer = PartSpec("gqa_attention", dict(
            hidden=cfg.hidden_size, heads=cfg.num_attention_heads, kv_heads=cfg.num_key_value_heads,
            head_dim=cfg.head_dim, eps=cfg.rms_norm_eps, qk_norm=cfg.use_qk_norm, position=position,
            window=cfg.sliding_window,
            q_proj=p + "self_attn.q_proj.weight", k_proj=p + "self_attn.k_proj.weight",
            v_proj=p + "self_attn.v_proj.weight", o_proj=p + "self_attn.o_proj.weight",
            q_norm=p + "self_attn.query_layernorm.weight", k_norm=p + "self_attn.key_layernorm.weight"))
        ffn = PartSpec("swiglu", dict(hidden=cfg.hidden_size, intermediate=cfg.intermediate_size,
                                      gate_proj=p + "mlp.gate_proj.weight", up_proj=p + "mlp.up_proj.weight",
                                      down_proj=p + "mlp.down_proj.weight"))
        norm = lambda name: PartSpec("rmsnorm", dict(dim=cfg.hidden_size, eps=cfg.rms_norm_eps, weight=p + name))
        layers.append(PartSpec("pre_norm", dict(norm1=norm("input_layernorm.weight"), mixer=mixer,
                                                norm2=norm("post_attention_layernorm.weight"), feed_forward=ffn)))
    return ModelSpec(
        vocab=cfg.vocab_size, hidden=cfg.hidden_size, embedding="model.embed_tokens.weight", layers=layers,
        final_norm=PartSpec("rmsnorm", dict(dim=cfg.hidden_size, eps=cfg.rms_norm_eps, weight="model.norm.weight")),
        head=None if cfg.tie_word_embeddings else "lm_head.weight", max_positions=cfg.max_position_embeddings,
        head_copy="lm_head.weight" if cfg.tie_word_embeddings else None,
        ignorable_tensors=[r".*\.rotary_emb\.inv_freq"])


def tensor_shapes(cfg: HunyuanDenseConfig):
    from .model import DecoderModel
    return DecoderModel(build_spec(cfg)).tensors()


register_architecture(ARCHITECTURE, HunyuanDenseConfig, build_spec, tensor_shapes)
