"""The Qwen3 dense decoder, composed from parts (the model that src/qwen.cc of lucciola runs).

Tensor names as lucciola binds them: model.embed_tokens.weight, model.norm.weight, lm_head.weight
(src/qwen.cc:77-84) and, per layer, input_layernorm, self_attn.{q,k,v,o}_proj, self_attn.{q,k}_norm,
post_attention_layernorm, mlp.{gate,up,down}_proj (src/qwen.cc:285-308)."""
from __future__ import annotations

from ..config.model_config import SLIDING_ATTENTION, Qwen3Config
from ..config.registry import register_architecture
from ..parts.attention import GQAttention
from ..parts.base import Runtime
from ..parts.block import PreNormBlock
from ..parts.embedding import OutputHead, TokenEmbedding
from ..parts.mlp import SwiGLUFeedForward
from ..parts.norm import RMSNorm
from ..parts.rope import RotaryEmbedding
from .decoder import DecoderModel, LayerCall


def build_qwen3(cfg: Qwen3Config, rt: Runtime) -> DecoderModel:
    rope = RotaryEmbedding(rt, cfg.head_dim, cfg.rope_theta)
    embedding = TokenEmbedding(rt, "model.embed_tokens.weight", cfg.vocab_size, cfg.hidden_size)
    blocks = []
    for i, kind in enumerate(cfg.layer_types):
        p = f"model.layers.{i}"
        window = cfg.sliding_window if kind == SLIDING_ATTENTION else 0
        mixer = GQAttention(rt, f"{p}.self_attn", cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads,
                            cfg.head_dim, rope, qk_norm_eps=cfg.rms_norm_eps, window=window or 0)
        ffn = SwiGLUFeedForward(rt, f"{p}.mlp", cfg.hidden_size, cfg.intermediate_size)
        blocks.append(PreNormBlock(
            mixer, ffn,
            RMSNorm(rt, f"{p}.input_layernorm.weight", cfg.hidden_size, cfg.rms_norm_eps),
            RMSNorm(rt, f"{p}.post_attention_layernorm.weight", cfg.hidden_size, cfg.rms_norm_eps),
            rt.act_dtype))
    calls = [LayerCall(i, i) for i in range(cfg.num_hidden_layers)]
    final_norm = RMSNorm(rt, "model.norm.weight", cfg.hidden_size, cfg.rms_norm_eps)
    head = OutputHead(rt, "lm_head.weight", cfg.vocab_size, cfg.hidden_size, embedding if cfg.tie_word_embeddings else None)
    return DecoderModel(rt, embedding, blocks, calls, final_norm, head, cfg.vocab_size, cfg.max_position_embeddings,
                        cfg.eos_token_ids)


register_architecture(Qwen3Config.ARCHITECTURE, Qwen3Config.from_dict, build_qwen3, replace=True)
