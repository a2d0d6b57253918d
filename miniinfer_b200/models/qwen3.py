"""Qwen3 dense decoder, put together from parts (architecture: miniinfer/models/fused_qwen3.py).

Per layer: RMSNorm -> attention (fused QKV without bias, per-head RMSNorm of q and k, rotary
encoding over the whole head, scale head_dim^-0.5) -> RMSNorm -> SwiGLU feed-forward, pre-norm
residual wiring; a final RMSNorm and an LM head that is the embedding table when
``tie_word_embeddings`` is set.  Every size and constant comes from the configuration.
"""

from __future__ import annotations

from ..config.model_config import Qwen3Config
from ..config.registry import register_model
from ..parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, LMHead, TokenEmbedding, make
from .spec import ModelSpec


@register_model("Qwen3ForCausalLM", Qwen3Config)
def build_qwen3(cfg: Qwen3Config) -> ModelSpec:
  H, hd = cfg.hidden_size, cfg.head_dim
  rope = make(POSITION_ENCODINGS, "rotary", "rotary", hd, cfg.rope_theta, cfg.max_position_embeddings)
  embedding = TokenEmbedding("model.embed_tokens", cfg.vocab_size, H)
  blocks = []
  for i in range(cfg.num_hidden_layers):
    p = f"model.layers.{i}"
    mixer = make(MIXERS, "attention", f"{p}.self_attn", H, cfg.num_attention_heads, cfg.num_key_value_heads, hd,
                 hd ** -0.5, cfg.rms_norm_eps, rope, cfg.window_of_layer(i))
    ffn = make(FEED_FORWARDS, "swiglu", f"{p}.mlp", H, cfg.intermediate_size)
    blocks.append(make(BLOCKS, "pre_norm", p,
                       make(NORMS, "rmsnorm", f"{p}.input_layernorm", H, cfg.rms_norm_eps), mixer,
                       make(NORMS, "rmsnorm", f"{p}.post_attention_layernorm", H, cfg.rms_norm_eps), ffn))
  final_norm = make(NORMS, "rmsnorm", "model.norm", H, cfg.rms_norm_eps)
  tied = bool(cfg.tie_word_embeddings)
  lm_head = LMHead("lm_head", cfg.vocab_size, H, tied_to=embedding if tied else None)
  aliases = {"lm_head.weight": "model.embed_tokens.weight"} if tied else {}
  return ModelSpec(config=cfg, embedding=embedding, blocks=blocks, final_norm=final_norm, lm_head=lm_head,
                   position_encodings=[rope], aliases=aliases, init_std=cfg.initializer_range)
