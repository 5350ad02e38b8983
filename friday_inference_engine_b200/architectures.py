"""The architectures this library ships: how each turns its configuration into parts.

Qwen2ForCausalLM, the Qwen2.5 dense decoder: token table; per layer a pre-norm block
of grouped-query attention (biased q/k/v, rotary NeoX encoding, optional window) and a
SwiGLU feed-forward, RMSNorm before each; final RMSNorm; head (own matrix, or the token
table when tie_word_embeddings).  Tensor names are the Hugging Face ones; the
reference's GGUF names map to them one to one (token_embd -> model.embed_tokens,
blk.L.attn_norm -> model.layers.L.input_layernorm, attn_q/k/v -> self_attn.q/k/v_proj,
attn_output -> self_attn.o_proj, ffn_norm -> post_attention_layernorm,
ffn_gate/up/down -> mlp.gate/up/down_proj, output_norm -> model.norm, output ->
lm_head; transformer.cpp:299-362, 1000-1005).
"""
from .config.qwen2 import ARCHITECTURE as QWEN2, Qwen2Config
from .parts.spec import LayerCall, ModelSpec, PartSpec
from .registry import register_architecture


def qwen2_spec(cfg: Qwen2Config) -> ModelSpec:
    layers = []
    for l in range(cfg.num_hidden_layers):
        position = PartSpec("rotary_neox", {"theta": cfg.rope_theta, "head_dim": cfg.head_dim})
        mixer = PartSpec("gqa_attention", {
            "n_heads": cfg.num_attention_heads, "n_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "position": position, "qkv_bias": True, "out_bias": False, "window": cfg.window_of(l),
        }, prefix="self_attn.")
        ffn = PartSpec("swiglu", {"inner": cfg.intermediate_size}, prefix="mlp.")
        norm1 = PartSpec("rmsnorm", {"eps": cfg.rms_norm_eps}, prefix="input_layernorm.")
        norm2 = PartSpec("rmsnorm", {"eps": cfg.rms_norm_eps}, prefix="post_attention_layernorm.")
        layers.append(PartSpec("prenorm", {"norm1": norm1, "mixer": mixer, "norm2": norm2, "feed_forward": ffn},
                               prefix="model.layers.%d." % l))
    return ModelSpec(
        architecture=cfg.architecture,
        vocab_size=cfg.vocab_size,
        width=cfg.hidden_size,
        max_positions=cfg.max_position_embeddings,
        embedding="model.embed_tokens.weight",
        layers=layers,
        program=[LayerCall(layer=l, cache=l) for l in range(cfg.num_hidden_layers)],
        final_norm=PartSpec("rmsnorm", {"eps": cfg.rms_norm_eps}, prefix="model.norm."),
        head=None if cfg.tie_word_embeddings else "lm_head.weight",
    )


register_architecture(QWEN2, Qwen2Config, qwen2_spec)
