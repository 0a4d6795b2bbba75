"""The architectures this engine knows: for each, its configuration class and the function
that writes the model down as data (which parts every layer has, and the order of runs).
"""
from __future__ import annotations

from ..parts.registry import register_architecture
from ..parts.spec import BlockSpec, ModelSpec, PartSpec, RunStep
from .model_config import Qwen2Config


# what follows "model.layers.N." in the names of each part's tensors
QWEN2_NAMES = {"mixer_norm": "input_layernorm.", "mixer": "self_attn.",
               "feed_forward_norm": "post_attention_layernorm.", "feed_forward": "mlp."}


def qwen2_spec(config: Qwen2Config) -> ModelSpec:
    """Qwen2ForCausalLM as AIR defines it (src/model/qwen2_contract.cpp:33-139) and
    computes it (src/reference/reference_executor.cpp:325-428): every layer is a pre-norm
    block of grouped-query attention with q/k/v bias and half-split rotary encoding, and a
    SwiGLU feed-forward; a final RMSNorm; an output matrix that is either lm_head.weight or
    the embedding table."""
    e, d = config.hidden_size, config.head_dim
    position = PartSpec("rope_half", {"rotary_dim": d, "theta": config.rope_theta,
                                      "max_positions": config.max_position_embeddings})
    layers = []
    for i in range(config.num_hidden_layers):
        norm = PartSpec("rms", {"size": e, "eps": config.rms_norm_eps})
        layers.append(BlockSpec(
            kind="pre_norm", prefix=f"model.layers.{i}.",
            parts={"mixer_norm": norm,
                   "mixer": PartSpec("attention", {
                       "hidden": e, "heads": config.num_attention_heads, "kv_heads": config.num_key_value_heads,
                       "head_dim": d, "qkv_bias": config.attention_bias, "window": config.layer_window(i),
                       "position": position}),
                   "feed_forward_norm": norm,
                   "feed_forward": PartSpec("swiglu", {"hidden": e, "intermediate": config.intermediate_size})},
            names=QWEN2_NAMES))
    return ModelSpec(
        architecture=config.architecture, hidden_size=e, vocab_size=config.vocab_size,
        max_positions=config.max_position_embeddings, layers=tuple(layers),
        order=tuple(RunStep(i) for i in range(config.num_hidden_layers)),
        final_norm=PartSpec("rms", {"size": e, "eps": config.rms_norm_eps}),
        embedding_name="model.embed_tokens.weight", final_norm_prefix="model.norm.",
        output_name=None if config.tie_word_embeddings else "lm_head.weight",
        eos_token_id=config.eos_token_id)


register_architecture("Qwen2ForCausalLM", Qwen2Config, qwen2_spec)
