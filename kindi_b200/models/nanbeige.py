"""The Llama-arch dense Nanbeige decoder as a ``ModelSpec``.

What the architecture is (``kindi/nanbeige.py:676-726``, one layer's kernel sequence): token embedding without
scaling; per layer pre-norm RMSNorm, grouped-query attention with rotary position encoding over the full head, no
biases, SwiGLU feed-forward; final RMSNorm; a head that is the embedding table when the embeddings are tied
(``kindi/tp.py:850-851``: "head = token_embd when output.weight is absent"). Tensor names are the safetensors
folder's (``kindi/dspine.py:249-258`` lists the layer names the reference itself reads from such files).
Every number comes from the typed configuration.
"""
from __future__ import annotations

from ..config.model_config import ModelConfig
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, default_schedule


def build_spec(cfg: ModelConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"eps": cfg.rms_norm_eps})
    position = PartSpec("rotary", {"base": cfg.rope_theta, "rotary_dim": cfg.head_dim})
    ffn = PartSpec("swiglu", {"intermediate": cfg.intermediate_size})
    layers = []
    for i in range(cfg.num_hidden_layers):
        mixer = PartSpec("attention", {
            "n_heads": cfg.num_attention_heads, "n_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "window": cfg.layer_window(i), "position": position})
        block = PartSpec("prenorm", {"norm1": norm, "mixer": mixer, "norm2": norm, "feed_forward": ffn})
        layers.append(LayerSpec(block, "model.layers.%d." % i))
    spec = ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab_size, width=cfg.hidden_size, layers=tuple(layers),
        schedule=default_schedule(cfg.num_hidden_layers), final_norm=norm,
        embedding_name="model.embed_tokens.weight", final_norm_prefix="model.norm.",
        head_name=None if cfg.tie_word_embeddings else "lm_head.weight",
        stop_token_ids=cfg.eos_token_ids, max_positions=cfg.max_position_embeddings)
    spec.validate()
    return spec


for _name in ("LlamaForCausalLM", "NanbeigeForCausalLM", "llama", "nanbeige"):
    register_architecture(_name, build_spec)
