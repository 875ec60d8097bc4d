"""The Llama-arch dense Nanbeige decoder: its config.json keys, its typed configuration and its ``ModelSpec``.

What the architecture is (``kindi/nanbeige.py:676-726``, one layer's kernel sequence): token embedding without
scaling; per layer pre-norm RMSNorm, grouped-query attention with rotary position encoding over the full head, no
biases, SwiGLU feed-forward; final RMSNorm; a head that is the embedding table when the embeddings are tied
(``kindi/tp.py:850-851``: "head = token_embd when output.weight is absent"). Tensor names are the safetensors
folder's (``kindi/dspine.py:249-258`` lists the layer names the reference itself reads from such files).

The keys are the ones a Llama-style ``config.json`` carries; they are the same ones the reference reads where it
reads such a file (``kindi/dspine.py:220-227``: hidden_size, num_attention_heads, num_key_value_heads, head_dim,
num_hidden_layers, intermediate_size, rms_norm_eps, rope_theta or rope_parameters.rope_theta), plus what its GGUF
path takes from the file's metadata (``kindi/nanbeige.py:249-259``: block count, widths, head counts, norm epsilon,
rope base with default 10000.0, context length, vocabulary size). Everything that is particular to this
architecture - which keys are required, which values it refuses - lives in this file; every number of the model
comes from the typed configuration.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..config.model_config import ConfigError, ConfigReader, architecture_name
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, default_schedule


@dataclass(frozen=True)
class LlamaConfig:
    """The Llama-arch dense decoder's hyper-parameters (Nanbeige is this architecture).

    ``head_dim`` defaults to hidden_size // num_attention_heads as in ``kindi/nanbeige.py:257``; ``rope_theta``
    defaults to 10000.0 as in ``kindi/nanbeige.py:256``; ``rms_norm_eps`` has no default, as in
    ``kindi/nanbeige.py:255``.
    """

    architecture: str
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool = False
    max_position_embeddings: Optional[int] = None
    sliding_window: Optional[int] = None
    layer_types: Optional[Tuple[str, ...]] = None     # "full_attention" | "sliding_attention" per layer
    bos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    torch_dtype: str = "bfloat16"

    @property
    def gqa_ratio(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def layer_window(self, layer: int) -> Optional[int]:
        """the attention window of a layer (None: all keys)"""
        if self.sliding_window is None:
            return None
        if self.layer_types is None:
            return self.sliding_window
        return self.sliding_window if self.layer_types[layer] == "sliding_attention" else None

    # ------------------------------------------------------------------ reading
    @staticmethod
    def from_dict(d: Mapping[str, Any]) -> "LlamaConfig":
        r = ConfigReader(d)
        r.ignore("architectures", "model_type")
        arch = architecture_name(d)
        hidden = r.integer("hidden_size")
        heads = r.integer("num_attention_heads")
        if heads <= 0:
            raise ConfigError("config.json: num_attention_heads must be positive, found %d" % heads)
        kv = r.integer("num_key_value_heads", heads)
        head_dim = r.integer("head_dim", None)
        if head_dim is None:
            if hidden % heads:
                raise ConfigError("config.json: hidden_size %d is not a multiple of num_attention_heads %d and "
                                  "head_dim is not given" % (hidden, heads))
            head_dim = hidden // heads
        theta = r.number("rope_theta", None)
        rp = r.any("rope_parameters")
        if rp is not None and not isinstance(rp, Mapping):
            raise ConfigError("config.json: rope_parameters must be an object, found %r" % (rp,))
        if theta is None:
            theta = ConfigReader(rp, "config.json: rope_parameters").number("rope_theta", 10000.0) if rp else 10000.0
        scaling = r.any("rope_scaling")
        if scaling is None and rp is not None and rp.get("rope_type", "default") not in ("default", None):
            scaling = rp
        if scaling is not None and not (isinstance(scaling, Mapping)
                                        and scaling.get("rope_type", scaling.get("type")) in ("default", None)):
            raise ConfigError("config.json: rope_scaling %r is not supported by this architecture's position "
                              "encoding (plain rotary only)" % (scaling,))
        # keys of the wider Llama family that change what a forward pass computes: accepted only when they say "off"
        r.neutral("attention_bias", (False,), "the architecture has no biases")
        r.neutral("mlp_bias", (False,), "the architecture has no biases")
        r.neutral("hidden_act", ("silu",), "the feed-forward is SwiGLU ('silu')")
        r.neutral("partial_rotary_factor", (1, 1.0), "the rotation covers the whole head")
        r.neutral("attention_multiplier", (), "scores are scaled by 1 / sqrt(head_dim)")
        r.neutral("query_pre_attn_scalar", (), "scores are scaled by 1 / sqrt(head_dim)")
        r.neutral("logits_scaling", (1, 1.0), "logits are not scaled")
        r.neutral("logit_scale", (1, 1.0), "logits are not scaled")
        r.neutral("residual_multiplier", (1, 1.0), "branches are added unscaled")
        r.neutral("embedding_multiplier", (1, 1.0), "embedding rows are used as stored")
        r.neutral("final_logit_softcapping", (), "logits are not capped")
        r.neutral("attn_logit_softcapping", (), "scores are not capped")
        r.neutral("qk_norm", (False,), "queries and keys are not normalised")
        r.neutral("use_qk_norm", (False,), "queries and keys are not normalised")
        r.neutral("num_local_experts", (0, 1), "the feed-forward is dense")
        r.neutral("num_experts", (0, 1), "the feed-forward is dense")
        r.neutral("quantization_config", (), "weights are bfloat16 or float32 tensors")
        window = r.integer("sliding_window", None)
        if window is not None and window <= 0:
            raise ConfigError("config.json: sliding_window must be positive, found %d" % window)
        if not r.boolean("use_sliding_window", True):
            window = None                       # the folder carries a window and says that it is not in use
        n_layers = r.integer("num_hidden_layers")
        lt = r.any("layer_types")
        if lt is not None:
            if (not isinstance(lt, (list, tuple)) or len(lt) != n_layers
                    or any(t not in ("full_attention", "sliding_attention") for t in lt)):
                raise ConfigError("config.json: layer_types must list 'full_attention' or 'sliding_attention' for "
                                  "each of the %d layers, found %r" % (n_layers, lt))
            if "sliding_attention" in lt and window is None:
                raise ConfigError("config.json: layer_types names sliding_attention but sliding_window is missing")
            lt = tuple(lt)
        cfg = LlamaConfig(
            architecture=arch,
            vocab_size=r.integer("vocab_size"),
            hidden_size=hidden,
            intermediate_size=r.integer("intermediate_size"),
            num_hidden_layers=n_layers,
            num_attention_heads=heads,
            num_key_value_heads=kv,
            head_dim=head_dim,
            rms_norm_eps=r.number("rms_norm_eps"),
            rope_theta=theta,
            tie_word_embeddings=r.boolean("tie_word_embeddings", False),
            max_position_embeddings=r.integer("max_position_embeddings", None),
            sliding_window=window,
            layer_types=lt,
            bos_token_id=r.integer("bos_token_id", None),
            eos_token_ids=r.id_list("eos_token_id"),
            torch_dtype=r.string("torch_dtype", None) or r.string("dtype", "bfloat16"),
        )
        r.ignore("dtype")
        r.finish()
        cfg.validate()
        return cfg

    # ------------------------------------------------------------------ checks
    def validate(self) -> None:
        for k in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                  "num_key_value_heads", "head_dim"):
            if getattr(self, k) <= 0:
                raise ConfigError("config.json: %s must be positive, found %d" % (k, getattr(self, k)))
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError("config.json: num_attention_heads %d is not a multiple of num_key_value_heads %d"
                              % (self.num_attention_heads, self.num_key_value_heads))
        if self.head_dim % 2:
            raise ConfigError("config.json: head_dim %d must be even (rotary pairs)" % self.head_dim)
        if not (self.rms_norm_eps > 0.0):
            raise ConfigError("config.json: rms_norm_eps must be positive, found %r" % self.rms_norm_eps)
        if not (self.rope_theta > 0.0):
            raise ConfigError("config.json: rope_theta must be positive, found %r" % self.rope_theta)
        if self.max_position_embeddings is not None and self.max_position_embeddings <= 0:
            raise ConfigError("config.json: max_position_embeddings must be positive, found %d"
                              % self.max_position_embeddings)

    def to_dict(self) -> dict:
        """the config.json that reads back as this configuration"""
        d = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "attention_bias": False,
            "mlp_bias": False,
            "torch_dtype": self.torch_dtype,
        }
        if self.max_position_embeddings is not None:
            d["max_position_embeddings"] = self.max_position_embeddings
        if self.sliding_window is not None:
            d["sliding_window"] = self.sliding_window
        if self.layer_types is not None:
            d["layer_types"] = list(self.layer_types)
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.eos_token_ids:
            d["eos_token_id"] = self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else list(self.eos_token_ids)
        return d


def read_config(raw: Mapping[str, Any]) -> LlamaConfig:
    return LlamaConfig.from_dict(raw)


EMBEDDING = "model.embed_tokens.weight"
HEAD = "lm_head.weight"


def build_spec(cfg: LlamaConfig) -> ModelSpec:
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
    tied = cfg.tie_word_embeddings
    spec = ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab_size, width=cfg.hidden_size, layers=tuple(layers),
        schedule=default_schedule(cfg.num_hidden_layers), final_norm=norm, final_norm_prefix="model.norm.",
        embedding=PartSpec("table", {"name": EMBEDDING, "vocab": cfg.vocab_size}),
        head=PartSpec("linear", {"name": HEAD, "tied_to": EMBEDDING if tied else None, "vocab": cfg.vocab_size}),
        stop_token_ids=cfg.eos_token_ids, max_positions=cfg.max_position_embeddings,
        # older exports store each layer's rotary frequencies as a buffer; they are recomputed from rope_theta here
        may_ignore=("*.rotary_emb.inv_freq",),
        # a tied model may still store its head: accepted when it is the embedding table, bit for bit
        copies={HEAD: EMBEDDING} if tied else {})
    spec.validate()
    return spec


for _name in ("LlamaForCausalLM", "NanbeigeForCausalLM", "llama", "nanbeige"):
    register_architecture(_name, build_spec, read_config)
