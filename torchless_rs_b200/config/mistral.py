"""Typed configuration of the Mistral dense decoder, read from its config.json keys.

Keys and defaults follow the reference where it reads them
(src/loader/formats/safetensors.rs:701-765, src/loader/mod.rs:35-81,
src/loader/formats/gguf.rs:1194-1202): hidden_size, intermediate_size,
num_hidden_layers, num_attention_heads, vocab_size are required;
num_key_value_heads defaults to the number of heads; rope_theta to 10000;
rms_norm_eps (or layer_norm_eps) to 1e-5; max_position_embeddings to 4096.
The reference parses sliding_window (src/loader/parameters.rs:800) but its
Mistral attention never applies it and takes head_dim = hidden/heads
(src/model/mod.rs:143); here sliding_window is applied and head_dim may be
given on its own.
"""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Optional, Tuple

from .errors import ConfigError
from .reader import KeyReader
from .spec import LayerSpec, ModelSpec, PartSpec

HEAD_DIM_STEP = 16

# The names a Mistral layer's tensors carry under `model.layers.<i>`
# (src/model/mod.rs:395-414, src/model/architecture.rs:114-130).
LAYER_TENSOR_NAMES = {"mixer_norm": "input_layernorm", "mixer": "self_attn",
                      "feed_forward_norm": "post_attention_layernorm", "feed_forward": "mlp"}


@dataclass(frozen=True)
class MistralConfig:
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rope_theta: float
    rms_norm_eps: float
    sliding_window: Optional[int]
    hidden_act: str = "silu"
    tie_word_embeddings: bool = False
    bos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    # one entry per layer, "sliding_attention" or "full_attention"; empty = every
    # layer uses sliding_window when it is set
    layer_types: Tuple[str, ...] = ()
    torch_dtype: str = "bfloat16"
    architecture: str = "MistralForCausalLM"
    model_type: str = "mistral"

    @classmethod
    def from_dict(cls, data: dict, where: str = "config.json") -> "MistralConfig":
        r = KeyReader(data, where)
        hidden = r.integer("hidden_size")
        heads = r.integer("num_attention_heads")
        kv_heads = r.integer("num_key_value_heads", heads)
        head_dim = r.integer("head_dim", None)
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(
                    f"{where}: hidden_size {hidden} is not a multiple of num_attention_heads "
                    f"{heads} and no head_dim is given")
            head_dim = hidden // heads
        eps = r.number("rms_norm_eps", None)
        if eps is None:
            eps = r.number("layer_norm_eps", 1e-5)
        window = r.integer("sliding_window", None)
        eos = data.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, list) and all(isinstance(t, int) for t in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError(f"{where}: key 'eos_token_id' must be an integer or a list of integers")
        archs = r.list_of("architectures", None)
        cfg = cls(
            hidden_size=hidden,
            intermediate_size=r.integer("intermediate_size"),
            num_hidden_layers=r.integer("num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            vocab_size=r.integer("vocab_size"),
            max_position_embeddings=r.integer("max_position_embeddings", 4096),
            rope_theta=r.number("rope_theta", 10000.0),
            rms_norm_eps=eps,
            sliding_window=window,
            hidden_act=r.string("hidden_act", "silu"),
            tie_word_embeddings=r.boolean("tie_word_embeddings", False),
            bos_token_id=r.integer("bos_token_id", None, minimum=0),
            eos_token_ids=eos_ids,
            layer_types=tuple(r.list_of("layer_types", ())),
            torch_dtype=r.string("torch_dtype", r.string("dtype", "bfloat16")),
            architecture=(archs[0] if archs else "MistralForCausalLM"),
            model_type=r.string("model_type", "mistral"),
        )
        cfg.validate(where)
        return cfg

    def validate(self, where: str = "config") -> None:
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"{where}: num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % HEAD_DIM_STEP or not 16 <= self.head_dim <= 256:
            raise ConfigError(
                f"{where}: head_dim {self.head_dim} is not supported: the attention kernels take "
                f"head sizes from 16 to 256 in steps of {HEAD_DIM_STEP}")
        if self.tie_word_embeddings:
            # the reference loads lm_head.weight as a tensor of its own (src/model/mod.rs:369) and its
            # Mistral traits say tie_embeddings = false (src/model/architecture.rs:491)
            raise ConfigError(f"{where}: tie_word_embeddings is true, but this architecture's head is a "
                              f"tensor of its own (lm_head.weight)")
        if self.hidden_act != "silu":
            raise ConfigError(f"{where}: hidden_act '{self.hidden_act}' is not supported (only 'silu')")
        for t in self.eos_token_ids:
            if not 0 <= t < self.vocab_size:
                raise ConfigError(f"{where}: eos_token_id {t} lies outside the vocabulary")
        if self.layer_types:
            if len(self.layer_types) != self.num_hidden_layers:
                raise ConfigError(
                    f"{where}: layer_types has {len(self.layer_types)} entries for "
                    f"{self.num_hidden_layers} layers")
            for t in self.layer_types:
                if t not in ("sliding_attention", "full_attention"):
                    raise ConfigError(f"{where}: layer_types entry '{t}' is not known")
                if t == "sliding_attention" and not self.sliding_window:
                    raise ConfigError(f"{where}: layer_types asks for a window but sliding_window is null")

    def to_dict(self) -> dict:
        """The config.json dictionary that reads back to this configuration."""
        d = asdict(self)
        d["architectures"] = [d.pop("architecture")]
        eos = d.pop("eos_token_ids")
        d["eos_token_id"] = None if not eos else (eos[0] if len(eos) == 1 else list(eos))
        d["layer_types"] = list(d["layer_types"])
        if not d["layer_types"]:
            del d["layer_types"]
        return d

    def layer_window(self, layer: int) -> Optional[int]:
        if not self.sliding_window:
            return None
        if self.layer_types and self.layer_types[layer] == "full_attention":
            return None
        return self.sliding_window

    def model_spec(self) -> ModelSpec:
        """The arrangement of the reference's Mistral (src/model/mod.rs:391-424,
        src/model/architecture.rs:487-502): pre-norm blocks of grouped-query
        attention with rotary positions and a SwiGLU feed-forward, RMSNorm
        everywhere, no biases."""
        norm = PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.rms_norm_eps})
        rope = PartSpec("rope_half_split", {"head_dim": self.head_dim, "theta": self.rope_theta})
        ffn = PartSpec("swiglu", {"hidden_size": self.hidden_size,
                                  "intermediate_size": self.intermediate_size})
        layers = []
        for i in range(self.num_hidden_layers):
            mixer = PartSpec("attention", {
                "hidden_size": self.hidden_size,
                "num_heads": self.num_attention_heads,
                "num_kv_heads": self.num_key_value_heads,
                "head_dim": self.head_dim,
                "window": self.layer_window(i),
            })
            layers.append(LayerSpec(
                prefix=f"model.layers.{i}", block=PartSpec("prenorm"), mixer=mixer,
                feed_forward=ffn, norms={"mixer_norm": norm, "feed_forward_norm": norm},
                names=LAYER_TENSOR_NAMES, position=rope))
        spec = ModelSpec(
            hidden_size=self.hidden_size, vocab_size=self.vocab_size,
            embedding_name="model.embed_tokens.weight", head_name="lm_head.weight",
            tie_head_to_embedding=self.tie_word_embeddings,
            final_norm=norm, final_norm_prefix="model.norm",
            layers=tuple(layers), order=tuple(range(self.num_hidden_layers)),
            stop_token_ids=self.eos_token_ids)
        spec.validate()
        return spec
