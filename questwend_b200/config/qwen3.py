"""Configuration of the Qwen3 dense decoder, read from its own config.json keys.

Which key means what follows the reference's ``load_hparams``
(core/model.cpp:504-567): layers, width, feed-forward width, heads, key/value
heads (default: as many as heads, :520), head size (default width / heads,
:526-527), RoPE base (:522), one epsilon for every norm (:523), the trained
context length (:521) and the vocabulary size (:561-566).  The reference has
no path for an attention bias, a RoPE scaling or a sliding window
(core/runtime.cpp:300-301, 1039-1041), so a configuration that asks for one is
refused here instead of being run wrongly.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .base import ConfigError, ConfigReader, ModelConfig
from ..kernels.limits import head_dim_refusal

ARCHITECTURE = "Qwen3ForCausalLM"


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    num_hidden_layers: int
    hidden_size: int
    intermediate_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    rope_theta: float
    rms_norm_eps: float
    tie_word_embeddings: bool | None          # None: decided by the presence of lm_head.weight
    max_position_embeddings: int | None
    eos_token_ids: tuple = field(default_factory=tuple)
    bos_token_id: int | None = None
    torch_dtype: str | None = None

    architecture = ARCHITECTURE

    @classmethod
    def from_reader(cls, r: ConfigReader) -> "Qwen3Config":
        w = r.where
        model_type = r.string("model_type", None)
        if model_type is not None and model_type != "qwen3":
            raise ConfigError(f"{w}: key 'model_type' is {model_type!r}, expected 'qwen3'")
        n_layers = r.integer("num_hidden_layers", minimum=1)
        hidden = r.integer("hidden_size", minimum=1)
        inter = r.integer("intermediate_size", minimum=1)
        heads = r.integer("num_attention_heads", minimum=1)
        kv_heads = r.integer("num_key_value_heads", heads, minimum=1)
        if r.has("head_dim"):
            head_dim = r.integer("head_dim", minimum=1)
        else:
            if hidden % heads:
                raise ConfigError(f"{w}: key 'head_dim' is missing and 'hidden_size' ({hidden}) is "
                                  f"not a multiple of 'num_attention_heads' ({heads})")
            head_dim = hidden // heads
        vocab = r.integer("vocab_size", minimum=1)
        eps = r.number("rms_norm_eps", positive=True)

        # RoPE base: a top-level key, or inside 'rope_parameters' in newer files.
        rope_params = r.mapping("rope_parameters", None)
        if r.has("rope_theta"):
            theta = r.number("rope_theta", positive=True)
        elif rope_params is not None and rope_params.get("rope_theta") is not None:
            theta = float(rope_params["rope_theta"])
            if not theta > 0:
                raise ConfigError(f"{w}: key 'rope_parameters.rope_theta' must be > 0, got {theta}")
        else:
            raise ConfigError(f"{w}: required key 'rope_theta' is missing")
        for key, params in (("rope_scaling", r.mapping("rope_scaling", None)),
                            ("rope_parameters", rope_params)):
            if params is None:
                continue
            kind = params.get("rope_type", params.get("type", "default"))
            if kind not in (None, "default"):
                raise ConfigError(f"{w}: key '{key}' asks for RoPE scaling '{kind}'; this "
                                  f"architecture rotates with the plain base only")
        if r.boolean("attention_bias", False):
            raise ConfigError(f"{w}: key 'attention_bias' is true; this architecture has no "
                              f"attention bias tensors")
        if r.boolean("use_sliding_window", False):
            raise ConfigError(f"{w}: key 'use_sliding_window' is true; this architecture "
                              f"attends to all earlier keys")
        if r.has("layer_types"):
            lt = r.data["layer_types"]
            if not isinstance(lt, list) or any(t != "full_attention" for t in lt):
                raise ConfigError(f"{w}: key 'layer_types' must name 'full_attention' only, got {lt!r}")
            if len(lt) != n_layers:
                raise ConfigError(f"{w}: key 'layer_types' has {len(lt)} entries for "
                                  f"{n_layers} layers")
        act = r.string("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"{w}: key 'hidden_act' is {act!r}; the feed-forward here is SiLU-gated")
        if heads % kv_heads:
            raise ConfigError(f"{w}: key 'num_attention_heads' ({heads}) must be a multiple of "
                              f"'num_key_value_heads' ({kv_heads})")
        if head_dim % 2:
            raise ConfigError(f"{w}: key 'head_dim' ({head_dim}) must be even: RoPE rotates pairs")
        refusal = head_dim_refusal(head_dim)
        if refusal:
            which = "key 'head_dim'" if r.has("head_dim") else "'hidden_size' / 'num_attention_heads' (no key 'head_dim')"
            raise ConfigError(f"{w}: {which} gives a head size of {head_dim}: {refusal}")
        tie = r.boolean("tie_word_embeddings", None)
        max_pos = r.integer("max_position_embeddings", None, minimum=1)
        eos = tuple(r.int_list("eos_token_id", []))
        bos = r.integer("bos_token_id", None)
        dtype = r.string("torch_dtype", None) or r.string("dtype", None)
        return cls(num_hidden_layers=n_layers, hidden_size=hidden, intermediate_size=inter,
                   num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
                   vocab_size=vocab, rope_theta=theta, rms_norm_eps=eps, tie_word_embeddings=tie,
                   max_position_embeddings=max_pos, eos_token_ids=eos, bos_token_id=bos,
                   torch_dtype=dtype)

    def to_dict(self) -> dict:
        d = {
            "architectures": [ARCHITECTURE],
            "model_type": "qwen3",
            "num_hidden_layers": self.num_hidden_layers,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "rope_theta": self.rope_theta,
            "rms_norm_eps": self.rms_norm_eps,
            "hidden_act": "silu",
            "attention_bias": False,
        }
        if self.tie_word_embeddings is not None:
            d["tie_word_embeddings"] = self.tie_word_embeddings
        if self.max_position_embeddings is not None:
            d["max_position_embeddings"] = self.max_position_embeddings
        if self.eos_token_ids:
            d["eos_token_id"] = (self.eos_token_ids[0] if len(self.eos_token_ids) == 1
                                 else list(self.eos_token_ids))
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.torch_dtype is not None:
            d["torch_dtype"] = self.torch_dtype
        return d
