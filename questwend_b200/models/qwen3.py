"""Qwen3 dense decoder: configuration -> plan.

Every layer is the same here: a pre-norm block around grouped-query attention
with per-head q/k RMS norm and NeoX rotation over the whole head, and a SiLU-gated
feed-forward; one epsilon for all norms; tensors under their Hugging Face names.
The reference builds the same layer in ``build_graph`` (core/runtime.cpp:976-1100,
the branch with ``gated == false`` and no experts) and names the tensors
``blk.N.attn_q.weight`` and so on (core/runtime.cpp:268-279).
"""
from __future__ import annotations

from ..config.qwen3 import ARCHITECTURE, Qwen3Config
from ..config.registry import register_architecture
from ..engine.plan import LayerSpec, ModelPlan, Run
from ..parts.base import PartSpec


def qwen3_plan(cfg: Qwen3Config) -> ModelPlan:
    norm = PartSpec("rms", {"dim": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    position = PartSpec("rotary_neox", {"theta": cfg.rope_theta, "rotary_dim": cfg.head_dim})
    mixer = PartSpec("gqa", {"hidden_size": cfg.hidden_size, "n_heads": cfg.num_attention_heads,
                             "n_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                             "qk_norm": True, "norm_eps": cfg.rms_norm_eps, "window": 0})
    ffn = PartSpec("gated_mlp", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size})
    layers = [LayerSpec(block=PartSpec("pre_norm", {"mixer_norm": "input_layernorm",
                                                    "ffn_norm": "post_attention_layernorm",
                                                    "mixer_prefix": "self_attn", "ffn_prefix": "mlp"},
                                       prefix=f"model.layers.{i}."),
                        mixer=mixer, feed_forward=ffn, norm=norm, position=position)
              for i in range(cfg.num_hidden_layers)]
    return ModelPlan(
        architecture=ARCHITECTURE,
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("token", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                                     "name": "embed_tokens.weight"}, prefix="model."),
        layers=layers,
        schedule=[Run(i) for i in range(cfg.num_hidden_layers)],
        final_norm=PartSpec("rms", {"dim": cfg.hidden_size, "eps": cfg.rms_norm_eps}, prefix="model.norm."),
        head=PartSpec("linear", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                                 "tied": cfg.tie_word_embeddings, "name": "lm_head.weight",
                                 "tied_to": "model.embed_tokens.weight"}),
        stop_token_ids=tuple(cfg.eos_token_ids),
        max_position=cfg.max_position_embeddings,
    )


register_architecture(ARCHITECTURE, Qwen3Config, qwen3_plan, replace=True)
