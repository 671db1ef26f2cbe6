"""Configuration and registry (no GPU)."""
import json

import pytest

import questwend_b200  # noqa: F401
from questwend_b200.config import ConfigError, architectures, config_from_dict, get_architecture, load_config
from questwend_b200.config.qwen3 import Qwen3Config
from helpers import TINY_A, TINY_B


def test_reads_every_key_of_both_tiny_configs():
    a, b = config_from_dict(TINY_A), config_from_dict(TINY_B)
    assert isinstance(a, Qwen3Config)
    assert (a.num_hidden_layers, a.hidden_size, a.intermediate_size, a.num_attention_heads,
            a.num_key_value_heads, a.head_dim, a.vocab_size) == (2, 64, 128, 4, 2, 16, 256)
    assert (a.rope_theta, a.rms_norm_eps, a.tie_word_embeddings) == (10000.0, 1e-6, True)
    assert (b.num_hidden_layers, b.hidden_size, b.intermediate_size, b.num_attention_heads,
            b.num_key_value_heads, b.head_dim, b.vocab_size) == (3, 96, 200, 6, 1, 32, 384)
    assert (b.rope_theta, b.rms_norm_eps, b.tie_word_embeddings) == (1e6, 1e-5, False)


def test_defaults_follow_the_reference():
    d = {k: v for k, v in TINY_A.items() if k not in ("num_key_value_heads", "head_dim", "tie_word_embeddings")}
    c = config_from_dict(d)
    assert c.num_key_value_heads == c.num_attention_heads          # core/model.cpp:520
    assert c.head_dim == c.hidden_size // c.num_attention_heads   # core/model.cpp:526-527
    assert c.tie_word_embeddings is None                           # decided by the tensor's presence


def test_round_trip_through_to_dict():
    for d in (TINY_A, TINY_B):
        c = config_from_dict(d)
        assert config_from_dict(c.to_dict()) == c


def test_rope_theta_inside_rope_parameters():
    d = {k: v for k, v in TINY_A.items() if k != "rope_theta"}
    d["rope_parameters"] = {"rope_theta": 5000.0, "rope_type": "default"}
    assert config_from_dict(d).rope_theta == 5000.0


def test_eos_as_int_or_list():
    assert config_from_dict({**TINY_A, "eos_token_id": 7}).eos_token_ids == (7,)
    assert config_from_dict({**TINY_A, "eos_token_id": [7, 9]}).eos_token_ids == (7, 9)


@pytest.mark.parametrize("key", ["num_hidden_layers", "hidden_size", "intermediate_size", "num_attention_heads",
                                 "vocab_size", "rope_theta", "rms_norm_eps"])
def test_missing_key_is_named(key):
    d = {k: v for k, v in TINY_B.items() if k != key}
    with pytest.raises(ConfigError, match=key):
        config_from_dict(d)


@pytest.mark.parametrize("patch,word", [
    ({"attention_bias": True}, "attention_bias"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"use_sliding_window": True}, "use_sliding_window"),
    ({"layer_types": ["full_attention", "sliding_attention"]}, "layer_types"),
    ({"num_key_value_heads": 3}, "num_key_value_heads"),
    ({"head_dim": 15}, "head_dim"),
    ({"hidden_size": "64"}, "hidden_size"),
    ({"hidden_size": 64.5}, "hidden_size"),
    ({"rms_norm_eps": 0}, "rms_norm_eps"),
    ({"num_hidden_layers": 0}, "num_hidden_layers"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"model_type": "llama"}, "model_type"),
    ({"tie_word_embeddings": "yes"}, "tie_word_embeddings"),
])
def test_rejections_name_the_key(patch, word):
    with pytest.raises(ConfigError, match=word):
        config_from_dict({**TINY_A, **patch})


@pytest.mark.parametrize("head_dim", [24, 320])
def test_a_head_size_the_kernels_do_not_take_is_refused_before_any_weight_is_read(head_dim, tmp_path):
    """Not at the first step, with gigabytes of weights on the device: when the configuration is read, with the key's
    name; and, for an architecture whose configuration does not check, when the attention part is built."""
    with pytest.raises(ConfigError, match="key 'head_dim'.*multiples of 16"):
        config_from_dict({**TINY_A, "head_dim": head_dim})
    with pytest.raises(ConfigError, match="'hidden_size' / 'num_attention_heads'"):
        config_from_dict({k: v for k, v in {**TINY_A, "hidden_size": 4 * head_dim}.items() if k != "head_dim"})
    import torch
    from questwend_b200.parts import PartSpec, Runtime, build_part
    spec = PartSpec("gqa", {"hidden_size": 64, "n_heads": 4, "n_kv_heads": 2, "head_dim": head_dim}, prefix="layers.0.mix.")
    with pytest.raises(ValueError, match="layers.0.mix.*'head_dim'.*multiples of 16"):
        build_part("mixer", spec, Runtime(torch.device("cpu"), torch.float32))
    build_part("mixer", PartSpec("gqa", {"hidden_size": 64, "n_heads": 4, "n_kv_heads": 2, "head_dim": 48}),
               Runtime(torch.device("cpu"), torch.float32))


def test_unknown_architecture_lists_the_known():
    with pytest.raises(ConfigError, match="Qwen3ForCausalLM"):
        config_from_dict({**TINY_A, "architectures": ["NoSuchModel"]})
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({k: v for k, v in TINY_A.items() if k != "architectures"})
    assert "Qwen3ForCausalLM" in architectures()


def test_load_config_from_folder(tmp_path):
    with pytest.raises(ConfigError, match="config.json"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{ not json")
    with pytest.raises(ConfigError, match="JSON"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    assert load_config(str(tmp_path)) == config_from_dict(TINY_B)


def test_plan_is_data():
    cfg = config_from_dict(TINY_B)
    plan = get_architecture(cfg.architecture).plan(cfg)
    assert len(plan.layers) == 3 and [r.layer for r in plan.schedule] == [0, 1, 2]
    layer = plan.layers[1]
    assert layer.mixer.kind == "gqa" and layer.feed_forward.kind == "gated_mlp" and layer.norm.kind == "rms"
    assert layer.mixer.params["head_dim"] == 32 and layer.norm.params["eps"] == 1e-5
    assert layer.position.params == {"theta": 1e6, "rotary_dim": 32}
    names = {t.name for t in plan.manifest()}
    assert "model.layers.2.self_attn.q_norm.weight" in names and "lm_head.weight" in names
    shapes = {t.name: t.shape for t in plan.manifest()}
    assert shapes["model.layers.0.self_attn.q_proj.weight"] == (192, 96)
    assert shapes["model.layers.0.mlp.down_proj.weight"] == (96, 200)


def test_info_counts_weights_and_cache():
    from questwend_b200.cli import model_info
    cfgd = TINY_B
    info = model_info(config_from_dict(dict(cfgd)), "float32")
    L, D, F, V = cfgd["num_hidden_layers"], cfgd["hidden_size"], cfgd["intermediate_size"], cfgd["vocab_size"]
    Hq, Hkv, hd = cfgd["num_attention_heads"], cfgd["num_key_value_heads"], cfgd["head_dim"]
    per_layer = (Hq + 2 * Hkv) * hd * D + Hq * hd * D + 3 * F * D + 2 * D + 2 * hd
    params = L * per_layer + V * D * (1 if cfgd.get("tie_word_embeddings") else 2) + D
    assert info["parameters"] == params
    assert info["memory"] == {"dtype": "float32", "weight_bytes": 4 * params,
                              "cache_bytes_per_token": L * 2 * Hkv * hd * 4, "state_bytes_per_sequence": 0}
    half = model_info(config_from_dict(dict(cfgd)), "bfloat16")["memory"]
    assert half["weight_bytes"] == 2 * params and half["cache_bytes_per_token"] == L * 2 * Hkv * hd * 2


def test_ring_split_counts_match_a_walk_over_the_blocks():
    """The table that says into how many planes the ring product's split form cuts a tile is closed-form arithmetic; the
    kernel's blocks walk their shares stage by stage.  Both must agree, also on which plane a block's piece is."""
    from questwend_b200.kernels import ops
    for N, K, blocks in [(4096, 4096, 148), (4096, 12288, 148), (5120, 25600, 148), (2400, 2048, 148), (200, 1000, 7),
                         (37, 4096, 5), (64, 520, 11), (1000, 96, 13), (16, 256, 1), (48, 768, 9)]:
        n_tiles, n_stages = -(-N // 16), -(-K // 256)
        all_stages = n_tiles * n_stages
        holders = [[] for _ in range(n_tiles)]           # per tile: the blocks that hold a piece, in order
        for b in range(blocks):
            begin, end = all_stages * b // blocks, all_stages * (b + 1) // blocks
            for stage in range(begin, end):
                t = stage // n_stages
                if not holders[t] or holders[t][-1] != b:
                    holders[t].append(b)
        counts = ops.ring_split_counts(N, K, blocks)
        assert counts == [len(h) for h in holders], (N, K, blocks)
        for t, hs in enumerate(holders):                 # the kernel's plane of a later piece: block - the tile's first block
            first = ((t * n_stages + 1) * blocks - 1) // all_stages
            assert hs == list(range(first, first + len(hs))), (N, K, blocks, t)
