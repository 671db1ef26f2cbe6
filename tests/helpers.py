"""Shared by the tests: the two tiny configurations, model folders, traces."""
from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Two tiny Qwen3 configurations that differ in every size and option.
TINY_A = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 2,
          "hidden_size": 64, "intermediate_size": 128, "num_attention_heads": 4, "num_key_value_heads": 2,
          "head_dim": 16, "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
          "tie_word_embeddings": True}
TINY_B = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 3,
          "hidden_size": 96, "intermediate_size": 200, "num_attention_heads": 6, "num_key_value_heads": 1,
          "head_dim": 32, "vocab_size": 384, "rope_theta": 1e6, "rms_norm_eps": 1e-5,
          "tie_word_embeddings": False}
# Two more with the head sizes and head groups that the tensor-core kernels take (64 and 128; 2 and 4 query heads per
# key/value head), still small everywhere else.
TINY_C = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 2,
          "hidden_size": 128, "intermediate_size": 192, "num_attention_heads": 4, "num_key_value_heads": 2,
          "head_dim": 64, "vocab_size": 320, "rope_theta": 50000.0, "rms_norm_eps": 1e-6,
          "tie_word_embeddings": False}
TINY_D = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 2,
          "hidden_size": 192, "intermediate_size": 264, "num_attention_heads": 8, "num_key_value_heads": 2,
          "head_dim": 128, "vocab_size": 296, "rope_theta": 1e6, "rms_norm_eps": 1e-5,
          "tie_word_embeddings": True}
TINY = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 2), "D": (TINY_D, 3)}

FP32_TOL = 1e-4        # max |delta| <= FP32_TOL * max |logit|, 32-bit engine against the plain implementation
BF16_TOL = 2.0 ** -7   # the same for the bfloat16 engine against the plain implementation that rounds where
                       # the engine rounds: one bfloat16 unit in the last place (2^-8 relative) on the logits'
                       # scale, doubled for the places where the two round a value to different neighbours


def make_folder(path, cfgd, seed, dtype):
    import questwend_b200 as qw
    from questwend_b200.config.registry import config_from_dict
    qw.write_model_folder(str(path), config_from_dict(cfgd), seed, dtype)
    return str(path)


def rel_err(got, ref) -> float:
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    return float(np.abs(got - ref).max() / np.abs(ref).max())


def run_trace(model_dir, dtype, steps, max_tokens, out_dir, timeout=600):
    """Run bin/trace_run on a list of step dicts; returns {step: float32 array [wanted, vocab]}."""
    os.makedirs(out_dir, exist_ok=True)
    text = "".join(json.dumps(s) + "\n" for s in steps)
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir,
                           "--dtype", dtype, "--out", out_dir, "--max-tokens", str(max_tokens)],
                          input=text, capture_output=True, text=True, timeout=timeout)
    assert proc.returncode == 0, f"trace_run failed:\n{proc.stdout}\n{proc.stderr}"
    done = [line for line in proc.stdout.splitlines() if line.startswith("done ")]
    assert [d.split()[1] for d in done] == [str(s["step"]) for s in steps], proc.stdout
    with open(os.path.join(model_dir, "config.json")) as f:
        V = json.load(f)["vocab_size"]
    out = {}
    for s in steps:
        n = sum(len(e.get("want", [])) for e in s["entries"])
        path = os.path.join(out_dir, f"{s['step']}.f32")
        if n:
            out[s["step"]] = np.fromfile(path, dtype="<f4").reshape(n, V)
        else:
            assert not os.path.exists(path)
    return out
