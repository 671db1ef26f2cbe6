#!/usr/bin/env python3
"""Makes tests/golden/qwen3_tiny_{A,B}.npz: the logits of kishida/questwend's own CPU code
on the two tiny random models of the tests.

    python tests/golden/make_golden.py --reference <checkout of kishida/questwend> [--build-dir DIR]

It builds the reference's ``questwend_core`` library with CMake (CPU only, no network), compiles
``ref_driver.cpp`` against it, writes each tiny model with this library's random-weights mode
(32-bit, the seeds of tests/helpers.py), hands the very same numbers to the driver under the
reference's GGUF tensor names, and stores: the token ids, the reference's logits at every
position (tokens fed one at a time), its last-position logits for the whole prompt fed at once,
and a SHA-256 of model.safetensors so that a test can tell whether it regenerated the same weights.
tests/test_plain.py compares the plain implementation with these files.
"""
import argparse
import hashlib
import json
import os
import struct
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from helpers import TINY, make_folder  # noqa: E402
import plain_model as pm  # noqa: E402

N_TOKENS = 40


def gguf_name(hf: str) -> str:
    """Hugging Face tensor name -> the GGUF name the reference looks up (core/runtime.cpp:268-279,
    core/model.cpp:581-584)."""
    top = {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight": "output_norm.weight",
           "lm_head.weight": "output.weight"}
    if hf in top:
        return top[hf]
    parts = hf.split(".")
    layer, rest = parts[2], ".".join(parts[3:])
    sub = {"input_layernorm.weight": "attn_norm.weight", "post_attention_layernorm.weight": "ffn_norm.weight",
           "self_attn.q_proj.weight": "attn_q.weight", "self_attn.k_proj.weight": "attn_k.weight",
           "self_attn.v_proj.weight": "attn_v.weight", "self_attn.o_proj.weight": "attn_output.weight",
           "self_attn.q_norm.weight": "attn_q_norm.weight", "self_attn.k_norm.weight": "attn_k_norm.weight",
           "mlp.gate_proj.weight": "ffn_gate.weight", "mlp.up_proj.weight": "ffn_up.weight",
           "mlp.down_proj.weight": "ffn_down.weight"}[rest]
    return f"blk.{layer}.{sub}"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="a checkout of kishida/questwend (read only)")
    ap.add_argument("--build-dir", default=os.path.join(tempfile.gettempdir(), "questwend_ref_build"))
    args = ap.parse_args()
    ref, bd = args.reference, args.build_dir
    subprocess.check_call(["cmake", "-S", ref, "-B", bd, "-G", "Ninja", "-DGGML_NATIVE=OFF", "-DGGML_OPENMP=OFF",
                           "-DCMAKE_BUILD_TYPE=Release", "-DBUILD_SHARED_LIBS=OFF"])
    subprocess.check_call(["cmake", "--build", bd, "--target", "questwend_core"])
    libs = []
    for root, _, files in os.walk(bd):
        libs += [os.path.join(root, f) for f in files if f.endswith(".a")]
    order = ["questwend_core", "ggml.a", "ggml-cpu", "ggml-base"]
    libs.sort(key=lambda p: next((i for i, o in enumerate(order) if o in os.path.basename(p)), 99))
    driver = os.path.join(bd, "ref_driver")
    subprocess.check_call(["g++", "-O2", "-std=c++17", os.path.join(HERE, "ref_driver.cpp"), "-I", os.path.join(ref, "core"),
                           "-I", os.path.join(ref, "third_party/ggml/include"), "-o", driver, "-Wl,--start-group"] + libs +
                          ["-Wl,--end-group", "-lpthread", "-ldl", "-lm", "-fopenmp"])
    for name, (cfgd, seed) in TINY.items():
        with tempfile.TemporaryDirectory() as tmp:
            folder = make_folder(os.path.join(tmp, "m"), cfgd, seed, "float32")
            cfg, w = pm.read_model_folder(folder)
            sha = hashlib.sha256(open(os.path.join(folder, "model.safetensors"), "rb").read()).hexdigest()
            tokens = np.random.default_rng(100 + seed).integers(0, cfgd["vocab_size"], N_TOKENS).astype(np.int32)
            dump = os.path.join(tmp, "dump.bin")
            with open(dump, "wb") as f:
                f.write(struct.pack("<9i", cfgd["num_hidden_layers"], cfgd["hidden_size"], cfgd["num_attention_heads"],
                                    cfgd["num_key_value_heads"], cfgd["head_dim"], cfgd["intermediate_size"],
                                    cfgd["vocab_size"], int(cfgd["tie_word_embeddings"]), N_TOKENS))
                f.write(struct.pack("<2f", cfgd["rope_theta"], cfgd["rms_norm_eps"]))
                f.write(tokens.tobytes())
                for hf, arr in w.items():
                    g = gguf_name(hf).encode()
                    f.write(struct.pack("<i", len(g)) + g + struct.pack("<i", arr.ndim) +
                            struct.pack(f"<{arr.ndim}i", *arr.shape) + arr.astype("<f4").tobytes())
            out = os.path.join(tmp, "out.bin")
            subprocess.check_call([driver, dump, os.path.join(tmp, "tiny.gguf"), out])
            raw = np.fromfile(out, dtype="<f4")
            V = cfgd["vocab_size"]
            assert raw.size == (N_TOKENS + 1) * V, raw.size
            np.savez_compressed(os.path.join(HERE, f"qwen3_tiny_{name}.npz"), tokens=tokens,
                                logits_token_by_token=raw[:N_TOKENS * V].reshape(N_TOKENS, V),
                                logits_whole_last=raw[N_TOKENS * V:], weights_sha256=np.array(sha),
                                config=np.array(json.dumps(cfgd)), seed=np.array(seed))
            plain = pm.forward_logits(cfg, w, tokens.tolist())
            plain16 = pm.forward_logits(cfg, w, tokens.tolist(), round16="f16")
            got = raw[:N_TOKENS * V].reshape(N_TOKENS, V)
            scale = np.abs(plain).max()
            print(f"{name}: reference vs plain float64 {np.abs(got - plain).max() / scale:.3e}; "
                  f"vs plain with the reference's half roundings {np.abs(got - plain16).max() / scale:.3e}")


if __name__ == "__main__":
    main()
