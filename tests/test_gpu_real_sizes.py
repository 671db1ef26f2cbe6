"""One layer with the layer sizes of real models (widths 1024, 4096 and 5120; 16/8, 32/8, 40/8 and 64/8 heads of 128) and a
vocabulary that is no power of two: the kernels' tile loops, grids and strides run at the sizes they are tuned for,
against the plain implementation (needs a B200; model folders of up to 1.3 GB in a temporary place)."""
import shutil

import numpy as np
import pytest

import plain_model as pm
import questwend_b200 as qw
from helpers import BF16_TOL, FP32_TOL, rel_err
from questwend_b200.config import config_from_dict

pytestmark = pytest.mark.gpu

def real(hidden, heads, kv_heads, inter, tied):
    return {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 1, "hidden_size": hidden,
            "intermediate_size": inter, "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": 128,
            "vocab_size": 8003, "rope_theta": 1e6, "rms_norm_eps": 1e-6, "tie_word_embeddings": tied}


# the layer sizes of Qwen3-0.6B (2 query heads a key/value head, q wider than the model, tied head), 8B (4), 14B (5: no
# divisor of the attention kernel's 128 rows) and 32B (8)
REAL = {"0.6b": real(1024, 16, 8, 3072, True), "8b": real(4096, 32, 8, 12288, False),
        "14b": real(5120, 40, 8, 17408, False), "32b": real(5120, 64, 8, 25600, False)}


@pytest.fixture(scope="module", params=sorted(REAL))
def model(request, tmp_path_factory):
    folder = str(tmp_path_factory.mktemp("real_sizes_" + request.param.replace(".", "_")))
    qw.write_model_folder(folder, config_from_dict(REAL[request.param]), seed=2, dtype="bfloat16")
    cfg, w = pm.read_model_folder(folder)
    yield folder, cfg, w
    shutil.rmtree(folder, ignore_errors=True)          # up to a gigabyte a folder: not left for pytest's later clean-up


def run_cut(eng, toks, cuts):
    (s,) = eng.open_sequences(1)
    rows, pos = [], 0
    for c in cuts:
        rows.append(eng.step([qw.StepEntry(s, toks[pos:pos + c], list(range(c)))]).cpu().numpy())
        pos += c
    eng.close_sequences([s])
    return np.concatenate(rows)


def test_bfloat16_whole_and_cut(model):
    folder, cfg, w = model
    toks = np.random.default_rng(0).integers(0, cfg["vocab_size"], 700).tolist()
    ref = pm.forward_logits(cfg, w, toks, round16="bf16")
    eng = qw.Engine.from_folder(folder, dtype="bfloat16", max_tokens=2048)
    # whole (the tcgen05 product and attention); a long prompt, a short one and single tokens; single tokens first
    for cuts in ([700], [600, 60] + [1] * 40, [3] + [1] * 50 + [647]):
        got = run_cut(eng, toks, cuts)
        assert rel_err(got, ref) < BF16_TOL, cuts[:3]


def test_float32_prompt_then_tokens(model):
    folder, cfg, w = model
    toks = np.random.default_rng(1).integers(0, cfg["vocab_size"], 200).tolist()
    ref = pm.forward_logits(cfg, w, toks)
    eng = qw.Engine.from_folder(folder, dtype="float32", max_tokens=1024)
    assert rel_err(run_cut(eng, toks, [150] + [1] * 50), ref) < FP32_TOL
