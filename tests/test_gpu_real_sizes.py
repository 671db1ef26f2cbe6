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


def test_bfloat16_unequal_batch_that_shrinks(model):
    """24 sequences with unequal prompts start together and end at different steps, so that the decode steps have 24, 17,
    16, 9, 8 and 1 rows: at these widths each of those counts takes other kernels (the few-rows product's forms, the
    library), and each sequence must get the logits it gets alone."""
    folder, cfg, w = model
    rng = np.random.default_rng(4)
    decode_steps = [1] * 7 + [2] + [3] * 7 + [4] + [5] * 7 + [7]
    rng.shuffle(decode_steps)
    heads = rng.integers(1, 20, 24).tolist()
    heads[:3] = [1, 64, 70]
    seqs = [rng.integers(0, cfg["vocab_size"], h + d).tolist() for h, d in zip(heads, decode_steps)]
    eng = qw.Engine.from_folder(folder, dtype="bfloat16", max_tokens=24 * 64 + 128, max_batch=24)
    slots = eng.open_sequences(24)
    got = [[] for _ in seqs]
    first = eng.step([qw.StepEntry(s, t[:h], list(range(h))) for s, t, h in zip(slots, seqs, heads)]).cpu().numpy()
    off = 0
    for i, h in enumerate(heads):
        got[i] += list(first[off:off + h])
        off += h
    pos = list(heads)
    live = list(range(24))
    counts = []
    while live:
        counts.append(len(live))
        out = eng.step([qw.StepEntry(slots[i], [seqs[i][pos[i]]], [0]) for i in live]).cpu().numpy()
        for row, i in zip(out, live):
            got[i].append(row)
            pos[i] += 1
        ended = [i for i in live if pos[i] == len(seqs[i])]
        eng.close_sequences([slots[i] for i in ended])
        live = [i for i in live if i not in ended]
    assert counts == [24, 17, 16, 9, 8, 1, 1]
    for i, t in enumerate(seqs):
        ref = pm.forward_logits(cfg, w, t, round16="bf16")
        err = np.abs(np.stack(got[i]) - ref).max(axis=1) / np.abs(ref).max()
        assert err.max() < BF16_TOL, f"sequence {i} (prompt of {heads[i]}): position {int(np.argmax(err))} off by {err.max():.3e}"


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_output_head_at_the_real_vocabulary(dtype):
    """The head product at 151,936 rows of W (width 1,024 keeps it at 311 MB), for the row counts a step can bring: few
    (the weight-streaming kernels), 9 to 16, and more (the library), against a float64 product of the same numbers."""
    import torch
    from questwend_b200.parts.base import PartSpec, Runtime
    from questwend_b200.parts.registry import build_part
    V, D = 151936, 1024
    dev = torch.device("cuda:0")
    tdtype = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    g = torch.Generator(device=dev).manual_seed(7)
    W = (torch.randn((V, D), generator=g, device=dev) * 0.02).to(tdtype)
    head = build_part("head", PartSpec("linear", {"vocab_size": V, "hidden_size": D, "tied": False,
                                                  "name": "lm_head.weight", "tied_to": "embed"}), Runtime(dev, tdtype))
    head.bind({"lm_head.weight": W})
    cols = np.concatenate([np.arange(0, 300), np.arange(75000, 75300), np.arange(V - 300, V)])     # both ends and the middle
    Wd = W[torch.from_numpy(cols).to(dev)].double().cpu().numpy()
    for M in (1, 8, 13, 16, 24, 64):
        x = torch.randn((M, D), generator=g, device=dev).to(tdtype)
        y = head.forward(x)
        assert tuple(y.shape) == (M, V) and y.dtype == torch.float32
        ref = x.double().cpu().numpy() @ Wd.T
        got = y[:, torch.from_numpy(cols).to(dev)].double().cpu().numpy()
        assert rel_err(got, ref) < (1e-5 if dtype == "float32" else 1e-4), M
        # every column is a sum of the same kind: the largest of all columns agrees with a float64 product of that row
        top = y.argmax(dim=1)
        ref_top = (x.double() @ W[top].double().t()).diagonal()
        assert torch.allclose(y.gather(1, top[:, None])[:, 0].double(), ref_top, rtol=1e-3, atol=1e-4)


def test_early_launches_change_no_token(tmp_path):
    """Kernels that are launched before their predecessor has ended (the few-rows products, decode attention, the norms
    and the merge between them) must read what the predecessor wrote, not what lay there a step before.  Greedy
    generation from CUDA graphs at the 8B widths, two layers, in a process of its own with those launches and in one
    without (QWB200_PDL=0): the same kernels and sums, so every token must be the same.  Random weights make nearly flat
    distributions: a value read too early shows as another token (with x read through the read-only path, `__ldg`, in
    the few-rows product this test fails)."""
    import json
    import os
    import subprocess
    import sys

    cfgd = dict(REAL["8b"], num_hidden_layers=2, vocab_size=4099)
    folder = str(tmp_path / "model")
    qw.write_model_folder(folder, config_from_dict(cfgd), seed=4, dtype="bfloat16")
    script = (
        "import json, sys, numpy as np\n"
        "import questwend_b200 as qw\n"
        "eng = qw.Engine.from_folder(sys.argv[1], dtype='bfloat16', max_tokens=4096)\n"
        "rng = np.random.default_rng(5)\n"
        "out = {}\n"
        "for n in (1, 3, 8):\n"
        "    prompts = [rng.integers(0, eng.vocab_size, int(k)).tolist() for k in rng.integers(5, 90, n)]\n"
        "    out[n] = [r.tokens for r in qw.generate(eng, prompts, max_new_tokens=40, ignore_eos=True)]\n"
        "print('TOKENS ' + json.dumps(out))\n")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    got = {}
    for pdl in ("some", "0"):
        env = dict(os.environ, QWB200_PDL=pdl, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
        proc = subprocess.run([sys.executable, "-c", script, folder], capture_output=True, text=True, timeout=600, env=env)
        assert proc.returncode == 0, proc.stderr[-2000:]
        line = [l for l in proc.stdout.splitlines() if l.startswith("TOKENS ")][-1]
        got[pdl] = json.loads(line[len("TOKENS "):])
    shutil.rmtree(folder, ignore_errors=True)
    assert got["some"] == got["0"]
