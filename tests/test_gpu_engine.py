"""The engine through its Python entry points: long decoding, the first tokens of a sequence, greedy and
sampled generation, slots used again, refusals (needs a B200)."""
import numpy as np
import pytest
import torch

import plain_model as pm
import questwend_b200 as qw
from helpers import BF16_TOL, FP32_TOL, TINY, make_folder, rel_err
from questwend_b200.cache import CacheFull
from questwend_b200.engine.engine import EngineError, StepEntry

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, (cfgd, seed) in TINY.items():
        for dtype in ("float32", "bfloat16"):
            out[name, dtype] = make_folder(tmp_path_factory.mktemp(f"{name}_{dtype}"), cfgd, seed, dtype)
    return out


def tol(dtype):
    return FP32_TOL if dtype == "float32" else BF16_TOL


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D"])
def test_long_decoding(folders, name, dtype):
    """300 tokens one by one after a short prompt: across pages (64) and across runs of the decode kernels (64 or 256)."""
    folder = folders[name, dtype]
    cfg, w = pm.read_model_folder(folder)
    eng = qw.Engine.from_folder(folder, dtype=dtype, max_tokens=512)
    rng = np.random.default_rng(3)
    toks = rng.integers(0, cfg["vocab_size"], 310).tolist()
    ref = pm.forward_logits(cfg, w, toks, round16=None if dtype == "float32" else "bf16")
    (s,) = eng.open_sequences(1)
    rows = list(eng.step([StepEntry(s, toks[:10], list(range(10)))]).cpu().numpy())
    for t in toks[10:]:
        rows.append(eng.step([StepEntry(s, [t], [0])]).cpu().numpy()[0])
    err = np.abs(np.stack(rows) - ref).max(axis=1) / np.abs(ref).max()
    assert err.max() < tol(dtype), f"first position off: {int(np.argmax(err > tol(dtype)))}"
    eng.close_sequences([s])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_first_tokens_of_a_sequence(folders, name, dtype):
    """Position 0 has one key and no rotation; prompts of one and two tokens, then one token each."""
    folder = folders[name, dtype]
    cfg, w = pm.read_model_folder(folder)
    eng = qw.Engine.from_folder(folder, dtype=dtype, max_tokens=256)
    seqs = [[5, 9, 2, 7], [11, 3, 3, 8], [0, 1, 2, 3]]
    heads = [1, 2, 4]
    refs = [pm.forward_logits(cfg, w, t, round16=None if dtype == "float32" else "bf16") for t in seqs]
    slots = eng.open_sequences(3)
    first = eng.step([StepEntry(s, t[:h], list(range(h))) for s, t, h in zip(slots, seqs, heads)]).cpu().numpy()
    off = 0
    for r, h in zip(refs, heads):
        assert rel_err(first[off:off + h], r[:h]) < tol(dtype)
        off += h
    for j in (1, 2, 3):
        live = [i for i in range(3) if heads[i] <= j]
        out = eng.step([StepEntry(slots[i], [seqs[i][j]], [0]) for i in live]).cpu().numpy()
        for row, i in zip(out, live):
            assert rel_err(row, refs[i][j]) < tol(dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["C", "D"])
def test_long_prompts_in_one_step(folders, name, dtype):
    """A step of 690 rows (prompts of 640 and 50 tokens): many row blocks and key tiles for the tcgen05 attention and the
    library products, then a second step that continues from the cache.  (The tcgen05 gate/up product wants a model
    width of 2,048 and more: the tests at real layer sizes reach it.)"""
    folder = folders[name, dtype]
    cfg, w = pm.read_model_folder(folder)
    eng = qw.Engine.from_folder(folder, dtype=dtype, max_tokens=1024)
    rng = np.random.default_rng(11)
    seqs = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (660, 50)]
    refs = [pm.forward_logits(cfg, w, t, round16=None if dtype == "float32" else "bf16") for t in seqs]
    slots = eng.open_sequences(2)
    heads = [640, 50]
    want = [[0, 1, 63, 64, 65, 300, 511, 512, 638, 639], list(range(50))]
    first = eng.step([StepEntry(s, t[:h], wt) for s, t, h, wt in zip(slots, seqs, heads, want)]).cpu().numpy()
    assert rel_err(first[:10], refs[0][want[0]]) < tol(dtype)
    assert rel_err(first[10:], refs[1]) < tol(dtype)
    more = eng.step([StepEntry(slots[0], seqs[0][640:], list(range(20)))]).cpu().numpy()    # 20 more tokens of the first
    assert rel_err(more, refs[0][640:]) < tol(dtype)
    eng.close_sequences(slots)


@pytest.mark.parametrize("use_graph", [True, False])
def test_greedy_generation_matches_the_plain_implementation(folders, use_graph):
    folder = folders["B", "float32"]
    cfg, w = pm.read_model_folder(folder)
    rng = np.random.default_rng(8)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (5, 1, 17, 9, 3)]
    want = [pm.greedy_continue(cfg, w, p, 10) for p in prompts]
    eng = qw.Engine.from_folder(folder, dtype="float32", max_tokens=1024, max_batch=2)   # three batches, slots reused
    stats = qw.GenerationStats()
    res = qw.generate(eng, prompts, max_new_tokens=10, use_graph=use_graph, stats=stats, ignore_eos=True)
    assert [r.tokens for r in res] == want and stats.batches == 3
    # a stop token ends a sequence early and is not emitted; the others go on
    stop = want[2][4]
    res = qw.generate(eng, prompts, max_new_tokens=10, stop_ids=[stop], use_graph=use_graph)
    for r, full in zip(res, want):
        cut = full.index(stop) if stop in full else len(full)
        assert r.tokens == full[:cut] and r.finish_reason == ("stop" if stop in full else "length")
    assert eng.cache.slots.n_free == 2 and eng.cache.free_pages() == [eng.cache.n_pages]


@pytest.mark.parametrize("name", ["B", "C", "D"])
def test_bfloat16_greedy_generation(folders, name):
    folder = folders[name, "bfloat16"]
    cfg, w = pm.read_model_folder(folder)
    prompts = [[3, 14, 15, 92, 65], [35, 89, 79], [32, 38, 46, 26, 43, 38, 32, 79, 50]]
    want = [pm.greedy_continue(cfg, w, p, 8, round16="bf16") for p in prompts]
    eng = qw.Engine.from_folder(folder, dtype="bfloat16", max_tokens=1024)
    got = [r.tokens for r in qw.generate(eng, prompts, max_new_tokens=8, ignore_eos=True)]
    assert got == want


@pytest.mark.parametrize("name,dtype", [("C", "bfloat16"), ("D", "bfloat16"), ("B", "float32")])
def test_long_generation_from_graphs_matches_plain_steps(folders, name, dtype):
    """300 new tokens for prompts of unequal lengths: every sequence crosses pages, runs of the decode kernels and the
    graphs' length bounds (256, 512) at a different step.  The graph replays and the plain steps run the same kernels
    on the same numbers, so the tokens are the same; the first ones are checked against the plain implementation."""
    folder = folders[name, dtype]
    cfg, w = pm.read_model_folder(folder)
    rng = np.random.default_rng(21)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (5, 200, 250, 64)]
    eng = qw.Engine.from_folder(folder, dtype=dtype, max_tokens=4 * 640)
    plain = qw.generate(eng, prompts, max_new_tokens=300, ignore_eos=True, use_graph=False)
    graph = qw.generate(eng, prompts, max_new_tokens=300, ignore_eos=True, use_graph=True)
    assert [r.tokens for r in graph] == [r.tokens for r in plain]
    assert all(len(r.tokens) == 300 for r in graph)
    first = pm.greedy_continue(cfg, w, prompts[0], 6, round16=None if dtype == "float32" else "bf16")
    assert graph[0].tokens[:6] == first
    assert eng.cache.free_pages() == [eng.cache.n_pages] * eng.cache.n_groups()


def test_sampled_generation_is_a_function_of_the_seed(folders):
    folder = folders["A", "float32"]
    eng = qw.Engine.from_folder(folder, dtype="float32", max_tokens=1024, max_batch=3)
    prompts = [[1, 2, 3], [4, 5], [6, 7, 8, 9]]
    sp = qw.SamplingParams(temperature=0.8, top_k=40, top_p=0.95, seed=5)
    a = [r.tokens for r in qw.generate(eng, prompts, max_new_tokens=12, sampling=sp, ignore_eos=True)]
    b = [r.tokens for r in qw.generate(eng, prompts, max_new_tokens=12, sampling=sp, ignore_eos=True, use_graph=False)]
    assert a == b                                           # graph replay and plain stepping draw the same
    c = [r.tokens for r in qw.generate(eng, prompts, max_new_tokens=12, ignore_eos=True,
                                       sampling=qw.SamplingParams(temperature=0.8, top_k=40, top_p=0.95, seed=6))]
    assert a != c
    # one sequence at a time (other batches) gives every sequence the same tokens
    eng1 = qw.Engine.from_folder(folder, dtype="float32", max_tokens=1024, max_batch=1)
    d = [r.tokens for r in qw.generate(eng1, prompts, max_new_tokens=12, sampling=sp, ignore_eos=True)]
    assert a == d
    # penalties change the outcome and keep it reproducible
    pen = qw.SamplingParams(temperature=0.0, repeat_penalty=1.5, frequency_penalty=0.5)
    e = [r.tokens for r in qw.generate(eng, prompts, max_new_tokens=12, sampling=pen, ignore_eos=True)]
    f = [r.tokens for r in qw.generate(eng, prompts, max_new_tokens=12, sampling=pen, ignore_eos=True, use_graph=False)]
    g = [r.tokens for r in qw.generate(eng, prompts, max_new_tokens=12, ignore_eos=True)]
    assert e == f and e != g


def test_refusals_leave_the_cache_as_it_was(folders):
    eng = qw.Engine.from_folder(folders["A", "float32"], dtype="float32", max_tokens=128, max_batch=2)
    a, b = eng.open_sequences(2)
    with pytest.raises(EngineError, match="vocabulary"):
        eng.step([StepEntry(a, [1, 256], [])])
    with pytest.raises(EngineError, match="at least one token"):
        eng.step([StepEntry(a, [], [])])
    with pytest.raises(EngineError, match="twice"):
        eng.step([StepEntry(a, [1], []), StepEntry(a, [2], [])])
    with pytest.raises(EngineError, match="wanted place"):
        eng.step([StepEntry(a, [1, 2], [2])])
    with pytest.raises(CacheFull):
        eng.step([StepEntry(a, [1] * 100, []), StepEntry(b, [1] * 100, [])])     # 2 + 2 pages, the cache has 2
    assert eng.cache.length(a) == 0 and eng.cache.free_pages() == [2]
    eng.step([StepEntry(a, [1] * 64, []), StepEntry(b, [1] * 64, [])])
    with pytest.raises(CacheFull):
        eng.step([StepEntry(a, [1], [0])])
    assert eng.cache.length(a) == 64
    with pytest.raises(EngineError, match="CUDA"):
        qw.Engine.from_folder(folders["A", "float32"], dtype="float32", device="cpu", max_tokens=64)


def test_a_32bit_folder_in_the_bfloat16_engine_and_back(folders):
    """The engine's dtype decides how the matrices are held, whatever the file holds."""
    cfg, w = pm.read_model_folder(folders["A", "float32"])
    toks = list(range(3, 40))
    eng = qw.Engine.from_folder(folders["A", "float32"], dtype="bfloat16", max_tokens=128)
    (s,) = eng.open_sequences(1)
    got = eng.step([StepEntry(s, toks, list(range(len(toks))))]).cpu().numpy()
    w16 = {k: pm.round_bf16(v) if v.ndim == 2 else v for k, v in w.items()}
    assert rel_err(got, pm.forward_logits(cfg, w16, toks, round16="bf16")) < BF16_TOL
    assert eng.model.blocks[0].norm1.weight.dtype == torch.float32
    cfg, w = pm.read_model_folder(folders["A", "bfloat16"])
    eng = qw.Engine.from_folder(folders["A", "bfloat16"], dtype="float32", max_tokens=128)
    (s,) = eng.open_sequences(1)
    got = eng.step([StepEntry(s, toks, list(range(len(toks))))]).cpu().numpy()
    assert rel_err(got, pm.forward_logits(cfg, w, toks)) < FP32_TOL


def test_command_line(folders, tmp_path):
    import os, subprocess, sys
    from helpers import ROOT
    folder = folders["B", "float32"]
    cfg, w = pm.read_model_folder(folder)
    want = [pm.greedy_continue(cfg, w, p, 5) for p in ([3, 14, 15], [9, 26])]
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "qw-cli"), "-m", folder, "-p", "3 14 15", "-p", "9,26",
                           "-n", "5", "--dtype", "float32", "--log-tokens-per-sec", "--ignore-eos"],
                          capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr
    assert [[int(x) for x in line.split()] for line in proc.stdout.strip().splitlines()] == want
    assert "tok/s" in proc.stderr
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "qw-cli"), "-m", folder, "--info"],
                          capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0 and '"parameters"' in proc.stdout


def test_command_line_random_weights_and_step_profile(tmp_path):
    """``--random <config.json> --seed N``: weights drawn from the seed (with ``--save`` into a folder that the plain
    implementation reads too); ``--profile-step``: a line per decode step."""
    import json, os, subprocess, sys
    from helpers import ROOT, TINY_B
    cfg_path = tmp_path / "b.json"
    cfg_path.write_text(json.dumps(TINY_B))
    cli = [sys.executable, os.path.join(ROOT, "bin", "qw-cli")]
    saved = str(tmp_path / "saved")
    proc = subprocess.run(cli + ["--random", str(cfg_path), "--seed", "4", "--save", saved, "-p", "3 14 15", "-n", "6",
                                 "--dtype", "float32", "--ignore-eos", "--profile-step"],
                          capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr
    cfg, w = pm.read_model_folder(saved)
    assert [int(x) for x in proc.stdout.split()] == pm.greedy_continue(cfg, w, [3, 14, 15], 6)
    prof = [line for line in proc.stderr.splitlines() if line.startswith("[prof] step=")]
    assert len(prof) == 5 and all("device=" in line and "wait=" in line for line in prof)
    proc = subprocess.run(cli + ["--random", str(cfg_path), "--seed", "4", "-p", "3 14 15", "-p", "7", "-n", "4", "--ignore-eos"],
                          capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr
    lines = proc.stdout.strip().splitlines()
    assert len(lines) == 2 and all(len(line.split()) == 4 for line in lines)


@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_products_left_in_pieces_for_the_next_norm(folders, name, monkeypatch):
    """The ring product's split form leaves the o and down products as sums over pieces of k, which the norm that follows
    adds onto the residual stream.  It is chosen for matrices with more tiles than SMs; here it is forced onto the tiny
    models' matrices (up to 7 blocks; model D's tiles are cut in two), and the engine must give the plain implementation's logits:
    whole prompts, single tokens, a batch, and generation from graphs."""
    from questwend_b200.kernels import ops

    used = []

    def forced(N, K, n_sm, device):
        blocks = min(7, -(-N // 16) * -(-K // 256))
        counts = ops.ring_split_counts(N, K, blocks)
        if max(counts) > ops.RING_SPLIT_MAX_PLANES:
            return None
        used.append((N, K, max(counts)))
        return blocks, max(counts), torch.tensor(counts, dtype=torch.uint8, device=device)

    monkeypatch.setattr(ops, "_ring_split_plan", forced)
    monkeypatch.setattr(ops, "_RING_PLANS", {})
    folder = folders[name, "bfloat16"]
    cfg, w = pm.read_model_folder(folder)
    eng = qw.Engine.from_folder(folder, dtype="bfloat16", max_tokens=1024)
    rng = np.random.default_rng(11)
    toks = rng.integers(0, cfg["vocab_size"], 90).tolist()
    ref = pm.forward_logits(cfg, w, toks, round16="bf16")
    a, b = eng.open_sequences(2)
    rows = list(eng.step([StepEntry(a, toks[:7], list(range(7))), StepEntry(b, toks[:3], [])])[:7].cpu().numpy())
    both = eng.step([StepEntry(a, [toks[7]], [0]), StepEntry(b, [toks[3]], [0])]).cpu().numpy()
    rows.append(both[0])
    assert rel_err(both[1], ref[3]) < BF16_TOL
    eng.close_sequences([b])
    for t in toks[8:]:
        rows.append(eng.step([StepEntry(a, [t], [0])]).cpu().numpy()[0])
    eng.close_sequences([a])
    assert used, "no matrix of this model took the split form"
    assert name != "D" or max(u[2] for u in used) >= 2
    err = np.abs(np.stack(rows) - ref).max(axis=1) / np.abs(ref).max()
    assert err.max() < BF16_TOL, f"first position off: {int(np.argmax(err > BF16_TOL))}"
    prompts = [[3, 14, 15, 92, 65], [35, 89, 79], [32, 38, 46, 26, 43, 38, 32, 79, 50]]
    want = [pm.greedy_continue(cfg, w, p, 12, round16="bf16") for p in prompts]
    assert [r.tokens for r in qw.generate(eng, prompts, max_new_tokens=12, ignore_eos=True)] == want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D"])
def test_decoding_after_a_rewind(folders, name, dtype):
    """The reference's rewind (core/runtime.cpp:2804-2811): a sequence is cut back to a shorter length and goes on with
    other tokens.  The keys and values beyond the cut stay in their pages (nothing is zeroed) and must neither be read nor
    survive: 150 tokens, cut back to 70 (into the second page) and to 64 (a page's edge), then 40 other tokens, some as a
    short prompt and the rest one by one, against the plain implementation on the sequence as it now is."""
    folder = folders[name, dtype]
    cfg, w = pm.read_model_folder(folder)
    eng = qw.Engine.from_folder(folder, dtype=dtype, max_tokens=512)
    rng = np.random.default_rng(8)
    first = rng.integers(0, cfg["vocab_size"], 150).tolist()
    (s,) = eng.open_sequences(1)
    eng.step([StepEntry(s, first, [])])
    for keep in (70, 64):
        eng.cache.truncate(s, keep)
        assert eng.cache.length(s) == keep
        other = rng.integers(0, cfg["vocab_size"], 40).tolist()
        ref = pm.forward_logits(cfg, w, first[:keep] + other, round16=None if dtype == "float32" else "bf16")[keep:]
        rows = list(eng.step([StepEntry(s, other[:9], list(range(9)))]).cpu().numpy())
        for t in other[9:]:
            rows.append(eng.step([StepEntry(s, [t], [0])]).cpu().numpy()[0])
        err = np.abs(np.stack(rows) - ref).max(axis=1) / np.abs(ref).max()
        assert err.max() < tol(dtype), f"after a cut to {keep}: first position off: {keep + int(np.argmax(err > tol(dtype)))}"
    eng.close_sequences([s])
    assert eng.cache.free_pages() == [eng.cache.n_pages]


def test_the_smoke_entry_point():
    """What the build's smoke check does (a few greedy tokens of a tiny random model in both dtypes against the plain
    implementation, and a 640-token prompt): it raises on a mismatch."""
    import importlib.util
    import os

    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "__graft_entry__.py")
    spec = importlib.util.spec_from_file_location("graft_entry_for_test", path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    module.smoke()
