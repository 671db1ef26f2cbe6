"""The command line and the benchmark's argument handling, as far as they go without a GPU: what is refused and how,
what ``--info`` and ``--random --save`` give."""
import json
import os
import subprocess
import sys

import pytest

import plain_model as pm
from helpers import TINY_A, TINY_B
from questwend_b200 import cli

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_parse_ids():
    assert cli.parse_ids("1 2  3") == [1, 2, 3]
    assert cli.parse_ids("7,8, 9") == [7, 8, 9]
    with pytest.raises(SystemExit):
        cli.parse_ids("1 two 3")


def test_the_command_line_wants_one_source_of_weights_and_a_prompt(tmp_path, capsys):
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(TINY_A))
    with pytest.raises(SystemExit, match="either -m"):
        cli.main(["-p", "1 2"])
    with pytest.raises(SystemExit, match="either -m"):
        cli.main(["-m", str(tmp_path), "--random", str(cfg), "-p", "1 2"])
    with pytest.raises(SystemExit, match="--save goes with --random"):
        cli.main(["-m", str(tmp_path), "--save", str(tmp_path / "x")])
    assert cli.main(["--random", str(cfg), "--save", str(tmp_path / "model"), "--seed", "3"]) == 0
    assert capsys.readouterr().out.strip() == str(tmp_path / "model")
    with pytest.raises(SystemExit, match="no prompt"):
        cli.main(["-m", str(tmp_path / "model")])


def test_random_save_writes_a_folder_that_reads_back(tmp_path):
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(TINY_B))
    for seed in (3, 4):
        assert cli.main(["--random", str(cfg), "--save", str(tmp_path / f"m{seed}"), "--seed", str(seed), "--dtype", "float32"]) == 0
    config, w3 = pm.read_model_folder(str(tmp_path / "m3"))
    _, w4 = pm.read_model_folder(str(tmp_path / "m4"))
    assert config["num_hidden_layers"] == TINY_B["num_hidden_layers"] and config["head_dim"] == TINY_B["head_dim"]
    assert set(w3) == set(w4) and any((w3[k] != w4[k]).any() for k in w3)          # the seed decides the weights
    again = tmp_path / "again"
    assert cli.main(["--random", str(cfg), "--save", str(again), "--seed", "3", "--dtype", "float32"]) == 0
    _, w3b = pm.read_model_folder(str(again))
    assert all((w3[k] == w3b[k]).all() for k in w3)


def test_info_counts_from_the_configuration_alone(tmp_path, capsys):
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(TINY_A))
    assert cli.main(["--random", str(cfg), "--info"]) == 0
    info = json.loads(capsys.readouterr().out)
    assert info["config"]["architectures"] == ["Qwen3ForCausalLM"] and info["layers"] == TINY_A["num_hidden_layers"]
    D, V, L = TINY_A["hidden_size"], TINY_A["vocab_size"], TINY_A["num_hidden_layers"]
    assert info["parameters"] > V * D + L * 3 * D * TINY_A["intermediate_size"]
    mem = info["memory"]
    assert mem["dtype"] == "bfloat16" and mem["state_bytes_per_sequence"] == 0
    assert mem["cache_bytes_per_token"] == L * 2 * TINY_A["num_key_value_heads"] * TINY_A["head_dim"] * 2


def test_the_options_of_the_reference_command_line_are_there():
    """Names and meanings follow the reference's generation program (cli/main.cpp:139-150: -m, -p, -n, --temp,
    --top-k, --repeat-penalty, --repeat-last-n and their neighbours)."""
    ap = cli.build_parser()
    known = {s for a in ap._actions for s in a.option_strings}
    for name in ("-m", "-p", "-n", "--n-ctx", "--temp", "--top-k", "--top-p", "--seed", "--repeat-penalty", "--repeat-last-n",
                 "--presence-penalty", "--frequency-penalty", "--ignore-eos", "--random", "--save", "--info", "--dtype"):
        assert name in known, name
    args = ap.parse_args(["-m", "x", "-p", "1 2", "-p", "3", "-n", "7", "--temp", "0.5", "--top-k", "5"])
    assert args.prompts == ["1 2", "3"] and args.max_tokens == 7 and args.temp == 0.5 and args.top_k == 5 and args.top_p == 0.95


def test_bench_refuses_more_than_one_gpu_with_one_line():
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--gpus", "2"], capture_output=True, text=True, timeout=120)
    assert p.returncode == 2
    lines = [line for line in (p.stdout + p.stderr).splitlines() if line.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_replay_protocol_with_a_stand_in_engine(tmp_path, monkeypatch, capsys):
    """trace_run's own part of the work: a slot per request at its first step, a file only for a step that wants
    logits (rows in the order of the entries and of ``want``), ``done <step>`` after every step, slots given back at
    ``end``.  The engine is a stand-in that records its calls; the real one is replayed in the GPU tests."""
    import io

    import numpy as np
    import torch

    from questwend_b200 import replay
    from questwend_b200.engine import engine as engine_module

    calls = []

    class StandIn:
        def __init__(self):
            self.free = list(range(5))

        def open_sequences(self, n):
            got, self.free = self.free[:n], self.free[n:]
            calls.append(("open", got))
            return got

        def close_sequences(self, slots):
            calls.append(("close", list(slots)))
            self.free = sorted(self.free + list(slots))

        def step(self, entries):
            calls.append(("step", [(e.slot, list(e.tokens), list(e.want)) for e in entries]))
            rows = [[e.slot, e.tokens[w], w] for e in entries for w in e.want]
            return torch.tensor(rows, dtype=torch.float32).reshape(len(rows), 3)

    made = {}

    def from_folder(folder, **kw):
        made.update(kw, folder=folder)
        return StandIn()

    monkeypatch.setattr(engine_module.Engine, "from_folder", staticmethod(from_folder))
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}, {"id": "b", "tokens": [9], "want": [0]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [4], "want": []}, {"id": "b", "tokens": [7], "want": []}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": [8], "want": [0]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "c", "tokens": [1, 2], "want": [1]}], "end": ["c", "never-seen"]}]
    monkeypatch.setattr(sys, "stdin", io.StringIO("".join(json.dumps(s) + "\n" for s in steps) + "\n"))
    out = tmp_path / "out"
    assert replay.main(["--model", "somewhere", "--dtype", "float32", "--out", str(out), "--max-tokens", "200"]) == 0
    assert made["folder"] == "somewhere" and made["dtype"] == "float32" and made["max_tokens"] == 200 and made["max_batch"] == 4
    assert capsys.readouterr().out.split() == ["done", "0", "done", "1", "done", "2", "done", "3"]
    assert sorted(os.listdir(out)) == ["0.f32", "2.f32", "3.f32"]                  # step 1 wanted nothing
    assert np.fromfile(out / "0.f32", dtype="<f4").reshape(3, 3).tolist() == [[0, 5, 0], [0, 3, 2], [1, 9, 0]]
    assert np.fromfile(out / "2.f32", dtype="<f4").tolist() == [0, 8, 0]
    assert np.fromfile(out / "3.f32", dtype="<f4").tolist() == [0, 2, 1]           # c in a slot that was given back
    assert [c for c in calls if c[0] != "step"] == [("open", [0]), ("open", [1]), ("close", [1]), ("close", [0]), ("open", [0]),
                                                    ("close", [0])]
