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
