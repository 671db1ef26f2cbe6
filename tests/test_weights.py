"""Safetensors, the loader's one error, random weights (no GPU)."""
import json
import os
import struct

import numpy as np
import pytest
import torch

import questwend_b200  # noqa: F401
from questwend_b200.config import config_from_dict, get_architecture
from questwend_b200.weights import (MATRIX, VECTOR, SafetensorsError, SafetensorsFile, TensorSpec, WeightsError,
                                    held_dtype, load_tensors, random_tensors, write_safetensors)
from helpers import TINY_A, TINY_B, make_folder
import plain_model as pm


def test_safetensors_round_trip(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int32).reshape(2, 3),
         "empty": torch.zeros(0, 4)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t, metadata={"k": "v"})
    f = SafetensorsFile(p)
    assert set(f.names()) == set(t) and f.metadata == {"k": "v"}
    for k, v in t.items():
        got = f.tensor(k)
        assert got.dtype == v.dtype and got.shape == v.shape and torch.equal(got, v)
    f.close()
    # the independent reader of the plain implementation reads the same numbers
    plain = pm.read_safetensors(p)
    assert np.array_equal(plain["b"], t["b"].to(torch.float64).numpy())


def test_truncated_and_broken_files(tmp_path):
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, {"a": torch.randn(4, 4)})
    raw = open(p, "rb").read()
    open(p, "wb").write(raw[:-8])
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(p)
    open(p, "wb").write(raw[:4])
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(p)
    open(p, "wb").write(struct.pack("<Q", 5) + b"{oops")
    with pytest.raises(SafetensorsError, match="JSON"):
        SafetensorsFile(p)
    with pytest.raises(SafetensorsError, match="neither"):
        load_tensors(str(tmp_path / "nowhere"), [], torch.float32, "cpu")


def _folder_with(tmp_path, cfgd, edit):
    d = make_folder(tmp_path / "m", cfgd, 3, "float32")
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    f.close()
    edit(tensors)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    cfg = config_from_dict(cfgd)
    return d, get_architecture(cfg.architecture).plan(cfg).manifest()


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    def edit(t):
        del t["model.layers.1.mlp.up_proj.weight"]
        del t["model.norm.weight"]
        t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
        t["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(32, 32)
        t["model.layers.2.self_attn.q_norm.weight"] = torch.zeros(16)
    d, manifest = _folder_with(tmp_path, TINY_B, edit)
    with pytest.raises(WeightsError) as e:
        load_tensors(d, manifest, torch.float32, "cpu")
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert {n for n, _, _ in err.wrong_shape} == {"model.layers.0.self_attn.k_proj.weight",
                                                  "model.layers.2.self_attn.q_norm.weight"}
    msg = str(err)
    for word in ("missing (2)", "unexpected (1)", "wrong shape (2)", "[32, 32]", "expected [32, 96]"):
        assert word in msg


def test_integer_tensor_where_floats_belong(tmp_path):
    def edit(t):
        t["model.norm.weight"] = torch.ones(96, dtype=torch.int32)
    d, manifest = _folder_with(tmp_path, TINY_B, edit)
    with pytest.raises(WeightsError, match="wrong dtype"):
        load_tensors(d, manifest, torch.float32, "cpu")


def test_tied_head(tmp_path):
    # tied and no stored head: fine; tied with a stored copy: ignored; untied without a head: missing
    d = make_folder(tmp_path / "a", TINY_A, 0, "float32")
    cfg = config_from_dict(TINY_A)
    manifest = get_architecture(cfg.architecture).plan(cfg).manifest()
    w = load_tensors(d, manifest, torch.float32, "cpu")
    assert "lm_head.weight" not in w
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    f.close()
    tensors["lm_head.weight"] = torch.zeros(256, 64)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    assert "lm_head.weight" not in load_tensors(d, manifest, torch.float32, "cpu")
    cfg_b = config_from_dict({**TINY_A, "tie_word_embeddings": False})
    manifest_b = get_architecture(cfg_b.architecture).plan(cfg_b).manifest()
    del tensors["lm_head.weight"]
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    with pytest.raises(WeightsError, match="lm_head.weight"):
        load_tensors(d, manifest_b, torch.float32, "cpu")
    # undecided (no key): the tensor's presence decides, as in the reference (core/runtime.cpp:1093-1094)
    cfg_c = config_from_dict({k: v for k, v in TINY_A.items() if k != "tie_word_embeddings"})
    manifest_c = get_architecture(cfg_c.architecture).plan(cfg_c).manifest()
    assert "lm_head.weight" not in load_tensors(d, manifest_c, torch.float32, "cpu")


def test_held_dtypes():
    m, v = TensorSpec("m", (2, 2), MATRIX), TensorSpec("v", (2,), VECTOR)
    assert held_dtype(m, torch.float32, torch.bfloat16) == torch.bfloat16
    assert held_dtype(m, torch.bfloat16, torch.float32) == torch.float32
    assert held_dtype(v, torch.float32, torch.bfloat16) == torch.float32     # stored in 32-bit stays so
    assert held_dtype(v, torch.bfloat16, torch.bfloat16) == torch.bfloat16
    assert held_dtype(v, torch.bfloat16, torch.float32) == torch.float32


def test_random_weights_are_a_function_of_the_seed(tmp_path):
    cfg = config_from_dict(TINY_B)
    manifest = get_architecture(cfg.architecture).plan(cfg).manifest()
    a = random_tensors(manifest, 5, torch.float32)
    again = random_tensors(manifest, 5, torch.float32)
    c = random_tensors(manifest, 6, torch.float32)
    assert all(torch.equal(a[n], again[n]) for n in a)
    only = random_tensors([s for s in manifest if s.name == "model.norm.weight" or s.name.startswith("model.embed")],
                          5, torch.float32)
    assert set(only) == {"model.embed_tokens.weight", "model.norm.weight"}
    assert not torch.equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    emb = a["model.embed_tokens.weight"]
    assert abs(float(emb.std()) - 0.02) < 2e-3 and abs(float(emb.mean())) < 2e-3
    nw = a["model.layers.0.self_attn.q_norm.weight"]
    assert float(nw.min()) >= 0.9 and float(nw.max()) <= 1.1 and float(nw.std()) > 0.01


def test_model_folder(tmp_path):
    d = make_folder(tmp_path / "b", TINY_B, 1, "bfloat16")
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    cfg = json.load(open(os.path.join(d, "config.json")))
    assert cfg["architectures"] == ["Qwen3ForCausalLM"] and cfg["torch_dtype"] == "bfloat16"
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    assert f.info("lm_head.weight") == (torch.bfloat16, (384, 96))
    f.close()
    d2 = make_folder(tmp_path / "b2", TINY_B, 1, "bfloat16")
    assert open(os.path.join(d, "model.safetensors"), "rb").read() == open(os.path.join(d2, "model.safetensors"), "rb").read()


def test_sharded_folder(tmp_path):
    d = make_folder(tmp_path / "s", TINY_A, 0, "float32")
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    f.close()
    os.unlink(os.path.join(d, "model.safetensors"))
    names = list(tensors)
    half = len(names) // 2
    shards = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
    weight_map = {}
    for fname, ns in shards.items():
        write_safetensors(os.path.join(d, fname), {n: tensors[n] for n in ns})
        weight_map.update({n: fname for n in ns})
    json.dump({"weight_map": weight_map}, open(os.path.join(d, "model.safetensors.index.json"), "w"))
    cfg = config_from_dict(TINY_A)
    w = load_tensors(d, get_architecture(cfg.architecture).plan(cfg).manifest(), torch.float32, "cpu")
    assert all(torch.equal(w[n], tensors[n]) for n in names)


def test_command_line_writes_a_random_model_folder(tmp_path, capsys):
    """``qw-cli --random <config.json> --seed N --save <folder>``: a folder from a configuration and a seed, the same numbers
    as ``write_model_folder`` with that seed, without a GPU."""
    import json
    from questwend_b200 import cli
    cfg_path = tmp_path / "b.json"
    cfg_path.write_text(json.dumps(TINY_B))
    out = tmp_path / "from_cli"
    assert cli.main(["--random", str(cfg_path), "--seed", "3", "--save", str(out), "--dtype", "float32"]) == 0
    assert capsys.readouterr().out.strip() == str(out)
    other = make_folder(tmp_path / "direct", TINY_B, 3, "float32")
    a, b = SafetensorsFile(str(out / "model.safetensors")), SafetensorsFile(other + "/model.safetensors")
    assert sorted(a.names()) == sorted(b.names()) and all(torch.equal(a.tensor(k), b.tensor(k)) for k in a.names())
    assert json.loads((out / "config.json").read_text())["num_hidden_layers"] == 3
    with pytest.raises(SystemExit, match="either -m"):
        cli.main(["--seed", "3"])
    with pytest.raises(SystemExit, match="--save goes with --random"):
        cli.main(["-m", other, "--save", str(out)])
