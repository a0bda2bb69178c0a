"""Configuration keys, defaults and refusals; the registry; weight errors; random-weights mode."""
import json
import os
import struct

import pytest
import torch

import tiny_configs as tc
from geneinfer_b200.config import (ConfigError, LlamaConfig, known_architectures, parse_config, resolve_architecture)
from geneinfer_b200.weights import (SafetensorsError, SafetensorsFile, WeightsError, load_model_folder,
                                    write_random_model, write_safetensors)

MINIMAL = {"model_type": "llama", "hidden_size": 48, "intermediate_size": 80, "num_hidden_layers": 2,
           "num_attention_heads": 3, "vocab_size": 100}


def test_defaults_of_a_minimal_config():
    arch, cfg = parse_config(MINIMAL)
    assert arch.name == "LlamaForCausalLM" and isinstance(cfg, LlamaConfig)
    assert (cfg.num_key_value_heads, cfg.head_dim, cfg.max_position_embeddings) == (3, 16, 2048)
    assert (cfg.rope_theta, cfg.rms_norm_eps, cfg.rope_scaling, cfg.tie_word_embeddings) == (10000.0, 1e-6, None, False)
    nulls = dict(MINIMAL, num_key_value_heads=None, head_dim=None, rope_scaling=None, rms_norm_eps=None)
    assert parse_config(nulls)[1] == cfg                       # JSON null counts as absent


def test_both_tiny_configs_and_every_field():
    a, b = parse_config(tc.TINY_A)[1], parse_config(tc.TINY_B)[1]
    assert (a.attn_dim, a.kv_dim, b.attn_dim, b.kv_dim) == (64, 32, 96, 32)
    assert b.rope_scaling.factor == 32.0 and b.rope_scaling.original_max_position == 64
    assert a.tie_word_embeddings and not b.tie_word_embeddings
    spec = b.model_spec()
    assert len(spec.layers) == 3 and [e.layer for e in spec.schedule] == [0, 1, 2]
    m = spec.layers[0].mixer.params
    assert (m["num_heads"], m["num_kv_heads"], m["head_dim"]) == (3, 1, 32)
    assert spec.layers[0].mixer_norm.params["eps"] == 1e-6 and spec.final_norm.params["size"] == 96
    assert parse_config(json.loads(json.dumps(b.to_json())))[1] == b


@pytest.mark.parametrize("change,word", [
    ({"hidden_size": None}, "hidden_size"), ({"vocab_size": 0}, "vocab_size"), ({"num_hidden_layers": 2.5}, "num_hidden_layers"),
    ({"intermediate_size": 10 ** 9}, "intermediate_size"), ({"model_type": "gpt2", "architectures": ["LlamaForCausalLM"]}, "model_type"),
    ({"hidden_act": "gelu"}, "hidden_act"), ({"attention_bias": True}, "attention_bias"), ({"mlp_bias": True}, "mlp_bias"),
    ({"hidden_size": 50}, "divisible"), ({"num_key_value_heads": 2}, "divisible"), ({"head_dim": 15}, "even"),
    ({"rope_scaling": {"type": "linear", "factor": 2.0}}, "linear"), ({"rope_scaling": {"rope_type": "yarn"}}, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8.0}}, "low_freq_factor"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 0.5, "low_freq_factor": 1, "high_freq_factor": 4,
                       "original_max_position_embeddings": 64}}, "factor"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8, "low_freq_factor": 4, "high_freq_factor": 4,
                       "original_max_position_embeddings": 64}}, "low_freq_factor"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8, "low_freq_factor": 1, "high_freq_factor": 4,
                       "original_max_position_embeddings": 64.5}}, "integer"),
    ({"rope_scaling": 3}, "object"),
])
def test_refusals_name_the_key(change, word):
    with pytest.raises(ConfigError, match=word):
        parse_config(dict(MINIMAL, **change))


def test_registry_by_name_and_by_model_type():
    assert "LlamaForCausalLM" in known_architectures()
    assert resolve_architecture({"architectures": ["LlamaForCausalLM"]}).name == "LlamaForCausalLM"
    assert resolve_architecture({"model_type": "llama"}).name == "LlamaForCausalLM"
    with pytest.raises(ConfigError, match="Qwen3ForCausalLM.*known: .*LlamaForCausalLM"):
        resolve_architecture({"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3"})
    with pytest.raises(ConfigError, match="no known architecture"):
        resolve_architecture({"model_type": "mamba"})
    assert parse_config(dict(MINIMAL, rope_scaling={"type": "default"}))[1].rope_scaling is None


def test_random_weights_are_reproducible_and_independent_of_dtype(tmp_path):
    d1 = write_random_model(tc.TINY_B, 5, str(tmp_path / "one"), "float32")
    d2 = write_random_model(tc.TINY_B, 5, str(tmp_path / "two"), "bfloat16")
    d3 = write_random_model(tc.TINY_B, 6, str(tmp_path / "three"), "float32")
    _, cfg, p1 = load_model_folder(d1)
    _, _, p2 = load_model_folder(d2)
    _, _, p3 = load_model_folder(d3)
    assert cfg == parse_config(tc.TINY_B)[1]
    assert set(p1) == set(p2) and len(p1) == 3 * 6 + 3
    for k in p1:
        assert p1[k].dtype == torch.float32 and p2[k].dtype == torch.bfloat16      # stored precision is kept
        assert torch.equal(p1[k].to(torch.bfloat16), p2[k])                        # same draw, rounded when stored
    assert not torch.equal(p1["layers.0.mixer.w_o"], p3["layers.0.mixer.w_o"])
    assert p1["layers.1.mixer.w_qkv"].shape == (96 + 2 * 32, 96) and p1["layers.1.feed_forward.w_gate_up"].shape == (320, 96)
    assert abs(float(p1["embedding.weight"].std()) - 0.02) < 2e-3 and abs(float(p1["final_norm.weight"].mean()) - 1) < 0.02
    tied = load_model_folder(write_random_model(tc.TINY_A, 1, str(tmp_path / "tied"), "float32"))[2]
    assert tied["head.weight"] is tied["embedding.weight"]


def _rewrite(model_dir, edit):
    """Rewrites model.safetensors after ``edit(list of (name, tensor))``."""
    path = os.path.join(model_dir, "model.safetensors")
    with SafetensorsFile(path) as st:
        tensors = [(n, st.tensor(n)) for n in st.names()]
    write_safetensors(path, edit(tensors))


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = write_random_model(tc.TINY_A, 1, str(tmp_path / "m"), "float32")

    def edit(ts):
        out = []
        for n, t in ts:
            if n == "model.layers.1.mlp.up_proj.weight":
                continue                                                   # missing
            if n == "model.layers.0.self_attn.k_proj.weight":
                t = t[:, :32].contiguous()                                 # wrong shape
            if n == "model.norm.weight":
                t = t.to(torch.int32)                                      # wrong dtype
            out.append((n, t))
        out.append(("model.layers.0.self_attn.q_norm.weight", torch.ones(16)))          # unexpected
        out.append(("model.layers.0.self_attn.rotary_emb.inv_freq", torch.ones(8)))     # known to be unused: allowed
        out.append(("lm_head.weight", torch.zeros(256, 64)))                            # redundant in a tied model: allowed
        return out

    _rewrite(d, edit)
    with pytest.raises(WeightsError) as e:
        load_model_folder(d)
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.q_norm.weight"]
    assert len(err.wrong) == 2 and "[32, 32], expected [32, 64]" in str(err) and "I32" in str(err)
    assert "missing tensors (1)" in str(err) and "unexpected tensors (1)" in str(err)


def test_float16_is_widened_and_extras_that_are_known_are_ignored(tmp_path):
    d = write_random_model(tc.TINY_A, 1, str(tmp_path / "m"), "float32")
    before = load_model_folder(d)[2]["layers.0.mixer.w_o"]
    _rewrite(d, lambda ts: [(n, t.half() if "o_proj" in n else t) for n, t in ts] +
             [("model.layers.1.self_attn.rotary_emb.inv_freq", torch.ones(8))])
    after = load_model_folder(d)[2]["layers.0.mixer.w_o"]
    assert after.dtype == torch.float32 and torch.equal(after, before.half().float())


def test_broken_files_and_folders(tmp_path):
    d = write_random_model(tc.TINY_A, 1, str(tmp_path / "m"), "float32")
    path = os.path.join(d, "model.safetensors")
    blob = open(path, "rb").read()

    def broken(data, word):
        with open(path, "wb") as f:
            f.write(data)
        with pytest.raises(SafetensorsError, match=word):
            load_model_folder(d)

    broken(blob[:5], "too small")
    broken(struct.pack("<Q", len(blob) * 2) + blob[8:], "does not fit")
    broken(struct.pack("<Q", 200 * 1024 * 1024) + blob[8:], "does not fit")
    (n,) = struct.unpack("<Q", blob[:8])
    broken(blob[:8] + b"{" * n + blob[8 + n:], "invalid header JSON")
    broken(blob[:8 + n + 100], "outside the data region")
    header = json.loads(blob[8:8 + n])
    name = "model.norm.weight"
    header[name]["shape"] = [65]
    text = json.dumps(header).encode()
    broken(struct.pack("<Q", len(text)) + text + blob[8 + n:], "do not match shape")
    header[name] = 7
    text = json.dumps(header).encode()
    broken(struct.pack("<Q", len(text)) + text + blob[8 + n:], "not an object")
    os.remove(path)
    with pytest.raises(SafetensorsError, match="no model.safetensors"):
        load_model_folder(d)
    open(os.path.join(d, "model.safetensors.index.json"), "w").write("{}")
    with pytest.raises(SafetensorsError, match="weight_map"):
        load_model_folder(d)
    os.remove(os.path.join(d, "model.safetensors.index.json"))
    os.remove(os.path.join(d, "config.json"))
    with pytest.raises(ConfigError, match="no config.json"):
        load_model_folder(d)
    open(os.path.join(d, "config.json"), "w").write("{not json")
    with pytest.raises(ConfigError, match="config.json"):
        load_model_folder(d)


def test_checkpoint_in_several_files(tmp_path):
    """model.safetensors.index.json names the file of every tensor: the folder loads like the single
    file it was cut from; a file that is missing, a tensor that is not where the index puts it and
    a tensor nobody asked for are reported."""
    from geneinfer_b200.weights import write_safetensors
    single = tc.make_model_dir(tc.TINY_B, tc.WEIGHTS_B, str(tmp_path / "single"))
    want = load_model_folder(single)[2]
    st = SafetensorsFile(os.path.join(single, "model.safetensors"))
    names = st.names()
    d = tmp_path / "sharded"
    d.mkdir()
    (d / "config.json").write_text(open(os.path.join(single, "config.json")).read())
    files = ["model-00001-of-00003.safetensors", "model-00002-of-00003.safetensors", "model-00003-of-00003.safetensors"]
    weight_map = {}
    for k, f in enumerate(files):
        mine = names[k::3]
        write_safetensors(str(d / f), [(n, st.tensor(n)) for n in mine])
        weight_map.update({n: f for n in mine})
    index = d / "model.safetensors.index.json"
    index.write_text(json.dumps({"metadata": {"total_size": 1}, "weight_map": weight_map}))
    got = load_model_folder(str(d))[2]
    assert set(got) == set(want) and all(torch.equal(got[k], want[k]) and got[k].dtype == want[k].dtype for k in want)
    # a tensor that the index puts into the wrong file
    moved = dict(weight_map)
    moved[names[0]] = files[1]
    index.write_text(json.dumps({"weight_map": moved}))
    with pytest.raises(SafetensorsError, match="is not in model-00002"):
        load_model_folder(str(d))
    # a tensor that the index leaves out is missing for the configuration; one that a file holds beyond the plan is unexpected
    index.write_text(json.dumps({"weight_map": {n: f for n, f in weight_map.items() if n != names[3]}}))
    assert load_model_folder(str(d))[2].keys() == want.keys()        # still found: the file holds it
    write_safetensors(str(d / files[2]), [(n, st.tensor(n)) for n in names[2::3] if n != names[2]] + [("stray.weight", torch.zeros(3))])
    index.write_text(json.dumps({"weight_map": {n: f for n, f in weight_map.items() if n != names[2]}}))
    with pytest.raises(WeightsError) as e:
        load_model_folder(str(d))
    assert e.value.missing == [names[2]] and e.value.unexpected == ["stray.weight"]
    # a file of the index that is not there
    os.remove(d / files[0])
    index.write_text(json.dumps({"weight_map": weight_map}))
    with pytest.raises(SafetensorsError, match="cannot open"):
        load_model_folder(str(d))
    st.close()


def test_bench_says_that_it_runs_on_one_gpu():
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--gpus", "2", "--steps", "2", "--warmup", "1"],
                       capture_output=True, text=True, timeout=120)
    assert p.returncode == 2 and len(p.stdout.strip().splitlines()) == 1 and "one GPU" in p.stdout


def test_timeline_records_are_grouped_into_launches():
    """ops/timeline.py: time-ordered records of (kernel, event, block, ns) become launches (a kernel's launch ends where one
    of its blocks enters again), per block the first stamp of an event and, for leaving, the last warp's."""
    import numpy as np
    from geneinfer_b200.ops import timeline
    rec = np.array([
        [1, 0, 0, 0], [1, 0, 1, 10], [101, 0, 0, 20], [1, 1, 0, 100], [1, 1, 1, 110], [1, 6, 0, 200], [1, 6, 1, 210],
        [101, 1, 0, 300], [101, 2, 0, 350], [101, 6, 0, 400], [101, 6, 0, 450],      # two warps leave: the later one counts
        [1, 0, 0, 500], [1, 1, 0, 600], [1, 1, 0, 650], [1, 6, 0, 700],              # block 0 enters again: a new launch
    ], dtype=np.int64)
    found = timeline.launches(rec)
    assert [(l["kernel"], sorted(l["blocks"])) for l in found] == [(1, [0, 1]), (101, [0]), (1, [0])]
    assert found[0]["blocks"][1] == {0: 10, 1: 110, 6: 210}
    assert found[1]["blocks"][0] == {0: 20, 1: 300, 2: 350, 6: 450}
    assert found[2]["blocks"][0] == {0: 500, 1: 600, 6: 700}
    text = timeline.table(found, 0, 3).splitlines()
    assert len(text) == 3 and "rmsnorm" in text[0] and "2 blocks" in text[0] and "waited 0.10..0.11" in text[0]
    assert "product qkv+rope" in text[1] and "first operands 0.35..0.35" in text[1]
