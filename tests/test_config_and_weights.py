"""Configuration, registry, safetensors io, weight binding errors, random-weights mode."""
import json
import os
import struct

import pytest
import torch

from arle_b200.config import (ConfigError, Qwen3Config, UnknownArchitecture, config_from_dict, load_config,
                              registered_architectures)
from arle_b200.parts import DecoderModel, declared_weights
from arle_b200.weights import (SafetensorsError, SafetensorsFile, WeightError, load_weights, random_tensors,
                               write_random_model, write_safetensors)
from tiny_models import CONFIGS, TINY_A, TINY_B, TINY_C, make_model_dir


def test_qwen3_config_reads_every_size_from_keys():
    c = Qwen3Config.from_dict(TINY_B)
    assert (c.hidden_size, c.intermediate_size, c.num_hidden_layers) == (96, 176, 3)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (6, 1, 32)
    assert (c.vocab_size, c.rms_norm_eps, c.rope_theta, c.tie_word_embeddings) == (500, 1e-5, 1e6, False)
    assert c.max_position_embeddings == 1024 and c.stop_token_ids == (3,) and c.layer_windows == (None,) * 3


def test_aliases_and_defaults():
    d = dict(TINY_A)
    d["num_kv_heads"] = d.pop("num_key_value_heads")
    d["context_length"] = d.pop("max_position_embeddings")
    d.pop("head_dim")
    c = Qwen3Config.from_dict(d)
    assert c.num_key_value_heads == 2 and c.max_position_embeddings == 512 and c.head_dim == 64 // 4


@pytest.mark.parametrize("key", ["hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                                 "num_key_value_heads", "vocab_size", "rms_norm_eps", "rope_theta",
                                 "tie_word_embeddings", "max_position_embeddings"])
def test_missing_required_key_is_named(key):
    d = dict(TINY_A)
    d.pop(key)
    with pytest.raises(ConfigError, match=key):
        Qwen3Config.from_dict(d)


@pytest.mark.parametrize("patch,word", [({"num_key_value_heads": 3}, "multiple"), ({"head_dim": 15}, "even"),
                                        ({"attention_bias": True}, "attention_bias"),
                                        ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"),
                                        ({"hidden_act": "gelu"}, "hidden_act"), ({"hidden_size": 0}, "hidden_size"),
                                        ({"rms_norm_eps": -1}, "rms_norm_eps"),
                                        ({"layer_types": ["full_attention"]}, "layer_types"),
                                        ({"layer_types": ["sliding_attention", "full_attention"]}, "sliding_window")])
def test_invalid_values_are_refused(patch, word):
    with pytest.raises(ConfigError, match=word):
        Qwen3Config.from_dict(dict(TINY_A, **patch))


def test_window_layers_from_keys():
    assert Qwen3Config.from_dict(TINY_C).layer_windows == (None, None, 21, 21)
    d = dict(TINY_A, sliding_window=9, layer_types=["sliding_attention", "full_attention"])
    assert Qwen3Config.from_dict(d).layer_windows == (9, None)
    assert Qwen3Config.from_dict(dict(TINY_A, sliding_window=9)).layer_windows == (None, None)   # use_sliding_window off


def test_generation_config_stop_ids(tmp_path):
    d = make_model_dir("A", root=str(tmp_path))
    with open(os.path.join(d, "generation_config.json"), "w") as f:
        json.dump({"eos_token_id": [7, 9]}, f)
    assert load_config(d).stop_token_ids == (7, 9)


def test_registry():
    assert "Qwen3ForCausalLM" in registered_architectures()
    assert isinstance(config_from_dict(TINY_A), Qwen3Config)
    with pytest.raises(UnknownArchitecture, match="Qwen3ForCausalLM"):
        config_from_dict(dict(TINY_A, architectures=["LlamaForCausalLM"]))
    with pytest.raises(UnknownArchitecture):
        config_from_dict({k: v for k, v in TINY_A.items() if k != "architectures"})


def test_model_spec_has_no_sizes_of_its_own():
    for cfg in CONFIGS.values():
        c = config_from_dict(cfg)
        spec = c.to_model_spec()
        decls = {d.name: d.shape for d in declared_weights(spec)}
        nq, nkv, hd, H, I = (cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                             cfg["hidden_size"], cfg["intermediate_size"])
        assert decls["model.layers.0.self_attn.q_proj.weight"] == (nq * hd, H)
        assert decls["model.layers.0.self_attn.k_proj.weight"] == (nkv * hd, H)
        assert decls["model.layers.0.self_attn.o_proj.weight"] == (H, nq * hd)
        assert decls["model.layers.0.mlp.down_proj.weight"] == (H, I)
        assert decls["model.layers.0.self_attn.q_norm.weight"] == (hd,)
        assert ("lm_head.weight" in decls) == (not cfg["tie_word_embeddings"])
        assert len(decls) == 11 * cfg["num_hidden_layers"] + 2 + (0 if cfg["tie_word_embeddings"] else 1)


def test_safetensors_roundtrip_and_library_agreement(tmp_path):
    from safetensors.torch import load_file

    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int64),
         "c": torch.randn(2, 2, 2), "d": torch.zeros(0, 4)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t, {"k": "v"})
    f = SafetensorsFile(p)
    theirs = load_file(p)
    assert sorted(f.names()) == sorted(t) and f.metadata == {"k": "v"}
    for k in t:
        assert torch.equal(f.tensor(k), t[k]) and torch.equal(theirs[k], t[k])


def test_safetensors_malformed(tmp_path):
    p = str(tmp_path / "bad.safetensors")
    with open(p, "wb") as f:
        f.write(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(p)
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", len(hdr)) + hdr + b"\x00" * 8)
    with pytest.raises(SafetensorsError, match="truncated"):
        SafetensorsFile(p)
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 12]}}).encode()
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", len(hdr)) + hdr + b"\x00" * 16)
    with pytest.raises(SafetensorsError, match="needs 16 bytes"):
        SafetensorsFile(p)
    hdr = json.dumps({"a": {"dtype": "Q4", "shape": [4], "data_offsets": [0, 4]}}).encode()
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", len(hdr)) + hdr + b"\x00" * 4)
    with pytest.raises(SafetensorsError, match="unknown dtype"):
        SafetensorsFile(p)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = make_model_dir("B", root=str(tmp_path))
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    t = {n: f.tensor(n).clone() for n in f.names()}
    del t["model.layers.1.mlp.up_proj.weight"], t["model.norm.weight"]
    t["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 96, dtype=torch.bfloat16)
    t["model.layers.9.extra.weight"] = torch.zeros(1)
    write_safetensors(os.path.join(d, "model.safetensors"), t)
    spec = load_config(d).to_model_spec()
    with pytest.raises(WeightError) as e:
        load_weights(d, declared_weights(spec), spec.ignored_tensors)
    msg = str(e.value)
    assert sorted(e.value.missing) == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.value.unexpected == ["model.layers.9.extra.weight"]
    assert e.value.wrong_shape == [("model.layers.0.self_attn.k_proj.weight", (32, 96), (16, 96))]
    for word in ("missing (2)", "unexpected (1)", "wrong shape", "expected [32, 96], got [16, 96]"):
        assert word in msg


def test_kept_precisions_and_tied_head(tmp_path):
    d = make_model_dir("A", root=str(tmp_path))
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    t = {n: f.tensor(n).clone() for n in f.names()}
    t["model.norm.weight"] = t["model.norm.weight"].float()           # stored in 32-bit: stays so
    t["model.layers.0.mlp.up_proj.weight"] = t["model.layers.0.mlp.up_proj.weight"].half()
    t["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)   # present though tied: ignored
    write_safetensors(os.path.join(d, "model.safetensors"), t)
    spec = load_config(d).to_model_spec()
    w = load_weights(d, declared_weights(spec), spec.ignored_tensors)
    assert w["model.norm.weight"].dtype == torch.float32
    assert w["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16
    assert w["model.embed_tokens.weight"].dtype == torch.bfloat16 and "lm_head.weight" not in w


def test_sharded_checkpoint(tmp_path):
    d = make_model_dir("A", root=str(tmp_path))
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    names = f.names()
    half = len(names) // 2
    wm = {}
    for i, part in enumerate((names[:half], names[half:])):
        fn = f"model-{i}.safetensors"
        write_safetensors(os.path.join(d, fn), {n: f.tensor(n).clone() for n in part})
        wm.update({n: fn for n in part})
    os.remove(os.path.join(d, "model.safetensors"))
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as fh:
        json.dump({"weight_map": wm}, fh)
    spec = load_config(d).to_model_spec()
    assert len(load_weights(d, declared_weights(spec))) == len(names)
    # a tensor stored in two shards is an error, named with both files
    write_safetensors(os.path.join(d, "model-1.safetensors"),
                      {n: f.tensor(n).clone() for n in names[half:] + names[:1]})
    with pytest.raises(WeightError) as e:
        load_weights(d, declared_weights(spec))
    assert names[0] in str(e.value) and "model-0.safetensors" in str(e.value) and "model-1.safetensors" in str(e.value)


def test_random_model_is_seeded_and_order_free(tmp_path):
    a = make_model_dir("B", seed=3, root=str(tmp_path / "1"))
    b = make_model_dir("B", seed=3, root=str(tmp_path / "2"))
    c = make_model_dir("B", seed=4, root=str(tmp_path / "3"))
    fa, fb, fc = (SafetensorsFile(os.path.join(x, "model.safetensors")) for x in (a, b, c))
    for n in fa.names():
        assert torch.equal(fa.tensor(n), fb.tensor(n))
    assert not torch.equal(fa.tensor("lm_head.weight"), fc.tensor("lm_head.weight"))
    decls = declared_weights(load_config(a).to_model_spec())
    alone = random_tensors([d for d in decls if d.name == "lm_head.weight"], 3, 0.03, 0.2)
    assert torch.equal(alone["lm_head.weight"], fa.tensor("lm_head.weight"))
    g = fa.tensor("model.norm.weight").float()
    assert g.min() >= 0.8 - 1e-2 and g.max() <= 1.2 + 1e-2 and abs(fa.tensor("lm_head.weight").float().std() - 0.03) < 3e-3
    assert json.load(open(os.path.join(a, "config.json"))) == CONFIGS["B"]


def test_random_values_do_not_depend_on_the_device():
    """The generator is integer arithmetic on (seed, name, element index): chunks computed apart
    equal the whole, and (on a machine with a GPU) the GPU's values equal the CPU's bit for bit."""
    from arle_b200.weights import random_init as ri
    from arle_b200.parts.base import WeightDecl

    decls = [WeightDecl("w", (300, 70)), WeightDecl("g", (130,), init="gain")]
    whole = random_tensors(decls, 9, 0.02, 0.1)
    old = ri._CHUNK
    ri._CHUNK = 1000
    try:
        pieces = random_tensors(decls, 9, 0.02, 0.1)
    finally:
        ri._CHUNK = old
    assert all(torch.equal(whole[k], pieces[k]) for k in whole)
    w = random_tensors(decls[:1], 9, 1.0, 0.1, dtype=torch.float32)["w"].double()
    assert abs(w.mean()) < 0.02 and abs(w.std() - 1.0) < 0.02 and 2.7 < (w ** 4).mean() < 3.1 and w.abs().max() < 6.0
    if torch.cuda.is_available():
        gpu = random_tensors(decls, 9, 0.02, 0.1, device="cuda")
        assert all(torch.equal(whole[k], gpu[k].cpu()) for k in whole)


def test_command_line_writes_a_random_model_folder(tmp_path):
    """`python -m arle_b200 random-model`: a folder with config.json and model.safetensors that the
    loader accepts, the same bytes as the library call with the same seed."""
    import subprocess
    import sys
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(CONFIGS["A"]))
    out = tmp_path / "model"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "arle_b200", "random-model", "--config", str(cfg_path), "--seed", "5",
                        "--sigma", "0.02", "--gain-jitter", "0.1", "--out", str(out)], capture_output=True, text=True, cwd=root)
    assert r.returncode == 0, r.stderr
    ref = make_model_dir("A", seed=5, root=str(tmp_path / "lib"))
    fa, fb = SafetensorsFile(str(out / "model.safetensors")), SafetensorsFile(os.path.join(ref, "model.safetensors"))
    assert sorted(fa.names()) == sorted(fb.names())
    for n in fa.names():
        assert torch.equal(fa.tensor(n), fb.tensor(n))
    assert json.load(open(out / "config.json")) == CONFIGS["A"]


def test_model_build_maps_cache_layers_and_groups():
    m = DecoderModel(config_from_dict(TINY_C).to_model_spec())
    assert m.entry_cache_layer == [0, 1, 2, 3] and [n.window for n in m.cache_needs] == [None, None, 21, 21]
    assert m.state_needs == []
