"""Configuration, registry, safetensors container and weight errors (no GPU)."""
import json
import os
import struct

import pytest
import torch

import tiny
from cretif_b200.config import (ConfigError, LlamaConfig, ModelSpec, PartSpec, ScheduleEntry,
                                build_llama_spec, llama_config_from_dict, load_config,
                                register_architecture, registered_architectures,
                                resolve_architecture)
from cretif_b200.engine.model import manifest
from cretif_b200.weights import (CheckpointError, WeightSpec, load_weights, random_weights,
                                 read_header, read_tensors, write_model_folder, write_tensors)
from cretif_b200.weights.random_model import write_random_model


def test_llama_config_reads_its_keys():
    cfg = llama_config_from_dict(tiny.TINY_B)
    assert (cfg.hidden_size, cfg.num_hidden_layers, cfg.num_attention_heads) == (96, 3, 3)
    assert cfg.num_key_value_heads == 1 and cfg.head_dim == 32 and cfg.n_groups == 3
    assert cfg.q_dim == 96 and cfg.kv_dim == 32
    assert cfg.rms_norm_eps == 1e-6 and cfg.rope_theta == 100000.0
    assert cfg.eos_token_ids == [3, 5] and not cfg.tie_word_embeddings
    # defaults the reference uses when a key is absent
    raw = {k: v for k, v in tiny.TINY_A.items() if k not in ("rms_norm_eps", "rope_theta",
                                                             "num_key_value_heads")}
    cfg = llama_config_from_dict(raw)
    assert cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 10000.0
    assert cfg.num_key_value_heads == cfg.num_attention_heads
    # an explicit head size need not divide the width
    cfg = llama_config_from_dict(tiny.TINY_C)
    assert cfg.head_dim == 48 and cfg.q_dim == 240 and cfg.rope_interleaved
    # round trip through config.json
    assert llama_config_from_dict(cfg.to_dict()) == cfg


@pytest.mark.parametrize("patch,word", [
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"rope_scaling": {"type": "linear", "factor": 2.0}}, "rope_scaling"),
    ({"attention_bias": True}, "bias"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"vocab_size": 0}, "vocab_size"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"eos_token_id": 999}, "vocabulary"),
    ({"num_hidden_layers": "2"}, "integer"),
])
def test_llama_config_refuses(patch, word):
    with pytest.raises(ConfigError, match=word):
        llama_config_from_dict({**tiny.TINY_A, **patch})


def test_missing_keys_and_unknown_architecture(tmp_path):
    raw = dict(tiny.TINY_A)
    del raw["intermediate_size"]
    with pytest.raises(ConfigError, match="intermediate_size"):
        llama_config_from_dict(raw)
    with pytest.raises(ConfigError, match="registered"):
        resolve_architecture("NopeForCausalLM")
    assert "LlamaForCausalLM" in registered_architectures()
    (tmp_path / "config.json").write_text(json.dumps({"architectures": ["NopeForCausalLM"]}))
    with pytest.raises(ConfigError, match="NopeForCausalLM"):
        load_config(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="JSON"):
        load_config(str(tmp_path))
    with pytest.raises(ConfigError, match="no config.json"):
        load_config(str(tmp_path / "absent"))


def test_spec_is_data_and_validated():
    spec = build_llama_spec(llama_config_from_dict(tiny.TINY_A))
    assert len(spec.layers) == 2 and [e.layer for e in spec.schedule] == [0, 1]
    mixer, ffn = spec.layers[0].branches
    assert (mixer.role, mixer.part.kind, mixer.norm.kind) == ("mixer", "attention", "rmsnorm")
    assert (ffn.role, ffn.part.kind, ffn.post_norm) == ("feed_forward", "gated_mlp", None)
    assert mixer.part.params["position"]["pairing"] == "half"
    assert mixer.part.params["window"] == 0
    assert spec.head.params["tied"] is True
    # a schedule may visit a layer twice or borrow an earlier visit's cache
    spec.schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, cache=1)]
    spec.validate()
    spec.schedule = [ScheduleEntry(0), ScheduleEntry(5)]
    with pytest.raises(ValueError, match="layer 5"):
        spec.validate()
    spec.schedule = [ScheduleEntry(0, cache=0)]
    with pytest.raises(ValueError, match="earlier"):
        spec.validate()
    spec.schedule = [ScheduleEntry(0), ScheduleEntry(1, cache=0), ScheduleEntry(0, cache=1)]
    with pytest.raises(ValueError, match="borrows"):
        spec.validate()


def test_manifest_names_and_shapes():
    for name, raw in tiny.CONFIGS.items():
        cfg = llama_config_from_dict(raw)
        names, ignorable = manifest(build_llama_spec(cfg))
        L = cfg.num_hidden_layers
        assert len(names) == 9 * L + 2 + (0 if cfg.tie_word_embeddings else 1)
        assert names["model.embed_tokens.weight"].shape == (cfg.vocab_size, cfg.hidden_size)
        assert names["model.layers.0.self_attn.q_proj.weight"].shape == (cfg.q_dim, cfg.hidden_size)
        assert names["model.layers.0.self_attn.k_proj.weight"].shape == (cfg.kv_dim, cfg.hidden_size)
        assert names["model.layers.0.self_attn.o_proj.weight"].shape == (cfg.hidden_size, cfg.q_dim)
        assert names[f"model.layers.{L - 1}.mlp.down_proj.weight"].shape == (
            cfg.hidden_size, cfg.intermediate_size)
        assert names["model.norm.weight"].init == (1.0, 0.02)
        assert ("lm_head.weight" in names) == (not cfg.tie_word_embeddings)
        assert ignorable == ({"lm_head.weight"} if cfg.tie_word_embeddings else set())


def test_safetensors_round_trip_and_dtypes(tmp_path):
    path = str(tmp_path / "x.safetensors")
    tensors = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.randn(7),
               "c": torch.arange(6, dtype=torch.int64).reshape(2, 3),
               "d": torch.randn(2, 2).to(torch.float16)}
    write_tensors(path, tensors, metadata={"k": "v"})
    header, start = read_header(path)
    assert set(header) == set(tensors) and header["a"]["dtype"] == "BF16"
    back = read_tensors(path)
    for k in tensors:
        assert back[k].dtype == tensors[k].dtype and torch.equal(back[k], tensors[k])
    # the container is the common one: the safetensors library reads it too
    from safetensors import safe_open
    with safe_open(path, framework="pt") as f:
        assert torch.equal(f.get_tensor("a"), tensors["a"])
        assert f.metadata()["k"] == "v"
    assert set(read_tensors(path, ["b"])) == {"b"}


def test_safetensors_corruption_is_refused(tmp_path):
    path = str(tmp_path / "x.safetensors")
    write_tensors(path, {"a": torch.randn(4, 4)})
    data = open(path, "rb").read()
    open(path, "wb").write(data[:-8])                      # data reaches beyond the file
    with pytest.raises(CheckpointError, match="beyond the end"):
        read_header(path)
    open(path, "wb").write(data[:4])
    with pytest.raises(CheckpointError, match="too short"):
        read_header(path)
    open(path, "wb").write(struct.pack("<Q", 10 ** 12) + data[8:])
    with pytest.raises(CheckpointError, match="header length"):
        read_header(path)
    open(path, "wb").write(struct.pack("<Q", 8) + b"not json" + data)
    with pytest.raises(CheckpointError, match="JSON"):
        read_header(path)
    (n,) = struct.unpack("<Q", data[:8])
    hdr = json.loads(data[8:8 + n])
    hdr["a"]["shape"] = [4, 5]
    text = json.dumps(hdr).encode()
    open(path, "wb").write(struct.pack("<Q", len(text)) + text + data[8 + n:])
    with pytest.raises(CheckpointError, match="needs 80 bytes"):
        read_header(path)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = llama_config_from_dict(tiny.TINY_A)
    names, ignorable = manifest(build_llama_spec(cfg))
    tensors = random_weights(names, seed=1)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64, dtype=torch.bfloat16)
    tensors["model.layers.0.input_layernorm.weight"] = torch.zeros(64, dtype=torch.int32)
    write_model_folder(str(tmp_path), cfg.to_dict(), tensors)
    with pytest.raises(CheckpointError) as e:
        load_weights(str(tmp_path), names, ignorable)
    msg = str(e.value)
    assert "missing tensors (2)" in msg and "model.norm.weight" in msg
    assert "model.layers.1.mlp.up_proj.weight" in msg
    assert "unexpected tensors (1)" in msg and "inv_freq" in msg
    assert "wrong shapes or types (2)" in msg
    assert "k_proj.weight: expected [32, 64], file has [16, 64]" in msg
    assert "input_layernorm.weight: expected a floating tensor" in msg


def test_loader_keeps_stored_dtypes_and_ignores_a_tied_head(tmp_path):
    cfg = llama_config_from_dict(tiny.TINY_A)
    names, ignorable = manifest(build_llama_spec(cfg))
    tensors = random_weights(names, seed=2)
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float()      # stored in 32-bit
    tensors["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)    # unused when tied
    write_model_folder(str(tmp_path), cfg.to_dict(), tensors)
    got = load_weights(str(tmp_path), names, ignorable)
    assert got["model.norm.weight"].dtype == torch.float32
    assert got["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert "lm_head.weight" not in got
    with pytest.raises(CheckpointError, match="no model.safetensors"):
        load_weights(str(tmp_path / "nowhere"), names)


def test_sharded_checkpoint(tmp_path):
    cfg = llama_config_from_dict(tiny.TINY_A)
    names, ignorable = manifest(build_llama_spec(cfg))
    tensors = random_weights(names, seed=3)
    keys = sorted(tensors)
    shards = {"model-1.safetensors": keys[::2], "model-2.safetensors": keys[1::2]}
    weight_map = {}
    for fname, ks in shards.items():
        write_tensors(str(tmp_path / fname), {k: tensors[k] for k in ks})
        weight_map.update({k: fname for k in ks})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    got = load_weights(str(tmp_path), names, ignorable)
    assert all(torch.equal(got[k], tensors[k]) for k in keys)


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    write_random_model(str(tmp_path / "m"), tiny.TINY_B, seed=7)
    write_random_model(str(tmp_path / "n"), tiny.TINY_B, seed=7)
    write_random_model(str(tmp_path / "o"), tiny.TINY_B, seed=8, dtype=torch.float32)
    _, cfg, spec = load_config(str(tmp_path / "m"))
    names, ign = manifest(spec)
    a = load_weights(str(tmp_path / "m"), names, ign)
    b = load_weights(str(tmp_path / "n"), names, ign)
    c = load_weights(str(tmp_path / "o"), names, ign)
    assert all(torch.equal(a[k], b[k]) for k in a)                 # the seed decides
    assert not torch.equal(a["lm_head.weight"].float(), c["lm_head.weight"])
    assert c["lm_head.weight"].dtype == torch.float32 and a["lm_head.weight"].dtype == torch.bfloat16
    w = c["model.layers.0.mlp.gate_proj.weight"]
    assert abs(w.mean().item()) < 2e-3 and abs(w.std().item() - 0.02) < 2e-3
    n = c["model.norm.weight"]
    assert abs(n.mean().item() - 1.0) < 1e-2
    # a tensor's values do not depend on which other tensors the model has
    sub = random_weights({"lm_head.weight": names["lm_head.weight"]}, seed=7)
    assert torch.equal(sub["lm_head.weight"], a["lm_head.weight"])


def test_registering_another_architecture():
    def from_dict(raw):
        return llama_config_from_dict({**raw, "architectures": ["LlamaForCausalLM"]})

    def build(cfg):
        spec = build_llama_spec(cfg)
        spec.architecture = "TwiceLlama"
        spec.schedule = spec.schedule + spec.schedule        # every layer runs twice
        return spec
    register_architecture("TwiceLlama", from_dict, build)
    arch = resolve_architecture("TwiceLlama")
    spec = arch.build_spec(arch.config_from_dict(tiny.TINY_A))
    spec.validate()
    assert len(spec.schedule) == 4 and len(spec.layers) == 2
