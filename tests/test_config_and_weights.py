"""Configuration, registry, safetensors round trip, and the loader's one clear error."""
import json

import pytest
import torch

import tiny_models
from dotllm_b200.config import (LlamaConfig, build_spec, config_from_dict, load_config,
                                register_architecture, registered_architectures)
from dotllm_b200.errors import ConfigError, WeightsError
from dotllm_b200.models.decoder import DecoderModel
from dotllm_b200.parts.base import Runtime
from dotllm_b200.weights import (SafetensorsFile, check_names_and_shapes, load_into, save_safetensors,
                                 write_random_model)

CPU = Runtime(torch.float32, torch.device("cpu"))


def test_llama_config_reads_its_keys_and_defaults():
    cfg = config_from_dict(tiny_models.TINY_B)
    assert isinstance(cfg, LlamaConfig)
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads,
            cfg.head_dim, cfg.intermediate_size, cfg.vocab_size) == (3, 192, 6, 6, 32, 512, 384)
    assert cfg.rope_scaling.factor == 8.0 and cfg.rope_scaling.original_max_position_embeddings == 64
    assert cfg.eos_token_id == (7, 9) and cfg.rms_norm_eps == 1e-6 and not cfg.tie_word_embeddings
    minimal = config_from_dict({"architectures": ["LlamaForCausalLM"], "vocab_size": 10, "hidden_size": 12,
                                "intermediate_size": 20, "num_hidden_layers": 1, "num_attention_heads": 3})
    assert minimal.num_key_value_heads == 3 and minimal.head_dim == 4          # defaults of the reference
    assert minimal.rms_norm_eps == 1e-5 and minimal.rope_theta == 10000.0
    assert minimal.max_position_embeddings == 2048 and minimal.rope_scaling is None
    assert config_from_dict(minimal.to_dict()) == minimal                       # round trip
    assert config_from_dict({"model_type": "llama", **{k: v for k, v in tiny_models.TINY_A.items()
                                                       if k != "architectures"}}).hidden_size == 64


@pytest.mark.parametrize("change,needle", [
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "unsupported rope_scaling"),
    ({"attention_bias": True}, "bias"),
    ({"vocab_size": None}, "vocab_size"),
    ({"num_hidden_layers": 0}, "positive"),
    ({"architectures": ["MambaForCausalLM"]}, "unknown architecture"),
])
def test_config_errors(change, needle):
    with pytest.raises(ConfigError, match=needle):
        config_from_dict({**tiny_models.TINY_A, **change})


def test_config_file_errors(tmp_path):
    with pytest.raises(ConfigError, match="no config.json"):
        load_config(tmp_path)
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        load_config(tmp_path)


def test_registry_takes_new_architectures():
    assert "LlamaForCausalLM" in registered_architectures()

    class OtherConfig(LlamaConfig):
        pass

    def build(cfg):
        from dotllm_b200.models.llama import build_llama_spec
        return build_llama_spec(cfg)

    register_architecture("OtherForCausalLM", OtherConfig, build)
    cfg = config_from_dict({**tiny_models.TINY_A, "architectures": ["OtherForCausalLM"]})
    assert type(cfg) is OtherConfig or isinstance(cfg, OtherConfig)
    assert len(build_spec(config_from_dict(tiny_models.TINY_A)).layers) == 2


def test_spec_schedule_is_validated():
    from dataclasses import replace
    from dotllm_b200.config.spec import ScheduleEntry
    spec = build_spec(config_from_dict(tiny_models.TINY_A))
    replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(1, cache_of=1))).validate()
    with pytest.raises(ConfigError):
        replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(5))).validate()
    with pytest.raises(ConfigError):
        replace(spec, schedule=(ScheduleEntry(0, cache_of=0),)).validate()
    with pytest.raises(ConfigError):
        replace(spec, schedule=(ScheduleEntry(0), ScheduleEntry(1, cache_of=0), ScheduleEntry(1, cache_of=1))).validate()


def test_safetensors_round_trip_and_dtypes(tmp_path):
    g = torch.Generator().manual_seed(0)
    tensors = {"a": torch.randn(3, 5, generator=g), "b": torch.randn(7, generator=g).to(torch.bfloat16),
               "c": torch.arange(6, dtype=torch.int64).view(2, 3), "d": torch.randn(2, 2, generator=g).to(torch.float16),
               "e": torch.zeros(0, 4)}
    path = tmp_path / "t.safetensors"
    save_safetensors(path, tensors, metadata={"k": "v"})
    with SafetensorsFile(path) as f:
        assert sorted(f.names()) == sorted(tensors) and f.metadata == {"k": "v"}
        for name, t in tensors.items():
            got = f.tensor(name).clone()
            assert got.dtype == t.dtype and torch.equal(got, t)
    import safetensors.torch as st                       # the format is the public one
    other = st.load_file(str(path))
    assert all(torch.equal(other[n], tensors[n]) for n in tensors)


def test_safetensors_rejects_broken_files(tmp_path):
    p = tmp_path / "x.safetensors"
    p.write_bytes(b"abc")
    with pytest.raises(WeightsError, match="too short"):
        SafetensorsFile(p)
    p.write_bytes((10 ** 9).to_bytes(8, "little") + b"{}")
    with pytest.raises(WeightsError, match="header length"):
        SafetensorsFile(p)
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 8)           # truncated data
    with pytest.raises(WeightsError, match="offsets"):
        SafetensorsFile(p)
    with pytest.raises(WeightsError, match="no model.safetensors"):
        from dotllm_b200.weights import open_model_files
        open_model_files(tmp_path / "nowhere")


def test_loader_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = tiny_models.make_folder(tmp_path, "A")
    with SafetensorsFile(folder / "model.safetensors") as f:
        tensors = {n: f.tensor(n).clone() for n in f.names()}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(64)
    tensors["model.layers.0.self_attn.k_proj.weight"] = torch.zeros(16, 64)
    save_safetensors(folder / "model.safetensors", tensors)
    model = DecoderModel(build_spec(load_config(folder)), CPU)
    with pytest.raises(WeightsError) as info:
        load_into(model, folder)
    msg = str(info.value)
    assert "model.layers.1.mlp.up_proj.weight" in msg and "model.norm.weight" in msg
    assert "model.layers.0.self_attn.q_proj.bias" in msg
    assert "model.layers.0.self_attn.k_proj.weight expected [32, 64] found [16, 64]" in msg
    assert info.value.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert info.value.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert not model.bound


def test_tied_and_untied_heads(tmp_path):
    a = tiny_models.make_folder(tmp_path, "A")
    with SafetensorsFile(a / "model.safetensors") as f:
        names = set(f.names())
        assert "lm_head.weight" not in names
        tensors = {n: f.tensor(n).clone() for n in names}
    model = load_into(DecoderModel(build_spec(load_config(a)), CPU), a)
    assert model.head.weight is model.embedding.table
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()   # a copy in the file is tolerated
    save_safetensors(a / "model.safetensors", tensors)
    load_into(DecoderModel(build_spec(load_config(a)), CPU), a)
    b = tiny_models.make_folder(tmp_path, "B")
    with SafetensorsFile(b / "model.safetensors") as f:
        tensors = {n: f.tensor(n).clone() for n in f.names()}
    del tensors["lm_head.weight"]
    save_safetensors(b / "model.safetensors", tensors)
    with pytest.raises(WeightsError, match="lm_head.weight"):
        load_into(DecoderModel(build_spec(load_config(b)), CPU), b)


def test_stored_precision_is_kept_and_roles_decide_the_compute_dtype(tmp_path):
    folder = tiny_models.make_folder(tmp_path, "A", dtype=torch.bfloat16)
    with SafetensorsFile(folder / "model.safetensors") as f:
        assert f.dtype_tag("model.layers.0.mlp.down_proj.weight") == "BF16"
        assert f.dtype_tag("model.layers.0.input_layernorm.weight") == "F32"     # gains stay 32-bit
    m = load_into(DecoderModel(build_spec(load_config(folder)), Runtime(torch.bfloat16, torch.device("cpu"))), folder)
    assert m.blocks[0].mixer.w_qkv.dtype == torch.bfloat16
    assert m.blocks[0].mixer_norm.gain.dtype == torch.float32
    m32 = load_into(DecoderModel(build_spec(load_config(folder)), CPU), folder)
    assert m32.blocks[0].mixer.w_qkv.dtype == torch.float32
    assert torch.equal(m32.blocks[0].mixer.w_qkv, m.blocks[0].mixer.w_qkv.float())


def test_random_weights_are_reproducible_and_as_declared(tmp_path):
    cfg = config_from_dict(tiny_models.TINY_A)
    a = write_random_model(tmp_path / "a", cfg, seed=5, dtype=torch.float32)
    b = write_random_model(tmp_path / "b", cfg, seed=5, dtype=torch.float32)
    c = write_random_model(tmp_path / "c", cfg, seed=6, dtype=torch.float32)
    assert (a / "model.safetensors").read_bytes() == (b / "model.safetensors").read_bytes()
    assert (a / "model.safetensors").read_bytes() != (c / "model.safetensors").read_bytes()
    assert load_config(a) == cfg
    with SafetensorsFile(a / "model.safetensors") as f:
        w = f.tensor("model.layers.0.mlp.gate_proj.weight").clone()
        g = f.tensor("model.norm.weight").clone()
    assert w.shape == (176, 64) and abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
    assert torch.equal(g, torch.ones(64))
    folder = tiny_models.make_folder(tmp_path, "A")
    with SafetensorsFile(folder / "model.safetensors") as f:
        g = f.tensor("model.norm.weight").clone()
    assert float(g.min()) >= 0.9 and float(g.max()) <= 1.1 and float(g.std()) > 0.01


def test_check_names_and_shapes_passes_when_all_is_well():
    from dotllm_b200.parts.base import WeightSpec
    check_names_and_shapes({"w": (2, 3), "extra": (1,)}, {"w": WeightSpec((2, 3))}, optional={"extra"})


def test_generation_config_names_the_stop_tokens(tmp_path):
    folder = tiny_models.make_folder(tmp_path, "A")                     # config.json: eos 2, bos 1
    assert load_config(folder).eos_token_id == (2,)
    (folder / "generation_config.json").write_text(json.dumps({"eos_token_id": [9, 2, 11], "bos_token_id": 5}))
    cfg = load_config(folder)
    assert cfg.eos_token_id == (9, 2, 11) and cfg.bos_token_id == 1     # its ids first, duplicates dropped; bos was given
    assert build_spec(cfg).stop_token_ids == (9, 2, 11)
    b = tiny_models.make_folder(tmp_path, "C")                          # no ids in config.json
    (b / "generation_config.json").write_text(json.dumps({"eos_token_id": 7, "bos_token_id": 3}))
    cfg = load_config(b)
    assert cfg.eos_token_id == (7,) and cfg.bos_token_id == 3
    (b / "generation_config.json").write_text("[1, 2")
    with pytest.raises(ConfigError, match="generation_config.json"):
        load_config(b)


def test_a_checkpoint_in_two_shards_loads_like_one_file(tmp_path):
    folder = tiny_models.make_folder(tmp_path, "B")
    whole = load_into(DecoderModel(build_spec(load_config(folder)), CPU), folder)
    with SafetensorsFile(folder / "model.safetensors") as f:
        tensors = {n: f.tensor(n).clone() for n in f.names()}
    names = sorted(tensors)
    first, second = names[:len(names) // 2], names[len(names) // 2:]
    save_safetensors(folder / "model-00001-of-00002.safetensors", {n: tensors[n] for n in first})
    save_safetensors(folder / "model-00002-of-00002.safetensors", {n: tensors[n] for n in second})
    index = {"metadata": {}, "weight_map": {**{n: "model-00001-of-00002.safetensors" for n in first},
                                            **{n: "model-00002-of-00002.safetensors" for n in second}}}
    (folder / "model.safetensors.index.json").write_text(json.dumps(index))
    (folder / "model.safetensors").unlink()
    sharded = load_into(DecoderModel(build_spec(load_config(folder)), CPU), folder)
    for (_, a), (_, b) in zip(whole.named_parts(), sharded.named_parts()):
        for name, value in vars(a).items():
            if isinstance(value, torch.Tensor):
                assert torch.equal(value, getattr(b, name)), name
    # a tensor that the second shard lacks is reported by name, as for a single file
    save_safetensors(folder / "model-00002-of-00002.safetensors", {n: tensors[n] for n in second[1:]})
    with pytest.raises(WeightsError) as info:
        load_into(DecoderModel(build_spec(load_config(folder)), CPU), folder)
    assert info.value.missing == [second[0]]
