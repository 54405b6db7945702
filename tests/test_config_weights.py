"""Configuration parsing and refusals; weight loading errors; the random-weights mode."""
import json
import os
import struct

import pytest
import torch

from helpers import CONFIGS, TINY_A, TINY_B, make_model_dir


def test_qwen3_config_defaults_and_keys():
    from marin_b200.config import Qwen3Config

    cfg = Qwen3Config.from_dict(TINY_B)
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim) == (3, 96, 8, 2, 32)
    assert cfg.q_dim == 256 and cfg.kv_dim == 64 and cfg.rope_theta == 1e6 and cfg.rms_norm_eps == 1e-5
    assert not cfg.tie_word_embeddings
    raw = dict(TINY_A)
    del raw["num_key_value_heads"], raw["head_dim"]
    cfg = Qwen3Config.from_dict(raw)
    assert cfg.num_key_value_heads == 4 and cfg.head_dim == 16          # defaults: heads, hidden / heads
    # the published Qwen3-1.7B sizes give the published parameter count (crates/model/src/qwen3/config.rs tests)
    big = Qwen3Config.from_dict({"model_type": "qwen3", "hidden_size": 2048, "intermediate_size": 6144, "num_hidden_layers": 28,
                                 "num_attention_heads": 16, "num_key_value_heads": 8, "head_dim": 128, "vocab_size": 151936,
                                 "max_position_embeddings": 40960, "rms_norm_eps": 1e-6, "rope_theta": 1000000, "tie_word_embeddings": True})
    assert big.parameter_count() == 1_720_574_976


def test_eos_from_generation_config_wins():
    from marin_b200.config import Qwen3Config

    cfg = Qwen3Config.from_dict({**TINY_A, "eos_token_id": 7}, {"eos_token_id": [3, 4]})
    assert cfg.eos_token_ids == [3, 4] and cfg.eos_from_generation_config
    assert Qwen3Config.from_dict({**TINY_A, "eos_token_id": 7}).eos_token_ids == [7]


@pytest.mark.parametrize("change,needle", [
    ({"attention_bias": True}, "attention_bias"),
    ({"use_sliding_window": True}, "sliding window"),
    ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"),
    ({"rope_parameters": {"rope_theta": 1e4, "rope_type": "llama3"}}, "rope type"),
    ({"hidden_act": "gelu"}, "activation"),
    ({"model_type": "llama"}, "model_type"),
    ({"num_key_value_heads": 3}, "shared evenly"),
    ({"head_dim": 15}, "even"),
    ({"hidden_size": 0}, "above 0"),
    ({"rms_norm_eps": float("nan")}, "finite"),
    ({"rope_theta": None, "rope_parameters": None}, "rope_theta"),
    ({"vocab_size": None}, "vocab_size"),
    ({"num_hidden_layers": "2"}, "integer"),
])
def test_unsupported_and_broken_configs_are_refused(change, needle):
    from marin_b200.config import ConfigError, Qwen3Config

    with pytest.raises(ConfigError, match=needle):
        Qwen3Config.from_dict({**TINY_A, **change})


def test_registry_chooses_by_config_json(tmp_path):
    from marin_b200.config import ConfigError, load_config
    from marin_b200.models import registered

    assert "Qwen3ForCausalLM" in registered()
    d = make_model_dir(str(tmp_path / "m"), TINY_B, seed=1)
    assert type(load_config(d)).__name__ == "Qwen3Config"
    with open(os.path.join(d, "config.json"), "w") as fh:
        json.dump({"architectures": ["NopeForCausalLM"], "model_type": "nope"}, fh)
    with pytest.raises(ConfigError, match="registered"):
        load_config(d)


def test_spec_is_data_layer_by_layer():
    from marin_b200.config import Qwen3Config
    from marin_b200.models import Model, architecture_of

    cfg = Qwen3Config.from_dict(TINY_B)
    spec = architecture_of(cfg).build_spec(cfg)
    assert [e.layer for e in spec.schedule] == [0, 1, 2] and len(spec.layers) == 3
    assert spec.layers[1].mixer.kind == "gqa_attention" and spec.layers[1].feedforward.kind == "swiglu"
    assert spec.layers[2].mixer.params["head_dim"] == 32 and spec.layers[0].norm.params["eps"] == 1e-5
    names = {s.name: s.shape for s in Model(spec).tensor_specs()}
    assert names["model.layers.2.self_attn.q_proj.weight"] == (256, 96)
    assert names["model.layers.0.self_attn.k_norm.weight"] == (32,)
    assert names["lm_head.weight"] == (384, 96) and len(names) == 3 + 11 * 3


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    from marin_b200.config import Qwen3Config, load_config
    from marin_b200.models import Model, architecture_of
    from marin_b200.weights import load_tensors, write_random_model

    cfg = Qwen3Config.from_dict(TINY_A)
    d = write_random_model(str(tmp_path / "r"), cfg, seed=5)
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    again = load_config(d)
    assert again.head_dim == 16 and again.tie_word_embeddings
    model = Model(architecture_of(again).build_spec(again))
    tensors = load_tensors(d, model.tensor_specs(), model.spec.ignorable)
    assert all(t.dtype == torch.bfloat16 for t in tensors.values())
    w = tensors["model.layers.0.mlp.gate_proj.weight"].float()
    n = tensors["model.layers.1.input_layernorm.weight"].float()
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(n.mean()) - 1.0) < 0.03 and 0.02 < float(n.std()) < 0.08
    # same seed, same values; a tensor's values do not depend on the others; another seed differs
    d2 = write_random_model(str(tmp_path / "r2"), cfg, seed=5)
    t2 = load_tensors(d2, model.tensor_specs(), model.spec.ignorable)
    assert all(torch.equal(tensors[k], t2[k]) for k in tensors)
    d3 = write_random_model(str(tmp_path / "r3"), cfg, seed=6, dtype=torch.float32)
    t3 = load_tensors(d3, model.tensor_specs(), model.spec.ignorable)
    assert t3["model.norm.weight"].dtype == torch.float32            # stored in 32-bit, stays so
    assert not torch.equal(t3["model.norm.weight"], tensors["model.norm.weight"].float())
    # the safetensors library reads the same bytes
    from safetensors.torch import load_file
    lib = load_file(os.path.join(d, "model.safetensors"))
    assert all(torch.equal(lib[k], tensors[k]) for k in tensors)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    from marin_b200.config import Qwen3Config
    from marin_b200.models import Model, architecture_of
    from marin_b200.weights import WeightError, load_tensors, random_tensors, write_safetensors

    cfg = Qwen3Config.from_dict(TINY_B)
    model = Model(architecture_of(cfg).build_spec(cfg))
    d = str(tmp_path / "bad")
    os.makedirs(d)
    tensors = dict(random_tensors(cfg, 1))
    del tensors["model.layers.1.mlp.up_proj.weight"], tensors["lm_head.weight"]
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(96, 96, dtype=torch.bfloat16)
    tensors["model.layers.2.self_attn.k_norm.weight"] = tensors["model.layers.2.self_attn.k_norm.weight"].to(torch.float16)
    tensors["model.layers.7.extra.weight"] = torch.zeros(3, dtype=torch.bfloat16)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors.items())
    with pytest.raises(WeightError) as err:
        load_tensors(d, model.tensor_specs(), model.spec.ignorable)
    text = str(err.value)
    assert "5 problem(s)" in text
    assert "missing tensor `model.layers.1.mlp.up_proj.weight` [320, 96]" in text
    assert "missing tensor `lm_head.weight`" in text
    assert "`model.layers.0.self_attn.q_proj.weight` has shape [96, 96] but config.json implies [256, 96]" in text
    assert "`model.layers.2.self_attn.k_norm.weight` is F16" in text
    assert "unexpected tensor `model.layers.7.extra.weight` [3]" in text


def test_unknown_tensors_may_be_left_unread_on_request(tmp_path, capsys):
    """``extra_tensors="warn"``: tensors the model does not know are named once and skipped (the reference ignores
    them: crates/model/src/qwen3/weight_bytes.rs:9-10); what is missing or mis-shaped is an error all the same."""
    from marin_b200.config import Qwen3Config
    from marin_b200.models import Model, architecture_of
    from marin_b200.weights import WeightError, load_tensors, random_tensors, write_safetensors

    cfg = Qwen3Config.from_dict(TINY_A)
    model = Model(architecture_of(cfg).build_spec(cfg))
    d = str(tmp_path / "extras")
    os.makedirs(d)
    tensors = dict(random_tensors(cfg, 1))
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8, dtype=torch.float32)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors.items())
    with pytest.raises(WeightError, match="unexpected tensor `model.layers.0.self_attn.rotary_emb.inv_freq`"):
        load_tensors(d, model.tensor_specs(), model.spec.ignorable)
    ignored = []
    got = load_tensors(d, model.tensor_specs(), model.spec.ignorable, "warn", ignored)
    assert ignored == ["model.layers.0.self_attn.rotary_emb.inv_freq"] and ignored[0] not in got
    assert "1 tensor(s) the model does not know were left unread" in capsys.readouterr().err
    del tensors["model.norm.weight"]
    write_safetensors(os.path.join(d, "model.safetensors"), tensors.items())
    with pytest.raises(WeightError, match="1 problem"):
        load_tensors(d, model.tensor_specs(), model.spec.ignorable, "warn")
    with pytest.raises(ValueError, match="extra_tensors"):
        load_tensors(d, model.tensor_specs(), model.spec.ignorable, "ignore")


def test_a_shape_whose_product_overflows_is_refused(tmp_path):
    """A crafted header whose sizes multiply past 64 bits must not wrap around into a product that matches its bytes."""
    from marin_b200.weights import SafetensorsError
    from marin_b200.weights.safetensors_io import SafetensorsFile

    path = str(tmp_path / "overflow.safetensors")
    for shape in ([1 << 33, 1 << 33, 4], [1 << 59, 8], [3, 1 << 40], [1 << 32, 1 << 32]):
        header = json.dumps({"w": {"dtype": "F32", "shape": shape, "data_offsets": [0, 64]}}).encode()
        with open(path, "wb") as fh:
            fh.write(struct.pack("<Q", len(header)) + header + b"\0" * 64)
        with pytest.raises(SafetensorsError, match="more elements than the file has bytes"):
            SafetensorsFile(path)
    header = json.dumps({"w": {"dtype": "F32", "shape": [0, 1 << 59], "data_offsets": [0, 0]}}).encode()     # empty: fine
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(header)) + header)
    assert tuple(SafetensorsFile(path).tensors["w"].shape) == (0, 1 << 59)


def test_tied_model_may_carry_an_unused_head(tmp_path):
    from marin_b200.config import Qwen3Config
    from marin_b200.models import Model, architecture_of
    from marin_b200.weights import load_tensors, random_tensors, write_safetensors

    cfg = Qwen3Config.from_dict(TINY_A)
    model = Model(architecture_of(cfg).build_spec(cfg))
    d = str(tmp_path / "tied")
    os.makedirs(d)
    tensors = dict(random_tensors(cfg, 1))
    tensors["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors.items())
    assert "lm_head.weight" not in load_tensors(d, model.tensor_specs(), model.spec.ignorable)


def test_truncated_and_sharded_files(tmp_path):
    from marin_b200.config import Qwen3Config
    from marin_b200.models import Model, architecture_of
    from marin_b200.weights import SafetensorsError, load_tensors, random_tensors, write_safetensors

    cfg = Qwen3Config.from_dict(TINY_A)
    model = Model(architecture_of(cfg).build_spec(cfg))
    tensors = list(random_tensors(cfg, 1))
    d = str(tmp_path / "sharded")
    os.makedirs(d)
    half = len(tensors) // 2
    write_safetensors(os.path.join(d, "model-00001-of-00002.safetensors"), tensors[:half])
    write_safetensors(os.path.join(d, "model-00002-of-00002.safetensors"), tensors[half:])
    index = {"weight_map": {n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
                            for i, (n, _) in enumerate(tensors)}}
    json.dump(index, open(os.path.join(d, "model.safetensors.index.json"), "w"))
    got = load_tensors(d, model.tensor_specs(), model.spec.ignorable)
    assert all(torch.equal(got[n], t) for n, t in tensors)
    # a tensor in two shards
    write_safetensors(os.path.join(d, "model-00002-of-00002.safetensors"), tensors[half - 1:])
    with pytest.raises(SafetensorsError, match="in both"):
        load_tensors(d, model.tensor_specs(), model.spec.ignorable)
    # a partial download
    t = str(tmp_path / "trunc")
    os.makedirs(t)
    write_safetensors(os.path.join(t, "model.safetensors"), tensors)
    data = open(os.path.join(t, "model.safetensors"), "rb").read()
    open(os.path.join(t, "model.safetensors"), "wb").write(data[: len(data) - 100])
    with pytest.raises(SafetensorsError, match="partial download"):
        load_tensors(t, model.tensor_specs(), model.spec.ignorable)
    open(os.path.join(t, "model.safetensors"), "wb").write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="header"):
        load_tensors(t, model.tensor_specs(), model.spec.ignorable)
    with pytest.raises(SafetensorsError, match="neither"):
        load_tensors(str(tmp_path), model.tensor_specs(), model.spec.ignorable)
