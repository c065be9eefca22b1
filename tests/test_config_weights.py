"""Configuration, registry, weight loading errors and the random-weights mode (CPU)."""
import json
import os

import pytest
import torch

from infinilm_b200.config import (ConfigError, MiniCPM4Config, config_from_json, describe_model, load_config,
                                  lookup_architecture, register_architecture, unregister_architecture)
from infinilm_b200.models.causal_lm import CausalLM
from infinilm_b200.parts.position import longrope_choice, rotary_inv_freq
from infinilm_b200.weights import (DictSource, FolderSource, SafetensorsFile, WeightError, check_against,
                                   random_tensors, stored_precision, write_model_folder, write_safetensors)
from tiny_configs import TINY, tiny_a, tiny_b, tiny_c


def test_fields_come_from_config_json():
    for name, fn in TINY.items():
        raw = fn()
        cfg = config_from_json(raw)
        assert isinstance(cfg, MiniCPM4Config)
        assert cfg.hidden_size == raw["hidden_size"] and cfg.num_hidden_layers == raw["num_hidden_layers"]
        assert cfg.num_attention_heads == raw["num_attention_heads"] and cfg.num_key_value_heads == raw["num_key_value_heads"]
        assert cfg.head_dim == raw["head_dim"] and cfg.intermediate_size == raw["intermediate_size"]
        assert cfg.vocab_size == raw["vocab_size"] and cfg.rms_norm_eps == raw["rms_norm_eps"]
        assert cfg.scale_emb == raw["scale_emb"] and cfg.scale_depth == raw["scale_depth"]
        assert cfg.logit_scale == pytest.approx(raw["dim_model_base"] / raw["hidden_size"])
        assert cfg.residual_scale == pytest.approx(raw["scale_depth"] / raw["num_hidden_layers"] ** 0.5)


def test_defaults_and_derived():
    raw = tiny_a()
    del raw["head_dim"], raw["rope_theta"]
    raw["bias"] = True
    cfg = config_from_json(raw)
    assert cfg.head_dim == 16 and cfg.rope_theta == 10000.0
    assert cfg.attention_bias and cfg.mlp_bias and not cfg.attention_output_bias
    assert cfg.eos_token_ids == [2]
    assert config_from_json(tiny_b()).eos_token_ids == [1, 3]
    c = config_from_json(tiny_c())
    assert c.rotary_dim == 24 and c.torch_dtype == "bfloat16"
    raw = tiny_a()
    del raw["dim_model_base"]
    assert config_from_json(raw).logit_scale == 1.0


@pytest.mark.parametrize("key", ["hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                                 "intermediate_size", "vocab_size", "rms_norm_eps", "max_position_embeddings"])
def test_missing_required_key_is_named(key):
    raw = tiny_a()
    del raw[key]
    with pytest.raises(ConfigError, match=key):
        config_from_json(raw)


def test_bad_values():
    raw = tiny_a(); raw["hidden_size"] = "64"
    with pytest.raises(ConfigError, match="hidden_size"):
        config_from_json(raw)
    raw = tiny_a(); raw["num_key_value_heads"] = 3
    with pytest.raises(ConfigError, match="multiple"):
        config_from_json(raw)
    raw = tiny_a(); del raw["torch_dtype"]
    with pytest.raises(ConfigError, match="dtype"):
        config_from_json(raw)
    raw = tiny_a(); raw["quantization_config"] = {"quant_method": "awq"}
    with pytest.raises(ConfigError, match="quantiz"):
        config_from_json(raw)
    raw = tiny_b(); raw["rope_scaling"]["rope_type"] = "yarn"
    with pytest.raises(ConfigError, match="yarn"):
        config_from_json(raw)
    raw = tiny_b(); del raw["rope_scaling"]["long_factor"]
    with pytest.raises(ConfigError, match="long_factor"):
        config_from_json(raw)
    raw = tiny_b(); raw["rope_scaling"]["short_factor"] = [1.0] * 5
    with pytest.raises(ConfigError, match="entries"):
        config_from_json(raw)


def test_sizes_the_kernels_do_not_take_are_refused_when_the_model_is_built():
    """A head size that is no multiple of 16 (or beyond 256) is refused by the mixer with the size named, before any
    weight is read or any kernel runs."""
    for hd in (40, 8, 272):
        raw = tiny_a(); raw["head_dim"] = hd
        with pytest.raises(ValueError, match=f"head_dim {hd}"):
            CausalLM(describe_model(config_from_json(raw)), torch.bfloat16)
    raw = tiny_a(); raw["head_dim"] = 48                                   # steps of 16 are taken
    CausalLM(describe_model(config_from_json(raw)), torch.bfloat16)


def test_registry_lookup_and_unknown():
    assert lookup_architecture({"architectures": ["MiniCPMForCausalLM"]}).config_cls is MiniCPM4Config
    assert lookup_architecture({"model_type": "minicpm4"}).config_cls is MiniCPM4Config
    with pytest.raises(ConfigError, match="Unsupported model_type"):
        lookup_architecture({"architectures": ["LlamaForCausalLM"], "model_type": "llama"})
    with pytest.raises(ConfigError):
        lookup_architecture({})
    # another architecture registers without touching the framework
    arch = register_architecture(["ToyArch"], MiniCPM4Config, lambda c: None)
    assert lookup_architecture({"architectures": ["ToyArch"]}) is arch
    unregister_architecture("ToyArch")
    with pytest.raises(ConfigError):
        lookup_architecture({"architectures": ["ToyArch"]})


def test_model_description_is_data():
    cfg = config_from_json(tiny_b())
    spec = describe_model(cfg)
    assert len(spec.layers) == 3 and [s.layer for s in spec.order] == [0, 1, 2]
    assert spec.layers[0].mixer.kind == "attention" and spec.layers[0].ffn.kind == "swiglu"
    assert spec.layers[1].mixer.params["position"].kind == "longrope"
    assert describe_model(config_from_json(tiny_a())).layers[0].mixer.params["position"].kind == "rope"
    names = {p.full_name(ws.name) for p, ws in CausalLM(spec, torch.float32).weight_specs()}
    assert "model.layers.2.self_attn.k_proj.weight" in names and "lm_head.weight" in names and "model.norm.weight" in names
    assert len(names) == 1 + 3 * 9 + 1 + 1


def test_longrope_choice():
    f, m = longrope_choice([1.0] * 4, [2.0] * 4, 64, 256, None)
    assert f == [2.0] * 4 and m == pytest.approx((1 + __import__("math").log(4) / __import__("math").log(64)) ** 0.5)
    f, m = longrope_choice([1.0] * 4, [2.0] * 4, 64, 64, None)
    assert f == [1.0] * 4 and m == 1.0
    inv = rotary_inv_freq(8, 10000.0, [1.0, 2.0, 3.0, 4.0])
    assert inv[0] == 1.0 and inv[1] == pytest.approx(1 / (2 * 10000 ** 0.25))


# -- weights ----------------------------------------------------------------------------------
def _model(raw):
    cfg = config_from_json(raw)
    return cfg, CausalLM(describe_model(cfg), torch.float32)


def test_random_folder_roundtrip(tmp_path):
    cfg, model = _model(tiny_b())
    d = write_model_folder(cfg, 3, str(tmp_path / "m"))
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    cfg2 = load_config(d)
    assert cfg2.hidden_size == cfg.hidden_size and cfg2.rope_scaling.kind == "longrope"
    src = FolderSource(d)
    check_against(model, src)
    t = random_tensors(cfg, 3)
    for n in src.names():
        assert torch.equal(src.get(n), t[n]), n
    # seeded: the same seed gives the same tensors, another seed other ones; order does not matter
    assert torch.equal(random_tensors(cfg, 3)["model.norm.weight"], t["model.norm.weight"])
    assert not torch.equal(random_tensors(cfg, 4)["model.norm.weight"], t["model.norm.weight"])
    src.close()


def test_tied_head_has_no_tensor():
    cfg, model = _model(tiny_a())
    t = random_tensors(cfg, 0)
    assert "lm_head.weight" not in t
    check_against(model, DictSource(t))                      # the embedding stands in
    cfg_b, _ = _model(tiny_b())
    assert "lm_head.weight" in random_tensors(cfg_b, 0)


def test_one_error_lists_everything():
    cfg, model = _model(tiny_b())
    t = dict(random_tensors(cfg, 0))
    del t["model.layers.1.mlp.up_proj.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)
    t["model.layers.2.self_attn.q_proj.weight"] = torch.zeros(10, 192)
    t["model.layers.0.mlp.down_proj.weight"] = torch.zeros(192, 320, dtype=torch.int32)      # integers offered for a matrix
    t["model.layers.0.input_layernorm.weight"] = torch.ones(192, dtype=torch.int64)
    with pytest.raises(WeightError) as ei:
        check_against(model, DictSource(t))
    e = ei.value
    assert e.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert e.wrong_shape == [("model.layers.2.self_attn.q_proj.weight", (10, 192), (192, 192))]
    assert len(e.other) == 2 and all("wrong kind of numbers" in o for o in e.other)
    msg = str(e)
    for s in ("missing", "unexpected", "wrong shape", "up_proj", "inv_freq", "[10, 192]", "down_proj.weight is stored as torch.int32",
              "input_layernorm.weight is stored as torch.int64"):
        assert s in msg


def test_a_head_that_config_json_calls_untied_must_be_in_the_checkpoint():
    """An absent lm_head.weight is taken from the embedding table, as InfiniLM does - unless config.json says
    "tie_word_embeddings": false: then the checkpoint is incomplete and the error says so."""
    raw = tiny_b()
    assert raw["tie_word_embeddings"] is False
    cfg, model = _model(raw)
    t = dict(random_tensors(cfg, 0))
    del t["lm_head.weight"]
    with pytest.raises(WeightError) as ei:
        check_against(model, DictSource(t))
    assert ei.value.missing == ["lm_head.weight"]
    raw2 = dict(raw)
    del raw2["tie_word_embeddings"]                          # the key is absent: tied by absence of the tensor
    _, model2 = _model(raw2)
    check_against(model2, DictSource(t))


def test_stored_precision_rules():
    assert stored_precision(torch.zeros(2, dtype=torch.bfloat16), "matrix").dtype == torch.bfloat16
    assert stored_precision(torch.zeros(2, dtype=torch.float16), "matrix").dtype == torch.bfloat16
    assert stored_precision(torch.zeros(2, dtype=torch.float32), "vector").dtype == torch.float32
    assert stored_precision(torch.zeros(2, dtype=torch.float64), "vector").dtype == torch.float32
    assert stored_precision(torch.zeros(2, dtype=torch.int64), "table").dtype == torch.int32


def test_safetensors_reader_checks(tmp_path):
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, {"a": torch.arange(6, dtype=torch.float32).reshape(2, 3),
                          "b": torch.ones(4, dtype=torch.bfloat16), "c": torch.arange(3, dtype=torch.int64)})
    f = SafetensorsFile(p)
    assert sorted(f.names()) == ["a", "b", "c"]
    assert f.info("a") == (torch.float32, (2, 3)) and f.tensor("a")[1, 2] == 5
    assert f.tensor("b").dtype == torch.bfloat16 and f.tensor("c").tolist() == [0, 1, 2]
    f.close()
    # the same bytes through the safetensors package, if present
    try:
        from safetensors import safe_open
        with safe_open(p, "pt") as g:
            assert torch.equal(g.get_tensor("a"), torch.arange(6, dtype=torch.float32).reshape(2, 3))
    except ImportError:
        pass
    bad = str(tmp_path / "bad.safetensors")
    with open(bad, "wb") as fh:
        fh.write(b"\x10\x00\x00")
    with pytest.raises(IOError):
        SafetensorsFile(bad)
    os.makedirs(str(tmp_path / "empty"))
    with pytest.raises(IOError, match="no .safetensors"):
        FolderSource(str(tmp_path / "empty"))
