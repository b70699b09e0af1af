"""``config.json`` reader against the cases of berth's own tests (crates/berth-exl3/src/config.rs:393-550)."""
import copy
import json

import pytest

from berth_b200.checkpoint import CheckpointError
from berth_b200.config import Calibration, ModelConfig


def sample() -> dict:
    return {
        "architectures": ["Qwen3_5ForConditionalGeneration", "Ignored"],
        "unused_top": 1,
        "tie_word_embeddings": True,
        "text_config": {
            "num_hidden_layers": 2, "hidden_size": 32, "head_dim": 16, "num_attention_heads": 4, "num_key_value_heads": 2,
            "vocab_size": 128, "tie_word_embeddings": False, "layer_types": ["linear_attention", "full_attention"],
            "linear_conv_kernel_dim": 4, "linear_num_key_heads": 16, "linear_num_value_heads": 48, "linear_key_head_dim": 128,
            "linear_value_head_dim": 128, "attn_output_gate": True, "future_field": "ignored"},
        "quantization_config": {
            "quant_method": "exl3", "version": "1.5.0", "bits": 4.0, "head_bits": 6, "codebook": "mul1", "vision_bits": 6,
            "mtp_bits": 4, "out_scales": "always", "calibration": {"rows": 250, "cols": 2048},
            "original_quantization_config": {"quant_method": "other"}},
    }


def test_reads_text_config_ahead_of_the_top_level():
    cfg = ModelConfig.from_bytes(json.dumps(sample()).encode())
    assert cfg.arch_string == "Qwen3_5ForConditionalGeneration"
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.head_dim) == (2, 32, 16)
    assert cfg.tie_word_embeddings is False
    assert cfg.intermediate_size is None and cfg.num_experts is None and not cfg.is_moe
    assert cfg.layer_types == ("linear_attention", "full_attention")
    assert cfg.linear_num_value_heads == 48 and cfg.attn_output_gate is True
    q = cfg.quantization
    assert (q.quant_method, q.bits, q.head_bits, q.codebook, q.vision_bits) == ("exl3", 4.0, 6, "mul1", 6)
    assert q.calibration == Calibration(250, 2048)


def test_falls_back_to_the_top_level_per_field():
    value = sample()
    del value["text_config"]["tie_word_embeddings"]
    assert ModelConfig.from_value(value).tie_word_embeddings is True
    bare = sample()
    text = bare.pop("text_config")
    bare.update(text)
    cfg = ModelConfig.from_value(bare)
    assert cfg.hidden_size == 32 and cfg.tie_word_embeddings is False


@pytest.mark.parametrize("key", ["head_dim", "attn_output_gate", "layer_types", "linear_conv_kernel_dim"])
def test_missing_required_field_names_the_field(key):
    value = sample()
    del value["text_config"][key]
    with pytest.raises(CheckpointError, match=f"missing field `{key}`"):
        ModelConfig.from_value(value)


def test_missing_quantization_config():
    value = sample()
    del value["quantization_config"]
    with pytest.raises(CheckpointError, match="quantization_config"):
        ModelConfig.from_value(value)


def test_optional_moe_and_other_layer_type():
    value = sample()
    value["text_config"].update({"intermediate_size": 17408, "num_experts": 256, "num_experts_per_tok": 8,
                                 "moe_intermediate_size": 512, "shared_expert_intermediate_size": 512,
                                 "layer_types": ["linear_attention", "qsa"]})
    cfg = ModelConfig.from_value(value)
    assert (cfg.intermediate_size, cfg.num_experts, cfg.num_experts_per_tok) == (17408, 256, 8)
    assert (cfg.moe_intermediate_size, cfg.shared_expert_intermediate_size) == (512, 512)
    assert cfg.layer_types[1] == "qsa" and cfg.is_moe


def test_layer_types_must_match_the_layer_count():
    value = sample()
    value["text_config"]["layer_types"] = ["full_attention"]
    with pytest.raises(CheckpointError, match="layer_types"):
        ModelConfig.from_value(value)


def test_empty_architectures_names_the_field():
    value = sample()
    value["architectures"] = []
    with pytest.raises(CheckpointError, match="architectures"):
        ModelConfig.from_value(value)


def test_integer_valued_float_counts_as_an_integer():
    value = sample()
    value["quantization_config"]["head_bits"] = 6.0
    assert ModelConfig.from_value(value).quantization.head_bits == 6


@pytest.mark.parametrize("path,bad,needle", [
    (("text_config", "hidden_size"), -1, "field `hidden_size`: expected a non-negative integer, got -1"),
    (("text_config", "hidden_size"), 2.5, "expected a non-negative integer, got 2.5"),
    (("text_config", "hidden_size"), 1 << 32, "does not fit in u32"),
    (("text_config", "attn_output_gate"), 1, "field `attn_output_gate`: expected a bool, got 1"),
    (("text_config", "layer_types"), "full_attention", 'field `layer_types`: expected an array, got string "full_attention"'),
    (("text_config", "layer_types"), [1, 2], "expected strings, got 1"),
    (("quantization_config", "bits"), "4", "field `bits`: expected a number"),
    (("quantization_config", "bits"), -1.0, "expected a non-negative finite number"),
    (("quantization_config", "quant_method"), 3, "field `quant_method`: expected a string, got 3"),
    (("quantization_config", "calibration"), [250, 2048], "field `calibration`: expected an object, got an array"),
    (("architectures",), "Qwen", "field `architectures`: expected an array"),
    (("architectures",), [""], "architecture string is empty"),
    (("text_config",), 7, "field `text_config`: expected an object, got 7"),
])
def test_wrong_types_name_the_field(path, bad, needle):
    value = copy.deepcopy(sample())
    node = value
    for key in path[:-1]:
        node = node[key]
    node[path[-1]] = bad
    with pytest.raises(CheckpointError) as e:
        ModelConfig.from_value(value)
    assert needle in str(e.value)


def test_not_json_and_not_an_object(tmp_path):
    with pytest.raises(CheckpointError, match="config.json"):
        ModelConfig.from_bytes(b"{not json")
    with pytest.raises(CheckpointError, match="expected a JSON object"):
        ModelConfig.from_value([1])
    with pytest.raises(CheckpointError, match="config.json"):
        ModelConfig.from_directory(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(sample()))
    assert ModelConfig.from_directory(str(tmp_path)).vocab_size == 128
