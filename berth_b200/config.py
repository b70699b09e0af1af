"""``config.json`` of an EXL3 checkpoint: the host-side mirror of berth's ``ModelConfig`` / ``QuantizationConfig``
(crates/berth-exl3/src/config.rs:6-160).

Text-stack fields are read from ``text_config`` when that object holds the key, otherwise from the top level;
``architectures`` and ``quantization_config`` are always top-level; unknown keys are ignored; integers may be written
as integer-valued floats (``6.0``).  A failure raises :class:`~berth_b200.checkpoint.CheckpointError` with berth's
wording: ``missing field `name``` or ``field `name`: detail`` (crates/berth-exl3/src/error.rs:6-13).  Pure host logic;
the kernels take shapes and bitrates from the tensors, this is what an engine sizes its layers from (hidden size, MoE
dimensions, layer kinds, head bitrate).
"""
from __future__ import annotations

import dataclasses
import json
import math
import os

from .checkpoint import CheckpointError

U32_MAX = 0xFFFFFFFF


@dataclasses.dataclass(frozen=True)
class Calibration:
    """``quantization_config.calibration`` (config.rs:16-23)."""
    rows: int
    cols: int


@dataclasses.dataclass(frozen=True)
class QuantizationConfig:
    """config.rs:25-50.  ``codebook`` is the conversion-wide setting; each linear's codebook comes from its tensors."""
    quant_method: str
    bits: float
    head_bits: int
    codebook: str | None
    version: str | None
    vision_bits: int | None
    mtp_bits: int | None
    out_scales: str | None
    calibration: Calibration | None


@dataclasses.dataclass(frozen=True)
class ModelConfig:
    """config.rs:52-103.  ``layer_types`` holds ``"linear_attention"``, ``"full_attention"`` or any other string as
    written (berth's ``LayerType::Other``)."""
    arch_string: str
    num_hidden_layers: int
    hidden_size: int
    intermediate_size: int | None
    head_dim: int
    num_attention_heads: int
    num_key_value_heads: int
    vocab_size: int
    tie_word_embeddings: bool
    layer_types: tuple
    linear_conv_kernel_dim: int
    linear_num_key_heads: int
    linear_num_value_heads: int
    linear_key_head_dim: int
    linear_value_head_dim: int
    attn_output_gate: bool
    num_experts: int | None
    num_experts_per_tok: int | None
    moe_intermediate_size: int | None
    shared_expert_intermediate_size: int | None
    quantization: QuantizationConfig

    @property
    def is_moe(self) -> bool:
        return self.num_experts is not None

    @staticmethod
    def from_bytes(data: bytes) -> "ModelConfig":
        try:
            value = json.loads(data)
        except ValueError as e:
            raise CheckpointError(f"config.json: {e}") from None
        return ModelConfig.from_value(value)

    @staticmethod
    def from_directory(directory: str) -> "ModelConfig":
        path = os.path.join(directory, "config.json")
        try:
            with open(path, "rb") as f:
                data = f.read()
        except OSError as e:
            raise CheckpointError(f"{path}: {e.strerror}") from None
        return ModelConfig.from_bytes(data)

    @staticmethod
    def from_value(value) -> "ModelConfig":
        if not isinstance(value, dict):
            raise _bad("config.json", "expected a JSON object")
        root = value
        text = root.get("text_config")
        if text is not None and not isinstance(text, dict):
            raise _bad("text_config", f"expected an object, got {_describe(text)}")
        arch = _arch_string(root)
        layers = _u32(_require(root, text, "num_hidden_layers"), "num_hidden_layers")
        layer_types = _layer_types(_require(root, text, "layer_types"))
        if len(layer_types) != layers:
            raise _bad("layer_types", f"length {len(layer_types)} does not match num_hidden_layers {layers}")
        if "quantization_config" not in root:
            raise _missing("quantization_config")
        req = lambda key: _u32(_require(root, text, key), key)
        opt = lambda key: None if _lookup(root, text, key) is _ABSENT else _u32(_lookup(root, text, key), key)
        return ModelConfig(
            arch_string=arch, num_hidden_layers=layers, hidden_size=req("hidden_size"),
            intermediate_size=opt("intermediate_size"), head_dim=req("head_dim"),
            num_attention_heads=req("num_attention_heads"), num_key_value_heads=req("num_key_value_heads"),
            vocab_size=req("vocab_size"), tie_word_embeddings=_bool(_require(root, text, "tie_word_embeddings"), "tie_word_embeddings"),
            layer_types=layer_types, linear_conv_kernel_dim=req("linear_conv_kernel_dim"),
            linear_num_key_heads=req("linear_num_key_heads"), linear_num_value_heads=req("linear_num_value_heads"),
            linear_key_head_dim=req("linear_key_head_dim"), linear_value_head_dim=req("linear_value_head_dim"),
            attn_output_gate=_bool(_require(root, text, "attn_output_gate"), "attn_output_gate"),
            num_experts=opt("num_experts"), num_experts_per_tok=opt("num_experts_per_tok"),
            moe_intermediate_size=opt("moe_intermediate_size"),
            shared_expert_intermediate_size=opt("shared_expert_intermediate_size"),
            quantization=_quant(root["quantization_config"]))


_ABSENT = object()


def _missing(field: str) -> CheckpointError:
    return CheckpointError(f"missing field `{field}`")


def _bad(field: str, detail: str) -> CheckpointError:
    return CheckpointError(f"field `{field}`: {detail}")


def _describe(v) -> str:
    """config.rs:381-391."""
    if v is None:
        return "null"
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, (int, float)):
        return json.dumps(v)
    if isinstance(v, str):
        return f"string {json.dumps(v)}" if len(v.encode()) < 64 else "a long string"
    if isinstance(v, list):
        return "an array"
    return "an object"


def _lookup(root: dict, text: dict | None, key: str):
    if text is not None and key in text:
        return text[key]
    return root.get(key, _ABSENT)


def _require(root: dict, text: dict | None, key: str):
    v = _lookup(root, text, key)
    if v is _ABSENT:
        raise _missing(key)
    return v


def _u32(v, field: str) -> int:
    """Integers, or floats that are exactly an integer (config.rs:360-379)."""
    if isinstance(v, int) and not isinstance(v, bool):
        if v >= 0:
            if v > U32_MAX:
                raise _bad(field, f"integer {v} does not fit in u32")
            return v
    elif isinstance(v, float) and math.isfinite(v) and v >= 0.0 and v == math.floor(v) and v <= U32_MAX:
        return int(v)
    raise _bad(field, f"expected a non-negative integer, got {_describe(v)}")


def _bool(v, field: str) -> bool:
    if not isinstance(v, bool):
        raise _bad(field, f"expected a bool, got {_describe(v)}")
    return v


def _string(v, field: str) -> str:
    if not isinstance(v, str):
        raise _bad(field, f"expected a string, got {_describe(v)}")
    return v


def _arch_string(root: dict) -> str:
    if "architectures" not in root:
        raise _missing("architectures")
    v = root["architectures"]
    if not isinstance(v, list):
        raise _bad("architectures", f"expected an array, got {_describe(v)}")
    if not v:
        raise _bad("architectures", "expected a non-empty array")
    if not isinstance(v[0], str):
        raise _bad("architectures", f"expected a string, got {_describe(v[0])}")
    if not v[0]:
        raise _bad("architectures", "architecture string is empty")
    return v[0]


def _layer_types(v) -> tuple:
    if not isinstance(v, list):
        raise _bad("layer_types", f"expected an array, got {_describe(v)}")
    for item in v:
        if not isinstance(item, str):
            raise _bad("layer_types", f"expected strings, got {_describe(item)}")
    return tuple(v)


def _quant(v) -> QuantizationConfig:
    if not isinstance(v, dict):
        raise _bad("quantization_config", f"expected an object, got {_describe(v)}")

    def req(key, conv):
        if key not in v:
            raise _missing(key)
        return conv(v[key], key)

    def opt(key, conv):
        return conv(v[key], key) if key in v else None

    def number(x, key):
        if isinstance(x, bool) or not isinstance(x, (int, float)):
            raise _bad(key, f"expected a number, got {_describe(x)}")
        x = float(x)
        if not math.isfinite(x) or x < 0.0:
            raise _bad(key, f"expected a non-negative finite number, got {x}")
        return x

    calibration = None
    if "calibration" in v:
        c = v["calibration"]
        if not isinstance(c, dict):
            raise _bad("calibration", f"expected an object, got {_describe(c)}")
        for key in ("rows", "cols"):
            if key not in c:
                raise _missing(f"calibration.{key}")
        calibration = Calibration(_u32(c["rows"], "calibration.rows"), _u32(c["cols"], "calibration.cols"))
    return QuantizationConfig(quant_method=req("quant_method", _string), bits=req("bits", number), head_bits=req("head_bits", _u32),
                              codebook=opt("codebook", _string), version=opt("version", _string),
                              vision_bits=opt("vision_bits", _u32), mtp_bits=opt("mtp_bits", _u32),
                              out_scales=opt("out_scales", _string), calibration=calibration)
