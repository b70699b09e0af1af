"""``config.json`` of an EXL3 checkpoint: the host-side mirror of berth's ``ModelConfig`` / ``QuantizationConfig``
(crates/berth-exl3/src/config.rs:6-160).

Text-stack fields are read from ``text_config`` when that object holds the key, otherwise from the top level;
``architectures`` and ``quantization_config`` are always top-level; unknown keys are ignored; integers may be written
as integer-valued floats (``6.0``).  A failure raises :class:`~berth_b200.checkpoint.CheckpointError` with berth's
wording: ``missing field `name``` or ``field `name`: detail`` (crates/berth-exl3/src/error.rs:6-13).  The parsing runs in the
library (``berth_config_parse`` / ``berth_config_open`` of include/berth_b200_checkpoint.h, host memory only); the kernels
take shapes and bitrates from the tensors, this is what an engine sizes its layers from (hidden size, MoE dimensions,
layer kinds, head bitrate).
"""
from __future__ import annotations

import ctypes as C
import dataclasses
import json
import os

from . import _lib
from .checkpoint import CheckpointError


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
        """Parses ``config.json`` bytes with the library's reader (``berth_config_parse``)."""
        return _from_native(lambda out: _lib.lib().berth_config_parse(data, len(data), C.byref(out)))

    @staticmethod
    def from_directory(directory: str) -> "ModelConfig":
        return _from_native(lambda out: _lib.lib().berth_config_open(os.fsencode(directory), C.byref(out)))

    @staticmethod
    def from_value(value) -> "ModelConfig":
        """An already-decoded ``config.json`` value (serialised again for the library's reader)."""
        return ModelConfig.from_bytes(json.dumps(value).encode())


def _from_native(call) -> ModelConfig:
    out = C.POINTER(_lib.ModelConfigStruct)()
    if call(out) != 0:
        raise CheckpointError(_lib.lib().berth_ckpt_last_error().decode())
    try:
        c = out.contents
        s = lambda v: None if v is None else v.decode()
        o = lambda v: None if v < 0 else int(v)
        cal = None if c.calibration_rows < 0 else Calibration(int(c.calibration_rows), int(c.calibration_cols))
        quant = QuantizationConfig(quant_method=s(c.quant_method), bits=float(c.bits), head_bits=int(c.head_bits), codebook=s(c.codebook),
                                   version=s(c.version), vision_bits=o(c.vision_bits), mtp_bits=o(c.mtp_bits),
                                   out_scales=s(c.out_scales), calibration=cal)
        return ModelConfig(
            arch_string=s(c.arch_string), num_hidden_layers=int(c.num_hidden_layers), hidden_size=int(c.hidden_size),
            intermediate_size=o(c.intermediate_size), head_dim=int(c.head_dim), num_attention_heads=int(c.num_attention_heads),
            num_key_value_heads=int(c.num_key_value_heads), vocab_size=int(c.vocab_size),
            tie_word_embeddings=bool(c.tie_word_embeddings), layer_types=tuple(c.layer_types[i].decode() for i in range(c.n_layer_types)),
            linear_conv_kernel_dim=int(c.linear_conv_kernel_dim), linear_num_key_heads=int(c.linear_num_key_heads),
            linear_num_value_heads=int(c.linear_num_value_heads), linear_key_head_dim=int(c.linear_key_head_dim),
            linear_value_head_dim=int(c.linear_value_head_dim), attn_output_gate=bool(c.attn_output_gate),
            num_experts=o(c.num_experts), num_experts_per_tok=o(c.num_experts_per_tok), moe_intermediate_size=o(c.moe_intermediate_size),
            shared_expert_intermediate_size=o(c.shared_expert_intermediate_size), quantization=quant)
    finally:
        _lib.lib().berth_config_free(out)
