"""Host-side mirror of berth's ``berth-exl3`` crate over the C ABI of include/berth_b200_checkpoint.h.

``Checkpoint.open`` / ``linears`` / ``other_tensors`` (crates/berth-exl3/src/checkpoint.rs:30-72),
``LinearExl3`` with ``Bitrate`` / ``Codebook`` / ``HadamardScale`` (src/linear.rs:14-155), ``unpack_signs``
(src/signs.rs:25-45).  On top of that, what an engine needs to hand a linear or an MoE layer to the kernels:
``load_linear`` (trellis, fp16 input and output scales, bits, codebook as numpy arrays) and ``load_experts``
(the per-expert tensors of one layer stacked into the arrays ``berth_b200.moe.MoeLayer`` takes).
Parsing and validation run in the library; a failure raises :class:`CheckpointError` with the library's message.
"""
from __future__ import annotations

import ctypes as C
import dataclasses
import os

import numpy as np

from . import _lib
from .kernels import Codebook

DTYPES = ("BOOL", "U8", "I8", "I16", "U16", "I32", "U32", "I64", "U64", "F16", "BF16", "F32", "F64", "F8_E4M3", "F8_E5M2", "F8_E8M0")
_NUMPY = {"BOOL": np.bool_, "U8": np.uint8, "I8": np.int8, "I16": np.int16, "U16": np.uint16, "I32": np.int32, "U32": np.uint32,
          "I64": np.int64, "U64": np.uint64, "F16": np.float16, "BF16": np.uint16, "F32": np.float32, "F64": np.float64,
          "F8_E4M3": np.uint8, "F8_E5M2": np.uint8, "F8_E8M0": np.uint8}


class CheckpointError(RuntimeError):
    """``berth_exl3::Error``."""


@dataclasses.dataclass(frozen=True)
class TensorInfo:
    """crates/berth-exl3/src/safetensors.rs:14-30."""
    name: str
    shard: str
    dtype: str
    shape: tuple
    offset: int
    length: int


@dataclasses.dataclass(frozen=True)
class LinearExl3:
    """crates/berth-exl3/src/linear.rs:118-138.  ``k`` is bits per weight (x.5 for the half rates)."""
    prefix: str
    trellis: TensorInfo
    input_scale: TensorInfo
    output_scale: TensorInfo
    input_packed: bool
    output_packed: bool
    bias: TensorInfo | None
    codebook: Codebook
    k: float

    @property
    def in_features(self) -> int:
        return int(self.trellis.shape[0]) * 16

    @property
    def out_features(self) -> int:
        return int(self.trellis.shape[1]) * 16


def _err() -> str:
    return (_lib.lib().berth_ckpt_last_error() or b"").decode()


def _tensor(t) -> TensorInfo:
    return TensorInfo(t.name.decode(), t.shard.decode(), DTYPES[t.dtype], tuple(int(t.shape[i]) for i in range(t.rank)),
                      int(t.offset), int(t.length))


def _linear(l) -> LinearExl3:
    return LinearExl3(l.prefix.decode(), _tensor(l.trellis), _tensor(l.input_scale), _tensor(l.output_scale), bool(l.input_packed),
                      bool(l.output_packed), _tensor(l.bias) if l.has_bias else None, Codebook(l.codebook), l.bits_x2 / 2)


def unpack_signs(packed) -> np.ndarray:
    """Packed little-endian int16 sign words (bytes or an int16/uint16 array) -> fp16 bit patterns (uint16):
    bit i of a word is element i, set = -1.0 (0xBC00), clear = +1.0 (0x3C00)."""
    raw = packed if isinstance(packed, (bytes, bytearray)) else np.ascontiguousarray(packed).tobytes()
    out = np.empty(len(raw) * 8, np.uint16)
    buf = (C.c_char * len(raw)).from_buffer_copy(raw) if raw else None
    if _lib.lib().berth_unpack_signs(buf, len(raw), out.ctypes.data) != 0:
        raise CheckpointError(_err())
    return out


class Checkpoint:
    """An opened checkpoint directory (single ``model.safetensors`` or a sharded index)."""

    def __init__(self, directory: str):
        h = C.c_void_p()
        if _lib.lib().berth_ckpt_open(os.fsencode(directory), C.byref(h)) != 0:
            raise CheckpointError(_err())
        self._h = h
        self.directory = directory

    @classmethod
    def open(cls, directory: str) -> "Checkpoint":
        return cls(directory)

    def close(self) -> None:
        if getattr(self, "_h", None):
            _lib.lib().berth_ckpt_close(self._h)
            self._h = None

    __del__ = close

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # ------------------------------------------------------------------ index
    def _list(self, count, at, info_type, convert):
        l = _lib.lib()
        out = []
        for i in range(count(self._h)):
            info = info_type()
            if at(self._h, i, C.byref(info)) != 0:
                raise CheckpointError(_err())
            out.append(convert(info))
        return out

    def tensors(self) -> list:
        l = _lib.lib()
        return self._list(l.berth_ckpt_n_tensors, l.berth_ckpt_tensor_at, _lib.TensorInfo, _tensor)

    def linears(self) -> list:
        """Every EXL3 linear, sorted by prefix."""
        l = _lib.lib()
        return self._list(l.berth_ckpt_n_linears, l.berth_ckpt_linear_at, _lib.LinearInfo, _linear)

    def other_tensors(self) -> list:
        """Tensors that belong to no linear (norms, embeddings, router weights, ...), in name order."""
        l = _lib.lib()
        return self._list(l.berth_ckpt_n_others, l.berth_ckpt_other_at, _lib.TensorInfo, _tensor)

    def tensor(self, name: str) -> TensorInfo:
        info = _lib.TensorInfo()
        if _lib.lib().berth_ckpt_tensor(self._h, name.encode(), C.byref(info)) != 0:
            raise CheckpointError(_err())
        return _tensor(info)

    def linear(self, prefix: str) -> LinearExl3:
        info = _lib.LinearInfo()
        if _lib.lib().berth_ckpt_linear(self._h, prefix.encode(), C.byref(info)) != 0:
            raise CheckpointError(_err())
        return _linear(info)

    # ------------------------------------------------------------------ data
    def read(self, name: str) -> np.ndarray:
        """The tensor's data as a numpy array of its shape (BF16 and the F8 types as raw uint16 / uint8)."""
        t = self.tensor(name)
        out = np.empty(t.shape, _NUMPY[t.dtype])
        if _lib.lib().berth_ckpt_read(self._h, name.encode(), out.ctypes.data, out.nbytes) != 0:
            raise CheckpointError(_err())
        return out

    def scale_f16(self, prefix: str, output_side: bool) -> np.ndarray:
        """The linear's input or output scale as fp16 bit patterns, unpacking ``su`` / ``sv`` where the checkpoint
        stores packed signs (``LinearExl3::unpack_{input,output}_signs`` folded into the read)."""
        lin = self.linear(prefix)
        n = lin.out_features if output_side else lin.in_features
        out = np.empty(n, np.uint16)
        if _lib.lib().berth_ckpt_scale_f16(self._h, prefix.encode(), int(output_side), out.ctypes.data, n) != 0:
            raise CheckpointError(_err())
        return out

    def load_linear(self, prefix: str) -> dict:
        """What ``Exl3Linear`` / ``kernels.exl3_linear`` take: trellis uint16 [K/16][N/16][16*bits], suh / svh as fp16
        bit patterns, ``bits`` and ``cb``.  Half-integer bitrates and biases have no kernel: they fail closed."""
        lin = self.linear(prefix)
        if lin.k != int(lin.k):
            raise CheckpointError(f"`{prefix}.trellis`: no linked kernel for the half-integer bitrate {lin.k}")
        if lin.bias is not None:
            raise CheckpointError(f"`{prefix}.bias`: biased linears are not supported")   # crates/berth-engine/src/mlp.rs:64-112
        return {"trellis": self.read(prefix + ".trellis").view(np.uint16), "suh": self.scale_f16(prefix, False),
                "svh": self.scale_f16(prefix, True), "bits": int(lin.k), "cb": int(lin.codebook)}

    def load_experts(self, layer_prefix: str, n_experts: int) -> dict:
        """The routed experts of one MoE block stacked for ``MoeLayer``: ``{gate,up,down}_{trellis,suh,svh}`` with a
        leading expert dimension, from the per-expert tensors ``<layer_prefix>.experts.<e>.<proj>_proj.*``
        (crates/berth-plan/tests/plan.rs:100-116).  All experts must share shape, bitrate and codebook."""
        out, bits, cb = {}, None, None
        for proj in ("gate", "up", "down"):
            parts = [self.load_linear(f"{layer_prefix}.experts.{e}.{proj}_proj") for e in range(n_experts)]
            for p in parts:
                if (p["bits"], p["cb"]) != (parts[0]["bits"], parts[0]["cb"]) or p["trellis"].shape != parts[0]["trellis"].shape:
                    raise CheckpointError(f"`{layer_prefix}.experts`: experts differ in shape, bitrate or codebook")
            if bits is None:
                bits, cb = parts[0]["bits"], parts[0]["cb"]
            elif (bits, cb) != (parts[0]["bits"], parts[0]["cb"]):
                raise CheckpointError(f"`{layer_prefix}.experts`: projections differ in bitrate or codebook")
            for key in ("trellis", "suh", "svh"):
                out[f"{proj}_{key}"] = np.stack([p[key] for p in parts])
        out["bits"], out["cb"], out["n_experts"] = bits, cb, n_experts
        return out
