"""Loads ``libberth_b200.so`` and declares the C ABI of ``include/berth_b200.h``."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(_HERE, "libberth_b200.so")
CSRC = os.path.join(_HERE, "csrc")

_vp, _i, _i64, _f, _u64 = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_uint64
_ip = C.POINTER(C.c_int)


class MoeWeights(C.Structure):
    """``berth_moe_weights`` of include/berth_b200.h."""
    _fields_ = [(n, _i) for n in ("hidden", "inter", "shared_inter", "n_experts", "top_k", "k_bits", "codebook")] + [
        (n, _vp) for n in (
            "w_router", "router_bias", "gate_trellis", "up_trellis", "down_trellis",
            "gate_suh", "gate_svh", "up_suh", "up_svh", "down_suh", "down_svh",
            "sh_gate_trellis", "sh_up_trellis", "sh_down_trellis",
            "sh_gate_suh", "sh_gate_svh", "sh_up_suh", "sh_up_svh", "sh_down_suh", "sh_down_svh")]


class TensorInfo(C.Structure):
    """``berth_tensor_info`` of include/berth_b200_checkpoint.h."""
    _fields_ = [("name", C.c_char_p), ("shard", C.c_char_p), ("dtype", _i), ("rank", _i), ("shape", _u64 * 8),
                ("offset", _u64), ("length", _u64)]


class LinearInfo(C.Structure):
    """``berth_linear_info`` of include/berth_b200_checkpoint.h."""
    _fields_ = [("prefix", C.c_char_p), ("trellis", TensorInfo), ("input_scale", TensorInfo), ("output_scale", TensorInfo),
                ("bias", TensorInfo), ("input_packed", _i), ("output_packed", _i), ("has_bias", _i), ("codebook", _i),
                ("bits_x2", _i)]


class ModelConfigStruct(C.Structure):
    """``berth_model_config`` of include/berth_b200_checkpoint.h."""
    _fields_ = [("arch_string", C.c_char_p)] + [(n, C.c_uint32) for n in (
        "num_hidden_layers", "hidden_size", "head_dim", "num_attention_heads", "num_key_value_heads", "vocab_size")] + [
        ("tie_word_embeddings", _i), ("attn_output_gate", _i)] + [(n, C.c_uint32) for n in (
            "linear_conv_kernel_dim", "linear_num_key_heads", "linear_num_value_heads", "linear_key_head_dim",
            "linear_value_head_dim")] + [(n, _i64) for n in (
                "intermediate_size", "num_experts", "num_experts_per_tok", "moe_intermediate_size",
                "shared_expert_intermediate_size", "n_layer_types")] + [
        ("layer_types", C.POINTER(C.c_char_p)), ("quant_method", C.c_char_p), ("bits", C.c_double), ("head_bits", C.c_uint32),
        ("codebook", C.c_char_p), ("version", C.c_char_p), ("out_scales", C.c_char_p)] + [(n, _i64) for n in (
            "vision_bits", "mtp_bits", "calibration_rows", "calibration_cols")] + [("strings", _vp)]


_tip, _lip = C.POINTER(TensorInfo), C.POINTER(LinearInfo)

# name -> (restype, argtypes); every symbol the headers declare.
SIGNATURES = {
    "berth_exl3_linear": (_i, [_vp] * 6 + [_i] * 6 + [_vp]),
    "berth_exl3_linear_static_scratch": (_i, [_vp] * 6 + [_i] * 6 + [_vp]),
    "berth_exl3_linear_argmax": (_i, [_vp] * 7 + [_i] * 6 + [_vp]),
    "berth_exl3_linear_sample": (_i, [_vp] * 7 + [_i] * 6 + [_f, C.c_uint, _i, _vp]),
    "berth_exl3_linear_add": (_i, [_vp] * 7 + [_i] * 5 + [_vp]),
    "berth_exl3_linear_silu": (_i, [_vp] * 8 + [_f] + [_i] * 6 + [_vp]),
    "berth_exl3_linear_stack": (_i, [_vp] * 6 + [_i] * 7 + [_vp]),
    "berth_exl3_weights_streamed": (_i, [_i]),
    "berth_exl3_linear_multi": (_i, [_vp] * 7 + [_i] * 6 + [_vp]),
    "berth_argmax_key_decode": (None, [_u64, C.POINTER(C.c_int32), C.POINTER(C.c_float)]),
    "berth_exl3_last_error": (C.c_char_p, []),
    "berth_exl3_last_launch": (C.c_char_p, []),
    "berth_device_cc": (_i, [_i]),
    "berth_device_sms": (_i, [_i]),
    "berth_device_status": (_i, [_i]),
    "berth_exl3_decode_rate": (_i, [_i] * 5 + [C.POINTER(C.c_double)] * 2),
    "berth_exl3_pipe_probe": (_i, [_i, _i, C.POINTER(C.c_double)]),
    "berth_exl3_gemm_tune_key": (_u64, [_i] * 9),
    "berth_exl3_smoke_int8": (_i, [_i]),
    "berth_exl3_smoke_gemm": (_i, []),
    "berth_prefill_exl3_linear": (_i, [_vp] * 7 + [_i] * 6 + [_vp]),
    "berth_prefill_last_error": (C.c_char_p, []),
    "berth_prefill_last_launch": (C.c_char_p, []),
    "berth_exl3_gemv_cfg": (_i, [_i] * 8),
    "berth_prefill_reconstruct": (_i, [_vp, _vp] + [_i] * 6 + [_vp]),
    "berth_prefill_had_r_128": (_i, [_vp] * 3 + [_i] * 4 + [_vp]),
    "berth_ops_silu_mul": (_i, [_vp] * 3 + [_i64, _f, _vp]),
    "berth_ops_add_f32": (_i, [_vp] * 3 + [_i, _vp]),
    "berth_ops_rms_norm": (_i, [_vp] * 3 + [_i, _i, _f, _f, _f, _i, _vp]),
    "berth_ops_rms_norm_f16": (_i, [_vp] * 3 + [_i, _i, _f, _f, _f, _vp]),
    "berth_ops_rms_norm_res_in": (_i, [_vp] * 4 + [_i, _i, _f, _f, _f, _i, _vp]),
    "berth_moe_router_topk": (_i, [_vp] * 6 + [_i] * 4 + [_vp]),
    "berth_moe_workspace_bytes": (C.c_size_t, [_i] * 6),
    "berth_moe_layer": (_i, [C.POINTER(MoeWeights), _vp, _i, _vp, _vp, _vp, _vp, C.c_size_t, _vp]),
    "berth_moe_experts_workspace_bytes": (C.c_size_t, [_i] * 5),
    "berth_moe_sort_rows": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp, _vp, C.c_size_t, _i, _i, _i, _i, _vp]),
    "berth_moe_gather": (_i, [_vp, _vp, _i, _i, _vp, _i, _vp]),
    "berth_moe_experts": (_i, [C.POINTER(MoeWeights), _vp, _vp, _i, _vp, C.c_size_t, _i, _i, _vp]),
    "berth_moe_combine": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "berth_moe_ep_send_workspace_bytes": (C.c_size_t, [_i, _i, _i]),
    "berth_moe_ep_send": (_i, [_vp, _i, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, C.c_size_t, _vp]),
    "berth_moe_ep_experts_workspace_bytes": (C.c_size_t, [_i, _i, _i, _i, _i, _i]),
    "berth_moe_ep_experts": (_i, [C.POINTER(MoeWeights), _vp, _i, _vp, _i, _vp, _i, _vp, _vp, _vp, C.c_size_t, _i, _i, _i, _vp]),
    "berth_moe_p2p_send_workspace_bytes": (C.c_size_t, [_i, _i, _i, _i]),
    "berth_moe_p2p_send": (_i, [_vp, _i, _vp, _vp, _i, _i, _i, _vp, _vp, _vp, _i, _i, C.c_uint, _vp, _vp, _vp, _i, _vp, C.c_size_t, _vp]),
    "berth_moe_p2p_experts_workspace_bytes": (C.c_size_t, [_i, _i, _i, _i]),
    "berth_moe_p2p_experts": (_i, [C.POINTER(MoeWeights), _vp, _i, _vp, _i, _i, C.c_uint, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _vp,
                                   _vp, C.c_size_t, _vp]),
    "berth_prefill_hgemm": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "berth_ops_mgemm": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _vp]),
    "berth_ops_mgemm_tune_key": (C.c_uint64, [_i] * 12),
    "berth_moe_last_error": (C.c_char_p, []),
    "berth_moe_last_launch": (C.c_char_p, []),
    "berth_ops_last_error": (C.c_char_p, []),
    "berth_ops_last_launch": (C.c_char_p, []),
    "berth_ckpt_open": (_i, [C.c_char_p, C.POINTER(_vp)]),
    "berth_ckpt_close": (None, [_vp]),
    "berth_ckpt_n_tensors": (_i64, [_vp]),
    "berth_ckpt_n_linears": (_i64, [_vp]),
    "berth_ckpt_n_others": (_i64, [_vp]),
    "berth_ckpt_tensor_at": (_i, [_vp, _i64, _tip]),
    "berth_ckpt_tensor": (_i, [_vp, C.c_char_p, _tip]),
    "berth_ckpt_linear_at": (_i, [_vp, _i64, _lip]),
    "berth_ckpt_linear": (_i, [_vp, C.c_char_p, _lip]),
    "berth_ckpt_other_at": (_i, [_vp, _i64, _tip]),
    "berth_ckpt_read": (_i, [_vp, C.c_char_p, _vp, _u64]),
    "berth_ckpt_scale_f16": (_i, [_vp, C.c_char_p, _i, _vp, _u64]),
    "berth_unpack_signs": (_i, [_vp, _u64, _vp]),
    "berth_config_parse": (_i, [C.c_char_p, _u64, _vp]),
    "berth_config_open": (_i, [C.c_char_p, _vp]),
    "berth_config_free": (None, [_vp]),
    "berth_ckpt_last_error": (C.c_char_p, []),
}

_lib = None


def build(verbose: bool = False) -> str:
    """Compile the CUDA library in-tree with the Makefile under csrc/ (nvcc, sm_100a)."""
    out = None if verbose else subprocess.DEVNULL
    subprocess.run(["make", "-C", CSRC, "-j8"], check=True, stdout=out)
    return SO_PATH


def lib() -> C.CDLL:
    """The loaded library.  Raises if it has not been built: there is no fallback."""
    global _lib
    if _lib is None:
        if not os.path.exists(SO_PATH):
            raise RuntimeError(
                f"{SO_PATH} is missing: build it with `make -C {CSRC}` (or __graft_entry__.build()); "
                "berth_b200 has no CPU or PyTorch fallback")
        l = C.CDLL(SO_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(l, name)   # AttributeError here = header and library disagree
            fn.restype = res
            fn.argtypes = args
        _lib = l
    return _lib
