"""ctypes front end of the CPU oracle (``libexl3_oracle.so``).

Test infrastructure only.  Tests, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py`` may import this module; the shipped package
(``berth_b200``) never does.  Arrays are numpy; fp16 values travel as ``uint16`` bit
patterns or ``float16`` arrays (both accepted).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libexl3_oracle.so")


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside this file (gcc, OpenMP)."""
    src_newer = (not os.path.exists(_SO)) or any(
        os.path.getmtime(os.path.join(_HERE, f)) > os.path.getmtime(_SO)
        for f in ("exl3_oracle.c", "exl3_oracle.h", "Makefile")
    )
    if force or src_newer:
        subprocess.run(["make", "-C", _HERE, "-B", "libexl3_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = C.CDLL(_SO)
        _declare(_lib)
    return _lib


_vp, _i, _i64, _f = C.c_void_p, C.c_int, C.c_int64, C.c_float


class MoeWeights(C.Structure):
    _fields_ = [(n, _i) for n in ("hidden", "inter", "shared_inter", "n_experts", "top_k", "bits", "cb")] + [
        (n, _vp)
        for n in (
            "w_router", "router_bias", "gate_trellis", "up_trellis", "down_trellis",
            "gate_suh", "gate_svh", "up_suh", "up_svh", "down_suh", "down_svh",
            "sh_gate_trellis", "sh_up_trellis", "sh_down_trellis",
            "sh_gate_suh", "sh_gate_svh", "sh_up_suh", "sh_up_svh", "sh_down_suh", "sh_down_svh",
        )
    ]


def _declare(l: C.CDLL) -> None:
    l.exl3o_h2f.restype = C.c_float
    l.exl3o_h2f.argtypes = [C.c_uint16]
    l.exl3o_f2h.restype = C.c_uint16
    l.exl3o_f2h.argtypes = [C.c_float]
    l.exl3o_d2h.restype = C.c_uint16
    l.exl3o_d2h.argtypes = [C.c_double]
    l.exl3o_codebook.restype = C.c_uint16
    l.exl3o_codebook.argtypes = [C.c_uint32, _i]
    l.exl3o_hexp_neg.restype = C.c_uint16
    l.exl3o_hexp_neg.argtypes = [C.c_uint16]
    l.exl3o_unpack_signs.argtypes = [_vp, _i64, _vp]
    l.exl3o_tile_states.argtypes = [_vp, _i, _vp]
    l.exl3o_decode_tile.argtypes = [_vp, _i, _i, _vp]
    l.exl3o_reconstruct.argtypes = [_vp, _i, _i, _i, _i, _i, _i, _vp, _i]
    l.exl3o_had_r_128.argtypes = [_vp, _vp, _vp, _i, _i, _i, _i]
    l.exl3o_linear.restype = _i
    l.exl3o_linear.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i]
    l.exl3o_linear_f64.restype = _i
    l.exl3o_linear_f64.argtypes = [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i]
    l.exl3o_silu_mul.argtypes = [_vp, _vp, _vp, _i64, _f]
    l.exl3o_sample_keys.argtypes = [_vp, _i, _i, _f, C.c_uint32, _i, _vp, _vp]
    l.exl3o_sample_keys.restype = None
    l.exl3o_add_f32.argtypes = [_vp, _vp, _vp, _i64]
    l.exl3o_rms_norm.argtypes = [_vp, _i, _vp, _i, _vp, _vp, _i, _i, _f, _f, _f]
    l.exl3o_rms_norm.restype = None
    l.exl3o_gemv_cfg.restype = _i
    l.exl3o_gemv_cfg.argtypes = [_i] * 8
    l.exl3o_gemm_tune_key.restype = C.c_uint64
    l.exl3o_gemm_tune_key.argtypes = [_i] * 9
    l.exl3o_router_logits.argtypes = [_vp, _vp, _vp, _vp, _i, _i, _i]
    l.exl3o_router_topk.argtypes = [_vp, _vp, _vp, _i, _i, _i]
    l.exl3o_moe_layer.restype = _i
    l.exl3o_moe_layer.argtypes = [C.POINTER(MoeWeights), _vp, _i, _vp, _vp, _vp]
    l.exl3o_moe_layer_f64.restype = _i
    l.exl3o_moe_layer_f64.argtypes = [C.POINTER(MoeWeights), _vp, _i, _vp, _vp, _vp]
    l.exl3o_num_threads.restype = _i
    l.exl3o_set_num_threads.argtypes = [_i]


def _u16(a) -> np.ndarray:
    a = np.asarray(a)
    if a.dtype == np.float16 or a.dtype == np.int16:
        a = a.view(np.uint16)
    assert a.dtype == np.uint16, a.dtype
    return np.ascontiguousarray(a)


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def num_threads() -> int:
    return lib().exl3o_num_threads()


def set_num_threads(n: int) -> None:
    lib().exl3o_set_num_threads(n)


def codebook(states, cb: int) -> np.ndarray:
    """fp16 weights (as float16) of an array of 16-bit states."""
    s = np.asarray(states, dtype=np.uint32).ravel()
    out = np.empty(s.shape, np.uint16)
    f = lib().exl3o_codebook
    for i, v in enumerate(s):
        out[i] = f(int(v), cb)
    return out.view(np.float16).reshape(np.shape(states))


def hexp_neg(g) -> np.ndarray:
    g = _u16(g).ravel()
    f = lib().exl3o_hexp_neg
    return np.array([f(int(v)) for v in g], np.uint16).view(np.float16)


def unpack_signs(packed) -> np.ndarray:
    p = _u16(packed).ravel()
    out = np.empty(p.size * 16, np.uint16)
    lib().exl3o_unpack_signs(_p(p), p.size, _p(out))
    return out


def tile_states(words, bits: int) -> np.ndarray:
    w = _u16(words).ravel()
    assert w.size == 16 * bits
    out = np.empty(256, np.uint16)
    lib().exl3o_tile_states(_p(w), bits, _p(out))
    return out


def decode_tile(words, bits: int, cb: int) -> np.ndarray:
    w = _u16(words).ravel()
    assert w.size == 16 * bits
    out = np.empty((16, 16), np.uint16)
    lib().exl3o_decode_tile(_p(w), bits, cb, _p(out))
    return out.view(np.float16)


def reconstruct(trellis, size_k: int, full_n: int, bits: int, cb: int, n_offset: int = 0,
                slice_n: int | None = None) -> np.ndarray:
    """fp16 W[size_k][slice_n] of columns [n_offset, n_offset+slice_n)."""
    t = _u16(trellis).ravel()
    slice_n = full_n - n_offset if slice_n is None else slice_n
    assert t.size == (size_k // 16) * (full_n // 16) * 16 * bits
    w = np.empty((size_k, slice_n), np.uint16)
    lib().exl3o_reconstruct(_p(t), size_k, full_n, n_offset, slice_n, bits, cb, _p(w), slice_n)
    return w.view(np.float16)


def had_r_128(x, scale, pre_scale: bool) -> np.ndarray:
    x = np.ascontiguousarray(x)
    rows, cols = x.shape
    fp32 = x.dtype == np.float32
    xin = x if fp32 else _u16(x)
    out = np.empty_like(xin)
    sc = None if scale is None else _u16(scale)
    lib().exl3o_had_r_128(_p(xin), _p(out), _p(sc), int(pre_scale), rows, cols, int(fp32))
    return out if fp32 else out.view(np.float16)


def linear(a, trellis, suh, svh, size_k: int, size_n: int, bits: int, cb: int, out_fp32: bool):
    """Returns (c, a_had): c float16 or float32 [m][n], a_had float16 [m][k]."""
    a = _u16(a).reshape(-1, size_k)
    m = a.shape[0]
    c = np.empty((m, size_n), np.float32 if out_fp32 else np.uint16)
    a_had = np.empty((m, size_k), np.uint16)
    rc = lib().exl3o_linear(_p(a), _p(_u16(trellis)), _p(c), _p(_u16(suh)), _p(a_had), _p(_u16(svh)),
                            m, size_k, size_n, bits, cb, int(out_fp32))
    if rc != 0:
        raise ValueError("exl3o_linear: bad shape")
    return (c if out_fp32 else c.view(np.float16)), a_had.view(np.float16)


def linear_f64(a, trellis, suh, svh, size_k: int, size_n: int, bits: int, cb: int) -> np.ndarray:
    a = _u16(a).reshape(-1, size_k)
    m = a.shape[0]
    c = np.empty((m, size_n), np.float64)
    rc = lib().exl3o_linear_f64(_p(a), _p(_u16(trellis)), _p(c), _p(_u16(suh)), _p(_u16(svh)),
                                m, size_k, size_n, bits, cb)
    if rc != 0:
        raise ValueError("exl3o_linear_f64: bad shape")
    return c


def sample_keys(outputs: np.ndarray, inv_temp: float, random: int, mode: int):
    """Keys and scores of the sampling epilogue for stored outputs ``[rows][n]`` (any float dtype, taken as fp32):
    ``(keys uint64 [rows], scores fp32 [rows][n])``; mode 0 greedy, 1 Gumbel."""
    o = np.ascontiguousarray(outputs.astype(np.float32))
    rows, n = o.shape
    keys = np.zeros(rows, np.uint64)
    scores = np.zeros((rows, n), np.float32)
    lib().exl3o_sample_keys(_p(o), rows, n, float(inv_temp), int(random) & 0xFFFFFFFF, int(mode), _p(keys), _p(scores))
    return keys, scores


def silu_mul(gate, up, act_limit: float = 0.0) -> np.ndarray:
    g, u = _u16(gate).ravel(), _u16(up).ravel()
    out = np.empty_like(g)
    lib().exl3o_silu_mul(_p(g), _p(u), _p(out), g.size, act_limit)
    return out.view(np.float16).reshape(np.shape(gate))


def add_f32(a, b) -> np.ndarray:
    a = np.ascontiguousarray(a, np.float32)
    b = np.ascontiguousarray(b, np.float32)
    c = np.empty_like(a)
    lib().exl3o_add_f32(_p(a), _p(b), _p(c), a.size)
    return c


def rms_norm(x, weight, weight_bf16: bool, epsilon: float, constant_bias: float = 0.0, constant_scale: float = 1.0,
             residual=None):
    """RMSNorm rows of ``x`` (float32, or float16 for the _f16 form) with ``weight`` (uint16 bit patterns: bfloat16 or
    float16).  Returns the float16 rows; with ``residual`` (float32 array, updated in place: residual += x) the rows
    normalised are the updated residual (RES_IN)."""
    x = np.ascontiguousarray(x)
    rows, dim = x.shape
    is_f16 = x.dtype == np.float16
    if not is_f16:
        x = x.astype(np.float32, copy=False)
    w = _u16(weight)
    y = np.empty((rows, dim), np.uint16)
    if residual is not None:
        assert residual.dtype == np.float32 and residual.flags["C_CONTIGUOUS"] and residual.shape == (rows, dim)
    lib().exl3o_rms_norm(_p(x.view(np.uint16) if is_f16 else x), 1 if is_f16 else 0, _p(w), 1 if weight_bf16 else 0, _p(y),
                         None if residual is None else _p(residual), rows, dim, epsilon, constant_bias, constant_scale)
    return y.view(np.float16)


def gemv_cfg(cc, m, k, n, bits, cb, mode, narrow_coresident) -> int:
    return lib().exl3o_gemv_cfg(cc, m, k, n, bits, cb, mode, narrow_coresident)


def gemm_tune_key(m, k, n, bits, out_fp32, device, cc, sms, cb) -> int:
    return lib().exl3o_gemm_tune_key(m, k, n, bits, out_fp32, device, cc, sms, cb)


def router_logits(x, w_router, bias=None) -> np.ndarray:
    x = _u16(x)
    w = _u16(w_router)
    T, H = x.shape
    E = w.shape[1]
    b = None if bias is None else np.ascontiguousarray(bias, np.float32)
    out = np.empty((T, E), np.float32)
    lib().exl3o_router_logits(_p(x), _p(w), _p(b), _p(out), T, H, E)
    return out


def router_topk(logits, k: int):
    logits = np.ascontiguousarray(logits, np.float32)
    T, E = logits.shape
    idx = np.empty((T, k), np.int32)
    w = np.empty((T, k), np.float32)
    lib().exl3o_router_topk(_p(logits), _p(idx), _p(w), T, E, k)
    return idx, w


def _moe_struct(wts: dict):
    """wts: dict produced by berth_b200.synth.moe_layer_weights (numpy arrays)."""
    keep = []
    s = MoeWeights()
    for name in ("hidden", "inter", "shared_inter", "n_experts", "top_k", "bits", "cb"):
        setattr(s, name, int(wts[name]))
    for name, _ in MoeWeights._fields_[7:]:
        v = wts.get(name)
        if v is None:
            setattr(s, name, None)
            continue
        arr = np.ascontiguousarray(v, np.float32) if name == "router_bias" else _u16(v)
        keep.append(arr)
        setattr(s, name, arr.ctypes.data)
    return s, keep


def moe_layer(wts: dict, x):
    """Returns (out fp32 [T][hidden], topk_idx int32 [T][k], topk_w fp32 [T][k])."""
    x = _u16(x)
    T = x.shape[0]
    s, keep = _moe_struct(wts)
    out = np.empty((T, s.hidden), np.float32)
    idx = np.empty((T, s.top_k), np.int32)
    tw = np.empty((T, s.top_k), np.float32)
    rc = lib().exl3o_moe_layer(C.byref(s), _p(x), T, _p(out), _p(idx), _p(tw))
    if rc != 0:
        raise ValueError("exl3o_moe_layer: bad shape")
    del keep
    return out, idx, tw


def moe_layer_f64(wts: dict, x, topk_idx, topk_w) -> np.ndarray:
    x = _u16(x)
    T = x.shape[0]
    s, keep = _moe_struct(wts)
    idx = np.ascontiguousarray(topk_idx, np.int32)
    tw = np.ascontiguousarray(topk_w, np.float32)
    out = np.empty((T, s.hidden), np.float64)
    rc = lib().exl3o_moe_layer_f64(C.byref(s), _p(x), T, _p(idx), _p(tw), _p(out))
    if rc != 0:
        raise ValueError("exl3o_moe_layer_f64: bad shape")
    del keep
    return out
