"""Seeded synthetic EXL3 tensors (numpy only).

Every tensor is a pure function of ``(seed, name, index)`` through a counter-based
splitmix64 generator, so the CPU checker and the GPU path are handed identical bytes and a
fixture can be regenerated anywhere.  Distributions follow the benchmark configurations:
trellis words uniform uint16; ``suh``/``svh`` a random sign times N(1, 0.05) in fp16;
activations N(0, 1) fp16, optionally with a fraction of elements multiplied by a constant
(outliers); router weight N(0, 0.02) fp16.  The master seed 1234 mirrors
``scripts/dump_exl3_reference.py:31`` of berth.
"""
from __future__ import annotations

import numpy as np

MASTER_SEED = 1234
_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        x = (x + np.uint64(0x9E3779B97F4A7C15)) & _M64
        z = x
        z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
        z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
        return z ^ (z >> np.uint64(31))


def _fnv1a64(name: str) -> int:
    h = 0xCBF29CE484222325
    for b in name.encode():
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


def raw_u64(seed: int, name: str, n: int, stream: int = 0) -> np.ndarray:
    """n 64-bit words of the stream keyed by (seed, name, stream)."""
    key = _splitmix64(np.array([(seed * 0x9E3779B97F4A7C15 + _fnv1a64(name) + stream * 0xD1B54A32D192ED03)
                                & 0xFFFFFFFFFFFFFFFF], np.uint64))[0]
    idx = np.arange(n, dtype=np.uint64)
    with np.errstate(over="ignore"):
        return _splitmix64((idx * np.uint64(0x2545F4914F6CDD1D) + key) & _M64)


def uniform01(seed: int, name: str, n: int, stream: int = 0) -> np.ndarray:
    """float64 in (0, 1)."""
    return ((raw_u64(seed, name, n, stream) >> np.uint64(11)).astype(np.float64) + 0.5) * (1.0 / (1 << 53))


def normal(seed: int, name: str, n: int) -> np.ndarray:
    """float64 N(0,1) by Box-Muller on two streams."""
    u1 = uniform01(seed, name, n, 1)
    u2 = uniform01(seed, name, n, 2)
    return np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)


def trellis(seed: int, name: str, size_k: int, size_n: int, bits: int) -> np.ndarray:
    """uint16 [K/16][N/16][16*bits], uniform words."""
    n = (size_k // 16) * (size_n // 16) * 16 * bits
    nw = (n + 3) // 4
    words = raw_u64(seed, name, nw).view(np.uint16)[:n]
    return np.ascontiguousarray(words).reshape(size_k // 16, size_n // 16, 16 * bits)


def sign_scale(seed: int, name: str, n: int, gain: float = 1.0) -> np.ndarray:
    """float16 [n]: random sign times N(1, 0.05), times `gain`."""
    mag = 1.0 + 0.05 * normal(seed, name, n)
    sign = np.where(raw_u64(seed, name, n, 3) & np.uint64(1), -1.0, 1.0)
    return (sign * mag * gain).astype(np.float16)


def activations(seed: int, name: str, rows: int, cols: int, outlier_frac: float = 0.0,
                outlier_mul: float = 20.0) -> np.ndarray:
    """float16 [rows][cols] ~ N(0,1); a Bernoulli(outlier_frac) subset is multiplied by outlier_mul."""
    x = normal(seed, name, rows * cols)
    if outlier_frac > 0.0:
        hit = uniform01(seed, name, rows * cols, 4) < outlier_frac
        x = np.where(hit, x * outlier_mul, x)
    return x.astype(np.float16).reshape(rows, cols)


def router_weight(seed: int, name: str, hidden: int, n_experts: int) -> np.ndarray:
    """float16 [hidden][n_experts] ~ N(0, 0.02)."""
    return (0.02 * normal(seed, name, hidden * n_experts)).astype(np.float16).reshape(hidden, n_experts)


def zipf_router_bias(seed: int, name: str, n_experts: int, s: float = 1.1, strength: float = 1.0) -> np.ndarray:
    """float32 [n_experts]: additive router bias strength*ln(rank^-s) over a seeded rank permutation,
    which skews expert popularity towards a Zipf(s) law."""
    order = np.argsort(raw_u64(seed, name, n_experts, 5), kind="stable")
    rank = np.empty(n_experts, np.int64)
    rank[order] = np.arange(1, n_experts + 1)
    return (strength * (-s) * np.log(rank.astype(np.float64))).astype(np.float32)


def linear_weights(seed: int, name: str, size_k: int, size_n: int, bits: int, fan_in_gain: bool = False) -> dict:
    """One EXL3 linear.  With fan_in_gain the output sign-scale carries 1/sqrt(size_k), the factor a
    trained checkpoint's scales carry; chains of linears (MLP, experts) need it or their fp16
    intermediates overflow with unit-variance codebook weights."""
    gain = 1.0 / np.sqrt(size_k) if fan_in_gain else 1.0
    return {
        "trellis": trellis(seed, name + ".trellis", size_k, size_n, bits),
        "suh": sign_scale(seed, name + ".suh", size_k),
        "svh": sign_scale(seed, name + ".svh", size_n, gain),
        "size_k": size_k, "size_n": size_n, "bits": bits,
    }


def _stack(seed, name, n, size_k, size_n, bits):
    t = np.stack([trellis(seed, f"{name}.{e}.trellis", size_k, size_n, bits) for e in range(n)])
    suh = np.stack([sign_scale(seed, f"{name}.{e}.suh", size_k) for e in range(n)])
    svh = np.stack([sign_scale(seed, f"{name}.{e}.svh", size_n, 1.0 / np.sqrt(size_k)) for e in range(n)])
    return t, suh, svh


def moe_layer_weights(seed: int, name: str, hidden: int, inter: int, n_experts: int, top_k: int,
                      bits: int, cb: int, shared_inter: int | None = None,
                      router_bias: np.ndarray | None = None) -> dict:
    """Weights of one A3B-style MoE layer.  Expert stacks: gate/up trellis
    (E, hidden/16, inter/16, 16*bits), down (E, inter/16, hidden/16, 16*bits); suh/svh stacks
    [E][.]; optional shared expert with its own intermediate size.  Every svh carries the
    1/sqrt(fan_in) gain (see linear_weights), so activations keep unit scale through the layer."""
    w = {"hidden": hidden, "inter": inter, "n_experts": n_experts, "top_k": top_k, "bits": bits,
         "cb": cb, "shared_inter": shared_inter or 0,
         "w_router": router_weight(seed, name + ".gate.weight", hidden, n_experts),
         "router_bias": router_bias}
    w["gate_trellis"], w["gate_suh"], w["gate_svh"] = _stack(seed, name + ".experts.gate_proj", n_experts, hidden, inter, bits)
    w["up_trellis"], w["up_suh"], w["up_svh"] = _stack(seed, name + ".experts.up_proj", n_experts, hidden, inter, bits)
    w["down_trellis"], w["down_suh"], w["down_svh"] = _stack(seed, name + ".experts.down_proj", n_experts, inter, hidden, bits)
    if shared_inter:
        for p, (k, n) in (("gate", (hidden, shared_inter)), ("up", (hidden, shared_inter)),
                          ("down", (shared_inter, hidden))):
            lw = linear_weights(seed, f"{name}.shared_expert.{p}_proj", k, n, bits, fan_in_gain=True)
            w[f"sh_{p}_trellis"], w[f"sh_{p}_suh"], w[f"sh_{p}_svh"] = lw["trellis"], lw["suh"], lw["svh"]
    return w
