"""The CPU oracle against everything berth's own tree pins for this path, and against
independent restatements (numpy / pure Python) of the parts nothing pins."""
import math
import os

import numpy as np
import pytest

from berth_b200 import synth


# ---------------------------------------------------------------- fp16 helpers

def test_h2f_all_patterns(oracle):
    lib = oracle.lib()
    bits = np.arange(65536, dtype=np.uint16)
    ref = bits.view(np.float16).astype(np.float32)
    got = np.array([lib.exl3o_h2f(int(b)) for b in bits], np.float32)
    same = (got.view(np.uint32) == ref.view(np.uint32)) | (np.isnan(got) & np.isnan(ref))
    assert same.all()


def test_f2h_d2h_match_numpy(oracle):
    lib = oracle.lib()
    rng = np.random.default_rng(7)
    f = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 20000),
        np.array([0.0, -0.0, 65504.0, 65520.0, 65519.9, 1e-8, 5.96e-8, 2.98e-8, 2.99e-8, 6.1e-5, -6.1e-5,
                  np.inf, -np.inf], np.float32)])
    with np.errstate(over="ignore"):
        ref = f.astype(np.float16).view(np.uint16)
        refd = f.astype(np.float64).astype(np.float16).view(np.uint16)
    got = np.array([lib.exl3o_f2h(float(v)) for v in f], np.uint16)
    gotd = np.array([lib.exl3o_d2h(float(v)) for v in f.astype(np.float64)], np.uint16)
    assert (got == ref).all()
    assert (gotd == refd).all()
    # halfway cases between adjacent fp16 values round to even (double has the exact midpoint)
    h = np.arange(0x0001, 0x7bff, 37, dtype=np.uint16)
    lo = h.view(np.float16).astype(np.float64)
    hi = (h + 1).astype(np.uint16).view(np.float16).astype(np.float64)
    mid = (lo + hi) / 2
    exp = np.where(h & 1, h + 1, h).astype(np.uint16)
    got = np.array([lib.exl3o_d2h(float(v)) for v in mid], np.uint16)
    assert (got == exp).all()


# ---------------------------------------------------------------- pinned by berth's tree

def test_unpack_signs_known_answers(oracle):
    # crates/berth-exl3/src/signs.rs:52-91
    one, neg = 0x3C00, 0xBC00
    s = oracle.unpack_signs(np.array([1], np.uint16))
    assert s[0] == neg and (s[1:] == one).all() and s.size == 16
    s = oracle.unpack_signs(np.array([0x8000], np.uint16))
    assert (s[:15] == one).all() and s[15] == neg
    assert (oracle.unpack_signs(np.array([0], np.uint16)) == one).all()
    assert (oracle.unpack_signs(np.array([0xFFFF], np.uint16)) == neg).all()
    s = oracle.unpack_signs(np.array([0x0005, 0x0001], np.uint16))
    assert s.size == 32 and s[0] == neg and s[1] == one and s[2] == neg and s[16] == neg and s[17] == one


def test_silu_mul_golden_bit_exact(oracle, golden_dir):
    d = os.path.join(golden_dir, "berth_ops")
    g = np.fromfile(os.path.join(d, "silu.gate.bin"), np.uint16)
    u = np.fromfile(os.path.join(d, "silu.up.bin"), np.uint16)
    o = np.fromfile(os.path.join(d, "silu.out.bin"), np.uint16)
    assert g.size == 17408
    got = oracle.silu_mul(g, u, 0.0).view(np.uint16)
    assert int((got != o).sum()) == 0


def test_add_f32_golden_bit_exact(oracle, golden_dir):
    d = os.path.join(golden_dir, "berth_ops")
    a = np.fromfile(os.path.join(d, "add.a.bin"), np.float32)
    b = np.fromfile(os.path.join(d, "add.b.bin"), np.float32)
    c = np.fromfile(os.path.join(d, "add.c.bin"), np.float32)
    assert (oracle.add_f32(a, b).view(np.uint32) == c.view(np.uint32)).all()


def test_hexp_neg_exhaustive(oracle):
    """fp16(exp(-g)) from the fixed fp32 fmaf sequence equals the correctly rounded fp16 exp for
    every fp16 argument except two whose exact value lies within 1e-8 (relative) of a rounding
    midpoint, which no fp32 evaluation can resolve."""
    bits = np.arange(65536, dtype=np.uint16)
    g = bits.view(np.float16).astype(np.float64)
    with np.errstate(over="ignore", invalid="ignore"):
        ref = np.exp(-g).astype(np.float16).view(np.uint16)   # double exp, one rounding
    got = oracle.hexp_neg(bits).view(np.uint16)
    nan = np.isnan(g)
    bad = np.where((got != ref) & ~nan)[0]
    assert sorted(bad.tolist()) == [0x9F79, 0xA5CF]
    assert (np.abs(got[bad].astype(int) - ref[bad].astype(int)) == 1).all()
    assert np.isnan(got[nan].view(np.float16)).all()


def test_gemv_cfg_truth_table(oracle):
    # crates/berth-kernels/src/prefill_lin.rs:386-442
    AMP, ADA, MODE, K, CB, NARROW = 2, 3, 1, 4, 2, 164
    f = oracle.gemv_cfg
    for m in (3, 5, 8):
        assert f(AMP, m, 5120, 17408, K, CB, MODE, NARROW) == -1
        assert f(AMP, m, 17408, 5120, K, CB, MODE, NARROW) == 0
        assert f(AMP, m, 6144, 5120, K, CB, MODE, NARROW) == 0
        assert f(AMP, m, 10240, 5120, K, CB, MODE, NARROW) == 0
    assert f(AMP, 9, 17408, 5120, K, CB, MODE, NARROW) == -1
    assert f(AMP, 2, 17408, 5120, K, CB, MODE, NARROW) == 0
    assert f(AMP, 3, 17408, 5120, K, CB, 0, NARROW) == -1
    assert f(AMP, 3, 5120, 8192, K, CB, MODE, NARROW) == 1
    assert f(ADA, 3, 5120, 8192, K, CB, MODE, NARROW) == -1


def test_gemm_tune_key_known_answer(oracle):
    # crates/berth-kernels/src/lib.rs:224-233: lm_head, device 0, CC_AMPERE = 2, 82 SMs
    assert oracle.gemm_tune_key(1, 5120, 248320, 6, 0, 0, 2, 82, 2) == 0x51F40C1BD7CAE3A7


# ---------------------------------------------------------------- spec v0 restated independently

def _py_states(words, bits):
    stream = []
    for w in words:
        stream += [(int(w) >> (15 - i)) & 1 for i in range(16)]
    L = len(stream)
    out = []
    for t in range(256):
        s = 0
        for i in range(16):
            s = (s << 1) | stream[(t * bits + i) % L]
        out.append(s)
    return out


def _py_codebook(s, cb):
    if cb == 2:
        x = (s * 0x83DCD12D) & 0xFFFFFFFF
        u = sum((x >> (8 * i)) & 0xFF for i in range(4))
        S = float(np.uint16(0x1EEE).view(np.float16))
        B = float(np.uint16(0xC931).view(np.float16))
        h = float(np.uint16(0x6400 + u).view(np.float16))   # = 1024 + u
        return np.float16(np.float64(h) * S + B)      # exact in double, one rounding
    x = (s * 89226354 + 64248484) & 0xFFFFFFFF if cb == 0 else (s * 0xCBAC1FED) & 0xFFFFFFFF
    x = (x & 0x8FFF8FFF) ^ 0x3B603B60
    lo = np.uint16(x & 0xFFFF).view(np.float16)
    hi = np.uint16(x >> 16).view(np.float16)
    return np.float16(np.float32(lo) + np.float32(hi))


def _py_coords(t):
    lane, j = t >> 3, t & 7
    g, q = lane >> 2, lane & 3
    return 2 * q + (j & 1) + 8 * (j >> 2), g + 8 * ((j >> 1) & 1)


@pytest.mark.parametrize("bits", [1, 2, 3, 4, 5, 6, 7, 8])
def test_tile_states_and_decode_vs_python(oracle, bits):
    words = synth.raw_u64(99, f"tile{bits}", 4 * bits).view(np.uint16)[:16 * bits]
    st = oracle.tile_states(words, bits)
    assert list(st) == _py_states(words, bits)
    for cb in (0, 1, 2):
        tile = oracle.decode_tile(words, bits, cb)
        exp = np.zeros((16, 16), np.float16)
        for t, s in enumerate(_py_states(words, bits)):
            r, c = _py_coords(t)
            exp[r, c] = _py_codebook(s, cb)
        assert (tile.view(np.uint16) == exp.view(np.uint16)).all()


def test_tile_coords_is_a_permutation():
    seen = {_py_coords(t) for t in range(256)}
    assert len(seen) == 256


def test_tail_biting_wraps(oracle):
    # the last states of a tile read their low bits from the start of the same tile
    bits = 4
    words = np.zeros(64, np.uint16)
    words[0] = 0xABCD
    st = oracle.tile_states(words, bits)
    assert st[0] == 0xABCD
    assert st[255] == 0x0ABC and st[254] == 0x00AB and st[253] == 0x000A and st[252] == 0


@pytest.mark.parametrize("cb", [0, 1, 2])
def test_codebook_distribution(oracle, cb):
    w = oracle.codebook(np.arange(65536), cb).astype(np.float64)
    assert abs(w.mean()) < 0.02
    assert 0.8 < w.std() < 1.4            # roughly unit variance
    assert np.abs(w).max() < 4.2


def test_codebook_all_states_vs_python(oracle):
    states = np.arange(0, 65536, 97)
    for cb in (0, 1, 2):
        got = oracle.codebook(states, cb)
        exp = np.array([_py_codebook(int(s), cb) for s in states], np.float16)
        assert (got.view(np.uint16) == exp.view(np.uint16)).all()


def test_reconstruct_band_equals_full(oracle):
    K, N, bits = 64, 384, 3
    t = synth.trellis(5, "w", K, N, bits)
    full = oracle.reconstruct(t, K, N, bits, 1)
    band = oracle.reconstruct(t, K, N, bits, 1, n_offset=128, slice_n=256)
    assert (band.view(np.uint16) == full[:, 128:384].view(np.uint16)).all()


def _hadamard(n):
    h = np.array([[1.0]])
    while h.shape[0] < n:
        h = np.block([[h, h], [h, -h]])
    return h


def test_had_r_128_vs_matrix(oracle):
    rows, cols = 3, 384
    x = synth.activations(3, "hx", rows, cols)
    sc = synth.sign_scale(3, "hs", cols)
    H = _hadamard(128) / math.sqrt(128.0)
    xs = x.astype(np.float64) * sc.astype(np.float64)
    exp_pre = np.concatenate([xs[:, b:b + 128] @ H for b in range(0, cols, 128)], axis=1)
    got_pre = oracle.had_r_128(x, sc, True).astype(np.float64)
    assert np.abs(got_pre - exp_pre).max() <= 2e-3 * np.abs(exp_pre).max()
    x32 = x.astype(np.float32)
    exp_post = np.concatenate([x.astype(np.float64)[:, b:b + 128] @ H for b in range(0, cols, 128)], axis=1) * sc.astype(np.float64)
    got_post = oracle.had_r_128(x32, sc, False).astype(np.float64)
    assert np.abs(got_post - exp_post).max() <= 1e-5 * np.abs(exp_post).max()
    # the transform is an involution up to rounding
    back = oracle.had_r_128(oracle.had_r_128(x32, None, False), None, False)
    assert np.abs(back - x32).max() < 1e-4


@pytest.mark.parametrize("bits,cb,out_fp32", [(4, 0, False), (3, 1, True), (5, 2, False), (4, 2, True)])
def test_linear_vs_dense_numpy(oracle, bits, cb, out_fp32):
    M, K, N = 3, 256, 384
    w = synth.linear_weights(11, f"lin{bits}{cb}", K, N, bits)
    x = synth.activations(11, "x", M, K)
    W = oracle.reconstruct(w["trellis"], K, N, bits, cb).astype(np.float64)
    H = _hadamard(128) / math.sqrt(128.0)
    xs = x.astype(np.float64) * w["suh"].astype(np.float64)
    ah = np.concatenate([xs[:, b:b + 128] @ H for b in range(0, K, 128)], axis=1)
    c = ah @ W
    y = np.concatenate([c[:, b:b + 128] @ H for b in range(0, N, 128)], axis=1) * w["svh"].astype(np.float64)
    y64 = oracle.linear_f64(x, w["trellis"], w["suh"], w["svh"], K, N, bits, cb)
    assert np.abs(y64 - y).max() <= 1e-10 * np.abs(y).max()
    got, a_had = oracle.linear(x, w["trellis"], w["suh"], w["svh"], K, N, bits, cb, out_fp32)
    rms = np.sqrt((y64 ** 2).mean())
    err = np.abs(got.astype(np.float64) - y64) / rms
    assert err.max() <= 1e-2 and err.mean() <= 1e-3
    assert (a_had.view(np.uint16) == oracle.had_r_128(x, w["suh"], True).view(np.uint16)).all()


# ---------------------------------------------------------------- MoE pieces

def test_router_logits_and_topk(oracle):
    T, H, E, k = 5, 256, 32, 4
    x = synth.activations(21, "rx", T, H)
    wr = synth.router_weight(21, "rw", H, E)
    logits = oracle.router_logits(x, wr)
    ref = x.astype(np.float64) @ wr.astype(np.float64)
    assert np.abs(logits - ref).max() < 1e-4
    idx, w = oracle.router_topk(logits, k)
    for t in range(T):
        order = sorted(range(E), key=lambda e: (-logits[t, e], e))[:k]
        assert list(idx[t]) == order
        p = np.exp(logits[t].astype(np.float64) - logits[t].max())
        p /= p.sum()
        assert np.allclose(w[t], p[order] / p[order].sum(), rtol=1e-5)
    assert np.allclose(w.sum(axis=1), 1.0, atol=1e-6)


def test_router_topk_ties_go_to_lower_index(oracle):
    logits = np.zeros((2, 16), np.float32)
    logits[1, [3, 7, 9]] = 1.0
    idx, w = oracle.router_topk(logits, 4)
    assert list(idx[0]) == [0, 1, 2, 3]
    assert list(idx[1]) == [3, 7, 9, 0]
    assert np.allclose(w[0], 0.25)


def test_moe_layer_vs_composition(oracle):
    H, I, E, k, bits, cb, T = 128, 128, 4, 2, 4, 0, 3
    wts = synth.moe_layer_weights(31, "moe", H, I, E, k, bits, cb, shared_inter=128)
    x = synth.activations(31, "mx", T, H)
    out, idx, tw = oracle.moe_layer(wts, x)
    exp = np.zeros((T, H), np.float64)
    def expert(xr, pre, e=None):
        sel = (lambda a: a[e]) if e is not None else (lambda a: a)
        g, _ = oracle.linear(xr, sel(wts[f"{pre}gate_trellis"]), sel(wts[f"{pre}gate_suh"]), sel(wts[f"{pre}gate_svh"]), H, I, bits, cb, False)
        u, _ = oracle.linear(xr, sel(wts[f"{pre}up_trellis"]), sel(wts[f"{pre}up_suh"]), sel(wts[f"{pre}up_svh"]), H, I, bits, cb, False)
        h = oracle.silu_mul(g, u)
        y, _ = oracle.linear(h, sel(wts[f"{pre}down_trellis"]), sel(wts[f"{pre}down_suh"]), sel(wts[f"{pre}down_svh"]), I, H, bits, cb, False)
        return y.astype(np.float64)
    for t in range(T):
        for s in range(k):
            exp[t] += float(tw[t, s]) * expert(x[t:t + 1], "", int(idx[t, s]))[0]
        exp[t] += expert(x[t:t + 1], "sh_")[0]
    assert np.abs(out - exp).max() <= 1e-5 * np.abs(exp).max()
    y64 = oracle.moe_layer_f64(wts, x, idx, tw)
    rms = np.sqrt((y64 ** 2).mean())
    err = np.abs(out - y64) / rms
    assert err.max() <= 1e-2 and err.mean() <= 1e-3


def _bf16(a):
    """float32 array -> bfloat16 bit patterns (round to nearest even)."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


@pytest.mark.parametrize("rows,dim", [(1, 5120), (3, 2048), (2, 132)])
def test_rms_norm_oracle_against_float64(oracle, rows, dim):
    """The checker's RMSNorm (one published formula, this build's summation order) against a float64 evaluation of
    y = x / sqrt(mean(x^2) + eps) * (w + bias) * scale: within fp16 rounding; the RES_IN form updates the residual
    exactly (fp32 add) and normalises the updated row; the fp16-input form agrees with the fp32 form on fp16 data."""
    rng = np.random.default_rng(11)
    x = rng.standard_normal((rows, dim)).astype(np.float32) * 3.0
    w32 = (rng.standard_normal(dim) * 0.1).astype(np.float32)
    eps, bias, scale = 1e-6, 1.0, 1.0
    for wbf in (True, False):
        w = _bf16(w32) if wbf else w32.astype(np.float16).view(np.uint16)
        wf = (w.astype(np.uint32) << 16).view(np.float32) if wbf else w.view(np.float16).astype(np.float32)
        y = oracle.rms_norm(x, w, wbf, eps, bias, scale).astype(np.float64)
        x64 = x.astype(np.float64)
        ref = x64 / np.sqrt((x64 ** 2).mean(axis=1, keepdims=True) + eps) * (wf.astype(np.float64) + bias) * scale
        assert np.abs(y - ref).max() <= 2.0 ** -10 * np.abs(ref).max()
        res = rng.standard_normal((rows, dim)).astype(np.float32)
        res0 = res.copy()
        y2 = oracle.rms_norm(x, w, wbf, eps, bias, scale, residual=res)
        assert (res == res0 + x).all()
        assert (y2.view(np.uint16) == oracle.rms_norm(res, w, wbf, eps, bias, scale).view(np.uint16)).all()
    xh = x.astype(np.float16)
    w = _bf16(w32)
    assert (oracle.rms_norm(xh, w, True, eps, bias, scale).view(np.uint16)
            == oracle.rms_norm(xh.astype(np.float32), w, True, eps, bias, scale).view(np.uint16)).all()


def test_sampling_keys_of_the_checker(oracle):
    """exl3o_sample_keys: greedy keys name the arg-max (ties to the lower column, -0 = +0); the Gumbel noise has the
    standard Gumbel's mean and variance, is a pure function of (random, row, column), and independent across rows."""
    rng = np.random.RandomState(5)
    x = rng.randn(3, 4096).astype(np.float32)
    x[1, 7] = x[1, 100] = 9.0
    x[2] = 0.0
    x[2, 5] = -0.0
    keys, scores = oracle.sample_keys(x, 1.0, 0, 0)
    assert (scores == x).all()
    cols = [0xFFFFFFFF - (int(k) & 0xFFFFFFFF) for k in keys]
    assert cols == [int(np.argmax(x[0])), 7, 0]
    keys1, s1 = oracle.sample_keys(x, 1.0, 42, 1)
    g = (s1 - x).astype(np.float64)
    assert abs(g.mean() - 0.5772) < 0.03 and abs(g.std() - 1.2825) < 0.05
    assert abs(np.corrcoef(g[0], g[1])[0, 1]) < 0.05
    assert (oracle.sample_keys(x, 1.0, 42, 1)[1] == s1).all() and (oracle.sample_keys(x, 1.0, 43, 1)[1] != s1).mean() > 0.99
    assert [0xFFFFFFFF - (int(k) & 0xFFFFFFFF) for k in keys1] == [int(np.argmax(s1[r])) for r in range(3)]
    # inv_temp scales the outputs before the noise is added: fmaf(x, inv_temp, g)
    _, s2 = oracle.sample_keys(x, 2.0, 42, 1)
    assert np.allclose(s2 - 2.0 * x.astype(np.float64), g, atol=1e-5)


# ---------------------------------------------------------------- committed golden vectors of the checker itself

def _golden_meta(golden_dir):
    import json
    d = os.path.join(golden_dir, "exl3_spec_v0")
    with open(os.path.join(d, "meta.json")) as f:
        return d, json.load(f)


def test_checker_reproduces_its_committed_golden_vectors(oracle, golden_dir):
    """tests/golden/exl3_spec_v0: the generator run again gives, byte for byte, the committed files and digests (decoded
    tiles of tiny matrices at 3/4/5 bpw for the three codebooks, configuration 0's output row, 64 sampled tiles and the
    digest of its whole decoded matrix, the top-8 tables of configuration 3 at 1/64/1024 tokens)."""
    import hashlib
    import importlib.util
    d, meta = _golden_meta(golden_dir)
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(d, "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    files = mod.generate()
    assert set(files) == set(meta["files"])
    for name, (arr, entry) in files.items():
        m = meta["files"][name]
        raw = np.ascontiguousarray(arr).tobytes()
        with open(os.path.join(d, name), "rb") as f:
            assert f.read() == raw, name
        assert hashlib.sha256(raw).hexdigest() == m["sha256"], name
        for key, value in entry.items():
            if key.startswith("sha256_"):
                assert m[key] == value, (name, key)
