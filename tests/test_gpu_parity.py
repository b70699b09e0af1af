"""Parity of the CUDA path (through the C ABI) with the CPU oracle on the same seeded inputs.

Integer/byte work (decoded weight tiles, rotated activations, silu_mul, add) must be
bit-exact; fp32-accumulated linear outputs must be within max relative error 1e-2 and mean
relative error 1e-3 of the fp64 evaluation, errors taken relative to the RMS of the fp64 output.
"""
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from berth_b200 import Codebook, OutDtype, kernels, synth   # noqa: E402
from tests.gpu_util import MAX_REL, MEAN_REL, assert_close, dev, host_u16, rel_errors, run_linear   # noqa: E402


# ---------------------------------------------------------------- decoded weight tiles: bit-exact

@pytest.mark.parametrize("bits", [1, 2, 3, 4, 5, 6, 7, 8])
@pytest.mark.parametrize("cb", [0, 1, 2])
def test_reconstruct_bit_exact_small(oracle, bits, cb):
    K, N = 128, 256
    t = synth.trellis(1234, f"rec{bits}", K, N, bits)
    out = torch.zeros((K, N), dtype=torch.float16, device="cuda")
    kernels.prefill_lin.reconstruct(out, dev(t), K, N, N, 0, bits, cb)
    exp = oracle.reconstruct(t, K, N, bits, cb).view(np.uint16)
    assert int((host_u16(out) != exp).sum()) == 0


def test_reconstruct_column_band(oracle):
    K, N, bits, cb = 64, 640, 4, 2
    t = synth.trellis(1234, "band", K, N, bits)
    out = torch.zeros((K, 256), dtype=torch.float16, device="cuda")
    kernels.prefill_lin.reconstruct(out, dev(t), K, 256, N, 384, bits, cb)
    exp = oracle.reconstruct(t, K, N, bits, cb, n_offset=384, slice_n=256).view(np.uint16)
    assert int((host_u16(out) != exp).sum()) == 0


@pytest.mark.parametrize("cb", [0, 1, 2])
def test_reconstruct_bit_exact_config0(oracle, cb):
    """All 122,880 tiles of the 5120 x 6144, 4 bpw matrix."""
    K, N, bits = 5120, 6144, 4
    t = synth.trellis(1234, "c0.trellis", K, N, bits)
    out = torch.zeros((K, N), dtype=torch.float16, device="cuda")
    kernels.prefill_lin.reconstruct(out, dev(t), K, N, N, 0, bits, cb)
    exp = oracle.reconstruct(t, K, N, bits, cb).view(np.uint16)
    assert int((host_u16(out) != exp).sum()) == 0


# ---------------------------------------------------------------- Hadamard: bit-exact

@pytest.mark.parametrize("fp32", [False, True])
@pytest.mark.parametrize("pre", [False, True])
def test_had_r_128_bit_exact(oracle, fp32, pre):
    rows, cols = 5, 640
    x = synth.activations(7, "hadx", rows, cols)
    sc = synth.sign_scale(7, "hads", cols)
    xin = x.astype(np.float32) if fp32 else x
    d_in = dev(xin)
    d_out = torch.empty_like(d_in)
    kernels.prefill_lin.had_r_128(d_in, d_out, dev(sc), pre, rows, cols, fp32)
    exp = oracle.had_r_128(xin, sc, pre)
    got = d_out.cpu().numpy()
    if fp32:
        assert (got.view(np.uint32) == exp.view(np.uint32)).all()
    else:
        assert (got.view(np.uint16) == exp.view(np.uint16)).all()
    # in place
    kernels.prefill_lin.had_r_128(d_in, d_in, dev(sc), pre, rows, cols, fp32)
    assert torch.equal(d_in, d_out)


# ---------------------------------------------------------------- silu_mul / add: bit-exact, golden

def test_silu_mul_golden_and_oracle(oracle, golden_dir):
    d = os.path.join(golden_dir, "berth_ops")
    g = np.fromfile(os.path.join(d, "silu.gate.bin"), np.uint16)
    u = np.fromfile(os.path.join(d, "silu.up.bin"), np.uint16)
    o = np.fromfile(os.path.join(d, "silu.out.bin"), np.uint16)
    dg, du = dev(g), dev(u)
    out = torch.empty_like(dg)
    kernels.ops.silu_mul(dg, du, out, g.size, 0.0)
    assert int((host_u16(out) != o).sum()) == 0
    # aliasing: out may be gate
    kernels.ops.silu_mul(dg, du, dg, g.size, 0.0)
    assert int((host_u16(dg) != o).sum()) == 0
    # every finite fp16 gate value against the oracle, two different up values
    allg = np.arange(65536, dtype=np.uint16)
    fin = np.isfinite(allg.view(np.float16))
    allg = allg[fin]
    if allg.size & 1:
        allg = allg[:-1]
    for upv in (1.0, -0.3333):
        up = np.full(allg.size, upv, np.float16)
        out = torch.empty(allg.size, dtype=torch.float16, device="cuda")
        kernels.ops.silu_mul(dev(allg), dev(up), out, allg.size, 0.0)
        exp = oracle.silu_mul(allg, up).view(np.uint16)
        got = host_u16(out)
        both_nan = np.isnan(got.view(np.float16)) & np.isnan(exp.view(np.float16))
        assert ((got == exp) | both_nan).all()
    # clamp
    x = synth.activations(3, "sg", 1, 4096).ravel() * np.float16(4)
    y = synth.activations(3, "su", 1, 4096).ravel() * np.float16(4)
    out = torch.empty(4096, dtype=torch.float16, device="cuda")
    kernels.ops.silu_mul(dev(x), dev(y), out, 4096, 2.5)
    assert (host_u16(out) == oracle.silu_mul(x, y, 2.5).view(np.uint16)).all()


def test_add_f32_golden(golden_dir):
    d = os.path.join(golden_dir, "berth_ops")
    a = np.fromfile(os.path.join(d, "add.a.bin"), np.float32)
    b = np.fromfile(os.path.join(d, "add.b.bin"), np.float32)
    c = np.fromfile(os.path.join(d, "add.c.bin"), np.float32)
    da, db = dev(a), dev(b)
    kernels.ops.add_f32(da, db, da, a.size)   # c aliases a
    assert (da.cpu().numpy().view(np.uint32) == c.view(np.uint32)).all()


# ---------------------------------------------------------------- the linear

@pytest.mark.parametrize("m", [1, 2, 5, 8, 9, 16, 17, 32])
@pytest.mark.parametrize("bits,cb,out_fp32", [(4, 0, False), (4, 2, True), (3, 1, False), (5, 2, False), (6, 2, True)])
def test_linear_small_vs_oracle(oracle, m, bits, cb, out_fp32):
    K, N = 512, 384
    w = synth.linear_weights(1234, f"lin{bits}{cb}", K, N, bits)
    x = synth.activations(1234, f"x{m}", m, K)
    c, ah = run_linear(x, w, bits, cb, out_fp32)
    y64 = oracle.linear_f64(x, w["trellis"], w["suh"], w["svh"], K, N, bits, cb)
    mx, mean = rel_errors(c, y64)
    assert mx <= MAX_REL and mean <= MEAN_REL, (mx, mean)
    exp_c, exp_ah = oracle.linear(x, w["trellis"], w["suh"], w["svh"], K, N, bits, cb, out_fp32)
    assert (ah == exp_ah.view(np.uint16)).all()          # rotated activations: bit-exact
    # against the fp32 oracle the only difference is summation order
    rms = np.sqrt((y64 ** 2).mean())
    assert np.abs(c.astype(np.float64) - exp_c.astype(np.float64)).max() <= 4e-3 * rms
    assert "k_exl3_gemv" in kernels.last_launch()   # a matrix this small stays on the decode GEMV at every row count


@pytest.mark.parametrize("m", [17, 24, 32])
@pytest.mark.parametrize("K,N,bits,cb,out_fp32", [(5120, 2048, 4, 2, False), (2048, 5120, 4, 0, True), (17408, 640, 3, 1, True),
                                                  (1024, 12288, 8, 2, False), (256, 39936, 5, 2, True), (12288, 1024, 6, 2, False),
                                                  (1152, 8704, 7, 0, True), (640, 19072, 2, 1, False), (8192, 2304, 1, 2, True)])
def test_small_batch_tensor_path_vs_oracle(oracle, m, K, N, bits, cb, out_fp32):
    """17..32 rows of a matrix with at least eight weight stages per SM run on the persistent split-K tensor-core kernel:
    shapes whose bands are shared by many CTAs (few bands, long K), held whole by one CTA (many bands, short K) and
    mixtures; checked against the fp64 oracle, the rotated rows bit for bit, and for run-to-run identical bits (the slabs
    of a shared band are summed in CTA order)."""
    w = synth.linear_weights(1234, f"sk{bits}{cb}.{K}.{N}", K, N, bits)
    x = synth.activations(1234, f"sk.x{m}.{K}", m, K)
    c, ah = run_linear(x, w, bits, cb, out_fp32)
    assert "k_exl3_gemm_tc_splitk" in kernels.last_launch()
    y64 = oracle.linear_f64(x, w["trellis"], w["suh"], w["svh"], K, N, bits, cb)
    assert_close(c, y64)
    _, exp_ah = oracle.linear(x[:1], w["trellis"], w["suh"], w["svh"], K, N, bits, cb, out_fp32)
    assert (ah[:1] == exp_ah.view(np.uint16)).all()
    for _ in range(3):
        c2, _ = run_linear(x, w, bits, cb, out_fp32)
        assert (c2.view(np.uint16 if not out_fp32 else np.uint32) == c.view(np.uint16 if not out_fp32 else np.uint32)).all()
    assert kernels.device_status(torch.cuda.current_device()) == 0


@pytest.mark.parametrize("bits", [1, 2, 7, 8])
def test_linear_every_bitrate(oracle, bits):
    K, N, m, cb = 256, 256, 3, 2
    w = synth.linear_weights(1234, f"rate{bits}", K, N, bits)
    x = synth.activations(1234, "xr", m, K)
    c, _ = run_linear(x, w, bits, cb, True)
    y64 = oracle.linear_f64(x, w["trellis"], w["suh"], w["svh"], K, N, bits, cb)
    mx, mean = rel_errors(c, y64)
    assert mx <= MAX_REL and mean <= MEAN_REL, (mx, mean)


def test_linear_split_k_shapes(oracle):
    """Tall (deep split-K, chunked activations) and wide (no split) shapes."""
    for (K, N, m) in ((4096, 128, 4), (4352, 256, 32), (128, 2048, 1), (2176, 640, 17)):
        w = synth.linear_weights(1234, f"sk{K}x{N}", K, N, 4)
        x = synth.activations(1234, f"skx{K}", m, K)
        c, ah = run_linear(x, w, 4, 0, False)
        y64 = oracle.linear_f64(x, w["trellis"], w["suh"], w["svh"], K, N, 4, 0)
        mx, mean = rel_errors(c, y64)
        assert mx <= MAX_REL and mean <= MEAN_REL, (K, N, m, mx, mean)


def test_linear_is_deterministic_and_counters_reset():
    K, N, m = 2048, 512, 3
    w = synth.linear_weights(1234, "det", K, N, 4)
    x = synth.activations(1234, "detx", m, K)
    first, _ = run_linear(x, w, 4, 1, True)
    for _ in range(3):
        again, _ = run_linear(x, w, 4, 1, True)
        assert (again.view(np.uint32) == first.view(np.uint32)).all()


@pytest.mark.parametrize("cb", [0, 2])
def test_linear_config0_vs_oracle(oracle, cb):
    """benchmark configuration 0: in=5120, out=6144, 4 bpw, one fp16 row, fp16 out."""
    K, N, bits = 5120, 6144, 4
    w = synth.linear_weights(1234, "c0", K, N, bits)
    x = synth.activations(1234, "c0.x", 1, K)
    c, ah = run_linear(x, w, bits, cb, False)
    y64 = oracle.linear_f64(x, w["trellis"], w["suh"], w["svh"], K, N, bits, cb)
    mx, mean = rel_errors(c, y64)
    assert mx <= MAX_REL and mean <= MEAN_REL, (mx, mean)
    exp_ah = oracle.had_r_128(x, w["suh"], True)
    assert (ah == exp_ah.view(np.uint16)).all()


def test_prefill_entry_point_rows(oracle):
    """berth_prefill_exl3_linear over row counts berth's prefill tests use (2, 47, 144, 145)."""
    K, N, bits, cb = 256, 256, 4, 2
    w = synth.linear_weights(1234, "pf", K, N, bits)
    for m in (2, 47, 144, 145):
        x = synth.activations(1234, f"pfx{m}", m, K)
        c, ah = run_linear(x, w, bits, cb, m % 2 == 0, prefill=True)
        y64 = oracle.linear_f64(x, w["trellis"], w["suh"], w["svh"], K, N, bits, cb)
        mx, mean = rel_errors(c, y64)
        assert mx <= MAX_REL and mean <= MEAN_REL, (m, mx, mean)
        assert (ah == oracle.had_r_128(x, w["suh"], True).view(np.uint16)).all()


# ---------------------------------------------------------------- full 27B shapes: properties

def _torch_reference(x, w, bits, cb):
    """y = H(H(x*suh) W) svh evaluated on the GPU in fp32/fp64 from the library's own bit-exact-checked
    reconstruct output: a size-independent cross-check of the fused kernel at full size."""
    K, N = w["size_k"], w["size_n"]
    W = torch.empty((K, N), dtype=torch.float16, device="cuda")
    kernels.prefill_lin.reconstruct(W, dev(w["trellis"]), K, N, N, 0, bits, cb)
    H = torch.tensor([[1.0]], dtype=torch.float64, device="cuda")
    while H.shape[0] < 128:
        H = torch.cat([torch.cat([H, H], 1), torch.cat([H, -H], 1)], 0)
    H = H / (128.0 ** 0.5)
    xs = dev(x).double() * dev(w["suh"]).double()
    ah = (xs.view(-1, K // 128, 128) @ H).view(-1, K)
    c = ah @ W.double()
    y = (c.view(-1, N // 128, 128) @ H).view(-1, N) * dev(w["svh"]).double()
    return y.cpu().numpy()


@pytest.mark.parametrize("name,K,N,out_fp32", [("gate", 5120, 17408, False), ("down", 17408, 5120, True),
                                               ("k", 5120, 1024, False), ("o", 6144, 5120, True)])
@pytest.mark.parametrize("m", [1, 8, 32])
def test_linear_27b_shapes_full_size(name, K, N, out_fp32, m):
    bits, cb = 4, 2
    w = synth.linear_weights(1234, f"l0.{name}", K, N, bits)
    x = synth.activations(1234, f"l0.{name}.x", m, K)
    c, _ = run_linear(x, w, bits, cb, out_fp32)
    y64 = _torch_reference(x, w, bits, cb)
    mx, mean = rel_errors(c, y64)
    assert mx <= MAX_REL and mean <= MEAN_REL, (mx, mean)
    # linearity in the activations: f(x1 + x2) = f(x1) + f(x2) up to rounding
    if m == 1:
        x2 = synth.activations(1234, f"l0.{name}.x2", 1, K)
        c2, _ = run_linear(x2, w, bits, cb, True)
        c1, _ = run_linear(x, w, bits, cb, True)
        xs = (x.astype(np.float32) + x2.astype(np.float32)).astype(np.float16)
        cs, _ = run_linear(xs, w, bits, cb, True)
        rms = np.sqrt((cs.astype(np.float64) ** 2).mean())
        assert np.abs(cs - (c1 + c2)).max() <= 5e-3 * rms


def test_no_bounded_wait_ran_out():
    """Every pipeline wait inside the decode kernels is bounded; none may have expired so far."""
    K, N = 1024, 512
    w = synth.linear_weights(1234, "status", K, N, 4)
    run_linear(synth.activations(1234, "status.x", 2, K), w, 4, 0, False)
    assert kernels.device_status(torch.cuda.current_device()) == 0


# ---------------------------------------------------------------- tensor-core prefill GEMM (rows > 32)

@pytest.mark.parametrize("m,K,N,bits,cb,out_fp32", [(33, 128, 128, 4, 2, True), (128, 256, 256, 4, 0, False),
                                                   (200, 512, 384, 3, 1, True), (513, 1024, 256, 5, 2, False),
                                                   (1499, 512, 128, 4, 2, True), (640, 256, 640, 6, 0, False)])
def test_prefill_gemm_vs_oracle(oracle, m, K, N, bits, cb, out_fp32):
    w = synth.linear_weights(1234, f"tc{K}x{N}b{bits}", K, N, bits)
    x = synth.activations(1234, f"tc.x{m}", m, K, outlier_frac=0.001)
    c, ah = run_linear(x, w, bits, cb, out_fp32, prefill=True)
    assert "k_exl3_gemm_tc" in kernels.prefill_lin.last_launch()
    assert kernels.device_status(torch.cuda.current_device()) == 0
    y64 = oracle.linear_f64(x, w["trellis"], w["suh"], w["svh"], K, N, bits, cb)
    mx, mean = rel_errors(c, y64)
    assert mx <= MAX_REL and mean <= MEAN_REL, (mx, mean)
    assert (ah == oracle.had_r_128(x, w["suh"], True).view(np.uint16)).all()


def test_prefill_gemm_matches_decode_kernel():
    """The GEMM (rows > 32) and the GEMV (rows <= 32) agree row by row."""
    K, N, bits, cb = 1024, 512, 4, 2
    w = synth.linear_weights(1234, "tcvsgemv", K, N, bits)
    x = synth.activations(1234, "tcvsgemv.x", 96, K)
    big, _ = run_linear(x, w, bits, cb, True, prefill=True)
    rms = np.sqrt((big.astype(np.float64) ** 2).mean())
    for r0 in (0, 32, 64):
        small, _ = run_linear(x[r0:r0 + 32], w, bits, cb, True)
        assert np.abs(big[r0:r0 + 32] - small).max() <= 1e-3 * rms


# ---------------------------------------------------------------- sliced multi-linear (berth_ops_mgemm)
@pytest.mark.parametrize("cb", [2, 0])
@pytest.mark.parametrize("m,out_fp32", [(1, True), (1, False), (3, False), (5, False), (20, True)])
def test_sliced_multi_linear_vs_oracle(oracle, m, out_fp32, cb):
    """Three linears sharing one input in one launch (the q / k / v bundle of berth's attention layers,
    crates/berth-kernels/tests/ops.rs:250-345, at reduced sizes): every source's output against the fp64
    evaluation of that source alone, and the rotated input slab of every source bit for bit.  MUL1 sources run on the
    integer-path multi-matrix launch up to four rows, everything else as column slices through berth_ops_mgemm."""
    from berth_b200.engine import Exl3Linear, Gpu, SlicedMultiLinear
    K, bits = 512, 4
    widths = (1536, 512, 256)
    gpu = Gpu(torch.cuda.current_device())
    ws = [synth.linear_weights(1234, f"mg{i}", K, n, bits) for i, n in enumerate(widths)]
    lins = [Exl3Linear(gpu, f"mg{i}", w["trellis"], w["suh"], w["svh"], bits, Codebook(cb), max_rows=m) for i, w in enumerate(ws)]
    out = OutDtype.F32 if out_fp32 else OutDtype.F16
    ml = SlicedMultiLinear(gpu, lins, out, max_rows=m)
    assert ml.width == 256 and ml.slices == 9
    x = synth.activations(1234, f"mg.x{m}", m, K)
    outs = ml.forward_n(gpu, m, dev(x))
    torch.cuda.synchronize()
    assert kernels.device_status(torch.cuda.current_device()) == 0
    if cb == 2 and m <= SlicedMultiLinear.MULTI_ROWS:
        assert "3 matrices" in kernels.last_launch()
    else:
        assert "sliced" in kernels.ops.last_launch()
    ah = host_u16(ml.a_had).reshape(len(ws), m, K)
    for i, w in enumerate(ws):
        y64 = oracle.linear_f64(x, w["trellis"], w["suh"], w["svh"], K, widths[i], bits, cb)
        mx, mean = rel_errors(outs[i][:m].float().cpu().numpy(), y64)
        assert mx <= MAX_REL and mean <= MEAN_REL, (i, mx, mean)
        assert (ah[i] == oracle.had_r_128(x, w["suh"], True).view(np.uint16)).all()


@pytest.mark.parametrize("m,per_matrix_input,out_fp32,cb", [(1, False, True, 2), (5, True, False, 2), (20, True, True, 0), (2, False, False, 1)])
def test_uniform_multi_linear_vs_oracle(oracle, m, per_matrix_input, out_fp32, cb):
    """berth_ops_mgemm in its uniform mode (all slice lists null): several equally shaped matrices, outputs one behind the
    other, one input for all matrices or one each; every matrix against the fp64 evaluation of that matrix alone, and its
    rotated-input slab bit for bit."""
    K, N, bits, nmat = 512, 512, 4, 3
    ws = [synth.linear_weights(1234, f"uni{i}", K, N, bits) for i in range(nmat)]
    xs = synth.activations(1234, f"uni.x{m}", (nmat if per_matrix_input else 1) * m, K).reshape(-1, m, K)
    td, sd, vd = [dev(w["trellis"]) for w in ws], [dev(w["suh"]) for w in ws], [dev(w["svh"]) for w in ws]
    u64 = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device="cuda")
    dt = torch.float32 if out_fp32 else torch.float16
    c = torch.full((nmat, m, N), float("nan"), dtype=dt, device="cuda")
    ah = torch.zeros((nmat, m, K), dtype=torch.float16, device="cuda")
    xd = dev(np.ascontiguousarray(xs))
    tag = kernels.ops.exl3_mgemm(xd, u64(td), c, u64(sd), ah, u64(vd), m, K, N, bits, Codebook(cb), OutDtype.F32 if out_fp32 else OutDtype.F16,
                                 nmat if per_matrix_input else 1, nmat, None, None, None, None, 0)
    torch.cuda.synchronize()
    assert tag in (1, 2, 4) and "k_uniform_lists" in kernels.ops.last_launch()
    assert kernels.device_status(torch.cuda.current_device()) == 0
    got, gah = c.float().cpu().numpy(), host_u16(ah).reshape(nmat, m, K)
    for i, w in enumerate(ws):
        x = xs[i if per_matrix_input else 0]
        y64 = oracle.linear_f64(x, w["trellis"], w["suh"], w["svh"], K, N, bits, cb)
        assert_close(got[i], y64, f"matrix {i}")
        assert (gah[i] == oracle.had_r_128(x, w["suh"], True).view(np.uint16)).all()


@pytest.mark.parametrize("m,k,n,ldc,out_fp32", [(5, 64, 48, 48, False), (130, 256, 512, 640, True), (47, 5120, 128, 128, False)])
def test_prefill_hgemm_vs_numpy(m, k, n, ldc, out_fp32):
    """berth_prefill_hgemm: c[m][ldc] = a[m][k] . b[k][n] in fp16 with fp32 accumulation; columns past n stay untouched."""
    a = synth.activations(77, f"hg.a{m}", m, k)
    b = (synth.activations(77, f"hg.b{k}", k, n).astype(np.float32) / np.sqrt(k)).astype(np.float16)
    dt = torch.float32 if out_fp32 else torch.float16
    c = torch.full((m, ldc), -7.0, dtype=dt, device="cuda")
    kernels.prefill_lin.hgemm(dev(a), dev(b), c, m, k, n, ldc, OutDtype.F32 if out_fp32 else OutDtype.F16)
    torch.cuda.synchronize()
    assert kernels.prefill_lin.last_launch() == "cublasGemmEx"
    got = c.float().cpu().numpy()
    ref = a.astype(np.float64) @ b.astype(np.float64)
    mx, mean = rel_errors(got[:, :n], ref)
    assert mx <= MAX_REL and mean <= MEAN_REL, (mx, mean)
    assert (got[:, n:] == -7.0).all()


def test_lm_head_shape_6bpw_against_decoded_slices():
    """The lm_head regime of berth (crates/berth-kernels/csrc/gemm_k6.cu:1-34: K = 6 bpw, N = 248320, one row): far
    too large for the CPU checker, so three 128-column slices are decoded with berth_prefill_reconstruct (bit-exact
    against the checker at small sizes) and multiplied in fp64 on the GPU; the full launch must agree on them."""
    K, N, bits, cb = 5120, 248320, 6, 2
    w = synth.linear_weights(1234, "lmh", K, N, bits)
    x = synth.activations(1234, "lmh.x", 1, K)
    c, ah = run_linear(x, w, bits, cb, True)
    assert kernels.device_status(torch.cuda.current_device()) == 0
    assert np.isfinite(c).all()
    td = dev(w["trellis"])
    a_rot = torch.from_numpy(ah.view(np.float16).astype(np.float64)).cuda()          # H128(x * suh) / sqrt(128), [1][K]
    hmat = torch.ones((1, 1), dtype=torch.float64, device="cuda")
    for _ in range(7):
        hmat = torch.cat((torch.cat((hmat, hmat), 1), torch.cat((hmat, -hmat), 1)), 0)
    for n0 in (0, 128 * 977, N - 128):
        wt = torch.empty((K, 128), dtype=torch.float16, device="cuda")
        rc = _lib_reconstruct(wt, td, K, 128, N, n0, bits, cb)
        assert rc == 0
        y = (a_rot @ wt.double())                                                      # [1][128]
        y = (y @ hmat) / np.sqrt(128.0) * torch.from_numpy(w["svh"][n0:n0 + 128].astype(np.float64)).cuda()
        mx, mean = rel_errors(c[:, n0:n0 + 128], y.cpu().numpy())
        assert mx <= MAX_REL and mean <= MEAN_REL, (n0, mx, mean)


def _lib_reconstruct(out, trellis, size_k, slice_n, full_n, n_offset, bits, cb):
    from berth_b200 import _lib
    return _lib.lib().berth_prefill_reconstruct(out.data_ptr(), trellis.data_ptr(), size_k, slice_n, full_n, n_offset, bits, cb, None)


# ---------------------------------------------------------------- from a checkpoint on disk

def test_linear_loaded_from_a_checkpoint(oracle, tmp_path):
    """A linear written as a safetensors checkpoint with packed input signs and an fp16 output scale, read back by
    the library's checkpoint reader and run: the same bits as the linear run from the arrays, and parity with the
    oracle on what was read."""
    from berth_b200.checkpoint import Checkpoint
    from tests.test_checkpoint_host import t, write_safetensors
    K, N, bits, cb, m = 512, 384, 4, 2, 3
    w = synth.linear_weights(1234, "ckpt", K, N, bits)
    su = (synth.raw_u64(1234, "ckpt.su", K // 16) & 0xFFFF).astype(np.uint16)
    write_safetensors(tmp_path / "model.safetensors", [
        t("model.layers.0.mlp.gate_proj.trellis", "I16", (K // 16, N // 16, 16 * bits), w["trellis"].view(np.int16)),
        t("model.layers.0.mlp.gate_proj.su", "I16", (K // 16,), su.view(np.int16)),
        t("model.layers.0.mlp.gate_proj.svh", "F16", (N,), w["svh"].view(np.float16)),
        t("model.layers.0.mlp.gate_proj.mul1", "I32", ())])
    with Checkpoint.open(str(tmp_path)) as ck:
        lin = ck.linear("model.layers.0.mlp.gate_proj")
        assert (lin.k, int(lin.codebook), lin.input_packed, lin.output_packed) == (4.0, 2, True, False)
        got = ck.load_linear(lin.prefix)
    assert (got["trellis"].reshape(-1) == w["trellis"].reshape(-1)).all() and (got["svh"] == w["svh"].view(np.uint16)).all()
    assert (got["suh"] == oracle.unpack_signs(su)).all()
    x = synth.activations(1234, "ckpt.x", m, K)
    c, ah = run_linear(x, dict(got, size_k=K, size_n=N), got["bits"], got["cb"], False)
    exp_c, exp_ah = oracle.linear(x, got["trellis"], got["suh"], got["svh"], K, N, bits, cb, False)
    assert (ah == exp_ah.view(np.uint16)).all()
    y64 = oracle.linear_f64(x, got["trellis"], got["suh"], got["svh"], K, N, bits, cb)
    mx, mean = rel_errors(c, y64)
    assert mx <= MAX_REL and mean <= MEAN_REL, (mx, mean)


# ---------------------------------------------------------------- arg-max in the finishing step

def _argmax_run(x, w, bits, cb, out_fp32, with_c=True):
    m, k = x.shape
    n = w["size_n"]
    xd, td, sd, vd = dev(x), dev(w["trellis"]), dev(w["suh"]), dev(w["svh"])
    c = torch.full((m, n), float("nan"), dtype=torch.float32 if out_fp32 else torch.float16, device="cuda")
    ah = torch.zeros((m, k), dtype=torch.float16, device="cuda")
    best = torch.full((m,), -1, dtype=torch.int64, device="cuda")     # the call zeroes the keys itself
    kernels.exl3_linear_argmax(xd, td, c if with_c else None, sd, ah, vd, best, m, k, n, bits, Codebook(cb),
                               OutDtype.F32 if out_fp32 else OutDtype.F16)
    torch.cuda.synchronize()
    assert kernels.device_status(torch.cuda.current_device()) == 0
    return c.cpu().numpy(), [kernels.argmax_key_decode(int(v)) for v in best.cpu().numpy().view(np.uint64)]


@pytest.mark.parametrize("m", [1, 2, 7, 32])
@pytest.mark.parametrize("bits,cb,out_fp32,K,N", [(4, 2, True, 512, 384), (6, 2, False, 1024, 2048), (3, 0, True, 256, 128),
                                                  (4, 1, False, 2048, 6144)])
def test_linear_argmax_matches_the_stored_outputs(m, bits, cb, out_fp32, K, N):
    """The key of every row = (largest stored output, lowest column holding it); the outputs themselves are the
    bits of the plain linear wherever that runs the decode kernel too (from 17 rows a large matrix goes through the
    split-K tensor-core kernel: same values within the accumulation tolerance); without an output buffer the keys
    are the same."""
    w = synth.linear_weights(1234, f"am{bits}{cb}{K}", K, N, bits)
    x = synth.activations(1234, f"am.x{m}", m, K)
    plain, _ = run_linear(x, w, bits, cb, out_fp32)
    same_kernel = "k_exl3_gemv" in kernels.last_launch()
    c, keys = _argmax_run(x, w, bits, cb, out_fp32)
    if same_kernel:
        assert (c.view(np.uint32 if out_fp32 else np.uint16) == plain.view(np.uint32 if out_fp32 else np.uint16)).all()
    else:
        rms = np.sqrt((plain.astype(np.float64) ** 2).mean())
        assert np.abs(c.astype(np.float64) - plain.astype(np.float64)).max() <= 4e-3 * rms
    for r, (tok, val) in enumerate(keys):
        assert tok == int(np.argmax(c[r])) and val == float(c[r, tok]), (r, tok, val)
    _, keys_only = _argmax_run(x, w, bits, cb, out_fp32, with_c=False)
    assert keys_only == keys
    assert "arg-max" in kernels.last_launch()


@pytest.mark.parametrize("m", [1, 3, 32])
@pytest.mark.parametrize("bits,cb,out_fp32,K,N", [(4, 2, True, 512, 384), (6, 2, False, 1024, 2048), (3, 0, True, 256, 128),
                                                  (4, 1, False, 1024, 6144)])
def test_linear_sample_gumbel_keys_match_the_checker(oracle, m, bits, cb, out_fp32, K, N):
    """berth_exl3_linear_sample, mode 1: every row's key is, bit for bit, the checker's key for the outputs the call
    stored (score = output * inv_temp + Gumbel noise of (random, row, column)); mode 0 gives the greedy keys of
    berth_exl3_linear_argmax; another `random` draws other tokens; without an output buffer the keys are the same."""
    w = synth.linear_weights(1234, f"gs{bits}{cb}{K}", K, N, bits)
    x = synth.activations(1234, f"gs.x{m}", m, K)
    xd, td, sd, vd = dev(x), dev(w["trellis"]), dev(w["suh"]), dev(w["svh"])
    dt = torch.float32 if out_fp32 else torch.float16
    out = OutDtype.F32 if out_fp32 else OutDtype.F16

    def run(inv_temp, random, mode, with_c=True):
        c = torch.full((m, N), float("nan"), dtype=dt, device="cuda") if with_c else None
        ah = torch.zeros((m, K), dtype=torch.float16, device="cuda")
        best = torch.full((m,), -1, dtype=torch.int64, device="cuda")
        kernels.exl3_linear_sample(xd, td, c, sd, ah, vd, best, m, K, N, bits, Codebook(cb), out, inv_temp, random, mode)
        torch.cuda.synchronize()
        return (None if c is None else c.float().cpu().numpy()), best.cpu().numpy().view(np.uint64)

    c, keys = run(0.7, 20240517, 1)
    assert "Gumbel" in kernels.last_launch()
    exp_keys, scores = oracle.sample_keys(c, 0.7, 20240517, 1)
    assert (keys == exp_keys).all()
    for r in range(m):
        tok, val = kernels.argmax_key_decode(int(keys[r]))
        assert tok == int(np.argmax(scores[r])) and val == float(scores[r, tok])
    _, keys_no_c = run(0.7, 20240517, 1, with_c=False)
    assert (keys_no_c == keys).all()
    c2, keys2 = run(0.7, 99, 1)
    assert (keys2 == oracle.sample_keys(c2, 0.7, 99, 1)[0]).all()
    if N >= 2048:
        assert (keys2 != keys).any()
    cg, greedy = run(1.0, 0, 0)
    assert (greedy == oracle.sample_keys(cg, 1.0, 0, 0)[0]).all()
    assert [kernels.argmax_key_decode(int(k))[0] for k in greedy] == [int(np.argmax(cg[r])) for r in range(m)]
    assert kernels.device_status(torch.cuda.current_device()) == 0


def test_linear_sample_draws_follow_the_softmax():
    """Gumbel arg-max over many values of `random` draws tokens with the softmax probabilities of the row: the
    empirical frequencies of the most likely tokens agree with softmax(outputs * inv_temp) within sampling error."""
    K, N, bits, cb, inv_temp = 256, 128, 4, 2, 0.5
    w = synth.linear_weights(1234, "gsd", K, N, bits)
    x = synth.activations(1234, "gsd.x", 1, K)
    xd, td, sd, vd = dev(x), dev(w["trellis"]), dev(w["suh"]), dev(w["svh"])
    c = torch.empty((1, N), dtype=torch.float32, device="cuda")
    ah = torch.zeros((1, K), dtype=torch.float16, device="cuda")
    best = torch.zeros((1,), dtype=torch.int64, device="cuda")
    draws = 4000
    counts = np.zeros(N)
    for r in range(draws):
        kernels.exl3_linear_sample(xd, td, c, sd, ah, vd, best, 1, K, N, bits, Codebook(cb), OutDtype.F32, inv_temp, 7919 * r + 1, 1)
        counts[kernels.argmax_key_decode(int(best.cpu().numpy().view(np.uint64)[0]))[0]] += 1
    logits = c.cpu().numpy()[0].astype(np.float64) * inv_temp
    p = np.exp(logits - logits.max())
    p /= p.sum()
    top = np.argsort(-p)[:5]
    for t in top:
        sigma = np.sqrt(p[t] * (1 - p[t]) / draws)
        assert abs(counts[t] / draws - p[t]) <= 5 * sigma + 1e-3, (t, counts[t] / draws, p[t])


def test_linear_sample_fails_closed():
    K, N = 256, 128
    w = synth.linear_weights(1234, "gsf", K, N, 4)
    xd, td, sd, vd = dev(synth.activations(1234, "gsf.x", 1, K)), dev(w["trellis"]), dev(w["suh"]), dev(w["svh"])
    c = torch.empty((1, N), dtype=torch.float32, device="cuda")
    ah = torch.zeros((1, K), dtype=torch.float16, device="cuda")
    best = torch.zeros((1,), dtype=torch.int64, device="cuda")
    with pytest.raises(kernels.Error, match="mode must be 0 or 1"):
        kernels.exl3_linear_sample(xd, td, c, sd, ah, vd, best, 1, K, N, 4, Codebook(2), OutDtype.F32, 1.0, 1, 2)
    with pytest.raises(kernels.Error, match="inv_temp"):
        kernels.exl3_linear_sample(xd, td, c, sd, ah, vd, best, 1, K, N, 4, Codebook(2), OutDtype.F32, 0.0, 1, 1)
    with pytest.raises(kernels.Error, match="null"):
        kernels.exl3_linear_sample(xd, td, c, sd, ah, vd, None, 1, K, N, 4, Codebook(2), OutDtype.F32, 1.0, 1, 1)
    with pytest.raises(kernels.Error, match="size_m"):
        kernels.exl3_linear_sample(xd, td, c, sd, ah, vd, best, 33, K, N, 4, Codebook(2), OutDtype.F32, 1.0, 1, 1)


def test_linear_argmax_ties():
    """Zero activations give a row of zeros of either sign: every column ties as a value, the key names column 0."""
    K, N, bits, cb = 256, 512, 4, 2
    w = synth.linear_weights(1234, "amt", K, N, bits)
    x = synth.activations(1234, "amt.x", 3, K)
    x[1] = 0
    plain, _ = run_linear(x, w, bits, cb, True)
    assert (plain[1] == 0).all()
    _, keys = _argmax_run(x, w, bits, cb, True)
    assert keys[1] == (0, 0.0)
    assert keys[0][0] == int(np.argmax(plain[0])) and keys[2][0] == int(np.argmax(plain[2]))


# ---------------------------------------------------------------- MUL1 on the integer tensor path (tensor-memory decode kernel)

@pytest.mark.parametrize("bits", [1, 2, 3, 4, 5, 6, 7, 8])
def test_integer_path_one_row_every_bitrate(oracle, bits):
    """One row of a MUL1 linear goes through k_exl3_gemv_i8 with the rotation inside the kernel; the output within the
    tolerance in both its forms, the rotated activations bit for bit."""
    K, N, cb = 1024, 768, 2
    w = synth.linear_weights(1234, f"i8b{bits}", K, N, bits)
    x = synth.activations(1234, "i8.x1", 1, K)
    for out_fp32 in (True, False):
        c, ah = run_linear(x, w, bits, cb, out_fp32)
        assert "k_exl3_gemv_i8" in kernels.last_launch() and "fused" in kernels.last_launch()
        assert kernels.device_status(torch.cuda.current_device()) == 0
        y64 = oracle.linear_f64(x, w["trellis"], w["suh"], w["svh"], K, N, bits, cb)
        assert_close(c, y64, f"bits {bits}")
        assert (ah == oracle.had_r_128(x, w["suh"], True).view(np.uint16)).all()


def test_integer_path_config0_and_run_to_run(oracle):
    """Configuration 0 (5120 x 6144, 4 bpw, one row) on the integer path: within tolerance, and bit-identical from run
    to run (the split-K partial sums are added in CTA order whichever CTA finishes a band group)."""
    K, N, bits, cb = 5120, 6144, 4, 2
    w = synth.linear_weights(1234, "c0", K, N, bits)
    x = synth.activations(1234, "c0.x", 1, K)
    c1, _ = run_linear(x, w, bits, cb, True)
    assert "k_exl3_gemv_i8" in kernels.last_launch()
    y64 = oracle.linear_f64(x, w["trellis"], w["suh"], w["svh"], K, N, bits, cb)
    assert_close(c1, y64, "c0")
    for _ in range(3):
        c2, _ = run_linear(x, w, bits, cb, True)
        assert (c1.view(np.uint32) == c2.view(np.uint32)).all()
    assert kernels.device_status(torch.cuda.current_device()) == 0


def test_integer_path_outlier_rows(oracle):
    """Activations with a few x20 outliers and one block of zeros: the block fixed point keeps its precision (a scale
    per 128 rotated inputs), a zero block quantises to zero."""
    K, N, bits, cb = 2048, 512, 4, 2
    w = synth.linear_weights(1234, "i8out", K, N, bits)
    x = synth.activations(1234, "i8out.x", 1, K, outlier_frac=0.01).copy()
    x[0, 256:384] = 0
    c, ah = run_linear(x, w, bits, cb, True)
    assert "k_exl3_gemv_i8" in kernels.last_launch()
    y64 = oracle.linear_f64(x, w["trellis"], w["suh"], w["svh"], K, N, bits, cb)
    assert_close(c, y64, "outliers")
    assert (ah == oracle.had_r_128(x, w["suh"], True).view(np.uint16)).all()


@pytest.mark.parametrize("ns,m,K,N,bits,out_fp32", [(2, 1, 512, 512, 4, True), (3, 3, 1024, 640, 4, False), (2, 4, 640, 384, 3, True),
                                                    (2, 7, 640, 384, 5, False), (2, 8, 512, 256, 4, True),
                                                    (2, 2, 256, 25600, 4, True), (2, 6, 256, 25600, 6, False)])
def test_stacked_linear_vs_oracle(oracle, ns, m, K, N, bits, out_fp32):
    """berth_exl3_linear_stack: ns equally shaped MUL1 matrices applied to the same rows in one launch; every matrix's
    output against the fp64 evaluation of that matrix alone, its rotated rows bit for bit.  Up to four rows rotate
    inside the kernel, above the limb tiles come from a rotation kernel; the two wide shapes give every CTA whole band
    groups (finished inside the decode kernel without split-K slabs)."""
    cb = 2
    ws = [synth.linear_weights(1234, f"st{i}.{K}x{N}b{bits}", K, N, bits) for i in range(ns)]
    x = synth.activations(1234, f"st.x{m}", m, K)
    tr = dev(np.stack([w["trellis"] for w in ws]))
    su, sv = dev(np.stack([w["suh"] for w in ws])), dev(np.stack([w["svh"] for w in ws]))
    c = torch.full((ns, m, N), float("nan"), dtype=torch.float32 if out_fp32 else torch.float16, device="cuda")
    ah = torch.zeros((ns, m, K), dtype=torch.float16, device="cuda")
    kernels.exl3_linear_stack(dev(x), tr, c, su, ah, sv, ns, m, K, N, bits, Codebook(cb), OutDtype.F32 if out_fp32 else OutDtype.F16)
    torch.cuda.synchronize()
    assert kernels.device_status(torch.cuda.current_device()) == 0
    assert f"stack of {ns}" in kernels.last_launch()
    got, ahh = c.float().cpu().numpy(), host_u16(ah)
    for i, w in enumerate(ws):
        y64 = oracle.linear_f64(x, w["trellis"], w["suh"], w["svh"], K, N, bits, cb)
        assert_close(got[i], y64, f"matrix {i}")
        assert (ahh[i] == oracle.had_r_128(x, w["suh"], True).view(np.uint16)).all()


def test_stacked_linear_fails_closed():
    K, N, bits = 256, 256, 4
    z = lambda *s, dt=torch.float16: torch.zeros(s, dtype=dt, device="cuda")
    tr = torch.zeros((2, K // 16, N // 16, 16 * bits), dtype=torch.int16, device="cuda")
    for m, cb in ((9, 2), (1, 0), (1, 1)):
        with pytest.raises(kernels.Error, match="no linked kernel"):
            kernels.exl3_linear_stack(z(m, K), tr, z(2, m, N), z(2, K), z(2, m, K), z(2, N), 2, m, K, N, bits, Codebook(cb), OutDtype.F16)
    with pytest.raises(kernels.Error, match="null"):
        kernels.exl3_linear_stack(None, tr, z(2, 1, N), z(2, K), z(2, 1, K), z(2, N), 2, 1, K, N, bits, Codebook(2), OutDtype.F16)


def test_decode_rate_diagnostic():
    """The bare decode-rate diagnostic runs on every path and reports a plausible figure."""
    for cb, path in ((0, 0), (1, 0), (2, 0), (2, 1), (2, 2)):
        w, mhz = kernels.decode_rate(4, Codebook(cb), path, 16, 256)
        assert 4.0 < w < 64.0 and 500.0 < mhz < 3000.0, (cb, path, w, mhz)
    with pytest.raises(kernels.Error):
        kernels.decode_rate(4, Codebook(0), 2, 16, 16)


# ---------------------------------------------------------------- configuration 2 at its own shapes

def _hadamard128():
    h = torch.ones((1, 1), dtype=torch.float64, device="cuda")
    for _ in range(7):
        h = torch.cat((torch.cat((h, h), 1), torch.cat((h, -h), 1)), 0)
    return h


@pytest.mark.parametrize("name,K,N,bits,out_fp32", [("gate", 5120, 17408, 4, False), ("down", 17408, 5120, 5, True),
                                                    ("q", 5120, 6144, 4, False), ("k", 5120, 1024, 3, False),
                                                    ("o", 6144, 5120, 4, True)])
def test_prefill_config2_shapes_against_decoded_bands(name, K, N, bits, out_fp32):
    """Benchmark configuration 2 at its own sizes: 4096 rows with 0.1 % of the activations multiplied by 20, the 27B
    projection shapes at 3 / 4 / 5 bpw, fp16 or fp32 outputs as the MLP and attention layers take them.  Too large for
    the CPU checker, so eight 128-column bands per matrix are decoded with berth_prefill_reconstruct (bit-exact
    against the checker) and evaluated in fp64 on the GPU from the rotated rows the launch wrote; the launch must
    agree on them within the tolerance (both forms) and produce no infinity or NaN anywhere."""
    M, cb = 4096, 2
    w = synth.linear_weights(1234, f"c2.{name}", K, N, bits, fan_in_gain=True)
    x = synth.activations(1234, f"c2.x.{name}", M, K, outlier_frac=0.001)
    xd, td, sd, vd = dev(x), dev(w["trellis"]), dev(w["suh"]), dev(w["svh"])
    c = torch.empty((M, N), dtype=torch.float32 if out_fp32 else torch.float16, device="cuda")
    ah = torch.empty((M, K), dtype=torch.float16, device="cuda")
    scratch = torch.empty(16, dtype=torch.float16, device="cuda")
    kernels.prefill_lin.exl3_linear(xd, td, c, sd, ah, vd, scratch, M, K, N, bits, Codebook(cb), OutDtype.F32 if out_fp32 else OutDtype.F16)
    torch.cuda.synchronize()
    assert "k_exl3_gemm_tc" in kernels.prefill_lin.last_launch()
    assert kernels.device_status(torch.cuda.current_device()) == 0
    assert bool(torch.isfinite(c).all())
    a_rot = ah.double()
    hmat = _hadamard128()
    bands = sorted({0, N // 128 - 1} | {int(b) for b in np.random.default_rng(7).integers(0, N // 128, 6)})
    svh = torch.from_numpy(w["svh"].astype(np.float64)).cuda()
    for b in bands:
        n0 = b * 128
        wt = torch.empty((K, 128), dtype=torch.float16, device="cuda")
        assert _lib_reconstruct(wt, td, K, 128, N, n0, bits, cb) == 0
        y = (a_rot @ wt.double()) @ hmat / np.sqrt(128.0) * svh[n0:n0 + 128]
        assert_close(c[:, n0:n0 + 128].double().cpu().numpy(), y.cpu().numpy(), f"{name} band {b}")


# ---------------------------------------------------------------- RMSNorm and the residual add: bit-exact

def _bf16_bits(a):
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


@pytest.mark.parametrize("rows,dim", [(1, 5120), (5, 2048), (3, 132), (64, 6144)])
@pytest.mark.parametrize("wbf", [True, False])
def test_rms_norm_bit_exact(oracle, rows, dim, wbf):
    """berth_ops_rms_norm, _f16 and _res_in against the checker, bit for bit (same summation order, every other step
    one correctly rounded fp32 operation); the residual rows of the _res_in form as well."""
    x = synth.activations(21, f"rms.x{rows}x{dim}", rows, dim).astype(np.float32) * 2.5
    w32 = synth.activations(21, f"rms.w{dim}", 1, dim).astype(np.float32)[0] * 0.1
    w = _bf16_bits(w32) if wbf else w32.astype(np.float16).view(np.uint16)
    eps, bias, scale = 1e-6, 1.0, 0.75
    wd = dev(w)
    y = torch.zeros((rows, dim), dtype=torch.float16, device="cuda")
    kernels.ops.rms_norm(torch.from_numpy(x).cuda(), wd, y, rows, dim, eps, bias, scale, wbf)
    torch.cuda.synchronize()
    assert "k_rms_norm" in kernels.ops.last_launch()
    assert (host_u16(y) == oracle.rms_norm(x, w, wbf, eps, bias, scale).view(np.uint16)).all()
    res = synth.activations(21, f"rms.r{rows}x{dim}", rows, dim).astype(np.float32)
    res_d = torch.from_numpy(res.copy()).cuda()
    kernels.ops.rms_norm_res_in(torch.from_numpy(x).cuda(), wd, y, res_d, rows, dim, eps, bias, scale, wbf)
    torch.cuda.synchronize()
    exp_res = res.copy()
    exp_y = oracle.rms_norm(x, w, wbf, eps, bias, scale, residual=exp_res)
    assert (res_d.cpu().numpy().view(np.uint32) == exp_res.view(np.uint32)).all()
    assert (host_u16(y) == exp_y.view(np.uint16)).all()
    if wbf:
        xh = x.astype(np.float16)
        kernels.ops.rms_norm_f16(dev(xh), wd, y, rows, dim, eps, bias, scale)
        torch.cuda.synchronize()
        assert (host_u16(y) == oracle.rms_norm(xh, w, True, eps, bias, scale).view(np.uint16)).all()


@pytest.mark.parametrize("m,K,N,bits,cb", [(1, 1024, 768, 4, 2), (1, 5120, 6144, 4, 2), (3, 512, 640, 4, 2), (20, 512, 256, 5, 2),
                                           (1, 1024, 512, 4, 0), (6, 512, 384, 3, 1)])
def test_linear_add_equals_linear_then_add(oracle, m, K, N, bits, cb):
    """berth_exl3_linear_add (the residual added in the decode kernel's last step) gives bit for bit what
    berth_exl3_linear with fp32 output followed by berth_ops_add_f32 gives, also in place on the residual; and the
    sum is the checker's fp64 linear plus the residual within the tolerance."""
    w = synth.linear_weights(1234, f"ladd{K}x{N}b{bits}", K, N, bits)
    x = synth.activations(1234, f"ladd.x{m}", m, K)
    r = synth.activations(1234, f"ladd.r{m}", m, N).astype(np.float32) * 4.0
    xd, td, sd, vd = dev(x), dev(w["trellis"]), dev(w["suh"]), dev(w["svh"])
    rd = torch.from_numpy(r).cuda()
    ah = torch.zeros((m, K), dtype=torch.float16, device="cuda")
    y = torch.empty((m, N), dtype=torch.float32, device="cuda")
    kernels.exl3_linear(xd, td, y, sd, ah, vd, m, K, N, bits, Codebook(cb), OutDtype.F32)
    unfused = torch.empty_like(y)
    kernels.ops.add_f32(rd, y, unfused, m * N)
    fused = torch.full((m, N), float("nan"), dtype=torch.float32, device="cuda")
    kernels.exl3_linear_add(xd, td, fused, sd, ah, vd, rd, m, K, N, bits, Codebook(cb))
    assert "residual" in kernels.last_launch()
    inplace = rd.clone()
    kernels.exl3_linear_add(xd, td, inplace, sd, ah, vd, inplace, m, K, N, bits, Codebook(cb))
    torch.cuda.synchronize()
    assert kernels.device_status(torch.cuda.current_device()) == 0
    assert torch.equal(fused.view(torch.int32), unfused.view(torch.int32))
    assert torch.equal(inplace.view(torch.int32), unfused.view(torch.int32))
    y64 = oracle.linear_f64(x, w["trellis"], w["suh"], w["svh"], K, N, bits, cb)
    mx, mean = rel_errors(fused.cpu().numpy() - r, y64)
    assert mx <= MAX_REL and mean <= MEAN_REL


@pytest.mark.parametrize("m,K,N,bits,cb,limit,res", [
    (1, 1024, 768, 4, 2, 0.0, False), (1, 17408, 5120, 4, 2, 0.0, True), (1, 2048, 1024, 6, 2, 3.0, False),
    (2, 1024, 512, 4, 2, 0.0, True), (2, 512, 384, 3, 0, 0.0, False), (3, 512, 640, 4, 2, 1.5, True),
    (8, 1024, 256, 5, 1, 0.0, False), (16, 512, 256, 2, 2, 0.0, False), (20, 512, 256, 5, 2, 0.0, True)])
def test_linear_silu_equals_silu_mul_then_linear(oracle, m, K, N, bits, cb, limit, res):
    """berth_exl3_linear_silu (silu(gate) * up formed inside the linear's rotation, optionally the residual added in the
    last step) gives bit for bit the output AND the rotated activations of berth_ops_silu_mul followed by the same
    decode launch on the activation buffer; and the output is the checker's fp64 linear of the checker's silu_mul within
    the tolerance.  Covers the in-kernel rotation of both decode kernels and the separate rotation kernel, with a clamp
    and without, and gate values large enough for the sigmoid to saturate."""
    w = synth.linear_weights(1234, f"lsilu{K}x{N}b{bits}", K, N, bits)
    g = (synth.activations(1234, f"lsilu.g{m}", m, K).astype(np.float32) * 3.0).astype(np.float16)
    g[0, :4] = np.array([30.0, -30.0, 0.0, -0.0], dtype=np.float16)
    u = synth.activations(1234, f"lsilu.u{m}", m, K)
    r = synth.activations(1234, f"lsilu.r{m}", m, N).astype(np.float32) * 4.0
    gd, ud, td, sd, vd = dev(g), dev(u), dev(w["trellis"]), dev(w["suh"]), dev(w["svh"])
    rd = torch.from_numpy(r).cuda()
    out = OutDtype.F32 if res else OutDtype.F16
    odt = torch.float32 if res else torch.float16
    act = torch.empty((m, K), dtype=torch.float16, device="cuda")
    kernels.ops.silu_mul(gd, ud, act, m * K, limit)
    ah0 = torch.zeros((m, K), dtype=torch.float16, device="cuda")
    unfused = torch.empty((m, N), dtype=odt, device="cuda")
    if res:
        kernels.exl3_linear_add(act, td, unfused, sd, ah0, vd, rd, m, K, N, bits, Codebook(cb))
    else:
        kernels.exl3_linear(act, td, unfused, sd, ah0, vd, m, K, N, bits, Codebook(cb), out)
    ah1 = torch.zeros((m, K), dtype=torch.float16, device="cuda")
    fused = torch.full((m, N), float("nan"), dtype=odt, device="cuda")
    kernels.exl3_linear_silu(gd, ud, td, fused, sd, ah1, vd, m, K, N, bits, Codebook(cb), out, limit, rd if res else None)
    assert "silu(gate) * up in the rotation" in kernels.last_launch()
    torch.cuda.synchronize()
    assert kernels.device_status(torch.cuda.current_device()) == 0
    view = torch.int32 if res else torch.int16
    assert torch.equal(ah1.view(torch.int16), ah0.view(torch.int16))
    assert torch.equal(fused.view(view), unfused.view(view))
    act_o = oracle.silu_mul(g, u, limit)
    assert np.array_equal(act.cpu().numpy().view(np.uint16), act_o.view(np.uint16))
    y64 = oracle.linear_f64(act_o, w["trellis"], w["suh"], w["svh"], K, N, bits, cb)
    got = fused.float().cpu().numpy() - (r if res else 0.0)
    mx, mean = rel_errors(got, y64)
    assert mx <= MAX_REL and mean <= MEAN_REL


def test_linear_silu_rejects_what_it_cannot_run():
    z = torch.zeros(4096, dtype=torch.float16, device="cuda")
    t = torch.zeros((8, 8, 64), dtype=torch.int16, device="cuda")
    with pytest.raises(kernels.Error, match="size_m must be <= 32"):
        kernels.exl3_linear_silu(z, z, t, z, z, z, z, 33, 128, 128, 4, Codebook(2), OutDtype.F16)
    with pytest.raises(kernels.Error, match="residual is added to fp32 outputs only"):
        kernels.exl3_linear_silu(z, z, t, z, z, z, z, 1, 128, 128, 4, Codebook(2), OutDtype.F16, 0.0, z)


def test_small_batch_tensor_path_random_shapes_vs_decode_kernel():
    """Forty seeded random shapes (17..32 rows, every bitrate and codebook, K and N any multiples of 128 large enough for the
    split-K kernel): its outputs against the decode GEMV's (berth_exl3_linear_add with a zero residual always runs that
    kernel) within the accumulation tolerance of two fp32 summation orders, and a clean status."""
    rng = np.random.RandomState(20240611)
    sms = kernels.device_sms(torch.cuda.current_device()) if hasattr(kernels, "device_sms") else 148
    done = 0
    while done < 40:
        K = 128 * int(rng.randint(1, 33))
        N = 128 * int(rng.randint(1, 65))
        if (N // 128) * (K // 64) < 8 * sms:
            continue
        m, bits, cb = int(rng.randint(17, 33)), int(rng.randint(1, 9)), int(rng.randint(0, 3))
        w = synth.linear_weights(1234, f"skr{done}", K, N, bits)
        x = synth.activations(1234, f"skr.x{done}", m, K)
        xd, td, sd, vd = dev(x), dev(w["trellis"]), dev(w["suh"]), dev(w["svh"])
        ah = torch.zeros((m, K), dtype=torch.float16, device="cuda")
        c = torch.full((m, N), float("nan"), dtype=torch.float32, device="cuda")
        kernels.exl3_linear(xd, td, c, sd, ah, vd, m, K, N, bits, Codebook(cb), OutDtype.F32)
        assert "k_exl3_gemm_tc_splitk" in kernels.last_launch(), (m, K, N)
        ref = torch.empty_like(c)
        kernels.exl3_linear_add(xd, td, ref, sd, ah, vd, torch.zeros_like(c), m, K, N, bits, Codebook(cb))
        torch.cuda.synchronize()
        a, b = c.double().cpu().numpy(), ref.double().cpu().numpy()
        rms = np.sqrt((b ** 2).mean())
        assert np.isfinite(a).all() and np.abs(a - b).max() <= 4e-3 * rms, (m, K, N, bits, cb, np.abs(a - b).max() / rms)
        done += 1
    assert kernels.device_status(torch.cuda.current_device()) == 0


# ---------------------------------------------------------------- several MUL1 matrices of different widths in one launch

@pytest.mark.parametrize("m", [1, 2, 4, 7])
@pytest.mark.parametrize("K,Ns,bits,out_fp32", [(512, [384, 128, 128], 4, False), (5120, [6144, 1024, 1024], 4, False),
                                                (1024, [256, 2048], 5, True), (640, [128], 3, True),
                                                (2048, [1024, 128, 640, 384], 6, False)])
def test_linear_multi_vs_oracle(oracle, m, K, Ns, bits, out_fp32):
    """berth_exl3_linear_multi (q, k and v of an attention block as one integer-path launch): every matrix against the
    fp64 oracle, its rotated rows bit for bit, identical bits on a second run, clean status."""
    ws = [synth.linear_weights(1234, f"multi{K}.{i}.{n}.{bits}", K, n, bits, fan_in_gain=True) for i, n in enumerate(Ns)]
    x = synth.activations(1234, f"multi.x{m}.{K}", m, K)
    xd = dev(x)
    dt = torch.float32 if out_fp32 else torch.float16
    td = [dev(w["trellis"]) for w in ws]
    sd = [dev(w["suh"]) for w in ws]
    vd = [dev(w["svh"]) for w in ws]
    runs = []
    for _ in range(2):
        cs = [torch.full((m, n), float("nan"), dtype=dt, device="cuda") for n in Ns]
        ahs = [torch.zeros((m, K), dtype=torch.float16, device="cuda") for _ in Ns]
        kernels.exl3_linear_multi(xd, kernels.pointer_list(td), kernels.pointer_list(cs), kernels.pointer_list(sd),
                                  kernels.pointer_list(ahs), kernels.pointer_list(vd), kernels.int_list(Ns), len(Ns), m, K, bits,
                                  Codebook(2), OutDtype.F32 if out_fp32 else OutDtype.F16)
        torch.cuda.synchronize()
        runs.append(([c.cpu().numpy() for c in cs], [host_u16(ah) for ah in ahs]))
    assert "k_exl3_gemv_i8" in kernels.last_launch() and f"{len(Ns)} matrices" in kernels.last_launch()
    assert kernels.device_status(torch.cuda.current_device()) == 0
    view = np.uint32 if out_fp32 else np.uint16
    for i, (w, n) in enumerate(zip(ws, Ns)):
        c, ah = runs[0][0][i], runs[0][1][i]
        y64 = oracle.linear_f64(x, w["trellis"], w["suh"], w["svh"], K, n, bits, 2)
        assert_close(c, y64, f"matrix {i}")
        assert (ah.reshape(m, K) == oracle.had_r_128(x, w["suh"], True).view(np.uint16)).all()
        assert (runs[1][0][i].view(view) == c.view(view)).all()


def test_linear_multi_fails_closed():
    K, Ns, bits = 256, [128, 128], 4
    ws = [synth.linear_weights(1234, f"multi.fc{i}", K, n, bits) for i, n in enumerate(Ns)]
    x = dev(synth.activations(1234, "multi.fc.x", 1, K))
    td, sd, vd = [dev(w["trellis"]) for w in ws], [dev(w["suh"]) for w in ws], [dev(w["svh"]) for w in ws]
    cs = [torch.zeros((1, n), dtype=torch.float16, device="cuda") for n in Ns]
    ahs = [torch.zeros((1, K), dtype=torch.float16, device="cuda") for _ in Ns]
    lists = lambda k: (kernels.pointer_list(td * k), kernels.pointer_list(cs * k), kernels.pointer_list(sd * k),
                       kernels.pointer_list(ahs * k), kernels.pointer_list(vd * k), kernels.int_list(Ns * k))
    with pytest.raises(kernels.Error, match="no linked kernel"):
        kernels.exl3_linear_multi(x, *lists(1), 2, 1, K, bits, Codebook(0), OutDtype.F16)
    with pytest.raises(kernels.Error, match="no linked kernel"):
        kernels.exl3_linear_multi(x, *lists(1), 2, 9, K, bits, Codebook(2), OutDtype.F16)
    with pytest.raises(kernels.Error, match="n_matrices"):
        kernels.exl3_linear_multi(x, *lists(3), 6, 1, K, bits, Codebook(2), OutDtype.F16)
    with pytest.raises(kernels.Error, match="multiple of 128"):
        kernels.exl3_linear_multi(x, *lists(1)[:5], kernels.int_list([128, 64]), 2, 1, K, bits, Codebook(2), OutDtype.F16)


# ---------------------------------------------------------------- the CUDA kernels against the committed golden vectors

def _golden(golden_dir):
    import json
    d = os.path.join(golden_dir, "exl3_spec_v0")
    with open(os.path.join(d, "meta.json")) as f:
        return d, json.load(f)["files"]


def test_cuda_decode_against_committed_golden_tiles(golden_dir):
    """The decoded weights of the tiny golden matrices (3/4/5 bpw, three codebooks) and of configuration 0 as the CUDA
    reconstruct kernel produces them: the committed rows and sampled tiles byte for byte, the whole matrices by digest."""
    import hashlib
    d, files = _golden(golden_dir)
    for bits in (3, 4, 5):
        for cb in (0, 1, 2):
            m = files[f"tiny.b{bits}.cb{cb}.head.bin"]
            t = dev(synth.trellis(1234, m["tensor"], 128, 256, bits))
            out = torch.empty((128, 256), dtype=torch.float16, device="cuda")
            kernels.prefill_lin.reconstruct(out, t, 128, 256, 256, 0, bits, Codebook(cb))
            got = host_u16(out).reshape(128, 256)
            head = np.fromfile(os.path.join(d, f"tiny.b{bits}.cb{cb}.head.bin"), np.uint16).reshape(16, 256)
            assert (got[:16] == head).all()
            assert hashlib.sha256(got.tobytes()).hexdigest() == m["sha256_whole_decoded_matrix"]
    m = files["c0.tiles.bin"]
    K, N = m["size_k"], m["size_n"]
    w = synth.linear_weights(1234, m["tensor"], K, N, m["bits"])
    out = torch.empty((K, N), dtype=torch.float16, device="cuda")
    kernels.prefill_lin.reconstruct(out, dev(w["trellis"]), K, N, N, 0, m["bits"], Codebook(m["codebook"]))
    got = host_u16(out).reshape(K, N)
    tiles = np.fromfile(os.path.join(d, "c0.tiles.bin"), np.uint16).reshape(64, 16, 16)
    for i, (kt, nt) in enumerate(m["positions"]):
        assert (got[16 * kt:16 * kt + 16, 16 * nt:16 * nt + 16] == tiles[i]).all(), (kt, nt)
    assert hashlib.sha256(got.tobytes()).hexdigest() == m["sha256_whole_decoded_matrix"]


@pytest.mark.parametrize("path", ["decode", "static_scratch", "prefill_rows"])
def test_cuda_linear_against_committed_golden_c0(golden_dir, path):
    """Configuration 0 (5120 x 6144, 4 bpw, MUL1, one row) through the decode linear, the allocation-free entry point and
    (as 33 copies of the row) the prefill linear: within the tolerance of the committed fp64 row, within the accumulation
    tolerance of the committed fp32 row of the checker, rotated activations by digest."""
    import hashlib
    d, files = _golden(golden_dir)
    m = files["c0.y.bin"]
    K, N, bits, cb = m["size_k"], m["size_n"], m["bits"], m["codebook"]
    w = synth.linear_weights(1234, m["tensor"], K, N, bits)
    x = synth.activations(1234, m["activations"], 1, K)
    y32 = np.fromfile(os.path.join(d, "c0.y.bin"), np.float32).reshape(1, N)
    y64 = np.fromfile(os.path.join(d, "c0.y64.bin"), np.float64).reshape(1, N)
    rows = 33 if path == "prefill_rows" else 1
    xd, td, sd, vd = dev(np.repeat(x, rows, axis=0)), dev(w["trellis"]), dev(w["suh"]), dev(w["svh"])
    c = torch.full((rows, N), float("nan"), dtype=torch.float32, device="cuda")
    ah = torch.zeros((rows, K), dtype=torch.float16, device="cuda")
    if path == "static_scratch":
        kernels.exl3_linear_static_scratch(xd, td, c, sd, ah, vd, rows, K, N, bits, Codebook(cb), OutDtype.F32)
    else:
        kernels.exl3_linear(xd, td, c, sd, ah, vd, rows, K, N, bits, Codebook(cb), OutDtype.F32)
    torch.cuda.synchronize()
    got = c.cpu().numpy()
    for r in (0, rows - 1):
        assert_close(got[r:r + 1], y64, f"{path} row {r}")
        assert np.abs(got[r:r + 1].astype(np.float64) - y32).max() <= 4e-3 * np.sqrt((y64 ** 2).mean())
    assert hashlib.sha256(host_u16(ah).reshape(rows, K)[0].tobytes()).hexdigest() == m["sha256_rotated_activations"]
    assert kernels.device_status(torch.cuda.current_device()) == 0


@pytest.mark.parametrize("T", [1, 64, 1024])
def test_cuda_router_against_committed_golden_topk(golden_dir, T):
    """Configuration 3's router at 1, 64 and 1024 tokens: the top-8 table byte for byte, the logits by digest."""
    import hashlib
    from berth_b200 import moe
    d, files = _golden(golden_dir)
    m = files[f"c3.topk.T{T}.bin"]
    H, E, k = m["hidden"], m["n_experts"], m["top_k"]
    x = dev(synth.activations(1234, m["activations"], T, H))
    wr = dev(synth.router_weight(1234, m["router"], H, E))
    logits = torch.empty((T, E), dtype=torch.float32, device="cuda")
    idx = torch.empty((T, k), dtype=torch.int32, device="cuda")
    tw = torch.empty((T, k), dtype=torch.float32, device="cuda")
    moe.router_topk(x, wr, None, idx, tw, logits, T, H, E, k)
    torch.cuda.synchronize()
    exp = np.fromfile(os.path.join(d, f"c3.topk.T{T}.bin"), np.int32).reshape(T, k)
    assert (idx.cpu().numpy() == exp).all()
    assert hashlib.sha256(logits.cpu().numpy().tobytes()).hexdigest() == m["sha256_logits_f32"]
    w = tw.cpu().numpy()
    assert np.abs(w.sum(axis=1) - 1.0).max() <= 1e-6 and (np.diff(w, axis=1) <= 1e-7).all()   # renormalised, descending


def test_weights_streamed_guard_changes_no_result():
    """berth_exl3_weights_streamed(1): the decode kernels fetch no weights before their predecessor on the stream has
    ended.  Every decode kernel (integer path, fp16 path with and without in-kernel rotation, split-K tensor-core path,
    stacked and multi-matrix launches) gives the same bits with the guard on, also when the weights are copied into place
    on the same stream directly before each launch."""
    cases = [(1, 1024, 768, 4, 2), (2, 1024, 768, 4, 0), (7, 512, 640, 5, 2), (20, 2048, 5120, 4, 2), (32, 512, 256, 3, 1)]
    assert kernels.weights_streamed(False) is False
    try:
        for m, K, N, bits, cb in cases:
            w = synth.linear_weights(1234, f"guard{K}x{N}", K, N, bits)
            x = synth.activations(1234, f"guard.x{m}", m, K)
            ref, _ = run_linear(x, w, bits, cb, True)
            name = kernels.last_launch()
            kernels.weights_streamed(True)
            got, _ = run_linear(x, w, bits, cb, True)
            assert kernels.last_launch() == name
            assert (got.view(np.uint32) == ref.view(np.uint32)).all(), (m, K, N)
            # weights copied into place on the stream right before the launch, several times over
            xd, sd, vd = dev(x), dev(w["suh"]), dev(w["svh"])
            src, other = dev(w["trellis"]), dev(synth.trellis(1234, "guard.other", K, N, bits))
            td = torch.empty_like(src)
            c = torch.empty((m, N), dtype=torch.float32, device="cuda")
            ah = torch.zeros((m, K), dtype=torch.float16, device="cuda")
            for _ in range(8):
                td.copy_(other)
                kernels.exl3_linear(xd, td, c, sd, ah, vd, m, K, N, bits, Codebook(cb), OutDtype.F32)
                td.copy_(src)
                kernels.exl3_linear(xd, td, c, sd, ah, vd, m, K, N, bits, Codebook(cb), OutDtype.F32)
            torch.cuda.synchronize()
            assert (c.cpu().numpy().view(np.uint32) == ref.view(np.uint32)).all(), (m, K, N)
            assert kernels.weights_streamed(False) is True
    finally:
        kernels.weights_streamed(False)
    assert kernels.device_status(torch.cuda.current_device()) == 0
