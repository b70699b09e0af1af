"""The C boundary without a GPU: the library loads, exports every symbol the header declares,
and rejects bad arguments before any CUDA call with the wording berth's own boundary tests
look for (crates/berth-kernels/src/lib.rs:236-319, src/prefill_lin.rs:338-383, src/ops.rs:775-857)."""
import ctypes
import os
import re

import pytest

from berth_b200 import Codebook, Error, OutDtype, _lib, kernels

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
P = 64  # non-null, never dereferenced: the checks return first


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(_lib.SO_PATH):
        _lib.build()
    return _lib.lib()


def _declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for f in os.listdir(inc):
        text = open(os.path.join(inc, f)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(berth_\w+)\s*\(", text))
    return names


def test_every_declared_symbol_is_exported_and_bound(lib):
    declared = _declared_symbols()
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
    assert declared == set(_lib.SIGNATURES), "Python binding table and header disagree"


def test_exl3_linear_null_and_bad_sizes_do_not_call_cuda(lib):
    with pytest.raises(Error, match="null"):
        kernels.exl3_linear(None, None, None, None, None, None, 1, 128, 256, 4, Codebook.Mul1, OutDtype.F16)
    assert kernels.last_launch() == ""
    with pytest.raises(Error, match="multiple of 16"):
        kernels.exl3_linear(P, P, P, P, P, P, 1, 15, 256, 4, Codebook.Mul1, OutDtype.F32)
    with pytest.raises(Error, match="multiple of 128"):
        kernels.exl3_linear(P, P, P, P, P, P, 1, 16, 100, 4, Codebook.Mul1, OutDtype.F16)
    with pytest.raises(Error, match="positive"):
        kernels.exl3_linear(P, P, P, P, P, P, 0, 16, 128, 4, Codebook.Mul1, OutDtype.F16)
    with pytest.raises(Error, match="K must be in 1..=8"):
        kernels.exl3_linear(P, P, P, P, P, P, 1, 128, 128, 9, Codebook.Mul1, OutDtype.F16)
    assert lib.berth_exl3_linear(P, P, P, P, P, P, 1, 128, 128, 4, 3, 0, None) == -1
    assert "codebook" in kernels.last_error()
    assert kernels.last_error() != ""


def test_prefill_null_and_m1_do_not_launch(lib):
    pl = kernels.prefill_lin
    with pytest.raises(Error, match="null"):
        pl.exl3_linear(None, None, None, None, None, None, None, 2, 128, 256, 4, Codebook.Mul1, OutDtype.F16)
    assert pl.last_launch() == ""
    with pytest.raises(Error, match="size_m"):
        pl.exl3_linear(P, P, P, P, P, P, None, 1, 128, 256, 4, Codebook.Mul1, OutDtype.F16)
    with pytest.raises(Error, match="w_scratch"):
        pl.exl3_linear(P, P, P, P, P, P, None, 145, 128, 256, 4, Codebook.Mul1, OutDtype.F16)
    with pytest.raises(Error, match="multiple of 16"):
        pl.exl3_linear(P, P, P, P, P, P, None, 2, 24, 256, 4, Codebook.Mul1, OutDtype.F16)
    with pytest.raises(Error, match="multiple of 128"):
        pl.exl3_linear(P, P, P, P, P, P, None, 2, 128, 200, 4, Codebook.Mul1, OutDtype.F16)


def test_ops_argument_checks(lib):
    with pytest.raises(Error, match="null"):
        kernels.ops.silu_mul(None, P, P, 16)
    with pytest.raises(Error, match="positive and even"):
        kernels.ops.silu_mul(P, P, P, 17)
    with pytest.raises(Error, match="positive and even"):
        kernels.ops.silu_mul(P, P, P, 0)
    with pytest.raises(Error, match="null"):
        kernels.ops.add_f32(P, None, P, 4)
    with pytest.raises(Error, match="positive"):
        kernels.ops.add_f32(P, P, P, 0)
    with pytest.raises(Error, match="multiple of 128"):
        kernels.prefill_lin.reconstruct(P, P, 16, 100, 128, 0, 4, 2)
    with pytest.raises(Error, match="exceeds"):
        kernels.prefill_lin.reconstruct(P, P, 16, 256, 256, 128, 4, 2)
    with pytest.raises(Error, match="multiple of 128"):
        kernels.prefill_lin.had_r_128(P, P, None, True, 1, 100, False)


def test_lm_head_tune_key_matches_berth(lib):
    # crates/berth-kernels/src/lib.rs:224-233
    assert kernels.gemm_tune_key(1, 5120, 248320, 6, 0, 0, 2, 82, int(Codebook.Mul1)) == 0x51F40C1BD7CAE3A7


def test_prefill_hgemm_rejected_launches(lib):
    # crates/berth-kernels/csrc/prefill_lin/linear.cu:402-405
    import ctypes as C
    p = C.c_void_p(8)
    assert lib.berth_prefill_hgemm(None, p, p, 4, 64, 64, 64, 0, None) == -1 and "null" in kernels.prefill_lin.last_error()
    assert lib.berth_prefill_hgemm(p, p, p, 4, 64, 64, 32, 0, None) == -1 and "bad shape" in kernels.prefill_lin.last_error()
    assert lib.berth_prefill_hgemm(p, p, p, 0, 64, 64, 64, 0, None) == -1 and "bad shape" in kernels.prefill_lin.last_error()


def test_mgemm_tune_keys_match_berth(lib):
    # crates/berth-kernels/src/ops.rs:738-773: the two multi-linear bundles of the 27B decode (device 0, CC class 2, 82 SMs)
    f = kernels.ops.mgemm_tune_key
    assert f(1, 5120, 2048, 4, OutDtype.F32, 0, 2, 82, Codebook.Mul1, 1, 8, True) == 0xD2297A8A33A33F5B
    assert f(1, 5120, 1024, 4, OutDtype.F16, 0, 2, 82, Codebook.Mul1, 1, 14, True) == 0x9C25A0752178FB4A


def test_mgemm_rejected_launches_do_not_call_cuda(lib):
    # crates/berth-kernels/src/ops.rs:775-857: null pointers, a K with no kernel, size_k not a multiple of 16
    import ctypes as C
    l = lib
    null = None
    p = C.c_void_p(8)     # never dereferenced: every case below fails before any CUDA call
    rc = l.berth_ops_mgemm(null, null, null, null, null, null, 1, 5120, 2048, 4, 2, 1, 1, 8, null, null, null, null, 0, null)
    assert rc == -1 and "null" in kernels.ops.last_error()
    assert kernels.ops.last_launch() == ""
    rc = l.berth_ops_mgemm(p, p, p, p, p, p, 1, 5120, 2048, 9, 2, 1, 1, 8, null, null, null, null, 0, null)
    assert rc == -1 and "no linked kernel" in kernels.ops.last_error()
    rc = l.berth_ops_mgemm(p, p, p, p, p, p, 1, 15, 2048, 4, 2, 0, 1, 1, null, null, null, null, 0, null)
    assert rc == -1 and "multiple of 16" in kernels.ops.last_error()
    rc = l.berth_ops_mgemm(p, p, p, p, p, p, 1, 5120, 2048, 4, 2, 0, 1, 8, p, null, p, p, 2, null)
    assert rc == -1 and "sliced mode requires" in kernels.ops.last_error()
    rc = l.berth_ops_mgemm(p, p, p, p, p, p, 1, 5120, 2048, 4, 2, 0, 2, 8, p, p, p, p, 2, null)
    assert rc == -1 and "single-input" in kernels.ops.last_error()
    rc = l.berth_ops_mgemm(p, p, p, p, p, p, 1, 5120, 2048, 4, 2, 0, 3, 8, null, null, null, null, 0, null)
    assert rc == -1 and "uniform mode" in kernels.ops.last_error()     # inputs: one for all matrices, or one each
    rc = l.berth_ops_mgemm(p, p, p, p, p, p, 1, 5120, 2048, 4, 2, 0, 1, 8, null, null, null, null, 2, null)
    assert rc == -1 and "num_had_src requires" in kernels.ops.last_error()


def test_exl3_gemv_cfg_matches_27b_shapes(lib):
    # crates/berth-kernels/src/prefill_lin.rs:386-442
    f = kernels.prefill_lin.exl3_gemv_cfg
    AMP, ADA, MODE, K, CB, NARROW = 2, 3, 1, 4, 2, 164
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


def test_library_matches_oracle_on_host_logic(lib, oracle):
    import itertools
    for cc, m, k, n, bits, cb, mode in itertools.product((2, 3, 5), (1, 4, 9), (2048, 5120), (5120, 8192, 17408),
                                                         (2, 3, 4, 5), (0, 2), (0, 1, 2, 3, 4)):
        assert kernels.prefill_lin.exl3_gemv_cfg(cc, m, k, n, bits, cb, mode, 164) == oracle.gemv_cfg(
            cc, m, k, n, bits, cb, mode, 164)
    for m in (1, 2, 3, 16, 17, 31, 32, 63, 64, 127, 128, 4096):
        assert kernels.gemm_tune_key(m, 5120, 6144, 4, 1, 0, 5, 148, 2) == oracle.gemm_tune_key(
            m, 5120, 6144, 4, 1, 0, 5, 148, 2)


def test_product_does_not_touch_the_oracle():
    """Nothing under berth_b200/ may import, link or execute the CPU checker."""
    pkg = os.path.join(ROOT, "berth_b200")
    for dirpath, _, files in os.walk(pkg):
        if os.path.basename(dirpath) == "build":
            continue
        for f in files:
            if not f.endswith((".py", ".cu", ".cuh", ".cpp", ".h", "Makefile")):
                continue
            text = open(os.path.join(dirpath, f), errors="replace").read()
            for needle in ("exl3o_", "import oracle", "from oracle", "libexl3_oracle"):
                assert needle not in text, f"{f} references the oracle ({needle})"


def test_argmax_key_decode_known_answers(lib):
    """key = (order-preserving bits of the fp32 value) << 32 | (0xffffffff - column)."""
    import struct

    def key(value, col):
        bits = struct.unpack("<I", struct.pack("<f", value))[0]
        order = (~bits & 0xFFFFFFFF) if bits & 0x80000000 else bits | 0x80000000
        return (order << 32) | (0xFFFFFFFF - col)

    for value, col in ((1.5, 0), (-2.25, 7), (0.0, 248319), (-0.0, 1), (3.0e38, 12345), (-1.0e-40, 4)):
        tok, val = kernels.argmax_key_decode(key(value, col))
        assert tok == col and struct.pack("<f", val) == struct.pack("<f", value)
    # larger value wins; at equal value the lower column wins
    assert key(2.0, 9) > key(1.0, 3) and key(-1.0, 9) > key(-2.0, 3) and key(1.0, 3) > key(1.0, 9) and key(0.5, 0) > key(-0.5, 0)
    with pytest.raises(Error, match="null"):
        kernels.exl3_linear_argmax(None, None, None, None, None, None, None, 1, 128, 256, 4, Codebook.Mul1, OutDtype.F16)
    with pytest.raises(Error, match="size_m"):
        kernels.exl3_linear_argmax(P, P, P, P, P, P, P, 33, 128, 256, 4, Codebook.Mul1, OutDtype.F16)


def test_rms_norm_argument_checks(lib):
    """Checks of crates/berth-kernels/csrc/ops/norm.cu:107-127, before any CUDA call."""
    o = kernels.ops
    with pytest.raises(Error, match="null device pointer"):
        o.rms_norm(None, P, P, 1, 128, 1e-6, 1.0, 1.0, True)
    with pytest.raises(Error, match="RES_IN requires a residual pointer"):
        o.rms_norm_res_in(P, P, P, None, 1, 128, 1e-6, 1.0, 1.0, True)
    with pytest.raises(Error, match="rows and dim must be positive"):
        o.rms_norm(P, P, P, 0, 128, 1e-6, 1.0, 1.0, True)
    with pytest.raises(Error, match="multiple of 4"):
        o.rms_norm_f16(P, P, P, 1, 130, 1e-6, 1.0, 1.0)
    assert lib.berth_ops_rms_norm(P, P, P, 1, 128, 1e-6, 1.0, 1.0, 2, None) == -1
    assert "weight_bf16 must be 0 or 1" in o.last_error()


def test_linear_add_and_stack_argument_checks(lib):
    with pytest.raises(Error, match="null"):
        kernels.exl3_linear_add(P, P, P, P, P, P, None, 1, 128, 128, 4, Codebook.Mul1)
    with pytest.raises(Error, match="size_m must be <= 32"):
        kernels.exl3_linear_add(P, P, P, P, P, P, P, 33, 128, 128, 4, Codebook.Mul1)
    with pytest.raises(Error, match="multiple of 128"):
        kernels.exl3_linear_add(P, P, P, P, P, P, P, 1, 128, 100, 4, Codebook.Mul1)
    with pytest.raises(Error, match="n_matrices"):
        kernels.exl3_linear_stack(P, P, P, P, P, P, 0, 1, 128, 128, 4, Codebook.Mul1, OutDtype.F16)
    with pytest.raises(Error, match="no linked kernel"):
        kernels.exl3_linear_stack(P, P, P, P, P, P, 2, 9, 128, 128, 4, Codebook.Mul1, OutDtype.F16)


def test_linear_silu_argument_checks(lib):
    """berth_exl3_linear_silu refuses on the host, before any CUDA call: a missing gate or up, more rows than the decode
    kernels take, a residual with fp16 output, and the shapes berth_exl3_linear refuses."""
    with pytest.raises(Error, match="null"):
        kernels.exl3_linear_silu(P, None, P, P, P, P, P, 1, 128, 128, 4, Codebook.Mul1, OutDtype.F32)
    with pytest.raises(Error, match="size_m must be <= 32"):
        kernels.exl3_linear_silu(P, P, P, P, P, P, P, 33, 128, 128, 4, Codebook.Mul1, OutDtype.F32)
    with pytest.raises(Error, match="fp32 outputs only"):
        kernels.exl3_linear_silu(P, P, P, P, P, P, P, 1, 128, 128, 4, Codebook.Mul1, OutDtype.F16, 0.0, P)
    with pytest.raises(Error, match="multiple of 128"):
        kernels.exl3_linear_silu(P, P, P, P, P, P, P, 1, 128, 100, 4, Codebook.Mul1, OutDtype.F32)
    with pytest.raises(Error, match="K must be in 1..=8"):
        kernels.exl3_linear_silu(P, P, P, P, P, P, P, 1, 128, 128, 9, Codebook.Mul1, OutDtype.F32)


def test_weights_streamed_switch_returns_the_previous_setting(lib):
    assert lib.berth_exl3_weights_streamed(1) == 0
    assert lib.berth_exl3_weights_streamed(1) == 1
    assert lib.berth_exl3_weights_streamed(0) == 1
    assert lib.berth_exl3_weights_streamed(0) == 0
