"""The host-side callers of the linear (berth_b200.engine), driven the way berth's own engine tests drive theirs
(crates/berth-engine/tests/exl3_linear.rs:10-36, tests/mlp_layer.rs:24-71): an ``Exl3Linear`` decode and prefill
launch, and the whole ``MlpLayer`` chain gate / up / silu / down, each against the CPU checker's chain."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from berth_b200 import Codebook, OutDtype, kernels, synth   # noqa: E402
from berth_b200.engine import Error, Exl3Linear, Gpu, MlpLayer, RowScratch, StackedLinear   # noqa: E402
from tests.gpu_util import assert_close, dev, host_u16   # noqa: E402


def _oracle_linear64(orc, x, w, K, N, bits, cb):
    return orc.linear_f64(x, w["trellis"], w["suh"], w["svh"], K, N, bits, cb)


@pytest.mark.parametrize("cb", [0, 2])
def test_exl3_linear_forward_and_forward_n(oracle, cb):
    """``Exl3Linear::forward`` (one row) and ``forward_n`` (several rows, decode path), fp16 and fp32 outputs."""
    K, N, bits = 1024, 768, 4
    gpu = Gpu(torch.cuda.current_device())
    w = synth.linear_weights(1234, f"eng.lin{cb}", K, N, bits)
    lin = Exl3Linear(gpu, "eng.lin", w["trellis"], w["suh"], w["svh"], bits, Codebook(cb), max_rows=1)
    assert lin.compressed_bytes() == K * N * bits // 8
    x = synth.activations(1234, "eng.x", 5, K)
    c = torch.full((1, N), float("nan"), dtype=torch.float32, device="cuda")
    lin.forward(gpu, dev(x[:1]), c, OutDtype.F32)
    torch.cuda.synchronize()
    assert_close(c.cpu().numpy(), _oracle_linear64(oracle, x[:1], w, K, N, bits, cb), "forward")
    c5 = torch.full((5, N), float("nan"), dtype=torch.float16, device="cuda")
    lin.forward_n(gpu, 5, dev(x), c5, OutDtype.F16)          # grows its rotated-input scratch
    torch.cuda.synchronize()
    assert_close(c5.float().cpu().numpy(), _oracle_linear64(oracle, x, w, K, N, bits, cb), "forward_n")
    assert (host_u16(lin.a_had[:5 * K]).reshape(5, K) == oracle.had_r_128(x, w["suh"], True).view(np.uint16)).all()
    with pytest.raises(Error, match="buffer too small"):
        lin.forward_n(gpu, 5, dev(x), c, OutDtype.F32)
    assert kernels.device_status(torch.cuda.current_device()) == 0


@pytest.mark.parametrize("rows", [2, 33, 150])
def test_exl3_linear_forward_rows(oracle, rows):
    """``Exl3Linear::forward_rows`` (prefill path with a ``RowScratch``): the decode kernel up to 32 rows, the
    tensor-core GEMM above, the weight scratch only required above 144 rows."""
    K, N, bits, cb = 512, 640, 4, 2
    gpu = Gpu(torch.cuda.current_device())
    w = synth.linear_weights(1234, "eng.rows", K, N, bits)
    lin = Exl3Linear(gpu, "eng.rows", w["trellis"], w["suh"], w["svh"], bits, Codebook(cb))
    scratch = RowScratch(gpu, rows, K, N)
    x = synth.activations(1234, f"eng.rows.x{rows}", rows, K)
    c = torch.full((rows, N), float("nan"), dtype=torch.float32, device="cuda")
    lin.forward_rows(gpu, rows, dev(x), c, OutDtype.F32, scratch)
    torch.cuda.synchronize()
    assert_close(c.cpu().numpy(), _oracle_linear64(oracle, x, w, K, N, bits, cb), f"rows {rows}")
    assert (host_u16(scratch.a_had[:rows * K]).reshape(rows, K) == oracle.had_r_128(x, w["suh"], True).view(np.uint16)).all()
    with pytest.raises(Error, match="scratch too small"):
        lin.forward_rows(gpu, rows + 1, dev(x), c, OutDtype.F32, scratch)
    assert kernels.device_status(torch.cuda.current_device()) == 0


def _mlp_oracle(orc, x, ws, H, I, bits, cb):
    """The checker's chain with the fp16 rounding points of the layer: gate and up to fp16, silu(gate) * up to fp16,
    down evaluated in fp64 on those fp16 activations."""
    g, _ = orc.linear(x, ws["gate"]["trellis"], ws["gate"]["suh"], ws["gate"]["svh"], H, I, bits, cb, False)
    u, _ = orc.linear(x, ws["up"]["trellis"], ws["up"]["suh"], ws["up"]["svh"], H, I, bits, cb, False)
    act = orc.silu_mul(g, u)
    return g, u, act, orc.linear_f64(act, ws["down"]["trellis"], ws["down"]["suh"], ws["down"]["svh"], I, H, bits, cb)


@pytest.mark.parametrize("cb,rows", [(2, 1), (2, 3), (2, 8), (2, 20), (0, 1), (0, 6)])
def test_mlp_layer_forward_vs_oracle(oracle, cb, rows):
    """``MlpLayer::forward`` / ``forward_n``: down(silu(gate(x)) * up(x)), fp32 out.  MUL1 layers run gate and up as one
    stacked launch up to eight rows; the intermediate activations are compared too (within one fp16 step of the
    checker's, whose gate/up accumulate in another order), the output against the fp64 evaluation of the checker's
    chain."""
    H, I, bits = 512, 1024, 4
    gpu = Gpu(torch.cuda.current_device())
    ws = {n: synth.linear_weights(1234, f"eng.mlp{cb}.{n}", k, nn, bits, fan_in_gain=True)
          for n, k, nn in (("gate", H, I), ("up", H, I), ("down", I, H))}
    lin = {n: Exl3Linear(gpu, f"mlp.{n}_proj", w["trellis"], w["suh"], w["svh"], bits, Codebook(cb), max_rows=rows) for n, w in ws.items()}
    mlp = MlpLayer(gpu, lin["gate"], lin["up"], lin["down"], max_rows=rows)
    assert (mlp.gate_up is not None) == (cb == 2)
    assert mlp.compressed_bytes() == 3 * H * I * bits // 8
    x = synth.activations(1234, f"eng.mlp.x{rows}", rows, H)
    out = torch.full((rows, H), float("nan"), dtype=torch.float32, device="cuda")
    if rows == 1:
        mlp.forward(gpu, dev(x), out)
    else:
        mlp.forward_n(gpu, rows, dev(x), out)
    torch.cuda.synchronize()
    assert kernels.device_status(torch.cuda.current_device()) == 0
    if cb == 2 and rows <= StackedLinear.BEST_ROWS:
        assert "stack of 2" in kernels.last_launch() or "k_exl3_gemv" in kernels.last_launch()
    g, u, act, y64 = _mlp_oracle(oracle, x, ws, H, I, bits, cb)
    own_act = mlp.activation(gpu).cpu().numpy().reshape(rows, I)   # up to 16 rows the layer never writes it out
    got_act = own_act.astype(np.float32)
    rms_act = np.sqrt((act.astype(np.float64) ** 2).mean())
    assert np.abs(got_act - act.astype(np.float32)).max() <= 2e-2 * rms_act
    # the layer's own activations differ from the checker's by fp16 steps, which the down projection carries on: compare
    # with the fp64 evaluation of the down projection on the LAYER's activations, and loosely with the checker's chain
    y64_own = oracle.linear_f64(own_act, ws["down"]["trellis"], ws["down"]["suh"],
                                ws["down"]["svh"], I, H, bits, cb)
    assert_close(out.cpu().numpy(), y64_own, "down on the layer's activations")
    rms = np.sqrt((y64 ** 2).mean())
    assert np.abs(out.cpu().numpy() - y64).max() <= 2e-2 * rms


def test_mlp_layer_prefill_vs_oracle(oracle):
    """``MlpLayer::prefill`` (crates/berth-engine/src/mlp.rs:219-305) at 160 rows: three tensor-core launches and the
    element-wise kernel."""
    H, I, bits, cb, rows = 256, 512, 4, 2, 160
    gpu = Gpu(torch.cuda.current_device())
    ws = {n: synth.linear_weights(1234, f"eng.pre.{n}", k, nn, bits, fan_in_gain=True)
          for n, k, nn in (("gate", H, I), ("up", H, I), ("down", I, H))}
    lin = {n: Exl3Linear(gpu, f"pre.{n}_proj", w["trellis"], w["suh"], w["svh"], bits, Codebook(cb)) for n, w in ws.items()}
    mlp = MlpLayer(gpu, lin["gate"], lin["up"], lin["down"])
    scratch = RowScratch(gpu, rows, max(H, I), max(H, I))
    x = synth.activations(1234, "eng.pre.x", rows, H, outlier_frac=0.001)
    out = torch.full((rows, H), float("nan"), dtype=torch.float32, device="cuda")
    mlp.prefill(gpu, rows, dev(x), out, scratch)
    torch.cuda.synchronize()
    assert kernels.device_status(torch.cuda.current_device()) == 0
    act_own = mlp.activated[:rows * I].cpu().numpy().reshape(rows, I)
    y64_own = oracle.linear_f64(act_own, ws["down"]["trellis"], ws["down"]["suh"], ws["down"]["svh"], I, H, bits, cb)
    assert_close(out.cpu().numpy(), y64_own, "prefill down")
    _, _, act, y64 = _mlp_oracle(oracle, x, ws, H, I, bits, cb)
    rms_act = np.sqrt((act.astype(np.float64) ** 2).mean())
    assert np.abs(act_own.astype(np.float32) - act.astype(np.float32)).max() <= 2e-2 * rms_act
    assert np.abs(out.cpu().numpy() - y64).max() <= 2e-2 * np.sqrt((y64 ** 2).mean())


def test_mlp_layer_rejects_mismatched_shapes():
    gpu = Gpu(torch.cuda.current_device())
    mk = lambda k, n: Exl3Linear(gpu, "x", torch.zeros((k // 16, n // 16, 64), dtype=torch.int16, device="cuda"),
                                 torch.zeros(k, dtype=torch.float16, device="cuda"), torch.zeros(n, dtype=torch.float16, device="cuda"),
                                 4, Codebook(2))
    with pytest.raises(Error, match="up is"):
        MlpLayer(gpu, mk(256, 512), mk(256, 256), mk(512, 256))
    with pytest.raises(Error, match="down is"):
        MlpLayer(gpu, mk(256, 512), mk(256, 512), mk(256, 256))
