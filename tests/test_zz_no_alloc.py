"""The allocation-free decode linear (``berth_exl3_linear_static_scratch``).

Some hosts cannot let a library call cudaMalloc: their planner has already placed every byte of
HBM, or their decode loop cannot absorb the device-wide stall of an allocation.  For them the
library offers the same linear with its split-K scratch in a fixed array inside the library
image.  This test drives that entry point through the C ABI twice in a row (the second call
finds the scratch exactly as the first left it) and compares both results with the ordinary
entry point's output on the same inputs and with the CPU checker's fp64 evaluation; afterwards
the status word of the fixed scratch (read through berth_device_status) must be clean.
Collected last on purpose, so a failure here cannot hide the result of any other test.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from berth_b200 import Codebook, Error, OutDtype, kernels, synth   # noqa: E402
from tests.gpu_util import assert_close, dev   # noqa: E402


@pytest.mark.parametrize("m,K,N,bits,cb,out_fp32", [(1, 5120, 6144, 4, 2, False), (3, 2048, 1024, 4, 0, True),
                                                   (32, 1024, 640, 5, 1, False)])
def test_static_scratch_matches_ordinary_entry_point_twice(oracle, m, K, N, bits, cb, out_fp32):
    w = synth.linear_weights(1234, f"noalloc{K}x{N}", K, N, bits)
    x = synth.activations(1234, f"noalloc.x{m}", m, K)
    xd, td, sd, vd = dev(x), dev(w["trellis"]), dev(w["suh"]), dev(w["svh"])
    dt = torch.float32 if out_fp32 else torch.float16
    out = OutDtype.F32 if out_fp32 else OutDtype.F16
    ref = torch.empty((m, N), dtype=dt, device="cuda")
    ah_ref = torch.zeros((m, K), dtype=torch.float16, device="cuda")
    kernels.exl3_linear(xd, td, ref, sd, ah_ref, vd, m, K, N, bits, Codebook(cb), out)
    torch.cuda.synchronize()
    ref_h = ref.float().cpu().numpy().astype(np.float64)
    rms = np.sqrt((ref_h ** 2).mean())
    for call in range(2):
        got = torch.full((m, N), float("nan"), dtype=dt, device="cuda")
        ah = torch.zeros((m, K), dtype=torch.float16, device="cuda")
        kernels.exl3_linear_static_scratch(xd, td, got, sd, ah, vd, m, K, N, bits, Codebook(cb), out)
        torch.cuda.synchronize()
        assert "static-scratch" in kernels.last_launch()
        diff = np.abs(got.float().cpu().numpy().astype(np.float64) - ref_h)
        # same kernel; only the split-K factor (hence the summation order) may differ
        assert diff.max() <= 2e-3 * rms, (call, diff.max() / rms)
        assert torch.equal(ah, ah_ref)
        if call == 1:
            y64 = oracle.linear_f64(x, w["trellis"], w["suh"], w["svh"], K, N, bits, cb)
            assert_close(got.float().cpu().numpy(), y64, "static scratch")
    assert kernels.device_status(torch.cuda.current_device()) == 0


def test_static_scratch_rejects_sizes_beyond_its_maximum():
    P = 64
    with pytest.raises(Error, match="exceeds the maximum of 32 rows"):
        kernels.exl3_linear_static_scratch(P, P, P, P, P, P, 33, 128, 128, 4, Codebook.Mul1, OutDtype.F16)
    with pytest.raises(Error, match="exceeds the maximum of 131072 columns"):
        kernels.exl3_linear_static_scratch(P, P, P, P, P, P, 1, 128, 131072 + 128, 4, Codebook.Mul1, OutDtype.F16)
    with pytest.raises(Error, match="null"):
        kernels.exl3_linear_static_scratch(None, P, P, P, P, P, 1, 128, 128, 4, Codebook.Mul1, OutDtype.F16)
    # 17..32 rows are processed in four groups of eight: size_k * 4 must fit (refused before any launch)
    with pytest.raises(Error, match="exceeds the maximum of size_k"):
        kernels.exl3_linear_static_scratch(P, P, P, P, P, P, 17, 40960, 128, 4, Codebook.Mul1, OutDtype.F16)
    with pytest.raises(Error, match="exceeds the maximum of size_k"):
        kernels.exl3_linear_static_scratch(P, P, P, P, P, P, 9, 69632, 128, 4, Codebook.Default, OutDtype.F16)
