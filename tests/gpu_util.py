"""Helpers shared by the GPU parity tests: device buffers from numpy, the tolerance rule."""
import numpy as np
import torch

from berth_b200 import Codebook, OutDtype, kernels


def dev(a: np.ndarray) -> torch.Tensor:
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        a = a.view(np.int16)
    return torch.from_numpy(a).cuda()


def host_u16(t: torch.Tensor) -> np.ndarray:
    return t.cpu().numpy().view(np.uint16)


def run_linear(x, w, bits, cb, out_fp32, prefill=False):
    """x float16 [m][k] numpy; w dict(trellis,suh,svh,size_k,size_n).  Returns (c numpy, a_had uint16 numpy)."""
    m, k = x.shape
    n = w["size_n"]
    xd, td, sd, vd = dev(x), dev(w["trellis"]), dev(w["suh"]), dev(w["svh"])
    c = torch.full((m, n), float("nan"), dtype=torch.float32 if out_fp32 else torch.float16, device="cuda")
    ah = torch.zeros((m, k), dtype=torch.float16, device="cuda")
    out = OutDtype.F32 if out_fp32 else OutDtype.F16
    if prefill:
        scratch = torch.empty(1, dtype=torch.float16, device="cuda")
        kernels.prefill_lin.exl3_linear(xd, td, c, sd, ah, vd, scratch, m, k, n, bits, Codebook(cb), out)
    else:
        kernels.exl3_linear(xd, td, c, sd, ah, vd, m, k, n, bits, Codebook(cb), out)
    torch.cuda.synchronize()
    return c.cpu().numpy(), host_u16(ah)


def rel_errors(got, y64):
    """(max, mean) of |got - y64| / rms(y64): the scale of the 1e-2 / 1e-3 gates."""
    y64 = np.asarray(y64, np.float64)
    rms = np.sqrt((y64 ** 2).mean())
    err = np.abs(np.asarray(got, np.float64) - y64) / rms
    return float(err.max()), float(err.mean())


MAX_REL, MEAN_REL = 1e-2, 1e-3   # tolerance of fp32-accumulated outputs against the fp64 evaluation


def elementwise_rel_errors(got, y64):
    """(max, mean) of |got - y64| / |y64| over the elements with |y64| >= rms(y64): the literal element-wise reading
    of the tolerance, where it is well defined (an element-wise ratio blows up at the zero crossings of a zero-mean
    output, which is why rel_errors divides by the RMS instead)."""
    y64 = np.asarray(y64, np.float64)
    got = np.asarray(got, np.float64)
    rms = np.sqrt((y64 ** 2).mean())
    big = np.abs(y64) >= rms
    if not big.any():
        return 0.0, 0.0
    err = np.abs(got[big] - y64[big]) / np.abs(y64[big])
    return float(err.max()), float(err.mean())


def assert_close(got, y64, what=""):
    """Both forms of the tolerance: errors relative to rms(y64) over all elements, and element-wise relative errors
    over the elements of at least RMS magnitude; max <= 1e-2 and mean <= 1e-3 each.  Returns the four numbers."""
    assert np.isfinite(np.asarray(got, np.float64)).all(), (what, "non-finite output")
    mx, mean = rel_errors(got, y64)
    emx, emean = elementwise_rel_errors(got, y64)
    assert mx <= MAX_REL and mean <= MEAN_REL, (what, "relative to rms", mx, mean)
    assert emx <= MAX_REL and emean <= MEAN_REL, (what, "element-wise", emx, emean)
    return mx, mean, emx, emean
