"""Host-side mirror of berth's ``berth-kernels`` crate over the C ABI.

Function names, argument order and error behaviour follow the Rust wrappers:
``exl3_linear`` / ``last_launch`` / ``last_error`` (crates/berth-kernels/src/lib.rs:135-205),
``prefill_lin::exl3_linear`` / ``exl3_gemv_cfg`` (src/prefill_lin.rs:117-161,224),
``ops::silu_mul`` / ``ops::add_f32`` (src/ops.rs:507-520).  Pointers are device addresses: pass
an ``int`` or anything with ``data_ptr()`` (a torch CUDA tensor).  A non-zero return code of
the library raises :class:`Error` with the library's message, as ``Error::Launch`` does.
"""
from __future__ import annotations

import enum

from . import _lib


class Error(RuntimeError):
    """``berth_kernels::Error::Launch``."""


class Codebook(enum.IntEnum):
    """crates/berth-kernels/src/lib.rs:54-63."""
    Default = 0
    Mcg = 1
    Mul1 = 2


class OutDtype(enum.IntEnum):
    """crates/berth-kernels/src/lib.rs:70-84."""
    F16 = 0
    F32 = 1


def _ptr(x):
    if x is None:
        return None
    if isinstance(x, int):
        return x
    return x.data_ptr()


def _stream(stream):
    if stream is None:
        return None
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream


def _s(b) -> str:
    return (b or b"").decode("utf-8", "replace")


def last_launch() -> str:
    return _s(_lib.lib().berth_exl3_last_launch())


def last_error() -> str:
    return _s(_lib.lib().berth_exl3_last_error())


def exl3_linear(a, trellis, c, suh, a_had, svh, size_m: int, size_k: int, size_n: int, k_bits: int,
                codebook: Codebook, out: OutDtype, stream=None) -> None:
    """One EXL3 linear ``C = A @ trellis`` with the Hadamard sign-scales; decode passes size_m = 1."""
    l = _lib.lib()
    rc = l.berth_exl3_linear(_ptr(a), _ptr(trellis), _ptr(c), _ptr(suh), _ptr(a_had), _ptr(svh), size_m, size_k,
                             size_n, k_bits, int(codebook), int(out), _stream(stream))
    if rc != 0:
        raise Error(last_error() or f"exl3 linear launch failed ({rc})")


def exl3_linear_static_scratch(a, trellis, c, suh, a_had, svh, size_m: int, size_k: int, size_n: int, k_bits: int,
                               codebook: Codebook, out: OutDtype, stream=None) -> None:
    """:func:`exl3_linear` for hosts that must not allocate device memory (their own planner owns
    all of HBM, or the decode loop cannot take a ``cudaMalloc`` stall): the scratch is a fixed array
    of about 6.1 MiB inside the library, shared by every call on the device.  ``size_m <= 32``,
    ``size_n <= 131072``, ``size_k * ceil(size_m / 8) <= 131072``; calls must not overlap on the GPU;
    make the first call on a device before any stream capture."""
    rc = _lib.lib().berth_exl3_linear_static_scratch(_ptr(a), _ptr(trellis), _ptr(c), _ptr(suh), _ptr(a_had),
                                                     _ptr(svh), size_m, size_k, size_n, k_bits, int(codebook),
                                                     int(out), _stream(stream))
    if rc != 0:
        raise Error(last_error() or f"exl3 linear (static scratch) launch failed ({rc})")


def exl3_linear_add(a, trellis, c, suh, a_had, svh, residual, size_m: int, size_k: int, size_n: int, k_bits: int,
                    codebook: Codebook, stream=None) -> None:
    """:func:`exl3_linear` (``size_m <= 32``, fp32 output) with ``residual`` added in the kernel's last step;
    ``c`` may be ``residual``."""
    rc = _lib.lib().berth_exl3_linear_add(_ptr(a), _ptr(trellis), _ptr(c), _ptr(suh), _ptr(a_had), _ptr(svh), _ptr(residual), size_m,
                                          size_k, size_n, k_bits, int(codebook), _stream(stream))
    if rc != 0:
        raise Error(last_error() or f"exl3 linear add launch failed ({rc})")


def exl3_linear_silu(gate, up, trellis, c, suh, a_had, svh, size_m: int, size_k: int, size_n: int, k_bits: int,
                     codebook: Codebook, out: OutDtype, act_limit: float = 0.0, residual=None, stream=None) -> None:
    """``c = [residual +] linear(silu(gate) * up)`` for ``size_m <= 32`` rows: the down projection of an MLP with the
    activation formed inside the linear's rotation, bit for bit what ``ops.silu_mul`` followed by :func:`exl3_linear`
    (and ``ops.add_f32``) gives, without the activation's launch and buffer."""
    rc = _lib.lib().berth_exl3_linear_silu(_ptr(gate), _ptr(up), _ptr(trellis), _ptr(c), _ptr(suh), _ptr(a_had), _ptr(svh),
                                           _ptr(residual) if residual is not None else None, float(act_limit), size_m, size_k,
                                           size_n, k_bits, int(codebook), int(out), _stream(stream))
    if rc != 0:
        raise Error(last_error() or f"exl3 linear silu launch failed ({rc})")


def exl3_linear_stack(a, trellis_stack, c, suh_stack, a_had, svh_stack, n_matrices: int, size_m: int, size_k: int, size_n: int,
                      k_bits: int, codebook: Codebook, out: OutDtype, stream=None) -> None:
    """``n_matrices`` equally shaped MUL1 linears (stored one behind the other) applied to the same ``size_m <= 8`` rows in
    one decode launch; ``c`` is ``[n_matrices][size_m][size_n]``, ``a_had`` ``[n_matrices][size_m][size_k]``."""
    rc = _lib.lib().berth_exl3_linear_stack(_ptr(a), _ptr(trellis_stack), _ptr(c), _ptr(suh_stack), _ptr(a_had), _ptr(svh_stack),
                                            n_matrices, size_m, size_k, size_n, k_bits, int(codebook), int(out), _stream(stream))
    if rc != 0:
        raise Error(last_error() or f"exl3 linear stack launch failed ({rc})")


def pointer_list(xs):
    """A host array of device addresses (one per tensor or integer address of ``xs``) for :func:`exl3_linear_multi`."""
    import ctypes
    return (ctypes.c_void_p * max(len(xs), 1))(*[_ptr(x) for x in xs])


def int_list(xs):
    """A host array of C ints for :func:`exl3_linear_multi`."""
    import ctypes
    return (ctypes.c_int * max(len(xs), 1))(*[int(v) for v in xs])


def exl3_linear_multi(a, trellis_list, c_list, suh_list, a_had_list, svh_list, size_n_list, n_matrices: int, size_m: int,
                      size_k: int, k_bits: int, codebook: Codebook, out: OutDtype, stream=None) -> None:
    """Up to four MUL1 linears of different widths applied to the same ``size_m <= 8`` rows in one decode launch (q, k and v
    of an attention block).  The lists are host arrays built with :func:`pointer_list` / :func:`int_list` (one entry per
    matrix); build them once per layer, not per call."""
    rc = _lib.lib().berth_exl3_linear_multi(_ptr(a), trellis_list, c_list, suh_list, a_had_list, svh_list, size_n_list, n_matrices,
                                            size_m, size_k, k_bits, int(codebook), int(out), _stream(stream))
    if rc != 0:
        raise Error(last_error() or f"exl3 linear multi launch failed ({rc})")


def exl3_linear_argmax(a, trellis, c, suh, a_had, svh, best, size_m: int, size_k: int, size_n: int, k_bits: int,
                       codebook: Codebook, out: OutDtype, stream=None) -> None:
    """:func:`exl3_linear` (``size_m <= 32``) that also leaves, in the device array ``best`` (``size_m`` 64-bit keys),
    the largest output of every row: the greedy token of an lm_head without a pass over the logits.  ``c`` may be
    ``None`` (the logits are then not written).  :func:`argmax_key_decode` splits a key read back from the device."""
    rc = _lib.lib().berth_exl3_linear_argmax(_ptr(a), _ptr(trellis), _ptr(c), _ptr(suh), _ptr(a_had), _ptr(svh), _ptr(best),
                                             size_m, size_k, size_n, k_bits, int(codebook), int(out), _stream(stream))
    if rc != 0:
        raise Error(last_error() or f"exl3 linear argmax launch failed ({rc})")


def exl3_linear_sample(a, trellis, c, suh, a_had, svh, best, size_m: int, size_k: int, size_n: int, k_bits: int,
                       codebook: Codebook, out: OutDtype, inv_temp: float, random: int, mode: int, stream=None) -> None:
    """:func:`exl3_linear_argmax` with berth's fused sampler in either of its modes taken in the finishing step: ``mode`` 0
    greedy, 1 Gumbel arg-max over ``outputs * inv_temp`` with the noise of ``(random, row, column)`` -- one draw from the
    softmax per row.  The keys in ``best`` carry the winning score and column."""
    rc = _lib.lib().berth_exl3_linear_sample(_ptr(a), _ptr(trellis), _ptr(c), _ptr(suh), _ptr(a_had), _ptr(svh), _ptr(best),
                                             size_m, size_k, size_n, k_bits, int(codebook), int(out), float(inv_temp),
                                             int(random) & 0xFFFFFFFF, int(mode), _stream(stream))
    if rc != 0:
        raise Error(last_error() or f"exl3 linear sample launch failed ({rc})")


def argmax_key_decode(key: int) -> tuple:
    """(token, value) of a key written by :func:`exl3_linear_argmax`; ties went to the lower token."""
    import ctypes as C
    tok, val = C.c_int32(), C.c_float()
    _lib.lib().berth_argmax_key_decode(int(key) & 0xFFFFFFFFFFFFFFFF, C.byref(tok), C.byref(val))
    return tok.value, val.value


def device_cc(device: int) -> int:
    return _lib.lib().berth_device_cc(device)


def weights_streamed(on: bool) -> bool:
    """Process-wide: ``True`` makes every decode kernel wait for its predecessor on the stream before it fetches weights (for
    hosts that write a trellis directly before the linear that reads it); returns the previous setting."""
    return bool(_lib.lib().berth_exl3_weights_streamed(1 if on else 0))


def device_sms(device: int) -> int:
    return _lib.lib().berth_device_sms(device)


def device_status(device: int) -> int:
    """Reads and clears the bounded-wait status word of the decode kernels (synchronises)."""
    return _lib.lib().berth_device_status(device)


def decode_rate(k_bits: int, codebook: Codebook, path: int, warps: int = 16, iters: int = 4096) -> tuple:
    """Bare decode rate of one SM (diagnostic): (weights per clock per SM, SM MHz during the run) of the decode
    GEMV's inner loop on shared-memory-resident tiles.  ``path`` 0 = fp16 tensor path, 1 = MUL1 integer tensor path."""
    import ctypes as C
    w, mhz = C.c_double(), C.c_double()
    rc = _lib.lib().berth_exl3_decode_rate(k_bits, int(codebook), path, warps, iters, C.byref(w), C.byref(mhz))
    if rc != 0:
        raise Error(last_error() or f"decode rate failed ({rc})")
    return w.value, mhz.value


def pipe_probe(kind: int, iters: int = 4096) -> float:
    """Cycles one bundle of independent instructions costs a warp scheduler (diagnostic; kinds in include/berth_b200.h)."""
    import ctypes as C
    v = C.c_double()
    rc = _lib.lib().berth_exl3_pipe_probe(kind, iters, C.byref(v))
    if rc != 0:
        raise Error(last_error() or f"pipe probe failed ({rc})")
    return v.value


def gemm_tune_key(size_m, size_k, size_n, k_bits, out_fp32, device, cc, sms, cb) -> int:
    return _lib.lib().berth_exl3_gemm_tune_key(size_m, size_k, size_n, k_bits, out_fp32, device, cc, sms, cb)


class prefill_lin:
    """crates/berth-kernels/src/prefill_lin.rs."""

    @staticmethod
    def last_launch() -> str:
        return _s(_lib.lib().berth_prefill_last_launch())

    @staticmethod
    def last_error() -> str:
        return _s(_lib.lib().berth_prefill_last_error())

    @staticmethod
    def exl3_linear(a, trellis, c, suh, a_had, svh, w_scratch, size_m, size_k, size_n, k_bits,
                    codebook: Codebook, out: OutDtype, stream=None) -> None:
        l = _lib.lib()
        rc = l.berth_prefill_exl3_linear(_ptr(a), _ptr(trellis), _ptr(c), _ptr(suh), _ptr(a_had), _ptr(svh),
                                         _ptr(w_scratch), size_m, size_k, size_n, k_bits, int(codebook), int(out),
                                         _stream(stream))
        if rc != 0:
            raise Error(prefill_lin.last_error() or f"prefill exl3 linear launch failed ({rc})")

    @staticmethod
    def hgemm(a, b, c, size_m, size_k, size_n, ldc, out: OutDtype, stream=None) -> None:
        rc = _lib.lib().berth_prefill_hgemm(_ptr(a), _ptr(b), _ptr(c), size_m, size_k, size_n, ldc, int(out),
                                            _stream(stream))
        if rc != 0:
            raise Error(prefill_lin.last_error() or f"prefill hgemm launch failed ({rc})")

    @staticmethod
    def exl3_gemv_cfg(cc, size_m, size_k, size_n, k_bits, cb, mode, narrow_coresident) -> int:
        return _lib.lib().berth_exl3_gemv_cfg(cc, size_m, size_k, size_n, k_bits, int(cb), mode, narrow_coresident)

    @staticmethod
    def reconstruct(unpacked, packed, size_k, slice_n, full_n, n_offset, k_bits, codebook, stream=None) -> None:
        rc = _lib.lib().berth_prefill_reconstruct(_ptr(unpacked), _ptr(packed), size_k, slice_n, full_n, n_offset,
                                                  k_bits, int(codebook), _stream(stream))
        if rc != 0:
            raise Error(prefill_lin.last_error())

    @staticmethod
    def had_r_128(inp, out, scale, pre_scale: bool, rows, cols, fp32: bool, stream=None) -> None:
        rc = _lib.lib().berth_prefill_had_r_128(_ptr(inp), _ptr(out), _ptr(scale), int(pre_scale), rows, cols,
                                                int(fp32), _stream(stream))
        if rc != 0:
            raise Error(prefill_lin.last_error())


class ops:
    """crates/berth-kernels/src/ops.rs."""

    @staticmethod
    def last_launch() -> str:
        return _s(_lib.lib().berth_ops_last_launch())

    @staticmethod
    def last_error() -> str:
        return _s(_lib.lib().berth_ops_last_error())

    @staticmethod
    def silu_mul(gate, up, out, numel: int, act_limit: float = 0.0, stream=None) -> None:
        rc = _lib.lib().berth_ops_silu_mul(_ptr(gate), _ptr(up), _ptr(out), numel, act_limit, _stream(stream))
        if rc != 0:
            raise Error(ops.last_error() or f"silu_mul launch failed ({rc})")

    @staticmethod
    def exl3_mgemm(a, b_list, c, suh_list, a_had, svh_list, size_m: int, size_k: int, size_n: int, k_bits: int, codebook,
                   out, bszm_in: int, bszm_out: int, size_n_list, c_ptrs, n_stride_list, had_src_list, num_had_src: int,
                   stream=None) -> int:
        """``ops::exl3_mgemm`` (crates/berth-kernels/src/ops.rs:317-367): returns the positive shape tag."""
        rc = _lib.lib().berth_ops_mgemm(_ptr(a), _ptr(b_list), _ptr(c), _ptr(suh_list), _ptr(a_had), _ptr(svh_list), size_m, size_k,
                                        size_n, k_bits, int(codebook), int(out), bszm_in, bszm_out, _ptr(size_n_list), _ptr(c_ptrs),
                                        _ptr(n_stride_list), _ptr(had_src_list), num_had_src, _stream(stream))
        if rc > 0:
            return rc
        raise Error(ops.last_error() or f"exl3_mgemm launch failed ({rc})")

    @staticmethod
    def mgemm_tune_key(size_m: int, size_k: int, size_n: int, k_bits: int, out, device: int, cc: int, sms: int, codebook,
                       bszm_in: int, bszm_out: int, sliced: bool) -> int:
        """``ops::mgemm_tune_key`` (crates/berth-kernels/src/ops.rs:215-245)."""
        return int(_lib.lib().berth_ops_mgemm_tune_key(size_m, size_k, size_n, k_bits, int(out), device, cc, sms, int(codebook),
                                                       bszm_in, bszm_out, 1 if sliced else 0))

    @staticmethod
    def add_f32(a, b, c, n: int, stream=None) -> None:
        rc = _lib.lib().berth_ops_add_f32(_ptr(a), _ptr(b), _ptr(c), n, _stream(stream))
        if rc != 0:
            raise Error(ops.last_error() or f"add_f32 launch failed ({rc})")

    @staticmethod
    def rms_norm(x, weight, y, rows: int, dim: int, epsilon: float, constant_bias: float, constant_scale: float,
                 weight_bf16: bool, stream=None) -> None:
        """``ops::rms_norm`` (crates/berth-kernels/src/ops.rs): fp32 rows -> fp16 rows."""
        rc = _lib.lib().berth_ops_rms_norm(_ptr(x), _ptr(weight), _ptr(y), rows, dim, epsilon, constant_bias, constant_scale,
                                           1 if weight_bf16 else 0, _stream(stream))
        if rc != 0:
            raise Error(ops.last_error() or f"rms_norm launch failed ({rc})")

    @staticmethod
    def rms_norm_f16(x, weight, y, rows: int, dim: int, epsilon: float, constant_bias: float, constant_scale: float,
                     stream=None) -> None:
        """``ops::rms_norm_f16``: fp16 rows, bfloat16 weight -> fp16 rows."""
        rc = _lib.lib().berth_ops_rms_norm_f16(_ptr(x), _ptr(weight), _ptr(y), rows, dim, epsilon, constant_bias, constant_scale,
                                               _stream(stream))
        if rc != 0:
            raise Error(ops.last_error() or f"rms_norm_f16 launch failed ({rc})")

    @staticmethod
    def rms_norm_res_in(x, weight, y, residual, rows: int, dim: int, epsilon: float, constant_bias: float, constant_scale: float,
                        weight_bf16: bool, stream=None) -> None:
        """``ops::rms_norm_res_in``: residual += x in place (fp32), y = the norm of the updated residual."""
        rc = _lib.lib().berth_ops_rms_norm_res_in(_ptr(x), _ptr(weight), _ptr(y), _ptr(residual), rows, dim, epsilon, constant_bias,
                                                  constant_scale, 1 if weight_bf16 else 0, _stream(stream))
        if rc != 0:
            raise Error(ops.last_error() or f"rms_norm_res_in launch failed ({rc})")
