"""Host-side callers of the EXL3 linear, mirroring ``berth-engine``:
``Gpu`` (crates/berth-engine/src/device.rs:15-43), ``Exl3Linear`` (device.rs:77-164,206-268),
``RowScratch`` (device.rs:178-204) and ``MlpLayer`` (crates/berth-engine/src/mlp.rs:25-150,219-305).

PyTorch is used only to own device memory and streams; every computation is a call into
``libberth_b200.so`` through :mod:`berth_b200.kernels`.  Buffers are torch CUDA tensors.
"""
from __future__ import annotations

import numpy as np
import torch

from . import kernels
from .kernels import Codebook, OutDtype

ACT_LIMIT = 0.0          # crates/berth-engine/src/mlp.rs:22
MAX_RECONSTRUCT_N = 32768  # crates/berth-engine/src/device.rs:176


class Error(RuntimeError):
    """``berth_engine::Error`` (Weights / Input)."""


class Gpu:
    """One device and the stream every launch of a model goes to."""

    def __init__(self, device: int = 0, stream: torch.cuda.Stream | None = None):
        if not torch.cuda.is_available():
            raise Error("berth_b200 needs a CUDA device: there is no CPU path")
        self.device = torch.device("cuda", device)
        torch.cuda.set_device(self.device)
        self.stream = stream if stream is not None else torch.cuda.current_stream(self.device)
        self.sms = kernels.device_sms(device)

    def raw_stream(self) -> int:
        return self.stream.cuda_stream

    def zeroed(self, nbytes: int) -> torch.Tensor:
        return torch.zeros(nbytes, dtype=torch.uint8, device=self.device)

    def upload(self, a: np.ndarray) -> torch.Tensor:
        a = np.ascontiguousarray(a)
        if a.dtype == np.uint16:
            a = a.view(np.int16)
        return torch.from_numpy(a).to(self.device, non_blocking=False)


class Exl3Linear:
    """One EXL3 linear resident on the device: trellis, fp16 sign-scales and the fp16 scratch the
    kernel writes the rotated input to."""

    def __init__(self, gpu: Gpu, prefix: str, trellis, suh, svh, k_bits: int, codebook: Codebook, max_rows: int = 1):
        self.prefix = prefix
        self.trellis = trellis if isinstance(trellis, torch.Tensor) else gpu.upload(trellis)
        self.suh = suh if isinstance(suh, torch.Tensor) else gpu.upload(suh)
        self.svh = svh if isinstance(svh, torch.Tensor) else gpu.upload(svh)
        self.size_k = int(self.suh.numel())
        self.size_n = int(self.svh.numel())
        self.k_bits = int(k_bits)
        self.codebook = Codebook(codebook)
        if tuple(self.trellis.shape) != (self.size_k // 16, self.size_n // 16, 16 * self.k_bits):
            raise Error(f"{prefix}: trellis shape {tuple(self.trellis.shape)} does not match "
                        f"({self.size_k // 16}, {self.size_n // 16}, {16 * self.k_bits})")
        self.a_had = torch.zeros(max_rows * self.size_k, dtype=torch.float16, device=gpu.device)

    @classmethod
    def load(cls, gpu: Gpu, tensors: dict, prefix: str, k_bits: int, codebook: Codebook) -> "Exl3Linear":
        """From a mapping ``<prefix>.trellis/.suh/.svh`` -> array, the grouping rule of
        crates/berth-exl3/src/linear.rs:122-138."""
        for part in ("trellis", "suh", "svh"):
            if f"{prefix}.{part}" not in tensors:
                raise Error(f"{prefix} is not an EXL3 linear (no {part})")
        if f"{prefix}.bias" in tensors:
            raise Error(f"{prefix}: bias is present and is not applied")
        return cls(gpu, prefix, tensors[f"{prefix}.trellis"], tensors[f"{prefix}.suh"], tensors[f"{prefix}.svh"],
                   k_bits, codebook)

    def compressed_bytes(self) -> int:
        return self.trellis.numel() * 2

    def forward(self, gpu: Gpu, a: torch.Tensor, c: torch.Tensor, out: OutDtype) -> None:
        """``c = a @ W`` for one row: a fp16 [size_k], c [size_n] of ``out``."""
        self.forward_n(gpu, 1, a, c, out)

    def forward_n(self, gpu: Gpu, rows: int, a: torch.Tensor, c: torch.Tensor, out: OutDtype) -> None:
        """Decode-path launch for ``rows`` rows (crates/berth-engine/src/device.rs:285-366)."""
        out_bytes = 2 if out == OutDtype.F16 else 4
        if a.numel() * a.element_size() < rows * self.size_k * 2 or \
                c.numel() * c.element_size() < rows * self.size_n * out_bytes:
            raise Error(f"{self.prefix}: buffer too small")
        if self.a_had.numel() < rows * self.size_k:
            self.a_had = torch.zeros(rows * self.size_k, dtype=torch.float16, device=gpu.device)
        kernels.exl3_linear(a, self.trellis, c, self.suh, self.a_had, self.svh, rows, self.size_k, self.size_n,
                            self.k_bits, self.codebook, out, gpu.raw_stream())

    def forward_silu_n(self, gpu: Gpu, rows: int, gate: torch.Tensor, up: torch.Tensor, c: torch.Tensor, out: OutDtype,
                       act_limit: float = 0.0, residual: torch.Tensor | None = None) -> None:
        """``c = [residual +] (silu(gate) * up) @ W`` for up to 32 rows, the activation formed inside the launch (the
        down projection of an MLP: crates/berth-engine/src/mlp.rs:128-160 without the ``silu_mul`` launch)."""
        out_bytes = 2 if out == OutDtype.F16 else 4
        need = rows * self.size_k * 2
        if gate.numel() * gate.element_size() < need or up.numel() * up.element_size() < need or \
                c.numel() * c.element_size() < rows * self.size_n * out_bytes:
            raise Error(f"{self.prefix}: buffer too small")
        if self.a_had.numel() < rows * self.size_k:
            self.a_had = torch.zeros(rows * self.size_k, dtype=torch.float16, device=gpu.device)
        kernels.exl3_linear_silu(gate, up, self.trellis, c, self.suh, self.a_had, self.svh, rows, self.size_k, self.size_n,
                                 self.k_bits, self.codebook, out, act_limit, residual, gpu.raw_stream())

    def forward_argmax(self, gpu: Gpu, rows: int, a: torch.Tensor, best: torch.Tensor, c: torch.Tensor | None = None,
                       out: OutDtype = OutDtype.F32) -> None:
        """The decode launch of an lm_head with the greedy token of every row taken in its finishing step:
        ``best`` (int64 [rows], device) receives the keys ``kernels.argmax_key_decode`` splits; ``c`` is optional."""
        if a.numel() * a.element_size() < rows * self.size_k * 2 or best.numel() * best.element_size() < rows * 8:
            raise Error(f"{self.prefix}: buffer too small")
        if self.a_had.numel() < rows * self.size_k:
            self.a_had = torch.zeros(rows * self.size_k, dtype=torch.float16, device=gpu.device)
        kernels.exl3_linear_argmax(a, self.trellis, c, self.suh, self.a_had, self.svh, best, rows, self.size_k, self.size_n,
                                   self.k_bits, self.codebook, out, gpu.raw_stream())

    def forward_rows(self, gpu: Gpu, rows: int, a: torch.Tensor, c: torch.Tensor, out: OutDtype,
                     scratch: "RowScratch") -> None:
        """Prefill-path launch, rows > 1 (crates/berth-engine/src/device.rs:210-268)."""
        if rows > scratch.max_rows or self.size_k > scratch.max_k or self.size_n > scratch.max_n:
            raise Error(f"{self.prefix}: scratch too small")
        kernels.prefill_lin.exl3_linear(a, self.trellis, c, self.suh, scratch.a_had, self.svh,
                                        scratch.weight if rows > 144 else None, rows, self.size_k, self.size_n,
                                        self.k_bits, self.codebook, out, gpu.raw_stream())


class SlicedMultiLinear:
    """Several EXL3 linears that share one input, run as one launch over column slices of their greatest common
    width (the fork's ``SlicedMultiLinear``, which berth drives through ``ops::exl3_mgemm``,
    crates/berth-kernels/tests/ops.rs:250-345): the q / k / v projections of an attention layer, or the qkv and z
    projections of a gated-delta-net layer.  All sources must share size_k, k_bits and codebook."""

    def __init__(self, gpu: Gpu, sources: list, out: OutDtype, max_rows: int = 1, outputs: list | None = None):
        import math
        first = sources[0]
        for s in sources:
            if (s.size_k, s.k_bits, s.codebook) != (first.size_k, first.k_bits, first.codebook):
                raise Error("SlicedMultiLinear: sources must share size_k, k_bits and codebook")
        self.sources, self.out, self.max_rows = sources, out, max_rows
        self.size_k, self.k_bits, self.codebook = first.size_k, first.k_bits, first.codebook
        self.width = 0
        for s in sources:
            self.width = math.gcd(self.width, s.size_n)
        elem = 2 if out == OutDtype.F16 else 4
        dt = torch.float16 if out == OutDtype.F16 else torch.float32
        if outputs is None:
            outputs = [torch.empty((max_rows, s.size_n), dtype=dt, device=gpu.device) for s in sources]
        for o, s in zip(outputs, sources):
            if o.dtype != dt or tuple(o.shape) != (max_rows, s.size_n) or not o.is_contiguous():
                raise Error("SlicedMultiLinear: an output must be a contiguous [max_rows][size_n] tensor of the output type")
        self.outputs = list(outputs)
        b, svh, c, widths, strides, had = [], [], [], [], [], []
        for i, s in enumerate(sources):
            for n0 in range(0, s.size_n, self.width):
                b.append(s.trellis.data_ptr() + (n0 // 16) * 16 * self.k_bits * 2)
                svh.append(s.svh.data_ptr() + n0 * 2)
                c.append(self.outputs[i].data_ptr() + n0 * elem)
                widths.append(self.width); strides.append(s.size_n); had.append(i)
        u64 = lambda v: torch.tensor(v, dtype=torch.int64, device=gpu.device)
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=gpu.device)
        self.b_list, self.svh_list, self.c_ptrs = u64(b), u64(svh), u64(c)
        self.suh_list = u64([s.suh.data_ptr() for s in sources])
        self.size_n_list, self.n_stride_list, self.had_src_list = i32(widths), i32(strides), i32(had)
        self.slices = len(b)
        self.a_had = torch.zeros(len(sources) * max_rows * self.size_k, dtype=torch.float16, device=gpu.device)
        self.carrier = torch.empty(1, dtype=dt, device=gpu.device)
        # MUL1 sources, few of them: the library's multi-matrix decode launch takes the addresses from host arrays
        # (one TMA view per matrix, rotation inside the kernel) and is the faster path for the smallest batches.
        self.multi = None
        if self.codebook == Codebook.Mul1 and len(sources) <= 4:
            n = len(sources)
            row_bytes = self.size_k * 2
            self.multi = (kernels.pointer_list([s.trellis for s in sources]), kernels.pointer_list(self.outputs),
                          kernels.pointer_list([s.suh for s in sources]),
                          kernels.pointer_list([self.a_had.data_ptr() + i * max_rows * row_bytes for i in range(n)]),
                          kernels.pointer_list([s.svh for s in sources]), kernels.int_list([s.size_n for s in sources]), n)

    MULTI_ROWS = 4   # up to here the multi-matrix launch is used (above, the sliced launch of the fp16-path kernel)

    def forward_n(self, gpu: Gpu, rows: int, a: torch.Tensor) -> list:
        """One launch; returns the per-source outputs ``[max_rows][size_n]`` (the first ``rows`` rows are written)."""
        if rows > self.max_rows:
            raise Error(f"SlicedMultiLinear: {rows} rows exceed max_rows = {self.max_rows}")
        if self.multi is not None and rows <= self.MULTI_ROWS:
            t, c, suh, ah, svh, sizes, n = self.multi
            kernels.exl3_linear_multi(a, t, c, suh, ah, svh, sizes, n, rows, self.size_k, self.k_bits, self.codebook, self.out,
                                      gpu.stream)
            return self.outputs
        kernels.ops.exl3_mgemm(a, self.b_list, self.carrier, self.suh_list, self.a_had, self.svh_list, rows, self.size_k, self.width,
                               self.k_bits, self.codebook, self.out, 1, self.slices, self.size_n_list, self.c_ptrs,
                               self.n_stride_list, self.had_src_list, len(self.sources), gpu.stream)
        return self.outputs


class StackedLinear:
    """Equally shaped MUL1 linears that share one input (gate and up of an MLP), stored one behind the other so that
    one decode launch (``kernels.exl3_linear_stack``) runs all of them on up to eight rows.  Construction moves the
    sources' tensors into the stack and re-points the sources at their slices, so no weight is held twice."""

    MAX_ROWS = 8        # what the library's stacked launch accepts
    BEST_ROWS = 4       # up to here it is measured faster than one launch per matrix (above, the limb tiles of the rows cost more)

    def __init__(self, gpu: Gpu, sources: list, max_rows: int = 1):
        first = sources[0]
        for s in sources:
            if (s.size_k, s.size_n, s.k_bits, s.codebook) != (first.size_k, first.size_n, first.k_bits, first.codebook):
                raise Error("StackedLinear: sources must share shape, k_bits and codebook")
        if first.codebook != Codebook.Mul1:
            raise Error("StackedLinear: the stacked launch exists for the MUL1 codebook only")
        self.sources = sources
        self.size_k, self.size_n, self.k_bits, self.codebook = first.size_k, first.size_n, first.k_bits, first.codebook
        self.trellis = torch.stack([s.trellis for s in sources]).contiguous()
        self.suh = torch.stack([s.suh for s in sources]).contiguous()
        self.svh = torch.stack([s.svh for s in sources]).contiguous()
        for i, s in enumerate(sources):
            s.trellis, s.suh, s.svh = self.trellis[i], self.suh[i], self.svh[i]
        self.a_had = torch.zeros(len(sources) * max_rows * self.size_k, dtype=torch.float16, device=gpu.device)

    def forward_n(self, gpu: Gpu, rows: int, a: torch.Tensor, c: torch.Tensor, out: OutDtype) -> None:
        """``c`` is ``[len(sources)][rows][size_n]`` of ``out``."""
        if rows > self.MAX_ROWS:
            raise Error(f"StackedLinear: {rows} rows exceed {self.MAX_ROWS}")
        n = len(self.sources)
        out_bytes = 2 if out == OutDtype.F16 else 4
        if a.numel() * a.element_size() < rows * self.size_k * 2 or c.numel() * c.element_size() < n * rows * self.size_n * out_bytes:
            raise Error("StackedLinear: buffer too small")
        if self.a_had.numel() < n * rows * self.size_k:
            self.a_had = torch.zeros(n * rows * self.size_k, dtype=torch.float16, device=gpu.device)
        kernels.exl3_linear_stack(a, self.trellis, c, self.suh, self.a_had, self.svh, n, rows, self.size_k, self.size_n,
                                  self.k_bits, self.codebook, out, gpu.raw_stream())


class RowScratch:
    """Scratch shared by every linear of a prefill chunk.  ``weight`` is kept because the
    boundary requires a non-null pointer above 144 rows; the B200 kernels never write it, so it
    is a token allocation rather than size_k * min(size_n, 32768) halves."""

    def __init__(self, gpu: Gpu, max_rows: int, max_k: int, max_n: int):
        self.a_had = torch.zeros(max_rows * max_k, dtype=torch.float16, device=gpu.device)
        self.weight = torch.zeros(16, dtype=torch.float16, device=gpu.device)
        self.max_rows, self.max_k, self.max_n = max_rows, max_k, max_n


class MlpLayer:
    """``output = down(silu(gate(input)) * up(input))``; gate/up fp16 out, down fp32 out."""

    # up to here the down projection takes silu(gate) * up inside its own rotation (one launch and one buffer less; the
    # decode kernel serves these row counts anyway); above, the element-wise kernel runs and the dispatcher chooses
    FUSED_ACT_ROWS = 16

    def __init__(self, gpu: Gpu, gate: Exl3Linear, up: Exl3Linear, down: Exl3Linear, max_rows: int = 1):
        if gate.size_k != up.size_k or gate.size_n != up.size_n:
            raise Error(f"gate is {gate.size_k}x{gate.size_n}, up is {up.size_k}x{up.size_n}")
        if down.size_k != gate.size_n or down.size_n != gate.size_k:
            raise Error(f"down is {down.size_k}x{down.size_n}, gate is {gate.size_k}x{gate.size_n}")
        self.gate, self.up, self.down = gate, up, down
        self.hidden, self.intermediate = gate.size_k, gate.size_n
        if self.intermediate < 2 or self.intermediate % 2:
            raise Error(f"intermediate {self.intermediate} must be positive and even")
        # gate and up as one decode launch where the library has one and it pays (MUL1, same bitrate, up to four rows)
        self.gate_up = None
        if gate.codebook == Codebook.Mul1 and up.codebook == Codebook.Mul1 and gate.k_bits == up.k_bits:
            self.gate_up = StackedLinear(gpu, [gate, up], max_rows)
        self._alloc(gpu, max_rows)

    def _alloc(self, gpu: Gpu, rows: int) -> None:
        n = rows * self.intermediate
        self.max_rows = rows
        self.gate_up_out = torch.zeros(2 * n, dtype=torch.float16, device=gpu.device)   # gate rows, then up rows
        self.gate_out, self.up_out = self.gate_up_out[:n], self.gate_up_out[n:]
        self.activated = torch.zeros(n, dtype=torch.float16, device=gpu.device)

    @classmethod
    def load_prefixed(cls, gpu: Gpu, tensors: dict, prefix: str, k_bits: int, codebook: Codebook) -> "MlpLayer":
        parts = [Exl3Linear.load(gpu, tensors, f"{prefix}.{p}", k_bits, codebook)
                 for p in ("gate_proj", "up_proj", "down_proj")]
        return cls(gpu, *parts)

    def compressed_bytes(self) -> int:
        return self.gate.compressed_bytes() + self.up.compressed_bytes() + self.down.compressed_bytes()

    def forward(self, gpu: Gpu, inp: torch.Tensor, output: torch.Tensor) -> None:
        self.forward_n(gpu, 1, inp, output)

    def forward_n(self, gpu: Gpu, rows: int, inp: torch.Tensor, output: torch.Tensor) -> None:
        """inp fp16 [rows][hidden]; output fp32 [rows][hidden]."""
        if inp.numel() * inp.element_size() < rows * self.hidden * 2 or \
                output.numel() * output.element_size() < rows * self.hidden * 4:
            raise Error(f"{self.gate.prefix}: buffer too small")
        if rows > self.max_rows:
            self._alloc(gpu, rows)
        n = rows * self.intermediate
        if self.gate_up is not None and rows <= StackedLinear.BEST_ROWS:
            gate_out, up_out = self.gate_up_out[:n], self.gate_up_out[n:2 * n]
            self.gate_up.forward_n(gpu, rows, inp, self.gate_up_out, OutDtype.F16)
        else:
            gate_out, up_out = self.gate_out, self.up_out
            self.gate.forward_n(gpu, rows, inp, gate_out, OutDtype.F16)
            self.up.forward_n(gpu, rows, inp, up_out, OutDtype.F16)
        self._last = (gate_out, up_out, n)
        if rows <= self.FUSED_ACT_ROWS:
            self.down.forward_silu_n(gpu, rows, gate_out, up_out, output, OutDtype.F32, ACT_LIMIT)
        else:
            kernels.ops.silu_mul(gate_out, up_out, self.activated, n, ACT_LIMIT, gpu.raw_stream())
            self.down.forward_n(gpu, rows, self.activated, output, OutDtype.F32)

    def activation(self, gpu: Gpu) -> torch.Tensor:
        """``silu(gate) * up`` of the last ``forward_n`` as fp16 ``[rows * intermediate]``.  Up to ``FUSED_ACT_ROWS`` rows
        the down projection forms it on the fly and nothing holds it; this writes it out (the element-wise kernel on the
        gate and up outputs, the same bits) for a caller that wants to look at it."""
        gate_out, up_out, n = self._last
        kernels.ops.silu_mul(gate_out, up_out, self.activated, n, ACT_LIMIT, gpu.raw_stream())
        return self.activated[:n]

    def prefill(self, gpu: Gpu, rows: int, inp: torch.Tensor, output: torch.Tensor, scratch: RowScratch) -> None:
        """crates/berth-engine/src/mlp.rs:219-305."""
        if rows > self.max_rows:
            self._alloc(gpu, rows)
        self.gate.forward_rows(gpu, rows, inp, self.gate_out, OutDtype.F16, scratch)
        self.up.forward_rows(gpu, rows, inp, self.up_out, OutDtype.F16, scratch)
        kernels.ops.silu_mul(self.gate_out, self.up_out, self.activated, rows * self.intermediate, ACT_LIMIT,
                             gpu.raw_stream())
        self.down.forward_rows(gpu, rows, self.activated, output, OutDtype.F32, scratch)
