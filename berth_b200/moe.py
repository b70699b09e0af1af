"""Host side of the A3B-style mixture-of-experts layer.

berth has only the shape contract of this block (``MoeDims`` / ``Ffn::Moe`` in
crates/berth-plan/src/shape.rs:59-69 and plan.rs:43-57); ``MoeLayer`` is the caller an engine
would put next to ``MlpLayer``.  Weights live on the device as expert stacks; every computation
is a call into ``libberth_b200.so``; the workspace is allocated once by the caller (torch owns
the memory) and handed to the library, which allocates nothing per layer.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _lib
from .kernels import Error, _s

_PTR_FIELDS = [n for n, _ in _lib.MoeWeights._fields_[7:]]


def last_error() -> str:
    return _s(_lib.lib().berth_moe_last_error())


def last_launch() -> str:
    return _s(_lib.lib().berth_moe_last_launch())


def router_topk(x, w_router, router_bias, topk_idx, topk_w, logits, T, hidden, n_experts, top_k, stream=None) -> None:
    p = lambda t: None if t is None else t.data_ptr()
    rc = _lib.lib().berth_moe_router_topk(p(x), p(w_router), p(router_bias), p(topk_idx), p(topk_w), p(logits), T, hidden,
                                          n_experts, top_k, None if stream is None else stream.cuda_stream)
    if rc != 0:
        raise Error(last_error() or f"moe router launch failed ({rc})")


class MoeLayer:
    """One MoE layer resident on a GPU.  ``weights`` is the dict of ``berth_b200.synth.moe_layer_weights``
    (or the same keys filled from a checkpoint): numpy arrays are uploaded, torch tensors are kept."""

    def __init__(self, device: torch.device, weights: dict, max_tokens: int):
        self.device = device
        self.dims = {k: int(weights[k]) for k in ("hidden", "inter", "shared_inter", "n_experts", "top_k", "bits", "cb")}
        self._keep = {}
        self.c = _lib.MoeWeights()
        self.c.hidden, self.c.inter, self.c.shared_inter = self.dims["hidden"], self.dims["inter"], self.dims["shared_inter"]
        self.c.n_experts, self.c.top_k = self.dims["n_experts"], self.dims["top_k"]
        self.c.k_bits, self.c.codebook = self.dims["bits"], self.dims["cb"]
        for name in _PTR_FIELDS:
            v = weights.get(name)
            if v is None:
                setattr(self.c, name, None)
                continue
            if not isinstance(v, torch.Tensor):
                a = np.ascontiguousarray(v)
                if a.dtype == np.uint16:
                    a = a.view(np.int16)
                v = torch.from_numpy(a).to(device)
            self._keep[name] = v
            setattr(self.c, name, v.data_ptr())
        self.max_tokens = 0
        self._alloc(max_tokens)

    def _alloc(self, T: int) -> None:
        d = self.dims
        need = _lib.lib().berth_moe_workspace_bytes(T, d["hidden"], d["inter"], d["shared_inter"], d["n_experts"], d["top_k"])
        self.workspace = torch.empty(need, dtype=torch.uint8, device=self.device)
        self.max_tokens = T

    def expert_bytes(self) -> int:
        return sum(self._keep[n].numel() * 2 for n in ("gate_trellis", "up_trellis", "down_trellis"))

    def forward(self, x: torch.Tensor, out: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor, stream=None) -> None:
        """x fp16 [T][hidden] -> out fp32 [T][hidden]; topk_idx int32 [T][k], topk_w fp32 [T][k] receive the routing."""
        T = x.shape[0]
        if T > self.max_tokens:
            self._alloc(T)
        rc = _lib.lib().berth_moe_layer(C.byref(self.c), x.data_ptr(), T, out.data_ptr(), topk_idx.data_ptr(),
                                        topk_w.data_ptr(), self.workspace.data_ptr(), self.workspace.numel(),
                                        None if stream is None else stream.cuda_stream)
        if rc != 0:
            raise Error(last_error() or f"moe layer launch failed ({rc})")
