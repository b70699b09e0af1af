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


def _cur_stream(device) -> int:
    """Raw handle of torch's current stream on `device`: the stream the layers' tensors are ordered on."""
    return torch.cuda.current_stream(device).cuda_stream


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

    def __init__(self, device: torch.device, weights: dict, max_tokens: int, fuse_shared: bool = True, pair_gate_up: bool = True):
        self.device = device
        self.dims = {k: int(weights[k]) for k in ("hidden", "inter", "shared_inter", "n_experts", "top_k", "bits", "cb")}
        self._keep = {}
        self.c = _lib.MoeWeights()
        self.c.hidden, self.c.inter, self.c.shared_inter = self.dims["hidden"], self.dims["inter"], self.dims["shared_inter"]
        self.c.n_experts, self.c.top_k = self.dims["n_experts"], self.dims["top_k"]
        self.c.k_bits, self.c.codebook = self.dims["bits"], self.dims["cb"]
        def on_device(v):
            if isinstance(v, torch.Tensor):
                return v.to(device)
            a = np.ascontiguousarray(v)
            if a.dtype == np.uint16:
                a = a.view(np.int16)
            return torch.from_numpy(a).to(device)

        # A shared expert of the experts' shape is stored as matrix n_experts of every stack: the library then
        # runs it inside the grouped expert launches instead of three launches of its own.
        stacked = set()
        if self.dims["shared_inter"] == self.dims["inter"] and fuse_shared and \
                all(weights.get(f"sh_{p}_{k}") is not None for p in ("gate", "up", "down") for k in ("trellis", "suh", "svh")):
            E = self.dims["n_experts"]
            for p in ("gate", "up", "down"):
                for k in ("trellis", "suh", "svh"):
                    both = torch.cat((on_device(weights[f"{p}_{k}"]), on_device(weights[f"sh_{p}_{k}"]).unsqueeze(0)))
                    self._keep[f"{p}_{k}"] = both
                    self._keep[f"sh_{p}_{k}"] = both[E]
                    setattr(self.c, f"{p}_{k}", both.data_ptr())
                    setattr(self.c, f"sh_{p}_{k}", both[E].data_ptr())
                    stacked.update((f"{p}_{k}", f"sh_{p}_{k}"))
        for name in _PTR_FIELDS:
            if name in stacked:
                continue
            v = weights.get(name)
            if v is None:
                setattr(self.c, name, None)
                continue
            v = on_device(v)
            self._keep[name] = v
            setattr(self.c, name, v.data_ptr())
        # The up stack directly behind the gate stack (trellis and output scales): the library then runs both
        # projections as one grouped launch over a doubled problem table.
        if pair_gate_up:
            for k in ("trellis", "svh"):
                g, u = self._keep.get(f"gate_{k}"), self._keep.get(f"up_{k}")
                if g is None or u is None or g.shape != u.shape or g.dtype != u.dtype:
                    continue
                n = g.shape[0]
                pair = torch.cat((g, u))
                for p, part in (("gate", pair[:n]), ("up", pair[n:])):
                    self._keep[f"{p}_{k}"] = part
                    setattr(self.c, f"{p}_{k}", part.data_ptr())
                    if f"sh_{p}_{k}" in stacked:
                        self._keep[f"sh_{p}_{k}"] = part[n - 1]
                        setattr(self.c, f"sh_{p}_{k}", part[n - 1].data_ptr())
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


# ---------------------------------------------------------------------------------------------
# Expert parallelism.  berth runs on one GPU (crates/berth-cuda/src/context.rs:46-49); sharding the
# experts of the MoE layer over the GPUs of one NVSwitch box is new here.  Tokens stay
# data-parallel (each rank routes its own tokens), experts are split in contiguous blocks,
# and the only exchange steps are two all-to-alls: routed rows out, expert outputs back.

SHORT_K = 2048


def cap_rows_hint(hint: int, hidden: int, inter: int) -> int:
    """With short inner dimensions the expert stage keeps 128-row problems however many rows an expert has (the library's
    own layer does the same): a 128-row item's epilogue runs under the next item's main loop, a taller item's does not."""
    return 128 if hint > 128 and min(hidden, inter) <= SHORT_K else hint


class GpuStages:
    """The compute stages of the layer on one GPU, through the C ABI.  ``weights`` holds this
    rank's expert stacks (``n_experts`` = number of LOCAL experts), the full router and the shared
    expert."""

    def __init__(self, device: torch.device, weights: dict, n_experts_total: int, max_rows: int, max_rows_per_expert: int):
        self.device = device
        self.layer = MoeLayer.__new__(MoeLayer)
        MoeLayer.__init__(self.layer, device, weights, 1)
        self.d = self.layer.dims
        self.E = n_experts_total
        self.max_rows, self.mrpe = max_rows, max_rows_per_expert
        self.force_hint = None    # tests: a fixed rows-per-expert figure (problem height) instead of the derived one
        l = _lib.lib()
        # one scratch for the send-side sort over all experts, one for the local experts; the expert stage picks
        # its row chunk per call (see rows_hint), so the scratch is sized for the largest of the possible plans
        hints = [h for h in (8, 16, 32, 128, 256, 384, 512) if h <= max(8, max_rows_per_expert)] + [max_rows_per_expert]
        size = lambda n_exp: max(l.berth_moe_experts_workspace_bytes(max_rows, n_exp, self.d["hidden"], self.d["inter"], h) for h in hints)
        self.ews_all = torch.empty(size(self.E), dtype=torch.uint8, device=device)
        self.ews_loc = torch.empty(size(self.d["n_experts"]), dtype=torch.uint8, device=device)
        from .engine import Exl3Linear, Gpu
        self.shared = None
        if self.d["shared_inter"]:
            from .kernels import Codebook
            g = Gpu(device.index if device.index is not None else torch.cuda.current_device())
            k = self.layer._keep
            mk = lambda p: Exl3Linear(g, f"shared_expert.{p}_proj", k[f"sh_{p}_trellis"], k[f"sh_{p}_suh"], k[f"sh_{p}_svh"],
                                      self.d["bits"], Codebook(self.d["cb"]))
            self.shared = (g, mk("gate"), mk("up"), mk("down"))

    def _check(self, rc):
        if rc != 0:
            raise Error(last_error() or f"moe stage failed ({rc})")

    def route(self, x):
        T, H = x.shape
        k = self.d["top_k"]
        idx = torch.empty((T, k), dtype=torch.int32, device=self.device)
        w = torch.empty((T, k), dtype=torch.float32, device=self.device)
        logits = torch.empty((T, self.E), dtype=torch.float32, device=self.device)
        router_topk(x, self.layer._keep["w_router"], self.layer._keep.get("router_bias"), idx, w, logits, T, H, self.E, k)
        return idx, w

    def rows_hint(self, n_rows: int, n_local: int) -> int:
        """Rows-per-expert figure the expert stage sizes its problems for: twice the mean, at least 1, at most
        the construction-time bound.  sort(for_experts=True) and experts() of one layer call must agree on it,
        which they do because both see the same row count."""
        if self.force_hint is not None:
            return self.force_hint
        return cap_rows_hint(max(1, min(self.mrpe, -(-2 * n_rows // max(n_local, 1)))), self.d["hidden"], self.d["inter"])

    def sort(self, keys, e0: int, n_local: int, for_experts: bool = False):
        """Stable sort by expert.  for_experts=True also leaves the problem table of the following
        experts() call in the local-expert scratch (n_local must then be this rank's expert count)."""
        n = keys.numel()
        perm = torch.empty(max(n, 1), dtype=torch.int32, device=self.device)
        inv = torch.empty(max(n, 1), dtype=torch.int32, device=self.device)
        offsets = torch.empty(n_local + 1, dtype=torch.int32, device=self.device)
        ews = self.ews_loc if for_experts else self.ews_all
        if n == 0:   # an empty torch tensor has a null data pointer
            keys = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._check(_lib.lib().berth_moe_sort_rows(keys.data_ptr(), n, e0, n_local, perm.data_ptr(), inv.data_ptr(), offsets.data_ptr(),
                                                   ews.data_ptr(), ews.numel(), self.max_rows, self.d["hidden"], self.d["inter"],
                                                   self.rows_hint(n, n_local), _cur_stream(self.device)))
        return perm[:n], inv[:n], offsets

    def gather(self, src, index, div: int):
        n, H = index.numel(), src.shape[1]
        dst = torch.empty((n, H), dtype=torch.float16, device=self.device)
        if n:
            self._check(_lib.lib().berth_moe_gather(src.data_ptr(), index.data_ptr(), div, n, dst.data_ptr(), H, _cur_stream(self.device)))
        return dst

    def experts(self, xr):
        R = xr.shape[0]
        yr = torch.empty_like(xr)
        if R == 0:     # a rank that received no rows (few tokens, many ranks): nothing to launch
            return yr
        self._check(_lib.lib().berth_moe_experts(C.byref(self.layer.c), xr.data_ptr(), yr.data_ptr(), R, self.ews_loc.data_ptr(),
                                                 self.ews_loc.numel(), self.max_rows, self.rows_hint(R, self.d["n_experts"]), _cur_stream(self.device)))
        return yr

    def shared_expert(self, x, stream=None):
        """Shared expert of x on the current stream, or on `stream` (only for more than 32 rows: the decode
        kernels share one per-device scratch, so they must stay on one stream; the prefill kernels do not)."""
        if self.shared is None:
            return None
        from .kernels import OutDtype, ops
        g, gate, up, down = self.shared
        T = x.shape[0]
        if stream is not None:
            if T <= 32:
                raise Error("shared expert: the decode kernels must stay on the layer's stream")
            if getattr(self, "_side_gpu", None) is None or self._side_gpu.stream is not stream:
                from .engine import Gpu
                self._side_gpu = Gpu(g.device.index if hasattr(g.device, "index") else g.device, stream=stream)
            g = self._side_gpu
        si, H = self.d["shared_inter"], self.d["hidden"]
        a = torch.empty((T, si), dtype=torch.float16, device=self.device)
        b = torch.empty((T, si), dtype=torch.float16, device=self.device)
        y = torch.empty((T, H), dtype=torch.float16, device=self.device)
        fwd = (lambda lin, i, o: lin.forward_n(g, T, i, o, OutDtype.F16)) if T <= 32 else None
        if fwd is None:
            from .engine import RowScratch
            sc = RowScratch(g, T, max(H, si), max(H, si))
            fwd = lambda lin, i, o: lin.forward_rows(g, T, i, o, OutDtype.F16, sc)
        fwd(gate, x, a)
        fwd(up, x, b)
        ops.silu_mul(a, b, a, T * si, 0.0, g.stream)
        fwd(down, a, y)
        return y

    # ---- one library call per side of the exchange
    def ep_send(self, x, max_tokens: int):
        """Route, sort and gather the local tokens: (topk_idx, topk_w, inv, send_rows, counts per expert)."""
        l = _lib.lib()
        T, H = x.shape
        k, E = self.d["top_k"], self.E
        if getattr(self, "_send_ws", None) is None or self._send_cap < T:
            self._send_cap = max(T, max_tokens)
            self._send_ws = torch.empty(l.berth_moe_ep_send_workspace_bytes(self._send_cap, E, k), dtype=torch.uint8, device=self.device)
        idx = torch.empty((T, k), dtype=torch.int32, device=self.device)
        w = torch.empty((T, k), dtype=torch.float32, device=self.device)
        inv = torch.empty(T * k, dtype=torch.int32, device=self.device)
        rows = torch.empty((T * k, H), dtype=torch.float16, device=self.device)
        counts = torch.empty(E, dtype=torch.int32, device=self.device)
        kp = self.layer._keep
        bias = kp.get("router_bias")
        self._check(l.berth_moe_ep_send(x.data_ptr(), T, kp["w_router"].data_ptr(), None if bias is None else bias.data_ptr(), H, E, k,
                                        idx.data_ptr(), w.data_ptr(), inv.data_ptr(), rows.data_ptr(), counts.data_ptr(),
                                        self._send_ws.data_ptr(), self._send_ws.numel(), _cur_stream(self.device)))
        return idx, w, inv, rows, counts

    def shared_is_stacked(self) -> bool:
        """True if the shared expert sits behind the local expert stacks (MoeLayer puts it there when it has the
        experts' shape), so that ep_experts can run it inside the grouped launches."""
        d, kp = self.d, self.layer._keep
        return bool(d["shared_inter"]) and d["shared_inter"] == d["inter"] and "sh_gate_trellis" in kp and \
            kp["sh_gate_trellis"].data_ptr() == kp["gate_trellis"].data_ptr() + d["n_experts"] * kp["gate_trellis"][0].numel() * 2

    def ep_experts(self, recv_rows, cnt_recv, world: int, x_local, max_tokens: int):
        """Received rows -> expert outputs in arrival order (+ the shared expert's output for the local tokens
        when it is stacked behind the experts)."""
        l = _lib.lib()
        R, H = recv_rows.shape
        T = x_local.shape[0]
        nl = self.d["n_experts"]
        if getattr(self, "_exp_ws", None) is None or self._exp_tokens < T:
            self._exp_tokens = max(T, max_tokens)
            self._exp_ws = torch.empty(l.berth_moe_ep_experts_workspace_bytes(self.max_rows, self._exp_tokens, world, nl, H, self.d["inter"]),
                                       dtype=torch.uint8, device=self.device)
        back = torch.empty((R, H), dtype=torch.float16, device=self.device)
        stacked = self.shared_is_stacked() and T > 0
        ysh = torch.empty((T, H), dtype=torch.float16, device=self.device) if stacked else None
        self._check(l.berth_moe_ep_experts(C.byref(self.layer.c), recv_rows.data_ptr() if R else None, R, cnt_recv.data_ptr(), world,
                                           x_local.data_ptr() if T else None, T, back.data_ptr() if R else None,
                                           None if ysh is None else ysh.data_ptr(), self._exp_ws.data_ptr(), self._exp_ws.numel(),
                                           self.max_rows, self._exp_tokens, self.rows_hint(R, nl), _cur_stream(self.device)))
        return back, ysh

    def combine(self, y, inv, w, ysh):
        T, k = w.shape
        H = y.shape[1]
        out = torch.empty((T, H), dtype=torch.float32, device=self.device)
        self._check(_lib.lib().berth_moe_combine(y.data_ptr(), inv.data_ptr(), w.data_ptr(), None if ysh is None else ysh.data_ptr(),
                                                 out.data_ptr(), T, H, k, _cur_stream(self.device)))
        return out


class EpMoeLayer:
    """Expert-parallel MoE layer over a ``torch.distributed`` group (NCCL on GPUs, gloo in the CPU
    tests).  ``stages`` provides route / sort / gather / experts / shared_expert / combine on this
    rank's device; this class owns only the exchange logic:

        route local tokens -> sort (token, slot) pairs by expert (= by destination rank, experts
        are split in contiguous blocks) -> all-to-all rows + expert ids -> regroup by local expert
        -> experts -> undo the regrouping -> all-to-all back -> weighted combine + shared expert.
    """

    def __init__(self, stages, group, n_experts: int, top_k: int):
        import torch.distributed as dist
        self.dist, self.group, self.stages = dist, group, stages
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if n_experts % self.world:
            raise Error(f"{n_experts} experts do not split evenly over {self.world} ranks")
        self.E, self.k = n_experts, top_k
        self.n_local = n_experts // self.world
        self.e0 = self.rank * self.n_local
        self.last_stats = {}

    def forward(self, x: torch.Tensor):
        """x fp16 [T_local][hidden] -> (out fp32 [T_local][hidden], topk_idx, topk_w).

        Exchange steps per layer: one all-to-all of per-expert row counts (fixed size, so it needs nothing
        from the host), ONE host read of the resulting send/receive sizes, one all-to-all of the routed rows
        and one of the expert outputs.  The expert id of every received row follows from the counts (a
        source sends its rows sorted by expert), so no key travels with the rows.  The shared expert runs on
        a side stream while the rows are away."""
        dist, st = self.dist, self.stages
        T, k, W, nl = x.shape[0], self.k, self.world, self.n_local
        dev = x.device
        if hasattr(st, "ep_send") and T:
            return self._forward_fused(x)
        if T:
            idx, w = st.route(x)
        else:   # a rank without tokens still takes part in the exchanges
            idx = torch.empty((0, k), dtype=torch.int32, device=dev)
            w = torch.empty((0, k), dtype=torch.float32, device=dev)
        keys = idx.reshape(-1)
        perm, inv, offsets = st.sort(keys, 0, self.E)                     # rows sorted by expert = by rank
        ysh = self._shared_async(x) if T else None
        send_rows = st.gather(x, perm, k)
        cnt_send = (offsets[1:] - offsets[:-1]).contiguous()             # rows per expert, [W * n_local]
        cnt_recv = torch.empty_like(cnt_send)                              # [source rank][local expert]
        dist.all_to_all_single(cnt_recv, cnt_send, group=self.group)
        sizes = torch.stack((cnt_send.view(W, nl).sum(1), cnt_recv.view(W, nl).sum(1))).to("cpu")   # the one host sync
        send_counts, recv_counts = sizes[0].tolist(), sizes[1].tolist()
        R = sum(recv_counts)
        recv_rows = torch.empty((R, x.shape[1]), dtype=x.dtype, device=dev)
        dist.all_to_all_single(recv_rows, send_rows, recv_counts, send_counts, group=self.group)
        # expert of every received row: source by source, experts ascending, cnt_recv[s][e] rows each
        local_ids = (torch.arange(nl, dtype=torch.int32, device=dev) + self.e0).repeat(W)
        recv_keys = torch.repeat_interleave(local_ids, cnt_recv.long(), output_size=R) if R else \
            torch.empty(0, dtype=torch.int32, device=dev)
        perm2, inv2, _ = st.sort(recv_keys, self.e0, nl, for_experts=True)   # regroup by local expert
        xr = st.gather(recv_rows, perm2, 1)
        yr = st.experts(xr)
        back = st.gather(yr, inv2, 1)                                      # expert outputs in arrival order
        y_sorted = torch.empty_like(send_rows)
        dist.all_to_all_single(y_sorted, back, send_counts, recv_counts, group=self.group)
        if T:
            if ysh is not None and not self._shared_inline:
                torch.cuda.current_stream(dev).wait_event(self._shared_done)
            out = st.combine(y_sorted, inv, w, ysh)
        else:
            out = torch.empty((0, x.shape[1]), dtype=torch.float32, device=dev)
        self.last_stats = {"sent_rows": T * k, "recv_rows": R, "send_counts": send_counts, "recv_counts": recv_counts}
        return out, idx, w

    def _forward_fused(self, x: torch.Tensor):
        """The same exchange with one library call on each side of it (GPU stages)."""
        dist, st = self.dist, self.stages
        T, k, W, nl = x.shape[0], self.k, self.world, self.n_local
        dev = x.device
        idx, w, inv, send_rows, cnt_send = st.ep_send(x, T)
        cnt_recv = torch.empty_like(cnt_send)                              # [source rank][local expert]
        dist.all_to_all_single(cnt_recv, cnt_send, group=self.group)
        sizes = torch.stack((cnt_send.view(W, nl).sum(1), cnt_recv.view(W, nl).sum(1))).to("cpu")   # the one host sync
        send_counts, recv_counts = sizes[0].tolist(), sizes[1].tolist()
        R = sum(recv_counts)
        recv_rows = torch.empty((R, x.shape[1]), dtype=x.dtype, device=dev)
        dist.all_to_all_single(recv_rows, send_rows, recv_counts, send_counts, group=self.group)
        back, ysh = st.ep_experts(recv_rows, cnt_recv, W, x, T)
        if ysh is None and getattr(st, "shared", None) is not None:
            ysh = st.shared_expert(x)
        y_sorted = torch.empty_like(send_rows)
        dist.all_to_all_single(y_sorted, back, send_counts, recv_counts, group=self.group)
        out = st.combine(y_sorted, inv, w, ysh)
        self.last_stats = {"sent_rows": T * k, "recv_rows": R, "send_counts": send_counts, "recv_counts": recv_counts}
        return out, idx, w

    def _shared_async(self, x):
        """Shared expert of the local tokens; on a CUDA device on a side stream, so that it overlaps the
        exchange and the routed experts (the caller waits for self._shared_done before the combine)."""
        st = self.stages
        if x.device.type != "cuda" or getattr(st, "shared", None) is None or x.shape[0] <= 32:
            self._shared_inline = True
            return st.shared_expert(x)
        self._shared_inline = False
        if not hasattr(self, "_side"):
            self._side = torch.cuda.Stream(device=x.device)
            self._shared_done = torch.cuda.Event()
        main = torch.cuda.current_stream(x.device)
        self._side.wait_stream(main)
        with torch.cuda.stream(self._side):
            ysh = st.shared_expert(x, stream=self._side)
            self._shared_done.record(self._side)
        x.record_stream(self._side)
        if ysh is not None:
            ysh.record_stream(main)
        return ysh


class P2pMoeLayer:
    """Expert-parallel MoE layer whose exchange is done by the kernels themselves over peer memory: routed
    rows are stored straight into the owning rank's buffer at their final, expert-sorted position, expert
    outputs straight back into the sender's buffer, with three flag barriers per layer.  No collective call
    and no host synchronisation inside a layer.  The symmetric buffers come from
    ``torch.distributed._symmetric_memory`` (one allocation per buffer, rendezvous over `group`); the ranks
    must share one NVSwitch box.  ``stages`` is this rank's ``GpuStages`` (local expert stacks)."""

    def __init__(self, stages: GpuStages, group, n_experts: int, top_k: int, max_tokens: int, max_rows: int):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        self.dist, self.group, self.stages = dist, group, stages
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > 8:
            raise Error("P2pMoeLayer: at most 8 ranks")
        if n_experts % self.world:
            raise Error(f"{n_experts} experts do not split evenly over {self.world} ranks")
        self.E, self.k, self.n_local = n_experts, top_k, n_experts // self.world
        self.max_tokens, self.max_rows, self.max_send = max_tokens, max_rows, max_tokens * top_k
        d, dev, l = stages.d, stages.device, _lib.lib()
        H = d["hidden"]
        gname = group.group_name if hasattr(group, "group_name") else group

        def symmetric(nbytes):
            t = symm_mem.empty(nbytes, dtype=torch.uint8, device=dev)
            t.zero_()
            h = symm_mem.rendezvous(t, gname)
            ptrs = (C.c_void_p * self.world)(*[int(p) for p in h.buffer_ptrs])
            return t, h, ptrs

        self._cnt, self._cnt_h, self.cnt_ptrs = symmetric(self.world * n_experts * 4)
        self._flags, self._flags_h, self.flag_ptrs = symmetric(3 * 8 * 4)
        self._recv, self._recv_h, self.recv_ptrs = symmetric(max_rows * H * 2)
        self._ret, self._ret_h, self.ret_ptrs = symmetric(max(self.max_send, 1) * H * 2)
        torch.cuda.synchronize(dev)
        dist.barrier(group)          # every rank's flags are zero before the first epoch
        self.epoch = 0
        self.send_ws = torch.empty(l.berth_moe_p2p_send_workspace_bytes(max(max_tokens, 1), n_experts, top_k, self.world), dtype=torch.uint8, device=dev)
        self.exp_ws = torch.empty(l.berth_moe_p2p_experts_workspace_bytes(max_rows, self.n_local, H, d["inter"]), dtype=torch.uint8, device=dev)
        self.ret_rows = self._ret.view(torch.float16).view(-1, H)
        self.last_stats = {}
        self.profile = False      # True: forward() records CUDA events between its phases (see phase_ms)
        self._ev = None

    def forward(self, x: torch.Tensor):
        """x fp16 [T_local][hidden] -> (out fp32 [T_local][hidden], topk_idx, topk_w).  Asynchronous on the
        current stream; all ranks must call it the same number of times."""
        st, l = self.stages, _lib.lib()
        T, H = x.shape
        if T > self.max_tokens:
            raise Error(f"P2pMoeLayer: {T} tokens exceed max_tokens = {self.max_tokens}")
        dev, k = x.device, self.k
        self.epoch += 1
        if self.profile:
            self._ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            self._ev[0].record()
        idx = torch.empty((T, k), dtype=torch.int32, device=dev)
        w = torch.empty((T, k), dtype=torch.float32, device=dev)
        inv = torch.empty(max(T * k, 1), dtype=torch.int32, device=dev)
        kp = st.layer._keep
        bias = kp.get("router_bias")
        p = lambda t: t.data_ptr() if t.numel() else None
        st._check(l.berth_moe_p2p_send(p(x), T, kp["w_router"].data_ptr(), None if bias is None else bias.data_ptr(), H, self.E, k,
                                       p(idx), p(w), inv.data_ptr(), self.rank, self.world, self.epoch, self.cnt_ptrs, self.flag_ptrs,
                                       self.recv_ptrs, self.max_rows, self.send_ws.data_ptr(), self.send_ws.numel(), _cur_stream(dev)))
        if self.profile:
            self._ev[1].record()
        stacked = st.shared_is_stacked() and T > 0
        ysh = torch.empty((T, H), dtype=torch.float16, device=dev) if stacked else None
        # rows per local expert to size the problems for: twice the mean if every rank holds as many tokens as this one
        hint = cap_rows_hint(max(1, min(1024, -(-2 * max(T, 1) * self.world * k // self.E))), H, st.d["inter"])
        st._check(l.berth_moe_p2p_experts(C.byref(st.layer.c), p(x), T, None if ysh is None else ysh.data_ptr(), self.rank, self.world,
                                          self.epoch, self.E, k, T, self.cnt_ptrs, self.flag_ptrs, self.recv_ptrs, self.ret_ptrs,
                                          self.max_rows, max(self.max_send, 1), hint, self.send_ws.data_ptr(), self.exp_ws.data_ptr(),
                                          self.exp_ws.numel(), _cur_stream(dev)))
        if self.profile:
            self._ev[2].record()
        if T == 0:
            if self.profile:
                self._ev[3].record()
            return torch.empty((0, H), dtype=torch.float32, device=dev), idx, w
        if ysh is None and getattr(st, "shared", None) is not None:
            ysh = st.shared_expert(x)
        out = st.combine(self.ret_rows[: T * k], inv[: T * k], w, ysh)
        if self.profile:
            self._ev[3].record()
        return out, idx, w

    def phase_ms(self) -> dict:
        """After a forward() with ``profile`` set and a synchronize: milliseconds of its three phases -- send (route,
        top-k, sort, publish counts, barrier, peer stores of the rows, barrier), experts (problem table, the three grouped
        projections, peer stores of the outputs, barrier) and combine."""
        e = self._ev
        return {"send": e[0].elapsed_time(e[1]), "experts": e[1].elapsed_time(e[2]), "combine": e[2].elapsed_time(e[3])}
