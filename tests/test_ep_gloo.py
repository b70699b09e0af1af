"""Expert-parallel exchange logic on CPU: two gloo ranks, the compute stages replaced by the CPU
oracle, result compared with the single-process layer on all tokens."""
import os
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist            # noqa: E402
import torch.multiprocessing as mp          # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class OracleStages:
    """route / sort / gather / experts / shared_expert / combine with numpy + the CPU oracle."""

    def __init__(self, wts, e0, n_local, orc):
        self.w, self.e0, self.n_local, self.orc = wts, e0, n_local, orc

    def route(self, x):
        logits = self.orc.router_logits(x.numpy(), self.w["w_router"], self.w.get("router_bias"))
        idx, w = self.orc.router_topk(logits, self.w["top_k"])
        return torch.from_numpy(idx), torch.from_numpy(w)

    def sort(self, keys, e0, n_local, for_experts=False):
        k = keys.numpy()
        perm = np.argsort(k, kind="stable").astype(np.int32)
        inv = np.empty_like(perm)
        inv[perm] = np.arange(perm.size, dtype=np.int32)
        counts = np.bincount(k - e0, minlength=n_local)[:n_local]
        offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
        return torch.from_numpy(perm), torch.from_numpy(inv), torch.from_numpy(offsets)

    def gather(self, src, index, div):
        return src[(index.long() // div)].contiguous()

    def _expert(self, x, pre, e=None):
        o, w = self.orc, self.w
        sel = (lambda a: a[e]) if e is not None else (lambda a: a)
        H, I = w["hidden"], (w["inter"] if e is not None else w["shared_inter"])
        g, _ = o.linear(x, sel(w[f"{pre}gate_trellis"]), sel(w[f"{pre}gate_suh"]), sel(w[f"{pre}gate_svh"]), H, I, w["bits"], w["cb"], False)
        u, _ = o.linear(x, sel(w[f"{pre}up_trellis"]), sel(w[f"{pre}up_suh"]), sel(w[f"{pre}up_svh"]), H, I, w["bits"], w["cb"], False)
        h = o.silu_mul(g, u)
        y, _ = o.linear(h, sel(w[f"{pre}down_trellis"]), sel(w[f"{pre}down_suh"]), sel(w[f"{pre}down_svh"]), I, H, w["bits"], w["cb"], False)
        return y

    def experts(self, xr):
        # rows arrive grouped by local expert; the keys are recovered from the last sort
        out = np.empty(xr.shape, np.float16)
        for j in range(self.n_local):
            lo, hi = self._last_offsets[j], self._last_offsets[j + 1]
            if hi > lo:
                out[lo:hi] = self._expert(xr.numpy()[lo:hi], "", j)
        return torch.from_numpy(out)

    def shared_expert(self, x):
        if not self.w["shared_inter"]:
            return None
        return torch.from_numpy(self._expert(x.numpy(), "sh_"))

    def combine(self, y, inv, w, ysh):
        T, k = w.shape
        yy = y.numpy().astype(np.float64)[inv.numpy().reshape(T, k)]
        out = (w.numpy().astype(np.float64)[:, :, None] * yy).sum(axis=1)
        if ysh is not None:
            out = out + ysh.numpy().astype(np.float64)
        return torch.from_numpy(out.astype(np.float32))


def _worker(rank, world, port, tmp):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from berth_b200 import moe, synth
    from oracle import exl3_oracle as orc
    orc.set_num_threads(2)
    H, I, E, k, bits, cb, T = 128, 128, 8, 2, 4, 2, 6
    full = synth.moe_layer_weights(77, "ep", H, I, E, k, bits, cb, shared_inter=128)
    n_local = E // world
    local = dict(full)
    for name in ("gate", "up", "down"):
        for part in ("trellis", "suh", "svh"):
            local[f"{name}_{part}"] = full[f"{name}_{part}"][rank * n_local:(rank + 1) * n_local]
    local["n_experts"] = n_local
    stages = OracleStages(local, rank * n_local, n_local, orc)
    orig_sort = stages.sort

    def sort(keys, e0, nl, for_experts=False):
        perm, inv, off = orig_sort(keys, e0, nl)
        if for_experts:
            stages._last_offsets = off.numpy()
        return perm, inv, off
    stages.sort = sort
    layer = moe.EpMoeLayer(stages, dist.group.WORLD, E, k)
    x_all = synth.activations(77, "ep.x", T * world, H)
    x = torch.from_numpy(x_all[rank * T:(rank + 1) * T].copy())
    out, idx, w = layer.forward(x)
    np.save(os.path.join(tmp, f"out{rank}.npy"), out.numpy())
    np.save(os.path.join(tmp, f"idx{rank}.npy"), idx.numpy())
    assert layer.last_stats["sent_rows"] == T * k
    total = torch.tensor([layer.last_stats["recv_rows"]])
    dist.all_reduce(total)
    assert int(total) == T * k * world          # every routed row arrived somewhere exactly once
    dist.destroy_process_group()


def test_ep_two_ranks_match_single_process(oracle, tmp_path):
    world, port = 2, 29517 + (os.getpid() % 200)
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    from berth_b200 import synth
    H, I, E, k, bits, cb, T = 128, 128, 8, 2, 4, 2, 6
    full = synth.moe_layer_weights(77, "ep", H, I, E, k, bits, cb, shared_inter=128)
    x_all = synth.activations(77, "ep.x", T * world, H)
    exp_out, exp_idx, _ = oracle.moe_layer(full, x_all)
    got = np.concatenate([np.load(tmp_path / f"out{r}.npy") for r in range(world)])
    idx = np.concatenate([np.load(tmp_path / f"idx{r}.npy") for r in range(world)])
    assert (idx == exp_idx).all()
    assert np.abs(got - exp_out).max() <= 1e-5 * np.abs(exp_out).max()
