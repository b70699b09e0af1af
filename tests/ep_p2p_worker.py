"""Worker of the multi-GPU expert-parallel tests: one rank of a torchrun launch.  Builds this rank's expert block of
a small MoE layer and runs the rank's tokens through both expert-parallel layers -- the peer-memory exchange
(``P2pMoeLayer``) and the NCCL exchange (``EpMoeLayer``) -- for several token counts (including ranks without tokens)
with a uniform and with a strongly skewed router.  Every token of every rank is compared with the CPU checker's
whole-layer evaluation of the same token: routing bit-exact, outputs within the fp32-accumulation tolerance of the fp64
evaluation (both forms) and within 6e-3 of the RMS of the checker's own fp32 layer; the two layers agree with each other
to the same bound.  (They are not bit-identical in general: each sizes the row chunks of its expert launches from its own
estimate of the rows per expert, so the same rows can run through kernels with another summation order, and the experts'
outputs are rounded to fp16 before the combine -- one fp16 step of the largest expert output is a few thousandths of the
layer's RMS.)  Prints one
"EP-CASE ..." line per case and "P2P-OK <rank>" on success."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from berth_b200 import kernels, moe, synth   # noqa: E402
from oracle import exl3_oracle as orc   # noqa: E402  (the checker; this file is a test)
from tests.gpu_util import assert_close   # noqa: E402


def main() -> None:
    rank, local, world = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    orc.build()
    H, I, E, K, bits, cb = 256, 128, 32, 4, 4, 2
    n_local = E // world
    for skew in (False, True):
        bias = synth.zipf_router_bias(1234, "p2pw.bias", E, s=1.1, strength=1.0) if skew else None
        full = synth.moe_layer_weights(1234, "p2pw", H, I, E, K, bits, cb, shared_inter=I, router_bias=bias)
        w = dict(full, n_experts=n_local)
        lo, hi = rank * n_local, (rank + 1) * n_local
        for p in ("gate", "up", "down"):
            for k in ("trellis", "suh", "svh"):
                w[f"{p}_{k}"] = np.ascontiguousarray(full[f"{p}_{k}"][lo:hi])
        # a skewed router sends most rows to a few experts: size the buffers for every row landing on one rank
        stages = moe.GpuStages(dev, w, E, max_rows=64 * K * world + 64, max_rows_per_expert=256)
        ep = moe.EpMoeLayer(stages, dist.group.WORLD, E, K)
        p2p = moe.P2pMoeLayer(stages, dist.group.WORLD, E, K, max_tokens=64, max_rows=64 * K * world + 64)
        for T in (1, 5 * world, 64 * world):
            t_loc = T // world if T >= world else (1 if rank < T else 0)
            xh = synth.activations(1234, f"p2pw.x{T}.r{rank}", max(t_loc, 1), H)[:t_loc]
            x = torch.from_numpy(np.ascontiguousarray(synth.activations(1234, f"p2pw.x{T}.r{rank}", max(t_loc, 1), H))).to(dev)[:t_loc]
            o1, i1, w1 = ep.forward(x)
            for _ in range(2):
                o2, i2, w2 = p2p.forward(x)
            torch.cuda.synchronize()
            assert kernels.device_status(local) == 0
            assert bool((i1 == i2).all()) and bool((w1 == w2).all())
            worst = 0.0
            if t_loc:
                exp_out, exp_idx, exp_w = orc.moe_layer(full, np.ascontiguousarray(xh))
                y64 = orc.moe_layer_f64(full, np.ascontiguousarray(xh), exp_idx, exp_w)
                rms = float(np.sqrt((y64 ** 2).mean()))
                assert (i2.cpu().numpy() == exp_idx).all(), "routing differs from the checker"
                assert float(np.abs(w2.cpu().numpy() - exp_w).max()) <= 1e-6
                for name, o in (("nccl", o1), ("peer-memory", o2)):
                    got = o.cpu().numpy()
                    assert_close(got, y64, f"{name} T={T} rank {rank}")
                    d = float(np.abs(got - exp_out).max())
                    assert d <= 6e-3 * rms, (name, T, d / rms)
                    worst = max(worst, d / rms)
                diff = float((o1 - o2).abs().max())
                assert diff <= 6e-3 * rms, (T, diff / rms)
            counts = torch.bincount(i2.flatten().to(torch.int64), minlength=E) if t_loc else torch.zeros(E, dtype=torch.int64, device=dev)
            dist.all_reduce(counts)
            if rank == 0:
                c = counts.cpu().numpy()
                print(f"EP-CASE world={world} skew={int(skew)} tokens={T} busiest_expert_rows={int(c.max())} mean_rows={c.mean():.1f} "
                      f"rank0_worst_vs_checker={worst:.2e}rms status=0", flush=True)
        del ep, p2p, stages
    dist.barrier()
    print(f"P2P-OK {rank}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
