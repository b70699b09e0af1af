"""Worker of test_peer_memory_layer_matches_nccl_layer: one rank of a torchrun launch.  Builds this rank's expert
block of a small MoE layer and checks that the peer-memory layer and the NCCL layer give identical results
(same routing, same rows per expert in the same order, hence bit-identical outputs wherever both run the shared
expert through the same kernels) for several token counts, including a rank without tokens.  Prints "P2P-OK <rank>" on success."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from berth_b200 import kernels, moe, synth   # noqa: E402


def main() -> None:
    rank, local, world = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    H, I, E, K, bits, cb = 256, 128, 32, 4, 4, 2
    n_local = E // world
    full = synth.moe_layer_weights(1234, "p2pw", H, I, E, K, bits, cb, shared_inter=I)
    w = dict(full, n_experts=n_local)
    lo, hi = rank * n_local, (rank + 1) * n_local
    for p in ("gate", "up", "down"):
        for k in ("trellis", "suh", "svh"):
            w[f"{p}_{k}"] = np.ascontiguousarray(full[f"{p}_{k}"][lo:hi])
    stages = moe.GpuStages(dev, w, E, max_rows=64 * K * world, max_rows_per_expert=256)
    ep = moe.EpMoeLayer(stages, dist.group.WORLD, E, K)
    p2p = moe.P2pMoeLayer(stages, dist.group.WORLD, E, K, max_tokens=64, max_rows=64 * K * world + 64)
    for T in (1, 5 * world, 64 * world):
        t_loc = T // world if T >= world else (1 if rank < T else 0)
        x = torch.from_numpy(synth.activations(1234, f"p2pw.x{T}.r{rank}", max(t_loc, 1), H)).to(dev)[:t_loc]
        o1, i1, w1 = ep.forward(x)
        for _ in range(2):
            o2, i2, w2 = p2p.forward(x)
        torch.cuda.synchronize()
        assert kernels.device_status(local) == 0
        assert bool((i1 == i2).all()) and bool((w1 == w2).all())
        if t_loc:
            diff = float((o1 - o2).abs().max())
            if t_loc <= 32:
                assert diff == 0.0, (T, diff)
            else:
                # above 32 tokens the NCCL layer runs the shared expert through the prefill linear on a side stream, the
                # peer-memory layer inside the grouped decode launches: other summation order, fp32-accumulation tolerance
                assert diff <= 1e-2 * float(o1.abs().max()), (T, diff, float(o1.abs().max()))
    dist.barrier()
    print(f"P2P-OK {rank}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
