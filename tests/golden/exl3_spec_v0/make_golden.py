"""Generates the seeded golden vectors of this directory from the CPU checker (oracle/) and the seeded synthetic tensors
(berth_b200/synth.py, master seed 1234), in the style of berth's testdata/*/meta.json: small raw files plus SHA-256
digests of the large arrays.  They fix the checker's own results ("spec v0" of the trellis decode, the linear and the
router), so that a later change of the checker, of the generators or of the CUDA kernels shows against committed bytes.

    python tests/golden/exl3_spec_v0/make_golden.py          # rewrites the files beside this script

Contents (meta.json lists every file with its shape, dtype and digest):
  tiny.b{3,4,5}.cb{0,1,2}.head.bin   first 16 rows of the decoded fp16 weights [128][256] of a tiny matrix; the digest of
                                     the whole decoded matrix is in meta.json
  c0.y.bin                           the checker's fp32 output of configuration 0 (5120 x 6144, 4 bpw, MUL1, one row)
  c0.y64.bin                         the fp64 evaluation of the same row
  c0.tiles.bin                       64 sampled decoded 16x16 tiles (fp16) of that matrix; meta.json holds their (k-tile,
                                     n-tile) positions and the digest of the whole decoded matrix
  c3.topk.T{1,64,1024}.bin           router top-8 indices (int32 [T][8]) of configuration 3 (hidden 2048, 256 experts);
                                     digests of the logits and of the routing weights in meta.json
"""
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.abspath(os.path.join(HERE, "..", "..", "..")))

from berth_b200 import synth                    # noqa: E402
from oracle import exl3_oracle as oracle        # noqa: E402

SEED = 1234


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def tiny_cases():
    for bits in (3, 4, 5):
        for cb in (0, 1, 2):
            yield bits, cb, f"golden.tiny.b{bits}.cb{cb}"


def c0_tile_positions():
    """64 seeded (k-tile, n-tile) positions of the 320 x 384 tiles of configuration 0."""
    r = synth.raw_u64(SEED, "golden.c0.tiles", 128)
    return [(int(r[2 * i] % 320), int(r[2 * i + 1] % 384)) for i in range(64)]


def generate() -> dict:
    """name -> (array to store or None, meta entry)."""
    out = {}
    for bits, cb, name in tiny_cases():
        t = synth.trellis(SEED, name, 128, 256, bits)
        w = oracle.reconstruct(t, 128, 256, bits, cb).view(np.uint16).reshape(128, 256)
        out[f"tiny.b{bits}.cb{cb}.head.bin"] = (w[:16], {"dtype": "f16 bits", "shape": [16, 256], "bits": bits, "codebook": cb,
                                                         "tensor": name, "sha256_whole_decoded_matrix": sha(w)})
    K, N, bits, cb = 5120, 6144, 4, 2
    w = synth.linear_weights(SEED, "golden.c0", K, N, bits)
    x = synth.activations(SEED, "golden.c0.x", 1, K)
    y, a_had = oracle.linear(x, w["trellis"], w["suh"], w["svh"], K, N, bits, cb, True)
    y64 = oracle.linear_f64(x, w["trellis"], w["suh"], w["svh"], K, N, bits, cb)
    dec = oracle.reconstruct(w["trellis"], K, N, bits, cb).view(np.uint16).reshape(K, N)
    pos = c0_tile_positions()
    tiles = np.stack([dec[16 * kt:16 * kt + 16, 16 * nt:16 * nt + 16] for kt, nt in pos])
    c0 = {"size_k": K, "size_n": N, "bits": bits, "codebook": cb, "tensor": "golden.c0", "activations": "golden.c0.x"}
    out["c0.y.bin"] = (y.astype(np.float32), dict(c0, dtype="f32", shape=[1, N], sha256_rotated_activations=sha(a_had.view(np.uint16))))
    out["c0.y64.bin"] = (y64.astype(np.float64), dict(c0, dtype="f64", shape=[1, N]))
    out["c0.tiles.bin"] = (tiles, dict(c0, dtype="f16 bits", shape=[64, 16, 16], positions=pos, sha256_whole_decoded_matrix=sha(dec)))
    H, E, k = 2048, 256, 8
    wr = synth.router_weight(SEED, "golden.c3.gate.weight", H, E)
    for T in (1, 64, 1024):
        xt = synth.activations(SEED, f"golden.c3.x{T}", T, H)
        logits = oracle.router_logits(xt, wr)
        idx, tw = oracle.router_topk(logits, k)
        out[f"c3.topk.T{T}.bin"] = (idx.astype(np.int32), {"dtype": "i32", "shape": [T, k], "hidden": H, "n_experts": E, "top_k": k,
                                                           "router": "golden.c3.gate.weight", "activations": f"golden.c3.x{T}",
                                                           "sha256_logits_f32": sha(logits.astype(np.float32)),
                                                           "sha256_weights_f32": sha(tw.astype(np.float32))})
    return out


def main() -> None:
    files = generate()
    meta = {"seed": SEED, "generator": "tests/golden/exl3_spec_v0/make_golden.py", "spec": "v0 (oracle/exl3_oracle.c header)", "files": {}}
    for name, (arr, entry) in files.items():
        np.ascontiguousarray(arr).tofile(os.path.join(HERE, name))
        meta["files"][name] = dict(entry, bytes=int(np.ascontiguousarray(arr).nbytes), sha256=sha(arr))
    with open(os.path.join(HERE, "meta.json"), "w") as f:
        json.dump(meta, f, indent=1, sort_keys=True)
        f.write("\n")


if __name__ == "__main__":
    main()
