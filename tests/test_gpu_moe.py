"""MoE layer parity: router top-k indices bit-exact against the CPU oracle (ties to the lower
expert index), layer output within the fp32-accumulation tolerance of the fp64 evaluation."""
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from berth_b200 import kernels, moe, synth   # noqa: E402
from tests.gpu_util import MAX_REL, MEAN_REL, assert_close, dev, rel_errors   # noqa: E402


def _route(x, wr, bias, k):
    T, H = x.shape
    E = wr.shape[1]
    idx = torch.empty((T, k), dtype=torch.int32, device="cuda")
    w = torch.empty((T, k), dtype=torch.float32, device="cuda")
    logits = torch.empty((T, E), dtype=torch.float32, device="cuda")
    b = None if bias is None else torch.from_numpy(bias).cuda()
    moe.router_topk(dev(x), dev(wr), b, idx, w, logits, T, H, E, k)
    torch.cuda.synchronize()
    return idx.cpu().numpy(), w.cpu().numpy(), logits.cpu().numpy()


@pytest.mark.parametrize("T", [1, 64, 301, 1024])
def test_router_topk_config3_bit_exact(oracle, T):
    """1 and 64 tokens run the narrow logits kernel with one chunk per warp, 301 and 1024 the 128-expert-wide one
    (301: ragged last token tile)."""
    H, E, k = 2048, 256, 8
    x = synth.activations(1234, f"c3.x{T}", T, H)
    wr = synth.router_weight(1234, "c3.gate.weight", H, E)
    idx, w, logits = _route(x, wr, None, k)
    exp_logits = oracle.router_logits(x, wr)
    assert (logits.view(np.uint32) == exp_logits.view(np.uint32)).all()      # fixed summation order
    exp_idx, exp_w = oracle.router_topk(exp_logits, k)
    assert (idx == exp_idx).all()
    assert np.abs(w - exp_w).max() <= 1e-6
    assert np.allclose(w.sum(axis=1), 1.0, atol=1e-5)


def test_router_ties_and_bias(oracle):
    H, E, k = 128, 64, 4
    x = np.zeros((3, H), np.float16)           # all logits equal -> ties everywhere
    wr = synth.router_weight(5, "tie.w", H, E)
    idx, w, _ = _route(x, wr, None, k)
    assert (idx == np.arange(k)[None, :]).all()
    assert np.allclose(w, 1.0 / k)
    bias = synth.zipf_router_bias(5, "tie.b", E)
    x = synth.activations(5, "tie.x", 7, H)
    idx, w, logits = _route(x, wr, bias, k)
    exp_logits = oracle.router_logits(x, wr, bias)
    assert (logits.view(np.uint32) == exp_logits.view(np.uint32)).all()
    exp_idx, _ = oracle.router_topk(exp_logits, k)
    assert (idx == exp_idx).all()


def test_router_topk_nan_rows_give_valid_indices():
    """A token row of NaN activations (all its logits NaN), a row whose logits are NaN for some experts only, and an
    ordinary row: the k indices of every row are distinct and inside [0, E) -- the dispatch and combine kernels index
    arrays with them -- and the ordinary row is unaffected.  Only berth_moe_router_topk runs: it writes indices and
    weights and dereferences nothing through them."""
    H, E, k = 128, 64, 8
    x = synth.activations(9, "nan.x", 3, H).copy()
    x[0, :] = np.float16("nan")
    wr = synth.router_weight(9, "nan.w", H, E).copy()
    idx, w, logits = _route(x, wr, None, k)
    assert np.isnan(logits[0]).all()
    for t in range(3):
        assert len(set(idx[t].tolist())) == k and idx[t].min() >= 0 and idx[t].max() < E, (t, idx[t])
    assert (idx[0] == np.arange(k)).all()                      # nothing compares: the lowest experts, in order
    # NaN for half of the experts of row 1: the finite ones win first
    wr2 = wr.copy()
    wr2[:, ::2] = np.float16("nan")
    idx2, w2, logits2 = _route(x[1:2], wr2, None, k)
    assert np.isnan(logits2[0, ::2]).all() and np.isfinite(logits2[0, 1::2]).all()
    assert (idx2[0] % 2 == 1).all() and len(set(idx2[0].tolist())) == k
    order = np.argsort(-logits2[0, 1::2], kind="stable")[:k] * 2 + 1
    assert (idx2[0] == order).all()


def test_moe_layer_with_nan_row_returns(oracle):
    """The whole layer with one NaN token among ordinary ones: it returns with a clean status, the NaN row's output is
    NaN, and every other token's output is what it is without the NaN row."""
    H, I, E, k, bits, cb = 256, 128, 32, 4, 4, 2
    wts = synth.moe_layer_weights(1234, "moe42", H, I, E, k, bits, cb, shared_inter=128)
    x = synth.activations(1234, "nanrow.x", 6, H).copy()
    clean, idx_c, _ = _run_layer(wts, x)
    x[2, :] = np.float16("nan")
    out, idx, w = _run_layer(wts, x)                            # asserts device_status == 0
    assert np.isnan(out[2]).all()
    keep = [0, 1, 3, 4, 5]
    assert (idx[keep] == idx_c[keep]).all()
    assert (out[keep].view(np.uint32) == clean[keep].view(np.uint32)).all()
    assert len(set(idx[2].tolist())) == k and 0 <= idx[2].min() and idx[2].max() < E


def _run_layer(wts, x, fuse_shared=True, pair_gate_up=True):
    T = x.shape[0]
    layer = moe.MoeLayer(torch.device("cuda"), wts, T, fuse_shared=fuse_shared, pair_gate_up=pair_gate_up)
    out = torch.full((T, wts["hidden"]), float("nan"), dtype=torch.float32, device="cuda")
    idx = torch.empty((T, wts["top_k"]), dtype=torch.int32, device="cuda")
    w = torch.empty((T, wts["top_k"]), dtype=torch.float32, device="cuda")
    layer.forward(dev(x), out, idx, w)
    torch.cuda.synchronize()
    assert kernels.device_status(torch.cuda.current_device()) == 0
    return out.cpu().numpy(), idx.cpu().numpy(), w.cpu().numpy()


@pytest.mark.parametrize("T", [1, 5, 40, 130])
@pytest.mark.parametrize("bits,cb,shared", [(4, 2, 128), (4, 0, 0), (3, 1, 256)])
def test_moe_layer_small_vs_oracle(oracle, T, bits, cb, shared):
    H, I, E, k = 256, 128, 32, 4
    wts = synth.moe_layer_weights(1234, f"moe{bits}{cb}", H, I, E, k, bits, cb, shared_inter=shared)
    x = synth.activations(1234, f"moe.x{T}", T, H)
    out, idx, w = _run_layer(wts, x)
    exp_out, exp_idx, exp_w = oracle.moe_layer(wts, x)
    assert (idx == exp_idx).all()                       # routing: bit-exact
    assert np.abs(w - exp_w).max() <= 1e-6
    y64 = oracle.moe_layer_f64(wts, x, exp_idx, exp_w)
    mx, mean = rel_errors(out, y64)
    assert mx <= MAX_REL and mean <= MEAN_REL, (mx, mean)
    rms = np.sqrt((y64 ** 2).mean())
    assert np.abs(out - exp_out).max() <= 4e-3 * rms


@pytest.mark.parametrize("T", [1, 64])
def test_moe_layer_config3_vs_oracle(oracle, T):
    """benchmark configuration 3: hidden 2048, 256 experts + shared, top-8, intermediate 512, 4 bpw."""
    H, I, E, k, bits, cb = 2048, 512, 256, 8, 4, 2
    wts = synth.moe_layer_weights(1234, "c3", H, I, E, k, bits, cb, shared_inter=512)
    x = synth.activations(1234, f"c3.x{T}", T, H)
    out, idx, w = _run_layer(wts, x)
    exp_out, exp_idx, exp_w = oracle.moe_layer(wts, x)
    assert (idx == exp_idx).all()
    y64 = oracle.moe_layer_f64(wts, x, exp_idx, exp_w)
    mx, mean = rel_errors(out, y64)
    assert mx <= MAX_REL and mean <= MEAN_REL, (mx, mean)


def test_moe_layer_config3_1024_tokens_sampled_vs_oracle(oracle):
    """Configuration 3 at 1024 tokens: the grouped tensor-core launches at their own sizes (2048 / 512, 257 matrices,
    the doubled gate/up table, persistent CTAs).  Routing of all 1024 tokens bit-exact against the checker; the outputs
    of twelve sampled tokens against the checker's layer and its fp64 evaluation (the layer is row-wise, so a token's
    output does not depend on the batch it sits in)."""
    H, I, E, k, bits, cb, T = 2048, 512, 256, 8, 4, 2, 1024
    wts = synth.moe_layer_weights(1234, "c3", H, I, E, k, bits, cb, shared_inter=512)
    x = synth.activations(1234, f"c3.x{T}", T, H)
    out, idx, w = _run_layer(wts, x)
    assert "k_exl3_gemm_tc_grouped" in moe.last_launch()
    exp_idx, exp_w = oracle.router_topk(oracle.router_logits(x, wts["w_router"]), k)
    assert (idx == exp_idx).all() and np.abs(w - exp_w).max() <= 1e-6
    sample = np.array([0, 1, 77, 128, 255, 256, 383, 511, 640, 777, 1000, 1023])
    xs = np.ascontiguousarray(x[sample])
    exp_out, idx_s, w_s = oracle.moe_layer(wts, xs)
    assert (idx_s == idx[sample]).all()
    y64 = oracle.moe_layer_f64(wts, xs, idx_s, w_s)
    assert_close(out[sample], y64, "c3 T=1024 sample")
    assert np.abs(out[sample] - exp_out).max() <= 4e-3 * np.sqrt((y64 ** 2).mean())


@pytest.mark.parametrize("T", [400, 1000])
@pytest.mark.parametrize("fuse_shared,pair", [(True, True), (False, False)])
def test_moe_layer_many_rows_per_expert_vs_oracle(oracle, T, fuse_shared, pair):
    """Few experts and many rows each (100 to 250 rows per expert on average, far more on the popular ones): with
    inner dimensions this short the layer keeps 128-row problems on the grouped tensor-core kernel (two epilogue
    teams for the down projection); every token against the checker, with the shared expert stacked behind the experts
    and the paired gate/up table, and without either."""
    H, I, E, k, bits, cb = 256, 128, 32, 8, 4, 2
    wts = synth.moe_layer_weights(1234, "wide", H, I, E, k, bits, cb, shared_inter=128)
    x = synth.activations(1234, f"wide.x{T}", T, H)
    out, idx, w = _run_layer(wts, x, fuse_shared=fuse_shared, pair_gate_up=pair)
    assert "k_exl3_gemm_tc_grouped" in moe.last_launch() and "tile=128x" in moe.last_launch()
    exp_out, exp_idx, exp_w = oracle.moe_layer(wts, x)
    assert (idx == exp_idx).all() and np.abs(w - exp_w).max() <= 1e-6
    y64 = oracle.moe_layer_f64(wts, x, exp_idx, exp_w)
    assert_close(out, y64, f"T={T}")
    assert np.abs(out - exp_out).max() <= 4e-3 * np.sqrt((y64 ** 2).mean())


@pytest.mark.parametrize("T,hint", [(400, 256), (600, 384), (1000, 384), (1000, 128)])
def test_expert_stage_wide_grouped_tiles_vs_oracle(oracle, T, hint):
    """The expert stage with 256- and 384-row problems (two and three 128-row sub-tiles of the grouped tensor-core
    kernel, what a layer with long inner dimensions plans): the staged path (sort / gather / experts / gather / combine
    through the C ABI) with the problem height fixed, every token against the checker."""
    H, I, E, k, bits, cb = 256, 128, 32, 8, 4, 2
    wts = synth.moe_layer_weights(1234, "wide", H, I, E, k, bits, cb, shared_inter=128)
    x = synth.activations(1234, f"wide.x{T}", T, H)
    stages = moe.GpuStages(torch.device("cuda", torch.cuda.current_device()), wts, E, max_rows=T * k, max_rows_per_expert=T)
    stages.force_hint = hint
    layer = moe.EpMoeLayer.__new__(moe.EpMoeLayer)
    layer.dist, layer.group, layer.stages = _OneRankDist, None, stages
    layer.world, layer.rank, layer.E, layer.k, layer.n_local, layer.e0, layer.last_stats = 1, 0, E, k, E, 0, {}
    out, idx, w = layer.forward(dev(x))
    torch.cuda.synchronize()
    assert kernels.device_status(torch.cuda.current_device()) == 0
    exp_out, exp_idx, exp_w = oracle.moe_layer(wts, x)
    assert (idx.cpu().numpy() == exp_idx).all()
    y64 = oracle.moe_layer_f64(wts, x, exp_idx, exp_w)
    assert_close(out.cpu().numpy(), y64, f"T={T} hint={hint}")


def test_moe_layer_skewed_routing_property():
    """Zipf-biased router at 1024 tokens: every token's output equals the same token run alone
    (the layer is row-wise), which checks dispatch / permutation / combine at full size without
    the CPU checker."""
    H, I, E, k, bits, cb = 2048, 512, 256, 8, 4, 2
    bias = synth.zipf_router_bias(1234, "c4.bias", E, s=1.1, strength=0.25)
    wts = synth.moe_layer_weights(1234, "c3", H, I, E, k, bits, cb, shared_inter=512, router_bias=bias)
    x = synth.activations(1234, "c4.x", 1024, H)
    out, idx, w = _run_layer(wts, x)
    counts = np.bincount(idx.ravel(), minlength=E)
    assert counts.sum() == 1024 * k and counts.max() > 2 * counts.mean()      # visibly skewed
    rms = np.sqrt((out.astype(np.float64) ** 2).mean())
    for t in (0, 17, 500, 1023):
        o1, i1, w1 = _run_layer(wts, x[t:t + 1])
        assert (i1[0] == idx[t]).all()
        assert np.abs(o1[0] - out[t]).max() <= 4e-3 * rms


class _OneRankDist:
    """A one-rank stand-in for torch.distributed: an all-to-all among one rank is a copy."""
    @staticmethod
    def get_world_size(group=None):
        return 1

    @staticmethod
    def get_rank(group=None):
        return 0

    @staticmethod
    def all_to_all_single(out, inp, out_splits=None, in_splits=None, group=None):
        out.copy_(inp)


@pytest.mark.parametrize("T", [1, 48])
def test_expert_parallel_stages_match_fused_layer(T):
    """The staged path the expert-parallel host uses (sort / gather / experts / gather / combine through
    the C ABI) gives the same result as berth_moe_layer."""
    H, I, E, k, bits, cb = 256, 128, 32, 4, 4, 2
    wts = synth.moe_layer_weights(1234, "ep1", H, I, E, k, bits, cb, shared_inter=128)
    x = synth.activations(1234, f"ep1.x{T}", T, H)
    ref, ref_idx, _ = _run_layer(wts, x)
    stages = moe.GpuStages(torch.device("cuda", torch.cuda.current_device()), wts, E, max_rows=T * k, max_rows_per_expert=T)
    layer = moe.EpMoeLayer.__new__(moe.EpMoeLayer)
    layer.dist, layer.group, layer.stages = _OneRankDist, None, stages
    layer.world, layer.rank, layer.E, layer.k, layer.n_local, layer.e0, layer.last_stats = 1, 0, E, k, E, 0, {}
    out, idx, w = layer.forward(dev(x))
    torch.cuda.synchronize()
    assert (idx.cpu().numpy() == ref_idx).all()
    rms = np.sqrt((ref.astype(np.float64) ** 2).mean())
    assert np.abs(out.cpu().numpy() - ref).max() <= 1e-3 * rms
    assert layer.last_stats["recv_rows"] == T * k


@pytest.mark.parametrize("T", [1, 40, 130])
def test_shared_expert_inside_the_grouped_launches(T):
    """A shared expert stored behind the expert stacks runs as matrix E of the grouped launches; the result
    agrees with the layer that runs it through three linears of its own (same routing, outputs within the
    fp16 rounding of the intermediate activations)."""
    H, I, E, k = 256, 128, 32, 4
    wts = synth.moe_layer_weights(1234, "fuse", H, I, E, k, 4, 2, shared_inter=I)
    x = synth.activations(1234, f"fuse.x{T}", T, H)
    fused, idx_f, w_f = _run_layer(wts, x, fuse_shared=True)
    plain, idx_p, w_p = _run_layer(wts, x, fuse_shared=False)
    assert (idx_f == idx_p).all() and (w_f == w_p).all()
    rms = np.sqrt((plain.astype(np.float64) ** 2).mean())
    assert np.abs(fused - plain).max() <= 5e-3 * rms


@pytest.mark.parametrize("T", [1, 5, 40, 130, 300])
@pytest.mark.parametrize("shared", [0, 128])
def test_gate_and_up_as_one_stack(T, shared):
    """With the up stack stored directly behind the gate stack both projections run as one grouped launch over a
    doubled problem table: same kernels, same summation order, hence the same bits as two launches."""
    H, I, E, k = 256, 128, 32, 4
    wts = synth.moe_layer_weights(1234, "pair", H, I, E, k, 4, 2, shared_inter=shared)
    x = synth.activations(1234, f"pair.x{T}", T, H)
    one, idx_1, w_1 = _run_layer(wts, x, pair_gate_up=True)
    two, idx_2, w_2 = _run_layer(wts, x, pair_gate_up=False)
    assert (idx_1 == idx_2).all() and (w_1 == w_2).all()
    assert (one.view(np.uint32) == two.view(np.uint32)).all()


def test_moe_layer_loaded_from_a_checkpoint(tmp_path):
    """The experts of a layer written as per-expert checkpoint tensors (`<layer>.experts.<e>.<proj>_proj.*`), read
    back with Checkpoint.load_experts and run: the same bits as the layer built from the arrays."""
    from berth_b200.checkpoint import Checkpoint
    from tests.test_checkpoint_host import t, write_safetensors
    H, I, E, k, bits, cb, T = 256, 128, 32, 4, 4, 2, 9
    wts = synth.moe_layer_weights(1234, "ck", H, I, E, k, bits, cb)
    tensors = []
    for e in range(E):
        for proj, (K, N) in (("gate", (H, I)), ("up", (H, I)), ("down", (I, H))):
            pre = f"model.layers.0.mlp.experts.{e}.{proj}_proj"
            tensors += [t(pre + ".trellis", "I16", (K // 16, N // 16, 16 * bits), wts[f"{proj}_trellis"][e].view(np.int16)),
                        t(pre + ".suh", "F16", (K,), wts[f"{proj}_suh"][e]), t(pre + ".svh", "F16", (N,), wts[f"{proj}_svh"][e]),
                        t(pre + ".mul1", "I32", ())]
    write_safetensors(tmp_path / "model.safetensors", tensors)
    with Checkpoint.open(str(tmp_path)) as ck:
        assert len(ck.linears()) == 3 * E
        got = ck.load_experts("model.layers.0.mlp", E)
    assert (got["bits"], got["cb"]) == (bits, cb)
    loaded = dict(wts)
    for proj in ("gate", "up", "down"):
        for part in ("trellis", "suh", "svh"):
            assert (got[f"{proj}_{part}"].view(np.uint16) == np.asarray(wts[f"{proj}_{part}"]).view(np.uint16)).all()
            loaded[f"{proj}_{part}"] = got[f"{proj}_{part}"]
    x = synth.activations(1234, "ck.x", T, H)
    a, idx_a, w_a = _run_layer(wts, x)
    b, idx_b, w_b = _run_layer(loaded, x)
    assert (idx_a == idx_b).all() and (a.view(np.uint32) == b.view(np.uint32)).all()


def test_peer_memory_layer_on_one_rank():
    """P2pMoeLayer (exchange by peer-memory stores and flag barriers inside the kernels) on a single-rank
    group: the rank is its own peer, so the whole send / deliver / experts / return / combine chain runs,
    and the result equals the fused single-GPU layer's."""
    import torch.distributed as dist
    if not dist.is_available() or not dist.is_nccl_available():
        pytest.skip("torch.distributed with NCCL is not available")
    H, I, E, k, bits, cb = 256, 128, 32, 4, 4, 2
    wts = synth.moe_layer_weights(1234, "p2p1", H, I, E, k, bits, cb, shared_inter=128)
    own_group = not dist.is_initialized()
    if own_group:
        dist.init_process_group("nccl", init_method="tcp://127.0.0.1:29533", rank=0, world_size=1,
                                device_id=torch.device("cuda", torch.cuda.current_device()))
    try:
        device = torch.device("cuda", torch.cuda.current_device())
        stages = moe.GpuStages(device, wts, E, max_rows=64 * k + 64, max_rows_per_expert=64)
        try:
            layer = moe.P2pMoeLayer(stages, dist.group.WORLD, E, k, max_tokens=64, max_rows=64 * k + 64)
        except Exception as exc:   # symmetric memory needs driver support that not every box has
            pytest.skip(f"symmetric memory unavailable: {exc!r}")
        for T in (1, 48):
            x = synth.activations(1234, f"p2p1.x{T}", T, H)
            ref, ref_idx, _ = _run_layer(wts, x)
            for _ in range(2):    # twice: the epochs of the flag barriers advance
                out, idx, w = layer.forward(dev(x))
            torch.cuda.synchronize()
            assert kernels.device_status(torch.cuda.current_device()) == 0
            assert (idx.cpu().numpy() == ref_idx).all()
            rms = np.sqrt((ref.astype(np.float64) ** 2).mean())
            assert np.abs(out.cpu().numpy() - ref).max() <= 1e-3 * rms
    finally:
        if own_group:
            dist.destroy_process_group()


def test_expert_stage_overflow_sets_status_and_returns():
    """A peer-memory layer on one rank whose receive buffer is sized for fewer rows than the routing produces: the
    senders drop the rows that do not fit, the problem table of the receiving side is cut at the buffer, status bit 64
    is raised, the call returns (no wild access), and the next call with a fitting batch is clean."""
    import torch.distributed as dist
    if not dist.is_available() or not dist.is_nccl_available():
        pytest.skip("torch.distributed with NCCL is not available")
    H, I, E, k, bits, cb = 256, 128, 32, 4, 4, 2
    wts = synth.moe_layer_weights(1234, "p2p1", H, I, E, k, bits, cb, shared_inter=128)
    own_group = not dist.is_initialized()
    if own_group:
        dist.init_process_group("nccl", init_method="tcp://127.0.0.1:29534", rank=0, world_size=1,
                                device_id=torch.device("cuda", torch.cuda.current_device()))
    try:
        device = torch.device("cuda", torch.cuda.current_device())
        max_rows = 40 * k + 40                      # fits 40 tokens (and their shared-expert rows)
        stages = moe.GpuStages(device, wts, E, max_rows=max_rows, max_rows_per_expert=64)
        try:
            layer = moe.P2pMoeLayer(stages, dist.group.WORLD, E, k, max_tokens=64, max_rows=max_rows)
        except Exception as exc:
            pytest.skip(f"symmetric memory unavailable: {exc!r}")
        assert kernels.device_status(torch.cuda.current_device()) == 0
        x = synth.activations(1234, "p2p.over.x", 64, H)          # 64 tokens: 256 + 64 rows > 200
        out, idx, w = layer.forward(dev(x))
        torch.cuda.synchronize()
        assert kernels.device_status(torch.cuda.current_device()) & 64
        x = synth.activations(1234, "p2p.fit.x", 24, H)
        ref, ref_idx, _ = _run_layer(wts, x)
        out, idx, w = layer.forward(dev(x))
        torch.cuda.synchronize()
        assert kernels.device_status(torch.cuda.current_device()) == 0
        assert (idx.cpu().numpy() == ref_idx).all()
        assert np.abs(out.cpu().numpy() - ref).max() <= 1e-3 * np.sqrt((ref.astype(np.float64) ** 2).mean())
    finally:
        if own_group:
            dist.destroy_process_group()


def test_expert_parallel_flag_wait_runs_out_and_reports():
    """The bounded wait of the expert-parallel exchange, made to run out without harming anything: rank 0 of a
    two-rank exchange whose "peer" buffers are ordinary local allocations that nobody else writes.  The flag of rank 1
    never arrives, the wait gives up after its limit (well under a second per barrier), the call returns, and
    berth_device_status reports bit 32; a following ordinary layer call is clean.  No rank is killed, nothing faults:
    every store of the call lands in the local stand-in buffers."""
    import ctypes as C
    from berth_b200 import _lib
    H, E, k, T, world = 256, 32, 4, 8, 2
    l = _lib.lib()
    dev_ = torch.device("cuda", torch.cuda.current_device())
    x = dev(synth.activations(1234, "flag.x", T, H))
    wr = dev(synth.router_weight(1234, "flag.w", H, E))
    z = lambda n, dt=torch.uint8: torch.zeros(n, dtype=dt, device=dev_)
    max_rows = T * k + T
    cnt = [z(world * E * 4) for _ in range(world)]
    flags = [z(3 * 8 * 4) for _ in range(world)]
    recv = [z(max_rows * H * 2) for _ in range(world)]
    ptrs = lambda ts: (C.c_void_p * world)(*[t.data_ptr() for t in ts])
    ws = z(l.berth_moe_p2p_send_workspace_bytes(T, E, k, world))
    idx, w, inv = z(T * k, torch.int32), z(T * k, torch.float32), z(T * k, torch.int32)
    assert kernels.device_status(torch.cuda.current_device()) == 0
    rc = l.berth_moe_p2p_send(x.data_ptr(), T, wr.data_ptr(), None, H, E, k, idx.data_ptr(), w.data_ptr(), inv.data_ptr(), 0, world, 1,
                              ptrs(cnt), ptrs(flags), ptrs(recv), max_rows, ws.data_ptr(), ws.numel(), None)
    assert rc == 0, moe.last_error()
    torch.cuda.synchronize()                       # returns: the waits are bounded
    assert kernels.device_status(torch.cuda.current_device()) & 32
    assert kernels.device_status(torch.cuda.current_device()) == 0      # read-and-clear
    assert int(idx.min()) >= 0 and int(idx.max()) < E                    # the routing itself was done
    wts = synth.moe_layer_weights(1234, "moe42", 256, 128, 32, 4, 4, 2, shared_inter=128)
    _run_layer(wts, synth.activations(1234, "flag.after", 3, 256))      # asserts a clean status


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_layers_vs_oracle_on_real_ranks(world):
    """`world` ranks on `world` GPUs (skipped on a smaller box): every token of every rank through the peer-memory
    exchange and through the NCCL exchange against the CPU checker's whole layer, uniform and skewed routing, ranks
    without tokens included (tests/ep_p2p_worker.py)."""
    import subprocess
    import sys as _sys
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ep_p2p_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([_sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world), "--master-addr",
                        "127.0.0.1", "--master-port", str(29541 + world), worker], capture_output=True, text=True, timeout=900, env=env)
    ranks = "\n".join(line for line in r.stderr.splitlines() if line.startswith("[rank"))   # the workers' own tracebacks
    assert r.returncode == 0, r.stdout[-1500:] + ranks[-3000:]
    for i in range(world):
        assert f"P2P-OK {i}" in r.stdout
    print(r.stdout)
