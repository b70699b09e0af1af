// EXL3 decode GEMV (size_m <= 32): trellis tiles streamed through shared memory by TMA, decoded
// in registers and accumulated on the tensor cores by one persistent launch; a tiny rotation
// kernel for the activations runs before it and a wide finishing kernel (split-K sum, 128-wide
// Hadamard, output scale) after it, the three chained by programmatic dependent launch.
//
// Roofline: HBM.  Algorithmic bytes per launch = K*N*BITS/8 + 2K + 2N + 2MK + out_bytes*M*N.
// At 4 bits per weight the roofline asks for ~36 weights per cycle per SM, while the two
// integer pipes of an SM (ALU: lop3/prmt/shf; FMA-heavy: imad/dp4a/dp2a) issue 2 warp
// instructions per cycle each, so the design goal is the fewest integer instructions per
// weight, spread evenly over both pipes:
//   * window extraction for 4-bit tiles with byte permutes: 13 operations for 8 windows;
//   * 3INST / MCG: multiply(-add) + one lop3 per weight, and NO half add: the two fp16 halves of
//     the codebook word are fed to the MMA as two k-slots against a duplicated activation, so
//     the tensor core performs lo + hi (fp32, exact) -- 2 MMAs per 16x16 tile per 8 tokens;
//   * MUL1: multiply + dp4a with accumulator 0x6400 yields the fp16 bits of 1024 + byte sum;
//     the affine map w = S*h + B is applied once per output in the epilogue
//     (S*acc + B*sum(x)), not per weight -- 1 MMA per tile.
//
// Work decomposition: "units" of 128 rows x BU*128 columns (8 k-tile rows; BU = 2 bands below
// 8 bits so that one k-tile row of a unit is a >= 2 KiB contiguous run, which is what the TMA
// engine needs to stream near HBM speed) ordered band-group-major; CTA c of G (= number of SMs)
// takes the contiguous unit range [c*U/G, (c+1)*U/G), so every SM streams the same number of
// bytes with no tail wave.  A range covers at most one partial band group at its head and one
// at its tail; their partial sums go to slabs (2 per CTA) which k_gemv_finish, one warp per
// (straddled band, row), sums in CTA order -- deterministic, nothing ever waits on a peer, and the loads
// of that sum are spread over the whole GPU instead of trailing behind the last CTA to arrive.
//
// Inside a CTA (21 warps, one CTA per SM):
//   warp 16      producer: one lane issues one 2-D TMA copy (8 rows x one run) per unit into a
//                ring of unit-sized stages guarded by full/empty mbarriers;
//   warps 0..15  consumers: a warp owns NT tile columns and every RW-th k-tile row of every
//                unit, keeping NT*TG*4 fp32 accumulators per lane (TG token groups of 8 for
//                m <= 8, 16, 32); at the end of a segment it dumps them into a double-buffered
//                shared slab and carries on -- consumers never meet at a barrier;
//   warps 17..20 epilogue: reduce the dumped slabs in fixed order and write the split-K slab, or,
//                when the CTA holds a band group's whole K, finish the bands themselves (MUL1
//                affine correction, Hadamard, svh, store), in the background of the streaming warps.
// Every mbarrier wait is bounded; a wait that runs out sets a status bit and carries on.
#include "gemv_common.cuh"
#include "silu.cuh"
#include "../../include/berth_b200.h"

#include <cuda.h>

#include <algorithm>
#include <mutex>

namespace berth {

namespace {

constexpr int kConsumerWarps = 16;
constexpr int kEpiWarps = 4;
constexpr int kProducerWarp = kConsumerWarps;
constexpr int kThreads = (kConsumerWarps + 1 + kEpiWarps) * 32;
constexpr int kEpiThreads = kEpiWarps * 32;
constexpr int kRingBytes = 96 * 1024;
constexpr int kFusedUnits = 26;   // most units per CTA for which the rotated activations fit in shared memory

// Compile-time geometry of a (BITS, TG) instance.
template <int BITS, int TG>
struct Geo {
    static constexpr int NW = 8 * BITS;                       // 32-bit words per tile
    static constexpr int BU = BITS <= 4 ? 2 : 1;              // bands per unit (a TMA box row holds at most 256 8-byte elements)
    static constexpr int TILE_COLS = 8 * BU;
    static constexpr int ROW_BYTES = TILE_COLS * NW * 4;      // one k-tile row of a unit
    static constexpr int W_BYTES = 8 * ROW_BYTES;             // trellis bytes of a unit
    static constexpr int ACT_BYTES = 8 * TG * 256;            // fragment-ordered activations of a unit
    static constexpr int STAGE_BYTES = W_BYTES + ACT_BYTES;
    static constexpr int S = kRingBytes / STAGE_BYTES;        // ring depth
    static constexpr int NT = 4 / TG;                         // tile columns per consumer warp
    static constexpr int CG = TILE_COLS / NT;                 // column groups
    static constexpr int RW = kConsumerWarps / CG;            // row streams
    static constexpr int RPW = 8 / RW;                        // k-tile rows per warp per unit
    static constexpr int TOK = 8 * TG;
    static constexpr int PITCH = BU * 128 + 4;                // floats per token row in shared slabs
    static constexpr int RED_SLAB = TOK * PITCH;
    static constexpr size_t SMEM = size_t(kRingBytes) + size_t(2 * RW + 1) * RED_SLAB * 4 + size_t(2 * S) * 8;
    // in-kernel rotation (TG == 1): the CTA's own rotated activations, one 2 KiB block per unit
    static constexpr size_t SMEM_FUSED = SMEM + size_t(kFusedUnits) * ACT_BYTES;
    static_assert(TG != 1 || SMEM_FUSED <= 227 * 1024, "shared memory of the in-kernel rotation variant");
    static_assert(S >= 2 && RW >= 1 && RW * RPW == 8 && CG * RW == kConsumerWarps, "geometry");
};

__device__ __forceinline__ void epi_sync()
{
    asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
}
// Hand-over of the partial-sum buffers between the streaming warps and the epilogue warps through
// hardware named barriers (ids 2,3 = buffer filled, 4,5 = buffer drained): the waiting side blocks in
// the barrier unit and takes no issue slots, the signalling side does not wait.  Every barrier counts
// all streaming and all epilogue threads.
constexpr int kHandoverThreads = (kConsumerWarps + kEpiWarps) * 32;
__device__ __forceinline__ void handover_signal(int id)
{
    asm volatile("bar.arrive %0, %1;" ::"r"(id), "n"(kHandoverThreads) : "memory");
}
__device__ __forceinline__ void handover_wait(int id)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "n"(kHandoverThreads) : "memory");
}
__device__ __forceinline__ void consumer_sync()
{
    asm volatile("bar.sync 6, %0;" ::"n"(kConsumerWarps * 32) : "memory");
}
__device__ __forceinline__ void grid_dependency_wait() { pdl_wait(); }
__device__ __forceinline__ void grid_launch_dependents() { pdl_trigger(); }

// ---------------------------------------------------------------- the kernel
// FUSED (TG == 1, dense launches whose CTAs take at most kFusedUnits units and never a whole band
// group): no rotation kernel runs before this one; the streaming warps rotate the 128-blocks of the
// CTA's own units into shared memory while the first weight stages are in flight, and the CTAs
// that hold band group 0 also write the rotated activations and their block sums for the caller
// and the finishing kernel.
template <int BITS, int CB, int TG, bool FUSED>
__global__ void __launch_bounds__(kThreads, 1) k_exl3_gemv(const __grid_constant__ CUtensorMap tmap, const GemvArgs p)
{
    static_assert(!FUSED || TG == 1, "in-kernel rotation is built for one token group");
    using G_ = Geo<BITS, TG>;
    constexpr int NW = G_::NW, BU = G_::BU, ROW_BYTES = G_::ROW_BYTES, W_BYTES = G_::W_BYTES, ACT_BYTES = G_::ACT_BYTES;
    constexpr int STAGE_BYTES = G_::STAGE_BYTES, S = G_::S;
    constexpr int NT = G_::NT, CG = G_::CG, RW = G_::RW, RPW = G_::RPW, TOK = G_::TOK, PITCH = G_::PITCH;
    constexpr int RED_SLAB = G_::RED_SLAB;

    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* ring = smem;
    float* red = reinterpret_cast<float*>(smem + kRingBytes);                 // [2][RW][TOK][PITCH]
    float* outbuf = red + 2 * RW * RED_SLAB;                                  // [TOK][PITCH]
    uint64_t* bars = reinterpret_cast<uint64_t*>(outbuf + RED_SLAB);
    uint32_t* actbuf = reinterpret_cast<uint32_t*>(smem + G_::SMEM);          // FUSED: [kFusedUnits][ACT_BYTES / 4]

    // Let the next kernel on the stream (normally the next linear's rotation) become resident now; it
    // waits for this grid's completion before it touches memory.
    grid_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bands = p.n >> 7, kblocks = p.k >> 7;
    const int bgroups = (bands + BU - 1) / BU;          // band groups of one problem
    const bool sliced = p.b_list != nullptr;
    const bool grouped = p.problems != nullptr || sliced;
    const int nprob = sliced ? p.n_slices : (p.problems ? min(max(__ldg(p.n_problems), 0), p.max_problems) : 1);
    const long long U = (long long) nprob * bgroups * kblocks;
    const int cta = blockIdx.x;
    const int G = U < (long long) gridDim.x ? int(U) : int(gridDim.x);   // CTAs that own units
    if (cta >= G) {
        grid_dependency_wait();   // a grid must not complete before its predecessors: its successor relies on that
        return;
    }
    const long long u0 = unit_begin(cta, U, G), u1 = unit_begin(cta + 1, U, G);
    const int nunits = int(u1 - u0);
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + S);

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, kConsumerWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == kProducerWarp) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            if (!sliced) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap) : "memory");
            // unit -> TMA coordinates of the weights and source of the activation block
            auto issue_weights = [&](int i, uint32_t dst, uint32_t bar) {
                const long long u = u0 + i;
                const int gbg = int(u / kblocks), kb = int(u - (long long) gbg * kblocks);
                const int pi = gbg / bgroups, lbg = gbg - pi * bgroups;
                if (sliced) {
                    // the slice's address comes from a device array, so no tensor map: one bulk copy per k-tile row
                    const unsigned char* base = reinterpret_cast<const unsigned char*>(__ldg(p.b_list + pi));
                    const size_t row_stride = size_t(__ldg(p.n_stride_list + pi) / 16) * (NW * 4);
#pragma unroll
                    for (int r = 0; r < 8; ++r)
                        bulk_load_1d(dst + r * ROW_BYTES, base + size_t(kb * 8 + r) * row_stride + size_t(lbg) * ROW_BYTES, ROW_BYTES, bar);
                    return;
                }
                const int z = p.problems ? load_problem(p.problems, pi, p.n_matrices, TOK, p.max_rows).z : 0;
                tma_load_3d(dst, &tmap, lbg * (ROW_BYTES / 8), kb * 8, z, bar);
            };
            auto issue_acts = [&](int i, uint32_t dst, uint32_t bar) {
                const long long u = u0 + i;
                const int gbg = int(u / kblocks), kb = int(u - (long long) gbg * kblocks);
                const int pi = gbg / bgroups;
                const int act = sliced ? __ldg(p.had_src_list + pi) : pi;
                bulk_load_1d(dst, p.afrag + (size_t(act) * kblocks + kb) * (ACT_BYTES / 4), ACT_BYTES, bar);
            };
            // The weights do not depend on the rotation kernel: fill the ring with them first,
            // then wait for the activations and complete those stages.
            const int pre = nunits < S ? nunits : S;
            // (a grouped launch's problem table was written before the rotation kernel started, so it
            // is already visible here)
            constexpr uint32_t kStageTx = FUSED ? W_BYTES : STAGE_BYTES;
            if (p.defer_weights) grid_dependency_wait();   // the caller may have written the weights just before this launch
            for (int i = 0; i < pre; ++i) {
                mbar_arrive_expect_tx(full0 + 8 * i, kStageTx);
                issue_weights(i, smem_u32(ring + i * STAGE_BYTES), full0 + 8 * i);
            }
            if constexpr (!FUSED) {
                grid_dependency_wait();
                for (int i = 0; i < pre; ++i) issue_acts(i, smem_u32(ring + i * STAGE_BYTES + W_BYTES), full0 + 8 * i);
            }
            int s = 0, lap = 1;
            for (int i = pre; i < nunits; ++i) {
                mbar_wait_parked(empty0 + 8 * s, (lap - 1) & 1, p.status, kStEmptyTimeout);
                mbar_arrive_expect_tx(full0 + 8 * s, kStageTx);
                const uint32_t dst = smem_u32(ring + s * STAGE_BYTES);
                issue_weights(i, dst, full0 + 8 * s);
                if constexpr (!FUSED) issue_acts(i, dst + W_BYTES, full0 + 8 * s);
                if (++s == S) { s = 0; ++lap; }
            }
        }
        return;
    }

    if (warp < kConsumerWarps) {
        // ------------------------------------------------------------ consumers
        const int cg = warp % CG, rs = warp / CG;
        const int g = lane >> 2, q = lane & 3, lane1 = (lane + 1) & 31;
        if constexpr (FUSED) {
            grid_dependency_wait();   // the activations come from the preceding kernels
            for (int i = threadIdx.x; i < nunits * (ACT_BYTES / 4); i += kConsumerWarps * 32) actbuf[i] = 0u;   // rows >= m stay zero
            consumer_sync();
            const int ntask = nunits * p.m;
            for (int task = warp; task < ntask; task += kConsumerWarps) {
                const int i = task / p.m, t = task - i * p.m;
                const long long uu = u0 + i;
                const int gbg = int(uu / kblocks), kb = int(uu - (long long) gbg * kblocks);
                float sx;
                const uint2 o = rotate_block<CB == 2>(p.a + size_t(t) * p.k, p.suh, kb, lane, sx, p.a_up ? p.a_up + size_t(t) * p.k : nullptr, p.act_limit);
                // lane holds k_in = 4*(lane&3) .. +3 of k-tile (lane/4) of the block: half h = k_in/8, pair index (k_in%8)/2
                *reinterpret_cast<uint2*>(actbuf + i * (ACT_BYTES / 4) + ((lane >> 2) * 2 + ((lane & 3) >> 1)) * 32 + t * 4 + 2 * (lane & 1)) = o;
                if (gbg == 0) {   // band group 0 meets every 128-block exactly once
                    *reinterpret_cast<uint2*>(p.a_had + size_t(t) * p.k + kb * 128 + lane * 4) = o;
                    if (CB == 2 && lane == 0) p.blocksum[t * kblocks + kb] = sx;
                }
            }
            consumer_sync();
        }
        int s = 0, phase = 0, flush = 0, ui = 0;
        long long u = u0;
        while (u < u1) {
            const Segment sg = segment_at(u, u0, u1, kblocks);
            float acc[NT][TG][4];
#pragma unroll
            for (int t = 0; t < NT; ++t)
#pragma unroll
                for (int tg = 0; tg < TG; ++tg) acc[t][tg][0] = acc[t][tg][1] = acc[t][tg][2] = acc[t][tg][3] = 0.f;

            for (int j = 0; j < sg.units; ++j) {
                mbar_wait(full0 + 8 * s, phase, p.status, kStFullTimeout);
                const uint32_t* stage = reinterpret_cast<const uint32_t*>(ring + s * STAGE_BYTES) + cg * NT * NW;
                const uint32_t* act = FUSED ? actbuf + ui * (ACT_BYTES / 4)
                                            : reinterpret_cast<const uint32_t*>(ring + s * STAGE_BYTES + W_BYTES);
                ++ui;
#pragma unroll
                for (int i = 0; i < RPW; ++i) {
                    dq::RowFrag<CB, TG> f;
                    f.load(act + (rs + RW * i) * (TG * 64), lane);
                    const uint32_t* rowp = stage + (rs + RW * i) * (ROW_BYTES / 4);
#pragma unroll
                    for (int t = 0; t < NT; ++t) {
                        uint32_t st[8];
                        dq::tile_states<BITS, CB>(rowp + t * NW, lane, lane1, st);
                        dq::tile_mma<CB, TG>(st, acc[t], f);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty0 + 8 * s);
                if (++s == S) { s = 0; phase ^= 1; }
            }

            // ---- dump this segment's partial sums; the epilogue warps take it from here
            const int buf = flush & 1;
            if (flush >= 2) handover_wait(4 + buf);   // the epilogue warps have drained this buffer
            float* mine = red + (buf * RW + rs) * RED_SLAB;
#pragma unroll
            for (int t = 0; t < NT; ++t)
#pragma unroll
                for (int tg = 0; tg < TG; ++tg) {
                    const int t0 = tg * 8 + 2 * q, c0 = (cg * NT + t) * 16 + g;
                    mine[t0 * PITCH + c0] = acc[t][tg][0];
                    mine[(t0 + 1) * PITCH + c0] = acc[t][tg][1];
                    mine[t0 * PITCH + c0 + 8] = acc[t][tg][2];
                    mine[(t0 + 1) * PITCH + c0 + 8] = acc[t][tg][3];
                }
            handover_signal(2 + buf);
            ++flush;
            u += sg.units;
        }
        return;
    }

    // ---------------------------------------------------------------- epilogue warps
    {
        const int ew = warp - kProducerWarp - 1;      // 0..3
        const int et = threadIdx.x - (kProducerWarp + 1) * 32;   // 0..127 = column inside a band
        // Block sums and the problem table come from the preceding kernels, and the slabs may still be
        // read by the finishing kernel of the previous linear.
        grid_dependency_wait();
        const int slab_rows = p.problems ? TOK : p.m;
        const size_t slab_floats = size_t(slab_rows) * BU * 128;
        int flush = 0;
        long long u = u0;
        while (u < u1) {
            const Segment sg = segment_at(u, u0, u1, kblocks);
            // the problem this band group belongs to: its rows, output rows, sign-scale vector
            const int pi = sg.bg / bgroups, lbg = sg.bg - pi * bgroups;
            const ProblemView pv = problem_view(p, pi, TOK);
            const int rows = pv.rows, row0 = pv.row0;
            const int buf = flush & 1;
            // A whole band group is finished here: fetch what that needs (the row sums of the rotated
            // activations, the output scales) while the streaming warps are still busy with the segment.
            constexpr int kRowsPerWarp = TOK / kEpiWarps;
            float sxr[kRowsPerWarp];
            uint2 svr[BU];
            if (sg.whole) {
                const float* bsum = p.blocksum + size_t(pv.act) * slab_rows * kblocks;
#pragma unroll
                for (int r = 0; r < kRowsPerWarp; ++r) {
                    const int row = ew + r * kEpiWarps;
                    sxr[r] = (CB == 2 && row < rows) ? row_sum(bsum + size_t(row) * kblocks, kblocks, lane) : 0.f;
                }
#pragma unroll
                for (int b = 0; b < BU; ++b) {
                    const int band = lbg * BU + b;
                    svr[b] = band < bands ? __ldg(reinterpret_cast<const uint2*>(pv.svh + band * 128 + lane * 4)) : make_uint2(0u, 0u);
                }
            }
            handover_wait(2 + buf);
            // fixed-order reduction over the row streams: thread et owns column et of every band
            float* dst = sg.whole ? outbuf : p.slabs + size_t(sg.head ? 2 * cta : 2 * cta + 1) * slab_floats;
            const int dpitch = sg.whole ? PITCH : BU * 128;
            for (int tok = 0; tok < TOK && tok < rows; ++tok) {
#pragma unroll
                for (int b = 0; b < BU; ++b) {
                    float v = 0.f;
#pragma unroll
                    for (int w = 0; w < RW; ++w) v = __fadd_rn(v, red[(buf * RW + w) * RED_SLAB + tok * PITCH + b * 128 + et]);
                    if (sg.whole) dst[tok * dpitch + b * 128 + et] = v;
                    else __stcg(dst + tok * dpitch + b * 128 + et, v);
                }
            }
            handover_signal(4 + buf);   // the streaming warps may refill this buffer
            if (sg.whole) {
                epi_sync();   // outbuf complete
#pragma unroll
                for (int r = 0; r < kRowsPerWarp; ++r) {
                    const int row = ew + r * kEpiWarps;
                    if (row < rows) {
#pragma unroll
                        for (int b = 0; b < BU; ++b) {
                            const int band = lbg * BU + b;
                            if (band < bands) {   // ragged last band group
                                float4 t = *reinterpret_cast<const float4*>(outbuf + row * PITCH + b * 128 + lane * 4);
                                float v[4] = {t.x, t.y, t.z, t.w};
                                finish_band<CB == 2 ? 1 : 0>(v, sxr[r], lane, svr[b], band, pv.c, size_t(row0 + row), pv.ldc, p.out_fp32, p.argmax, p.residual, p.sample);
                            }
                        }
                    }
                }
                epi_sync();   // outbuf is free again
            }
            ++flush;
            u += sg.units;
        }
    }
}

// Finishing kernel of the decode GEMV.  A band group whose K was split over several CTAs straddles
// at least one boundary between consecutive CTA ranges, so the grid is (boundary, chunk of eight
// (band, row) tasks): the block of the first boundary inside a band group takes that band group, one
// warp per task sums the row's split-K slabs in CTA order (eight independent loads in flight),
// applies the MUL1 affine correction, the 128-wide Hadamard and the output scale, and stores.  Band
// groups whose whole K sat in one CTA straddle no boundary; the decode kernel finished those.
__global__ void __launch_bounds__(256) k_gemv_finish(const FinishArgs p)
{
    grid_launch_dependents();
    grid_dependency_wait();
    const int lane = threadIdx.x & 31;
    const int bands = p.n >> 7, kblocks = p.k >> 7, bu = p.bu;
    const int bgroups = (bands + bu - 1) / bu;
    const int nprob = p.b_list ? p.n_slices : (p.problems ? min(max(__ldg(p.n_problems), 0), p.max_problems) : (p.n_stack > 1 ? p.n_stack : 1));
    const long long U = (long long) nprob * bgroups * kblocks;
    const int G = U < (long long) p.main_grid ? int(U) : p.main_grid;
    const int c = blockIdx.x + 1;                      // the boundary between the ranges of CTA c-1 and CTA c
    if (c >= G) return;
    const long long ub = unit_begin(c, U, G);
    const int gbg = int(ub / kblocks);
    const long long g0 = (long long) gbg * kblocks;    // first unit of the band group around the boundary
    if (ub == g0) return;                              // the boundary is a band-group start: nothing straddles it
    if (unit_begin(c - 1, U, G) > g0) return;          // an earlier boundary lies inside the same band group
    const int slab_rows = p.problems ? p.tok : p.m;
    const int task = blockIdx.y * 8 + (threadIdx.x >> 5);
    if (task >= bu * slab_rows) return;
    const int b = task / slab_rows, row = task - b * slab_rows;
    const int pi = gbg / bgroups, lbg = gbg - pi * bgroups, band = lbg * bu + b;
    if (band >= bands) return;   // ragged last band group
    const ProblemView pv = problem_view(p, pi, p.tok);
    const int rows = pv.rows, row0 = pv.row0;
    if (row >= rows) return;
    // slabs of this band group, in CTA order: the first CTA's tail (or head, if its range starts
    // exactly here), then the heads of the following CTAs
    const int first_cta = c - 1;
    const int last_cta = unit_owner(g0 + kblocks - 1, U, G);
    const int first_slab = (unit_begin(first_cta, U, G) >= g0) ? 2 * first_cta : 2 * first_cta + 1;
    const int nsl = last_cta - first_cta + 1;
    const size_t slab_floats = size_t(slab_rows) * bu * 128;
    const uint2 sr = __ldg(reinterpret_cast<const uint2*>(pv.svh + band * 128 + lane * 4));
    const float sx = p.mul1 ? row_sum(p.blocksum + (size_t(pv.act) * slab_rows + row) * kblocks, kblocks, lane) : 0.f;
    const float* base = p.slabs + (size_t(row) * bu + b) * 128 + lane * 4;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    for (int i0 = 0; i0 < nsl; i0 += 8) {
        float4 t[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int si = i0 + i;
            const int slab = si == 0 ? first_slab : 2 * (first_cta + si);
            t[i] = si < nsl ? __ldcg(reinterpret_cast<const float4*>(base + size_t(slab) * slab_floats))
                            : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (i0 + i < nsl) {
                v[0] = __fadd_rn(v[0], t[i].x); v[1] = __fadd_rn(v[1], t[i].y);
                v[2] = __fadd_rn(v[2], t[i].z); v[3] = __fadd_rn(v[3], t[i].w);
            }
        }
    }
    if (p.mul1 == 2) finish_band<2>(v, sx, lane, sr, band, pv.c, size_t(row0 + row), pv.ldc, p.out_fp32, p.argmax, p.residual, p.sample);
    else if (p.mul1) finish_band<1>(v, sx, lane, sr, band, pv.c, size_t(row0 + row), pv.ldc, p.out_fp32, p.argmax, p.residual, p.sample);
    else finish_band<0>(v, sx, lane, sr, band, pv.c, size_t(row0 + row), pv.ldc, p.out_fp32, p.argmax, p.residual, p.sample);
}

// ---------------------------------------------------------------- rotation of the activations
// a_had = fp16(H128(a * suh) / sqrt(128)) in the caller's [m][k] buffer; the same values again in
// MMA fragment order for the decode kernel (afrag[k/16][TG][2][8][4] words: the pair
// (k = 16*ktile + 8*h + 2*q, +1) of token 8*tg + t at word ((ktile*TG + tg)*2 + h)*32 + 4*t + q, zero
// for tokens >= m); blocksum[row][b] = sum of the 128 rounded values of a block.
// One warp per (token row, 128-block).  Lets the dependent GEMV start early (programmatic launch).
// With suh_list the sign-scale vector is entry `src` of that device array of addresses (sliced multi-linear).
__global__ void __launch_bounds__(128) k_rotate_in(const __half* __restrict__ a, const __half* __restrict__ suh_in,
                                                   __half* __restrict__ a_had, uint32_t* __restrict__ afrag,
                                                   float* __restrict__ blocksum, int rows, int rows_pad, int k,
                                                   const unsigned long long* __restrict__ suh_list, int src, long long a_src_stride,
                                                   const __half* __restrict__ a_up, float act_limit)
{
    // Trigger first: the decode kernel behind this one may then take each SM as the previous decode
    // kernel leaves it and prefetch its weights; it still waits for this grid, which itself waits here
    // for everything before it (the activations and the scratch this kernel overwrites).
    grid_launch_dependents();
    grid_dependency_wait();
    const int lane = threadIdx.x & 31, kblocks = k >> 7, tgs = rows_pad >> 3;
    const __half* suh = suh_in;
    if (suh_list) {   // blockIdx.y = source: its own sign-scale vector, rotated-input slab, fragment set and block sums
        src += blockIdx.y;
        suh = reinterpret_cast<const __half*>(__ldg(suh_list + src));
        a += size_t(src) * size_t(a_src_stride);   // (uniform multi-linear with one input per matrix; else every source reads the same rows)
        a_had += size_t(src) * rows * k;
        afrag += size_t(src) * (k >> 4) * tgs * 64;
        blocksum += size_t(src) * rows * kblocks;
    }
    const int total = rows_pad * kblocks;
    for (int idx = blockIdx.x * 4 + (threadIdx.x >> 5); idx < total; idx += gridDim.x * 4) {
        const int row = idx / kblocks, b = idx - row * kblocks;
        uint2 o = make_uint2(0u, 0u);
        if (row < rows) {
            float sx;
            o = rotate_block<true>(a + size_t(row) * k, suh, b, lane, sx, a_up ? a_up + size_t(row) * k : nullptr, act_limit);
            *reinterpret_cast<uint2*>(a_had + size_t(row) * k + b * 128 + lane * 4) = o;
            if (lane == 0) blocksum[row * kblocks + b] = sx;
        }
        // lane holds k_in = 4*(lane&3) .. +3 of k-tile (8*b + lane/4): half h = k_in/8, pair index q = (k_in%8)/2
        const int ktile = b * 8 + (lane >> 2), hsel = (lane & 3) >> 1, q = 2 * (lane & 1);
        const size_t w = ((size_t(ktile) * tgs + (row >> 3)) * 2 + hsel) * 32 + (row & 7) * 4 + q;
        *reinterpret_cast<uint2*>(afrag + w) = o;
    }
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link-time libcuda dependency).
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled()
{
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        cuda_ok(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q), "cuTensorMapEncodeTiled entry point");
        if (!p || q != cudaDriverEntryPointSuccess) throw std::runtime_error("cuTensorMapEncodeTiled is not available in this driver");
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

}  // namespace

// 3-D view of a trellis stack: z = matrix, y = k-tile row (K/16), x = the row's (N/16) tiles of
// 32*bits bytes in 8-byte elements; box = one unit (8 rows x BU bands of one matrix).  Columns
// past the matrix read as zero.
CUtensorMap trellis_map(const void* trellis, int n_matrices, int size_k, int size_n, int bits, int box_bytes)
{
    if (reinterpret_cast<uintptr_t>(trellis) % 16 != 0) throw std::runtime_error("exl3 linear: trellis must be 16-byte aligned");
    CUtensorMap map;
    const cuuint64_t row_bytes = cuuint64_t(size_n / 16) * 32 * bits;
    const cuuint64_t dims[3] = {row_bytes / 8, cuuint64_t(size_k / 16), cuuint64_t(n_matrices)};
    const cuuint64_t strides[2] = {row_bytes, row_bytes * cuuint64_t(size_k / 16)};
    const cuuint32_t box[3] = {cuuint32_t(box_bytes / 8), 8, 1};
    const cuuint32_t elem[3] = {1, 1, 1};
    CUresult r = encode_tiled()(&map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 3, const_cast<void*>(trellis), dims, strides, box, elem,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) throw std::runtime_error("exl3 linear: cuTensorMapEncodeTiled failed (" + std::to_string(int(r)) + ")");
    return map;
}

namespace {

template <int BITS, int CB, int TG, bool FUSED>
size_t launch_one(const void* trellis, int n_matrices, const GemvArgs& args, int grid, cudaStream_t stream)
{
    using G_ = Geo<BITS, TG>;
    auto kern = k_exl3_gemv<BITS, CB, TG, FUSED>;
    constexpr size_t kSmem = FUSED ? G_::SMEM_FUSED : G_::SMEM;
    static bool attr_set[kMaxDevices] = {};
    const int dev = current_device();
    if (!attr_set[dev]) {
        cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSmem)), "gemv smem attribute");
        attr_set[dev] = true;
    }
    CUtensorMap map = {};   // a sliced launch addresses its weights through a device array, not through this map
    if (!args.b_list) map = trellis_map(trellis, n_matrices, args.k, args.n, BITS, G_::ROW_BYTES);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cuda_ok(cudaLaunchKernelEx(&cfg, kern, map, args), "k_exl3_gemv launch");
    return kSmem;
}

template <int BITS, int CB>
size_t launch_tg(int tg, bool fused, const void* t, int nm, const GemvArgs& a, int grid, cudaStream_t st)
{
    switch (tg) {
        case 1: return fused ? launch_one<BITS, CB, 1, true>(t, nm, a, grid, st) : launch_one<BITS, CB, 1, false>(t, nm, a, grid, st);
        case 2: return launch_one<BITS, CB, 2, false>(t, nm, a, grid, st);
        default: return launch_one<BITS, CB, 4, false>(t, nm, a, grid, st);
    }
}

template <int BITS>
size_t launch_cb(int cb, int tg, bool fused, const void* t, int nm, const GemvArgs& a, int grid, cudaStream_t st)
{
    switch (cb) {
        case 0: return launch_tg<BITS, 0>(tg, fused, t, nm, a, grid, st);
        case 1: return launch_tg<BITS, 1>(tg, fused, t, nm, a, grid, st);
        default: return launch_tg<BITS, 2>(tg, fused, t, nm, a, grid, st);
    }
}

size_t launch_bits(int k_bits, int cb, int tg, bool fused, const void* t, int nm, const GemvArgs& a, int grid, cudaStream_t st)
{
    switch (k_bits) {
        case 1: return launch_cb<1>(cb, tg, fused, t, nm, a, grid, st);
        case 2: return launch_cb<2>(cb, tg, fused, t, nm, a, grid, st);
        case 3: return launch_cb<3>(cb, tg, fused, t, nm, a, grid, st);
        case 4: return launch_cb<4>(cb, tg, fused, t, nm, a, grid, st);
        case 5: return launch_cb<5>(cb, tg, fused, t, nm, a, grid, st);
        case 6: return launch_cb<6>(cb, tg, fused, t, nm, a, grid, st);
        case 7: return launch_cb<7>(cb, tg, fused, t, nm, a, grid, st);
        case 8: return launch_cb<8>(cb, tg, fused, t, nm, a, grid, st);
        default: throw std::runtime_error("exl3 linear: K must be in 1..=8");
    }
}

// Rotation for a grouped launch: routed rows [R][k]; one block per problem, its warps share the
// (row, 128-block) pairs of the problem's real rows; the row's expert picks the sign-scale vector.
// Rows past the problem's count are left as they are: a token is a column of the MMA, so whatever
// sits there reaches only accumulators that nobody stores.
// MODE bits: kFragDual = a second scale stack with its own fragment and block-sum outputs (gate and up read the
// row once); kFragGather = row r < n_perm reads src row perm[r] / div, later rows src row r - n_perm;
// kFragSilu = the input is silu(src) * src_u, rounded to fp16 as the element-wise kernel rounds it.
constexpr int kFragDual = 1, kFragGather = 2, kFragSilu = 4;

template <int MODE>
__global__ void __launch_bounds__(256) k_rotate_rows(const RotateFragArgs a)
{
    grid_dependency_wait();      // the problem table comes from the preceding kernel
    grid_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, k = a.k, kblocks = k >> 7, tgs = a.tok >> 3;
    const int nprob = min(max(__ldg(a.n_problems), 0), a.max_problems);
    for (int pi = blockIdx.x; pi < nprob; pi += gridDim.x) {
        const GemvProblem pr = load_problem(a.problems, pi, a.n_matrices, a.tok, a.max_rows);
        const size_t so = size_t(pr.z) * k;
        const int pairs = pr.rows * kblocks;
#pragma unroll 4
        for (int pair = warp; pair < pairs; pair += 8) {
            const int lr = pair / kblocks, b = pair - lr * kblocks;
            const int row = pr.row0 + lr, kcol = b * 128 + lane * 4;
            int src_row = row;
            if constexpr (MODE & kFragGather) src_row = row < a.n_perm ? min(max(__ldg(a.perm + row) / a.div, 0), max(a.n_perm / a.div - 1, 0)) : row - a.n_perm;
            uint2 x = *reinterpret_cast<const uint2*>(a.src + size_t(src_row) * k + kcol);
            if constexpr (MODE & kFragSilu) {
                const uint2 u = *reinterpret_cast<const uint2*>(a.src_u + size_t(src_row) * k + kcol);
                const __half2 g0 = *reinterpret_cast<const __half2*>(&x.x), g1 = *reinterpret_cast<const __half2*>(&x.y);
                const __half2 u0 = *reinterpret_cast<const __half2*>(&u.x), u1 = *reinterpret_cast<const __half2*>(&u.y);
                x.x = dq::pack_half2(silu_mul_one(__low2half(g0), __low2half(u0), 0.0f), silu_mul_one(__high2half(g0), __high2half(u0), 0.0f));
                x.y = dq::pack_half2(silu_mul_one(__low2half(g1), __low2half(u1), 0.0f), silu_mul_one(__high2half(g1), __high2half(u1), 0.0f));
            }
            const int ktile = b * 8 + (lane >> 2), hsel = (lane & 3) >> 1, q = 2 * (lane & 1);
            const size_t w = (((size_t(pi) * (k >> 4) + ktile) * tgs + (lr >> 3)) * 2 + hsel) * 32 + (lr & 7) * 4 + q;
            const size_t bs = (size_t(pi) * a.tok + lr) * kblocks + b;
            float sx;
            const uint2 o = rotate_bits<true>(x, __ldg(reinterpret_cast<const uint2*>(a.suh_a + so + kcol)), lane, sx);
            if (lane == 0) a.bsum_a[bs] = sx;
            *reinterpret_cast<uint2*>(a.afrag_a + w) = o;
            if constexpr (MODE & kFragDual) {
                const uint2 o2 = rotate_bits<true>(x, __ldg(reinterpret_cast<const uint2*>(a.suh_b + so + kcol)), lane, sx);
                if (a.pair) {   // the same arrays, problem pi + nprob
                    if (lane == 0) a.bsum_a[bs + size_t(nprob) * a.tok * kblocks] = sx;
                    *reinterpret_cast<uint2*>(a.afrag_a + w + size_t(nprob) * (k >> 4) * tgs * 64) = o2;
                } else {
                    if (lane == 0) a.bsum_b[bs] = sx;
                    *reinterpret_cast<uint2*>(a.afrag_b + w) = o2;
                }
            }
        }
    }
}

}  // namespace

// The finishing kernel behind a decode launch of `main_grid` CTAs (nothing to do behind a single CTA).
void launch_finish(const GemvArgs& a, int bu, int tok, int main_grid, int mul1, cudaStream_t stream)
{
    if (main_grid < 2) return;
    FinishArgs f;
    f.slabs = a.slabs; f.blocksum = a.blocksum; f.c = a.c; f.argmax = a.argmax; f.sample = a.sample; f.residual = a.residual; f.svh = a.svh;
    f.problems = a.problems; f.n_problems = a.n_problems;
    f.max_problems = a.max_problems; f.n_matrices = a.n_matrices; f.max_rows = a.max_rows;
    f.m = a.m; f.k = a.k; f.n = a.n; f.out_fp32 = a.out_fp32;
    f.bu = bu; f.tok = tok; f.main_grid = main_grid; f.mul1 = mul1;
    f.b_list = a.b_list; f.svh_list = a.svh_list; f.c_list = a.c_list; f.n_stride_list = a.n_stride_list; f.had_src_list = a.had_src_list;
    f.n_slices = a.n_slices;
    f.n_stack = a.n_stack;
    const int slab_rows = a.problems ? tok : a.m;
    launch_pdl(k_gemv_finish, dim3(main_grid - 1, (bu * slab_rows + 7) / 8), dim3(256), 0, stream, "k_gemv_finish launch", f);
}


// Launches rotation + decode GEMV for up to 32 rows.  `sc` is the split-K scratch: the library's
// per-device workspace or the fixed in-image array of the allocation-free entry point.
std::string launch_gemv(const void* a, const void* trellis, void* c, const void* suh, void* a_had, const void* svh,
                        int size_m, int size_k, int size_n, int k_bits, int codebook, int out_fp32,
                        const GemvScratch& sc, int sms, cudaStream_t stream, unsigned long long* argmax, const float* residual,
                        const SampleArgs& sample, const ActInput& act)
{
    if (residual && !out_fp32) throw std::runtime_error("exl3 linear: the residual is added to fp32 outputs only");
    if (size_m > 32) throw std::runtime_error("exl3 gemv: size_m must be <= 32");
    if (size_k % 128 != 0)
        throw std::runtime_error("exl3 linear: no linked kernel for size_k that is not a multiple of 128 (128-wide Hadamard)");
    if (k_bits < 1 || k_bits > 8) throw std::runtime_error("exl3 linear: K must be in 1..=8");
    // MUL1, one row, every CTA's units within the limb area of the in-kernel rotation: integer tensor path with the
    // weights in tensor memory (measured a few percent ahead of this kernel there, behind it elsewhere)
    if (codebook == 2 && size_m == 1 && gemv_i8_rotates_in_kernel(size_m, size_k, size_n, k_bits, sms))
        return launch_gemv_i8(a, trellis, c, suh, a_had, svh, size_m, size_k, size_n, k_bits, out_fp32, sc, sms, stream, argmax, 1, residual, sample, act);
    const int tg = size_m <= 8 ? 1 : (size_m <= 16 ? 2 : 4);
    const int bu = k_bits <= 4 ? 2 : 1;   // bands per unit, as Geo<BITS, TG>::BU
    const int bands = size_n / 128, kblocks = size_k / 128, bgroups = (bands + bu - 1) / bu;
    if (size_t(size_m) * kblocks > sc.blocksum_floats)
        throw std::runtime_error("exl3 gemv: size_m * size_k / 128 exceeds the block-sum table of the scratch");
    const long long units = (long long) bgroups * kblocks;
    // One CTA per SM, but never more than 16 CTAs per band group: the last arriver of a band
    // group sums one slab per CTA, and a matrix that small is latency bound anyway.
    int grid = int(std::min<long long>(std::min<long long>(sms, units), (long long) bgroups * 16));
    // two slabs of [m][bu*128] fp32 per CTA
    const size_t per_cta = size_t(2) * size_m * bu * 128 * sizeof(float);
    if (size_t(grid) * per_cta > sc.slab_bytes) grid = int(sc.slab_bytes / per_cta);
    if (grid < 1) throw std::runtime_error("exl3 gemv: split-K scratch is too small for this shape");

    const size_t afrag_bytes = size_t(size_k / 16) * tg * 256;
    if (afrag_bytes > sc.afrag_bytes)
        throw std::runtime_error("exl3 gemv: size_k * ceil(size_m / 8) exceeds the activation-fragment area of the scratch");
    // In-kernel rotation for one or two rows (with more, the per-CTA repetition of the rotation costs more
    // than the separate kernel), when every CTA's units fit its shared-memory block and no CTA holds a
    // whole band group.
    const long long units_per_cta = (units + grid - 1) / grid;
    const bool fused = size_m <= 2 && units_per_cta <= kFusedUnits && units_per_cta < kblocks;
    if (!fused) {
        const int rot_total = 8 * tg * kblocks;
        launch_pdl(k_rotate_in, dim3(std::min((rot_total + 3) / 4, 4 * sms)), dim3(128), 0, stream, "k_rotate_in launch",
                   static_cast<const __half*>(a), static_cast<const __half*>(suh), static_cast<__half*>(a_had), sc.afrag,
                   sc.blocksum, size_m, 8 * tg, size_k, (const unsigned long long*) nullptr, 0, 0LL,
                   static_cast<const __half*>(act.up), act.limit);
    }

    GemvArgs args{};
    args.defer_weights = weights_streamed() ? 1 : 0;
    args.afrag = sc.afrag;
    args.blocksum = sc.blocksum;
    args.a_up = static_cast<const __half*>(act.up);
    args.act_limit = act.limit;
    args.a = static_cast<const __half*>(a);
    args.suh = static_cast<const __half*>(suh);
    args.a_had = static_cast<__half*>(a_had);
    args.c = c;
    args.argmax = argmax;
    args.sample = sample;
    args.residual = residual;
    args.svh = static_cast<const __half*>(svh);
    args.slabs = sc.slabs;
    args.counters = nullptr;
    args.status = sc.status;
    args.m = size_m; args.k = size_k; args.n = size_n;
    args.out_fp32 = out_fp32;
    args.problems = nullptr;
    args.n_problems = nullptr;
    args.max_problems = 1; args.n_matrices = 1; args.max_rows = size_m;
    args.b_list = nullptr; args.svh_list = nullptr; args.c_list = nullptr; args.n_stride_list = nullptr; args.had_src_list = nullptr;
    args.n_slices = 0;
    args.n_stack = 0;
    const size_t smem = launch_bits(k_bits, codebook, tg, fused, trellis, 1, args, grid, stream);
    launch_finish(args, bu, 8 * tg, grid, codebook == 2 ? 1 : 0, stream);
    return std::string(fused ? "" : "k_rotate_in + ") + "k_exl3_gemv<" + std::to_string(k_bits) + "," + std::to_string(codebook) + "," +
           std::to_string(tg) + (fused ? ",fused" : "") + "> grid=" + std::to_string(grid) + " block=" + std::to_string(kThreads) + " smem=" + std::to_string(smem) +
           " + k_gemv_finish";
}

void rotate_rows_frag(const RotateFragArgs& a, bool dual, bool silu, int sms, cudaStream_t stream)
{
    if (a.k % 128 != 0) throw std::runtime_error("exl3 grouped gemv: size_k must be a multiple of 128");
    if (a.tok != 8 && a.tok != 16 && a.tok != 32) throw std::runtime_error("exl3 grouped gemv: token groups must be 1, 2 or 4");
    if (!a.src || !a.suh_a || !a.afrag_a || !a.bsum_a || (dual && (!a.suh_b || (!a.pair && (!a.afrag_b || !a.bsum_b)))) || (silu && !a.src_u))
        throw std::runtime_error("exl3 grouped gemv: null rotation pointer");
    if (silu && (dual || a.perm)) throw std::runtime_error("exl3 grouped gemv: the silu rotation takes one plain input");
    const dim3 grid(std::max(1, std::min(a.max_problems, 16 * sms)));
    const int mode = (dual ? kFragDual : 0) | (a.perm ? kFragGather : 0) | (silu ? kFragSilu : 0);
    switch (mode) {
        case 0: launch_pdl(k_rotate_rows<0>, grid, dim3(256), 0, stream, "k_rotate_rows launch", a); break;
        case kFragDual: launch_pdl(k_rotate_rows<kFragDual>, grid, dim3(256), 0, stream, "k_rotate_rows launch", a); break;
        case kFragGather: launch_pdl(k_rotate_rows<kFragGather>, grid, dim3(256), 0, stream, "k_rotate_rows launch", a); break;
        case kFragDual | kFragGather:
            launch_pdl(k_rotate_rows<kFragDual | kFragGather>, grid, dim3(256), 0, stream, "k_rotate_rows launch", a);
            break;
        default: launch_pdl(k_rotate_rows<kFragSilu>, grid, dim3(256), 0, stream, "k_rotate_rows launch", a); break;
    }
}

std::string launch_gemv_grouped_rotated(const void* trellis_stack, int n_experts, void* c, const void* svh_stack,
                                        const GemvProblem* problems, const int* n_problems, int max_problems, int max_rows, int tg,
                                        const uint32_t* afrag, float* blocksum, int size_k, int size_n, int k_bits, int codebook,
                                        int out_fp32, const GemvScratch& sc, int sms, cudaStream_t stream)
{
    if (size_k % 128 != 0 || size_n % 128 != 0)
        throw std::runtime_error("exl3 grouped gemv: size_k and size_n must be multiples of 128");
    if (tg != 1 && tg != 2 && tg != 4) throw std::runtime_error("exl3 grouped gemv: token groups must be 1, 2 or 4");
    const int bu = k_bits <= 4 ? 2 : 1;
    int grid = sms;
    const size_t per_cta = size_t(2) * 8 * tg * bu * 128 * sizeof(float);
    if (size_t(grid) * per_cta > sc.slab_bytes) grid = int(sc.slab_bytes / per_cta);
    if (grid < 1) throw std::runtime_error("exl3 grouped gemv: split-K scratch is too small");
    GemvArgs args{};
    args.defer_weights = weights_streamed() ? 1 : 0;
    args.afrag = afrag;
    args.blocksum = blocksum;
    args.a = nullptr; args.suh = nullptr; args.a_had = nullptr;
    args.c = c;
    args.argmax = nullptr;
    args.residual = nullptr;
    args.svh = static_cast<const __half*>(svh_stack);
    args.problems = problems;
    args.n_problems = n_problems;
    args.max_problems = max_problems;
    args.n_matrices = n_experts;
    args.max_rows = max_rows;
    args.slabs = sc.slabs;
    args.counters = nullptr;
    args.status = sc.status;
    args.m = 8 * tg; args.k = size_k; args.n = size_n;
    args.out_fp32 = out_fp32;
    args.b_list = nullptr; args.svh_list = nullptr; args.c_list = nullptr; args.n_stride_list = nullptr; args.had_src_list = nullptr;
    args.n_slices = 0;
    args.n_stack = 0;
    const size_t smem = launch_bits(k_bits, codebook, tg, false, trellis_stack, n_experts, args, grid, stream);
    launch_finish(args, bu, 8 * tg, grid, codebook == 2 ? 1 : 0, stream);
    return "k_exl3_gemv<" + std::to_string(k_bits) + "," + std::to_string(codebook) + "," + std::to_string(tg) +
           ",grouped> grid=" + std::to_string(grid) + " block=" + std::to_string(kThreads) + " smem=" + std::to_string(smem) +
           " + k_gemv_finish";
}

std::string launch_gemv_grouped(const void* xr, const void* trellis_stack, int n_experts, void* c, const void* suh_stack,
                                const void* svh_stack, const GemvProblem* problems, const int* n_problems, int max_problems,
                                int max_rows, int tg, uint32_t* afrag, float* blocksum, int size_k, int size_n, int k_bits,
                                int codebook, int out_fp32, const GemvScratch& sc, int sms, cudaStream_t stream)
{
    if (tg != 1 && tg != 2 && tg != 4) throw std::runtime_error("exl3 grouped gemv: token groups must be 1, 2 or 4");
    RotateFragArgs r{};
    r.src = static_cast<const __half*>(xr);
    r.suh_a = static_cast<const __half*>(suh_stack);
    r.afrag_a = afrag; r.bsum_a = blocksum;
    r.problems = problems; r.n_problems = n_problems;
    r.tok = 8 * tg; r.k = size_k; r.max_problems = max_problems; r.n_matrices = n_experts; r.max_rows = max_rows;
    rotate_rows_frag(r, false, false, sms, stream);
    return "k_rotate_rows + " + launch_gemv_grouped_rotated(trellis_stack, n_experts, c, svh_stack, problems, n_problems, max_problems,
                                                            max_rows, tg, afrag, blocksum, size_k, size_n, k_bits, codebook, out_fp32, sc,
                                                            sms, stream);
}

// The slice lists of a uniform multi-linear (count equally shaped matrices, outputs one behind the other): output i at
// c + i * out_stride_bytes, row stride n, rotated input i.
__global__ void __launch_bounds__(256) k_uniform_lists(unsigned long long c_base, unsigned long long out_stride_bytes, int n, int count,
                                                       unsigned long long* __restrict__ c_list, int* __restrict__ n_stride,
                                                       int* __restrict__ had_src)
{
    grid_launch_dependents();
    grid_dependency_wait();   // the previous launch may still be reading the lists
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += gridDim.x * blockDim.x) {
        c_list[i] = c_base + (unsigned long long) i * out_stride_bytes;
        n_stride[i] = n;
        had_src[i] = i;
    }
}

std::string launch_gemv_sliced(const void* a, const void* b_list, const void* suh_list, void* a_had, const void* svh_list,
                               const void* c_list, const int* n_stride_list, const int* had_src_list, int num_had_src, int n_slices,
                               int size_m, int size_k, int size_n, int k_bits, int codebook, int out_fp32, const GemvScratch& sc,
                               int sms, cudaStream_t stream, long long a_src_stride);

// Uniform multi-linear: the library writes the slice lists itself and runs the sliced launch with every matrix as one
// slice (and one rotated input per matrix, from the shared rows or from the matrix's own).
std::string launch_gemv_uniform(const void* a, const void* b_list, const void* suh_list, void* a_had, const void* svh_list, void* c,
                                int count, bool per_matrix_input, int size_m, int size_k, int size_n, int k_bits, int codebook,
                                int out_fp32, const GemvScratch& sc, int sms, cudaStream_t stream)
{
    if (count < 1 || size_t(count) > kGemvListEntries)
        throw std::runtime_error("exl3_mgemm: the uniform mode takes 1 to " + std::to_string(kGemvListEntries) + " matrices");
    unsigned long long* c_list = sc.lists;
    int* n_stride = reinterpret_cast<int*>(sc.lists + kGemvListEntries);
    int* had_src = n_stride + kGemvListEntries;
    const unsigned long long stride = (unsigned long long) size_m * size_n * (out_fp32 ? 4 : 2);
    launch_pdl(k_uniform_lists, dim3((count + 255) / 256), dim3(256), 0, stream, "k_uniform_lists launch",
               (unsigned long long) reinterpret_cast<uintptr_t>(c), stride, size_n, count, c_list, n_stride, had_src);
    return "k_uniform_lists + " + launch_gemv_sliced(a, b_list, suh_list, a_had, svh_list, c_list, n_stride, had_src, count, count, size_m,
                                                      size_k, size_n, k_bits, codebook, out_fp32, sc, sms, stream,
                                                      per_matrix_input ? (long long) size_m * size_k : 0LL);
}

// Sliced multi-linear on the decode kernel: `n_slices` column slices of width size_n, cut from `num_had_src`
// matrices, all applied to the same size_m rows of `a`.  Every list is a DEVICE array (see GemvArgs).
std::string launch_gemv_sliced(const void* a, const void* b_list, const void* suh_list, void* a_had, const void* svh_list,
                               const void* c_list, const int* n_stride_list, const int* had_src_list, int num_had_src, int n_slices,
                               int size_m, int size_k, int size_n, int k_bits, int codebook, int out_fp32, const GemvScratch& sc,
                               int sms, cudaStream_t stream, long long a_src_stride)
{
    if (size_m > 32) throw std::runtime_error("exl3_mgemm: no linked kernel for size_m above 32");
    if (size_k % 128 != 0)
        throw std::runtime_error("exl3_mgemm: no linked kernel for size_k that is not a multiple of 128 (128-wide Hadamard)");
    const int tg = size_m <= 8 ? 1 : (size_m <= 16 ? 2 : 4);
    const int bu = k_bits <= 4 ? 2 : 1;
    if (size_n % (bu * 128) != 0)
        throw std::runtime_error("exl3_mgemm: no linked kernel for a slice width that is not a multiple of " + std::to_string(bu * 128));
    const int bands = size_n / 128, kblocks = size_k / 128, bgroups = bands / bu;
    if (size_t(num_had_src) * size_m * kblocks > sc.blocksum_floats)
        throw std::runtime_error("exl3_mgemm: sources x size_m x size_k / 128 exceed the block-sum table of the scratch");
    const size_t afrag_bytes = size_t(size_k / 16) * tg * 256;
    if (afrag_bytes * num_had_src > sc.afrag_bytes)
        throw std::runtime_error("exl3_mgemm: sources x size_k x ceil(size_m / 8) exceed the activation-fragment area of the scratch");
    const long long units = (long long) n_slices * bgroups * kblocks;
    int grid = int(std::min<long long>(sms, units));
    const size_t per_cta = size_t(2) * size_m * bu * 128 * sizeof(float);
    if (size_t(grid) * per_cta > sc.slab_bytes) grid = int(sc.slab_bytes / per_cta);
    if (grid < 1) throw std::runtime_error("exl3_mgemm: split-K scratch is too small for this shape");
    const int rot_total = 8 * tg * kblocks;
    launch_pdl(k_rotate_in, dim3(std::min((rot_total + 3) / 4, 4 * sms), num_had_src), dim3(128), 0, stream, "k_rotate_in launch",
               static_cast<const __half*>(a), (const __half*) nullptr, static_cast<__half*>(a_had), sc.afrag, sc.blocksum, size_m, 8 * tg,
               size_k, static_cast<const unsigned long long*>(suh_list), 0, a_src_stride, (const __half*) nullptr, 0.f);
    GemvArgs args{};
    args.defer_weights = weights_streamed() ? 1 : 0;
    args.afrag = sc.afrag;
    args.blocksum = sc.blocksum;
    args.a = nullptr; args.suh = nullptr; args.a_had = nullptr;
    args.c = nullptr;
    args.argmax = nullptr;
    args.residual = nullptr;
    args.svh = nullptr;
    args.problems = nullptr;
    args.n_problems = nullptr;
    args.max_problems = n_slices; args.n_matrices = 1; args.max_rows = size_m;
    args.slabs = sc.slabs;
    args.counters = nullptr;
    args.status = sc.status;
    args.m = size_m; args.k = size_k; args.n = size_n;
    args.out_fp32 = out_fp32;
    args.b_list = static_cast<const unsigned long long*>(b_list);
    args.svh_list = static_cast<const unsigned long long*>(svh_list);
    args.c_list = static_cast<const unsigned long long*>(c_list);
    args.n_stride_list = n_stride_list;
    args.had_src_list = had_src_list;
    args.n_slices = n_slices;
    args.n_stack = 0;
    const size_t smem = launch_bits(k_bits, codebook, tg, false, nullptr, 1, args, grid, stream);
    launch_finish(args, bu, 8 * tg, grid, codebook == 2 ? 1 : 0, stream);
    return "k_rotate_in x" + std::to_string(num_had_src) + " sources + k_exl3_gemv<" + std::to_string(k_bits) + "," + std::to_string(codebook) + "," +
           std::to_string(tg) + ",sliced> grid=" + std::to_string(grid) + " block=" + std::to_string(kThreads) + " smem=" +
           std::to_string(smem) + " + k_gemv_finish";
}

}  // namespace berth

// ------------------------------------------------------------------------------------------
// Decode linear for callers that must not allocate device memory.
//
// Who needs it: a host that has already handed every byte of HBM to its own planner (berth's
// placement plan budgets the whole device), or a decode loop that cannot afford the implicit
// device-wide synchronisation of cudaMalloc on its first launch.  The ordinary entry point
// creates its split-K workspace with cudaMalloc at the first launch on a device; this one
// keeps a fixed scratch area inside the library image instead, so it never calls cudaMalloc,
// cudaFree or any allocating routine.
//
// The scratch is one file-scope __device__ array: 4 MiB of fp32 partial-sum slabs, 2 MiB for the
// rotated activations in fragment order, one fp32 block sum per (row, 128 inputs) (128 KiB), 16 KiB of
// band-group arrival counters and a status word (which berth_device_status reads and clears together with
// the ordinary workspace's).  At 17..32 rows the 4 MiB of slabs hold the partial sums of 64 CTAs, so the
// launch runs on 64 SMs there; up to 16 rows it takes the whole GPU.  Every GPU that loads the library carries it until the process exits.  All calls on
// a device share it and it keeps whatever the previous call left behind: nothing needs clearing,
// slabs, fragments and block sums are fully overwritten before they are read.  Two calls that
// overlap on the GPU (different streams) race on it; issue them on one stream.
namespace berth {
namespace {

constexpr size_t kStaticSlabBytes = size_t(4) << 20;   // 4 MiB of split-K partial sums
constexpr int kStaticMaxBands = 1024;                  // size_n <= 131072
constexpr int kStaticMaxRows = 32;
constexpr int kStaticMaxKBlocks = 1024;                // size_k <= 131072
constexpr size_t kStaticBlocksumBytes = size_t(kStaticMaxRows) * kStaticMaxKBlocks * sizeof(float);
constexpr size_t kStaticAfragBytes = size_t(2) << 20;   // size_k * ceil(size_m / 8) <= 131072
constexpr size_t kStaticCounterWords = 4096;             // band groups of the integer tensor path

static __device__ __align__(256) unsigned char g_static_scratch[kStaticSlabBytes + kStaticAfragBytes + kStaticBlocksumBytes + kStaticCounterWords * 4 + 256];

GemvScratch g_static_ptr[kMaxDevices];
std::mutex g_static_mu;

// The array's name is only a host-side handle; the device address has to be asked for, once
// per device, while that device is current.
GemvScratch static_scratch(int device)
{
    std::lock_guard<std::mutex> lock(g_static_mu);
    GemvScratch& s = g_static_ptr[device];
    if (!s.slabs) {
        void* base = nullptr;
        cuda_ok(cudaGetSymbolAddress(&base, g_static_scratch), "cudaGetSymbolAddress(static scratch)");
        if (!base) throw std::runtime_error("exl3 linear (static scratch): symbol address is null");
        unsigned char* b = static_cast<unsigned char*>(base);
        s.slabs = reinterpret_cast<float*>(b);
        s.slab_bytes = kStaticSlabBytes;
        b += kStaticSlabBytes;
        s.afrag = reinterpret_cast<uint32_t*>(b);
        s.afrag_bytes = kStaticAfragBytes;
        b += kStaticAfragBytes;
        s.blocksum = reinterpret_cast<float*>(b);
        s.blocksum_floats = size_t(kStaticMaxRows) * kStaticMaxKBlocks;
        b += kStaticBlocksumBytes;
        s.counters = reinterpret_cast<unsigned*>(b);   // (a __device__ array starts out zeroed)
        s.counter_words = kStaticCounterWords;
        b += kStaticCounterWords * 4;
        s.status = reinterpret_cast<unsigned*>(b);
    }
    return s;
}

}  // namespace

// Status word of the fixed in-image scratch on `device`: read and cleared (0 if the entry point was never used there).
int read_static_status(int device)
{
    GemvScratch s;
    {
        std::lock_guard<std::mutex> lock(g_static_mu);
        s = g_static_ptr[device];
    }
    if (!s.status) return 0;
    unsigned v = 0;
    cuda_ok(cudaMemcpy(&v, s.status, sizeof v, cudaMemcpyDeviceToHost), "static status read");
    if (v) cuda_ok(cudaMemset(s.status, 0, sizeof v), "static status clear");
    return int(v);
}
}  // namespace berth

extern "C" int berth_exl3_linear_static_scratch(const void* a, const void* trellis, void* c, const void* suh,
                                                void* a_had, const void* svh, int size_m, int size_k, int size_n,
                                                int k_bits, int codebook, int out_fp32, void* stream)
{
    using namespace berth;
    CallState& st = exl3_state();
    return guarded(st, [&] {
        if (!a || !trellis || !c || !suh || !a_had || !svh) throw std::runtime_error("exl3 linear: null device pointer");
        if (size_m < 1 || size_k < 1 || size_n < 1) throw std::runtime_error("exl3 linear: sizes must be positive");
        if (k_bits < 1 || k_bits > 8) throw std::runtime_error("exl3 linear: K must be in 1..=8");
        if (codebook < 0 || codebook > 2)
            throw std::runtime_error("exl3 linear: codebook must be 0 (default), 1 (mcg), or 2 (mul1)");
        if (size_k % 16 != 0) throw std::runtime_error("exl3 linear: size_k must be a multiple of 16");
        if (size_n % 128 != 0) throw std::runtime_error("exl3 linear: size_n must be a multiple of 128");
        if (size_m > kStaticMaxRows)
            throw std::runtime_error("exl3 linear (static scratch): size_m " + std::to_string(size_m) +
                                     " exceeds the maximum of " + std::to_string(kStaticMaxRows) + " rows");
        if (size_n / 128 > kStaticMaxBands)
            throw std::runtime_error("exl3 linear (static scratch): size_n " + std::to_string(size_n) +
                                     " exceeds the maximum of " + std::to_string(kStaticMaxBands * 128) + " columns");
        // rows are processed in groups of 8, 16 or 32 (as launch_gemv does); the rotated rows of a group share the 2 MiB area
        const int row_groups = size_m <= 8 ? 1 : (size_m <= 16 ? 2 : 4);
        if (size_k / 128 > kStaticMaxKBlocks || size_t(size_k) * row_groups > 131072)
            throw std::runtime_error("exl3 linear (static scratch): size_k " + std::to_string(size_k) + " with " +
                                     std::to_string(size_m) + " rows exceeds the maximum of size_k * g <= 131072 (g = 1, 2, 4 for up to 8, 16, 32 rows)");
        const int device = current_device();
        const DeviceInfo& info = device_info(device);
        if (info.major != 10)
            throw std::runtime_error("exl3 linear: no linked kernel for this GPU (library is built for sm_100a only)");
        GemvScratch s = static_scratch(device);
        cudaStream_t cs = (cudaStream_t) stream;
        st.launch = launch_gemv(a, trellis, c, suh, a_had, svh, size_m, size_k, size_n, k_bits, codebook, out_fp32, s,
                                info.sms, cs) + " static-scratch";
    });
}
