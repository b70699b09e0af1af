// A3B-style mixture-of-experts layer on top of the grouped decode kernel: router (fixed-order
// fp32 logits, warp top-k with ties to the lower expert index, softmax over the selection),
// dispatch (per-expert count, exclusive scan, stable permutation, row gather, problem table),
// grouped gate/up/SiLU/down over the routed rows, weighted combine plus shared expert.
// berth has the shape contract of this block but no operator; the arithmetic contract is the
// one the CPU checker under oracle/ states (router summation order, tie rule, rounding points).
#include "exl3_decode.cuh"
#include "../../include/berth_b200.h"

#include <algorithm>

namespace berth {

std::string linear_rows(const void* a, const void* trellis, void* c, const void* suh, void* a_had, const void* svh,
                        int size_m, int size_k, int size_n, int k_bits, int codebook, int out_fp32, cudaStream_t stream);
void silu_mul_rows(const void* gate, const void* up, void* out, const int* n_rows, int max_rows, int row_elems, cudaStream_t stream);

namespace {

// ---------------------------------------------------------------- router
// logits[t][e] = sum over 32 chunks of H/32 sequential fmaf, chunks combined by a halving tree
// ((p0+p16)+(p8+p24))+...: the summation order of the CPU checker, so the top-k indices can be
// compared bit for bit.  Block = 16 warps x 32 experts for kRouterTok tokens: a warp accumulates
// chunks j and j+16 with coalesced reads of the router rows (each row read once per token tile).
constexpr int kRouterTok = 8;
// The halving tree over the 32 chunk sums, p[c] at base[c * kRouterTok * 33]: V(c, 32) = p[c],
// V(c, s) = V(c, 2s) + V(c + s, 2s), result V(0, 1) -- evaluated depth first, a handful of registers.
template <int S>
__device__ __forceinline__ float chunk_tree(const float* base, int c)
{
    if constexpr (S == 32) return base[c * (kRouterTok * 33)];
    else return __fadd_rn(chunk_tree<2 * S>(base, c), chunk_tree<2 * S>(base, c + S));
}
// Dynamic shared memory: the token tile as fp32 [kRouterTok][H], then the chunk sums [32][kRouterTok][33].
// WARPS = 16: each warp accumulates two of the 32 chunks, one after the other; 512 threads and ~97 KiB per block,
// so that two blocks share an SM and one block's load and reduction phases overlap the other's arithmetic.
// WARPS = 32: one chunk per warp, for launches of fewer blocks than SMs, which the latency of a chunk's loads bounds.
template <int WARPS>
__global__ void __launch_bounds__(WARPS * 32, WARPS == 16 ? 2 : 1) k_moe_router_logits(const __half* __restrict__ x, const __half* __restrict__ w,
                                                                            const float* __restrict__ bias, float* __restrict__ logits,
                                                                            int T, int H, int E)
{
    pdl_trigger();   // launched as a programmatic dependent: let the successor become resident, then wait for the predecessor
    pdl_wait();
    extern __shared__ __align__(16) float rsm[];
    float* xs = rsm;                                                    // [kRouterTok][H]
    float (*part)[kRouterTok][33] = reinterpret_cast<float (*)[kRouterTok][33]>(rsm + kRouterTok * H);
    const int wq = threadIdx.x >> 5, el = threadIdx.x & 31;
    const int e = blockIdx.x * 32 + el, t0 = blockIdx.y * kRouterTok;
    const int chunk = H / 32;
    // the tile's activations, converted once (rows past T repeat the last token; their sums are never stored)
    for (int i = threadIdx.x * 2; i < kRouterTok * H; i += WARPS * 64) {
        const int tt = i / H, h = i - tt * H;
        const __half2 v = *reinterpret_cast<const __half2*>(x + size_t(min(t0 + tt, T - 1)) * H + h);
        xs[i] = __low2float(v);
        xs[i + 1] = __high2float(v);
    }
    __syncthreads();
    const int vec_end = (chunk & 3) == 0 ? chunk : 0;   // quads are 16-byte aligned only if the chunk is a multiple of 4
    for (int j = wq; j < 32; j += WARPS) {
        const __half* wr = w + size_t(j) * chunk * E + e;
        const float* xj = xs + j * chunk;
        float acc[kRouterTok];
#pragma unroll
        for (int tt = 0; tt < kRouterTok; ++tt) acc[tt] = 0.f;
        // eight router rows in flight per pass, the next eight already requested; the products are still
        // added one by one in k order
        int i0 = 0;
        __half nxt[8];
        if (8 <= vec_end) {
#pragma unroll
            for (int ii = 0; ii < 8; ++ii) nxt[ii] = wr[size_t(ii) * E];
        }
        for (; i0 + 8 <= vec_end; i0 += 8) {
            float wv[8];
#pragma unroll
            for (int ii = 0; ii < 8; ++ii) wv[ii] = __half2float(nxt[ii]);
            if (i0 + 16 <= vec_end) {
#pragma unroll
                for (int ii = 0; ii < 8; ++ii) nxt[ii] = wr[size_t(i0 + 8 + ii) * E];
            }
#pragma unroll
            for (int tt = 0; tt < kRouterTok; ++tt) {
                const float4 a = *reinterpret_cast<const float4*>(xj + tt * H + i0);
                const float4 b = *reinterpret_cast<const float4*>(xj + tt * H + i0 + 4);
                acc[tt] = __fmaf_rn(a.x, wv[0], acc[tt]); acc[tt] = __fmaf_rn(a.y, wv[1], acc[tt]);
                acc[tt] = __fmaf_rn(a.z, wv[2], acc[tt]); acc[tt] = __fmaf_rn(a.w, wv[3], acc[tt]);
                acc[tt] = __fmaf_rn(b.x, wv[4], acc[tt]); acc[tt] = __fmaf_rn(b.y, wv[5], acc[tt]);
                acc[tt] = __fmaf_rn(b.z, wv[6], acc[tt]); acc[tt] = __fmaf_rn(b.w, wv[7], acc[tt]);
            }
        }
        for (; i0 < chunk; ++i0) {   // the rest, or all of it for an odd chunk
            const float wv = __half2float(wr[size_t(i0) * E]);
#pragma unroll
            for (int tt = 0; tt < kRouterTok; ++tt) acc[tt] = __fmaf_rn(xj[tt * H + i0], wv, acc[tt]);
        }
#pragma unroll
        for (int tt = 0; tt < kRouterTok; ++tt) part[j][tt][el] = acc[tt];
    }
    __syncthreads();
    // warp tt reduces token tt: lane = expert; the same halving tree as a 32-lane xor butterfly's lane 0
    if (wq < kRouterTok && t0 + wq < T) {
        logits[size_t(t0 + wq) * E + e] = __fadd_rn(chunk_tree<1>(&part[0][wq][el], 0), bias ? bias[e] : 0.f);
    }
}

// The same sums for launches that fill the GPU: 128 experts x kRouterTok tokens per block, a lane holds four experts
// (2l, 2l+1, 64+2l, 65+2l of the block's 128), so one broadcast read of the token tile feeds four multiply-adds
// instead of one -- the narrow kernel above is bound by those shared-memory reads, not by arithmetic.  Warp w adds
// chunks w and w+16, which is the first level of the halving tree; the remaining 16-leaf tree runs at the end.
constexpr int kWidePitch = 132;   // floats per (chunk pair, token) row of the partial sums
template <int S>
__device__ __forceinline__ float chunk_tree16(const float* base, int c)
{
    if constexpr (S == 16) return base[c * (kRouterTok * kWidePitch)];
    else return __fadd_rn(chunk_tree16<2 * S>(base, c), chunk_tree16<2 * S>(base, c + S));
}
__global__ void __launch_bounds__(512, 1) k_moe_router_logits_wide(const __half* __restrict__ x, const __half* __restrict__ w,
                                                                   const float* __restrict__ bias, float* __restrict__ logits,
                                                                   int T, int H, int E)
{
    pdl_trigger();   // launched as a programmatic dependent: let the successor become resident, then wait for the predecessor
    pdl_wait();
    extern __shared__ __align__(16) float rsm[];
    float* xs = rsm;                              // [kRouterTok][H]
    float* part = rsm + kRouterTok * H;           // [16][kRouterTok][kWidePitch]
    const int wq = threadIdx.x >> 5, el = threadIdx.x & 31;
    const int e0 = blockIdx.x * 128, t0 = blockIdx.y * kRouterTok;
    const int chunk = H / 32;                     // a multiple of 8 (checked by the host)
    for (int i = threadIdx.x * 2; i < kRouterTok * H; i += 1024) {
        const int tt = i / H, h = i - tt * H;
        const __half2 v = *reinterpret_cast<const __half2*>(x + size_t(min(t0 + tt, T - 1)) * H + h);
        xs[i] = __low2float(v);
        xs[i + 1] = __high2float(v);
    }
    __syncthreads();
    for (int half = 0; half < 2; ++half) {
        const int j = wq + 16 * half;
        const __half* wr = w + size_t(j) * chunk * E + e0 + 2 * el;
        const float* xj = xs + j * chunk;
        float acc[kRouterTok][4];
#pragma unroll
        for (int tt = 0; tt < kRouterTok; ++tt) acc[tt][0] = acc[tt][1] = acc[tt][2] = acc[tt][3] = 0.f;
        uint32_t nxt[8][2];
#pragma unroll
        for (int ii = 0; ii < 8; ++ii) {
            nxt[ii][0] = *reinterpret_cast<const uint32_t*>(wr + size_t(ii) * E);
            nxt[ii][1] = *reinterpret_cast<const uint32_t*>(wr + size_t(ii) * E + 64);
        }
        for (int i0 = 0; i0 < chunk; i0 += 8) {
            float wv[8][4];
#pragma unroll
            for (int ii = 0; ii < 8; ++ii) {
                const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&nxt[ii][0]));
                const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&nxt[ii][1]));
                wv[ii][0] = lo.x; wv[ii][1] = lo.y; wv[ii][2] = hi.x; wv[ii][3] = hi.y;
            }
            if (i0 + 8 < chunk) {
#pragma unroll
                for (int ii = 0; ii < 8; ++ii) {
                    nxt[ii][0] = *reinterpret_cast<const uint32_t*>(wr + size_t(i0 + 8 + ii) * E);
                    nxt[ii][1] = *reinterpret_cast<const uint32_t*>(wr + size_t(i0 + 8 + ii) * E + 64);
                }
            }
#pragma unroll
            for (int tt = 0; tt < kRouterTok; ++tt) {
                const float4 a = *reinterpret_cast<const float4*>(xj + tt * H + i0);
                const float4 b = *reinterpret_cast<const float4*>(xj + tt * H + i0 + 4);
                const float xv[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
                for (int ii = 0; ii < 8; ++ii) {   // k ascending for every accumulator: the checker's order
#pragma unroll
                    for (int q = 0; q < 4; ++q) acc[tt][q] = __fmaf_rn(xv[ii], wv[ii][q], acc[tt][q]);
                }
            }
        }
        // first tree level: chunk w + chunk w+16 (only this warp touches these rows)
#pragma unroll
        for (int tt = 0; tt < kRouterTok; ++tt) {
            float* row = part + (wq * kRouterTok + tt) * kWidePitch;
            float2 lo = make_float2(acc[tt][0], acc[tt][1]), hi = make_float2(acc[tt][2], acc[tt][3]);
            if (half) {
                const float2 plo = *reinterpret_cast<const float2*>(row + 2 * el), phi = *reinterpret_cast<const float2*>(row + 64 + 2 * el);
                lo = make_float2(__fadd_rn(plo.x, lo.x), __fadd_rn(plo.y, lo.y));
                hi = make_float2(__fadd_rn(phi.x, hi.x), __fadd_rn(phi.y, hi.y));
            }
            *reinterpret_cast<float2*>(row + 2 * el) = lo;
            *reinterpret_cast<float2*>(row + 64 + 2 * el) = hi;
        }
    }
    __syncthreads();
    // warp tt finishes token tt: lane = four experts
    if (wq < kRouterTok && t0 + wq < T) {
        const float* base = part + wq * kWidePitch;
        float* out = logits + size_t(t0 + wq) * E + e0;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int col = (q >> 1) * 64 + 2 * el + (q & 1);
            out[col] = __fadd_rn(chunk_tree16<1>(base + col, 0), bias ? bias[e0 + col] : 0.f);
        }
    }
}

// One warp per token: k rounds of arg-max, value descending then index ascending.
__global__ void __launch_bounds__(128) k_moe_topk(const float* __restrict__ logits, int32_t* __restrict__ topk_idx,
                                                  float* __restrict__ topk_w, int T, int E, int k)
{
    pdl_trigger();   // launched as a programmatic dependent: let the successor become resident, then wait for the predecessor
    pdl_wait();
    const int t = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= T) return;
    const float* l = logits + size_t(t) * E;
    constexpr int kMaxPerLane = 32;   // E <= 1024
    float v[kMaxPerLane];
    const int per = (E + 31) / 32;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) v[i] = (i < per && lane + 32 * i < E) ? l[lane + 32 * i] : -INFINITY;
    unsigned taken = 0;   // bit i: this lane's i-th expert already selected
    float first = 0.f, mine = 0.f, sum = 0.f;
    for (int s = 0; s < k; ++s) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < kMaxPerLane; ++i)
            if (i < per && !((taken >> i) & 1u) && lane + 32 * i < E) {
                const int idx = lane + 32 * i;
                if (v[i] > bv || (v[i] == bv && idx < bi)) { bv = v[i]; bi = idx; }
            }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            const float ov = __shfl_xor_sync(dq::kFull, bv, off);
            const int oi = __shfl_xor_sync(dq::kFull, bi, off);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (bi == 0x7fffffff) {
            // nothing compared greater than -inf: what is left of the row is NaN (or the row is all -inf).  Take the lowest
            // expert not selected yet, so that the k indices are always distinct and inside [0, E): the dispatch and
            // combine kernels index arrays with them.
            int fi = 0x7fffffff;
#pragma unroll
            for (int i = kMaxPerLane - 1; i >= 0; --i)
                if (i < per && !((taken >> i) & 1u) && lane + 32 * i < E) fi = lane + 32 * i;
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) fi = min(fi, __shfl_xor_sync(dq::kFull, fi, off));
            bi = fi;
        }
        if ((bi & 31) == lane) taken |= 1u << (bi >> 5);
        if (s == 0) first = bv;
        const float ex = expf(bv - first);
        sum += ex;
        if (lane == s) mine = ex;      // k <= 32
        if (lane == 0) topk_idx[size_t(t) * k + s] = bi;
    }
    if (lane < k) topk_w[size_t(t) * k + lane] = mine / sum;
}

// Status bits of the expert stage: a peer's flag never arrived; rows did not fit a receive buffer or a problem table.
enum : unsigned { kStEpTimeout = 32u, kStEpOverflow = 64u };

// ---------------------------------------------------------------- dispatch
// counts[j] = number of entries whose key is e0 + j.  One block per local expert.
__global__ void __launch_bounds__(256) k_moe_count(const int32_t* __restrict__ keys, int n, int e0, int* __restrict__ counts)
{
    pdl_trigger();   // launched as a programmatic dependent: let the successor become resident, then wait for the predecessor
    pdl_wait();
    const int e = e0 + blockIdx.x;
    int c = 0;
    for (int i = threadIdx.x; i < n; i += 256) c += (keys[i] == e);
    __shared__ int red[8];
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) c += __shfl_xor_sync(dq::kFull, c, off);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
        int s = 0;
        for (int i = 0; i < 8; ++i) s += red[i];
        counts[blockIdx.x] = s;
    }
}

// offsets[0..n_local] = exclusive scan of counts; problem table: every expert's rows in chunks of
// `chunk` rows, experts in ascending order.  One block of 1024 threads, one expert per thread.
// With extra_rows > 0 one more matrix (index n_local, the shared expert held behind the stack) takes
// extra_rows rows after the routed ones: offsets[n_local + 1] then ends the table.
// (scan_problems: the body, for a block of 1024 threads where thread j brings expert j's count; returns the
// expert's first row.)
// pair_rows > 0: the table is written twice, the second copy behind the first with every matrix index raised by
// pair_matrices and every first row by pair_rows, and n_problems[1] = the doubled count: one grouped launch over the
// doubled table then runs two stacks that lie behind one another (gate and up) on the same rows.
// max_problems / max_rows: capacity of one copy of the table and of the row arrays.  Counts that ask for more (a skewed
// exchange that delivered more rows than the caller sized the stage for) are cut there -- entries past the table are
// not written, first rows stay inside the arrays -- and kStEpOverflow is raised in `status`: wrong numbers with a status
// bit, never a write past the table.
__device__ __forceinline__ int scan_problems(int c_routed, int* __restrict__ offsets, GemvProblem* __restrict__ problems,
                                             int* __restrict__ n_problems, int n_routed, int chunk, int extra_rows, int pair_rows,
                                             int pair_matrices, int max_problems, int max_rows, unsigned* status)
{
    __shared__ int wrows[32], wprob[32];
    const int j = threadIdx.x, lane = j & 31, warp = j >> 5;
    const int n_local = n_routed + (extra_rows > 0 ? 1 : 0);
    const int c = j < n_routed ? c_routed : (j < n_local ? extra_rows : 0);
    const int np = (c + chunk - 1) / chunk;
    int prow = c, pprob = np;     // inclusive warp scans
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int a = __shfl_up_sync(dq::kFull, prow, off), b = __shfl_up_sync(dq::kFull, pprob, off);
        if (lane >= off) { prow += a; pprob += b; }
    }
    if (lane == 31) { wrows[warp] = prow; wprob[warp] = pprob; }
    __syncthreads();
    if (warp == 0) {
        int a = wrows[lane], b = wprob[lane];
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int ua = __shfl_up_sync(dq::kFull, a, off), ub = __shfl_up_sync(dq::kFull, b, off);
            if (lane >= off) { a += ua; b += ub; }
        }
        wrows[lane] = a; wprob[lane] = b;
    }
    __syncthreads();
    const int row0 = prow - c + (warp ? wrows[warp - 1] : 0);
    const int p0 = pprob - np + (warp ? wprob[warp - 1] : 0);
    const int total = min(wprob[31], max_problems);   // problems of one copy that fit the table
    if (j < n_local) {
        offsets[j] = min(row0, max_rows);
        for (int i = 0; i < np && p0 + i < max_problems; ++i) {
            GemvProblem pr;
            pr.z = j; pr.row0 = row0 + i * chunk; pr.rows = min(chunk, c - i * chunk); pr.pad = 0;
            if (pr.row0 + pr.rows > max_rows) {   // rows past the arrays: cut the problem (load_problem clamps the rest)
                pr.rows = max(0, max_rows - pr.row0);
                pr.row0 = min(pr.row0, max_rows);
            }
            problems[p0 + i] = pr;
            if (pair_rows > 0) {
                pr.z += pair_matrices; pr.row0 += pair_rows;
                problems[total + p0 + i] = pr;
            }
        }
    }
    if (j == 0) {
        offsets[n_local] = min(wrows[31], max_rows);
        n_problems[0] = total;
        n_problems[1] = pair_rows > 0 ? 2 * total : 0;
        if ((wprob[31] > max_problems || wrows[31] > max_rows) && status) atomicOr(status, kStEpOverflow);
    }
    return row0;
}

__global__ void __launch_bounds__(1024) k_moe_scan(const int* __restrict__ counts, int* __restrict__ offsets,
                                                   GemvProblem* __restrict__ problems, int* __restrict__ n_problems,
                                                   int n_routed, int chunk, int extra_rows, int pair_rows, int pair_matrices,
                                                   int max_problems, int max_rows, unsigned* status)
{
    pdl_trigger();   // launched as a programmatic dependent: let the successor become resident, then wait for the predecessor
    pdl_wait();
    scan_problems(threadIdx.x < n_routed ? counts[threadIdx.x] : 0, offsets, problems, n_problems, n_routed, chunk, extra_rows, pair_rows,
                  pair_matrices, max_problems, max_rows, status);
}

// Count, scan and stable scatter in one block for a short key list (n <= kSmallKeys).  Warp 0 walks the keys 32 at
// a time: lanes with the same key find one another with match.any, an entry's rank within its expert is the
// expert's running count plus the equal keys in lower lanes.  Then thread j scans expert j's count and every entry
// goes to its expert's first row plus its rank.  Same outputs as k_moe_count + k_moe_scan + k_moe_scatter.
constexpr int kSmallKeys = 2048;
__global__ void __launch_bounds__(1024) k_moe_dispatch_small(const int32_t* __restrict__ keys, int n, int e0, int* __restrict__ counts,
                                                             int* __restrict__ offsets, GemvProblem* __restrict__ problems,
                                                             int* __restrict__ n_problems, int n_routed, int chunk, int extra_rows,
                                                             int pair_rows, int pair_matrices, int32_t* __restrict__ perm,
                                                             int32_t* __restrict__ inv, int max_problems, int max_rows, unsigned* status)
{
    pdl_trigger();   // launched as a programmatic dependent: let the successor become resident, then wait for the predecessor
    pdl_wait();
    __shared__ int s_slot[kSmallKeys], s_rank[kSmallKeys], s_cnt[1025], s_row0[1024];
    const int j = threadIdx.x, lane = j & 31;
    for (int i = j; i < n; i += blockDim.x) {
        const int key = keys[i] - e0;
        s_slot[i] = (key >= 0 && key < n_routed) ? key : n_routed;   // slot n_routed collects the keys of other ranks
    }
    if (j <= n_routed) s_cnt[j] = 0;
    __syncthreads();
    if (j < 32) {
        for (int base = 0; base < n; base += 32) {
            const int i = base + lane;
            const int slot = i < n ? s_slot[i] : n_routed;
            const unsigned same = __match_any_sync(dq::kFull, slot);
            const int before = s_cnt[slot];
            __syncwarp();
            if (lane == __ffs(same) - 1) s_cnt[slot] = before + __popc(same);
            __syncwarp();
            if (i < n) s_rank[i] = before + __popc(same & ((1u << lane) - 1u));
        }
    }
    __syncthreads();
    const int c = j < n_routed ? s_cnt[j] : 0;
    if (j < n_routed) counts[j] = c;
    const int row0 = scan_problems(c, offsets, problems, n_problems, n_routed, chunk, extra_rows, pair_rows, pair_matrices, max_problems,
                                   max_rows, status);
    if (j < n_routed) s_row0[j] = row0;
    __syncthreads();
    for (int i = j; i < n; i += blockDim.x) {
        const int slot = s_slot[i];
        if (slot < n_routed) {
            const int pos = s_row0[slot] + s_rank[i];
            perm[pos] = i;
            inv[i] = pos;
        }
    }
}

// Stable permutation: block j walks the entries in order, 1024 at a time; the r-th entry with key e0 + j goes to
// position offsets[j] + r.  perm[pos] = entry, inv[entry] = pos.
__global__ void __launch_bounds__(1024) k_moe_scatter(const int32_t* __restrict__ keys, int n, int e0,
                                                      const int* __restrict__ offsets, int32_t* __restrict__ perm,
                                                      int32_t* __restrict__ inv)
{
    pdl_trigger();   // launched as a programmatic dependent: let the successor become resident, then wait for the predecessor
    pdl_wait();
    const int e = e0 + blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __shared__ int wsum[2][32];   // per-warp hit counts, double buffered: one barrier per pass
    int running = offsets[blockIdx.x];
    int buf = 0;
    for (int base = 0; base < n; base += 1024, buf ^= 1) {
        const int i = base + threadIdx.x;
        const bool hit = i < n && keys[i] == e;
        const unsigned ballot = __ballot_sync(dq::kFull, hit);
        if (lane == 0) wsum[buf][warp] = __popc(ballot);
        __syncthreads();
        // every warp reduces the 32 counts: lanes below the warp's index give the hits before it
        const int c = wsum[buf][lane];
        int before = lane < warp ? c : 0, total = c;
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            before += __shfl_xor_sync(dq::kFull, before, off);
            total += __shfl_xor_sync(dq::kFull, total, off);
        }
        if (hit) {
            const int pos = running + before + __popc(ballot & ((1u << lane) - 1u));
            perm[pos] = i;
            inv[i] = pos;
        }
        running += total;
    }
}

// xr[pos][:] = x[perm[pos] / div][:]  (div = top_k when entries are (token, slot) pairs).
__global__ void __launch_bounds__(256) k_moe_gather_rows(const __half* __restrict__ x, const int32_t* __restrict__ perm,
                                                         const int* __restrict__ n_rows, int div, __half* __restrict__ xr, int H)
{
    pdl_trigger();   // launched as a programmatic dependent: let the successor become resident, then wait for the predecessor
    pdl_wait();
    const int R = __ldg(n_rows);
    for (int pos = blockIdx.x; pos < R; pos += gridDim.x) {
        const uint4* src = reinterpret_cast<const uint4*>(x + size_t(perm[pos] / div) * H);
        uint4* dst = reinterpret_cast<uint4*>(xr + size_t(pos) * H);
        for (int i = threadIdx.x; i < H / 8; i += 256) dst[i] = src[i];
    }
}

// Same with the row count known on the host.
__global__ void __launch_bounds__(256) k_moe_gather_n(const __half* __restrict__ x, const int32_t* __restrict__ index, int n,
                                                      int div, __half* __restrict__ dst, int H)
{
    pdl_trigger();   // launched as a programmatic dependent: let the successor become resident, then wait for the predecessor
    pdl_wait();
    for (int pos = blockIdx.x; pos < n; pos += gridDim.x) {
        const uint4* src = reinterpret_cast<const uint4*>(x + size_t(index[pos] / div) * H);
        uint4* d = reinterpret_cast<uint4*>(dst + size_t(pos) * H);
        for (int i = threadIdx.x; i < H / 8; i += 256) d[i] = src[i];
    }
}

// out[t][h] = sum_s w[t][s] * y[inv[t*k+s]][h]  (fmaf chain in slot order)  + ysh[t][h]
__global__ void __launch_bounds__(256) k_moe_combine(const __half* __restrict__ y, const int32_t* __restrict__ inv,
                                                     const float* __restrict__ topk_w, const __half* __restrict__ ysh,
                                                     float* __restrict__ out, int H, int k, int n_rows)
{
    pdl_trigger();   // launched as a programmatic dependent: let the successor become resident, then wait for the predecessor
    pdl_wait();
    // block = (token, 512 columns); the token's row positions and weights first, so that the k row reads of a column
    // pair are independent loads.  Positions are forced into [0, n_rows): a stale index array gives wrong numbers, never
    // a wild address.
    __shared__ int s_pos[32];
    __shared__ float s_w[32];
    const int t = blockIdx.x;
    if (threadIdx.x < k) {
        s_pos[threadIdx.x] = min(max(inv[size_t(t) * k + threadIdx.x], 0), n_rows - 1);
        s_w[threadIdx.x] = topk_w[size_t(t) * k + threadIdx.x];
    }
    __syncthreads();
    const int h = blockIdx.y * 512 + threadIdx.x * 2;
    if (h >= H) return;
    float a0 = 0.f, a1 = 0.f;
    for (int s0 = 0; s0 < k; s0 += 8) {
        __half2 v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (s0 + i < k) v[i] = *reinterpret_cast<const __half2*>(y + size_t(s_pos[s0 + i]) * H + h);
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (s0 + i < k) {   // fmaf chain in slot order
                a0 = __fmaf_rn(s_w[s0 + i], __low2float(v[i]), a0);
                a1 = __fmaf_rn(s_w[s0 + i], __high2float(v[i]), a1);
            }
    }
    if (ysh) {
        const __half2 v = *reinterpret_cast<const __half2*>(ysh + size_t(t) * H + h);
        a0 = __fadd_rn(a0, __low2float(v));
        a1 = __fadd_rn(a1, __high2float(v));
    }
    *reinterpret_cast<float2*>(out + size_t(t) * H + h) = make_float2(a0, a1);
}

// Expert-parallel receive side: the rows of source s arrive sorted by local expert, cnt[s][e] of them per
// expert.  seg_off[i] = first row of segment i = s * n_local + e (exclusive scan, one block, up to 1024 segments).
__global__ void __launch_bounds__(1024) k_moe_segment_scan(const int32_t* __restrict__ cnt, int n_seg, int* __restrict__ seg_off)
{
    __shared__ int wsum[32];
    const int j = threadIdx.x, lane = j & 31, warp = j >> 5;
    const int c = j < n_seg ? max(cnt[j], 0) : 0;
    int incl = c;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int a = __shfl_up_sync(dq::kFull, incl, off);
        if (lane >= off) incl += a;
    }
    if (lane == 31) wsum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int a = wsum[lane];
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int u = __shfl_up_sync(dq::kFull, a, off);
            if (lane >= off) a += u;
        }
        wsum[lane] = a;
    }
    __syncthreads();
    if (j < n_seg) seg_off[j] = incl - c + (warp ? wsum[warp - 1] : 0);
    if (j == 0) seg_off[n_seg] = wsum[31];
}
// keys[row] = local expert of the row: block = segment.
__global__ void __launch_bounds__(128) k_moe_segment_keys(const int* __restrict__ seg_off, int n_local, int max_rows, int32_t* __restrict__ keys)
{
    const int seg = blockIdx.x, e = seg % n_local;
    const int r0 = seg_off[seg], r1 = min(seg_off[seg + 1], max_rows);
    for (int r = r0 + threadIdx.x; r < r1; r += 128) keys[r] = e;
}

// ---------------------------------------------------------------- expert parallelism over peer memory
// The ranks of one NVSwitch box exchange routed rows and expert outputs with plain stores into each other's
// memory (symmetric buffers whose per-rank addresses the host passes in) and three flag barriers per layer;
// no collective library call and no host synchronisation.  Every wait on a peer is bounded: when it runs out
// it sets a status bit and the layer carries on with whatever is there.
constexpr int kMaxPeers = 8;
struct PeerPtrs { void* p[kMaxPeers]; };

// Thread s < W: tell rank s that this rank has reached `phase` of layer call `epoch`, then wait for rank s to
// say the same.  flags: uint32 [3 phases][kMaxPeers sources] on every rank.  Everything this block wrote to
// peer memory before the call is visible to a peer that has seen the flag.
__device__ __forceinline__ void ep_signal_and_wait(const PeerPtrs& flags, int phase, int rank, int W, unsigned epoch, unsigned* status)
{
    __threadfence_system();
    __syncthreads();
    const int s = threadIdx.x;
    if (s < W) {
        volatile unsigned* remote = static_cast<volatile unsigned*>(flags.p[s]) + phase * kMaxPeers + rank;
        *remote = epoch;
        volatile unsigned* mine = static_cast<volatile unsigned*>(flags.p[rank]) + phase * kMaxPeers + s;
        bool ok = false;
        for (unsigned i = 0; i < (1u << 22); ++i) {
            if (int(*mine - epoch) >= 0) { ok = true; break; }
            __nanosleep(100);
        }
        if (!ok) atomicOr(status, kStEpTimeout);
        __threadfence_system();
    }
    __syncthreads();
}

// Exclusive scan of one value per thread over a block of 1024 (value 0 beyond n); returns the prefix, total in *total.
__device__ __forceinline__ int block_exclusive_scan(int v, int* wsum /*[32] shared*/, int* total)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int a = __shfl_up_sync(dq::kFull, incl, off);
        if (lane >= off) incl += a;
    }
    __syncthreads();   // wsum may still be read from an earlier call
    if (lane == 31) wsum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int a = wsum[lane];
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int u = __shfl_up_sync(dq::kFull, a, off);
            if (lane >= off) a += u;
        }
        wsum[lane] = a;
    }
    __syncthreads();
    if (total) *total = wsum[31];
    return incl - v + (warp ? wsum[warp - 1] : 0);
}

// Publish this rank's rows-per-expert to every rank (cnt_all [W][E] on each), barrier 0, then build from the
// full matrix (one block of 1024 threads, E <= 1024):
//   dst0[e]         first row, in the owner's receive buffer, of this rank's rows for expert e
//                   (the owner holds expert blocks in order, each block source by source);
//   counts_local[j] rows arriving here for local expert j, from all sources;
//   send_off[s][j]  position of source s's first row for local expert j in s's own sorted send order.
__global__ void __launch_bounds__(1024) k_ep_publish_tables(const int* __restrict__ counts, PeerPtrs cnt_all, PeerPtrs flags, int rank, int W,
                                                            int E, int n_local, unsigned epoch, int* __restrict__ dst0,
                                                            int* __restrict__ counts_local, int* __restrict__ send_off, unsigned* status)
{
    __shared__ int wsum[32];
    __shared__ int prefix[1025];
    const int e = threadIdx.x;
    if (e < E) {
        const int c = max(counts[e], 0);
        for (int d = 0; d < W; ++d) static_cast<int*>(cnt_all.p[d])[rank * E + e] = c;
    }
    ep_signal_and_wait(flags, 0, rank, W, epoch, status);
    const volatile int* cnt = static_cast<const volatile int*>(cnt_all.p[rank]);
    int tot = 0, before = 0;
    if (e < E)
        for (int s = 0; s < W; ++s) {
            const int c = cnt[s * E + e];
            if (s < rank) before += c;
            tot += c;
        }
    const int pre = block_exclusive_scan(e < E ? tot : 0, wsum, nullptr);
    if (e <= E) prefix[e] = pre;
    __syncthreads();
    if (e < E) {
        const int owner0 = (e / n_local) * n_local;          // first expert of the owner's block
        dst0[e] = pre - prefix[owner0] + before;
        const int e0 = rank * n_local;
        if (e >= e0 && e < e0 + n_local) counts_local[e - e0] = tot;
    }
    for (int s = 0; s < W; ++s) {
        const int ps = block_exclusive_scan(e < E ? cnt[s * E + e] : 0, wsum, nullptr);
        const int e0 = rank * n_local;
        if (e >= e0 && e < e0 + n_local) send_off[s * n_local + (e - e0)] = ps;
    }
}

// Row pos of this rank's sorted send order -> the receive buffer of the rank that owns its expert.
// One row of H halves from src to dst, whole warp: the 16-byte pieces of a pass are loaded together before any is
// stored, so that a row's loads are in flight at once (dst may be peer memory).
__device__ __forceinline__ void copy_row_warp(const __half* __restrict__ src, __half* __restrict__ dst, int H, int lane)
{
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    const int n = H / 8;
    for (int base = 0; base < n; base += 256) {
        uint4 v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int idx = base + i * 32 + lane;
            if (idx < n) v[i] = s4[idx];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int idx = base + i * 32 + lane;
            if (idx < n) d4[idx] = v[i];
        }
    }
}

// Row pos of this rank's sorted send order -> the receive buffer of the rank that owns its expert.  The position tables
// sit in shared memory (a row's expert is found by bisection there, not through dependent global loads) and every warp
// moves a row of its own, eight rows in flight per block.
__global__ void __launch_bounds__(256) k_ep_dispatch(const __half* __restrict__ x, const int32_t* __restrict__ perm,
                                                     const int* __restrict__ offsets_send, const int* __restrict__ dst0, PeerPtrs recv_rows,
                                                     int E, int n_local, int top_k, int H, int n_send, int max_rows, unsigned* status)
{
    __shared__ int s_off[1025], s_dst[1024];   // E <= 1024
    for (int i = threadIdx.x; i < E; i += 256) { s_off[i] = offsets_send[i]; s_dst[i] = dst0[i]; }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int pos = blockIdx.x * 8 + warp; pos < n_send; pos += gridDim.x * 8) {
        int lo = 0, hi = E - 1;   // the last expert whose first position is <= pos and that has rows there
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (s_off[mid] <= pos) lo = mid; else hi = mid - 1;
        }
        const int e = lo;
        const int dst = s_dst[e] + pos - s_off[e];
        if (dst < 0 || dst >= max_rows) {
            if (lane == 0) atomicOr(status, kStEpOverflow);
            continue;
        }
        const int tok = min(max(perm[pos] / top_k, 0), n_send / top_k - 1);   // (n_send = tokens x top_k)
        copy_row_warp(x + size_t(tok) * H, static_cast<__half*>(recv_rows.p[e / n_local]) + size_t(dst) * H, H, lane);
    }
    __threadfence_system();
}

__global__ void __launch_bounds__(32) k_ep_barrier(PeerPtrs flags, int phase, int rank, int W, unsigned epoch, unsigned* status)
{
    ep_signal_and_wait(flags, phase, rank, W, epoch, status);
}

// dst[*row_off + r] = src[r] for r < rows (rows of H halves): the local tokens behind the received rows.
__global__ void __launch_bounds__(256) k_rows_to_offset(const __half* __restrict__ src, __half* __restrict__ dst, const int* __restrict__ row_off,
                                                        int rows, int H, int max_rows)
{
    const int off = min(max(__ldg(row_off), 0), max_rows - rows);
    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
        const uint4* s = reinterpret_cast<const uint4*>(src + size_t(r) * H);
        uint4* d = reinterpret_cast<uint4*>(dst + size_t(off + r) * H);
        for (int i = threadIdx.x; i < H / 8; i += 256) d[i] = s[i];
    }
}
__global__ void __launch_bounds__(256) k_rows_from_offset(const __half* __restrict__ src, __half* __restrict__ dst, const int* __restrict__ row_off,
                                                          int rows, int H, int max_rows)
{
    const int off = min(max(__ldg(row_off), 0), max_rows - rows);
    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
        const uint4* s = reinterpret_cast<const uint4*>(src + size_t(off + r) * H);
        uint4* d = reinterpret_cast<uint4*>(dst + size_t(r) * H);
        for (int i = threadIdx.x; i < H / 8; i += 256) d[i] = s[i];
    }
}

// Expert output row p (rows sorted by local expert, inside an expert source by source) -> the source's return
// buffer at the position the row had in the source's sorted send order.  Tables in shared memory, a row per warp.
__global__ void __launch_bounds__(256) k_ep_return(const __half* __restrict__ yr, const int* __restrict__ offsets, PeerPtrs cnt_all,
                                                   const int* __restrict__ send_off, PeerPtrs ret_rows, int rank, int W, int E, int n_local,
                                                   int H, int max_rows, int max_send, unsigned* status)
{
    __shared__ int s_off[1025], s_cnt[1024], s_so[1024];   // W * n_local = E <= 1024
    const int* cnt = static_cast<const int*>(cnt_all.p[rank]);
    for (int i = threadIdx.x; i <= n_local; i += 256) s_off[i] = offsets[i];
    for (int i = threadIdx.x; i < W * n_local; i += 256) {
        const int sr = i / n_local, j = i - sr * n_local;
        s_cnt[i] = cnt[sr * E + rank * n_local + j];
        s_so[i] = send_off[i];
    }
    __syncthreads();
    const int R = min(max(s_off[n_local], 0), max_rows);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int p = blockIdx.x * 8 + warp; p < R; p += gridDim.x * 8) {
        int lo = 0, hi = n_local - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (s_off[mid] <= p) lo = mid; else hi = mid - 1;
        }
        const int j = lo;
        int q = p - s_off[j], sr = 0;
        for (; sr < W - 1; ++sr) {
            const int c = s_cnt[sr * n_local + j];
            if (q < c) break;
            q -= c;
        }
        const int srcpos = s_so[sr * n_local + j] + q;
        if (srcpos < 0 || srcpos >= max_send) {
            if (lane == 0) atomicOr(status, kStEpOverflow);
            continue;
        }
        copy_row_warp(yr + size_t(p) * H, static_cast<__half*>(ret_rows.p[sr]) + size_t(srcpos) * H, H, lane);
    }
    __threadfence_system();
}

inline size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

// How the expert stage cuts an expert's rows into problems: up to 32 rows per problem go through the
// grouped decode GEMV (8, 16 or 32 rows = 1, 2 or 4 token groups), more through the grouped tensor-core
// GEMM (128..384 rows = 1..3 sub-tiles).  An expert with more rows than one chunk takes several problems.
struct ExpertPlan {
    int chunk;   // rows per problem
    int tg;      // token groups of the GEMV path, 0 on the GEMM path
    int nsub;    // 128-row sub-tiles of the GEMM path, 0 on the GEMV path
};
ExpertPlan expert_plan(int rows_per_expert)
{
    if (rows_per_expert <= 8) return {8, 1, 0};
    if (rows_per_expert <= 16) return {16, 2, 0};
    if (rows_per_expert <= 32) return {32, 4, 0};
    const int nsub = std::min(3, (rows_per_expert + 127) / 128);
    return {128 * nsub, 0, nsub};
}

// Rows-per-expert figure for T tokens routed top_k ways over n_experts: twice the mean, never beyond
// what one expert can receive.
// With short inner dimensions (expert shapes: K = hidden or inter) the plan stays at 128-row problems however many
// rows an expert has: a 128-row item's accumulator is double buffered, so its epilogue runs under the next item's
// main loop, while a 256- or 384-row item fills tensor memory with one accumulator and exposes an epilogue that is as
// long as 2 K / 64 decode stages (measured on 8448 tokens of the A3B shapes: gate+up 516 against 605 us, down 652
// against 685 us).  Taller items pay from K of several thousand, where the weights' decode per item dominates.
constexpr int kShortK = 2048;
int routed_rows_hint(int T, int top_k, int n_experts, int hidden = 0, int inter = 0)
{
    const long long twice_mean = (2LL * T * top_k + n_experts - 1) / n_experts;
    int h = int(std::min<long long>(T, std::max<long long>(twice_mean, 1)));   // the caller turns this into a plan
    if (h > 128 && hidden > 0 && std::min(hidden, inter) <= kShortK) h = 128;
    return h;
}

// Workspace carve-up of the expert stage for up to R routed rows.
struct ExpertScratch {
    int* counts; int* offsets; int* n_problems; GemvProblem* problems;
    uint32_t* afrag; uint32_t* afrag2; float* blocksum; float* blocksum2; __half* g; __half* u; int max_problems;
    size_t bytes;
};
ExpertScratch carve_experts(void* base, int R, int n_local, int hidden, int inter, const ExpertPlan& plan)
{
    ExpertScratch s{};
    const int chunk = plan.chunk;
    s.max_problems = R / chunk + n_local;
    const int kmax = std::max(hidden, inter);
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off += align256(bytes); return o; };
    const size_t o_counts = take(size_t(n_local) * 4), o_offsets = take(size_t(n_local + 2) * 4), o_np = take(8);
    const size_t o_prob = take(size_t(2) * s.max_problems * sizeof(GemvProblem));   // room for the doubled (gate + up) table
    // rotated activations: fragment order per problem (GEMV) or plain rows (GEMM); room for the rows rotated with
    // the gate scales and, behind them, with the up scales (one rotation launch writes both)
    const size_t half_afrag = plan.tg ? size_t(s.max_problems) * (hidden / 16) * plan.tg * 256 : size_t(R) * hidden * 2;
    const size_t o_afrag = take(std::max(2 * half_afrag, plan.tg ? size_t(s.max_problems) * (kmax / 16) * plan.tg * 256 : size_t(R) * kmax * 2));
    const size_t half_bsum = plan.tg ? size_t(s.max_problems) * chunk * (hidden / 128) * 4 : 128;
    const size_t o_bsum = take(std::max(2 * half_bsum, plan.tg ? size_t(s.max_problems) * chunk * (kmax / 128) * 4 : 256));
    const size_t o_g = take(size_t(2) * R * inter * 2);   // gate outputs, then up outputs
    s.bytes = off;
    if (base) {
        char* b = static_cast<char*>(base);
        s.counts = (int*) (b + o_counts); s.offsets = (int*) (b + o_offsets); s.n_problems = (int*) (b + o_np);
        s.problems = (GemvProblem*) (b + o_prob); s.afrag = (uint32_t*) (b + o_afrag); s.afrag2 = (uint32_t*) (b + o_afrag + half_afrag);
        s.blocksum = (float*) (b + o_bsum); s.blocksum2 = (float*) (b + o_bsum + half_bsum);
        s.g = (__half*) (b + o_g); s.u = s.g + size_t(R) * inter;
    }
    return s;
}

// True if the shared expert has the experts' shape and each of its nine tensors starts exactly where the
// corresponding stack of n_experts matrices ends, i.e. the stacks really hold n_experts + 1 matrices.
bool shared_behind_stacks(const berth_moe_weights* w)
{
    if (w->shared_inter <= 0 || w->shared_inter != w->inter) return false;
    const size_t E = size_t(w->n_experts), H = size_t(w->hidden), I = size_t(w->inter);
    const size_t t_hi = H / 16 * (I / 16) * 16 * size_t(w->k_bits) * 2;   // bytes of one hidden x inter trellis
    auto at = [](const void* base, size_t bytes) { return static_cast<const void*>(static_cast<const char*>(base) + bytes); };
    return w->sh_gate_trellis == at(w->gate_trellis, E * t_hi) && w->sh_up_trellis == at(w->up_trellis, E * t_hi) &&
           w->sh_down_trellis == at(w->down_trellis, E * t_hi) && w->sh_gate_suh == at(w->gate_suh, E * H * 2) &&
           w->sh_gate_svh == at(w->gate_svh, E * I * 2) && w->sh_up_suh == at(w->up_suh, E * H * 2) &&
           w->sh_up_svh == at(w->up_svh, E * I * 2) && w->sh_down_suh == at(w->down_suh, E * I * 2) &&
           w->sh_down_svh == at(w->down_svh, E * H * 2);
}

// `routes`: the caller also runs the router over w->n_experts (an expert-parallel rank's block need not be a multiple of 32).
// True if the up stack of n_matrices matrices (trellis and output scales) starts exactly where the gate stack
// ends: one grouped launch over a doubled problem table then runs both projections.
bool up_behind_gate(const berth_moe_weights* w, int n_matrices)
{
    const size_t H = size_t(w->hidden), I = size_t(w->inter);
    const size_t t_hi = H / 16 * (I / 16) * 16 * size_t(w->k_bits) * 2;
    auto at = [](const void* base, size_t bytes) { return static_cast<const void*>(static_cast<const char*>(base) + bytes); };
    return w->up_trellis == at(w->gate_trellis, size_t(n_matrices) * t_hi) && w->up_svh == at(w->gate_svh, size_t(n_matrices) * I * 2);
}

void check_moe_shapes(const berth_moe_weights* w, int T, bool routes = false)
{
    if (!w) throw std::runtime_error("moe: null weights");
    if (T < 1) throw std::runtime_error("moe: T must be positive");
    if (w->hidden % 128 || w->inter % 128 || w->hidden < 128 || w->inter < 128)
        throw std::runtime_error("moe: hidden and inter must be multiples of 128");
    if (w->shared_inter % 128) throw std::runtime_error("moe: shared_inter must be a multiple of 128");
    if (w->n_experts < 1 || w->n_experts > 1024 || (routes && w->n_experts % 32))
        throw std::runtime_error("moe: n_experts must be a multiple of 32 up to 1024");
    if (w->top_k < 1 || w->top_k > 32 || w->top_k > w->n_experts) throw std::runtime_error("moe: top_k must be in 1..=32");
    if (w->hidden % 32) throw std::runtime_error("moe: hidden must be a multiple of 32");
    if (w->k_bits < 1 || w->k_bits > 8) throw std::runtime_error("moe: K must be in 1..=8");
    if (w->codebook < 0 || w->codebook > 2) throw std::runtime_error("moe: codebook must be 0, 1, or 2");
}

void router_topk(const void* x, const void* w_router, const float* bias, int32_t* topk_idx, float* topk_w, float* logits,
                 int T, int H, int E, int k, cudaStream_t st)
{
    const size_t smem = size_t(kRouterTok) * H * 4 + size_t(32) * kRouterTok * 33 * 4;
    if (smem > 200 * 1024) throw std::runtime_error("moe router: hidden is too large for the router's shared-memory tile");
    static bool attr_set[kMaxDevices] = {};
    const int dev = current_device();
    if (!attr_set[dev]) {
        cuda_ok(cudaFuncSetAttribute(k_moe_router_logits<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024), "router smem attribute");
        cuda_ok(cudaFuncSetAttribute(k_moe_router_logits<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024), "router smem attribute");
        attr_set[dev] = true;
    }
    const dim3 rgrid(E / 32, (T + kRouterTok - 1) / kRouterTok);
    const size_t smem_wide = size_t(kRouterTok) * H * 4 + size_t(16) * kRouterTok * kWidePitch * 4;
    if (E % 128 == 0 && H % 256 == 0 && smem_wide <= 200 * 1024 && int(rgrid.x * rgrid.y) > 2 * device_info(dev).sms) {
        static bool wide_set[kMaxDevices] = {};
        if (!wide_set[dev]) {
            cuda_ok(cudaFuncSetAttribute(k_moe_router_logits_wide, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024), "router smem attribute");
            wide_set[dev] = true;
        }
        launch_pdl(k_moe_router_logits_wide, dim3(E / 128, rgrid.y), dim3(512), smem_wide, st, "k_moe_router_logits_wide launch",
                   (const __half*) x, (const __half*) w_router, bias, logits, T, H, E);
    } else if (int(rgrid.x * rgrid.y) <= device_info(dev).sms)
        launch_pdl(k_moe_router_logits<32>, rgrid, dim3(32 * 32), smem, st, "k_moe_router_logits launch", (const __half*) x,
                   (const __half*) w_router, bias, logits, T, H, E);
    else
        launch_pdl(k_moe_router_logits<16>, rgrid, dim3(16 * 32), smem, st, "k_moe_router_logits launch", (const __half*) x,
                   (const __half*) w_router, bias, logits, T, H, E);
    cuda_ok(cudaGetLastError(), "k_moe_router_logits launch");
    launch_pdl(k_moe_topk, dim3((T + 3) / 4), dim3(128), 0, st, "k_moe_topk launch", logits, topk_idx, topk_w, T, E, k);
    cuda_ok(cudaGetLastError(), "k_moe_topk launch");
}

// keys[n] -> counts/offsets/problems + perm/inv; experts [e0, e0 + n_local).
void dispatch(const int32_t* keys, int n, int e0, int n_local, int chunk, const ExpertScratch& s, int32_t* perm, int32_t* inv,
              cudaStream_t st, int extra_rows = 0, int pair_rows = 0, int pair_matrices = 0)
{
    unsigned* status = gemv_workspace(current_device()).status;
    const int max_rows = n + extra_rows;   // the arrays the caller carved for this stage
    if (n_local + (extra_rows > 0 ? 1 : 0) > 1024) throw std::runtime_error("moe: too many local experts for the scan kernel");
    if (n <= kSmallKeys) {
        launch_pdl(k_moe_dispatch_small, dim3(1), dim3(1024), 0, st, "k_moe_dispatch_small launch", keys, n, e0, s.counts, s.offsets, s.problems, s.n_problems, n_local, chunk, extra_rows, pair_rows, pair_matrices, perm, inv, s.max_problems, max_rows, status);
        cuda_ok(cudaGetLastError(), "k_moe_dispatch_small launch");
        return;
    }
    launch_pdl(k_moe_count, dim3(n_local), dim3(256), 0, st, "k_moe_count launch", keys, n, e0, s.counts);
    cuda_ok(cudaGetLastError(), "k_moe_count launch");
    launch_pdl(k_moe_scan, dim3(1), dim3(1024), 0, st, "k_moe_scan launch", s.counts, s.offsets, s.problems, s.n_problems, n_local, chunk, extra_rows, pair_rows, pair_matrices, s.max_problems, max_rows, status);
    cuda_ok(cudaGetLastError(), "k_moe_scan launch");
    launch_pdl(k_moe_scatter, dim3(n_local), dim3(1024), 0, st, "k_moe_scatter launch", keys, n, e0, s.offsets, perm, inv);
    cuda_ok(cudaGetLastError(), "k_moe_scatter launch");
}

// Where the expert stage's input rows come from when they are not in place: row r < n_perm is row perm[r] / div
// of the array handed in as xr, later rows are its rows r - n_perm (perm == nullptr: xr holds the rows themselves).
struct RowSource {
    const int32_t* perm = nullptr;
    int div = 1, n_perm = 0;
    bool paired = false;   // the problem table was written twice (scan_problems, pair_rows = max_rows) and up lies behind gate
};

// Grouped gate/up -> silu*up -> down over routed rows xr [R][hidden]; yr fp16 [R][hidden].
std::string experts(const berth_moe_weights* w, const void* gate_t, const void* up_t, const void* down_t, const void* gsuh,
                    const void* gsvh, const void* usuh, const void* usvh, const void* dsuh, const void* dsvh, int n_local,
                    const void* xr, void* yr, int R, int max_rows, const ExpertPlan& plan, const ExpertScratch& s, const GemvScratch& sc,
                    int sms, cudaStream_t st, const int* rows_dev = nullptr, const RowSource& src = RowSource{})
{
    const int H = w->hidden, I = w->inter;
    // (the activation between the projections runs inside the rotation of the down projection, over the rows of the
    // problem table; neither row count is needed here)
    (void) R; (void) rows_dev;
    // paired: gate and up are the two halves of one stack, the doubled problem table sends the second half's
    // outputs to rows max_rows.. of the gate output buffer
    const bool paired = src.paired;
    const __half* u_out = paired ? s.g + size_t(max_rows) * I : s.u;
    if (plan.nsub) {
        // one rotation launch for gate and up (the row is read once), the activation inside the rotation for down
        RotateArgs r{};
        r.src = static_cast<const __half*>(xr);
        r.perm = src.perm; r.div = src.div; r.n_perm = src.n_perm;
        r.suh_a = static_cast<const __half*>(gsuh); r.suh_b = static_cast<const __half*>(usuh);
        r.out_a = reinterpret_cast<__half*>(s.afrag);
        r.out_b = paired ? r.out_a + size_t(max_rows) * H : reinterpret_cast<__half*>(s.afrag2);
        r.problems = s.problems; r.n_problems = s.n_problems;
        r.chunk = plan.chunk; r.k = H; r.max_problems = s.max_problems; r.n_matrices = n_local; r.max_rows = max_rows;
        rotate_rows_grouped(r, true, false, sms, st);
        std::string d;
        if (paired) {
            d = launch_gemm_tc_grouped_rotated(s.afrag, gate_t, 2 * n_local, s.g, gsvh, s.problems, s.n_problems + 1, 2 * s.max_problems,
                                               2 * max_rows, plan.nsub, H, I, w->k_bits, w->codebook, 0, sc.status, sms, st);
        } else {
            d = launch_gemm_tc_grouped_rotated(s.afrag, gate_t, n_local, s.g, gsvh, s.problems, s.n_problems, s.max_problems, max_rows,
                                               plan.nsub, H, I, w->k_bits, w->codebook, 0, sc.status, sms, st);
            launch_gemm_tc_grouped_rotated(s.afrag2, up_t, n_local, s.u, usvh, s.problems, s.n_problems, s.max_problems, max_rows, plan.nsub,
                                           H, I, w->k_bits, w->codebook, 0, sc.status, sms, st);
        }
        RotateArgs rd{};
        rd.src = s.g; rd.src_u = u_out;
        rd.suh_a = static_cast<const __half*>(dsuh);
        rd.out_a = reinterpret_cast<__half*>(s.afrag);
        rd.problems = s.problems; rd.n_problems = s.n_problems;
        rd.chunk = plan.chunk; rd.k = I; rd.max_problems = s.max_problems; rd.n_matrices = n_local; rd.max_rows = max_rows;
        rotate_rows_grouped(rd, false, true, sms, st);
        launch_gemm_tc_grouped_rotated(s.afrag, down_t, n_local, yr, dsvh, s.problems, s.n_problems, s.max_problems, max_rows, plan.nsub, I,
                                       H, w->k_bits, w->codebook, 0, sc.status, sms, st);
        return std::string("k_rotate_rows_plain<gate+up> + ") + (paired ? "1 x (gate and up as one stack) " : "2 x ") + d +
               " + k_rotate_rows_plain<silu> + 1 x (same, down)";
    }
    const int tg = plan.tg;
    RotateFragArgs r{};
    r.src = static_cast<const __half*>(xr);
    r.perm = src.perm; r.div = src.div; r.n_perm = src.n_perm;
    r.suh_a = static_cast<const __half*>(gsuh); r.suh_b = static_cast<const __half*>(usuh);
    r.afrag_a = s.afrag; r.afrag_b = s.afrag2; r.bsum_a = s.blocksum; r.bsum_b = s.blocksum2;
    r.problems = s.problems; r.n_problems = s.n_problems;
    r.tok = 8 * tg; r.k = H; r.max_problems = s.max_problems; r.n_matrices = n_local; r.max_rows = max_rows;
    r.pair = paired ? 1 : 0;
    rotate_rows_frag(r, true, false, sms, st);
    std::string d;
    if (paired) {
        d = launch_gemv_grouped_rotated(gate_t, 2 * n_local, s.g, gsvh, s.problems, s.n_problems + 1, 2 * s.max_problems, 2 * max_rows, tg,
                                        s.afrag, s.blocksum, H, I, w->k_bits, w->codebook, 0, sc, sms, st);
    } else {
        d = launch_gemv_grouped_rotated(gate_t, n_local, s.g, gsvh, s.problems, s.n_problems, s.max_problems, max_rows, tg, s.afrag,
                                        s.blocksum, H, I, w->k_bits, w->codebook, 0, sc, sms, st);
        launch_gemv_grouped_rotated(up_t, n_local, s.u, usvh, s.problems, s.n_problems, s.max_problems, max_rows, tg, s.afrag2, s.blocksum2, H,
                                    I, w->k_bits, w->codebook, 0, sc, sms, st);
    }
    RotateFragArgs rd{};
    rd.src = s.g; rd.src_u = u_out;
    rd.suh_a = static_cast<const __half*>(dsuh);
    rd.afrag_a = s.afrag; rd.bsum_a = s.blocksum;
    rd.problems = s.problems; rd.n_problems = s.n_problems;
    rd.tok = 8 * tg; rd.k = I; rd.max_problems = s.max_problems; rd.n_matrices = n_local; rd.max_rows = max_rows;
    rotate_rows_frag(rd, false, true, sms, st);
    launch_gemv_grouped_rotated(down_t, n_local, yr, dsvh, s.problems, s.n_problems, s.max_problems, max_rows, tg, s.afrag, s.blocksum, I, H,
                                w->k_bits, w->codebook, 0, sc, sms, st);
    return std::string("k_rotate_rows<gate+up> + ") + (paired ? "1 x (gate and up as one stack: " : "2 x (") + d +
           ") + k_rotate_rows<silu> + 1 x (same, down)";
}

}  // namespace
}  // namespace berth

using namespace berth;

extern "C" const char* berth_moe_last_error(void) { return moe_state().err.c_str(); }
extern "C" const char* berth_moe_last_launch(void) { return moe_state().launch.c_str(); }

extern "C" int berth_moe_router_topk(const void* x, const void* w_router, const float* router_bias, int32_t* topk_idx,
                                     float* topk_w, float* logits, int T, int hidden, int n_experts, int top_k, void* stream)
{
    CallState& st = moe_state();
    return guarded(st, [&] {
        if (!x || !w_router || !topk_idx || !topk_w || !logits) throw std::runtime_error("moe router: null device pointer");
        if (T < 1) throw std::runtime_error("moe router: T must be positive");
        if (hidden < 32 || hidden % 32) throw std::runtime_error("moe router: hidden must be a multiple of 32");
        if (n_experts < 32 || n_experts % 32 || n_experts > 1024)
            throw std::runtime_error("moe router: n_experts must be a multiple of 32 up to 1024");
        if (top_k < 1 || top_k > 32 || top_k > n_experts) throw std::runtime_error("moe router: top_k must be in 1..=32");
        router_topk(x, w_router, router_bias, topk_idx, topk_w, logits, T, hidden, n_experts, top_k, (cudaStream_t) stream);
        st.launch = "k_moe_router_logits grid=" + std::to_string(n_experts / 32) + "x" + std::to_string((T + kRouterTok - 1) / kRouterTok) + " + k_moe_topk";
    });
}

// ---- the stages of the layer, exported one by one for hosts that put a collective between them
// (expert parallelism: sort -> gather -> all-to-all -> sort -> gather -> experts -> gather ->
// all-to-all -> combine).  `ews` is the expert-stage scratch of berth_moe_experts_workspace_bytes.

extern "C" size_t berth_moe_experts_workspace_bytes(int max_rows, int n_local, int hidden, int inter, int max_rows_per_expert)
{
    if (max_rows < 1 || n_local < 1 || hidden < 128 || inter < 128) return 0;
    return carve_experts(nullptr, max_rows, n_local, hidden, inter, expert_plan(max_rows_per_expert)).bytes + 256;
}

static ExpertScratch expert_scratch(void* ews, size_t ews_bytes, int max_rows, int n_local, int hidden, int inter, int mrpe)
{
    if (!ews) throw std::runtime_error("moe: null expert workspace");
    const size_t need = berth_moe_experts_workspace_bytes(max_rows, n_local, hidden, inter, mrpe);
    if (ews_bytes < need)
        throw std::runtime_error("moe: expert workspace of " + std::to_string(ews_bytes) + " bytes is smaller than the " +
                                 std::to_string(need) + " required");
    void* b = reinterpret_cast<void*>((reinterpret_cast<uintptr_t>(ews) + 255) & ~uintptr_t(255));
    return carve_experts(b, max_rows, n_local, hidden, inter, expert_plan(mrpe));
}

extern "C" int berth_moe_sort_rows(const int32_t* keys, int n, int e0, int n_local, int32_t* perm, int32_t* inv,
                                   int32_t* offsets_out, void* ews, size_t ews_bytes, int max_rows, int hidden, int inter,
                                   int max_rows_per_expert, void* stream)
{
    CallState& st = moe_state();
    return guarded(st, [&] {
        if ((n > 0 && !keys) || !perm || !inv) throw std::runtime_error("moe sort: null device pointer");
        if (n < 0 || n > max_rows) throw std::runtime_error("moe sort: n must be within 0..max_rows");
        if (n_local < 1 || n_local > 1024) throw std::runtime_error("moe sort: n_local must be in 1..=1024");
        ExpertScratch es = expert_scratch(ews, ews_bytes, max_rows, n_local, hidden, inter, max_rows_per_expert);
        dispatch(keys, n, e0, n_local, expert_plan(max_rows_per_expert).chunk, es, perm, inv, (cudaStream_t) stream);
        if (offsets_out)
            cuda_ok(cudaMemcpyAsync(offsets_out, es.offsets, size_t(n_local + 1) * 4, cudaMemcpyDeviceToDevice, (cudaStream_t) stream),
                    "moe sort offsets copy");
        st.launch = "k_moe_count + k_moe_scan + k_moe_scatter grid=" + std::to_string(n_local);
    });
}

// dst[i][:] = src[index[i] / div][:] for i < n (fp16 rows of `hidden` elements).
extern "C" int berth_moe_gather(const void* src, const int32_t* index, int div, int n, void* dst, int hidden, void* stream)
{
    CallState& st = moe_state();
    return guarded(st, [&] {
        if (!src || !index || !dst) throw std::runtime_error("moe gather: null device pointer");
        if (n < 0 || div < 1 || hidden < 8 || hidden % 8) throw std::runtime_error("moe gather: bad sizes");
        if (n == 0) return;
        k_moe_gather_n<<<std::min(n, 148 * 8), 256, 0, (cudaStream_t) stream>>>((const __half*) src, index, n, div, (__half*) dst, hidden);
        cuda_ok(cudaGetLastError(), "k_moe_gather launch");
        st.launch = "k_moe_gather_n";
    });
}

extern "C" int berth_moe_experts(const berth_moe_weights* w, const void* xr, void* yr, int n_rows, void* ews, size_t ews_bytes,
                                 int max_rows, int max_rows_per_expert, void* stream)
{
    CallState& st = moe_state();
    return guarded(st, [&] {
        check_moe_shapes(w, 1);
        if (!xr || !yr) throw std::runtime_error("moe experts: null device pointer");
        if (n_rows < 0 || n_rows > max_rows) throw std::runtime_error("moe experts: n_rows must be within 0..max_rows");
        const int device = current_device();
        const DeviceInfo& info = device_info(device);
        if (info.major != 10) throw std::runtime_error("moe experts: no linked kernel for this GPU (library is built for sm_100a only)");
        ExpertScratch es = expert_scratch(ews, ews_bytes, max_rows, w->n_experts, w->hidden, w->inter, max_rows_per_expert);
        if (n_rows == 0) return;
        st.launch = experts(w, w->gate_trellis, w->up_trellis, w->down_trellis, w->gate_suh, w->gate_svh, w->up_suh, w->up_svh,
                            w->down_suh, w->down_svh, w->n_experts, xr, yr, n_rows, n_rows, expert_plan(max_rows_per_expert), es,
                            gemv_workspace(device), info.sms, (cudaStream_t) stream);
    });
}

extern "C" int berth_moe_combine(const void* y, const int32_t* inv, const float* topk_w, const void* ysh, void* out, int T,
                                 int hidden, int top_k, void* stream)
{
    CallState& st = moe_state();
    return guarded(st, [&] {
        if (!y || !inv || !topk_w || !out) throw std::runtime_error("moe combine: null device pointer");
        if (T < 1 || hidden < 2 || hidden % 2 || top_k < 1 || top_k > 32) throw std::runtime_error("moe combine: bad sizes (top_k must be in 1..=32)");
        k_moe_combine<<<dim3(T, (hidden + 511) / 512), 256, 0, (cudaStream_t) stream>>>((const __half*) y, inv, topk_w, (const __half*) ysh, (float*) out, hidden, top_k, 0x7fffffff);
        cuda_ok(cudaGetLastError(), "k_moe_combine launch");
        st.launch = "k_moe_combine grid=" + std::to_string(T);
    });
}

// ---- expert parallelism with one library call per side of the exchange

extern "C" size_t berth_moe_ep_send_workspace_bytes(int T, int n_experts, int top_k)
{
    if (T < 1 || n_experts < 1 || top_k < 1) return 0;
    const size_t R = size_t(T) * top_k;
    return align256(size_t(T) * n_experts * 4) + align256(R * 4) + align256(size_t(n_experts + 2) * 4) + 256 +
           align256((R / 8 + n_experts + 1) * sizeof(GemvProblem)) + 512;
}

extern "C" int berth_moe_ep_send(const void* x, int T, const void* w_router, const float* router_bias, int hidden, int n_experts,
                                 int top_k, int32_t* topk_idx, float* topk_w, int32_t* inv, void* send_rows, int32_t* counts,
                                 void* ws, size_t ws_bytes, void* stream)
{
    CallState& st = moe_state();
    return guarded(st, [&] {
        if (!x || !w_router || !topk_idx || !topk_w || !inv || !send_rows || !counts || !ws)
            throw std::runtime_error("moe ep send: null device pointer");
        if (T < 1) throw std::runtime_error("moe ep send: T must be positive");
        if (hidden < 32 || hidden % 32) throw std::runtime_error("moe ep send: hidden must be a multiple of 32");
        if (n_experts < 32 || n_experts % 32 || n_experts > 1024)
            throw std::runtime_error("moe ep send: n_experts must be a multiple of 32 up to 1024");
        if (top_k < 1 || top_k > 32 || top_k > n_experts) throw std::runtime_error("moe ep send: top_k must be in 1..=32");
        if (ws_bytes < berth_moe_ep_send_workspace_bytes(T, n_experts, top_k)) throw std::runtime_error("moe ep send: workspace too small");
        cudaStream_t cs = (cudaStream_t) stream;
        const int R = T * top_k;
        char* b = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(ws) + 255) & ~uintptr_t(255));
        auto take = [&](size_t bytes) { char* p = b; b += align256(bytes); return p; };
        float* logits = (float*) take(size_t(T) * n_experts * 4);
        int32_t* perm = (int32_t*) take(size_t(R) * 4);
        ExpertScratch es{};
        es.counts = counts;
        es.offsets = (int*) take(size_t(n_experts + 2) * 4);
        es.n_problems = (int*) take(4);
        es.problems = (GemvProblem*) take((size_t(R) / 8 + n_experts + 1) * sizeof(GemvProblem));
        es.max_problems = R / 8 + n_experts;
        router_topk(x, w_router, router_bias, topk_idx, topk_w, logits, T, hidden, n_experts, top_k, cs);
        dispatch(topk_idx, R, 0, n_experts, 8, es, perm, inv, cs);
        launch_pdl(k_moe_gather_rows, dim3(std::min(R, 148 * 8)), dim3(256), 0, cs, "k_moe_gather_rows launch", (const __half*) x, perm, es.offsets + n_experts, top_k, (__half*) send_rows, hidden);
        cuda_ok(cudaGetLastError(), "k_moe_gather_rows launch");
        st.launch = "k_moe_router_logits + k_moe_topk + k_moe_count/scan/scatter + k_moe_gather_rows";
    });
}

static const int kPlanHints[] = {8, 16, 32, 128, 256, 384};

extern "C" size_t berth_moe_ep_experts_workspace_bytes(int max_rows, int max_tokens, int world, int n_local, int hidden, int inter)
{
    if (max_rows < 1 || max_tokens < 0 || world < 1 || n_local < 1 || hidden < 128 || inter < 128) return 0;
    size_t es = 0;
    for (int h : kPlanHints) es = std::max(es, carve_experts(nullptr, max_rows + max_tokens, n_local + 1, hidden, inter, expert_plan(h)).bytes);
    return 3 * align256(size_t(max_rows) * 4) + align256(size_t(world * n_local + 1) * 4) +
           2 * align256(size_t(max_rows + max_tokens) * hidden * 2) + es + 1024;
}

extern "C" int berth_moe_ep_experts(const berth_moe_weights* w, const void* recv_rows, int n_rows, const int32_t* cnt_recv, int world,
                                    const void* x_local, int T_local, void* back, void* ysh, void* ws, size_t ws_bytes, int max_rows,
                                    int max_tokens, int rows_hint, void* stream)
{
    CallState& st = moe_state();
    return guarded(st, [&] {
        check_moe_shapes(w, 1);
        if (!cnt_recv || !ws || (n_rows > 0 && (!recv_rows || !back))) throw std::runtime_error("moe ep experts: null device pointer");
        if (n_rows < 0 || n_rows > max_rows) throw std::runtime_error("moe ep experts: n_rows must be within 0..max_rows");
        if (T_local < 0 || T_local > max_tokens) throw std::runtime_error("moe ep experts: T_local must be within 0..max_tokens");
        const int NL = w->n_experts, H = w->hidden, I = w->inter;
        if (world < 1 || world * NL > 1024) throw std::runtime_error("moe ep experts: world x local experts must be at most 1024");
        const bool with_shared = ysh != nullptr && T_local > 0;
        if (with_shared && (!x_local || !shared_behind_stacks(w)))
            throw std::runtime_error("moe ep experts: the shared expert must be stored behind the expert stacks to run here");
        if (ws_bytes < berth_moe_ep_experts_workspace_bytes(max_rows, max_tokens, world, NL, H, I))
            throw std::runtime_error("moe ep experts: workspace too small");
        const int device = current_device();
        const DeviceInfo& info = device_info(device);
        if (info.major != 10) throw std::runtime_error("moe ep experts: no linked kernel for this GPU (library is built for sm_100a only)");
        cudaStream_t cs = (cudaStream_t) stream;
        const int TS = with_shared ? T_local : 0;
        const int RT = n_rows + TS, NM = with_shared ? NL + 1 : NL;
        if (RT == 0) return;
        const ExpertPlan plan = expert_plan(std::max(rows_hint, 1));
        char* b = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(ws) + 255) & ~uintptr_t(255));
        auto take = [&](size_t bytes) { char* p = b; b += align256(bytes); return p; };
        int32_t* keys = (int32_t*) take(size_t(max_rows) * 4);
        int32_t* perm = (int32_t*) take(size_t(max_rows) * 4);
        int32_t* inv = (int32_t*) take(size_t(max_rows) * 4);
        int* seg_off = (int*) take(size_t(world * NL + 1) * 4);
        __half* xr = (__half*) take(size_t(max_rows + max_tokens) * H * 2);
        __half* yr = (__half*) take(size_t(max_rows + max_tokens) * H * 2);
        ExpertScratch es = carve_experts(b, RT, NM, H, I, plan);
        if (n_rows > 0) {
            k_moe_segment_scan<<<1, 1024, 0, cs>>>(cnt_recv, world * NL, seg_off);
            k_moe_segment_keys<<<world * NL, 128, 0, cs>>>(seg_off, NL, n_rows, keys);
            cuda_ok(cudaGetLastError(), "k_moe_segment_keys launch");
        }
        RowSource in_place{};
        in_place.paired = up_behind_gate(w, NM);
        dispatch(keys, n_rows, 0, NL, plan.chunk, es, perm, inv, cs, TS, in_place.paired ? RT : 0, NM);
        if (n_rows > 0) {
            launch_pdl(k_moe_gather_rows, dim3(std::min(n_rows, 148 * 8)), dim3(256), 0, cs, "k_moe_gather_rows launch", (const __half*) recv_rows, perm, es.offsets + NL, 1, xr, H);
            cuda_ok(cudaGetLastError(), "k_moe_gather_rows launch");
        }
        if (TS) cuda_ok(cudaMemcpyAsync(xr + size_t(n_rows) * H, x_local, size_t(TS) * H * 2, cudaMemcpyDeviceToDevice, cs), "moe ep experts: shared rows copy");
        st.launch = experts(w, w->gate_trellis, w->up_trellis, w->down_trellis, w->gate_suh, w->gate_svh, w->up_suh, w->up_svh,
                            w->down_suh, w->down_svh, NM, xr, yr, RT, RT, plan, es, gemv_workspace(device), info.sms, cs, nullptr, in_place);
        if (n_rows > 0) {
            launch_pdl(k_moe_gather_n, dim3(std::min(n_rows, 148 * 8)), dim3(256), 0, cs, "k_moe_gather_n launch", yr, inv, n_rows, 1, (__half*) back, H);
            cuda_ok(cudaGetLastError(), "k_moe_gather launch");
        }
        if (TS) cuda_ok(cudaMemcpyAsync(ysh, yr + size_t(n_rows) * H, size_t(TS) * H * 2, cudaMemcpyDeviceToDevice, cs), "moe ep experts: shared output copy");
        st.launch = "k_moe_segment_scan/keys + k_moe_count/scan/scatter + k_moe_gather_rows + 3 x (" + st.launch + ") + k_silu_mul + k_moe_gather_n";
    });
}

// ---- expert parallelism over peer memory: two calls per layer, no collective, no host synchronisation

namespace {
struct P2pSendWs {
    float* logits; int32_t* perm; int* counts; int* offsets; int* n_problems; GemvProblem* problems;
    int* dst0; int* counts_local; int* send_off; size_t bytes;
};
P2pSendWs carve_p2p_send(void* base, int T, int E, int top_k, int world, int n_local)
{
    P2pSendWs s{};
    const size_t R = size_t(T) * top_k;
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off += align256(bytes); return o; };
    const size_t o_log = take(size_t(T) * E * 4), o_perm = take(R * 4), o_cnt = take(size_t(E) * 4), o_off = take(size_t(E + 2) * 4);
    const size_t o_np = take(4), o_prob = take((R / 8 + E + 1) * sizeof(GemvProblem)), o_dst = take(size_t(E) * 4);
    const size_t o_cl = take(size_t(n_local + 1) * 4), o_so = take(size_t(world) * n_local * 4);
    s.bytes = off;
    if (base) {
        char* b = static_cast<char*>(base);
        s.logits = (float*) (b + o_log); s.perm = (int32_t*) (b + o_perm); s.counts = (int*) (b + o_cnt); s.offsets = (int*) (b + o_off);
        s.n_problems = (int*) (b + o_np); s.problems = (GemvProblem*) (b + o_prob); s.dst0 = (int*) (b + o_dst);
        s.counts_local = (int*) (b + o_cl); s.send_off = (int*) (b + o_so);
    }
    return s;
}
PeerPtrs peer_ptrs(const void* const* ptrs, int world, const char* what)
{
    PeerPtrs p{};
    if (!ptrs) throw std::runtime_error(std::string("moe p2p: null ") + what + " pointer list");
    for (int i = 0; i < world; ++i) {
        if (!ptrs[i]) throw std::runtime_error(std::string("moe p2p: null ") + what + " pointer of a rank");
        p.p[i] = const_cast<void*>(ptrs[i]);
    }
    return p;
}
void check_p2p_world(int rank, int world, int n_experts, int n_local)
{
    if (world < 1 || world > kMaxPeers) throw std::runtime_error("moe p2p: world must be in 1..=8");
    if (rank < 0 || rank >= world) throw std::runtime_error("moe p2p: rank out of range");
    if (n_local < 1 || n_local * world != n_experts) throw std::runtime_error("moe p2p: experts must split evenly over the ranks");
    if (n_experts > 1024 || n_experts % 32) throw std::runtime_error("moe p2p: n_experts must be a multiple of 32 up to 1024");
}
}  // namespace

extern "C" size_t berth_moe_p2p_send_workspace_bytes(int T, int n_experts, int top_k, int world)
{
    if (T < 1 || n_experts < 1 || top_k < 1 || world < 1 || n_experts % world) return 0;
    return carve_p2p_send(nullptr, T, n_experts, top_k, world, n_experts / world).bytes + 512;
}

extern "C" int berth_moe_p2p_send(const void* x, int T, const void* w_router, const float* router_bias, int hidden, int n_experts,
                                  int top_k, int32_t* topk_idx, float* topk_w, int32_t* inv, int rank, int world, unsigned epoch,
                                  const void* const* cnt_all, const void* const* flags, const void* const* recv_rows, int max_rows,
                                  void* ws, size_t ws_bytes, void* stream)
{
    CallState& st = moe_state();
    return guarded(st, [&] {
        if (!w_router || !ws || (T > 0 && (!x || !topk_idx || !topk_w || !inv))) throw std::runtime_error("moe p2p send: null device pointer");
        if (T < 0) throw std::runtime_error("moe p2p send: T must not be negative");   // a rank without tokens still joins the exchange
        if (hidden < 32 || hidden % 32) throw std::runtime_error("moe p2p send: hidden must be a multiple of 32");
        if (top_k < 1 || top_k > 32 || top_k > n_experts) throw std::runtime_error("moe p2p send: top_k must be in 1..=32");
        const int n_local = world > 0 ? n_experts / world : 0;
        check_p2p_world(rank, world, n_experts, n_local);
        if (ws_bytes < berth_moe_p2p_send_workspace_bytes(std::max(T, 1), n_experts, top_k, world))
            throw std::runtime_error("moe p2p send: workspace too small");
        const PeerPtrs pc = peer_ptrs(cnt_all, world, "count table"), pf = peer_ptrs(flags, world, "flag"), pr = peer_ptrs(recv_rows, world, "receive buffer");
        const int device = current_device();
        unsigned* status = gemv_workspace(device).status;
        cudaStream_t cs = (cudaStream_t) stream;
        const int R = T * top_k;
        void* base = reinterpret_cast<void*>((reinterpret_cast<uintptr_t>(ws) + 255) & ~uintptr_t(255));
        const P2pSendWs s = carve_p2p_send(base, std::max(T, 1), n_experts, top_k, world, n_local);
        ExpertScratch es{};
        es.counts = s.counts; es.offsets = s.offsets; es.n_problems = s.n_problems; es.problems = s.problems;
        es.max_problems = std::max(T, 1) * top_k / 8 + n_experts;   // as carve_p2p_send sized the table
        if (T > 0) {
            router_topk(x, w_router, router_bias, topk_idx, topk_w, s.logits, T, hidden, n_experts, top_k, cs);
            dispatch(topk_idx, R, 0, n_experts, 8, es, s.perm, inv, cs);
        } else {
            cuda_ok(cudaMemsetAsync(s.counts, 0, size_t(n_experts) * 4, cs), "moe p2p send: clear counts");
        }
        k_ep_publish_tables<<<1, 1024, 0, cs>>>(s.counts, pc, pf, rank, world, n_experts, n_local, epoch, s.dst0, s.counts_local, s.send_off, status);
        cuda_ok(cudaGetLastError(), "k_ep_publish_tables launch");
        if (R > 0) {
            k_ep_dispatch<<<std::min((R + 7) / 8, 148 * 4), 256, 0, cs>>>((const __half*) x, s.perm, s.offsets, s.dst0, pr, n_experts, n_local, top_k, hidden, R,
                                                               max_rows, status);
            cuda_ok(cudaGetLastError(), "k_ep_dispatch launch");
        }
        k_ep_barrier<<<1, 32, 0, cs>>>(pf, 1, rank, world, epoch, status);
        cuda_ok(cudaGetLastError(), "k_ep_barrier launch");
        st.launch = "k_moe_router_logits + k_moe_topk + k_moe_count/scan/scatter + k_ep_publish_tables + k_ep_dispatch + k_ep_barrier";
    });
}

extern "C" size_t berth_moe_p2p_experts_workspace_bytes(int max_rows, int n_local, int hidden, int inter)
{
    if (max_rows < 1 || n_local < 1 || hidden < 128 || inter < 128) return 0;
    size_t es = 0;
    for (int h : kPlanHints) es = std::max(es, carve_experts(nullptr, max_rows, n_local + 1, hidden, inter, expert_plan(h)).bytes);
    return align256(size_t(max_rows) * hidden * 2) + es + 1024;
}

extern "C" int berth_moe_p2p_experts(const berth_moe_weights* w, const void* x_local, int T_local, void* ysh, int rank, int world,
                                     unsigned epoch, int n_experts_total, int top_k, int send_tokens, const void* const* cnt_all,
                                     const void* const* flags, const void* const* recv_rows, const void* const* ret_rows, int max_rows,
                                     int max_send, int rows_hint, void* send_ws, void* ws, size_t ws_bytes, void* stream)
{
    CallState& st = moe_state();
    return guarded(st, [&] {
        check_moe_shapes(w, 1);
        if (!send_ws || !ws) throw std::runtime_error("moe p2p experts: null workspace");
        const int NL = w->n_experts, H = w->hidden, I = w->inter;
        check_p2p_world(rank, world, n_experts_total, NL);
        if (T_local < 0 || T_local >= max_rows) throw std::runtime_error("moe p2p experts: T_local must be below max_rows");
        const bool with_shared = ysh != nullptr && T_local > 0;
        if (with_shared && (!x_local || !shared_behind_stacks(w)))
            throw std::runtime_error("moe p2p experts: the shared expert must be stored behind the expert stacks to run here");
        if (ws_bytes < berth_moe_p2p_experts_workspace_bytes(max_rows, NL, H, I)) throw std::runtime_error("moe p2p experts: workspace too small");
        const PeerPtrs pc = peer_ptrs(cnt_all, world, "count table"), pf = peer_ptrs(flags, world, "flag");
        const PeerPtrs pr = peer_ptrs(recv_rows, world, "receive buffer"), pt = peer_ptrs(ret_rows, world, "return buffer");
        const int device = current_device();
        const DeviceInfo& info = device_info(device);
        if (info.major != 10) throw std::runtime_error("moe p2p experts: no linked kernel for this GPU (library is built for sm_100a only)");
        const GemvScratch sc = gemv_workspace(device);
        cudaStream_t cs = (cudaStream_t) stream;
        void* sbase = reinterpret_cast<void*>((reinterpret_cast<uintptr_t>(send_ws) + 255) & ~uintptr_t(255));
        const P2pSendWs sw = carve_p2p_send(sbase, std::max(send_tokens, 1), n_experts_total, top_k, world, NL);
        const int TS = with_shared ? T_local : 0, NM = with_shared ? NL + 1 : NL;
        const ExpertPlan plan = expert_plan(std::max(rows_hint, 1));
        char* b = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(ws) + 255) & ~uintptr_t(255));
        __half* yr = reinterpret_cast<__half*>(b);
        b += align256(size_t(max_rows) * H * 2);
        ExpertScratch es = carve_experts(b, max_rows, NM, H, I, plan);
        es.counts = sw.counts_local;
        __half* xr = static_cast<__half*>(pr.p[rank]);
        RowSource in_place{};
        in_place.paired = up_behind_gate(w, NM);
        launch_pdl(k_moe_scan, dim3(1), dim3(1024), 0, cs, "k_moe_scan launch", es.counts, es.offsets, es.problems, es.n_problems, NL, plan.chunk, TS,
                   in_place.paired ? max_rows : 0, NM, es.max_problems, max_rows, sc.status);
        cuda_ok(cudaGetLastError(), "k_moe_scan launch");
        if (TS) {
            k_rows_to_offset<<<std::min(TS, 148 * 8), 256, 0, cs>>>((const __half*) x_local, xr, es.offsets + NL, TS, H, max_rows);
            cuda_ok(cudaGetLastError(), "k_rows_to_offset launch");
        }
        st.launch = experts(w, w->gate_trellis, w->up_trellis, w->down_trellis, w->gate_suh, w->gate_svh, w->up_suh, w->up_svh,
                            w->down_suh, w->down_svh, NM, xr, yr, 0, max_rows, plan, es, sc, info.sms, cs, es.offsets + NM, in_place);
        k_ep_return<<<148 * 4, 256, 0, cs>>>(yr, es.offsets, pc, sw.send_off, pt, rank, world, n_experts_total, NL, H, max_rows, max_send, sc.status);
        cuda_ok(cudaGetLastError(), "k_ep_return launch");
        k_ep_barrier<<<1, 32, 0, cs>>>(pf, 2, rank, world, epoch, sc.status);
        cuda_ok(cudaGetLastError(), "k_ep_barrier launch");
        if (TS) {
            k_rows_from_offset<<<std::min(TS, 148 * 8), 256, 0, cs>>>(yr, (__half*) ysh, es.offsets + NL, TS, H, max_rows);
            cuda_ok(cudaGetLastError(), "k_rows_from_offset launch");
        }
        st.launch = "k_moe_scan + 3 x (" + st.launch + ") + k_silu_mul_rows + k_ep_return + k_ep_barrier";
    });
}

extern "C" size_t berth_moe_workspace_bytes(int T, int hidden, int inter, int shared_inter, int n_experts, int top_k)
{
    if (T < 1 || hidden < 128 || inter < 128 || n_experts < 1 || top_k < 1) return 0;
    const int R = T * top_k;
    // sized for the layout with the shared expert's rows behind the routed ones (T more rows, one more matrix)
    const ExpertScratch es = carve_experts(nullptr, R + T, n_experts + 1, hidden, inter, expert_plan(routed_rows_hint(T, top_k, n_experts, hidden, inter)));
    size_t total = 0;
    total += align256(size_t(T) * n_experts * 4);            // logits
    total += 2 * align256(size_t(R) * 4);                    // perm, inv
    total += align256(size_t(R + T) * hidden * 2);           // yr
    total += es.bytes;
    if (shared_inter > 0) {
        total += 3 * align256(size_t(T) * shared_inter * 2);                 // shared gate, up outputs + rotated
        total += align256(size_t(T) * hidden * 2) * 2;                        // shared out, rotated input
    }
    return total + 4096;
}

extern "C" int berth_moe_layer(const berth_moe_weights* w, const void* x, int T, void* out, int32_t* topk_idx, float* topk_w,
                               void* workspace, size_t workspace_bytes, void* stream)
{
    CallState& st = moe_state();
    return guarded(st, [&] {
        check_moe_shapes(w, T, true);
        if (!x || !out || !topk_idx || !topk_w || !workspace) throw std::runtime_error("moe layer: null device pointer");
        if (!w->w_router || !w->gate_trellis || !w->up_trellis || !w->down_trellis || !w->gate_suh || !w->gate_svh ||
            !w->up_suh || !w->up_svh || !w->down_suh || !w->down_svh)
            throw std::runtime_error("moe layer: null weight pointer");
        const size_t need = berth_moe_workspace_bytes(T, w->hidden, w->inter, w->shared_inter, w->n_experts, w->top_k);
        if (workspace_bytes < need)
            throw std::runtime_error("moe layer: workspace of " + std::to_string(workspace_bytes) + " bytes is smaller than the " +
                                     std::to_string(need) + " required");
        const int device = current_device();
        const DeviceInfo& info = device_info(device);
        if (info.major != 10) throw std::runtime_error("moe layer: no linked kernel for this GPU (library is built for sm_100a only)");
        GemvScratch sc = gemv_workspace(device);
        cudaStream_t cs = (cudaStream_t) stream;
        const int H = w->hidden, I = w->inter, E = w->n_experts, K = w->top_k, R = T * K, SI = w->shared_inter;
        const ExpertPlan plan = expert_plan(routed_rows_hint(T, K, E, H, I));

        char* b = static_cast<char*>(workspace);
        b = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(b) + 255) & ~uintptr_t(255));
        auto take = [&](size_t bytes) { char* p = b; b += align256(bytes); return p; };
        float* logits = (float*) take(size_t(T) * E * 4);
        int32_t* perm = (int32_t*) take(size_t(R) * 4);
        int32_t* inv = (int32_t*) take(size_t(R) * 4);
        // A shared expert whose tensors sit directly behind the expert stacks (and has the experts' shape) is
        // run as matrix E of the grouped launches: its rows are the layer's own tokens, appended to the routed rows.
        const bool fused_shared = shared_behind_stacks(w);
        const int RT = fused_shared ? R + T : R, NM = fused_shared ? E + 1 : E;
        __half* yr = (__half*) take(size_t(R + T) * H * 2);
        ExpertScratch es = carve_experts(b, RT, NM, H, I, plan);
        b += carve_experts(nullptr, R + T, E + 1, H, I, plan).bytes;

        router_topk(x, w->w_router, w->router_bias, topk_idx, topk_w, logits, T, H, E, K, cs);
        const bool paired = up_behind_gate(w, NM);
        dispatch(topk_idx, R, 0, E, plan.chunk, es, perm, inv, cs, fused_shared ? T : 0, paired ? RT : 0, NM);
        // the rotation kernel of gate and up gathers the routed rows (and the shared expert's) from x itself
        RowSource rows_from{};
        rows_from.perm = perm; rows_from.div = K; rows_from.n_perm = R;
        rows_from.paired = paired;
        st.launch = experts(w, w->gate_trellis, w->up_trellis, w->down_trellis, w->gate_suh, w->gate_svh, w->up_suh, w->up_svh,
                            w->down_suh, w->down_svh, NM, x, yr, RT, RT, plan, es, sc, info.sms, cs, nullptr, rows_from);

        __half* ysh = fused_shared ? yr + size_t(R) * H : nullptr;
        if (SI > 0 && !fused_shared) {
            if (!w->sh_gate_trellis || !w->sh_up_trellis || !w->sh_down_trellis) throw std::runtime_error("moe layer: null shared-expert pointer");
            __half* sg = (__half*) take(size_t(T) * SI * 2);
            __half* su = (__half*) take(size_t(T) * SI * 2);
            __half* sr = (__half*) take(size_t(T) * SI * 2);     // rotated-input scratch of the down projection
            ysh = (__half*) take(size_t(T) * H * 2);
            __half* xrot = (__half*) take(size_t(T) * H * 2);    // rotated-input scratch of gate / up
            linear_rows(x, w->sh_gate_trellis, sg, w->sh_gate_suh, xrot, w->sh_gate_svh, T, H, SI, w->k_bits, w->codebook, 0, cs);
            linear_rows(x, w->sh_up_trellis, su, w->sh_up_suh, xrot, w->sh_up_svh, T, H, SI, w->k_bits, w->codebook, 0, cs);
            if (berth_ops_silu_mul(sg, su, sg, int64_t(T) * SI, 0.0f, cs) != 0) throw std::runtime_error(berth_ops_last_error());
            linear_rows(sg, w->sh_down_trellis, ysh, w->sh_down_suh, sr, w->sh_down_svh, T, SI, H, w->k_bits, w->codebook, 0, cs);
        }
        launch_pdl(k_moe_combine, dim3(T, (H + 511) / 512), dim3(256), 0, cs, "k_moe_combine launch", yr, inv, topk_w, ysh, (float*) out, H, K, R);
        cuda_ok(cudaGetLastError(), "k_moe_combine launch");
        st.launch = std::string("k_moe_router_logits + k_moe_topk + ") + (R <= kSmallKeys ? "k_moe_dispatch_small" : "k_moe_count/scan/scatter") +
                    " + " + st.launch + " + k_moe_combine" + (fused_shared ? " [shared expert as matrix E of the grouped launches]" : "");
    });
}
