// EXL3 decode linear for the MUL1 codebook (size_m <= 8) on the 5th-generation tensor cores'
// integer path, with the decoded weights in TENSOR MEMORY.
//
// Why a second decode kernel.  On this SM the legacy warp-level MMA (mma.sync) executes on the same
// pipe as lop3 / prmt / shf and holds it for 8 cycles per instruction, so in the fp16 decode kernel
// (gemv.cu) the tensor-core instruction competes with the window extraction for the one pipe that
// already binds.  tcgen05.mma is asynchronous and takes no issue slot of the decoding warps.  And
// for MUL1 a weight is S*(1024 + u) + B with u = the byte sum of x = state * 0x83DCD12D: the 32-bit
// register x is four u8 k-slots of a kind::i8 MMA, so against an activation replicated over the
// four slots the tensor core forms the byte sum by itself.  Per weight the decoding warps are left
// with the window extraction and ONE multiply; the fp16 path spends a multiply, a dp4a, half a
// byte permute and an eighth of an 8-cycle mma.sync on top of the extraction.
//
// Arithmetic.  sum_k a_k w_k = S * sum_k a_k u_k + (1024 S + B) * sum_k a_k.  The rotated activations
// enter as 16-bit block fixed point: per (row, 128 rotated inputs) one fp32 scale = max|a| / 32512 and
// v = rint(a / scale), split into two signed 8-bit limbs v = 256 hi + lo.  The limbs of a row are two
// of the N columns of the MMA; the s32 accumulation is exact and is folded into an fp32 accumulator
// once per 128 inputs: acc += scale * (256 hi_sum + lo_sum).  The constant term uses the same
// quantised values (block sums = scale * sum v), so the result is exactly the product with the
// quantised activations up to fp32 rounding; the quantisation step is 2^-15 of the block maximum,
// finer than the fp16 rounding of the rotated activations that every path of this library shares.
//
// Work decomposition, TMA ring, split-K slabs and the finishing kernel are those of gemv.cu: units of
// 128 inputs x BU*128 outputs in band-group-major order, CTA c takes a contiguous range.  Inside a CTA
// (22 warps, one CTA per SM):
//   warp 20      TMA producer: per unit one 3-D box of trellis words into a ring stage, and (unless the CTA
//                rotates its activations itself, see FUSED below) one bulk copy of the unit's activation limbs;
//   warps 0..15  decode: warp (quarter q, stream s) takes tile columns 2q, 2q+1 of one band -- the
//                output columns whose TMEM lanes it may write -- for half of the unit's k-tile rows:
//                shared-memory words -> eight states -> eight products x -> one tcgen05.st per tile
//                (the lane layout of the tile format is the 16x128b store shape); the eight warps of a
//                half-unit fill one tensor-memory stage and hand it over through an mbarrier;
//   warp 21      allocates tensor memory; one elected lane issues per half-unit stage BU*8 MMAs
//                (M = 128 output columns, N = 16 limb columns, K = 32 bytes = 8 weights), A from
//                tensor memory, B = the limb tile in shared memory (K-major, no swizzle), D = s32 in
//                tensor memory, double buffered per unit; commits release the stage, the ring stage
//                and publish the accumulator;
//   warps 16..19 epilogue: thread = output column; reads the unit's s32 sums (tcgen05.ld), applies
//                the block scales, and at the end of a segment writes the split-K slab or finishes
//                the band (affine correction, Hadamard, svh) as gemv.cu does.
// Every wait is bounded; a wait that runs out sets a status bit, the kernel carries on with whatever
// is there, frees its tensor memory and returns.
//
// Roofline: HBM.  Algorithmic bytes per launch = K*N*BITS/8 + 2K + 2N + 2MK + out_bytes*M*N.
#include "gemv_common.cuh"
#include "../../include/berth_b200.h"

#include <algorithm>

namespace berth {
namespace {

constexpr int kDecodeWarps = 16;
constexpr int kEpiWarp0 = 16, kEpiWarps = 4;
constexpr int kProducerWarp = 20, kMmaWarp = 21;
constexpr int kThreads = 22 * 32;
constexpr int kEpiThreads = kEpiWarps * 32;
constexpr int kSmemBudget = 227 * 1024;

// Compile-time geometry: BITS bits per weight, NB groups of four rows (two limb columns each); FUSED = the
// limb tiles of all the CTA's units live in a shared-memory area of their own instead of the ring stages.
template <int BITS, int NB, bool FUSED>
struct GeoI8 {
    static constexpr int NW = 8 * BITS;
    static constexpr int BU = BITS <= 4 ? 2 : 1;
    static constexpr int TILE_COLS = 8 * BU;
    static constexpr int ROW_BYTES = TILE_COLS * NW * 4;
    static constexpr int W_BYTES = 8 * ROW_BYTES;
    static constexpr int CHUNK_BYTES = NB * 256;               // limbs of 8 weights-k: NB groups of 8 rows x 32 bytes
    static constexpr int L_BYTES = 16 * CHUNK_BYTES;           // limbs of one unit: 16 MMA k-steps
    static constexpr int B_BYTES = L_BYTES + 128;              // ... followed by the unit's block scales and block sums (16 fp32 each)
    static_assert(NB <= 4, "the 128-byte tail of a limb record holds 16 rows");
    static constexpr int STAGE_BYTES = FUSED ? W_BYTES : W_BYTES + B_BYTES;
    static constexpr int TOK = 4 * NB;
    static constexpr int NCOL = NB <= 2 ? 16 : 8 * NB;         // N of the MMA (16 is the least for M = 128)
    static constexpr int PITCH = BU * 128 + 4;
    static constexpr int OUT_FLOATS = TOK * PITCH;
    static constexpr int D_COLS = 2 * BU * NCOL;               // two accumulator buffers
    static constexpr int A_STAGE_COLS = BU * 64;               // half a unit: 4 k-tile rows x 16 columns per band
    static constexpr int NA_RAW = (512 - D_COLS) / A_STAGE_COLS;
    static constexpr int NA = NA_RAW > 4 ? 4 : NA_RAW;
    static constexpr int kBarBytes = 512;
    static constexpr int RING_MAX = kSmemBudget - 1024 - OUT_FLOATS * 4 - kBarBytes - 64;
    static constexpr int kMinArea = 80 * 1024;                 // in-kernel rotation: least size of the limb area
    static constexpr int S_RAW = (RING_MAX - (FUSED ? kMinArea : 0)) / STAGE_BYTES;
    static constexpr int S = S_RAW > 12 ? 12 : S_RAW;
    static constexpr int AREA_BYTES = FUSED ? RING_MAX - S * STAGE_BYTES : 0;
    static constexpr size_t SMEM = 1024 + size_t(S) * STAGE_BYTES + OUT_FLOATS * 4 + kBarBytes + AREA_BYTES;
    // in-kernel rotation: a unit's limb tile holds 2*rows limb rows per core matrix (rows = 1, 2 or 4), core
    // matrices 32*rows bytes apart, 16 k-steps of two core matrices, plus four scales and four block sums; 512 bytes of the area stay
    // free because the MMA reads whole 8-row core matrices (the rows past 2*rows are never used)
    __host__ __device__ static constexpr int fused_tile_bytes(int rows) { return 1024 * rows; }
    __host__ __device__ static constexpr int fused_max_units(int rows) { return (AREA_BYTES - 512) / (fused_tile_bytes(rows) + 32); }
    static_assert(S >= 2 && NA >= 2, "ring and tensor-memory stages");
    static_assert(W_BYTES % 128 == 0 && STAGE_BYTES % 128 == 0, "TMA destination alignment");
    static_assert((2 * S + 2 * NA + 4) * 8 <= kBarBytes, "barrier area");
};

// ---------------------------------------------------------------- tcgen05 wrappers
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]^T, kind::i8: A = 128 rows x 32 u8 in tensor memory (lane = row, four
// k-slots per 32-bit column), B = N rows x 32 s8 K-major in shared memory, D = 128 lanes x N s32 columns.
__device__ __forceinline__ void tc_mma_ts_i8(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Instruction descriptor: D s32, A u8, B s8, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t idesc_i8(int n) { return (2u << 4) | (0u << 7) | (1u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(128 >> 4) << 24); }
// Shared-memory descriptor of a K-major operand without swizzle: 8-row x 16-byte core matrices of 128
// contiguous bytes; the next core matrix along K lies `lbo` bytes further, the next group of 8 rows `sbo` bytes.
__device__ __forceinline__ uint64_t smem_desc_kmajor(uint32_t addr, uint32_t lbo, uint32_t sbo)
{
    uint64_t d = 0;
    d |= uint64_t((addr & 0x3FFFF) >> 4);
    d |= uint64_t(lbo >> 4) << 16;     // leading byte offset: core matrices along K
    d |= uint64_t(sbo >> 4) << 32;     // stride byte offset: 8-row groups
    d |= uint64_t(1) << 46;            // descriptor version of sm_100
    return d;
}
// The products x of one tile into tensor memory: 16 lanes x 16 columns at taddr; thread 4g+q supplies
// lanes g, g+8 (output columns of the tile) and columns q, q+4 (first MMA k-step), q+8, q+12 (second).
__device__ __forceinline__ void tc_st_tile(uint32_t taddr, const uint32_t (&x)[8])
{
    asm volatile("tcgen05.st.sync.aligned.16x128b.x4.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(x[0]), "r"(x[2]), "r"(x[1]),
                 "r"(x[3]), "r"(x[4]), "r"(x[6]), "r"(x[5]), "r"(x[7])
                 : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// 32 lanes x N consecutive 32-bit columns (N = 2, 8, 16 or 32) of this warp's TMEM lane quarter; no wait.
template <int N>
__device__ __forceinline__ void tc_ld(uint32_t taddr, int* r)
{
    static_assert(N == 2 || N == 8 || N == 16 || N == 32, "tcgen05.ld width");
    if constexpr (N == 2) {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(taddr));
    } else if constexpr (N == 8) {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                     : "r"(taddr));
    } else if constexpr (N == 16) {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                     : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                       "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                     : "r"(taddr));
    } else {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
            "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
              "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
              "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
              "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
            : "r"(taddr));
    }
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ bool elect_one()
{
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory"); }

// The lane's four rotated fp16 values of one 128-block (lane = 4 consecutive inputs) -> block fixed point.
// Writes the two limbs of each value, replicated over the four bytes of a 32-bit word (the four u8 k-slots of a
// weight's product), at their place in the block's limb tile: `tile_row` = tile + (row / 4) * 256 +
// 2 * (row % 4) * 16, k-step stride `chunk_stride`, core-matrix stride `lbo` (256 * row groups and 128 in a ring
// stage).  Tile layout: [MMA k-step 16][row group]
// [core matrix 2][limb row 8][16 bytes], limb row = 2 * (row % 4) + (0 high, 1 low); k-step c of a k-tile row
// holds, in this order, the inputs 2c (c < 4) and 2(c-4)+1 of its eight.  Returns the block's scale
// (max|a| / 32512) and, in every lane, the sum of the block's 128 integers.
__device__ __forceinline__ float quantise_block(uint2 o, int lane, unsigned char* tile_row, int chunk_stride, int lbo, int& isum)
{
    const __half2 h01 = *reinterpret_cast<const __half2*>(&o.x), h23 = *reinterpret_cast<const __half2*>(&o.y);
    const float hv[4] = {__low2float(h01), __high2float(h01), __low2float(h23), __high2float(h23)};
    // the block maximum in one warp reduction: non-negative floats order as their bit patterns do; a lane of NaNs counts
    // as 0 (fmaxf drops NaNs) unless every lane is one
    float amax = fmaxf(fmaxf(fabsf(hv[0]), fabsf(hv[1])), fmaxf(fabsf(hv[2]), fabsf(hv[3])));
    const bool lane_nan = amax != amax;
    const unsigned top = __reduce_max_sync(dq::kFull, lane_nan ? 0u : __float_as_uint(amax));
    amax = __all_sync(dq::kFull, lane_nan) ? amax : __uint_as_float(top);
    // (a multiplication and an approximate division: the scale only has to be the one the sums are multiplied by later,
    // and |a| * inv stays below 32512.5)
    const float scale = __fmul_rn(amax, 1.0f / 32512.0f);
    const float inv = amax > 0.f ? __fdividef(32512.0f, amax) : 0.f;
    isum = 0;
    const int kt = lane >> 2;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const int v = __float2int_rn(__fmul_rn(hv[e], inv));
        isum += v;
        const int hi = (v + 128) >> 8, lo = v - 256 * hi;
        const int r = 4 * (lane & 3) + e;                       // input inside the k-tile row
        const int chunk = kt * 2 + (r >> 3), c = ((r & 7) >> 1) + 4 * (r & 1);
        unsigned char* w = tile_row + chunk * chunk_stride + (c >> 2) * lbo + 4 * (c & 3);
        *reinterpret_cast<uint32_t*>(w) = uint32_t(hi & 0xff) * 0x01010101u;
        *reinterpret_cast<uint32_t*>(w + 16) = uint32_t(lo & 0xff) * 0x01010101u;
    }
    isum = __reduce_add_sync(dq::kFull, isum);
    return scale;
}

// ---------------------------------------------------------------- the kernel
// FUSED (one group of four rows, dense launches in which no CTA holds a whole band group and every CTA's units fit
// the limb area): no rotation kernel runs before this one and no limb tile travels through L2; while the first weight
// stages are in flight the decoding and epilogue warps rotate and quantise the 128-block of every unit of the CTA
// into a shared-memory area of its own (tiles of 2 * rows limb rows, a quarter of the ring-stage tile for one row),
// and the CTAs that hold band group 0 also write the rotated activations and block sums for the caller and the
// finishing kernel.
// The trellis views of a launch: one 3-D map (z = matrix of an equally shaped stack), or one map per matrix of a
// launch over matrices of different widths.
struct I8Maps {
    CUtensorMap m[kMaxHetMatrices];
};

// ONE: the launch has one row (the epilogue warps then read two accumulator columns per band instead of eight and keep one
// row's sums: they share their schedulers with the decode warps).
template <int BITS, int NB, bool FUSED, bool ONE>
__global__ void __launch_bounds__(kThreads, 1) k_exl3_gemv_i8(const __grid_constant__ I8Maps maps, const GemvArgs p)
{
    static_assert(!FUSED || NB == 1, "in-kernel rotation is built for one group of four rows");
    static_assert(!ONE || FUSED, "the one-row form exists for the in-kernel rotation only");
    using G_ = GeoI8<BITS, NB, FUSED>;
    constexpr int NW = G_::NW, BU = G_::BU, ROW_BYTES = G_::ROW_BYTES, W_BYTES = G_::W_BYTES, B_BYTES = G_::B_BYTES;
    constexpr int STAGE_BYTES = G_::STAGE_BYTES, S = G_::S, NA = G_::NA, TOK = ONE ? 1 : G_::TOK, NCOL = G_::NCOL, PITCH = G_::PITCH;
    constexpr int CHUNK_BYTES = G_::CHUNK_BYTES, A_STAGE_COLS = G_::A_STAGE_COLS, D_COLS = G_::D_COLS;

    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* ring = smem;
    float* outbuf = reinterpret_cast<float*>(ring + S * STAGE_BYTES);          // [TOK][PITCH]
    uint64_t* bars = reinterpret_cast<uint64_t*>(outbuf + G_::OUT_FLOATS);
    unsigned char* area = reinterpret_cast<unsigned char*>(bars) + G_::kBarBytes;   // FUSED: limb tiles, then four scales per unit
    __shared__ uint32_t s_tmem_base;
    // FUSED: limb rows per core matrix = 2 * frows, core matrices frows * 32 bytes apart
    const int frows = p.m <= 1 ? 1 : (p.m == 2 ? 2 : 4);
    const int flbo = 32 * frows, ftile = G_::fused_tile_bytes(frows);

    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bands = p.n >> 7, kblocks = p.k >> 7;
    const int bgroups = (bands + BU - 1) / BU;
    const int nprob = p.problems ? min(max(__ldg(p.n_problems), 0), p.max_problems) : (p.n_stack > 1 ? p.n_stack : 1);
    const long long U = p.het ? (long long) p.het_bg[p.n_stack] * kblocks : (long long) nprob * bgroups * kblocks;
    // band group of the launch -> matrix and band group inside it
    auto split_bg = [&](int gbg, int& pi, int& lbg) {
        if (p.het) {
            pi = 0;
            while (pi + 1 < p.n_stack && gbg >= p.het_bg[pi + 1]) ++pi;
            lbg = gbg - p.het_bg[pi];
        } else if (gbg < bgroups) {   // (one matrix: no division)
            pi = 0;
            lbg = gbg;
        } else {
            pi = gbg / bgroups;
            lbg = gbg - pi * bgroups;
        }
    };
    const int cta = blockIdx.x;
    const int G = U < (long long) gridDim.x ? int(U) : int(gridDim.x);
    if (cta >= G) {
        pdl_wait();   // a grid must not complete before its predecessors: its successor relies on that
        return;
    }
    const long long u0 = unit_begin(cta, U, G), u1 = unit_begin(cta + 1, U, G);
    const int nunits = int(u1 - u0);
    const int gbg0 = int(u0 / kblocks), kb0 = int(u0 - (long long) gbg0 * kblocks);   // the CTA's first band group and 128-block
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * S;
    const uint32_t afull0 = empty0 + 8 * S, aempty0 = afull0 + 8 * NA;
    const uint32_t dfull0 = aempty0 + 8 * NA, dempty0 = dfull0 + 16;

    // The weights are the long pole of a short launch: one lane of the producer warp arms the ring's "full" barriers
    // and issues the first stages' TMA copies before anything else in the CTA happens.
    int pr_pi = 0, pr_lbg = 0, pr_kb = 0;   // producer lane: matrix, band group and 128-block of the next unit to fetch
    const int pre = nunits < S ? nunits : S;
    // FUSED: the first kPre0 stages are requested before the CTA's set-up barrier, the rest of the first lap right after it
    // (a CTA that starts when its predecessor's last CTAs leave has this set-up on its critical path)
    constexpr int kPre0 = FUSED ? 4 : S;
    const int pre0 = pre < kPre0 ? pre : kPre0;
    constexpr uint32_t kStageTx = FUSED ? W_BYTES : STAGE_BYTES;
    auto issue_weights = [&](uint32_t dst, uint32_t bar) {
        const int z = p.problems ? load_problem(p.problems, pr_pi, p.n_matrices, TOK, p.max_rows).z : (p.het ? 0 : pr_pi);
        tma_load_3d(dst, &maps.m[p.het ? pr_pi : 0], pr_lbg * (ROW_BYTES / 8), pr_kb * 8, z, bar);
    };
    auto next_unit = [&]() {
        if (++pr_kb == kblocks) {
            pr_kb = 0;
            if (++pr_lbg == (p.het ? p.het_bg[pr_pi + 1] - p.het_bg[pr_pi] : bgroups)) { pr_lbg = 0; ++pr_pi; }
        }
    };
    if (warp == kProducerWarp && lane == 0) {
        for (int s = 0; s < S; ++s) mbar_init(full0 + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        pr_kb = kb0;
        split_bg(gbg0, pr_pi, pr_lbg);
        asm volatile("prefetch.tensormap [%0];" ::"l"(&maps.m[p.het ? pr_pi : 0]) : "memory");
        if (p.defer_weights) pdl_wait();   // the caller may have written the weights just before this launch
        for (int i = 0; i < pre0; ++i) {
            mbar_arrive_expect_tx(full0 + 8 * i, kStageTx);
            issue_weights(smem_u32(ring + i * STAGE_BYTES), full0 + 8 * i);
            if (FUSED || i + 1 < pre) next_unit();   // (the limb tiles of these stages follow below, from the same coordinates)
        }
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            // decoding warps (trellis words); when the limb tiles travel through the ring also the MMAs (limb tile) and the
            // epilogue warps (scales)
            mbar_init(empty0 + 8 * s, FUSED ? kDecodeWarps : kDecodeWarps + 1 + kEpiWarps);
        }
        for (int s = 0; s < NA; ++s) {
            mbar_init(afull0 + 8 * s, kDecodeWarps);
            mbar_init(aempty0 + 8 * s, 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(dfull0 + 8 * s, 1);
            mbar_init(dempty0 + 8 * s, kEpiWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = s_tmem_base;             // accumulators: [buffer][band][NCOL]
    const uint32_t tmem_a = tmem_d + D_COLS;         // weight stages: [NA][band][k-tile row of the half][16]
    float* fscales = reinterpret_cast<float*>(area + size_t(nunits) * ftile + 512);   // FUSED: [unit][4 scales, 4 block sums]

    if constexpr (FUSED) {
        // In-kernel rotation: while the first weight stages are in flight, the decoding and the epilogue warps
        // rotate and quantise the 128-block of every unit of the CTA (one warp per unit and row) into the limb area.
        if (warp != kProducerWarp) {
            if (warp != kMmaWarp) {
                pdl_wait();   // the activations come from the preceding kernels
                const int w20 = warp;   // decode warps 0..15, epilogue warps 16..19
                for (int task = w20; task < nunits * p.m; task += kDecodeWarps + kEpiWarps) {
                    const int j = p.m == 1 ? task : task / p.m, t = task - j * p.m;
                    int gbg = gbg0, kb = kb0 + j;   // unit u0 + j of the launch: no 64-bit division per task
                    if (kb >= kblocks) {
                        const int dg = kb >= 2 * kblocks ? kb / kblocks : 1;
                        gbg += dg;
                        kb -= dg * kblocks;
                    }
                    int pi, lbg;   // matrix of the stack, band group inside it
                    split_bg(gbg, pi, lbg);
                    float sx;
                    const uint2 o = rotate_block<false>(p.a + size_t(t) * p.k, p.het ? p.het_suh[pi] : p.suh + size_t(pi) * p.k, kb, lane, sx,
                                                               p.a_up ? p.a_up + size_t(t) * p.k : nullptr, p.act_limit);
                    int isum;
                    const float scale = quantise_block(o, lane, area + size_t(j) * ftile + t * 32, 2 * flbo, flbo, isum);
                    if (lane == 0) {
                        fscales[j * 8 + t] = scale;
                        fscales[j * 8 + 4 + t] = __fmul_rn(scale, __int2float_rn(isum));
                    }
                    if (lbg == 0) {   // band group 0 of a matrix meets every 128-block exactly once: the caller's copy
                        __half* ah = p.het ? p.het_a_had[pi] + size_t(t) * p.k : p.a_had + (size_t(pi) * p.m + t) * p.k;
                        *reinterpret_cast<uint2*>(ah + kb * 128 + lane * 4) = o;
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the MMA reads the tiles through the async proxy
            }
            asm volatile("bar.sync 2, %0;" ::"n"((kDecodeWarps + kEpiWarps + 1) * 32) : "memory");   // tiles and scales are in place
        }
    }

    if (warp == kProducerWarp) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            auto issue_limbs = [&](int pi, int kb, uint32_t dst, uint32_t bar) {
                bulk_load_1d(dst, reinterpret_cast<const unsigned char*>(p.afrag) + (size_t(pi) * kblocks + kb) * B_BYTES, B_BYTES, bar);
            };
            for (int i = pre0; i < pre; ++i) {   // FUSED: the rest of the first lap
                mbar_arrive_expect_tx(full0 + 8 * i, kStageTx);
                issue_weights(smem_u32(ring + i * STAGE_BYTES), full0 + 8 * i);
                next_unit();
            }
            pdl_wait();
            if constexpr (!FUSED) {
                // the limb tiles of the stages whose weights are already on their way: replay the coordinates from u0
                int gbg = int(u0 / kblocks);
                int kb = int(u0 - (long long) gbg * kblocks);
                for (int i = 0; i < pre; ++i) {
                    int pi, lbg;
                    split_bg(gbg, pi, lbg);
                    issue_limbs(pi, kb, smem_u32(ring + i * STAGE_BYTES + W_BYTES), full0 + 8 * i);
                    if (++kb == kblocks) { kb = 0; ++gbg; }
                }
                if (pre > 0) next_unit();
            }
            int s = 0, lap = 1;
            for (int i = pre; i < nunits; ++i) {
                mbar_wait_parked(empty0 + 8 * s, (lap - 1) & 1, p.status, kStEmptyTimeout);
                mbar_arrive_expect_tx(full0 + 8 * s, kStageTx);
                const uint32_t dst = smem_u32(ring + s * STAGE_BYTES);
                issue_weights(dst, full0 + 8 * s);
                if constexpr (!FUSED) issue_limbs(pr_pi, pr_kb, dst + W_BYTES, full0 + 8 * s);
                next_unit();
                if (++s == S) { s = 0; ++lap; }
            }
        }
    } else if (warp < kDecodeWarps) {
        // ------------------------------------------------------------ decode warps
        const int quarter = warp & 3, stream = warp >> 2;
        const int band_l = BU == 2 ? (stream & 1) : 0;              // band of the unit this warp decodes
        constexpr int NROWS = BU == 2 ? 2 : 1;                      // k-tile rows per warp and half-unit stage
        const int r0 = BU == 2 ? 2 * (stream >> 1) : stream;        // first of them inside the half
        const int lane1 = (lane + 1) & 31;
        // the warp's first tile inside a ring stage, and its first tensor-memory address inside a weight stage
        const int word0 = r0 * (ROW_BYTES / 4) + (band_l * 8 + 2 * quarter) * NW;
        const uint32_t taddr0 = tmem_a + (uint32_t(32 * quarter) << 16) + band_l * 64 + 16 * r0;
        int s = 0, phase = 0;
        int a_idx = 0, a_par = 1;   // weight stage in tensor memory and the parity of its "released" barrier (first lap: free)
        int pending = -1;           // weight stage whose stores are issued but not yet handed over
        // The hand-over of a stage (wait for its stores, fence, arrive) is deferred until the first tiles of the
        // next stage are decoded, so that the store latency hides behind that work.
        auto hand_over = [&]() {
            if (pending >= 0) {
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(afull0 + 8 * pending);
                pending = -1;
            }
        };
        for (int i = 0; i < nunits; ++i) {
            mbar_wait(full0 + 8 * s, phase, p.status, kStFullTimeout);   // (tight polling: a parked wait wakes up too late here)
            const uint32_t* stage = reinterpret_cast<const uint32_t*>(ring + s * STAGE_BYTES) + word0;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t taddr = taddr0 + a_idx * A_STAGE_COLS;
#pragma unroll
                for (int rr = 0; rr < NROWS; ++rr) {
                    const uint32_t* rowp = stage + (4 * h + rr) * (ROW_BYTES / 4);
                    uint32_t x[2][8];
#pragma unroll
                    for (int t = 0; t < 2; ++t) {
                        uint32_t st[8];
                        dq::tile_states_i8<BITS>(rowp + t * NW, lane, lane1, st);
#pragma unroll
                        for (int j = 0; j < 8; ++j) x[t][j] = st[j] * 0x83DCD12Du;
                    }
                    if (rr == 0) {
                        hand_over();
                        // the MMAs that read this weight stage one lap ago are done (first lap: passes at once)
                        mbar_wait(aempty0 + 8 * a_idx, a_par, p.status, kStTmemTimeout);
                        tc_fence_after();
                    }
#pragma unroll
                    for (int t = 0; t < 2; ++t) tc_st_tile(taddr + (uint32_t(16 * t) << 16) + 16 * rr, x[t]);
                }
                pending = a_idx;
                if (++a_idx == NA) { a_idx = 0; a_par ^= 1; }
                if (i == 0 && h == 0) hand_over();   // the launch's first stage: the MMA warp is waiting for it
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * s);   // every word of the ring stage has been read
            if (++s == S) { s = 0; phase ^= 1; }
        }
        hand_over();
    } else if (warp == kMmaWarp) {
        // ------------------------------------------------------------ MMA issuer
        // The whole warp runs the loop and one elected lane issues, so that addresses and descriptors live in
        // uniform registers.
        const uint32_t idesc = idesc_i8(NCOL);
        // With one group of four rows the second group of eight limb rows the MMA asks for (N = 16) aliases the
        // next k-step's rows: those eight accumulator columns are never read.
        constexpr uint32_t kSbo = 256;
        int s = 0, phase = 0, a_idx = 0, a_par = 0;
        for (int i = 0; i < nunits; ++i) {
            const int buf = i & 1;
            if constexpr (!FUSED) mbar_wait_suspended(full0 + 8 * s, phase, p.status, kStFullTimeout);   // the unit's limb tile has landed
            if (i >= 2) mbar_wait_suspended(dempty0 + 8 * buf, ((i >> 1) - 1) & 1, p.status, kStTmemTimeout);   // accumulator drained
            const uint64_t b_desc0 = FUSED ? smem_desc_kmajor(smem_u32(area + size_t(i) * ftile), flbo, 2 * flbo)
                                           : smem_desc_kmajor(smem_u32(ring + s * STAGE_BYTES + W_BYTES), 128, kSbo);
            const uint32_t chunk_step = FUSED ? uint32_t(2 * flbo) >> 4 : uint32_t(CHUNK_BYTES) >> 4;
            const uint32_t d_base = tmem_d + buf * (BU * NCOL);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                mbar_wait_suspended(afull0 + 8 * a_idx, a_par, p.status, kStTmemTimeout);
                tc_fence_after();
                const uint32_t a_base = tmem_a + a_idx * A_STAGE_COLS;
                if (elect_one()) {
#pragma unroll
                    for (int b = 0; b < BU; ++b)
#pragma unroll
                        for (int r = 0; r < 4; ++r)
#pragma unroll
                            for (int j = 0; j < 2; ++j) {
                                const int chunk = (4 * h + r) * 2 + j;
                                tc_mma_ts_i8(d_base + b * NCOL, a_base + b * 64 + r * 16 + 8 * j,
                                             b_desc0 + uint64_t(chunk * chunk_step), idesc, (h | r | j) ? 1u : 0u);
                            }
                    tc_commit(aempty0 + 8 * a_idx);
                    if (h == 1) {
                        tc_commit(dfull0 + 8 * buf);
                        if constexpr (!FUSED) tc_commit(empty0 + 8 * s);
                    }
                }
                __syncwarp();
                if (++a_idx == NA) { a_idx = 0; a_par ^= 1; }
            }
            if (++s == S) { s = 0; phase ^= 1; }
        }
    } else {
        // ------------------------------------------------------------ epilogue warps
        const int ew = warp - kEpiWarp0;                      // 0..3 = TMEM lane quarter
        const int et = ew * 32 + lane;                        // output column inside a band = TMEM lane
        const uint32_t lane_base = uint32_t(32 * ew) << 16;
        // Activations (or their limb tiles and block sums) come from the preceding kernels.
        pdl_wait();
        const int slab_rows = p.m;
        const size_t slab_floats = size_t(slab_rows) * BU * 128;
        const size_t slab_stride = slab_floats + 32;          // ... followed by the rows' partial sums of the activations
        __shared__ int s_last;
        int ui = 0, rs = 0, rphase = 0;
        long long u = u0;
        while (u < u1) {
            const Segment sg = segment_at(u, u0, u1, kblocks);
            int pi, lbg;
            split_bg(sg.bg, pi, lbg);
            ProblemView pv = problem_view(p, pi, TOK);
            if (p.het) {
                pv.z = 0; pv.act = pi;
                pv.svh = p.het_svh[pi]; pv.c = p.het_c[pi]; pv.ldc = p.het_n[pi];
            }
            const int bands_pi = p.het ? p.het_n[pi] >> 7 : bands;
            const int rows = min(pv.rows, TOK), row0 = pv.row0;
            float acc[BU][TOK], sxp[TOK];   // per row: dot products of this thread's column(s); sum of the quantised activations
#pragma unroll
            for (int t = 0; t < TOK; ++t) {
                sxp[t] = 0.f;
#pragma unroll
                for (int b = 0; b < BU; ++b) acc[b][t] = 0.f;
            }
            for (int j = 0; j < sg.units; ++j, ++ui) {
                const int buf = ui & 1;
                float sc[TOK], bs[TOK];
                if constexpr (FUSED) {
#pragma unroll
                    for (int t = 0; t < TOK; ++t) {
                        sc[t] = t < rows ? fscales[ui * 8 + t] : 0.f;
                        bs[t] = t < rows ? fscales[ui * 8 + 4 + t] : 0.f;
                    }
                } else {
                    // the unit's block scales and block sums travel with its limb tile
                    mbar_wait_suspended(full0 + 8 * rs, rphase, p.status, kStFullTimeout);
                    const float* scp = reinterpret_cast<const float*>(ring + rs * STAGE_BYTES + W_BYTES + G_::L_BYTES);
#pragma unroll
                    for (int t = 0; t < TOK; ++t) {
                        sc[t] = t < rows ? scp[t] : 0.f;
                        bs[t] = t < rows ? scp[16 + t] : 0.f;
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(empty0 + 8 * rs);
                    if (++rs == S) { rs = 0; rphase ^= 1; }
                }
                mbar_wait_suspended(dfull0 + 8 * buf, (ui >> 1) & 1, p.status, kStTmemTimeout);
                tc_fence_after();
                const uint32_t d_base = tmem_d + buf * (BU * NCOL) + lane_base;
                // the unit's s32 sums: column 2t = high-limb sum of row t, 2t+1 = low-limb sum
                int r[BU][2 * TOK];
#pragma unroll
                for (int b = 0; b < BU; ++b) tc_ld<2 * TOK>(d_base + b * NCOL, r[b]);
                tc_wait_ld();
                tc_fence_before();   // the accumulator buffer is in registers: hand it back before the arithmetic
                __syncwarp();
                if (lane == 0) mbar_arrive(dempty0 + 8 * buf);
#pragma unroll
                for (int t = 0; t < TOK; ++t) {
                    sxp[t] = __fadd_rn(sxp[t], bs[t]);
#pragma unroll
                    for (int b = 0; b < BU; ++b)
                        acc[b][t] = __fmaf_rn(sc[t], __int2float_rn(r[b][2 * t] * 256 + r[b][2 * t + 1]), acc[b][t]);
                }
            }
            // ---- the segment's sums: thread et owns column et of every band
            constexpr int kTasksPerWarp = (TOK * BU + kEpiWarps - 1) / kEpiWarps;
            if (sg.whole) {
                // the CTA held the band group's whole K: finish the bands here
#pragma unroll
                for (int tok = 0; tok < TOK; ++tok)
                    if (tok < rows)
#pragma unroll
                        for (int b = 0; b < BU; ++b) outbuf[tok * PITCH + b * 128 + et] = acc[b][tok];
                epi_sync();   // outbuf complete
#pragma unroll
                for (int q = 0; q < kTasksPerWarp; ++q) {
                    const int task = ew + q * kEpiWarps, row = task / BU, b = task - row * BU, band = lbg * BU + b;
                    if (row < rows && band < bands_pi) {   // (ragged last band group)
                        float sx = 0.f;
#pragma unroll
                        for (int t = 0; t < TOK; ++t) sx = t == row ? sxp[t] : sx;
                        const uint2 sv = __ldg(reinterpret_cast<const uint2*>(pv.svh + band * 128 + lane * 4));
                        const float4 t4 = *reinterpret_cast<const float4*>(outbuf + row * PITCH + b * 128 + lane * 4);
                        float v[4] = {t4.x, t4.y, t4.z, t4.w};
                        finish_band<2>(v, sx, lane, sv, band, pv.c, size_t(row0 + row), pv.ldc, p.out_fp32, p.argmax, p.residual, p.sample);
                    }
                }
                epi_sync();   // outbuf is free again
            } else {
                // K was split: leave the partial sums in this CTA's slab; the CTA that arrives last at the band group's
                // counter sums the group's slabs in CTA order (so the result does not depend on who was last) and
                // finishes the bands.  Nobody waits for anybody.
                float* slab = p.slabs + size_t(sg.head ? 2 * cta : 2 * cta + 1) * slab_stride;
#pragma unroll
                for (int tok = 0; tok < TOK; ++tok)
                    if (tok < rows) {
#pragma unroll
                        for (int b = 0; b < BU; ++b) __stcg(slab + tok * (BU * 128) + b * 128 + et, acc[b][tok]);
                        if (et == tok) __stcg(slab + slab_floats + tok, sxp[tok]);
                    }
                const long long g0 = (long long) sg.bg * kblocks;
                const int first_cta = unit_owner(g0, U, G), last_cta = unit_owner(g0 + kblocks - 1, U, G);
                epi_sync();
                if (et == 0) {
                    // release: the slab stores of the 128 threads, ordered before this by the barrier; acquire: the slabs of
                    // the CTAs that arrived earlier, handed on to the other threads by the next barrier
                    unsigned old;
                    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(old) : "l"(p.counters + sg.bg) : "memory");
                    s_last = old + 1u == unsigned(last_cta - first_cta + 1);
                    if (s_last) p.counters[sg.bg] = 0u;   // ready for the next launch
                }
                epi_sync();
                if (s_last) {
                    const int first_slab = unit_begin(first_cta, U, G) >= g0 ? 2 * first_cta : 2 * first_cta + 1;
#pragma unroll
                    for (int q = 0; q < kTasksPerWarp; ++q) {
                        const int task = ew + q * kEpiWarps, row = task / BU, b = task - row * BU, band = lbg * BU + b;
                        if (row < rows && band < bands_pi) {
                            const uint2 sv = __ldg(reinterpret_cast<const uint2*>(pv.svh + band * 128 + lane * 4));
                            float v[4] = {0.f, 0.f, 0.f, 0.f}, sx = 0.f;
                            for (int c = first_cta; c <= last_cta; ++c) {
                                const float* sl = p.slabs + size_t(c == first_cta ? first_slab : 2 * c) * slab_stride;
                                const float4 t4 = __ldcg(reinterpret_cast<const float4*>(sl + row * (BU * 128) + b * 128 + lane * 4));
                                sx = __fadd_rn(sx, __ldcg(sl + slab_floats + row));
                                v[0] = __fadd_rn(v[0], t4.x); v[1] = __fadd_rn(v[1], t4.y);
                                v[2] = __fadd_rn(v[2], t4.z); v[3] = __fadd_rn(v[3], t4.w);
                            }
                            finish_band<2>(v, sx, lane, sv, band, pv.c, size_t(row0 + row), pv.ldc, p.out_fp32, p.argmax, p.residual, p.sample);
                        }
                    }
                }
            }
            u += sg.units;
        }
    }

    // ---------------------------------------------------------------- release tensor memory
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(512u) : "memory");
    }
}

// ---------------------------------------------------------------- rotation + quantisation of the activations
// One warp per (row, 128-block): a_had = fp16(H128(a * suh) / sqrt(128)) into the caller's buffer (bit-exact
// with the other paths); then the block's fixed-point form: scale = max|a_had| / 32512, v = rint(a_had / scale),
// v = 256 hi + lo with hi in [-127, 127], lo in [-128, 127].  Each limb is written replicated over the four
// bytes of a 32-bit word (the four u8 k-slots of a weight's product) at its place in the limb tile of the
// block: [MMA k-step 16][row group nb][core matrix 2][limb row 8][16 bytes], limb row = 2 * (row % 4) + (0 high,
// 1 low); k-step c of a k-tile row holds, in this order, the inputs 2c (c < 4) and 2(c-4)+1 of its eight.
// The block's scales (one fp32 per row, 16 slots) and block sums (scale * sum v, 16 slots) follow its limbs; the block
// sums also go to blocksum[row][block].  Rows of a group that do not exist are
// not written: their accumulator columns are never read.
__global__ void __launch_bounds__(128) k_rotate_in_i8(const __half* __restrict__ a, const __half* __restrict__ suh,
                                                      __half* __restrict__ a_had, unsigned char* __restrict__ limbs,
                                                      float* __restrict__ blocksum, int rows, int k, int nb,
                                                      const __half* __restrict__ a_up, float act_limit)
{
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31, kblocks = k >> 7;
    const int total = rows * kblocks;
    for (int idx = blockIdx.x * 4 + (threadIdx.x >> 5); idx < total; idx += gridDim.x * 4) {
        const int row = idx / kblocks, b = idx - row * kblocks;
        float sx;
        const uint2 o = rotate_block<false>(a + size_t(row) * k, suh, b, lane, sx, a_up ? a_up + size_t(row) * k : nullptr, act_limit);
        *reinterpret_cast<uint2*>(a_had + size_t(row) * k + b * 128 + lane * 4) = o;
        const size_t record = size_t(16) * nb * 256 + 128;          // limbs, then the block's scales (one per row)
        int isum;
        const float scale = quantise_block(o, lane, limbs + size_t(b) * record + size_t(row >> 2) * 256 + (2 * (row & 3)) * 16, nb * 256, 128, isum);
        if (lane == 0) {
            float* tail = reinterpret_cast<float*>(limbs + size_t(b) * record + size_t(16) * nb * 256);   // 16 scales, then 16 block sums
            const float bsum = __fmul_rn(scale, __int2float_rn(isum));
            tail[row] = scale;
            tail[16 + row] = bsum;
            blocksum[size_t(row) * kblocks + b] = bsum;
        }
    }
}

// Most units per CTA whose limb tiles fit the limb area of the in-kernel rotation.
int fused_max_units(int k_bits, int rows)
{
    switch (k_bits) {
        case 1: return GeoI8<1, 1, true>::fused_max_units(rows);
        case 2: return GeoI8<2, 1, true>::fused_max_units(rows);
        case 3: return GeoI8<3, 1, true>::fused_max_units(rows);
        case 4: return GeoI8<4, 1, true>::fused_max_units(rows);
        case 5: return GeoI8<5, 1, true>::fused_max_units(rows);
        case 6: return GeoI8<6, 1, true>::fused_max_units(rows);
        case 7: return GeoI8<7, 1, true>::fused_max_units(rows);
        default: return GeoI8<8, 1, true>::fused_max_units(rows);
    }
}

template <int BITS, int NB, bool FUSED, bool ONE = false>
size_t launch_one(const void* const* trellis, int n_matrices, const GemvArgs& args, int grid, cudaStream_t stream)
{
    using G_ = GeoI8<BITS, NB, FUSED>;
    auto kern = k_exl3_gemv_i8<BITS, NB, FUSED, ONE>;
    static bool attr_set[kMaxDevices] = {};
    const int dev = current_device();
    if (!attr_set[dev]) {
        cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(G_::SMEM)), "gemv i8 smem attribute");
        attr_set[dev] = true;
    }
    I8Maps maps;
    if (args.het) {
        for (int i = 0; i < kMaxHetMatrices; ++i) {
            const int j = i < n_matrices ? i : 0;
            maps.m[i] = trellis_map(trellis[j], 1, args.k, args.het_n[j], BITS, G_::ROW_BYTES);
        }
    } else {
        maps.m[0] = trellis_map(trellis[0], n_matrices, args.k, args.n, BITS, G_::ROW_BYTES);
        for (int i = 1; i < kMaxHetMatrices; ++i) maps.m[i] = maps.m[0];
    }
    launch_pdl(kern, dim3(grid), dim3(kThreads), G_::SMEM, stream, "k_exl3_gemv_i8 launch", maps, args);
    return G_::SMEM;
}

template <int BITS>
size_t launch_nb(int nb, bool fused, const void* const* t, int nm, const GemvArgs& a, int grid, cudaStream_t st)
{
    switch (nb) {
        case 1:
            if (fused) return a.m == 1 ? launch_one<BITS, 1, true, true>(t, nm, a, grid, st) : launch_one<BITS, 1, true>(t, nm, a, grid, st);
            return launch_one<BITS, 1, false>(t, nm, a, grid, st);
        default: return launch_one<BITS, 2, false>(t, nm, a, grid, st);
    }
}

size_t launch_bits(int k_bits, int nb, bool fused, const void* const* t, int nm, const GemvArgs& a, int grid, cudaStream_t st)
{
    switch (k_bits) {
        case 1: return launch_nb<1>(nb, fused, t, nm, a, grid, st);
        case 2: return launch_nb<2>(nb, fused, t, nm, a, grid, st);
        case 3: return launch_nb<3>(nb, fused, t, nm, a, grid, st);
        case 4: return launch_nb<4>(nb, fused, t, nm, a, grid, st);
        case 5: return launch_nb<5>(nb, fused, t, nm, a, grid, st);
        case 6: return launch_nb<6>(nb, fused, t, nm, a, grid, st);
        case 7: return launch_nb<7>(nb, fused, t, nm, a, grid, st);
        case 8: return launch_nb<8>(nb, fused, t, nm, a, grid, st);
        default: throw std::runtime_error("exl3 linear: K must be in 1..=8");
    }
}

}  // namespace

bool gemv_i8_rotates_in_kernel(int size_m, int size_k, int size_n, int k_bits, int sms)
{
    if (size_m < 1 || size_m > 4 || size_k % 128 != 0 || k_bits < 1 || k_bits > 8) return false;
    const int bu = k_bits <= 4 ? 2 : 1;
    const int bands = size_n / 128, kblocks = size_k / 128, bgroups = (bands + bu - 1) / bu;
    const long long units = (long long) bgroups * kblocks;
    const int grid = int(std::min<long long>(std::min<long long>(sms, units), (long long) bgroups * 16));
    if (grid < 1) return false;
    const long long units_per_cta = (units + grid - 1) / grid;
    return units_per_cta < kblocks && units_per_cta <= fused_max_units(k_bits, size_m <= 1 ? 1 : (size_m == 2 ? 2 : 4));
}

// Rotation + decode linear for up to kI8MaxRows rows of a MUL1 matrix (or of a stack of n_stack equally shaped ones);
// same contract as launch_gemv.
std::string launch_gemv_i8(const void* a, const void* trellis, void* c, const void* suh, void* a_had, const void* svh,
                           int size_m, int size_k, int size_n, int k_bits, int out_fp32, const GemvScratch& sc, int sms,
                           cudaStream_t stream, unsigned long long* argmax, int n_stack, const float* residual, const SampleArgs& sample,
                           const ActInput& act)
{
    if (n_stack < 1) n_stack = 1;
    if (size_m > kI8MaxRows) throw std::runtime_error("exl3 gemv (integer tensor path): size_m must be <= 8");
    if (size_k % 128 != 0)
        throw std::runtime_error("exl3 linear: no linked kernel for size_k that is not a multiple of 128 (128-wide Hadamard)");
    if (k_bits < 1 || k_bits > 8) throw std::runtime_error("exl3 linear: K must be in 1..=8");
    const int nb = size_m <= 4 ? 1 : 2;
    const int bu = k_bits <= 4 ? 2 : 1;
    const int bands = size_n / 128, kblocks = size_k / 128, bgroups = (bands + bu - 1) / bu;
    if (size_t(n_stack) * size_m * kblocks > sc.blocksum_floats)
        throw std::runtime_error("exl3 gemv: matrices x size_m x size_k / 128 exceed the block-sum table of the scratch");
    const size_t limb_bytes = size_t(kblocks) * (size_t(16) * nb * 256 + 128);
    if (limb_bytes * n_stack > sc.afrag_bytes)
        throw std::runtime_error("exl3 gemv: matrices x size_k x ceil(size_m / 4) exceed the activation area of the scratch");
    const long long units = (long long) n_stack * bgroups * kblocks;
    int grid = int(std::min<long long>(std::min<long long>(sms, units), (long long) n_stack * bgroups * 16));
    const size_t per_cta = size_t(2) * (size_t(size_m) * bu * 128 + 32) * sizeof(float);
    if (size_t(grid) * per_cta > sc.slab_bytes) grid = int(sc.slab_bytes / per_cta);
    if (grid < 1) throw std::runtime_error("exl3 gemv: split-K scratch is too small for this shape");
    if (size_t(n_stack) * bgroups > sc.counter_words)
        throw std::runtime_error("exl3 gemv: matrices x size_n / 128 exceed the band-group counters of the scratch");

    // In-kernel rotation for up to four rows when no CTA holds a whole band group (such a CTA finishes its bands
    // itself and needs every block sum of the row, which other CTAs would still be writing).
    const long long units_per_cta = (units + grid - 1) / grid;
    const int frows = size_m <= 1 ? 1 : (size_m == 2 ? 2 : 4);
    const bool fused = nb == 1 && units_per_cta < kblocks && units_per_cta <= fused_max_units(k_bits, frows);
    const int rot_total = size_m * kblocks;
    if (!fused)
        for (int i = 0; i < n_stack; ++i)
            launch_pdl(k_rotate_in_i8, dim3(std::min((rot_total + 3) / 4, 4 * sms)), dim3(128), 0, stream, "k_rotate_in_i8 launch",
                       static_cast<const __half*>(a), static_cast<const __half*>(suh) + size_t(i) * size_k,
                       static_cast<__half*>(a_had) + size_t(i) * size_m * size_k,
                       reinterpret_cast<unsigned char*>(sc.afrag) + size_t(i) * limb_bytes, sc.blocksum + size_t(i) * size_m * kblocks,
                       size_m, size_k, nb, static_cast<const __half*>(act.up), act.limit);

    GemvArgs args{};
    args.defer_weights = weights_streamed() ? 1 : 0;
    args.afrag = sc.afrag;
    args.blocksum = sc.blocksum;
    args.a = static_cast<const __half*>(a);
    args.a_up = static_cast<const __half*>(act.up);
    args.act_limit = act.limit;
    args.suh = static_cast<const __half*>(suh);
    args.a_had = static_cast<__half*>(a_had);
    args.c = c;
    args.argmax = argmax;
    args.sample = sample;
    args.residual = residual;
    args.svh = static_cast<const __half*>(svh);
    args.slabs = sc.slabs;
    args.counters = sc.counters;
    args.status = sc.status;
    args.m = size_m; args.k = size_k; args.n = size_n;
    args.out_fp32 = out_fp32;
    args.max_problems = 1; args.n_matrices = n_stack; args.max_rows = size_m;
    args.n_stack = n_stack;
    const size_t smem = launch_bits(k_bits, nb, fused, &trellis, n_stack, args, grid, stream);
    return std::string(fused ? "" : "k_rotate_in_i8 + ") + "k_exl3_gemv_i8<" + std::to_string(k_bits) + "," + std::to_string(nb) + (fused ? ",fused" : "") + (n_stack > 1 ? ",stack of " + std::to_string(n_stack) : "") + "> grid=" + std::to_string(grid) +
           " block=" + std::to_string(kThreads) + " smem=" + std::to_string(smem);
}

// The same kernel over up to four MUL1 matrices of different widths applied to the same rows (q, k and v of an attention
// block), each with its own tensors: the band groups of all matrices form one unit list, so launch latency, pipeline ramp
// and the in-kernel rotation are paid once.  The pointer arrays are host arrays.
std::string launch_gemv_i8_multi(const void* a, const void* const* trellis, void* const* c, const void* const* suh,
                                 void* const* a_had, const void* const* svh, const int* size_n, int n_matrices, int size_m,
                                 int size_k, int k_bits, int out_fp32, const GemvScratch& sc, int sms, cudaStream_t stream)
{
    if (n_matrices < 1 || n_matrices > kMaxHetMatrices) throw std::runtime_error("exl3 linear multi: 1 to 4 matrices");
    if (size_m < 1 || size_m > kI8MaxRows) throw std::runtime_error("exl3 linear multi: size_m must be in 1..=8");
    if (size_k % 128 != 0)
        throw std::runtime_error("exl3 linear: no linked kernel for size_k that is not a multiple of 128 (128-wide Hadamard)");
    if (k_bits < 1 || k_bits > 8) throw std::runtime_error("exl3 linear: K must be in 1..=8");
    const int nb = size_m <= 4 ? 1 : 2;
    const int bu = k_bits <= 4 ? 2 : 1;
    const int kblocks = size_k / 128;
    GemvArgs args{};
    args.defer_weights = weights_streamed() ? 1 : 0;
    args.het = 1;
    int total_bg = 0, max_n = 0;
    for (int i = 0; i < n_matrices; ++i) {
        if (size_n[i] < 128 || size_n[i] % 128 != 0) throw std::runtime_error("exl3 linear multi: size_n must be a multiple of 128");
        args.het_bg[i] = total_bg;
        total_bg += (size_n[i] / 128 + bu - 1) / bu;
        args.het_n[i] = size_n[i];
        args.het_suh[i] = static_cast<const __half*>(suh[i]);
        args.het_svh[i] = static_cast<const __half*>(svh[i]);
        args.het_c[i] = c[i];
        args.het_a_had[i] = static_cast<__half*>(a_had[i]);
        max_n = std::max(max_n, size_n[i]);
    }
    for (int i = n_matrices; i <= kMaxHetMatrices; ++i) args.het_bg[i] = total_bg;
    if (size_t(n_matrices) * size_m * kblocks > sc.blocksum_floats)
        throw std::runtime_error("exl3 gemv: matrices x size_m x size_k / 128 exceed the block-sum table of the scratch");
    const size_t limb_bytes = size_t(kblocks) * (size_t(16) * nb * 256 + 128);
    if (limb_bytes * n_matrices > sc.afrag_bytes)
        throw std::runtime_error("exl3 gemv: matrices x size_k x ceil(size_m / 4) exceed the activation area of the scratch");
    const long long units = (long long) total_bg * kblocks;
    int grid = int(std::min<long long>(std::min<long long>(sms, units), (long long) total_bg * 16));
    const size_t per_cta = size_t(2) * (size_t(size_m) * bu * 128 + 32) * sizeof(float);
    if (size_t(grid) * per_cta > sc.slab_bytes) grid = int(sc.slab_bytes / per_cta);
    if (grid < 1) throw std::runtime_error("exl3 gemv: split-K scratch is too small for this shape");
    if (size_t(total_bg) > sc.counter_words) throw std::runtime_error("exl3 gemv: band groups exceed the counters of the scratch");
    const long long units_per_cta = (units + grid - 1) / grid;
    const int frows = size_m <= 1 ? 1 : (size_m == 2 ? 2 : 4);
    const bool fused = nb == 1 && units_per_cta < kblocks && units_per_cta <= fused_max_units(k_bits, frows);
    const int rot_total = size_m * kblocks;
    if (!fused)
        for (int i = 0; i < n_matrices; ++i)
            launch_pdl(k_rotate_in_i8, dim3(std::min((rot_total + 3) / 4, 4 * sms)), dim3(128), 0, stream, "k_rotate_in_i8 launch",
                       static_cast<const __half*>(a), args.het_suh[i], args.het_a_had[i],
                       reinterpret_cast<unsigned char*>(sc.afrag) + size_t(i) * limb_bytes, sc.blocksum + size_t(i) * size_m * kblocks,
                       size_m, size_k, nb, (const __half*) nullptr, 0.f);
    args.afrag = sc.afrag;
    args.blocksum = sc.blocksum;
    args.a = static_cast<const __half*>(a);
    args.suh = args.het_suh[0];
    args.a_had = args.het_a_had[0];
    args.c = c[0];
    args.svh = args.het_svh[0];
    args.slabs = sc.slabs;
    args.counters = sc.counters;
    args.status = sc.status;
    args.m = size_m; args.k = size_k; args.n = max_n;
    args.out_fp32 = out_fp32;
    args.max_problems = 1; args.n_matrices = n_matrices; args.max_rows = size_m;
    args.n_stack = n_matrices;
    const size_t smem = launch_bits(k_bits, nb, fused, trellis, n_matrices, args, grid, stream);
    return std::string(fused ? "" : "k_rotate_in_i8 + ") + "k_exl3_gemv_i8<" + std::to_string(k_bits) + "," + std::to_string(nb) +
           (fused ? ",fused" : "") + "," + std::to_string(n_matrices) + " matrices> grid=" + std::to_string(grid) + " block=" +
           std::to_string(kThreads) + " smem=" + std::to_string(smem);
}

}  // namespace berth
