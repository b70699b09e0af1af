// Prefill EXL3 linear on the 5th-generation tensor cores (size_m > 32):
//   C = H128( a_had . W ) * svh,  a_had = H128(A * suh) (rotated beforehand by k_had128),
// with W never materialised in HBM, nor in shared memory: trellis tiles arrive by TMA, sixteen
// decode warps expand them (bit-exact fp16 weights) and store the fragments straight into TENSOR
// MEMORY, which is where tcgen05.mma takes its A operand from.  The product is computed transposed,
//   D[n][row] = sum_k W[k][n] * a_had[row][k],
// so the weights are the 128-row A operand (tensor memory), the activations the B operand (shared
// memory, K-major, 128-byte swizzle, up to 256 rows per instruction) and the fp32 accumulator holds
// one output column per TMEM lane.  Why: with both operands in shared memory a 128x128x16 MMA reads
// 8 KiB per 64 cycles, which is all the shared-memory bandwidth of an SM, and the TMA writes and the
// decode warps' traffic come on top (measured: 1815 cycles per 64-deep stage of a 512-row tile against
// 1084 for the tensor pipe).  With the weights in tensor memory the activations are read from shared
// memory once per stage and nothing else.  The MMA fragment layout of the decoder (lane = 4*g + q holds
// (n = g, g+8; k = 2q, 2q+1, 2q+8, 2q+9)) is exactly the 16x128b store shape of tensor memory, so a tile
// costs one tcgen05.st.
//
// Tile: one CTA owns 128 output columns (one Hadamard band) for up to 384 token rows (384 fp32
// accumulator columns; the other 128 TMEM columns hold four 64-deep weight stages).
// Roofline: tensor pipe; FLOPs = 2*M*K*N.
//
// Warp roles (24 warps, one CTA per SM):
//   warp 0      TMA producer: activation stages (boxes of 128 rows x 64 k) and raw trellis stages
//               (4 k-tile rows x 8 tiles);
//   warp 1      TMEM allocation + the single MMA-issuing thread;
//   warps 8..23 decode: trellis words -> fp16 pairs -> tensor memory, two tiles per warp and stage;
//   warps 4..7 and, after their last stage, the decode warps: epilogue in five teams of four warps.  A thread
//               owns output column n = its TMEM lane; 128-point Hadamard over n by warp shuffles (strides
//               1..16) and a shared-memory exchange between the four warps of the team (32, 64), output
//               scale, coalesced stores.
// Grouped launches (the experts of an MoE layer) take blockIdx.y as an index into a device-side
// problem table {matrix of the stack, first row, rows}; the MMA then covers only the problem's rows
// (rounded up to 16), which is what makes small per-expert batches cheap.
// All waits are bounded: a wait that runs out sets a status bit and the kernel carries on and
// exits (wrong output, no hang).
#include "exl3_decode.cuh"
#include "silu.cuh"

#include <cuda.h>

#include <algorithm>

namespace berth {
namespace {

constexpr int kThreads = 768;
constexpr int kDecodeWarp0 = 8, kDecodeWarps = 16;
constexpr int kEpiWarp0 = 4;
constexpr int BN = 128, BK = 64, SUB = 128, MAX_SUB = 3;
constexpr int SA = 3;   // activation stages
constexpr int SW = 4;   // decoded-weight stages in tensor memory (32 columns each)
constexpr int kBarrierBytes = 512;
constexpr int A_SUB_BYTES = SUB * BK * 2;          // 16 KiB
constexpr int A_STAGE_BYTES = MAX_SUB * A_SUB_BYTES;
constexpr int kAccCols = MAX_SUB * SUB;            // accumulator columns; weight stages follow
constexpr long long kWaitCycles = 500000000LL;

enum : unsigned { kStGemmTimeout = 16u };

template <int BITS>
struct TGeo {
    static constexpr int NW = 8 * BITS;
    static constexpr int TROW_BYTES = 8 * NW * 4;          // one k-tile row of the band
    static constexpr int T_STAGE_BYTES = 4 * TROW_BYTES;   // 64 k rows
    // Raw trellis stages: as many as fit beside the activation ring (and the epilogue buffers of the grouped
    // kernel), 4 to 16.  Weights that are read once come from DRAM, a microsecond or two away under load; four
    // stages of 0.4 us each did not cover that.
    static constexpr int kEpilogueExtra = (32 * 129 + 2 * 128) * 4;
    static constexpr int kFree = 227 * 1024 - 1024 - SA * A_STAGE_BYTES - kEpilogueExtra - kBarrierBytes - 2048 /*static shared*/;
    static constexpr int ST = kFree / T_STAGE_BYTES < 4 ? 4 : (kFree / T_STAGE_BYTES > 16 ? 16 : kFree / T_STAGE_BYTES);
    static constexpr size_t SMEM = 1024 /*align slack*/ + size_t(SA) * A_STAGE_BYTES + size_t(ST) * T_STAGE_BYTES + kBarrierBytes;
};

struct GemmArgs {
    void* c;
    const __half* svh;       // [n], or the stack [matrices][n] of a grouped launch
    unsigned* status;
    int m, k, n, out_fp32;   // m = rows of the activation / output arrays
    int nsub_max;   // 128-row sub-tiles per CTA (1..3): the row block of a CTA is nsub_max*128 tokens
    const GemvProblem* problems;   // grouped launch: one entry per (matrix, chunk of <= nsub_max*128 rows); else null
    const int* n_problems;
    int max_problems, n_matrices;
    int epi2;   // grouped launch with 128-row problems and a short K: two epilogue teams and three decode groups (see the kernel)
};

// ---------------------------------------------------------------- PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t) __cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned* status)
{
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > kWaitCycles) {
            atomicOr(status, kStGemmTimeout);
            return false;
        }
    }
    return true;
}
// The same for warps that wait long (producer, decode, epilogue): sleep between polls, so that the one
// thread that issues the MMAs is not competing for issue slots with spinning warps.
__device__ __forceinline__ bool mbar_wait_parked(uint32_t bar, uint32_t parity, unsigned* status, unsigned ns)
{
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        __nanosleep(ns);
        if (clock64() - t0 > kWaitCycles) {
            atomicOr(status, kStGemmTimeout);
            return false;
        }
    }
    return true;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]^T: A = 128 rows x 16 k fp16 in tensor memory (lane = row, two k per
// 32-bit column), B = N rows x 16 k K-major in shared memory, D = 128 lanes x N fp32 columns.
__device__ __forceinline__ void tc_mma_ts_f16(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Instruction descriptor: D fp32, A/B fp16, both K-major, M = 128, N = n (a multiple of 16 up to 256).
__device__ __forceinline__ uint32_t idesc_n(int n) { return (1u << 4) | (uint32_t(n >> 3) << 17) | (uint32_t(128 >> 4) << 24); }
// One decoded 16x16 tile (the four fragment registers of mma.m16n8k16's A operand) into tensor memory:
// 16 lanes x 8 columns starting at taddr; thread 4*g+q supplies (lane g | g+8, columns q | q+4).
__device__ __forceinline__ void tc_st_frag(uint32_t taddr, const uint32_t (&w)[4])
{
    asm volatile("tcgen05.st.sync.aligned.16x128b.x2.b32 [%0], {%1,%2,%3,%4};" ::"r"(taddr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                 : "memory");
}
// The same without the memory clobber: tensor memory aliases no C++ object, and every hand-over of a stage goes
// through tc_wait_st and an mbarrier operation, which do clobber; the compiler may then schedule the shared-memory
// loads and the arithmetic of the next tiles across the store.
__device__ __forceinline__ void tc_st_frag_free(uint32_t taddr, const uint32_t (&w)[4])
{
    asm volatile("tcgen05.st.sync.aligned.16x128b.x2.b32 [%0], {%1,%2,%3,%4};" ::"r"(taddr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]));
}
// Two k-tile rows of one tile column at once: 16 lanes x 16 columns.
__device__ __forceinline__ void tc_st_frag2_free(uint32_t taddr, const uint32_t (&w0)[4], const uint32_t (&w1)[4])
{
    asm volatile("tcgen05.st.sync.aligned.16x128b.x4.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(w0[0]), "r"(w0[1]), "r"(w0[2]),
                 "r"(w0[3]), "r"(w1[0]), "r"(w1[1]), "r"(w1[2]), "r"(w1[3]));
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// 32 lanes x 32 consecutive fp32 columns of this warp's TMEM lane quarter.
__device__ __forceinline__ void tc_ld32(uint32_t taddr, float (&v)[32])
{
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 bytes, groups
// of 8 rows 1024 bytes apart (start address and offsets in 16-byte units; version 1 = sm_100).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr)
{
    uint64_t d = 0;
    d |= uint64_t((addr & 0x3FFFF) >> 4);        // start address
    d |= uint64_t(1) << 16;                      // leading byte offset (unused for swizzled K-major)
    d |= uint64_t(1024 >> 4) << 32;              // stride byte offset
    d |= uint64_t(1) << 46;                      // descriptor version
    d |= uint64_t(2) << 61;                      // SWIZZLE_128B
    return d;
}
constexpr int kEpiTeams = 5;
// Barrier of one epilogue team (four warps); ids 1..5.
__device__ __forceinline__ void team_sync(int team) { asm volatile("bar.sync %0, 128;" ::"r"(team + 1) : "memory"); }
// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one()
{
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}

// One epilogue pass of a team of four warps (one per TMEM lane quarter; barrier id `team` + 1): 32 token
// rows (accumulator columns tacc .. tacc+31 of the warp's lanes) of one band.  The accumulator has one
// output column n per TMEM lane, so a thread first holds 32 rows of one n; the tile is transposed through
// shared memory (xch, kXchFloats floats, rows of 129 with the 32-blocks rotated by 8 per block: no bank
// conflict on either side) so that thread t then holds the 32 consecutive n of block t%4 of row t/4.
// 128-point Hadamard over n with ascending strides: 1..16 in registers, 32 and 64 between the four
// threads of a row by shuffles (sgn * v + o is o - v or v + o, rounded once); then the output scale
// (svh_s: the band's 128 scales as fp32) and 16-byte stores of rows row0 .. row0+31 below row_end.
constexpr int kXchPitch = 129;
constexpr int kXchFloats = 32 * kXchPitch;
__device__ __forceinline__ void epilogue_rows(float (&v)[32], float* xch, const float* svh_s, int team, int quarter, int lane, void* c,
                                              int out_fp32, int ldc, int col0, int row0, int row_end)
{
    {
        float* wp = xch + 32 * quarter + ((lane - 8 * quarter) & 31);
#pragma unroll
        for (int j = 0; j < 32; ++j) wp[j * kXchPitch] = v[j];
    }
    team_sync(team);
    const int t = quarter * 32 + lane, r = t >> 2, cc = t & 3;
    {
        const float* rp = xch + r * kXchPitch + 32 * cc;
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = rp[(i - 8 * cc) & 31];
    }
    team_sync(team);   // xch may be overwritten by the next pass
#pragma unroll
    for (int s = 1; s < 32; s <<= 1)
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (!(i & s)) {
                const float a = v[i], b = v[i | s];
                v[i] = __fadd_rn(a, b);
                v[i | s] = __fsub_rn(a, b);
            }
#pragma unroll
    for (int bit = 0; bit < 2; ++bit) {
        const float sgn = (cc >> bit) & 1 ? -1.f : 1.f;   // -1 where this thread holds the upper block of the butterfly
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __fmaf_rn(sgn, v[i], __shfl_xor_sync(dq::kFull, v[i], 1 << bit));
    }
    const int row = row0 + r;
    if (row < row_end) {
        const float* sp = svh_s + 32 * cc;
        if (out_fp32) {
            float* dst = static_cast<float*>(c) + size_t(row) * ldc + col0 + 32 * cc;
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
                const float4 sc = *reinterpret_cast<const float4*>(sp + i);
                float4 o;
                o.x = __fmul_rn(__fmul_rn(v[i], kRScale), sc.x); o.y = __fmul_rn(__fmul_rn(v[i + 1], kRScale), sc.y);
                o.z = __fmul_rn(__fmul_rn(v[i + 2], kRScale), sc.z); o.w = __fmul_rn(__fmul_rn(v[i + 3], kRScale), sc.w);
                *reinterpret_cast<float4*>(dst + i) = o;
            }
        } else {
            __half* dst = static_cast<__half*>(c) + size_t(row) * ldc + col0 + 32 * cc;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
                const float4 s0 = *reinterpret_cast<const float4*>(sp + i), s1 = *reinterpret_cast<const float4*>(sp + i + 4);
                uint4 o;
                o.x = dq::pack_half2(__float2half_rn(__fmul_rn(__fmul_rn(v[i], kRScale), s0.x)), __float2half_rn(__fmul_rn(__fmul_rn(v[i + 1], kRScale), s0.y)));
                o.y = dq::pack_half2(__float2half_rn(__fmul_rn(__fmul_rn(v[i + 2], kRScale), s0.z)), __float2half_rn(__fmul_rn(__fmul_rn(v[i + 3], kRScale), s0.w)));
                o.z = dq::pack_half2(__float2half_rn(__fmul_rn(__fmul_rn(v[i + 4], kRScale), s1.x)), __float2half_rn(__fmul_rn(__fmul_rn(v[i + 5], kRScale), s1.y)));
                o.w = dq::pack_half2(__float2half_rn(__fmul_rn(__fmul_rn(v[i + 6], kRScale), s1.z)), __float2half_rn(__fmul_rn(__fmul_rn(v[i + 7], kRScale), s1.w)));
                *reinterpret_cast<uint4*>(dst + i) = o;
            }
        }
    }
}
__device__ __noinline__ void epilogue_pass(uint32_t tacc, float* xch, const float* svh_s, int team, int quarter, int lane, void* c,
                                           int out_fp32, int ldc, int col0, int row0, int row_end)
{
    float v[32];
    tc_ld32(tacc, v);
    epilogue_rows(v, xch, svh_s, team, quarter, lane, c, out_fp32, ldc, col0, row0, row_end);
}

// One 64-deep stage of one band decoded into tensor memory by one group of four decode warps (the four groups take
// the stages round robin, group g always into weight stage g of tensor memory): the warp takes all four k-tile rows
// of the stage and tile columns 2*quarter, 2*quarter+1 = output columns 32*quarter .. +31, which are the TMEM lanes
// it may access (warp index % 4 == quarter).  `wait_w` = the stage of tensor memory must first be released.
// (Sixteen warps sharing every stage, a quarter of this work per barrier round trip, spent more instructions on the
// hand-over than on the weights.)
template <int BITS, int CB, bool SPIN = false>
__device__ __forceinline__ void decode_stage(const unsigned char* tstage, uint32_t tmem_wstage, int quarter, int lane, bool wait_w,
                                             uint32_t empty_w_bar, uint32_t empty_w_parity, unsigned* status)
{
    constexpr int NW = 8 * BITS, TROW_BYTES = 8 * NW * 4;
#pragma unroll
    for (int krow = 0; krow < 4; ++krow) {
        const uint32_t* trow = reinterpret_cast<const uint32_t*>(tstage + krow * TROW_BYTES);
        uint32_t w[2][4];
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            uint32_t s[8];
            const uint32_t* tile = trow + (2 * quarter + t) * NW;
            if constexpr (BITS == 4) dq::states_4bit<(CB != 2) ? 6 : 0>(tile[lane], tile[(lane + 1) & 31], s);
            else dq::lane_states<BITS>(tile, lane, s);
            dq::decode_frag<CB>(s, w[t]);
        }
        if (krow == 0 && wait_w) {   // the MMAs that read this weight stage are done
            if constexpr (SPIN) mbar_wait(empty_w_bar, empty_w_parity, status);
            else mbar_wait_parked(empty_w_bar, empty_w_parity, status, 40);
            tc_fence_after();
        }
#pragma unroll
        for (int t = 0; t < 2; ++t) tc_st_frag(tmem_wstage + (uint32_t(32 * quarter + 16 * t) << 16) + 8 * krow, w[t]);
    }
    tc_wait_st();
    tc_fence_before();
    __syncwarp();
}

// ---------------------------------------------------------------- the kernel
template <int BITS, int CB>
__global__ void __launch_bounds__(kThreads, 1) k_exl3_gemm_tc(const __grid_constant__ CUtensorMap tmap_a,
                                                              const __grid_constant__ CUtensorMap tmap_t, const GemmArgs p)
{
    using TG_ = TGeo<BITS>;
    constexpr int NW = TG_::NW, TROW_BYTES = TG_::TROW_BYTES, T_STAGE_BYTES = TG_::T_STAGE_BYTES, ST = TG_::ST;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int band = blockIdx.x;
    int z = 0, m0 = blockIdx.y * (p.nsub_max * SUB), rows_here = min(p.m - m0, p.nsub_max * SUB);
    if (p.problems) {
        // (the table was written by kernels that completed before this launch)
        if (int(blockIdx.y) >= min(max(__ldg(p.n_problems), 0), p.max_problems)) return;
        const GemvProblem pr = load_problem(p.problems, blockIdx.y, p.n_matrices, p.nsub_max * SUB, p.m);
        z = pr.z; m0 = pr.row0; rows_here = pr.rows;
        if (rows_here < 1) return;
    }
    const int row_end = m0 + rows_here;
    const int nsub = (rows_here + SUB - 1) / SUB;
    const int rows_pad = (rows_here + 15) & ~15;          // MMA N granularity
    const int n1 = min(rows_pad, 256), n2 = rows_pad - n1;   // rows of the first / second MMA of a k step
    const int kstages = p.k / BK;

    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* a_ring = smem;
    unsigned char* t_ring = a_ring + SA * A_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(t_ring + ST * T_STAGE_BYTES);
    __shared__ uint32_t s_tmem_base;

    const uint32_t full_a = smem_u32(bars), empty_a = full_a + 8 * SA;
    const uint32_t full_w = empty_a + 8 * SA, empty_w = full_w + 8 * SW;
    const uint32_t full_t = empty_w + 8 * SW, empty_t = full_t + 8 * ST;
    const uint32_t acc_full = empty_t + 8 * ST;

    if (threadIdx.x == 0) {
        for (int s = 0; s < SA; ++s) { mbar_init(full_a + 8 * s, 1); mbar_init(empty_a + 8 * s, 1); }
        for (int s = 0; s < SW; ++s) { mbar_init(full_w + 8 * s, 4); mbar_init(empty_w + 8 * s, 1); }
        for (int s = 0; s < ST; ++s) { mbar_init(full_t + 8 * s, 1); mbar_init(empty_t + 8 * s, 4); }
        mbar_init(acc_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem_base;
    const uint32_t tmem_w = tmem + kAccCols;   // weight stages: 32 columns (64 k) each

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_t) : "memory");
            int sa = 0, pa = 0, st = 0, pt = 0;
            for (int ks = 0; ks < kstages; ++ks) {
                // raw trellis: 4 k-tile rows of this band
                if (ks >= ST) mbar_wait_parked(empty_t + 8 * st, pt ^ 1, p.status, 100);
                mbar_arrive_expect_tx(full_t + 8 * st, T_STAGE_BYTES);
                tma_load_3d(smem_u32(t_ring + st * T_STAGE_BYTES), &tmap_t, band * (TROW_BYTES / 8), ks * 4, z, full_t + 8 * st);
                if (++st == ST) { st = 0; pt ^= 1; }
                // activations: nsub boxes of 128 rows x 64 k (rows past the array read as zero)
                if (ks >= SA) mbar_wait_parked(empty_a + 8 * sa, pa ^ 1, p.status, 100);
                mbar_arrive_expect_tx(full_a + 8 * sa, nsub * A_SUB_BYTES);
                for (int sub = 0; sub < nsub; ++sub)
                    tma_load_2d(smem_u32(a_ring + sa * A_STAGE_BYTES + sub * A_SUB_BYTES), &tmap_a, ks * BK, m0 + sub * SUB,
                                full_a + 8 * sa);
                if (++sa == SA) { sa = 0; pa ^= 1; }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        // The whole warp runs the loop and one elected lane issues: addresses and descriptors then live in
        // uniform registers.  (Issued from a single-lane branch every operand was moved from the vector to
        // the uniform register file first, about 160 cycles per 16-deep step, more than the MMA itself.)
        const uint32_t id1 = idesc_n(n1), id2 = idesc_n(n2 > 0 ? n2 : 16);
        int sa = 0, pa = 0, sw = 0, pw = 0;
        for (int ks = 0; ks < kstages; ++ks) {
            mbar_wait(full_a + 8 * sa, pa, p.status);
            mbar_wait(full_w + 8 * sw, pw, p.status);
            tc_fence_after();
            const uint32_t x_base = smem_u32(a_ring + sa * A_STAGE_BYTES);
            const uint64_t x_desc1 = smem_desc_sw128(x_base), x_desc2 = smem_desc_sw128(x_base + 2 * A_SUB_BYTES);
            const uint32_t w_t = tmem_w + sw * 32;
            const uint32_t bar_a = empty_a + 8 * sa, bar_w = empty_w + 8 * sw;
            if (elect_one()) {
#pragma unroll
                for (int k16 = 0; k16 < BK / 16; ++k16) {   // +32 bytes (2 x 16-byte units) per 16 k inside the swizzle atom
                    tc_mma_ts_f16(tmem, w_t + 8 * k16, x_desc1 + 2 * k16, id1, (ks | k16) ? 1u : 0u);
                    if (n2 > 0) tc_mma_ts_f16(tmem + 256, w_t + 8 * k16, x_desc2 + 2 * k16, id2, (ks | k16) ? 1u : 0u);
                }
                tc_commit(bar_a);   // both arrive when the MMAs above have read their operands
                tc_commit(bar_w);
            }
            __syncwarp();
            if (++sa == SA) { sa = 0; pa ^= 1; }
            if (++sw == SW) { sw = 0; pw ^= 1; }
        }
        if (elect_one()) tc_commit(acc_full);
        __syncwarp();
    } else if (warp >= kDecodeWarp0) {
        // ------------------------------------------------------------ decode warps
        const int g = (warp - kDecodeWarp0) >> 2, quarter = warp & 3;   // group g: stages g, g+4, ... into weight stage g
        static_assert(SW == 4 && ST >= 4, "one weight stage per decode group");
        int st = g, pt = 0, pw = 0;
        for (int ks = g; ks < kstages; ks += 4) {
            mbar_wait_parked(full_t + 8 * st, pt, p.status, 40);
            decode_stage<BITS, CB>(t_ring + st * T_STAGE_BYTES, tmem_w + g * 32, quarter, lane, ks >= SW, empty_w + 8 * g, pw ^ 1, p.status);
            if (lane == 0) {
                mbar_arrive(full_w + 8 * g);
                mbar_arrive(empty_t + 8 * st);
            }
            st += 4;
            if (st >= ST) { st -= ST; pt ^= 1; }
            pw ^= 1;
        }
    }

    // ---------------------------------------------------------------- epilogue
    // Five teams of four warps (one warp per TMEM lane quarter): the epilogue warps and, once their
    // last stage is stored, the four decode groups.  Team i takes the 32-row passes i, i+5, ...
    // Thread = output column n = 32*quarter + lane (its TMEM lane).
    int team = -1;
    if (warp >= kEpiWarp0 && warp < kEpiWarp0 + 4) team = 0;
    else if (warp >= kDecodeWarp0) team = 1 + ((warp - kDecodeWarp0) >> 2);
    if (team >= 0) {
        const int quarter = warp & 3;
        const int n = quarter * 32 + lane;
        const float scale = __half2float(p.svh[size_t(z) * p.n + band * BN + n]);
        mbar_wait_parked(acc_full, 0, p.status, team == 0 ? 1000 : 100);
        tc_fence_after();
        // per team: transposition buffer and the band's scales, in the activation ring, which is idle by now
        float* xch = reinterpret_cast<float*>(a_ring) + team * (kXchFloats + 128);
        float* svh_s = xch + kXchFloats;
        svh_s[n] = scale;
        team_sync(team);
        for (int c0 = 32 * team; c0 < rows_pad; c0 += 32 * kEpiTeams)
            epilogue_pass(tmem + (uint32_t(quarter * 32) << 16) + c0, xch, svh_s, team, quarter, lane, p.c, p.out_fp32, p.n, band * BN,
                          m0 + c0, row_end);
        tc_fence_before();
    }

    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// ---------------------------------------------------------------- the grouped kernel
// Persistent variant for the expert stacks of an MoE layer: work items are (problem, band) pairs, band
// fastest; CTA c takes items c, c + gridDim.x, ...  The rings and the decode / MMA pipeline run on across
// item boundaries, and with one 128-row sub-tile per problem the accumulator is double buffered, so the
// epilogue of an item (four dedicated warps) overlaps the main loop of the next.  Per item the MMA covers
// only the problem's rows (rounded up to 16).
template <int BITS>
struct GGeo {
    static constexpr int T_STAGE_BYTES = TGeo<BITS>::T_STAGE_BYTES;
    static constexpr size_t SMEM = TGeo<BITS>::SMEM + (kXchFloats + 2 * 128) * 4 /*transposition buffer and scales of the epilogue*/;
};

// Three views of the activations (boxes of 32, 64 and 128 rows x 64 k): an item loads only as many rows as
// its problem has, rounded up to a box; with 128-row boxes for 32-row problems the activation traffic of an
// MoE layer at 1024 tokens was four times its weight traffic.
template <int BITS, int CB>
__global__ void __launch_bounds__(kThreads, 1) k_exl3_gemm_tc_grouped(const __grid_constant__ CUtensorMap tmap_a,
                                                                      const __grid_constant__ CUtensorMap tmap_a64,
                                                                      const __grid_constant__ CUtensorMap tmap_a32,
                                                                      const __grid_constant__ CUtensorMap tmap_t, const GemmArgs p)
{
    using TG_ = TGeo<BITS>;
    constexpr int TROW_BYTES = TG_::TROW_BYTES, T_STAGE_BYTES = TG_::T_STAGE_BYTES, ST = TG_::ST;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bands = p.n / BN;
    const int chunk = p.nsub_max * SUB;
    // (the table was written by kernels that completed before this launch)
    const int nprob = min(max(__ldg(p.n_problems), 0), p.max_problems);
    const int n_items = nprob * bands;
    if (int(blockIdx.x) >= n_items) return;
    const int my_items = (n_items - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x);
    const int nbuf = p.nsub_max == 1 ? 2 : 1;           // accumulator buffers of `chunk` columns each
    const int kstages = p.k / BK;

    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* a_ring = smem;
    unsigned char* t_ring = a_ring + SA * A_STAGE_BYTES;
    float* xch = reinterpret_cast<float*>(t_ring + ST * T_STAGE_BYTES);
    float* svh_s = xch + kXchFloats;                   // two buffers of 128 scales, alternating between items
    uint64_t* bars = reinterpret_cast<uint64_t*>(svh_s + 2 * 128);
    __shared__ uint32_t s_tmem_base;

    // The activation ring holds as many stages as fit its 144 KiB: 9 of one 128-row sub-tile, 4 of two, 3 of three.
    // With short stages (a 32-row problem's stage is 0.4 us of decode) three stages in flight did not cover an L2 miss.
    constexpr int kMaxSA = 9;
    const int a_stage = p.nsub_max * A_SUB_BYTES;
    // With a short K a 128-row item's main loop (K / 64 stages of decode) is shorter than its epilogue (four passes of
    // transposition, Hadamard and stores by one team of four warps), and the decode warps wait for accumulators.  Then the
    // fourth decode group works as a second epilogue team instead: team e drains accumulator buffer e (items e, e+2, ...),
    // three groups decode into three weight stages.  Its transposition buffer lies behind seven activation stages.
    const bool epi2 = p.epi2 != 0 && p.nsub_max == 1;
    const int G = epi2 ? 3 : 4;                        // decode groups = weight stages in use
    const int SAg = epi2 ? 7 : (SA * A_STAGE_BYTES) / a_stage;
    float* xch1 = reinterpret_cast<float*>(a_ring + 7 * A_SUB_BYTES);
    const uint32_t full_a = smem_u32(bars), empty_a = full_a + 8 * kMaxSA;
    const uint32_t full_w = empty_a + 8 * kMaxSA, empty_w = full_w + 8 * SW;
    const uint32_t full_t = empty_w + 8 * SW, empty_t = full_t + 8 * ST;
    const uint32_t acc_full = empty_t + 8 * ST, acc_empty = acc_full + 16;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMaxSA; ++s) { mbar_init(full_a + 8 * s, 1); mbar_init(empty_a + 8 * s, 1); }
        for (int s = 0; s < SW; ++s) { mbar_init(full_w + 8 * s, 4); mbar_init(empty_w + 8 * s, 1); }
        for (int s = 0; s < ST; ++s) { mbar_init(full_t + 8 * s, 1); mbar_init(empty_t + 8 * s, 4); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full + 8 * b, 1); mbar_init(acc_empty + 8 * b, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // the problems of this CTA's first items, so that no role waits for the table at an item boundary
    constexpr int kCachedItems = 64;
    __shared__ GemvProblem s_prob[kCachedItems];
    if (int(threadIdx.x) >= 64 && int(threadIdx.x) < 64 + min(my_items, kCachedItems)) {
        const int item = int(blockIdx.x) + (int(threadIdx.x) - 64) * int(gridDim.x);
        s_prob[threadIdx.x - 64] = load_problem(p.problems, item / bands, p.n_matrices, chunk, p.m);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem_base;
    const uint32_t tmem_w = tmem + kAccCols;   // weight stages: 32 columns (64 k) each

    // item `it` of this CTA -> its problem and band
    auto item_at = [&](int it, int& band, GemvProblem& pr) {
        const int item = int(blockIdx.x) + it * int(gridDim.x);
        const int pi = item / bands;
        band = item - pi * bands;
        pr = it < kCachedItems ? s_prob[it] : load_problem(p.problems, pi, p.n_matrices, chunk, p.m);
    };

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer of the trellis stages
        // (its own thread: the weight stream then runs as far ahead as its ring allows and never waits for a slot
        // of the activation ring, which is shorter and is released later, by the MMAs)
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_t) : "memory");
            int st = 0, pt = 0, cnt = 0;
            for (int it = 0; it < my_items; ++it) {
                int band; GemvProblem pr;
                item_at(it, band, pr);
                for (int ks = 0; ks < kstages; ++ks, ++cnt) {
                    if (cnt >= ST) mbar_wait_parked(empty_t + 8 * st, pt ^ 1, p.status, 100);
                    mbar_arrive_expect_tx(full_t + 8 * st, T_STAGE_BYTES);
                    tma_load_3d(smem_u32(t_ring + st * T_STAGE_BYTES), &tmap_t, band * (TROW_BYTES / 8), ks * 4, pr.z, full_t + 8 * st);
                    if (++st == ST) { st = 0; pt ^= 1; }
                }
            }
        }
    } else if (warp == 2) {
        // ------------------------------------------------------------ TMA producer of the activation stages
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a64) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a32) : "memory");
            int sa = 0, pa = 0, cnt = 0;
            for (int it = 0; it < my_items; ++it) {
                int band; GemvProblem pr;
                item_at(it, band, pr);
                const int nsub = (pr.rows + SUB - 1) / SUB;
                // one box of 32 or 64 rows for a small problem, else 128-row boxes
                const CUtensorMap* amap = pr.rows <= 32 ? &tmap_a32 : (pr.rows <= 64 ? &tmap_a64 : &tmap_a);
                const int box_bytes = pr.rows <= 32 ? 32 * BK * 2 : (pr.rows <= 64 ? 64 * BK * 2 : A_SUB_BYTES);
                for (int ks = 0; ks < kstages; ++ks, ++cnt) {
                    if (cnt >= SAg) mbar_wait_parked(empty_a + 8 * sa, pa ^ 1, p.status, 100);
                    mbar_arrive_expect_tx(full_a + 8 * sa, max(nsub, 1) * box_bytes);
                    for (int sub = 0; sub < max(nsub, 1); ++sub)
                        tma_load_2d(smem_u32(a_ring + sa * a_stage + sub * A_SUB_BYTES), amap, ks * BK, pr.row0 + sub * SUB,
                                    full_a + 8 * sa);
                    if (++sa == SAg) { sa = 0; pa ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (whole warp, one elected lane issues)
        int sa = 0, pa = 0, sw = 0, pw = 0;
        for (int it = 0; it < my_items; ++it) {
            int band; GemvProblem pr;
            item_at(it, band, pr);
            const int rows_pad = max((pr.rows + 15) & ~15, 16);
            const int n1 = min(rows_pad, 256), n2 = rows_pad - n1;
            const uint32_t id1 = idesc_n(n1), id2 = idesc_n(n2 > 0 ? n2 : 16);
            const int buf = it % nbuf;
            const uint32_t tacc = tmem + buf * chunk;
            if (it >= nbuf) {   // the epilogue has drained this accumulator
                mbar_wait(acc_empty + 8 * buf, ((it / nbuf) - 1) & 1, p.status);
                tc_fence_after();
            }
            for (int ks = 0; ks < kstages; ++ks) {
                mbar_wait(full_a + 8 * sa, pa, p.status);
                mbar_wait(full_w + 8 * sw, pw, p.status);
                tc_fence_after();
                const uint32_t x_base = smem_u32(a_ring + sa * a_stage);
                const uint64_t x_desc1 = smem_desc_sw128(x_base), x_desc2 = smem_desc_sw128(x_base + 2 * A_SUB_BYTES);
                const uint32_t w_t = tmem_w + sw * 32;
                const uint32_t bar_a = empty_a + 8 * sa, bar_w = empty_w + 8 * sw;
                if (elect_one()) {
#pragma unroll
                    for (int k16 = 0; k16 < BK / 16; ++k16) {
                        tc_mma_ts_f16(tacc, w_t + 8 * k16, x_desc1 + 2 * k16, id1, (ks | k16) ? 1u : 0u);
                        if (n2 > 0) tc_mma_ts_f16(tacc + 256, w_t + 8 * k16, x_desc2 + 2 * k16, id2, (ks | k16) ? 1u : 0u);
                    }
                    tc_commit(bar_a);
                    tc_commit(bar_w);
                }
                __syncwarp();
                if (++sa == SAg) { sa = 0; pa ^= 1; }
                if (++sw == G) { sw = 0; pw ^= 1; }
            }
            if (elect_one()) tc_commit(acc_full + 8 * buf);
            __syncwarp();
        }
    } else if (warp >= kDecodeWarp0 && !(epi2 && warp >= kDecodeWarp0 + 12)) {
        // ------------------------------------------------------------ decode warps
        const int g = (warp - kDecodeWarp0) >> 2, quarter = warp & 3;   // group g: stages g, g+G, ... into weight stage g
        static_assert(SW == 4 && ST >= 4, "one weight stage per decode group");
        int st = g, pt = 0, pw = 0;
        const int total = my_items * kstages;
        for (int cnt = g; cnt < total; cnt += G) {
            mbar_wait_parked(full_t + 8 * st, pt, p.status, 40);
            decode_stage<BITS, CB>(t_ring + st * T_STAGE_BYTES, tmem_w + g * 32, quarter, lane, cnt >= G, empty_w + 8 * g, pw ^ 1, p.status);
            if (lane == 0) {
                mbar_arrive(full_w + 8 * g);
                mbar_arrive(empty_t + 8 * st);
            }
            st += G;
            if (st >= ST) { st -= ST; pt ^= 1; }
            pw ^= 1;
        }
    } else if (warp >= kEpiWarp0) {
        // ------------------------------------------------------------ epilogue warps: team 0 (warps 4..7), and with two
        // teams the last four warps as team 1
        const int team = warp >= kDecodeWarp0 ? 1 : 0;
        const int step = epi2 ? 2 : 1;
        float* xc = team ? xch1 : xch;
        float* svs = team ? xch1 + kXchFloats : svh_s;
        const int quarter = warp & 3;
        const int n = quarter * 32 + lane;
        int turn = 0;
        for (int it = team; it < my_items; it += step, turn ^= 1) {
            int band; GemvProblem pr;
            item_at(it, band, pr);
            float* sv = svs + turn * 128;   // (the other buffer may still be read by a slower warp of the team's previous item)
            sv[n] = __half2float(p.svh[size_t(pr.z) * p.n + band * BN + n]);
            const int buf = it % nbuf;
            mbar_wait_parked(acc_full + 8 * buf, (it / nbuf) & 1, p.status, 200);
            tc_fence_after();
            team_sync(team);   // the scales are in place
            const int rows_pad = (pr.rows + 15) & ~15;
            for (int c0 = 0; c0 < rows_pad; c0 += 32)
                epilogue_pass(tmem + buf * chunk + (uint32_t(quarter * 32) << 16) + c0, xc, sv, team, quarter, lane, p.c, p.out_fp32, p.n,
                              band * BN, pr.row0 + c0, pr.row0 + pr.rows);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty + 8 * buf);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// decode_stage for the small-batch kernel, where the decode warps are the bottleneck: tight polling, and the hand-over
// of a stage to the MMA warp (wait for the tensor-memory stores, fence, arrive on `pend_w`) is deferred until the
// first k-tile row of the NEXT stage sits decoded in registers, so the stores' latency is covered by decode work.
// The caller hands over the last stage itself.
template <int BITS, int CB>
__device__ __forceinline__ void sk_decode_stage(const unsigned char* tstage, uint32_t tmem_wstage, int quarter, int lane, bool wait_w,
                                                uint32_t empty_w_bar, uint32_t empty_w_parity, unsigned* status, uint32_t pend_w)
{
    constexpr int NW = 8 * BITS, TROW_BYTES = 8 * NW * 4;
    // All eight tiles of the warp are decoded into registers before the first store: a tensor-memory store holds
    // its source registers until it has read them, so decoding the next tile into the registers of a store in
    // flight stalls the warp for the store's latency.
    uint32_t w[4][2][4];
    if constexpr (BITS == 4) {
        uint32_t r0[4][2], r1[4][2];
#pragma unroll
        for (int krow = 0; krow < 4; ++krow)
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                const uint32_t* tile = reinterpret_cast<const uint32_t*>(tstage + krow * TROW_BYTES) + (2 * quarter + t) * NW;
                r0[krow][t] = tile[lane];
                r1[krow][t] = tile[(lane + 1) & 31];
            }
#pragma unroll
        for (int krow = 0; krow < 4; ++krow)
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                uint32_t s[8];
                dq::states_4bit<(CB != 2) ? 6 : 0>(r0[krow][t], r1[krow][t], s);
                dq::decode_frag<CB>(s, w[krow][t]);
            }
    } else {
#pragma unroll
        for (int krow = 0; krow < 4; ++krow)
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                uint32_t s[8];
                dq::lane_states<BITS>(reinterpret_cast<const uint32_t*>(tstage + krow * TROW_BYTES) + (2 * quarter + t) * NW, lane, s);
                dq::decode_frag<CB>(s, w[krow][t]);
            }
    }
    if (pend_w) {
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(pend_w);
    }
    if (wait_w) {   // the MMAs that read this weight stage are done
        mbar_wait(empty_w_bar, empty_w_parity, status);
        tc_fence_after();
    }
#pragma unroll
    for (int kp = 0; kp < 2; ++kp)
#pragma unroll
        for (int t = 0; t < 2; ++t)
            tc_st_frag2_free(tmem_wstage + (uint32_t(32 * quarter + 16 * t) << 16) + 16 * kp, w[2 * kp][t], w[2 * kp + 1][t]);
}

// ---------------------------------------------------------------- the small-batch kernel (9..32 rows)
// Decode batches too large for the mma.sync decode kernel's row groups and far too small to fill the prefill
// tiles: one persistent CTA per SM, and the matrix's work -- `bands * (K / 64)` stages of 64 x 128 weights, band
// major -- is cut into gridDim.x equal contiguous ranges, so every SM decodes the same number of weights whatever
// the matrix's shape (a 1024-wide k/v projection has 8 bands; by bands alone it would use 8 SMs).  A range that
// crosses a band boundary closes one accumulator and opens the other (two buffers of 32 TMEM columns), and the
// epilogue warps drain the closed one while the pipeline runs on.  A band that one CTA holds whole is finished
// from tensor memory as in the prefill kernel.  A band shared by several CTAs goes through fp32 slabs (two per
// CTA: its first segment, and any later one), which k_sk_finish, chained behind, sums in CTA order -- a fixed
// order -- and finishes (Hadamard, output scale, store) with one warp per band and row.  (A last-arriver tail in
// this kernel was measured first: one CTA summing up to nineteen slabs of 32 rows took 20 us on the k/v shape.)
// Nobody waits for another CTA.  Rows: the MMA's N is the row count rounded to 16; the activation box is 32
// rows (rows past the array read as zero).
struct SplitKArgs {
    void* c;
    const __half* svh;
    unsigned* status;
    float* slabs;          // [grid][2][32][128] fp32
    int m, k, n, out_fp32, grid;
    int defer_weights;     // no weight fetch before griddepcontrol.wait (berth_exl3_weights_streamed)
};
constexpr int kSkRows = 32;                       // rows of the activation box and of a slab
constexpr int kSkAStageBytes = kSkRows * BK * 2;  // 4 KiB
constexpr int kSkSA = 8;                          // activation stages
constexpr int kSkSW = 8;                          // decoded-weight stages in tensor memory: two per decode group, so that a
                                                  // group stores its next stage while the MMAs still read the previous one
constexpr int kSkWCol0 = 2 * kSkRows;             // TMEM: two accumulators of 32 columns, then the weight stages
template <int BITS>
struct SGeo {
    static constexpr int T_STAGE_BYTES = TGeo<BITS>::T_STAGE_BYTES;
    static constexpr int ST = (160 * 1024) / T_STAGE_BYTES > 24 ? 24 : (160 * 1024) / T_STAGE_BYTES;   // 24 stages up to 6 bpw, 20 at 8
    static constexpr int kBars = 2 * kSkSA + 2 * kSkSW + 2 * ST + 4;
    static constexpr size_t SMEM = 1024 /*align slack*/ + size_t(kSkSA) * kSkAStageBytes + size_t(ST) * T_STAGE_BYTES +
                                   (kXchFloats + 2 * 128) * 4 + kBars * 8;
};
__host__ __device__ inline long long sk_range_begin(int c, long long U, int G) { return (long long) c * U / G; }
// the CTA whose range holds unit u
__host__ __device__ inline int sk_range_owner(long long u, long long U, int G) { return int(((u + 1) * G + U - 1) / U) - 1; }

template <int BITS, int CB>
__global__ void __launch_bounds__(kThreads, 1) k_exl3_gemm_tc_splitk(const __grid_constant__ CUtensorMap tmap_a,
                                                                     const __grid_constant__ CUtensorMap tmap_t, const SplitKArgs p)
{
    using SG_ = SGeo<BITS>;
    constexpr int TROW_BYTES = TGeo<BITS>::TROW_BYTES, T_STAGE_BYTES = SG_::T_STAGE_BYTES, ST = SG_::ST;
    pdl_trigger();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bands = p.n / BN, kstages = p.k / BK;
    const long long U = (long long) bands * kstages;
    const int G = int(gridDim.x);
    const long long u0 = sk_range_begin(blockIdx.x, U, G), u1 = sk_range_begin(blockIdx.x + 1, U, G);
    const int total = int(u1 - u0);
    if (total < 1) return;
    const int band0 = int(u0 / kstages), ks00 = int(u0 - (long long) band0 * kstages);
    const int rows_pad = max((min(p.m, kSkRows) + 15) & ~15, 16);

    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* a_ring = smem;
    unsigned char* t_ring = a_ring + kSkSA * kSkAStageBytes;
    float* xch = reinterpret_cast<float*>(t_ring + ST * T_STAGE_BYTES);
    float* svh_s = xch + kXchFloats;                   // two buffers of 128 scales, alternating between segments
    uint64_t* bars = reinterpret_cast<uint64_t*>(svh_s + 2 * 128);
    __shared__ uint32_t s_tmem_base;

    const uint32_t full_a = smem_u32(bars), empty_a = full_a + 8 * kSkSA;
    const uint32_t full_w = empty_a + 8 * kSkSA, empty_w = full_w + 8 * kSkSW;
    const uint32_t full_t = empty_w + 8 * kSkSW, empty_t = full_t + 8 * ST;
    const uint32_t acc_full = empty_t + 8 * ST, acc_empty = acc_full + 16;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kSkSA; ++s) { mbar_init(full_a + 8 * s, 1); mbar_init(empty_a + 8 * s, 1); }
        for (int s = 0; s < kSkSW; ++s) { mbar_init(full_w + 8 * s, 4); mbar_init(empty_w + 8 * s, 1); }
        for (int s = 0; s < ST; ++s) { mbar_init(full_t + 8 * s, 1); mbar_init(empty_t + 8 * s, 4); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full + 8 * b, 1); mbar_init(acc_empty + 8 * b, 4); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem_base;
    const uint32_t tmem_w = tmem + kSkWCol0;   // weight stages: 32 columns (64 k) each

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer of the trellis stages
        // Its own thread, so that the weight stream runs as far ahead as its ring allows (the DRAM latency under
        // load is several stage times) and never waits for a slot of the short activation ring.  The weights are
        // never written by a kernel, so they may be fetched while the predecessor on the stream is still running.
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_t) : "memory");
            int tb = band0, tks = ks00, st = 0, pt = 0;
            if (p.defer_weights) pdl_wait();   // the caller may have written the weights just before this launch
            for (int i = 0; i < total; ++i) {
                if (i >= ST) mbar_wait_parked(empty_t + 8 * st, pt ^ 1, p.status, 100);
                mbar_arrive_expect_tx(full_t + 8 * st, T_STAGE_BYTES);
                tma_load_3d(smem_u32(t_ring + st * T_STAGE_BYTES), &tmap_t, tb * (TROW_BYTES / 8), tks * 4, 0, full_t + 8 * st);
                if (++st == ST) { st = 0; pt ^= 1; }
                if (++tks == kstages) { tks = 0; ++tb; }
            }
        }
    } else if (warp == 2) {
        // ------------------------------------------------------------ TMA producer of the activation stages
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
            pdl_wait();   // the rotated rows are the predecessor's output
            int aks = ks00, sa = 0, pa = 0;
            for (int i = 0; i < total; ++i) {
                if (i >= kSkSA) mbar_wait_parked(empty_a + 8 * sa, pa ^ 1, p.status, 100);
                mbar_arrive_expect_tx(full_a + 8 * sa, kSkAStageBytes);
                tma_load_2d(smem_u32(a_ring + sa * kSkAStageBytes), &tmap_a, aks * BK, 0, full_a + 8 * sa);
                if (++sa == kSkSA) { sa = 0; pa ^= 1; }
                if (++aks == kstages) aks = 0;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (whole warp, one elected lane issues)
        const uint32_t id = idesc_n(rows_pad);
        int sa = 0, pa = 0, sw = 0, pw = 0, ks = ks00, seg = 0, first = 1;
        for (int i = 0; i < total; ++i) {
            const int buf = seg & 1;
            if (first && seg >= 2) {   // the epilogue has drained this accumulator
                mbar_wait(acc_empty + 8 * buf, ((seg >> 1) - 1) & 1, p.status);
                tc_fence_after();
            }
            mbar_wait(full_a + 8 * sa, pa, p.status);
            mbar_wait(full_w + 8 * sw, pw, p.status);
            tc_fence_after();
            const uint64_t x_desc = smem_desc_sw128(smem_u32(a_ring + sa * kSkAStageBytes));
            const uint32_t w_t = tmem_w + sw * 32, tacc = tmem + buf * kSkRows;
            const uint32_t bar_a = empty_a + 8 * sa, bar_w = empty_w + 8 * sw;
            const bool last = (ks + 1 == kstages) || (i + 1 == total);
            if (elect_one()) {
#pragma unroll
                for (int k16 = 0; k16 < BK / 16; ++k16) tc_mma_ts_f16(tacc, w_t + 8 * k16, x_desc + 2 * k16, id, (first && k16 == 0) ? 0u : 1u);
                tc_commit(bar_a);
                tc_commit(bar_w);
                if (last) tc_commit(acc_full + 8 * buf);
            }
            __syncwarp();
            if (++sa == kSkSA) { sa = 0; pa ^= 1; }
            if (++sw == kSkSW) { sw = 0; pw ^= 1; }
            first = 0;
            if (last) { ++seg; first = 1; ks = 0; } else ++ks;
        }
    } else if (warp >= kDecodeWarp0) {
        // ------------------------------------------------------------ decode warps
        const int g = (warp - kDecodeWarp0) >> 2, quarter = warp & 3;   // group g: stages g, g+4, ... into weight stages g, g+4 in turn
        static_assert(kSkSW == 8 && ST >= 4, "two weight stages per decode group");
        int st = g, pt = 0, j = 0;
        uint32_t pend_w = 0;
        for (int cnt = g; cnt < total; cnt += 4, ++j) {
            mbar_wait(full_t + 8 * st, pt, p.status);
            const int ws = g + 4 * (j & 1);
            sk_decode_stage<BITS, CB>(t_ring + st * T_STAGE_BYTES, tmem_w + ws * 32, quarter, lane, j >= 2, empty_w + 8 * ws,
                                      ((j >> 1) - 1) & 1, p.status, pend_w);
            pend_w = full_w + 8 * ws;
            __syncwarp();   // every lane has read its words of the trellis stage
            if (lane == 0) mbar_arrive(empty_t + 8 * st);
            st += 4;
            if (st >= ST) { st -= ST; pt ^= 1; }
        }
        if (pend_w) {
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(pend_w);
        }
    } else if (warp >= kEpiWarp0 && warp < kEpiWarp0 + 4) {
        // ------------------------------------------------------------ epilogue warps
        const int quarter = warp & 3;
        const int n = quarter * 32 + lane;
        pdl_wait();   // slabs, counters and the output may still be in use by the predecessor
        int seg = 0;
        for (long long u = u0; u < u1; ++seg) {
            const int band = int(u / kstages), ks0 = int(u - (long long) band * kstages);
            const int len = int(min((long long) (kstages - ks0), u1 - u));
            u += len;
            float* sv = svh_s + (seg & 1) * 128;
            sv[n] = __half2float(p.svh[band * BN + n]);
            const int buf = seg & 1;
            mbar_wait_parked(acc_full + 8 * buf, (seg >> 1) & 1, p.status, 200);
            tc_fence_after();
            float v[32];
            tc_ld32(tmem + buf * kSkRows + (uint32_t(quarter * 32) << 16), v);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty + 8 * buf);   // the values are in registers
            if (len < kstages) {
                // a shared band: this segment's partial sums into the CTA's slab
                float* slab = p.slabs + (size_t(blockIdx.x) * 2 + (seg ? 1 : 0)) * (kSkRows * BN);
#pragma unroll
                for (int r = 0; r < 32; ++r)
                    if (r < rows_pad) __stcg(slab + r * BN + n, v[r]);
                continue;
            }
            epilogue_rows(v, xch, sv, 0, quarter, lane, p.c, p.out_fp32, p.n, band * BN, 0, p.m);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// The shared bands of k_exl3_gemm_tc_splitk: block (band, group of four rows), one warp per row, a lane holds four
// consecutive columns.  The slabs of the CTAs whose ranges meet the band are summed in CTA order (four loads in
// flight per lane), then Hadamard, output scale, store.  Bands that one CTA held whole were finished by the main
// kernel; their blocks return at once.
__global__ void __launch_bounds__(128) k_sk_finish(const SplitKArgs p)
{
    pdl_trigger();
    const int band = blockIdx.x, lane = threadIdx.x & 31, row = blockIdx.y * 4 + (threadIdx.x >> 5);
    const int bands = p.n / BN, kstages = p.k / BK, G = p.grid;
    const long long U = (long long) bands * kstages;
    const int c_lo = sk_range_owner((long long) band * kstages, U, G);
    const int c_hi = sk_range_owner((long long) (band + 1) * kstages - 1, U, G);
    pdl_wait();   // (before any return: a grid must not complete before its predecessor, its successor relies on that)
    if (c_lo == c_hi || row >= p.m) return;
    auto slab_of = [&](int cc) {
        // CTA cc's slab of this band: slot 0 when the band is where its range begins
        const int first_band = int(sk_range_begin(cc, U, G) / kstages);
        return p.slabs + ((size_t(cc) * 2 + (first_band == band ? 0 : 1)) * kSkRows + row) * BN + 4 * lane;
    };
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    for (int cc = c_lo; cc <= c_hi; cc += 4) {
        float4 x[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
            x[i] = cc + i <= c_hi ? __ldcg(reinterpret_cast<const float4*>(slab_of(cc + i))) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int i = 0; i < 4; ++i)
            if (cc + i <= c_hi) {
                v[0] = __fadd_rn(v[0], x[i].x); v[1] = __fadd_rn(v[1], x[i].y);
                v[2] = __fadd_rn(v[2], x[i].z); v[3] = __fadd_rn(v[3], x[i].w);
            }
    }
    dq::had128_warp(v, lane);
    const uint2 sr = __ldg(reinterpret_cast<const uint2*>(p.svh + band * BN + 4 * lane));
    const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&sr.x)), s23 = __half22float2(*reinterpret_cast<const __half2*>(&sr.y));
    const float o0 = __fmul_rn(__fmul_rn(v[0], kRScale), s01.x), o1 = __fmul_rn(__fmul_rn(v[1], kRScale), s01.y);
    const float o2 = __fmul_rn(__fmul_rn(v[2], kRScale), s23.x), o3 = __fmul_rn(__fmul_rn(v[3], kRScale), s23.y);
    const size_t at = size_t(row) * p.n + band * BN + 4 * lane;
    if (p.out_fp32) {
        *reinterpret_cast<float4*>(static_cast<float*>(p.c) + at) = make_float4(o0, o1, o2, o3);
    } else {
        uint2 o;
        o.x = dq::pack_half2(__float2half_rn(o0), __float2half_rn(o1));
        o.y = dq::pack_half2(__float2half_rn(o2), __float2half_rn(o3));
        *reinterpret_cast<uint2*>(static_cast<__half*>(p.c) + at) = o;
    }
}

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

CUtensorMap make_map(CUtensorMapDataType type, const void* base, cuuint64_t inner, cuuint64_t outer, cuuint64_t row_bytes,
                     cuuint32_t box_inner, cuuint32_t box_outer, CUtensorMapSwizzle swizzle)
{
    if (reinterpret_cast<uintptr_t>(base) % 16 != 0) throw std::runtime_error("exl3 linear: tensors must be 16-byte aligned");
    CUtensorMap map;
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t elem[2] = {1, 1};
    CUresult r = encode_tiled()(&map, type, 2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) throw std::runtime_error("exl3 linear: cuTensorMapEncodeTiled failed (" + std::to_string(int(r)) + ")");
    return map;
}

// 3-D view of a trellis stack: z = matrix, y = k-tile row (K/16), x = the row in 8-byte elements;
// box = 4 k-tile rows x 8 tiles (one 64 x 128 weight stage) of one matrix.
CUtensorMap make_trellis_map(const void* base, int n_matrices, int size_k, int size_n, int bits, int trow_bytes)
{
    if (reinterpret_cast<uintptr_t>(base) % 16 != 0) throw std::runtime_error("exl3 linear: tensors must be 16-byte aligned");
    CUtensorMap map;
    const cuuint64_t row_bytes = cuuint64_t(size_n / 16) * 32 * bits;
    const cuuint64_t dims[3] = {row_bytes / 8, cuuint64_t(size_k / 16), cuuint64_t(n_matrices)};
    const cuuint64_t strides[2] = {row_bytes, row_bytes * cuuint64_t(size_k / 16)};
    const cuuint32_t box[3] = {cuuint32_t(trow_bytes / 8), 4, 1};
    const cuuint32_t elem[3] = {1, 1, 1};
    CUresult r = encode_tiled()(&map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 3, const_cast<void*>(base), dims, strides, box, elem,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) throw std::runtime_error("exl3 linear: cuTensorMapEncodeTiled failed (" + std::to_string(int(r)) + ")");
    return map;
}

template <int BITS, int CB>
void launch_tc(const void* a_had, const void* trellis, const GemmArgs& args, cudaStream_t stream)
{
    using TG_ = TGeo<BITS>;
    auto kern = k_exl3_gemm_tc<BITS, CB>;
    static bool attr_set[kMaxDevices] = {};
    const int dev = current_device();
    if (!attr_set[dev]) {
        cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(TG_::SMEM)), "gemm smem attribute");
        attr_set[dev] = true;
    }
    // activations [m][k] fp16: box 64 k x 128 rows, 128-byte swizzle (the tensor core's K-major layout)
    const CUtensorMap map_a = make_map(CU_TENSOR_MAP_DATA_TYPE_FLOAT16, a_had, cuuint64_t(args.k), cuuint64_t(args.m),
                                       cuuint64_t(args.k) * 2, BK, SUB, CU_TENSOR_MAP_SWIZZLE_128B);
    const CUtensorMap map_t = make_trellis_map(trellis, args.problems ? args.n_matrices : 1, args.k, args.n, BITS, TG_::TROW_BYTES);
    if (args.problems) {
        auto gk = k_exl3_gemm_tc_grouped<BITS, CB>;
        static bool gattr_set[kMaxDevices] = {};
        if (!gattr_set[dev]) {
            cuda_ok(cudaFuncSetAttribute(gk, cudaFuncAttributeMaxDynamicSharedMemorySize, int(GGeo<BITS>::SMEM)), "grouped gemm smem attribute");
            gattr_set[dev] = true;
        }
        const long long items = (long long) args.max_problems * (args.n / BN);
        const int grid = int(std::min<long long>(items, device_info(dev).sms));
        const CUtensorMap map_a64 = make_map(CU_TENSOR_MAP_DATA_TYPE_FLOAT16, a_had, cuuint64_t(args.k), cuuint64_t(args.m),
                                             cuuint64_t(args.k) * 2, BK, 64, CU_TENSOR_MAP_SWIZZLE_128B);
        const CUtensorMap map_a32 = make_map(CU_TENSOR_MAP_DATA_TYPE_FLOAT16, a_had, cuuint64_t(args.k), cuuint64_t(args.m),
                                             cuuint64_t(args.k) * 2, BK, 32, CU_TENSOR_MAP_SWIZZLE_128B);
        gk<<<grid, kThreads, GGeo<BITS>::SMEM, stream>>>(map_a, map_a64, map_a32, map_t, args);
        cuda_ok(cudaGetLastError(), "k_exl3_gemm_tc_grouped launch");
        return;
    }
    dim3 grid(args.n / BN, (args.m + args.nsub_max * SUB - 1) / (args.nsub_max * SUB));
    kern<<<grid, kThreads, TG_::SMEM, stream>>>(map_a, map_t, args);
    cuda_ok(cudaGetLastError(), "k_exl3_gemm_tc launch");
}

template <int BITS>
void launch_tc_cb(int cb, const void* a_had, const void* trellis, const GemmArgs& a, cudaStream_t st)
{
    switch (cb) {
        case 0: launch_tc<BITS, 0>(a_had, trellis, a, st); break;
        case 1: launch_tc<BITS, 1>(a_had, trellis, a, st); break;
        default: launch_tc<BITS, 2>(a_had, trellis, a, st); break;
    }
}

void launch_tc_bits(int k_bits, int codebook, const void* a_had, const void* trellis, const GemmArgs& args, cudaStream_t stream)
{
    switch (k_bits) {
        case 1: launch_tc_cb<1>(codebook, a_had, trellis, args, stream); break;
        case 2: launch_tc_cb<2>(codebook, a_had, trellis, args, stream); break;
        case 3: launch_tc_cb<3>(codebook, a_had, trellis, args, stream); break;
        case 4: launch_tc_cb<4>(codebook, a_had, trellis, args, stream); break;
        case 5: launch_tc_cb<5>(codebook, a_had, trellis, args, stream); break;
        case 6: launch_tc_cb<6>(codebook, a_had, trellis, args, stream); break;
        case 7: launch_tc_cb<7>(codebook, a_had, trellis, args, stream); break;
        case 8: launch_tc_cb<8>(codebook, a_had, trellis, args, stream); break;
        default: throw std::runtime_error("exl3 linear: K must be in 1..=8");
    }
}

template <int BITS, int CB>
void launch_sk(const void* a_had, const void* trellis, const SplitKArgs& args, int grid, cudaStream_t stream)
{
    using SG_ = SGeo<BITS>;
    auto kern = k_exl3_gemm_tc_splitk<BITS, CB>;
    static bool attr_set[kMaxDevices] = {};
    const int dev = current_device();
    if (!attr_set[dev]) {
        cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SG_::SMEM)), "split-k gemm smem attribute");
        attr_set[dev] = true;
    }
    const CUtensorMap map_a = make_map(CU_TENSOR_MAP_DATA_TYPE_FLOAT16, a_had, cuuint64_t(args.k), cuuint64_t(args.m),
                                       cuuint64_t(args.k) * 2, BK, kSkRows, CU_TENSOR_MAP_SWIZZLE_128B);
    const CUtensorMap map_t = make_trellis_map(trellis, 1, args.k, args.n, BITS, TGeo<BITS>::TROW_BYTES);
    launch_pdl(kern, dim3(grid), dim3(kThreads), SG_::SMEM, stream, "k_exl3_gemm_tc_splitk launch", map_a, map_t, args);
}

template <int BITS>
void launch_sk_cb(int cb, const void* a_had, const void* trellis, const SplitKArgs& a, int grid, cudaStream_t st)
{
    switch (cb) {
        case 0: launch_sk<BITS, 0>(a_had, trellis, a, grid, st); break;
        case 1: launch_sk<BITS, 1>(a_had, trellis, a, grid, st); break;
        default: launch_sk<BITS, 2>(a_had, trellis, a, grid, st); break;
    }
}

void launch_sk_bits(int k_bits, int codebook, const void* a_had, const void* trellis, const SplitKArgs& args, int grid, cudaStream_t stream)
{
    switch (k_bits) {
        case 1: launch_sk_cb<1>(codebook, a_had, trellis, args, grid, stream); break;
        case 2: launch_sk_cb<2>(codebook, a_had, trellis, args, grid, stream); break;
        case 3: launch_sk_cb<3>(codebook, a_had, trellis, args, grid, stream); break;
        case 4: launch_sk_cb<4>(codebook, a_had, trellis, args, grid, stream); break;
        case 5: launch_sk_cb<5>(codebook, a_had, trellis, args, grid, stream); break;
        case 6: launch_sk_cb<6>(codebook, a_had, trellis, args, grid, stream); break;
        case 7: launch_sk_cb<7>(codebook, a_had, trellis, args, grid, stream); break;
        case 8: launch_sk_cb<8>(codebook, a_had, trellis, args, grid, stream); break;
        default: throw std::runtime_error("exl3 linear: K must be in 1..=8");
    }
}

// Rotation of the rows of a grouped launch: out[row] = fp16(H128(x[row] * suh[matrix of the row]) / sqrt(128)).
// One warp per row: it finds the row's problem by bisection over the table of first rows (problems are sorted by
// first row and cover [0, total rows) without gaps; the block keeps the table in shared memory when it fits), then
// walks the row 256 elements at a time: a lane holds eight consecutive elements, sixteen lanes one 128-block, so
// strides 1, 2, 4 of the butterfly stay in registers and 8..64 take four shuffle rounds.
// MODE bits: kRotDual = a second scale stack and output from the same input row (gate and up of an MLP);
// kRotGather = row r < n_perm reads src row perm[r] / div, later rows read src row r - n_perm;
// kRotSilu = the input row is silu(src) * src_u, rounded to fp16 as the element-wise kernel rounds it.
constexpr int kRotDual = 1, kRotGather = 2, kRotSilu = 4, kRotTable = 2048;

__device__ __forceinline__ void had128_lane8(float (&v)[8], int lane)
{
#pragma unroll
    for (int s = 1; s < 8; s <<= 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if ((i & s) == 0) {
                const float a = v[i], b = v[i + s];
                v[i] = __fadd_rn(a, b);
                v[i + s] = __fsub_rn(a, b);
            }
        }
    }
#pragma unroll
    for (int off = 1; off < 16; off <<= 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float o = __shfl_xor_sync(dq::kFull, v[i], off);
            v[i] = (lane & off) ? __fsub_rn(o, v[i]) : __fadd_rn(v[i], o);
        }
    }
}

__device__ __forceinline__ void rotate_store8(const float (&x)[8], const __half* suh, __half* out, int lane, bool active)
{
    float v[8];
    uint4 sm = make_uint4(0u, 0u, 0u, 0u);
    if (active) sm = __ldg(reinterpret_cast<const uint4*>(suh));
    const uint32_t sw[4] = {sm.x, sm.y, sm.z, sm.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&sw[i]));
        v[2 * i] = __fmul_rn(x[2 * i], f.x);
        v[2 * i + 1] = __fmul_rn(x[2 * i + 1], f.y);
    }
    had128_lane8(v, lane);
    if (active) {
        uint4 o;
        o.x = dq::pack_half2(__float2half_rn(__fmul_rn(v[0], kRScale)), __float2half_rn(__fmul_rn(v[1], kRScale)));
        o.y = dq::pack_half2(__float2half_rn(__fmul_rn(v[2], kRScale)), __float2half_rn(__fmul_rn(v[3], kRScale)));
        o.z = dq::pack_half2(__float2half_rn(__fmul_rn(v[4], kRScale)), __float2half_rn(__fmul_rn(v[5], kRScale)));
        o.w = dq::pack_half2(__float2half_rn(__fmul_rn(v[6], kRScale)), __float2half_rn(__fmul_rn(v[7], kRScale)));
        *reinterpret_cast<uint4*>(out) = o;
    }
}

template <int MODE>
__global__ void __launch_bounds__(256) k_rotate_rows_plain(const RotateArgs a)
{
    __shared__ int s_row0[kRotTable];
    pdl_trigger();   // launched as a programmatic dependent; the problem table comes from the preceding kernels
    pdl_wait();
    const int lane = threadIdx.x & 31, k = a.k;
    const int nprob = min(max(__ldg(a.n_problems), 0), a.max_problems);
    if (nprob < 1) return;
    const bool tab = nprob <= kRotTable;
    if (tab) {
        for (int i = threadIdx.x; i < nprob; i += blockDim.x) s_row0[i] = __ldg(&a.problems[i].row0);
        __syncthreads();
    }
    const GemvProblem last = load_problem(a.problems, nprob - 1, a.n_matrices, a.chunk, a.max_rows);
    const int total_rows = min(last.row0 + last.rows, a.max_rows);
    for (int row = blockIdx.x * 8 + (threadIdx.x >> 5); row < total_rows; row += gridDim.x * 8) {
        int src_row = row;
        if constexpr (MODE & kRotGather) src_row = row < a.n_perm ? min(max(__ldg(a.perm + row) / a.div, 0), max(a.n_perm / a.div - 1, 0)) : row - a.n_perm;
        int lo = 0, hi = nprob - 1;   // the last problem whose first row is <= row
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            const int r0 = tab ? s_row0[mid] : __ldg(&a.problems[mid].row0);
            if (r0 <= row) lo = mid; else hi = mid - 1;
        }
        const GemvProblem pr = load_problem(a.problems, lo, a.n_matrices, a.chunk, a.max_rows);
        if (row < pr.row0 || row >= pr.row0 + pr.rows) continue;   // a table with gaps: leave the row alone
        const __half* xs = a.src + size_t(src_row) * k;
        const size_t so = size_t(pr.z) * k, ro = size_t(row) * k;
#pragma unroll 2
        for (int c0 = 0; c0 < k; c0 += 256) {
            const int c = c0 + lane * 8;
            const bool active = c < k;
            float x[8];
            uint4 xm = make_uint4(0u, 0u, 0u, 0u);
            if (active) xm = *reinterpret_cast<const uint4*>(xs + c);
            uint32_t xw[4] = {xm.x, xm.y, xm.z, xm.w};
            if constexpr (MODE & kRotSilu) {
                uint4 um = make_uint4(0u, 0u, 0u, 0u);
                if (active) um = *reinterpret_cast<const uint4*>(a.src_u + size_t(src_row) * k + c);
                const uint32_t uw[4] = {um.x, um.y, um.z, um.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const __half2 g = *reinterpret_cast<const __half2*>(&xw[i]), u = *reinterpret_cast<const __half2*>(&uw[i]);
                    xw[i] = dq::pack_half2(silu_mul_one(__low2half(g), __low2half(u), 0.0f), silu_mul_one(__high2half(g), __high2half(u), 0.0f));
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&xw[i]));
                x[2 * i] = f.x; x[2 * i + 1] = f.y;
            }
            rotate_store8(x, a.suh_a + so + c, a.out_a + ro + c, lane, active);
            if constexpr (MODE & kRotDual) rotate_store8(x, a.suh_b + so + c, a.out_b + ro + c, lane, active);
        }
    }
}
}  // namespace

void had_r_128(const void* input, void* output, const void* scale, int pre_scale, int rows, int cols, int fp32,
               cudaStream_t stream);

// Prefill linear for any row count > 32: rotate the activations, then the tensor-core GEMM.
std::string launch_gemm_tc(const void* a, const void* trellis, void* c, const void* suh, void* a_had, const void* svh,
                           int size_m, int size_k, int size_n, int k_bits, int codebook, int out_fp32, unsigned* status,
                           cudaStream_t stream)
{
    if (size_k % 128 != 0)
        throw std::runtime_error("exl3 linear: no linked kernel for size_k that is not a multiple of 128 (128-wide Hadamard)");
    had_r_128(a, a_had, suh, 1, size_m, size_k, 0, stream);
    GemmArgs args;
    args.c = c;
    args.svh = static_cast<const __half*>(svh);
    args.status = status;
    args.m = size_m; args.k = size_k; args.n = size_n;
    args.out_fp32 = out_fp32;
    args.problems = nullptr; args.n_problems = nullptr; args.max_problems = 0; args.n_matrices = 1;
    args.epi2 = 0;
    // Rows per CTA: 128, 256 or 384.  More rows per decoded weight keep the kernel MMA bound, fewer rows give
    // more CTAs; pick the count with the least (waves x time of one CTA), the latter from the measured stage
    // and epilogue times of the three tile heights (ns per 64-deep stage; ns per epilogue; 1.2 us to start).
    {
        static const int kStageNs[MAX_SUB] = {430, 490, 540}, kEpilogueNs[MAX_SUB] = {4000, 7400, 10300};
        const int sms = device_info(current_device()).sms;
        const int bands = size_n / BN;
        long long best = -1;
        for (int ns = 1; ns <= MAX_SUB; ++ns) {
            const long long ctas = (long long) bands * ((size_m + ns * SUB - 1) / (ns * SUB));
            const long long waves = (ctas + sms - 1) / sms;
            const long long cost = waves * ((long long) (size_k / BK) * kStageNs[ns - 1] + kEpilogueNs[ns - 1] + 1200);
            if (best < 0 || cost <= best) { best = cost; args.nsub_max = ns; }   // ties: more rows per CTA
        }
    }
    launch_tc_bits(k_bits, codebook, a_had, trellis, args, stream);
    return "k_had128<f16,pre> + k_exl3_gemm_tc<" + std::to_string(k_bits) + "," + std::to_string(codebook) + "> grid=" +
           std::to_string(size_n / BN) + "x" + std::to_string((size_m + args.nsub_max * SUB - 1) / (args.nsub_max * SUB)) +
           " block=" + std::to_string(kThreads) + " tile=" + std::to_string(args.nsub_max * SUB) + "x128x64 tmem=512";
}

// Decode batches of up to 32 rows on the tensor-core path: rotate the rows, then the persistent split-K kernel.
std::string launch_gemm_tc_splitk(const void* a, const void* trellis, void* c, const void* suh, void* a_had, const void* svh,
                                  int size_m, int size_k, int size_n, int k_bits, int codebook, int out_fp32, const GemvScratch& sc,
                                  int sms, cudaStream_t stream)
{
    if (size_k % 128 != 0)
        throw std::runtime_error("exl3 linear: no linked kernel for size_k that is not a multiple of 128 (128-wide Hadamard)");
    if (size_m < 1 || size_m > kSkRows) throw std::runtime_error("exl3 linear (small-batch tensor path): size_m must be in 1..=32");
    const long long units = (long long) (size_n / BN) * (size_k / BK);
    int grid = int(std::min<long long>(sms, units));
    const size_t per_cta = size_t(2) * kSkRows * BN * sizeof(float);
    if (size_t(grid) * per_cta > sc.slab_bytes) grid = int(sc.slab_bytes / per_cta);
    if (grid < 1) throw std::runtime_error("exl3 linear: split-K scratch is too small for this shape");
    had_r_128(a, a_had, suh, 1, size_m, size_k, 0, stream);
    SplitKArgs args;
    args.defer_weights = weights_streamed() ? 1 : 0;
    args.c = c;
    args.svh = static_cast<const __half*>(svh);
    args.status = sc.status;
    args.slabs = sc.slabs;
    args.m = size_m; args.k = size_k; args.n = size_n;
    args.out_fp32 = out_fp32;
    args.grid = grid;
    launch_sk_bits(k_bits, codebook, a_had, trellis, args, grid, stream);
    // shared bands exist unless every range boundary falls on a band boundary
    const bool shared = units % grid != 0 || (units / grid) % (size_k / BK) != 0;
    if (shared)
        launch_pdl(k_sk_finish, dim3(size_n / BN, (size_m + 3) / 4), dim3(128), 0, stream, "k_sk_finish launch", args);
    return "k_had128<f16,pre> + k_exl3_gemm_tc_splitk<" + std::to_string(k_bits) + "," + std::to_string(codebook) + "> grid=" +
           std::to_string(grid) + " block=" + std::to_string(kThreads) + " stage=64x128 rows=" + std::to_string((size_m + 15) / 16 * 16) +
           (shared ? " + k_sk_finish" : "");
}

void rotate_rows_grouped(const RotateArgs& a, bool dual, bool silu, int sms, cudaStream_t stream)
{
    if (a.k % 128 != 0) throw std::runtime_error("exl3 grouped gemm: size_k must be a multiple of 128");
    if (!a.src || !a.suh_a || !a.out_a || (dual && (!a.suh_b || !a.out_b)) || (silu && !a.src_u))
        throw std::runtime_error("exl3 grouped gemm: null rotation pointer");
    if (silu && (dual || a.perm)) throw std::runtime_error("exl3 grouped gemm: the silu rotation takes one plain input");
    const dim3 grid(std::max(1, std::min((a.max_rows + 7) / 8, 8 * sms)));
    const int mode = (dual ? kRotDual : 0) | (a.perm ? kRotGather : 0) | (silu ? kRotSilu : 0);
    switch (mode) {
        case 0: launch_pdl(k_rotate_rows_plain<0>, grid, dim3(256), 0, stream, "k_rotate_rows_plain launch", a); break;
        case kRotDual: launch_pdl(k_rotate_rows_plain<kRotDual>, grid, dim3(256), 0, stream, "k_rotate_rows_plain launch", a); break;
        case kRotGather: launch_pdl(k_rotate_rows_plain<kRotGather>, grid, dim3(256), 0, stream, "k_rotate_rows_plain launch", a); break;
        case kRotDual | kRotGather: launch_pdl(k_rotate_rows_plain<kRotDual | kRotGather>, grid, dim3(256), 0, stream, "k_rotate_rows_plain launch", a); break;
        default: launch_pdl(k_rotate_rows_plain<kRotSilu>, grid, dim3(256), 0, stream, "k_rotate_rows_plain launch", a); break;
    }
    cuda_ok(cudaGetLastError(), "k_rotate_rows_plain launch");
}

std::string launch_gemm_tc_grouped_rotated(const void* xr_had, const void* trellis_stack, int n_matrices, void* c, const void* svh_stack,
                                           const GemvProblem* problems, const int* n_problems, int max_problems, int max_rows, int nsub,
                                           int size_k, int size_n, int k_bits, int codebook, int out_fp32, unsigned* status, int sms,
                                           cudaStream_t stream)
{
    (void) sms;
    if (size_k % 128 != 0 || size_n % 128 != 0)
        throw std::runtime_error("exl3 grouped gemm: size_k and size_n must be multiples of 128");
    if (nsub < 1 || nsub > MAX_SUB) throw std::runtime_error("exl3 grouped gemm: row chunks must be 128, 256 or 384 rows");
    if (max_problems < 1 || max_problems > 65535) throw std::runtime_error("exl3 grouped gemm: problem count out of range");
    GemmArgs args;
    args.c = c;
    args.svh = static_cast<const __half*>(svh_stack);
    args.status = status;
    args.m = max_rows; args.k = size_k; args.n = size_n;
    args.out_fp32 = out_fp32;
    args.nsub_max = nsub;
    args.problems = problems; args.n_problems = n_problems; args.max_problems = max_problems; args.n_matrices = n_matrices;
    // a main loop of at most sixteen stages is shorter than the epilogue of a 128-row item
    args.epi2 = (nsub == 1 && size_k <= 1024) ? 1 : 0;
    launch_tc_bits(k_bits, codebook, xr_had, trellis_stack, args, stream);
    return "k_exl3_gemm_tc_grouped<" + std::to_string(k_bits) + "," + std::to_string(codebook) + "> persistent items<=" +
           std::to_string(size_n / BN) + "x" + std::to_string(max_problems) + " block=" + std::to_string(kThreads) + " tile=" +
           std::to_string(nsub * SUB) + "x128x64 tmem=512";
}

// Grouped prefill linear over a stack of equally shaped matrices: problem i applies matrix z_i to rows
// [row0_i, row0_i + rows_i) of xr (rows_i <= 128 * nsub); xr_had [max_rows][k] receives the rotated rows.
std::string launch_gemm_tc_grouped(const void* xr, void* xr_had, const void* trellis_stack, int n_matrices, void* c,
                                   const void* suh_stack, const void* svh_stack, const GemvProblem* problems, const int* n_problems,
                                   int max_problems, int max_rows, int nsub, int size_k, int size_n, int k_bits, int codebook,
                                   int out_fp32, unsigned* status, int sms, cudaStream_t stream)
{
    if (max_problems < 1 || max_problems > 65535) throw std::runtime_error("exl3 grouped gemm: problem count out of range");
    RotateArgs r{};
    r.src = static_cast<const __half*>(xr);
    r.suh_a = static_cast<const __half*>(suh_stack);
    r.out_a = static_cast<__half*>(xr_had);
    r.problems = problems; r.n_problems = n_problems;
    r.chunk = nsub * SUB; r.k = size_k; r.max_problems = max_problems; r.n_matrices = n_matrices; r.max_rows = max_rows;
    rotate_rows_grouped(r, false, false, sms, stream);
    return "k_rotate_rows_plain + " + launch_gemm_tc_grouped_rotated(xr_had, trellis_stack, n_matrices, c, svh_stack, problems, n_problems,
                                                                     max_problems, max_rows, nsub, size_k, size_n, k_bits, codebook,
                                                                     out_fp32, status, sms, stream);
}

}  // namespace berth
