// Prefill EXL3 linear on the 5th-generation tensor cores (size_m > 32):
//   C = H128( a_had . W ) * svh,  a_had = H128(A * suh) (rotated beforehand by k_had128),
// with W never materialised in HBM: trellis tiles arrive by TMA, eight decode warps expand
// them (bit-exact fp16 weights) straight into the swizzled K-major shared-memory operand of
// tcgen05.mma, the fp32 accumulators live in tensor memory, and the epilogue applies the
// output Hadamard and the svh sign-scale before the only write of C.
//
// Tile: one CTA owns 128 output columns (one Hadamard band) for up to 512 token rows -- four
// 128x128 fp32 accumulators, all 512 TMEM columns -- so every decoded weight feeds 512 tokens:
// per 64-deep k stage the tensor pipe needs 4 x (128x128x64) MACs = 1024 cycles while the decode
// warps expand 32 tiles (~1600 warp instructions), which keeps the kernel MMA bound.
// Roofline: tensor pipe; FLOPs = 2*M*K*N.
//
// Warp roles (16 warps, one CTA per SM):
//   warp 0      TMA producer: A stages (4 boxes of 128 rows x 64 k, 128-byte swizzle) and raw
//               trellis stages (4 k-tile rows x 8 tiles);
//   warp 1      TMEM allocation + the single MMA-issuing thread;
//   warps 4..7  epilogue: tcgen05.ld, Hadamard, scale, store (warp w reads TMEM lanes 32*(w%4)..);
//   warps 8..15 decode: trellis words -> fp16 pairs -> swizzled B stage.
// All waits are bounded: a wait that runs out sets a status bit and the kernel carries on and
// exits (wrong output, no hang).
#include "exl3_decode.cuh"

#include <cuda.h>

#include <algorithm>

namespace berth {
namespace {

constexpr int kThreads = 512;
constexpr int kDecodeWarp0 = 8, kDecodeWarps = 8;
constexpr int kEpiWarp0 = 4;
constexpr int BN = 128, BK = 64, SUB = 128, MAX_SUB = 4;
constexpr int SA = 2;   // A stages
constexpr int SB = 3;   // decoded-B stages
constexpr int ST = 4;   // raw trellis stages
constexpr int A_SUB_BYTES = SUB * BK * 2;          // 16 KiB
constexpr int A_STAGE_BYTES = MAX_SUB * A_SUB_BYTES;
constexpr int B_STAGE_BYTES = BN * BK * 2;         // 16 KiB
constexpr long long kWaitCycles = 500000000LL;

enum : unsigned { kStGemmTimeout = 16u };

template <int BITS>
struct TGeo {
    static constexpr int NW = 8 * BITS;
    static constexpr int TROW_BYTES = 8 * NW * 4;          // one k-tile row of the band
    static constexpr int T_STAGE_BYTES = 4 * TROW_BYTES;   // 64 k rows
    static constexpr size_t SMEM = 1024 /*align slack*/ + size_t(SA) * A_STAGE_BYTES + size_t(SB) * B_STAGE_BYTES +
                                   size_t(ST) * T_STAGE_BYTES + 256 /*barriers*/;
};

struct GemmArgs {
    void* c;
    const __half* svh;
    unsigned* status;
    int m, k, n, out_fp32;
    int nsub_max;   // 128-row sub-tiles per CTA (1..4): the row block of a CTA is nsub_max*128 tokens
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
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]^T, fp16 in, fp32 out, 128 x 128 x 16.
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
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
__device__ __forceinline__ void tc_st32(uint32_t taddr, const float (&v)[32])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
          "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
          "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
          "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
          "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])),
          "r"(__float_as_uint(v[19])), "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])),
          "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])),
          "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])),
          "r"(__float_as_uint(v[31]))
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
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
// Instruction descriptor: D fp32, A/B fp16, both K-major, M = 128, N = 128.
constexpr uint32_t kIdesc = (1u << 4) | (uint32_t(BN >> 3) << 17) | (uint32_t(SUB >> 4) << 24);

// 32-point Hadamard butterfly (strides 1..16) on registers.
__device__ __forceinline__ void had32_regs(float (&v)[32])
{
#pragma unroll
    for (int s = 1; s < 32; s <<= 1)
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (!(i & s)) {
                const float a = v[i], b = v[i | s];
                v[i] = a + b;
                v[i | s] = a - b;
            }
}

// ---------------------------------------------------------------- the kernel
template <int BITS, int CB>
__global__ void __launch_bounds__(kThreads, 1) k_exl3_gemm_tc(const __grid_constant__ CUtensorMap tmap_a,
                                                              const __grid_constant__ CUtensorMap tmap_t, const GemmArgs p)
{
    using TG_ = TGeo<BITS>;
    constexpr int NW = TG_::NW, TROW_BYTES = TG_::TROW_BYTES, T_STAGE_BYTES = TG_::T_STAGE_BYTES;

    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* a_ring = smem;
    unsigned char* b_ring = a_ring + SA * A_STAGE_BYTES;
    unsigned char* t_ring = b_ring + SB * B_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(t_ring + ST * T_STAGE_BYTES);
    __shared__ uint32_t s_tmem_base;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int band = blockIdx.x, m0 = blockIdx.y * (p.nsub_max * SUB);
    const int rows_here = min(p.m - m0, p.nsub_max * SUB);
    const int nsub = (rows_here + SUB - 1) / SUB;
    const int kstages = p.k / BK;

    const uint32_t full_a = smem_u32(bars), empty_a = full_a + 8 * SA;
    const uint32_t full_b = empty_a + 8 * SA, empty_b = full_b + 8 * SB;
    const uint32_t full_t = empty_b + 8 * SB, empty_t = full_t + 8 * ST;
    const uint32_t acc_full = empty_t + 8 * ST;

    if (threadIdx.x == 0) {
        for (int s = 0; s < SA; ++s) { mbar_init(full_a + 8 * s, 1); mbar_init(empty_a + 8 * s, 1); }
        for (int s = 0; s < SB; ++s) { mbar_init(full_b + 8 * s, kDecodeWarps); mbar_init(empty_b + 8 * s, 1); }
        for (int s = 0; s < ST; ++s) { mbar_init(full_t + 8 * s, 1); mbar_init(empty_t + 8 * s, kDecodeWarps); }
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

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_t) : "memory");
            int sa = 0, pa = 0, st = 0, pt = 0;
            for (int ks = 0; ks < kstages; ++ks) {
                // raw trellis: 4 k-tile rows of this band
                if (ks >= ST) mbar_wait(empty_t + 8 * st, pt ^ 1, p.status);
                mbar_arrive_expect_tx(full_t + 8 * st, T_STAGE_BYTES);
                tma_load_2d(smem_u32(t_ring + st * T_STAGE_BYTES), &tmap_t, band * (TROW_BYTES / 8), ks * 4, full_t + 8 * st);
                if (++st == ST) { st = 0; pt ^= 1; }
                // activations: nsub boxes of 128 rows x 64 k
                if (ks >= SA) mbar_wait(empty_a + 8 * sa, pa ^ 1, p.status);
                mbar_arrive_expect_tx(full_a + 8 * sa, nsub * A_SUB_BYTES);
                for (int sub = 0; sub < nsub; ++sub)
                    tma_load_2d(smem_u32(a_ring + sa * A_STAGE_BYTES + sub * A_SUB_BYTES), &tmap_a, ks * BK, m0 + sub * SUB,
                                full_a + 8 * sa);
                if (++sa == SA) { sa = 0; pa ^= 1; }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            int sa = 0, pa = 0, sb = 0, pb = 0;
            for (int ks = 0; ks < kstages; ++ks) {
                mbar_wait(full_a + 8 * sa, pa, p.status);
                mbar_wait(full_b + 8 * sb, pb, p.status);
                tc_fence_after();
                const uint32_t a_base = smem_u32(a_ring + sa * A_STAGE_BYTES);
                const uint64_t b_desc0 = smem_desc_sw128(smem_u32(b_ring + sb * B_STAGE_BYTES));
                for (int sub = 0; sub < nsub; ++sub) {
                    const uint64_t a_desc0 = smem_desc_sw128(a_base + sub * A_SUB_BYTES);
#pragma unroll
                    for (int k16 = 0; k16 < BK / 16; ++k16)   // +32 bytes (2 x 16-byte units) per 16 k inside the swizzle atom
                        tc_mma_f16(tmem + sub * BN, a_desc0 + 2 * k16, b_desc0 + 2 * k16, kIdesc, (ks | k16) ? 1u : 0u);
                }
                tc_commit(empty_a + 8 * sa);   // both arrive when the MMAs above have read their operands
                tc_commit(empty_b + 8 * sb);
                if (++sa == SA) { sa = 0; pa ^= 1; }
                if (++sb == SB) { sb = 0; pb ^= 1; }
            }
            tc_commit(acc_full);
        }
    } else if (warp >= kDecodeWarp0) {
        // ------------------------------------------------------------ decode warps
        const int d = warp - kDecodeWarp0;
        const int krow = d >> 1, col0 = (d & 1) * 4;   // this warp: k-tile row krow of the stage, tile columns col0..col0+3
        const int g = lane >> 2, q = lane & 3;
        int st = 0, pt = 0, sb = 0, pb = 0;
        for (int ks = 0; ks < kstages; ++ks) {
            mbar_wait(full_t + 8 * st, pt, p.status);
            if (ks >= SB) mbar_wait(empty_b + 8 * sb, pb ^ 1, p.status);
            const uint32_t* trow = reinterpret_cast<const uint32_t*>(t_ring + st * T_STAGE_BYTES + krow * TROW_BYTES);
            unsigned char* bst = b_ring + sb * B_STAGE_BYTES;
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                uint32_t s[8], w[4];
                dq::lane_states<BITS>(trow + (col0 + t) * NW, lane, s);
                dq::decode_frag<CB>(s, w);
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const int n = (col0 + t) * 16 + g + 8 * (r & 1);
                    const int chunk = 2 * krow + (r >> 1);           // 16-byte chunk of k = 16*krow + 8*(r>>1) + 2q
                    *reinterpret_cast<uint32_t*>(bst + n * 128 + ((chunk ^ (n & 7)) << 4) + 4 * q) = w[r];
                }
            }
            fence_proxy_async();   // generic-proxy stores -> visible to the tensor core's async proxy
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(full_b + 8 * sb);
                mbar_arrive(empty_t + 8 * st);
            }
            if (++st == ST) { st = 0; pt ^= 1; }
            if (++sb == SB) { sb = 0; pb ^= 1; }
        }
    } else if (warp >= kEpiWarp0 && warp < kEpiWarp0 + 4) {
        // ------------------------------------------------------------ epilogue
        const int quarter = warp & 3;
        mbar_wait(acc_full, 0, p.status);
        tc_fence_after();
        const float* dummy = nullptr; (void) dummy;
        for (int sub = 0; sub < nsub; ++sub) {
            const uint32_t tbase = tmem + (uint32_t(quarter * 32) << 16) + sub * BN;
            // strides 64 and 32 across the four 32-column blocks, in place in tensor memory
            {
                float x0[32], x2[32];
                tc_ld32(tbase + 0, x0); tc_ld32(tbase + 64, x2);
#pragma unroll
                for (int i = 0; i < 32; ++i) { const float a = x0[i], b = x2[i]; x0[i] = a + b; x2[i] = a - b; }
                tc_st32(tbase + 0, x0); tc_st32(tbase + 64, x2);
                tc_ld32(tbase + 32, x0); tc_ld32(tbase + 96, x2);
#pragma unroll
                for (int i = 0; i < 32; ++i) { const float a = x0[i], b = x2[i]; x0[i] = a + b; x2[i] = a - b; }
                tc_st32(tbase + 32, x0); tc_st32(tbase + 96, x2);
            }
            const int row = m0 + sub * SUB + quarter * 32 + lane;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                float y0[32], y1[32];
                tc_ld32(tbase + half * 64, y0); tc_ld32(tbase + half * 64 + 32, y1);
#pragma unroll
                for (int i = 0; i < 32; ++i) { const float a = y0[i], b = y1[i]; y0[i] = a + b; y1[i] = a - b; }
                had32_regs(y0);
                had32_regs(y1);
                if (row < p.m) {
#pragma unroll
                    for (int blk = 0; blk < 2; ++blk) {
                        float (&y)[32] = blk ? y1 : y0;
                        const int col = band * BN + half * 64 + blk * 32;
                        if (p.out_fp32) {
                            float* dst = static_cast<float*>(p.c) + size_t(row) * p.n + col;
#pragma unroll
                            for (int i = 0; i < 32; i += 4) {
                                float4 o;
                                o.x = y[i] * kRScale * __half2float(p.svh[col + i]);
                                o.y = y[i + 1] * kRScale * __half2float(p.svh[col + i + 1]);
                                o.z = y[i + 2] * kRScale * __half2float(p.svh[col + i + 2]);
                                o.w = y[i + 3] * kRScale * __half2float(p.svh[col + i + 3]);
                                *reinterpret_cast<float4*>(dst + i) = o;
                            }
                        } else {
                            __half* dst = static_cast<__half*>(p.c) + size_t(row) * p.n + col;
#pragma unroll
                            for (int i = 0; i < 32; i += 8) {
                                uint4 o;
                                uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
                                for (int j = 0; j < 4; ++j)
                                    ow[j] = dq::pack_half2(
                                        __float2half_rn(y[i + 2 * j] * kRScale * __half2float(p.svh[col + i + 2 * j])),
                                        __float2half_rn(y[i + 2 * j + 1] * kRScale * __half2float(p.svh[col + i + 2 * j + 1])));
                                *reinterpret_cast<uint4*>(dst + i) = o;
                            }
                        }
                    }
                }
            }
        }
        tc_fence_before();
    }

    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
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
    // trellis as [k/16][row bytes / 8] 8-byte elements: box = 8 tiles x 4 k-tile rows
    const cuuint64_t row_bytes = cuuint64_t(args.n / 16) * 32 * BITS;
    const CUtensorMap map_t = make_map(CU_TENSOR_MAP_DATA_TYPE_UINT64, trellis, row_bytes / 8, cuuint64_t(args.k / 16), row_bytes,
                                       TG_::TROW_BYTES / 8, 4, CU_TENSOR_MAP_SWIZZLE_NONE);
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
    // Rows per CTA: 128..512.  More rows per decoded weight keep the kernel MMA bound (the decode
    // warps need ~640 cycles per 64-deep stage, one 128-row sub-tile 256), fewer rows give more
    // CTAs; pick the count with the fewest (waves x stage time) on this device.
    {
        const int sms = device_info(current_device()).sms;
        const int bands = size_n / BN;
        long long best = -1;
        for (int ns = 1; ns <= MAX_SUB; ++ns) {
            const long long ctas = (long long) bands * ((size_m + ns * SUB - 1) / (ns * SUB));
            const long long waves = (ctas + sms - 1) / sms;
            const long long cost = waves * std::max(ns * 256, 640);
            if (best < 0 || cost <= best) { best = cost; args.nsub_max = ns; }   // ties: more rows per CTA
        }
    }
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
    return "k_had128<f16,pre> + k_exl3_gemm_tc<" + std::to_string(k_bits) + "," + std::to_string(codebook) + "> grid=" +
           std::to_string(size_n / BN) + "x" + std::to_string((size_m + args.nsub_max * SUB - 1) / (args.nsub_max * SUB)) +
           " block=" + std::to_string(kThreads) + " tile=" + std::to_string(args.nsub_max * SUB) + "x128x64 tmem=512";
}

}  // namespace berth
