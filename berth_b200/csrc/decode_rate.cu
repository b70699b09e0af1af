// Bare decode rate of one SM: the inner loop of the decode GEMV (shared-memory tile words ->
// window extraction -> codebook arithmetic -> tensor-core MMA) run on tiles that already sit in
// shared memory, with no global-memory traffic, no pipeline and no epilogue.  The figure it returns
// (weights per clock per SM) is the ceiling the instruction issue of the SM puts on any kernel
// built from these primitives; at BITS bits per weight the HBM roofline asks for
// hbm_bytes_per_clock_per_sm * 8 / BITS weights per clock per SM.  Diagnostic only: no counterpart
// in berth, nothing on the product path calls it.
#include "exl3_decode.cuh"
#include "../../include/berth_b200.h"

#include <vector>

namespace berth {
namespace {

constexpr int kRateTiles = 64;   // distinct tiles in shared memory (re-read round robin)

// PATH 0: fp16 path (3INST / MCG: two fp16 halves as two k-slots; MUL1: dp4a byte sum + pair
// packing, one m16n8k16 per tile), four tile columns per warp sharing one activation fragment.
// PATH 1: MUL1 on the integer tensor path with the legacy warp-level MMA (multiply only, two m16n8k32
// per tile), two tile columns per warp, partial sums converted to fp32 after every four k-tile rows.
// PATH 2: MUL1 on the integer tensor path as the decode kernel runs it: multiply only, the eight
// products of a tile stored into tensor memory (one tcgen05.st per tile), no MMA issued here (the
// asynchronous tcgen05.mma takes no issue slot of the decoding warps).
template <int BITS, int CB, int PATH>
__global__ void __launch_bounds__(1024, 1) k_decode_rate(uint32_t seed, int iters, unsigned long long* cycles,
                                                         unsigned long long* nanos, float* sink)
{
    constexpr int NW = 8 * BITS;
    extern __shared__ __align__(16) uint32_t sm[];
    uint32_t* tiles = sm;                       // [kRateTiles][NW]
    uint32_t* act = sm + kRateTiles * NW;       // 8 k-tile rows x 128 words
    for (int i = threadIdx.x; i < kRateTiles * NW + 8 * 128; i += blockDim.x) {
        uint32_t x = (seed + i) * 0x9E3779B1u;
        x ^= x >> 15; x *= 0x85EBCA77u; x ^= x >> 13;
        sm[i] = x;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, lane1 = (lane + 1) & 31;
    __shared__ uint32_t tmem_base_s;
    if (PATH == 2 && warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"((uint32_t) __cvta_generic_to_shared(&tmem_base_s)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = PATH == 2 ? tmem_base_s : 0u;
    unsigned long long t0 = clock64(), n0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(n0));
    float total = 0.f;
    if constexpr (PATH == 2) {
        const uint32_t tbase = tmem_base + (uint32_t(32 * (warp & 3)) << 16);
        uint32_t keep = 0;
        for (int it = 0; it < iters; ++it) {
#pragma unroll
            for (int r = 0; r < 4; ++r) {
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    uint32_t st[8], x[8];
                    dq::tile_states_i8<BITS>(tiles + ((warp * 8 + it * 8 + r * 2 + t) % kRateTiles) * NW, lane, lane1, st);
#pragma unroll
                    for (int j = 0; j < 8; ++j) x[j] = st[j] * 0x83DCD12Du;
                    keep ^= x[0];
                    asm volatile("tcgen05.st.sync.aligned.16x128b.x4.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                                 ::"r"(tbase + (uint32_t(16 * t) << 16) + 16 * ((warp >> 2) * 4 + r)), "r"(x[0]), "r"(x[2]), "r"(x[1]), "r"(x[3]),
                                   "r"(x[4]), "r"(x[6]), "r"(x[5]), "r"(x[7])
                                 : "memory");
                }
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
        total = __uint_as_float(keep);
    } else if constexpr (PATH == 0) {
        float acc[4][1][4] = {};
        for (int it = 0; it < iters; ++it) {
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                dq::RowFrag<CB, 1> f;
                f.load(act + ((it + r) & 7) * 64, lane);
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    uint32_t st[8];
                    dq::tile_states<BITS, CB>(tiles + ((warp * 8 + it * 8 + r * 4 + t) % kRateTiles) * NW, lane, lane1, st);
                    dq::tile_mma<CB, 1>(st, acc[t], f);
                }
            }
        }
#pragma unroll
        for (int t = 0; t < 4; ++t) total += acc[t][0][0] + acc[t][0][1] + acc[t][0][2] + acc[t][0][3];
    } else {
        float facc[2][2] = {};
        for (int it = 0; it < iters; ++it) {
            int acc[2][1][4] = {};
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                uint4 b[1];
                b[0] = *reinterpret_cast<const uint4*>(act + ((it + r) & 7) * 128 + lane * 4);
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    uint32_t st[8];
                    dq::tile_states_i8<BITS>(tiles + ((warp * 8 + it * 8 + r * 2 + t) % kRateTiles) * NW, lane, lane1, st);
                    dq::tile_mma_i8<1>(st, acc[t], b);
                }
            }
            const float scale = __uint_as_float(0x3f800000u + (it & 7));
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                facc[t][0] = fmaf(scale, float(acc[t][0][0] * 256 + acc[t][0][1]), facc[t][0]);
                facc[t][1] = fmaf(scale, float(acc[t][0][2] * 256 + acc[t][0][3]), facc[t][1]);
            }
        }
        total = facc[0][0] + facc[0][1] + facc[1][0] + facc[1][1];
    }
    __syncthreads();
    unsigned long long t1 = clock64(), n1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(n1));
    if (threadIdx.x == 0) {
        cycles[blockIdx.x] = t1 - t0;
        nanos[blockIdx.x] = n1 - n0;
    }
    if (total == 12345.678f) sink[0] = total;   // keeps the arithmetic alive
    if (PATH == 2) {
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (warp == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
        }
    }
}

// Pipe probe: which instructions of the decode loop share an issue pipe.  Every warp runs `iters` iterations of a fixed
// bundle on independent registers: KIND 0 = two mma.sync.m16n8k16; 1 = the same plus eight lop3; 2 = the same plus eight
// 32-bit multiplies; 3 = eight lop3 plus eight multiplies, no MMA; 4 = two mma.sync.m16n8k32 (u8 x s8); 5 = those plus
// eight lop3.  Returns cycles per iteration and scheduler (the block has 16 warps, four per scheduler).
template <int KIND>
__global__ void __launch_bounds__(512, 1) k_pipe_probe(uint32_t seed, int iters, unsigned long long* cycles, uint32_t* sink)
{
    uint32_t v[8], w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { v[i] = seed + threadIdx.x * 7 + i; w[i] = seed * 3 + threadIdx.x * 5 + i; }
    float f[2][4] = {};
    int d[2][4] = {};
    const uint32_t c1 = seed | 1, c2 = seed ^ 0x5555;
    __syncthreads();
    const unsigned long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
        if constexpr (KIND == 0 || KIND == 1 || KIND == 2) {
            uint32_t a0[4] = {v[0], v[1], v[2], v[3]}, a1[4] = {w[0], w[1], w[2], w[3]};
            dq::mma_16816(f[0], a0, c1, c2);
            dq::mma_16816(f[1], a1, c1, c2);
        }
        if constexpr (KIND == 4 || KIND == 5) {
            dq::mma_16832_u8s8(d[0], v[0], v[1], v[2], v[3], c1, c2);
            dq::mma_16832_u8s8(d[1], w[0], w[1], w[2], w[3], c1, c2);
        }
        if constexpr (KIND == 1 || KIND == 3 || KIND == 5) {
#pragma unroll
            for (int i = 4; i < 8; ++i) { v[i] = dq::lop3_mask_xor(v[i]); w[i] = dq::lop3_mask_xor(w[i] + 1); }
        }
        if constexpr (KIND == 2 || KIND == 3) {
#pragma unroll
            for (int i = 4; i < 8; ++i) {
                asm volatile("mad.lo.u32 %0, %0, 0x83DCD12D, 0;" : "+r"(v[KIND == 3 ? i - 4 : i]));   // (KIND 3: registers the lop3s do not touch)
                asm volatile("mad.lo.u32 %0, %0, 0x83DCD12D, 0;" : "+r"(w[KIND == 3 ? i - 4 : i]));
            }
        }
    }
    const unsigned long long t1 = clock64();
    uint32_t acc = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc ^= v[i] ^ w[i];
#pragma unroll
    for (int i = 0; i < 4; ++i) acc ^= __float_as_uint(f[0][i] + f[1][i]) ^ uint32_t(d[0][i] ^ d[1][i]);
    if (threadIdx.x == 0) cycles[blockIdx.x] = t1 - t0;
    if (acc == 0x12345678u) sink[0] = acc;
}

template <int BITS, int CB, int PATH>
void launch_rate(int grid, int warps, int iters, unsigned long long* cyc, unsigned long long* ns, float* sink, cudaStream_t st)
{
    const size_t smem = size_t(kRateTiles * 8 * BITS + 8 * 128) * 4;
    auto kern = k_decode_rate<BITS, CB, PATH>;
    cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)), "decode rate smem attribute");
    kern<<<grid, warps * 32, smem, st>>>(0x1234567u, iters, cyc, ns, sink);
    cuda_ok(cudaGetLastError(), "k_decode_rate launch");
}

template <int BITS>
void launch_rate_bits(int cb, int path, int grid, int warps, int iters, unsigned long long* cyc, unsigned long long* ns, float* sink,
                      cudaStream_t st)
{
    if (path >= 1) {
        if (cb != 2) throw std::runtime_error("decode rate: the integer tensor path exists for the MUL1 codebook only");
        if (path == 2) return launch_rate<BITS, 2, 2>(grid, warps, iters, cyc, ns, sink, st);
        return launch_rate<BITS, 2, 1>(grid, warps, iters, cyc, ns, sink, st);
    }
    switch (cb) {
        case 0: return launch_rate<BITS, 0, 0>(grid, warps, iters, cyc, ns, sink, st);
        case 1: return launch_rate<BITS, 1, 0>(grid, warps, iters, cyc, ns, sink, st);
        default: return launch_rate<BITS, 2, 0>(grid, warps, iters, cyc, ns, sink, st);
    }
}

}  // namespace
}  // namespace berth

extern "C" int berth_exl3_decode_rate(int k_bits, int codebook, int path, int warps, int iters, double* weights_per_clk_sm,
                                      double* sm_mhz)
{
    using namespace berth;
    return guarded(exl3_state(), [&] {
        if (!weights_per_clk_sm || !sm_mhz) throw std::runtime_error("decode rate: null result pointer");
        if (codebook < 0 || codebook > 2) throw std::runtime_error("decode rate: codebook must be 0, 1 or 2");
        if (path < 0 || path > 2) throw std::runtime_error("decode rate: path must be 0 (fp16), 1 (integer, mma.sync) or 2 (integer, tensor memory)");
        if (path == 2 && warps > 16) throw std::runtime_error("decode rate: the tensor-memory path takes at most 16 warps (512 columns)");
        if (warps < 1 || warps > 32 || iters < 1 || iters > (1 << 20)) throw std::runtime_error("decode rate: warps 1..32, iters 1..2^20");
        const int device = current_device();
        const int sms = device_info(device).sms;
        unsigned long long *cyc = nullptr, *ns = nullptr;
        float* sink = nullptr;
        cuda_ok(cudaMalloc(&cyc, size_t(sms) * 8), "decode rate alloc");
        cuda_ok(cudaMalloc(&ns, size_t(sms) * 8), "decode rate alloc");
        cuda_ok(cudaMalloc(&sink, 4), "decode rate alloc");
        auto run = [&] {
            switch (k_bits) {
                case 3: launch_rate_bits<3>(codebook, path, sms, warps, iters, cyc, ns, sink, nullptr); break;
                case 4: launch_rate_bits<4>(codebook, path, sms, warps, iters, cyc, ns, sink, nullptr); break;
                case 5: launch_rate_bits<5>(codebook, path, sms, warps, iters, cyc, ns, sink, nullptr); break;
                case 6: launch_rate_bits<6>(codebook, path, sms, warps, iters, cyc, ns, sink, nullptr); break;
                default: throw std::runtime_error("decode rate: k_bits must be 3, 4, 5 or 6");
            }
        };
        try {
            run();   // warm-up
            run();
            cuda_ok(cudaDeviceSynchronize(), "decode rate sync");
            std::vector<unsigned long long> hc(sms), hn(sms);
            cuda_ok(cudaMemcpy(hc.data(), cyc, size_t(sms) * 8, cudaMemcpyDeviceToHost), "decode rate read");
            cuda_ok(cudaMemcpy(hn.data(), ns, size_t(sms) * 8, cudaMemcpyDeviceToHost), "decode rate read");
            double c = 0, n = 0;
            for (int i = 0; i < sms; ++i) { c += double(hc[i]); n += double(hn[i]); }
            const double weights = double(warps) * 32 * 8 * 8 * iters;   // eight tiles per warp and iteration on both paths
            *weights_per_clk_sm = weights / (c / sms);
            *sm_mhz = n > 0 ? c / n * 1000.0 : 0.0;
        } catch (...) {
            cudaFree(cyc); cudaFree(ns); cudaFree(sink);
            throw;
        }
        cudaFree(cyc); cudaFree(ns); cudaFree(sink);
    });
}

extern "C" int berth_exl3_pipe_probe(int kind, int iters, double* clk_per_iteration_per_scheduler)
{
    using namespace berth;
    return guarded(exl3_state(), [&] {
        if (!clk_per_iteration_per_scheduler) throw std::runtime_error("pipe probe: null result pointer");
        if (kind < 0 || kind > 5 || iters < 1 || iters > (1 << 20)) throw std::runtime_error("pipe probe: kind 0..5, iters 1..2^20");
        const int sms = device_info(current_device()).sms;
        unsigned long long* cyc = nullptr;
        uint32_t* sink = nullptr;
        cuda_ok(cudaMalloc(&cyc, size_t(sms) * 8), "pipe probe alloc");
        cuda_ok(cudaMalloc(&sink, 4), "pipe probe alloc");
        try {
            for (int rep = 0; rep < 2; ++rep) {
                switch (kind) {
                    case 0: k_pipe_probe<0><<<sms, 512>>>(12345u, iters, cyc, sink); break;
                    case 1: k_pipe_probe<1><<<sms, 512>>>(12345u, iters, cyc, sink); break;
                    case 2: k_pipe_probe<2><<<sms, 512>>>(12345u, iters, cyc, sink); break;
                    case 3: k_pipe_probe<3><<<sms, 512>>>(12345u, iters, cyc, sink); break;
                    case 4: k_pipe_probe<4><<<sms, 512>>>(12345u, iters, cyc, sink); break;
                    default: k_pipe_probe<5><<<sms, 512>>>(12345u, iters, cyc, sink); break;
                }
                cuda_ok(cudaGetLastError(), "k_pipe_probe launch");
            }
            cuda_ok(cudaDeviceSynchronize(), "pipe probe sync");
            std::vector<unsigned long long> h(sms);
            cuda_ok(cudaMemcpy(h.data(), cyc, size_t(sms) * 8, cudaMemcpyDeviceToHost), "pipe probe read");
            double c = 0;
            for (int i = 0; i < sms; ++i) c += double(h[i]);
            *clk_per_iteration_per_scheduler = c / sms / iters / 4.0;   // four warps per scheduler run the bundle one after the other
        } catch (...) {
            cudaFree(cyc); cudaFree(sink);
            throw;
        }
        cudaFree(cyc); cudaFree(sink);
    });
}
