// Fused EXL3 decode GEMV (size_m <= 32): input Hadamard, trellis decode in registers, tensor-core
// accumulate, split-K reduction by the last CTA to arrive, output Hadamard -- one launch.
//
// Work decomposition: grid = (N/128 column bands, KSPLIT).  A CTA of 8 warps owns one band over
// a contiguous range of 128-row blocks; warp w owns the tile column w of the band (16 columns)
// for every k-tile of the range, so no cross-warp reduction is needed: each warp reads one
// 16*BITS*2-byte tile per k-tile (eight warps together read one contiguous 8-tile run), decodes
// its eight weights per lane into an m16n8k16 A fragment (transposed tile: rows = weight
// columns) and multiplies by the rotated activations held in shared memory (B fragment, 8
// tokens per MMA).  Partial sums go to a per-split slab of the workspace; the CTA that arrives
// last on the band's counter adds the slabs in split order (deterministic), applies the output
// Hadamard and the svh sign-scale and writes C.
//
// Roofline: HBM.  Algorithmic bytes per launch = K*N*BITS/8 + 2K + 2N + 2MK + out_bytes*M*N.
#include "exl3_decode.cuh"
#include "../../include/berth_b200.h"

#include <algorithm>
#include <mutex>

namespace berth {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kPrefetch = 8;  // k-tiles in flight per warp

struct GemvArgs {
    const __half* a;
    const uint32_t* trellis;
    void* c;
    const __half* suh;
    __half* a_had;
    const __half* svh;
    float* ws;
    unsigned* counters;
    int m, k, n;
    int out_fp32;
    int kb_per_split;  // 128-row blocks per split
    int ksplit;
    int chunk_kb;      // 128-row blocks whose rotated activations fit in shared memory at once
};

template <int MG>
struct Smem {
    // rotated activations [8*MG][chunk_k + 8] fp16, then the band's partial sums [8*MG][132] fp32
    static __host__ __device__ int ah_stride(int chunk_k) { return chunk_k + 8; }
    static __host__ __device__ size_t bytes(int chunk_k)
    {
        return size_t(8 * MG) * ah_stride(chunk_k) * sizeof(__half) + size_t(8 * MG) * 132 * sizeof(float);
    }
};

template <int BITS, int CB, int MG>
__global__ void __launch_bounds__(kThreads) k_exl3_gemv(const GemvArgs p)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int NW = 8 * BITS;                     // raw 32-bit words per tile
    constexpr int NL = dq::LaneWords<BITS>::value;   // words a lane needs per tile
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int band = blockIdx.x, split = blockIdx.y;
    const int kblocks = p.k >> 7;
    const int kb0 = split * p.kb_per_split;
    const int kb1 = min(kb0 + p.kb_per_split, kblocks);
    const int chunk_k = p.chunk_kb * 128;
    const int ahs = Smem<MG>::ah_stride(chunk_k);
    __half* ah = reinterpret_cast<__half*>(smem_raw);
    float* outbuf = reinterpret_cast<float*>(smem_raw + size_t(8 * MG) * ahs * sizeof(__half));
    const uint32_t* ah32 = reinterpret_cast<const uint32_t*>(ah);
    const int ahs32 = ahs >> 1;
    const int tiles_n = p.n >> 4;
    const int g = lane >> 2, q = lane & 3;

    int lw, lr;
    dq::lane_span<BITS>(lane, lw, lr);
    int lw1 = lw + 1; if (lw1 >= NW) lw1 -= NW;
    int lw2 = lw1 + 1; if (lw2 >= NW) lw2 -= NW;

    float acc[MG][4];
#pragma unroll
    for (int i = 0; i < MG; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }

    for (int kb = kb0; kb < kb1; kb += p.chunk_kb) {
        const int nkb = min(p.chunk_kb, kb1 - kb);
        __syncthreads();  // the previous chunk's readers are done with `ah`
        // ---- rotated activations of this chunk: one warp per (token row, 128-block)
        for (int idx = warp; idx < 8 * MG * nkb; idx += kWarps) {
            const int row = idx / nkb, b = idx - row * nkb;
            const int kcol = (kb + b) * 128 + lane * 4;
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (row < p.m) {
                uint2 xr = *reinterpret_cast<const uint2*>(p.a + size_t(row) * p.k + kcol);
                uint2 sr = *reinterpret_cast<const uint2*>(p.suh + kcol);
                __half2 x0 = *reinterpret_cast<__half2*>(&xr.x), x1 = *reinterpret_cast<__half2*>(&xr.y);
                __half2 s0 = *reinterpret_cast<__half2*>(&sr.x), s1 = *reinterpret_cast<__half2*>(&sr.y);
                v[0] = __fmul_rn(__low2float(x0), __low2float(s0));
                v[1] = __fmul_rn(__high2float(x0), __high2float(s0));
                v[2] = __fmul_rn(__low2float(x1), __low2float(s1));
                v[3] = __fmul_rn(__high2float(x1), __high2float(s1));
                dq::had128_warp(v, lane);
            }
            uint2 o;
            o.x = dq::pack_half2(__float2half_rn(__fmul_rn(v[0], kRScale)), __float2half_rn(__fmul_rn(v[1], kRScale)));
            o.y = dq::pack_half2(__float2half_rn(__fmul_rn(v[2], kRScale)), __float2half_rn(__fmul_rn(v[3], kRScale)));
            *reinterpret_cast<uint2*>(ah + size_t(row) * ahs + b * 128 + lane * 4) = o;
            if (band == 0 && row < p.m) *reinterpret_cast<uint2*>(p.a_had + size_t(row) * p.k + kcol) = o;
        }
        __syncthreads();

        // ---- main loop: this warp's tile column over the chunk's k-tiles
        const int nkt = nkb * 8;
        const uint32_t* tp = p.trellis + (size_t(kb) * 8 * tiles_n + band * 8 + warp) * NW;
        const size_t tstride = size_t(tiles_n) * NW;  // words between consecutive k-tiles
        uint32_t buf[kPrefetch][NL];
#pragma unroll
        for (int i = 0; i < kPrefetch; ++i) {
            if (i < nkt) {
                const uint32_t* t = tp + i * tstride;
                buf[i][0] = __ldcs(t + lw);
                if constexpr (BITS != 4) buf[i][1] = __ldcs(t + lw1);
                if constexpr (NL > 2) buf[i][2] = __ldcs(t + lw2);
            }
        }
        for (int kt0 = 0; kt0 < nkt; kt0 += kPrefetch) {
#pragma unroll
            for (int i = 0; i < kPrefetch; ++i) {
                const int kt = kt0 + i;
                if (kt < nkt) {
                    uint32_t r0 = buf[i][0], r1, r2 = 0;
                    if constexpr (BITS == 4) r1 = __shfl_sync(dq::kFull, r0, (lane + 1) & 31);
                    else r1 = buf[i][1];
                    if constexpr (NL > 2) r2 = buf[i][2];
                    // refill this slot with the tile kPrefetch k-tiles ahead
                    if (kt + kPrefetch < nkt) {
                        const uint32_t* t = tp + size_t(kt + kPrefetch) * tstride;
                        buf[i][0] = __ldcs(t + lw);
                        if constexpr (BITS != 4) buf[i][1] = __ldcs(t + lw1);
                        if constexpr (NL > 2) buf[i][2] = __ldcs(t + lw2);
                    }
                    uint32_t s[8], af[4];
                    dq::lane_states_regs<BITS>(r0, r1, r2, lane, s);
                    dq::decode_frag<CB>(s, af);
                    const int kw = kt * 8 + q;  // 32-bit word of (k = 16*kt + 2q) in a row of `ah`
#pragma unroll
                    for (int mg = 0; mg < MG; ++mg) {
                        const uint32_t b0 = ah32[(mg * 8 + g) * ahs32 + kw];
                        const uint32_t b1 = ah32[(mg * 8 + g) * ahs32 + kw + 4];
                        dq::mma_16816(acc[mg], af, b0, b1);
                    }
                }
            }
        }
    }

    // ---- band partial sums to shared memory: D[n][tok], n = 16*warp + {g, g+8}, tok = 8*mg + {2q, 2q+1}
#pragma unroll
    for (int mg = 0; mg < MG; ++mg) {
        const int t0 = mg * 8 + 2 * q, c0 = warp * 16 + g;
        outbuf[t0 * 132 + c0] = acc[mg][0];
        outbuf[(t0 + 1) * 132 + c0] = acc[mg][1];
        outbuf[t0 * 132 + c0 + 8] = acc[mg][2];
        outbuf[(t0 + 1) * 132 + c0 + 8] = acc[mg][3];
    }
    __syncthreads();

    if (p.ksplit > 1) {
        // slab [split][m][n]; 32 lanes x float4 = one 128-column row
        for (int row = warp; row < p.m; row += kWarps) {
            float4 v = *reinterpret_cast<const float4*>(outbuf + row * 132 + lane * 4);
            __stcg(reinterpret_cast<float4*>(p.ws + (size_t(split) * p.m + row) * p.n + band * 128 + lane * 4), v);
        }
        __threadfence();
        __syncthreads();
        __shared__ unsigned s_last;
        if (threadIdx.x == 0) s_last = (atomicAdd(p.counters + band, 1u) == unsigned(p.ksplit - 1));
        __syncthreads();
        if (!s_last) return;
        __threadfence();
    }

    // ---- epilogue (last CTA of the band): sum the slabs in split order, rotate, scale, store
    for (int row = warp; row < p.m; row += kWarps) {
        float v[4];
        if (p.ksplit > 1) {
            v[0] = v[1] = v[2] = v[3] = 0.f;
            for (int s = 0; s < p.ksplit; ++s) {
                float4 t = __ldcg(reinterpret_cast<const float4*>(p.ws + (size_t(s) * p.m + row) * p.n + band * 128 + lane * 4));
                v[0] = __fadd_rn(v[0], t.x); v[1] = __fadd_rn(v[1], t.y);
                v[2] = __fadd_rn(v[2], t.z); v[3] = __fadd_rn(v[3], t.w);
            }
        } else {
            float4 t = *reinterpret_cast<const float4*>(outbuf + row * 132 + lane * 4);
            v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
        }
        dq::had128_warp(v, lane);
        const int col = band * 128 + lane * 4;
        uint2 sr = *reinterpret_cast<const uint2*>(p.svh + col);
        __half2 s0 = *reinterpret_cast<__half2*>(&sr.x), s1 = *reinterpret_cast<__half2*>(&sr.y);
        v[0] = __fmul_rn(__fmul_rn(v[0], kRScale), __low2float(s0));
        v[1] = __fmul_rn(__fmul_rn(v[1], kRScale), __high2float(s0));
        v[2] = __fmul_rn(__fmul_rn(v[2], kRScale), __low2float(s1));
        v[3] = __fmul_rn(__fmul_rn(v[3], kRScale), __high2float(s1));
        if (p.out_fp32) {
            *reinterpret_cast<float4*>(static_cast<float*>(p.c) + size_t(row) * p.n + col) = make_float4(v[0], v[1], v[2], v[3]);
        } else {
            uint2 o;
            o.x = dq::pack_half2(__float2half_rn(v[0]), __float2half_rn(v[1]));
            o.y = dq::pack_half2(__float2half_rn(v[2]), __float2half_rn(v[3]));
            *reinterpret_cast<uint2*>(static_cast<__half*>(p.c) + size_t(row) * p.n + col) = o;
        }
    }
    if (p.ksplit > 1 && threadIdx.x == 0) p.counters[band] = 0;  // self-resetting for the next launch
}

template <int BITS, int CB, int MG>
void launch_one(const GemvArgs& args, dim3 grid, size_t smem, cudaStream_t stream)
{
    auto kern = k_exl3_gemv<BITS, CB, MG>;
    static thread_local bool attr_set[kMaxDevices] = {};
    int dev = current_device();
    if (!attr_set[dev]) {
        cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024), "gemv smem attribute");
        attr_set[dev] = true;
    }
    kern<<<grid, kThreads, smem, stream>>>(args);
}

template <int BITS, int CB>
void launch_mg(int mg, const GemvArgs& a, dim3 grid, size_t smem, cudaStream_t st)
{
    switch (mg) {
        case 1: launch_one<BITS, CB, 1>(a, grid, smem, st); break;
        case 2: launch_one<BITS, CB, 2>(a, grid, smem, st); break;
        default: launch_one<BITS, CB, 4>(a, grid, smem, st); break;
    }
}

template <int BITS>
void launch_cb(int cb, int mg, const GemvArgs& a, dim3 grid, size_t smem, cudaStream_t st)
{
    switch (cb) {
        case 0: launch_mg<BITS, 0>(mg, a, grid, smem, st); break;
        case 1: launch_mg<BITS, 1>(mg, a, grid, smem, st); break;
        default: launch_mg<BITS, 2>(mg, a, grid, smem, st); break;
    }
}

}  // namespace

// Shared-memory budget for the rotated activations: 8*MG rows x chunk_k fp16 <= 32 KiB.
static int max_chunk_kb(int mg) { return 2048 / 128 / mg; }

// Launches the decode GEMV.  `ws`/`counters` = split-K scratch (the library's per-device
// workspace, or a caller-provided region of `ws_bytes` bytes and `n/128` zeroed counters).
std::string launch_gemv(const void* a, const void* trellis, void* c, const void* suh, void* a_had, const void* svh,
                        int size_m, int size_k, int size_n, int k_bits, int codebook, int out_fp32, float* ws,
                        size_t ws_bytes, unsigned* counters, int sms, cudaStream_t stream)
{
    if (size_m > 32) throw std::runtime_error("exl3 gemv: size_m must be <= 32");
    if (size_k % 128 != 0)
        throw std::runtime_error("exl3 linear: no linked kernel for size_k that is not a multiple of 128 (128-wide Hadamard)");
    if (k_bits < 1 || k_bits > 8) throw std::runtime_error("exl3 linear: K must be in 1..=8");
    const int mg = size_m <= 8 ? 1 : (size_m <= 16 ? 2 : 4);
    const int bands = size_n / 128, kblocks = size_k / 128;
    if (bands > kGemvMaxBands) throw std::runtime_error("exl3 gemv: size_n exceeds the band counter table");

    // Split K until about four CTAs per SM exist, each keeping at least two 128-row blocks.
    const int target = sms * 4;
    int want = std::max(1, (target + bands - 1) / bands);
    want = std::min(want, std::max(1, kblocks / 2));
    int kbps = (kblocks + want - 1) / want;
    int ksplit = (kblocks + kbps - 1) / kbps;
    while (ksplit > 1 && size_t(ksplit) * size_m * size_n * sizeof(float) > ws_bytes) {
        ++kbps;
        ksplit = (kblocks + kbps - 1) / kbps;
    }
    const int chunk_kb = std::min(kbps, max_chunk_kb(mg));

    GemvArgs args;
    args.a = static_cast<const __half*>(a);
    args.trellis = static_cast<const uint32_t*>(trellis);
    args.c = c;
    args.suh = static_cast<const __half*>(suh);
    args.a_had = static_cast<__half*>(a_had);
    args.svh = static_cast<const __half*>(svh);
    args.ws = ws;
    args.counters = counters;
    args.m = size_m; args.k = size_k; args.n = size_n;
    args.out_fp32 = out_fp32;
    args.kb_per_split = kbps;
    args.ksplit = ksplit;
    args.chunk_kb = chunk_kb;
    dim3 grid(bands, ksplit);
    const size_t smem = size_t(8 * mg) * (chunk_kb * 128 + 8) * sizeof(__half) + size_t(8 * mg) * 132 * sizeof(float);
    switch (k_bits) {
        case 1: launch_cb<1>(codebook, mg, args, grid, smem, stream); break;
        case 2: launch_cb<2>(codebook, mg, args, grid, smem, stream); break;
        case 3: launch_cb<3>(codebook, mg, args, grid, smem, stream); break;
        case 4: launch_cb<4>(codebook, mg, args, grid, smem, stream); break;
        case 5: launch_cb<5>(codebook, mg, args, grid, smem, stream); break;
        case 6: launch_cb<6>(codebook, mg, args, grid, smem, stream); break;
        case 7: launch_cb<7>(codebook, mg, args, grid, smem, stream); break;
        default: launch_cb<8>(codebook, mg, args, grid, smem, stream); break;
    }
    cuda_ok(cudaGetLastError(), "k_exl3_gemv launch");
    return "k_exl3_gemv<" + std::to_string(k_bits) + "," + std::to_string(codebook) + "," + std::to_string(mg) + "> grid=" +
           std::to_string(bands) + "x" + std::to_string(ksplit) + " block=" + std::to_string(kThreads) +
           " smem=" + std::to_string(smem);
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
// The scratch is one file-scope __device__ array: kStaticPartialBytes of fp32 partial sums plus
// one arrival counter per 128-column band.  Every GPU that loads the library carries it until
// the process exits.  All calls on a device share it and it keeps whatever the previous call
// left behind: the counters are cleared on the stream before each launch, the partial sums are
// fully overwritten before they are read.  Two calls that overlap on the GPU (different
// streams) race on it; issue them on one stream.
namespace berth {
namespace {

constexpr size_t kStaticPartialBytes = size_t(4) << 20;   // 4 MiB of split-K partial sums
constexpr int kStaticMaxBands = 1024;                     // size_n <= 131072
constexpr int kStaticMaxRows = 32;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticPartialBytes + kStaticMaxBands * sizeof(unsigned)];

struct StaticScratch {
    float* partial = nullptr;
    unsigned* counters = nullptr;
};
StaticScratch g_static_ptr[kMaxDevices];
std::mutex g_static_mu;

// The array's name is only a host-side handle; the device address has to be asked for, once
// per device, while that device is current.
StaticScratch static_scratch(int device)
{
    std::lock_guard<std::mutex> lock(g_static_mu);
    StaticScratch& s = g_static_ptr[device];
    if (!s.partial) {
        void* base = nullptr;
        cuda_ok(cudaGetSymbolAddress(&base, g_static_scratch), "cudaGetSymbolAddress(static scratch)");
        if (!base) throw std::runtime_error("exl3 linear (static scratch): symbol address is null");
        s.partial = static_cast<float*>(base);
        s.counters = reinterpret_cast<unsigned*>(static_cast<unsigned char*>(base) + kStaticPartialBytes);
    }
    return s;
}

}  // namespace
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
        const int device = current_device();
        const DeviceInfo& info = device_info(device);
        if (info.major != 10)
            throw std::runtime_error("exl3 linear: no linked kernel for this GPU (library is built for sm_100a only)");
        StaticScratch s = static_scratch(device);
        cudaStream_t cs = (cudaStream_t) stream;
        // Arrival counters must start at zero; the partial sums need no clearing.
        cuda_ok(cudaMemsetAsync(s.counters, 0, size_t(size_n / 128) * sizeof(unsigned), cs), "static scratch counter reset");
        st.launch = launch_gemv(a, trellis, c, suh, a_had, svh, size_m, size_k, size_n, k_bits, codebook, out_fp32,
                                s.partial, kStaticPartialBytes, s.counters, info.sms, cs) + " static-scratch";
    });
}

