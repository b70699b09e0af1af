// Bandwidth-bound helpers of the EXL3 path: trellis -> fp16 weight reconstruction, the
// standalone 128-wide Hadamard, silu(gate)*up and the fp32 residual add.
#include "exl3_decode.cuh"
#include "silu.cuh"
#include "../../include/berth_b200.h"

#include <algorithm>

namespace berth {
namespace {

// ---------------------------------------------------------------- reconstruct
// One CTA = one k-tile row of one 128-column band: 8 warps decode one 16x16 tile each into a
// [16][128] shared tile, then the CTA writes sixteen 256-byte rows.
// Algorithmic bytes per weight: BITS/8 read + 2 written.
template <int BITS, int CB>
__global__ void __launch_bounds__(256) k_trellis_decode(__half* __restrict__ out, const uint32_t* __restrict__ trellis,
                                                        int tiles_n_full, int tile_n0, int slice_n)
{
    __shared__ __align__(16) __half tile[16][128 + 8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kt = blockIdx.y, band = blockIdx.x;
    const uint32_t* src = trellis + (size_t(kt) * tiles_n_full + tile_n0 + band * 8 + warp) * (8 * BITS);
    uint32_t s[8];
    dq::lane_states<BITS>(src, lane, s);
    const int g = lane >> 2, q = lane & 3;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int col = g + 8 * ((j >> 1) & 1);
        const int row = 2 * q + (j & 1) + 8 * (j >> 2);
        tile[row][warp * 16 + col] = dq::decode<CB>(s[j]);
    }
    __syncthreads();
    // 16 rows x 128 halves = 16 x 16 uint4
    const int row = threadIdx.x >> 4, seg = threadIdx.x & 15;
    uint4 v = *reinterpret_cast<const uint4*>(&tile[row][seg * 8]);
    *reinterpret_cast<uint4*>(out + (size_t(kt) * 16 + row) * slice_n + band * 128 + seg * 8) = v;
}

template <int BITS>
void launch_decode_cb(int cb, dim3 grid, cudaStream_t st, __half* out, const uint32_t* t, int tnf, int tn0, int sn)
{
    switch (cb) {
        case 0: k_trellis_decode<BITS, 0><<<grid, 256, 0, st>>>(out, t, tnf, tn0, sn); break;
        case 1: k_trellis_decode<BITS, 1><<<grid, 256, 0, st>>>(out, t, tnf, tn0, sn); break;
        default: k_trellis_decode<BITS, 2><<<grid, 256, 0, st>>>(out, t, tnf, tn0, sn); break;
    }
}

void check_div(int value, int by, const char* what)
{
    if (value % by != 0)
        throw std::runtime_error(std::string("prefill reconstruct: ") + what + " must be a multiple of " + std::to_string(by));
}

// ---------------------------------------------------------------- had_r_128
// One warp per (row, 128-block); lane holds 4 consecutive elements.  4 or 8 bytes per element.
template <bool FP32, bool PRE>
__global__ void __launch_bounds__(128) k_had128(const void* __restrict__ in, void* __restrict__ out,
                                                const __half* __restrict__ scale, int rows, int blocks_per_row)
{
    pdl_trigger();
    pdl_wait();   // the input may be the output of the predecessor on the stream
    const int lane = threadIdx.x & 31;
    const long long total = (long long) rows * blocks_per_row;
    for (long long idx = (long long) blockIdx.x * 4 + (threadIdx.x >> 5); idx < total; idx += (long long) gridDim.x * 4) {
        const int b = int(idx % blocks_per_row);
        const size_t base = size_t(idx) * 128 + lane * 4;
        float v[4], sc[4] = {1.f, 1.f, 1.f, 1.f};
        if (scale) {
            uint2 raw = *reinterpret_cast<const uint2*>(scale + b * 128 + lane * 4);
            __half2 s0 = *reinterpret_cast<__half2*>(&raw.x), s1 = *reinterpret_cast<__half2*>(&raw.y);
            sc[0] = __low2float(s0); sc[1] = __high2float(s0); sc[2] = __low2float(s1); sc[3] = __high2float(s1);
        }
        if constexpr (FP32) {
            float4 x = *reinterpret_cast<const float4*>(static_cast<const float*>(in) + base);
            v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
        } else {
            uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const __half*>(in) + base);
            __half2 x0 = *reinterpret_cast<__half2*>(&raw.x), x1 = *reinterpret_cast<__half2*>(&raw.y);
            v[0] = __low2float(x0); v[1] = __high2float(x0); v[2] = __low2float(x1); v[3] = __high2float(x1);
        }
        if constexpr (PRE) {
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] = __fmul_rn(v[i], sc[i]);
        }
        dq::had128_warp(v, lane);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[i] = __fmul_rn(v[i], kRScale);
            if constexpr (!PRE) v[i] = __fmul_rn(v[i], sc[i]);
        }
        if constexpr (FP32) {
            *reinterpret_cast<float4*>(static_cast<float*>(out) + base) = make_float4(v[0], v[1], v[2], v[3]);
        } else {
            uint2 o;
            o.x = dq::pack_half2(__float2half_rn(v[0]), __float2half_rn(v[1]));
            o.y = dq::pack_half2(__float2half_rn(v[2]), __float2half_rn(v[3]));
            *reinterpret_cast<uint2*>(static_cast<__half*>(out) + base) = o;
        }
    }
}

// ---------------------------------------------------------------- silu_mul
__global__ void __launch_bounds__(256) k_silu_mul(const __half2* gate, const __half2* up,
                                                  __half2* out, long long pairs, float limit)
{
    pdl_trigger();
    pdl_wait();
    for (long long i = (long long) blockIdx.x * 256 + threadIdx.x; i < pairs; i += (long long) gridDim.x * 256) {
        __half2 g = gate[i], u = up[i];
        out[i] = __halves2half2(silu_mul_one(__low2half(g), __low2half(u), limit),
                                silu_mul_one(__high2half(g), __high2half(u), limit));
    }
}

// The same over the first *n_rows rows of `row_pairs` half pairs each (row count known on the device only).
__global__ void __launch_bounds__(256) k_silu_mul_rows(const __half2* gate, const __half2* up, __half2* out,
                                                       const int* __restrict__ n_rows, int max_rows, int row_pairs, float limit)
{
    const long long pairs = (long long) min(max(__ldg(n_rows), 0), max_rows) * row_pairs;
    for (long long i = (long long) blockIdx.x * 256 + threadIdx.x; i < pairs; i += (long long) gridDim.x * 256) {
        __half2 g = gate[i], u = up[i];
        out[i] = __halves2half2(silu_mul_one(__low2half(g), __low2half(u), limit),
                                silu_mul_one(__high2half(g), __high2half(u), limit));
    }
}

__global__ void __launch_bounds__(256) k_add_f32(const float* a, const float* b, float* c, int n)
{
    pdl_trigger();
    pdl_wait();
    int i = blockIdx.x * 256 + threadIdx.x;
    if (i < n) c[i] = __fadd_rn(a[i], b[i]);
}

// RMSNorm of one row per block (128 threads): y = fp16(((v * r) * (w + bias)) * scale), r = 1 / sqrt(mean(v^2) + eps),
// v = x, or with RES_IN the residual row after residual += x (written back).  The sum of squares is taken in a fixed
// order -- thread j folds the groups of four elements j, j + 128, ... with fmaf, the 128 partial sums are added by a
// halving tree inside each warp and as (w0 + w1) + (w2 + w3) across the four warps -- and every other step is one
// correctly rounded fp32 operation, so the rows equal the CPU checker's bit for bit.
template <bool X_F16, bool W_BF16, bool RES_IN>
__global__ void __launch_bounds__(128) k_rms_norm(const void* __restrict__ x_, const uint16_t* __restrict__ w, __half* __restrict__ y,
                                                  float* __restrict__ residual, int dim, float eps, float bias, float scale)
{
    pdl_trigger();
    pdl_wait();
    const size_t row = blockIdx.x;
    const int j = threadIdx.x, lane = j & 31, warp = j >> 5, chunks = dim >> 2;
    auto load4 = [&](int c) {
        float4 v;
        if constexpr (X_F16) {
            const uint2 h = *reinterpret_cast<const uint2*>(static_cast<const __half*>(x_) + row * dim + 4 * c);
            const __half2 a = *reinterpret_cast<const __half2*>(&h.x), b = *reinterpret_cast<const __half2*>(&h.y);
            v = make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
        } else {
            v = *reinterpret_cast<const float4*>(static_cast<const float*>(x_) + row * dim + 4 * c);
        }
        return v;
    };
    float s = 0.f;
    for (int c = j; c < chunks; c += 128) {
        float4 v = load4(c);
        if constexpr (RES_IN) {
            float4* rp = reinterpret_cast<float4*>(residual + row * dim + 4 * c);
            const float4 r = *rp;
            v = make_float4(__fadd_rn(r.x, v.x), __fadd_rn(r.y, v.y), __fadd_rn(r.z, v.z), __fadd_rn(r.w, v.w));
            *rp = v;
        }
        s = __fmaf_rn(v.x, v.x, s); s = __fmaf_rn(v.y, v.y, s); s = __fmaf_rn(v.z, v.z, s); s = __fmaf_rn(v.w, v.w, s);
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, off));
    __shared__ float ws[4];
    if (lane == 0) ws[warp] = s;
    __syncthreads();
    const float total = __fadd_rn(__fadd_rn(ws[0], ws[1]), __fadd_rn(ws[2], ws[3]));
    const float rinv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, float(dim)), eps)));
    for (int c = j; c < chunks; c += 128) {
        float4 v;
        if constexpr (RES_IN) v = *reinterpret_cast<const float4*>(residual + row * dim + 4 * c);   // this thread's own stores
        else v = load4(c);
        const uint2 wr = *reinterpret_cast<const uint2*>(w + 4 * c);
        float wf[4];
        if constexpr (W_BF16) {
            wf[0] = __uint_as_float(wr.x << 16); wf[1] = __uint_as_float(wr.x & 0xffff0000u);
            wf[2] = __uint_as_float(wr.y << 16); wf[3] = __uint_as_float(wr.y & 0xffff0000u);
        } else {
            const __half2 a = *reinterpret_cast<const __half2*>(&wr.x), b = *reinterpret_cast<const __half2*>(&wr.y);
            wf[0] = __low2float(a); wf[1] = __high2float(a); wf[2] = __low2float(b); wf[3] = __high2float(b);
        }
        const float in[4] = {v.x, v.y, v.z, v.w};
        __half o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
            o[i] = __float2half_rn(__fmul_rn(__fmul_rn(__fmul_rn(in[i], rinv), __fadd_rn(wf[i], bias)), scale));
        uint2 st;
        st.x = dq::pack_half2(o[0], o[1]);
        st.y = dq::pack_half2(o[2], o[3]);
        *reinterpret_cast<uint2*>(y + row * dim + 4 * c) = st;
    }
}

// Host checks of crates/berth-kernels/csrc/ops/norm.cu:107-127 (berth), same wording.
void check_rms(const void* x, const void* w, const void* y, const void* r, int rows, int dim, bool res_in, int weight_bf16)
{
    if (!x || !w || !y) throw std::runtime_error("rms_norm: null device pointer");
    if (res_in && !r) throw std::runtime_error("rms_norm: RES_IN requires a residual pointer");
    if (rows < 1 || dim < 1) throw std::runtime_error("rms_norm: rows and dim must be positive");
    if (dim % 4 != 0) throw std::runtime_error("rms_norm: dim must be a multiple of 4");
    if (weight_bf16 != 0 && weight_bf16 != 1) throw std::runtime_error("rms_norm: weight_bf16 must be 0 or 1");
}

template <bool X_F16, bool W_BF16, bool RES_IN>
std::string launch_rms(const void* x, const void* w, void* y, void* r, int rows, int dim, float eps, float bias, float scale, cudaStream_t st)
{
    launch_pdl(k_rms_norm<X_F16, W_BF16, RES_IN>, dim3(rows), dim3(128), 0, st, "rms_norm launch", x, static_cast<const uint16_t*>(w),
               static_cast<__half*>(y), static_cast<float*>(r), dim, eps, bias, scale);
    return std::string("k_rms_norm<") + (X_F16 ? "half" : "float") + "," + (W_BF16 ? "bfloat16" : "half") + (RES_IN ? ",res_in" : "") +
           "> block=128 grid=" + std::to_string(rows);
}

}  // namespace

// SiLU(gate) * up over the first *n_rows rows (device-side count, at most max_rows) of row_elems fp16 each.
void silu_mul_rows(const void* gate, const void* up, void* out, const int* n_rows, int max_rows, int row_elems, cudaStream_t stream)
{
    const long long pairs = (long long) max_rows * (row_elems / 2);
    const int grid = int(std::max<long long>(1, std::min<long long>((pairs + 255) / 256, 148LL * 8)));
    k_silu_mul_rows<<<grid, 256, 0, stream>>>((const __half2*) gate, (const __half2*) up, (__half2*) out, n_rows, max_rows, row_elems / 2, 0.0f);
    cuda_ok(cudaGetLastError(), "silu_mul_rows launch");
}

// Internal C++ entry points (shared with the prefill path).
void reconstruct(void* unpacked, const void* packed, int size_k, int slice_n, int full_n, int n_offset,
                 int k_bits, int codebook, cudaStream_t stream)
{
    check_div(size_k, 16, "K");
    check_div(slice_n, 128, "slice N");
    check_div(full_n, 16, "full N");
    check_div(n_offset, 128, "n_offset");
    if (n_offset < 0 || n_offset + slice_n > full_n)
        throw std::runtime_error("prefill reconstruct: slice exceeds the trellis");
    dim3 grid(slice_n / 128, size_k / 16);
    __half* out = static_cast<__half*>(unpacked);
    const uint32_t* t = static_cast<const uint32_t*>(packed);
    const int tnf = full_n / 16, tn0 = n_offset / 16;
    switch (k_bits) {
        case 1: launch_decode_cb<1>(codebook, grid, stream, out, t, tnf, tn0, slice_n); break;
        case 2: launch_decode_cb<2>(codebook, grid, stream, out, t, tnf, tn0, slice_n); break;
        case 3: launch_decode_cb<3>(codebook, grid, stream, out, t, tnf, tn0, slice_n); break;
        case 4: launch_decode_cb<4>(codebook, grid, stream, out, t, tnf, tn0, slice_n); break;
        case 5: launch_decode_cb<5>(codebook, grid, stream, out, t, tnf, tn0, slice_n); break;
        case 6: launch_decode_cb<6>(codebook, grid, stream, out, t, tnf, tn0, slice_n); break;
        case 7: launch_decode_cb<7>(codebook, grid, stream, out, t, tnf, tn0, slice_n); break;
        case 8: launch_decode_cb<8>(codebook, grid, stream, out, t, tnf, tn0, slice_n); break;
        default: throw std::runtime_error("prefill reconstruct: K must be in 1..=8");
    }
    cuda_ok(cudaPeekAtLastError(), "k_trellis_decode");
}

void had_r_128(const void* input, void* output, const void* scale, int pre_scale, int rows, int cols, int fp32,
               cudaStream_t stream)
{
    if (cols % 128 != 0) throw std::runtime_error("prefill had_r_128: had columns must be a multiple of 128");
    if (rows < 1) throw std::runtime_error("prefill had_r_128: rows must be positive");
    const int bpr = cols / 128;
    long long total = (long long) rows * bpr;
    int grid = int(std::min<long long>((total + 3) / 4, 148LL * 16));
    const __half* sc = static_cast<const __half*>(scale);
    if (fp32) {
        if (pre_scale) launch_pdl(k_had128<true, true>, dim3(grid), dim3(128), 0, stream, "k_had128", input, output, sc, rows, bpr);
        else launch_pdl(k_had128<true, false>, dim3(grid), dim3(128), 0, stream, "k_had128", input, output, sc, rows, bpr);
    } else {
        if (pre_scale) launch_pdl(k_had128<false, true>, dim3(grid), dim3(128), 0, stream, "k_had128", input, output, sc, rows, bpr);
        else launch_pdl(k_had128<false, false>, dim3(grid), dim3(128), 0, stream, "k_had128", input, output, sc, rows, bpr);
    }
}

}  // namespace berth

using namespace berth;

extern "C" int berth_prefill_reconstruct(void* unpacked, const void* packed, int size_k, int slice_n, int full_n,
                                         int n_offset, int k_bits, int codebook, void* stream)
{
    CallState& st = prefill_state();
    return guarded(st, [&] {
        if (!unpacked || !packed) throw std::runtime_error("prefill reconstruct: null device pointer");
        if (size_k < 1 || slice_n < 1 || full_n < 1) throw std::runtime_error("prefill reconstruct: sizes must be positive");
        if (codebook < 0 || codebook > 2) throw std::runtime_error("prefill reconstruct: codebook must be 0, 1, or 2");
        reconstruct(unpacked, packed, size_k, slice_n, full_n, n_offset, k_bits, codebook, (cudaStream_t) stream);
        st.launch = "k_trellis_decode<" + std::to_string(k_bits) + "," + std::to_string(codebook) + "> block=256 grid=" +
                    std::to_string(slice_n / 128) + "x" + std::to_string(size_k / 16);
    });
}

extern "C" int berth_prefill_had_r_128(const void* input, void* output, const void* scale, int pre_scale, int rows,
                                       int cols, int fp32, void* stream)
{
    CallState& st = prefill_state();
    return guarded(st, [&] {
        if (!input || !output) throw std::runtime_error("prefill had_r_128: null device pointer");
        had_r_128(input, output, scale, pre_scale, rows, cols, fp32, (cudaStream_t) stream);
        st.launch = std::string("k_had128<") + (fp32 ? "f32" : "f16") + (pre_scale ? ",pre" : ",post") + "> block=128";
    });
}

extern "C" int berth_ops_silu_mul(const void* gate, const void* up, void* out, int64_t numel, float act_limit,
                                  void* stream)
{
    CallState& st = ops_state();
    return guarded(st, [&] {
        if (!gate || !up || !out) throw std::runtime_error("silu_mul: null device pointer");
        if (numel < 2 || (numel & 1)) throw std::runtime_error("silu_mul: numel must be positive and even");
        long long pairs = numel / 2;
        int grid = int(std::min<long long>((pairs + 255) / 256, 148LL * 8));
        launch_pdl(k_silu_mul, dim3(grid), dim3(256), 0, (cudaStream_t) stream, "silu_mul launch", (const __half2*) gate,
                   (const __half2*) up, (__half2*) out, pairs, act_limit);
        st.launch = "k_silu_mul block=256 grid=" + std::to_string(grid);
    });
}

extern "C" int berth_ops_add_f32(const void* a, const void* b, void* c, int n, void* stream)
{
    CallState& st = ops_state();
    return guarded(st, [&] {
        if (!a || !b || !c) throw std::runtime_error("add_f32: null device pointer");
        if (n < 1) throw std::runtime_error("add_f32: n must be positive");
        int grid = (n + 255) / 256;
        launch_pdl(k_add_f32, dim3(grid), dim3(256), 0, (cudaStream_t) stream, "add_f32 launch", (const float*) a,
                   (const float*) b, (float*) c, n);
        st.launch = "k_add_f32 block=256 grid=" + std::to_string(grid);
    });
}

// RMSNorm of berth's decode blocks: crates/berth-kernels/csrc/ops/norm.cu:129-224 (same symbols, arguments, checks).
extern "C" int berth_ops_rms_norm(const void* x, const void* weight, void* y, int rows, int dim, float epsilon, float constant_bias,
                                  float constant_scale, int weight_bf16, void* stream)
{
    CallState& st = ops_state();
    return guarded(st, [&] {
        check_rms(x, weight, y, nullptr, rows, dim, false, weight_bf16);
        cudaStream_t cs = (cudaStream_t) stream;
        st.launch = weight_bf16 ? launch_rms<false, true, false>(x, weight, y, nullptr, rows, dim, epsilon, constant_bias, constant_scale, cs)
                                : launch_rms<false, false, false>(x, weight, y, nullptr, rows, dim, epsilon, constant_bias, constant_scale, cs);
    });
}

extern "C" int berth_ops_rms_norm_f16(const void* x, const void* weight, void* y, int rows, int dim, float epsilon, float constant_bias,
                                      float constant_scale, void* stream)
{
    CallState& st = ops_state();
    return guarded(st, [&] {
        check_rms(x, weight, y, nullptr, rows, dim, false, 1);
        st.launch = launch_rms<true, true, false>(x, weight, y, nullptr, rows, dim, epsilon, constant_bias, constant_scale, (cudaStream_t) stream);
    });
}

extern "C" int berth_ops_rms_norm_res_in(const void* x, const void* weight, void* y, void* residual, int rows, int dim, float epsilon,
                                         float constant_bias, float constant_scale, int weight_bf16, void* stream)
{
    CallState& st = ops_state();
    return guarded(st, [&] {
        check_rms(x, weight, y, residual, rows, dim, true, weight_bf16);
        cudaStream_t cs = (cudaStream_t) stream;
        st.launch = weight_bf16 ? launch_rms<false, true, true>(x, weight, y, residual, rows, dim, epsilon, constant_bias, constant_scale, cs)
                                : launch_rms<false, false, true>(x, weight, y, residual, rows, dim, epsilon, constant_bias, constant_scale, cs);
    });
}
