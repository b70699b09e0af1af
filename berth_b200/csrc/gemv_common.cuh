// Pieces shared by the decode kernels of the EXL3 linear (gemv.cu: fp16 tensor path for every
// codebook; gemv_i8.cu: MUL1 on the integer tensor path with the weights in tensor memory): the
// unit partition, launch arguments, mbarrier / TMA wrappers with bounded waits, the activation
// rotation, the last steps of an output band, and the finishing kernel's launcher.
#pragma once

#include "exl3_decode.cuh"
#include "silu.cuh"

#include <cuda.h>

namespace berth {

// ---------------------------------------------------------------- partition (host + device)
__host__ __device__ inline long long unit_begin(int c, long long U, int G) { return (long long) c * U / G; }
__host__ __device__ inline int unit_owner(long long u, long long U, int G) { return int(((u + 1) * G + U - 1) / U) - 1; }

// Bits of the status word a bounded wait sets when it runs out: a weight stage never arrived / was never
// released (TMA ring), a tensor-memory stage or accumulator was never handed over (integer tensor path).
enum StatusBits : unsigned { kStFullTimeout = 1u, kStEmptyTimeout = 2u, kStTmemTimeout = 4u };


constexpr int kMaxHetMatrices = 4;

struct GemvArgs {
    const uint32_t* afrag;    // rotated activations in MMA fragment order [problem][k/16][TG][2][8][4] words
    float* blocksum;          // [problem][8*TG or m][k/128]: sum of each rotated 128-block (MUL1 epilogue)
    const __half* a;          // in-kernel rotation only: activations [m][k], input sign-scale [k], and the
    const __half* suh;        //   caller's buffer for the rotated activations [m][k]
    __half* a_had;
    const __half* a_up;       // may be null; else the rotation's input is silu(a) * a_up (rows [m][k]), clamped to +-act_limit
    float act_limit;          //   when that is not 0, every step rounded to fp16 as k_silu_mul rounds it
    void* c;                  // output rows [rows][n]
    unsigned long long* argmax;   // dense launch only, may be null: per row the key of its largest output (finish_band)
    SampleArgs sample;            // how those keys are scored
    int defer_weights;            // no weight fetch before griddepcontrol.wait (berth_exl3_weights_streamed)
    const float* residual;        // dense launch with fp32 output only, may be null: rows [m][n] added to the output (may be c itself)
    const __half* svh;        // [n], or the stack [experts][n] when grouped
    const GemvProblem* problems;   // grouped launch: one entry per (expert, chunk of <= 8*TG rows); else null
    const int* n_problems;         // grouped launch: device-side count
    int max_problems, n_matrices, max_rows;   // bounds the table entries are clamped to
    float* slabs;             // [2*G][m][BU*128]
    unsigned* counters;       // integer tensor path: one arrival counter per band group, zero between launches
    unsigned* status;
    int m, k, n, out_fp32;
    // Sliced multi-linear (several column slices of several matrices applied to one input): device arrays
    // with one entry per slice -- trellis address of the slice's first tile, its output scales, its
    // output address, the full width of the matrix it was cut from (row stride of trellis and output),
    // and which of the rotated inputs it takes.  Null b_list = not sliced.
    const unsigned long long* b_list;
    const unsigned long long* svh_list;
    const unsigned long long* c_list;
    const int* n_stride_list;
    const int* had_src_list;
    int n_slices;
    // Stack of n_stack equally shaped matrices applied to the same rows (integer tensor path only; 0 or 1 = one
    // matrix): matrix i has its trellis at index i of the 3-D map, its sign-scale vectors at suh + i*k and
    // svh + i*n, and writes c + i*m*n, a_had + i*m*k and block sums i*m*(k/128).
    int n_stack;
    // The same for matrices of different widths (q, k and v of an attention block), each with its own tensors
    // (integer tensor path only): het != 0; matrix i owns band groups het_bg[i] .. het_bg[i+1]-1 of the launch, is
    // het_n[i] columns wide, and has its own sign-scale vectors, output and rotated-activation buffer.
    int het;
    int het_bg[kMaxHetMatrices + 1];
    int het_n[kMaxHetMatrices];
    const __half* het_suh[kMaxHetMatrices];
    const __half* het_svh[kMaxHetMatrices];
    void* het_c[kMaxHetMatrices];
    __half* het_a_had[kMaxHetMatrices];
};

// What the roles of the decode kernel need to know about problem pi of a launch.
struct ProblemView {
    int rows, row0, z;       // rows of the problem, first row in the activation / output arrays, matrix of the stack
    int act;                 // which rotated-activation block set and block-sum table it reads
    const __half* svh;       // output scales of the problem's matrix (column 0 of the problem)
    void* c;                 // output base (row 0, column 0 of the problem)
    int ldc;                 // output row stride in elements
};
template <typename Args>
__device__ __forceinline__ ProblemView problem_view(const Args& p, int pi, int tok)
{
    ProblemView v;
    v.rows = p.m; v.row0 = 0; v.z = 0; v.act = 0; v.svh = p.svh; v.c = p.c; v.ldc = p.n;
    if (p.b_list) {
        v.act = __ldg(p.had_src_list + pi);
        v.svh = reinterpret_cast<const __half*>(__ldg(p.svh_list + pi));
        v.c = reinterpret_cast<void*>(__ldg(p.c_list + pi));
        v.ldc = __ldg(p.n_stride_list + pi);
    } else if (p.problems) {
        const GemvProblem pr = load_problem(p.problems, pi, p.n_matrices, tok, p.max_rows);
        v.rows = pr.rows; v.row0 = pr.row0; v.z = pr.z; v.act = pi;
        v.svh = p.svh + size_t(pr.z) * p.n;
    } else if (p.n_stack > 1) {
        v.z = pi; v.act = pi;
        v.svh = p.svh + size_t(pi) * p.n;
        v.c = static_cast<unsigned char*>(p.c) + size_t(pi) * p.m * p.n * (p.out_fp32 ? 4 : 2);
    }
    return v;
}

// ---------------------------------------------------------------- mbarrier / TMA PTX
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
// Bounded waits.  Both give up after roughly half a second, record `code` in the status word and
// return false; the caller carries on with whatever is there.
//   mbar_wait:        for the streaming warps, which expect the data to be there: tight polling;
//   mbar_wait_parked: for the producer, which waits about a microsecond per stage: sleeps between
//                     polls so that it leaves the issue slots to the decoding warps.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned* status, unsigned code)
{
    if (mbar_try_wait(bar, parity)) return true;
    for (uint32_t i = 0; i < (1u << 24); ++i)
        if (mbar_try_wait(bar, parity)) return true;
    atomicOr(status, code);
    return false;
}
__device__ __forceinline__ bool mbar_wait_parked(uint32_t bar, uint32_t parity, unsigned* status, unsigned code)
{
    if (mbar_try_wait(bar, parity)) return true;
    for (uint32_t i = 0; i < (1u << 21); ++i) {
        __nanosleep(200);
        if (mbar_try_wait(bar, parity)) return true;
    }
    atomicOr(status, code);
    return false;
}
// For warps that wait long and have nothing else to do (an MMA issuer waiting for operands, an epilogue waiting
// for an accumulator): try_wait with a suspend-time hint, so that the hardware parks the thread until the phase
// completes (immediate wake-up) instead of the thread polling through the issue slots of the decoding warps.
__device__ __forceinline__ bool mbar_wait_suspended(uint32_t bar, uint32_t parity, unsigned* status, unsigned code)
{
    for (uint32_t i = 0; i < (1u << 16); ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity), "r"(10000u)
            : "memory");
        if (ok) return true;
    }
    atomicOr(status, code);
    return false;
}
// One box of the trellis view (x in 8-byte elements, y in k-tile rows, z = matrix of the stack)
// into shared memory.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
                 : "memory");
}
// Contiguous global -> shared bulk copy (16-byte aligned, size a multiple of 16).
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
// One 128-block of one activation row, whole warp: fp16(H128(x * suh) / sqrt(128)); the lane gets
// elements 4*lane .. 4*lane+3 packed as two half pairs.  SUM: `sx` = sum of the 128 rounded values
// (every lane), which the MUL1 epilogue needs.
template <bool SUM>
__device__ __forceinline__ uint2 rotate_bits(uint2 xr, uint2 sr, int lane, float& sx);

template <bool SUM>
__device__ __forceinline__ uint2 rotate_block(const __half* __restrict__ xrow, const __half* __restrict__ suh, int kb, int lane, float& sx,
                                              const __half* __restrict__ urow = nullptr, float act_limit = 0.f)
{
    const int kcol = kb * 128 + lane * 4;
    uint2 xr = *reinterpret_cast<const uint2*>(xrow + kcol);
    const uint2 sr = *reinterpret_cast<const uint2*>(suh + kcol);
    if (urow) {   // the input is silu(xrow) * urow, rounded as the element-wise kernel rounds it
        const uint2 ur = *reinterpret_cast<const uint2*>(urow + kcol);
        const __half* g = reinterpret_cast<const __half*>(&xr);
        const __half* u = reinterpret_cast<const __half*>(&ur);
        __half o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) o[i] = silu_mul_one(g[i], u[i], act_limit);
        xr.x = dq::pack_half2(o[0], o[1]);
        xr.y = dq::pack_half2(o[2], o[3]);
    }
    return rotate_bits<SUM>(xr, sr, lane, sx);
}

// The same from the lane's four input values and four scales, already loaded.
template <bool SUM>
__device__ __forceinline__ uint2 rotate_bits(uint2 xr, uint2 sr, int lane, float& sx)
{
    __half2 x0 = *reinterpret_cast<__half2*>(&xr.x), x1 = *reinterpret_cast<__half2*>(&xr.y);
    __half2 s0 = *reinterpret_cast<__half2*>(&sr.x), s1 = *reinterpret_cast<__half2*>(&sr.y);
    float v[4];
    v[0] = __fmul_rn(__low2float(x0), __low2float(s0));
    v[1] = __fmul_rn(__high2float(x0), __high2float(s0));
    v[2] = __fmul_rn(__low2float(x1), __low2float(s1));
    v[3] = __fmul_rn(__high2float(x1), __high2float(s1));
    dq::had128_warp(v, lane);
    __half h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __float2half_rn(__fmul_rn(v[i], kRScale));
    uint2 o;
    o.x = dq::pack_half2(h[0], h[1]);
    o.y = dq::pack_half2(h[2], h[3]);
    sx = 0.f;
    if constexpr (SUM) {
        sx = __fadd_rn(__fadd_rn(__half2float(h[0]), __half2float(h[1])), __fadd_rn(__half2float(h[2]), __half2float(h[3])));
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) sx = __fadd_rn(sx, __shfl_xor_sync(dq::kFull, sx, off));
    }
    return o;
}

// Sum over a row's block sums (the MUL1 epilogue's sum of the rotated activations), whole warp.
__device__ __forceinline__ float row_sum(const float* bsum, int kblocks, int lane)
{
    float sx = 0.f;
    for (int b = lane; b < kblocks; b += 32) sx = __fadd_rn(sx, __ldg(bsum + b));
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) sx = __fadd_rn(sx, __shfl_xor_sync(dq::kFull, sx, off));
    return sx;
}

// Last steps of one output band of one row: v = the lane's four fp32 dot products (columns
// band*128 + 4*lane ..).  MUL1: w = S*h + B per weight  =>  sum_k x_k w_k = S*acc + B*sum_k x_k.
// MUL1 = 1: the accumulator holds sum x*(1024 + u) (fp16 tensor path); 2: it holds sum x*u (integer tensor path),
// so the constant term is (1024 S + B) * sum x.
// Natural logarithm of a positive normal float from exact steps only (bit tricks, IEEE add / multiply / divide, fused
// multiply-adds in a fixed order), so that the CPU checker reproduces it bit for bit: x = 2^e * m with m in
// (sqrt(1/2), sqrt(2)], t = (m - 1) / (m + 1), log m = 2 t (1 + t^2/3 + t^4/5 + t^6/7 + t^8/9).
__device__ __forceinline__ float det_log(float x)
{
    const uint32_t bits = __float_as_uint(x);
    int e = int(bits >> 23) - 127;
    float m = __uint_as_float((bits & 0x007fffffu) | 0x3f800000u);
    if (m > 1.41421354f) { m = __fmul_rn(m, 0.5f); e += 1; }
    const float t = __fdiv_rn(__fsub_rn(m, 1.0f), __fadd_rn(m, 1.0f));
    const float t2 = __fmul_rn(t, t);
    float p = __fmaf_rn(t2, 0.111111112f, 0.142857149f);
    p = __fmaf_rn(t2, p, 0.2f);
    p = __fmaf_rn(t2, p, 0.333333343f);
    p = __fmaf_rn(t2, p, 1.0f);
    return __fmaf_rn(__int2float_rn(e), 0.693147182f, __fmul_rn(__fadd_rn(t, t), p));
}
// Standard Gumbel noise of output (row, column) of a launch seeded with `random`: a 32-bit mixing hash of the three,
// its upper 23 bits as u = (k + 1/2) / 2^23 in (0, 1), g = -log(-log(u)).
__device__ __forceinline__ float gumbel_noise(unsigned random, unsigned row, unsigned col)
{
    uint32_t x = random ^ (row * 0x9E3779B9u) ^ (col * 0x85EBCA6Bu);
    x ^= x >> 16; x *= 0x7FEB352Du; x ^= x >> 15; x *= 0x846CA68Bu; x ^= x >> 16;
    const float u = __fmul_rn(__fadd_rn(__uint2float_rn(x >> 9), 0.5f), 1.1920929e-7f);   // 2^-23
    return -det_log(-det_log(u));
}

// The same out of line: the fp16-path kernel finishes whole band groups inside its streaming loop, and the rarely taken
// sampling branch would otherwise sit, four times unrolled, in that loop's instruction footprint (measured on the 6 bpw
// lm_head: 416 -> 411 us); the integer-path kernel measured better with the inline form.
static __device__ __noinline__ float gumbel_noise_call(unsigned random, unsigned row, unsigned col) { return gumbel_noise(random, row, col); }

template <int MUL1>
// `best` (may be null): per output row one 64-bit key, (order-preserving bits of the value) << 32 | ~column, raised
// with atomicMax to the row's largest output: the greedy token of an lm_head without a pass over the logits (ties go
// to the lower column; the value is the one that would be stored, fp16-rounded for fp16 outputs).  `c` may then be null.
// With sample.gumbel the key's value is stored output * inv_temp + Gumbel noise of (row, column) instead: the row's key
// then names one draw from softmax(outputs * inv_temp).
__device__ __forceinline__ void finish_band(float (&v)[4], float sx, int lane, uint2 sr, int band, void* c,
                                            size_t out_row, int n, int out_fp32, unsigned long long* best = nullptr,
                                            const float* residual = nullptr, const SampleArgs sample = SampleArgs{})
{
    const int col = band * 128 + lane * 4;
    if constexpr (MUL1 != 0) {
        const float S1 = __half2float(__ushort_as_half(dq::kMul1S));
        const float B1 = __half2float(__ushort_as_half(dq::kMul1B));
        const float bsx = __fmul_rn(MUL1 == 2 ? __fmaf_rn(1024.0f, S1, B1) : B1, sx);
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = __fmaf_rn(S1, v[i], bsx);
    }
    dq::had128_warp(v, lane);
    uint2 srm = sr;
    __half2 s0 = *reinterpret_cast<__half2*>(&srm.x), s1 = *reinterpret_cast<__half2*>(&srm.y);
    v[0] = __fmul_rn(__fmul_rn(v[0], kRScale), __low2float(s0));
    v[1] = __fmul_rn(__fmul_rn(v[1], kRScale), __high2float(s0));
    v[2] = __fmul_rn(__fmul_rn(v[2], kRScale), __low2float(s1));
    v[3] = __fmul_rn(__fmul_rn(v[3], kRScale), __high2float(s1));
    if (out_fp32) {
        if (residual) {   // c = residual + linear (fp32 outputs only; c may be the residual itself: each element is read, then written, by one thread)
            const float4 r = *reinterpret_cast<const float4*>(residual + out_row * n + col);
            v[0] = __fadd_rn(r.x, v[0]); v[1] = __fadd_rn(r.y, v[1]); v[2] = __fadd_rn(r.z, v[2]); v[3] = __fadd_rn(r.w, v[3]);
        }
        if (c) *reinterpret_cast<float4*>(static_cast<float*>(c) + out_row * n + col) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
        const __half h0 = __float2half_rn(v[0]), h1 = __float2half_rn(v[1]), h2 = __float2half_rn(v[2]), h3 = __float2half_rn(v[3]);
        uint2 o;
        o.x = dq::pack_half2(h0, h1);
        o.y = dq::pack_half2(h2, h3);
        if (c) *reinterpret_cast<uint2*>(static_cast<__half*>(c) + out_row * n + col) = o;
        if (best) { v[0] = __half2float(h0); v[1] = __half2float(h1); v[2] = __half2float(h2); v[3] = __half2float(h3); }
    }
    if (best) {
        unsigned long long key = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float score = v[i];
            if (sample.gumbel) {
                const float g = MUL1 == 2 ? gumbel_noise(sample.random, unsigned(out_row), unsigned(col + i))
                                          : gumbel_noise_call(sample.random, unsigned(out_row), unsigned(col + i));
                score = __fmaf_rn(v[i], sample.inv_temp, g);
            }
            const uint32_t bits = __float_as_uint(__fadd_rn(score, 0.0f));   // (-0 counts as +0, as a comparison of values would)
            const uint32_t ord = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
            const unsigned long long k = (static_cast<unsigned long long>(ord) << 32) | (0xffffffffu - uint32_t(col + i));
            key = k > key ? k : key;
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            const unsigned long long o = __shfl_xor_sync(dq::kFull, key, off);
            key = o > key ? o : key;
        }
        if (lane == 0) atomicMax(best + out_row, key);
    }
}

// One segment (part of one band group) of a CTA's unit range.
struct Segment {
    int bg, kb_begin, units;
    bool head;       // starts at the CTA's first unit (slab 2c) or later (slab 2c+1)
    bool whole;      // covers the band group's whole K: finished in the decode kernel, no slab
};
__device__ __forceinline__ Segment segment_at(long long u, long long u0, long long u1, int kblocks)
{
    Segment s;
    s.bg = int(u / kblocks);
    s.kb_begin = int(u - (long long) s.bg * kblocks);
    const long long left = u1 - u;
    s.units = left < (long long) (kblocks - s.kb_begin) ? int(left) : kblocks - s.kb_begin;
    s.head = (u == u0);
    s.whole = (s.kb_begin == 0 && s.units == kblocks);
    return s;
}

struct FinishArgs {
    const float* slabs;
    const float* blocksum;
    void* c;
    unsigned long long* argmax;
    SampleArgs sample;
    const float* residual;
    const __half* svh;
    const GemvProblem* problems;
    const int* n_problems;
    int max_problems, n_matrices, max_rows;
    int m, k, n, out_fp32, bu, tok, main_grid, mul1;
    const unsigned long long* b_list;      // sliced launch (see GemvArgs), else null
    const unsigned long long* svh_list;
    const unsigned long long* c_list;
    const int* n_stride_list;
    const int* had_src_list;
    int n_slices;
    int n_stack;                           // stack of equally shaped matrices (see GemvArgs), else 0
};


// The finishing kernel behind a decode launch of `main_grid` CTAs (nothing to do behind a single CTA).
// mul1: 0 = no affine correction, 1 = fp16 path (accumulated 1024 + u), 2 = integer path (accumulated u).
void launch_finish(const GemvArgs& a, int bu, int tok, int main_grid, int mul1, cudaStream_t stream);

// 3-D TMA view of a trellis stack: z = matrix, y = k-tile row (K/16), x = the row's (N/16) tiles of
// 32*bits bytes in 8-byte elements; box = box_bytes x 8 rows of one matrix.  Columns past the matrix read as zero.
CUtensorMap trellis_map(const void* trellis, int n_matrices, int size_k, int size_n, int bits, int box_bytes);

}  // namespace berth
