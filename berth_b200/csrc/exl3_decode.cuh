// Device-side EXL3 decode primitives: trellis window extraction, the three procedural
// codebooks, the 128-wide Hadamard butterfly on a warp, and the m16n8k16 MMA wrapper.
//
// Format (the checker in oracle/exl3_oracle.c states the same rules on the CPU):
//   * a 16x16 tile is 16*BITS uint16 words read most-significant-bit first as one cyclic
//     stream of 256*BITS bits; weight t (0..255) is decoded from the 16-bit window that starts
//     at stream bit t*BITS (tail-biting: positions wrap);
//   * weight t = 8*lane + j sits at col = (lane>>2) + 8*((j>>1)&1),
//     row = 2*(lane&3) + (j&1) + 8*(j>>2): the eight weights of a lane are the four fp16 pairs
//     of an m16n8k16 A fragment of the transposed tile (row index = weight column);
//   * codebook 0 (3INST): x = s*89226354 + 64248484; x = (x & 0x8fff8fff) ^ 0x3b603b60;
//     w = half(x.lo) + half(x.hi);  codebook 1 (MCG): x = s*0xCBAC1FED, same tail;
//     codebook 2 (MUL1): x = s*0x83DCD12D, u = byte sum of x, h = fp16 with bits 0x6400+u
//     (= 1024+u), w = fma(h, S, B) in fp16.
#pragma once

#include "common.cuh"

namespace berth {
namespace dq {

constexpr unsigned kFull = 0xffffffffu;
constexpr unsigned short kMul1S = 0x1EEE;  // 1/147.8
constexpr unsigned short kMul1B = 0xC931;  // -(1024+510)/147.8

__device__ __forceinline__ uint32_t lop3_mask_xor(uint32_t x)
{
    asm("lop3.b32 %0, %0, 0x8fff8fff, 0x3b603b60, 0x6a;" : "+r"(x));
    return x;
}

// The 32-bit word of codebooks 0 and 1 after multiply(+add) and mask/xor: two fp16 halves whose
// sum is the weight.
template <int CB>
__device__ __forceinline__ uint32_t mix32(uint32_t s)
{
    static_assert(CB == 0 || CB == 1, "mix32 is defined for the 3INST and MCG codebooks");
    uint32_t x = (CB == 0) ? s * 89226354u + 64248484u : s * 0xCBAC1FEDu;
    return lop3_mask_xor(x);
}

// fp16 bit pattern of 1024 + (byte sum of the MUL1 product): 0x6400 is 1024.0 with a unit in the
// last place of 1, so adding the sum (0..1020) to the pattern adds it to the value.
__device__ __forceinline__ uint32_t mul1_h1024(uint32_t s)
{
    return __dp4a(s * 0x83DCD12Du, 0x01010101u, 0x6400u);
}

// One state -> one fp16 weight, bit-exact with the specification.
template <int CB>
__device__ __forceinline__ __half decode(uint32_t s)
{
    if constexpr (CB == 2) {
        return __hfma(__ushort_as_half((unsigned short) mul1_h1024(s)), __ushort_as_half(kMul1S), __ushort_as_half(kMul1B));
    } else {
        uint32_t x = mix32<CB>(s);
        __half2 h = *reinterpret_cast<__half2*>(&x);
        return __hadd(__low2half(h), __high2half(h));
    }
}

__device__ __forceinline__ uint32_t pack_half2(__half lo, __half hi)
{
    __half2 h = __halves2half2(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Number of 32-bit words a lane needs to cover its eight windows (7*BITS+16 bits after a start
// offset of up to 24 bits).
template <int BITS>
struct LaneWords {
    static constexpr int rmax = (BITS % 4 == 0) ? 0 : ((BITS % 2 == 0) ? 16 : 24);
    static constexpr int value = (rmax + 7 * BITS + 16 + 31) / 32;
};

// Raw (little-endian uint16 pair) word -> stream order (first uint16 in the high half).
__device__ __forceinline__ uint32_t stream_order(uint32_t raw) { return __byte_perm(raw, 0, 0x1032); }

// Index of the first raw 32-bit word of the lane's span inside the tile, and the residual
// left shift (a multiple of 8 below 32).
template <int BITS>
__device__ __forceinline__ void lane_span(int lane, int& word, int& shift)
{
    int bitpos = 8 * lane * BITS;
    word = bitpos >> 5;
    shift = bitpos & 31;
}

// Eight 16-bit states from the lane's stream-ordered words a0,a1,a2 (a2 ignored when the span
// fits two words) already shifted so that the lane's first window starts at bit 31 of a0.
template <int BITS>
__device__ __forceinline__ void states_aligned(uint32_t a0, uint32_t a1, uint32_t a2, uint32_t (&s)[8])
{
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int p = j * BITS;
        const int wi = p >> 5, sh = p & 31;
        uint32_t hi = wi == 0 ? a0 : (wi == 1 ? a1 : a2);
        uint32_t lo = wi == 0 ? a1 : (wi == 1 ? a2 : 0u);
        s[j] = __funnelshift_l(lo, hi, sh) >> 16;
    }
}

// Loads the lane's words from a tile (global or shared pointer to its 8*BITS raw words), with
// the tail-biting wrap, and returns the eight states.
template <int BITS>
__device__ __forceinline__ void lane_states(const uint32_t* tile, int lane, uint32_t (&s)[8])
{
    constexpr int NW = 8 * BITS;
    constexpr int NL = LaneWords<BITS>::value;
    int w, r;
    lane_span<BITS>(lane, w, r);
    int w1 = w + 1; if (w1 >= NW) w1 -= NW;
    uint32_t a0 = stream_order(tile[w]);
    uint32_t a1 = stream_order(tile[w1]);
    uint32_t a2 = 0;
    if constexpr (NL > 2) {
        int w2 = w1 + 1; if (w2 >= NW) w2 -= NW;
        a2 = stream_order(tile[w2]);
    }
    if constexpr (BITS % 4 != 0) {
        a0 = __funnelshift_l(a1, a0, r);
        a1 = __funnelshift_l(a2, a1, r);
        a2 = a2 << r;
    }
    states_aligned<BITS>(a0, a1, a2, s);
}

// Same from raw words already in registers (the order lane_states would load them in).
template <int BITS>
__device__ __forceinline__ void lane_states_regs(uint32_t r0, uint32_t r1, uint32_t r2, int lane, uint32_t (&s)[8])
{
    int w, r;
    lane_span<BITS>(lane, w, r);
    uint32_t a0 = stream_order(r0), a1 = stream_order(r1), a2 = stream_order(r2);
    if constexpr (BITS % 4 != 0) {
        a0 = __funnelshift_l(a1, a0, r);
        a1 = __funnelshift_l(a2, a1, r);
        a2 = a2 << r;
    }
    states_aligned<BITS>(a0, a1, a2, s);
}

// Half-word selection on the FMA-heavy pipe: dp2a.lo(a, b) = a.h0*b.byte0 + a.h1*b.byte1.
__device__ __forceinline__ uint32_t lo16_heavy(uint32_t a)
{
    uint32_t d;
    asm("dp2a.lo.u32.u32 %0, %1, 0x0001, 0;" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ uint32_t hi16_heavy(uint32_t a)
{
    uint32_t d;
    asm("dp2a.lo.u32.u32 %0, %1, 0x0100, 0;" : "=r"(d) : "r"(a));
    return d;
}

// 4-bit tiles: eight 16-bit windows from the lane's raw word r0 and the next lane's r1
// (13 integer operations).  Stream bytes in order: r0.b1 r0.b0 r0.b3 r0.b2 r1.b1 r1.b0.
// HEAVY = how many of the six half-word selections go to the FMA-heavy pipe (0, 2, 4 or 6), for
// balancing the two integer pipes against the arithmetic of the codebook that follows.
template <int HEAVY>
__device__ __forceinline__ void states_4bit(uint32_t r0, uint32_t r1, uint32_t (&s)[8])
{
    static_assert(HEAVY == 0 || HEAVY == 2 || HEAVY == 4 || HEAVY == 6, "number of selections on the FMA-heavy pipe");
    s[2] = __byte_perm(r0, 0u, 0x4403);
    const uint32_t z = r1 & 0xff00u;
    s[6] = __byte_perm(r0, z, 0x4425);
    const uint32_t a0 = __byte_perm(r0, 0u, 0x1032), a1 = __byte_perm(r1, 0u, 0x1032);
    const uint32_t c4 = __funnelshift_l(a1, a0, 4), c12 = __funnelshift_l(a1, a0, 12);
    if constexpr (HEAVY >= 2) { s[0] = lo16_heavy(r0); s[4] = hi16_heavy(r0); }
    else { s[0] = r0 & 0xffffu; s[4] = r0 >> 16; }
    if constexpr (HEAVY >= 4) { s[1] = hi16_heavy(c4); s[5] = lo16_heavy(c4); }
    else { s[1] = c4 >> 16; s[5] = c4 & 0xffffu; }
    if constexpr (HEAVY >= 6) { s[3] = hi16_heavy(c12); s[7] = lo16_heavy(c12); }
    else { s[3] = c12 >> 16; s[7] = c12 & 0xffffu; }
}

// Eight states -> the four packed fp16 pairs (j=0,1), (2,3), (4,5), (6,7): the A fragment
// a0..a3 of mma.m16n8k16 for the transposed tile.
template <int CB>
__device__ __forceinline__ void decode_frag(const uint32_t (&s)[8], uint32_t (&a)[4])
{
    if constexpr (CB == 2) {
        // pack the two 16-bit patterns of 1024 + byte sum first, then one half2 fma per pair (the same
        // per-element arithmetic as decode<2>, half the instructions)
        const uint32_t sc = uint32_t(kMul1S) | (uint32_t(kMul1S) << 16), bi = uint32_t(kMul1B) | (uint32_t(kMul1B) << 16);
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const uint32_t h = __byte_perm(mul1_h1024(s[2 * r]), mul1_h1024(s[2 * r + 1]), 0x5410);
            const __half2 w = __hfma2(*reinterpret_cast<const __half2*>(&h), *reinterpret_cast<const __half2*>(&sc),
                                      *reinterpret_cast<const __half2*>(&bi));
            a[r] = *reinterpret_cast<const uint32_t*>(&w);
        }
    } else {
        // 3INST / MCG: the weight is the sum of the two halves of the mixed word; add the words of two weights pairwise
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const uint32_t x0 = mix32<CB>(s[2 * r]), x1 = mix32<CB>(s[2 * r + 1]);
            const uint32_t lo = __byte_perm(x0, x1, 0x5410), hi = __byte_perm(x0, x1, 0x7632);   // (lo0, lo1), (hi0, hi1)
            const __half2 w = __hadd2(*reinterpret_cast<const __half2*>(&lo), *reinterpret_cast<const __half2*>(&hi));
            a[r] = *reinterpret_cast<const uint32_t*>(&w);
        }
    }
}

// D(16x8, fp32) += A(16x16, fp16, row) * B(16x8, fp16, col)
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// ---------------------------------------------------------------- per-tile decode + MMA (decode GEMV, fp16 path)
template <int BITS, int CB>
__device__ __forceinline__ void tile_states(const uint32_t* tile, int lane, int lane1, uint32_t (&s)[8])
{
    // the codebooks whose arithmetic leans on the ALU pipe take their half-word selections on the FMA-heavy pipe
    if constexpr (BITS == 4) states_4bit<(CB != 2) ? 6 : 0>(tile[lane], tile[lane1], s);
    else lane_states<BITS>(tile, lane, s);
}

// Duplicated activation pairs for the lo/hi-as-k-slots scheme: from b0 = (x[2q], x[2q+1]) and
// b1 = (x[2q+8], x[2q+9]) make (x,x) pairs.
struct DupFrag { uint32_t e0, e1, o0, o1; };
__device__ __forceinline__ DupFrag dup_pairs(uint32_t b0, uint32_t b1)
{
    DupFrag d;
    d.e0 = __byte_perm(b0, 0u, 0x1010);  // (x[2q],   x[2q])
    d.o0 = __byte_perm(b0, 0u, 0x3232);  // (x[2q+1], x[2q+1])
    d.e1 = __byte_perm(b1, 0u, 0x1010);  // (x[2q+8], x[2q+8])
    d.o1 = __byte_perm(b1, 0u, 0x3232);  // (x[2q+9], x[2q+9])
    return d;
}

// Activation operand of one k-tile row: raw pairs for MUL1, duplicated pairs otherwise.
template <int CB, int TG>
struct RowFrag {
    uint32_t b0[TG], b1[TG];
    DupFrag dup[TG];
    // `act` = the k-tile row's block in shared memory: [TG][2][32 lanes] words, lane = 4*token + q
    __device__ __forceinline__ void load(const uint32_t* act, int lane)
    {
#pragma unroll
        for (int tg = 0; tg < TG; ++tg) {
            b0[tg] = act[tg * 64 + lane];
            b1[tg] = act[tg * 64 + 32 + lane];
            if constexpr (CB != 2) dup[tg] = dup_pairs(b0[tg], b1[tg]);
        }
    }
};

template <int CB, int TG>
__device__ __forceinline__ void tile_mma(const uint32_t (&s)[8], float (&acc)[TG][4], const RowFrag<CB, TG>& f)
{
    if constexpr (CB == 2) {
        uint32_t h[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) h[j] = mul1_h1024(s[j]);
        uint32_t a[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) a[r] = __byte_perm(h[2 * r], h[2 * r + 1], 0x5410);
#pragma unroll
        for (int tg = 0; tg < TG; ++tg) mma_16816(acc[tg], a, f.b0[tg], f.b1[tg]);
    } else {
        uint32_t w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) w[j] = mix32<CB>(s[j]);
        const uint32_t ae[4] = {w[0], w[2], w[4], w[6]};   // rows 2q, 2q+8 of columns g, g+8
        const uint32_t ao[4] = {w[1], w[3], w[5], w[7]};   // rows 2q+1, 2q+9
#pragma unroll
        for (int tg = 0; tg < TG; ++tg) {
            mma_16816(acc[tg], ae, f.dup[tg].e0, f.dup[tg].e1);
            mma_16816(acc[tg], ao, f.dup[tg].o0, f.dup[tg].o1);
        }
    }
}

// ---------------------------------------------------------------- MUL1 on the integer tensor path
// For the MUL1 codebook a weight is S*(1024 + u) + B with u = the byte sum of x = s*0x83DCD12D, so
// sum_k a_k w_k = S * sum_k a_k u_k + (1024 S + B) * sum_k a_k.  The register x IS four u8 k-slots of
// an m16n8k32 integer MMA: against the activation replicated over the four slots the tensor core
// forms a_k * (b0 + b1 + b2 + b3) by itself, so the decode is window extraction plus ONE multiply
// per weight -- no byte sum, no pair packing.  The activations enter as 16-bit block fixed point
// (two signed 8-bit limbs, value = 256*hi + lo, one fp32 scale per rotated 128-block); the limbs of
// a token are two of the eight columns of B, so one MMA pair per tile serves four tokens.  The
// integer accumulation is exact; the only error is the 16-bit rounding of the rotated activation
// (relative 2^-16 of the block maximum, below fp16's own rounding of the same value).
//
// D(16x8, s32) += A(16x32, u8, row) * B(32x8, s8, col)
__device__ __forceinline__ void mma_16832_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// States of a tile for the integer path: the multiply is the only FMA-heavy work per weight, so
// four of the six half-word selections of a 4-bit tile move there (9 ALU : 12 FMA-heavy per 8 weights; measured best).
#ifndef BERTH_I8_HEAVY
#define BERTH_I8_HEAVY 4
#endif
template <int BITS>
__device__ __forceinline__ void tile_states_i8(const uint32_t* tile, int lane, int lane1, uint32_t (&s)[8])
{
    if constexpr (BITS == 4) states_4bit<BERTH_I8_HEAVY>(tile[lane], tile[lane1], s);
    else lane_states<BITS>(tile, lane, s);
}

// One 16x16 tile against NG groups of four tokens.  Lane 4g+q holds the weights of output columns
// g, g+8 at k-rows 2q, 2q+1, 2q+8, 2q+9 (s[0..7] in the order of the tile format); b[ng] = the lane's
// four B words of the k-tile row: the limb of column g (token g/2 of the group, limb g%2: 0 = high)
// at those four k-rows, each replicated over the four bytes.  acc[ng] = (col g, token q high),
// (col g, token q low), (col g+8, high), (col g+8, low).
template <int NG>
__device__ __forceinline__ void tile_mma_i8(const uint32_t (&s)[8], int (&acc)[NG][4], const uint4 (&b)[NG])
{
    uint32_t x[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = s[j] * 0x83DCD12Du;
#pragma unroll
    for (int ng = 0; ng < NG; ++ng) {
        mma_16832_u8s8(acc[ng], x[0], x[2], x[1], x[3], b[ng].x, b[ng].y);
        mma_16832_u8s8(acc[ng], x[4], x[6], x[5], x[7], b[ng].z, b[ng].w);
    }
}

// Unnormalised 128-point Sylvester-Hadamard transform across a warp; lane L holds elements
// 4L..4L+3.  Strides 1,2 in registers, 4..64 by shuffles; lower index gets a+b, upper a-b, so
// every output equals the sequential butterfly of the checker bit for bit.
__device__ __forceinline__ void had128_warp(float (&v)[4], int lane)
{
    float a = __fadd_rn(v[0], v[1]), b = __fsub_rn(v[0], v[1]);
    float c = __fadd_rn(v[2], v[3]), d = __fsub_rn(v[2], v[3]);
    v[0] = __fadd_rn(a, c); v[2] = __fsub_rn(a, c);
    v[1] = __fadd_rn(b, d); v[3] = __fsub_rn(b, d);
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float o = __shfl_xor_sync(kFull, v[i], off);
            v[i] = (lane & off) ? __fsub_rn(o, v[i]) : __fadd_rn(v[i], o);
        }
    }
}

}  // namespace dq
}  // namespace berth
