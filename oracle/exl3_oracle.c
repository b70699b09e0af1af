/*
 * CPU oracle for the EXL3 trellis-linear / A3B-MoE path.  Test infrastructure only; see
 * exl3_oracle.h for what may use it and for the "parity unpinned" statement.
 *
 * ------------------------------------------------------------------------------------
 * EXL3 arithmetic, spec v0 (NOT verified against exllamav3 tree de35ffbe...; every item
 * marked [berth] is stated by berth's own sources, every item marked [pub] by the QTIP
 * paper, every item marked [v0] is this build's documented choice)
 * ------------------------------------------------------------------------------------
 * Tensor layout [berth: crates/berth-kernels/src/lib.rs:93-103, src/ops.rs:268-283]
 *   trellis  uint16 [K/16][N/16][16*bits]   one 16x16 weight tile = 16*bits words
 *   suh fp16 [K], svh fp16 [N]; a column band starting at n0 begins (n0/16)*16*bits words
 *   into a k-tile row and keeps the full row stride.
 * Tile bit stream [v0]
 *   The 16*bits words of a tile form a cyclic stream of L = 256*bits bits; stream bit p is
 *   bit (15 - p%16) of word p/16 (most significant bit first).  The trellis is tail-biting
 *   [berth: docs/exl3.md:13]: positions are taken modulo L.
 * States [pub: bitshift trellis, 16-bit state, bits new bits per weight]
 *   state_t = the 16-bit big-endian window of the stream starting at position t*bits,
 *   t = 0..255.  Consecutive states overlap in 16-bits bits.
 * Position of weight t inside the tile [v0, tensor-core fragment order as berth's docs
 *   describe the fork's tiles]
 *   lane = t>>3, j = t&7, g = lane>>2, q = lane&3
 *   col = g + 8*((j>>1)&1),  row = 2*q + (j&1) + 8*(j>>2)
 *   i.e. the eight weights of a lane are the four fp16 pairs of an m16n8k16 operand fragment.
 * Codebooks: state s (16 bit) -> fp16 weight
 *   cb 0 "3INST" [pub, and berth: ptx/sm86_probes.cu:154-159 for the lop3 constants]
 *        x = s*89226354 + 64248484 (mod 2^32); x = (x & 0x8fff8fff) ^ 0x3b603b60;
 *        w = fp16(x[15:0]) + fp16(x[31:16])  (one fp16 add, round to nearest even)
 *   cb 1 "MCG"  [v0 multiplier]  x = s*0xCBAC1FED (mod 2^32); then mask/xor/add as cb 0
 *   cb 2 "MUL1" [berth: ptx/sm86_probes.cu:237-249 for the multiplier; v0 for the rest]
 *        x = s*0x83DCD12D (mod 2^32); u = sum of the four bytes of x (0..1020);
 *        h = the fp16 whose bit pattern is 0x6400 + u, i.e. the value 1024 + u exactly;
 *        w = fp16 fma(h, S, B) with S = 0x1EEE (0.0067673) and B = 0xC931 (-10.3828),
 *        one rounding: the byte sum centred (mean 1534*S = 10.381) and scaled to about
 *        unit variance without any integer-to-float conversion.
 * Hadamard [berth: csrc/prefill_lin/reconstruct.cu:31-67]
 *   Sylvester H_128 in natural order on each contiguous 128 block, fp32 butterflies with
 *   strides 1,2,4,...,64 (lower index gets a+b, upper a-b), then * 0.088388347648f.
 *   Input side: v = fp32(x)*fp32(suh) before the transform, result rounded to fp16 (a_had).
 *   Output side: transform the fp32 accumulators, * r_scale, then * fp32(svh), round to the
 *   output type.
 * Linear [berth: csrc/prefill_lin/linear.cu:201-230]
 *   a_had = H(x*suh); c[m][n] = sum_k fp32(a_had[m][k]) * fp32(W[k][n]) (fp32, ascending k);
 *   y = H(c)*svh.
 * ------------------------------------------------------------------------------------
 */
#include "exl3_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define R_SCALE 0.088388347648f

/* ------------------------------------------------------------------ fp16 helpers */

float exl3o_h2f(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* Round a non-negative finite double magnitude to fp16 bits (no sign), nearest even. */
static uint16_t mag_to_h(double m)
{
    if (m == 0.0) return 0;
    int e;
    double fr = frexp(m, &e); /* m = fr * 2^e, fr in [0.5,1) */
    int exp = e - 1;          /* m = (2fr) * 2^exp, 2fr in [1,2) */
    if (exp > 15) return 0x7c00;
    double scaled;
    if (exp < -14) {
        scaled = ldexp(m, 24); /* subnormal: units of 2^-24 */
        double r = nearbyint(scaled);
        return (uint16_t) r;   /* may carry into the smallest normal, which is correct */
    }
    scaled = ldexp(fr, 11); /* in [1024, 2048) */
    double r = nearbyint(scaled);
    uint32_t mant = (uint32_t) r;
    if (mant == 2048) { mant = 1024; exp++; if (exp > 15) return 0x7c00; }
    return (uint16_t)(((uint32_t)(exp + 15) << 10) | (mant - 1024));
}

uint16_t exl3o_d2h(double d)
{
    uint16_t sign = signbit(d) ? 0x8000u : 0;
    if (isnan(d)) return 0x7e00;
    if (isinf(d)) return sign | 0x7c00;
    return sign | mag_to_h(fabs(d));
}

uint16_t exl3o_f2h(float f) { return exl3o_d2h((double) f); }

/* ------------------------------------------------------------------ format */

void exl3o_unpack_signs(const uint16_t* packed, int64_t n_words, uint16_t* out)
{
    for (int64_t w = 0; w < n_words; ++w)
        for (int b = 0; b < 16; ++b)
            out[w * 16 + b] = ((packed[w] >> b) & 1) ? 0xBC00 : 0x3C00;
}

/* ------------------------------------------------------------------ codebook */

#define MUL1_S 0x1EEE
#define MUL1_B 0xC931

uint16_t exl3o_codebook(uint32_t state, int cb)
{
    state &= 0xffffu;
    if (cb == 2) {
        uint32_t x = state * 0x83DCD12Du;
        int u = (int)(x & 0xff) + (int)((x >> 8) & 0xff) + (int)((x >> 16) & 0xff) + (int)(x >> 24);
        double v = (double) (1024 + u) * (double) exl3o_h2f(MUL1_S) + (double) exl3o_h2f(MUL1_B);
        return exl3o_d2h(v); /* exact product and sum in fp64, one rounding = fp16 fma */
    }
    uint32_t x = (cb == 0) ? state * 89226354u + 64248484u : state * 0xCBAC1FEDu;
    x = (x & 0x8fff8fffu) ^ 0x3b603b60u;
    float lo = exl3o_h2f((uint16_t)(x & 0xffff));
    float hi = exl3o_h2f((uint16_t)(x >> 16));
    return exl3o_f2h(lo + hi); /* both in [0.125,2): the fp32 sum is exact */
}

/* ------------------------------------------------------------------ tile */

void exl3o_tile_states(const uint16_t* words, int bits, uint16_t* states)
{
    const int L = 256 * bits;
    for (int t = 0; t < 256; ++t) {
        uint32_t s = 0;
        int p = t * bits;
        for (int i = 0; i < 16; ++i) {
            int pos = (p + i) % L;
            uint32_t bit = (words[pos >> 4] >> (15 - (pos & 15))) & 1u;
            s = (s << 1) | bit;
        }
        states[t] = (uint16_t) s;
    }
}

void exl3o_tile_coords(int t, int* row, int* col)
{
    int lane = t >> 3, j = t & 7, g = lane >> 2, q = lane & 3;
    *col = g + 8 * ((j >> 1) & 1);
    *row = 2 * q + (j & 1) + 8 * (j >> 2);
}

void exl3o_decode_tile(const uint16_t* words, int bits, int cb, uint16_t* tile)
{
    uint16_t states[256];
    exl3o_tile_states(words, bits, states);
    for (int t = 0; t < 256; ++t) {
        int r, c;
        exl3o_tile_coords(t, &r, &c);
        tile[r * 16 + c] = exl3o_codebook(states[t], cb);
    }
}

void exl3o_reconstruct(const uint16_t* trellis, int size_k, int full_n, int n_offset,
                       int slice_n, int bits, int cb, uint16_t* w, int ldw)
{
    const int tiles_k = size_k / 16, tiles_n = full_n / 16, tw = 16 * bits;
    const int nt0 = n_offset / 16, nt = slice_n / 16;
#pragma omp parallel for collapse(2) schedule(static)
    for (int kt = 0; kt < tiles_k; ++kt)
        for (int j = 0; j < nt; ++j) {
            uint16_t tile[256];
            exl3o_decode_tile(trellis + ((size_t) kt * tiles_n + nt0 + j) * tw, bits, cb, tile);
            for (int r = 0; r < 16; ++r)
                memcpy(w + (size_t)(kt * 16 + r) * ldw + j * 16, tile + r * 16, 32);
        }
}

/* ------------------------------------------------------------------ Hadamard */

static void had128_f32(float* v)
{
    for (int s = 1; s < 128; s <<= 1)
        for (int i = 0; i < 128; ++i)
            if (!(i & s)) {
                float a = v[i], b = v[i | s];
                v[i] = a + b;
                v[i | s] = a - b;
            }
}

static void had128_f64(double* v)
{
    for (int s = 1; s < 128; s <<= 1)
        for (int i = 0; i < 128; ++i)
            if (!(i & s)) {
                double a = v[i], b = v[i | s];
                v[i] = a + b;
                v[i | s] = a - b;
            }
}

void exl3o_had_r_128(const void* in, void* out, const uint16_t* scale, int pre_scale,
                     int rows, int cols, int fp32)
{
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r)
        for (int b = 0; b < cols / 128; ++b) {
            float v[128];
            size_t base = (size_t) r * cols + (size_t) b * 128;
            for (int i = 0; i < 128; ++i) {
                float x = fp32 ? ((const float*) in)[base + i]
                               : exl3o_h2f(((const uint16_t*) in)[base + i]);
                if (pre_scale && scale) x = x * exl3o_h2f(scale[b * 128 + i]);
                v[i] = x;
            }
            had128_f32(v);
            for (int i = 0; i < 128; ++i) {
                float y = v[i] * R_SCALE;
                if (!pre_scale && scale) y = y * exl3o_h2f(scale[b * 128 + i]);
                if (fp32) ((float*) out)[base + i] = y;
                else ((uint16_t*) out)[base + i] = exl3o_f2h(y);
            }
        }
}

/* ------------------------------------------------------------------ linear */

static int linear_shape_ok(int m, int k, int n, int bits, int cb)
{
    return m >= 1 && k >= 128 && n >= 128 && k % 128 == 0 && n % 128 == 0 && bits >= 1 &&
           bits <= 8 && cb >= 0 && cb <= 2;
}

int exl3o_linear(const uint16_t* a, const uint16_t* trellis, void* c, const uint16_t* suh,
                 uint16_t* a_had, const uint16_t* svh, int size_m, int size_k, int size_n,
                 int bits, int cb, int out_fp32)
{
    if (!linear_shape_ok(size_m, size_k, size_n, bits, cb)) return -1;
    uint16_t* ah = a_had ? a_had : (uint16_t*) malloc((size_t) size_m * size_k * 2);
    exl3o_had_r_128(a, ah, suh, 1, size_m, size_k, 0);
    float* ahf = (float*) malloc((size_t) size_m * size_k * sizeof(float));
    for (size_t i = 0; i < (size_t) size_m * size_k; ++i) ahf[i] = exl3o_h2f(ah[i]);

#pragma omp parallel
    {
        uint16_t* wh = (uint16_t*) malloc((size_t) size_k * 128 * 2);
        float* wf = (float*) malloc((size_t) size_k * 128 * sizeof(float));
        float* acc = (float*) malloc((size_t) size_m * 128 * sizeof(float));
#pragma omp for schedule(dynamic, 1)
        for (int nb = 0; nb < size_n / 128; ++nb) {
            /* decode this 128-column band (single-threaded inside the parallel region) */
            const int tiles_n = size_n / 16, tw = 16 * bits;
            for (int kt = 0; kt < size_k / 16; ++kt)
                for (int j = 0; j < 8; ++j) {
                    uint16_t tile[256];
                    exl3o_decode_tile(trellis + ((size_t) kt * tiles_n + nb * 8 + j) * tw, bits, cb, tile);
                    for (int r = 0; r < 16; ++r)
                        memcpy(wh + (size_t)(kt * 16 + r) * 128 + j * 16, tile + r * 16, 32);
                }
            for (size_t i = 0; i < (size_t) size_k * 128; ++i) wf[i] = exl3o_h2f(wh[i]);
            memset(acc, 0, (size_t) size_m * 128 * sizeof(float));
            for (int m = 0; m < size_m; ++m) {
                float* am = acc + (size_t) m * 128;
                const float* xm = ahf + (size_t) m * size_k;
                for (int k = 0; k < size_k; ++k) {
                    const float x = xm[k];
                    const float* wr = wf + (size_t) k * 128;
                    for (int n = 0; n < 128; ++n) am[n] += x * wr[n];
                }
                had128_f32(am);
                for (int n = 0; n < 128; ++n) {
                    float y = am[n] * R_SCALE;
                    y = y * exl3o_h2f(svh[nb * 128 + n]);
                    size_t o = (size_t) m * size_n + (size_t) nb * 128 + n;
                    if (out_fp32) ((float*) c)[o] = y;
                    else ((uint16_t*) c)[o] = exl3o_f2h(y);
                }
            }
        }
        free(wh); free(wf); free(acc);
    }
    free(ahf);
    if (!a_had) free(ah);
    return 0;
}

/* fp64 evaluation of one row band; ah64 = H(x*suh)/sqrt(128) in fp64 [m][k]. */
static void linear_f64_core(const double* ah64, const uint16_t* trellis, double* c,
                            const uint16_t* svh, int size_m, int size_k, int size_n, int bits, int cb)
{
    const double rs = 1.0 / sqrt(128.0);
#pragma omp parallel
    {
        double* wd = (double*) malloc((size_t) size_k * 128 * sizeof(double));
        double* acc = (double*) malloc((size_t) size_m * 128 * sizeof(double));
#pragma omp for schedule(dynamic, 1)
        for (int nb = 0; nb < size_n / 128; ++nb) {
            const int tiles_n = size_n / 16, tw = 16 * bits;
            for (int kt = 0; kt < size_k / 16; ++kt)
                for (int j = 0; j < 8; ++j) {
                    uint16_t tile[256];
                    exl3o_decode_tile(trellis + ((size_t) kt * tiles_n + nb * 8 + j) * tw, bits, cb, tile);
                    for (int r = 0; r < 16; ++r)
                        for (int cc = 0; cc < 16; ++cc)
                            wd[(size_t)(kt * 16 + r) * 128 + j * 16 + cc] = exl3o_h2f(tile[r * 16 + cc]);
                }
            memset(acc, 0, (size_t) size_m * 128 * sizeof(double));
            for (int m = 0; m < size_m; ++m) {
                double* am = acc + (size_t) m * 128;
                const double* xm = ah64 + (size_t) m * size_k;
                for (int k = 0; k < size_k; ++k) {
                    const double x = xm[k];
                    const double* wr = wd + (size_t) k * 128;
                    for (int n = 0; n < 128; ++n) am[n] += x * wr[n];
                }
                had128_f64(am);
                for (int n = 0; n < 128; ++n)
                    c[(size_t) m * size_n + (size_t) nb * 128 + n] =
                        am[n] * rs * (double) exl3o_h2f(svh[nb * 128 + n]);
            }
        }
        free(wd); free(acc);
    }
}

/* x given in fp64 [m][k] (not yet rotated). */
static void linear_f64_from_d(const double* x, const uint16_t* trellis, double* c,
                              const uint16_t* suh, const uint16_t* svh, int size_m, int size_k,
                              int size_n, int bits, int cb)
{
    const double rs = 1.0 / sqrt(128.0);
    double* ah = (double*) malloc((size_t) size_m * size_k * sizeof(double));
    for (int m = 0; m < size_m; ++m)
        for (int b = 0; b < size_k / 128; ++b) {
            double v[128];
            for (int i = 0; i < 128; ++i)
                v[i] = x[(size_t) m * size_k + b * 128 + i] * (double) exl3o_h2f(suh[b * 128 + i]);
            had128_f64(v);
            for (int i = 0; i < 128; ++i) ah[(size_t) m * size_k + b * 128 + i] = v[i] * rs;
        }
    linear_f64_core(ah, trellis, c, svh, size_m, size_k, size_n, bits, cb);
    free(ah);
}

int exl3o_linear_f64(const uint16_t* a, const uint16_t* trellis, double* c, const uint16_t* suh,
                     const uint16_t* svh, int size_m, int size_k, int size_n, int bits, int cb)
{
    if (!linear_shape_ok(size_m, size_k, size_n, bits, cb)) return -1;
    double* x = (double*) malloc((size_t) size_m * size_k * sizeof(double));
    for (size_t i = 0; i < (size_t) size_m * size_k; ++i) x[i] = exl3o_h2f(a[i]);
    linear_f64_from_d(x, trellis, c, suh, svh, size_m, size_k, size_n, bits, cb);
    free(x);
    return 0;
}

/* ------------------------------------------------------------------ silu_mul, add */

/* exp(x) in fp32 from fmaf/mul only, so the same sequence gives the same bits on any IEEE
 * machine; rounding it to fp16 equals the correctly rounded fp16 exp for every fp16 argument
 * except 0x9f79 and 0xa5cf, whose exact results sit within 1e-8 of a rounding midpoint
 * (checked exhaustively by the tests). */
static float exp_f32_det(float x)
{
    if (x > 12.0f) x = 12.0f;   /* fp16 overflows above exp(11.09) */
    if (x < -20.0f) x = -20.0f; /* fp16 underflows below exp(-17.4) */
    float n = rintf(x * 1.44269504088896341f);
    float r = fmaf(n, -0.693145751953125f, x);
    r = fmaf(n, -1.42860682030941723e-6f, r);
    float p = 1.0f / 5040.0f;
    p = fmaf(p, r, 1.0f / 720.0f);
    p = fmaf(p, r, 1.0f / 120.0f);
    p = fmaf(p, r, 1.0f / 24.0f);
    p = fmaf(p, r, 1.0f / 6.0f);
    p = fmaf(p, r, 0.5f);
    p = fmaf(p, r, 1.0f);
    p = fmaf(p, r, 1.0f);
    int32_t e = (int32_t) n;
    uint32_t bits = (uint32_t)(e + 127) << 23;
    float scale;
    memcpy(&scale, &bits, 4);
    return p * scale;
}

uint16_t exl3o_hexp_neg(uint16_t g)
{
    float x = -exl3o_h2f(g);
    if (isnan(x)) return 0x7e00;
    return exl3o_f2h(exp_f32_det(x));
}

static uint16_t silu_mul_one(uint16_t g, uint16_t u, float act_limit)
{
    /* e = h(exp(-g)); d = h(1+e); r = h(1/d); s = h(g*r); out = h(s*u)  (bit-exact against
     * testdata/kernels/ops/silu.out.bin) */
    float e = exl3o_h2f(exl3o_hexp_neg(g));
    float d = exl3o_h2f(exl3o_f2h(1.0f + e));
    float r = exl3o_h2f(exl3o_f2h(1.0f / d));
    float s = exl3o_h2f(exl3o_f2h(exl3o_h2f(g) * r));
    float up = exl3o_h2f(u);
    uint16_t prod = exl3o_f2h(s * up);
    if (act_limit != 0.0f) {
        /* csrc/ops/act.cu: a non-zero limit clamps the product; berth only passes 0 (mlp.rs:22).
         * v0: clamp the rounded product to [-h(limit), +h(limit)]. */
        float lim = exl3o_h2f(exl3o_f2h(fabsf(act_limit)));
        float p = exl3o_h2f(prod);
        if (p > lim) p = lim;
        if (p < -lim) p = -lim;
        prod = exl3o_f2h(p);
    }
    return prod;
}

void exl3o_silu_mul(const uint16_t* gate, const uint16_t* up, uint16_t* out, int64_t numel,
                    float act_limit)
{
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < numel; ++i) out[i] = silu_mul_one(gate[i], up[i], act_limit);
}

/* Scores and keys of the sampling epilogue (berth_exl3_linear_sample; berth: fused sampler modes 0 and 1,
 * crates/berth-kernels/csrc/sample/fused.cu:45-135).  The noise generator is this build's ("spec v0": berth draws
 * from curand's Philox stream inside the fork's kernel): a 32-bit mixing hash of (random, row, column), its upper 23
 * bits as u = (k + 1/2) / 2^23, g = -log(-log(u)) with the logarithm below -- exact steps in a fixed order, every
 * one a correctly rounded fp32 operation, so the device reproduces it bit for bit. */
static float det_log(float x)
{
    union { uint32_t u; float f; } v;
    v.f = x;
    int e = (int) (v.u >> 23) - 127;
    v.u = (v.u & 0x007fffffu) | 0x3f800000u;
    float m = v.f;
    if (m > 1.41421354f) { m = m * 0.5f; e += 1; }
    const float t = (m - 1.0f) / (m + 1.0f);
    const float t2 = t * t;
    float p = fmaf(t2, 0.111111112f, 0.142857149f);
    p = fmaf(t2, p, 0.2f);
    p = fmaf(t2, p, 0.333333343f);
    p = fmaf(t2, p, 1.0f);
    return fmaf((float) e, 0.693147182f, (t + t) * p);
}
static float gumbel_noise(uint32_t random, uint32_t row, uint32_t col)
{
    uint32_t x = random ^ (row * 0x9E3779B9u) ^ (col * 0x85EBCA6Bu);
    x ^= x >> 16; x *= 0x7FEB352Du; x ^= x >> 15; x *= 0x846CA68Bu; x ^= x >> 16;
    const float u = ((float) (x >> 9) + 0.5f) * 1.1920929e-7f;
    return -det_log(-det_log(u));
}
/* keys[r] = the largest of (order-preserving bits of score) << 32 | ~column over the columns of row r, score = the
 * output itself (mode 0) or fmaf(output, inv_temp, noise) (mode 1); outputs fp32 [rows][n] as stored (fp16 outputs
 * converted).  scores (may be NULL) receives every score. */
void exl3o_sample_keys(const float* outputs, int rows, int n, float inv_temp, uint32_t random, int mode, uint64_t* keys,
                       float* scores)
{
    for (int r = 0; r < rows; ++r) {
        uint64_t best = 0;
        for (int c = 0; c < n; ++c) {
            float s = outputs[(size_t) r * n + c];
            if (mode) s = fmaf(s, inv_temp, gumbel_noise(random, (uint32_t) r, (uint32_t) c));
            if (scores) scores[(size_t) r * n + c] = s;
            union { uint32_t u; float f; } v;
            v.f = s + 0.0f;
            const uint32_t ord = (v.u & 0x80000000u) ? ~v.u : (v.u | 0x80000000u);
            const uint64_t k = ((uint64_t) ord << 32) | (uint64_t) (0xffffffffu - (uint32_t) c);
            if (k > best) best = k;
        }
        keys[r] = best;
    }
}

void exl3o_add_f32(const float* a, const float* b, float* c, int64_t n)
{
    for (int64_t i = 0; i < n; ++i) c[i] = a[i] + b[i];
}

/* RMSNorm of berth's decode blocks (crates/berth-kernels/csrc/ops/norm.cu:129-224: berth_ops_rms_norm,
 * _f16, _res_in; semantics of crates/berth-engine/src/model.rs:76-100: epsilon inside the reciprocal square
 * root, constant_bias added to the weight, constant_scale multiplies the normalised row):
 *   y[e] = fp16( ((x[e] * r) * (w[e] + constant_bias)) * constant_scale ),  r = 1 / sqrt(mean(x^2) + epsilon),
 * every step one correctly rounded fp32 operation.  The device kernel of berth lives in the absent fork, so the
 * summation order of mean(x^2) is this build's ("spec v0"): 128 partial sums, partial j taking the groups of
 * four consecutive elements j, j + 128, j + 256, ... in ascending order with fmaf(x, x, s); the 128 partials
 * are added as four groups of 32 by a halving tree (strides 16, 8, 4, 2, 1), the four group sums as
 * (g0 + g1) + (g2 + g3).  x_is_f16: the input row is fp16 (the _f16 entry point), else fp32.
 * weight_bf16: the weight is bfloat16, else fp16.  residual != NULL (RES_IN): residual += x first (fp32, in
 * place), and the row that is normalised is the updated residual. */
static float bf16_to_f32(uint16_t b)
{
    union { uint32_t u; float f; } v;
    v.u = (uint32_t) b << 16;
    return v.f;
}

void exl3o_rms_norm(const void* x, int x_is_f16, const uint16_t* weight, int weight_bf16, uint16_t* y, float* residual,
                    int rows, int dim, float epsilon, float constant_bias, float constant_scale)
{
    for (int r = 0; r < rows; ++r) {
        float part[128];
        for (int j = 0; j < 128; ++j) part[j] = 0.0f;
        float* res = residual ? residual + (size_t) r * dim : NULL;
        for (int e = 0; e < dim; ++e) {
            float v = x_is_f16 ? exl3o_h2f(((const uint16_t*) x)[(size_t) r * dim + e]) : ((const float*) x)[(size_t) r * dim + e];
            if (res) { res[e] = res[e] + v; v = res[e]; }
            const int j = (e / 4) % 128;
            part[j] = fmaf(v, v, part[j]);
        }
        float grp[4];
        for (int g = 0; g < 4; ++g) {
            float t[32];
            for (int i = 0; i < 32; ++i) t[i] = part[32 * g + i];
            for (int off = 16; off >= 1; off >>= 1)
                for (int i = 0; i < off; ++i) t[i] = t[i] + t[i + off];
            grp[g] = t[0];
        }
        const float total = (grp[0] + grp[1]) + (grp[2] + grp[3]);
        const float mean = total / (float) dim;
        const float rinv = 1.0f / sqrtf(mean + epsilon);
        for (int e = 0; e < dim; ++e) {
            const float v = res ? res[e]
                                : (x_is_f16 ? exl3o_h2f(((const uint16_t*) x)[(size_t) r * dim + e]) : ((const float*) x)[(size_t) r * dim + e]);
            const float w = (weight_bf16 ? bf16_to_f32(weight[e]) : exl3o_h2f(weight[e])) + constant_bias;
            y[(size_t) r * dim + e] = exl3o_f2h(((v * rinv) * w) * constant_scale);
        }
    }
}

/* ------------------------------------------------------------------ host integer logic */

int exl3o_gemv_cfg(int cc, int m, int k, int n, int bits, int cb, int mode, int narrow_coresident)
{
    enum { CC_AMPERE = 2, CC_ADA = 3 };
    if (mode == 0) return -1;
    if (bits < 2 || bits > 4) return -1;
    if (bits != 4 && cb == 0) return -1;
    if (m > 8) return -1;
    if (k % 128 || n % 128) return -1;
    if (mode == 2) return n <= 8192 ? 0 : 1;
    if (mode == 3) return 0;
    if (mode == 4) return 1;
    if (bits == 2) return n <= 8192 ? 0 : 1;
    if (bits == 3 && cc == CC_ADA) return n <= 8192 ? 0 : 1;
    if (n / 32 <= narrow_coresident) return 0;
    if (k <= 2048 && n <= 8192) return 0;
    if (bits == 3) return -1;
    if (n >= 8192 && k <= 4096) return 1;
    if (n >= 8192 && n <= 10240 && k <= 5120 && cc == CC_AMPERE) return 1;
    return -1;
}

uint64_t exl3o_gemm_tune_key(int m, int k, int n, int bits, int out_fp32, int device, int cc,
                             int sms, int cb)
{
    if (m < 2) m = 2;
    uint64_t mk;
    if (m <= 16) {
        uint64_t p = 1;
        while (p < (uint64_t) m) p <<= 1;
        mk = p < 16 ? p : 16;
    } else if (m <= 31) mk = 32;
    else if (m <= 63) mk = 64;
    else if (m <= 127) mk = 128;
    else mk = 512;
    uint64_t h = 1469598103934665603ull;
    const uint64_t v[9] = {mk, (uint64_t) k, (uint64_t) n, (uint64_t) bits, out_fp32 ? 1u : 0u,
                           (uint64_t) device, (uint64_t) cc, (uint64_t) sms, (uint64_t) cb};
    for (int i = 0; i < 9; ++i) { h ^= v[i]; h *= 1099511628211ull; }
    return h;
}

/* ------------------------------------------------------------------ MoE */

void exl3o_router_logits(const uint16_t* x, const uint16_t* w_router, const float* bias,
                         float* logits, int T, int H, int E)
{
    const int chunk = H / 32;
#pragma omp parallel for collapse(2) schedule(static)
    for (int t = 0; t < T; ++t)
        for (int e = 0; e < E; ++e) {
            float p[32];
            for (int j = 0; j < 32; ++j) {
                float acc = 0.0f;
                for (int i = 0; i < chunk; ++i) {
                    int h = j * chunk + i;
                    acc = fmaf(exl3o_h2f(x[(size_t) t * H + h]), exl3o_h2f(w_router[(size_t) h * E + e]), acc);
                }
                p[j] = acc;
            }
            for (int off = 16; off >= 1; off >>= 1) {
                float q[32];
                for (int j = 0; j < 32; ++j) q[j] = p[j] + p[j ^ off];
                memcpy(p, q, sizeof p);
            }
            logits[(size_t) t * E + e] = p[0] + (bias ? bias[e] : 0.0f);
        }
}

void exl3o_router_topk(const float* logits, int32_t* topk_idx, float* topk_w, int T, int E, int k)
{
#pragma omp parallel for schedule(static)
    for (int t = 0; t < T; ++t) {
        const float* l = logits + (size_t) t * E;
        int32_t* idx = topk_idx + (size_t) t * k;
        /* selection: k passes, strictly-greater comparison scanning upward = ties to lower index */
        for (int s = 0; s < k; ++s) {
            int best = -1;
            for (int e = 0; e < E; ++e) {
                int taken = 0;
                for (int p = 0; p < s; ++p) taken |= (idx[p] == e);
                if (taken) continue;
                if (best < 0 || l[e] > l[best]) best = e;
            }
            idx[s] = best;
        }
        if (topk_w) {
            /* softmax over the selected logits = full softmax renormalised over the selection */
            float mx = l[idx[0]];
            float ex[64], sum = 0.0f;
            for (int s = 0; s < k; ++s) { ex[s] = expf(l[idx[s]] - mx); sum += ex[s]; }
            for (int s = 0; s < k; ++s) topk_w[(size_t) t * k + s] = ex[s] / sum;
        }
    }
}

static size_t trellis_words(int k, int n, int bits) { return (size_t)(k / 16) * (n / 16) * 16 * bits; }

/* one SiLU-gated expert on one token row; y fp16[hidden] */
static void expert_row(const uint16_t* x, const uint16_t* gt, const uint16_t* ut, const uint16_t* dt,
                       const uint16_t* gsuh, const uint16_t* gsvh, const uint16_t* usuh,
                       const uint16_t* usvh, const uint16_t* dsuh, const uint16_t* dsvh, int hidden,
                       int inter, int bits, int cb, uint16_t* y, int rows)
{
    uint16_t* g = (uint16_t*) malloc((size_t) rows * inter * 2);
    uint16_t* u = (uint16_t*) malloc((size_t) rows * inter * 2);
    exl3o_linear(x, gt, g, gsuh, NULL, gsvh, rows, hidden, inter, bits, cb, 0);
    exl3o_linear(x, ut, u, usuh, NULL, usvh, rows, hidden, inter, bits, cb, 0);
    exl3o_silu_mul(g, u, g, (int64_t) rows * inter, 0.0f);
    exl3o_linear(g, dt, y, dsuh, NULL, dsvh, rows, inter, hidden, bits, cb, 0);
    free(g); free(u);
}

int exl3o_moe_layer(const exl3o_moe_weights* w, const uint16_t* x, int T, float* out,
                    int32_t* topk_idx, float* topk_w)
{
    const int H = w->hidden, I = w->inter, E = w->n_experts, K = w->top_k;
    if (T < 1 || K < 1 || K > 64 || K > E || H % 128 || I % 128) return -1;
    float* logits = (float*) malloc((size_t) T * E * sizeof(float));
    int32_t* idx = topk_idx ? topk_idx : (int32_t*) malloc((size_t) T * K * sizeof(int32_t));
    float* tw = topk_w ? topk_w : (float*) malloc((size_t) T * K * sizeof(float));
    exl3o_router_logits(x, w->w_router, w->router_bias, logits, T, H, E);
    exl3o_router_topk(logits, idx, tw, T, E, K);

    /* per (token, slot) expert output, fp16 */
    uint16_t* y = (uint16_t*) calloc((size_t) T * K * H, 2);
    const size_t gw = trellis_words(H, I, w->bits), dw = trellis_words(I, H, w->bits);
    for (int e = 0; e < E; ++e) {
        int cnt = 0;
        for (int i = 0; i < T * K; ++i) cnt += (idx[i] == e);
        if (!cnt) continue;
        uint16_t* xe = (uint16_t*) malloc((size_t) cnt * H * 2);
        uint16_t* ye = (uint16_t*) malloc((size_t) cnt * H * 2);
        int r = 0;
        for (int i = 0; i < T * K; ++i)
            if (idx[i] == e) memcpy(xe + (size_t)(r++) * H, x + (size_t)(i / K) * H, (size_t) H * 2);
        expert_row(xe, w->gate_trellis + e * gw, w->up_trellis + e * gw, w->down_trellis + e * dw,
                   w->gate_suh + (size_t) e * H, w->gate_svh + (size_t) e * I,
                   w->up_suh + (size_t) e * H, w->up_svh + (size_t) e * I,
                   w->down_suh + (size_t) e * I, w->down_svh + (size_t) e * H, H, I, w->bits,
                   w->cb, ye, cnt);
        r = 0;
        for (int i = 0; i < T * K; ++i)
            if (idx[i] == e) memcpy(y + (size_t) i * H, ye + (size_t)(r++) * H, (size_t) H * 2);
        free(xe); free(ye);
    }
    uint16_t* ysh = NULL;
    if (w->sh_gate_trellis) {
        ysh = (uint16_t*) malloc((size_t) T * H * 2);
        expert_row(x, w->sh_gate_trellis, w->sh_up_trellis, w->sh_down_trellis, w->sh_gate_suh,
                   w->sh_gate_svh, w->sh_up_suh, w->sh_up_svh, w->sh_down_suh, w->sh_down_svh, H,
                   w->shared_inter, w->bits, w->cb, ysh, T);
    }
    for (int t = 0; t < T; ++t)
        for (int h = 0; h < H; ++h) {
            float acc = 0.0f;
            for (int s = 0; s < K; ++s)
                acc = fmaf(tw[(size_t) t * K + s], exl3o_h2f(y[((size_t) t * K + s) * H + h]), acc);
            if (ysh) acc = acc + exl3o_h2f(ysh[(size_t) t * H + h]);
            out[(size_t) t * H + h] = acc;
        }
    free(y); free(ysh); free(logits);
    if (!topk_idx) free(idx);
    if (!topk_w) free(tw);
    return 0;
}

/* SiLU-gated expert in fp64 on `rows` token rows given as fp64. */
static void expert_rows_f64(const double* x, const uint16_t* gt, const uint16_t* ut, const uint16_t* dt,
                            const uint16_t* gsuh, const uint16_t* gsvh, const uint16_t* usuh,
                            const uint16_t* usvh, const uint16_t* dsuh, const uint16_t* dsvh,
                            int hidden, int inter, int bits, int cb, double* y, int rows)
{
    double* g = (double*) malloc((size_t) rows * inter * sizeof(double));
    double* u = (double*) malloc((size_t) rows * inter * sizeof(double));
    linear_f64_from_d(x, gt, g, gsuh, gsvh, rows, hidden, inter, bits, cb);
    linear_f64_from_d(x, ut, u, usuh, usvh, rows, hidden, inter, bits, cb);
    for (size_t i = 0; i < (size_t) rows * inter; ++i) g[i] = g[i] / (1.0 + exp(-g[i])) * u[i];
    linear_f64_from_d(g, dt, y, dsuh, dsvh, rows, inter, hidden, bits, cb);
    free(g); free(u);
}

int exl3o_moe_layer_f64(const exl3o_moe_weights* w, const uint16_t* x, int T,
                        const int32_t* topk_idx, const float* topk_w, double* out)
{
    const int H = w->hidden, I = w->inter, E = w->n_experts, K = w->top_k;
    if (T < 1 || H % 128 || I % 128) return -1;
    const size_t gw = trellis_words(H, I, w->bits), dw = trellis_words(I, H, w->bits);
    double* xd = (double*) malloc((size_t) T * H * sizeof(double));
    for (size_t i = 0; i < (size_t) T * H; ++i) xd[i] = exl3o_h2f(x[i]);
    memset(out, 0, (size_t) T * H * sizeof(double));
    for (int e = 0; e < E; ++e) {
        int cnt = 0;
        for (int i = 0; i < T * K; ++i) cnt += (topk_idx[i] == e);
        if (!cnt) continue;
        double* xe = (double*) malloc((size_t) cnt * H * sizeof(double));
        double* ye = (double*) malloc((size_t) cnt * H * sizeof(double));
        int r = 0;
        for (int i = 0; i < T * K; ++i)
            if (topk_idx[i] == e) memcpy(xe + (size_t)(r++) * H, xd + (size_t)(i / K) * H, (size_t) H * 8);
        expert_rows_f64(xe, w->gate_trellis + e * gw, w->up_trellis + e * gw, w->down_trellis + e * dw,
                        w->gate_suh + (size_t) e * H, w->gate_svh + (size_t) e * I,
                        w->up_suh + (size_t) e * H, w->up_svh + (size_t) e * I,
                        w->down_suh + (size_t) e * I, w->down_svh + (size_t) e * H, H, I, w->bits,
                        w->cb, ye, cnt);
        r = 0;
        for (int i = 0; i < T * K; ++i)
            if (topk_idx[i] == e) {
                const double wt = topk_w[i];
                double* o = out + (size_t)(i / K) * H;
                const double* yr = ye + (size_t)(r++) * H;
                for (int h = 0; h < H; ++h) o[h] += wt * yr[h];
            }
        free(xe); free(ye);
    }
    if (w->sh_gate_trellis) {
        double* ysh = (double*) malloc((size_t) T * H * sizeof(double));
        expert_rows_f64(xd, w->sh_gate_trellis, w->sh_up_trellis, w->sh_down_trellis, w->sh_gate_suh,
                        w->sh_gate_svh, w->sh_up_suh, w->sh_up_svh, w->sh_down_suh, w->sh_down_svh,
                        H, w->shared_inter, w->bits, w->cb, ysh, T);
        for (size_t i = 0; i < (size_t) T * H; ++i) out[i] += ysh[i];
        free(ysh);
    }
    free(xd);
    return 0;
}

int exl3o_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void exl3o_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void) n;
#endif
}
