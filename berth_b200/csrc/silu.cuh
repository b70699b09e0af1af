// silu(gate) * up on fp16 values, every step rounded as the CPU checker rounds it (shared by the
// element-wise kernel and by the rotation kernel that applies it on the fly).
#pragma once

#include "common.cuh"

namespace berth {

// exp(x) from fmaf/mul only: the same operation sequence as the CPU checker, hence the same
// bits.  x is clamped to the range where fp16 neither overflows nor underflows.
__device__ __forceinline__ float exp_f32_det(float x)
{
    x = fminf(x, 12.0f);
    x = fmaxf(x, -20.0f);
    float n = rintf(__fmul_rn(x, 1.44269504088896341f));
    float r = __fmaf_rn(n, -0.693145751953125f, x);
    r = __fmaf_rn(n, -1.42860682030941723e-6f, r);
    float p = 1.0f / 5040.0f;
    p = __fmaf_rn(p, r, 1.0f / 720.0f);
    p = __fmaf_rn(p, r, 1.0f / 120.0f);
    p = __fmaf_rn(p, r, 1.0f / 24.0f);
    p = __fmaf_rn(p, r, 1.0f / 6.0f);
    p = __fmaf_rn(p, r, 0.5f);
    p = __fmaf_rn(p, r, 1.0f);
    p = __fmaf_rn(p, r, 1.0f);
    return __fmul_rn(p, __int_as_float((int(n) + 127) << 23));
}

// e = h(exp(-g)); d = h(1+e); r = h(1/d); s = h(g*r); out = h(s*u): every step rounded to fp16,
// which reproduces berth's silu.out.bin fixture bit for bit.
__device__ __forceinline__ __half silu_mul_one(__half g, __half u, float limit)
{
    const float gf = __half2float(g);
    __half e = (gf != gf) ? __ushort_as_half(0x7e00) : __float2half_rn(exp_f32_det(-gf));
    __half d = __float2half_rn(__fadd_rn(1.0f, __half2float(e)));
    __half r = __float2half_rn(__fdiv_rn(1.0f, __half2float(d)));
    __half s = __float2half_rn(__fmul_rn(gf, __half2float(r)));
    __half o = __float2half_rn(__fmul_rn(__half2float(s), __half2float(u)));
    if (limit != 0.0f) {
        float lim = __half2float(__float2half_rn(fabsf(limit)));
        float p = __half2float(o);
        p = p > lim ? lim : p;
        p = p < -lim ? -lim : p;
        o = __float2half_rn(p);
    }
    return o;
}

}  // namespace berth
