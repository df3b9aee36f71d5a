// det_math.cuh -- activation functions built from IEEE binary32 add / multiply / fused multiply-add and integer
// operations only, so that a CPU restatement with the same operation order returns the same bits.
//
// The hardware's ex2.approx / rcp.approx / erff are a few ulps accurate but their bits are not specified, and an
// activation value that lands on the other side of a quantization threshold changes a code byte.  The epilogues
// that quantize act(x) (SwiGLU -> NVFP4, bias + gelu/silu -> MXFP8) therefore use the functions below: every
// operation is a correctly rounded one (explicit __f*_rn intrinsics, which the compiler never contracts or
// reassociates), and the CPU oracle repeats them one for one (oracle/nvfp4_oracle.c, "deterministic activations").
//
//   exp2(t), |t| <= 125: n = round(t) through the 1.5 * 2^23 trick, f = t - n in [-0.5, 0.5], 2^f by the degree-6
//       Taylor polynomial of e^(f ln 2) (relative error <= 1.3e-7), 2^n added into the exponent field.
//   1/d, d a positive normal number: integer first guess (error <= 12.5 %), three Newton steps x += x (1 - d x).
//   silu(x) = x / (1 + e^-x);  gelu(x) = x * Phi(x) with erfc from Abramowitz & Stegun 7.1.26
//       (|error of erf| <= 1.5e-7), Phi(x) = 1 - erfc(|x|/sqrt 2)/2 for x >= 0 and erfc(|x|/sqrt 2)/2 for x < 0.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace tfp4 {

__device__ __forceinline__ float det_exp2(float t) {
    t = fminf(fmaxf(t, -125.0f), 125.0f);                 // NaN -> -125 (min / max return the number)
    const float r = __fadd_rn(t, 12582912.0f);            // 1.5 * 2^23: the integer nearest to t sits in the low bits
    const float n = __fadd_rn(r, -12582912.0f);
    const float f = __fadd_rn(t, -n);
    float p = 0x1.430912p-13f;
    p = __fmaf_rn(p, f, 0x1.5d87fep-10f);
    p = __fmaf_rn(p, f, 0x1.3b2ab6p-7f);
    p = __fmaf_rn(p, f, 0x1.c6b08ep-5f);
    p = __fmaf_rn(p, f, 0x1.ebfbep-3f);
    p = __fmaf_rn(p, f, 0x1.62e43p-1f);
    p = __fmaf_rn(p, f, 1.0f);
    return __uint_as_float(__float_as_uint(p) + (__float_as_uint(r) << 23));
}

__device__ __forceinline__ float det_rcp(float d) {
    float x = __uint_as_float(0x7EF311C7u - __float_as_uint(d));
#pragma unroll
    for (int i = 0; i < 3; ++i) {
        const float e = __fmaf_rn(-d, x, 1.0f);
        x = __fmaf_rn(x, e, x);
    }
    return x;
}

__device__ __forceinline__ float det_silu(float x) {
    const float e = det_exp2(__fmul_rn(x, -0x1.715476p+0f));      // e^-x
    return __fmul_rn(x, det_rcp(__fadd_rn(1.0f, e)));
}

__device__ __forceinline__ float det_gelu(float x) {
    const float z = __fmul_rn(fabsf(x), 0x1.6a09e6p-1f);           // |x| / sqrt 2
    const float t = det_rcp(__fmaf_rn(0x1.4f740ap-2f, z, 1.0f));
    float p = 0x1.0fb844p+0f;
    p = __fmaf_rn(p, t, -0x1.7401c6p+0f);
    p = __fmaf_rn(p, t, 0x1.6be1c6p+0f);
    p = __fmaf_rn(p, t, -0x1.23531cp-2f);
    p = __fmaf_rn(p, t, 0x1.04f20cp-2f);
    p = __fmul_rn(p, t);
    const float e = det_exp2(__fmul_rn(__fmul_rn(z, z), -0x1.715476p+0f));   // e^(-z^2)
    const float hc = __fmul_rn(0.5f, __fmul_rn(p, e));              // erfc(z) / 2
    const float phi = (x < 0.0f) ? hc : __fadd_rn(1.0f, -hc);
    return __fmul_rn(x, phi);
}

}  // namespace tfp4
