// quant_block.cuh -- the per-block arithmetic of the NVFP4 quantizer (scale byte and e2m1 codes of 8 elements),
// shared by the quantizer kernels (quant.cu) and by the GEMM epilogues that quantize their own output (gemm_duo.cuh).
// The comment at the top of quant.cu derives why these forms return the reference's bytes.
#pragma once

#include "common.cuh"

namespace tfp4 {

namespace {

// eight floats -> eight e2m1 codes (hardware round-to-nearest-even, saturating), element i in nibble i; the four
// byte results are joined inside one statement so that the packing can fold into the conversions
__device__ __forceinline__ uint32_t pack_codes_rne(const float (&y)[8]) {
    uint32_t w;
    asm("{\n\t.reg .b8 t0, t1, t2, t3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 t0, %2, %1;\n\tcvt.rn.satfinite.e2m1x2.f32 t1, %4, %3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 t2, %6, %5;\n\tcvt.rn.satfinite.e2m1x2.f32 t3, %8, %7;\n\t"
        "mov.b32 %0, {t0, t1, t2, t3};\n\t}"
        : "=r"(w)
        : "f"(y[0]), "f"(y[1]), "f"(y[2]), "f"(y[3]), "f"(y[4]), "f"(y[5]), "f"(y[6]), "f"(y[7]));
    return w;
}

// Arguments by value: a reference to the caller's array would pin that array in local memory
// (a store of all eight values per row on the common path, for a call that almost never happens).
__device__ __noinline__ uint32_t pack_codes_literal_v(float f0, float f1, float f2, float f3, float f4, float f5,
                                                      float f6, float f7, float ds) {
    const float f[8] = {f0, f1, f2, f3, f4, f5, f6, f7};
    uint32_t w = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) w |= e2m1_ties_up(__fdiv_rn(f[i], ds)) << (4 * i);
    return w;
}
__device__ __noinline__ uint32_t code_literal(float f, float ds) { return e2m1_ties_up(__fdiv_rn(f, ds)); }
__device__ __forceinline__ uint32_t pack_codes_literal(const float (&f)[8], float ds) {
    return pack_codes_literal_v(f[0], f[1], f[2], f[3], f[4], f[5], f[6], f[7], ds);
}

__device__ __forceinline__ float fma_pz(float a, float b) {  // a*b + (+0): maps -0 to +0
    float d;
    asm("fma.rn.f32 %0, %1, %2, 0f00000000;" : "=f"(d) : "f"(a), "f"(b));
    return d;
}

// two products a0*b, a1*b in one packed instruction, each + (+0) like fma_pz
__device__ __forceinline__ void mul2_pz(float& d0, float& d1, float a0, float a1, float b) {
    uint64_t av, bv, dv;
    asm("mov.b64 %0, {%1, %2};" : "=l"(av) : "f"(a0), "f"(a1));
    asm("mov.b64 %0, {%1, %1};" : "=l"(bv) : "f"(b));
    asm("{\n\t.reg .b64 z;\n\tmov.b64 z, 0;\n\tfma.rn.f32x2 %0, %1, %2, z;\n\t}" : "=l"(dv) : "l"(av), "l"(bv));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d0), "=f"(d1) : "l"(dv));
}

// One half block (8 consecutive elements held by this lane, the other 8 by lane ^ 1): the block's scale
// byte `sc`; returns the decode scale ds = dec(sc) * ts.  Every lane of the warp must call it (one shuffle).
// rts_lo / rts_hi: 1/ts biased by -+2^-20 (bracket modes only).
template <int MODE>
__device__ __forceinline__ float block_scale8(const float (&f)[8], float ts, float rts_lo, float rts_hi, uint32_t& sc) {
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    float pre = amax * (1.0f / 6.0f);
    if (MODE == 1 || MODE == 3) {
        // (amax * (1/6)) / ts without the IEEE division in the common case: two products with reciprocals of ts
        // biased by +-2^-20 bracket the quotient (and its float rounding); e4m3 rounding is monotonic, so when
        // both ends encode alike that is the encoding of the quotient.  Otherwise (about 2^-16 of the blocks)
        // the literal division decides.
        const uint32_t both = f32x2_to_e4m3x2(pre * rts_lo, pre * rts_hi);
        sc = both & 0x7fu;
        if (sc != ((both >> 8) & 0x7fu)) sc = f32x2_to_e4m3x2(__fdiv_rn(pre, ts), 0.f) & 0x7fu;
    } else {
        if (MODE != 0) pre = __fdiv_rn(pre, ts);   // (amax * (1/6)) / ts, the reference's operand order
        sc = f32x2_to_e4m3x2(pre, 0.f) & 0x7fu;
    }
    const float sf = e4m3_to_f32(sc);
    return (MODE != 0) ? sf * ts : sf;
}

// The eight e2m1 codes of this lane's elements (element i in nibble i) for the decode scale ds.
template <int MODE>
__device__ __forceinline__ uint32_t block_codes8(const float (&f)[8], float ds) {
    uint32_t codes = 0;
    if (MODE == 0) {
        const float rb = __frcp_rn(ds) * 1.000000476837158203125f;   // * (1 + 2^-21)
        float y[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) y[i] = fma_pz(f[i], rb);
        codes = pack_codes_rne(y);
    } else if (MODE == 1 || MODE == 3) {
        // 1/ds to within one ulp is enough here: the +-2^-20 margins still bracket the true quotient
        float rr;
        asm("rcp.approx.f32 %0, %1;" : "=f"(rr) : "f"(ds));
        const float r_hi = rr * 1.00000095367431640625f;   // 1 + 2^-20
        const float r_lo = rr * 0.99999904632568359375f;   // 1 - 2^-20
        float yh[8], yl[8];
        bool tiny = false;
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
            mul2_pz(yh[i], yh[i + 1], f[i], f[i + 1], r_hi);
            mul2_pz(yl[i], yl[i + 1], f[i], f[i + 1], r_lo);
        }
        if (MODE == 1) {
#pragma unroll
            for (int i = 0; i < 8; ++i)   // 0 < |x| < 2^-100 (bits 0x0d800000): quotient may underflow
                tiny |= ((__float_as_uint(f[i]) & 0x7fffffffu) - 1u) < 0x0d7fffffu;
        }
        codes = pack_codes_rne(yh);
        const uint32_t cl = pack_codes_rne(yl);
        if (MODE == 1 && tiny) {
            codes = pack_codes_literal(f, ds);
        } else if (cl != codes) {
            // only the elements whose two ends disagree take the division (16-bit inputs times a
            // short per-tensor scale land exactly on rounding boundaries far more often than chance)
            const uint32_t diff = cl ^ codes;
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if ((diff >> (4 * i)) & 0xfu)
                    codes = (codes & ~(0xfu << (4 * i))) | (code_literal(f[i], ds) << (4 * i));
        }
    } else {
        codes = pack_codes_literal(f, ds);
    }
    return codes;
}

}  // namespace

}  // namespace tfp4
