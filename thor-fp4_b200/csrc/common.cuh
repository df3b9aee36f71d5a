// common.cuh -- shared helpers of the sm_100a NVFP4 library.
//
// Format recap (identical to the reference project, csrc/thor_fp4_core.cu:16-33):
//   * codes: e2m1, two per byte, element 2j in the low nibble, row-major (R, K/2);
//   * block scales: one byte per 16 (NVFP4, UE4M3) or 32 (MX, UE8M0) elements,
//     stored in 128-row x 4-scale "atoms" of 512 bytes:
//       byte(r, s) = ((r/128) * (S/4) + s/4) * 512 + 16*(r%32) + 4*((r%128)/32) + s%4
//     which is exactly what tcgen05.cp.32x128b.warpx4 moves into tensor memory;
//   * an optional per-tensor FP32 scale rides the GEMM's alpha.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>
#include <cstdio>

#define TFP4_OK 0
#define TFP4_ERR_CUDA (-1)
#define TFP4_ERR_DRIVER (-2)
#define TFP4_ERR_BAD_K (-3)
#define TFP4_ERR_NO_PLAN (-4)
#define TFP4_ERR_LAUNCH (-5)
#define TFP4_ERR_BAD_M (-6)
#define TFP4_ERR_BAD_ARG (-7)
#define TFP4_ERR_DEVICE_TIMEOUT (-8)

#define TFP4_CK(x)                                                                         \
    do {                                                                                   \
        cudaError_t e_ = (x);                                                              \
        if (e_ != cudaSuccess) {                                                           \
            fprintf(stderr, "thor_fp4_b200: CUDA error %s at %s:%d\n", cudaGetErrorString(e_), \
                    __FILE__, __LINE__);                                                   \
            return TFP4_ERR_CUDA;                                                          \
        }                                                                                  \
    } while (0)

namespace tfp4 {

enum InDtype { IN_F32 = 0, IN_F16 = 1, IN_BF16 = 2 };
enum OutDtype { OUT_F16 = 0, OUT_BF16 = 1, OUT_F32 = 2 };

__host__ __device__ __forceinline__ int64_t pad128(int64_t r) { return (r + 127) / 128 * 128; }

// byte index of scale (row r, scale column s), S scale columns per row
__host__ __device__ __forceinline__ int64_t sf_index(int64_t r, int64_t s, int64_t S) {
    int64_t a = r >> 7, b = (r & 127) >> 5, c = r & 31;
    return (a * (S >> 2) + (s >> 2)) * 512 + 16 * c + 4 * b + (s & 3);
}

// ---------------------------------------------------------------------------
// scalar format conversions (device)
// ---------------------------------------------------------------------------

// two floats -> two e4m3 bytes (round-to-nearest-even, saturate to +-448):
// result bits [7:0] = enc(lo), [15:8] = enc(hi)
__device__ __forceinline__ uint32_t f32x2_to_e4m3x2(float lo, float hi) {
    uint32_t r;
    asm("{\n\t.reg .b16 t;\n\tcvt.rn.satfinite.e4m3x2.f32 t, %1, %2;\n\tcvt.u32.u16 %0, t;\n\t}"
        : "=r"(r)
        : "f"(hi), "f"(lo));
    return r;
}

// four floats -> four e4m3 bytes in one word (byte i = enc(v_i)); both conversions and the packing in one statement
__device__ __forceinline__ uint32_t f32x4_to_e4m3x4(float v0, float v1, float v2, float v3) {
    uint32_t r;
    asm("{\n\t.reg .b16 t0, t1;\n\tcvt.rn.satfinite.e4m3x2.f32 t0, %2, %1;\n\t"
        "cvt.rn.satfinite.e4m3x2.f32 t1, %4, %3;\n\tmov.b32 %0, {t0, t1};\n\t}"
        : "=r"(r)
        : "f"(v0), "f"(v1), "f"(v2), "f"(v3));
    return r;
}

// e4m3 byte -> float (exact)
__device__ __forceinline__ float e4m3_to_f32(uint32_t b) {
    uint32_t h2;
    unsigned short s = (unsigned short)(b & 0xffu);
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(s));
    __half_raw hr;
    hr.x = (unsigned short)(h2 & 0xffffu);
    return __half2float(__half(hr));
}

// two floats -> one byte of two e2m1 codes, round-to-nearest-EVEN, saturating,
// NaN -> +6: bits [3:0] = enc(lo), [7:4] = enc(hi)
__device__ __forceinline__ uint32_t f32x2_to_e2m1x2_rne(float lo, float hi) {
    unsigned short r;
    asm("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tmov.b16 %0, {t, 0};\n\t}"
        : "=h"(r)
        : "f"(hi), "f"(lo));
    return (uint32_t)r;
}

// one byte of two e2m1 codes -> two floats (exact; code 8 decodes to -0)
__device__ __forceinline__ void e2m1x2_to_f32x2(uint32_t byte, float& lo, float& hi) {
    uint32_t h2;
    unsigned short s = (unsigned short)(byte & 0xffu);
    asm("{\n\t.reg .b8 t, z;\n\tmov.b16 {t, z}, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, t;\n\t}" : "=r"(h2) : "h"(s));
    float2 f = __half22float2(*reinterpret_cast<__half2*>(&h2));
    lo = f.x;
    hi = f.y;
}

// one word of eight e2m1 codes -> eight floats (element i from nibble i); the word is split into its bytes
// inside one statement so that the byte selection can fold into the conversions
__device__ __forceinline__ void e2m1x8_to_f32x8(uint32_t word, float (&o)[8]) {
    uint32_t h0, h1, h2, h3;
    asm("{\n\t.reg .b8 t0, t1, t2, t3;\n\tmov.b32 {t0, t1, t2, t3}, %4;\n\t"
        "cvt.rn.f16x2.e2m1x2 %0, t0;\n\tcvt.rn.f16x2.e2m1x2 %1, t1;\n\t"
        "cvt.rn.f16x2.e2m1x2 %2, t2;\n\tcvt.rn.f16x2.e2m1x2 %3, t3;\n\t}"
        : "=r"(h0), "=r"(h1), "=r"(h2), "=r"(h3) : "r"(word));
    const uint32_t h[4] = {h0, h1, h2, h3};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h[i]));
        o[2 * i] = f.x;
        o[2 * i + 1] = f.y;
    }
}

// e2m1 code with the reference's rule: sign = (v < 0), magnitude clamped to 6,
// midpoints of {0,.5,1,1.5,2,3,4,6} round UP (csrc/thor_fp4_core.cu:77-92)
__device__ __forceinline__ uint32_t e2m1_ties_up(float v) {
    uint32_t sign = v < 0.f ? 8u : 0u;
    float a = fminf(fabsf(v), 6.0f);
    uint32_t code = (a >= 0.25f) + (a >= 0.75f) + (a >= 1.25f) + (a >= 1.75f) + (a >= 2.5f) +
                    (a >= 3.5f) + (a >= 5.0f);
    return sign | code;
}

// widen 8 consecutive elements starting at p (16-byte aligned for 16-bit types,
// 32-byte aligned for f32) to float
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&f)[8]);

template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&f)[8]) {
    float4 a = __ldg(reinterpret_cast<const float4*>(p));
    float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
    f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[8]) {
    uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

template <>
__device__ __forceinline__ void load8<__half>(const __half* p, float (&f)[8]) {
    uint4 v = __ldg(reinterpret_cast<const uint4*>(p));
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
        float2 ff = __half22float2(h);
        f[2 * i] = ff.x;
        f[2 * i + 1] = ff.y;
    }
}

// raw 8-element fetch (kept in registers while older rows are processed) and its widening
// Programmatic dependent launch.  griddep_launch: the next kernel in the stream, if it was launched with the
// programmatic-serialization attribute, may start its prologue once every CTA of this grid has got here.
// griddep_wait: blocks until the preceding grid has completed and its writes are visible (returns at once
// when the kernel was launched without the attribute).
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename T> struct Raw8 { uint4 a; };
template <> struct Raw8<float> { uint4 a, b; };

template <typename T>
__device__ __forceinline__ Raw8<T> fetch8(const T* p) {
    Raw8<T> r;
    r.a = __ldg(reinterpret_cast<const uint4*>(p));
    return r;
}
template <>
__device__ __forceinline__ Raw8<float> fetch8<float>(const float* p) {
    Raw8<float> r;
    r.a = __ldg(reinterpret_cast<const uint4*>(p));
    r.b = __ldg(reinterpret_cast<const uint4*>(p) + 1);
    return r;
}
template <typename T>
__device__ __forceinline__ Raw8<T> zero8() {
    Raw8<T> r;
    r.a = make_uint4(0u, 0u, 0u, 0u);
    if constexpr (sizeof(T) == 4) r.b = make_uint4(0u, 0u, 0u, 0u);
    return r;
}
__device__ __forceinline__ void widen8(const Raw8<float>& r, float (&f)[8]) {
    f[0] = __uint_as_float(r.a.x); f[1] = __uint_as_float(r.a.y); f[2] = __uint_as_float(r.a.z); f[3] = __uint_as_float(r.a.w);
    f[4] = __uint_as_float(r.b.x); f[5] = __uint_as_float(r.b.y); f[6] = __uint_as_float(r.b.z); f[7] = __uint_as_float(r.b.w);
}
__device__ __forceinline__ void widen8(const Raw8<__nv_bfloat16>& r, float (&f)[8]) {
    const uint32_t w[4] = {r.a.x, r.a.y, r.a.z, r.a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
__device__ __forceinline__ void widen8(const Raw8<__half>& r, float (&f)[8]) {
    const uint32_t w[4] = {r.a.x, r.a.y, r.a.z, r.a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 ff = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        f[2 * i] = ff.x;
        f[2 * i + 1] = ff.y;
    }
}

template <typename T>
__device__ __forceinline__ T cast_out(float v);
template <>
__device__ __forceinline__ float cast_out<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half cast_out<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 cast_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

}  // namespace tfp4
