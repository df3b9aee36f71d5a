// cvt_rate.cu -- how many narrow-format conversions per clock does one SM retire?
// One CTA of 1024 threads per SM; every thread runs 8 independent conversions per iteration and
// folds the results into one word (one LOP3 per conversion, full rate).  Reports thread-level
// conversions per clock per SM for
//   cvt.rn.satfinite.e2m1x2.f32     (the NVFP4 quantizer's code conversion, two elements each)
//   cvt.rn.bf16x2.f32, cvt.rn.f16x2.f32   (the GEMM epilogue's packing)
//   fma.rn.f32                       (reference: 128 per clock per SM)
//   an integer/float-ALU rounding of two floats to e2m1 (no conversion instruction)
// Result on B200: e2m1x2 64 per clock per SM (half rate, so 128 elements per clock: not what bounds the
// quantizer), bf16x2 / f16x2 at the FMA rate, the ALU rounding 4 pairs per clock (no alternative).
// Build: nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o cvt_rate cvt_rate.cu
#include <cstdio>
#include <cstdint>
#include <cstdlib>
#include <cuda_runtime.h>
#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e), __LINE__); exit(1);} } while (0)

// e2m1 code of |y| <= 6 (round to nearest even) without a conversion instruction: below 2 the grid is 0.5
// (a magic-number add rounds to it), from 2 up one mantissa bit survives (integer rounding on the float's bits)
__device__ __forceinline__ uint32_t e2m1_alu(float y) {
    const uint32_t s = (__float_as_uint(y) >> 28) & 8u;
    float a = fminf(fabsf(y), 6.0f);
    const float lo = (a + 4194304.0f) - 4194304.0f;            // multiples of 0.5, ties to even
    uint32_t u = __float_as_uint(a);
    u = (u + 0x1fffffu + ((u >> 22) & 1u)) >> 22;              // exponent and one mantissa bit, ties to even
    const uint32_t hi = u - 252u;                              // 2.0 (exponent 128, mantissa 0) -> code 4
    const uint32_t lc = (uint32_t)(int)(lo * 2.0f);            // 0, .5, 1, 1.5, 2 -> 0..4
    return s | (a < 1.75f ? lc : hi);
}

template <int OP>
__global__ void __launch_bounds__(1024) rate_kernel(int iters, float seed, unsigned long long* cyc, uint32_t* sink) {
    float x[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = seed * (float)(threadIdx.x + 1 + i);
    uint32_t acc = 0;
    __syncthreads();
    const long long t0 = clock64();
#pragma unroll 1
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            uint32_t r = 0;
            const float a = x[i], b = x[(i + 1) & 7];
            if (OP == 0) {
                asm volatile("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tcvt.u32.u8 %0, t;\n\t}" : "=r"(r) : "f"(a), "f"(b));
            } else if (OP == 2) {
                asm volatile("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(a), "f"(b));
            } else if (OP == 3) {
                asm volatile("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(a), "f"(b));
            } else if (OP == 4) {
                float d;
                asm volatile("fma.rn.f32 %0, %1, %2, %1;" : "=f"(d) : "f"(a), "f"(b));
                r = __float_as_uint(d);
            } else {
                r = e2m1_alu(a) | (e2m1_alu(b) << 4);
            }
            acc ^= r;
        }
        if (OP == 6) {   // keep the ALU variant's inputs live and changing
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = __uint_as_float(__float_as_uint(x[i]) ^ (acc & 0x00010000u));
        }
    }
    const long long t1 = clock64();
    __syncthreads();
    if (threadIdx.x == 0) cyc[blockIdx.x] = (unsigned long long)(t1 - t0);
    if (acc == 0x12345678u) sink[0] = acc;
}

template <int OP>
void run(const char* name, int sms, unsigned long long* d_cyc, uint32_t* d_sink) {
    const int iters = 4096;
    rate_kernel<OP><<<sms, 1024>>>(64, 0.37f, d_cyc, d_sink);
    rate_kernel<OP><<<sms, 1024>>>(iters, 0.37f, d_cyc, d_sink);
    CK(cudaDeviceSynchronize());
    unsigned long long* h = (unsigned long long*)malloc(sizeof(unsigned long long) * sms);
    CK(cudaMemcpy(h, d_cyc, sizeof(unsigned long long) * sms, cudaMemcpyDeviceToHost));
    unsigned long long mx = 0;
    for (int i = 0; i < sms; ++i) mx = h[i] > mx ? h[i] : mx;
    free(h);
    printf("%-36s %7.2f per clock per SM\n", name, 1024.0 * iters * 8 / (double)mx);
}

int main() {
    cudaDeviceProp prop;
    CK(cudaGetDeviceProperties(&prop, 0));
    const int sms = prop.multiProcessorCount;
    unsigned long long* d_cyc;
    uint32_t* d_sink;
    CK(cudaMalloc(&d_cyc, sizeof(unsigned long long) * sms));
    CK(cudaMalloc(&d_sink, 4));
    run<4>("fma.rn.f32 (+1 LOP3)", sms, d_cyc, d_sink);
    run<0>("cvt.rn.satfinite.e2m1x2.f32", sms, d_cyc, d_sink);
    run<2>("cvt.rn.bf16x2.f32", sms, d_cyc, d_sink);
    run<3>("cvt.rn.f16x2.f32", sms, d_cyc, d_sink);
    run<6>("ALU rounding of a pair to e2m1", sms, d_cyc, d_sink);
    return 0;
}
