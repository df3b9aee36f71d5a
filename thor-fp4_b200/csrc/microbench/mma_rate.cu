// mma_rate.cu -- how fast does the tensor pipe of one SM execute back-to-back tcgen05.mma?
// One CTA per SM, operands and scale factors resident (no loads), one thread issues 4 MMAs per
// iteration plus (optionally) a commit.  Reports cycles per MMA (clock64), nanoseconds per MMA
// (globaltimer), the SM clock during the loop, and the TFLOP/s this would be on the whole GPU.
// Kinds: NVFP4 (mxf4nvf4 scale_vec::4X), MXFP4 (2X), MXFP8 block-scaled, bf16, e4m3, e2m1 in f8f6f4;
// N = 64 / 128 / 256; zero, random and constant operand bits (the clock under power cap depends on them).
// Result on B200: 128 cycles per 128x256x64-byte MMA for every kind, 109 cycles at N = 128.
// Build: nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o mma_rate mma_rate.cu
#include <cstdio>
#include <cstdint>
#include <cstdlib>
#include <cuda_runtime.h>
#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e), __LINE__); exit(1);} } while (0)
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t desc_sw128(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3fffu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ uint64_t gtimer() { uint64_t t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
// KIND: 0 mxf4nvf4 4X, 1 mxf8f6f4 block_scale, 2 f16 (bf16), 3 f8f6f4 (e4m3), 4 mxf4 2X(mxf4nvf4 scale_vec::2X ue8m0), 5 f8f6f4 with e2m1 inputs
template <int KIND>
__device__ __forceinline__ void mma(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa, uint32_t sfb, uint32_t acc) {
    if (KIND == 0)
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
                     ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc), "r"(sfa), "r"(sfb) : "memory");
    else if (KIND == 1)
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
                     ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc), "r"(sfa), "r"(sfb) : "memory");
    else if (KIND == 2)
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                     ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
    else if (KIND == 3 || KIND == 5)
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
                     ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
    else
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
                     ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc), "r"(sfa), "r"(sfb) : "memory");
}
template <int KIND, int BN>
__global__ void __launch_bounds__(128) rate_kernel(int iters, int fill, int commit_every, unsigned long long* stats) {
    extern __shared__ uint8_t raw[];
    uint8_t* sm = (uint8_t*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint32_t tmem_slot;
    __shared__ __align__(8) uint64_t bar[2];
    const int tid = threadIdx.x, warp = tid >> 5;
    constexpr int A_BYTES = 128 * 128, B_BYTES = BN * 128, NST = 2;
    uint32_t* w = (uint32_t*)sm;
    for (int i = tid; i < NST * (A_BYTES + B_BYTES) / 4; i += 128) {
        uint32_t v = 0;
        if (fill == 1) { v = (i * 2654435761u) ^ (i >> 3); if (KIND == 2) v &= 0x3fff3fffu; if (KIND == 3 || KIND==1) v &= 0x3f3f3f3fu; }
        if (fill == 2) v = (KIND == 2) ? 0x3f803f80u : ((KIND == 0 || KIND == 4) ? 0x22222222u : 0x38383838u);
        w[i] = v;
    }
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar[0])));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar[1])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_slot;
    // scale columns 256..511: ones (0x38 ue4m3 = 1.0 ; 0x7f ue8m0 = 1.0)
    {
        uint32_t v = (KIND == 0) ? 0x38383838u : 0x7f7f7f7fu;
        if (fill == 0) v = 0;
        for (int c = 0; c < 256; c += 1) {
            asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(tmem + ((uint32_t)(warp * 32) << 16) + 256 + c), "r"(v) : "memory");
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    uint32_t idesc;
    if (KIND == 0) idesc = (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | (0u << 23) | (8u << 24);
    else if (KIND == 4) idesc = (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | (1u << 23) | (8u << 24);
    else if (KIND == 1) idesc = (0u << 7) | (0u << 10) | ((uint32_t)(BN >> 3) << 17) | (1u << 23) | (8u << 24);
    else if (KIND == 2) idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | (8u << 24);
    else if (KIND == 3) idesc = (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(BN >> 3) << 17) | (8u << 24);
    else idesc = (1u << 4) | (5u << 7) | (5u << 10) | ((uint32_t)(BN >> 3) << 17) | (8u << 24);
    if (tid == 0) {
        const uint32_t base = smem_u32(sm);
        long long c0 = clock64(); uint64_t g0 = gtimer();
        for (int it = 0; it < iters; ++it) {
            const uint32_t st = (uint32_t)(it & 1);
            const uint64_t a0 = desc_sw128(base + st * (A_BYTES + B_BYTES));
            const uint64_t b0 = desc_sw128(base + st * (A_BYTES + B_BYTES) + A_BYTES);
            const uint32_t sfa = tmem + 256 + (it & 3) * 48, sfb = sfa + 16;
#pragma unroll
            for (int j = 0; j < 4; ++j)
                mma<KIND>(tmem, a0 + 2 * j, b0 + 2 * j, idesc, sfa + 4 * j, sfb + 8 * j, (it | j) ? 1u : 0u);
            if (commit_every && (it % commit_every) == commit_every - 1)
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bar[1])) : "memory");
        }
        long long c_issue = clock64();
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bar[0])) : "memory");
        uint32_t done = 0; long long lim = clock64() + 4000000000ll;
        while (!done && clock64() < lim)
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(done) : "r"(smem_u32(&bar[0])), "r"(0u) : "memory");
        long long c1 = clock64(); uint64_t g1 = gtimer();
        if (blockIdx.x < 256) {
            stats[blockIdx.x * 4 + 0] = (unsigned long long)(c1 - c0);
            stats[blockIdx.x * 4 + 1] = (unsigned long long)(g1 - g0);
            stats[blockIdx.x * 4 + 2] = (unsigned long long)(c_issue - c0);
            stats[blockIdx.x * 4 + 3] = done;
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
}
template <int KIND, int BN>
void run(const char* name, int grid, int iters, int fill, int commit_every, unsigned long long* d_stats) {
    const int smem = 2 * (128 * 128 + BN * 128) + 1024;
    CK(cudaFuncSetAttribute(rate_kernel<KIND, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    for (int rep = 0; rep < 2; ++rep) {
        rate_kernel<KIND, BN><<<grid, 128, smem>>>(iters, fill, commit_every, d_stats);
        CK(cudaDeviceSynchronize());
    }
    unsigned long long h[1024];
    CK(cudaMemcpy(h, d_stats, sizeof(h), cudaMemcpyDeviceToHost));
    double cyc = 0, ns = 0, iss = 0; int n = grid < 256 ? grid : 256, ok = 1;
    for (int i = 0; i < n; ++i) { cyc += h[4 * i]; ns += h[4 * i + 1]; iss += h[4 * i + 2]; ok &= (int)h[4 * i + 3]; }
    cyc /= n; ns /= n; iss /= n;
    const double mmas = 4.0 * iters;
    const double kel = (KIND == 0 || KIND == 4) ? 64 : (KIND == 2 ? 16 : 32);
    printf("%-10s N=%3d grid=%3d fill=%d commit=%d: %.1f cyc/MMA (issue %.1f)  %.1f ns/MMA  clk=%.0f MHz  -> %.0f TFLOPS on %d SMs  done=%d\n",
           name, BN, grid, fill, commit_every, cyc / mmas, iss / mmas, ns / mmas, cyc / ns * 1e3, 2.0 * 128 * BN * kel * mmas / ns * 1e-3 * grid, grid, ok);
}
int main(int argc, char** argv) {
    unsigned long long* d_stats; CK(cudaMalloc(&d_stats, 1024 * 8));
    const int iters = 20000;
    for (int grid : {1, 148}) for (int fill : {0, 1, 2}) {
        run<0, 256>("nvf4_4x", grid, iters, fill, 1, d_stats);
        run<0, 128>("nvf4_4x", grid, iters, fill, 1, d_stats);
        run<0, 64>("nvf4_4x", grid, iters, fill, 1, d_stats);
        run<4, 256>("mxf4_2x", grid, iters, fill, 1, d_stats);
        run<1, 256>("mxf8", grid, iters, fill, 1, d_stats);
        run<2, 256>("bf16", grid, iters, fill, 1, d_stats);
        run<2, 128>("bf16", grid, iters, fill, 1, d_stats);
        run<3, 256>("e4m3", grid, iters, fill, 1, d_stats);
        run<5, 256>("e2m1_f8f6f4", grid, iters, fill, 1, d_stats);
    }
    run<0, 256>("nvf4_4x", 148, iters, 1, 0, d_stats);
    run<0, 256>("nvf4_4x", 148, iters, 1, 8, d_stats);
    return 0;
}
