// issue_styles.cu -- does the way a warp issues tcgen05.mma matter?  Same MMA stream (4 MMAs + commit
// per group, depth-4 wait on the commit barriers), issued by: thread 0 in a divergent branch; the whole
// warp with the MMA predicated inside the asm; the whole warp with if (elect_one()); the same with the
// stage loop unrolled.  Result on B200: 512 cycles per group (the MMA bound) only for the warp-uniform
// forms or the unrolled ones; a diverged single thread with a wait in its loop loses 10-15 %.
// Build: nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o issue_styles issue_styles.cu
#include <cstdio>
#include <cstdint>
#include <cstdlib>
#include <cuda_runtime.h>
#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e), __LINE__); exit(1);} } while (0)
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t desc_sw128(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3fffu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void mma_nv(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa, uint32_t sfb, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
                 ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc), "r"(sfa), "r"(sfb) : "memory");
}
__device__ __forceinline__ void mma_nv_if(uint32_t on, uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa, uint32_t sfb, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %7, 0;\n\t@q tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
                 ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc), "r"(sfa), "r"(sfb), "r"(on) : "memory");
}
__device__ __forceinline__ void commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void commit_if(uint32_t on, uint32_t bar) {
    asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %1, 0;\n\t@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(bar), "r"(on) : "memory");
}
__device__ __forceinline__ uint32_t test_wait(uint32_t bar, uint32_t par) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(done) : "r"(bar), "r"(par) : "memory");
    return done;
}
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void binit(uint64_t* b, uint32_t n) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(n)); }

// STYLE 0: thread 0 in a divergent branch, no waits      1: same + depth-4 wait
//       2: warp-uniform, predicated asm, depth-4 wait     3: warp-uniform, if(elect_one) around issue, depth-4 wait
//       4: warp-uniform, predicated asm, wait, loop unrolled over 4 stages with all operands precomputed
//       5: thread 0 divergent, wait, unrolled/precomputed  6: style 2 without wait
template <int STYLE>
__global__ void __launch_bounds__(128) mma_style(int iters, unsigned long long* stats) {
    extern __shared__ uint8_t raw[];
    uint8_t* sm = (uint8_t*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint32_t tmem_slot;
    __shared__ __align__(8) uint64_t bar[8];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int i = tid; i < 4 * 49152 / 4; i += 128) ((uint32_t*)sm)[i] = 0x22222222u;
    if (tid == 0) { for (int i = 0; i < 8; ++i) binit(&bar[i], 1); asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
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
    for (int c = 0; c < 256; ++c)
        asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(tmem + ((uint32_t)(warp * 32) << 16) + 256 + c), "r"(0x38383838u) : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t idesc = (1u << 7) | (1u << 10) | ((uint32_t)(256 >> 3) << 17) | (8u << 24);
    const uint32_t base = smem_u32(sm);
    const uint32_t bar0 = smem_u32(&bar[0]);
    long long c0 = 0, c1 = 0; int ok = 1;
    if (STYLE == 0 || STYLE == 1) {
        if (tid == 0) {
            c0 = clock64();
            for (int it = 0; it < iters && ok; ++it) {
                const int s = it & 3;
                const uint64_t a0 = desc_sw128(base + s * 49152), b0 = desc_sw128(base + s * 49152 + 16384);
                const uint32_t sfa = tmem + 256 + s * 48, sfb = sfa + 16;
                if (STYLE == 1 && it >= 4) { int n = 0; while (!test_wait(bar0 + 8 * s, ((it >> 2) - 1) & 1)) if (++n > 100000000) { ok = 0; break; } }
#pragma unroll
                for (int j = 0; j < 4; ++j) mma_nv(tmem, a0 + 2 * j, b0 + 2 * j, idesc, sfa + 4 * j, sfb + 8 * j, (it | j) ? 1u : 0u);
                commit(bar0 + 8 * s);
            }
            c1 = clock64();
        }
    } else if (STYLE == 2 || STYLE == 3 || STYLE == 6) {
        if (warp == 0) {
            const uint32_t on = lane == 0;
            c0 = clock64();
            for (int it = 0; it < iters && ok; ++it) {
                const int s = it & 3;
                const uint64_t a0 = desc_sw128(base + s * 49152), b0 = desc_sw128(base + s * 49152 + 16384);
                const uint32_t sfa = tmem + 256 + s * 48, sfb = sfa + 16;
                if (STYLE != 6 && it >= 4) { int n = 0; while (!test_wait(bar0 + 8 * s, ((it >> 2) - 1) & 1)) if (++n > 100000000) { ok = 0; break; } }
                if (STYLE == 3) {
                    if (elect_one()) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) mma_nv(tmem, a0 + 2 * j, b0 + 2 * j, idesc, sfa + 4 * j, sfb + 8 * j, (it | j) ? 1u : 0u);
                        commit(bar0 + 8 * s);
                    }
                    __syncwarp();
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) mma_nv_if(on, tmem, a0 + 2 * j, b0 + 2 * j, idesc, sfa + 4 * j, sfb + 8 * j, (it | j) ? 1u : 0u);
                    commit_if(on, bar0 + 8 * s);
                }
            }
            c1 = clock64();
        }
    } else {
        const bool mine = (STYLE == 4) ? (warp == 0) : (tid == 0);
        if (mine) {
            const uint32_t on = (STYLE == 4) ? (lane == 0) : 1u;
            c0 = clock64();
            for (int it4 = 0; it4 < iters / 4 && ok; ++it4) {
#pragma unroll
                for (int s = 0; s < 4; ++s) {
                    const uint64_t a0 = desc_sw128(base + s * 49152), b0 = desc_sw128(base + s * 49152 + 16384);
                    const uint32_t sfa = tmem + 256 + s * 48, sfb = sfa + 16;
                    if (it4 >= 1) { int n = 0; while (!test_wait(bar0 + 8 * s, (it4 - 1) & 1)) if (++n > 100000000) { ok = 0; break; } }
#pragma unroll
                    for (int j = 0; j < 4; ++j) mma_nv_if(on, tmem, a0 + 2 * j, b0 + 2 * j, idesc, sfa + 4 * j, sfb + 8 * j, (it4 | s | j) ? 1u : 0u);
                    commit_if(on, bar0 + 8 * s);
                }
            }
            c1 = clock64();
        }
    }
    if (tid == 0) {
        // drain: one more commit, then wait for it
        commit(bar0 + 8 * 7);
        int n = 0; while (!test_wait(bar0 + 8 * 7, 0)) if (++n > 100000000) { ok = 0; break; }
        stats[0] = (unsigned long long)(clock64() - c0); stats[1] = ok; stats[2] = (unsigned long long)(c1 - c0);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
}
template <int STYLE>
void run(const char* name, unsigned long long* d) {
    unsigned long long h[3]; const int iters = 4000;
    CK(cudaFuncSetAttribute(mma_style<STYLE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    for (int r = 0; r < 2; ++r) { mma_style<STYLE><<<1, 128, 200 * 1024>>>(iters, d); CK(cudaDeviceSynchronize()); CK(cudaMemcpy(h, d, 24, cudaMemcpyDeviceToHost)); }
    printf("style %d (%s): %.1f cycles per group of 4 MMAs (issue loop %.1f) ok=%llu\n", STYLE, name, (double)h[0] / iters, (double)h[2] / iters, h[1]);
}
int main() {
    unsigned long long* d; CK(cudaMalloc(&d, 64));
    run<0>("thread 0 divergent, no waits", d);
    run<1>("thread 0 divergent, depth-4 wait", d);
    run<2>("warp-uniform predicated asm, wait", d);
    run<3>("warp-uniform if(elect_one), wait", d);
    run<4>("warp-uniform predicated, unrolled x4 stages, wait", d);
    run<5>("thread 0 divergent, unrolled x4 stages, wait", d);
    run<6>("warp-uniform predicated asm, no wait", d);
    return 0;
}
