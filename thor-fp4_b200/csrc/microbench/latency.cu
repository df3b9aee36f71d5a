// latency.cu -- latencies that bound a TMA + mbarrier + tcgen05 pipeline on one SM:
//   * commit chain: 4 MMAs + tcgen05.commit, waiting for the commit `depth` groups back
//   * barrier ping-pong between two warps of a CTA, and between the two CTAs of a cluster
//   * cp.async.bulk loads of 512 B / 16 KB / 32 KB from L2, `depth` in flight, on 1 and on 148 SMs
//   * ld.shared + 3 x tcgen05.st.x4 + tcgen05.wait::st (the scale-loader step)
// Every wait is bounded.  Results on B200: ~180 cycles per hop inside a CTA, ~550 between CTAs of a
// cluster, ~470 cycles for a small L2-resident bulk load, 60-85 bytes per cycle and SM with all SMs loading.
// Build: nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o latency latency.cu
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
__device__ __forceinline__ void commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t test_wait(uint32_t bar, uint32_t par) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(done) : "r"(bar), "r"(par) : "memory");
    return done;
}
__device__ __forceinline__ uint32_t test_wait_cl(uint32_t bar, uint32_t par) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(done) : "r"(bar), "r"(par) : "memory");
    return done;
}
__device__ __forceinline__ bool wait(uint32_t bar, uint32_t par) {
    long long lim = clock64() + 400000000ll;
    while (!test_wait(bar, par)) if (clock64() > lim) return false;
    return true;
}
__device__ __forceinline__ bool wait_cl(uint32_t bar, uint32_t par) {
    long long lim = clock64() + 400000000ll;
    while (!test_wait_cl(bar, par)) if (clock64() > lim) return false;
    return true;
}
__device__ __forceinline__ void arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void arrive_remote(uint32_t bar, uint32_t cta) {
    asm volatile("{\n\t.reg .b32 r;\n\tmapa.shared::cluster.u32 r, %0, %1;\n\tmbarrier.arrive.release.cluster.shared::cluster.b64 _, [r];\n\t}" ::"r"(bar), "r"(cta) : "memory");
}
__device__ __forceinline__ void binit(uint64_t* b, uint32_t n) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(n)); }

// mode 0: depth-D chain of (4 MMAs + commit), wait for the commit D groups back before issuing the next
__global__ void __launch_bounds__(128) commit_lat(int iters, int depth, unsigned long long* stats) {
    extern __shared__ uint8_t raw[];
    uint8_t* sm = (uint8_t*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint32_t tmem_slot;
    __shared__ __align__(8) uint64_t bar[8];
    const int tid = threadIdx.x, warp = tid >> 5;
    for (int i = tid; i < (16384 + 32768) / 4; i += 128) ((uint32_t*)sm)[i] = 0x22222222u;
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
    const uint32_t idesc = (1u << 7) | (1u << 10) | ((uint32_t)(256 >> 3) << 17) | (8u << 24);
    if (tid == 0) {
        const uint32_t base = smem_u32(sm);
        const uint64_t a0 = desc_sw128(base), b0 = desc_sw128(base + 16384);
        int ok = 1;
        long long c0 = clock64();
        for (int it = 0; it < iters && ok; ++it) {
            const int s = it % depth;
            if (it >= depth) ok = wait(smem_u32(&bar[s]), ((it / depth) - 1) & 1);
#pragma unroll
            for (int j = 0; j < 4; ++j) mma_nv(tmem, a0 + 2 * j, b0 + 2 * j, idesc, tmem + 256 + 4 * j, tmem + 272 + 8 * j, 1u);
            commit(smem_u32(&bar[s]));
        }
        // drain
        for (int it = iters; it < iters + depth && ok; ++it) { const int s = it % depth; ok = wait(smem_u32(&bar[s]), ((it / depth) - 1) & 1); }
        long long c1 = clock64();
        stats[0] = (unsigned long long)(c1 - c0); stats[1] = ok;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
}

// local ping-pong between warp 0 and warp 1 (one lane each)
__global__ void __launch_bounds__(64) hop_local(int iters, unsigned long long* stats) {
    __shared__ __align__(8) uint64_t bar[2];
    if (threadIdx.x == 0) { binit(&bar[0], 1); binit(&bar[1], 1); }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) {
        int ok = 1;
        long long c0 = clock64();
        for (int it = 0; it < iters && ok; ++it) {
            if (warp == 0) { arrive(smem_u32(&bar[0])); ok = wait(smem_u32(&bar[1]), it & 1); }
            else { ok = wait(smem_u32(&bar[0]), it & 1); arrive(smem_u32(&bar[1])); }
        }
        if (warp == 0) { stats[0] = (unsigned long long)(clock64() - c0); stats[1] = ok; }
    }
}
// cluster ping-pong: CTA0 arrives on CTA1's bar, CTA1 answers on CTA0's bar
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(32) hop_cluster(int iters, unsigned long long* stats) {
    __shared__ __align__(8) uint64_t bar[1];
    uint32_t rank; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    if (threadIdx.x == 0) { binit(&bar[0], 1); asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (threadIdx.x == 0) {
        int ok = 1;
        long long c0 = clock64();
        for (int it = 0; it < iters && ok; ++it) {
            if (rank == 0) { arrive_remote(smem_u32(&bar[0]), 1); ok = wait_cl(smem_u32(&bar[0]), it & 1); }
            else { ok = wait_cl(smem_u32(&bar[0]), it & 1); arrive_remote(smem_u32(&bar[0]), 0); }
        }
        if (rank == 0) { stats[0] = (unsigned long long)(clock64() - c0); stats[1] = ok; }
    }
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// bulk load latency: one thread issues a cp.async.bulk of `bytes` and waits, serially; src walks a buffer (L2-resident after first pass)
__global__ void __launch_bounds__(32) bulk_lat(const uint8_t* src, size_t span, int bytes, int iters, int depth, unsigned long long* stats) {
    extern __shared__ uint8_t raw[];
    uint8_t* sm = (uint8_t*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t bar[8];
    if (threadIdx.x == 0) { for (int i = 0; i < 8; ++i) binit(&bar[i], 1); asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
    __syncthreads();
    if (threadIdx.x == 0) {
        int ok = 1;
        size_t off = (size_t)blockIdx.x * 1048576 % span;
        long long c0 = clock64();
        for (int it = 0; it < iters + depth && ok; ++it) {
            const int s = it % depth;
            if (it >= depth) ok = wait(smem_u32(&bar[s]), ((it / depth) - 1) & 1);
            if (it < iters) {
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&bar[s])), "r"((uint32_t)bytes) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(smem_u32(sm + s * bytes)), "l"(src + off), "r"((uint32_t)bytes), "r"(smem_u32(&bar[s])) : "memory");
                off += bytes; if (off + bytes > span) off = 0;
            }
        }
        if (blockIdx.x == 0) { stats[0] = (unsigned long long)(clock64() - c0); stats[1] = ok; }
    }
}
// ld.shared 16B + tcgen05.st x4 + wait::st round, by 4 warps
__global__ void __launch_bounds__(128) st_lat(int iters, unsigned long long* stats) {
    __shared__ uint32_t tmem_slot;
    __shared__ __align__(16) uint32_t buf[2048];
    const int tid = threadIdx.x, warp = tid >> 5;
    for (int i = tid; i < 2048; i += 128) buf[i] = i;
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_slot + ((uint32_t)(warp * 32) << 16);
    long long c0 = clock64();
    for (int it = 0; it < iters; ++it) {
        uint32_t v[4];
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(smem_u32(&buf[(tid * 4 + it * 16) & 2047])) : "memory");
#pragma unroll
        for (int q = 0; q < 3; ++q)
            asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(tmem + 256 + q * 4), "r"(v[0] + q), "r"(v[1]), "r"(v[2]), "r"(v[3]) : "memory");
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    }
    if (tid == 0) { stats[0] = (unsigned long long)(clock64() - c0); stats[1] = 1; }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_slot), "r"(512u) : "memory");
}
int main() {
    unsigned long long* d; CK(cudaMalloc(&d, 64)); unsigned long long h[2];
    auto rd = [&]() { CK(cudaDeviceSynchronize()); CK(cudaMemcpy(h, d, 16, cudaMemcpyDeviceToHost)); };
    CK(cudaFuncSetAttribute(commit_lat, cudaFuncAttributeMaxDynamicSharedMemorySize, 51200));
    for (int depth : {1, 2, 3, 4, 6}) {
        const int iters = 4000;
        for (int r = 0; r < 2; ++r) { commit_lat<<<1, 128, 51200>>>(iters, depth, d); rd(); }
        printf("commit chain depth %d: %.1f cycles per group of 4 MMAs (ideal 512) ok=%llu\n", depth, (double)h[0] / iters, h[1]);
    }
    for (int r = 0; r < 2; ++r) { hop_local<<<1, 64>>>(20000, d); rd(); }
    printf("local barrier ping-pong: %.1f cycles per round trip ok=%llu\n", (double)h[0] / 20000, h[1]);
    for (int r = 0; r < 2; ++r) { hop_cluster<<<2, 32>>>(20000, d); rd(); }
    printf("cluster barrier ping-pong: %.1f cycles per round trip ok=%llu\n", (double)h[0] / 20000, h[1]);
    uint8_t* src; const size_t span = 64u << 20; CK(cudaMalloc(&src, span)); CK(cudaMemset(src, 1, span));
    CK(cudaFuncSetAttribute(bulk_lat, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    for (int grid : {1, 148}) for (int bytes : {512, 16384, 32768}) for (int depth : {1, 2, 4}) {
        if (bytes * depth > 190 * 1024) continue;
        const int iters = 2000;
        for (int r = 0; r < 2; ++r) { bulk_lat<<<grid, 32, 200 * 1024>>>(src, span, bytes, iters, depth, d); rd(); }
        printf("bulk load grid=%3d bytes=%5d depth=%d: %.1f cycles per load  (%.1f B/cycle/SM) ok=%llu\n", grid, bytes, depth, (double)h[0] / iters, bytes * (double)iters / h[0], h[1]);
    }
    for (int r = 0; r < 2; ++r) { st_lat<<<1, 128>>>(5000, d); rd(); }
    printf("ld.shared + 3x tcgen05.st.x4 + wait::st: %.1f cycles per round\n", (double)h[0] / 5000);
    return 0;
}
