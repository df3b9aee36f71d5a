// pair_mma.cu -- tcgen05.mma.cta_group::2 on a cluster of two CTAs: raw rate of 256x256x64 NVFP4 MMAs
// (128 cycles each, like the single-CTA 128x256x64), what polls, votes, clock reads and commits to
// rotating barriers cost when placed between the MMAs (nothing, as long as the issuing warp stays
// converged), and the round trip leader commit -> peer CTA sees it -> remote arrive -> leader (about
// 770 cycles, hidden from a depth of two groups on).
// Build: nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o pair_mma pair_mma.cu
#include <cstdio>
#include <cstdint>
#include <cstdlib>
#include <cuda_runtime.h>
#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e), __LINE__); exit(1);} } while (0)
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t desc_sw128(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3fffu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void mma2(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa, uint32_t sfb, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
                 ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc), "r"(sfa), "r"(sfb) : "memory");
}
__device__ __forceinline__ void commit2(uint32_t bar) {
    asm volatile("{\n\t.reg .b16 m;\n\tmov.b16 m, 3;\n\ttcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n\t}" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void commit2_local(uint32_t bar) {   // arrive only on the leader's own barrier
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
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
template <bool CL>
__device__ __forceinline__ bool waitb(uint32_t bar, uint32_t par) {
    int n = 0;
    while (!(CL ? test_wait_cl(bar, par) : test_wait(bar, par))) if (++n > 50000000) return false;
    return true;
}
__device__ __forceinline__ void arrive_remote(uint32_t bar, uint32_t cta) {
    asm volatile("{\n\t.reg .b32 r;\n\tmapa.shared::cluster.u32 r, %0, %1;\n\tmbarrier.arrive.release.cluster.shared::cluster.b64 _, [r];\n\t}" ::"r"(bar), "r"(cta) : "memory");
}
__device__ __forceinline__ void binit(uint64_t* b, uint32_t n) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(n)); }
__device__ __forceinline__ void csync() { asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// MODE 0: leader issues groups of 4 MMAs + multicast commit, no waits
// MODE 1: depth-D chain: before group it, the leader waits for "ack" of group it-D, where the ack is a remote arrive
//         by a peer warp that saw the multicast commit of that group on its own barrier (plus a local leader warp doing the same)
// MODE 2: depth-D chain on the commit alone (leader waits for its own barrier of group it-D)
template <int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(128) pair_kernel(int iters, int depth, unsigned long long* stats) {
    extern __shared__ uint8_t raw[];
    uint8_t* sm = (uint8_t*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
    __shared__ uint32_t tmem_slot;
    __shared__ __align__(8) uint64_t cbar[8];   // commit targets (both CTAs)
    __shared__ __align__(8) uint64_t abar[8];   // acks (leader)
    uint32_t rank; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int i = tid; i < 4 * 32768 / 4; i += 128) ((uint32_t*)sm)[i] = 0x22222222u;
    if (tid == 0) { for (int i = 0; i < 8; ++i) { binit(&cbar[i], 1); binit(&abar[i], 2); } asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    csync();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_slot;
    for (int c = 0; c < 256; ++c)
        asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(tmem + ((uint32_t)(warp * 32) << 16) + 256 + c), "r"(0x38383838u) : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    csync();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t idesc = (1u << 7) | (1u << 10) | ((uint32_t)(256 >> 3) << 17) | (16u << 24);
    const uint32_t base = smem_u32(sm), c0b = smem_u32(&cbar[0]), a0b = smem_u32(&abar[0]);
    int ok = 1; uint32_t sink = 0;
    if (warp == 0 && rank == 0) {
        int dd = -1;
        long long c0 = clock64();
        for (int it = 0; it < iters && ok; ++it) {
            const int s = it & 3; if (++dd == depth) dd = 0; const int d = dd;
            if (MODE == 1 && it >= depth) ok = waitb<false>(a0b + 8 * d, ((it / depth) - 1) & 1);
            if (MODE == 2 && it >= depth) ok = waitb<false>(c0b + 8 * d, ((it / depth) - 1) & 1);
            if (MODE == 3) sink += test_wait(a0b + 8 * 7, 0);                 // unrelated barrier, never completes
            if (MODE == 4) { uint32_t v; asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a0b + 8 * 7) : "memory"); sink += v; }
            if (MODE == 5) { sink += test_wait(a0b + 8 * 7, 0); sink += test_wait(a0b + 8 * 6, 0); }
            if (MODE == 6) sink += (uint32_t)__all_sync(0xffffffffu, it >= 0);
            if (MODE == 7) sink += (uint32_t)clock64();
            if (MODE == 9) sink += test_wait(c0b, it & 1);                    // the commit target itself, result ignored
            if (MODE == 10) sink += test_wait(c0b + 8 * d, it & 1);
            if (MODE >= 11 && MODE <= 14) {
                // warp-uniform: lane 0 issues through the predicate; polls between the MMAs, consumed afterwards
                const uint64_t a0 = desc_sw128(base + s * 32768), b0 = desc_sw128(base + s * 32768 + 16384);
                const uint32_t sfa = tmem + 256 + s * 48, sfb = sfa + 16;
                uint32_t r1 = 1, r2 = 1;
                if (lane == 0) mma2(tmem, a0, b0, idesc, sfa, sfb, it ? 1u : 0u);
                if (MODE == 11 || MODE == 13) r1 = test_wait(a0b + 8 * 7, 1);
                if (lane == 0) mma2(tmem, a0 + 2, b0 + 2, idesc, sfa + 4, sfb + 8, 1u);
                if (MODE == 11 || MODE == 13) r2 = test_wait(a0b + 8 * 6, 1);
                if (lane == 0) mma2(tmem, a0 + 4, b0 + 4, idesc, sfa + 8, sfb + 16, 1u);
                if (lane == 0) mma2(tmem, a0 + 6, b0 + 6, idesc, sfa + 12, sfb + 24, 1u);
                if (lane == 0) commit2(c0b + 8 * (it & 3));
                if (MODE == 12) { r1 = test_wait(a0b + 8 * 7, 1); r2 = test_wait(a0b + 8 * 6, 1); }
                if (MODE == 14) { if (it >= 4) ok = waitb<false>(c0b + 8 * (it & 3), ((it >> 2) - 1) & 1); }   // poll consumed BEFORE this group's MMAs would be mode 2; here after
                if (MODE == 13) { if (!__all_sync(0xffffffffu, r1 && r2)) ok = 0; }
                else if (!(r1 && r2)) ok = 0;
            } else
            if (lane == 0) {
                const uint64_t a0 = desc_sw128(base + s * 32768), b0 = desc_sw128(base + s * 32768 + 16384);
                const uint32_t sfa = tmem + 256 + s * 48, sfb = sfa + 16;
#pragma unroll
                for (int j = 0; j < 4; ++j) mma2(tmem, a0 + 2 * j, b0 + 2 * j, idesc, sfa + 4 * j, sfb + 8 * j, (it | j) ? 1u : 0u);
                commit2(c0b + 8 * ((MODE == 0 || MODE == 9 || (MODE >= 3 && MODE <= 7)) ? 0 : (MODE == 8 ? (it & 3) : d)));
            }
            __syncwarp();
        }
        long long c1 = clock64();
        if (lane == 0) {
            commit2_local(c0b + 8 * 7);
            ok &= waitb<false>(c0b + 8 * 7, 0);
            stats[0] = (unsigned long long)(clock64() - c0); stats[1] = ok + (sink & 0); stats[2] = (unsigned long long)(c1 - c0);
        }
    } else if (warp == 1 && MODE == 1) {
        // ack warp in both CTAs: sees commit of group it on its own barrier, arrives on the leader's ack barrier
        if (lane == 0)
            for (int it = 0; it < iters && ok; ++it) {
                const int d = it % depth;
                ok = waitb<true>(c0b + 8 * d, (it / depth) & 1);
                arrive_remote(a0b + 8 * d, 0);
            }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    csync();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
}
template <int MODE>
void run(const char* name, int grid, int depth, unsigned long long* d) {
    unsigned long long h[3]; const int iters = 4000;
    CK(cudaFuncSetAttribute(pair_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 140 * 1024));
    for (int r = 0; r < 2; ++r) { pair_kernel<MODE><<<grid, 128, 140 * 1024>>>(iters, depth, d); CK(cudaDeviceSynchronize()); CK(cudaMemcpy(h, d, 24, cudaMemcpyDeviceToHost)); }
    printf("%s grid=%d depth=%d: %.1f cycles per group of 4 pair-MMAs (issue loop %.1f) ok=%llu\n", name, grid, depth, (double)h[0] / iters, (double)h[2] / iters, h[1]);
}
int main() {
    unsigned long long* d; CK(cudaMalloc(&d, 64));
    run<0>("pair MMA, no waits", 2, 1, d);
    run<0>("pair MMA, no waits", 148, 1, d);
    run<8>("pair MMA, commits rotate over 4 barriers", 2, 1, d);
    run<9>("pair MMA, one commit barrier, polled", 2, 1, d);
    run<10>("pair MMA, rotating commit barriers, polled", 2, 4, d);
    run<11>("polls between MMAs, consumed after the group", 2, 1, d);
    run<12>("polls after the commit, consumed at once", 2, 1, d);
    run<13>("polls between MMAs, vote, consumed", 2, 1, d);
    run<14>("blocking wait on own commit 4 groups back, after the group", 2, 1, d);
    run<3>("pair MMA + dummy test_wait", 2, 1, d);
    run<4>("pair MMA + dummy ld.shared", 2, 1, d);
    run<5>("pair MMA + 2 dummy test_wait", 2, 1, d);
    run<6>("pair MMA + vote", 2, 1, d);
    run<7>("pair MMA + clock64", 2, 1, d);
    for (int depth : {1, 2, 3, 4, 6}) run<2>("pair MMA, wait own commit", 2, depth, d);
    for (int depth : {1, 2, 3, 4, 6}) run<1>("pair MMA, wait acks of both CTAs", 2, depth, d);
    return 0;
}
