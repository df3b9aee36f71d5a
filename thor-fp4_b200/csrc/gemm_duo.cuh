// gemm_duo.cuh -- the large-batch NVFP4 GEMM: a cluster of two CTAs computes a 256-token x
// 256-feature tile with tcgen05.mma.cta_group::2.  Included by gemm.cu inside its anonymous
// namespace, after the single-CTA kernel and its PTX wrappers.
//
// Why this shape.  Measured on B200: one 128x256x64 NVFP4 MMA takes 128 cycles whatever feeds it
// (and one 256x256x64 MMA of a CTA pair the same 128), a barrier hop inside a CTA costs ~180
// cycles, a hop between the CTAs of a cluster ~550, an L2-resident 16 KB TMA load ~650, and all
// SMs together pull ~85 bytes per cycle and SM out of L2.  A single CTA with a 128x256 tile needs
// 105 bytes per cycle and has room for three 54 KB stages, i.e. 1000 cycles of cover for a
// 1700-cycle refill chain: it is bound by both.  Here each CTA loads only its own 128 token rows
// and its own 128 of the 256 feature rows per K block (32 KB, 64 bytes per cycle at full MMA
// rate), and five stages fit: 2000 cycles of cover.
//
// Orientation.  Tokens are the MMA's M side (lane of the accumulator), features its N side
// (column): a thread of the epilogue holds consecutive features of one token, i.e. a contiguous
// piece of an output row.
//
//   warp 0      producer, both CTAs: per K block two TMA loads (own tokens, own feature half)
//   warp 1      leader: MMA issuer.  peer: relays "my operands landed" to the leader's barrier
//   warps 2-5,  epilogue, two warps per tensor-memory lane quarter (columns 0-127 and 128-255):
//   11-14       tcgen05.ld 32 columns -> alpha, bias, cast -> swizzled shared memory -> one TMA store
//               per warp and 32 rows x 128 bytes of the output (32 f32 or 64 16-bit columns); the accumulator is handed back as soon as a
//               warp's last columns are in registers (fma + convert + st.shared of a 128 x 256 tile
//               take one warp per quarter ~2200 cycles, which no MMA can overlap)
//   warps 6-9   scale loaders: scale atoms of two K blocks at a time, shared memory ->
//               registers -> tcgen05.st into the scale slots of tensor memory
//   warp 10     scale producer: bulk copies of the scale atoms, two K blocks per copy, running
//               ahead of the operand pipeline
// Barriers.  full[s] (leader: own bytes + the peer's relay + the 8 loader warps of both CTAs, i.e. "operands landed and
// scales in tensor memory" is ONE barrier and one poll per K block for the MMA issuer - two barriers and two polls cost
// 2 % at 8192^3; peer: own bytes), empty[s] / tfull: local in each CTA, signalled by the leader's tcgen05.commit with a
// two-CTA mask.  sfl[i]: scale atoms landed (local).  sfree[i]: the four loader warps have read scale stage i (local).
// tempty: 16 arrivals (8 epilogue warps of each CTA).  Every wait is bounded.
// The MMA issuer polls with mbarrier.test_wait; every other warp waits with try_wait, which parks
// the warp: ten warps spinning on shared-memory barriers slow the issuer's own polls down.  Arrivals on the other CTA's barriers are
// relaxed: a releasing arrive at cluster scope first waits for everything its thread has in
// flight (bulk copies, global stores), measured at 500-1200 cycles per arrival.

constexpr int DUO_THREADS = 480;
// NVFP4 main loop: operand descriptors and scale addresses of every stage precomputed outside the tile loop (0.7 % at
// 8192^3 against re-deriving them in every K block's statement)
constexpr bool DUO_PRE = true;

struct DuoCfg {
    static constexpr int TILE_M = 256, TILE_N = 256;
    static constexpr int OP_STAGES = 5;
    static constexpr int X_BYTES = 128 * KB_BYTES;            // own token rows, one K block
    static constexpr int W_BYTES = 128 * KB_BYTES;            // own half of the feature rows
    static constexpr int SF_STAGES = 2;                       // each holds the scales of two K blocks
    static constexpr int SF_PART = 8 * 512;                   // the scale atoms of 128 rows for two K blocks
    static constexpr int SF_STAGE_BYTES = 3 * SF_PART;        // own tokens, feature rows 0-127, feature rows 128-255
    static constexpr int NSLOT = 5;                           // scale slots in tensor memory: one per operand stage
    static constexpr int SF_COL = 256;                        // behind the 256 accumulator columns
    static constexpr int EPI_BUF = 32 * 128;                  // per epilogue warp: 32 rows x 128 bytes
    static constexpr int EPI_BYTES = 8 * EPI_BUF;             // eight epilogue warps
    static constexpr int BAR_BYTES = 512;
    static constexpr int SMEM_BYTES =
        OP_STAGES * (X_BYTES + W_BYTES) + EPI_BYTES + SF_STAGES * SF_STAGE_BYTES + BAR_BYTES + 1024;
    static constexpr uint32_t IDESC = (1u << 7) | (1u << 10) | ((uint32_t)(TILE_N >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
    // MXFP8 tokens (A operand, e4m3 = 0 at bit 7) x MXFP4 weights (B operand, e2m1 = 5 at bit 10), UE8M0 scales (bit 23);
    // MMA j of a K block takes scale byte j of the 32-bit scale columns (ids at bits 29 and 4)
    static constexpr uint32_t IDESC_MX = (0u << 7) | (5u << 10) | ((uint32_t)(TILE_N >> 3) << 17) | (1u << 23) | ((uint32_t)(256 >> 4) << 24);
    static constexpr uint32_t IDESC_MX1 = IDESC_MX | (1u << 29) | (1u << 4);
    static constexpr uint32_t IDESC_MX2 = IDESC_MX | (2u << 29) | (2u << 4);
    static constexpr uint32_t IDESC_MX3 = IDESC_MX | (3u << 29) | (3u << 4);
    static_assert(SF_COL + NSLOT * TMEM_SF_SLOT_COLS <= TMEM_COLS, "scale slots do not fit");
    static_assert(NSLOT == OP_STAGES, "K block i uses operand stage and scale slot i % OP_STAGES alike");
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory");
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void tc_mma_pair_nvf4(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                 uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
}
// arrives on the barrier at this shared-memory offset in both CTAs once all earlier MMAs are done
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    asm volatile(
        "{\n\t.reg .b16 m;\n\tmov.b16 m, 3;\n\t"
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n\t}"
        ::"r"(bar) : "memory");
}
// Remote arrival without a release fence.  What the arrival publishes is already complete when
// it is made - a TMA transfer whose barrier the thread has seen flip, tensor-memory stores after
// tcgen05.wait::st, tensor-memory loads after tcgen05.wait::ld - so no fence is needed.
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Waiting with a long suspend hint: the warp sleeps in hardware until the phase completes (or the
// hint, in nanoseconds, runs out) instead of re-issuing polls that compete with the MMA issuer
// for the shared-memory instruction queue of their SM partition.  Bounded like every other wait.
__device__ __forceinline__ bool mbar_wait_sleep(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code,
                                                long long limit = WAIT_CYCLES) {
    const long long t0 = clock64();
    for (uint32_t it = 0;; ++it) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity), "r"(20000u)
            : "memory");
        if (ok) return true;
        if ((it & 7u) == 7u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > limit) {
                *abort_flag = code;
                return false;
            }
        }
    }
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int x, int y, uint32_t src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(map), "r"(x), "r"(y), "r"(src) : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// at most one of this thread's bulk-store groups may still be reading shared memory
__device__ __forceinline__ void bulk_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// two FP32 fused multiply-adds in one instruction (the epilogue's arithmetic is bound by the
// throughput of its SM partition, not by latency: fewer instructions is what helps)
__device__ __forceinline__ void fma2(float& d0, float& d1, float a0, float a1, float b, float c0, float c1) {
    uint64_t av, bv, cv, dv;
    asm("mov.b64 %0, {%1, %2};" : "=l"(av) : "f"(a0), "f"(a1));
    asm("mov.b64 %0, {%1, %1};" : "=l"(bv) : "f"(b));
    asm("mov.b64 %0, {%1, %2};" : "=l"(cv) : "f"(c0), "f"(c1));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(dv) : "l"(av), "l"(bv), "l"(cv));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d0), "=f"(d1) : "l"(dv));
}
// 32 accumulator columns of one token row -> alpha, bias -> floats
__device__ __forceinline__ void duo_scale(const uint32_t (&v)[32], float (&f)[32], int64_t n, int64_t N, float alpha,
                                          const float* bias) {
    if (bias != nullptr) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
            float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
            if (n + i + 4 <= N) b = __ldg(reinterpret_cast<const float4*>(bias + n + i));
            fma2(f[i], f[i + 1], __uint_as_float(v[i]), __uint_as_float(v[i + 1]), alpha, b.x, b.y);
            fma2(f[i + 2], f[i + 3], __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]), alpha, b.z, b.w);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; i += 2)
            fma2(f[i], f[i + 1], __uint_as_float(v[i]), __uint_as_float(v[i + 1]), alpha, 0.f, 0.f);
    }
}
// 32 columns as 16-bit values: four 16-byte chunks of a 128-byte row, chunk index XOR (row & 7)
// (the 128-byte swizzle the TMA store expects)
__device__ __forceinline__ void duo_put16(const float (&f)[32], uint32_t row_addr, int chunk0, int row, bool bf16) {
    uint32_t h[16];
    if (bf16) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            __nv_bfloat162 t = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
            h[i] = *reinterpret_cast<uint32_t*>(&t);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            __half2 t = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
            h[i] = *reinterpret_cast<uint32_t*>(&t);
        }
    }
#pragma unroll
    for (int c = 0; c < 4; ++c)
        st_shared_v4(row_addr + (uint32_t)(((chunk0 + c) ^ (row & 7)) << 4), h[4 * c], h[4 * c + 1], h[4 * c + 2], h[4 * c + 3]);
}
__device__ __forceinline__ void duo_put32(const float (&f)[32], uint32_t row_addr, int row) {
#pragma unroll
    for (int c = 0; c < 8; ++c)
        st_shared_v4(row_addr + (uint32_t)((c ^ (row & 7)) << 4), __float_as_uint(f[4 * c]), __float_as_uint(f[4 * c + 1]),
                     __float_as_uint(f[4 * c + 2]), __float_as_uint(f[4 * c + 3]));
}

// One K block of the two-CTA MMA stream in a single statement: up to four MMAs (K = 64 each,
// operands 32 bytes further into the 128-byte swizzle span each time, so only the low descriptor
// word changes), the look-ahead polls of the next K block's two barriers between them, the commit
// that frees the stage in both CTAs and, after a tile's last K block, the commit that hands the
// accumulator to the epilogue.  The issuing warp is a single thread of control, four to five cycles
// per dependent instruction and about fifteen per branch, and the tensor pipe runs only about one
// MMA ahead of it: whatever the warp executes per K block beyond ~500 cycles is lost MMA time, so
// nothing is recomputed or branched on here that the caller can hand over in a register.
// n_mma: MMAs to issue (4, or fewer in a ragged last K block).  Returns 1 if both polled barriers
// had completed the polled phase.
__device__ __forceinline__ uint32_t duo_kblock(uint32_t on, uint32_t accumulate, uint32_t n_mma, uint32_t last,
                                               uint32_t d, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t sf,
                                               uint32_t full_next, uint32_t par_next,
                                               uint32_t empty_bar, uint32_t tfull_bar) {
    uint32_t ready;
    asm volatile(
        "{\n\t"
        ".reg .pred q, q0, q1, q2, q3, ql, pa, pt, pf;\n\t"
        ".reg .b16 m;\n\t"
        ".reg .b32 a1, a2, a3, b1, b2, b3, f1, f2, f3, g0, g1, g2, g3;\n\t"
        ".reg .b64 da0, da1, da2, da3, db0, db1, db2, db3;\n\t"
        "setp.ne.b32 q, %1, 0;\n\t"
        "setp.ne.b32 pa, %2, 0;\n\t"
        "setp.gt.and.u32 q0, %3, 0, q;\n\t"
        "setp.gt.and.u32 q1, %3, 1, q;\n\t"
        "setp.gt.and.u32 q2, %3, 2, q;\n\t"
        "setp.gt.and.u32 q3, %3, 3, q;\n\t"
        "setp.ne.and.b32 ql, %4, 0, q;\n\t"
        "setp.eq.b32 pt, 0, 0;\n\t"
        "mov.b16 m, 3;\n\t"
        "add.u32 a1, %6, 2;\n\tadd.u32 a2, %6, 4;\n\tadd.u32 a3, %6, 6;\n\t"
        "add.u32 b1, %7, 2;\n\tadd.u32 b2, %7, 4;\n\tadd.u32 b3, %7, 6;\n\t"
        "mov.b64 da0, {%6, %8};\n\tmov.b64 da1, {a1, %8};\n\tmov.b64 da2, {a2, %8};\n\tmov.b64 da3, {a3, %8};\n\t"
        "mov.b64 db0, {%7, %8};\n\tmov.b64 db1, {b1, %8};\n\tmov.b64 db2, {b2, %8};\n\tmov.b64 db3, {b3, %8};\n\t"
        "add.u32 f1, %9, 4;\n\tadd.u32 f2, %9, 8;\n\tadd.u32 f3, %9, 12;\n\t"
        "add.u32 g0, %9, 16;\n\tadd.u32 g1, %9, 24;\n\tadd.u32 g2, %9, 32;\n\tadd.u32 g3, %9, 40;\n\t"
        "@q0 tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%5], da0, db0, %14, [%9], [g0], pa;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 pf, [%10], %11;\n\t"
        "@q1 tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%5], da1, db1, %14, [f1], [g1], pt;\n\t"
        "@q2 tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%5], da2, db2, %14, [f2], [g2], pt;\n\t"
        "@q3 tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%5], da3, db3, %14, [f3], [g3], pt;\n\t"
        "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%12], m;\n\t"
        "@ql tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%13], m;\n\t"
        "selp.u32 %0, 1, 0, pf;\n\t"
        "}"
        : "=r"(ready)
        : "r"(on), "r"(accumulate), "r"(n_mma), "r"(last), "r"(d), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(sf),
          "r"(full_next), "r"(par_next), "r"(empty_bar), "r"(tfull_bar), "n"(DuoCfg::IDESC)
        : "memory");
    return ready;
}

// duo_kblock with every address handed over: the low descriptor words of the four MMAs' operands and the eight scale
// addresses are loop-invariant per stage, so the caller keeps them in registers instead of this statement re-deriving
// them (13 additions) for every K block.
__device__ __forceinline__ uint32_t duo_kblock_pre(uint32_t on, uint32_t accumulate, uint32_t n_mma, uint32_t last, uint32_t d,
                                                   const uint32_t (&a)[4], const uint32_t (&b)[4], uint32_t desc_hi,
                                                   const uint32_t (&sfa)[4], const uint32_t (&sfb)[4],
                                                   uint32_t full_next, uint32_t par_next,
                                                   uint32_t empty_bar, uint32_t tfull_bar) {
    uint32_t ready;
    asm volatile(
        "{\n\t"
        ".reg .pred q, q0, q1, q2, q3, ql, pa, pt, pf;\n\t"
        ".reg .b16 m;\n\t"
        ".reg .b64 da0, da1, da2, da3, db0, db1, db2, db3;\n\t"
        "setp.ne.b32 q, %1, 0;\n\t"
        "setp.ne.b32 pa, %2, 0;\n\t"
        "setp.gt.and.u32 q0, %3, 0, q;\n\t"
        "setp.gt.and.u32 q1, %3, 1, q;\n\t"
        "setp.gt.and.u32 q2, %3, 2, q;\n\t"
        "setp.gt.and.u32 q3, %3, 3, q;\n\t"
        "setp.ne.and.b32 ql, %4, 0, q;\n\t"
        "setp.eq.b32 pt, 0, 0;\n\t"
        "mov.b16 m, 3;\n\t"
        "mov.b64 da0, {%6, %14};\n\tmov.b64 da1, {%7, %14};\n\tmov.b64 da2, {%8, %14};\n\tmov.b64 da3, {%9, %14};\n\t"
        "mov.b64 db0, {%10, %14};\n\tmov.b64 db1, {%11, %14};\n\tmov.b64 db2, {%12, %14};\n\tmov.b64 db3, {%13, %14};\n\t"
        "@q0 tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%5], da0, db0, %27, [%15], [%19], pa;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 pf, [%23], %24;\n\t"
        "@q1 tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%5], da1, db1, %27, [%16], [%20], pt;\n\t"
        "@q2 tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%5], da2, db2, %27, [%17], [%21], pt;\n\t"
        "@q3 tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%5], da3, db3, %27, [%18], [%22], pt;\n\t"
        "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%25], m;\n\t"
        "@ql tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%26], m;\n\t"
        "selp.u32 %0, 1, 0, pf;\n\t"
        "}"
        : "=r"(ready)
        : "r"(on), "r"(accumulate), "r"(n_mma), "r"(last), "r"(d),
          "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]), "r"(b[2]), "r"(b[3]), "r"(desc_hi),
          "r"(sfa[0]), "r"(sfa[1]), "r"(sfa[2]), "r"(sfa[3]), "r"(sfb[0]), "r"(sfb[1]), "r"(sfb[2]), "r"(sfb[3]),
          "r"(full_next), "r"(par_next), "r"(empty_bar), "r"(tfull_bar), "n"(DuoCfg::IDESC)
        : "memory");
    return ready;
}

// The same for MXFP8 tokens x MXFP4 weights: four kind::mxf8f6f4 MMAs of K = 32, one scale byte per row and MMA
// (byte j of the K block's 32-bit scale columns, selected in the instruction descriptor and in the top bits of
// the scale address).
__device__ __forceinline__ uint32_t duo_kblock_mx(uint32_t on, uint32_t accumulate, uint32_t n_mma, uint32_t last,
                                                  uint32_t d, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t sf,
                                                  uint32_t full_next, uint32_t par_next,
                                                  uint32_t empty_bar, uint32_t tfull_bar) {
    uint32_t ready;
    asm volatile(
        "{\n\t"
        ".reg .pred q, q0, q1, q2, q3, ql, pa, pt, pf;\n\t"
        ".reg .b16 m;\n\t"
        ".reg .b32 a1, a2, a3, b1, b2, b3, f1, f2, f3, g0, g1, g2, g3;\n\t"
        ".reg .b64 da0, da1, da2, da3, db0, db1, db2, db3;\n\t"
        "setp.ne.b32 q, %1, 0;\n\t"
        "setp.ne.b32 pa, %2, 0;\n\t"
        "setp.gt.and.u32 q0, %3, 0, q;\n\t"
        "setp.gt.and.u32 q1, %3, 1, q;\n\t"
        "setp.gt.and.u32 q2, %3, 2, q;\n\t"
        "setp.gt.and.u32 q3, %3, 3, q;\n\t"
        "setp.ne.and.b32 ql, %4, 0, q;\n\t"
        "setp.eq.b32 pt, 0, 0;\n\t"
        "mov.b16 m, 3;\n\t"
        "add.u32 a1, %6, 2;\n\tadd.u32 a2, %6, 4;\n\tadd.u32 a3, %6, 6;\n\t"
        "add.u32 b1, %7, 2;\n\tadd.u32 b2, %7, 4;\n\tadd.u32 b3, %7, 6;\n\t"
        "mov.b64 da0, {%6, %8};\n\tmov.b64 da1, {a1, %8};\n\tmov.b64 da2, {a2, %8};\n\tmov.b64 da3, {a3, %8};\n\t"
        "mov.b64 db0, {%7, %8};\n\tmov.b64 db1, {b1, %8};\n\tmov.b64 db2, {b2, %8};\n\tmov.b64 db3, {b3, %8};\n\t"
        "or.b32 f1, %9, 0x40000000;\n\tor.b32 f2, %9, 0x80000000;\n\tor.b32 f3, %9, 0xC0000000;\n\t"
        "add.u32 g0, %9, 16;\n\tor.b32 g1, g0, 0x40000000;\n\tor.b32 g2, g0, 0x80000000;\n\tor.b32 g3, g0, 0xC0000000;\n\t"
        "@q0 tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%5], da0, db0, %14, [%9], [g0], pa;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 pf, [%10], %11;\n\t"
        "@q1 tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%5], da1, db1, %15, [f1], [g1], pt;\n\t"
        "@q2 tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%5], da2, db2, %16, [f2], [g2], pt;\n\t"
        "@q3 tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%5], da3, db3, %17, [f3], [g3], pt;\n\t"
        "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%12], m;\n\t"
        "@ql tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%13], m;\n\t"
        "selp.u32 %0, 1, 0, pf;\n\t"
        "}"
        : "=r"(ready)
        : "r"(on), "r"(accumulate), "r"(n_mma), "r"(last), "r"(d), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(sf),
          "r"(full_next), "r"(par_next), "r"(empty_bar), "r"(tfull_bar), "n"(DuoCfg::IDESC_MX),
          "n"(DuoCfg::IDESC_MX1), "n"(DuoCfg::IDESC_MX2), "n"(DuoCfg::IDESC_MX3)
        : "memory");
    return ready;
}

// Tile index -> (token tile mt, feature tile nt).  gm <= 0: token tiles fastest (a wave of CTA pairs shares few weight
// tiles and spreads over many token tiles).  gm > 0: bands of gm token tiles, feature tiles fastest inside a band, so a
// wave covers about gm x (pairs / gm) tiles and every operand tile in flight is shared by several pairs.
// m_shift rotates the token tiles (mt -> (mt + m_shift) mod tiles_m): the push epilogue gives every rank a different
// rotation, so that at any time the ranks store into different owners' memory instead of all into the same one.
__device__ __forceinline__ void duo_tile_coords(int64_t tile, int64_t tiles_m, int64_t tiles_n, int gm, int64_t m_shift,
                                                int64_t& mt, int64_t& nt) {
    if (gm <= 0) {
        nt = tile / tiles_m;
        mt = tile - nt * tiles_m;
    } else {
        const int64_t band = (int64_t)gm * tiles_n;
        const int64_t g = tile / band, r = tile - g * band;
        const int64_t m0 = g * gm;
        const int64_t rows = (tiles_m - m0 < gm) ? (tiles_m - m0) : gm;
        nt = r / rows;
        mt = m0 + (r - nt * rows);
    }
    mt += m_shift;
    if (mt >= tiles_m) mt -= tiles_m;
}

template <int V> struct IntTag { static constexpr int value = V; };

// One 32-column chunk of the SwiGLU epilogue: columns 0-15 are gate features j..j+15, columns 16-31 the matching up
// features.  h = silu(alpha * gate) * (alpha * up) in FP32 (reproducible silu, det_math.cuh), then the activation
// quantizer's block arithmetic with per-tensor scale 1: sc = ue4m3(amax * (1/6)), codes = e2m1_ties_up(h / dec(sc))
// through the bracketed reciprocal path of quant_block.cuh.  lo / hi: the codes of h[0..7] / h[8..15].
__device__ __forceinline__ void swiglu_block16(const uint32_t (&v)[32], float alpha, uint32_t& lo, uint32_t& hi, uint32_t& sc) {
    float h0[8], h1[8];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        h0[i] = __fmul_rn(det_silu(__fmul_rn(alpha, __uint_as_float(v[i]))), __fmul_rn(alpha, __uint_as_float(v[16 + i])));
        h1[i] = __fmul_rn(det_silu(__fmul_rn(alpha, __uint_as_float(v[8 + i]))), __fmul_rn(alpha, __uint_as_float(v[24 + i])));
        amax = fmaxf(amax, fmaxf(fabsf(h0[i]), fabsf(h1[i])));
    }
    sc = f32x2_to_e4m3x2(__fmul_rn(amax, 1.0f / 6.0f), 0.f) & 0x7fu;
    const float ds = e4m3_to_f32(sc);
    lo = block_codes8<1>(h0, ds);
    hi = block_codes8<1>(h1, ds);
}

// One 32-column chunk of the MXFP8 epilogue = one MX block: y = act(alpha * acc + bias[n]) (act 0 identity, 1 gelu,
// 2 silu; reproducible forms), block scale byte = the power of two at or above amax * (1/448), codes = e4m3(y / 2^e)
// (an exact scaling).  bias: this chunk's 32 floats or null.  w: 32 code bytes.
__device__ __forceinline__ void act_mx8_block32(const uint32_t (&v)[32], float alpha, const float* bias, int act,
                                                uint32_t (&w)[8], uint32_t& scb) {
    float y[32];
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
        float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
        if (bias != nullptr) b = __ldg(reinterpret_cast<const float4*>(bias + i));
        const float bb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float t = __fmul_rn(alpha, __uint_as_float(v[i + j]));
            if (bias != nullptr) t = __fadd_rn(t, bb[j]);
            y[i + j] = t;
        }
    }
    if (act == 1) {
#pragma unroll
        for (int i = 0; i < 32; ++i) y[i] = det_gelu(y[i]);
    } else if (act == 2) {
#pragma unroll
        for (int i = 0; i < 32; ++i) y[i] = det_silu(y[i]);
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(y[i]));
    // power of two at or above amax / 448 (csrc/thor_fp4_core.cu:612-619 of the reference project)
    const float a = __fmul_rn(amax, 1.0f / 448.0f);
    uint32_t sb = 0u;
    if (a > 0.f) {
        const uint32_t u = __float_as_uint(a);
        if ((u >> 23) == 0u) sb = (u > 0x00400000u) ? 1u : 0u;
        else sb = (u >> 23) + ((u & 0x007fffffu) ? 1u : 0u);
        if (sb > 254u) sb = 254u;
    }
    scb = sb;
    const int e = 127 - (int)sb;
    const float inv = e >= -126 ? __uint_as_float((uint32_t)(e + 127) << 23) : __uint_as_float(0x00400000u);
#pragma unroll
    for (int i = 0; i < 8; ++i)
        w[i] = f32x4_to_e4m3x4(__fmul_rn(y[4 * i], inv), __fmul_rn(y[4 * i + 1], inv), __fmul_rn(y[4 * i + 2], inv),
                               __fmul_rn(y[4 * i + 3], inv));
}

// KIND 0: NVFP4 x NVFP4 (256 elements of K per K block, four scale atoms per 128 rows and K block);
// KIND 1: MXFP8 tokens x MXFP4 weights (128 elements per K block, one atom; the 4-bit weights are expanded by TMA
// to one byte per code in shared memory, and that copy credits its packed size to the barrier).
//
// EPI selects what the epilogue makes of the FP32 accumulator (a thread holds 32 consecutive features of one token):
//   0  out = cast(alpha * acc + bias) through shared memory and TMA stores;
//   1  SwiGLU + NVFP4: the weight rows alternate in blocks of 16 (16 gate features, the 16 matching up features), so a
//      32-column chunk is one 16-element quantization block of h = silu(alpha * gate) * (alpha * up); the thread
//      quantizes it with the activation quantizer's arithmetic (per-tensor scale 1) and stores the e2m1 codes and
//      UE4M3 scale bytes straight into the A-operand buffers of the next GEMM - no [M, 2I] tensor reaches memory;
//   2  bias + activation + MXFP8: a 32-column chunk is one MX block of act(alpha * acc + bias[n]); e4m3 codes and
//      UE8M0 scale bytes (power of two at or above amax / 448) go to the next layer's A-operand buffers.
//   3  tensor-parallel push: the plain output of mode 0, but every 32-row block of the tile is stored (TMA, over
//      NVLink for a peer) into the staging buffer of the rank that owns those token rows - one tensor map per owner -
//      so the partial products of a row-parallel layer reach their owners while the main loop is still running;
//      a sum over the staged partials completes the reduce-scatter.
constexpr int PUSH_MAX_RANKS = 8;
struct PushMaps { CUtensorMap m[PUSH_MAX_RANKS]; };
template <int EPI> struct DuoOutMaps { using type = CUtensorMap; };
template <> struct DuoOutMaps<3> { using type = PushMaps; };

// the output tensor map of owner o (push epilogue) or the one output map (every other mode)
template <int EPI>
__device__ __forceinline__ const CUtensorMap* duo_push_map(const typename DuoOutMaps<EPI>::type& t, int64_t o) {
    if constexpr (EPI == 3) return &t.m[o];
    else return &t;
}

template <int KIND, bool DBG, int EPI>
__global__ void __launch_bounds__(DUO_THREADS, 1)
gemm_duo_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                const __grid_constant__ typename DuoOutMaps<EPI>::type tmO, const GemmParams p) {
    using C = DuoCfg;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sX = smem;
    uint8_t* sWh = sX + (size_t)C::OP_STAGES * C::X_BYTES;
    uint8_t* sEpi = sWh + (size_t)C::OP_STAGES * C::W_BYTES;
    uint8_t* sSF = sEpi + C::EPI_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sSF + (size_t)C::SF_STAGES * C::SF_STAGE_BYTES);
    uint64_t* full_bar = bars;                               // [OP_STAGES]
    uint64_t* empty_bar = full_bar + C::OP_STAGES;           // [OP_STAGES]
    uint64_t* sfl_bar = empty_bar + C::OP_STAGES;            // [SF_STAGES]
    uint64_t* sfree_bar = sfl_bar + C::SF_STAGES;            // [SF_STAGES]
    uint64_t* tfull_bar = sfree_bar + C::SF_STAGES;          // [1]
    uint64_t* tempty_bar = tfull_bar + 1;                    // [1]          used in the leader
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();                 // 0 = leader
    const bool leader = rank == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::OP_STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), leader ? 10 : 1);      // leader: own bytes, the peer's relay, 8 loader warps
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int s = 0; s < C::SF_STAGES; ++s) {
            mbar_init(smem_u32(&sfl_bar[s]), 1);
            mbar_init(smem_u32(&sfree_bar[s]), 4);
        }
        mbar_init(smem_u32(tfull_bar), 1);
        mbar_init(smem_u32(tempty_bar), 16);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();      // the peer's barriers are initialised before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // everything above touched only this CTA's shared and tensor memory; the operands may still be being
    // written by the kernel before this one (programmatic dependent launch), so wait for it here
    griddep_wait();
    griddep_launch();

    const int64_t tiles_m = (p.M + C::TILE_M - 1) / C::TILE_M;
    const int64_t tiles_n = (p.N + C::TILE_N - 1) / C::TILE_N;
    const int64_t total_tiles = tiles_m * tiles_n;
    const int64_t first = blockIdx.x >> 1, stride = gridDim.x >> 1;
    const int k_blocks = p.k_blocks;
    const int grans = (k_blocks + 1) >> 1;                   // scale granules (two K blocks) per tile
    const uint32_t full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar);
    const uint32_t sfl0 = smem_u32(sfl_bar), sfree0 = smem_u32(sfree_bar);
    // test hooks (tfp4_set_debug) exist only in the DBG instantiation; the production one carries none of their branches
    const int dbg = DBG ? p.debug : 0;
    const bool prof = DBG && (dbg & 1024) != 0;
    // test hook 512: the producer never signals its barriers and every wait gives up after ~10 ms instead of ~1 s,
    // which exercises the give-up path (abort flag, status word, orderly teardown) without hanging anything
    const bool starve = DBG && (dbg & 512) != 0;
    const long long wlim = starve ? 20000000ll : WAIT_CYCLES;
    constexpr int ATOMS = (KIND == 0) ? 4 : 1;               // scale atoms per 128 rows and K block
    constexpr uint32_t TX_BYTES = (KIND == 0) ? (uint32_t)(C::X_BYTES + C::W_BYTES) : (uint32_t)(C::X_BYTES + C::W_BYTES / 2);

    if (warp == 0) {
        // ------------------------------------------------------------ producer (both CTAs)
        // Every role walks the stage ring continuously across tiles and keeps one phase bit per stage,
        // toggled on each use of the stage.
        uint32_t pmask = 0, s = 0;
        bool ok = true;
        long long c_wait = 0;
        const CUtensorMap* my_map = (lane == 0) ? &tmX : &tmW;
        const uint32_t my_dst = (lane == 0) ? smem_u32(sX) : smem_u32(sWh);
        for (int64_t tile = first; tile < total_tiles && ok; tile += stride) {
            int64_t nt, mt;
            duo_tile_coords(tile, tiles_m, tiles_n, p.raster_gm, p.m_shift, mt, nt);
            const int my_y = (lane == 0) ? (int)(mt * C::TILE_M + rank * 128) : (int)(nt * C::TILE_N + rank * 128);
            for (int kb = 0; kb < k_blocks; ++kb) {
                const uint32_t ph = (pmask >> s) & 1u;
                pmask ^= 1u << s;
                const long long t0 = prof ? clock64() : 0;
                if (!mbar_wait_sleep(empty0 + 8 * s, ph ^ 1u, abort_flag, 1, wlim)) { ok = false; break; }
                if (prof) c_wait += clock64() - t0;
                const uint32_t bar = full0 + 8 * s;
                if (starve) {
                    // nothing is signalled: the consumers' waits run out
                } else if (dbg & 8) {
                    if (lane == 0) mbar_arrive(bar);
                } else {
                    // rows or K bytes outside the tensors are zero-filled and still counted in full
                    if (lane == 0) mbar_expect_tx(bar, TX_BYTES);
                    __syncwarp();
                    if (lane < 2) tma_load_2d(my_dst + s * C::X_BYTES, my_map, kb * KB_BYTES, my_y, bar);
                }
                if (++s == C::OP_STAGES) s = 0;
            }
        }
        
        if (!ok && lane == 0) {
            // let copies already issued land before the CTA's shared memory goes away
            const long long t0 = clock64();
            while (clock64() - t0 < 4000000ll) {}
        }
    } else if (warp == 1) {
        if (leader) {
            // -------------------------------------------------------- MMA issuer
            // The warp walks the loop together (uniform control flow keeps the operands in uniform
            // registers); lane 0's instructions are the ones that take effect.  The K loop is unrolled
            // over the five stages, so every address below is a base register plus a constant.  Per K
            // block: one statement with the MMAs, the polls of the next K block's barriers and the
            // commits (duo_kblock); the blocking, bounded wait is only the fallback when a poll failed.
            uint32_t mmask = 0, tcount = 0;                  // phase bit per stage; tiles done
            int s_start = 0;                                 // stage of the tile's first K block
            const uint32_t on = (lane == 0) ? 1u : 0u;
            const uint32_t full_mma = (dbg & 4) ? 0u : 4u;   // test hook: no MMAs, commits only
            bool ok = true, peek = false;
            const uint64_t adesc_base = desc_sw128(smem_u32(sX)), bdesc_base = desc_sw128(smem_u32(sWh));
            const uint32_t desc_hi = (uint32_t)(adesc_base >> 32);
            const uint32_t a_lo0 = (uint32_t)adesc_base, b_lo0 = (uint32_t)bdesc_base;
            const uint32_t sf0 = tmem_base + C::SF_COL;
            const uint32_t tfull_a = smem_u32(tfull_bar);
            const uint32_t last_atoms = (dbg & 4) ? 0u : (uint32_t)p.last_atoms;
            // per stage: the low descriptor words of the four MMAs' operands (32 bytes further into the swizzle span each)
            // and their scale addresses (token scales 4 columns per MMA, feature scales 8)
            uint32_t pre_a[C::OP_STAGES][4], pre_b[C::OP_STAGES][4], pre_sfa[C::OP_STAGES][4], pre_sfb[C::OP_STAGES][4];
#pragma unroll
            for (int u = 0; u < C::OP_STAGES; ++u)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    pre_a[u][j] = a_lo0 + u * (C::X_BYTES >> 4) + 2 * j;
                    pre_b[u][j] = b_lo0 + u * (C::W_BYTES >> 4) + 2 * j;
                    pre_sfa[u][j] = sf0 + u * TMEM_SF_SLOT_COLS + 4 * j;
                    pre_sfb[u][j] = sf0 + u * TMEM_SF_SLOT_COLS + 16 + 8 * j;
                }
            long long c_acc = 0, c_wait = 0, s_obs = 0, s_commit = 0;
            uint32_t n_miss = 0;
            const long long c_begin = clock64();
            for (int64_t tile = first; tile < total_tiles && ok; tile += stride, ++tcount) {
                const long long ta = prof ? clock64() : 0;
                if (!mbar_wait(smem_u32(tempty_bar), (tcount & 1u) ^ 1u, abort_flag, 2, wlim)) { ok = false; break; }
                if (prof) c_acc += clock64() - ta;
                if (prof && tcount > 0) s_obs += clock64();
                // K block kb sits in stage (s_start + kb) % OP_STAGES: walk the unrolled ring, entering at s_start
                for (int base = -s_start; base < k_blocks && ok; base += C::OP_STAGES) {
#pragma unroll
                    for (int u = 0; u < C::OP_STAGES; ++u) {
                        const int kb = base + u;
                        if ((unsigned)kb < (unsigned)k_blocks) {
                            const uint32_t ph = (mmask >> u) & 1u;
                            mmask ^= 1u << u;
                            if (!peek) {
                                // scales of this K block are in tensor memory of both CTAs; operands of both CTAs landed
                                const long long t0 = prof ? clock64() : 0;
                                if (!mbar_wait(full0 + 8 * u, ph, abort_flag, 3, wlim)) { ok = false; break; }
                                if (prof) { c_wait += clock64() - t0; ++n_miss; }
                            }
                            tc_fence_after();
                            const bool last = kb + 1 == k_blocks;
                            const int un = (u + 1) % C::OP_STAGES;         // the next K block's stage (also across tiles)
                            uint32_t ready;
                            if constexpr (KIND == 0 && DUO_PRE) {
                                ready = duo_kblock_pre(on, kb > 0 ? 1u : 0u, last ? last_atoms : full_mma, last ? 1u : 0u, tmem_base,
                                                       pre_a[u], pre_b[u], desc_hi, pre_sfa[u], pre_sfb[u],
                                                       full0 + 8 * un, (mmask >> un) & 1u, empty0 + 8 * u, tfull_a);
                            } else {
                                ready = (KIND == 0 ? duo_kblock : duo_kblock_mx)(on, kb > 0 ? 1u : 0u, last ? last_atoms : full_mma, last ? 1u : 0u, tmem_base,
                                           a_lo0 + u * (C::X_BYTES >> 4), b_lo0 + u * (C::W_BYTES >> 4), desc_hi,
                                           sf0 + u * TMEM_SF_SLOT_COLS, full0 + 8 * un, (mmask >> un) & 1u,
                                           empty0 + 8 * u, tfull_a);
                            }
                            peek = __all_sync(0xffffffffu, ready != 0u) && !(dbg & 32);
                        }
                    }
                }
                s_start = (s_start + k_blocks) % C::OP_STAGES;
                if (prof && tile + stride < total_tiles) s_commit += clock64();
            }
            if (prof && lane == 0 && p.stats != nullptr && blockIdx.x < 256) {
                p.stats[blockIdx.x * 4 + 0] = (unsigned long long)(clock64() - c_begin);
                p.stats[blockIdx.x * 4 + 1] = (unsigned long long)c_wait;
                p.stats[blockIdx.x * 4 + 2] = (unsigned long long)n_miss;
                p.stats[blockIdx.x * 4 + 3] = (unsigned long long)c_acc;
                p.stats[1024 + blockIdx.x * 2] = (unsigned long long)s_commit;
                p.stats[1024 + blockIdx.x * 2 + 1] = (unsigned long long)s_obs;
            }
        } else {
            // -------------------------------------------------------- relay (peer CTA)
            uint32_t rmask = 0, s = 0;
            bool ok = true;
            const uint32_t full0_leader = map_to_cta(full0, 0);
            for (int64_t tile = first; tile < total_tiles && ok; tile += stride) {
                for (int kb = 0; kb < k_blocks; ++kb) {
                    const uint32_t ph = (rmask >> s) & 1u;
                    rmask ^= 1u << s;
                    if (!mbar_wait_sleep(full0 + 8 * s, ph, abort_flag, 9, wlim)) { ok = false; break; }
                    if (lane == 0) mbar_arrive_cluster_relaxed(full0_leader + 8 * s);
                    if (++s == C::OP_STAGES) s = 0;
                }
            }
        }
    } else if (warp < 6 || warp >= 11) {
        // ------------------------------------------------------------ epilogue (warps 2..5 and 11..14, both CTAs)
        const int q = warp & 3;                              // tensor-memory lane quarter this warp may read
        const int half = warp >= 11 ? 1 : 0;                 // which 128 of the 256 accumulator columns
        uint32_t tcount = 0;
        bool ok = true;
        const uint32_t tempty_leader = map_to_cta(smem_u32(tempty_bar), 0);
        const uint32_t t_lane = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(half * 128);
        const bool out16 = p.out_dtype != OUT_F32, bf16 = p.out_dtype == OUT_BF16;
        const uint32_t my_buf = smem_u32(sEpi) + (uint32_t)(half * 4 + q) * C::EPI_BUF;
        if constexpr (EPI == 0 || EPI == 3) {
            for (int64_t tile = first; tile < total_tiles && ok; tile += stride, ++tcount) {
                int64_t nt, mt;
            duo_tile_coords(tile, tiles_m, tiles_n, p.raster_gm, p.m_shift, mt, nt);
                if (!mbar_wait_sleep(smem_u32(tfull_bar), tcount & 1u, abort_flag, 4, wlim)) { ok = false; break; }
                tc_fence_after();
                if (dbg & 64) {
                    // test hook: a slow epilogue (the accumulator is held ~40k cycles longer), so that the main loop
                    // runs into a full pipeline at every tile
                    const long long t0 = clock64();
                    while (clock64() - t0 < 40000ll) {}
                }
                const int64_t row0 = mt * C::TILE_M + rank * 128 + q * 32;     // first of this warp's 32 token rows
                const int64_t n0 = nt * C::TILE_N + half * 128;                // first of this warp's 128 feature columns
                // One 32-column chunk of an f32 output: alpha, bias, swizzled shared memory (32 rows x 128 bytes), TMA store.
                auto emit = [&](const uint32_t (&v)[32], int c) {
                    const int64_t nn = n0 + c;
                    if (lane == 0) bulk_wait_read_0();       // the store issued from this block one chunk ago has read it
                    __syncwarp();
                    float f[32];
                    duo_scale(v, f, nn, p.N, p.alpha, p.bias);
                    duo_put32(f, my_buf + (uint32_t)lane * 128u, lane);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        // rows beyond M and bytes beyond the row end are clipped by the copy engine; a chunk that
                        // lies outside altogether still closes an (empty) group, so that the group counts above hold
                        if (row0 < p.M && nn < p.N && !(dbg & 1)) {
                            // push epilogue: the owner of these 32 token rows (push_rows is a multiple of 32: a block has one owner)
                            const int64_t o = (EPI == 3) ? row0 / p.push_rows : 0;
                            tma_store_2d(duo_push_map<EPI>(tmO, o), (int)(nn * 4), (int)(row0 - o * p.push_rows), my_buf);
                        }
                        bulk_commit_group();
                    }
                };
                // 16-bit outputs: two chunks per store, so that a stored row is 128 bytes (32 rows x 128 bytes, 128-byte
                // swizzle).  Over NVLink (push epilogue) the width of the written rows sets the rate: 64-byte rows left a rank
                // at 400 GB/s, 128-byte rows at 600 (256-byte rows of f32 from an un-swizzled staging block were no faster);
                // to local memory half as many stores took 1 % off the 8192^3 GEMM.
                auto emit_pair = [&](const uint32_t (&v0)[32], const uint32_t (&v1)[32], int c) {
                    const int64_t nn = n0 + c;
                    float f0[32], f1[32];
                    duo_scale(v0, f0, nn, p.N, p.alpha, EPI == 0 ? p.bias : nullptr);
                    duo_scale(v1, f1, nn + 32, p.N, p.alpha, EPI == 0 ? p.bias : nullptr);
                    const int64_t o = p.push_rows > 0 ? row0 / p.push_rows : 0;
                    if (lane == 0) bulk_wait_read_0();
                    __syncwarp();
                    duo_put16(f0, my_buf + (uint32_t)lane * 128u, 0, lane, bf16);
                    duo_put16(f1, my_buf + (uint32_t)lane * 128u, 4, lane, bf16);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        if (row0 < p.M && nn < p.N && !(dbg & 1))
                            tma_store_2d(duo_push_map<EPI>(tmO, o), (int)(nn * 2), (int)(row0 - o * p.push_rows), my_buf);
                        bulk_commit_group();
                    }
                };
                if (out16) {
                    uint32_t va[32], vb[32];
                    tc_ld32(t_lane, va);
                    tc_ld32(t_lane + 32u, vb);
                    tc_wait_ld();
                    emit_pair(va, vb, 0);
                    tc_ld32(t_lane + 64u, va);
                    tc_ld32(t_lane + 96u, vb);
                    tc_wait_ld();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster_relaxed(tempty_leader);      // this warp's columns are all in registers
                    emit_pair(va, vb, 64);
                    continue;
                }
                // The warp's 128 columns are four chunks.  Two are read at once; the third is read while the second is
                // emitted and the fourth right after, so the accumulator goes back to the MMA issuer after two chunks'
                // worth of arithmetic instead of three.
                uint32_t va[32], vb[32];
                tc_ld32(t_lane, va);
                tc_ld32(t_lane + 32u, vb);
                tc_wait_ld();
                emit(va, 0);
                tc_ld32(t_lane + 64u, va);
                emit(vb, 32);
                tc_wait_ld();
                tc_ld32(t_lane + 96u, vb);
                tc_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster_relaxed(tempty_leader);      // this warp's columns are all in registers
                emit(va, 64);
                emit(vb, 96);
            }
        } else {
            // quantizing epilogues: nothing goes through shared memory; every thread owns one token row
            uint8_t* const q_codes = reinterpret_cast<uint8_t*>(p.out);
            uint8_t* const q_scales = reinterpret_cast<uint8_t*>(p.out2);
            const int64_t Mpad = pad128(p.M);
            // EPI 1: h has N/2 features, N/4 code bytes and N/32 scale columns per row; EPI 2: N code bytes, N/32 scale columns
            const int64_t code_ld = (EPI == 1) ? (p.N >> 2) : p.N;
            const int64_t atoms_per_tile = ((p.N >> 5) + 3) >> 2;
            for (int64_t tile = first; tile < total_tiles && ok; tile += stride, ++tcount) {
                int64_t nt, mt;
            duo_tile_coords(tile, tiles_m, tiles_n, p.raster_gm, p.m_shift, mt, nt);
                if (!mbar_wait_sleep(smem_u32(tfull_bar), tcount & 1u, abort_flag, 4, wlim)) { ok = false; break; }
                tc_fence_after();
                const int64_t row = mt * C::TILE_M + rank * 128 + q * 32 + lane;      // this thread's token
                const int64_t n0 = nt * C::TILE_N + half * 128;                       // first of this warp's 128 columns
                uint32_t cw[8];
                uint32_t scw = 0;
                auto emit = [&](const uint32_t (&v)[32], auto ci_tag) {
                    constexpr int ci = decltype(ci_tag)::value;      // compile-time: cw[] stays in registers
                    const int64_t nn = n0 + 32 * ci;
                    if constexpr (EPI == 1) {
                        uint32_t lo, hi, sc;
                        swiglu_block16(v, p.alpha, lo, hi, sc);
                        if (row >= p.M || nn >= p.N) { lo = hi = sc = 0u; }            // padding rows are written as zeros
                        cw[2 * ci] = lo;
                        cw[2 * ci + 1] = hi;
                        scw |= sc << (8 * ci);
                    } else {
                        uint32_t w[8], sc = 0u;
                        if (nn < p.N) {
                            act_mx8_block32(v, p.alpha, p.bias != nullptr ? p.bias + nn : nullptr, p.epi_act, w, sc);
                            if (row < p.M && !(dbg & 1)) {
                                uint4* dst = reinterpret_cast<uint4*>(q_codes + row * code_ld + nn);
                                dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
                                dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
                            }
                        }
                        scw |= sc << (8 * ci);
                    }
                };
                uint32_t va[32], vb[32];
                tc_ld32(t_lane, va);
                tc_ld32(t_lane + 32u, vb);
                tc_wait_ld();
                emit(va, IntTag<0>{});
                tc_ld32(t_lane + 64u, va);
                emit(vb, IntTag<1>{});
                tc_wait_ld();
                tc_ld32(t_lane + 96u, vb);
                tc_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster_relaxed(tempty_leader);      // this warp's columns are all in registers
                emit(va, IntTag<2>{});
                emit(vb, IntTag<3>{});
                if (n0 < p.N && !(dbg & 1)) {
                    const int64_t atom = (row >> 7) * atoms_per_tile + (n0 >> 7);     // 128 columns = 4 scale columns = one atom
                    if constexpr (EPI == 1) {
                        if (row < Mpad) {
                            uint4* dst = reinterpret_cast<uint4*>(q_codes + row * code_ld + (n0 >> 2));
                            dst[0] = make_uint4(cw[0], cw[1], cw[2], cw[3]);
                            dst[1] = make_uint4(cw[4], cw[5], cw[6], cw[7]);
                            *reinterpret_cast<uint32_t*>(q_scales + atom * 512 + 16 * lane + 4 * q) = scw;
                        }
                    } else if (row < p.M) {
                        *reinterpret_cast<uint32_t*>(q_scales + atom * 512 + 16 * lane + 4 * q) = scw;
                    }
                }
            }
        }
        if (lane == 0) bulk_wait_all();
    } else if (warp < 10) {
        // ------------------------------------------------------------ scale loaders (warps 6..9, both CTAs)
        const int q = warp & 3;
        uint32_t g = 0, lmask = 0, slot = 0;                 // granule counter; phase bits of the scale slots; slot = stage of the next K block
        bool ok = true;
        const bool profl = false;
        long long c_sfl = 0, c_empty = 0, c_st = 0;
        const uint32_t sf_base = smem_u32(sSF);
        const uint32_t full_leader = map_to_cta(full0, 0);
        const uint32_t t_q = tmem_base + ((uint32_t)(q * 32) << 16) + C::SF_COL;
        for (int64_t tile = first; tile < total_tiles && ok; tile += stride) {
            for (int gi = 0; gi < grans && ok; ++gi, ++g) {
                const uint32_t st = g & 1u, gph = (g >> 1) & 1u;
                long long t0 = profl ? clock64() : 0;
                if (!mbar_wait_sleep(sfl0 + 8 * st, gph, abort_flag, 6, wlim)) { ok = false; break; }
                if (profl) c_sfl += clock64() - t0;
                // the atoms of the granule's two K blocks: ATOMS each per part, consecutive in shared memory
                uint32_t va[8 * ATOMS], vw0[8 * ATOMS], vw1[8 * ATOMS];
                const uint32_t src = sf_base + st * C::SF_STAGE_BYTES + lane * 16;
#pragma unroll
                for (int j = 0; j < 2 * ATOMS; ++j) {
                    ld_shared_v4(src + 512 * j, &va[4 * j]);
                    ld_shared_v4(src + C::SF_PART + 512 * j, &vw0[4 * j]);
                    ld_shared_v4(src + 2 * C::SF_PART + 512 * j, &vw1[4 * j]);
                }
                // The stage goes back to the scale producer here, before the values are used.  A shared-memory load has
                // only been issued at this point: when the load/store queue of the SM is backed up (an epilogue writing
                // with bank conflicts was enough), the arrival below overtook the last loads and the next copy into the
                // stage changed what they returned.  So the barrier address is made to depend on every load (acc & 0):
                // the arrival cannot issue before all of them have delivered their registers.
                uint32_t acc = 0;
#pragma unroll
                for (int j = 0; j < 2 * ATOMS; ++j) acc |= va[4 * j] | vw0[4 * j] | vw1[4 * j];
                acc &= (uint32_t)p.zero;
                __syncwarp();
                if (lane == 0) mbar_arrive(sfree0 + 8 * st + acc);
                const int nkb = (2 * gi + 2 <= k_blocks) ? 2 : 1;
#pragma unroll
                for (int b = 0; b < 2; ++b) {
                    if (b < nkb) {
                        {
                            // the slot is free once the MMAs of the K block that used this stage last are done
                            // (a stage never used yet passes at once: the barrier's fresh phase counts as odd)
                            const uint32_t sph = (lmask >> slot) & 1u;
                            lmask ^= 1u << slot;
                            t0 = profl ? clock64() : 0;
                            if (!mbar_wait_sleep(empty0 + 8 * slot, sph ^ 1u, abort_flag, 7, wlim)) { ok = false; break; }
                            if (profl) c_empty += clock64() - t0;
                        }
                        tc_fence_after();
                        t0 = profl ? clock64() : 0;
                        if (!(dbg & 2)) {
                            const uint32_t t_base = t_q + slot * TMEM_SF_SLOT_COLS;
                            if constexpr (KIND == 0) {
                                tc_st<16>(t_base, va + 16 * b);
                                // feature-side scales: MMA j reads 8 columns, rows 0-127 then rows 128-255
                                uint32_t u[32];
#pragma unroll
                                for (int j = 0; j < 4; ++j)
#pragma unroll
                                    for (int w = 0; w < 4; ++w) {
                                        u[8 * j + w] = vw0[16 * b + 4 * j + w];
                                        u[8 * j + 4 + w] = vw1[16 * b + 4 * j + w];
                                    }
                                tc_st<16>(t_base + TMEM_SFA_OFF, u);
                                tc_st<16>(t_base + TMEM_SFA_OFF + 16, u + 16);
                            } else {
                                // one atom per part: 4 columns of token scales, 4 + 4 of feature scales
                                tc_st<4>(t_base, va + 4 * b);
                                tc_st<4>(t_base + TMEM_SFA_OFF, vw0 + 4 * b);
                                tc_st<4>(t_base + TMEM_SFA_OFF + 4, vw1 + 4 * b);
                            }
                            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                        }
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster_relaxed(full_leader + 8 * slot);
                        if (profl) c_st += clock64() - t0;
                        if (++slot == (uint32_t)C::NSLOT) slot = 0;
                    }
                }
            }
        }
        if (profl && lane == 0 && p.stats != nullptr && blockIdx.x < 256) {
            p.stats[blockIdx.x * 4 + 1] = (unsigned long long)c_sfl;
            p.stats[blockIdx.x * 4 + 2] = (unsigned long long)c_st;
            p.stats[blockIdx.x * 4 + 3] = (unsigned long long)c_empty;
        }
    } else {
        // ------------------------------------------------------------ scale producer (warp 10, both CTAs)
        // lanes 0..2: scales of own tokens, of feature rows 0-127, of feature rows 128-255
        uint32_t g = 0;
        bool ok = true;
        const uint32_t sf_base = smem_u32(sSF);
        for (int64_t tile = first; tile < total_tiles && ok; tile += stride) {
            int64_t nt, mt;
            duo_tile_coords(tile, tiles_m, tiles_n, p.raster_gm, p.m_shift, mt, nt);
            const int64_t ta = 2 * mt + rank, tw = 2 * nt;
            const bool a_ok = ta < p.rows_a_tiles, w1_ok = tw + 1 < p.rows_w_tiles;
            const uint8_t* my_src = (lane == 0) ? p.sfA + ta * p.sf_tile_stride
                                                : p.sfW + (tw + (lane == 2 ? 1 : 0)) * p.sf_tile_stride;
            const bool my_ok = (lane == 0) ? a_ok : (lane == 1 ? true : (lane == 2 ? w1_ok : false));
            const uint32_t parts = 1u + (a_ok ? 1u : 0u) + (w1_ok ? 1u : 0u);
            for (int gi = 0; gi < grans; ++gi, ++g) {
                const uint32_t st = g & 1u;
                if (!mbar_wait_sleep(sfree0 + 8 * st, ((g >> 1) & 1u) ^ 1u, abort_flag, 10, wlim)) { ok = false; break; }
                const int kb0 = 2 * gi;
                int atoms = 0;
                for (int kb = kb0; kb < kb0 + 2 && kb < k_blocks; ++kb) atoms += (KIND == 0) ? ((kb == k_blocks - 1) ? p.last_atoms : 4) : 1;
                const uint32_t bytes = (uint32_t)atoms * 512u;
                const uint32_t bar = sfl0 + 8 * st;
                if (dbg & 8) {
                    if (lane == 0) mbar_arrive(bar);
                } else {
                    if (lane == 0) mbar_expect_tx(bar, bytes * parts);
                    __syncwarp();
                    if (my_ok)
                        bulk_load(sf_base + st * C::SF_STAGE_BYTES + (uint32_t)lane * C::SF_PART,
                                  my_src + (int64_t)kb0 * (ATOMS * 512), bytes, bar);
                }
            }
        }
        if (!ok && lane == 0) {
            const long long t0 = clock64();
            while (clock64() - t0 < 4000000ll) {}
        }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag != 0 && p.status != nullptr) atomicCAS(p.status, 0, *abort_flag);
    cluster_sync_all();      // neither CTA leaves while the other may still read its memory or signal it
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
    }
}
