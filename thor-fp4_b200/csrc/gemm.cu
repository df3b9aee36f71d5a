// gemm.cu -- hand-written tcgen05 block-scaled GEMMs for sm_100a and their host side.
//
//   out[m, n] = cast( alpha * sum_k deq(act)[m, k] * deq(W)[n, k] + bias[n] )
//
// This replaces the reference's cuBLASLt call (csrc/thor_fp4_core.cu:697-757) and its CUTLASS
// variants (csrc/cutlass_kernels.cu:191-224).  Two kernels share the PTX wrappers below:
//   * gemm_duo_kernel (gemm_duo.cuh): CTA pairs, 256-token x 256-feature tiles, the path of every
//     batch above 128 tokens with enough tiles to fill the GPU;
//   * gemm_bs_kernel (this file): one CTA per tile, computed as (W @ act^T) - the 128-row MMA "M" side
//     is a tile of WEIGHT rows and the "N" side a tile of BN tokens, so a batch of any size only pads
//     the narrow side; with split K (f32 partial tiles + splitk_reduce_kernel) it is the small-batch path.
//
// gemm_bs_kernel, per CTA (persistent over output tiles, 320 threads):
//   warp 0      producer: per 128-byte K block one TMA tile of W codes, one of
//               act codes (128B-swizzled) and the matching 512-byte scale atoms
//               (plain bulk copies - atoms of one K block are contiguous),
//               all completing on the stage's "full" mbarrier;
//   warp 1      MMA issuer: 4 tcgen05.mma.block_scale per stage accumulate in
//               tensor memory; tcgen05.commit releases the stage / publishes the
//               accumulator;
//   warps 6..9  scale loaders: scale atoms shared memory -> registers -> tcgen05.st
//               into a scale slot of tensor memory (tcgen05.cp costs more tensor-pipe
//               time than the MMAs it feeds);
//   warps 2..5  epilogue: tcgen05.ld 32 lanes x 32 columns, alpha / bias / cast,
//               transposed through shared memory, 16-byte row-major stores; with
//               BN <= 128 two accumulators alternate so the
//               epilogue of tile i overlaps the main loop of tile i+1.
//
// KIND 0: NVFP4 x NVFP4   (kind::mxf4nvf4, UE4M3 scale per 16, 256 elements per K block)
// KIND 1: MXFP8 act x MXFP4 weight (kind::mxf8f6f4, UE8M0 scale per 32, 128 elements per
//         K block; the 4-bit weights are expanded by TMA to one byte per element)
//
// Every wait is bounded: on expiry the CTA raises an abort flag, records a
// status word the host reads, drains and frees its tensor memory.
#include <cuda.h>

#include <cstring>
#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"
#include "det_math.cuh"
#include "quant_block.cuh"

namespace tfp4 {

namespace {

constexpr int BM = 128;             // weight rows per tile (MMA M)
constexpr int KB_BYTES = 128;       // bytes of K per stage and row (one swizzle span)
constexpr int GEMM_THREADS = 320;   // producer, MMA issuer, 4 epilogue warps, 4 scale-loader warps
constexpr int TMEM_COLS = 512;
constexpr int TMEM_SF_SLOT_COLS = 48;   // 16 columns of weight-side scales + up to 32 of token-side scales
constexpr int TMEM_SFA_OFF = 16;
constexpr long long WAIT_CYCLES = 2000000000ll;   // ~1 s at 2 GHz

struct GemmParams {
    const uint8_t* sfW;      // weight scales (tile layout)
    const uint8_t* sfA;      // activation scales (tile layout)
    void* out;
    void* out2;              // quantizing epilogues: the scale-tile buffer (out then holds the codes)
    int32_t epi_act;         // MXFP8 epilogue: 0 identity, 1 gelu, 2 silu
    int32_t raster_gm;       // two-CTA kernel: tile order (see duo_tile_coords)
    int64_t push_rows;       // push epilogue: token rows per owning rank
    int64_t m_shift;         // two-CTA kernel: rotation of the token tiles (push epilogue: a different one per rank)
    const float* bias;       // may be null
    float alpha;
    int64_t M, N, K;
    int64_t m_tiles, n_tiles;
    int64_t sf_tile_stride;  // bytes between consecutive 128-row scale tiles = (S/4)*512
    int32_t rows_w_tiles;    // number of 128-row scale tiles of W
    int32_t rows_a_tiles;    // number of 128-row scale tiles of act
    int32_t out_dtype;
    int32_t k_blocks;
    int32_t last_atoms;      // NVFP4: 64-element MMAs in the last K block (1..4); MX: 32-element ones
    int32_t stages;
    int32_t splits;          // K is cut into this many ranges; > 1: partial sums go to `ws` (f32, [split][M][N - ws_n0]:
                             // only the columns of the cut tiles are held)
    int32_t kb_per_split;
    int32_t whole_tiles;     // the first `whole_tiles` output tiles are one work item each (all of K, final output);
                             // the tiles after them are cut into `splits` K ranges (0: every tile is cut)
    float* ws;
    int64_t ws_n0;           // first output column of the cut tiles (a multiple of 128; 0 when every tile is cut)
    int32_t zero;            // always 0, but only known at run time: lets an address depend on loaded values (see the
                             // scale loaders of the two-CTA kernel) without changing it
    int32_t debug;           // test hook: bit0 no stores, bit1 no scale copies, bit2 no MMA, bit3 no loads, bit4 no tmem loads,
                             // bit5 no look-ahead polls, bit6 slow epilogue (two-CTA kernel)
    int* status;             // host-visible status word (0 = ok)
    unsigned long long* stats;   // host-visible per-CTA cycle counters (debug bit 1024): 4 per CTA, then 2 more per CTA from entry 1024
};

// Work item -> (output tile, K range).  Items [0, whole_tiles) are whole tiles; item whole_tiles + j is K range
// j % splits of tile whole_tiles + j / splits.  Cutting only the tiles that do not fill a last wave of CTAs evens
// out tile counts such as 224 on 148 SMs without paying partial sums for every tile.
struct WorkItem {
    int64_t tl;      // output tile (weight-tile major)
    int32_t sp;      // K range index
    int32_t kb0, kb1;
    bool partial;    // f32 partial sums to the workspace instead of the final output
};
__device__ __forceinline__ WorkItem decode_item(const GemmParams& p, int64_t item) {
    WorkItem w;
    if (item < p.whole_tiles) {
        w.tl = item; w.sp = 0; w.kb0 = 0; w.kb1 = p.k_blocks; w.partial = false;
    } else {
        const int64_t j = item - p.whole_tiles;
        w.tl = p.whole_tiles + j / p.splits;
        w.sp = (int32_t)(j % p.splits);
        w.kb0 = w.sp * p.kb_per_split;
        w.kb1 = (w.kb0 + p.kb_per_split < p.k_blocks) ? w.kb0 + p.kb_per_split : p.k_blocks;
        w.partial = p.splits > 1;
    }
    return w;
}

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// non-blocking poll (try_wait may park the thread for a while when the phase is not complete)
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// bounded wait: false if the abort flag is up or the time limit passed.  Polls with the
// non-blocking test_wait: try_wait parks the thread and wakes it late, which costs more than the
// issue slots of the handful of waiting warps.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code,
                                          long long limit = WAIT_CYCLES) {
    if (mbar_test_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t it = 1;; ++it) {
        if (mbar_test_wait(bar, parity)) return true;
        if ((it & 255u) == 0u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > limit) {
                *abort_flag = code;
                return false;
            }
        }
    }
}
// the same, parking between polls (for warps that wait long and should not take issue slots)
__device__ __forceinline__ bool mbar_wait_parked(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t it = 1;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 63u) == 0u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > WAIT_CYCLES) {
                *abort_flag = code;
                return false;
            }
        }
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
template <int KIND>
__device__ __forceinline__ void tc_mma(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                       uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
    if (KIND == 0) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
            ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
            ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
            : "memory");
    }
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}
// shared-memory matrix descriptor, K-major operand tile whose rows are one
// 128-byte swizzle span: 8-row groups 1024 bytes apart, SWIZZLE_128B, version 1
__device__ __forceinline__ uint64_t desc_sw128(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3fffu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

// Epilogue of one tile, run by the four epilogue warps (128 threads) of a CTA.  The accumulator
// holds output feature n on lane n and token m in column m, the transpose of the row-major
// output; 32-token chunks are therefore turned around in shared memory ([token][feature],
// two 16 KB buffers) and leave as 16-byte stores that cover whole output rows of the tile
// (256 or 512 contiguous bytes per token row) instead of 2-byte stores 2*N bytes apart.
constexpr int EPI_STAGE_BYTES = 2 * 16384;
template <int BN>
__device__ __forceinline__ void drain_tile(const GemmParams& p, uint32_t tmem_acc, int ew, int lane,
                                           int64_t n_base, int64_t m0, uint8_t* stage,
                                           void* out_ptr, int out_dtype, const float* bias, int64_t ld, int64_t col0) {
    // out_ptr is a row-major matrix with `ld` elements per row whose first column is output column `col0`
    // (the final output: ld = N, col0 = 0; a split-K partial block: the cut columns only)
    const int64_t n = n_base + ew * 32 + lane;
    const float bias_n = (bias != nullptr && n < p.N) ? bias[n] : 0.f;
    const float alpha = p.alpha;
    const int esize = (out_dtype == OUT_F32) ? 4 : 2;
    const int row_bytes = BM * esize;                 // one token row of the tile
    const int tid = ew * 32 + lane;
    if (p.debug & 16) return;
    const uint32_t t_lane = tmem_acc + ((uint32_t)(ew * 32) << 16);
    const int per_row = row_bytes >> 4;               // 16-byte pieces per token row
    const int pieces = 32 * per_row;
    uint8_t* out = reinterpret_cast<uint8_t*>(out_ptr);
    auto emit = [&](const uint32_t (&v)[32], int c0) {
        if ((p.debug & 1) || m0 + c0 >= p.M) return;  // uniform across the four warps
        uint8_t* buf = stage + ((c0 >> 5) & 1) * 16384;
        uint8_t* mine = buf + tid * esize;
        if (out_dtype == OUT_BF16) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
                *reinterpret_cast<__nv_bfloat16*>(mine + i * row_bytes) = __float2bfloat16_rn(fmaf(alpha, __uint_as_float(v[i]), bias_n));
        } else if (out_dtype == OUT_F16) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
                *reinterpret_cast<__half*>(mine + i * row_bytes) = __float2half_rn(fmaf(alpha, __uint_as_float(v[i]), bias_n));
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
                *reinterpret_cast<float*>(mine + i * row_bytes) = fmaf(alpha, __uint_as_float(v[i]), bias_n);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");   // the four epilogue warps only
        for (int idx = tid; idx < pieces; idx += 128) {
            const int row = idx / per_row, piece = idx - row * per_row;
            const int64_t m = m0 + c0 + row;
            const int64_t nn = n_base + (int64_t)piece * (16 / esize);
            if (m < p.M && nn < p.N) {
                const uint4 val = *reinterpret_cast<const uint4*>(buf + row * row_bytes + piece * 16);
                *reinterpret_cast<uint4*>(out + (m * ld + (nn - col0)) * esize) = val;
            }
        }
    };
    // the tensor-memory read of the next 32 columns is in flight while the current ones are emitted
    uint32_t va[32], vb[32];
    tc_ld32(t_lane, va);
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 64) {
        tc_wait_ld();
        if (c0 + 32 < BN) tc_ld32(t_lane + (uint32_t)(c0 + 32), vb);
        emit(va, c0);
        if (c0 + 32 < BN) {
            tc_wait_ld();
            if (c0 + 64 < BN) tc_ld32(t_lane + (uint32_t)(c0 + 64), va);
            emit(vb, c0 + 32);
        }
    }
}

template <int KIND, int BN>
struct Cfg {
    static constexpr int ACC_STAGES = (2 * BN + 2 * TMEM_SF_SLOT_COLS <= TMEM_COLS) ? 2 : 1;
    static constexpr int SF_COL = ACC_STAGES * BN;
    // scale slots in tensor memory: as many as fit behind the accumulators (at most 4)
    static constexpr int NSLOT_FIT = (TMEM_COLS - ACC_STAGES * BN) / TMEM_SF_SLOT_COLS;                    // scale slots follow the accumulators
    static constexpr int SF_TILES = (BN + 127) / 128;                 // 128-row scale tiles on the token side
    static constexpr int ATOMS = (KIND == 0) ? 4 : 1;                 // scale atoms per 128 rows per stage
    static constexpr int W_BYTES = BM * KB_BYTES;                     // 16 KB
    // bytes the W tile load credits to its mbarrier: the 4-bit weights of the mixed kind are expanded
    // to one byte per code in shared memory, but the copy is accounted at its packed global size
    static constexpr int W_TX_BYTES = (KIND == 0) ? W_BYTES : W_BYTES / 2;
    static constexpr int A_BYTES = BN * KB_BYTES;
    static constexpr int SFW_BYTES = ATOMS * 512;
    static constexpr int SFA_BYTES = SF_TILES * ATOMS * 512;
    static constexpr int STAGE_BYTES = W_BYTES + A_BYTES + SFW_BYTES + SFA_BYTES;
    static constexpr int SMEM_BUDGET = 227 * 1024 - 1024 - 256 - EPI_STAGE_BYTES;   // alignment slack, barriers, epilogue staging
    static constexpr int STAGES = (SMEM_BUDGET / STAGE_BYTES) > 8 ? 8 : (SMEM_BUDGET / STAGE_BYTES);
    static_assert(STAGES >= 3, "pipeline too shallow");
    // scale slots in tensor memory: one per pipeline stage wherever that many fit behind the accumulators
    // (every tile width but 192), so that K block i uses stage and slot i % STAGES alike; never more slots
    // than stages (a loader waits on the stage barrier of the K block NSLOT iterations back; with more slots
    // than stages that barrier could run two phases ahead of the waiter)
    static constexpr int NSLOT = NSLOT_FIT < STAGES ? (NSLOT_FIT < 4 ? NSLOT_FIT : 4) : STAGES;
    static constexpr bool SLOT_IS_STAGE = NSLOT == STAGES;
    static_assert(BN == 192 || SLOT_IS_STAGE, "the unrolled MMA loop needs a scale slot per stage");
    static_assert(NSLOT <= 8, "eight scale-slot barriers are laid out");
    static_assert(NSLOT >= 2, "need two scale slots");
    static_assert((W_BYTES % 1024) == 0 && (A_BYTES % 1024) == 0, "operand tiles must keep 1024-byte alignment");
    // instruction descriptor (block-scaled form): formats, N>>3 at bit 17, scale format at 23, M>>4 at 24
    static constexpr uint32_t IDESC =
        (KIND == 0 ? ((1u << 7) | (1u << 10)) : ((5u << 7) | (0u << 10))) |
        ((uint32_t)(BN >> 3) << 17) | ((KIND == 0 ? 0u : 1u) << 23) | ((uint32_t)(BM >> 4) << 24);
};

__device__ __forceinline__ void tc_commit_if(uint32_t on, uint32_t bar) {
    asm volatile(
        "{\n\t.reg .pred q;\n\tsetp.ne.b32 q, %1, 0;\n\t"
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
        ::"r"(bar), "r"(on) : "memory");
}
template <int KIND>
__device__ __forceinline__ void tc_mma_if(uint32_t on, uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
    if (KIND == 0) {
        asm volatile(
            "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %7, 0;\n\t"
            "@q tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
            ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb), "r"(on)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %7, 0;\n\t"
            "@q tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
            ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb), "r"(on)
            : "memory");
    }
}

__device__ __forceinline__ void ld_shared_v4(uint32_t addr, uint32_t* v) {
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(addr) : "memory");
}
// store N consecutive 32-bit columns of this warp's 32 tensor-memory lanes (lane i <- thread i)
template <int N>
__device__ __forceinline__ void tc_st(uint32_t taddr, const uint32_t* v);
template <>
__device__ __forceinline__ void tc_st<4>(uint32_t taddr, const uint32_t* v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};"
                 ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]) : "memory");
}
template <>
__device__ __forceinline__ void tc_st<16>(uint32_t taddr, const uint32_t* v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                 ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
                   "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]) : "memory");
}

// One K block of the single-CTA MMA stream in one statement (see duo_kblock in gemm_duo.cuh for why): up
// to four MMAs, the look-ahead polls of the next K block's barriers between them, the commit that frees the
// stage and, under a predicate, the commit that publishes the accumulator.  A = weight tile, B = token tile;
// SFB_STEP = scale columns of the token side per MMA (4 per 128 tokens).
template <int KIND, int SFB_STEP, uint32_t IDESC>
__device__ __forceinline__ uint32_t bs_kblock(uint32_t on, uint32_t accumulate, uint32_t n_mma, uint32_t last, uint32_t d,
                                              uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t sfa, uint32_t sfb,
                                              uint32_t full_next, uint32_t sf_next, uint32_t par_next, uint32_t empty_bar,
                                              uint32_t tfull_bar) {
    uint32_t ready;
    if (KIND == 0) {
        asm volatile(
            "{\n\t"
            ".reg .pred q, q0, q1, q2, q3, ql, pa, pt, pf, ps;\n\t"
            ".reg .b32 a1, a2, a3, b1, b2, b3, f1, f2, f3, g1, g2, g3;\n\t"
            ".reg .b64 da0, da1, da2, da3, db0, db1, db2, db3;\n\t"
            "setp.ne.b32 q, %1, 0;\n\t"
            "setp.ne.b32 pa, %2, 0;\n\t"
            "setp.gt.and.u32 q0, %3, 0, q;\n\t"
            "setp.gt.and.u32 q1, %3, 1, q;\n\t"
            "setp.gt.and.u32 q2, %3, 2, q;\n\t"
            "setp.gt.and.u32 q3, %3, 3, q;\n\t"
            "setp.ne.and.b32 ql, %4, 0, q;\n\t"
            "setp.eq.b32 pt, 0, 0;\n\t"
            "add.u32 a1, %6, 2;\n\tadd.u32 a2, %6, 4;\n\tadd.u32 a3, %6, 6;\n\t"
            "add.u32 b1, %7, 2;\n\tadd.u32 b2, %7, 4;\n\tadd.u32 b3, %7, 6;\n\t"
            "mov.b64 da0, {%6, %8};\n\tmov.b64 da1, {a1, %8};\n\tmov.b64 da2, {a2, %8};\n\tmov.b64 da3, {a3, %8};\n\t"
            "mov.b64 db0, {%7, %8};\n\tmov.b64 db1, {b1, %8};\n\tmov.b64 db2, {b2, %8};\n\tmov.b64 db3, {b3, %8};\n\t"
            "add.u32 f1, %9, 4;\n\tadd.u32 f2, %9, 8;\n\tadd.u32 f3, %9, 12;\n\t"
            "add.u32 g1, %10, %17;\n\tadd.u32 g2, g1, %17;\n\tadd.u32 g3, g2, %17;\n\t"
            "@q0 tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%5], da0, db0, %16, [%9], [%10], pa;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 pf, [%11], %13;\n\t"
            "@q1 tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%5], da1, db1, %16, [f1], [g1], pt;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 ps, [%12], %13;\n\t"
            "@q2 tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%5], da2, db2, %16, [f2], [g2], pt;\n\t"
            "@q3 tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%5], da3, db3, %16, [f3], [g3], pt;\n\t"
            "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%14];\n\t"
            "@ql tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%15];\n\t"
            "and.pred pf, pf, ps;\n\t"
            "selp.u32 %0, 1, 0, pf;\n\t"
            "}"
            : "=r"(ready)
            : "r"(on), "r"(accumulate), "r"(n_mma), "r"(last), "r"(d), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(sfa), "r"(sfb),
              "r"(full_next), "r"(sf_next), "r"(par_next), "r"(empty_bar), "r"(tfull_bar), "n"(IDESC), "n"(SFB_STEP)
            : "memory");
    } else {
        // one scale byte per row and MMA: byte j of the 32-bit scale columns (descriptor ids and address top bits)
        asm volatile(
            "{\n\t"
            ".reg .pred q, q0, q1, q2, q3, ql, pa, pt, pf, ps;\n\t"
            ".reg .b32 a1, a2, a3, b1, b2, b3, f1, f2, f3, g1, g2, g3;\n\t"
            ".reg .b64 da0, da1, da2, da3, db0, db1, db2, db3;\n\t"
            "setp.ne.b32 q, %1, 0;\n\t"
            "setp.ne.b32 pa, %2, 0;\n\t"
            "setp.gt.and.u32 q0, %3, 0, q;\n\t"
            "setp.gt.and.u32 q1, %3, 1, q;\n\t"
            "setp.gt.and.u32 q2, %3, 2, q;\n\t"
            "setp.gt.and.u32 q3, %3, 3, q;\n\t"
            "setp.ne.and.b32 ql, %4, 0, q;\n\t"
            "setp.eq.b32 pt, 0, 0;\n\t"
            "add.u32 a1, %6, 2;\n\tadd.u32 a2, %6, 4;\n\tadd.u32 a3, %6, 6;\n\t"
            "add.u32 b1, %7, 2;\n\tadd.u32 b2, %7, 4;\n\tadd.u32 b3, %7, 6;\n\t"
            "mov.b64 da0, {%6, %8};\n\tmov.b64 da1, {a1, %8};\n\tmov.b64 da2, {a2, %8};\n\tmov.b64 da3, {a3, %8};\n\t"
            "mov.b64 db0, {%7, %8};\n\tmov.b64 db1, {b1, %8};\n\tmov.b64 db2, {b2, %8};\n\tmov.b64 db3, {b3, %8};\n\t"
            "or.b32 f1, %9, 0x40000000;\n\tor.b32 f2, %9, 0x80000000;\n\tor.b32 f3, %9, 0xC0000000;\n\t"
            "or.b32 g1, %10, 0x40000000;\n\tor.b32 g2, %10, 0x80000000;\n\tor.b32 g3, %10, 0xC0000000;\n\t"
            "@q0 tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%5], da0, db0, %16, [%9], [%10], pa;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 pf, [%11], %13;\n\t"
            "@q1 tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%5], da1, db1, %17, [f1], [g1], pt;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 ps, [%12], %13;\n\t"
            "@q2 tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%5], da2, db2, %18, [f2], [g2], pt;\n\t"
            "@q3 tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%5], da3, db3, %19, [f3], [g3], pt;\n\t"
            "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%14];\n\t"
            "@ql tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%15];\n\t"
            "and.pred pf, pf, ps;\n\t"
            "selp.u32 %0, 1, 0, pf;\n\t"
            "}"
            : "=r"(ready)
            : "r"(on), "r"(accumulate), "r"(n_mma), "r"(last), "r"(d), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(sfa), "r"(sfb),
              "r"(full_next), "r"(sf_next), "r"(par_next), "r"(empty_bar), "r"(tfull_bar), "n"(IDESC),
              "n"(IDESC | (1u << 29) | (1u << 4)), "n"(IDESC | (2u << 29) | (2u << 4)), "n"(IDESC | (3u << 29) | (3u << 4))
            : "memory");
    }
    return ready;
}

template <int KIND, int BN, bool DBG>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bs_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmA,
               const GemmParams p) {
    using C = Cfg<KIND, BN>;
    constexpr int STAGES = C::STAGES;
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte aligned carve-up: [STAGES x W] [STAGES x act] [STAGES x sfW] [STAGES x sfA] [barriers]
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sW = smem;
    uint8_t* sA = sW + (size_t)STAGES * C::W_BYTES;
    uint8_t* sSFW = sA + (size_t)STAGES * C::A_BYTES;
    uint8_t* sSFA = sSFW + (size_t)STAGES * C::SFW_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sSFA + (size_t)STAGES * C::SFA_BYTES);
    uint64_t* full_bar = bars;                         // [STAGES]
    uint64_t* empty_bar = bars + STAGES;               // [STAGES]
    uint64_t* tfull_bar = bars + 2 * STAGES;           // [ACC_STAGES]
    uint64_t* tempty_bar = tfull_bar + C::ACC_STAGES;  // [ACC_STAGES]
    uint64_t* sffull_bar = tempty_bar + C::ACC_STAGES; // [2] scale slot filled (one arrival per loader warp)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sffull_bar + 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    uint8_t* epi_stage = reinterpret_cast<uint8_t*>(bars) + 256;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int a = 0; a < C::ACC_STAGES; ++a) {
            mbar_init(smem_u32(&tfull_bar[a]), 1);
            mbar_init(smem_u32(&tempty_bar[a]), 4);   // one arrival per epilogue warp
        }
        for (int i = 0; i < 8; ++i) mbar_init(smem_u32(&sffull_bar[i]), 4);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // everything above touched only this CTA's shared and tensor memory; the operands may still be being
    // written by the kernel before this one (programmatic dependent launch), so wait for it here
    griddep_wait();
    griddep_launch();
    // test hooks (tfp4_set_debug) exist only in the DBG instantiation
    const int dbg = DBG ? p.debug : 0;

    // work item = (weight tile, token tile, K range); the K range is the fastest index
    const int64_t total_tiles = p.whole_tiles + (p.m_tiles * p.n_tiles - p.whole_tiles) * p.splits;   // work items
    const int k_blocks = p.k_blocks;
    const uint32_t full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar);

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        // The whole warp walks the loop; the copies of one K block are issued by different lanes
        // of the same instruction (lane 0: W tile, lane 1: token tile, lanes 2..: scale atoms), so a
        // stage costs one issue slot per copy kind instead of five back-to-back issues by one thread.
        {
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (int64_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const WorkItem wi = decode_item(p, tile);
                const int64_t tl = wi.tl;
                const int64_t nt = tl / p.m_tiles, mt = tl - nt * p.m_tiles;
                const int kb0 = wi.kb0, kb1 = wi.kb1;
                const int64_t a_tile0 = (mt * BN) >> 7;     // first 128-row scale tile of this token tile
                int a_tiles = 0;
#pragma unroll
                for (int t = 0; t < C::SF_TILES; ++t)
                    if (a_tile0 + t < p.rows_a_tiles) ++a_tiles;
                // per-lane copy description
                const CUtensorMap* my_map = (lane == 0) ? &tmW : &tmA;
                const int my_y = (lane == 0) ? (int)(nt * BM) : (int)(mt * BN);
                const uint32_t my_tile_dst = (lane == 0) ? smem_u32(sW) : smem_u32(sA);
                const uint32_t my_tile_bytes = (lane == 0) ? (uint32_t)C::W_BYTES : (uint32_t)C::A_BYTES;
                const uint8_t* my_sf_src = (lane == 2) ? p.sfW + nt * p.sf_tile_stride
                                                       : p.sfA + (a_tile0 + (lane - 3)) * p.sf_tile_stride;
                const uint32_t my_sf_dst = (lane == 2) ? smem_u32(sSFW) : smem_u32(sSFA) + (uint32_t)(lane - 3) * C::ATOMS * 512;
                const uint32_t my_sf_stage = (lane == 2) ? (uint32_t)C::SFW_BYTES : (uint32_t)C::SFA_BYTES;
                const bool sf_lane = lane >= 2 && lane < 3 + a_tiles;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(empty0 + 8 * s, ph ^ 1u, abort_flag, 1)) { ok = false; break; }
                    const uint32_t bar = full0 + 8 * s;
                    if (dbg & 8) {
                        if (lane == 0) mbar_arrive(bar);
                    } else {
                        const int atoms = (kb == k_blocks - 1) ? ((KIND == 0) ? p.last_atoms : 1) : C::ATOMS;
                        const uint32_t sf_bytes = (uint32_t)atoms * 512u;
                        if (lane == 0)
                            mbar_expect_tx(bar, (uint32_t)(C::W_TX_BYTES + C::A_BYTES) + sf_bytes * (uint32_t)(1 + a_tiles));
                        __syncwarp();
                        if (lane < 2) {
                            tma_load_2d(my_tile_dst + s * my_tile_bytes, my_map, kb * KB_BYTES, my_y, bar);
                        } else if (sf_lane) {
                            bulk_load(my_sf_dst + s * my_sf_stage, my_sf_src + (int64_t)kb * C::ATOMS * 512, sf_bytes, bar);
                        }
                    }
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
            }
            if (!ok && lane == 0) {
                // let copies already issued land before the CTA's shared memory goes away
                const long long t0 = clock64();
                while (clock64() - t0 < 4000000ll) {}
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        // The whole warp walks the loop (uniform control flow); lane 0 alone issues.
        if constexpr (C::SLOT_IS_STAGE) {
            // K loop unrolled over the stage ring (addresses = base + constant), one statement per K block with
            // the look-ahead polls inside (bs_kblock); the blocking, bounded wait is only the fallback.
            const uint32_t on = (lane == 0) ? 1u : 0u;
            uint32_t mmask = 0, tcount = 0;               // phase bit per stage; work items done
            int s_start = 0;                              // stage of the work item's first K block
            bool ok = true, peek = false;
            const uint64_t adesc_base = desc_sw128(smem_u32(sW)), bdesc_base = desc_sw128(smem_u32(sA));
            const uint32_t desc_hi = (uint32_t)(adesc_base >> 32);
            const uint32_t a_lo0 = (uint32_t)adesc_base, b_lo0 = (uint32_t)bdesc_base;
            const uint32_t sf0 = tmem_base + C::SF_COL;
            const uint32_t sffull0 = smem_u32(sffull_bar);
            const uint32_t full_mma = (dbg & 4) ? 0u : 4u;
            const uint32_t last_atoms = (dbg & 4) ? 0u : (uint32_t)p.last_atoms;
            for (int64_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tcount) {
                const uint32_t acc = tcount % C::ACC_STAGES;
                const uint32_t acc_ph = (tcount / C::ACC_STAGES) & 1u;
                if (!mbar_wait(smem_u32(&tempty_bar[acc]), acc_ph ^ 1u, abort_flag, 2)) { ok = false; break; }
                const uint32_t d_tmem = tmem_base + acc * BN;
                const uint32_t tfull_a = smem_u32(&tfull_bar[acc]);
                const WorkItem wi = decode_item(p, tile);
                const int kb0 = wi.kb0, kb1 = wi.kb1;
                const int nkb = kb1 - kb0;
                for (int base = -s_start; base < nkb && ok; base += STAGES) {
#pragma unroll
                    for (int u = 0; u < STAGES; ++u) {
                        const int r = base + u;
                        if ((unsigned)r < (unsigned)nkb) {
                            const uint32_t ph = (mmask >> u) & 1u;
                            mmask ^= 1u << u;
                            if (!peek) {
                                if (!mbar_wait(sffull0 + 8 * u, ph, abort_flag, 5)) { ok = false; break; }
                                if (!mbar_wait(full0 + 8 * u, ph, abort_flag, 3)) { ok = false; break; }
                            }
                            tc_fence_after();
                            const bool last = r + 1 == nkb;
                            const int un = (u + 1) % STAGES;
                            const uint32_t sfw = sf0 + u * TMEM_SF_SLOT_COLS;
                            const uint32_t ready = bs_kblock<KIND, 4 * C::SF_TILES, C::IDESC>(
                                on, r > 0 ? 1u : 0u, (kb0 + r == k_blocks - 1) ? last_atoms : full_mma, last ? 1u : 0u, d_tmem,
                                a_lo0 + u * (C::W_BYTES >> 4), b_lo0 + u * (C::A_BYTES >> 4), desc_hi, sfw, sfw + TMEM_SFA_OFF,
                                full0 + 8 * un, sffull0 + 8 * un, (mmask >> un) & 1u, empty0 + 8 * u, tfull_a);
                            peek = __all_sync(0xffffffffu, ready != 0u) && !(dbg & 32);
                        }
                    }
                }
                s_start = (s_start + nkb) % STAGES;
            }
        } else {
        const uint32_t on = (lane == 0) ? 1u : 0u;
        uint32_t s = 0, ph = 0, tcount = 0, it = 0;
        bool ok = true, peek_full = false, peek_sf = false;
        long long c_full = 0, c_cp = 0, c_mma = 0;
        const bool prof = (dbg & 1024) != 0;
        const long long c_begin = clock64();
        const uint32_t w_base = smem_u32(sW), a_base = smem_u32(sA);
        for (int64_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tcount) {
            const uint32_t acc = tcount % C::ACC_STAGES;
            const uint32_t acc_ph = (tcount / C::ACC_STAGES) & 1u;
            if (!mbar_wait(smem_u32(&tempty_bar[acc]), acc_ph ^ 1u, abort_flag, 2)) { ok = false; break; }
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + acc * BN;
            // token tiles of 192 start at row 0 or 64 of a 128-row scale atom: rows 32c..32c+31 of
            // an atom sit in scale column c, so the token-side scale address moves by 0 or 2 columns
            const WorkItem wi = decode_item(p, tile);
            const uint32_t sf_off = (BN == 192) ? (uint32_t)((((wi.tl % p.m_tiles) * BN) & 127) >> 5) : 0u;
            const int kb0 = wi.kb0, kb1 = wi.kb1;
            for (int kb = kb0; kb < kb1; ++kb) {
                long long c0 = 0, c1 = 0, c2 = 0, c3 = 0;
                if (prof) c0 = clock64();
                // the barriers of this K block were polled once while the previous block's MMAs were
                // being issued; spin only if that poll failed
                const uint32_t slot = it % C::NSLOT;
                if (!(peek_full || mbar_wait(full0 + 8 * s, ph, abort_flag, 3))) { ok = false; break; }
                if (prof) c1 = clock64();
                if (!(peek_sf || mbar_wait(smem_u32(&sffull_bar[slot]), (it / C::NSLOT) & 1u, abort_flag, 5))) { ok = false; break; }
                tc_fence_after();
                const int n_mma = (kb == k_blocks - 1) ? p.last_atoms : 4;
                const uint32_t sfw_c = tmem_base + C::SF_COL + slot * TMEM_SF_SLOT_COLS;
                const uint32_t sfa_c = sfw_c + TMEM_SFA_OFF + sf_off;
                const uint32_t s_n = (s + 1 == STAGES) ? 0u : s + 1;
                const uint32_t ph_n = (s + 1 == STAGES) ? ph ^ 1u : ph;
                peek_full = false;
                peek_sf = false;
                if (prof) c2 = clock64();
                const uint64_t adesc0 = desc_sw128(w_base + s * C::W_BYTES);
                const uint64_t bdesc0 = desc_sw128(a_base + s * C::A_BYTES);
                if (!(dbg & 4)) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (j < n_mma) {
                            uint32_t idesc = C::IDESC, sfw_t, sfa_t;
                            if (KIND == 0) {
                                sfw_t = sfw_c + 4 * j;
                                sfa_t = sfa_c + 4 * j * C::SF_TILES;
                            } else {
                                // one scale byte per row per MMA: byte j of the 4-byte column
                                idesc |= ((uint32_t)j << 29) | ((uint32_t)j << 4);
                                sfw_t = sfw_c | ((uint32_t)j << 30);
                                sfa_t = sfa_c | ((uint32_t)j << 30);
                            }
                            // advancing K by 64 (or 32) elements = 32 bytes inside the swizzle span
                            if (dbg & 64) {
                                if (elect_one()) tc_mma<KIND>(d_tmem, adesc0 + 2 * j, bdesc0 + 2 * j, idesc, sfw_t, sfa_t, (kb > kb0 || j > 0) ? 1u : 0u);
                            } else {
                                tc_mma_if<KIND>(on, d_tmem, adesc0 + 2 * j, bdesc0 + 2 * j, idesc, sfw_t, sfa_t,
                                                (kb > kb0 || j > 0) ? 1u : 0u);
                            }
                        }
                        if (j == 2 && !(dbg & 32)) {
                            // issuing an MMA returns only when the pipe takes it, i.e. while its predecessor
                            // still runs: poll the next K block's barriers in that shadow (non-blocking),
                            // so that nothing but the commit sits between this block's last MMA and the
                            // next block's first
                            peek_full = mbar_test_wait(full0 + 8 * s_n, ph_n);
                            peek_sf = mbar_test_wait(smem_u32(&sffull_bar[(it + 1) % C::NSLOT]), ((it + 1) / C::NSLOT) & 1u);
                        }
                    }
                }
                tc_commit_if(on, empty0 + 8 * s);
                if (prof) {
                    c3 = clock64();
                    c_full += c1 - c0;
                    c_cp += c2 - c1;
                    c_mma += c3 - c2;
                }
                ++it;
                if (++s == STAGES) { s = 0; ph ^= 1u; }
            }
            if (ok) tc_commit_if(on, smem_u32(&tfull_bar[acc]));
        }
        if (prof && lane == 0 && p.stats != nullptr && blockIdx.x < 256) {
            p.stats[blockIdx.x * 4 + 0] = (unsigned long long)(clock64() - c_begin);
            p.stats[blockIdx.x * 4 + 1] = (unsigned long long)c_full;
            p.stats[blockIdx.x * 4 + 2] = (unsigned long long)c_cp;
            p.stats[blockIdx.x * 4 + 3] = (unsigned long long)c_mma;
        }
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        const int ew = warp & 3;                       // tensor-memory lane quarter this warp may read
        uint32_t tcount = 0;
        bool ok = true;
        for (int64_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tcount) {
            const WorkItem wi = decode_item(p, tile);
            const int64_t sp = wi.sp, tl = wi.tl;
            const int64_t nt = tl / p.m_tiles, mt = tl - nt * p.m_tiles;
            const uint32_t acc = tcount % C::ACC_STAGES;
            const uint32_t acc_ph = (tcount / C::ACC_STAGES) & 1u;
            if (!mbar_wait_parked(smem_u32(&tfull_bar[acc]), acc_ph, abort_flag, 4)) { ok = false; break; }
            tc_fence_after();
            if (wi.partial)   // partial sum of this K range, f32, bias and cast happen in the reduction
                drain_tile<BN>(p, tmem_base + acc * BN, ew, lane, nt * BM, mt * BN, epi_stage,
                               p.ws + sp * p.M * (p.N - p.ws_n0), OUT_F32, nullptr, p.N - p.ws_n0, p.ws_n0);
            else
                drain_tile<BN>(p, tmem_base + acc * BN, ew, lane, nt * BM, mt * BN, epi_stage, p.out, p.out_dtype, p.bias,
                               p.N, 0);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[acc]));
        }
    } else {
        // ------------------------------------------------------------ scale loaders (warps 6..9)
        // tcgen05.cp would run in the MMA pipe (~70 cycles per 512-byte atom, 12 atoms per K
        // block, more than the four MMAs themselves).  Instead each of these warps reads the
        // atoms of a K block from shared memory - an atom is exactly 32 lanes x 16 bytes - and
        // stores them into its own quarter of the tensor-memory lanes with tcgen05.st; the four
        // warps together give the replication across lane quarters the MMA expects.
        const int q = warp & 3;
        uint32_t s = 0, ph = 0, it = 0;
        // stage / phase of the K block two iterations back (whose MMAs must be done before
        // its scale slot is overwritten)
        uint32_t s2 = 0, ph2 = 0;
        bool ok = true;
        const uint32_t sfw_base = smem_u32(sSFW), sfa_base = smem_u32(sSFA);
        for (int64_t tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            const WorkItem wi = decode_item(p, tile);
            const int kb0 = wi.kb0, kb1 = wi.kb1;
            for (int kb = kb0; kb < kb1; ++kb) {
                if (!mbar_wait(full0 + 8 * s, ph, abort_flag, 6)) { ok = false; break; }
                if (it >= C::NSLOT) {
                    if (!mbar_wait(empty0 + 8 * s2, ph2, abort_flag, 7)) { ok = false; break; }
                    if (++s2 == STAGES) { s2 = 0; ph2 ^= 1u; }
                }
                tc_fence_after();
                const uint32_t slot = it % C::NSLOT;
                const uint32_t t_base = tmem_base + ((uint32_t)(q * 32) << 16) + C::SF_COL + slot * TMEM_SF_SLOT_COLS;
                if (!(dbg & 2)) {
                    uint32_t v[C::ATOMS * 4];
                    const uint32_t src_w = sfw_base + s * C::SFW_BYTES + lane * 16;
#pragma unroll
                    for (int j = 0; j < C::ATOMS; ++j) ld_shared_v4(src_w + 512 * j, &v[4 * j]);
                    tc_st<C::ATOMS * 4>(t_base, v);
#pragma unroll
                    for (int t = 0; t < C::SF_TILES; ++t) {
                        // token-side atom (j, t) goes to columns 16 + 4 * (j * SF_TILES + t)
                        const uint32_t src_a = sfa_base + s * C::SFA_BYTES + t * C::ATOMS * 512 + lane * 16;
#pragma unroll
                        for (int j = 0; j < C::ATOMS; ++j) ld_shared_v4(src_a + 512 * j, &v[4 * j]);
#pragma unroll
                        for (int j = 0; j < C::ATOMS; ++j)
                            tc_st<4>(t_base + TMEM_SFA_OFF + 4 * (j * C::SF_TILES + t), &v[4 * j]);
                    }
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&sffull_bar[slot]));
                ++it;
                if (++s == STAGES) { s = 0; ph ^= 1u; }
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag != 0 && p.status != nullptr) atomicCAS(p.status, 0, *abort_flag);
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
    }
}

// Sum of the split-K partial tiles: out[m, n] = cast( sum_s ws[s][m][n] + bias[n] ), four elements
// per thread, splits added in a fixed order (deterministic).
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ ws, int splits, int64_t M, int64_t N, int64_t n0,
                     const float* __restrict__ bias, void* __restrict__ out, int out_dtype) {
    // columns [n0, N) of every row are the cut tiles (the columns before them were written by whole-tile items)
    // (the partial sums hold those columns only: [split][M][N - n0])
    const int64_t width = N - n0, MW = M * width;
    const int64_t e = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (e >= MW) return;
    const int64_t i = (e / width) * N + n0 + (e % width);
    griddep_wait();     // launched while the GEMM still runs; its partial sums are complete after this
    float4 acc = *reinterpret_cast<const float4*>(ws + e);
    for (int s = 1; s < splits; ++s) {
        const float4 v = *reinterpret_cast<const float4*>(ws + (int64_t)s * MW + e);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (bias != nullptr) {
        const float4 b = *reinterpret_cast<const float4*>(bias + (i % N));
        acc.x += b.x; acc.y += b.y; acc.z += b.z; acc.w += b.w;
    }
    if (out_dtype == OUT_F32) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + i) = acc;
    } else if (out_dtype == OUT_BF16) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
        uint2 v = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(out) + i) = v;
    } else {
        __half2 lo = __floats2half2_rn(acc.x, acc.y), hi = __floats2half2_rn(acc.z, acc.w);
        uint2 v = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(out) + i) = v;
    }
}

#include "gemm_duo.cuh"

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

constexpr int kStatsWords = 256 * 6;    // debug counters: 4 per CTA for up to 256 CTAs, then 2 more per CTA

struct DeviceState {
    int sm_count = 0;
    int max_smem = 0;
    int* status_host = nullptr;   // pinned, mapped
    int* status_dev = nullptr;
    unsigned long long* stats_host = nullptr;
    unsigned long long* stats_dev = nullptr;
    // Split-K partial sums.  One block per owner: a stream for eager calls, a capture sequence for calls recorded
    // into a CUDA graph (the graph may later replay on any stream, so its kernels must not share a block with
    // eager calls of other streams).  A block that has become too small is replaced, never freed: kernels already
    // launched and graphs already captured keep its address.
    struct WsBlock { float* ptr = nullptr; size_t bytes = 0; };
    std::map<uint64_t, WsBlock> ws_by_owner;
    size_t ws_retired_bytes = 0;
    bool duo_attr_set = false;
    bool attr_set[2][5] = {{false, false, false, false, false}, {false, false, false, false, false}};
};

std::mutex g_mu;
EncodeTiledFn g_encode = nullptr;
std::map<int, DeviceState> g_dev;
uint64_t g_plan_hits = 0, g_plan_misses = 0;

struct PlanKey {
    const void* pA; const void* pB; int64_t M, N, K; int kind; int bn; int dev;
    bool operator<(const PlanKey& o) const {
        return std::tie(pA, pB, M, N, K, kind, bn, dev) < std::tie(o.pA, o.pB, o.M, o.N, o.K, o.kind, o.bn, o.dev);
    }
};
struct Plan {
    CUtensorMap tmW, tmA;
};
std::map<PlanKey, Plan> g_plans;

int ensure_driver() {
    if (g_encode) return TFP4_OK;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || fn == nullptr) {
        fprintf(stderr, "thor_fp4_b200: cuTensorMapEncodeTiled not available (%s)\n", cudaGetErrorString(e));
        return TFP4_ERR_DRIVER;
    }
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    return TFP4_OK;
}

// per-device state; the pinned status / counter words are created only when `with_pinned`
// (a caller that brings its own scratch never reaches an allocating call)
int ensure_device(DeviceState** out, bool with_pinned = true) {
    int dev = 0;
    TFP4_CK(cudaGetDevice(&dev));
    auto it = g_dev.find(dev);
    if (it == g_dev.end()) {
        DeviceState st;
        TFP4_CK(cudaDeviceGetAttribute(&st.sm_count, cudaDevAttrMultiProcessorCount, dev));
        TFP4_CK(cudaDeviceGetAttribute(&st.max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        it = g_dev.emplace(dev, st).first;
    }
    DeviceState& st = it->second;
    if (with_pinned && st.status_host == nullptr) {
        TFP4_CK(cudaHostAlloc(reinterpret_cast<void**>(&st.status_host), sizeof(int), cudaHostAllocMapped));
        *st.status_host = 0;
        TFP4_CK(cudaHostGetDevicePointer(reinterpret_cast<void**>(&st.status_dev), st.status_host, 0));
        TFP4_CK(cudaHostAlloc(reinterpret_cast<void**>(&st.stats_host), kStatsWords * sizeof(unsigned long long), cudaHostAllocMapped));
        TFP4_CK(cudaHostGetDevicePointer(reinterpret_cast<void**>(&st.stats_dev), st.stats_host, 0));
    }
    *out = &st;
    return TFP4_OK;
}

// rows x row_bytes byte matrix, box = 128 bytes x box_rows, 128-byte swizzle
int encode_map(CUtensorMap* map, CUtensorMapDataType dt, const void* base, uint64_t inner_elems,
               uint64_t rows, uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_rows,
               CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
    cuuint64_t dims[2] = {inner_elems, rows};
    cuuint64_t strides[1] = {row_stride_bytes};
    cuuint32_t box[2] = {box_inner, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        fprintf(stderr, "thor_fp4_b200: cuTensorMapEncodeTiled failed (%d)\n", (int)r);
        return TFP4_ERR_DRIVER;
    }
    return TFP4_OK;
}

int g_pdl = 1;          // 1: GEMM and split-K reduction are launched as programmatic dependents of the kernel before them

template <int KIND, int BN>
int launch(DeviceState* st, const Plan& plan, GemmParams& p, int bn_slot, cudaStream_t stream) {
    using C = Cfg<KIND, BN>;
    // every CTA allocates all 512 tensor-memory columns: the shared-memory request also keeps
    // the kernel at one CTA per SM
    size_t smem = (size_t)C::STAGES * C::STAGE_BYTES + 256 + EPI_STAGE_BYTES + 1024;
    if (smem < 120 * 1024) smem = 120 * 1024;
    if ((int)smem > st->max_smem) return TFP4_ERR_NO_PLAN;
    p.stages = C::STAGES;
    if (!st->attr_set[KIND][bn_slot]) {
        TFP4_CK(cudaFuncSetAttribute(gemm_bs_kernel<KIND, BN, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     st->max_smem));
        TFP4_CK(cudaFuncSetAttribute(gemm_bs_kernel<KIND, BN, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     st->max_smem));
        st->attr_set[KIND][bn_slot] = true;
    }
    const int64_t tiles = p.m_tiles * p.n_tiles;
    const int64_t tiles_all = p.whole_tiles + (tiles - p.whole_tiles) * p.splits;
    const unsigned grid_all = (unsigned)(tiles_all < st->sm_count ? tiles_all : st->sm_count);
    // Launched with programmatic stream serialization: the kernel may become resident and run its prologue
    // (barriers, tensor-memory allocation) while the kernel before it in the stream - normally the activation
    // quantizer - drains; it waits for that kernel's completion before its first global access.  The same
    // holds for the reduction after a split-K GEMM.
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid_all);
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl ? 1 : 0;
    // the instantiation with the test hooks runs only while a debug mask is set
    cudaError_t e = p.debug ? cudaLaunchKernelEx(&cfg, gemm_bs_kernel<KIND, BN, true>, plan.tmW, plan.tmA, p)
                            : cudaLaunchKernelEx(&cfg, gemm_bs_kernel<KIND, BN, false>, plan.tmW, plan.tmA, p);
    if (e == cudaSuccess && p.splits > 1) {
        const int64_t n0 = p.ws_n0;
        const int64_t elems = p.M * (p.N - n0);
        cfg.gridDim = dim3((unsigned)((elems / 4 + 255) / 256));
        cfg.blockDim = dim3(256);
        cfg.dynamicSmemBytes = 0;
        e = cudaLaunchKernelEx(&cfg, splitk_reduce_kernel, (const float*)p.ws, (int)p.splits, (int64_t)p.M, (int64_t)p.N, n0,
                               (const float*)p.bias, (void*)p.out, (int)p.out_dtype);
    }
    if (e != cudaSuccess) {
        fprintf(stderr, "thor_fp4_b200: GEMM launch failed: %s\n", cudaGetErrorString(e));
        return TFP4_ERR_LAUNCH;
    }
    return TFP4_OK;
}

// tensor maps of GEMM outputs (byte view; one store = 32 rows x 32 columns: 64 bytes wide with the 64-byte swizzle
// for 16-bit outputs, 128 bytes wide with the 128-byte swizzle for f32), cached per buffer and shape
struct OutKey {
    const void* out; int64_t M, N; int esize; int dev;
    bool operator<(const OutKey& o) const { return std::tie(out, M, N, esize, dev) < std::tie(o.out, o.M, o.N, o.esize, o.dev); }
};
std::map<OutKey, CUtensorMap> g_out_maps;

int out_map(const CUtensorMap** map, void* out, int64_t M, int64_t N, int esize, int dev) {
    OutKey key{out, M, N, esize, dev};
    auto it = g_out_maps.find(key);
    if (it == g_out_maps.end()) {
        CUtensorMap m;
        int rc = encode_map(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, out, (uint64_t)(N * esize), (uint64_t)M, (uint64_t)(N * esize),
                            128, 32, CU_TENSOR_MAP_SWIZZLE_128B);   // one store = 32 rows x 128 bytes: 64 16-bit or 32 f32 columns
        if (rc) return rc;
        if (g_out_maps.size() > 4096) g_out_maps.clear();
        it = g_out_maps.emplace(key, m).first;
    }
    *map = &it->second;
    return TFP4_OK;
}

template <int KIND, int EPI>
cudaError_t launch_duo_inst(const cudaLaunchConfig_t& cfg, const Plan& plan, const CUtensorMap& tm_out, const GemmParams& p) {
    // the instantiation with the test hooks runs only while a debug mask is set
    return p.debug ? cudaLaunchKernelEx(&cfg, gemm_duo_kernel<KIND, true, EPI>, plan.tmW, plan.tmA, tm_out, p)
                   : cudaLaunchKernelEx(&cfg, gemm_duo_kernel<KIND, false, EPI>, plan.tmW, plan.tmA, tm_out, p);
}

// epi 0: plain output (any kind); 1: SwiGLU + NVFP4 (kind 0); 2: bias + activation + MXFP8 (kind 1)
// what the GEMM's epilogue makes of the accumulator (see gemm_duo.cuh): 0 plain output, 1 SwiGLU + NVFP4, 2 bias +
// activation + MXFP8; out2 = scale-tile buffer of the quantized output, act = activation of mode 2
struct EpilogueSpec {
    int epi = 0;
    void* out2 = nullptr;
    int act = 0;
    void* const* push_dest = nullptr;   // mode 3: per owning rank, where this rank's partial rows for that owner go
    int push_ranks = 0;
    int64_t push_rows = 0;              // token rows per owner
    int push_first = 0;                 // the owner this rank's first tiles go to (ranks start at different owners)
};

// tensor maps of the push epilogue's destinations, cached like the output maps
struct PushKey {
    const void* d[PUSH_MAX_RANKS]; int n; int64_t rows, M, N; int esize; int dev;
    bool operator<(const PushKey& o) const {
        for (int i = 0; i < PUSH_MAX_RANKS; ++i)
            if (d[i] != o.d[i]) return d[i] < o.d[i];
        return std::tie(n, rows, M, N, esize, dev) < std::tie(o.n, o.rows, o.M, o.N, o.esize, o.dev);
    }
};
std::map<PushKey, PushMaps> g_push_maps;

int push_maps(const PushMaps** out, const EpilogueSpec& es, int64_t M, int64_t N, int esize, int dev) {
    PushKey key{};
    for (int i = 0; i < es.push_ranks; ++i) key.d[i] = es.push_dest[i];
    key.n = es.push_ranks; key.rows = es.push_rows; key.M = M; key.N = N; key.esize = esize; key.dev = dev;
    auto it = g_push_maps.find(key);
    if (it == g_push_maps.end()) {
        PushMaps pm;
        memset(&pm, 0, sizeof(pm));
        for (int o = 0; o < es.push_ranks; ++o) {
            int64_t rows = M - (int64_t)o * es.push_rows;
            if (rows > es.push_rows) rows = es.push_rows;
            if (rows <= 0) { pm.m[o] = pm.m[0]; continue; }      // no token row of this owner exists: never selected
            // one store = 32 rows x 128 bytes (two 32-column chunks of a 16-bit output, one of an f32 output), 128-byte swizzle
            int rc = encode_map(&pm.m[o], CU_TENSOR_MAP_DATA_TYPE_UINT8, es.push_dest[o], (uint64_t)(N * esize), (uint64_t)rows,
                                (uint64_t)(N * esize), 128, 32, CU_TENSOR_MAP_SWIZZLE_128B);
            if (rc) return rc;
        }
        for (int o = es.push_ranks; o < PUSH_MAX_RANKS; ++o) pm.m[o] = pm.m[0];
        if (g_push_maps.size() > 1024) g_push_maps.clear();
        it = g_push_maps.emplace(key, pm).first;
    }
    *out = &it->second;
    return TFP4_OK;
}

int launch_duo(DeviceState* st, const Plan& plan, GemmParams& p, int kind, int epi, int dev, cudaStream_t stream,
               const EpilogueSpec* es) {
    const CUtensorMap* tm_out = &plan.tmA;      // the quantizing epilogues store with plain instructions: no output map
    const PushMaps* pm = nullptr;
    if (epi == 3) {
        int rc = push_maps(&pm, *es, p.M, p.N, p.out_dtype == OUT_F32 ? 4 : 2, dev);
        if (rc) return rc;
    }
    if (epi == 0) {
        int rc = out_map(&tm_out, p.out, p.M, p.N, p.out_dtype == OUT_F32 ? 4 : 2, dev);
        if (rc) return rc;
    }
    const size_t smem = DuoCfg::SMEM_BYTES;
    if ((int)smem > st->max_smem) return TFP4_ERR_NO_PLAN;
    p.stages = DuoCfg::OP_STAGES;
    if (!st->duo_attr_set) {
#define TFP4_DUO_ATTR(K_, E_)                                                                                                   \
        TFP4_CK(cudaFuncSetAttribute(gemm_duo_kernel<K_, false, E_>, cudaFuncAttributeMaxDynamicSharedMemorySize, st->max_smem)); \
        TFP4_CK(cudaFuncSetAttribute(gemm_duo_kernel<K_, true, E_>, cudaFuncAttributeMaxDynamicSharedMemorySize, st->max_smem));
        TFP4_DUO_ATTR(0, 0) TFP4_DUO_ATTR(1, 0) TFP4_DUO_ATTR(0, 1) TFP4_DUO_ATTR(1, 2) TFP4_DUO_ATTR(0, 3)
#undef TFP4_DUO_ATTR
        st->duo_attr_set = true;
    }
    const int64_t tiles = ((p.M + DuoCfg::TILE_M - 1) / DuoCfg::TILE_M) * ((p.N + DuoCfg::TILE_N - 1) / DuoCfg::TILE_N);
    const int64_t pairs = st->sm_count / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * (tiles < pairs ? tiles : pairs)));
    cfg.blockDim = dim3(DUO_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // prologue overlaps the quantizer's tail
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_pdl ? 2 : 1;
    cudaError_t e;
    if (epi == 3)
        e = p.debug ? cudaLaunchKernelEx(&cfg, gemm_duo_kernel<0, true, 3>, plan.tmW, plan.tmA, *pm, p)
                    : cudaLaunchKernelEx(&cfg, gemm_duo_kernel<0, false, 3>, plan.tmW, plan.tmA, *pm, p);
    else if (epi == 1) e = launch_duo_inst<0, 1>(cfg, plan, *tm_out, p);
    else if (epi == 2) e = launch_duo_inst<1, 2>(cfg, plan, *tm_out, p);
    else if (kind == 0) e = launch_duo_inst<0, 0>(cfg, plan, *tm_out, p);
    else e = launch_duo_inst<1, 0>(cfg, plan, *tm_out, p);
    if (e != cudaSuccess) {
        fprintf(stderr, "thor_fp4_b200: two-CTA GEMM launch failed: %s\n", cudaGetErrorString(e));
        return TFP4_ERR_LAUNCH;
    }
    return TFP4_OK;
}

// scratch supplied by the caller of gemm_block_scaled_ws instead of the library's own
struct ExtScratch {
    int* status;                 // device-visible status word
    unsigned long long* stats;   // kStatsWords counters (may be null)
    float* ws;                   // split-K partial sums
    size_t ws_bytes;
};

// The split-K workspace of the stream (or capture sequence) this call belongs to, at least `need` bytes.
// Allocates only when that owner has no block yet or its block is too small - i.e. on the first call of a
// shape, like the plan itself; the old block stays allocated (it may be referenced by work in flight or by a
// captured graph).  While the stream is being captured the allocation is made with the thread's capture mode
// relaxed for the duration of the cudaMalloc, which is executed immediately and is not part of the graph.
int workspace_for(DeviceState* st, cudaStream_t stream, size_t need, float** out) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    unsigned long long cap_id = 0;
    if (cudaStreamGetCaptureInfo(stream, &cap, &cap_id) != cudaSuccess) {
        cudaGetLastError();
        cap = cudaStreamCaptureStatusNone;
    }
    const bool capturing = cap == cudaStreamCaptureStatusActive;
    const uint64_t owner = capturing ? ((1ull << 63) | (uint64_t)cap_id) : (uint64_t)reinterpret_cast<uintptr_t>(stream);
    DeviceState::WsBlock& blk = st->ws_by_owner[owner];
    if (blk.bytes < need) {
        const size_t gran = (size_t)4 << 20;
        size_t bytes = ((need + gran - 1) / gran) * gran;
        if (bytes < ((size_t)8 << 20)) bytes = (size_t)8 << 20;
        float* ptr = nullptr;
        cudaStreamCaptureMode mode = cudaStreamCaptureModeRelaxed;
        if (capturing) cudaThreadExchangeStreamCaptureMode(&mode);
        const cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&ptr), bytes);
        if (capturing) cudaThreadExchangeStreamCaptureMode(&mode);
        if (e != cudaSuccess) {
            fprintf(stderr, "thor_fp4_b200: cudaMalloc of %zu bytes of split-K workspace failed: %s\n", bytes, cudaGetErrorString(e));
            cudaGetLastError();
            return TFP4_ERR_CUDA;
        }
        st->ws_retired_bytes += blk.bytes;     // the superseded block is kept, not freed
        blk.ptr = ptr;
        blk.bytes = bytes;
    }
    *out = blk.ptr;
    return TFP4_OK;
}

int g_raster_gm = 0;    // 0 automatic, -1 token tiles fastest, n > 0 bands of n token tiles
int g_force_bn = 0;
int g_force_splits = 0;    // 0 automatic, 1 never split K, n split into (about) n ranges
int g_pair_mode = -1;   // -1: automatic (256x256 two-CTA kernel for batches above 128 tokens with enough tiles); 0: single-CTA
                        // kernel only; 1 or 2: the two-CTA kernel whenever the shape allows it
int g_debug = 0;

}  // namespace

// kind 0: NVFP4 x NVFP4 ; kind 1: MXFP8 activations x MXFP4 weights
int gemm_block_scaled_ws(int kind, const void* packedA, const void* sblkA, const void* packedB,
                         const void* sblkB, float alpha, const float* bias, void* out, int64_t M, int64_t N,
                         int64_t K, int out_dtype, cudaStream_t stream, const ExtScratch* ext,
                         const EpilogueSpec* es = nullptr) {
    const int epi = es ? es->epi : 0;
    if (M < 1 || N < 8 || (N % 8) != 0) {
        fprintf(stderr, "thor_fp4: gemm needs M >= 1, N >= 8, N %% 8 == 0 (got M=%ld N=%ld)\n", (long)M, (long)N);
        return TFP4_ERR_BAD_M;
    }
    const int64_t kq = kind == 0 ? 64 : 128;
    if (K <= 0 || (K % kq) != 0) {
        fprintf(stderr, "thor_fp4: gemm needs K %% %ld == 0 (got %ld)\n", (long)kq, (long)K);
        return TFP4_ERR_BAD_K;
    }
    if (!packedA || !sblkA || !packedB || !sblkB || !out || out_dtype < 0 || out_dtype > 2 ||
        (reinterpret_cast<uintptr_t>(packedA) & 31) || (reinterpret_cast<uintptr_t>(packedB) & 31) ||
        (reinterpret_cast<uintptr_t>(sblkA) & 15) || (reinterpret_cast<uintptr_t>(sblkB) & 15) ||
        (reinterpret_cast<uintptr_t>(out) & 15)) {
        fprintf(stderr, "thor_fp4: gemm bad argument (code buffers 32-byte, scale buffers and output 16-byte aligned)\n");
        return TFP4_ERR_BAD_ARG;
    }
    std::lock_guard<std::mutex> lk(g_mu);
    int rc = ensure_driver();
    if (rc) return rc;
    DeviceState* st = nullptr;
    rc = ensure_device(&st, ext == nullptr);
    if (rc) return rc;
    if (ext == nullptr && *st->status_host != 0) {
        fprintf(stderr, "thor_fp4_b200: an earlier GEMM gave up waiting on the device (code %d)\n", *st->status_host);
        return TFP4_ERR_DEVICE_TIMEOUT;
    }
    // token tiles narrower than a 128-row scale atom are used only when the whole batch fits
    // one tile (the tile then starts at row 0 of its atom)
    int bn = g_force_bn;
    if (bn != 0 && bn < 128 && M > bn) bn = 0;
    if (bn == 0) {
        if (M <= 128) bn = M <= 32 ? 32 : (M <= 64 ? 64 : 128);
        else if (M <= 192) bn = 192;
        else bn = 256;   // measured: the wider tile wins even though its accumulator is drained serially
    }
    int dev = 0;
    cudaGetDevice(&dev);
    // 256 x 256 tiles on CTA pairs: NVFP4, no forced tile width or K split; chosen automatically once
    // there are enough tiles to occupy most CTA pairs (smaller batches do better on single-CTA tiles with split K)
    const int64_t duo_tiles = ((M + 255) / 256) * ((N + 255) / 256);
    const bool duo_ok = M > 128 && N >= 64 && g_force_bn == 0 && g_force_splits <= 1 && st->sm_count >= 2;
    // measured: from 192 tokens on the two-CTA kernel is level with or ahead of the single-CTA one even when its
    // 256x256 tiles fill only part of the GPU (8192 x 8192 at 256 tokens: 18.6 against 20.7 us)
    // the quantizing epilogues exist in the two-CTA kernel only (any batch size: rows past M are zero-filled tiles)
    if (epi != 0 && st->sm_count < 2) return TFP4_ERR_NO_PLAN;
    const bool duo = epi != 0 || (duo_ok && (g_pair_mode >= 1 ||
                                (g_pair_mode == -1 && (M >= 192 || duo_tiles * 8 >= (int64_t)(st->sm_count / 2) * 5))));
    if (duo) bn = 256;
    const uint32_t box_a = duo ? 128u : (uint32_t)bn;
    PlanKey key{packedA, packedB, M, N, K, kind, duo ? 1256 : bn, dev};
    auto it = g_plans.find(key);
    if (it == g_plans.end()) {
        ++g_plan_misses;
        Plan pl;
        const uint64_t rowsW = (uint64_t)pad128(N), rowsA = (uint64_t)pad128(M);
        if (kind == 0) {
            rc = encode_map(&pl.tmW, CU_TENSOR_MAP_DATA_TYPE_UINT8, packedB, (uint64_t)K / 2, rowsW, (uint64_t)K / 2, 128, BM);
            if (rc) return rc;
            rc = encode_map(&pl.tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, packedA, (uint64_t)K / 2, rowsA, (uint64_t)K / 2, 128, box_a);
            if (rc) return rc;
        } else {
            // 4-bit weights, expanded by TMA to 16 codes per 16 bytes of shared memory
            rc = encode_map(&pl.tmW, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, packedB, (uint64_t)K, rowsW, (uint64_t)K / 2, 128, BM);
            if (rc) return rc;
            rc = encode_map(&pl.tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, packedA, (uint64_t)K, rowsA, (uint64_t)K, 128, box_a);
            if (rc) return rc;
        }
        if (g_plans.size() > 4096) g_plans.clear();
        it = g_plans.emplace(key, pl).first;
    } else {
        ++g_plan_hits;
    }
    GemmParams p;
    p.sfW = static_cast<const uint8_t*>(sblkB);
    p.sfA = static_cast<const uint8_t*>(sblkA);
    p.out = out;
    p.out2 = es ? es->out2 : nullptr;
    p.epi_act = es ? es->act : 0;
    // Tile order of the two-CTA kernel.  Each of the two dies keeps its own copy of what its SMs read in its half of
    // the L2, so about 60 MB of operands stay resident per die.  With the token tiles fastest a wave of CTA pairs
    // touches every token tile: fine while all of the activation codes fit, a re-fetch per wave when they do not
    // (16384 x 8192 at K = 8192: 510 -> 469 us; the SwiGLU block's down projection, K = 28672: 2035 -> 1727 us).
    // Bands of gm token tiles whose codes and scales take about 34 MB keep the band resident while the weights stream.
    p.push_rows = es ? es->push_rows : 0;
    p.m_shift = 0;
    if (es && es->epi == 3) {       // start at the first token tile of owner `push_first`
        const int64_t tiles_m256 = (M + 255) / 256;
        p.m_shift = ((int64_t)es->push_first * es->push_rows / 256) % tiles_m256;
    }
    p.raster_gm = 0;
    if (g_raster_gm > 0) {
        p.raster_gm = g_raster_gm;
    } else if (g_raster_gm == 0) {
        const int64_t tile_bytes = 256 * (kind == 0 ? (K / 2 + K / 16) : (K + K / 32));
        const int64_t tiles_m256 = (M + 255) / 256;
        const int64_t gm = (int64_t)34000000 / tile_bytes;
        if (gm < tiles_m256) p.raster_gm = (int32_t)(gm < 1 ? 1 : gm);
    }
    p.bias = bias;
    p.alpha = alpha;
    p.M = M; p.N = N; p.K = K;
    p.m_tiles = (M + bn - 1) / bn;
    p.n_tiles = (N + BM - 1) / BM;
    const int64_t S = kind == 0 ? K / 16 : K / 32;
    p.sf_tile_stride = (S / 4) * 512;
    p.rows_w_tiles = (int32_t)(pad128(N) / 128);
    p.rows_a_tiles = (int32_t)(pad128(M) / 128);
    p.out_dtype = out_dtype;
    const int64_t kb_elems = kind == 0 ? 256 : 128;
    p.k_blocks = (int32_t)((K + kb_elems - 1) / kb_elems);
    const int64_t rem = K - (int64_t)(p.k_blocks - 1) * kb_elems;
    p.last_atoms = (int32_t)(kind == 0 ? rem / 64 : rem / 32);
    p.stages = 0;
    // split K when the output tiles alone would leave most SMs idle (small batches): each K range
    // becomes a work item writing an f32 partial tile, summed by a second kernel
    p.splits = 1;
    p.kb_per_split = p.k_blocks;
    p.whole_tiles = 0;
    p.ws = nullptr;
    p.ws_n0 = 0;
    {
        const int64_t tiles = p.m_tiles * p.n_tiles;
        int want = g_force_splits > 0 ? g_force_splits : 0;
        if (want == 0) {
            want = (!duo && tiles * 2 <= st->sm_count && p.k_blocks >= 8) ? (int)(st->sm_count / tiles) : 1;
            if (!duo && M <= 128 && p.k_blocks >= 8) {
                // Weight-streaming regime (partial sums are negligible next to the weights): pick the split that
                // minimises waves x (K blocks per work item + pipeline fill), which also evens out tile counts
                // that do not divide the SM count (e.g. 224 tiles on 148 SMs).
                int best = 1;
                int64_t best_cost = INT64_MAX;
                for (int sp = 1; sp <= 16 && sp <= p.k_blocks / 4; ++sp) {
                    const int64_t waves = (tiles * sp + st->sm_count - 1) / st->sm_count;
                    // a cut tile also writes and re-reads M x 128 f32 partial sums (weighted as M / 32 K blocks of time, fitted to measurements)
                    // and the reduction kernel costs about four K blocks of time
                    const int64_t cost = waves * ((p.k_blocks + sp - 1) / sp + 6 + (sp > 1 ? M / 32 : 0)) + (sp > 1 ? 4 : 0);
                    if (cost < best_cost) { best_cost = cost; best = sp; }
                }
                want = best;
                // Uneven cut: tiles that fill whole waves of CTAs stay whole (no partial sums, no reduction for
                // them); only the remainder is cut, into as many K ranges as make its last wave short.
                const int64_t whole = (tiles / st->sm_count) * st->sm_count;
                if (g_force_splits == 0 && p.m_tiles == 1 && whole > 0 && whole < tiles) {
                    const int64_t r = tiles - whole;
                    for (int sp = 2; sp <= 16 && sp <= p.k_blocks / 4; ++sp) {
                        const int64_t waves = (r * sp + st->sm_count - 1) / st->sm_count;
                        const int64_t cost = (whole / st->sm_count) * (p.k_blocks + 6) +
                                             waves * ((p.k_blocks + sp - 1) / sp + 6 + M / 32) + 4;
                        if (cost < best_cost) { best_cost = cost; want = sp; p.whole_tiles = (int32_t)whole; }
                    }
                }
            }
        }
        if (want > p.k_blocks / 4) want = p.k_blocks / 4;
        if (want > 16) want = 16;
        if (duo) want = 1;
        // partial sums are held for the cut tiles' columns only (the automatic plans cut at most about one wave of
        // CTAs worth of tiles: <= 148 x 128 columns x 128 tokens x 4 bytes = 9.7 MB); a scratch that is too small
        // for the automatic cut gets fewer K ranges (down to none), a forced cut that does not fit is refused
        const size_t cap = ext != nullptr ? ext->ws_bytes : ((size_t)1 << 30);
        size_t need = 0;
        for (;; --want) {
            p.splits = 1;
            p.kb_per_split = p.k_blocks;
            if (want > 1) {
                p.kb_per_split = (p.k_blocks + want - 1) / want;
                p.splits = (p.k_blocks + p.kb_per_split - 1) / p.kb_per_split;
            }
            if (p.splits <= 1) {
                p.splits = 1;
                p.whole_tiles = 0;
                need = 0;
                break;
            }
            p.ws_n0 = (int64_t)(p.whole_tiles / p.m_tiles) * BM;     // whole_tiles is a multiple of m_tiles
            need = (size_t)p.splits * (size_t)M * (size_t)(N - p.ws_n0) * sizeof(float);
            if (need <= cap) break;
            if (g_force_splits > 0) {      // an explicitly requested cut is not silently changed
                fprintf(stderr, "thor_fp4: split-K into %d ranges needs %zu bytes of scratch, %zu available\n", p.splits, need, cap);
                return TFP4_ERR_BAD_ARG;
            }
        }
        if (p.splits > 1) {
            if (ext != nullptr) {
                p.ws = ext->ws;
            } else {
                rc = workspace_for(st, stream, need, &p.ws);
                if (rc) return rc;
            }
        }
    }
    p.zero = 0;
    p.debug = g_debug;
    p.status = ext ? ext->status : st->status_dev;
    p.stats = ext ? ext->stats : st->stats_dev;
    const Plan& pl = it->second;
    if (duo) return launch_duo(st, pl, p, kind, epi, dev, stream, es);
#define TFP4_GO(KINDV)                                                          \
    switch (bn) {                                                               \
        case 32: return launch<KINDV, 32>(st, pl, p, 0, stream);                \
        case 64: return launch<KINDV, 64>(st, pl, p, 1, stream);                \
        case 128: return launch<KINDV, 128>(st, pl, p, 2, stream);              \
        case 192: return launch<KINDV, 192>(st, pl, p, 4, stream);              \
        default: return launch<KINDV, 256>(st, pl, p, 3, stream);               \
    }
    if (kind == 0) { TFP4_GO(0) } else { TFP4_GO(1) }
#undef TFP4_GO
}

int gemm_block_scaled(int kind, const void* packedA, const void* sblkA, const void* packedB,
                      const void* sblkB, float alpha, const float* bias, void* out, int64_t M, int64_t N,
                      int64_t K, int out_dtype, cudaStream_t stream) {
    return gemm_block_scaled_ws(kind, packedA, sblkA, packedB, sblkB, alpha, bias, out, M, N, K, out_dtype, stream,
                                nullptr);
}

// Gate/up GEMM of a SwiGLU block with the activation, the product and the NVFP4 quantization of the hidden tensor in the
// epilogue.  packedB / sblkB: the stacked weight [2I, K] whose rows alternate in blocks of 16 (gate rows j..j+15, up
// rows j..j+15, ...), N = 2I.  h_packed / h_sblk: codes [pad128(M), I/2] and UE4M3 scale tiles of
// h = silu(alpha * x Wg^T) * (alpha * x Wu^T), quantized with per-tensor scale 1; rows M..pad128(M) are written as zeros.
int gemm_swiglu_nvfp4(const void* packedA, const void* sblkA, const void* packedB, const void* sblkB, float alpha,
                      void* h_packed, void* h_sblk, int64_t M, int64_t N, int64_t K, cudaStream_t stream) {
    if (N <= 0 || (N % 128) != 0) {
        fprintf(stderr, "thor_fp4: the SwiGLU epilogue needs 2 * intermediate %% 128 == 0 (got N=%ld)\n", (long)N);
        return TFP4_ERR_BAD_M;
    }
    if (!h_sblk || (reinterpret_cast<uintptr_t>(h_sblk) & 15)) {
        fprintf(stderr, "thor_fp4: the SwiGLU epilogue needs a 16-byte aligned scale buffer\n");
        return TFP4_ERR_BAD_ARG;
    }
    EpilogueSpec es;
    es.epi = 1;
    es.out2 = h_sblk;
    return gemm_block_scaled_ws(0, packedA, sblkA, packedB, sblkB, alpha, nullptr, h_packed, M, N, K, OUT_BF16, stream,
                                nullptr, &es);
}

// MXFP8 x MXFP4 GEMM whose epilogue adds bias[n], applies the activation (0 identity, 1 gelu, 2 silu) and re-quantizes
// to MXFP8: D = e4m3 codes [M, N] (one byte each, rows past M untouched), SFD = UE8M0 scale tiles (power of two at or
// above amax / 448 per 32 features).  N % 32 == 0, K % 128 == 0.
int gemm_mx8_out(const void* packedA, const void* sblkA, const void* packedB, const void* sblkB, float alpha,
                 const float* bias, int act, void* D, void* SFD, int64_t M, int64_t N, int64_t K, cudaStream_t stream) {
    if (!SFD || (reinterpret_cast<uintptr_t>(SFD) & 15) || act < 0 || act > 2 || (bias && (reinterpret_cast<uintptr_t>(bias) & 15))) {
        fprintf(stderr, "thor_fp4: the MXFP8 epilogue needs 16-byte aligned scale and bias buffers and act in 0..2\n");
        return TFP4_ERR_BAD_ARG;
    }
    if (N <= 0 || (N % 32) != 0) {
        fprintf(stderr, "thor_fp4: the MXFP8 epilogue needs N %% 32 == 0 (got %ld)\n", (long)N);
        return TFP4_ERR_NO_PLAN;
    }
    EpilogueSpec es;
    es.epi = 2;
    es.out2 = SFD;
    es.act = act;
    return gemm_block_scaled_ws(1, packedA, sblkA, packedB, sblkB, alpha, bias, D, M, N, K, OUT_BF16, stream, nullptr, &es);
}

// Row-parallel GEMM of a tensor-parallel block with the first half of the reduce-scatter in its epilogue: this rank's
// partial product (M, N) is stored, 32-row block by 32-row block, into the staging buffers of the ranks that own the
// token rows - dest[o] = where this rank's rows for owner o go, a row-major (rows_per_dest, N) matrix of out_dtype
// (f32, f16 or bf16) in owner o's memory (peer-mapped; dest[own rank] is local).  The stores are TMA stores issued by the
// epilogue warps while the main loop runs; sum_slots on the owner completes the reduction.
int gemm_push(const void* packedA, const void* sblkA, const void* packedB, const void* sblkB, float alpha, void* const* dest,
              int n_dest, int64_t rows_per_dest, int first_dest, int64_t M, int64_t N, int64_t K, int out_dtype,
              cudaStream_t stream) {
    if (n_dest < 1 || n_dest > PUSH_MAX_RANKS || rows_per_dest <= 0 || (rows_per_dest % 32) != 0 || (int64_t)n_dest * rows_per_dest < M ||
        dest == nullptr || (out_dtype != OUT_F32 && out_dtype != OUT_BF16 && out_dtype != OUT_F16)) {
        fprintf(stderr, "thor_fp4: gemm_push needs 1..%d destinations, rows per destination a multiple of 32 covering M, f32, f16 or bf16 partials\n",
                PUSH_MAX_RANKS);
        return TFP4_ERR_BAD_ARG;
    }
    for (int i = 0; i < n_dest; ++i)
        if (dest[i] == nullptr || (reinterpret_cast<uintptr_t>(dest[i]) & 15)) {
            fprintf(stderr, "thor_fp4: gemm_push destination %d is null or not 16-byte aligned\n", i);
            return TFP4_ERR_BAD_ARG;
        }
    EpilogueSpec es;
    es.epi = 3;
    es.push_dest = dest;
    es.push_ranks = n_dest;
    es.push_rows = rows_per_dest;
    es.push_first = (first_dest >= 0 && first_dest < n_dest) ? first_dest : 0;
    return gemm_block_scaled_ws(0, packedA, sblkA, packedB, sblkB, alpha, nullptr, dest[0], M, N, K, out_dtype, stream, nullptr, &es);
}

// ---------------------------------------------------------------------------------------------
// Allocation-free entry.  Some hosts of this library may not allocate device or pinned memory at
// call time: a serving process whose device memory was carved up completely at start-up, a plug-in
// that runs under an allocator it does not own, or a latency-bound loop that cannot afford the
// device-wide synchronisation an allocation or a free implies.  For them the GEMM's scratch - the
// status word the kernel's bounded waits report to, the debug counters and the split-K partial
// sums - lives in this fixed array of device memory instead of cudaHostAlloc / cudaMalloc
// blocks.  Every GPU that loads the library carries the array until the process exits.
// ---------------------------------------------------------------------------------------------
constexpr size_t kNoAllocScratchBytes = 16u << 20;     // the stated maximum: 16 MiB in total
constexpr size_t kNoAllocHeaderBytes = 16u << 10;      // status word at 0, counters at 256, then partial sums
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

namespace {
std::mutex g_noalloc_mu;
std::map<int, unsigned char*> g_noalloc_addr;          // device ordinal -> device address of the array

// The array's name is only a host-side handle; the kernel needs its device address, looked up once
// per device with that device current.
int noalloc_scratch(unsigned char** out) {
    int dev = 0;
    TFP4_CK(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    auto it = g_noalloc_addr.find(dev);
    if (it == g_noalloc_addr.end()) {
        unsigned char* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            fprintf(stderr, "thor_fp4_b200: cudaGetSymbolAddress(scratch) failed: %s\n", cudaGetErrorString(e));
            return TFP4_ERR_CUDA;
        }
        it = g_noalloc_addr.emplace(dev, ptr).first;
    }
    *out = it->second;
    return TFP4_OK;
}
}  // namespace

// NVFP4 GEMM (+ optional bias) with all scratch in the fixed array above.  No cudaMalloc, cudaFree,
// cudaHostAlloc or other allocating call is made.  The first call on a device looks the array's
// address up (do it before any stream capture).  Split-K partial sums beyond the array's capacity
// are refused with -7 and a message.  All calls share the array: calls that overlap on the GPU
// (different streams) race on it; calls on one stream are safe.  The partial sums are fully
// rewritten by every call and need no clearing; the status word starts at zero when the library is
// loaded and stays set after a kernel gave up waiting (read / reset it with gemm_noalloc_status).
int gemm_noalloc(const void* packedA, const void* sblkA, const void* packedB, const void* sblkB, float alpha,
                 const float* bias, void* out, int64_t M, int64_t N, int64_t K, int out_dtype, cudaStream_t stream) {
    unsigned char* base = nullptr;
    int rc = noalloc_scratch(&base);
    if (rc) return rc;
    ExtScratch ext;
    ext.status = reinterpret_cast<int*>(base);
    ext.stats = reinterpret_cast<unsigned long long*>(base + 256);
    ext.ws = reinterpret_cast<float*>(base + kNoAllocHeaderBytes);
    ext.ws_bytes = kNoAllocScratchBytes - kNoAllocHeaderBytes;
    return gemm_block_scaled_ws(0, packedA, sblkA, packedB, sblkB, alpha, bias, out, M, N, K, out_dtype, stream, &ext);
}

// Blocking read (and optional reset) of the status word kept in the fixed array; not for hot paths.
int gemm_noalloc_status(int reset) {
    unsigned char* base = nullptr;
    if (noalloc_scratch(&base)) return -1;
    int v = 0;
    if (cudaMemcpy(&v, base, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (reset && v != 0) cudaMemset(base, 0, sizeof(int));
    return v;
}

size_t gemm_noalloc_capacity() { return kNoAllocScratchBytes - kNoAllocHeaderBytes; }

void gemm_set_splits(int n) { g_force_splits = n < -1 ? 0 : n; }   // -1: automatic, every tile cut alike (A/B)

int gemm_warm() {
    std::lock_guard<std::mutex> lk(g_mu);
    int rc = ensure_driver();
    if (rc) return rc;
    DeviceState* st = nullptr;
    return ensure_device(&st);
}

void gemm_set_debug(int d) { g_debug = d; }
void gemm_set_raster(int gm) { g_raster_gm = gm; }
void gemm_set_pair_mode(int m) { g_pair_mode = m; }
void gemm_set_pdl(int on) { g_pdl = on ? 1 : 0; }

// per-CTA cycle counters of the MMA-issuing thread, written when debug bit 1024 is set:
// {total, waiting for operands, waiting for the accumulator, issuing}
int gemm_debug_stats(unsigned long long* out, int n_ctas) {
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceState* st = nullptr;
    if (ensure_device(&st)) return -1;
    for (int i = 0; i < n_ctas * 4 && i < 256 * 4; ++i) out[i] = st->stats_host[i];
    return 0;
}

void gemm_set_token_tile(int bn) { g_force_bn = (bn == 32 || bn == 64 || bn == 128 || bn == 192 || bn == 256) ? bn : 0; }

int gemm_status_word() {
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceState* st = nullptr;
    if (ensure_device(&st)) return -1;
    return *st->status_host;
}

void gemm_clear_status() {
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceState* st = nullptr;
    if (ensure_device(&st) == 0) *st->status_host = 0;
}

void gemm_plan_stats(uint64_t* hits, uint64_t* misses) {
    std::lock_guard<std::mutex> lk(g_mu);
    *hits = g_plan_hits;
    *misses = g_plan_misses;
}

}  // namespace tfp4
