// gemm_duo.cuh -- the large-batch NVFP4 GEMM: a cluster of two CTAs computes a 256-token x
// 256-feature tile with tcgen05.mma.cta_group::2.  Included by gemm.cu inside its anonymous
// namespace, after the single-CTA kernel, its PTX wrappers and gemm_pair.cuh.
//
// Why this shape.  Measured on B200: one 128x256x64 NVFP4 MMA takes 128 cycles whatever feeds it,
// a barrier hop inside a CTA costs ~180 cycles, a hop between the CTAs of a cluster ~550, an
// L2-resident 16 KB TMA load ~650, and all SMs together pull ~85 bytes per cycle and SM out of L2.
// A single CTA with a 128x256 tile needs 105 bytes per cycle and has room for three 54 KB stages,
// i.e. 1000 cycles of cover for a 1700-cycle refill chain: it is bound by both.  Here each CTA
// loads only its own 128 token rows and its own 128 of the 256 feature rows per K block (32 KB,
// 64 bytes per cycle at full MMA rate), so six stages fit: 2500 cycles of cover.
//
// Orientation.  Tokens are the MMA's M side (lane of the accumulator), features its N side
// (column): a thread of the epilogue then holds 32 consecutive features of one token, which are
// contiguous in the row-major output, and stores them directly - no transposition through
// shared memory, which is what keeps the six stages affordable.
//
//   warp 0      producer, both CTAs: per K block two TMA loads (own tokens, own feature half)
//   warp 1      leader: MMA issuer.  peer: relays "my operands landed" to the leader's barrier
//   warps 2-5   epilogue: tcgen05.ld 32 lanes x 32 columns -> alpha, bias, cast -> 16-byte stores
//   warps 6-9   scale loaders: scale atoms (own pipeline, four K blocks ahead of the operands)
//               shared memory -> registers -> tcgen05.st into one of four scale slots
// Barriers.  full[s] (leader: own bytes + the peer's relay; peer: own bytes), empty[s] / tfull:
// local in each CTA, signalled by the leader's tcgen05.commit with a two-CTA mask.  sfl[i]: scale
// atoms landed (local).  sfree[i]: the four loader warps have read scale stage i (local).
// sffull[slot] / tempty: in the leader, 8 arrivals (4 warps of each CTA).  Every wait is bounded.
// All waits poll with CTA-scope mbarrier.test_wait: a cluster-scope acquire on the MMA-issuing
// thread was measured to cost ~250 cycles per poll even when it succeeds at once (it waits for
// the thread's outstanding tcgen05 work), which alone halves the MMA rate.

struct DuoCfg {
    static constexpr int TILE_M = 256, TILE_N = 256;
    static constexpr int OP_STAGES = 6;
    static constexpr int X_BYTES = 128 * KB_BYTES;            // own token rows, one K block
    static constexpr int W_BYTES = 128 * KB_BYTES;            // own half of the feature rows
    static constexpr int SF_STAGES = 4;
    static constexpr int SF_PART = 4 * 512;                   // the scale atoms of 128 rows for one K block
    static constexpr int SF_STAGE_BYTES = 3 * SF_PART;        // own tokens, feature rows 0-127, feature rows 128-255
    static constexpr int NSLOT = 4;                           // scale slots in tensor memory
    static constexpr int SF_COL = 256;                        // behind the 256 accumulator columns
    static constexpr int BAR_BYTES = 512;
    static constexpr int SMEM_BYTES = OP_STAGES * (X_BYTES + W_BYTES) + SF_STAGES * SF_STAGE_BYTES + BAR_BYTES + 1024;
    static constexpr uint32_t IDESC = (1u << 7) | (1u << 10) | ((uint32_t)(TILE_N >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
    static_assert(SF_COL + NSLOT * TMEM_SF_SLOT_COLS <= TMEM_COLS, "scale slots do not fit");
    static_assert(NSLOT < OP_STAGES, "a loader waits on the stage barrier NSLOT K blocks back");
};

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
// Remote arrival without a release fence.  A releasing arrive at cluster scope first waits for
// everything the thread has in flight (its bulk copies, its global stores): measured 500-1200
// cycles per arrival here.  What the arrival publishes is already complete when it is made - a
// TMA transfer whose barrier the thread has seen flip, tensor-memory stores after
// tcgen05.wait::st, tensor-memory loads after tcgen05.wait::ld - so no fence is needed.
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void st_global_v4(void* ptr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(ptr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// one 32-column chunk of one token row: alpha, bias, cast, 16-byte stores (columns beyond N dropped)
__device__ __forceinline__ void duo_emit(const uint32_t (&v)[32], uint8_t* out_row, int64_t n, int64_t N, float alpha,
                                         const float* bias, int out_dtype) {
    float f[32];
    if (bias != nullptr) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
            float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
            if (n + i + 4 <= N) b = __ldg(reinterpret_cast<const float4*>(bias + n + i));
            f[i] = fmaf(alpha, __uint_as_float(v[i]), b.x);
            f[i + 1] = fmaf(alpha, __uint_as_float(v[i + 1]), b.y);
            f[i + 2] = fmaf(alpha, __uint_as_float(v[i + 2]), b.z);
            f[i + 3] = fmaf(alpha, __uint_as_float(v[i + 3]), b.w);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) f[i] = fmaf(alpha, __uint_as_float(v[i]), 0.f);
    }
    if (out_dtype == OUT_F32) {
        float* o = reinterpret_cast<float*>(out_row) + n;
#pragma unroll
        for (int i = 0; i < 32; i += 4)
            if (n + i + 4 <= N)
                st_global_v4(o + i, __float_as_uint(f[i]), __float_as_uint(f[i + 1]), __float_as_uint(f[i + 2]), __float_as_uint(f[i + 3]));
    } else {
        uint32_t h[16];
        if (out_dtype == OUT_BF16) {
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
        uint16_t* o = reinterpret_cast<uint16_t*>(out_row) + n;
#pragma unroll
        for (int i = 0; i < 32; i += 8)
            if (n + i + 8 <= N) st_global_v4(o + i, h[i / 2], h[i / 2 + 1], h[i / 2 + 2], h[i / 2 + 3]);
    }
}

__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_duo_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const GemmParams p) {
    using C = DuoCfg;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sX = smem;
    uint8_t* sWh = sX + (size_t)C::OP_STAGES * C::X_BYTES;
    uint8_t* sSF = sWh + (size_t)C::OP_STAGES * C::W_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sSF + (size_t)C::SF_STAGES * C::SF_STAGE_BYTES);
    uint64_t* full_bar = bars;                               // [OP_STAGES]
    uint64_t* empty_bar = full_bar + C::OP_STAGES;           // [OP_STAGES]
    uint64_t* sfl_bar = empty_bar + C::OP_STAGES;            // [SF_STAGES]
    uint64_t* sfree_bar = sfl_bar + C::SF_STAGES;            // [SF_STAGES]
    uint64_t* sffull_bar = sfree_bar + C::SF_STAGES;         // [NSLOT]     used in the leader
    uint64_t* tfull_bar = sffull_bar + C::NSLOT;             // [1]
    uint64_t* tempty_bar = tfull_bar + 1;                    // [1]         used in the leader
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();                 // 0 = leader
    const bool leader = rank == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::OP_STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), leader ? 2 : 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int s = 0; s < C::SF_STAGES; ++s) {
            mbar_init(smem_u32(&sfl_bar[s]), 1);
            mbar_init(smem_u32(&sfree_bar[s]), 4);
        }
        for (int i = 0; i < C::NSLOT; ++i) mbar_init(smem_u32(&sffull_bar[i]), 8);
        mbar_init(smem_u32(tfull_bar), 1);
        mbar_init(smem_u32(tempty_bar), 8);
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

    const int64_t tiles_m = (p.M + C::TILE_M - 1) / C::TILE_M;
    const int64_t tiles_n = (p.N + C::TILE_N - 1) / C::TILE_N;
    const int64_t total_tiles = tiles_m * tiles_n;
    const int64_t first = blockIdx.x >> 1, stride = gridDim.x >> 1;
    const int k_blocks = p.k_blocks;
    const uint32_t full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar);
    const uint32_t sfl0 = smem_u32(sfl_bar), sfree0 = smem_u32(sfree_bar), sffull0 = smem_u32(sffull_bar);

    if (warp == 0) {
        // ------------------------------------------------------------ producer (both CTAs)
        uint32_t s = 0, ph = 0;
        bool ok = true;
        const bool prof = (p.debug & 1024) != 0;
        long long c_wait = 0;
        const CUtensorMap* my_map = (lane == 0) ? &tmX : &tmW;
        const uint32_t my_dst = (lane == 0) ? smem_u32(sX) : smem_u32(sWh);
        for (int64_t tile = first; tile < total_tiles && ok; tile += stride) {
            const int64_t nt = tile / tiles_m, mt = tile - nt * tiles_m;
            const int my_y = (lane == 0) ? (int)(mt * C::TILE_M + rank * 128) : (int)(nt * C::TILE_N + rank * 128);
            for (int kb = 0; kb < k_blocks; ++kb) {
                const long long t0 = prof ? clock64() : 0;
                if (!mbar_wait(empty0 + 8 * s, ph ^ 1u, abort_flag, 1)) { ok = false; break; }
                if (prof) c_wait += clock64() - t0;
                const uint32_t bar = full0 + 8 * s;
                if (p.debug & 8) {
                    if (lane == 0) mbar_arrive(bar);
                } else {
                    // rows or K bytes outside the tensors are zero-filled and still counted in full
                    if (lane == 0) mbar_expect_tx(bar, (uint32_t)(C::X_BYTES + C::W_BYTES));
                    __syncwarp();
                    if (lane < 2) tma_load_2d(my_dst + s * C::X_BYTES, my_map, kb * KB_BYTES, my_y, bar);
                }
                if (++s == C::OP_STAGES) { s = 0; ph ^= 1u; }
            }
        }
        if (prof && lane == 0 && !leader && p.stats != nullptr && blockIdx.x < 256) p.stats[blockIdx.x * 4 + 0] = (unsigned long long)c_wait;
        if (!ok && lane == 0) {
            // let copies already issued land before the CTA's shared memory goes away
            const long long t0 = clock64();
            while (clock64() - t0 < 4000000ll) {}
        }
    } else if (warp == 1) {
        if (leader) {
            // -------------------------------------------------------- MMA issuer
            // The warp walks the loop together; one elected lane issues.  Nothing but two barrier
            // polls and a few adds sits between the last MMA of a K block and the first of the next:
            // the tensor pipe runs at most about one instruction ahead of its issuer.
            uint32_t s = 0, ph = 0, slot = 0, sph = 0, tcount = 0;
            bool ok = true;
            const uint64_t adesc_base = desc_sw128(smem_u32(sX)), bdesc_base = desc_sw128(smem_u32(sWh));
            const bool prof = (p.debug & 1024) != 0;
            long long c_full = 0, c_sf = 0, c_issue = 0, c_acc = 0;
            const long long c_begin = clock64();
            for (int64_t tile = first; tile < total_tiles && ok; tile += stride, ++tcount) {
                const long long ta = prof ? clock64() : 0;
                if (!mbar_wait(smem_u32(tempty_bar), (tcount & 1u) ^ 1u, abort_flag, 2)) { ok = false; break; }
                if (prof) c_acc += clock64() - ta;
                tc_fence_after();
                for (int kb = 0; kb < k_blocks; ++kb) {
                    long long t0 = 0, t1 = 0, t2 = 0;
                    if (prof) t0 = clock64();
                    if (!mbar_wait(full0 + 8 * s, ph, abort_flag, 3)) { ok = false; break; }
                    if (prof) t1 = clock64();
                    if (!mbar_wait(sffull0 + 8 * slot, sph, abort_flag, 5)) { ok = false; break; }
                    if (prof) t2 = clock64();
                    tc_fence_after();
                    const int n_mma = (kb == k_blocks - 1) ? p.last_atoms : 4;
                    if (elect_one()) {
                        const uint64_t adesc = adesc_base + (uint64_t)(s * (C::X_BYTES >> 4));
                        const uint64_t bdesc = bdesc_base + (uint64_t)(s * (C::W_BYTES >> 4));
                        const uint32_t sf = tmem_base + C::SF_COL + slot * TMEM_SF_SLOT_COLS;
                        if (!(p.debug & 4)) {
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                if (j < n_mma)
                                    tc_mma_pair_nvf4(tmem_base, adesc + 2 * j, bdesc + 2 * j, C::IDESC, sf + 4 * j,
                                                     sf + TMEM_SFA_OFF + 8 * j, (kb > 0 || j > 0) ? 1u : 0u);
                        }
                        tc_commit_pair(empty0 + 8 * s);          // frees stage s (and scale slot) in both CTAs
                        if (kb == k_blocks - 1) tc_commit_pair(smem_u32(tfull_bar));   // accumulator ready in both CTAs
                    }
                    __syncwarp();
                    if (prof) { c_full += t1 - t0; c_sf += t2 - t1; c_issue += clock64() - t2; }
                    if (++s == C::OP_STAGES) { s = 0; ph ^= 1u; }
                    if (++slot == C::NSLOT) { slot = 0; sph ^= 1u; }
                }
            }
            if (prof && lane == 0 && p.stats != nullptr && blockIdx.x < 256) {
                p.stats[blockIdx.x * 4 + 0] = (unsigned long long)(clock64() - c_begin);
                p.stats[blockIdx.x * 4 + 1] = (unsigned long long)c_full;
                p.stats[blockIdx.x * 4 + 2] = (unsigned long long)c_sf;
                p.stats[blockIdx.x * 4 + 3] = (unsigned long long)(c_issue + (c_acc << 32));
            }
        } else {
            // -------------------------------------------------------- relay (peer CTA)
            uint32_t s = 0, ph = 0;
            bool ok = true;
            const uint32_t full0_leader = map_to_cta(full0, 0);
            for (int64_t tile = first; tile < total_tiles && ok; tile += stride) {
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(full0 + 8 * s, ph, abort_flag, 9)) { ok = false; break; }
                    if (lane == 0) mbar_arrive_cluster_relaxed(full0_leader + 8 * s);
                    if (++s == C::OP_STAGES) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
        const int q = warp & 3;                              // tensor-memory lane quarter this warp may read
        uint32_t tcount = 0;
        bool ok = true;
        const uint32_t tempty_leader = map_to_cta(smem_u32(tempty_bar), 0);
        const uint32_t t_lane = tmem_base + ((uint32_t)(q * 32) << 16);
        const int esize = (p.out_dtype == OUT_F32) ? 4 : 2;
        for (int64_t tile = first; tile < total_tiles && ok; tile += stride, ++tcount) {
            const int64_t nt = tile / tiles_m, mt = tile - nt * tiles_m;
            if (!mbar_wait(smem_u32(tfull_bar), tcount & 1u, abort_flag, 4)) { ok = false; break; }
            tc_fence_after();
            const int64_t m = mt * C::TILE_M + rank * 128 + q * 32 + lane;
            const int64_t n0 = nt * C::TILE_N;
            uint8_t* out_row = reinterpret_cast<uint8_t*>(p.out) + (size_t)m * (size_t)p.N * esize;
            const bool row_ok = m < p.M && !(p.debug & 1);
            // the read of the next 32 columns is in flight while the current ones are converted and stored
            uint32_t va[32], vb[32];
            tc_ld32(t_lane, va);
#pragma unroll 1
            for (int c = 0; c < C::TILE_N; c += 64) {
                tc_wait_ld();
                tc_ld32(t_lane + (uint32_t)(c + 32), vb);
                if (row_ok && n0 + c < p.N) duo_emit(va, out_row, n0 + c, p.N, p.alpha, p.bias, p.out_dtype);
                tc_wait_ld();
                if (c + 64 < C::TILE_N) {
                    tc_ld32(t_lane + (uint32_t)(c + 64), va);
                } else {
                    // the accumulator is in registers: hand it back before the last stores
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster_relaxed(tempty_leader);
                }
                if (row_ok && n0 + c + 32 < p.N) duo_emit(vb, out_row, n0 + c + 32, p.N, p.alpha, p.bias, p.out_dtype);
            }
        }
    } else {
        // ------------------------------------------------------------ scale loaders (warps 6..9, both CTAs)
        const int q = warp & 3;
        const bool issuer = warp == 6;                       // this warp also issues the scale-atom copies
        uint32_t sfs = 0, sfph = 0, slot = 0, es = 0, eph = 0, it = 0;
        bool ok = true;
        const bool prof = (p.debug & 1024) != 0 && issuer && !leader;
        long long c_sfl = 0, c_free = 0, c_empty = 0, c_st = 0, c_arr = 0, c_ld = 0;
        const uint32_t sf_base = smem_u32(sSF);
        const uint32_t sffull_leader = map_to_cta(sffull0, 0);
        // the copies run SF_STAGES K blocks ahead of the loaders: a second (tile, kb) cursor
        int64_t tile2 = first;
        int kb2 = 0;
        uint32_t sfs2 = 0;
        auto issue_sf = [&]() {
            // lanes 0..2: scales of own tokens, of feature rows 0-127, of feature rows 128-255
            if (tile2 >= total_tiles) return;
            const int64_t nt2 = tile2 / tiles_m, mt2 = tile2 - nt2 * tiles_m;
            const int atoms = (kb2 == k_blocks - 1) ? p.last_atoms : 4;
            const uint32_t bytes = (uint32_t)atoms * 512u;
            const int64_t ta = 2 * mt2 + rank, tw = 2 * nt2;
            const bool a_ok = ta < p.rows_a_tiles, w1_ok = tw + 1 < p.rows_w_tiles;
            const uint32_t bar = sfl0 + 8 * sfs2;
            if (p.debug & 8) {
                if (lane == 0) mbar_arrive(bar);
            } else {
                if (lane == 0) mbar_expect_tx(bar, bytes * (uint32_t)(1 + (a_ok ? 1 : 0) + (w1_ok ? 1 : 0)));
                __syncwarp();
                const uint32_t dst = sf_base + sfs2 * C::SF_STAGE_BYTES + (uint32_t)lane * C::SF_PART;
                const int64_t koff = (int64_t)kb2 * C::SF_PART;
                if (lane == 0 && a_ok) bulk_load(dst, p.sfA + ta * p.sf_tile_stride + koff, bytes, bar);
                if (lane == 1) bulk_load(dst, p.sfW + tw * p.sf_tile_stride + koff, bytes, bar);
                if (lane == 2 && w1_ok) bulk_load(dst, p.sfW + (tw + 1) * p.sf_tile_stride + koff, bytes, bar);
            }
            if (++kb2 == k_blocks) { kb2 = 0; tile2 += stride; }
            if (++sfs2 == C::SF_STAGES) sfs2 = 0;
        };
        if (issuer)
            for (int i = 0; i < C::SF_STAGES; ++i) issue_sf();
        for (int64_t tile = first; tile < total_tiles && ok; tile += stride) {
            for (int kb = 0; kb < k_blocks; ++kb) {
                long long t0 = prof ? clock64() : 0;
                if (!mbar_wait(sfl0 + 8 * sfs, sfph, abort_flag, 6)) { ok = false; break; }
                if (prof) c_sfl += clock64() - t0;
                t0 = prof ? clock64() : 0;
                uint32_t va[16], vw[2][16];
                const uint32_t src = sf_base + sfs * C::SF_STAGE_BYTES + lane * 16;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    ld_shared_v4(src + 512 * j, &va[4 * j]);
                    ld_shared_v4(src + C::SF_PART + 512 * j, &vw[0][4 * j]);
                    ld_shared_v4(src + 2 * C::SF_PART + 512 * j, &vw[1][4 * j]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(sfree0 + 8 * sfs);
                if (prof) c_ld += clock64() - t0;
                if (issuer) {
                    // refill this scale stage once all four warps have it in registers
                    t0 = prof ? clock64() : 0;
                    if (!mbar_wait(sfree0 + 8 * sfs, sfph, abort_flag, 10)) { ok = false; break; }
                    if (prof) c_free += clock64() - t0;
                    issue_sf();
                }
                if (it >= C::NSLOT) {
                    // the slot is free once the MMAs of the K block NSLOT back are done
                    t0 = prof ? clock64() : 0;
                    if (!mbar_wait(empty0 + 8 * es, eph, abort_flag, 7)) { ok = false; break; }
                    if (prof) c_empty += clock64() - t0;
                    if (++es == C::OP_STAGES) { es = 0; eph ^= 1u; }
                }
                tc_fence_after();
                t0 = prof ? clock64() : 0;
                if (!(p.debug & 2)) {
                    const uint32_t t_base = tmem_base + ((uint32_t)(q * 32) << 16) + C::SF_COL + slot * TMEM_SF_SLOT_COLS;
                    tc_st<16>(t_base, va);
                    // feature-side scales: MMA j reads 8 columns, rows 0-127 then rows 128-255
                    uint32_t u[32];
#pragma unroll
                    for (int j = 0; j < 4; ++j)
#pragma unroll
                        for (int t = 0; t < 2; ++t)
#pragma unroll
                            for (int w = 0; w < 4; ++w) u[8 * j + 4 * t + w] = vw[t][4 * j + w];
                    tc_st<16>(t_base + TMEM_SFA_OFF, u);
                    tc_st<16>(t_base + TMEM_SFA_OFF + 16, u + 16);
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                }
                tc_fence_before();
                __syncwarp();
                long long t1 = prof ? clock64() : 0;
                if (lane == 0) mbar_arrive_cluster_relaxed(sffull_leader + 8 * slot);
                if (prof) { c_st += t1 - t0; c_arr += clock64() - t1; }
                ++it;
                if (++sfs == C::SF_STAGES) { sfs = 0; sfph ^= 1u; }
                if (++slot == C::NSLOT) slot = 0;
            }
        }
        if (prof && lane == 0 && p.stats != nullptr && blockIdx.x < 256) {
            p.stats[blockIdx.x * 4 + 1] = (unsigned long long)c_sfl;
            p.stats[blockIdx.x * 4 + 2] = (unsigned long long)c_free;
            p.stats[blockIdx.x * 4 + 3] = (unsigned long long)c_empty;
            p.stats[600 + blockIdx.x * 2] = (unsigned long long)c_st;
            p.stats[600 + blockIdx.x * 2 + 1] = (unsigned long long)(c_arr + (c_ld << 32));
        }
        if (!ok && issuer && lane == 0) {
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
