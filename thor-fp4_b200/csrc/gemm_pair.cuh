// gemm_pair.cuh -- the two-CTA (cta_group::2) form of the block-scaled GEMM kernel; included by
// gemm.cu inside its anonymous namespace, after the single-CTA kernel and its PTX wrappers.
//
// A cluster of two CTAs (one SM each) computes a 256-row (weights) x BN-token tile with
// tcgen05.mma.cta_group::2, issued by the leader CTA alone: each instruction does twice the work
// of the single-CTA form for the same issue cost, which is what bounds the single-CTA kernel.
//   * CTA r owns weight rows [256*nt + 128*r, +128): its W tile, its W scales, its accumulator
//     (128 tensor-memory lanes x BN columns), its half of the epilogue.
//   * The token tile is split in halves: CTA r loads token rows [m0 + r*BN/2, +BN/2) into its own
//     shared memory; the MMA reads both halves.  No load is multicast: each CTA issues plain TMA
//     loads for what it needs, and both CTAs load the (small) token-side scale atoms of the whole
//     tile, because each CTA's MMA half needs every token's scales in its own tensor memory.
//   * Barriers.  full[s]: in the leader, counts the operand bytes of BOTH CTAs (the peer's TMA
//     loads signal the leader's barrier, which cp.async.bulk.tensor.cta_group::2 permits).
//     sfl[s]: local, scale atoms landed.  sffull[slot]: in the leader, 8 arrivals (4 loader warps
//     per CTA; the peer arrives remotely).  empty[s] / tfull[a]: local in each CTA, signalled by
//     the leader's tcgen05.commit with a two-CTA multicast mask.  tempty[a]: in the leader, 8
//     arrivals (4 epilogue warps per CTA).
// Every wait is bounded, as in the single-CTA kernel.

template <int KIND, int BN>
struct PairCfg {
    static constexpr int HALF = BN / 2;                                // token rows held by each CTA
    static constexpr int ACC_STAGES = (2 * BN + 2 * TMEM_SF_SLOT_COLS <= TMEM_COLS) ? 2 : 1;
    static constexpr int SF_COL = ACC_STAGES * BN;
    // scale slots in tensor memory: as many as fit behind the accumulators (at most 4)
    static constexpr int NSLOT_FIT = (TMEM_COLS - ACC_STAGES * BN) / TMEM_SF_SLOT_COLS;
    static constexpr int SF_TILES = (BN + 127) / 128;
    static constexpr int ATOMS = (KIND == 0) ? 4 : 1;
    static constexpr int W_BYTES = BM * KB_BYTES;
    static constexpr int W_TX_BYTES = (KIND == 0) ? W_BYTES : W_BYTES / 2;
    static constexpr int A_BYTES = HALF * KB_BYTES;
    static constexpr int SFW_BYTES = ATOMS * 512;
    static constexpr int SFA_BYTES = SF_TILES * ATOMS * 512;
    static constexpr int STAGE_BYTES = W_BYTES + A_BYTES + SFW_BYTES + SFA_BYTES;
    static constexpr int SMEM_BUDGET = 227 * 1024 - 1024 - 512 - EPI_STAGE_BYTES;
    static constexpr int STAGES = (SMEM_BUDGET / STAGE_BYTES) > 8 ? 8 : (SMEM_BUDGET / STAGE_BYTES);
    static_assert(STAGES >= 3, "pipeline too shallow");
    // scale slots in tensor memory: at most 4, and never more than pipeline stages (a loader
    // waits on the stage barrier of the K block NSLOT iterations back; with more slots than stages
    // that barrier could run two phases ahead of the waiter)
    static constexpr int NSLOT = NSLOT_FIT < (STAGES < 4 ? STAGES : 4) ? NSLOT_FIT : (STAGES < 4 ? STAGES : 4);
    static_assert(NSLOT >= 2, "need two scale slots");
    static_assert((W_BYTES % 1024) == 0 && (A_BYTES % 1024) == 0, "operand tiles must keep 1024-byte alignment");
    // M = 256 across the pair
    static constexpr uint32_t IDESC =
        (KIND == 0 ? ((1u << 7) | (1u << 10)) : ((5u << 7) | (0u << 10))) |
        ((uint32_t)(BN >> 3) << 17) | ((KIND == 0 ? 0u : 1u) << 23) | ((uint32_t)(256 >> 4) << 24);
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
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// waits on barriers that the peer CTA (or its asynchronous copies) signals: cluster-scope acquire
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t it = 1;; ++it) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if ((it & 255u) == 0u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > WAIT_CYCLES) {
                *abort_flag = code;
                return false;
            }
        }
    }
}
// TMA tile load whose completion bytes are credited to a barrier that may live in the peer CTA
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar_cluster)
        : "memory");
}
__device__ __forceinline__ void tc_commit_pair_if(uint32_t on, uint32_t bar) {
    asm volatile(
        "{\n\t.reg .pred q;\n\t.reg .b16 m;\n\tsetp.ne.b32 q, %1, 0;\n\tmov.b16 m, 3;\n\t"
        "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], m;\n\t}"
        ::"r"(bar), "r"(on) : "memory");
}
template <int KIND>
__device__ __forceinline__ void tc_mma_pair_if(uint32_t on, uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
    if (KIND == 0) {
        asm volatile(
            "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %7, 0;\n\t"
            "@q tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
            ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb), "r"(on)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %7, 0;\n\t"
            "@q tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
            ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb), "r"(on)
            : "memory");
    }
}

template <int KIND, int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmA,
                 const GemmParams p) {
    using C = PairCfg<KIND, BN>;
    constexpr int STAGES = C::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sW = smem;
    uint8_t* sA = sW + (size_t)STAGES * C::W_BYTES;
    uint8_t* sSFW = sA + (size_t)STAGES * C::A_BYTES;
    uint8_t* sSFA = sSFW + (size_t)STAGES * C::SFW_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sSFA + (size_t)STAGES * C::SFA_BYTES);
    uint64_t* full_bar = bars;                          // [STAGES]   used in the leader
    uint64_t* empty_bar = bars + STAGES;                // [STAGES]   local
    uint64_t* sfl_bar = bars + 2 * STAGES;              // [STAGES]   local
    uint64_t* peer_bar = bars + 3 * STAGES;             // [STAGES]   in the leader: the peer's operands landed
    uint64_t* tfull_bar = bars + 4 * STAGES;            // [ACC_STAGES] local
    uint64_t* tempty_bar = tfull_bar + C::ACC_STAGES;   // [ACC_STAGES] used in the leader
    uint64_t* sffull_bar = tempty_bar + C::ACC_STAGES;  // [2]        used in the leader
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sffull_bar + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    uint8_t* epi_stage = reinterpret_cast<uint8_t*>(bars) + 512;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();            // 0 = leader
    const bool leader = rank == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
            mbar_init(smem_u32(&sfl_bar[s]), 1);
            mbar_init(smem_u32(&peer_bar[s]), 1);
        }
        for (int a = 0; a < C::ACC_STAGES; ++a) {
            mbar_init(smem_u32(&tfull_bar[a]), 1);
            mbar_init(smem_u32(&tempty_bar[a]), 8);     // 4 epilogue warps of each CTA
        }
        for (int i = 0; i < 4; ++i) mbar_init(smem_u32(&sffull_bar[i]), 8);   // 4 loader warps of each CTA
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

    const int64_t n_pairs = (p.n_tiles + 1) / 2;        // 256-row weight tiles
    const int64_t total_tiles = p.m_tiles * n_pairs;
    const int64_t first = blockIdx.x >> 1, stride = gridDim.x >> 1;
    const int k_blocks = p.k_blocks;
    const uint32_t full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar), sfl0 = smem_u32(sfl_bar);
    const uint32_t peer0 = smem_u32(peer_bar);

    if (warp == 0) {
        // ------------------------------------------------------------ producer (both CTAs)
        // whole warp in the loop; lane 0: W tile, lane 1: token half-tile, lanes 2..: scale atoms
        {
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (int64_t tile = first; tile < total_tiles && ok; tile += stride) {
                const int64_t np = tile / p.m_tiles, mt = tile - np * p.m_tiles;
                const int64_t nt = 2 * np + rank;                       // this CTA's 128-row weight tile
                const bool w_ok = nt < p.rows_w_tiles;                  // odd tile counts: the peer has no rows
                const int64_t a_tile0 = (mt * BN) >> 7;
                int a_tiles = 0;
#pragma unroll
                for (int t = 0; t < C::SF_TILES; ++t)
                    if (a_tile0 + t < p.rows_a_tiles) ++a_tiles;
                const CUtensorMap* my_map = (lane == 0) ? &tmW : &tmA;
                const int my_y = (lane == 0) ? (int)(nt * BM) : (int)(mt * BN + rank * C::HALF);
                const uint32_t my_tile_dst = (lane == 0) ? smem_u32(sW) : smem_u32(sA);
                const uint32_t my_tile_bytes = (lane == 0) ? (uint32_t)C::W_BYTES : (uint32_t)C::A_BYTES;
                const uint8_t* my_sf_src = (lane == 2) ? p.sfW + nt * p.sf_tile_stride
                                                       : p.sfA + (a_tile0 + (lane - 3)) * p.sf_tile_stride;
                const uint32_t my_sf_dst = (lane == 2) ? smem_u32(sSFW) : smem_u32(sSFA) + (uint32_t)(lane - 3) * C::ATOMS * 512;
                const uint32_t my_sf_stage = (lane == 2) ? (uint32_t)C::SFW_BYTES : (uint32_t)C::SFA_BYTES;
                const bool sf_lane = (lane == 2 && w_ok) || (lane >= 3 && lane < 3 + a_tiles);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(empty0 + 8 * s, ph ^ 1u, abort_flag, 1)) { ok = false; break; }
                    const uint32_t bar = full0 + 8 * s;
                    const uint32_t sbar = sfl0 + 8 * s;
                    if (p.debug & 8) {
                        if (lane == 0) {
                            mbar_arrive(full0 + 8 * s);
                            mbar_arrive(sbar);
                        }
                    } else {
                        const int atoms = (kb == k_blocks - 1) ? ((KIND == 0) ? p.last_atoms : 1) : C::ATOMS;
                        const uint32_t sf_bytes = (uint32_t)atoms * 512u;
                        if (lane == 0) {
                            // operand bytes land on the CTA's own barrier (out-of-range rows are zero-filled
                            // by TMA and still counted); scale atoms on a second local one
                            mbar_expect_tx(full0 + 8 * s, (uint32_t)(C::W_TX_BYTES + C::A_BYTES));
                            mbar_expect_tx(sbar, sf_bytes * (uint32_t)((w_ok ? 1 : 0) + a_tiles));
                        }
                        __syncwarp();
                        if (lane < 2) {
                            tma_load_2d(my_tile_dst + s * my_tile_bytes, my_map, kb * KB_BYTES, my_y, bar);
                        } else if (sf_lane) {
                            bulk_load(my_sf_dst + s * my_sf_stage, my_sf_src + (int64_t)kb * C::ATOMS * 512, sf_bytes, sbar);
                        }
                    }
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
            }
            if (!ok && lane == 0) {
                const long long t0 = clock64();
                while (clock64() - t0 < 4000000ll) {}
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader CTA only)
        if (leader) {
            const uint32_t on = (lane == 0) ? 1u : 0u;
            uint32_t s = 0, ph = 0, tcount = 0, it = 0;
            bool ok = true;
            const uint32_t w_base = smem_u32(sW), a_base = smem_u32(sA);
            for (int64_t tile = first; tile < total_tiles && ok; tile += stride, ++tcount) {
                const uint32_t acc = tcount % C::ACC_STAGES;
                const uint32_t acc_ph = (tcount / C::ACC_STAGES) & 1u;
                if (!mbar_wait_cluster(smem_u32(&tempty_bar[acc]), acc_ph ^ 1u, abort_flag, 2)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                const uint32_t sf_off = (BN == 192) ? (uint32_t)((((tile % p.m_tiles) * BN) & 127) >> 5) : 0u;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    const uint32_t slot = it % C::NSLOT;
                    if (!mbar_wait(full0 + 8 * s, ph, abort_flag, 3)) { ok = false; break; }
                    if (!mbar_wait_cluster(peer0 + 8 * s, ph, abort_flag, 8)) { ok = false; break; }
                    if (!mbar_wait_cluster(smem_u32(&sffull_bar[slot]), (it / C::NSLOT) & 1u, abort_flag, 5)) { ok = false; break; }
                    tc_fence_after();
                    const int n_mma = (kb == k_blocks - 1) ? p.last_atoms : 4;
                    const uint32_t sfw_c = tmem_base + C::SF_COL + slot * TMEM_SF_SLOT_COLS;
                    const uint32_t sfa_c = sfw_c + TMEM_SFA_OFF + sf_off;
                    const uint64_t adesc0 = desc_sw128(w_base + s * C::W_BYTES);
                    const uint64_t bdesc0 = desc_sw128(a_base + s * C::A_BYTES);
                    if (!(p.debug & 4)) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            if (j < n_mma) {
                                uint32_t idesc = C::IDESC, sfw_t, sfa_t;
                                if (KIND == 0) {
                                    sfw_t = sfw_c + 4 * j;
                                    sfa_t = sfa_c + 4 * j * C::SF_TILES;
                                } else {
                                    idesc |= ((uint32_t)j << 29) | ((uint32_t)j << 4);
                                    sfw_t = sfw_c | ((uint32_t)j << 30);
                                    sfa_t = sfa_c | ((uint32_t)j << 30);
                                }
                                tc_mma_pair_if<KIND>(on, d_tmem, adesc0 + 2 * j, bdesc0 + 2 * j, idesc, sfw_t, sfa_t,
                                                     (kb > 0 || j > 0) ? 1u : 0u);
                            }
                        }
                    }
                    tc_commit_pair_if(on, empty0 + 8 * s);      // frees stage s in both CTAs
                    ++it;
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
                if (ok) tc_commit_pair_if(on, smem_u32(&tfull_bar[acc]));   // accumulator ready in both CTAs
            }
        }
        else {
            // peer CTA: this warp only relays "my operands of stage s have landed" to the leader, one
            // remote arrival per stage (crediting the peer's TMA bytes to a barrier in the leader
            // directly measured several times slower)
            uint32_t s = 0, ph = 0;
            bool ok = true;
            const uint32_t peer0_leader = map_to_cta(peer0, 0);
            for (int64_t tile = first; tile < total_tiles && ok; tile += stride) {
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(full0 + 8 * s, ph, abort_flag, 9)) { ok = false; break; }
                    if (lane == 0) mbar_arrive_cluster(peer0_leader + 8 * s);
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp < 6) {
        // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
        const int ew = warp & 3;
        uint32_t tcount = 0;
        bool ok = true;
        const uint32_t tempty_leader = map_to_cta(smem_u32(tempty_bar), 0);
        for (int64_t tile = first; tile < total_tiles && ok; tile += stride, ++tcount) {
            const int64_t np = tile / p.m_tiles, mt = tile - np * p.m_tiles;
            const uint32_t acc = tcount % C::ACC_STAGES;
            const uint32_t acc_ph = (tcount / C::ACC_STAGES) & 1u;
            if (!mbar_wait_parked(smem_u32(&tfull_bar[acc]), acc_ph, abort_flag, 4)) { ok = false; break; }
            tc_fence_after();
            drain_tile<BN>(p, tmem_base + acc * BN, ew, lane, (2 * np + rank) * BM, mt * BN, epi_stage, p.out, p.out_dtype, p.bias);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty_leader + 8 * acc);
        }
    } else {
        // ------------------------------------------------------------ scale loaders (warps 6..9, both CTAs)
        const int q = warp & 3;
        uint32_t s = 0, ph = 0, it = 0, s2 = 0, ph2 = 0;
        bool ok = true;
        const uint32_t sfw_base = smem_u32(sSFW), sfa_base = smem_u32(sSFA);
        const uint32_t sffull_leader = map_to_cta(smem_u32(sffull_bar), 0);
        for (int64_t tile = first; tile < total_tiles && ok; tile += stride) {
            for (int kb = 0; kb < k_blocks; ++kb) {
                if (!mbar_wait(sfl0 + 8 * s, ph, abort_flag, 6)) { ok = false; break; }
                if (it >= C::NSLOT) {
                    if (!mbar_wait(empty0 + 8 * s2, ph2, abort_flag, 7)) { ok = false; break; }
                    if (++s2 == STAGES) { s2 = 0; ph2 ^= 1u; }
                }
                tc_fence_after();
                const uint32_t slot = it % C::NSLOT;
                const uint32_t t_base = tmem_base + ((uint32_t)(q * 32) << 16) + C::SF_COL + slot * TMEM_SF_SLOT_COLS;
                if (!(p.debug & 2)) {
                    uint32_t v[C::ATOMS * 4];
                    const uint32_t src_w = sfw_base + s * C::SFW_BYTES + lane * 16;
#pragma unroll
                    for (int j = 0; j < C::ATOMS; ++j) ld_shared_v4(src_w + 512 * j, &v[4 * j]);
                    tc_st<C::ATOMS * 4>(t_base, v);
#pragma unroll
                    for (int t = 0; t < C::SF_TILES; ++t) {
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
                if (lane == 0) mbar_arrive_cluster(sffull_leader + 8 * slot);
                ++it;
                if (++s == STAGES) { s = 0; ph ^= 1u; }
            }
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
