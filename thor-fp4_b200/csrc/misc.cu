// misc.cu -- dequantize, scale un-scatter and the register-dequant GEMV.
//
// These are the diagnostic / small-batch companions of the quantizer and the
// tensor-core GEMM; their arithmetic follows the reference kernels exactly
// where a bit pattern is produced (dequantize, scale decode) and to FP32
// rounding where a sum is produced (GEMV).
#include "common.cuh"

namespace tfp4 {

namespace {

// NVFP4 -> f32: value = (lut[code] * sign) * (dec(sf) * ts); one thread per
// 16-element block.  csrc/thor_fp4_core.cu:321-339.
__global__ void __launch_bounds__(256)
dequant_f32_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ sblk, float ts,
                   int64_t R, int64_t K, float* __restrict__ out) {
    const int64_t S = K >> 4;
    const int64_t total = R * S;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / S, s = i - r * S;
        const float ds = e4m3_to_f32(sblk[sf_index(r, s, S)]) * ts;
        const uint2 c = __ldg(reinterpret_cast<const uint2*>(packed + r * (K >> 1) + s * 8));
        const uint32_t w[2] = {c.x, c.y};
        float4* dst = reinterpret_cast<float4*>(out + r * K + s * 16);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float v[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                e2m1x2_to_f32x2((w[h] >> (8 * j)) & 0xffu, v[2 * j], v[2 * j + 1]);
                v[2 * j] *= ds;
                v[2 * j + 1] *= ds;
            }
            dst[2 * h] = make_float4(v[0], v[1], v[2], v[3]);
            dst[2 * h + 1] = make_float4(v[4], v[5], v[6], v[7]);
        }
    }
}

// tile-layout UE4M3 bytes -> plain f32 (R, K/16).  csrc/thor_fp4_core.cu:353-362.
__global__ void __launch_bounds__(256)
scales_f32_kernel(const uint8_t* __restrict__ sblk, int64_t R, int64_t S, float* __restrict__ out) {
    const int64_t total = R * S;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / S, s = i - r * S;
        out[i] = e4m3_to_f32(sblk[sf_index(r, s, S)]);
    }
}

// tile-layout bytes -> plain (R, K/16) bytes.  csrc/thor_fp4_core.cu:343-351.
// One thread moves the 4 bytes that are adjacent in both layouts.
__global__ void __launch_bounds__(256)
scales_gemv_kernel(const uint8_t* __restrict__ sblk, int64_t R, int64_t S, uint8_t* __restrict__ out) {
    const int64_t D = S >> 2;
    const int64_t total = R * D;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / D, d = i - r * D;
        const uint32_t v = *reinterpret_cast<const uint32_t*>(sblk + sf_index(r, 4 * d, S));
        *reinterpret_cast<uint32_t*>(out + r * S + 4 * d) = v;
    }
}

// ---------------------------------------------------------------------------
// GEMV: out (M<=8, N) = x (M, K) @ dequant(W)^T, activations exact, FP32
// accumulation (csrc/thor_fp4_core.cu:412-518).  Weight-streaming kernel:
//   * a lane owns a fixed run of CPL codes (16 bytes = two blocks for M <= 2, 8 bytes = one block
//     above) of the K axis and keeps the matching activations of all M rows in registers, so the
//     inner loop reads nothing but weights: one 16-/8-byte load plus the block scale bytes per row;
//   * a warp covers 32 * CPL consecutive codes of a row per load (512 / 256 contiguous bytes); the
//     8 warps of a CTA take the K chunks round-robin (K = 8192, M <= 2: one chunk each, activations
//     loaded once);
//   * a CTA owns a contiguous, balanced range of weight rows and walks it four rows at a time with
//     the next four rows' loads already in flight;
//   * per row: 16 codes are accumulated against the activations, scaled once by dec(scale) * ts,
//     reduced over the warp by shuffles, and added by lane 0 to this warp's slot in shared memory;
//     the 8 slots are summed in a fixed order at the end (deterministic).
// ---------------------------------------------------------------------------
constexpr int GV_THREADS = 256;
constexpr int GV_WARPS = GV_THREADS / 32;
constexpr int GV_RU = 4;            // rows per step (two steps in flight)
constexpr int GV_MAX_ROWS = 64;     // rows per CTA (shared-memory slots)

template <int LB> struct GvRaw;
template <> struct GvRaw<16> { uint4 w; uint32_t sc; };
template <> struct GvRaw<8> { uint2 w; uint32_t sc; };

template <int LB>
__device__ __forceinline__ GvRaw<LB> gv_fetch(const uint8_t* wp, const uint8_t* sp, bool on) {
    GvRaw<LB> r;
    if constexpr (LB == 16) {
        r.w = on ? __ldg(reinterpret_cast<const uint4*>(wp)) : make_uint4(0u, 0u, 0u, 0u);
        r.sc = on ? (uint32_t)__ldg(reinterpret_cast<const unsigned short*>(sp)) : 0u;
    } else {
        r.w = on ? __ldg(reinterpret_cast<const uint2*>(wp)) : make_uint2(0u, 0u);
        r.sc = on ? (uint32_t)__ldg(sp) : 0u;
    }
    return r;
}

template <typename XT, int MT, int LB>
__global__ void __launch_bounds__(GV_THREADS, (MT <= 4) ? 2 : 1)
gemv_nvfp4_kernel(const XT* __restrict__ x, int M, const uint8_t* __restrict__ pB,
                  const uint8_t* __restrict__ sgemv, float ts, int64_t N, int64_t K,
                  void* __restrict__ out, int out_dtype) {
    constexpr int CPL = 2 * LB;          // codes per lane per row
    constexpr int BPL = CPL / 16;        // scale blocks per lane per row
    constexpr int CHUNK = 32 * CPL;      // codes per warp per row
    __shared__ float sacc[GV_WARPS][GV_MAX_ROWS][MT];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t S = K >> 4;
    // balanced contiguous row range of this CTA (at most GV_MAX_ROWS rows: the grid is sized for that)
    const int64_t n_begin = (N * (int64_t)blockIdx.x) / gridDim.x;
    const int64_t n_end = (N * ((int64_t)blockIdx.x + 1)) / gridDim.x;
    const int rows = (int)(n_end - n_begin);
    for (int i = threadIdx.x; i < GV_WARPS * GV_MAX_ROWS * MT; i += GV_THREADS) (&sacc[0][0][0])[i] = 0.f;
    __syncthreads();

    const int n_chunks = (int)((K + CHUNK - 1) / CHUNK);
    for (int c = warp; c < n_chunks; c += GV_WARPS) {
        const int64_t k0 = (int64_t)c * CHUNK + lane * CPL;
        const bool on = k0 < K;          // K % 64 == 0: a lane's run is inside or outside as a whole
        float xr[MT][CPL];
#pragma unroll
        for (int m = 0; m < MT; ++m) {
#pragma unroll
            for (int j = 0; j < CPL; j += 8) {
                float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                if (on && m < M) load8<XT>(x + (int64_t)m * K + k0 + j, f);
#pragma unroll
                for (int i = 0; i < 8; ++i) xr[m][j + i] = f[i];
            }
        }
        const uint8_t* wp = pB + n_begin * (K >> 1) + (k0 >> 1);
        const uint8_t* sp = sgemv + n_begin * S + (k0 >> 4);
        GvRaw<LB> cur[GV_RU], nxt[GV_RU];
#pragma unroll
        for (int u = 0; u < GV_RU; ++u) cur[u] = gv_fetch<LB>(wp + (int64_t)u * (K >> 1), sp + (int64_t)u * S, on && u < rows);
        for (int r0 = 0; r0 < rows; r0 += GV_RU) {
#pragma unroll
            for (int u = 0; u < GV_RU; ++u) {
                const int rn = r0 + GV_RU + u;
                nxt[u] = gv_fetch<LB>(wp + (int64_t)rn * (K >> 1), sp + (int64_t)rn * S, on && rn < rows);
            }
#pragma unroll
            for (int u = 0; u < GV_RU; ++u) {
                uint32_t words[LB / 4];
                if constexpr (LB == 16) { words[0] = cur[u].w.x; words[1] = cur[u].w.y; words[2] = cur[u].w.z; words[3] = cur[u].w.w; }
                else { words[0] = cur[u].w.x; words[1] = cur[u].w.y; }
                float acc[MT];
#pragma unroll
                for (int m = 0; m < MT; ++m) acc[m] = 0.f;
#pragma unroll
                for (int blk = 0; blk < BPL; ++blk) {
                    float part[MT];
#pragma unroll
                    for (int m = 0; m < MT; ++m) part[m] = 0.f;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {        // two words = 16 codes = one scale block
                        float wv[8];
                        e2m1x8_to_f32x8(words[blk * 2 + h], wv);
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
#pragma unroll
                            for (int m = 0; m < MT; ++m) part[m] = fmaf(wv[i], xr[m][blk * 16 + 8 * h + i], part[m]);
                        }
                    }
                    const float sc = e4m3_to_f32((cur[u].sc >> (8 * blk)) & 0xffu) * ts;
#pragma unroll
                    for (int m = 0; m < MT; ++m) acc[m] = fmaf(part[m], sc, acc[m]);
                }
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    float v = acc[m];
#pragma unroll
                    for (int off = 16; off; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
                    if (lane == 0 && r0 + u < rows) sacc[warp][r0 + u][m] += v;
                }
            }
#pragma unroll
            for (int u = 0; u < GV_RU; ++u) cur[u] = nxt[u];
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < rows * MT; i += GV_THREADS) {
        const int r = i / MT, m = i - r * MT;
        if (m >= M) continue;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < GV_WARPS; ++w) v += sacc[w][r][m];
        const int64_t o = (int64_t)m * N + n_begin + r;
        if (out_dtype == OUT_F16) reinterpret_cast<__half*>(out)[o] = __float2half_rn(v);
        else if (out_dtype == OUT_BF16) reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(v);
        else reinterpret_cast<float*>(out)[o] = v;
    }
}
unsigned blocks_for(int64_t total, int threads) {
    int64_t b = (total + threads - 1) / threads;
    const int64_t cap = 148 * 16;
    return (unsigned)(b < 1 ? 1 : (b > cap ? cap : b));
}

template <typename XT>
int launch_gemv(const void* x, int64_t M, int64_t K, const uint8_t* pB, const uint8_t* sg, float ts,
                void* out, int64_t N, int out_dtype, cudaStream_t stream) {
    // two CTAs per SM for M <= 4 (one for 5..8 rows, whose activations fill the registers); more CTAs
    // when the rows per CTA would exceed the shared-memory slots
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int64_t ctas = (int64_t)sms * (M <= 4 ? 2 : 1);
    const int64_t need = (N + GV_MAX_ROWS - 1) / GV_MAX_ROWS;
    if (ctas < need) ctas = need;
    if (ctas > N) ctas = N;
    const unsigned grid = (unsigned)ctas;
    const XT* xp = static_cast<const XT*>(x);
    const int m = (int)M;
    if (M <= 1) gemv_nvfp4_kernel<XT, 1, 16><<<grid, GV_THREADS, 0, stream>>>(xp, m, pB, sg, ts, N, K, out, out_dtype);
    else if (M <= 2) gemv_nvfp4_kernel<XT, 2, 16><<<grid, GV_THREADS, 0, stream>>>(xp, m, pB, sg, ts, N, K, out, out_dtype);
    else if (M <= 4) gemv_nvfp4_kernel<XT, 4, 8><<<grid, GV_THREADS, 0, stream>>>(xp, m, pB, sg, ts, N, K, out, out_dtype);
    else if (M <= 6) gemv_nvfp4_kernel<XT, 6, 8><<<grid, GV_THREADS, 0, stream>>>(xp, m, pB, sg, ts, N, K, out, out_dtype);
    else gemv_nvfp4_kernel<XT, 8, 8><<<grid, GV_THREADS, 0, stream>>>(xp, m, pB, sg, ts, N, K, out, out_dtype);
    TFP4_CK(cudaGetLastError());
    return TFP4_OK;
}

}  // namespace

int dequant_f32(const uint8_t* packed, const uint8_t* sblk, float ts, int64_t R, int64_t K,
                float* out, cudaStream_t stream) {
    if (K <= 0 || (K % 64) != 0) return TFP4_ERR_BAD_K;
    if (R <= 0) return TFP4_OK;
    if ((reinterpret_cast<uintptr_t>(packed) & 7) || (reinterpret_cast<uintptr_t>(out) & 15)) {
        fprintf(stderr, "thor_fp4: tfp4_dequant_f32 needs packed 8-byte and out 16-byte aligned\n");
        return TFP4_ERR_BAD_ARG;
    }
    dequant_f32_kernel<<<blocks_for(R * (K >> 4), 256), 256, 0, stream>>>(packed, sblk, ts, R, K, out);
    TFP4_CK(cudaGetLastError());
    return TFP4_OK;
}

int scales_f32(const uint8_t* sblk, int64_t R, int64_t K, float* out, cudaStream_t stream) {
    if (K <= 0 || (K % 64) != 0) return TFP4_ERR_BAD_K;
    if (R <= 0) return TFP4_OK;
    scales_f32_kernel<<<blocks_for(R * (K >> 4), 256), 256, 0, stream>>>(sblk, R, K >> 4, out);
    TFP4_CK(cudaGetLastError());
    return TFP4_OK;
}

int scales_gemv(const uint8_t* sblk, int64_t R, int64_t K, uint8_t* out, cudaStream_t stream) {
    if (K <= 0 || (K % 64) != 0) return TFP4_ERR_BAD_K;
    if (R <= 0) return TFP4_OK;
    if ((reinterpret_cast<uintptr_t>(sblk) & 3) || (reinterpret_cast<uintptr_t>(out) & 3)) {
        fprintf(stderr, "thor_fp4: tfp4_scales_gemv needs 4-byte aligned buffers\n");
        return TFP4_ERR_BAD_ARG;
    }
    scales_gemv_kernel<<<blocks_for(R * (K >> 6), 256), 256, 0, stream>>>(sblk, R, K >> 4, out);
    TFP4_CK(cudaGetLastError());
    return TFP4_OK;
}

int gemv(const void* x, int64_t M, int64_t K, int in_dtype, const uint8_t* packedB,
         const uint8_t* sgemvB, float tsB, void* out, int64_t N, int out_dtype, cudaStream_t stream) {
    if (M < 1 || M > 8) {
        fprintf(stderr, "thor_fp4 gemv: M must be 1..8 (got %ld)\n", (long)M);
        return TFP4_ERR_BAD_M;
    }
    if (K <= 0 || (K % 64) != 0) {
        fprintf(stderr, "thor_fp4 gemv: K must be a multiple of 64 (got %ld)\n", (long)K);
        return TFP4_ERR_BAD_K;
    }
    if (N <= 0 || !x || !packedB || !sgemvB || !out || in_dtype < 0 || in_dtype > 2 || out_dtype < 0 ||
        out_dtype > 2 || (reinterpret_cast<uintptr_t>(packedB) & 15) || (reinterpret_cast<uintptr_t>(sgemvB) & 1)) {
        fprintf(stderr, "thor_fp4 gemv: bad argument (weights must be 16-byte aligned)\n");
        return TFP4_ERR_BAD_ARG;
    }
    if (reinterpret_cast<uintptr_t>(x) & (in_dtype == IN_F32 ? 31 : 15)) {
        fprintf(stderr, "thor_fp4 gemv: activations must be 16-byte (f32: 32-byte) aligned\n");
        return TFP4_ERR_BAD_ARG;
    }
    switch (in_dtype) {
        case IN_F32: return launch_gemv<float>(x, M, K, packedB, sgemvB, tsB, out, N, out_dtype, stream);
        case IN_F16: return launch_gemv<__half>(x, M, K, packedB, sgemvB, tsB, out, N, out_dtype, stream);
        default: return launch_gemv<__nv_bfloat16>(x, M, K, packedB, sgemvB, tsB, out, N, out_dtype, stream);
    }
}

}  // namespace tfp4
