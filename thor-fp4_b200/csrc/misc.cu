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
// accumulation (csrc/thor_fp4_core.cu:412-518).  Bandwidth-bound: a warp
// streams RPW weight rows with one 16-byte load per lane per row (32 codes)
// plus the two scale bytes from the un-scattered (N, K/16) copy; the M x 1024
// activation chunk sits in shared memory transposed so that lane l reads word
// j*32 + l without bank conflicts.  Each 16-code block is accumulated against
// the activations first and scaled once.
// ---------------------------------------------------------------------------
constexpr int GV_THREADS = 256;
constexpr int GV_RPW = 4;        // weight rows per warp
constexpr int GV_KC = 1024;      // activation chunk = 32 lanes x 32 codes

template <typename XT>
__device__ __forceinline__ float to_f32(XT v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename XT, int MT>
__global__ void __launch_bounds__(GV_THREADS)
gemv_nvfp4_kernel(const XT* __restrict__ x, int M, const uint8_t* __restrict__ pB,
                  const uint8_t* __restrict__ sgemv, float ts, int64_t N, int64_t K,
                  void* __restrict__ out, int out_dtype) {
    __shared__ float xs[MT * GV_KC];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t S = K >> 4;
    const int64_t n0 = ((int64_t)blockIdx.x * (GV_THREADS / 32) + warp) * GV_RPW;
    float acc[GV_RPW][MT];
#pragma unroll
    for (int rr = 0; rr < GV_RPW; ++rr)
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[rr][m] = 0.f;

    for (int64_t c0 = 0; c0 < K; c0 += GV_KC) {
        const int ce = (int)((K - c0 < GV_KC) ? (K - c0) : GV_KC);
        __syncthreads();
        for (int i = threadIdx.x; i < MT * GV_KC; i += GV_THREADS) {
            const int m = i / GV_KC, kk = i - m * GV_KC;
            float v = 0.f;
            if (m < M && kk < ce) v = to_f32<XT>(x[(int64_t)m * K + c0 + kk]);
            xs[m * GV_KC + (kk & 31) * 32 + (kk >> 5)] = v;
        }
        __syncthreads();
        const int k_lane = lane * 32;
        if (k_lane < ce) {
            uint4 w[GV_RPW];
            uint32_t sc[GV_RPW];
#pragma unroll
            for (int rr = 0; rr < GV_RPW; ++rr) {
                const int64_t n = n0 + rr;
                if (n < N) {
                    w[rr] = __ldg(reinterpret_cast<const uint4*>(pB + n * (K >> 1) + ((c0 + k_lane) >> 1)));
                    sc[rr] = *reinterpret_cast<const unsigned short*>(sgemv + n * S + ((c0 + k_lane) >> 4));
                } else {
                    w[rr] = make_uint4(0u, 0u, 0u, 0u);
                    sc[rr] = 0u;
                }
            }
#pragma unroll
            for (int half = 0; half < 2; ++half) {       // two 16-code blocks per lane
                float part[GV_RPW][MT];
#pragma unroll
                for (int rr = 0; rr < GV_RPW; ++rr)
#pragma unroll
                    for (int m = 0; m < MT; ++m) part[rr][m] = 0.f;
#pragma unroll
                for (int b = 0; b < 8; ++b) {            // 8 bytes = 16 codes
                    const int j = half * 16 + 2 * b;     // element index inside the lane's 32
                    float xa[MT], xb[MT];
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        xa[m] = xs[m * GV_KC + j * 32 + lane];
                        xb[m] = xs[m * GV_KC + (j + 1) * 32 + lane];
                    }
#pragma unroll
                    for (int rr = 0; rr < GV_RPW; ++rr) {
                        const uint32_t word = half == 0 ? (b < 4 ? w[rr].x : w[rr].y) : (b < 4 ? w[rr].z : w[rr].w);
                        float lo, hi;
                        e2m1x2_to_f32x2((word >> (8 * (b & 3))) & 0xffu, lo, hi);
#pragma unroll
                        for (int m = 0; m < MT; ++m) {
                            part[rr][m] = fmaf(lo, xa[m], part[rr][m]);
                            part[rr][m] = fmaf(hi, xb[m], part[rr][m]);
                        }
                    }
                }
#pragma unroll
                for (int rr = 0; rr < GV_RPW; ++rr) {
                    const float s = e4m3_to_f32((sc[rr] >> (8 * half)) & 0xffu) * ts;
#pragma unroll
                    for (int m = 0; m < MT; ++m) acc[rr][m] = fmaf(part[rr][m], s, acc[rr][m]);
                }
            }
        }
    }
#pragma unroll
    for (int rr = 0; rr < GV_RPW; ++rr) {
        const int64_t n = n0 + rr;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float v = acc[rr][m];
#pragma unroll
            for (int off = 16; off; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
            if (lane == 0 && n < N && m < M) {
                const int64_t o = (int64_t)m * N + n;
                if (out_dtype == OUT_F16) reinterpret_cast<__half*>(out)[o] = __float2half_rn(v);
                else if (out_dtype == OUT_BF16) reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(v);
                else reinterpret_cast<float*>(out)[o] = v;
            }
        }
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
    const int rows_per_cta = (GV_THREADS / 32) * GV_RPW;
    const unsigned grid = (unsigned)((N + rows_per_cta - 1) / rows_per_cta);
    const XT* xp = static_cast<const XT*>(x);
    const int m = (int)M;
    if (M <= 1) gemv_nvfp4_kernel<XT, 1><<<grid, GV_THREADS, 0, stream>>>(xp, m, pB, sg, ts, N, K, out, out_dtype);
    else if (M <= 2) gemv_nvfp4_kernel<XT, 2><<<grid, GV_THREADS, 0, stream>>>(xp, m, pB, sg, ts, N, K, out, out_dtype);
    else if (M <= 4) gemv_nvfp4_kernel<XT, 4><<<grid, GV_THREADS, 0, stream>>>(xp, m, pB, sg, ts, N, K, out, out_dtype);
    else gemv_nvfp4_kernel<XT, 8><<<grid, GV_THREADS, 0, stream>>>(xp, m, pB, sg, ts, N, K, out, out_dtype);
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
    switch (in_dtype) {
        case IN_F32: return launch_gemv<float>(x, M, K, packedB, sgemvB, tsB, out, N, out_dtype, stream);
        case IN_F16: return launch_gemv<__half>(x, M, K, packedB, sgemvB, tsB, out, N, out_dtype, stream);
        default: return launch_gemv<__nv_bfloat16>(x, M, K, packedB, sgemvB, tsB, out, N, out_dtype, stream);
    }
}

}  // namespace tfp4
