// peer.cu -- the parts of the tensor-parallel exchange that sit beside the GEMM: staging buffers that other
// processes of the node can map (CUDA IPC), and the sum over the staged partial products that completes the
// reduce-scatter begun in the GEMM's push epilogue (gemm_duo.cuh, mode 3).  The reference project is single-GPU
// and has no counterpart of this file.
#include <type_traits>
#include <cstring>

#include "common.cuh"

namespace tfp4 {

namespace {

// out[i] = cast( sum_s stage[s * elems + i] ), s ascending (a fixed order: every rank and every run adds alike).
// 16 bytes of every slot per thread and step; the slots of one output element are read back to back.
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
sum_slots_kernel(const TI* __restrict__ stage, int n, int64_t elems, TO* __restrict__ out) {
    constexpr int V = 16 / sizeof(TI);      // elements per 16-byte load: 4 (f32) or 8 (f16, bf16)
    griddep_wait();
    const int64_t stride = (int64_t)gridDim.x * blockDim.x * V;
    for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * V; i < elems; i += stride) {
        float acc[V];
#pragma unroll
        for (int j = 0; j < V; ++j) acc[j] = 0.f;
        for (int s = 0; s < n; ++s) {
            const uint4 raw = *reinterpret_cast<const uint4*>(stage + (int64_t)s * elems + i);
            if constexpr (sizeof(TI) == 4) {
                acc[0] += __uint_as_float(raw.x); acc[1] += __uint_as_float(raw.y);
                acc[2] += __uint_as_float(raw.z); acc[3] += __uint_as_float(raw.w);
            } else {
                const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if constexpr (std::is_same<TI, __half>::value) {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
                        acc[2 * j] += f.x;
                        acc[2 * j + 1] += f.y;
                    } else {
                        acc[2 * j] += __uint_as_float(w[j] << 16);
                        acc[2 * j + 1] += __uint_as_float(w[j] & 0xffff0000u);
                    }
                }
            }
        }
        if constexpr (sizeof(TO) == 4) {
#pragma unroll
            for (int j = 0; j < V; j += 4)
                *reinterpret_cast<float4*>(out + i + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
        } else {
            uint32_t w[V / 2];
#pragma unroll
            for (int j = 0; j < V / 2; ++j) {
                const TO a = cast_out<TO>(acc[2 * j]), b = cast_out<TO>(acc[2 * j + 1]);
                w[j] = (uint32_t)(*reinterpret_cast<const uint16_t*>(&a)) | ((uint32_t)(*reinterpret_cast<const uint16_t*>(&b)) << 16);
            }
            if constexpr (V == 4) *reinterpret_cast<uint2*>(out + i) = make_uint2(w[0], w[1]);
            else *reinterpret_cast<uint4*>(out + i) = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
}

template <typename TI, typename TO>
int launch_sum(const void* stage, int n, int64_t elems, void* out, cudaStream_t stream) {
    constexpr int V = 16 / sizeof(TI);
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int64_t ctas = (elems / V + 255) / 256;
    if (ctas > (int64_t)sms * 8) ctas = (int64_t)sms * 8;
    sum_slots_kernel<TI, TO><<<(unsigned)ctas, 256, 0, stream>>>(static_cast<const TI*>(stage), n, elems, static_cast<TO*>(out));
    TFP4_CK(cudaGetLastError());
    return TFP4_OK;
}

}  // namespace

// stage: n slots of (rows, N) partial products, in_dtype 0 f32 / 1 f16 / 2 bf16 (the library's input-type codes);
// out (rows, N) of out_dtype 0 f16 / 1 bf16 / 2 f32.
int sum_slots(const void* stage, int n, int64_t rows, int64_t N, int in_dtype, void* out, int out_dtype, cudaStream_t stream) {
    const int64_t elems = rows * N;
    if (!stage || !out || n < 1 || elems <= 0 || (elems % 8) != 0 || (in_dtype != IN_F32 && in_dtype != IN_BF16 && in_dtype != IN_F16) ||
        out_dtype < 0 || out_dtype > 2 || (reinterpret_cast<uintptr_t>(stage) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) {
        fprintf(stderr, "thor_fp4: tfp4_sum_slots bad argument (f32, f16 or bf16 slots, rows * N %% 8 == 0, 16-byte aligned buffers)\n");
        return TFP4_ERR_BAD_ARG;
    }
#define TFP4_SUM(TI)                                                                         \
    switch (out_dtype) {                                                                     \
        case OUT_F32: return launch_sum<TI, float>(stage, n, elems, out, stream);            \
        case OUT_F16: return launch_sum<TI, __half>(stage, n, elems, out, stream);           \
        default: return launch_sum<TI, __nv_bfloat16>(stage, n, elems, out, stream);         \
    }
    if (in_dtype == IN_F32) { TFP4_SUM(float) } else if (in_dtype == IN_F16) { TFP4_SUM(__half) } else { TFP4_SUM(__nv_bfloat16) }
#undef TFP4_SUM
}

// A device buffer other processes of this node can map: cudaMalloc + an IPC handle (64 bytes) to hand to them.
int peer_alloc(size_t bytes, void** ptr, unsigned char* handle64) {
    if (!ptr || !handle64 || bytes == 0) return TFP4_ERR_BAD_ARG;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    TFP4_CK(cudaMalloc(ptr, bytes));
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, *ptr);
    if (e != cudaSuccess) {
        fprintf(stderr, "thor_fp4_b200: cudaIpcGetMemHandle failed: %s\n", cudaGetErrorString(e));
        cudaFree(*ptr);
        *ptr = nullptr;
        return TFP4_ERR_CUDA;
    }
    memcpy(handle64, &h, 64);
    return TFP4_OK;
}

// Map a buffer another process exported with peer_alloc; the pointer is valid on the current device (peer access
// over NVLink is enabled by the call).
int peer_open(const unsigned char* handle64, void** ptr) {
    if (!ptr || !handle64) return TFP4_ERR_BAD_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
        fprintf(stderr, "thor_fp4_b200: cudaIpcOpenMemHandle failed: %s\n", cudaGetErrorString(e));
        return TFP4_ERR_CUDA;
    }
    return TFP4_OK;
}

// One device-to-device copy on the stream (a peer destination goes over NVLink through the copy engines: no SM is used,
// so it runs beside a GEMM that occupies every SM).  One cudaMemcpyAsync per call.
int peer_copy(void* dst, const void* src, size_t bytes, cudaStream_t stream) {
    if (!dst || !src) return TFP4_ERR_BAD_ARG;
    if (bytes == 0) return TFP4_OK;
    TFP4_CK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, stream));
    return TFP4_OK;
}

int peer_close(void* ptr) {
    if (ptr) TFP4_CK(cudaIpcCloseMemHandle(ptr));
    return TFP4_OK;
}

int peer_free(void* ptr) {
    if (ptr) TFP4_CK(cudaFree(ptr));
    return TFP4_OK;
}

}  // namespace tfp4
