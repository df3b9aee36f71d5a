// api.cu -- the extern "C" surface of libthorfp4_b200.so (see include/thorfp4_b200.h).
#include <cstring>

#include "common.cuh"
#include "../../include/thorfp4_b200.h"

namespace tfp4 {
int quant_nvfp4(const void*, int64_t, int64_t, int, float, uint8_t*, uint8_t*, cudaStream_t);
int quant_mx(const void*, int64_t, int64_t, int, int, uint8_t*, uint8_t*, cudaStream_t);
int mx8_mul(const void*, const void*, const void*, const void*, void*, void*, int64_t, int64_t, cudaStream_t);
int dequant_f32(const uint8_t*, const uint8_t*, float, int64_t, int64_t, float*, cudaStream_t);
int scales_f32(const uint8_t*, int64_t, int64_t, float*, cudaStream_t);
int scales_gemv(const uint8_t*, int64_t, int64_t, uint8_t*, cudaStream_t);
int gemv(const void*, int64_t, int64_t, int, const uint8_t*, const uint8_t*, float, void*, int64_t, int, cudaStream_t);
int gemm_block_scaled(int, const void*, const void*, const void*, const void*, float, const float*, void*,
                      int64_t, int64_t, int64_t, int, cudaStream_t);
void gemm_set_token_tile(int);
void gemm_set_debug(int);
void gemm_set_raster(int);
void gemm_set_pair_mode(int);
void gemm_set_pdl(int);
void quant_set_pdl(int);
void gemm_set_splits(int);
void quant_set_tile_rows(int);
int act_quant_mx8(const void*, const float*, int64_t, int64_t, int, int, uint8_t*, uint8_t*, cudaStream_t);
int fake_quant_nvfp4(const void*, int64_t, int, float, void*, int, cudaStream_t);
int swiglu_quant_nvfp4(const void*, int64_t, int64_t, int, uint8_t*, uint8_t*, cudaStream_t);
int gemm_swiglu_nvfp4(const void*, const void*, const void*, const void*, float, void*, void*, int64_t, int64_t, int64_t,
                      cudaStream_t);
int gemm_mx8_out(const void*, const void*, const void*, const void*, float, const float*, int, void*, void*, int64_t,
                 int64_t, int64_t, cudaStream_t);
int gemm_push(const void*, const void*, const void*, const void*, float, void* const*, int, int64_t, int, int64_t, int64_t,
              int64_t, int, cudaStream_t);
int sum_slots(const void*, int, int64_t, int64_t, int, void*, int, cudaStream_t);
int peer_alloc(size_t, void**, unsigned char*);
int peer_open(const unsigned char*, void**);
int peer_close(void*);
int peer_copy(void*, const void*, size_t, cudaStream_t);
int peer_free(void*);
int gemm_noalloc(const void*, const void*, const void*, const void*, float, const float*, void*, int64_t, int64_t,
                 int64_t, int, cudaStream_t);
int gemm_noalloc_status(int);
size_t gemm_noalloc_capacity();
int gemm_debug_stats(unsigned long long*, int);
int gemm_status_word();
void gemm_clear_status();
void gemm_plan_stats(uint64_t*, uint64_t*);
int gemm_warm();
}  // namespace tfp4

namespace {
struct Variant { const char* name; int kind; };
// names of csrc/cutlass_kernels.cu:191-219 in the reference project (its MXFP4 x MXFP4
// entries compute garbage there and are not offered)
const Variant kVariants[] = {
    {"nvfp4_128x128x256_c1", 0},      {"nvfp4_128x128x256_c1_a32", 0},  {"nvfp4_128x128x256_c2x1", 0},
    {"nvfp4_128x256x256_c2x1", 0},    {"nvfp4_128x128x128_c1", 0},      {"nvfp4_128x128x64_c1", 0},
    {"mxfp8xfp4_128x128x256_c1", 1},  {"mxfp8xfp4_128x128x256_c2x1", 1}, {"mxfp8xfp4_128x256x256_c2x1", 1},
    {"mxfp8xfp4_128x128x128_c1", 1},  {"mxfp8xfp4_128x128x128_c2x1", 1}, {"mxfp8xfp4_128x256x128_c2x1", 1},
    {"mxfp8xfp4_256x128x256_c2x1", 1},
};
constexpr int kNVariants = (int)(sizeof(kVariants) / sizeof(kVariants[0]));
// names of csrc/fused_kernels.cu:224-247 in the reference project: activation of the epilogue; the tile numbers of a
// name select nothing here (one two-CTA kernel serves them all)
struct FusedVariant { const char* name; int act; };      // act: 0 identity, 1 gelu, 2 silu
const FusedVariant kFusedVariants[] = {
    {"mx8out_gelu_128x128x256_c1", 1},  {"mx8out_gelu_128x128x256_c2x1", 1}, {"mx8out_gelu_128x256x256_c2x1", 1},
    {"mx8out_gelu_128x128x128_c2x1", 1}, {"mx8out_silu_128x128x256_c1", 2},  {"mx8out_silu_128x256x256_c2x1", 2},
    {"mx8out_ident_128x128x256_c1", 0}, {"mx8out_ident_128x256x256_c2x1", 0},
};
constexpr int kNFusedVariants = (int)(sizeof(kFusedVariants) / sizeof(kFusedVariants[0]));
inline cudaStream_t S(void* s) { return static_cast<cudaStream_t>(s); }
}  // namespace

extern "C" {

int tfp4_init(size_t) { return tfp4::gemm_warm(); }
size_t tfp4_cublaslt_version(void) { return 1000000u + 100u * 0u + 1u; }

int64_t tfp4_pad_rows(int64_t R) { return tfp4::pad128(R); }
int64_t tfp4_packed_bytes(int64_t R, int64_t K) { return tfp4::pad128(R) * K / 2; }
int64_t tfp4_scale_bytes(int64_t R, int64_t K) { return tfp4::pad128(R) * ((K / 16 + 3) / 4 * 4); }
int64_t tfp4_mx_packed_bytes(int64_t R, int64_t K, int kind) { return tfp4::pad128(R) * (kind == 0 ? K / 2 : K); }
int64_t tfp4_mx_scale_bytes(int64_t R, int64_t K) { return tfp4::pad128(R) * ((K / 32 + 3) / 4 * 4); }

int tfp4_quant(const void* x, int64_t R, int64_t K, int in_dtype, float ts, uint8_t* packed, uint8_t* sblk,
               void* stream) {
    return tfp4::quant_nvfp4(x, R, K, in_dtype, ts, packed, sblk, S(stream));
}
int tfp4_quant_mx(const void* x, int64_t R, int64_t K, int in_dtype, int kind, uint8_t* packed, uint8_t* sblk,
                  void* stream) {
    return tfp4::quant_mx(x, R, K, in_dtype, kind, packed, sblk, S(stream));
}
int tfp4_mx8_mul(const void* ap, const void* as, const void* bp, const void* bs, void* op, void* os, int64_t R,
                 int64_t K, void* stream) {
    return tfp4::mx8_mul(ap, as, bp, bs, op, os, R, K, S(stream));
}
int tfp4_gemm(const void* pA, const void* sA, float tsA, const void* pB, const void* sB, float tsB, void* out,
              int64_t M, int64_t N, int64_t K, int out_dtype, void* stream) {
    if ((K % 64) != 0) {
        fprintf(stderr, "thor_fp4: K must be a multiple of 64 (got %ld)\n", (long)K);
        return TFP4_ERR_BAD_K;
    }
    return tfp4::gemm_block_scaled(0, pA, sA, pB, sB, tsA * tsB, nullptr, out, M, N, K, out_dtype, S(stream));
}
int tfp4_gemm_bias(const void* pA, const void* sA, float tsA, const void* pB, const void* sB, float tsB,
                   const float* bias, void* out, int64_t M, int64_t N, int64_t K, int out_dtype, void* stream) {
    return tfp4::gemm_block_scaled(0, pA, sA, pB, sB, tsA * tsB, bias, out, M, N, K, out_dtype, S(stream));
}
int tfp4_linear(const void* x, int64_t M, int64_t K, int in_dtype, float act_ts, uint8_t* act_packed, uint8_t* act_sblk,
                const void* w_packed, const void* w_sblk, float w_ts, const float* bias, void* out, int64_t N,
                int out_dtype, void* stream) {
    int rc = tfp4_quant(x, M, K, in_dtype, act_ts, act_packed, act_sblk, stream);
    if (rc) return rc;
    return tfp4_gemm_bias(act_packed, act_sblk, act_ts, w_packed, w_sblk, w_ts, bias, out, M, N, K, out_dtype, stream);
}
int tfp4_gemv(const void* x, int64_t M, int64_t K, int in_dtype, const uint8_t* pB, const uint8_t* sg, float tsB,
              void* out, int64_t N, int out_dtype, void* stream) {
    return tfp4::gemv(x, M, K, in_dtype, pB, sg, tsB, out, N, out_dtype, S(stream));
}
int tfp4_scales_gemv(const uint8_t* sblk, int64_t R, int64_t K, uint8_t* out, void* stream) {
    return tfp4::scales_gemv(sblk, R, K, out, S(stream));
}
int tfp4_dequant_f32(const uint8_t* packed, const uint8_t* sblk, float ts, int64_t R, int64_t K, float* out,
                     void* stream) {
    return tfp4::dequant_f32(packed, sblk, ts, R, K, out, S(stream));
}
int tfp4_scales_f32(const uint8_t* sblk, int64_t R, int64_t K, float* out, void* stream) {
    return tfp4::scales_f32(sblk, R, K, out, S(stream));
}

int tfc4_n_variants(void) { return kNVariants; }
const char* tfc4_variant_name(int i) { return (i >= 0 && i < kNVariants) ? kVariants[i].name : nullptr; }
int tfc4_variant_index(const char* name) {
    if (!name) return -1;
    for (int i = 0; i < kNVariants; ++i)
        if (strcmp(name, kVariants[i].name) == 0) return i;
    return -1;
}
int tfc4_gemm(int variant, const void* A, const void* SA, const void* B, const void* SB, void* D, int64_t M,
              int64_t N, int64_t K, float alpha, void* stream) {
    if (variant < 0 || variant >= kNVariants) {
        fprintf(stderr, "thor_fp4: bad variant %d (0..%d)\n", variant, kNVariants - 1);
        return TFP4_ERR_CUDA;
    }
    return tfp4::gemm_block_scaled(kVariants[variant].kind, A, SA, B, SB, alpha, nullptr, D, M, N, K,
                                   tfp4::OUT_BF16, S(stream));
}

int tfc4_gemm_ex(int variant, const void* A, const void* SA, const void* B, const void* SB, const float* bias, void* D,
                 int64_t M, int64_t N, int64_t K, float alpha, int out_dtype, void* stream) {
    if (variant < 0 || variant >= kNVariants) {
        fprintf(stderr, "thor_fp4: bad variant %d (0..%d)\n", variant, kNVariants - 1);
        return TFP4_ERR_CUDA;
    }
    return tfp4::gemm_block_scaled(kVariants[variant].kind, A, SA, B, SB, alpha, bias, D, M, N, K, out_dtype, S(stream));
}

int tfc4f_n_variants(void) { return kNFusedVariants; }
const char* tfc4f_variant_name(int i) { return (i >= 0 && i < kNFusedVariants) ? kFusedVariants[i].name : nullptr; }
int tfc4f_variant_index(const char* name) {
    if (!name) return -1;
    for (int i = 0; i < kNFusedVariants; ++i)
        if (strcmp(name, kFusedVariants[i].name) == 0) return i;
    return -1;
}
int64_t tfc4f_sfd_bytes(int64_t M, int64_t N) { return tfp4::pad128(M) * ((N / 32 + 3) / 4 * 4); }
int tfc4f_gemm(int variant, const void* A, const void* SA, const void* B, const void* SB, const float* bias, void* D,
               void* SFD, int64_t M, int64_t N, int64_t K, float alpha, void* stream) {
    // argument checks and their codes as in the reference (csrc/fused_kernels.cu:423-445)
    if (variant < 0 || variant >= kNFusedVariants) {
        fprintf(stderr, "thor_fp4 fused: bad variant %d (0..%d)\n", variant, kNFusedVariants - 1);
        return -1;
    }
    if (K % 128 != 0) {
        fprintf(stderr, "thor_fp4 fused: K must be a multiple of 128 (got %ld)\n", (long)K);
        return -3;
    }
    if (N % 32 != 0) {
        fprintf(stderr, "thor_fp4 fused: N must be a multiple of 32 (got %ld)\n", (long)N);
        return -4;
    }
    if (!bias) {
        fprintf(stderr, "thor_fp4 fused: bias pointer is required (pass zeros)\n");
        return -5;
    }
    return tfp4::gemm_mx8_out(A, SA, B, SB, alpha, bias, kFusedVariants[variant].act, D, SFD, M, N, K, S(stream));
}

int tfp4_swiglu_gemm(const void* pA, const void* sA, float tsA, const void* pW, const void* sW, float tsW, void* h_packed,
                     void* h_sblk, int64_t M, int64_t N, int64_t K, void* stream) {
    return tfp4::gemm_swiglu_nvfp4(pA, sA, pW, sW, tsA * tsW, h_packed, h_sblk, M, N, K, S(stream));
}

int tfp4_gemm_push(const void* pA, const void* sA, float tsA, const void* pB, const void* sB, float tsB, void* const* dest,
                   int n_dest, int64_t rows_per_dest, int first_dest, int64_t M, int64_t N, int64_t K, int out_dtype,
                   void* stream) {
    return tfp4::gemm_push(pA, sA, pB, sB, tsA * tsB, dest, n_dest, rows_per_dest, first_dest, M, N, K, out_dtype, S(stream));
}
int tfp4_sum_slots(const void* stage, int n, int64_t rows, int64_t N, int in_dtype, void* out, int out_dtype, void* stream) {
    return tfp4::sum_slots(stage, n, rows, N, in_dtype, out, out_dtype, S(stream));
}
int tfp4_peer_alloc(size_t bytes, void** ptr, unsigned char* handle64) { return tfp4::peer_alloc(bytes, ptr, handle64); }
int tfp4_peer_open(const unsigned char* handle64, void** ptr) { return tfp4::peer_open(handle64, ptr); }
int tfp4_peer_close(void* ptr) { return tfp4::peer_close(ptr); }
int tfp4_peer_copy(void* dst, const void* src, size_t bytes, void* stream) { return tfp4::peer_copy(dst, src, bytes, S(stream)); }
int tfp4_peer_free(void* ptr) { return tfp4::peer_free(ptr); }

int tfp4_swiglu_quant(const void* gu, int64_t R, int64_t I, int in_dtype, uint8_t* packed, uint8_t* sblk, void* stream) {
    return tfp4::swiglu_quant_nvfp4(gu, R, I, in_dtype, packed, sblk, S(stream));
}

int tfp4_act_quant_mx8(const void* acc, const float* bias, int64_t R, int64_t N, int in_dtype, int act, uint8_t* packed,
                       uint8_t* sblk, void* stream) {
    return tfp4::act_quant_mx8(acc, bias, R, N, in_dtype, act, packed, sblk, S(stream));
}

int tfp4_fake_quant(const void* x, int64_t n, int in_dtype, float tensor_scale, void* y, int out_dtype, void* stream) {
    return tfp4::fake_quant_nvfp4(x, n, in_dtype, tensor_scale, y, out_dtype, S(stream));
}

int tfp4_gemm_noalloc(const void* pA, const void* sA, float tsA, const void* pB, const void* sB, float tsB,
                      const float* bias, void* out, int64_t M, int64_t N, int64_t K, int out_dtype, void* stream) {
    if ((K % 64) != 0) {
        fprintf(stderr, "thor_fp4: K must be a multiple of 64 (got %ld)\n", (long)K);
        return TFP4_ERR_BAD_K;
    }
    return tfp4::gemm_noalloc(pA, sA, pB, sB, tsA * tsB, bias, out, M, N, K, out_dtype, S(stream));
}
int tfp4_gemm_noalloc_status(int reset) { return tfp4::gemm_noalloc_status(reset); }
size_t tfp4_gemm_noalloc_capacity(void) { return tfp4::gemm_noalloc_capacity(); }

void tfp4_set_quant_tile_rows(int rows) { tfp4::quant_set_tile_rows(rows); }
int tfp4_status(void) { return tfp4::gemm_status_word(); }
void tfp4_clear_status(void) { tfp4::gemm_clear_status(); }
void tfp4_plan_stats(uint64_t* hits, uint64_t* misses) { tfp4::gemm_plan_stats(hits, misses); }
void tfp4_set_token_tile(int bn) { tfp4::gemm_set_token_tile(bn); }
void tfp4_set_debug(int bits) { tfp4::gemm_set_debug(bits); }
void tfp4_set_raster(int gm) { tfp4::gemm_set_raster(gm); }
void tfp4_set_pair_mode(int mode) { tfp4::gemm_set_pair_mode(mode); }
void tfp4_set_dependent_launch(int on) {
    tfp4::gemm_set_pdl(on);
    tfp4::quant_set_pdl(on);
}
void tfp4_set_splits(int n) { tfp4::gemm_set_splits(n); }
int tfp4_debug_stats(unsigned long long* out, int n_ctas) { return tfp4::gemm_debug_stats(out, n_ctas); }

}  // extern "C"
