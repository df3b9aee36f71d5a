/*
 * thorfp4_b200.h -- C ABI of libthorfp4_b200.so, the sm_100a NVFP4 linear-layer engine.
 *
 * Drop-in for the entry points the thor-fp4 Python binding loads with ctypes
 * (src/thor_fp4/_ext.py:36-94 of that project): same names, argument order,
 * argument meaning and error convention (0 on success, a negative code and one
 * line on stderr otherwise).  Every pointer is a raw device pointer owned by
 * the caller; `stream` is a cudaStream_t passed as void*; calls only enqueue
 * work on that stream and never synchronise.  Buffers are sized with the
 * *_bytes helpers (rows padded to 128, scale columns to 4).
 *
 * Error codes: -1 CUDA runtime, -2 driver entry point / tensor-map encode,
 * -3 bad K, -4 no kernel configuration, -5 launch failed, -6 bad M or N,
 * -7 bad pointer / alignment / enum, -8 an earlier GEMM on this device ran
 * into its bounded wait (see tfp4_status).
 */
#ifndef THORFP4_B200_H
#define THORFP4_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* in_dtype: 0 f32, 1 f16, 2 bf16.   out_dtype: 0 f16, 1 bf16, 2 f32. */

/* Replaces tfp4_init (csrc/thor_fp4_core.cu:524-531).  Resolves the driver entry
 * point and the per-device state of the current device; ws_bytes is accepted and
 * ignored (no library workspace exists). */
int tfp4_init(size_t ws_bytes);

/* Replaces tfp4_cublaslt_version (csrc/thor_fp4_core.cu:533).  No cuBLASLt is
 * linked; returns the build id of this library (1000000 + 100*major + minor). */
size_t tfp4_cublaslt_version(void);

/* Buffer sizing, identical to csrc/thor_fp4_core.cu:535-550. */
int64_t tfp4_pad_rows(int64_t R);
int64_t tfp4_packed_bytes(int64_t R, int64_t K);
int64_t tfp4_scale_bytes(int64_t R, int64_t K);
int64_t tfp4_mx_packed_bytes(int64_t R, int64_t K, int kind);
int64_t tfp4_mx_scale_bytes(int64_t R, int64_t K);

/* Replaces tfp4_quant (csrc/thor_fp4_core.cu:555-578): row-major (R,K) -> e2m1 codes
 * + UE4M3 scale bytes in the 128x4 tile layout, bit-exact with the reference.  One
 * fused kernel, no scratch.  Rows R..pad(R) of both outputs are written as zeros.
 * x must be 16-byte aligned (32 for f32). */
int tfp4_quant(const void* x, int64_t R, int64_t K, int in_dtype, float ts,
               uint8_t* packed, uint8_t* sblk, void* stream);

/* Replaces tfp4_quant_mx (csrc/thor_fp4_core.cu:581-602): kind 0 = MXFP4 (e2m1),
 * kind 1 = MXFP8 (e4m3); UE8M0 scale per 32. */
int tfp4_quant_mx(const void* x, int64_t R, int64_t K, int in_dtype, int kind,
                  uint8_t* packed, uint8_t* sblk, void* stream);

/* Replaces tfp4_mx8_mul (csrc/thor_fp4_core.cu:657-675): h = a*b on MXFP8 tensors,
 * ceil-power-of-two scales; K % 128 == 0. */
int tfp4_mx8_mul(const void* ap, const void* as, const void* bp, const void* bs,
                 void* op, void* os, int64_t R, int64_t K, void* stream);

/* Replaces tfp4_gemm (csrc/thor_fp4_core.cu:697-757): out (M,N) row-major =
 * (tsA*tsB) * A(M,K) @ B(N,K)^T on NVFP4 buffers, FP32 accumulation in tensor
 * memory, computed as (B @ A^T) with no transpose.  M >= 1, N >= 8, N % 8 == 0,
 * K % 64 == 0.  Code buffers 32-byte, scale buffers 16-byte aligned. */
int tfp4_gemm(const void* packedA, const void* sblkA, float tsA,
              const void* packedB, const void* sblkB, float tsB,
              void* out, int64_t M, int64_t N, int64_t K, int out_dtype, void* stream);

/* Addition over the reference ABI: the same GEMM with the bias add and the cast
 * fused into the epilogue, out = cast(alpha*acc + bias[n]) with one rounding
 * (the reference adds the bias afterwards in the output dtype,
 * src/thor_fp4/linear.py:264-265).  bias: N floats or NULL. */
int tfp4_gemm_bias(const void* packedA, const void* sblkA, float tsA,
                   const void* packedB, const void* sblkB, float tsB,
                   const float* bias, void* out, int64_t M, int64_t N, int64_t K,
                   int out_dtype, void* stream);

/* The two calls one forward pass of the reference's Linear makes (src/thor_fp4/linear.py:240-262: tfp4_quant of the
 * activation into the layer's cached buffers, then tfp4_gemm, then the bias add) as one entry point, for hosts
 * where the per-call cost of the foreign-function boundary matters (small batches are launch-bound).  Same
 * arguments and error codes as the two calls. */
int tfp4_linear(const void* x, int64_t M, int64_t K, int in_dtype, float act_ts,
                uint8_t* act_packed, uint8_t* act_sblk,
                const void* w_packed, const void* w_sblk, float w_ts,
                const float* bias, void* out, int64_t N, int out_dtype, void* stream);

/* Replaces the work between the two GEMMs of the reference's gated MLP (src/thor_fp4/fused.py:163-173:
 * activation, elementwise product, re-quantization of the hidden tensor; csrc K14 mx8_mul for the MX form)
 * for the NVFP4 block: gu is the [R, 2*I] f16/bf16 output of the stacked gate/up GEMM (I gate values,
 * then I up values per row); writes the NVFP4 codes and scale tiles of h = silu(gate) * up (FP32 math,
 * h rounded to the input type, per-tensor scale 1) exactly as tfp4_quant would from h.  in_dtype 1 f16, 2 bf16.
 * The unfused form of tfp4_swiglu_gemm below (stacked halves instead of alternating blocks; gate, up and h each
 * rounded to the 16-bit type). */
int tfp4_swiglu_quant(const void* gu, int64_t R, int64_t I, int in_dtype,
                      uint8_t* packed, uint8_t* sblk, void* stream);

/* Replaces the epilogue work of the reference's fused MX layers (csrc/fused_kernels.cu:74-123, src/thor_fp4/fused.py:81-135:
 * bias[n], activation, MXFP8 re-quantization of the layer output) as one pass over the f16/bf16 GEMM output acc [R, N]:
 * writes the e4m3 codes and UE8M0 scale tiles of act(acc + bias), block scale = the power of two at or above
 * amax * (1/448) (the reference's fused-epilogue and mx8_mul recipe: nothing saturates; tfp4_quant_mx rounds the scale
 * to the nearest power of two instead).  in_dtype 0 f32, 1 f16, 2 bf16; act: 0 identity, 1 gelu (erf form), 2 silu;
 * bias may be null; N % 32 == 0. */
int tfp4_act_quant_mx8(const void* acc, const float* bias, int64_t R, int64_t N, int in_dtype, int act,
                       uint8_t* packed, uint8_t* sblk, void* stream);

/* Replaces the forward pass of the reference's quantization-aware-training fake quantizer (src/thor_fp4/quant.py:32-53,
 * a chain of torch kernels over FP32 temporaries) as one pass: y = dequantize(quantize(x)) over n elements taken as
 * consecutive 16-element blocks, with the scale bytes and codes tfp4_quant would produce (ties up, IEEE division,
 * blocks whose scale byte is 0 give zeros); no codes or scales are stored.  n % 16 == 0; in_dtype 0 f32, 1 f16,
 * 2 bf16; out_dtype 0 f16, 1 bf16, 2 f32 (the reference returns f32; a 16-bit output is that value rounded once). */
int tfp4_fake_quant(const void* x, int64_t n, int in_dtype, float tensor_scale, void* y, int out_dtype, void* stream);

/* No counterpart in the reference.  tfp4_gemm_bias for callers that must not allocate at call time
 * (device memory fully pre-partitioned at start-up, a plug-in under a foreign allocator, a loop
 * that cannot afford the device-wide synchronisation of an allocation or a free): the kernel's scratch - status word, counters, split-K partial sums - sits in a
 * fixed 16 MiB array of device memory that every GPU loading the library holds until exit, so no
 * cudaMalloc / cudaFree / cudaHostAlloc is ever called.  The first call on a device looks up the
 * array's address: make it before any stream capture.  A shape whose partial sums exceed
 * tfp4_gemm_noalloc_capacity() bytes is refused with -7 and a message.  Calls share the array, so calls
 * that overlap on the GPU (different streams) race; the status word is sticky: read / reset it with
 * tfp4_gemm_noalloc_status (blocking copy, not for hot paths). */
int tfp4_gemm_noalloc(const void* packedA, const void* sblkA, float tsA,
                      const void* packedB, const void* sblkB, float tsB,
                      const float* bias, void* out, int64_t M, int64_t N, int64_t K,
                      int out_dtype, void* stream);
int tfp4_gemm_noalloc_status(int reset);
size_t tfp4_gemm_noalloc_capacity(void);

/* Replaces tfp4_gemv (csrc/thor_fp4_core.cu:796-840): exact activations (M <= 8)
 * against NVFP4 weights, FP32 accumulation; sgemvB from tfp4_scales_gemv. */
int tfp4_gemv(const void* x, int64_t M, int64_t K, int in_dtype,
              const uint8_t* packedB, const uint8_t* sgemvB, float tsB,
              void* out, int64_t N, int out_dtype, void* stream);

/* Replaces tfp4_scales_gemv (csrc/thor_fp4_core.cu:782-790). */
int tfp4_scales_gemv(const uint8_t* sblk, int64_t R, int64_t K, uint8_t* out, void* stream);

/* Replaces tfp4_dequant_f32 (csrc/thor_fp4_core.cu:761-768). */
int tfp4_dequant_f32(const uint8_t* packed, const uint8_t* sblk, float ts,
                     int64_t R, int64_t K, float* out, void* stream);

/* Replaces tfp4_scales_f32 (csrc/thor_fp4_core.cu:771-778). */
int tfp4_scales_f32(const uint8_t* sblk, int64_t R, int64_t K, float* out, void* stream);

/* Replaces the optional second library's registry (csrc/cutlass_kernels.cu:229-263):
 * the same variant names resolve to the one tcgen05 kernel of this library (the
 * tile numbers in a name only pick the token-tile width).  tfc4_gemm: D (M,N) bf16 =
 * alpha * A @ B^T; "nvfp4_*" variants take NVFP4 operands, "mxfp8xfp4_*" variants
 * MXFP8 activations (A) and MXFP4 weights (B), K % 128 == 0. */
int tfc4_n_variants(void);
const char* tfc4_variant_name(int i);
int tfc4_variant_index(const char* name);
int tfc4_gemm(int variant, const void* A, const void* SA, const void* B, const void* SB,
              void* D, int64_t M, int64_t N, int64_t K, float alpha, void* stream);

/* Addition over tfc4_gemm: the same variants with bias[n] (N floats or NULL) fused into the epilogue and any output type
 * (0 f16, 1 bf16, 2 f32) - the MXFP8 x MXFP4 path with its FP32 accumulator observable, which the parity tests of the
 * fused epilogues below start from. */
int tfc4_gemm_ex(int variant, const void* A, const void* SA, const void* B, const void* SB, const float* bias,
                 void* D, int64_t M, int64_t N, int64_t K, float alpha, int out_dtype, void* stream);

/* Replaces the fused-epilogue library of the reference (csrc/fused_kernels.cu:379-447, bound at src/thor_fp4/_ext.py:82-94):
 * MXFP8 activations A (M,K) x MXFP4 weights B (N,K) with the inter-layer work in the GEMM's epilogue -
 * D = e4m3 codes (M*N bytes, row-major) and SFD = UE8M0 scale tiles (tfc4f_sfd_bytes, the 128x4 layout) of
 * act(alpha * A @ B^T + bias[n]); the variant name picks the activation (gelu | silu | ident; its tile numbers pick
 * nothing here), the block scale is the power of two at or above amax / 448 (csrc/fused_kernels.cu:74-123).  Same
 * argument checks and codes as the reference: -1 bad variant, -3 K % 128, -4 N % 32, -5 null bias.  gelu and silu are
 * computed from correctly rounded FP32 operations only, so the bytes are reproducible on a CPU. */
int tfc4f_n_variants(void);
const char* tfc4f_variant_name(int i);
int tfc4f_variant_index(const char* name);
int64_t tfc4f_sfd_bytes(int64_t M, int64_t N);
int tfc4f_gemm(int variant, const void* A, const void* SA, const void* B, const void* SB, const float* bias,
               void* D, void* SFD, int64_t M, int64_t N, int64_t K, float alpha, void* stream);

/* The NVFP4 counterpart of that fused layer for the SwiGLU block (the reference's gated block is the MXFP8 chain of
 * src/thor_fp4/fused.py:199-232: two fused GEMMs, tfp4_mx8_mul, a third GEMM): ONE gate/up GEMM whose epilogue computes
 * h = silu(alpha * x Wg^T) * (alpha * x Wu^T) in FP32 and quantizes it to NVFP4 (the arithmetic of tfp4_quant with
 * per-tensor scale 1), alpha = tsA * tsW.  packedW / sblkW: the stacked weight (N = 2 * intermediate rows, K) whose rows
 * alternate in blocks of 16 - gate rows j..j+15, then up rows j..j+15.  h_packed / h_sblk: codes (pad128(M),
 * intermediate / 2) and scale tiles of h, ready as the A operand of the down projection; rows M..pad128(M) are written
 * as zeros.  N % 128 == 0, K % 64 == 0.  No (M, 2 * intermediate) tensor is written to memory. */
int tfp4_swiglu_gemm(const void* packedA, const void* sblkA, float tsA, const void* packedW, const void* sblkW, float tsW,
                     void* h_packed, void* h_sblk, int64_t M, int64_t N, int64_t K, void* stream);

/* No counterpart in the reference (it is single-GPU): the exchange of a tensor-parallel block whose last layer is
 * row-parallel, with the transfer inside the GEMM.
 * tfp4_gemm_push: tfp4_gemm whose epilogue stores this rank's partial product (M, N), 32 token rows at a time, into the
 *   staging buffer of the rank that owns those rows: dest[o] (host array of n_dest <= 8 device pointers) = where this
 *   rank's rows for owner o go, a row-major (rows_per_dest, N) matrix of out_dtype (0 f16, 1 bf16 or 2 f32) in owner o's memory,
 *   mapped into this process (tfp4_peer_open; dest[own rank] is local memory).  Owner o holds token rows
 *   [o * rows_per_dest, (o + 1) * rows_per_dest); rows_per_dest % 32 == 0.  The stores are TMA stores issued by the
 *   epilogue warps while the tensor cores work on the next tile, so the NVLink transfer overlaps the GEMM.  first_dest:
 *   the owner whose token tiles this rank computes first (pass own rank + 1): every rank then walks the owners in a
 *   different rotation and no owner's links take every rank's stores at once.
 * tfp4_sum_slots: out (rows, N) = sum over the n staged partials stage[s] (s ascending: the same order on every rank),
 *   in_dtype 0 f32 / 1 f16 / 2 bf16, out_dtype 0 f16 / 1 bf16 / 2 f32.  16-bit partials halve the NVLink bytes: f16 rounds
 *   each partial at 2^-12 relative (an 8-rank sum stays within 1e-3 of the f32 exchange, but a partial beyond 65504
 *   overflows), bf16 at 2^-9 (about 2e-3 after the sum).  Run it after every rank's push has completed (a barrier
 *   on the host or a collective in stream order between the two calls).
 * tfp4_peer_alloc / _open / _close / _free: a device buffer with a 64-byte CUDA IPC handle that the other processes of
 *   the node open to obtain a pointer valid on their device.
 * tfp4_peer_copy: one device-to-device copy in stream order (cudaMemcpyAsync); towards a mapped peer buffer it goes over
 *   NVLink through the copy engines and uses no SM - the transfer of the "copy" exchange, which runs beside the next
 *   token chunk's GEMMs. */
int tfp4_gemm_push(const void* packedA, const void* sblkA, float tsA, const void* packedB, const void* sblkB, float tsB,
                   void* const* dest, int n_dest, int64_t rows_per_dest, int first_dest, int64_t M, int64_t N, int64_t K,
                   int out_dtype, void* stream);
int tfp4_sum_slots(const void* stage, int n, int64_t rows, int64_t N, int in_dtype, void* out, int out_dtype, void* stream);
int tfp4_peer_alloc(size_t bytes, void** ptr, unsigned char* handle64);
int tfp4_peer_open(const unsigned char* handle64, void** ptr);
int tfp4_peer_close(void* ptr);
int tfp4_peer_copy(void* dst, const void* src, size_t bytes, void* stream);
int tfp4_peer_free(void* ptr);

/* Additions: status word of the current device (0 = healthy; otherwise the role
 * whose bounded wait expired: 1 producer, 2 accumulator hand-back, 3 operands,
 * 4 epilogue), its reset, plan-cache counters, and a test hook that pins the
 * token-tile width (0 = automatic; 32, 64, 128 or 256). */
int tfp4_status(void);
void tfp4_clear_status(void);
void tfp4_plan_stats(uint64_t* hits, uint64_t* misses);
void tfp4_set_token_tile(int bn);

/* Further test / profiling hooks (no counterpart in the reference): pair_mode -1 (default) = the two-CTA
 * (cta_group::2) kernel for batches above 128 tokens with enough tiles, 0 = single-CTA kernel only, 1 or 2 = the
 * two-CTA kernel whenever the shape allows it; debug bits switch off parts of the GEMM kernel
 * for ablation timing (bit0 stores, bit1 scale copies, bit2 MMAs, bit3 loads, bit4 tensor-memory
 * reads, bit5 the MMA issuer's look-ahead polls; bit6 makes the two-CTA kernel's epilogue hold the accumulator about
 * 40k cycles per tile, so that every tile starts from a stalled, full pipeline - results must not change; bit 512
 * starves the consumers so that the bounded waits give up; bit 1024 records per-CTA cycle counters read back with
 * tfp4_debug_stats: 4 values per CTA). */
void tfp4_set_pair_mode(int mode);
/* No counterpart in the reference.  1 (default): the GEMM kernels and the split-K reduction are launched with
 * programmatic stream serialization, so their prologue overlaps the tail of the kernel before them in the stream
 * (normally the activation quantizer) and they wait for its completion before touching global memory; 0: plain
 * stream order (A/B timing). */
void tfp4_set_dependent_launch(int on);
/* K split of small-batch GEMMs: 0 automatic (tiles that fill whole waves of CTAs stay whole, the rest are cut),
 * -1 automatic with every tile cut alike, 1 never, n = about n K ranges for every tile (test hook). */
void tfp4_set_splits(int n);
void tfp4_set_debug(int bits);
/* tile order of the two-CTA kernel: 0 = automatic (bands of token tiles sized to stay resident in L2 while the weights
 * stream, once the activation no longer fits), -1 = token tiles fastest, gm > 0 = bands of gm token tiles with the
 * feature tiles fastest inside a band (A/B timing) */
void tfp4_set_raster(int gm);
/* test hook: force the NVFP4 quantizer's tile height (64 or 128 rows; 0 = automatic) */
void tfp4_set_quant_tile_rows(int rows);
int tfp4_debug_stats(unsigned long long* out, int n_ctas);

#ifdef __cplusplus
}
#endif
#endif
