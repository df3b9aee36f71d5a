// quant.cu -- fused activation / weight quantizers for sm_100a.
//
// One kernel per call (the reference runs two and round-trips the scales through
// an f32 scratch array, csrc/thor_fp4_core.cu:127-217,555-578): each CTA owns a
// 128-row x 256-column tile, i.e. whole 512-byte scale atoms, reads its input
// with 128-bit loads, reduces the per-block amax with warp shuffles, writes the
// e2m1 codes straight to their row-major place and stages the scale bytes in
// shared memory so that every atom leaves as one contiguous 512-byte store.
// Rows past R inside the last 128-row tile are written as zeros.
//
// Bit-exactness with the reference arithmetic
//   sc = ue4m3(amax * (1/6) / ts), ds = dec(sc) * ts, code = e2m1_ties_up(x / ds)
// is kept without an IEEE division per element:
//
//   EXACT16 path (16-bit input, ts == 1).  ds is an e4m3 value (<= 4 significant
//   bits) and the rounding thresholds t are {.25,.75,1.25,1.75,2.5,3.5,5}
//   (<= 3 bits), so t*ds is exactly representable in bf16, f16 and f32.  For an
//   f32 quotient q = RN(x/ds):  q >= t  <=>  x >= t*ds, because no f32 lies in
//   [t*ds*(1-2^-25), t*ds).  With x and t*ds both numbers of the 16-bit input
//   format, x < t*ds implies x <= t*ds*(1-2^-11).  Hence y = x * rb with
//   rb = RN(1/ds)*(1+2^-21) satisfies y > t when x >= t*ds and y < t otherwise
//   (the bias 2^-21 dominates the three roundings, 3*2^-24, and is far below the
//   2^-11 gap), so the hardware round-to-nearest-EVEN conversion of y returns the
//   reference's ties-UP code: y never sits on a midpoint.  y = fma(x, rb, +0)
//   turns -0 into +0 (the reference's sign is (q < 0)); 0*inf = NaN and +-inf map
//   to magnitude 6 exactly as the reference's x/0 does; NaN -> +6.
//
//   BRACKET path (f32 input, or ts != 1).  y_lo = x*r*(1-2^-20) and
//   y_hi = x*r*(1+2^-20) strictly bracket RN(x/ds).  If both convert to the same
//   code no rounding midpoint lies between them and that code is the reference's;
//   otherwise (probability ~1e-5 per element) the lane recomputes its 8 codes with
//   the literal IEEE division and compare chain.  Lanes holding a non-zero
//   |x| < 2^-100 (the quotient may underflow to -0, whose sign the reference
//   drops) and calls with an out-of-range ts also take the literal route.
#include "common.cuh"
#include "det_math.cuh"
#include "quant_block.cuh"

namespace tfp4 {

namespace {

template <bool B> struct BoolTag { static constexpr bool value = B; };

constexpr int QT_ROWS = 128;   // rows per CTA tile = one scale-atom height
constexpr int QT_COLS = 256;   // columns per CTA tile = 16 elements x 16 lanes (NVFP4 quantizer), 8 x 32 (MX kernels)
constexpr int QT_THREADS = 256;
constexpr int QT_UNROLL = 4;   // rows in flight per warp

// 16 consecutive elements of one row = one quantization block, held by ONE lane: raw bits as loaded
// (two 16-byte loads for 16-bit inputs, four for f32) and their widening to float.
template <typename T> struct Raw16 { uint4 v[sizeof(T) == 2 ? 2 : 4]; };

template <typename T>
__device__ __forceinline__ Raw16<T> fetch16(const T* p) {
    Raw16<T> r;
#pragma unroll
    for (int i = 0; i < (int)(sizeof(T) == 2 ? 2 : 4); ++i) r.v[i] = __ldg(reinterpret_cast<const uint4*>(p) + i);
    return r;
}
template <typename T>
__device__ __forceinline__ Raw16<T> zero16() {
    Raw16<T> r;
#pragma unroll
    for (int i = 0; i < (int)(sizeof(T) == 2 ? 2 : 4); ++i) r.v[i] = make_uint4(0u, 0u, 0u, 0u);
    return r;
}
__device__ __forceinline__ void widen16(const Raw16<float>& r, float (&lo)[8], float (&hi)[8]) {
    const uint4 q[4] = {r.v[0], r.v[1], r.v[2], r.v[3]};
    lo[0] = __uint_as_float(q[0].x); lo[1] = __uint_as_float(q[0].y); lo[2] = __uint_as_float(q[0].z); lo[3] = __uint_as_float(q[0].w);
    lo[4] = __uint_as_float(q[1].x); lo[5] = __uint_as_float(q[1].y); lo[6] = __uint_as_float(q[1].z); lo[7] = __uint_as_float(q[1].w);
    hi[0] = __uint_as_float(q[2].x); hi[1] = __uint_as_float(q[2].y); hi[2] = __uint_as_float(q[2].z); hi[3] = __uint_as_float(q[2].w);
    hi[4] = __uint_as_float(q[3].x); hi[5] = __uint_as_float(q[3].y); hi[6] = __uint_as_float(q[3].z); hi[7] = __uint_as_float(q[3].w);
}
template <typename T>
__device__ __forceinline__ void widen16(const Raw16<T>& r, float (&lo)[8], float (&hi)[8]) {
    Raw8<T> a, b;
    a.a = r.v[0];
    b.a = r.v[1];
    widen8(a, lo);
    widen8(b, hi);
}

// The scale byte of a 16-element block held by one lane (f = its two halves) and the decode scale ds = dec(sc) * ts.
// Same arithmetic as block_scale8 (quant_block.cuh) without the shuffle between the two lanes of a pair.
template <int MODE>
__device__ __forceinline__ float block_scale16(const float (&lo)[8], const float (&hi)[8], float ts, float rts_lo, float rts_hi,
                                               uint32_t& sc) {
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fmaxf(fabsf(lo[i]), fabsf(hi[i])));
    float pre = amax * (1.0f / 6.0f);
    if (MODE == 1 || MODE == 3) {
        const uint32_t both = f32x2_to_e4m3x2(pre * rts_lo, pre * rts_hi);
        sc = both & 0x7fu;
        if (sc != ((both >> 8) & 0x7fu)) sc = f32x2_to_e4m3x2(__fdiv_rn(pre, ts), 0.f) & 0x7fu;
    } else {
        if (MODE != 0) pre = __fdiv_rn(pre, ts);   // (amax * (1/6)) / ts, the reference's operand order
        sc = f32x2_to_e4m3x2(pre, 0.f) & 0x7fu;
    }
    const float sf = e4m3_to_f32(sc);
    return (MODE != 0) ? sf * ts : sf;
}

// MODE 0: EXACT16 (16-bit input, ts == 1); 1: BRACKET; 2: LITERAL (always divide);
// 3: BRACKET without the tiny-input check (16-bit input and ts <= 128: the smallest non-zero
// input, 2^-133, divided by the largest ds, 448 * 128, stays far above the 2^-150 underflow bound).
// ROWS: rows per CTA, 128 (whole scale atoms) or 64 (half atoms; finer tiles for small grids).
// GATED: x is the output [R, 2K] of the stacked gate/up GEMM (row = K gate values, then K up values);
// the quantized tensor is h = round_to_T(silu(gate) * up), computed in FP32, held in T like the
// unfused block holds it, and quantized with the same code path (one pass instead of an elementwise
// kernel with FP32 temporaries followed by the quantizer).
//
// Work split.  A lane owns one whole 16-element block (32 contiguous bytes of a 16-bit row): the block's amax,
// scale byte and multiplier are computed once, by the lane that needs them, with no exchange between lanes.
// A half-warp covers the tile's 256 columns of one row (512 contiguous bytes), so a warp works on two rows at a
// time: warp w, half h handles tile rows 16 * it + 2 * w + h.  Codes leave as 8 bytes per lane (128 contiguous
// bytes per half-warp); scale bytes are staged in shared memory and leave as whole 512-byte atoms.
template <typename T, int MODE, int ROWS, bool GATED = false>
__global__ void __launch_bounds__(QT_THREADS, sizeof(T) == 2 ? 4 : 3)
quant_nvfp4_kernel(const T* __restrict__ x, int64_t R, int64_t K, float ts,
                   uint8_t* __restrict__ packed, uint8_t* __restrict__ sblk, int64_t tiles_x, int64_t n_tiles) {
    __shared__ __align__(16) uint8_t s_sf[4 * 512];
    // Programmatic dependent launch on both sides: this grid may have been made resident while the kernel
    // before it (the GEMM producing x, or the GEMM still reading the previous contents of packed / sblk) was
    // finishing, so it waits for that kernel here; and the GEMM that consumes this tensor may set itself up
    // while the tail of this grid runs.
    griddep_wait();
    griddep_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = lane >> 4, l16 = lane & 15;
    constexpr int STEPS = ROWS / 16;                   // 16 rows per step and CTA (8 warps x 2 half-warps)
    // steps (= rows per lane) per buffer set; two sets alternate.  The variants with more arithmetic per block keep one
    // row per set: with two they spill
    constexpr int UNROLL = (MODE == 0 && !GATED) ? 2 : 1;
    const int64_t ld = GATED ? 2 * K : K;              // input row stride in elements
    const int64_t Rpad = pad128(R);

    // reciprocals of the per-tensor scale biased by +-2^-20 (bracket modes only)
    const float rts = __frcp_rn(ts);
    const float rts_hi = rts * 1.00000095367431640625f, rts_lo = rts * 0.99999904632568359375f;

    // MODE 0: the multiplier of a block depends only on its scale byte (127 values): RN(1 / dec(sc)) * (1 + 2^-21),
    // computed once per CTA with the arithmetic the per-row code used, then one shared-memory read per block
    __shared__ float s_rb[128];
    if (MODE == 0 && threadIdx.x < 128)
        s_rb[threadIdx.x] = __frcp_rn(e4m3_to_f32(threadIdx.x)) * 1.000000476837158203125f;

    constexpr int NSRC = GATED ? 2 : 1;
    // Persistent over tiles: the grid is sized to the CTAs that are resident at once and every CTA walks the tiles
    // tile = blockIdx.x, + gridDim.x, ...  With whole-wave launches a tile count such as 2048 on 592 resident CTAs
    // runs 4 waves for 3.46 waves of work; here the CTAs differ by at most one (finer, 64-row) tile.
#pragma unroll 1
    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int64_t ty = tile / tiles_x;
    const int64_t r0 = ty * ROWS;
    const int ra = (ROWS == 128) ? 0 : (int)(r0 & 127);   // first row of this tile inside its scale atom
    const int64_t c0 = (tile - ty * tiles_x) * QT_COLS;
    const int64_t col = c0 + l16 * 16;
    const bool col_ok = col < K;
    reinterpret_cast<uint2*>(s_sf)[threadIdx.x] = make_uint2(0u, 0u);
    __syncthreads();      // staging cleared (and, first time round, the multiplier table written)

    // the tile loop, instantiated twice: tiles wholly inside the tensor (no row or column checks) and edge tiles
    auto run_tile = [&](auto full_tag) {
        constexpr bool FULL = decltype(full_tag)::value;
        auto fetch_rows = [&](int it, Raw16<T> (&dst)[NSRC][UNROLL]) {
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int64_t r = r0 + 16 * (it + u) + 2 * warp + half;
#pragma unroll
                for (int g = 0; g < NSRC; ++g)
                    dst[g][u] = (FULL || (col_ok && r < R)) ? fetch16<T>(x + r * ld + g * K + col) : zero16<T>();
            }
        };
        auto process = [&](int it, Raw16<T> (&cur)[NSRC][UNROLL]) {
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                float lo[8], hi[8];
                widen16(cur[0][u], lo, hi);
                if constexpr (GATED) {
                    float ulo[8], uhi[8];
                    widen16(cur[NSRC - 1][u], ulo, uhi);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        // silu from correctly rounded operations only (det_math.cuh): the CPU oracle repeats them
                        // bit for bit, so the codes of h can be checked byte by byte; h is held in T
                        lo[i] = static_cast<float>(static_cast<T>(__fmul_rn(det_silu(lo[i]), ulo[i])));
                        hi[i] = static_cast<float>(static_cast<T>(__fmul_rn(det_silu(hi[i]), uhi[i])));
                    }
                }
                const int rl = 16 * (it + u) + 2 * warp + half;
                const int64_t r = r0 + rl;
                uint32_t c_lo = 0, c_hi = 0;
                if (FULL || r < R) {
                    uint32_t sc;
                    const float ds = block_scale16<MODE>(lo, hi, ts, rts_lo, rts_hi, sc);
                    if (FULL || col_ok)      // scale column l16 of the tile: atom l16 / 4, byte 16 * (row % 32) + 4 * (row / 32) + l16 % 4
                        s_sf[(l16 >> 2) * 512 + 16 * ((ra + rl) & 31) + 4 * ((ra + rl) >> 5) + (l16 & 3)] = (uint8_t)sc;
                    if constexpr (MODE == 0) {
                        const float rb = s_rb[sc];
                        float ya[8], yb[8];
#pragma unroll
                        for (int i = 0; i < 8; i += 2) {
                            mul2_pz(ya[i], ya[i + 1], lo[i], lo[i + 1], rb);
                            mul2_pz(yb[i], yb[i + 1], hi[i], hi[i + 1], rb);
                        }
                        c_lo = pack_codes_rne(ya);
                        c_hi = pack_codes_rne(yb);
                    } else {
                        c_lo = block_codes8<MODE>(lo, ds);
                        c_hi = block_codes8<MODE>(hi, ds);
                    }
                }
                if (FULL || (col_ok && r < Rpad))
                    *reinterpret_cast<uint2*>(packed + r * (K >> 1) + (col >> 1)) = make_uint2(c_lo, c_hi);
            }
        };
        // two sets of row buffers used alternately: the loads of one are in flight while the other is processed
        Raw16<T> buf_a[NSRC][UNROLL], buf_b[NSRC][UNROLL];
        fetch_rows(0, buf_a);
#pragma unroll 1
        for (int it = 0; it < STEPS; it += 2 * UNROLL) {
            if (it + UNROLL < STEPS) fetch_rows(it + UNROLL, buf_b);
            process(it, buf_a);
            if (it + 2 * UNROLL < STEPS) fetch_rows(it + 2 * UNROLL, buf_a);
            if (it + UNROLL < STEPS) process(it + UNROLL, buf_b);
        }
    };
    if (r0 + ROWS <= R && c0 + QT_COLS <= K) run_tile(BoolTag<true>{});
    else run_tile(BoolTag<false>{});
    __syncthreads();
    // scale bytes out: whole 512-byte atoms (ROWS == 128) or this CTA's half of each atom
    const int64_t D = K >> 6;                          // atoms per 128-row tile
    const int64_t d0 = c0 >> 6;
    const int n_atoms = (int)((K - c0 >= QT_COLS) ? 4 : ((K - c0) >> 6));
    uint8_t* dst = sblk + ((r0 >> 7) * D + d0) * 512;
    if (ROWS == 128) {
        const int atom = threadIdx.x >> 6;             // 64 threads x 8 bytes per atom
        if (atom < n_atoms)
            *reinterpret_cast<uint2*>(dst + threadIdx.x * 8) = reinterpret_cast<const uint2*>(s_sf)[threadIdx.x];
    } else if (threadIdx.x < 128) {
        // rows ra..ra+63 own bytes [8h, 8h+8) of every 16-byte lane row, h = ra / 64
        const int atom = threadIdx.x >> 5, off = atom * 512 + 16 * (threadIdx.x & 31) + (ra >> 3);
        if (atom < n_atoms)
            *reinterpret_cast<uint2*>(dst + off) = *reinterpret_cast<const uint2*>(s_sf + off);
    }
    __syncthreads();      // the staging bytes have been read before the next tile clears them
    }
}

// ---------------------------------------------------------------------------
// Fake quantizer (the forward pass of quantization-aware training): y = dequantize(quantize(x)) in
// one pass, no codes or scales stored.  Follows src/thor_fp4/quant.py:32-53: the value is
// code * sign * (dec(sc) * ts) with the same scale byte and codes as the quantizer above, and a
// block whose scale byte is 0 gives zeros.  The tensor is flat: consecutive 16-element blocks,
// a lane holds 8 elements, lane pairs share a block.
// ---------------------------------------------------------------------------
constexpr int FQ_THREADS = 256;
constexpr int FQ_UNROLL = 4;   // chunks of 8 elements in flight per thread

template <typename T, typename TO, int MODE>
__global__ void __launch_bounds__(FQ_THREADS)
fake_quant_nvfp4_kernel(const T* __restrict__ x, int64_t n_chunks, float ts, TO* __restrict__ y) {
    const float rts = __frcp_rn(ts);
    const float rts_hi = rts * 1.00000095367431640625f, rts_lo = rts * 0.99999904632568359375f;
    const int64_t per_cta = (int64_t)FQ_THREADS * FQ_UNROLL;
    // n_chunks is even and a CTA's first chunk is even, so a lane and its partner (lane ^ 1) are inside
    // or outside together; chunks past the end are processed as zeros (every lane takes the shuffle)
    for (int64_t base = (int64_t)blockIdx.x * per_cta; base < n_chunks; base += (int64_t)gridDim.x * per_cta) {
        Raw8<T> raw[FQ_UNROLL];
#pragma unroll
        for (int u = 0; u < FQ_UNROLL; ++u) {
            const int64_t c = base + u * FQ_THREADS + threadIdx.x;
            raw[u] = c < n_chunks ? fetch8<T>(x + c * 8) : zero8<T>();
        }
#pragma unroll
        for (int u = 0; u < FQ_UNROLL; ++u) {
            const int64_t c = base + u * FQ_THREADS + threadIdx.x;
            float f[8];
            widen8(raw[u], f);
            uint32_t sc;
            const float ds = block_scale8<MODE>(f, ts, rts_lo, rts_hi, sc);
            const uint32_t codes = block_codes8<MODE>(f, ds);
            const float dz = sc != 0u ? ds : 0.f;     // scale byte 0: the block decodes to zeros
            float o[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                e2m1x2_to_f32x2((codes >> (8 * i)) & 0xffu, o[2 * i], o[2 * i + 1]);
                o[2 * i] *= dz;
                o[2 * i + 1] *= dz;
            }
            if (c < n_chunks) {
                if constexpr (sizeof(TO) == 4) {
                    float4* dst = reinterpret_cast<float4*>(y + c * 8);
                    dst[0] = make_float4(o[0], o[1], o[2], o[3]);
                    dst[1] = make_float4(o[4], o[5], o[6], o[7]);
                } else {
                    uint32_t w[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const TO a = cast_out<TO>(o[2 * i]), b = cast_out<TO>(o[2 * i + 1]);
                        w[i] = (uint32_t)(*reinterpret_cast<const uint16_t*>(&a)) |
                               ((uint32_t)(*reinterpret_cast<const uint16_t*>(&b)) << 16);
                    }
                    *reinterpret_cast<uint4*>(y + c * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------
// MX quantizer: UE8M0 (power-of-two) scale per 32 elements; kind 0 = e2m1 codes
// (ties up, as the NVFP4 path), kind 1 = e4m3 codes (hardware RNE, saturating).
// Follows csrc/thor_fp4_core.cu:224-309.  Dividing by the power-of-two scale is
// done as an exact multiplication by its reciprocal (same correctly rounded
// result as the reference's x / ds, including sub-normal quotients).
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t ue8m0_nearest(float v) {
    // nearest power of two, midpoint ties up; !(v > 0) -> 0; csrc/thor_fp4_core.cu:105-113
    if (!(v > 0.f)) return 0u;
    const uint32_t u = __float_as_uint(v);
    if (u == 0x7f800000u) return 127u;   // the reference's frexpf(+inf) reports exponent 0 -> scale 1
    uint32_t b;
    if ((u >> 23) == 0u) b = (u >= 0x00600000u) ? 1u : 0u;   // sub-normal v
    else b = (u + 0x00400000u) >> 23;
    return b > 254u ? 254u : b;
}

__device__ __forceinline__ uint32_t ue8m0_ceil(float v);

// ACT >= 0: x is a GEMM output; the quantized tensor is act(x + bias[col]) (FP32 math; 0 identity, 1 gelu (erf form),
// 2 silu; both from the reproducible operations of det_math.cuh) - the bias add, activation and re-quantization between two layers of an MX chain in one pass.  Like the
// reference's fused epilogue and its mx8_mul, this form takes the block scale as the power of two at or above
// amax * (1/448), so that no value saturates (the plain quantizer rounds the scale to the nearest power of two).
template <typename T, int KIND, int ACT = -1>
__global__ void __launch_bounds__(QT_THREADS)
quant_mx_kernel(const T* __restrict__ x, int64_t R, int64_t K,
                uint8_t* __restrict__ packed, uint8_t* __restrict__ sblk, const float* __restrict__ bias = nullptr) {
    __shared__ __align__(16) uint8_t s_sf[2 * 512];
    griddep_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t r0 = (int64_t)blockIdx.y * QT_ROWS;
    const int64_t c0 = (int64_t)blockIdx.x * QT_COLS;
    const int64_t col = c0 + lane * 8;
    const bool col_ok = col < K;
    const int64_t Rpad = pad128(R);
    const int64_t S = K >> 5;
    const bool whole_atoms = (S & 3) == 0;   // K % 128 == 0

    if (threadIdx.x < 128) reinterpret_cast<uint2*>(s_sf)[threadIdx.x] = make_uint2(0u, 0u);
    __syncthreads();

#pragma unroll 1
    for (int it = 0; it < QT_ROWS / 8; it += QT_UNROLL) {
        float f[QT_UNROLL][8];
#pragma unroll
        for (int u = 0; u < QT_UNROLL; ++u) {
            const int64_t r = r0 + warp + 8 * (it + u);
            if (col_ok && r < R) {
                load8<T>(x + r * K + col, f[u]);
                if constexpr (ACT >= 0) {
                    float b[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                    if (bias != nullptr) {
                        const float4 b0 = __ldg(reinterpret_cast<const float4*>(bias + col));
                        const float4 b1 = __ldg(reinterpret_cast<const float4*>(bias + col + 4));
                        b[0] = b0.x; b[1] = b0.y; b[2] = b0.z; b[3] = b0.w; b[4] = b1.x; b[5] = b1.y; b[6] = b1.z; b[7] = b1.w;
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float v = __fadd_rn(f[u][i], b[i]);
                        if (ACT == 1) f[u][i] = det_gelu(v);          // reproducible forms (det_math.cuh), repeated
                        else if (ACT == 2) f[u][i] = det_silu(v);     // bit for bit by the CPU oracle
                        else f[u][i] = v;
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) f[u][i] = 0.f;
            }
        }
#pragma unroll
        for (int u = 0; u < QT_UNROLL; ++u) {
            const int rl = warp + 8 * (it + u);
            const int64_t r = r0 + rl;
            uint32_t w0 = 0, w1 = 0;
            if (r < R) {   // warp-uniform: every lane takes part in the shuffles
                float amax = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[u][i]));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
                const uint32_t scb = (ACT >= 0) ? ue8m0_ceil(__fmul_rn(amax, 1.0f / 448.0f))
                                                : ue8m0_nearest(__fdiv_rn(amax, KIND == 0 ? 6.0f : 448.0f));
                // 1/ds = 2^(127 - scb), exactly representable for scb in [0, 254]
                const int e = 127 - (int)scb;
                const float inv = e >= -126 ? __uint_as_float((uint32_t)(e + 127) << 23)
                                            : __uint_as_float(0x00400000u);   // 2^-127
                if ((lane & 3) == 0 && col_ok) {
                    const int sl = lane >> 2;   // 0..7
                    if (whole_atoms) {
                        s_sf[(sl >> 2) * 512 + 16 * (rl & 31) + 4 * (rl >> 5) + (sl & 3)] = (uint8_t)scb;
                    } else {
                        sblk[sf_index(r, (c0 >> 5) + sl, S)] = (uint8_t)scb;
                    }
                }
                if (KIND == 0) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) w0 |= e2m1_ties_up(f[u][i] * inv) << (4 * i);
                } else {
                    w0 = f32x4_to_e4m3x4(f[u][0] * inv, f[u][1] * inv, f[u][2] * inv, f[u][3] * inv);
                    w1 = f32x4_to_e4m3x4(f[u][4] * inv, f[u][5] * inv, f[u][6] * inv, f[u][7] * inv);
                }
            }
            if (col_ok && r < Rpad) {
                if (KIND == 0) *reinterpret_cast<uint32_t*>(packed + r * (K >> 1) + (col >> 1)) = w0;
                else *reinterpret_cast<uint2*>(packed + r * K + col) = make_uint2(w0, w1);
            }
        }
    }
    __syncthreads();
    if (whole_atoms) {
        const int64_t D = S >> 2;
        const int64_t d0 = c0 >> 7;
        const int n_atoms = (int)((K - c0 >= QT_COLS) ? 2 : ((K - c0) >> 7));
        const int atom = threadIdx.x >> 6;
        if (atom < n_atoms) {
            uint2 v = reinterpret_cast<const uint2*>(s_sf)[threadIdx.x];
            uint8_t* dst = sblk + ((int64_t)blockIdx.y * D + d0 + atom) * 512 + (threadIdx.x & 63) * 8;
            *reinterpret_cast<uint2*>(dst) = v;
        }
    }
}

// ---------------------------------------------------------------------------
// MXFP8 elementwise product with ceil-power-of-two scales
// (csrc/thor_fp4_core.cu:612-652): one lane = 8 elements, 4 lanes = one block.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t ue8m0_ceil(float v) {
    if (!(v > 0.f)) return 0u;
    const uint32_t u = __float_as_uint(v);
    uint32_t b;
    if ((u >> 23) == 0u) b = (u > 0x00400000u) ? 1u : 0u;   // sub-normal: ceil(log2 v) <= -126
    else b = (u >> 23) + ((u & 0x007fffffu) ? 1u : 0u);
    return b > 254u ? 254u : b;
}

__device__ __forceinline__ float pow2_from_ue8m0(uint32_t b) {   // 2^(b-127), b in [0,254]
    return b ? __uint_as_float(b << 23) : __uint_as_float(0x00400000u);
}

__global__ void __launch_bounds__(QT_THREADS)
mx8_mul_kernel(const uint8_t* __restrict__ ap, const uint8_t* __restrict__ as,
               const uint8_t* __restrict__ bp, const uint8_t* __restrict__ bs,
               uint8_t* __restrict__ op, uint8_t* __restrict__ os, int64_t R, int64_t K) {
    __shared__ __align__(16) uint8_t s_sf[2 * 512];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t r0 = (int64_t)blockIdx.y * QT_ROWS;
    const int64_t c0 = (int64_t)blockIdx.x * QT_COLS;
    const int64_t col = c0 + lane * 8;
    const bool col_ok = col < K;
    const int64_t S = K >> 5;
    if (threadIdx.x < 128) reinterpret_cast<uint2*>(s_sf)[threadIdx.x] = make_uint2(0u, 0u);
    __syncthreads();
#pragma unroll 1
    for (int it = 0; it < QT_ROWS / 8; ++it) {
        const int rl = warp + 8 * it;
        const int64_t r = r0 + rl;
        if (r >= R) continue;   // warp-uniform
        float fa = 1.f, fb = 1.f;
        uint2 av = make_uint2(0u, 0u), bv = make_uint2(0u, 0u);
        if (col_ok) {
            const int64_t si = sf_index(r, col >> 5, S);
            fa = pow2_from_ue8m0(as[si]);
            fb = pow2_from_ue8m0(bs[si]);
            av = __ldg(reinterpret_cast<const uint2*>(ap + r * K + col));
            bv = __ldg(reinterpret_cast<const uint2*>(bp + r * K + col));
        }
        const uint32_t aw[2] = {av.x, av.y}, bw[2] = {bv.x, bv.y};
        float f[8];
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float a = e4m3_to_f32((aw[i >> 2] >> (8 * (i & 3))) & 0xffu);
            const float b = e4m3_to_f32((bw[i >> 2] >> (8 * (i & 3))) & 0xffu);
            f[i] = __fmul_rn(__fmul_rn(__fmul_rn(a, fa), b), fb);
            amax = fmaxf(amax, fabsf(f[i]));
        }
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        const uint32_t scb = ue8m0_ceil(__fmul_rn(amax, 1.0f / 448.0f));
        const int e = 127 - (int)scb;
        const float inv = e >= -126 ? __uint_as_float((uint32_t)(e + 127) << 23)
                                    : __uint_as_float(0x00400000u);
        if ((lane & 3) == 0 && col_ok) {
            const int sl = lane >> 2;
            s_sf[(sl >> 2) * 512 + 16 * (rl & 31) + 4 * (rl >> 5) + (sl & 3)] = (uint8_t)scb;
        }
        const uint32_t w0 = f32x2_to_e4m3x2(f[0] * inv, f[1] * inv) | (f32x2_to_e4m3x2(f[2] * inv, f[3] * inv) << 16);
        const uint32_t w1 = f32x2_to_e4m3x2(f[4] * inv, f[5] * inv) | (f32x2_to_e4m3x2(f[6] * inv, f[7] * inv) << 16);
        if (col_ok) *reinterpret_cast<uint2*>(op + r * K + col) = make_uint2(w0, w1);
    }
    __syncthreads();
    const int64_t D = S >> 2;
    const int64_t d0 = c0 >> 7;
    const int n_atoms = (int)((K - c0 >= QT_COLS) ? 2 : ((K - c0) >> 7));
    const int atom = threadIdx.x >> 6;
    if (atom < n_atoms) {
        uint2 v = reinterpret_cast<const uint2*>(s_sf)[threadIdx.x];
        uint8_t* dst = os + ((int64_t)blockIdx.y * D + d0 + atom) * 512 + (threadIdx.x & 63) * 8;
        *reinterpret_cast<uint2*>(dst) = v;
    }
}

int g_quant_pdl = 1;   // 1: the NVFP4 quantizer is launched as a programmatic dependent of the kernel before it

// resident CTAs of the quantizer on the current device (4 per SM for 16-bit inputs, 3 for f32: the launch bounds)
int quant_slots(int elem_size) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return sms * (elem_size == 2 ? 4 : 3);
}

template <typename T, int ROWS>
int launch_quant_nvfp4_rows(const T* xp, int64_t R, int64_t K, float ts, uint8_t* packed, uint8_t* sblk,
                            cudaStream_t stream) {
    // the tiles cover the padded rows so that the rows past R of the last 128-row tile get their zeros
    const int64_t tiles_x = (K + QT_COLS - 1) / QT_COLS, n_tiles = tiles_x * (pad128(R) / ROWS);
    const int64_t slots = quant_slots((int)sizeof(T));
    const bool ts_sane = (ts >= 0x1p-100f) && (ts <= 0x1p30f);   // false for NaN too
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(n_tiles < slots ? n_tiles : slots));
    cfg.blockDim = dim3(QT_THREADS);
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = g_quant_pdl ? 1 : 0;
    if (!ts_sane) {
        TFP4_CK(cudaLaunchKernelEx(&cfg, quant_nvfp4_kernel<T, 2, ROWS>, xp, R, K, ts, packed, sblk, tiles_x, n_tiles));
    } else if (sizeof(T) == 2 && ts == 1.0f) {
        TFP4_CK(cudaLaunchKernelEx(&cfg, quant_nvfp4_kernel<T, 0, ROWS>, xp, R, K, ts, packed, sblk, tiles_x, n_tiles));
    } else if (sizeof(T) == 2 && ts <= 128.0f) {
        TFP4_CK(cudaLaunchKernelEx(&cfg, quant_nvfp4_kernel<T, 3, ROWS>, xp, R, K, ts, packed, sblk, tiles_x, n_tiles));
    } else {
        TFP4_CK(cudaLaunchKernelEx(&cfg, quant_nvfp4_kernel<T, 1, ROWS>, xp, R, K, ts, packed, sblk, tiles_x, n_tiles));
    }
    return TFP4_OK;
}

int g_quant_rows = 0;   // test hook: 64 / 128 forces the tile height, 0 = automatic

template <typename T>
int launch_quant_nvfp4(const void* x, int64_t R, int64_t K, float ts, uint8_t* packed,
                       uint8_t* sblk, cudaStream_t stream) {
    // 128-row tiles (whole scale atoms: 512-byte scale stores) when every resident CTA gets many of them; 64-row
    // tiles (half atoms) when the count per CTA is small, where one tile more or less per CTA is a visible share
    const int64_t tiles128 = ((K + QT_COLS - 1) / QT_COLS) * (pad128(R) / 128);
    const T* xp = static_cast<const T*>(x);
    if (g_quant_rows == 64) return launch_quant_nvfp4_rows<T, 64>(xp, R, K, ts, packed, sblk, stream);
    if (g_quant_rows == 128) return launch_quant_nvfp4_rows<T, 128>(xp, R, K, ts, packed, sblk, stream);
    const int64_t slots = quant_slots((int)sizeof(T));
    const int64_t rounds = (tiles128 + slots - 1) / slots;      // tiles of the busiest CTA
    // more than 4 % of the busiest CTA's time idle elsewhere (8192 x 8192: 2048 tiles on 592 CTAs = 4 rounds for 3.46)
    if (rounds * slots * 100 > tiles128 * 104) return launch_quant_nvfp4_rows<T, 64>(xp, R, K, ts, packed, sblk, stream);
    return launch_quant_nvfp4_rows<T, 128>(xp, R, K, ts, packed, sblk, stream);
}

template <typename T, typename TO>
int launch_fake_quant(const void* x, int64_t n, float ts, void* y, cudaStream_t stream) {
    const int64_t n_chunks = n / 8;
    const int64_t per_cta = (int64_t)FQ_THREADS * FQ_UNROLL;
    int64_t ctas = (n_chunks + per_cta - 1) / per_cta;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (ctas > (int64_t)sms * 16) ctas = (int64_t)sms * 16;   // grid-stride beyond 16 CTAs per SM
    const T* xp = static_cast<const T*>(x);
    TO* yp = static_cast<TO*>(y);
    const bool ts_sane = (ts >= 0x1p-100f) && (ts <= 0x1p30f);
    if (!ts_sane) {
        fake_quant_nvfp4_kernel<T, TO, 2><<<(unsigned)ctas, FQ_THREADS, 0, stream>>>(xp, n_chunks, ts, yp);
    } else if (sizeof(T) == 2 && ts == 1.0f) {
        fake_quant_nvfp4_kernel<T, TO, 0><<<(unsigned)ctas, FQ_THREADS, 0, stream>>>(xp, n_chunks, ts, yp);
    } else if (sizeof(T) == 2 && ts <= 128.0f) {
        fake_quant_nvfp4_kernel<T, TO, 3><<<(unsigned)ctas, FQ_THREADS, 0, stream>>>(xp, n_chunks, ts, yp);
    } else {
        fake_quant_nvfp4_kernel<T, TO, 1><<<(unsigned)ctas, FQ_THREADS, 0, stream>>>(xp, n_chunks, ts, yp);
    }
    TFP4_CK(cudaGetLastError());
    return TFP4_OK;
}

template <typename T>
int launch_fake_quant_in(const void* x, int64_t n, float ts, void* y, int out_dtype, cudaStream_t stream) {
    switch (out_dtype) {
        case OUT_F32: return launch_fake_quant<T, float>(x, n, ts, y, stream);
        case OUT_F16: return launch_fake_quant<T, __half>(x, n, ts, y, stream);
        default: return launch_fake_quant<T, __nv_bfloat16>(x, n, ts, y, stream);
    }
}

template <typename T>
int launch_quant_mx(const void* x, int64_t R, int64_t K, int kind, uint8_t* packed, uint8_t* sblk,
                    cudaStream_t stream) {
    dim3 grid((unsigned)((K + QT_COLS - 1) / QT_COLS), (unsigned)((R + QT_ROWS - 1) / QT_ROWS));
    const T* xp = static_cast<const T*>(x);
    if (kind == 0) quant_mx_kernel<T, 0><<<grid, QT_THREADS, 0, stream>>>(xp, R, K, packed, sblk);
    else quant_mx_kernel<T, 1><<<grid, QT_THREADS, 0, stream>>>(xp, R, K, packed, sblk);
    TFP4_CK(cudaGetLastError());
    return TFP4_OK;
}

bool misaligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) != 0; }

}  // namespace

// act(acc + bias) -> MXFP8 codes and UE8M0 (ceil) scale tiles in one pass; acc = [R, N] f32/f16/bf16, N % 32 == 0
int act_quant_mx8(const void* acc, const float* bias, int64_t R, int64_t N, int in_dtype, int act, uint8_t* packed,
                  uint8_t* sblk, cudaStream_t stream) {
    if (N <= 0 || (N % 32) != 0) {
        fprintf(stderr, "thor_fp4: tfp4_act_quant_mx8 needs N %% 32 == 0 (got %ld)\n", (long)N);
        return TFP4_ERR_BAD_K;
    }
    if (R <= 0) return TFP4_OK;
    if (!acc || !packed || !sblk || in_dtype < 0 || in_dtype > 2 || act < 0 || act > 2 || misaligned(acc, in_dtype == IN_F32 ? 32 : 16) ||
        misaligned(packed, 8) || misaligned(sblk, 8) || (bias && misaligned(bias, 16))) {
        fprintf(stderr, "thor_fp4: tfp4_act_quant_mx8 bad argument (act 0..2, input 16-byte (f32: 32-byte) and bias 16-byte aligned)\n");
        return TFP4_ERR_BAD_ARG;
    }
    dim3 grid((unsigned)((N + QT_COLS - 1) / QT_COLS), (unsigned)((R + QT_ROWS - 1) / QT_ROWS));
#define TFP4_AQ(TT, A) quant_mx_kernel<TT, 1, A><<<grid, QT_THREADS, 0, stream>>>(static_cast<const TT*>(acc), R, N, packed, sblk, bias)
    if (in_dtype == IN_BF16) {
        if (act == 0) TFP4_AQ(__nv_bfloat16, 0); else if (act == 1) TFP4_AQ(__nv_bfloat16, 1); else TFP4_AQ(__nv_bfloat16, 2);
    } else if (in_dtype == IN_F16) {
        if (act == 0) TFP4_AQ(__half, 0); else if (act == 1) TFP4_AQ(__half, 1); else TFP4_AQ(__half, 2);
    } else {
        if (act == 0) TFP4_AQ(float, 0); else if (act == 1) TFP4_AQ(float, 1); else TFP4_AQ(float, 2);
    }
#undef TFP4_AQ
    TFP4_CK(cudaGetLastError());
    return TFP4_OK;
}

void quant_set_tile_rows(int rows) { g_quant_rows = (rows == 64 || rows == 128) ? rows : 0; }

// h = silu(gate) * up from the stacked GEMM output gu [R, 2K] (16-bit), quantized to NVFP4 with
// per-tensor scale 1: codes [R, K/2] and scale tiles exactly as quant_nvfp4 would produce from h.
int swiglu_quant_nvfp4(const void* gu, int64_t R, int64_t K, int in_dtype, uint8_t* packed, uint8_t* sblk,
                       cudaStream_t stream) {
    if (K <= 0 || (K % 64) != 0) {
        fprintf(stderr, "thor_fp4: intermediate size must be a multiple of 64 (got %ld)\n", (long)K);
        return TFP4_ERR_BAD_K;
    }
    if (R <= 0) return TFP4_OK;
    if (!gu || !packed || !sblk || (in_dtype != IN_F16 && in_dtype != IN_BF16) || misaligned(gu, 16) ||
        misaligned(packed, 4) || misaligned(sblk, 8)) {
        fprintf(stderr, "thor_fp4: tfp4_swiglu_quant needs a 16-byte aligned f16/bf16 input, packed 4-byte, sblk 8-byte aligned\n");
        return TFP4_ERR_BAD_ARG;
    }
    const int64_t tiles_x = (K + QT_COLS - 1) / QT_COLS, n_tiles = tiles_x * (pad128(R) / 128);
    const int64_t slots = quant_slots(2);
    dim3 grid((unsigned)(n_tiles < slots ? n_tiles : slots));
    cudaLaunchAttribute attr[1];       // dependent of the gate/up GEMM before it (waits for it before its first load)
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(QT_THREADS);
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = g_quant_pdl ? 1 : 0;
    if (in_dtype == IN_BF16)
        TFP4_CK(cudaLaunchKernelEx(&cfg, quant_nvfp4_kernel<__nv_bfloat16, 0, 128, true>,
                                   static_cast<const __nv_bfloat16*>(gu), R, K, 1.0f, packed, sblk, tiles_x, n_tiles));
    else
        TFP4_CK(cudaLaunchKernelEx(&cfg, quant_nvfp4_kernel<__half, 0, 128, true>, static_cast<const __half*>(gu), R, K, 1.0f,
                                   packed, sblk, tiles_x, n_tiles));
    return TFP4_OK;
}

int quant_nvfp4(const void* x, int64_t R, int64_t K, int in_dtype, float ts, uint8_t* packed,
                uint8_t* sblk, cudaStream_t stream) {
    if (K <= 0 || (K % 64) != 0) {
        fprintf(stderr, "thor_fp4: K must be a multiple of 64 (got %ld)\n", (long)K);
        return TFP4_ERR_BAD_K;
    }
    if (R <= 0) return TFP4_OK;
    if (!x || !packed || !sblk || in_dtype < 0 || in_dtype > 2) {
        fprintf(stderr, "thor_fp4: tfp4_quant bad argument\n");
        return TFP4_ERR_BAD_ARG;
    }
    if (misaligned(x, in_dtype == IN_F32 ? 32 : 16) || misaligned(packed, 4) || misaligned(sblk, 8)) {
        fprintf(stderr, "thor_fp4: tfp4_quant needs x 16-byte (f32: 32-byte) aligned, packed 4, sblk 8\n");
        return TFP4_ERR_BAD_ARG;
    }
    switch (in_dtype) {
        case IN_F32: return launch_quant_nvfp4<float>(x, R, K, ts, packed, sblk, stream);
        case IN_F16: return launch_quant_nvfp4<__half>(x, R, K, ts, packed, sblk, stream);
        default: return launch_quant_nvfp4<__nv_bfloat16>(x, R, K, ts, packed, sblk, stream);
    }
}

void quant_set_pdl(int on) { g_quant_pdl = on ? 1 : 0; }

int fake_quant_nvfp4(const void* x, int64_t n, int in_dtype, float ts, void* y, int out_dtype, cudaStream_t stream) {
    if (n < 0 || (n % 16) != 0) {
        fprintf(stderr, "thor_fp4: tfp4_fake_quant needs a multiple of 16 elements (got %ld)\n", (long)n);
        return TFP4_ERR_BAD_K;
    }
    if (n == 0) return TFP4_OK;
    if (!x || !y || in_dtype < 0 || in_dtype > 2 || out_dtype < 0 || out_dtype > 2 ||
        misaligned(x, in_dtype == IN_F32 ? 32 : 16) || misaligned(y, out_dtype == OUT_F32 ? 32 : 16)) {
        fprintf(stderr, "thor_fp4: tfp4_fake_quant bad argument (buffers 16-byte, f32 ones 32-byte aligned)\n");
        return TFP4_ERR_BAD_ARG;
    }
    switch (in_dtype) {
        case IN_F32: return launch_fake_quant_in<float>(x, n, ts, y, out_dtype, stream);
        case IN_F16: return launch_fake_quant_in<__half>(x, n, ts, y, out_dtype, stream);
        default: return launch_fake_quant_in<__nv_bfloat16>(x, n, ts, y, out_dtype, stream);
    }
}

int quant_mx(const void* x, int64_t R, int64_t K, int in_dtype, int kind, uint8_t* packed,
             uint8_t* sblk, cudaStream_t stream) {
    if (K <= 0 || (K % 64) != 0) {
        fprintf(stderr, "thor_fp4: K must be a multiple of 64 (got %ld)\n", (long)K);
        return TFP4_ERR_BAD_K;
    }
    if (R <= 0) return TFP4_OK;
    if (!x || !packed || !sblk || in_dtype < 0 || in_dtype > 2 || kind < 0 || kind > 1) {
        fprintf(stderr, "thor_fp4: tfp4_quant_mx bad argument\n");
        return TFP4_ERR_BAD_ARG;
    }
    if (misaligned(x, in_dtype == IN_F32 ? 32 : 16) || misaligned(packed, 8) || misaligned(sblk, 8)) {
        fprintf(stderr, "thor_fp4: tfp4_quant_mx needs x 16-byte (f32: 32-byte) aligned, packed/sblk 8\n");
        return TFP4_ERR_BAD_ARG;
    }
    switch (in_dtype) {
        case IN_F32: return launch_quant_mx<float>(x, R, K, kind, packed, sblk, stream);
        case IN_F16: return launch_quant_mx<__half>(x, R, K, kind, packed, sblk, stream);
        default: return launch_quant_mx<__nv_bfloat16>(x, R, K, kind, packed, sblk, stream);
    }
}

int mx8_mul(const void* ap, const void* as, const void* bp, const void* bs, void* op, void* os,
            int64_t R, int64_t K, cudaStream_t stream) {
    if (K <= 0 || (K % 128) != 0) {
        fprintf(stderr, "thor_fp4: mx8_mul needs K %% 128 == 0 (got %ld)\n", (long)K);
        return TFP4_ERR_BAD_K;
    }
    if (R <= 0) return TFP4_OK;
    if (misaligned(ap, 8) || misaligned(bp, 8) || misaligned(op, 8) || misaligned(os, 8)) {
        fprintf(stderr, "thor_fp4: mx8_mul needs 8-byte aligned buffers\n");
        return TFP4_ERR_BAD_ARG;
    }
    dim3 grid((unsigned)((K + QT_COLS - 1) / QT_COLS), (unsigned)((R + QT_ROWS - 1) / QT_ROWS));
    mx8_mul_kernel<<<grid, QT_THREADS, 0, stream>>>(
        (const uint8_t*)ap, (const uint8_t*)as, (const uint8_t*)bp, (const uint8_t*)bs,
        (uint8_t*)op, (uint8_t*)os, R, K);
    TFP4_CK(cudaGetLastError());
    return TFP4_OK;
}

}  // namespace tfp4
