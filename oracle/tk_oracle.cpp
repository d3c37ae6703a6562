// CPU ORACLE — test infrastructure only.
//
// Plain C++ restatement of the arithmetic of the ThunderKittens quantized-inference
// path.  It exists to CHECK the CUDA library; nothing in the product path links,
// loads or calls it.  Every function cites the reference file:line it restates
// (paths are relative to the ThunderKittens source tree).
//
// Pinning of this oracle:
//   * codecs (e2m1 / e4m3 / e8m0 / bf16) are cross-checked against the host
//     implementations in the CUDA toolkit headers cuda_fp4.h / cuda_fp8.h /
//     cuda_bf16.h, the same functions the reference kernels call;
//   * the GEMM loops are cross-checked against the reference's own kernels/gemm/common.cuh
//     bodies compiled for the host (oracle/_ref, built by oracle/build.py);
//   * the quantizers are cross-checked against golden vectors produced by importing the
//     reference's torch specs (tests/golden/make_golden.py);
//   * MoE combine and skinny-M GEMMs have no counterpart in the reference: parity unpinned
//     for those two, the restatement here is the specification.
//
// Build: g++ -O3 -march=x86-64-v3 -fopenmp -shared -fPIC (see oracle/build.py).

#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <vector>
#include <algorithm>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

inline uint32_t f2u(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }
inline float u2f(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }

// ---------------------------------------------------------------- bf16 ------------------
inline float bf16_to_f32(uint16_t h) { return u2f(uint32_t(h) << 16); }
// round-to-nearest-even; NaN -> 0x7fff (what __float2bfloat16_rn returns on the host and device)
inline uint16_t f32_to_bf16(float f) {
    uint32_t u = f2u(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fffu;
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return uint16_t(u >> 16);
}

// ---------------------------------------------------------------- e2m1 ------------------
// Magnitudes {0, .5, 1, 1.5, 2, 3, 4, 6}; sign in bit 3.  Round to nearest even, saturate
// to +-6 (cvt.rn.satfinite.e2m1x2.f32; nvfp4_b200_gemm.cu:524, 572).  NaN -> +6 (0x7),
// which is what the toolkit's host conversion returns.
const float kE2M1[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
inline uint8_t f32_to_e2m1(float x) {
    uint32_t u = f2u(x);
    uint8_t sign = uint8_t((u >> 31) << 3);
    float a = std::fabs(x);
    if (a != a) return 0x7;  // NaN
    uint8_t m;
    // midpoints: .25 .75 1.25 1.75 2.5 3.5 5 ; ties go to the even code (even mantissa bit)
    if      (a <= 0.25f) m = 0;            // tie .25 -> 0   (code 0 even)
    else if (a <  0.75f) m = 1;            // tie .75 -> 1.0 (code 2 even)
    else if (a <= 1.25f) m = 2;            // tie 1.25 -> 1.0
    else if (a <  1.75f) m = 3;            // tie 1.75 -> 2.0 (code 4)
    else if (a <= 2.5f)  m = 4;            // tie 2.5 -> 2.0
    else if (a <  3.5f)  m = 5;            // tie 3.5 -> 4.0 (code 6)
    else if (a <= 5.0f)  m = 6;            // tie 5 -> 4.0
    else                 m = 7;
    return uint8_t(sign | m);
}
inline float e2m1_to_f32(uint8_t c) {
    float v = kE2M1[c & 7];
    return (c & 8) ? -v : v;
}

// ---------------------------------------------------------------- e4m3 ------------------
// OCP e4m3fn: bias 7, max 448, no inf, NaN = 0x7f.  Round to nearest even, saturate to finite
// (__nv_fp8_e4m3(float) uses __NV_SATFINITE; nvfp4_b200_gemm.cu:506, mxfp8_b200_gemm.cu:405).
inline uint8_t f32_to_e4m3(float x) {
    uint32_t u = f2u(x);
    uint8_t sign = uint8_t((u >> 24) & 0x80);
    uint32_t au = u & 0x7fffffffu;
    if (au > 0x7f800000u) return 0x7f;                        // NaN (sign dropped, as the toolkit does)
    float a = u2f(au);
    if (a >= 448.0f) {
        // values in (448, 464) round to 448; >= 464 saturates to 448 too
        return uint8_t(sign | 0x7e);
    }
    if (a < 0.0009765625f /* 2^-10 = half of min subnormal 2^-9 */) {
        return sign;                                          // rounds to zero (tie 2^-10 -> 0, even)
    }
    if (a == 0.0009765625f) return sign;
    int e; // a = m * 2^e, m in [1,2)
    uint32_t exp = au >> 23;
    uint32_t man = au & 0x7fffffu;
    e = int(exp) - 127;
    if (exp == 0) { // fp32 subnormal: far below e4m3 range, already handled above
        return sign;
    }
    if (e < -6) {
        // e4m3 subnormal: value = k * 2^-9, k in 0..7 ; RNE of a / 2^-9
        float q = a * 512.0f; // exact (power of two scaling)
        float r = std::nearbyintf(q); // default rounding mode = RNE
        int k = int(r);
        if (k >= 8) return uint8_t(sign | 0x08); // rounds up into the first normal (2^-6)
        return uint8_t(sign | k);
    }
    // normal: keep 3 mantissa bits
    uint32_t keep = man >> 20;
    uint32_t rest = man & 0xfffffu;
    uint32_t half = 0x80000u;
    if (rest > half || (rest == half && (keep & 1u))) {
        keep++;
        if (keep == 8) { keep = 0; e++; }
    }
    int be = e + 7;
    if (be > 15 || (be == 15 && keep == 7)) return uint8_t(sign | 0x7e); // would be NaN slot / overflow
    return uint8_t(sign | (be << 3) | keep);
}
inline float e4m3_to_f32(uint8_t c) {
    uint32_t sign = (c & 0x80) ? 1u : 0u;
    uint32_t be = (c >> 3) & 0xf;
    uint32_t m = c & 7;
    float v;
    if (be == 0xf && m == 7) v = NAN;
    else if (be == 0) v = float(m) * 0.001953125f; // m * 2^-9
    else v = std::ldexp(1.0f + float(m) * 0.125f, int(be) - 7);
    return sign ? -v : v;
}

// ---------------------------------------------------------------- e8m0 ------------------
// byte = biased exponent (bias 127); value 2^(b-127); 0xff = NaN.
// __nv_cvt_float_to_e8m0(x, __NV_SATFINITE, cudaRoundPosInf) (mxfp8_b200_gemm.cu:396):
// |x| rounded UP to the next power of two, saturating at 2^127 (0xfe); zero and fp32
// subnormals... follow the toolkit: |x| is first rounded up to bf16, then the exponent is
// taken and bumped if any mantissa bit is set.
inline uint8_t f32_to_e8m0_rp_sat(float x) {
    uint32_t au = f2u(x) & 0x7fffffffu;
    if (au > 0x7f800000u) return 0xff;                 // NaN
    if (au == 0x7f800000u) return 0xfe;                // inf saturates
    uint32_t exp = au >> 23;
    uint32_t man = au & 0x7fffffu;
    if (exp == 0) {
        // zero -> 0 ; subnormal rounds up to 2^-126 (b=1) unless it is exactly 0
        if (man == 0) return 0;
        // a subnormal is <= 2^-126 * (1 - 2^-23); rounding up gives 2^-126 at most, 2^-127 when
        // it is <= 2^-127
        return (man <= 0x400000u) ? 0 : 1;
    }
    uint32_t b = exp + (man ? 1u : 0u);
    if (b > 0xfe) b = 0xfe;
    return uint8_t(b);
}
inline float e8m0_to_f32(uint8_t b) {
    if (b == 0xff) return NAN;
    if (b == 0) return u2f(0x00400000u); // 2^-127 (fp32 subnormal)
    return u2f(uint32_t(b) << 23);
}

// ------------------------------------------------------- scale swizzle index ------------
// kernels/gemm/common.cuh:105-116 ; same formula in nvfp4_b200_gemm.cu:530-536 and
// mxfp8_b200_gemm.cu:417-418.  One 512-byte chunk per (128 rows x 4 K-blocks).
inline size_t scale_swizzle_idx(int row, int k_block, int k_blocks) {
    int m_block = row / 128;
    int groups = k_blocks / 4;
    int group = k_block / 4;
    int local = (row % 32) * 16 + ((row / 32) % 4) * 4 + (k_block % 4);
    return (size_t(m_block) * groups + group) * 512 + local;
}

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

} // namespace

extern "C" {

int tko_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// Thread count of the OpenMP runtime this library (and anything else bound to the same runtime) uses from now on.
void tko_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

// ------------------------------------------------------------------ codecs (arrays) -----
void tko_f32_to_bf16(const float* in, uint16_t* out, size_t n) { for (size_t i = 0; i < n; i++) out[i] = f32_to_bf16(in[i]); }
void tko_bf16_to_f32(const uint16_t* in, float* out, size_t n) { for (size_t i = 0; i < n; i++) out[i] = bf16_to_f32(in[i]); }
void tko_f32_to_e4m3(const float* in, uint8_t* out, size_t n) { for (size_t i = 0; i < n; i++) out[i] = f32_to_e4m3(in[i]); }
void tko_e4m3_to_f32(const uint8_t* in, float* out, size_t n) { for (size_t i = 0; i < n; i++) out[i] = e4m3_to_f32(in[i]); }
void tko_f32_to_e8m0(const float* in, uint8_t* out, size_t n) { for (size_t i = 0; i < n; i++) out[i] = f32_to_e8m0_rp_sat(in[i]); }
void tko_e8m0_to_f32(const uint8_t* in, float* out, size_t n) { for (size_t i = 0; i < n; i++) out[i] = e8m0_to_f32(in[i]); }
// nvfp4_utils::fp32_to_fp4x2_kernel / fp4x2_to_fp32_kernel (nvfp4_b200_gemm.cu:568-583):
// element 2i in the low nibble, 2i+1 in the high nibble.
void tko_fp32_to_fp4x2(const float* in, uint8_t* out, size_t n_pairs) {
    for (size_t i = 0; i < n_pairs; i++) out[i] = uint8_t(f32_to_e2m1(in[2 * i]) | (f32_to_e2m1(in[2 * i + 1]) << 4));
}
void tko_fp4x2_to_fp32(const uint8_t* in, float* out, size_t n_pairs) {
    for (size_t i = 0; i < n_pairs; i++) { out[2 * i] = e2m1_to_f32(in[i] & 0xf); out[2 * i + 1] = e2m1_to_f32(in[i] >> 4); }
}

size_t tko_scale_swizzle_idx(int row, int k_block, int k_blocks) { return scale_swizzle_idx(row, k_block, k_blocks); }

// kernels/gemm/common.cuh:28-48 fill_kernel<RANDOM>: splitmix64 of (seed+idx), upper 24 bits -> [0,1)
void tko_fill_uniform_f32(float* out, size_t n, uint64_t seed, float lo, float hi) {
    for (size_t i = 0; i < n; i++) {
        uint64_t x = seed + i;
        x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ULL;
        x = (x ^ (x >> 27)) * 0x94d049bb133111ebULL;
        x = x ^ (x >> 31);
        float u = float(x >> 40) * (1.0f / 16777216.0f);
        out[i] = u * (hi - lo) + lo;
    }
}

// ------------------------------------------------------------------ NVFP4 quantize ------
// Per-tensor absolute maximum of a bf16 tensor, as a float
// (nvfp4_quantize::absmax_kernel, nvfp4_b200_gemm.cu:360-418; NaNs are dropped by __hmax).
float tko_absmax_bf16(const uint16_t* A, size_t n) {
    uint16_t best = 0;
    for (size_t i = 0; i < n; i++) {
        uint16_t a = A[i] & 0x7fffu;
        if (a > 0x7f80u) continue;
        best = std::max(best, a);
    }
    return bf16_to_f32(best);
}

// assoc = 0: the kernel's association (nvfp4_b200_gemm.cu:420-422, 447-449, 506, 512-513):
//             sg_dec = amax / 2688 ; sg_enc = 1 / max(sg_dec, 1e-12)
// assoc = 1: the torch spec's association (nvfp4_b200/test_quantize.py:28-29):
//             sg_enc = 2688 / max(amax, 1e-12) ; sg_dec = 1 / sg_enc
// Everything after that is common:
//   scale_e4m3 = e4m3_rn(amax16 / 6 * sg_enc)                       (l.506 / spec l.36-37)
//   s_enc      = 1 / max(float(scale_e4m3) * sg_dec, 1e-12)         (l.513 / spec l.39)
//   code       = e2m1_rn(x * s_enc)                                 (l.519-524 / spec l.41)
// All operations are IEEE fp32 here (the reference kernel is built with --use_fast_math, whose
// approximate reciprocal cannot be restated on a CPU; the CUDA library's default mode uses the
// same IEEE operations as this function).
// scale_2d: the block amax is shared by the 16 rows of a 16x16 block (l.494-501 / spec l.32-34).
// amax_in >= 0 supplies the per-tensor amax (row-sharded tensors); < 0 computes it from A.
// Rows are padded to a multiple of 128 in the scale tensor only; pad bytes are written as 0.
void tko_nvfp4_quantize(const uint16_t* A, int M, int K, int scale_2d, int assoc, float amax_in,
                        uint8_t* codes, uint8_t* sc, float* sg_out) {
    const int k_blocks = K / 16;
    const float amax = amax_in >= 0.f ? amax_in : tko_absmax_bf16(A, size_t(M) * K);
    float sg_dec, sg_enc;
    if (assoc == 0) {
        sg_dec = amax / (6.0f * 448.0f);
        sg_enc = 1.0f / std::fmax(sg_dec, 0.000000000001f);
    } else {
        sg_enc = (6.0f * 448.0f) / std::fmax(amax, 0.000000000001f);
        sg_dec = 1.0f / sg_enc;
    }
    *sg_out = sg_dec;
    const int Mp = ceil_div(M, 128) * 128;
    std::memset(sc, 0, size_t(Mp / 128) * (k_blocks / 4) * 512);
#pragma omp parallel for schedule(static)
    for (int r0 = 0; r0 < M; r0 += 16) {
        const int r1 = std::min(r0 + 16, M);
        for (int kb = 0; kb < k_blocks; kb++) {
            float amax2d = 0.f;
            float amax_row[16];
            for (int r = r0; r < r1; r++) {
                uint16_t best = 0;
                for (int j = 0; j < 16; j++) {
                    uint16_t a = A[size_t(r) * K + kb * 16 + j] & 0x7fffu;
                    if (a > 0x7f80u) continue;
                    best = std::max(best, a);
                }
                amax_row[r - r0] = bf16_to_f32(best);
                amax2d = std::fmax(amax2d, amax_row[r - r0]);
            }
            for (int r = r0; r < r1; r++) {
                const float am = scale_2d ? amax2d : amax_row[r - r0];
                const uint8_t s8 = f32_to_e4m3(am / 6.0f * sg_enc);
                sc[scale_swizzle_idx(r, kb, k_blocks)] = s8;
                const float s_local = e4m3_to_f32(s8);
                const float s_enc = 1.0f / std::fmax(s_local * sg_dec, 0.000000000001f);
                for (int j = 0; j < 16; j += 2) {
                    const size_t idx = size_t(r) * K + kb * 16 + j;
                    const uint8_t lo = f32_to_e2m1(bf16_to_f32(A[idx]) * s_enc);
                    const uint8_t hi = f32_to_e2m1(bf16_to_f32(A[idx + 1]) * s_enc);
                    codes[idx / 2] = uint8_t(lo | (hi << 4));
                }
            }
        }
    }
}

// ------------------------------------------------------------------ MXFP8 quantize ------
// mxfp8_quantize::kernel (mxfp8_b200_gemm.cu:386-421):
//   scale  = max(amax32 * 0.002232142857f, 1e-12f)
//   s_e8m0 = e8m0(scale, round toward +inf, saturate finite)
//   code   = e4m3_rn(x * (1 / 2^s))            (the reciprocal of a power of two is exact)
void tko_mxfp8_quantize(const uint16_t* A, int M, int K, uint8_t* codes, uint8_t* sc) {
    const int k_blocks = K / 32;
    const int Mp = ceil_div(M, 128) * 128;
    std::memset(sc, 0, size_t(Mp / 128) * (k_blocks / 4) * 512);
#pragma omp parallel for schedule(static)
    for (int r = 0; r < M; r++) {
        for (int kb = 0; kb < k_blocks; kb++) {
            uint16_t best = 0;
            for (int j = 0; j < 32; j++) {
                uint16_t a = A[size_t(r) * K + kb * 32 + j] & 0x7fffu;
                if (a > 0x7f80u) continue;
                best = std::max(best, a);
            }
            const float scale = std::fmax(bf16_to_f32(best) * 0.002232142857f, 0.000000000001f);
            const uint8_t s8 = f32_to_e8m0_rp_sat(scale);
            sc[scale_swizzle_idx(r, kb, k_blocks)] = s8;
            const float inv = 1.0f / e8m0_to_f32(s8);
            for (int j = 0; j < 32; j++) {
                const size_t idx = size_t(r) * K + kb * 32 + j;
                codes[idx] = f32_to_e4m3(bf16_to_f32(A[idx]) * inv);
            }
        }
    }
}

// ------------------------------------------------------------------ GEMM oracles --------
// All three follow the per-output-element loops of kernels/gemm/common.cuh: a single fp32
// accumulator per output, k ascending, products formed as (a*sa)*(b*sb) with each factor rounded
// to fp32 first, accumulated with a fused multiply-add (the reference kernels are compiled with
// --use_fast_math, i.e. -fmad=true, so `acc += x*y` contracts to FMA), the per-tensor scale
// applied once at the end and a single rounding to bf16.
//
// Implementation: the dequantised factors (a*sa) and (b*sb) are materialised per row slab /
// column block and the k loop runs over 64 output columns at a time so the compiler can
// vectorise ACROSS outputs; each output still sees exactly the sequential-k FMA chain.
//
// rows [row0, row0+nrows) of D are produced (a slab), D points at the slab's first row.

} // extern "C"

namespace {
constexpr int CB = 64;  // columns per block

template <class DeqA, class DeqB>
void gemm_slab(uint16_t* D, int N, int K, int row0, int nrows, float final_scale, DeqA deqA, DeqB deqB) {
    const int ncb = ceil_div(N, CB);
#pragma omp parallel
    {
        std::vector<float> bt(size_t(K) * CB);   // [k][c]
        std::vector<float> arow(K);
#pragma omp for schedule(dynamic, 1)
        for (int cb = 0; cb < ncb; cb++) {
            const int c0 = cb * CB;
            const int cn = std::min(CB, N - c0);
            for (int c = 0; c < CB; c++) {
                if (c < cn) {
                    deqB(c0 + c, arow.data());
                    for (int k = 0; k < K; k++) bt[size_t(k) * CB + c] = arow[k];
                } else {
                    for (int k = 0; k < K; k++) bt[size_t(k) * CB + c] = 0.f;
                }
            }
            for (int r = 0; r < nrows; r++) {
                deqA(row0 + r, arow.data());
                float acc[CB];
                for (int c = 0; c < CB; c++) acc[c] = 0.f;
                for (int k = 0; k < K; k++) {
                    const float a = arow[k];
                    const float* b = &bt[size_t(k) * CB];
#pragma omp simd
                    for (int c = 0; c < CB; c++) acc[c] = __builtin_fmaf(a, b[c], acc[c]);
                }
                for (int c = 0; c < cn; c++) D[size_t(r) * N + c0 + c] = f32_to_bf16(acc[c] * final_scale);
            }
        }
    }
}
} // namespace

extern "C" {

// reference_nvfp4_gemm_kernel, kernels/gemm/common.cuh:173-231
void tko_nvfp4_gemm(const uint8_t* A, const uint8_t* A_sc, const float* A_sg,
                    const uint8_t* B, const uint8_t* B_sc, const float* B_sg,
                    uint16_t* D, int M, int N, int K, int row0, int nrows) {
    (void)M;
    const int kb = K / 16;
    auto deq = [kb, K](const uint8_t* X, const uint8_t* Xs) {
        return [=](int row, float* out) {
            for (int k = 0; k < K; k += 2) {
                uint8_t byte = X[size_t(row) * (K / 2) + k / 2];
                float s = e4m3_to_f32(Xs[scale_swizzle_idx(row, k / 16, kb)]);
                out[k] = e2m1_to_f32(byte & 0xf) * s;
                out[k + 1] = e2m1_to_f32(byte >> 4) * s;
            }
        };
    };
    const float gs = (*A_sg) * (*B_sg);
    gemm_slab(D, N, K, row0, nrows, gs, deq(A, A_sc), deq(B, B_sc));
}

// reference_blockscaled_gemm_kernel<fp8e4m3, fp8e8m0, bf16, 32>, kernels/gemm/common.cuh:118-161
// (no per-tensor scale: the final multiply is by 1.0f, which is exact)
void tko_mxfp8_gemm(const uint8_t* A, const uint8_t* A_sc, const uint8_t* B, const uint8_t* B_sc,
                    uint16_t* D, int M, int N, int K, int row0, int nrows) {
    (void)M;
    const int kb = K / 32;
    auto deq = [kb, K](const uint8_t* X, const uint8_t* Xs) {
        return [=](int row, float* out) {
            for (int k = 0; k < K; k++) {
                float s = e8m0_to_f32(Xs[scale_swizzle_idx(row, k / 32, kb)]);
                out[k] = e4m3_to_f32(X[size_t(row) * K + k]) * s;
            }
        };
    };
    gemm_slab(D, N, K, row0, nrows, 1.0f, deq(A, A_sc), deq(B, B_sc));
}

// reference_gemm_kernel<bf16, bf16, transpose_b=true>, kernels/gemm/common.cuh:73-98
void tko_bf16_gemm(const uint16_t* A, const uint16_t* B, uint16_t* D, int M, int N, int K, int row0, int nrows) {
    (void)M;
    auto deq = [K](const uint16_t* X) {
        return [=](int row, float* out) { for (int k = 0; k < K; k++) out[k] = bf16_to_f32(X[size_t(row) * K + k]); };
    };
    gemm_slab(D, N, K, row0, nrows, 1.0f, deq(A), deq(B));
}

// reference_gemm_kernel<fp8e4m3, bf16, transpose_b=true>: the oracle of the reference's dense fp8 GEMM
// (kernels/gemm/fp8_b200/fp8_b200_gemm.cu:298 over kernels/gemm/common.cuh:73-98)
void tko_fp8_gemm(const uint8_t* A, const uint8_t* B, uint16_t* D, int M, int N, int K, int row0, int nrows) {
    (void)M;
    auto deq = [K](const uint8_t* X) {
        return [=](int row, float* out) { for (int k = 0; k < K; k++) out[k] = e4m3_to_f32(X[size_t(row) * K + k]); };
    };
    gemm_slab(D, N, K, row0, nrows, 1.0f, deq(A), deq(B));
}

// Same arithmetic as tko_nvfp4_gemm with fp32 output (no final rounding) — used for the relative
// Frobenius-error gate, where the reference result is "dequantize then fp32 accumulate".
void tko_nvfp4_gemm_f32(const uint8_t* A, const uint8_t* A_sc, const float* A_sg,
                        const uint8_t* B, const uint8_t* B_sc, const float* B_sg,
                        float* D, int N, int K, int row0, int nrows) {
    std::vector<uint16_t> tmp; (void)tmp;
    const int kb = K / 16;
    const float gs = (*A_sg) * (*B_sg);
#pragma omp parallel for schedule(dynamic, 1)
    for (int r = 0; r < nrows; r++) {
        std::vector<float> a(K), b(K);
        for (int k = 0; k < K; k += 2) {
            uint8_t byte = A[size_t(row0 + r) * (K / 2) + k / 2];
            float s = e4m3_to_f32(A_sc[scale_swizzle_idx(row0 + r, k / 16, kb)]);
            a[k] = e2m1_to_f32(byte & 0xf) * s; a[k + 1] = e2m1_to_f32(byte >> 4) * s;
        }
        for (int c = 0; c < N; c++) {
            double acc = 0.0;
            for (int k = 0; k < K; k += 2) {
                uint8_t byte = B[size_t(c) * (K / 2) + k / 2];
                float s = e4m3_to_f32(B_sc[scale_swizzle_idx(c, k / 16, kb)]);
                acc += double(a[k]) * double(e2m1_to_f32(byte & 0xf) * s);
                acc += double(a[k + 1]) * double(e2m1_to_f32(byte >> 4) * s);
            }
            D[size_t(r) * N + c] = float(acc * double(gs));
        }
    }
}

// ------------------------------------------------------------------ MoE ------------------
// Routing for the MoE configuration: softmax over the expert logits, top-k by probability
// (ties -> lower expert id), probabilities renormalised over the chosen k.  The reference
// benchmark draws experts with torch.multinomial (moe_dispatch_gemm/benchmark.py:112-121) and
// has no gate weights; this routing is the one the benchmark configuration names, parity unpinned.
void tko_moe_route(const float* logits, int T, int E, int top_k, int32_t* experts, float* weights) {
#pragma omp parallel for schedule(static)
    for (int t = 0; t < T; t++) {
        const float* l = logits + size_t(t) * E;
        float mx = l[0];
        for (int e = 1; e < E; e++) mx = std::fmax(mx, l[e]);
        std::vector<float> p(E);
        float sum = 0.f;
        for (int e = 0; e < E; e++) { p[e] = std::exp(l[e] - mx); sum += p[e]; }
        for (int e = 0; e < E; e++) p[e] /= sum;
        std::vector<char> used(E, 0);
        float wsum = 0.f;
        for (int j = 0; j < top_k; j++) {
            int best = -1;
            for (int e = 0; e < E; e++) if (!used[e] && (best < 0 || p[e] > p[best])) best = e;
            used[best] = 1;
            experts[size_t(t) * top_k + j] = best;
            weights[size_t(t) * top_k + j] = p[best];
            wsum += p[best];
        }
        for (int j = 0; j < top_k; j++) weights[size_t(t) * top_k + j] /= wsum;
    }
}

// Dispatch schedule (moe_dispatch_gemm/benchmark.py:123-149): per expert the routed tokens in
// ascending global token order, each expert segment padded to a multiple of 128 rows with
// (-1,-1).  Output rows are (src_rank, src_row); tokens_per_rank tokens live on each rank.
// padded_per_expert[E] is written for all experts; the index list is produced for the experts
// [e0, e1) owned by one rank, and slot_of[T*top_k] receives, for the (token, j) pairs routed to
// those experts, the local padded row they occupy (-1 elsewhere) — the combine step's gather map.
// Returns the number of padded local rows.
int tko_moe_schedule(const int32_t* experts, int T, int E, int top_k, int tokens_per_rank,
                     int e0, int e1, int32_t* padded_per_expert, int32_t* pull_idx /* [rows][2] */,
                     int32_t* slot_of, int max_rows) {
    std::vector<int> cnt(E, 0);
    for (size_t i = 0; i < size_t(T) * top_k; i++) cnt[experts[i]]++;
    for (int e = 0; e < E; e++) padded_per_expert[e] = (cnt[e] + 127) / 128 * 128;
    std::vector<int> start(E, 0);
    int rows = 0;
    for (int e = e0; e < e1; e++) { start[e] = rows; rows += padded_per_expert[e]; }
    if (rows > max_rows) return -rows;
    for (int i = 0; i < rows * 2; i++) pull_idx[i] = -1;
    if (slot_of) for (size_t i = 0; i < size_t(T) * top_k; i++) slot_of[i] = -1;
    std::vector<int> fill(E, 0);
    for (int t = 0; t < T; t++)
        for (int j = 0; j < top_k; j++) {
            int e = experts[size_t(t) * top_k + j];
            if (e < e0 || e >= e1) continue;
            int row = start[e] + fill[e]++;
            pull_idx[2 * row] = t / tokens_per_rank;
            pull_idx[2 * row + 1] = t % tokens_per_rank;
            if (slot_of) slot_of[size_t(t) * top_k + j] = row;
        }
    return rows;
}

// Combine (no counterpart in the reference; parity unpinned): out[t] = bf16( sum_j w[t,j] * Y[row(t,j)] )
// accumulated in fp32 in ascending j with a fused multiply-add.  Y rows are bf16, I wide.
void tko_moe_combine(const uint16_t* Y, const int32_t* slot_of, const float* weights, int T, int top_k, int I,
                     uint16_t* out) {
#pragma omp parallel for schedule(static)
    for (int t = 0; t < T; t++) {
        for (int i = 0; i < I; i++) {
            float acc = 0.f;
            for (int j = 0; j < top_k; j++) {
                int row = slot_of[size_t(t) * top_k + j];
                if (row < 0) continue;
                acc = __builtin_fmaf(weights[size_t(t) * top_k + j], bf16_to_f32(Y[size_t(row) * I + i]), acc);
            }
            out[size_t(t) * I + i] = f32_to_bf16(acc);
        }
    }
}

} // extern "C"
