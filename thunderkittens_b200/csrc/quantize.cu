// NVFP4 / MXFP8 quantize: IEEE arithmetic policies and host launchers.
#include "quantize_impl.cuh"
#include "internal.h"

namespace tkb {

// The reference's torch specification (kernels/gemm/nvfp4_b200/test_quantize.py:28-41), every
// operation a correctly rounded IEEE fp32 operation:
//   sg_enc = 2688 / max(amax, 1e-12);  sg_dec = 1 / sg_enc
//   scale  = (amax16 / 6) * sg_enc;    s_enc  = 1 / max(float(e4m3(scale)) * sg_dec, 1e-12)
struct ArithSpec {
    static __device__ __forceinline__ void global_scales(float amax, float& sg_dec, float& sg_enc) {
        sg_enc = __fdiv_rn(6.0f * 448.0f, fmaxf(amax, 0.000000000001f));
        sg_dec = __frcp_rn(sg_enc);
    }
    static __device__ __forceinline__ float block_scale(float amax16, float sg_enc) { return __fmul_rn(__fdiv_rn(amax16, 6.0f), sg_enc); }
    static __device__ __forceinline__ float block_enc(float s_local, float sg_dec) { return __frcp_rn(fmaxf(__fmul_rn(s_local, sg_dec), 0.000000000001f)); }
    static __device__ __forceinline__ float scale_value(float x, float s_enc) { return __fmul_rn(x, s_enc); }
};

// The reference kernel's association (nvfp4_b200_gemm.cu:420-422, 447-449): sg_dec = amax / 2688 is
// formed first and sg_enc = 1 / max(sg_dec, 1e-12) derived from it; correctly rounded IEEE operations.
struct ArithKernelIeee : ArithSpec {
    static __device__ __forceinline__ void global_scales(float amax, float& sg_dec, float& sg_enc) {
        sg_dec = __fdiv_rn(amax, 6.0f * 448.0f);
        sg_enc = __frcp_rn(fmaxf(sg_dec, 0.000000000001f));
    }
};

// Per-tensor |max| only (row-sharded tensors reduce this across ranks before quantizing).
__global__ void __launch_bounds__(Q_THREADS)
absmax_kernel(const __nv_bfloat16* __restrict__ A, int64_t lda, int M, int K, unsigned int* out_bits) {
    __shared__ float s_warp[Q_THREADS / 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tiles_n = (K + QT_COLS - 1) / QT_COLS;
    const int num_tiles = ((M + QT_ROWS - 1) / QT_ROWS) * tiles_n;
    float local = 0.f;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        uint4 v[8];
        load_tile(A, lda, M, K, tile_coord(tile, tiles_n), warp, lane, v);
#pragma unroll
        for (int i = 0; i < 8; i++) local = fmaxf(local, amax8(v[i]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) local = fmaxf(local, __shfl_xor_sync(0xffffffffu, local, o));
    if (lane == 0) s_warp[warp] = local;
    __syncthreads();
    if (threadIdx.x == 0) {
        float m = s_warp[0];
#pragma unroll
        for (int w = 1; w < Q_THREADS / 32; w++) m = fmaxf(m, s_warp[w]);
        atomicMax(out_bits, __float_as_uint(m));
    }
}

// ------------------------------------------------------------------------------ MXFP8 -----
// e8m0 code of a positive, finite or infinite, normal float, rounded toward +inf and saturated to the largest finite code:
// what __nv_cvt_float_to_e8m0(x, __NV_SATFINITE, cudaRoundPosInf) returns for such x (the reference's call,
// mxfp8_b200_gemm.cu:396), in three integer instructions: any mantissa bit carries into the exponent field.
__device__ __forceinline__ uint32_t e8m0_round_up(float x) {
    const uint32_t e = (__float_as_uint(x) + 0x007fffffu) >> 23;
    return e > 254u ? 254u : e;
}

__global__ void __launch_bounds__(Q_THREADS)
mxfp8_quantize_kernel(const __nv_bfloat16* __restrict__ A, int64_t lda, uint8_t* __restrict__ codes, int64_t ldc,
                      uint8_t* __restrict__ sc, int M, int K) {
    __shared__ __align__(16) uint8_t s_sc[2][512];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tiles_n = (K + QT_COLS - 1) / QT_COLS;
    const int num_tiles = ((M + QT_ROWS - 1) / QT_ROWS) * tiles_n;
    const int k_chunks = K / 128;
    int buf = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, buf ^= 1) {
        const TileCoord tc = tile_coord(t, tiles_n);
        uint4 v[8];
        load_tile(A, lda, M, K, tc, warp, lane, v);
        const int kb_local = (lane & 15) >> 2;        // 32-element block within the tile
        const int col = tc.col0 + (lane & 15) * 8;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int r = warp * 16 + 2 * i + (lane >> 4);
            float a = amax8(v[i]);
            a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 1));
            a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 2));
            const float scale = fmaxf(__fmul_rn(a, 0.002232142857f), 0.000000000001f);
            const uint32_t s8 = e8m0_round_up(scale);
            if ((lane & 3) == 0) s_sc[buf][(r & 31) * 16 + (r >> 5) * 4 + kb_local] = (tc.row0 + r < M) ? uint8_t(s8) : uint8_t(0);   // rows past M: 0
            // 1 / 2^(s8-127) = 2^(127-s8), exact for every finite e8m0 code: exponent field 254 - s8, and the denormal 2^-127 for s8 = 254
            const float inv = __uint_as_float(s8 == 254u ? 0x00400000u : (254u - s8) << 23);
            const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
            uint32_t out[2] = {0, 0};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float2 f = bf16x2_to_f2(w[j]);
                f.x = __fmul_rn(f.x, inv);
                f.y = __fmul_rn(f.y, inv);
                out[j >> 1] |= uint32_t(__nv_cvt_float2_to_fp8x2(f, __NV_SATFINITE, __NV_E4M3)) << (16 * (j & 1));
            }
            const int row = tc.row0 + r;
            if (row < M && col < K) *reinterpret_cast<uint2*>(codes + int64_t(row) * ldc + col) = make_uint2(out[0], out[1]);
        }
        __syncthreads();
        if (threadIdx.x < 128 && tc.col0 / 128 < k_chunks) {
            uint32_t* dst = reinterpret_cast<uint32_t*>(sc + (int64_t(tc.row0 / 128) * k_chunks + tc.col0 / 128) * 512);
            dst[threadIdx.x] = reinterpret_cast<const uint32_t*>(&s_sc[buf][0])[threadIdx.x];
        }
    }
}


// fp32 <-> packed e2m1 helpers (nvfp4_utils::fp32_to_fp4x2_kernel / fp4x2_to_fp32_kernel,
// nvfp4_b200_gemm.cu:568-583)
__global__ void fp32_to_fp4x2_kernel(const float2* __restrict__ in, uint8_t* __restrict__ out, size_t n_pairs) {
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n_pairs; i += size_t(blockDim.x) * gridDim.x)
        out[i] = (uint8_t)__nv_cvt_float2_to_fp4x2(in[i], __NV_E2M1, cudaRoundNearest);
}
__global__ void fp4x2_to_fp32_kernel(const uint8_t* __restrict__ in, float2* __restrict__ out, size_t n_pairs) {
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n_pairs; i += size_t(blockDim.x) * gridDim.x) {
        __half2_raw h = __nv_cvt_fp4x2_to_halfraw2(in[i], __NV_E2M1);
        out[i] = __half22float2(*reinterpret_cast<__half2*>(&h));
    }
}


cudaError_t launch_nvfp4_quantize_fast(const NvQuantArgs& a);   // quantize_fast.cu

cudaError_t launch_nvfp4_quantize_mode(const NvQuantArgs& a, int mode) {
    switch (mode) {
        case 0: return launch_nvfp4_quantize<ArithSpec>(a);
        case 1: return launch_nvfp4_quantize<ArithKernelIeee>(a);
        case 2: return launch_nvfp4_quantize_fast(a);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_absmax(const void* A, int64_t lda, int M, int K, unsigned int* out_bits, int sm_count, cudaStream_t s) {
    const int tiles = ((M + QT_ROWS - 1) / QT_ROWS) * ((K + QT_COLS - 1) / QT_COLS);
    int grid = sm_count * 4 < tiles ? sm_count * 4 : tiles;
    absmax_kernel<<<grid < 1 ? 1 : grid, Q_THREADS, 0, s>>>(static_cast<const __nv_bfloat16*>(A), lda, M, K, out_bits);
    return cudaGetLastError();
}

cudaError_t launch_mxfp8_quantize(const void* A, int64_t lda, void* codes, int64_t ldc, void* sc, int M, int K, int sm_count,
                                  cudaStream_t s) {
    const int tiles = ((M + QT_ROWS - 1) / QT_ROWS) * ((K + QT_COLS - 1) / QT_COLS);
    // a persistent grid of exactly the CTAs that are resident at once: with more, the second batch of CTAs starts when the first
    // ends and the tiles no longer divide evenly (8 CTAs per SM over 4096 tiles: 3 or 4 tiles per CTA, two batches = 8 tile
    // times for 6.9 tiles' worth of work per resident slot)
    static int blocks_per_sm = 0;
    if (blocks_per_sm == 0) {
        int b = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&b, mxfp8_quantize_kernel, Q_THREADS, 0) != cudaSuccess || b < 1) b = 4;
        blocks_per_sm = b > 8 ? 8 : b;
    }
    static const int bps_env = getenv("TKB_MXQ_BLOCKS_PER_SM") ? atoi(getenv("TKB_MXQ_BLOCKS_PER_SM")) : 0;
    const int per_sm = bps_env > 0 ? bps_env : blocks_per_sm;
    int grid = sm_count * per_sm < tiles ? sm_count * per_sm : tiles;
    mxfp8_quantize_kernel<<<grid < 1 ? 1 : grid, Q_THREADS, 0, s>>>(static_cast<const __nv_bfloat16*>(A), lda,
                                                                  static_cast<uint8_t*>(codes), ldc, static_cast<uint8_t*>(sc), M, K);
    return cudaGetLastError();
}

cudaError_t launch_fp32_to_fp4x2(const float* in, void* out, size_t n_pairs, cudaStream_t s) {
    fp32_to_fp4x2_kernel<<<1024, 128, 0, s>>>(reinterpret_cast<const float2*>(in), static_cast<uint8_t*>(out), n_pairs);
    return cudaGetLastError();
}
cudaError_t launch_fp4x2_to_fp32(const void* in, float* out, size_t n_pairs, cudaStream_t s) {
    fp4x2_to_fp32_kernel<<<1024, 128, 0, s>>>(static_cast<const uint8_t*>(in), reinterpret_cast<float2*>(out), n_pairs);
    return cudaGetLastError();
}

} // namespace tkb
