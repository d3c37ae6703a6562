// NVFP4 / MXFP8 quantize: IEEE arithmetic policies and host launchers.
#include "quantize_impl.cuh"
#include "internal.h"
#include "ptx.cuh"

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


// The same quantizer for large tensors, one 128 x 128 tile per CTA of 128 threads: the tile arrives as two TMA boxes of 128 rows x
// 128 bytes (128-byte swizzle), thread t owns row t (4 blocks of 32 elements, no shuffles), the e4m3 codes go back into the first
// half of the same buffer and leave as one TMA store, the 512-byte scale chunk as one coalesced store.  With ~33 KB of shared
// memory and 128 threads per CTA six or seven CTAs share an SM, each with one bulk load or store in flight, and no load/store
// instruction touches global memory except the scale chunk.  Chunk c (16 bytes) of row r of a box sits at r * 128 + ((c ^ (r & 7)) << 4):
// a quarter-warp (8 consecutive rows) reads 8 different chunks, which covers all 32 banks once.
constexpr int MXT_THREADS = 128;
constexpr int MXT_SMEM = 2 * 128 * 128 + 1024;

__global__ void __launch_bounds__(MXT_THREADS)
mxfp8_quantize_tile_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmC, uint8_t* __restrict__ sc,
                           int M, int K, int* status, long long limit) {
    extern __shared__ uint8_t mx_smem_raw[];
    __shared__ __align__(8) uint64_t bar;
    __shared__ __align__(16) uint32_t s_sc[128];
    __shared__ int s_abort;
    const uint32_t base = (smem_u32(mx_smem_raw) + 1023u) & ~1023u;
    const int t = threadIdx.x;
    const int tiles_n = K / 128;
    const int row0 = (blockIdx.x / tiles_n) * 128, col0 = (blockIdx.x % tiles_n) * 128;
    if (t == 0) {
        s_abort = 0;
        mbar_init(smem_u32(&bar), 1);
        fence_mbar_init();
        mbar_arrive_expect_tx(smem_u32(&bar), 2 * 128 * 128);
        tma_load_2d(base, &tmA, smem_u32(&bar), col0, row0);
        tma_load_2d(base + 128 * 128, &tmA, smem_u32(&bar), col0 + 64, row0);
    }
    __syncthreads();
    WaitCtx wc{&s_abort, status, limit};
    const bool ok = mbar_wait(wc, smem_u32(&bar), 0);
    uint4 v[16];
    const uint32_t row_base = base + uint32_t(t) * 128u;
    const uint32_t sw = uint32_t(t & 7);
#pragma unroll
    for (int c = 0; c < 16; c++) {
        const uint32_t a = row_base + uint32_t(c >> 3) * (128u * 128u) + ((uint32_t(c & 7) ^ sw) << 4);
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v[c].x), "=r"(v[c].y), "=r"(v[c].z), "=r"(v[c].w) : "r"(a));
    }
    // every row is in registers: the first half of the buffer becomes the output tile.  The outcome of the wait is agreed on
    // by the whole CTA, so that all of its threads leave together if it ran out
    if (!__syncthreads_and(ok ? 1 : 0)) {
        if (t == 0) {                // the copy that was issued must still land before this CTA may exit (bounded)
            const long long t0 = clock64();
            while (!mbar_try_wait_sleep(smem_u32(&bar), 0, 20000u))
                if (clock64() - t0 > limit) break;
        }
        return;
    }
    uint32_t scales = 0;
#pragma unroll
    for (int kb = 0; kb < 4; kb++) {
        float a = fmaxf(fmaxf(amax8(v[4 * kb]), amax8(v[4 * kb + 1])), fmaxf(amax8(v[4 * kb + 2]), amax8(v[4 * kb + 3])));
        const float scale = fmaxf(__fmul_rn(a, 0.002232142857f), 0.000000000001f);
        const uint32_t s8 = e8m0_round_up(scale);
        scales |= s8 << (8 * kb);
        const float inv = __uint_as_float(s8 == 254u ? 0x00400000u : (254u - s8) << 23);
#pragma unroll
        for (int h = 0; h < 2; h++) {            // 16 codes = one 16-byte chunk of the output row
            const uint32_t w[8] = {v[4 * kb + 2 * h].x, v[4 * kb + 2 * h].y, v[4 * kb + 2 * h].z, v[4 * kb + 2 * h].w,
                                   v[4 * kb + 2 * h + 1].x, v[4 * kb + 2 * h + 1].y, v[4 * kb + 2 * h + 1].z, v[4 * kb + 2 * h + 1].w};
            uint32_t out[4] = {0, 0, 0, 0};
#pragma unroll
            for (int j = 0; j < 8; j++) {
                float2 f = bf16x2_to_f2(w[j]);
                f.x = __fmul_rn(f.x, inv);
                f.y = __fmul_rn(f.y, inv);
                out[j >> 1] |= uint32_t(__nv_cvt_float2_to_fp8x2(f, __NV_SATFINITE, __NV_E4M3)) << (16 * (j & 1));
            }
            st_shared_v4(row_base + ((uint32_t(2 * kb + h) ^ sw) << 4), out[0], out[1], out[2], out[3]);
        }
    }
    s_sc[(t & 31) * 4 + (t >> 5)] = (row0 + t < M) ? scales : 0u;          // rows past M: scale 0
    fence_proxy_async();
    __syncthreads();
    reinterpret_cast<uint32_t*>(sc + (int64_t(row0 / 128) * tiles_n + col0 / 128) * 512)[t] = s_sc[t];
    if (t == 0) {
        tma_store_2d(&tmC, base, col0, row0);         // rows past M are clipped
        tma_store_commit();
        tma_store_wait_read<0>();                     // the buffer must outlive the copy's reads
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

cudaError_t launch_mxfp8_quantize_tiles(const CUtensorMap& tmA, const CUtensorMap& tmC, void* sc, int M, int K, int* status, long long limit,
                                        cudaStream_t s) {
    static_assert(MXT_SMEM <= 48 * 1024, "no opt-in needed for the dynamic shared memory");
    const int tiles = ((M + 127) / 128) * (K / 128);
    mxfp8_quantize_tile_kernel<<<tiles, MXT_THREADS, MXT_SMEM, s>>>(tmA, tmC, static_cast<uint8_t*>(sc), M, K, status, limit);
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
