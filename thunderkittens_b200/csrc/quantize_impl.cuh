// bf16 -> NVFP4 / MXFP8 quantize kernels (HBM-bound, CUDA cores only).
//
// Replaces nvfp4_quantize::{zero,absmax,divide,quantize}_kernel (ThunderKittens
// kernels/gemm/nvfp4_b200/nvfp4_b200_gemm.cu:356-545) and mxfp8_quantize::kernel
// (kernels/gemm/mxfp8_b200/mxfp8_b200_gemm.cu:328-430).  Same outputs (packed nibbles, swizzled
// 512-byte scale chunks, fp32 per-tensor scale), different dataflow:
//   * one persistent launch: tiles of 128 rows x 128 columns are walked grid-stride, each thread
//     owns 8 consecutive bf16 (one 16-byte load) of 8 rows, so a half-warp reads one 256-byte row
//     segment and writes one 64-byte (NVFP4) or 128-byte (MXFP8) code segment: fully coalesced,
//     no shared-memory round trip for the data;
//   * the per-tensor amax pass of NVFP4 is fused into the same launch (cooperative grid, one
//     bounded grid barrier between the two passes; the second pass re-reads through L2);
//   * block amax comes from warp shuffles between the 2 (NVFP4) or 4 (MXFP8) lanes that share a
//     block; scales are staged in 1 KB of shared memory so each 512-byte chunk leaves as one
//     coalesced store.
// The arithmetic policy `Arith` fixes the exact floating-point operation sequence (see
// quantize.cu / quantize_fast.cu).
#pragma once
#include <cstdint>
#include <cstdlib>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_fp4.h>
#include <cuda_runtime.h>
#include "quantize_types.h"
#include "ptx.cuh"

namespace tkb {


constexpr int QT_ROWS = 128, QT_COLS = 128, Q_THREADS = 256;

__device__ __forceinline__ uint32_t habs2_max(uint32_t a, uint32_t b) {
    __nv_bfloat162 x = __habs2(*reinterpret_cast<__nv_bfloat162*>(&a));
    __nv_bfloat162 y = __habs2(*reinterpret_cast<__nv_bfloat162*>(&b));
    __nv_bfloat162 m = __hmax2(x, y);
    return *reinterpret_cast<uint32_t*>(&m);
}
// max |x| over the 8 bf16 packed in v, as a float (NaNs are dropped by __hmax2, as in the reference)
__device__ __forceinline__ float amax8(const uint4& v) {
    uint32_t m = habs2_max(habs2_max(v.x, v.y), habs2_max(v.z, v.w));
    __nv_bfloat162 mm = *reinterpret_cast<__nv_bfloat162*>(&m);
    return __bfloat162float(__hmax(mm.x, mm.y));
}
__device__ __forceinline__ float2 bf16x2_to_f2(uint32_t w) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
__device__ __forceinline__ float e4m3_to_float(uint8_t c) {
    __half_raw h = __nv_cvt_fp8_to_halfraw(c, __NV_E4M3);
    return __half2float(*reinterpret_cast<__half*>(&h));
}

struct TileCoord { int row0, col0; };
__device__ __forceinline__ TileCoord tile_coord(int tile, int tiles_n) {
    return TileCoord{(tile / tiles_n) * QT_ROWS, (tile % tiles_n) * QT_COLS};
}

// Loads this thread's 8 x 16 bytes of a tile (zeros outside the matrix).
__device__ __forceinline__ void load_tile(const __nv_bfloat16* A, int64_t lda, int M, int K, TileCoord tc, int warp, int lane,
                                          uint4 (&v)[8]) {
    const int col = tc.col0 + (lane & 15) * 8;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int row = tc.row0 + warp * 16 + 2 * i + (lane >> 4);
        if (row < M && col < K) v[i] = __ldg(reinterpret_cast<const uint4*>(A + int64_t(row) * lda + col));
        else v[i] = make_uint4(0, 0, 0, 0);
    }
}

// Bounded grid barrier on a QuantWork slot.  Returns the agreed per-tensor amax, or a negative
// value when a wait ran out (status receives the timeout code).
// With an exchange (xch.world > 1) the last block to arrive also trades this GPU's maximum with the other
// ranks over NVLink (one posted 64-bit store per peer, then bounded polls of its own slots) before it
// releases the grid, so a row-sharded tensor is quantized with the amax of the whole tensor in one launch.
constexpr unsigned int kAmaxFailed = 0xffffffffu;      // never a maximum of bf16 magnitudes (NaNs are dropped)
template <int THREADS = Q_THREADS>
__device__ __forceinline__ float grid_amax_barrier(QuantWork* ws, float block_amax, int* status, const QuantExchange& xch, long long spin_limit) {
    __shared__ float s_amax;
    __shared__ float s_warp[THREADS / 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) block_amax = fmaxf(block_amax, __shfl_xor_sync(0xffffffffu, block_amax, o));
    if (lane == 0) s_warp[warp] = block_amax;
    __syncthreads();
    if (threadIdx.x == 0) {
        float m = s_warp[0];
#pragma unroll
        for (int w = 1; w < THREADS / 32; w++) m = fmaxf(m, s_warp[w]);
        atomicMax(&ws->amax_bits, __float_as_uint(m));
        __threadfence();
        const unsigned int prev = atomicAdd(&ws->arrived, 1u);
        const bool exchange = xch.world > 1;
        const unsigned int epoch = xch.epoch_ptr ? *reinterpret_cast<const volatile unsigned int*>(xch.epoch_ptr) + 1u : xch.epoch;
        const unsigned int target = gridDim.x + (exchange ? 1u : 0u);
        const long long t0 = clock64();
        if (exchange && prev == gridDim.x - 1) {
            __threadfence();
            float g = __uint_as_float(*reinterpret_cast<volatile unsigned int*>(&ws->amax_bits));
            const unsigned long long mine = (static_cast<unsigned long long>(epoch) << 32) | __float_as_uint(g);
            for (int pr = 0; pr < xch.world; pr++)
                if (pr != xch.rank) asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(xch.slots[pr] + xch.rank), "l"(mine) : "memory");
            bool got_all = true;
            for (int pr = 0; pr < xch.world && got_all; pr++) {
                if (pr == xch.rank) continue;
                unsigned long long got;
                while (true) {
                    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(got) : "l"(xch.slots[xch.rank] + pr) : "memory");
                    if (int(unsigned(got >> 32) - epoch) >= 0) break;
                    if (clock64() - t0 > spin_limit) { got_all = false; break; }
                }
                if (got_all) g = fmaxf(g, __uint_as_float(unsigned(got & 0xffffffffu)));
            }
            atomicMax(&ws->amax_bits, got_all ? __float_as_uint(g) : kAmaxFailed);
            __threadfence();
            atomicAdd(&ws->arrived, 1u);
        }
        bool ok = true;
        while (*reinterpret_cast<volatile unsigned int*>(&ws->arrived) < target) {
            if (clock64() - t0 > 2 * spin_limit) { ok = false; break; }
        }
        __threadfence();
        const unsigned int bits = *reinterpret_cast<volatile unsigned int*>(&ws->amax_bits);
        if (bits == kAmaxFailed) ok = false;
        if (!ok && status) atomicExch(status, 4 /* timeout */);
        s_amax = ok ? __uint_as_float(bits) : -1.0f;
    }
    __syncthreads();
    return s_amax;
}

// Called by thread 0 of every block once it no longer needs the slot: the last block to leave restores
// the slot for the next call (off the critical path of the quantization itself).
__device__ __forceinline__ void grid_amax_depart(QuantWork* ws) {
    if (atomicAdd(&ws->departed, 1u) == gridDim.x - 1) {
        ws->amax_bits = 0u; ws->departed = 0u;
        __threadfence();
        ws->arrived = 0u;
    }
}

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Quantizes one 128 x 128 tile held in registers (thread layout of load_tile) and stores codes and scales.  s_sc: this
// iteration's 1 KB staging buffer for the tile's scale bytes.  RING: the calling CTA has a producer warp besides the
// Q_THREADS consumer threads, which synchronise among themselves on a named barrier.
template <class Arith, bool SCALE_2D, bool RING>
__device__ __forceinline__ void nv_quantize_store_tile(const uint4 (&v)[8], TileCoord tc, int warp, int lane, float sg_dec, float sg_enc,
                                                       uint8_t (&s_sc)[2][512], uint8_t* __restrict__ codes, int64_t ldc, uint8_t* __restrict__ sc,
                                                       int64_t ldsc, int sc_rowmajor, int M, int K, int k_chunks) {
    float am[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        float a = amax8(v[i]);
        am[i] = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 1));
    }
    if constexpr (SCALE_2D) {
        float a = am[0];
#pragma unroll
        for (int i = 1; i < 8; i++) a = fmaxf(a, am[i]);
        a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 16));
#pragma unroll
        for (int i = 0; i < 8; i++) am[i] = a;
    }
    const int kb_local = (lane & 15) >> 1;        // 16-element block within the 128-column tile
    const int col = tc.col0 + (lane & 15) * 8;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int r = warp * 16 + 2 * i + (lane >> 4);     // row within the tile
        const uint8_t s8 = (uint8_t)__nv_cvt_float_to_fp8(Arith::block_scale(am[i], sg_enc), __NV_SATFINITE, __NV_E4M3);
        if ((lane & 1) == 0) {
            if (sc_rowmajor) (&s_sc[0][0])[r * 8 + kb_local] = s8;                       // [row][8 blocks of the tile]
            else s_sc[kb_local >> 2][(r & 31) * 16 + (r >> 5) * 4 + (kb_local & 3)] = s8;   // 512-byte chunk layout
        }
        const float s_enc = Arith::block_enc(e4m3_to_float(s8), sg_dec);
        const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
        uint32_t packed = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            float2 f = bf16x2_to_f2(w[j]);
            f.x = Arith::scale_value(f.x, s_enc);
            f.y = Arith::scale_value(f.y, s_enc);
            packed |= uint32_t(__nv_cvt_float2_to_fp4x2(f, __NV_E2M1, cudaRoundNearest)) << (8 * j);
        }
        const int row = tc.row0 + r;
        if (row < M && col < K) *reinterpret_cast<uint32_t*>(codes + int64_t(row) * ldc + col / 2) = packed;
    }
    if constexpr (RING) asm volatile("bar.sync 1, %0;" ::"n"(Q_THREADS) : "memory");      // the consumer warps only
    else __syncthreads();
    if (sc_rowmajor) {
        // plain [M, K/16] scale rows (used where rows travel individually, e.g. MoE dispatch)
        const int r = threadIdx.x >> 1, half = threadIdx.x & 1;     // 4 scale bytes (64 columns) per thread
        if (tc.row0 + r < M && tc.col0 + half * 64 < K)
            *reinterpret_cast<uint32_t*>(sc + int64_t(tc.row0 + r) * ldsc + tc.col0 / 16 + half * 4) =
                reinterpret_cast<const uint32_t*>(&s_sc[0][0])[r * 2 + half];
    } else {
        const int c = threadIdx.x >> 7, word = threadIdx.x & 127;
        const int kc = tc.col0 / 64 + c;
        if (kc < k_chunks) {
            uint32_t* dst = reinterpret_cast<uint32_t*>(sc + (int64_t(tc.row0 / 128) * k_chunks + kc) * 512);
            dst[word] = reinterpret_cast<const uint32_t*>(&s_sc[c][0])[word];
        }
    }
}

// ------------------------------------------------------------------------------ NVFP4 -----
// Arith supplies:
//   static void global_scales(float amax, float& sg_dec, float& sg_enc)
//   static float block_scale(float amax16, float sg_enc)             value fed to the e4m3 conversion
//   static float block_enc(float s_local_dec, float sg_dec)          multiplier applied to the inputs
//   static float scale_value(float x, float s_enc)
// RESIDENT: the grid has one CTA per tile and the tile stays in registers between the amax pass and the
// quantization (one read of the input); otherwise the grid is persistent and the input is read twice.
template <class Arith, bool SCALE_2D, bool FUSED_AMAX, bool RESIDENT>
__global__ void __launch_bounds__(Q_THREADS)
nvfp4_quantize_kernel(const __nv_bfloat16* __restrict__ A, int64_t lda, uint8_t* __restrict__ codes, int64_t ldc,
                      uint8_t* __restrict__ sc, float* __restrict__ sg, const float* __restrict__ amax_in, QuantWork* ws,
                      int M, int K, int* status, int sc_rowmajor, int64_t ldsc, const QuantExchange xch, long long spin_limit) {
    __shared__ __align__(16) uint8_t s_sc[2][2][512];   // [double buffer][chunk][byte]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tiles_n = (K + QT_COLS - 1) / QT_COLS;
    const int tiles_m = (M + QT_ROWS - 1) / QT_ROWS;
    const int num_tiles = tiles_m * tiles_n;
    const int k_chunks = K / 64;

    // launched with programmatic stream serialization: everything above overlapped the previous kernel's tail
    pdl_wait();
    pdl_launch_dependents();
    if (xch.stamp != nullptr && blockIdx.x == 0) {
        const unsigned int epoch = xch.epoch_ptr ? *reinterpret_cast<const volatile unsigned int*>(xch.epoch_ptr) + 1u : xch.epoch;
        for (int i = threadIdx.x; i < xch.stamp_count; i += Q_THREADS) xch.stamp[i] = epoch;
    }
    float amax;
    uint4 v[8];
    if constexpr (FUSED_AMAX) {
        float local = 0.f;
        if constexpr (RESIDENT) {
            load_tile(A, lda, M, K, tile_coord(blockIdx.x, tiles_n), warp, lane, v);
#pragma unroll
            for (int i = 0; i < 8; i++) local = fmaxf(local, amax8(v[i]));
        } else {
            // two tiles (256 bytes per thread) in flight per iteration
            for (int tile = blockIdx.x; tile < num_tiles; tile += 2 * gridDim.x) {
                uint4 v2[8];
                const int tile2 = tile + gridDim.x;
                load_tile(A, lda, M, K, tile_coord(tile, tiles_n), warp, lane, v);
                if (tile2 < num_tiles) load_tile(A, lda, M, K, tile_coord(tile2, tiles_n), warp, lane, v2);
                else {
#pragma unroll
                    for (int i = 0; i < 8; i++) v2[i] = make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int i = 0; i < 8; i++) local = fmaxf(local, fmaxf(amax8(v[i]), amax8(v2[i])));
            }
        }
        amax = grid_amax_barrier(ws, local, status, xch, spin_limit);
        if (amax < 0.f) {
            if (threadIdx.x == 0) grid_amax_depart(ws);      // keep the slot usable for later calls
            return;
        }
    } else {
        amax = *amax_in;
    }
    float sg_dec, sg_enc;
    Arith::global_scales(amax, sg_dec, sg_enc);
    if (blockIdx.x == 0 && threadIdx.x == 0) *sg = sg_dec;

    int buf = 0;
    // walk the tiles in reverse: the tail of the amax pass is the part most likely still in L2
    for (int t = RESIDENT ? int(blockIdx.x) : num_tiles - 1 - int(blockIdx.x); t >= 0; t -= RESIDENT ? num_tiles : int(gridDim.x), buf ^= 1) {
        const TileCoord tc = tile_coord(t, tiles_n);
        if (!(RESIDENT && FUSED_AMAX)) load_tile(A, lda, M, K, tc, warp, lane, v);
        nv_quantize_store_tile<Arith, SCALE_2D, false>(v, tc, warp, lane, sg_dec, sg_enc, s_sc[buf], codes, ldc, sc, ldsc, sc_rowmajor, M, K, k_chunks);
        // the next iteration writes the other staging buffer; the one after that is fenced by the
        // __syncthreads() of the iteration in between
    }
    if constexpr (FUSED_AMAX) {
        if (threadIdx.x == 0) grid_amax_depart(ws);
    }
}


// ------------------------------------------------------------------------------ NVFP4, tile per CTA, TMA in and out -----
// Large tensors (two or more 128 x 128 tiles per SM, K % 128 == 0, chunked 1-D scales, fused amax): persistent CTAs of 128
// threads with one 32 KB tile buffer each, as many as are resident at once (six per SM).  A tile arrives as two TMA boxes of
// 128 rows x 128 bytes (128-byte swizzle); thread t owns row t.  Pass 1 takes the amax of the CTA's tiles; after the grid
// barrier pass 2 walks them in reverse, so the tile that is still in shared memory needs no second load and the ones before it
// are the part of the input most likely still in L2.  The codes of a tile (128 rows x 64 bytes) go into the front of the same
// buffer (64-byte swizzle: a quarter-warp's 16-byte stores cover all banks) and leave as one TMA store, the two 512-byte scale
// chunks as coalesced stores.  No load or store instruction touches the tensor itself, and six independent CTAs per SM keep
// a bulk copy in flight while the others convert.
constexpr int QTT_THREADS = 128;
constexpr int QTT_SMEM = 2 * 128 * 128 + 1024;

__device__ __forceinline__ void qtt_load_row(uint32_t base, int t, uint4 (&v)[16]) {
    const uint32_t row_base = base + uint32_t(t) * 128u, sw = uint32_t(t & 7);
#pragma unroll
    for (int c = 0; c < 16; c++) {
        const uint32_t a = row_base + uint32_t(c >> 3) * (128u * 128u) + ((uint32_t(c & 7) ^ sw) << 4);
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v[c].x), "=r"(v[c].y), "=r"(v[c].z), "=r"(v[c].w) : "r"(a));
    }
}

template <class Arith>
__global__ void __launch_bounds__(QTT_THREADS, 6)
nvfp4_quantize_tile_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmC, uint8_t* __restrict__ sc,
                           float* __restrict__ sg, QuantWork* ws, int M, int K, int* status, const QuantExchange xch, long long spin_limit,
                           long long wait_limit) {
    extern __shared__ uint8_t qtt_smem_raw[];
    __shared__ __align__(8) uint64_t bar;
    __shared__ __align__(16) uint32_t s_sc[2][128];
    __shared__ int s_abort;
    const uint32_t base = (smem_u32(qtt_smem_raw) + 1023u) & ~1023u;
    const int t = threadIdx.x;
    const int tiles_n = K / 128, tiles_m = (M + 127) / 128;
    const int num_tiles = tiles_m * tiles_n;
    const int k_chunks = K / 64;
    const int n_mine = (num_tiles - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x);      // the grid never exceeds the tiles
    if (t == 0) {
        s_abort = 0;
        mbar_init(smem_u32(&bar), 1);
        fence_mbar_init();
    }
    __syncthreads();
    pdl_wait();
    pdl_launch_dependents();
    if (xch.stamp != nullptr && blockIdx.x == 0) {
        const unsigned int epoch = xch.epoch_ptr ? *reinterpret_cast<const volatile unsigned int*>(xch.epoch_ptr) + 1u : xch.epoch;
        for (int i = t; i < xch.stamp_count; i += QTT_THREADS) xch.stamp[i] = epoch;
    }
    WaitCtx wc{&s_abort, status, wait_limit};
    uint32_t phase = 0;
    auto issue = [&](int tile) {          // thread 0 only
        const int row0 = (tile / tiles_n) * 128, col0 = (tile % tiles_n) * 128;
        mbar_arrive_expect_tx(smem_u32(&bar), 2 * 128 * 128);
        tma_load_2d(base, &tmA, smem_u32(&bar), col0, row0);
        tma_load_2d(base + 128 * 128, &tmA, smem_u32(&bar), col0 + 64, row0);
    };
    // every thread of the CTA leaves a loop at the same iteration: the outcome of a wait is agreed on before it is acted on
    auto arrived = [&]() -> bool {
        const bool ok = mbar_wait(wc, smem_u32(&bar), phase);
        const bool all = __syncthreads_and(ok ? 1 : 0) != 0;
        if (!all) {
            // giving up: the copy that was issued must still land before this CTA may exit (bounded, status already set)
            if (t == 0) {
                const long long t0 = clock64();
                while (!mbar_try_wait_sleep(smem_u32(&bar), phase, 20000u))
                    if (clock64() - t0 > wait_limit) break;
            }
            __syncthreads();
        }
        phase ^= 1u;
        return all;
    };

    // ---- pass 1: the amax of this CTA's tiles ----
    uint4 v[16];
    uint32_t m2 = 0u;                      // running maximum of |x| as packed bf16 pairs
    bool ok = true;
    for (int i = 0; i < n_mine && ok; i++) {
        if (t == 0) issue(int(blockIdx.x) + i * int(gridDim.x));
        ok = arrived();
        if (!ok) break;
        qtt_load_row(base, t, v);
#pragma unroll
        for (int c = 0; c < 16; c++) m2 = habs2_max(m2, habs2_max(habs2_max(v[c].x, v[c].y), habs2_max(v[c].z, v[c].w)));
        if (i + 1 < n_mine) __syncthreads();          // every row is in registers before the next tile overwrites the buffer
    }
    __nv_bfloat162 mm = *reinterpret_cast<__nv_bfloat162*>(&m2);
    const float local = __bfloat162float(__hmax(mm.x, mm.y));
    const float amax = grid_amax_barrier<QTT_THREADS>(ws, local, status, xch, spin_limit);       // a CTA whose load failed still takes part
    if (amax < 0.f || !ok) {
        if (t == 0) grid_amax_depart(ws);
        return;
    }
    float sg_dec, sg_enc;
    Arith::global_scales(amax, sg_dec, sg_enc);
    if (blockIdx.x == 0 && t == 0) *sg = sg_dec;

    // ---- pass 2: quantize, last tile first (its rows are still in v) ----
    const uint32_t row_out = base + uint32_t(t) * 64u, sw_out = uint32_t(t >> 1) & 3u;
    for (int i = n_mine - 1; i >= 0; i--) {
        const int tile = int(blockIdx.x) + i * int(gridDim.x);
        const int row0 = (tile / tiles_n) * 128, col0 = (tile % tiles_n) * 128;
        if (i != n_mine - 1) {
            if (t == 0) issue(tile);
            if (!arrived()) break;
            qtt_load_row(base, t, v);
        }
        __syncthreads();                   // every row is in registers: the front of the buffer becomes the output tile
        uint32_t scw[2] = {0u, 0u};
#pragma unroll
        for (int b = 0; b < 8; b++) {       // 16-value block b of this thread's row: chunks 2b and 2b + 1
            const float a16 = fmaxf(amax8(v[2 * b]), amax8(v[2 * b + 1]));
            const uint8_t s8 = (uint8_t)__nv_cvt_float_to_fp8(Arith::block_scale(a16, sg_enc), __NV_SATFINITE, __NV_E4M3);
            scw[b >> 2] |= uint32_t(s8) << (8 * (b & 3));
            const float s_enc = Arith::block_enc(e4m3_to_float(s8), sg_dec);
            const uint32_t w[8] = {v[2 * b].x, v[2 * b].y, v[2 * b].z, v[2 * b].w, v[2 * b + 1].x, v[2 * b + 1].y, v[2 * b + 1].z, v[2 * b + 1].w};
            uint32_t packed[2] = {0u, 0u};
#pragma unroll
            for (int j = 0; j < 8; j++) {
                float2 f = bf16x2_to_f2(w[j]);
                f.x = Arith::scale_value(f.x, s_enc);
                f.y = Arith::scale_value(f.y, s_enc);
                packed[j >> 2] |= uint32_t(__nv_cvt_float2_to_fp4x2(f, __NV_E2M1, cudaRoundNearest)) << (8 * (j & 3));
            }
            // 8 bytes of codes at byte 8 b of the 64-byte output row: half of 16-byte chunk b / 2
            const uint32_t a = row_out + (((uint32_t(b) >> 1) ^ sw_out) << 4) + (uint32_t(b) & 1u) * 8u;
            asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(a), "r"(packed[0]), "r"(packed[1]) : "memory");
        }
        // rows past M were loaded as zeros: their amax, scale byte and codes are 0, like the register-tile kernel writes them
        s_sc[0][(t & 31) * 4 + (t >> 5)] = scw[0];
        s_sc[1][(t & 31) * 4 + (t >> 5)] = scw[1];
        fence_proxy_async();
        __syncthreads();
#pragma unroll
        for (int c = 0; c < 2; c++) {
            const int kc = col0 / 64 + c;
            if (kc < k_chunks) reinterpret_cast<uint32_t*>(sc + (int64_t(row0 / 128) * k_chunks + kc) * 512)[t] = s_sc[c][t];
        }
        if (t == 0) {
            tma_store_2d(&tmC, base, col0 / 2, row0);         // rows past M are clipped
            tma_store_commit();
            tma_store_wait_read<0>();                         // before the next load (issued by this thread) overwrites the staging tile
        }
    }
    if (t == 0) grid_amax_depart(ws);
}

} // namespace tkb

// ------------------------------------------------------------------------------ host ------
namespace tkb {


template <class Arith, bool S2D, bool FUSED, bool RESIDENT>
inline cudaError_t launch_nvfp4_quantize_t(const NvQuantArgs& a) {
    auto kern = nvfp4_quantize_kernel<Arith, S2D, FUSED, RESIDENT>;
    const int tiles = ((a.M + QT_ROWS - 1) / QT_ROWS) * ((a.K + QT_COLS - 1) / QT_COLS);
    static int blocks_per_sm = 0;   // same for every instantiation's first call; cheap to query once each
    if (blocks_per_sm == 0) {
        int b = 0;
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&b, kern, Q_THREADS, 0);
        if (e != cudaSuccess) return e;
        blocks_per_sm = b < 1 ? 1 : (b > 4 ? 4 : b);
    }
    static const int bps_env = getenv("TKB_NVQ_BLOCKS_PER_SM") ? atoi(getenv("TKB_NVQ_BLOCKS_PER_SM")) : 0;     // tuning aid; must not exceed what is resident
    int grid = a.sm_count * (bps_env > 0 && bps_env <= blocks_per_sm ? bps_env : blocks_per_sm);
    if (grid > tiles) grid = tiles;
    if (grid < 1) grid = 1;
    if (RESIDENT) {
        if (tiles > grid) return cudaErrorInvalidConfiguration;   // caller checks nvfp4_quantize_resident_ok first
        grid = tiles;
    }
    const __nv_bfloat16* A = static_cast<const __nv_bfloat16*>(a.A);
    uint8_t* codes = static_cast<uint8_t*>(a.codes);
    uint8_t* sc = static_cast<uint8_t*>(a.sc);
    int64_t lda = a.lda, ldc = a.ldc;
    float* sg = a.sg; const float* amax_in = a.amax_in; QuantWork* ws = a.ws; int M = a.M, K = a.K; int* status = a.status;
    int sc_rowmajor = a.sc_rowmajor;
    int64_t ldsc = a.ldsc;
    const QuantExchange xch = a.xch;
    long long spin_limit = a.spin_limit;
    // Programmatic stream serialization: the kernel may be scheduled while its predecessor in the stream drains;
    // it executes griddepcontrol.wait before touching global memory.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(Q_THREADS); cfg.dynamicSmemBytes = 0; cfg.stream = a.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, A, lda, codes, ldc, sc, sg, amax_in, ws, M, K, status, sc_rowmajor, ldsc, xch, spin_limit);
}

// One tile per CTA with the whole grid resident (needed by the grid barrier)?
inline bool nvfp4_quantize_resident_ok(const NvQuantArgs& a) {
    const long long tiles = (long long)((a.M + QT_ROWS - 1) / QT_ROWS) * ((a.K + QT_COLS - 1) / QT_COLS);
    return tiles <= (long long)a.sm_count * 2;
}


// ------------------------------------------------------------------------------ NVFP4, at most 16 rows -----
// Activations of a decode step (M <= 16): the whole tensor is a few hundred KB, so the general kernel's persistent grid
// and global-memory grid barrier cost more than the work.  Here one thread-block cluster of ceil(K / 1024) <= 8 CTAs
// covers the tensor: CTA c owns columns [1024 c, 1024 c + 1024), warp w of it the 16 x 128 tile at column 128 w, held in
// registers for both passes (one read of the input).  The per-tensor amax crosses the cluster through distributed
// shared memory and one cluster barrier; no global scratch, no atomics.  Same arithmetic, same output layout (rows of
// the single 128-row scale block past M are written as zeros).
constexpr int QS_MAX_ROWS = 16, QS_COLS_PER_CTA = 1024, QS_MAX_CTAS = 8;

template <class Arith>
__global__ void __launch_bounds__(Q_THREADS)
nvfp4_quantize_skinny_kernel(const __nv_bfloat16* __restrict__ A, int64_t lda, uint8_t* __restrict__ codes, int64_t ldc,
                             uint8_t* __restrict__ sc, float* __restrict__ sg, int M, int K) {
    __shared__ __align__(16) uint8_t s_chunks[QS_COLS_PER_CTA / 64][512];     // this CTA's 16 scale chunks, as stored
    __shared__ float s_warp[Q_THREADS / 32];
    __shared__ float s_peer[QS_MAX_CTAS];                                     // written by every CTA of the cluster
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t cta, ncta;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(cta));
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(ncta));
    pdl_wait();
    pdl_launch_dependents();
    for (int i = threadIdx.x; i < int(sizeof(s_chunks) / 16); i += Q_THREADS) reinterpret_cast<uint4*>(&s_chunks[0][0])[i] = make_uint4(0, 0, 0, 0);
    const TileCoord tc{0, int(cta) * QS_COLS_PER_CTA + warp * QT_COLS};
    uint4 v[8];
    load_tile(A, lda, M, K, tc, 0, lane, v);          // rows 2 i + (lane >> 4), columns tc.col0 + 8 (lane & 15)
    float local = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) local = fmaxf(local, amax8(v[i]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) local = fmaxf(local, __shfl_xor_sync(0xffffffffu, local, o));
    if (lane == 0) s_warp[warp] = local;
    __syncthreads();
    if (threadIdx.x < ncta) {          // thread t hands this CTA's maximum to CTA t of the cluster
        float m = s_warp[0];
#pragma unroll
        for (int w = 1; w < Q_THREADS / 32; w++) m = fmaxf(m, s_warp[w]);
        const uint32_t local_addr = static_cast<uint32_t>(__cvta_generic_to_shared(&s_peer[cta]));
        uint32_t remote;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(uint32_t(threadIdx.x)));
        asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(m) : "memory");
    }
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    float amax = 0.f;
    for (uint32_t i = 0; i < ncta; i++) amax = fmaxf(amax, s_peer[i]);
    float sg_dec, sg_enc;
    Arith::global_scales(amax, sg_dec, sg_enc);
    if (cta == 0 && threadIdx.x == 0) *sg = sg_dec;

    const int kb_local = (lane & 15) >> 1;            // 16-element block within the warp's 128 columns
    const int col = tc.col0 + (lane & 15) * 8;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int r = 2 * i + (lane >> 4);
        float a = amax8(v[i]);
        a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 1));
        const uint8_t s8 = (uint8_t)__nv_cvt_float_to_fp8(Arith::block_scale(a, sg_enc), __NV_SATFINITE, __NV_E4M3);
        if ((lane & 1) == 0) s_chunks[warp * 2 + (kb_local >> 2)][r * 16 + (kb_local & 3)] = s8;        // rows < 32: byte r * 16 + k-block % 4
        const float s_enc = Arith::block_enc(e4m3_to_float(s8), sg_dec);
        const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
        uint32_t packed = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            float2 f = bf16x2_to_f2(w[j]);
            f.x = Arith::scale_value(f.x, s_enc);
            f.y = Arith::scale_value(f.y, s_enc);
            packed |= uint32_t(__nv_cvt_float2_to_fp4x2(f, __NV_E2M1, cudaRoundNearest)) << (8 * j);
        }
        if (r < M && col < K) *reinterpret_cast<uint32_t*>(codes + int64_t(r) * ldc + col / 2) = packed;
    }
    __syncthreads();
    const int k_chunks = K / 64;
    for (int i = threadIdx.x; i < int(sizeof(s_chunks) / 16); i += Q_THREADS) {
        const int kc = int(cta) * (QS_COLS_PER_CTA / 64) + i / 32;
        if (kc < k_chunks) reinterpret_cast<uint4*>(sc + int64_t(kc) * 512)[i % 32] = reinterpret_cast<const uint4*>(&s_chunks[0][0])[i];
    }
}

template <class Arith>
inline cudaError_t launch_nvfp4_quantize_skinny(const NvQuantArgs& a) {
    auto kern = nvfp4_quantize_skinny_kernel<Arith>;
    const int ctas = (a.K + QS_COLS_PER_CTA - 1) / QS_COLS_PER_CTA;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas); cfg.blockDim = dim3(Q_THREADS); cfg.dynamicSmemBytes = 0; cfg.stream = a.stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = ctas; attr[1].val.clusterDim.y = 1; attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<const __nv_bfloat16*>(a.A), a.lda, static_cast<uint8_t*>(a.codes), a.ldc,
                              static_cast<uint8_t*>(a.sc), a.sg, a.M, a.K);
}

// The cluster kernel covers: fused amax, 1-D scales, operand layout, one GPU, M <= 16, K <= 8192.
inline bool nvfp4_quantize_skinny_ok(const NvQuantArgs& a) {
    return a.amax_in == nullptr && !a.scale_2d && !a.sc_rowmajor && a.xch.world <= 1 && a.xch.stamp == nullptr && a.M <= QS_MAX_ROWS &&
           a.K <= QS_COLS_PER_CTA * QS_MAX_CTAS;
}

template <class Arith>
inline cudaError_t launch_nvfp4_quantize_tiles(const NvQuantArgs& a) {
    auto kern = nvfp4_quantize_tile_kernel<Arith>;
    static int blocks_per_sm = 0;
    if (blocks_per_sm == 0) {
        static_assert(QTT_SMEM <= 48 * 1024, "no opt-in needed for the dynamic shared memory");
        int b = 0;
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&b, kern, QTT_THREADS, QTT_SMEM);
        if (e != cudaSuccess) return e;
        blocks_per_sm = b < 1 ? 1 : b;
    }
    const int tiles = ((a.M + 127) / 128) * (a.K / 128);
    static const int bps_env = getenv("TKB_NVQ_TILE_BLOCKS_PER_SM") ? atoi(getenv("TKB_NVQ_TILE_BLOCKS_PER_SM")) : 0;     // tuning aid; never above what is resident
    int grid = a.sm_count * (bps_env > 0 && bps_env <= blocks_per_sm ? bps_env : blocks_per_sm);      // all resident at once: the grid barrier needs it
    if (grid > tiles) grid = tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(QTT_THREADS); cfg.dynamicSmemBytes = QTT_SMEM; cfg.stream = a.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, a.tmA, a.tmC, static_cast<uint8_t*>(a.sc), a.sg, a.ws, a.M, a.K, a.status, a.xch, a.spin_limit, a.wait_limit);
}

template <class Arith>
inline cudaError_t launch_nvfp4_quantize(const NvQuantArgs& a) {
    if (nvfp4_quantize_skinny_ok(a)) return launch_nvfp4_quantize_skinny<Arith>(a);
    if (a.use_tiles && a.amax_in == nullptr && !a.scale_2d && !a.sc_rowmajor && !nvfp4_quantize_resident_ok(a)) return launch_nvfp4_quantize_tiles<Arith>(a);
    const bool fused = a.amax_in == nullptr;
    const bool res = fused && nvfp4_quantize_resident_ok(a);
    if (a.scale_2d) {
        if (res) return launch_nvfp4_quantize_t<Arith, true, true, true>(a);
        return fused ? launch_nvfp4_quantize_t<Arith, true, true, false>(a) : launch_nvfp4_quantize_t<Arith, true, false, false>(a);
    }
    if (res) return launch_nvfp4_quantize_t<Arith, false, true, true>(a);
    return fused ? launch_nvfp4_quantize_t<Arith, false, true, false>(a) : launch_nvfp4_quantize_t<Arith, false, false, false>(a);
}

} // namespace tkb
