// Block-scaled and dense GEMMs for sm_100a: D[M,N] (bf16) = A[M,K] * B[N,K]^T, fp32 accumulation
// in tensor memory.  One kernel template covers the three operand formats of the path:
//   KIND_NVFP4 : e2m1 codes (2 per byte), one e4m3 scale per 16 K-elements, fp32 per-tensor scales
//                (replaces nvfp4_gemm::kernel, kernels/gemm/nvfp4_b200/nvfp4_b200_gemm.cu:88-307)
//   KIND_MXFP8 : e4m3 codes, one ue8m0 scale per 32 K-elements
//                (replaces mxfp8_gemm::kernel, kernels/gemm/mxfp8_b200/mxfp8_b200_gemm.cu:83-292)
//   KIND_BF16  : dense control (replaces kernel<C>, kernels/gemm/bf16_b200/bf16_b200_gemm.cu:61-253)
//   KIND_FP8   : dense e4m3 (replaces kernels/gemm/fp8_b200/fp8_b200_gemm.cu, the bf16 kernel with 8-bit operands)
//
// Design (one CTA per SM, persistent over output tiles):
//   * A stage of the operand ring always holds exactly 128 bytes of K per row (64 bf16, 128 e4m3,
//     256 e2m1), i.e. one 128-byte-swizzle panel: one TMA box per operand per stage and four
//     tcgen05.mma per stage (32 bytes of K each) for every format.
//   * CTAS == 2: two CTAs of a cluster form one 256 x BN tile (cta_group::2).  Each CTA loads its own
//     128 rows of A, its half of the B rows, its A scales and ALL of the tile's B scales.  Loads
//     are plain (non-multicast) TMA copies whose completion bytes are credited to the leader CTA's
//     "full" barrier; the leader's MMA thread releases a stage in both CTAs with one commit.
//   * warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner, warps 2.. = epilogue.
//   * Scale factors travel shared memory -> tensor memory with tcgen05.cp right before the MMAs
//     that use them, into one of four rotating slots next to the accumulator.
//   * Two accumulators where tensor memory has room for them next to the scale slots (the dense kinds and
//     every kind with the 128-wide N tile): the epilogue of a tile overlaps the MMAs of the next.  The
//     block-scaled kinds with the 256-wide tile have one (256 fp32 columns + scale slots leave no room):
//     the epilogue first drains it into registers as packed bf16, hands TMEM back to the MMA warp,
//     and only then writes D, so the stores overlap the next tile's main loop.  Each epilogue warp
//     owns a private 4 KB staging box (32 rows x 64 columns, 128-byte swizzle) and issues its own
//     TMA stores: whole 128-byte lines reach L2, no cross-warp synchronisation, and rows / columns
//     past M / N are clipped by the TMA unit.
//   * Every mbarrier wait is bounded (ptx.cuh); on a timeout the kernel records the status, leaves
//     its loops, joins the final cluster barrier, frees TMEM and returns.
#include <atomic>
#include <cstdlib>
#include <cuda_fp8.h>
#include <cuda_fp4.h>
#include "ptx.cuh"
#include "internal.h"
#include "ag_schedule.h"

namespace tkb {

template <int KIND, int CTAS, int BN, int MH = 1>
struct GemmCfg {
    static_assert(CTAS == 1 || CTAS == 2, "");
    static_assert(BN == 128 || BN == 256, "");
    // MH = 2 (dense kinds, CTA pairs, N tile 256): every CTA carries TWO 128-row halves of A per stage against the same B rows,
    // i.e. a 512 x 256 cluster tile with one accumulator per half: a third more FLOPs per byte that crosses from L2 into
    // shared memory than the 256 x 256 tile, which is what bounds the dense kernels
    static_assert(MH == 1 || (MH == 2 && CTAS == 2 && BN == 256 && (KIND == KIND_BF16 || KIND == KIND_FP8)), "");
    static constexpr int BM = 128 * CTAS * MH;            // rows of D per cluster tile
    static constexpr int MMA_M = 128 * CTAS;              // rows of one MMA instruction (per CTA pair)
    static constexpr int BN_CTA = BN / CTAS;              // rows of B each CTA loads
    static constexpr int KB = KIND == KIND_BF16 ? 64 : (KIND == KIND_NVFP4 ? 256 : 128);   // K elements per stage (128 bytes)
    static constexpr int A_BYTES = MH * 128 * 128;
    static constexpr int B_BYTES = BN_CTA * 128;
    static constexpr int SF_CHUNKS = KIND == KIND_NVFP4 ? 4 : (KIND == KIND_MXFP8 ? 1 : 0);  // 512-byte chunks per 128 rows per stage
    static constexpr int SFA_BYTES = SF_CHUNKS * 512;
    static constexpr int SFB_BYTES = SF_CHUNKS * 512 * (BN / 128);
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
    static constexpr int EPI_WARPS = BN == 256 ? 8 : 4;
    static constexpr int EPI_WARP_BYTES = 32 * 128;                  // one 32-row x 64-column bf16 store box per warp
    static constexpr int EPI_BYTES = EPI_WARPS * EPI_WARP_BYTES;
    static constexpr int SMEM_BUDGET = 227 * 1024 - 2048 - EPI_BYTES;
    static constexpr int STAGES_RAW = SMEM_BUDGET / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 2048;   // + alignment slack (base and staging area)
    static constexpr int THREADS = (2 + EPI_WARPS) * 32;
    static constexpr int COLS_PER_EPI_WARP = BN / (EPI_WARPS / 4);   // 128
    // tensor memory: accumulator at column 0, then rotating scale slots
    static constexpr int SFA_COLS = SF_CHUNKS * 4;                   // per stage
    static constexpr int SFB_COLS = SF_CHUNKS * 4 * (BN / 128);
    static constexpr int SF_SLOTS = 4;
    static constexpr int TMEM_COLS = 512;
    // two accumulators where they fit next to the scale slots (dense kinds, or N tile 128): the epilogue of tile i then overlaps
    // the MMAs of tile i + 1; otherwise one
    static constexpr int ACC_COLS = MH * BN;              // columns of one accumulator set (half h at column h * BN)
    static constexpr int ACC_BUFS = (2 * ACC_COLS + SF_SLOTS * (SFA_COLS + SFB_COLS) <= TMEM_COLS) ? 2 : 1;
    static constexpr int SF_BASE = ACC_BUFS * ACC_COLS;
    static_assert(ACC_BUFS * ACC_COLS + SF_SLOTS * (SFA_COLS + SFB_COLS) <= TMEM_COLS, "tensor memory overflow");
    static_assert(STAGES >= 3, "not enough pipeline stages");
    static constexpr uint32_t TX_BYTES = CTAS * STAGE_BYTES;
};

struct GemmParams {
    const float* sgA; const float* sgB;
    int M, N, K;
    int group;                  // row blocks that share a sweep over the columns
    int rot;                    // row block at which the tile order starts (reduce-scatter mode)
    int* status;
    unsigned long long* prof;   // optional: per-CTA wait-cycle counters (see tkb_gemm_set_profile_buffer)
    long long wait_limit;       // clock cycles any wait of the kernel may last
    // quantizing epilogue (MODE_QUANT): the bf16 result is quantized to NVFP4 before it leaves the SM
    uint8_t* q_codes; uint8_t* q_sc; float* q_sg; const float* q_amax; int q_arith;
    // reduce-scatter epilogue (MODE_RS): tensor maps (device memory) of every rank's output rows, rows per rank
    const CUtensorMap* rs_maps; int rs_rows;
};

// NVFP4 quantization of one 16-value block held as 8 packed bf16 pairs, with the IEEE arithmetic of the standalone
// quantizer (quantize.cu: ArithSpec / ArithKernelIeee): returns the e4m3 scale byte, `codes` receives 8 bytes.
__device__ __forceinline__ uint8_t quant_block16(const uint32_t (&w)[8], float sg_dec, float sg_enc, uint2& codes) {
    uint32_t m = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        __nv_bfloat162 a = __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
        __nv_bfloat162 b = __hmax2(a, *reinterpret_cast<__nv_bfloat162*>(&m));
        m = *reinterpret_cast<uint32_t*>(&b);
    }
    const __nv_bfloat162 mm = *reinterpret_cast<__nv_bfloat162*>(&m);
    const float amax16 = __bfloat162float(__hmax(mm.x, mm.y));
    const uint8_t s8 = (uint8_t)__nv_cvt_float_to_fp8(__fmul_rn(__fdiv_rn(amax16, 6.0f), sg_enc), __NV_SATFINITE, __NV_E4M3);
    const __half_raw hr = __nv_cvt_fp8_to_halfraw(s8, __NV_E4M3);
    const float s_local = __half2float(*reinterpret_cast<const __half*>(&hr));
    const float s_enc = __frcp_rn(fmaxf(__fmul_rn(s_local, sg_dec), 0.000000000001f));
    uint32_t out[2] = {0u, 0u};
#pragma unroll
    for (int i = 0; i < 8; i++) {
        float2 f = make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
        f.x = __fmul_rn(f.x, s_enc);
        f.y = __fmul_rn(f.y, s_enc);
        out[i >> 2] |= uint32_t(__nv_cvt_float2_to_fp4x2(f, __NV_E2M1, cudaRoundNearest)) << (8 * (i & 3));
    }
    codes = make_uint2(out[0], out[1]);
    return s8;
}

// All-gather mode (tensor-parallel GEMM): the A operand is row-sharded over `world` GPUs.  Every rank
// keeps a full-size buffer for the gathered codes and scales and quantizes its own shard into its own
// slice.  That slice reaches every peer's buffers over NVLink (plain loads and stores, no multicast) in one
// of three ways: two extra "push warps" in every CTA of this kernel, `comm_ctas` CTAs of this kernel set
// aside for it, or copy engines driven by the host (the kernel then only waits on the arrival flags).  The
// CTAs multiply meanwhile, own rows first, then the other shards in the order in which they arrive.

// tile index -> (row block, column block).  `group` row-blocks share a sweep over the columns (L2
// reuse); `rot` rotates the row-block order (all-gather mode starts with the rank's own rows).
__device__ __forceinline__ void tile_to_block(int tile, int tiles_m, int tiles_n, int group, int rot, int& m_blk, int& n_blk) {
    const int per_group = group * tiles_n;
    const int g = tile / per_group, in_g = tile % per_group;
    const int first_m = g * group;
    const int gsz = min(group, tiles_m - first_m);
    m_blk = first_m + in_g % gsz + rot;
    if (m_blk >= tiles_m) m_blk -= tiles_m;
    n_blk = in_g / gsz;
}

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu_u32(unsigned int* p, unsigned int v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bounded spin until a global epoch flag has reached `value` (epochs only grow).  False on timeout / abort.
__device__ __forceinline__ bool flag_wait(const WaitCtx& w, const unsigned int* flag, unsigned int value) {
    if (int(ld_acquire_sys(flag) - value) >= 0) return true;
    const long long t0 = clock64();
    while (int(ld_acquire_sys(flag) - value) < 0) {
        if (*w.abort_flag) return false;
        if (clock64() - t0 > w.limit) {
            *w.abort_flag = 1;
            if (w.status) atomicExch(w.status, (int)TKB_DEV_TIMEOUT);
            return false;
        }
        __nanosleep(64);
    }
    return true;
}
// 1-D bulk copies (16-byte aligned, size a multiple of 16): global (possibly a peer GPU) -> shared, shared -> global
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 ::"l"(reinterpret_cast<uint64_t>(dst)), "r"(src), "r"(bytes) : "memory");
}

// One comm CTA: PUSHES its share of this rank's quantized rows into the peers' buffers with plain loads (local) and
// stores (NVLink, posted).  The load/store units keep far more remote writes in flight per SM than the bulk-copy engine
// does (measured here: about 11 GB/s per CTA with 16 KB bulk stores to a peer), so a handful of CTAs can fill the links;
// a pull over NVLink would be limited per SM by the read round trip.
//   * A unit is one 64-row part of a 256-row block for one destination: the codes of those rows (contiguous) and
//     a quarter of the block's scale bytes.  Destinations are served in the order in which they will consume this
//     rank's rows (rank-1 first), four at a time, and the units are dealt round-robin to the comm CTAs, so
//     neighbouring CTAs write to different peers (ag_schedule.h).
//   * Warps 1.. copy (16 bytes per lane, UNROLL loads in flight per lane); warp 0 publishes: after the CTA barrier
//     that ends a unit, its lane 0 makes the unit's stores visible system-wide (fence) and stores the epoch into the
//     destination's `arrived` array while the other warps already copy the next unit.
//   * With peer_done set, the first store to a destination waits until that rank's kernel of epoch-2 (the last
//     reader of the buffer set being overwritten) has finished.
// prof (optional, 8 counters of this CTA, written by thread 0): [0] total cycles, [1] waiting for done flags,
// [2] fence + flag store.
__device__ __forceinline__ uint4 ld_nc_v4(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
template <int UNROLL = 16>
__device__ __forceinline__ void ag_copy_span(const uint8_t* src, uint8_t* dst, uint32_t bytes, int t, int nthr) {
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    const uint32_t n = bytes / 16;
    for (uint32_t base = 0; base < n; base += uint32_t(nthr) * UNROLL) {
        uint4 v[UNROLL];
#pragma unroll
        for (int i = 0; i < UNROLL; i++) {
            const uint32_t idx = base + uint32_t(i * nthr + t);
            if (idx < n) v[i] = ld_nc_v4(s4 + idx);
        }
#pragma unroll
        for (int i = 0; i < UNROLL; i++) {
            const uint32_t idx = base + uint32_t(i * nthr + t);
            if (idx < n) d4[idx] = v[i];
        }
    }
}
__device__ void ag_push(const AgParams& ag, int comm_idx, int k_bytes, int sc_bytes_per_mblock, const WaitCtx& wc, unsigned long long* prof) {
    const AgGeometry geo{ag.rank, ag.world, ag.blocks_per_rank, k_bytes, sc_bytes_per_mblock, ag.parts, kAgFanOut};
    const int units = ag_units(geo);
    const unsigned int* done = ag.peer_done[ag.rank];
    const int tid = threadIdx.x, nthr = int(blockDim.x) - 32;
    long long t_done = 0, t_pub = 0;
    const long long t_begin = clock64();
    int checked_dst = -1;
    for (int u = comm_idx; u < units; u += ag.comm_ctas) {
        // whole spans as single pieces: the cursor arithmetic is the one the host-side enumeration checks
        const AgPiece codes = ag_piece(geo, AgCursor{u, 0, 0u}, 0xffffffffu);
        const AgPiece scales = ag_piece(geo, AgCursor{u, 1, 0u}, 0xffffffffu);
        if (codes.dst_rank != checked_dst) {                 // uniform over the CTA
            if (tid == 0 && done != nullptr && ag.epoch > 2u) {
                const long long t0 = clock64();
                flag_wait(wc, done + codes.dst_rank, ag.epoch - 2u);      // on timeout: abort flag + status, read below
                t_done += clock64() - t0;
            }
            __syncthreads();
            if (*wc.abort_flag) break;                        // every thread reads it after the same barrier
            checked_dst = codes.dst_rank;
        }
        if (tid >= 32) {
            ag_copy_span(ag.codes + codes.off, const_cast<uint8_t*>(ag.peer_codes[codes.dst_rank]) + codes.off, codes.bytes, tid - 32, nthr);
            ag_copy_span(ag.scales + scales.off, const_cast<uint8_t*>(ag.peer_scales[scales.dst_rank]) + scales.off, scales.bytes, tid - 32, nthr);
        }
        __syncthreads();                                      // the unit's stores have been issued by every copy warp
        if (tid == 0) {
            const long long t0 = clock64();
            __threadfence_system();                           // cumulative over the stores ordered before the barrier
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(ag.peer_arrived[codes.dst_rank] + codes.flag), "r"(ag.epoch) : "memory");
            t_pub += clock64() - t0;
        }
    }
    if (prof && tid == 0) { prof[0] = clock64() - t_begin; prof[1] = t_done; prof[2] = t_pub; prof[3] = 0; prof[4] = 0; }
}

// The same push spread over EVERY CTA of the kernel: two extra warps per CTA (threads t = 0..63 of them) move units
// cta, cta + n_ctas, ... while the CTA's other warps multiply.  What limits SM-issued stores to a peer is a per-SM bound
// (about 10 GB/s, whether 2 or 8 warps issue them and whether they are plain or bulk stores), so the way to fill the links
// is to use all the SMs a little instead of a few SMs entirely, and no SM is taken from the GEMM.  Units are 16-row parts
// (ag.parts = 16) in the same consumption order as above, four destinations at a time.  No done-flag
// wait: the caller's amax exchange orders the steps (see tkb_ag_linear_nvfp4).
// Rolling copy for the push warps: U loads stay in flight per thread all the time (a register is reloaded right after its
// store has been issued) instead of alternating between a round of loads and a round of stores.
template <int U>
__device__ __forceinline__ void ag_copy_rolling(const uint8_t* src, uint8_t* dst, uint32_t bytes, int t, int nthr) {
    const uint4* s4 = reinterpret_cast<const uint4*>(src) + t;
    uint4* d4 = reinterpret_cast<uint4*>(dst) + t;
    const int n = (int(bytes / 16) - t + nthr - 1) / nthr;          // 16-byte pieces of this thread: t, t + nthr, ...
    uint4 v[U];
#pragma unroll
    for (int i = 0; i < U; i++)
        if (i < n) v[i] = ld_nc_v4(s4 + size_t(i) * nthr);
    for (int base = 0; base < n; base += U) {
#pragma unroll
        for (int i = 0; i < U; i++) {
            const int k = base + i;
            if (k < n) {
                d4[size_t(k) * nthr] = v[i];
                if (k + U < n) v[i] = ld_nc_v4(s4 + size_t(k + U) * nthr);
            }
        }
    }
}

__device__ void ag_push_warps(const AgParams& ag, unsigned int epoch, int cta, int n_ctas, int t, int k_bytes, int sc_bytes_per_mblock) {
    const AgGeometry geo{ag.rank, ag.world, ag.blocks_per_rank, k_bytes, sc_bytes_per_mblock, ag.parts, kAgFanOutPushWarps};
    const int units = ag_units(geo);
    for (int u = cta; u < units; u += n_ctas) {
        const AgPiece codes = ag_piece(geo, AgCursor{u, 0, 0u}, 0xffffffffu);
        const AgPiece scales = ag_piece(geo, AgCursor{u, 1, 0u}, 0xffffffffu);
        ag_copy_rolling<16>(ag.codes + codes.off, const_cast<uint8_t*>(ag.peer_codes[codes.dst_rank]) + codes.off, codes.bytes, t, 64);
        ag_copy_rolling<16>(ag.scales + scales.off, const_cast<uint8_t*>(ag.peer_scales[scales.dst_rank]) + scales.off, scales.bytes, t, 64);
        asm volatile("bar.sync 2, 64;" ::: "memory");       // both push warps have issued the unit's stores
        if (t == 0) {
            __threadfence_system();                           // cumulative over the stores ordered before the barrier
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(ag.peer_arrived[codes.dst_rank] + codes.flag), "r"(epoch) : "memory");
        }
    }
}

// Every CTA of the all-gather kernel calls this (one thread) when it has finished: the last one to arrive tells the
// peers that this rank no longer reads the buffer set of this epoch.
__device__ __forceinline__ void ag_exit(const AgParams& ag, unsigned int epoch_now) {
    if (ag.exit_counter == nullptr) return;
    __threadfence();
    const unsigned int prev = atomicAdd(ag.exit_counter, 1u);
    if (prev == gridDim.x - 1) {
        *reinterpret_cast<volatile unsigned int*>(ag.exit_counter) = 0u;       // ready for the next launch
        if (ag.epoch_counter != nullptr) *reinterpret_cast<volatile unsigned int*>(ag.epoch_counter) = epoch_now;     // this step is complete
        __threadfence_system();
        for (int pr = 0; pr < ag.world; pr++)
            if (pr != ag.rank && ag.peer_done[pr] != nullptr)
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(ag.peer_done[pr] + ag.rank), "r"(ag.epoch) : "memory");
    }
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void* map, uint32_t bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const void* map, uint32_t cluster_bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(x), "r"(y), "r"(z) : "memory");
}

// One comm CTA of the MoE kernel (all of its threads): fills its share of the 128-row blocks of the local
// activation buffer.  A quantized token travels as ONE row of k_bytes of codes followed by sc_row_bytes of
// scales.  Per block the 128 (source rank, source row) pairs of the dispatch list are pulled from the owners'
// buffers through a ring of row slots; when a row has landed, thread 0 forwards its codes to the local operand
// row with a bulk store and the other threads drop its scales into the 512-byte chunk layout the tensor core
// wants, which is stored as one contiguous span at the end.  Padding rows (-1) become zeros.
__device__ void moe_pull(const MoeParams& moe, int comm_idx, int k_bytes, int sc_row_bytes, uint32_t smem, uint32_t smem_avail, uint64_t* bars,
                         const WaitCtx& wc) {
    extern __shared__ uint8_t smem_raw_[];
    uint8_t* sm = smem_raw_ + (smem - smem_u32(smem_raw_));
    const int num_blocks = *moe.num_blocks;
    const int row_bytes = k_bytes + sc_row_bytes;
    const int sc_block_bytes = sc_row_bytes * 128;
    uint8_t* sc_sw = sm;                                          // [sc_row_bytes/4][512] chunk layout, as stored
    uint8_t* zero_row = sc_sw + sc_block_bytes;                   // k_bytes of zeros
    const uint32_t ring0_off = uint32_t(sc_block_bytes + ((k_bytes + 127) & ~127));
    const int ring = min(32, int((smem_avail - ring0_off) / uint32_t(row_bytes)));
    const int ahead = ring - 16;                                  // loads in flight; the two batches of 8 slots behind may still be read by stores
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int groups = sc_row_bytes / 4;                          // 4 scale bytes (64 K-elements) per row per chunk
    for (int i = tid; i < k_bytes / 4; i += nthr) reinterpret_cast<uint32_t*>(zero_row)[i] = 0;
    fence_proxy_async();
    __syncthreads();
    if (tid == 0) {
        for (int pr = 0; pr < moe.world; pr++)
            if (pr != moe.rank && !flag_wait(wc, moe.ready + pr, moe.epoch)) break;
    }
    __syncthreads();
    uint32_t issued = 0, done = 0;                                // rows over the whole kernel: ring position / phase
    constexpr int BATCH = 8;                                      // rows handled between two CTA barriers
    for (int blk = comm_idx; blk < num_blocks; blk += moe.comm_ctas) {
        __syncthreads();
        if (*wc.abort_flag) break;                                // read by every thread right after the same barrier
        const int* idx = moe.pull_idx + size_t(blk) * 128 * 2;
        int next = 0;
        for (int r0 = 0; r0 < 128; r0 += BATCH) {
            // Top up the loads, one batch at a time; within a batch every row is issued by its own lane (a single
            // thread cannot issue small bulk copies fast enough).  Slots of batches older than the previous one are
            // free: their stores were waited for below.
            while (next < 128 && int(issued - done) < ahead) {
                if (tid >= 32 && tid < 32 + BATCH) {
                    const int rr = next + (tid - 32);
                    const int src = idx[2 * rr], row = idx[2 * rr + 1];
                    const uint32_t slot = (issued + (tid - 32)) % ring;
                    if (src >= 0) {
                        mbar_arrive_expect_tx(smem_u32(&bars[slot]), row_bytes);
                        bulk_load(smem + ring0_off + slot * row_bytes, moe.peer_rows[src] + size_t(row) * row_bytes, row_bytes, smem_u32(&bars[slot]));
                    } else {
                        mbar_arrive(smem_u32(&bars[slot]));        // keeps the slot's phase in step
                    }
                }
                issued += BATCH; next += BATCH;
            }
            bool landed = true;
            for (int i = 0; i < BATCH && landed; i++) landed = mbar_wait(wc, smem_u32(&bars[(done + i) % ring]), ((done + i) / ring) & 1);
            if (!landed) break;          // every thread waits on the same barriers and sees the same abort flag: a uniform exit
            if (tid < BATCH) {
                // one lane per row forwards the codes; its previous store (one batch ago) has long been read
                const int r = r0 + tid;
                const uint32_t slot = (done + tid) % ring;
                tma_store_wait_read<0>();
                bulk_store(moe.codes + (size_t(blk) * 128 + r) * k_bytes, idx[2 * r] >= 0 ? smem + ring0_off + slot * row_bytes : smem_u32(zero_row), k_bytes);
                tma_store_commit();
            }
            for (int i = tid; i < BATCH * groups; i += nthr) {
                const int rr = i / groups, kc = i % groups, r = r0 + rr;
                const uint32_t slot = (done + rr) % ring;
                const uint32_t v = idx[2 * r] >= 0 ? *reinterpret_cast<const uint32_t*>(sm + ring0_off + slot * row_bytes + k_bytes + kc * 4) : 0u;
                *reinterpret_cast<uint32_t*>(sc_sw + kc * 512 + (r & 31) * 16 + (r >> 5) * 4) = v;
            }
            done += BATCH;
            __syncthreads();       // scale bytes of the batch are read; code stores of the batch BEFORE it were waited for above
        }
        if (tid < BATCH) tma_store_wait<0>();                      // this block's code rows are in local memory
        fence_proxy_async();
        __syncthreads();
        if (tid == 0) {
            bulk_store(moe.scales + size_t(blk) * sc_block_bytes, smem_u32(sc_sw), sc_block_bytes);
            tma_store_commit();
            tma_store_wait<0>();                                   // codes and scales of this block are in local memory
            __threadfence();
            st_release_gpu_u32(moe.arrived + blk, moe.epoch);
        }
    }
}

template <int KIND, int CTAS, int BN, int MODE, int MH = 1>
__global__ void __launch_bounds__(GemmCfg<KIND, CTAS, BN, MH>::THREADS + (MODE == MODE_AG ? 64 : 0), 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmSA, const __grid_constant__ CUtensorMap tmSB,
            const __grid_constant__ CUtensorMap tmD, const GemmParams p, const CommParams cp) {
    using C = GemmCfg<KIND, CTAS, BN, MH>;
    constexpr bool SCALED = KIND == KIND_NVFP4 || KIND == KIND_MXFP8;
    constexpr bool AG = MODE == MODE_AG;
    constexpr bool MOE = MODE == MODE_MOE;
    static_assert(!AG || (KIND == KIND_NVFP4 && CTAS == 2 && BN == 256), "all-gather mode: NVFP4, CTA pairs, N tile 256");
    static_assert(!MOE || (KIND == KIND_NVFP4 && CTAS == 1 && BN == 256), "MoE mode: NVFP4, single CTA, 128 x 256 tiles");
    const AgParams& ag = cp.ag;
    const MoeParams& moe = cp.moe;

    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[C::STAGES];
    __shared__ __align__(8) uint64_t bar_empty[C::STAGES];
    __shared__ __align__(8) uint64_t bar_tmem_full[2];
    __shared__ __align__(8) uint64_t bar_tmem_empty[2];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
    __shared__ unsigned int s_ag_all;      // all-gather mode: set by the CTA's spare warps once every remote row of the step has arrived
    __shared__ __align__(8) uint64_t bar_comm[MODE == MODE_MOE ? 32 : 1];   // comm CTAs of the MoE / all-gather modes

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta_rank = CTAS == 2 ? cluster_ctarank() : 0;
    const bool is_leader = cta_rank == 0;

    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sA = smem_base;
    const uint32_t sB = sA + C::STAGES * C::A_BYTES;
    const uint32_t sSA = sB + C::STAGES * C::B_BYTES;
    const uint32_t sSB = sSA + C::STAGES * C::SFA_BYTES;
    const uint32_t sEpi = (sSB + C::STAGES * C::SFB_BYTES + 1023u) & ~1023u;

    // MoE mode: the number of 128-row blocks that hold routed tokens is only known on the device
    const int tiles_m = MOE ? *moe.num_blocks : (p.M + C::BM - 1) / C::BM;
    const int tiles_n = (p.N + BN - 1) / BN;
    const int num_tiles = tiles_m * tiles_n;
    const int num_kb = (p.K + C::KB - 1) / C::KB;
    // all-gather mode: the first comm_ctas CTAs (whole clusters) only move data
    const int comm_ctas = AG ? ag.comm_ctas : (MOE ? moe.comm_ctas : 0);
    const int comm_units = comm_ctas / CTAS;
    const bool is_comm = int(blockIdx.x) < comm_ctas;
    const int first_tile = (CTAS == 2 ? int(cluster_id_x()) : int(blockIdx.x)) - comm_units;
    const int tile_stride = (CTAS == 2 ? int(num_clusters_x()) : int(gridDim.x)) - comm_units;
    const int tile_group = AG ? ag.blocks_per_rank : (MOE ? 1 : p.group);
    const int tile_rot = AG ? ag.rank * ag.blocks_per_rank : p.rot;

    if (threadIdx.x == 0) {
        s_abort = 0;
        s_ag_all = 0u;
        for (int s = 0; s < C::STAGES; s++) { mbar_init(smem_u32(&bar_full[s]), 1); mbar_init(smem_u32(&bar_empty[s]), 1); }
        for (int b = 0; b < 2; b++) {
            mbar_init(smem_u32(&bar_tmem_full[b]), 1);
            mbar_init(smem_u32(&bar_tmem_empty[b]), CTAS * C::EPI_WARPS);
        }
        fence_mbar_init();
        prefetch_tensormap(&tmA); prefetch_tensormap(&tmB); prefetch_tensormap(&tmD);
        if (SCALED) { prefetch_tensormap(&tmSA); prefetch_tensormap(&tmSB); }
    }
    if (warp == 1 && !is_comm) {
        tmem_alloc<CTAS>(smem_u32(&s_tmem_base), C::TMEM_COLS);
        tmem_relinquish<CTAS>();
    }
    tc_fence_before();
    if constexpr (CTAS == 2) cluster_sync(); else __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = s_tmem_base;
    WaitCtx wc{&s_abort, p.status, p.wait_limit};
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // successors launched with programmatic serialization wait on their own

    if constexpr (MOE || AG) {
        if (is_comm) asm volatile("griddepcontrol.wait;" ::: "memory");
    }
    if constexpr (MOE) {
        if (is_comm) {
            if (threadIdx.x == 0) {
                for (int i = 0; i < 32; i++) mbar_init(smem_u32(&bar_comm[i]), 1);
                fence_mbar_init();
            }
            __syncthreads();
            moe_pull(moe, int(blockIdx.x), p.K / 2, p.K / 16, smem_base, C::STAGES * C::STAGE_BYTES + C::EPI_BYTES, bar_comm, wc);   // needs 1 + K/64 <= blockDim.x
            __syncthreads();
            return;
        }
    }
    if constexpr (AG) {
        if (is_comm) {
            ag_push(ag, int(blockIdx.x), p.K / 2, (p.K / 64) * 512, wc, p.prof ? p.prof + blockIdx.x * 8 : nullptr);
            __syncthreads();
            if (threadIdx.x == 0) ag_exit(ag, ag.epoch);
            cluster_sync();      // matches the teardown barrier of the compute clusters' code path below
            return;
        }
    }

    if (warp == 0) {
        // ------------------------------------------------------------- TMA producer ----------
        if (elect_one()) {
            uint32_t stage = 0, phase = 0, issued = 0;
            bool ok = true;
            long long waited = 0, waited_flags = 0;
            asm volatile("griddepcontrol.wait;" ::: "memory");      // operands may come from the previous kernel in the stream
            // the arrival epoch of this step: given by the host, or one past the device's count of completed steps
            unsigned int ag_epoch = 0;
            if constexpr (AG) ag_epoch = ag.epoch_counter ? *reinterpret_cast<volatile unsigned int*>(ag.epoch_counter) + 1u : ag.epoch;
            (void)ag_epoch;
            unsigned long long ag_seen = 0ull;      // all-gather mode: row blocks whose arrival this thread has already observed
            bool ag_all = false;
            (void)ag_seen; (void)ag_all;
            const long long t_begin = clock64();
            for (int tile = first_tile; tile < num_tiles && ok; tile += tile_stride) {
                int m_blk, n_blk;
                tile_to_block(tile, tiles_m, tiles_n, tile_group, tile_rot, m_blk, n_blk);
                const int a_row = m_blk * C::BM + int(cta_rank) * 128 * MH;
                // MoE mode: the B operand is the weight matrix of the expert that owns this row block
                const int expert = MOE ? moe.block_expert[m_blk] : 0;
                const int b_row = expert * (MOE ? moe.expert_rows : 0) + n_blk * BN + int(cta_rank) * C::BN_CTA;
                const int b_sblk = expert * (MOE ? moe.expert_rows / 128 : 0) + n_blk * (BN / 128);
                if constexpr (MOE) {
                    if (!flag_wait(wc, moe.arrived + m_blk, moe.epoch)) { ok = false; break; }
                    fence_proxy_async_all();
                }
                if constexpr (AG) {
                    const int src = m_blk / ag.blocks_per_rank;
                    if (src != ag.rank) {
                        const long long t0 = clock64();
                        // Once the CTA's spare warps have seen every remote row of the step arrive (s_ag_all, released at CTA scope
                        // after their system-scope fence), nothing is left to check.  Before that: one check per block and CTA,
                        // since a block that was seen complete stays complete for the rest of the step.
                        if (!ag_all) {
                            unsigned int v;
                            asm volatile("ld.acquire.cta.shared.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(&s_ag_all)) : "memory");
                            if (v) { ag_all = true; fence_proxy_async_all(); }
                        }
                        if (!ag_all && (m_blk >= 64 || !((ag_seen >> m_blk) & 1ull))) {
                            const unsigned int* fl = ag.peer_arrived[ag.rank] + m_blk * ag.parts;
                            // all flags of the block with independent (relaxed, system-scope) loads first; only a block that is
                            // not complete yet is waited for flag by flag.  The fence below turns the observation into an acquire.
                            bool all = true;
                            for (int q = 0; q < ag.parts; q += 4) {
                                uint4 f;
                                asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(f.x), "=r"(f.y), "=r"(f.z), "=r"(f.w) : "l"(fl + q) : "memory");
                                all = all && int(f.x - ag_epoch) >= 0 && int(f.y - ag_epoch) >= 0 && int(f.z - ag_epoch) >= 0 && int(f.w - ag_epoch) >= 0;
                            }
                            if (!all)
                                for (int part = 0; part < ag.parts && ok; part++) ok = flag_wait(wc, fl + part, ag_epoch);
                            if (!ok) break;
                            __threadfence_system();
                            fence_proxy_async_all();
                            if (m_blk < 64) ag_seen |= 1ull << m_blk;
                        }
                        waited_flags += clock64() - t0;
                    }
                }
                for (int kb = 0; kb < num_kb; kb++) {
                    { const long long t0 = clock64();
                      if (!mbar_wait(wc, smem_u32(&bar_empty[stage]), phase ^ 1)) { ok = false; break; }
                      waited += clock64() - t0; }
                    const uint32_t full_local = smem_u32(&bar_full[stage]);
                    if (is_leader) mbar_arrive_expect_tx(full_local, C::TX_BYTES);
                    const int kx = kb * 128 / (KIND == KIND_BF16 ? 2 : 1);   // inner coordinate in tensor-map elements (bf16 or bytes)
                    if constexpr (CTAS == 2) {
                        const uint32_t full = mapa(full_local, 0);
                        tma_load_2d_pair(sA + stage * C::A_BYTES, &tmA, full, kx, a_row);
                        tma_load_2d_pair(sB + stage * C::B_BYTES, &tmB, full, kx, b_row);
                        if constexpr (SCALED) {
                            tma_load_3d_pair(sSA + stage * C::SFA_BYTES, &tmSA, full, 0, kb * C::SF_CHUNKS, m_blk * CTAS + int(cta_rank));
#pragma unroll
                            for (int j = 0; j < BN / 128; j++)
                                tma_load_3d_pair(sSB + stage * C::SFB_BYTES + j * C::SFA_BYTES, &tmSB, full, 0, kb * C::SF_CHUNKS,
                                                 b_sblk + j);
                        }
                    } else {
                        tma_load_2d(sA + stage * C::A_BYTES, &tmA, full_local, kx, a_row);
                        tma_load_2d(sB + stage * C::B_BYTES, &tmB, full_local, kx, b_row);
                        if constexpr (SCALED) {
                            tma_load_3d(sSA + stage * C::SFA_BYTES, &tmSA, full_local, 0, kb * C::SF_CHUNKS, m_blk);
#pragma unroll
                            for (int j = 0; j < BN / 128; j++)
                                tma_load_3d(sSB + stage * C::SFB_BYTES + j * C::SFA_BYTES, &tmSB, full_local, 0, kb * C::SF_CHUNKS,
                                            b_sblk + j);
                        }
                    }
                    issued++;
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (p.prof) {
                p.prof[blockIdx.x * 8 + 0] = waited; p.prof[blockIdx.x * 8 + 7] = waited_flags;
                bool pushing = false;
                if constexpr (AG) pushing = ag.push_warps != 0;
                if (!pushing) p.prof[blockIdx.x * 8 + 1] = clock64() - t_begin;
            }
            // tail: do not leave while stage releases from the MMA thread may still be in flight
            for (int s = 0; s < C::STAGES && ok; s++) {
                ok = mbar_wait(wc, smem_u32(&bar_empty[stage]), phase ^ 1);
                if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
            }
            if (!ok) {
                // giving up: the copies already issued must land before this CTA (pair) may exit.  Both CTAs' bytes are
                // credited to the leader's barriers; the other CTA just leaves the copies time and then meets the leader
                // at the teardown barrier.
                if (is_leader) drain_ring(bar_full, C::STAGES, issued, p.wait_limit);
                else __nanosleep(50000);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------- MMA issuer ------------
        if (is_leader && elect_one()) {
            uint32_t stage = 0, phase = 0, tile_count = 0, slot = 0;
            bool ok = true;
            long long wait_acc = 0, wait_full = 0;
            const long long t_begin = clock64();
            for (int tile = first_tile; tile < num_tiles && ok; tile += tile_stride) {
                { const long long t0 = clock64();
                  if (!mbar_wait(wc, smem_u32(&bar_tmem_empty[tile_count % C::ACC_BUFS]), ((tile_count / C::ACC_BUFS) & 1u) ^ 1u)) { ok = false; break; }
                  wait_acc += clock64() - t0; }
                tc_fence_after();
                const uint32_t acc_t = tmem_base + (tile_count % C::ACC_BUFS) * C::ACC_COLS;
                for (int kb = 0; kb < num_kb; kb++) {
                    { const long long t0 = clock64();
                      if (!mbar_wait(wc, smem_u32(&bar_full[stage]), phase)) { ok = false; break; }
                      wait_full += clock64() - t0; }
                    tc_fence_after();
                    const uint32_t sfa_t = tmem_base + C::SF_BASE + slot * (C::SFA_COLS + C::SFB_COLS);
                    const uint32_t sfb_t = sfa_t + C::SFA_COLS;
                    if constexpr (SCALED) {
#pragma unroll
                        for (int c = 0; c < C::SF_CHUNKS; c++) {
                            tc_cp_scale<CTAS>(sfa_t + 4 * c, smem_desc_scale(sSA + stage * C::SFA_BYTES + c * 512));
#pragma unroll
                            for (int j = 0; j < BN / 128; j++)
                                tc_cp_scale<CTAS>(sfb_t + (BN / 128) * 4 * c + 4 * j,
                                                  smem_desc_scale(sSB + stage * C::SFB_BYTES + j * C::SFA_BYTES + c * 512));
                        }
                    }
                    const uint64_t b_desc = smem_desc_sw128(sB + stage * C::B_BYTES);
#pragma unroll
                    for (int h = 0; h < MH; h++) {
                        const uint64_t a_desc = smem_desc_sw128(sA + stage * C::A_BYTES + h * 128 * 128);
                        const uint32_t acc_h = acc_t + h * BN;
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            const uint32_t acc = (kb > 0 || j > 0) ? 1u : 0u;
                            // +32 bytes of K inside the 128-byte swizzle panel = +2 in the (addr >> 4) field
                            if constexpr (KIND == KIND_BF16) {
                                mma_f16<CTAS>(acc_h, a_desc + 2 * j, b_desc + 2 * j, idesc_bf16(C::MMA_M, BN), acc);
                            } else if constexpr (KIND == KIND_FP8) {
                                mma_f8<CTAS>(acc_h, a_desc + 2 * j, b_desc + 2 * j, idesc_fp8(C::MMA_M, BN), acc);
                            } else if constexpr (KIND == KIND_MXFP8) {
                                mma_mxfp8<CTAS>(acc_h, a_desc + 2 * j, b_desc + 2 * j, idesc_mxfp8(C::MMA_M, BN, j), acc, sfa_t, sfb_t);
                            } else {
                                mma_nvfp4<CTAS>(acc_h, a_desc + 2 * j, b_desc + 2 * j, idesc_nvfp4(C::MMA_M, BN), acc, sfa_t + 4 * j,
                                                sfb_t + (BN / 128) * 4 * j);
                            }
                        }
                    }
                    tc_commit<CTAS>(smem_u32(&bar_empty[stage]));       // frees the stage (in both CTAs)
                    if (++stage == C::STAGES) { stage = 0; phase ^= 1; }
                    slot = (slot + 1) % C::SF_SLOTS;
                }
                tc_commit<CTAS>(smem_u32(&bar_tmem_full[tile_count % C::ACC_BUFS]));     // accumulator complete (both CTAs)
                tile_count++;
            }
            if (p.prof) { p.prof[blockIdx.x * 8 + 2] = wait_acc; p.prof[blockIdx.x * 8 + 3] = wait_full; p.prof[blockIdx.x * 8 + 4] = clock64() - t_begin; }
        }
        __syncwarp();
    } else if (warp < 2 + C::EPI_WARPS) {
        // ------------------------------------------------------------- epilogue --------------
        const int ew = warp - 2;
        const int quarter = warp & 3;                    // TMEM lane quarter this warp may read
        const int col_base = (ew >> 2) * C::COLS_PER_EPI_WARP;
        asm volatile("griddepcontrol.wait;" ::: "memory");          // D may still be read, and the scales written, by the previous kernel
        float alpha = 1.0f;
        if constexpr (KIND == KIND_NVFP4) alpha = __fmul_rn(*p.sgA, *p.sgB);
        float q_sg_dec = 0.f, q_sg_enc = 0.f;
        if constexpr (MODE == MODE_QUANT) {
            const float amax = *p.q_amax;
            if (p.q_arith == 0) {          // the torch specification's association
                q_sg_enc = __fdiv_rn(6.0f * 448.0f, fmaxf(amax, 0.000000000001f));
                q_sg_dec = __frcp_rn(q_sg_enc);
            } else {                       // the reference kernel's association
                q_sg_dec = __fdiv_rn(amax, 6.0f * 448.0f);
                q_sg_enc = __frcp_rn(fmaxf(q_sg_dec, 0.000000000001f));
            }
            if (blockIdx.x == 0 && warp == 2 && lane == 0) *p.q_sg = q_sg_dec;
        }
        (void)q_sg_dec; (void)q_sg_enc;
        const uint32_t tmem_empty_leader0 = CTAS == 2 ? mapa(smem_u32(&bar_tmem_empty[0]), 0) : smem_u32(&bar_tmem_empty[0]);
        const uint32_t tmem_empty_leader1 = CTAS == 2 ? mapa(smem_u32(&bar_tmem_empty[1]), 0) : smem_u32(&bar_tmem_empty[1]);
        const uint32_t stage_box = sEpi + ew * C::EPI_WARP_BYTES;
        const uint64_t d_policy = l2_policy_evict_first();     // D is written once and never read here: keep the operands in L2 instead
        uint32_t tile_count = 0;
        bool ok = true;
        long long wait_tf = 0, drain = 0;
        for (int tile = first_tile; tile < num_tiles && ok; tile += tile_stride) {
            int m_blk, n_blk;
            tile_to_block(tile, tiles_m, tiles_n, tile_group, tile_rot, m_blk, n_blk);
            const long long t0 = clock64();
            const uint32_t buf = tile_count % C::ACC_BUFS;
            if (!mbar_wait(wc, smem_u32(&bar_tmem_full[buf]), (tile_count / C::ACC_BUFS) & 1u)) { ok = false; break; }
            const long long t1 = clock64();
            wait_tf += t1 - t0;
            tile_count++;
            tc_fence_after();
            // Drain: both halves of this warp's 128 accumulator columns are requested back to back and only waited
            // for once; tensor memory goes back to the MMA warp before any arithmetic on the values.
#pragma unroll
            for (int mh = 0; mh < MH; mh++) {                // the accumulator halves of a tall tile, one after the other
            uint32_t r0[64], r1[64];
            tmem_ld_32x64(tmem_base + (uint32_t(quarter * 32) << 16) + buf * C::ACC_COLS + mh * BN + col_base, r0);
            tmem_ld_32x64(tmem_base + (uint32_t(quarter * 32) << 16) + buf * C::ACC_COLS + mh * BN + col_base + 64, r1);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0 && mh == MH - 1) {                 // the last half is in registers: tensor memory goes back
                const uint32_t tmem_empty_leader = buf ? tmem_empty_leader1 : tmem_empty_leader0;
                if constexpr (CTAS == 2) mbar_arrive_cluster(tmem_empty_leader); else mbar_arrive(tmem_empty_leader);
            }
            uint32_t packed[C::COLS_PER_EPI_WARP / 2];
#pragma unroll
            for (int i = 0; i < 32; i++) {
                packed[i] = pack_bf16x2(__fmul_rn(__uint_as_float(r0[2 * i]), alpha), __fmul_rn(__uint_as_float(r0[2 * i + 1]), alpha));
                packed[32 + i] = pack_bf16x2(__fmul_rn(__uint_as_float(r1[2 * i]), alpha), __fmul_rn(__uint_as_float(r1[2 * i + 1]), alpha));
            }
            drain += clock64() - t1;
            const int row0 = m_blk * C::BM + int(cta_rank) * 128 * MH + mh * 128 + quarter * 32;
            const int col0 = n_blk * BN + col_base;
            if constexpr (MODE == MODE_QUANT) {
                // This thread holds row `row0 + lane`, columns col0 .. col0 + 127 of D as bf16: eight 16-value blocks.
                // Codes: 64 contiguous bytes of the row; scales: two 4-byte words in the 512-byte chunks of its row block.
                const int row = row0 + lane;
                const int k_chunks_out = p.N / 64;
                uint32_t sc_word[2] = {0u, 0u};
                if (row < p.M) {
                    uint4* crow = reinterpret_cast<uint4*>(p.q_codes + size_t(row) * (p.N / 2) + col0 / 2);
#pragma unroll
                    for (int j = 0; j < 8; j += 2) {
                        uint2 c0, c1;
                        const uint32_t (&w0)[8] = *reinterpret_cast<const uint32_t (*)[8]>(&packed[8 * j]);
                        const uint32_t (&w1)[8] = *reinterpret_cast<const uint32_t (*)[8]>(&packed[8 * j + 8]);
                        const uint8_t s0 = quant_block16(w0, q_sg_dec, q_sg_enc, c0);
                        const uint8_t s1 = quant_block16(w1, q_sg_dec, q_sg_enc, c1);
                        sc_word[j >> 2] |= (uint32_t(s0) << (8 * (j & 3))) | (uint32_t(s1) << (8 * ((j + 1) & 3)));
                        if (col0 + 16 * j < p.N) crow[j >> 1] = make_uint4(c0.x, c0.y, c1.x, c1.y);
                    }
                }
                // rows past M inside the last 128-row block get zero scales, like the standalone quantizer writes them
                if (col0 < p.N && m_blk * CTAS + int(cta_rank) < (p.M + 127) / 128) {
                    uint8_t* chunk = p.q_sc + (size_t(m_blk * CTAS + int(cta_rank)) * k_chunks_out + col0 / 64) * 512 + lane * 16 + quarter * 4;
                    *reinterpret_cast<uint32_t*>(chunk) = sc_word[0];
                    if (col0 + 64 < p.N) *reinterpret_cast<uint32_t*>(chunk + 512) = sc_word[1];
                }
                continue;
            }
#pragma unroll
            for (int h = 0; h < C::COLS_PER_EPI_WARP / 64; h++) {
                // the previous store of this warp must have finished reading the staging box
                if (lane == 0) tma_store_wait_read<0>();
                __syncwarp();
#pragma unroll
                for (int j = 0; j < 8; j++)      // 16-byte chunk j of this thread's 128-byte row, 128-byte swizzle
                    st_shared_v4(stage_box + lane * 128 + ((j ^ (lane & 7)) << 4), packed[h * 32 + 4 * j], packed[h * 32 + 4 * j + 1],
                                 packed[h * 32 + 4 * j + 2], packed[h * 32 + 4 * j + 3]);
                fence_proxy_async();
                __syncwarp();
                if (lane == 0 && row0 < p.M && col0 + 64 * h < p.N) {
                    if constexpr (MODE == MODE_RS) {
                        // the rank that owns these 32 rows adds the box to its output (over NVLink unless it is this rank)
                        const int owner = row0 / p.rs_rows;
                        tma_reduce_add_2d(p.rs_maps + owner, stage_box, col0 + 64 * h, row0 - owner * p.rs_rows);
                    } else {
                        tma_store_2d_hint(&tmD, stage_box, col0 + 64 * h, row0, d_policy);
                    }
                    tma_store_commit();
                }
            }
            }       // accumulator halves
        }
        if (lane == 0) tma_store_wait<0>();
        __syncwarp();
        if (p.prof && warp == 2 && lane == 0) { p.prof[blockIdx.x * 8 + 5] = wait_tf; p.prof[blockIdx.x * 8 + 6] = drain; }
    } else {
        // ------------------------------------------------------------- push warps (all-gather mode) ----
        if constexpr (AG) {
            if (ag.world > 1 && !is_comm) {
                asm volatile("griddepcontrol.wait;" ::: "memory");      // the rows come from the quantize kernel before this one
                const unsigned int ag_epoch = ag.epoch_counter ? *reinterpret_cast<volatile unsigned int*>(ag.epoch_counter) + 1u : ag.epoch;
                const int t = int(threadIdx.x) - C::THREADS;
                if (ag.push_warps) {
                    const long long tp0 = clock64();
                    ag_push_warps(ag, ag_epoch, int(blockIdx.x), int(gridDim.x), t, p.K / 2, (p.K / 64) * 512);
                    if (p.prof && t == 0) p.prof[blockIdx.x * 8 + 1] = clock64() - tp0;      // push warps: slot 1 holds the cycles this CTA pushed for
                }
                // Then these two warps watch the arrival flags of ALL remote rows (a few KB, 16 bytes per thread and round) and
                // tell the producer thread through shared memory when the step's gather is complete, which takes the flag checks
                // (a system-scope fence each) out of the producer's way for the rest of the step.  Bounded like every wait;
                // giving up here reports nothing: the producer's own waits do.
                const unsigned int* fl = ag.peer_arrived[ag.rank];
                const int chunks = tiles_m * ag.parts / 4;                               // 4 flags per 16-byte chunk
                const int own_lo = ag.rank * ag.blocks_per_rank * ag.parts / 4, own_hi = own_lo + ag.blocks_per_rank * ag.parts / 4;
                const long long t0 = clock64();
                while (true) {
                    unsigned int mine = 1u;
                    for (int c = t; c < chunks; c += 64) {
                        if (c >= own_lo && c < own_hi) continue;                         // own rows raise no flags
                        uint4 f;
                        asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(f.x), "=r"(f.y), "=r"(f.z), "=r"(f.w) : "l"(fl + 4 * c) : "memory");
                        if (int(f.x - ag_epoch) < 0 || int(f.y - ag_epoch) < 0 || int(f.z - ag_epoch) < 0 || int(f.w - ag_epoch) < 0) mine = 0u;
                    }
                    unsigned int all;
                    asm volatile("{\n\t.reg .pred pin, pout;\n\tsetp.ne.u32 pin, %1, 0;\n\tbar.red.and.pred pout, 2, 64, pin;\n\tselp.u32 %0, 1, 0, pout;\n\t}"
                                 : "=r"(all) : "r"(mine) : "memory");
                    if (all) {
                        if (t == 0) {
                            __threadfence_system();
                            asm volatile("st.release.cta.shared.u32 [%0], %1;" ::"r"(smem_u32(&s_ag_all)), "r"(1u) : "memory");
                        }
                        break;
                    }
                    // giving up is decided together as well: every one of the 64 threads must take part in each barrier above
                    const unsigned int quit = (s_abort || clock64() - t0 > p.wait_limit) ? 1u : 0u;
                    unsigned int any_quit;
                    asm volatile("{\n\t.reg .pred pin, pout;\n\tsetp.ne.u32 pin, %1, 0;\n\tbar.red.or.pred pout, 2, 64, pin;\n\tselp.u32 %0, 1, 0, pout;\n\t}"
                                 : "=r"(any_quit) : "r"(quit) : "memory");
                    if (any_quit) break;
                    __nanosleep(4000);                  // 148 CTAs re-reading a few KB of flags: rare enough not to show in the L2 traffic
                }
            }
        }
    }

    // ----------------------------------------------------------------- teardown --------------
    tc_fence_before();
    if constexpr (CTAS == 2) cluster_sync(); else __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc<CTAS>(tmem_base, C::TMEM_COLS);
    }
    if constexpr (AG) {
        // (read before this CTA's own arrival on the exit counter, so before the last CTA can have advanced the count)
        const unsigned int ag_epoch_exit = (threadIdx.x == 0 && ag.epoch_counter) ? *reinterpret_cast<volatile unsigned int*>(ag.epoch_counter) + 1u : ag.epoch;
        if (threadIdx.x == 0) ag_exit(ag, ag_epoch_exit);      // after the barrier: this CTA's operand loads and output stores are complete
    }
}

// ------------------------------------------------------------------------------ host -------
template <int KIND, int CTAS, int BN, int MODE = MODE_PLAIN, int MH = 1>
static cudaError_t launch_t(const GemmArgs& a) {
    using C = GemmCfg<KIND, CTAS, BN, MH>;
    auto kern = gemm_kernel<KIND, CTAS, BN, MODE, MH>;
    // the attribute belongs to the (kernel, device) pair: remember it per device, not per process
    static std::atomic<bool> attr_set[64] = {};
    int dev = 0;
    if (cudaError_t e = cudaGetDevice(&dev); e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64 || !attr_set[dev].load(std::memory_order_acquire)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) attr_set[dev].store(true, std::memory_order_release);
    }
    const int tiles = ((a.M + C::BM - 1) / C::BM) * ((a.N + BN - 1) / BN);
    const int comm_units = MODE == MODE_AG ? a.comm.ag.comm_ctas / CTAS : (MODE == MODE_MOE ? a.comm.moe.comm_ctas / CTAS : 0);
    int units = a.sm_count / CTAS - comm_units;
    if (units > tiles && MODE != MODE_MOE) units = tiles;
    if (units < 1) units = 1;
    units += comm_units;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(units * CTAS, 1, 1);
    cfg.blockDim = dim3(C::THREADS + (MODE == MODE_AG ? 64 : 0), 1, 1);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = a.stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CTAS; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    // programmatic stream serialization: CTAs may be scheduled while the previous kernel drains (they set up barriers and
    // tensor memory, then execute griddepcontrol.wait before touching global memory)
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 2;
    static const int group_env = getenv("TKB_GEMM_GROUP") ? atoi(getenv("TKB_GEMM_GROUP")) : 0;
    GemmParams p{a.sgA, a.sgB, a.M, a.N, a.K, group_env > 0 ? group_env : 16, 0, a.status, a.prof, api_wait_limit(),
                 static_cast<uint8_t*>(a.q_codes), static_cast<uint8_t*>(a.q_sc), a.q_sg, a.q_amax, a.q_arith, a.rs_maps, a.rs_rows_per_rank};
    if (MODE == MODE_RS && a.rs_world > 0) {
        // start with the rows of the next rank, so that the ranks do not all add into the same owner at the same time
        p.group = a.rs_rows_per_rank / C::BM;
        p.rot = ((a.rs_rank + 1) % a.rs_world) * p.group;
    }
    return cudaLaunchKernelEx(&cfg, kern, a.tmA, a.tmB, a.tmSA, a.tmSB, a.tmD, p, a.comm);
}

template <int KIND>
static cudaError_t launch_k(const GemmArgs& a) {
    if constexpr (KIND == KIND_BF16 || KIND == KIND_FP8) {
        if (a.config & 4) return launch_t<KIND, 2, 256, MODE_PLAIN, 2>(a);      // 512 x 256 cluster tiles
    }
    switch (a.config & 3) {
        case 0: return launch_t<KIND, 2, 256>(a);
        case 1: return launch_t<KIND, 1, 256>(a);
        case 2: return launch_t<KIND, 2, 128>(a);
        default: return launch_t<KIND, 1, 128>(a);
    }
}

// Row slots of the MoE dispatch ring for hidden size K (the arithmetic of moe_pull on the shared memory of its kernel instance)
int moe_dispatch_ring(int K) {
    using C = GemmCfg<KIND_NVFP4, 1, 256>;
    const long avail = long(C::STAGES) * C::STAGE_BYTES + C::EPI_BYTES;
    const long ring0 = 128L * (K / 16) + (((K / 2) + 127) & ~127);
    const long ring = (avail - ring0) / (K / 2 + K / 16);
    return int(ring < 0 ? 0 : (ring > 32 ? 32 : ring));
}

int gemm_tile_n(int config) { return (config & 2) ? 128 : 256; }
int gemm_tile_m(int config) { return (config & 4) ? 512 : ((config & 1) ? 128 : 256); }

cudaError_t launch_gemm(const GemmArgs& a) {
    if (a.mode == MODE_AG) return launch_t<KIND_NVFP4, 2, 256, MODE_AG>(a);
    if (a.mode == MODE_QUANT) return launch_t<KIND_NVFP4, 2, 256, MODE_QUANT>(a);
    if (a.mode == MODE_RS) return launch_t<KIND_NVFP4, 2, 256, MODE_RS>(a);
    if (a.mode == MODE_MOE) return launch_t<KIND_NVFP4, 1, 256, MODE_MOE>(a);
    switch (a.kind) {
        case KIND_BF16: return launch_k<KIND_BF16>(a);
        case KIND_MXFP8: return launch_k<KIND_MXFP8>(a);
        case KIND_NVFP4: return launch_k<KIND_NVFP4>(a);
        case KIND_FP8: return launch_k<KIND_FP8>(a);
        default: return cudaErrorInvalidValue;
    }
}

} // namespace tkb
