// Skinny-M ("decode") NVFP4 GEMM for sm_100a: D[M,N] (bf16) = X[M,K] * W[N,K]^T with M <= 128.
//
// The reference's nvfp4_gemm (kernels/gemm/nvfp4_b200/nvfp4_b200_gemm.cu:88-307) needs M % 256 == 0,
// so it has no kernel for these shapes; the arithmetic is the same block-scaled product as the large
// GEMM and is checked against the same oracle.  The problem is bound by streaming the weights
// (N*K/2 bytes of codes + N*K/16 bytes of scales) from HBM once, so the design is about keeping
// every SM's TMA queue full and the work split evenly:
//   * operands are swapped: the 128-row weight slab is the MMA's M side (tcgen05.mma M=128), the
//     (padded) activation rows are its N side (N = 16/32/64/128), so no tensor-core work is wasted
//     on padding a 1..128-row activation up to a 128/256-row tile;
//   * stream-K: the (slab, 256-wide K-block) work items are cut into one contiguous, equal range per
//     CTA (one persistent CTA per SM).  A CTA that starts a slab finishes it; a
//     CTA that only covers the tail of a slab writes its fp32 partial tile to scratch first thing
//     and raises a flag.  The finisher reaches its (last) head segment after all its other work, so
//     the partials it needs are normally already there; its wait is bounded like every other wait;
//   * warp 0 = TMA producer, warp 1 = MMA issuer, warps 2..5 = epilogue; two accumulator buffers in
//     tensor memory so the epilogue of one segment overlaps the main loop of the next.
#include <cstdlib>
#include <cstring>
#include <atomic>
#include <mutex>
#include "ptx.cuh"
#include "internal.h"

namespace tkb {

template <int NB>
struct DecodeCfg {
    static_assert(NB == 16 || NB == 32 || NB == 64 || NB == 128, "");
    static constexpr int W_BYTES = 128 * 128;            // 128 weight rows x 256 e2m1 of K
    static constexpr int X_BYTES = NB * 128;
    static constexpr int SF_BYTES = 4 * 512;             // 4 scale chunks (4 x 64 K) per 128 rows
    static constexpr int STAGE_BYTES = W_BYTES + X_BYTES + 2 * SF_BYTES;
    // 32 or more activation rows: the output tile (NB rows x 128 weight rows, bf16) is staged in shared memory and leaves as one
    // TMA store; 16 rows are few enough to store from registers (16 stores of 64 contiguous bytes per warp)
    static constexpr bool STAGED_OUT = NB >= 32;
    static constexpr int OUT_BYTES = STAGED_OUT ? NB * 256 : 0;
    static constexpr int STAGES_RAW = (227 * 1024 - 3072 - OUT_BYTES) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 10 ? 10 : STAGES_RAW;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + OUT_BYTES + 2048;
    static constexpr int THREADS = 6 * 32;
    static constexpr int SF_SLOTS = 4;
    static constexpr int SF_BASE = 2 * (NB < 32 ? 32 : NB);      // accumulators at columns 0 and ACC_STRIDE
    static constexpr int ACC_STRIDE = NB < 32 ? 32 : NB;
    static constexpr int TMEM_COLS = 512;
    static constexpr uint32_t TX_BYTES = STAGE_BYTES;
    static constexpr int CHUNK = NB < 32 ? NB : 32;      // accumulator columns read per tcgen05.ld
};

struct DecodeParams {
    const float* sgX; const float* sgW;
    __nv_bfloat16* D; int64_t ldd;
    int M, N, K;
    float* partials;            // [grid][NB][128] fp32
    unsigned int* flags;        // [grid]
    unsigned int epoch;
    int* status;
    unsigned long long* prof;   // optional (tkb_gemm_set_profile_buffer): 8 words per CTA, see decode_kernel
    long long wait_limit;       // clock cycles any wait of the kernel may last
    int prefetch_weights;       // the weights were complete before the previous kernel in the stream started: load them before the dependency wait
    int stages;                 // operand-ring stages to use (clamped to what the instance has)
};

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d_d(uint32_t dst, const void* map, uint32_t bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(unsigned int* p, unsigned int v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void epi_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

struct Segment { int slab, kb0, kb1; };

// Work range of CTA g and iteration over its segments (identical in every role).
struct WorkRange {
    long long item, end; int kblk;
    __device__ WorkRange(int g, int grid, int slabs, int kblk_) : kblk(kblk_) {
        const long long items = (long long)slabs * kblk_;
        item = items * g / grid;
        end = items * (g + 1) / grid;
    }
    __device__ bool next(Segment& s) {
        if (item >= end) return false;
        s.slab = int(item / kblk);
        s.kb0 = int(item % kblk);
        const long long left = end - item;
        s.kb1 = int(min((long long)kblk, s.kb0 + left));
        item += s.kb1 - s.kb0;
        return true;
    }
};

template <int NB>
__global__ void __launch_bounds__(DecodeCfg<NB>::THREADS, 1)
decode_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
              const __grid_constant__ CUtensorMap tmSW, const __grid_constant__ CUtensorMap tmSX, const __grid_constant__ CUtensorMap tmD,
              const DecodeParams p) {
    using C = DecodeCfg<NB>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[C::STAGES];
    __shared__ __align__(8) uint64_t bar_empty[C::STAGES];
    __shared__ __align__(8) uint64_t bar_acc_full[2];
    __shared__ __align__(8) uint64_t bar_acc_empty[2];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
    __shared__ int s_flag_ok;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // profile words of this CTA (global nanosecond timer): [0] CTA start, [1] producer past the dependency wait, [2] first
    // stage landed, [3] last MMA issued, [4] epilogue finished, [5] ns the epilogue waited for other CTAs' partial tiles,
    // [6] ns the MMA thread waited for operands, [7] ns the epilogue spent on its segments after their accumulators were complete
    unsigned long long* prof = p.prof ? p.prof + size_t(blockIdx.x) * 16 : nullptr;      // ([8] tensor-memory reads, [9] partial-tile
    // stores and their publication, [10] stores of D, [11] segments: epilogue thread 64, ns)
    if (prof && threadIdx.x == 0) prof[0] = global_ns();
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sW = smem_base;
    const uint32_t sX = sW + C::STAGES * C::W_BYTES;
    const uint32_t sSW = (sX + C::STAGES * C::X_BYTES + 1023u) & ~1023u;
    const uint32_t sSX = sSW + C::STAGES * C::SF_BYTES;
    const uint32_t sOut = sSX + C::STAGES * C::SF_BYTES;      // [NB][128] bf16: D rows of one slab, stored by TMA (128-byte aligned)

    const int slabs = (p.N + 127) / 128;
    const int kblk = (p.K + 255) / 256;
    // stages of the operand ring in use: fewer than fit spreads the start-up burst (every SM filling its whole ring at once
    // queues ~180 KB per SM in the memory system, and the SMs served last stay that far behind to the end)
    const int nst = p.stages < 3 ? 3 : (p.stages > C::STAGES ? C::STAGES : p.stages);

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < C::STAGES; s++) { mbar_init(smem_u32(&bar_full[s]), 1); mbar_init(smem_u32(&bar_empty[s]), 1); }
        for (int b = 0; b < 2; b++) { mbar_init(smem_u32(&bar_acc_full[b]), 1); mbar_init(smem_u32(&bar_acc_empty[b]), 4); }
        fence_mbar_init();
        prefetch_tensormap(&tmW); prefetch_tensormap(&tmX); prefetch_tensormap(&tmSW); prefetch_tensormap(&tmSX);
        if (C::STAGED_OUT) prefetch_tensormap(&tmD);
    }
    if (warp == 1) {
        tmem_alloc<1>(smem_u32(&s_tmem_base), C::TMEM_COLS);
        tmem_relinquish<1>();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = s_tmem_base;
    WaitCtx wc{&s_abort, p.status, p.wait_limit};
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        // ----------------------------------------------------------------- TMA producer -----
        if (elect_one()) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            // With prefetch_weights the caller states that the weights do not depend on the kernel that runs before
            // this one in the stream (typically the activation quantizer): fill the ring with weight tiles first, only
            // then wait for that kernel and add the activation tiles of the same stages.  Without it nothing is read
            // before the wait.
            int prefetched = 0;
            if (p.prefetch_weights) {
                WorkRange wr(blockIdx.x, gridDim.x, slabs, kblk);
                Segment sg;
                while (prefetched < nst && wr.next(sg))
                    for (int kb = sg.kb0; kb < sg.kb1 && prefetched < nst; kb++, prefetched++) {
                        const uint32_t full = smem_u32(&bar_full[prefetched]);
                        mbar_arrive_expect_tx(full, C::TX_BYTES);
                        tma_load_2d(sW + prefetched * C::W_BYTES, &tmW, full, kb * 128, sg.slab * 128);
                        tma_load_3d_d(sSW + prefetched * C::SF_BYTES, &tmSW, full, 0, kb * 4, sg.slab);
                    }
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            if (prof) prof[1] = global_ns();
            WorkRange wr(blockIdx.x, gridDim.x, slabs, kblk);
            Segment sg;
            int item = 0;
            while (ok && wr.next(sg)) {
                for (int kb = sg.kb0; kb < sg.kb1; kb++, item++) {
                    const uint32_t full = smem_u32(&bar_full[stage]);
                    if (item >= prefetched) {
                        if (!mbar_wait(wc, smem_u32(&bar_empty[stage]), phase ^ 1)) { ok = false; break; }
                        mbar_arrive_expect_tx(full, C::TX_BYTES);
                        tma_load_2d(sW + stage * C::W_BYTES, &tmW, full, kb * 128, sg.slab * 128);
                        tma_load_3d_d(sSW + stage * C::SF_BYTES, &tmSW, full, 0, kb * 4, sg.slab);
                    }
                    tma_load_2d(sX + stage * C::X_BYTES, &tmX, full, kb * 128, 0);
                    tma_load_3d_d(sSX + stage * C::SF_BYTES, &tmSX, full, 0, kb * 4, 0);
                    if (++stage == uint32_t(nst)) { stage = 0; phase ^= 1; }
                }
            }
            for (int s = 0; s < nst && ok; s++) {
                ok = mbar_wait(wc, smem_u32(&bar_empty[stage]), phase ^ 1);
                if (++stage == uint32_t(nst)) { stage = 0; phase ^= 1; }
            }
            if (!ok) drain_ring(bar_full, nst, uint32_t(item > prefetched ? item : prefetched), p.wait_limit);   // giving up: let the issued copies land
        }
        __syncwarp();
    } else if (warp == 1) {
        // ----------------------------------------------------------------- MMA issuer -------
        if (elect_one()) {
            uint32_t stage = 0, phase = 0, slot = 0;
            int seg_idx = 0;
            bool ok = true, first = true;
            unsigned long long waited = 0;
            WorkRange wr(blockIdx.x, gridDim.x, slabs, kblk);
            Segment sg;
            while (ok && wr.next(sg)) {
                const int buf = seg_idx & 1;
                if (!mbar_wait(wc, smem_u32(&bar_acc_empty[buf]), ((seg_idx >> 1) & 1) ^ 1)) { ok = false; break; }
                tc_fence_after();
                const uint32_t acc_t = tmem_base + buf * C::ACC_STRIDE;
                for (int kb = sg.kb0; kb < sg.kb1; kb++) {
                    if (prof) {
                        const unsigned long long t0 = global_ns();
                        if (!mbar_wait(wc, smem_u32(&bar_full[stage]), phase)) { ok = false; break; }
                        const unsigned long long t1 = global_ns();
                        waited += t1 - t0;
                        if (first) { prof[2] = t1; first = false; }
                    } else if (!mbar_wait(wc, smem_u32(&bar_full[stage]), phase)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sfa_t = tmem_base + C::SF_BASE + slot * 32;
                    const uint32_t sfb_t = sfa_t + 16;
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        tc_cp_scale<1>(sfa_t + 4 * c, smem_desc_scale(sSW + stage * C::SF_BYTES + c * 512));
                        tc_cp_scale<1>(sfb_t + 4 * c, smem_desc_scale(sSX + stage * C::SF_BYTES + c * 512));
                    }
                    const uint64_t a_desc = smem_desc_sw128(sW + stage * C::W_BYTES);
                    const uint64_t b_desc = smem_desc_sw128(sX + stage * C::X_BYTES);
#pragma unroll
                    for (int j = 0; j < 4; j++)
                        mma_nvfp4<1>(acc_t, a_desc + 2 * j, b_desc + 2 * j, idesc_nvfp4(128, NB), (kb > sg.kb0 || j > 0) ? 1u : 0u,
                                     sfa_t + 4 * j, sfb_t + 4 * j);
                    tc_commit<1>(smem_u32(&bar_empty[stage]));
                    if (++stage == uint32_t(nst)) { stage = 0; phase ^= 1; }
                    slot = (slot + 1) % C::SF_SLOTS;
                }
                tc_commit<1>(smem_u32(&bar_acc_full[buf]));
                seg_idx++;
            }
            if (prof) { prof[3] = global_ns(); prof[6] = waited; }
        }
        __syncwarp();
    } else {
        // ----------------------------------------------------------------- epilogue ----------
        const int quarter = warp & 3;
        const int n_local = quarter * 32 + lane;           // weight row inside the slab
        asm volatile("griddepcontrol.wait;" ::: "memory");   // the activation scale comes from the previous kernel; D / scratch may still be read by it
        const float alpha = __fmul_rn(*p.sgX, *p.sgW);
        int seg_idx = 0;
        bool ok = true;
        WorkRange wr(blockIdx.x, gridDim.x, slabs, kblk);
        Segment sg;
        while (ok && wr.next(sg)) {
            const int buf = seg_idx & 1;
            const bool head = sg.kb0 == 0;
            const bool complete = head && sg.kb1 == kblk;
            const int n = sg.slab * 128 + n_local;
            // An incomplete head adds the partial tiles of the CTAs that hold the rest of its slab.  Those CTAs met that slab
            // first thing, so their tiles are normally there long before this segment's own MMAs end: wait for their flags and
            // fetch the tiles into registers (summed in CTA order) BEFORE waiting for the accumulator, so that the round trip
            // to L2 overlaps the main loop instead of following it.
            float psum[NB];
            int contrib_lo = 0, contrib_hi = 0;
            if (head && !complete) {
                const long long items = (long long)slabs * kblk;
                const long long slab_end = (long long)(sg.slab + 1) * kblk;
                contrib_lo = int(blockIdx.x) + 1;
                contrib_hi = contrib_lo;
                while (contrib_hi < int(gridDim.x) && items * contrib_hi / gridDim.x < slab_end) contrib_hi++;
                if (threadIdx.x == 64) {
                    int good = 1;
                    const unsigned long long tw0 = prof ? global_ns() : 0ull;
                    for (int h = contrib_lo; h < contrib_hi && good; h++) {
                        const long long t0 = clock64();
                        while (ld_acquire_gpu(p.flags + h) != p.epoch) {
                            if (s_abort || clock64() - t0 > p.wait_limit) {
                                good = 0; s_abort = 1;
                                if (p.status) atomicExch(p.status, (int)TKB_DEV_TIMEOUT);
                                break;
                            }
                            __nanosleep(32);
                        }
                    }
                    s_flag_ok = good;
                    if (prof) prof[5] += global_ns() - tw0;
                }
                epi_barrier();
                if (!s_flag_ok) ok = false;
#pragma unroll
                for (int c = 0; c < NB; c++) psum[c] = 0.f;
                if (ok) {
                    for (int h = contrib_lo; h < contrib_hi; h++) {
                        const float* src = p.partials + size_t(h) * NB * 128 + n_local;
#pragma unroll
                        for (int c = 0; c < NB; c++) psum[c] += __ldcg(src + c * 128);
                    }
                }
            }
            if (C::STAGED_OUT && head) {
                // this segment writes D through the staging tile: the TMA store of the previous one must have read it
                if (threadIdx.x == 64) tma_store_wait_read<0>();
                epi_barrier();
            }
            if (!mbar_wait(wc, smem_u32(&bar_acc_full[buf]), (seg_idx >> 1) & 1)) { ok = false; break; }
            tc_fence_after();
            const unsigned long long t_seg = (prof && threadIdx.x == 64) ? global_ns() : 0ull;
#pragma unroll
            for (int c0 = 0; c0 < NB; c0 += C::CHUNK) {
                float v[C::CHUNK];
                const unsigned long long t_c0 = (prof && threadIdx.x == 64) ? global_ns() : 0ull;
                if constexpr (C::CHUNK == 32) {
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + (uint32_t(quarter * 32) << 16) + buf * C::ACC_STRIDE + c0, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
                } else {
                    uint32_t r[16];
                    tmem_ld_32x16(tmem_base + (uint32_t(quarter * 32) << 16) + buf * C::ACC_STRIDE + c0, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
                }
                const unsigned long long t_ld = (prof && threadIdx.x == 64) ? global_ns() : 0ull;
                if (prof && threadIdx.x == 64) prof[8] += t_ld - t_c0;
                if (c0 + C::CHUNK >= NB) {
                    // last chunk read: the accumulator buffer can be reused
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&bar_acc_empty[buf]));
                }
                if (!head) {
                    float* dst = p.partials + (size_t(blockIdx.x) * NB + c0) * 128 + n_local;
#pragma unroll
                    for (int i = 0; i < C::CHUNK; i++) __stcg(dst + i * 128, v[i]);
                    if (prof && threadIdx.x == 64) prof[9] += global_ns() - t_ld;
                } else {
                    if (!complete) {
#pragma unroll
                        for (int i = 0; i < C::CHUNK; i++) v[i] += psum[c0 + i];
                    }
                    if constexpr (C::STAGED_OUT) {
                        // D[m][n] for this thread's weight row n: one 2-byte shared-memory store per activation row (a warp fills
                        // 64 contiguous bytes, no bank conflict); the tile leaves as ONE TMA store of NB rows x 256 bytes below
#pragma unroll
                        for (int i = 0; i < C::CHUNK; i++) {
                            const __nv_bfloat16 b = __float2bfloat16_rn(__fmul_rn(v[i], alpha));
                            asm volatile("st.shared.b16 [%0], %1;" ::"r"(sOut + uint32_t(c0 + i) * 256u + uint32_t(n_local) * 2u), "h"(__bfloat16_as_ushort(b)) : "memory");
                        }
                    } else if (n < p.N) {
#pragma unroll
                        for (int i = 0; i < C::CHUNK; i++)
                            if (c0 + i < p.M) p.D[int64_t(c0 + i) * p.ldd + n] = __float2bfloat16_rn(__fmul_rn(v[i], alpha));
                    }
                    if (prof && threadIdx.x == 64) prof[10] += global_ns() - t_ld;
                }
            }
            if (C::STAGED_OUT && head) {
                fence_proxy_async();
                epi_barrier();
                if (threadIdx.x == 64) {          // rows past M and columns past N are clipped by the TMA unit
                    tma_store_2d(&tmD, sOut, sg.slab * 128, 0);
                    tma_store_commit();
                }
            }
            if (head && !complete) {
                // every epilogue thread has read the partial tiles: put the contributors' flags back to 0 so that a
                // later launch that carries the same epoch (a replayed CUDA graph) does not mistake them for fresh
                if (!C::STAGED_OUT) epi_barrier();          // (the staged path has just passed a barrier)
                if (threadIdx.x == 64)
                    for (int h = contrib_lo; h < contrib_hi; h++) st_release_gpu(p.flags + h, 0u);
            }
            if (!head) {
                // publish the partial tile: all four epilogue warps have stored, then one release
                const unsigned long long t_pub = (prof && threadIdx.x == 64) ? global_ns() : 0ull;
                epi_barrier();
                if (threadIdx.x == 64) {
                    __threadfence();
                    st_release_gpu(p.flags + blockIdx.x, p.epoch);
                    if (prof) prof[9] += global_ns() - t_pub;
                }
            }
            if (prof && threadIdx.x == 64) { prof[7] += global_ns() - t_seg; prof[11] += 1; }
            seg_idx++;
        }
        if (C::STAGED_OUT && threadIdx.x == 64) tma_store_wait<0>();
        if (prof && threadIdx.x == 64) prof[4] = global_ns();
        __syncwarp();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc<1>(tmem_base, C::TMEM_COLS);
    }
}

template <int NB>
static cudaError_t launch_decode_t(const DecodeArgs& a) {
    using C = DecodeCfg<NB>;
    auto kern = decode_kernel<NB>;
    // the attribute belongs to the (kernel, device) pair: remember it per device, not per process
    static std::atomic<bool> attr_set[64] = {};
    int dev = 0;
    if (cudaError_t e = cudaGetDevice(&dev); e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64 || !attr_set[dev].load(std::memory_order_acquire)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) attr_set[dev].store(true, std::memory_order_release);
    }
    const long long items = (long long)((a.N + 127) / 128) * ((a.K + 255) / 256);
    int grid = a.sm_count;
    if (grid > a.max_grid) grid = a.max_grid;
    if (grid > items) grid = int(items);
    if (grid < 1) grid = 1;
    static const int stages_env = getenv("TKB_DECODE_STAGES") ? atoi(getenv("TKB_DECODE_STAGES")) : 0;      // tuning aid
    // 6 stages (~108 KB of weights per SM) measured best: with all 10 the start-up burst queues so much that the SMs served
    // last trail by ~4 us to the end; with 4 or fewer the HBM pipe is no longer full
    const int stages = stages_env > 0 ? stages_env : 6;
    DecodeParams p{a.sgX, a.sgW, static_cast<__nv_bfloat16*>(a.D), a.ldd, a.M, a.N, a.K, a.partials, a.flags, a.epoch, a.status, a.prof, api_wait_limit(), a.prefetch_weights, stages};
    CUtensorMap tmW = a.tmW, tmX = a.tmX, tmSW = a.tmSW, tmSX = a.tmSX, tmD = a.tmD;
    // Programmatic stream serialization: the kernel may start while its predecessor in the stream drains; it prefetches
    // weights, and executes griddepcontrol.wait before anything that depends on (or could disturb) earlier kernels.
    // All CTAs of the grid are expected to be resident together (grid <= SM count, one CTA per SM); the stream-K waits
    // are bounded, so a CTA that is kept off the GPU for long shows up as a reported timeout, not a hang.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(C::THREADS); cfg.dynamicSmemBytes = C::SMEM_BYTES; cfg.stream = a.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, tmW, tmX, tmSW, tmSX, tmD, p);
}

int decode_padded_rows(int M) { return M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128)); }

cudaError_t launch_decode(const DecodeArgs& a) {
    switch (decode_padded_rows(a.M)) {
        case 16: return launch_decode_t<16>(a);
        case 32: return launch_decode_t<32>(a);
        case 64: return launch_decode_t<64>(a);
        default: return launch_decode_t<128>(a);
    }
}

} // namespace tkb

// ---------------------------------------------------------------------------------------------------------
// Allocation-free variant of the skinny-M GEMM.
//
// Some hosts of this library may not allocate device memory at the point where they call it: inference
// runtimes that size every buffer at start-up and treat an allocation on the request path as a bug (it
// synchronises the device and can fail under memory pressure), and plug-in interfaces whose "enqueue"
// hook forbids cudaMalloc.  The regular entry point
// tkb_nvfp4_gemm creates a per-device context and its stream-K scratch with cudaMalloc on first use, so those
// callers get this second door: the scratch lives in a fixed array that is part of the loaded module.
//
// The array costs kStaticScratchBytes (about 1.3 MB) of device memory on every GPU that loads the library,
// for as long as the process lives, which is why it is sized for the smallest activation tile only: M <= 16
// (one 16 x 128 fp32 partial tile and one flag per CTA, up to kStaticMaxGrid CTAs).
namespace tkb {

constexpr int kStaticMaxGrid = 160;
constexpr int kStaticMaxM = 16;
constexpr size_t kStaticPartialBytes = size_t(kStaticMaxGrid) * 16 * 128 * sizeof(float);
constexpr size_t kStaticFlagBytes = size_t(kStaticMaxGrid) * sizeof(unsigned int);
constexpr size_t kStaticScratchBytes = kStaticPartialBytes + 1024;     // flags live in the last 1 KB

static_assert(kStaticFlagBytes <= 1024, "flag area");
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

int api_fail(int code, const char* fmt, ...);     // api.cu: records the calling thread's error message

namespace {
constexpr int kStaticMaxDevices = 64;
struct StaticDev { std::atomic<bool> ready; unsigned char* scratch; int sm_count; };
StaticDev g_static_dev[kStaticMaxDevices];
std::mutex g_static_mu;

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                             const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn g_static_encode = nullptr;

bool encode_2d(CUtensorMap* m, const void* base, uint64_t inner_bytes, uint64_t rows, uint32_t box_rows) {
    cuuint64_t dims[2] = {inner_bytes, rows};
    cuuint64_t strides[1] = {inner_bytes};
    cuuint32_t box[2] = {128, box_rows};
    cuuint32_t estr[2] = {1, 1};
    return g_static_encode(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
bool encode_scales(CUtensorMap* m, const void* base, uint64_t row_blocks, uint64_t k_chunks) {
    cuuint64_t dims[3] = {128, k_chunks, row_blocks};
    cuuint64_t strides[2] = {512, 512 * k_chunks};
    cuuint32_t box[3] = {128, 4, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    return g_static_encode(m, CU_TENSOR_MAP_DATA_TYPE_INT32, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
} // namespace
} // namespace tkb

extern "C" int tkb_nvfp4_gemm_skinny_static(const void* X, const void* X_sc, const float* X_sg, const void* W, const void* W_sc,
                                            const float* W_sg, void* D, int64_t ldd, int M, int N, int K, void* stream) {
    using namespace tkb;
    if (!X || !X_sc || !X_sg || !W || !W_sc || !W_sg || !D) return api_fail(1, "gemm_skinny_static: null pointer");
    if (M < 1 || M > kStaticMaxM)
        return api_fail(1, "gemm_skinny_static: M=%d is outside 1..%d, the range the built-in %zu-byte scratch array is sized for; "
                           "use tkb_nvfp4_gemm for larger M", M, kStaticMaxM, kStaticScratchBytes);
    if (N < 1 || K < 64 || K % 64 || N % 8) return api_fail(1, "gemm_skinny_static: need N %% 8 == 0 and K a positive multiple of 64 (N=%d K=%d)", N, K);
    if (ldd == 0) ldd = N;
    if (ldd < N) return api_fail(1, "gemm_skinny_static: ldd must be >= N");
    // (M <= 16 stores D from registers: the output tensor map of the wider instances stays unset and is never touched)
    if ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(X_sc) | reinterpret_cast<uintptr_t>(W_sc)) & 15u)
        return api_fail(2, "gemm_skinny_static: operand and scale pointers must be 16-byte aligned");
    int dev = 0;
    cudaError_t ce = cudaGetDevice(&dev);
    if (ce != cudaSuccess) return api_fail(3, "gemm_skinny_static: cudaGetDevice failed: %s", cudaGetErrorString(ce));
    if (dev < 0 || dev >= kStaticMaxDevices) return api_fail(1, "gemm_skinny_static: device ordinal %d out of range", dev);
    StaticDev& sd = g_static_dev[dev];
    if (!sd.ready.load(std::memory_order_acquire)) {
        // First call on this device (it is the current device): resolve the device address of the scratch
        // array.  The array's name is only a host-side handle for the symbol, never a pointer a kernel can use.
        std::lock_guard<std::mutex> lk(g_static_mu);
        if (!sd.ready.load(std::memory_order_relaxed)) {
            void* p = nullptr;
            ce = cudaGetSymbolAddress(&p, g_static_scratch);
            if (ce != cudaSuccess || !p) return api_fail(3, "gemm_skinny_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(ce));
            int major = 0, sms = 0;
            ce = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
            if (ce == cudaSuccess) ce = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            if (ce != cudaSuccess) return api_fail(3, "gemm_skinny_static: cudaDeviceGetAttribute failed: %s", cudaGetErrorString(ce));
            if (major != 10) return api_fail(5, "gemm_skinny_static: device %d is not sm_100", dev);
            if (!g_static_encode) {
                void* fn = nullptr;
                cudaDriverEntryPointQueryResult q;
                ce = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
                if (ce != cudaSuccess || !fn || q != cudaDriverEntryPointSuccess) return api_fail(5, "gemm_skinny_static: cuTensorMapEncodeTiled is unavailable");
                g_static_encode = reinterpret_cast<EncodeFn>(fn);
            }
            sd.scratch = static_cast<unsigned char*>(p);
            sd.sm_count = sms;
            sd.ready.store(true, std::memory_order_release);       // publishes scratch and sm_count
        }
    }
    DecodeArgs a;
    memset(&a, 0, sizeof(a));
    if (!encode_2d(&a.tmW, W, uint64_t(K / 2), uint64_t(N), 128) || !encode_2d(&a.tmX, X, uint64_t(K / 2), uint64_t(M), 16) ||
        !encode_scales(&a.tmSW, W_sc, uint64_t((N + 127) / 128), uint64_t(K / 64)) || !encode_scales(&a.tmSX, X_sc, 1, uint64_t(K / 64)))
        return api_fail(3, "gemm_skinny_static: cuTensorMapEncodeTiled failed");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    unsigned int* flags = reinterpret_cast<unsigned int*>(sd.scratch + kStaticPartialBytes);
    // The array keeps whatever the previous call left in it.  Partial tiles are always written before they
    // are read, but a flag still holding the value 1 would be taken for "already published": clear them.
    ce = cudaMemsetAsync(flags, 0, kStaticFlagBytes, s);
    if (ce != cudaSuccess) return api_fail(3, "gemm_skinny_static: cudaMemsetAsync failed: %s", cudaGetErrorString(ce));
    a.sgX = X_sg; a.sgW = W_sg; a.D = D; a.ldd = ldd; a.M = M; a.N = N; a.K = K;
    a.partials = reinterpret_cast<float*>(sd.scratch); a.flags = flags; a.epoch = 1; a.max_grid = kStaticMaxGrid;
    a.status = nullptr; a.sm_count = sd.sm_count; a.stream = s;
    a.prefetch_weights = 0;
    ce = launch_decode(a);
    if (ce != cudaSuccess) return api_fail(3, "gemm_skinny_static: launch failed: %s", cudaGetErrorString(ce));
    return 0;
}
