// MoE layer pieces around the grouped expert GEMM: routing, dispatch schedule, combine, and the entry point of
// the fused dispatch + grouped NVFP4 GEMM (the kernel itself is the MoE mode of gemm.cu).
//
// Replaces the reference's moe_dispatch_gemm path (kernels/parallel/moe_dispatch_gemm/moe_dispatch_gemm_h100.cu:
// 13-293, Hopper/wgmma only, bf16 rows and weights) and the schedule that its benchmark builds on the CPU in
// Python loops (moe_dispatch_gemm/benchmark.py:112-166).  Differences that matter to a caller:
//   * everything data-dependent stays on the device: expert counts, padded segment sizes, the pull list, the
//     number of row blocks and the combine map are produced by two small kernels, so a layer needs no host
//     synchronisation;
//   * rows travel as NVFP4 codes followed by their e4m3 scales (one 4032-byte row per 7168-wide token instead of
//     14336 bytes of bf16) and are pulled straight into the grouped GEMM's operand buffers by some CTAs of the GEMM kernel;
//   * within an expert segment rows are in ascending global token order (the reference walks source ranks as a
//     ring starting at the local rank); segments are padded to 128 rows with (-1, -1) entries as in the reference;
//   * combine (no counterpart in the reference): out[t] = bf16(sum_j w[t,j] * Y[row(t,j)]), fp32 accumulation in
//     ascending j, rows read from the expert ranks over NVLink.
#include <atomic>
#include <cstring>
#include "../../include/tkb200.h"
#include "internal.h"
#include "ptx.cuh"

namespace tkb {

int api_fail(int code, const char* fmt, ...);
int api_device(int* sm_count, int** status);
unsigned long long* api_profile_buffer();             // api.cu: tkb_gemm_set_profile_buffer
int api_small_scratch(size_t bytes, void** ptr);      // api.cu: library-owned temporaries, null when too large
int api_make_gemm_maps(GemmArgs* g, int kind, const void* A, int64_t lda_bytes, const void* A_sc, const void* B, int64_t ldb_bytes,
                       const void* B_sc, void* D, int64_t ldd, int M, int N, int K);

// ------------------------------------------------------------------------------ routing ------
// softmax over E logits, top-k by probability (ties -> lower expert id), weights renormalised over the k.
// One warp per token; E % 32 == 0, E <= 256.
template <int PER>
__global__ void moe_route_kernel(const float* __restrict__ logits, int T, int top_k, int* __restrict__ experts, float* __restrict__ weights) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= T) return;
    constexpr int E = PER * 32;
    float p[PER];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < PER; i++) { p[i] = logits[size_t(warp) * E + i * 32 + lane]; mx = fmaxf(mx, p[i]); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    // sum in expert order (lane-major within each group of 32) so that it is the same on every launch
#pragma unroll
    for (int i = 0; i < PER; i++) { p[i] = expf(p[i] - mx); }
#pragma unroll
    for (int i = 0; i < PER; i++) {
        float s = p[i];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        sum += s;
    }
#pragma unroll
    for (int i = 0; i < PER; i++) p[i] = __fdiv_rn(p[i], sum);
    unsigned used = 0;
    float wsum = 0.f, myw = 0.f; int mye = 0;
    for (int j = 0; j < top_k; j++) {
        float best = -1.f; int bi = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < PER; i++)
            if (!(used & (1u << i)) && p[i] > best) { best = p[i]; bi = i * 32 + lane; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        if ((bi & 31) == lane) used |= 1u << (bi >> 5);
        wsum += best;
        if (lane == j) { myw = best; mye = bi; }
    }
    if (lane < top_k) {
        experts[size_t(warp) * top_k + lane] = mye;
        weights[size_t(warp) * top_k + lane] = __fdiv_rn(myw, wsum);
    }
}

// ------------------------------------------------------------------------------ schedule -----
// CTA e walks the whole (token, slot) -> expert list.  Warp w owns the contiguous span w of the list, so
// positions come out in ascending list order without any block-wide synchronisation inside the loops.
__device__ __forceinline__ int span_len(int total) { return ((total + 31) / 32 + 31) / 32 * 32; }

__global__ void __launch_bounds__(1024) moe_count_kernel(const int* __restrict__ experts_all, int total, int* __restrict__ counts,
                                                        int* __restrict__ padded) {
    __shared__ int s_cnt[32];
    const int e = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int span = span_len(total), lo = warp * span, hi = min(total, lo + span);
    int c = 0;
    for (int i = lo + lane; i < hi + ((32 - (hi - lo) % 32) % 32); i += 32)
        c += __popc(__ballot_sync(0xffffffffu, i < hi && experts_all[i] == e));
    if (lane == 0) s_cnt[warp] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = 0;
        for (int w = 0; w < 32; w++) t += s_cnt[w];
        counts[e] = t;
        padded[e] = (t + 127) / 128 * 128;
    }
}

__global__ void __launch_bounds__(1024)
moe_assign_kernel(const int* __restrict__ experts_all, int total, int top_k, int E, int world, int rank, int tokens_per_rank,
                  const int* __restrict__ counts, const int* __restrict__ padded, int* __restrict__ pull_idx, int* __restrict__ block_expert,
                  int* __restrict__ num_blocks, int* __restrict__ comb_idx, int cap_rows, int* status) {
    __shared__ int s_cnt[32];
    __shared__ int s_base[33];
    const int e = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e_per = E / world, owner = e / e_per, e_local = e % e_per;
    int seg = 0;
    for (int x = owner * e_per; x < e; x++) seg += padded[x];
    const int span = span_len(total), lo = warp * span, hi = min(total, lo + span);
    const int hi_pad = hi + ((32 - (hi - lo) % 32) % 32);
    int c = 0;
    for (int i = lo + lane; i < hi_pad; i += 32) c += __popc(__ballot_sync(0xffffffffu, i < hi && experts_all[i] == e));
    if (lane == 0) s_cnt[warp] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = 0;
        for (int w = 0; w < 32; w++) { s_base[w] = t; t += s_cnt[w]; }
        s_base[32] = t;
    }
    __syncthreads();
    const bool mine = owner == rank;
    const bool fits = seg + padded[e] <= cap_rows;
    if (mine && !fits && threadIdx.x == 0 && status) atomicExch(status, 6 /* capacity */);
    int run = s_base[warp];
    for (int i = lo + lane; i < hi_pad; i += 32) {
        const bool hit = i < hi && experts_all[i] == e;
        const unsigned b = __ballot_sync(0xffffffffu, hit);
        if (hit) {
            const int pos = run + __popc(b & ((1u << lane) - 1u));
            const int tok = i / top_k;
            if (mine && fits) {
                pull_idx[2 * (seg + pos)] = tok / tokens_per_rank;
                pull_idx[2 * (seg + pos) + 1] = tok % tokens_per_rank;
            }
            if (tok / tokens_per_rank == rank) {
                const int li = (tok % tokens_per_rank) * top_k + i % top_k;
                comb_idx[2 * li] = owner;
                comb_idx[2 * li + 1] = seg + pos;
            }
        }
        run += __popc(b);
    }
    if (mine && fits) {
        for (int r = counts[e] + threadIdx.x; r < padded[e]; r += blockDim.x) { pull_idx[2 * (seg + r)] = -1; pull_idx[2 * (seg + r) + 1] = -1; }
        for (int b = threadIdx.x; b < padded[e] / 128; b += blockDim.x) block_expert[seg / 128 + b] = e_local;
    }
    if (mine && e_local == 0 && threadIdx.x == 0) {
        int t = 0;
        for (int x = owner * e_per; x < (owner + 1) * e_per; x++) t += padded[x];
        *num_blocks = t <= cap_rows ? t / 128 : 0;
    }
}

// ------------------------------------------------------------------------------ schedule as a counting sort ----
// The same schedule as moe_count_kernel + moe_assign_kernel: the (token, slot) -> expert list is cut into chunks of
// 1024 entries (one CTA each, one entry per thread); (1) every chunk counts its entries per expert, (2) one CTA per
// expert turns its row of counts into per-chunk starting positions (block scan) and the padded segment size, (3) every
// chunk ranks its entries among the earlier entries of the same expert (warps in order, lanes in order) and writes the
// pull list and the combine map; the first CTAs also write this rank's block table, its padding rows and the block
// count.  Positions are in ascending list order, exactly as the expert-per-CTA kernels produce them, but the list is
// read twice instead of 2 * E times.
constexpr int kSchedChunk = 1024;

__global__ void __launch_bounds__(kSchedChunk)
moe_sched_hist_kernel(const int* __restrict__ experts_all, int total, int E, int nchunks, int* __restrict__ hist /* [E][nchunks] */) {
    __shared__ int s_cnt[256];
    for (int e = threadIdx.x; e < E; e += blockDim.x) s_cnt[e] = 0;
    __syncthreads();
    const int i = blockIdx.x * kSchedChunk + threadIdx.x;
    if (i < total) atomicAdd(&s_cnt[experts_all[i]], 1);
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) hist[size_t(e) * nchunks + blockIdx.x] = s_cnt[e];
}

// CTA e: exclusive prefix of expert e's per-chunk counts (nchunks <= 1024 * 32 handled in rounds of blockDim.x)
__global__ void __launch_bounds__(1024)
moe_sched_scan_kernel(int* __restrict__ hist, int nchunks, int* __restrict__ counts, int* __restrict__ padded) {
    __shared__ int s_warp[32];
    __shared__ int s_carry;
    const int e = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int* row = hist + size_t(e) * nchunks;
    if (threadIdx.x == 0) s_carry = 0;
    __syncthreads();
    for (int c0 = 0; c0 < nchunks; c0 += blockDim.x) {
        const int c = c0 + threadIdx.x;
        const int v = c < nchunks ? row[c] : 0;
        int incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += t;
        }
        if (lane == 31) s_warp[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            int w = s_warp[lane];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, w, o);
                if (lane >= o) w += t;
            }
            s_warp[lane] = w;
        }
        __syncthreads();
        const int carry = s_carry;
        if (c < nchunks) row[c] = carry + incl - v + (warp > 0 ? s_warp[warp - 1] : 0);
        __syncthreads();
        if (threadIdx.x == 0) s_carry = carry + s_warp[31];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        const int total = s_carry;
        counts[e] = total;
        padded[e] = (total + 127) / 128 * 128;
    }
}

__global__ void __launch_bounds__(kSchedChunk)
moe_sched_assign_kernel(const int* __restrict__ experts_all, int total, int top_k, int E, int world, int rank, int tokens_per_rank,
                        const int* __restrict__ hist /* per-chunk starts, [E][nchunks] */, int nchunks, const int* __restrict__ counts,
                        const int* __restrict__ padded, int* __restrict__ pull_idx, int* __restrict__ block_expert, int* __restrict__ num_blocks,
                        int* __restrict__ comb_idx, int cap_rows, int* status) {
    __shared__ int s_warp_cnt[32][256];
    __shared__ int s_seg[256];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int e_per = E / world;
    // start of every expert's segment inside its owner's buffer
    for (int x = threadIdx.x; x < E; x += blockDim.x) {
        int seg = 0;
        for (int y = (x / e_per) * e_per; y < x; y++) seg += padded[y];
        s_seg[x] = seg;
    }
    for (int x = lane; x < E; x += 32) s_warp_cnt[warp][x] = 0;
    __syncthreads();
    // this rank's experts, dealt to the first CTAs: block table and padding rows; CTA 0: block count / capacity error
    for (int x = rank * e_per + blockIdx.x; x < (rank + 1) * e_per; x += gridDim.x) {
        const int seg = s_seg[x], pad = padded[x];
        if (seg + pad <= cap_rows) {
            for (int r = counts[x] + threadIdx.x; r < pad; r += blockDim.x) { pull_idx[2 * (seg + r)] = -1; pull_idx[2 * (seg + r) + 1] = -1; }
            for (int b = threadIdx.x; b < pad / 128; b += blockDim.x) block_expert[seg / 128 + b] = x - rank * e_per;
        }
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        int t = 0;
        for (int x = rank * e_per; x < (rank + 1) * e_per; x++) t += padded[x];
        *num_blocks = t <= cap_rows ? t / 128 : 0;
        if (t > cap_rows && status) atomicExch(status, 6 /* capacity */);
    }
    const int i = blockIdx.x * kSchedChunk + threadIdx.x;
    const bool live = i < total;
    const int e = live ? experts_all[i] : -1 - lane;                      // dead lanes match nobody
    const unsigned same = __match_any_sync(0xffffffffu, e);
    const int rank_in_warp = __popc(same & ((1u << lane) - 1u));
    if (live && rank_in_warp == 0) s_warp_cnt[warp][e] = __popc(same);    // first lane of each group
    __syncthreads();
    if (!live) return;
    int before = 0;
    for (int w = 0; w < warp; w++) before += s_warp_cnt[w][e];
    const int pos = hist[size_t(e) * nchunks + blockIdx.x] + before + rank_in_warp;
    const int owner = e / e_per, seg = s_seg[e];
    const int tok = i / top_k;
    if (owner == rank && seg + padded[e] <= cap_rows) {
        pull_idx[2 * (seg + pos)] = tok / tokens_per_rank;
        pull_idx[2 * (seg + pos) + 1] = tok % tokens_per_rank;
    }
    if (tok / tokens_per_rank == rank) {
        const int li = (tok % tokens_per_rank) * top_k + i % top_k;
        comb_idx[2 * li] = owner;
        comb_idx[2 * li + 1] = seg + pos;
    }
}

// ------------------------------------------------------------------------------ gather ------
// Dispatch as a kernel of its own (comm_ctas == 0 in tkb_moe_dispatch_gemm): every SM pulls routed rows, instead of a few
// CTAs inside the GEMM kernel.  One CTA per 128-row block of the local operand buffer at a time: the block's (source
// rank, source row) pairs are read from the pull list, the rows' codes are copied with 16-byte loads (NVLink for remote
// rows, up to 8 in flight per thread) into the operand rows, the rows' scales are dropped into the 512-byte chunk layout
// in shared memory and stored as one contiguous span; then the block's arrival epoch is published, on which the GEMM's
// producers wait.  Padding rows (-1) become zeros.
struct PeerRowBytes { const uint8_t* p[kMaxWorld]; };

__device__ __forceinline__ uint4 ld_cg_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_cg_u32(const void* p) {
    uint32_t v;
    asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

__global__ void __launch_bounds__(512)
moe_gather_kernel(PeerRowBytes rows, const int* __restrict__ pull_idx, const int* __restrict__ num_blocks, uint8_t* __restrict__ codes,
                  uint8_t* __restrict__ scales, unsigned int* arrived, const unsigned int* ready, unsigned int epoch, int k_bytes,
                  int sc_row_bytes, int world, int rank, int* status, long long limit) {
    extern __shared__ __align__(16) uint8_t s_sc[];          // [sc_row_bytes / 4][512]: the block's scales as stored
    __shared__ int s_idx[256];
    __shared__ int s_ok;
    const int tid = threadIdx.x, nthr = blockDim.x;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (tid == 0) {
        // the peers' tokens of this call are quantized (their kernels signalled it)
        int ok = 1;
        const long long t0 = clock64();
        for (int pr = 0; pr < world && ok; pr++) {
            if (pr == rank) continue;
            while (true) {
                unsigned int v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(ready + pr) : "memory");
                if (int(v - epoch) >= 0) break;
                if (clock64() - t0 > limit) { ok = 0; if (status) atomicExch(status, (int)TKB_DEV_TIMEOUT); break; }
                __nanosleep(100);
            }
        }
        s_ok = ok;
    }
    __syncthreads();
    if (!s_ok) return;
    const int nb = *num_blocks;
    const int row_bytes = k_bytes + sc_row_bytes;
    const int k16 = k_bytes / 16, words = sc_row_bytes / 4;
    const int sc_block_bytes = sc_row_bytes * 128;
    constexpr int UNROLL = 8;
    for (int blk = blockIdx.x; blk < nb; blk += gridDim.x) {
        __syncthreads();                                     // the previous block's staging has been stored
        if (tid < 256) s_idx[tid] = pull_idx[size_t(blk) * 256 + tid];
        __syncthreads();
        // codes: 128 x k16 pieces of 16 bytes, consecutive threads on consecutive pieces of a row
        const int pieces = 128 * k16;
        for (int base = tid; base < pieces; base += nthr * UNROLL) {
            uint4 v[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; u++) {
                const int pc = base + u * nthr;
                v[u] = make_uint4(0, 0, 0, 0);
                if (pc < pieces) {
                    const int r = pc / k16, c = pc - r * k16;
                    const int src = s_idx[2 * r];
                    if (src >= 0) v[u] = ld_cg_v4(rows.p[src] + size_t(s_idx[2 * r + 1]) * row_bytes + size_t(c) * 16);
                }
            }
#pragma unroll
            for (int u = 0; u < UNROLL; u++) {
                const int pc = base + u * nthr;
                if (pc < pieces) {
                    const int r = pc / k16, c = pc - r * k16;
                    *reinterpret_cast<uint4*>(codes + (size_t(blk) * 128 + r) * k_bytes + size_t(c) * 16) = v[u];
                }
            }
        }
        // scales: one 32-bit word (64 K-elements) per row and chunk
        const int nwords = 128 * words;
        for (int base = tid; base < nwords; base += nthr * UNROLL) {
            uint32_t v[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; u++) {
                const int w = base + u * nthr;
                v[u] = 0u;
                if (w < nwords) {
                    const int r = w / words, kc = w - r * words;
                    const int src = s_idx[2 * r];
                    if (src >= 0) v[u] = ld_cg_u32(rows.p[src] + size_t(s_idx[2 * r + 1]) * row_bytes + k_bytes + size_t(kc) * 4);
                }
            }
#pragma unroll
            for (int u = 0; u < UNROLL; u++) {
                const int w = base + u * nthr;
                if (w < nwords) {
                    const int r = w / words, kc = w - r * words;
                    *reinterpret_cast<uint32_t*>(s_sc + size_t(kc) * 512 + (r & 31) * 16 + (r >> 5) * 4) = v[u];
                }
            }
        }
        __syncthreads();
        for (int i = tid; i < sc_block_bytes / 16; i += nthr)
            reinterpret_cast<uint4*>(scales + size_t(blk) * sc_block_bytes)[i] = reinterpret_cast<const uint4*>(s_sc)[i];
        __threadfence();
        __syncthreads();
        if (tid == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(arrived + blk), "r"(epoch) : "memory");
    }
}

// ------------------------------------------------------------------------------ combine ------
struct PeerRows { const __nv_bfloat16* p[kMaxWorld]; };

__global__ void __launch_bounds__(256)
moe_combine_kernel(PeerRows Y, int64_t ldy, const int* __restrict__ comb_idx, const float* __restrict__ weights, int top_k, int I,
                   __nv_bfloat16* __restrict__ out) {
    const int t = blockIdx.x;
    for (int v = threadIdx.x; v < I / 8; v += blockDim.x) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int j0 = 0; j0 < top_k; j0 += 4) {
            uint4 q[4]; float w[4];
#pragma unroll
            for (int jj = 0; jj < 4; jj++) {
                const int j = j0 + jj;
                if (j < top_k) {
                    const int dst = comb_idx[2 * (t * top_k + j)], row = comb_idx[2 * (t * top_k + j) + 1];
                    w[jj] = weights[t * top_k + j];
                    q[jj] = __ldcg(reinterpret_cast<const uint4*>(Y.p[dst] + int64_t(row) * ldy + v * 8));
                } else { w[jj] = 0.f; q[jj] = make_uint4(0, 0, 0, 0); }
            }
#pragma unroll
            for (int jj = 0; jj < 4; jj++) {
                const uint32_t u[4] = {q[jj].x, q[jj].y, q[jj].z, q[jj].w};
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    acc[2 * k] = fmaf(w[jj], __uint_as_float(u[k] << 16), acc[2 * k]);
                    acc[2 * k + 1] = fmaf(w[jj], __uint_as_float(u[k] & 0xffff0000u), acc[2 * k + 1]);
                }
            }
        }
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]); o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
        *reinterpret_cast<uint4*>(out + int64_t(t) * I + v * 8) = o;
    }
}

} // namespace tkb

using namespace tkb;

#define TKB_CUDA_M(expr)                                                                                      \
    do {                                                                                                      \
        cudaError_t _e = (expr);                                                                              \
        if (_e != cudaSuccess) return api_fail(TKB_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
    } while (0)

extern "C" {

int tkb_moe_route(const float* logits, int T, int E, int top_k, int* experts, float* weights, void* stream) {
    if (!logits || !experts || !weights) return api_fail(TKB_ERR_INVALID_ARG, "moe_route: null pointer");
    if (T < 1 || E % 32 || E < 32 || E > 256 || top_k < 1 || top_k > 32 || top_k > E)
        return api_fail(TKB_ERR_INVALID_ARG, "moe_route: need E in {32,..,256} (multiple of 32) and 1 <= top_k <= 32");
    int sm; int* status;
    if (int e = api_device(&sm, &status)) return e;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int blocks = (T + 7) / 8;
    switch (E / 32) {
        case 1: moe_route_kernel<1><<<blocks, 256, 0, s>>>(logits, T, top_k, experts, weights); break;
        case 2: moe_route_kernel<2><<<blocks, 256, 0, s>>>(logits, T, top_k, experts, weights); break;
        case 3: moe_route_kernel<3><<<blocks, 256, 0, s>>>(logits, T, top_k, experts, weights); break;
        case 4: moe_route_kernel<4><<<blocks, 256, 0, s>>>(logits, T, top_k, experts, weights); break;
        case 5: moe_route_kernel<5><<<blocks, 256, 0, s>>>(logits, T, top_k, experts, weights); break;
        case 6: moe_route_kernel<6><<<blocks, 256, 0, s>>>(logits, T, top_k, experts, weights); break;
        case 7: moe_route_kernel<7><<<blocks, 256, 0, s>>>(logits, T, top_k, experts, weights); break;
        default: moe_route_kernel<8><<<blocks, 256, 0, s>>>(logits, T, top_k, experts, weights); break;
    }
    TKB_CUDA_M(cudaGetLastError());
    return TKB_OK;
}

int tkb_moe_schedule(const int* experts_all, int T, int top_k, int E, int world, int rank, int* counts, int* padded_per_expert,
                     int* pull_idx, int* block_expert, int* num_blocks, int* comb_idx, int cap_rows, void* stream) {
    if (!experts_all || !counts || !padded_per_expert || !pull_idx || !block_expert || !num_blocks || !comb_idx)
        return api_fail(TKB_ERR_INVALID_ARG, "moe_schedule: null pointer");
    if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world || E < 1 || T < 1 || E % world || T % world || cap_rows % 128 || top_k < 1)
        return api_fail(TKB_ERR_INVALID_ARG, "moe_schedule: E and T must divide by world (<= %d), cap_rows by 128", kMaxWorld);
    int sm; int* status;
    if (int e = api_device(&sm, &status)) return e;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // counting-sort schedule when its temporaries (per-chunk counts) fit the library's scratch
    const int total = T * top_k, nchunks = (total + kSchedChunk - 1) / kSchedChunk;
    void* scratch = nullptr;
    if (E <= 256)
        if (int e = api_small_scratch(size_t(nchunks) * E * sizeof(int), &scratch)) return e;
    if (scratch) {
        int* hist = static_cast<int*>(scratch);
        moe_sched_hist_kernel<<<nchunks, kSchedChunk, 0, s>>>(experts_all, total, E, nchunks, hist);
        moe_sched_scan_kernel<<<E, 1024, 0, s>>>(hist, nchunks, counts, padded_per_expert);
        moe_sched_assign_kernel<<<nchunks, kSchedChunk, 0, s>>>(experts_all, total, top_k, E, world, rank, T / world, hist, nchunks, counts,
                                                                padded_per_expert, pull_idx, block_expert, num_blocks, comb_idx, cap_rows, status);
        TKB_CUDA_M(cudaGetLastError());
        return TKB_OK;
    }
    moe_count_kernel<<<E, 1024, 0, s>>>(experts_all, T * top_k, counts, padded_per_expert);
    moe_assign_kernel<<<E, 1024, 0, s>>>(experts_all, T * top_k, top_k, E, world, rank, T / world, counts, padded_per_expert, pull_idx,
                                         block_expert, num_blocks, comb_idx, cap_rows, status);
    TKB_CUDA_M(cudaGetLastError());
    return TKB_OK;
}

int tkb_moe_dispatch_gemm(void* const* peer_rows, const float* X_sg, void* codes, void* scales,
                          const void* W, const void* W_sc, const float* W_sg, void* Y, int64_t ldy, const int* pull_idx,
                          const int* block_expert, const int* num_blocks, const void* ready, void* arrived, unsigned int epoch, int K,
                          int I, int experts_local, int cap_rows, int rank, int world, int comm_ctas, void* stream) {
    if (!peer_rows || !X_sg || !codes || !scales || !W || !W_sc || !W_sg || !Y || !pull_idx || !block_expert ||
        !num_blocks || !ready || !arrived)
        return api_fail(TKB_ERR_INVALID_ARG, "moe_dispatch_gemm: null pointer");
    if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world) return api_fail(TKB_ERR_INVALID_ARG, "moe_dispatch_gemm: bad rank/world");
    if (K < 256 || K % 256 || I < 128 || I % 128 || cap_rows % 128 || cap_rows < 128)
        return api_fail(TKB_ERR_INVALID_ARG, "moe_dispatch_gemm: need K %% 256 == 0, I %% 128 == 0, cap_rows %% 128 == 0");
    int sm; int* status;
    if (int e = api_device(&sm, &status)) return e;
    // dispatch staging per comm CTA: a block's scales (128 x K/16 bytes), a zero row and a ring of row slots of which 16 trail the
    // loads (two batches whose stores may still read them), so at least 24 are needed to keep a batch of 8 loads in flight;
    // one thread per 64 K-elements
    if (comm_ctas > 0 && (moe_dispatch_ring(K) < 24 || K / 64 + 1 > 320))
        return api_fail(TKB_ERR_INVALID_ARG, "moe_dispatch_gemm: K=%d is too large for the dispatch staging in shared memory (%d row slots, 24 needed)",
                        K, moe_dispatch_ring(K));
    if (comm_ctas < 0 || comm_ctas > sm / 2) return api_fail(TKB_ERR_INVALID_ARG, "moe_dispatch_gemm: comm_ctas must be in [0, %d]", sm / 2);
    if (comm_ctas == 0) {
        // dispatch by a gather kernel on all SMs; the GEMM that follows waits on the per-block arrival epochs it publishes
        const size_t smem = size_t(K / 16) * 128;
        if (smem > 200 * 1024) return api_fail(TKB_ERR_INVALID_ARG, "moe_dispatch_gemm: K=%d is too large for the gather kernel's scale staging", K);
        static std::atomic<bool> attr_set[64] = {};
        int dev = 0;
        TKB_CUDA_M(cudaGetDevice(&dev));
        if (dev < 0 || dev >= 64 || !attr_set[dev].load(std::memory_order_acquire)) {
            TKB_CUDA_M(cudaFuncSetAttribute(moe_gather_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            if (dev >= 0 && dev < 64) attr_set[dev].store(true, std::memory_order_release);
        }
        PeerRowBytes pr;
        for (int i = 0; i < kMaxWorld; i++) pr.p[i] = i < world ? static_cast<const uint8_t*>(peer_rows[i]) : nullptr;
        const int per_sm = smem <= 100 * 1024 ? 2 : 1;
        int grid = cap_rows / 128 < sm * per_sm ? cap_rows / 128 : sm * per_sm;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid); cfg.blockDim = dim3(512); cfg.dynamicSmemBytes = smem; cfg.stream = static_cast<cudaStream_t>(stream);
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
        TKB_CUDA_M(cudaLaunchKernelEx(&cfg, moe_gather_kernel, pr, pull_idx, num_blocks, static_cast<uint8_t*>(codes), static_cast<uint8_t*>(scales),
                                      static_cast<unsigned int*>(arrived), static_cast<const unsigned int*>(ready), epoch, K / 2, K / 16, world, rank,
                                      status, api_wait_limit()));
    }
    if (ldy == 0) ldy = I;
    GemmArgs g;
    memset(&g, 0, sizeof(g));
    g.kind = KIND_NVFP4; g.config = 1;        // single CTA, N tile 256
    if (int e = api_make_gemm_maps(&g, KIND_NVFP4, codes, K / 2, scales, W, K / 2, W_sc, Y, ldy, cap_rows, I, K)) return e;
    // the B maps above cover one expert; rebuild them over the stacked experts
    GemmArgs gb;
    memset(&gb, 0, sizeof(gb));
    gb.kind = KIND_NVFP4; gb.config = 1;
    if (int e = api_make_gemm_maps(&gb, KIND_NVFP4, codes, K / 2, scales, W, K / 2, W_sc, Y, ldy, cap_rows, I * experts_local, K)) return e;
    g.tmB = gb.tmB; g.tmSB = gb.tmSB;
    g.sgA = X_sg; g.sgB = W_sg; g.M = cap_rows; g.N = I; g.K = K; g.status = status; g.sm_count = sm;
    g.stream = static_cast<cudaStream_t>(stream);
    g.mode = MODE_MOE;
    g.prof = api_profile_buffer();
    MoeParams& m = g.comm.moe;
    for (int i = 0; i < world; i++) m.peer_rows[i] = static_cast<const uint8_t*>(peer_rows[i]);
    m.codes = static_cast<uint8_t*>(codes); m.scales = static_cast<uint8_t*>(scales);
    m.pull_idx = pull_idx; m.block_expert = block_expert; m.num_blocks = num_blocks;
    m.ready = static_cast<const unsigned int*>(ready); m.arrived = static_cast<unsigned int*>(arrived);
    m.epoch = epoch; m.rank = rank; m.world = world; m.comm_ctas = comm_ctas; m.expert_rows = I;
    TKB_CUDA_M(launch_gemm(g));
    return TKB_OK;
}

int tkb_moe_combine(void* const* peer_Y, int64_t ldy, const int* comb_idx, const float* weights, void* out, int T_local, int top_k, int I,
                    int world, void* stream) {
    if (!peer_Y || !comb_idx || !weights || !out) return api_fail(TKB_ERR_INVALID_ARG, "moe_combine: null pointer");
    if (world < 1 || world > kMaxWorld || I % 8 || T_local < 1) return api_fail(TKB_ERR_INVALID_ARG, "moe_combine: bad arguments");
    if (ldy == 0) ldy = I;
    PeerRows pr;
    for (int i = 0; i < kMaxWorld; i++) pr.p[i] = i < world ? static_cast<const __nv_bfloat16*>(peer_Y[i]) : nullptr;
    moe_combine_kernel<<<T_local, 256, 0, static_cast<cudaStream_t>(stream)>>>(pr, ldy, comb_idx, weights, top_k, I, static_cast<__nv_bfloat16*>(out));
    TKB_CUDA_M(cudaGetLastError());
    return TKB_OK;
}

int tkb_moe_layer_nvfp4(const tkb_moe_state* st, unsigned int epoch, const float* logits_local, const void* X_local, const void* W,
                        const void* W_sc, const float* W_sg, void* out, int comm_ctas, int arithmetic, void* stream) {
    if (!st || !logits_local || !X_local || !W || !W_sc || !W_sg || !out || epoch == 0)
        return api_fail(TKB_ERR_INVALID_ARG, "moe_layer: null pointer or epoch 0");
    const int w = st->world, r = st->rank, b = int(epoch % 2u);
    if (w < 1 || w > kMaxWorld || r < 0 || r >= w || st->T % w || st->E % w) return api_fail(TKB_ERR_INVALID_ARG, "moe_layer: bad world / rank / T / E");
    const int Tl = st->T / w, El = st->E / w;
    // flag array of every rank: [0, w) tokens quantized ("ready"), [w, 2w) expert outputs complete, [2w, 3w) layer call finished
    unsigned int* fl = static_cast<unsigned int*>(st->flags[r]);
    if (int e = tkb_moe_route(logits_local, Tl, st->E, st->top_k, static_cast<int*>(st->experts_local), static_cast<float*>(st->weights), stream)) return e;
    // everything of parity b was last used by call epoch - 2: every peer must have finished that call before it is overwritten
    if (w > 1 && epoch > 2)
        if (int e = tkb_wait_flags(fl + 2 * w, w, r, epoch - 2, stream)) return e;
    if (int e = tkb_all_to_all(st->experts_all[b], st->experts_local, size_t(Tl) * st->top_k * 4, 1, r, w, st->counters, b * w, (epoch + 1) / 2, stream))
        return e;
    if (int e = tkb_moe_schedule(static_cast<const int*>(st->experts_all[b][r]), st->T, st->top_k, st->E, w, r, static_cast<int*>(st->counts),
                                 static_cast<int*>(st->padded), static_cast<int*>(st->pull_idx), static_cast<int*>(st->block_expert),
                                 static_cast<int*>(st->num_blocks), static_cast<int*>(st->comb_idx), st->cap_rows, stream)) return e;
    // this rank's tokens, quantized with the amax of all tokens (exchanged inside the kernel), as self-contained rows
    if (int e = tkb_nvfp4_quantize_sharded(X_local, 0, st->xq_rows[b][r], nullptr, st->sg, Tl, st->H, 1, arithmetic, st->slots[b], w, r, epoch, stream))
        return e;
    if (w > 1) {
        if (int e = tkb_signal_peers(st->flags, w, r, r, epoch, 0, stream)) return e;
        // Y is rewritten below: every peer must have finished combining the previous call from it
        if (epoch > 1)
            if (int e = tkb_wait_flags(fl + 2 * w, w, r, epoch - 1, stream)) return e;
    }
    if (int e = tkb_moe_dispatch_gemm(st->xq_rows[b], st->sg, st->codes, st->scales, W, W_sc, W_sg, st->Y[r], 0, static_cast<const int*>(st->pull_idx),
                                      static_cast<const int*>(st->block_expert), static_cast<const int*>(st->num_blocks), fl, st->arrived, epoch,
                                      st->H, st->I, El, st->cap_rows, r, w, comm_ctas, stream)) return e;
    if (w > 1) {
        if (int e = tkb_signal_peers(st->flags, w, r, w + r, epoch, 0, stream)) return e;      // my expert outputs are complete
        if (int e = tkb_wait_flags(fl + w, w, r, epoch, stream)) return e;                    // everybody's are
    }
    if (int e = tkb_moe_combine(st->Y, 0, static_cast<const int*>(st->comb_idx), static_cast<const float*>(st->weights), out, Tl, st->top_k, st->I, w, stream))
        return e;
    if (w > 1)
        if (int e = tkb_signal_peers(st->flags, w, r, 2 * w + r, epoch, 0, stream)) return e;   // done with the peers' tokens and outputs
    return TKB_OK;
}

} // extern "C"
