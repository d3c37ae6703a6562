// Single-node multi-GPU plumbing and the collective-fused entry points of the C ABI.
//
// Replaces, for the hot path only, what the reference builds from TKParallelTensor / KittensBroker
// (include/pyutils/parallel_tensor.cuh:23-336, broker.cuh:340-547: VMM allocations exchanged as POSIX
// file descriptors over unix sockets, optional NVSwitch multicast object) and its device-side
// signal / wait / barrier helpers (include/ops/thread/util/sync.cuh:296-327).  Here:
//   * symmetric buffers are plain cudaMalloc allocations exported with CUDA IPC handles; the 64-byte
//     handles travel through whatever channel the host program already has (torch.distributed in the
//     Python layer), so there are no fixed shared-memory or socket names to collide on;
//   * flags are 32-bit epochs in those buffers, written across GPUs with system-scope release stores
//     and read with bounded acquire spins; nothing uses multicast or multimem.
#include <cstddef>
#include <cstring>
#include <new>
#include "../../include/tkb200.h"
#include "internal.h"
#include "ptx.cuh"
#include "ag_schedule.h"

namespace tkb {

int api_fail(int code, const char* fmt, ...);          // api.cu
int api_device(int* sm_count, int** status);
unsigned long long* api_profile_buffer();             // api.cu: tkb_gemm_set_profile_buffer           // api.cu
int api_quantize_sharded(const void* A_bf16, int64_t lda, void* codes, void* sc, float* sg, int M, int K, int layout, int arithmetic,
                         void* const* peer_slots, int world, int rank, unsigned int epoch, unsigned int* stamp, int stamp_count,
                         const unsigned int* epoch_ptr, void* stream);   // api.cu
int api_make_gemm_maps(GemmArgs* g, int kind, const void* A, int64_t lda_bytes, const void* A_sc, const void* B, int64_t ldb_bytes,
                       const void* B_sc, void* D, int64_t ldd, int M, int N, int K);   // api.cu
int api_make_output_map(CUtensorMap* m, void* D, int rows, int cols, int64_t ldd);     // api.cu: bf16 [rows, cols], box 64 x 32, 128-byte swizzle
int api_make_operand_a_maps(GemmArgs* g, const void* A, const void* A_sc, int M, int K);   // api.cu: NVFP4 A operand + scales over M rows

struct PeerPtrs { unsigned int* p[kMaxWorld]; };
constexpr int kAllToAll4dMaxGrid = 592;   // CTAs of tkb_all_to_all_4d at most (part of its counter protocol)
constexpr int kAgMaxCopyStreams = 4;
constexpr int kAllToAllParts = 4;      // CTAs per destination in tkb_all_to_all (part of its counter protocol)

__global__ void signal_peers_kernel(PeerPtrs peers, int world, int rank, int index, unsigned int value, int include_self) {
    const int t = threadIdx.x;
    if (t < world && (t != rank || include_self)) {
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peers.p[t] + index), "r"(value) : "memory");
    }
}

// Waits until every flags[i] (i != skip) has reached `value` (epochs only grow).
__global__ void wait_flags_kernel(const unsigned int* flags, int count, int skip, unsigned int value, int* status, long long limit) {
    const int t = threadIdx.x;
    if (t < count && t != skip) {
        const long long t0 = clock64();
        while (true) {
            unsigned int v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + t) : "memory");
            if (int(v - value) >= 0) break;
            if (clock64() - t0 > limit) {
                if (status) atomicExch(status, (int)TKB_DEV_TIMEOUT);
                break;
            }
            __nanosleep(100);
        }
    }
}

// Max all-reduce of one float across the ranks without a library collective: every rank stores (epoch, value
// bits) into slot[rank] of every peer's slot array and then waits (bounded) until all of its own slots carry the
// epoch.  About one NVLink round trip instead of a collective launch.
struct PeerSlots { unsigned long long* p[kMaxWorld]; };
__global__ void amax_allreduce_kernel(PeerSlots slots, int world, int rank, unsigned int epoch, const float* local, float* out, int* status, long long limit) {
    const int t = threadIdx.x;
    float v = 0.f;
    if (t < world) {
        const unsigned long long mine = (static_cast<unsigned long long>(epoch) << 32) | __float_as_uint(*local);
        asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(slots.p[t] + rank), "l"(mine) : "memory");
        const long long t0 = clock64();
        unsigned long long got;
        while (true) {
            asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(got) : "l"(slots.p[rank] + t) : "memory");
            if (int(unsigned(got >> 32) - epoch) >= 0) break;
            if (clock64() - t0 > limit) { if (status) atomicExch(status, (int)TKB_DEV_TIMEOUT); break; }
        }
        v = __uint_as_float(unsigned(got & 0xffffffffu));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if (t == 0) *out = v;
}

// Contiguous all-to-all by pushes: chunk p of `in` (bytes_per_peer each; the same chunk for everybody when
// `gather` is set) goes to offset rank * bytes_per_peer of peer p's output; each CTA then bumps a counter on the
// receiving side (system-scope release add).  blockIdx.y = destination, blockIdx.x = part of the chunk.
struct PeerBytes { unsigned char* p[kMaxWorld]; };
__global__ void all_to_all_push_kernel(PeerBytes out, const unsigned char* in, size_t bytes_per_peer, int gather, int rank, int world,
                                       PeerPtrs counters, int counter_base) {
    const int dst = blockIdx.y;
    const unsigned char* src = in + (gather ? 0 : size_t(dst) * bytes_per_peer);
    unsigned char* d = out.p[dst] + size_t(rank) * bytes_per_peer;
    const size_t per = (bytes_per_peer / 16 + gridDim.x - 1) / gridDim.x;       // 16-byte vectors per CTA
    const size_t v0 = size_t(blockIdx.x) * per, v1 = min(bytes_per_peer / 16, v0 + per);
    for (size_t v = v0 + threadIdx.x; v < v1; v += blockDim.x)
        reinterpret_cast<uint4*>(d)[v] = __ldg(reinterpret_cast<const uint4*>(src) + v);
    if (blockIdx.x == gridDim.x - 1)
        for (size_t b = (bytes_per_peer / 16) * 16 + threadIdx.x; b < bytes_per_peer; b += blockDim.x) d[b] = src[b];
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(counters.p[dst] + counter_base + rank), "r"(1u) : "memory");
    }
}

// General 4-D all-to-all (all_to_all::kernel<S,G>, kernels/parallel/all_to_all/all_to_all.cu:37-94): element
// (i0, i1, i2, i3) of this rank's input goes to rank i[S] / out[S], at index i[S] % out[S] along the scatter axis and
// i[G] + in[G] * rank along the gather axis (out[S] = in[S] / world, out[G] = in[G] * world).  Threads move 16-byte
// vectors along the innermost axis with plain loads (local) and stores (NVLink, posted); when a CTA is through, it
// bumps a counter on every rank (system-scope release add).
struct A2A4Params {
    unsigned char* out[kMaxWorld];
    unsigned int* counters[kMaxWorld];
    long long in_dims[4];        // innermost in 16-byte vectors
    long long out_dims[4];
    int scatter, gather, rank, world, counter_base;
};
__global__ void __launch_bounds__(256) all_to_all_4d_kernel(const unsigned char* __restrict__ in, const A2A4Params p) {
    const long long total = p.in_dims[0] * p.in_dims[1] * p.in_dims[2] * p.in_dims[3];
    for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < total; v += (long long)gridDim.x * blockDim.x) {
        long long idx[4], rest = v;
#pragma unroll
        for (int a = 3; a >= 0; a--) { idx[a] = rest % p.in_dims[a]; rest /= p.in_dims[a]; }
        const int dst = int(idx[p.scatter] / p.out_dims[p.scatter]);
        idx[p.scatter] %= p.out_dims[p.scatter];
        idx[p.gather] += p.in_dims[p.gather] * p.rank;
        const long long o = ((idx[0] * p.out_dims[1] + idx[1]) * p.out_dims[2] + idx[2]) * p.out_dims[3] + idx[3];
        reinterpret_cast<uint4*>(p.out[dst])[o] = __ldg(reinterpret_cast<const uint4*>(in) + v);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        for (int d = 0; d < p.world; d++)
            asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p.counters[d] + p.counter_base + p.rank), "r"(1u) : "memory");
    }
}
// All ranks have entered: one add per peer, then a bounded wait for everybody's.
__global__ void a2a_enter_kernel(PeerPtrs counters, int base, int rank, int world, unsigned int epoch, int* status, long long limit) {
    const int t = threadIdx.x;
    if (t < world) asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(counters.p[t] + base + rank), "r"(1u) : "memory");
    if (t < world) {
        const long long t0 = clock64();
        while (true) {
            unsigned int v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(counters.p[rank] + base + t) : "memory");
            if (int(v - epoch) >= 0) break;
            if (clock64() - t0 > limit) { if (status) atomicExch(status, (int)TKB_DEV_TIMEOUT); break; }
            __nanosleep(100);
        }
    }
}

} // namespace tkb

using namespace tkb;

#define TKB_CUDA_C(expr)                                                                                      \
    do {                                                                                                      \
        cudaError_t _e = (expr);                                                                              \
        if (_e != cudaSuccess) return api_fail(TKB_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
    } while (0)

extern "C" {

int tkb_dev_alloc(size_t bytes, void** ptr) {
    if (!ptr || bytes == 0) return api_fail(TKB_ERR_INVALID_ARG, "dev_alloc: null output or zero size");
    TKB_CUDA_C(cudaMalloc(ptr, bytes));
    TKB_CUDA_C(cudaMemset(*ptr, 0, bytes));
    TKB_CUDA_C(cudaDeviceSynchronize());
    return TKB_OK;
}
int tkb_dev_free(void* ptr) {
    TKB_CUDA_C(cudaFree(ptr));
    return TKB_OK;
}
int tkb_ipc_export(const void* ptr, void* handle64) {
    if (!ptr || !handle64) return api_fail(TKB_ERR_INVALID_ARG, "ipc_export: null pointer");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    cudaIpcMemHandle_t h;
    TKB_CUDA_C(cudaIpcGetMemHandle(&h, const_cast<void*>(ptr)));
    memcpy(handle64, &h, 64);
    return TKB_OK;
}
int tkb_ipc_open(const void* handle64, void** ptr) {
    if (!ptr || !handle64) return api_fail(TKB_ERR_INVALID_ARG, "ipc_open: null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    TKB_CUDA_C(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return TKB_OK;
}
int tkb_ipc_close(void* ptr) {
    TKB_CUDA_C(cudaIpcCloseMemHandle(ptr));
    return TKB_OK;
}

int tkb_signal_peers(void* const* peer_flags, int world, int rank, int index, unsigned int value, int include_self, void* stream) {
    if (!peer_flags || world < 1 || world > kMaxWorld || rank < 0 || rank >= world || index < 0)
        return api_fail(TKB_ERR_INVALID_ARG, "signal_peers: bad arguments (world must be 1..%d)", kMaxWorld);
    PeerPtrs pp;
    for (int i = 0; i < kMaxWorld; i++) pp.p[i] = i < world ? static_cast<unsigned int*>(peer_flags[i]) : nullptr;
    signal_peers_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(pp, world, rank, index, value, include_self);
    TKB_CUDA_C(cudaGetLastError());
    return TKB_OK;
}

int tkb_wait_flags(const void* flags, int count, int skip, unsigned int value, void* stream) {
    if (!flags || count < 1 || count > 1024) return api_fail(TKB_ERR_INVALID_ARG, "wait_flags: bad arguments");
    int sm; int* status;
    if (int e = api_device(&sm, &status)) return e;
    wait_flags_kernel<<<1, ((count + 31) / 32) * 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const unsigned int*>(flags), count, skip,
                                                                                         value, status, api_wait_limit());
    TKB_CUDA_C(cudaGetLastError());
    return TKB_OK;
}

int tkb_amax_allreduce(void* const* peer_slots, int world, int rank, unsigned int epoch, const float* local, float* out, void* stream) {
    if (!peer_slots || !local || !out || world < 1 || world > kMaxWorld || rank < 0 || rank >= world)
        return api_fail(TKB_ERR_INVALID_ARG, "amax_allreduce: bad arguments (world must be 1..%d)", kMaxWorld);
    int sm; int* status;
    if (int e = api_device(&sm, &status)) return e;
    PeerSlots ps;
    for (int i = 0; i < kMaxWorld; i++) ps.p[i] = i < world ? static_cast<unsigned long long*>(peer_slots[i]) : nullptr;
    amax_allreduce_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(ps, world, rank, epoch, local, out, status, api_wait_limit());
    TKB_CUDA_C(cudaGetLastError());
    return TKB_OK;
}

int tkb_all_to_all(void* const* peer_out, const void* in, size_t bytes_per_peer, int gather, int rank, int world, void* const* peer_counters,
                   int counter_base, unsigned int epoch, void* stream) {
    if (!peer_out || !in || !peer_counters || world < 1 || world > kMaxWorld || rank < 0 || rank >= world || bytes_per_peer == 0 || counter_base < 0)
        return api_fail(TKB_ERR_INVALID_ARG, "all_to_all: bad arguments (world must be 1..%d)", kMaxWorld);
    if ((reinterpret_cast<uintptr_t>(in) & 15u) || (bytes_per_peer & 15u))
        return api_fail(TKB_ERR_BAD_ALIGNMENT, "all_to_all: input and chunk size must be 16-byte aligned");
    int sm; int* status;
    if (int e = api_device(&sm, &status)) return e;
    PeerBytes pb; PeerPtrs pc;
    for (int i = 0; i < kMaxWorld; i++) {
        pb.p[i] = i < world ? static_cast<unsigned char*>(peer_out[i]) : nullptr;
        pc.p[i] = i < world ? static_cast<unsigned int*>(peer_counters[i]) : nullptr;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int parts = kAllToAllParts;
    all_to_all_push_kernel<<<dim3(parts, world), 256, 0, s>>>(pb, static_cast<const unsigned char*>(in), bytes_per_peer, gather, rank, world, pc,
                                                              counter_base);
    TKB_CUDA_C(cudaGetLastError());
    // every sender adds `parts` to its counter per call: wait until all of them have reached epoch * parts
    wait_flags_kernel<<<1, 32, 0, s>>>(static_cast<const unsigned int*>(peer_counters[rank]) + counter_base, world, -1, epoch * unsigned(parts), status, api_wait_limit());
    TKB_CUDA_C(cudaGetLastError());
    return TKB_OK;
}

int tkb_all_to_all_4d(void* const* peer_out, const void* in, const long long* dims, int elem_bytes, int scatter_axis, int gather_axis, int rank,
                      int world, void* const* peer_counters, int counter_base, unsigned int epoch, void* stream) {
    if (!peer_out || !in || !dims || !peer_counters) return api_fail(TKB_ERR_INVALID_ARG, "all_to_all_4d: null pointer");
    if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world || counter_base < 0 || epoch == 0)
        return api_fail(TKB_ERR_INVALID_ARG, "all_to_all_4d: bad rank / world / counters / epoch");
    if (scatter_axis < 0 || scatter_axis > 3 || gather_axis < 0 || gather_axis > 3 || scatter_axis == gather_axis)
        return api_fail(TKB_ERR_INVALID_ARG, "all_to_all_4d: scatter and gather axes must be two different axes in 0..3");
    if (elem_bytes != 1 && elem_bytes != 2 && elem_bytes != 4 && elem_bytes != 8) return api_fail(TKB_ERR_INVALID_ARG, "all_to_all_4d: element size must be 1, 2, 4 or 8 bytes");
    for (int a = 0; a < 4; a++)
        if (dims[a] < 1) return api_fail(TKB_ERR_INVALID_ARG, "all_to_all_4d: dims must be positive");
    if (dims[scatter_axis] % world) return api_fail(TKB_ERR_INVALID_ARG, "all_to_all_4d: the scattered axis must divide by the world size");
    const long long inner_bytes = dims[3] * elem_bytes;
    if (inner_bytes % 16 || (scatter_axis == 3 && (inner_bytes / world) % 16) || (reinterpret_cast<uintptr_t>(in) & 15u))
        return api_fail(TKB_ERR_BAD_ALIGNMENT, "all_to_all_4d: the innermost axis (and its per-rank part, if scattered) must be whole 16-byte vectors");
    int sm; int* status;
    if (int e = api_device(&sm, &status)) return e;
    A2A4Params p;
    memset(&p, 0, sizeof(p));
    PeerPtrs pc;
    for (int i = 0; i < kMaxWorld; i++) {
        p.out[i] = i < world ? static_cast<unsigned char*>(peer_out[i]) : nullptr;
        p.counters[i] = i < world ? static_cast<unsigned int*>(peer_counters[i]) : nullptr;
        pc.p[i] = p.counters[i];
        if (i < world && (!p.out[i] || !p.counters[i] || (reinterpret_cast<uintptr_t>(p.out[i]) & 15u)))
            return api_fail(TKB_ERR_INVALID_ARG, "all_to_all_4d: null or misaligned buffer of rank %d", i);
    }
    for (int a = 0; a < 4; a++) p.in_dims[a] = p.out_dims[a] = a == 3 ? inner_bytes / 16 : dims[a];
    p.out_dims[scatter_axis] = p.in_dims[scatter_axis] / world;
    p.out_dims[gather_axis] = p.in_dims[gather_axis] * world;
    p.scatter = scatter_axis; p.gather = gather_axis; p.rank = rank; p.world = world; p.counter_base = counter_base + world;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // counters [base, base + world): "rank r has entered call `epoch`" (nobody writes into a peer that may still be reading
    // its output of the previous call); [base + world, base + 2 * world): CTAs of rank r that are through
    a2a_enter_kernel<<<1, 32, 0, s>>>(pc, counter_base, rank, world, epoch, status, api_wait_limit());
    TKB_CUDA_C(cudaGetLastError());
    const long long total = p.in_dims[0] * p.in_dims[1] * p.in_dims[2] * p.in_dims[3];
    const int grid = int(total / 2048 < 1 ? 1 : (total / 2048 > kAllToAll4dMaxGrid ? kAllToAll4dMaxGrid : total / 2048));   // the same on every rank
    all_to_all_4d_kernel<<<grid, 256, 0, s>>>(static_cast<const unsigned char*>(in), p);
    TKB_CUDA_C(cudaGetLastError());
    wait_flags_kernel<<<1, 32, 0, s>>>(static_cast<const unsigned int*>(peer_counters[rank]) + counter_base + world, world, -1, epoch * unsigned(grid), status, api_wait_limit());
    TKB_CUDA_C(cudaGetLastError());
    return TKB_OK;
}

static int ag_gemm_impl(void* const* peer_codes, void* const* peer_scales, const float* X_sg, const void* W, const void* W_sc,
                        const float* W_sg, void* D, int64_t ldd, int M, int N_local, int K, int rank, int world, void* const* peer_arrived,
                        void* const* peer_done, void* exit_counter, unsigned int epoch, int comm_ctas, void* epoch_counter, void* stream) {
    if (!peer_codes || !peer_scales || !X_sg || !W || !W_sc || !W_sg || !D || !peer_arrived)
        return api_fail(TKB_ERR_INVALID_ARG, "ag_gemm: null pointer");
    if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world) return api_fail(TKB_ERR_INVALID_ARG, "ag_gemm: world must be 1..%d", kMaxWorld);
    if (M < 1 || M % (256 * world)) return api_fail(TKB_ERR_INVALID_ARG, "ag_gemm: M=%d must be a positive multiple of 256 * world", M);
    if (K < 64 || K % 64 || N_local < 8 || N_local % 8) return api_fail(TKB_ERR_INVALID_ARG, "ag_gemm: K %% 64 and N %% 8 must be 0");
    int sm; int* status;
    if (int e = api_device(&sm, &status)) return e;
    const bool push_warps = comm_ctas == TKB_AG_PUSH_WARPS;      // two push warps in every CTA instead of dedicated comm CTAs
    if (push_warps) comm_ctas = 0;
    if (comm_ctas < 0 || comm_ctas % 2 || comm_ctas > sm - 2) return api_fail(TKB_ERR_INVALID_ARG, "ag_gemm: comm_ctas must be even and leave compute CTAs");
    // comm_ctas == 0 with world > 1: the caller moves the rows itself (copy engines, see tkb_ag_linear_nvfp4) and raises the arrival flags
    if (peer_done && !exit_counter) return api_fail(TKB_ERR_INVALID_ARG, "ag_gemm: peer_done needs an exit counter");
    if (epoch_counter && (!exit_counter || comm_ctas != 0)) return api_fail(TKB_ERR_INVALID_ARG, "ag_gemm: a device-side epoch needs an exit counter and comm_ctas == 0");
    GemmArgs g;
    memset(&g, 0, sizeof(g));
    g.kind = KIND_NVFP4; g.config = 0;
    if (ldd == 0) ldd = N_local;
    if (int e = api_make_gemm_maps(&g, KIND_NVFP4, peer_codes[rank], K / 2, peer_scales[rank], W, K / 2, W_sc, D, ldd, M, N_local, K)) return e;
    g.sgA = X_sg; g.sgB = W_sg; g.M = M; g.N = N_local; g.K = K; g.status = status; g.sm_count = sm;
    g.stream = static_cast<cudaStream_t>(stream);
    g.mode = MODE_AG;
    g.prof = api_profile_buffer();
    for (int i = 0; i < world; i++) {
        g.comm.ag.peer_codes[i] = static_cast<const uint8_t*>(peer_codes[i]);
        g.comm.ag.peer_scales[i] = static_cast<const uint8_t*>(peer_scales[i]);
    }
    g.comm.ag.codes = static_cast<uint8_t*>(peer_codes[rank]);
    g.comm.ag.scales = static_cast<uint8_t*>(peer_scales[rank]);
    for (int i = 0; i < world; i++) g.comm.ag.peer_arrived[i] = static_cast<unsigned int*>(peer_arrived[i]);
    if (peer_done) {
        for (int i = 0; i < world; i++) {
            if (!peer_done[i]) return api_fail(TKB_ERR_INVALID_ARG, "ag_gemm: null done array for rank %d", i);
            g.comm.ag.peer_done[i] = static_cast<unsigned int*>(peer_done[i]);
        }
        g.comm.ag.exit_counter = static_cast<unsigned int*>(exit_counter);
    }
    if (epoch_counter) {
        g.comm.ag.exit_counter = static_cast<unsigned int*>(exit_counter);
        g.comm.ag.epoch_counter = static_cast<unsigned int*>(epoch_counter);
    }
    g.comm.ag.epoch = epoch; g.comm.ag.rank = rank; g.comm.ag.world = world; g.comm.ag.blocks_per_rank = M / world / 256;
    g.comm.ag.comm_ctas = world > 1 ? comm_ctas : 0;
    g.comm.ag.push_warps = push_warps && world > 1 ? 1 : 0;
    g.comm.ag.parts = push_warps ? kAgPartsPushWarps : kAgPartsPerBlock;
    TKB_CUDA_C(launch_gemm(g));
    return TKB_OK;
}

int tkb_ag_gemm_nvfp4(void* const* peer_codes, void* const* peer_scales, const float* X_sg, const void* W, const void* W_sc,
                      const float* W_sg, void* D, int64_t ldd, int M, int N_local, int K, int rank, int world, void* const* peer_arrived,
                      void* const* peer_done, void* exit_counter, unsigned int epoch, int comm_ctas, void* stream) {
    return ag_gemm_impl(peer_codes, peer_scales, X_sg, W, W_sc, W_sg, D, ldd, M, N_local, K, rank, world, peer_arrived, peer_done, exit_counter, epoch,
                        comm_ctas, nullptr, stream);
}

int tkb_debug_struct_layout(int which, int field) {
    // sizeof / offsetof of the state structs of the C ABI, for bindings that mirror them by hand
#define TKB_OFF(T, m) case __COUNTER__ - base: return int(offsetof(T, m));
    if (which == 0) {
        if (field == 0) return int(sizeof(tkb_ag_state));
        enum { base = __COUNTER__ };
        switch (field) {
            TKB_OFF(tkb_ag_state, rank) TKB_OFF(tkb_ag_state, world) TKB_OFF(tkb_ag_state, M) TKB_OFF(tkb_ag_state, K)
            TKB_OFF(tkb_ag_state, codes) TKB_OFF(tkb_ag_state, scales) TKB_OFF(tkb_ag_state, arrived) TKB_OFF(tkb_ag_state, slots)
            TKB_OFF(tkb_ag_state, done) TKB_OFF(tkb_ag_state, amax) TKB_OFF(tkb_ag_state, sg) TKB_OFF(tkb_ag_state, exit_counter)
            TKB_OFF(tkb_ag_state, copy) TKB_OFF(tkb_ag_state, epoch_counter)
            default: return -1;
        }
    }
    if (which == 2) {
        if (field == 0) return int(sizeof(tkb_rs_state));
        enum { base = __COUNTER__ };
        switch (field) {
            TKB_OFF(tkb_rs_state, rank) TKB_OFF(tkb_rs_state, world) TKB_OFF(tkb_rs_state, M) TKB_OFF(tkb_rs_state, N)
            TKB_OFF(tkb_rs_state, out) TKB_OFF(tkb_rs_state, flags) TKB_OFF(tkb_rs_state, maps)
            default: return -1;
        }
    }
    if (which == 1) {
        if (field == 0) return int(sizeof(tkb_moe_state));
        enum { base = __COUNTER__ };
        switch (field) {
            TKB_OFF(tkb_moe_state, rank) TKB_OFF(tkb_moe_state, world) TKB_OFF(tkb_moe_state, T) TKB_OFF(tkb_moe_state, H)
            TKB_OFF(tkb_moe_state, I) TKB_OFF(tkb_moe_state, E) TKB_OFF(tkb_moe_state, top_k) TKB_OFF(tkb_moe_state, cap_rows)
            TKB_OFF(tkb_moe_state, xq_rows) TKB_OFF(tkb_moe_state, slots) TKB_OFF(tkb_moe_state, experts_all) TKB_OFF(tkb_moe_state, Y)
            TKB_OFF(tkb_moe_state, flags) TKB_OFF(tkb_moe_state, counters) TKB_OFF(tkb_moe_state, codes) TKB_OFF(tkb_moe_state, scales)
            TKB_OFF(tkb_moe_state, experts_local) TKB_OFF(tkb_moe_state, weights) TKB_OFF(tkb_moe_state, counts) TKB_OFF(tkb_moe_state, padded)
            TKB_OFF(tkb_moe_state, pull_idx) TKB_OFF(tkb_moe_state, block_expert) TKB_OFF(tkb_moe_state, num_blocks)
            TKB_OFF(tkb_moe_state, comb_idx) TKB_OFF(tkb_moe_state, arrived) TKB_OFF(tkb_moe_state, sg)
            default: return -1;
        }
    }
#undef TKB_OFF
    return -1;
}

int tkb_debug_ag_schedule(int M, int K, int rank, int world, int comm_ctas, int comm_idx, int piece_bytes, long long* out, int max_pieces) {
    return tkb_debug_ag_schedule_parts(M, K, rank, world, comm_ctas, comm_idx, piece_bytes, kAgPartsPerBlock, out, max_pieces);
}

int tkb_debug_ag_schedule_parts(int M, int K, int rank, int world, int comm_ctas, int comm_idx, int piece_bytes, int parts, long long* out,
                                int max_pieces) {
    if ((parts != kAgPartsPerBlock && parts != kAgPartsPushWarps) || world < 2 || world > kMaxWorld || rank < 0 || rank >= world || M < 1 || M % (256 * world) || K < 64 || K % 64 || comm_ctas < 1 ||
        comm_idx < 0 || comm_idx >= comm_ctas || piece_bytes < 16 || piece_bytes % 16 || (!out && max_pieces > 0))
        return -api_fail(TKB_ERR_INVALID_ARG, "debug_ag_schedule: bad arguments");
    const AgGeometry geo{rank, world, M / world / 256, K / 2, (K / 64) * 512, parts, parts == kAgPartsPerBlock ? kAgFanOut : kAgFanOutPushWarps};
    const int units = ag_units(geo);
    AgCursor c{comm_idx, 0, 0u};
    int n = 0;
    while (c.u < units) {
        const AgPiece pc = ag_piece(geo, c, uint32_t(piece_bytes));
        const bool last = ag_advance(c, pc, comm_ctas);
        if (n < max_pieces) {
            long long* o = out + size_t(n) * 6;
            o[0] = pc.dst_rank; o[1] = pc.span; o[2] = (long long)pc.off; o[3] = pc.bytes; o[4] = pc.flag; o[5] = last ? 1 : 0;
        }
        n++;
    }
    return n;
}

// ---- GEMM + reduce-scatter (row-parallel partner of the all-gather GEMM) ------------------------------------------------
int tkb_rs_maps_create(const tkb_rs_state* st, void** device_maps) {
    if (!st || !device_maps) return api_fail(TKB_ERR_INVALID_ARG, "rs_maps_create: null pointer");
    const int w = st->world;
    if (w < 1 || w > kMaxWorld || st->M < 1 || st->M % (256 * w) || st->N < 8 || st->N % 8)
        return api_fail(TKB_ERR_INVALID_ARG, "rs_maps_create: need world 1..%d, M %% (256 * world) == 0, N %% 8 == 0", kMaxWorld);
    int sm; int* status;
    if (int e = api_device(&sm, &status)) return e;
    CUtensorMap maps[kMaxWorld];
    memset(maps, 0, sizeof(maps));
    for (int i = 0; i < w; i++) {
        if (!st->out[i]) return api_fail(TKB_ERR_INVALID_ARG, "rs_maps_create: null output buffer of rank %d", i);
        if (int e = api_make_output_map(&maps[i], st->out[i], st->M / w, st->N, st->N)) return e;
    }
    void* dev = nullptr;
    TKB_CUDA_C(cudaMalloc(&dev, sizeof(maps)));
    cudaError_t ce = cudaMemcpy(dev, maps, sizeof(maps), cudaMemcpyHostToDevice);
    if (ce != cudaSuccess) { cudaFree(dev); return api_fail(TKB_ERR_CUDA, "rs_maps_create: %s", cudaGetErrorString(ce)); }
    *device_maps = dev;
    return TKB_OK;
}
int tkb_rs_maps_destroy(void* device_maps) {
    if (device_maps) TKB_CUDA_C(cudaFree(device_maps));
    return TKB_OK;
}

int tkb_gemm_rs_nvfp4(const tkb_rs_state* st, unsigned int epoch, const void* A, const void* A_sc, const float* A_sg, const void* B,
                      const void* B_sc, const float* B_sg, int K_local, void* stream) {
    if (!st || !A || !A_sc || !A_sg || !B || !B_sc || !B_sg || epoch == 0) return api_fail(TKB_ERR_INVALID_ARG, "gemm_rs: null pointer or epoch 0");
    const int w = st->world, r = st->rank;
    if (w < 1 || w > kMaxWorld || r < 0 || r >= w || st->M % (256 * w) || st->N % 8 || !st->maps)
        return api_fail(TKB_ERR_INVALID_ARG, "gemm_rs: bad world / rank / M / N, or no tensor maps (tkb_rs_maps_create)");
    if (K_local < 64 || K_local % 64) return api_fail(TKB_ERR_INVALID_ARG, "gemm_rs: K_local must be a positive multiple of 64");
    int sm; int* status;
    if (int e = api_device(&sm, &status)) return e;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int rows = st->M / w;
    // 1. this rank's output rows start from zero; nobody may add into them before that (first flag exchange)
    TKB_CUDA_C(cudaMemsetAsync(st->out[r], 0, size_t(rows) * st->N * 2, s));
    if (w > 1) {
        if (int e = tkb_signal_peers(st->flags, w, r, r, epoch, 0, s)) return e;
        if (int e = tkb_wait_flags(st->flags[r], w, r, epoch, s)) return e;
    }
    // 2. the GEMM; every 32 x 64 box of bf16 results is added into the owner's rows by the memory system
    GemmArgs g;
    memset(&g, 0, sizeof(g));
    g.kind = KIND_NVFP4; g.config = 0;
    if (int e = api_make_gemm_maps(&g, KIND_NVFP4, A, K_local / 2, A_sc, B, K_local / 2, B_sc, st->out[r], st->N, rows, st->N, K_local)) return e;
    // (the output map built above only serves as a valid descriptor: this mode stores through rs_maps)
    if (int e = api_make_operand_a_maps(&g, A, A_sc, st->M, K_local)) return e;
    g.sgA = A_sg; g.sgB = B_sg; g.M = st->M; g.N = st->N; g.K = K_local; g.status = status; g.sm_count = sm; g.stream = s;
    g.mode = MODE_RS;
    g.rs_maps = static_cast<const CUtensorMap*>(st->maps); g.rs_rows_per_rank = rows; g.rs_rank = r; g.rs_world = w;
    TKB_CUDA_C(launch_gemm(g));
    // 3. the rows are complete when every rank's kernel has finished (second flag exchange)
    if (w > 1) {
        if (int e = tkb_signal_peers(st->flags, w, r, w + r, epoch, 0, s)) return e;
        if (int e = tkb_wait_flags(static_cast<unsigned int*>(st->flags[r]) + w, w, r, epoch, s)) return e;
    }
    return TKB_OK;
}

// Streams, events and the arrival-flag pattern of the copy-engine gather (tkb_ag_copy_create).
struct AgCopyCtx {
    int n_streams, stamp_count, device;
    cudaStream_t stream[kAgMaxCopyStreams];
    cudaEvent_t quantized;                        // recorded in the caller's stream after the quantize launch
    cudaEvent_t copied[2][kAgMaxCopyStreams];     // per buffer set: this rank's slice has been read by all copies of the call
    unsigned int* stamp[2];                       // per buffer set: stamp_count words holding the epoch of the call
};

int tkb_ag_copy_create(int n_streams, int stamp_count, void** handle) {
    if (!handle || n_streams < 1 || n_streams > kAgMaxCopyStreams || stamp_count < 1)
        return api_fail(TKB_ERR_INVALID_ARG, "ag_copy_create: need 1..%d streams, stamp_count >= 1 and an output pointer", kAgMaxCopyStreams);
    AgCopyCtx* c = new (std::nothrow) AgCopyCtx();
    if (!c) return api_fail(TKB_ERR_CUDA, "ag_copy_create: out of host memory");
    memset(c, 0, sizeof(*c));
    c->n_streams = n_streams; c->stamp_count = stamp_count;
    cudaError_t e = cudaGetDevice(&c->device);
    for (int i = 0; i < n_streams && e == cudaSuccess; i++) e = cudaStreamCreateWithFlags(&c->stream[i], cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->quantized, cudaEventDisableTiming);
    for (int b = 0; b < 2 && e == cudaSuccess; b++) {
        for (int i = 0; i < n_streams && e == cudaSuccess; i++) e = cudaEventCreateWithFlags(&c->copied[b][i], cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaMalloc(&c->stamp[b], size_t(stamp_count) * sizeof(unsigned int));
        if (e == cudaSuccess) e = cudaMemset(c->stamp[b], 0, size_t(stamp_count) * sizeof(unsigned int));
    }
    if (e != cudaSuccess) {
        tkb_ag_copy_destroy(c);
        return api_fail(TKB_ERR_CUDA, "ag_copy_create: %s", cudaGetErrorString(e));
    }
    *handle = c;
    return TKB_OK;
}

int tkb_ag_copy_destroy(void* handle) {
    AgCopyCtx* c = static_cast<AgCopyCtx*>(handle);
    if (!c) return TKB_OK;
    for (int i = 0; i < kAgMaxCopyStreams; i++)
        if (c->stream[i]) { cudaStreamSynchronize(c->stream[i]); cudaStreamDestroy(c->stream[i]); }
    if (c->quantized) cudaEventDestroy(c->quantized);
    for (int b = 0; b < 2; b++) {
        for (int i = 0; i < kAgMaxCopyStreams; i++)
            if (c->copied[b][i]) cudaEventDestroy(c->copied[b][i]);
        if (c->stamp[b]) cudaFree(c->stamp[b]);
    }
    delete c;
    return TKB_OK;
}

// One step of the column-parallel layer with the gather done by copy engines.  `quantized` is recorded in `main` after the
// quantize launch, copied[j] in copy stream j after the step's last copy there; with wait_prev, `main` first waits for
// copied[] as left by the step two calls ago (the same buffer set).
// Ordering argument: the amax exchange inside the quantize kernel is a barrier over the ranks for this epoch, and a rank only
// reaches it after its GEMM of the previous step (same stream).  So once this rank's quantize kernel has finished, no peer
// still reads the buffer set of two steps ago, which is the one written now; no separate acknowledgement is needed.  The copy
// streams carry copies only (no kernels), so they never compete with the persistent GEMM kernel for an SM.  The epoch is
// read on the device (st->epoch_counter), which is what makes the step replayable from a graph.
static int ag_ce_step(const tkb_ag_state* st, AgCopyCtx* c, cudaEvent_t quantized, cudaEvent_t* copied, bool wait_prev, unsigned int epoch,
                      const void* X_local, const void* W, const void* W_sc, const float* W_sg, void* D, int64_t ldd, int N_local, int arithmetic,
                      cudaStream_t main) {
    const int w = st->world, r = st->rank, b = int(epoch % 2u);
    const int rows = st->M / w, flags_per_rank = rows / 64;
    if (c->stamp_count < flags_per_rank) return api_fail(TKB_ERR_INVALID_ARG, "ag_linear: tkb_ag_copy_create was given fewer than M / world / 64 flags");
    if (!st->epoch_counter) return api_fail(TKB_ERR_INVALID_ARG, "ag_linear: the copy-engine gather needs st->epoch_counter");
    uint8_t* my_codes = static_cast<uint8_t*>(st->codes[b][r]) + size_t(r) * rows * (st->K / 2);
    uint8_t* my_scales = static_cast<uint8_t*>(st->scales[b][r]) + size_t(r) * (rows / 128) * (st->K / 64) * 512;
    if (wait_prev)
        for (int i = 0; i < c->n_streams; i++) TKB_CUDA_C(cudaStreamWaitEvent(main, copied[i], 0));
    if (int e = api_quantize_sharded(X_local, 0, my_codes, my_scales, st->sg, rows, st->K, 0, arithmetic, st->slots[b], w, r, epoch, c->stamp[b],
                                     flags_per_rank, static_cast<const unsigned int*>(st->epoch_counter), main))
        return e;
    TKB_CUDA_C(cudaEventRecord(quantized, main));
    // the GEMM goes into the queue first: it starts with this rank's own rows while the host is still issuing the copies
    if (int e = ag_gemm_impl(st->codes[b], st->scales[b], st->sg, W, W_sc, W_sg, D, ldd, st->M, N_local, st->K, r, w, st->arrived[b], nullptr,
                             st->exit_counter, epoch, 0, st->epoch_counter, main))
        return e;
    const size_t code_bytes = size_t(rows) * (st->K / 2), code_off = size_t(r) * code_bytes;
    const size_t sc_bytes = size_t(rows / 128) * (st->K / 64) * 512, sc_off = size_t(r) * sc_bytes;
    for (int i = 0; i < c->n_streams; i++) TKB_CUDA_C(cudaStreamWaitEvent(c->stream[i], quantized, 0));
    for (int i = 1; i < w; i++) {
        const int d = (r + w - i) % w;           // in the order in which the peers consume this rank's rows
        cudaStream_t cs = c->stream[(i - 1) % c->n_streams];
        TKB_CUDA_C(cudaMemcpyAsync(static_cast<uint8_t*>(st->codes[b][d]) + code_off, my_codes, code_bytes, cudaMemcpyDeviceToDevice, cs));
        TKB_CUDA_C(cudaMemcpyAsync(static_cast<uint8_t*>(st->scales[b][d]) + sc_off, my_scales, sc_bytes, cudaMemcpyDeviceToDevice, cs));
        // stream order: the flags leave after the rows they announce have been written
        TKB_CUDA_C(cudaMemcpyAsync(static_cast<unsigned int*>(st->arrived[b][d]) + size_t(r) * flags_per_rank, c->stamp[b],
                                   size_t(flags_per_rank) * sizeof(unsigned int), cudaMemcpyDeviceToDevice, cs));
    }
    for (int i = 0; i < c->n_streams; i++) TKB_CUDA_C(cudaEventRecord(copied[i], c->stream[i]));
    return TKB_OK;
}

int tkb_ag_linear_nvfp4(const tkb_ag_state* st, unsigned int epoch, const void* X_local, const void* W, const void* W_sc, const float* W_sg,
                        void* D, int64_t ldd, int N_local, int comm_ctas, int arithmetic, void* stream) {
    if (!st || !X_local || epoch == 0) return api_fail(TKB_ERR_INVALID_ARG, "ag_linear: null state/input or epoch 0");
    const int w = st->world, r = st->rank, b = int(epoch % 2u);
    if (w < 1 || w > kMaxWorld || r < 0 || r >= w || st->M % (256 * w)) return api_fail(TKB_ERR_INVALID_ARG, "ag_linear: bad world / rank / M");
    const int rows = st->M / w;
    if (!st->exit_counter) return api_fail(TKB_ERR_INVALID_ARG, "ag_linear: null exit counter");
    uint8_t* my_codes = static_cast<uint8_t*>(st->codes[b][r]) + size_t(r) * rows * (st->K / 2);
    uint8_t* my_scales = static_cast<uint8_t*>(st->scales[b][r]) + size_t(r) * (rows / 128) * (st->K / 64) * 512;
    cudaStream_t main = static_cast<cudaStream_t>(stream);
    if (comm_ctas == TKB_AG_PUSH_WARPS) {
        // Two launches: the quantize kernel (whose amax exchange orders this step after every peer's previous one, so that
        // nobody still reads the buffer set that the pushes overwrite) and the GEMM with push warps in every CTA.
        if (int e = tkb_nvfp4_quantize_sharded(X_local, 0, my_codes, my_scales, st->sg, rows, st->K, 0, arithmetic, st->slots[b], w, r, epoch, stream))
            return e;
        return ag_gemm_impl(st->codes[b], st->scales[b], st->sg, W, W_sc, W_sg, D, ldd, st->M, N_local, st->K, r, w, st->arrived[b], nullptr,
                            nullptr, epoch, TKB_AG_PUSH_WARPS, nullptr, stream);
    }
    const bool ce = w > 1 && comm_ctas < 0;          // gather by copy engines instead of comm CTAs
    if (!ce) {
        // This rank's slice of its own buffers is only read by its own kernels (earlier in this stream); what the peers
        // read are the copies the comm CTAs push, and those wait for the peers' epoch - 2 kernels themselves.
        if (int e = tkb_nvfp4_quantize_sharded(X_local, 0, my_codes, my_scales, st->sg, rows, st->K, 0, arithmetic, st->slots[b], w, r, epoch, stream))
            return e;
        return tkb_ag_gemm_nvfp4(st->codes[b], st->scales[b], st->sg, W, W_sc, W_sg, D, ldd, st->M, N_local, st->K, r, w, st->arrived[b],
                                 st->done, st->exit_counter, epoch, w > 1 ? comm_ctas : 0, stream);
    }
    AgCopyCtx* c = static_cast<AgCopyCtx*>(st->copy);
    if (!c) return api_fail(TKB_ERR_INVALID_ARG, "ag_linear: the copy-engine gather needs st->copy from tkb_ag_copy_create");
    // the copies of epoch - 2 read the slice and the flag pattern that are about to be overwritten
    return ag_ce_step(st, c, c->quantized, c->copied[b], epoch > 2, epoch, X_local, W, W_sc, W_sg, D, ldd, N_local, arithmetic, main);
}

// ---- the same step, recorded once and replayed: a CUDA graph of `steps` consecutive calls -------------------------------
struct AgGraph { cudaGraph_t graph; cudaGraphExec_t exec; AgCopyCtx* copy; int steps; };

int tkb_ag_graph_create(const tkb_ag_state* st, unsigned int first_epoch, int steps, const void* const* X_local, const void* const* W,
                        const void* const* W_sc, const float* const* W_sg, void* const* D, int64_t ldd, int N_local, int arithmetic, void** handle) {
    if (!st || !handle || !X_local || !W || !W_sc || !W_sg || !D) return api_fail(TKB_ERR_INVALID_ARG, "ag_graph_create: null pointer");
    if (steps < 2 || steps % 2 || steps > 64) return api_fail(TKB_ERR_INVALID_ARG, "ag_graph_create: steps must be even (both buffer sets), 2..64");
    if (first_epoch == 0) return api_fail(TKB_ERR_INVALID_ARG, "ag_graph_create: epochs start at 1");
    AgCopyCtx* c = static_cast<AgCopyCtx*>(st->copy);
    if (st->world < 2 || !c || !st->epoch_counter) return api_fail(TKB_ERR_INVALID_ARG, "ag_graph_create: needs world > 1, st->copy and st->epoch_counter");
    int sm; int* status;
    if (int e = api_device(&sm, &status)) return e;          // creates the per-device context before the capture starts
    cudaStream_t cap = nullptr;
    cudaEvent_t quantized[64] = {}, copied[64][kAgMaxCopyStreams] = {};
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    int rc = TKB_OK;
    cudaError_t ce = cudaStreamCreateWithFlags(&cap, cudaStreamNonBlocking);
    for (int i = 0; i < steps && ce == cudaSuccess; i++) {
        ce = cudaEventCreateWithFlags(&quantized[i], cudaEventDisableTiming);
        for (int j = 0; j < c->n_streams && ce == cudaSuccess; j++) ce = cudaEventCreateWithFlags(&copied[i][j], cudaEventDisableTiming);
    }
    bool capturing = false;
    if (ce == cudaSuccess) { ce = cudaStreamBeginCapture(cap, cudaStreamCaptureModeThreadLocal); capturing = ce == cudaSuccess; }
    for (int i = 0; i < steps && ce == cudaSuccess && rc == TKB_OK; i++) {
        // inside the graph a step waits for the copies of the step two before it; the first two steps have nothing to wait for,
        // because the graph ends only when all of its copies have ended and a launch starts after the previous one has ended
        if (i >= 2)
            for (int j = 0; j < c->n_streams && ce == cudaSuccess; j++) ce = cudaStreamWaitEvent(cap, copied[i - 2][j], 0);
        if (ce == cudaSuccess)
            rc = ag_ce_step(st, c, quantized[i], copied[i], false, first_epoch + unsigned(i), X_local[i], W[i], W_sc[i], W_sg[i], D[i], ldd, N_local,
                            arithmetic, cap);
    }
    if (capturing) {
        for (int i = steps - 2; i < steps && ce == cudaSuccess && rc == TKB_OK; i++)        // join the copy streams of the last two steps
            for (int j = 0; j < c->n_streams && ce == cudaSuccess; j++) ce = cudaStreamWaitEvent(cap, copied[i][j], 0);
        cudaError_t ee = cudaStreamEndCapture(cap, &graph);       // always ends the capture, also after an error
        if (ce == cudaSuccess) ce = ee;
    }
    if (ce == cudaSuccess && rc == TKB_OK) ce = cudaGraphInstantiate(&exec, graph, 0);
    for (int i = 0; i < steps; i++) {
        if (quantized[i]) cudaEventDestroy(quantized[i]);
        for (int j = 0; j < kAgMaxCopyStreams; j++) if (copied[i][j]) cudaEventDestroy(copied[i][j]);
    }
    if (cap) cudaStreamDestroy(cap);
    if (rc != TKB_OK || ce != cudaSuccess) {
        if (graph) cudaGraphDestroy(graph);
        if (rc != TKB_OK) return rc;
        return api_fail(TKB_ERR_CUDA, "ag_graph_create: %s", cudaGetErrorString(ce));
    }
    AgGraph* g = new (std::nothrow) AgGraph{graph, exec, c, steps};
    if (!g) { cudaGraphExecDestroy(exec); cudaGraphDestroy(graph); return api_fail(TKB_ERR_CUDA, "ag_graph_create: out of host memory"); }
    *handle = g;
    return TKB_OK;
}

int tkb_ag_graph_launch(void* handle, void* stream) {
    AgGraph* g = static_cast<AgGraph*>(handle);
    if (!g) return api_fail(TKB_ERR_INVALID_ARG, "ag_graph_launch: null handle");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // copies of earlier, individually issued steps may still read the slices that the graph's first steps overwrite
    for (int b = 0; b < 2; b++)
        for (int j = 0; j < g->copy->n_streams; j++) TKB_CUDA_C(cudaStreamWaitEvent(s, g->copy->copied[b][j], 0));
    TKB_CUDA_C(cudaGraphLaunch(g->exec, s));
    return TKB_OK;
}

int tkb_ag_graph_destroy(void* handle) {
    AgGraph* g = static_cast<AgGraph*>(handle);
    if (!g) return TKB_OK;
    cudaGraphExecDestroy(g->exec);
    cudaGraphDestroy(g->graph);
    delete g;
    return TKB_OK;
}

} // extern "C"
