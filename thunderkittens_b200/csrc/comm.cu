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
#include <cstring>
#include "../../include/tkb200.h"
#include "internal.h"
#include "ptx.cuh"

namespace tkb {

int api_fail(int code, const char* fmt, ...);          // api.cu
int api_device(int* sm_count, int** status);           // api.cu
int api_make_gemm_maps(GemmArgs* g, int kind, const void* A, int64_t lda_bytes, const void* A_sc, const void* B, int64_t ldb_bytes,
                       const void* B_sc, void* D, int64_t ldd, int M, int N, int K);   // api.cu

struct PeerPtrs { unsigned int* p[kMaxWorld]; };

__global__ void signal_peers_kernel(PeerPtrs peers, int world, int rank, int index, unsigned int value, int include_self) {
    const int t = threadIdx.x;
    if (t < world && (t != rank || include_self)) {
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peers.p[t] + index), "r"(value) : "memory");
    }
}

// Waits until every flags[i] (i != skip) has reached `value` (epochs only grow).
__global__ void wait_flags_kernel(const unsigned int* flags, int count, int skip, unsigned int value, int* status) {
    const int t = threadIdx.x;
    if (t < count && t != skip) {
        const long long t0 = clock64();
        while (true) {
            unsigned int v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + t) : "memory");
            if (int(v - value) >= 0) break;
            if (clock64() - t0 > TKB_WAIT_LIMIT_CYCLES) {
                if (status) atomicExch(status, (int)TKB_DEV_TIMEOUT);
                break;
            }
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
    int sm; int* status;
    if (int e = api_device(&sm, &status)) return e;
    if (!flags || count < 1 || count > 1024) return api_fail(TKB_ERR_INVALID_ARG, "wait_flags: bad arguments");
    wait_flags_kernel<<<1, ((count + 31) / 32) * 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const unsigned int*>(flags), count, skip,
                                                                                         value, status);
    TKB_CUDA_C(cudaGetLastError());
    return TKB_OK;
}

int tkb_ag_gemm_nvfp4(void* const* peer_codes, void* const* peer_scales, const float* X_sg, const void* W, const void* W_sc,
                      const float* W_sg, void* D, int64_t ldd, int M, int N_local, int K, int rank, int world, void* const* peer_arrived,
                      unsigned int epoch, int comm_ctas, void* stream) {
    int sm; int* status;
    if (int e = api_device(&sm, &status)) return e;
    if (!peer_codes || !peer_scales || !X_sg || !W || !W_sc || !W_sg || !D || !peer_arrived)
        return api_fail(TKB_ERR_INVALID_ARG, "ag_gemm: null pointer");
    if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world) return api_fail(TKB_ERR_INVALID_ARG, "ag_gemm: world must be 1..%d", kMaxWorld);
    if (M % (256 * world)) return api_fail(TKB_ERR_INVALID_ARG, "ag_gemm: M=%d must be a multiple of 256 * world", M);
    if (K % 64 || N_local % 8) return api_fail(TKB_ERR_INVALID_ARG, "ag_gemm: K %% 64 and N %% 8 must be 0");
    if (comm_ctas < 0 || comm_ctas % 2 || comm_ctas > sm - 2) return api_fail(TKB_ERR_INVALID_ARG, "ag_gemm: comm_ctas must be even and leave compute CTAs");
    if (world > 1 && comm_ctas == 0) return api_fail(TKB_ERR_INVALID_ARG, "ag_gemm: world > 1 needs comm_ctas >= 2");
    GemmArgs g;
    memset(&g, 0, sizeof(g));
    g.kind = KIND_NVFP4; g.config = 0;
    if (ldd == 0) ldd = N_local;
    if (int e = api_make_gemm_maps(&g, KIND_NVFP4, peer_codes[rank], K / 2, peer_scales[rank], W, K / 2, W_sc, D, ldd, M, N_local, K)) return e;
    g.sgA = X_sg; g.sgB = W_sg; g.M = M; g.N = N_local; g.K = K; g.status = status; g.sm_count = sm;
    g.stream = static_cast<cudaStream_t>(stream);
    g.mode = MODE_AG;
    for (int i = 0; i < world; i++) {
        g.comm.ag.peer_codes[i] = static_cast<const uint8_t*>(peer_codes[i]);
        g.comm.ag.peer_scales[i] = static_cast<const uint8_t*>(peer_scales[i]);
    }
    g.comm.ag.codes = static_cast<uint8_t*>(peer_codes[rank]);
    g.comm.ag.scales = static_cast<uint8_t*>(peer_scales[rank]);
    for (int i = 0; i < world; i++) g.comm.ag.peer_arrived[i] = static_cast<unsigned int*>(peer_arrived[i]);
    g.comm.ag.epoch = epoch; g.comm.ag.rank = rank; g.comm.ag.world = world; g.comm.ag.blocks_per_rank = M / world / 256;
    g.comm.ag.comm_ctas = world > 1 ? comm_ctas : 0;
    TKB_CUDA_C(launch_gemm(g));
    return TKB_OK;
}

} // extern "C"
