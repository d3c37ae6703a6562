// C-ABI entry points of libtkb200: argument validation, per-device context (SM count, status word,
// quantize scratch), TMA tensor-map construction, launches.  Declarations and the reference entry
// each function replaces: include/tkb200.h.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <atomic>

#include "../../include/tkb200.h"
#include "internal.h"
#include "quantize_types.h"

namespace tkb {

static thread_local char g_err[512] = "";

int api_fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}
#define TKB_CUDA(expr)                                                                                   \
    do {                                                                                                 \
        cudaError_t _e = (expr);                                                                         \
        if (_e != cudaSuccess) return api_fail(TKB_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
    } while (0)

// ------------------------------------------------------------------ per-device context -----
constexpr int kMaxDevices = 64;
constexpr int kQuantSlots = 256;
constexpr int kDecodeRing = 4;                           // streams of one device that may use the skinny-M GEMM
constexpr int kSmallScratchRing = 4;
constexpr size_t kSmallScratchBytes = 2u << 20;
constexpr int kDecodeMaxGrid = 160;                      // CTAs the scratch is sized for
constexpr size_t kDecodePartialFloats = size_t(kDecodeMaxGrid) * 128 * 128;

struct DeviceCtx {
    bool ready = false;
    int sm_count = 0;
    int cc_major = 0;
    int* status = nullptr;          // device int, zero when healthy
    QuantWork* quant_ws = nullptr;  // kQuantSlots zeroed slots, each returned to zero by the kernel that used it
    std::atomic<unsigned> next_slot{0};
    // skinny-M GEMM scratch: kDecodeRing independent sets of (per-CTA fp32 partial tiles, per-CTA flags)
    unsigned char* small_scratch = nullptr;     // kSmallScratchRing buffers of kSmallScratchBytes for short-lived kernel temporaries
    std::atomic<unsigned> small_scratch_calls{0};
    float* decode_partials = nullptr;
    unsigned int* decode_flags = nullptr;
    // one scratch set per stream that has used the kernel: calls on one stream are ordered by the stream, calls on different
    // streams never share a set
    cudaStream_t decode_stream[kDecodeRing] = {};
    bool decode_stream_used[kDecodeRing] = {};
    unsigned decode_calls[kDecodeRing] = {};
};
static DeviceCtx g_ctx[kMaxDevices];
static std::mutex g_ctx_mu;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;
static unsigned long long* g_prof = nullptr;   // tkb_gemm_set_profile_buffer
constexpr long long kDefaultWaitLimit = 2000000000ll;      // about one second at B200 clocks
static std::atomic<long long> g_wait_limit{kDefaultWaitLimit};
long long api_wait_limit() { return g_wait_limit.load(std::memory_order_relaxed); }

static int get_ctx(DeviceCtx** out) {
    int dev = 0;
    TKB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return api_fail(TKB_ERR_INVALID_ARG, "device ordinal %d out of range", dev);
    DeviceCtx& c = g_ctx[dev];
    if (!c.ready) {
        std::lock_guard<std::mutex> lk(g_ctx_mu);
        if (!c.ready) {
            cudaDeviceProp prop;
            TKB_CUDA(cudaGetDeviceProperties(&prop, dev));
            if (prop.major != 10) return api_fail(TKB_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", dev, prop.major, prop.minor);
            c.sm_count = prop.multiProcessorCount;
            c.cc_major = prop.major;
            TKB_CUDA(cudaMalloc(&c.status, sizeof(int)));
            TKB_CUDA(cudaMemset(c.status, 0, sizeof(int)));
            TKB_CUDA(cudaMalloc(&c.quant_ws, sizeof(QuantWork) * kQuantSlots));
            TKB_CUDA(cudaMemset(c.quant_ws, 0, sizeof(QuantWork) * kQuantSlots));
            if (!g_encode) {
                void* fn = nullptr;
                cudaDriverEntryPointQueryResult q;
                TKB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
                if (!fn || q != cudaDriverEntryPointSuccess) return api_fail(TKB_ERR_UNSUPPORTED, "driver does not export cuTensorMapEncodeTiled");
                g_encode = reinterpret_cast<EncodeTiledFn>(fn);
            }
            TKB_CUDA(cudaDeviceSynchronize());
            c.ready = true;
        }
    }
    *out = &c;
    return TKB_OK;
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// 2-D K-major operand map: inner dimension = K in `elem_bytes`-sized elements, 128-byte swizzle,
// box = 128 bytes of K x box_rows rows.  Out-of-range rows / K are zero-filled by the TMA unit.
static int make_operand_map(CUtensorMap* m, const void* base, CUtensorMapDataType dt, int elem_bytes, uint64_t inner_elems,
                            uint64_t rows, uint64_t pitch_bytes, uint32_t box_rows) {
    cuuint64_t dims[2] = {inner_elems, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {uint32_t(128 / elem_bytes), box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(m, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return api_fail(TKB_ERR_CUDA, "cuTensorMapEncodeTiled(operand) failed with CUresult %d", int(r));
    return TKB_OK;
}
// 3-D scale map over [row_blocks][k_chunks][128 x int32] (512-byte chunks), box = chunks_per_stage chunks.
static int make_scale_map(CUtensorMap* m, const void* base, uint64_t row_blocks, uint64_t k_chunks, uint32_t chunks_per_stage) {
    cuuint64_t dims[3] = {128, k_chunks, row_blocks};
    cuuint64_t strides[2] = {512, 512 * k_chunks};
    cuuint32_t box[3] = {128, chunks_per_stage, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = g_encode(m, CU_TENSOR_MAP_DATA_TYPE_INT32, 3, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return api_fail(TKB_ERR_CUDA, "cuTensorMapEncodeTiled(scales) failed with CUresult %d", int(r));
    return TKB_OK;
}

static int ensure_decode_scratch(DeviceCtx* c) {
    if (c->decode_partials) return TKB_OK;
    std::lock_guard<std::mutex> lk(g_ctx_mu);
    if (c->decode_partials) return TKB_OK;
    float* part = nullptr; unsigned int* flags = nullptr;
    TKB_CUDA(cudaMalloc(&part, kDecodeRing * kDecodePartialFloats * sizeof(float)));
    TKB_CUDA(cudaMalloc(&flags, kDecodeRing * kDecodeMaxGrid * sizeof(unsigned int)));
    TKB_CUDA(cudaMemset(flags, 0, kDecodeRing * kDecodeMaxGrid * sizeof(unsigned int)));
    TKB_CUDA(cudaDeviceSynchronize());
    c->decode_flags = flags;
    c->decode_partials = part;
    return TKB_OK;
}

// Skinny-M NVFP4 GEMM (M <= 128): X is the activation (A operand of the public call), W the weight.
static int decode_common(DeviceCtx* c, const void* X, const void* X_sc, const float* X_sg, const void* W, const void* W_sc,
                         const float* W_sg, void* D, int64_t ldd, int M, int N, int K, int prefetch_weights, void* stream) {
    if (int e = ensure_decode_scratch(c)) return e;
    DecodeArgs d;
    memset(&d, 0, sizeof(d));
    const int nb = decode_padded_rows(M);
    if (int e = make_operand_map(&d.tmW, W, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, uint64_t(K / 2), N, K / 2, 128)) return e;
    if (int e = make_operand_map(&d.tmX, X, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, uint64_t(K / 2), M, K / 2, nb)) return e;
    if (int e = make_scale_map(&d.tmSW, W_sc, (N + 127) / 128, K / 64, 4)) return e;
    if (int e = make_scale_map(&d.tmSX, X_sc, 1, K / 64, 4)) return e;
    {   // output tile of one 128-row weight slab: 128 columns of D x the padded activation rows, not swizzled
        cuuint64_t dims[2] = {uint64_t(N), uint64_t(M)};
        cuuint64_t strides[1] = {uint64_t(ldd) * 2};
        cuuint32_t box[2] = {128, uint32_t(nb)};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = g_encode(&d.tmD, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, D, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return api_fail(TKB_ERR_CUDA, "cuTensorMapEncodeTiled(skinny output) failed with CUresult %d", int(r));
    }
    unsigned call = 0;
    int ring = -1;
    {
        std::lock_guard<std::mutex> lk(g_ctx_mu);
        const cudaStream_t key = static_cast<cudaStream_t>(stream);
        for (int i = 0; i < kDecodeRing && ring < 0; i++)
            if (c->decode_stream_used[i] && c->decode_stream[i] == key) ring = i;
        for (int i = 0; i < kDecodeRing && ring < 0; i++)
            if (!c->decode_stream_used[i]) { c->decode_stream_used[i] = true; c->decode_stream[i] = key; ring = i; }
        if (ring >= 0) call = c->decode_calls[ring]++;
    }
    if (ring < 0)
        return api_fail(TKB_ERR_INVALID_ARG, "gemm (M <= 128): this device already runs the skinny-M kernel on %d other streams, which is as many scratch "
                                         "sets as the library keeps; use one of those streams", kDecodeRing);
    d.sgX = X_sg; d.sgW = W_sg; d.D = D; d.ldd = ldd; d.M = M; d.N = N; d.K = K;
    d.partials = c->decode_partials + ring * kDecodePartialFloats;
    d.flags = c->decode_flags + ring * kDecodeMaxGrid;
    d.epoch = call + 1;                         // strictly increasing per scratch set, never 0
    d.max_grid = kDecodeMaxGrid;
    d.status = c->status; d.sm_count = c->sm_count; d.stream = static_cast<cudaStream_t>(stream); d.prof = g_prof;
    d.prefetch_weights = prefetch_weights;
    TKB_CUDA(launch_decode(d));
    return TKB_OK;
}

static int pick_config(int kind, int config, int M, int N, int sm_count) {
    const bool dense = kind == KIND_BF16 || kind == KIND_FP8;
    if (config == TKB_GEMM_PAIR_M512_N256) return 4;
    if (config >= TKB_GEMM_PAIR_N256 && config <= TKB_GEMM_SINGLE_N128) return config - 1;
    // bf16: 512 x 256 cluster tiles (two 128-row halves of A per CTA) once they fill two waves of CTA pairs: measured 705 against
    // 728 us at 8192^3.  Not for fp8: its 4 stages of 48 KB hold half the K-time of the 6 x 32 KB ring (379 against 358-367 us).
    if (kind == KIND_BF16 && long((M + 511) / 512) * ((N + 255) / 256) >= sm_count) return 4;
    (void)dense;
    // default: CTA pairs; 256-wide N tiles unless that leaves most of the SMs without a tile
    const long tiles256 = long((M + 255) / 256) * ((N + 255) / 256);
    if (tiles256 * 2 >= sm_count || (N % 256 == 0 && tiles256 * 4 >= sm_count)) return 0;
    return 2;
}

// bf16 output map: box 64 columns x 32 rows, 128-byte swizzle (one epilogue warp's staging box)
int api_make_output_map(CUtensorMap* m, void* D, int rows, int cols, int64_t ldd) {
    cuuint64_t dims[2] = {uint64_t(cols), uint64_t(rows)};
    cuuint64_t strides[1] = {uint64_t(ldd) * 2};
    cuuint32_t box[2] = {64, 32};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = g_encode(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, D, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return api_fail(TKB_ERR_CUDA, "cuTensorMapEncodeTiled(output) failed with CUresult %d", int(r));
    return TKB_OK;
}

// NVFP4 A operand (codes + chunked scales) over M rows, for callers whose A has more rows than the output map they pass
int api_make_operand_a_maps(GemmArgs* gp, const void* A, const void* A_sc, int M, int K) {
    if (int e = make_operand_map(&gp->tmA, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, uint64_t(K / 2), M, K / 2, 128)) return e;
    return make_scale_map(&gp->tmSA, A_sc, (M + 127) / 128, K / 64, 4);
}

// Tensor maps of one GEMM call (g->kind / g->config already set).
int api_make_gemm_maps(GemmArgs* gp, int kind, const void* A, int64_t lda_bytes, const void* A_sc, const void* B, int64_t ldb_bytes,
                       const void* B_sc, void* D, int64_t ldd, int M, int N, int K) {
    GemmArgs& g = *gp;
    const int ctas = (g.config & 1) ? 1 : 2;
    const int bn = gemm_tile_n(g.config);
    const int elem_bytes = kind == KIND_BF16 ? 2 : 1;
    const CUtensorMapDataType dt = kind == KIND_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    const uint64_t inner = kind == KIND_NVFP4 ? uint64_t(K / 2) : uint64_t(K);
    if (int e = make_operand_map(&g.tmA, A, dt, elem_bytes, inner, M, lda_bytes, (g.config & 4) ? 256 : 128)) return e;
    if (int e = make_operand_map(&g.tmB, B, dt, elem_bytes, inner, N, ldb_bytes, bn / ctas)) return e;
    if (kind == KIND_NVFP4 || kind == KIND_MXFP8) {
        const int kc = kind == KIND_NVFP4 ? K / 64 : K / 128;
        const int per_stage = kind == KIND_NVFP4 ? 4 : 1;
        if (int e = make_scale_map(&g.tmSA, A_sc, (M + 127) / 128, kc, per_stage)) return e;
        if (int e = make_scale_map(&g.tmSB, B_sc, (N + 127) / 128, kc, per_stage)) return e;
    } else {
        g.tmSA = g.tmA; g.tmSB = g.tmB;
    }
    if (int e = api_make_output_map(&g.tmD, D, M, N, ldd)) return e;
    return TKB_OK;
}

unsigned long long* api_profile_buffer() { return g_prof; }

// A buffer of library-owned device scratch for temporaries that live for a few consecutive launches of one call (up to
// kSmallScratchRing calls may be in flight per device).  *ptr is null when the request is larger than a buffer: the
// caller then takes a path that needs none.
int api_small_scratch(size_t bytes, void** ptr) {
    *ptr = nullptr;
    DeviceCtx* c;
    if (int e = get_ctx(&c)) return e;
    if (bytes > kSmallScratchBytes) return TKB_OK;
    if (!c->small_scratch) {
        std::lock_guard<std::mutex> lk(g_ctx_mu);
        if (!c->small_scratch) {
            unsigned char* p = nullptr;
            TKB_CUDA(cudaMalloc(&p, kSmallScratchRing * kSmallScratchBytes));
            c->small_scratch = p;
        }
    }
    *ptr = c->small_scratch + (c->small_scratch_calls.fetch_add(1) % kSmallScratchRing) * kSmallScratchBytes;
    return TKB_OK;
}

int api_device(int* sm_count, int** status) {
    DeviceCtx* c;
    if (int e = get_ctx(&c)) return e;
    *sm_count = c->sm_count;
    *status = c->status;
    return TKB_OK;
}

static int gemm_common(int kind, const void* A, int64_t lda_bytes, const void* A_sc, const float* A_sg, const void* B,
                       int64_t ldb_bytes, const void* B_sc, const float* B_sg, void* D, int64_t ldd, int M, int N, int K, int config,
                       void* stream) {
    // pure argument errors first: they are reported the same way with or without a device
    if (!A || !B || !D) return api_fail(TKB_ERR_INVALID_ARG, "gemm: null operand pointer");
    if (M < 1 || N < 1 || K < 1) return api_fail(TKB_ERR_INVALID_ARG, "gemm: M, N, K must be positive (got %d, %d, %d)", M, N, K);
    if (config < 0 || config > TKB_GEMM_PAIR_M512_N256) return api_fail(TKB_ERR_INVALID_ARG, "gemm: unknown config %d", config);
    if (config == TKB_GEMM_PAIR_M512_N256 && kind != KIND_BF16 && kind != KIND_FP8)
        return api_fail(TKB_ERR_INVALID_ARG, "gemm: the 512 x 256 tile exists for the dense kinds only (the block-scaled kinds need the tensor memory for their scales)");
    if ((config == TKB_GEMM_SKINNY || config == TKB_GEMM_SKINNY_PREFETCH) && (kind != KIND_NVFP4 || M > 128))
        return api_fail(TKB_ERR_INVALID_ARG, "gemm: the skinny-M kernel needs NVFP4 operands and M <= 128");
    const int kmult = kind == KIND_NVFP4 ? 64 : (kind == KIND_MXFP8 ? 128 : (kind == KIND_FP8 ? 16 : 8));
    if (K % kmult) return api_fail(TKB_ERR_INVALID_ARG, "gemm: K=%d must be a multiple of %d for this format", K, kmult);
    if (N % 8) return api_fail(TKB_ERR_INVALID_ARG, "gemm: N=%d must be a multiple of 8", N);
    if (ldd == 0) ldd = N;
    if (ldd < N || ldd % 8) return api_fail(TKB_ERR_BAD_ALIGNMENT, "gemm: ldd=%lld must be >= N and a multiple of 8 elements", (long long)ldd);
    if (!aligned16(A) || !aligned16(B) || !aligned16(D) || lda_bytes % 16 || ldb_bytes % 16)
        return api_fail(TKB_ERR_BAD_ALIGNMENT, "gemm: operand base pointers and row pitches must be 16-byte aligned");
    if (kind == KIND_NVFP4 || kind == KIND_MXFP8) {
        if (!A_sc || !B_sc) return api_fail(TKB_ERR_INVALID_ARG, "gemm: null scale pointer");
        if (!aligned16(A_sc) || !aligned16(B_sc)) return api_fail(TKB_ERR_BAD_ALIGNMENT, "gemm: scale tensors must be 16-byte aligned");
    }
    if (kind == KIND_NVFP4 && (!A_sg || !B_sg)) return api_fail(TKB_ERR_INVALID_ARG, "gemm: null per-tensor scale pointer");
    DeviceCtx* c;
    if (int e = get_ctx(&c)) return e;

    if (kind == KIND_NVFP4 && M <= 128 && (config == TKB_GEMM_DEFAULT || config == TKB_GEMM_SKINNY || config == TKB_GEMM_SKINNY_PREFETCH))
        return decode_common(c, A, A_sc, A_sg, B, B_sc, B_sg, D, ldd, M, N, K, config == TKB_GEMM_SKINNY_PREFETCH ? 1 : 0, stream);

    GemmArgs g;
    memset(&g, 0, sizeof(g));
    g.kind = kind;
    g.config = pick_config(kind, config, M, N, c->sm_count);
    if (int e = api_make_gemm_maps(&g, kind, A, lda_bytes, A_sc, B, ldb_bytes, B_sc, D, ldd, M, N, K)) return e;
    g.sgA = A_sg; g.sgB = B_sg; g.M = M; g.N = N; g.K = K;
    g.status = c->status; g.prof = g_prof; g.sm_count = c->sm_count; g.stream = static_cast<cudaStream_t>(stream);
    TKB_CUDA(launch_gemm(g));
    return TKB_OK;
}

static int nvfp4_quantize_common(const void* A, int64_t lda, void* codes, void* sc, float* sg, const float* amax, int M, int K,
                                 int scale_2d, int arithmetic, void* stream, int sc_rowmajor = 0, const QuantExchange* xch = nullptr) {
    // sc_rowmajor: codes and scales share one row of K/2 + K/16 bytes (codes first); `sc` is ignored
    if (sc_rowmajor) sc = static_cast<uint8_t*>(codes) + K / 2;
    if (!A || !codes || !sc || !sg) return api_fail(TKB_ERR_INVALID_ARG, "nvfp4_quantize: null pointer");
    if (M < 1 || K < 64 || K % 64) return api_fail(TKB_ERR_INVALID_ARG, "nvfp4_quantize: need M >= 1 and K a positive multiple of 64 (got M=%d K=%d)", M, K);
    if (arithmetic < 0 || arithmetic > 2) return api_fail(TKB_ERR_INVALID_ARG, "nvfp4_quantize: unknown arithmetic %d", arithmetic);
    if (lda == 0) lda = K;
    if (lda < K || lda % 8) return api_fail(TKB_ERR_BAD_ALIGNMENT, "nvfp4_quantize: lda must be >= K and a multiple of 8 elements");
    if (!aligned16(A) || !aligned16(codes) || !aligned16(sc)) return api_fail(TKB_ERR_BAD_ALIGNMENT, "nvfp4_quantize: buffers must be 16-byte aligned");
    if (xch && amax && xch->world > 1) return api_fail(TKB_ERR_INVALID_ARG, "nvfp4_quantize: the cross-rank amax exchange belongs to the fused-amax kernel (no amax input)");
    DeviceCtx* c;
    if (int e = get_ctx(&c)) return e;
    NvQuantArgs a;
    a.A = A; a.lda = lda; a.codes = codes; a.ldc = sc_rowmajor ? K / 2 + K / 16 : K / 2; a.ldsc = K / 2 + K / 16; a.sc = sc; a.sg = sg; a.amax_in = amax;
    a.ws = c->quant_ws + (c->next_slot.fetch_add(1) % kQuantSlots);
    a.M = M; a.K = K; a.scale_2d = scale_2d ? 1 : 0; a.status = c->status;
    a.stream = static_cast<cudaStream_t>(stream); a.sm_count = c->sm_count; a.sc_rowmajor = sc_rowmajor;
    a.spin_limit = api_wait_limit();
    memset(&a.xch, 0, sizeof(a.xch));
    if (xch) a.xch = *xch;
    // Large tensors in the operand layout: the tile-per-CTA kernel, fed and drained by TMA (the launcher keeps the register-tile
    // kernels for tensors of at most two tiles per SM, which stay resident between the passes).
    static const int tma_env = getenv("TKB_NVQ_TMA") ? atoi(getenv("TKB_NVQ_TMA")) : 1;      // tuning aid: 0 = register-tile kernels only
    a.use_tiles = 0; a.wait_limit = api_wait_limit();
    memset(&a.tmA, 0, sizeof(a.tmA)); memset(&a.tmC, 0, sizeof(a.tmC));
    if (tma_env && !amax && !scale_2d && !sc_rowmajor && K % 128 == 0 && long((M + 127) / 128) * (K / 128) > 2L * c->sm_count) {
        cuuint64_t dims[2] = {uint64_t(K), uint64_t(M)};
        cuuint64_t strides[1] = {uint64_t(lda) * 2};
        cuuint32_t box[2] = {64, 128};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = g_encode(&a.tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(A), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return api_fail(TKB_ERR_CUDA, "cuTensorMapEncodeTiled(nvfp4_quantize input) failed with CUresult %d", int(r));
        cuuint64_t cdims[2] = {uint64_t(K / 2), uint64_t(M)};
        cuuint64_t cstrides[1] = {uint64_t(K / 2)};
        cuuint32_t cbox[2] = {64, 128};
        r = g_encode(&a.tmC, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, codes, cdims, cstrides, cbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return api_fail(TKB_ERR_CUDA, "cuTensorMapEncodeTiled(nvfp4_quantize output) failed with CUresult %d", int(r));
        a.use_tiles = 1;
    }
    TKB_CUDA(launch_nvfp4_quantize_mode(a, arithmetic));
    return TKB_OK;
}

// tkb_nvfp4_quantize_sharded plus an optional stamp: `stamp_count` device words that the kernel fills with `epoch`.
int api_quantize_sharded(const void* A_bf16, int64_t lda, void* codes, void* sc, float* sg, int M, int K, int layout, int arithmetic,
                         void* const* peer_slots, int world, int rank, unsigned int epoch, unsigned int* stamp, int stamp_count,
                         const unsigned int* epoch_ptr, void* stream) {
    if (world < 1 || world > 8 || rank < 0 || rank >= world) return api_fail(TKB_ERR_INVALID_ARG, "nvfp4_quantize_sharded: world must be 1..8 and 0 <= rank < world");
    if (layout != 0 && layout != 1) return api_fail(TKB_ERR_INVALID_ARG, "nvfp4_quantize_sharded: layout must be 0 (operand) or 1 (self-contained rows)");
    if (world > 1 && (!peer_slots || epoch == 0)) return api_fail(TKB_ERR_INVALID_ARG, "nvfp4_quantize_sharded: null slot table or epoch 0");
    QuantExchange x;
    memset(&x, 0, sizeof(x));
    x.world = world; x.rank = rank; x.epoch = epoch; x.stamp = stamp; x.stamp_count = stamp ? stamp_count : 0; x.epoch_ptr = epoch_ptr;
    for (int i = 0; i < world && world > 1; i++) {
        if (!peer_slots[i]) return api_fail(TKB_ERR_INVALID_ARG, "nvfp4_quantize_sharded: null slot array for rank %d", i);
        x.slots[i] = static_cast<unsigned long long*>(peer_slots[i]);
    }
    return nvfp4_quantize_common(A_bf16, lda, codes, layout ? nullptr : sc, sg, nullptr, M, K, 0, arithmetic, stream, layout, (world > 1 || stamp) ? &x : nullptr);
}

} // namespace tkb

using namespace tkb;

extern "C" {

int tkb_version(void) { return 100; }
const char* tkb_last_error(void) { return g_err; }

int tkb_gemm_set_profile_buffer(void* device_u64) {
    g_prof = static_cast<unsigned long long*>(device_u64);
    return TKB_OK;
}

int tkb_set_wait_limit_cycles(long long cycles) {
    if (cycles < 0) return api_fail(TKB_ERR_INVALID_ARG, "set_wait_limit_cycles: negative limit");
    g_wait_limit.store(cycles == 0 ? kDefaultWaitLimit : cycles, std::memory_order_relaxed);
    return TKB_OK;
}

int tkb_device_status(void* stream, int* status) {
    DeviceCtx* c;
    if (int e = get_ctx(&c)) return e;
    if (!status) return api_fail(TKB_ERR_INVALID_ARG, "device_status: null output");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    TKB_CUDA(cudaStreamSynchronize(s));
    TKB_CUDA(cudaMemcpy(status, c->status, sizeof(int), cudaMemcpyDeviceToHost));
    if (*status) {
        TKB_CUDA(cudaMemset(c->status, 0, sizeof(int)));
        // A kernel that gave up may have left its stream-K bookkeeping half way (flags raised and not put back): start
        // the skinny-M scratch from zero again.  The caller has just synchronised its stream; other streams' calls in flight
        // at this moment belong to the same failed state.
        if (c->decode_flags) {
            TKB_CUDA(cudaDeviceSynchronize());
            TKB_CUDA(cudaMemset(c->decode_flags, 0, kDecodeRing * kDecodeMaxGrid * sizeof(unsigned int)));
        }
    }
    return TKB_OK;
}

int tkb_nvfp4_quantize(const void* A_bf16, int64_t lda, void* codes, void* sc, float* sg, int M, int K, int scale_2d, int arithmetic,
                       void* stream) {
    return nvfp4_quantize_common(A_bf16, lda, codes, sc, sg, nullptr, M, K, scale_2d, arithmetic, stream);
}

int tkb_nvfp4_quantize_with_amax(const void* A_bf16, int64_t lda, void* codes, void* sc, float* sg, const float* amax, int M, int K,
                                 int scale_2d, int arithmetic, void* stream) {
    if (!amax) return api_fail(TKB_ERR_INVALID_ARG, "nvfp4_quantize_with_amax: null amax");
    return nvfp4_quantize_common(A_bf16, lda, codes, sc, sg, amax, M, K, scale_2d, arithmetic, stream);
}

int tkb_nvfp4_quantize_rows(const void* A_bf16, int64_t lda, void* rows, float* sg, const float* amax, int M, int K, int arithmetic,
                            void* stream) {
    if (!amax) return api_fail(TKB_ERR_INVALID_ARG, "nvfp4_quantize_rows: null amax");
    return nvfp4_quantize_common(A_bf16, lda, rows, nullptr, sg, amax, M, K, 0, arithmetic, stream, 1);
}

int tkb_nvfp4_quantize_sharded(const void* A_bf16, int64_t lda, void* codes, void* sc, float* sg, int M, int K, int layout, int arithmetic,
                               void* const* peer_slots, int world, int rank, unsigned int epoch, void* stream) {
    return api_quantize_sharded(A_bf16, lda, codes, sc, sg, M, K, layout, arithmetic, peer_slots, world, rank, epoch, nullptr, 0, nullptr, stream);
}

int tkb_absmax_bf16(const void* A_bf16, int64_t lda, int M, int K, float* amax, void* stream) {
    if (!A_bf16 || !amax) return api_fail(TKB_ERR_INVALID_ARG, "absmax: null pointer");
    if (M < 1 || K < 8 || K % 8) return api_fail(TKB_ERR_INVALID_ARG, "absmax: need M >= 1 and K a positive multiple of 8");
    if (lda == 0) lda = K;
    if (lda < K || lda % 8 || !aligned16(A_bf16)) return api_fail(TKB_ERR_BAD_ALIGNMENT, "absmax: A must be 16-byte aligned with lda %% 8 == 0");
    DeviceCtx* c;
    if (int e = get_ctx(&c)) return e;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    TKB_CUDA(cudaMemsetAsync(amax, 0, sizeof(float), s));
    TKB_CUDA(launch_absmax(A_bf16, lda, M, K, reinterpret_cast<unsigned int*>(amax), c->sm_count, s));
    return TKB_OK;
}

int tkb_mxfp8_quantize(const void* A_bf16, int64_t lda, void* codes, void* sc, int M, int K, void* stream) {
    if (!A_bf16 || !codes || !sc) return api_fail(TKB_ERR_INVALID_ARG, "mxfp8_quantize: null pointer");
    if (M < 1 || K < 128 || K % 128) return api_fail(TKB_ERR_INVALID_ARG, "mxfp8_quantize: need M >= 1 and K a positive multiple of 128 (got M=%d K=%d)", M, K);
    if (lda == 0) lda = K;
    if (lda < K || lda % 8) return api_fail(TKB_ERR_BAD_ALIGNMENT, "mxfp8_quantize: lda must be >= K and a multiple of 8 elements");
    if (!aligned16(A_bf16) || !aligned16(codes) || !aligned16(sc)) return api_fail(TKB_ERR_BAD_ALIGNMENT, "mxfp8_quantize: buffers must be 16-byte aligned");
    DeviceCtx* c;
    if (int e = get_ctx(&c)) return e;
    // Large tensors: one 128 x 128 tile per CTA, moved by TMA in both directions.  Small ones (fewer tiles than two per SM) keep
    // the register-tile kernel, whose 32-row tiles spread over more SMs.
    static const int tma_env = getenv("TKB_MXQ_TMA") ? atoi(getenv("TKB_MXQ_TMA")) : -1;      // tuning aid: 0 / 1 force a kernel
    const long tiles128 = long((M + 127) / 128) * (K / 128);
    const bool use_tiles = tma_env >= 0 ? tma_env != 0 : tiles128 >= 2L * c->sm_count;
    if (use_tiles) {
        CUtensorMap tmA, tmC;
        {
            cuuint64_t dims[2] = {uint64_t(K), uint64_t(M)};
            cuuint64_t strides[1] = {uint64_t(lda) * 2};
            cuuint32_t box[2] = {64, 128};
            cuuint32_t estr[2] = {1, 1};
            CUresult r = g_encode(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(A_bf16), dims, strides, box, estr,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return api_fail(TKB_ERR_CUDA, "cuTensorMapEncodeTiled(mxfp8_quantize input) failed with CUresult %d", int(r));
        }
        {
            cuuint64_t dims[2] = {uint64_t(K), uint64_t(M)};
            cuuint64_t strides[1] = {uint64_t(K)};
            cuuint32_t box[2] = {128, 128};
            cuuint32_t estr[2] = {1, 1};
            CUresult r = g_encode(&tmC, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, codes, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (r != CUDA_SUCCESS) return api_fail(TKB_ERR_CUDA, "cuTensorMapEncodeTiled(mxfp8_quantize output) failed with CUresult %d", int(r));
        }
        TKB_CUDA(launch_mxfp8_quantize_tiles(tmA, tmC, sc, M, K, c->status, api_wait_limit(), static_cast<cudaStream_t>(stream)));
        return TKB_OK;
    }
    TKB_CUDA(launch_mxfp8_quantize(A_bf16, lda, codes, K, sc, M, K, c->sm_count, static_cast<cudaStream_t>(stream)));
    return TKB_OK;
}

int tkb_fp32_to_fp4x2(const float* in, void* out, size_t n_pairs, void* stream) {
    if (!in || !out) return api_fail(TKB_ERR_INVALID_ARG, "fp32_to_fp4x2: null pointer");
    if (reinterpret_cast<uintptr_t>(in) & 7u) return api_fail(TKB_ERR_BAD_ALIGNMENT, "fp32_to_fp4x2: input must be 8-byte aligned");
    if (n_pairs == 0) return TKB_OK;
    DeviceCtx* c;
    if (int e = get_ctx(&c)) return e;
    TKB_CUDA(launch_fp32_to_fp4x2(in, out, n_pairs, static_cast<cudaStream_t>(stream)));
    return TKB_OK;
}
int tkb_fp4x2_to_fp32(const void* in, float* out, size_t n_pairs, void* stream) {
    if (!in || !out) return api_fail(TKB_ERR_INVALID_ARG, "fp4x2_to_fp32: null pointer");
    if (reinterpret_cast<uintptr_t>(out) & 7u) return api_fail(TKB_ERR_BAD_ALIGNMENT, "fp4x2_to_fp32: output must be 8-byte aligned");
    if (n_pairs == 0) return TKB_OK;
    DeviceCtx* c;
    if (int e = get_ctx(&c)) return e;
    TKB_CUDA(launch_fp4x2_to_fp32(in, out, n_pairs, static_cast<cudaStream_t>(stream)));
    return TKB_OK;
}

int tkb_nvfp4_gemm_ex(const void* A, const void* A_sc, const float* A_sg, const void* B, const void* B_sc, const float* B_sg, void* D,
                      int64_t ldd, int M, int N, int K, int config, void* stream) {
    return gemm_common(KIND_NVFP4, A, K / 2, A_sc, A_sg, B, K / 2, B_sc, B_sg, D, ldd, M, N, K, config, stream);
}
int tkb_nvfp4_gemm(const void* A, const void* A_sc, const float* A_sg, const void* B, const void* B_sc, const float* B_sg, void* D,
                   int64_t ldd, int M, int N, int K, void* stream) {
    return tkb_nvfp4_gemm_ex(A, A_sc, A_sg, B, B_sc, B_sg, D, ldd, M, N, K, TKB_GEMM_DEFAULT, stream);
}
int tkb_nvfp4_gemm_quant(const void* A, const void* A_sc, const float* A_sg, const void* B, const void* B_sc, const float* B_sg,
                         const float* out_amax, void* D_codes, void* D_sc, float* D_sg, int M, int N, int K, int arithmetic, void* stream) {
    if (!A || !A_sc || !A_sg || !B || !B_sc || !B_sg || !out_amax || !D_codes || !D_sc || !D_sg) return api_fail(TKB_ERR_INVALID_ARG, "gemm_quant: null pointer");
    if (M < 1 || N < 64 || N % 64 || K < 64 || K % 64) return api_fail(TKB_ERR_INVALID_ARG, "gemm_quant: need M >= 1, N %% 64 == 0, K %% 64 == 0 (got %d, %d, %d)", M, N, K);
    if (arithmetic != TKB_NVFP4_SPEC && arithmetic != TKB_NVFP4_KERNEL_IEEE)
        return api_fail(TKB_ERR_INVALID_ARG, "gemm_quant: the fused epilogue offers the two IEEE arithmetics only");
    if (!aligned16(A) || !aligned16(B) || !aligned16(A_sc) || !aligned16(B_sc) || !aligned16(D_codes) || !aligned16(D_sc))
        return api_fail(TKB_ERR_BAD_ALIGNMENT, "gemm_quant: buffers must be 16-byte aligned");
    DeviceCtx* c;
    if (int e = get_ctx(&c)) return e;
    GemmArgs g;
    memset(&g, 0, sizeof(g));
    g.kind = KIND_NVFP4; g.config = 0;
    // the bf16 output map is built over the code buffer only to have a valid descriptor: this mode never stores through it
    if (int e = api_make_gemm_maps(&g, KIND_NVFP4, A, K / 2, A_sc, B, K / 2, B_sc, D_codes, N, M, N, K)) return e;
    g.sgA = A_sg; g.sgB = B_sg; g.M = M; g.N = N; g.K = K;
    g.status = c->status; g.prof = g_prof; g.sm_count = c->sm_count; g.stream = static_cast<cudaStream_t>(stream);
    g.mode = MODE_QUANT;
    g.q_codes = D_codes; g.q_sc = D_sc; g.q_sg = D_sg; g.q_amax = out_amax; g.q_arith = arithmetic == TKB_NVFP4_SPEC ? 0 : 1;
    TKB_CUDA(launch_gemm(g));
    return TKB_OK;
}
int tkb_mxfp8_gemm_ex(const void* A, const void* A_sc, const void* B, const void* B_sc, void* D, int64_t ldd, int M, int N, int K,
                      int config, void* stream) {
    return gemm_common(KIND_MXFP8, A, K, A_sc, nullptr, B, K, B_sc, nullptr, D, ldd, M, N, K, config, stream);
}
int tkb_mxfp8_gemm(const void* A, const void* A_sc, const void* B, const void* B_sc, void* D, int64_t ldd, int M, int N, int K,
                   void* stream) {
    return tkb_mxfp8_gemm_ex(A, A_sc, B, B_sc, D, ldd, M, N, K, TKB_GEMM_DEFAULT, stream);
}
int tkb_bf16_gemm_ex(const void* A, int64_t lda, const void* B, int64_t ldb, void* D, int64_t ldd, int M, int N, int K, int config,
                     void* stream) {
    if (lda == 0) lda = K;
    if (ldb == 0) ldb = K;
    if (lda < K || ldb < K) return api_fail(TKB_ERR_INVALID_ARG, "bf16_gemm: lda/ldb must be >= K");
    return gemm_common(KIND_BF16, A, lda * 2, nullptr, nullptr, B, ldb * 2, nullptr, nullptr, D, ldd, M, N, K, config, stream);
}
int tkb_bf16_gemm(const void* A, int64_t lda, const void* B, int64_t ldb, void* D, int64_t ldd, int M, int N, int K, void* stream) {
    return tkb_bf16_gemm_ex(A, lda, B, ldb, D, ldd, M, N, K, TKB_GEMM_DEFAULT, stream);
}
int tkb_fp8_gemm_ex(const void* A, int64_t lda, const void* B, int64_t ldb, void* D, int64_t ldd, int M, int N, int K, int config,
                    void* stream) {
    if (lda == 0) lda = K;
    if (ldb == 0) ldb = K;
    if (lda < K || ldb < K) return api_fail(TKB_ERR_INVALID_ARG, "fp8_gemm: lda/ldb must be >= K");
    if (config == TKB_GEMM_SKINNY || config == TKB_GEMM_SKINNY_PREFETCH) return api_fail(TKB_ERR_INVALID_ARG, "fp8_gemm: no skinny-M kernel for this format");
    return gemm_common(KIND_FP8, A, lda, nullptr, nullptr, B, ldb, nullptr, nullptr, D, ldd, M, N, K, config, stream);
}
int tkb_fp8_gemm(const void* A, int64_t lda, const void* B, int64_t ldb, void* D, int64_t ldd, int M, int N, int K, void* stream) {
    return tkb_fp8_gemm_ex(A, lda, B, ldb, D, ldd, M, N, K, TKB_GEMM_DEFAULT, stream);
}

} // extern "C"
