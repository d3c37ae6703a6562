/* tkb200 — C ABI of the B200 (sm_100a) quantized-inference kernels.
 *
 * Drop-in replacements for the entry points that ThunderKittens exposes through its per-kernel
 * pybind modules (`_C`).  Each function below names the reference entry it replaces (file:line in
 * the ThunderKittens tree).  Conventions shared by every call:
 *   - plain device pointers, sizes and a CUDA stream (cudaStream_t passed as void*; NULL = the
 *     legacy default stream); no torch types, no allocation of user buffers, no synchronisation;
 *   - the caller owns every input and output buffer, exactly as with the reference kernels
 *     (include/pyutils/torchutils.cuh:97-115 checks and wraps caller tensors);
 *   - return value: TKB_OK or an error code; tkb_last_error() gives the message of the calling
 *     thread's last failure.  Nothing here throws, prints or exits (the reference TORCH_CHECKs,
 *     throws std::runtime_error or exit()s: torchutils.cuh:35-83, common/util.cuh:412-431);
 *   - layouts are the reference's: e2m1 codes two per byte with element 2i in the low nibble,
 *     e4m3 / ue8m0 scales in 512-byte chunks of (128 rows x 4 K-blocks) with byte
 *     (row%32)*16 + (row/32%4)*4 + kblock%4, chunks ordered [row/128][kblock/4]
 *     (kernels/gemm/common.cuh:105-116), row-major bf16 outputs, both GEMM operands K-contiguous.
 *   - every device-side wait is bounded; a launch that gave up records TKB_ERR_TIMEOUT, visible
 *     through tkb_device_status().
 */
#ifndef TKB200_H
#define TKB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    TKB_OK = 0,
    TKB_ERR_INVALID_ARG = 1,   /* null pointer, bad size or unsupported shape */
    TKB_ERR_BAD_ALIGNMENT = 2, /* base pointers / leading dimensions must be 16-byte aligned */
    TKB_ERR_CUDA = 3,          /* a CUDA runtime or driver call failed */
    TKB_ERR_TIMEOUT = 4,       /* a bounded device-side wait ran out */
    TKB_ERR_UNSUPPORTED = 5,   /* not an sm_100 device / driver without tensor-map support */
    TKB_ERR_CAPACITY = 6       /* device status only: a caller-sized buffer was too small (MoE row capacity) */
};

/* NVFP4 quantizer arithmetic (see tkb_nvfp4_quantize) */
enum {
    TKB_NVFP4_SPEC = 0,        /* the reference's torch specification (test_quantize.py:9-52), IEEE fp32; reproducible on a CPU */
    TKB_NVFP4_KERNEL_IEEE = 1, /* the reference kernel's operation order, IEEE fp32 */
    TKB_NVFP4_KERNEL_FAST = 2  /* the reference kernel's operation order AND its --use_fast_math build: bit-identical to the
                                  reference kernel's output on a B200 (what the Python layer uses by default) */
};

/* GEMM tile configuration override for tkb_*_gemm_ex (0 = library default) */
enum {
    TKB_GEMM_DEFAULT = 0,
    TKB_GEMM_PAIR_N256 = 1,    /* two-CTA 256 x 256 tiles */
    TKB_GEMM_SINGLE_N256 = 2,  /* one-CTA 128 x 256 tiles */
    TKB_GEMM_PAIR_N128 = 3,    /* two-CTA 256 x 128 tiles */
    TKB_GEMM_SINGLE_N128 = 4,  /* one-CTA 128 x 128 tiles */
    TKB_GEMM_SKINNY = 5,       /* NVFP4, M <= 128: weight-streaming stream-K kernel (the default for such M) */
    TKB_GEMM_SKINNY_PREFETCH = 6, /* the same kernel for STATIC weights: the caller states that B, B_sc were complete before the
                                  kernel that precedes this call in the stream started (weights quantized ahead of time), so
                                  the kernel may load them while that kernel (typically the activation quantizer) still runs.
                                  With any other config nothing is read before the preceding kernel has finished. */
    TKB_GEMM_PAIR_M512_N256 = 7 /* dense kinds (bf16, fp8) only: two-CTA 512 x 256 tiles, two 128-row halves of A per CTA against the
                                  same B rows (the default for these kinds once the tiles fill the GPU) */
};

int tkb_version(void);
const char* tkb_last_error(void);

/* Status word written by kernels of the current device (0 = no kernel reported a problem).
 * Synchronises `stream`, returns the word through *status and clears it. */
int tkb_device_status(void* stream, int* status);

/* Upper bound, in SM clock cycles, on every device-side wait of kernels launched after the call (mbarrier waits, flag
 * spins, grid barriers, cross-rank exchanges); 0 restores the default of 2e9 cycles, about one second.  When a wait runs
 * out the kernel records TKB_ERR_TIMEOUT in the device status word, abandons its work and returns: outputs of that launch
 * are undefined, the context stays usable.  The reference's waits are unbounded (include/ops/thread/util/sync.cuh:311-318).
 * Process-wide. */
int tkb_set_wait_limit_cycles(long long cycles);

/* Diagnostics (no counterpart in the reference): when set to a device buffer of 8 x uint64 per launched CTA,
 * GEMM kernels record per-CTA wait cycles: [0] producer waiting for a free stage, [1] producer total (all-gather mode with push warps: cycles the CTA's push warps were busy),
 * [2] MMA thread waiting for the accumulator to be drained, [3] MMA thread waiting for operands, [4] MMA total,
 * [5] epilogue waiting for the accumulator, [6] epilogue drain, [7] producer waiting for rows of other ranks (all-gather
 * mode; its comm CTAs record [0] total, [1] waiting for peers' done flags, [2] fences and flag stores).  The skinny-M kernel
 * (M <= 128) records 16 words per CTA instead, in nanoseconds of the global timer: [0] start, [1] past the dependency wait, [2] first
 * stage issued, [3] last MMA issued, [4] epilogue done, [5] waiting for partial tiles of other CTAs, [6] MMA thread waiting for
 * operands, [7] epilogue busy, [8] tensor-memory loads, [9] partial-tile stores and publish, [10] output stores, [11] segments.
 * NULL (default) switches it off. */
int tkb_gemm_set_profile_buffer(void* device_u64);

/* ---- quantize ----------------------------------------------------------------------------- */

/* Replaces nvfp4_quantize(A_bf16, A_fp4x2, A_sc, A_sc_global, scale_2d)
 * (kernels/gemm/nvfp4_b200/nvfp4_b200_gemm.cu:772-794, kernels 356-545).
 *   A_bf16 [M, K] bf16, leading dimension lda elements (0 = K); K % 64 == 0; any M >= 1
 *   codes  [M, K/2] bytes; sc [ceil(M/128), K/64, 512] e4m3 (rows past M are written as 0);
 *   sg     fp32[1] = per-tensor decode scale amax/2688
 * One launch; the per-tensor amax pass is fused (cooperative grid). */
int tkb_nvfp4_quantize(const void* A_bf16, int64_t lda, void* codes, void* sc, float* sg, int M, int K, int scale_2d,
                       int arithmetic, void* stream);

/* Same, with the per-tensor amax supplied by the caller as a device float (row-sharded tensors:
 * reduce tkb_absmax_bf16 over the shards first so every shard quantizes like the full tensor). */
int tkb_nvfp4_quantize_with_amax(const void* A_bf16, int64_t lda, void* codes, void* sc, float* sg, const float* amax, int M,
                                 int K, int scale_2d, int arithmetic, void* stream);

/* Same arithmetic, but every row is written as one self-contained record rows[M, K/2 + K/16]: the row's K/2 code
 * bytes followed by its K/16 scale bytes in K order.  This is the form in which quantized rows travel between GPUs
 * (MoE dispatch re-tiles the scales into 512-byte chunks at the destination).  No counterpart in the reference,
 * whose dispatch moves bf16 rows.  K % 256 == 0. */
int tkb_nvfp4_quantize_rows(const void* A_bf16, int64_t lda, void* rows, float* sg, const float* amax, int M, int K, int arithmetic,
                            void* stream);

/* Quantize of a ROW-SHARDED tensor in one launch: every rank passes its own rows, the per-tensor amax is
 * max-reduced across the ranks inside the kernel (the last CTA to reach the kernel's grid barrier trades the rank's
 * maximum with the peers over NVLink: one posted store per peer, bounded polls), so all shards are quantized exactly
 * like the whole tensor and *sg is the same on every rank.  peer_slots[i]: rank i's array of `world` zero-initialised
 * 64-bit words in a symmetric buffer (as for tkb_amax_allreduce); epoch grows by one per call on a slot table and
 * consecutive calls must alternate between two tables (a peer may be one call ahead).  layout 0: codes [M, K/2] +
 * chunked scales `sc` (GEMM operand form); layout 1: self-contained rows as tkb_nvfp4_quantize_rows (`sc` unused).
 * world == 1 is tkb_nvfp4_quantize.  Every rank must make the call.  No counterpart in the reference. */
int tkb_nvfp4_quantize_sharded(const void* A_bf16, int64_t lda, void* codes, void* sc, float* sg, int M, int K, int layout, int arithmetic,
                               void* const* peer_slots, int world, int rank, unsigned int epoch, void* stream);

/* max |x| of a bf16 matrix into *amax (device float; overwritten).  Part of
 * nvfp4_quantize::absmax_kernel (nvfp4_b200_gemm.cu:360-418) exposed for sharded tensors. */
int tkb_absmax_bf16(const void* A_bf16, int64_t lda, int M, int K, float* amax, void* stream);

/* Replaces mxfp8_quantize(A_bf16, A_fp8, A_sc) (kernels/gemm/mxfp8_b200/mxfp8_b200_gemm.cu:605-619, kernel 328-430).
 *   codes [M, K] e4m3; sc [ceil(M/128), K/128, 512] ue8m0; K % 128 == 0 */
int tkb_mxfp8_quantize(const void* A_bf16, int64_t lda, void* codes, void* sc, int M, int K, void* stream);

/* Replace fp32_to_fp4x2 / fp4x2_to_fp32 (nvfp4_b200_gemm.cu:796-826); the caller allocates the output. */
int tkb_fp32_to_fp4x2(const float* in, void* out, size_t n_pairs, void* stream);
int tkb_fp4x2_to_fp32(const void* in, float* out, size_t n_pairs, void* stream);

/* ---- GEMM: D[M,N] bf16 = A[M,K] . B[N,K]^T ---------------------------------------------- */

/* Replaces nvfp4_gemm(A, A_sc, A_sc_global, B, B_sc, B_sc_global, D) (nvfp4_b200_gemm.cu:748-770).
 *   A [M, K/2] bytes, B [N, K/2] bytes (row pitch K/2); A_sc/B_sc swizzled e4m3 chunks with
 *   ceil(rows/128) row blocks; A_sg/B_sg fp32[1]; D [M, N] bf16 with leading dimension ldd (0 = N).
 *   K % 64 == 0, N % 8 == 0; any M, N (the reference needs M,N,K % 256 == 0).
 *   M <= 128 ("decode" shapes, which the reference kernel cannot run) goes to a weight-streaming kernel that
 *   uses library-owned scratch (per-CTA fp32 partial tiles), one set per stream: up to 4 streams of one device may
 *   use it (a fifth is refused with TKB_ERR_INVALID_ARG rather than sharing scratch with a call in flight).  A CUDA graph
 *   captured from such a call must not be replayed on several streams at once. */
int tkb_nvfp4_gemm(const void* A, const void* A_sc, const float* A_sg, const void* B, const void* B_sc, const float* B_sg,
                   void* D, int64_t ldd, int M, int N, int K, void* stream);
int tkb_nvfp4_gemm_ex(const void* A, const void* A_sc, const float* A_sg, const void* B, const void* B_sc, const float* B_sg,
                      void* D, int64_t ldd, int M, int N, int K, int config, void* stream);

/* The skinny-M NVFP4 GEMM (M <= 16) for callers that must not allocate device memory where they call it:
 * runtimes that reserve every buffer at start-up and forbid allocation on the request path, and plug-in "enqueue"
 * hooks that are not allowed to call cudaMalloc.  It has no counterpart in the reference.  Same operands and
 * result as tkb_nvfp4_gemm, but it neither creates the per-device context nor any scratch buffer: the stream-K
 * scratch (one 16 x 128 fp32 partial tile and a flag per CTA, about 1.3 MB) is an array built into the library,
 * which every GPU that loads the library holds until the process exits.  Hence the limit M <= 16; larger M is
 * rejected with TKB_ERR_INVALID_ARG.  The first call on a device looks up the array's device address; make that
 * first call outside any stream capture.  All calls on a device share the array: calls that may overlap on the
 * GPU (different streams) race and must be ordered by the caller.  Device-side timeouts are not reported. */
int tkb_nvfp4_gemm_skinny_static(const void* X, const void* X_sc, const float* X_sg, const void* W, const void* W_sc,
                                 const float* W_sg, void* D, int64_t ldd, int M, int N, int K, void* stream);

/* NVFP4 GEMM whose result leaves the kernel quantized to NVFP4 (no counterpart in the reference; the specification is
 * tkb_nvfp4_quantize_with_amax applied to the bf16 result of tkb_nvfp4_gemm, and the outputs are bit-identical to that
 * sequence): D_codes [M, N/2], D_sc [ceil(M/128), N/64, 512], D_sg[1], quantized with the caller's per-tensor amax
 * `out_amax` (device float, e.g. a calibrated activation range).  arithmetic: TKB_NVFP4_SPEC or TKB_NVFP4_KERNEL_IEEE.
 * N % 64 == 0, K % 64 == 0.  State: written and compiled, NOT yet run on a GPU, no test yet. */
int tkb_nvfp4_gemm_quant(const void* A, const void* A_sc, const float* A_sg, const void* B, const void* B_sc, const float* B_sg,
                         const float* out_amax, void* D_codes, void* D_sc, float* D_sg, int M, int N, int K, int arithmetic, void* stream);

/* Replaces mxfp8_gemm(A, A_sc, B, B_sc, D) (mxfp8_b200_gemm.cu:585-603).  K % 128 == 0, N % 8 == 0. */
int tkb_mxfp8_gemm(const void* A, const void* A_sc, const void* B, const void* B_sc, void* D, int64_t ldd, int M, int N, int K,
                   void* stream);
int tkb_mxfp8_gemm_ex(const void* A, const void* A_sc, const void* B, const void* B_sc, void* D, int64_t ldd, int M, int N, int K,
                      int config, void* stream);

/* Replaces the standalone bf16 GEMM (kernels/gemm/bf16_b200/bf16_b200_gemm.cu:61-253, launched at
 * l.300-330; it has no pybind entry).  lda/ldb in elements (0 = K); K % 8 == 0, N % 8 == 0. */
int tkb_bf16_gemm(const void* A, int64_t lda, const void* B, int64_t ldb, void* D, int64_t ldd, int M, int N, int K, void* stream);
int tkb_bf16_gemm_ex(const void* A, int64_t lda, const void* B, int64_t ldb, void* D, int64_t ldd, int M, int N, int K,
                     int config, void* stream);

/* Replaces the standalone dense fp8 GEMM (kernels/gemm/fp8_b200/fp8_b200_gemm.cu: the bf16 kernel with e4m3 operands,
 * checked at l.298 against reference_gemm<fp8e4m3, bf16>).  A [M, K], B [N, K] e4m3 bytes, lda/ldb in bytes (0 = K),
 * fp32 accumulation, bf16 out; K % 16 == 0, N % 8 == 0.
 * State: written and compiled, not yet run on a GPU; no GPU test covers it yet. */
int tkb_fp8_gemm(const void* A, int64_t lda, const void* B, int64_t ldb, void* D, int64_t ldd, int M, int N, int K, void* stream);
int tkb_fp8_gemm_ex(const void* A, int64_t lda, const void* B, int64_t ldb, void* D, int64_t ldd, int M, int N, int K,
                    int config, void* stream);

/* ---- single-node multi-GPU plumbing ------------------------------------------------------------
 * Replaces, for this path, TKParallelTensor / KittensBroker (include/pyutils/parallel_tensor.cuh:23-336,
 * include/pyutils/broker.cuh:340-547) and the device-side signal / wait helpers
 * (include/ops/thread/util/sync.cuh:296-327).  One process per GPU.  A symmetric buffer is a tkb_dev_alloc
 * allocation on every rank; its 64-byte CUDA IPC handle is exchanged by the host program and opened with
 * tkb_ipc_open, which yields a device pointer into the peer's memory (NVLink peer access). */
int tkb_dev_alloc(size_t bytes, void** ptr);          /* zero-filled, IPC-exportable device memory */
int tkb_dev_free(void* ptr);
int tkb_ipc_export(const void* ptr, void* handle64);
int tkb_ipc_open(const void* handle64, void** ptr);
int tkb_ipc_close(void* ptr);
/* Stores `value` into element `index` of a 32-bit flag array on every peer (system-scope release; peer_flags[i]
 * is rank i's array as seen from this rank).  Replaces signal_all (sync.cuh:301-309). */
int tkb_signal_peers(void* const* peer_flags, int world, int rank, int index, unsigned int value, int include_self, void* stream);
/* Blocks the stream until flags[i] >= value for all i != skip (bounded device-side wait; epochs only grow).
 * Replaces wait / barrier_all (sync.cuh:311-327). */
int tkb_wait_flags(const void* flags, int count, int skip, unsigned int value, void* stream);

/* max over the ranks of one float per rank (the per-tensor amax of a row-sharded tensor) without a library
 * collective: peer_slots[i] is rank i's array of `world` 64-bit slots (zero-initialised symmetric buffer), epoch a
 * counter that grows by one per call.  About one NVLink round trip.  No counterpart in the reference, which keeps
 * tensors whole. */
int tkb_amax_allreduce(void* const* peer_slots, int world, int rank, unsigned int epoch, const float* local, float* out, void* stream);

/* Contiguous all-to-all over NVLink by pushes.  Replaces tk_all_to_all(output, input, barrier, scatter_axis,
 * gather_axis) (kernels/parallel/all_to_all/all_to_all.cu:119-179) for the case where the scattered / gathered
 * axis is the outermost one: chunk p of `in` (bytes_per_peer bytes; the same chunk for everyone if gather != 0,
 * i.e. an all-gather) lands at offset rank * bytes_per_peer of peer p's output.  peer_counters[i] + counter_base:
 * `world` 32-bit counters on rank i, zero-initialised; epoch grows by one per call on the same counters.  The call
 * returns after enqueueing the pushes and a bounded wait for all incoming chunks. */
int tkb_all_to_all(void* const* peer_out, const void* in, size_t bytes_per_peer, int gather, int rank, int world, void* const* peer_counters,
                   int counter_base, unsigned int epoch, void* stream);

/* The general form of tk_all_to_all(output, input, barrier, scatter_axis, gather_axis) (all_to_all.cu:119-179, kernel 37-94):
 * `in` is this rank's 4-D tensor of dims[4] elements of elem_bytes each; element (i0,i1,i2,i3) goes to rank
 * i[scatter] / (dims[scatter] / world), at i[scatter] % (dims[scatter] / world) along the scatter axis and
 * i[gather] + dims[gather] * rank along the gather axis of that rank's output (dims with the scatter axis divided and the
 * gather axis multiplied by world).  The innermost axis (and its per-rank part when it is the scattered one) must be whole
 * 16-byte vectors.  peer_counters[i] + counter_base: 2 * world zero-initialised 32-bit counters on rank i; epoch grows by
 * one per call on the same counters and the tensor shape must not change between calls on them.  The call enqueues a
 * bounded all-ranks-entered hand-shake, the pushes and a bounded wait for all incoming data.
 * State: written and compiled, NOT yet run on a GPU. */
int tkb_all_to_all_4d(void* const* peer_out, const void* in, const long long* dims, int elem_bytes, int scatter_axis, int gather_axis, int rank,
                      int world, void* const* peer_counters, int counter_base, unsigned int epoch, void* stream);

/* Tensor-parallel all-gather GEMM, NVFP4.  Replaces all_gather_matmul(A, B, C, barrier, num_comm_sms)
 * (kernels/parallel/ag_gemm/ag_gemm_b200.cu:280-305; the reference ships bf16 and fp8 variants only).
 *   D[M, N_local] = gather_rows(Xq)[M, K] . W_local[N_local, K]^T.
 * peer_codes[i] / peer_scales[i]: rank i's gathered buffers ([M, K/2] bytes, [M/128, K/64, 512] bytes) as seen
 * from this rank; entry `rank` is local.  Each rank quantizes its M/world rows (with the all-reduced per-tensor
 * amax, so X_sg is the same everywhere) into its own slice of its own buffers; comm_ctas CTAs of the kernel push
 * that slice into every peer's buffers over NVLink while the rest multiply, own rows first.  peer_arrived[i]: rank
 * i's array of M/8 32-bit arrival epochs (entry `rank` local); a rank writes the entries of its own rows on every peer:
 * 4 per 256 gathered rows with comm CTAs or copy engines, 16 per 256 rows with push warps.
 * comm_ctas == TKB_AG_PUSH_WARPS: no CTA is set aside; every CTA of the kernel carries two extra warps that push a share of
 * the slice (16-row units, destinations in the order in which they need the rows, four at a time) while its other warps multiply; peer_done must be NULL (the caller orders the steps).  Before a buffer set is reused every peer must have finished reading it:
 *   - peer_done == NULL: the caller sees to that itself (tkb_signal_peers / tkb_wait_flags);
 *   - else peer_done[i] is rank i's array of `world` 32-bit epochs and exit_counter a zeroed device word owned by
 *     this rank: the kernel's last CTA stores `epoch` into entry `rank` of every peer's array, and its comm CTAs
 *     wait (bounded) for entry d of the local array to reach epoch - 2 before they first write to rank d
 *     (two buffer sets alternate, so epoch - 2 was the last reader of this one).
 * M % (256 * world) == 0. */
#define TKB_AG_COPY_ENGINES (-1)
#define TKB_AG_PUSH_WARPS (-2)
int tkb_ag_gemm_nvfp4(void* const* peer_codes, void* const* peer_scales, const float* X_sg, const void* W, const void* W_sc,
                      const float* W_sg, void* D, int64_t ldd, int M, int N_local, int K, int rank, int world, void* const* peer_arrived,
                      void* const* peer_done, void* exit_counter, unsigned int epoch, int comm_ctas, void* stream);

/* Diagnostics, host only (no GPU needed, no counterpart in the reference): enumerates, in order, the pieces that comm
 * CTA `comm_idx` of `comm_ctas` pushes in tkb_ag_gemm_nvfp4 for the given problem and rank.  Six values per piece:
 * destination rank, span (0 codes, 1 scales), byte offset in the gathered buffer, bytes, arrival-flag index, 1 if the
 * piece completes its unit.  Returns the number of pieces (even if larger than max_pieces), or -code on bad arguments. */
int tkb_debug_ag_schedule(int M, int K, int rank, int world, int comm_ctas, int comm_idx, int piece_bytes, long long* out, int max_pieces);
/* The same with `parts` flagged parts per 256-row block: 4 (comm CTAs) or 16 (push warps: comm_ctas = CTAs of the kernel). */
int tkb_debug_ag_schedule_parts(int M, int K, int rank, int world, int comm_ctas, int comm_idx, int piece_bytes, int parts, long long* out,
                                int max_pieces);

/* One call for a whole step of the column-parallel layer: tkb_nvfp4_quantize_sharded of the local rows into this rank's
 * slice, then the gather and the GEMM.  `st` holds the symmetric buffers of both buffer sets as seen from this rank (index
 * [set][rank]); the set used is epoch % 2, and epoch must grow by one per call, starting at 1, on every rank alike.
 *   comm_ctas > 0: the gather is done by that many CTAs of the GEMM kernel (tkb_ag_gemm_nvfp4, epoch hand-shake inside).
 *   comm_ctas == TKB_AG_PUSH_WARPS (-2): the gather is done by two extra warps in EVERY CTA of the GEMM kernel (SM-issued stores to
 *     a peer are bounded per SM, so all SMs pushing a little fills the links where a few comm CTAs cannot); two launches per
 *     step, no acknowledgement flags: the amax exchange inside the quantize kernel orders a step after every peer's previous one.
 *   comm_ctas == TKB_AG_COPY_ENGINES (-1): the gather is done by the GPU's copy engines: per peer one cudaMemcpyAsync for the codes, one for the
 *     scales and one for the arrival flags (stream order makes the flags land last), spread over the streams of st->copy in
 *     the order in which the peers need this rank's rows, while every SM multiplies (the GEMM kernel waits, bounded, on the
 *     arrival flags of each 256-row block).  One peer copy per call: no batched-copy API is involved.  In this mode the
 *     kernels take the epoch from st->epoch_counter on the device (the host's `epoch` only selects the buffer set), which
 *     is what allows tkb_ag_graph_create to record steps once and replay them.
 * Host-side convenience over the entry points above; no counterpart in the reference. */
typedef struct tkb_ag_state {
    int rank, world, M, K;
    void* codes[2][8];      /* [M, K/2] gathered codes */
    void* scales[2][8];     /* [M/128, K/64, 512] gathered scales */
    void* arrived[2][8];    /* [M/8] arrival epochs (M/64 in use unless push warps gather) */
    void* slots[2][8];      /* [world] 64-bit amax all-reduce slots */
    void* done[8];          /* [world] 32-bit "my kernel of epoch e is finished" flags */
    float* amax;            /* device scratch, 1 float */
    float* sg;              /* device, 1 float: the per-tensor scale of the gathered activations */
    void* exit_counter;     /* device, one zeroed 32-bit word */
    void* copy;             /* optional: handle from tkb_ag_copy_create, needed by the copy-engine gather (comm_ctas < 0) */
    void* epoch_counter;    /* copy-engine gather: device, one zeroed 32-bit word; the kernels keep the count of completed steps in it */
} tkb_ag_state;
/* Streams, events and the flag pattern of the copy-engine gather, for the current device: n_streams (1..4) copy streams,
 * stamp_count >= M / world / 64.  Store the handle in tkb_ag_state.copy; destroy it after the last call has finished. */
int tkb_ag_copy_create(int n_streams, int stamp_count, void** handle);
int tkb_ag_copy_destroy(void* handle);
int tkb_ag_linear_nvfp4(const tkb_ag_state* st, unsigned int epoch, const void* X_local_bf16, const void* W, const void* W_sc,
                        const float* W_sg, void* D, int64_t ldd, int N_local, int comm_ctas, int arithmetic, void* stream);

/* `steps` consecutive tkb_ag_linear_nvfp4 calls (copy-engine gather) recorded as ONE CUDA graph: step i reads X_local[i],
 * W[i], W_sc[i], W_sg[i] and writes D[i] (the arrays may repeat pointers), its epoch is first_epoch + i.  steps is even, so
 * that a replay always starts on the same buffer set; launch the graph only when the next epoch of the state has the parity
 * of first_epoch, and count `steps` epochs per launch.  Replaying takes one cudaGraphLaunch on the host instead of about
 * thirty driver calls per step, which matters when a step lasts ~100 us.  Every rank creates and launches its graph alike.
 * The quantize launches inside a graph keep the scratch slots they were recorded with.  No counterpart in the reference
 * (its kernels take per-call host arguments). */
int tkb_ag_graph_create(const tkb_ag_state* st, unsigned int first_epoch, int steps, const void* const* X_local_bf16, const void* const* W,
                        const void* const* W_sc, const float* const* W_sg, void* const* D, int64_t ldd, int N_local, int arithmetic, void** handle);
int tkb_ag_graph_launch(void* handle, void* stream);
int tkb_ag_graph_destroy(void* handle);

/* GEMM + reduce-scatter, NVFP4: the row-parallel partner of the all-gather GEMM.  Replaces gemm_rs / matmul_reduce_scatter
 * (kernels/parallel/gemm_rs/gemm_rs_b200.cu:77-200, entry 204-233; bf16 and fp8 operands there).  Every rank holds a K-slice
 * of both operands, A_r [M, K_local] and B_r [N, K_local] (NVFP4, each quantized on its own: the per-tensor scales are applied
 * per rank), and ends up with its M / world rows of D = sum_r A_r . B_r^T as bf16.  As in the reference, the partial tiles are
 * converted to bf16 and ADDED into the owner's rows by the memory system (cp.reduce.async.bulk.tensor ... add, over NVLink for
 * remote owners), so the sum over the ranks is a bf16 accumulation whose order is not fixed: results agree with an fp32 sum to
 * about 1e-2 relative, not bit for bit.  st->out[i]: rank i's output [M / world, N] bf16 (symmetric buffer), st->flags[i]:
 * rank i's 2 * world zeroed 32-bit epochs, st->maps: from tkb_rs_maps_create (tensor maps of all outputs, in device memory).
 * A call zeroes the rank's rows, exchanges flags (nobody adds before everybody has zeroed), multiplies, exchanges flags again
 * (the rows are complete when every rank's kernel has finished); epoch grows by one per call on every rank alike.
 * M % (256 * world) == 0, N % 8 == 0, K_local % 64 == 0. */
typedef struct tkb_rs_state {
    int rank, world, M, N;
    void* out[8];
    void* flags[8];
    void* maps;
} tkb_rs_state;
int tkb_rs_maps_create(const tkb_rs_state* st, void** device_maps);
int tkb_rs_maps_destroy(void* device_maps);
int tkb_gemm_rs_nvfp4(const tkb_rs_state* st, unsigned int epoch, const void* A, const void* A_sc, const float* A_sg, const void* B,
                      const void* B_sc, const float* B_sg, int K_local, void* stream);

/* ---- MoE layer -----------------------------------------------------------------------------------
 * Replaces moe_dispatch_gemm(pre_tokens, post_tokens, weights, outputs, padded_tokens_per_expert,
 * pull_dispatch_indices, barrier, num_comm_sms, num_padded_local_tokens)
 * (kernels/parallel/moe_dispatch_gemm/moe_dispatch_gemm_h100.cu:260-299; Hopper-only in the reference) and the
 * schedule its benchmark builds on the CPU (moe_dispatch_gemm/benchmark.py:112-166).  Experts are sharded
 * E/world per rank (expert e lives on rank e / (E/world)), tokens T/world per rank. */

/* softmax over E logits per token, top_k experts by probability (ties -> lower id), weights renormalised over the
 * chosen k.  logits [T, E] fp32 -> experts [T, top_k] int32, weights [T, top_k] fp32.  E % 32 == 0, E <= 256.
 * (The reference benchmark draws experts with torch.multinomial and has no gate weights: benchmark.py:112-121.) */
int tkb_moe_route(const float* logits, int T, int E, int top_k, int* experts, float* weights, void* stream);

/* Dispatch schedule on the device from the chosen experts of ALL tokens (experts_all [T, top_k], identical on every
 * rank).  Outputs: counts[E] (scratch), padded_per_expert[E] (counts rounded up to 128), and for this rank
 * pull_idx[cap_rows][2] = (source rank, source row) per row of its expert segments (ascending global token order,
 * (-1,-1) padding), block_expert[cap_rows/128] (local expert of each 128-row block), num_blocks[1], and
 * comb_idx[(T/world)*top_k][2] = (expert rank, row there) for this rank's own tokens.  If the rank's segments do
 * not fit in cap_rows the device status becomes TKB_ERR_CAPACITY and num_blocks is 0. */
int tkb_moe_schedule(const int* experts_all, int T, int top_k, int E, int world, int rank, int* counts, int* padded_per_expert,
                     int* pull_idx, int* block_expert, int* num_blocks, int* comb_idx, int cap_rows, void* stream);

/* Dispatch fused with the grouped expert GEMM: Y[row, :] = Xq[src(row)] . W[expert(row)]^T for every row of this
 * rank's expert segments.  peer_rows[i] [T/world, K/2 + K/16] are rank i's quantized tokens
 * (tkb_nvfp4_quantize_rows with the all-reduced amax; X_sg is that common scale);
 * codes [cap_rows, K/2] and scales [cap_rows/128, K/64, 512] are local operand buffers the kernel fills;
 * W [experts_local * I, K/2], W_sc [experts_local * I / 128, K/64, 512], W_sg[1]: the rank's stacked expert weights;
 * Y [cap_rows, I] bf16 (leading dimension ldy, 0 = I).  ready [world] / arrived [cap_rows/128]: epoch arrays.
 * comm_ctas > 0: that many CTAs of the GEMM kernel pull rows over NVLink while the others multiply.  comm_ctas == 0: a gather
 * kernel on all SMs pulls the rows first (16-byte loads, NVLink for remote rows) and publishes per-block arrival epochs, then
 * every SM multiplies; two launches.  K % 256 == 0, I % 128 == 0. */
int tkb_moe_dispatch_gemm(void* const* peer_rows, const float* X_sg, void* codes, void* scales,
                          const void* W, const void* W_sc, const float* W_sg, void* Y, int64_t ldy, const int* pull_idx,
                          const int* block_expert, const int* num_blocks, const void* ready, void* arrived, unsigned int epoch, int K,
                          int I, int experts_local, int cap_rows, int rank, int world, int comm_ctas, void* stream);

/* Combine (no counterpart in the reference): out[t, :] = bf16(sum_j weights[t,j] * Y_{rank(t,j)}[row(t,j), :]), fp32
 * accumulation in ascending j.  peer_Y[i]: rank i's Y buffer as seen from this rank. */
int tkb_moe_combine(void* const* peer_Y, int64_t ldy, const int* comb_idx, const float* weights, void* out, int T_local, int top_k, int I,
                    int world, void* stream);

/* One call for a whole layer: route -> exchange of the chosen experts -> schedule -> tkb_nvfp4_quantize_sharded of this
 * rank's tokens (self-contained rows) -> dispatch fused with the grouped GEMM -> combine, with the epoch hand-shakes in
 * between, all enqueued on `stream`.  `st` holds the symmetric buffers as seen from this rank (index [rank], or
 * [set][rank] for the two alternating sets; set = epoch % 2) and the rank's local work buffers; epoch grows by one per
 * call, starting at 1, on every rank alike.  logits_local [T/world, E] fp32, X_local [T/world, H] bf16, out [T/world, I]
 * bf16.  Host-side convenience over the entry points above; no counterpart in the reference. */
typedef struct tkb_moe_state {
    int rank, world, T, H, I, E, top_k, cap_rows;
    void* xq_rows[2][8];       /* [T/world, H/2 + H/16] quantized tokens */
    void* slots[2][8];         /* [world] 64-bit amax exchange slots */
    void* experts_all[2][8];   /* [T, top_k] int32: every token's chosen experts */
    void* Y[8];                /* [cap_rows, I] bf16 expert outputs */
    void* flags[8];            /* [3 * world] epochs: tokens quantized, expert outputs complete, call finished */
    void* counters[8];         /* [2 * world] arrival counters of the expert exchange */
    void* codes; void* scales; /* local operand buffers [cap_rows, H/2], [cap_rows/128, H/64, 512] */
    void* experts_local; void* weights;                 /* [T/world, top_k] int32 / fp32 */
    void* counts; void* padded;                         /* [E] int32 */
    void* pull_idx; void* block_expert; void* num_blocks; void* comb_idx; void* arrived;   /* as in tkb_moe_schedule / dispatch */
    float* sg;                 /* device, 1 float: per-tensor scale of the tokens */
} tkb_moe_state;
int tkb_moe_layer_nvfp4(const tkb_moe_state* st, unsigned int epoch, const float* logits_local, const void* X_local_bf16, const void* W,
                        const void* W_sc, const float* W_sg, void* out, int comm_ctas, int arithmetic, void* stream);

/* For bindings that mirror the state structs by hand (ctypes, cgo, JNI ...): which = 0 tkb_ag_state, 1 tkb_moe_state, 2 tkb_rs_state;
 * field 0 = sizeof, field i >= 1 = offsetof the i-th member in declaration order; -1 past the last member.  Host only. */
int tkb_debug_struct_layout(int which, int field);

#ifdef __cplusplus
}
#endif
#endif /* TKB200_H */
