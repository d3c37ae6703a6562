// Internal declarations shared by the translation units of libtkb200 (not part of the C ABI).
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace tkb {

enum GemmKind : int { KIND_BF16 = 0, KIND_MXFP8 = 1, KIND_NVFP4 = 2, KIND_FP8 = 3 };   // FP8: dense e4m3, no scales

struct QuantWork;
struct NvQuantArgs;

// quantize.cu / quantize_fast.cu
cudaError_t launch_nvfp4_quantize_mode(const NvQuantArgs& a, int mode);
cudaError_t launch_absmax(const void* A, int64_t lda, int M, int K, unsigned int* out_bits, int sm_count, cudaStream_t s);
cudaError_t launch_mxfp8_quantize(const void* A, int64_t lda, void* codes, int64_t ldc, void* sc, int M, int K, int sm_count,
                                  cudaStream_t s);
cudaError_t launch_mxfp8_quantize_tiles(const CUtensorMap& tmA, const CUtensorMap& tmC, void* sc, int M, int K, int* status, long long limit,
                                        cudaStream_t s);
cudaError_t launch_fp32_to_fp4x2(const float* in, void* out, size_t n_pairs, cudaStream_t s);
cudaError_t launch_fp4x2_to_fp32(const void* in, float* out, size_t n_pairs, cudaStream_t s);

// api.cu: clock cycles a device-side wait may last (tkb_set_wait_limit_cycles)
long long api_wait_limit();

// gemm.cu
constexpr int kMaxWorld = 8;
struct AgParams {
    const uint8_t* peer_codes[kMaxWorld];    // base of every rank's gathered-codes buffer [M, K/2] (own entry = local)
    const uint8_t* peer_scales[kMaxWorld];   // base of every rank's gathered-scales buffer [M/128, K/64, 512]
    uint8_t* codes; uint8_t* scales;         // this rank's buffers (same as peer_*[rank], writable)
    unsigned int* peer_arrived[kMaxWorld];   // every rank's arrival epochs, `parts` per 256 gathered rows ([M / 8] words allocated); the entries of
                                             // rank s's rows in rank r's array are written by rank s when those rows have landed on r
    unsigned int* peer_done[kMaxWorld];      // optional (all null = the caller orders the epochs itself): every rank's [world] array of
                                             // "kernel finished" epochs; entry s of rank r's array is written by rank s
    unsigned int* exit_counter;              // with peer_done: zeroed device word, counts the CTAs that have left the kernel
    unsigned int epoch;
    int rank, world, blocks_per_rank, comm_ctas;
    int parts;                               // arrival flags per 256 gathered rows: 4 (comm CTAs, copy engines) or 16 (push warps)
    int push_warps;                          // non-zero: every CTA of the kernel carries two extra warps that push this rank's rows
    // optional (comm_ctas == 0 only): a device word that counts completed steps.  The kernel waits for arrival epoch
    // *epoch_counter + 1 instead of `epoch`, and its last CTA to finish (exit_counter) adds one to the word.
    unsigned int* epoch_counter;
};

// MoE mode: dispatch (pull of routed token rows from their home ranks) fused with the grouped expert GEMM.
struct MoeParams {
    const uint8_t* peer_rows[kMaxWorld];     // every rank's quantized tokens [tokens_per_rank, K/2 + K/16]: codes, then that row's scales
    uint8_t* codes; uint8_t* scales;         // local gathered activations [cap_rows, K/2], chunked scales [cap_rows/128, K/64, 512]
    const int* pull_idx;                     // [cap_rows][2] (source rank, source row), -1 = padding
    const int* block_expert;                 // [cap_rows/128] local expert of each 128-row block
    const int* num_blocks;                   // device scalar: blocks in use
    const unsigned int* ready;               // [world] epochs: peers' tokens are quantized
    unsigned int* arrived;                   // [cap_rows/128] epochs: block is in local memory
    unsigned int epoch;
    int rank, world, comm_ctas, expert_rows; // expert_rows = rows of one expert's weight matrix (the GEMM's N)
};
enum GemmMode : int { MODE_PLAIN = 0, MODE_AG = 1, MODE_MOE = 2, MODE_QUANT = 4, MODE_RS = 8 };   // QUANT: the epilogue writes D as NVFP4; RS: reduce-scatter
struct CommParams { AgParams ag; MoeParams moe; };

struct GemmArgs {
    int kind;                 // GemmKind
    int config;               // bit 0: 0 = CTA pair (cta_group::2), 1 = single CTA; bit 1: 0 = N tile 256, 1 = N tile 128
    CUtensorMap tmA, tmB, tmSA, tmSB, tmD;   // tmD: bf16 output, box 64 columns x 32 rows, 128-byte swizzle
    const float* sgA; const float* sgB;
    int M, N, K;
    int* status;
    unsigned long long* prof;   // optional per-CTA wait counters, 8 x uint64 per CTA
    int sm_count;
    cudaStream_t stream;
    int mode;                 // GemmMode
    CommParams comm;
    // MODE_QUANT: D leaves the kernel as NVFP4 codes + chunked scales quantized with a caller-supplied amax
    void* q_codes; void* q_sc; float* q_sg; const float* q_amax; int q_arith;   // q_arith: 0 = spec association, 1 = kernel association (IEEE)
    // MODE_RS: the bf16 tiles are reduce-added into the output of the rank that owns their rows.  rs_maps: `rs_world` tensor maps in
    // DEVICE memory, map i over rank i's output [M / world, N] bf16 (box 64 x 32, 128-byte swizzle, as tmD); rs_rank rotates the tile order
    const CUtensorMap* rs_maps; int rs_rows_per_rank, rs_rank, rs_world;
};
cudaError_t launch_gemm(const GemmArgs& a);
int moe_dispatch_ring(int K);     // row slots the MoE dispatch ring gets for hidden size K (needs >= 24)
int gemm_tile_n(int config);
int gemm_tile_m(int config);

// decode.cu
struct DecodeArgs {
    CUtensorMap tmW, tmX, tmSW, tmSX;
    CUtensorMap tmD;          // D [M, N] bf16, leading dimension ldd: box 128 columns x padded rows, no swizzle
    const float* sgX; const float* sgW;
    void* D; int64_t ldd;
    int M, N, K;
    float* partials; unsigned int* flags; unsigned int epoch; int max_grid;
    int* status; int sm_count; cudaStream_t stream;
    unsigned long long* prof;   // optional per-CTA timeline, 8 x uint64 per CTA
    int prefetch_weights;       // TKB_GEMM_SKINNY_PREFETCH
};
cudaError_t launch_decode(const DecodeArgs& a);
int decode_padded_rows(int M);

} // namespace tkb
