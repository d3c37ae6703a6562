// Host-visible types of the quantize kernels (shared by api.cu and the kernel translation units).
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace tkb {

struct QuantWork {            // one slot of library-owned scratch per in-flight NVFP4 quantize call
    unsigned int amax_bits;   // running maximum of |x| as fp32 bits (non-negative floats order as uints)
    unsigned int arrived;     // grid-barrier arrival counter
    unsigned int departed;    // blocks that have consumed amax_bits; the last one re-zeroes the slot
    unsigned int pad;
};

// Row-sharded tensors: the per-tensor amax is max-reduced across the GPUs inside the quantize kernel (world <= 1: off).
// slots[p] = rank p's array of `world` 64-bit words (epoch << 32 | amax bits), word r written by rank r.
struct QuantExchange {
    unsigned long long* slots[8];
    int world, rank;
    unsigned int epoch;
    // optional: `stamp_count` words that block 0 fills with `epoch` (the arrival-flag pattern that copy engines
    // forward to the peers after the rows of this call, see tkb_ag_linear_nvfp4)
    unsigned int* stamp; int stamp_count;
    // optional: the epoch lives on the device (a count of completed steps, see tkb_ag_state.epoch_counter); the kernel then uses
    // *epoch_ptr + 1 and ignores `epoch`, so that the launch can be replayed from a CUDA graph
    const unsigned int* epoch_ptr;
};

struct NvQuantArgs {
    const void* A; int64_t lda; void* codes; int64_t ldc; void* sc; float* sg; const float* amax_in; QuantWork* ws;
    int M, K, scale_2d; int* status; cudaStream_t stream; int sm_count;
    long long spin_limit;   // clock cycles the grid barrier / cross-rank exchange may wait
    int sc_rowmajor;   // 0: 512-byte chunk layout (GEMM operand); 1: plain scale rows of K/16 bytes, ldsc bytes apart
    int64_t ldsc;
    QuantExchange xch;
    // optional (large tensors, K % 128 == 0): tensor maps of the input (bf16, box 64 x 128, 128-byte swizzle) and of the codes
    // (bytes, box 64 x 128, 64-byte swizzle) for the tile-per-CTA kernel; use_tiles = 0 keeps the register-tile kernels
    CUtensorMap tmA, tmC; int use_tiles;
    long long wait_limit;   // clock cycles a wait for a TMA load may last
};

} // namespace tkb
