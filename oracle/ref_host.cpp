// CPU ORACLE support — test infrastructure only.
//
// Runs the reference's own naive GEMM kernels (kernels/gemm/common.cuh:73-98, 118-161, 173-231),
// its fill kernel (l.28-48) and its scale-swizzle index (l.105-116) on the host: every CUDA
// thread of the <<<grid, block>>> launch becomes one iteration of a loop that sets the emulated
// blockIdx/threadIdx.  common.cuh is compiled from where it lies in the reference tree; the only
// change is made on the fly by oracle/build.py, which strips the `<<<...>>>` launch syntax
// from the (unused here) launcher wrappers so a host compiler can parse the file.  The stripped
// intermediate lives in a temporary directory; the shared object goes to oracle/_ref/ and is never
// committed.
#include <omp.h>
#define KITTENS_BLACKWELL 1
#include "kittens.cuh"
#include REF_COMMON_CUH   // set by the build recipe to the stripped temporary copy

thread_local dim3 blockIdx, threadIdx, blockDim, gridDim;

namespace {
template <class F>
void launch2d(int M, int N, F body) {
    const int gx = (N + 15) / 16, gy = (M + 15) / 16;
#pragma omp parallel for collapse(2) schedule(dynamic, 4)
    for (int by = 0; by < gy; by++)
        for (int bx = 0; bx < gx; bx++) {
            blockDim = dim3(16, 16, 1);
            gridDim = dim3(gx, gy, 1);
            blockIdx = dim3(bx, by, 0);
            for (int ty = 0; ty < 16; ty++)
                for (int tx = 0; tx < 16; tx++) {
                    threadIdx = dim3(tx, ty, 0);
                    body();
                }
        }
}
} // namespace

extern "C" {

void tkref_nvfp4_gemm(const void* A, const void* A_sc, const float* A_sg, const void* B, const void* B_sc,
                      const float* B_sg, void* D, int M, int N, int K) {
    launch2d(M, N, [&] {
        reference_nvfp4_gemm_kernel<__nv_bfloat16>((__nv_bfloat16*)D, (const __nv_fp4x2_e2m1*)A, (const __nv_fp4x2_e2m1*)B,
                                                   (const __nv_fp8_e4m3*)A_sc, (const __nv_fp8_e4m3*)B_sc, A_sg, B_sg, M, N, K);
    });
}

void tkref_mxfp8_gemm(const void* A, const void* A_sc, const void* B, const void* B_sc, void* D, int M, int N, int K) {
    launch2d(M, N, [&] {
        reference_blockscaled_gemm_kernel<__nv_fp8_e4m3, __nv_fp8_e8m0, __nv_bfloat16, 32>(
            (__nv_bfloat16*)D, (const __nv_fp8_e4m3*)A, (const __nv_fp8_e4m3*)B, (const __nv_fp8_e8m0*)A_sc,
            (const __nv_fp8_e8m0*)B_sc, M, N, K);
    });
}

void tkref_bf16_gemm(const void* A, const void* B, void* D, int M, int N, int K) {
    launch2d(M, N, [&] {
        reference_gemm_kernel<__nv_bfloat16, __nv_bfloat16, true>((__nv_bfloat16*)D, (const __nv_bfloat16*)A,
                                                                  (const __nv_bfloat16*)B, M, N, K);
    });
}

// fp8 (e4m3) dense GEMM as kernels/gemm/fp8_b200/fp8_b200_gemm.cu:298 checks it
void tkref_fp8_gemm(const void* A, const void* B, void* D, int M, int N, int K) {
    launch2d(M, N, [&] {
        reference_gemm_kernel<__nv_fp8_e4m3, __nv_bfloat16, true>((__nv_bfloat16*)D, (const __nv_fp8_e4m3*)A,
                                                                  (const __nv_fp8_e4m3*)B, M, N, K);
    });
}

void tkref_fill_uniform_f32(float* out, size_t n, uint64_t seed, float lo, float hi) {
    const size_t nb = (n + 255) / 256;
    for (size_t b = 0; b < nb; b++) {
        blockDim = dim3(256, 1, 1);
        gridDim = dim3((unsigned)nb, 1, 1);
        blockIdx = dim3((unsigned)b, 0, 0);
        for (int t = 0; t < 256; t++) {
            threadIdx = dim3(t, 0, 0);
            fill_kernel<float, FillMode::RANDOM>(out, n, seed, lo, hi);
        }
    }
}

// OpenMP threads of this library's parallel loops (launchers such as torchrun export OMP_NUM_THREADS=1)
void tkref_set_num_threads(int n) { if (n > 0) omp_set_num_threads(n); }

int tkref_scale_swizzle_idx(int row, int k_block, int k_blocks) { return scale_swizzle_idx(row, k_block, k_blocks); }

} // extern "C"
