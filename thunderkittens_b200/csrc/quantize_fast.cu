// NVFP4 quantize, "reference-kernel arithmetic" policy.  This translation unit is the only one
// compiled with --use_fast_math, like every ThunderKittens kernel (kernels/common.mk:40): the
// expressions below are the reference kernel's (nvfp4_b200_gemm.cu:421, 449, 506, 513, 519-521)
// written as plain C so that the compiler lowers `/` and `1.0f/x` to the same approximate
// division / reciprocal instructions it picks for the reference.  Results can differ from the IEEE
// policies at rounding ties; there is no CPU restatement of the approximate instructions.
#include "quantize_impl.cuh"
#include "internal.h"

namespace tkb {

struct ArithKernelFast {
    static __device__ __forceinline__ void global_scales(float amax, float& sg_dec, float& sg_enc) {
        float sg = amax;
        sg /= 6.0f * 448.0f;
        sg_dec = sg;
        sg_enc = 1.0f / fmaxf(sg_dec, 0.000000000001f);
    }
    static __device__ __forceinline__ float block_scale(float amax16, float sg_enc) { return amax16 / 6.0f * sg_enc; }
    static __device__ __forceinline__ float block_enc(float s_local, float sg_dec) { return 1.0f / fmaxf(s_local * sg_dec, 0.000000000001f); }
    static __device__ __forceinline__ float scale_value(float x, float s_enc) { return x * s_enc; }
};

cudaError_t launch_nvfp4_quantize_fast(const NvQuantArgs& a) { return launch_nvfp4_quantize<ArithKernelFast>(a); }

} // namespace tkb
