// CPU ORACLE support — test infrastructure only.
//
// Thin C exports of the HOST implementations of the narrow-float conversions that ship in the
// CUDA toolkit headers (cuda_fp4.h, cuda_fp8.h, cuda_bf16.h).  The reference kernels call exactly
// these functions (nvfp4_b200_gemm.cu:506,524,572,579; mxfp8_b200_gemm.cu:396-406;
// kernels/gemm/common.cuh:46,139-143,195-216), so they pin the hand-written codecs of
// tk_oracle.cpp.  Also stands in for the reference's CUDA-only `_C.fp32_to_fp4x2` /
// `_C.fp4x2_to_fp32` helpers when the reference's torch specs are imported on a machine
// without a GPU (tests/golden/make_golden.py).
//
// Build: g++ -O2 -I$CUDA_HOME/include -shared -fPIC (see oracle/build.py).
#include <cstddef>
#include <cstdint>
#include <cuda_fp8.h>
#include <cuda_fp4.h>
#include <cuda_bf16.h>

extern "C" {

void nvh_f32_to_e4m3(const float* in, uint8_t* out, size_t n) {
    for (size_t i = 0; i < n; i++) out[i] = __nv_cvt_float_to_fp8(in[i], __NV_SATFINITE, __NV_E4M3);
}
void nvh_e4m3_to_f32(const uint8_t* in, float* out, size_t n) {
    for (size_t i = 0; i < n; i++) { __nv_fp8_e4m3 v; v.__x = in[i]; out[i] = float(v); }
}
void nvh_f32_to_e8m0(const float* in, uint8_t* out, size_t n) {
    for (size_t i = 0; i < n; i++) out[i] = __nv_cvt_float_to_e8m0(in[i], __NV_SATFINITE, cudaRoundPosInf);
}
void nvh_e8m0_to_f32(const uint8_t* in, float* out, size_t n) {
    for (size_t i = 0; i < n; i++) { __nv_fp8_e8m0 v; v.__x = in[i]; out[i] = float(v); }
}
void nvh_fp32_to_fp4x2(const float* in, uint8_t* out, size_t n_pairs) {
    for (size_t i = 0; i < n_pairs; i++) {
        float2 v; v.x = in[2 * i]; v.y = in[2 * i + 1];
        out[i] = __nv_cvt_float2_to_fp4x2(v, __NV_E2M1, cudaRoundNearest);
    }
}
void nvh_fp4x2_to_fp32(const uint8_t* in, float* out, size_t n_pairs) {
    for (size_t i = 0; i < n_pairs; i++) {
        __nv_fp4x2_e2m1 v; v.__x = in[i];
        float2 f = static_cast<float2>(v);
        out[2 * i] = f.x; out[2 * i + 1] = f.y;
    }
}
void nvh_f32_to_bf16(const float* in, uint16_t* out, size_t n) {
    for (size_t i = 0; i < n; i++) { __nv_bfloat16 b = __float2bfloat16(in[i]); out[i] = *reinterpret_cast<uint16_t*>(&b); }
}

} // extern "C"
