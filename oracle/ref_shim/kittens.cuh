// CPU ORACLE support — test infrastructure only.
//
// Stand-in for ThunderKittens' umbrella header, used ONLY to compile the reference's
// kernels/gemm/common.cuh (its naive GEMM kernels, fill kernel and scale-swizzle index) as HOST
// code.  common.cuh needs two things from the real header: the CUDA execution-space keywords
// and built-in index variables, and `kittens::base_types::convertor<To,From>::convert`.  The
// convertors below use the same CUDA-toolkit host conversions the real ones do
// (include/common/base_types.cuh:549-660).  The kernel BODIES stay the reference's own text.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_fp4.h>

// CUDA built-ins, emulated per host thread (the driver loop in ref_host.cpp sets them).
extern thread_local dim3 blockIdx, threadIdx, blockDim, gridDim;

namespace kittens {
using bf16 = __nv_bfloat16;
using fp8e4m3 = __nv_fp8_e4m3;
using fp8e8m0 = __nv_fp8_e8m0;
namespace base_types {
template <typename To, typename From> struct convertor {
    static inline To convert(const From& u) { return (To)u; }
};
template <> struct convertor<float, bf16> { static inline float convert(const bf16& u) { return __bfloat162float(u); } };
template <> struct convertor<bf16, float> { static inline bf16 convert(const float& u) { return __float2bfloat16_rn(u); } };
template <> struct convertor<float, fp8e4m3> { static inline float convert(const fp8e4m3& u) { return float(u); } };
template <> struct convertor<fp8e4m3, float> { static inline fp8e4m3 convert(const float& u) { return __nv_fp8_e4m3(u); } };
template <> struct convertor<float, fp8e8m0> { static inline float convert(const fp8e8m0& u) { return float(u); } };
template <> struct convertor<fp8e8m0, float> { static inline fp8e8m0 convert(const float& u) { return __nv_fp8_e8m0(u); } };
} // namespace base_types
} // namespace kittens
