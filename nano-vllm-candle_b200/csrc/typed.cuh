// Element access for kernels that exist in two storage formats: bf16 (serving) and fp32 (the exact mode, every
// product and sum in IEEE binary32, no tensor-core path).  Arithmetic is fp32 in both.
#pragma once
#include "common.cuh"

#ifdef __CUDACC__
template <typename T> __device__ __forceinline__ float ld_f(const T* p);
template <> __device__ __forceinline__ float ld_f<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ld_f<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

template <typename T> __device__ __forceinline__ void st_f(T* p, float v);
template <> __device__ __forceinline__ void st_f<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void st_f<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// the library's accurate tanh (the build does not use fast-math): (1 - e) / (1 + e) loses digits near zero
__device__ __forceinline__ float tanh_f32(float x) { return tanhf(x); }
__device__ __forceinline__ float sigmoid_f32(float x) { return 1.0f / (1.0f + expf(-x)); }
// gelu, tanh form: 0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))
__device__ __forceinline__ float gelu_tanh_f32(float z) {
  return 0.5f * z * (1.0f + tanh_f32(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
#endif

// dispatch on NVC_DT_* : FN is a generic lambda called with a null pointer of the element type
#define NVC_DISPATCH_DT(dt, T, ...)                      \
  do {                                                   \
    if ((dt) == NVC_DT_F32) { using T = float; __VA_ARGS__; } \
    else { using T = __nv_bfloat16; __VA_ARGS__; }       \
  } while (0)
