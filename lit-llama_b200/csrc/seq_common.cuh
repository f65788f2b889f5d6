// Shared helpers of libb200seq (sequence-mixer kernels, sm_100a only).
#pragma once
#include "../../include/b2l_seq.h"
#include "b2l_common.cuh"

namespace b2l {

// An "act" element is bf16 or f32; kernels are templated on it and compute in f32.
template <typename T> __device__ __forceinline__ float ld_act(const T* p, size_t i);
template <> __device__ __forceinline__ float ld_act<__nv_bfloat16>(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }
template <> __device__ __forceinline__ float ld_act<float>(const float* p, size_t i) { return p[i]; }
template <typename T> __device__ __forceinline__ void st_act(T* p, size_t i, float v);
template <> __device__ __forceinline__ void st_act<__nv_bfloat16>(__nv_bfloat16* p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ void st_act<float>(float* p, size_t i, float v) { p[i] = v; }

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// A gated unit from the two halves of one product: act(a) * b, or the clamped unit g = min(a, limit),
// u = clamp(b, -limit, limit), g * sigmoid(1.702 g) * (u + 1).
__device__ __forceinline__ float gated_pair(float a, float b, int act, float limit) {
  if (act == B2L_SEQ_ACT_CLAMPED_SWISH) {
    const float g = fminf(a, limit), u = fminf(fmaxf(b, -limit), limit);
    return g * sigmoid_f(1.702f * g) * (u + 1.0f);
  }
  return (act == B2L_SEQ_ACT_GELU_TANH ? gelu_tanh_f(a) : (act == B2L_SEQ_ACT_SILU ? silu_f(a) : sigmoid_f(a))) * b;
}

// Calls `fn.template operator()<T>()` with the element type of act_dtype.
#define B2L_SEQ_DISPATCH(act_dtype, ...)                                   \
  do {                                                                     \
    if ((act_dtype) == B2L_BF16) { using act_t = __nv_bfloat16; __VA_ARGS__; } \
    else if ((act_dtype) == B2L_F32) { using act_t = float; __VA_ARGS__; }  \
    else { b2l::set_error("act_dtype %d unsupported", (int)(act_dtype)); return B2L_E_UNSUPPORTED; } \
  } while (0)

}  // namespace b2l
