// Activation arithmetic shared by the stand-alone activation kernels (activation.cu) and the fused epilogue of
// the tensor-core grouped GEMM (gemm_tc.cu). Formulas: scattermoe/mlp.py:41, :81-87 and
// scattermoe/utils/replace_moe.py:39-43, :76-83 of the reference.
#pragma once

#include <cuda_runtime.h>

namespace smoe {

enum { LAYOUT_PLAIN = 0, LAYOUT_GLU_SECOND = 1, LAYOUT_GLU_FIRST = 2, LAYOUT_GPT_OSS = 3 };
enum { ACT_SILU = 0, ACT_GELU_ERF = 1, ACT_GELU_TANH = 2, ACT_RELU = 3, ACT_IDENTITY = 4 };

// FAST (16-bit storage): hardware exp2 / reciprocal approximations, relative error ~1e-6, far below the 2^-9 of
// the rounding to bf16 that follows; the IEEE expf + division of the exact path made these kernels ALU-bound
// (2.7 TB/s measured on the backward pass). fp32 storage keeps the exact path.
template <bool FAST>
__device__ __forceinline__ float sigmoidf_(float x) {
  return FAST ? __fdividef(1.0f, 1.0f + __expf(-x)) : 1.0f / (1.0f + expf(-x));
}

// The activation function is a template parameter: with a run-time `switch` inside the element loop the compiler
// evaluated every branch (erff, tanhf, exp) and selected, which made the fused GEMM epilogue twice as slow as the
// GEMM itself. Callers switch ONCE around a block of elements with SMOE_ACT_SWITCH.
template <int ACT, bool FAST>
__device__ __forceinline__ float act_fwd(float x) {
  if (ACT == ACT_SILU) return x * sigmoidf_<FAST>(x);
  if (ACT == ACT_GELU_ERF) return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
  if (ACT == ACT_GELU_TANH) {
    const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    return 0.5f * x * (1.0f + tanhf(u));
  }
  if (ACT == ACT_RELU) return x > 0.f ? x : 0.f;
  return x;
}

template <int ACT, bool FAST>
__device__ __forceinline__ float act_bwd(float x) {   // d act(x) / dx
  if (ACT == ACT_SILU) {
    const float s = sigmoidf_<FAST>(x);
    return s * (1.0f + x * (1.0f - s));
  }
  if (ACT == ACT_GELU_ERF) {
    const float cdf = 0.5f * (1.0f + erff(x * 0.70710678118654752f));
    const float pdf = 0.3989422804014327f * (FAST ? __expf(-0.5f * x * x) : expf(-0.5f * x * x));
    return cdf + x * pdf;
  }
  if (ACT == ACT_GELU_TANH) {
    const float x2 = x * x;
    const float u = 0.7978845608028654f * (x + 0.044715f * x * x2);
    const float t = tanhf(u);
    const float du = 0.7978845608028654f * (1.0f + 3.0f * 0.044715f * x2);
    return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * du;
  }
  if (ACT == ACT_RELU) return x > 0.f ? 1.f : 0.f;
  return 1.f;
}

// Runs BODY with `ACT_` bound to the compile-time value of the run-time activation code `act`.
#define SMOE_ACT_SWITCH(act, ...)                                             \
  switch (act) {                                                              \
    case ::smoe::ACT_SILU: { constexpr int ACT_ = ::smoe::ACT_SILU; __VA_ARGS__ } break;            \
    case ::smoe::ACT_GELU_ERF: { constexpr int ACT_ = ::smoe::ACT_GELU_ERF; __VA_ARGS__ } break;    \
    case ::smoe::ACT_GELU_TANH: { constexpr int ACT_ = ::smoe::ACT_GELU_TANH; __VA_ARGS__ } break;  \
    case ::smoe::ACT_RELU: { constexpr int ACT_ = ::smoe::ACT_RELU; __VA_ARGS__ } break;            \
    default: { constexpr int ACT_ = ::smoe::ACT_IDENTITY; __VA_ARGS__ } break;                      \
  }

}  // namespace smoe
