// Device math shared by all kernels: activations, their derivatives from the
// pre-activation value, and the Adam update.  Formulas follow the reference's scalar
// definitions (include/deepity/utils/Activations.h:44-115, constants
// include/deepity/utils/activations/Gelu.h:19-22).  tanh and the logistic function are
// built from ex2.approx and the fast reciprocal: tanh(x) = 1 - 2/(e^(2x)+1), absolute error
// below 5e-7 over the whole range (measured against double), i.e. 200x inside the 1e-4
// parity bound against the CPU path and 2000x tighter than the tanh.approx.f32 instruction
// the reference GPU backend uses (src/backend/cuda/CUDACommon.cuh:42-93), at a quarter of
// the instruction count of libm's tanhf — the activation runs once per output element in
// every GEMM epilogue, so its cost is on the critical path.
#pragma once
#include <cuda_runtime.h>

#include "deepity_b200.h"

namespace dpc
{
constexpr float kGelu1 = 0.7978845608f;
constexpr float kGelu2 = 0.044715f;

__device__ __forceinline__ float fast_tanh(float x)
{
  // e^(2x) overflows to +inf (result 1) and underflows to 0 (result -1) gracefully.
  const float e = __expf(2.0f * x);
  return 1.0f - __fdividef(2.0f, e + 1.0f);
}

__device__ __forceinline__ float fast_sigmoid(float x)
{
  return __fdividef(1.0f, 1.0f + __expf(-x));
}

__device__ __forceinline__ float act_fwd(int act, float z)
{
  switch (act)
  {
  case DPC_ACT_RELU:
    return z > 0.0f ? z : 0.0f;
  case DPC_ACT_GELU:
  {
    float zsq = z * z;
    float inner = kGelu1 * z + (kGelu2 * kGelu1) * zsq * z;
    return 0.5f * z * (1.0f + fast_tanh(inner));
  }
  case DPC_ACT_SIGMOID:
    return fast_sigmoid(z);
  case DPC_ACT_ESIGMOID:
    return 0.5f + 0.5f * (z / (1.0f + fabsf(z)));
  case DPC_ACT_TANH:
    return fast_tanh(z);
  case DPC_ACT_HARD_TANH:
    return fminf(fmaxf(z, -1.0f), 1.0f);
  default:
    return z;
  }
}

__device__ __forceinline__ float act_deriv(int act, float z)
{
  switch (act)
  {
  case DPC_ACT_RELU:
    return z > 0.0f ? 1.0f : 0.0f;
  case DPC_ACT_GELU:
  {
    float zsq = z * z;
    float inner = kGelu1 * z + (kGelu2 * kGelu1) * zsq * z;
    float t = fast_tanh(inner);
    float gprime = kGelu1 + (3.0f * kGelu2 * kGelu1) * zsq;
    return 0.5f * (1.0f + t) + 0.5f * z * gprime * (1.0f - t * t);
  }
  case DPC_ACT_SIGMOID:
  {
    float s = fast_sigmoid(z);
    return s * (1.0f - s);
  }
  case DPC_ACT_ESIGMOID:
  {
    float a = 1.0f + fabsf(z);
    return 0.5f / (a * a);
  }
  case DPC_ACT_TANH:
  {
    float t = fast_tanh(z);
    return 1.0f - t * t;
  }
  case DPC_ACT_HARD_TANH:
    return (z > -1.0f && z < 1.0f) ? 1.0f : 0.0f;
  default:
    return 1.0f;
  }
}

// f'(preact) recovered from the activation value f(preact) itself, bit-identical to
// act_deriv(act, preact) for the activations where that is possible (see act_has_output_deriv).
__device__ __host__ __forceinline__ bool act_has_output_deriv(int act)
{
  return act == DPC_ACT_TANH || act == DPC_ACT_SIGMOID || act == DPC_ACT_RELU ||
         act == DPC_ACT_LINEAR || act == DPC_ACT_HARD_TANH;
}
__device__ __forceinline__ float act_deriv_from_output(int act, float f)
{
  switch (act)
  {
  case DPC_ACT_TANH:
    return 1.0f - f * f;
  case DPC_ACT_SIGMOID:
    return f * (1.0f - f);
  case DPC_ACT_RELU:
    return f > 0.0f ? 1.0f : 0.0f;
  case DPC_ACT_HARD_TANH:
    return (f > -1.0f && f < 1.0f) ? 1.0f : 0.0f;
  default:
    return 1.0f;
  }
}

// Activation and derivative together (one transcendental for tanh / sigmoid / gelu).
__device__ __forceinline__ void act_both(int act, float z, float& f, float& d)
{
  switch (act)
  {
  case DPC_ACT_TANH:
  {
    float t = fast_tanh(z);
    f = t;
    d = 1.0f - t * t;
    return;
  }
  case DPC_ACT_SIGMOID:
  {
    float s = fast_sigmoid(z);
    f = s;
    d = s * (1.0f - s);
    return;
  }
  case DPC_ACT_GELU:
  {
    float zsq = z * z;
    float inner = kGelu1 * z + (kGelu2 * kGelu1) * zsq * z;
    float t = fast_tanh(inner);
    float gprime = kGelu1 + (3.0f * kGelu2 * kGelu1) * zsq;
    f = 0.5f * z * (1.0f + t);
    d = 0.5f * (1.0f + t) + 0.5f * z * gprime * (1.0f - t * t);
    return;
  }
  default:
    f = act_fwd(act, z);
    d = act_deriv(act, z);
  }
}

// Eight elements at once with ONE dispatch on the activation: with a run-time activation id the
// per-element switch above costs a branch chain per element (a GEMM epilogue ran 3.5x slower with
// it than with a compile-time activation); here the branch is taken once per eight elements.
template <bool WITH_DERIV>
__device__ __forceinline__ void act_both8(int act, const float (&z)[8], float (&f)[8], float (&d)[8])
{
#define DPC_ACT8(A)                                        \
  case A:                                                  \
    _Pragma("unroll") for (int q = 0; q < 8; ++q)          \
    {                                                      \
      if (WITH_DERIV)                                      \
        act_both(A, z[q], f[q], d[q]);                     \
      else                                                 \
        f[q] = act_fwd(A, z[q]), d[q] = 1.0f;              \
    }                                                      \
    break;
  switch (act)
  {
    DPC_ACT8(DPC_ACT_RELU)
    DPC_ACT8(DPC_ACT_GELU)
    DPC_ACT8(DPC_ACT_SIGMOID)
    DPC_ACT8(DPC_ACT_ESIGMOID)
    DPC_ACT8(DPC_ACT_TANH)
    DPC_ACT8(DPC_ACT_HARD_TANH)
  default:
#pragma unroll
    for (int q = 0; q < 8; ++q)
      f[q] = z[q], d[q] = 1.0f;
  }
#undef DPC_ACT8
}

// Adam / AdamW step size, src/backend/CPUBackend.cpp:721-772:
// step = lr*sqrt(1-beta2^t)/(1-beta1^t), t already incremented (clamped to >= 1).
__device__ __forceinline__ float adam_step_size(float lr, int t)
{
  float tf = (float)(t < 1 ? 1 : t);
  float b1t = 1.0f - powf(0.9f, tf);
  float b2t = 1.0f - powf(0.999f, tf);
  return lr * sqrtf(b2t) / b1t;
}

// One element of the chunk kernels (src/backend/CPUBackendHighway.cpp:799-805,832-839).
// lr_wd < 0 means plain Adam, otherwise AdamW's decoupled decay p -= lr_wd*p first.
__device__ __forceinline__ float adam_update(float p, float g, float& m, float& v, float step,
                                              float lr_wd)
{
  const float b1 = 0.9f, b2 = 0.999f, eps = 1e-8f;
  m = b1 * m + (1.0f - b1) * g;
  v = b2 * v + (1.0f - b2) * (g * g);
  if (lr_wd >= 0.0f)
    p -= lr_wd * p;
  p -= step * m / (sqrtf(v) + eps);
  return p;
}
} // namespace dpc
