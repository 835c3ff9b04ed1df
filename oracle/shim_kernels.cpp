// Oracle build shim (test infrastructure; never linked into the product).
//
// The reference CPU backend (src/backend/CPUBackend.cpp) calls a handful of
// elementwise kernels that live in a separate Google-Highway translation unit
// (declared in src/backend/CPUBackendHighway.h:36-131) and a few scalar SLEEF
// entry points.  Neither Highway nor a SLEEF development package exists in
// this image, so the functions are restated here as plain scalar loops from
// the formulas the reference documents for them (the scalar tails of
// src/backend/CPUBackendHighway.cpp:799-805,832-839 and
// include/deepity/utils/Activations.h:44-151).  Everything else in the oracle
// is the reference's own source, compiled where it lies.
#include <algorithm>
#include <cmath>
#include <cstddef>
#include <cstring>

#include <deepity/utils/Activations.h>

#include "CPUBackendHighway.h"

extern "C"
{
// Scalar SLEEF names used by Activations.h and CPUBackend::AdamStep; libm's
// float routines are correctly rounded to well under 1 ulp for these inputs.
float Sleef_tanhf_u10(float x) { return std::tanh(x); }
float Sleef_powf_u10(float a, float b) { return std::pow(a, b); }
float Sleef_sqrtf(float a) { return std::sqrt(a); }
float Sleef_expf_u10(float a) { return std::exp(a); }
float Sleef_logf_u10(float a) { return std::log(a); }
void scipy_openblas_set_num_threads(int);
void openblas_set_num_threads(int n) { scipy_openblas_set_num_threads(n); }
}

namespace Deep
{
void MultiplyIntoDispatch(float* dst, const float* a, const float* b, size_t n) noexcept
{
  for (size_t i = 0; i < n; ++i)
    dst[i] = a[i] * b[i];
}

void FillDispatch(float* buf, size_t n, float value) noexcept
{
  std::fill_n(buf, n, value);
}

void AddBiasPerChannelDispatch(float* buf, const float* bias, size_t channels,
                               size_t spatialSize) noexcept
{
  for (size_t c = 0; c < channels; ++c)
    for (size_t j = 0; j < spatialSize; ++j)
      buf[c * spatialSize + j] += bias[c];
}

void FusedActivationDerivativeMultiplyDispatch(float* dst, const float* a, float* activatedInOut,
                                               ActivationType dType, size_t n) noexcept
{
  for (size_t i = 0; i < n; ++i)
  {
    float d = ActivationDerivativeFromActivatedScalar(dType, activatedInOut[i]);
    dst[i] = a[i] * d;
    activatedInOut[i] = d;
  }
}

void FusedStateUpdateDispatch(float* z, const float* feedback, ActivationType dType, const float* e,
                              size_t n, float ir) noexcept
{
  for (size_t i = 0; i < n; ++i)
    z[i] += ir * ((feedback[i] * ActivationDerivativeScalar(dType, z[i])) - e[i]);
}

void FusedStateUpdateMomentumDispatch(float* z, float* v, const float* feedback,
                                      ActivationType dType, const float* e, size_t n, float ir,
                                      float beta) noexcept
{
  for (size_t i = 0; i < n; ++i)
  {
    float u = feedback[i] * ActivationDerivativeScalar(dType, z[i]) - e[i];
    v[i] = beta * v[i] + (1.0f - beta) * u;
    z[i] += ir * v[i];
  }
}

void FusedActivationDerivativeMultiplyFromPreactDispatch(float* dst, const float* a,
                                                          const float* preact, ActivationType dType,
                                                          size_t n) noexcept
{
  for (size_t i = 0; i < n; ++i)
    dst[i] = a[i] * ActivationDerivativeScalar(dType, preact[i]);
}

void ComputeSoftmaxCrossEntropyErrorRowDispatch(float* eRow, const float* zRow,
                                                 const float* muRow, size_t nextSize) noexcept
{
  float mx = muRow[0];
  for (size_t j = 1; j < nextSize; ++j)
    mx = std::max(mx, muRow[j]);
  float s = 0.0f;
  for (size_t j = 0; j < nextSize; ++j)
  {
    eRow[j] = std::exp(muRow[j] - mx);
    s += eRow[j];
  }
  for (size_t j = 0; j < nextSize; ++j)
    eRow[j] = zRow[j] - eRow[j] / s;
}

void AdamStepChunkDispatch(float* param, const float* grad, float* m, float* v, size_t start,
                           size_t end, float stepSize, float beta1, float beta2,
                           float eps) noexcept
{
  for (size_t i = start; i < end; ++i)
  {
    float g = grad[i];
    m[i] = beta1 * m[i] + (1.0f - beta1) * g;
    v[i] = beta2 * v[i] + (1.0f - beta2) * (g * g);
    param[i] -= stepSize * m[i] / (std::sqrt(v[i]) + eps);
  }
}

void AdamWStepChunkDispatch(float* param, const float* grad, float* m, float* v, size_t start,
                            size_t end, float stepSize, float beta1, float beta2, float eps,
                            float lrWeightDecay) noexcept
{
  for (size_t i = start; i < end; ++i)
  {
    float g = grad[i];
    m[i] = beta1 * m[i] + (1.0f - beta1) * g;
    v[i] = beta2 * v[i] + (1.0f - beta2) * (g * g);
    param[i] -= lrWeightDecay * param[i];
    param[i] -= stepSize * m[i] / (std::sqrt(v[i]) + eps);
  }
}

void ComputeErrorAndActivationChunkDispatch(float* e, float* zF, const float* z, const float* mu,
                                             ActivationType activationType, size_t start,
                                             size_t end) noexcept
{
  for (size_t i = start; i < end; ++i)
  {
    e[i] = z[i] - mu[i];
    zF[i] = ActivationScalar(activationType, z[i]);
  }
}
} // namespace Deep
