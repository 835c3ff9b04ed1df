// libDeepityCUDA.so for B200: the plugin the reference's loader looks for.
//
// The reference resolves its GPU backend at run time: CreateBackend(DEVICE_GPU)
// (src/backend/Backend.cpp:13-14) dlopens "libDeepityCUDA.so" next to the host module and calls
// the one exported symbol Deepity_CreateCUDABackend (src/backend/CUDAPluginLoader.cpp:52-107,
// src/backend/cuda/CUDAPluginExports.cpp:12-21), which returns a heap object implementing
// Deep::IComputeBackend (include/deepity/backend/IComputeBackend.h:18-625) that the host later
// deletes through the virtual destructor.  This file is that object for sm_100a: an unmodified
// reference network constructed with DEVICE_GPU drives the kernels of b200_backend.cu through it.
// It includes the reference's own interface header (from the reference checkout given at build
// time) -- a plugin has to match the vtable it is loaded against -- and nothing else of the
// reference.
//
// Error behaviour follows the reference's GPU backend: compute methods are noexcept and report
// CUDA failures on stderr (src/backend/cuda/CUDACommon.cuh:16-25), Allocate returns nullptr on
// failure, the constructor throws when no device is usable
// (src/backend/cuda/CUDABackendCore.cu:35-45).  The Try* fast paths that exist only for the CPU's
// oneDNN build, and the fused convolution entries, return false: the callers then take their
// documented MatMul / Im2Col fall-backs, which run here.
#include <deepity/backend/IComputeBackend.h>

#include <stdexcept>

#include "b200_backend.h"

namespace
{
using Deep::ActivationType;
using Deep::DeviceType;

inline int Id(ActivationType t)
{
  return static_cast<int>(t);
}
// a forward-flavoured type's derivative enumerator directly follows it
// (include/deepity/utils/ActivationType.h:15-32)
inline bool IsForward(ActivationType t)
{
  return t != ActivationType::NONE && (Id(t) % 2) == 0;
}

class B200Backend final : public Deep::IComputeBackend
{
public:
  B200Backend() : c(b200::create())
  {
    if (!c)
      throw std::runtime_error("DeepityCUDA (b200): no usable CUDA device");
  }
  ~B200Backend() override { b200::destroy(c); }

  // graphs
  void BeginGraphCapture(size_t slot) noexcept override { b200::graph_begin(c, slot); }
  bool EndGraphCapture(size_t slot) noexcept override { return b200::graph_end(c, slot); }
  void ReplayGraph(size_t slot) noexcept override { b200::graph_replay(c, slot); }
  void Synchronize() noexcept override { b200::synchronize(c); }

  // memory
  float* Allocate(size_t n) override { return b200::allocate(c, n); }
  void Free(float* p) noexcept override { b200::release(c, p); }
  void Zero(float* p, size_t n) noexcept override { b200::zero(c, p, n); }
  void Copy(float* dst, const float* src, size_t n) noexcept override { b200::copy(c, dst, src, n); }
  void Copy2D(float* dst, size_t dstStride, const float* src, size_t srcStride, size_t rows,
              size_t cols) noexcept override
  {
    b200::copy2d(c, dst, dstStride, src, srcStride, rows, cols);
  }
  void CopyFromHost(float* dst, const float* src, size_t n) noexcept override
  {
    b200::copy_from_host(c, dst, src, n);
  }
  void CopyToHost(float* dst, const float* src, size_t n) noexcept override
  {
    b200::copy_to_host(c, dst, src, n);
  }
  void RandomizeNormal(float* buf, size_t n, float mean, float stddev, uint32_t seed) noexcept override
  {
    b200::randomize_normal(c, buf, n, mean, stddev, seed);
  }
  void RandomizeUniform(float* buf, size_t n, float lo, float hi, uint32_t seed) noexcept override
  {
    b200::randomize_uniform(c, buf, n, lo, hi, seed);
  }
  // nothing here is sized by the batch or grown lazily: no scratch to prepare before a capture
  void PrepareForBatchSize(size_t) noexcept override {}
  bool PrewarmBatchedGemmScratch(size_t) noexcept override { return true; }
  bool PrewarmGroupedGemmScratch(bool, bool, int, int, int, int64_t, int64_t, int64_t,
                                 size_t) noexcept override
  {
    return true;
  }

  // GEMM
  void MatMul(bool ta, bool tb, int M, int N, int K, float alpha, const float* A, int lda,
              const float* B, int ldb, float beta, float* C, int ldc) noexcept override
  {
    b200::sgemm(c, ta, tb, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
  }
  void MatMulAccum(bool ta, bool tb, int M, int N, int K, float alpha, const float* A, int lda,
                   const float* B, int ldb, float beta, float* C, int ldc) noexcept override
  {
    b200::sgemm(c, ta, tb, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
  }
  void MatMulAccumMixed(bool ta, bool tb, int M, int N, int K, float alpha, const float* A, int lda,
                        const float* B, int ldb, float beta, float* C, int ldc) noexcept override
  {
    b200::sgemm(c, ta, tb, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
  }
  void SetAllowTF32(bool allow) noexcept override { b200::set_allow_tf32(c, allow); }
  void MatMulBatched(bool ta, bool tb, int M, int N, int K, float alpha, const float* const* A,
                     int lda, const float* const* B, int ldb, float beta, float* const* C, int ldc,
                     int batchCount) noexcept override
  {
    b200::sgemm_batched(c, ta, tb, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc, batchCount);
  }

  // reductions
  void SumRows(float* dst, const float* src, size_t batch, size_t width) noexcept override
  {
    b200::sum_rows(c, dst, src, batch, width, 1);
  }
  void SumRowsBatched(float* dst, const float* src, size_t batch, size_t width,
                      size_t layers) noexcept override
  {
    b200::sum_rows(c, dst, src, batch, width, layers);
  }
  void SumRowsAccum(float* dst, const float* src, size_t batch, size_t width) noexcept override
  {
    b200::sum_rows(c, dst, src, batch, width, 1);
  }
  float Sum(const float* buf, size_t n) noexcept override { return b200::sum(c, buf, n); }

  // elementwise
  void Scale(float* buf, size_t n, float alpha) noexcept override { b200::scale(c, buf, n, alpha); }
  void AxpyInto(float* y, const float* x, size_t n, float alpha) noexcept override
  {
    b200::axpy(c, y, x, n, alpha);
  }
  void AxpyIntoAccum(float* y, const float* x, size_t n, float alpha) noexcept override
  {
    b200::axpy(c, y, x, n, alpha);
  }
  void AxpyIntoFromAccum(float* y, const float* x, size_t n, float alpha) noexcept override
  {
    b200::axpy(c, y, x, n, alpha);
  }
  void AddBiasBroadcast(float* buf, const float* bias, size_t batch, size_t width) noexcept override
  {
    b200::add_bias(c, buf, bias, batch, width, 1);
  }
  void AddBiasBroadcastBatched(float* buf, const float* bias, size_t batch, size_t width,
                               size_t layers) noexcept override
  {
    b200::add_bias(c, buf, bias, batch, width, layers);
  }
  bool TryFusedMatMulBias(bool, bool, int, int, int, const float*, int, const float*, int, const float*,
                          float*, int) noexcept override
  {
    return false;
  }
  bool TryFusedMatMul(bool, bool, int, int, int, float, const float*, int, const float*, int, float*,
                      int) noexcept override
  {
    return false;
  }
  bool TryFusedFeedbackUpdate(ActivationType, int, int, int, const float*, const float*, float*,
                              const float*, float, float*, float*) noexcept override
  {
    return false;
  }

  // activations
  void Activation(ActivationType type, float* buf, size_t n) noexcept override
  {
    b200::activation(c, Id(type), buf, buf, n);
  }
  void ActivationInto(ActivationType type, float* dst, const float* src, size_t n) noexcept override
  {
    b200::activation(c, Id(type), dst, src, n);
  }
  void ActivationDerivative(ActivationType type, float* buf, size_t n, bool activated) noexcept override
  {
    b200::activation_derivative(c, Derivative(type), buf, buf, n, activated);
  }
  void ActivationDerivativeInto(ActivationType type, float* dst, const float* src,
                                size_t n) noexcept override
  {
    b200::activation_derivative(c, Derivative(type), dst, src, n, false);
  }
  void ActivationDerivativeIntoAccum(ActivationType type, float* dst, const float* src,
                                     size_t n) noexcept override
  {
    b200::activation_derivative(c, Derivative(type), dst, src, n, false);
  }

  // predictive coding
  void FusedStateUpdateMomentum(float* z, float* v, const float* feedback, ActivationType dType,
                                const float* e, size_t n, float ir, float beta) noexcept override
  {
    b200::state_update(c, z, v, feedback, Derivative(dType), e, n, ir, beta);
  }
  void FusedStateUpdate(float* z, const float* feedback, ActivationType dType, const float* e, size_t n,
                        float ir) noexcept override
  {
    b200::state_update(c, z, nullptr, feedback, Derivative(dType), e, n, ir, 0.0f);
  }
  float ComputeErrorAndEnergy(float* e, const float* z, const float* mu, size_t n) noexcept override
  {
    return b200::compute_error_energy(c, e, z, mu, n);
  }
  void ComputeError(float* e, const float* z, const float* mu, size_t n) noexcept override
  {
    b200::compute_error(c, e, z, mu, n);
  }
  bool TryComputeErrorAndActivation(ActivationType type, float* e, float* zF, const float* z,
                                    const float* mu, size_t n) noexcept override
  {
    b200::error_and_activation(c, Id(type), e, zF, z, mu, n);
    return true;
  }
  float ComputeSoftmaxCrossEntropyErrorAndEnergy(float* e, const float* z, const float* mu, size_t batch,
                                                 size_t width, float*) noexcept override
  {
    return b200::softmax_ce_error_energy(c, e, z, mu, batch, width);
  }
  void ComputeSoftmaxCrossEntropyError(float* e, const float* z, const float* mu, size_t batch,
                                       size_t width) noexcept override
  {
    b200::softmax_ce_error(c, e, z, mu, batch, width);
  }
  bool TryFusedForwardPass(ActivationType, const float*, const float*, const float*, float*, int, int,
                           int) noexcept override
  {
    return false;
  }

  // convolution
  void Im2Col(const float* input, int batch, int channels, int height, int width, int kh, int kw, int sh,
              int sw, int ph, int pw, float* columns) noexcept override
  {
    b200::im2col(c, input, batch, channels, height, width, kh, kw, sh, sw, ph, pw, columns);
  }
  void Col2Im(const float* columns, int batch, int channels, int height, int width, int kh, int kw,
              int sh, int sw, int ph, int pw, float* image) noexcept override
  {
    b200::col2im(c, columns, batch, channels, height, width, kh, kw, sh, sw, ph, pw, image);
  }
  void MaxPool2DForward(const float* input, int batch, int channels, int height, int width, int ph,
                        int pw, int sh, int sw, float* output, int* argmax) noexcept override
  {
    b200::maxpool_forward(c, input, batch, channels, height, width, ph, pw, sh, sw, output, argmax);
  }
  void MaxPool2DBackward(const float* outGrad, const int* argmax, int batch, int channels, int height,
                         int width, int outH, int outW, float* inGrad) noexcept override
  {
    b200::maxpool_backward(c, outGrad, argmax, batch, channels, height, width, outH, outW, inGrad);
  }
  void RepackForBatchedGemm(float* dst, const float* src, size_t batch, size_t rows,
                            size_t cols) noexcept override
  {
    b200::repack_for_batched_gemm(c, dst, src, batch, rows, cols);
  }
  bool TryFusedConvForward(const float*, const float*, float*, float, int, int, int, int, int, int, int,
                           int, int, int, int) noexcept override
  {
    return false;
  }
  bool TryFusedConvBackwardData(const float*, const float*, float*, float, int, int, int, int, int, int,
                                int, int, int, int, int) noexcept override
  {
    return false;
  }
  bool TryFusedConvBackwardFilter(const float*, const float*, float*, float, float, int, int, int, int,
                                  int, int, int, int, int, int, int) noexcept override
  {
    return false;
  }
  void PrepareConvWorkspace(int, int, int, int, int, int, int, int, int, int, int) noexcept override {}

  // optimizer
  void IncrementCounter(int* counter) noexcept override { b200::increment_counter(c, counter); }
  void CopyCounterToHost(int* hostDst, const int* counter) noexcept override
  {
    b200::counter_to_host(c, hostDst, counter);
  }
  void CopyCounterFromHost(int* counter, const int* hostSrc) noexcept override
  {
    b200::counter_from_host(c, counter, hostSrc);
  }
  void AdamStep(float* param, const float* grad, float* m, float* v, size_t n, const int* t,
                const float* lr, float beta1, float beta2, float eps) noexcept override
  {
    b200::adam(c, param, grad, m, v, n, t, lr, -1.0f, beta1, beta2, eps);
  }
  void AdamWStep(float* param, const float* grad, float* m, float* v, size_t n, const int* t,
                 const float* lr, float weightDecay, float beta1, float beta2,
                 float eps) noexcept override
  {
    b200::adam(c, param, grad, m, v, n, t, lr, weightDecay, beta1, beta2, eps);
  }

  DeviceType GetDeviceType() const noexcept override { return DeviceType::DEVICE_GPU; }
  std::uintptr_t GetStreamHandle() const noexcept override { return b200::stream_handle(c); }

  void MultiplyInto(float* dst, const float* a, const float* b, size_t n) noexcept override
  {
    b200::multiply(c, dst, a, b, n);
  }
  void MultiplyIntoAccum(float* dst, const float* a, const float* b, size_t n) noexcept override
  {
    b200::multiply(c, dst, a, b, n);
  }
  void FusedActivationDerivativeMultiply(float* dst, const float* a, float* activatedInOut,
                                         ActivationType dType, size_t n) noexcept override
  {
    b200::derivative_multiply(c, Derivative(dType), dst, a, activatedInOut, n, true, true);
  }
  void FusedActivationDerivativeMultiplyFromPreact(float* dst, const float* a, const float* preact,
                                                   ActivationType dType, size_t n) noexcept override
  {
    b200::derivative_multiply(c, Derivative(dType), dst, a, const_cast<float*>(preact), n, false, false);
  }
  void Fill(float* buf, size_t n, float value) noexcept override { b200::fill(c, buf, n, value); }
  void CenterRows(float* buf, size_t rows, size_t cols) noexcept override
  {
    b200::center_rows(c, buf, rows, cols);
  }
  void AddBiasPerChannel(float* buf, const float* bias, size_t channels, size_t spatial) noexcept override
  {
    b200::add_bias_per_channel(c, buf, bias, 1, channels, spatial);
  }
  void AddBiasPerChannelNCHW(float* buf, const float* bias, size_t batch, size_t channels,
                             size_t spatial) noexcept override
  {
    b200::add_bias_per_channel(c, buf, bias, batch, channels, spatial);
  }

  // precision-weighted ops
  float ComputePrecisionWeightedErrorAndEnergy(float* e, const float* z, const float* mu, const float* p,
                                               size_t batch, size_t width) noexcept override
  {
    return b200::precision_error_energy(c, e, z, mu, p, batch, width);
  }
  void ComputePrecisionWeightedError(float* e, const float* z, const float* mu, const float* p,
                                     size_t batch, size_t width) noexcept override
  {
    b200::precision_error(c, e, z, mu, p, batch, width);
  }
  void AxpyBroadcastInto(float* y, const float* x, const float* factor, size_t batch, size_t width,
                         float alpha) noexcept override
  {
    b200::axpy_broadcast(c, y, x, factor, batch, width, alpha);
  }
  void MultiplyBroadcastInto(float* dst, const float* a, const float* factor, const float* b,
                             size_t batch, size_t width) noexcept override
  {
    b200::multiply_broadcast(c, dst, a, factor, b, batch, width);
  }
  void UpdatePrecisionFromError(float* p, float* log_p, const float* e, size_t batch, size_t width,
                                float pr) noexcept override
  {
    b200::update_precision(c, p, log_p, e, batch, width, pr);
  }

private:
  // callers pass either flavour where a derivative is meant (the reference's dispatch tables key on
  // both): map a forward enumerator to its derivative, leave derivative enumerators and NONE alone
  static int Derivative(ActivationType t) { return IsForward(t) ? Id(t) + 1 : Id(t); }

  b200::Ctx* c;
};
} // namespace

extern "C" __attribute__((visibility("default"))) Deep::IComputeBackend* Deepity_CreateCUDABackend()
{
  return new B200Backend();
}
