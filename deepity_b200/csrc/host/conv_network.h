// Host-side convolutional network: the reference's SimpleConvPCNetwork / SimpleConvPCLayer API
// (include/deepity/networks/SimpleConvPCNetwork.h, include/deepity/layers/SimpleConvPCLayer.h)
// re-stated over the dpc_conv_* C ABI.  Same method names, argument meaning and call order;
// pointers returned by the layer accessors are DEVICE pointers.
#pragma once
#include "pc_network.h"

namespace Deep
{
class SimpleConvPCNetwork;

class SimpleConvPCLayer
{
public:
  float* GetBeliefs() noexcept { return d.z; }
  const float* GetErrors() const noexcept { return d.e; }
  const float* GetMu() const noexcept { return d.mu; }
  float* GetWeights() noexcept { return d.W; }
  float* GetBiases() noexcept { return d.b; }
  size_t GetInputSize() const noexcept { return (size_t)d.in_c * d.in_h * d.in_w; }
  size_t GetOutputSize() const noexcept { return (size_t)d.out_c * d.out_h * d.out_w; }
  size_t GetBatchSize() const noexcept { return (size_t)batch; }
  int GetInChannels() const noexcept { return d.in_c; }
  int GetOutChannels() const noexcept { return d.out_c; }
  int GetInHeight() const noexcept { return d.in_h; }
  int GetInWidth() const noexcept { return d.in_w; }
  int GetOutHeight() const noexcept { return d.out_h; }
  int GetOutWidth() const noexcept { return d.out_w; }
  int GetKernelH() const noexcept { return d.k_h; }
  int GetKernelW() const noexcept { return d.k_w; }
  float GetLearningRate() const noexcept { return d.lr; }
  float GetInferenceRate() const noexcept { return d.ir; }
  float GetLambda() const noexcept { return d.lmbda; }
  bool IsClamped() const noexcept { return clamped; }
  void InvalidateMuCache() noexcept { cacheValid = false; }
  ActivationType GetActivationType() const noexcept { return (ActivationType)d.act; }

  dpc_conv_layer d{};
  int batch = 0;
  bool clamped = false, cacheValid = false;
  // The reference keeps prediction and activation derivative in ONE buffer: CalculateState
  // leaves the prediction there, UpdateState the derivative; UpdateWeights gates the error
  // with whatever it finds.  true = "prediction", so a weight update must gate with mu.
  bool gateIsPrediction = true;
};

class SimpleConvPCNetwork
{
public:
  explicit SimpleConvPCNetwork(int batchSize, DeviceType device = DeviceType::DEVICE_GPU,
                               int deviceIndex = 0);
  ~SimpleConvPCNetwork();
  SimpleConvPCNetwork(const SimpleConvPCNetwork&) = delete;
  SimpleConvPCNetwork& operator=(const SimpleConvPCNetwork&) = delete;

  void AddLayer(int inChannels, int outChannels, int inHeight, int inWidth, int kernelH,
                int kernelW, int strideH, int strideW, int padH, int padW, float lr, float ir,
                float lmbda, ActivationType aType, ActivationType dType);
  void SetOptimizer(OptimizerType opt);
  void Compile();
  void RandomizeWeights(std::mt19937& rng, const char* distribution = "normal");
  void ResetState();
  void Clamp(const std::vector<float>& input);
  float CalculateState(bool needEnergy = true);
  void UpdateState();
  void UpdateWeights();
  void ProjectForward();
  void SetCenterWeights(bool enabled) { centerWeights = enabled; DropGraphs(); }
  void SetLearningRate(float lr);
  void SetInferenceRate(float ir);
  void SetLambda(float lmbda);
  void SetUseGraph(bool enabled) { useGraph = enabled; DropGraphs(); }

  float TrainStep(const std::vector<float>& x, const std::vector<float>& y, int inferenceSteps);
  float TrainStepWithProjection(const std::vector<float>& x, const std::vector<float>& y,
                                int inferenceSteps);
  std::vector<float> Predict(const std::vector<float>& x, int inferenceSteps);
  std::vector<float> PredictWithProjection(const std::vector<float>& x, int inferenceSteps);

  float TrainStepRaw(const float* x, size_t nx, const float* y, size_t ny, int steps,
                     bool withProjection, bool onDevice);
  void PredictRaw(const float* x, size_t nx, int steps, bool withProjection, float* out,
                  size_t nout);

  const std::vector<std::unique_ptr<SimpleConvPCLayer>>& GetLayers() const noexcept { return layers; }
  SimpleConvPCLayer* GetTerminalLayer() noexcept { return layers.back().get(); }
  int GetBatchSize() const noexcept { return batchSize; }
  dpc_ctx* Context() noexcept { return ctx; }
  dpc_conv_plan* Plan();
  bool IsCompiled() const noexcept { return plan != nullptr; }
  int64_t LaunchCount() const;
  bool FindTensor(int layer, const std::string& name, float** ptr, size_t* count);

private:
  void Check(int rc) const;
  void RequireCompiled() const;
  void SyncPlan();
  void DropGraphs();
  void ClampRaw(int layer, const float* data, size_t n, bool onDevice);
  void ForwardLayer(int i, int flags);
  void Settle(int steps);

  int batchSize;
  dpc_ctx* ctx = nullptr;
  dpc_conv_plan* plan = nullptr;
  std::vector<std::unique_ptr<SimpleConvPCLayer>> layers;
  std::vector<void*> allocations;
  float *pinnedX = nullptr, *pinnedY = nullptr, *pinnedOut = nullptr;
  OptimizerType opt = OptimizerType::SGD;
  bool centerWeights = false, useGraph = true, dirty = false;
  long graphKey[4] = {-1, -1, -1, -1};
};
} // namespace Deep
