// Host-side networks: the reference's C++ network API re-stated over the dpc_* C ABI.
//
// Deep::SimplePCNetwork / DirectKPPCNetwork / FullPCNetwork keep the method names,
// argument meaning and call order of the reference classes
// (include/deepity/networks/{SimplePCNetwork,DirectKPPCNetwork,FullPCNetwork}.h) so that
// code written against them keeps compiling; underneath, every phase is one or a few
// grouped kernel launches on flat device buffers instead of one backend call per
// primitive per layer.  This file includes only deepity_b200.h: it talks to the GPU
// exclusively through the C ABI.
#pragma once
#include <cstdint>
#include <memory>
#include <random>
#include <stdexcept>
#include <string>
#include <vector>

#include "deepity_b200.h"

namespace Deep
{
// A dpc_* call returned a negative status; carries it through the C++ layer to the C ABI.
struct StatusError : std::runtime_error
{
  int status;
  StatusError(int rc, const std::string& msg) : std::runtime_error(msg), status(rc) {}
};

enum class DeviceType
{
  DEVICE_CPU,
  DEVICE_GPU
};

// Same enumerators and order as include/deepity/utils/ActivationType.h:15-32.
enum class ActivationType : uint8_t
{
  RELU,
  dRELU,
  GELU,
  dGELU,
  SIGMOID,
  dSIGMOID,
  eSIGMOID,
  d_eSIGMOID,
  TANH,
  dTANH,
  LINEAR,
  dLINEAR,
  HARD_TANH,
  dHARD_TANH,
  NONE
};

enum class OptimizerType
{
  SGD,
  ADAM,
  ADAMW
};

enum class NetworkKind
{
  SIMPLE = 0,
  DIRECT_KP = 1,
  FULL = 2
};

class PCNetwork;

// A layer as the reference exposes it: sizes, hyper-parameters and DEVICE pointers.
class PCLayer
{
public:
  size_t GetInputSize() const noexcept { return (size_t)d.size; }
  size_t GetOutputSize() const noexcept { return (size_t)d.next_size; }
  size_t GetTerminalSize() const noexcept { return (size_t)d.terminal_size; }
  size_t GetBatchSize() const noexcept { return (size_t)batch; }
  size_t GetPsiStride() const noexcept { return (size_t)d.psi_stride; }
  float* GetBeliefs() noexcept { return d.z; }
  const float* GetErrors() const noexcept { return d.e; }
  const float* GetMu() const noexcept { return d.mu; }
  float* GetWeights() noexcept { return d.W; }
  float* GetBiases() noexcept { return d.b; }
  const float* GetDirectFeedbackWeights() const noexcept { return d.Psi; }
  bool IsClamped() const noexcept { return clamped; }
  void InvalidateMuCache() noexcept { cacheValid = false; }
  float GetLearningRate() const noexcept { return d.lr; }
  float GetInferenceRate() const noexcept { return d.ir; }
  float GetFeedbackRate() const noexcept { return d.fl; }
  float GetLambda() const noexcept { return d.lmbda; }
  float GetMuPCScale() const noexcept { return d.a; }
  ActivationType GetActivationType() const noexcept { return (ActivationType)d.act; }

  dpc_layer d{};
  int batch = 0;
  bool clamped = false;
  bool cacheValid = false;
};

class PCNetwork
{
public:
  PCNetwork(NetworkKind kind, int batchSize, int device = 0);
  virtual ~PCNetwork();
  PCNetwork(const PCNetwork&) = delete;
  PCNetwork& operator=(const PCNetwork&) = delete;

  void AddLayerImpl(size_t size, size_t nextSize, size_t terminalSize, float lr, float ir,
                    float fl, float lmbda, ActivationType aType);
  void Compile();
  void RandomizeWeights(std::mt19937& rng, const char* distribution = "normal");

  void ResetState(bool beliefsOverwritten = false);
  void Clamp(const std::vector<float>& input);
  void ClampHost(int layer, const float* data, size_t n);
  void ClampDevice(int layer, const float* data, size_t n);
  void UnclampTerminal() { layers.back()->clamped = false; }

  void ProjectForward();
  float CalculateTerminalError();
  void DirectFeedbackUpdate();
  float CalculateState(bool needEnergy);
  void UpdateState();
  float Step(bool computeEnergy = true);
  void UpdateWeights();

  float TrainStep(const std::vector<float>& x, const std::vector<float>& y, int inferenceSteps);
  std::vector<float> Predict(const std::vector<float>& x, int inferenceSteps);

  // mode 0: TrainStep; 1: SimplePCNetwork::TrainStepWithProjection; 2: the Python-level
  // SimplePCN.train_step loop.  Pointers are host (onDevice=false) or device memory.
  float TrainStepRaw(int mode, const float* x, size_t nx, const float* y, size_t ny, int steps,
                     bool onDevice, bool readEnergy);
  void PredictRaw(const float* x, size_t nx, int steps, bool withProjection, float* out,
                  size_t nout);

  void SetOptimizer(OptimizerType o);
  void SetPsiOptimizer(OptimizerType o);
  void SetCenterWeights(bool enabled);
  void SetLearningRate(float lr);
  void SetFeedbackRate(float fl);
  void SetInferenceRate(float ir);
  void SetPsiDecay(float decay);
  void SetUseCrossEntropy(bool enabled);
  void SetUseMuPCScaling(bool enabled);
  void SetUseResidualConnections(bool enabled);
  void SetUseIPC(bool enabled);
  void SetUseEPC(bool enabled);
  void EPCStep();
  void SetUseMomentum(bool enabled, float beta = 0.9f);
  void SetPrecision(int precision);
  void SetUseGraph(bool enabled);
  // Layer sharding: the last layer is a copy of the neighbour rank's first layer (it owns no
  // weights here but carries that layer's Psi); the terminal error arrives by broadcast.
  void SetGhostTop(bool enabled);
  float* TerminalErrorBuffer() noexcept { return ghostET; }
  // Batch sharding: this network holds batchSize of globalBatch rows; every weight-shaped
  // update is split into "stage raw gradient sums", a call of `sync` (which sums `count`
  // floats at `dev` over the shards, ordered on `stream`) and "apply with globalBatch".
  // sync == nullptr returns to the fused updates.  Steps are not captured into a graph
  // while a sync function is set.
  using GradientSyncFn = int (*)(void* user, float* dev, int64_t count, void* stream);
  void SetGradientSync(GradientSyncFn sync, void* user, int globalBatch);
  float* GradientBuffer(size_t* count) noexcept
  {
    *count = gradCount;
    return gradBuffer;
  }

  std::vector<std::unique_ptr<PCLayer>>& GetLayers() noexcept { return layers; }
  PCLayer* GetTerminalLayer() noexcept { return layers.back().get(); }
  int GetBatchSize() const noexcept { return batchSize; }
  NetworkKind GetKind() const noexcept { return kind; }
  dpc_ctx* Context() noexcept { return ctx; }
  dpc_plan* Plan() noexcept { return plan; }
  bool IsCompiled() const noexcept { return plan != nullptr; }
  // Re-uploads the layer table if a setter changed it since the last step and brings lazily
  // skipped predictions up to date.
  void FlushSettings()
  {
    SyncPlan();
    RefreshPredictions(); // whoever drives single phases next expects mu / preact in memory
  }
  int64_t LaunchCount() const;
  double TrainStepFlops(int steps) const;

  // Tensor lookup for the binding layer; returns false when the layer has no such tensor.
  bool FindTensor(int layer, const std::string& name, float** ptr, size_t* rows, size_t* cols,
                  size_t* stride);
  // Device address of an Adam / AdamW step counter ("step", "psi_step":
  // Layer::GetOptimizerCounters) or nullptr when the layer has none.
  int32_t* Counter(int layer, const std::string& name);
  // One entry per tensor of Layer::GetStateDict() / GetOptimizerStateDict() of every weight layer.
  struct StateEntry
  {
    int layer;
    std::string name;
    size_t rows, cols, stride;
    bool optimizer;
  };
  std::vector<StateEntry> StateDict();

private:
  void Check(int rc) const;
  void RequireCompiled() const;
  void Dirty(); // hyper-parameters changed: re-upload the plan, drop captured graphs
  void SyncPlan();
  void EnsureOptimizerState();
  void EnsureGradientStaging();
  void RefreshPredictions();
  void SyncGradients(size_t count);
  void ForwardRange(int first, int count, int flags);
  void RunTrainPhases(int mode, int steps);
  void RunPredictPhases(int steps, bool withProjection);

  NetworkKind kind;
  int batchSize;
  dpc_ctx* ctx = nullptr;
  dpc_plan* plan = nullptr;
  std::vector<std::unique_ptr<PCLayer>> layers;
  std::vector<void*> allocations;
  float* pinnedX = nullptr;
  float* pinnedY = nullptr;
  float* pinnedOut = nullptr;

  OptimizerType opt = OptimizerType::SGD, optPsi = OptimizerType::SGD;
  bool centerWeights = false, crossEntropy = false, useMuPC = false, useResidual = false;
  bool useEPC = false, useIPC = false, useMomentum = false, useGraph = true, dirty = false;
  bool adamAllocated = false, psiAdamAllocated = false, pendingAsync = false;
  float momentumBeta = 0.9f, psiDecay = -1.0f;
  bool ghostTop = false;
  float* ghostET = nullptr;
  GradientSyncFn gradSync = nullptr;
  void* gradUser = nullptr;
  int globalBatch = 0;
  float* gradBuffer = nullptr; // [g_W of every layer | g_b | g_Psi], each padded to 64 floats
  size_t gradCount = 0, gradWCount = 0;
  bool predictionsStale = false; // mu / preact in memory are older than the last energy pass
  bool sweepFeedsDfa = false; // inside a DirectKP train step, between sweep and direct feedback
  int transientFlag = 0; // DPC_FWD_TRANSIENT while a whole train step is being issued
  // key of the graph captured in slot s: mode*1e6+steps (train) or steps (predict); -1 none
  long graphKey[4] = {-1, -1, -1, -1};
};

// Thin named wrappers keeping the reference's constructors and AddLayer signatures.
class DirectKPPCNetwork : public PCNetwork
{
public:
  explicit DirectKPPCNetwork(int batchSize, DeviceType = DeviceType::DEVICE_GPU, int device = 0)
      : PCNetwork(NetworkKind::DIRECT_KP, batchSize, device)
  {
  }
  void AddLayer(size_t size, size_t nextSize, size_t terminalSize, float lr, float ir, float fl,
                float lmbda, ActivationType aType, ActivationType /*dType*/)
  {
    AddLayerImpl(size, nextSize, terminalSize, lr, ir, fl, lmbda, aType);
  }
};

class FullPCNetwork : public PCNetwork
{
public:
  explicit FullPCNetwork(int batchSize, DeviceType = DeviceType::DEVICE_GPU, int device = 0)
      : PCNetwork(NetworkKind::FULL, batchSize, device)
  {
  }
  void AddLayer(size_t size, size_t nextSize, size_t terminalSize, float lr, float ir, float fl,
                float lmbda, ActivationType aType, ActivationType /*dType*/)
  {
    AddLayerImpl(size, nextSize, terminalSize, lr, ir, fl, lmbda, aType);
  }
  float TrainStepDevice(const float* xDevice, size_t xN, const float* yDevice, size_t yN,
                        int inferenceSteps)
  {
    return TrainStepRaw(0, xDevice, xN, yDevice, yN, inferenceSteps, true, true);
  }
};

class SimplePCNetwork : public PCNetwork
{
public:
  explicit SimplePCNetwork(int batchSize, DeviceType = DeviceType::DEVICE_GPU, int device = 0)
      : PCNetwork(NetworkKind::SIMPLE, batchSize, device)
  {
  }
  void AddLayer(int size, int nextSize, float lr, float ir, float lmbda, ActivationType aType,
                ActivationType /*dType*/)
  {
    AddLayerImpl(size, nextSize, 0, lr, ir, 0.0f, lmbda, aType);
  }
  float TrainStepWithProjection(const std::vector<float>& x, const std::vector<float>& y,
                                int inferenceSteps, bool computeEnergy = true)
  {
    float e = TrainStepRaw(1, x.data(), x.size(), y.data(), y.size(), inferenceSteps, false,
                           computeEnergy);
    return computeEnergy ? e : 0.0f;
  }
};
} // namespace Deep
