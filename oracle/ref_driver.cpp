// Oracle driver (test infrastructure; never linked into the product).
//
// A flat C interface over the reference's own CPU networks
// (include/deepity/networks/{SimplePCNetwork,DirectKPPCNetwork,FullPCNetwork}.h)
// so that Python tests and the benchmark's CPU leg can build a network from a
// spec, push explicit W/b/Psi, run TrainStep/Predict or single phases, and read
// every state tensor back.  It is compiled together with the reference sources
// where they lie; nothing of the reference is copied.
//
// Tensor names: "z" "e" "mu" (states), "W" "b" "Psi" (parameters), and the
// optimizer-state names of Layer::GetOptimizerStateDict ("weight.m" ...).
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include <omp.h>

#include <deepity/backend/Backend.h>
#include <deepity/networks/DirectKPPCNetwork.h>
#include <deepity/networks/FullPCNetwork.h>
#include <deepity/networks/SimplePCNetwork.h>

#include "cblas.h"

using namespace Deep;

namespace
{
enum Kind
{
  KIND_SIMPLE = 0,
  KIND_DKP = 1,
  KIND_FULL = 2
};

struct Net
{
  int kind;
  int batch;
  int device = 0; // 0: the reference's CPU backend, 1: whatever plugin its loader finds (GPU)
  std::unique_ptr<SimplePCNetwork> simple;
  std::unique_ptr<DirectKPPCNetwork> dkp;
  std::unique_ptr<FullPCNetwork> full;
};

ActivationType Forward(int act)
{
  return static_cast<ActivationType>(act);
}
// Each derivative enumerator directly follows its forward one
// (include/deepity/utils/ActivationType.h:15-32).
ActivationType Derivative(int act)
{
  return static_cast<ActivationType>(act + 1);
}

struct View
{
  float* p = nullptr;
  size_t rows = 0, cols = 0, stride = 0;
};

template <typename LayerT> View StateView(LayerT* l, const std::string& name)
{
  View v;
  const size_t B = l->GetBatchSize(), s = l->GetInputSize(), n = l->GetOutputSize();
  if (name == "z")
    v = {l->GetBeliefs(), B, s, s};
  else if (name == "e")
    v = {const_cast<float*>(l->GetErrors()), B, s, s};
  else if (name == "mu" && n > 0)
    v = {const_cast<float*>(l->GetMu()), B, n, n};
  else if (name == "W" && n > 0)
    v = {l->GetWeights(), n, s, s};
  else if (name == "b" && n > 0)
    v = {l->GetBiases(), 1, n, n};
  return v;
}

template <typename LayerT> View ParamView(LayerT* l, const std::string& name)
{
  View v = StateView(l, name);
  if (v.p)
    return v;
  auto lookup = [&](const std::map<std::string, TensorDescriptor>& d) -> bool
  {
    auto it = d.find(name);
    if (it == d.end() || it->second.data == nullptr)
      return false;
    const auto& t = it->second;
    size_t cols = t.shape.empty() ? 0 : t.shape.back();
    size_t rows = 1;
    for (size_t i = 0; i + 1 < t.shape.size(); ++i)
      rows *= t.shape[i];
    v = {t.data, rows, cols, t.rowStride ? t.rowStride : cols};
    return true;
  };
  if (lookup(l->GetStateDict()))
    return v;
  lookup(l->GetOptimizerStateDict());
  return v;
}

View FindTensor(Net* n, int layer, const char* name)
{
  std::string nm(name);
  switch (n->kind)
  {
  case KIND_SIMPLE:
    if (layer < 0 || layer >= (int)n->simple->GetLayers().size())
      return {};
    return ParamView(n->simple->GetLayers()[layer].get(), nm);
  case KIND_DKP:
    if (layer < 0 || layer >= (int)n->dkp->GetLayers().size())
      return {};
    return ParamView(n->dkp->GetLayers()[layer].get(), nm);
  default:
    if (layer < 0 || layer >= (int)n->full->GetLayers().size())
      return {};
    return ParamView(n->full->GetLayers()[layer].get(), nm);
  }
}
IComputeBackend* BackendOf(Net* n)
{
  if (n->kind == KIND_SIMPLE)
    return n->simple->GetLayers().front()->GetBackend();
  if (n->kind == KIND_DKP)
    return n->dkp->GetLayers().front()->GetBackend();
  return n->full->GetLayers().front()->GetBackend();
}
} // namespace

extern "C"
{
void* ref_create(int kind, int batch)
{
  auto* n = new Net{kind, batch, 0, nullptr, nullptr, nullptr};
  if (kind == KIND_SIMPLE)
    n->simple = std::make_unique<SimplePCNetwork>(batch);
  else if (kind == KIND_DKP)
    n->dkp = std::make_unique<DirectKPPCNetwork>(batch);
  else
    n->full = std::make_unique<FullPCNetwork>(batch);
  return n;
}

// The same networks on DEVICE_GPU: the reference's loader (src/backend/CUDAPluginLoader.cpp:52-107)
// then dlopens libDeepityCUDA.so from the directory of this library.  NULL when that fails
// (no plugin there, no device).
void* ref_create_on_gpu(int kind, int batch)
{
  try
  {
    auto* n = new Net{kind, batch, 1, nullptr, nullptr, nullptr};
    if (kind == KIND_SIMPLE)
      n->simple = std::make_unique<SimplePCNetwork>(batch, DeviceType::DEVICE_GPU);
    else if (kind == KIND_DKP)
      n->dkp = std::make_unique<DirectKPPCNetwork>(batch, DeviceType::DEVICE_GPU);
    else
      n->full = std::make_unique<FullPCNetwork>(batch, DeviceType::DEVICE_GPU);
    return n;
  }
  catch (const std::exception& e)
  {
    fprintf(stderr, "ref_create_on_gpu: %s\n", e.what());
    return nullptr;
  }
}

void ref_destroy(void* h)
{
  delete static_cast<Net*>(h);
}

int ref_add_layer(void* h, int size, int next, int terminal, float lr, float ir, float fl,
                  float lmbda, int act)
{
  auto* n = static_cast<Net*>(h);
  if (n->kind == KIND_SIMPLE)
    n->simple->AddLayer(size, next, lr, ir, lmbda, Forward(act), Derivative(act));
  else if (n->kind == KIND_DKP)
    n->dkp->AddLayer(size, next, terminal, lr, ir, fl, lmbda, Forward(act), Derivative(act));
  else
    n->full->AddLayer(size, next, terminal, lr, ir, fl, lmbda, Forward(act), Derivative(act));
  return 0;
}

// option names: "optimizer" "psi_optimizer" (0 SGD, 1 ADAM, 2 ADAMW),
// "center_weights", "psi_decay", Simple: "cross_entropy"; Full: "mupc" "residual" "ipc" "epc"
// "momentum" (value = beta) "cross_entropy".
int ref_set_option(void* h, const char* name, int ivalue, float fvalue)
{
  auto* n = static_cast<Net*>(h);
  std::string nm(name);
  auto opt = static_cast<OptimizerType>(ivalue);
  try
  {
    if (n->kind == KIND_SIMPLE)
    {
      if (nm == "optimizer")
        n->simple->SetOptimizer(opt);
      else if (nm == "center_weights")
        n->simple->SetCenterWeights(ivalue != 0);
      else if (nm == "cross_entropy")
        n->simple->GetTerminalLayer()->SetCrossEntropy(ivalue != 0);
      else
        return -1;
    }
    else if (n->kind == KIND_DKP)
    {
      if (nm == "optimizer")
        n->dkp->SetOptimizer(opt);
      else if (nm == "psi_optimizer")
        n->dkp->SetPsiOptimizer(opt);
      else if (nm == "center_weights")
        n->dkp->SetCenterWeights(ivalue != 0);
      else if (nm == "psi_decay")
        n->dkp->SetPsiDecay(fvalue);
      else
        return -1;
    }
    else
    {
      if (nm == "optimizer")
        n->full->SetOptimizer(opt);
      else if (nm == "psi_optimizer")
        n->full->SetPsiOptimizer(opt);
      else if (nm == "center_weights")
        n->full->SetCenterWeights(ivalue != 0);
      else if (nm == "mupc")
        n->full->SetUseMuPCScaling(ivalue != 0);
      else if (nm == "residual")
        n->full->SetUseResidualConnections(ivalue != 0);
      else if (nm == "ipc")
        n->full->SetUseIPC(ivalue != 0);
      else if (nm == "epc")
        n->full->SetUseEPC(ivalue != 0);
      else if (nm == "momentum")
        n->full->SetUseMomentum(ivalue != 0, fvalue);
      else if (nm == "cross_entropy")
        n->full->SetUseCrossEntropy(ivalue != 0);
      else
        return -1;
    }
  }
  catch (...)
  {
    return -2;
  }
  return 0;
}

int ref_compile(void* h)
{
  auto* n = static_cast<Net*>(h);
  try
  {
    if (n->kind == KIND_SIMPLE)
      n->simple->Compile();
    else if (n->kind == KIND_DKP)
      n->dkp->Compile();
    else
      n->full->Compile();
  }
  catch (...)
  {
    return -1;
  }
  return 0;
}

int ref_num_layers(void* h)
{
  auto* n = static_cast<Net*>(h);
  if (n->kind == KIND_SIMPLE)
    return (int)n->simple->GetLayers().size();
  if (n->kind == KIND_DKP)
    return (int)n->dkp->GetLayers().size();
  return (int)n->full->GetLayers().size();
}

// Returns rows*cols of the logical tensor, 0 if the layer has no such tensor.
int64_t ref_tensor_size(void* h, int layer, const char* name)
{
  View v = FindTensor(static_cast<Net*>(h), layer, name);
  return v.p ? (int64_t)(v.rows * v.cols) : 0;
}

int ref_get_tensor(void* h, int layer, const char* name, float* out, int64_t count)
{
  auto* n = static_cast<Net*>(h);
  View v = FindTensor(n, layer, name);
  if (!v.p || (int64_t)(v.rows * v.cols) != count)
    return -1;
  std::vector<float> staged;
  const float* src = v.p;
  if (n->device)
  {
    // the tensor lives in device memory: stage it through the network's backend
    staged.resize(v.rows * v.stride);
    BackendOf(n)->CopyToHost(staged.data(), v.p, staged.size());
    src = staged.data();
  }
  for (size_t r = 0; r < v.rows; ++r)
    std::memcpy(out + r * v.cols, src + r * v.stride, v.cols * sizeof(float));
  return 0;
}

int ref_set_tensor(void* h, int layer, const char* name, const float* in, int64_t count)
{
  auto* n = static_cast<Net*>(h);
  View v = FindTensor(n, layer, name);
  if (!v.p || (int64_t)(v.rows * v.cols) != count)
    return -1;
  if (n->device)
  {
    std::vector<float> staged(v.rows * v.stride, 0.0f);
    for (size_t r = 0; r < v.rows; ++r)
      std::memcpy(staged.data() + r * v.stride, in + r * v.cols, v.cols * sizeof(float));
    BackendOf(n)->CopyFromHost(v.p, staged.data(), staged.size());
    return 0;
  }
  for (size_t r = 0; r < v.rows; ++r)
    std::memcpy(v.p + r * v.stride, in + r * v.cols, v.cols * sizeof(float));
  return 0;
}

float ref_train_step(void* h, const float* x, int64_t nx, const float* y, int64_t ny, int T)
{
  auto* n = static_cast<Net*>(h);
  std::vector<float> xv(x, x + nx), yv(y, y + ny);
  if (n->kind == KIND_SIMPLE)
    return n->simple->TrainStep(xv, yv, T);
  if (n->kind == KIND_DKP)
    return n->dkp->TrainStep(xv, yv, T);
  return n->full->TrainStep(xv, yv, T);
}

// SimplePCNetwork only: the graph-captured entry point the Python wrapper
// binds as train_step_with_projection (src/networks/SimplePCNetwork.cpp:179-252).
float ref_train_step_with_projection(void* h, const float* x, int64_t nx, const float* y,
                                     int64_t ny, int T, int computeEnergy)
{
  auto* n = static_cast<Net*>(h);
  if (n->kind != KIND_SIMPLE)
    return -1.0f;
  std::vector<float> xv(x, x + nx), yv(y, y + ny);
  return n->simple->TrainStepWithProjection(xv, yv, T, computeEnergy != 0);
}

int ref_predict(void* h, const float* x, int64_t nx, int T, int withProjection, float* out,
                int64_t nout)
{
  auto* n = static_cast<Net*>(h);
  std::vector<float> xv(x, x + nx), r;
  if (n->kind == KIND_SIMPLE)
    r = withProjection ? n->simple->PredictWithProjection(xv, T) : n->simple->Predict(xv, T);
  else if (n->kind == KIND_DKP)
    r = n->dkp->Predict(xv, T);
  else
    r = n->full->Predict(xv, T);
  if ((int64_t)r.size() != nout)
    return -1;
  std::memcpy(out, r.data(), r.size() * sizeof(float));
  return 0;
}

// Single phases, for the Python-level SimplePCN.train_step loop
// (deepity/SimplePCN.py:269-293) and for phase-by-phase parity tests.
// op: "reset" "clamp_x" "clamp_y" "unclamp_y" "project_forward" "terminal_error" "dfa"
//     "calculate_state" "calculate_state_energy" "update_state" "step" "update_weights"
float ref_phase(void* h, const char* op, const float* data, int64_t count)
{
  auto* n = static_cast<Net*>(h);
  std::string o(op);
  std::vector<float> v;
  if (data && count > 0)
    v.assign(data, data + count);
  if (n->kind == KIND_SIMPLE)
  {
    auto& net = *n->simple;
    if (o == "reset")
      net.ResetState();
    else if (o == "clamp_x")
      net.Clamp(v);
    else if (o == "clamp_y")
      net.GetTerminalLayer()->ClampState(v);
    else if (o == "unclamp_y")
      net.GetTerminalLayer()->UnclampState();
    else if (o == "project_forward")
      net.ProjectForward();
    else if (o == "calculate_state")
      return net.CalculateState(false);
    else if (o == "calculate_state_energy")
      return net.CalculateState(true);
    else if (o == "update_state")
      net.UpdateState();
    else if (o == "update_weights")
      net.UpdateWeights();
    else
      return -1.0f;
    return 0.0f;
  }
  if (n->kind == KIND_DKP)
  {
    auto& net = *n->dkp;
    if (o == "reset")
      net.ResetState();
    else if (o == "clamp_x")
      net.Clamp(v);
    else if (o == "clamp_y")
      net.GetTerminalLayer()->ClampState(v);
    else if (o == "unclamp_y")
      net.GetTerminalLayer()->UnclampState();
    else if (o == "project_forward")
      net.ProjectForward();
    else if (o == "terminal_error")
      return net.CalculateTerminalError();
    else if (o == "dfa")
      net.DirectFeedbackUpdate();
    else if (o == "step")
      return net.Step(false);
    else if (o == "update_weights")
      net.UpdateWeights();
    else
      return -1.0f;
    return 0.0f;
  }
  auto& net = *n->full;
  if (o == "reset")
    net.ResetState();
  else if (o == "clamp_x")
    net.Clamp(v);
  else if (o == "clamp_y")
    net.GetTerminalLayer()->ClampState(v);
  else if (o == "unclamp_y")
    net.GetTerminalLayer()->UnclampState();
  else if (o == "project_forward")
    net.ProjectForward();
  else if (o == "terminal_error")
    return net.CalculateTerminalError();
  else if (o == "dfa")
    net.DirectFeedbackUpdate();
  else if (o == "step")
    return net.Step(false);
  else if (o == "update_weights")
    net.UpdateWeights();
  else
    return -1.0f;
  return 0.0f;
}

// One GEMM through the reference's backend interface on host arrays (device 1: the GPU plugin the
// loader finds; 0: the CPU backend): C = alpha*op(A)*op(B) + beta*C with BLAS leading dimensions.
// For primitive-level checks of a plugin's MatMul (tests/tMatMulLargeAsymmetricVerify.cpp's idea).
// a_elems/b_elems/c_elems: sizes of the host arrays.  allow_tf32 < 0 leaves the backend's default.
int ref_backend_matmul(int device, int transA, int transB, int M, int N, int K, float alpha,
                       const float* A, int64_t a_elems, int lda, const float* B, int64_t b_elems,
                       int ldb, float beta, float* C, int64_t c_elems, int ldc, int allow_tf32)
{
  try
  {
    std::unique_ptr<IComputeBackend> be =
        CreateBackend(device ? DeviceType::DEVICE_GPU : DeviceType::DEVICE_CPU);
    if (allow_tf32 >= 0)
      be->SetAllowTF32(allow_tf32 != 0);
    float* dA = be->Allocate((size_t)a_elems);
    float* dB = be->Allocate((size_t)b_elems);
    float* dC = be->Allocate((size_t)c_elems);
    if (!dA || !dB || !dC)
      return -2;
    be->CopyFromHost(dA, A, (size_t)a_elems);
    be->CopyFromHost(dB, B, (size_t)b_elems);
    be->CopyFromHost(dC, C, (size_t)c_elems);
    be->MatMul(transA != 0, transB != 0, M, N, K, alpha, dA, lda, dB, ldb, beta, dC, ldc);
    be->Synchronize();
    be->CopyToHost(C, dC, (size_t)c_elems);
    be->Free(dA);
    be->Free(dB);
    be->Free(dC);
    return 0;
  }
  catch (const std::exception& e)
  {
    fprintf(stderr, "ref_backend_matmul: %s\n", e.what());
    return -1;
  }
}

// Host threading the reference chose for this batch size
// (include/deepity/utils/Optimize.h:108-131) and the BLAS build string.
int ref_omp_threads(void)
{
  return omp_get_max_threads();
}
int ref_num_procs(void)
{
  return omp_get_num_procs();
}
const char* ref_blas_config(void)
{
  return scipy_openblas_get_config();
}
int ref_blas_threads(void)
{
  return scipy_openblas_get_num_threads();
}
// Caps the thread count below what DynamicThread picked (a host whose CPU quota or affinity
// mask is smaller than omp_get_num_procs() reports would otherwise be oversubscribed).
// DynamicThread is memoised on its own target, so the cap holds until the batch size changes.
void ref_set_threads(int n)
{
  if (n < 1)
    n = 1;
  omp_set_num_threads(n);
  scipy_openblas_set_num_threads(n);
}
}
