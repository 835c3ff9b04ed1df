// Oracle driver for the convolutional network (test infrastructure; never linked into the
// product).  A flat C interface over the reference's own CPU SimpleConvPCNetwork
// (include/deepity/networks/SimpleConvPCNetwork.h), compiled together with the reference
// sources where they lie.  Tensor names: "z" "e" "mu" "W" "b".
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <exception>
#include <memory>
#include <string>
#include <vector>

#include <deepity/networks/SimpleConvPCNetwork.h>

using namespace Deep;

namespace
{
struct ConvNet
{
  int batch;
  std::unique_ptr<SimpleConvPCNetwork> net;
  int device; // 1: the tensors live in device memory (the network runs on the backend plugin)
};

IComputeBackend* BackendOf(ConvNet* n)
{
  return n->net->GetLayers().front()->GetBackend();
}

bool Find(ConvNet* n, int layer, const char* name, float** p, size_t* count)
{
  const auto& layers = n->net->GetLayers();
  if (layer < 0 || layer >= (int)layers.size())
    return false;
  SimpleConvPCLayer* l = layers[layer].get();
  const size_t B = l->GetBatchSize(), s = l->GetInputSize(), o = l->GetOutputSize();
  const size_t rowLen = (size_t)l->GetInChannels() * l->GetKernelH() * l->GetKernelW();
  const std::string nm(name);
  *p = nullptr;
  if (nm == "z")
    *p = l->GetBeliefs(), *count = B * s;
  else if (nm == "e")
    *p = const_cast<float*>(l->GetErrors()), *count = B * s;
  else if (nm == "mu" && o > 0)
    *p = const_cast<float*>(l->GetMu()), *count = B * o;
  else if (nm == "W" && o > 0)
    *p = l->GetWeights(), *count = (size_t)l->GetOutChannels() * rowLen;
  else if (nm == "b" && o > 0)
    *p = l->GetBiases(), *count = (size_t)l->GetOutChannels();
  return *p != nullptr;
}
} // namespace

extern "C"
{
void* refc_create(int batch)
{
  auto* n = new ConvNet{batch, std::make_unique<SimpleConvPCNetwork>(batch), 0};
  return n;
}

// The same network on DEVICE_GPU: the reference's loader then dlopens libDeepityCUDA.so from the
// directory of this library.  NULL when that fails (no plugin, no usable device).
void* refc_create_on_gpu(int batch)
{
  try
  {
    return new ConvNet{batch, std::make_unique<SimpleConvPCNetwork>(batch, DeviceType::DEVICE_GPU), 1};
  }
  catch (const std::exception& e)
  {
    fprintf(stderr, "refc_create_on_gpu: %s\n", e.what());
    return nullptr;
  }
}

void refc_destroy(void* h)
{
  delete static_cast<ConvNet*>(h);
}

int refc_add_layer(void* h, int inC, int outC, int inH, int inW, int kH, int kW, int sH, int sW,
                   int pH, int pW, float lr, float ir, float lmbda, int act)
{
  auto* n = static_cast<ConvNet*>(h);
  // Each derivative enumerator directly follows its forward one
  // (include/deepity/utils/ActivationType.h:15-32).
  n->net->AddLayer(inC, outC, inH, inW, kH, kW, sH, sW, pH, pW, lr, ir, lmbda,
                   static_cast<ActivationType>(act), static_cast<ActivationType>(act + 1));
  return 0;
}

int refc_set_option(void* h, const char* name, int ivalue, float)
{
  auto* n = static_cast<ConvNet*>(h);
  const std::string nm(name);
  if (nm == "optimizer")
    n->net->SetOptimizer(static_cast<OptimizerType>(ivalue));
  else if (nm == "center_weights")
    n->net->SetCenterWeights(ivalue != 0);
  else
    return -1;
  return 0;
}

int refc_compile(void* h)
{
  static_cast<ConvNet*>(h)->net->Compile();
  return 0;
}

int64_t refc_tensor_size(void* h, int layer, const char* name)
{
  float* p;
  size_t c = 0;
  return Find(static_cast<ConvNet*>(h), layer, name, &p, &c) ? (int64_t)c : -1;
}

int refc_get_tensor(void* h, int layer, const char* name, float* out, int64_t count)
{
  float* p;
  size_t c = 0;
  auto* n = static_cast<ConvNet*>(h);
  if (!Find(n, layer, name, &p, &c) || (int64_t)c != count)
    return -1;
  if (n->device)
    BackendOf(n)->CopyToHost(out, p, c);
  else
    std::memcpy(out, p, c * sizeof(float));
  return 0;
}

int refc_set_tensor(void* h, int layer, const char* name, const float* in, int64_t count)
{
  float* p;
  size_t c = 0;
  auto* n = static_cast<ConvNet*>(h);
  if (!Find(n, layer, name, &p, &c) || (int64_t)c != count)
    return -1;
  if (n->device)
    BackendOf(n)->CopyFromHost(p, in, c);
  else
    std::memcpy(p, in, c * sizeof(float));
  return 0;
}

float refc_train_step(void* h, const float* x, int64_t nx, const float* y, int64_t ny, int T,
                      int withProjection)
{
  auto* n = static_cast<ConvNet*>(h);
  std::vector<float> xv(x, x + nx), yv(y, y + ny);
  return withProjection ? n->net->TrainStepWithProjection(xv, yv, T) : n->net->TrainStep(xv, yv, T);
}

int refc_predict(void* h, const float* x, int64_t nx, int T, int withProjection, float* out,
                 int64_t nout)
{
  auto* n = static_cast<ConvNet*>(h);
  std::vector<float> xv(x, x + nx);
  std::vector<float> r = withProjection ? n->net->PredictWithProjection(xv, T) : n->net->Predict(xv, T);
  if ((int64_t)r.size() != nout)
    return -1;
  std::memcpy(out, r.data(), r.size() * sizeof(float));
  return 0;
}
}
