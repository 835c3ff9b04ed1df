// Host orchestration of the convolutional predictive-coding train step over the dpc_conv_* C
// ABI.  Phase order and per-layer semantics follow the reference's CPU path:
//   src/networks/SimpleConvPCNetwork.cpp (TrainStep, TrainStepWithProjection, Predict*)
//   src/layers/SimpleConvPCLayer.cpp     (CalculateState, ComputeMuOnly, UpdateState, UpdateWeights)
#include "conv_network.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <functional>

namespace Deep
{
namespace
{
size_t Pad64c(size_t n)
{
  return (n + 63) & ~(size_t)63;
}
} // namespace

void SimpleConvPCNetwork::Check(int rc) const
{
  if (rc != DPC_OK)
    throw std::runtime_error(std::string("deepity_b200: ") + dpc_last_error());
}

void SimpleConvPCNetwork::RequireCompiled() const
{
  if (!plan)
    throw std::logic_error("deepity_b200: network used before Compile()");
}

SimpleConvPCNetwork::SimpleConvPCNetwork(int batchSize, DeviceType device, int deviceIndex)
    : batchSize(batchSize)
{
  if (batchSize <= 0)
    throw std::invalid_argument("deepity_b200: batch size must be positive");
  if (device != DeviceType::DEVICE_GPU)
    throw std::invalid_argument("deepity_b200: this build has no CPU backend");
  Check(dpc_create(deviceIndex, &ctx));
}

SimpleConvPCNetwork::~SimpleConvPCNetwork()
{
  if (ctx)
    dpc_sync(ctx);
  if (plan)
    dpc_conv_plan_destroy(plan);
  for (void* p : allocations)
    dpc_free(ctx, p);
  for (float* p : {pinnedX, pinnedY, pinnedOut})
    if (p)
      dpc_free_host(ctx, p);
  if (ctx)
    dpc_destroy(ctx);
}

void SimpleConvPCNetwork::AddLayer(int inChannels, int outChannels, int inHeight, int inWidth,
                                   int kernelH, int kernelW, int strideH, int strideW, int padH,
                                   int padW, float lr, float ir, float lmbda, ActivationType aType,
                                   ActivationType dType)
{
  if (plan)
    throw std::logic_error("deepity_b200: AddLayer() after Compile()");
  if (inChannels <= 0 || inHeight <= 0 || inWidth <= 0 || outChannels < 0)
    throw std::invalid_argument("deepity_b200: bad conv layer shape");
  if ((int)dType != (int)aType + 1)
    throw std::invalid_argument("deepity_b200: derivative type does not match the activation");
  auto l = std::make_unique<SimpleConvPCLayer>();
  dpc_conv_layer& d = l->d;
  d.in_c = inChannels, d.out_c = outChannels, d.in_h = inHeight, d.in_w = inWidth;
  d.k_h = kernelH, d.k_w = kernelW, d.s_h = strideH, d.s_w = strideW, d.p_h = padH, d.p_w = padW;
  if (outChannels > 0)
  {
    if (kernelH <= 0 || kernelW <= 0 || strideH <= 0 || strideW <= 0 || padH < 0 || padW < 0)
      throw std::invalid_argument("deepity_b200: bad conv kernel geometry");
    // ConvOutDim, include/deepity/utils/Im2Col.h:47-50
    d.out_h = (inHeight + 2 * padH - kernelH) / strideH + 1;
    d.out_w = (inWidth + 2 * padW - kernelW) / strideW + 1;
    if (d.out_h <= 0 || d.out_w <= 0)
      throw std::invalid_argument("deepity_b200: conv kernel larger than its padded input");
  }
  d.act = (int)aType;
  d.opt = (int)opt;
  d.lr = lr, d.ir = ir, d.lmbda = lmbda;
  l->batch = batchSize;
  layers.push_back(std::move(l));
}

void SimpleConvPCNetwork::SetOptimizer(OptimizerType o)
{
  if (plan && o != opt && o != OptimizerType::SGD && layers.front()->d.m_W == nullptr)
    throw std::logic_error("deepity_b200: select an Adam-type optimizer before Compile()");
  opt = o;
  for (auto& l : layers)
    l->d.opt = (int)o;
  dirty = true;
}

void SimpleConvPCNetwork::Compile()
{
  if (plan)
    throw std::logic_error("deepity_b200: Compile() called twice");
  if (layers.size() < 2)
    throw std::logic_error("deepity_b200: a network needs at least two layers");
  const size_t B = (size_t)batchSize;
  size_t total = 0, ints = 0;
  const bool adam = opt != OptimizerType::SGD;
  for (auto& l : layers)
  {
    const dpc_conv_layer& d = l->d;
    const size_t in = B * d.in_c * d.in_h * d.in_w;
    total += 2 * Pad64c(in);
    if (d.out_c > 0)
    {
      const size_t out = B * d.out_c * d.out_h * d.out_w;
      const size_t nw = (size_t)d.out_c * d.in_c * d.k_h * d.k_w;
      total += 3 * Pad64c(out) + (adam ? 4 : 2) * Pad64c(nw) + (adam ? 4 : 2) * Pad64c(d.out_c);
      ints += 64;
    }
  }
  total += ints;
  void* base = nullptr;
  Check(dpc_alloc(ctx, total * sizeof(float), &base));
  allocations.push_back(base);
  Check(dpc_zero(ctx, base, total * sizeof(float)));
  float* cur = static_cast<float*>(base);
  auto take = [&](size_t n)
  {
    float* p = cur;
    cur += Pad64c(n);
    return p;
  };
  for (auto& l : layers)
  {
    dpc_conv_layer& d = l->d;
    const size_t in = B * d.in_c * d.in_h * d.in_w;
    d.z = take(in);
    d.e = take(in);
    d.opt = (int)opt;
    if (d.out_c > 0)
    {
      const size_t out = B * d.out_c * d.out_h * d.out_w;
      const size_t nw = (size_t)d.out_c * d.in_c * d.k_h * d.k_w;
      d.preact = take(out), d.mu = take(out), d.g = take(out);
      d.W = take(nw), d.g_W = take(nw);
      d.b = take(d.out_c), d.g_b = take(d.out_c);
      if (adam)
      {
        d.m_W = take(nw), d.v_W = take(nw);
        d.m_b = take(d.out_c), d.v_b = take(d.out_c);
      }
      d.t = reinterpret_cast<int32_t*>(take(64));
    }
  }
  void* p = nullptr;
  const size_t inN = B * layers.front()->GetInputSize(), outN = B * layers.back()->GetInputSize();
  Check(dpc_alloc_host(ctx, inN * sizeof(float), &p));
  pinnedX = static_cast<float*>(p);
  Check(dpc_alloc_host(ctx, outN * sizeof(float), &p));
  pinnedY = static_cast<float*>(p);
  Check(dpc_alloc_host(ctx, outN * sizeof(float), &p));
  pinnedOut = static_cast<float*>(p);
  std::vector<dpc_conv_layer> table;
  for (auto& l : layers)
    table.push_back(l->d);
  Check(dpc_conv_plan_create(ctx, table.data(), (int)table.size(), batchSize, &plan));
  Check(dpc_sync(ctx));
  dirty = false;
}

void SimpleConvPCNetwork::DropGraphs()
{
  if (!ctx)
    return;
  for (int s = 0; s < 4; ++s)
  {
    dpc_graph_drop(ctx, s);
    graphKey[s] = -1;
  }
}

void SimpleConvPCNetwork::SyncPlan()
{
  if (!dirty || !plan)
    return;
  std::vector<dpc_conv_layer> table;
  for (auto& l : layers)
    table.push_back(l->d);
  Check(dpc_conv_plan_update(plan, table.data(), (int)table.size()));
  DropGraphs();
  dirty = false;
}

dpc_conv_plan* SimpleConvPCNetwork::Plan()
{
  SyncPlan();
  return plan;
}

void SimpleConvPCNetwork::SetLearningRate(float lr)
{
  for (auto& l : layers)
    l->d.lr = lr;
  dirty = true;
}
void SimpleConvPCNetwork::SetInferenceRate(float ir)
{
  for (auto& l : layers)
    l->d.ir = ir;
  dirty = true;
}
void SimpleConvPCNetwork::SetLambda(float lmbda)
{
  for (auto& l : layers)
    l->d.lmbda = lmbda;
  dirty = true;
}

void SimpleConvPCNetwork::RandomizeWeights(std::mt19937& rng, const char* distribution)
{
  RequireCompiled();
  // W ~ N(0, sqrt(2 / (inC*kH*kW))) (src/layers/SimpleConvPCLayer.cpp:172-186); a
  // "normal(a,b)" / "uniform(a,b)" string overrides it
  // (include/deepity/utils/RandomizeDistribution.h:27-47).  One host mt19937 stream.
  char name[16] = {0};
  float pa = 0.0f, pb = 1.0f;
  const bool parsed =
      distribution && std::sscanf(distribution, " %15[a-zA-Z] ( %f , %f )", name, &pa, &pb) == 3;
  std::uniform_int_distribution<uint32_t> seedDist;
  for (auto& l : layers)
  {
    if (l->d.out_c <= 0)
      continue;
    const size_t rows = (size_t)l->d.in_c * l->d.k_h * l->d.k_w;
    std::vector<float> w((size_t)l->d.out_c * rows);
    std::mt19937 wr(seedDist(rng));
    if (parsed && std::strcmp(name, "uniform") == 0)
    {
      std::uniform_real_distribution<float> d(pa, pb);
      for (auto& v : w)
        v = d(wr);
    }
    else
    {
      std::normal_distribution<float> d(parsed ? pa : 0.0f,
                                        parsed ? pb : std::sqrt(2.0f / (float)rows));
      for (auto& v : w)
        v = d(wr);
    }
    Check(dpc_copy_h2d_sync(ctx, l->d.W, w.data(), w.size() * sizeof(float)));
  }
}

void SimpleConvPCNetwork::ResetState()
{
  RequireCompiled();
  for (auto& l : layers) // only the beliefs: SimpleConvPCLayer::ResetState
    Check(dpc_zero(ctx, l->d.z, (size_t)batchSize * l->GetInputSize() * sizeof(float)));
}

void SimpleConvPCNetwork::ClampRaw(int layer, const float* data, size_t n, bool onDevice)
{
  RequireCompiled();
  SimpleConvPCLayer* l = layers.at(layer).get();
  const size_t count = std::min(n, (size_t)batchSize * l->GetInputSize());
  if (onDevice)
    Check(dpc_copy_d2d(ctx, l->d.z, data, count * sizeof(float)));
  else
  {
    float* stage = layer == 0 ? pinnedX : pinnedY;
    std::memcpy(stage, data, count * sizeof(float));
    Check(dpc_copy_h2d(ctx, l->d.z, stage, count * sizeof(float)));
  }
  l->clamped = true;
  l->cacheValid = false;
}

void SimpleConvPCNetwork::Clamp(const std::vector<float>& input)
{
  ClampRaw(0, input.data(), input.size(), false);
}

// ComputeMuOnly of layer i with whatever the caller wants fused in; a clamped layer computes
// its prediction once and reuses it (SimpleConvPCLayer.cpp:224-229, 287-292).
void SimpleConvPCNetwork::ForwardLayer(int i, int flags)
{
  SimpleConvPCLayer* l = layers[i].get();
  if (l->d.out_c <= 0)
    return;
  if (l->clamped && l->cacheValid)
    Check(dpc_conv_forward(plan, i, flags | DPC_CONV_CACHED));
  else
  {
    Check(dpc_conv_forward(plan, i, flags));
    if (l->clamped)
      l->cacheValid = true;
  }
}

float SimpleConvPCNetwork::CalculateState(bool needEnergy)
{
  RequireCompiled();
  SyncPlan();
  const int n = (int)layers.size();
  // The bottom layer has no prediction from below: its error is zero.
  Check(dpc_zero(ctx, layers[0]->d.e, (size_t)batchSize * layers[0]->GetInputSize() * sizeof(float)));
  for (int i = 0; i + 1 < n; ++i)
  {
    ForwardLayer(i, DPC_CONV_ERR_NEXT | (needEnergy ? DPC_CONV_ENERGY : 0));
    layers[i]->gateIsPrediction = true;
  }
  return 0.0f; // the energy stays in the plan's device accumulator
}

void SimpleConvPCNetwork::UpdateState()
{
  RequireCompiled();
  SyncPlan();
  const int n = (int)layers.size();
  for (int i = 0; i < n; ++i)
  {
    SimpleConvPCLayer* l = layers[i].get();
    if (l->d.out_c > 0)
      l->gateIsPrediction = false; // the reference overwrites mu with f'(preact) here
    if (l->clamped)
      continue;
    Check(dpc_conv_update_state(plan, i));
  }
}

void SimpleConvPCNetwork::UpdateWeights()
{
  RequireCompiled();
  SyncPlan();
  const int n = (int)layers.size();
  for (int i = 0; i + 1 < n; ++i)
  {
    if (layers[i]->gateIsPrediction)
      Check(dpc_conv_gate_with_prediction(plan, i));
    Check(dpc_conv_update_weights(plan, i, centerWeights ? 1 : 0));
  }
}

void SimpleConvPCNetwork::ProjectForward()
{
  RequireCompiled();
  SyncPlan();
  const int n = (int)layers.size();
  for (int i = 0; i + 1 < n; ++i)
    ForwardLayer(i, layers[i + 1]->clamped ? 0 : DPC_CONV_COPY_NEXT);
}

void SimpleConvPCNetwork::Settle(int steps)
{
  for (int t = 0; t < steps; ++t)
  {
    CalculateState(false);
    UpdateState();
  }
}

float SimpleConvPCNetwork::TrainStepRaw(const float* x, size_t nx, const float* y, size_t ny,
                                        int steps, bool withProjection, bool onDevice)
{
  RequireCompiled();
  if (steps < 0)
    throw std::invalid_argument("deepity_b200: bad inference step count");
  SyncPlan();
  const int n = (int)layers.size();
  ResetState();
  ClampRaw(0, x, nx, onDevice);
  ClampRaw(n - 1, y, ny, onDevice);
  for (int i = 1; i + 1 < n; ++i)
    layers[i]->clamped = false;
  // What the weight update will find in the reference's shared mu buffer depends on the
  // previous call when no settling step runs: keep that bit in the graph key.
  const bool gate0 = layers[0]->gateIsPrediction;
  auto phases = [&]
  {
    if (withProjection)
      ProjectForward();
    Settle(steps);
    UpdateWeights();
    Check(dpc_conv_energy_reset(plan));
    CalculateState(true);
  };
  if (useGraph)
  {
    const long key = ((long)steps * 2 + (withProjection ? 1 : 0)) * 2 + (gate0 ? 1 : 0);
    if (graphKey[0] != key)
    {
      Check(dpc_graph_begin(ctx, 0));
      try
      {
        phases();
      }
      catch (...)
      {
        dpc_graph_end(ctx, 0);
        dpc_graph_drop(ctx, 0);
        graphKey[0] = -1;
        throw;
      }
      Check(dpc_graph_end(ctx, 0));
      graphKey[0] = key;
    }
    Check(dpc_graph_launch(ctx, 0));
    for (auto& l : layers)
    {
      if (l->clamped && l->d.out_c > 0)
        l->cacheValid = true;
      l->gateIsPrediction = true;
    }
  }
  else
    phases();
  double energy = 0.0;
  Check(dpc_conv_energy_read(plan, &energy));
  layers.back()->clamped = false;
  return (float)energy;
}

float SimpleConvPCNetwork::TrainStep(const std::vector<float>& x, const std::vector<float>& y,
                                     int inferenceSteps)
{
  return TrainStepRaw(x.data(), x.size(), y.data(), y.size(), inferenceSteps, false, false);
}

float SimpleConvPCNetwork::TrainStepWithProjection(const std::vector<float>& x,
                                                   const std::vector<float>& y, int inferenceSteps)
{
  return TrainStepRaw(x.data(), x.size(), y.data(), y.size(), inferenceSteps, true, false);
}

void SimpleConvPCNetwork::PredictRaw(const float* x, size_t nx, int steps, bool withProjection,
                                     float* out, size_t nout)
{
  RequireCompiled();
  SyncPlan();
  const int n = (int)layers.size();
  const size_t count = (size_t)batchSize * layers.back()->GetInputSize();
  if (nout != count)
    throw std::invalid_argument("deepity_b200: Predict() output buffer has the wrong size");
  ResetState();
  ClampRaw(0, x, nx, false);
  for (int i = 1; i < n; ++i)
    layers[i]->clamped = false;
  auto phases = [&]
  {
    if (withProjection)
      ProjectForward();
    Settle(steps);
  };
  if (useGraph)
  {
    const long key = (long)steps * 2 + (withProjection ? 1 : 0);
    if (graphKey[1] != key)
    {
      Check(dpc_graph_begin(ctx, 1));
      try
      {
        phases();
      }
      catch (...)
      {
        dpc_graph_end(ctx, 1);
        dpc_graph_drop(ctx, 1);
        graphKey[1] = -1;
        throw;
      }
      Check(dpc_graph_end(ctx, 1));
      graphKey[1] = key;
    }
    Check(dpc_graph_launch(ctx, 1));
    for (auto& l : layers)
    {
      if (l->clamped && l->d.out_c > 0)
        l->cacheValid = true;
      if (l->d.out_c > 0)
        l->gateIsPrediction = steps == 0;
    }
  }
  else
    phases();
  Check(dpc_copy_d2h_sync(ctx, pinnedOut, layers.back()->d.z, count * sizeof(float)));
  std::memcpy(out, pinnedOut, count * sizeof(float));
}

std::vector<float> SimpleConvPCNetwork::Predict(const std::vector<float>& x, int inferenceSteps)
{
  std::vector<float> r((size_t)batchSize * layers.back()->GetInputSize());
  PredictRaw(x.data(), x.size(), inferenceSteps, false, r.data(), r.size());
  return r;
}

std::vector<float> SimpleConvPCNetwork::PredictWithProjection(const std::vector<float>& x,
                                                              int inferenceSteps)
{
  std::vector<float> r((size_t)batchSize * layers.back()->GetInputSize());
  PredictRaw(x.data(), x.size(), inferenceSteps, true, r.data(), r.size());
  return r;
}

int64_t SimpleConvPCNetwork::LaunchCount() const
{
  return dpc_launch_count(ctx);
}

bool SimpleConvPCNetwork::FindTensor(int layer, const std::string& name, float** ptr, size_t* count)
{
  if (layer < 0 || layer >= (int)layers.size() || !plan)
    return false;
  const dpc_conv_layer& d = layers[layer]->d;
  const size_t B = (size_t)batchSize;
  const size_t in = B * d.in_c * d.in_h * d.in_w;
  const size_t out = B * d.out_c * d.out_h * d.out_w;
  const size_t nw = (size_t)d.out_c * d.in_c * d.k_h * d.k_w;
  float* p = nullptr;
  size_t c = 0;
  if (name == "z")
    p = d.z, c = in;
  else if (name == "e")
    p = d.e, c = in;
  else if (d.out_c > 0)
  {
    if (name == "mu")
      p = d.mu, c = out;
    else if (name == "preact")
      p = d.preact, c = out;
    else if (name == "W")
      p = d.W, c = nw;
    else if (name == "b")
      p = d.b, c = d.out_c;
    else if (name == "weight.m")
      p = d.m_W, c = nw;
    else if (name == "weight.v")
      p = d.v_W, c = nw;
    else if (name == "bias.m")
      p = d.m_b, c = d.out_c;
    else if (name == "bias.v")
      p = d.v_b, c = d.out_c;
  }
  if (!p)
    return false;
  *ptr = p, *count = c;
  return true;
}
} // namespace Deep

// =======================================================================================
// C ABI: dpcn_conv_*
// =======================================================================================
struct dpcn_conv_net
{
  std::unique_ptr<Deep::SimpleConvPCNetwork> net;
  int batch = 0, device = 0;
};

namespace dpc
{
void set_error(const std::string& msg);
}

namespace
{
int GuardC(const std::function<void()>& fn)
{
  try
  {
    fn();
    return DPC_OK;
  }
  catch (const std::invalid_argument& e)
  {
    dpc::set_error(e.what());
    return DPC_ERR_INVALID;
  }
  catch (const std::logic_error& e)
  {
    dpc::set_error(e.what());
    return DPC_ERR_STATE;
  }
  catch (const std::exception& e)
  {
    const std::string msg = e.what();
    dpc::set_error(msg);
    return msg.find("no CUDA device") != std::string::npos ? DPC_ERR_NO_DEVICE : DPC_ERR_CUDA;
  }
}
} // namespace

int dpcn_conv_create(int batch, int device, dpcn_conv_net** out)
{
  if (!out)
  {
    dpc::set_error("dpcn_conv_create: bad argument");
    return DPC_ERR_INVALID;
  }
  return GuardC(
      [&]
      {
        auto n = std::make_unique<dpcn_conv_net>();
        n->batch = batch, n->device = device;
        n->net = std::make_unique<Deep::SimpleConvPCNetwork>(batch, Deep::DeviceType::DEVICE_GPU,
                                                            device);
        *out = n.release();
      });
}

int dpcn_conv_destroy(dpcn_conv_net* net)
{
  delete net;
  return DPC_OK;
}

int dpcn_conv_add_layer(dpcn_conv_net* net, int in_c, int out_c, int in_h, int in_w, int k_h,
                        int k_w, int s_h, int s_w, int p_h, int p_w, float lr, float ir,
                        float lmbda, int act)
{
  if (!net)
    return DPC_ERR_INVALID;
  return GuardC(
      [&]
      {
        net->net->AddLayer(in_c, out_c, in_h, in_w, k_h, k_w, s_h, s_w, p_h, p_w, lr, ir, lmbda,
                           (Deep::ActivationType)act, (Deep::ActivationType)(act + 1));
      });
}

int dpcn_conv_set_option(dpcn_conv_net* net, const char* name, int iv, float fv)
{
  if (!net || !name)
    return DPC_ERR_INVALID;
  const std::string nm(name);
  return GuardC(
      [&]
      {
        Deep::SimpleConvPCNetwork& n = *net->net;
        if (nm == "optimizer")
          n.SetOptimizer((Deep::OptimizerType)iv);
        else if (nm == "center_weights")
          n.SetCenterWeights(iv != 0);
        else if (nm == "learning_rate")
          n.SetLearningRate(fv);
        else if (nm == "inference_rate")
          n.SetInferenceRate(fv);
        else if (nm == "lambda")
          n.SetLambda(fv);
        else if (nm == "use_graph")
          n.SetUseGraph(iv != 0);
        else
          throw std::invalid_argument("deepity_b200: unknown option '" + nm + "'");
      });
}

int dpcn_conv_compile(dpcn_conv_net* net)
{
  if (!net)
    return DPC_ERR_INVALID;
  return GuardC([&] { net->net->Compile(); });
}

int dpcn_conv_num_layers(dpcn_conv_net* net)
{
  return net ? (int)net->net->GetLayers().size() : DPC_ERR_INVALID;
}

int dpcn_conv_layer_shape(dpcn_conv_net* net, int layer, int* out4)
{
  if (!net || !out4 || layer < 0 || layer >= (int)net->net->GetLayers().size())
    return DPC_ERR_INVALID;
  const dpc_conv_layer& d = net->net->GetLayers()[layer]->d;
  out4[0] = d.out_c, out4[1] = d.out_h, out4[2] = d.out_w, out4[3] = d.in_c * d.k_h * d.k_w;
  return DPC_OK;
}

int64_t dpcn_conv_tensor_size(dpcn_conv_net* net, int layer, const char* name)
{
  float* p;
  size_t c = 0;
  if (!net || !name || !net->net->FindTensor(layer, name, &p, &c))
    return -1;
  return (int64_t)c;
}

int dpcn_conv_get_tensor(dpcn_conv_net* net, int layer, const char* name, float* host_out,
                         int64_t count)
{
  if (!net || !name || !host_out)
    return DPC_ERR_INVALID;
  return GuardC(
      [&]
      {
        float* p;
        size_t c = 0;
        if (!net->net->FindTensor(layer, name, &p, &c) || (int64_t)c != count)
          throw std::invalid_argument(std::string("deepity_b200: no tensor '") + name +
                                      "' of that size on this layer");
        if (dpc_copy_d2h_sync(net->net->Context(), host_out, p, c * sizeof(float)) != DPC_OK)
          throw std::runtime_error(dpc_last_error());
      });
}

int dpcn_conv_set_tensor(dpcn_conv_net* net, int layer, const char* name, const float* host_in,
                         int64_t count)
{
  if (!net || !name || !host_in)
    return DPC_ERR_INVALID;
  return GuardC(
      [&]
      {
        float* p;
        size_t c = 0;
        if (!net->net->FindTensor(layer, name, &p, &c) || (int64_t)c != count)
          throw std::invalid_argument(std::string("deepity_b200: no tensor '") + name +
                                      "' of that size on this layer");
        if (dpc_copy_h2d_sync(net->net->Context(), p, host_in, c * sizeof(float)) != DPC_OK)
          throw std::runtime_error(dpc_last_error());
        for (auto& l : net->net->GetLayers())
          l->InvalidateMuCache();
      });
}

int dpcn_conv_randomize(dpcn_conv_net* net, uint32_t seed)
{
  if (!net)
    return DPC_ERR_INVALID;
  return GuardC(
      [&]
      {
        std::mt19937 rng(seed);
        net->net->RandomizeWeights(rng);
      });
}

int dpcn_conv_train_step(dpcn_conv_net* net, const float* x, int64_t nx, const float* y,
                         int64_t ny, int steps, int with_projection, int on_device,
                         float* energy_out)
{
  if (!net || !x || !y || nx < 0 || ny < 0)
    return DPC_ERR_INVALID;
  return GuardC(
      [&]
      {
        const float e = net->net->TrainStepRaw(x, (size_t)nx, y, (size_t)ny, steps,
                                               with_projection != 0, on_device != 0);
        if (energy_out)
          *energy_out = e;
      });
}

int dpcn_conv_predict(dpcn_conv_net* net, const float* x, int64_t nx, int steps,
                      int with_projection, float* host_out, int64_t nout)
{
  if (!net || !x || !host_out)
    return DPC_ERR_INVALID;
  return GuardC([&]
                { net->net->PredictRaw(x, (size_t)nx, steps, with_projection != 0, host_out, (size_t)nout); });
}

dpc_ctx* dpcn_conv_context(dpcn_conv_net* net)
{
  return net ? net->net->Context() : nullptr;
}

dpc_conv_plan* dpcn_conv_plan(dpcn_conv_net* net)
{
  if (!net || !net->net->IsCompiled())
    return nullptr;
  return net->net->Plan();
}

int64_t dpcn_conv_launch_count(dpcn_conv_net* net)
{
  return net ? net->net->LaunchCount() : 0;
}
