// Host orchestration of the predictive-coding train step over the dpc_* C ABI.
// Phase order and per-layer semantics follow the reference's CPU path:
//   DirectKP  src/networks/DirectKPPCNetwork.cpp:349-603
//   Full      src/networks/FullPCNetwork.cpp:51-251, 350-466
//   Simple    src/networks/SimplePCNetwork.cpp:57-252, deepity/SimplePCN.py:269-293
#include "pc_network.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <functional>

namespace Deep
{
namespace
{
size_t Pad64(size_t n)
{
  return (n + 63) & ~(size_t)63;
}
} // namespace

void PCNetwork::Check(int rc) const
{
  if (rc != DPC_OK)
    throw StatusError(rc, std::string("deepity_b200: ") + dpc_last_error());
}

void PCNetwork::RequireCompiled() const
{
  if (!plan)
    throw std::logic_error("deepity_b200: network used before Compile()");
}

PCNetwork::PCNetwork(NetworkKind kind, int batchSize, int device)
    : kind(kind)
    , batchSize(batchSize)
{
  if (batchSize <= 0)
    throw std::invalid_argument("deepity_b200: batch size must be positive");
  Check(dpc_create(device, &ctx));
}

PCNetwork::~PCNetwork()
{
  if (ctx)
    dpc_sync(ctx);
  if (plan)
    dpc_plan_destroy(plan);
  for (void* p : allocations)
    dpc_free(ctx, p);
  if (pinnedX)
    dpc_free_host(ctx, pinnedX);
  if (pinnedY)
    dpc_free_host(ctx, pinnedY);
  if (pinnedOut)
    dpc_free_host(ctx, pinnedOut);
  if (ctx)
    dpc_destroy(ctx);
}

void PCNetwork::AddLayerImpl(size_t size, size_t nextSize, size_t terminalSize, float lr, float ir,
                             float fl, float lmbda, ActivationType aType)
{
  if (plan)
    throw std::logic_error("deepity_b200: AddLayer() after Compile()");
  if (size == 0)
    throw std::invalid_argument("deepity_b200: layer size must be positive");
  if (!layers.empty() && layers.back()->d.next_size != (int)size)
    throw std::invalid_argument("deepity_b200: layer size does not match the previous nextSize");
  auto l = std::make_unique<PCLayer>();
  l->batch = batchSize;
  l->d.size = (int)size;
  l->d.next_size = (int)nextSize;
  l->d.terminal_size = (int)terminalSize;
  l->d.psi_stride = (int)terminalSize;
  l->d.act = (int)aType;
  l->d.flags = 0;
  if (kind == NetworkKind::SIMPLE)
    l->d.flags |= DPC_LAYER_INPUT_ACT;
  if (kind == NetworkKind::FULL)
    l->d.flags |= DPC_LAYER_FULLPC_PSI;
  l->d.a = 1.0f;
  l->d.lr = lr;
  l->d.ir = ir;
  l->d.fl = fl;
  l->d.lmbda = lmbda;
  l->d.psi_decay = psiDecay;
  l->d.momentum_beta = momentumBeta;
  l->d.opt = (int)opt;
  l->d.opt_psi = (int)optPsi;
  layers.push_back(std::move(l));
}

void PCNetwork::Compile()
{
  if (plan)
    throw std::logic_error("deepity_b200: Compile() called twice");
  if (layers.size() < 2)
    throw std::invalid_argument("deepity_b200: a network needs at least one weight layer and "
                                "the terminal layer");
  if (layers.back()->d.next_size != 0)
    throw std::invalid_argument("deepity_b200: the last layer must have nextSize == 0");
  const int n = (int)layers.size();
  // Same check as DirectKPPCNetwork::Compile() (src/networks/DirectKPPCNetwork.cpp:677-684).
  if (kind != NetworkKind::SIMPLE && !ghostTop &&
      layers.back()->d.size != layers.back()->d.terminal_size)
    throw std::invalid_argument(
        "Compile(): terminalSize (" + std::to_string(layers.back()->d.terminal_size) +
        ") passed to AddLayer() doesn't match the actual terminal layer's size (" +
        std::to_string(layers.back()->d.size) + ").");

  // muPC scales and residual wiring, src/networks/FullPCNetwork.cpp:405-465.
  if (kind == NetworkKind::FULL && (useMuPC || useResidual))
  {
    const int L = n - 1, H = L - 1;
    if (useMuPC && L >= 1)
    {
      const float d_in = (float)layers[0]->d.size;
      float N = 0.0f;
      if (H > 0)
        for (int i = 0; i < L - 1; ++i)
          N = std::max(N, (float)layers[i]->d.next_size);
      else
        N = (float)layers[L - 1]->d.next_size;
      for (int l = 1; l <= L; ++l)
      {
        float a;
        if (l == 1)
          a = std::pow(d_in, -0.5f);
        else if (l == L)
          a = 1.0f / N;
        else
          a = std::pow(N * (float)L, -0.5f);
        layers[l - 1]->d.a = a;
      }
    }
    if (useResidual)
      for (int l = 2; l <= H; ++l)
      {
        PCLayer* layer = layers[l - 1].get();
        if (layer->d.size != layer->d.next_size)
          throw std::invalid_argument("Compile(): residual connections require matching width, "
                                      "layer index " + std::to_string(l - 1));
        layer->d.flags |= DPC_LAYER_RESIDUAL;
      }
  }
  if (crossEntropy)
    layers.back()->d.flags |= DPC_LAYER_SOFTMAX_CE;

  // Flat arenas, one per tensor kind, layers in order: consecutive identical layers end up
  // at a constant stride, which is what the grouped kernels want.
  const size_t B = (size_t)batchSize;
  enum
  {
    A_Z, A_E, A_W, A_B, A_PRE, A_MU, A_FE, A_PSI, A_ZF, A_V, A_ADJ, A_COUNT
  };
  size_t total[A_COUNT] = {};
  if (ghostTop)
    total[A_PSI] += Pad64((size_t)layers.back()->d.size * layers.back()->d.terminal_size) +
                    Pad64(B * layers.back()->d.terminal_size);
  for (auto& l : layers)
  {
    const size_t s = l->d.size, nx = l->d.next_size, ts = l->d.terminal_size;
    total[A_Z] += Pad64(B * s);
    total[A_E] += Pad64(B * s);
    if (useMomentum)
      total[A_V] += Pad64(B * s);
    if (useEPC && nx > 0)
      total[A_ADJ] += Pad64(B * s);
    if (nx > 0)
    {
      total[A_W] += Pad64(nx * s);
      total[A_B] += Pad64(nx);
      total[A_MU] += Pad64(B * nx);
      if (kind == NetworkKind::SIMPLE)
        total[A_ZF] += Pad64(B * s);
      else
      {
        total[A_PRE] += Pad64(B * nx);
        total[A_FE] += Pad64(B * nx);
        total[A_PSI] += Pad64(s * ts);
      }
    }
  }
  float* base[A_COUNT] = {};
  for (int k = 0; k < A_COUNT; ++k)
  {
    if (total[k] == 0)
      continue;
    void* p = nullptr;
    Check(dpc_alloc(ctx, total[k] * sizeof(float), &p));
    allocations.push_back(p);
    Check(dpc_zero(ctx, p, total[k] * sizeof(float)));
    base[k] = static_cast<float*>(p);
  }
  size_t off[A_COUNT] = {};
  auto take = [&](int k, size_t count) -> float*
  {
    float* p = base[k] + off[k];
    off[k] += Pad64(count);
    return p;
  };
  for (auto& l : layers)
  {
    const size_t s = l->d.size, nx = l->d.next_size, ts = l->d.terminal_size;
    l->d.z = take(A_Z, B * s);
    l->d.e = take(A_E, B * s);
    if (useMomentum)
      l->d.v = take(A_V, B * s);
    if (useEPC && nx > 0)
      l->d.adj = take(A_ADJ, B * s);
    if (nx > 0)
    {
      l->d.W = take(A_W, nx * s);
      l->d.b = take(A_B, nx);
      l->d.mu = take(A_MU, B * nx);
      if (kind == NetworkKind::SIMPLE)
        l->d.zF = take(A_ZF, B * s);
      else
      {
        l->d.preact = take(A_PRE, B * nx);
        l->d.fe = take(A_FE, B * nx);
        l->d.Psi = take(A_PSI, s * ts);
      }
    }
  }
  if (ghostTop)
  {
    PCLayer* g = layers.back().get();
    g->d.Psi = take(A_PSI, (size_t)g->d.size * g->d.terminal_size);
    ghostET = take(A_PSI, B * g->d.terminal_size);
  }
  size_t inN = B * layers.front()->d.size, outN = B * layers.back()->d.size;
  void* p = nullptr;
  Check(dpc_alloc_host(ctx, inN * sizeof(float), &p));
  pinnedX = static_cast<float*>(p);
  Check(dpc_alloc_host(ctx, outN * sizeof(float), &p));
  pinnedY = static_cast<float*>(p);
  Check(dpc_alloc_host(ctx, outN * sizeof(float), &p));
  pinnedOut = static_cast<float*>(p);

  EnsureOptimizerState();
  EnsureGradientStaging();
  std::vector<dpc_layer> table;
  for (auto& l : layers)
    table.push_back(l->d);
  Check(dpc_plan_create(ctx, table.data(), n, batchSize, &plan));
  if (ghostTop)
    Check(dpc_plan_set_terminal_error(plan, ghostET));
  Check(dpc_sync(ctx));
  dirty = false;
}

void PCNetwork::EnsureOptimizerState()
{
  const bool needAdam = opt != OptimizerType::SGD;
  const bool needPsiAdam = kind != NetworkKind::SIMPLE && optPsi != OptimizerType::SGD;
  auto grab = [&](size_t floats) -> float*
  {
    void* p = nullptr;
    Check(dpc_alloc(ctx, floats * sizeof(float), &p));
    allocations.push_back(p);
    Check(dpc_zero(ctx, p, floats * sizeof(float)));
    return static_cast<float*>(p);
  };
  if (needAdam && !adamAllocated)
  {
    size_t tw = 0, tb = 0, nl = 0;
    for (auto& l : layers)
      if (l->d.next_size > 0)
        tw += Pad64((size_t)l->d.next_size * l->d.size), tb += Pad64(l->d.next_size), ++nl;
    float* mw = grab(tw);
    float* vw = grab(tw);
    float* mb = grab(tb);
    float* vb = grab(tb);
    int32_t* t = reinterpret_cast<int32_t*>(grab(Pad64(nl)));
    size_t ow = 0, ob = 0, ot = 0;
    for (auto& l : layers)
      if (l->d.next_size > 0)
      {
        l->d.m_W = mw + ow, l->d.v_W = vw + ow;
        l->d.m_b = mb + ob, l->d.v_b = vb + ob;
        l->d.t = t + ot++;
        ow += Pad64((size_t)l->d.next_size * l->d.size);
        ob += Pad64(l->d.next_size);
      }
    adamAllocated = true;
  }
  if (needPsiAdam && !psiAdamAllocated)
  {
    size_t tp = 0, nl = 0;
    for (auto& l : layers)
      if (l->d.next_size > 0)
        tp += Pad64((size_t)l->d.size * l->d.psi_stride), ++nl;
    float* mp = grab(tp);
    float* vp = grab(tp);
    int32_t* t = reinterpret_cast<int32_t*>(grab(Pad64(nl)));
    size_t op = 0, ot = 0;
    for (auto& l : layers)
      if (l->d.next_size > 0)
      {
        l->d.m_Psi = mp + op, l->d.v_Psi = vp + op;
        l->d.t_Psi = t + ot++;
        op += Pad64((size_t)l->d.size * l->d.psi_stride);
      }
    psiAdamAllocated = true;
  }
}

void PCNetwork::EnsureGradientStaging()
{
  // Staging is needed for batch sharding, and lets Adam-type weight updates of the tensor-core
  // layers run as "product into the staging buffer + elementwise optimizer".
  if (!(gradSync || opt != OptimizerType::SGD) || gradBuffer)
    return;
  size_t tw = 0, tb = 0, tp = 0;
  for (auto& l : layers)
    if (l->d.next_size > 0)
    {
      tw += Pad64((size_t)l->d.next_size * l->d.size);
      tb += Pad64(l->d.next_size);
      if (l->d.Psi)
        tp += Pad64((size_t)l->d.size * l->d.psi_stride);
    }
  void* p = nullptr;
  gradCount = tw + tb + tp;
  gradWCount = tw;
  Check(dpc_alloc(ctx, gradCount * sizeof(float), &p));
  allocations.push_back(p);
  Check(dpc_zero(ctx, p, gradCount * sizeof(float)));
  gradBuffer = static_cast<float*>(p);
  size_t ow = 0, ob = tw, op = tw + tb;
  for (auto& l : layers)
    if (l->d.next_size > 0)
    {
      l->d.g_W = gradBuffer + ow;
      l->d.g_b = gradBuffer + ob;
      ow += Pad64((size_t)l->d.next_size * l->d.size);
      ob += Pad64(l->d.next_size);
      if (l->d.Psi)
      {
        l->d.g_Psi = gradBuffer + op;
        op += Pad64((size_t)l->d.size * l->d.psi_stride);
      }
    }
}

void PCNetwork::SetGradientSync(GradientSyncFn sync, void* user, int global)
{
  if (sync && (global < batchSize || global % batchSize != 0))
    throw std::invalid_argument("deepity_b200: global batch must be a multiple of the local batch");
  gradSync = sync;
  gradUser = user;
  globalBatch = sync ? global : 0;
  Dirty();
}

void PCNetwork::SyncGradients(size_t count)
{
  if (gradSync(gradUser, gradBuffer, (int64_t)count, dpc_stream(ctx)) != 0)
    throw std::runtime_error("deepity_b200: the gradient sync function reported a failure");
}

void PCNetwork::Dirty()
{
  dirty = true;
}

void PCNetwork::SyncPlan()
{
  if (!dirty || !plan)
    return;
  EnsureOptimizerState();
  EnsureGradientStaging();
  std::vector<dpc_layer> table;
  for (auto& l : layers)
    table.push_back(l->d);
  Check(dpc_plan_update(plan, table.data(), (int)table.size()));
  for (int s = 0; s < 4; ++s)
  {
    Check(dpc_graph_drop(ctx, s));
    graphKey[s] = -1;
  }
  dirty = false;
}

void PCNetwork::RandomizeWeights(std::mt19937& rng, const char* distribution)
{
  RequireCompiled();
  // Default initialisation of the reference layers: W ~ N(0, sqrt(2/(size+next))) (unit
  // variance under muPC), Psi ~ N(0, sqrt(2/(size+terminal)))
  // (src/layers/DirectKPPCLayer.cpp:184-217, src/layers/FullPCLayer.cpp:163-184).  A
  // "normal(a,b)" / "uniform(a,b)" string overrides W's distribution
  // (include/deepity/utils/RandomizeDistribution.h:27-47).  Values come from one host
  // mt19937 stream; the reference's own stream depends on its thread count, so explicit
  // set_tensor calls are the way to reproduce a given initialisation.
  char name[16] = {0};
  float pa = 0.0f, pb = 1.0f;
  const bool parsed =
      distribution && std::sscanf(distribution, " %15[a-zA-Z] ( %f , %f )", name, &pa, &pb) == 3;
  std::uniform_int_distribution<uint32_t> seedDist;
  for (auto& l : layers)
  {
    if (l->d.next_size <= 0)
      continue;
    const size_t s = l->d.size, nx = l->d.next_size, ts = l->d.terminal_size;
    float limit = (kind == NetworkKind::FULL && useMuPC) ? 1.0f : std::sqrt(2.0f / (s + nx));
    std::vector<float> w(nx * s);
    std::mt19937 wr(seedDist(rng));
    if (parsed && std::strcmp(name, "uniform") == 0)
    {
      std::uniform_real_distribution<float> d(pa, pb);
      for (auto& v : w)
        v = d(wr);
    }
    else
    {
      std::normal_distribution<float> d(parsed ? pa : 0.0f, parsed ? pb : limit);
      for (auto& v : w)
        v = d(wr);
    }
    Check(dpc_copy_h2d_sync(ctx, l->d.W, w.data(), w.size() * sizeof(float)));
    if (l->d.Psi)
    {
      std::vector<float> psi(s * l->d.psi_stride, 0.0f);
      std::mt19937 pr(seedDist(rng));
      std::normal_distribution<float> d(0.0f, std::sqrt(2.0f / (s + ts)));
      for (size_t r = 0; r < s; ++r)
        for (size_t c = 0; c < ts; ++c)
          psi[r * l->d.psi_stride + c] = d(pr);
      Check(dpc_copy_h2d_sync(ctx, l->d.Psi, psi.data(), psi.size() * sizeof(float)));
    }
  }
  Check(dpc_plan_invalidate(plan, 0, (int)layers.size(), DPC_WROTE_W));
}

// ------------------------------------------------------------------------------- state
void PCNetwork::ResetState(bool beliefsOverwritten)
{
  RequireCompiled();
  const size_t B = (size_t)batchSize;
  // z of every layer lives in one arena: one memset covers them all (the reference's
  // batched run does the same for its flat buffer, DirectKPPCNetwork.cpp:38-55).  A train step
  // or prediction that opens with the full forward sweep overwrites every belief (the clamped
  // ends by the clamp copies, the rest by the sweep) before anything reads one, so there the
  // memset would only cost 4 bytes of HBM traffic per belief: it is skipped.
  if (!beliefsOverwritten)
  {
    float* z0 = layers.front()->d.z;
    float* zend = layers.back()->d.z + Pad64(B * layers.back()->d.size);
    Check(dpc_zero(ctx, z0, (size_t)(zend - z0) * sizeof(float)));
    Check(dpc_plan_invalidate(plan, 0, (int)layers.size(), DPC_WROTE_Z));
  }
  if (kind == NetworkKind::FULL) // FullPCLayer::ResetState, src/layers/FullPCLayer.cpp:664-671
  {
    float* e0 = layers.front()->d.e;
    float* eend = layers.back()->d.e + Pad64(B * layers.back()->d.size);
    Check(dpc_zero(ctx, e0, (size_t)(eend - e0) * sizeof(float)));
    if (useMomentum && layers.front()->d.v)
    {
      float* v0 = layers.front()->d.v;
      float* vend = layers.back()->d.v + Pad64(B * layers.back()->d.size);
      Check(dpc_zero(ctx, v0, (size_t)(vend - v0) * sizeof(float)));
    }
  }
}

void PCNetwork::ClampHost(int layer, const float* data, size_t n)
{
  RequireCompiled();
  PCLayer* l = layers.at(layer).get();
  const size_t cap = (size_t)batchSize * l->d.size;
  const size_t count = std::min(n, cap);
  float* stage = (layer == 0) ? pinnedX : pinnedY;
  if (pendingAsync)
  {
    // A previous stream-ordered step may still be reading the staging buffers.
    Check(dpc_sync(ctx));
    pendingAsync = false;
  }
  if (layer != 0 && layer != (int)layers.size() - 1)
  {
    Check(dpc_copy_h2d_sync(ctx, l->d.z, data, count * sizeof(float)));
  }
  else
  {
    std::memcpy(stage, data, count * sizeof(float));
    Check(dpc_copy_h2d(ctx, l->d.z, stage, count * sizeof(float)));
  }
  Check(dpc_plan_invalidate(plan, layer, 1, DPC_WROTE_Z));
  l->clamped = true;
  l->cacheValid = false;
}

void PCNetwork::ClampDevice(int layer, const float* data, size_t n)
{
  RequireCompiled();
  PCLayer* l = layers.at(layer).get();
  const size_t count = std::min(n, (size_t)batchSize * l->d.size);
  Check(dpc_copy_d2d(ctx, l->d.z, data, count * sizeof(float)));
  Check(dpc_plan_invalidate(plan, layer, 1, DPC_WROTE_Z));
  l->clamped = true;
  l->cacheValid = false;
}

void PCNetwork::Clamp(const std::vector<float>& input)
{
  ClampHost(0, input.data(), input.size());
}

// ------------------------------------------------------------------------------ phases
// ComputeMuOnly over a range: clamped layers with a valid cache keep their stored
// prediction (src/layers/DirectKPPCLayer.cpp:275-280), the others run grouped.
void PCNetwork::ForwardRange(int first, int count, int flags)
{
  int i = first;
  const int end = first + count;
  while (i < end)
  {
    PCLayer* l = layers[i].get();
    if (l->d.next_size <= 0)
    {
      ++i;
      continue;
    }
    if (l->clamped && l->cacheValid)
    {
      // Nothing to do when neither the copy, the error nor fe is wanted.
      if (flags & (DPC_FWD_COPY_NEXT | DPC_FWD_ERR_NEXT | DPC_FWD_FE | DPC_FWD_ENERGY))
        Check(dpc_forward(plan, i, 1, flags | DPC_FWD_CACHED));
      ++i;
      continue;
    }
    if (l->clamped)
    {
      // This pass fills the clamped layer's cache (first use in a step, or after iPC
      // invalidated it): its preact/mu must reach memory whatever the caller elides.
      Check(dpc_forward(plan, i, 1, flags & ~(DPC_FWD_TRANSIENT | DPC_FWD_NO_MU)));
      l->cacheValid = true;
      ++i;
      continue;
    }
    int j = i;
    while (j < end && layers[j]->d.next_size > 0 && !layers[j]->clamped)
      ++j;
    Check(dpc_forward(plan, i, j - i, flags));
    i = j;
  }
}

void PCNetwork::ProjectForward()
{
  RequireCompiled();
  const int n = (int)layers.size();
  bool plain = true;
  for (int i = 0; i < n - 1; ++i)
  {
    if (layers[i]->clamped && layers[i]->cacheValid)
      plain = false;
    if (i > 0 && layers[i]->clamped)
      plain = false;
  }
  if (plain)
  {
    // Inside a whole train step only the clamped input layer's mu is read again before it is
    // recomputed (its cached prediction); the others skip the store.
    int extra = transientFlag ? DPC_FWD_NO_MU : 0;
    if (extra && sweepFeedsDfa)
      extra |= DPC_FWD_NO_PREACT; // the direct-feedback update takes f' from the copied outputs
    Check(dpc_project_forward_ex(plan, 0, n - 1, layers.back()->clamped ? 1 : 0, extra));
    for (int i = 0; i < n - 1; ++i)
      if (layers[i]->clamped)
        layers[i]->cacheValid = true;
    return;
  }
  for (int i = 0; i + 1 < n; ++i)
    ForwardRange(i, 1, layers[i + 1]->clamped ? 0 : DPC_FWD_COPY_NEXT);
}

float PCNetwork::CalculateTerminalError()
{
  RequireCompiled();
  Check(dpc_error(plan, (int)layers.size() - 1, 0));
  return 0.0f;
}

void PCNetwork::DirectFeedbackUpdate()
{
  RequireCompiled();
  if (kind == NetworkKind::SIMPLE)
    return;
  const int n = (int)layers.size();
  if (kind == NetworkKind::FULL)
  {
    // Refresh preact against the settled z first (src/networks/FullPCNetwork.cpp:72-82).
    ForwardRange(0, n - 1, 0);
  }
  const int decayW = (kind == NetworkKind::FULL ? DPC_DFA_DECAY_W : 0) |
                     (sweepFeedsDfa && !gradSync ? DPC_DFA_FROM_OUTPUT : 0);
  if (gradSync)
  {
    Check(dpc_weight_gradients(plan, 0, n - 1, 1));
    SyncGradients(gradWCount);
    Check(dpc_apply_gradients(plan, 0, n - 1, 1, globalBatch, decayW & DPC_DFA_DECAY_W));
  }
  else
    Check(dpc_direct_feedback(plan, 0, n - 1, decayW));
}

// CalculateState for every layer, in the reference's order: each layer's error uses the
// prediction its lower neighbour has just refreshed.  Energy goes to the plan's accumulator.
static int StateFlags(NetworkKind kind, bool needEnergy)
{
  int f = DPC_FWD_ERR_NEXT;
  if (needEnergy)
    f |= DPC_FWD_ENERGY;
  if (kind != NetworkKind::SIMPLE)
    f |= DPC_FWD_FE;
  return f;
}

float PCNetwork::CalculateState(bool needEnergy)
{
  RequireCompiled();
  const int n = (int)layers.size();
  Check(dpc_zero(ctx, layers[0]->d.e, (size_t)batchSize * layers[0]->d.size * sizeof(float)));
  int flags = StateFlags(kind, needEnergy) | transientFlag;
  // The energy pass that closes a train step is followed by no state update: nobody reads fe,
  // and its predictions are written only if somebody asks for them (RefreshPredictions).
  if (needEnergy && transientFlag)
    flags &= ~DPC_FWD_FE;
  ForwardRange(0, n - 1, flags);
  if (layers.back()->d.flags & DPC_LAYER_SOFTMAX_CE)
  {
    Check(dpc_error(plan, n - 1, needEnergy ? 1 : 0));
    if (kind != NetworkKind::SIMPLE)
      Check(dpc_feedback_error(plan, n - 2, 1));
  }
  return 0.0f;
}

void PCNetwork::UpdateState()
{
  RequireCompiled();
  const int n = (int)layers.size();
  // FullPC: under an unclamped cross-entropy terminal the top hidden layer gets no
  // top-down signal (src/layers/FullPCLayer.cpp:318-324).
  const bool topDownMeaningless = kind == NetworkKind::FULL &&
                                  (layers.back()->d.flags & DPC_LAYER_SOFTMAX_CE) &&
                                  !layers.back()->clamped;
  int i = 0;
  while (i < n)
  {
    if (layers[i]->clamped)
    {
      ++i;
      continue;
    }
    if (topDownMeaningless && i == n - 2)
    {
      Check(dpc_relax(plan, i));
      ++i;
      continue;
    }
    int j = i;
    while (j < n && !layers[j]->clamped && !(topDownMeaningless && j == n - 2))
      ++j;
    Check(dpc_update_state(plan, i, j - i));
    i = j;
  }
}

// ePC settling step, src/networks/FullPCNetwork.cpp:99-131: a forward sweep that rebuilds each
// hidden belief from the prediction below plus its error, then a top-down sweep that chains the
// adjoint through every layer and moves the errors.
void PCNetwork::EPCStep()
{
  RequireCompiled();
  const int n = (int)layers.size();
  ForwardRange(0, 1, 0);
  for (int i = 1; i + 1 < n; ++i)
  {
    Check(dpc_epc_reconstruct(plan, i));
    ForwardRange(i, 1, 0);
  }
  Check(dpc_error(plan, n - 1, 0));
  bool firstHop = true;
  for (int i = n - 2; i >= 1; --i)
  {
    Check(dpc_epc_adjoint(plan, i, firstHop ? 1 : 0, firstHop ? -1.0f : 1.0f,
                          layers[i]->clamped ? 1 : 0));
    firstHop = false;
  }
}

float PCNetwork::Step(bool computeEnergy)
{
  double e = 0.0;
  if (computeEnergy)
    Check(dpc_energy_reset(plan));
  CalculateState(computeEnergy);
  UpdateState();
  if (computeEnergy)
    Check(dpc_energy_read(plan, &e));
  return (float)e;
}

void PCNetwork::UpdateWeights()
{
  RequireCompiled();
  SyncPlan();
  const int n = (int)layers.size();
  if (kind != NetworkKind::SIMPLE)
  {
    // preact/mu are one settling step behind z: refresh them, and with them the local
    // gradient fe = e_above * f'(preact) (src/networks/DirectKPPCNetwork.cpp:481-495).
    ForwardRange(0, n - 1, DPC_FWD_FE | transientFlag);
  }
  if (gradSync)
  {
    Check(dpc_weight_gradients(plan, 0, n - 1, 0));
    SyncGradients(gradCount);
    Check(dpc_apply_gradients(plan, 0, n - 1, 0, globalBatch, centerWeights ? 1 : 0));
  }
  else
    Check(dpc_update_weights(plan, 0, n - 1, centerWeights ? 1 : 0));
}

// Inside a whole train step the predictions of the settling passes and of the pre-update
// refresh are consumed only through the fused e / fe outputs (the final energy pass
// recomputes and stores them), so those passes need not write preact/mu at all.  A softmax
// head reads preact of the layer below through a separate kernel, so it keeps the stores.
struct TransientScope
{
  int& flag;
  TransientScope(int& f, bool on) : flag(f) { flag = on ? DPC_FWD_TRANSIENT : 0; }
  ~TransientScope() { flag = 0; }
};

// The last pass of a train step computes every layer's prediction for the energy but does not
// store it; whoever wants to look at mu / preact afterwards gets them recomputed here from the
// same beliefs and weights (a clamped layer keeps its cached prediction, as in the reference).
void PCNetwork::RefreshPredictions()
{
  if (!predictionsStale || !plan)
    return;
  predictionsStale = false;
  ForwardRange(0, (int)layers.size() - 1, 0);
  Check(dpc_sync(ctx));
}

void PCNetwork::RunTrainPhases(int mode, int steps)
{
  const int n = (int)layers.size();
  TransientScope scope(transientFlag, kind != NetworkKind::SIMPLE &&
                                          !(layers.back()->d.flags & DPC_LAYER_SOFTMAX_CE));
  auto settle = [&](bool energy)
  {
    CalculateState(energy);
    UpdateState();
  };
  if (kind == NetworkKind::DIRECT_KP)
  {
    // The direct-feedback update follows the sweep at once: z[l+1] still equals f(preact[l]),
    // so it can take f' from z[l+1] and the sweep need not store preact -- when every
    // activation's derivative is a function of its output and no gradient staging is on.
    bool fromOutput = !gradSync && !ghostTop;
    for (int i = 0; i + 1 < n && fromOutput; ++i)
    {
      const int a = layers[i]->d.act;
      fromOutput = a == DPC_ACT_TANH || a == DPC_ACT_SIGMOID || a == DPC_ACT_RELU ||
                   a == DPC_ACT_LINEAR || a == DPC_ACT_HARD_TANH;
      for (int k = 1; k + 1 < n; ++k)
        fromOutput = fromOutput && !layers[k]->clamped;
    }
    sweepFeedsDfa = fromOutput;
    ProjectForward();
    CalculateTerminalError();
    DirectFeedbackUpdate();
    sweepFeedsDfa = false;
    for (int t = 0; t < steps; ++t)
      settle(false);
    UpdateWeights();
    Check(dpc_energy_reset(plan));
    CalculateState(true);
  }
  else if (kind == NetworkKind::FULL)
  {
    ProjectForward();
    CalculateTerminalError();
    for (int t = 0; t < steps; ++t)
    {
      if (useEPC)
        EPCStep();
      else
        settle(false);
      if (useIPC)
      {
        UpdateWeights();
        for (auto& l : layers)
          l->InvalidateMuCache();
      }
    }
    DirectFeedbackUpdate();
    if (!useIPC)
      UpdateWeights();
    Check(dpc_energy_reset(plan));
    CalculateState(true);
  }
  else if (mode == 0)
  {
    for (int t = 0; t < steps; ++t)
      settle(false);
    Check(dpc_energy_reset(plan));
    CalculateState(true);
    UpdateWeights();
  }
  else if (mode == 1)
  {
    ProjectForward();
    for (int t = 0; t < steps; ++t)
      settle(false);
    UpdateWeights();
    Check(dpc_energy_reset(plan));
    CalculateState(true);
  }
  else
  {
    Check(dpc_energy_reset(plan));
    for (int t = 0; t < steps; ++t)
      settle(true);
    UpdateWeights();
  }
  (void)n;
}

float PCNetwork::TrainStepRaw(int mode, const float* x, size_t nx, const float* y, size_t ny,
                              int steps, bool onDevice, bool readEnergy)
{
  RequireCompiled();
  if (steps < 0 || mode < 0 || mode > 2)
    throw std::invalid_argument("deepity_b200: bad inference step count or mode");
  if (kind != NetworkKind::SIMPLE)
    mode = 0;
  SyncPlan();
  const int n = (int)layers.size();
  predictionsStale = false; // everything is recomputed from here on
  // DirectKP / Full steps open with the forward sweep over the whole stack; x and y must then
  // cover their layers completely (a short buffer leaves the rest at zero, as the memset would)
  const bool sweepOverwrites = kind != NetworkKind::SIMPLE &&
                               nx >= (size_t)batchSize * layers.front()->d.size &&
                               ny >= (size_t)batchSize * layers.back()->d.size;
  ResetState(sweepOverwrites);
  if (onDevice)
  {
    ClampDevice(0, x, nx);
    ClampDevice(n - 1, y, ny);
  }
  else
  {
    ClampHost(0, x, nx);
    ClampHost(n - 1, y, ny);
  }
  for (int i = 1; i + 1 < n; ++i)
    layers[i]->clamped = false;
  // A recorded step holds no host logic: whatever operand copies are stale now are rebuilt
  // before the graph runs, so that recording and every replay start from the same state.
  Check(dpc_plan_sync_operands(plan));

  if (useGraph && !gradSync)
  {
    const long key = (long)mode * 1000000L + steps;
    if (graphKey[0] != key)
    {
      Check(dpc_graph_begin(ctx, 0));
      try
      {
        RunTrainPhases(mode, steps);
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
    // The replay does what RunTrainPhases did while recording; bring the host flags to the
    // same end state (the input layer's prediction is cached again).
    for (auto& l : layers)
      if (l->clamped && l->d.next_size > 0)
        l->cacheValid = true;
  }
  else
    RunTrainPhases(mode, steps);
  // (same condition as the TransientScope of RunTrainPhases; a graph replay runs no host code)
  predictionsStale =
      kind != NetworkKind::SIMPLE && !(layers.back()->d.flags & DPC_LAYER_SOFTMAX_CE);

  double energy = 0.0;
  if (readEnergy)
    Check(dpc_energy_read(plan, &energy));
  else
    pendingAsync = true;
  UnclampTerminal();
  return (float)energy;
}

float PCNetwork::TrainStep(const std::vector<float>& x, const std::vector<float>& y,
                           int inferenceSteps)
{
  return TrainStepRaw(0, x.data(), x.size(), y.data(), y.size(), inferenceSteps, false, true);
}

void PCNetwork::RunPredictPhases(int steps, bool withProjection)
{
  const int n = (int)layers.size();
  if (withProjection)
    ProjectForward();
  for (int t = 0; t < steps; ++t)
  {
    if (useEPC)
      EPCStep();
    else
    {
      CalculateState(false);
      UpdateState();
    }
  }
  if (kind == NetworkKind::FULL && (layers.back()->d.flags & DPC_LAYER_SOFTMAX_CE))
  {
    // The cross-entropy head reports the logits below it
    // (src/networks/FullPCNetwork.cpp:285-291).
    ForwardRange(n - 2, 1, DPC_FWD_COPY_NEXT);
  }
}

void PCNetwork::PredictRaw(const float* x, size_t nx, int steps, bool withProjection, float* out,
                           size_t nout)
{
  RequireCompiled();
  SyncPlan();
  const int n = (int)layers.size();
  const size_t count = (size_t)batchSize * layers.back()->d.size;
  if (nout != count)
    throw std::invalid_argument("deepity_b200: Predict() output buffer has the wrong size");
  if (kind != NetworkKind::SIMPLE)
    withProjection = true;
  predictionsStale = false;
  ResetState(withProjection && kind != NetworkKind::SIMPLE &&
             nx >= (size_t)batchSize * layers.front()->d.size);
  ClampHost(0, x, nx);
  for (int i = 1; i < n; ++i)
    layers[i]->clamped = false;
  Check(dpc_plan_sync_operands(plan));
  if (useGraph)
  {
    const long key = (long)steps * 2 + (withProjection ? 1 : 0);
    if (graphKey[1] != key)
    {
      Check(dpc_graph_begin(ctx, 1));
      try
      {
        RunPredictPhases(steps, withProjection);
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
      if (l->clamped && l->d.next_size > 0)
        l->cacheValid = true;
  }
  else
    RunPredictPhases(steps, withProjection);
  Check(dpc_copy_d2h_sync(ctx, pinnedOut, layers.back()->d.z, count * sizeof(float)));
  std::memcpy(out, pinnedOut, count * sizeof(float));
}

std::vector<float> PCNetwork::Predict(const std::vector<float>& x, int inferenceSteps)
{
  std::vector<float> r((size_t)batchSize * layers.back()->d.size);
  PredictRaw(x.data(), x.size(), inferenceSteps, kind != NetworkKind::SIMPLE, r.data(), r.size());
  return r;
}

// ------------------------------------------------------------------------------ setters
void PCNetwork::SetOptimizer(OptimizerType o)
{
  opt = o;
  for (auto& l : layers)
    l->d.opt = (int)o;
  Dirty();
}
void PCNetwork::SetPsiOptimizer(OptimizerType o)
{
  optPsi = o;
  for (auto& l : layers)
    l->d.opt_psi = (int)o;
  Dirty();
}
void PCNetwork::SetCenterWeights(bool enabled)
{
  if (enabled == centerWeights)
    return;
  centerWeights = enabled;
  Dirty();
}
void PCNetwork::SetLearningRate(float lr)
{
  for (auto& l : layers)
    l->d.lr = lr;
  Dirty();
}
void PCNetwork::SetFeedbackRate(float fl)
{
  for (auto& l : layers)
    l->d.fl = fl;
  Dirty();
}
void PCNetwork::SetInferenceRate(float ir)
{
  for (auto& l : layers)
    l->d.ir = ir;
  Dirty();
}
void PCNetwork::SetPsiDecay(float decay)
{
  psiDecay = decay;
  for (auto& l : layers)
    l->d.psi_decay = decay;
  Dirty();
}
void PCNetwork::SetUseCrossEntropy(bool enabled)
{
  crossEntropy = enabled;
  if (!layers.empty() && plan)
  {
    if (enabled)
      layers.back()->d.flags |= DPC_LAYER_SOFTMAX_CE;
    else
      layers.back()->d.flags &= ~DPC_LAYER_SOFTMAX_CE;
  }
  Dirty();
}
void PCNetwork::SetUseMuPCScaling(bool enabled)
{
  if (plan)
    throw std::logic_error("deepity_b200: SetUseMuPCScaling() must precede Compile()");
  useMuPC = enabled;
}
void PCNetwork::SetUseResidualConnections(bool enabled)
{
  if (plan)
    throw std::logic_error("deepity_b200: SetUseResidualConnections() must precede Compile()");
  useResidual = enabled;
}
void PCNetwork::SetUseEPC(bool enabled)
{
  if (plan)
    throw std::logic_error("deepity_b200: SetUseEPC() must precede Compile()");
  if (kind != NetworkKind::FULL)
    throw std::invalid_argument("deepity_b200: ePC exists for FullPCNetwork only");
  useEPC = enabled;
}
void PCNetwork::SetUseIPC(bool enabled)
{
  useIPC = enabled;
  Dirty();
}
void PCNetwork::SetUseMomentum(bool enabled, float beta)
{
  if (plan)
    throw std::logic_error("deepity_b200: SetUseMomentum() must precede Compile()");
  useMomentum = enabled;
  momentumBeta = beta;
  for (auto& l : layers)
    l->d.momentum_beta = beta;
}
void PCNetwork::SetPrecision(int precision)
{
  Check(dpc_set_precision(ctx, precision));
  Dirty();
}
void PCNetwork::SetGhostTop(bool enabled)
{
  if (plan)
    throw std::logic_error("deepity_b200: SetGhostTop() must precede Compile()");
  ghostTop = enabled;
}
void PCNetwork::SetUseGraph(bool enabled)
{
  useGraph = enabled;
  Dirty();
}

int64_t PCNetwork::LaunchCount() const
{
  return dpc_launch_count(ctx);
}

// Algorithmic GEMM FLOPs of one train step (2*M*N*K per GEMM actually required by the
// CPU semantics; a clamped input layer computes its prediction once per step).
double PCNetwork::TrainStepFlops(int T) const
{
  const double B = batchSize;
  const int n = (int)layers.size();
  double total = 0.0;
  for (int i = 0; i + 1 < n; ++i)
  {
    const double s = layers[i]->d.size, nx = layers[i]->d.next_size, ts = layers[i]->d.terminal_size;
    const double g = 2.0 * B * s * nx;
    double fwd, fb, wg;
    if (kind == NetworkKind::DIRECT_KP)
    {
      fwd = T + 3, fb = T, wg = 2; // P0, T x P3a, refresh, final energy; DFA + learn
      if (i + 2 >= n)
        wg = 1; // upper neighbour is the terminal: no DFA
      total += 2.0 * B * s * ts;                // Psi update
      if (i + 2 < n)
        total += 2.0 * B * nx * ts;             // DFA projection
    }
    else if (kind == NetworkKind::FULL)
    {
      fwd = T + 4, fb = T, wg = 2;
      if (i + 2 >= n)
        wg = 1;
      total += 2.0 * B * s * ts;
      if (i + 2 < n)
        total += 2.0 * B * nx * ts;
    }
    else
    {
      fwd = T + 1, fb = T, wg = 1;
    }
    if (i == 0)
    {
      fwd = 1; // clamped: cached after the first evaluation
      fb = 0;  // clamped: never updated
    }
    total += g * (fwd + fb + wg);
  }
  return total;
}

int32_t* PCNetwork::Counter(int layer, const std::string& name)
{
  if (layer < 0 || layer >= (int)layers.size() || !plan)
    return nullptr;
  SyncPlan(); // an optimizer chosen after Compile() gets its state here
  const dpc_layer& d = layers[layer]->d;
  if (d.next_size <= 0)
    return nullptr;
  if (name == "step")
    return d.opt != DPC_OPT_SGD ? d.t : nullptr;
  if (name == "psi_step")
    return (d.Psi && d.opt_psi != DPC_OPT_SGD) ? d.t_Psi : nullptr;
  return nullptr;
}

// What Layer::GetStateDict() and GetOptimizerStateDict() list for every weight layer
// (src/layers/DirectKPPCLayer.cpp:219-235, src/layers/SimplePCLayer.cpp, FullPCLayer.cpp).
std::vector<PCNetwork::StateEntry> PCNetwork::StateDict()
{
  std::vector<StateEntry> out;
  if (!plan)
    return out;
  SyncPlan();
  for (int i = 0; i < (int)layers.size(); ++i)
  {
    const dpc_layer& d = layers[i]->d;
    if (d.next_size <= 0)
      continue;
    const size_t s = d.size, n = d.next_size, ts = d.terminal_size, ps = d.psi_stride;
    out.push_back({i, "W", n, s, s, false});
    out.push_back({i, "b", 1, n, n, false});
    if (d.Psi)
      out.push_back({i, "Psi", s, ts, ps, false});
    if (d.opt != DPC_OPT_SGD && d.m_W)
    {
      out.push_back({i, "weight.m", n, s, s, true});
      out.push_back({i, "weight.v", n, s, s, true});
      out.push_back({i, "bias.m", 1, n, n, true});
      out.push_back({i, "bias.v", 1, n, n, true});
    }
    if (d.Psi && d.opt_psi != DPC_OPT_SGD && d.m_Psi)
    {
      out.push_back({i, "psi.m", s, ts, ps, true});
      out.push_back({i, "psi.v", s, ts, ps, true});
    }
  }
  return out;
}

bool PCNetwork::FindTensor(int layer, const std::string& name, float** ptr, size_t* rows,
                           size_t* cols, size_t* stride)
{
  if (layer < 0 || layer >= (int)layers.size() || !plan)
    return false;
  const dpc_layer& d = layers[layer]->d;
  const size_t B = batchSize, s = d.size, n = d.next_size, ts = d.terminal_size;
  float* p = nullptr;
  size_t r = 0, c = 0, st = 0;
  if (name == "z")
    p = d.z, r = B, c = s;
  else if (name == "e")
    p = d.e, r = B, c = s;
  else if (name == "v")
    p = d.v, r = B, c = s;
  else if (name == "zF")
    p = d.zF, r = B, c = s;
  else if (name == "adj")
    p = d.adj, r = B, c = s;
  else if (name == "Psi" && n == 0 && d.Psi)
    p = d.Psi, r = s, c = ts, st = d.psi_stride;
  else if (name == "eT" && ghostET && layer == (int)layers.size() - 1)
    p = ghostET, r = B, c = ts;
  else if (n > 0)
  {
    if (name == "mu" || name == "preact")
      RefreshPredictions();
    if (name == "mu")
      p = d.mu, r = B, c = n;
    else if (name == "preact")
      p = d.preact, r = B, c = n;
    else if (name == "fe")
      p = d.fe, r = B, c = n;
    else if (name == "W")
      p = d.W, r = n, c = s;
    else if (name == "b")
      p = d.b, r = 1, c = n;
    else if (name == "Psi")
      p = d.Psi, r = s, c = ts, st = d.psi_stride;
    else if (name == "weight.m")
      p = d.m_W, r = n, c = s;
    else if (name == "weight.v")
      p = d.v_W, r = n, c = s;
    else if (name == "bias.m")
      p = d.m_b, r = 1, c = n;
    else if (name == "bias.v")
      p = d.v_b, r = 1, c = n;
    else if (name == "psi.m")
      p = d.m_Psi, r = s, c = ts, st = d.psi_stride;
    else if (name == "psi.v")
      p = d.v_Psi, r = s, c = ts, st = d.psi_stride;
  }
  if (!p)
    return false;
  *ptr = p, *rows = r, *cols = c, *stride = st ? st : c;
  return true;
}
} // namespace Deep

// =======================================================================================
// dpcn_* : the binding surface (C linkage from deepity_b200.h).
// =======================================================================================
struct dpcn_net
{
  std::unique_ptr<Deep::PCNetwork> net;
  int kind;
};

namespace dpc
{
void set_error(const std::string& msg); // dpc_core.cu: message slot behind dpc_last_error()
}

namespace
{
// No exception crosses the C boundary: host-level failures become a status code plus the
// message that dpc_last_error() returns.
int Guard(const std::function<void()>& fn)
{
  try
  {
    fn();
    return DPC_OK;
  }
  catch (const Deep::StatusError& e)
  {
    // a dpc_* call failed underneath: its status travels up unchanged (DPC_ERR_TIMEOUT ...)
    dpc::set_error(e.what());
    return e.status;
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

int dpcn_create(int kind, int batch, int device, dpcn_net** out)
{
  if (!out || kind < 0 || kind > 2)
  {
    dpc::set_error("dpcn_create: bad argument");
    return DPC_ERR_INVALID;
  }
  return Guard(
      [&]
      {
        auto* n = new dpcn_net();
        n->kind = kind;
        n->net = std::make_unique<Deep::PCNetwork>((Deep::NetworkKind)kind, batch, device);
        *out = n;
      });
}

int dpcn_destroy(dpcn_net* net)
{
  delete net;
  return DPC_OK;
}

int dpcn_add_layer(dpcn_net* net, int size, int next_size, int terminal_size, float lr, float ir,
                   float fl, float lmbda, int act)
{
  if (!net || size <= 0 || next_size < 0)
  {
    dpc::set_error("dpcn_add_layer: bad argument");
    return DPC_ERR_INVALID;
  }
  return Guard([&] {
    net->net->AddLayerImpl(size, next_size, terminal_size, lr, ir, fl, lmbda,
                           (Deep::ActivationType)act);
  });
}

int dpcn_set_option(dpcn_net* net, const char* name, int iv, float fv)
{
  if (!net || !name)
  {
    dpc::set_error("dpcn_set_option: null argument");
    return DPC_ERR_INVALID;
  }
  const std::string nm(name);
  return Guard(
      [&]
      {
        Deep::PCNetwork& n = *net->net;
        if (nm == "optimizer")
          n.SetOptimizer((Deep::OptimizerType)iv);
        else if (nm == "psi_optimizer")
          n.SetPsiOptimizer((Deep::OptimizerType)iv);
        else if (nm == "center_weights")
          n.SetCenterWeights(iv != 0);
        else if (nm == "psi_decay")
          n.SetPsiDecay(fv);
        else if (nm == "learning_rate")
          n.SetLearningRate(fv);
        else if (nm == "feedback_rate")
          n.SetFeedbackRate(fv);
        else if (nm == "inference_rate")
          n.SetInferenceRate(fv);
        else if (nm == "cross_entropy")
          n.SetUseCrossEntropy(iv != 0);
        else if (nm == "mupc")
          n.SetUseMuPCScaling(iv != 0);
        else if (nm == "residual")
          n.SetUseResidualConnections(iv != 0);
        else if (nm == "ipc")
          n.SetUseIPC(iv != 0);
        else if (nm == "epc")
          n.SetUseEPC(iv != 0);
        else if (nm == "momentum")
          n.SetUseMomentum(iv != 0, fv);
        else if (nm == "precision")
          n.SetPrecision(iv);
        else if (nm == "ghost_top")
          n.SetGhostTop(iv != 0);
        else if (nm == "use_graph")
          n.SetUseGraph(iv != 0);
        else
          throw std::invalid_argument("unknown option '" + nm + "'");
      });
}

int dpcn_compile(dpcn_net* net)
{
  if (!net)
    return DPC_ERR_INVALID;
  return Guard([&] { net->net->Compile(); });
}

int dpcn_num_layers(dpcn_net* net)
{
  return net ? (int)net->net->GetLayers().size() : DPC_ERR_INVALID;
}

int64_t dpcn_tensor_size(dpcn_net* net, int layer, const char* name)
{
  float* p;
  size_t r, c, st;
  if (!net || !name || !net->net->FindTensor(layer, name, &p, &r, &c, &st))
    return 0;
  return (int64_t)(r * c);
}

// Device address of an optimizer step counter, or NULL (no such layer / SGD).
static int32_t* CounterPtr(dpcn_net* net, int layer, const char* name)
{
  if (!net || !name)
    return nullptr;
  return net->net->Counter(layer, name);
}

int dpcn_get_counter(dpcn_net* net, int layer, const char* name, int32_t* out)
{
  if (!net || !name || !out)
    return DPC_ERR_INVALID;
  std::string nm(name);
  if (nm != "step" && nm != "psi_step")
  {
    dpc::set_error("dpcn_get_counter: the counters are \"step\" and \"psi_step\"");
    return DPC_ERR_INVALID;
  }
  int32_t* p = CounterPtr(net, layer, name);
  if (!p)
  {
    dpc::set_error("dpcn_get_counter: this layer has no such counter (SGD, or no weights)");
    return DPC_ERR_STATE;
  }
  return dpc_copy_d2h_sync(net->net->Context(), out, p, sizeof(int32_t));
}

int dpcn_set_counter(dpcn_net* net, int layer, const char* name, int32_t value)
{
  if (!net || !name)
    return DPC_ERR_INVALID;
  std::string nm(name);
  if (nm != "step" && nm != "psi_step")
  {
    dpc::set_error("dpcn_set_counter: the counters are \"step\" and \"psi_step\"");
    return DPC_ERR_INVALID;
  }
  int32_t* p = CounterPtr(net, layer, name);
  if (!p)
  {
    dpc::set_error("dpcn_set_counter: this layer has no such counter (SGD, or no weights)");
    return DPC_ERR_STATE;
  }
  return dpc_copy_h2d_sync(net->net->Context(), p, &value, sizeof(int32_t));
}

int dpcn_state_dict_size(dpcn_net* net)
{
  if (!net)
    return DPC_ERR_INVALID;
  return (int)net->net->StateDict().size();
}

int dpcn_state_dict_entry(dpcn_net* net, int index, int* layer, char* name, int name_bytes,
                          int64_t* rows, int64_t* cols, int64_t* row_stride, int* optimizer_state)
{
  if (!net)
    return DPC_ERR_INVALID;
  const auto dict = net->net->StateDict();
  if (index < 0 || index >= (int)dict.size())
  {
    dpc::set_error("dpcn_state_dict_entry: index out of range");
    return DPC_ERR_INVALID;
  }
  const auto& e = dict[index];
  if (layer)
    *layer = e.layer;
  if (name && name_bytes > 0)
    snprintf(name, (size_t)name_bytes, "%s", e.name.c_str());
  if (rows)
    *rows = (int64_t)e.rows;
  if (cols)
    *cols = (int64_t)e.cols;
  if (row_stride)
    *row_stride = (int64_t)e.stride;
  if (optimizer_state)
    *optimizer_state = e.optimizer ? 1 : 0;
  return DPC_OK;
}

int dpcn_tensor_ptr(dpcn_net* net, int layer, const char* name, void** out, int64_t* row_stride)
{
  float* p;
  size_t r, c, st;
  if (!net || !name || !out || !net->net->FindTensor(layer, name, &p, &r, &c, &st))
  {
    dpc::set_error("dpcn_tensor_ptr: no such tensor");
    return DPC_ERR_INVALID;
  }
  *out = p;
  if (row_stride)
    *row_stride = (int64_t)st;
  return DPC_OK;
}

int dpcn_get_tensor(dpcn_net* net, int layer, const char* name, float* host_out, int64_t count)
{
  float* p;
  size_t r, c, st;
  if (!net || !name || !host_out || !net->net->FindTensor(layer, name, &p, &r, &c, &st) ||
      (int64_t)(r * c) != count)
  {
    dpc::set_error("dpcn_get_tensor: no such tensor or wrong element count");
    return DPC_ERR_INVALID;
  }
  dpc_ctx* ctx = net->net->Context();
  if (st == c)
    return dpc_copy_d2h_sync(ctx, host_out, p, r * c * sizeof(float));
  std::vector<float> tmp(r * st);
  int rc = dpc_copy_d2h_sync(ctx, tmp.data(), p, tmp.size() * sizeof(float));
  if (rc != DPC_OK)
    return rc;
  for (size_t i = 0; i < r; ++i)
    std::memcpy(host_out + i * c, tmp.data() + i * st, c * sizeof(float));
  return DPC_OK;
}

int dpcn_set_tensor(dpcn_net* net, int layer, const char* name, const float* host_in,
                    int64_t count)
{
  float* p;
  size_t r, c, st;
  if (!net || !name || !host_in || !net->net->FindTensor(layer, name, &p, &r, &c, &st) ||
      (int64_t)(r * c) != count)
  {
    dpc::set_error("dpcn_set_tensor: no such tensor or wrong element count");
    return DPC_ERR_INVALID;
  }
  dpc_ctx* ctx = net->net->Context();
  const std::string nm(name);
  if (nm == "z" || nm == "W" || nm == "fe")
    dpc_plan_invalidate(net->net->Plan(), layer, 1,
                        nm == "z" ? DPC_WROTE_Z : (nm == "W" ? DPC_WROTE_W : DPC_WROTE_FE));
  if (st == c)
    return dpc_copy_h2d_sync(ctx, p, host_in, r * c * sizeof(float));
  std::vector<float> tmp(r * st, 0.0f);
  for (size_t i = 0; i < r; ++i)
    std::memcpy(tmp.data() + i * st, host_in + i * c, c * sizeof(float));
  return dpc_copy_h2d_sync(ctx, p, tmp.data(), tmp.size() * sizeof(float));
}

int dpcn_randomize(dpcn_net* net, uint32_t seed)
{
  if (!net)
    return DPC_ERR_INVALID;
  return Guard(
      [&]
      {
        std::mt19937 rng(seed);
        net->net->RandomizeWeights(rng, "normal");
      });
}

int dpcn_train_step(dpcn_net* net, const float* x, int64_t nx, const float* y, int64_t ny,
                    int steps, float* energy_out)
{
  return dpcn_train_step_mode(net, 0, x, nx, y, ny, steps, energy_out);
}

int dpcn_train_step_mode(dpcn_net* net, int mode, const float* x, int64_t nx, const float* y,
                         int64_t ny, int steps, float* energy_out)
{
  if (!net || !x || !y || nx <= 0 || ny <= 0)
  {
    dpc::set_error("dpcn_train_step: null or empty input");
    return DPC_ERR_INVALID;
  }
  return Guard(
      [&]
      {
        float e = net->net->TrainStepRaw(mode, x, (size_t)nx, y, (size_t)ny, steps, false,
                                         energy_out != nullptr);
        if (energy_out)
          *energy_out = e;
      });
}

int dpcn_train_step_device(dpcn_net* net, const float* x_dev, int64_t nx, const float* y_dev,
                           int64_t ny, int steps, float* energy_out)
{
  if (!net || !x_dev || !y_dev || nx <= 0 || ny <= 0)
  {
    dpc::set_error("dpcn_train_step_device: null or empty input");
    return DPC_ERR_INVALID;
  }
  return Guard(
      [&]
      {
        float e = net->net->TrainStepRaw(0, x_dev, (size_t)nx, y_dev, (size_t)ny, steps, true,
                                         energy_out != nullptr);
        if (energy_out)
          *energy_out = e;
      });
}

int dpcn_predict(dpcn_net* net, const float* x, int64_t nx, int steps, int with_projection,
                 float* host_out, int64_t nout)
{
  if (!net || !x || !host_out || nx <= 0)
  {
    dpc::set_error("dpcn_predict: null or empty input");
    return DPC_ERR_INVALID;
  }
  return Guard([&] {
    net->net->PredictRaw(x, (size_t)nx, steps, with_projection != 0, host_out, (size_t)nout);
  });
}

int dpcn_reset_state(dpcn_net* net)
{
  if (!net)
    return DPC_ERR_INVALID;
  return Guard([&] { net->net->ResetState(); });
}

dpc_ctx* dpcn_context(dpcn_net* net)
{
  return net ? net->net->Context() : nullptr;
}

dpc_plan* dpcn_plan(dpcn_net* net)
{
  if (!net)
    return nullptr;
  net->net->FlushSettings();
  return net->net->Plan();
}

int dpcn_set_gradient_sync(dpcn_net* net, dpcn_sync_fn sync, void* user, int global_batch)
{
  if (!net)
    return DPC_ERR_INVALID;
  return Guard([&] { net->net->SetGradientSync(sync, user, global_batch); });
}

int64_t dpcn_launch_count(dpcn_net* net)
{
  return net ? net->net->LaunchCount() : 0;
}

double dpcn_train_step_flops(dpcn_net* net, int steps)
{
  return net ? net->net->TrainStepFlops(steps) : 0.0;
}
