// Context, memory, CUDA graphs, plans and the phase entry points of the dpc_* C ABI.
#include <cstdio>
#include <cstring>
#include <string>

#include "dpc_internal.h"
#include "dpc_simt.cuh"

namespace dpc
{
static thread_local std::string g_error;

void set_error(const std::string& msg)
{
  g_error = msg;
}
int fail(int code, const std::string& msg)
{
  g_error = msg;
  return code;
}
int cuda_fail(cudaError_t err, const char* what)
{
  g_error = std::string(what) + ": " + cudaGetErrorString(err);
  return err == cudaErrorNoDevice || err == cudaErrorInsufficientDriver ? DPC_ERR_NO_DEVICE
                                                                         : DPC_ERR_CUDA;
}

static int check_launch(dpc_ctx* ctx, const char* what)
{
  ctx->launches += 1;
  cudaError_t err = cudaPeekAtLastError();
  if (err != cudaSuccess)
    return cuda_fail(cudaGetLastError(), what);
  return DPC_OK;
}

// How many CTAs of a cluster share the batch rows of one block's columns in the batch reductions
// (Psi update, bias column sums): doubled while the launch has fewer than four CTAs per SM (a CTA's
// time is one chain of dependent row loads: more, shorter chains hide more latency) and every CTA
// keeps at least `min_rows` rows.  1 for launches over many layers.
static int row_split(const dpc_ctx* ctx, long long blocks, int batch, int min_rows)
{
  int R = 1;
  while (R < 8 && blocks * R < 4LL * ctx->sm_count && batch / (2 * R) >= min_rows)
    R *= 2;
  return R;
}

// kern<<<(grid.x, grid.y, R), threads, 0, st>>> as clusters of R CTAs along z (R = 1: a plain launch)
template <typename... KArgs, typename... Args>
static void launch_row_split(void (*kern)(KArgs...), dim3 grid, int threads, int R, cudaStream_t st,
                             Args... args)
{
  if (R <= 1)
  {
    kern<<<grid, threads, 0, st>>>(args...);
    return;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid.x, grid.y, (unsigned)R);
  cfg.blockDim = dim3((unsigned)threads);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = (unsigned)R;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kern, args...); // an error stays pending for check_launch()
}

static int check_range(dpc_plan* p, int first, int count)
{
  if (!p)
    return fail(DPC_ERR_INVALID, "null plan");
  if (first < 0 || count < 0 || first + count > p->n)
    return fail(DPC_ERR_INVALID, "layer range out of bounds");
  return DPC_OK;
}

static inline int cdiv(int a, int b)
{
  return (a + b - 1) / b;
}

// Largest GEMM tile grid over a range for the given op.
static void max_tiles(const dpc_plan* p, int first, int count, int op, int& tx, int& ty)
{
  tx = ty = 0;
  for (int i = first; i < first + count; ++i)
  {
    const dpc_layer& L = p->h[i];
    if (L.next_size <= 0)
      continue;
    int M, N;
    if (op == OP_FWD)
      M = p->batch, N = L.next_size;
    else if (op == OP_FB)
      M = p->batch, N = L.size;
    else
      M = L.next_size, N = L.size;
    tx = std::max(tx, cdiv(N, BN));
    ty = std::max(ty, cdiv(M, BM));
  }
}

static int elem_blocks(const dpc_plan* p, size_t max_elems)
{
  size_t blocks = (max_elems + 1023) / 1024; // 256 threads x 4 elements each
  size_t cap = (size_t)p->ctx->sm_count * 8;
  if (blocks > cap)
    blocks = cap;
  return (int)std::max<size_t>(blocks, 1);
}

constexpr int kMaxZ = 32768; // layers per launch (gridDim.y/z limit is 65535)
} // namespace dpc

using namespace dpc;

// The C linkage of every dpc_* definition below comes from its declaration in
// deepity_b200.h.
const char* dpc_last_error(void)
{
  return g_error.c_str();
}

const char* dpc_version(void)
{
  return "deepity_b200 0.1 (sm_100a)";
}

int dpc_create(int device, dpc_ctx** out)
{
  if (!out)
    return fail(DPC_ERR_INVALID, "dpc_create: null out");
  int n = 0;
  cudaError_t err = cudaGetDeviceCount(&n);
  if (err != cudaSuccess || n == 0)
  {
    cudaGetLastError();
    return fail(DPC_ERR_NO_DEVICE, "no CUDA device available (this library has no CPU fallback)");
  }
  if (device < 0 || device >= n)
    return fail(DPC_ERR_INVALID, "dpc_create: device index out of range");
  DPC_CUDA(cudaSetDevice(device));
  auto* ctx = new dpc_ctx();
  ctx->device = device;
  cudaDeviceProp prop;
  DPC_CUDA(cudaGetDeviceProperties(&prop, device));
  ctx->sm_count = prop.multiProcessorCount;
  DPC_CUDA(cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking));
  // streams that consecutive single tensor-core layers of one phase fork to (see dispatch_range)
  if (!getenv("DPC_DISABLE_LAYER_STREAMS"))
  {
    bool ok = cudaEventCreateWithFlags(&ctx->fork_ev, cudaEventDisableTiming) == cudaSuccess;
    for (int s = 0; s < dpc_ctx::kSide && ok; ++s)
      ok = cudaStreamCreateWithFlags(&ctx->side[s], cudaStreamNonBlocking) == cudaSuccess &&
           cudaEventCreateWithFlags(&ctx->join_ev[s], cudaEventDisableTiming) == cudaSuccess;
    if (!ok)
    {
      const cudaError_t e = cudaGetLastError();
      dpc_destroy(ctx);
      return cuda_fail(e, "creating the per-layer streams");
    }
  }
  *out = ctx;
  return DPC_OK;
}

int dpc_destroy(dpc_ctx* ctx)
{
  if (!ctx)
    return DPC_OK;
  cudaSetDevice(ctx->device);
  for (int s = 0; s < dpc_ctx::kSlots; ++s)
  {
    if (ctx->execs[s])
      cudaGraphExecDestroy(ctx->execs[s]);
    if (ctx->graphs[s])
      cudaGraphDestroy(ctx->graphs[s]);
  }
  if (ctx->stream)
  {
    cudaStreamSynchronize(ctx->stream);
    cudaStreamDestroy(ctx->stream);
  }
  for (int s = 0; s < dpc_ctx::kSide; ++s)
  {
    if (ctx->side[s])
    {
      cudaStreamSynchronize(ctx->side[s]);
      cudaStreamDestroy(ctx->side[s]);
    }
    if (ctx->join_ev[s])
      cudaEventDestroy(ctx->join_ev[s]);
  }
  if (ctx->fork_ev)
    cudaEventDestroy(ctx->fork_ev);
  delete ctx;
  return DPC_OK;
}

int dpc_set_precision(dpc_ctx* ctx, int precision)
{
  if (!ctx || (precision != DPC_PRECISION_FP32 && precision != DPC_PRECISION_TF32 &&
               precision != DPC_PRECISION_MIXED))
    return fail(DPC_ERR_INVALID, "dpc_set_precision: bad argument");
  ctx->precision = precision;
  return DPC_OK;
}

int dpc_get_precision(dpc_ctx* ctx)
{
  return ctx ? ctx->precision : DPC_ERR_INVALID;
}

void* dpc_stream(dpc_ctx* ctx)
{
  return ctx ? (void*)ctx->stream : nullptr;
}

int64_t dpc_launch_count(dpc_ctx* ctx)
{
  return ctx ? ctx->launches : 0;
}

int dpc_alloc(dpc_ctx* ctx, size_t bytes, void** out)
{
  if (!ctx || !out)
    return fail(DPC_ERR_INVALID, "dpc_alloc: null argument");
  DPC_CUDA(cudaSetDevice(ctx->device));
  DPC_CUDA(cudaMalloc(out, bytes ? bytes : 16));
  return DPC_OK;
}

int dpc_free(dpc_ctx* ctx, void* ptr)
{
  if (!ctx)
    return fail(DPC_ERR_INVALID, "dpc_free: null context");
  if (ptr)
    DPC_CUDA(cudaFree(ptr));
  return DPC_OK;
}

int dpc_zero(dpc_ctx* ctx, void* ptr, size_t bytes)
{
  if (!ctx || (!ptr && bytes))
    return fail(DPC_ERR_INVALID, "dpc_zero: null argument");
  DPC_CUDA(cudaMemsetAsync(ptr, 0, bytes, ctx->stream));
  return DPC_OK;
}

int dpc_copy_d2d(dpc_ctx* ctx, void* dst, const void* src, size_t bytes)
{
  if (!ctx)
    return fail(DPC_ERR_INVALID, "null context");
  DPC_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
  return DPC_OK;
}

int dpc_copy_h2d(dpc_ctx* ctx, void* dst, const void* host_src, size_t bytes)
{
  if (!ctx)
    return fail(DPC_ERR_INVALID, "null context");
  DPC_CUDA(cudaMemcpyAsync(dst, host_src, bytes, cudaMemcpyHostToDevice, ctx->stream));
  return DPC_OK;
}

int dpc_copy_d2h(dpc_ctx* ctx, void* host_dst, const void* src, size_t bytes)
{
  if (!ctx)
    return fail(DPC_ERR_INVALID, "null context");
  DPC_CUDA(cudaMemcpyAsync(host_dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  return DPC_OK;
}

int dpc_copy_h2d_sync(dpc_ctx* ctx, void* dst, const void* host_src, size_t bytes)
{
  int rc = dpc_copy_h2d(ctx, dst, host_src, bytes);
  if (rc != DPC_OK)
    return rc;
  DPC_CUDA(cudaStreamSynchronize(ctx->stream));
  return DPC_OK;
}

int dpc_copy_d2h_sync(dpc_ctx* ctx, void* host_dst, const void* src, size_t bytes)
{
  int rc = dpc_copy_d2h(ctx, host_dst, src, bytes);
  if (rc != DPC_OK)
    return rc;
  DPC_CUDA(cudaStreamSynchronize(ctx->stream));
  return DPC_OK;
}

int dpc_alloc_host(dpc_ctx* ctx, size_t bytes, void** out)
{
  if (!ctx || !out)
    return fail(DPC_ERR_INVALID, "dpc_alloc_host: null argument");
  DPC_CUDA(cudaMallocHost(out, bytes ? bytes : 16));
  return DPC_OK;
}

int dpc_free_host(dpc_ctx* ctx, void* ptr)
{
  (void)ctx;
  if (ptr)
    DPC_CUDA(cudaFreeHost(ptr));
  return DPC_OK;
}

int dpc_sync(dpc_ctx* ctx)
{
  if (!ctx)
    return fail(DPC_ERR_INVALID, "null context");
  DPC_CUDA(cudaStreamSynchronize(ctx->stream));
  return DPC_OK;
}

namespace dpc
{
__global__ void gather_rows_kernel(const float* __restrict__ src, const int64_t* __restrict__ index,
                                   int64_t first, int rows, int64_t cols, float* __restrict__ dst,
                                   int vec)
{
  const int64_t per_row = vec ? cols / 4 : cols;
  const int64_t total = (int64_t)rows * per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x)
  {
    const int64_t r = i / per_row, c = i - r * per_row;
    const int64_t s = index[first + r];
    if (vec)
      reinterpret_cast<float4*>(dst + r * cols)[c] =
          __ldg(reinterpret_cast<const float4*>(src + s * cols) + c);
    else
      dst[r * cols + c] = src[s * cols + c];
  }
}
} // namespace dpc

int dpc_gather_rows(dpc_ctx* ctx, const float* src_dev, const int64_t* index_dev, int64_t first,
                    int rows, int64_t cols, float* dst_dev)
{
  if (!ctx || !src_dev || !index_dev || !dst_dev || rows < 0 || cols <= 0 || first < 0)
    return fail(DPC_ERR_INVALID, "dpc_gather_rows: bad argument");
  if (rows == 0)
    return DPC_OK;
  const int vec = cols % 4 == 0 && ((uintptr_t)src_dev % 16) == 0 && ((uintptr_t)dst_dev % 16) == 0;
  const int64_t total = (int64_t)rows * (vec ? cols / 4 : cols);
  const int blocks = (int)std::min<int64_t>((total + 255) / 256, (int64_t)ctx->sm_count * 16);
  dpc::gather_rows_kernel<<<blocks, 256, 0, ctx->stream>>>(src_dev, index_dev, first, rows, cols,
                                                          dst_dev, vec);
  return check_launch(ctx, "gather_rows kernel");
}

int dpc_graph_begin(dpc_ctx* ctx, int slot)
{
  if (!ctx || slot < 0 || slot >= dpc_ctx::kSlots)
    return fail(DPC_ERR_INVALID, "dpc_graph_begin: bad slot");
  if (ctx->capturing_slot >= 0)
    return fail(DPC_ERR_STATE, "dpc_graph_begin: a capture is already open");
  DPC_CUDA(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
  ctx->capturing_slot = slot;
  ctx->launches_at_begin = ctx->launches;
  return DPC_OK;
}

int dpc_graph_end(dpc_ctx* ctx, int slot)
{
  if (!ctx || slot != ctx->capturing_slot)
    return fail(DPC_ERR_STATE, "dpc_graph_end: slot does not match the open capture");
  ctx->capturing_slot = -1;
  // Recorded launches run when the graph is replayed, not now.
  ctx->graph_kernels[slot] = ctx->launches - ctx->launches_at_begin;
  ctx->launches = ctx->launches_at_begin;
  cudaGraph_t graph = nullptr;
  DPC_CUDA(cudaStreamEndCapture(ctx->stream, &graph));
  if (ctx->execs[slot])
    cudaGraphExecDestroy(ctx->execs[slot]);
  if (ctx->graphs[slot])
    cudaGraphDestroy(ctx->graphs[slot]);
  ctx->execs[slot] = nullptr;
  ctx->graphs[slot] = graph;
  DPC_CUDA(cudaGraphInstantiate(&ctx->execs[slot], graph, 0));
  return DPC_OK;
}

int dpc_graph_launch(dpc_ctx* ctx, int slot)
{
  if (!ctx || slot < 0 || slot >= dpc_ctx::kSlots || !ctx->execs[slot])
    return fail(DPC_ERR_STATE, "dpc_graph_launch: nothing captured in this slot");
  DPC_CUDA(cudaGraphLaunch(ctx->execs[slot], ctx->stream));
  ctx->launches += ctx->graph_kernels[slot];
  return DPC_OK;
}

int dpc_graph_drop(dpc_ctx* ctx, int slot)
{
  if (!ctx || slot < 0 || slot >= dpc_ctx::kSlots)
    return fail(DPC_ERR_INVALID, "dpc_graph_drop: bad slot");
  if (ctx->execs[slot])
    cudaGraphExecDestroy(ctx->execs[slot]);
  if (ctx->graphs[slot])
    cudaGraphDestroy(ctx->graphs[slot]);
  ctx->execs[slot] = nullptr;
  ctx->graphs[slot] = nullptr;
  return DPC_OK;
}

// ------------------------------------------------------------------------------ plans
static int validate_layers(const dpc_layer* layers, int n, int batch)
{
  if (!layers || n < 2 || batch <= 0)
    return fail(DPC_ERR_INVALID, "plan: need at least two layers and a positive batch");
  for (int i = 0; i < n; ++i)
  {
    const dpc_layer& L = layers[i];
    if (L.size <= 0 || !L.z || !L.e)
      return fail(DPC_ERR_INVALID, "plan: layer " + std::to_string(i) + " lacks z/e or size");
    if (i + 1 < n)
    {
      if (L.next_size != layers[i + 1].size)
        return fail(DPC_ERR_INVALID, "plan: next_size of layer " + std::to_string(i) +
                                         " does not match the size of the layer above");
      if (!L.W || !L.b || !L.mu)
        return fail(DPC_ERR_INVALID, "plan: layer " + std::to_string(i) + " lacks W/b/mu");
      const bool simple = (L.flags & DPC_LAYER_INPUT_ACT) != 0;
      if (!simple && (!L.preact || !L.fe))
        return fail(DPC_ERR_INVALID, "plan: layer " + std::to_string(i) + " lacks preact/fe");
      if (simple && !L.zF)
        return fail(DPC_ERR_INVALID, "plan: SimplePC layer " + std::to_string(i) + " lacks zF");
      if ((L.flags & DPC_LAYER_RESIDUAL) && L.size != L.next_size)
        return fail(DPC_ERR_INVALID, "plan: residual layer must be square");
      if (L.opt != DPC_OPT_SGD && (!L.m_W || !L.v_W || !L.m_b || !L.v_b || !L.t))
        return fail(DPC_ERR_INVALID, "plan: Adam state missing on layer " + std::to_string(i));
      if (L.Psi && L.opt_psi != DPC_OPT_SGD && (!L.m_Psi || !L.v_Psi || !L.t_Psi))
        return fail(DPC_ERR_INVALID, "plan: Psi Adam state missing on layer " + std::to_string(i));
      // (the last layer of a layer-sharded block is not the terminal: only the stride is checked)
      if (L.Psi && (L.psi_stride < L.terminal_size || L.terminal_size <= 0))
        return fail(DPC_ERR_INVALID, "plan: terminal_size / psi_stride mismatch on layer " +
                                         std::to_string(i));
    }
    else if (L.next_size != 0)
      return fail(DPC_ERR_INVALID, "plan: the last layer must be weight-less (next_size 0)");
  }
  return DPC_OK;
}

int dpc_plan_create(dpc_ctx* ctx, const dpc_layer* layers, int n_layers, int batch,
                    dpc_plan** out)
{
  if (!ctx || !out)
    return fail(DPC_ERR_INVALID, "dpc_plan_create: null argument");
  int rc = validate_layers(layers, n_layers, batch);
  if (rc != DPC_OK)
    return rc;
  auto* p = new dpc_plan();
  p->ctx = ctx;
  p->n = n_layers;
  p->batch = batch;
  p->h.assign(layers, layers + n_layers);
  p->e_terminal = layers[n_layers - 1].e;
  cudaError_t err = cudaMalloc(&p->d, sizeof(dpc_layer) * n_layers);
  if (err == cudaSuccess)
    err = cudaMalloc(&p->energy, sizeof(double));
  if (err == cudaSuccess)
    err = cudaMallocHost(&p->energy_host, sizeof(double));
  if (err == cudaSuccess)
    err = cudaMemcpy(p->d, layers, sizeof(dpc_layer) * n_layers, cudaMemcpyHostToDevice);
  if (err == cudaSuccess)
    err = cudaMemset(p->energy, 0, sizeof(double));
  if (err != cudaSuccess)
  {
    dpc_plan_destroy(p);
    return cuda_fail(err, "dpc_plan_create");
  }
  rc = tc_plan_init(p);
  if (rc < 0)
  {
    dpc_plan_destroy(p);
    return rc;
  }
  *out = p;
  return DPC_OK;
}

int dpc_plan_update(dpc_plan* p, const dpc_layer* layers, int n_layers)
{
  if (!p || n_layers != p->n)
    return fail(DPC_ERR_INVALID, "dpc_plan_update: layer count differs from the plan");
  int rc = validate_layers(layers, n_layers, p->batch);
  if (rc != DPC_OK)
    return rc;
  DPC_CUDA(cudaStreamSynchronize(p->ctx->stream));
  if (p->e_terminal == p->h[p->n - 1].e)
    p->e_terminal = layers[n_layers - 1].e;
  p->h.assign(layers, layers + n_layers);
  DPC_CUDA(cudaMemcpy(p->d, layers, sizeof(dpc_layer) * n_layers, cudaMemcpyHostToDevice));
  tc_plan_free(p);
  rc = tc_plan_init(p);
  return rc < 0 ? rc : DPC_OK;
}

int dpc_plan_destroy(dpc_plan* p)
{
  if (!p)
    return DPC_OK;
  tc_plan_free(p);
  if (p->d)
    cudaFree(p->d);
  if (p->energy)
    cudaFree(p->energy);
  if (p->energy_host)
    cudaFreeHost(p->energy_host);
  delete p;
  return DPC_OK;
}

int dpc_plan_set_terminal_error(dpc_plan* p, const float* e_terminal_dev)
{
  if (!p)
    return fail(DPC_ERR_INVALID, "null plan");
  p->e_terminal = e_terminal_dev ? e_terminal_dev : p->h[p->n - 1].e;
  return DPC_OK;
}

int dpc_plan_set_chain_trace(dpc_plan* p, void* trace_dev)
{
  if (!p)
    return fail(DPC_ERR_INVALID, "null plan");
  tc_set_chain_trace(p, static_cast<unsigned long long*>(trace_dev));
  return DPC_OK;
}

int dpc_plan_tensor_run(dpc_plan* p, int* first, int* count)
{
  if (!p)
    return fail(DPC_ERR_INVALID, "null plan");
  if (first)
    *first = p->run.first;
  if (count)
    *count = p->run.count;
  return DPC_OK;
}

int dpc_plan_describe(dpc_plan* p, char* buf, int buf_bytes)
{
  if (!p || !buf || buf_bytes <= 0)
    return fail(DPC_ERR_INVALID, "dpc_plan_describe: null argument");
  const std::string d = tc_describe(p);
  snprintf(buf, (size_t)buf_bytes, "%s", d.c_str());
  return DPC_OK;
}

int dpc_plan_invalidate(dpc_plan* p, int first, int count, int what)
{
  int rc = check_range(p, first, count);
  if (rc != DPC_OK)
    return rc;
  if (what & DPC_WROTE_Z)
    tc_touch(p, 0, first, count);
  if (what & DPC_WROTE_FE)
    tc_touch(p, 1, first, count);
  if (what & DPC_WROTE_W)
    tc_touch(p, 2, first, count);
  return DPC_OK;
}

int dpc_plan_sync_operands(dpc_plan* p)
{
  if (!p)
    return fail(DPC_ERR_INVALID, "null plan");
  return tc_sync_planes(p);
}

int dpc_plan_set_wait_limit(dpc_plan* p, double milliseconds, int sweep_target_bias)
{
  if (!p)
    return fail(DPC_ERR_INVALID, "null plan");
  cudaDeviceProp prop;
  DPC_CUDA(cudaGetDeviceProperties(&prop, p->ctx->device));
  // clock64() counts SM clocks; take the maximum clock so the limit is never shorter than asked
  const long long cycles =
      milliseconds > 0.0 ? (long long)(milliseconds * 1e-3 * (double)prop.clockRate * 1e3) : 0;
  tc_set_wait_limit(p, cycles, sweep_target_bias);
  return DPC_OK;
}

// ------------------------------------------------------------------------------ phases
// The CUDA-core kernels write the fp32 tensors only: tell the tensor-core path which of its
// operand planes have gone stale.
static void wrote(dpc_plan* p, int kind, int first, int count)
{
  if (p->run.count > 0 && count > 0)
    tc_touch(p, kind, first, count);
}
enum
{
  K_Z = 0,
  K_FE = 1,
  K_W = 2
};

static FePlanes fe_planes(dpc_plan* p)
{
  FePlanes P;
  void* base = nullptr;
  tc_fe_planes(p, &base, &P.run_first, &P.run_count, &P.elems, &P.only);
  P.fe = static_cast<__nv_bfloat16*>(base);
  return P;
}

static int forward_simt(dpc_plan* p, int first, int count, int flags)
{
  cudaStream_t st = p->ctx->stream;
  for (int f = first; f < first + count; f += kMaxZ)
  {
    const int c = std::min(kMaxZ, first + count - f);
    if (flags & DPC_FWD_CACHED)
    {
      size_t mx = 0;
      for (int i = f; i < f + c; ++i)
        mx = std::max(mx, (size_t)p->batch * std::max(p->h[i].next_size, 0));
      dim3 grid(elem_blocks(p, mx), c);
      cached_forward_kernel<<<grid, NTHREADS, 0, st>>>(p->d, f, p->n, p->batch, flags, p->energy);
    }
    else
    {
      int tx, ty;
      max_tiles(p, f, c, OP_FWD, tx, ty);
      if (tx == 0)
        continue;
      // heads (at most 16 output units) with vector-loadable rows: one warp per batch row
      bool narrow = true;
      for (int i = f; i < f + c && narrow; ++i)
      {
        const dpc_layer& L = p->h[i];
        if (L.next_size <= 0)
          continue;
        narrow = L.next_size <= 16 && L.size % 4 == 0 && L.size >= 128 &&
                 !(L.flags & DPC_LAYER_INPUT_ACT) && ((uintptr_t)L.z % 16) == 0 &&
                 ((uintptr_t)L.W % 16) == 0;
      }
      if (narrow)
      {
        if (p->batch >= 2048)
        {
          dim3 grid(cdiv(p->batch, 2 * (NTHREADS / 32)), 1, c);
          narrow_forward_kernel<2><<<grid, NTHREADS, 0, st>>>(p->d, f, p->n, p->batch, flags, p->energy);
        }
        else
        {
          dim3 grid(cdiv(p->batch, NTHREADS / 32), 1, c);
          narrow_forward_kernel<1><<<grid, NTHREADS, 0, st>>>(p->d, f, p->n, p->batch, flags, p->energy);
        }
      }
      else
      {
        dim3 grid(tx, ty, c);
        pc_gemm_kernel<OP_FWD><<<grid, NTHREADS, 0, st>>>(p->d, f, p->n, p->batch, flags, 0,
                                                         p->energy);
      }
    }
    int rc = check_launch(p->ctx, "forward kernel");
    if (rc != DPC_OK)
      return rc;
  }
  if (flags & DPC_FWD_FE)
    wrote(p, K_FE, first, count);
  if (flags & DPC_FWD_COPY_NEXT)
    wrote(p, K_Z, first + 1, count);
  return DPC_OK;
}

// Splits [first, first+count) into what the tensor-core path takes (the part inside the run as
// one piece, single layers outside it that fit the CTA-pair kernels one by one) and maximal
// pieces for the CUDA-core kernels.  A piece the tensor-core entry point declines (returns 1)
// goes to the CUDA-core kernels too.
// `independent`: the layers of the range neither read what another layer of the range writes nor
// write the same tensors (true of a settle pass, a state update and a weight update; not of a
// sweep).  Consecutive single layers on the tensor cores then go to up to four streams that fork
// from and join the context's stream (inside a graph capture: parallel branches), because one such
// layer alone fills only a part of the GPU.
template <typename TcFn, typename SimtFn>
static int dispatch_range(dpc_plan* p, int first, int count, TcFn tc, SimtFn simt,
                          bool independent = false)
{
  const int end = first + count;
  const int run0 = p->run.first, run1 = p->run.first + p->run.count;
  dpc_ctx* ctx = p->ctx;
  int i = first;
  while (i < end)
  {
    int j, rc;
    if (independent && ctx->fork_ev && tc_extra_layer(p, i) && i + 1 < end &&
        tc_extra_layer(p, i + 1))
    {
      j = i + 2;
      while (j < end && tc_extra_layer(p, j))
        ++j;
      cudaStream_t main_stream = ctx->stream;
      const int used = std::min(j - i - 1, dpc_ctx::kSide);
      bool forked = cudaEventRecord(ctx->fork_ev, main_stream) == cudaSuccess;
      for (int s = 0; s < used && forked; ++s)
        forked = cudaStreamWaitEvent(ctx->side[s], ctx->fork_ev, 0) == cudaSuccess;
      if (!forked)
        return cuda_fail(cudaGetLastError(), "fork of the per-layer streams");
      rc = DPC_OK;
      for (int q = i; q < j && rc == DPC_OK; ++q)
      {
        const int lane = (q - i) % (used + 1);
        ctx->stream = lane == 0 ? main_stream : ctx->side[lane - 1];
        rc = tc(q, 1);
        if (rc > 0)
          rc = simt(q, 1);
      }
      ctx->stream = main_stream;
      // join whatever happened: a capture must not end with a stream still forked
      bool joined = true;
      for (int s = 0; s < used; ++s)
        joined &= cudaEventRecord(ctx->join_ev[s], ctx->side[s]) == cudaSuccess &&
                  cudaStreamWaitEvent(main_stream, ctx->join_ev[s], 0) == cudaSuccess;
      if (rc != DPC_OK)
        return rc;
      if (!joined)
        return cuda_fail(cudaGetLastError(), "join of the per-layer streams");
      i = j;
      continue;
    }
    if (p->run.count > 0 && i >= run0 && i < run1)
    {
      j = std::min(end, run1);
      rc = tc(i, j - i);
    }
    else if (tc_extra_layer(p, i))
    {
      j = i + 1;
      rc = tc(i, 1);
    }
    else
    {
      j = i + 1;
      while (j < end && !(p->run.count > 0 && j >= run0 && j < run1) && !tc_extra_layer(p, j))
        ++j;
      rc = 1;
    }
    if (rc < 0)
      return rc;
    if (rc != DPC_OK && (rc = simt(i, j - i)) != DPC_OK)
      return rc;
    i = j;
  }
  return DPC_OK;
}

int dpc_forward(dpc_plan* p, int first, int count, int flags)
{
  int rc = check_range(p, first, count);
  if (rc != DPC_OK)
    return rc;
  if (flags & DPC_FWD_CACHED)
    return forward_simt(p, first, count, flags);
  return dispatch_range(
      p, first, count, [&](int f, int c) { return tc_forward(p, f, c, flags); },
      [&](int f, int c) { return forward_simt(p, f, c, flags); },
      /*independent=*/!(flags & DPC_FWD_COPY_NEXT));
}

int dpc_project_forward(dpc_plan* p, int first, int count, int skip_last_copy)
{
  return dpc_project_forward_ex(p, first, count, skip_last_copy, 0);
}

int dpc_project_forward_ex(dpc_plan* p, int first, int count, int skip_last_copy, int extra)
{
  extra &= DPC_FWD_NO_MU | DPC_FWD_NO_PREACT;
  int rc = check_range(p, first, count);
  if (rc != DPC_OK)
    return rc;
  int i0 = first;
  // The part of the sweep inside the tensor-core run goes out as one persistent launch.
  if (p->run.count > 0 && first <= p->run.first && first + count >= p->run.first + p->run.count &&
      !(skip_last_copy && p->run.first + p->run.count + 1 == p->n))
  {
    for (int i = first; i < p->run.first; ++i)
      if ((rc = dpc_forward(p, i, 1, DPC_FWD_COPY_NEXT | (i == first ? 0 : extra))) != DPC_OK)
        return rc;
    // (the chain kernel itself keeps mu of the sweep's very first layer when it starts there)
    rc = tc_project_forward(p, p->run.first, p->run.count,
                            DPC_FWD_COPY_NEXT | extra | (p->run.first == first ? (1 << 10) : 0));
    if (rc < 0)
      return rc;
    i0 = rc == DPC_OK ? p->run.first + p->run.count : p->run.first;
  }
  for (int i = i0; i < first + count; ++i)
  {
    if (p->h[i].next_size <= 0)
      continue;
    int flags = DPC_FWD_COPY_NEXT | (i == first ? 0 : extra);
    if (skip_last_copy && i + 2 == p->n)
      flags = 0;
    rc = dpc_forward(p, i, 1, flags);
    if (rc != DPC_OK)
      return rc;
  }
  return DPC_OK;
}

int dpc_error(dpc_plan* p, int layer, int with_energy)
{
  int rc = check_range(p, layer, 1);
  if (rc != DPC_OK)
    return rc;
  if (layer == 0)
    return fail(DPC_ERR_INVALID, "dpc_error: the input layer has no prediction below it");
  const dpc_layer& L = p->h[layer];
  cudaStream_t st = p->ctx->stream;
  if (L.flags & DPC_LAYER_SOFTMAX_CE)
  {
    int blocks = std::min(cdiv(p->batch, NTHREADS / 32), p->ctx->sm_count * 8);
    softmax_ce_kernel<<<blocks, NTHREADS, 0, st>>>(p->d, layer, p->batch, with_energy, p->energy);
  }
  else
  {
    error_kernel<<<elem_blocks(p, (size_t)p->batch * L.size), NTHREADS, 0, st>>>(
        p->d, layer, p->batch, with_energy, p->energy);
  }
  return check_launch(p->ctx, "error kernel");
}

int dpc_feedback_error(dpc_plan* p, int first, int count)
{
  int rc = check_range(p, first, count);
  if (rc != DPC_OK || count == 0)
    return rc;
  for (int f = first; f < first + count; f += kMaxZ)
  {
    const int c = std::min(kMaxZ, first + count - f);
    size_t mx = 0;
    for (int i = f; i < f + c; ++i)
      mx = std::max(mx, (size_t)p->batch * std::max(p->h[i].next_size, 0));
    dim3 grid(elem_blocks(p, mx), c);
    feedback_error_kernel<<<grid, NTHREADS, 0, p->ctx->stream>>>(p->d, f, p->n, p->batch);
    if ((rc = check_launch(p->ctx, "feedback_error kernel")) != DPC_OK)
      return rc;
  }
  wrote(p, K_FE, first, count);
  return DPC_OK;
}

// Largest output width of layers [f, f+c) when every one of them is "narrow above" (1..16 output
// units, an input width that is a multiple of 128, 16-byte aligned tensors, a batch of at least 256
// rows: the layer under a head on a large batch), else 0.  Such layers have kernels of their own
// for the state update and the weight update (narrow_state_kernel, narrow_weight_kernel).
static int narrow_above(const dpc_plan* p, int f, int c)
{
  if (p->batch < 256)
    return 0;
  int widest = 0;
  for (int i = f; i < f + c; ++i)
  {
    const dpc_layer& L = p->h[i];
    const bool simple = (L.flags & DPC_LAYER_INPUT_ACT) != 0;
    const float* g = simple ? (i + 1 < p->n ? p->h[i + 1].e : nullptr) : L.fe;
    const float* zin = simple ? L.zF : L.z;
    if (L.next_size <= 0 || L.next_size > 16 || L.size % 128 != 0 || !g || !zin || !L.W || !L.z ||
        !L.e || ((uintptr_t)zin % 16) != 0 || ((uintptr_t)L.W % 16) != 0 || ((uintptr_t)L.z % 16) != 0 ||
        ((uintptr_t)L.e % 16) != 0 || (L.v && ((uintptr_t)L.v % 16) != 0) ||
        (i + 1 < p->n && p->h[i + 1].e && ((uintptr_t)p->h[i + 1].e % 16) != 0))
      return 0;
    widest = std::max(widest, L.next_size);
  }
  return widest;
}

static int update_state_simt(dpc_plan* p, int first, int count)
{
  cudaStream_t st = p->ctx->stream;
  wrote(p, K_Z, first, count);
  for (int f = first; f < first + count; f += kMaxZ)
  {
    const int c = std::min(kMaxZ, first + count - f);
    int tx, ty;
    // Layers whose upper neighbour does not exist are handled by the relax kernel below.
    int cg = (f + c == p->n) ? c - 1 : c;
    int narrow_kc = cg > 0 ? narrow_above(p, f, cg) : 0;
    if (narrow_kc > 0)
    {
      // layers under a narrow one (the heads): 128 columns x a share of the batch rows per block
      int mxs = 0;
      for (int i = f; i < f + cg; ++i)
        mxs = std::max(mxs, p->h[i].size);
      const int gx = cdiv(mxs, 128);
      int rpb = p->batch;
      while (rpb > 128 && (long long)gx * cg * cdiv(p->batch, rpb) < 2 * p->ctx->sm_count)
        rpb = cdiv(rpb / 2, 128) * 128;
      dim3 grid(gx, cdiv(p->batch, rpb), cg);
      if (narrow_kc <= 12)
        narrow_state_kernel<12><<<grid, 256, 0, st>>>(p->d, f, p->n, p->batch, rpb);
      else
        narrow_state_kernel<16><<<grid, 256, 0, st>>>(p->d, f, p->n, p->batch, rpb);
      int rc = check_launch(p->ctx, "narrow update_state kernel");
      if (rc != DPC_OK)
        return rc;
    }
    else if (cg > 0)
    {
      max_tiles(p, f, cg, OP_FB, tx, ty);
      if (tx > 0)
      {
        dim3 grid(tx, ty, cg);
        pc_gemm_kernel<OP_FB><<<grid, NTHREADS, 0, st>>>(p->d, f, p->n, p->batch, 0, 0, p->energy);
        int rc = check_launch(p->ctx, "update_state kernel");
        if (rc != DPC_OK)
          return rc;
      }
    }
    bool any_weightless = false;
    size_t mx = 0;
    for (int i = f; i < f + c; ++i)
      if (p->h[i].next_size <= 0 || i + 1 >= p->n)
      {
        any_weightless = true;
        mx = std::max(mx, (size_t)p->batch * p->h[i].size);
      }
    if (any_weightless)
    {
      dim3 grid(elem_blocks(p, mx), c);
      relax_kernel<<<grid, NTHREADS, 0, st>>>(p->d, f, p->n, p->batch, 1);
      int rc = check_launch(p->ctx, "relax kernel");
      if (rc != DPC_OK)
        return rc;
    }
  }
  return DPC_OK;
}

int dpc_update_state(dpc_plan* p, int first, int count)
{
  int rc = check_range(p, first, count);
  if (rc != DPC_OK)
    return rc;
  return dispatch_range(
      p, first, count, [&](int f, int c) { return tc_update_state(p, f, c); },
      [&](int f, int c) { return update_state_simt(p, f, c); }, /*independent=*/true);
}

int dpc_epc_reconstruct(dpc_plan* p, int layer)
{
  int rc = check_range(p, layer, 1);
  if (rc != DPC_OK)
    return rc;
  if (layer == 0)
    return fail(DPC_ERR_INVALID, "dpc_epc_reconstruct: the input layer has nothing below it");
  wrote(p, K_Z, layer, 1);
  epc_reconstruct_kernel<<<elem_blocks(p, (size_t)p->batch * p->h[layer].size), NTHREADS, 0,
                           p->ctx->stream>>>(p->d, layer, p->batch);
  return check_launch(p->ctx, "epc_reconstruct kernel");
}

int dpc_epc_adjoint(dpc_plan* p, int layer, int from_terminal, float scale, int clamped)
{
  int rc = check_range(p, layer, 1);
  if (rc != DPC_OK)
    return rc;
  const dpc_layer& L = p->h[layer];
  if (layer + 1 >= p->n || L.next_size <= 0 || !L.adj || !L.fe || !L.preact)
    return fail(DPC_ERR_INVALID, "dpc_epc_adjoint: layer has no weights, no adjoint buffer or no "
                                 "upper neighbour");
  const float* src = from_terminal ? p->h[p->n - 1].e : p->h[layer + 1].adj;
  if (!src)
    return fail(DPC_ERR_INVALID, "dpc_epc_adjoint: the layer above has no adjoint buffer");
  cudaStream_t st = p->ctx->stream;
  wrote(p, K_FE, layer, 1);
  epc_source_kernel<<<elem_blocks(p, (size_t)p->batch * L.next_size), NTHREADS, 0, st>>>(
      p->d, layer, p->batch, src);
  if ((rc = check_launch(p->ctx, "epc_source kernel")) != DPC_OK)
    return rc;
  // hop scale travels as float bits with the lowest mantissa bit replaced by the clamp flag
  // (scale is +1 or -1, whose lowest mantissa bit is zero)
  union
  {
    float f;
    int i;
  } u;
  u.f = scale;
  const int packed = (u.i & ~1) | (clamped ? 1 : 0);
  dim3 grid(cdiv(L.size, BN), cdiv(p->batch, BM), 1);
  pc_gemm_kernel<OP_FB><<<grid, NTHREADS, 0, st>>>(p->d, layer, p->n, p->batch, packed, FB_ADJOINT,
                                                  p->energy, src);
  return check_launch(p->ctx, "epc_adjoint kernel");
}

int dpc_relax(dpc_plan* p, int layer)
{
  int rc = check_range(p, layer, 1);
  if (rc != DPC_OK)
    return rc;
  dim3 grid(elem_blocks(p, (size_t)p->batch * p->h[layer].size), 1);
  wrote(p, K_Z, layer, 1);
  relax_kernel<<<grid, NTHREADS, 0, p->ctx->stream>>>(p->d, layer, p->n, p->batch, 0);
  return check_launch(p->ctx, "relax kernel");
}

static int weight_gemm_simt(dpc_plan* p, int first, int count, int mode, int flags)
{
  if (!(mode & WG_GRAD_ONLY))
    wrote(p, K_W, first, count);
  for (int f = first; f < first + count; f += kMaxZ)
  {
    const int c = std::min(kMaxZ, first + count - f);
    int tx, ty;
    const int narrow_kc = narrow_above(p, f, c);
    bool staged_ok = true;
    for (int i = f; i < f + c; ++i)
      staged_ok &= !(mode & WG_GRAD_ONLY) || (p->h[i].g_W != nullptr);
    if (narrow_kc > 0 && staged_ok)
    {
      // heads on a large batch: the batch split over warps and the CTAs of a cluster
      int mxs = 0;
      for (int i = f; i < f + c; ++i)
        mxs = std::max(mxs, p->h[i].size);
      dim3 g(cdiv(mxs, 128), c);
      const int R = row_split(p->ctx, (long long)g.x * c, p->batch, 256);
      if (narrow_kc <= 12)
        launch_row_split(narrow_weight_kernel<12>, g, 256, R, p->ctx->stream, p->d, f, p->n,
                         p->batch, flags, mode);
      else
        launch_row_split(narrow_weight_kernel<16>, g, 256, R, p->ctx->stream, p->d, f, p->n,
                         p->batch, flags, mode);
      int rc = check_launch(p->ctx, "narrow weight kernel");
      if (rc != DPC_OK)
        return rc;
      continue;
    }
    max_tiles(p, f, c, OP_WG, tx, ty);
    if (tx == 0)
      continue;
    dim3 grid(tx, ty, c);
    pc_gemm_kernel<OP_WG><<<grid, NTHREADS, 0, p->ctx->stream>>>(p->d, f, p->n, p->batch, flags,
                                                                mode, p->energy);
    int rc = check_launch(p->ctx, "weight kernel");
    if (rc != DPC_OK)
      return rc;
  }
  return DPC_OK;
}

// The DFA projection over layers [first, first+count): four-units-per-thread kernel where the
// shapes allow it, the general kernel elsewhere.
static int launch_dfa_proj(dpc_plan* p, int first, int count, int from_output)
{
  cudaStream_t st = p->ctx->stream;
  wrote(p, K_FE, first, count);
  const FePlanes planes = fe_planes(p);
  auto vec_ok = [&](int i)
  {
    const dpc_layer& L = p->h[i];
    return L.next_size > 0 && L.next_size % 4 == 0 && L.terminal_size <= 16 &&
           ((uintptr_t)L.fe % 16 == 0) && ((uintptr_t)L.preact % 16 == 0) &&
           (i + 1 >= p->n || (uintptr_t)p->h[i + 1].z % 16 == 0);
  };
  int i = first;
  while (i < first + count)
  {
    const bool v = vec_ok(i);
    int j = i + 1;
    while (j < first + count && j - i < kMaxZ && vec_ok(j) == v &&
           (!v || p->h[j].terminal_size == p->h[i].terminal_size))
      ++j;
    const int c = j - i;
    int mxn = 1;
    for (int k = i; k < j; ++k)
      mxn = std::max(mxn, p->h[k].next_size);
    bool wide = v;
    for (int k = i; k < j && wide; ++k)
      wide = p->h[k].next_size <= 0 || p->h[k].next_size % 128 == 0;
    const int ts4 = cdiv(std::max(p->h[i].terminal_size, 1), 4);
    if (wide && ts4 <= 4 && cdiv(mxn, 128) * c >= 2 * p->ctx->sm_count)
    {
      // blocks of 128 columns x the whole batch
      dim3 grid(cdiv(mxn, 128), c);
      if (ts4 <= 1)
        dfa_proj128_kernel<1><<<grid, 256, 0, st>>>(p->d, i, p->n, p->batch, p->e_terminal, from_output, planes);
      else if (ts4 == 2)
        dfa_proj128_kernel<2><<<grid, 256, 0, st>>>(p->d, i, p->n, p->batch, p->e_terminal, from_output, planes);
      else if (ts4 == 3)
        dfa_proj128_kernel<3><<<grid, 256, 0, st>>>(p->d, i, p->n, p->batch, p->e_terminal, from_output, planes);
      else
        dfa_proj128_kernel<4><<<grid, 256, 0, st>>>(p->d, i, p->n, p->batch, p->e_terminal, from_output, planes);
    }
    else if (v)
    {
      const int rpb =
          cdiv(mxn, 256) * cdiv(p->batch, DFA4_ROWS) * c >= 4 * p->ctx->sm_count ? DFA4_ROWS : 32;
      dim3 grid(cdiv(mxn, 256), cdiv(p->batch, rpb), c);
      if (ts4 <= 1)
        dfa_proj4_kernel<1><<<grid, 64, 0, st>>>(p->d, i, p->n, p->batch, p->e_terminal, from_output, rpb, planes);
      else if (ts4 == 2)
        dfa_proj4_kernel<2><<<grid, 64, 0, st>>>(p->d, i, p->n, p->batch, p->e_terminal, from_output, rpb, planes);
      else if (ts4 == 3)
        dfa_proj4_kernel<3><<<grid, 64, 0, st>>>(p->d, i, p->n, p->batch, p->e_terminal, from_output, rpb, planes);
      else
        dfa_proj4_kernel<4><<<grid, 64, 0, st>>>(p->d, i, p->n, p->batch, p->e_terminal, from_output, rpb, planes);
    }
    else
    {
      dim3 grid(cdiv(mxn, 128), cdiv(p->batch, DFA_ROWS), c);
      dfa_proj_kernel<<<grid, 128, 0, st>>>(p->d, i, p->n, p->batch, p->e_terminal, from_output);
    }
    int rc = check_launch(p->ctx, "dfa_proj kernel");
    if (rc != DPC_OK)
      return rc;
    if (v && planes.fe)
      tc_fe_written(p, i, c); // this kernel wrote the operand copies itself
    i = j;
  }
  return DPC_OK;
}

int dpc_direct_feedback(dpc_plan* p, int first, int count, int decay_w)
{
  int rc = check_range(p, first, count);
  if (rc != DPC_OK || count == 0)
    return rc;
  // Only layers with an upper neighbour can take part.
  if (first + count == p->n)
    count -= 1;
  if (count <= 0)
    return DPC_OK;
  if ((rc = launch_dfa_proj(p, first, count, (decay_w & DPC_DFA_FROM_OUTPUT) ? 1 : 0)) != DPC_OK)
    return rc;
  decay_w &= DPC_DFA_DECAY_W;
  const int flags = decay_w ? 1 : 0;
  return dispatch_range(
      p, first, count, [&](int f, int c) { return tc_weight_gemm(p, f, c, WG_DFA, decay_w); },
      [&](int f, int c) { return weight_gemm_simt(p, f, c, WG_DFA, flags); }, /*independent=*/true);
}

// Psi update (or its raw sums) of layers [f, f+c): the 128-columns-per-block kernel when every
// layer of the launch that has feedback weights is a multiple of 128 wide with at most 16
// terminal units, the general kernel otherwise.
static int launch_psi_update(dpc_plan* p, int f, int c, int max_size, int grad_only)
{
  cudaStream_t st = p->ctx->stream;
  bool fast = true;
  int ts = 0;
  for (int i = f; i < f + c && i < p->n; ++i)
  {
    const dpc_layer& L = p->h[i];
    if (L.next_size <= 0 || L.Psi == nullptr || (L.flags & DPC_LAYER_INPUT_ACT))
      continue;
    if (L.size % 128 != 0 || L.terminal_size > 16)
      fast = false;
    ts = std::max(ts, L.terminal_size);
  }
  if (fast && ts > 0)
  {
    dim3 g(std::max(1, cdiv(max_size, 128)), c);
    const int R = row_split(p->ctx, (long long)g.x * c, p->batch, 256);
    if (ts <= 12)
      launch_row_split(psi_update4_kernel<12>, g, 256, R, st, p->d, f, p->n, p->batch,
                       p->e_terminal, grad_only);
    else
      launch_row_split(psi_update4_kernel<16>, g, 256, R, st, p->d, f, p->n, p->batch,
                       p->e_terminal, grad_only);
  }
  else
  {
    dim3 g(std::max(1, cdiv(max_size, 64)), c);
    psi_update_kernel<<<g, 256, 0, st>>>(p->d, f, p->n, p->batch, p->e_terminal, grad_only);
  }
  return check_launch(p->ctx, grad_only ? "psi gradient kernel" : "psi_update kernel");
}

int dpc_update_weights(dpc_plan* p, int first, int count, int center_rows)
{
  int rc = check_range(p, first, count);
  if (rc != DPC_OK || count == 0)
    return rc;
  if (first + count == p->n)
    count -= 1;
  if (count <= 0)
    return DPC_OK;
  cudaStream_t st = p->ctx->stream;
  bool any_adam = false, any_psi = false;
  int max_next = 0, max_size = 0;
  for (int i = first; i < first + count; ++i)
  {
    const dpc_layer& L = p->h[i];
    any_adam |= L.opt != DPC_OPT_SGD || (L.Psi && L.opt_psi != DPC_OPT_SGD);
    any_psi |= L.Psi != nullptr && !(L.flags & DPC_LAYER_INPUT_ACT);
    max_next = std::max(max_next, L.next_size);
    max_size = std::max(max_size, L.size);
  }
  if (any_adam)
  {
    bump_counters_kernel<<<cdiv(count, 256), 256, 0, st>>>(p->d, first, count, p->n);
    if ((rc = check_launch(p->ctx, "bump_counters kernel")) != DPC_OK)
      return rc;
  }
  rc = dispatch_range(
      p, first, count,
      [&](int f, int c) -> int
      {
        bool all_sgd = true, all_staged = true;
        for (int i = f; i < f + c; ++i)
        {
          all_sgd &= p->h[i].opt == DPC_OPT_SGD;
          all_staged &= p->h[i].g_W != nullptr;
        }
        if (all_sgd)
          return tc_weight_gemm(p, f, c, WG_LEARN);
        if (!all_staged)
          return 1;
        // Adam-type optimizers: tensor-core product into the staging buffer, then the
        // optimizer as an elementwise kernel over W (b and Psi follow below as usual).
        int r = tc_weight_gemm(p, f, c, WG_LEARN | WG_GRAD_ONLY);
        if (r != DPC_OK)
          return r;
        size_t max_w = 1;
        for (int i = f; i < f + c; ++i)
          max_w = std::max(max_w, (size_t)p->h[i].next_size * p->h[i].size);
        for (int g = f; g < f + c; g += kMaxZ)
        {
          const int cc = std::min(kMaxZ, f + c - g);
          dim3 grid(elem_blocks(p, max_w), cc);
          wrote(p, K_W, g, cc);
          apply_gradients_kernel<<<grid, NTHREADS, 0, p->ctx->stream>>>(p->d, g, p->n, p->batch, 2, 0);
          if ((r = check_launch(p->ctx, "apply_gradients kernel")) != DPC_OK)
            return r;
        }
        return DPC_OK;
      },
      [&](int f, int c) { return weight_gemm_simt(p, f, c, WG_LEARN, 0); }, /*independent=*/true);
  if (rc != DPC_OK)
    return rc;
  for (int f = first; f < first + count; f += kMaxZ)
  {
    const int c = std::min(kMaxZ, first + count - f);
    if ((rc = tc_fe_need(p, f, c)) != DPC_OK)
      return rc;
    const FePlanes fp = fe_planes(p);
    // 256 threads: blocks of 64 columns where the feedback error is read from its planes,
    // one column per thread (grid-stride) elsewhere
    const bool by_blocks = fp.only || p->batch >= kBiasBlockRows;
    dim3 gb(std::max(1, cdiv(max_next, by_blocks ? 64 : 256)), c);
    launch_row_split(bias_update_kernel, gb, 256,
                     by_blocks ? row_split(p->ctx, (long long)gb.x * c, p->batch, 256) : 1, st, p->d,
                     f, p->n, p->batch, 0, fp);
    if ((rc = check_launch(p->ctx, "bias_update kernel")) != DPC_OK)
      return rc;
    if (any_psi)
    {
      if ((rc = launch_psi_update(p, f, c, max_size, 0)) != DPC_OK)
        return rc;
    }
    if (center_rows)
    {
      dim3 gc(std::min(max_next, 1024), c);
      wrote(p, K_W, f, c);
      center_rows_kernel<<<gc, 256, 0, st>>>(p->d, f, p->n);
      if ((rc = check_launch(p->ctx, "center_rows kernel")) != DPC_OK)
        return rc;
    }
  }
  return DPC_OK;
}

static int staging_ready(dpc_plan* p, int first, int count, int which)
{
  for (int i = first; i < first + count; ++i)
  {
    const dpc_layer& L = p->h[i];
    if (L.next_size <= 0)
      continue;
    if (!L.g_W || (which == 0 && (!L.g_b || (L.Psi && !(L.flags & DPC_LAYER_INPUT_ACT) && !L.g_Psi))))
      return fail(DPC_ERR_INVALID, "layer has no gradient staging buffers");
  }
  return DPC_OK;
}

int dpc_weight_gradients(dpc_plan* p, int first, int count, int which)
{
  int rc = check_range(p, first, count);
  if (rc != DPC_OK || count == 0)
    return rc;
  if (which != 0 && which != 1)
    return fail(DPC_ERR_INVALID, "which must be 0 (learn) or 1 (direct feedback)");
  if (first + count == p->n)
    count -= 1;
  if (count <= 0)
    return DPC_OK;
  if ((rc = staging_ready(p, first, count, which)) != DPC_OK)
    return rc;
  cudaStream_t st = p->ctx->stream;
  if (which == 1)
  {
    if ((rc = launch_dfa_proj(p, first, count, 0)) != DPC_OK)
      return rc;
    return dispatch_range(
        p, first, count,
        [&](int f, int c) { return tc_weight_gemm(p, f, c, WG_DFA | WG_GRAD_ONLY); },
        [&](int f, int c) { return weight_gemm_simt(p, f, c, WG_DFA | WG_GRAD_ONLY, 0); },
        /*independent=*/true);
  }
  rc = dispatch_range(
      p, first, count,
      [&](int f, int c) { return tc_weight_gemm(p, f, c, WG_LEARN | WG_GRAD_ONLY); },
      [&](int f, int c) { return weight_gemm_simt(p, f, c, WG_LEARN | WG_GRAD_ONLY, 0); },
      /*independent=*/true);
  if (rc != DPC_OK)
    return rc;
  bool any_psi = false;
  int max_next = 0, max_size = 0;
  for (int i = first; i < first + count; ++i)
  {
    const dpc_layer& L = p->h[i];
    any_psi |= L.Psi != nullptr && !(L.flags & DPC_LAYER_INPUT_ACT);
    max_next = std::max(max_next, L.next_size);
    max_size = std::max(max_size, L.size);
  }
  for (int f = first; f < first + count; f += kMaxZ)
  {
    const int c = std::min(kMaxZ, first + count - f);
    if ((rc = tc_fe_need(p, f, c)) != DPC_OK)
      return rc;
    const FePlanes fp = fe_planes(p);
    const bool by_blocks = fp.only || p->batch >= kBiasBlockRows;
    dim3 gb(std::max(1, cdiv(max_next, by_blocks ? 64 : 256)), c);
    launch_row_split(bias_update_kernel, gb, 256,
                     by_blocks ? row_split(p->ctx, (long long)gb.x * c, p->batch, 256) : 1, st, p->d,
                     f, p->n, p->batch, 1, fp);
    if ((rc = check_launch(p->ctx, "bias gradient kernel")) != DPC_OK)
      return rc;
    if (any_psi)
    {
      if ((rc = launch_psi_update(p, f, c, max_size, 1)) != DPC_OK)
        return rc;
    }
  }
  return DPC_OK;
}

int dpc_apply_gradients(dpc_plan* p, int first, int count, int which, int global_batch, int option)
{
  int rc = check_range(p, first, count);
  if (rc != DPC_OK || count == 0)
    return rc;
  if ((which != 0 && which != 1) || global_batch <= 0)
    return fail(DPC_ERR_INVALID, "bad which / global_batch");
  if (first + count == p->n)
    count -= 1;
  if (count <= 0)
    return DPC_OK;
  if ((rc = staging_ready(p, first, count, which)) != DPC_OK)
    return rc;
  cudaStream_t st = p->ctx->stream;
  bool any_adam = false;
  int max_next = 0;
  size_t max_w = 1;
  for (int i = first; i < first + count; ++i)
  {
    const dpc_layer& L = p->h[i];
    any_adam |= L.opt != DPC_OPT_SGD || (L.Psi && L.opt_psi != DPC_OPT_SGD);
    max_next = std::max(max_next, L.next_size);
    max_w = std::max(max_w, (size_t)std::max(L.next_size, 0) * L.size);
  }
  if (which == 0 && any_adam)
  {
    bump_counters_kernel<<<cdiv(count, 256), 256, 0, st>>>(p->d, first, count, p->n);
    if ((rc = check_launch(p->ctx, "bump_counters kernel")) != DPC_OK)
      return rc;
  }
  for (int f = first; f < first + count; f += kMaxZ)
  {
    const int c = std::min(kMaxZ, first + count - f);
    dim3 grid(elem_blocks(p, max_w), c);
    wrote(p, K_W, f, c);
    apply_gradients_kernel<<<grid, NTHREADS, 0, st>>>(p->d, f, p->n, global_batch, which, option ? 1 : 0);
    if ((rc = check_launch(p->ctx, "apply_gradients kernel")) != DPC_OK)
      return rc;
    if (which == 0 && option)
    {
      dim3 gc(std::min(max_next, 1024), c);
      center_rows_kernel<<<gc, 256, 0, st>>>(p->d, f, p->n);
      if ((rc = check_launch(p->ctx, "center_rows kernel")) != DPC_OK)
        return rc;
    }
  }
  return DPC_OK;
}

int dpc_energy_reset(dpc_plan* p)
{
  if (!p)
    return fail(DPC_ERR_INVALID, "null plan");
  DPC_CUDA(cudaMemsetAsync(p->energy, 0, sizeof(double), p->ctx->stream));
  return DPC_OK;
}

int dpc_energy_read(dpc_plan* p, double* out)
{
  if (!p || !out)
    return fail(DPC_ERR_INVALID, "null argument");
  DPC_CUDA(cudaMemcpyAsync(p->energy_host, p->energy, sizeof(double), cudaMemcpyDeviceToHost,
                           p->ctx->stream));
  DPC_CUDA(cudaStreamSynchronize(p->ctx->stream));
  *out = *p->energy_host;
  return tc_check_error(p);
}
