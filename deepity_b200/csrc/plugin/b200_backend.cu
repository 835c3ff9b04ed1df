// Device side of the DeepityCUDA plugin: every primitive of the reference's compute-backend
// interface (include/deepity/backend/IComputeBackend.h:18-625) as CUDA kernels for sm_100a.
// The semantics of each primitive follow the interface's own documentation and the reference's
// CPU implementation (src/backend/CPUBackend.cpp), which is the parity target.
//
// GEMMs of tile-aligned shapes run on the tensor cores (tcgen05.mma kind::tf32, operands staged
// by TMA, accumulators in tensor memory: b200_gemm_tc.cuh) when TF32 is allowed, the way the
// reference's own GPU backend defaults to TF32 (src/backend/cuda/CUDABackendCore.cu:54-67);
// everything else, and every GEMM after SetAllowTF32(false), runs on an fp32 CUDA-core kernel.
#include "b200_backend.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

#include "b200_gemm_tc.cuh"

namespace b200
{
namespace
{
constexpr int kThreads = 256;
constexpr int kPartials = 1024; // per-block partial sums of the two-pass reductions

#define B200_CHECK(call)                                                                         \
  do                                                                                             \
  {                                                                                              \
    cudaError_t err__ = (call);                                                                  \
    if (err__ != cudaSuccess)                                                                    \
      fprintf(stderr, "DeepityCUDA (b200): %s failed: %s\n", #call, cudaGetErrorString(err__)); \
  } while (0)

inline int blocks_for(size_t n, int cap)
{
  size_t b = (n + kThreads - 1) / kThreads;
  return (int)std::max<size_t>(1, std::min<size_t>(b, (size_t)cap));
}

// ---- activations: the reference's scalar definitions (include/deepity/utils/Activations.h:44-151)
constexpr float kGelu1 = 0.7978845608f, kGelu2 = 0.044715f;
enum
{
  A_RELU = 0,
  A_GELU = 2,
  A_SIGMOID = 4,
  A_ESIGMOID = 6,
  A_TANH = 8,
  A_LINEAR = 10,
  A_HARD_TANH = 12
};

__device__ __forceinline__ float act_forward(int type, float z)
{
  switch (type)
  {
  case A_RELU:
    return z > 0.0f ? z : 0.0f;
  case A_GELU:
  {
    const float inner = kGelu1 * z + (kGelu2 * kGelu1) * z * z * z;
    return 0.5f * z * (1.0f + tanhf(inner));
  }
  case A_SIGMOID:
    return 1.0f / (1.0f + expf(-z));
  case A_ESIGMOID:
    return 0.5f + 0.5f * (z / (1.0f + fabsf(z)));
  case A_TANH:
    return tanhf(z);
  case A_HARD_TANH:
    return fminf(fmaxf(z, -1.0f), 1.0f);
  default:
    return z;
  }
}

// dtype: derivative-flavoured enumerator (forward + 1)
__device__ __forceinline__ float act_derivative(int dtype, float z)
{
  switch (dtype - 1)
  {
  case A_RELU:
    return z > 0.0f ? 1.0f : 0.0f;
  case A_GELU:
  {
    const float zsq = z * z;
    const float t = tanhf(kGelu1 * z + (kGelu2 * kGelu1) * zsq * z);
    const float gprime = kGelu1 + (3.0f * kGelu2 * kGelu1) * zsq;
    return 0.5f * (1.0f + t) + 0.5f * z * gprime * (1.0f - t * t);
  }
  case A_SIGMOID:
  {
    const float s = 1.0f / (1.0f + expf(-z));
    return s * (1.0f - s);
  }
  case A_ESIGMOID:
  {
    const float a = 1.0f + fabsf(z);
    return 0.5f / (a * a);
  }
  case A_TANH:
  {
    const float t = tanhf(z);
    return 1.0f - t * t;
  }
  case A_HARD_TANH:
    return (z > -1.0f && z < 1.0f) ? 1.0f : 0.0f;
  default:
    return 1.0f;
  }
}

// from the activated value (Activations.h:117-140; GELU has no closed form: its argument is
// treated as the pre-activation, as the reference does)
__device__ __forceinline__ float act_derivative_from_activated(int dtype, float a)
{
  switch (dtype - 1)
  {
  case A_RELU:
    return a > 0.0f ? 1.0f : 0.0f;
  case A_GELU:
    return act_derivative(dtype, a);
  case A_SIGMOID:
    return a * (1.0f - a);
  case A_ESIGMOID:
    return 2.0f * a * (1.0f - a);
  case A_TANH:
    return 1.0f - a * a;
  case A_HARD_TANH:
    return (a > -1.0f && a < 1.0f) ? 1.0f : 0.0f;
  default:
    return 1.0f;
  }
}

#define GRID_STRIDE(i, n)                                                                        \
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < (n);                        \
       i += (size_t)gridDim.x * blockDim.x)

// ------------------------------------------------------------------------------ elementwise
__global__ void k_scale(float* buf, size_t n, float alpha)
{
  GRID_STRIDE(i, n) buf[i] *= alpha;
}
__global__ void k_axpy(float* y, const float* x, size_t n, float alpha)
{
  GRID_STRIDE(i, n) y[i] += alpha * x[i];
}
__global__ void k_fill(float* buf, size_t n, float v)
{
  GRID_STRIDE(i, n) buf[i] = v;
}
__global__ void k_multiply(float* dst, const float* a, const float* b, size_t n)
{
  GRID_STRIDE(i, n) dst[i] = a[i] * b[i];
}
// buf[l][row][col] += bias[l][col]
__global__ void k_add_bias(float* buf, const float* bias, size_t batch, size_t width, size_t layers)
{
  const size_t per = batch * width, n = per * layers;
  GRID_STRIDE(i, n)
  {
    const size_t l = i / per, col = (i - l * per) % width;
    buf[i] += bias[l * width + col];
  }
}
// buf[b][c][s] += bias[c]
__global__ void k_add_bias_channel(float* buf, const float* bias, size_t batch, size_t channels,
                                   size_t spatial)
{
  const size_t n = batch * channels * spatial;
  GRID_STRIDE(i, n) buf[i] += bias[(i / spatial) % channels];
}
__global__ void k_axpy_broadcast(float* y, const float* x, const float* factor, size_t n, size_t width,
                                 float alpha)
{
  GRID_STRIDE(i, n) y[i] += alpha * x[i] * factor[i % width];
}
__global__ void k_multiply_broadcast(float* dst, const float* a, const float* factor, const float* b,
                                     size_t n, size_t width)
{
  GRID_STRIDE(i, n) dst[i] = a[i] * factor[i % width] * b[i];
}
__global__ void k_activation(int type, float* dst, const float* src, size_t n)
{
  GRID_STRIDE(i, n) dst[i] = act_forward(type, src[i]);
}
__global__ void k_activation_derivative(int dtype, float* dst, const float* src, size_t n,
                                        int from_activated)
{
  GRID_STRIDE(i, n)
  dst[i] = from_activated ? act_derivative_from_activated(dtype, src[i]) : act_derivative(dtype, src[i]);
}
__global__ void k_derivative_multiply(int dtype, float* dst, const float* a, float* x, size_t n,
                                      int from_activated, int write_back)
{
  GRID_STRIDE(i, n)
  {
    const float d = from_activated ? act_derivative_from_activated(dtype, x[i]) : act_derivative(dtype, x[i]);
    dst[i] = a[i] * d;
    if (write_back)
      x[i] = d;
  }
}
// z += ir * (feedback * f'(z) - e), optionally through the momentum buffer v
// (src/backend/CPUBackend.cpp:565-600)
__global__ void k_state_update(float* z, float* v, const float* feedback, int dtype, const float* e,
                               size_t n, float ir, float beta)
{
  GRID_STRIDE(i, n)
  {
    const float update = feedback[i] * act_derivative(dtype, z[i]) - e[i];
    if (v)
    {
      const float vv = beta * v[i] + (1.0f - beta) * update;
      v[i] = vv;
      z[i] += ir * vv;
    }
    else
      z[i] += ir * update;
  }
}
__global__ void k_error(float* e, const float* z, const float* mu, size_t n)
{
  GRID_STRIDE(i, n) e[i] = z[i] - mu[i];
}
__global__ void k_error_activation(int type, float* e, float* zf, const float* z, const float* mu,
                                   size_t n)
{
  GRID_STRIDE(i, n)
  {
    const float zi = z[i];
    e[i] = zi - mu[i];
    zf[i] = act_forward(type, zi);
  }
}
__global__ void k_precision_error(float* e, const float* z, const float* mu, size_t n)
{
  GRID_STRIDE(i, n) e[i] = z[i] - mu[i];
}

// ------------------------------------------------------------------------------ reductions
__device__ __forceinline__ double block_sum(double v)
{
  __shared__ double warp_sums[kThreads / 32];
  for (int o = 16; o > 0; o >>= 1)
    v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0)
    warp_sums[threadIdx.x >> 5] = v;
  __syncthreads();
  double s = 0.0;
  if (threadIdx.x == 0)
    for (int w = 0; w < kThreads / 32; ++w)
      s += warp_sums[w];
  __syncthreads();
  return s; // valid on thread 0
}
// pass 1 of the reductions: one partial per block; mode 0 sum(buf), 1 e = z - mu and
// 0.5*sum(e^2), 2 the precision-weighted energy (p has `width` entries)
__global__ void k_reduce_partials(int mode, float* e, const float* a, const float* b, const float* p,
                                  size_t n, size_t width, double* partials)
{
  double acc = 0.0;
  GRID_STRIDE(i, n)
  {
    if (mode == 0)
      acc += (double)a[i];
    else
    {
      const float d = a[i] - b[i];
      e[i] = d;
      if (mode == 1)
        acc += 0.5 * (double)d * (double)d;
      else
      {
        const float pp = fmaxf(p[i % width], 1e-8f);
        acc += 0.5 * (double)pp * (double)d * (double)d - 0.5 * (double)logf(pp);
      }
    }
  }
  const double s = block_sum(acc);
  if (threadIdx.x == 0)
    partials[blockIdx.x] = s;
}
// pass 2: one block adds the partials up in a fixed order (reproducible)
__global__ void k_reduce_final(const double* partials, int count, double* out)
{
  double acc = 0.0;
  for (int i = threadIdx.x; i < count; i += blockDim.x)
    acc += partials[i];
  const double s = block_sum(acc);
  if (threadIdx.x == 0)
    *out = s;
}
// dst[l][j] = sum_b src[l][b][j]: one thread per column, rows in order (CPUBackend.cpp:243-252)
__global__ void k_sum_rows(float* dst, const float* src, size_t batch, size_t width)
{
  const size_t l = blockIdx.y;
  const float* s = src + l * batch * width;
  for (size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x; j < width;
       j += (size_t)gridDim.x * blockDim.x)
  {
    float acc = 0.0f;
    for (size_t b = 0; b < batch; ++b)
      acc += s[b * width + j];
    dst[l * width + j] = acc;
  }
}
// one block per row: subtract the row mean (CPUBackend.cpp:254-275)
__global__ void k_center_rows(float* buf, size_t rows, size_t cols)
{
  for (size_t r = blockIdx.x; r < rows; r += gridDim.x)
  {
    float* row = buf + r * cols;
    double acc = 0.0;
    for (size_t c = threadIdx.x; c < cols; c += blockDim.x)
      acc += (double)row[c];
    __shared__ float mean;
    const double s = block_sum(acc);
    if (threadIdx.x == 0)
      mean = (float)(s / (double)cols);
    __syncthreads();
    for (size_t c = threadIdx.x; c < cols; c += blockDim.x)
      row[c] -= mean;
    __syncthreads();
  }
}
// softmax cross-entropy error, one warp per row (CPUBackend.cpp:658-714):
// probs = softmax(mu); e = z - probs; row energy = -sum z log(probs + 1e-8)
__global__ void k_softmax_ce(float* e, const float* z, const float* mu, size_t batch, size_t width,
                             double* partials)
{
  const int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  double energy = 0.0;
  for (size_t row = (size_t)blockIdx.x * warps + (threadIdx.x >> 5); row < batch;
       row += (size_t)gridDim.x * warps)
  {
    const size_t base = row * width;
    float mx = -INFINITY;
    for (size_t j = lane; j < width; j += 32)
      mx = fmaxf(mx, mu[base + j]);
    for (int o = 16; o > 0; o >>= 1)
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float se = 0.0f;
    for (size_t j = lane; j < width; j += 32)
      se += expf(mu[base + j] - mx);
    for (int o = 16; o > 0; o >>= 1)
      se += __shfl_xor_sync(0xffffffffu, se, o);
    float re = 0.0f;
    for (size_t j = lane; j < width; j += 32)
    {
      const float prob = expf(mu[base + j] - mx) / se;
      re -= z[base + j] * logf(prob + 1e-8f);
      e[base + j] = z[base + j] - prob;
    }
    for (int o = 16; o > 0; o >>= 1)
      re += __shfl_xor_sync(0xffffffffu, re, o);
    if (lane == 0)
      energy += (double)re;
  }
  if (partials)
  {
    const double s = block_sum(lane == 0 ? energy : 0.0);
    if (threadIdx.x == 0)
      partials[blockIdx.x] = s;
  }
}
// p, log_p per position from the batch's squared errors (CPUBackend.cpp:1031-1050)
__global__ void k_update_precision(float* p, float* log_p, const float* e, size_t batch, size_t width,
                                   float pr)
{
  GRID_STRIDE(i, width)
  {
    float grad = 0.0f;
    const float pi = p[i];
    for (size_t b = 0; b < batch; ++b)
    {
      const float err = e[b * width + i];
      grad += 0.5f * (pi * err * err - 1.0f);
    }
    grad /= (float)batch;
    float lp = log_p[i] - pr * grad;
    lp = fmaxf(-5.0f, fminf(lp, 5.0f));
    log_p[i] = lp;
    p[i] = expf(lp);
  }
}

// ------------------------------------------------------------------------------ optimizer
__global__ void k_increment(int* counter)
{
  *counter += 1;
}
// Adam / AdamW (CPUBackend.cpp:721-772, CPUBackendHighway.cpp:779-840): t and lr live on the device
__global__ void k_adam(float* param, const float* grad, float* m, float* v, size_t n, const int* t,
                       const float* lr, float weight_decay, float beta1, float beta2, float eps)
{
  const float tf = (float)*t, rate = *lr;
  const float step = rate * sqrtf(1.0f - powf(beta2, tf)) / (1.0f - powf(beta1, tf));
  GRID_STRIDE(i, n)
  {
    const float g = grad[i];
    const float mi = beta1 * m[i] + (1.0f - beta1) * g;
    const float vi = beta2 * v[i] + (1.0f - beta2) * (g * g);
    m[i] = mi;
    v[i] = vi;
    float pi = param[i];
    if (weight_decay >= 0.0f)
      pi -= rate * weight_decay * pi;
    param[i] = pi - step * mi / (sqrtf(vi) + eps);
  }
}

// ------------------------------------------------------------------------------ convolution helpers
// columns[b][(c*kh+ky)*kw+kx][oy*ow+ox] = input[b][c][oy*sh-ph+ky][ox*sw-pw+kx] or 0
__global__ void k_im2col(const float* input, int batch, int channels, int height, int width, int kh,
                         int kw, int sh, int sw, int ph, int pw, int oh, int ow, float* columns)
{
  const size_t rows = (size_t)channels * kh * kw, cols = (size_t)oh * ow, n = (size_t)batch * rows * cols;
  GRID_STRIDE(i, n)
  {
    const size_t b = i / (rows * cols), r = (i / cols) % rows, p = i % cols;
    const int c = (int)(r / (kh * kw)), ky = (int)(r / kw) % kh, kx = (int)(r % kw);
    const int y = (int)(p / ow) * sh - ph + ky, x = (int)(p % ow) * sw - pw + kx;
    columns[i] = (y >= 0 && y < height && x >= 0 && x < width)
                     ? input[((b * channels + c) * height + y) * width + x]
                     : 0.0f;
  }
}
// the adjoint as a gather: image[b][c][y][x] += sum over the window positions that cover (y,x)
__global__ void k_col2im(const float* columns, int batch, int channels, int height, int width, int kh,
                         int kw, int sh, int sw, int ph, int pw, int oh, int ow, float* image)
{
  const size_t rows = (size_t)channels * kh * kw, cols = (size_t)oh * ow;
  const size_t n = (size_t)batch * channels * height * width;
  GRID_STRIDE(i, n)
  {
    const int x = (int)(i % width), y = (int)(i / width) % height;
    const int c = (int)(i / ((size_t)width * height)) % channels;
    const size_t b = i / ((size_t)width * height * channels);
    float acc = 0.0f;
    for (int ky = 0; ky < kh; ++ky)
    {
      const int ty = y + ph - ky;
      if (ty < 0 || ty % sh != 0 || ty / sh >= oh)
        continue;
      for (int kx = 0; kx < kw; ++kx)
      {
        const int tx = x + pw - kx;
        if (tx < 0 || tx % sw != 0 || tx / sw >= ow)
          continue;
        const size_t r = ((size_t)c * kh + ky) * kw + kx;
        acc += columns[(b * rows + r) * cols + (size_t)(ty / sh) * ow + tx / sw];
      }
    }
    image[i] += acc;
  }
}
__global__ void k_maxpool_forward(const float* input, int batch, int channels, int height, int width,
                                  int ph, int pw, int sh, int sw, int oh, int ow, float* output,
                                  int* argmax)
{
  const size_t n = (size_t)batch * channels * oh * ow;
  GRID_STRIDE(i, n)
  {
    const int ox = (int)(i % ow), oy = (int)(i / ow) % oh;
    const size_t plane = i / ((size_t)oh * ow);
    const float* in = input + plane * height * width;
    float best = -INFINITY;
    int arg = 0;
    for (int ky = 0; ky < ph; ++ky)
      for (int kx = 0; kx < pw; ++kx)
      {
        const int y = oy * sh + ky, x = ox * sw + kx;
        if (y < height && x < width && in[y * width + x] > best)
          best = in[y * width + x], arg = y * width + x;
      }
    output[i] = best;
    argmax[i] = arg;
  }
}
__global__ void k_maxpool_backward(const float* out_grad, const int* argmax, size_t n, int out_plane,
                                   int in_plane, float* in_grad)
{
  GRID_STRIDE(i, n)
  atomicAdd(&in_grad[(i / out_plane) * in_plane + argmax[i]], out_grad[i]);
}
// dst[row][b][col] = src[b][row][col]
__global__ void k_repack(float* dst, const float* src, size_t batch, size_t rows, size_t cols)
{
  const size_t n = batch * rows * cols;
  GRID_STRIDE(i, n)
  {
    const size_t col = i % cols, row = (i / cols) % rows, b = i / (cols * rows);
    dst[(row * batch + b) * cols + col] = src[i];
  }
}

// ------------------------------------------------------------------------------ fp32 GEMM (CUDA cores)
// 64 x 64 x 16 tiles, 256 threads, 4 x 4 results per thread; any shape, stride and transposition.
template <bool TA, bool TB>
__global__ void __launch_bounds__(256)
    k_sgemm(int M, int N, int K, float alpha, const float* __restrict__ A, int lda,
            const float* __restrict__ B, int ldb, float beta, float* __restrict__ C, int ldc)
{
  __shared__ float As[16][64 + 4], Bs[16][64 + 4];
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += 16)
  {
#pragma unroll
    for (int it = 0; it < 4; ++it)
    {
      const int idx = threadIdx.x + it * 256;
      // walk the contiguous dimension of each operand with consecutive threads
      const int am = TA ? idx & 63 : idx >> 4, ak = TA ? idx >> 6 : idx & 15;
      const int gm = m0 + am, gk = k0 + ak;
      As[ak][am] = (gm < M && gk < K) ? (TA ? A[(size_t)gk * lda + gm] : A[(size_t)gm * lda + gk]) : 0.0f;
      const int bn = TB ? idx >> 4 : idx & 63, bk = TB ? idx & 15 : idx >> 6;
      const int gn = n0 + bn, gkb = k0 + bk;
      Bs[bk][bn] = (gn < N && gkb < K) ? (TB ? B[(size_t)gn * ldb + gkb] : B[(size_t)gkb * ldb + gn]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k)
    {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        a[i] = As[k][ty * 4 + i], b[i] = Bs[k][tx * 4 + i];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
  {
    const int m = m0 + ty * 4 + i;
    if (m >= M)
      continue;
#pragma unroll
    for (int j = 0; j < 4; ++j)
    {
      const int n = n0 + tx * 4 + j;
      if (n < N)
      {
        float* c = C + (size_t)m * ldc + n;
        *c = alpha * acc[i][j] + (beta != 0.0f ? beta * *c : 0.0f);
      }
    }
  }
}
} // namespace

// ------------------------------------------------------------------------------ context
struct Ctx
{
  int device = 0;
  int sm_count = 148;
  cudaStream_t stream = nullptr;
  bool allow_tf32 = true;
  bool tensor_cores = false; // sm_100 with a tensor-map encoder
  static constexpr int kSlots = 8;
  cudaGraph_t graphs[kSlots] = {};
  cudaGraphExec_t execs[kSlots] = {};
  double* partials = nullptr; // kPartials + 1 doubles
  double* host_result = nullptr; // pinned
  TcGemm tc;
};

Ctx* create()
{
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0)
  {
    cudaGetLastError();
    fprintf(stderr, "DeepityCUDA (b200): no CUDA device available\n");
    return nullptr;
  }
  auto* c = new Ctx();
  cudaGetDevice(&c->device);
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, c->device) == cudaSuccess)
  {
    c->sm_count = prop.multiProcessorCount;
    // DEEPITY_B200_NO_TENSOR_CORES keeps every GEMM on the fp32 CUDA-core kernel (a test switch)
    c->tensor_cores = prop.major == 10 && !getenv("DEEPITY_B200_NO_TENSOR_CORES") &&
                      c->tc.init((int)prop.sharedMemPerBlockOptin);
  }
  if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaMalloc(&c->partials, sizeof(double) * (kPartials + 1)) != cudaSuccess ||
      cudaMallocHost(&c->host_result, sizeof(double)) != cudaSuccess)
  {
    fprintf(stderr, "DeepityCUDA (b200): could not set up the device context\n");
    destroy(c);
    return nullptr;
  }
  return c;
}

void destroy(Ctx* c)
{
  if (!c)
    return;
  if (c->stream)
    cudaStreamSynchronize(c->stream);
  for (int s = 0; s < Ctx::kSlots; ++s)
  {
    if (c->execs[s])
      cudaGraphExecDestroy(c->execs[s]);
    if (c->graphs[s])
      cudaGraphDestroy(c->graphs[s]);
  }
  if (c->partials)
    cudaFree(c->partials);
  if (c->host_result)
    cudaFreeHost(c->host_result);
  if (c->stream)
    cudaStreamDestroy(c->stream);
  delete c;
}

// ---- graphs (src/backend/cuda/CUDABackendCore.cu:120-187 in the reference) ----------------
void graph_begin(Ctx* c, size_t slot)
{
  if (slot >= (size_t)Ctx::kSlots)
    return;
  B200_CHECK(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
}
bool graph_end(Ctx* c, size_t slot)
{
  if (slot >= (size_t)Ctx::kSlots)
    return false;
  cudaGraph_t g = nullptr;
  if (cudaStreamEndCapture(c->stream, &g) != cudaSuccess || !g)
  {
    cudaGetLastError();
    return false;
  }
  if (c->execs[slot])
    cudaGraphExecDestroy(c->execs[slot]);
  if (c->graphs[slot])
    cudaGraphDestroy(c->graphs[slot]);
  c->execs[slot] = nullptr;
  c->graphs[slot] = g;
  if (cudaGraphInstantiate(&c->execs[slot], g, 0) != cudaSuccess)
  {
    cudaGetLastError();
    c->execs[slot] = nullptr;
    return false;
  }
  return true;
}
void graph_replay(Ctx* c, size_t slot)
{
  if (slot < (size_t)Ctx::kSlots && c->execs[slot])
    B200_CHECK(cudaGraphLaunch(c->execs[slot], c->stream));
}
void synchronize(Ctx* c)
{
  B200_CHECK(cudaStreamSynchronize(c->stream));
}

// ---- memory -------------------------------------------------------------------------------
float* allocate(Ctx*, size_t n)
{
  void* p = nullptr;
  if (cudaMalloc(&p, std::max<size_t>(n, 4) * sizeof(float)) != cudaSuccess)
  {
    cudaGetLastError();
    return nullptr;
  }
  return static_cast<float*>(p);
}
void release(Ctx*, float* p)
{
  if (p)
    B200_CHECK(cudaFree(p));
}
void zero(Ctx* c, float* p, size_t n)
{
  if (n)
    B200_CHECK(cudaMemsetAsync(p, 0, n * sizeof(float), c->stream));
}
void copy(Ctx* c, float* dst, const float* src, size_t n)
{
  if (n)
    B200_CHECK(cudaMemcpyAsync(dst, src, n * sizeof(float), cudaMemcpyDeviceToDevice, c->stream));
}
void copy2d(Ctx* c, float* dst, size_t dst_stride, const float* src, size_t src_stride, size_t rows,
            size_t cols)
{
  if (rows && cols)
    B200_CHECK(cudaMemcpy2DAsync(dst, dst_stride * sizeof(float), src, src_stride * sizeof(float),
                                 cols * sizeof(float), rows, cudaMemcpyDeviceToDevice, c->stream));
}
void copy_from_host(Ctx* c, float* dst, const float* host_src, size_t n)
{
  if (!n)
    return;
  B200_CHECK(cudaMemcpyAsync(dst, host_src, n * sizeof(float), cudaMemcpyHostToDevice, c->stream));
  B200_CHECK(cudaStreamSynchronize(c->stream));
}
void copy_to_host(Ctx* c, float* host_dst, const float* src, size_t n)
{
  if (!n)
    return;
  B200_CHECK(cudaMemcpyAsync(host_dst, src, n * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
  B200_CHECK(cudaStreamSynchronize(c->stream));
}
void randomize_normal(Ctx* c, float* buf, size_t n, float mean, float stddev, uint32_t seed)
{
  std::mt19937 rng(seed);
  std::normal_distribution<float> d(mean, stddev);
  std::vector<float> h(n);
  for (auto& v : h)
    v = d(rng);
  copy_from_host(c, buf, h.data(), n);
}
void randomize_uniform(Ctx* c, float* buf, size_t n, float lo, float hi, uint32_t seed)
{
  std::mt19937 rng(seed);
  std::uniform_real_distribution<float> d(lo, hi);
  std::vector<float> h(n);
  for (auto& v : h)
    v = d(rng);
  copy_from_host(c, buf, h.data(), n);
}
uintptr_t stream_handle(const Ctx* c)
{
  return reinterpret_cast<uintptr_t>(c->stream);
}

// ---- GEMM ---------------------------------------------------------------------------------
void set_allow_tf32(Ctx* c, bool allow)
{
  c->allow_tf32 = allow;
}

void sgemm(Ctx* c, bool ta, bool tb, int M, int N, int K, float alpha, const float* A, int lda,
           const float* B, int ldb, float beta, float* C, int ldc)
{
  if (M <= 0 || N <= 0)
    return;
  if (c->tensor_cores && c->allow_tf32 &&
      c->tc.run(c->stream, ta, tb, M, N, K, alpha, A, lda, B, ldb, beta, C, ldc))
    return;
  dim3 grid((N + 63) / 64, (M + 63) / 64);
  if (!ta && !tb)
    k_sgemm<false, false><<<grid, 256, 0, c->stream>>>(M, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
  else if (!ta && tb)
    k_sgemm<false, true><<<grid, 256, 0, c->stream>>>(M, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
  else if (ta && !tb)
    k_sgemm<true, false><<<grid, 256, 0, c->stream>>>(M, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
  else
    k_sgemm<true, true><<<grid, 256, 0, c->stream>>>(M, N, K, alpha, A, lda, B, ldb, beta, C, ldc);
  B200_CHECK(cudaPeekAtLastError());
}

void sgemm_batched(Ctx* c, bool ta, bool tb, int M, int N, int K, float alpha,
                   const float* const* host_A, int lda, const float* const* host_B, int ldb,
                   float beta, float* const* host_C, int ldc, int batch_count)
{
  // the pointer arrays live on the host (the networks build them in std::vectors): one launch
  // per item; inside a captured graph the launches cost no host time on replay
  for (int i = 0; i < batch_count; ++i)
    sgemm(c, ta, tb, M, N, K, alpha, host_A[i], lda, host_B[i], ldb, beta, host_C[i], ldc);
}

// ---- reductions -----------------------------------------------------------------------------
static float finish_reduction(Ctx* c, int blocks)
{
  k_reduce_final<<<1, kThreads, 0, c->stream>>>(c->partials, blocks, c->partials + kPartials);
  B200_CHECK(cudaMemcpyAsync(c->host_result, c->partials + kPartials, sizeof(double),
                             cudaMemcpyDeviceToHost, c->stream));
  B200_CHECK(cudaStreamSynchronize(c->stream));
  return (float)*c->host_result;
}
void sum_rows(Ctx* c, float* dst, const float* src, size_t batch, size_t width, size_t layers)
{
  if (!width || !layers)
    return;
  dim3 grid((unsigned)std::min<size_t>((width + 127) / 128, 1024), (unsigned)layers);
  k_sum_rows<<<grid, 128, 0, c->stream>>>(dst, src, batch, width);
  B200_CHECK(cudaPeekAtLastError());
}
float sum(Ctx* c, const float* buf, size_t n)
{
  const int blocks = blocks_for(n, kPartials);
  k_reduce_partials<<<blocks, kThreads, 0, c->stream>>>(0, nullptr, buf, nullptr, nullptr, n, 1,
                                                       c->partials);
  return finish_reduction(c, blocks);
}

// ---- elementwise ----------------------------------------------------------------------------
#define LAUNCH_1D(kernel, n, ...)                                                                \
  do                                                                                             \
  {                                                                                              \
    if ((n) > 0)                                                                                 \
    {                                                                                            \
      kernel<<<blocks_for((n), c->sm_count * 16), kThreads, 0, c->stream>>>(__VA_ARGS__);        \
      B200_CHECK(cudaPeekAtLastError());                                                         \
    }                                                                                            \
  } while (0)

void scale(Ctx* c, float* buf, size_t n, float alpha)
{
  LAUNCH_1D(k_scale, n, buf, n, alpha);
}
void axpy(Ctx* c, float* y, const float* x, size_t n, float alpha)
{
  LAUNCH_1D(k_axpy, n, y, x, n, alpha);
}
void add_bias(Ctx* c, float* buf, const float* bias, size_t batch, size_t width, size_t layers)
{
  LAUNCH_1D(k_add_bias, batch * width * layers, buf, bias, batch, width, layers);
}
void add_bias_per_channel(Ctx* c, float* buf, const float* bias, size_t batch, size_t channels,
                          size_t spatial)
{
  LAUNCH_1D(k_add_bias_channel, batch * channels * spatial, buf, bias, batch, channels, spatial);
}
void multiply(Ctx* c, float* dst, const float* a, const float* b, size_t n)
{
  LAUNCH_1D(k_multiply, n, dst, a, b, n);
}
void fill(Ctx* c, float* buf, size_t n, float value)
{
  LAUNCH_1D(k_fill, n, buf, n, value);
}
void center_rows(Ctx* c, float* buf, size_t rows, size_t cols)
{
  if (!buf || !rows || !cols)
    return;
  k_center_rows<<<(unsigned)std::min<size_t>(rows, 4096), kThreads, 0, c->stream>>>(buf, rows, cols);
  B200_CHECK(cudaPeekAtLastError());
}
void axpy_broadcast(Ctx* c, float* y, const float* x, const float* factor, size_t batch, size_t width,
                    float alpha)
{
  LAUNCH_1D(k_axpy_broadcast, batch * width, y, x, factor, batch * width, width, alpha);
}
void multiply_broadcast(Ctx* c, float* dst, const float* a, const float* factor, const float* b,
                        size_t batch, size_t width)
{
  LAUNCH_1D(k_multiply_broadcast, batch * width, dst, a, factor, b, batch * width, width);
}
void activation(Ctx* c, int type, float* dst, const float* src, size_t n)
{
  LAUNCH_1D(k_activation, n, type, dst, src, n);
}
void activation_derivative(Ctx* c, int dtype, float* dst, const float* src, size_t n,
                           bool from_activated)
{
  LAUNCH_1D(k_activation_derivative, n, dtype, dst, src, n, from_activated ? 1 : 0);
}
void derivative_multiply(Ctx* c, int dtype, float* dst, const float* a, float* x, size_t n,
                         bool from_activated, bool write_back)
{
  LAUNCH_1D(k_derivative_multiply, n, dtype, dst, a, x, n, from_activated ? 1 : 0, write_back ? 1 : 0);
}

// ---- predictive-coding ops --------------------------------------------------------------------
void state_update(Ctx* c, float* z, float* v, const float* feedback, int dtype, const float* e,
                  size_t n, float ir, float beta)
{
  LAUNCH_1D(k_state_update, n, z, v, feedback, dtype, e, n, ir, beta);
}
void compute_error(Ctx* c, float* e, const float* z, const float* mu, size_t n)
{
  LAUNCH_1D(k_error, n, e, z, mu, n);
}
float compute_error_energy(Ctx* c, float* e, const float* z, const float* mu, size_t n)
{
  const int blocks = blocks_for(n, kPartials);
  k_reduce_partials<<<blocks, kThreads, 0, c->stream>>>(1, e, z, mu, nullptr, n, 1, c->partials);
  return finish_reduction(c, blocks);
}
void error_and_activation(Ctx* c, int type, float* e, float* zf, const float* z, const float* mu,
                          size_t n)
{
  LAUNCH_1D(k_error_activation, n, type, e, zf, z, mu, n);
}
void softmax_ce_error(Ctx* c, float* e, const float* z, const float* mu, size_t batch, size_t width)
{
  if (!batch || !width)
    return;
  const int blocks = (int)std::min<size_t>((batch + 7) / 8, (size_t)kPartials);
  k_softmax_ce<<<blocks, kThreads, 0, c->stream>>>(e, z, mu, batch, width, nullptr);
  B200_CHECK(cudaPeekAtLastError());
}
float softmax_ce_error_energy(Ctx* c, float* e, const float* z, const float* mu, size_t batch,
                              size_t width)
{
  if (!batch || !width)
    return 0.0f;
  const int blocks = (int)std::min<size_t>((batch + 7) / 8, (size_t)kPartials);
  k_softmax_ce<<<blocks, kThreads, 0, c->stream>>>(e, z, mu, batch, width, c->partials);
  return finish_reduction(c, blocks);
}
void precision_error(Ctx* c, float* e, const float* z, const float* mu, const float*, size_t batch,
                     size_t width)
{
  LAUNCH_1D(k_precision_error, batch * width, e, z, mu, batch * width);
}
float precision_error_energy(Ctx* c, float* e, const float* z, const float* mu, const float* p,
                             size_t batch, size_t width)
{
  const size_t n = batch * width;
  const int blocks = blocks_for(n, kPartials);
  k_reduce_partials<<<blocks, kThreads, 0, c->stream>>>(2, e, z, mu, p, n, width, c->partials);
  return finish_reduction(c, blocks);
}
void update_precision(Ctx* c, float* p, float* log_p, const float* e, size_t batch, size_t width,
                      float pr)
{
  LAUNCH_1D(k_update_precision, width, p, log_p, e, batch, width, pr);
}

// ---- convolution helpers ----------------------------------------------------------------------
void im2col(Ctx* c, const float* input, int batch, int channels, int height, int width, int kh, int kw,
            int sh, int sw, int ph, int pw, float* columns)
{
  const int oh = (height + 2 * ph - kh) / sh + 1, ow = (width + 2 * pw - kw) / sw + 1;
  const size_t n = (size_t)batch * channels * kh * kw * oh * ow;
  LAUNCH_1D(k_im2col, n, input, batch, channels, height, width, kh, kw, sh, sw, ph, pw, oh, ow, columns);
}
void col2im(Ctx* c, const float* columns, int batch, int channels, int height, int width, int kh, int kw,
            int sh, int sw, int ph, int pw, float* image)
{
  const int oh = (height + 2 * ph - kh) / sh + 1, ow = (width + 2 * pw - kw) / sw + 1;
  const size_t n = (size_t)batch * channels * height * width;
  LAUNCH_1D(k_col2im, n, columns, batch, channels, height, width, kh, kw, sh, sw, ph, pw, oh, ow, image);
}
void maxpool_forward(Ctx* c, const float* input, int batch, int channels, int height, int width, int ph,
                     int pw, int sh, int sw, float* output, int* argmax)
{
  const int oh = (height - ph) / sh + 1, ow = (width - pw) / sw + 1;
  const size_t n = (size_t)batch * channels * oh * ow;
  LAUNCH_1D(k_maxpool_forward, n, input, batch, channels, height, width, ph, pw, sh, sw, oh, ow, output,
            argmax);
}
void maxpool_backward(Ctx* c, const float* out_grad, const int* argmax, int batch, int channels,
                      int height, int width, int out_h, int out_w, float* in_grad)
{
  const size_t n = (size_t)batch * channels * out_h * out_w;
  LAUNCH_1D(k_maxpool_backward, n, out_grad, argmax, n, out_h * out_w, height * width, in_grad);
}
void repack_for_batched_gemm(Ctx* c, float* dst, const float* src, size_t batch, size_t rows,
                             size_t cols)
{
  LAUNCH_1D(k_repack, batch * rows * cols, dst, src, batch, rows, cols);
}

// ---- optimizer ----------------------------------------------------------------------------------
void increment_counter(Ctx* c, int* counter)
{
  k_increment<<<1, 1, 0, c->stream>>>(counter);
  B200_CHECK(cudaPeekAtLastError());
}
void counter_to_host(Ctx* c, int* host_dst, const int* counter)
{
  B200_CHECK(cudaMemcpyAsync(host_dst, counter, sizeof(int), cudaMemcpyDeviceToHost, c->stream));
  B200_CHECK(cudaStreamSynchronize(c->stream));
}
void counter_from_host(Ctx* c, int* counter, const int* host_src)
{
  B200_CHECK(cudaMemcpyAsync(counter, host_src, sizeof(int), cudaMemcpyHostToDevice, c->stream));
  B200_CHECK(cudaStreamSynchronize(c->stream));
}
void adam(Ctx* c, float* param, const float* grad, float* m, float* v, size_t n, const int* t,
          const float* lr, float weight_decay, float beta1, float beta2, float eps)
{
  LAUNCH_1D(k_adam, n, param, grad, m, v, n, t, lr, weight_decay, beta1, beta2, eps);
}
} // namespace b200
