// Convolutional predictive coding (SimpleConvPCLayer / SimpleConvPCNetwork of the reference):
// implicit-GEMM kernels on the CUDA cores.  No im2col buffer, no repack: the gathers that
// the reference materialises (Im2Col, Col2Im, RepackForBatchedGemm) happen while a tile is
// fetched, and bias, activation, error, gated error, state update and energy are epilogues.
//
// Layouts are the reference's: z, e [B, C, H, W]; W [O, C*kH*kW] (row index (c*kH+ky)*kW+kx);
// b [O]; preact, mu [B, O, oH, oW].
#include <algorithm>
#include <cstring>

#include "dpc_internal.h"
#include "dpc_math.cuh"

namespace dpc
{
namespace conv
{
constexpr int TM = 64, TN = 64, TK = 16, THREADS = 256, PADC = 4;

enum ConvOp
{
  C_FWD = 0, // preact[o, (b,p)] = sum_k W[o,k] * col(z)[k,(b,p)]       M=O    N=B*oH*oW K=C*kH*kW
  C_BWD = 1, // dz[c, (b,y,x)]   = sum_k W^T[c,k=(o,ky,kx)] * g gathered  M=C    N=B*H*W   K=O*kH*kW
  C_WG = 2   // dW[o, r]         = sum_(b,p) g[o,(b,p)] * col(z)[r,(b,p)] M=O    N=C*kH*kW K=B*oH*oW
};

struct Tile
{
  float a[TK][TM + PADC];
  float b[TK][TN + PADC];
};

__device__ __forceinline__ void block_energy(float local, double* energy)
{
  __shared__ float warp_sums[THREADS / 32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    local += __shfl_xor_sync(0xffffffffu, local, o);
  if ((threadIdx.x & 31) == 0)
    warp_sums[threadIdx.x >> 5] = local;
  __syncthreads();
  if (threadIdx.x == 0)
  {
    float s = 0.0f;
#pragma unroll
    for (int w = 0; w < THREADS / 32; ++w)
      s += warp_sums[w];
    atomicAdd(energy, (double)(0.5f * s));
  }
}

template <int OP>
__global__ void __launch_bounds__(THREADS)
    conv_gemm_kernel(const dpc_conv_layer L, float* __restrict__ z_up, float* __restrict__ e_up,
                     int batch, int flags, double* energy, int k_chunk,
                     float* __restrict__ split_out = nullptr)
{
  const int C = L.in_c, O = L.out_c, H = L.in_h, Wd = L.in_w, kH = L.k_h, kW = L.k_w;
  const int oH = L.out_h, oW = L.out_w, P = oH * oW, HW = H * Wd, KK = kH * kW;
  const int rows = C * KK;
  int M, N, K;
  if (OP == C_FWD)
    M = O, N = batch * P, K = rows;
  else if (OP == C_BWD)
    M = C, N = batch * HW, K = O * KK;
  else
    M = O, N = rows, K = batch * P;
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  // k_chunk > 0: the reduction is split over blockIdx.z and the partial sums are added
  // atomically into a zeroed buffer (g_W for the weight gradient, preact for the forward
  // product, `split_out` for the state update); a second kernel applies the epilogue.
  int k_begin = 0, k_end = K;
  if (k_chunk > 0)
  {
    k_begin = blockIdx.z * k_chunk;
    k_end = min(K, k_begin + k_chunk);
  }

  __shared__ Tile tile;
  const int t = threadIdx.x;
  const int tx = t & 15, ty = t >> 4;

  // ---- per-thread invariants of the B-operand gather: 4 consecutive n, one k per pass
  const int bn = n0 + ((t & 15) << 2);
  int nb[4], ny[4], nx[4]; // FWD/BWD: image and (already offset) pixel origin; WG: (c, ky, kx)
#pragma unroll
  for (int j = 0; j < 4; ++j)
  {
    const int n = bn + j;
    if (n >= N)
    {
      nb[j] = -1, ny[j] = nx[j] = 0;
      continue;
    }
    if (OP == C_FWD)
    {
      const int b = n / P, p = n - b * P;
      const int oy = p / oW, ox = p - oy * oW;
      nb[j] = b, ny[j] = oy * L.s_h - L.p_h, nx[j] = ox * L.s_w - L.p_w;
    }
    else if (OP == C_BWD)
    {
      const int b = n / HW, q = n - b * HW;
      const int y = q / Wd, x = q - y * Wd;
      nb[j] = b, ny[j] = y + L.p_h, nx[j] = x + L.p_w;
    }
    else
    {
      const int c = n / KK, r = n - c * KK;
      nb[j] = c, ny[j] = r / kW, nx[j] = r - (r / kW) * kW;
    }
  }

  float ra[4], rb[4];
  auto fetch = [&](int k0)
  {
    // A operand: row = t>>2, 4 consecutive k
    {
      const int m = m0 + (t >> 2);
      const int kb = k0 + ((t & 3) << 2);
#pragma unroll
      for (int j = 0; j < 4; ++j)
      {
        const int k = kb + j;
        float v = 0.0f;
        if (m < M && k < k_end)
        {
          if (OP == C_FWD)
            v = L.W[(size_t)m * rows + k];
          else if (OP == C_BWD)
          {
            const int o = k / KK, r = k - o * KK;
            v = L.W[(size_t)o * rows + m * KK + r];
          }
          else
          {
            const int b = k / P, p = k - b * P;
            v = L.g[((size_t)b * O + m) * P + p];
          }
        }
        ra[j] = v;
      }
    }
    // B operand: k = t>>4, 4 consecutive n
    {
      const int k = k0 + (t >> 4);
      int q0 = 0, q1 = 0, q2 = 0; // FWD: (c, ky, kx); BWD: (o, ky, kx); WG: (b, oy*s-p, ox*s-p)
      const bool kin = k < k_end;
      if (kin)
      {
        if (OP == C_FWD || OP == C_BWD)
        {
          q0 = k / KK;
          const int r = k - q0 * KK;
          q1 = r / kW, q2 = r - q1 * kW;
        }
        else
        {
          q0 = k / P;
          const int p = k - q0 * P;
          const int oy = p / oW;
          q1 = oy * L.s_h - L.p_h, q2 = (p - oy * oW) * L.s_w - L.p_w;
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
      {
        float v = 0.0f;
        if (kin && nb[j] >= 0)
        {
          if (OP == C_FWD)
          {
            const int iy = ny[j] + q1, ix = nx[j] + q2;
            if (iy >= 0 && iy < H && ix >= 0 && ix < Wd)
              v = L.z[(((size_t)nb[j] * C + q0) * H + iy) * Wd + ix];
          }
          else if (OP == C_BWD)
          {
            const int ty2 = ny[j] - q1, tx2 = nx[j] - q2;
            if (ty2 >= 0 && tx2 >= 0)
            {
              const int oy = ty2 / L.s_h, ox = tx2 / L.s_w;
              if (oy * L.s_h == ty2 && ox * L.s_w == tx2 && oy < oH && ox < oW)
                v = L.g[(((size_t)nb[j] * O + q0) * oH + oy) * oW + ox];
            }
          }
          else
          {
            const int iy = q1 + ny[j], ix = q2 + nx[j];
            if (iy >= 0 && iy < H && ix >= 0 && ix < Wd)
              v = L.z[(((size_t)q0 * C + nb[j]) * H + iy) * Wd + ix];
          }
        }
        rb[j] = v;
      }
    }
  };
  auto stash = [&]()
  {
    const int r = t >> 2, kq = (t & 3) << 2;
#pragma unroll
    for (int j = 0; j < 4; ++j)
      tile.a[kq + j][r] = ra[j];
    *reinterpret_cast<float4*>(&tile.b[t >> 4][(t & 15) << 2]) =
        make_float4(rb[0], rb[1], rb[2], rb[3]);
  };

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
      acc[i][j] = 0.0f;

  if (k_begin < k_end)
  {
    fetch(k_begin);
    stash();
    __syncthreads();
    for (int k0 = k_begin; k0 < k_end; k0 += TK)
    {
      const bool more = k0 + TK < k_end;
      if (more)
        fetch(k0 + TK);
#pragma unroll
      for (int k = 0; k < TK; ++k)
      {
        const float4 av = *reinterpret_cast<const float4*>(&tile.a[k][ty * 4]);
        const float4 bv = *reinterpret_cast<const float4*>(&tile.b[k][tx * 4]);
        const float a4[4] = {av.x, av.y, av.z, av.w};
        const float b4[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j)
            acc[i][j] = fmaf(a4[i], b4[j], acc[i][j]);
      }
      __syncthreads();
      if (more)
      {
        stash();
        __syncthreads();
      }
    }
  }

  // ------------------------------------------------------------------ epilogues
  if (OP != C_WG && k_chunk > 0)
  {
    float* dst = OP == C_FWD ? L.preact : split_out;
    const int PP = OP == C_FWD ? P : HW; // pixels per (image, channel) plane of the output
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
        if (n >= N)
          continue;
        const int b = n / PP, q = n - b * PP;
        atomicAdd(&dst[((size_t)b * M + m) * PP + q], acc[i][j]);
      }
    }
    return;
  }
  if (OP == C_FWD)
  {
    float esum = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i)
    {
      const int m = m0 + ty * 4 + i;
      if (m >= M)
        continue;
      const float bias = L.b[m];
#pragma unroll
      for (int j = 0; j < 4; ++j)
      {
        const int n = n0 + tx * 4 + j;
        if (n >= N)
          continue;
        const int b = n / P, p = n - b * P;
        const size_t o = ((size_t)b * O + m) * P + p;
        const float pre = acc[i][j] + bias;
        float mu, d;
        act_both(L.act, pre, mu, d);
        L.preact[o] = pre;
        L.mu[o] = mu;
        if (flags & DPC_CONV_COPY_NEXT)
          z_up[o] = mu;
        if (flags & DPC_CONV_ERR_NEXT)
        {
          const float e = ((flags & DPC_CONV_COPY_NEXT) ? mu : z_up[o]) - mu;
          e_up[o] = e;
          esum += e * e;
          L.g[o] = e * d;
        }
      }
    }
    if (flags & DPC_CONV_ENERGY)
      block_energy(esum, energy);
  }
  else if (OP == C_BWD)
  {
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
        if (n >= N)
          continue;
        const int b = n / HW, q = n - b * HW;
        const size_t o = ((size_t)b * C + m) * HW + q;
        L.z[o] += L.ir * (acc[i][j] - L.e[o]);
      }
    }
  }
  else
  {
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
          atomicAdd(&L.g_W[(size_t)m * rows + n], acc[i][j]);
      }
    }
  }
}

// Second half of a split forward product: preact holds the raw sums; bias, activation, the
// error of the layer above, the gated error and the energy as in the fused epilogue.
__global__ void conv_forward_finish_kernel(const dpc_conv_layer L, float* __restrict__ z_up,
                                           float* __restrict__ e_up, int batch, int flags,
                                           double* energy)
{
  const int P = L.out_h * L.out_w;
  const size_t total = (size_t)batch * L.out_c * P;
  float esum = 0.0f;
  for (size_t o = (size_t)blockIdx.x * blockDim.x + threadIdx.x; o < total;
       o += (size_t)gridDim.x * blockDim.x)
  {
    const int oc = (int)((o / P) % L.out_c);
    const float pre = L.preact[o] + L.b[oc];
    float mu, d;
    act_both(L.act, pre, mu, d);
    L.preact[o] = pre;
    L.mu[o] = mu;
    if (flags & DPC_CONV_COPY_NEXT)
      z_up[o] = mu;
    if (flags & DPC_CONV_ERR_NEXT)
    {
      const float e = ((flags & DPC_CONV_COPY_NEXT) ? mu : z_up[o]) - mu;
      e_up[o] = e;
      esum += e * e;
      L.g[o] = e * d;
    }
  }
  if (flags & DPC_CONV_ENERGY)
    block_energy(esum, energy);
}

// Second half of a split state update: z += ir*(dz - e) with dz = the summed partials.
__global__ void conv_state_finish_kernel(const dpc_conv_layer L, const float* __restrict__ dz,
                                         int batch)
{
  const size_t total = (size_t)batch * L.in_c * L.in_h * L.in_w;
  for (size_t o = (size_t)blockIdx.x * blockDim.x + threadIdx.x; o < total;
       o += (size_t)gridDim.x * blockDim.x)
    L.z[o] += L.ir * (dz[o] - L.e[o]);
}

// A clamped layer whose prediction is cached: no convolution, preact/mu are read back.
__global__ void conv_cached_forward_kernel(const dpc_conv_layer L, float* __restrict__ z_up,
                                           float* __restrict__ e_up, int batch, int flags,
                                           double* energy)
{
  const size_t total = (size_t)batch * L.out_c * L.out_h * L.out_w;
  float esum = 0.0f;
  for (size_t o = (size_t)blockIdx.x * blockDim.x + threadIdx.x; o < total;
       o += (size_t)gridDim.x * blockDim.x)
  {
    const float mu = L.mu[o];
    if (flags & DPC_CONV_COPY_NEXT)
      z_up[o] = mu;
    if (flags & DPC_CONV_ERR_NEXT)
    {
      const float e = ((flags & DPC_CONV_COPY_NEXT) ? mu : z_up[o]) - mu;
      e_up[o] = e;
      esum += e * e;
      L.g[o] = e * act_deriv(L.act, L.preact[o]);
    }
  }
  if (flags & DPC_CONV_ENERGY)
    block_energy(esum, energy);
}

// g = e_above * mu with mu still holding the prediction: what the reference's weight update
// reads when no state update came after the last CalculateState
// (src/layers/SimpleConvPCLayer.cpp:414 with mu from :279-285).
__global__ void conv_gate_with_prediction_kernel(const dpc_conv_layer L,
                                                 const float* __restrict__ e_up, int batch)
{
  const size_t total = (size_t)batch * L.out_c * L.out_h * L.out_w;
  for (size_t o = (size_t)blockIdx.x * blockDim.x + threadIdx.x; o < total;
       o += (size_t)gridDim.x * blockDim.x)
    L.g[o] = e_up[o] * L.mu[o];
}

// z -= ir*e for a layer without weights (the terminal layer when it is not clamped).
__global__ void conv_relax_kernel(const dpc_conv_layer L, int batch)
{
  const size_t total = (size_t)batch * L.in_c * L.in_h * L.in_w;
  for (size_t o = (size_t)blockIdx.x * blockDim.x + threadIdx.x; o < total;
       o += (size_t)gridDim.x * blockDim.x)
    L.z[o] -= L.ir * L.e[o];
}

// g_b[o] = sum over (b, p) of g: one block per output channel, fixed summation order.
__global__ void conv_bias_grad_kernel(const dpc_conv_layer L, int batch)
{
  const int o = blockIdx.x, P = L.out_h * L.out_w;
  float s = 0.0f;
  for (int idx = threadIdx.x; idx < batch * P; idx += blockDim.x)
  {
    const int b = idx / P, p = idx - b * P;
    s += L.g[((size_t)b * L.out_c + o) * P + p];
  }
  __shared__ float red[32];
#pragma unroll
  for (int w = 16; w > 0; w >>= 1)
    s += __shfl_xor_sync(0xffffffffu, s, w);
  if ((threadIdx.x & 31) == 0)
    red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0)
  {
    float tsum = 0.0f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w)
      tsum += red[w];
    L.g_b[o] = tsum;
  }
}

// SGD / Adam / AdamW on W and b from the raw sums in g_W, g_b
// (src/layers/SimpleConvPCLayer.cpp:424-556: SGD rate lr/B with decay (1-lambda) first;
// Adam-type gradients are -(1/B) * sum).
__global__ void conv_apply_kernel(const dpc_conv_layer L, int batch)
{
  const size_t nW = (size_t)L.out_c * L.in_c * L.k_h * L.k_w;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t nthr = (size_t)gridDim.x * blockDim.x;
  const float Bf = (float)batch;
  if (L.opt == DPC_OPT_SGD)
  {
    const float alpha = L.lr / Bf;
    const float decay = L.lmbda > 0.0f ? 1.0f - L.lmbda : 1.0f;
    for (size_t o = tid; o < nW; o += nthr)
    {
      float w = L.W[o];
      if (decay != 1.0f)
        w *= decay;
      L.W[o] = fmaf(alpha, L.g_W[o], w);
    }
    for (size_t j = tid; j < (size_t)L.out_c; j += nthr)
      L.b[j] = fmaf(alpha, L.g_b[j], L.b[j]);
    return;
  }
  const float step = adam_step_size(L.lr, *L.t);
  const float lr_wd = L.opt == DPC_OPT_ADAMW ? L.lr * L.lmbda : -1.0f;
  const float gs = -1.0f / Bf;
  for (size_t o = tid; o < nW; o += nthr)
  {
    float m = L.m_W[o], v = L.v_W[o];
    L.W[o] = adam_update(L.W[o], gs * L.g_W[o], m, v, step, lr_wd);
    L.m_W[o] = m;
    L.v_W[o] = v;
  }
  for (size_t j = tid; j < (size_t)L.out_c; j += nthr)
  {
    float m = L.m_b[j], v = L.v_b[j];
    L.b[j] = adam_update(L.b[j], gs * L.g_b[j], m, v, step, -1.0f);
    L.m_b[j] = m;
    L.v_b[j] = v;
  }
}

__global__ void conv_bump_counter_kernel(int32_t* t)
{
  *t += 1;
}

// Row centring of W [O, C*kH*kW] (src/backend/CPUBackend.cpp:250-272): one block per row.
__global__ void conv_center_rows_kernel(const dpc_conv_layer L)
{
  const int rows = L.in_c * L.k_h * L.k_w;
  float* row = L.W + (size_t)blockIdx.x * rows;
  float s = 0.0f;
  for (int c = threadIdx.x; c < rows; c += blockDim.x)
    s += row[c];
  __shared__ float red[32];
#pragma unroll
  for (int w = 16; w > 0; w >>= 1)
    s += __shfl_xor_sync(0xffffffffu, s, w);
  if ((threadIdx.x & 31) == 0)
    red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0)
  {
    float tsum = 0.0f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w)
      tsum += red[w];
    red[0] = tsum;
  }
  __syncthreads();
  const float mean = red[0] / (float)rows;
  for (int c = threadIdx.x; c < rows; c += blockDim.x)
    row[c] -= mean;
}
} // namespace conv
} // namespace dpc

using namespace dpc;
using namespace dpc::conv;

struct dpc_conv_plan
{
  dpc_ctx* ctx = nullptr;
  int n = 0, batch = 0;
  std::vector<dpc_conv_layer> h;
  double* energy = nullptr;
  double* energy_host = nullptr;
  float* scratch = nullptr; // one state-sized buffer for split state updates (largest layer)
  size_t scratch_floats = 0;
};

namespace
{
// How many ways to split a reduction of length K over CTAs when the tile grid alone does not
// fill the GPU (returns 1 for "do not split"); k_chunk comes back as a multiple of TK.
int choose_split(int tiles, long long K, int sm_count, int* k_chunk)
{
  int splits = 1;
  if (tiles < sm_count && K >= 8 * TK)
    splits = (int)std::min<long long>((2LL * sm_count + tiles - 1) / tiles, K / (2 * TK));
  if (splits <= 1)
  {
    *k_chunk = 0;
    return 1;
  }
  long long chunk = (K + splits - 1) / splits;
  chunk = (chunk + TK - 1) / TK * TK;
  *k_chunk = (int)chunk;
  return (int)((K + chunk - 1) / chunk);
}

int conv_check_launch(dpc_ctx* ctx, const char* what)
{
  ctx->launches += 1;
  cudaError_t err = cudaPeekAtLastError();
  if (err != cudaSuccess)
    return cuda_fail(cudaGetLastError(), what);
  return DPC_OK;
}

inline int cdiv_i(long long a, long long b)
{
  return (int)((a + b - 1) / b);
}

int elem_grid(const dpc_conv_plan* p, size_t elems)
{
  size_t blocks = (elems + 1023) / 1024;
  const size_t cap = (size_t)p->ctx->sm_count * 8;
  return (int)std::max<size_t>(1, std::min(blocks, cap));
}

int validate(const dpc_conv_layer* l, int n)
{
  if (n < 2)
    return fail(DPC_ERR_INVALID, "a network needs at least two layers");
  for (int i = 0; i < n; ++i)
  {
    const dpc_conv_layer& L = l[i];
    if (L.in_c <= 0 || L.in_h <= 0 || L.in_w <= 0 || !L.z || !L.e)
      return fail(DPC_ERR_INVALID, "conv layer " + std::to_string(i) + ": bad input shape or state");
    if (L.out_c > 0)
    {
      if (L.k_h <= 0 || L.k_w <= 0 || L.s_h <= 0 || L.s_w <= 0 || L.p_h < 0 || L.p_w < 0)
        return fail(DPC_ERR_INVALID, "conv layer " + std::to_string(i) + ": bad kernel geometry");
      const int oh = (L.in_h + 2 * L.p_h - L.k_h) / L.s_h + 1;
      const int ow = (L.in_w + 2 * L.p_w - L.k_w) / L.s_w + 1;
      if (oh != L.out_h || ow != L.out_w || oh <= 0 || ow <= 0)
        return fail(DPC_ERR_INVALID, "conv layer " + std::to_string(i) + ": output size mismatch");
      if (!L.W || !L.b || !L.preact || !L.mu || !L.g || !L.g_W || !L.g_b)
        return fail(DPC_ERR_INVALID, "conv layer " + std::to_string(i) + ": missing tensors");
      if (L.opt != DPC_OPT_SGD && (!L.m_W || !L.v_W || !L.m_b || !L.v_b || !L.t))
        return fail(DPC_ERR_INVALID, "conv layer " + std::to_string(i) + ": missing Adam state");
      if (i + 1 >= n)
        return fail(DPC_ERR_INVALID, "the last layer must have out_c = 0");
      const dpc_conv_layer& U = l[i + 1];
      if (U.in_c != L.out_c || U.in_h != L.out_h || U.in_w != L.out_w)
        return fail(DPC_ERR_INVALID, "conv layer " + std::to_string(i) +
                                         ": output shape differs from the next layer's input");
    }
    else if (i + 1 != n)
      return fail(DPC_ERR_INVALID, "only the last layer may have out_c = 0");
  }
  return DPC_OK;
}

int check_layer(dpc_conv_plan* p, int layer)
{
  if (!p)
    return fail(DPC_ERR_INVALID, "null plan");
  if (layer < 0 || layer >= p->n)
    return fail(DPC_ERR_INVALID, "layer out of range");
  return DPC_OK;
}
} // namespace

int dpc_conv_plan_create(dpc_ctx* ctx, const dpc_conv_layer* layers, int n_layers, int batch,
                         dpc_conv_plan** out)
{
  if (!ctx || !layers || !out || batch <= 0)
    return fail(DPC_ERR_INVALID, "bad argument");
  int rc = validate(layers, n_layers);
  if (rc != DPC_OK)
    return rc;
  DPC_CUDA(cudaSetDevice(ctx->device));
  auto* p = new dpc_conv_plan();
  p->ctx = ctx, p->n = n_layers, p->batch = batch;
  p->h.assign(layers, layers + n_layers);
  if (cudaMalloc(&p->energy, sizeof(double)) != cudaSuccess ||
      cudaMallocHost(&p->energy_host, sizeof(double)) != cudaSuccess)
  {
    delete p;
    return cuda_fail(cudaGetLastError(), "conv plan allocation");
  }
  cudaMemset(p->energy, 0, sizeof(double));
  for (int i = 0; i < n_layers; ++i)
    p->scratch_floats = std::max(p->scratch_floats, (size_t)batch * layers[i].in_c *
                                                        layers[i].in_h * layers[i].in_w);
  if (cudaMalloc(&p->scratch, p->scratch_floats * sizeof(float)) != cudaSuccess)
  {
    cudaFree(p->energy);
    cudaFreeHost(p->energy_host);
    delete p;
    return cuda_fail(cudaGetLastError(), "conv plan scratch allocation");
  }
  *out = p;
  return DPC_OK;
}

int dpc_conv_plan_update(dpc_conv_plan* p, const dpc_conv_layer* layers, int n_layers)
{
  if (!p || !layers || n_layers != p->n)
    return fail(DPC_ERR_INVALID, "bad argument");
  int rc = validate(layers, n_layers);
  if (rc != DPC_OK)
    return rc;
  p->h.assign(layers, layers + n_layers);
  return DPC_OK;
}

int dpc_conv_plan_destroy(dpc_conv_plan* p)
{
  if (!p)
    return DPC_OK;
  cudaSetDevice(p->ctx->device);
  cudaStreamSynchronize(p->ctx->stream);
  if (p->energy)
    cudaFree(p->energy);
  if (p->energy_host)
    cudaFreeHost(p->energy_host);
  if (p->scratch)
    cudaFree(p->scratch);
  delete p;
  return DPC_OK;
}

int dpc_conv_forward(dpc_conv_plan* p, int layer, int flags)
{
  int rc = check_layer(p, layer);
  if (rc != DPC_OK)
    return rc;
  const dpc_conv_layer& L = p->h[layer];
  if (L.out_c <= 0)
    return DPC_OK;
  const dpc_conv_layer& U = p->h[layer + 1];
  cudaStream_t st = p->ctx->stream;
  const size_t outs = (size_t)p->batch * L.out_c * L.out_h * L.out_w;
  if (flags & DPC_CONV_CACHED)
  {
    if (!(flags & (DPC_CONV_COPY_NEXT | DPC_CONV_ERR_NEXT | DPC_CONV_ENERGY)))
      return DPC_OK;
    conv_cached_forward_kernel<<<elem_grid(p, outs), THREADS, 0, st>>>(L, U.z, U.e, p->batch,
                                                                      flags, p->energy);
    return conv_check_launch(p->ctx, "conv cached forward kernel");
  }
  const long long N = (long long)p->batch * L.out_h * L.out_w;
  dim3 grid(cdiv_i(N, TN), cdiv_i(L.out_c, TM), 1);
  int k_chunk = 0;
  const int splits = choose_split((int)(grid.x * grid.y), (long long)L.in_c * L.k_h * L.k_w,
                                  p->ctx->sm_count, &k_chunk);
  if (splits > 1)
  {
    grid.z = splits;
    DPC_CUDA(cudaMemsetAsync(L.preact, 0, outs * sizeof(float), st));
    conv_gemm_kernel<C_FWD><<<grid, THREADS, 0, st>>>(L, U.z, U.e, p->batch, flags, p->energy,
                                                     k_chunk);
    if ((rc = conv_check_launch(p->ctx, "conv forward kernel (split)")) != DPC_OK)
      return rc;
    conv_forward_finish_kernel<<<elem_grid(p, outs), THREADS, 0, st>>>(L, U.z, U.e, p->batch, flags,
                                                                      p->energy);
    return conv_check_launch(p->ctx, "conv forward finish kernel");
  }
  conv_gemm_kernel<C_FWD><<<grid, THREADS, 0, st>>>(L, U.z, U.e, p->batch, flags, p->energy, 0);
  return conv_check_launch(p->ctx, "conv forward kernel");
}

int dpc_conv_update_state(dpc_conv_plan* p, int layer)
{
  int rc = check_layer(p, layer);
  if (rc != DPC_OK)
    return rc;
  const dpc_conv_layer& L = p->h[layer];
  cudaStream_t st = p->ctx->stream;
  const size_t ins = (size_t)p->batch * L.in_c * L.in_h * L.in_w;
  if (L.out_c <= 0 || layer + 1 >= p->n)
  {
    conv_relax_kernel<<<elem_grid(p, ins), THREADS, 0, st>>>(L, p->batch);
    return conv_check_launch(p->ctx, "conv relax kernel");
  }
  const long long N = (long long)p->batch * L.in_h * L.in_w;
  dim3 grid(cdiv_i(N, TN), cdiv_i(L.in_c, TM), 1);
  int k_chunk = 0;
  const int splits = choose_split((int)(grid.x * grid.y), (long long)L.out_c * L.k_h * L.k_w,
                                  p->ctx->sm_count, &k_chunk);
  if (splits > 1)
  {
    grid.z = splits;
    DPC_CUDA(cudaMemsetAsync(p->scratch, 0, ins * sizeof(float), st));
    conv_gemm_kernel<C_BWD><<<grid, THREADS, 0, st>>>(L, nullptr, nullptr, p->batch, 0, p->energy,
                                                     k_chunk, p->scratch);
    if ((rc = conv_check_launch(p->ctx, "conv state update kernel (split)")) != DPC_OK)
      return rc;
    conv_state_finish_kernel<<<elem_grid(p, ins), THREADS, 0, st>>>(L, p->scratch, p->batch);
    return conv_check_launch(p->ctx, "conv state finish kernel");
  }
  conv_gemm_kernel<C_BWD><<<grid, THREADS, 0, st>>>(L, nullptr, nullptr, p->batch, 0, p->energy, 0);
  return conv_check_launch(p->ctx, "conv state update kernel");
}

int dpc_conv_gate_with_prediction(dpc_conv_plan* p, int layer)
{
  int rc = check_layer(p, layer);
  if (rc != DPC_OK)
    return rc;
  const dpc_conv_layer& L = p->h[layer];
  if (L.out_c <= 0)
    return DPC_OK;
  const size_t outs = (size_t)p->batch * L.out_c * L.out_h * L.out_w;
  conv_gate_with_prediction_kernel<<<elem_grid(p, outs), THREADS, 0, p->ctx->stream>>>(
      L, p->h[layer + 1].e, p->batch);
  return conv_check_launch(p->ctx, "conv gate kernel");
}

int dpc_conv_update_weights(dpc_conv_plan* p, int layer, int center_rows)
{
  int rc = check_layer(p, layer);
  if (rc != DPC_OK)
    return rc;
  const dpc_conv_layer& L = p->h[layer];
  if (L.out_c <= 0)
    return DPC_OK;
  cudaStream_t st = p->ctx->stream;
  const int rows = L.in_c * L.k_h * L.k_w;
  const long long K = (long long)p->batch * L.out_h * L.out_w;
  DPC_CUDA(cudaMemsetAsync(L.g_W, 0, sizeof(float) * (size_t)L.out_c * rows, st));
  // Split the long reduction (batch x output pixels) over enough CTAs to fill the GPU.
  const int tiles = cdiv_i(rows, TN) * cdiv_i(L.out_c, TM);
  int splits = std::max(1, std::min<int>((int)(K / (4 * TK)) + 1, (2 * p->ctx->sm_count) / tiles));
  int k_chunk = cdiv_i(K, splits);
  k_chunk = cdiv_i(k_chunk, TK) * TK;
  splits = cdiv_i(K, k_chunk);
  dim3 grid(cdiv_i(rows, TN), cdiv_i(L.out_c, TM), splits);
  conv_gemm_kernel<C_WG><<<grid, THREADS, 0, st>>>(L, nullptr, nullptr, p->batch, 0, p->energy,
                                                  k_chunk);
  if ((rc = conv_check_launch(p->ctx, "conv weight gradient kernel")) != DPC_OK)
    return rc;
  conv_bias_grad_kernel<<<L.out_c, 256, 0, st>>>(L, p->batch);
  if ((rc = conv_check_launch(p->ctx, "conv bias gradient kernel")) != DPC_OK)
    return rc;
  if (L.opt != DPC_OPT_SGD)
  {
    conv_bump_counter_kernel<<<1, 1, 0, st>>>(L.t);
    if ((rc = conv_check_launch(p->ctx, "conv counter kernel")) != DPC_OK)
      return rc;
  }
  conv_apply_kernel<<<elem_grid(p, (size_t)L.out_c * rows), THREADS, 0, st>>>(L, p->batch);
  if ((rc = conv_check_launch(p->ctx, "conv apply kernel")) != DPC_OK)
    return rc;
  if (center_rows)
  {
    conv_center_rows_kernel<<<L.out_c, 128, 0, st>>>(L);
    if ((rc = conv_check_launch(p->ctx, "conv center rows kernel")) != DPC_OK)
      return rc;
  }
  return DPC_OK;
}

int dpc_conv_energy_reset(dpc_conv_plan* p)
{
  if (!p)
    return fail(DPC_ERR_INVALID, "null plan");
  DPC_CUDA(cudaMemsetAsync(p->energy, 0, sizeof(double), p->ctx->stream));
  return DPC_OK;
}

int dpc_conv_energy_read(dpc_conv_plan* p, double* out)
{
  if (!p || !out)
    return fail(DPC_ERR_INVALID, "bad argument");
  DPC_CUDA(cudaMemcpyAsync(p->energy_host, p->energy, sizeof(double), cudaMemcpyDeviceToHost,
                           p->ctx->stream));
  DPC_CUDA(cudaStreamSynchronize(p->ctx->stream));
  *out = *p->energy_host;
  return DPC_OK;
}
