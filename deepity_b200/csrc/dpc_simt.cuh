// CUDA-core (fp32 FFMA) kernels for every phase of the predictive-coding train step.
// They handle any shape (ragged, tiny terminal widths, unaligned leading dimensions) and
// are the path for layers outside the tensor-core run.  One launch covers a whole range
// of layers: blockIdx.z selects the layer, blockIdx.x/y the output tile; CTAs outside a
// layer's own tile grid return at once.
#pragma once
#include <cuda_bf16.h>
#include "dpc_math.cuh"

namespace dpc
{
constexpr int BM = 64, BN = 64, BK = 16, NTHREADS = 256, PAD = 4;

enum GemmOp
{
  OP_FWD = 0, // mu = f(a z W^T + b)             M=B  N=next K=size
  OP_FB = 1,  // z += ir (a fe W - e)            M=B  N=size K=next
  OP_WG = 2   // W += alpha g^T zin              M=next N=size K=B
};

// mode of OP_WG
enum
{
  WG_LEARN = 0, // UpdateWeights: g = fe (or e_above for Simple), rate lr, optimizer
  WG_DFA = 1,   // DirectFeedbackUpdate: g = fe (holds proj), rate fl, plain accumulate
  // or-ed in: only store the raw sum g^T zin in the layer's gradient staging buffer g_W; the
  // update is applied later by apply_gradients_kernel (after a sum over batch shards)
  WG_GRAD_ONLY = 2
};
// mode of OP_FB
enum
{
  FB_STATE = 0,  // UpdateState
  FB_ADJOINT = 1 // ePC ComputeAdjoint + UpdateErrorEPC (fe holds src * f'(preact))
};

struct Tile
{
  float a[BK][BM + PAD];
  float b[BK][BN + PAD];
};

// Operand whose rows are the M/N index with k contiguous: G[(row0+r)*ld + k0+k].
template <bool kAct>
__device__ __forceinline__ void fetch_kmajor(float (&reg)[4], const float* __restrict__ G, int ld,
                                             int row0, int k0, int nrows, int K, bool vec,
                                             int act)
{
  const int t = threadIdx.x;
  const int r = row0 + (t >> 2), k = k0 + ((t & 3) << 2);
  if (r < nrows && vec && k + 3 < K)
  {
    float4 v = *reinterpret_cast<const float4*>(G + (size_t)r * ld + k);
    reg[0] = v.x, reg[1] = v.y, reg[2] = v.z, reg[3] = v.w;
  }
  else
  {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      reg[j] = (r < nrows && k + j < K) ? G[(size_t)r * ld + k + j] : 0.0f;
  }
  if (kAct)
  {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      reg[j] = (r < nrows && k + j < K) ? act_fwd(act, reg[j]) : 0.0f;
  }
}

template <int COLS>
__device__ __forceinline__ void stash_kmajor(float (*S)[COLS + PAD], const float (&reg)[4])
{
  const int t = threadIdx.x;
  const int r = t >> 2, k = (t & 3) << 2;
#pragma unroll
  for (int j = 0; j < 4; ++j)
    S[k + j][r] = reg[j];
}

// Operand stored [K, cols] with cols contiguous: G[(k0+k)*ld + col0+c].
__device__ __forceinline__ void fetch_mnmajor(float (&reg)[4], const float* __restrict__ G, int ld,
                                              int col0, int k0, int ncols, int K, bool vec)
{
  const int t = threadIdx.x;
  const int k = k0 + (t >> 4), c = col0 + ((t & 15) << 2);
  if (k < K && vec && c + 3 < ncols)
  {
    float4 v = *reinterpret_cast<const float4*>(G + (size_t)k * ld + c);
    reg[0] = v.x, reg[1] = v.y, reg[2] = v.z, reg[3] = v.w;
  }
  else
  {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      reg[j] = (k < K && c + j < ncols) ? G[(size_t)k * ld + c + j] : 0.0f;
  }
}

template <int COLS>
__device__ __forceinline__ void stash_mnmajor(float (*S)[COLS + PAD], const float (&reg)[4])
{
  const int t = threadIdx.x;
  const int k = t >> 4, c = (t & 15) << 2;
  *reinterpret_cast<float4*>(&S[k][c]) = make_float4(reg[0], reg[1], reg[2], reg[3]);
}

__device__ __forceinline__ bool aligned16(const void* p)
{
  return (reinterpret_cast<uintptr_t>(p) & 15) == 0;
}

__device__ __forceinline__ void block_energy_add(float local, double* energy)
{
  __shared__ float warp_sums[NTHREADS / 32];
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
    for (int w = 0; w < NTHREADS / 32; ++w)
      s += warp_sums[w];
    atomicAdd(energy, (double)(0.5f * s));
  }
}

// ---------------------------------------------------------------------------------------
// Row split over a thread-block cluster.  The reductions over the batch below (Psi update, bias
// column sums) give one block a strip of columns and all rows, which fills the GPU when a launch
// covers thousands of layers but not when it covers four.  Such launches go out as clusters of R
// CTAs along z: CTA r of a cluster takes every R-th group of rows, leaves its partial sums in its
// own shared memory, and CTA 0 adds the others' in rank order through distributed shared memory
// (a fixed order: the result does not depend on timing).  Without the cluster attribute R is 1.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t rows_cluster_rank()
{
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t rows_cluster_size()
{
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void rows_cluster_sync()
{
  asm volatile("barrier.cluster.arrive.release.aligned;\n"
               "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the float at the same shared-memory address in CTA `rank` of the cluster
__device__ __forceinline__ float rows_cluster_load(const float* own, uint32_t rank)
{
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(own);
  uint32_t ra;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(a), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(ra) : "memory");
  return v;
}

// ---------------------------------------------------------------------------------------
// Forward pass of narrow layers (at most 16 output units: the heads, e.g. 1024 -> 10).  The tiled
// kernel below gives such a layer one column of 64 x 64 tiles, i.e. batch/64 CTAs that each walk
// all of K: latency-bound (96 us for 4096 x 10 x 1024 against 3 us of traffic).  Here a warp owns
// one batch row: its lanes stride over K with 16-byte loads of the row and of the (L1-resident)
// weight rows, the partial dot products are reduced by shuffles, and lane 2j finishes output unit
// j with the same epilogue as the tiled kernel.  Needs size % 4 == 0 and 16-byte aligned z, W.
// ---------------------------------------------------------------------------------------
// Sums a[0..15] over the 32 lanes with 16 shuffles instead of 80: each step a lane hands the half
// of its values that its partner keeps to the partner and adds the partner's to the half it
// keeps.  Returns the total of a[(lane >> 1) & 15] (lanes 2n and 2n + 1 both end with unit n).
__device__ __forceinline__ float warp_reduce16(float (&a)[16], int lane)
{
#pragma unroll
  for (int w = 8; w >= 1; w >>= 1)
  {
    const bool upper = (lane & (2 * w)) != 0;
#pragma unroll
    for (int i = 0; i < w; ++i)
    {
      const float send = upper ? a[i] : a[i + w];
      const float keep = upper ? a[i + w] : a[i];
      a[i] = keep + __shfl_xor_sync(0xffffffffu, send, 2 * w);
    }
  }
  return a[0] + __shfl_xor_sync(0xffffffffu, a[0], 1);
}

// RPW batch rows per warp (2 on large batches: every weight vector fetched from L1 then serves two
// rows).
template <int RPW>
__global__ void __launch_bounds__(NTHREADS)
    narrow_forward_kernel(const dpc_layer* __restrict__ layers, int first, int n_layers, int batch,
                          int flags, double* energy)
{
  const int li = first + blockIdx.z;
  const dpc_layer L = layers[li];
  if (L.next_size <= 0)
    return;
  const int N = L.next_size, K = L.size;
  const dpc_layer* Lup = (li + 1 < n_layers) ? &layers[li + 1] : nullptr;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = (blockIdx.x * (NTHREADS / 32) + warp) * RPW;
  float acc[RPW][16];
#pragma unroll
  for (int r = 0; r < RPW; ++r)
#pragma unroll
    for (int j = 0; j < 16; ++j)
      acc[r][j] = 0.0f;
  if (m0 < batch)
  {
    // 1024 elements of the rows at a time: the lane's eight 16-byte loads per row are all issued
    // before the first use (4 KB in flight per row), then every weight row is walked over the
    // same chunk
    for (int kc = 0; kc < K; kc += 1024)
    {
      const int k0 = kc + lane * 4;
      float4 zv[RPW][8];
#pragma unroll
      for (int r = 0; r < RPW; ++r)
      {
        const float* zrow = L.z + (size_t)(m0 + r) * K;
#pragma unroll
        for (int i = 0; i < 8; ++i)
          zv[r][i] = (m0 + r < batch && k0 + i * 128 < K)
                         ? *reinterpret_cast<const float4*>(zrow + k0 + i * 128)
                         : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      }
#pragma unroll
      for (int j = 0; j < 16; ++j)
      {
        if (j < N)
        {
          const float* wrow = L.W + (size_t)j * K + k0;
#pragma unroll
          for (int i = 0; i < 8; ++i)
          {
            if (k0 + i * 128 < K)
            {
              const float4 wv = __ldg(reinterpret_cast<const float4*>(wrow + i * 128));
#pragma unroll
              for (int r = 0; r < RPW; ++r)
              {
                acc[r][j] = fmaf(zv[r][i].x, wv.x, acc[r][j]);
                acc[r][j] = fmaf(zv[r][i].y, wv.y, acc[r][j]);
                acc[r][j] = fmaf(zv[r][i].z, wv.z, acc[r][j]);
                acc[r][j] = fmaf(zv[r][i].w, wv.w, acc[r][j]);
              }
            }
          }
        }
      }
    }
  }
  float esum = 0.0f;
  const bool next_ce = Lup && (Lup->flags & DPC_LAYER_SOFTMAX_CE);
  const bool do_err = (flags & DPC_FWD_ERR_NEXT) && Lup && !next_ce;
  const bool do_fe = (flags & DPC_FWD_FE) && Lup && !(next_ce && (flags & DPC_FWD_ERR_NEXT));
  const bool do_copy = (flags & DPC_FWD_COPY_NEXT) && Lup;
#pragma unroll
  for (int r = 0; r < RPW; ++r)
  {
    // lanes 2n and 2n+1 end with the sum of output unit n; the even one finishes it
    const float mine = warp_reduce16(acc[r], lane);
    const int m = m0 + r, n = lane >> 1;
    if (m < batch && !(lane & 1) && n < N)
    {
      const size_t o = (size_t)m * N + n;
      const float pre = L.a * mine + L.b[n];
      float mu, d = 1.0f;
      if (do_fe)
        act_both(L.act, pre, mu, d);
      else
        mu = act_fwd(L.act, pre);
      if (L.flags & DPC_LAYER_RESIDUAL)
        mu += L.z[o];
      if (!(flags & DPC_FWD_TRANSIENT))
      {
        const bool no_mu = do_copy && (flags & DPC_FWD_NO_MU);
        if (L.preact && !(no_mu && (flags & DPC_FWD_NO_PREACT)))
          L.preact[o] = pre;
        if (!no_mu)
          L.mu[o] = mu;
      }
      if (do_copy)
        Lup->z[o] = mu;
      float e = 0.0f;
      if (do_err)
      {
        e = (do_copy ? mu : Lup->z[o]) - mu;
        Lup->e[o] = e;
        esum += e * e;
      }
      else if (do_fe)
        e = Lup->e[o];
      if (do_fe)
        L.fe[o] = e * d;
    }
  }
  if (flags & DPC_FWD_ENERGY)
    block_energy_add(do_err ? esum : 0.0f, energy);
}

// ---------------------------------------------------------------------------------------
// The grouped GEMM kernel.  OP selects operand layouts and the fused epilogue.
// ---------------------------------------------------------------------------------------
template <int OP>
__global__ void __launch_bounds__(NTHREADS)
    pc_gemm_kernel(const dpc_layer* __restrict__ layers, int first, int n_layers, int batch,
                   int flags, int mode, double* energy, const float* __restrict__ epc_src = nullptr)
{
  const int li = first + blockIdx.z;
  const dpc_layer L = layers[li];
  if (L.next_size <= 0)
    return;
  const bool simple = (L.flags & DPC_LAYER_INPUT_ACT) != 0;

  int M, N, K;
  if (OP == OP_FWD)
    M = batch, N = L.next_size, K = L.size;
  else if (OP == OP_FB)
    M = batch, N = L.size, K = L.next_size;
  else
    M = L.next_size, N = L.size, K = batch;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  if (m0 >= M || n0 >= N)
    return;
  const bool wg_stage = OP == OP_WG && (mode & WG_GRAD_ONLY);
  if (OP == OP_WG)
    mode &= ~WG_GRAD_ONLY;
  if (OP == OP_WG && mode == WG_DFA)
  {
    // DirectFeedbackUpdate is a no-op unless the layer above owns feedback weights.
    if (li + 1 >= n_layers || layers[li + 1].Psi == nullptr)
      return;
  }

  const dpc_layer* Lup = (li + 1 < n_layers) ? &layers[li + 1] : nullptr;
  const float* A;
  const float* Bm;
  int lda, ldb;
  if (OP == OP_FWD)
    A = L.z, lda = L.size, Bm = L.W, ldb = L.size;
  else if (OP == OP_FB)
    A = (simple && mode == FB_STATE) ? Lup->e : L.fe, lda = L.next_size, Bm = L.W, ldb = L.size;
  else
    A = (simple && mode == WG_LEARN) ? Lup->e : L.fe, lda = L.next_size,
    Bm = simple ? L.zF : L.z, ldb = L.size;

  __shared__ Tile tile;
  const bool vecA = aligned16(A) && (lda % 4 == 0);
  const bool vecB = aligned16(Bm) && (ldb % 4 == 0);
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
      acc[i][j] = 0.0f;

  float ra[4], rb[4];
  auto fetch = [&](int k0)
  {
    if (OP == OP_FWD)
    {
      if (simple)
        fetch_kmajor<true>(ra, A, lda, m0, k0, M, K, vecA, L.act);
      else
        fetch_kmajor<false>(ra, A, lda, m0, k0, M, K, vecA, 0);
      fetch_kmajor<false>(rb, Bm, ldb, n0, k0, N, K, vecB, 0);
    }
    else if (OP == OP_FB)
    {
      fetch_kmajor<false>(ra, A, lda, m0, k0, M, K, vecA, 0);
      fetch_mnmajor(rb, Bm, ldb, n0, k0, N, K, vecB);
    }
    else
    {
      fetch_mnmajor(ra, A, lda, m0, k0, M, K, vecA);
      fetch_mnmajor(rb, Bm, ldb, n0, k0, N, K, vecB);
    }
  };
  auto stash = [&](int k0)
  {
    if (OP == OP_WG)
      stash_mnmajor<BM>(tile.a, ra);
    else
      stash_kmajor<BM>(tile.a, ra);
    if (OP == OP_FWD)
      stash_kmajor<BN>(tile.b, rb);
    else
      stash_mnmajor<BN>(tile.b, rb);
    if (OP == OP_FWD && simple && blockIdx.x == 0 && L.zF != nullptr)
    {
      // SimplePC keeps f(z) as last fed to the GEMM for its weight update
      // (src/layers/SimplePCLayer.cpp:146-150).
      const int t = threadIdx.x;
      const int r = m0 + (t >> 2), k = k0 + ((t & 3) << 2);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (r < M && k + j < K)
          L.zF[(size_t)r * L.size + k + j] = ra[j];
    }
  };

  fetch(0);
  stash(0);
  __syncthreads();
  for (int k0 = 0; k0 < K; k0 += BK)
  {
    const bool more = k0 + BK < K;
    if (more)
      fetch(k0 + BK);
#pragma unroll
    for (int k = 0; k < BK; ++k)
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
      stash(k0 + BK);
      __syncthreads();
    }
  }

  // ------------------------------------------------------------------ epilogues
  float esum = 0.0f;
  if (OP == OP_FWD)
  {
    const bool next_ce = Lup && (Lup->flags & DPC_LAYER_SOFTMAX_CE);
    const bool do_err = (flags & DPC_FWD_ERR_NEXT) && Lup && !next_ce;
    const bool do_fe = (flags & DPC_FWD_FE) && Lup && !simple && !(next_ce && (flags & DPC_FWD_ERR_NEXT));
    const bool do_copy = (flags & DPC_FWD_COPY_NEXT) && Lup;
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
        const size_t o = (size_t)m * N + n;
        const float pre = L.a * acc[i][j] + L.b[n];
        float mu, d = 1.0f;
        if (simple)
          mu = pre;
        else
        {
          if (do_fe)
            act_both(L.act, pre, mu, d);
          else
            mu = act_fwd(L.act, pre);
          if (L.flags & DPC_LAYER_RESIDUAL)
            mu += L.z[o];
        }
        if (!(flags & DPC_FWD_TRANSIENT))
        {
          const bool no_mu = do_copy && (flags & DPC_FWD_NO_MU);
          if (L.preact && !(no_mu && (flags & DPC_FWD_NO_PREACT)))
            L.preact[o] = pre;
          if (!no_mu)
            L.mu[o] = mu;
        }
        if (do_copy)
          Lup->z[o] = mu;
        float e = 0.0f;
        if (do_err)
        {
          e = (do_copy ? mu : Lup->z[o]) - mu;
          Lup->e[o] = e;
          esum += e * e;
        }
        else if (do_fe)
          e = Lup->e[o];
        if (do_fe)
          L.fe[o] = e * d;
      }
    }
    if (flags & DPC_FWD_ENERGY)
      block_energy_add(do_err ? esum : 0.0f, energy);
  }
  else if (OP == OP_FB)
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
        const size_t o = (size_t)m * N + n;
        if (mode == FB_ADJOINT)
        {
          // ePC: adjoint of this layer and the error update driven by it.  `flags` carries the
          // hop scale (+1 or -1) as float bits with bit 0 replaced by the clamp flag.
          const float scale = __int_as_float(flags & ~1);
          const bool clamped = flags & 1;
          float adj = (L.a * scale) * acc[i][j];
          if (L.flags & DPC_LAYER_RESIDUAL)
            adj += scale * epc_src[o];
          L.adj[o] = adj;
          if (!clamped)
            L.e[o] = (1.0f - L.ir) * L.e[o] - L.ir * adj;
          continue;
        }
        float z = L.z[o];
        if (simple)
        {
          z += L.ir * (acc[i][j] * act_deriv(L.act, z) - L.e[o]);
        }
        else
        {
          const float fb = L.a * acc[i][j] - L.e[o];
          if (L.v)
          {
            const float v = L.momentum_beta * L.v[o] + (1.0f - L.momentum_beta) * fb;
            L.v[o] = v;
            z += L.ir * v;
          }
          else
            z += L.ir * fb;
          if (L.flags & DPC_LAYER_RESIDUAL)
            z += L.ir * Lup->e[o];
        }
        L.z[o] = z;
      }
    }
  }
  else
  {
    if (wg_stage)
    {
#pragma unroll
      for (int i = 0; i < 4; ++i)
      {
        const int m = m0 + ty * 4 + i;
#pragma unroll
        for (int j = 0; j < 4; ++j)
        {
          const int n = n0 + tx * 4 + j;
          if (m < M && n < N)
            L.g_W[(size_t)m * N + n] = acc[i][j];
        }
      }
      return;
    }
    const float Bf = (float)batch;
    const bool adam = (mode == WG_LEARN) && (L.opt != DPC_OPT_SGD);
    float alpha, decay = 1.0f, step = 0.0f, lr_wd = -1.0f;
    if (mode == WG_DFA)
    {
      alpha = L.fl * L.a / Bf;
      if ((flags & 1) && L.lmbda > 0.0f && L.fl != 0.0f)
        decay = 1.0f - L.lmbda;
    }
    else if (!adam)
    {
      alpha = simple ? (L.lr / Bf) : (L.a * L.lr / Bf);
      if (L.lmbda > 0.0f)
        decay = 1.0f - L.lmbda;
    }
    else
    {
      alpha = -1.0f * L.a;
      step = adam_step_size(L.lr, *L.t);
      if (L.opt == DPC_OPT_ADAMW)
        lr_wd = L.lr * L.lmbda;
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
        if (n >= N)
          continue;
        const size_t o = (size_t)m * N + n;
        float w = L.W[o];
        if (!adam)
        {
          if (decay != 1.0f)
            w *= decay;
          w = fmaf(alpha, acc[i][j], w);
        }
        else
        {
          float mm = L.m_W[o], vv = L.v_W[o];
          w = adam_update(w, alpha * acc[i][j], mm, vv, step, lr_wd);
          L.m_W[o] = mm;
          L.v_W[o] = vv;
        }
        L.W[o] = w;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// Elementwise / skinny kernels (grouped over layers with blockIdx.y = layer in range).
// ---------------------------------------------------------------------------------------

// The forward epilogue for a layer whose prediction is cached (clamped input layer):
// no GEMM, preact/mu are read from memory.
__global__ void cached_forward_kernel(const dpc_layer* __restrict__ layers, int first,
                                      int n_layers, int batch, int flags, double* energy)
{
  const int li = first + blockIdx.y;
  const dpc_layer L = layers[li];
  const dpc_layer* Lup = (li + 1 < n_layers) ? &layers[li + 1] : nullptr;
  float esum = 0.0f;
  if (L.next_size > 0 && Lup)
  {
    const bool simple = (L.flags & DPC_LAYER_INPUT_ACT) != 0;
    const bool next_ce = (Lup->flags & DPC_LAYER_SOFTMAX_CE) != 0;
    const bool do_err = (flags & DPC_FWD_ERR_NEXT) && !next_ce;
    const bool do_fe = (flags & DPC_FWD_FE) && !simple && !(next_ce && (flags & DPC_FWD_ERR_NEXT));
    const bool do_copy = (flags & DPC_FWD_COPY_NEXT) != 0;
    const size_t total = (size_t)batch * L.next_size;
    for (size_t o = (size_t)blockIdx.x * blockDim.x + threadIdx.x; o < total;
         o += (size_t)gridDim.x * blockDim.x)
    {
      const float mu = L.mu[o];
      if (do_copy)
        Lup->z[o] = mu;
      float e = 0.0f;
      if (do_err)
      {
        e = (do_copy ? mu : Lup->z[o]) - mu;
        Lup->e[o] = e;
        esum += e * e;
      }
      else if (do_fe)
        e = Lup->e[o];
      if (do_fe)
        L.fe[o] = e * act_deriv(L.act, L.preact[o]);
    }
  }
  if (flags & DPC_FWD_ENERGY)
    block_energy_add(esum, energy);
}

// e = z - mu_below (+ energy), src/backend/CPUBackend.cpp:602-629.
__global__ void error_kernel(const dpc_layer* __restrict__ layers, int li, int batch,
                             int with_energy, double* energy)
{
  const dpc_layer L = layers[li];
  const dpc_layer Lb = layers[li - 1];
  const size_t total = (size_t)batch * L.size;
  float esum = 0.0f;
  for (size_t o = (size_t)blockIdx.x * blockDim.x + threadIdx.x; o < total;
       o += (size_t)gridDim.x * blockDim.x)
  {
    const float e = L.z[o] - Lb.mu[o];
    L.e[o] = e;
    esum += e * e;
  }
  if (with_energy)
    block_energy_add(esum, energy);
}

// Softmax cross-entropy error, one warp per batch row:
// e = z - softmax(mu_below), E = -sum z*log(p + 1e-8)   (CPUBackend.cpp:658-695).
__global__ void softmax_ce_kernel(const dpc_layer* __restrict__ layers, int li, int batch,
                                  int with_energy, double* energy)
{
  const dpc_layer L = layers[li];
  const float* mu = layers[li - 1].mu;
  const int n = L.size;
  const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
  float row_energy = 0.0f;
  for (int r = blockIdx.x * warps + (threadIdx.x >> 5); r < batch; r += gridDim.x * warps)
  {
    const float* mrow = mu + (size_t)r * n;
    const float* zrow = L.z + (size_t)r * n;
    float* erow = L.e + (size_t)r * n;
    float mx = -INFINITY;
    for (int j = lane; j < n; j += 32)
      mx = fmaxf(mx, mrow[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float s = 0.0f;
    for (int j = lane; j < n; j += 32)
      s += expf(mrow[j] - mx);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      s += __shfl_xor_sync(0xffffffffu, s, o);
    for (int j = lane; j < n; j += 32)
    {
      const float p = expf(mrow[j] - mx) / s;
      const float z = zrow[j];
      row_energy -= z * logf(p + 1e-8f);
      erow[j] = z - p;
    }
  }
  if (with_energy)
  {
    // block_energy_add halves its input (Gaussian energy); cross-entropy is not halved.
    block_energy_add(2.0f * row_energy, energy);
  }
}

// fe[l] = e[l+1] * f'(preact[l])
__global__ void feedback_error_kernel(const dpc_layer* __restrict__ layers, int first,
                                      int n_layers, int batch)
{
  const int li = first + blockIdx.y;
  if (li + 1 >= n_layers)
    return;
  const dpc_layer L = layers[li];
  if (L.next_size <= 0 || (L.flags & DPC_LAYER_INPUT_ACT))
    return;
  const float* e_up = layers[li + 1].e;
  const size_t total = (size_t)batch * L.next_size;
  for (size_t o = (size_t)blockIdx.x * blockDim.x + threadIdx.x; o < total;
       o += (size_t)gridDim.x * blockDim.x)
    L.fe[o] = e_up[o] * act_deriv(L.act, L.preact[o]);
}

// ePC: fe[l] = src * f'(preact[l]) with an explicit source (terminal error or adj[l+1]).
__global__ void epc_source_kernel(const dpc_layer* __restrict__ layers, int li, int batch,
                                  const float* __restrict__ src)
{
  const dpc_layer L = layers[li];
  const size_t total = (size_t)batch * L.next_size;
  for (size_t o = (size_t)blockIdx.x * blockDim.x + threadIdx.x; o < total;
       o += (size_t)gridDim.x * blockDim.x)
    L.fe[o] = src[o] * act_deriv(L.act, L.preact[o]);
}

// ePC: z[l] = mu[l-1] + e[l]   (src/layers/FullPCLayer.cpp:574-582)
__global__ void epc_reconstruct_kernel(const dpc_layer* __restrict__ layers, int li, int batch)
{
  const dpc_layer L = layers[li];
  const float* mu = layers[li - 1].mu;
  const size_t total = (size_t)batch * L.size;
  for (size_t o = (size_t)blockIdx.x * blockDim.x + threadIdx.x; o < total;
       o += (size_t)gridDim.x * blockDim.x)
    L.z[o] = mu[o] + L.e[o];
}

// z -= ir*e for layers of the range that have no weights or no upper neighbour.
__global__ void relax_kernel(const dpc_layer* __restrict__ layers, int first, int n_layers,
                             int batch, int only_weightless)
{
  const int li = first + blockIdx.y;
  const dpc_layer L = layers[li];
  if (only_weightless && L.next_size > 0 && li + 1 < n_layers)
    return;
  const size_t total = (size_t)batch * L.size;
  for (size_t o = (size_t)blockIdx.x * blockDim.x + threadIdx.x; o < total;
       o += (size_t)gridDim.x * blockDim.x)
    L.z[o] -= L.ir * L.e[o];
}

// DFA projection: fe[l] = (e_T · Psi[l+1]^T) * f'(preact[l])   (K = terminal_size).
// One thread per output unit j with its Psi row in registers; a block covers DFA_ROWS batch
// rows whose terminal errors sit in shared memory, so preact/fe stream through coalesced.
constexpr int DFA_ROWS = 32;
__global__ void dfa_proj_kernel(const dpc_layer* __restrict__ layers, int first, int n_layers,
                                int batch, const float* __restrict__ eT, int from_output)
{
  const int li = first + blockIdx.z;
  if (li + 1 >= n_layers)
    return;
  const dpc_layer L = layers[li];
  const dpc_layer Lup = layers[li + 1];
  if (L.next_size <= 0 || Lup.Psi == nullptr)
    return;
  const int TS = L.terminal_size, n = L.next_size;
  const int b0 = blockIdx.y * DFA_ROWS;
  if (b0 >= batch || (int)(blockIdx.x * blockDim.x) >= n)
    return;
  __shared__ __align__(16) float es[DFA_ROWS][16];
  for (int kc = 0; kc < TS; kc += 16)
  {
    const int kn = min(16, TS - kc);
    __syncthreads();
    for (int idx = threadIdx.x; idx < DFA_ROWS * 16; idx += blockDim.x)
    {
      const int r = idx >> 4, k = idx & 15;
      es[r][k] = (b0 + r < batch && k < kn) ? eT[(size_t)(b0 + r) * TS + kc + k] : 0.0f;
    }
    __syncthreads();
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j < n)
    {
      float psi[16];
      const float* pr = Lup.Psi + (size_t)j * Lup.psi_stride + kc;
#pragma unroll
      for (int k = 0; k < 16; ++k)
        psi[k] = k < kn ? pr[k] : 0.0f;
      const bool last = kc + 16 >= TS;
#pragma unroll 4
      for (int r = 0; r < DFA_ROWS; ++r)
      {
        if (b0 + r >= batch)
          break;
        float acc = 0.0f;
#pragma unroll
        for (int k4 = 0; k4 < 16; k4 += 4)
        {
          const float4 e4 = *reinterpret_cast<const float4*>(&es[r][k4]);
          acc = fmaf(e4.x, psi[k4], acc);
          acc = fmaf(e4.y, psi[k4 + 1], acc);
          acc = fmaf(e4.z, psi[k4 + 2], acc);
          acc = fmaf(e4.w, psi[k4 + 3], acc);
        }
        const size_t o = (size_t)(b0 + r) * n + j;
        if (kc > 0)
          acc += L.fe[o];
        if (last)
          acc *= (from_output && act_has_output_deriv(L.act))
                     ? act_deriv_from_output(L.act, Lup.z[o])
                     : act_deriv(L.act, L.preact[o]);
        L.fe[o] = acc;
      }
    }
  }
}

// The tensor-core path's bf16 "hi"/"mid" operand copies of the feedback errors of the layers
// [run_first, run_first + run_count): layer l has its hi plane at fe + 2 (l - run_first) * elems
// and its mid plane elems further on.  fe == NULL: no copies.  only != 0: the fp32 tensor of
// those layers is not kept at all (nothing reads it), the copies are the feedback error.
struct FePlanes
{
  __nv_bfloat16* fe;
  int run_first, run_count, only;
  long long elems;
};
__device__ __forceinline__ __nv_bfloat16* fe_plane_of(const FePlanes& P, int li)
{
  return (P.fe && li >= P.run_first && li < P.run_first + P.run_count)
             ? P.fe + 2 * (long long)(li - P.run_first) * P.elems
             : nullptr;
}

// The same projection, four output units per thread with 128-bit accesses, for the common
// Rows per block of the aligned kernel: its per-thread rows of Psi are strided 4-byte loads that
// cost as much L2 traffic as 32 rows of useful data, so a block amortises them over up to 128 rows
// (the host picks fewer when that would leave SMs without a block).
constexpr int DFA4_ROWS = 128;
// aligned case: next_size a multiple of 4, terminal_size <= 4*TS4, 16-byte aligned rows.
template <int TS4>
__global__ void __launch_bounds__(64)
    dfa_proj4_kernel(const dpc_layer* __restrict__ layers, int first, int n_layers, int batch,
                     const float* __restrict__ eT, int from_output, int rows_per_block,
                     FePlanes planes)
{
  const int li = first + blockIdx.z;
  if (li + 1 >= n_layers)
    return;
  const dpc_layer L = layers[li];
  const dpc_layer Lup = layers[li + 1];
  if (L.next_size <= 0 || Lup.Psi == nullptr)
    return;
  const int TS = L.terminal_size, n = L.next_size;
  const int b0 = blockIdx.y * rows_per_block; // rows_per_block <= DFA4_ROWS
  const int j = (blockIdx.x * 64 + threadIdx.x) * 4;
  if (b0 >= batch || (int)(blockIdx.x * 256) >= n)
    return;
  __shared__ __align__(16) float es[DFA4_ROWS][TS4 * 4];
  for (int idx = threadIdx.x; idx < rows_per_block * TS4 * 4; idx += 64)
  {
    const int r = idx / (TS4 * 4), k = idx - r * (TS4 * 4);
    es[r][k] = (b0 + r < batch && k < TS) ? eT[(size_t)(b0 + r) * TS + k] : 0.0f;
  }
  __syncthreads();
  if (j >= n)
    return;
  float psi[4][TS4 * 4];
#pragma unroll
  for (int c = 0; c < 4; ++c)
#pragma unroll
    for (int k = 0; k < TS4 * 4; ++k)
      psi[c][k] = k < TS ? Lup.Psi[(size_t)(j + c) * Lup.psi_stride + k] : 0.0f;
  const bool out_d = from_output && act_has_output_deriv(L.act);
  const float* src = out_d ? Lup.z : L.preact;
  const int rows = min(rows_per_block, batch - b0);
  __nv_bfloat16* hi = fe_plane_of(planes, li);
  const bool keep_fp32 = !(hi && planes.only);
#pragma unroll 8
  for (int r = 0; r < rows; ++r)
  {
    const size_t o = (size_t)(b0 + r) * n + j;
    const float4 s4 = *reinterpret_cast<const float4*>(src + o);
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int k4 = 0; k4 < TS4; ++k4)
    {
      const float4 e4 = *reinterpret_cast<const float4*>(&es[r][k4 * 4]);
#pragma unroll
      for (int c = 0; c < 4; ++c)
      {
        acc[c] = fmaf(e4.x, psi[c][k4 * 4], acc[c]);
        acc[c] = fmaf(e4.y, psi[c][k4 * 4 + 1], acc[c]);
        acc[c] = fmaf(e4.z, psi[c][k4 * 4 + 2], acc[c]);
        acc[c] = fmaf(e4.w, psi[c][k4 * 4 + 3], acc[c]);
      }
    }
    const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
    float out[4];
#pragma unroll
    for (int c = 0; c < 4; ++c)
      out[c] = acc[c] * (out_d ? act_deriv_from_output(L.act, sv[c]) : act_deriv(L.act, sv[c]));
    if (keep_fp32)
      *reinterpret_cast<float4*>(L.fe + o) = make_float4(out[0], out[1], out[2], out[3]);
    if (hi)
    {
      const __nv_bfloat162 h0 = __floats2bfloat162_rn(out[0], out[1]);
      const __nv_bfloat162 h1 = __floats2bfloat162_rn(out[2], out[3]);
      const __nv_bfloat162 m0 =
          __floats2bfloat162_rn(out[0] - __low2float(h0), out[1] - __high2float(h0));
      const __nv_bfloat162 m1 =
          __floats2bfloat162_rn(out[2] - __low2float(h1), out[3] - __high2float(h1));
      uint2 hv, mv;
      hv.x = *reinterpret_cast<const uint32_t*>(&h0), hv.y = *reinterpret_cast<const uint32_t*>(&h1);
      mv.x = *reinterpret_cast<const uint32_t*>(&m0), mv.y = *reinterpret_cast<const uint32_t*>(&m1);
      *reinterpret_cast<uint2*>(hi + o) = hv;
      *reinterpret_cast<uint2*>(hi + planes.elems + o) = mv;
    }
  }
}

// The aligned projection for wide layers (next_size a multiple of 128) when there are enough
// layers to fill the GPU with blocks of 128 columns x the whole batch: the 128 rows of Psi a
// block needs come in through shared memory with coalesced loads ONCE per block (the kernel above
// re-reads them with strided loads for every 128 batch rows), lane l of every warp owns columns
// 4l..4l+3, warp w the batch rows w, w+8, ...: every access of a warp is one whole row segment.
template <int TS4>
__global__ void __launch_bounds__(256)
    dfa_proj128_kernel(const dpc_layer* __restrict__ layers, int first, int n_layers, int batch,
                       const float* __restrict__ eT, int from_output, FePlanes planes)
{
  const int li = first + blockIdx.y;
  if (li + 1 >= n_layers)
    return;
  const dpc_layer L = layers[li];
  const dpc_layer Lup = layers[li + 1];
  if (L.next_size <= 0 || Lup.Psi == nullptr)
    return;
  const int TS = L.terminal_size, n = L.next_size;
  const int j0 = blockIdx.x * 128;
  if (j0 >= n)
    return;
  constexpr int KC = TS4 * 4, ROWS = 128;
  __shared__ __align__(16) float es[ROWS][KC];
  __shared__ float ps[128][KC + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int idx = threadIdx.x; idx < 128 * KC; idx += 256)
  {
    const int r = idx / KC, k = idx - r * KC;
    ps[r][k] = k < TS ? Lup.Psi[(size_t)(j0 + r) * Lup.psi_stride + k] : 0.0f;
  }
  __syncthreads();
  float psi[4][KC];
#pragma unroll
  for (int c = 0; c < 4; ++c)
#pragma unroll
    for (int k = 0; k < KC; ++k)
      psi[c][k] = ps[4 * lane + c][k];
  const bool out_d = from_output && act_has_output_deriv(L.act);
  const float* src = out_d ? Lup.z : L.preact;
  __nv_bfloat16* hi = fe_plane_of(planes, li);
  const bool keep_fp32 = !(hi && planes.only);
  const int j = j0 + 4 * lane;
  for (int b0 = 0; b0 < batch; b0 += ROWS)
  {
    __syncthreads();
    for (int idx = threadIdx.x; idx < ROWS * KC; idx += 256)
    {
      const int r = idx / KC, k = idx - r * KC;
      es[r][k] = (b0 + r < batch && k < TS) ? eT[(size_t)(b0 + r) * TS + k] : 0.0f;
    }
    __syncthreads();
    const int rows = min(ROWS, batch - b0);
#pragma unroll 4
    for (int r = warp; r < rows; r += 8)
    {
      const size_t o = (size_t)(b0 + r) * n + j;
      const float4 s4 = *reinterpret_cast<const float4*>(src + o);
      float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int k4 = 0; k4 < TS4; ++k4)
      {
        const float4 e4 = *reinterpret_cast<const float4*>(&es[r][k4 * 4]);
#pragma unroll
        for (int c = 0; c < 4; ++c)
        {
          acc[c] = fmaf(e4.x, psi[c][k4 * 4], acc[c]);
          acc[c] = fmaf(e4.y, psi[c][k4 * 4 + 1], acc[c]);
          acc[c] = fmaf(e4.z, psi[c][k4 * 4 + 2], acc[c]);
          acc[c] = fmaf(e4.w, psi[c][k4 * 4 + 3], acc[c]);
        }
      }
      const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
      float out[4];
#pragma unroll
      for (int c = 0; c < 4; ++c)
        out[c] = acc[c] * (out_d ? act_deriv_from_output(L.act, sv[c]) : act_deriv(L.act, sv[c]));
      if (keep_fp32)
        *reinterpret_cast<float4*>(L.fe + o) = make_float4(out[0], out[1], out[2], out[3]);
      if (hi)
      {
        const __nv_bfloat162 h0 = __floats2bfloat162_rn(out[0], out[1]);
        const __nv_bfloat162 h1 = __floats2bfloat162_rn(out[2], out[3]);
        const __nv_bfloat162 m0 =
            __floats2bfloat162_rn(out[0] - __low2float(h0), out[1] - __high2float(h0));
        const __nv_bfloat162 m1 =
            __floats2bfloat162_rn(out[2] - __low2float(h1), out[3] - __high2float(h1));
        uint2 hv, mv;
        hv.x = *reinterpret_cast<const uint32_t*>(&h0), hv.y = *reinterpret_cast<const uint32_t*>(&h1);
        mv.x = *reinterpret_cast<const uint32_t*>(&m0), mv.y = *reinterpret_cast<const uint32_t*>(&m1);
        *reinterpret_cast<uint2*>(hi + o) = hv;
        *reinterpret_cast<uint2*>(hi + planes.elems + o) = mv;
      }
    }
  }
}

// Adam step counters: t += 1 once per UpdateWeights (src/backend/cuda/CUDABackendOptimizer.cu:20-31).
__global__ void bump_counters_kernel(const dpc_layer* __restrict__ layers, int first, int count,
                                     int n_layers)
{
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count)
    return;
  const int li = first + i;
  const dpc_layer L = layers[li];
  if (L.next_size <= 0 || li + 1 >= n_layers)
    return;
  if (L.opt != DPC_OPT_SGD && L.t)
    *L.t += 1;
  if (!(L.flags & DPC_LAYER_INPUT_ACT) && L.opt_psi != DPC_OPT_SGD && L.t_Psi)
    *L.t_Psi += 1;
}

// b (+)= rate * s for one output unit (or s into the staging buffer): what follows the column sum.
__device__ __forceinline__ void bias_apply(const dpc_layer& L, int j, float s, int batch, int grad_only)
{
  if (grad_only)
    L.g_b[j] = s;
  else if (L.opt == DPC_OPT_SGD)
    L.b[j] += (L.lr / (float)batch) * s;
  else
  {
    float m = L.m_b[j], v = L.v_b[j];
    L.b[j] = adam_update(L.b[j], -s, m, v, adam_step_size(L.lr, *L.t), -1.0f);
    L.m_b[j] = m;
    L.v_b[j] = v;
  }
}

// Bias update from the column sums of the local gradient: one thread per output unit,
// summing the batch in row order like CPUBackend::SumRows (CPUBackend.cpp:243-248).
// Layers whose feedback error exists only as bf16 planes (see FePlanes) are summed by whole
// blocks instead: 32 row groups x 8 threads of 8 columns each (16-byte loads of both planes,
// hi + mid = fe to 2^-17), then a fixed-order reduction over the row groups in shared memory.
constexpr int kBiasBlockRows = 256;
__global__ void bias_update_kernel(const dpc_layer* __restrict__ layers, int first, int n_layers,
                                   int batch, int grad_only, FePlanes planes)
{
  const int li = first + blockIdx.y;
  if (li + 1 >= n_layers)
    return;
  const dpc_layer L = layers[li];
  if (L.next_size <= 0)
    return;
  const bool simple = (L.flags & DPC_LAYER_INPUT_ACT) != 0;
  const float* g = simple ? layers[li + 1].e : L.fe;
  const int n = L.next_size;
  const __nv_bfloat16* hi = (!simple && planes.only) ? fe_plane_of(planes, li) : nullptr;
  // Summed by whole blocks: the plane-only layers, and fp32 gradients of large batches (the
  // one-thread-per-column loop below keeps the reference's row order for the small cases).
  const bool wide = n % 64 == 0 && blockDim.x == 256 &&
                    (hi || (batch >= kBiasBlockRows && ((uintptr_t)g % 16) == 0));
  const uint32_t R = rows_cluster_size(), rank = rows_cluster_rank();
  if (wide)
  {
    __shared__ float part[32][65];
    __shared__ float mine[64];
    const int rg = threadIdx.x >> 3, c8 = (threadIdx.x & 7) * 8;
    for (int j0 = blockIdx.x * 64; j0 < n; j0 += gridDim.x * 64)
    {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (hi)
      {
        for (int b = rg + 32 * (int)rank; b < batch; b += 32 * (int)R)
        {
          const size_t o = (size_t)b * n + j0 + c8;
          const uint4 h = *reinterpret_cast<const uint4*>(hi + o);
          const uint4 m = *reinterpret_cast<const uint4*>(hi + planes.elems + o);
          const uint32_t hw[4] = {h.x, h.y, h.z, h.w}, mw[4] = {m.x, m.y, m.z, m.w};
#pragma unroll
          for (int q = 0; q < 4; ++q)
          {
            // a bf16 is the upper half of the fp32 with the same value
            acc[2 * q] += __uint_as_float(hw[q] << 16) + __uint_as_float(mw[q] << 16);
            acc[2 * q + 1] += __uint_as_float(hw[q] & 0xffff0000u) + __uint_as_float(mw[q] & 0xffff0000u);
          }
        }
      }
      else
      {
#pragma unroll 4
        for (int b = rg + 32 * (int)rank; b < batch; b += 32 * (int)R)
        {
          const size_t o = (size_t)b * n + j0 + c8;
          const float4 x = *reinterpret_cast<const float4*>(g + o);
          const float4 y = *reinterpret_cast<const float4*>(g + o + 4);
          acc[0] += x.x, acc[1] += x.y, acc[2] += x.z, acc[3] += x.w;
          acc[4] += y.x, acc[5] += y.y, acc[6] += y.z, acc[7] += y.w;
        }
      }
      __syncthreads();
#pragma unroll
      for (int q = 0; q < 8; ++q)
        part[rg][c8 + q] = acc[q];
      __syncthreads();
      float s = 0.0f;
      if (threadIdx.x < 64)
      {
        for (int r = 0; r < 32; ++r)
          s += part[r][threadIdx.x];
        if (R > 1 && rank != 0)
          mine[threadIdx.x] = s;
      }
      if (R > 1)
      {
        rows_cluster_sync();
        if (rank == 0 && threadIdx.x < 64)
          for (uint32_t r = 1; r < R; ++r)
            s += rows_cluster_load(&mine[threadIdx.x], r);
        rows_cluster_sync(); // `mine` of the other CTAs may be rewritten (or go away) only now
      }
      if (threadIdx.x < 64 && rank == 0)
        bias_apply(L, j0 + threadIdx.x, s, batch, grad_only);
    }
    return;
  }
  if (rank != 0)
    return; // (a row-split launch over a layer that takes the column loop: one CTA does it all)
  for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < n; j += gridDim.x * blockDim.x)
  {
    float s = 0.0f;
    if (hi)
      for (int b = 0; b < batch; ++b)
        s += __bfloat162float(hi[(size_t)b * n + j]) +
             __bfloat162float(hi[planes.elems + (size_t)b * n + j]);
    else
      for (int b = 0; b < batch; ++b)
        s += g[(size_t)b * n + j];
    bias_apply(L, j, s, batch, grad_only);
  }
}

// One entry of the feedback-weight update: Psi[row][k] takes the raw sum over the batch of
// z[b][row] * e_T[b][k] (SGD with optional decay, Adam, AdamW, or the sum itself into g_Psi).
__device__ __forceinline__ void psi_apply(const dpc_layer& L, int row, int k, float sum, int batch,
                                          int grad_only, bool full_kind, float rate)
{
  const size_t o = (size_t)row * L.psi_stride + k;
  if (grad_only)
    L.g_Psi[o] = sum;
  else if (L.opt_psi == DPC_OPT_SGD)
  {
    const float decay = (!full_kind && L.psi_decay > 0.0f) ? 1.0f - L.psi_decay : 1.0f;
    float p = L.Psi[o];
    if (decay != 1.0f)
      p *= decay;
    L.Psi[o] = fmaf(rate / (float)batch, sum, p);
  }
  else
  {
    const float step = adam_step_size(rate, *L.t_Psi);
    float lr_wd = -1.0f;
    if (L.opt_psi == DPC_OPT_ADAMW)
      lr_wd = rate * ((!full_kind && L.psi_decay >= 0.0f) ? L.psi_decay : L.lmbda);
    float m = L.m_Psi[o], v = L.v_Psi[o];
    L.Psi[o] = adam_update(L.Psi[o], -sum, m, v, step, lr_wd);
    L.m_Psi[o] = m;
    L.v_Psi[o] = v;
  }
}

// sum over the batch of zin[b][col + c] * g[b][k] for c < 4, k < KC: the common core of the Psi
// update and of the weight update of a narrow layer.  A block owns 128 columns of zin, lane l of
// every warp the columns 4l..4l+3 (one 16-byte load per batch row: a warp reads a whole 512-byte row
// segment), warp w the batch rows w, w+8, ...; the rows of g (at most KC wide, ldg apart) of 128
// batch rows at a time sit in shared memory.  The eight warps' partial sums are added in a fixed
// tree order through shared memory, then the CTAs of a row-split cluster in rank order.  Returns
// true in the threads that end up with the sums (warp 0 of CTA 0 of the cluster).
// (Measured alternatives, both slower: two columns per lane at twice the blocks per SM, and the
// rows of g of the whole batch in shared memory so that the row loop has no barrier.)
template <int KC>
__device__ __forceinline__ bool batch_outer4(const float* __restrict__ zin, int s, int col,
                                             const float* __restrict__ g, int ldg, int TS,
                                             int batch, float (&acc)[4][KC], float (*es)[KC],
                                             float (*part)[4 * KC][32])
{
  constexpr int ROWS = 128;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int c = 0; c < 4; ++c)
#pragma unroll
    for (int k = 0; k < KC; ++k)
      acc[c][k] = 0.0f;
  const uint32_t R = rows_cluster_size(), rank = rows_cluster_rank();
  for (int b0 = (int)rank * ROWS; b0 < batch; b0 += (int)R * ROWS)
  {
    __syncthreads();
    for (int idx = threadIdx.x; idx < ROWS * KC; idx += 256)
    {
      const int r = idx / KC, k = idx - r * KC;
      es[r][k] = (b0 + r < batch && k < TS) ? g[(size_t)(b0 + r) * ldg + k] : 0.0f;
    }
    __syncthreads();
    const int rows = min(ROWS, batch - b0);
#pragma unroll 4
    for (int r = warp; r < rows; r += 8)
    {
      const float4 z4 = *reinterpret_cast<const float4*>(zin + (size_t)(b0 + r) * s + col);
      const float zv[4] = {z4.x, z4.y, z4.z, z4.w};
#pragma unroll
      for (int k4 = 0; k4 < KC; k4 += 4)
      {
        const float4 e4 = *reinterpret_cast<const float4*>(&es[r][k4]);
#pragma unroll
        for (int c = 0; c < 4; ++c)
        {
          acc[c][k4] = fmaf(zv[c], e4.x, acc[c][k4]);
          acc[c][k4 + 1] = fmaf(zv[c], e4.y, acc[c][k4 + 1]);
          acc[c][k4 + 2] = fmaf(zv[c], e4.z, acc[c][k4 + 2]);
          acc[c][k4 + 3] = fmaf(zv[c], e4.w, acc[c][k4 + 3]);
        }
      }
    }
  }
  // tree over the warps: (w, w+4), then (w, w+2), then (0, 1)
#pragma unroll
  for (int half = 4; half >= 1; half >>= 1)
  {
    __syncthreads();
    if (warp >= half && warp < 2 * half)
    {
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int k = 0; k < KC; ++k)
          part[warp - half][c * KC + k][lane] = acc[c][k];
    }
    __syncthreads();
    if (warp < half)
    {
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int k = 0; k < KC; ++k)
          acc[c][k] += part[warp][c * KC + k][lane];
    }
  }
  if (R > 1)
  {
    // (part[0] was last read by this same warp 0 in the tree above)
    if (rank != 0 && warp == 0)
    {
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int k = 0; k < KC; ++k)
          part[0][c * KC + k][lane] = acc[c][k];
    }
    rows_cluster_sync();
    if (rank == 0 && warp == 0)
    {
      for (uint32_t r = 1; r < R; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int k = 0; k < KC; ++k)
            acc[c][k] += rows_cluster_load(&part[0][c * KC + k][lane], r);
    }
    rows_cluster_sync(); // nobody leaves while CTA 0 may still read its shared memory
  }
  return rank == 0 && warp == 0;
}

// The Psi update for the common aligned case (layer width a multiple of 128, at most KC terminal
// units, KC = 12 or 16): a block owns 128 rows of Psi (= 128 columns of z).
template <int KC>
__global__ void __launch_bounds__(256)
    psi_update4_kernel(const dpc_layer* __restrict__ layers, int first, int n_layers, int batch,
                       const float* __restrict__ eT, int grad_only)
{
  const int li = first + blockIdx.y;
  if (li + 1 >= n_layers)
    return;
  const dpc_layer L = layers[li];
  if (L.next_size <= 0 || L.Psi == nullptr || (L.flags & DPC_LAYER_INPUT_ACT))
    return;
  const int TS = L.terminal_size, s = L.size;
  const bool full_kind = (L.flags & DPC_LAYER_FULLPC_PSI) != 0;
  const float rate = full_kind ? L.fl * L.a : L.fl;
  if ((int)blockIdx.x * 128 >= s)
    return;
  __shared__ __align__(16) float es[128][KC];
  __shared__ float part[4][4 * KC][32];
  const int col = blockIdx.x * 128 + (threadIdx.x & 31) * 4;
  float acc[4][KC];
  if (!batch_outer4<KC>(L.z, s, col, eT, TS, TS, batch, acc, es, part))
    return;
#pragma unroll
  for (int c = 0; c < 4; ++c)
#pragma unroll
    for (int k = 0; k < KC; ++k)
      if (k < TS)
        psi_apply(L, col + c, k, acc[c][k], batch, grad_only, full_kind, rate);
}

// State update of a layer below a narrow one (at most KC <= 16 units above, own width a multiple of
// 128: the layer under a head, e.g. z[4096 x 1024] += ir (a fe[4096 x 10] W[10 x 1024] - e)).  The
// product has a K of 10: the tiled kernel spends its time on tile bookkeeping.  Here lane l of
// every warp keeps the weights of columns 4l..4l+3 in registers, a block owns 128 columns and
// `rows_per_block` batch rows, warp w the rows w, w+8, ...; the rows of the feedback error go
// through shared memory 128 at a time.  Same arithmetic per element as pc_gemm_kernel<OP_FB>.
template <int KC>
__global__ void __launch_bounds__(256)
    narrow_state_kernel(const dpc_layer* __restrict__ layers, int first, int n_layers, int batch,
                        int rows_per_block)
{
  const int li = first + blockIdx.z;
  if (li + 1 >= n_layers)
    return;
  const dpc_layer L = layers[li];
  if (L.next_size <= 0)
    return;
  const dpc_layer* Lup = &layers[li + 1];
  const bool simple = (L.flags & DPC_LAYER_INPUT_ACT) != 0;
  const bool residual = (L.flags & DPC_LAYER_RESIDUAL) != 0;
  const int K = L.next_size, s = L.size;
  if ((int)blockIdx.x * 128 >= s)
    return;
  const float* g = simple ? Lup->e : L.fe;
  constexpr int ROWS = 128;
  __shared__ __align__(16) float gs[ROWS][KC];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = blockIdx.x * 128 + lane * 4;
  float w[4][KC];
#pragma unroll
  for (int k = 0; k < KC; ++k)
  {
    float4 w4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (k < K)
      w4 = *reinterpret_cast<const float4*>(L.W + (size_t)k * s + col);
    w[0][k] = w4.x, w[1][k] = w4.y, w[2][k] = w4.z, w[3][k] = w4.w;
  }
  const int b_begin = blockIdx.y * rows_per_block;
  const int b_end = min(batch, b_begin + rows_per_block);
  for (int b0 = b_begin; b0 < b_end; b0 += ROWS)
  {
    __syncthreads();
    for (int idx = threadIdx.x; idx < ROWS * KC; idx += 256)
    {
      const int r = idx / KC, k = idx - r * KC;
      gs[r][k] = (b0 + r < b_end && k < K) ? g[(size_t)(b0 + r) * K + k] : 0.0f;
    }
    __syncthreads();
    const int rows = min(ROWS, b_end - b0);
#pragma unroll 2
    for (int r = warp; r < rows; r += 8)
    {
      const size_t o = (size_t)(b0 + r) * s + col;
      const float4 e4 = *reinterpret_cast<const float4*>(L.e + o);
      const float4 z4 = *reinterpret_cast<const float4*>(L.z + o);
      float4 v4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f), u4 = v4;
      if (!simple && L.v)
        v4 = *reinterpret_cast<const float4*>(L.v + o);
      if (!simple && residual)
        u4 = *reinterpret_cast<const float4*>(Lup->e + o);
      float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int k4 = 0; k4 < KC; k4 += 4)
      {
        const float4 g4 = *reinterpret_cast<const float4*>(&gs[r][k4]);
#pragma unroll
        for (int c = 0; c < 4; ++c)
        {
          acc[c] = fmaf(g4.x, w[c][k4], acc[c]);
          acc[c] = fmaf(g4.y, w[c][k4 + 1], acc[c]);
          acc[c] = fmaf(g4.z, w[c][k4 + 2], acc[c]);
          acc[c] = fmaf(g4.w, w[c][k4 + 3], acc[c]);
        }
      }
      float zz[4] = {z4.x, z4.y, z4.z, z4.w};
      const float ee[4] = {e4.x, e4.y, e4.z, e4.w};
      float vv[4] = {v4.x, v4.y, v4.z, v4.w};
      const float uu[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
      for (int c = 0; c < 4; ++c)
      {
        if (simple)
          zz[c] += L.ir * (acc[c] * act_deriv(L.act, zz[c]) - ee[c]);
        else
        {
          const float fb = L.a * acc[c] - ee[c];
          if (L.v)
          {
            vv[c] = L.momentum_beta * vv[c] + (1.0f - L.momentum_beta) * fb;
            zz[c] += L.ir * vv[c];
          }
          else
            zz[c] += L.ir * fb;
          if (residual)
            zz[c] += L.ir * uu[c];
        }
      }
      if (!simple && L.v)
        *reinterpret_cast<float4*>(L.v + o) = make_float4(vv[0], vv[1], vv[2], vv[3]);
      *reinterpret_cast<float4*>(L.z + o) = make_float4(zz[0], zz[1], zz[2], zz[3]);
    }
  }
}

// One entry of a weight update from the raw sum over the batch (the epilogue of
// pc_gemm_kernel<OP_WG> for one element).
__device__ __forceinline__ void weight_apply(const dpc_layer& L, size_t o, float sum, int batch,
                                             int mode, int flags, bool simple)
{
  if (mode & WG_GRAD_ONLY)
  {
    L.g_W[o] = sum;
    return;
  }
  const float Bf = (float)batch;
  float w = L.W[o];
  if (mode == WG_LEARN && L.opt != DPC_OPT_SGD)
  {
    float lr_wd = -1.0f;
    if (L.opt == DPC_OPT_ADAMW)
      lr_wd = L.lr * L.lmbda;
    float mm = L.m_W[o], vv = L.v_W[o];
    w = adam_update(w, -1.0f * L.a * sum, mm, vv, adam_step_size(L.lr, *L.t), lr_wd);
    L.m_W[o] = mm;
    L.v_W[o] = vv;
  }
  else
  {
    float alpha, decay = 1.0f;
    if (mode == WG_DFA)
    {
      alpha = L.fl * L.a / Bf;
      if ((flags & 1) && L.lmbda > 0.0f && L.fl != 0.0f)
        decay = 1.0f - L.lmbda;
    }
    else
    {
      alpha = simple ? (L.lr / Bf) : (L.a * L.lr / Bf);
      if (L.lmbda > 0.0f)
        decay = 1.0f - L.lmbda;
    }
    if (decay != 1.0f)
      w *= decay;
    w = fmaf(alpha, sum, w);
  }
  L.W[o] = w;
}

// Weight update of a narrow layer (at most KC <= 16 output units, input width a multiple of 128:
// the heads, e.g. W[10 x 1024] += alpha fe^T z over a batch of 4096).  The tiled kernel gives such
// a layer size/64 blocks that each walk the whole batch; here the batch is split over warps and
// over the CTAs of a cluster as in the Psi update, whose shape this product shares.
template <int KC>
__global__ void __launch_bounds__(256)
    narrow_weight_kernel(const dpc_layer* __restrict__ layers, int first, int n_layers, int batch,
                         int flags, int mode)
{
  const int li = first + blockIdx.y;
  const dpc_layer L = layers[li];
  if (L.next_size <= 0)
    return;
  const bool simple = (L.flags & DPC_LAYER_INPUT_ACT) != 0;
  const int base_mode = mode & ~WG_GRAD_ONLY;
  if (base_mode == WG_DFA && (li + 1 >= n_layers || layers[li + 1].Psi == nullptr))
    return; // DirectFeedbackUpdate is a no-op unless the layer above owns feedback weights
  const int M = L.next_size, s = L.size;
  if ((int)blockIdx.x * 128 >= s)
    return;
  const float* g = (simple && base_mode == WG_LEARN) ? layers[li + 1].e : L.fe;
  const float* zin = simple ? L.zF : L.z;
  __shared__ __align__(16) float es[128][KC];
  __shared__ float part[4][4 * KC][32];
  const int col = blockIdx.x * 128 + (threadIdx.x & 31) * 4;
  float acc[4][KC];
  if (!batch_outer4<KC>(zin, s, col, g, M, M, batch, acc, es, part))
    return;
#pragma unroll
  for (int c = 0; c < 4; ++c)
#pragma unroll
    for (int k = 0; k < KC; ++k)
      if (k < M)
        weight_apply(L, (size_t)k * s + col + c, acc[c][k], batch, mode, flags, simple);
}

// Feedback-weight update Psi[l] (+)= (fl*a/B) z[l]^T e_T.  A block of 256 threads owns 64 rows of
// Psi (= 64 columns of z): thread (g, i) adds up the batch rows b = g, g+4, ... for column i with
// the terminal columns in registers (chunks of 16), the four row groups are then summed in a
// fixed order through shared memory.  The terminal errors of PSI_ROWS batch rows at a time go
// through shared memory (zero padded to 16 columns).
__global__ void __launch_bounds__(256)
    psi_update_kernel(const dpc_layer* __restrict__ layers, int first, int n_layers, int batch,
                      const float* __restrict__ eT, int grad_only)
{
  const int li = first + blockIdx.y;
  if (li + 1 >= n_layers)
    return;
  const dpc_layer L = layers[li];
  if (L.next_size <= 0 || L.Psi == nullptr || (L.flags & DPC_LAYER_INPUT_ACT))
    return;
  const int TS = L.terminal_size, s = L.size;
  const bool full_kind = (L.flags & DPC_LAYER_FULLPC_PSI) != 0;
  const float rate = full_kind ? L.fl * L.a : L.fl;
  constexpr int PSI_ROWS = 64, GROUPS = 4, COLS = 64;
  __shared__ __align__(16) float es[PSI_ROWS][16];
  __shared__ float part[GROUPS][COLS][17];
  const int g = threadIdx.x >> 6, ci = threadIdx.x & 63;
  for (int i0 = blockIdx.x * COLS; i0 < s; i0 += gridDim.x * COLS)
  {
    const int i = i0 + ci;
    for (int kc = 0; kc < TS; kc += 16)
    {
      float acc[16];
#pragma unroll
      for (int k = 0; k < 16; ++k)
        acc[k] = 0.0f;
      const int kn = min(16, TS - kc);
      for (int b0 = 0; b0 < batch; b0 += PSI_ROWS)
      {
        __syncthreads();
        for (int idx = threadIdx.x; idx < PSI_ROWS * 16; idx += blockDim.x)
        {
          const int r = idx >> 4, k = idx & 15;
          es[r][k] = (b0 + r < batch && k < kn) ? eT[(size_t)(b0 + r) * TS + kc + k] : 0.0f;
        }
        __syncthreads();
        if (i < s)
        {
          const int rows = min(PSI_ROWS, batch - b0);
#pragma unroll 4
          for (int r = g; r < rows; r += GROUPS)
          {
            const float zv = L.z[(size_t)(b0 + r) * s + i];
#pragma unroll
            for (int k4 = 0; k4 < 16; k4 += 4)
            {
              const float4 e4 = *reinterpret_cast<const float4*>(&es[r][k4]);
              acc[k4] = fmaf(zv, e4.x, acc[k4]);
              acc[k4 + 1] = fmaf(zv, e4.y, acc[k4 + 1]);
              acc[k4 + 2] = fmaf(zv, e4.z, acc[k4 + 2]);
              acc[k4 + 3] = fmaf(zv, e4.w, acc[k4 + 3]);
            }
          }
        }
      }
#pragma unroll
      for (int k = 0; k < 16; ++k)
        part[g][ci][k] = acc[k];
      __syncthreads();
      // thread t < 64 * 4: column t / 4, terminal columns 4 (t % 4) .. +3
      const int rc = threadIdx.x >> 2, k0 = (threadIdx.x & 3) * 4, row = i0 + rc;
      if (row < s)
      {
#pragma unroll
        for (int q = 0; q < 4; ++q)
        {
          const int k = k0 + q;
          if (k >= kn)
            continue;
          const float sum = ((part[0][rc][k] + part[1][rc][k]) + part[2][rc][k]) + part[3][rc][k];
          psi_apply(L, row, kc + k, sum, batch, grad_only, full_kind, rate);
        }
      }
      __syncthreads();
    }
  }
}

// Applies staged gradients (the raw sums that the WG_GRAD_ONLY weight kernel and the grad_only
// bias / Psi kernels left in g_W, g_b, g_Psi, possibly summed over batch shards since) with
// exactly the formulas of the fused updates above; `batch` is the batch the sums cover (the
// global one).  which = WG_LEARN: W, b and Psi; WG_DFA: W only (DirectFeedbackUpdate);
// 2: W only with the learn-step formulas (b and Psi are updated by their own fused kernels).
__global__ void apply_gradients_kernel(const dpc_layer* __restrict__ layers, int first,
                                       int n_layers, int batch, int which, int flags)
{
  const int li = first + blockIdx.y;
  if (li + 1 >= n_layers)
    return;
  const dpc_layer L = layers[li];
  if (L.next_size <= 0)
    return;
  const bool simple = (L.flags & DPC_LAYER_INPUT_ACT) != 0;
  const float Bf = (float)batch;
  const size_t nW = (size_t)L.next_size * L.size;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t nthr = (size_t)gridDim.x * blockDim.x;
  if (which == WG_DFA)
  {
    if (layers[li + 1].Psi == nullptr)
      return;
    const float alpha = L.fl * L.a / Bf;
    const float decay = ((flags & 1) && L.lmbda > 0.0f && L.fl != 0.0f) ? 1.0f - L.lmbda : 1.0f;
    for (size_t o = tid; o < nW; o += nthr)
    {
      float w = L.W[o];
      if (decay != 1.0f)
        w *= decay;
      L.W[o] = fmaf(alpha, L.g_W[o], w);
    }
    return;
  }
  if (L.opt == DPC_OPT_SGD)
  {
    const float alpha = simple ? (L.lr / Bf) : (L.a * L.lr / Bf);
    const float decay = L.lmbda > 0.0f ? 1.0f - L.lmbda : 1.0f;
    for (size_t o = tid; o < nW; o += nthr)
    {
      float w = L.W[o];
      if (decay != 1.0f)
        w *= decay;
      L.W[o] = fmaf(alpha, L.g_W[o], w);
    }
    if (which != 2)
      for (size_t j = tid; j < (size_t)L.next_size; j += nthr)
        L.b[j] += (L.lr / Bf) * L.g_b[j];
  }
  else
  {
    const float step = adam_step_size(L.lr, *L.t);
    const float lr_wd = L.opt == DPC_OPT_ADAMW ? L.lr * L.lmbda : -1.0f;
    const float alpha = -1.0f * L.a;
    for (size_t o = tid; o < nW; o += nthr)
    {
      float mm = L.m_W[o], vv = L.v_W[o];
      L.W[o] = adam_update(L.W[o], alpha * L.g_W[o], mm, vv, step, lr_wd);
      L.m_W[o] = mm;
      L.v_W[o] = vv;
    }
    if (which != 2)
      for (size_t j = tid; j < (size_t)L.next_size; j += nthr)
      {
        float m = L.m_b[j], v = L.v_b[j];
        L.b[j] = adam_update(L.b[j], -L.g_b[j], m, v, step, -1.0f);
        L.m_b[j] = m;
        L.v_b[j] = v;
      }
  }
  if (L.Psi == nullptr || simple || which == 2)
    return;
  const bool full_kind = (L.flags & DPC_LAYER_FULLPC_PSI) != 0;
  const float rate = full_kind ? L.fl * L.a : L.fl;
  const int TS = L.terminal_size;
  const size_t nP = (size_t)L.size * TS;
  if (L.opt_psi == DPC_OPT_SGD)
  {
    const float decay = (!full_kind && L.psi_decay > 0.0f) ? 1.0f - L.psi_decay : 1.0f;
    const float alpha = rate / Bf;
    for (size_t q = tid; q < nP; q += nthr)
    {
      const size_t o = (q / TS) * L.psi_stride + q % TS;
      float p = L.Psi[o];
      if (decay != 1.0f)
        p *= decay;
      L.Psi[o] = fmaf(alpha, L.g_Psi[o], p);
    }
  }
  else
  {
    const float step = adam_step_size(rate, *L.t_Psi);
    float lr_wd = -1.0f;
    if (L.opt_psi == DPC_OPT_ADAMW)
      lr_wd = rate * ((!full_kind && L.psi_decay >= 0.0f) ? L.psi_decay : L.lmbda);
    for (size_t q = tid; q < nP; q += nthr)
    {
      const size_t o = (q / TS) * L.psi_stride + q % TS;
      float m = L.m_Psi[o], v = L.v_Psi[o];
      L.Psi[o] = adam_update(L.Psi[o], -L.g_Psi[o], m, v, step, lr_wd);
      L.m_Psi[o] = m;
      L.v_Psi[o] = v;
    }
  }
}

// Row centring of W: subtract each row's mean (src/backend/CPUBackend.cpp:250-272).
__global__ void center_rows_kernel(const dpc_layer* __restrict__ layers, int first, int n_layers)
{
  const int li = first + blockIdx.y;
  if (li + 1 >= n_layers)
    return;
  const dpc_layer L = layers[li];
  if (L.next_size <= 0)
    return;
  __shared__ float red[32];
  for (int r = blockIdx.x; r < L.next_size; r += gridDim.x)
  {
    float* row = L.W + (size_t)r * L.size;
    float s = 0.0f;
    for (int c = threadIdx.x; c < L.size; c += blockDim.x)
      s += row[c];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0)
      red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x < 32)
    {
      float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.0f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
        t += __shfl_xor_sync(0xffffffffu, t, o);
      if (threadIdx.x == 0)
        red[0] = t;
    }
    __syncthreads();
    const float mean = red[0] / (float)L.size;
    for (int c = threadIdx.x; c < L.size; c += blockDim.x)
      row[c] -= mean;
    __syncthreads();
  }
}
} // namespace dpc
