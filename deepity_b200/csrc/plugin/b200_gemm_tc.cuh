// General fp32 GEMM on the tensor cores for the DeepityCUDA plugin:
//   C[M,N] = alpha * op(A) * op(B) + beta * C,   row-major operands, one TF32 pass
// (tcgen05.mma kind::tf32, fp32 accumulation in tensor memory), the arithmetic the reference's
// own GPU backend uses by default (src/backend/cuda/CUDABackendGemm.cu:435-445,
// CUDABackendCore.cu:54-67).  One CTA per 128 x BN output tile: warp 0 streams 32-wide k-blocks
// of both operands through a shared-memory ring by TMA (2-D tensor maps built per call from the
// caller's pointers and leading dimensions; every CTA loads its own tiles), warp 1 issues the MMAs, warps 2-5
// read the accumulator (one tensor-memory quarter each) and apply alpha / beta.
//
// Either operand may be "K-major" (k contiguous in memory: A not transposed, B transposed) or
// "MN-major" (A transposed, B not transposed).  32-bit MN-major operands need the 128-byte
// swizzle with 32-byte atoms and are staged as slabs of 32 columns.
//
// Shapes that do not tile (M % 128, N % 64, K % 32, unaligned pointers or leading dimensions)
// are refused (run() returns false) and go to the caller's CUDA-core kernel.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

#include "../dpc_tcgen05.cuh"

namespace b200
{
namespace gemm_tc
{
using namespace dpc::ptx;

constexpr int BM = 128, BK = 32, STAGES_MAX = 6;

struct Params
{
  int M, N, K;
  float alpha, beta;
  float* C;
  int ldc;
  int* error_flag;
};

template <int BN, bool A_MN, bool B_MN>
struct Cfg
{
  static constexpr int A_BYTES = BM * BK * 4, B_BYTES = BN * BK * 4;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = STAGES_MAX;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
  static constexpr uint32_t IDESC = (1u << 4) | (2u << 7) | (2u << 10) | ((A_MN ? 1u : 0u) << 15) |
                                    ((B_MN ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) |
                                    ((uint32_t)(BM >> 4) << 24);
};

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(192, 1)
    gemm_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                const Params P)
{
  using C = Cfg<BN, A_MN, B_MN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + C::STAGES;
  uint64_t* tfull = bars + 2 * C::STAGES;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tfull + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int kblocks = P.K / BK;

  if (threadIdx.x == 0)
  {
    for (int s = 0; s < C::STAGES; ++s)
    {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(tfull, 1);
    *abort_flag = 0;
    *reinterpret_cast<volatile long long*>(abort_flag + 2) = kWaitCyclesDefault;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1)
  {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_holder)),
                 "r"((uint32_t)BN)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0)
  {
    if (lane == 0)
    {
      uint32_t phase = 1;
      for (int kb = 0, s = 0; kb < kblocks; ++kb, s = (s + 1 == C::STAGES ? 0 : s + 1))
      {
        if (s == 0 && kb != 0)
          phase ^= 1;
        if (!mbar_wait(&empty[s], phase, abort_flag))
          break;
        uint8_t* a_dst = smem + s * C::STAGE_BYTES;
        uint8_t* b_dst = a_dst + C::A_BYTES;
        const int k0 = kb * BK;
        mbar_expect_tx(&full[s], C::STAGE_BYTES);
        if (!A_MN)
          tma_load_2d(a_dst, &mapA, &full[s], k0, m0);
        else
          for (int i = 0; i < BM / 32; ++i)
            tma_load_2d(a_dst + i * (BK * 128), &mapA, &full[s], m0 + 32 * i, k0);
        if (!B_MN)
          tma_load_2d(b_dst, &mapB, &full[s], k0, n0);
        else
          for (int i = 0; i < BN / 32; ++i)
            tma_load_2d(b_dst + i * (BK * 128), &mapB, &full[s], n0 + 32 * i, k0);
      }
    }
  }
  else if (warp == 1)
  {
    if (lane == 0)
    {
      // K-major fp32 tiles: 128-byte rows, 8 per swizzle atom (1024 B between row groups), 32 B per
      // K = 8 step.  MN-major: slabs of 32 columns BK*128 bytes apart, 4 k-rows per 32-byte-atom
      // swizzle group (512 B between groups), 1024 B per K = 8 step.
      const uint64_t da0 = make_desc(smem_u32(smem), A_MN ? BK * 128 : 16, A_MN ? 512 : 1024, A_MN ? 1 : 2);
      const uint64_t db0 = make_desc(smem_u32(smem) + C::A_BYTES, B_MN ? BK * 128 : 16,
                                     B_MN ? 512 : 1024, B_MN ? 1 : 2);
      const uint32_t a_adv = A_MN ? 1024 : 32, b_adv = B_MN ? 1024 : 32;
      uint32_t phase = 0;
      bool alive = true;
      for (int kb = 0, s = 0; kb < kblocks; ++kb)
      {
        if (!mbar_wait(&full[s], phase, abort_flag))
        {
          alive = false;
          break;
        }
        tc_fence_after();
        const uint64_t sa = da0 + (uint64_t)(s * (C::STAGE_BYTES >> 4));
        const uint64_t sb = db0 + (uint64_t)(s * (C::STAGE_BYTES >> 4));
#pragma unroll
        for (int ks = 0; ks < BK / 8; ++ks)
          tc_mma_tf32(tmem_base, sa + (uint64_t)(ks * (a_adv >> 4)), sb + (uint64_t)(ks * (b_adv >> 4)),
                      C::IDESC, (kb | ks) != 0);
        tc_commit(&empty[s]);
        if (++s == C::STAGES)
          s = 0, phase ^= 1;
      }
      if (alive)
        tc_commit(tfull);
    }
  }
  else
  {
    // epilogue: warp w reads tensor-memory lanes 32 (w & 3) .. +31 = rows of the tile
    const int quarter = warp & 3;
    const int m = m0 + quarter * 32 + lane;
    if (kblocks == 0 || mbar_wait(tfull, 0, abort_flag))
    {
      tc_fence_after();
      float* crow = P.C + (size_t)m * P.ldc + n0;
      for (int c = 0; c < BN; c += 32)
      {
        float v[32];
        if (kblocks > 0)
          tc_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + c, v);
        else
        {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            v[i] = 0.0f;
        }
#pragma unroll
        for (int i = 0; i < 32; i += 4)
        {
          float4 o = make_float4(P.alpha * v[i], P.alpha * v[i + 1], P.alpha * v[i + 2], P.alpha * v[i + 3]);
          if (P.beta != 0.0f)
          {
            const float4 old = *reinterpret_cast<const float4*>(crow + c + i);
            o.x += P.beta * old.x, o.y += P.beta * old.y, o.z += P.beta * old.z, o.w += P.beta * old.w;
          }
          *reinterpret_cast<float4*>(crow + c + i) = o;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag)
    atomicExch(P.error_flag, 1);
  if (warp == 1)
  {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)BN)
                 : "memory");
  }
}
} // namespace gemm_tc

// Host side: tensor-map encoder, eligibility, dispatch over (BN, operand layouts).
struct TcGemm
{
  typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                               CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                               CUtensorMapFloatOOBfill);
  EncodeFn encode = nullptr;
  int max_smem = 0;
  int* error_flag = nullptr;

  bool init(int shared_optin)
  {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return false;
    encode = reinterpret_cast<EncodeFn>(p);
    max_smem = shared_optin;
    if (cudaMalloc(&error_flag, sizeof(int)) != cudaSuccess)
      return false;
    cudaMemset(error_flag, 0, sizeof(int));
    return true;
  }

  // matrix stored row-major with `rows` rows of `cols` floats, leading dimension ld
  bool make_map(CUtensorMap* map, const float* base, int rows, int cols, int ld, int box_rows,
                bool mn_major) const
  {
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
    cuuint32_t box[2] = {32, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
  }

  template <int BN, bool A_MN, bool B_MN>
  bool launch(cudaStream_t stream, const CUtensorMap& a, const CUtensorMap& b, const gemm_tc::Params& P)
  {
    using C = gemm_tc::Cfg<BN, A_MN, B_MN>;
    static bool configured = false;
    auto kern = gemm_tc::gemm_kernel<BN, A_MN, B_MN>;
    if (!configured)
    {
      if (C::SMEM_BYTES > max_smem ||
          cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) !=
              cudaSuccess)
        return false;
      configured = true;
    }
    dim3 grid(P.N / BN, P.M / gemm_tc::BM);
    kern<<<grid, 192, C::SMEM_BYTES, stream>>>(a, b, P);
    return cudaPeekAtLastError() == cudaSuccess;
  }

  bool run(cudaStream_t stream, bool ta, bool tb, int M, int N, int K, float alpha, const float* A,
           int lda, const float* B, int ldb, float beta, float* C, int ldc)
  {
    if (!encode || M % gemm_tc::BM != 0 || N % 64 != 0 || K % gemm_tc::BK != 0 || K <= 0)
      return false;
    if (((uintptr_t)A | (uintptr_t)B | (uintptr_t)C) % 16 != 0 || lda % 4 != 0 || ldb % 4 != 0 ||
        ldc % 4 != 0)
      return false;
    const int BN = N % 128 == 0 ? 128 : 64;
    // A as stored: !ta -> [M, K] (K-major), ta -> [K, M] (MN-major); B as stored: tb -> [N, K]
    // (K-major), !tb -> [K, N] (MN-major)
    const bool a_mn = ta, b_mn = !tb;
    CUtensorMap ma, mb;
    if (!(a_mn ? make_map(&ma, A, K, M, lda, 32, true) : make_map(&ma, A, M, K, lda, gemm_tc::BM, false)))
      return false;
    if (!(b_mn ? make_map(&mb, B, K, N, ldb, 32, true) : make_map(&mb, B, N, K, ldb, BN, false)))
      return false;
    gemm_tc::Params P{M, N, K, alpha, beta, C, ldc, error_flag};
#define B200_TC_CASE(bn, amn, bmn)                                                               \
  if (BN == bn && a_mn == amn && b_mn == bmn)                                                    \
    return launch<bn, amn, bmn>(stream, ma, mb, P);
    B200_TC_CASE(128, false, false)
    B200_TC_CASE(128, false, true)
    B200_TC_CASE(128, true, false)
    B200_TC_CASE(128, true, true)
    B200_TC_CASE(64, false, false)
    B200_TC_CASE(64, false, true)
    B200_TC_CASE(64, true, false)
    B200_TC_CASE(64, true, true)
#undef B200_TC_CASE
    return false;
  }
};
} // namespace b200
