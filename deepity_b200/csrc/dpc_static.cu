// dpc_error_energy_static — the one entry point of this library that allocates nothing.
//
// Some callers must not (or cannot) call cudaMalloc: code that runs between the captures of a
// CUDA graph, services whose device memory is owned entirely by a framework's pool so that a
// stray cudaMalloc fragments or exhausts it, control loops that forbid allocation after
// start-up.  For them this file offers the error/energy kernel — e = z - mu and
// E = 0.5 * sum(e^2), the first half of CalculateState — with its reduction scratch in a
// file-scope device array instead of memory obtained at run time.  Every GPU that loads the
// library holds that array (a little over 8 KB) until the process exits.
#include <cuda_runtime.h>

#include <atomic>

#include <cstdint>
#include <string>

#include "dpc_internal.h"

namespace
{
constexpr int kStaticMaxBlocks = 1024;
constexpr int kStaticThreads = 256;
// Largest element count accepted: 2^26 elements (256 MiB per tensor); each block then walks
// at most 64 Ki elements.
constexpr int64_t kStaticMaxElements = (int64_t)1 << 26;

// Scratch: one partial sum per block, then (last slot) the ticket counter that elects the
// block which adds the partials up.  Host code may not use this name as an address: it is
// only a stand-in on the host side, the device address comes from cudaGetSymbolAddress.
static __device__ __align__(256) double dpc_static_scratch[kStaticMaxBlocks + 1];

__global__ void __launch_bounds__(kStaticThreads)
    error_energy_static_kernel(const float* __restrict__ z, const float* __restrict__ mu,
                               float* __restrict__ e, int64_t n, float* __restrict__ energy_out,
                               double* scratch)
{
  __shared__ double warp_sums[kStaticThreads / 32];
  __shared__ bool is_last;
  double local = 0.0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
  {
    const float d = z[i] - mu[i];
    e[i] = d;
    local += (double)d * (double)d;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    local += __shfl_xor_sync(0xffffffffu, local, o);
  if ((threadIdx.x & 31) == 0)
    warp_sums[threadIdx.x >> 5] = local;
  __syncthreads();
  if (threadIdx.x == 0)
  {
    double s = 0.0;
    for (int w = 0; w < kStaticThreads / 32; ++w)
      s += warp_sums[w];
    scratch[blockIdx.x] = s;
    __threadfence();
    unsigned int* ticket = reinterpret_cast<unsigned int*>(&scratch[kStaticMaxBlocks]);
    is_last = atomicAdd(ticket, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (is_last && threadIdx.x == 0)
  {
    __threadfence();
    double total = 0.0;
    // The partial sums were written by other blocks: read them from L2, past this SM's L1.
    for (unsigned int b = 0; b < gridDim.x; ++b) // fixed order: the result is reproducible
      total += __ldcg(&scratch[b]);
    *energy_out = (float)(0.5 * total);
    *reinterpret_cast<unsigned int*>(&scratch[kStaticMaxBlocks]) = 0u; // ready for the next call
  }
}

// Device address of the scratch array, looked up once per device.
constexpr int kMaxDevices = 64;
std::atomic<double*> g_scratch_addr[kMaxDevices] = {};
} // namespace

int dpc_error_energy_static(void* stream, const float* z_dev, const float* mu_dev, float* e_dev,
                            int64_t count, float* energy_dev)
{
  if (!z_dev || !mu_dev || !e_dev || !energy_dev || count <= 0)
    return dpc::fail(DPC_ERR_INVALID, "dpc_error_energy_static: null pointer or empty input");
  if (count > kStaticMaxElements)
    return dpc::fail(DPC_ERR_TOO_LARGE,
                     "dpc_error_energy_static: " + std::to_string(count) +
                         " elements exceed the fixed maximum of " +
                         std::to_string(kStaticMaxElements) +
                         " (the scratch array is static; use dpc_error for larger tensors)");
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess)
    return dpc::cuda_fail(err, "cudaGetDevice");
  if (device < 0 || device >= kMaxDevices)
    return dpc::fail(DPC_ERR_INVALID, "dpc_error_energy_static: device index out of range");
  double* scratch = g_scratch_addr[device].load(std::memory_order_acquire);
  if (!scratch)
  {
    // Set-up, once per device, with that device current: the array's name is not a device
    // address in host code, so ask the runtime for it.
    void* p = nullptr;
    err = cudaGetSymbolAddress(&p, dpc_static_scratch);
    if (err != cudaSuccess || !p)
      return dpc::cuda_fail(err, "cudaGetSymbolAddress(dpc_static_scratch)");
    // (two threads racing here store the same address)
    scratch = static_cast<double*>(p);
    g_scratch_addr[device].store(scratch, std::memory_order_release);
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The ticket must start at zero even if an earlier call never completed.
  err = cudaMemsetAsync(scratch + kStaticMaxBlocks, 0, sizeof(double), st);
  if (err != cudaSuccess)
    return dpc::cuda_fail(err, "cudaMemsetAsync(static ticket)");
  const int64_t want = (count + kStaticThreads * 4 - 1) / (kStaticThreads * 4);
  const int blocks = (int)(want < 1 ? 1 : (want > kStaticMaxBlocks ? kStaticMaxBlocks : want));
  error_energy_static_kernel<<<blocks, kStaticThreads, 0, st>>>(z_dev, mu_dev, e_dev, count,
                                                                energy_dev, scratch);
  err = cudaPeekAtLastError();
  if (err != cudaSuccess)
    return dpc::cuda_fail(cudaGetLastError(), "error_energy_static_kernel launch");
  return DPC_OK;
}
