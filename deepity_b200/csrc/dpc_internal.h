// Internal declarations shared by the translation units of libdeepity_b200.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <string>
#include <vector>

#include "deepity_b200.h"

namespace dpc
{
void set_error(const std::string& msg);
int fail(int code, const std::string& msg);
int cuda_fail(cudaError_t err, const char* what);

#define DPC_CUDA(call)                                                                            \
  do                                                                                              \
  {                                                                                               \
    cudaError_t err__ = (call);                                                                   \
    if (err__ != cudaSuccess)                                                                     \
      return dpc::cuda_fail(err__, #call);                                                        \
  } while (0)

// Description of the maximal run of identical square layers that the tensor-core
// kernels can process with one 3-D tensor map per operand (layer = outermost coordinate).
struct TensorRun
{
  int first = 0, count = 0; // layers [first, first+count), 0 = none
  int width = 0;            // size == next_size == width
  // element strides between consecutive layers of the run
  int64_t z_stride = 0, w_stride = 0, b_stride = 0, out_stride = 0;
};
} // namespace dpc

struct dpc_ctx
{
  int device = 0;
  cudaStream_t stream = nullptr;
  int precision = DPC_PRECISION_FP32;
  int sm_count = 0;
  int64_t launches = 0;
  static constexpr int kSlots = 8;
  cudaGraph_t graphs[kSlots] = {};
  cudaGraphExec_t execs[kSlots] = {};
  int capturing_slot = -1;
  int64_t launches_at_begin = 0;
  int64_t graph_kernels[kSlots] = {};
  // Streams that fork from `stream` and join it again within one phase call (never visible to the
  // caller): consecutive single tensor-core layers of a phase run side by side on them.
  static constexpr int kSide = 3;
  cudaStream_t side[kSide] = {};
  cudaEvent_t fork_ev = nullptr, join_ev[kSide] = {};
};

struct dpc_plan
{
  dpc_ctx* ctx = nullptr;
  int n = 0, batch = 0;
  std::vector<dpc_layer> h; // host copy of the table
  dpc_layer* d = nullptr;   // device copy
  double* energy = nullptr; // device accumulator
  double* energy_host = nullptr; // pinned
  const float* e_terminal = nullptr; // terminal error the DFA / Psi kernels read
  dpc::TensorRun run;
  void* tc = nullptr; // tensor-core path state (tensor maps), owned by dpc_tc.cu
};

namespace dpc
{
// dpc_tc.cu — tensor-core (tcgen05/TMEM/TMA) path.  Each returns DPC_OK when it handled
// layers [first, first+count) completely, 1 when the range is not eligible (the caller
// then uses the CUDA-core kernels), or a negative status.
int tc_plan_init(dpc_plan* plan);
void tc_plan_free(dpc_plan* plan);
int tc_forward(dpc_plan* plan, int first, int count, int flags);
int tc_update_state(dpc_plan* plan, int first, int count);
int tc_project_forward(dpc_plan* plan, int first, int count, int flags);
// mode: 0 learn, 1 direct feedback, +2: only store the raw sums in the layers' g_W.
int tc_weight_gemm(dpc_plan* plan, int first, int count, int mode, int decay_w = 0);
// Synchronous: reads the device-side status flag the kernels raise when a bounded wait runs
// out; DPC_ERR_TIMEOUT if it was raised.
int tc_check_error(dpc_plan* plan);
void tc_set_chain_trace(dpc_plan* plan, unsigned long long* buf);
// Operand planes (bf16 hi/mid copies of the run's beliefs, feedback errors and weights that the
// 3xBF16 kernels read).  tc_touch: something outside dpc_tc.cu wrote the fp32 tensors `kind`
// (0 beliefs, 1 feedback errors, 2 weights) of layers [first, first+count); tc_sync_planes:
// re-split everything that is stale now (before a CUDA graph of a step is recorded or replayed).
void tc_touch(dpc_plan* plan, int kind, int first, int count);
// The feedback-error planes for kernels outside dpc_tc.cu that write or read them: device
// base (NULL: none), the run they cover, elements per plane, and whether the run's fp32 feedback
// errors are not kept at all.  tc_fe_written: such a kernel wrote planes of layers
// [first, first+count) itself; tc_fe_need: bring the planes of those layers up to date.
void tc_fe_planes(dpc_plan* plan, void** base, int* run_first, int* run_count, long long* elems,
                  int* only);
void tc_fe_written(dpc_plan* plan, int first, int count);
int tc_fe_need(dpc_plan* plan, int first, int count);
int tc_sync_planes(dpc_plan* plan);
// Limit of every bounded device-side wait in clock cycles (<= 0: the default, ~2 s) and a bias
// on the forward sweep's publication target (test hook: a target nothing reaches).
void tc_set_wait_limit(dpc_plan* plan, long long cycles, int chain_target_bias);
std::string tc_describe(dpc_plan* plan);
// Single layers outside the run whose shapes fit the CTA-pair tensor-core kernels (batch, input
// and output width multiples of 256).  Same return convention as the run's entry points.
bool tc_extra_layer(dpc_plan* plan, int layer);
int tc_extra_forward(dpc_plan* plan, int layer, int flags);
int tc_extra_update_state(dpc_plan* plan, int layer);
int tc_extra_weight_gemm(dpc_plan* plan, int layer, int mode, int decay_w);
} // namespace dpc
