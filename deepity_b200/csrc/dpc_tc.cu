// Tensor-core (tcgen05 / TMEM / TMA) path — placeholder until the kernels land: every
// entry reports "range not eligible" so the CUDA-core kernels run.
#include "dpc_internal.h"

namespace dpc
{
int tc_plan_init(dpc_plan* plan)
{
  plan->run = TensorRun();
  return DPC_OK;
}
void tc_plan_free(dpc_plan*) {}
int tc_forward(dpc_plan*, int, int, int)
{
  return 1;
}
int tc_update_state(dpc_plan*, int, int)
{
  return 1;
}
int tc_weight_gemm(dpc_plan*, int, int, int)
{
  return 1;
}
} // namespace dpc
