/*
 * deepity_b200 — C ABI of the B200 (sm_100a) predictive-coding train-step library.
 *
 * Two levels, both plain C (pointers, sizes, opaque handles, int status codes; no
 * exceptions cross this boundary, no torch types):
 *
 *   dpc_*   phase kernels on DEVICE pointers.  They stand where the reference's layer
 *           classes call its compute backend (include/deepity/backend/IComputeBackend.h)
 *           — but one call covers a whole phase of many layers instead of one primitive
 *           of one layer.  All work is stream-ordered on the context's stream; only the
 *           functions marked "synchronous" wait for the GPU.
 *   dpcn_*  whole networks (SimplePC / DirectKPPC / FullPC) with HOST buffers in and
 *           out.  They are what the reference's Python binding binds
 *           (bindings/NetworkBindings.cpp:562-646, 836-1067, 1069-1357).
 *
 * Every function returns DPC_OK (0) or a negative dpc_status; dpc_last_error() gives
 * the message of the last failure on the calling thread.  There is no CPU fallback:
 * without a CUDA device every call fails with DPC_ERR_NO_DEVICE.
 *
 * Which kernels run is decided per plan from the layer shapes (dpc_plan_describe tells); a plan
 * whose shapes qualify for the tensor-core kernels but cannot get them (no sm_100 device, a
 * refused tensor map, no memory for the operand copies) says so once on stderr.  Environment
 * switches, read when a plan is created or a phase is launched -- diagnostic aids that the
 * tests use to compare code paths, not tuning knobs:
 *   DPC_DISABLE_TENSOR_CORES   every layer on the CUDA-core kernels
 *   DPC_DISABLE_CTA_PAIRS      single-CTA 128-row tiles instead of cta_group::2 pairs
 *   DPC_FP32_SCHEME=tf32x3     FP32 mode with three TF32 passes instead of three BF16 passes
 *   DPC_DISABLE_PLANES         3xBF16 operands split inside the kernels, not pre-split copies
 *   DPC_KEEP_FE_FP32           keep writing the fp32 feedback errors beside their bf16 copies
 *   DPC_DISABLE_STAGED_INPUT / DPC_DISABLE_STAGED_OUTPUT
 *                              epilogues of the pair-tile kernels read / write global memory lane
 *                              by lane instead of through shared memory and bulk tensor copies
 *   DPC_DISABLE_KSPLIT         forward sweep without the two-CTA split of K
 *   DPC_DISABLE_RECTANGULAR    single layers outside the run of identical square layers stay on
 *                              the CUDA-core kernels even where their shapes fit the pair tiles
 *   DPC_RECTANGULAR_MIN_WORK   such a layer goes to the pair tiles only when batch x inputs x
 *                              outputs is at least this (default 2^29: below it the CUDA-core
 *                              kernels, which take all layers of a phase in one launch, are as fast)
 *   DPC_DISABLE_LAYER_STREAMS  consecutive such layers of one phase are launched one after the other
 *                              on the context's stream instead of side by side on internal streams
 *                              that fork from it and join it again
 */
#ifndef DEEPITY_B200_H
#define DEEPITY_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define DPC_API __attribute__((visibility("default")))
#else
#define DPC_API
#endif

typedef enum dpc_status
{
  DPC_OK = 0,
  DPC_ERR_INVALID = -1,   /* bad argument / shape / handle            */
  DPC_ERR_NO_DEVICE = -2, /* no usable CUDA device                    */
  DPC_ERR_CUDA = -3,      /* a CUDA runtime or driver call failed     */
  DPC_ERR_STATE = -4,     /* call order (e.g. train step before compile) */
  DPC_ERR_TIMEOUT = -5,   /* a bounded device-side wait gave up       */
  DPC_ERR_TOO_LARGE = -6  /* size beyond a documented fixed maximum   */
} dpc_status;

/* Activation ids: the forward enumerators of Deep::ActivationType
 * (include/deepity/utils/ActivationType.h:15-32), so a host that already holds that
 * enum passes it through unchanged.  The derivative is implied. */
typedef enum dpc_act
{
  DPC_ACT_RELU = 0,
  DPC_ACT_GELU = 2,
  DPC_ACT_SIGMOID = 4,
  DPC_ACT_ESIGMOID = 6,
  DPC_ACT_TANH = 8,
  DPC_ACT_LINEAR = 10,
  DPC_ACT_HARD_TANH = 12
} dpc_act;

/* Deep::OptimizerType, include/deepity/utils/AdamOptimizer.h:12-17. */
typedef enum dpc_opt
{
  DPC_OPT_SGD = 0,
  DPC_OPT_ADAM = 1,
  DPC_OPT_ADAMW = 2
} dpc_opt;

/* GEMM arithmetic.  FP32: every product and sum in fp32 (CUDA cores, or a three-pass operand
 * split -- 3xBF16 for SGD networks, 3xTF32 otherwise -- on the tensor cores where the shape allows) — the mode judged at 1e-4 against the CPU
 * reference.  TF32: one tensor-core pass with fp32 accumulation, the analogue of the
 * reference's default cuBLAS TF32 math mode (src/backend/cuda/CUDABackendCore.cu:54-67,
 * IComputeBackend::SetAllowTF32); judged at the reference's own 1e-2 CPU-vs-GPU bound.
 * MIXED (not the default, no counterpart in the reference): the state path -- forward sweep,
 * settling passes, energy -- as in FP32; the gradient path of the tensor-core layers -- the
 * prediction refresh before learning and the two weight-shaped products -- as in TF32, when
 * every weight optimizer is SGD.  The TF32 rounding (5e-4 relative) then lands on the UPDATE
 * of W, not on W; judged at 1e-3.  Where a plan keeps pre-split bf16 operand copies (the default
 * for SGD networks on 256-multiple shapes) the mode runs exactly what FP32 runs: those kernels are
 * faster than the one-pass TF32 ones and more exact. */
typedef enum dpc_precision
{
  DPC_PRECISION_FP32 = 0,
  DPC_PRECISION_TF32 = 1,
  DPC_PRECISION_MIXED = 2
} dpc_precision;

typedef struct dpc_ctx dpc_ctx;
typedef struct dpc_plan dpc_plan;

/* ------------------------------------------------------------------------------------
 * Context: device, stream, graph slots.  Replaces CUDABackend's constructor and the
 * plugin entry Deepity_CreateCUDABackend (src/backend/cuda/CUDAPluginExports.cpp:12-21,
 * src/backend/cuda/CUDABackendCore.cu:26-73).
 * ---------------------------------------------------------------------------------- */
DPC_API const char* dpc_last_error(void);
DPC_API const char* dpc_version(void);
DPC_API int dpc_create(int device, dpc_ctx** out);
DPC_API int dpc_destroy(dpc_ctx* ctx);
DPC_API int dpc_set_precision(dpc_ctx* ctx, int precision); /* IComputeBackend::SetAllowTF32 */
DPC_API int dpc_get_precision(dpc_ctx* ctx);
/* cudaStream_t of the context, as void* (IComputeBackend::GetStreamHandle). */
DPC_API void* dpc_stream(dpc_ctx* ctx);
/* Number of kernels this library has launched on the context since creation. */
DPC_API int64_t dpc_launch_count(dpc_ctx* ctx);

/* Memory (IComputeBackend::Allocate/Free/Zero/Copy/CopyFromHost/CopyToHost,
 * include/deepity/backend/IComputeBackend.h:52-77).  Sizes in BYTES.  alloc/free and the
 * *_sync copies are synchronous; the others are stream-ordered. */
DPC_API int dpc_alloc(dpc_ctx* ctx, size_t bytes, void** out);
DPC_API int dpc_free(dpc_ctx* ctx, void* ptr);
DPC_API int dpc_zero(dpc_ctx* ctx, void* ptr, size_t bytes);
DPC_API int dpc_copy_d2d(dpc_ctx* ctx, void* dst, const void* src, size_t bytes);
DPC_API int dpc_copy_h2d(dpc_ctx* ctx, void* dst, const void* host_src, size_t bytes);
DPC_API int dpc_copy_d2h(dpc_ctx* ctx, void* host_dst, const void* src, size_t bytes);
DPC_API int dpc_copy_h2d_sync(dpc_ctx* ctx, void* dst, const void* host_src, size_t bytes);
DPC_API int dpc_copy_d2h_sync(dpc_ctx* ctx, void* host_dst, const void* src, size_t bytes);
DPC_API int dpc_alloc_host(dpc_ctx* ctx, size_t bytes, void** out); /* pinned */
DPC_API int dpc_free_host(dpc_ctx* ctx, void* ptr);
DPC_API int dpc_sync(dpc_ctx* ctx); /* IComputeBackend::Synchronize */
/* dst[r, :] = src[index[first + r], :] for r in [0, rows), rows of `cols` floats, all pointers
 * device memory, ordered on the context's stream.  The mini-batch gather of an epoch loop over a
 * data set that stays on the device (deepity/utils.py:19-143 slices a shuffled host array per
 * batch instead). */
DPC_API int dpc_gather_rows(dpc_ctx* ctx, const float* src_dev, const int64_t* index_dev,
                            int64_t first, int rows, int64_t cols, float* dst_dev);

/* CUDA graphs (IComputeBackend::BeginGraphCapture/EndGraphCapture/ReplayGraph,
 * src/backend/cuda/CUDABackendCore.cu:120-187).  slot in [0, 8). */
DPC_API int dpc_graph_begin(dpc_ctx* ctx, int slot);
DPC_API int dpc_graph_end(dpc_ctx* ctx, int slot);
DPC_API int dpc_graph_launch(dpc_ctx* ctx, int slot);
DPC_API int dpc_graph_drop(dpc_ctx* ctx, int slot);

/* ------------------------------------------------------------------------------------
 * Layer description.  One entry per layer of a network, input layer first, the
 * weight-less terminal layer last (next_size == 0, parameter pointers NULL).  Tensors are
 * fp32 row-major:  z,e,zF,v [B,size];  W [next_size,size];  b [next_size];
 * preact,mu,fe [B,next_size];  Psi [size,psi_stride] (terminal_size logical columns).
 * The fields mirror DirectKPPCLayer::ExternalMemory
 * (include/deepity/layers/DirectKPPCLayer.h:165-199).
 * ---------------------------------------------------------------------------------- */
enum
{
  DPC_LAYER_INPUT_ACT = 1 << 0, /* SimplePC convention: mu = f(z)·Wᵀ + b, derivative applied at
                                   the destination (src/layers/SimplePCLayer.cpp:132-257).
                                   Otherwise mu = f(a·z·Wᵀ + b) (DirectKP/Full). */
  DPC_LAYER_RESIDUAL = 1 << 1,  /* FullPC: mu += z  (src/layers/FullPCLayer.cpp:283-289) */
  DPC_LAYER_SOFTMAX_CE = 1 << 2, /* this layer's error is z - softmax(mu_below)
                                    (src/backend/CPUBackend.cpp:658-714) */
  DPC_LAYER_FULLPC_PSI = 1 << 3  /* FullPC's feedback-weight rule: rate fl*a, AdamW decay lmbda,
                                    no psi_decay (src/layers/FullPCLayer.cpp:466-510) */
};

typedef struct dpc_layer
{
  int32_t size, next_size, terminal_size, psi_stride;
  int32_t act;   /* dpc_act */
  int32_t flags; /* DPC_LAYER_* */
  float a;       /* muPC forward scale, 1 when unused (FullPCLayer::SetMuPCScale) */
  float lr, ir, fl, lmbda;
  float psi_decay;     /* < 0: optimizer default (DirectKPPCLayer.cpp:444-446,492-494) */
  float momentum_beta; /* used when v != NULL (FullPCLayer.cpp:353-363) */
  int32_t opt, opt_psi; /* dpc_opt */
  float *z, *e;
  float *W, *b;
  float *preact, *mu, *fe;
  float* Psi;
  float* zF; /* DPC_LAYER_INPUT_ACT only: f(z) as last fed to the GEMM */
  float* v;  /* state momentum or NULL */
  float* adj; /* ePC adjoint [B,size] or NULL (FullPCLayer::ComputeAdjoint) */
  float *m_W, *v_W, *m_b, *v_b, *m_Psi, *v_Psi; /* Adam moments or NULL */
  int32_t *t, *t_Psi;                           /* Adam step counters on the device or NULL */
  /* Gradient staging (batch-sharded training) or NULL: raw sums fe^T z [next,size],
   * column sums of fe [next] and z^T e_T [size,psi_stride], written by
   * dpc_weight_gradients and consumed by dpc_apply_gradients. */
  float *g_W, *g_b, *g_Psi;
} dpc_layer;

/* A plan = the layer table uploaded once, plus whatever the kernels precompute for it
 * (uniform runs for the tensor-core path, tensor maps).  Replaces what
 * DirectKPPCNetwork::Compile() prepares for its batched run
 * (src/networks/DirectKPPCNetwork.cpp:692-944). */
DPC_API int dpc_plan_create(dpc_ctx* ctx, const dpc_layer* layers, int n_layers, int batch,
                            dpc_plan** out);
/* Re-upload after a hyper-parameter / optimizer / pointer change (same layer count). */
DPC_API int dpc_plan_update(dpc_plan* plan, const dpc_layer* layers, int n_layers);
DPC_API int dpc_plan_destroy(dpc_plan* plan);
/* Terminal error used by dpc_direct_feedback and the Psi update.  NULL (default): the e
 * buffer of the plan's last layer.  A layer-sharded network whose last local layer is only a
 * copy of the neighbour rank's first layer points this at the buffer that receives the
 * broadcast terminal error [batch, terminal_size]. */
DPC_API int dpc_plan_set_terminal_error(dpc_plan* plan, const float* e_terminal_dev);
/* Profiling aid: a device buffer of 256*8 uint64 in which CTA 0 of the forward-sweep kernel
 * records globaltimer stamps per layer (dependency seen, first operands landed, accumulator
 * complete, stores issued, published, ...).  NULL switches it off (default). */
DPC_API int dpc_plan_set_chain_trace(dpc_plan* plan, void* trace_dev);
/* Layers [first, first+count) that the tensor-core path covers (0 if none). */
DPC_API int dpc_plan_tensor_run(dpc_plan* plan, int* first, int* count);
/* One line of text on which kernels the plan's weight layers run (tcgen05 tile shape and
 * arithmetic scheme of the run, how many layers stay on the CUDA-core kernels), the
 * counterpart of asking the reference which GEMM path a shape took
 * (src/backend/cuda/CUDABackendGemm.cu:435-445).  Truncated to buf_bytes. */
DPC_API int dpc_plan_describe(dpc_plan* plan, char* buf, int buf_bytes);
/* The tensor-core kernels of an SGD network in FP32 mode read bf16 "hi"/"mid" operand copies of
 * z, fe and W of the run's layers, which every kernel of this library keeps up to date.  A
 * caller that writes one of these tensors ITSELF through a device pointer (dpcn_tensor_ptr, a
 * memcpy, an NCCL receive into z of a boundary layer) must say so before the next phase call;
 * the copies of those layers are then rebuilt on next use.  what: bit set of DPC_WROTE_*.
 * dpc_plan_sync_operands rebuilds everything stale now (stream-ordered); the network classes
 * call it before a step is recorded into, or replayed from, a CUDA graph.  No counterpart in
 * the reference, whose GEMMs read the fp32 tensors directly. */
enum
{
  DPC_WROTE_Z = 1,
  DPC_WROTE_FE = 2,
  DPC_WROTE_W = 4
};
DPC_API int dpc_plan_invalidate(dpc_plan* plan, int first, int count, int what);
DPC_API int dpc_plan_sync_operands(dpc_plan* plan);
/* Every device-side wait of the tensor-core kernels (pipeline barriers, the forward sweep's
 * row-block publications) gives up after this long; the kernel then drains, frees its tensor
 * memory and returns, and the next dpc_energy_read reports DPC_ERR_TIMEOUT.  milliseconds <= 0
 * restores the default (about 2 s).  sweep_target_bias is added to the number of publications
 * the forward sweep waits for per row block: a positive value makes that wait impossible to
 * satisfy (the host-side way to exercise the time-out path; 0 in normal use).  The reference
 * has no device-side waits (src/backend/cuda/CUDACommon.cuh:16-25 only logs CUDA errors). */
DPC_API int dpc_plan_set_wait_limit(dpc_plan* plan, double milliseconds, int sweep_target_bias);

/* ---- phases.  Layer ranges are [first, first+count) over the plan's table. ---------- */
enum
{
  DPC_FWD_COPY_NEXT = 1 << 0, /* z[l+1] = mu[l]  (ProjectForward's copy)                  */
  DPC_FWD_ERR_NEXT = 1 << 1,  /* e[l+1] = z[l+1] - mu[l]  (ComputeError of the layer above)*/
  DPC_FWD_ENERGY = 1 << 2,    /* with ERR_NEXT: energy += 0.5*sum e[l+1]^2                 */
  DPC_FWD_FE = 1 << 3,        /* fe[l] = e[l+1] * f'(preact[l]); e[l+1] is the one just
                                 computed with ERR_NEXT, else the one in memory            */
  DPC_FWD_CACHED = 1 << 4,    /* skip the GEMM, reuse preact/mu in memory (a clamped layer's
                                 cached prediction, DirectKPPCLayer.cpp:275-280)          */
  DPC_FWD_NO_MU = 1 << 9,     /* with COPY_NEXT: mu[l] itself is not written (z[l+1] holds the
                                 same values and mu is recomputed before anyone reads it)  */
  DPC_FWD_NO_PREACT = 1 << 11, /* with COPY_NEXT and NO_MU: preact[l] is not written either (the
                                 next reader, dpc_direct_feedback with DPC_DFA_FROM_OUTPUT,
                                 takes f'(preact[l]) from z[l+1] = f(preact[l]))           */
  DPC_FWD_TRANSIENT = 1 << 8  /* preact/mu of this pass are consumed only through the fused
                                 e/fe outputs and recomputed before anyone reads them: do
                                 not write them to memory                                  */
};

/* ComputeMuOnly for every layer of the range, all independent
 * (DirectKPPCLayer.cpp:267-310, FullPCLayer.cpp:246-298, SimplePCLayer.cpp:132-183),
 * with the error of the layer above and the feedback error fused in on request. */
DPC_API int dpc_forward(dpc_plan* plan, int first, int count, int flags);
/* The sequential forward sweep: for l in range: ComputeMuOnly(l); z[l+1] = mu[l] unless
 * l+1 is the last layer and skip_last_copy != 0 (a clamped target)
 * (DirectKPPCNetwork::ProjectForward, src/networks/DirectKPPCNetwork.cpp:349-371). */
DPC_API int dpc_project_forward(dpc_plan* plan, int first, int count, int skip_last_copy);
/* Same, with extra DPC_FWD_* flags (DPC_FWD_NO_MU) applied to every layer of the sweep but its
 * first (a clamped input layer's prediction is cached and read again). */
DPC_API int dpc_project_forward_ex(dpc_plan* plan, int first, int count, int skip_last_copy,
                                   int extra_flags);
/* Error of one layer against the prediction below: Gaussian e = z - mu, or softmax
 * cross-entropy when the layer has DPC_LAYER_SOFTMAX_CE.  with_energy accumulates into the
 * plan's energy accumulator (CPUBackend.cpp:602-629, 658-714). */
DPC_API int dpc_error(dpc_plan* plan, int layer, int with_energy);
/* fe[l] = e[l+1] * f'(preact[l]) over a range (the first two lines of UpdateState /
 * UpdateWeights, DirectKPPCLayer.cpp:334-335,372-373). */
DPC_API int dpc_feedback_error(dpc_plan* plan, int first, int count);
/* UpdateState for every layer of the range (all independent, Jacobi):
 * DirectKP/Full z += ir*(a*fe·W - e) (+momentum, +residual), Simple
 * z += ir*(f'(z)*(e_above·W) - e); layers without weights or upper neighbour: z -= ir*e
 * (DirectKPPCLayer.cpp:318-359, FullPCLayer.cpp:300-380, SimplePCLayer.cpp:185-257).
 * Layers listed as clamped by the caller must simply be left out of the range. */
DPC_API int dpc_update_state(dpc_plan* plan, int first, int count);
/* ePC settling (FullPCNetwork::EPCStep, src/networks/FullPCNetwork.cpp:99-131):
 * dpc_epc_reconstruct: z[l] = mu[l-1] + e[l]  (FullPCLayer::ReconstructBelief);
 * dpc_epc_adjoint: adj[l] = a*scale*((src * f'(preact[l]))·W[l]) (+ scale*src with residual),
 * then e[l] = (1-ir)*e[l] - ir*adj[l] unless `clamped` (ComputeAdjoint + UpdateErrorEPC,
 * src/layers/FullPCLayer.cpp:584-640).  src is the terminal error (from_terminal != 0,
 * scale -1 on that first hop) or adj[l+1]. */
DPC_API int dpc_epc_reconstruct(dpc_plan* plan, int layer);
DPC_API int dpc_epc_adjoint(dpc_plan* plan, int layer, int from_terminal, float scale,
                            int clamped);
/* z -= ir*e for one layer (the "output layer" branch of UpdateState). */
DPC_API int dpc_relax(dpc_plan* plan, int layer);
/* DirectFeedbackUpdate for every layer of the range whose upper neighbour has Psi:
 * proj = (e_T·Psi[l+1]ᵀ) * f'(preact[l]);  W[l] += (fl*a/B) projᵀ·z[l]
 * (DirectKPPCLayer.cpp:503-549, FullPCLayer.cpp:514-572).  decay_w is a bit set: bit 0
 * applies the FullPC (1-lmbda) pre-scale; bit 1 (DPC_DFA_FROM_OUTPUT) tells that z[l+1]
 * still equals f(preact[l]) for the layers of the range (the call follows the forward sweep
 * directly), so f' is taken from z[l+1] where the activation allows it -- same values, one
 * transcendental less per element, and preact need not have been stored. */
enum
{
  DPC_DFA_DECAY_W = 1,
  DPC_DFA_FROM_OUTPUT = 2
};
DPC_API int dpc_direct_feedback(dpc_plan* plan, int first, int count, int decay_w);
/* UpdateWeights for every layer of the range from fe[l] (DirectKP/Full) or e[l+1]
 * (Simple): W, b and Psi with SGD / Adam / AdamW, optional row centring
 * (DirectKPPCLayer.cpp:361-501, FullPCLayer.cpp:382-512, SimplePCLayer.cpp:259-350,
 * CPUBackend.cpp:250-272, 721-772). */
DPC_API int dpc_update_weights(dpc_plan* plan, int first, int count, int center_rows);
/* The two halves of dpc_direct_feedback (which = 1) and dpc_update_weights (which = 0) for
 * batch-sharded training: the first leaves the raw gradient sums of this process's batch rows
 * in the layers' staging buffers (g_W only for which = 1); the caller sums the buffers over
 * the shards (an all-reduce); the second applies them with the reference's update formulas
 * (DirectKPPCLayer.cpp:361-549, FullPCLayer.cpp:382-572, SimplePCLayer.cpp:259-350,
 * CPUBackendHighway.cpp:779-840), `global_batch` taking the place of the batch size in every
 * 1/B factor.  option: decay_w (which = 1) or center_rows (which = 0).  The reference has no
 * multi-GPU code; with one shard the pair computes what the fused call computes. */
DPC_API int dpc_weight_gradients(dpc_plan* plan, int first, int count, int which);
DPC_API int dpc_apply_gradients(dpc_plan* plan, int first, int count, int which,
                                int global_batch, int option);
/* The error/energy kernel for callers that must not allocate device memory (code between
 * graph captures, hosts whose framework owns every byte of the GPU, loops that forbid
 * allocation once running).  It has no counterpart in the reference.  e = z - mu over
 * `count` floats and *energy_dev = 0.5*sum(e^2), all four pointers device memory the caller
 * provides, work ordered on `stream` (a cudaStream_t; NULL = the default stream) of the
 * device that is current on the calling thread.  Nothing is allocated or freed: the
 * reduction scratch is a static device array of 1025 doubles that every GPU loading this
 * library holds until exit.  count may not exceed 2^26 (DPC_ERR_TOO_LARGE otherwise).  The
 * first call on a device looks up the array's address; make that call before any stream
 * capture.  All calls share the one array, which keeps what the last call left in it (the
 * entry clears the part that must start at zero): two calls whose kernels overlap on the GPU
 * race, so order them on one stream or with events. */
DPC_API int dpc_error_energy_static(void* stream, const float* z_dev, const float* mu_dev,
                                    float* e_dev, int64_t count, float* energy_dev);
/* Energy accumulator of the plan (device-resident double). */
DPC_API int dpc_energy_reset(dpc_plan* plan);
DPC_API int dpc_energy_read(dpc_plan* plan, double* out); /* synchronous */

/* ------------------------------------------------------------------------------------
 * Networks with host buffers: the binding surface.  kind: 0 SimplePCNetwork,
 * 1 DirectKPPCNetwork, 2 FullPCNetwork (include/deepity/networks/*.h).
 * ---------------------------------------------------------------------------------- */
typedef struct dpcn_net dpcn_net;

DPC_API int dpcn_create(int kind, int batch, int device, dpcn_net** out);
DPC_API int dpcn_destroy(dpcn_net* net);
/* AddLayer(size, nextSize, terminalSize, lr, ir, fl, lmbda, aType, dType)
 * (include/deepity/networks/DirectKPPCNetwork.h:80-81); terminal_size and fl are ignored
 * for kind 0. */
DPC_API int dpcn_add_layer(dpcn_net* net, int size, int next_size, int terminal_size, float lr,
                           float ir, float fl, float lmbda, int act);
/* Options by name, before or after compile as the reference allows: "optimizer",
 * "psi_optimizer" (ivalue = dpc_opt), "center_weights", "psi_decay" (fvalue),
 * "learning_rate", "feedback_rate", "inference_rate" (fvalue), "cross_entropy", "mupc",
 * "residual", "ipc", "epc", "momentum" (ivalue on/off, fvalue beta), "precision" (dpc_precision), "ghost_top" (before
 * compile: the last layer is a copy of a neighbour rank's layer, see deepity_b200/sharded.py),
 * "use_graph" (capture the step into a CUDA graph, default on). */
DPC_API int dpcn_set_option(dpcn_net* net, const char* name, int ivalue, float fvalue);
DPC_API int dpcn_compile(dpcn_net* net);
DPC_API int dpcn_num_layers(dpcn_net* net);
/* Tensor access by layer and name: "z" "e" "mu" "preact" "W" "b" "Psi" "weight.m"
 * "weight.v" "bias.m" "bias.v" "psi.m" "psi.v" (Layer::GetStateDict names,
 * src/layers/DirectKPPCLayer.cpp:219-241).  count = logical element count. */
DPC_API int64_t dpcn_tensor_size(dpcn_net* net, int layer, const char* name);
DPC_API int dpcn_get_tensor(dpcn_net* net, int layer, const char* name, float* host_out,
                            int64_t count);
DPC_API int dpcn_set_tensor(dpcn_net* net, int layer, const char* name, const float* host_in,
                            int64_t count);
/* Adam / AdamW step counters of a weight layer by the reference's names: "step" (W and b) and
 * "psi_step" (Psi) (Layer::GetOptimizerCounters, include/deepity/layers/Layer.h:100-134,
 * src/layers/DirectKPPCLayer.cpp:237-241; IComputeBackend::CopyCounterToHost/FromHost).  They
 * live on the device; get is synchronous.  DPC_ERR_STATE when the optimizer is SGD (no counter). */
DPC_API int dpcn_get_counter(dpcn_net* net, int layer, const char* name, int32_t* out);
DPC_API int dpcn_set_counter(dpcn_net* net, int layer, const char* name, int32_t value);
/* Enumeration of everything a checkpoint of the reference holds for this network
 * (Layer::GetStateDict + GetOptimizerStateDict of every weight layer,
 * src/layers/DirectKPPCLayer.cpp:219-235): entry `index` in [0, dpcn_state_dict_size) gives the
 * layer, the tensor name as dpcn_get_tensor takes it ("W" "b" "Psi" "weight.m" ...), its logical
 * shape rows x cols (rows = 1 for vectors), the element stride between rows on the device
 * (TensorDescriptor::rowStride) and whether it is optimizer state. */
DPC_API int dpcn_state_dict_size(dpcn_net* net);
DPC_API int dpcn_state_dict_entry(dpcn_net* net, int index, int* layer, char* name, int name_bytes,
                                  int64_t* rows, int64_t* cols, int64_t* row_stride,
                                  int* optimizer_state);
/* Device pointer of a tensor (zero-copy consumers; FullPCNetwork::TrainStepDevice idea). */
DPC_API int dpcn_tensor_ptr(dpcn_net* net, int layer, const char* name, void** out,
                            int64_t* row_stride);
/* RandomizeWeights(rng, distribution): N(0, sqrt(2/(size+next))) for W and
 * N(0, sqrt(2/(size+terminal))) for Psi from a host mt19937 stream
 * (src/layers/DirectKPPCLayer.cpp:184-217); parity tests set weights explicitly. */
DPC_API int dpcn_randomize(dpcn_net* net, uint32_t seed);
/* TrainStep(x, y, T) -> energy; x,y host pointers (synchronous: returns the energy). */
DPC_API int dpcn_train_step(dpcn_net* net, const float* x, int64_t nx, const float* y,
                            int64_t ny, int steps, float* energy_out);
/* Same with x,y already on this device; energy_out may be NULL to skip the read-back
 * (then the call is stream-ordered only). */
DPC_API int dpcn_train_step_device(dpcn_net* net, const float* x_dev, int64_t nx,
                                   const float* y_dev, int64_t ny, int steps,
                                   float* energy_out);
/* SimplePCNetwork::TrainStepWithProjection (src/networks/SimplePCNetwork.cpp:179-252) and the
 * Python-level SimplePCN.train_step loop (deepity/SimplePCN.py:269-293; mode 2 returns the
 * SUM of per-step energies).  mode: 0 TrainStep, 1 with projection, 2 python loop. */
DPC_API int dpcn_train_step_mode(dpcn_net* net, int mode, const float* x, int64_t nx,
                                 const float* y, int64_t ny, int steps, float* energy_out);
/* Predict(x, T) -> terminal beliefs [B, terminal] into host_out. */
DPC_API int dpcn_predict(dpcn_net* net, const float* x, int64_t nx, int steps,
                         int with_projection, float* host_out, int64_t nout);
/* ResetState(): zero every belief (FullPC: also errors and momentum). Stream-ordered. */
DPC_API int dpcn_reset_state(dpcn_net* net);
/* The network's context and plan, for callers that drive single phases themselves
 * (layer-sharded multi-GPU stepping, per-kernel timing).  Valid after dpcn_compile;
 * owned by the network. */
DPC_API dpc_ctx* dpcn_context(dpcn_net* net);
DPC_API dpc_plan* dpcn_plan(dpcn_net* net);
/* Batch sharding (the reference has no multi-GPU code; this is the "wide, shallow nets"
 * regime): this network holds `batch` of `global_batch` rows.  From now on every
 * DirectFeedbackUpdate / UpdateWeights inside a train step stages raw gradient sums, calls
 * sync(user, dev, count, stream) -- which must leave in dev[0..count) the sum over all
 * shards, ordered on `stream` (an NCCL all-reduce); non-zero return aborts the step -- and
 * applies them with global_batch in the 1/B factors.  sync = NULL switches back.  Steps are
 * not captured into a CUDA graph while a sync function is set. */
typedef int (*dpcn_sync_fn)(void* user, float* dev, int64_t count, void* stream);
DPC_API int dpcn_set_gradient_sync(dpcn_net* net, dpcn_sync_fn sync, void* user,
                                   int global_batch);
/* Kernel launches issued by the network's context so far. */
DPC_API int64_t dpcn_launch_count(dpcn_net* net);
/* Algorithmic FLOPs of one train step with `steps` settling steps (GEMM terms only). */
DPC_API double dpcn_train_step_flops(dpcn_net* net, int steps);

/* ------------------------------------------------------------------------------------
 * Convolutional predictive coding: SimpleConvPCLayer / SimpleConvPCNetwork
 * (include/deepity/layers/SimpleConvPCLayer.h, src/layers/SimpleConvPCLayer.cpp,
 * src/networks/SimpleConvPCNetwork.cpp).  Layouts are the reference's: z, e [B,C,H,W];
 * W [O, C*kH*kW]; b [O]; preact, mu [B,O,oH,oW].  The gathers the reference materialises
 * (Im2Col / Col2Im, include/deepity/utils/Im2Col.h:78-259, RepackForBatchedGemm,
 * CPUBackend.cpp:869-892) are done on the fly by implicit-GEMM kernels.
 * ---------------------------------------------------------------------------------- */
typedef struct dpc_conv_layer
{
  int32_t in_c, out_c, in_h, in_w; /* out_c = 0: the terminal layer (no weights) */
  int32_t k_h, k_w, s_h, s_w, p_h, p_w;
  int32_t out_h, out_w; /* ConvOutDim, Im2Col.h:47-50 */
  int32_t act, opt;     /* dpc_act, dpc_opt */
  float lr, ir, lmbda;
  float *z, *e;
  float *W, *b;
  float *preact, *mu;
  float* g;         /* gated error e_above * f'(preact) ("bottom_up_cols") [B,O,oH,oW] */
  float *g_W, *g_b; /* raw gradient sums [O, C*kH*kW], [O] */
  float *m_W, *v_W, *m_b, *v_b;
  int32_t* t;
} dpc_conv_layer;

typedef struct dpc_conv_plan dpc_conv_plan;
enum
{
  DPC_CONV_COPY_NEXT = 1 << 0, /* z[l+1] = mu[l] (ProjectForward)                          */
  DPC_CONV_ERR_NEXT = 1 << 1,  /* e[l+1] = z[l+1] - mu[l], g[l] = e[l+1] * f'(preact[l])   */
  DPC_CONV_ENERGY = 1 << 2,    /* with ERR_NEXT: energy += 0.5*sum e[l+1]^2                */
  DPC_CONV_CACHED = 1 << 4     /* clamped layer with a valid cache: reuse preact/mu        */
};
DPC_API int dpc_conv_plan_create(dpc_ctx* ctx, const dpc_conv_layer* layers, int n_layers,
                                 int batch, dpc_conv_plan** out);
DPC_API int dpc_conv_plan_update(dpc_conv_plan* plan, const dpc_conv_layer* layers, int n_layers);
DPC_API int dpc_conv_plan_destroy(dpc_conv_plan* plan);
/* ComputeMuOnly of one layer (SimpleConvPCLayer.cpp:214-300) with the error of the layer above
 * (CalculateState, :188-212) and the gated error fused in on request. */
DPC_API int dpc_conv_forward(dpc_conv_plan* plan, int layer, int flags);
/* UpdateState (SimpleConvPCLayer.cpp:302-400): z += ir*(W^T (*) g - e), the transposed
 * convolution written as a gather; a layer without weights relaxes, z -= ir*e. */
DPC_API int dpc_conv_update_state(dpc_conv_plan* plan, int layer);
/* g = e_above * mu: the gate the reference's UpdateWeights sees when no UpdateState ran since
 * the last CalculateState (its mu buffer then still holds the prediction, :414). */
DPC_API int dpc_conv_gate_with_prediction(dpc_conv_plan* plan, int layer);
/* UpdateWeights (SimpleConvPCLayer.cpp:402-556) + optional CenterWeights. */
DPC_API int dpc_conv_update_weights(dpc_conv_plan* plan, int layer, int center_rows);
DPC_API int dpc_conv_energy_reset(dpc_conv_plan* plan);
DPC_API int dpc_conv_energy_read(dpc_conv_plan* plan, double* out); /* synchronous */

/* The network with host buffers (include/deepity/networks/SimpleConvPCNetwork.h:30-131,
 * bindings/NetworkBindings.cpp:1850-2000). */
typedef struct dpcn_conv_net dpcn_conv_net;
DPC_API int dpcn_conv_create(int batch, int device, dpcn_conv_net** out);
DPC_API int dpcn_conv_destroy(dpcn_conv_net* net);
/* AddLayer(inChannels, outChannels, inHeight, inWidth, kernelH, kernelW, strideH, strideW,
 * padH, padW, lr, ir, lmbda, aType, dType). */
DPC_API int dpcn_conv_add_layer(dpcn_conv_net* net, int in_c, int out_c, int in_h, int in_w,
                                int k_h, int k_w, int s_h, int s_w, int p_h, int p_w, float lr,
                                float ir, float lmbda, int act);
/* "optimizer" (before compile), "center_weights", "learning_rate", "inference_rate",
 * "lambda", "use_graph". */
DPC_API int dpcn_conv_set_option(dpcn_conv_net* net, const char* name, int ivalue, float fvalue);
DPC_API int dpcn_conv_compile(dpcn_conv_net* net);
DPC_API int dpcn_conv_num_layers(dpcn_conv_net* net);
/* Per-layer geometry after compile: out[0..3] = out_c, out_h, out_w, in_c*k_h*k_w. */
DPC_API int dpcn_conv_layer_shape(dpcn_conv_net* net, int layer, int* out4);
/* names: "z" "e" "mu" "preact" "W" "b" "weight.m" "weight.v" "bias.m" "bias.v" */
DPC_API int64_t dpcn_conv_tensor_size(dpcn_conv_net* net, int layer, const char* name);
DPC_API int dpcn_conv_get_tensor(dpcn_conv_net* net, int layer, const char* name, float* host_out,
                                 int64_t count);
DPC_API int dpcn_conv_set_tensor(dpcn_conv_net* net, int layer, const char* name,
                                 const float* host_in, int64_t count);
DPC_API int dpcn_conv_randomize(dpcn_conv_net* net, uint32_t seed);
/* TrainStep / TrainStepWithProjection; on_device != 0: x and y are device pointers. */
DPC_API int dpcn_conv_train_step(dpcn_conv_net* net, const float* x, int64_t nx, const float* y,
                                 int64_t ny, int steps, int with_projection, int on_device,
                                 float* energy_out);
/* Predict / PredictWithProjection -> terminal beliefs into host_out. */
DPC_API int dpcn_conv_predict(dpcn_conv_net* net, const float* x, int64_t nx, int steps,
                              int with_projection, float* host_out, int64_t nout);
DPC_API dpc_ctx* dpcn_conv_context(dpcn_conv_net* net);
DPC_API dpc_conv_plan* dpcn_conv_plan(dpcn_conv_net* net);
DPC_API int64_t dpcn_conv_launch_count(dpcn_conv_net* net);

#ifdef __cplusplus
}
#endif
#endif /* DEEPITY_B200_H */
