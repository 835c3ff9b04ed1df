// Device primitives behind the DeepityCUDA plugin (libDeepityCUDA.so).
//
// The plugin's exported object implements the reference's backend interface
// (include/deepity/backend/IComputeBackend.h:18-625 of the reference); every one of its
// virtual methods forwards to one function of this header.  The split keeps the reference's
// own headers (which pull in SLEEF / x86 intrinsics) out of the CUDA translation unit:
// deepity_cuda_plugin.cpp is compiled by the host compiler against the reference's include
// tree, b200_backend.cu by nvcc against nothing but this header.
//
// Conventions: all pointers are device pointers unless named host*, all matrices fp32
// row-major, all work is ordered on the backend's one stream; functions marked SYNC wait
// for the stream.  Activation ids are the enumerators of Deep::ActivationType
// (include/deepity/utils/ActivationType.h:15-32): forward types are even, the matching
// derivative is forward + 1, NONE = 14.
#pragma once
#include <cstddef>
#include <cstdint>

namespace b200
{
struct Ctx; // stream, graph slots, tensor-map encoder, scratch for reductions

Ctx* create();         // nullptr when no usable CUDA device (the message goes to stderr)
void destroy(Ctx* c);

// ---- graphs, memory ---------------------------------------------------------------------
void graph_begin(Ctx* c, size_t slot);
bool graph_end(Ctx* c, size_t slot);
void graph_replay(Ctx* c, size_t slot);
void synchronize(Ctx* c);                                   // SYNC
float* allocate(Ctx* c, size_t n);                          // nullptr on failure
void release(Ctx* c, float* p);
void zero(Ctx* c, float* p, size_t n);
void copy(Ctx* c, float* dst, const float* src, size_t n);
void copy2d(Ctx* c, float* dst, size_t dst_stride, const float* src, size_t src_stride, size_t rows,
            size_t cols);
void copy_from_host(Ctx* c, float* dst, const float* host_src, size_t n); // SYNC
void copy_to_host(Ctx* c, float* host_dst, const float* src, size_t n);   // SYNC
void randomize_normal(Ctx* c, float* buf, size_t n, float mean, float stddev, uint32_t seed);
void randomize_uniform(Ctx* c, float* buf, size_t n, float lo, float hi, uint32_t seed);
uintptr_t stream_handle(const Ctx* c);

// ---- GEMM: C = alpha * op(A) * op(B) + beta * C (BLAS SGEMM on row-major operands) ----------
void set_allow_tf32(Ctx* c, bool allow);
void sgemm(Ctx* c, bool trans_a, bool trans_b, int M, int N, int K, float alpha, const float* A,
           int lda, const float* B, int ldb, float beta, float* C, int ldc);
// host arrays of device pointers, one GEMM per entry
void sgemm_batched(Ctx* c, bool trans_a, bool trans_b, int M, int N, int K, float alpha,
                   const float* const* host_A, int lda, const float* const* host_B, int ldb,
                   float beta, float* const* host_C, int ldc, int batch_count);

// ---- reductions ---------------------------------------------------------------------------
void sum_rows(Ctx* c, float* dst, const float* src, size_t batch, size_t width, size_t layers);
float sum(Ctx* c, const float* buf, size_t n);              // SYNC

// ---- elementwise --------------------------------------------------------------------------
void scale(Ctx* c, float* buf, size_t n, float alpha);
void axpy(Ctx* c, float* y, const float* x, size_t n, float alpha);
void add_bias(Ctx* c, float* buf, const float* bias, size_t batch, size_t width, size_t layers);
void add_bias_per_channel(Ctx* c, float* buf, const float* bias, size_t batch, size_t channels,
                          size_t spatial);
void multiply(Ctx* c, float* dst, const float* a, const float* b, size_t n);
void fill(Ctx* c, float* buf, size_t n, float value);
void center_rows(Ctx* c, float* buf, size_t rows, size_t cols);
void axpy_broadcast(Ctx* c, float* y, const float* x, const float* factor, size_t batch,
                    size_t width, float alpha);
void multiply_broadcast(Ctx* c, float* dst, const float* a, const float* factor, const float* b,
                        size_t batch, size_t width);

// ---- activations (type = Deep::ActivationType enumerator) ----------------------------------
void activation(Ctx* c, int type, float* dst, const float* src, size_t n); // dst may equal src
// derivative-flavoured type; from_activated: src holds f(z) instead of z
void activation_derivative(Ctx* c, int dtype, float* dst, const float* src, size_t n,
                           bool from_activated);
// dst = a * f'(x); write_back: x is then overwritten with f'(x) (x holds the activated value)
void derivative_multiply(Ctx* c, int dtype, float* dst, const float* a, float* x, size_t n,
                         bool from_activated, bool write_back);

// ---- predictive-coding ops ------------------------------------------------------------------
void state_update(Ctx* c, float* z, float* v /*or nullptr*/, const float* feedback, int dtype,
                  const float* e, size_t n, float ir, float beta);
void compute_error(Ctx* c, float* e, const float* z, const float* mu, size_t n);
float compute_error_energy(Ctx* c, float* e, const float* z, const float* mu, size_t n); // SYNC
void error_and_activation(Ctx* c, int type, float* e, float* zf, const float* z, const float* mu,
                          size_t n);
void softmax_ce_error(Ctx* c, float* e, const float* z, const float* mu, size_t batch, size_t width);
float softmax_ce_error_energy(Ctx* c, float* e, const float* z, const float* mu, size_t batch,
                              size_t width); // SYNC
void precision_error(Ctx* c, float* e, const float* z, const float* mu, const float* p, size_t batch,
                     size_t width);
float precision_error_energy(Ctx* c, float* e, const float* z, const float* mu, const float* p,
                             size_t batch, size_t width); // SYNC
void update_precision(Ctx* c, float* p, float* log_p, const float* e, size_t batch, size_t width,
                      float pr);

// ---- convolution helpers --------------------------------------------------------------------
void im2col(Ctx* c, const float* input, int batch, int channels, int height, int width, int kh, int kw,
            int sh, int sw, int ph, int pw, float* columns);
void col2im(Ctx* c, const float* columns, int batch, int channels, int height, int width, int kh, int kw,
            int sh, int sw, int ph, int pw, float* image);
void maxpool_forward(Ctx* c, const float* input, int batch, int channels, int height, int width, int ph,
                     int pw, int sh, int sw, float* output, int* argmax);
void maxpool_backward(Ctx* c, const float* out_grad, const int* argmax, int batch, int channels,
                      int height, int width, int out_h, int out_w, float* in_grad);
void repack_for_batched_gemm(Ctx* c, float* dst, const float* src, size_t batch, size_t rows,
                             size_t cols);

// ---- optimizer ------------------------------------------------------------------------------
void increment_counter(Ctx* c, int* counter);
void counter_to_host(Ctx* c, int* host_dst, const int* counter);   // SYNC
void counter_from_host(Ctx* c, int* counter, const int* host_src); // SYNC
// t and lr are read on the device; weight_decay < 0: plain Adam
void adam(Ctx* c, float* param, const float* grad, float* m, float* v, size_t n, const int* t,
          const float* lr, float weight_decay, float beta1, float beta2, float eps);
} // namespace b200
