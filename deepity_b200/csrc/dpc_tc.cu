// Tensor-core path: grouped, persistent, warp-specialised GEMM kernels for sm_100a.
//
//   * operands staged by TMA (cp.async.bulk.tensor, 128-byte swizzle) into a multi-stage
//     shared-memory ring, one tensor map per operand with the LAYER as outermost coordinate,
//     so one launch walks every (layer, tile) of a run of identical square layers;
//   * tcgen05.mma (kind::tf32, M=128, N=128|256, K=8) issued by one thread, fp32 accumulators
//     in tensor memory, double-buffered so the epilogue of tile i overlaps the main loop of
//     tile i+1;
//   * fp32 mode, scheme 1 = 3xTF32: the raw fp32 tile feeds the tensor core as the "high" part
//     (the hardware reads the top 19 bits), four extra warps compute the exact remainders into a
//     second pair of tiles, and each k-step issues A*B_lo + A_lo*B + A*B;
//   * fp32 mode, scheme 2 = 3xBF16 (kind::f16): the four extra warps split the raw tile into
//     bf16(x) and bf16(x - bf16(x)) tiles in a second ring of slots, rewritten into the bf16
//     operand layouts (K-major 64-byte swizzle, MN-major 128-byte swizzle), and each k-step
//     issues hi*mid + mid*hi + hi*hi: half the tensor-pipe time and power of scheme 1 at a
//     per-product error of 2^-16, used when every weight optimizer is SGD;
//   * fp32 mode, scheme 3 = 3xBF16 from PRE-SPLIT operands: every kernel of this file that writes a
//     belief, a feedback error or a weight of the run also writes its bf16 "hi" and "mid" planes
//     (same bytes as the fp32 tensor), so the grouped kernels load tensor-core-ready tiles by TMA
//     (128-byte rows of 64 bf16, 128-byte swizzle) and run the one-ring pipeline of the TF32 mode
//     with three MMAs per k-step: same arithmetic as scheme 2, no split warps, no second ring;
//   * the predictive-coding elementwise work runs in the epilogue straight out of tensor
//     memory: bias + activation + error + energy + feedback error (forward), the state
//     update (feedback), the SGD weight update (weight-shaped product).
//
// Three operand layouts are needed (row-major fp32 everywhere):
//   forward   D[B,n]  = z[B,s]  · W[n,s]^T      A K-major,  B K-major
//   feedback  D[B,s]  = fe[B,n] · W[n,s]        A K-major,  B MN-major
//   weights   D[n,s]  = fe[B,n]^T · z[B,s]      A MN-major, B MN-major
//
// Every wait on an mbarrier is bounded by a clock; on expiry the kernel raises a flag in
// global memory, all roles drain and the CTA frees its tensor memory and returns.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include <cuda_bf16.h>

#include "dpc_internal.h"
#include "dpc_math.cuh"
#include "dpc_tcgen05.cuh"

namespace dpc
{
namespace
{
constexpr int TBM = 128;  // UMMA M (rows of D per tile)
constexpr int TBK = 32;   // fp32 elements per pipeline stage along K = one 128-byte swizzle row
constexpr int UMMA_K = 8; // K of one tcgen05.mma.kind::tf32
using namespace ptx; // mbarriers, TMA, tcgen05, descriptors: dpc_tcgen05.cuh

enum
{
  TC_FWD = 0,
  TC_FB = 1,
  TC_WG = 2
};
constexpr int WG_LEARN_MODE = 0, WG_DFA_MODE = 1, WG_GRAD_MODE = 2; // GRAD is or-ed in

struct TcState
{
  bool ok = false;
  CUtensorMap z_km, z_km64, fe_km, w_km32, w_km64, w_km128, w_km256, z_mn, fe_mn, w_mn;
  // beliefs / errors of the run's layers AND the layer above its last one (layer coordinate
  // l+1 = the layer above l): what the forward epilogue reads, staged through shared memory
  CUtensorMap zup_km, eup_km;
  bool up_maps = false;
  int* chain_counters = nullptr; // device: [layers of the run][row blocks]
  unsigned long long* trace = nullptr; // optional timing trace buffer of the chain kernel
  int* error_flag = nullptr; // device
  int* error_host = nullptr; // pinned
  int max_smem = 0;
  long long wait_cycles = kWaitCyclesDefault;
  int chain_target_bias = 0; // test hook: added to the sweep's publication target
  // Pre-split operand planes (bf16 hi/mid) of the run's beliefs (count+1 layers), feedback
  // errors and weights, their tensor maps (layer coordinate 2l + plane) and, per layer, whether
  // the planes lag behind the fp32 tensor (1 = must be re-split before a kernel reads them).
  __nv_bfloat16 *zp = nullptr, *fep = nullptr, *wp = nullptr;
  CUtensorMap zp_km, zp_km64, zp_mn, fep_km, fep_mn, wp_km128, wp_km64, wp_mn;
  CUtensorMap e_st, fep_st; // bulk-store maps: errors (fp32) and feedback-error planes (bf16)
  CUtensorMap z_st, zp_st;  // beliefs (fp32) and their planes, for the feedback kernel
  CUtensorMap w_st, wp_st;  // weights (fp32) and their planes, for the weight kernel
  bool store_maps = false;
  std::vector<uint8_t> dirty[3];
  bool planes = false;
  // The run's feedback errors exist only as planes: every reader of them is a kernel that takes
  // the planes (feedback and weight-shaped products of this file, the bias column sums).
  bool fe_only = false;
  bool warned_fallback = false;
  // Single layers outside the run that still fit the CTA-pair kernels (batch and output width
  // multiples of 256, input width a multiple of 8, e.g. a 3072 -> 1024 or a 784 -> 256 first
  // layer): one set of tensor maps each.
  // SimplePC layers (DPC_LAYER_INPUT_ACT) multiply f(z) instead of z and the error of the layer
  // above instead of a feedback error: for them z_* cover zF and fe_* cover e of the layer above.
  struct Extra
  {
    int layer;
    bool simple;
    CUtensorMap z_km, w_km128, fe_km, w_mn, fe_mn, z_mn;
  };
  std::vector<Extra> extras;
};
enum
{
  PL_Z = 0,
  PL_FE = 1,
  PL_W = 2
};

struct TcParams
{
  const dpc_layer* layers;
  int first, count, n_layers, batch;
  int run_first;
  int M, N, K;
  int tiles_m, tiles_n;
  int flags, mode;
  double* energy;
  int* error_flag;
  // Chain mode (the sequential forward sweep): CTA b owns output tile b of EVERY layer and
  // walks the layers in order; chain_counters[layer][row block] counts the CTAs
  // that have published their part of the next layer's input rows.
  int chain;
  int* chain_counters;
  int chain_target;
  // Optional timing trace of the chain kernel (NULL in normal use): for CTA 0 and the first
  // 256 layers, globaltimer stamps of [dependency seen, first operands landed, accumulator
  // complete, epilogue stores issued, published].
  unsigned long long* trace;
  // Pair-mode forward: 0 = the epilogue reads nothing from the layer above, 1 = its belief
  // (tensor map mapU covers the z arena), 2 = its stored error (mapU covers the e arena); the
  // tile is then brought into shared memory by TMA instead of per-lane global loads.
  int stage_in;
  // Pre-split operand planes of the run (NULL: not maintained by this launch).  Layer r of the
  // run (r = layer - run_first) has its "hi" plane at base + 2r * elems and its "mid" plane at
  // base + (2r+1) * elems; beliefs have one layer more than the run (the layer above it).
  __nv_bfloat16 *zp, *fep, *wp;
  long long act_elems, w_elems; // elements per plane: batch x width, width x width
  long long wait_cycles;        // limit of every bounded wait of this launch
  int fe_only;                  // the fp32 feedback error of the run's layers is not written
  int tstore;                   // the store maps of the launch are valid (staged epilogue outputs)
};

// Chain mode: wait (bounded) until `target` epilogue warps have published one row block of the
// previous layer's output, then order the TMA (async proxy) reads after that observation.
__device__ __forceinline__ bool chain_wait(const int* ctr, int target, volatile int* abort_flag)
{
  const long long t0 = clock64();
  for (;;)
  {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(ctr) : "memory");
    if (v >= target)
      break;
    if (*abort_flag)
      return false;
    if (clock64() - t0 > wait_limit(abort_flag))
    {
      *abort_flag = 1;
      return false;
    }
  }
  // (the proxy fence restricted to global memory: the full one also drains shared-memory
  // traffic and costs about 0.4 us more per layer of the sweep)
  asm volatile("fence.proxy.async.global;" ::: "memory");
  return true;
}

__device__ __forceinline__ void trace_stamp(const TcParams& P, int layer, int slot)
{
  if (P.trace && blockIdx.x == 0 && layer < 256)
  {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    P.trace[layer * 8 + slot] = t;
  }
}

// Forward epilogue of one 128 x BN tile for the 32 rows of one warp.  ACT >= 0 fixes the
// activation at compile time (the per-element switch disappears), ACT < 0 reads it from the
// layer.  The operand read from the layer above is fetched one chunk ahead when PREFETCH.
// The fields of the layer table the forward epilogue needs, fetched BEFORE the warp waits for
// the accumulator so their latency overlaps the main loop (registers are scarce: only these).
// ---- BF16 split of a raw fp32 tile (THREE_X == 2): hi = bf16(x), mid = bf16(x - hi); the three
// products hi*mid, mid*hi, hi*hi drop terms of relative size 2^-16 only.
__device__ __forceinline__ void split8(const float4& a, const float4& b, uint4& hi, uint4& mid)
{
  auto two = [](float x0, float x1, uint32_t& h, uint32_t& m) {
    const __nv_bfloat162 hh = __floats2bfloat162_rn(x0, x1);
    const __nv_bfloat162 mm = __floats2bfloat162_rn(x0 - __low2float(hh), x1 - __high2float(hh));
    h = *reinterpret_cast<const uint32_t*>(&hh);
    m = *reinterpret_cast<const uint32_t*>(&mm);
  };
  two(a.x, a.y, hi.x, mid.x);
  two(a.z, a.w, hi.y, mid.y);
  two(b.x, b.y, hi.z, mid.z);
  two(b.z, b.w, hi.w, mid.w);
}
// Eight consecutive elements of a tensor into its two operand planes (16-byte stores).
__device__ __forceinline__ void st_planes8(__nv_bfloat16* hi, long long plane_elems, size_t off,
                                           const float* v)
{
  uint4 h, m;
  split8(make_float4(v[0], v[1], v[2], v[3]), make_float4(v[4], v[5], v[6], v[7]), h, m);
  *reinterpret_cast<uint4*>(hi + off) = h;
  *reinterpret_cast<uint4*>(hi + plane_elems + off) = m;
}
// K-major.  Raw: ROWS rows of 32 floats, 128 bytes per row, 16-byte chunks xor-ed with (row & 7)
// (what TMA's 128-byte swizzle wrote).  Out: ROWS rows of 32 bf16, 64 bytes per row, atoms of 8
// rows, 16-byte chunks xor-ed with ((row >> 1) & 3): the K-major 64-byte-swizzle operand layout.
// Eight neighbouring lanes take the eight rows of an atom: loads and stores are conflict-free.
template <int ROWS>
__device__ __forceinline__ void split_kmajor(const uint8_t* raw, uint8_t* hi, uint8_t* mid, int tid)
{
  // work item idx = tid + 128 j covers row r0 + 32 j, k-chunk kc: the swizzle terms depend on
  // (r & 7) only, so they are per-thread constants.  All loads are issued before any store (the
  // compiler cannot prove that the output tiles do not alias the raw one).
  constexpr int NIT = ROWS * 4 / 128;
  const int r0 = ((tid >> 5) << 3) | (tid & 7), kc = (tid >> 3) & 3;
  if (ROWS * 4 < 128 && tid >= ROWS * 4)
    return;
  const uint8_t* src0 = raw + r0 * 128 + (((2 * kc) ^ (r0 & 7)) << 4);
  const uint8_t* src1 = raw + r0 * 128 + (((2 * kc + 1) ^ (r0 & 7)) << 4);
  const int off = (r0 >> 3) * 512 + (r0 & 7) * 64 + ((kc ^ ((r0 >> 1) & 3)) << 4);
  constexpr int N = NIT > 0 ? NIT : 1;
  float4 a[N], b[N];
#pragma unroll
  for (int j = 0; j < N; ++j)
  {
    a[j] = *reinterpret_cast<const float4*>(src0 + j * 4096);
    b[j] = *reinterpret_cast<const float4*>(src1 + j * 4096);
  }
#pragma unroll
  for (int j = 0; j < N; ++j)
  {
    uint4 h, m;
    split8(a[j], b[j], h, m);
    *reinterpret_cast<uint4*>(hi + off + j * 2048) = h;
    *reinterpret_cast<uint4*>(mid + off + j * 2048) = m;
  }
}
// MN-major.  Raw: slabs of 32 columns, each 32 k-rows of 128 bytes, 32-byte units xor-ed with
// (k & 3).  Out: blocks of 64 columns, each 32 k-rows of 128 bytes (64 bf16), 16-byte chunks
// xor-ed with (k & 7): the MN-major 128-byte-swizzle operand layout.  Neighbouring lanes pair rows
// k and k+4 and read their halves in opposite order, which keeps loads and stores conflict-free.
template <int E>
__device__ __forceinline__ void split_mnmajor(const uint8_t* raw, uint8_t* hi, uint8_t* mid, int tid)
{
  // work item idx = tid + 128 j covers slab j, k-row k, 32-byte unit u: per-thread constants
  constexpr int N = E / 32;
  const int l = tid & 31, p = l & 1, u = (l >> 1) & 3;
  const int k = ((tid >> 5) << 3) + (l >> 3) + (p << 2);
  const uint8_t* unit = raw + k * 128 + ((u ^ (k & 3)) << 5);
  float4 first[N], second[N];
#pragma unroll
  for (int j = 0; j < N; ++j)
  {
    first[j] = *reinterpret_cast<const float4*>(unit + j * 4096 + (p << 4));
    second[j] = *reinterpret_cast<const float4*>(unit + j * 4096 + ((p ^ 1) << 4));
  }
#pragma unroll
  for (int j = 0; j < N; ++j)
  {
    // (first, second) is (upper, lower) half on odd lanes: convert in load order, then put the
    // packed words in column order with selects instead of a divergent branch
    uint4 h, m;
    split8(first[j], second[j], h, m);
    if (p)
    {
      h = make_uint4(h.z, h.w, h.x, h.y);
      m = make_uint4(m.z, m.w, m.x, m.y);
    }
    const int c = ((j & 1) << 2) | u;
    const int off = (j >> 1) * 4096 + k * 128 + ((c ^ (k & 7)) << 4);
    *reinterpret_cast<uint4*>(hi + off) = h;
    *reinterpret_cast<uint4*>(mid + off) = m;
  }
}

struct FwdMeta
{
  float a;
  int flags, act, up_flags;
  const float* b;
  const float* z;
  float *preact, *mu, *fe, *up_z, *up_e;
  __nv_bfloat16 *fe_hi, *upz_hi; // operand planes of fe[l] and z[l+1], or NULL
};

__device__ __forceinline__ void load_fwd_meta(const TcParams& P, int li, FwdMeta& M)
{
  const dpc_layer* Lp = &P.layers[li];
  M.a = Lp->a, M.flags = Lp->flags, M.act = Lp->act, M.b = Lp->b, M.z = Lp->z;
  // SimplePC: the activation was applied to the operand (zF = f(z)); the prediction is linear
  if (Lp->flags & DPC_LAYER_INPUT_ACT)
    M.act = DPC_ACT_LINEAR;
  M.preact = Lp->preact, M.mu = Lp->mu, M.fe = Lp->fe;
  if (li + 1 < P.n_layers)
  {
    const dpc_layer* Lup = Lp + 1;
    M.up_z = Lup->z, M.up_e = Lup->e, M.up_flags = Lup->flags;
  }
  else
    M.up_z = M.up_e = nullptr, M.up_flags = 0;
  const long long r = li - P.run_first;
  M.fe_hi = P.fep ? P.fep + 2 * r * P.act_elems : nullptr;
  M.upz_hi = P.zp ? P.zp + 2 * (r + 1) * P.act_elems : nullptr;
}

// Where the staged operand of the layer above sits (pair-mode forward only).
struct InStage
{
  const uint8_t* buf; // IN_BUFS buffers of 128 rows x 128 bytes, 128-byte swizzle
  uint64_t* full;
  uint64_t* empty;
  uint32_t seq;  // sequence number of this tile's first 32-column box
  int row;       // this lane's row inside the 128-row box
  int nbufs;     // power of two
  volatile int* abort_flag;
  const uint8_t* rx; // K-split sweep: the peer's partial sums for this CTA's 32 columns
  // Output staging (pair-mode forward on pre-split operands): this warp's two 4 KB buffers
  // ([e: 32 rows x 64 B][fe hi: 32 x 32 B][fe mid: 32 x 32 B]), the running count of chunks it
  // has staged, the store maps and the coordinates of its 32 rows.  out == NULL: direct stores.
  uint8_t* out;
  uint32_t* out_seq;
  const CUtensorMap *map_e, *map_fe;
  int out_row0, layer_e, layer_fe;
  // Sequential sweep: the fp32 copy of the belief a lane produced (16 columns) is kept in
  // registers and stored after the row block has been published; only the operand planes, which
  // the next layer's tensor cores read, are on the dependent path.  NULL: stored at once.
  float* defer;
  size_t* defer_o;
};

template <int ACT, int BN, int GROUPS, bool PREFETCH, bool STAGED = false, bool KSUM = false,
          int ACC_STRIDE = 0>
__device__ __forceinline__ void fwd_epilogue_tile(const TcParams& P, const FwdMeta& L,
                                                  const float* bias_pre, uint32_t taddr, int m,
                                                  int n0, int grp, float& esum, int tl,
                                                  bool active, const InStage* in = nullptr)
{
  const int act = ACT >= 0 ? ACT : L.act;
  const bool Lup = L.up_z != nullptr;
  const bool next_ce = Lup && (L.up_flags & DPC_LAYER_SOFTMAX_CE);
  const bool do_err = (P.flags & DPC_FWD_ERR_NEXT) && Lup && !next_ce;
  const bool do_fe = (P.flags & DPC_FWD_FE) && Lup && !(L.flags & DPC_LAYER_INPUT_ACT) &&
                     !(next_ce && (P.flags & DPC_FWD_ERR_NEXT));
  const bool do_copy = (P.flags & DPC_FWD_COPY_NEXT) && Lup;
  const bool store = !(P.flags & DPC_FWD_TRANSIENT);
  // bit 10 (internal): the launch starts at the first layer of the sweep, whose mu is kept
  const bool no_mu = do_copy && (P.flags & DPC_FWD_NO_MU) && !((P.flags & (1 << 10)) && tl == 0);
  const bool residual = (L.flags & DPC_LAYER_RESIDUAL) != 0;
  float* up_z = L.up_z;
  float* up_e = L.up_e;
  // What the epilogue reads from the layer above: its belief (fresh error) or its stored
  // error (feedback error from the error already in memory).
  const float* up_src_all = (do_err && !do_copy) ? up_z : ((do_fe && !do_err) ? up_e : nullptr);
  const float* up_src = up_src_all;
  const size_t row = (size_t)m * P.N + n0;
  constexpr int CW = 16; // columns per step
  float up[CW], upn[CW];
  if (!active)
    up_src = nullptr; // lanes that hold no accumulator row touch no memory
  const bool staged = STAGED && P.stage_in != 0 && up_src_all != nullptr;
  if (staged)
    up_src = nullptr; // the operand comes from shared memory, box by box
  // Errors and feedback-error planes leave through shared memory and bulk tensor stores (whole
  // 64- and 32-byte row segments per store instead of one 32-byte sector per lane and
  // instruction): only in the passes that write nothing else.
  const bool tstore = STAGED && in->out != nullptr && !store && !do_copy && (do_err || do_fe) &&
                      (!do_fe || (P.fe_only && L.fe_hi != nullptr));
  const int lane = threadIdx.x & 31;
  if (up_src)
  {
#pragma unroll
    for (int k = 0; k < CW; k += 8)
      ld8(up_src + row + grp * CW + k, &up[k]);
  }
#pragma unroll 1
  for (int c = grp; c < BN / CW; c += GROUPS)
  {
    const size_t o = row + c * CW;
    float v[CW];
    if (STAGED && staged)
    {
      // 16 columns = one half of a 32-column box; every epilogue warp visits every box once
      const uint32_t q = in->seq + (uint32_t)(c >> 1);
      const uint32_t b = q & (uint32_t)(in->nbufs - 1);
      const uint32_t par = (q / (uint32_t)in->nbufs) & 1u;
      if (!mbar_wait(&in->full[b], par, in->abort_flag))
        return;
      const uint8_t* rowp = in->buf + (size_t)b * (128 * 128) + in->row * 128;
#pragma unroll
      for (int i = 0; i < 4; ++i)
      {
        const int ch = (((c & 1) << 2) + i) ^ (in->row & 7);
        const float4 x = *reinterpret_cast<const float4*>(rowp + ch * 16);
        up[4 * i] = x.x, up[4 * i + 1] = x.y, up[4 * i + 2] = x.z, up[4 * i + 3] = x.w;
      }
      __syncwarp();
      if ((threadIdx.x & 31) == 0)
        mbar_arrive(&in->empty[b]);
    }
    uint8_t* obuf = nullptr;
    if (STAGED && tstore)
    {
      // the buffer staged two chunks ago must have been read by its stores
      obuf = in->out + ((*in->out_seq) & 1u) * 4096u;
      if (lane == 0)
        bulk_wait_read<1>();
      __syncwarp();
    }
    tc_ld16(taddr + c * CW, v);
    if (ACC_STRIDE > 0)
    {
      // the hi*mid products were accumulated beside the tile (see Cfg::NACC)
      float v1[CW];
      tc_ld16(taddr + ACC_STRIDE + c * CW, v1);
#pragma unroll
      for (int i = 0; i < CW; ++i)
        v[i] += v1[i];
    }
    if (KSUM)
    {
      // add the other CTA's half of the K sum (rows of 128 bytes, 16-byte chunks swizzled by row)
      const uint8_t* rowp = in->rx + in->row * 128;
#pragma unroll
      for (int i = 0; i < 4; ++i)
      {
        const float4 x = *reinterpret_cast<const float4*>(rowp + (((c * 4 + i) ^ (in->row & 7)) << 4));
        v[4 * i] += x.x, v[4 * i + 1] += x.y, v[4 * i + 2] += x.z, v[4 * i + 3] += x.w;
      }
    }
    if (tl >= 0 && c == grp && threadIdx.x == 64)
      trace_stamp(P, tl, 5);
    if (PREFETCH && up_src && c + GROUPS < BN / CW)
    {
#pragma unroll
      for (int k = 0; k < CW; k += 8)
        ld8(up_src + o + GROUPS * CW + k, &upn[k]);
    }
#pragma unroll
    for (int k = 0; k < CW; k += 8)
    {
      float bb[8], pre[8], mu[8], d[8], e[8];
      if (BN / GROUPS <= 32)
      {
#pragma unroll
        for (int q = 0; q < 8; ++q)
          bb[q] = bias_pre[((c - grp) / GROUPS) * CW + k + q];
      }
      else
        ld8(L.b + n0 + c * CW + k, bb);
#pragma unroll
      for (int q = 0; q < 8; ++q)
        pre[q] = L.a * v[k + q] + bb[q];
      if (do_fe)
        act_both8<true>(act, pre, mu, d);
      else
        act_both8<false>(act, pre, mu, d);
      if (residual && active)
      {
        float zz[8];
        ld8(L.z + o + k, zz);
#pragma unroll
        for (int q = 0; q < 8; ++q)
          mu[q] += zz[q];
      }
      if (store && active)
      {
        if (L.preact && !(no_mu && (P.flags & DPC_FWD_NO_PREACT))) // (SimplePC keeps no preact)
          st8(L.preact + o + k, pre);
        if (!no_mu)
          st8(L.mu + o + k, mu);
      }
      if (do_copy && active)
      {
        if (BN / GROUPS == 16 && in && in->defer)
        {
#pragma unroll
          for (int q = 0; q < 8; ++q)
            in->defer[k + q] = mu[q];
          *in->defer_o = o;
        }
        else
        st8(up_z + o + k, mu);
        if (L.upz_hi)
          st_planes8(L.upz_hi, P.act_elems, o + k, mu);
      }
      if (do_err)
      {
#pragma unroll
        for (int q = 0; q < 8; ++q)
        {
          e[q] = (do_copy || !active) ? 0.0f : up[k + q] - mu[q];
          esum += e[q] * e[q];
        }
        if (STAGED && tstore)
        {
          // 64-byte rows, 16-byte chunks xor-ed with (row >> 1) & 3: the 64-byte swizzle
          const int q = k >> 2;
          *reinterpret_cast<float4*>(obuf + lane * 64 + ((q ^ ((lane >> 1) & 3)) << 4)) =
              make_float4(e[0], e[1], e[2], e[3]);
          *reinterpret_cast<float4*>(obuf + lane * 64 + (((q + 1) ^ ((lane >> 1) & 3)) << 4)) =
              make_float4(e[4], e[5], e[6], e[7]);
        }
        else if (active)
          st8(up_e + o + k, e);
      }
      else if (do_fe)
      {
#pragma unroll
        for (int q = 0; q < 8; ++q)
          e[q] = active ? up[k + q] : 0.0f;
      }
      if (do_fe)
      {
#pragma unroll
        for (int q = 0; q < 8; ++q)
          e[q] *= d[q];
        if (STAGED && tstore)
        {
          // 32-byte rows, 16-byte chunks xor-ed with (row >> 2) & 1: the 32-byte swizzle
          uint4 h, mm;
          split8(make_float4(e[0], e[1], e[2], e[3]), make_float4(e[4], e[5], e[6], e[7]), h, mm);
          const int off = lane * 32 + ((((k >> 3) & 1) ^ ((lane >> 2) & 1)) << 4);
          *reinterpret_cast<uint4*>(obuf + 2048 + off) = h;
          *reinterpret_cast<uint4*>(obuf + 3072 + off) = mm;
        }
        else if (active)
        {
          if (!P.fe_only)
            st8(L.fe + o + k, e);
          if (L.fe_hi)
            st_planes8(L.fe_hi, P.act_elems, o + k, e);
        }
      }
      if (tl >= 0 && c == grp && k == 0 && threadIdx.x == 64)
        trace_stamp(P, tl, 6);
    }
    if (STAGED && tstore)
    {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0)
      {
        const int col = n0 + c * CW;
        if (do_err)
          tma_store_3d(in->map_e, obuf, col, in->out_row0, in->layer_e);
        if (do_fe)
        {
          tma_store_3d(in->map_fe, obuf + 2048, col, in->out_row0, 2 * in->layer_fe); // hi + mid
        }
        bulk_commit();
      }
      *in->out_seq += 1;
    }
    if (up_src && c + GROUPS < BN / CW)
    {
      if (PREFETCH)
      {
#pragma unroll
        for (int k = 0; k < CW; ++k)
          up[k] = upn[k];
      }
      else
      {
#pragma unroll
        for (int k = 0; k < CW; k += 8)
          ld8(up_src + o + GROUPS * CW + k, &up[k]);
      }
    }
  }
}

// ------------------------------------------------------------------------------ kernel
// Warp roles: 0 TMA producer, 1 MMA issuer (+ tensor-memory owner), 2..9 epilogue,
// 10..13 operand split (fp32 modes only): THREE_X == 1 writes the TF32 remainder tile beside the
// raw one; THREE_X == 2 reads the raw tile and writes bf16 "hi" and "mid" tiles into a second ring.
// PAIR: two CTAs of a cluster (cta_group::2) compute one 256 x BN tile.  Each CTA stages its own
// 128 rows of A and its own half of B (BN/2 rows) and holds its 128 rows of the accumulator in
// its own tensor memory, so per output element half as many operand bytes cross L2 -> SM and
// shared memory as with two independent 128 x BN/2 tiles.
// KS = 2 (sequential sweep only): two CTAs of a cluster share one 128 x BN tile, each running
// the main loop over half of K; they exchange the half of the partial tile the other one
// finishes through distributed shared memory.  Halves every CTA's operand traffic per layer.
template <int OP, int BN, int THREE_X, int BM = 128, bool PAIR = false, int KS = 1>
struct Cfg
{
  static constexpr int RX_BYTES = KS == 2 ? 128 * 32 * 4 : 0; // partial tile from the peer
  static constexpr bool A_MN = (OP == TC_WG);
  static constexpr bool B_MN = (OP != TC_FWD);
  static constexpr int BN_LOCAL = PAIR ? BN / 2 : BN; // rows of B this CTA stages
  static constexpr int TILE_M = PAIR ? 2 * BM : BM;   // rows of D per work item
  // THREE_X: 0 one TF32 pass; 1 three TF32 passes over (x, x - tf32(x)); 2 three BF16 passes over
  // (bf16(x), bf16(x - bf16(x))) split in the kernel, at twice the tensor rate; 3 the same three
  // BF16 passes over operand planes that were split when the tensors were written.
  static constexpr bool B16 = THREE_X == 2;
  static constexpr bool PRE = THREE_X == 3;
  static constexpr bool BF = B16 || PRE;                  // bf16 MMAs (K = 16 per instruction)
  static constexpr bool SPLITW = THREE_X == 1 || THREE_X == 2; // four operand-split warps
  static constexpr int KB = PRE ? 64 : TBK; // elements of K per pipeline stage (128-byte rows)
  // PRE: [hi plane][mid plane] of each operand, 2 bytes per element
  static constexpr int A_BYTES = PRE ? BM * 64 * 2 * 2 : BM * TBK * 4;
  static constexpr int B_BYTES = PRE ? BN_LOCAL * 64 * 2 * 2 : BN_LOCAL * TBK * 4;
  static constexpr int RAWB = A_BYTES + B_BYTES;
  // B16: two rings of RAWB-byte slots.  NR raw slots (TMA -> split warps) are held only while a
  // load is in flight and being split; NB slots of [A hi][A mid][B hi][B mid] (split warps ->
  // tensor core) only while the MMAs read them.  Otherwise one ring of STAGES stages.
  static constexpr int SLOTS_RAW = (196608 - RX_BYTES) / RAWB;
  static constexpr int NB = 2; // (3 + 3 slots measured the same as 4 + 2)
  static constexpr int NR = SLOTS_RAW - NB > 6 ? 6 : (SLOTS_RAW - NB < 2 ? 2 : SLOTS_RAW - NB);
  static constexpr int STAGE_BYTES = B16 ? RAWB : RAWB * (THREE_X == 1 ? 2 : 1);
  // at most 8 stages: the barrier block after the ring is sized for that
  static constexpr int STAGES_RAW =
      (196608 - ((PAIR && OP == TC_FWD && !THREE_X) ? 4 * BM * 32 * 4 : 0) - RX_BYTES) / STAGE_BYTES;
  // The K-split sweep on pre-split operands has four k-blocks per layer: with four stages all of a
  // layer's operands are in flight at once (three stages left the fourth k-block waiting for a
  // stage to drain: one more load latency on the dependent path of every layer).
  static constexpr bool TSTORE = PRE && PAIR && OP == TC_FWD; // staged epilogue outputs
  // Pair-mode feedback kernel on pre-split operands: the error and the belief of the tile come in
  // through shared memory (16-column boxes filled by a TMA warp), the updated belief is written
  // back into its box and leaves, with its operand planes, through bulk tensor stores.
  static constexpr bool FBIO = PRE && PAIR && OP == TC_FB;
  // ... and the weight kernel likewise: the weight tile comes in through 16-column boxes, is
  // updated in place and leaves with its planes through bulk tensor stores.
  static constexpr bool WGIO = PRE && PAIR && OP == TC_WG;
  static constexpr int STAGES = B16 ? NR
                                : (TSTORE || FBIO || WGIO) ? 2
                                : (PRE && KS == 2) ? 4
                                : (STAGES_RAW < 2 ? 2 : (STAGES_RAW > 8 ? 8 : STAGES_RAW));
  static constexpr int RING_BYTES = B16 ? (NR + NB) * RAWB : STAGES * STAGE_BYTES;
  static constexpr int EPI_WARPS = 8;
  static constexpr int THREADS =
      (2 + EPI_WARPS + (SPLITW ? 4 : 0) + ((PAIR && (OP == TC_FWD || FBIO || WGIO)) ? 1 : 0)) * 32;
  // K-split sweep on pre-split operands: a narrow tile's main loop is bound by the shared-memory
  // reads of its MMAs (every tcgen05.mma reads its A and B tiles again: 6 KB for 128x64x16).  The
  // "hi" and "mid" tiles of B lie back to back in a stage, so ONE instruction with N = 2 BN
  // multiplies A_hi with both (columns [0,BN) = hi*hi, [BN,2BN) = hi*mid) and a second one adds
  // A_mid * B_hi to the first half: 14 KB instead of 18 KB per k-step, two instructions instead of
  // three.  The epilogue adds the two halves.
  static constexpr int NACC = (PRE && KS == 2) ? 2 : 1;
  static constexpr uint32_t IDESC_WIDE = (1u << 4) | (1u << 7) | (1u << 10) |
                                         ((uint32_t)((2 * BN) >> 3) << 17) |
                                         ((uint32_t)((PAIR ? 2 * BM : BM) >> 4) << 24);
  static constexpr int TMEM_RAW = 2 * BN * NACC;
  static constexpr int TMEM_COLS = TMEM_RAW <= 32 ? 32 : TMEM_RAW <= 64 ? 64 : TMEM_RAW <= 128 ? 128
                                   : TMEM_RAW <= 256 ? 256 : 512;
  // Pair-mode forward: the operand of the layer above (128 rows x 32 columns per box, 16 KB)
  // arrives through IN_BUFS shared-memory buffers filled by a dedicated TMA warp.
  static constexpr bool STAGE_IN = PAIR && OP == TC_FWD;
  // FBIO: [error: 128 rows x 64 B][belief: 128 rows x 64 B] per buffer, 64-byte swizzle
  // WGIO: [weights: 128 rows x 64 B] per buffer
  static constexpr int IN_BYTES = FBIO ? 2 * BM * 16 * 4 : WGIO ? BM * 16 * 4 : BM * 32 * 4;
  static constexpr int IN_BUFS = STAGE_IN ? (THREE_X ? 2 : 4) : ((FBIO || WGIO) ? 4 : 0);
  // forward: two 4 KB output buffers per epilogue warp; feedback: one 2 KB buffer per warp for the
  // planes (the belief itself is updated in place in its input box)
  static constexpr int OUT_BYTES =
      TSTORE ? EPI_WARPS * 2 * 4096 : ((FBIO || WGIO) ? EPI_WARPS * 2048 : 0);
  static constexpr int SMEM_BYTES =
      RING_BYTES + IN_BUFS * IN_BYTES + OUT_BYTES + RX_BYTES + 1024 /*align*/ + 512 /*barriers*/;
  static_assert(SMEM_BYTES <= 232448, "more than the 227 KB of shared memory a CTA can have");
  static constexpr uint32_t FMT = BF ? 1u : 2u; // operand format: 1 = BF16, 2 = TF32
  static constexpr uint32_t IDESC = (1u << 4) | (FMT << 7) | (FMT << 10) | ((A_MN ? 1u : 0u) << 15) |
                                    ((B_MN ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) |
                                    ((uint32_t)(TILE_M >> 4) << 24);
  static_assert(!PAIR || (BM == 128 && BN % 64 == 0), "pair tiles are 256 x BN");
  static_assert(KS == 1 || (KS == 2 && !PAIR && OP == TC_FWD && BM == 128 && BN == 64),
                "the K-split sweep uses 128 x 64 tiles");
};

template <int OP, int BN, int THREE_X, int BM = 128, bool PAIR = false, int KS = 1>
__global__ void __launch_bounds__(Cfg<OP, BN, THREE_X, BM, PAIR, KS>::THREADS, 1)
    pc_tc_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                 const __grid_constant__ CUtensorMap mapU, const __grid_constant__ CUtensorMap mapSE,
                 const __grid_constant__ CUtensorMap mapSF, const TcParams P)
{
  using C = Cfg<OP, BN, THREE_X, BM, PAIR, KS>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~(uintptr_t)1023);
  uint8_t* stage_base = smem;
  uint8_t* in_base = smem + C::RING_BYTES; // staged operand of the layer above
  uint8_t* out_base = in_base + C::IN_BUFS * C::IN_BYTES; // staged epilogue outputs
  uint8_t* rx_base = out_base + C::OUT_BYTES; // K-split sweep: peer's partial tile
  uint64_t* bars = reinterpret_cast<uint64_t*>(rx_base + C::RX_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + C::STAGES;
  uint64_t* xf = bars + 2 * C::STAGES;
  uint64_t* rempty = bars + 3 * C::STAGES; // B16: raw slot read by the split warps
  uint64_t* tfull = bars + 4 * C::STAGES;
  uint64_t* tempty = tfull + 2;
  uint64_t* in_full = tempty + 2;
  uint64_t* in_empty = in_full + 4;
  uint64_t* rx_full = in_empty + 4;
  uint64_t* pub = rx_full + 1; // sweep: the epilogue warps' stores of a layer are issued
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(pub + 1);
  // 8-byte aligned: [0] the abort flag, [2..3] the wait limit in cycles (see wait_limit())
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_per_layer = P.tiles_m * P.tiles_n;
  const int total_tiles = P.count * tiles_per_layer;
  // Pair mode: the two CTAs of a cluster walk the same work items; rank 0 issues the MMAs.
  const uint32_t rank = PAIR ? cluster_ctarank() : 0;
  const bool leader = rank == 0;
  // K-split sweep: which half of K this CTA multiplies and which 32 columns it finishes.
  const uint32_t krank = KS > 1 ? cluster_ctarank() : 0;
  const int t_begin = P.chain ? 0 : (PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x);
  const int t_end = P.chain ? P.count : total_tiles;
  const int t_step = P.chain ? 1 : (PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x);
  // (a K that is not a multiple of the stage depth: the copies of the last block read zeros
  // beyond the tensor's extent)
  const int kblocks = (P.K + C::KB - 1) / C::KB / KS;

  if (threadIdx.x == 0)
  {
    for (int s = 0; s < C::STAGES; ++s)
    {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
      mbar_init(&xf[s], PAIR ? 8 : 4); // transform warps of both CTAs arrive on the leader's
      mbar_init(&rempty[s], 4);
    }
    for (int a = 0; a < 2; ++a)
    {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], PAIR ? 2 * C::EPI_WARPS : C::EPI_WARPS);
    }
    for (int b = 0; b < C::IN_BUFS; ++b)
    {
      mbar_init(&in_full[b], 1);
      mbar_init(&in_empty[b], (C::FBIO || C::WGIO) ? C::EPI_WARPS / 2 : C::EPI_WARPS);
    }
    mbar_init(rx_full, 1);
    mbar_init(pub, C::EPI_WARPS);
    *abort_flag = 0;
    *reinterpret_cast<volatile long long*>(abort_flag + 2) = P.wait_cycles;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1)
  {
    if (PAIR)
    {
      // one warp of each CTA of the pair takes part in the paired allocation
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                       smem_u32(tmem_holder)),
                   "r"((uint32_t)C::TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    else
    {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                       smem_u32(tmem_holder)),
                   "r"((uint32_t)C::TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  if (PAIR || KS > 1)
    cluster_sync_all(); // the peer's barriers are initialised before anything signals them
  else
    __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t peer_rx = KS > 1 ? mapa_u32(smem_u32(rx_base), krank ^ 1) : 0;
  const uint32_t peer_rx_full = KS > 1 ? mapa_u32(smem_u32(rx_full), krank ^ 1) : 0;
  // Barriers of the leader CTA as seen from either CTA (shared::cluster addresses).
  const uint32_t lead_full = PAIR ? mapa_u32(smem_u32(full), 0) : 0;
  const uint32_t lead_xf = PAIR ? mapa_u32(smem_u32(xf), 0) : 0;
  const uint32_t lead_tempty = PAIR ? mapa_u32(smem_u32(tempty), 0) : 0;
  const uint32_t peer_empty = PAIR ? mapa_u32(smem_u32(empty), rank ^ 1) : 0;
  const uint32_t peer_tfull = PAIR ? mapa_u32(smem_u32(tfull), rank ^ 1) : 0;

  if (warp == 0)
  {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0)
    {
      int s = 0;
      uint32_t phase = 1; // parity to wait for on empty[s]; flips each time the ring wraps
      bool alive = true;
      for (int t = t_begin; t < t_end && alive; t += t_step)
      {
        const int lrel = P.chain ? t : t / tiles_per_layer;
        const int rem = P.chain ? (int)blockIdx.x / KS : t % tiles_per_layer;
        // this CTA's rows of A and rows of B (pair mode: its half of each)
        const int m0 = (rem / P.tiles_n) * C::TILE_M + (int)rank * BM;
        const int n0 = (rem % P.tiles_n) * BN + (int)rank * C::BN_LOCAL;
        const int lcoord = P.first + lrel - P.run_first;
        for (int kb = 0; kb < kblocks; ++kb, s = (s + 1 == C::STAGES ? 0 : s + 1))
        {
          if (s == 0 && !(t == t_begin && kb == 0))
            phase ^= 1;
          if (!(C::B16 ? mbar_wait(&rempty[s], phase, abort_flag)
                       : (PAIR ? mbar_wait_cluster(&empty[s], phase, abort_flag)
                               : mbar_wait(&empty[s], phase, abort_flag))))
          {
            alive = false;
            break;
          }
          if (C::B16) // the split warps' reads of the slot come before the copy that refills it
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          uint8_t* a_dst = stage_base + s * C::STAGE_BYTES;
          uint8_t* b_dst = a_dst + C::A_BYTES;
          const int k0 = ((int)krank * kblocks + kb) * C::KB;
          // One operand of one stage: fp32 tiles are one box (K-major) or slabs of 32 columns
          // (MN-major); pre-split operands are the "hi" and "mid" planes (layer coordinates 2l and
          // 2l+1), each one box of 64 k-columns (K-major) or slabs of 64 columns (MN-major).
          auto load_operand = [&](uint8_t* dst, const CUtensorMap* map, bool mn, int rows, int r0,
                                  int bytes, uint64_t* bar_local, uint32_t bar_pair, bool pair,
                                  int kk) {
            auto one = [&](uint8_t* d, int c0, int c1, int c2) {
              if (pair)
                tma_load_3d_pair(d, map, bar_pair, c0, c1, c2);
              else
                tma_load_3d(d, map, bar_local, c0, c1, c2);
            };
            if (C::PRE)
            {
              for (int pl = 0; pl < 2; ++pl)
              {
                uint8_t* d = dst + pl * (bytes / 2);
                if (!mn)
                  one(d, kk, r0, 2 * lcoord + pl);
                else
                  for (int i = 0; i < rows / 64; ++i)
                    one(d + i * (C::KB * 128), r0 + 64 * i, kk, 2 * lcoord + pl);
              }
            }
            else if (!mn)
              one(dst, kk, r0, lcoord);
            else
              for (int i = 0; i < rows / 32; ++i)
                one(dst + i * (TBK * 128), r0 + 32 * i, kk, lcoord);
          };
          if (PAIR && !C::SPLITW)
          {
            // No in-kernel operand transform: the MMA thread of the leader waits on ITS full[s]
            // for the tiles of both CTAs, so both CTAs' copies count their bytes there.
            if (leader)
              mbar_expect_tx(&full[s], 2 * (C::A_BYTES + C::B_BYTES));
            const uint32_t bar = lead_full + (uint32_t)(s * 8);
            load_operand(b_dst, &mapB, C::B_MN, C::BN_LOCAL, n0, C::B_BYTES, nullptr, bar, true, k0);
            load_operand(a_dst, &mapA, C::A_MN, BM, m0, C::A_BYTES, nullptr, bar, true, k0);
            continue;
          }
          mbar_expect_tx(&full[s], C::A_BYTES + C::B_BYTES);
          load_operand(b_dst, &mapB, C::B_MN, C::BN_LOCAL, n0, C::B_BYTES, &full[s], 0, false, k0);
          if (P.chain && kb == 0 && t > 0)
          {
            // The rows of this layer's input are the previous layer's output: wait until every
            // tile of that row block has been published (the weights above are already on
            // their way).
            // K-split: this CTA's half of K is the output of half of the previous layer's column
            // tiles, which count themselves in on a counter of their own (fewer CTAs to wait for)
            const int dep = KS == 2 ? ((t - 1) * P.tiles_m + m0 / C::TILE_M) * 2 + (int)krank
                                    : (t - 1) * P.tiles_m + m0 / C::TILE_M;
            if (!chain_wait(&P.chain_counters[dep], P.chain_target,
                            abort_flag))
              alive = false; // the A copy below still runs so the stage's byte count completes
            trace_stamp(P, t, 0);
          }
          load_operand(a_dst, &mapA, C::A_MN, BM, m0, C::A_BYTES, &full[s], 0, false, k0);
          if (!alive)
            break;
        }
      }
      if (!alive)
      {
        // Let copies already in flight land before the CTA's shared memory goes away.
        for (int s = 0; s < C::STAGES; ++s)
        {
          const long long t0 = clock64();
          while (clock64() - t0 < 2000000LL)
          {
          }
        }
      }
    }
  }
  else if (warp == 1)
  {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0 && leader)
    {
      int s = 0, tile_iter = 0;
      uint32_t phase = 0; // parity to wait for on full[s] / xf[s]
      bool alive = true;
      // 32-bit tiles, MN-major: 4 k-rows of 128 bytes per swizzle atom (512 B between k-groups),
      // slabs of 32 columns TBK*128 bytes apart; K-major: 8 rows per atom (1024 B between groups).
      // BF16 tiles split in the kernel (32 k per stage): MN-major blocks of 64 columns TBK*128
      // bytes apart, 8 k-rows of 128 bytes per atom, 16 k-rows per instruction; K-major 64-byte
      // rows, 8 per atom (512 B between groups).  Pre-split BF16 tiles (64 k per stage) are what
      // TMA's 128-byte swizzle writes: K-major 128-byte rows, 8 per atom (1024 B between groups);
      // MN-major blocks of 64 columns KB*128 bytes apart.
      const uint32_t a_lbo = C::A_MN ? C::KB * 128 : 16, b_lbo = C::B_MN ? C::KB * 128 : 16;
      const uint32_t a_adv = C::BF ? (C::A_MN ? 2048 : 32) : (C::A_MN ? 1024 : UMMA_K * 4);
      const uint32_t b_adv = C::BF ? (C::B_MN ? 2048 : 32) : (C::B_MN ? 1024 : UMMA_K * 4);
      const uint32_t a_sbo = C::PRE ? 1024 : C::B16 ? (C::A_MN ? 1024 : 512) : (C::A_MN ? 512 : 1024);
      const uint32_t b_sbo = C::PRE ? 1024 : C::B16 ? (C::B_MN ? 1024 : 512) : (C::B_MN ? 512 : 1024);
      const uint32_t a_lay = C::PRE ? 2 : C::B16 ? (C::A_MN ? 2 : 4) : (C::A_MN ? 1 : 2);
      const uint32_t b_lay = C::PRE ? 2 : C::B16 ? (C::B_MN ? 2 : 4) : (C::B_MN ? 1 : 2);
      // BF16 split: the slots of [A hi][A mid][B hi][B mid] follow the NR raw slots
      constexpr uint32_t OPB = C::B16 ? C::NR * C::RAWB : 0;
      constexpr int MS = C::B16 ? C::NB : C::STAGES; // slots the tensor core cycles through
      const uint64_t da0 = make_desc(smem_u32(stage_base) + OPB, a_lbo, a_sbo, a_lay);
      const uint64_t db0 = make_desc(smem_u32(stage_base) + OPB + C::A_BYTES, b_lbo, b_sbo, b_lay);
      constexpr int KSTEPS = C::BF ? C::KB / 16 : TBK / UMMA_K;
      for (int t = t_begin; t < t_end && alive; t += t_step, ++tile_iter)
      {
        const int acc = tile_iter & 1;
        if (!(PAIR ? mbar_wait_cluster(&tempty[acc], ((tile_iter >> 1) & 1) ^ 1, abort_flag)
                   : mbar_wait(&tempty[acc], ((tile_iter >> 1) & 1) ^ 1, abort_flag)))
          break;
        tc_fence_after();
        const uint32_t d_tmem0 = tmem_base + acc * (BN * C::NACC);
        for (int kb = 0; kb < kblocks; ++kb)
        {
          uint64_t* ready = C::SPLITW ? &xf[s] : &full[s];
          if (!(PAIR ? mbar_wait_cluster(ready, phase, abort_flag)
                     : mbar_wait(ready, phase, abort_flag)))
          {
            alive = false;
            break;
          }
          tc_fence_after();
          if (P.chain && kb == 0)
            trace_stamp(P, t, 1);
          // Descriptors differ between stages and k-steps only in the 14-bit start-address
          // field (units of 16 bytes): one add per operand per instruction.
          const uint64_t sa = da0 + (uint64_t)(s * (C::STAGE_BYTES >> 4));
          const uint64_t sb = db0 + (uint64_t)(s * (C::STAGE_BYTES >> 4));
#pragma unroll
          for (int ks = 0; ks < KSTEPS; ++ks)
          {
            const uint64_t da = sa + (uint64_t)(ks * (a_adv >> 4));
            const uint64_t db = sb + (uint64_t)(ks * (b_adv >> 4));
            const uint32_t d_tmem = d_tmem0;
            const uint32_t first = (kb | ks) != 0;
            if (C::BF)
            {
              const uint64_t dam = da + (uint64_t)((C::A_BYTES / 2) >> 4);
              const uint64_t dbm = db + (uint64_t)((C::B_BYTES / 2) >> 4);
              if (PAIR)
              {
                tc_mma_bf16_pair(d_tmem, da, dbm, C::IDESC, first);
                tc_mma_bf16_pair(d_tmem, dam, db, C::IDESC, 1);
                tc_mma_bf16_pair(d_tmem, da, db, C::IDESC, 1);
              }
              else if (C::NACC == 2)
              {
                tc_mma_bf16(d_tmem, da, db, C::IDESC_WIDE, first); // A_hi x [B_hi ; B_mid]
                tc_mma_bf16(d_tmem, dam, db, C::IDESC, 1);         // + A_mid x B_hi
              }
              else
              {
                tc_mma_bf16(d_tmem, da, dbm, C::IDESC, first);
                tc_mma_bf16(d_tmem, dam, db, C::IDESC, 1);
                tc_mma_bf16(d_tmem, da, db, C::IDESC, 1);
              }
            }
            else if (THREE_X == 1)
            {
              const uint64_t dal = da + (uint64_t)((C::A_BYTES + C::B_BYTES) >> 4);
              const uint64_t dbl = db + (uint64_t)((C::A_BYTES + C::B_BYTES) >> 4);
              if (PAIR)
              {
                tc_mma_tf32_pair(d_tmem, da, dbl, C::IDESC, first);
                tc_mma_tf32_pair(d_tmem, dal, db, C::IDESC, 1);
                tc_mma_tf32_pair(d_tmem, da, db, C::IDESC, 1);
              }
              else
              {
                tc_mma_tf32(d_tmem, da, dbl, C::IDESC, first);
                tc_mma_tf32(d_tmem, dal, db, C::IDESC, 1);
                tc_mma_tf32(d_tmem, da, db, C::IDESC, 1);
              }
            }
            else if (PAIR)
              tc_mma_tf32_pair(d_tmem, da, db, C::IDESC, first);
            else
              tc_mma_tf32(d_tmem, da, db, C::IDESC, first);
          }
          if (PAIR)
          {
            // release the stage in both CTAs (two plain commits, one per CTA)
            tc_commit_pair(smem_u32(&empty[s]));
            tc_commit_pair(peer_empty + (uint32_t)(s * 8));
          }
          else
            tc_commit(&empty[s]);
          if (++s == MS)
            s = 0, phase ^= 1;
        }
        if (alive)
        {
          if (PAIR)
          {
            tc_commit_pair(smem_u32(&tfull[acc]));
            tc_commit_pair(peer_tfull + (uint32_t)(acc * 8));
          }
          else
            tc_commit(&tfull[acc]);
        }
      }
    }
  }
  else if (warp < 2 + C::EPI_WARPS)
  {
    // ---------------------------------------------------------------- epilogue
    // Two (or more) warps share each 32-lane quarter of tensor memory and take alternate
    // 32-column chunks.  Per chunk: issue every global load first (256-bit vectors, one
    // full 32-byte sector per lane), then read the accumulators, compute, store.
    const int quarter = warp & 3; // tensor-memory lanes this warp may read
    const int grp = (warp - 2) >> 2;
    constexpr int GROUPS = C::EPI_WARPS / 4;
    float esum = 0.0f;
    int tile_iter = 0;
    uint32_t out_seq = 0; // chunks this warp has staged for bulk stores
    for (int t = t_begin; t < t_end; t += t_step, ++tile_iter)
    {
      const int lrel = P.chain ? t : t / tiles_per_layer;
      const int rem = P.chain ? (int)blockIdx.x / KS : t % tiles_per_layer;
      // M=128: lane i of quarter q holds row 32q+i.  M=64: rows 16q..16q+15 sit in lanes 0..15 of
      // quarter q and the upper 16 lanes hold nothing.
      const bool active = BM == 128 || lane < 16;
      const int m = (rem / P.tiles_n) * C::TILE_M + (int)rank * BM +
                    (BM == 128 ? quarter * 32 + lane : quarter * 16 + (lane & 15));
      // K-split sweep: this CTA finishes columns [32*krank, 32*krank+32) of the 64-wide tile
      constexpr int BNE = KS == 2 ? 32 : BN;
      const int n0 = (rem % P.tiles_n) * BN + (KS == 2 ? 32 * (int)krank : 0);
      const int li = P.first + lrel;
      const dpc_layer* Lup = (li + 1 < P.n_layers) ? &P.layers[li + 1] : nullptr;
      const int acc = tile_iter & 1;
      FwdMeta meta;
      float bias_pre[32];
      float defer_z[16];
      size_t defer_o = 0;
      bool deferred = false;
      if (OP == TC_FWD)
      {
        load_fwd_meta(P, li, meta);
        if (BNE / GROUPS <= 32)
        {
          // Narrow tiles (the sequential sweep): this warp's bias values are fetched now too.
#pragma unroll
          for (int i = 0; i < (BNE / GROUPS) / 16; ++i)
#pragma unroll
            for (int k = 0; k < 16; k += 8)
              ld8(meta.b + n0 + (grp + GROUPS * i) * 16 + k, &bias_pre[i * 16 + k]);
        }
      }
      if (!(PAIR ? mbar_wait_cluster(&tfull[acc], (tile_iter >> 1) & 1, abort_flag)
                 : mbar_wait(&tfull[acc], (tile_iter >> 1) & 1, abort_flag)))
        break;
      tc_fence_after();
      if (P.chain && warp == 2 && lane == 0)
        trace_stamp(P, t, 2);
      uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * (BN * C::NACC);

      if (OP == TC_FWD)
      {
        constexpr bool PF = THREE_X == 0;
        constexpr bool SI = C::STAGE_IN;
        constexpr bool KSUM = KS == 2;
        constexpr int AS = C::NACC == 2 ? BN : 0;
        InStage in;
        in.buf = in_base, in.full = in_full, in.empty = in_empty;
        in.seq = (uint32_t)tile_iter * (uint32_t)(BN / 32);
        in.row = quarter * 32 + lane, in.nbufs = C::IN_BUFS > 0 ? C::IN_BUFS : 1;
        in.abort_flag = abort_flag;
        in.rx = rx_base;
        in.out = (C::TSTORE && P.tstore) ? out_base + (warp - 2) * 8192 : nullptr;
        in.out_seq = &out_seq;
        in.map_e = &mapSE, in.map_fe = &mapSF;
        in.out_row0 = m - lane; // the row of this warp's lane 0
        in.layer_e = li + 1 - P.run_first, in.layer_fe = li - P.run_first;
        // (one 16-column chunk per warp: the narrow tiles of the sweep; only where the next
        // layer's tensor cores read the operand planes -- in the other schemes the fp32 belief
        // IS the operand and must be stored before the publication)
        deferred = C::PRE && P.chain && (BNE / GROUPS == 16) && (P.flags & DPC_FWD_COPY_NEXT) &&
                   active && meta.up_z != nullptr && meta.upz_hi != nullptr;
        in.defer = deferred ? defer_z : nullptr, in.defer_o = &defer_o;
        if (KS == 2)
        {
          // Hand the peer this CTA's partial sums of the 32 columns the peer finishes (16 per
          // warp), then wait for the peer's partial sums of this CTA's own 32 columns.
          const uint32_t peer = krank ^ 1u;
          float pv[16];
          tc_ld16(taddr + 32 * peer + 16 * grp, pv);
          if (C::NACC == 2)
          {
            float p1[16];
            tc_ld16(taddr + BN + 32 * peer + 16 * grp, p1);
#pragma unroll
            for (int i = 0; i < 16; ++i)
              pv[i] += p1[i];
          }
          const int row = quarter * 32 + lane;
          const uint32_t dst = peer_rx + (uint32_t)row * 128u;
          // asynchronous remote stores that count their bytes on the peer's barrier: no separate
          // release + arrive round trip
#pragma unroll
          for (int i = 0; i < 4; ++i)
          {
            const uint32_t a = dst + (uint32_t)((((grp << 2) + i) ^ (row & 7)) << 4);
            asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 "
                         "[%0], {%1, %2, %3, %4}, [%5];" ::"r"(a),
                         "f"(pv[4 * i]), "f"(pv[4 * i + 1]), "f"(pv[4 * i + 2]), "f"(pv[4 * i + 3]),
                         "r"(peer_rx_full)
                         : "memory");
          }
          // this CTA expects the peer's 128 rows x 128 bytes once per layer
          if (warp == 2 && lane == 0)
            mbar_expect_tx(rx_full, 128 * 128);
          if (!mbar_wait_cluster(rx_full, (uint32_t)(tile_iter & 1), abort_flag))
            break;
          taddr += 32 * krank; // this CTA's own columns of the accumulator
        }
        switch (meta.act)
        {
        case DPC_ACT_TANH:
          fwd_epilogue_tile<DPC_ACT_TANH, BNE, GROUPS, PF, SI, KSUM, AS>(P, meta, bias_pre, taddr, m, n0, grp, esum, P.chain ? t : -1, active, &in);
          break;
        case DPC_ACT_GELU:
          fwd_epilogue_tile<DPC_ACT_GELU, BNE, GROUPS, PF, SI, KSUM, AS>(P, meta, bias_pre, taddr, m, n0, grp, esum, P.chain ? t : -1, active, &in);
          break;
        default:
          fwd_epilogue_tile<-1, BNE, GROUPS, false, SI, KSUM, AS>(P, meta, bias_pre, taddr, m, n0, grp, esum, P.chain ? t : -1, active, &in);
        }
      }
      else if (OP == TC_FB)
      {
        const dpc_layer L = P.layers[li];
        const bool residual = (L.flags & DPC_LAYER_RESIDUAL) != 0;
        __nv_bfloat16* z_hi = P.zp ? P.zp + 2 * (long long)(li - P.run_first) * P.act_elems : nullptr;
        if (C::FBIO && P.tstore)
        {
          // 16-column chunks; the two warp groups take alternate chunks, so every box is read
          // by the four warps of one group (one 32-row quarter each).
          const int row = quarter * 32 + lane;
          const int lz = li - P.run_first;
          uint8_t* obuf = out_base + (warp - 2) * 2048;
          bool ok = true;
          for (int c = grp; c < BN / 16 && ok; c += GROUPS)
          {
            const uint32_t q = (uint32_t)tile_iter * (uint32_t)(BN / 16) + (uint32_t)c;
            constexpr uint32_t NBUF = C::IN_BUFS > 0 ? C::IN_BUFS : 1;
            const uint32_t b = q & (NBUF - 1);
            if (!mbar_wait(&in_full[b], (q / NBUF) & 1u, abort_flag))
            {
              ok = false;
              break;
            }
            uint8_t* ebuf = in_base + b * C::IN_BYTES;
            uint8_t* zbuf = ebuf + BM * 64;
            float ee[16], zz[16], v[16];
            const int sw = (row >> 1) & 3;
#pragma unroll
            for (int i = 0; i < 4; ++i)
            {
              const float4 x = *reinterpret_cast<const float4*>(ebuf + row * 64 + ((i ^ sw) << 4));
              const float4 y = *reinterpret_cast<const float4*>(zbuf + row * 64 + ((i ^ sw) << 4));
              ee[4 * i] = x.x, ee[4 * i + 1] = x.y, ee[4 * i + 2] = x.z, ee[4 * i + 3] = x.w;
              zz[4 * i] = y.x, zz[4 * i + 1] = y.y, zz[4 * i + 2] = y.z, zz[4 * i + 3] = y.w;
            }
            tc_ld16(taddr + c * 16, v);
#pragma unroll
            for (int k = 0; k < 16; ++k)
              zz[k] += L.ir * (L.a * v[k] - ee[k]);
#pragma unroll
            for (int i = 0; i < 4; ++i)
              *reinterpret_cast<float4*>(zbuf + row * 64 + ((i ^ sw) << 4)) =
                  make_float4(zz[4 * i], zz[4 * i + 1], zz[4 * i + 2], zz[4 * i + 3]);
#pragma unroll
            for (int k = 0; k < 16; k += 8)
            {
              // 32-byte rows, 16-byte chunks xor-ed with (row >> 2) & 1: the 32-byte swizzle
              uint4 h, mm;
              split8(make_float4(zz[k], zz[k + 1], zz[k + 2], zz[k + 3]),
                     make_float4(zz[k + 4], zz[k + 5], zz[k + 6], zz[k + 7]), h, mm);
              const int off = lane * 32 + ((((k >> 3) & 1) ^ ((lane >> 2) & 1)) << 4);
              *reinterpret_cast<uint4*>(obuf + off) = h;
              *reinterpret_cast<uint4*>(obuf + 1024 + off) = mm;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0)
            {
              const int col = n0 + c * 16, row0 = m - lane;
              tma_store_3d(&mapSE, zbuf + quarter * 2048, col, row0, lz);
              tma_store_3d(&mapSF, obuf, col, row0, 2 * lz); // hi + mid
              bulk_commit();
              // the stores have read their shared memory: the box may be refilled, the plane
              // buffer rewritten
              bulk_wait_read<0>();
              mbar_arrive(&in_empty[b]);
            }
            __syncwarp();
          }
          if (!ok)
            break;
        }
        else
        for (int c = grp; c < BN / 32; c += GROUPS)
        {
          // columns of this chunk inside the tensor (a multiple of 8; the same for every lane)
          const int nv = P.N - (n0 + c * 32);
          if (nv <= 0)
            break;
          const size_t o = (size_t)m * P.N + n0 + c * 32;
          float ee[32], zz[32], v[32];
#pragma unroll
          for (int k = 0; k < 32; k += 8)
          {
            if (k >= nv)
              continue;
            ld8(L.e + o + k, &ee[k]);
            ld8(L.z + o + k, &zz[k]);
          }
          tc_ld32(taddr + c * 32, v);
#pragma unroll
          for (int k = 0; k < 32; k += 8)
          {
            if (k >= nv)
              continue;
            float fb[8];
#pragma unroll
            for (int q = 0; q < 8; ++q)
              fb[q] = L.a * v[k + q] - ee[k + q];
            if (L.flags & DPC_LAYER_INPUT_ACT)
            {
              // SimplePC (src/layers/SimplePCLayer.cpp:205-257): z += ir (f'(z) (e_above W) - e)
#pragma unroll
              for (int q = 0; q < 8; ++q)
                zz[k + q] += L.ir * (v[k + q] * act_deriv(L.act, zz[k + q]) - ee[k + q]);
            }
            else if (L.v)
            {
              float vv[8];
              ld8(L.v + o + k, vv);
#pragma unroll
              for (int q = 0; q < 8; ++q)
              {
                vv[q] = L.momentum_beta * vv[q] + (1.0f - L.momentum_beta) * fb[q];
                zz[k + q] += L.ir * vv[q];
              }
              st8(L.v + o + k, vv);
            }
            else
            {
#pragma unroll
              for (int q = 0; q < 8; ++q)
                zz[k + q] += L.ir * fb[q];
            }
            if (residual)
            {
              float uu[8];
              ld8(Lup->e + o + k, uu);
#pragma unroll
              for (int q = 0; q < 8; ++q)
                zz[k + q] += L.ir * uu[q];
            }
            st8(L.z + o + k, &zz[k]);
            if (z_hi)
              st_planes8(z_hi, P.act_elems, o + k, &zz[k]);
          }
        }
      }
      else
      {
        const dpc_layer L = P.layers[li];
        const float Bf = (float)P.batch;
        float alpha, decay = 1.0f;
        if ((P.mode & 1) == WG_DFA_MODE)
        {
          alpha = L.fl * L.a / Bf;
          // the FullPC pre-scale of the direct-feedback update (FullPCLayer.cpp:514-572)
          if ((P.flags & 1) && L.lmbda > 0.0f && L.fl != 0.0f)
            decay = 1.0f - L.lmbda;
        }
        else
        {
          alpha = (L.flags & DPC_LAYER_INPUT_ACT) ? L.lr / Bf : L.a * L.lr / Bf;
          if (L.lmbda > 0.0f)
            decay = 1.0f - L.lmbda;
        }
        if (P.mode & WG_GRAD_MODE)
        {
          // raw sums into the gradient staging buffer: an optimizer kernel (Adam-type updates,
          // or a sum over batch shards first) applies them
          for (int c = grp; c < BN / 32; c += GROUPS)
          {
            const int nv = P.N - (n0 + c * 32);
            if (nv <= 0)
              break;
            const size_t o = (size_t)m * P.N + n0 + c * 32;
            float v[32];
            tc_ld32(taddr + c * 32, v);
#pragma unroll
            for (int k = 0; k < 32; k += 8)
              if (k < nv)
                st8(L.g_W + o + k, &v[k]);
          }
        }
        else if (C::WGIO && P.tstore)
        {
          const int row = quarter * 32 + lane;
          const int lw = li - P.run_first;
          uint8_t* obuf = out_base + (warp - 2) * 2048;
          bool ok = true;
          for (int c = grp; c < BN / 16 && ok; c += GROUPS)
          {
            constexpr uint32_t NBUF = C::IN_BUFS > 0 ? C::IN_BUFS : 1;
            const uint32_t q = (uint32_t)tile_iter * (uint32_t)(BN / 16) + (uint32_t)c;
            const uint32_t b = q & (NBUF - 1);
            if (!mbar_wait(&in_full[b], (q / NBUF) & 1u, abort_flag))
            {
              ok = false;
              break;
            }
            uint8_t* wbuf = in_base + b * C::IN_BYTES;
            float w[16], v[16];
            const int sw = (row >> 1) & 3;
#pragma unroll
            for (int i = 0; i < 4; ++i)
            {
              const float4 x = *reinterpret_cast<const float4*>(wbuf + row * 64 + ((i ^ sw) << 4));
              w[4 * i] = x.x, w[4 * i + 1] = x.y, w[4 * i + 2] = x.z, w[4 * i + 3] = x.w;
            }
            tc_ld16(taddr + c * 16, v);
#pragma unroll
            for (int k = 0; k < 16; ++k)
            {
              if (decay != 1.0f)
                w[k] *= decay;
              w[k] = fmaf(alpha, v[k], w[k]);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
              *reinterpret_cast<float4*>(wbuf + row * 64 + ((i ^ sw) << 4)) =
                  make_float4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
#pragma unroll
            for (int k = 0; k < 16; k += 8)
            {
              uint4 h, mm;
              split8(make_float4(w[k], w[k + 1], w[k + 2], w[k + 3]),
                     make_float4(w[k + 4], w[k + 5], w[k + 6], w[k + 7]), h, mm);
              const int off = lane * 32 + ((((k >> 3) & 1) ^ ((lane >> 2) & 1)) << 4);
              *reinterpret_cast<uint4*>(obuf + off) = h;
              *reinterpret_cast<uint4*>(obuf + 1024 + off) = mm;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0)
            {
              const int col = n0 + c * 16, row0 = m - lane;
              tma_store_3d(&mapSE, wbuf + quarter * 2048, col, row0, lw);
              tma_store_3d(&mapSF, obuf, col, row0, 2 * lw); // hi + mid
              bulk_commit();
              bulk_wait_read<0>();
              mbar_arrive(&in_empty[b]);
            }
            __syncwarp();
          }
          if (!ok)
            break;
        }
        else
        {
        __nv_bfloat16* w_hi = P.wp ? P.wp + 2 * (long long)(li - P.run_first) * P.w_elems : nullptr;
        for (int c = grp; c < BN / 32; c += GROUPS)
        {
          const int nv = P.N - (n0 + c * 32);
          if (nv <= 0)
            break;
          const size_t o = (size_t)m * P.N + n0 + c * 32;
          float w[32], v[32];
#pragma unroll
          for (int k = 0; k < 32; k += 8)
            if (k < nv)
              ld8(L.W + o + k, &w[k]);
          tc_ld32(taddr + c * 32, v);
#pragma unroll
          for (int k = 0; k < 32; k += 8)
          {
            if (k >= nv)
              continue;
#pragma unroll
            for (int q = 0; q < 8; ++q)
            {
              if (decay != 1.0f)
                w[k + q] *= decay;
              w[k + q] = fmaf(alpha, v[k + q], w[k + q]);
            }
            st8(L.W + o + k, &w[k]);
            if (w_hi)
              st_planes8(w_hi, P.w_elems, o + k, &w[k]);
          }
        }
        }
      }
      if (P.chain && warp == 2 && lane == 0)
        trace_stamp(P, t, 3);
      if (P.chain)
      {
        // Publish this CTA's part of the next layer's input rows.
        // Every lane orders its stores before later reads by the TMA engine (async proxy), the
        // warps meet on a shared-memory barrier, and ONE thread makes the CTA's stores visible
        // device wide and counts the CTA in: one fence and one atomic per CTA and layer instead of
        // eight, 0.8 us less per layer.  The other warps do not wait for it.
        asm volatile("fence.proxy.async.global;" ::: "memory");
        __syncwarp();
        if (lane == 0)
          mbar_arrive(pub);
        if (warp == 2 && lane == 0)
        {
          if (mbar_wait(pub, (uint32_t)(tile_iter & 1), abort_flag))
          {
            asm volatile("fence.acq_rel.gpu;" ::: "memory");
            // (K-split: the counter of the half of K that this tile's columns belong to)
            const int pub_idx =
                KS == 2 ? (lrel * P.tiles_m + rem / P.tiles_n) * 2 + ((rem % P.tiles_n) * 2 >= P.tiles_n ? 1 : 0)
                        : lrel * P.tiles_m + rem / P.tiles_n;
            atomicAdd(&P.chain_counters[pub_idx], 1);
          }
        }
        if (OP == TC_FWD && deferred)
        {
          st8(meta.up_z + defer_o, defer_z);
          st8(meta.up_z + defer_o + 8, defer_z + 8);
        }
        if (warp == 2 && lane == 0)
          trace_stamp(P, t, 4);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0)
      {
        if (PAIR)
          mbar_arrive_cluster(lead_tempty + (uint32_t)(acc * 8));
        else
          mbar_arrive(&tempty[acc]);
      }
    }
    if ((C::TSTORE || C::FBIO || C::WGIO) && lane == 0)
      bulk_wait_all(); // this warp's bulk stores are complete before its shared memory goes away
    if (OP == TC_FWD && (P.flags & DPC_FWD_ENERGY))
    {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
        esum += __shfl_xor_sync(0xffffffffu, esum, o);
      if (lane == 0)
        atomicAdd(P.energy, (double)(0.5f * esum));
    }
  }
  else if (C::STAGE_IN && warp == 2 + C::EPI_WARPS + (C::SPLITW ? 4 : 0))
  {
    // ---------------------------------------------------------------- staged-operand loader
    // Brings this CTA's 128 rows of the layer above (belief or error) into shared memory, one
    // 32-column box at a time, in the order the epilogue warps consume them.
    if (lane == 0 && P.stage_in)
    {
      constexpr uint32_t NBUF = C::IN_BUFS > 0 ? C::IN_BUFS : 1;
      uint32_t q = 0;
      bool alive = true;
      for (int t = t_begin; t < t_end && alive; t += t_step)
      {
        const int lrel = t / tiles_per_layer, rem = t % tiles_per_layer;
        const int m0 = (rem / P.tiles_n) * C::TILE_M + (int)rank * BM;
        const int n0 = (rem % P.tiles_n) * BN;
        const int lcoord = P.first + lrel - P.run_first + 1;
        for (int j = 0; j < BN / 32; ++j, ++q)
        {
          const uint32_t b = q & (NBUF - 1);
          if (!mbar_wait(&in_empty[b], ((q / NBUF) & 1u) ^ 1u, abort_flag))
          {
            alive = false;
            break;
          }
          // order the epilogue warps' (generic-proxy) reads of this buffer before the copy
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          mbar_expect_tx(&in_full[b], C::IN_BYTES);
          tma_load_3d(in_base + b * C::IN_BYTES, &mapU, &in_full[b], n0 + 32 * j, m0, lcoord);
        }
      }
    }
  }
  else if ((C::FBIO || C::WGIO) && warp == 2 + C::EPI_WARPS)
  {
    // ---------------------------------------------------------------- staged error / belief loader
    // This CTA's 128 rows of the layer's error and belief, one 16-column chunk at a time, each as
    // four 32-row slices (the box shape of the store maps, which also serve as load maps).
    if (lane == 0 && P.tstore)
    {
      uint32_t q = 0;
      bool alive = true;
      for (int t = t_begin; t < t_end && alive; t += t_step)
      {
        const int lrel = t / tiles_per_layer, rem = t % tiles_per_layer;
        const int m0 = (rem / P.tiles_n) * C::TILE_M + (int)rank * BM;
        const int n0 = (rem % P.tiles_n) * BN;
        const int lcoord = P.first + lrel - P.run_first;
        for (int c = 0; c < BN / 16; ++c, ++q)
        {
          constexpr uint32_t NBUF = C::IN_BUFS > 0 ? C::IN_BUFS : 1;
          const uint32_t b = q & (NBUF - 1);
          if (!mbar_wait(&in_empty[b], ((q / NBUF) & 1u) ^ 1u, abort_flag))
          {
            alive = false;
            break;
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          mbar_expect_tx(&in_full[b], C::IN_BYTES);
          uint8_t* ebuf = in_base + b * C::IN_BYTES;
          uint8_t* zbuf = ebuf + BM * 64;
          for (int s4 = 0; s4 < BM / 32; ++s4)
          {
            if (C::WGIO) // the weight tile alone
              tma_load_3d(ebuf + s4 * 2048, &mapSE, &in_full[b], n0 + 16 * c, m0 + 32 * s4, lcoord);
            else
            {
              tma_load_3d(ebuf + s4 * 2048, &mapU, &in_full[b], n0 + 16 * c, m0 + 32 * s4, lcoord);
              tma_load_3d(zbuf + s4 * 2048, &mapSE, &in_full[b], n0 + 16 * c, m0 + 32 * s4, lcoord);
            }
          }
        }
      }
    }
  }
  else if (C::SPLITW)
  {
    // ---------------------------------------------------------------- remainder transform
    // lo = x - (x with the low 13 mantissa bits cleared): exactly what the tensor core drops
    // when it reads the raw tile as TF32.  Elementwise on identical offsets, so the swizzled
    // layout of the tile carries over unchanged.
    const int tid = threadIdx.x - (2 + C::EPI_WARPS) * 32;
    int s = 0, sb = 0;
    uint32_t phase = 0, phase_b = 1; // phase_b: parity to wait for on empty[sb] (B16)
    bool alive = true;
    for (int t = t_begin; t < t_end && alive; t += t_step)
    {
      for (int kb = 0; kb < kblocks; ++kb, s = (s + 1 == C::STAGES ? 0 : s + 1), phase ^= (s == 0))
      {
        if (!mbar_wait(&full[s], phase, abort_flag))
        {
          alive = false;
          break;
        }
        if (C::B16)
        {
          // the slot the tensor core reads must have been released by its last MMAs
          if (!(PAIR ? mbar_wait_cluster(&empty[sb], phase_b, abort_flag)
                     : mbar_wait(&empty[sb], phase_b, abort_flag)))
          {
            alive = false;
            break;
          }
          uint8_t* raw = stage_base + s * C::RAWB;
          uint8_t* out = stage_base + (C::NR + sb) * C::RAWB;
          if (C::A_MN)
            split_mnmajor<BM>(raw, out, out + C::A_BYTES / 2, tid);
          else
            split_kmajor<BM>(raw, out, out + C::A_BYTES / 2, tid);
          if (C::B_MN)
            split_mnmajor<C::BN_LOCAL>(raw + C::A_BYTES, out + C::A_BYTES,
                                       out + C::A_BYTES + C::B_BYTES / 2, tid);
          else
            split_kmajor<C::BN_LOCAL>(raw + C::A_BYTES, out + C::A_BYTES,
                                      out + C::A_BYTES + C::B_BYTES / 2, tid);
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0)
          {
            mbar_arrive(&rempty[s]); // the raw slot may be refilled
            if (PAIR)
              mbar_arrive_cluster(lead_xf + (uint32_t)(sb * 8));
            else
              mbar_arrive(&xf[sb]);
          }
          if (++sb == C::NB)
            sb = 0, phase_b ^= 1;
          continue;
        }
        const float4* src = reinterpret_cast<const float4*>(stage_base + s * C::STAGE_BYTES);
        float4* dst = reinterpret_cast<float4*>(stage_base + s * C::STAGE_BYTES + C::A_BYTES +
                                                C::B_BYTES);
        constexpr int N4 = (C::A_BYTES + C::B_BYTES) / 16;
#pragma unroll 4
        for (int i = tid; i < N4; i += 128)
        {
          const float4 x = src[i];
          float4 r;
          r.x = x.x - __uint_as_float(__float_as_uint(x.x) & 0xffffe000u);
          r.y = x.y - __uint_as_float(__float_as_uint(x.y) & 0xffffe000u);
          r.z = x.z - __uint_as_float(__float_as_uint(x.z) & 0xffffe000u);
          r.w = x.w - __uint_as_float(__float_as_uint(x.w) & 0xffffe000u);
          dst[i] = r;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0)
        {
          if (PAIR)
            mbar_arrive_cluster(lead_xf + (uint32_t)(s * 8));
          else
            mbar_arrive(&xf[s]);
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  if (PAIR || KS > 1)
    cluster_sync_all(); // neither CTA leaves while the other may still touch its memory
  else
    __syncthreads();
  if (threadIdx.x == 0 && *abort_flag)
    atomicExch(P.error_flag, 1);
  if (warp == 1)
  {
    tc_fence_after();
    if (PAIR)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                   "r"((uint32_t)C::TMEM_COLS)
                   : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                   "r"((uint32_t)C::TMEM_COLS)
                   : "memory");
  }
}


// ------------------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn()
{
  static EncodeTiledFn fn = nullptr;
  if (!fn)
  {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// fp32 tensor [layers][rows][cols] (cols contiguous) with a (32 x box_rows x 1) box.
bool make_map(CUtensorMap* map, const float* base, int cols, int rows, int layers,
              int64_t layer_stride_elems, int box_rows, bool mn_major)
{
  EncodeTiledFn fn = encode_fn();
  if (!fn)
    return false;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)layers};
  cuuint64_t strides[2] = {(cuuint64_t)cols * 4, (cuuint64_t)layer_stride_elems * 4};
  cuuint32_t box[3] = {32, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// bf16 operand planes [planes][rows][cols] (cols contiguous) with a (64 x box_rows x 1) box:
// 128-byte rows under the 128-byte swizzle, for K-major and MN-major operands alike.
bool make_map_bf16(CUtensorMap* map, const __nv_bfloat16* base, int cols, int rows, int planes,
                   int64_t plane_elems, int box_rows)
{
  EncodeTiledFn fn = encode_fn();
  if (!fn)
    return false;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)planes};
  cuuint64_t strides[2] = {(cuuint64_t)cols * 2, (cuuint64_t)plane_elems * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<__nv_bfloat16*>(base), dims,
                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Store maps of the staged epilogue: [planes][rows][cols] with a (16 x 32 x 1) box, i.e. one warp's
// 32 rows of a 16-column chunk; rows of 64 bytes (fp32, 64-byte swizzle) or 32 bytes (bf16,
// 32-byte swizzle) in shared memory.
bool make_store_map(CUtensorMap* map, const void* base, bool bf16, int cols, int rows, int planes,
                    int64_t plane_elems)
{
  EncodeTiledFn fn = encode_fn();
  if (!fn)
    return false;
  const cuuint64_t eb = bf16 ? 2 : 4;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)planes};
  cuuint64_t strides[2] = {(cuuint64_t)cols * eb, (cuuint64_t)plane_elems * eb};
  // bf16 planes: the hi and the mid plane of a layer (neighbours in the outer dimension) go out
  // in ONE store from two adjacent 1 KB tiles
  cuuint32_t box[3] = {16, 32, bf16 ? 2u : 1u};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  bf16 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_64B,
                  CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Re-splits the operand planes of `kind` for layers [first, first + gridDim.y) from the fp32
// tensors (after something other than a kernel of this file wrote them).
__global__ void split_planes_kernel(const dpc_layer* __restrict__ layers, int first, int run_first,
                                    int kind, __nv_bfloat16* base, long long elems)
{
  const dpc_layer& L = layers[first + blockIdx.y];
  const float* src = kind == PL_Z ? L.z : (kind == PL_FE ? L.fe : L.W);
  __nv_bfloat16* hi = base + 2 * (long long)(first + (int)blockIdx.y - run_first) * elems;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < elems;
       i += (long long)gridDim.x * blockDim.x * 8)
  {
    const float4 a = *reinterpret_cast<const float4*>(src + i);
    const float4 b = *reinterpret_cast<const float4*>(src + i + 4);
    uint4 h, m;
    split8(a, b, h, m);
    *reinterpret_cast<uint4*>(hi + i) = h;
    *reinterpret_cast<uint4*>(hi + elems + i) = m;
  }
}

template <int OP, int BN, int THREE_X, int BM = 128, bool PAIR = false, int KS = 1>
int launch(dpc_plan* p, TcState* st, const CUtensorMap& a, const CUtensorMap& b, TcParams P,
           const CUtensorMap* up = nullptr)
{
  // forward: up = staged operand of the layer above, stores of errors and fe planes; feedback:
  // loads of the layer's error, loads and stores of its belief, stores of the belief's planes
  const CUtensorMap& u = (OP == TC_FB && P.tstore) ? st->e_st : (up ? *up : a);
  const CUtensorMap& se = P.tstore ? (OP == TC_FB ? st->z_st : OP == TC_WG ? st->w_st : st->e_st) : a;
  const CUtensorMap& sf =
      P.tstore ? (OP == TC_FB ? st->zp_st : OP == TC_WG ? st->wp_st : st->fep_st) : a;
  using C = Cfg<OP, BN, THREE_X, BM, PAIR, KS>;
  static bool configured = false;
  auto kern = pc_tc_kernel<OP, BN, THREE_X, BM, PAIR, KS>;
  if (!configured)
  {
    if (C::SMEM_BYTES > st->max_smem)
      return 1;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::SMEM_BYTES);
    if (e != cudaSuccess)
      return cuda_fail(e, "cudaFuncSetAttribute(tensor-core kernel)");
    configured = true;
  }
  const int total = P.count * P.tiles_m * P.tiles_n;
  if (PAIR || KS > 1)
  {
    // one cluster of two CTAs per work item, as many clusters as SM pairs (the sweep: one
    // cluster per tile, all of them resident at once)
    const int pairs = P.chain ? P.tiles_m * P.tiles_n : std::min(total, p->ctx->sm_count / 2);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(C::THREADS);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = p->ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, a, b, u, se, sf, P);
    p->ctx->launches += 1;
    if (e != cudaSuccess)
      return cuda_fail(e, "tensor-core pair kernel launch");
    return DPC_OK;
  }
  const int grid = P.chain ? P.tiles_m * P.tiles_n : std::min(total, p->ctx->sm_count);
  kern<<<grid, C::THREADS, C::SMEM_BYTES, p->ctx->stream>>>(a, b, u, se, sf, P);
  p->ctx->launches += 1;
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess)
    return cuda_fail(cudaGetLastError(), "tensor-core kernel launch");
  return DPC_OK;
}

bool range_in_run(const dpc_plan* p, int first, int count)
{
  return p->run.count > 0 && count > 0 && first >= p->run.first &&
         first + count <= p->run.first + p->run.count;
}
} // namespace

static bool pair_ok(int rows, int cols);
static int split_scheme(const dpc_plan* p);

// Operand planes for the run (see TcState): allocated when the plan will use the 3xBF16 scheme on
// CTA-pair tiles.  DPC_DISABLE_PLANES keeps the in-kernel split (used to compare the two).
static bool planes_init(dpc_plan* plan, TcState* st, int first, int count, int H)
{
  const int B = plan->batch;
  if (getenv("DPC_DISABLE_PLANES") || split_scheme(plan) != 2 || !pair_ok(B, H))
    return true;
  const size_t act = (size_t)B * H, w = (size_t)H * H;
  if (cudaMalloc(&st->zp, 2 * (size_t)(count + 1) * act * sizeof(__nv_bfloat16)) != cudaSuccess ||
      cudaMalloc(&st->fep, 2 * (size_t)count * act * sizeof(__nv_bfloat16)) != cudaSuccess ||
      cudaMalloc(&st->wp, 2 * (size_t)count * w * sizeof(__nv_bfloat16)) != cudaSuccess)
  {
    cudaGetLastError();
    return false;
  }
  bool ok = true;
  ok &= make_map_bf16(&st->zp_km, st->zp, H, B, 2 * (count + 1), (int64_t)act, TBM);
  ok &= make_map_bf16(&st->zp_km64, st->zp, H, B, 2 * (count + 1), (int64_t)act, 64);
  ok &= make_map_bf16(&st->zp_mn, st->zp, H, B, 2 * (count + 1), (int64_t)act, 64);
  ok &= make_map_bf16(&st->fep_km, st->fep, H, B, 2 * count, (int64_t)act, TBM);
  ok &= make_map_bf16(&st->fep_mn, st->fep, H, B, 2 * count, (int64_t)act, 64);
  ok &= make_map_bf16(&st->wp_km128, st->wp, H, H, 2 * count, (int64_t)w, 128);
  ok &= make_map_bf16(&st->wp_km64, st->wp, H, H, 2 * count, (int64_t)w, 64);
  ok &= make_map_bf16(&st->wp_mn, st->wp, H, H, 2 * count, (int64_t)w, 64);
  if (!ok)
    return false;
  st->dirty[PL_Z].assign(count + 1, 1);
  st->dirty[PL_FE].assign(count, 1);
  st->dirty[PL_W].assign(count, 1);
  st->planes = true;
  // fp32 feedback errors can be dropped when nothing but the plane-reading kernels consumes
  // them: no ePC adjoint chain (it keeps its source in fe), feedback weights above every layer
  // of the run (else the direct-feedback product falls to the CUDA-core kernel, which reads fp32).
  st->fe_only = !getenv("DPC_KEEP_FE_FP32");
  for (int i = first; i < first + count && st->fe_only; ++i)
    st->fe_only = !plan->h[i].adj && i + 1 < plan->n && plan->h[i + 1].Psi != nullptr;
  return true;
}

static void planes_free(TcState* st)
{
  if (st->zp)
    cudaFree(st->zp);
  if (st->fep)
    cudaFree(st->fep);
  if (st->wp)
    cudaFree(st->wp);
  st->zp = st->fep = st->wp = nullptr;
  st->planes = false;
}

static bool run_init(dpc_plan* plan, TcState* st, int best_first, int best_count);

int tc_plan_init(dpc_plan* plan)
{
  plan->run = TensorRun();
  auto* st = new TcState();
  plan->tc = st;
  if (getenv("DPC_DISABLE_TENSOR_CORES"))
    return DPC_OK;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, plan->ctx->device) != cudaSuccess || prop.major != 10)
  {
    // tcgen05 exists on sm_100 only; other devices keep the CUDA-core path
    fprintf(stderr, "deepity_b200: device %d is not sm_100: every layer runs on the CUDA-core "
                    "kernels\n", plan->ctx->device);
    return DPC_OK;
  }
  st->max_smem = (int)prop.sharedMemPerBlockOptin;
  const int B = plan->batch, n = plan->n;
  if (B % TBM != 0)
    return DPC_OK;
  // Longest run of identical square DirectKP/Full layers at constant strides.
  int best_first = 0, best_count = 0;
  int i = 0;
  while (i + 1 < n)
  {
    const dpc_layer& L0 = plan->h[i];
    const bool ok0 = L0.next_size == L0.size && L0.size % 256 == 0 && L0.size >= 256 &&
                     !(L0.flags & DPC_LAYER_INPUT_ACT) && L0.fe && L0.preact &&
                     ((uintptr_t)L0.z % 128 == 0) && ((uintptr_t)L0.W % 128 == 0) &&
                     ((uintptr_t)L0.fe % 128 == 0);
    if (!ok0)
    {
      ++i;
      continue;
    }
    int j = i + 1;
    int64_t zs = 0, ws = 0, fs = 0;
    while (j + 1 < n)
    {
      const dpc_layer& Lj = plan->h[j];
      const dpc_layer& Lp = plan->h[j - 1];
      if (Lj.size != L0.size || Lj.next_size != L0.size || (Lj.flags & DPC_LAYER_INPUT_ACT))
        break;
      const int64_t dz = Lj.z - Lp.z, dw = Lj.W - Lp.W, df = Lj.fe - Lp.fe;
      if (j == i + 1)
        zs = dz, ws = dw, fs = df;
      if (dz != zs || dw != ws || df != fs || dz <= 0 || dw <= 0 || df <= 0)
        break;
      ++j;
    }
    if (j - i > best_count)
    {
      best_first = i, best_count = j - i;
      plan->run.z_stride = zs, plan->run.w_stride = ws, plan->run.out_stride = fs;
    }
    i = j;
  }
  if (cudaMalloc(&st->error_flag, sizeof(int)) != cudaSuccess ||
      cudaMemset(st->error_flag, 0, sizeof(int)) != cudaSuccess ||
      cudaMallocHost(&st->error_host, sizeof(int)) != cudaSuccess)
    return DPC_OK;
  *st->error_host = 0;
  if (best_count >= 1 && !run_init(plan, st, best_first, best_count))
    best_count = 0;
  // Layers outside the run whose three products fit the 256 x 256 CTA-pair tiles.
  // One launch per layer and product only pays when the product is large: a 256 x 256 tile takes
  // about 25 us from launch to its last store however few tiles there are, while the CUDA-core
  // kernels take all layers of a phase in one launch.  Measured on SimplePC networks of four equal
  // layers (whose launches of one phase run side by side on four streams), this path against the
  // CUDA-core kernels by batch x inputs x outputs: 2^28 equal, 2^29 1.5x, 2^30 1.9x, 2^32 2.8x
  // faster; a lone first layer: 2^28.6 equal, 2^31.6 5 % of the step.  Hence 2^29;
  // DPC_RECTANGULAR_MIN_WORK overrides it.
  long long min_work = 1LL << 29;
  if (const char* e = getenv("DPC_RECTANGULAR_MIN_WORK"))
    min_work = atoll(e);
  if (pair_ok(B, 256) && !getenv("DPC_DISABLE_RECTANGULAR"))
    for (int l = 0; l + 1 < n; ++l)
    {
      if (best_count > 0 && l >= best_first && l < best_first + best_count)
        continue;
      const dpc_layer& L = plan->h[l];
      const bool simple = (L.flags & DPC_LAYER_INPUT_ACT) != 0;
      // operands: the belief (SimplePC: f(z), kept in zF) and the feedback error (SimplePC: the
      // error of the layer above)
      const float* a_in = simple ? L.zF : L.z;
      const float* a_out = simple ? plan->h[l + 1].e : L.fe;
      if ((long long)B * L.size * L.next_size < min_work)
        continue;
      // (the input width may be any multiple of 8 from 64 up, e.g. 784: the operand copies of the
      // last K block and of the last column tile read zeros beyond the extent and the epilogues
      // stop at the last column)
      if (L.next_size <= 0 || L.size % 8 != 0 || L.size < 64 || L.next_size % 256 != 0 || !a_in || !a_out ||
          !L.W || !L.z || (!simple && !L.preact) || plan->h[l + 1].size != L.next_size ||
          ((uintptr_t)a_in % 128) != 0 || ((uintptr_t)L.W % 128) != 0 || ((uintptr_t)a_out % 128) != 0)
        continue;
      TcState::Extra x;
      x.layer = l;
      x.simple = simple;
      const int s_in = L.size, s_out = L.next_size;
      bool ok = true;
      ok &= make_map(&x.z_km, a_in, s_in, B, 1, (int64_t)B * s_in, TBM, false);
      ok &= make_map(&x.z_mn, a_in, s_in, B, 1, (int64_t)B * s_in, 32, true);
      ok &= make_map(&x.fe_km, a_out, s_out, B, 1, (int64_t)B * s_out, TBM, false);
      ok &= make_map(&x.fe_mn, a_out, s_out, B, 1, (int64_t)B * s_out, 32, true);
      ok &= make_map(&x.w_km128, L.W, s_in, s_out, 1, (int64_t)s_in * s_out, 128, false);
      ok &= make_map(&x.w_mn, L.W, s_in, s_out, 1, (int64_t)s_in * s_out, 32, true);
      if (ok)
        st->extras.push_back(x);
      else
        fprintf(stderr, "deepity_b200: a tensor map for layer %d was refused: it runs on the "
                        "CUDA-core kernels\n", l);
    }
  st->ok = best_count > 0 || !st->extras.empty();
  return DPC_OK;
}

// Tensor maps, sweep counters and operand planes of the run [best_first, best_first + best_count).
static bool run_init(dpc_plan* plan, TcState* st, int best_first, int best_count)
{
  const int B = plan->batch, n = plan->n;
  if (best_count == 1)
  {
    const dpc_layer& L0 = plan->h[best_first];
    plan->run.z_stride = (int64_t)B * L0.size;
    plan->run.w_stride = (int64_t)L0.size * L0.size;
    plan->run.out_stride = (int64_t)B * L0.size;
  }
  const dpc_layer& L0 = plan->h[best_first];
  const int H = L0.size;
  bool ok = true;
  ok &= make_map(&st->z_km, L0.z, H, B, best_count, plan->run.z_stride, TBM, false);
  ok &= make_map(&st->z_km64, L0.z, H, B, best_count, plan->run.z_stride, 64, false);
  ok &= make_map(&st->fe_km, L0.fe, H, B, best_count, plan->run.out_stride, TBM, false);
  ok &= make_map(&st->w_km32, L0.W, H, H, best_count, plan->run.w_stride, 32, false);
  ok &= make_map(&st->w_km64, L0.W, H, H, best_count, plan->run.w_stride, 64, false);
  ok &= make_map(&st->w_km128, L0.W, H, H, best_count, plan->run.w_stride, 128, false);
  ok &= make_map(&st->w_km256, L0.W, H, H, best_count, plan->run.w_stride, 256, false);
  ok &= make_map(&st->z_mn, L0.z, H, B, best_count, plan->run.z_stride, 32, true);
  ok &= make_map(&st->fe_mn, L0.fe, H, B, best_count, plan->run.out_stride, 32, true);
  ok &= make_map(&st->w_mn, L0.W, H, H, best_count, plan->run.w_stride, 32, true);
  if (!ok)
  {
    // the driver refused a tensor map: stay on the CUDA-core path, audibly
    fprintf(stderr, "deepity_b200: a tensor map for layers %d..%d was refused: they run on the "
                    "CUDA-core kernels\n", best_first, best_first + best_count - 1);
    return false;
  }
  {
    // Maps over beliefs and errors that also cover the layer above the run's last layer (it
    // has the run's width, and sits one stride further when the arenas are contiguous).
    const int top = best_first + best_count;
    bool fits = top < n && best_count >= 1 && plan->h[top].size == H && plan->h[top].e &&
                ((uintptr_t)L0.e % 128 == 0);
    if (fits && best_count >= 2)
    {
      const int64_t es = plan->h[best_first + 1].e - L0.e;
      fits = es == plan->run.z_stride;
      for (int j = best_first + 1; fits && j <= top; ++j)
        fits = plan->h[j].z - plan->h[j - 1].z == plan->run.z_stride &&
               plan->h[j].e - plan->h[j - 1].e == es;
    }
    else if (fits)
      fits = plan->h[top].z - L0.z == plan->run.z_stride && plan->h[top].e - L0.e == plan->run.z_stride;
    if (fits)
      st->up_maps = make_map(&st->zup_km, L0.z, H, B, best_count + 1, plan->run.z_stride, TBM, false) &&
                    make_map(&st->eup_km, L0.e, H, B, best_count + 1, plan->run.z_stride, TBM, false);
  }
  if (cudaMalloc(&st->chain_counters, sizeof(int) * (size_t)best_count * (B / 64)) != cudaSuccess)
    return false;
  plan->run.first = best_first;
  plan->run.count = best_count;
  plan->run.width = H;
  if (planes_init(plan, st, best_first, best_count, H) && st->planes && st->up_maps &&
      !getenv("DPC_DISABLE_STAGED_OUTPUT"))
  {
    // errors of the run's layers and the layer above it sit at the belief stride (checked for
    // up_maps above): one store map covers them
    st->store_maps =
        make_store_map(&st->e_st, L0.e, false, H, B, best_count + 1, plan->run.z_stride) &&
        make_store_map(&st->fep_st, st->fep, true, H, B, 2 * best_count, (int64_t)B * H) &&
        make_store_map(&st->z_st, L0.z, false, H, B, best_count + 1, plan->run.z_stride) &&
        make_store_map(&st->zp_st, st->zp, true, H, B, 2 * (best_count + 1), (int64_t)B * H) &&
        make_store_map(&st->w_st, L0.W, false, H, H, best_count, plan->run.w_stride) &&
        make_store_map(&st->wp_st, st->wp, true, H, H, 2 * best_count, (int64_t)H * H);
  }
  if (!st->planes && !getenv("DPC_DISABLE_PLANES") && split_scheme(plan) == 2 && pair_ok(B, H))
  {
    // no memory (or no tensor map) for the planes: the kernels split the operands themselves
    planes_free(st);
    fprintf(stderr, "deepity_b200: operand planes unavailable for this plan, using the in-kernel "
                    "operand split\n");
  }
  return true;
}

void tc_plan_free(dpc_plan* plan)
{
  auto* st = static_cast<TcState*>(plan->tc);
  if (!st)
    return;
  if (st->error_flag)
    cudaFree(st->error_flag);
  if (st->chain_counters)
    cudaFree(st->chain_counters);
  if (st->error_host)
    cudaFreeHost(st->error_host);
  planes_free(st);
  delete st;
  plan->tc = nullptr;
  plan->run = TensorRun();
}

void tc_set_chain_trace(dpc_plan* plan, unsigned long long* buf)
{
  auto* st = static_cast<TcState*>(plan->tc);
  if (st)
    st->trace = buf;
}

int tc_check_error(dpc_plan* plan)
{
  auto* st = static_cast<TcState*>(plan->tc);
  if (!st || !st->ok)
    return DPC_OK;
  if (cudaMemcpyAsync(st->error_host, st->error_flag, sizeof(int), cudaMemcpyDeviceToHost,
                      plan->ctx->stream) != cudaSuccess ||
      cudaStreamSynchronize(plan->ctx->stream) != cudaSuccess)
    return fail(DPC_ERR_CUDA, "reading the tensor-core status flag failed");
  if (*st->error_host)
  {
    cudaMemsetAsync(st->error_flag, 0, sizeof(int), plan->ctx->stream);
    return fail(DPC_ERR_TIMEOUT, "a tensor-core kernel gave up waiting on a pipeline barrier");
  }
  return DPC_OK;
}

// CTA-pair kernels take 256 x 256 tiles; DPC_DISABLE_CTA_PAIRS keeps the single-CTA kernels
// (used by the tests that compare the two).
static bool pair_ok(int rows, int cols)
{
  static const bool off = getenv("DPC_DISABLE_CTA_PAIRS") != nullptr;
  return !off && rows % 256 == 0 && cols % 256 == 0;
}

static bool all_sgd(const dpc_plan* p)
{
  for (int i = 0; i < p->n; ++i)
    if (p->h[i].next_size > 0 && p->h[i].opt != DPC_OPT_SGD)
      return false;
  return true;
}

// DPC_PRECISION_MIXED: gradient-path products in one TF32 pass when every weight optimizer is
// SGD (an Adam-type update would turn the TF32 rounding of a near-zero gradient into a full step).
// Not where the plan has operand planes: the three-BF16-pass kernels on pre-split operands are
// faster than the one-pass TF32 kernels on fp32 tensors (they read half the operand bytes per
// pass pair and need no fp32 feedback errors) AND exact to 2^-16, so the mode then runs exactly
// what the FP32 mode runs.
static bool fast_grad(const dpc_plan* p)
{
  const auto* st = static_cast<const TcState*>(p->tc);
  return p->ctx->precision == DPC_PRECISION_MIXED && all_sgd(p) && !(st && st->planes);
}

// fp32 mode: how the operands are split for the tensor cores.  2 = three BF16 passes over
// (bf16(x), bf16(x - bf16(x))): per-product error 2^-16, measured 2e-5 on whole train steps against
// the 1e-4 bound, at twice the tensor rate of 1 = three TF32 passes (error 2^-21).  Adam-type
// updates amplify rounding noise up to a full step per element, so networks that use them keep
// scheme 1; so does anything run with DPC_FP32_SCHEME=tf32x3.  One scheme per plan: the sweep and
// the settling passes must round alike for the errors right after the sweep to vanish.
static int split_scheme(const dpc_plan* p)
{
  const char* env = getenv("DPC_FP32_SCHEME");
  if (env && !strcmp(env, "tf32x3"))
    return 1;
  return all_sgd(p) ? 2 : 1;
}

// ---- operand planes: which layers lag behind their fp32 tensors -----------------------------
// Indices are relative to the run; beliefs have one entry more (the layer above the run).
static void planes_mark(TcState* st, int kind, int r0, int r1, uint8_t v)
{
  if (!st->planes)
    return;
  auto& d = st->dirty[kind];
  r0 = std::max(r0, 0);
  r1 = std::min(r1, (int)d.size());
  for (int i = r0; i < r1; ++i)
    d[i] = v;
}

// Brings the planes of layers [r0, r1) up to date (one split launch per maximal stale sub-range).
static int planes_need(dpc_plan* p, TcState* st, int kind, int r0, int r1)
{
  if (!st->planes)
    return DPC_OK;
  auto& d = st->dirty[kind];
  r0 = std::max(r0, 0);
  r1 = std::min(r1, (int)d.size());
  const long long H = p->run.width;
  const long long elems = kind == PL_W ? H * H : (long long)p->batch * H;
  __nv_bfloat16* base = kind == PL_Z ? st->zp : (kind == PL_FE ? st->fep : st->wp);
  int i = r0;
  while (i < r1)
  {
    if (!d[i])
    {
      ++i;
      continue;
    }
    int j = i;
    while (j < r1 && d[j] && j - i < 32768)
      ++j;
    dim3 grid((unsigned)std::min<long long>((elems / 8 + 255) / 256, 1024), (unsigned)(j - i));
    split_planes_kernel<<<grid, 256, 0, p->ctx->stream>>>(p->d, p->run.first + i, p->run.first,
                                                          kind, base, elems);
    p->ctx->launches += 1;
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess)
      return cuda_fail(cudaGetLastError(), "split_planes kernel launch");
    for (int k = i; k < j; ++k)
      d[k] = 0;
    i = j;
  }
  return DPC_OK;
}

// Pre-split operands are read when the plan runs the 3xBF16 scheme in an fp32-accurate mode.
static bool planes_on(const dpc_plan* p, const TcState* st)
{
  return st->planes && p->ctx->precision != DPC_PRECISION_TF32 && split_scheme(p) == 2;
}
// ... and every kernel of this file then writes the planes of what it produces (in the pure
// TF32 mode nobody reads them: they are left to go stale and marked so).
static bool planes_kept(const dpc_plan* p, const TcState* st)
{
  return planes_on(p, st);
}

// The fp32 feedback errors of the run are dropped wherever the planes are kept (FP32 mode and the
// mixed mode, which then runs the same kernels).
static bool fe_only_now(const dpc_plan* p, const TcState* st)
{
  return planes_kept(p, st) && st->fe_only && p->ctx->precision != DPC_PRECISION_TF32;
}

static TcParams base_params(dpc_plan* p, TcState* st, int first, int count, int M, int N, int K,
                            int BN, int flags, int mode, int BM = TBM)
{
  TcParams P;
  const bool keep = planes_kept(p, st);
  P.zp = keep ? st->zp : nullptr;
  P.fep = keep ? st->fep : nullptr;
  P.wp = keep ? st->wp : nullptr;
  P.act_elems = (long long)p->batch * p->run.width;
  P.w_elems = (long long)p->run.width * p->run.width;
  P.wait_cycles = st->wait_cycles;
  P.fe_only = fe_only_now(p, st) ? 1 : 0;
  P.tstore = 0;
  P.layers = p->d;
  P.first = first;
  P.count = count;
  P.n_layers = p->n;
  P.batch = p->batch;
  P.run_first = p->run.first;
  P.M = M, P.N = N, P.K = K;
  P.tiles_m = M / BM;
  P.tiles_n = (N + BN - 1) / BN; // a last column tile may reach beyond N: its epilogue stops at N
  P.flags = flags;
  P.mode = mode;
  P.energy = p->energy;
  P.error_flag = st->error_flag;
  P.chain = 0;
  P.chain_counters = nullptr;
  P.chain_target = 0;
  P.trace = nullptr;
  P.stage_in = 0;
  return P;
}

int tc_forward(dpc_plan* p, int first, int count, int flags)
{
  auto* st = static_cast<TcState*>(p->tc);
  if (st && st->ok && count == 1 && !range_in_run(p, first, 1))
    return tc_extra_forward(p, first, flags);
  if (!st || !st->ok || !range_in_run(p, first, count))
    return 1;
  const int H = p->run.width, B = p->batch;
  // the pass after the last settling step: it only refreshes the errors the learning phase reads
  const bool refresh =
      (flags & DPC_FWD_FE) && !(flags & DPC_FWD_ERR_NEXT) && (flags & DPC_FWD_TRANSIENT);
  const bool tf32 = p->ctx->precision == DPC_PRECISION_TF32 || (refresh && fast_grad(p));
  const int scheme = split_scheme(p);
  const int r0 = first - p->run.first;
  int rc;
  if (pair_ok(B, H))
  {
    TcParams P = base_params(p, st, first, count, B, H, H, 256, flags, 0, 256);
    // What the epilogue reads from the layer above is the same for every layer of the launch
    // unless a softmax head sits right above the range: stage it through shared memory.
    const CUtensorMap* up = nullptr;
    bool ce = false;
    for (int i = first; i <= first + count && i < p->n; ++i)
      ce |= (p->h[i].flags & DPC_LAYER_SOFTMAX_CE) != 0;
    if (st->up_maps && !ce && !getenv("DPC_DISABLE_STAGED_INPUT"))
    {
      if ((flags & DPC_FWD_ERR_NEXT) && !(flags & DPC_FWD_COPY_NEXT))
        P.stage_in = 1, up = &st->zup_km;
      else if ((flags & DPC_FWD_FE) && !(flags & DPC_FWD_ERR_NEXT))
        P.stage_in = 2, up = &st->eup_km;
    }
    if (!tf32 && planes_on(p, st))
    {
      if ((rc = planes_need(p, st, PL_Z, r0, r0 + count)) != DPC_OK ||
          (rc = planes_need(p, st, PL_W, r0, r0 + count)) != DPC_OK)
        return rc;
      P.tstore = (st->store_maps && P.stage_in != 0) ? 1 : 0;
      rc = launch<TC_FWD, 256, 3, 128, true>(p, st, st->zp_km, st->wp_km128, P, up);
    }
    else
      rc = tf32 ? launch<TC_FWD, 256, 0, 128, true>(p, st, st->z_km, st->w_km128, P, up)
         : scheme == 2 ? launch<TC_FWD, 256, 2, 128, true>(p, st, st->z_km, st->w_km128, P, up)
                       : launch<TC_FWD, 256, 1, 128, true>(p, st, st->z_km, st->w_km128, P, up);
  }
  else if (tf32)
    rc = launch<TC_FWD, 256, 0>(p, st, st->z_km, st->w_km256,
                                base_params(p, st, first, count, B, H, H, 256, flags, 0));
  else
  {
    TcParams P = base_params(p, st, first, count, B, H, H, 128, flags, 0);
    rc = scheme == 2 ? launch<TC_FWD, 128, 2>(p, st, st->z_km, st->w_km128, P)
                     : launch<TC_FWD, 128, 1>(p, st, st->z_km, st->w_km128, P);
  }
  if (rc == DPC_OK)
  {
    // every variant's epilogue keeps the planes of what it writes (when the plan has planes)
    const uint8_t stale = planes_kept(p, st) ? 0 : 1;
    if (flags & DPC_FWD_FE)
      planes_mark(st, PL_FE, r0, r0 + count, stale);
    if (flags & DPC_FWD_COPY_NEXT)
      planes_mark(st, PL_Z, r0 + 1, r0 + count + 1, stale);
  }
  return rc;
}

// The sequential forward sweep over layers [first, first+count) of the run as ONE persistent
// launch: 128 x 64 output tiles, one CTA per tile, every CTA walking all layers and
// synchronising per row block through counters in global memory (no grid-wide barrier: a
// row block of layer l+1 only needs the same row block of layer l).  All CTAs must be
// resident at once, so the tile grid may not exceed the SM count.
int tc_project_forward(dpc_plan* p, int first, int count, int flags)
{
  auto* st = static_cast<TcState*>(p->tc);
  if (!st || !st->ok || !range_in_run(p, first, count) || count < 2)
    return 1;
  const int H = p->run.width, B = p->batch;
  // Narrow 128 x 32 tiles: B/128 * H/32 CTAs (128 for the 1024 x 512 layers of the deep-stack
  // benchmark) keep the epilogue and the publish step on the dependent path short.  (Tiles of
  // 64 rows were measured too: a tcgen05.mma costs about the same whatever M and N are, so
  // they do not shorten the chain.)
  const int BNC = ((B / TBM) * (H / 32) <= p->ctx->sm_count) ? 32 : 64;
  const int tiles = (B / TBM) * (H / BNC);
  if (tiles > p->ctx->sm_count)
  {
    if (!st->warned_fallback)
      fprintf(stderr, "deepity_b200: the forward sweep of this plan needs %d resident CTAs (> %d "
                      "SMs): falling back to one launch per layer\n", tiles, p->ctx->sm_count);
    st->warned_fallback = true;
    return 1;
  }
  TcParams P = base_params(p, st, first, count, B, H, H, BNC, flags, 0);
  P.chain = 1;
  P.chain_counters = st->chain_counters;
  P.chain_target = (H / BNC) + st->chain_target_bias; // CTAs per row block
  P.trace = st->trace;
  cudaError_t e = cudaMemsetAsync(st->chain_counters, 0, sizeof(int) * (size_t)count * (B / 64),
                                  p->ctx->stream);
  if (e != cudaSuccess)
    return cuda_fail(e, "cudaMemsetAsync(chain counters)");
  const bool tf32 = p->ctx->precision == DPC_PRECISION_TF32;
  const int scheme = split_scheme(p);
  const int r0 = first - p->run.first;
  int rc;
  // K-split variant: 128 x 64 tiles, two CTAs (one cluster) per tile with half of K each.
  // Summing K in two halves rounds differently from the settling passes' single accumulation,
  // so right after the sweep e = z - mu is ~1e-7 where it is exactly 0 with matching orders
  // (as in the reference, which uses one GEMM routine for both).  Harmless for SGD; Adam-type
  // updates normalise such noise up to a full step, so they keep the single-accumulation sweep.
  const int ks_tiles = (B / TBM) * (H / 64);
  if (all_sgd(p) && 2 * ks_tiles <= p->ctx->sm_count && (H / 64) % 2 == 0 &&
      !getenv("DPC_DISABLE_KSPLIT"))
  {
    TcParams Q = base_params(p, st, first, count, B, H, H, 64, flags, 0);
    Q.chain = 1, Q.chain_counters = st->chain_counters, Q.trace = st->trace;
    // CTAs that produce one half of K: half of the column tiles x CTAs per tile
    Q.chain_target = (H / 64) + st->chain_target_bias;
    if (!tf32 && planes_on(p, st))
    {
      // the first layer's input and every layer's weights must be split; the sweep itself
      // writes the planes of every belief it produces
      if ((rc = planes_need(p, st, PL_Z, r0, r0 + 1)) != DPC_OK ||
          (rc = planes_need(p, st, PL_W, r0, r0 + count)) != DPC_OK)
        return rc;
      rc = launch<TC_FWD, 64, 3, 128, false, 2>(p, st, st->zp_km, st->wp_km64, Q);
    }
    else
      rc = tf32 ? launch<TC_FWD, 64, 0, 128, false, 2>(p, st, st->z_km, st->w_km64, Q)
         : scheme == 2 ? launch<TC_FWD, 64, 2, 128, false, 2>(p, st, st->z_km, st->w_km64, Q)
                       : launch<TC_FWD, 64, 1, 128, false, 2>(p, st, st->z_km, st->w_km64, Q);
  }
  else if (BNC == 32)
    rc = tf32 ? launch<TC_FWD, 32, 0>(p, st, st->z_km, st->w_km32, P)
       : scheme == 2 ? launch<TC_FWD, 32, 2>(p, st, st->z_km, st->w_km32, P)
                     : launch<TC_FWD, 32, 1>(p, st, st->z_km, st->w_km32, P);
  else
    rc = tf32 ? launch<TC_FWD, 64, 0>(p, st, st->z_km, st->w_km64, P)
       : scheme == 2 ? launch<TC_FWD, 64, 2>(p, st, st->z_km, st->w_km64, P)
                     : launch<TC_FWD, 64, 1>(p, st, st->z_km, st->w_km64, P);
  if (rc == DPC_OK && (flags & DPC_FWD_COPY_NEXT))
    planes_mark(st, PL_Z, r0 + 1, r0 + count + 1, planes_kept(p, st) ? 0 : 1);
  return rc;
}

int tc_update_state(dpc_plan* p, int first, int count)
{
  auto* st = static_cast<TcState*>(p->tc);
  if (st && st->ok && count == 1 && !range_in_run(p, first, 1))
    return tc_extra_update_state(p, first);
  if (!st || !st->ok || !range_in_run(p, first, count))
    return 1;
  const int H = p->run.width, B = p->batch;
  const bool tf32 = p->ctx->precision == DPC_PRECISION_TF32;
  const int scheme = split_scheme(p);
  const int r0 = first - p->run.first;
  int rc;
  if (pair_ok(B, H))
  {
    TcParams P = base_params(p, st, first, count, B, H, H, 256, 0, 0, 256);
    if (!tf32 && planes_on(p, st))
    {
      if ((rc = planes_need(p, st, PL_FE, r0, r0 + count)) != DPC_OK ||
          (rc = planes_need(p, st, PL_W, r0, r0 + count)) != DPC_OK)
        return rc;
      // plain updates (no momentum, no residual term) take their error and belief through
      // shared memory and write belief and planes with bulk stores
      bool plain = st->store_maps && !getenv("DPC_DISABLE_STAGED_OUTPUT") &&
                   !getenv("DPC_DISABLE_STAGED_INPUT");
      for (int i = first; i < first + count && plain; ++i)
        plain = !p->h[i].v && !(p->h[i].flags & DPC_LAYER_RESIDUAL);
      P.tstore = plain ? 1 : 0;
      rc = launch<TC_FB, 256, 3, 128, true>(p, st, st->fep_km, st->wp_mn, P);
    }
    else
      rc = tf32 ? launch<TC_FB, 256, 0, 128, true>(p, st, st->fe_km, st->w_mn, P)
         : scheme == 2 ? launch<TC_FB, 256, 2, 128, true>(p, st, st->fe_km, st->w_mn, P)
                       : launch<TC_FB, 256, 1, 128, true>(p, st, st->fe_km, st->w_mn, P);
  }
  else if (tf32)
    rc = launch<TC_FB, 256, 0>(p, st, st->fe_km, st->w_mn,
                               base_params(p, st, first, count, B, H, H, 256, 0, 0));
  else
  {
    TcParams P = base_params(p, st, first, count, B, H, H, 128, 0, 0);
    rc = scheme == 2 ? launch<TC_FB, 128, 2>(p, st, st->fe_km, st->w_mn, P)
                     : launch<TC_FB, 128, 1>(p, st, st->fe_km, st->w_mn, P);
  }
  if (rc == DPC_OK)
    planes_mark(st, PL_Z, r0, r0 + count, planes_kept(p, st) ? 0 : 1);
  return rc;
}

int tc_weight_gemm(dpc_plan* p, int first, int count, int mode, int decay_w)
{
  auto* st = static_cast<TcState*>(p->tc);
  if (st && st->ok && count == 1 && !range_in_run(p, first, 1))
    return tc_extra_weight_gemm(p, first, mode, decay_w);
  if (!st || !st->ok || !range_in_run(p, first, count))
    return 1;
  for (int i = first; i < first + count; ++i)
  {
    const dpc_layer& L = p->h[i];
    bool eligible = true;
    if (mode == WG_LEARN_MODE && L.opt != DPC_OPT_SGD)
      eligible = false; // Adam-type updates go through the staging buffer (mode | WG_GRAD_MODE)
    if ((mode & WG_GRAD_MODE) && (!L.g_W || ((uintptr_t)L.g_W % 32) != 0))
      eligible = false;
    if ((mode & 1) == WG_DFA_MODE && (i + 1 >= p->n || !p->h[i + 1].Psi))
      eligible = false;
    if (!eligible)
    {
      if (fe_only_now(p, st))
        return fail(DPC_ERR_STATE, "weight-shaped product of a tensor-core layer is not eligible "
                                   "for the tensor-core kernel, and the fp32 feedback errors the "
                                   "CUDA-core kernel would read are not kept (DPC_KEEP_FE_FP32=1 "
                                   "keeps them)");
      return 1;
    }
  }
  const int H = p->run.width, B = p->batch;
  const bool tf32 = p->ctx->precision == DPC_PRECISION_TF32 || fast_grad(p);
  const int scheme = split_scheme(p);
  const int r0 = first - p->run.first;
  int rc;
  if (pair_ok(H, H))
  {
    TcParams P = base_params(p, st, first, count, H, H, B, 256, decay_w ? 1 : 0, mode, 256);
    if (!tf32 && planes_on(p, st))
    {
      if ((rc = planes_need(p, st, PL_FE, r0, r0 + count)) != DPC_OK ||
          (rc = planes_need(p, st, PL_Z, r0, r0 + count)) != DPC_OK)
        return rc;
      // in-place SGD updates take the weight tile through shared memory and write it and its
      // planes back with bulk stores
      P.tstore = (st->store_maps && !(mode & WG_GRAD_MODE) && !getenv("DPC_DISABLE_STAGED_OUTPUT") &&
                  !getenv("DPC_DISABLE_STAGED_INPUT"))
                     ? 1
                     : 0;
      rc = launch<TC_WG, 256, 3, 128, true>(p, st, st->fep_mn, st->zp_mn, P);
    }
    else
      rc = tf32 ? launch<TC_WG, 256, 0, 128, true>(p, st, st->fe_mn, st->z_mn, P)
         : scheme == 2 ? launch<TC_WG, 256, 2, 128, true>(p, st, st->fe_mn, st->z_mn, P)
                       : launch<TC_WG, 256, 1, 128, true>(p, st, st->fe_mn, st->z_mn, P);
  }
  else if (tf32)
    rc = launch<TC_WG, 256, 0>(
        p, st, st->fe_mn, st->z_mn,
        base_params(p, st, first, count, H, H, B, 256, decay_w ? 1 : 0, mode));
  else
  {
    TcParams P = base_params(p, st, first, count, H, H, B, 128, decay_w ? 1 : 0, mode);
    rc = scheme == 2 ? launch<TC_WG, 128, 2>(p, st, st->fe_mn, st->z_mn, P)
                     : launch<TC_WG, 128, 1>(p, st, st->fe_mn, st->z_mn, P);
  }
  if (rc == DPC_OK && !(mode & WG_GRAD_MODE))
    planes_mark(st, PL_W, r0, r0 + count, planes_kept(p, st) ? 0 : 1);
  return rc;
}

// ---- operand planes: what the rest of the library tells this file ---------------------------
// kind: 0 beliefs, 1 feedback errors, 2 weights.  Something outside this file wrote the fp32
// tensors of layers [first, first+count): their planes must be re-split before the next use.
void tc_touch(dpc_plan* p, int kind, int first, int count)
{
  auto* st = static_cast<TcState*>(p->tc);
  if (!st || !st->planes || kind < 0 || kind > 2)
    return;
  planes_mark(st, kind, first - p->run.first, first + count - p->run.first, 1);
}

void tc_fe_planes(dpc_plan* p, void** base, int* run_first, int* run_count, long long* elems,
                  int* only)
{
  auto* st = static_cast<TcState*>(p->tc);
  const bool on = st && st->planes && planes_on(p, st);
  *base = on ? st->fep : nullptr;
  *run_first = p->run.first;
  *run_count = on ? p->run.count : 0;
  *elems = (long long)p->batch * p->run.width;
  *only = (on && fe_only_now(p, st)) ? 1 : 0;
}

void tc_fe_written(dpc_plan* p, int first, int count)
{
  auto* st = static_cast<TcState*>(p->tc);
  if (st && st->planes)
    planes_mark(st, PL_FE, first - p->run.first, first + count - p->run.first, 0);
}

int tc_fe_need(dpc_plan* p, int first, int count)
{
  auto* st = static_cast<TcState*>(p->tc);
  if (!st || !st->planes || !planes_on(p, st))
    return DPC_OK;
  return planes_need(p, st, PL_FE, first - p->run.first, first + count - p->run.first);
}

int tc_sync_planes(dpc_plan* p)
{
  auto* st = static_cast<TcState*>(p->tc);
  if (!st || !st->planes || !planes_on(p, st))
    return DPC_OK;
  for (int kind = 0; kind < 3; ++kind)
  {
    int rc = planes_need(p, st, kind, 0, (int)st->dirty[kind].size());
    if (rc != DPC_OK)
      return rc;
  }
  return DPC_OK;
}

// ---- single layers outside the run (TcState::Extra) --------------------------------------------
// The same CTA-pair kernels on tensor maps of one layer: operands are the fp32 tensors (one TF32
// pass, three TF32 passes, or the three-BF16-pass split inside the kernel; no operand planes), the
// layer coordinate of every load is 0, the epilogue reads the layer above with per-lane loads.
static const TcState::Extra* find_extra(const TcState* st, int layer)
{
  for (const auto& x : st->extras)
    if (x.layer == layer)
      return &x;
  return nullptr;
}

bool tc_extra_layer(dpc_plan* p, int layer)
{
  auto* st = static_cast<TcState*>(p->tc);
  return st && st->ok && find_extra(st, layer) != nullptr;
}

static TcParams extra_params(dpc_plan* p, TcState* st, int layer, int M, int N, int K, int flags,
                             int mode)
{
  TcParams P = base_params(p, st, layer, 1, M, N, K, 256, flags, mode, 256);
  P.run_first = layer; // the maps hold this layer only
  P.zp = P.fep = P.wp = nullptr;
  P.fe_only = 0;
  return P;
}

// SimplePC: zF = f(z), the operand of the layer's forward product and of its weight update
// (src/layers/SimplePCLayer.cpp:146-150 keeps f(z) as last fed to the GEMM).
__global__ void input_activation_kernel(const dpc_layer* __restrict__ layers, int layer, long long n)
{
  const dpc_layer& L = layers[layer];
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n;
       i += (long long)gridDim.x * blockDim.x * 4)
  {
    const float4 z = *reinterpret_cast<const float4*>(L.z + i);
    const float in[8] = {z.x, z.y, z.z, z.w, 0.0f, 0.0f, 0.0f, 0.0f};
    float f[8], d[8];
    act_both8<false>(L.act, in, f, d);
    *reinterpret_cast<float4*>(L.zF + i) = make_float4(f[0], f[1], f[2], f[3]);
  }
}

int tc_extra_forward(dpc_plan* p, int layer, int flags)
{
  auto* st = static_cast<TcState*>(p->tc);
  const TcState::Extra* x = (st && st->ok) ? find_extra(st, layer) : nullptr;
  if (!x)
    return 1;
  const dpc_layer& L = p->h[layer];
  const bool refresh =
      (flags & DPC_FWD_FE) && !(flags & DPC_FWD_ERR_NEXT) && (flags & DPC_FWD_TRANSIENT);
  const bool tf32 = p->ctx->precision == DPC_PRECISION_TF32 || (refresh && fast_grad(p));
  const int scheme = split_scheme(p);
  if (x->simple)
  {
    const long long n = (long long)p->batch * L.size; // a multiple of 4
    const unsigned blocks = (unsigned)std::min<long long>((n / 4 + 255) / 256, 4096);
    input_activation_kernel<<<blocks, 256, 0, p->ctx->stream>>>(p->d, layer, n);
    p->ctx->launches += 1;
    if (cudaPeekAtLastError() != cudaSuccess)
      return cuda_fail(cudaGetLastError(), "input_activation kernel launch");
  }
  TcParams P = extra_params(p, st, layer, p->batch, L.next_size, L.size, flags, 0);
  const int rc =
      tf32 ? launch<TC_FWD, 256, 0, 128, true>(p, st, x->z_km, x->w_km128, P)
      : scheme == 2 ? launch<TC_FWD, 256, 2, 128, true>(p, st, x->z_km, x->w_km128, P)
                    : launch<TC_FWD, 256, 1, 128, true>(p, st, x->z_km, x->w_km128, P);
  // the belief it may have written can be the first layer of the run: its planes are stale
  if (rc == DPC_OK && (flags & DPC_FWD_COPY_NEXT))
    tc_touch(p, PL_Z, layer + 1, 1);
  return rc;
}

int tc_extra_update_state(dpc_plan* p, int layer)
{
  auto* st = static_cast<TcState*>(p->tc);
  const TcState::Extra* x = (st && st->ok) ? find_extra(st, layer) : nullptr;
  if (!x)
    return 1;
  const dpc_layer& L = p->h[layer];
  const bool tf32 = p->ctx->precision == DPC_PRECISION_TF32;
  const int scheme = split_scheme(p);
  TcParams P = extra_params(p, st, layer, p->batch, L.size, L.next_size, 0, 0);
  return tf32 ? launch<TC_FB, 256, 0, 128, true>(p, st, x->fe_km, x->w_mn, P)
       : scheme == 2 ? launch<TC_FB, 256, 2, 128, true>(p, st, x->fe_km, x->w_mn, P)
                     : launch<TC_FB, 256, 1, 128, true>(p, st, x->fe_km, x->w_mn, P);
}

int tc_extra_weight_gemm(dpc_plan* p, int layer, int mode, int decay_w)
{
  auto* st = static_cast<TcState*>(p->tc);
  const TcState::Extra* x = (st && st->ok) ? find_extra(st, layer) : nullptr;
  if (!x)
    return 1;
  const dpc_layer& L = p->h[layer];
  if (mode == WG_LEARN_MODE && L.opt != DPC_OPT_SGD)
    return 1; // Adam-type updates go through the staging buffer (mode | WG_GRAD_MODE)
  if ((mode & WG_GRAD_MODE) && (!L.g_W || ((uintptr_t)L.g_W % 32) != 0))
    return 1;
  if ((mode & 1) == WG_DFA_MODE && (layer + 1 >= p->n || !p->h[layer + 1].Psi))
    return 1;
  const bool tf32 = p->ctx->precision == DPC_PRECISION_TF32 || fast_grad(p);
  const int scheme = split_scheme(p);
  TcParams P = extra_params(p, st, layer, L.next_size, L.size, p->batch, decay_w ? 1 : 0, mode);
  return tf32 ? launch<TC_WG, 256, 0, 128, true>(p, st, x->fe_mn, x->z_mn, P)
       : scheme == 2 ? launch<TC_WG, 256, 2, 128, true>(p, st, x->fe_mn, x->z_mn, P)
                     : launch<TC_WG, 256, 1, 128, true>(p, st, x->fe_mn, x->z_mn, P);
}

void tc_set_wait_limit(dpc_plan* p, long long cycles, int chain_target_bias)
{
  auto* st = static_cast<TcState*>(p->tc);
  if (!st)
    return;
  st->wait_cycles = cycles > 0 ? cycles : kWaitCyclesDefault;
  st->chain_target_bias = chain_target_bias;
}

// One line on which kernels the plan's weight layers run.
std::string tc_describe(dpc_plan* p)
{
  auto* st = static_cast<TcState*>(p->tc);
  const int weight_layers = p->n - 1;
  if (!st || !st->ok)
    return "all " + std::to_string(weight_layers) + " weight layers on CUDA cores";
  const bool tf32 = p->ctx->precision == DPC_PRECISION_TF32;
  std::string out;
  int on_tc = 0;
  if (p->run.count > 0)
  {
    const bool pair = pair_ok(p->batch, p->run.width);
    std::string mode = tf32 ? "1xTF32"
                       : split_scheme(p) == 2 ? (planes_on(p, st) ? "3xBF16 from pre-split planes"
                                                                 : "3xBF16 split in the kernel")
                                              : "3xTF32";
    if (fast_grad(p))
      mode += " (gradient path 1xTF32)";
    out = "layers " + std::to_string(p->run.first) + ".." +
          std::to_string(p->run.first + p->run.count - 1) + " on tcgen05 (" +
          (pair ? "CTA pairs 256x256" : "single-CTA tiles") + ", " + mode + "); ";
    on_tc += p->run.count;
  }
  if (!st->extras.empty())
  {
    out += "layer";
    for (const auto& x : st->extras)
      out += " " + std::to_string(x.layer) + " (" + std::to_string(p->h[x.layer].size) + "->" +
             std::to_string(p->h[x.layer].next_size) + ")";
    out += std::string(" on tcgen05 (CTA pairs 256x256, ") +
           (tf32 ? "1xTF32" : split_scheme(p) == 2 ? "3xBF16 split in the kernel" : "3xTF32") + "); ";
    on_tc += (int)st->extras.size();
  }
  return out + std::to_string(weight_layers - on_tc) + " weight layers on CUDA cores";
}
} // namespace dpc
