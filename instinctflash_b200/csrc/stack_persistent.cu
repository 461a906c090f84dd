// Persistent whole-stack kernel for the skinny-M (M <= 128) action-expert loop.
//
// One cooperative launch walks a program of operators (FP8 GEMMs, the gated activation +
// quantiser, the residual + RMS norm + quantiser) over all layers and flow steps, instead of one
// launch per operator (the reference's expert loop is ~1500 launches per inference,
// instinctflash/engines/pi05/engine.py:225-253).  At M = 50 a GEMM moves 1.5-8 MB of weights,
// 0.3-1.3 us of HBM time: launch latency, not bandwidth, bounds the per-operator path.
//
// Design (one CTA per SM, 224 threads):
//   warp 0     W producer: streams 64-row weight tiles through a shared-memory ring by TMA, four
//              128-byte K slabs per instruction and stage (the operands are mapped as
//              [K / 128][rows][128 bytes]).  Weights do not depend on activations, so it runs
//              ahead across operator boundaries: while the grid waits at a dependency, up to
//              96 KB of the next operator's weights per SM are already in flight (14 MB over the
//              GPU, a whole layer).
//   warp 6     A producer: loads the activation tile of each K step into the same stage; it is
//              the one that waits for grid-wide dependencies.
//   warp 1     MMA issuer: tcgen05.mma 128 x 64 x 32 (rows >= M are padding, never stored),
//              two TMEM accumulators.
//   warps 2-5  epilogue / row operators: drain accumulators (raw bf16, or fp32 split-K partials),
//              and run the row operators (one row per CTA) between GEMM phases.
// Dependencies between operators are grid-wide counters in global memory (one per dependency,
// zeroed by the host before the launch): every CTA arrives once after its outputs are visible,
// consumers spin with a time budget.  Split-K partials are summed in a fixed order by the
// consuming row operator, so results do not depend on timing.
// Every wait is bounded; on a timeout the kernel records where, raises a global abort word that
// all spinning CTAs watch, drains and returns.
#include <cooperative_groups.h>
#include <cuda.h>
#include <cuda_runtime.h>
#include <string.h>

#include "../../include/iflb200.h"
#include "rowmath.cuh"

namespace iflb200 {
namespace stackk {

constexpr int BM = 128;       // UMMA M (rows >= M are padding)
constexpr int BN = 64;        // weight rows (output columns) per tile
constexpr int BK = 128;       // bytes per K step
constexpr int kSlabs = 4;     // 128-byte K slabs per stage and per TMA instruction: a CTA can issue a TMA
                              // instruction about every 0.2 us, so a K step per instruction made the
                              // activation loads of an operator (eight of them) its longest part
constexpr int STAGES = 3;     // stages of kSlabs slabs (M <= 64); two for the 128-row activation box
constexpr int A_ROWS = 64;    // rows of the activation box actually loaded (M <= 64) ...
constexpr int A_ROWS_WIDE = 128;  // ... or 128 (64 < M <= 128), with 8 stages
constexpr int kThreads = 224;
constexpr uint64_t kWaitBudgetNs = 2000000000ull;
// Time budget of every wait inside the kernel (read only on the slow path of a wait).
__device__ uint64_t g_stack_wait_budget_ns = kWaitBudgetNs;

enum : int { OP_GEMM = 1, OP_GATED = 2, OP_RESNORM = 3, OP_GEMM_GATED = 4, OP_ENCODE = 5 };
constexpr int HW = BN / 2;  // hidden units per work item of the gated GEMM (gate columns | up columns)

struct Op {  // mirrors iflb200_stack_op
  int32_t type, wait_bar, arrive_bar, tile_offset;
  int32_t N, K, split_k, act;
  int32_t tm_a, tm_w, pad0, pad1;
  void* out;
  const void* in;
  const float* row_scale;
  const float* col_scale;
  float* out_scale;
  float* res;
  int64_t ld_out, ld_in;
  float eps;
  int32_t pad2;
  float* aux;  // GEMM_GATED / ENCODE: row maxima of |h| (float bits); RESNORM: words to leave at zero (or null)
};
static_assert(sizeof(Op) == sizeof(iflb200_stack_op), "layout of iflb200_stack_op");
__device__ __forceinline__ bool is_gemm(const Op& op) { return op.type == OP_GEMM || op.type == OP_GEMM_GATED; }

__device__ __forceinline__ uint32_t ld_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Order generic-proxy accesses (plain loads/stores) against async-proxy ones (TMA) on data that
// other CTAs produce and consume inside this launch.
__device__ __forceinline__ void fence_proxy_async_all() {
  asm volatile("fence.proxy.async;" ::: "memory");
}
__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

#ifdef IFLB200_TRACE
// Experiments only (never part of the product library): wall-clock stamps of CTA 0's roles for
// operators [kTraceFirst, kTraceFirst + 16), event slots per operator below.
constexpr int kTraceFirst = 40;
__device__ unsigned long long g_stack_trace[16][16];
__device__ __forceinline__ void trace(int oi, int ev) {
  if (blockIdx.x == 0 && oi >= kTraceFirst && oi < kTraceFirst + 16) g_stack_trace[oi - kTraceFirst][ev] = globaltimer_ns();
}
#define TRACE(oi, ev) trace(oi, ev)
#else
#define TRACE(oi, ev)
#endif

struct Shared {
  uint32_t full[STAGES][2];
  uint32_t empty[STAGES][2];
  uint32_t tfull[2][2];
  uint32_t tempty[2][2];
  uint32_t tmem_base;
  uint32_t abort_flag;
  float red[3][4];
};

// status[0]: first timeout record (role << 24 | kind << 16 | op), status[1]: abort word
__device__ __forceinline__ bool wait_mbar(uint32_t bar, uint32_t parity, volatile uint32_t* local_abort,
                                          uint32_t* status, uint32_t code) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = 0;
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*local_abort) return false;
    if (++spins > 1024) {
      if (t0 == 0) t0 = globaltimer_ns();
      __nanosleep(64);
      if ((spins & 1023) == 0 && ld_acquire(status + 1)) {
        *local_abort = 1;
        return false;
      }
      if (globaltimer_ns() - t0 > g_stack_wait_budget_ns) {
        *local_abort = 1;
        atomicCAS(status, 0u, code);
        atomicExch(status + 1, 1u);
        return false;
      }
    }
  }
}

// Grid-wide dependency: wait until `target` CTAs have arrived on counter `bar`.
__device__ __forceinline__ bool wait_grid(const uint32_t* bar, uint32_t target, volatile uint32_t* local_abort,
                                          uint32_t* status, uint32_t code) {
  uint64_t t0 = 0;
  uint32_t spins = 0;
  while (ld_acquire(bar) < target) {
    if (*local_abort) return false;
    if (++spins > 64) {
      if (t0 == 0) t0 = globaltimer_ns();
      __nanosleep(32);
      if ((spins & 255) == 0 && ld_acquire(status + 1)) {
        *local_abort = 1;
        return false;
      }
      if (globaltimer_ns() - t0 > g_stack_wait_budget_ns) {
        *local_abort = 1;
        atomicCAS(status, 0u, code);
        atomicExch(status + 1, 1u);
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ int gemm_items(const Op& op) {
  return op.type == OP_GEMM_GATED ? (op.N + HW - 1) / HW : ((op.N + BN - 1) / BN) * op.split_k;
}

// k-step range of one split
__device__ __forceinline__ void split_range(const Op& op, int split, int& kb0, int& kb1) {
  const int steps = (op.K + BK - 1) / BK;
  if (op.type == OP_GEMM_GATED) {
    kb0 = 0;
    kb1 = steps;
    return;
  }
  kb0 = (int)(((int64_t)steps * split) / op.split_k);
  kb1 = (int)(((int64_t)steps * (split + 1)) / op.split_k);
}

// Row operators run on the 128 threads of the four epilogue warps; `t` = 0..127.
__device__ __forceinline__ float block_reduce128(float v, bool is_max, float* slot, int t) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xFFFFFFFFu, v, o);
    v = is_max ? max_f32(v, other) : __fadd_rn(v, other);
  }
  if ((t & 31) == 0) slot[t >> 5] = v;
  named_barrier_sync(1, 128);
  float r = slot[0];
#pragma unroll
  for (int i = 1; i < 4; ++i) r = is_max ? max_f32(r, slot[i]) : __fadd_rn(r, slot[i]);
  return r;
}

__device__ __forceinline__ void unpack_bf16x8(const uint4& u, float (&o)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    o[2 * i] = __uint_as_float(w[i] << 16);
    o[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ void load_f32x8_cg(const float* p, float (&o)[8]) {
  const float4 a = __ldcg(reinterpret_cast<const float4*>(p));
  const float4 b = __ldcg(reinterpret_cast<const float4*>(p + 4));
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w;
  o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
__device__ __forceinline__ void load_f32x8(const float* p, float (&o)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w;
  o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
__device__ __forceinline__ void store_codes8(uint8_t* p, const float (&v)[8], float inv) {
  const uint32_t lo = cvt_e4m3x4(__fmul_rn(v[0], inv), __fmul_rn(v[1], inv), __fmul_rn(v[2], inv), __fmul_rn(v[3], inv));
  const uint32_t hi = cvt_e4m3x4(__fmul_rn(v[4], inv), __fmul_rn(v[5], inv), __fmul_rn(v[6], inv), __fmul_rn(v[7], inv));
  *reinterpret_cast<uint2*>(p) = make_uint2(lo, hi);
}

constexpr int kRowIters = 8;  // 128 threads x 8 chunks x 8 elements = 8192 columns at most

// gated_act_quant of one row (instinctflash/kernels/activation.py:20-43 arithmetic).
__device__ void row_gated(const Op& op, int m, int t, float* red) {
  const int F = op.N;
  const __nv_bfloat16* gr = reinterpret_cast<const __nv_bfloat16*>(op.in) + (int64_t)m * op.ld_in;
  const __nv_bfloat16* ur = gr + F;
  const float rs = __ldcg(op.row_scale + m);
  float h[kRowIters][8];
  float amax = 0.0f;
  uint4 rg[kRowIters], ru[kRowIters];
#pragma unroll
  for (int it = 0; it < kRowIters; ++it) {
    const int c0 = (it * 128 + t) * 8;
    const bool on = c0 < F;
    rg[it] = on ? __ldcg(reinterpret_cast<const uint4*>(gr + c0)) : make_uint4(0, 0, 0, 0);  // written by other SMs:
    ru[it] = on ? __ldcg(reinterpret_cast<const uint4*>(ur + c0)) : make_uint4(0, 0, 0, 0);  // read through L2
  }
#pragma unroll
  for (int it = 0; it < kRowIters; ++it) {
    const int c0 = (it * 128 + t) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) h[it][i] = 0.0f;
    if (c0 < F) {
      float g[8], u[8], cg[8], cu[8];
      unpack_bf16x8(rg[it], g);
      unpack_bf16x8(ru[it], u);
      load_f32x8(op.col_scale + c0, cg);
      load_f32x8(op.col_scale + F + c0, cu);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        g[i] = __fmul_rn(__fmul_rn(g[i], rs), cg[i]);
        u[i] = __fmul_rn(__fmul_rn(u[i], rs), cu[i]);
      }
      if (op.act == IFLB200_ACT_GELU_TANH) {
#pragma unroll
        for (int i = 0; i < 8; ++i) h[it][i] = __fmul_rn(u[i], gelu_tanh_ref(g[i]));
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) h[it][i] = __fmul_rn(u[i], silu_ref(g[i]));
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = max_f32(amax, fabsf(h[it][i]));
    }
  }
  amax = block_reduce128(amax, true, red, t);
  float scale, inv;
  quant_scales(amax, scale, inv);
  if (t == 0) op.out_scale[m] = scale;
  uint8_t* qr = reinterpret_cast<uint8_t*>(op.out) + (int64_t)m * op.ld_out;
#pragma unroll
  for (int it = 0; it < kRowIters; ++it) {
    const int c0 = (it * 128 + t) * 8;
    if (c0 < F) store_codes8(qr + c0, h[it], inv);
  }
}

// Residual part + RMS norm + quantiser of one row (instinctflash/kernels/norm.py:44-80 for the
// flag set delta, delta_row, delta_col, fp32 residual).  The GEMM's accumulator arrives either as
// raw bf16 (split_k == 1) or as split_k fp32 partials, summed here in split order and rounded to
// bf16: the same rounding point as the raw accumulator.
__device__ void row_resnorm(const Op& op, int M, int m, int t, float (*red)[4]) {
  const int D = op.N;
  float* rr = op.res + (int64_t)m * D;
  const float drs = __ldcg(op.row_scale + m);
  float x[kRowIters][8];
  float sumsq = 0.0f;
#pragma unroll
  for (int it = 0; it < kRowIters; ++it) {
    const int c0 = (it * 128 + t) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) x[it][i] = 0.0f;
    if (c0 < D) {
      float d[8], cs[8], r[8];
      if (op.split_k > 1) {
        // partials in groups of eight: the loads of a group are all in flight before the first add
        // (the sum itself runs in split order)
        const float* p0 = reinterpret_cast<const float*>(op.in) + (int64_t)m * op.ld_in + c0;
        const int64_t step = (int64_t)M * op.ld_in;
        load_f32x8_cg(p0, d);
        for (int s = 1; s < op.split_k; s += 8) {
          float e[8][8];
#pragma unroll
          for (int q = 0; q < 8; ++q)
            if (s + q < op.split_k) load_f32x8_cg(p0 + (s + q) * step, e[q]);
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            if (s + q < op.split_k) {
#pragma unroll
              for (int i = 0; i < 8; ++i) d[i] = __fadd_rn(d[i], e[q][i]);
            }
          }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) d[i] = __bfloat162float(__float2bfloat16_rn(d[i]));
      } else {
        const uint4 u = __ldcg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(op.in) +
                                                              (int64_t)m * op.ld_in + c0));
        unpack_bf16x8(u, d);
      }
      load_f32x8(op.col_scale + c0, cs);
      load_f32x8(rr + c0, r);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        x[it][i] = __fmaf_rn(__fmul_rn(d[i], drs), cs[i], r[i]);
        sumsq = __fmaf_rn(x[it][i], x[it][i], sumsq);
      }
      *reinterpret_cast<float4*>(rr + c0) = make_float4(x[it][0], x[it][1], x[it][2], x[it][3]);
      *reinterpret_cast<float4*>(rr + c0 + 4) = make_float4(x[it][4], x[it][5], x[it][6], x[it][7]);
    }
  }
  const float var = div_full(block_reduce128(sumsq, false, red[0], t), (float)D);
  const float rstd = rsqrt_approx_ftz(__fadd_rn(var, op.eps));
  float amax = 0.0f;
#pragma unroll
  for (int it = 0; it < kRowIters; ++it) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      x[it][i] = __fmul_rn(x[it][i], rstd);
      amax = max_f32(amax, fabsf(x[it][i]));
    }
  }
  amax = block_reduce128(amax, true, red[1], t);
  float scale, inv;
  quant_scales(amax, scale, inv);
  if (t == 0) {
    op.out_scale[m] = scale;
    if (op.aux) op.aux[m] = 0.0f;  // row maximum of the gated GEMM before this operator: consumed, start over
  }
  uint8_t* qr = reinterpret_cast<uint8_t*>(op.out) + (int64_t)m * op.ld_out;
#pragma unroll
  for (int it = 0; it < kRowIters; ++it) {
    const int c0 = (it * 128 + t) * 8;
    if (c0 < D) store_codes8(qr + c0, x[it], inv);
  }
}

// Quantiser pass after the gated GEMM: codes of one part of a row of h (fp32) with the row's
// scale taken from the maxima the GEMM epilogues left in op.aux.  No reduction: a row is split
// over op.split_k parts so that all SMs share the rows.
__device__ void row_encode(const Op& op, int item, int t) {
  const int F = op.N, parts = op.split_k;
  const int m = item / parts, part = item - m * parts;
  const int width = ((F + parts - 1) / parts + 7) / 8 * 8;
  const int begin = part * width, end = min(F, begin + width);
  const float* hr = reinterpret_cast<const float*>(op.in) + (int64_t)m * op.ld_in;
  float scale, inv;
  quant_scales(__ldcg(op.aux + m), scale, inv);
  if (part == 0 && t == 0) op.out_scale[m] = scale;
  uint8_t* qr = reinterpret_cast<uint8_t*>(op.out) + (int64_t)m * op.ld_out;
  float v[kRowIters][8];
#pragma unroll
  for (int it = 0; it < kRowIters; ++it) {
    const int c0 = begin + (it * 128 + t) * 8;
    if (c0 < end) load_f32x8_cg(hr + c0, v[it]);
  }
#pragma unroll
  for (int it = 0; it < kRowIters; ++it) {
    const int c0 = begin + (it * 128 + t) * 8;
    if (c0 < end) store_codes8(qr + c0, v[it], inv);
  }
}

// Gated activation on one row's 32 gate and 32 up accumulators of a work item (the arithmetic of
// instinctflash/kernels/activation.py:26-43 on the bf16-rounded accumulators): h in fp32 to
// memory, the row's maximum of |h| raised in op.aux with atomicMax on the float's bits.
__device__ __forceinline__ void gated_epilogue_row(const Op& op, const uint32_t (&rg)[32], const uint32_t (&ru)[32],
                                                   int m, int n0) {
  const float rs = __ldcg(op.row_scale + m);
  float* hr = reinterpret_cast<float*>(op.out) + (int64_t)m * op.ld_out + n0;
  float row_max = 0.0f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (n0 + 8 * j >= op.N) break;  // widths are multiples of 8
    float g[8], u[8], cg[8], cu[8], h[8];
    load_f32x8(op.col_scale + n0 + 8 * j, cg);
    load_f32x8(op.col_scale + op.N + n0 + 8 * j, cu);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      g[i] = __bfloat162float(__float2bfloat16_rn(__uint_as_float(rg[8 * j + i])));
      u[i] = __bfloat162float(__float2bfloat16_rn(__uint_as_float(ru[8 * j + i])));
      g[i] = __fmul_rn(__fmul_rn(g[i], rs), cg[i]);
      u[i] = __fmul_rn(__fmul_rn(u[i], rs), cu[i]);
    }
    if (op.act == IFLB200_ACT_GELU_TANH) {
#pragma unroll
      for (int i = 0; i < 8; i += 2) {
        gelu_tanh_ref2(g[i], g[i + 1]);
        h[i] = __fmul_rn(u[i], g[i]);
        h[i + 1] = __fmul_rn(u[i + 1], g[i + 1]);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) h[i] = __fmul_rn(u[i], silu_ref(g[i]));
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) row_max = max_f32(row_max, fabsf(h[i]));
    *reinterpret_cast<float4*>(hr + 8 * j) = make_float4(h[0], h[1], h[2], h[3]);
    *reinterpret_cast<float4*>(hr + 8 * j + 4) = make_float4(h[4], h[5], h[6], h[7]);
  }
  atomicMax(reinterpret_cast<uint32_t*>(op.aux) + m, __float_as_uint(row_max));
}

template <int AROWS, int NSTAGES>
__global__ void __launch_bounds__(kThreads, 1)
stack_persistent_kernel(const Op* __restrict__ ops, int num_ops, const CUtensorMap* __restrict__ maps,
                        uint32_t* __restrict__ bars, int M, uint32_t* __restrict__ status) {
  constexpr int kASlab = AROWS * BK;  // one K slab of the activation box
  constexpr int kWSlab = BN * BK;
  constexpr int kABytes = kSlabs * kASlab;
  constexpr int kWBytes = kSlabs * kWSlab;
  constexpr int kStageBytes = kABytes + kWBytes;
  constexpr uint32_t kIdesc = make_idesc_e4m3_f32(BM, BN);
  constexpr uint32_t kTmemCols = 2 * BN;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);
  Shared* sh = reinterpret_cast<Shared*>(smem + NSTAGES * kStageBytes + ((AROWS < BM) ? (BM - AROWS) * BK : 0));
  auto full_bar = [&](int s) { return smem_u32(&sh->full[s][0]); };
  auto empty_bar = [&](int s) { return smem_u32(&sh->empty[s][0]); };
  auto tfull_bar = [&](int a) { return smem_u32(&sh->tfull[a][0]); };
  auto tempty_bar = [&](int a) { return smem_u32(&sh->tempty[a][0]); };
  volatile uint32_t* abort_flag = &sh->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int cta = blockIdx.x;
  const int ncta = gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NSTAGES; ++s) {
      mbar_init(full_bar(s), 2);   // W producer + A producer, each with its own byte count
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);
    }
    sh->abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&sh->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;

  if (warp == 0 || warp == 6) {
    // ---------------------------------------------------------------- producers
    const bool is_w = warp == 0;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int oi = 0; ok && oi < num_ops; ++oi) {
      const Op& op = ops[oi];
      if (!is_gemm(op)) continue;
      const int items = gemm_items(op);
      bool waited = is_w || op.wait_bar < 0;
      for (int item = (cta + ncta - (op.tile_offset % ncta)) % ncta; ok && item < items; item += ncta) {
        const int n_blk = item / op.split_k;
        int kb0, kb1;
        split_range(op, item % op.split_k, kb0, kb1);
        for (int kb = kb0; kb < kb1; kb += kSlabs) {
          // the A producer reaches a stage after the W producer has freed and re-armed it or
          // before; either way both wait for the stage to be empty themselves
          ok = __all_sync(0xFFFFFFFFu, wait_mbar(empty_bar(stage), phase ^ 1, abort_flag, status,
                                                 ((is_w ? 1u : 6u) << 24) | (1u << 16) | (uint32_t)oi));
          if (!ok) break;
          if (!waited) {
            // first activation load of an operator that consumes another operator's output
            if (lane == 0) TRACE(oi, 0);
            ok = __all_sync(0xFFFFFFFFu, wait_grid(bars + op.wait_bar, (uint32_t)ncta, abort_flag, status,
                                                   (6u << 24) | (5u << 16) | (uint32_t)oi));
            if (!ok) break;
            fence_proxy_async_all();  // activations were written with plain stores by other CTAs
            waited = true;
            if (lane == 0) TRACE(oi, 1);
          }
          if (lane == 0) {
            const uint32_t sa = base + stage * kStageBytes;
            if (is_w) {
              mbar_arrive_expect_tx(full_bar(stage), kWBytes);
              // kSlabs slabs from slab kb on (slabs past the end of K read as zeros; slabs past
              // the end of this item's K range are loaded and not used)
              if (op.type == OP_GEMM_GATED)  // gate rows and up rows of the item's hidden units in one box
                tma_load_4d(sa + kABytes, maps + op.tm_w, full_bar(stage), 0, n_blk * HW, 0, kb);
              else
                tma_load_3d(sa + kABytes, maps + op.tm_w, full_bar(stage), 0, n_blk * BN, kb);
            } else {
              mbar_arrive_expect_tx(full_bar(stage), kABytes);
              tma_load_3d(sa, maps + op.tm_a, full_bar(stage), 0, 0, kb);
              if (kb == kb0) TRACE(oi, 2);
              if (kb + kSlabs >= kb1) TRACE(oi, 3);
            }
          }
          __syncwarp();
          if (++stage == NSTAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
    // drain after a timeout: give loads in flight time to land before shared memory goes away
    if (!ok) {
      for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    int stage = 0;
    uint32_t phase = 0;
    uint32_t it = 0;
    bool ok = true;
    for (int oi = 0; ok && oi < num_ops; ++oi) {
      const Op& op = ops[oi];
      if (!is_gemm(op)) continue;
      const int items = gemm_items(op);
      for (int item = (cta + ncta - (op.tile_offset % ncta)) % ncta; ok && item < items; item += ncta, ++it) {
        int kb0, kb1;
        split_range(op, item % op.split_k, kb0, kb1);
        const uint32_t acc = it & 1u;
        const uint32_t acc_phase = (it >> 1) & 1u;
        ok = __all_sync(0xFFFFFFFFu, wait_mbar(tempty_bar(acc), acc_phase ^ 1, abort_flag, status,
                                               (2u << 24) | (2u << 16) | (uint32_t)oi));
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; kb += kSlabs) {
          ok = __all_sync(0xFFFFFFFFu, wait_mbar(full_bar(stage), phase, abort_flag, status,
                                                 (2u << 24) | (3u << 16) | (uint32_t)oi));
          if (!ok) break;
          tc_fence_after();
          if (lane == 0) {
            if (kb == kb0) TRACE(oi, 4);
            const uint32_t sa = base + stage * kStageBytes;
#pragma unroll
            for (int sl = 0; sl < kSlabs; ++sl) {
              if (kb + sl >= kb1) break;
              const uint64_t da = make_kmajor_sw128_desc(sa + sl * kASlab);
              const uint64_t db = make_kmajor_sw128_desc(sa + kABytes + sl * kWSlab);
#pragma unroll
              for (int j = 0; j < BK / 32; ++j)
                mma_f8f6f4(d_tmem, da + 2 * j, db + 2 * j, kIdesc, (kb + sl > kb0 || j > 0) ? 1u : 0u);
            }
            mma_commit(empty_bar(stage));
          }
          __syncwarp();
          if (++stage == NSTAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        if (lane == 0) {
          mma_commit(tfull_bar(acc));
          TRACE(oi, 5);
        }
        __syncwarp();
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue / row operators
    const int quad = warp & 3;
    const int t = (warp - 2) * 32 + lane;  // 0..127 among the epilogue threads
    uint32_t it = 0;
    bool ok = true;
    for (int oi = 0; ok && oi < num_ops; ++oi) {
      const Op& op = ops[oi];
      if (is_gemm(op)) {
        const int items = gemm_items(op);
        for (int item = (cta + ncta - (op.tile_offset % ncta)) % ncta; ok && item < items; item += ncta, ++it) {
          const int n_blk = item / op.split_k;
          const int split = item % op.split_k;  // every split has at least one K step (checked on the host)
          const uint32_t acc = it & 1u;
          const uint32_t acc_phase = (it >> 1) & 1u;
          const int m = quad * 32 + lane;
          const bool row_ok = m < M;
          ok = __all_sync(0xFFFFFFFFu, wait_mbar(tfull_bar(acc), acc_phase, abort_flag, status,
                                                 (3u << 24) | (4u << 16) | (uint32_t)oi));
          if (!ok) break;
          tc_fence_after();
          if (t == 0) TRACE(oi, 6);
          const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN;
          if (op.type == OP_GEMM_GATED) {
            uint32_t rg[32], ru[32];
            tmem_ld_32x32b_x32(t_row, rg);
            tmem_ld_32x32b_x32(t_row + HW, ru);
            tmem_ld_wait();
            if (row_ok) gated_epilogue_row(op, rg, ru, m, n_blk * HW);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
            if (t == 0) TRACE(oi, 7);
            continue;
          }
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            const int n0 = n_blk * BN + c * 32;
            if (n0 >= op.N) break;
            uint32_t r[32];
            tmem_ld_32x32b_x32(t_row + c * 32, r);
            tmem_ld_wait();
            if (!row_ok) continue;
            const int valid = min(32, op.N - n0);
            if (op.split_k > 1) {
              float* o = reinterpret_cast<float*>(op.out) + ((int64_t)split * M + m) * op.ld_out + n0;
#pragma unroll
              for (int j = 0; j < 8; ++j)
                if (4 * j < valid)
                  *reinterpret_cast<float4*>(o + 4 * j) =
                      make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                  __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
            } else {
              __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(op.out) + (int64_t)m * op.ld_out + n0;
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                if (8 * j < valid) {
                  uint4 u;
                  u.x = f32_to_bf16_bits(__uint_as_float(r[8 * j + 0])) | (f32_to_bf16_bits(__uint_as_float(r[8 * j + 1])) << 16);
                  u.y = f32_to_bf16_bits(__uint_as_float(r[8 * j + 2])) | (f32_to_bf16_bits(__uint_as_float(r[8 * j + 3])) << 16);
                  u.z = f32_to_bf16_bits(__uint_as_float(r[8 * j + 4])) | (f32_to_bf16_bits(__uint_as_float(r[8 * j + 5])) << 16);
                  u.w = f32_to_bf16_bits(__uint_as_float(r[8 * j + 6])) | (f32_to_bf16_bits(__uint_as_float(r[8 * j + 7])) << 16);
                  *reinterpret_cast<uint4*>(o + 8 * j) = u;
                }
              }
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(tempty_bar(acc));
          if (t == 0) TRACE(oi, 7);
        }
        if (!ok) break;
      } else {
        if (op.wait_bar >= 0) {
          bool got = true;
          if (t == 0) TRACE(oi, 8);
          if (t == 0) got = wait_grid(bars + op.wait_bar, (uint32_t)ncta, abort_flag, status, (3u << 24) | (5u << 16) | (uint32_t)oi);
          named_barrier_sync(1, 128);
          (void)got;
          if (*abort_flag) {
            ok = false;
            break;
          }
          (void)ld_acquire(bars + op.wait_bar);  // every thread acquires what the counter publishes
          __threadfence();
          if (t == 0) TRACE(oi, 9);
        }
        if (op.type == OP_ENCODE) {
          for (int item = cta; item < M * op.split_k; item += ncta) row_encode(op, item, t);
        } else {
          for (int m = cta; m < M; m += ncta) {
            if (op.type == OP_GATED) row_gated(op, m, t, sh->red[0]);
            else row_resnorm(op, M, m, t, sh->red);
            named_barrier_sync(1, 128);  // reduction scratch reused by the next row
          }
        }
        if (t == 0) TRACE(oi, 10);
      }
      if (op.arrive_bar >= 0) {
        fence_proxy_async_all();  // outputs may be read by other CTAs' TMA loads
        __threadfence();
        if (t == 0) TRACE(oi, 11);
        named_barrier_sync(1, 128);
        if (t == 0) atomicAdd(bars + op.arrive_bar, 1u);
        if (t == 0) TRACE(oi, 12);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace stackk
}  // namespace iflb200

using namespace iflb200;
using namespace iflb200::stackk;

namespace iflb200 {
// 0 restores the default.  Applies to the current device; synchronises it.
int set_stack_wait_budget_ns(uint64_t ns) {
  const uint64_t v = ns ? ns : kWaitBudgetNs;
  return (int)cudaMemcpyToSymbol(g_stack_wait_budget_ns, &v, sizeof(v));
}
}  // namespace iflb200

typedef CUresult (*EncodeTiledFn2)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

extern "C" int iflb200_encode_operand_map(void* out128, const void* ptr, int rows, int K, int64_t ld, int box_rows) {
  if (!out128 || !ptr || rows <= 0 || K < 16 || K % 16 || ld < K || ld % 16 || box_rows <= 0 || box_rows > 256)
    return IFLB200_ERR_ARG;
  if (reinterpret_cast<uintptr_t>(ptr) & 15) return IFLB200_ERR_ALIGN;
  static EncodeTiledFn2 fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return IFLB200_ERR_DRIVER;
    fn = reinterpret_cast<EncodeTiledFn2>(p);
  }
  if (K % BK) return IFLB200_ERR_SHAPE;  // operands are mapped as [K / 128][rows][128 bytes]
  alignas(64) CUtensorMap tm;
  const cuuint64_t dims[3] = {(cuuint64_t)BK, (cuuint64_t)rows, (cuuint64_t)(K / BK)};
  const cuuint64_t strides[2] = {(cuuint64_t)ld, (cuuint64_t)BK};
  const cuuint32_t box[3] = {(cuuint32_t)BK, (cuuint32_t)box_rows, (cuuint32_t)kSlabs};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = fn(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return IFLB200_ERR_DRIVER;
  memcpy(out128, &tm, sizeof(tm));
  return IFLB200_OK;
}

#ifdef IFLB200_TRACE
extern "C" __attribute__((visibility("default"))) int iflb200_exp_stack_trace(unsigned long long* out256) {
  return (int)cudaMemcpyFromSymbol(out256, g_stack_trace, sizeof(unsigned long long) * 256);
}
#endif

extern "C" int iflb200_encode_gated_weight_map(void* out128, const void* ptr, int F, int K, int64_t ld) {
  if (!out128 || !ptr || F <= 0 || F % 8 || K < 16 || K % 16 || ld < K || ld % 16) return IFLB200_ERR_ARG;
  if (K % BK) return IFLB200_ERR_SHAPE;
  if (reinterpret_cast<uintptr_t>(ptr) & 15) return IFLB200_ERR_ALIGN;
  void* fp = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fp, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return IFLB200_ERR_DRIVER;
  EncodeTiledFn2 fn = reinterpret_cast<EncodeTiledFn2>(fp);
  alignas(64) CUtensorMap tm;
  const cuuint64_t dims[4] = {(cuuint64_t)BK, (cuuint64_t)F, 2, (cuuint64_t)(K / BK)};
  const cuuint64_t strides[3] = {(cuuint64_t)ld, (cuuint64_t)ld * (cuuint64_t)F, (cuuint64_t)BK};
  const cuuint32_t box[4] = {(cuuint32_t)BK, (cuuint32_t)HW, 2, (cuuint32_t)kSlabs};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = fn(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return IFLB200_ERR_DRIVER;
  memcpy(out128, &tm, sizeof(tm));
  return IFLB200_OK;
}

extern "C" int iflb200_stack_activation_box_rows(int M) { return M <= A_ROWS ? A_ROWS : A_ROWS_WIDE; }
extern "C" int iflb200_stack_weight_box_rows(void) { return BN; }

extern "C" int iflb200_stack_run(const void* ops, int num_ops, const void* tensor_maps, void* barriers,
                                 int num_barriers, int M, void* status2, void* stream) {
  if (!ops || num_ops <= 0 || !tensor_maps || !barriers || num_barriers < 0 || !status2) return IFLB200_ERR_ARG;
  if (M <= 0 || M > BM) return IFLB200_ERR_SHAPE;
  if (reinterpret_cast<uintptr_t>(tensor_maps) & 63) return IFLB200_ERR_ALIGN;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  int sms = 0, major = 0, coop = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
  if (major != 10 || !coop) return IFLB200_ERR_DEVICE;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // the dependency counters and the abort word start at zero on every launch
  e = cudaMemsetAsync(barriers, 0, sizeof(uint32_t) * (size_t)num_barriers, s);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemsetAsync(reinterpret_cast<uint32_t*>(status2) + 1, 0, sizeof(uint32_t), s);
  if (e != cudaSuccess) return (int)e;
  const Op* dops = reinterpret_cast<const Op*>(ops);
  const CUtensorMap* dmaps = reinterpret_cast<const CUtensorMap*>(tensor_maps);
  uint32_t* dbars = reinterpret_cast<uint32_t*>(barriers);
  uint32_t* dstatus = reinterpret_cast<uint32_t*>(status2);
  void* args[] = {(void*)&dops, (void*)&num_ops, (void*)&dmaps, (void*)&dbars, (void*)&M, (void*)&dstatus};
  const bool narrow = M <= A_ROWS;
  const size_t smem = (narrow ? (size_t)STAGES * kSlabs * (A_ROWS * BK + BN * BK) + (BM - A_ROWS) * BK
                              : (size_t)2 * kSlabs * (A_ROWS_WIDE * BK + BN * BK)) +
                      sizeof(Shared) + 1024;
  const void* fn = narrow ? (const void*)stack_persistent_kernel<A_ROWS, STAGES>
                          : (const void*)stack_persistent_kernel<A_ROWS_WIDE, 2>;
  static bool attr_set[2][64] = {};
  if (dev < 64 && !attr_set[narrow][dev]) {
    e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr_set[narrow][dev] = true;
  }
  int per_sm = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, kThreads, smem);
  if (e != cudaSuccess) return (int)e;
  if (per_sm < 1) return IFLB200_ERR_DEVICE;
  e = cudaLaunchCooperativeKernel(fn, dim3(sms), dim3(kThreads), args, smem, s);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaGetLastError();
}
