// Row kernels of the FP8 linear path for sm_100a: the per-token e4m3 quantiser and the
// consumers of raw GEMM accumulators.  One group of TPR threads owns one row and keeps it in
// registers, so each element is read once and written once; loads are 128-bit, codes are
// stored 8 at a time.  All of them are HBM-bound: bytes per row are in the comments.
#include <cuda_runtime.h>

#include "../../include/iflb200.h"
#include "launch.cuh"
#include "rowmath.cuh"

// The file compiles as one translation unit, or as three (IFLB200_ROW_PART = 0, 1, 2) so that
// the build can run them in parallel: 0 = row_quant + dequant_rows, 1 = gated_act_quant + the
// per-tensor pack, 2 = residual_norm_quant.
#ifndef IFLB200_ROW_PART
#define IFLB200_ROW_PART -1
#endif

namespace iflb200 {

// One thread waits for the kernel before this one in the stream, the others park at the CTA
// barrier: a CTA that became resident early costs the still-running kernel next to it nothing.
__device__ __forceinline__ void row_dependency_wait() {
  if (threadIdx.x == 0) grid_dependency_wait();
  __syncthreads();
}

// Row kernels let the next kernel in the stream be scheduled as soon as their last CTAs start.
__device__ __forceinline__ void row_trigger() { grid_launch_dependents(); }

// CTAs have 256 threads.  A row is owned by a group of TPR threads, each holding IT chunks of 8
// elements: narrow rows share a CTA (TPR = 32 / 64 / 128, one chunk per thread), wide rows take
// the whole CTA with 1, 2, 4 or 8 chunks per thread (up to 16384 columns).  Measured on B200,
// 256-thread groups beat wider ones at every size: the two or three block-wide synchronisations
// per row are hidden by the other CTAs resident on the SM, not by more threads per row.
constexpr int kRowThreads = 256;
constexpr int kMaxWidth = kRowThreads * 8 * 8;  // 16384 columns

// --------------------------------------------------------------------------------------------
// Chunks of 8 elements.  FAST kernels are launched when every buffer obeys the 16-byte rule and
// the row width is a multiple of 8: every access is one or two 128-bit instructions and a chunk
// is either wholly inside the row or wholly outside, so there is no per-element masking.  The
// other instantiation is fully element-wise (any alignment, any width).
// --------------------------------------------------------------------------------------------
template <typename T>
struct Raw8 {  // eight elements as they sit in memory
  uint4 u;
};
template <>
struct Raw8<float> {
  float4 a, b;
};
template <typename T>
__device__ __forceinline__ Raw8<T> raw_zero() {
  Raw8<T> r;
  r.u = make_uint4(0u, 0u, 0u, 0u);
  return r;
}
template <>
__device__ __forceinline__ Raw8<float> raw_zero<float>() {
  Raw8<float> r;
  r.a = make_float4(0.f, 0.f, 0.f, 0.f);
  r.b = r.a;
  return r;
}
template <typename T>
__device__ __forceinline__ Raw8<T> raw_load(const T* p) {
  Raw8<T> r;
  r.u = *reinterpret_cast<const uint4*>(p);
  return r;
}
template <>
__device__ __forceinline__ Raw8<float> raw_load<float>(const float* p) {
  Raw8<float> r;
  r.a = *reinterpret_cast<const float4*>(p);
  r.b = *reinterpret_cast<const float4*>(p + 4);
  return r;
}
template <typename T>
__device__ __forceinline__ Raw8<T> raw_gather(const T* row_ptr, int c0, int width) {
  uint32_t w[4] = {0u, 0u, 0u, 0u};
  const uint16_t* p = reinterpret_cast<const uint16_t*>(row_ptr);
#pragma unroll
  for (int i = 0; i < 8; ++i)
    if (c0 + i < width) w[i >> 1] |= (uint32_t)p[c0 + i] << (16 * (i & 1));
  Raw8<T> r;
  r.u = make_uint4(w[0], w[1], w[2], w[3]);
  return r;
}
template <>
__device__ __forceinline__ Raw8<float> raw_gather<float>(const float* row_ptr, int c0, int width) {
  float f[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = (c0 + i < width) ? row_ptr[c0 + i] : 0.0f;
  Raw8<float> r;
  r.a = make_float4(f[0], f[1], f[2], f[3]);
  r.b = make_float4(f[4], f[5], f[6], f[7]);
  return r;
}
// All loads of a row are issued through this before the first value is used, so a thread has
// every chunk in flight at once.  `on`: the chunk belongs to a live row and starts inside it.
template <bool FAST, typename T>
__device__ __forceinline__ Raw8<T> fetch(const T* row_ptr, int c0, int width, bool on) {
  if (!on) return raw_zero<T>();
  if (FAST) return raw_load<T>(row_ptr + c0);
  return raw_gather<T>(row_ptr, c0, width);
}
__device__ __forceinline__ void unpack(const Raw8<__nv_bfloat16>& r, float (&o)[8]) {
  const uint32_t w[4] = {r.u.x, r.u.y, r.u.z, r.u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    o[2 * i] = __uint_as_float(w[i] << 16);
    o[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ void unpack(const Raw8<__half>& r, float (&o)[8]) {
  const uint32_t w[4] = {r.u.x, r.u.y, r.u.z, r.u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    o[2 * i] = f.x;
    o[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void unpack(const Raw8<float>& r, float (&o)[8]) {
  o[0] = r.a.x; o[1] = r.a.y; o[2] = r.a.z; o[3] = r.a.w;
  o[4] = r.b.x; o[5] = r.b.y; o[6] = r.b.z; o[7] = r.b.w;
}
// float32 vector operand (scales, bias, gates, norm weights) for one chunk.
template <bool FAST>
__device__ __forceinline__ void load_f32(const float* p, int c0, int width, float (&o)[8]) {
  if (FAST) {
    unpack(raw_load<float>(p + c0), o);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = (c0 + i < width) ? p[c0 + i] : 0.0f;
  }
}
// Zero the elements of a chunk that lie beyond the row end (element-wise kernels only).
template <bool FAST>
__device__ __forceinline__ void mask_tail(float (&v)[8], int c0, int width) {
  if (!FAST) {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = (c0 + i < width) ? v[i] : 0.0f;
  }
}
template <bool FAST>
__device__ __forceinline__ void store_codes(uint8_t* row_ptr, int c0, int width, const float (&v)[8], float inv) {
  float s[8];
  const uint64_t inv2 = pack2(inv, inv);
#pragma unroll
  for (int i = 0; i < 8; i += 2) unpack2(mul2(pack2(v[i], v[i + 1]), inv2), s[i], s[i + 1]);
  const uint32_t lo = cvt_e4m3x4(s[0], s[1], s[2], s[3]);
  const uint32_t hi = cvt_e4m3x4(s[4], s[5], s[6], s[7]);
  if (FAST) {
    *reinterpret_cast<uint2*>(row_ptr + c0) = make_uint2(lo, hi);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (c0 + i < width) row_ptr[c0 + i] = (uint8_t)(((i < 4 ? lo : hi) >> (8 * (i & 3))) & 0xFF);
  }
}
template <bool FAST>
__device__ __forceinline__ void store_out(void* base, int dtype, int64_t row_off, int c0, int width,
                                          const float (&v)[8]) {
  if (dtype == IFLB200_F32) {
    float* o = reinterpret_cast<float*>(base) + row_off + c0;
    if (FAST) {
      *reinterpret_cast<float4*>(o) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(o + 4) = make_float4(v[4], v[5], v[6], v[7]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (c0 + i < width) o[i] = v[i];
    }
    return;
  }
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    w[i] = (dtype == IFLB200_BF16) ? (f32_to_bf16_bits(v[2 * i]) | (f32_to_bf16_bits(v[2 * i + 1]) << 16))
                                   : (f32_to_f16_bits(v[2 * i]) | (f32_to_f16_bits(v[2 * i + 1]) << 16));
  uint16_t* o = reinterpret_cast<uint16_t*>(base) + row_off + c0;
  if (FAST) {
    *reinterpret_cast<uint4*>(o) = make_uint4(w[0], w[1], w[2], w[3]);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (c0 + i < width) o[i] = (uint16_t)(w[i >> 1] >> (16 * (i & 1)));
  }
}
template <typename T>
__host__ __device__ constexpr int dtype_of();
template <>
__host__ __device__ constexpr int dtype_of<float>() { return IFLB200_F32; }
template <>
__host__ __device__ constexpr int dtype_of<__nv_bfloat16>() { return IFLB200_BF16; }
template <>
__host__ __device__ constexpr int dtype_of<__half>() { return IFLB200_F16; }

// --------------------------------------------------------------------------------------------
// Reductions over the TPR threads of one row (TPR a multiple of 32; rows never share a warp).
// `slot` is a per-reduction shared array of kRowThreads/32 floats.
// --------------------------------------------------------------------------------------------
template <int TPR, bool IS_MAX>
__device__ __forceinline__ float row_reduce(float v, float* slot) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float other = __shfl_xor_sync(0xFFFFFFFFu, v, o);
    v = IS_MAX ? max_f32(v, other) : __fadd_rn(v, other);
  }
  if (TPR > 32) {
    const int warp = threadIdx.x >> 5;
    if ((threadIdx.x & 31) == 0) slot[warp] = v;
    __syncthreads();
    constexpr int WPR = TPR / 32;
    const int first = (warp / WPR) * WPR;
    float r = slot[first];
#pragma unroll
    for (int i = 1; i < WPR; ++i) r = IS_MAX ? max_f32(r, slot[first + i]) : __fadd_rn(r, slot[first + i]);
    v = r;
  }
  return v;
}

// Resident CTAs per SM the compiler must leave room for (register cap): the block-wide
// synchronisations of one row are hidden by the other CTAs on the SM.
template <int IT>
__host__ __device__ constexpr int row_min_blocks() {
  return IT <= 2 ? 3 : 2;
}
// residual_norm_quant: three CTAs per SM for up to three chunks per thread (85 registers; capping
// at 64 for a fourth CTA spills and was measured slower: 7.7 against 4.9 us at 816 x 2048).
template <int IT>
__host__ __device__ constexpr int resnorm_min_blocks() {
  return IT <= 3 ? 3 : 2;
}

// --------------------------------------------------------------------------------------------
// row_quant: 2K (bf16 in) + K (codes out) + 4 bytes per row.
// --------------------------------------------------------------------------------------------
constexpr int kMaxMirrors = 7;  // copies of a result in the buffers of the other GPUs of a group of up to eight

struct RowQuantArgs {
  const void* x;
  int64_t ld_x;
  int M, K, iters;
  const float* row;
  const float* col;
  const float* bias;
  int gelu;
  uint8_t* q;
  int64_t ld_q;
  float* qs;
  // Column-sharded rows (tensor parallel): phase 1 writes the shard's row maximum to `amax` and
  // stops; phase 2 takes the row maximum from `amax` (after an all-reduce-max over the shards)
  // instead of its own, so the codes equal those of the unsharded row.  0: one pass.  Phase 3 is
  // phase 2 that also leaves amax[m] at zero (the maxima came from a GEMM epilogue's atomicMax,
  // which needs the words to start at zero the next time).
  int phase;
  float* amax;
  // phase 1 only: further copies of the row maxima (the other GPUs' slots for this rank, peer-mapped)
  float* amax_mirror[kMaxMirrors];
  int mirrors;
};

__device__ __forceinline__ void write_row_max(const RowQuantArgs& a, int m, float amax) {
  a.amax[m] = amax;
#pragma unroll
  for (int k = 0; k < kMaxMirrors; ++k)
    if (k < a.mirrors) a.amax_mirror[k][m] = amax;
}

// PLAIN: no prologue.  The row then stays in registers as loaded (4 registers per 8 elements)
// and is widened twice, once for the maximum and once for the cast, which keeps enough CTAs
// resident to cover the HBM latency.
template <typename XT, int TPR, int IT, bool PLAIN, bool FAST>
__global__ void __launch_bounds__(kRowThreads, PLAIN ? (IT <= 2 ? 4 : 3) : row_min_blocks<IT>())
row_quant_kernel(const RowQuantArgs a) {
  row_dependency_wait();  // inputs may come from the kernel before this one in the stream
  row_trigger();
  __shared__ float red[kRowThreads / 32];
  const int t = threadIdx.x % TPR;
  const int m = blockIdx.x * (kRowThreads / TPR) + threadIdx.x / TPR;
  const bool live = m < a.M;
  const XT* xr = reinterpret_cast<const XT*>(a.x) + (live ? (int64_t)m * a.ld_x : 0);
  const float rs = (live && a.row) ? a.row[m] : 1.0f;

  Raw8<XT> raw[IT];
#pragma unroll
  for (int it = 0; it < IT; ++it) {
    const int c0 = (it * TPR + t) * 8;
    raw[it] = fetch<FAST, XT>(xr, c0, a.K, it < a.iters && live && c0 < a.K);
  }
  float amax = 0.0f;
  if (PLAIN) {
#pragma unroll
    for (int it = 0; it < IT; ++it) {
      float w[8];
      unpack(raw[it], w);
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = max_f32(amax, fabsf(w[i]));
    }
    amax = row_reduce<TPR, true>(amax, red);
    if (a.phase == 1) {
      if (live && t == 0) write_row_max(a, m, amax);
      return;
    }
    if (a.phase >= 2 && live) amax = a.amax[m];
    if (a.phase == 3) {  // every thread of the row has its copy: leave the word at zero for the next producer
      __syncthreads();
      if (live && t == 0) a.amax[m] = 0.0f;
    }
    float scale, inv;
    quant_scales(amax, scale, inv);
    if (!live) return;
    if (t == 0) a.qs[m] = scale;
    uint8_t* qr = a.q + (int64_t)m * a.ld_q;
#pragma unroll
    for (int it = 0; it < IT; ++it) {
      const int c0 = (it * TPR + t) * 8;
      if (it < a.iters && c0 < a.K) {
        float w[8];
        unpack(raw[it], w);
        store_codes<FAST>(qr, c0, a.K, w, inv);
      }
    }
    return;
  }
  float v[IT][8];
#pragma unroll
  for (int it = 0; it < IT; ++it) {
    const int c0 = (it * TPR + t) * 8;
    unpack(raw[it], v[it]);
    if (it < a.iters && live && c0 < a.K) {
      float cs[8], bs[8];
      if (a.col) load_f32<FAST>(a.col, c0, a.K, cs);
      if (a.bias) load_f32<FAST>(a.bias, c0, a.K, bs);
      Chain8 ch(v[it]);
      if (a.row) ch.mul(rs);
      if (a.col) ch.mul(cs);
      if (a.bias) ch.add(bs);
      ch.done(v[it]);
      if (a.gelu) {
#pragma unroll
        for (int i = 0; i < 8; i += 2) gelu_tanh_ref2(v[it][i], v[it][i + 1]);
      }
      mask_tail<FAST>(v[it], c0, a.K);
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = max_f32(amax, fabsf(v[it][i]));
    }
  }
  amax = row_reduce<TPR, true>(amax, red);
  if (a.phase == 1) {
    if (live && t == 0) write_row_max(a, m, amax);
    return;
  }
  if (a.phase >= 2 && live) amax = a.amax[m];
  if (a.phase == 3) {
    __syncthreads();
    if (live && t == 0) a.amax[m] = 0.0f;
  }
  float scale, inv;
  quant_scales(amax, scale, inv);
  if (!live) return;
  if (t == 0) a.qs[m] = scale;
  uint8_t* qr = a.q + (int64_t)m * a.ld_q;
#pragma unroll
  for (int it = 0; it < IT; ++it) {
    const int c0 = (it * TPR + t) * 8;
    if (it < a.iters && c0 < a.K) store_codes<FAST>(qr, c0, a.K, v[it], inv);
  }
}

// --------------------------------------------------------------------------------------------
// gated_act_quant: 4F (bf16 g,u in) + F (codes out) + 4 bytes per row.  Bound by instruction
// issue, not by HBM: ~40 instructions per element (the reference's ex2.approx / div.full chains).
// --------------------------------------------------------------------------------------------
struct GatedArgs {
  const void* gu;
  int64_t ld_gu;
  int M, F, iters;
  const float* row;
  const float* col;
  int act;
  uint8_t* q;
  int64_t ld_q;
  float* qs;
};

template <typename XT, int TPR, int IT, bool FAST>
__global__ void __launch_bounds__(kRowThreads, row_min_blocks<IT>())
gated_act_quant_kernel(const GatedArgs a) {
  row_dependency_wait();  // inputs may come from the kernel before this one in the stream
  row_trigger();
  __shared__ float red[kRowThreads / 32];
  const int t = threadIdx.x % TPR;
  const int m = blockIdx.x * (kRowThreads / TPR) + threadIdx.x / TPR;
  const bool live = m < a.M;
  const XT* gr = reinterpret_cast<const XT*>(a.gu) + (live ? (int64_t)m * a.ld_gu : 0);
  const XT* ur = gr + a.F;
  const float rs = (live && a.row) ? a.row[m] : 1.0f;

  Raw8<XT> rg[IT], ru[IT];
#pragma unroll
  for (int it = 0; it < IT; ++it) {
    const int c0 = (it * TPR + t) * 8;
    const bool on = it < a.iters && live && c0 < a.F;
    rg[it] = fetch<FAST, XT>(gr, c0, a.F, on);
    ru[it] = fetch<FAST, XT>(ur, c0, a.F, on);
  }
  float h[IT][8];
  float amax = 0.0f;
#pragma unroll
  for (int it = 0; it < IT; ++it) {
    const int c0 = (it * TPR + t) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) h[it][i] = 0.0f;
    if (it < a.iters && live && c0 < a.F) {
      float g[8], u[8];
      unpack(rg[it], g);
      unpack(ru[it], u);
      if (a.row) {
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
          const uint64_t rs2 = pack2(rs, rs);
          unpack2(mul2(pack2(g[i], g[i + 1]), rs2), g[i], g[i + 1]);
          unpack2(mul2(pack2(u[i], u[i + 1]), rs2), u[i], u[i + 1]);
        }
      }
      if (a.col) {
        float cg[8], cu[8];
        load_f32<FAST>(a.col, c0, a.F, cg);
        load_f32<FAST>(a.col + a.F, c0, a.F, cu);
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
          unpack2(mul2(pack2(g[i], g[i + 1]), pack2(cg[i], cg[i + 1])), g[i], g[i + 1]);
          unpack2(mul2(pack2(u[i], u[i + 1]), pack2(cu[i], cu[i + 1])), u[i], u[i + 1]);
        }
      }
      if (a.act == IFLB200_ACT_GELU_TANH) {
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
          gelu_tanh_ref2(g[i], g[i + 1]);
          unpack2(mul2(pack2(u[i], u[i + 1]), pack2(g[i], g[i + 1])), h[it][i], h[it][i + 1]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) h[it][i] = __fmul_rn(u[i], silu_ref(g[i]));
      }
      mask_tail<FAST>(h[it], c0, a.F);
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = max_f32(amax, fabsf(h[it][i]));
    }
  }
  amax = row_reduce<TPR, true>(amax, red);
  float scale, inv;
  quant_scales(amax, scale, inv);
  if (!live) return;
  if (t == 0) a.qs[m] = scale;
  uint8_t* qr = a.q + (int64_t)m * a.ld_q;
#pragma unroll
  for (int it = 0; it < IT; ++it) {
    const int c0 = (it * TPR + t) * 8;
    if (it < a.iters && c0 < a.F) store_codes<FAST>(qr, c0, a.F, h[it], inv);
  }
}

// --------------------------------------------------------------------------------------------
// dequant_rows: 2D in + out bytes per row; flat, one chunk per thread.
// --------------------------------------------------------------------------------------------
struct DequantArgs {
  const void* x;
  int64_t ld_x;
  int M, D;
  const float* row;
  const float* col;
  const float* bias;
  void* y;
  int y_dtype;
  int64_t ld_y;
};

template <typename XT, bool FAST>
__global__ void __launch_bounds__(256) dequant_rows_kernel(const DequantArgs a) {
  row_dependency_wait();  // inputs may come from the kernel before this one in the stream
  row_trigger();
  const int m = blockIdx.y;
  const int c0 = (blockIdx.x * 256 + threadIdx.x) * 8;
  if (c0 >= a.D) return;
  const XT* xr = reinterpret_cast<const XT*>(a.x) + (int64_t)m * a.ld_x;
  float v[8], cs[8], bs[8];
  unpack(fetch<FAST, XT>(xr, c0, a.D, true), v);
  if (a.col) load_f32<FAST>(a.col, c0, a.D, cs);
  if (a.bias) load_f32<FAST>(a.bias, c0, a.D, bs);
  const float rs = a.row ? a.row[m] : 1.0f;
  Chain8 ch(v);
  if (a.row) ch.mul(rs);
  if (a.col) ch.mul(cs);
  if (a.bias) ch.add(bs);
  ch.done(v);
  store_out<FAST>(a.y, a.y_dtype, (int64_t)m * a.ld_y, c0, a.D, v);
}

// --------------------------------------------------------------------------------------------
// residual_norm_quant: (f32 residual) 2D delta + 4D res in, 4D res + D codes out, + 4 bytes.
// --------------------------------------------------------------------------------------------
struct ResNormArgs {
  void* res;
  int64_t ld_res;
  int M, D, iters;
  const __nv_bfloat16* delta;
  int64_t ld_delta;
  // the delta as fp32 partial sums of a K-split GEMM, [dsplits][M][ld_delta] (delta is null then): summed in
  // split order and rounded to bf16, the raw accumulator's rounding point
  const float* dpart;
  int dsplits;
  const float* drow;
  const float* dcol;
  const float* bias;
  const float* gate;
  int write_res;
  int layernorm;
  const float* weight;
  const float* beta;
  const float* mod_scale;
  const float* mod_shift;
  const int32_t* mod_index;
  float eps;
  uint8_t* q;
  int64_t ld_q;
  float* qs;
  void* y;
  int y_dtype;
  int64_t ld_y;
  // partial-sum form only: further copies of the codes and row scales (same row stride as q), the
  // other GPUs' replicas of the next block's input, written from the same registers
  uint8_t* q_mirror[kMaxMirrors];
  float* qs_mirror[kMaxMirrors];
  int mirrors;
};

template <typename RT>
__device__ __forceinline__ float round_through(float x);
template <>
__device__ __forceinline__ float round_through<float>(float x) { return x; }
template <>
__device__ __forceinline__ float round_through<__nv_bfloat16>(float x) {
  return __bfloat162float(__float2bfloat16_rn(x));
}

// PART: the delta arrives as fp32 partial sums of a K-split GEMM (a.dpart) instead of a raw bf16
// accumulator; a separate instantiation so that the ordinary one keeps its registers.
template <typename RT, int TPR, int IT, bool FAST, bool PART = false>
__global__ void __launch_bounds__(kRowThreads, PART ? 2 : resnorm_min_blocks<IT>())
residual_norm_quant_kernel(const ResNormArgs a) {
  row_dependency_wait();  // inputs may come from the kernel before this one in the stream
  row_trigger();
  __shared__ float red[3][kRowThreads / 32];
  const int t = threadIdx.x % TPR;
  const int m = blockIdx.x * (kRowThreads / TPR) + threadIdx.x / TPR;
  const bool live = m < a.M;
  RT* rr = reinterpret_cast<RT*>(a.res) + (live ? (int64_t)m * a.ld_res : 0);
  const __nv_bfloat16* dr = a.delta ? a.delta + (live ? (int64_t)m * a.ld_delta : 0) : nullptr;
  const float* dp = PART ? a.dpart + (live ? (int64_t)m * a.ld_delta : 0) : nullptr;
  const int64_t dp_plane = (int64_t)a.M * a.ld_delta;
  const int64_t mofs = (live && a.mod_index) ? (int64_t)a.mod_index[m] * a.D : 0;
  const float drs = (live && a.drow) ? a.drow[m] : 1.0f;
  const float fD = (float)a.D;

  Raw8<RT> rres[IT];
  Raw8<__nv_bfloat16> rdel[IT];
#pragma unroll
  for (int it = 0; it < IT; ++it) {
    const int c0 = (it * TPR + t) * 8;
    const bool on = it < a.iters && live && c0 < a.D;
    rres[it] = fetch<FAST, RT>(rr, c0, a.D, on);
    rdel[it] = fetch<FAST, __nv_bfloat16>(dr, c0, a.D, on && dr != nullptr && !PART);
  }
  float x[IT][8];
  float sum = 0.0f, sumsq = 0.0f;
#pragma unroll
  for (int it = 0; it < IT; ++it) {
    const int c0 = (it * TPR + t) * 8;
    unpack(rres[it], x[it]);
    if (it < a.iters && live && c0 < a.D) {
      if (dr || PART) {
        float d[8], cs[8], bs[8], gs[8];
        if constexpr (PART) {
          // kGroup planes in flight together (all eight for rows of one chunk per thread: the skinny
          // expert shapes, where a second dependent round trip is a tenth of the kernel), added in split order
          constexpr int kGroup = IT == 1 ? 8 : 4;
#pragma unroll
          for (int i = 0; i < 8; ++i) d[i] = 0.0f;
#pragma unroll 1
          for (int s0 = 0; s0 < a.dsplits; s0 += kGroup) {
            float e[kGroup][8];
#pragma unroll
            for (int sp = 0; sp < kGroup; ++sp)
              if (s0 + sp < a.dsplits) load_f32<FAST>(dp + (s0 + sp) * dp_plane, c0, a.D, e[sp]);
#pragma unroll
            for (int sp = 0; sp < kGroup; ++sp) {
              if (s0 + sp < a.dsplits) {
#pragma unroll
                for (int i = 0; i < 8; ++i) d[i] = (s0 + sp == 0) ? e[sp][i] : __fadd_rn(d[i], e[sp][i]);
              }
            }
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) d[i] = __bfloat162float(__float2bfloat16_rn(d[i]));
        } else {
          unpack(rdel[it], d);
        }
        if (a.dcol) load_f32<FAST>(a.dcol, c0, a.D, cs);
        if (a.bias) load_f32<FAST>(a.bias, c0, a.D, bs);
        if (a.gate) load_f32<FAST>(a.gate + mofs, c0, a.D, gs);
        Chain8 ch(d);
        if (a.drow) ch.mul(drs);
        if (a.dcol) ch.mul(cs);
        if (a.bias) ch.add(bs);
        if (a.gate) ch.mul(gs);
        ch.add(x[it]);  // x + d, contracted with d's last multiply when there is one
        ch.done(x[it]);
        if (a.write_res) {
#pragma unroll
          for (int i = 0; i < 8; ++i) x[it][i] = round_through<RT>(x[it][i]);
        }
        mask_tail<FAST>(x[it], c0, a.D);
        if (a.write_res) store_out<FAST>(a.res, dtype_of<RT>(), (int64_t)m * a.ld_res, c0, a.D, x[it]);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        sum = __fadd_rn(sum, x[it][i]);
        sumsq = __fmaf_rn(x[it][i], x[it][i], sumsq);
      }
    }
  }
  if (a.q == nullptr && a.y == nullptr) return;  // residual update only (uniform across the CTA)

  float rstd;
  if (a.layernorm) {
    const float mean = div_full(row_reduce<TPR, false>(sum, red[0]), fD);
    float sq = 0.0f;
#pragma unroll
    for (int it = 0; it < IT; ++it) {
      const int c0 = (it * TPR + t) * 8;
      if (it < a.iters && live && c0 < a.D) {
#pragma unroll
        for (int i = 0; i < 8; i += 2)  // x - mean == x + (-mean), two lanes per instruction
          unpack2(add2(pack2(x[it][i], x[it][i + 1]), pack2(-mean, -mean)), x[it][i], x[it][i + 1]);
        mask_tail<FAST>(x[it], c0, a.D);
#pragma unroll
        for (int i = 0; i < 8; ++i) sq = __fmaf_rn(x[it][i], x[it][i], sq);
      }
    }
    const float var = div_full(row_reduce<TPR, false>(sq, red[1]), fD);
    rstd = rsqrt_approx_ftz(__fadd_rn(var, a.eps));
  } else {
    const float var = div_full(row_reduce<TPR, false>(sumsq, red[1]), fD);
    rstd = rsqrt_approx_ftz(__fadd_rn(var, a.eps));
  }

  float amax = 0.0f;
#pragma unroll
  for (int it = 0; it < IT; ++it) {
    const int c0 = (it * TPR + t) * 8;
    if (it < a.iters && live && c0 < a.D) {
      float ws[8], bs[8], ms[8], mh[8];
      if (a.weight) load_f32<FAST>(a.weight, c0, a.D, ws);
      if (a.beta) load_f32<FAST>(a.beta, c0, a.D, bs);
      if (a.mod_scale) {
        load_f32<FAST>(a.mod_scale + mofs, c0, a.D, ms);
        load_f32<FAST>(a.mod_shift + mofs, c0, a.D, mh);
      }
      Chain8 ch(x[it]);
      ch.mul(rstd);
      if (a.weight) ch.mul(ws);
      if (a.beta) ch.add(bs);
      if (a.mod_scale) {
#pragma unroll
        for (int i = 0; i < 8; i += 2) unpack2(add2(pack2(ms[i], ms[i + 1]), pack2(1.0f, 1.0f)), ms[i], ms[i + 1]);
        ch.mul(ms);
        ch.add(mh);
      }
      ch.done(x[it]);
      mask_tail<FAST>(x[it], c0, a.D);
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = max_f32(amax, fabsf(x[it][i]));
      if (a.y) store_out<FAST>(a.y, a.y_dtype, (int64_t)m * a.ld_y, c0, a.D, x[it]);
    }
  }
  if (a.q == nullptr) return;
  amax = row_reduce<TPR, true>(amax, red[2]);
  float scale, inv;
  quant_scales(amax, scale, inv);
  if (!live) return;
  if (t == 0) a.qs[m] = scale;
  uint8_t* qr = a.q + (int64_t)m * a.ld_q;
#pragma unroll
  for (int it = 0; it < IT; ++it) {
    const int c0 = (it * TPR + t) * 8;
    if (it < a.iters && c0 < a.D) store_codes<FAST>(qr, c0, a.D, x[it], inv);
  }
  if constexpr (PART) {
#pragma unroll
    for (int k = 0; k < kMaxMirrors; ++k) {
      if (k < a.mirrors) {
        if (t == 0) a.qs_mirror[k][m] = scale;
        uint8_t* qm = a.q_mirror[k] + (int64_t)m * a.ld_q;
#pragma unroll
        for (int it = 0; it < IT; ++it) {
          const int c0 = (it * TPR + t) * 8;
          if (it < a.iters && c0 < a.D) store_codes<FAST>(qm, c0, a.D, x[it], inv);
        }
      }
    }
  }
}

#if IFLB200_ROW_PART == 1 || IFLB200_ROW_PART == -1
// --------------------------------------------------------------------------------------------
// Per-tensor pack (the torch-FP8-linear recipe)
// --------------------------------------------------------------------------------------------
constexpr int kPackThreads = 256;
constexpr int kPackMaxCtas = 1024;

// Maximum of |x| as an integer maximum of the bf16 magnitude bits: finite values order like
// their bits, and every NaN pattern is larger than infinity, so NaN propagates.
__global__ void __launch_bounds__(kPackThreads)
amax_partial_kernel(const uint16_t* __restrict__ x, int64_t n, uint32_t* __restrict__ partial) {
  row_dependency_wait();  // inputs may come from the kernel before this one in the stream
  row_trigger();
  __shared__ uint32_t red[kPackThreads / 32];
  uint32_t best = 0;
  const int64_t nvec = n / 8;
  const bool vec = (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  const int64_t stride = (int64_t)gridDim.x * kPackThreads;
  if (vec) {
    const uint4* xv = reinterpret_cast<const uint4*>(x);
    for (int64_t i = (int64_t)blockIdx.x * kPackThreads + threadIdx.x; i < nvec; i += stride) {
      const uint4 u = xv[i];
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        best = max(best, w[k] & 0x7FFFu);
        best = max(best, (w[k] >> 16) & 0x7FFFu);
      }
    }
    for (int64_t i = nvec * 8 + (int64_t)blockIdx.x * kPackThreads + threadIdx.x; i < n; i += stride)
      best = max(best, (uint32_t)x[i] & 0x7FFFu);
  } else {
    for (int64_t i = (int64_t)blockIdx.x * kPackThreads + threadIdx.x; i < n; i += stride)
      best = max(best, (uint32_t)x[i] & 0x7FFFu);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xFFFFFFFFu, best, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < kPackThreads / 32; ++i) best = max(best, red[i]);
    partial[blockIdx.x] = best;
  }
}

__device__ __forceinline__ float pack_one(float x, float scale) {
  const float d = __fdiv_rn(x, scale);
  return (d != d) ? d : fminf(fmaxf(d, -448.0f), 448.0f);
}

// n_partial > 0: dynamic scale from the partial maxima (every CTA recomputes it; CTA 0 writes
// it out).  n_partial == 0: fixed scale read from scale_in.
__global__ void __launch_bounds__(kPackThreads)
pack_kernel(const uint16_t* __restrict__ x, int64_t n, const uint32_t* __restrict__ partial,
            int n_partial, const float* __restrict__ scale_in, float* __restrict__ scale_out,
            uint8_t* __restrict__ q) {
  row_dependency_wait();  // inputs may come from the kernel before this one in the stream
  row_trigger();
  __shared__ uint32_t red[kPackThreads / 32];
  __shared__ float s_scale;
  if (n_partial > 0) {
    uint32_t best = 0;
    for (int i = threadIdx.x; i < n_partial; i += kPackThreads) best = max(best, partial[i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xFFFFFFFFu, best, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int i = 1; i < kPackThreads / 32; ++i) best = max(best, red[i]);
      float sc;
      if (best > 0x7F80u) {
        sc = __uint_as_float(0x7FC00000u);
      } else {
        const float amax = __uint_as_float(best << 16);
        sc = __fmul_rn(fmaxf(amax, 1e-12f), (float)(1.0 / 448.0));
      }
      s_scale = sc;
      if (blockIdx.x == 0) *scale_out = sc;
    }
    __syncthreads();
  } else {
    if (threadIdx.x == 0) s_scale = *scale_in;
    __syncthreads();
  }
  const float scale = s_scale;
  const bool vec = ((reinterpret_cast<uintptr_t>(x) & 15) == 0) && ((reinterpret_cast<uintptr_t>(q) & 7) == 0);
  const int64_t stride = (int64_t)gridDim.x * kPackThreads;
  const int64_t nvec = vec ? n / 8 : 0;
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  for (int64_t i = (int64_t)blockIdx.x * kPackThreads + threadIdx.x; i < nvec; i += stride) {
    const uint4 u = xv[i];
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
    float f[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      f[2 * k] = pack_one(__uint_as_float(w[k] << 16), scale);
      f[2 * k + 1] = pack_one(__uint_as_float(w[k] & 0xFFFF0000u), scale);
    }
    reinterpret_cast<uint2*>(q)[i] =
        make_uint2(cvt_e4m3x4(f[0], f[1], f[2], f[3]), cvt_e4m3x4(f[4], f[5], f[6], f[7]));
  }
  for (int64_t i = nvec * 8 + (int64_t)blockIdx.x * kPackThreads + threadIdx.x; i < n; i += stride)
    q[i] = (uint8_t)(cvt_e4m3x2(pack_one(__uint_as_float((uint32_t)x[i] << 16), scale), 0.0f) & 0xFF);
}

#endif  // pack kernels

// --------------------------------------------------------------------------------------------
// Host side: geometry selection and launches
// --------------------------------------------------------------------------------------------
static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
static inline bool aligned8(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 7) == 0; }
static inline int esize(int dtype) { return dtype == IFLB200_F32 ? 4 : 2; }
static inline bool dtype_ok(int d) { return d == IFLB200_F32 || d == IFLB200_BF16 || d == IFLB200_F16; }

// Geometry of a row kernel: threads per row and chunks per thread (see kRowThreads above).
struct RowGeom {
  int tpr;
  int iters;
};
// experiments: force the group size (0 = choose); one definition shared by the three units
#if IFLB200_ROW_PART == 0 || IFLB200_ROW_PART == -1
int g_row_tpr_override = 0;
#else
extern int g_row_tpr_override;
#endif

static RowGeom pick_geom(int width) {
  const int chunks = (width + 7) / 8;
  int tpr = 32;
  while (tpr < kRowThreads && tpr < chunks) tpr *= 2;
  if (g_row_tpr_override && (chunks + g_row_tpr_override - 1) / g_row_tpr_override <= 8) tpr = g_row_tpr_override;
  RowGeom g;
  g.tpr = tpr;
  g.iters = (chunks + tpr - 1) / tpr;
  return g;
}

// Calls `launch(tpr_tag, it_tag)` with compile-time tags for the geometry: groups narrower than
// the CTA always hold one chunk per thread; full-CTA groups hold 1, 2, 4 or 8.
template <int V>
struct IntTag {
  static constexpr int value = V;
};
template <typename F>
static void dispatch_geom(const RowGeom& g, F&& launch) {
  if (g.iters <= 1) {
    switch (g.tpr) {
      case 32: launch(IntTag<32>{}, IntTag<1>{}); return;
      case 64: launch(IntTag<64>{}, IntTag<1>{}); return;
      case 128: launch(IntTag<128>{}, IntTag<1>{}); return;
      default: launch(IntTag<256>{}, IntTag<1>{}); return;
    }
  }
  switch (g.tpr) {  // forced narrow groups with several chunks (experiments): deepest variant
    case 32: launch(IntTag<32>{}, IntTag<8>{}); return;
    case 64: launch(IntTag<64>{}, IntTag<8>{}); return;
    case 128:
      if (g.iters <= 2) launch(IntTag<128>{}, IntTag<2>{});
      else if (g.iters == 3) launch(IntTag<128>{}, IntTag<3>{});
      else if (g.iters <= 4) launch(IntTag<128>{}, IntTag<4>{});
      else launch(IntTag<128>{}, IntTag<8>{});
      return;
    default: break;
  }
  if (g.iters <= 2) launch(IntTag<256>{}, IntTag<2>{});
  else if (g.iters == 3) launch(IntTag<256>{}, IntTag<3>{});
  else if (g.iters <= 4) launch(IntTag<256>{}, IntTag<4>{});
  else launch(IntTag<256>{}, IntTag<8>{});
}

// The element-wise (any alignment) kernels exist in one geometry only: a full-CTA group with up
// to 8 chunks per thread.
static RowGeom slow_geom(int width) {
  RowGeom g;
  g.tpr = kRowThreads;
  g.iters = ((width + 7) / 8 + kRowThreads - 1) / kRowThreads;
  return g;
}

template <typename XT>
static void launch_row_quant(RowQuantArgs a, bool fast, cudaStream_t s) {
  const bool plain = !(a.row || a.col || a.bias || a.gelu);
  if (!fast) {
    a.iters = slow_geom(a.K).iters;
    if (plain) launch_dep(row_quant_kernel<XT, kRowThreads, 8, true, false>, dim3(a.M), dim3(kRowThreads), 0, s, 1, dependent_launch_for(a.M), a);
    else launch_dep(row_quant_kernel<XT, kRowThreads, 8, false, false>, dim3(a.M), dim3(kRowThreads), 0, s, 1, dependent_launch_for(a.M), a);
    return;
  }
  const RowGeom g = pick_geom(a.K);
  a.iters = g.iters;
  dispatch_geom(g, [&](auto tpr, auto it) {
    constexpr int TPR = decltype(tpr)::value, IT = decltype(it)::value;
    const int grid = (a.M + kRowThreads / TPR - 1) / (kRowThreads / TPR);
    if (plain) launch_dep(row_quant_kernel<XT, TPR, IT, true, true>, dim3(grid), dim3(kRowThreads), 0, s, 1, dependent_launch_for(a.M), a);
    else launch_dep(row_quant_kernel<XT, TPR, IT, false, true>, dim3(grid), dim3(kRowThreads), 0, s, 1, dependent_launch_for(a.M), a);
  });
}
template <typename XT>
static void launch_gated(GatedArgs a, bool fast, cudaStream_t s) {
  if (!fast) {
    a.iters = slow_geom(a.F).iters;
    launch_dep(gated_act_quant_kernel<XT, kRowThreads, 8, false>, dim3(a.M), dim3(kRowThreads), 0, s, 1, dependent_launch_for(a.M), a);
    return;
  }
  const RowGeom g = pick_geom(a.F);
  a.iters = g.iters;
  dispatch_geom(g, [&](auto tpr, auto it) {
    constexpr int TPR = decltype(tpr)::value, IT = decltype(it)::value;
    const int grid = (a.M + kRowThreads / TPR - 1) / (kRowThreads / TPR);
    launch_dep(gated_act_quant_kernel<XT, TPR, IT, true>, dim3(grid), dim3(kRowThreads), 0, s, 1, dependent_launch_for(a.M), a);
  });
}
// The partial-sum form: rows of at most 8192 columns on the aligned path.
template <typename RT>
static int launch_resnorm_partials(ResNormArgs a, bool fast, cudaStream_t s) {
  if (!fast || a.D > 8192) return IFLB200_ERR_SHAPE;
  if (a.D <= 1024) {
    a.iters = 1;
    launch_dep(residual_norm_quant_kernel<RT, 128, 1, true, true>, dim3((a.M + 1) / 2), dim3(kRowThreads), 0, s, 1,
               dependent_launch_for(a.M), a);
  } else if (a.D <= 2048) {
    a.iters = 1;
    launch_dep(residual_norm_quant_kernel<RT, kRowThreads, 1, true, true>, dim3(a.M), dim3(kRowThreads), 0, s, 1,
               dependent_launch_for(a.M), a);
  } else if (a.D <= 3072) {  // 128 threads x 3 chunks use every chunk slot; two rows per CTA
    a.iters = 3;
    launch_dep(residual_norm_quant_kernel<RT, 128, 3, true, true>, dim3((a.M + 1) / 2), dim3(kRowThreads), 0, s, 1,
               dependent_launch_for(a.M), a);
  } else if (a.D <= 4096) {
    a.iters = 2;
    launch_dep(residual_norm_quant_kernel<RT, kRowThreads, 2, true, true>, dim3(a.M), dim3(kRowThreads), 0, s, 1,
               dependent_launch_for(a.M), a);
  } else if (a.D <= 6144) {
    a.iters = 3;
    launch_dep(residual_norm_quant_kernel<RT, kRowThreads, 3, true, true>, dim3(a.M), dim3(kRowThreads), 0, s, 1,
               dependent_launch_for(a.M), a);
  } else {
    a.iters = 4;
    launch_dep(residual_norm_quant_kernel<RT, kRowThreads, 4, true, true>, dim3(a.M), dim3(kRowThreads), 0, s, 1,
               dependent_launch_for(a.M), a);
  }
  return IFLB200_OK;
}

template <typename RT>
static void launch_resnorm(ResNormArgs a, bool fast, cudaStream_t s) {
  if (!fast) {
    a.iters = slow_geom(a.D).iters;
    launch_dep(residual_norm_quant_kernel<RT, kRowThreads, 8, false>, dim3(a.M), dim3(kRowThreads), 0, s, 1, dependent_launch_for(a.M), a);
    return;
  }
  RowGeom g = pick_geom(a.D);
  // 1025..2048 columns: two rows per CTA, two chunks per thread (measured at 816 x 2048 with an
  // f32 residual: 4.9 us against 5.7 us with one row per CTA; the reference's kernel 4.4 us)
  if (g.tpr == kRowThreads && g.iters == 1 && g_row_tpr_override == 0) {
    g.tpr = 128;
    g.iters = 2;
  }
  // 2049..3072 columns: 128 threads x 3 chunks use every chunk slot (256 x 2 leaves a quarter empty)
  const int chunks = (a.D + 7) / 8;
  if (g.tpr == kRowThreads && g.iters == 2 && chunks <= 384 && g_row_tpr_override == 0) {
    g.tpr = 128;
    g.iters = 3;
  }
  a.iters = g.iters;
  dispatch_geom(g, [&](auto tpr, auto it) {
    constexpr int TPR = decltype(tpr)::value, IT = decltype(it)::value;
    const int grid = (a.M + kRowThreads / TPR - 1) / (kRowThreads / TPR);
    launch_dep(residual_norm_quant_kernel<RT, TPR, IT, true>, dim3(grid), dim3(kRowThreads), 0, s, 1, dependent_launch_for(a.M), a);
  });
}

}  // namespace iflb200

using namespace iflb200;

#if IFLB200_ROW_PART == 0 || IFLB200_ROW_PART == -1
extern "C" int iflb200_row_set_group(int threads_per_row) {
  if (threads_per_row != 0 && (threads_per_row < 32 || threads_per_row > kRowThreads ||
                               (threads_per_row & (threads_per_row - 1))))
    return IFLB200_ERR_ARG;
  iflb200::g_row_tpr_override = threads_per_row;
  return IFLB200_OK;
}

static int row_quant_impl(const void* x, int x_dtype, int64_t ld_x, int M, int K, const float* row,
                          const float* col, const float* bias, int gelu, void* q, int64_t ld_q, float* qs,
                          int phase, float* amax, void* stream, float* const* amax_mirrors = nullptr,
                          int mirrors = 0) {
  if (M < 0 || K < 0) return IFLB200_ERR_ARG;
  if (mirrors < 0 || mirrors > kMaxMirrors || (mirrors > 0 && (!amax_mirrors || phase != 1))) return IFLB200_ERR_ARG;
  if (M == 0 || K == 0) return IFLB200_OK;
  if (!x) return IFLB200_ERR_ARG;
  if (phase != 1 && (!q || !qs)) return IFLB200_ERR_ARG;
  if (phase != 0 && !amax) return IFLB200_ERR_ARG;
  if (!dtype_ok(x_dtype)) return IFLB200_ERR_DTYPE;
  if (K > kMaxWidth) return IFLB200_ERR_SHAPE;
  if (ld_x < K || (phase != 1 && ld_q < K)) return IFLB200_ERR_ARG;
  RowQuantArgs a;
  a.x = x; a.ld_x = ld_x; a.M = M; a.K = K;
  a.row = row; a.col = col; a.bias = bias; a.gelu = gelu;
  a.q = reinterpret_cast<uint8_t*>(q); a.ld_q = ld_q; a.qs = qs;
  a.phase = phase; a.amax = amax;
  a.mirrors = mirrors;
  for (int k = 0; k < kMaxMirrors; ++k) {
    a.amax_mirror[k] = k < mirrors ? amax_mirrors[k] : nullptr;
    if (k < mirrors && !a.amax_mirror[k]) return IFLB200_ERR_ARG;
  }
  const bool fast = K % 8 == 0 && aligned16(x) && (ld_x * esize(x_dtype)) % 16 == 0 &&
                    (phase == 1 || (aligned8(q) && ld_q % 8 == 0)) && (!col || aligned16(col)) &&
                    (!bias || aligned16(bias));
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (x_dtype == IFLB200_BF16) launch_row_quant<__nv_bfloat16>(a, fast, s);
  else if (x_dtype == IFLB200_F16) launch_row_quant<__half>(a, fast, s);
  else launch_row_quant<float>(a, fast, s);
  return (int)cudaGetLastError();
}

extern "C" int iflb200_row_quant(const void* x, int x_dtype, int64_t ld_x, int M, int K,
                                 const float* row, const float* col, const float* bias, int gelu,
                                 void* q, int64_t ld_q, float* qs, void* stream) {
  return row_quant_impl(x, x_dtype, ld_x, M, K, row, col, bias, gelu, q, ld_q, qs, 0, nullptr, stream);
}

extern "C" int iflb200_row_quant_sharded(const void* x, int x_dtype, int64_t ld_x, int M, int K,
                                         const float* row, const float* col, const float* bias, int gelu,
                                         int phase, float* amax, void* q, int64_t ld_q, float* qs,
                                         void* stream) {
  if (phase != 1 && phase != 2 && phase != 3) return IFLB200_ERR_ARG;
  return row_quant_impl(x, x_dtype, ld_x, M, K, row, col, bias, gelu, q, ld_q, qs, phase, amax, stream);
}

extern "C" int iflb200_row_max_sharded(const void* x, int x_dtype, int64_t ld_x, int M, int K, const float* row,
                                       const float* col, const float* bias, int gelu, float* amax,
                                       float* const* amax_mirrors, int mirrors, void* stream) {
  return row_quant_impl(x, x_dtype, ld_x, M, K, row, col, bias, gelu, nullptr, 0, nullptr, 1, amax, stream,
                        amax_mirrors, mirrors);
}

#endif

#if IFLB200_ROW_PART == 0 || IFLB200_ROW_PART == -1
// Quantiser pass over fp32 rows whose maxima are already known (the second half of the gated GEMM):
// no reduction, so a row is cut into pieces of 2048 columns for separate CTAs and the pass runs as a
// flat elementwise kernel (816 x 16384: 6528 CTAs instead of 816 CTAs that each hold a whole row).
// The maxima are read, never written; `amax_zero` (another buffer, or NULL) is cleared for the
// producer after next -- clearing the buffer that is being read would race with the row's other CTAs.
template <bool FAST>
__global__ void __launch_bounds__(kRowThreads)
quant_from_amax_kernel(const float* __restrict__ h, int64_t ld_h, int M, int F, const float* __restrict__ amax,
                       float* __restrict__ amax_zero, uint8_t* __restrict__ q, int64_t ld_q, float* __restrict__ qs) {
  row_dependency_wait();  // h and amax come from the kernel before this one in the stream
  row_trigger();
  const int m = blockIdx.y;
  const int c0 = (blockIdx.x * kRowThreads + threadIdx.x) * 8;
  float scale, inv;
  quant_scales(amax[m], scale, inv);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    qs[m] = scale;
    if (amax_zero) amax_zero[m] = 0.0f;
  }
  if (c0 >= F) return;
  float v[8];
  load_f32<FAST>(h + (int64_t)m * ld_h, c0, F, v);
  store_codes<FAST>(q + (int64_t)m * ld_q, c0, F, v, inv);
}

extern "C" int iflb200_quant_from_amax(const float* h, int64_t ld_h, int M, int F, const float* amax, float* amax_zero,
                                       void* q, int64_t ld_q, float* qs, void* stream) {
  if (M < 0 || F < 0) return IFLB200_ERR_ARG;
  if (M == 0 || F == 0) return IFLB200_OK;
  if (!h || !amax || !q || !qs || amax_zero == amax) return IFLB200_ERR_ARG;
  if (ld_h < F || ld_q < F) return IFLB200_ERR_ARG;
  if (M > 65535) return IFLB200_ERR_SHAPE;
  const bool fast = F % 8 == 0 && aligned16(h) && (ld_h * 4) % 16 == 0 && aligned8(q) && ld_q % 8 == 0;
  const dim3 grid((unsigned)((F + kRowThreads * 8 - 1) / (kRowThreads * 8)), (unsigned)M);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (fast)
    launch_dep(quant_from_amax_kernel<true>, grid, dim3(kRowThreads), 0, s, 1, dependent_launch_for(M), h, ld_h, M, F, amax,
               amax_zero, reinterpret_cast<uint8_t*>(q), ld_q, qs);
  else
    launch_dep(quant_from_amax_kernel<false>, grid, dim3(kRowThreads), 0, s, 1, dependent_launch_for(M), h, ld_h, M, F, amax,
               amax_zero, reinterpret_cast<uint8_t*>(q), ld_q, qs);
  return (int)cudaGetLastError();
}
#endif

#if IFLB200_ROW_PART == 1 || IFLB200_ROW_PART == -1
extern "C" int iflb200_gated_act_quant(const void* gu, int gu_dtype, int64_t ld_gu, int M, int F,
                                       const float* row, const float* col, int act,
                                       void* q, int64_t ld_q, float* qs, void* stream) {
  if (M < 0 || F < 0) return IFLB200_ERR_ARG;
  if (F > 16384) return IFLB200_ERR_SHAPE;
  if (act != IFLB200_ACT_GELU_TANH && act != IFLB200_ACT_SILU) return IFLB200_ERR_ARG;
  if (M == 0 || F == 0) return IFLB200_OK;
  if (!gu || !q || !qs) return IFLB200_ERR_ARG;
  if (!dtype_ok(gu_dtype)) return IFLB200_ERR_DTYPE;
  if (ld_gu < 2 * (int64_t)F || ld_q < F) return IFLB200_ERR_ARG;
  GatedArgs a;
  a.gu = gu; a.ld_gu = ld_gu; a.M = M; a.F = F; a.row = row; a.col = col; a.act = act;
  a.q = reinterpret_cast<uint8_t*>(q); a.ld_q = ld_q; a.qs = qs;
  const int es = esize(gu_dtype);
  const bool fast = F % 8 == 0 && aligned16(gu) && (ld_gu * es) % 16 == 0 && aligned8(q) && ld_q % 8 == 0 &&
                    (!col || aligned16(col));
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (gu_dtype == IFLB200_BF16) launch_gated<__nv_bfloat16>(a, fast, s);
  else if (gu_dtype == IFLB200_F16) launch_gated<__half>(a, fast, s);
  else launch_gated<float>(a, fast, s);
  return (int)cudaGetLastError();
}

#endif

#if IFLB200_ROW_PART == 0 || IFLB200_ROW_PART == -1
extern "C" int iflb200_dequant_rows(const void* x, int x_dtype, int64_t ld_x, int M, int D,
                                    const float* row, const float* col, const float* bias,
                                    void* y, int y_dtype, int64_t ld_y, void* stream) {
  if (M < 0 || D < 0) return IFLB200_ERR_ARG;
  if (M == 0 || D == 0) return IFLB200_OK;
  if (!x || !y) return IFLB200_ERR_ARG;
  if (!dtype_ok(x_dtype) || !dtype_ok(y_dtype)) return IFLB200_ERR_DTYPE;
  if (ld_x < D || ld_y < D) return IFLB200_ERR_ARG;
  if (M > 65535 * 1024) return IFLB200_ERR_SHAPE;
  DequantArgs a;
  a.x = x; a.ld_x = ld_x; a.M = M; a.D = D; a.row = row; a.col = col; a.bias = bias;
  a.y = y; a.y_dtype = y_dtype; a.ld_y = ld_y;
  const bool fast = D % 8 == 0 && aligned16(x) && (ld_x * esize(x_dtype)) % 16 == 0 && aligned16(y) &&
                    (ld_y * esize(y_dtype)) % 16 == 0 && (!col || aligned16(col)) && (!bias || aligned16(bias));
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int chunks = (D + 2047) / 2048;
  // blockIdx.y carries the row: split very tall inputs into slabs of 65535 rows.
  for (int m0 = 0; m0 < M; m0 += 65535) {
    DequantArgs b = a;
    const int rows = (M - m0 < 65535) ? (M - m0) : 65535;
    b.M = rows;
    b.x = reinterpret_cast<const char*>(x) + (int64_t)m0 * ld_x * esize(x_dtype);
    b.y = reinterpret_cast<char*>(y) + (int64_t)m0 * ld_y * esize(y_dtype);
    b.row = row ? row + m0 : nullptr;
    const dim3 grid(chunks, rows);
    if (fast) {
      if (x_dtype == IFLB200_BF16) launch_dep(dequant_rows_kernel<__nv_bfloat16, true>, dim3(grid), dim3(256), 0, s, 1, dependent_launch_for(b.M), b);
      else if (x_dtype == IFLB200_F16) launch_dep(dequant_rows_kernel<__half, true>, dim3(grid), dim3(256), 0, s, 1, dependent_launch_for(b.M), b);
      else launch_dep(dequant_rows_kernel<float, true>, dim3(grid), dim3(256), 0, s, 1, dependent_launch_for(b.M), b);
    } else {
      if (x_dtype == IFLB200_BF16) launch_dep(dequant_rows_kernel<__nv_bfloat16, false>, dim3(grid), dim3(256), 0, s, 1, dependent_launch_for(b.M), b);
      else if (x_dtype == IFLB200_F16) launch_dep(dequant_rows_kernel<__half, false>, dim3(grid), dim3(256), 0, s, 1, dependent_launch_for(b.M), b);
      else launch_dep(dequant_rows_kernel<float, false>, dim3(grid), dim3(256), 0, s, 1, dependent_launch_for(b.M), b);
    }
  }
  return (int)cudaGetLastError();
}

#endif

#if IFLB200_ROW_PART == 2 || IFLB200_ROW_PART == -1
static int resnorm_impl(void* res, int res_dtype, int64_t ld_res, int M, int D, const void* delta, int delta_splits,
                        int64_t ld_delta, const float* delta_row, const float* delta_col, const float* bias,
                        const float* gate, int write_res, int layernorm, const float* weight, const float* beta,
                        const float* mod_scale, const float* mod_shift, const int32_t* mod_index, float eps, void* q,
                        int64_t ld_q, float* qs, void* y, int y_dtype, int64_t ld_y, void* stream,
                        void* const* q_mirrors = nullptr, float* const* qs_mirrors = nullptr, int mirrors = 0) {
  if (M < 0 || D < 0) return IFLB200_ERR_ARG;
  if (mirrors < 0 || mirrors > kMaxMirrors || (mirrors > 0 && (!q_mirrors || !qs_mirrors || !q || !delta_splits)))
    return IFLB200_ERR_ARG;
  if (M == 0 || D == 0) return IFLB200_OK;
  if (!res) return IFLB200_ERR_ARG;
  if (res_dtype != IFLB200_F32 && res_dtype != IFLB200_BF16) return IFLB200_ERR_DTYPE;
  if (y && !dtype_ok(y_dtype)) return IFLB200_ERR_DTYPE;
  if (D > kMaxWidth) return IFLB200_ERR_SHAPE;
  if (q && !qs) return IFLB200_ERR_ARG;
  if ((mod_scale == nullptr) != (mod_shift == nullptr)) return IFLB200_ERR_ARG;
  if (ld_res < D || (delta && ld_delta < D) || (q && ld_q < D) || (y && ld_y < D)) return IFLB200_ERR_ARG;
  ResNormArgs a;
  a.res = res; a.ld_res = ld_res; a.M = M; a.D = D;
  a.delta = delta_splits ? nullptr : reinterpret_cast<const __nv_bfloat16*>(delta);
  a.dpart = delta_splits ? reinterpret_cast<const float*>(delta) : nullptr;
  a.dsplits = delta_splits;
  a.ld_delta = ld_delta;
  a.drow = delta ? delta_row : nullptr; a.dcol = delta ? delta_col : nullptr;
  a.bias = delta ? bias : nullptr; a.gate = delta ? gate : nullptr;
  a.write_res = (write_res && delta) ? 1 : 0;
  a.layernorm = layernorm; a.weight = weight; a.beta = beta;
  a.mod_scale = mod_scale; a.mod_shift = mod_shift; a.mod_index = mod_index; a.eps = eps;
  a.q = reinterpret_cast<uint8_t*>(q); a.ld_q = ld_q; a.qs = qs;
  a.y = y; a.y_dtype = y_dtype; a.ld_y = ld_y;
  a.mirrors = mirrors;
  bool mirrors_ok = true;
  for (int k = 0; k < kMaxMirrors; ++k) {
    a.q_mirror[k] = k < mirrors ? reinterpret_cast<uint8_t*>(q_mirrors[k]) : nullptr;
    a.qs_mirror[k] = k < mirrors ? qs_mirrors[k] : nullptr;
    if (k < mirrors && (!a.q_mirror[k] || !a.qs_mirror[k])) return IFLB200_ERR_ARG;
    if (k < mirrors && !aligned8(a.q_mirror[k])) mirrors_ok = false;
  }
  if (!mirrors_ok) return IFLB200_ERR_ALIGN;
  const bool tables_ok = (!a.dcol || aligned16(a.dcol)) && (!a.bias || aligned16(a.bias)) &&
                         (!a.gate || aligned16(a.gate)) && (!weight || aligned16(weight)) &&
                         (!beta || aligned16(beta)) && (!mod_scale || aligned16(mod_scale)) &&
                         (!mod_shift || aligned16(mod_shift));
  const bool fast = D % 8 == 0 && aligned16(res) && (ld_res * esize(res_dtype)) % 16 == 0 &&
                    (!delta || (aligned16(delta) && (ld_delta * (delta_splits ? 4 : 2)) % 16 == 0)) &&
                    (!q || (aligned8(q) && ld_q % 8 == 0)) &&
                    (!y || (aligned16(y) && (ld_y * esize(y_dtype)) % 16 == 0)) && tables_ok;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (delta_splits) {
    const int st = res_dtype == IFLB200_F32 ? launch_resnorm_partials<float>(a, fast, s)
                                            : launch_resnorm_partials<__nv_bfloat16>(a, fast, s);
    if (st != IFLB200_OK) return st;
    return (int)cudaGetLastError();
  }
  if (res_dtype == IFLB200_F32) launch_resnorm<float>(a, fast, s);
  else launch_resnorm<__nv_bfloat16>(a, fast, s);
  return (int)cudaGetLastError();
}

extern "C" int iflb200_residual_norm_quant(void* res, int res_dtype, int64_t ld_res, int M, int D,
                                           const void* delta, int64_t ld_delta,
                                           const float* delta_row, const float* delta_col,
                                           const float* bias, const float* gate, int write_res,
                                           int layernorm, const float* weight, const float* beta,
                                           const float* mod_scale, const float* mod_shift,
                                           const int32_t* mod_index, float eps,
                                           void* q, int64_t ld_q, float* qs,
                                           void* y, int y_dtype, int64_t ld_y, void* stream) {
  return resnorm_impl(res, res_dtype, ld_res, M, D, delta, 0, ld_delta, delta_row, delta_col, bias, gate, write_res,
                      layernorm, weight, beta, mod_scale, mod_shift, mod_index, eps, q, ld_q, qs, y, y_dtype, ld_y, stream);
}

extern "C" int iflb200_residual_norm_quant_partials(void* res, int res_dtype, int64_t ld_res, int M, int D,
                                                    const float* delta_partials, int splits, int64_t ld_delta,
                                                    const float* delta_row, const float* delta_col,
                                                    const float* bias, const float* gate, int write_res,
                                                    int layernorm, const float* weight, const float* beta,
                                                    const float* mod_scale, const float* mod_shift,
                                                    const int32_t* mod_index, float eps,
                                                    void* q, int64_t ld_q, float* qs,
                                                    void* y, int y_dtype, int64_t ld_y, void* stream) {
  if (!delta_partials || splits < 1 || splits > 8) return IFLB200_ERR_ARG;
  return resnorm_impl(res, res_dtype, ld_res, M, D, delta_partials, splits, ld_delta, delta_row, delta_col, bias, gate,
                      write_res, layernorm, weight, beta, mod_scale, mod_shift, mod_index, eps, q, ld_q, qs, y, y_dtype,
                      ld_y, stream);
}

extern "C" int iflb200_residual_norm_quant_peers(void* res, int res_dtype, int64_t ld_res, int M, int D,
                                                 const float* delta_partials, int splits, int64_t ld_delta,
                                                 const float* delta_row, const float* delta_col, const float* bias,
                                                 const float* gate, int write_res, int layernorm, const float* weight,
                                                 const float* beta, const float* mod_scale, const float* mod_shift,
                                                 const int32_t* mod_index, float eps, void* q, int64_t ld_q, float* qs,
                                                 void* const* q_mirrors, float* const* qs_mirrors, int mirrors,
                                                 void* stream) {
  if (!delta_partials || splits < 1 || splits > 8) return IFLB200_ERR_ARG;
  return resnorm_impl(res, res_dtype, ld_res, M, D, delta_partials, splits, ld_delta, delta_row, delta_col, bias, gate,
                      write_res, layernorm, weight, beta, mod_scale, mod_shift, mod_index, eps, q, ld_q, qs, nullptr, 0,
                      0, stream, q_mirrors, qs_mirrors, mirrors);
}

#endif

#if IFLB200_ROW_PART == 1 || IFLB200_ROW_PART == -1
static int pack_grid(int64_t n) {
  int64_t ctas = (n + (int64_t)kPackThreads * 8 * 4 - 1) / ((int64_t)kPackThreads * 8 * 4);
  if (ctas < 1) ctas = 1;
  if (ctas > kPackMaxCtas) ctas = kPackMaxCtas;
  return (int)ctas;
}

extern "C" size_t iflb200_pack_workspace_bytes(int64_t n) {
  return (size_t)pack_grid(n < 0 ? 0 : n) * sizeof(uint32_t);
}

extern "C" int iflb200_dynamic_pack_bf16_e4m3(const void* x, int64_t n, void* q, float* scale,
                                              void* workspace, size_t workspace_bytes,
                                              void* stream) {
  if (n <= 0 || !x || !q || !scale) return IFLB200_ERR_ARG;
  if (!workspace || workspace_bytes < iflb200_pack_workspace_bytes(n)) return IFLB200_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(x) & 1) || (reinterpret_cast<uintptr_t>(workspace) & 3))
    return IFLB200_ERR_ALIGN;
  const int grid = pack_grid(n);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  uint32_t* partial = reinterpret_cast<uint32_t*>(workspace);
  launch_dep(amax_partial_kernel, dim3(grid), dim3(kPackThreads), 0, s, 1, dependent_launch_for(n >> 12), reinterpret_cast<const uint16_t*>(x), n, partial);
  launch_dep(pack_kernel, dim3(grid), dim3(kPackThreads), 0, s, 1, dependent_launch_for(n >> 12), reinterpret_cast<const uint16_t*>(x), n, partial, grid,
                                            nullptr, scale, reinterpret_cast<uint8_t*>(q));
  return (int)cudaGetLastError();
}

extern "C" int iflb200_pack_bf16_e4m3(const void* x, int64_t n, const float* scale, void* q,
                                      void* stream) {
  if (n < 0 || !scale) return IFLB200_ERR_ARG;
  if (n == 0) return IFLB200_OK;
  if (!x || !q) return IFLB200_ERR_ARG;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  launch_dep(pack_kernel, dim3(pack_grid(n)), dim3(kPackThreads), 0, s, 1, dependent_launch_for(n >> 12), reinterpret_cast<const uint16_t*>(x), n, nullptr,
                                                    0, scale, nullptr, reinterpret_cast<uint8_t*>(q));
  return (int)cudaGetLastError();
}
// --------------------------------------------------------------------------------------------
// Dynamic pack for callers that cannot allocate.
//
// The dynamic pack needs a few hundred words of scratch (one partial maximum per CTA of the first
// kernel).  Hosts that drive this library from a fixed memory plan -- an embedded control loop
// whose device memory was carved up at start-up, a C or C++ runtime that has no caching
// allocator behind it, a real-time loop that cannot afford the device-wide stall of a
// cudaMalloc -- have nowhere to get that scratch from.  For them
// the scratch lives in the library image itself: a file-scope device array, resident on every GPU
// that loads the library until the process exits (4 KB).
//
// Host code must not pass the array's name to a kernel: on the host that name is only a
// stand-in symbol, not a device address.  The address is looked up once per device with
// cudaGetSymbolAddress while that device is current, and that pointer is what the kernels get.
// --------------------------------------------------------------------------------------------
static __device__ __align__(256) uint32_t g_pack_noalloc_scratch[kPackMaxCtas];

static int pack_noalloc_scratch(uint32_t** out) {
  static uint32_t* resolved[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return IFLB200_ERR_DEVICE;
  uint32_t* p = __atomic_load_n(&resolved[dev], __ATOMIC_ACQUIRE);
  if (p == nullptr) {
    // First call on this device (which is the current one): resolve the symbol.  Two host
    // threads racing here resolve the same address; the store is idempotent.
    void* addr = nullptr;
    e = cudaGetSymbolAddress(&addr, g_pack_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    if (addr == nullptr) return IFLB200_ERR_DEVICE;
    p = reinterpret_cast<uint32_t*>(addr);
    __atomic_store_n(&resolved[dev], p, __ATOMIC_RELEASE);
  }
  *out = p;
  return IFLB200_OK;
}

extern "C" int iflb200_dynamic_pack_bf16_e4m3_noalloc(const void* x, int64_t n, void* q, float* scale,
                                                      void* stream) {
  if (n <= 0 || !x || !q || !scale) return IFLB200_ERR_ARG;
  if (n > IFLB200_PACK_NOALLOC_MAX_ELEMENTS) return IFLB200_ERR_TOO_LARGE;
  if (reinterpret_cast<uintptr_t>(x) & 1) return IFLB200_ERR_ALIGN;
  uint32_t* partial = nullptr;
  const int st = pack_noalloc_scratch(&partial);
  if (st != IFLB200_OK) return st;
  const int grid = pack_grid(n);  // <= kPackMaxCtas words of scratch, all written before they are read
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  launch_dep(amax_partial_kernel, dim3(grid), dim3(kPackThreads), 0, s, 1, dependent_launch_for(n >> 12), reinterpret_cast<const uint16_t*>(x), n, partial);
  launch_dep(pack_kernel, dim3(grid), dim3(kPackThreads), 0, s, 1, dependent_launch_for(n >> 12), reinterpret_cast<const uint16_t*>(x), n, partial, grid, nullptr,
                                            scale, reinterpret_cast<uint8_t*>(q));
  return (int)cudaGetLastError();
}
#endif

