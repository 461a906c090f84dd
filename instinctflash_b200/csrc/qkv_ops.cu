// Consumers of the raw fused-QKV accumulator for sm_100a: dequantisation (row and column
// scales, bias), RMS norm of Q and K, rotary embedding, and the scatter of K and V into their
// cache rows.  Two layouts, as in the reference:
//
//   qkv_split  (instinctflash/kernels/rope.py:22-114): per-head RMS norm, rotary pairs
//              (i, i + HD/2) inside a head; one warp owns one (token, head).
//   wan_qkv    (instinctflash/kernels/wan.py:20-104): RMS norm over the full width of Q or K,
//              rotary pairs (2j, 2j+1); one CTA owns one (row, part) with the part in registers.
//
// Element arithmetic is the order the reference's kernels compile to for sm_100: a multiply
// that feeds an add is one fma.rn, every other multiply rounds on its own; of the two products
// of a rotation the one with the sine is rounded and the one with the cosine is fused; the
// mean of squares is div.full(sum, n), the scale rsqrt.approx.ftz; sine and cosine are the
// accurate single-precision library functions.  Only the order in which the squares are summed
// differs from the reference (its order is a property of its thread layout), so outputs that go
// through a norm agree to rounding, the others bit for bit.
//
// Both are HBM-bound: out_bytes + in_bytes per element, every element read and written once.
#include <cuda_runtime.h>

#include <type_traits>

#include "../../include/iflb200.h"
#include "launch.cuh"
#include "rowmath.cuh"

namespace iflb200 {

namespace {

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// raw * row * col + bias with the reference's contraction (any of the three may be absent)
__device__ __forceinline__ float dequant(float raw, bool has_row, float r, const float* col, const float* bias,
                                         int64_t c) {
  Chain x(raw);
  if (has_row) x.mul(r);
  if (col) x.mul(col[c]);
  if (bias) x.add(bias[c]);
  return x.done();
}

__device__ __forceinline__ void rotate(float& a, float& b, float cs, float sn) {
  // (a, b) <- (a cos - b sin, b cos + a sin): sine products rounded, cosine products fused
  const float bs = __fmul_rn(b, sn);
  const float as = __fmul_rn(a, sn);
  const float na = __fmaf_rn(a, cs, -bs);
  const float nb = __fmaf_rn(b, cs, as);
  a = na;
  b = nb;
}

// --------------------------------------------------------------------------------------------
// qkv_split: one warp per (token, head); lane l holds elements l, l+32, ... of each half.
// --------------------------------------------------------------------------------------------
struct QkvSplitArgs {
  const void* qkv;
  int64_t ld_qkv;
  int T, HQ, HKV, HD;
  const float *row, *col, *bias, *q_norm, *k_norm;
  float eps;
  const float *inv_freq, *pos;
  int64_t ld_pos;
  const int32_t* sections;
  const int32_t* kv_base_dev;
  int kv_base;
  void *q, *k, *v;
  int64_t sq_t, sq_h, sk_t, sk_h, sv_t, sv_h;
};

template <typename XT, typename OT, int NJ>
__global__ void __launch_bounds__(256) qkv_split_kernel(const QkvSplitArgs a) {
  if (threadIdx.x == 0) grid_dependency_wait();
  __syncthreads();
  grid_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int heads = a.HQ + 2 * a.HKV;
  const int64_t unit = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (unit >= (int64_t)a.T * heads) return;
  const int t = (int)(unit / heads);
  const int h = (int)(unit % heads);
  const int half = a.HD >> 1;
  const XT* src = reinterpret_cast<const XT*>(a.qkv) + (int64_t)t * a.ld_qkv + (int64_t)h * a.HD;
  const bool has_row = a.row != nullptr;
  const float r = has_row ? a.row[t] : 1.0f;

  float lo[NJ], hi[NJ];
  XT rl[NJ], rh[NJ];
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    const int i = lane + 32 * j;
    const bool on = i < half;
    rl[j] = on ? src[i] : XT(0.0f);
    rh[j] = on ? src[half + i] : XT(0.0f);
  }
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    const int i = lane + 32 * j;
    if (i < half) {
      lo[j] = dequant(to_f32(rl[j]), has_row, r, a.col, a.bias, (int64_t)h * a.HD + i);
      hi[j] = dequant(to_f32(rh[j]), has_row, r, a.col, a.bias, (int64_t)h * a.HD + half + i);
    } else {
      lo[j] = 0.0f;
      hi[j] = 0.0f;
    }
  }
  if (h < a.HQ + a.HKV) {
    const float* nw = h < a.HQ ? a.q_norm : a.k_norm;
    if (nw) {
      float sl = 0.0f, sh = 0.0f;
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        sl = __fmaf_rn(lo[j], lo[j], sl);
        sh = __fmaf_rn(hi[j], hi[j], sh);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        sl = __fadd_rn(sl, __shfl_xor_sync(0xFFFFFFFFu, sl, o));
        sh = __fadd_rn(sh, __shfl_xor_sync(0xFFFFFFFFu, sh, o));
      }
      const float rs = rsqrt_approx_ftz(__fadd_rn(div_full(__fadd_rn(sl, sh), (float)a.HD), a.eps));
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        const int i = lane + 32 * j;
        if (i < half) {
          lo[j] = __fmul_rn(__fmul_rn(lo[j], rs), nw[i]);
          hi[j] = __fmul_rn(__fmul_rn(hi[j], rs), nw[half + i]);
        }
      }
    }
    if (a.inv_freq) {
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        const int i = lane + 32 * j;
        if (i < half) {
          const int sec = a.sections ? a.sections[i] : 0;
          const float ang = __fmul_rn(a.pos[(int64_t)t * a.ld_pos + sec], a.inv_freq[i]);
          rotate(lo[j], hi[j], cosf(ang), sinf(ang));
        }
      }
    }
  }
  const int64_t kv_row = (int64_t)(a.kv_base_dev ? *a.kv_base_dev : a.kv_base) + t;
  OT* dst;
  if (h < a.HQ) dst = reinterpret_cast<OT*>(a.q) + (int64_t)t * a.sq_t + (int64_t)h * a.sq_h;
  else if (h < a.HQ + a.HKV) dst = reinterpret_cast<OT*>(a.k) + kv_row * a.sk_t + (int64_t)(h - a.HQ) * a.sk_h;
  else dst = reinterpret_cast<OT*>(a.v) + kv_row * a.sv_t + (int64_t)(h - a.HQ - a.HKV) * a.sv_h;
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    const int i = lane + 32 * j;
    if (i < half) {
      dst[i] = from_f32<OT>(lo[j]);
      dst[half + i] = from_f32<OT>(hi[j]);
    }
  }
}

// The shapes the engines use (bf16 accumulator, 16-bit outputs, head widths 64 / 128 / 256, every
// pointer and stride a multiple of VEC elements): lane l holds the VEC consecutive elements
// l*VEC .. l*VEC+VEC-1 of each half, one 2*VEC-byte access each.
template <int VEC>
struct Pack;
template <>
struct Pack<1> { using type = uint16_t; };
template <>
struct Pack<2> { using type = uint32_t; };
template <>
struct Pack<4> { using type = uint2; };

template <int VEC>
__device__ __forceinline__ void load_vec_f32(const float* p, float (&o)[VEC]) {
  if constexpr (VEC == 4) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  } else if constexpr (VEC == 2) {
    const float2 v = *reinterpret_cast<const float2*>(p);
    o[0] = v.x; o[1] = v.y;
  } else {
    o[0] = *p;
  }
}

template <typename OT, int VEC>
__global__ void __launch_bounds__(256) qkv_split_vec_kernel(const QkvSplitArgs a) {
  using P = typename Pack<VEC>::type;
  if (threadIdx.x == 0) grid_dependency_wait();
  __syncthreads();
  grid_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int heads = a.HQ + 2 * a.HKV;
  const int64_t unit = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (unit >= (int64_t)a.T * heads) return;
  const int t = (int)(unit / heads);
  const int h = (int)(unit % heads);
  constexpr int half = 32 * VEC;
  const int i0 = lane * VEC;
  const __nv_bfloat16* src =
      reinterpret_cast<const __nv_bfloat16*>(a.qkv) + (int64_t)t * a.ld_qkv + (int64_t)h * (2 * half) + i0;
  const P pl = *reinterpret_cast<const P*>(src);
  const P ph = *reinterpret_cast<const P*>(src + half);
  const bool has_row = a.row != nullptr;
  const float r = has_row ? a.row[t] : 1.0f;
  const bool qk = h < a.HQ + a.HKV;
  const bool rope = qk && a.inv_freq != nullptr;
  float ang[VEC];
  if (rope) {
    float fr[VEC];
    load_vec_f32<VEC>(a.inv_freq + i0, fr);
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      const int sec = a.sections ? a.sections[i0 + e] : 0;
      ang[e] = __fmul_rn(a.pos[(int64_t)t * a.ld_pos + sec], fr[e]);
    }
  }
  float lo[VEC], hi[VEC];
  {
    const __nv_bfloat16* el = reinterpret_cast<const __nv_bfloat16*>(&pl);
    const __nv_bfloat16* eh = reinterpret_cast<const __nv_bfloat16*>(&ph);
    const int64_t c = (int64_t)h * (2 * half) + i0;
    float cl[VEC], chh[VEC], bl[VEC], bh[VEC];
    if (a.col) { load_vec_f32<VEC>(a.col + c, cl); load_vec_f32<VEC>(a.col + c + half, chh); }
    if (a.bias) { load_vec_f32<VEC>(a.bias + c, bl); load_vec_f32<VEC>(a.bias + c + half, bh); }
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      Chain xl(to_f32(el[e])), xh(to_f32(eh[e]));
      if (has_row) { xl.mul(r); xh.mul(r); }
      if (a.col) { xl.mul(cl[e]); xh.mul(chh[e]); }
      if (a.bias) { xl.add(bl[e]); xh.add(bh[e]); }
      lo[e] = xl.done();
      hi[e] = xh.done();
    }
  }
  if (qk) {
    const float* nw = h < a.HQ ? a.q_norm : a.k_norm;
    if (nw) {
      float sl = 0.0f, sh = 0.0f;
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        sl = __fmaf_rn(lo[e], lo[e], sl);
        sh = __fmaf_rn(hi[e], hi[e], sh);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        sl = __fadd_rn(sl, __shfl_xor_sync(0xFFFFFFFFu, sl, o));
        sh = __fadd_rn(sh, __shfl_xor_sync(0xFFFFFFFFu, sh, o));
      }
      const float rs = rsqrt_approx_ftz(__fadd_rn(div_full(__fadd_rn(sl, sh), (float)(2 * half)), a.eps));
      float wl[VEC], wh[VEC];
      load_vec_f32<VEC>(nw + i0, wl);
      load_vec_f32<VEC>(nw + half + i0, wh);
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        lo[e] = __fmul_rn(__fmul_rn(lo[e], rs), wl[e]);
        hi[e] = __fmul_rn(__fmul_rn(hi[e], rs), wh[e]);
      }
    }
    if (rope) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) rotate(lo[e], hi[e], cosf(ang[e]), sinf(ang[e]));
    }
  }
  const int64_t kv_row = (int64_t)(a.kv_base_dev ? *a.kv_base_dev : a.kv_base) + t;
  OT* dst;
  if (h < a.HQ) dst = reinterpret_cast<OT*>(a.q) + (int64_t)t * a.sq_t + (int64_t)h * a.sq_h;
  else if (qk) dst = reinterpret_cast<OT*>(a.k) + kv_row * a.sk_t + (int64_t)(h - a.HQ) * a.sk_h;
  else dst = reinterpret_cast<OT*>(a.v) + kv_row * a.sv_t + (int64_t)(h - a.HQ - a.HKV) * a.sv_h;
  P ol, oh;
  OT* wl_ = reinterpret_cast<OT*>(&ol);
  OT* wh_ = reinterpret_cast<OT*>(&oh);
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    wl_[e] = from_f32<OT>(lo[e]);
    wh_[e] = from_f32<OT>(hi[e]);
  }
  *reinterpret_cast<P*>(dst + i0) = ol;
  *reinterpret_cast<P*>(dst + half + i0) = oh;
}

template <typename OT>
cudaError_t launch_qkv_split_vec(const QkvSplitArgs& a, cudaStream_t s) {
  const int64_t units = (int64_t)a.T * (a.HQ + 2 * a.HKV);
  const dim3 grid((unsigned)((units + 7) / 8));
  const bool dep = dependent_launch_for(a.T);
  if (a.HD == 256) return launch_dep(qkv_split_vec_kernel<OT, 4>, grid, dim3(256), 0, s, 1, dep, a);
  if (a.HD == 128) return launch_dep(qkv_split_vec_kernel<OT, 2>, grid, dim3(256), 0, s, 1, dep, a);
  return launch_dep(qkv_split_vec_kernel<OT, 1>, grid, dim3(256), 0, s, 1, dep, a);
}

// every access of the vector kernel is 2*VEC bytes (16-bit data) or 4*VEC bytes (float32 vectors)
bool qkv_split_vec_ok(const QkvSplitArgs& a, int qkv_dtype, int out_dtype) {
  if (qkv_dtype != IFLB200_BF16 || out_dtype == IFLB200_F32) return false;
  if (a.HD != 64 && a.HD != 128 && a.HD != 256) return false;
  const int vec = a.HD / 64;
  auto al = [&](const void* p, int bytes) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) % bytes) == 0; };
  auto mult = [&](int64_t v) { return v % vec == 0; };
  return al(a.qkv, 2 * vec) && mult(a.ld_qkv) && al(a.q, 2 * vec) && al(a.k, 2 * vec) && al(a.v, 2 * vec) &&
         mult(a.sq_t) && mult(a.sq_h) && mult(a.sk_t) && mult(a.sk_h) && mult(a.sv_t) && mult(a.sv_h) &&
         al(a.col, 4 * vec) && al(a.bias, 4 * vec) && al(a.q_norm, 4 * vec) && al(a.k_norm, 4 * vec) &&
         al(a.inv_freq, 4 * vec);
}

template <typename XT, typename OT>
cudaError_t launch_qkv_split(const QkvSplitArgs& a, cudaStream_t s) {
  const int64_t units = (int64_t)a.T * (a.HQ + 2 * a.HKV);
  const dim3 grid((unsigned)((units + 7) / 8));
  const int nj = (a.HD / 2 + 31) / 32;
  const bool dep = dependent_launch_for(a.T);
  if (nj <= 1) return launch_dep(qkv_split_kernel<XT, OT, 1>, grid, dim3(256), 0, s, 1, dep, a);
  if (nj <= 2) return launch_dep(qkv_split_kernel<XT, OT, 2>, grid, dim3(256), 0, s, 1, dep, a);
  if (nj <= 4) return launch_dep(qkv_split_kernel<XT, OT, 4>, grid, dim3(256), 0, s, 1, dep, a);
  return launch_dep(qkv_split_kernel<XT, OT, 8>, grid, dim3(256), 0, s, 1, dep, a);
}

template <typename XT>
cudaError_t launch_qkv_split_out(const QkvSplitArgs& a, int out_dtype, cudaStream_t s) {
  if (out_dtype == IFLB200_F16) return launch_qkv_split<XT, __half>(a, s);
  if (out_dtype == IFLB200_BF16) return launch_qkv_split<XT, __nv_bfloat16>(a, s);
  return launch_qkv_split<XT, float>(a, s);
}

// --------------------------------------------------------------------------------------------
// wan_qkv: one CTA per (row, part); thread t holds chunks t, t+TPB, ... of eight consecutive
// elements (four rotary pairs), NCH of them.  The host picks NCH in {1,2,4,8} and a block of
// ceil(chunks / NCH) threads rounded up to a warp (at most 256), so the part fits the CTA with
// little padding (3072 columns: 192 threads x 2 chunks; 5120: 160 x 4).  FAST: every pointer and
// stride obeys the 16-byte rule, the width is a multiple of 8 and the head width a multiple of 8,
// so all accesses are 128-bit and a chunk lies inside one head.
// --------------------------------------------------------------------------------------------
#ifndef IFLB200_WAN_MAX_THREADS
#define IFLB200_WAN_MAX_THREADS 256
#endif
constexpr int kWanMaxThreads = IFLB200_WAN_MAX_THREADS;
constexpr int kWanMaxChunks = 8;

struct WanQkvArgs {
  const void* raw;
  int64_t ld_raw;
  int rows, tokens, H, HD;
  const float *row, *col, *bias, *q_norm, *k_norm;
  float eps;
  const float *inv_freq, *pos;
  int64_t ld_pos;
  const int32_t *sections, *slots;
  void *q, *k, *v;
  int64_t ld_q, sk_b, sk_s, sv_b, sv_s;
};

template <bool FAST, typename XT>
__device__ __forceinline__ void load8(const XT* p, int n, float (&o)[8]) {
  if (FAST) {
    if constexpr (sizeof(XT) == 4) {
      const float4 u = *reinterpret_cast<const float4*>(p);
      const float4 w = *reinterpret_cast<const float4*>(p + 4);
      o[0] = u.x; o[1] = u.y; o[2] = u.z; o[3] = u.w; o[4] = w.x; o[5] = w.y; o[6] = w.z; o[7] = w.w;
    } else {
      const uint4 u = *reinterpret_cast<const uint4*>(p);
      const XT* e = reinterpret_cast<const XT*>(&u);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = to_f32(e[i]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = i < n ? to_f32(p[i]) : 0.0f;
  }
}

template <bool FAST, typename OT>
__device__ __forceinline__ void store8(OT* p, int n, const float (&v)[8]) {
  if (FAST) {
    if constexpr (sizeof(OT) == 4) {
      *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
    } else {
      uint4 u;
      OT* e = reinterpret_cast<OT*>(&u);
#pragma unroll
      for (int i = 0; i < 8; ++i) e[i] = from_f32<OT>(v[i]);
      *reinterpret_cast<uint4*>(p) = u;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (i < n) p[i] = from_f32<OT>(v[i]);
  }
}

template <typename XT, typename OT, int NCH, bool FAST>
__global__ void __launch_bounds__(kWanMaxThreads) wan_qkv_kernel(const WanQkvArgs a) {
  __shared__ float s_cos[256], s_sin[256];  // one angle per rotary pair of a head (HD <= 512)
  __shared__ float s_red[kWanMaxThreads / 32];
  if (threadIdx.x == 0) grid_dependency_wait();
  __syncthreads();
  grid_launch_dependents();
  const int tpb = blockDim.x;
  const int row = blockIdx.x;
  const int part = blockIdx.y;  // 0 = Q, 1 = K, 2 = V
  const int b = row / a.tokens;
  const int t = row - b * a.tokens;
  const int D = a.H * a.HD;
  const float* nw = part == 0 ? a.q_norm : (part == 1 ? a.k_norm : nullptr);
  const bool rope = a.inv_freq != nullptr && part < 2;
  const int64_t col0 = (int64_t)part * D;
  const XT* src = reinterpret_cast<const XT*>(a.raw) + (int64_t)row * a.ld_raw + col0;
  const float* colp = a.col ? a.col + col0 : nullptr;
  const float* biasp = a.bias ? a.bias + col0 : nullptr;
  const bool has_row = a.row != nullptr;
  const float r = has_row ? a.row[row] : 1.0f;

  // every load of the part is issued before anything is used
  float x[NCH][8];
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int d0 = (threadIdx.x + c * tpb) * 8;
    if (d0 < D) load8<FAST, XT>(src + d0, D - d0, x[c]);
  }
  if (rope) {
    const int half = a.HD >> 1;
    for (int j = threadIdx.x; j < half; j += tpb) {
      const float ang = __fmul_rn(a.pos[(int64_t)t * a.ld_pos + a.sections[j]], a.inv_freq[j]);
      s_cos[j] = cosf(ang);
      s_sin[j] = sinf(ang);
    }
  }
  float ss = 0.0f;
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int d0 = (threadIdx.x + c * tpb) * 8;
    if (d0 < D) {
      float cs[8], bs[8];
      if (colp) load8<FAST, float>(colp + d0, D - d0, cs);
      if (biasp) load8<FAST, float>(biasp + d0, D - d0, bs);
      Chain8 ch(x[c]);
      if (has_row) ch.mul(r);
      if (colp) ch.mul(cs);
      if (biasp) ch.add(bs);
      ch.done(x[c]);
      if (!FAST) {
#pragma unroll
        for (int i = 0; i < 8; ++i) x[c][i] = d0 + i < D ? x[c][i] : 0.0f;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) ss = __fmaf_rn(x[c][i], x[c][i], ss);
    }
  }
  if (nw) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xFFFFFFFFu, ss, o));
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = ss;
  }
  __syncthreads();  // partial sums and the angle table
  if (nw) {
    float tot = s_red[0];
    for (int w = 1; w < (tpb >> 5); ++w) tot = __fadd_rn(tot, s_red[w]);
    const float rs = rsqrt_approx_ftz(__fadd_rn(div_full(tot, (float)D), a.eps));
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int d0 = (threadIdx.x + c * tpb) * 8;
      if (d0 < D) {
        float ws[8];
        load8<FAST, float>(nw + d0, D - d0, ws);
#pragma unroll
        for (int i = 0; i < 8; ++i) x[c][i] = __fmul_rn(__fmul_rn(x[c][i], rs), ws[i]);
      }
    }
  }
  if (rope) {
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int d0 = (threadIdx.x + c * tpb) * 8;
      if (d0 < D) {
        if (FAST) {
          const int j0 = (d0 % a.HD) >> 1;  // the chunk lies inside one head
#pragma unroll
          for (int i = 0; i < 8; i += 2) rotate(x[c][i], x[c][i + 1], s_cos[j0 + (i >> 1)], s_sin[j0 + (i >> 1)]);
        } else {
#pragma unroll
          for (int i = 0; i < 8; i += 2) {
            if (d0 + i + 1 < D) {  // D is even and d0 a multiple of 8: a pair never straddles heads
              const int j = ((d0 + i) % a.HD) >> 1;
              rotate(x[c][i], x[c][i + 1], s_cos[j], s_sin[j]);
            }
          }
        }
      }
    }
  }
  OT* dst;
  if (part == 0) {
    dst = reinterpret_cast<OT*>(a.q) + (int64_t)row * a.ld_q;
  } else {
    const int64_t slot = a.slots ? a.slots[t] : t;
    dst = part == 1 ? reinterpret_cast<OT*>(a.k) + (int64_t)b * a.sk_b + slot * a.sk_s
                    : reinterpret_cast<OT*>(a.v) + (int64_t)b * a.sv_b + slot * a.sv_s;
  }
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int d0 = (threadIdx.x + c * tpb) * 8;
    if (d0 < D) store8<FAST, OT>(dst + d0, D - d0, x[c]);
  }
}

template <typename XT, typename OT, bool FAST>
cudaError_t launch_wan_geom(const WanQkvArgs& a, int parts, cudaStream_t s) {
  const int chunks = (a.H * a.HD + 7) / 8;
  int nch = 1;
  while (nch < kWanMaxChunks && (chunks + nch - 1) / nch > kWanMaxThreads) nch *= 2;
  const int threads = (((chunks + nch - 1) / nch + 31) / 32) * 32;
  const dim3 grid((unsigned)a.rows, (unsigned)parts), block((unsigned)threads);
  const bool dep = dependent_launch_for(a.rows);
  switch (nch) {
    case 1: return launch_dep(wan_qkv_kernel<XT, OT, 1, FAST>, grid, block, 0, s, 1, dep, a);
    case 2: return launch_dep(wan_qkv_kernel<XT, OT, 2, FAST>, grid, block, 0, s, 1, dep, a);
    case 4: return launch_dep(wan_qkv_kernel<XT, OT, 4, FAST>, grid, block, 0, s, 1, dep, a);
    default: return launch_dep(wan_qkv_kernel<XT, OT, 8, FAST>, grid, block, 0, s, 1, dep, a);
  }
}

template <typename XT, typename OT>
cudaError_t launch_wan_out(const WanQkvArgs& a, int parts, bool fast, cudaStream_t s) {
  // the 128-bit instantiation exists for the raw accumulator type the engines produce (bf16)
  if constexpr (std::is_same<XT, __nv_bfloat16>::value && sizeof(OT) == 2) {
    if (fast) return launch_wan_geom<XT, OT, true>(a, parts, s);
  }
  return launch_wan_geom<XT, OT, false>(a, parts, s);
}

template <typename XT>
cudaError_t launch_wan_qkv(const WanQkvArgs& a, int parts, int out_dtype, bool fast, cudaStream_t s) {
  if (out_dtype == IFLB200_F16) return launch_wan_out<XT, __half>(a, parts, fast, s);
  if (out_dtype == IFLB200_BF16) return launch_wan_out<XT, __nv_bfloat16>(a, parts, fast, s);
  return launch_wan_out<XT, float>(a, parts, fast, s);
}

bool float_dtype(int d) { return d == IFLB200_F32 || d == IFLB200_BF16 || d == IFLB200_F16; }
int dtype_size(int d) { return d == IFLB200_F32 ? 4 : 2; }
bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace
}  // namespace iflb200

using namespace iflb200;

extern "C" int iflb200_qkv_split(const void* qkv, int qkv_dtype, int64_t ld_qkv, int T, int heads_q, int heads_kv,
                                 int head_dim, const float* row, const float* col, const float* bias,
                                 const float* q_norm, const float* k_norm, float eps, const float* inv_freq,
                                 const float* pos, int64_t ld_pos, const int32_t* sections,
                                 const int32_t* kv_base_dev, int kv_base, void* q_out, int64_t q_stride_t,
                                 int64_t q_stride_h, void* k_out, int64_t k_stride_t, int64_t k_stride_h,
                                 void* v_out, int64_t v_stride_t, int64_t v_stride_h, int out_dtype,
                                 void* stream) {
  if (T < 0 || heads_q < 0 || heads_kv < 0 || head_dim < 0) return IFLB200_ERR_ARG;
  if (!float_dtype(qkv_dtype) || !float_dtype(out_dtype)) return IFLB200_ERR_DTYPE;
  if (T == 0 || heads_q + heads_kv == 0) return IFLB200_OK;
  if (head_dim < 2 || (head_dim & 1) || head_dim > 512) return IFLB200_ERR_SHAPE;
  if (!qkv || (heads_q && !q_out) || (heads_kv && (!k_out || !v_out))) return IFLB200_ERR_ARG;
  if (inv_freq && !pos) return IFLB200_ERR_ARG;
  if ((q_norm == nullptr) != (k_norm == nullptr)) return IFLB200_ERR_ARG;
  if (ld_qkv < (int64_t)(heads_q + 2 * heads_kv) * head_dim) return IFLB200_ERR_ARG;
  if (!kv_base_dev && kv_base < 0) return IFLB200_ERR_ARG;
  QkvSplitArgs a;
  a.qkv = qkv; a.ld_qkv = ld_qkv; a.T = T; a.HQ = heads_q; a.HKV = heads_kv; a.HD = head_dim;
  a.row = row; a.col = col; a.bias = bias; a.q_norm = q_norm; a.k_norm = k_norm; a.eps = eps;
  a.inv_freq = inv_freq; a.pos = pos; a.ld_pos = ld_pos; a.sections = sections;
  a.kv_base_dev = kv_base_dev; a.kv_base = kv_base;
  a.q = q_out; a.k = k_out; a.v = v_out;
  a.sq_t = q_stride_t; a.sq_h = q_stride_h; a.sk_t = k_stride_t; a.sk_h = k_stride_h;
  a.sv_t = v_stride_t; a.sv_h = v_stride_h;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (qkv_split_vec_ok(a, qkv_dtype, out_dtype))
    e = out_dtype == IFLB200_F16 ? launch_qkv_split_vec<__half>(a, s) : launch_qkv_split_vec<__nv_bfloat16>(a, s);
  else if (qkv_dtype == IFLB200_BF16) e = launch_qkv_split_out<__nv_bfloat16>(a, out_dtype, s);
  else if (qkv_dtype == IFLB200_F16) e = launch_qkv_split_out<__half>(a, out_dtype, s);
  else e = launch_qkv_split_out<float>(a, out_dtype, s);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

extern "C" int iflb200_wan_qkv(const void* raw, int raw_dtype, int64_t ld_raw, int rows, int tokens, int heads,
                               int head_dim, const float* row, const float* col, const float* bias,
                               const float* q_norm, const float* k_norm, float eps, const float* inv_freq,
                               const float* pos, int64_t ld_pos, const int32_t* sections, const int32_t* slots,
                               void* q_out, int64_t ld_q, void* k_pool, int64_t k_stride_b, int64_t k_stride_s,
                               void* v_pool, int64_t v_stride_b, int64_t v_stride_s, int out_dtype,
                               void* stream) {
  if (rows < 0 || tokens <= 0 || heads <= 0 || head_dim <= 0) return IFLB200_ERR_ARG;
  if (!float_dtype(raw_dtype) || !float_dtype(out_dtype)) return IFLB200_ERR_DTYPE;
  if (rows == 0) return IFLB200_OK;
  if ((head_dim & 1) || head_dim > 512) return IFLB200_ERR_SHAPE;
  const int64_t D = (int64_t)heads * head_dim;
  if (D > (int64_t)kWanMaxThreads * kWanMaxChunks * 8 || D > 8192) return IFLB200_ERR_SHAPE;
  if (!raw || !q_out) return IFLB200_ERR_ARG;
  if (v_pool && !k_pool) return IFLB200_ERR_ARG;  // parts are Q, then K, then V
  if (inv_freq && (!pos || !sections)) return IFLB200_ERR_ARG;
  const int parts = 1 + (k_pool ? 1 : 0) + (v_pool ? 1 : 0);
  if (ld_raw < parts * D || ld_q < D) return IFLB200_ERR_ARG;
  WanQkvArgs a;
  a.raw = raw; a.ld_raw = ld_raw; a.rows = rows; a.tokens = tokens; a.H = heads; a.HD = head_dim;
  a.row = row; a.col = col; a.bias = bias; a.q_norm = q_norm; a.k_norm = k_norm; a.eps = eps;
  a.inv_freq = inv_freq; a.pos = pos; a.ld_pos = ld_pos; a.sections = sections; a.slots = slots;
  a.q = q_out; a.k = k_pool; a.v = v_pool;
  a.ld_q = ld_q; a.sk_b = k_stride_b; a.sk_s = k_stride_s; a.sv_b = v_stride_b; a.sv_s = v_stride_s;
  const int xs = dtype_size(raw_dtype), os = dtype_size(out_dtype);
  const int xe = 16 / xs, oe = 16 / os;  // elements per 16 bytes
  const bool fast = (D % 8 == 0) && (head_dim % 8 == 0) && aligned16(raw) && ld_raw % xe == 0 && aligned16(q_out) &&
                    ld_q % oe == 0 && (!col || aligned16(col)) && (!bias || aligned16(bias)) &&
                    (!q_norm || aligned16(q_norm)) && (!k_norm || aligned16(k_norm)) &&
                    (!k_pool || (aligned16(k_pool) && k_stride_b % oe == 0 && k_stride_s % oe == 0)) &&
                    (!v_pool || (aligned16(v_pool) && v_stride_b % oe == 0 && v_stride_s % oe == 0));
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (raw_dtype == IFLB200_BF16) e = launch_wan_qkv<__nv_bfloat16>(a, parts, out_dtype, fast, s);
  else if (raw_dtype == IFLB200_F16) e = launch_wan_qkv<__half>(a, parts, out_dtype, fast, s);
  else e = launch_wan_qkv<float>(a, parts, out_dtype, fast, s);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}
