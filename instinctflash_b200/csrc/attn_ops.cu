// Merge of split-KV attention partials with the per-token e4m3 quantiser of the merged row: the
// producer of the O projection's FP8 input in the reference engines
// (instinctflash/kernels/attention.py:109-145, _attn_combine with QUANT).
//
// The attention kernel leaves, per split sp, batch b, KV head and query row r = token * GROUP + h,
// an unnormalised output vector PO (BLOCK_D floats, BLOCK_D = head_dim rounded up to a power of
// two), the running maximum PM and the running sum PL.  For one token this kernel computes, for
// every query head and every d < head_dim, in the instruction order the reference compiles to:
//     m   = max over sp of PM                       (max.f32, starting from -inf)
//     w   = ex2.approx.ftz(PM[sp] - m)
//     l   = fma(w, PL[sp], l)                       (from 0, splits in order)
//     acc = fma(w, PO[sp][d], acc)                  (from 0, splits in order)
//     out = div.full(acc, l)
// stores out in O's type (optional), and quantises the token's full row of heads * head_dim
// values with one scale: amax = max(max |out|, 1e-8), qs = div.full(amax, 448),
// code = cvt.rn.satfinite.e4m3(out * div.full(448, amax)).  The row maximum is order-independent,
// every other operation is per element, so codes and scales equal the reference's bit for bit.
//
// One CTA per (token, batch); a thread owns chunks of four consecutive d of one head.  HBM-bound:
// splits * (4 * BLOCK_D + 8) bytes in per (head, token), head_dim * (1 + sizeof(O)) bytes out.
#include <cuda_runtime.h>

#include "../../include/iflb200.h"
#include "launch.cuh"
#include "rowmath.cuh"

namespace iflb200 {

constexpr int kCombineThreads = 256;
constexpr int kCombineIters = 8;  // 256 threads x 8 chunks x 4 values = 8192 values per token row

struct CombineArgs {
  const float* po;
  const float* pm;
  const float* pl;
  void* o;
  int o_dtype;
  int64_t sob, sot, soh;
  uint8_t* q;
  int64_t ld_q;
  float* qs;
  int tokens, batch, group, heads_kv, head_dim, block_d, splits;
};

__device__ __forceinline__ float ex2_approx_ftz(float a) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(a));
  return r;
}

__global__ void __launch_bounds__(kCombineThreads) attn_combine_quant_kernel(const CombineArgs a) {
  grid_dependency_wait();  // the partials come from the kernel before this one in the stream
  grid_launch_dependents();
  __shared__ float red[kCombineThreads / 32];
  const int t = blockIdx.x, b = blockIdx.y;
  const int chunks_per_head = a.head_dim / 4;
  const int heads = a.group * a.heads_kv;
  const int total = heads * chunks_per_head;
  const int n_rows = a.tokens * a.group;
  float out[kCombineIters][4];
  float amax = 0.0f;
#pragma unroll
  for (int it = 0; it < kCombineIters; ++it) {
    const int c = it * kCombineThreads + threadIdx.x;
#pragma unroll
    for (int i = 0; i < 4; ++i) out[it][i] = 0.0f;
    if (c < total) {
      const int head = c / chunks_per_head, d = (c - head * chunks_per_head) * 4;
      const int kvh = head / a.group, h = head - kvh * a.group;
      const int64_t row = (int64_t)t * a.group + h;
      float m = __uint_as_float(0xFF800000u);  // -inf
      for (int sp = 0; sp < a.splits; ++sp) {
        const int64_t base = (((int64_t)sp * a.batch + b) * a.heads_kv + kvh) * n_rows + row;
        m = max_f32(m, __ldg(a.pm + base));
      }
      float l = 0.0f, acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      for (int sp = 0; sp < a.splits; ++sp) {
        const int64_t base = (((int64_t)sp * a.batch + b) * a.heads_kv + kvh) * n_rows + row;
        const float w = ex2_approx_ftz(__fsub_rn(__ldg(a.pm + base), m));
        l = __fmaf_rn(w, __ldg(a.pl + base), l);
        const float4 v = __ldg(reinterpret_cast<const float4*>(a.po + base * a.block_d + d));
        acc[0] = __fmaf_rn(w, v.x, acc[0]);
        acc[1] = __fmaf_rn(w, v.y, acc[1]);
        acc[2] = __fmaf_rn(w, v.z, acc[2]);
        acc[3] = __fmaf_rn(w, v.w, acc[3]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        out[it][i] = div_full(acc[i], l);
        amax = max_f32(amax, fabsf(out[it][i]));
      }
      if (a.o) {
        const int64_t off = (int64_t)b * a.sob + (int64_t)t * a.sot + (int64_t)head * a.soh + d;
        if (a.o_dtype == IFLB200_F32) {
          *reinterpret_cast<float4*>(reinterpret_cast<float*>(a.o) + off) =
              make_float4(out[it][0], out[it][1], out[it][2], out[it][3]);
        } else if (a.o_dtype == IFLB200_F16) {
          uint2 u;
          u.x = f32_to_f16_bits(out[it][0]) | (f32_to_f16_bits(out[it][1]) << 16);
          u.y = f32_to_f16_bits(out[it][2]) | (f32_to_f16_bits(out[it][3]) << 16);
          *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(a.o) + off) = u;
        } else {
          uint2 u;
          u.x = f32_to_bf16_bits(out[it][0]) | (f32_to_bf16_bits(out[it][1]) << 16);
          u.y = f32_to_bf16_bits(out[it][2]) | (f32_to_bf16_bits(out[it][3]) << 16);
          *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(a.o) + off) = u;
        }
      }
    }
  }
  if (!a.q) return;  // merge only (uniform)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = max_f32(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < kCombineThreads / 32; ++i) amax = max_f32(amax, red[i]);
  float scale, inv;
  quant_scales(amax, scale, inv);
  if (threadIdx.x == 0) a.qs[t] = scale;
  uint8_t* qr = a.q + (int64_t)t * a.ld_q;
#pragma unroll
  for (int it = 0; it < kCombineIters; ++it) {
    const int c = it * kCombineThreads + threadIdx.x;
    if (c < total) {
      const int head = c / chunks_per_head, d = (c - head * chunks_per_head) * 4;
      *reinterpret_cast<uint32_t*>(qr + (int64_t)head * a.head_dim + d) =
          cvt_e4m3x4(__fmul_rn(out[it][0], inv), __fmul_rn(out[it][1], inv), __fmul_rn(out[it][2], inv),
                     __fmul_rn(out[it][3], inv));
    }
  }
}

}  // namespace iflb200

using namespace iflb200;

extern "C" int iflb200_attn_combine_quant(const float* po, const float* pm, const float* pl, int splits, int batch,
                                          int tokens, int heads_q, int heads_kv, int head_dim, void* o, int o_dtype,
                                          int64_t o_stride_b, int64_t o_stride_t, int64_t o_stride_h, void* q,
                                          int64_t ld_q, float* qs, void* stream) {
  if (splits < 0 || batch < 0 || tokens < 0 || heads_q <= 0 || heads_kv <= 0 || head_dim <= 0) return IFLB200_ERR_ARG;
  if (splits == 0 || batch == 0 || tokens == 0) return IFLB200_OK;
  if (!po || !pm || !pl || (!o && !q) || (q && !qs)) return IFLB200_ERR_ARG;
  if (heads_q % heads_kv || head_dim % 4 || head_dim > 512) return IFLB200_ERR_SHAPE;
  if ((int64_t)heads_q * head_dim > (int64_t)kCombineThreads * kCombineIters * 4) return IFLB200_ERR_SHAPE;
  if (q && batch != 1) return IFLB200_ERR_SHAPE;  // as the reference: the quantised row is indexed by token alone
  if (o && o_dtype != IFLB200_F32 && o_dtype != IFLB200_F16 && o_dtype != IFLB200_BF16) return IFLB200_ERR_DTYPE;
  if (q && ld_q < (int64_t)heads_q * head_dim) return IFLB200_ERR_ARG;
  const int es = (o_dtype == IFLB200_F32) ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(po) & 15) || (q && ((reinterpret_cast<uintptr_t>(q) & 3) || ld_q % 4)) ||
      (o && ((reinterpret_cast<uintptr_t>(o) % (4 * es)) || (o_stride_b * es) % (4 * es) || (o_stride_t * es) % (4 * es) ||
             (o_stride_h * es) % (4 * es))))
    return IFLB200_ERR_ALIGN;
  int block_d = 1;
  while (block_d < head_dim) block_d <<= 1;
  CombineArgs a;
  a.po = po; a.pm = pm; a.pl = pl;
  a.o = o; a.o_dtype = o_dtype; a.sob = o_stride_b; a.sot = o_stride_t; a.soh = o_stride_h;
  a.q = reinterpret_cast<uint8_t*>(q); a.ld_q = ld_q; a.qs = qs;
  a.tokens = tokens; a.batch = batch; a.group = heads_q / heads_kv; a.heads_kv = heads_kv;
  a.head_dim = head_dim; a.block_d = block_d; a.splits = splits;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const cudaError_t e = launch_dep(attn_combine_quant_kernel, dim3(tokens, batch), dim3(kCombineThreads), 0, s, 1,
                                   dependent_launch_for(tokens), a);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}
