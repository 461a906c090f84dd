// Element-wise arithmetic shared by the row kernels and the GEMM epilogues.  Every operation
// is an explicitly rounded fp32 instruction in the order the reference's Triton kernels
// compile to for sm_100 (instinctflash/kernels/norm.py:44-80,135-147,168-175 and
// instinctflash/kernels/activation.py:26-43): a multiply that feeds an add is contracted
// into one fma.rn, every other multiply and add rounds on its own.
#pragma once
#include "ptx.cuh"

namespace iflb200 {

// Two fp32 lanes in one 64-bit register for the packed add / mul / fma of sm_100 (each lane
// rounds exactly like the scalar instruction, so results are unchanged; the instruction count of
// the issue-bound row kernels is what they halve).
__device__ __forceinline__ uint64_t pack2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}

// A value with at most one multiplication not yet rounded, so that a following add can be
// contracted with it:  x*a*b + c  ->  fma(mul(x, a), b, c).
struct Chain {
  float v;
  float p;
  bool pending;
  __device__ __forceinline__ explicit Chain(float x) : v(x), p(1.0f), pending(false) {}
  __device__ __forceinline__ void mul(float f) {
    if (pending) v = __fmul_rn(v, p);
    p = f;
    pending = true;
  }
  __device__ __forceinline__ void add(float c) {
    if (pending) {
      v = __fmaf_rn(v, p, c);
      pending = false;
    } else {
      v = __fadd_rn(v, c);
    }
  }
  __device__ __forceinline__ float done() {
    if (pending) {
      v = __fmul_rn(v, p);
      pending = false;
    }
    return v;
  }
};

// The same for the eight elements of a chunk at once.  Which operations exist is decided by
// kernel arguments, the same for every element, so `pending` is uniform: the compiler emits
// one uniform branch per stage and chunk instead of selects per element.
struct Chain8 {
  float v[8];
  float p[8];
  bool pending;
  __device__ __forceinline__ explicit Chain8(const float (&x)[8]) : pending(false) {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = x[i];
  }
  __device__ __forceinline__ void flush() {
    if (pending) {
#pragma unroll
      for (int i = 0; i < 8; i += 2) unpack2(mul2(pack2(v[i], v[i + 1]), pack2(p[i], p[i + 1])), v[i], v[i + 1]);
    }
  }
  __device__ __forceinline__ void mul(const float (&f)[8]) {
    flush();
#pragma unroll
    for (int i = 0; i < 8; ++i) p[i] = f[i];
    pending = true;
  }
  __device__ __forceinline__ void mul(float f) {
    flush();
#pragma unroll
    for (int i = 0; i < 8; ++i) p[i] = f;
    pending = true;
  }
  __device__ __forceinline__ void add(const float (&c)[8]) {
    if (pending) {
#pragma unroll
      for (int i = 0; i < 8; i += 2)
        unpack2(fma2(pack2(v[i], v[i + 1]), pack2(p[i], p[i + 1]), pack2(c[i], c[i + 1])), v[i], v[i + 1]);
      pending = false;
    } else {
#pragma unroll
      for (int i = 0; i < 8; i += 2) unpack2(add2(pack2(v[i], v[i + 1]), pack2(c[i], c[i + 1])), v[i], v[i + 1]);
    }
  }
  __device__ __forceinline__ void done(float (&out)[8]) {
    flush();
    pending = false;
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = v[i];
  }
};

// gelu_pytorch_tanh as written in the reference: 0.5*v*(1 + (2/(1+exp(-2*inner)) - 1)),
// inner = 0.79788456*(v + 0.044715*v^3), with exp lowered to ex2.approx and the division to
// div.full (instinctflash/kernels/norm.py:143-145, instinctflash/kernels/activation.py:35-37).
__device__ __forceinline__ float gelu_tanh_ref(float v) {
  const float a1 = __fmul_rn(v, __uint_as_float(0x3D372713u));  // 0.044715
  const float a2 = __fmul_rn(v, a1);
  const float t = __fmaf_rn(v, a2, v);
  const float inner = __fmul_rn(t, __uint_as_float(0x3F4C422Au));  // 0.7978846
  const float half = __fmul_rn(v, 0.5f);
  const float m2 = __fmul_rn(inner, -2.0f);
  const float z = __fmul_rn(m2, __uint_as_float(0x3FB8AA3Bu));  // log2(e)
  const float e = ex2_approx(z);
  const float den = __fadd_rn(e, 1.0f);
  const float d = div_full(2.0f, den);
  const float s1 = __fadd_rn(d, -1.0f);
  const float s2 = __fadd_rn(s1, 1.0f);
  return __fmul_rn(half, s2);
}

// The same for two elements, with the packed instructions.
__device__ __forceinline__ void gelu_tanh_ref2(float& x0, float& x1) {
  const uint64_t v = pack2(x0, x1);
  const float k1 = __uint_as_float(0x3D372713u), k2 = __uint_as_float(0x3F4C422Au), kl = __uint_as_float(0x3FB8AA3Bu);
  const uint64_t a1 = mul2(v, pack2(k1, k1));
  const uint64_t a2 = mul2(v, a1);
  const uint64_t t = fma2(v, a2, v);
  const uint64_t inner = mul2(t, pack2(k2, k2));
  const uint64_t half = mul2(v, pack2(0.5f, 0.5f));
  const uint64_t m2 = mul2(inner, pack2(-2.0f, -2.0f));
  const uint64_t z = mul2(m2, pack2(kl, kl));
  float z0, z1;
  unpack2(z, z0, z1);
  const uint64_t den = add2(pack2(ex2_approx(z0), ex2_approx(z1)), pack2(1.0f, 1.0f));
  float d0, d1;
  unpack2(den, d0, d1);
  const uint64_t s1 = add2(pack2(div_full(2.0f, d0), div_full(2.0f, d1)), pack2(-1.0f, -1.0f));
  const uint64_t s2 = add2(s1, pack2(1.0f, 1.0f));
  unpack2(mul2(half, s2), x0, x1);
}

// silu as written in the reference: g / (1 + exp(-g)).
__device__ __forceinline__ float silu_ref(float g) {
  const float z = __fmul_rn(-g, __uint_as_float(0x3FB8AA3Bu));
  const float e = ex2_approx(z);
  return div_full(g, __fadd_rn(e, 1.0f));
}

// Tail of every producer: row maximum floored at 1e-8, the dequantisation scale and the
// multiplier applied before the e4m3 cast, both by div.full.f32.
__device__ __forceinline__ void quant_scales(float amax, float& scale, float& inv) {
  amax = max_f32(amax, __uint_as_float(0x322BCC77u));
  scale = div_full(amax, 448.0f);
  inv = div_full(448.0f, amax);
}

__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ float to_f32(__half x) { return __half2float(x); }
__device__ __forceinline__ float to_f32(float x) { return x; }

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t b) { return __uint_as_float(b << 16); }

// fp32 -> bf16 round-to-nearest-even, as bits (NaN kept quiet).
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float f) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f));
}
__device__ __forceinline__ uint32_t f32_to_f16_bits(float f) {
  return (uint32_t)__half_as_ushort(__float2half_rn(f));
}

}  // namespace iflb200
