/*
 * CPU restatement of the reference's FP8 linear path.  TEST INFRASTRUCTURE ONLY: the checker
 * for tests/, the smoke check and the CPU-baseline leg of bench.py; the product never calls it.
 *
 * Each function restates one operator of the InstinctFlash reference, element by element, in
 * the fp32 instruction order its Triton kernel compiles to for sm_100 (a multiply feeding an
 * add is one fmaf; every other multiply/add rounds on its own):
 *   oracle_row_quant            instinctflash/kernels/norm.py:128-147
 *   oracle_dequant_rows         instinctflash/kernels/norm.py:162-175
 *   oracle_gated_act_quant      instinctflash/kernels/activation.py:20-43
 *   oracle_residual_norm_quant  instinctflash/kernels/norm.py:26-94 (no router)
 *   oracle_gemm_raw             instinctflash/kernels/fp8.py:50-53
 *   oracle_fp8_linear           fp8.py:50-53 + norm.py:162-175 (and the exact-rounding form)
 *   oracle_pack_tensor          instinctflash/runtime/fp8_pack.py:27-92
 *   oracle_e4m3_encode          instinctflash/runtime/fp8_pack.py:12-23 (integer RNE cast)
 *   oracle_qkv_split            instinctflash/kernels/rope.py:22-83
 *   oracle_wan_qkv              instinctflash/kernels/wan.py:20-82
 *   oracle_attn_combine_quant   instinctflash/kernels/attention.py:109-145
 *
 * Known, documented differences from the GPU reference: the GPU uses the approximate PTX
 * instructions div.full.f32, ex2.approx.f32 and rsqrt.approx.ftz.f32; here they are IEEE
 * division, exp2f and 1/sqrtf.  A quantiser scale can therefore differ from the GPU's by one
 * ulp on some rows and a code by one step at a rounding boundary; tests that compare the GPU
 * kernels with this oracle allow exactly that and count it, while the bit-exact comparison is
 * made against vectors recorded from the reference's own kernels on a B200 (tests/golden).
 * The row sums of the normalisation are accumulated in double here (the GPU order is
 * layout-specific), so normalised outputs are tolerance-class by construction.  The rotary
 * consumers take sine and cosine from the C library where the GPU has its own single-precision
 * routines (both within a few ulp of the true value): rotated outputs are tolerance-class too.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ scalar formats */
static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

static inline float bf16_round(float f) {
  uint32_t u = f2u(f);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return u2f(u | 0x00400000u);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return u2f(u & 0xFFFF0000u);
}
static inline float f16_round(float f) { return (float)(_Float16)f; }
static inline float round_to(float f, int dtype) {
  return dtype == 1 ? bf16_round(f) : dtype == 2 ? f16_round(f) : f;
}

static float e4m3_table[256];
static int e4m3_table_ready = 0;
static void e4m3_init(void) {
  if (e4m3_table_ready) return;
  for (int c = 0; c < 256; ++c) {
    const int e = (c >> 3) & 15, m = c & 7;
    float v;
    if (e == 15 && m == 7) v = NAN;
    else if (e == 0) v = ldexpf((float)m, -9);
    else v = ldexpf(1.0f + (float)m / 8.0f, e - 7);
    e4m3_table[c] = (c & 0x80) ? -v : v;
  }
  e4m3_table_ready = 1;
}

/* fp32 -> e4m3fn, round to nearest even, saturating to +-448, NaN -> 0x7F|sign
 * (cvt.rn.satfinite.e4m3x2.f32).  Integer restatement. */
ORACLE_API uint8_t oracle_e4m3_encode(float value) {
  const uint32_t bits = f2u(value);
  const uint32_t mag = bits & 0x7FFFFFFFu;
  const uint8_t sign = (uint8_t)((bits >> 24) & 0x80u);
  uint32_t code;
  if (mag > 0x7F800000u) return (uint8_t)(sign | 0x7F);
  if (mag >= 0x43E00000u) {            /* >= 448 (incl. inf): saturate */
    code = 0x7E;
  } else if (mag < (121u << 23)) {     /* below 2^-6: subnormal, one step = 2^-9 */
    const float a = u2f(mag) + 16384.0f; /* 2^14: one fp32 ulp there is 2^-9, RNE by the add */
    code = f2u(a) - (141u << 23);
  } else {
    code = ((mag + 0x7FFFFu + ((mag >> 20) & 1u)) >> 20) - 960u;
    if (code > 0x7E) code = 0x7E;
  }
  return (uint8_t)(sign | code);
}
ORACLE_API float oracle_e4m3_decode(uint8_t code) { e4m3_init(); return e4m3_table[code]; }

/* ------------------------------------------------------------------ op chain */
typedef struct { float v, p; int pending; } chain_t;
static inline void ch_init(chain_t* c, float x) { c->v = x; c->p = 1.0f; c->pending = 0; }
static inline void ch_mul(chain_t* c, float f) {
  if (c->pending) c->v = c->v * c->p;
  c->p = f; c->pending = 1;
}
static inline void ch_add(chain_t* c, float a) {
  if (c->pending) { c->v = fmaf(c->v, c->p, a); c->pending = 0; }
  else c->v = c->v + a;
}
static inline float ch_done(chain_t* c) {
  if (c->pending) { c->v = c->v * c->p; c->pending = 0; }
  return c->v;
}

static inline float gelu_tanh_ref(float v) {
  const float a1 = v * u2f(0x3D372713u);
  const float a2 = v * a1;
  const float t = fmaf(v, a2, v);
  const float inner = t * u2f(0x3F4C422Au);
  const float half = v * 0.5f;
  const float m2 = inner * -2.0f;
  const float z = m2 * u2f(0x3FB8AA3Bu);
  const float e = exp2f(z);
  const float den = e + 1.0f;
  const float d = 2.0f / den;
  const float s1 = d + -1.0f;
  const float s2 = s1 + 1.0f;
  return half * s2;
}
static inline float silu_ref(float g) {
  const float z = -g * u2f(0x3FB8AA3Bu);
  const float e = exp2f(z);
  return g / (e + 1.0f);
}

/* max.f32 semantics: a NaN operand is ignored */
static inline float max_nn(float a, float b) { return (b != b) ? a : (a != a) ? b : (a > b ? a : b); }

static void quant_tail(const float* h, int K, uint8_t* q, float* qs) {
  float amax = 0.0f;
  for (int k = 0; k < K; ++k) amax = max_nn(amax, fabsf(h[k]));
  amax = max_nn(amax, u2f(0x322BCC77u));
  *qs = amax / 448.0f;
  const float inv = 448.0f / amax;
  for (int k = 0; k < K; ++k) q[k] = oracle_e4m3_encode(h[k] * inv);
}

/* ------------------------------------------------------------------ operators */
/* x: [M,K] fp32 (already widened from its storage type), ld in elements */
ORACLE_API void oracle_row_quant(const float* x, int64_t ld_x, int M, int K, const float* row,
                                 const float* col, const float* bias, int gelu, uint8_t* q,
                                 int64_t ld_q, float* qs) {
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m) {
    float* h = (float*)malloc(sizeof(float) * (size_t)K);
    for (int k = 0; k < K; ++k) {
      chain_t c; ch_init(&c, x[m * ld_x + k]);
      if (row) ch_mul(&c, row[m]);
      if (col) ch_mul(&c, col[k]);
      if (bias) ch_add(&c, bias[k]);
      float v = ch_done(&c);
      if (gelu) v = gelu_tanh_ref(v);
      h[k] = v;
    }
    quant_tail(h, K, q + m * ld_q, qs + m);
    free(h);
  }
}

/* The two phases of the quantiser for column-sharded rows (tensor parallel): phase 1 returns
 * the local row maxima of |v|, phase 2 quantises with maxima supplied by the caller (the
 * all-reduce-max over the shards).  v is the same prologue chain as oracle_row_quant. */
ORACLE_API void oracle_row_quant_sharded(const float* x, int64_t ld_x, int M, int K, const float* row,
                                         const float* col, const float* bias, int gelu, int phase,
                                         float* amax_io, uint8_t* q, int64_t ld_q, float* qs) {
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m) {
    float* h = (float*)malloc(sizeof(float) * (size_t)K);
    float amax = 0.0f;
    for (int k = 0; k < K; ++k) {
      chain_t c; ch_init(&c, x[m * ld_x + k]);
      if (row) ch_mul(&c, row[m]);
      if (col) ch_mul(&c, col[k]);
      if (bias) ch_add(&c, bias[k]);
      float v = ch_done(&c);
      if (gelu) v = gelu_tanh_ref(v);
      h[k] = v;
      amax = max_nn(amax, fabsf(v));
    }
    if (phase == 1) {
      amax_io[m] = amax;
    } else {
      float a = max_nn(amax_io[m], u2f(0x322BCC77u));
      qs[m] = a / 448.0f;
      const float inv = 448.0f / a;
      for (int k = 0; k < K; ++k) q[m * ld_q + k] = oracle_e4m3_encode(h[k] * inv);
    }
    free(h);
  }
}

ORACLE_API void oracle_dequant_rows(const float* x, int64_t ld_x, int M, int D, const float* row,
                                    const float* col, const float* bias, float* y, int64_t ld_y,
                                    int y_dtype) {
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < D; ++n) {
      chain_t c; ch_init(&c, x[m * ld_x + n]);
      if (row) ch_mul(&c, row[m]);
      if (col) ch_mul(&c, col[n]);
      if (bias) ch_add(&c, bias[n]);
      y[m * ld_y + n] = round_to(ch_done(&c), y_dtype);
    }
}

ORACLE_API void oracle_gated_act_quant(const float* gu, int64_t ld_gu, int M, int F, const float* row,
                                       const float* col, int act, uint8_t* q, int64_t ld_q, float* qs) {
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m) {
    float* h = (float*)malloc(sizeof(float) * (size_t)F);
    for (int k = 0; k < F; ++k) {
      float g = gu[m * ld_gu + k], u = gu[m * ld_gu + F + k];
      if (row) { g = g * row[m]; u = u * row[m]; }
      if (col) { g = g * col[k]; u = u * col[F + k]; }
      const float a = act == 0 ? gelu_tanh_ref(g) : silu_ref(g);
      h[k] = u * a;
    }
    quant_tail(h, F, q + m * ld_q, qs + m);
    free(h);
  }
}

/* res: [M,D] fp32 holding the residual values (widened); res_dtype says how a stored value
 * rounds (0 fp32, 1 bf16).  Outputs: res (updated when delta && write_res), y (optional,
 * rounded to y_dtype), q/qs (optional). */
ORACLE_API void oracle_residual_norm_quant(float* res, int64_t ld_res, int res_dtype, int M, int D,
                                           const float* delta, int64_t ld_delta, const float* drow,
                                           const float* dcol, const float* bias, const float* gate,
                                           int write_res, int layernorm, const float* weight,
                                           const float* beta, const float* mod_scale,
                                           const float* mod_shift, const int32_t* mod_index, float eps,
                                           uint8_t* q, int64_t ld_q, float* qs, float* y, int64_t ld_y,
                                           int y_dtype) {
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m) {
    float* x = (float*)malloc(sizeof(float) * (size_t)D);
    const int64_t mofs = mod_index ? (int64_t)mod_index[m] * D : 0;
    for (int n = 0; n < D; ++n) {
      float v = res[m * ld_res + n];
      if (delta) {
        chain_t c; ch_init(&c, delta[m * ld_delta + n]);
        if (drow) ch_mul(&c, drow[m]);
        if (dcol) ch_mul(&c, dcol[n]);
        if (bias) ch_add(&c, bias[n]);
        if (gate) ch_mul(&c, gate[mofs + n]);
        ch_add(&c, v);
        v = ch_done(&c);
        if (write_res) { v = round_to(v, res_dtype); res[m * ld_res + n] = v; }
      }
      x[n] = v;
    }
    if (q || y) {
      double s = 0.0, ss = 0.0;
      float mean = 0.0f;
      if (layernorm) {
        for (int n = 0; n < D; ++n) s += x[n];
        mean = (float)s / (float)D;
        for (int n = 0; n < D; ++n) { x[n] = x[n] - mean; ss += (double)x[n] * x[n]; }
      } else {
        for (int n = 0; n < D; ++n) ss += (double)x[n] * x[n];
      }
      const float var = (float)ss / (float)D;
      const float rstd = 1.0f / sqrtf(var + eps);
      for (int n = 0; n < D; ++n) {
        chain_t c; ch_init(&c, x[n]);
        ch_mul(&c, rstd);
        if (weight) ch_mul(&c, weight[n]);
        if (beta) ch_add(&c, beta[n]);
        if (mod_scale) { ch_mul(&c, mod_scale[mofs + n] + 1.0f); ch_add(&c, mod_shift[mofs + n]); }
        x[n] = ch_done(&c);
        if (y) y[m * ld_y + n] = round_to(x[n], y_dtype);
      }
      if (q) quant_tail(x, D, q + m * ld_q, qs + m);
    }
    free(x);
  }
}

/* Exact accumulator: every e4m3 product is a multiple of 2^-18 below 2^18, so a double sum of
 * up to 2^15 of them is exact in any order. */
static void gemm_acc_row(const float* a, const float* w, int N, int K, int64_t ld_w, float* acc) {
  for (int n = 0; n < N; ++n) {
    const float* wr = w + n * ld_w;
    double s = 0.0;
#pragma omp simd reduction(+ : s)
    for (int k = 0; k < K; ++k) s += (double)(a[k] * wr[k]);
    acc[n] = (float)s;
  }
}

/* a: [M,K] codes, w: [N,K] codes; acc_out: [M,N] fp32 = fp32_rn(exact sum) */
ORACLE_API void oracle_gemm_acc(const uint8_t* a, int64_t ld_a, const uint8_t* w, int64_t ld_w, int M,
                                int N, int K, float* acc_out, int64_t ld_out) {
  e4m3_init();
  float* wf = (float*)malloc(sizeof(float) * (size_t)N * K);
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n)
    for (int k = 0; k < K; ++k) wf[(size_t)n * K + k] = e4m3_table[w[n * ld_w + k]];
#pragma omp parallel for schedule(dynamic, 1)
  for (int m = 0; m < M; ++m) {
    float* af = (float*)malloc(sizeof(float) * (size_t)K);
    for (int k = 0; k < K; ++k) af[k] = e4m3_table[a[m * ld_a + k]];
    gemm_acc_row(af, wf, N, K, K, acc_out + m * ld_out);
    free(af);
  }
  free(wf);
}

/* raw[M,N] = bf16_rn(acc), returned widened to fp32 */
ORACLE_API void oracle_gemm_raw(const uint8_t* a, int64_t ld_a, const uint8_t* w, int64_t ld_w, int M,
                                int N, int K, float* raw, int64_t ld_out) {
  oracle_gemm_acc(a, ld_a, w, ld_w, M, N, K, raw, ld_out);
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) raw[m * ld_out + n] = bf16_round(raw[m * ld_out + n]);
}

/* y = out_dtype(chain(r, row, col, bias)), r = bf16(acc) (exact == 0) or acc (exact == 1).
 * row_stride / col_stride 0 = one per-tensor scale. */
ORACLE_API void oracle_fp8_linear(const uint8_t* a, int64_t ld_a, const uint8_t* w, int64_t ld_w, int M,
                                  int N, int K, const float* row, int row_stride, const float* col,
                                  int col_stride, const float* bias, int exact, float* y, int64_t ld_y,
                                  int y_dtype) {
  oracle_gemm_acc(a, ld_a, w, ld_w, M, N, K, y, ld_y);
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      float r = y[m * ld_y + n];
      if (!exact) r = bf16_round(r);
      chain_t c; ch_init(&c, r);
      if (row) ch_mul(&c, row[(int64_t)m * row_stride]);
      if (col) ch_mul(&c, col[(int64_t)n * col_stride]);
      if (bias) ch_add(&c, bias[n]);
      y[m * ld_y + n] = round_to(ch_done(&c), y_dtype);
    }
}

/* Per-tensor recipe.  x: bf16 bit patterns.  dynamic != 0: scale computed from x (NaN
 * propagates) and written to *scale; else *scale is the input. */
ORACLE_API void oracle_pack_tensor(const uint16_t* x, int64_t n, int dynamic, float* scale, uint8_t* q) {
  if (dynamic) {
    float amax = 0.0f;
    int nan = 0;
    for (int64_t i = 0; i < n; ++i) {
      const float v = fabsf(u2f((uint32_t)x[i] << 16));
      if (v != v) nan = 1; else if (v > amax) amax = v;
    }
    const float floor_ = 1e-12f;
    *scale = nan ? NAN : (amax > floor_ ? amax : floor_) * (float)(1.0 / 448.0);
  }
  const float s = *scale;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    float d = u2f((uint32_t)x[i] << 16) / s;
    if (d == d) d = d < -448.0f ? -448.0f : (d > 448.0f ? 448.0f : d);
    q[i] = oracle_e4m3_encode(d);
  }
}

/* ------------------------------------------------------------------ QKV consumers */
static inline float rms_scale(double sum_sq, int n, float eps) {
  const float mean = (float)sum_sq / (float)n;
  return 1.0f / sqrtf(mean + eps);
}

/* (a, b) <- (a cos - b sin, b cos + a sin); the sine products are rounded, the cosine products
 * fused, as the reference's kernels compile (rope.py:67-69, wan.py:41-43). */
static inline void rotate_pair(float* a, float* b, float cs, float sn) {
  const float bs = *b * sn, as = *a * sn;
  const float na = fmaf(*a, cs, -bs), nb = fmaf(*b, cs, as);
  *a = na; *b = nb;
}

static inline float dequant_elem(float raw, const float* row_scale, const float* col, const float* bias,
                                 int64_t c) {
  chain_t ch; ch_init(&ch, raw);
  if (row_scale) ch_mul(&ch, *row_scale);
  if (col) ch_mul(&ch, col[c]);
  if (bias) ch_add(&ch, bias[c]);
  return ch_done(&ch);
}

/* instinctflash/kernels/rope.py:22-83.  qkv [T, (HQ+2*HKV)*HD] fp32 (widened); q [T,HQ,HD],
 * k/v [S,HKV,HD] dense fp32 holding values rounded to out_dtype; rows kv_base + t written. */
ORACLE_API void oracle_qkv_split(const float* qkv, int64_t ld, int T, int HQ, int HKV, int HD,
                                 const float* row, const float* col, const float* bias,
                                 const float* q_norm, const float* k_norm, float eps,
                                 const float* inv_freq, const float* pos, int64_t ld_pos,
                                 const int32_t* sections, int kv_base, float* q, float* k, float* v,
                                 int out_dtype) {
  const int half = HD / 2, heads = HQ + 2 * HKV;
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; ++t) {
    float* x = (float*)malloc(sizeof(float) * (size_t)HD);
    for (int h = 0; h < heads; ++h) {
      const float* src = qkv + (int64_t)t * ld + (int64_t)h * HD;
      for (int i = 0; i < HD; ++i)
        x[i] = dequant_elem(src[i], row ? row + t : NULL, col, bias, (int64_t)h * HD + i);
      if (h < HQ + HKV) {
        const float* nw = h < HQ ? q_norm : k_norm;
        if (nw) {
          double ss = 0.0;
          for (int i = 0; i < HD; ++i) ss += (double)x[i] * x[i];
          const float rs = rms_scale(ss, HD, eps);
          for (int i = 0; i < HD; ++i) x[i] = (x[i] * rs) * nw[i];
        }
        if (inv_freq) {
          for (int i = 0; i < half; ++i) {
            const float ang = pos[(int64_t)t * ld_pos + (sections ? sections[i] : 0)] * inv_freq[i];
            rotate_pair(&x[i], &x[half + i], cosf(ang), sinf(ang));
          }
        }
      }
      float* dst;
      if (h < HQ) dst = q + ((int64_t)t * HQ + h) * HD;
      else if (h < HQ + HKV) dst = k + ((int64_t)(kv_base + t) * HKV + (h - HQ)) * HD;
      else dst = v + ((int64_t)(kv_base + t) * HKV + (h - HQ - HKV)) * HD;
      for (int i = 0; i < HD; ++i) dst[i] = round_to(x[i], out_dtype);
    }
    free(x);
  }
}

/* instinctflash/kernels/wan.py:20-82.  raw [rows, parts*D] fp32; q [rows, D]; pools [B, S, D]
 * dense fp32 (values rounded to out_dtype), written at pool[row / tokens, slots[row % tokens]]. */
ORACLE_API void oracle_wan_qkv(const float* raw, int64_t ld, int rows, int tokens, int H, int HD, int parts,
                               const float* row, const float* col, const float* bias,
                               const float* q_norm, const float* k_norm, float eps,
                               const float* inv_freq, const float* pos, int64_t ld_pos,
                               const int32_t* sections, const int32_t* slots, int S, float* q,
                               float* kp, float* vp, int out_dtype) {
  const int D = H * HD, half = HD / 2;
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    float* x = (float*)malloc(sizeof(float) * (size_t)D);
    const int b = r / tokens, t = r % tokens;
    for (int part = 0; part < parts; ++part) {
      const int64_t col0 = (int64_t)part * D;
      const float* src = raw + (int64_t)r * ld + col0;
      for (int d = 0; d < D; ++d)
        x[d] = dequant_elem(src[d], row ? row + r : NULL, col ? col + col0 : NULL, bias ? bias + col0 : NULL, d);
      const float* nw = part == 0 ? q_norm : (part == 1 ? k_norm : NULL);
      if (nw) {
        double ss = 0.0;
        for (int d = 0; d < D; ++d) ss += (double)x[d] * x[d];
        const float rs = rms_scale(ss, D, eps);
        for (int d = 0; d < D; ++d) x[d] = (x[d] * rs) * nw[d];
      }
      if (inv_freq && part < 2) {
        for (int h = 0; h < H; ++h)
          for (int j = 0; j < half; ++j) {
            const float ang = pos[(int64_t)t * ld_pos + sections[j]] * inv_freq[j];
            rotate_pair(&x[h * HD + 2 * j], &x[h * HD + 2 * j + 1], cosf(ang), sinf(ang));
          }
      }
      const int slot = slots ? slots[t] : t;
      float* dst = part == 0 ? q + (int64_t)r * D
                             : (part == 1 ? kp : vp) + ((int64_t)b * S + slot) * D;
      for (int d = 0; d < D; ++d) dst[d] = round_to(x[d], out_dtype);
    }
    free(x);
  }
}

/* Merge of split-KV attention partials and the per-token quantiser of the merged row
 * (instinctflash/kernels/attention.py:109-145).  po [splits, batch, hkv, n_rows, block_d],
 * pm / pl [splits, batch, hkv, n_rows], n_rows = tokens * group, query row = t * group + h.
 * out [batch, tokens, heads_q, head_dim] receives the merged values in fp32 (the caller rounds
 * them to the output type); with q != NULL (batch 1) the token's full row is quantised with one
 * scale.  exp2f stands for the GPU's ex2.approx.ftz and '/' for div.full. */
ORACLE_API void oracle_attn_combine_quant(const float* po, const float* pm, const float* pl, int splits, int batch,
                                          int tokens, int heads_q, int heads_kv, int head_dim, int block_d,
                                          float* out, uint8_t* q, int64_t ld_q, float* qs) {
  const int group = heads_q / heads_kv;
  const int64_t n_rows = (int64_t)tokens * group;
  for (int b = 0; b < batch; ++b) {
    for (int t = 0; t < tokens; ++t) {
      float* orow = out + ((int64_t)b * tokens + t) * heads_q * head_dim;
      for (int head = 0; head < heads_q; ++head) {
        const int kvh = head / group, h = head % group;
        const int64_t row = (int64_t)t * group + h;
        float m = -INFINITY;
        for (int sp = 0; sp < splits; ++sp)
          m = max_nn(m, pm[(((int64_t)sp * batch + b) * heads_kv + kvh) * n_rows + row]);
        for (int d = 0; d < head_dim; ++d) {
          float l = 0.0f, acc = 0.0f;
          for (int sp = 0; sp < splits; ++sp) {
            const int64_t base = (((int64_t)sp * batch + b) * heads_kv + kvh) * n_rows + row;
            const float w = exp2f(pm[base] - m);
            l = fmaf(w, pl[base], l);
            acc = fmaf(w, po[base * block_d + d], acc);
          }
          orow[head * head_dim + d] = acc / l;
        }
      }
      if (q) quant_tail(orow, heads_q * head_dim, q + (int64_t)t * ld_q, qs + t);
    }
  }
}
