/*
 * iflb200 — C ABI of the B200 (sm_100a) FP8 linear path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle
 * (cudaStream_t passed as void*), enqueues work on that stream and returns at once
 * with an int status: 0 = ok, > 0 = a cudaError_t from the launch, < 0 = one of the
 * IFLB200_ERR_* codes below (argument rejected before any launch).  Nothing is
 * allocated, nothing synchronises, no host code reads device memory: every call can
 * be captured in a CUDA graph.  The caller owns every buffer.
 *
 * The comment on each declaration names the operator of the InstinctFlash reference
 * (path inside that project, line range) that the entry point replaces.
 *
 * Conventions
 *   - matrices are row-major with the last dimension contiguous; `ld_*` is the row
 *     stride in ELEMENTS;
 *   - e4m3 means the OCP "fn" variant (no infinities, 0x7F/0xFF = NaN, max 448);
 *   - aux vectors (row/col scales, bias, gate, norm weights) are float32;
 *   - optional pointers may be NULL.
 */
#ifndef IFLB200_H_
#define IFLB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define IFLB200_ABI_VERSION 1

#if defined(__GNUC__)
#define IFLB200_API __attribute__((visibility("default")))
#else
#define IFLB200_API
#endif

/* element types of activation-like buffers */
#define IFLB200_F32 0
#define IFLB200_BF16 1
#define IFLB200_F16 2

/* gated activations (instinctflash/kernels/activation.py:15-16) */
#define IFLB200_ACT_GELU_TANH 0
#define IFLB200_ACT_SILU 1

/* accumulator rounding of the fused GEMM epilogues */
#define IFLB200_ROUND_ENGINE 0 /* fp32 accumulator -> bf16 (RNE) -> fp32, then scales: the
                                  reference's gemm() + consumer memory round trip */
#define IFLB200_ROUND_EXACT 1  /* scales applied to the fp32 accumulator, one rounding */

/* status codes (< 0) */
#define IFLB200_OK 0
#define IFLB200_ERR_ARG (-1)       /* NULL where a pointer is required, negative size */
#define IFLB200_ERR_SHAPE (-2)     /* K or N not a multiple of 16, width above a kernel's maximum */
#define IFLB200_ERR_ALIGN (-3)     /* base pointer or row stride breaks the 16-byte rule */
#define IFLB200_ERR_DTYPE (-4)     /* element type code not supported by this entry point */
#define IFLB200_ERR_DRIVER (-5)    /* cuTensorMapEncodeTiled unavailable or refused the layout */
#define IFLB200_ERR_DEVICE (-6)    /* current device is not compute capability 10.x */
#define IFLB200_ERR_WORKSPACE (-7) /* workspace missing or too small */
#define IFLB200_ERR_TOO_LARGE (-8) /* input larger than the fixed capacity of a no-allocation entry point */

IFLB200_API int iflb200_abi_version(void);
IFLB200_API const char* iflb200_status_string(int status);

/*
 * Per-token (per-row) dynamic e4m3 quantiser with the optional consumer prologue.
 *   v[m,k]  = x[m,k] (*row[m]) (*col[k]) (+bias[k])  [-> gelu_tanh]
 *   amax    = max(max_k |v|, 1e-8);  qs[m] = amax / 448;  q[m,k] = e4m3(v * (448 / amax))
 * Both divisions are PTX div.full.f32, the cast is cvt.rn.satfinite, as the reference's
 * Triton kernel compiles to on sm_100.
 * Replaces: instinctflash/kernels/norm.py:128-158 (_row_quant_kernel, row_quant).
 */
IFLB200_API int iflb200_row_quant(const void* x, int x_dtype, int64_t ld_x, int M, int K,
                      const float* row, const float* col, const float* bias, int gelu,
                      void* q, int64_t ld_q, float* qs, void* stream);

/*
 * The quantiser for rows whose columns are sharded over several GPUs (tensor-parallel
 * column split).  Phase 1 writes each row's maximum of |v| over the LOCAL columns to amax[m]
 * and stops.  After an all-reduce-max of amax over the shards, phase 2 quantises the local
 * columns with the global maximum read from amax[m] and writes qs[m] and the codes: they are
 * bit-identical to the codes of the unsharded row.  (col and bias are the local slices.)
 * Phase 3 is phase 2 that also leaves amax[m] at zero afterwards: the second half of
 * iflb200_fp8_linear_gated, whose epilogue raises the maxima with atomicMax and needs the words
 * to start at zero again on the next call.
 * Extends instinctflash/kernels/norm.py:128-158, which is single-GPU; no reference counterpart
 * for the split itself.
 */
IFLB200_API int iflb200_row_quant_sharded(const void* x, int x_dtype, int64_t ld_x, int M, int K,
                              const float* row, const float* col, const float* bias, int gelu,
                              int phase, float* amax, void* q, int64_t ld_q, float* qs,
                              void* stream);

/*
 * Phase 1 of iflb200_row_quant_sharded that also writes the row maxima into up to 7 further
 * buffers: amax_mirrors is a HOST array of `mirrors` device pointers (the slots this rank owns in
 * the other GPUs' peer-mapped buffers), so the maxima need no separate transfer before the barrier
 * and the max over the ranks (iflb200_peer_exchange).  No reference counterpart.
 */
IFLB200_API int iflb200_row_max_sharded(const void* x, int x_dtype, int64_t ld_x, int M, int K,
                            const float* row, const float* col, const float* bias, int gelu,
                            float* amax, float* const* amax_mirrors, int mirrors, void* stream);

/*
 * Consumer of a raw accumulator: y[m,n] = out_dtype(x[m,n] (*row[m]) (*col[n]) (+bias[n])),
 * the last multiply fused with the bias add (fma.rn) exactly as the reference compiles.
 * Replaces: instinctflash/kernels/norm.py:162-185 (_dequant_rows_kernel, dequant_rows).
 */
IFLB200_API int iflb200_dequant_rows(const void* x, int x_dtype, int64_t ld_x, int M, int D,
                         const float* row, const float* col, const float* bias,
                         void* y, int y_dtype, int64_t ld_y, void* stream);

/*
 * Gated MLP activation on a raw accumulator [g | u] (each half F wide) followed by the
 * per-token quantiser:  h = act(g*row*col[:F]) * (u*row*col[F:]),  q/qs as in row_quant.
 * F <= 16384.
 * Replaces: instinctflash/kernels/activation.py:20-56 (_gated_act_quant_kernel, gated_act_quant).
 */
IFLB200_API int iflb200_gated_act_quant(const void* gu, int gu_dtype, int64_t ld_gu, int M, int F,
                            const float* row, const float* col, int act,
                            void* q, int64_t ld_q, float* qs, void* stream);

/*
 * Split of a raw fused QKV accumulator [Q heads | K heads | V heads] (head_dim wide each):
 * dequantisation (row, col, bias; each optional), per-head RMS norm of Q and K (q_norm and
 * k_norm [head_dim], both or neither), rotary embedding of Q and K with pairs (i, i + head_dim/2)
 * and angle pos[t, sections[i]] * inv_freq[i] (inv_freq null: no rotation; sections null:
 * column 0), and the store: Q at q_out[t, h], K and V at row kv_base + t of their caches, where
 * kv_base is read from the device when kv_base_dev is given.  Strides are in elements; pos is
 * a float32 table with row stride ld_pos.  head_dim even, <= 512.
 * Replaces: instinctflash/kernels/rope.py:22-114 (_qkv_split_kernel, qkv_split).
 */
IFLB200_API int iflb200_qkv_split(const void* qkv, int qkv_dtype, int64_t ld_qkv, int T, int heads_q,
                      int heads_kv, int head_dim, const float* row, const float* col,
                      const float* bias, const float* q_norm, const float* k_norm, float eps,
                      const float* inv_freq, const float* pos, int64_t ld_pos,
                      const int32_t* sections, const int32_t* kv_base_dev, int kv_base,
                      void* q_out, int64_t q_stride_t, int64_t q_stride_h,
                      void* k_out, int64_t k_stride_t, int64_t k_stride_h,
                      void* v_out, int64_t v_stride_t, int64_t v_stride_h, int out_dtype,
                      void* stream);

/*
 * Wan-DiT projection consumer on a raw accumulator [Q | K | V] (each heads*head_dim wide; K and
 * V present when their pools are given): dequantisation, RMS norm of Q and of K over the FULL
 * width (q_norm / k_norm [heads*head_dim], each optional), rotary embedding of adjacent pairs
 * (2j, 2j+1) of every head by pos[row % tokens, sections[j]] * inv_freq[j], dense store of Q
 * and scatter of K and V to pool[row / tokens, slots[row % tokens]] (slots null: the token).
 * heads*head_dim <= 8192, head_dim even, <= 512.
 * Replaces: instinctflash/kernels/wan.py:20-104 (_part, _wan_qkv_kernel, wan_qkv).
 */
IFLB200_API int iflb200_wan_qkv(const void* raw, int raw_dtype, int64_t ld_raw, int rows, int tokens,
                    int heads, int head_dim, const float* row, const float* col,
                    const float* bias, const float* q_norm, const float* k_norm, float eps,
                    const float* inv_freq, const float* pos, int64_t ld_pos,
                    const int32_t* sections, const int32_t* slots,
                    void* q_out, int64_t ld_q, void* k_pool, int64_t k_stride_b, int64_t k_stride_s,
                    void* v_pool, int64_t v_stride_b, int64_t v_stride_s, int out_dtype,
                    void* stream);

/*
 * Merge of split-KV attention partials and per-token e4m3 quantiser of the merged row (what feeds
 * the O projection).  po [splits, batch, heads_kv, tokens*group, block_d] float32 (block_d =
 * head_dim rounded up to a power of two), pm / pl [splits, batch, heads_kv, tokens*group] float32:
 * unnormalised outputs, running maxima (base-2 exponent domain) and running sums of the splits;
 * query row = token * group + head_in_group, group = heads_q / heads_kv.
 *   out = (sum_sp 2^(pm_sp - m) * po_sp) / (sum_sp 2^(pm_sp - m) * pl_sp),  m = max_sp pm_sp
 *   o[b, t, head, :] = o_dtype(out)                  (optional; strides in elements)
 *   qs[t] = max(max_{head,d} |out|, 1e-8) / 448;  q[t, head*head_dim + d] = e4m3(out * (448 / amax))
 * with the reference's instruction order (ex2.approx.ftz, fma chains in split order, div.full).
 * The quantised row is indexed by token alone: batch must be 1 when q is given, as in the
 * reference.  head_dim a multiple of 4, <= 512; heads_q*head_dim <= 8192.
 * Replaces: instinctflash/kernels/attention.py:109-145 (_attn_combine) and its launch at
 * :205-214.
 */
IFLB200_API int iflb200_attn_combine_quant(const float* po, const float* pm, const float* pl, int splits,
                               int batch, int tokens, int heads_q, int heads_kv, int head_dim,
                               void* o, int o_dtype, int64_t o_stride_b, int64_t o_stride_t,
                               int64_t o_stride_h, void* q, int64_t ld_q, float* qs, void* stream);

/*
 * Residual update + RMS/LayerNorm + affine + adaptive modulation + per-token quantiser,
 * one row per thread group (the MoE router tail of the reference kernel is not part of
 * this path).
 *   if delta: res[m] += (delta[m]*delta_row[m]*delta_col + bias) * gate[idx]   (stored in res's type)
 *   y = norm(res[m]) (*weight) (+beta);  y = y*(1+mod_scale[idx]) + mod_shift[idx]
 *   y_out[m] = y (optional);  q/qs[m] = quantiser(y) (optional)
 * gate / mod_scale / mod_shift are [D], or tables [n, D] indexed by mod_index[m] when given.
 * D <= 16384.  res_dtype is IFLB200_F32 or IFLB200_BF16; delta is bf16.
 * Replaces: instinctflash/kernels/norm.py:26-124 (_residual_norm_quant_kernel,
 * residual_norm_quant) without its `router` argument.
 */
IFLB200_API int iflb200_residual_norm_quant(void* res, int res_dtype, int64_t ld_res, int M, int D,
                                const void* delta, int64_t ld_delta,
                                const float* delta_row, const float* delta_col,
                                const float* bias, const float* gate, int write_res,
                                int layernorm, const float* weight, const float* beta,
                                const float* mod_scale, const float* mod_shift,
                                const int32_t* mod_index, float eps,
                                void* q, int64_t ld_q, float* qs,
                                void* y, int y_dtype, int64_t ld_y, void* stream);

/*
 * residual_norm_quant whose delta arrives as the fp32 partial sums of a K-split GEMM
 * (iflb200_gemm_fp8_partials): delta_partials [splits][M][ld_delta] float32, 1 <= splits <= 8.  The
 * planes are added in split order and the sum is rounded to bf16 -- the rounding point of the raw
 * accumulator -- before the chain of iflb200_residual_norm_quant runs on it.  D <= 8192, 16-byte
 * aligned rows.  Only the summation order of the accumulator differs from the unsplit sequence.
 * Extends instinctflash/kernels/norm.py:26-124 for split-K producers; no reference counterpart
 * for the split itself.
 */
IFLB200_API int iflb200_residual_norm_quant_partials(void* res, int res_dtype, int64_t ld_res, int M, int D,
                                const float* delta_partials, int splits, int64_t ld_delta,
                                const float* delta_row, const float* delta_col,
                                const float* bias, const float* gate, int write_res,
                                int layernorm, const float* weight, const float* beta,
                                const float* mod_scale, const float* mod_shift,
                                const int32_t* mod_index, float eps,
                                void* q, int64_t ld_q, float* qs,
                                void* y, int y_dtype, int64_t ld_y, void* stream);

/*
 * iflb200_residual_norm_quant_partials for the row owner of a tensor-parallel group: the planes are
 * the ranks' partial sums of this rank's rows (plane r written by rank r's
 * iflb200_gemm_fp8_rowblocks, summed in rank order: the reduce-scatter's sum at the same place
 * before the bf16 rounding), and the codes and row scales are also written into up to 7 further
 * buffers -- q_mirrors / qs_mirrors are HOST arrays of `mirrors` device pointers, the same rows of
 * the other GPUs' replicas of the next block's input (peer-mapped; row stride ld_q) -- from the
 * registers that hold them: the all-gather rides inside the kernel.  No `y` output.
 * No reference counterpart (the reference is single-GPU).
 */
IFLB200_API int iflb200_residual_norm_quant_peers(void* res, int res_dtype, int64_t ld_res, int M, int D,
                                const float* delta_partials, int splits, int64_t ld_delta,
                                const float* delta_row, const float* delta_col,
                                const float* bias, const float* gate, int write_res,
                                int layernorm, const float* weight, const float* beta,
                                const float* mod_scale, const float* mod_shift,
                                const int32_t* mod_index, float eps,
                                void* q, int64_t ld_q, float* qs,
                                void* const* q_mirrors, float* const* qs_mirrors, int mirrors,
                                void* stream);

/*
 * Raw-accumulator FP8 GEMM: out[M,N] (bf16) = bf16_rn(sum_k a[m,k] * w[n,k]), fp32
 * accumulation on the tcgen05 tensor cores, unit scales.  K, N multiples of 16.
 * Ordering on the stream (this and every other GEMM entry point): with dependent launch enabled
 * (iflb200_set_dependent_launch, the default) the kernel becomes resident while the kernel enqueued
 * immediately before it is still running and loads its first weight boxes before it waits for that
 * kernel; `a`, the scales and everything else are read
 * after the wait.  So `w` must not be an OUTPUT of the kernel enqueued immediately before on the
 * same stream (weights are packed at load time; activations may of course come from that kernel).
 * Replaces: instinctflash/kernels/fp8.py:50-53 (gemm -> torch._scaled_mm).
 */
IFLB200_API int iflb200_gemm_fp8_raw(const void* a, int64_t ld_a, const void* w, int64_t ld_w,
                         int M, int N, int K, void* out, int64_t ld_out, void* stream);

/*
 * Split-K for skinny activations (M <= 128): K is divided into `splits` ranges, each range of each
 * 64-column tile goes to its own CTA (tiles x splits CTAs, so that a deep reduction with few
 * output columns still uses the whole GPU), and every CTA writes its fp32 partial sums:
 *   out[s][m][n] = sum over the s-th K range of a[m,k] * w[n,k]       (no scales, no rounding)
 * The consumer (iflb200_residual_norm_quant_partials) adds the planes in split order, so the
 * result does not depend on timing.  K a multiple of 128; splits <= ceil(K / 512); `out` is
 * scratch owned by the caller, splits * M * ld_out floats.
 * Replaces: instinctflash/kernels/fp8.py:50-53 for the deep, narrow projections of the action
 * expert (instinctflash/engines/pi05/engine.py:244-250); the split has no reference counterpart.
 */
IFLB200_API int iflb200_gemm_fp8_partials(const void* a, int64_t ld_a, const void* w, int64_t ld_w,
                              int M, int N, int K, int splits, float* out, int64_t ld_out, void* stream);

/*
 * Fused linear: GEMM + the dequant_rows consumer in the epilogue.
 *   y[m,n] = out_dtype(fma(r*row_scale[m], col_scale[n], bias[n])),
 *   r = fp32(bf16_rn(acc)) in IFLB200_ROUND_ENGINE, r = acc in IFLB200_ROUND_EXACT.
 * row_scale_stride / col_scale_stride are 1 for per-token / per-channel vectors and 0
 * for a single per-tensor scale (the per-tensor recipe of torch_fp8_linear.py).  With
 * IFLB200_ROUND_EXACT and BOTH scales per-tensor the epilogue follows torch._scaled_mm's order,
 * y = out_dtype((acc * (row_scale * col_scale)) + bias) with every operation rounded on its own,
 * which reproduces that call's output bit for bit on B200.
 * Replaces: instinctflash/kernels/fp8.py:50-53 followed by
 * instinctflash/kernels/norm.py:162-185; with stride-0 scales and EXACT rounding also the
 * torch._scaled_mm call of instinctflash/runtime/torch_fp8_linear.py:74-78.
 */
IFLB200_API int iflb200_fp8_linear(const void* a, int64_t ld_a, const void* w, int64_t ld_w,
                       int M, int N, int K,
                       const float* row_scale, int row_scale_stride,
                       const float* col_scale, int col_scale_stride,
                       const void* bias, int bias_dtype, int rounding,
                       void* out, int out_dtype, int64_t ld_out, void* stream);

/*
 * Fused linear + residual update in the epilogue (in place on res):
 *   res[m,n] = res_dtype(res[m,n] + (r*row_scale[m]*col_scale[n] (+bias[n])) (*gate[idx[m],n]))
 * with the reference's contraction order (see residual_norm_quant).
 * Replaces: instinctflash/kernels/fp8.py:50-53 followed by the residual part of
 * instinctflash/kernels/norm.py:44-58.
 */
IFLB200_API int iflb200_fp8_linear_residual(const void* a, int64_t ld_a, const void* w, int64_t ld_w,
                                int M, int N, int K,
                                const float* row_scale, const float* col_scale,
                                const float* bias, const float* gate, const int32_t* gate_index,
                                void* res, int res_dtype, int64_t ld_res, void* stream);

/*
 * Fused linear + gated activation in the epilogue: w is the [2F, K] matrix [gate rows | up rows];
 * the kernel pairs the gate and up columns of the same hidden units in one tile and writes
 *   h[m,f] = (r_u*row_scale[m]*col_scale[F+f]) * act(r_g*row_scale[m]*col_scale[f])     (fp32)
 * with r_g, r_u the accumulators rounded to bf16 first (the reference's memory round trip) and
 * the reference's instruction order, and raises amax[m] (a non-negative float's bits, compared as
 * integers) to max_f |h[m,f]| with atomicMax.  amax[0..M) must be zero on entry;
 * iflb200_row_quant_sharded(h, IFLB200_F32, ..., phase 3, amax, q, qs) then writes exactly the
 * codes and scales of gated_act_quant and leaves amax at zero for the next call.  h is never
 * rounded to 16 bits, as in the reference.  F a multiple of 16.
 * Replaces: instinctflash/kernels/fp8.py:50-53 followed by the activation part of
 * instinctflash/kernels/activation.py:20-43 (the call pair at
 * instinctflash/engines/pi05/engine.py:210-212).
 */
IFLB200_API int iflb200_fp8_linear_gated(const void* a, int64_t ld_a, const void* w, int64_t ld_w,
                             int M, int F, int K, const float* row_scale, const float* col_scale,
                             int act, float* h, int64_t ld_h, uint32_t* amax, void* stream);

/*
 * The quantiser pass of iflb200_fp8_linear_gated as a flat kernel: q[m,f] = e4m3(h[m,f] * (448 /
 * max(amax[m], 1e-8))), qs[m] = max(amax[m], 1e-8) / 448 with the arithmetic of iflb200_row_quant
 * (the same bits as iflb200_row_quant_sharded phase 3).  Rows need no reduction here, so each is cut
 * into pieces of 2048 columns for separate CTAs.  amax is only read; amax_zero (a DIFFERENT buffer
 * of M floats, or NULL) is set to zero: callers alternate two buffers of row maxima between
 * consecutive gated GEMMs, each pass clearing the buffer the next GEMM will raise.  M <= 65535.
 * Replaces: the quantiser part of instinctflash/kernels/activation.py:44-56.
 */
IFLB200_API int iflb200_quant_from_amax(const float* h, int64_t ld_h, int M, int F, const float* amax, float* amax_zero,
                            void* q, int64_t ld_q, float* qs, void* stream);

/*
 * Per-tensor dynamic e4m3 pack (the torch-FP8-linear recipe):
 *   amax = max |x| (NaN propagates);  scale = max(amax, 1e-12) * fp32(1/448);
 *   q = e4m3_rn(clamp(x / scale, -448, 448))   (IEEE division, NaN propagates)
 * x is contiguous bf16 with n elements; workspace holds iflb200_pack_workspace_bytes(n)
 * bytes and needs no initialisation.
 * Replaces: instinctflash/runtime/fp8_pack.py:27-92 (dynamic_pack_bf16_e4m3 and its three
 * Triton kernels).
 */
IFLB200_API size_t iflb200_pack_workspace_bytes(int64_t n);
IFLB200_API int iflb200_dynamic_pack_bf16_e4m3(const void* x, int64_t n, void* q, float* scale,
                                   void* workspace, size_t workspace_bytes, void* stream);

/*
 * The dynamic pack for hosts that have no way to hand over scratch memory.  Same result as
 * iflb200_dynamic_pack_bf16_e4m3 (same kernels), but the partial-maximum scratch is a 4 KB device
 * array inside the library image, so the call needs no workspace and performs no allocation of
 * any kind (no cudaMalloc / cudaFree, no allocating library routine).  Meant for callers that
 * run from a memory plan fixed at start-up, have no allocator behind them, or sit in a
 * latency-critical loop where cudaMalloc's device-wide synchronisation is not acceptable.
 *   - n must not exceed IFLB200_PACK_NOALLOC_MAX_ELEMENTS; larger inputs are refused with
 *     IFLB200_ERR_TOO_LARGE before anything is launched.
 *   - The first call on each device looks up the array's device address (the device must be
 *     current); make that first call before any stream capture begins.
 *   - All calls on a device share the one array and it keeps whatever the previous call left in
 *     it.  Nothing in it has to start at zero (every word that is read was written by the same
 *     call), but two calls that overlap on the GPU -- different streams, or graph branches that
 *     may run concurrently -- race on it.  Keep calls on one device ordered.
 * This entry point has no counterpart in the reference.
 */
#define IFLB200_PACK_NOALLOC_MAX_ELEMENTS ((int64_t)1 << 28)
IFLB200_API int iflb200_dynamic_pack_bf16_e4m3_noalloc(const void* x, int64_t n, void* q, float* scale,
                                                       void* stream);

/*
 * Fixed-scale pack: q = e4m3_rn(clamp(x / scale[0], -448, 448)).
 * Replaces: instinctflash/runtime/fp8_pack.py:27-60 (_pack_kernel, pack_bf16_e4m3).
 */
IFLB200_API int iflb200_pack_bf16_e4m3(const void* x, int64_t n, const float* scale, void* q, void* stream);

/*
 * Persistent whole-stack execution for skinny activations (M <= 128): ONE cooperative launch
 * runs a program of operators over all layers and flow steps, with grid-wide dependency
 * counters between them and weights prefetched across operator boundaries.
 * Replaces the per-operator launch sequence of the reference's action-expert loop
 * (instinctflash/engines/pi05/engine.py:225-253: gemm / gated_act_quant / gemm /
 * residual_norm_quant per layer and flow step) for the operators listed below; arithmetic per
 * operator is that of the stand-alone entry points (a split-K GEMM sums its fp32 partials in
 * split order before the bf16 rounding point).
 *
 * `ops`, `tensor_maps` (128 bytes each, 64-byte aligned, written by
 * iflb200_encode_operand_map), `barriers` (num_barriers uint32) and `status2` (2 uint32) are
 * device buffers owned by the caller; barriers and status2[1] are zeroed by the call itself.
 * The program lives in device memory and is NOT validated by the call.  The caller guarantees:
 * K a multiple of 128 for every GEMM (the encoders below refuse other widths: operands are mapped
 * as [K / 128][rows][128 bytes] so that one TMA instruction brings four K slabs); N a multiple of 8 and row strides / base pointers of every operand 16-byte aligned; row
 * operators at most 8192 columns wide; every K split of a GEMM at least one 128-byte step
 * (split_k <= ceil(K / 128)); wait_bar / arrive_bar below num_barriers; every counter that an
 * operator waits on is the arrive_bar of an earlier operator (a counter nobody arrives on makes
 * the waiting operator run out of its time budget, see status2).
 * status2[0] != 0 after completion: a wait ran out of its time budget (role<<24 | kind<<16 | op).
 */
#define IFLB200_STACK_GEMM 1    /* out[M,N] = a[M,K] x w[N,K]^T: raw bf16 (split_k = 1) or fp32 partials [split_k][M][N] */
#define IFLB200_STACK_GATED 2   /* gated_act_quant of raw [M, 2N] -> codes [M,N] + row scales */
#define IFLB200_STACK_RESNORM 3 /* res += acc*row*col; RMS norm; quantiser -> codes [M,N] + row scales */
#define IFLB200_STACK_GEMM_GATED 4 /* a[M,K] x [gate | up][2N,K]^T with the gated activation in the epilogue:
                                      h[M,N] fp32 out, row maxima of |h| raised in aux (atomicMax) */
#define IFLB200_STACK_ENCODE 5  /* codes [M,N] + row scales from h [M,N] fp32 and the row maxima in aux;
                                   split_k = parts a row is divided into (work items = M * split_k) */
typedef struct {
  int32_t type;        /* IFLB200_STACK_* */
  int32_t wait_bar;    /* counter that must reach the grid size before activations are read; -1: none */
  int32_t arrive_bar;  /* counter this operator's CTAs bump when their outputs are visible; -1: none */
  int32_t tile_offset; /* GEMM: rotation of the work-item -> CTA assignment */
  int32_t N, K;        /* GEMM: output columns, reduction length; row operators: N = width */
  int32_t split_k;     /* GEMM: K splits (each at least one 128-byte step); GEMM_GATED: 1; RESNORM: partials to
                          sum (1: raw bf16 in); ENCODE: parts per row */
  int32_t act;         /* GATED: IFLB200_ACT_* */
  int32_t tm_a, tm_w;  /* GEMM: indices into tensor_maps (activation box, weight box; GEMM_GATED: a map written by
                          iflb200_encode_gated_weight_map) */
  int32_t pad0, pad1;
  void* out;           /* GEMM: raw bf16 / fp32 partials; GEMM_GATED: h fp32; row operators: e4m3 codes */
  const void* in;      /* GATED: raw bf16 [M, 2N]; RESNORM: raw bf16 [M,N] or fp32 partials; ENCODE: h fp32 [M,N] */
  const float* row_scale; /* GATED, GEMM_GATED: row scales of the GEMM input; RESNORM: delta_row */
  const float* col_scale; /* GATED, GEMM_GATED: [2N]; RESNORM: [N] */
  float* out_scale;    /* row operators: row scales out [M] */
  float* res;          /* RESNORM: residual stream fp32 [M,N], in place */
  int64_t ld_out, ld_in;
  float eps;           /* RESNORM */
  int32_t pad2;
  float* aux;          /* GEMM_GATED, ENCODE: row maxima of |h| [M] (zero before the first GEMM_GATED);
                          RESNORM: [M] words to leave at zero (the consumed maxima), or NULL */
} iflb200_stack_op;
IFLB200_API int iflb200_encode_operand_map(void* out128, const void* ptr, int rows, int K, int64_t ld, int box_rows);
IFLB200_API int iflb200_encode_gated_weight_map(void* out128, const void* ptr, int F, int K, int64_t ld);
IFLB200_API int iflb200_stack_activation_box_rows(int M);
IFLB200_API int iflb200_stack_weight_box_rows(void);
IFLB200_API int iflb200_stack_run(const void* ops, int num_ops, const void* tensor_maps, void* barriers,
                      int num_barriers, int M, void* status2, void* stream);

/*
 * Diagnostics of the tcgen05 GEMM: every wait inside the kernel is bounded; a wait that
 * runs out records (role, barrier, tile) in a device word and the kernel drains and
 * returns.  This reads the word (synchronises the given stream) and clears it.
 * Returns 0 if no kernel has timed out since the last call.  No reference counterpart.
 */
IFLB200_API int iflb200_gemm_take_timeout_record(uint32_t* record, void* stream);

/*
 * K-split linear of a tensor-parallel group as ONE launch whose stores go to several GPUs: `a` holds
 * `groups` blocks of `group_rows` activation rows ([groups * group_rows, K] e4m3); block g's fp32
 * accumulators a_g @ w^T (no scales, no rounding: the partial sums of this GPU's K range) are written
 * through d_out_maps[g], an array of `groups` 128-byte tensor maps in DEVICE memory (64-byte
 * aligned), each encoded by iflb200_encode_rowblock_map for a [group_rows, N] fp32 buffer that may
 * live on this GPU or be a peer-mapped buffer of another one (TMA stores over NVLink; loads never
 * touch peer memory).  The tiles of the blocks alternate in the launch order, so the stores towards
 * a peer are spread over the whole launch and drain under the main loops of the other tiles: the
 * transfer of a reduce-scatter rides inside the GEMM.  The K loop order is that of
 * iflb200_fp8_linear: the bits of block g equal those of a separate call on its rows.
 * No reference counterpart (the reference is single-GPU).
 */
IFLB200_API int iflb200_encode_rowblock_map(void* out, int rows, int N, int64_t ld_out, void* map128);
IFLB200_API int iflb200_gemm_fp8_rowblocks(const void* a, int64_t ld_a, const void* w, int64_t ld_w, int groups,
                               int group_rows, int N, int K, const void* d_out_maps, void* stream);

/*
 * Barrier between the GPUs of a tensor-parallel group over peer memory.  Every rank owns `p` flag
 * words that its peers can write (peer-mapped memory, zero at start); peer_flag_ptrs is a device
 * array of `p` pointers, entry r = the address of rank r's flag words as seen from this GPU
 * (entry `rank` is unused).  The call stores this rank's next arrival number into word `rank` of
 * every peer's flags (release, system scope) and waits until every word of my_flags has reached
 * it; `arrival` (one device word, zero at start) is advanced by the kernel, so the call can be
 * replayed from a CUDA graph.  Work enqueued before the call on this stream -- kernels and copies
 * that wrote into peers' memory -- is complete before the arrival is published; work enqueued after
 * it runs after every peer has arrived.  The wait is bounded (iflb200_set_wait_budget_us): when it
 * runs out, `status[0]` receives 0x50000000 | peer << 16 | arrival and the kernel returns; while
 * status[0] is non-zero later calls signal and return without waiting (the host reads and clears
 * the word).  Plain
 * peer loads and stores; no multicast.  One process per GPU; never call it for two ranks that
 * share a GPU.  No reference counterpart (the reference is single-GPU).
 */
IFLB200_API int iflb200_peer_barrier(const void* peer_flag_ptrs, void* my_flags, void* arrival, int rank, int p,
                         void* status, void* stream);

/*
 * The barrier with a reduction behind it, one single-CTA kernel: after every peer has arrived,
 *   max_out[i] = max over r < p of max_in[r * max_n + i], i < max_n
 * (max_in: this rank's [p][max_n] slots, slot r written by rank r -- iflb200_row_max_sharded's
 * mirrors -- the own slot by an earlier kernel of this stream): the all-reduce-max of the row
 * maxima between the two phases of iflb200_row_quant_sharded.  max_n == 0: the plain barrier.
 */
IFLB200_API int iflb200_peer_exchange(const void* peer_flag_ptrs, void* my_flags, void* arrival, int rank, int p,
                          void* status, const float* max_in, float* max_out, int max_n, void* stream);

/*
 * Time budget of the waits inside the tcgen05 GEMM and the persistent stack kernel, in
 * microseconds (0 restores the default of 2 s).  A wait that outlives it makes the kernel record
 * where it gave up (iflb200_gemm_take_timeout_record / status2[0] of iflb200_stack_run), drain and
 * return: the context stays usable.  Applies to the current device and synchronises it; not for
 * use during stream capture.  No reference counterpart.
 */
IFLB200_API int iflb200_set_wait_budget_us(int64_t microseconds);

/*
 * Which kernel the last GEMM call of this process launched (host-side record, no device access):
 * family 1 = single-CTA tiles, 2 / 3 = CTA pairs with one / two accumulators, +4 = the swapped
 * form, +8 = the gated form (paired gate / up columns), +16 = split-K partial planes, +32 = row blocks
 * to several destinations; the tile width in columns (tokens for the
 * swapped form); the cluster split-K factor.  Any pointer may be NULL.  For tests that must know
 * that a given kernel really ran.  No reference counterpart.
 */
IFLB200_API int iflb200_gemm_last_launch(int* family, int* tile_n, int* split_k);

/* Tuning overrides for experiments and tests (0 = heuristic). No reference counterpart. */
IFLB200_API int iflb200_gemm_set_config(int tile_n, int stages, int group_m);
/* Split-K of the GEMM over a thread-block cluster (partials summed over distributed shared
 * memory in rank order): 0 = cost model (deep reductions with too few tiles to fill the GPU),
 * 1 = never (the K loop is then a function of K alone and outputs are bit-identical to the
 * unsplit kernel), 2 / 4 = forced.  No reference counterpart. */
IFLB200_API int iflb200_gemm_set_split_k(int split_k);
/* Row kernels: force the number of threads that share one row (power of two, 32..1024;
 * 0 = heuristic).  For experiments and tests.  No reference counterpart. */
IFLB200_API int iflb200_row_set_group(int threads_per_row);
/* Programmatic dependent launch: a kernel launched this way may be scheduled while its
 * predecessor in the stream drains; it waits for the predecessor's results before its first
 * access to memory a kernel can write, and the GEMM warms L2 with its first weight boxes
 * meanwhile.  1 (default) = for calls over at most 2048 activation rows (short kernels, where
 * it shortens a layer stack; with thousands of rows it was measured slower), 0 = never,
 * 2 = always.  Results are identical in every mode.  No reference counterpart. */
IFLB200_API int iflb200_set_dependent_launch(int enable);
/* Kernel family: 0 = heuristic, 1 = single-CTA tiles only, 2 / 3 = 256x256 tiles on CTA pairs
 * (cta_group::2) with one / two tensor-memory accumulators; add 16 to store the epilogue
 * straight from registers instead of through shared memory and TMA; add 256 to take the
 * swapped form (tokens on the MMA's N side, 257..1024 tokens, two-byte raw or dequantised output;
 * not chosen by the heuristic) wherever it exists, 128 to forbid it, 512 to keep the swapped form
 * off CTA pairs; add 1024 / 2048 to run the gated form's 256-wide tiles with sixteen / eight
 * epilogue warps; add 4096 to keep the skinny-regime kernel on one K slab per TMA instruction.
 * Any other bit is refused.  Every mode writes the same output bits.  For
 * experiments and tests.  No reference counterpart. */
IFLB200_API int iflb200_gemm_set_mode(int mode);

#ifdef __cplusplus
}
#endif
#endif /* IFLB200_H_ */
