// FP8 (e4m3 x e4m3 -> fp32) GEMM for sm_100a with fused consumer epilogues.
//
//   out[M,N] = epilogue( sum_k A[m,k] * W[n,k] )        A [M,K], W [N,K], both K-major
//
// Persistent, warp-specialised, one CTA per SM:
//   warp 0      TMA producer: cp.async.bulk.tensor loads of a 128 x 128-byte A tile and a
//               BN x 128-byte W tile per stage, 128-byte swizzle, completion on an mbarrier;
//   warp 1      MMA issuer: one thread issues tcgen05.mma (128 x BN x 32 per instruction,
//               four per stage) into one of two TMEM accumulators and commits the stage's
//               "empty" barrier / the accumulator's "full" barrier;
//   warps 2..5  epilogue: tcgen05.ld the finished accumulator (one row per thread), apply the
//               consumer arithmetic of the reference in its exact order and store.
// The two TMEM accumulators let the epilogue of tile i overlap the main loop of tile i+1.
// The K loop order is a function of K alone (128-byte steps, no split), so an output element
// never depends on N, on the tile shape or on the grid: column-sharded weights give
// bit-identical columns.
//
// Every wait is bounded: a wait that runs out records where in g_timeout_record, raises a
// CTA-wide abort flag, every role leaves its loop, in-flight TMA loads are drained with a
// bounded wait, TMEM is freed and the kernel returns.
#include <cuda.h>
#include <cuda_runtime.h>
#include <string.h>

#include "../../include/iflb200.h"
#include "launch.cuh"
#include "rowmath.cuh"

namespace iflb200 {

constexpr int BM = 128;
constexpr int BK = 128;  // bytes == e4m3 elements per stage along K
constexpr int kGemmThreads = 320;  // TMA warp, MMA warp, eight epilogue warps
constexpr int kPrefetchSteps = 8;  // W boxes warmed in L2 ahead of the grid dependency wait
constexpr int kEpilogueWarps = 8;   // two per TMEM lane quadrant, each draining half of the columns
constexpr uint64_t kWaitBudgetNs = 2000000000ull;  // 2 s per wait, then abort

constexpr int kStagingBytes = kEpilogueWarps * 32 * 128;  // one 32-row x 128-byte buffer per epilogue warp

enum : int { EPI_RAW = 0, EPI_DEQUANT = 1, EPI_RESIDUAL = 2 };

struct GemmParams {
  int M, N, K;
  int num_m, num_n, num_k, num_tiles, group_m;
  int epilogue;
  int exact;  // 1: scales applied to the fp32 accumulator without the bf16 rounding; 2: the same with two
              // per-tensor scales in the order torch._scaled_mm applies them: (acc * (s_a * s_b)) + bias,
              // every operation rounded on its own (measured on B200: bit-identical to cuBLASLt's epilogue)
  const float* row;
  int row_stride;
  const float* col;
  int col_stride;
  const void* bias;
  int bias_dtype;
  const float* gate;
  const int32_t* gate_index;
  void* out;
  int out_dtype;
  int64_t ld_out;
  int split_k;     // > 1: the CTAs of a cluster share one tile, each a K range; partials are summed over DSMEM
  int a_bytes;     // bytes one activation box delivers per K step: 128 x (rows of the box)
  int partials;    // > 1: K is split over that many independent CTAs per tile; each writes its fp32 partial
                   // accumulator to out[split][M][ld_out] (summed in split order by the consumer)
  int act;         // gated form: IFLB200_ACT_*
  uint32_t* amax;  // gated form: per-row maximum of |h| as float bits, raised with atomicMax
  int tma_store;  // 1: the epilogue stages 128-byte row pieces in shared memory and TMA-stores them
  int half_rows;  // 1: 64-wide tiles of two-byte outputs leave as two 64-byte pieces per row, one per warp of a
                  // quadrant (the output map then has a 64-byte box), so both warps drain the accumulator
  // Row blocks to several destinations (tensor parallel, row-split linears): the activation holds
  // `groups` blocks of `group_rows` rows (M = group_rows); block g's tiles are stored through
  // out_maps[g] (tensor maps in global memory, e.g. one per GPU's buffer).  Tiles of the blocks
  // alternate, so stores to a slow destination (a peer over NVLink) are spread over the whole launch
  // and drain under the main loops of the other blocks' tiles.
  int groups;
  int group_rows;
  const CUtensorMap* out_maps;
};

// role << 24 | barrier kind << 16 | low 16 bits of the tile counter; 0 = no timeout.
__device__ uint32_t g_timeout_record[4];
// Time budget of every wait inside the GEMM kernels (read only on the slow path of a wait).
__device__ uint64_t g_gemm_wait_budget_ns = kWaitBudgetNs;
#ifdef IFLB200_TRACE
// Experiment builds only (-DIFLB200_TRACE; never in the product library): block 0 of each launch of
// the single-CTA kernel stamps the SM clock at a few points; slot 0 holds globaltimer at entry.
__device__ unsigned long long g_gemm_trace[64][16];
__device__ unsigned int g_gemm_trace_launch;
__device__ unsigned int g_gemm_trace_cur;  // id of the launch whose block 0 is tracing (helpers without the id)
#define GEMM_TRACE_IN_HELPER(slot, cond)                                                                       \
  do {                                                                                                         \
    if (blockIdx.x == 0 && (cond)) g_gemm_trace[g_gemm_trace_cur & 63][slot] = (unsigned long long)clock64(); \
  } while (0)
#define GEMM_TRACE(slot)                                                              \
  do {                                                                                \
    if (blockIdx.x == 0) g_gemm_trace[trace_id & 63][slot] = (unsigned long long)clock64(); \
  } while (0)
#else
#define GEMM_TRACE(slot) \
  do {                   \
  } while (0)
#define GEMM_TRACE_IN_HELPER(slot, cond) \
  do {                                   \
  } while (0)
#endif
int set_stack_wait_budget_ns(uint64_t ns);  // stack_persistent.cu
int set_peer_wait_budget_ns(uint64_t ns);   // xgpu_ops.cu

__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_dsmem_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ float ld_dsmem_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}

// SL: 128-byte K slabs per stage.  With SL > 1 one TMA instruction per operand brings SL slabs (the
// operands are mapped as [K / 128][rows][128 bytes]): a skinny GEMM's main loop is bound by the
// rate at which one SM can issue TMA instructions (about 0.2 us each, measured), not by bytes.
template <int BN, int STAGES, int EW = kEpilogueWarps, int SL = 1>
struct SmemLayout {
  static constexpr int kABytes = BM * BK * SL;
  static constexpr int kBBytes = BN * BK * SL;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // epilogue staging: one 32-row buffer per epilogue warp (TMA-store source), 128 bytes per row
  // with eight epilogue warps, 64 with sixteen
  static constexpr int kWarpStaging = EW > 8 ? 2048 : 4096;
  static constexpr int kStagingOffset = STAGES * kStageBytes;
  static constexpr int kBarOffset = kStagingOffset + EW * kWarpStaging;
  // full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], then the TMEM base word and the
  // abort flag.
  static constexpr int kNumBars = 2 * STAGES + 4;
  static constexpr int kTotal = kBarOffset + kNumBars * 8 + 16;
  static constexpr int kDynamic = kTotal + 1024;  // room to align the base to 1024 bytes
};

__device__ __forceinline__ void tile_coords(const GemmParams& p, int tile, int& m_blk, int& n_blk) {
  // Bands of group_m row blocks, column blocks outermost inside a band: CTAs that run at the
  // same time share W tiles through L2 and touch at most group_m A row blocks.
  const int band = p.group_m * p.num_n;
  const int g = tile / band;
  const int first_m = g * p.group_m;
  const int size = min(p.num_m - first_m, p.group_m);
  const int r = tile - g * band;
  m_blk = first_m + r % size;
  n_blk = r / size;
}

// The same with the destination block of the row-blocks form (block 0 otherwise).
__device__ __forceinline__ void tile_place(const GemmParams& p, int tile, int& m_blk, int& n_blk, int& grp) {
  grp = 0;
  if (p.groups > 1) {
    grp = tile % p.groups;
    tile /= p.groups;
  }
  tile_coords(p, tile, m_blk, n_blk);
}

// Bounded wait on an mbarrier phase.  Returns false when the CTA is aborting.
__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity, volatile uint32_t* abort,
                                             uint32_t code) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = 0;
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort) return false;
    if (++spins > 2048) {
      if (t0 == 0) t0 = globaltimer_ns();
      __nanosleep(128);
      if (globaltimer_ns() - t0 > g_gemm_wait_budget_ns) {
        *abort = 1;
        atomicCAS(&g_timeout_record[0], 0u, code);
        return false;
      }
    }
  }
}

template <int BN>
__device__ __forceinline__ void epilogue_chunk(const GemmParams& p, const uint32_t (&acc)[32], int m,
                                               int n0, bool row_ok, float rs, int64_t gofs) {
  // 32 consecutive columns of one row.
  float v[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const float a = __uint_as_float(acc[i]);
    v[i] = p.exact ? a : __bfloat162float(__float2bfloat16_rn(a));
  }
  if (!row_ok) return;
  const int valid = min(32, p.N - n0);  // multiple of 16 (N is), > 0
  if (p.epilogue == EPI_RAW) {
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (int64_t)m * p.ld_out + n0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (j * 8 < valid) {
        uint4 u;
        u.x = f32_to_bf16_bits(v[8 * j + 0]) | (f32_to_bf16_bits(v[8 * j + 1]) << 16);
        u.y = f32_to_bf16_bits(v[8 * j + 2]) | (f32_to_bf16_bits(v[8 * j + 3]) << 16);
        u.z = f32_to_bf16_bits(v[8 * j + 4]) | (f32_to_bf16_bits(v[8 * j + 5]) << 16);
        u.w = f32_to_bf16_bits(v[8 * j + 6]) | (f32_to_bf16_bits(v[8 * j + 7]) << 16);
        *reinterpret_cast<uint4*>(o + 8 * j) = u;
      }
    }
    return;
  }
  // Consumer arithmetic.  Column vectors are read with warp-uniform addresses (every thread
  // of the warp has the same columns), which the L1 serves as broadcasts.  The residual operand
  // is updated in place, so its loads cannot move above the stores of an earlier piece: all 32
  // columns are requested before the first is used (one memory round trip, not four).
  float res_all[32];
  if (p.epilogue == EPI_RESIDUAL) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (j * 8 < valid) {
        const int64_t off = (int64_t)m * p.ld_out + n0 + 8 * j;
        if (p.out_dtype == IFLB200_F32) {
          const float* o = reinterpret_cast<const float*>(p.out) + off;
          const float4 a = *reinterpret_cast<const float4*>(o);
          const float4 b = *reinterpret_cast<const float4*>(o + 4);
          res_all[8 * j + 0] = a.x; res_all[8 * j + 1] = a.y; res_all[8 * j + 2] = a.z; res_all[8 * j + 3] = a.w;
          res_all[8 * j + 4] = b.x; res_all[8 * j + 5] = b.y; res_all[8 * j + 6] = b.z; res_all[8 * j + 7] = b.w;
        } else {
          const uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.out) + off);
          const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            res_all[8 * j + 2 * i] = __uint_as_float(w[i] << 16);
            res_all[8 * j + 2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
          }
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (j * 8 >= valid) break;
    const int64_t off = (int64_t)m * p.ld_out + n0 + 8 * j;
    float res[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) res[i] = p.epilogue == EPI_RESIDUAL ? res_all[8 * j + i] : 0.0f;
    float y[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int n = n0 + 8 * j + i;
      if (p.exact == 2) {
        float t = __fmul_rn(v[8 * j + i], __fmul_rn(rs, __ldg(p.col)));
        if (p.bias)
          t = __fadd_rn(t, (p.bias_dtype == IFLB200_F32)
                               ? __ldg(reinterpret_cast<const float*>(p.bias) + n)
                               : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[n]));
        y[i] = t;
        continue;
      }
      Chain ch(v[8 * j + i]);
      if (p.row) ch.mul(rs);
      if (p.col) ch.mul(__ldg(p.col + (int64_t)n * p.col_stride));
      if (p.bias) {
        const float b = (p.bias_dtype == IFLB200_F32)
                            ? __ldg(reinterpret_cast<const float*>(p.bias) + n)
                            : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[n]);
        ch.add(b);
      }
      if (p.epilogue == EPI_RESIDUAL) {
        if (p.gate) ch.mul(__ldg(p.gate + gofs + n));
        ch.add(res[i]);  // res + d, contracted with d's last multiply when there is one
      }
      y[i] = ch.done();
    }
    if (p.out_dtype == IFLB200_F32) {
      float* o = reinterpret_cast<float*>(p.out) + off;
      *reinterpret_cast<float4*>(o) = make_float4(y[0], y[1], y[2], y[3]);
      *reinterpret_cast<float4*>(o + 4) = make_float4(y[4], y[5], y[6], y[7]);
    } else if (p.out_dtype == IFLB200_BF16) {
      uint4 u;
      u.x = f32_to_bf16_bits(y[0]) | (f32_to_bf16_bits(y[1]) << 16);
      u.y = f32_to_bf16_bits(y[2]) | (f32_to_bf16_bits(y[3]) << 16);
      u.z = f32_to_bf16_bits(y[4]) | (f32_to_bf16_bits(y[5]) << 16);
      u.w = f32_to_bf16_bits(y[6]) | (f32_to_bf16_bits(y[7]) << 16);
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.out) + off) = u;
    } else {
      uint4 u;
      u.x = f32_to_f16_bits(y[0]) | (f32_to_f16_bits(y[1]) << 16);
      u.y = f32_to_f16_bits(y[2]) | (f32_to_f16_bits(y[3]) << 16);
      u.z = f32_to_f16_bits(y[4]) | (f32_to_f16_bits(y[5]) << 16);
      u.w = f32_to_f16_bits(y[6]) | (f32_to_f16_bits(y[7]) << 16);
      *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(p.out) + off) = u;
    }
  }
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);  // one cvt.rn.bf16x2.f32
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// The per-column operands (column scale, bias) of the columns one epilogue warp drains from a tile,
// fetched BEFORE the warp waits for the accumulator: lane l holds columns n_first + 32*k + l, k < 4
// (a warp drains at most 128 columns).  Loading them per 32-column chunk after the accumulator had
// arrived put four dependent global-memory round trips on the critical path of every tile: a
// 64 x 4096 x 1024 linear with scales and bias took 9.7 us against 4.4 us for its raw-output form.
struct ColumnVectors {
  float cs[4], bs[4];
};
__device__ __forceinline__ ColumnVectors fetch_column_vectors(const GemmParams& p, int n_first, int n_count, int lane) {
  ColumnVectors v;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int n = n_first + 32 * k + lane;
    const bool in = 32 * k + lane < n_count && n < p.N;
    v.cs[k] = (p.col && in) ? __ldg(p.col + (int64_t)n * p.col_stride) : 0.0f;
    v.bs[k] = 0.0f;
    if (p.bias && in)
      v.bs[k] = (p.bias_dtype == IFLB200_F32) ? __ldg(reinterpret_cast<const float*>(p.bias) + n)
                                               : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[n]);
  }
  return v;
}

// Consumer arithmetic on 32 consecutive columns of one accumulator row (y in fp32, before the
// cast to the output type).  Scale / bias vectors are read with warp-uniform addresses.
// `pre`: lane l holds the column scale and bias of column n0 + l (fetched before the accumulator was
// waited for; see ColumnVectors) and every lane takes them from there instead of loading them now.
__device__ __forceinline__ void epilogue_values(const GemmParams& p, const uint32_t (&acc)[32], int n0, float rs,
                                                float (&y)[32], bool pre = false, float csl = 0.0f, float bsl = 0.0f) {
  if (p.exact) {
#pragma unroll
    for (int i = 0; i < 32; ++i) y[i] = __uint_as_float(acc[i]);
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) {  // the bf16 rounding point of the accumulator, two at a time
      const uint32_t w = pack_bf16x2(__uint_as_float(acc[2 * i]), __uint_as_float(acc[2 * i + 1]));
      y[2 * i] = __uint_as_float(w << 16);
      y[2 * i + 1] = __uint_as_float(w & 0xFFFF0000u);
    }
  }
  if (p.epilogue == EPI_RAW) return;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float v[8], cs[8], bs[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int n = n0 + 8 * j + i;
      const bool in = n < p.N;
      v[i] = y[8 * j + i];
      if (pre) {
        cs[i] = __shfl_sync(0xFFFFFFFFu, csl, 8 * j + i);
        bs[i] = __shfl_sync(0xFFFFFFFFu, bsl, 8 * j + i);
        continue;
      }
      cs[i] = (p.col && in) ? __ldg(p.col + (int64_t)n * p.col_stride) : 0.0f;
      bs[i] = 0.0f;
      if (p.bias && in)
        bs[i] = (p.bias_dtype == IFLB200_F32) ? __ldg(reinterpret_cast<const float*>(p.bias) + n)
                                               : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[n]);
    }
    if (p.exact == 2) {
      const float alpha = __fmul_rn(rs, __ldg(p.col));
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[i] = __fmul_rn(v[i], alpha);
        if (p.bias) v[i] = __fadd_rn(v[i], bs[i]);
      }
    } else {
      Chain8 ch(v);
      if (p.row) ch.mul(rs);
      if (p.col) ch.mul(cs);
      if (p.bias) ch.add(bs);
      ch.done(v);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) y[8 * j + i] = v[i];
  }
}

// Consumer arithmetic and output cast of 32 consecutive columns of this lane's row, written into
// the lane's 128-byte staging row (128-byte swizzle: 16-byte chunk index ^ (lane & 7)).  `sub` is
// the column offset inside the staged piece: 0 or 32 for two-byte outputs, 0 for four-byte ones.
__device__ __forceinline__ void stage_columns(const GemmParams& p, const uint32_t (&r)[32], int n_abs, float rs,
                                              uint8_t* mine, int sub, int lane, bool pre = false, float csl = 0.0f,
                                              float bsl = 0.0f) {
  const int es = (p.out_dtype == IFLB200_F32) ? 4 : 2;
  if (es == 2) {
    // 32 values = 64 bytes = four 16-byte chunks; chunk index within the 128-byte row
    const int first = sub / 8;  // 0 or 4
    // half-row pieces: 64-byte rows with the 64-byte swizzle (chunk index ^ ((row >> 1) & 3))
    const int sw = p.half_rows ? ((lane >> 1) & 3) : (lane & 7);
    if (p.epilogue == EPI_RAW) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 u;
        u.x = pack_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1]));
        u.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
        u.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
        u.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
        *reinterpret_cast<uint4*>(mine + (((first + j) ^ sw) * 16)) = u;
      }
    } else {
      float y[32];
      epilogue_values(p, r, n_abs, rs, y, pre, csl, bsl);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 u;
        if (p.out_dtype == IFLB200_BF16) {
          u.x = pack_bf16x2(y[8 * j + 0], y[8 * j + 1]);
          u.y = pack_bf16x2(y[8 * j + 2], y[8 * j + 3]);
          u.z = pack_bf16x2(y[8 * j + 4], y[8 * j + 5]);
          u.w = pack_bf16x2(y[8 * j + 6], y[8 * j + 7]);
        } else {
          u.x = pack_f16x2(y[8 * j + 0], y[8 * j + 1]);
          u.y = pack_f16x2(y[8 * j + 2], y[8 * j + 3]);
          u.z = pack_f16x2(y[8 * j + 4], y[8 * j + 5]);
          u.w = pack_f16x2(y[8 * j + 6], y[8 * j + 7]);
        }
        *reinterpret_cast<uint4*>(mine + (((first + j) ^ sw) * 16)) = u;
      }
    }
  } else {
    float y[32];
    epilogue_values(p, r, n_abs, rs, y, pre, csl, bsl);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      *reinterpret_cast<float4*>(mine + ((j ^ (lane & 7)) * 16)) =
          make_float4(y[4 * j + 0], y[4 * j + 1], y[4 * j + 2], y[4 * j + 3]);
  }
}

// Epilogue of one warp: its 32 accumulator rows x its half of the tile's columns, through shared
// memory.  128 bytes of each output row (64 two-byte or 32 four-byte columns) are staged with
// the 128-byte swizzle and written by one TMA store, so global memory sees whole 128-byte lines
// instead of 16-byte pieces of 32 different rows.
template <int BN>
__device__ __forceinline__ void epilogue_tma_store(const GemmParams& p, const CUtensorMap* tm_out, uint32_t t_row,
                                                   uint32_t staging, uint8_t* staging_ptr, int row0, int n_base,
                                                   int col_begin, int col_end, float rs, int lane, int z = -1,
                                                   const ColumnVectors* cv = nullptr) {
  const int es = (p.out_dtype == IFLB200_F32) ? 4 : 2;
  const int row_bytes = p.half_rows ? 64 : 128;
  const int cols_per_store = row_bytes / es;  // 64 or 32
  uint8_t* mine = staging_ptr + lane * row_bytes;
#pragma unroll 1
  for (int c = col_begin; c < col_end; c += cols_per_store) {
    const int n0 = n_base + c;
    if (n0 >= p.N) break;  // uniform
    if (lane == 0) bulk_wait_group_read<0>();  // the previous store has read the buffer
    __syncwarp();
#pragma unroll 1
    for (int sub = 0; sub < cols_per_store; sub += 32) {
      uint32_t r[32];
      tmem_ld_32x32b_x32(t_row + c + sub, r);
      tmem_ld_wait();
      GEMM_TRACE_IN_HELPER(10, threadIdx.x == 64 && c == col_begin && sub == 0);  // first chunk out of tensor memory
      if (cv != nullptr) {
        const int k = (c + sub - col_begin) >> 5;  // which of the warp's 32-column chunks (uniform)
        const float csl = k == 0 ? cv->cs[0] : (k == 1 ? cv->cs[1] : (k == 2 ? cv->cs[2] : cv->cs[3]));
        const float bsl = k == 0 ? cv->bs[0] : (k == 1 ? cv->bs[1] : (k == 2 ? cv->bs[2] : cv->bs[3]));
        stage_columns(p, r, n0 + sub, rs, mine, sub, lane, true, csl, bsl);
      } else {
        stage_columns(p, r, n0 + sub, rs, mine, sub, lane);
      }
      GEMM_TRACE_IN_HELPER(11, threadIdx.x == 64 && c == col_begin && sub == 0);  // first chunk staged
    }
    GEMM_TRACE_IN_HELPER(12, threadIdx.x == 64 && c == col_begin);  // first piece staged
    fence_proxy_async_smem();  // generic-proxy writes visible to the TMA unit
    __syncwarp();
    GEMM_TRACE_IN_HELPER(13, threadIdx.x == 64 && c == col_begin);  // fenced
    if (lane == 0) {
      if (z >= 0) tma_store_3d(tm_out, staging, n0, row0, z);  // partial sums: plane z of [splits][M][N]
      else tma_store_2d(tm_out, staging, n0, row0);
      bulk_commit_group();
    }
  }
}

// Column scales of the gated form for the chunks one epilogue warp handles (see epilogue_gated for
// the split of a tile over the warps), fetched before the accumulator is waited for.
template <int BN, int PARTS>
__device__ __forceinline__ void gated_scales(const GemmParams& p, int n_base, int part, int lane, float (&cgl)[4],
                                             float (&cul)[4]) {
  constexpr int kChunks = BN / 2 / 32;
  constexpr int kPerPart = kChunks >= PARTS ? kChunks / PARTS : 1;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int n = n_base + part * kPerPart * 32 + 32 * k + lane;
    const bool in = p.col && k < kPerPart && part * kPerPart < kChunks && n < p.N;
    cgl[k] = in ? __ldg(p.col + n) : 0.0f;
    cul[k] = in ? __ldg(p.col + p.N + n) : 0.0f;
  }
}

// Epilogue of the gated form.  A tile of BN accumulator columns holds BN/2 gate columns followed
// by the BN/2 up columns of the same hidden units (the producer loads the two halves of the
// [gate | up] weight matrix side by side), so the gated activation of
// instinctflash/kernels/activation.py:26-43 is evaluated on the accumulators in registers, in that
// kernel's instruction order:  g = (bf16(acc_g) * row) * col_g,  u = (bf16(acc_u) * row) * col_u,
// h = u * act(g).  h leaves as fp32 (the reference never rounds it to 16 bits before the
// quantiser), 128 bytes of each row per TMA store, and each row's maximum of |h| is raised in
// p.amax with an integer atomicMax on the float's bits: a maximum does not depend on the order
// it is taken in, so the row scale and the codes a later pass derives from it are exactly those of
// the one-kernel-per-row form.
// This is the one epilogue whose arithmetic (about 25 instructions per element) is comparable to
// the main loop's duration, so the warps of a TMEM lane quadrant (PARTS of them) split the hidden
// units of the tile, and the column scales come in as 128-bit loads with the ragged-width masking
// confined to the last chunk of a row.
template <int BN, int PARTS>
__device__ __forceinline__ void epilogue_gated(const GemmParams& p, const CUtensorMap* tm_out, uint32_t t_row,
                                               uint32_t staging, uint8_t* staging_ptr, int row0, int n_base,
                                               int part, int m, bool row_ok, float rs, int lane,
                                               const float (&cgl)[4], const float (&cul)[4]) {
  // cgl[k] / cul[k]: the gate / up column scale of hidden unit n_base + c_begin + 32k + lane, fetched
  // before the accumulator was waited for (gated_scales); every lane takes column i's from lane i.
  constexpr int HW = BN / 2;        // hidden units per tile
  constexpr int kChunks = HW / 32;  // chunks of 32 columns in a tile: 4, 2 or 1
  constexpr int kPerPart = kChunks >= PARTS ? kChunks / PARTS : 1;
  if (part * kPerPart >= kChunks) return;  // fewer chunks than warps in the quadrant: the first ones take them
  const int c_begin = part * kPerPart * 32;
  // Sixteen epilogue warps have 64 bytes of staging per row: a chunk leaves as two stores of 16
  // columns each (64-byte swizzle: 16-byte piece index ^ ((row >> 1) & 3)).
  constexpr bool kHalfRows = PARTS > 2;
  uint8_t* mine = staging_ptr + lane * (kHalfRows ? 64 : 128);
  float row_max = 0.0f;
  bool any = false;
#pragma unroll 1
  for (int k = 0; k < kPerPart; ++k) {
    const int c = c_begin + 32 * k;
    const int n0 = n_base + c;
    if (n0 >= p.N) break;  // uniform
    any = true;
    const bool whole = n0 + 32 <= p.N;  // uniform: all 32 columns of the chunk are hidden units
    uint32_t rg[32], ru[32];
    tmem_ld_32x32b_x32(t_row + c, rg);
    tmem_ld_32x32b_x32(t_row + HW + c, ru);
    tmem_ld_wait();
    if (lane == 0) bulk_wait_group_read<0>();  // the previous store has read the buffer
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (kHalfRows && j == 2) {  // first 16 columns staged: send them, then reuse the buffer
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(tm_out, staging, n0, row0);
          bulk_commit_group();
          bulk_wait_group_read<0>();
        }
        __syncwarp();
      }
      float g[8], u[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {  // the bf16 rounding point of the accumulators
        const uint32_t wg = pack_bf16x2(__uint_as_float(rg[8 * j + 2 * i]), __uint_as_float(rg[8 * j + 2 * i + 1]));
        const uint32_t wu = pack_bf16x2(__uint_as_float(ru[8 * j + 2 * i]), __uint_as_float(ru[8 * j + 2 * i + 1]));
        g[2 * i] = __uint_as_float(wg << 16);
        g[2 * i + 1] = __uint_as_float(wg & 0xFFFF0000u);
        u[2 * i] = __uint_as_float(wu << 16);
        u[2 * i + 1] = __uint_as_float(wu & 0xFFFF0000u);
      }
      if (p.row) {
        const uint64_t rs2 = pack2(rs, rs);
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
          unpack2(mul2(pack2(g[i], g[i + 1]), rs2), g[i], g[i + 1]);
          unpack2(mul2(pack2(u[i], u[i + 1]), rs2), u[i], u[i + 1]);
        }
      }
      if (p.col) {
        float cg[8], cu[8];
        const int n = n0 + 8 * j;
        (void)n;
        const float gl = k == 0 ? cgl[0] : (k == 1 ? cgl[1] : (k == 2 ? cgl[2] : cgl[3]));  // k is uniform
        const float ul = k == 0 ? cul[0] : (k == 1 ? cul[1] : (k == 2 ? cul[2] : cul[3]));
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          cg[i] = __shfl_sync(0xFFFFFFFFu, gl, 8 * j + i);
          cu[i] = __shfl_sync(0xFFFFFFFFu, ul, 8 * j + i);
        }
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
          unpack2(mul2(pack2(g[i], g[i + 1]), pack2(cg[i], cg[i + 1])), g[i], g[i + 1]);
          unpack2(mul2(pack2(u[i], u[i + 1]), pack2(cu[i], cu[i + 1])), u[i], u[i + 1]);
        }
      }
      float h[8];
      if (p.act == IFLB200_ACT_GELU_TANH) {
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
          gelu_tanh_ref2(g[i], g[i + 1]);
          unpack2(mul2(pack2(u[i], u[i + 1]), pack2(g[i], g[i + 1])), h[i], h[i + 1]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) h[i] = __fmul_rn(u[i], silu_ref(g[i]));
      }
      if (!whole) {  // columns past the hidden width: not stored, not in the maximum
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (n0 + 8 * j + i >= p.N) h[i] = 0.0f;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) row_max = max_f32(row_max, fabsf(h[i]));
      if (kHalfRows) {
        const int sw = (lane >> 1) & 3;
        *reinterpret_cast<float4*>(mine + (((2 * (j & 1)) ^ sw) * 16)) = make_float4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<float4*>(mine + (((2 * (j & 1) + 1) ^ sw) * 16)) = make_float4(h[4], h[5], h[6], h[7]);
      } else {
        *reinterpret_cast<float4*>(mine + (((2 * j) ^ (lane & 7)) * 16)) = make_float4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<float4*>(mine + (((2 * j + 1) ^ (lane & 7)) * 16)) = make_float4(h[4], h[5], h[6], h[7]);
      }
    }
    fence_proxy_async_smem();  // generic-proxy writes visible to the TMA unit
    __syncwarp();
    if (lane == 0 && (!kHalfRows || n0 + 16 < p.N)) {  // a ragged row can end after the first 16 columns
      tma_store_2d(tm_out, staging, kHalfRows ? n0 + 16 : n0, row0);
      bulk_commit_group();
    }
  }
  if (any && row_ok) atomicMax(p.amax + m, __float_as_uint(row_max));
}

// Epilogue of the swapped form (tokens on the MMA's N side): the accumulator holds the tile
// transposed, lane = output column n, TMEM column = token.  A warp turns 32 tokens x its 32 output
// columns into a [token][n] block of 32 x 64 bytes in shared memory (one 2-byte store per value:
// the 32 lanes of a store instruction fill 64 contiguous bytes of one token row, no bank
// conflict) and writes it with one TMA store; two blocks per warp alternate.  The last chunk of a
// token tile whose width is not a multiple of 32 starts at width - 32 and rewrites a few tokens of
// the chunk before it with the same values.  Two-byte outputs, raw or dequantised.
template <int BT>
__device__ __forceinline__ void epilogue_swapped(const GemmParams& p, const CUtensorMap* tm_out, uint32_t t_row,
                                                 uint32_t staging, uint8_t* staging_ptr, int n_row0, int tok0,
                                                 int half, int lane, int& buf) {
  constexpr int kChunks = (BT + 31) / 32;
  constexpr int kFirstHalf = (kChunks + 1) / 2;
  const int c_begin = half == 0 ? 0 : kFirstHalf, c_end = half == 0 ? kFirstHalf : kChunks;
  const int n = n_row0 + lane;  // this lane's output column
  const bool n_ok = n < p.M;    // p.M: rows of the MMA's M side = output columns
  float cs = 1.0f, bs = 0.0f;
  if (p.epilogue == EPI_DEQUANT && n_ok) {
    if (p.col) cs = __ldg(p.col + (int64_t)n * p.col_stride);
    if (p.bias)
      bs = (p.bias_dtype == IFLB200_F32) ? __ldg(reinterpret_cast<const float*>(p.bias) + n)
                                         : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[n]);
  }
  // `buf` lives across tiles: the two blocks alternate over the whole life of the warp, so the
  // block about to be written is always the one whose store was issued two stores ago
#pragma unroll 1
  for (int c = c_begin; c < c_end; ++c) {
    const int t0 = (c * 32 + 32 <= BT) ? c * 32 : BT - 32;  // chunk start inside the tile
    const int tok = tok0 + t0;
    if (tok >= p.N) continue;  // p.N: tokens
    if (n_row0 >= p.M) continue;
    uint32_t r[32];
    tmem_ld_32x32b_x32(t_row + t0, r);
    tmem_ld_wait();
    if (lane == 0) bulk_wait_group_read<1>();  // the store issued two chunks ago has read this block
    __syncwarp();
    uint8_t* blk = staging_ptr + buf * 2048 + lane * 2;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      float v = __uint_as_float(r[j]);
      if (p.epilogue == EPI_DEQUANT) {
        if (!p.exact) v = __bfloat162float(__float2bfloat16_rn(v));
        if (p.exact == 2) {
          v = __fmul_rn(v, __fmul_rn(__ldg(p.row), cs));
          if (p.bias) v = __fadd_rn(v, bs);
        } else {
          Chain ch(v);
          if (p.row) ch.mul(__ldg(p.row + (int64_t)min(tok + j, p.N - 1) * p.row_stride));
          if (p.col) ch.mul(cs);
          if (p.bias) ch.add(bs);
          v = ch.done();
        }
      }
      const uint16_t h = p.out_dtype == IFLB200_F16 ? (uint16_t)f32_to_f16_bits(v) : (uint16_t)f32_to_bf16_bits(v);
      *reinterpret_cast<uint16_t*>(blk + j * 64) = h;
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(tm_out, staging + buf * 2048, n_row0, tok);
      bulk_commit_group();
    }
    buf ^= 1;
  }
}

// SPLIT: 0 = never a cluster split-K, 1 = always (p.split_k > 1), 2 = decided by p.split_k.  The
// wide-tile kernels of the large-M regime exist in forms 0 and 1: measured inside the M = 816 layer
// stack, a kernel that carries both code paths ran the stack 5 % slower than the two specialised
// ones.  The 64-wide kernel of the skinny-M regime exists only in form 2, so that the launches of a
// layer, split or not, run the same code: there a second GEMM kernel per layer cost about 1 us per
// launch in instruction fetch (0.2 ms per pass of the M = 50 stack).
// GATED: the gated form (see epilogue_gated): a tile pairs BN/2 gate columns with the BN/2 up
// columns of the same hidden units; p.N counts hidden units.
// EW: epilogue warps (8, or 16 for the gated form: EW / 4 per TMEM lane quadrant).
template <int BN, int STAGES, int SPLIT, bool SWAP = false, bool GATED = false, int EW = kEpilogueWarps, int SL = 1>
__global__ void __launch_bounds__(64 + 32 * EW, 1)
gemm_fp8_tc5_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w,
                    const __grid_constant__ CUtensorMap tm_out, const GemmParams p) {
  using L = SmemLayout<BN, STAGES, EW, SL>;
  static_assert(EW == kEpilogueWarps || GATED, "only the gated epilogue is written for more than eight warps");
  static_assert(SL == 1 || (!GATED && !SWAP), "several slabs per load: ordinary form only");
  // two accumulators, each at a power-of-two column offset; BN in {64, 128, 192, 224, 256}
  constexpr uint32_t kAccStride = BN <= 64 ? 64 : (BN <= 128 ? 128 : 256);
  constexpr uint32_t kTmemCols = 2 * kAccStride;
  constexpr uint32_t kIdesc = make_idesc_e4m3_f32(BM, BN);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);

  const uint32_t bar0 = base + L::kBarOffset;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kBarOffset + L::kNumBars * 8);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
#ifdef IFLB200_TRACE
  __shared__ unsigned int trace_id_s;
  if (threadIdx.x == 0) {
    trace_id_s = blockIdx.x == 0 ? atomicAdd(&g_gemm_trace_launch, 1u) : 0u;
    if (blockIdx.x == 0) {
      g_gemm_trace_cur = trace_id_s;
      g_gemm_trace[trace_id_s & 63][0] = globaltimer_ns();
      g_gemm_trace[trace_id_s & 63][1] = (unsigned long long)clock64();
    }
  }
  __syncthreads();
  const unsigned int trace_id = trace_id_s;
#endif
  // Split-K: the S CTAs of a cluster work on the same tile, CTA r on K steps [kb0, kb1); one
  // tile per CTA (the host launches tiles x S CTAs, at most one wave).
  // Partials: K split over independent CTAs (no cluster), each writing its fp32 partial sums.
  const bool partials = SPLIT == 2 && p.partials > 1;
  const bool split = !partials && (SPLIT == 1 || (SPLIT == 2 && p.split_k > 1));
  const int k_parts = partials ? p.partials : (split ? p.split_k : 1);
  const int split_rank = partials ? (int)blockIdx.x % k_parts : (split ? (int)cluster_ctarank() : 0);
  const int tile_first = k_parts > 1 ? (int)blockIdx.x / k_parts : (int)blockIdx.x;
  const int tile_stride = k_parts > 1 ? p.num_tiles : (int)gridDim.x;
  // K ranges in whole stages (SL slabs each)
  const int k_stages = (p.num_k + SL - 1) / SL;
  const int kb0 = k_parts > 1 ? (int)(((int64_t)k_stages * split_rank) / k_parts) * SL : 0;
  const int kb1 = k_parts > 1 ? min(p.num_k, (int)(((int64_t)k_stages * (split_rank + 1)) / k_parts) * SL) : p.num_k;

  if (threadIdx.x == 0) {
    prefetch_tensormap(&tm_a);
    prefetch_tensormap(&tm_w);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), EW);  // one arrival per epilogue warp
    }
    tmem_slot[1] = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) GEMM_TRACE(2);  // barriers initialised, tensor memory allocated

  // Everything above touched no global memory.  While the kernel before this one in the stream
  // drains, pull the first W boxes of this CTA's first tile towards L2 (a prefetch cannot read
  // stale data into the kernel: the loads proper are issued after the dependency wait and L2 is
  // the coherence point), then wait for that kernel's results.
  if (warp == 0 && lane == 0 && tile_first < p.num_tiles) {
    int m_blk, n_blk, grp;
    tile_place(p, tile_first, m_blk, n_blk, grp);
    const int kb_end = kb1 < kb0 + kPrefetchSteps ? kb1 : kb0 + kPrefetchSteps;
    for (int kb = kb0; kb < kb_end; kb += SL) {
      if constexpr (GATED) {
        tma_prefetch_l2_3d(&tm_w, kb * BK, n_blk * (BN / 2), 0);
      } else if constexpr (SL > 1) {
        tma_prefetch_l2_3d(&tm_w, 0, n_blk * BN, kb);
      } else {
        tma_prefetch_l2_2d(&tm_w, kb * BK, n_blk * BN);
      }
    }
  }

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // The one thread that issues loads waits for the kernel before this one; the epilogue warps
    // are ordered behind it through the barriers (and re-check below), the MMA warp touches no
    // global memory.  Fewer waiting threads matter: a CTA that became resident early sits beside
    // a kernel that is still running.
    // The weight boxes of the first stages are issued BEFORE the dependency wait.  The weights are not
    // an output of the kernel before this one (the activations are), so their DRAM round trip -- the
    // longest single latency of a 4 us skinny kernel -- runs while that kernel drains; after the wait
    // only the activation boxes (mostly L2 hits) remain.  (Contract: see iflb200_gemm_fp8_raw.)
    int early = 0;
    if constexpr (!SWAP) {  // (in the swapped form the operand behind tm_a is the weight matrix)
      if (lane == 0 && tile_first < p.num_tiles) {
        int m_blk, n_blk, grp;
        tile_place(p, tile_first, m_blk, n_blk, grp);
        for (int kb = kb0; kb < kb1 && early < STAGES; kb += SL, ++early) {
          mbar_arrive_expect_tx(full_bar(early), (uint32_t)(SL * p.a_bytes) + L::kBBytes);
          const uint32_t sw = base + early * L::kStageBytes + L::kABytes;
          if constexpr (SL > 1) tma_load_3d(sw, &tm_w, full_bar(early), 0, n_blk * BN, kb);
          else if constexpr (GATED) tma_load_3d(sw, &tm_w, full_bar(early), kb * BK, n_blk * (BN / 2), 0);
          else tma_load_2d(sw, &tm_w, full_bar(early), kb * BK, n_blk * BN);
        }
      }
      early = __shfl_sync(0xFFFFFFFFu, early, 0);
    }
    if (lane == 0) grid_dependency_wait();
    if (lane == 0) GEMM_TRACE(3);  // the kernel before this one has completed
    __syncwarp();
    int stage = 0;
    uint32_t phase = 0;
    uint32_t armed = (1u << early) - 1u;  // stages armed at least once (the early ones: first phase, parity 0)
    uint32_t last_parity = 0;             // parity of the last arming per stage
    bool ok = true;
    uint32_t it = 0;
    int fill = 0;              // stage fills issued so far
    for (int tile = tile_first; ok && tile < p.num_tiles; tile += tile_stride, ++it) {
      int m_blk, n_blk, grp;
      tile_place(p, tile, m_blk, n_blk, grp);
      const int a_row = grp * p.group_rows + m_blk * BM;  // rows past a block's end belong to the next block: loaded, never stored
      for (int kb = kb0; kb < kb1; kb += SL, ++fill) {
        if (fill < early) {
          // armed above with its weight box in flight (stage == fill, first phase): the activation box only
          if (lane == 0) {
            if constexpr (SL > 1) tma_load_3d(base + stage * L::kStageBytes, &tm_a, full_bar(stage), 0, a_row, kb);
            else tma_load_2d(base + stage * L::kStageBytes, &tm_a, full_bar(stage), kb * BK, a_row);
          }
          armed |= 1u << stage;
          last_parity = (last_parity & ~(1u << stage)) | (phase << stage);
          __syncwarp();
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
          continue;
        }
        ok = __all_sync(0xFFFFFFFFu, wait_bounded(empty_bar(stage), phase ^ 1, abort_flag,
                                                  (1u << 24) | (1u << 16) | (it & 0xFFFF)));
        if (!ok) break;
        if (lane == 0) {
          mbar_arrive_expect_tx(full_bar(stage), (uint32_t)(SL * p.a_bytes) + L::kBBytes);
          const uint32_t sa = base + stage * L::kStageBytes;
          if constexpr (SL > 1) {
            // SL slabs of each operand per instruction; slabs past the end of K read as zeros
            tma_load_3d(sa, &tm_a, full_bar(stage), 0, a_row, kb);
            tma_load_3d(sa + L::kABytes, &tm_w, full_bar(stage), 0, n_blk * BN, kb);
          } else {
          tma_load_2d(sa, &tm_a, full_bar(stage), kb * BK, a_row);
          if constexpr (GATED) {
            // gate rows, then the up rows of the same hidden units: one B operand of BN rows, one
            // load (the weight is mapped as [2][F][K]; a second TMA instruction per stage cost the
            // main loop about a tenth of its rate)
            tma_load_3d(sa + L::kABytes, &tm_w, full_bar(stage), kb * BK, n_blk * (BN / 2), 0);
          } else {
            tma_load_2d(sa + L::kABytes, &tm_w, full_bar(stage), kb * BK, n_blk * BN);
          }
          }
        }
        armed |= 1u << stage;
        last_parity = (last_parity & ~(1u << stage)) | (phase << stage);
        __syncwarp();
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
    // This CTA's last loads are in flight: the next kernel in the stream may be scheduled now
    // (it becomes resident as CTAs of this grid leave and waits for the grid to complete).
    // Not earlier: CTAs parked at their dependency wait for the length of a long GEMM slow it.
    grid_launch_dependents();
    // Drain: every load this warp issued must have landed before the CTA's shared memory can
    // go away.  Normal exit: the consumer has already waited on all of them, these return at
    // once.  Abort: bounded.
    for (int s = 0; s < STAGES; ++s) {
      if (armed & (1u << s)) {
        const uint32_t par = (last_parity >> s) & 1u;
        uint32_t spins = 0;
        while (!mbar_try_wait(full_bar(s), par) && ++spins < (1u << 20)) __nanosleep(64);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    uint32_t it = 0;
    for (int tile = tile_first; ok && tile < p.num_tiles; tile += tile_stride, ++it) {
      const uint32_t acc = it & 1u;
      const uint32_t acc_phase = (it >> 1) & 1u;
      ok = __all_sync(0xFFFFFFFFu, wait_bounded(tempty_bar(acc), acc_phase ^ 1, abort_flag,
                                                (2u << 24) | (2u << 16) | (it & 0xFFFF)));
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * kAccStride;
      for (int kb = kb0; kb < kb1; kb += SL) {
        ok = __all_sync(0xFFFFFFFFu, wait_bounded(full_bar(stage), phase, abort_flag,
                                                  (2u << 24) | (3u << 16) | (it & 0xFFFF)));
        if (!ok) break;
        tc_fence_after();
        if (lane == 0 && it == 0 && kb == kb0) GEMM_TRACE(4);  // first operands have landed
        if (lane == 0) {
          const uint32_t sa = base + stage * L::kStageBytes;
#pragma unroll
          for (int sl = 0; sl < SL; ++sl) {
            if (kb + sl >= kb1) break;  // slabs past the end of K (zeros) need no instruction
            // the activation slabs follow each other at the size of the box that brought them
            const uint64_t da = make_kmajor_sw128_desc(sa + sl * (SL > 1 ? p.a_bytes : 0));
            const uint64_t db = make_kmajor_sw128_desc(sa + L::kABytes + sl * BN * BK);
#pragma unroll
            for (int j = 0; j < BK / 32; ++j) {
              // 32 bytes further along K inside the swizzled 128-byte row: +2 in 16-byte units.
              mma_f8f6f4(d_tmem, da + 2 * j, db + 2 * j, kIdesc, (kb + sl > kb0 || j > 0) ? 1u : 0u);
            }
          }
          mma_commit(empty_bar(stage));  // stage reusable once these MMAs have read it
        }
        __syncwarp();
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (!ok) break;
      if (lane == 0) mma_commit(tfull_bar(acc));  // accumulator complete
      if (lane == 0 && it == 0) GEMM_TRACE(5);  // last MMA of the first tile issued
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int quad = warp & 3;  // TMEM lanes [32*quad, 32*quad+32) are this warp's
    const int half = (warp - 2) >> 2;  // which half of the tile's columns this warp drains
    // the two warps of a quadrant split the tile's columns at a multiple of 64 (one 128-byte
    // store of two-byte outputs): 128 | rest for wide tiles, half | half for 128, all | none for 64
    constexpr int kColSplit = BN > 128 ? 128 : (BN == 128 ? 64 : BN);
    int col_begin = half == 0 ? 0 : kColSplit, col_end = half == 0 ? kColSplit : BN;
    if (BN == 64 && p.tma_store && (p.out_dtype == IFLB200_F32 || p.half_rows)) {  // 32 columns per store and warp
      col_begin = half * 32;
      col_end = col_begin + 32;
    }
    const uint32_t staging = base + L::kStagingOffset + (uint32_t)(warp - 2) * (uint32_t)L::kWarpStaging;
    uint8_t* staging_ptr = smem + L::kStagingOffset + (warp - 2) * L::kWarpStaging;
    bool ok = true;
    uint32_t it = 0;
    int swap_buf = 0;
    for (int tile = tile_first; ok && tile < p.num_tiles; tile += tile_stride, ++it) {
      int m_blk, n_blk, grp;
      tile_place(p, tile, m_blk, n_blk, grp);
      const CUtensorMap* tm_dst = p.groups > 1 ? p.out_maps + grp : &tm_out;
      const uint32_t acc = it & 1u;
      const uint32_t acc_phase = (it >> 1) & 1u;
      // Before the accumulator is waited for: the kernel before this one in the stream (these warps
      // have nothing else to do until the first tile is complete, and the producer waits for the
      // same thing before its first load), then this tile's per-column operands and row scale, so
      // that their latency runs under the main loop instead of after it.
      if (it == 0) grid_dependency_wait();
      const int m = m_blk * BM + quad * 32 + lane;
      const bool row_ok = m < p.M;
      const bool prefetch = !SWAP && !GATED && !split && p.tma_store && p.epilogue != EPI_RAW && col_end - col_begin <= 128;
      ColumnVectors cv;
      float rs_early = 1.0f;
      if (prefetch) {
        cv = fetch_column_vectors(p, n_blk * BN + col_begin, col_end - col_begin, lane);
        rs_early = (row_ok && p.row) ? __ldg(p.row + (int64_t)(grp * p.group_rows + m) * p.row_stride) : 1.0f;
      }
      float cgl[4], cul[4];
      if constexpr (GATED) {
        gated_scales<BN, EW / 4>(p, n_blk * (BN / 2), half, lane, cgl, cul);
        rs_early = (row_ok && p.row) ? __ldg(p.row + (int64_t)m * p.row_stride) : 1.0f;
      }
      ok = __all_sync(0xFFFFFFFFu, wait_bounded(tfull_bar(acc), acc_phase, abort_flag,
                                                (3u << 24) | (4u << 16) | (it & 0xFFFF)));
      if (!ok) break;
      tc_fence_after();
      if (warp == 2 && lane == 0 && it == 0) GEMM_TRACE(6);  // first accumulator complete
      const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * kAccStride;
      if constexpr (SWAP) {
        epilogue_swapped<BN>(p, &tm_out, t_row, staging, staging_ptr, m_blk * BM + quad * 32, n_blk * BN, half, lane,
                             swap_buf);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(acc));
        continue;
      }
      const float rs = (prefetch || GATED) ? rs_early : ((row_ok && p.row) ? __ldg(p.row + (int64_t)m * p.row_stride) : 1.0f);
      if constexpr (GATED) {
        epilogue_gated<BN, EW / 4>(p, &tm_out, t_row, staging, staging_ptr, m_blk * BM + quad * 32, n_blk * (BN / 2),
                                   half, m, row_ok, rs, lane, cgl, cul);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(acc));
        continue;
      }
      const int64_t gofs = (row_ok && p.gate_index) ? (int64_t)p.gate_index[m] * p.N : 0;
      if (split) {
        // one tile per CTA: the partial accumulator stays in tensor memory; the exchange with
        // the other CTAs of the cluster follows the role loops
      } else if (p.tma_store) {
        // whole 128-byte pieces through shared memory and TMA; a 32-column remainder of a
        // 224-wide tile (two-byte outputs) straight from registers
        const int per_store = (p.out_dtype == IFLB200_F32 || p.half_rows) ? 32 : 64;
        const int col_tma_end = col_begin + (col_end - col_begin) / per_store * per_store;
        epilogue_tma_store<BN>(p, tm_dst, t_row, staging, staging_ptr, m_blk * BM + quad * 32, n_blk * BN,
                               col_begin, col_tma_end, rs, lane,
                               (SPLIT == 2 && p.partials >= 1) ? split_rank : -1,  // a plane map takes a 3-D store
                               prefetch ? &cv : nullptr);
        if (BN % 64 != 0 && col_tma_end < col_end) {
          const int n0 = n_blk * BN + col_tma_end;
          if (n0 < p.N) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(t_row + col_tma_end, r);
            tmem_ld_wait();
            epilogue_chunk<BN>(p, r, m, n0, row_ok, rs, gofs);
          }
        }
      } else {
#pragma unroll 1
        for (int c = col_begin / 32; c < col_end / 32; ++c) {
          const int n0 = n_blk * BN + c * 32;
          if (n0 >= p.N) break;  // uniform
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_row + c * 32, r);
          tmem_ld_wait();
          epilogue_chunk<BN>(p, r, m, n0, row_ok, rs, gofs);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
    }
    if (warp == 2 && lane == 0) GEMM_TRACE(7);  // last store issued
    if (lane == 0) bulk_wait_group_read<0>();  // staging buffers no longer read by the TMA unit
    if (warp == 2 && lane == 0) GEMM_TRACE(8);  // and read by the TMA unit
    __syncwarp();
  }

  if (split) {
    // CTA r of the cluster reduces columns [r*BN/S, (r+1)*BN/S) of the tile: its own partial
    // comes from tensor memory, the peers write theirs into its shared memory, and the sum runs
    // in rank order (fixed, so the result does not depend on timing); then the consumer
    // arithmetic on the sums.  Nothing touches another CTA's memory after the second barrier, so
    // CTAs leave independently.
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = quad * 32 + lane;
    const bool reducing = warp >= 2 && !*abort_flag && tile_first < p.num_tiles;
    cluster_arrive();
    cluster_wait();  // every CTA of the cluster has finished its main loop: the stage rings are free
    if (reducing) {
      // Hand every column range to the CTA that reduces it: the values go straight into the
      // owner's shared memory (slot = this CTA's position among the owner's peers, column-major
      // so that lanes hit consecutive banks).  Remote stores are posted, no round trip per value.
      const int own = BN / p.split_k;
      const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16);  // accumulator 0: the only tile
#pragma unroll 1
      for (int c = half * (BN / 2); c < (half + 1) * (BN / 2); c += 32) {
        const int owner = c / own;
        if (owner == split_rank) continue;  // reduced here, from tensor memory
        const int slot = split_rank < owner ? split_rank : split_rank - 1;
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c, r);
        tmem_ld_wait();
        const uint32_t dst = map_to_cta(base, (uint32_t)owner) +
                             (uint32_t)(((slot * own + (c - owner * own)) * BM + row) * 4);
#pragma unroll
        for (int i = 0; i < 32; ++i) st_dsmem_f32(dst + (uint32_t)(i * BM * 4), __uint_as_float(r[i]));
      }
    }
    cluster_arrive();
    cluster_wait();  // the peers' columns have landed here
    uint32_t sum[2][32];
    int my_chunks = 0, c_first = 0;
    int m_blk = 0, n_blk = 0;
    if (reducing) {
      tile_coords(p, tile_first, m_blk, n_blk);
      const int own = BN / p.split_k;  // columns this CTA reduces (a multiple of 32, at most 128)
      const int n_chunks = own / 32;   // 1, 2 or 4: the two warps of a quadrant take adjacent halves
      my_chunks = n_chunks >= 2 ? n_chunks / 2 : (half == 0 ? 1 : 0);
      c_first = split_rank * own + (n_chunks >= 2 ? half * my_chunks * 32 : 0);
      const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16);  // accumulator 0: the only tile
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        if (k < my_chunks) {
          const int c = c_first + 32 * k;
          uint32_t mine[32];
          tmem_ld_32x32b_x32(t_row + c, mine);
          float rem[3][32];  // the peers in rank order (this CTA's own rank left out)
          const float* slots = reinterpret_cast<const float*>(smem);
#pragma unroll
          for (int q = 0; q < 3; ++q) {
            if (q + 1 < p.split_k) {
#pragma unroll
              for (int i = 0; i < 32; ++i) rem[q][i] = slots[(q * own + (c - split_rank * own) + i) * BM + row];
            }
          }
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float v = 0.0f;
#pragma unroll
            for (int r = 0; r < 4; ++r) {
              if (r < p.split_k) {
                const float before = r <= 2 ? rem[r <= 2 ? r : 0][i] : 0.0f;      // peer r when r < own rank
                const float after = r >= 1 ? rem[r >= 1 ? r - 1 : 0][i] : 0.0f;   // peer r when r > own rank
                const float t = r == split_rank ? __uint_as_float(mine[i]) : (r < split_rank ? before : after);
                v = r == 0 ? t : __fadd_rn(v, t);
              }
            }
            sum[k][i] = __float_as_uint(v);
          }
        }
      }
    }
    if (reducing && my_chunks > 0) {
      const int m = m_blk * BM + row;
      const bool row_ok = m < p.M;
      const float rs = (row_ok && p.row) ? __ldg(p.row + (int64_t)m * p.row_stride) : 1.0f;
      const int64_t gofs = (row_ok && p.gate_index) ? (int64_t)p.gate_index[m] * p.N : 0;
      const int per_store = (p.out_dtype == IFLB200_F32) ? 32 : 64;
      const int n_first = n_blk * BN + c_first;
      if (p.tma_store && my_chunks * 32 >= per_store && n_first < p.N) {
        uint8_t* mine_row = smem + L::kStagingOffset + (warp - 2) * 4096 + lane * 128;
        const uint32_t staging = base + L::kStagingOffset + (uint32_t)(warp - 2) * 4096u;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          if (k < my_chunks) {
            const int sub = (32 * k) % per_store;
            if (sub == 0 && k > 0) {
              if (lane == 0) bulk_wait_group_read<0>();  // the previous store has read the buffer
              __syncwarp();
            }
            stage_columns(p, sum[k], n_first + 32 * k, rs, mine_row, sub, lane);
            if (sub + 32 == per_store) {
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) {
                tma_store_2d(&tm_out, staging, n_first + 32 * k - sub, m_blk * BM + quad * 32);
                bulk_commit_group();
              }
            }
          }
        }
        if (lane == 0) bulk_wait_group_read<0>();
        __syncwarp();
      } else {
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int n0 = n_first + 32 * k;
          if (k < my_chunks && n0 < p.N) epilogue_chunk<BN>(p, sum[k], m, n0, row_ok, rs, gofs);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) GEMM_TRACE(9);  // all roles done
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// --------------------------------------------------------------------------------------------
// CTA-pair variant: one 256 x BN tile per pair of CTAs (a cluster of two, cta_group::2).
//
// Each CTA loads its own 128 rows of A and HALF of the W tile (BN/2 rows): 32 KB per 128-byte
// K step instead of 48 KB, for the same MMA work per SM.  The per-SM TMA request rate is what
// bounds the single-CTA kernel, so this is worth ~1.5x on the main loop, and the smaller stage
// leaves room for 6 stages.  The leader (even CTA) issues tcgen05.mma.cta_group::2, which reads
// both CTAs' shared memory and writes both CTAs' tensor memory (rows 0..127 of the tile in the
// leader, 128..255 in its peer).  Barriers: both CTAs' TMA loads complete on the leader's
// "full" barrier; the leader's commits arrive on the "empty" / "accumulator full" barriers of
// both CTAs; both CTAs' epilogue warps arrive on the leader's "accumulator empty" barrier.
// --------------------------------------------------------------------------------------------
template <int BN, int STAGES>
struct PairSmemLayout {
  static constexpr int kABytes = BM * BK;
  static constexpr int kBBytes = (BN / 2) * BK;
  static constexpr int kStageBytes = kABytes + kBBytes;  // per CTA
  static constexpr int kStagingOffset = STAGES * kStageBytes;
  static constexpr int kBarOffset = kStagingOffset + kStagingBytes;
  static constexpr int kNumBars = 2 * STAGES + 4;
  static constexpr int kTotal = kBarOffset + kNumBars * 8 + 16;
  static constexpr int kDynamic = kTotal + 1024;
};

template <int BN, int STAGES, int ACC, bool SWAP = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_fp8_tc5_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w,
                         const __grid_constant__ CUtensorMap tm_out, const GemmParams p) {
  using L = PairSmemLayout<BN, STAGES>;
  constexpr uint32_t kAccStride = BN <= 128 ? 128 : 256;  // accumulators at power-of-two column offsets
  constexpr uint32_t kTmemCols = ACC * kAccStride;         // 256 or 512
  constexpr uint32_t kIdesc = make_idesc_e4m3_f32(2 * BM, BN);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);

  const uint32_t bar0 = base + L::kBarOffset;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + 2 + a); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kBarOffset + L::kNumBars * 8);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x >> 1;
  const int pair_stride = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);   // leader's producer arms it; bytes of both CTAs complete it
      mbar_init(empty_bar(s), 1);  // one multicast commit from the leader
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 2 * kEpilogueWarps);  // the epilogue warps of both CTAs
    }
    tmem_slot[1] = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish_pair();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tm_a);
    prefetch_tensormap(&tm_w);
  }
  tc_fence_before();
  cluster_sync_all();  // barriers of both CTAs initialised before any remote signal
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  grid_dependency_wait();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    uint32_t it = 0;
    for (int tile = pair_id; ok && tile < p.num_tiles; tile += pair_stride, ++it) {
      int m_blk, n_blk;
      tile_coords(p, tile, m_blk, n_blk);
      const int m0 = m_blk * 2 * BM + (int)rank * BM;
      const int n0 = n_blk * BN + (int)rank * (BN / 2);
      for (int kb = 0; kb < p.num_k; ++kb) {
        ok = __all_sync(0xFFFFFFFFu, wait_bounded(empty_bar(stage), phase ^ 1, abort_flag,
                                                  (1u << 24) | (1u << 16) | (it & 0xFFFF)));
        if (!ok) break;
        if (lane == 0) {
          if (leader) mbar_arrive_expect_tx(full_bar(stage), 2 * L::kStageBytes);
          const uint32_t sa = base + stage * L::kStageBytes;
          const uint32_t lead_full = full_bar(stage) & kPeerBitMask;
          tma_load_2d_pair(sa, &tm_a, lead_full, kb * BK, m0);
          tma_load_2d_pair(sa + L::kABytes, &tm_w, lead_full, kb * BK, n0);
        }
        __syncwarp();
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
    grid_launch_dependents();  // last loads issued: the next kernel may be scheduled
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader only)
    if (leader) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      uint32_t it = 0;
      for (int tile = pair_id; ok && tile < p.num_tiles; tile += pair_stride, ++it) {
        const uint32_t acc = (ACC == 2) ? (it & 1u) : 0u;
        const uint32_t acc_phase = (ACC == 2) ? ((it >> 1) & 1u) : (it & 1u);
        ok = __all_sync(0xFFFFFFFFu, wait_bounded(tempty_bar(acc), acc_phase ^ 1, abort_flag,
                                                  (2u << 24) | (2u << 16) | (it & 0xFFFF)));
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kAccStride;
        for (int kb = 0; kb < p.num_k; ++kb) {
          ok = __all_sync(0xFFFFFFFFu, wait_bounded(full_bar(stage), phase, abort_flag,
                                                    (2u << 24) | (3u << 16) | (it & 0xFFFF)));
          if (!ok) break;
          tc_fence_after();
          if (lane == 0) {
            const uint32_t sa = base + stage * L::kStageBytes;
            const uint64_t da = make_kmajor_sw128_desc(sa);
            const uint64_t db = make_kmajor_sw128_desc(sa + L::kABytes);
#pragma unroll
            for (int j = 0; j < BK / 32; ++j)
              mma_f8f6f4_pair(d_tmem, da + 2 * j, db + 2 * j, kIdesc, (kb | j) != 0 ? 1u : 0u);
            mma_commit_pair(empty_bar(stage), 3);  // stage free in both CTAs
          }
          __syncwarp();
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        if (lane == 0) mma_commit_pair(tfull_bar(acc), 3);  // accumulator complete in both CTAs
        __syncwarp();
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps (both CTAs)
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    int col_begin = half * (BN / 2), col_end = col_begin + BN / 2;
    if (p.tma_store && BN / 2 < 128 / ((p.out_dtype == IFLB200_F32) ? 4 : 2)) {
      // a 64-wide tile of two-byte outputs is a single 128-byte store: the first warp of the
      // quadrant takes it all
      col_begin = 0;
      col_end = half == 0 ? BN : 0;
    }
    const uint32_t staging = base + L::kStagingOffset + (uint32_t)(warp - 2) * 4096u;
    uint8_t* staging_ptr = smem + L::kStagingOffset + (warp - 2) * 4096;
    bool ok = true;
    uint32_t it = 0;
    int swap_buf = 0;
    for (int tile = pair_id; ok && tile < p.num_tiles; tile += pair_stride, ++it) {
      int m_blk, n_blk;
      tile_coords(p, tile, m_blk, n_blk);
      const uint32_t acc = (ACC == 2) ? (it & 1u) : 0u;
      const uint32_t acc_phase = (ACC == 2) ? ((it >> 1) & 1u) : (it & 1u);
      const int m = m_blk * 2 * BM + (int)rank * BM + quad * 32 + lane;
      const bool row_ok = m < p.M;
      // this tile's per-column operands and row scale, fetched under the main loop (see ColumnVectors)
      const bool prefetch = !SWAP && p.tma_store && p.epilogue != EPI_RAW && col_end - col_begin <= 128;
      ColumnVectors cv;
      float rs_early = 1.0f;
      if (prefetch) {
        cv = fetch_column_vectors(p, n_blk * BN + col_begin, col_end - col_begin, lane);
        rs_early = (row_ok && p.row) ? __ldg(p.row + (int64_t)m * p.row_stride) : 1.0f;
      }
      ok = __all_sync(0xFFFFFFFFu, wait_bounded(tfull_bar(acc), acc_phase, abort_flag,
                                                (3u << 24) | (4u << 16) | (it & 0xFFFF)));
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * kAccStride;
      if constexpr (SWAP) {
        epilogue_swapped<BN>(p, &tm_out, t_row, staging, staging_ptr, m_blk * 2 * BM + (int)rank * BM + quad * 32,
                             n_blk * BN, half, lane, swap_buf);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(tempty_bar(acc), 0);
        continue;
      }
      const float rs = prefetch ? rs_early : ((row_ok && p.row) ? __ldg(p.row + (int64_t)m * p.row_stride) : 1.0f);
      const int64_t gofs = (row_ok && p.gate_index) ? (int64_t)p.gate_index[m] * p.N : 0;
      if (p.tma_store) {
        epilogue_tma_store<BN>(p, &tm_out, t_row, staging, staging_ptr,
                               m_blk * 2 * BM + (int)rank * BM + quad * 32, n_blk * BN, col_begin, col_end, rs, lane,
                               -1, prefetch ? &cv : nullptr);
      } else {
#pragma unroll 1
        for (int c = col_begin / 32; c < col_end / 32; ++c) {
          const int n0 = n_blk * BN + c * 32;
          if (n0 >= p.N) break;
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_row + c * 32, r);
          tmem_ld_wait();
          epilogue_chunk<BN>(p, r, m, n0, row_ok, rs, gofs);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty_bar(acc), 0);  // on the leader's barrier
    }
    if (lane == 0) bulk_wait_group_read<0>();
    __syncwarp();
  }

  // No CTA of the pair may leave (or free tensor memory) while its peer can still read its
  // shared memory, write its tensor memory or signal its barriers.  After a timed-out wait,
  // give loads that are still in flight time to land before shared memory goes away.
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

// --------------------------------------------------------------------------------------------
// Host side
// --------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// [rows, K] e4m3 matrix, K contiguous, row stride ld bytes; box = 128 bytes x box_rows with the
// 128-byte swizzle; out-of-range elements read as zero.
static int make_tensor_map(CUtensorMap* tm, const void* ptr, int rows, int K, int64_t ld, int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return IFLB200_ERR_DRIVER;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box,
                         estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? IFLB200_OK : IFLB200_ERR_DRIVER;
}

// [rows, K] e4m3 matrix, K a multiple of 128, seen as [K / 128][rows][128 bytes]: box = 128 bytes x
// box_rows x `slabs`, so that one load brings `slabs` consecutive 128-byte K slabs of the tile, each
// laid out in shared memory like the box of make_tensor_map.
static int make_slab_map(CUtensorMap* tm, const void* ptr, int rows, int K, int64_t ld, int box_rows, int slabs) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return IFLB200_ERR_DRIVER;
  const cuuint64_t dims[3] = {(cuuint64_t)BK, (cuuint64_t)rows, (cuuint64_t)(K / BK)};
  const cuuint64_t strides[2] = {(cuuint64_t)ld, (cuuint64_t)BK};
  const cuuint32_t box[3] = {(cuuint32_t)BK, (cuuint32_t)box_rows, (cuuint32_t)slabs};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? IFLB200_OK : IFLB200_ERR_DRIVER;
}

// The [gate | up] weight [2F, K] seen as [2][F][K]: box = 128 bytes x box_rows x 2, so that one
// load brings the gate rows and the up rows of the same hidden units, gate rows first.
static int make_gated_weight_map(CUtensorMap* tm, const void* ptr, int F, int K, int64_t ld, int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return IFLB200_ERR_DRIVER;
  const cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)F, 2};
  const cuuint64_t strides[2] = {(cuuint64_t)ld, (cuuint64_t)ld * (cuuint64_t)F};
  const cuuint32_t box[3] = {(cuuint32_t)BK, (cuuint32_t)box_rows, 2};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? IFLB200_OK : IFLB200_ERR_DRIVER;
}

// [M, N] output matrix of 2- or 4-byte elements; box = 128 bytes x 32 rows, 128-byte swizzle.
static int make_out_map(CUtensorMap* tm, void* ptr, int M, int N, int64_t ld, int esize, int row_bytes = 128) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return IFLB200_ERR_DRIVER;
  const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * esize};
  const cuuint32_t box[2] = {(cuuint32_t)(row_bytes / esize), 32u};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(tm, esize == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, ptr,
                         dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? IFLB200_OK : IFLB200_ERR_DRIVER;
}

// [tokens, N] output of two-byte elements for the swapped form: box = 32 columns (64 bytes) x 32
// token rows, no swizzle.
static int make_out_map_swapped(CUtensorMap* tm, void* ptr, int tokens, int N, int64_t ld) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return IFLB200_ERR_DRIVER;
  const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)tokens};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {32u, 32u};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, ptr, dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? IFLB200_OK : IFLB200_ERR_DRIVER;
}

// Rows of the activation box.  The MMA always reads 128 rows of the stage, but with at most 120
// activation rows the box only brings the rows that exist (rounded up to the 8-row swizzle atom):
// the TMA unit issues one request per 128-byte box row whether the row exists or not, and for a
// skinny GEMM those requests -- not the weight bytes -- are what the main loop waits for.  The rows
// of the stage that are never written hold stale shared memory; they only reach accumulator rows
// >= M, which no epilogue stores.
static int activation_box_rows(int M) { return M <= 120 ? (M + 7) / 8 * 8 : BM; }

struct DeviceInfo {
  int sm_count = 0;
  int cc_major = 0;
  bool ready = false;
};
static DeviceInfo g_dev[64];

static int device_info(DeviceInfo** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return IFLB200_ERR_DEVICE;
  DeviceInfo& d = g_dev[dev];
  if (!d.ready) {
    e = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return (int)e;
    e = cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return (int)e;
    d.ready = true;
  }
  if (d.cc_major != 10) return IFLB200_ERR_DEVICE;
  *out = &d;
  return IFLB200_OK;
}

int g_dependent_launch = 1;
// what the last call of run_gemm launched: {family, tile width, split_k, stages}; family 1 = single-CTA
// tiles, 2 / 3 = CTA pairs with one / two accumulators, +4 = swapped form, +8 = gated (paired columns)
static int g_last_launch[4] = {0, 0, 0, 0};
static int g_cfg_tile_n = 0, g_cfg_stages = 0, g_cfg_group_m = 0;
static int g_cfg_split_k = 0;  // 0: cost model, 1: never split K, 2/4/8: forced
static int g_cfg_direct_store = 0;  // 1: epilogue stores straight from registers (experiments)
static int g_cfg_pair_swap = 1;  // the swapped form on CTA pairs where the shape allows
static int g_cfg_swap = 0;  // 0: cost model, 1: never, 2: always where the form exists
static int g_cfg_slabs = 0;  // 1: one K slab per TMA instruction everywhere (experiments)
static int g_cfg_gated_warps = 0;  // gated form, 256-wide tiles: 0 heuristic, 8 or 16 epilogue warps
static int g_cfg_mode = 0;  // 0 auto, 1 single-CTA tiles only, 2 CTA pairs with one accumulator, 3 CTA pairs with two

template <int BN, int STAGES, int SPLIT, bool SWAP = false, bool GATED = false, int EW = kEpilogueWarps, int SL = 1>
static int launch_gemm_form(const CUtensorMap& ta, const CUtensorMap& tw, const CUtensorMap& to, const GemmParams& p,
                            int grid, cudaStream_t s) {
  using L = SmemLayout<BN, STAGES, EW, SL>;
  static_assert(L::kDynamic <= 227 * 1024, "stage ring + staging exceed the shared memory of an SM");
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return IFLB200_ERR_DEVICE;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fp8_tc5_kernel<BN, STAGES, SPLIT, SWAP, GATED, EW, SL>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic);
    if (e != cudaSuccess) return (int)e;
    attr_set[dev] = true;
  }
  const cudaError_t e = launch_dep(gemm_fp8_tc5_kernel<BN, STAGES, SPLIT, SWAP, GATED, EW, SL>, dim3(grid),
                                   dim3(64 + 32 * EW), L::kDynamic, s, p.split_k,
                                   dependent_launch_for(SWAP ? p.N : p.M), ta, tw, to, p);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

template <int BN, int STAGES>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tw, const CUtensorMap& to, const GemmParams& p,
                       int grid, cudaStream_t s) {
  if constexpr (BN == 64) {
    return launch_gemm_form<BN, STAGES, 2>(ta, tw, to, p, grid, s);
  } else {
    if constexpr ((BN & (BN - 1)) == 0) {  // the reduction splits power-of-two widths
      if (p.split_k > 1) return launch_gemm_form<BN, STAGES, 1>(ta, tw, to, p, grid, s);
    }
    return launch_gemm_form<BN, STAGES, 0>(ta, tw, to, p, grid, s);
  }
}

template <int BN, int STAGES, int ACC, bool SWAP = false>
static int launch_gemm_pair(const CUtensorMap& ta, const CUtensorMap& tw, const CUtensorMap& to,
                            const GemmParams& p, int grid, cudaStream_t s) {
  using L = PairSmemLayout<BN, STAGES>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fp8_tc5_pair_kernel<BN, STAGES, ACC, SWAP>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic);
    if (e != cudaSuccess) return (int)e;
    attr_set[dev] = true;
  }
  const cudaError_t e = launch_dep(gemm_fp8_tc5_pair_kernel<BN, STAGES, ACC, SWAP>, dim3(grid), dim3(kGemmThreads),
                                   L::kDynamic, s, 1, dependent_launch_for(SWAP ? p.N : p.M), ta, tw, to, p);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

static int run_gemm(const void* a, int64_t ld_a, const void* w, int64_t ld_w, GemmParams p, void* stream) {
  if (p.M < 0 || p.N < 0 || p.K < 0) return IFLB200_ERR_ARG;
  if (p.M == 0 || p.N == 0) return IFLB200_OK;
  if (!a || !w || !p.out) return IFLB200_ERR_ARG;
  if (p.K < 16 || p.K % 16 || p.N % 16) return IFLB200_ERR_SHAPE;
  if (ld_a < p.K || ld_w < p.K || p.ld_out < p.N) return IFLB200_ERR_ARG;
  const int oes = (p.out_dtype == IFLB200_F32) ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) || ld_a % 16 || ld_w % 16 ||
      (reinterpret_cast<uintptr_t>(p.out) & 15) || (p.ld_out * oes) % 16)
    return IFLB200_ERR_ALIGN;
  DeviceInfo* dev = nullptr;
  int st = device_info(&dev);
  if (st != IFLB200_OK) return st;

  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // Raw and dequant epilogues go through shared memory and TMA stores; the residual epilogue
  // updates its operand in place with plain loads and stores.
  CUtensorMap to;
  p.tma_store = (p.epilogue != EPI_RESIDUAL && g_cfg_direct_store == 0) ? 1 : 0;
  if (p.tma_store) {
    st = make_out_map(&to, p.out, p.M, p.N, p.ld_out, oes);
    if (st != IFLB200_OK) return st;
  } else {
    memset(&to, 0, sizeof(to));
  }
  // CTA pairs by choice of the heuristic.  A pair moves 32 KB per SM and K step instead of 48 KB
  // and its 256 x 256 tile takes about 0.87 of the time two SMs need for two 128 x 256 tiles
  // (measured per shape at M = 4680: 9216 x 3072 98.7 us on pairs in 10 waves against 103.7 us on
  // single CTAs in 9; 14336 x 3072 149.5 against 161.2; but 3072 x 14336 186 against 150 where the
  // pairs need 4 waves for 3).  So the pair kernel is taken when its wave count, weighted by that
  // factor, is below the single-CTA one.
  bool pair_by_heuristic = false;
  if (g_cfg_mode == 0 && g_cfg_tile_n == 0 && g_cfg_split_k == 0 && p.M >= 2048 && p.N >= 256) {
    const int64_t single_tiles = (int64_t)((p.M + BM - 1) / BM) * ((p.N + 255) / 256);
    const int64_t pair_tiles = (int64_t)((p.M + 2 * BM - 1) / (2 * BM)) * ((p.N + 255) / 256);
    const int64_t single_waves = (single_tiles + dev->sm_count - 1) / dev->sm_count;
    const int64_t pair_waves = (pair_tiles + dev->sm_count / 2 - 1) / (dev->sm_count / 2);
    pair_by_heuristic = pair_waves * 87 < single_waves * 100;
  }
  if ((g_cfg_mode >= 2 || pair_by_heuristic) && p.N >= 256) {
    // CTA pairs: 256 x 256 tiles, each CTA loads 128 rows of A and 128 rows of W per K step.
    constexpr int PBN = 256;
    p.num_m = (p.M + 2 * BM - 1) / (2 * BM);
    p.num_n = (p.N + PBN - 1) / PBN;
    p.num_k = (p.K + BK - 1) / BK;
    p.num_tiles = p.num_m * p.num_n;
    // band height (pair row blocks that run side by side and share W tiles through L2).  W is read
    // from DRAM once per band when it does not stay in L2 beside the output stream, so taller bands
    // read less (16384 x 15360 x 5120 with bands of 4: 1317 MB read for 163 MB of operands); a band's
    // own A rows must stay resident while the walk crosses the columns.  Measured inside the
    // M = 16384 stack: bands of 16 are 4 % faster than bands of 4, bands of 32 lose half of that
    // again; at M = 4680 (19 pair row blocks) one band of all rows is fastest (98.7 against 101.1 us
    // on 9216 x 3072).  So: 16, or every row block when a second band would be a sliver.
    p.group_m = g_cfg_group_m > 0 ? g_cfg_group_m : (p.num_m <= 24 ? p.num_m : 16);
    const int pairs = dev->sm_count / 2;
    const int grid = 2 * (p.num_tiles < pairs ? p.num_tiles : pairs);
    CUtensorMap ta, tw;
    st = make_tensor_map(&ta, a, p.M, p.K, ld_a, BM);
    if (st != IFLB200_OK) return st;
    st = make_tensor_map(&tw, w, p.N, p.K, ld_w, PBN / 2);
    if (st != IFLB200_OK) return st;
    g_last_launch[0] = g_cfg_mode == 2 ? 2 : 3; g_last_launch[1] = PBN; g_last_launch[2] = 1; g_last_launch[3] = 6;
    return g_cfg_mode == 2 ? launch_gemm_pair<PBN, 6, 1>(ta, tw, to, p, grid, s)
                           : launch_gemm_pair<PBN, 6, 2>(ta, tw, to, p, grid, s);  // two accumulators
  }

  // Tile width by a measured cost model: one 128-byte K step of a CTA costs about 590 / 690 /
  // 830 cycles for a 64 / 128 / 256 wide tile (24 / 32 / 48 KB through the SM's L2 port per
  // step; 192 and 224 interpolate), the kernel takes waves x steps x that, plus a fixed cost per
  // wave for prologue and the exposed epilogue.  The widths that are not powers of two are for
  // wave quantisation (7 row blocks x 32768 columns: 896 tiles of 256 = 6.05 waves of 148 SMs, i.e.
  // 7, but 1029 tiles of 224 = 6.95 waves of narrower tiles).  Timed alone the 224-wide kernel is
  // 2 % faster on that shape, inside the layer stack it was 4 us per launch slower (its 448-byte
  // tile rows start off the 128-byte line grid), so the model does not choose them by itself.
  p.num_m = (p.M + BM - 1) / BM;
  int bn = g_cfg_tile_n;
  int split = 1;
  {
    const int widths[5] = {256, 224, 192, 128, 64};
    const int64_t step_cycles[5] = {830, 790, 750, 690, 590};
    const int64_t steps = (p.K + BK - 1) / BK;
    int64_t best = 0;
    int best_bn = 0;
    for (int i = 0; i < 5; ++i) {
      if (g_cfg_tile_n && widths[i] != g_cfg_tile_n) continue;
      if (!g_cfg_tile_n && (widths[i] & (widths[i] - 1))) continue;  // 192 / 224: only when asked for (see above)
      if (!g_cfg_tile_n && widths[i] > 64 && p.N < widths[i]) continue;
      const int64_t tiles = (int64_t)p.num_m * ((p.N + widths[i] - 1) / widths[i]);
      // split-K over a cluster: one wave of tiles x S CTAs, S in {2, 4}, leaving each CTA >= 8 K
      // steps and >= 32 columns to reduce; the exchange of partials over distributed shared
      // memory, two cluster barriers and the reduction are a fixed cost per launch.
      for (int sk = 1; sk <= 4; sk *= 2) {
        if (g_cfg_split_k && sk != g_cfg_split_k) continue;
        if (sk > 1 && (tiles * sk > dev->sm_count || steps / sk < 8 || widths[i] / sk < 32)) continue;
        if (sk > 1 && (widths[i] & (widths[i] - 1))) continue;  // the reduction splits power-of-two widths
        const int64_t waves = sk > 1 ? 1 : (tiles + dev->sm_count - 1) / dev->sm_count;
        const int64_t cost = waves * ((steps / sk) * step_cycles[i] + 2500 + (sk > 1 ? 18000 : 0));
        if (best_bn == 0 || cost < best) {
          best = cost;
          best_bn = widths[i];
          split = sk;
        }
      }
    }
    if (best_bn == 0) return IFLB200_ERR_ARG;  // the forced configuration does not fit this problem
    bn = best_bn;
  }
  // Swapped form for a few hundred tokens: the tokens go on the MMA's N side in tiles of the width
  // that fits them (816 tokens = 4 x 208 with 2 % padding, where 7 row blocks of 128 carry 9 %), the
  // weight rows on its M side in blocks of 128 (256 on a CTA pair), and the epilogue stores the
  // tile transposed.  Same K loop, same accumulator bits.  Two-byte raw or dequantised outputs.
  // Measured on 816 x 32768 x 2048: 54.1 us on CTA pairs, 55.7 on single CTAs, against 53.9 for the
  // ordinary form (the main loops alone 44.8 / 46.2 / 45.5 us: a 208-wide MMA step is no shorter
  // than a 256-wide one), so the heuristic does not take it; iflb200_gemm_set_mode(256) does.
  if (g_cfg_swap != 1 && g_cfg_mode == 0 && g_cfg_tile_n == 0 && g_cfg_split_k == 0 && g_cfg_stages == 0 &&
      p.M > 256 && p.M <= 1024 && oes == 2 && p.tma_store && (p.epilogue == EPI_RAW || p.epilogue == EPI_DEQUANT)) {
    const int t_tiles = (p.M + 255) / 256;
    const int fit = ((p.M + t_tiles - 1) / t_tiles + 15) / 16 * 16;
    const int bt = fit <= 128 ? 128 : (fit <= 208 ? 208 : 256);  // the widths this form is built for
    const int64_t steps = (p.K + BK - 1) / BK;
    if (g_cfg_swap == 2) {
      GemmParams q = p;
      q.M = p.N;  // rows of the MMA's M side: output columns
      q.N = p.M;  // tokens
      q.num_m = (p.N + BM - 1) / BM;
      q.num_n = (p.M + bt - 1) / bt;
      q.num_k = (int)steps;
      q.num_tiles = q.num_m * q.num_n;
      q.group_m = g_cfg_group_m > 0 ? g_cfg_group_m : 8;
      q.split_k = 1;
      q.a_bytes = BM * BK;
      const int grid = q.num_tiles < dev->sm_count ? q.num_tiles : dev->sm_count;
      CUtensorMap tw_rows, ta_tokens, to_swapped;
      st = make_tensor_map(&tw_rows, w, p.N, p.K, ld_w, BM);
      if (st != IFLB200_OK) return st;
      st = make_tensor_map(&ta_tokens, a, p.M, p.K, ld_a, bt);
      if (st != IFLB200_OK) return st;
      st = make_out_map_swapped(&to_swapped, p.out, p.M, p.N, p.ld_out);
      if (st != IFLB200_OK) return st;
      if (p.N >= 2 * BM && bt >= 208 && g_cfg_pair_swap) {
        // weight rows in blocks of 256 on a CTA pair, each CTA loading half of the token tile
        q.num_m = (p.N + 2 * BM - 1) / (2 * BM);
        q.num_tiles = q.num_m * q.num_n;
        q.group_m = g_cfg_group_m > 0 ? g_cfg_group_m : 4;
        const int pairs = dev->sm_count / 2;
        const int pgrid = 2 * (q.num_tiles < pairs ? q.num_tiles : pairs);
        CUtensorMap ta_half;
        st = make_tensor_map(&ta_half, a, p.M, p.K, ld_a, bt / 2);
        if (st != IFLB200_OK) return st;
        g_last_launch[0] = 3 + 4; g_last_launch[1] = bt; g_last_launch[2] = 1; g_last_launch[3] = 6;
        return bt == 208 ? launch_gemm_pair<208, 6, 2, true>(tw_rows, ta_half, to_swapped, q, pgrid, s)
                         : launch_gemm_pair<256, 6, 2, true>(tw_rows, ta_half, to_swapped, q, pgrid, s);
      }
      g_last_launch[0] = 1 + 4; g_last_launch[1] = bt; g_last_launch[2] = 1; g_last_launch[3] = bt == 128 ? 6 : 4;
      switch (bt) {
        case 128: return launch_gemm_form<128, 6, 0, true>(tw_rows, ta_tokens, to_swapped, q, grid, s);
        case 208: return launch_gemm_form<208, 4, 0, true>(tw_rows, ta_tokens, to_swapped, q, grid, s);
        default: return launch_gemm_form<256, 4, 0, true>(tw_rows, ta_tokens, to_swapped, q, grid, s);
      }
    }
  }
  p.split_k = split;
  p.num_n = (p.N + bn - 1) / bn;
  p.num_k = (p.K + BK - 1) / BK;
  p.num_tiles = p.num_m * p.num_n;
  p.group_m = g_cfg_group_m > 0 ? g_cfg_group_m : 8;
  const int grid = split > 1 ? p.num_tiles * split : (p.num_tiles < dev->sm_count ? p.num_tiles : dev->sm_count);

  // 64-wide tiles of two-byte outputs with consumer arithmetic: a 64-byte piece per warp instead of
  // one 128-byte piece that the first warp of each quadrant stages alone (the epilogue of a skinny
  // launch overlaps nothing: 64 x 4096 x 1024 with scales and bias 5.7 -> 5.1 us; raw outputs, whose
  // staging is a handful of instructions, gain nothing from the second store and keep one piece).
  if (bn == 64 && split == 1 && p.tma_store && oes == 2 && p.epilogue != EPI_RAW) {
    st = make_out_map(&to, p.out, p.M, p.N, p.ld_out, oes, 64);
    if (st != IFLB200_OK) return st;
    p.half_rows = 1;
  }
  CUtensorMap ta, tw;
  const int a_rows = activation_box_rows(p.M);
  p.a_bytes = a_rows * BK;
  st = make_tensor_map(&ta, a, p.M, p.K, ld_a, a_rows);
  if (st != IFLB200_OK) return st;
  st = make_tensor_map(&tw, w, p.N, p.K, ld_w, bn);
  if (st != IFLB200_OK) return st;
  const int stages = g_cfg_stages;
  g_last_launch[0] = 1; g_last_launch[1] = bn; g_last_launch[2] = split; g_last_launch[3] = stages;
  // Skinny regime (64-wide tiles): four K slabs per TMA instruction where the layout allows it
  // (K a multiple of 128, at least one full stage per CTA); the K order is unchanged, so are the bits.
  if (bn == 64 && g_cfg_slabs != 1 && p.K % BK == 0 && p.num_k / split >= 4 && stages == 0) {
    CUtensorMap sa_map, sw_map;
    if (make_slab_map(&sa_map, a, p.M, p.K, ld_a, a_rows, 4) == IFLB200_OK &&
        make_slab_map(&sw_map, w, p.N, p.K, ld_w, bn, 4) == IFLB200_OK) {
      g_last_launch[3] = 104;
      return launch_gemm_form<64, 2, 2, false, false, kEpilogueWarps, 4>(sa_map, sw_map, to, p, grid, s);
    }
  }
  switch (bn) {
    case 256: return (stages == 3) ? launch_gemm<256, 3>(ta, tw, to, p, grid, s) : launch_gemm<256, 4>(ta, tw, to, p, grid, s);
    case 224: return launch_gemm<224, 4>(ta, tw, to, p, grid, s);
    case 192: return launch_gemm<192, 4>(ta, tw, to, p, grid, s);
    case 128: return (stages == 4) ? launch_gemm<128, 4>(ta, tw, to, p, grid, s) : launch_gemm<128, 6>(ta, tw, to, p, grid, s);
    case 64: return (stages == 4) ? launch_gemm<64, 4>(ta, tw, to, p, grid, s) : launch_gemm<64, 8>(ta, tw, to, p, grid, s);
    default: return IFLB200_ERR_ARG;
  }
}

// [splits][M][N] fp32 partial sums; box = 32 columns (128 bytes) x 32 rows x 1 plane.
static int make_partials_map(CUtensorMap* tm, void* ptr, int M, int N, int64_t ld, int splits) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return IFLB200_ERR_DRIVER;
  const cuuint64_t dims[3] = {(cuuint64_t)N, (cuuint64_t)M, (cuuint64_t)splits};
  const cuuint64_t strides[2] = {(cuuint64_t)ld * 4, (cuuint64_t)ld * 4 * (cuuint64_t)M};
  const cuuint32_t box[3] = {32u, 32u, 1u};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, ptr, dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? IFLB200_OK : IFLB200_ERR_DRIVER;
}

// Split-K over independent CTAs for skinny activations: out[s][m][n] = sum over the s-th K range of
// a[m,k] * w[n,k], fp32, no scales, no rounding; the consumer sums the planes in order (and rounds
// the sum to bf16, the raw accumulator's rounding point).  K a multiple of 128, M <= 128.
static int run_gemm_partials(const void* a, int64_t ld_a, const void* w, int64_t ld_w, int M, int N, int K, int splits,
                             float* out, int64_t ld_out, void* stream) {
  if (M < 0 || N < 0 || K < 0 || splits < 1) return IFLB200_ERR_ARG;
  if (M == 0 || N == 0) return IFLB200_OK;
  if (!a || !w || !out) return IFLB200_ERR_ARG;
  if (K < BK || K % BK || N % 16 || M > BM) return IFLB200_ERR_SHAPE;
  const int num_k = K / BK;
  if (splits > (num_k + 3) / 4) return IFLB200_ERR_SHAPE;  // every split owns at least one stage of four slabs
  if (ld_a < K || ld_w < K || ld_out < N) return IFLB200_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) || ld_a % 16 || ld_w % 16 ||
      (reinterpret_cast<uintptr_t>(out) & 15) || (ld_out * 4) % 16)
    return IFLB200_ERR_ALIGN;
  DeviceInfo* dev = nullptr;
  int st = device_info(&dev);
  if (st != IFLB200_OK) return st;
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.epilogue = EPI_DEQUANT;
  p.exact = 1;
  p.out = out; p.out_dtype = IFLB200_F32; p.ld_out = ld_out;
  p.split_k = 1;
  p.partials = splits;
  p.tma_store = 1;
  p.num_m = 1;
  p.num_n = (N + 63) / 64;
  p.num_k = num_k;
  p.num_tiles = p.num_n;
  p.group_m = 1;
  const int a_rows = activation_box_rows(M);
  p.a_bytes = a_rows * BK;
  CUtensorMap ta, tw, to;
  st = make_slab_map(&ta, a, M, K, ld_a, a_rows, 4);
  if (st != IFLB200_OK) return st;
  st = make_slab_map(&tw, w, N, K, ld_w, 64, 4);
  if (st != IFLB200_OK) return st;
  st = make_partials_map(&to, out, M, N, ld_out, splits);
  if (st != IFLB200_OK) return st;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  g_last_launch[0] = 1 + 16; g_last_launch[1] = 64; g_last_launch[2] = splits; g_last_launch[3] = 104;
  return launch_gemm_form<64, 2, 2, false, false, kEpilogueWarps, 4>(ta, tw, to, p, p.num_tiles * splits, s);
}

// Row blocks to several destinations: a holds `groups` blocks of `group_rows` rows; block g's
// fp32 accumulators (no scales, no rounding) go through d_out_maps[g], tensor maps in DEVICE memory
// encoded by iflb200_encode_rowblock_map for [group_rows][N] fp32 buffers (on this GPU or a peer).
static int run_gemm_rowblocks(const void* a, int64_t ld_a, const void* w, int64_t ld_w, int groups, int group_rows,
                              int N, int K, const void* d_out_maps, void* stream) {
  if (groups < 1 || groups > 64 || group_rows < 0 || N < 0 || K < 0) return IFLB200_ERR_ARG;
  if (group_rows == 0 || N == 0) return IFLB200_OK;
  if (!a || !w || !d_out_maps) return IFLB200_ERR_ARG;
  if (K < 16 || K % 16 || N % 16) return IFLB200_ERR_SHAPE;
  if (ld_a < K || ld_w < K) return IFLB200_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) || ld_a % 16 || ld_w % 16 ||
      (reinterpret_cast<uintptr_t>(d_out_maps) & 63))
    return IFLB200_ERR_ALIGN;
  DeviceInfo* dev = nullptr;
  int st = device_info(&dev);
  if (st != IFLB200_OK) return st;
  GemmParams p = {};
  p.M = group_rows; p.N = N; p.K = K;
  p.epilogue = EPI_DEQUANT;
  p.exact = 1;
  p.out = nullptr; p.out_dtype = IFLB200_F32; p.ld_out = N;
  p.split_k = 1;
  p.tma_store = 1;
  p.groups = groups; p.group_rows = group_rows;
  p.out_maps = reinterpret_cast<const CUtensorMap*>(d_out_maps);
  const int bn = N >= 256 ? 256 : (N >= 128 ? 128 : 64);
  p.num_m = (group_rows + BM - 1) / BM;
  p.num_n = (N + bn - 1) / bn;
  p.num_k = (K + BK - 1) / BK;
  p.num_tiles = groups * p.num_m * p.num_n;
  p.group_m = g_cfg_group_m > 0 ? g_cfg_group_m : 8;
  p.a_bytes = BM * BK;
  const int grid = p.num_tiles < dev->sm_count ? p.num_tiles : dev->sm_count;
  CUtensorMap ta, tw, to;
  memset(&to, 0, sizeof(to));
  st = make_tensor_map(&ta, a, groups * group_rows, K, ld_a, BM);
  if (st != IFLB200_OK) return st;
  st = make_tensor_map(&tw, w, N, K, ld_w, bn);
  if (st != IFLB200_OK) return st;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  g_last_launch[0] = 1 + 32; g_last_launch[1] = bn; g_last_launch[2] = 1; g_last_launch[3] = 0;
  switch (bn) {
    case 256: return launch_gemm<256, 4>(ta, tw, to, p, grid, s);
    case 128: return launch_gemm<128, 6>(ta, tw, to, p, grid, s);
    default: return launch_gemm<64, 8>(ta, tw, to, p, grid, s);
  }
}

// The gated form: W is [2F, K] = [gate rows | up rows]; h [M, F] fp32; amax [M] float bits.
static int run_gemm_gated(const void* a, int64_t ld_a, const void* w, int64_t ld_w, int M, int F, int K,
                          const float* row, const float* col, int act, float* h, int64_t ld_h, uint32_t* amax,
                          void* stream) {
  if (M < 0 || F < 0 || K < 0) return IFLB200_ERR_ARG;
  if (M == 0 || F == 0) return IFLB200_OK;
  if (!a || !w || !h || !amax) return IFLB200_ERR_ARG;
  if (act != IFLB200_ACT_GELU_TANH && act != IFLB200_ACT_SILU) return IFLB200_ERR_ARG;
  if (K < 16 || K % 16 || F % 16) return IFLB200_ERR_SHAPE;
  if (ld_a < K || ld_w < K || ld_h < F) return IFLB200_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) || ld_a % 16 || ld_w % 16 ||
      (reinterpret_cast<uintptr_t>(h) & 15) || (ld_h * 4) % 16 || (reinterpret_cast<uintptr_t>(amax) & 3))
    return IFLB200_ERR_ALIGN;
  DeviceInfo* dev = nullptr;
  int st = device_info(&dev);
  if (st != IFLB200_OK) return st;
  GemmParams p = {};
  p.M = M; p.N = F; p.K = K;
  p.epilogue = EPI_RAW;
  p.row = row; p.row_stride = 1;
  p.col = col; p.col_stride = 1;
  p.out = h; p.out_dtype = IFLB200_F32; p.ld_out = ld_h;
  p.split_k = 1;
  p.act = act;
  p.amax = amax;
  p.tma_store = 1;
  p.num_m = (M + BM - 1) / BM;
  p.num_k = (K + BK - 1) / BK;
  // tile width (gate + up columns) by the cost model of the ordinary form
  const int widths[3] = {256, 128, 64};
  const int64_t step_cycles[3] = {830, 690, 590};
  int bn = g_cfg_tile_n == 256 || g_cfg_tile_n == 128 || g_cfg_tile_n == 64 ? g_cfg_tile_n : 0;
  if (bn == 0) {
    int64_t best = 0;
    for (int i = 0; i < 3; ++i) {
      const int64_t tiles = (int64_t)p.num_m * ((F + widths[i] / 2 - 1) / (widths[i] / 2));
      const int64_t waves = (tiles + dev->sm_count - 1) / dev->sm_count;
      const int64_t cost = waves * (p.num_k * step_cycles[i] + 2500);
      if (bn == 0 || cost < best) {
        best = cost;
        bn = widths[i];
      }
    }
  }
  p.num_n = (F + bn / 2 - 1) / (bn / 2);
  p.num_tiles = p.num_m * p.num_n;
  p.group_m = g_cfg_group_m > 0 ? g_cfg_group_m : 8;
  const int grid = p.num_tiles < dev->sm_count ? p.num_tiles : dev->sm_count;
  CUtensorMap ta, tw, to;
  const int a_rows = activation_box_rows(M);
  p.a_bytes = a_rows * BK;
  st = make_tensor_map(&ta, a, M, K, ld_a, a_rows);
  if (st != IFLB200_OK) return st;
  st = make_gated_weight_map(&tw, w, F, K, ld_w, bn / 2);
  if (st != IFLB200_OK) return st;
  // sixteen epilogue warps unless eight are asked for: the activation's arithmetic per element is
  // heavy enough that the epilogue of a CTA's last tile, which nothing overlaps, is worth halving
  const bool sixteen = bn == 256 && g_cfg_gated_warps != 8;
  st = make_out_map(&to, h, M, F, ld_h, 4, sixteen ? 64 : 128);
  if (st != IFLB200_OK) return st;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  g_last_launch[0] = 1 + 8; g_last_launch[1] = bn; g_last_launch[2] = 1; g_last_launch[3] = 0;
  switch (bn) {
    case 256:
      // sixteen epilogue warps (64 bytes of staging per row each), or eight
      if (sixteen) return launch_gemm_form<256, 4, 0, false, true, 16>(ta, tw, to, p, grid, s);
      return launch_gemm_form<256, 4, 0, false, true>(ta, tw, to, p, grid, s);
    case 128: return launch_gemm_form<128, 6, 0, false, true>(ta, tw, to, p, grid, s);
    default: return launch_gemm_form<64, 8, 0, false, true>(ta, tw, to, p, grid, s);
  }
}

}  // namespace iflb200

using namespace iflb200;

extern "C" int iflb200_gemm_set_config(int tile_n, int stages, int group_m) {
  if (tile_n != 0 && tile_n != 64 && tile_n != 128 && tile_n != 192 && tile_n != 224 && tile_n != 256)
    return IFLB200_ERR_ARG;
  if (stages < 0 || group_m < 0) return IFLB200_ERR_ARG;
  g_cfg_tile_n = tile_n;
  g_cfg_stages = stages;
  g_cfg_group_m = group_m;
  return IFLB200_OK;
}

extern "C" int iflb200_gemm_set_split_k(int split_k) {
  if (split_k != 0 && split_k != 1 && split_k != 2 && split_k != 4) return IFLB200_ERR_ARG;
  g_cfg_split_k = split_k;
  return IFLB200_OK;
}

extern "C" int iflb200_set_dependent_launch(int enable) {
  if (enable < 0 || enable > 2) return IFLB200_ERR_ARG;
  g_dependent_launch = enable;
  return IFLB200_OK;
}

extern "C" int iflb200_gemm_set_mode(int mode) {
  // bit 4 (value 16) selects the direct-store epilogue; the low bits the kernel family
  const int family = mode & 15;
  if (mode < 0 || family > 3 || (mode & ~(15 | 16 | 128 | 256 | 512 | 1024 | 2048 | 4096)) || (mode & 384) == 384 ||
      (mode & 3072) == 3072)
    return IFLB200_ERR_ARG;
  g_cfg_gated_warps = (mode & 1024) ? 16 : ((mode & 2048) ? 8 : 0);
  g_cfg_slabs = (mode & 4096) ? 1 : 0;
  g_cfg_swap = (mode & 128) ? 1 : ((mode & 256) ? 2 : 0);  // 128: never the swapped form, 256: wherever it exists
  g_cfg_pair_swap = (mode & 512) ? 0 : 1;                  // 512: the swapped form on single CTAs only
  g_cfg_mode = family;
  g_cfg_direct_store = (mode & 16) ? 1 : 0;
  return IFLB200_OK;
}

extern "C" int iflb200_set_wait_budget_us(int64_t microseconds) {
  if (microseconds < 0) return IFLB200_ERR_ARG;
  const uint64_t ns = microseconds ? (uint64_t)microseconds * 1000ull : kWaitBudgetNs;
  const cudaError_t e = cudaMemcpyToSymbol(g_gemm_wait_budget_ns, &ns, sizeof(ns));
  if (e != cudaSuccess) return (int)e;
  const int st = set_stack_wait_budget_ns(ns);
  return st != 0 ? st : set_peer_wait_budget_ns(ns);
}

extern "C" int iflb200_gemm_last_launch(int* family, int* tile_n, int* split_k) {
  if (family) *family = g_last_launch[0];
  if (tile_n) *tile_n = g_last_launch[1];
  if (split_k) *split_k = g_last_launch[2];
  return IFLB200_OK;
}

extern "C" int iflb200_gemm_take_timeout_record(uint32_t* record, void* stream) {
  if (!record) return IFLB200_ERR_ARG;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  uint32_t host[4] = {0, 0, 0, 0};
  cudaError_t e = cudaMemcpyFromSymbolAsync(host, g_timeout_record, sizeof(host), 0, cudaMemcpyDeviceToHost, s);
  if (e != cudaSuccess) return (int)e;
  e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return (int)e;
  *record = host[0];
  if (host[0] != 0) {
    const uint32_t zero[4] = {0, 0, 0, 0};
    e = cudaMemcpyToSymbolAsync(g_timeout_record, zero, sizeof(zero), 0, cudaMemcpyHostToDevice, s);
    if (e != cudaSuccess) return (int)e;
    e = cudaStreamSynchronize(s);
  }
  return (int)e;
}

extern "C" int iflb200_gemm_fp8_raw(const void* a, int64_t ld_a, const void* w, int64_t ld_w, int M, int N,
                                    int K, void* out, int64_t ld_out, void* stream) {
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.epilogue = EPI_RAW;
  p.out = out; p.out_dtype = IFLB200_BF16; p.ld_out = ld_out;
  return run_gemm(a, ld_a, w, ld_w, p, stream);
}

extern "C" int iflb200_fp8_linear(const void* a, int64_t ld_a, const void* w, int64_t ld_w, int M, int N,
                                  int K, const float* row_scale, int row_scale_stride,
                                  const float* col_scale, int col_scale_stride, const void* bias,
                                  int bias_dtype, int rounding, void* out, int out_dtype, int64_t ld_out,
                                  void* stream) {
  if (out_dtype != IFLB200_F32 && out_dtype != IFLB200_BF16 && out_dtype != IFLB200_F16) return IFLB200_ERR_DTYPE;
  if (bias && bias_dtype != IFLB200_F32 && bias_dtype != IFLB200_BF16) return IFLB200_ERR_DTYPE;
  if (rounding != IFLB200_ROUND_ENGINE && rounding != IFLB200_ROUND_EXACT) return IFLB200_ERR_ARG;
  if ((row_scale_stride | 1) != 1 || (col_scale_stride | 1) != 1) return IFLB200_ERR_ARG;
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.epilogue = EPI_DEQUANT;
  p.exact = rounding == IFLB200_ROUND_EXACT;
  if (p.exact && row_scale && col_scale && row_scale_stride == 0 && col_scale_stride == 0) p.exact = 2;
  p.row = row_scale; p.row_stride = row_scale_stride;
  p.col = col_scale; p.col_stride = col_scale_stride;
  p.bias = bias; p.bias_dtype = bias_dtype;
  p.out = out; p.out_dtype = out_dtype; p.ld_out = ld_out;
  return run_gemm(a, ld_a, w, ld_w, p, stream);
}

extern "C" int iflb200_fp8_linear_residual(const void* a, int64_t ld_a, const void* w, int64_t ld_w, int M,
                                           int N, int K, const float* row_scale, const float* col_scale,
                                           const float* bias, const float* gate, const int32_t* gate_index,
                                           void* res, int res_dtype, int64_t ld_res, void* stream) {
  if (res_dtype != IFLB200_F32 && res_dtype != IFLB200_BF16) return IFLB200_ERR_DTYPE;
  GemmParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.epilogue = EPI_RESIDUAL;
  p.row = row_scale; p.row_stride = 1;
  p.col = col_scale; p.col_stride = 1;
  p.bias = bias; p.bias_dtype = IFLB200_F32;
  p.gate = gate; p.gate_index = gate ? gate_index : nullptr;
  p.out = res; p.out_dtype = res_dtype; p.ld_out = ld_res;
  return run_gemm(a, ld_a, w, ld_w, p, stream);
}

extern "C" int iflb200_gemm_fp8_partials(const void* a, int64_t ld_a, const void* w, int64_t ld_w, int M, int N,
                                         int K, int splits, float* out, int64_t ld_out, void* stream) {
  return run_gemm_partials(a, ld_a, w, ld_w, M, N, K, splits, out, ld_out, stream);
}

extern "C" int iflb200_encode_rowblock_map(void* out, int rows, int N, int64_t ld_out, void* map128) {
  if (!out || !map128 || rows < 1 || N < 1 || ld_out < N) return IFLB200_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(out) & 15) || (ld_out * 4) % 16) return IFLB200_ERR_ALIGN;
  CUtensorMap tm;
  const int st = make_out_map(&tm, out, rows, N, ld_out, 4);
  if (st != IFLB200_OK) return st;
  memcpy(map128, &tm, sizeof(tm));
  return IFLB200_OK;
}

extern "C" int iflb200_gemm_fp8_rowblocks(const void* a, int64_t ld_a, const void* w, int64_t ld_w, int groups,
                                          int group_rows, int N, int K, const void* d_out_maps, void* stream) {
  return run_gemm_rowblocks(a, ld_a, w, ld_w, groups, group_rows, N, K, d_out_maps, stream);
}

extern "C" int iflb200_fp8_linear_gated(const void* a, int64_t ld_a, const void* w, int64_t ld_w, int M, int F,
                                        int K, const float* row_scale, const float* col_scale, int act, float* h,
                                        int64_t ld_h, uint32_t* amax, void* stream) {
  return run_gemm_gated(a, ld_a, w, ld_w, M, F, K, row_scale, col_scale, act, h, ld_h, amax, stream);
}

extern "C" int iflb200_abi_version(void) { return IFLB200_ABI_VERSION; }

extern "C" const char* iflb200_status_string(int status) {
  switch (status) {
    case IFLB200_OK: return "ok";
    case IFLB200_ERR_ARG: return "invalid argument (null pointer, negative size or stride shorter than the row)";
    case IFLB200_ERR_SHAPE: return "unsupported shape (K and N must be multiples of 16; width above the kernel's maximum)";
    case IFLB200_ERR_ALIGN: return "pointer or row stride breaks the 16-byte alignment rule";
    case IFLB200_ERR_DTYPE: return "unsupported element type";
    case IFLB200_ERR_DRIVER: return "cuTensorMapEncodeTiled unavailable or rejected the layout";
    case IFLB200_ERR_DEVICE: return "current device is not a compute capability 10.x GPU";
    case IFLB200_ERR_WORKSPACE: return "workspace missing or too small";
    case IFLB200_ERR_TOO_LARGE: return "input exceeds the fixed capacity of this no-allocation entry point";
    default: return status > 0 ? cudaGetErrorString((cudaError_t)status) : "unknown status";
  }
}

#ifdef IFLB200_TRACE
extern "C" __attribute__((visibility("default"))) int iflb200_exp_gemm_trace(unsigned long long* out64x10, unsigned int* launches) {
  cudaError_t e = cudaMemcpyFromSymbol(out64x10, g_gemm_trace, sizeof(unsigned long long) * 64 * 16);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemcpyFromSymbol(launches, g_gemm_trace_launch, sizeof(unsigned int));
}
#endif
