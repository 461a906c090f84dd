// Barrier between the GPUs of a tensor-parallel group over peer memory (NVLink), for the exchange
// steps of the row-split FP8 linears: every rank writes its partial sums / codes / row maxima
// straight into its peers' buffers (the GEMM's TMA stores, the row kernels' stores through
// peer-mapped pointers) and then meets the others here before anyone reads.  The reference has
// nothing distributed; this replaces the latency of a library collective (15-20 us for an 18 KB
// all-reduce) by one single-CTA kernel, which can also reduce the row maxima of all ranks after it
// has waited.
//
// Each rank owns an array of `p` flag words in memory its peers can write.  Arrival number e of
// rank r is the store of e into word r of every peer's array (release, system scope: everything
// kernels earlier in this rank's stream wrote, to local or peer memory, is complete by stream
// order); the rank then waits until every word of its own array has reached e.  The arrival number
// lives in device memory and is advanced by the kernel itself, so a captured graph can be replayed.
// The wait is bounded: when the budget runs out the kernel records which peer was missing in
// `status` and returns, the context stays usable and the host reads the word after the run.
#include <cuda_runtime.h>

#include "../../include/iflb200.h"
#include "ptx.cuh"

namespace iflb200 {

constexpr uint64_t kPeerWaitBudgetNs = 2000000000ull;
__device__ uint64_t g_peer_wait_budget_ns = kPeerWaitBudgetNs;

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// One CTA.  Thread r < p publishes arrival e to peer r and waits for peer r's arrival e; then the
// CTA reduces `max_in` [p][max_n] (slot r written by rank r before its arrival, the local slot by an
// earlier kernel of this stream) to max_out[i] = max_r max_in[r][i] (optional).
__global__ void __launch_bounds__(1024) peer_exchange_kernel(uint32_t* const* __restrict__ peer_flags,
                                                            uint32_t* __restrict__ my_flags, uint32_t* __restrict__ arrival,
                                                            int rank, int p, uint32_t* __restrict__ status,
                                                            const float* __restrict__ max_in, float* __restrict__ max_out,
                                                            int max_n) {
  const uint32_t e = *arrival + 1;
  __syncthreads();  // every thread has read *arrival
  const int r = threadIdx.x;
  if (r < p && r != rank) {
    __threadfence_system();
    st_release_sys(peer_flags[r] + rank, e);
    uint64_t t0 = 0;
    uint32_t spins = 0;
    // a wait that ran out earlier stays on record until the host clears it: later barriers of the
    // same run signal and go on instead of spending the budget again
    const bool gave_up_before = *reinterpret_cast<volatile uint32_t*>(status) != 0;
    // arrival numbers only grow; the signed difference keeps the comparison right across wrap-around
    while (!gave_up_before && (int32_t)(ld_acquire_sys(my_flags + r) - e) < 0) {
      if (++spins > 256) {
        if (t0 == 0) t0 = globaltimer_ns();
        __nanosleep(64);
        if (globaltimer_ns() - t0 > g_peer_wait_budget_ns) {
          atomicCAS(status, 0u, 0x50000000u | ((uint32_t)r << 16) | (e & 0xFFFFu));  // peer r never arrived
          break;
        }
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) *arrival = e;
  for (int i = threadIdx.x; i < max_n; i += blockDim.x) {
    float m = __ldcg(max_in + i);
    for (int q = 1; q < p; ++q) m = fmaxf(m, __ldcg(max_in + (int64_t)q * max_n + i));
    max_out[i] = m;
  }
}

int set_peer_wait_budget_ns(uint64_t ns) {
  const uint64_t v = ns ? ns : kPeerWaitBudgetNs;
  return (int)cudaMemcpyToSymbol(g_peer_wait_budget_ns, &v, sizeof(v));
}

}  // namespace iflb200

using namespace iflb200;

extern "C" int iflb200_peer_exchange(const void* peer_flag_ptrs, void* my_flags, void* arrival, int rank, int p,
                                     void* status, const float* max_in, float* max_out, int max_n, void* stream) {
  if (!peer_flag_ptrs || !my_flags || !arrival || !status) return IFLB200_ERR_ARG;
  if (p < 1 || p > 32 || rank < 0 || rank >= p) return IFLB200_ERR_ARG;
  if (max_n < 0 || (max_n > 0 && (!max_in || !max_out))) return IFLB200_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(peer_flag_ptrs) & 7) || (reinterpret_cast<uintptr_t>(my_flags) & 3))
    return IFLB200_ERR_ALIGN;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  peer_exchange_kernel<<<1, max_n > 0 ? 1024 : 32, 0, s>>>(
      reinterpret_cast<uint32_t* const*>(peer_flag_ptrs), reinterpret_cast<uint32_t*>(my_flags),
      reinterpret_cast<uint32_t*>(arrival), rank, p, reinterpret_cast<uint32_t*>(status), max_in, max_out, max_n);
  return (int)cudaGetLastError();
}

extern "C" int iflb200_peer_barrier(const void* peer_flag_ptrs, void* my_flags, void* arrival, int rank, int p,
                                    void* status, void* stream) {
  return iflb200_peer_exchange(peer_flag_ptrs, my_flags, arrival, rank, p, status, nullptr, nullptr, 0, stream);
}
