// Context-parallel hand-off kernels: a rank writes a payload (its slice's final SSM state and total decay, the conv
// halo, or gradient rows on the way back) directly into a slot of other ranks' symmetric buffers with peer stores
// and then release-writes a per-sender flag there; receivers acquire-wait (bounded) on the flags of the ranks they
// depend on.  This is the data plane of parallel/context_parallel.py.  The reference leaves the hand-off to the
// external mamba_ssm Mamba2CP module (fms_acceleration_mcp/utils/utils.py:64-80).
#include "common.cuh"

namespace fmsb {

struct CpPeers {
  void* p[16];
};

__device__ __forceinline__ void cp_st_release(uint32_t* addr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t cp_ld_acquire(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// direction +1: targets are the ranks after `rank`; -1: the ranks before.  per_target_rows = 0: the same payload goes to
// every target; 1: payload is [world, nbytes] and row t goes to target t.  Slot `rank` of the target's buffer is written.
// One CTA per target; the last thread to finish publishes the flag.
__global__ void cp_push_kernel(const uint8_t* __restrict__ payload, long long nbytes, CpPeers slots, CpPeers signals,
                               long long slot_bytes, int rank, int world, int direction, int per_target_rows,
                               uint32_t epoch) {
  const int target = blockIdx.x;
  const bool serve = direction > 0 ? target > rank : target < rank;
  if (!serve) return;
  const uint8_t* src = payload + (per_target_rows ? (long long)target * nbytes : 0);
  uint8_t* dst = reinterpret_cast<uint8_t*>(slots.p[target]) + (long long)rank * slot_bytes;
  const long long n16 = nbytes / 16;
  for (long long i = threadIdx.x; i < n16; i += blockDim.x)
    reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
  for (long long i = n16 * 16 + threadIdx.x; i < nbytes; i += blockDim.x) dst[i] = src[i];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) cp_st_release(reinterpret_cast<uint32_t*>(signals.p[target]) + rank, epoch);
}

// Wait until every rank this one depends on (direction +1: all earlier ranks sent to me; -1: all later ranks) has
// published `epoch` in my flag array.
__global__ void cp_wait_kernel(const uint32_t* __restrict__ my_signals, int rank, int world, int direction, uint32_t epoch,
                               int* status) {
  const int s = threadIdx.x;
  if (s >= world) return;
  const bool dep = direction > 0 ? s < rank : s > rank;
  if (!dep) return;
  const long long t0 = clock64();
  while ((int32_t)(cp_ld_acquire(my_signals + s) - epoch) < 0) {
    if (clock64() - t0 > peer_wait_budget(status)) {
      report_status(status, kTimeoutPeerFlag);
      return;
    }
    if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) return;
  }
}

}  // namespace fmsb

using namespace fmsb;

extern "C" int fmsb_cp_push(const void* payload, long long nbytes, void* const* slot_ptrs, void* const* signal_ptrs,
                            long long slot_bytes, int rank, int world, int direction, int per_target_rows,
                            unsigned epoch, int* status, cudaStream_t stream) {
  if (world > 16 || nbytes > slot_bytes) return -2;
  (void)status;
  CpPeers s{}, g{};
  for (int i = 0; i < world; ++i) {
    s.p[i] = slot_ptrs[i];
    g.p[i] = signal_ptrs[i];
  }
  cp_push_kernel<<<world, 512, 0, stream>>>((const uint8_t*)payload, nbytes, s, g, slot_bytes, rank, world, direction,
                                            per_target_rows, epoch);
  return (int)cudaGetLastError();
}

extern "C" int fmsb_cp_wait(const void* my_signals, int rank, int world, int direction, int unused0, int unused1,
                            unsigned epoch, int* status, cudaStream_t stream) {
  (void)unused0;
  (void)unused1;
  cp_wait_kernel<<<1, 32, 0, stream>>>((const uint32_t*)my_signals, rank, world, direction, epoch, status);
  return (int)cudaGetLastError();
}
