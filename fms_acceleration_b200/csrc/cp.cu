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
// span: how far the payload travels (1: to the neighbour only, as the conv halo and the shifted label do; world: to
// every rank on that side).
__global__ void cp_push_kernel(const uint8_t* __restrict__ payload, long long nbytes, CpPeers slots, CpPeers signals,
                               long long slot_bytes, int rank, int world, int direction, int per_target_rows,
                               uint32_t epoch, int span) {
  const int target = blockIdx.x;
  const bool serve = direction > 0 ? (target > rank && target <= rank + span) : (target < rank && target >= rank - span);
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
                               int* status, int span) {
  const int s = threadIdx.x;
  if (s >= world) return;
  const bool dep = direction > 0 ? (s < rank && s >= rank - span) : (s > rank && s <= rank + span);
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


// ----------------------------------------------------------------------------------------
// State hand-off of the chunked SSD scan, issued by the scan's own state kernel.
//
// Slot layout (fp32): [F: nh * PN | logP: nh], one slot per sender in every receiver's buffer.
//   ssd_state_fwd_push   the inter-chunk recurrence of this rank's slice from a ZERO entering state; the final state
//                        F and the slice's total log-decay go straight into the slot `rank` of every LATER rank
//                        (peer stores from the thread that computed the element); the CTA that finishes last
//                        release-flags the receivers.  Also leaves the zero-start entering states of every chunk
//                        (16-bit), which the backward needs for the gradient of the decays along this path.
//   cp_prefix_fwd        receiver: bounded wait on the flags of the earlier ranks, then
//                        H_in = sum_{j<r} (prod_{j<i<r} P_i) F_j, left to right, per element.
//   cp_prefix_bwd_push   from dH_in: dF_j and dlogP_j for every earlier rank j, stored into slot `rank` of rank j's
//                        backward buffer; last CTA flags.
//   cp_sum_bwd           bounded wait on the later ranks, then the sum of what they sent.
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ bool cp_last_cta(unsigned* counter) {
  __shared__ bool last;
  __threadfence_system();  // this thread's peer stores are out before the CTA is counted
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned done = atomicAdd(counter, 1u) + 1u;
    last = done == gridDim.x;
    if (last) atomicExch(counter, 0u);  // ready for the next launch
  }
  __syncthreads();
  return last;
}

template <typename T>
__global__ void __launch_bounds__(256) ssd_state_fwd_push_kernel(
    const float* __restrict__ S, const float* __restrict__ Ltot, T* __restrict__ hprev0, int nc, int nh, int PN,
    CpPeers slots, long long slot_elems, CpPeers signals, int rank, int world, uint32_t epoch, unsigned* counter) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long total = (long long)nh * PN;
  if (idx < total) {
    const int h = (int)(idx / PN);
    float st = 0.f;
    for (int c = 0; c < nc; ++c) {
      hprev0[(long long)c * total + idx] = (T)st;
      st = __expf(Ltot[c * nh + h]) * st + S[(long long)c * total + idx];
    }
    for (int t = rank + 1; t < world; ++t)
      reinterpret_cast<float*>(slots.p[t])[(long long)rank * slot_elems + idx] = st;
  }
  if (idx < nh) {  // the slice's total log-decay per head
    float lp = 0.f;
    for (int c = 0; c < nc; ++c) lp += Ltot[c * nh + idx];
    for (int t = rank + 1; t < world; ++t)
      reinterpret_cast<float*>(slots.p[t])[(long long)rank * slot_elems + total + idx] = lp;
  }
  if (cp_last_cta(counter) && threadIdx.x > rank && (int)threadIdx.x < world)
    cp_st_release(reinterpret_cast<uint32_t*>(signals.p[threadIdx.x]) + rank, epoch);
}

// bounded wait of one CTA on the flags of ranks [lo, hi); returns false when it gave up
__device__ __forceinline__ bool cp_wait_range(const uint32_t* my_signals, int lo, int hi, uint32_t epoch, int* status) {
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  const int s = lo + (int)threadIdx.x;
  if (s < hi) {
    const long long t0 = clock64();
    while ((int32_t)(cp_ld_acquire(my_signals + s) - epoch) < 0) {
      if (clock64() - t0 > peer_wait_budget(status)) {
        report_status(status, kTimeoutPeerFlag);
        ok = 0;
        break;
      }
      if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) {
        ok = 0;
        break;
      }
    }
  }
  __syncthreads();
  return ok != 0;
}

__global__ void __launch_bounds__(256) cp_prefix_fwd_kernel(const float* __restrict__ my_slots, long long slot_elems,
                                                            const uint32_t* __restrict__ my_signals, int rank,
                                                            uint32_t epoch, int nh, int PN, float* __restrict__ h_in,
                                                            int* status) {
  if (!cp_wait_range(my_signals, 0, rank, epoch, status)) return;
  const long long total = (long long)nh * PN;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int h = (int)(idx / PN);
    float acc = 0.f;
    for (int j = 0; j < rank; ++j) {
      const float* slot = my_slots + (long long)j * slot_elems;
      acc = __expf(slot[total + h]) * acc + slot[idx];
    }
    h_in[idx] = acc;
  }
}

// One CTA per head.  dh [nh, PN]; my_slots: the forward slots of this rank (F_j, logP_j of the earlier ranks).
__global__ void __launch_bounds__(256) cp_prefix_bwd_push_kernel(
    const float* __restrict__ dh, const float* __restrict__ my_slots, long long slot_elems, CpPeers bwd_slots,
    CpPeers signals, int rank, int world, uint32_t epoch, int nh, int PN, unsigned* counter) {
  constexpr int kMax = 16;
  __shared__ float decay[kMax];
  __shared__ float red[kMax][8];
  const int h = blockIdx.x;
  const long long total = (long long)nh * PN;
  if ((int)threadIdx.x < rank) decay[threadIdx.x] = __expf(my_slots[(long long)threadIdx.x * slot_elems + total + h]);
  __syncthreads();
  float part[kMax];
#pragma unroll
  for (int j = 0; j < kMax; ++j) part[j] = 0.f;
  for (int e = threadIdx.x; e < PN; e += blockDim.x) {
    const long long idx = (long long)h * PN + e;
    // prefixes: pre[j] = state after absorbing the ranks below j
    float pre[kMax];
    pre[0] = 0.f;
#pragma unroll
    for (int j = 0; j < kMax - 1; ++j)
      if (j < rank) pre[j + 1] = decay[j] * pre[j] + my_slots[(long long)j * slot_elems + idx];
    float g = dh[idx];
#pragma unroll
    for (int j = kMax - 1; j >= 0; --j) {
      if (j < rank) {
        reinterpret_cast<float*>(bwd_slots.p[j])[(long long)rank * slot_elems + idx] = g;  // dF_j
        part[j] += g * pre[j];
        g *= decay[j];
      }
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int j = 0; j < kMax; ++j) {
    float v = warp_sum(part[j]);
    if (lane == 0) red[j][warp] = v;
  }
  __syncthreads();
  if ((int)threadIdx.x < rank) {
    float v = 0.f;
    for (int w = 0; w < 8; ++w) v += red[threadIdx.x][w];
    // dlogP_j = exp(logP_j) * <g_j, prefix_j>
    reinterpret_cast<float*>(bwd_slots.p[threadIdx.x])[(long long)rank * slot_elems + total + h] = v * decay[threadIdx.x];
  }
  if (cp_last_cta(counter) && (int)threadIdx.x < rank)
    cp_st_release(reinterpret_cast<uint32_t*>(signals.p[threadIdx.x]) + rank, epoch);
}

__global__ void __launch_bounds__(256) cp_sum_bwd_kernel(const float* __restrict__ my_bwd_slots, long long slot_elems,
                                                         const uint32_t* __restrict__ my_signals, int rank, int world,
                                                         uint32_t epoch, int nh, int PN, float* __restrict__ dF,
                                                         float* __restrict__ dlogP, int* status) {
  if (!cp_wait_range(my_signals, rank + 1, world, epoch, status)) return;
  const long long total = (long long)nh * PN + nh;  // F elements followed by the per-head decays
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int s = rank + 1; s < world; ++s) acc += my_bwd_slots[(long long)s * slot_elems + idx];
    if (idx < (long long)nh * PN) dF[idx] = acc;
    else dlogP[idx - (long long)nh * PN] = acc;
  }
}

}  // namespace fmsb

using namespace fmsb;

extern "C" int fmsb_cp_push(const void* payload, long long nbytes, void* const* slot_ptrs, void* const* signal_ptrs,
                            long long slot_bytes, int rank, int world, int direction, int per_target_rows,
                            unsigned epoch, int span, int* status, cudaStream_t stream) {
  if (world > 16 || nbytes > slot_bytes) return -2;
  (void)status;
  CpPeers s{}, g{};
  for (int i = 0; i < world; ++i) {
    s.p[i] = slot_ptrs[i];
    g.p[i] = signal_ptrs[i];
  }
  cp_push_kernel<<<world, 512, 0, stream>>>((const uint8_t*)payload, nbytes, s, g, slot_bytes, rank, world, direction,
                                            per_target_rows, epoch, span > 0 ? span : world);
  return (int)cudaGetLastError();
}

extern "C" int fmsb_cp_wait(const void* my_signals, int rank, int world, int direction, int span, int unused1,
                            unsigned epoch, int* status, cudaStream_t stream) {
  (void)unused1;
  cp_wait_kernel<<<1, 32, 0, stream>>>((const uint32_t*)my_signals, rank, world, direction, epoch, status,
                                       span > 0 ? span : world);
  return (int)cudaGetLastError();
}

static CpPeers cp_peers(void* const* arr, int world) {
  CpPeers p{};
  for (int i = 0; i < world && i < 16; ++i) p.p[i] = arr[i];
  return p;
}

// Zero-start inter-chunk recurrence of this rank's slice with the hand-off of (final state, total log-decay) to every
// later rank fused in.  S [nc, nh, PN] fp32, Ltot [nc, nh]; hprev0 [nc, nh, PN] 16-bit out; counter: one zeroed word.
extern "C" int fmsb_cp_state_push(const float* S, const float* Ltot, void* hprev0, int nc, int nh, int PN,
                                  void* const* slot_ptrs, long long slot_elems, void* const* signal_ptrs, int rank,
                                  int world, unsigned epoch, unsigned* counter, int dtype, cudaStream_t stream) {
  const long long total = (long long)nh * PN;
  if (world > 16 || total <= 0 || slot_elems < total + nh) return -2;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  CpPeers s = cp_peers(slot_ptrs, world), g = cp_peers(signal_ptrs, world);
  if (dtype == 1)
    ssd_state_fwd_push_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(S, Ltot, (__nv_bfloat16*)hprev0, nc, nh, PN, s,
                                                                        slot_elems, g, rank, world, epoch, counter);
  else if (dtype == 0)
    ssd_state_fwd_push_kernel<__half><<<blocks, 256, 0, stream>>>(S, Ltot, (__half*)hprev0, nc, nh, PN, s, slot_elems, g,
                                                                 rank, world, epoch, counter);
  else
    return -2;
  return (int)cudaGetLastError();
}

extern "C" int fmsb_cp_prefix_fwd(const float* my_slots, long long slot_elems, const void* my_signals, int rank,
                                  unsigned epoch, int nh, int PN, float* h_in, int* status, cudaStream_t stream) {
  if (rank > 16) return -2;
  cp_prefix_fwd_kernel<<<148, 256, 0, stream>>>(my_slots, slot_elems, (const uint32_t*)my_signals, rank, epoch, nh, PN,
                                                h_in, status);
  return (int)cudaGetLastError();
}

extern "C" int fmsb_cp_prefix_bwd(const float* dh, const float* my_slots, long long slot_elems, void* const* bwd_slot_ptrs,
                                  void* const* signal_ptrs, int rank, int world, unsigned epoch, int nh, int PN,
                                  unsigned* counter, cudaStream_t stream) {
  if (world > 16 || nh <= 0) return -2;
  cp_prefix_bwd_push_kernel<<<nh, 256, 0, stream>>>(dh, my_slots, slot_elems, cp_peers(bwd_slot_ptrs, world),
                                                    cp_peers(signal_ptrs, world), rank, world, epoch, nh, PN, counter);
  return (int)cudaGetLastError();
}

extern "C" int fmsb_cp_sum_bwd(const float* my_bwd_slots, long long slot_elems, const void* my_signals, int rank,
                               int world, unsigned epoch, int nh, int PN, float* dF, float* dlogP, int* status,
                               cudaStream_t stream) {
  if (world > 16) return -2;
  cp_sum_bwd_kernel<<<148, 256, 0, stream>>>(my_bwd_slots, slot_elems, (const uint32_t*)my_signals, rank, world, epoch, nh,
                                             PN, dF, dlogP, status);
  return (int)cudaGetLastError();
}
