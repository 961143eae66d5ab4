// Peer-memory communication kernels for one NVSwitch-connected node (up to 16 ranks).
//
// Every rank owns buffers inside a symmetric allocation and knows the device address of each
// peer's copy (`ptrs[r]`); kernels move data with plain peer loads/stores over NVLink and
// synchronise through per-rank signal words that peers write with release semantics.  There is
// no TMA multicast and no NCCL in here.  Signals carry a monotonically increasing epoch, so
// nothing has to be zeroed between steps; every wait is bounded and reports through the status
// word (common.cuh) instead of hanging.
//
// What these replace in the reference design:
//   * accelerate FSDP's per-layer parameter all-gather (NCCL)           -> allgather_pull
//   * fms_acceleration_foak/utils.py:39-43, one NCCL all_reduce per LoRA tensor in a gradient
//     hook (256 collectives per step for a 7B model)                    -> one allreduce over a
//     flat bucket: reduce-scatter (pull + fp32 sum + scale + cast) then all-gather
//   * FSDP's gradient reduce-scatter followed by a separate cast/scale  -> reduce_scatter_pull
#include "common.cuh"

namespace fmsb {

constexpr int kMaxRanks = 16;

struct PeerPtrs {
  void* p[kMaxRanks];
};

// ----------------------------------------------------------------------------------------
// signalling
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ void st_release_sys(uint32_t* addr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// Bounded wait until *addr >= epoch (signed distance, so epochs may wrap).
__device__ __forceinline__ bool wait_signal_ge(const uint32_t* addr, uint32_t epoch, int* status) {
  const long long t0 = clock64();
  while (true) {
    for (int i = 0; i < 64; ++i) {
      if ((int32_t)(ld_acquire_sys(addr) - epoch) >= 0) return true;
    }
    if (clock64() - t0 > peer_wait_budget(status)) {
      report_status(status, kTimeoutPeerFlag);
      return false;
    }
    if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) return false;
  }
}

// Tell every rank "rank `rank` reached `epoch` on channel `chan`", then wait until all ranks said so.
// signals[r] points at rank r's signal array laid out [channel][world].
__global__ void barrier_kernel(PeerPtrs signals, int rank, int world, int chan, uint32_t epoch, int* status) {
  const int t = threadIdx.x;
  if (t < world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(signals.p[t]) + chan * world + rank, epoch);
  }
  if (t < world) {
    wait_signal_ge(reinterpret_cast<const uint32_t*>(signals.p[rank]) + chan * world + t, epoch, status);
  }
}

// ----------------------------------------------------------------------------------------
// all-gather: every rank pulls the shards of all peers into its own full buffer
//   shard r lives at src.p[r] (shard_bytes each), destination dst[r * shard_bytes ...]
// ----------------------------------------------------------------------------------------
__global__ void allgather_pull_kernel(PeerPtrs src, uint8_t* __restrict__ dst, long long shard_bytes, int rank,
                                      int world) {
  // Each thread keeps UNROLL independent 16-byte peer loads in flight: over NVLink the latency is microseconds, so
  // the bandwidth of a pull is (bytes in flight) / latency.  Work is split per source shard, starting with the
  // successor of this rank so that the peers are not all hit in the same order.
  constexpr int UNROLL = 8;
  const long long shard16 = shard_bytes / 16;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  for (int s = 0; s < world; ++s) {
    const int owner = (rank + 1 + s) % world;
    const uint4* __restrict__ from = reinterpret_cast<const uint4*>(src.p[owner]);
    uint4* __restrict__ to = reinterpret_cast<uint4*>(dst) + (long long)owner * shard16;
    if (from == to) continue;  // gathering in place: this rank's own shard is already where it belongs
    for (long long base = tid; base < shard16; base += stride * UNROLL) {
      uint4 v[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long i = base + u * stride;
        if (i < shard16) v[u] = from[i];
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const long long i = base + u * stride;
        if (i < shard16) to[i] = v[u];
      }
    }
  }
}

// ----------------------------------------------------------------------------------------
// reduce-scatter (pull): rank r owns elements [r*n_own, (r+1)*n_own) of a flat gradient bucket.
// It reads that slice from every rank's bucket, sums in fp32, multiplies by `scale` and writes
//   out (own slice, dtype of the bucket or fp32).  Peers must have finished writing their buckets
//   (barrier before) and must not overwrite them until everybody has read (barrier after).
// ----------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void rs_accumulate(const uint4& v, float* acc) {
  constexpr int V = 16 / sizeof(T);
  const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
  for (int k = 0; k < V; ++k) {
    if (sizeof(T) == 4) acc[k] += *reinterpret_cast<const float*>(e + k);
    else if (std::is_same<T, __nv_bfloat16>::value) acc[k] += __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(e + k));
    else acc[k] += __half2float(*reinterpret_cast<const __half*>(e + k));
  }
}

// Each thread works on U vectors at a time, so U independent 16-byte peer loads are in flight per thread.  The pull
// rate over NVLink is (bytes in flight) / latency and the loaded latency is several microseconds: one load in flight
// per thread gave 60 GB/s per direction, four gave 190 GB/s, and the all-gather above reaches 650 GB/s with 6 MB in
// flight per GPU.  Results leave as 16-byte stores.
template <typename T, typename OutT>
__global__ void __launch_bounds__(512)
reduce_scatter_pull_kernel(PeerPtrs buckets, OutT* __restrict__ out, long long n_own, int rank, int world,
                           float scale) {
  constexpr int V = 16 / sizeof(T);
  constexpr int U = 8;
  const long long nvec = n_own / V;
  const long long base = (long long)rank * n_own;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < nvec; i0 += stride * U) {
    float acc[U][V];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int k = 0; k < V; ++k) acc[u][k] = 0.f;
#pragma unroll 1
    for (int rr = 0; rr < world; ++rr) {
      const int r = (rank + rr) % world;
      const uint4* __restrict__ src = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(buckets.p[r]) + base);
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        v[u] = i < nvec ? src[i] : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) rs_accumulate<T>(v[u], acc[u]);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i >= nvec) continue;
      OutT* o = out + i * V;
      if (sizeof(OutT) == 4) {
#pragma unroll
        for (int k = 0; k < V; k += 4)
          *reinterpret_cast<float4*>(reinterpret_cast<float*>(o) + k) =
              make_float4(acc[u][k] * scale, acc[u][k + 1] * scale, acc[u][k + 2] * scale, acc[u][k + 3] * scale);
      } else {
        uint4 w;
        uint32_t* ww = reinterpret_cast<uint32_t*>(&w);
#pragma unroll
        for (int k = 0; k < V; k += 2)
          ww[k / 2] = std::is_same<OutT, __nv_bfloat16>::value ? pack_bf16x2(acc[u][k] * scale, acc[u][k + 1] * scale)
                                                               : pack_f16x2(acc[u][k] * scale, acc[u][k + 1] * scale);
        *reinterpret_cast<uint4*>(o) = w;
      }
    }
  }
}

// One-kernel all-reduce of a flat bucket (two-shot over peer memory):
//   phase 1  barrier: every rank's bucket is complete
//   phase 2  each rank reduces its own slice (pull from all peers, fp32 sum, scale) and writes the
//            result back into EVERY rank's bucket slice (push), so the bucket ends up averaged everywhere
//   phase 3  barrier: all slices have landed
// Runs with gridDim.x CTAs; CTA 0 handles the cross-rank barriers and the grid is held together with
// a local atomic counter (all CTAs are co-resident: the launcher caps the grid at the SM count).
template <typename T>
__global__ void allreduce_bucket_kernel(PeerPtrs buckets, PeerPtrs signals, long long n, int rank, int world,
                                        float scale, int chan, uint32_t epoch, unsigned* grid_sync, int* status) {
  constexpr int V = 16 / sizeof(T);
  __shared__ int ok_sh;
  // ---- phase 1: cross-rank barrier by CTA 0, released to the other CTAs through grid_sync[0]
  if (blockIdx.x == 0) {
    if (threadIdx.x == 0) ok_sh = 1;
    __syncthreads();
    if (threadIdx.x < world) {
      __threadfence_system();
      st_release_sys(reinterpret_cast<uint32_t*>(signals.p[threadIdx.x]) + chan * world + rank, epoch);
      if (!wait_signal_ge(reinterpret_cast<const uint32_t*>(signals.p[rank]) + chan * world + threadIdx.x, epoch, status))
        ok_sh = 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      atomicExch(grid_sync, ok_sh ? epoch : 0xffffffffu);
    }
  }
  if (threadIdx.x == 0) {
    const long long t0 = clock64();
    unsigned v;
    while ((v = atomicAdd(grid_sync, 0u)) != epoch && v != 0xffffffffu) {
      if (clock64() - t0 > 2 * peer_wait_budget(status)) { report_status(status, kTimeoutPeerFlag); break; }
    }
    ok_sh = (v == epoch);
  }
  __syncthreads();
  if (!ok_sh) return;

  // ---- phase 2: reduce own slice, push the result to all ranks.  A thread keeps U vectors of two peers in
  // flight (2 * U independent 16-byte loads), so that a few CTAs already cover the NVLink latency.
  constexpr int U = 4;
  const long long n_own = n / world;  // n is padded to a multiple of world * V by the caller
  const long long nvec = n_own / V;
  const long long base = (long long)rank * n_own;
  const long long stride = (long long)gridDim.x * blockDim.x;
  auto add_vec = [](float (&acc)[V], const uint4& v) {
    const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
    for (int k = 0; k < V; ++k) {
      if (sizeof(T) == 4) acc[k] += *reinterpret_cast<const float*>(e + k);
      else if (std::is_same<T, __nv_bfloat16>::value) acc[k] += __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(e + k));
      else acc[k] += __half2float(*reinterpret_cast<const __half*>(e + k));
    }
  };
  for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < nvec; i0 += stride * U) {
    float acc[U][V];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int k = 0; k < V; ++k) acc[u][k] = 0.f;
    for (int rr = 0; rr < world; rr += 2) {
      const bool two = rr + 1 < world;
      const uint4* pa = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(buckets.p[(rank + rr) % world]) + base);
      const uint4* pb = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(buckets.p[(rank + rr + (two ? 1 : 0)) % world]) + base);
      uint4 va[U], vb[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        va[u] = vb[u] = make_uint4(0u, 0u, 0u, 0u);
        if (i < nvec) {
          va[u] = pa[i];
          if (two) vb[u] = pb[i];
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        add_vec(acc[u], va[u]);
        if (two) add_vec(acc[u], vb[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i >= nvec) continue;
      uint4 outv;
      T* oe = reinterpret_cast<T*>(&outv);
#pragma unroll
      for (int k = 0; k < V; ++k) {
        const float v = acc[u][k] * scale;
        if (sizeof(T) == 4) *reinterpret_cast<float*>(oe + k) = v;
        else if (std::is_same<T, __nv_bfloat16>::value) *reinterpret_cast<__nv_bfloat16*>(oe + k) = __float2bfloat16_rn(v);
        else *reinterpret_cast<__half*>(oe + k) = __float2half_rn(v);
      }
      for (int rr = 0; rr < world; ++rr) {
        const int r = (rank + rr) % world;
        *(reinterpret_cast<uint4*>(reinterpret_cast<T*>(buckets.p[r]) + base) + i) = outv;
      }
    }
  }
  // ---- phase 3: everyone's pushes are visible before anybody reads its bucket
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned arrived = atomicAdd(grid_sync + 1, 1u) + 1;
    if (arrived == gridDim.x) {
      atomicExch(grid_sync + 1, 0u);
      __threadfence_system();
      for (int t = 0; t < world; ++t)
        st_release_sys(reinterpret_cast<uint32_t*>(signals.p[t]) + (chan + 1) * world + rank, epoch);
      for (int t = 0; t < world; ++t)
        wait_signal_ge(reinterpret_cast<const uint32_t*>(signals.p[rank]) + (chan + 1) * world + t, epoch, status);
      __threadfence();
      atomicExch(grid_sync + 2, epoch);
    }
    const long long t0 = clock64();
    while (atomicAdd(grid_sync + 2, 0u) != epoch) {
      if (clock64() - t0 > 2 * peer_wait_budget(status)) { report_status(status, kTimeoutPeerFlag); break; }
      if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) break;
    }
  }
  __syncthreads();
}

// ----------------------------------------------------------------------------------------
// All-reduce through the NVSwitch multicast object (NVLS): every rank's bucket is bound to one multicast address range.
// A rank reduces ITS slice with multimem.ld_reduce (one instruction returns the sum over all ranks, added inside the
// switch), scales it, and multimem.st writes the result into every rank's bucket at once: per element one load and one
// store cross this GPU's links instead of world - 1 peer loads and world - 1 peer stores.  Barriers before and after
// as in allreduce_bucket_kernel.  `mc` is the multicast address of the bucket (same layout as the local one).
// ----------------------------------------------------------------------------------------
__device__ __forceinline__ void multimem_ld_reduce_bf16x8(const void* addr, float (&f)[8]) {
  uint32_t r0, r1, r2, r3;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "l"(addr)
               : "memory");
  const uint32_t r[4] = {r0, r1, r2, r3};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&r[i]);
    const float2 p = __bfloat1622float2(v);
    f[2 * i] = p.x;
    f[2 * i + 1] = p.y;
  }
}
__device__ __forceinline__ void multimem_st_bf16x8(void* addr, const float (&f)[8]) {
  const uint32_t r0 = pack_bf16x2(f[0], f[1]), r1 = pack_bf16x2(f[2], f[3]), r2 = pack_bf16x2(f[4], f[5]),
                 r3 = pack_bf16x2(f[6], f[7]);
  asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(addr), "r"(r0), "r"(r1), "r"(r2),
               "r"(r3)
               : "memory");
}
__device__ __forceinline__ void multimem_ld_reduce_f32x4(const void* addr, float (&f)[4]) {
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(f[0]), "=f"(f[1]), "=f"(f[2]), "=f"(f[3])
               : "l"(addr)
               : "memory");
}
__device__ __forceinline__ void multimem_st_f32x4(void* addr, const float (&f)[4]) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(f[0]), "f"(f[1]), "f"(f[2]),
               "f"(f[3])
               : "memory");
}

template <typename T>
__global__ void allreduce_multimem_kernel(T* mc, PeerPtrs signals, long long n, int rank, int world, float scale, int chan,
                                          uint32_t epoch, unsigned* grid_sync, int* status) {
  constexpr int V = 16 / sizeof(T);
  __shared__ int ok_sh;
  if (blockIdx.x == 0) {
    if (threadIdx.x == 0) ok_sh = 1;
    __syncthreads();
    if (threadIdx.x < world) {
      __threadfence_system();
      st_release_sys(reinterpret_cast<uint32_t*>(signals.p[threadIdx.x]) + chan * world + rank, epoch);
      if (!wait_signal_ge(reinterpret_cast<const uint32_t*>(signals.p[rank]) + chan * world + threadIdx.x, epoch, status))
        ok_sh = 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      atomicExch(grid_sync, ok_sh ? epoch : 0xffffffffu);
    }
  }
  if (threadIdx.x == 0) {
    const long long t0 = clock64();
    unsigned v;
    while ((v = atomicAdd(grid_sync, 0u)) != epoch && v != 0xffffffffu) {
      if (clock64() - t0 > 2 * peer_wait_budget(status)) { report_status(status, kTimeoutPeerFlag); break; }
    }
    ok_sh = (v == epoch);
  }
  __syncthreads();
  if (!ok_sh) return;
  const long long n_own = n / world;
  const long long nvec = n_own / V;
  T* base = mc + (long long)rank * n_own;
  // four reductions in flight per thread: a round trip through the switch takes microseconds
  constexpr int U = 4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < nvec; i0 += stride * U) {
    float f[U][V];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i < nvec) {
        if constexpr (sizeof(T) == 4) multimem_ld_reduce_f32x4(base + i * V, f[u]);
        else multimem_ld_reduce_bf16x8(base + i * V, f[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i >= nvec) continue;
#pragma unroll
      for (int k = 0; k < V; ++k) f[u][k] *= scale;
      if constexpr (sizeof(T) == 4) multimem_st_f32x4(base + i * V, f[u]);
      else multimem_st_bf16x8(base + i * V, f[u]);
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned arrived = atomicAdd(grid_sync + 1, 1u) + 1;
    if (arrived == gridDim.x) {
      atomicExch(grid_sync + 1, 0u);
      __threadfence_system();
      for (int t = 0; t < world; ++t)
        st_release_sys(reinterpret_cast<uint32_t*>(signals.p[t]) + (chan + 1) * world + rank, epoch);
      for (int t = 0; t < world; ++t)
        wait_signal_ge(reinterpret_cast<const uint32_t*>(signals.p[rank]) + (chan + 1) * world + t, epoch, status);
      __threadfence();
      atomicExch(grid_sync + 2, epoch);
    }
    const long long t0 = clock64();
    while (atomicAdd(grid_sync + 2, 0u) != epoch) {
      if (clock64() - t0 > 2 * peer_wait_budget(status)) { report_status(status, kTimeoutPeerFlag); break; }
      if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) break;
    }
  }
  __syncthreads();
}

// Bounded local wait used by tests of the time-out path: waits for a word that nobody sets.
__global__ void wait_flag_kernel(const uint32_t* flag, uint32_t epoch, int* status, long long budget_cycles) {
  const long long t0 = clock64();
  while ((int32_t)(ld_acquire_sys(flag) - epoch) < 0) {
    if (clock64() - t0 > budget_cycles) {
      report_status(status, kTimeoutPeerFlag);
      return;
    }
  }
}

}  // namespace fmsb

using namespace fmsb;

namespace fmsb_host {
int sm_count();
}

static PeerPtrs make_ptrs(void* const* arr, int world) {
  PeerPtrs p{};
  for (int i = 0; i < world && i < kMaxRanks; ++i) p.p[i] = arr[i];
  return p;
}

extern "C" int fmsb_comm_barrier(void* const* signal_ptrs, int rank, int world, int chan, unsigned epoch, int* status,
                                 cudaStream_t stream) {
  if (world > kMaxRanks) return -2;
  barrier_kernel<<<1, 32, 0, stream>>>(make_ptrs(signal_ptrs, world), rank, world, chan, epoch, status);
  return (int)cudaGetLastError();
}

// dst (local, world * shard_bytes) <- shards of all ranks.  shard_bytes must be a multiple of 16.
extern "C" int fmsb_comm_allgather(void* const* shard_ptrs, void* dst, long long shard_bytes, int rank, int world,
                                   int ctas, cudaStream_t stream) {
  if (world > kMaxRanks || shard_bytes % 16 != 0) return -2;
  if (shard_bytes == 0) return 0;
  if (ctas <= 0) ctas = 32;
  allgather_pull_kernel<<<ctas, 512, 0, stream>>>(make_ptrs(shard_ptrs, world), (uint8_t*)dst, shard_bytes, rank,
                                                  world);
  return (int)cudaGetLastError();
}

// out[n_own] = scale * sum_r bucket_r[rank*n_own : (rank+1)*n_own].  dtype of the buckets: 0 fp16, 1 bf16, 2 fp32;
// out_fp32 selects an fp32 result (master gradients) instead of the bucket dtype.
extern "C" int fmsb_comm_reduce_scatter(void* const* bucket_ptrs, void* out, long long n_own, int rank, int world,
                                        float scale, int dtype, int out_fp32, int ctas, cudaStream_t stream) {
  if (world > kMaxRanks) return -2;
  if (n_own == 0) return 0;
  const int V = dtype == 2 ? 4 : 8;
  if (n_own % V != 0 || (reinterpret_cast<uintptr_t>(out) & 15u)) return -2;
  if (ctas <= 0) ctas = 64;
  PeerPtrs b = make_ptrs(bucket_ptrs, world);
#define RS(T, O) reduce_scatter_pull_kernel<T, O><<<ctas, 512, 0, stream>>>(b, (O*)out, n_own, rank, world, scale)
  if (dtype == 2) RS(float, float);
  else if (dtype == 1) { if (out_fp32) RS(__nv_bfloat16, float); else RS(__nv_bfloat16, __nv_bfloat16); }
  else if (dtype == 0) { if (out_fp32) RS(__half, float); else RS(__half, __half); }
  else return -2;
#undef RS
  return (int)cudaGetLastError();
}

// In-place averaged (scale = 1/world) all-reduce of a flat symmetric bucket of n elements (n a multiple of
// world * 16 bytes).  grid_sync: 3 zero-initialised words in local memory.  Uses channels chan and chan+1.
extern "C" int fmsb_comm_allreduce(void* const* bucket_ptrs, void* const* signal_ptrs, long long n, int rank,
                                   int world, float scale, int dtype, int chan, unsigned epoch, unsigned* grid_sync,
                                   int ctas, int* status, cudaStream_t stream) {
  if (world > kMaxRanks) return -2;
  if (n == 0) return 0;
  const int V = dtype == 2 ? 4 : 8;
  if (n % ((long long)world * V) != 0) return -2;
  int maxc = fmsb_host::sm_count();
  if (ctas <= 0) ctas = 32;
  if (ctas > maxc) ctas = maxc;
  PeerPtrs b = make_ptrs(bucket_ptrs, world), s = make_ptrs(signal_ptrs, world);
  if (dtype == 2) allreduce_bucket_kernel<float><<<ctas, 512, 0, stream>>>(b, s, n, rank, world, scale, chan, epoch, grid_sync, status);
  else if (dtype == 1) allreduce_bucket_kernel<__nv_bfloat16><<<ctas, 512, 0, stream>>>(b, s, n, rank, world, scale, chan, epoch, grid_sync, status);
  else if (dtype == 0) allreduce_bucket_kernel<__half><<<ctas, 512, 0, stream>>>(b, s, n, rank, world, scale, chan, epoch, grid_sync, status);
  else return -2;
  return (int)cudaGetLastError();
}

extern "C" int fmsb_comm_wait_flag(const unsigned* flag, unsigned epoch, int* status, long long budget_cycles,
                                   cudaStream_t stream) {
  wait_flag_kernel<<<1, 1, 0, stream>>>(flag, epoch, status, budget_cycles);
  return (int)cudaGetLastError();
}

// The same all-reduce through the switch's multicast object: `mc_bucket` is the MULTICAST address of the symmetric
// bucket (0 elements allowed).  bf16 and fp32 buckets (the switch adds those; fp16 is not offered here).
extern "C" int fmsb_comm_allreduce_multimem(void* mc_bucket, void* const* signal_ptrs, long long n, int rank, int world,
                                            float scale, int dtype, int chan, unsigned epoch, unsigned* grid_sync, int ctas,
                                            int* status, cudaStream_t stream) {
  if (world > kMaxRanks || mc_bucket == nullptr) return -2;
  if (n == 0) return 0;
  const int V = dtype == 2 ? 4 : 8;
  if (n % ((long long)world * V) != 0 || (dtype != 1 && dtype != 2)) return -2;
  int maxc = fmsb_host::sm_count();
  if (ctas <= 0) ctas = 32;
  if (ctas > maxc) ctas = maxc;
  PeerPtrs s = make_ptrs(signal_ptrs, world);
  if (dtype == 2)
    allreduce_multimem_kernel<float><<<ctas, 512, 0, stream>>>((float*)mc_bucket, s, n, rank, world, scale, chan, epoch, grid_sync, status);
  else
    allreduce_multimem_kernel<__nv_bfloat16><<<ctas, 512, 0, stream>>>((__nv_bfloat16*)mc_bucket, s, n, rank, world, scale, chan, epoch, grid_sync, status);
  return (int)cudaGetLastError();
}
