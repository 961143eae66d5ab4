// Mixture-of-experts routing, dispatch and combine kernels (local and expert-parallel).
//
// Reference behaviour being reproduced (paths inside the reference project):
//   fms_acceleration_moe/utils/scattermoe.py:306-323        router: softmax (fp32) -> top-k -> renormalise
//   fms_acceleration_moe/utils/scattermoe.py:342-344 and
//   .../scattermoe_utils/khd/kernels/ops/__init__.py:26-56   sort by expert, per-128-row padded block offsets
//   .../scattermoe_utils/expert_parallel.py:97-232           expert-parallel all-to-all: exchange per-expert
//       counts, replicate every token top_k times grouped by destination expert, exchange rows, and on the way
//       back multiply by the routing weight and sum over top_k (with a host synchronisation per layer)
//   .../scattermoe_utils/megablocks/kernels/gather_scatter.py:37-278   row copy / scale / weight-gradient kernels
//
// Design here: no sort and no host synchronisation.  Tokens keep their order; a plan is computed on the
// device: expert histogram -> (expert-parallel: the histograms of all ranks are exchanged through peer
// memory) -> padded segment offsets of every expert in its owner's receive buffer -> a deterministic slot for
// every (token, k) pair.  `dispatch` then writes each token row straight into its slot, which lives in the
// owner rank's buffer (a peer store over NVLink when the owner is another rank), and `combine` reads the
// expert outputs back from the owners with the routing weight applied and the top-k sum fused.  Segments are
// padded to multiples of 128 rows and the pad rows are kept zero so that the grouped tcgen05 GEMMs
// (gemm_tcgen05.cu, modes 1 and 2) need no row masks.
#include "common.cuh"

namespace fmsb {

constexpr int kMoeMaxRanks = 16;
constexpr int kMoeMaxExperts = 512;

struct MoePeers {
  void* p[kMoeMaxRanks];
};

__device__ __forceinline__ void moe_st_release(uint32_t* addr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t moe_ld_acquire(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ bool moe_wait_ge(const uint32_t* addr, uint32_t epoch, int* status) {
  const long long t0 = clock64();
  while (true) {
    for (int i = 0; i < 64; ++i)
      if ((int32_t)(moe_ld_acquire(addr) - epoch) >= 0) return true;
    if (clock64() - t0 > peer_wait_budget(status)) {
      report_status(status, kTimeoutPeerFlag);
      return false;
    }
    if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) return false;
  }
}

// ----------------------------------------------------------------------------------------
// router: one warp per token.  logits [T, E] (fp32) -> probs of the top-k experts, renormalised.
// ----------------------------------------------------------------------------------------
template <int MAXPER>
__global__ void router_topk_kernel(const float* __restrict__ logits, int T, int E, int k, int renorm,
                                   int* __restrict__ topk_idx, float* __restrict__ topk_w) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= T) return;
  const float* row = logits + (long long)warp * E;
  float v[MAXPER];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < MAXPER; ++j) {
    const int e = lane + 32 * j;
    v[j] = e < E ? row[e] : -INFINITY;
    mx = fmaxf(mx, v[j]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < MAXPER; ++j) {
    v[j] = (lane + 32 * j) < E ? __expf(v[j] - mx) : 0.f;
    sum += v[j];
  }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
  float sel_sum = 0.f;
  float my_w = 0.f;
  int my_i = 0;
  for (int s = 0; s < k; ++s) {
    // arg-max over the warp; ties go to the lower expert index (as torch.topk on sorted indices)
    float best = -1.f;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < MAXPER; ++j) {
      const int e = lane + 32 * j;
      if (e < E && (v[j] > best || (v[j] == best && e < best_e))) {
        best = v[j];
        best_e = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_e = oe;
      }
    }
    if (lane == s) {
      my_w = best * inv;
      my_i = best_e;
    }
    sel_sum += best * inv;
#pragma unroll
    for (int j = 0; j < MAXPER; ++j)
      if (lane + 32 * j == best_e) v[j] = -2.f;  // taken
  }
  if (lane < k) {
    topk_idx[(long long)warp * k + lane] = my_i;
    topk_w[(long long)warp * k + lane] = renorm ? my_w / sel_sum : my_w;
  }
}

// Backward of the router: dlogits[t, e] from d(topk_w).  With p = softmax(logits), S = sum of the selected p and
// w_j = p_j / S (renorm) or w_j = p_j:  dL/dp_j = (g_j - sum_i g_i w_i) / S for selected j (renorm), g_j otherwise,
// 0 for unselected; then the softmax Jacobian.
template <int MAXPER>
__global__ void router_topk_bwd_kernel(const float* __restrict__ logits, const int* __restrict__ topk_idx,
                                       const float* __restrict__ topk_w, const float* __restrict__ dw, int T, int E,
                                       int k, int renorm, float* __restrict__ dlogits) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= T) return;
  const float* row = logits + (long long)warp * E;
  float p[MAXPER], dp[MAXPER];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < MAXPER; ++j) {
    const int e = lane + 32 * j;
    p[j] = e < E ? row[e] : -INFINITY;
    mx = fmaxf(mx, p[j]);
    dp[j] = 0.f;
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < MAXPER; ++j) {
    p[j] = (lane + 32 * j) < E ? __expf(p[j] - mx) : 0.f;
    sum += p[j];
  }
  sum = warp_sum(sum);
#pragma unroll
  for (int j = 0; j < MAXPER; ++j) p[j] /= sum;
  float gw = 0.f, S = 0.f;
  for (int s = 0; s < k; ++s) {
    const float g = dw[(long long)warp * k + s];
    const float w = topk_w[(long long)warp * k + s];
    gw += g * w;
    const int e = topk_idx[(long long)warp * k + s];
#pragma unroll
    for (int j = 0; j < MAXPER; ++j)
      if (lane + 32 * j == e) S += p[j];
  }
  S = warp_sum(S);
  for (int s = 0; s < k; ++s) {
    const float g = dw[(long long)warp * k + s];
    const int e = topk_idx[(long long)warp * k + s];
#pragma unroll
    for (int j = 0; j < MAXPER; ++j)
      if (lane + 32 * j == e) dp[j] = renorm ? (g - gw) / S : g;
  }
  float dot = 0.f;
#pragma unroll
  for (int j = 0; j < MAXPER; ++j) dot += dp[j] * p[j];
  dot = warp_sum(dot);
#pragma unroll
  for (int j = 0; j < MAXPER; ++j) {
    const int e = lane + 32 * j;
    if (e < E) dlogits[(long long)warp * E + e] = p[j] * (dp[j] - dot);
  }
}

// ----------------------------------------------------------------------------------------
// plan
// ----------------------------------------------------------------------------------------
// counts[e] = number of (token, k) pairs routed to global expert e (this rank's tokens)
__global__ void expert_count_kernel(const int* __restrict__ topk_idx, long long n, int E, int* __restrict__ counts) {
  extern __shared__ int sh[];
  for (int e = threadIdx.x; e < E; e += blockDim.x) sh[e] = 0;
  __syncthreads();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int e = topk_idx[i];
    if (e >= 0 && e < E) atomicAdd(&sh[e], 1);  // negative keys: entries without a pair
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x)
    if (sh[e]) atomicAdd(&counts[e], sh[e]);
}

// Exchange the histograms and derive the layout.  One CTA.
//   count_tables.p[r] : rank r's table int[world][E] (row s = histogram of source rank s); every rank writes its
//                       own histogram into row `rank` of every peer's table
//   signals.p[r]      : rank r's flag words, uint32[world] on the plan channel
// Outputs (local): seg_off[E_local + 1] padded (x128) offsets of my experts in my receive buffer,
//   seg_cnt[E_local] row counts, send_base[0..E) = first slot of MY rows of global expert e in its owner's buffer,
//   send_base[E..2E) = end of the valid slots of expert e.  When an owner's buffer (capacity rows) would overflow,
//   the excess rows are dropped consistently on every rank and *overflow is incremented.  That counter is
//   information for the host; it is NOT the status word, so the bounded waits of later kernels do not give up
//   because rows were dropped.
__global__ void moe_plan_kernel(MoePeers count_tables, MoePeers signals, const int* __restrict__ my_counts, int rank,
                                int world, int E, int capacity, uint32_t epoch, int* __restrict__ seg_off,
                                int* __restrict__ seg_cnt, int* __restrict__ send_base, int* needed, int* overflow,
                                int* status) {
  const int E_local = E / world;
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (world > 1) {
    // push my histogram to every rank, then signal
    for (int i = threadIdx.x; i < world * E; i += blockDim.x) {
      const int r = i / E, e = i % E;
      reinterpret_cast<int*>(count_tables.p[r])[rank * E + e] = my_counts[e];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < world) {
      moe_st_release(reinterpret_cast<uint32_t*>(signals.p[threadIdx.x]) + rank, epoch);
      if (!moe_wait_ge(reinterpret_cast<const uint32_t*>(signals.p[rank]) + threadIdx.x, epoch, status)) ok = 0;
    }
    __syncthreads();
    if (!ok) return;
  }
  const int* table = world > 1 ? reinterpret_cast<const int*>(count_tables.p[rank]) : my_counts;
  // every rank derives the layout of every owner (cheap, E <= 512)
  if (threadIdx.x == 0) {
    for (int owner = 0; owner < world; ++owner) {
      int off = 0, want = 0;  // want: rows the owner would need for nothing to be dropped
      for (int el = 0; el < E_local; ++el) {
        const int e = owner * E_local + el;
        int total = 0, before_me = 0;
        for (int s = 0; s < world; ++s) {
          const int c = world > 1 ? table[s * E + e] : table[e];
          if (s < rank) before_me += c;
          total += c;
        }
        // rows that do not fit into the owner's buffer are DROPPED (slot -1): nothing is ever written past the
        // buffer; the status word tells the host that the capacity factor was too small
        want += (total + 127) / 128 * 128;
        const int room = capacity - off;  // capacity and off are multiples of 128
        int kept = total;
        if (kept > room) {
          kept = room > 0 ? room : 0;
          if (overflow != nullptr) atomicAdd(overflow, 1);
        }
        send_base[e] = off + before_me;
        send_base[E + e] = off + kept;  // first slot that is no longer valid for expert e
        if (owner == rank) {
          seg_off[el] = off;
          seg_cnt[el] = kept;
        }
        off += (kept + 127) / 128 * 128;
      }
      if (owner == rank) seg_off[E_local] = off;
      if (needed != nullptr) atomicMax(needed, want);  // same value on every rank: all see all owners
    }
  }
}

// Deterministic slot of every (token, k) pair: the j-th pair (in token order) routed to expert e gets
// send_base[e] + j (or -1 past the expert's limit).  Three small launches over chunks of kAssignChunk pairs:
//   count   chunk_cnt[chunk][e] = pairs of the chunk routed to e
//   scan    chunk_cnt[chunk][e] <- send_base[e] + pairs of EARLIER chunks routed to e
//   assign  slot = chunk_cnt[chunk][e] + pairs of earlier warps of the chunk + earlier lanes of the warp with the same e
// Equal experts inside a warp are found with __match_any_sync, so there is no atomic and no sort anywhere.
constexpr int kAssignChunk = 1024;

// per-warp, per-expert pair counts of one chunk into wcnt[warp][e]; returns this lane's expert (or -1) and the
// mask of lanes of the warp that share it
__device__ __forceinline__ int assign_warp_counts(const int* __restrict__ topk_idx, long long n, int E, int* wcnt,
                                                  unsigned& peers) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 32 * E; i += blockDim.x) wcnt[i] = 0;
  __syncthreads();
  const long long i = (long long)blockIdx.x * kAssignChunk + threadIdx.x;
  const int e = i < n ? topk_idx[i] : -1;
  // lanes without a pair get distinct keys so that they match nobody
  peers = __match_any_sync(0xffffffffu, e >= 0 ? e : -1 - lane);
  if (e >= 0 && lane == __ffs(peers) - 1) wcnt[warp * E + e] = __popc(peers);
  __syncthreads();
  return e;
}

__global__ void __launch_bounds__(kAssignChunk) moe_assign_count_kernel(const int* __restrict__ topk_idx, long long n,
                                                                        int E, int* __restrict__ chunk_cnt) {
  extern __shared__ int wcnt[];
  unsigned peers;
  assign_warp_counts(topk_idx, n, E, wcnt, peers);
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int tot = 0;
#pragma unroll 8
    for (int w = 0; w < 32; ++w) tot += wcnt[w * E + e];
    chunk_cnt[(long long)blockIdx.x * E + e] = tot;
  }
}

// one CTA of 256 threads per expert: block-wide exclusive scan over the chunks, 256 chunks per trip
__global__ void __launch_bounds__(256) moe_assign_scan_kernel(int* __restrict__ chunk_cnt, int n_chunks, int E,
                                                              const int* __restrict__ send_base) {
  __shared__ int warp_tot[8];
  __shared__ int running;
  const int e = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) running = send_base[e];
  __syncthreads();
  for (int c0 = 0; c0 < n_chunks; c0 += 256) {
    const int c = c0 + threadIdx.x;
    const int v = c < n_chunks ? chunk_cnt[(long long)c * E + e] : 0;
    int incl = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += up;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    int before = running;
    for (int w = 0; w < warp; ++w) before += warp_tot[w];
    if (c < n_chunks) chunk_cnt[(long long)c * E + e] = before + incl - v;
    __syncthreads();
    if (threadIdx.x == 255) running = before + incl;
    __syncthreads();
  }
}

__global__ void __launch_bounds__(kAssignChunk) moe_assign_kernel(const int* __restrict__ topk_idx, long long n, int E,
                                                                  const int* __restrict__ chunk_cnt,
                                                                  const int* __restrict__ send_base,
                                                                  int* __restrict__ dest_row) {
  extern __shared__ int wcnt[];
  unsigned peers;
  const int e = assign_warp_counts(topk_idx, n, E, wcnt, peers);
  // exclusive prefix over the warps of the chunk, offset by the chunk's first slot
  for (int x = threadIdx.x; x < E; x += blockDim.x) {
    int run = chunk_cnt[(long long)blockIdx.x * E + x];
    for (int w = 0; w < 32; ++w) {
      const int v = wcnt[w * E + x];
      wcnt[w * E + x] = run;
      run += v;
    }
  }
  __syncthreads();
  if (e >= 0) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int slot = wcnt[warp * E + e] + __popc(peers & ((1u << lane) - 1));
    const long long i = (long long)blockIdx.x * kAssignChunk + threadIdx.x;
    dest_row[i] = slot < send_base[E + e] ? slot : -1;  // -1: dropped (capacity overflow)
  } else {
    const long long i = (long long)blockIdx.x * kAssignChunk + threadIdx.x;
    if (i < n) dest_row[i] = -1;  // entry without a pair (negative key)
  }
}

// ----------------------------------------------------------------------------------------
// dispatch / combine
// ----------------------------------------------------------------------------------------
// For every (token t, k): owner_buf[dest_row][:] = x[t][:] * (scale ? scale[t, k] : 1).  One warp per TOKEN: the
// row is read once into registers (up to 8 vectors of 16 bytes per lane at a time) and stored to its k
// destinations; lanes 0..k-1 fetch the (owner, row, scale) of the k pairs and hand them round by shuffle.
template <typename T, bool SCALED>
__global__ void __launch_bounds__(256) moe_dispatch_kernel(const T* __restrict__ x, long long ldx,
                                                           const int* __restrict__ topk_idx,
                                                           const int* __restrict__ dest_row,
                                                           const float* __restrict__ scale, long long n_tokens, int k,
                                                           int H, int E_local, MoePeers recv, long long ld_recv,
                                                           const float* __restrict__ meta_vals, MoePeers meta_recv,
                                                           int rows_per_src, const int* __restrict__ valid_cnt) {
  const long long t = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= n_tokens) return;
  // staged input (rows_per_src > 0): row t belongs to source block t / rows_per_src and is valid only below that
  // block's row count
  if (rows_per_src > 0 && (int)(t % rows_per_src) >= valid_cnt[t / rows_per_src]) return;
  int my_owner = 0, my_row = -1;
  float my_scale = 1.f;
  if (lane < k) {
    const long long pair = t * k + lane;
    my_owner = topk_idx != nullptr ? topk_idx[pair] / E_local : 0;
    my_row = dest_row[pair];
    if (SCALED) my_scale = scale[pair];
    // optional per-row scalar travelling with the row (the routing weight in the backward pass)
    if (meta_vals != nullptr && my_row >= 0) reinterpret_cast<float*>(meta_recv.p[my_owner])[my_row] = meta_vals[pair];
  }
  const T* src = x + t * ldx;
  const int nvec = H >> 3;
  for (int v0 = 0; v0 < nvec; v0 += 256) {
    uint4 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int vi = v0 + lane + 32 * j;
      if (vi < nvec) v[j] = *reinterpret_cast<const uint4*>(src + vi * 8);
    }
    for (int s = 0; s < k; ++s) {
      const int owner = __shfl_sync(0xffffffffu, my_owner, s);
      const int row = __shfl_sync(0xffffffffu, my_row, s);
      const float sc = __shfl_sync(0xffffffffu, my_scale, s);
      if (row < 0) continue;  // dropped pair
      T* dst = reinterpret_cast<T*>(recv.p[owner]) + (long long)row * ld_recv;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int vi = v0 + lane + 32 * j;
        if (vi >= nvec) continue;
        uint4 o = v[j];
        if (SCALED) {
          T* e = reinterpret_cast<T*>(&o);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            if (std::is_same<T, __nv_bfloat16>::value)
              reinterpret_cast<__nv_bfloat16*>(e)[i] = __float2bfloat16_rn(__bfloat162float(reinterpret_cast<__nv_bfloat16*>(e)[i]) * sc);
            else
              reinterpret_cast<__half*>(e)[i] = __float2half_rn(__half2float(reinterpret_cast<__half*>(e)[i]) * sc);
          }
        }
        *reinterpret_cast<uint4*>(dst + vi * 8) = o;
      }
    }
  }
}

// zero the pad rows [seg_off[e] + seg_cnt[e], seg_off[e + 1]) of a local buffer
template <typename T>
__global__ void moe_zero_pad_kernel(T* __restrict__ buf, long long ld, int H, const int* __restrict__ seg_off,
                                    const int* __restrict__ seg_cnt, int E_local) {
  const int e = blockIdx.x;
  const int r0 = seg_off[e] + seg_cnt[e], r1 = seg_off[e + 1];
  const int vec_per_row = H / 8;
  const long long total = (long long)(r1 - r0) * vec_per_row;
  for (long long i = threadIdx.x; i < total; i += blockDim.x) {
    const long long r = r0 + i / vec_per_row;
    const int c = (int)(i % vec_per_row) * 8;
    *reinterpret_cast<uint4*>(buf + r * ld + c) = make_uint4(0, 0, 0, 0);
  }
}

// out[t][:] = sum_k w[t, k] * owner_buf(t, k)[dest_row(t, k)][:]   (w == nullptr: plain sum).  One warp per token;
// the expert outputs are read from the owners' buffers (peer loads when remote).  Lanes 0..k-1 fetch the pair
// metadata once; the rows of two pairs (8 vectors of 16 bytes per lane) are in flight together.
// Predicated 16-byte load (zeros when `on` is false) that the compiler keeps where it is written: the combine kernel
// issues all loads of a pass as straight-line code before the first use (left to itself the compiler sinks each load
// next to its use and the gather runs one row at a time).
__device__ __forceinline__ uint4 ld_row16_if(const void* p, bool on) {
  uint4 v;
  asm volatile(
      "{\n\t.reg .pred q;\n\tsetp.ne.u32 q, %5, 0;\n\t"
      "mov.u32 %0, 0;\n\tmov.u32 %1, 0;\n\tmov.u32 %2, 0;\n\tmov.u32 %3, 0;\n\t"
      "@q ld.global.v4.u32 {%0, %1, %2, %3}, [%4];\n\t}"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(p), "r"((unsigned)on));
  return v;
}

// Empty statement that reads and redefines four loaded vectors.  Placed after the last load of a pass (volatile
// statements keep their order), it keeps every use of the loaded values behind ALL the loads of the pass.
__device__ __forceinline__ void pin_after_loads(uint4& a, uint4& b, uint4& c, uint4& d) {
  asm volatile("" : "+r"(a.x), "+r"(a.y), "+r"(a.z), "+r"(a.w), "+r"(b.x), "+r"(b.y), "+r"(b.z), "+r"(b.w), "+r"(c.x),
               "+r"(c.y), "+r"(c.z), "+r"(c.w), "+r"(d.x), "+r"(d.y), "+r"(d.z), "+r"(d.w));
}

template <typename T>
__device__ __forceinline__ void combine_add(float (&acc)[8], const uint4& v, float ws) {
  const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float f = std::is_same<T, __nv_bfloat16>::value
                        ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(e)[i])
                        : __half2float(reinterpret_cast<const __half*>(e)[i]);
    acc[i] += ws * f;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) moe_combine_kernel(MoePeers ybuf, long long ldy, const int* __restrict__ topk_idx,
                                                          const int* __restrict__ dest_row, const float* __restrict__ w,
                                                          long long T_tokens, int k, int H, int E_local,
                                                          T* __restrict__ out, long long ldo, int rows_per_src,
                                                          const int* __restrict__ valid_cnt) {
  const long long t = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= T_tokens) return;
  if (rows_per_src > 0 && (int)(t % rows_per_src) >= valid_cnt[t / rows_per_src]) return;  // see moe_dispatch_kernel
  int my_owner = 0, my_row = -1;
  float my_w = 1.f;
  if (lane < k) {
    const long long pair = t * k + lane;
    my_row = dest_row[pair];
    // entries without a row may carry a negative key: never index the peer table with it
    my_owner = (topk_idx != nullptr && my_row >= 0) ? topk_idx[pair] / E_local : 0;
    if (w != nullptr) my_w = w[pair];
  }
  // A pass covers 512 columns (two 16-byte vectors per lane) of up to eight source rows at once: sixteen independent
  // loads per lane are in flight before the first sum.  (Two rows at a time over 1024 columns left eight dependent
  // load rounds per token of a 1536-wide top-8 layer, and the gather ran at 0.45 of the copy bandwidth.)
  constexpr int CV = 2, RG = 8;
  const int nvec = H >> 3;
  for (int v0 = 0; v0 < nvec; v0 += 32 * CV) {
    float acc[CV][8];
#pragma unroll
    for (int j = 0; j < CV; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[j][i] = 0.f;
    for (int s0 = 0; s0 < k; s0 += RG) {
      uint4 a[RG][CV];
      float ws[RG];
#pragma unroll
      for (int u = 0; u < RG; ++u) {
        const int s = s0 + u;
        const int src = s < k ? s : 0;  // every lane takes part in the shuffles; rows beyond k contribute zeros
        const int o = __shfl_sync(0xffffffffu, my_owner, src);
        const int r = __shfl_sync(0xffffffffu, my_row, src);
        ws[u] = __shfl_sync(0xffffffffu, my_w, src);
        const bool on = s < k && r >= 0;  // a dropped pair contributes nothing
        const T* p = reinterpret_cast<const T*>(ybuf.p[o]) + (long long)(on ? r : 0) * ldy;
#pragma unroll
        for (int j = 0; j < CV; ++j) {
          const int vi = v0 + lane + 32 * j;
          a[u][j] = ld_row16_if(p + (vi < nvec ? vi : 0) * 8, on && vi < nvec);
        }
      }
#pragma unroll
      for (int u = 0; u < RG; u += 2) pin_after_loads(a[u][0], a[u][1], a[u + 1][0], a[u + 1][1]);
#pragma unroll
      for (int u = 0; u < RG; ++u)
#pragma unroll
        for (int j = 0; j < CV; ++j) combine_add<T>(acc[j], a[u][j], ws[u]);
    }
#pragma unroll
    for (int j = 0; j < CV; ++j) {
      const int vi = v0 + lane + 32 * j;
      if (vi >= nvec) continue;
      uint4 o;
      if (std::is_same<T, __nv_bfloat16>::value) {
        o.x = pack_bf16x2(acc[j][0], acc[j][1]); o.y = pack_bf16x2(acc[j][2], acc[j][3]);
        o.z = pack_bf16x2(acc[j][4], acc[j][5]); o.w = pack_bf16x2(acc[j][6], acc[j][7]);
      } else {
        o.x = pack_f16x2(acc[j][0], acc[j][1]); o.y = pack_f16x2(acc[j][2], acc[j][3]);
        o.z = pack_f16x2(acc[j][4], acc[j][5]); o.w = pack_f16x2(acc[j][6], acc[j][7]);
      }
      *reinterpret_cast<uint4*>(out + t * ldo + vi * 8) = o;
    }
  }
}

// dgate[t, k] = <owner_buf(t, k)[dest_row(t, k)], dout[t]>   (gradient of the routing weight).  One warp per pair.
template <typename T>
__global__ void moe_gate_grad_kernel(MoePeers ybuf, long long ldy, const int* __restrict__ topk_idx,
                                     const int* __restrict__ dest_row, const T* __restrict__ dout, long long lddo,
                                     long long n_pairs, int k, int H, int E_local, float* __restrict__ dgate) {
  const long long pair = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (pair >= n_pairs) return;
  const long long t = pair / k;
  if (dest_row[pair] < 0) {
    if (lane == 0) dgate[pair] = 0.f;
    return;
  }
  const int owner = topk_idx[pair] / E_local;
  const T* y = reinterpret_cast<const T*>(ybuf.p[owner]) + (long long)dest_row[pair] * ldy;
  const T* g = dout + t * lddo;
  float acc = 0.f;
  for (int c = lane * 8; c < H; c += 256) {
    const uint4 a = *reinterpret_cast<const uint4*>(y + c);
    const uint4 b = *reinterpret_cast<const uint4*>(g + c);
    const T* ea = reinterpret_cast<const T*>(&a);
    const T* eb = reinterpret_cast<const T*>(&b);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (std::is_same<T, __nv_bfloat16>::value)
        acc += __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(ea)[i]) * __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(eb)[i]);
      else
        acc += __half2float(reinterpret_cast<const __half*>(ea)[i]) * __half2float(reinterpret_cast<const __half*>(eb)[i]);
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) dgate[pair] = acc;
}

template <typename T>
__global__ void moe_rowdot_scale_kernel(const T* __restrict__ y, long long ldy, T* __restrict__ dy, long long lddy,
                                        const float* __restrict__ gate, float* __restrict__ dots,
                                        const int* __restrict__ seg_off, int E_local, int capacity, int H) {
  const long long row = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= capacity || row >= seg_off[E_local]) return;
  const float g = gate[row];
  const T* yr = y + row * ldy;
  T* dr = dy + row * lddy;
  float acc = 0.f;
  for (int c = lane * 8; c < H; c += 256) {
    const uint4 a = *reinterpret_cast<const uint4*>(yr + c);
    uint4 b = *reinterpret_cast<const uint4*>(dr + c);
    const T* ea = reinterpret_cast<const T*>(&a);
    T* eb = reinterpret_cast<T*>(&b);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (std::is_same<T, __nv_bfloat16>::value) {
        const float fb = __bfloat162float(reinterpret_cast<__nv_bfloat16*>(eb)[i]);
        acc += __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(ea)[i]) * fb;
        reinterpret_cast<__nv_bfloat16*>(eb)[i] = __float2bfloat16_rn(fb * g);
      } else {
        const float fb = __half2float(reinterpret_cast<__half*>(eb)[i]);
        acc += __half2float(reinterpret_cast<const __half*>(ea)[i]) * fb;
        reinterpret_cast<__half*>(eb)[i] = __float2half_rn(fb * g);
      }
    }
    *reinterpret_cast<uint4*>(dr + c) = b;
  }
  acc = warp_sum(acc);
  if (lane == 0) dots[row] = acc;
}

__global__ void moe_gather_scalar_kernel(MoePeers vals, const int* __restrict__ topk_idx,
                                         const int* __restrict__ dest_row, long long n_pairs, int E_local,
                                         float* __restrict__ out) {
  const long long pair = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (pair >= n_pairs) return;
  const int row = dest_row[pair];
  out[pair] = row < 0 ? 0.f : reinterpret_cast<const float*>(vals.p[topk_idx[pair] / E_local])[row];
}


// ----------------------------------------------------------------------------------------
// one row per (token, destination rank): staging
// ----------------------------------------------------------------------------------------
// A token whose top-k experts live on r different ranks crosses the links r times, not k times: the source
// writes the row ONCE per destination rank into that rank's staging block, together with the k slots (or -1) the
// row has to be replicated to inside the owner's expert-sorted buffer and the k routing weights.  The owner then
// replicates locally (moe_dispatch_kernel on its own memory), and on the way back reduces the up-to-k expert
// outputs of a staged row into one row before the source pulls it (moe_combine_kernel on its own memory).
//
// hit[t, r] = r when token t has at least one kept pair on rank r, else -1; cnt[r] = number of such tokens.
__global__ void moe_rank_hits_kernel(const int* __restrict__ topk_idx, const int* __restrict__ dest_row,
                                     long long n_tokens, int k, int E_local, int world, int* __restrict__ hit,
                                     int* __restrict__ cnt) {
  __shared__ int sh[kMoeMaxRanks];
  if (threadIdx.x < kMoeMaxRanks) sh[threadIdx.x] = 0;
  __syncthreads();
  const long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (t < n_tokens) {
    unsigned mask = 0;
    for (int j = 0; j < k; ++j)
      if (dest_row[t * k + j] >= 0) mask |= 1u << (topk_idx[t * k + j] / E_local);
    for (int r = 0; r < world; ++r) {
      const bool on = (mask >> r) & 1u;
      hit[t * world + r] = on ? r : -1;
      if (on) atomicAdd(&sh[r], 1);
    }
  }
  __syncthreads();
  if (threadIdx.x < world && sh[threadIdx.x]) atomicAdd(&cnt[threadIdx.x], sh[threadIdx.x]);
}

// One warp per token: x[t] goes to stage.p[r][stage_row[t, r]] for every rank r with stage_row >= 0; lanes 0..k-1
// deliver the row's metadata: meta_slot.p[r][row * k + j] = slot of pair j inside r's expert-sorted buffer when
// expert j lives on r (else -1), meta_gate.p[r][row * k + j] = routing weight of pair j.  CTA 0 also tells every
// rank how many rows this rank staged there (cnt_recv.p[r][me] = stage_cnt[r]).
template <typename T>
__global__ void __launch_bounds__(256) moe_dispatch_staged_kernel(
    const T* __restrict__ x, long long ldx, const int* __restrict__ topk_idx, const int* __restrict__ dest_row,
    const float* __restrict__ gates, const int* __restrict__ stage_row, const int* __restrict__ stage_cnt,
    long long n_tokens, int k, int H, int E_local, int world, int me, MoePeers stage, long long ld_stage,
    MoePeers meta_slot, MoePeers meta_gate, MoePeers cnt_recv) {
  if (blockIdx.x == 0 && threadIdx.x < world)
    reinterpret_cast<int*>(cnt_recv.p[threadIdx.x])[me] = stage_cnt[threadIdx.x];
  const long long t = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= n_tokens) return;
  int my_owner = -1, my_slot = -1;
  float my_gate = 1.f;
  if (lane < k) {
    const long long pair = t * k + lane;
    my_slot = dest_row[pair];
    my_owner = topk_idx[pair] / E_local;
    if (gates != nullptr) my_gate = gates[pair];
  }
  const int* srow = stage_row + t * world;
  for (int r = 0; r < world; ++r) {
    const int row = srow[r];
    if (row < 0 || lane >= k) continue;
    reinterpret_cast<int*>(meta_slot.p[r])[(long long)row * k + lane] = (my_owner == r) ? my_slot : -1;
    reinterpret_cast<float*>(meta_gate.p[r])[(long long)row * k + lane] = my_gate;
  }
  const T* src = x + t * ldx;
  const int nvec = H >> 3;
  for (int v0 = 0; v0 < nvec; v0 += 256) {
    uint4 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int vi = v0 + lane + 32 * j;
      if (vi < nvec) v[j] = *reinterpret_cast<const uint4*>(src + vi * 8);
    }
    for (int r = 0; r < world; ++r) {
      const int row = srow[r];
      if (row < 0) continue;
      T* dst = reinterpret_cast<T*>(stage.p[r]) + (long long)row * ld_stage;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int vi = v0 + lane + 32 * j;
        if (vi < nvec) *reinterpret_cast<uint4*>(dst + vi * 8) = v[j];
      }
    }
  }
}

}  // namespace fmsb

using namespace fmsb;

static MoePeers moe_ptrs(void* const* arr, int world) {
  MoePeers p{};
  for (int i = 0; i < world && i < kMoeMaxRanks; ++i) p.p[i] = arr[i];
  return p;
}

extern "C" int fmsb_moe_router(const float* logits, int T, int E, int k, int renorm, int* topk_idx, float* topk_w,
                               cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E > 256 || k > 32 || k > E) return -2;
  const int grid = (T * 32 + 255) / 256;
  if (E <= 64) router_topk_kernel<2><<<grid, 256, 0, stream>>>(logits, T, E, k, renorm, topk_idx, topk_w);
  else router_topk_kernel<8><<<grid, 256, 0, stream>>>(logits, T, E, k, renorm, topk_idx, topk_w);
  return (int)cudaGetLastError();
}

extern "C" int fmsb_moe_router_bwd(const float* logits, const int* topk_idx, const float* topk_w, const float* dw, int T,
                                   int E, int k, int renorm, float* dlogits, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E > 256 || k > 32) return -2;
  const int grid = (T * 32 + 255) / 256;
  if (E <= 64) router_topk_bwd_kernel<2><<<grid, 256, 0, stream>>>(logits, topk_idx, topk_w, dw, T, E, k, renorm, dlogits);
  else router_topk_bwd_kernel<8><<<grid, 256, 0, stream>>>(logits, topk_idx, topk_w, dw, T, E, k, renorm, dlogits);
  return (int)cudaGetLastError();
}

// counts must be zeroed by the caller.  Then plan + assign.  count_tables / signals may be null when world == 1.
// chunk_scratch: ceil(n_pairs / 1024) * E ints of work space for the slot assignment.
// overflow (may be null): incremented once per expert whose rows did not all fit; separate from the status word.
extern "C" int fmsb_moe_plan(const int* topk_idx, long long n_pairs, int E, int rank, int world, int capacity,
                             int* counts, void* const* count_tables, void* const* signals, unsigned epoch,
                             int* seg_off, int* seg_cnt, int* send_base, int* dest_row, int* needed,
                             int* chunk_scratch, int* overflow, int* status, cudaStream_t stream) {
  if (E > kMoeMaxExperts || world > kMoeMaxRanks || E % world != 0) return -2;
  if (n_pairs > 0 && chunk_scratch == nullptr) return -2;
  if (n_pairs > 0) {
    long long blocks = (n_pairs + 255) / 256;
    if (blocks > 1024) blocks = 1024;
    expert_count_kernel<<<(int)blocks, 256, E * sizeof(int), stream>>>(topk_idx, n_pairs, E, counts);
  }
  MoePeers ct = world > 1 ? moe_ptrs(count_tables, world) : MoePeers{};
  MoePeers sg = world > 1 ? moe_ptrs(signals, world) : MoePeers{};
  moe_plan_kernel<<<1, 256, 0, stream>>>(ct, sg, counts, rank, world, E, capacity, epoch, seg_off, seg_cnt, send_base,
                                         needed, overflow, status);
  if (n_pairs > 0) {
    const int n_chunks = (int)((n_pairs + kAssignChunk - 1) / kAssignChunk);
    const size_t smem = (size_t)32 * E * sizeof(int);  // at most 64 KB (E <= 512)
    if (smem > 48 * 1024) {
      cudaFuncSetAttribute(moe_assign_count_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      cudaFuncSetAttribute(moe_assign_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
    moe_assign_count_kernel<<<n_chunks, kAssignChunk, smem, stream>>>(topk_idx, n_pairs, E, chunk_scratch);
    moe_assign_scan_kernel<<<E, 256, 0, stream>>>(chunk_scratch, n_chunks, E, send_base);
    moe_assign_kernel<<<n_chunks, kAssignChunk, smem, stream>>>(topk_idx, n_pairs, E, chunk_scratch, send_base, dest_row);
  }
  return (int)cudaGetLastError();
}

extern "C" int fmsb_moe_dispatch(const void* x, long long ldx, const int* topk_idx, const int* dest_row,
                                 const float* scale, long long n_pairs, int k, int H, int E_local, void* const* recv,
                                 long long ld_recv, int world, int dtype, cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  if (H % 8 != 0 || ldx % 8 != 0 || ld_recv % 8 != 0 || k < 1 || k > 32 || n_pairs % k != 0) return -2;
  MoePeers r = moe_ptrs(recv, world);
  const long long n_tokens = n_pairs / k;
  const long long blocks = (n_tokens * 32 + 255) / 256;
#define FMSB_DISPATCH_CALL(T, SC) \
  moe_dispatch_kernel<T, SC><<<(unsigned)blocks, 256, 0, stream>>>((const T*)x, ldx, topk_idx, dest_row, scale, n_tokens, k, H, E_local, r, ld_recv, nullptr, MoePeers{}, 0, nullptr)
  if (dtype == 1) { if (scale != nullptr) FMSB_DISPATCH_CALL(__nv_bfloat16, true); else FMSB_DISPATCH_CALL(__nv_bfloat16, false); }
  else { if (scale != nullptr) FMSB_DISPATCH_CALL(__half, true); else FMSB_DISPATCH_CALL(__half, false); }
#undef FMSB_DISPATCH_CALL
  return (int)cudaGetLastError();
}

// Dispatch that also delivers one fp32 value per (token, k) pair into the owner's per-row array `meta_recv`.
extern "C" int fmsb_moe_dispatch_meta(const void* x, long long ldx, const int* topk_idx, const int* dest_row,
                                      const float* meta_vals, long long n_pairs, int k, int H, int E_local,
                                      void* const* recv, long long ld_recv, void* const* meta_recv, int world, int dtype,
                                      cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  if (H % 8 != 0 || ldx % 8 != 0 || ld_recv % 8 != 0 || meta_vals == nullptr || k < 1 || k > 32 || n_pairs % k != 0)
    return -2;
  MoePeers r = moe_ptrs(recv, world), m = moe_ptrs(meta_recv, world);
  const long long n_tokens = n_pairs / k;
  const long long blocks = (n_tokens * 32 + 255) / 256;
  if (dtype == 1)
    moe_dispatch_kernel<__nv_bfloat16, false><<<(unsigned)blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, ldx, topk_idx, dest_row, nullptr, n_tokens, k, H, E_local, r, ld_recv, meta_vals, m, 0, nullptr);
  else
    moe_dispatch_kernel<__half, false><<<(unsigned)blocks, 256, 0, stream>>>((const __half*)x, ldx, topk_idx, dest_row, nullptr, n_tokens, k, H, E_local, r, ld_recv, meta_vals, m, 0, nullptr);
  return (int)cudaGetLastError();
}

// Owner side of the routing-weight gradient: dots[row] = <y[row], dy[row]>, then dy[row] *= gate[row]; rows below
// seg_off[E_local] only (everything this rank received).  One warp per row.
extern "C" int fmsb_moe_rowdot_scale(const void* y, long long ldy, void* dy, long long lddy, const float* gate,
                                     float* dots, const int* seg_off, int E_local, int capacity, int H, int dtype,
                                     cudaStream_t stream) {
  if (capacity <= 0) return 0;
  if (H % 8 != 0 || ldy % 8 != 0 || lddy % 8 != 0) return -2;
  const long long blocks = ((long long)capacity * 32 + 255) / 256;
  if (dtype == 1)
    moe_rowdot_scale_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, stream>>>((const __nv_bfloat16*)y, ldy, (__nv_bfloat16*)dy, lddy, gate, dots, seg_off, E_local, capacity, H);
  else
    moe_rowdot_scale_kernel<__half><<<(unsigned)blocks, 256, 0, stream>>>((const __half*)y, ldy, (__half*)dy, lddy, gate, dots, seg_off, E_local, capacity, H);
  return (int)cudaGetLastError();
}

// out[pair] = owner's vals[dest_row[pair]] (0 for a dropped pair): 4 bytes per pair cross the link.
extern "C" int fmsb_moe_gather_scalar(void* const* vals, const int* topk_idx, const int* dest_row, long long n_pairs,
                                      int E_local, float* out, int world, cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  MoePeers v = moe_ptrs(vals, world);
  moe_gather_scalar_kernel<<<(unsigned)((n_pairs + 255) / 256), 256, 0, stream>>>(v, topk_idx, dest_row, n_pairs, E_local, out);
  return (int)cudaGetLastError();
}

extern "C" int fmsb_moe_zero_pad(void* buf, long long ld, int H, const int* seg_off, const int* seg_cnt, int E_local,
                                 int dtype, cudaStream_t stream) {
  if (E_local <= 0) return 0;
  if (H % 8 != 0 || ld % 8 != 0) return -2;
  if (dtype == 1) moe_zero_pad_kernel<__nv_bfloat16><<<E_local, 256, 0, stream>>>((__nv_bfloat16*)buf, ld, H, seg_off, seg_cnt, E_local);
  else moe_zero_pad_kernel<__half><<<E_local, 256, 0, stream>>>((__half*)buf, ld, H, seg_off, seg_cnt, E_local);
  return (int)cudaGetLastError();
}

extern "C" int fmsb_moe_combine(void* const* ybuf, long long ldy, const int* topk_idx, const int* dest_row,
                                const float* w, long long T_tokens, int k, int H, int E_local, void* out, long long ldo,
                                int world, int dtype, cudaStream_t stream) {
  if (T_tokens <= 0) return 0;
  if (H % 8 != 0 || ldy % 8 != 0 || ldo % 8 != 0 || k < 1 || k > 32) return -2;
  MoePeers y = moe_ptrs(ybuf, world);
  const long long blocks = (T_tokens * 32 + 255) / 256;
  if (dtype == 1)
    moe_combine_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, stream>>>(y, ldy, topk_idx, dest_row, w, T_tokens, k, H, E_local, (__nv_bfloat16*)out, ldo, 0, nullptr);
  else
    moe_combine_kernel<__half><<<(unsigned)blocks, 256, 0, stream>>>(y, ldy, topk_idx, dest_row, w, T_tokens, k, H, E_local, (__half*)out, ldo, 0, nullptr);
  return (int)cudaGetLastError();
}

extern "C" int fmsb_moe_gate_grad(void* const* ybuf, long long ldy, const int* topk_idx, const int* dest_row,
                                  const void* dout, long long lddo, long long n_pairs, int k, int H, int E_local,
                                  float* dgate, int world, int dtype, cudaStream_t stream) {
  if (n_pairs <= 0) return 0;
  MoePeers y = moe_ptrs(ybuf, world);
  const long long blocks = (n_pairs * 32 + 255) / 256;
  if (dtype == 1)
    moe_gate_grad_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, stream>>>(y, ldy, topk_idx, dest_row, (const __nv_bfloat16*)dout, lddo, n_pairs, k, H, E_local, dgate);
  else
    moe_gate_grad_kernel<__half><<<(unsigned)blocks, 256, 0, stream>>>(y, ldy, topk_idx, dest_row, (const __half*)dout, lddo, n_pairs, k, H, E_local, dgate);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------- staged exchange
// Staging layout of the per-(token, rank) exchange.  hit / stage_row are [n_tokens, world]; stage_base holds
// 2 * world ints: the first staging row of this rank's block (rank * rows_per_src) world times, then its end.
// chunk_scratch: ceil(n_tokens * world / 1024) * world ints.  stage_cnt[world] is zeroed here.
extern "C" int fmsb_moe_stage_plan(const int* topk_idx, const int* dest_row, long long n_tokens, int k, int E_local,
                                   int world, const int* stage_base, int* hit, int* stage_row, int* stage_cnt,
                                   int* chunk_scratch, cudaStream_t stream) {
  if (world > kMoeMaxRanks || k < 1 || k > 32) return -2;
  cudaError_t e = cudaMemsetAsync(stage_cnt, 0, sizeof(int) * world, stream);
  if (e != cudaSuccess) return (int)e;
  if (n_tokens <= 0) return 0;
  moe_rank_hits_kernel<<<(unsigned)((n_tokens + 255) / 256), 256, 0, stream>>>(topk_idx, dest_row, n_tokens, k, E_local,
                                                                             world, hit, stage_cnt);
  const long long n = n_tokens * world;
  const int n_chunks = (int)((n + kAssignChunk - 1) / kAssignChunk);
  const size_t smem = (size_t)32 * world * sizeof(int);
  moe_assign_count_kernel<<<n_chunks, kAssignChunk, smem, stream>>>(hit, n, world, chunk_scratch);
  moe_assign_scan_kernel<<<world, 256, 0, stream>>>(chunk_scratch, n_chunks, world, stage_base);
  moe_assign_kernel<<<n_chunks, kAssignChunk, smem, stream>>>(hit, n, world, chunk_scratch, stage_base, stage_row);
  return (int)cudaGetLastError();
}

// Source side: push every token row once per destination rank, with its slots and routing weights.
extern "C" int fmsb_moe_dispatch_staged(const void* x, long long ldx, const int* topk_idx, const int* dest_row,
                                        const float* gates, const int* stage_row, const int* stage_cnt,
                                        long long n_tokens, int k, int H, int E_local, int world, int me,
                                        void* const* stage, long long ld_stage, void* const* meta_slot,
                                        void* const* meta_gate, void* const* cnt_recv, int dtype, cudaStream_t stream) {
  if (world > kMoeMaxRanks || H % 8 != 0 || ldx % 8 != 0 || ld_stage % 8 != 0 || k < 1 || k > 32) return -2;
  MoePeers st = moe_ptrs(stage, world), ms = moe_ptrs(meta_slot, world), mg = moe_ptrs(meta_gate, world),
           cr = moe_ptrs(cnt_recv, world);
  long long blocks = (n_tokens * 32 + 255) / 256;
  if (blocks < 1) blocks = 1;  // the row counts are delivered even when this rank has no token
  if (dtype == 1)
    moe_dispatch_staged_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, stream>>>(
        (const __nv_bfloat16*)x, ldx, topk_idx, dest_row, gates, stage_row, stage_cnt, n_tokens, k, H, E_local, world, me,
        st, ld_stage, ms, mg, cr);
  else
    moe_dispatch_staged_kernel<__half><<<(unsigned)blocks, 256, 0, stream>>>(
        (const __half*)x, ldx, topk_idx, dest_row, gates, stage_row, stage_cnt, n_tokens, k, H, E_local, world, me, st,
        ld_stage, ms, mg, cr);
  return (int)cudaGetLastError();
}

// Owner side, local memory only: staged row i (block i / rows_per_src, valid below cnt[block]) is copied to the
// slots meta_slot[i, 0..k) of the expert-sorted buffer; slot_vals (optional, [rows, k]) is delivered per slot into
// slot_out (the routing weight of every received row in the backward pass).
extern "C" int fmsb_moe_replicate(const void* stage, long long ld_stage, const int* meta_slot, const float* slot_vals,
                                  float* slot_out, long long n_rows, int rows_per_src, const int* cnt, int k, int H,
                                  void* buf, long long ld_buf, int dtype, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (H % 8 != 0 || ld_stage % 8 != 0 || ld_buf % 8 != 0 || k < 1 || k > 32 || rows_per_src <= 0) return -2;
  MoePeers r{}, m{};
  r.p[0] = buf;
  m.p[0] = slot_out;
  const float* mv = slot_out != nullptr ? slot_vals : nullptr;
  const long long blocks = (n_rows * 32 + 255) / 256;
  if (dtype == 1)
    moe_dispatch_kernel<__nv_bfloat16, false><<<(unsigned)blocks, 256, 0, stream>>>(
        (const __nv_bfloat16*)stage, ld_stage, nullptr, meta_slot, nullptr, n_rows, k, H, 1, r, ld_buf, mv, m,
        rows_per_src, cnt);
  else
    moe_dispatch_kernel<__half, false><<<(unsigned)blocks, 256, 0, stream>>>(
        (const __half*)stage, ld_stage, nullptr, meta_slot, nullptr, n_rows, k, H, 1, r, ld_buf, mv, m, rows_per_src, cnt);
  return (int)cudaGetLastError();
}

// Owner side, local memory only: out[i] = sum_j w[i, j] * buf[meta_slot[i, j]] over the slots >= 0 of staged row i
// (w null: plain sum).  This is the reduction that lets one row per (token, rank) travel back.
extern "C" int fmsb_moe_prereduce(const void* buf, long long ld_buf, const int* meta_slot, const float* w,
                                  long long n_rows, int rows_per_src, const int* cnt, int k, int H, void* out,
                                  long long ld_out, int dtype, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (H % 8 != 0 || ld_buf % 8 != 0 || ld_out % 8 != 0 || k < 1 || k > 32 || rows_per_src <= 0) return -2;
  MoePeers y{};
  y.p[0] = const_cast<void*>(buf);
  const long long blocks = (n_rows * 32 + 255) / 256;
  if (dtype == 1)
    moe_combine_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, stream>>>(
        y, ld_buf, nullptr, meta_slot, w, n_rows, k, H, 1, (__nv_bfloat16*)out, ld_out, rows_per_src, cnt);
  else
    moe_combine_kernel<__half><<<(unsigned)blocks, 256, 0, stream>>>(y, ld_buf, nullptr, meta_slot, w, n_rows, k, H, 1,
                                                                   (__half*)out, ld_out, rows_per_src, cnt);
  return (int)cudaGetLastError();
}
