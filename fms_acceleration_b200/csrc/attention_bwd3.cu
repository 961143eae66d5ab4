// Attention backward, full-width issue order.  Replaces the backward half of flash_attn_varlen_func as used by the reference's
// padding-free plugin (fms_acceleration_aadp/flash_attn.py:108-199).
//
// What the timeline trace of an earlier half-tile design (128x64 products) showed: the single MMA-issuing thread, not the exponentials,
// was the critical path, because a 128x64x16 product costs almost as much issue/operand time as a 128x128x16 one.
// Here every product is 128 wide and the element-wise work is split into two stages that each overlap a pair of
// products:
//
//   dK/dV kernel (fixed key tile; K and V rows are the M side, queries are streamed)
//     MMA order      S^T(j)  dP^T(j) | dV(j)  S^T(j+1) | dK(j)  dP^T(j+1) | dV(j+1) ...
//     compute order            A(j): P^T = exp2(S^T..) -> packed over S^T      (needs S^T(j))
//                              B(j): dS^T = P^T o (dP^T - delta) -> over dP^T  (needs dP^T(j))
//     dV(j) waits for A(j), dK(j) for B(j); A(j+1) runs while dK(j), dP^T(j+1) execute.
//   dQ kernel (fixed query tile; Q and dO are copied ONCE into tensor memory as packed 16-bit and serve as the
//     A operand of S = Q K^T and dP = dO V^T, so those products read only the K / V tile from shared memory)
//     MMA order      S(j) dP(j) | S(j+1) | dQ(j) dP(j+1) | S(j+2) ...
//     compute order  load S(j) (then S(j+1) may overwrite it), P in registers, B(j): dS over dP(j)
//
// Tensor memory (512 columns): dK/dV: S^T 128 | dP^T 128 | dV D | dK D.   dQ: Q D/2 | dO D/2 | S 128 | dP 128 | dQ D.
// P is kept as packed 16-bit between the stages (it is the operand of dV in that precision anyway).
// Warp roles (320 threads): warp 0 TMA producer, warp 1 MMA issuer, warps 2-9 compute; a compute warp owns lane
// quarter `warp % 4` and 64 of the 128 columns.  Every wait is bounded.
#include "common.cuh"

namespace fmsb {

constexpr int B3_T = 128;  // tile edge (queries and keys)

struct AttnBwd3Params {
  int T, nh, nkv, d;
  float scale;
  const int* doc_start;
  const int* doc_end;
  const float* lse;    // [nh, T]
  const float* delta;  // [nh, T]
  void* dq;
  long long lddq;
  void* dk;
  long long lddk;
  void* dv;
  long long lddv;
  int fmt;
  int* status;
};

template <int D>
struct AttnBwd3Cfg {
  static constexpr int kTileBytes = 128 * D * 2;
  static constexpr int kHalfBytes = 128 * 64 * 2;
  static constexpr int kScalarBytes = 2 * 3 * 128 * 4;
  static constexpr int kSmemBytes = 6 * kTileBytes + kScalarBytes + 1024 + 256;
};

__device__ __forceinline__ uint32_t b3_pack2(float a, float b, int fmt) {
  return fmt == 1 ? pack_bf16x2(a, b) : pack_f16x2(a, b);
}
__device__ __forceinline__ void b3_unpack2(uint32_t w, int fmt, float& a, float& b) {
  if (fmt == 1) {
    a = __uint_as_float(w << 16);
    b = __uint_as_float(w & 0xffff0000u);
  } else {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
    a = f.x;
    b = f.y;
  }
}
__device__ __forceinline__ void b3_store_row_chunk(uint16_t* dst, const uint32_t (&r)[32], float mul, int fmt) {
#pragma unroll
  for (int i = 0; i < 32; i += 8) {
    uint4 u;
    u.x = b3_pack2(__uint_as_float(r[i]) * mul, __uint_as_float(r[i + 1]) * mul, fmt);
    u.y = b3_pack2(__uint_as_float(r[i + 2]) * mul, __uint_as_float(r[i + 3]) * mul, fmt);
    u.z = b3_pack2(__uint_as_float(r[i + 4]) * mul, __uint_as_float(r[i + 5]) * mul, fmt);
    u.w = b3_pack2(__uint_as_float(r[i + 6]) * mul, __uint_as_float(r[i + 7]) * mul, fmt);
    *reinterpret_cast<uint4*>(dst + i) = u;
  }
}
// Optional timeline trace (compile with -DFMSB_TRACE): one CTA of the dQ kernel records clock64() at the hand-off
// points of its MMA issuer and of one compute thread; read back with fmsb_attn_trace3_read.
#ifdef FMSB_TRACE
__device__ long long g_trace3[8192];
#define FMSB_TRACE3(cond, slot) do { if ((cond) && (slot) < 8192) g_trace3[(slot)] = clock64(); } while (0)
#else
#define FMSB_TRACE3(cond, slot) do { } while (0)
#endif

__device__ __forceinline__ void b3_compute_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// Column of K-step `ks` (16 elements = 8 packed columns) of a packed 128-element row: the warp of columns 0-63
// packs into columns 0-31, the warp of columns 64-127 into columns 64-95 (each overwrites only what it has read).
__device__ __forceinline__ uint32_t b3_pcol(int ks) { return static_cast<uint32_t>((ks >> 2) * 64 + (ks & 3) * 8); }

// ----------------------------------------------------------------------------------------
// dV[kv tile, kv head] = sum P^T dO ,  dK = scale * sum dS^T Q
// ----------------------------------------------------------------------------------------
template <int D, int FMT>
__global__ void __launch_bounds__(320, 1)
attn_bwd_dkv3_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                     const AttnBwd3Params p) {
  using Cfg = AttnBwd3Cfg<D>;
  constexpr int NH = D / 64;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sK = base;
  const uint32_t sV = base + Cfg::kTileBytes;
  auto sQ = [&](int s) { return base + Cfg::kTileBytes * (2 + 2 * s); };
  auto sdO = [&](int s) { return base + Cfg::kTileBytes * (3 + 2 * s); };
  const uint32_t scal = base + Cfg::kTileBytes * 6;
  const uint32_t bars = scal + Cfg::kScalarBytes;
  const uint32_t bar_kv = bars;
  auto bar_qdo_full = [&](int s) { return bars + 8u * (1 + s); };
  auto bar_qdo_empty = [&](int s) { return bars + 8u * (3 + s); };
  const uint32_t bar_s_full = bars + 8u * 5, bar_dp_full = bars + 8u * 6;
  const uint32_t bar_pa_full = bars + 8u * 7, bar_pb_full = bars + 8u * 8;
  const uint32_t bar_acc_done = bars + 8u * 9;
  const uint32_t holder = bars + 8u * 10;
  float* scal_f = reinterpret_cast<float*>(smem_raw + (scal - smem_u32(smem_raw)));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kt = blockIdx.x;
  const int hk = blockIdx.y;
  const int G = p.nh / p.nkv;
  const int k0 = kt * B3_T;
  const int k_last = min(k0 + B3_T - 1, p.T - 1);
  const int de_last = p.doc_end[k_last];
  const int qb_lo = kt;
  const int qb_hi = (de_last - 1) / B3_T;
  const int nq = qb_hi - qb_lo + 1;
  const int niter = nq * G;

  if (warp == 1 && lane == 0) {
    mbar_init(bar_kv, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_qdo_full(s), 1);
      mbar_init(bar_qdo_empty(s), 1);
    }
    mbar_init(bar_s_full, 1);
    mbar_init(bar_dp_full, 1);
    mbar_init(bar_pa_full, 8);
    mbar_init(bar_pb_full, 8);
    mbar_init(bar_acc_done, 1);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(holder, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem) : "r"(holder));
  const uint32_t tS = tmem, tdP = tmem + 128u, tdV = tmem + 256u, tdK = tmem + 256u + D;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(bar_kv, 2 * Cfg::kTileBytes);
#pragma unroll
      for (int h = 0; h < NH; ++h) {
        tma_load_2d(sK + h * Cfg::kHalfBytes, &tmK, bar_kv, hk * D + 64 * h, k0);
        tma_load_2d(sV + h * Cfg::kHalfBytes, &tmV, bar_kv, hk * D + 64 * h, k0);
      }
      for (int it = 0; it < niter; ++it) {
        const int s = it & 1;
        if (!mbar_wait(bar_qdo_empty(s), ((it >> 1) & 1) ^ 1u, p.status, kTimeoutProducer)) break;
        const int head = hk * G + it / nq;
        const int q0 = (qb_lo + it % nq) * B3_T;
        mbar_expect_tx(bar_qdo_full(s), 2 * Cfg::kTileBytes);
#pragma unroll
        for (int h = 0; h < NH; ++h) {
          tma_load_2d(sQ(s) + h * Cfg::kHalfBytes, &tmQ, bar_qdo_full(s), head * D + 64 * h, q0);
          tma_load_2d(sdO(s) + h * Cfg::kHalfBytes, &tmdO, bar_qdo_full(s), head * D + 64 * h, q0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_f16(128, 128, FMT, 0, 0);
      const uint32_t idesc_g = make_idesc_f16(128, D, FMT, 0, 1);
      const SmemDescBase dK = make_smem_desc_base(sK, 16, 1024), dV = make_smem_desc_base(sV, 16, 1024);
      auto issue_s = [&](int s) {  // S^T = K Q^T
        const SmemDescBase dQ = make_smem_desc_base(sQ(s), 16, 1024);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks / 4) * Cfg::kHalfBytes + (ks % 4) * 32;
          tc_mma_f16(tS, smem_desc_at(dK, off), smem_desc_at(dQ, off), idesc_s, ks != 0);
        }
        tc_commit(bar_s_full);
      };
      auto issue_dp = [&](int s) {  // dP^T = V dO^T
        const SmemDescBase ddO = make_smem_desc_base(sdO(s), 16, 1024);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks / 4) * Cfg::kHalfBytes + (ks % 4) * 32;
          tc_mma_f16(tdP, smem_desc_at(dV, off), smem_desc_at(ddO, off), idesc_s, ks != 0);
        }
        tc_commit(bar_dp_full);
      };
      auto issue_acc = [&](uint32_t acc, uint32_t a_tmem, uint32_t b_tile, bool first) {  // acc += A[tmem] . B[tile]
        const SmemDescBase b = make_smem_desc_base(b_tile, Cfg::kHalfBytes, 1024);
        tc_mma_f16_ts(acc, a_tmem + b3_pcol(0), smem_desc_at(b, 0), idesc_g, first ? 0u : 1u);
#pragma unroll
        for (int ks = 1; ks < 8; ++ks) tc_mma_f16_ts(acc, a_tmem + b3_pcol(ks), smem_desc_at(b, ks * 2048), idesc_g, 1u);
      };
      bool ok = mbar_wait(bar_kv, 0, p.status, kTimeoutMma);
      if (ok) ok = mbar_wait(bar_qdo_full(0), 0, p.status, kTimeoutMma);
      if (ok) {
        tc_fence_after();
        issue_s(0);
        issue_dp(0);
      }
      for (int it = 0; it < niter && ok; ++it) {
        const int s = it & 1;
        const bool more = it + 1 < niter;
        if (!mbar_wait(bar_pa_full, it & 1, p.status, kTimeoutMma)) { ok = false; break; }
        tc_fence_after();
        issue_acc(tdV, tS, sdO(s), it == 0);
        if (more) {
          if (!mbar_wait(bar_qdo_full(s ^ 1), ((it + 1) >> 1) & 1, p.status, kTimeoutMma)) { ok = false; break; }
          tc_fence_after();
          issue_s(s ^ 1);
        }
        if (!mbar_wait(bar_pb_full, it & 1, p.status, kTimeoutMma)) { ok = false; break; }
        tc_fence_after();
        issue_acc(tdK, tdP, sQ(s), it == 0);
        tc_commit(bar_qdo_empty(s));
        if (more) issue_dp(s ^ 1);
      }
      if (ok) tc_commit(bar_acc_done);
    }
  } else {
    const int quarter = warp & 3;
    const int chalf = (warp - 2) >> 2;  // columns [64*chalf, 64*chalf + 64)
    const int ctid = threadIdx.x - 64;
    const int kr = k0 + quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const float LOG2E = 1.4426950408889634f;
    const float sl2 = p.scale * LOG2E;
    auto fetch = [&](int it, float& f, int& i) {
      const int head = hk * G + it / nq;
      const int t = (qb_lo + it % nq) * B3_T + (ctid & 127);
      if (ctid < 128) {
        f = t < p.T ? p.lse[(long long)head * p.T + t] * LOG2E : 0.f;
        i = t < p.T ? p.doc_start[t] : 0x7fffffff;
      } else {
        f = t < p.T ? p.delta[(long long)head * p.T + t] : 0.f;
        i = 0;
      }
    };
    auto publish = [&](int buf, float f, int i) {
      float* b = scal_f + buf * 384;
      b[ctid] = f;  // [0,128): lse*log2e, [128,256): delta
      if (ctid < 128) reinterpret_cast<int*>(b)[256 + ctid] = i;
    };
    float nf;
    int ni;
    fetch(0, nf, ni);
    publish(0, nf, ni);
    b3_compute_sync();
    bool ok = true;
    const int c0 = chalf * 64;
    for (int it = 0; it < niter; ++it) {
      const bool more = it + 1 < niter;
      if (more) fetch(it + 1, nf, ni);
      const float* b = scal_f + (it & 1) * 384;
      const int* bi = reinterpret_cast<const int*>(b) + 256;
      const int q0 = (qb_lo + it % nq) * B3_T;
      const bool need_mask = !(q0 >= k0 + B3_T - 1 && bi[127] <= k0);
      uint32_t pk[32];
      // ---- stage A: P^T from S^T
      if (ok && !mbar_wait(bar_s_full, it & 1, p.status, kTimeoutEpilogue)) ok = false;
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t rs[32];
          tmem_ld_32x32(tS + lane_addr + c0 + c * 32, rs);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const int col = c0 + c * 32 + i;
            const float4 l4 = *reinterpret_cast<const float4*>(b + col);
            float pv[4];
            pv[0] = fast_exp2(__uint_as_float(rs[i]) * sl2 - l4.x);
            pv[1] = fast_exp2(__uint_as_float(rs[i + 1]) * sl2 - l4.y);
            pv[2] = fast_exp2(__uint_as_float(rs[i + 2]) * sl2 - l4.z);
            pv[3] = fast_exp2(__uint_as_float(rs[i + 3]) * sl2 - l4.w);
            if (need_mask) {
              const int4 s4 = *reinterpret_cast<const int4*>(bi + col);
              const int t = q0 + col;
              if (!(kr >= s4.x && kr <= t)) pv[0] = 0.f;
              if (!(kr >= s4.y && kr <= t + 1)) pv[1] = 0.f;
              if (!(kr >= s4.z && kr <= t + 2)) pv[2] = 0.f;
              if (!(kr >= s4.w && kr <= t + 3)) pv[3] = 0.f;
            }
            pk[c * 16 + i / 2] = b3_pack2(pv[0], pv[1], FMT);
            pk[c * 16 + i / 2 + 1] = b3_pack2(pv[2], pv[3], FMT);
          }
        }
        tmem_st_32x32(tS + lane_addr + c0, pk);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_pa_full);
      }
      // ---- stage B: dS^T = P^T o (dP^T - delta)
      if (ok && !mbar_wait(bar_dp_full, it & 1, p.status, kTimeoutEpilogue)) ok = false;
      if (ok) {
        tc_fence_after();
        uint32_t dk[32];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t rp[32];
          tmem_ld_32x32(tdP + lane_addr + c0 + c * 32, rp);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float4 d4 = *reinterpret_cast<const float4*>(b + 128 + c0 + c * 32 + i);
            float p0, p1, p2, p3;
            b3_unpack2(pk[c * 16 + i / 2], FMT, p0, p1);
            b3_unpack2(pk[c * 16 + i / 2 + 1], FMT, p2, p3);
            dk[c * 16 + i / 2] = b3_pack2(p0 * (__uint_as_float(rp[i]) - d4.x), p1 * (__uint_as_float(rp[i + 1]) - d4.y), FMT);
            dk[c * 16 + i / 2 + 1] =
                b3_pack2(p2 * (__uint_as_float(rp[i + 2]) - d4.z), p3 * (__uint_as_float(rp[i + 3]) - d4.w), FMT);
          }
        }
        tmem_st_32x32(tdP + lane_addr + c0, dk);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_pb_full);
      }
      if (more) publish((it + 1) & 1, nf, ni);
      b3_compute_sync();
    }
    if (ok && mbar_wait(bar_acc_done, 0, p.status, kTimeoutEpilogue)) {
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < D / 64; ++c) {
        const int col = chalf * (D / 2) + c * 32;
        uint32_t r[32];
        tmem_ld_32x32(tdV + lane_addr + col, r);
        tmem_ld_wait();
        if (kr < p.T)
          b3_store_row_chunk(reinterpret_cast<uint16_t*>(p.dv) + (long long)kr * p.lddv + hk * D + col, r, 1.f, FMT);
        tmem_ld_32x32(tdK + lane_addr + col, r);
        tmem_ld_wait();
        if (kr < p.T)
          b3_store_row_chunk(reinterpret_cast<uint16_t*>(p.dk) + (long long)kr * p.lddk + hk * D + col, r, p.scale,
                             FMT);
      }
    }
  }
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ----------------------------------------------------------------------------------------
// dQ[q tile, head] = scale * sum_j dS_j K_j
// ----------------------------------------------------------------------------------------
template <int D, int FMT>
__global__ void __launch_bounds__(320, 1)
attn_bwd_dq3_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                    const AttnBwd3Params p) {
  using Cfg = AttnBwd3Cfg<D>;
  constexpr int NH = D / 64;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = base;
  const uint32_t sdO = base + Cfg::kTileBytes;
  auto sK = [&](int s) { return base + Cfg::kTileBytes * (2 + 2 * s); };
  auto sV = [&](int s) { return base + Cfg::kTileBytes * (3 + 2 * s); };
  const uint32_t bars = base + Cfg::kTileBytes * 6 + Cfg::kScalarBytes;
  const uint32_t bar_q = bars;
  auto bar_kv_full = [&](int s) { return bars + 8u * (1 + s); };
  auto bar_kv_empty = [&](int s) { return bars + 8u * (3 + s); };
  const uint32_t bar_s_full = bars + 8u * 5, bar_dp_full = bars + 8u * 6;
  const uint32_t bar_sa_done = bars + 8u * 7, bar_pb_full = bars + 8u * 8;
  const uint32_t bar_acc_done = bars + 8u * 9, bar_qtm_full = bars + 8u * 10;
  const uint32_t holder = bars + 8u * 11;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;  // long tiles (late in their document) first
  const int head = blockIdx.y;
  const int hk = head / (p.nh / p.nkv);
  const int q0 = qt * B3_T;
  const int q_last = min(q0 + B3_T - 1, p.T - 1);
  const int ds_last = p.doc_start[q_last];
  const int kb_lo = p.doc_start[q0] / B3_T;
  const int nblk = q_last / B3_T - kb_lo + 1;

  if (warp == 1 && lane == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_kv_full(s), 1);
      mbar_init(bar_kv_empty(s), 1);
    }
    mbar_init(bar_s_full, 1);
    mbar_init(bar_dp_full, 1);
    mbar_init(bar_sa_done, 8);
    mbar_init(bar_pb_full, 8);
    mbar_init(bar_acc_done, 1);
    mbar_init(bar_qtm_full, 8);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(holder, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem) : "r"(holder));
  const uint32_t tQ = tmem, tdO = tmem + D / 2, tS = tmem + D, tdP = tmem + D + 128u, tdQ = tmem + D + 256u;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(bar_q, 2 * Cfg::kTileBytes);
#pragma unroll
      for (int h = 0; h < NH; ++h) {
        tma_load_2d(sQ + h * Cfg::kHalfBytes, &tmQ, bar_q, head * D + 64 * h, q0);
        tma_load_2d(sdO + h * Cfg::kHalfBytes, &tmdO, bar_q, head * D + 64 * h, q0);
      }
      for (int j = 0; j < nblk; ++j) {
        const int s = j & 1;
        if (!mbar_wait(bar_kv_empty(s), ((j >> 1) & 1) ^ 1u, p.status, kTimeoutProducer)) break;
        const int k0 = (kb_lo + j) * B3_T;
        mbar_expect_tx(bar_kv_full(s), 2 * Cfg::kTileBytes);
#pragma unroll
        for (int h = 0; h < NH; ++h) {
          tma_load_2d(sK(s) + h * Cfg::kHalfBytes, &tmK, bar_kv_full(s), hk * D + 64 * h, k0);
          tma_load_2d(sV(s) + h * Cfg::kHalfBytes, &tmV, bar_kv_full(s), hk * D + 64 * h, k0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_f16(128, 128, FMT, 0, 0);
      const uint32_t idesc_g = make_idesc_f16(128, D, FMT, 0, 1);
      auto issue_scores = [&](uint32_t acc, uint32_t a_tmem, uint32_t b_tile, uint32_t bar) {  // acc = A[tmem] . B^T
        const SmemDescBase b = make_smem_desc_base(b_tile, 16, 1024);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks / 4) * Cfg::kHalfBytes + (ks % 4) * 32;
          tc_mma_f16_ts(acc, a_tmem + ks * 8, smem_desc_at(b, off), idesc_s, ks != 0 ? 1u : 0u);
        }
        tc_commit(bar);
      };
      auto issue_dq = [&](int s, bool first) {  // dQ += dS K
        const SmemDescBase b = make_smem_desc_base(sK(s), Cfg::kHalfBytes, 1024);
        tc_mma_f16_ts(tdQ, tdP + b3_pcol(0), smem_desc_at(b, 0), idesc_g, first ? 0u : 1u);
#pragma unroll
        for (int ks = 1; ks < 8; ++ks) tc_mma_f16_ts(tdQ, tdP + b3_pcol(ks), smem_desc_at(b, ks * 2048), idesc_g, 1u);
      };
      const bool tr = blockIdx.x == gridDim.x / 2 && blockIdx.y == 0;
      FMSB_TRACE3(tr, 4000);
      bool ok = mbar_wait(bar_qtm_full, 0, p.status, kTimeoutMma);
      FMSB_TRACE3(tr, 4001);
      if (ok) ok = mbar_wait(bar_kv_full(0), 0, p.status, kTimeoutMma);
      if (ok) {
        tc_fence_after();
        issue_scores(tS, tQ, sK(0), bar_s_full);
        issue_scores(tdP, tdO, sV(0), bar_dp_full);
      }
      FMSB_TRACE3(tr, 4002);
      for (int j = 0; j < nblk && ok; ++j) {
        const int s = j & 1;
        const bool more = j + 1 < nblk;
        FMSB_TRACE3(tr, 4096 + 8 * j + 0);
        if (more) {
          // S(j) is in the compute warps' registers: S(j+1) may overwrite it while they work
          if (!mbar_wait(bar_sa_done, j & 1, p.status, kTimeoutMma)) { ok = false; break; }
          if (!mbar_wait(bar_kv_full(s ^ 1), ((j + 1) >> 1) & 1, p.status, kTimeoutMma)) { ok = false; break; }
          tc_fence_after();
          FMSB_TRACE3(tr, 4096 + 8 * j + 1);
          issue_scores(tS, tQ, sK(s ^ 1), bar_s_full);
          FMSB_TRACE3(tr, 4096 + 8 * j + 2);
        }
        if (!mbar_wait(bar_pb_full, j & 1, p.status, kTimeoutMma)) { ok = false; break; }
        tc_fence_after();
        FMSB_TRACE3(tr, 4096 + 8 * j + 3);
        issue_dq(s, j == 0);
        tc_commit(bar_kv_empty(s));
        FMSB_TRACE3(tr, 4096 + 8 * j + 4);
        if (more) issue_scores(tdP, tdO, sV(s ^ 1), bar_dp_full);
        FMSB_TRACE3(tr, 4096 + 8 * j + 5);
      }
      if (ok) tc_commit(bar_acc_done);
      FMSB_TRACE3(tr, 4003);
    }
  } else {
    const int quarter = warp & 3;
    const int chalf = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    const int t = q0 + row;
    const bool row_ok = t < p.T;
    const int ds = row_ok ? p.doc_start[t] : 0;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const float LOG2E = 1.4426950408889634f;
    const float sl2 = p.scale * LOG2E;
    const float lse2 = row_ok ? p.lse[(long long)head * p.T + t] * LOG2E : 0.f;
    const float dlt = row_ok ? p.delta[(long long)head * p.T + t] : 0.f;
    const int c0 = chalf * 64;
    const bool trc = blockIdx.x == gridDim.x / 2 && blockIdx.y == 0 && threadIdx.x == 64;
    FMSB_TRACE3(trc, 10);
    bool ok = mbar_wait(bar_q, 0, p.status, kTimeoutEpilogue);
    FMSB_TRACE3(trc, 11);
    // ---- Q and dO rows into tensor memory as packed 16-bit A operands (row = lane)
    if (ok) {
#pragma unroll
      for (int m = 0; m < 2; ++m) {
        const uint32_t src = (m == 0 ? sQ : sdO);
        const uint32_t dst = (m == 0 ? tQ : tdO);
        if constexpr (D == 128) {
          uint32_t w[32];
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) {
            const uint32_t addr = src + chalf * Cfg::kHalfBytes + static_cast<uint32_t>(row * 128 + ((ch ^ (row & 7)) << 4));
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(w[ch * 4]), "=r"(w[ch * 4 + 1]), "=r"(w[ch * 4 + 2]), "=r"(w[ch * 4 + 3])
                         : "r"(addr));
          }
          tmem_st_32x32(dst + lane_addr + chalf * 32, w);
        } else {
          uint32_t w[16];
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) {
            const int ch = chalf * 4 + c4;
            const uint32_t addr = src + static_cast<uint32_t>(row * 128 + ((ch ^ (row & 7)) << 4));
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(w[c4 * 4]), "=r"(w[c4 * 4 + 1]), "=r"(w[c4 * 4 + 2]), "=r"(w[c4 * 4 + 3])
                         : "r"(addr));
          }
          tmem_st_32x16(dst + lane_addr + chalf * 16, w);
        }
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_qtm_full);
    }
    FMSB_TRACE3(trc, 12);
    for (int j = 0; j < nblk && ok; ++j) {
      const int k0 = (kb_lo + j) * B3_T;
      const bool need_mask = !(q0 >= k0 + B3_T - 1 && ds_last <= k0) || !row_ok;
      FMSB_TRACE3(trc, 64 + 8 * j + 0);
      if (!mbar_wait(bar_s_full, j & 1, p.status, kTimeoutEpilogue)) { ok = false; break; }
      tc_fence_after();
      FMSB_TRACE3(trc, 64 + 8 * j + 1);
      uint32_t pk[32];
      {
        uint32_t rs0[32], rs1[32];
        tmem_ld_32x32(tS + lane_addr + c0, rs0);
        tmem_ld_32x32(tS + lane_addr + c0 + 32, rs1);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_sa_done);
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = fast_exp2(__uint_as_float(rs0[i]) * sl2 - lse2);
          float p1 = fast_exp2(__uint_as_float(rs0[i + 1]) * sl2 - lse2);
          float p2 = fast_exp2(__uint_as_float(rs1[i]) * sl2 - lse2);
          float p3 = fast_exp2(__uint_as_float(rs1[i + 1]) * sl2 - lse2);
          if (need_mask) {
            const int kk = k0 + c0 + i;
            if (!(row_ok && kk >= ds && kk <= t)) p0 = 0.f;
            if (!(row_ok && kk + 1 >= ds && kk + 1 <= t)) p1 = 0.f;
            if (!(row_ok && kk + 32 >= ds && kk + 32 <= t)) p2 = 0.f;
            if (!(row_ok && kk + 33 >= ds && kk + 33 <= t)) p3 = 0.f;
          }
          pk[i / 2] = b3_pack2(p0, p1, FMT);
          pk[16 + i / 2] = b3_pack2(p2, p3, FMT);
        }
      }
      FMSB_TRACE3(trc, 64 + 8 * j + 2);
      if (!mbar_wait(bar_dp_full, j & 1, p.status, kTimeoutEpilogue)) { ok = false; break; }
      tc_fence_after();
      FMSB_TRACE3(trc, 64 + 8 * j + 3);
      uint32_t dk[32];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t rp[32];
        tmem_ld_32x32(tdP + lane_addr + c0 + c * 32, rp);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0, p1;
          b3_unpack2(pk[c * 16 + i / 2], FMT, p0, p1);
          dk[c * 16 + i / 2] = b3_pack2(p0 * (__uint_as_float(rp[i]) - dlt), p1 * (__uint_as_float(rp[i + 1]) - dlt), FMT);
        }
      }
      tmem_st_32x32(tdP + lane_addr + c0, dk);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pb_full);
      FMSB_TRACE3(trc, 64 + 8 * j + 4);
    }
    FMSB_TRACE3(trc, 13);
    if (ok && mbar_wait(bar_acc_done, 0, p.status, kTimeoutEpilogue)) {
      tc_fence_after();
      FMSB_TRACE3(trc, 14);
#pragma unroll 1
      for (int c = 0; c < D / 64; ++c) {
        const int col = chalf * (D / 2) + c * 32;
        uint32_t r[32];
        tmem_ld_32x32(tdQ + lane_addr + col, r);
        tmem_ld_wait();
        if (row_ok)
          b3_store_row_chunk(reinterpret_cast<uint16_t*>(p.dq) + (long long)t * p.lddq + head * D + col, r, p.scale,
                             FMT);
      }
    }
  }
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace fmsb

using namespace fmsb;

#ifdef FMSB_TRACE
extern "C" int fmsb_attn_trace3_read(long long* host, int n) {
  if (n > 8192) n = 8192;
  return (int)cudaMemcpyFromSymbol(host, fmsb::g_trace3, sizeof(long long) * n);
}
#endif

static int b3_make_maps(CUtensorMap* tq, CUtensorMap* tk, CUtensorMap* tv, CUtensorMap* tdo, const void* q,
                        long long ldq, const void* k, long long ldk, const void* v, long long ldv, const void* dout,
                        long long lddo, int T, int nh, int nkv, int d) {
  using namespace fmsb_host;
  int rc;
  if ((rc = make_tmap_2d_16b(tq, q, T, (uint64_t)nh * d, ldq, 128, 64))) return rc;
  if ((rc = make_tmap_2d_16b(tk, k, T, (uint64_t)nkv * d, ldk, 128, 64))) return rc;
  if ((rc = make_tmap_2d_16b(tv, v, T, (uint64_t)nkv * d, ldv, 128, 64))) return rc;
  if ((rc = make_tmap_2d_16b(tdo, dout, T, (uint64_t)nh * d, lddo, 128, 64))) return rc;
  return 0;
}

template <typename K>
static int b3_set_smem(K kern, int bytes) {
  return (int)cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

extern "C" int fmsb_attn_bwd_dq3(const void* q, long long ldq, const void* k, long long ldk, const void* v,
                                 long long ldv, const void* dout, long long lddo, void* dq, long long lddq,
                                 const float* lse, const float* delta, const int* doc_start, const int* doc_end,
                                 int T, int nh, int nkv, int d, float scale, int fmt, int* status,
                                 cudaStream_t stream) {
  if (T <= 0) return 0;
  if (!(d == 64 || d == 128) || nh % nkv != 0) return -2;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (lddo % 8) || (lddq % 8)) return -2;
  CUtensorMap tq, tk, tv, tdo;
  int rc = b3_make_maps(&tq, &tk, &tv, &tdo, q, ldq, k, ldk, v, ldv, dout, lddo, T, nh, nkv, d);
  if (rc) return rc;
  AttnBwd3Params p{};
  p.T = T; p.nh = nh; p.nkv = nkv; p.d = d; p.scale = scale;
  p.doc_start = doc_start; p.doc_end = doc_end; p.lse = lse; p.delta = delta;
  p.dq = dq; p.lddq = lddq; p.fmt = fmt; p.status = status;
  dim3 grid((T + B3_T - 1) / B3_T, nh);
#define FMSB_B3(DD, FF)                                                                                          \
  do {                                                                                                           \
    static bool cfg = false;                                                                                     \
    if (!cfg) {                                                                                                  \
      if ((rc = b3_set_smem(attn_bwd_dq3_kernel<DD, FF>, AttnBwd3Cfg<DD>::kSmemBytes))) return rc;             \
      cfg = true;                                                                                                \
    }                                                                                                            \
    attn_bwd_dq3_kernel<DD, FF><<<grid, 320, AttnBwd3Cfg<DD>::kSmemBytes, stream>>>(tq, tk, tv, tdo, p);       \
  } while (0)
  if (d == 128 && fmt == 1) FMSB_B3(128, 1);
  else if (d == 128) FMSB_B3(128, 0);
  else if (fmt == 1) FMSB_B3(64, 1);
  else FMSB_B3(64, 0);
#undef FMSB_B3
  return (int)cudaGetLastError();
}

extern "C" int fmsb_attn_bwd_dkv3(const void* q, long long ldq, const void* k, long long ldk, const void* v,
                                  long long ldv, const void* dout, long long lddo, void* dk, long long lddk, void* dv,
                                  long long lddv, const float* lse, const float* delta, const int* doc_start,
                                  const int* doc_end, int T, int nh, int nkv, int d, float scale, int fmt,
                                  int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (!(d == 64 || d == 128) || nh % nkv != 0) return -2;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (lddo % 8) || (lddk % 8) || (lddv % 8)) return -2;
  CUtensorMap tq, tk, tv, tdo;
  int rc = b3_make_maps(&tq, &tk, &tv, &tdo, q, ldq, k, ldk, v, ldv, dout, lddo, T, nh, nkv, d);
  if (rc) return rc;
  AttnBwd3Params p{};
  p.T = T; p.nh = nh; p.nkv = nkv; p.d = d; p.scale = scale;
  p.doc_start = doc_start; p.doc_end = doc_end; p.lse = lse; p.delta = delta;
  p.dk = dk; p.lddk = lddk; p.dv = dv; p.lddv = lddv; p.fmt = fmt; p.status = status;
  dim3 grid((T + B3_T - 1) / B3_T, nkv);
#define FMSB_B3(DD, FF)                                                                                          \
  do {                                                                                                           \
    static bool cfg = false;                                                                                     \
    if (!cfg) {                                                                                                  \
      if ((rc = b3_set_smem(attn_bwd_dkv3_kernel<DD, FF>, AttnBwd3Cfg<DD>::kSmemBytes))) return rc;             \
      cfg = true;                                                                                                \
    }                                                                                                            \
    attn_bwd_dkv3_kernel<DD, FF><<<grid, 320, AttnBwd3Cfg<DD>::kSmemBytes, stream>>>(tq, tk, tv, tdo, p);       \
  } while (0)
  if (d == 128 && fmt == 1) FMSB_B3(128, 1);
  else if (d == 128) FMSB_B3(128, 0);
  else if (fmt == 1) FMSB_B3(64, 1);
  else FMSB_B3(64, 0);
#undef FMSB_B3
  return (int)cudaGetLastError();
}
