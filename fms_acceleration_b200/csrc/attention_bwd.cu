// Pipelined backward of the padding-free causal attention (second generation of the kernels in
// attention.cu; same interface, same mathematics, same layouts).
//
// Replaces the backward half of flash_attn_varlen_func as used by the reference's padding-free
// plugin (fms_acceleration_aadp/flash_attn.py:108-199).
//
// Both kernels keep every 128x128 score tile in tensor memory from the QK product to the last
// product that consumes it; nothing is staged through shared memory:
//
//   dK/dV kernel (fixed key tile, loop over query heads of the group and their query blocks)
//     S^T  = K Q^T          lanes = keys, columns = queries
//     dP^T = V dO^T
//     P^T  = exp2(S^T * scale*log2e - lse*log2e)        written over S^T  as packed 16-bit
//     dS^T = P^T o (dP^T - delta)                        written over dP^T as packed 16-bit
//     dV  += P^T dO , dK += dS^T Q                       A operand read from tensor memory
//   dQ kernel (fixed query tile, loop over key blocks)
//     S = Q K^T, dP = dO V^T, dS = P o (dP - delta) over dP, dQ += dS K (A from tensor memory)
//
// Each 128x128 tile is processed as two halves of 64 columns.  While the eight compute warps
// turn one half into P/dS, the tensor core runs the products of the other half, so the MMA
// issuer never waits for the exponentials in steady state:
//
//   MMA order per block i:  [S,dP](i,lo)  [acc](i-1,hi)  [S,dP](i,hi)  [acc](i,lo)
//
// Warp roles (320 threads): warp 0 TMA producer, warp 1 MMA issuer, warps 2-9 compute.  A compute
// warp owns the tensor-memory lane quarter `warp % 4` and one 32-column half of each 64-column half
// tile.  Every wait is bounded; a wait that runs out records a status code and the CTA unwinds.
#include "common.cuh"

namespace fmsb {

constexpr int B2_BQ = 128;
constexpr int B2_BK = 128;

struct AttnBwd2Params {
  int T, nh, nkv, d;
  float scale;
  const int* doc_start;
  const int* doc_end;
  const float* lse;    // [nh, T]
  const float* delta;  // [nh, T]
  void* dq;            // [T, nh*d]
  long long lddq;
  void* dk;            // [T, nkv*d]
  long long lddk;
  void* dv;
  long long lddv;
  int fmt;
  int* status;
};

template <int D>
struct AttnBwd2Cfg {
  static constexpr int kTileBytes = 128 * D * 2;
  static constexpr int kHalfBytes = 128 * 64 * 2;  // one [128 x 64] 16-bit TMA box
  static constexpr int kRowHalf = 64 * 128;        // byte offset of row 64 inside a [128 x 64] box
  // 2 fixed tiles + 2 stages x 2 streamed tiles + per-column scalars + barriers
  static constexpr int kScalarBytes = 2 * 3 * 128 * 4;
  static constexpr int kSmemBytes = 6 * kTileBytes + kScalarBytes + 1024 + 256;
};

__device__ __forceinline__ uint32_t b2_pack2(float a, float b, int fmt) {
  return fmt == 1 ? pack_bf16x2(a, b) : pack_f16x2(a, b);
}

__device__ __forceinline__ void b2_store_row_chunk(uint16_t* dst, const uint32_t (&r)[32], float mul, int fmt) {
#pragma unroll
  for (int i = 0; i < 32; i += 8) {
    uint4 u;
    u.x = b2_pack2(__uint_as_float(r[i]) * mul, __uint_as_float(r[i + 1]) * mul, fmt);
    u.y = b2_pack2(__uint_as_float(r[i + 2]) * mul, __uint_as_float(r[i + 3]) * mul, fmt);
    u.z = b2_pack2(__uint_as_float(r[i + 4]) * mul, __uint_as_float(r[i + 5]) * mul, fmt);
    u.w = b2_pack2(__uint_as_float(r[i + 6]) * mul, __uint_as_float(r[i + 7]) * mul, fmt);
    *reinterpret_cast<uint4*>(dst + i) = u;
  }
}

// Optional timeline trace (compile with -DFMSB_TRACE): CTA (0, 0) of the dK/dV kernel records clock64() at the
// hand-off points of its MMA issuer and of one compute thread; read back with fmsb_attn_trace_read.
#ifdef FMSB_TRACE
__device__ long long g_trace[8192];
#define FMSB_TRACE_AT(cond, slot) do { if ((cond) && (slot) < 8192) g_trace[(slot)] = clock64(); } while (0)
#else
#define FMSB_TRACE_AT(cond, slot) do { } while (0)
#endif

__device__ __forceinline__ void compute_bar_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// tensor-memory column of K-step `ks` (16 contraction elements = 8 columns) of a packed 16-bit
// half tile: the compute warp of columns 0-31 packs into columns 0-15, the one of columns 32-63
// into columns 32-47 (each warp only ever overwrites columns it has already read itself)
__device__ __forceinline__ uint32_t packed_col(int ks) { return static_cast<uint32_t>((ks >> 1) * 32 + (ks & 1) * 8); }

// ----------------------------------------------------------------------------------------
// dV[kv tile, kv head] = sum_{g,i} P^T dO ,  dK = scale * sum_{g,i} dS^T Q
// ----------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(320, 1)
attn_bwd_dkv2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                     const AttnBwd2Params p) {
  using Cfg = AttnBwd2Cfg<D>;
  constexpr int NH = D / 64;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sK = base;
  const uint32_t sV = base + Cfg::kTileBytes;
  auto sQ = [&](int s) { return base + Cfg::kTileBytes * (2 + 2 * s); };
  auto sdO = [&](int s) { return base + Cfg::kTileBytes * (3 + 2 * s); };
  const uint32_t scal = base + Cfg::kTileBytes * 6;  // [2 buffers][lse2 | delta | doc_start][128]
  const uint32_t bars = scal + Cfg::kScalarBytes;
  const uint32_t bar_kv = bars;
  auto bar_qdo_full = [&](int s) { return bars + 8u * (1 + s); };
  auto bar_qdo_empty = [&](int s) { return bars + 8u * (3 + s); };
  auto bar_s_full = [&](int h) { return bars + 8u * (5 + h); };
  auto bar_p_full = [&](int h) { return bars + 8u * (7 + h); };
  const uint32_t bar_acc_done = bars + 8u * 9;
  const uint32_t holder = bars + 8u * 10;
  float* scal_f = reinterpret_cast<float*>(smem_raw + (scal - smem_u32(smem_raw)));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kt = blockIdx.x;
  const int hk = blockIdx.y;
  const int G = p.nh / p.nkv;
  const int k0 = kt * B2_BK;
  const int k_last = min(k0 + B2_BK - 1, p.T - 1);
  const int de_last = p.doc_end[k_last];
  const int qb_lo = kt;  // queries before the tile cannot see its keys
  const int qb_hi = (de_last - 1) / B2_BQ;
  const int nq = qb_hi - qb_lo + 1;
  const int niter = nq * G;

  if (warp == 1 && lane == 0) {
    mbar_init(bar_kv, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_qdo_full(s), 1);
      mbar_init(bar_qdo_empty(s), 1);
      mbar_init(bar_s_full(s), 1);
      mbar_init(bar_p_full(s), 8);
    }
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
  auto tS = [&](int h) { return tmem + 64u * h; };
  auto tdP = [&](int h) { return tmem + 128u + 64u * h; };
  const uint32_t tdV = tmem + 256u, tdK = tmem + 256u + D;

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
        const int q0 = (qb_lo + it % nq) * B2_BQ;
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
      const uint32_t idesc_s = make_idesc_f16(128, 64, p.fmt, 0, 0);
      const uint32_t idesc_g = make_idesc_f16(128, D, p.fmt, 0, 1);
      const SmemDescBase dK = make_smem_desc_base(sK, 16, 1024), dV = make_smem_desc_base(sV, 16, 1024);
      // S^T and dP^T of query half `h` of the block in stage `s`
      auto issue_scores = [&](int s, int h) {
        const SmemDescBase dQ = make_smem_desc_base(sQ(s) + h * Cfg::kRowHalf, 16, 1024);
        const SmemDescBase ddO = make_smem_desc_base(sdO(s) + h * Cfg::kRowHalf, 16, 1024);
        const uint32_t ts = tS(h), tp = tdP(h);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks / 4) * Cfg::kHalfBytes + (ks % 4) * 32;
          tc_mma_f16(ts, smem_desc_at(dK, off), smem_desc_at(dQ, off), idesc_s, ks != 0);
        }
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks / 4) * Cfg::kHalfBytes + (ks % 4) * 32;
          tc_mma_f16(tp, smem_desc_at(dV, off), smem_desc_at(ddO, off), idesc_s, ks != 0);
        }
        tc_commit(bar_s_full(h));
      };
      // dV += P^T dO, dK += dS^T Q over the 64 queries of half `h` (4 steps of 16)
      auto issue_acc = [&](int s, int h, bool first) {
        const SmemDescBase bdO = make_smem_desc_base(sdO(s) + h * 4 * 2048, Cfg::kHalfBytes, 1024);
        const SmemDescBase bQ = make_smem_desc_base(sQ(s) + h * 4 * 2048, Cfg::kHalfBytes, 1024);
        const uint32_t ts = tS(h), tp = tdP(h);
        tc_mma_f16_ts(tdV, ts + packed_col(0), smem_desc_at(bdO, 0), idesc_g, first ? 0u : 1u);
#pragma unroll
        for (int ks = 1; ks < 4; ++ks) tc_mma_f16_ts(tdV, ts + packed_col(ks), smem_desc_at(bdO, ks * 2048), idesc_g, 1u);
        tc_mma_f16_ts(tdK, tp + packed_col(0), smem_desc_at(bQ, 0), idesc_g, first ? 0u : 1u);
#pragma unroll
        for (int ks = 1; ks < 4; ++ks) tc_mma_f16_ts(tdK, tp + packed_col(ks), smem_desc_at(bQ, ks * 2048), idesc_g, 1u);
      };
      bool ok = mbar_wait(bar_kv, 0, p.status, kTimeoutMma);
      const bool tr = blockIdx.x == 0 && blockIdx.y == 0;
      for (int it = 0; it < niter && ok; ++it) {
        const int s = it & 1;
        if (!mbar_wait(bar_qdo_full(s), (it >> 1) & 1, p.status, kTimeoutMma)) { ok = false; break; }
        tc_fence_after();
        FMSB_TRACE_AT(tr, 4096 + 8 * it + 0);
        issue_scores(s, 0);
        FMSB_TRACE_AT(tr, 4096 + 8 * it + 1);
        if (it > 0) {
          if (!mbar_wait(bar_p_full(1), (it - 1) & 1, p.status, kTimeoutMma)) { ok = false; break; }
          tc_fence_after();
          FMSB_TRACE_AT(tr, 4096 + 8 * it + 2);
          issue_acc((it - 1) & 1, 1, false);
          tc_commit(bar_qdo_empty((it - 1) & 1));
          FMSB_TRACE_AT(tr, 4096 + 8 * it + 3);
        }
        issue_scores(s, 1);
        FMSB_TRACE_AT(tr, 4096 + 8 * it + 4);
        if (!mbar_wait(bar_p_full(0), it & 1, p.status, kTimeoutMma)) { ok = false; break; }
        tc_fence_after();
        FMSB_TRACE_AT(tr, 4096 + 8 * it + 5);
        issue_acc(s, 0, it == 0);
        FMSB_TRACE_AT(tr, 4096 + 8 * it + 6);
      }
      if (ok && mbar_wait(bar_p_full(1), (niter - 1) & 1, p.status, kTimeoutMma)) {
        tc_fence_after();
        issue_acc((niter - 1) & 1, 1, false);
        tc_commit(bar_acc_done);
      }
    }
  } else {
    const int quarter = warp & 3;
    const int chalf = (warp - 2) >> 2;  // which 32-column half of a 64-column half tile
    const int ctid = threadIdx.x - 64;  // 0..255 among the compute threads
    const int kr = k0 + quarter * 32 + lane;  // key row of this thread (= tensor-memory lane)
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const float LOG2E = 1.4426950408889634f;
    const float sl2 = p.scale * LOG2E;
    // per-column scalars of a block: threads 0..127 fetch lse and doc_start, 128..255 fetch delta
    auto fetch = [&](int it, float& f, int& i) {
      const int head = hk * G + it / nq;
      const int t = (qb_lo + it % nq) * B2_BQ + (ctid & 127);
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
      if (ctid < 128) {
        b[ctid] = f;
        reinterpret_cast<int*>(b)[256 + ctid] = i;
      } else {
        b[ctid] = f;  // delta occupies [128, 256)
      }
    };
    float nf;
    int ni;
    fetch(0, nf, ni);
    publish(0, nf, ni);
    compute_bar_sync();
    bool ok = true;
    for (int it = 0; it < niter; ++it) {
      const bool more = it + 1 < niter;
      if (more) fetch(it + 1, nf, ni);
      const float* b = scal_f + (it & 1) * 384;
      const int* bi = reinterpret_cast<const int*>(b) + 256;
      const int q0 = (qb_lo + it % nq) * B2_BQ;
      // no masking when every query of the block sees every key of the tile
      const bool need_mask = !(q0 >= k0 + B2_BK - 1 && bi[127] <= k0);
#pragma unroll 1
      for (int h = 0; h < 2 && ok; ++h) {
        const bool tr = blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 64;
        FMSB_TRACE_AT(tr, 8 * (2 * it + h) + 0);
        if (!mbar_wait(bar_s_full(h), it & 1, p.status, kTimeoutEpilogue)) { ok = false; break; }
        tc_fence_after();
        FMSB_TRACE_AT(tr, 8 * (2 * it + h) + 1);
        const int c0 = h * 64 + chalf * 32;  // first query column of this thread's slice
        uint32_t rs[32], rp[32];
        tmem_ld_32x32(tS(h) + lane_addr + chalf * 32, rs);
        tmem_ld_32x32(tdP(h) + lane_addr + chalf * 32, rp);
        tmem_ld_wait();
        FMSB_TRACE_AT(tr, 8 * (2 * it + h) + 2);
        uint32_t pk[16], dk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 l4 = *reinterpret_cast<const float4*>(b + c0 + i);
          const float4 d4 = *reinterpret_cast<const float4*>(b + 128 + c0 + i);
          float pv[4];
          pv[0] = fast_exp2(__uint_as_float(rs[i]) * sl2 - l4.x);
          pv[1] = fast_exp2(__uint_as_float(rs[i + 1]) * sl2 - l4.y);
          pv[2] = fast_exp2(__uint_as_float(rs[i + 2]) * sl2 - l4.z);
          pv[3] = fast_exp2(__uint_as_float(rs[i + 3]) * sl2 - l4.w);
          if (need_mask) {
            const int4 s4 = *reinterpret_cast<const int4*>(bi + c0 + i);
            const int t = q0 + c0 + i;
            if (!(kr >= s4.x && kr <= t)) pv[0] = 0.f;
            if (!(kr >= s4.y && kr <= t + 1)) pv[1] = 0.f;
            if (!(kr >= s4.z && kr <= t + 2)) pv[2] = 0.f;
            if (!(kr >= s4.w && kr <= t + 3)) pv[3] = 0.f;
          }
          pk[i / 2] = b2_pack2(pv[0], pv[1], p.fmt);
          pk[i / 2 + 1] = b2_pack2(pv[2], pv[3], p.fmt);
          dk[i / 2] = b2_pack2(pv[0] * (__uint_as_float(rp[i]) - d4.x), pv[1] * (__uint_as_float(rp[i + 1]) - d4.y), p.fmt);
          dk[i / 2 + 1] =
              b2_pack2(pv[2] * (__uint_as_float(rp[i + 2]) - d4.z), pv[3] * (__uint_as_float(rp[i + 3]) - d4.w), p.fmt);
        }
        FMSB_TRACE_AT(tr, 8 * (2 * it + h) + 3);
        tmem_st_32x16(tS(h) + lane_addr + chalf * 32, pk);
        tmem_st_32x16(tdP(h) + lane_addr + chalf * 32, dk);
        tmem_st_wait();
        FMSB_TRACE_AT(tr, 8 * (2 * it + h) + 4);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_p_full(h));
        FMSB_TRACE_AT(tr, 8 * (2 * it + h) + 5);
      }
      if (more) publish((it + 1) & 1, nf, ni);
      compute_bar_sync();
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
          b2_store_row_chunk(reinterpret_cast<uint16_t*>(p.dv) + (long long)kr * p.lddv + hk * D + col, r, 1.f, p.fmt);
        tmem_ld_32x32(tdK + lane_addr + col, r);
        tmem_ld_wait();
        if (kr < p.T)
          b2_store_row_chunk(reinterpret_cast<uint16_t*>(p.dk) + (long long)kr * p.lddk + hk * D + col, r, p.scale,
                             p.fmt);
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
template <int D>
__global__ void __launch_bounds__(320, 1)
attn_bwd_dq2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                    const AttnBwd2Params p) {
  using Cfg = AttnBwd2Cfg<D>;
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
  auto bar_s_full = [&](int h) { return bars + 8u * (5 + h); };
  auto bar_p_full = [&](int h) { return bars + 8u * (7 + h); };
  const uint32_t bar_acc_done = bars + 8u * 9;
  const uint32_t holder = bars + 8u * 10;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;  // long tiles (late in their document) first
  const int head = blockIdx.y;
  const int hk = head / (p.nh / p.nkv);
  const int q0 = qt * B2_BQ;
  const int q_last = min(q0 + B2_BQ - 1, p.T - 1);
  const int ds_last = p.doc_start[q_last];
  const int kb_lo = p.doc_start[q0] / B2_BK;
  const int nblk = q_last / B2_BK - kb_lo + 1;

  if (warp == 1 && lane == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_kv_full(s), 1);
      mbar_init(bar_kv_empty(s), 1);
      mbar_init(bar_s_full(s), 1);
      mbar_init(bar_p_full(s), 8);
    }
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
  auto tS = [&](int h) { return tmem + 64u * h; };
  auto tdP = [&](int h) { return tmem + 128u + 64u * h; };
  const uint32_t tdQ = tmem + 256u;

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
        const int k0 = (kb_lo + j) * B2_BK;
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
      const uint32_t idesc_s = make_idesc_f16(128, 64, p.fmt, 0, 0);
      const uint32_t idesc_g = make_idesc_f16(128, D, p.fmt, 0, 1);
      const SmemDescBase dQd = make_smem_desc_base(sQ, 16, 1024), ddO = make_smem_desc_base(sdO, 16, 1024);
      auto issue_scores = [&](int s, int h) {
        const SmemDescBase dKh = make_smem_desc_base(sK(s) + h * Cfg::kRowHalf, 16, 1024);
        const SmemDescBase dVh = make_smem_desc_base(sV(s) + h * Cfg::kRowHalf, 16, 1024);
        const uint32_t ts = tS(h), tp = tdP(h);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks / 4) * Cfg::kHalfBytes + (ks % 4) * 32;
          tc_mma_f16(ts, smem_desc_at(dQd, off), smem_desc_at(dKh, off), idesc_s, ks != 0);
        }
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks / 4) * Cfg::kHalfBytes + (ks % 4) * 32;
          tc_mma_f16(tp, smem_desc_at(ddO, off), smem_desc_at(dVh, off), idesc_s, ks != 0);
        }
        tc_commit(bar_s_full(h));
      };
      auto issue_acc = [&](int s, int h, bool first) {
        const SmemDescBase bK = make_smem_desc_base(sK(s) + h * 4 * 2048, Cfg::kHalfBytes, 1024);
        const uint32_t tp = tdP(h);
        tc_mma_f16_ts(tdQ, tp + packed_col(0), smem_desc_at(bK, 0), idesc_g, first ? 0u : 1u);
#pragma unroll
        for (int ks = 1; ks < 4; ++ks) tc_mma_f16_ts(tdQ, tp + packed_col(ks), smem_desc_at(bK, ks * 2048), idesc_g, 1u);
      };
      bool ok = mbar_wait(bar_q, 0, p.status, kTimeoutMma);
      for (int j = 0; j < nblk && ok; ++j) {
        const int s = j & 1;
        if (!mbar_wait(bar_kv_full(s), (j >> 1) & 1, p.status, kTimeoutMma)) { ok = false; break; }
        tc_fence_after();
        issue_scores(s, 0);
        if (j > 0) {
          if (!mbar_wait(bar_p_full(1), (j - 1) & 1, p.status, kTimeoutMma)) { ok = false; break; }
          tc_fence_after();
          issue_acc((j - 1) & 1, 1, false);
          tc_commit(bar_kv_empty((j - 1) & 1));
        }
        issue_scores(s, 1);
        if (!mbar_wait(bar_p_full(0), j & 1, p.status, kTimeoutMma)) { ok = false; break; }
        tc_fence_after();
        issue_acc(s, 0, j == 0);
      }
      if (ok && mbar_wait(bar_p_full(1), (nblk - 1) & 1, p.status, kTimeoutMma)) {
        tc_fence_after();
        issue_acc((nblk - 1) & 1, 1, false);
        tc_commit(bar_acc_done);
      }
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
    bool ok = true;
    for (int j = 0; j < nblk && ok; ++j) {
      const int k0 = (kb_lo + j) * B2_BK;
      const bool need_mask = !(q0 >= k0 + B2_BK - 1 && ds_last <= k0) || !row_ok;
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        if (!mbar_wait(bar_s_full(h), j & 1, p.status, kTimeoutEpilogue)) { ok = false; break; }
        tc_fence_after();
        const int kk0 = k0 + h * 64 + chalf * 32;
        uint32_t rs[32], rp[32];
        tmem_ld_32x32(tS(h) + lane_addr + chalf * 32, rs);
        tmem_ld_32x32(tdP(h) + lane_addr + chalf * 32, rp);
        tmem_ld_wait();
        uint32_t dk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = fast_exp2(__uint_as_float(rs[i]) * sl2 - lse2);
          float p1 = fast_exp2(__uint_as_float(rs[i + 1]) * sl2 - lse2);
          if (need_mask) {
            const int kk = kk0 + i;
            if (!(row_ok && kk >= ds && kk <= t)) p0 = 0.f;
            if (!(row_ok && kk + 1 >= ds && kk + 1 <= t)) p1 = 0.f;
          }
          dk[i / 2] = b2_pack2(p0 * (__uint_as_float(rp[i]) - dlt), p1 * (__uint_as_float(rp[i + 1]) - dlt), p.fmt);
        }
        tmem_st_32x16(tdP(h) + lane_addr + chalf * 32, dk);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_p_full(h));
      }
    }
    if (ok && mbar_wait(bar_acc_done, 0, p.status, kTimeoutEpilogue)) {
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < D / 64; ++c) {
        const int col = chalf * (D / 2) + c * 32;
        uint32_t r[32];
        tmem_ld_32x32(tdQ + lane_addr + col, r);
        tmem_ld_wait();
        if (row_ok)
          b2_store_row_chunk(reinterpret_cast<uint16_t*>(p.dq) + (long long)t * p.lddq + head * D + col, r, p.scale,
                             p.fmt);
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
extern "C" int fmsb_attn_trace_read(long long* host, int n) {
  if (n > 8192) n = 8192;
  return (int)cudaMemcpyFromSymbol(host, fmsb::g_trace, sizeof(long long) * n);
}
#endif

static int b2_make_maps(CUtensorMap* tq, CUtensorMap* tk, CUtensorMap* tv, CUtensorMap* tdo, const void* q,
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
static int b2_set_smem(K kern, int bytes) {
  return (int)cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

extern "C" int fmsb_attn_bwd_dq2(const void* q, long long ldq, const void* k, long long ldk, const void* v,
                                 long long ldv, const void* dout, long long lddo, void* dq, long long lddq,
                                 const float* lse, const float* delta, const int* doc_start, const int* doc_end,
                                 int T, int nh, int nkv, int d, float scale, int fmt, int* status,
                                 cudaStream_t stream) {
  if (T <= 0) return 0;
  if (!(d == 64 || d == 128) || nh % nkv != 0) return -2;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (lddo % 8) || (lddq % 8)) return -2;
  CUtensorMap tq, tk, tv, tdo;
  int rc = b2_make_maps(&tq, &tk, &tv, &tdo, q, ldq, k, ldk, v, ldv, dout, lddo, T, nh, nkv, d);
  if (rc) return rc;
  AttnBwd2Params p{};
  p.T = T; p.nh = nh; p.nkv = nkv; p.d = d; p.scale = scale;
  p.doc_start = doc_start; p.doc_end = doc_end; p.lse = lse; p.delta = delta;
  p.dq = dq; p.lddq = lddq; p.fmt = fmt; p.status = status;
  dim3 grid((T + B2_BQ - 1) / B2_BQ, nh);
  if (d == 128) {
    static bool cfg = false;
    if (!cfg) { if ((rc = b2_set_smem(attn_bwd_dq2_kernel<128>, AttnBwd2Cfg<128>::kSmemBytes))) return rc; cfg = true; }
    attn_bwd_dq2_kernel<128><<<grid, 320, AttnBwd2Cfg<128>::kSmemBytes, stream>>>(tq, tk, tv, tdo, p);
  } else {
    static bool cfg = false;
    if (!cfg) { if ((rc = b2_set_smem(attn_bwd_dq2_kernel<64>, AttnBwd2Cfg<64>::kSmemBytes))) return rc; cfg = true; }
    attn_bwd_dq2_kernel<64><<<grid, 320, AttnBwd2Cfg<64>::kSmemBytes, stream>>>(tq, tk, tv, tdo, p);
  }
  return (int)cudaGetLastError();
}

extern "C" int fmsb_attn_bwd_dkv2(const void* q, long long ldq, const void* k, long long ldk, const void* v,
                                  long long ldv, const void* dout, long long lddo, void* dk, long long lddk, void* dv,
                                  long long lddv, const float* lse, const float* delta, const int* doc_start,
                                  const int* doc_end, int T, int nh, int nkv, int d, float scale, int fmt,
                                  int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (!(d == 64 || d == 128) || nh % nkv != 0) return -2;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (lddo % 8) || (lddk % 8) || (lddv % 8)) return -2;
  CUtensorMap tq, tk, tv, tdo;
  int rc = b2_make_maps(&tq, &tk, &tv, &tdo, q, ldq, k, ldk, v, ldv, dout, lddo, T, nh, nkv, d);
  if (rc) return rc;
  AttnBwd2Params p{};
  p.T = T; p.nh = nh; p.nkv = nkv; p.d = d; p.scale = scale;
  p.doc_start = doc_start; p.doc_end = doc_end; p.lse = lse; p.delta = delta;
  p.dk = dk; p.lddk = lddk; p.dv = dv; p.lddv = lddv; p.fmt = fmt; p.status = status;
  dim3 grid((T + B2_BK - 1) / B2_BK, nkv);
  if (d == 128) {
    static bool cfg = false;
    if (!cfg) { if ((rc = b2_set_smem(attn_bwd_dkv2_kernel<128>, AttnBwd2Cfg<128>::kSmemBytes))) return rc; cfg = true; }
    attn_bwd_dkv2_kernel<128><<<grid, 320, AttnBwd2Cfg<128>::kSmemBytes, stream>>>(tq, tk, tv, tdo, p);
  } else {
    static bool cfg = false;
    if (!cfg) { if ((rc = b2_set_smem(attn_bwd_dkv2_kernel<64>, AttnBwd2Cfg<64>::kSmemBytes))) return rc; cfg = true; }
    attn_bwd_dkv2_kernel<64><<<grid, 320, AttnBwd2Cfg<64>::kSmemBytes, stream>>>(tq, tk, tv, tdo, p);
  }
  return (int)cudaGetLastError();
}
