// Padding-free (varlen) causal flash attention for sm_100a on tcgen05 tensor cores.
//
// Replaces flash_attn_varlen_func as used by the reference's padding-free plugin
// (fms_acceleration_aadp/flash_attn.py:108-199: cu_seqlens derived from position_ids == 0,
// causal, grouped-query heads).  Tokens of all documents are packed along one axis; row t of
// document [start, end) attends to keys start..t.  The document structure is given as two
// int32 arrays over tokens: doc_start[t] and doc_end[t].
//
// Layout: q [T, nh*d], k/v [T, nkv*d] (any row stride, e.g. slices of one packed qkv buffer),
// o [T, nh*d], lse [nh, T] fp32 (natural log).  d in {64, 128}.
//
// This file holds the forward kernel (two query tiles per CTA, see below) and the delta = rowsum(dO*O)
// kernel; the backward kernels live in attention_bwd3.cu (in use) and attention_bwd.cu (cross-check).
#include "common.cuh"

namespace fmsb {

constexpr int ATT_BQ = 128;
constexpr int ATT_BK = 128;

struct AttnParams {
  int T, nh, nkv, d;
  float scale;           // softmax scale (1/sqrt(d))
  const int* doc_start;  // [T]
  const int* doc_end;    // [T]
  void* o;               // [T, nh*d]
  long long ldo;
  float* lse;            // [nh, T]
  int fmt;               // 0 fp16, 1 bf16
  int* status;
};

__device__ __forceinline__ uint32_t pack2(float a, float b, int fmt) {
  return fmt == 1 ? pack_bf16x2(a, b) : pack_f16x2(a, b);
}

// Byte offset of the 16-byte chunk `c16` (0..7 within a 64-element block) of row `r` inside a
// [rows x 64] 16-bit tile stored with the 128-byte swizzle.
__device__ __forceinline__ uint32_t swz_off(int r, int c16) {
  return static_cast<uint32_t>(r * 128 + ((c16 ^ (r & 7)) << 4));
}

// ----------------------------------------------------------------------------------------
// Forward, two query tiles per CTA ("ping-pong"): while the softmax warpgroup of one tile
// works, the tensor core runs the other tile's S and P.V products.  P never touches shared
// memory: each softmax thread overwrites the first 64 columns of its own S row in tensor
// memory with the 128 probabilities as packed 16-bit pairs and the P.V product reads its A
// operand from tensor memory.  The running maximum is only advanced (and O rescaled) when the
// block maximum exceeds it by more than 2^8, so most blocks skip the O round trip.
// ----------------------------------------------------------------------------------------
template <int D>
struct AttnFwd2Cfg {
  static constexpr int kTileBytes = 128 * D * 2;
  static constexpr int kHalfBytes = 128 * 64 * 2;
  static constexpr int kSmemBytes = 2 * kTileBytes /*Qa,Qb*/ + 2 * 2 * kTileBytes /*K,V x2 stages*/ + 1024 + 256;
};

template <int D, int FMT>
__global__ void __launch_bounds__(320, 1)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  using Cfg = AttnFwd2Cfg<D>;
  constexpr int NH = D / 64;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  auto sQ = [&](int x) { return base + Cfg::kTileBytes * x; };
  auto sK = [&](int s) { return base + Cfg::kTileBytes * (2 + 2 * s); };
  auto sV = [&](int s) { return base + Cfg::kTileBytes * (3 + 2 * s); };
  const uint32_t bars = base + Cfg::kTileBytes * 6;
  const uint32_t bar_q = bars;
  auto bar_kv_full = [&](int s) { return bars + 8u * (1 + s); };
  auto bar_kv_empty = [&](int s) { return bars + 8u * (3 + s); };
  auto bar_s_full = [&](int x) { return bars + 8u * (5 + x); };
  auto bar_p_full = [&](int x) { return bars + 8u * (7 + x); };
  auto bar_pv_done = [&](int x) { return bars + 8u * (9 + x); };
  const uint32_t holder = bars + 8u * 11;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;
  const int head = blockIdx.y;
  const int hk = head / (p.nh / p.nkv);
  const int q0 = qt * 256;
  // per-tile key-block ranges (tile 1 may lie completely beyond T)
  int blk_lo[2], blk_hi[2], ds_last_t[2];
  bool exists[2];
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    const int qs = q0 + 128 * x;
    exists[x] = qs < p.T;
    const int ql = min(qs + 127, p.T - 1);
    blk_lo[x] = exists[x] ? p.doc_start[qs] / ATT_BK : 0;
    blk_hi[x] = exists[x] ? ql / ATT_BK : -1;
    ds_last_t[x] = exists[x] ? p.doc_start[ql] : 0;
  }
  const int kb_lo = blk_lo[0];
  const int kb_hi = exists[1] ? blk_hi[1] : blk_hi[0];
  const int nblk = kb_hi - kb_lo + 1;
  auto active = [&](int x, int j) { const int kb = kb_lo + j; return exists[x] && kb >= blk_lo[x] && kb <= blk_hi[x]; };

  if (warp == 1 && lane == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_kv_full(s), 1);
      mbar_init(bar_kv_empty(s), 1);
      mbar_init(bar_s_full(s), 1);
      mbar_init(bar_p_full(s), 128);
      mbar_init(bar_pv_done(s), 1);
    }
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
  auto tS = [&](int x) { return tmem + 128u * x; };
  auto tO = [&](int x) { return tmem + 256u + 128u * x; };

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(bar_q, (exists[1] ? 2 : 1) * Cfg::kTileBytes);
      for (int x = 0; x < 2; ++x) {
        if (!exists[x]) continue;
#pragma unroll
        for (int h = 0; h < NH; ++h)
          tma_load_2d(sQ(x) + h * Cfg::kHalfBytes, &tmQ, bar_q, head * D + 64 * h, q0 + 128 * x);
      }
      for (int j = 0; j < nblk; ++j) {
        const int s = j & 1;
        if (!mbar_wait(bar_kv_empty(s), ((j >> 1) & 1) ^ 1u, p.status, kTimeoutProducer)) break;
        mbar_expect_tx(bar_kv_full(s), 2 * Cfg::kTileBytes);
        const int k0 = (kb_lo + j) * ATT_BK;
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
      const uint32_t idesc_o = make_idesc_f16(128, D, FMT, 0, 1);
      auto issue_s = [&](int x, int j) {
        const int s = j & 1;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks / 4) * Cfg::kHalfBytes + (ks % 4) * 32;
          tc_mma_f16(tS(x), make_smem_desc(sQ(x) + off, 16, 1024), make_smem_desc(sK(s) + off, 16, 1024), idesc_s,
                     ks != 0);
        }
        tc_commit(bar_s_full(x));
      };
      int cnt[2] = {0, 0};  // active blocks issued so far per tile
      bool ok = mbar_wait(bar_q, 0, p.status, kTimeoutMma);
      if (ok) ok = mbar_wait(bar_kv_full(0), 0, p.status, kTimeoutMma);
      if (ok) {
        tc_fence_after();
        for (int x = 0; x < 2; ++x)
          if (active(x, 0)) issue_s(x, 0);
      }
      for (int j = 0; j < nblk && ok; ++j) {
        const int s = j & 1;
        bool next_ready = false;
        for (int x = 0; x < 2 && ok; ++x) {
          if (active(x, j)) {
            if (!mbar_wait(bar_p_full(x), cnt[x] & 1, p.status, kTimeoutMma)) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < ATT_BK / 16; ++ks) {
              const uint64_t bdesc = make_smem_desc(sV(s) + ks * 2048, Cfg::kHalfBytes, 1024);
              tc_mma_f16_ts(tO(x), tS(x) + ks * 8, bdesc, idesc_o, (cnt[x] | ks) != 0);
            }
            tc_commit(bar_pv_done(x));
            cnt[x] += 1;
          }
          if (j + 1 < nblk && active(x, j + 1)) {
            if (!next_ready) {
              const int jn = j + 1;
              if (!mbar_wait(bar_kv_full(jn & 1), (jn >> 1) & 1, p.status, kTimeoutMma)) { ok = false; break; }
              tc_fence_after();
              next_ready = true;
            }
            issue_s(x, j + 1);
          }
        }
        if (ok) tc_commit(bar_kv_empty(s));
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax warpgroups
    const int x = (warp - 2) >> 2;  // tile handled by this warpgroup
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int t = q0 + 128 * x + row;
    const bool row_ok = t < p.T;
    const int ds = row_ok ? p.doc_start[t] : 0;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    const float sl2 = p.scale * 1.4426950408889634f;
    const int qs = q0 + 128 * x;
    float m_used = -1e30f, l_run = 0.f;
    int cnt = 0;
    bool ok = true;
    if (exists[x]) {
      for (int j = 0; j < nblk; ++j) {
        if (!active(x, j)) continue;
        const int k0 = (kb_lo + j) * ATT_BK;
        if (!mbar_wait(bar_s_full(x), cnt & 1, p.status, kTimeoutEpilogue)) { ok = false; break; }
        tc_fence_after();
        const bool need_mask = !(k0 >= ds_last_t[x] && k0 + ATT_BK - 1 <= qs) || !row_ok;
        float sv[128];
        {
          uint32_t r[32];
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            tmem_ld_32x32(tS(x) + lane_addr + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) sv[c * 32 + i] = __uint_as_float(r[i]);
          }
        }
        float m_blk = -1e30f;
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 128; ++i) {
            const int kk = k0 + i;
            if (!(row_ok && kk >= ds && kk <= t)) sv[i] = -1e30f;
            m_blk = fmaxf(m_blk, sv[i]);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 128; ++i) m_blk = fmaxf(m_blk, sv[i]);
        }
        // advance the reference maximum only when it is exceeded by more than 2^8
        float alpha = 1.f;
        const bool bump = (m_blk - m_used) * sl2 > 8.f || cnt == 0;
        if (bump) {
          const float m_new = fmaxf(m_used, m_blk);
          alpha = fast_exp2((m_used - m_new) * sl2);
          m_used = m_new;
        }
        const float mb = m_used * sl2;
        float l_blk = 0.f;
        uint32_t packed[64];
#pragma unroll
        for (int i = 0; i < 128; i += 2) {
          const float p0 = sv[i] <= -1e30f ? 0.f : fast_exp2(sv[i] * sl2 - mb);
          const float p1 = sv[i + 1] <= -1e30f ? 0.f : fast_exp2(sv[i + 1] * sl2 - mb);
          l_blk += p0 + p1;
          packed[i / 2] = pack2(p0, p1, FMT);
        }
        l_run = l_run * alpha + l_blk;
        // P (16-bit pairs) over the first 64 columns of this thread's own S row
        {
          uint32_t r[32];
#pragma unroll
          for (int c = 0; c < 2; ++c) {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = packed[c * 32 + i];
            tmem_st_32x32(tS(x) + lane_addr + c * 32, r);
          }
        }
        if (cnt > 0 && __any_sync(0xffffffffu, bump)) {
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(tO(x) + lane_addr + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st_32x32(tO(x) + lane_addr + c * 32, r);
          }
        }
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(bar_p_full(x));
        cnt += 1;
      }
      if (ok && cnt > 0 && mbar_wait(bar_pv_done(x), (cnt - 1) & 1, p.status, kTimeoutEpilogue)) {
        tc_fence_after();
        const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(tO(x) + lane_addr + c * 32, r);
          tmem_ld_wait();
          if (row_ok) {
            uint16_t* orow = reinterpret_cast<uint16_t*>(p.o) + (long long)t * p.ldo + head * D + c * 32;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 u;
              u.x = pack2(__uint_as_float(r[i]) * inv_l, __uint_as_float(r[i + 1]) * inv_l, FMT);
              u.y = pack2(__uint_as_float(r[i + 2]) * inv_l, __uint_as_float(r[i + 3]) * inv_l, FMT);
              u.z = pack2(__uint_as_float(r[i + 4]) * inv_l, __uint_as_float(r[i + 5]) * inv_l, FMT);
              u.w = pack2(__uint_as_float(r[i + 6]) * inv_l, __uint_as_float(r[i + 7]) * inv_l, FMT);
              *reinterpret_cast<uint4*>(orow + i) = u;
            }
          }
        }
        if (row_ok) p.lse[(long long)head * p.T + t] = m_used * p.scale + __logf(l_run);
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

// delta[h, t] = sum_d dO[t, h, d] * O[t, h, d].  LPI = d / 8 lanes share one (token, head): each loads 16 bytes of O
// and of dO, the partial dots meet by shuffle.  (With 4-byte loads, one warp per item, the kernel ran at a third of the
// copy bandwidth.)
template <typename T, int LPI>
__global__ void __launch_bounds__(256)
attn_delta_vec_kernel(const T* __restrict__ o, const T* __restrict__ dout, long long ldo, long long lddo,
                      float* __restrict__ delta, int T_tokens, int nh) {
  constexpr int D = LPI * 8;
  const long long items = (long long)T_tokens * nh;
  const int sub = threadIdx.x % LPI;
  // the loop bound is the same for all lanes of a warp (the shuffles below need every lane); lanes whose item lies
  // beyond the end work on zeros
  for (long long item0 = (blockIdx.x * (long long)blockDim.x + (threadIdx.x & ~31)) / LPI; item0 < items;
       item0 += (long long)gridDim.x * blockDim.x / LPI) {
    const long long item = item0 + (threadIdx.x & 31) / LPI;
    const bool valid = item < items;
    const int t = valid ? (int)(item / nh) : 0, h = valid ? (int)(item - (long long)t * nh) : 0;
    uint4 a = make_uint4(0u, 0u, 0u, 0u), b = a;
    if (valid) {
      a = *reinterpret_cast<const uint4*>(o + (long long)t * ldo + h * D + sub * 8);
      b = *reinterpret_cast<const uint4*>(dout + (long long)t * lddo + h * D + sub * 8);
    }
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 x, y;
      if (std::is_same<T, __nv_bfloat16>::value) {
        x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&aw[i]));
        y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&bw[i]));
      } else {
        x = __half22float2(*reinterpret_cast<const __half2*>(&aw[i]));
        y = __half22float2(*reinterpret_cast<const __half2*>(&bw[i]));
      }
      acc += x.x * y.x + x.y * y.y;
    }
#pragma unroll
    for (int off = LPI / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (sub == 0 && valid) delta[(long long)h * T_tokens + t] = acc;
  }
}

// The same with one warp per item and 4-byte loads: other head sizes and unaligned inputs.
template <typename T>
__global__ void attn_delta_kernel(const T* __restrict__ o, const T* __restrict__ dout, long long ldo, long long lddo,
                                  float* __restrict__ delta, int T_tokens, int nh, int d) {
  const int warps_per_block = blockDim.x >> 5;
  const long long item = (long long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  if (item >= (long long)T_tokens * nh) return;
  const int t = (int)(item / nh), h = (int)(item % nh);
  const int lane = threadIdx.x & 31;
  float acc = 0.f;
  for (int i = lane * 2; i < d; i += 64) {
    const T* po = o + (long long)t * ldo + h * d + i;
    const T* pd = dout + (long long)t * lddo + h * d + i;
    float a0, a1, b0, b1;
    if (sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value) {
      float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(po));
      float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(pd));
      a0 = a.x; a1 = a.y; b0 = b.x; b1 = b.y;
    } else {
      float2 a = __half22float2(*reinterpret_cast<const __half2*>(po));
      float2 b = __half22float2(*reinterpret_cast<const __half2*>(pd));
      a0 = a.x; a1 = a.y; b0 = b.x; b1 = b.y;
    }
    acc += a0 * b0 + a1 * b1;
  }
  acc = warp_sum(acc);
  if (lane == 0) delta[(long long)h * T_tokens + t] = acc;
}

}  // namespace fmsb

using namespace fmsb;

namespace fmsb_host {
int sm_count();
}

extern "C" int fmsb_attn_fwd(const void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv,
                             void* o, long long ldo, float* lse, const int* doc_start, const int* doc_end, int T,
                             int nh, int nkv, int d, float scale, int fmt, int* status, cudaStream_t stream) {
  using namespace fmsb_host;
  if (T <= 0) return 0;
  if (!(d == 64 || d == 128) || nh % nkv != 0) return -2;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (ldo % 8)) return -2;
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_tmap_2d_16b(&tq, q, T, (uint64_t)nh * d, ldq, 128, 64))) return rc;
  if ((rc = make_tmap_2d_16b(&tk, k, T, (uint64_t)nkv * d, ldk, 128, 64))) return rc;
  if ((rc = make_tmap_2d_16b(&tv, v, T, (uint64_t)nkv * d, ldv, 128, 64))) return rc;
  AttnParams p;
  p.T = T; p.nh = nh; p.nkv = nkv; p.d = d; p.scale = scale;
  p.doc_start = doc_start; p.doc_end = doc_end;
  p.o = o; p.ldo = ldo; p.lse = lse; p.fmt = fmt; p.status = status;
  dim3 grid((T + 255) / 256, nh);
#define FMSB_FWD2(DD, FF)                                                                                         \
  do {                                                                                                            \
    static bool cfg = false;                                                                                      \
    if (!cfg) {                                                                                                   \
      cudaError_t e = cudaFuncSetAttribute(attn_fwd2_kernel<DD, FF>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           AttnFwd2Cfg<DD>::kSmemBytes);                                          \
      if (e != cudaSuccess) return (int)e;                                                                        \
      cfg = true;                                                                                                 \
    }                                                                                                             \
    attn_fwd2_kernel<DD, FF><<<grid, 320, AttnFwd2Cfg<DD>::kSmemBytes, stream>>>(tq, tk, tv, p);                  \
  } while (0)
  if (d == 128 && fmt == 1) FMSB_FWD2(128, 1);
  else if (d == 128) FMSB_FWD2(128, 0);
  else if (fmt == 1) FMSB_FWD2(64, 1);
  else FMSB_FWD2(64, 0);
#undef FMSB_FWD2
  return (int)cudaGetLastError();
}

extern "C" int fmsb_attn_delta(const void* o, const void* dout, long long ldo, long long lddo, float* delta, int T,
                               int nh, int d, int fmt, cudaStream_t stream) {
  if (T <= 0) return 0;
  const long long items = (long long)T * nh;
  const bool vec_ok = (d == 64 || d == 128) && ldo % 8 == 0 && lddo % 8 == 0 &&
                      (reinterpret_cast<uintptr_t>(o) & 15u) == 0 && (reinterpret_cast<uintptr_t>(dout) & 15u) == 0;
  if (vec_ok) {
    // the loop's trip counts are whole warps: items * LPI threads rounded up to CTAs of 256, at most a few waves
    const int lpi = d / 8;
    long long ctas = (items * lpi + 255) / 256;
    if (ctas > 148 * 16) ctas = 148 * 16;
#define FMSB_DELTA(TT, L)                                                                                          \
  attn_delta_vec_kernel<TT, L><<<(int)ctas, 256, 0, stream>>>((const TT*)o, (const TT*)dout, ldo, lddo, delta, T, nh)
    if (fmt == 1) { if (lpi == 16) FMSB_DELTA(__nv_bfloat16, 16); else FMSB_DELTA(__nv_bfloat16, 8); }
    else { if (lpi == 16) FMSB_DELTA(__half, 16); else FMSB_DELTA(__half, 8); }
#undef FMSB_DELTA
    return (int)cudaGetLastError();
  }
  const int wpb = 8;
  const int grid = (int)((items + wpb - 1) / wpb);
  if (fmt == 1)
    attn_delta_kernel<__nv_bfloat16><<<grid, wpb * 32, 0, stream>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout,
                                                                    ldo, lddo, delta, T, nh, d);
  else
    attn_delta_kernel<__half><<<grid, wpb * 32, 0, stream>>>((const __half*)o, (const __half*)dout, ldo, lddo, delta, T,
                                                             nh, d);
  return (int)cudaGetLastError();
}
