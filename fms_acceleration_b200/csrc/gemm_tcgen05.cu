// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   D[M,N] = alpha * (A1 . B1^T  +  A2 . B2^T) + beta * C
//
// Two operand pairs are accumulated into the SAME tensor-memory accumulator, i.e. the
// contraction runs over the concatenation [A1 | A2] x [B1 | B2].  Pair 2 is how a LoRA update
// is fused into the base projection (A2 = s * X.A^T of shape [M, r], B2 = lora_B of shape
// [N, r]) without a second pass over D; it is optional (K2 = 0).
//
// Operand layouts ("K-major": the contraction index is contiguous in memory,
// "MN-major": the M (or N) index is contiguous):
//   a_mn = 0 : A stored [M, K] row-major          a_mn = 1 : A stored [K, M] row-major
//   b_mn = 0 : B stored [N, K] row-major          b_mn = 1 : B stored [K, N] row-major
// so y = x W^T, dx = dy W and dW = dy^T x are all served without a transposed copy.
//
// Structure of one CTA (320 threads, one CTA per SM, persistent over output tiles):
//   warp 0      : TMA producer  (cp.async.bulk.tensor, 128-byte swizzle, no multicast)
//   warp 1      : MMA issuer    (one lane issues tcgen05.mma, 128 x BN x 16 per instruction)
//   warps 2..9  : epilogue      (tcgen05.ld of the fp32 accumulator, scale/add, 16-byte stores); two warps per
//                 tensor-memory lane quarter, taking the even and the odd 32-column chunks of the tile, so that a
//                 short main loop (K of a few hundred) still covers the epilogue of the previous tile
// The accumulator is double buffered in tensor memory (2 x BN columns) so the epilogue of
// tile i overlaps the main loop of tile i+1.  All mbarrier waits are bounded (common.cuh).
//
// The role of this kernel in the reference design: it replaces the cuBLAS calls behind
// torch.matmul in fms_acceleration_foak/fused_ops/unsloth_lora/utils.py:250-283 (matmul_lora)
// and the "dequant then matmul" of fms_acceleration_peft/gptqmodel/nn_modules/triton_utils/dequant.py:132-161.
#include "common.cuh"
#include <cstdlib>
#include <mutex>

namespace fmsb {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int GROUP_M = 16;
constexpr int kGemmThreads = 320;   // 2 + 8 warps
constexpr int kEpilogueThreads = 256;

struct GemmParams {
  int M, N;
  int kblocks1, kblocks2;
  void* D;
  long long ldd;
  int d_fp32;
  const void* C;
  long long ldc;
  float alpha, beta;
  int fmt;  // 0 = fp16, 1 = bf16
  int* status;
  // grouped execution (mixture-of-experts): see fmsb_grouped_gemm
  int mode;                  // 0 plain, 1 grouped along M (rows of A/D segmented), 2 grouped along K (one D per group)
  int n_groups;
  const int* seg_off;        // [n_groups + 1] segment starts in rows, multiples of 128 (device memory)
  int b_group_rows;          // rows of B that belong to one group
  int b2_group_rows;         // rows of B2 that belong to one group (mode 1 with a second operand pair)
  int n_split;               // > 0: output columns >= n_split take their B tiles from the side-by-side map at
                             //      column - n_split (two weight matrices in one pass over A)
  int c_fp32;                // C holds fp32 (accumulating into an fp32 D over several launches)
  int tma_store;             // CTA-pair kernel: D (16-bit) leaves through shared memory and bulk tensor stores
  long long d_group_stride;  // elements between the D matrices of consecutive groups (mode 2)
  // mode 3: uniform batch indexed by (outer o, inner i), i < n_inner.  Operand offsets in elements of the
  // stored 2-D matrices: rows += o * x_ro + i * x_ri, columns += (i / x_div) * x_ci.
  int n_batch, n_inner;
  int a_ro, a_ri, a_ci, a_div;
  int b_ro, b_ri, b_ci, b_div;
  int d_ro, d_ri, d_ci;
};

struct TileInfo {
  int m0, n0;        // coordinates of the A rows / B columns of this tile
  int m_store;       // row offset used for stores (== m0 except in mode 2 where D is per group)
  int m_end;         // rows >= m_end are not stored
  int k_begin;       // first contraction element (mode 2: segment start)
  int kblocks1;      // 64-wide blocks of operand pair 1 for this tile
  int b_row_off;     // added to B's row coordinate (group offset)
  int b2_row_off;    // the same for the second operand pair
  long long d_off;   // element offset of this tile's D matrix
  int a_r, a_c, b_r, b_c;  // batch offsets (mode 3): rows / columns of the stored A and B
  int d_c;                 // column offset of D (mode 3)
};

template <int BN>
struct GemmCfg {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStagesRaw = (200 * 1024) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kTmemCols = (2 * BN) < 32 ? 32 : (2 * BN);
  // staging of the store epilogue (BN = 256 only): 8 warps x 2 slots x (32 rows x 64 B)
  static constexpr int kEpiBytes = BN == 256 ? 8 * 2 * 2048 : 0;
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 1024 /*align slack*/ + 256 /*barriers*/;
};

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int group_size = GROUP_M * tiles_n;
  const int group = t / group_size;
  const int first_m = group * GROUP_M;
  const int gm = min(tiles_m - first_m, GROUP_M);
  const int in_group = t - group * group_size;
  tm = first_m + in_group % gm;
  tn = in_group / gm;
}

// Decode persistent work item `t`.  Returns false when t is past the last tile.
template <int BN>
__device__ __forceinline__ bool get_tile(int t, const GemmParams& p, TileInfo& ti) {
  const int tiles_n = (p.N + BN - 1) / BN;
  ti.a_r = ti.a_c = ti.b_r = ti.b_c = ti.d_c = 0;
  ti.b2_row_off = 0;
  if (p.mode == 3) {
    const int tiles_m = (p.M + BM - 1) / BM;
    const int per = tiles_m * tiles_n;
    if (t >= per * p.n_batch) return false;
    const int b = t / per, r = t - b * per;
    const int o = b / p.n_inner, i = b - o * p.n_inner;
    ti.m0 = (r % tiles_m) * BM;
    ti.n0 = (r / tiles_m) * BN;
    ti.a_r = o * p.a_ro + i * p.a_ri;
    ti.a_c = (i / p.a_div) * p.a_ci;
    ti.b_r = o * p.b_ro + i * p.b_ri;
    ti.b_c = (i / p.b_div) * p.b_ci;
    ti.m_store = ti.m0 + o * p.d_ro + i * p.d_ri;
    ti.m_end = ti.m_store - ti.m0 + p.M;
    ti.d_c = i * p.d_ci;
    ti.k_begin = 0;
    ti.kblocks1 = p.kblocks1;
    ti.b_row_off = 0;
    ti.d_off = 0;
    return true;
  }
  if (p.mode == 0) {
    const int tiles_m = (p.M + BM - 1) / BM;
    if (t >= tiles_m * tiles_n) return false;
    int tm, tn;
    tile_coords(t, tiles_m, tiles_n, tm, tn);
    ti.m0 = tm * BM;
    ti.n0 = tn * BN;
    ti.m_store = ti.m0;
    ti.m_end = p.M;
    ti.k_begin = 0;
    ti.kblocks1 = p.kblocks1;
    ti.b_row_off = 0;
    ti.d_off = 0;
    return true;
  }
  if (p.mode == 1) {
    // segments of A/D rows, one B matrix per segment; M-fastest inside a segment so that the
    // CTAs running at the same time share the segment's B tiles
    int rem = t;
    for (int g = 0; g < p.n_groups; ++g) {
      const int s0 = p.seg_off[g];
      const int mt = (p.seg_off[g + 1] - s0) / BM;
      const int ntile = mt * tiles_n;
      if (rem < ntile) {
        ti.m0 = s0 + (rem % mt) * BM;
        ti.n0 = (rem / mt) * BN;
        ti.m_store = ti.m0;
        ti.m_end = p.seg_off[g + 1];
        ti.k_begin = 0;
        ti.kblocks1 = p.kblocks1;
        ti.b_row_off = g * p.b_group_rows;
        ti.b2_row_off = g * p.b2_group_rows;
        ti.d_off = 0;
        return true;
      }
      rem -= ntile;
    }
    return false;
  }
  // mode 2: D[g] = A[seg_g]^T B[seg_g]; the contraction runs over the rows of segment g
  const int tiles_m = (p.M + BM - 1) / BM;
  const int per_group = tiles_m * tiles_n;
  if (t >= per_group * p.n_groups) return false;
  const int g = t / per_group;
  const int r = t - g * per_group;
  ti.m0 = (r % tiles_m) * BM;
  ti.n0 = (r / tiles_m) * BN;
  ti.m_store = ti.m0;
  ti.m_end = p.M;
  ti.k_begin = p.seg_off[g];
  ti.kblocks1 = (p.seg_off[g + 1] - p.seg_off[g]) / BK;
  ti.b_row_off = 0;
  ti.d_off = (long long)g * p.d_group_stride;
  return true;
}

// Epilogue of one tile for one warp: read this warp's 32 accumulator lanes in 32-column chunks (every other chunk,
// starting at `cpar`), apply alpha / beta * C, convert and store.  `gm` is the global row of this thread's lane.
template <int BN>
__device__ __forceinline__ void epilogue_store_tile(const GemmParams& p, const TileInfo& ti, uint32_t taddr, int cpar,
                                                    int gm, int n0, bool empty_k) {
  constexpr int CH = BN >= 32 ? 32 : 16;
#pragma unroll 1
  for (int c = cpar; c < BN / CH; c += 2) {
    float v[CH];
    if constexpr (CH == 32) {
      uint32_t r[32];
      tmem_ld_32x32(taddr + c * CH, r);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = empty_k ? 0.f : __uint_as_float(r[i]);
    } else {
      uint32_t r[16];
      tmem_ld_32x16(taddr + c * CH, r);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = empty_k ? 0.f : __uint_as_float(r[i]);
    }
    const int gn = n0 + c * CH;
    if (gm < ti.m_end && gn < p.N) {
      const bool full = (gn + CH <= p.N);
#pragma unroll
      for (int i = 0; i < CH; ++i) v[i] *= p.alpha;
      if (p.C != nullptr && p.beta != 0.f) {
        if (p.c_fp32) {
          const float* crow = reinterpret_cast<const float*>(p.C) + ti.d_off + (long long)gm * p.ldc + gn + ti.d_c;
          if (full && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0)) {
#pragma unroll
            for (int i = 0; i < CH; i += 4) {
              const float4 f = *reinterpret_cast<const float4*>(crow + i);
              v[i] += p.beta * f.x;
              v[i + 1] += p.beta * f.y;
              v[i + 2] += p.beta * f.z;
              v[i + 3] += p.beta * f.w;
            }
          } else {
            for (int i = 0; i < CH; ++i)
              if (gn + i < p.N) v[i] += p.beta * crow[i];
          }
        } else if (p.fmt == 1) {
          const __nv_bfloat16* crow = reinterpret_cast<const __nv_bfloat16*>(p.C) + ti.d_off + (long long)gm * p.ldc + gn + ti.d_c;
          if (full && ((reinterpret_cast<uintptr_t>(crow) & 15) == 0)) {
#pragma unroll
            for (int i = 0; i < CH; i += 8) {
              uint4 u = *reinterpret_cast<const uint4*>(crow + i);
              const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float2 f = __bfloat1622float2(h[j]);
                v[i + 2 * j] += p.beta * f.x;
                v[i + 2 * j + 1] += p.beta * f.y;
              }
            }
          } else {
            for (int i = 0; i < CH; ++i)
              if (gn + i < p.N) v[i] += p.beta * __bfloat162float(crow[i]);
          }
        } else {
          const __half* crow = reinterpret_cast<const __half*>(p.C) + ti.d_off + (long long)gm * p.ldc + gn + ti.d_c;
          for (int i = 0; i < CH; ++i)
            if (gn + i < p.N) v[i] += p.beta * __half2float(crow[i]);
        }
      }
      if (p.d_fp32) {
        float* drow = reinterpret_cast<float*>(p.D) + ti.d_off + (long long)gm * p.ldd + gn + ti.d_c;
        if (full && ((reinterpret_cast<uintptr_t>(drow) & 15) == 0)) {
#pragma unroll
          for (int i = 0; i < CH; i += 4)
            *reinterpret_cast<float4*>(drow + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        } else {
          for (int i = 0; i < CH; ++i)
            if (gn + i < p.N) drow[i] = v[i];
        }
      } else {
        uint16_t* drow = reinterpret_cast<uint16_t*>(p.D) + ti.d_off + (long long)gm * p.ldd + gn + ti.d_c;
        if (full && ((reinterpret_cast<uintptr_t>(drow) & 15) == 0)) {
#pragma unroll
          for (int i = 0; i < CH; i += 8) {
            uint4 u;
            if (p.fmt == 1) {
              u.x = pack_bf16x2(v[i], v[i + 1]);
              u.y = pack_bf16x2(v[i + 2], v[i + 3]);
              u.z = pack_bf16x2(v[i + 4], v[i + 5]);
              u.w = pack_bf16x2(v[i + 6], v[i + 7]);
            } else {
              u.x = pack_f16x2(v[i], v[i + 1]);
              u.y = pack_f16x2(v[i + 2], v[i + 3]);
              u.z = pack_f16x2(v[i + 4], v[i + 5]);
              u.w = pack_f16x2(v[i + 6], v[i + 7]);
            }
            *reinterpret_cast<uint4*>(drow + i) = u;
          }
        } else {
          for (int i = 0; i < CH; ++i) {
            if (gn + i < p.N) {
              if (p.fmt == 1) {
                __nv_bfloat16 b = __float2bfloat16_rn(v[i]);
                drow[i] = *reinterpret_cast<uint16_t*>(&b);
              } else {
                __half b = __float2half_rn(v[i]);
                drow[i] = *reinterpret_cast<uint16_t*>(&b);
              }
            }
          }
        }
      }
    }
  }
}

// Epilogue of one tile for one warp through shared memory: every 32-column chunk of this warp's 32 accumulator lanes is
// converted to 16 bits, written into a 2 KB staging slot (64-byte rows, 64-byte swizzle so that the quarter-warp phases
// of the 16-byte stores hit distinct banks) and leaves with ONE bulk tensor store of a 32 x 32 box, which also clips the
// ragged edges of M and N.  Two slots per warp alternate; a slot is rewritten only after the store that read it.
template <int BN>
__device__ __forceinline__ void epilogue_store_tile_tma(const GemmParams& p, const CUtensorMap* tmD, uint32_t taddr,
                                                        int cpar, int row0, int gm, int n0, bool empty_k, uint32_t slots,
                                                        int lane, int& slot) {
  constexpr int CH = 32;
#pragma unroll 1
  for (int c = cpar; c < BN / CH; c += 2) {
    uint32_t r[32];
    tmem_ld_32x32(taddr + c * CH, r);
    tmem_ld_wait();
    float v[CH];
#pragma unroll
    for (int i = 0; i < CH; ++i) v[i] = (empty_k ? 0.f : __uint_as_float(r[i])) * p.alpha;
    const int gn = n0 + c * CH;
    if (p.C != nullptr && p.beta != 0.f && gm < p.M && gn < p.N) {
      if (p.fmt == 1) {
        const __nv_bfloat16* crow = reinterpret_cast<const __nv_bfloat16*>(p.C) + (long long)gm * p.ldc + gn;
        for (int i = 0; i < CH; ++i)
          if (gn + i < p.N) v[i] += p.beta * __bfloat162float(crow[i]);
      } else {
        const __half* crow = reinterpret_cast<const __half*>(p.C) + (long long)gm * p.ldc + gn;
        for (int i = 0; i < CH; ++i)
          if (gn + i < p.N) v[i] += p.beta * __half2float(crow[i]);
      }
    }
    const uint32_t buf = slots + static_cast<uint32_t>(slot) * 2048u;
    if (lane == 0) tma_store_wait_read<1>();  // the store that last read this slot (two stores ago) is done with it
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t w0, w1, w2, w3;
      if (p.fmt == 1) {
        w0 = pack_bf16x2(v[8 * j], v[8 * j + 1]); w1 = pack_bf16x2(v[8 * j + 2], v[8 * j + 3]);
        w2 = pack_bf16x2(v[8 * j + 4], v[8 * j + 5]); w3 = pack_bf16x2(v[8 * j + 6], v[8 * j + 7]);
      } else {
        w0 = pack_f16x2(v[8 * j], v[8 * j + 1]); w1 = pack_f16x2(v[8 * j + 2], v[8 * j + 3]);
        w2 = pack_f16x2(v[8 * j + 4], v[8 * j + 5]); w3 = pack_f16x2(v[8 * j + 6], v[8 * j + 7]);
      }
      const uint32_t chunk = static_cast<uint32_t>(j) ^ ((static_cast<uint32_t>(lane) >> 1) & 3u);  // 64-byte swizzle
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(buf + lane * 64u + chunk * 16u), "r"(w0), "r"(w1),
                   "r"(w2), "r"(w3)
                   : "memory");
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0 && gn < p.N && row0 < p.M) {
      tma_store_2d(tmD, buf, gn, row0);
      tma_store_commit();
    }
    slot ^= 1;
  }
}

template <int BN, int A_MN, int B_MN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA1, const __grid_constant__ CUtensorMap tmB1,
                    const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2,
                    const __grid_constant__ CUtensorMap tmBalt, const __grid_constant__ CUtensorMap tmD,
                    const GemmParams p) {
  using Cfg = GemmCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  // 128-byte swizzled tiles need 1024-byte alignment
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t epi_base = smem_base + Cfg::kStages * Cfg::kStageBytes;
  const uint32_t bar_base = epi_base + Cfg::kEpiBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (Cfg::kStages + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * Cfg::kStages + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * Cfg::kStages + 2 + a); };
  const uint32_t holder = bar_base + 8u * (2 * Cfg::kStages + 4);
  auto sA = [&](int s) { return smem_base + s * Cfg::kStageBytes; };
  auto sB = [&](int s) { return smem_base + s * Cfg::kStageBytes + Cfg::kABytes; };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (warp == 1 && lane == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), kEpilogueThreads);
    }
    fence_barrier_init();
  }
  if (warp == 0) {
    if (lane == 0) {
      prefetch_tmap(&tmA1);
      prefetch_tmap(&tmB1);
      if (p.kblocks2 > 0) {
        prefetch_tmap(&tmA2);
        prefetch_tmap(&tmB2);
      }
      if (p.n_split > 0) prefetch_tmap(&tmBalt);
    }
    __syncwarp();
    tmem_alloc(holder, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(holder));

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      TileInfo ti;
      for (int t = blockIdx.x; ok && get_tile<BN>(t, p, ti); t += gridDim.x) {
        const int m0 = ti.m0;
        const int kblocks = ti.kblocks1 + p.kblocks2;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, p.status, kTimeoutProducer)) {
            ok = false;
            break;
          }
          mbar_expect_tx(full_bar(stage), Cfg::kStageBytes);
          const bool second = kb >= ti.kblocks1;
          // right-hand weight matrix of a side-by-side pair; the second operand pair spans all N columns itself
          const bool alt = !second && p.n_split > 0 && ti.n0 >= p.n_split;
          const int n0 = alt ? ti.n0 - p.n_split : ti.n0;
          const CUtensorMap* ta = second ? &tmA2 : &tmA1;
          const CUtensorMap* tb = second ? &tmB2 : (alt ? &tmBalt : &tmB1);
          const int k0 = second ? (kb - ti.kblocks1) * BK : ti.k_begin + kb * BK;
          // the group offset applies to B's row coordinate: the k rows of an MN-major B, the n rows of a K-major B
          const int brow = second ? ti.b2_row_off : ti.b_row_off;
          // stored A: [M, K] (K-major) or [K, M] (MN-major); the batch offsets address rows / columns of the storage
          if (A_MN == 0) {
            tma_load_2d(sA(stage), ta, full_bar(stage), k0 + ti.a_c, m0 + ti.a_r);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sA(stage) + j * 8192, ta, full_bar(stage), m0 + 64 * j + ti.a_c, k0 + ti.a_r);
          }
          if (B_MN == 0) {
            tma_load_2d(sB(stage), tb, full_bar(stage), k0 + ti.b_c, n0 + brow + ti.b_r);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sB(stage) + j * 8192, tb, full_bar(stage), n0 + 64 * j + ti.b_c, k0 + brow + ti.b_r);
          }
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(BM, BN, p.fmt, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      TileInfo ti;
      for (int t = blockIdx.x; ok && get_tile<BN>(t, p, ti); t += gridDim.x) {
        const int kblocks = ti.kblocks1 + p.kblocks2;
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, p.status, kTimeoutMma)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, p.status, kTimeoutMma)) {
            ok = false;
            break;
          }
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = A_MN ? make_smem_desc(sA(stage) + k * 2048, 8192, 1024)
                                        : make_smem_desc(sA(stage) + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc(sB(stage) + k * 2048, 8192, 1024)
                                        : make_smem_desc(sB(stage) + k * 32, 16, 1024);
            tc_mma_f16(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit(empty_bar(stage));
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        if (kblocks == 0) {
          // empty segment (mode 2): nothing was accumulated; the epilogue writes zeros
        }
        tc_commit(tfull_bar(acc));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (8 warps)
    const int q = warp & 3;           // tensor-memory lane quarter this warp may read
    const int cpar = (warp - 2) >> 2;  // 0: even column chunks, 1: odd column chunks
    const int row = q * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    TileInfo ti;
    // store epilogue through shared memory (BN = 256, 16-bit D, plain and grouped-M modes): two 2 KB slots per warp
    const uint32_t my_slots = epi_base + static_cast<uint32_t>(warp - 2) * 4096u;
    int slot = 0;
    for (int t = blockIdx.x; get_tile<BN>(t, p, ti); t += gridDim.x) {
      const int gm = ti.m_store + row;
      const int n0 = ti.n0;
      const bool empty_k = (ti.kblocks1 + p.kblocks2) == 0;
      if (!mbar_wait(tfull_bar(acc), acc_phase, p.status, kTimeoutEpilogue)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * BN);
      bool stored = false;
      if constexpr (BN == 256) {
        // a box store writes 32 whole rows: only for tiles whose rows all belong to the segment
        if (p.tma_store && ti.m_store + BM <= ti.m_end) {
          epilogue_store_tile_tma<BN>(p, &tmD, taddr, cpar, ti.m_store + q * 32, gm, n0, empty_k, my_slots, lane, slot);
          stored = true;
        }
      }
      if (!stored) epilogue_store_tile<BN>(p, ti, taddr, cpar, gm, n0, empty_k);
      tc_fence_before();
      mbar_arrive(tempty_bar(acc));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if constexpr (BN == 256) {
      if (p.tma_store && lane == 0) tma_store_wait<0>();  // the staging slots stay valid until the last store has read them
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}


// ----------------------------------------------------------------------------------------
// CTA-pair variant (plain mode, 256 x 256 output tiles): a cluster of two CTAs on the two SMs of one TPC computes
// one tile with tcgen05.mma.cta_group::2 (M = 256, N = 256).  CTA r of the pair stages rows [m0 + 128 r, +128) of A
// and rows/columns [n0 + 128 r, +128) of B (its half of the N extent) per K block with its own tensor loads (no
// multicast), so per SM and K block 32 KB enter shared memory for a 256 x 256 x 64 product where the single-CTA kernel
// moves 48 KB for 128 x 256 x 64: B traffic per output element halves, and so does the number of MMA instructions per
// SM.  The pair's leader (cluster rank 0) issues all MMAs; they read both CTAs' shared memory and write 128 lanes of
// tensor memory in each CTA; every CTA drains its own lanes with the same 8 epilogue warps as the single-CTA kernel.
//
// Barriers (same shared-memory offsets in both CTAs):
//   full[s]    used in the leader only: 1 arrival (the leader's producer announces the bytes of BOTH CTAs' loads; the
//              peer's loads complete on the same barrier, possibly before the announcement: the byte count of a
//              phase may run negative, and a peer load of the next pass cannot start before this phase is over)
//   empty[s]   per CTA: released by the leader's commit (arrives in both CTAs)
//   tfull[a]   per CTA: accumulator a complete (leader's commit, both CTAs)
//   tempty[a]  used in the leader only: 16 arrivals (8 epilogue warps of each CTA)
// ----------------------------------------------------------------------------------------
constexpr int BM2 = 256;   // rows of a pair's tile
constexpr int BN2 = 256;   // columns of a pair's tile
constexpr int BNH = 128;   // B rows staged by each CTA

struct PairCfg {
  static constexpr int kABytes = BM * BK * 2;    // 16 KB
  static constexpr int kBBytes = BNH * BK * 2;   // 16 KB
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = 6;
  static constexpr int kTmemCols = 2 * BN2;      // two accumulators of 256 columns: all of tensor memory
  static constexpr int kEpiBytes = 8 * 2 * 2048;  // staging of the store epilogue: 8 warps x 2 slots x (32 rows x 64 B)
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + 1024 + 256;
};

template <int A_MN, int B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmA1, const __grid_constant__ CUtensorMap tmB1,
                         const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2,
                         const __grid_constant__ CUtensorMap tmD, const GemmParams p) {
  using Cfg = PairCfg;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t epi_base = smem_base + Cfg::kStages * Cfg::kStageBytes;
  const uint32_t bar_base = epi_base + Cfg::kEpiBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (Cfg::kStages + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * Cfg::kStages + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * Cfg::kStages + 2 + a); };
  const uint32_t holder = bar_base + 8u * (2 * Cfg::kStages + 4);
  auto sA = [&](int s) { return smem_base + s * Cfg::kStageBytes; };
  auto sB = [&](int s) { return smem_base + s * Cfg::kStageBytes + Cfg::kABytes; };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();        // 0: leader
  const int pair = blockIdx.x >> 1;
  const int n_pairs = gridDim.x >> 1;
  const int tiles_m = (p.M + BM2 - 1) / BM2;
  const int tiles_n = (p.N + BN2 - 1) / BN2;
  const int n_tiles = tiles_m * tiles_n;
  const int kblocks = p.kblocks1 + p.kblocks2;

  if (warp == 1 && lane == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 16);
    }
    fence_barrier_init();
  }
  if (warp == 0) {
    if (lane == 0) {
      prefetch_tmap(&tmA1);
      prefetch_tmap(&tmB1);
      if (p.kblocks2 > 0) {
        prefetch_tmap(&tmA2);
        prefetch_tmap(&tmB2);
      }
    }
    __syncwarp();
    tmem_alloc_pair(holder, Cfg::kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before either one signals the other
  tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(holder));

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (each CTA loads its own halves)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair; ok && t < n_tiles; t += n_pairs) {
        int tm, tn;
        tile_coords(t, tiles_m, tiles_n, tm, tn);
        const int m0 = tm * BM2 + (int)cta * BM;
        const int n0 = tn * BN2 + (int)cta * BNH;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, p.status, kTimeoutProducer)) {
            ok = false;
            break;
          }
          const uint32_t lead_full = mapa_shared(full_bar(stage), 0);
          if (cta == 0) mbar_expect_tx(full_bar(stage), 2 * Cfg::kStageBytes);
          const bool second = kb >= p.kblocks1;
          const CUtensorMap* ta = second ? &tmA2 : &tmA1;
          const CUtensorMap* tb = second ? &tmB2 : &tmB1;
          const int k0 = second ? (kb - p.kblocks1) * BK : kb * BK;
          if (A_MN == 0) {
            tma_load_2d_pair(sA(stage), ta, lead_full, k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sA(stage) + j * 8192, ta, lead_full, m0 + 64 * j, k0);
          }
          if (B_MN == 0) {
            tma_load_2d_pair(sB(stage), tb, lead_full, k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BNH / 64; ++j) tma_load_2d_pair(sB(stage) + j * 8192, tb, lead_full, n0 + 64 * j, k0);
          }
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && cta == 0) {
      const uint32_t idesc = make_idesc_f16(BM2, BN2, p.fmt, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = pair; ok && t < n_tiles; t += n_pairs) {
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, p.status, kTimeoutMma)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN2);
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, p.status, kTimeoutMma)) {
            ok = false;
            break;
          }
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = A_MN ? make_smem_desc(sA(stage) + k * 2048, 8192, 1024)
                                        : make_smem_desc(sA(stage) + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc(sB(stage) + k * 2048, 8192, 1024)
                                        : make_smem_desc(sB(stage) + k * 32, 16, 1024);
            tc_mma_f16_pair(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit_pair(empty_bar(stage), 3);  // the stage is free again in both CTAs
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        tc_commit_pair(tfull_bar(acc), 3);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (8 warps, this CTA's 128 rows)
    const int q = warp & 3;
    const int cpar = (warp - 2) >> 2;
    const int row = q * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    int slot = 0;
    const uint32_t my_slots = epi_base + static_cast<uint32_t>(warp - 2) * 4096u;
    if (p.tma_store && lane == 0) prefetch_tmap(&tmD);
    TileInfo ti;
    ti.d_off = 0;
    ti.d_c = 0;
    ti.m_end = p.M;
    for (int t = pair; t < n_tiles; t += n_pairs) {
      int tm, tn;
      tile_coords(t, tiles_m, tiles_n, tm, tn);
      const int row0 = tm * BM2 + (int)cta * BM + q * 32;
      const int gm = row0 + lane;
      const int n0 = tn * BN2;
      ti.n0 = n0;
      if (!mbar_wait(tfull_bar(acc), acc_phase, p.status, kTimeoutEpilogue)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * BN2);
      if (p.tma_store)
        epilogue_store_tile_tma<BN2>(p, &tmD, taddr, cpar, row0, gm, n0, kblocks == 0, my_slots, lane, slot);
      else
        epilogue_store_tile<BN2>(p, ti, taddr, cpar, gm, n0, kblocks == 0);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(tempty_bar(acc), 0));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (p.tma_store && lane == 0) tma_store_wait<0>();  // the staging slots stay valid until the last store has read them
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves (or frees tensor memory) while the other may still signal or read it
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, Cfg::kTmemCols);
  }
}

}  // namespace fmsb

// ========================================================================================
// host side
// ========================================================================================
namespace fmsb_host {

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
  });
  return fn;
}

int make_tmap_2d_16b(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride_elems,
                     uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn enc = get_encode_tiled();
  if (enc == nullptr) return -1;
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstr[1] = {row_stride_elems * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstr, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -static_cast<int>(r) - 100;
}

// 2-D row-major tensor of 16-bit elements with a 64-byte swizzle (staging of the store epilogue: 32 x 32 boxes).
int make_tmap_2d_16b_sw64(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride_elems,
                          uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn enc = get_encode_tiled();
  if (enc == nullptr) return -1;
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstr[1] = {row_stride_elems * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstr, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -static_cast<int>(r) - 100;
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

template <int BN, int A_MN, int B_MN>
int launch_gemm(const CUtensorMap& a1, const CUtensorMap& b1, const CUtensorMap& a2, const CUtensorMap& b2,
                const CUtensorMap& balt, const CUtensorMap& d, const fmsb::GemmParams& p, int max_ctas,
                cudaStream_t stream) {
  using Cfg = fmsb::GemmCfg<BN>;
  auto kern = fmsb::gemm_tcgen05_kernel<BN, A_MN, B_MN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  int ctas = sm_count();
  if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
  if (p.mode == 0) {
    const int tiles = ((p.M + fmsb::BM - 1) / fmsb::BM) * ((p.N + BN - 1) / BN);
    if (tiles < ctas) ctas = tiles;
  }
  if (ctas <= 0) return 0;
  kern<<<ctas, fmsb::kGemmThreads, Cfg::kSmemBytes, stream>>>(a1, b1, a2, b2, balt, d, p);
  return static_cast<int>(cudaGetLastError());
}

static int g_pair_occupancy = -1, g_pair_occupancy_error = -1;

// Clusters of two CTAs that can be resident at once (one pair per TPC when the kernel takes a whole SM).
template <int A_MN, int B_MN>
int launch_gemm_pair(const CUtensorMap& a1, const CUtensorMap& b1, const CUtensorMap& a2, const CUtensorMap& b2,
                     const CUtensorMap& d, const fmsb::GemmParams& p, int max_ctas, cudaStream_t stream) {
  using Cfg = fmsb::PairCfg;
  auto kern = fmsb::gemm_tcgen05_pair_kernel<A_MN, B_MN>;
  static int max_pairs = -1;
  if (max_pairs < 0) {
    g_pair_occupancy_error = 0;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sm_count(), 1, 1);
    cfg.blockDim = dim3(fmsb::kGemmThreads, 1, 1);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
    g_pair_occupancy_error = (int)e;
    g_pair_occupancy = n;
    max_pairs = (e == cudaSuccess && n > 0) ? n : sm_count() / 2;
    (void)cudaGetLastError();
    if (const char* env = getenv("FMSB_GEMM_PAIRS")) {
      const int v = atoi(env);
      if (v > 0) max_pairs = v;
    }
  }
  int pairs = max_pairs;
  if (max_ctas > 0 && max_ctas / 2 < pairs) pairs = max_ctas / 2;
  const int tiles = ((p.M + fmsb::BM2 - 1) / fmsb::BM2) * ((p.N + fmsb::BN2 - 1) / fmsb::BN2);
  if (tiles < pairs) pairs = tiles;
  if (pairs <= 0) return 0;
  kern<<<2 * pairs, fmsb::kGemmThreads, Cfg::kSmemBytes, stream>>>(a1, b1, a2, b2, d, p);
  return static_cast<int>(cudaGetLastError());
}

// store epilogue through shared memory and bulk tensor stores (1, default) or per-thread 16-byte stores (0)
static int g_pair_tma_store = 1;
static int g_single_tma_store = 1;

// 0: never, 1: when there are enough 256 x 256 tiles to fill the machine about twice (default), 2: whenever M and N
// reach 256; set through fmsb_gemm_set_pair_mode (tests compare both kernels on small shapes)
static int g_pair_mode = 1;

}  // namespace fmsb_host

// what the occupancy query answered for the CTA-pair kernel (after its first launch): clusters, or -(error) - 1
extern "C" int fmsb_gemm_pair_occupancy() {
  return fmsb_host::g_pair_occupancy_error > 0 ? -fmsb_host::g_pair_occupancy_error - 1 : fmsb_host::g_pair_occupancy;
}

// 1 (default): 16-bit D leaves through shared memory and bulk tensor stores (CTA-pair kernel, and the single-CTA kernel
// with BN = 256 in the plain and grouped-M modes); 0: per-thread 16-byte stores everywhere (the cross-check of the tests)
extern "C" int fmsb_gemm_set_pair_store(int tma_store) {
  const int old = fmsb_host::g_pair_tma_store;
  fmsb_host::g_pair_tma_store = tma_store;
  fmsb_host::g_single_tma_store = tma_store;
  return old;
}

extern "C" int fmsb_gemm_set_pair_mode(int mode) {
  const int old = fmsb_host::g_pair_mode;
  fmsb_host::g_pair_mode = mode;
  return old;
}

// D[M,N] = alpha * (A1.B1^T + A2.B2^T) + beta * C.   16-bit inputs (fmt 0 = fp16, 1 = bf16).
// Constraints: leading dimensions multiples of 8 elements; base pointers 16-byte aligned.  bn selects the N tile (16/32/64/128/256); MN-major B needs bn >= 64.
// max_ctas > 0 limits the grid (used to leave SMs to a concurrent communication kernel).
// Returns 0 or a CUDA / encode error code.  Time-outs are reported through *status.
// Optional extras of the grouped modes.
struct GroupExtra {
  const void* B_alt = nullptr;  // second weight matrix for output columns >= n_split (same layout and ldb as B)
  int n_split = 0;
  int b2_group_rows = 0;
  int c_fp32 = 0;
};

struct BatchDesc {
  int n_batch = 0, n_inner = 1;
  int a_ro = 0, a_ri = 0, a_ci = 0, a_div = 1;
  int b_ro = 0, b_ri = 0, b_ci = 0, b_div = 1;
  int d_ro = 0, d_ri = 0, d_ci = 0;
  long long a_cols = 0, b_cols = 0;  // column extents of the stored matrices (tensor-map bounds)
};

static int gemm_impl(const void* A1, long long lda1, const void* B1, long long ldb1, int K1,  //
                     const void* A2, long long lda2, const void* B2, long long ldb2, int K2,  //
                     int a_mn, int b_mn,                                                       //
                     void* D, long long ldd, int d_fp32, const void* C, long long ldc,        //
                     float alpha, float beta, int M, int N, int fmt, int bn, int max_ctas, int* status,
                     cudaStream_t stream, int mode, int n_groups, const int* seg_off, int b_group_rows,
                     long long d_group_stride, long long a_rows, long long b_rows, const BatchDesc* bd = nullptr,
                     const GroupExtra* gx = nullptr) {
  using namespace fmsb_host;
  if (M <= 0 || N <= 0) return 0;
  if (K1 <= 0 || K2 < 0) return -2;
  if ((lda1 % 8) || (ldb1 % 8) || (K2 > 0 && ((lda2 % 8) || (ldb2 % 8)))) return -2;
  if (b_mn && bn < 64) return -3;
  CUtensorMap ta1, tb1, ta2, tb2, tbalt;
  int rc;
  // CTA pairs: plain mode, 256-column tiles, enough 256 x 256 tiles to fill the machine about twice
  const bool use_pair = mode == 0 && bn == 256 && g_pair_mode != 0 && M >= 256 && N >= 256 &&
                        (g_pair_mode == 2 ||
                         (long long)((M + 255) / 256) * ((N + 255) / 256) >= 2LL * (sm_count() / 2));
  const int b_box_rows = use_pair ? fmsb::BNH : bn;
  // a_rows / b_rows: number of rows of the stored A / B matrices when it differs from the per-tile view
  // (grouped modes address several segments / expert matrices through one tensor map)
  const long long a_cols = bd && bd->a_cols > 0 ? bd->a_cols : 0, b_cols = bd && bd->b_cols > 0 ? bd->b_cols : 0;
  auto mk_a = [&](CUtensorMap* t, const void* A, long long lda, int K) {
    if (a_mn) return make_tmap_2d_16b(t, A, a_rows > 0 ? a_rows : K, a_cols > 0 ? a_cols : M, lda, 64, 64);
    return make_tmap_2d_16b(t, A, a_rows > 0 ? a_rows : M, a_cols > 0 ? a_cols : K, lda, fmsb::BM, 64);
  };
  // with n_split every one of the two side-by-side weight matrices is n_split columns wide
  const long long n_each = (gx != nullptr && gx->n_split > 0) ? gx->n_split : N;
  auto mk_b = [&](CUtensorMap* t, const void* B, long long ldb, int K, long long n_cols, long long rows) {
    if (b_mn) return make_tmap_2d_16b(t, B, rows > 0 ? rows : K, b_cols > 0 ? b_cols : n_cols, ldb, 64, 64);
    return make_tmap_2d_16b(t, B, rows > 0 ? rows : N, b_cols > 0 ? b_cols : K, ldb, b_box_rows, 64);
  };
  // stored rows of the second pair's B: its own group height times the number of groups (a low-rank factor is far
  // shorter than the weight it sits beside), so that reads past its end are zero-filled, not taken from memory
  const long long b2_rows = (gx != nullptr && gx->b2_group_rows > 0 && n_groups > 0)
                                ? (long long)gx->b2_group_rows * n_groups : b_rows;
  if ((rc = mk_a(&ta1, A1, lda1, K1))) return rc;
  if ((rc = mk_b(&tb1, B1, ldb1, K1, n_each, b_rows))) return rc;
  if (K2 > 0) {
    // the second pair covers all N output columns, also beside a side-by-side pair of first operands
    if ((rc = mk_a(&ta2, A2, lda2, K2))) return rc;
    if ((rc = mk_b(&tb2, B2, ldb2, K2, N, b2_rows))) return rc;
  } else {
    ta2 = ta1;
    tb2 = tb1;
  }
  tbalt = tb1;
  if (gx != nullptr && gx->n_split > 0) {
    if (gx->B_alt == nullptr || gx->n_split % bn != 0 || gx->n_split >= N) return -2;
    // same shape as B1: the column extent of one matrix is n_split (MN-major) / its row extent per group (K-major)
    if ((rc = mk_b(&tbalt, gx->B_alt, ldb1, K1, n_each, b_rows))) return rc;
  }
  fmsb::GemmParams p;
  p.M = M;
  p.N = N;
  p.kblocks1 = (K1 + fmsb::BK - 1) / fmsb::BK;
  p.kblocks2 = K2 > 0 ? (K2 + fmsb::BK - 1) / fmsb::BK : 0;
  p.D = D;
  p.ldd = ldd;
  p.d_fp32 = d_fp32;
  p.C = C;
  p.ldc = ldc;
  p.alpha = alpha;
  p.beta = beta;
  p.fmt = fmt;
  p.status = status;
  p.mode = mode;
  p.n_groups = n_groups;
  p.seg_off = seg_off;
  p.b_group_rows = b_group_rows;
  p.d_group_stride = d_group_stride;
  p.b2_group_rows = gx != nullptr ? gx->b2_group_rows : 0;
  p.n_split = gx != nullptr ? gx->n_split : 0;
  p.c_fp32 = gx != nullptr ? gx->c_fp32 : 0;
  p.tma_store = 0;
  p.n_batch = 0; p.n_inner = 1; p.a_div = p.b_div = 1;
  p.a_ro = p.a_ri = p.a_ci = p.b_ro = p.b_ri = p.b_ci = p.d_ro = p.d_ri = p.d_ci = 0;
  if (bd != nullptr) {
    p.n_batch = bd->n_batch; p.n_inner = bd->n_inner > 0 ? bd->n_inner : 1;
    p.a_ro = bd->a_ro; p.a_ri = bd->a_ri; p.a_ci = bd->a_ci; p.a_div = bd->a_div > 0 ? bd->a_div : 1;
    p.b_ro = bd->b_ro; p.b_ri = bd->b_ri; p.b_ci = bd->b_ci; p.b_div = bd->b_div > 0 ? bd->b_div : 1;
    p.d_ro = bd->d_ro; p.d_ri = bd->d_ri; p.d_ci = bd->d_ci;
  }

  if (use_pair) {
    CUtensorMap td = ta1;
    p.tma_store = 0;
    if (g_pair_tma_store && !d_fp32 && ldd % 8 == 0 && (reinterpret_cast<uintptr_t>(D) & 15) == 0 &&
        make_tmap_2d_16b_sw64(&td, D, (uint64_t)M, (uint64_t)N, (uint64_t)ldd, 32, 32) == 0)
      p.tma_store = 1;
    if (!a_mn && !b_mn) return launch_gemm_pair<0, 0>(ta1, tb1, ta2, tb2, td, p, max_ctas, stream);
    if (a_mn && !b_mn) return launch_gemm_pair<1, 0>(ta1, tb1, ta2, tb2, td, p, max_ctas, stream);
    if (!a_mn && b_mn) return launch_gemm_pair<0, 1>(ta1, tb1, ta2, tb2, td, p, max_ctas, stream);
    return launch_gemm_pair<1, 1>(ta1, tb1, ta2, tb2, td, p, max_ctas, stream);
  }
  // single-CTA kernel: the store epilogue through shared memory serves BN = 256 in the plain and grouped-M modes
  CUtensorMap td1 = ta1;
  if (bn == 256 && (mode == 0 || mode == 1) && bd == nullptr && g_single_tma_store && !d_fp32 && ldd % 8 == 0 &&
      (reinterpret_cast<uintptr_t>(D) & 15) == 0 &&
      make_tmap_2d_16b_sw64(&td1, D, (uint64_t)M, (uint64_t)N, (uint64_t)ldd, 32, 32) == 0)
    p.tma_store = 1;
#define FMSB_DISPATCH(BNV)                                                                          \
  if (bn == BNV) {                                                                                  \
    if (!a_mn && !b_mn) return launch_gemm<BNV, 0, 0>(ta1, tb1, ta2, tb2, tbalt, td1, p, max_ctas, stream);     \
    if (a_mn && !b_mn) return launch_gemm<BNV, 1, 0>(ta1, tb1, ta2, tb2, tbalt, td1, p, max_ctas, stream);      \
    if constexpr (BNV >= 64) {                                                                      \
      if (!a_mn && b_mn) return launch_gemm<BNV, 0, 1>(ta1, tb1, ta2, tb2, tbalt, td1, p, max_ctas, stream);    \
      if (a_mn && b_mn) return launch_gemm<BNV, 1, 1>(ta1, tb1, ta2, tb2, tbalt, td1, p, max_ctas, stream);     \
    }                                                                                               \
  }
  FMSB_DISPATCH(256)
  FMSB_DISPATCH(128)
  FMSB_DISPATCH(64)
  FMSB_DISPATCH(32)
  FMSB_DISPATCH(16)
#undef FMSB_DISPATCH
  return -4;
}

extern "C" int fmsb_gemm(const void* A1, long long lda1, const void* B1, long long ldb1, int K1,  //
                         const void* A2, long long lda2, const void* B2, long long ldb2, int K2,  //
                         int a_mn, int b_mn,                                                       //
                         void* D, long long ldd, int d_fp32, const void* C, long long ldc,        //
                         float alpha, float beta, int M, int N, int fmt, int bn, int max_ctas, int* status,
                         cudaStream_t stream) {
  return gemm_impl(A1, lda1, B1, ldb1, K1, A2, lda2, B2, ldb2, K2, a_mn, b_mn, D, ldd, d_fp32, C, ldc, alpha, beta, M,
                   N, fmt, bn, max_ctas, status, stream, 0, 0, nullptr, 0, 0, 0, 0);
}

// Grouped GEMM for mixture-of-experts layers.  seg_off[g] (device, n_groups + 1 ints, multiples of 128) are the
// row offsets of the expert segments inside the expert-sorted activation buffers.
//   mode 1: D[seg_g, :N] = A[seg_g, :K] . B_g      A [rows, K] K-major, rows = seg_off[n_groups] (a_rows >= that);
//           b_mn = 1: B_g = B[g*K : (g+1)*K, :N]    (weights stored [E, in, out], forward)
//           b_mn = 0: B_g = B[g*N : (g+1)*N, :K]^T  (same storage, input gradient)
//   mode 2: D_g[M, N] = A[seg_g, :M]^T . B[seg_g, :N]   (weight gradient; a_mn = b_mn = 1; D_g at D + g*d_group_stride)
extern "C" int fmsb_grouped_gemm(const void* A, long long lda, const void* B, long long ldb, int K, int b_mn, void* D,
                                 long long ldd, int d_fp32, const void* C, long long ldc, float alpha, float beta, int M,
                                 int N, int fmt, int bn, int mode, int n_groups, const int* seg_off,
                                 long long d_group_stride, long long a_rows, long long b_rows, int* status,
                                 cudaStream_t stream) {
  if (mode == 1) {
    const int b_group_rows = b_mn ? K : N;
    return gemm_impl(A, lda, B, ldb, K, nullptr, 0, nullptr, 0, 0, 0, b_mn, D, ldd, d_fp32, C, ldc, alpha, beta,
                     (int)a_rows, N, fmt, bn, 0, status, stream, 1, n_groups, seg_off, b_group_rows, 0, a_rows, b_rows);
  }
  if (mode == 2) {
    // K is only a placeholder here: the contraction length of each group comes from seg_off
    return gemm_impl(A, lda, B, ldb, 64, nullptr, 0, nullptr, 0, 0, 1, 1, D, ldd, d_fp32, C, ldc, alpha, beta, M, N,
                     fmt, bn, 0, status, stream, 2, n_groups, seg_off, 0, d_group_stride, a_rows, b_rows);
  }
  return -2;
}

// Uniform batched GEMM: for batch index (o, i), i < n_inner:  D_oi[M, N] = alpha * A_oi . B_oi^T (+ beta * C_oi),
// where the operands are windows of stored 2-D matrices.  desc = 13 ints:
//   {n_batch, n_inner, a_ro, a_ri, a_ci, a_div, b_ro, b_ri, b_ci, b_div, d_ro, d_ri, d_ci}
// rows += o * x_ro + i * x_ri and columns += (i / x_div) * x_ci of the STORED matrix (for an MN-major operand the
// stored rows are the contraction index).  a_rows/a_cols, b_rows/b_cols: extents of the stored matrices.
extern "C" int fmsb_batched_gemm(const void* A, long long lda, long long a_rows, long long a_cols, const void* B,
                                 long long ldb, long long b_rows, long long b_cols, int K, int a_mn, int b_mn, void* D,
                                 long long ldd, int d_fp32, const void* C, long long ldc, float alpha, float beta, int M,
                                 int N, int fmt, int bn, const int* desc, int* status, cudaStream_t stream) {
  BatchDesc bd;
  bd.n_batch = desc[0]; bd.n_inner = desc[1];
  bd.a_ro = desc[2]; bd.a_ri = desc[3]; bd.a_ci = desc[4]; bd.a_div = desc[5];
  bd.b_ro = desc[6]; bd.b_ri = desc[7]; bd.b_ci = desc[8]; bd.b_div = desc[9];
  bd.d_ro = desc[10]; bd.d_ri = desc[11]; bd.d_ci = desc[12];
  bd.a_cols = a_cols; bd.b_cols = b_cols;
  if (bd.n_batch <= 0) return 0;
  return gemm_impl(A, lda, B, ldb, K, nullptr, 0, nullptr, 0, 0, a_mn, b_mn, D, ldd, d_fp32, C, ldc, alpha, beta, M, N,
                   fmt, bn, 0, status, stream, 3, 0, nullptr, 0, 0, a_rows, b_rows, &bd);
}

// Grouped GEMM with the extras of the mixture-of-experts layer:
//   * B_alt / n_split (mode 1 forward and mode 2): output columns [n_split, N) are produced from B_alt instead of B,
//     so gate and up projection (two weight tensors of the same shape) run as ONE pass over A with N = 2 * n_split;
//     for mode 2 the analogue is the pair of weight gradients (B = the left, B_alt = the right gradient operand).
//   * A2 / B2 / K2 (mode 1): a second operand pair accumulated into the same tile, with its own per-group row
//     offset b2_group_rows: D[seg_g] = A[seg_g] . B_g + A2[seg_g] . B2_g  (input gradient through gate and up in one
//     launch, or a per-expert low-rank update next to the frozen expert weight).
//   * c_fp32: C is fp32 (D += over several launches when D is fp32).
extern "C" int fmsb_grouped_gemm2(const void* A, long long lda, const void* B, long long ldb, int K, int b_mn,
                                  const void* B_alt, int n_split, const void* A2, long long lda2, const void* B2,
                                  long long ldb2, int K2, void* D, long long ldd, int d_fp32, const void* C,
                                  long long ldc, int c_fp32, float alpha, float beta, int M, int N, int fmt, int bn,
                                  int mode, int n_groups, const int* seg_off, long long d_group_stride, long long a_rows,
                                  long long b_rows, int max_ctas, int* status, cudaStream_t stream) {
  GroupExtra gx;
  gx.B_alt = B_alt;
  gx.n_split = n_split;
  gx.c_fp32 = c_fp32;
  if (mode == 1) {
    const int b_group_rows = b_mn ? K : N;
    // with n_split the K-major (b_mn = 0) form would need per-matrix row counts: only the MN-major form is offered
    if (n_split > 0 && !b_mn) return -2;
    gx.b2_group_rows = K2 > 0 ? (b_mn ? K2 : N) : 0;
    return gemm_impl(A, lda, B, ldb, K, A2, lda2, B2, ldb2, K2, 0, b_mn, D, ldd, d_fp32, C, ldc, alpha, beta, (int)a_rows,
                     N, fmt, bn, max_ctas, status, stream, 1, n_groups, seg_off, b_group_rows, 0, a_rows, b_rows, nullptr,
                     &gx);
  }
  if (mode == 2) {
    if (K2 > 0) return -2;
    return gemm_impl(A, lda, B, ldb, 64, nullptr, 0, nullptr, 0, 0, 1, 1, D, ldd, d_fp32, C, ldc, alpha, beta, M, N, fmt,
                     bn, max_ctas, status, stream, 2, n_groups, seg_off, 0, d_group_stride, a_rows, b_rows, nullptr, &gx);
  }
  return -2;
}
