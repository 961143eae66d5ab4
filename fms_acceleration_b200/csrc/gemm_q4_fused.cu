// Fused gather + NF4/FP4 dequantise + GEMM + LoRA for sm_100a:
//
//     y[M, N] = alpha * ( x[M, K] . dequant(Wq)[N, K]^T  +  xa[M, R] . Bl[N, R]^T )
//
// The 4-bit weight never exists in 16 bits in global memory: dequant warps read the packed bytes (two
// values per byte, blocks of 64 values sharing one scale, the scales themselves optionally 8-bit "double
// quantised") straight from where they are stored - this GPU's memory or a PEER's shard of the flat
// packed array, through plain loads over NVLink - expand them with the 16-entry code book and write
// 16-bit values directly into the 128-byte-swizzled shared-memory operand tile that tcgen05.mma reads
// (generic-proxy stores, then fence.proxy.async, then an mbarrier arrive).  The activation tiles come
// in by TMA; the LoRA update (xa = x A^T computed beforehand, Bl = s*B) is accumulated by extra K blocks
// into the same tensor-memory accumulator.
//
// This is the kernel for FEW ROWS (M up to a few hundred: one or two 128-row tiles), where every weight
// byte is used once and the job is to stream 4-bit data at memory / link speed.  With thousands of rows
// each weight tile would be expanded again by every row tile; there the framework dequantises once into
// an L2-resident 16-bit buffer and runs gemm_tcgen05.cu.
//
// The same kernel serves GPTQ int4 weights (template parameter GPTQ): qweight [K/8, N] int32 holds eight consecutive
// k of one output column per word, which is exactly one 16-byte chunk of the K-major operand row; scales [K/g, N]
// and packed zero points [K/g, N/8] are per group of g input features (g a multiple of 64, groups in order).
// A dequant warp reads 32 neighbouring columns per load (coalesced) and writes 32 swizzled rows.  Reference
// counterpart: the fused dequantise-and-matmul Triton kernels of
// fms_acceleration_peft/gptqmodel/nn_modules/triton_utils/kernels.py:105-201.
//
// Reference counterparts (NF4 / FP4): bitsandbytes' cgemm_4bit_inference_naive / dequantize + matmul as called from
// fms_acceleration_foak/fused_ops/unsloth_lora/utils.py:119-136,190-203,262-279 and the NCCL all-gather
// of the FSDP-sharded packed parameter that precedes them.
//
// Roles (320 threads): warp 0 TMA producer (x, and xa/Bl for the LoRA blocks), warp 1 MMA issuer,
// warps 2-9 dequantise W tiles and afterwards run the epilogue.  4-stage ring.  Every wait is bounded.
#include "common.cuh"

namespace fmsb {

constexpr int Q4_BM = 128;
constexpr int Q4_BK = 64;
constexpr int Q4_STAGES = 4;
constexpr int Q4_MAX_RANKS = 16;
constexpr int Q4_DQ_THREADS = 256;  // 8 dequant warps: two per scheduler, so table look-ups of one hide behind the other

struct Q4Params {
  int M, N, K;
  int kblocks1, kblocks2;
  const uint8_t* shard[Q4_MAX_RANKS];  // flat packed array [N*K/2] split into `world` equal shards
  long long shard_bytes;
  int world;
  const float* absmax;       // [N*K/64] fp32, or null when double quantised
  const uint8_t* absmax_q;   // [N*K/64] codes into code256
  const float* code256;      // [256]
  const float* absmax2;      // [N*K/64/256]
  float offset;
  float code16[16];
  // GPTQ int4 (template parameter GPTQ = 1): W[k, n] = scales[g, n] * (q[k, n] - (zero[g, n] + zero_offset)), g = k / group
  const uint32_t* gq_weight;  // [K/8, N]
  const uint16_t* gq_scales;  // [K/group, N] in the compute format
  const uint32_t* gq_zeros;   // [K/group, N/8]
  int gq_group;               // input features per group: a multiple of 64
  int gq_zero_offset;
  void* D;
  long long ldd;
  float alpha;
  int fmt;  // 0 fp16, 1 bf16
  int* status;
};

template <int BN>
struct Q4Cfg {
  static constexpr int kABytes = Q4_BM * Q4_BK * 2;
  static constexpr int kBBytes = 128 * Q4_BK * 2;  // room for the widest tile (the LoRA B tile is BN rows too)
  static constexpr int kSmemBytes = Q4_STAGES * (kABytes + kBBytes) + 1024 + 256;
};

// Streaming loads of packed weights.  A thread's bytes of one K block are a 16- or 32-byte piece of a row whose
// neighbours along K are needed a few blocks later: ask L2 for the whole 256-byte neighbourhood on a miss so that
// DRAM is read in long bursts and the following K blocks of the row hit in L2.
__device__ __forceinline__ uint4 q4_ld16(const uint8_t* p) {
  uint4 v;
  asm volatile("ld.global.L2::256B.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 q4_ld8(const uint8_t* p) {
  uint2 v;
  asm volatile("ld.global.L2::256B.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

__device__ __forceinline__ uint32_t q4_ld4(const uint8_t* p) {
  uint32_t v;
  asm volatile("ld.global.L2::256B.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

__device__ __forceinline__ uint32_t q4_pack2(float a, float b, int fmt) {
  return fmt == 1 ? pack_bf16x2(a, b) : pack_f16x2(a, b);
}

template <int BN, int GPTQ>
__global__ void __launch_bounds__(64 + Q4_DQ_THREADS, 1)
gemm_q4_fused_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmXa,
                     const __grid_constant__ CUtensorMap tmBl, const Q4Params p) {
  using Cfg = Q4Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  auto sA = [&](int s) { return base + s * (Cfg::kABytes + Cfg::kBBytes); };
  auto sB = [&](int s) { return base + s * (Cfg::kABytes + Cfg::kBBytes) + Cfg::kABytes; };
  const uint32_t bars = base + Q4_STAGES * (Cfg::kABytes + Cfg::kBBytes);
  auto bar_a_full = [&](int s) { return bars + 8u * s; };
  auto bar_b_full = [&](int s) { return bars + 8u * (Q4_STAGES + s); };
  auto bar_empty = [&](int s) { return bars + 8u * (2 * Q4_STAGES + s); };
  const uint32_t bar_acc = bars + 8u * (3 * Q4_STAGES);
  const uint32_t holder = bar_acc + 8u;
  __shared__ float s_code[16];
  __shared__ float s_code256[256];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN;
  const int m0 = blockIdx.y * Q4_BM;
  const int kbt = p.kblocks1 + p.kblocks2;

  if (threadIdx.x < 16) s_code[threadIdx.x] = p.code16[threadIdx.x];
  if (p.absmax_q != nullptr)
    for (int i = threadIdx.x; i < 256; i += blockDim.x) s_code256[i] = p.code256[i];
  if (warp == 1 && lane == 0) {
    for (int s = 0; s < Q4_STAGES; ++s) {
      mbar_init(bar_a_full(s), 1);
      mbar_init(bar_b_full(s), Q4_DQ_THREADS / 32);  // one arrival per dequant warp
      mbar_init(bar_empty(s), 1);
    }
    mbar_init(bar_acc, 1);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(holder, 128);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem) : "r"(holder));

  if (warp == 0) {
    if (lane == 0) {
      for (int kb = 0; kb < kbt; ++kb) {
        const int s = kb % Q4_STAGES;
        if (!mbar_wait(bar_empty(s), ((kb / Q4_STAGES) & 1) ^ 1u, p.status, kTimeoutProducer)) break;
        if (kb < p.kblocks1) {
          mbar_expect_tx(bar_a_full(s), Cfg::kABytes);
          tma_load_2d(sA(s), &tmX, bar_a_full(s), kb * Q4_BK, m0);
        } else {
          const int k2 = (kb - p.kblocks1) * Q4_BK;
          mbar_expect_tx(bar_a_full(s), Cfg::kABytes + BN * Q4_BK * 2);
          tma_load_2d(sA(s), &tmXa, bar_a_full(s), k2, m0);
          tma_load_2d(sB(s), &tmBl, bar_a_full(s), k2, n0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(128, BN, p.fmt, 0, 0);
      bool ok = true;
      for (int kb = 0; kb < kbt && ok; ++kb) {
        const int s = kb % Q4_STAGES;
        const uint32_t par = (kb / Q4_STAGES) & 1;
        if (!mbar_wait(bar_a_full(s), par, p.status, kTimeoutMma)) { ok = false; break; }
        if (kb < p.kblocks1 && !mbar_wait(bar_b_full(s), par, p.status, kTimeoutMma)) { ok = false; break; }
        tc_fence_after();
        const SmemDescBase da = make_smem_desc_base(sA(s), 16, 1024), db = make_smem_desc_base(sB(s), 16, 1024);
#pragma unroll
        for (int ks = 0; ks < Q4_BK / 16; ++ks)
          tc_mma_f16(tmem, smem_desc_at(da, ks * 32), smem_desc_at(db, ks * 32), idesc, (kb | ks) != 0);
        tc_commit(bar_empty(s));
      }
      if (ok) tc_commit(bar_acc);
    }
  } else {
    // ------------------------------------------------------------------ dequantise W tiles [BN rows x 64]
    constexpr int TPR = Q4_DQ_THREADS / BN;  // threads per weight row
    constexpr int EPT = Q4_BK / TPR;     // elements per thread and K block: 32, 16 or 8
    const int tid = threadIdx.x - 64;    // 0..Q4_DQ_THREADS-1
    // NF4 / FP4: a row's bytes are contiguous, neighbouring threads share a row.  GPTQ: a word's neighbours in memory
    // are the same k of the next columns, so neighbouring threads take neighbouring rows of the tile.
    const int r = GPTQ ? tid % BN : tid / TPR;     // row inside the tile
    const int part = GPTQ ? tid / BN : tid % TPR;  // which slice of the row's 64 elements
    const int n = n0 + r;
    const bool row_ok = n < p.N;
    bool ok = true;
    // The packed bytes and the scale code of the next PF K blocks are kept in flight in registers: a weight
    // byte is used exactly once, so the loop is a stream and its speed is set by how many loads are outstanding.
    constexpr int PF = 8;
    constexpr int WPT = EPT / 8;  // 32-bit words (= 16-byte output chunks) per thread and K block
    uint32_t w[PF][WPT];
    uint32_t sq[PF];   // 8-bit code of the block scale (double quantised) or the fp32 scale's bits
    float s2[PF];      // second-level scale of the block
    auto issue = [&](int slot, int kb) {
#pragma unroll
      for (int i = 0; i < WPT; ++i) w[slot][i] = 0u;
      sq[slot] = 0u;
      s2[slot] = 0.f;
      if (!row_ok || kb >= p.kblocks1) return;
      if constexpr (GPTQ) {
        const int g = (kb * Q4_BK) / p.gq_group;
        const uint16_t sc = p.gq_scales[(long long)g * p.N + n];
        sq[slot] = __float_as_uint(p.fmt == 1 ? __uint_as_float((uint32_t)sc << 16) : __half2float(__ushort_as_half(sc)));
        const uint32_t zw = p.gq_zeros[(long long)g * (p.N >> 3) + (n >> 3)];
        s2[slot] = (float)(int)(((zw >> ((n & 7) * 4)) & 15u) + p.gq_zero_offset);
#pragma unroll
        for (int i = 0; i < WPT; ++i)
          w[slot][i] = q4_ld4(reinterpret_cast<const uint8_t*>(p.gq_weight + (long long)(kb * 8 + part * WPT + i) * p.N + n));
        return;
      }
      const long long e0 = (long long)n * p.K + (long long)kb * Q4_BK;  // first element of the 64-block
      const long long blk = e0 >> 6;
      if (p.absmax_q != nullptr) {
        sq[slot] = p.absmax_q[blk];
        s2[slot] = p.absmax2[blk >> 8];
      } else {
        sq[slot] = __float_as_uint(p.absmax[blk]);
      }
      const long long byte_off = (e0 >> 1) + part * (EPT / 2);
      const uint8_t* src = p.shard[byte_off / p.shard_bytes] + (byte_off % p.shard_bytes);
      if constexpr (EPT == 32) {
        const uint4 u0 = q4_ld16(src);
        w[slot][0] = u0.x; w[slot][1] = u0.y; w[slot][2] = u0.z; w[slot][3] = u0.w;
      } else if constexpr (EPT == 16) {
        const uint2 u0 = q4_ld8(src);
        w[slot][0] = u0.x; w[slot][1] = u0.y;
      } else {
        w[slot][0] = q4_ld4(src);
      }
    };
#pragma unroll
    for (int j = 0; j < PF; ++j) issue(j, j);
    for (int kb0 = 0; kb0 < p.kblocks1 && ok; kb0 += PF) {
#pragma unroll
      for (int j = 0; j < PF; ++j) {
        const int kb = kb0 + j;
        if (kb >= p.kblocks1 || !ok) break;
        const int s = kb % Q4_STAGES;
        const float scale = GPTQ ? __uint_as_float(sq[j])
                                 : (p.absmax_q != nullptr ? s_code256[sq[j]] * s2[j] + p.offset : __uint_as_float(sq[j]));
        const float zs = GPTQ ? -s2[j] * scale : 0.f;  // (q - z) * s = q * s - z * s
        if (!mbar_wait(bar_empty(s), ((kb / Q4_STAGES) & 1) ^ 1u, p.status, kTimeoutDequant)) { ok = false; break; }
        // one 32-bit word = 8 values = one 16-byte chunk of the swizzled row
#pragma unroll
        for (int i = 0; i < WPT; ++i) {
          uint32_t o[4];
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            const uint32_t byte = (w[j][i] >> (8 * b)) & 0xffu;
            if constexpr (GPTQ)  // low nibble first: the smaller k
              o[b] = q4_pack2(fmaf((float)(byte & 15u), scale, zs), fmaf((float)(byte >> 4), scale, zs), p.fmt);
            else
              o[b] = q4_pack2(s_code[byte >> 4] * scale, s_code[byte & 15] * scale, p.fmt);
          }
          const int chunk = part * WPT + i;  // 0..7 within the row
          const uint32_t addr = sB(s) + static_cast<uint32_t>(r * 128 + ((chunk ^ (r & 7)) << 4));
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(o[0]), "r"(o[1]), "r"(o[2]),
                       "r"(o[3])
                       : "memory");
        }
        fence_proxy_async_smem();  // every writer orders its own stores before the tensor core's reads
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_b_full(s));
        issue(j, kb + PF);
      }
    }
    // ------------------------------------------------------------------ epilogue
    if (ok && mbar_wait(bar_acc, 0, p.status, kTimeoutEpilogue)) {
      tc_fence_after();
      const int q = warp & 3;
      const int row = m0 + q * 32 + lane;
      const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
      // two warps share a lane quarter: warps 2-5 take the even 32-column groups, warps 6-9 the odd ones
#pragma unroll 1
      for (int c = (warp - 2) >> 2; c < BN / 32; c += 2) {
        uint32_t v[32];
        tmem_ld_32x32(tmem + lane_addr + c * 32, v);
        tmem_ld_wait();
        if (row < p.M) {
          uint16_t* dst = reinterpret_cast<uint16_t*>(p.D) + (long long)row * p.ldd + n0 + c * 32;
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            if (n0 + c * 32 + i < p.N) {  // N % 8 == 0: a group of 8 columns is in range as a whole
              uint4 u;
              u.x = q4_pack2(__uint_as_float(v[i]) * p.alpha, __uint_as_float(v[i + 1]) * p.alpha, p.fmt);
              u.y = q4_pack2(__uint_as_float(v[i + 2]) * p.alpha, __uint_as_float(v[i + 3]) * p.alpha, p.fmt);
              u.z = q4_pack2(__uint_as_float(v[i + 4]) * p.alpha, __uint_as_float(v[i + 5]) * p.alpha, p.fmt);
              u.w = q4_pack2(__uint_as_float(v[i + 6]) * p.alpha, __uint_as_float(v[i + 7]) * p.alpha, p.fmt);
              *reinterpret_cast<uint4*>(dst + i) = u;
            }
          }
        }
      }
    }
  }
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 128);
  }
}

}  // namespace fmsb

using namespace fmsb;

template <int BN, int GPTQ>
static int q4_launch(const CUtensorMap& tx, const CUtensorMap& txa, const CUtensorMap& tbl, const Q4Params& p,
                     cudaStream_t stream) {
  static bool cfg = false;
  if (!cfg) {
    cudaError_t e = cudaFuncSetAttribute(gemm_q4_fused_kernel<BN, GPTQ>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Q4Cfg<BN>::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    cfg = true;
  }
  dim3 grid((p.N + BN - 1) / BN, (p.M + Q4_BM - 1) / Q4_BM);
  gemm_q4_fused_kernel<BN, GPTQ><<<grid, 64 + Q4_DQ_THREADS, Q4Cfg<BN>::kSmemBytes, stream>>>(tx, txa, tbl, p);
  return (int)cudaGetLastError();
}

static int q4_maps(CUtensorMap* tx, CUtensorMap* txa, CUtensorMap* tbl, const void* x, long long ldx, const void* xa,
                   long long ldxa, const void* bl, long long ldbl, int r2, int M, int N, int K, int bn) {
  using namespace fmsb_host;
  int rc;
  if ((rc = make_tmap_2d_16b(tx, x, M, K, ldx, 128, 64))) return rc;
  if (xa != nullptr) {
    if ((rc = make_tmap_2d_16b(txa, xa, M, r2, ldxa, 128, 64))) return rc;
    if ((rc = make_tmap_2d_16b(tbl, bl, N, r2, ldbl, bn, 64))) return rc;
  } else {
    *txa = *tx;
    *tbl = *tx;
  }
  return 0;
}

// x [M, K] (ldx), packed shards (world pointers, shard_bytes each; world = 1: one local pointer), scales either
// `absmax` (fp32 per 64-block) or the double-quantised triple (absmax_q, code256, absmax2, offset); code16 = the
// 16-entry NF4 / FP4 table (host pointer); optional LoRA pair xa [M, R] (ldxa), bl [N, R] (ldbl), R = r2;
// y [M, N] (ldy).  K % 64 == 0, N % 8 == 0, leading dimensions % 8 == 0, bn in {32, 64, 128}.
extern "C" int fmsb_gemm_q4_fused(const void* x, long long ldx, void* const* packed_shards, long long shard_bytes,
                                  int world, const float* absmax, const void* absmax_q, const float* code256,
                                  const float* absmax2, float offset, const float* code16_host, const void* xa,
                                  long long ldxa, const void* bl, long long ldbl, int r2, void* y, long long ldy,
                                  float alpha, int M, int N, int K, int fmt, int bn, int* status,
                                  cudaStream_t stream) {
  using namespace fmsb_host;
  if (M <= 0 || N <= 0) return 0;
  if (K % 64 != 0 || N % 8 != 0 || (ldx % 8) || (ldy % 8) || world < 1 || world > Q4_MAX_RANKS) return -2;
  if (shard_bytes % 32 != 0 || shard_bytes * world < (long long)N * K / 2) return -2;
  if ((absmax == nullptr) == (absmax_q == nullptr)) return -2;
  if (xa != nullptr && ((ldxa % 8) || (ldbl % 8) || r2 <= 0 || bl == nullptr)) return -2;
  Q4Params p{};
  p.M = M; p.N = N; p.K = K;
  p.kblocks1 = K / 64;
  p.kblocks2 = xa != nullptr ? (r2 + 63) / 64 : 0;
  for (int i = 0; i < world; ++i) p.shard[i] = (const uint8_t*)packed_shards[i];
  p.shard_bytes = shard_bytes; p.world = world;
  p.absmax = absmax; p.absmax_q = (const uint8_t*)absmax_q; p.code256 = code256; p.absmax2 = absmax2; p.offset = offset;
  for (int i = 0; i < 16; ++i) p.code16[i] = code16_host[i];
  p.D = y; p.ldd = ldy; p.alpha = alpha; p.fmt = fmt; p.status = status;
  CUtensorMap tx, txa, tbl;
  if (int rc = q4_maps(&tx, &txa, &tbl, x, ldx, xa, ldxa, bl, ldbl, r2, M, N, K, bn)) return rc;
  if (bn == 128) return q4_launch<128, 0>(tx, txa, tbl, p, stream);
  if (bn == 64) return q4_launch<64, 0>(tx, txa, tbl, p, stream);
  if (bn == 32) return q4_launch<32, 0>(tx, txa, tbl, p, stream);
  return -2;
}

// GPTQ int4 form: y [M, N] = alpha * (x [M, K] . W [K, N] + xa [M, R] . bl [N, R]^T) with W given as qweight [K/8, N]
// (int32, eight k per word), scales [K/group, N] (16-bit, the format of x), qzeros [K/group, N/8] (int32) and
// zero_offset (1 for checkpoints that store the zero point minus one).  Groups follow the input features in order
// (no activation reordering) and group % 64 == 0; K % 64 == 0, N % 8 == 0; bn in {32, 64, 128}.
extern "C" int fmsb_gemm_gptq_fused(const void* x, long long ldx, const void* qweight, const void* scales,
                                    const void* qzeros, int group, int zero_offset, const void* xa, long long ldxa,
                                    const void* bl, long long ldbl, int r2, void* y, long long ldy, float alpha, int M,
                                    int N, int K, int fmt, int bn, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K % 64 != 0 || N % 8 != 0 || (ldx % 8) || (ldy % 8) || group <= 0 || group % 64 != 0 || K % group != 0) return -2;
  if (qweight == nullptr || scales == nullptr || qzeros == nullptr) return -2;
  if (xa != nullptr && ((ldxa % 8) || (ldbl % 8) || r2 <= 0 || bl == nullptr)) return -2;
  Q4Params p{};
  p.M = M; p.N = N; p.K = K;
  p.kblocks1 = K / 64;
  p.kblocks2 = xa != nullptr ? (r2 + 63) / 64 : 0;
  p.world = 1;
  p.gq_weight = (const uint32_t*)qweight; p.gq_scales = (const uint16_t*)scales; p.gq_zeros = (const uint32_t*)qzeros;
  p.gq_group = group; p.gq_zero_offset = zero_offset;
  p.D = y; p.ldd = ldy; p.alpha = alpha; p.fmt = fmt; p.status = status;
  CUtensorMap tx, txa, tbl;
  if (int rc = q4_maps(&tx, &txa, &tbl, x, ldx, xa, ldxa, bl, ldbl, r2, M, N, K, bn)) return rc;
  if (bn == 128) return q4_launch<128, 1>(tx, txa, tbl, p, stream);
  if (bn == 64) return q4_launch<64, 1>(tx, txa, tbl, p, stream);
  if (bn == 32) return q4_launch<32, 1>(tx, txa, tbl, p, stream);
  return -2;
}
