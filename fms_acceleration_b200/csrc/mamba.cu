// Mamba2 (state-space duality) support kernels for sm_100a: depthwise causal conv1d + SiLU and the inter-chunk
// state recurrence (with an initial state and a returned final state, which is what context parallelism hands
// from rank to rank).  The decay / mask construction and the element-wise passes are in mamba_scan.cu.
//
// The reference delegates all of this to the external mamba_ssm package
// (fms_acceleration_mcp/utils/utils.py:17-24,64-80); the math below is the chunked SSD algorithm:
//   h_t = exp(dt_t A) h_{t-1} + dt_t x_t (x) B_t,   y_t = C_t . h_t + D x_t
// with chunks of Q tokens, L_t the within-chunk inclusive cumulative sum of dt_t A:
//   intra-chunk  y_t += sum_{s<=t} (C_t.B_s) exp(L_t - L_s) dt_s x_s     (G = CB o decay, then G.X on tcgen05)
//   chunk state  S_c  = sum_s exp(L_end - L_s) dt_s x_s (x) B_s            (batched tcgen05 GEMM)
//   recurrence   H_{c+1} = exp(L_end,c) H_c + S_c                          (this file)
//   inter-chunk  y_t += exp(L_t) C_t . H_c                                 (batched tcgen05 GEMM)
#include "common.cuh"

namespace fmsb {

__device__ __forceinline__ float silu_f(float v) { return v * __fdividef(1.f, 1.f + __expf(-v)); }

// ---------------------------------------------------------------------------------------------------------
// Depthwise causal conv (4 taps) + SiLU on packed rows x [T, C].  A thread owns 8 neighbouring channels (one
// 16-byte vector) and walks down a run of rows with the last three input rows in registers, so every input
// element is read once.  seq_start[t] = first row of the sequence that contains row t (packed sequences do not
// leak into each other); rows before row 0 read `halo` ([3, C], the last rows of the previous context-parallel
// rank) when the sequence starts at row 0, else zero.
//   y[t, c] = silu(bias[c] + sum_j w[c, j] * xin[t - 3 + j, c])
// ---------------------------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ void cv_unpack8(const uint4& u, float (&f)[8]);
template <>
__device__ __forceinline__ void cv_unpack8<__nv_bfloat16>(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __bfloat1622float2(h[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}
template <>
__device__ __forceinline__ void cv_unpack8<__half>(const uint4& u, float (&f)[8]) {
  const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __half22float2(h[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}
template <typename T>
__device__ __forceinline__ uint4 cv_pack8(const float (&f)[8]);
template <>
__device__ __forceinline__ uint4 cv_pack8<__nv_bfloat16>(const float (&f)[8]) {
  return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}
template <>
__device__ __forceinline__ uint4 cv_pack8<__half>(const float (&f)[8]) {
  return make_uint4(pack_f16x2(f[0], f[1]), pack_f16x2(f[2], f[3]), pack_f16x2(f[4], f[5]), pack_f16x2(f[6], f[7]));
}

// taps of 8 channels: w is [C, 4], so the 32 values of a channel vector are contiguous
template <typename T>
__device__ __forceinline__ void cv_load_taps(const T* __restrict__ w, const T* __restrict__ bias, int c0,
                                             float (&wf)[4][8], float (&bf)[8]) {
  float tmp[4][8];
#pragma unroll
  for (int q = 0; q < 4; ++q) cv_unpack8<T>(*reinterpret_cast<const uint4*>(w + (long long)c0 * 4 + q * 8), tmp[q]);
#pragma unroll
  for (int ch = 0; ch < 8; ++ch)
#pragma unroll
    for (int j = 0; j < 4; ++j) wf[j][ch] = tmp[(ch * 4 + j) >> 3][(ch * 4 + j) & 7];
  if (bias != nullptr) {
    cv_unpack8<T>(*reinterpret_cast<const uint4*>(bias + c0), bf);
  } else {
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) bf[ch] = 0.f;
  }
}

// input row tt of a channel vector: x for tt >= 0, the halo (or zero) before row 0
template <typename T>
__device__ __forceinline__ void cv_load_row(const T* __restrict__ x, long long ldx, const T* __restrict__ halo, int C,
                                            int c0, int tt, int T_tokens, float (&f)[8]) {
  if (tt >= 0 && tt < T_tokens) {
    cv_unpack8<T>(*reinterpret_cast<const uint4*>(x + (long long)tt * ldx + c0), f);
  } else if (tt < 0 && tt >= -3 && halo != nullptr) {
    cv_unpack8<T>(*reinterpret_cast<const uint4*>(halo + (long long)(tt + 3) * C + c0), f);
  } else {
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) f[ch] = 0.f;
  }
}

constexpr int CONV_RT_FWD = 16;  // rows per thread, forward (3 extra row loads per run)
constexpr int CONV_RT = 32;      // rows per thread, backward (3 extra output rows per run)

// grid (ceil(C/8 / 128), ceil(T / CONV_RT_FWD)), block 128
template <typename T>
__global__ void __launch_bounds__(128) conv1d_fwd_kernel(const T* __restrict__ x, long long ldx, const T* __restrict__ w,
                                                         const T* __restrict__ bias, const T* __restrict__ halo,
                                                         const int* __restrict__ seq_start, T* __restrict__ y,
                                                         long long ldy, T* __restrict__ y2, long long ldy2, int split,
                                                         int T_tokens, int C) {
  const int cv = blockIdx.x * blockDim.x + threadIdx.x;
  if (cv * 8 >= C) return;
  const int c0 = cv * 8;
  // channels [0, split) go to y, the rest to y2 (the scan wants x dense and B|C apart)
  T* const yo = c0 < split ? y + c0 : y2 + (c0 - split);
  const long long ldo = c0 < split ? ldy : ldy2;
  const int t0 = blockIdx.y * CONV_RT_FWD, t1 = min(T_tokens, t0 + CONV_RT_FWD);
  float wf[4][8], bf[8], win[3][8];
  cv_load_taps<T>(w, bias, c0, wf, bf);
#pragma unroll
  for (int j = 0; j < 3; ++j) cv_load_row<T>(x, ldx, halo, C, c0, t0 - 3 + j, T_tokens, win[j]);
  // four rows per trip: their loads go out together, then the window slides over them
  for (int tb = t0; tb < t1; tb += 4) {
    uint4 raw[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (tb + u < t1) raw[u] = *reinterpret_cast<const uint4*>(x + (long long)(tb + u) * ldx + c0);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int t = tb + u;
      if (t >= t1) break;
      float cur[8], acc[8];
      cv_unpack8<T>(raw[u], cur);
      const int s0 = seq_start != nullptr ? seq_start[t] : 0;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        float a = bf[ch] + wf[3][ch] * cur[ch];
#pragma unroll
        for (int j = 0; j < 3; ++j)
          if (s0 == 0 || t - 3 + j >= s0) a += wf[j][ch] * win[j][ch];
        acc[ch] = silu_f(a);
      }
      *reinterpret_cast<uint4*>(yo + (long long)t * ldo) = cv_pack8<T>(acc);
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        win[0][ch] = win[1][ch];
        win[1][ch] = win[2][ch];
        win[2][ch] = cur[ch];
      }
    }
  }
}

template <typename T>
__device__ __forceinline__ void cv_unpack4(const uint2& u, float (&f)[4]);
template <>
__device__ __forceinline__ void cv_unpack4<__nv_bfloat16>(const uint2& u, float (&f)[4]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
  const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
template <>
__device__ __forceinline__ void cv_unpack4<__half>(const uint2& u, float (&f)[4]) {
  const __half2* h = reinterpret_cast<const __half2*>(&u);
  const float2 a = __half22float2(h[0]), b = __half22float2(h[1]);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
template <typename T>
__device__ __forceinline__ uint2 cv_pack4(const float (&f)[4]);
template <>
__device__ __forceinline__ uint2 cv_pack4<__nv_bfloat16>(const float (&f)[4]) {
  return make_uint2(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]));
}
template <>
__device__ __forceinline__ uint2 cv_pack4<__half>(const float (&f)[4]) {
  return make_uint2(pack_f16x2(f[0], f[1]), pack_f16x2(f[2], f[3]));
}
template <typename T>
__device__ __forceinline__ void cv_load_row4(const T* __restrict__ x, long long ldx, const T* __restrict__ halo, int C,
                                             int c0, int tt, int T_tokens, float (&f)[4]) {
  if (tt >= 0 && tt < T_tokens) {
    cv_unpack4<T>(*reinterpret_cast<const uint2*>(x + (long long)tt * ldx + c0), f);
  } else if (tt < 0 && tt >= -3 && halo != nullptr) {
    cv_unpack4<T>(*reinterpret_cast<const uint2*>(halo + (long long)(tt + 3) * C + c0), f);
  } else {
    f[0] = f[1] = f[2] = f[3] = 0.f;
  }
}

// Backward.  A thread owns input rows [t0, t0 + CONV_RT) of 4 channels (the per-thread state is four times the
// forward's, so the vector is halved) and walks over the OUTPUT rows to in [t0, t0 + CONV_RT + 3) that read
// them, recomputing pre[to] from the sliding window of inputs:
//   d[to]      = dy[to] * silu'(pre[to])
//   dx[t]      = sum_j w[j] d[t + 3 - j]                       (outputs of the same sequence)
//   dw[c, j]  += d[to] * xin[to - 3 + j],  db[c] += d[to]      (own output rows only; reduced over the block's
//                                                              row groups in shared memory, then one atomic each)
//   dhalo[r]   = gradient of the three rows before row 0 (written by the threads that own row 0)
// grid (ceil(C/4 / 64), ceil(T / (CONV_RT * 4))), block (64, 4); dw32 [C, 4] and db32 [C] fp32, zeroed by the caller.
template <typename T>
__global__ void __launch_bounds__(256, 2) conv1d_bwd_kernel(const T* __restrict__ dy, long long lddy,
                                                            const T* __restrict__ dy2, long long lddy2, int split,
                                                            const T* __restrict__ x, long long ldx,
                                                            const T* __restrict__ w, const T* __restrict__ bias,
                                                            const T* __restrict__ halo, const int* __restrict__ seq_start,
                                                            T* __restrict__ dx, long long lddx, T* __restrict__ dhalo,
                                                            float* __restrict__ dw32, float* __restrict__ db32,
                                                            int T_tokens, int C) {
  __shared__ float red[4][20][64];
  const int cv = blockIdx.x * 64 + threadIdx.x;
  const bool live = cv * 4 < C;
  const int c0 = cv * 4;
  const int t0 = (blockIdx.y * 4 + threadIdx.y) * CONV_RT;
  const int own_end = min(T_tokens, t0 + CONV_RT);
  const int to_end = min(T_tokens, t0 + CONV_RT + 3);
  float dwa[4][4], dba[4];
#pragma unroll
  for (int ch = 0; ch < 4; ++ch) {
    dba[ch] = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) dwa[j][ch] = 0.f;
  }
  if (live && t0 < T_tokens) {
    float wf[4][4], bf[4], win[3][4], dxa[4][4];
    {
      float tmp[2][8];
      cv_unpack8<T>(*reinterpret_cast<const uint4*>(w + (long long)c0 * 4), tmp[0]);
      cv_unpack8<T>(*reinterpret_cast<const uint4*>(w + (long long)c0 * 4 + 8), tmp[1]);
#pragma unroll
      for (int ch = 0; ch < 4; ++ch)
#pragma unroll
        for (int j = 0; j < 4; ++j) wf[j][ch] = tmp[(ch * 4 + j) >> 3][(ch * 4 + j) & 7];
      if (bias != nullptr) cv_unpack4<T>(*reinterpret_cast<const uint2*>(bias + c0), bf);
      else bf[0] = bf[1] = bf[2] = bf[3] = 0.f;
    }
#pragma unroll
    for (int j = 0; j < 3; ++j) cv_load_row4<T>(x, ldx, halo, C, c0, t0 - 3 + j, T_tokens, win[j]);
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) dxa[j][ch] = 0.f;
    // output gradient of channels [0, split) comes from dy, of the rest from dy2
    const T* const gy = c0 < split ? dy + c0 : dy2 + (c0 - split);
    const long long ldg = c0 < split ? lddy : lddy2;
    // two output rows per trip; the next trip's four loads are issued before this trip's arithmetic
    uint2 nx[2], ng[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      nx[u] = ng[u] = make_uint2(0u, 0u);
      if (t0 + u < to_end) {
        nx[u] = *reinterpret_cast<const uint2*>(x + (long long)(t0 + u) * ldx + c0);
        ng[u] = *reinterpret_cast<const uint2*>(gy + (long long)(t0 + u) * ldg);
      }
    }
    for (int tb = t0; tb < to_end; tb += 2) {
      uint2 cx[2], cg[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        cx[u] = nx[u];
        cg[u] = ng[u];
        const int tn = tb + 2 + u;
        if (tn < to_end) {
          nx[u] = *reinterpret_cast<const uint2*>(x + (long long)tn * ldx + c0);
          ng[u] = *reinterpret_cast<const uint2*>(gy + (long long)tn * ldg);
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int to = tb + u;
        if (to >= to_end) break;
        float cur[4], g[4];
        cv_unpack4<T>(cx[u], cur);
        cv_unpack4<T>(cg[u], g);
        const int s0 = seq_start != nullptr ? seq_start[to] : 0;
        const bool own = to < own_end;
        bool valid[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) valid[j] = (s0 == 0) || (to - 3 + j >= s0);
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          float p = bf[ch] + wf[3][ch] * cur[ch];
#pragma unroll
          for (int j = 0; j < 3; ++j)
            if (valid[j]) p += wf[j][ch] * win[j][ch];
          const float sg = __fdividef(1.f, 1.f + __expf(-p));
          const float d = g[ch] * sg * (1.f + p * (1.f - sg));
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (valid[j]) dxa[j][ch] += wf[j][ch] * d;
          if (own) {
            dba[ch] += d;
#pragma unroll
            for (int j = 0; j < 3; ++j)
              if (valid[j]) dwa[j][ch] += d * win[j][ch];
            dwa[3][ch] += d * cur[ch];
          }
        }
        // row to - 3 has now seen its four outputs
        const int r = to - 3;
        if (r >= t0 && r < own_end) {
          *reinterpret_cast<uint2*>(dx + (long long)r * lddx + c0) = cv_pack4<T>(dxa[0]);
        } else if (r < 0 && t0 == 0 && dhalo != nullptr) {
          *reinterpret_cast<uint2*>(dhalo + (long long)(r + 3) * C + c0) = cv_pack4<T>(dxa[0]);
        }
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          dxa[0][ch] = dxa[1][ch];
          dxa[1][ch] = dxa[2][ch];
          dxa[2][ch] = dxa[3][ch];
          dxa[3][ch] = 0.f;
          win[0][ch] = win[1][ch];
          win[1][ch] = win[2][ch];
          win[2][ch] = cur[ch];
        }
      }
    }
    // rows that no later output reads (the end of the tensor, or fewer than three rows in all)
#pragma unroll
    for (int k = 0; k < 3; ++k) {
      const int r = to_end - 3 + k;
      if (r >= t0 && r < own_end && r + 3 >= to_end) {
        *reinterpret_cast<uint2*>(dx + (long long)r * lddx + c0) = cv_pack4<T>(dxa[k]);
      } else if (r < 0 && t0 == 0 && dhalo != nullptr) {
        *reinterpret_cast<uint2*>(dhalo + (long long)(r + 3) * C + c0) = cv_pack4<T>(dxa[k]);
      }
    }
  }
  // tap and bias gradients: sum the block's four row groups, then one atomic per value
#pragma unroll
  for (int ch = 0; ch < 4; ++ch) {
#pragma unroll
    for (int j = 0; j < 4; ++j) red[threadIdx.y][ch * 4 + j][threadIdx.x] = dwa[j][ch];
    red[threadIdx.y][16 + ch][threadIdx.x] = dba[ch];
  }
  __syncthreads();
  if (threadIdx.y == 0 && live) {
#pragma unroll 4
    for (int k = 0; k < 20; ++k) {
      const float v = red[0][k][threadIdx.x] + red[1][k][threadIdx.x] + red[2][k][threadIdx.x] + red[3][k][threadIdx.x];
      if (k < 16) atomicAdd(dw32 + (long long)c0 * 4 + k, v);
      else if (db32 != nullptr) atomicAdd(db32 + c0 + (k - 16), v);
    }
  }
}

// Inter-chunk recurrence.  S [nc, nh, P*N] fp32 chunk states, Ltot [nc, nh]; h0 [nh, P*N] fp32 or null.
//   Hprev[c] (state entering chunk c, written in 16-bit for the GEMM and optionally fp32) and hT = state after the last.
template <typename T>
__global__ void ssd_state_fwd_kernel(const float* __restrict__ S, const float* __restrict__ Ltot,
                                     const float* __restrict__ h0, T* __restrict__ hprev, float* __restrict__ hT, int nc,
                                     int nh, int PN) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= (long long)nh * PN) return;
  const int h = (int)(idx / PN);
  float st = h0 != nullptr ? h0[idx] : 0.f;
  for (int c = 0; c < nc; ++c) {
    hprev[(long long)c * nh * PN + idx] = (T)st;
    st = __expf(Ltot[c * nh + h]) * st + S[(long long)c * nh * PN + idx];
  }
  hT[idx] = st;
}

// Reverse recurrence: given dHprev_direct[c] (gradient reaching the state that ENTERS chunk c through the
// inter-chunk output term) and dhT, produce dS[c] = total gradient of the state leaving chunk c (16-bit, the
// operand of the two GEMMs that follow), the gradient of the initial state dh0, and
// dLtot[c, h] += sum over the state of dstate_after[c] * exp(Ltot) * Hprev[c]  (dLtot zeroed by the caller; one
// atomic per warp when the warp's lanes share a head, else one per lane).
template <typename T>
__global__ void ssd_state_bwd_kernel(const float* __restrict__ dhprev_direct, const float* __restrict__ dhT,
                                     const float* __restrict__ Ltot, const T* __restrict__ hprev, T* __restrict__ dS,
                                     float* __restrict__ dh0, float* __restrict__ dLtot, int nc, int nh, int PN) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long total = (long long)nh * PN;
  const bool live = idx < total;
  const int h = live ? (int)(idx / PN) : -1;
  const int lane = threadIdx.x & 31;
  // the warp shares one head iff its first and last lane do (idx is consecutive within the warp)
  const int h_first = __shfl_sync(0xffffffffu, h, 0), h_last = __shfl_sync(0xffffffffu, h, 31);
  const bool uniform = h_first == h_last && h_first >= 0;
  float d_after = (live && dhT != nullptr) ? dhT[idx] : 0.f;  // gradient of the state leaving chunk c
  for (int c = nc - 1; c >= 0; --c) {
    float part = 0.f;
    if (live) {
      const long long o = (long long)c * nh * PN + idx;
      dS[o] = (T)d_after;
      const float e = __expf(Ltot[c * nh + h]);
      part = d_after * e * (float)hprev[o];
      d_after = e * d_after + (dhprev_direct != nullptr ? dhprev_direct[o] : 0.f);
    }
    if (uniform) {
#pragma unroll
      for (int m = 16; m > 0; m >>= 1) part += __shfl_xor_sync(0xffffffffu, part, m);
      if (lane == 0) atomicAdd(dLtot + c * nh + h_first, part);
    } else if (live) {
      atomicAdd(dLtot + c * nh + h, part);
    }
  }
  if (live && dh0 != nullptr) dh0[idx] = d_after;
}

}  // namespace fmsb

using namespace fmsb;

static bool conv_shape_ok(const void* p, long long ld, int C) {
  return C % 8 == 0 && ld % 8 == 0 && (reinterpret_cast<uintptr_t>(p) & 15) == 0;
}

// y2/ldy2/split: channels [split, C) are written to y2 (row step ldy2); pass y2 = nullptr for one output.
extern "C" int fmsb_conv1d_fwd(const void* x, long long ldx, const void* w, const void* bias, const void* halo,
                               const int* seq_start, void* y, long long ldy, void* y2, long long ldy2, int split, int T,
                               int C, int K, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (y2 == nullptr) { split = C; y2 = y; ldy2 = ldy; }
  if (K != 4 || split % 8 != 0 || split < 0 || split > C || !conv_shape_ok(x, ldx, C) || !conv_shape_ok(y, ldy, C) ||
      !conv_shape_ok(y2, ldy2, C) || !conv_shape_ok(w, 8, C) || (bias != nullptr && !conv_shape_ok(bias, 8, C)) ||
      (halo != nullptr && !conv_shape_ok(halo, 8, C)))
    return -2;
  const dim3 grid((C / 8 + 127) / 128, (T + CONV_RT_FWD - 1) / CONV_RT_FWD);
  if (dtype == 1)
    conv1d_fwd_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>((const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, (const __nv_bfloat16*)bias, (const __nv_bfloat16*)halo, seq_start, (__nv_bfloat16*)y, ldy, (__nv_bfloat16*)y2, ldy2, split, T, C);
  else if (dtype == 0)
    conv1d_fwd_kernel<__half><<<grid, 128, 0, stream>>>((const __half*)x, ldx, (const __half*)w, (const __half*)bias, (const __half*)halo, seq_start, (__half*)y, ldy, (__half*)y2, ldy2, split, T, C);
  else
    return -2;
  return (int)cudaGetLastError();
}

extern "C" int fmsb_conv1d_bwd(const void* dy, long long lddy, const void* dy2, long long lddy2, int split,
                               const void* x, long long ldx, const void* w, const void* bias, const void* halo,
                               const int* seq_start, void* dx, long long lddx, void* dhalo, float* dw32, float* db32,
                               int T, int C, int K, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (dy2 == nullptr) { split = C; dy2 = dy; lddy2 = lddy; }
  if (K != 4 || split % 8 != 0 || split < 0 || split > C || !conv_shape_ok(x, ldx, C) || !conv_shape_ok(dy, lddy, C) ||
      !conv_shape_ok(dy2, lddy2, C) || !conv_shape_ok(dx, lddx, C) || !conv_shape_ok(w, 8, C) ||
      (bias != nullptr && !conv_shape_ok(bias, 8, C)) || (halo != nullptr && !conv_shape_ok(halo, 8, C)) ||
      (dhalo != nullptr && !conv_shape_ok(dhalo, 8, C)))
    return -2;
  const dim3 grid((C / 4 + 63) / 64, (T + CONV_RT * 4 - 1) / (CONV_RT * 4));
  const dim3 block(64, 4);
  if (dtype == 1)
    conv1d_bwd_kernel<__nv_bfloat16><<<grid, block, 0, stream>>>((const __nv_bfloat16*)dy, lddy, (const __nv_bfloat16*)dy2, lddy2, split, (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, (const __nv_bfloat16*)bias, (const __nv_bfloat16*)halo, seq_start, (__nv_bfloat16*)dx, lddx, (__nv_bfloat16*)dhalo, dw32, db32, T, C);
  else if (dtype == 0)
    conv1d_bwd_kernel<__half><<<grid, block, 0, stream>>>((const __half*)dy, lddy, (const __half*)dy2, lddy2, split, (const __half*)x, ldx, (const __half*)w, (const __half*)bias, (const __half*)halo, seq_start, (__half*)dx, lddx, (__half*)dhalo, dw32, db32, T, C);
  else
    return -2;
  return (int)cudaGetLastError();
}

extern "C" int fmsb_ssd_state_fwd(const float* S, const float* Ltot, const float* h0, void* hprev, float* hT, int nc,
                                  int nh, int PN, int dtype, cudaStream_t stream) {
  const long long total = (long long)nh * PN;
  if (total <= 0) return 0;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == 1) ssd_state_fwd_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(S, Ltot, h0, (__nv_bfloat16*)hprev, hT, nc, nh, PN);
  else if (dtype == 0) ssd_state_fwd_kernel<__half><<<blocks, 256, 0, stream>>>(S, Ltot, h0, (__half*)hprev, hT, nc, nh, PN);
  else return -2;
  return (int)cudaGetLastError();
}

extern "C" int fmsb_ssd_state_bwd(const float* dhprev_direct, const float* dhT, const float* Ltot, const void* hprev,
                                  void* dS, float* dh0, float* dLtot, int nc, int nh, int PN, int dtype,
                                  cudaStream_t stream) {
  const long long total = (long long)nh * PN;
  if (total <= 0) return 0;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == 1) ssd_state_bwd_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(dhprev_direct, dhT, Ltot, (const __nv_bfloat16*)hprev, (__nv_bfloat16*)dS, dh0, dLtot, nc, nh, PN);
  else if (dtype == 0) ssd_state_bwd_kernel<__half><<<blocks, 256, 0, stream>>>(dhprev_direct, dhT, Ltot, (const __half*)hprev, (__half*)dS, dh0, dLtot, nc, nh, PN);
  else return -2;
  return (int)cudaGetLastError();
}
