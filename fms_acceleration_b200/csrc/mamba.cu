// Mamba2 (state-space duality) support kernels for sm_100a: depthwise causal conv1d + SiLU, the decay /
// mask construction of the intra-chunk term, and the inter-chunk state recurrence (with an initial state and
// a returned final state, which is what context parallelism hands from rank to rank).
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

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + __expf(-v)); }

// y[t, c] = silu(bias[c] + sum_j w[c, j] * xin[t - (K-1) + j, c]); rows before a sequence start read `halo`
// ([K-1, C], the last K-1 rows of the previous context-parallel rank) or zero.  seq_start[t] = first row of the
// sequence that contains row t (so packed sequences do not leak into each other).
template <typename T, int K>
__global__ void conv1d_fwd_kernel(const T* __restrict__ x, long long ldx, const T* __restrict__ w,
                                  const T* __restrict__ bias, const T* __restrict__ halo, const int* __restrict__ seq_start,
                                  T* __restrict__ y, long long ldy, T* __restrict__ pre_out, int T_tokens, int C) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long total = (long long)T_tokens * C;
  if (idx >= total) return;
  const int c = (int)(idx % C);
  const int t = (int)(idx / C);
  const int s0 = seq_start != nullptr ? seq_start[t] : 0;
  float acc = bias != nullptr ? (float)bias[c] : 0.f;
#pragma unroll
  for (int j = 0; j < K; ++j) {
    const int tt = t - (K - 1) + j;
    float v = 0.f;
    if (tt >= s0) v = (float)x[(long long)tt * ldx + c];
    else if (halo != nullptr && s0 == 0 && tt < 0) v = (float)halo[(long long)(tt + K - 1) * C + c];
    acc += (float)w[c * K + j] * v;
  }
  if (pre_out != nullptr) pre_out[idx] = (T)acc;
  y[(long long)t * ldy + c] = (T)silu_f(acc);
}

// dpre = dy * silu'(pre);  dx[t, c] = sum_j w[c, j] * dpre[t + (K-1) - j, c] for rows of the same sequence.
// dhalo[r, c] (r in [0, K-1)) receives the gradient that belongs to the previous rank's last rows.
template <typename T, int K>
__global__ void conv1d_bwd_kernel(const T* __restrict__ dy, long long lddy, const T* __restrict__ pre,
                                  const T* __restrict__ w, const int* __restrict__ seq_start,
                                  const int* __restrict__ seq_end, T* __restrict__ dx, long long lddx,
                                  float* __restrict__ dpre_out, T* __restrict__ dhalo, int T_tokens, int C) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long total = (long long)(T_tokens + (K - 1)) * C;
  if (idx >= total) return;
  const int c = (int)(idx % C);
  const int t = (int)(idx / C) - (K - 1);  // t in [-(K-1), T): negative rows are the halo
  const int s_end = t >= 0 ? (seq_end != nullptr ? seq_end[t] : T_tokens) : (seq_end != nullptr ? seq_end[0] : T_tokens);
  float acc = 0.f;
#pragma unroll
  for (int j = 0; j < K; ++j) {
    const int to = t + (K - 1) - j;  // output row that read input row t through tap j
    if (to < 0 || to >= s_end) continue;
    if (t < 0 && (seq_start != nullptr && seq_start[to] != 0)) continue;
    const float p = (float)pre[(long long)to * C + c];
    const float sg = 1.f / (1.f + __expf(-p));
    const float d = (float)dy[(long long)to * lddy + c] * sg * (1.f + p * (1.f - sg));
    acc += (float)w[c * K + j] * d;
  }
  if (t >= 0) {
    dx[(long long)t * lddx + c] = (T)acc;
    if (dpre_out != nullptr) {
      const float p = (float)pre[(long long)t * C + c];
      const float sg = 1.f / (1.f + __expf(-p));
      dpre_out[(long long)t * C + c] = (float)dy[(long long)t * lddy + c] * sg * (1.f + p * (1.f - sg));
    }
  } else if (dhalo != nullptr) {
    dhalo[(long long)(t + K - 1) * C + c] = (T)acc;
  }
}

// G[c, h, t, s] = CB[c, g(h), t, s] * exp(L[c,t,h] - L[c,s,h]) * dt[c,s,h]  for s <= t, else 0
//   CB [nc*G, Q, Q], L/dt [nc*Q, nh] fp32, out [nc*nh, Q, Q]
template <typename T>
__global__ void ssd_make_g_kernel(const T* __restrict__ cb, const float* __restrict__ L, const float* __restrict__ dt,
                                  T* __restrict__ g, int nc, int nh, int G, int Q) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long total = (long long)nc * nh * Q * Q;
  if (idx >= total) return;
  const int s = (int)(idx % Q);
  const int t = (int)((idx / Q) % Q);
  const int h = (int)((idx / ((long long)Q * Q)) % nh);
  const int c = (int)(idx / ((long long)Q * Q * nh));
  float v = 0.f;
  if (s <= t) {
    const int gi = h / (nh / G);
    const float cbv = (float)cb[(((long long)c * G + gi) * Q + t) * Q + s];
    const float lt = L[((long long)c * Q + t) * nh + h], ls = L[((long long)c * Q + s) * nh + h];
    v = cbv * __expf(lt - ls) * dt[((long long)c * Q + s) * nh + h];
  }
  g[idx] = (T)v;
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
// inter-chunk output term) and dhT, produce dS[c] = total gradient of the state leaving chunk c, the gradient of
// the initial state dh0, and dLtot[c, h] = sum over the state of dstate_after[c] * exp(Ltot) * Hprev[c].
template <typename T>
__global__ void ssd_state_bwd_kernel(const float* __restrict__ dhprev_direct, const float* __restrict__ dhT,
                                     const float* __restrict__ Ltot, const T* __restrict__ hprev, float* __restrict__ dS,
                                     float* __restrict__ dh0, float* __restrict__ dLtot_partial, int nc, int nh, int PN) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= (long long)nh * PN) return;
  const int h = (int)(idx / PN);
  float d_after = dhT != nullptr ? dhT[idx] : 0.f;  // gradient of the state leaving chunk c
  for (int c = nc - 1; c >= 0; --c) {
    dS[(long long)c * nh * PN + idx] = d_after;
    const float e = __expf(Ltot[c * nh + h]);
    // contribution to dLtot is reduced over idx by the caller (one partial per element)
    dLtot_partial[(long long)c * nh * PN + idx] = d_after * e * (float)hprev[(long long)c * nh * PN + idx];
    d_after = e * d_after + dhprev_direct[(long long)c * nh * PN + idx];
  }
  if (dh0 != nullptr) dh0[idx] = d_after;
}

}  // namespace fmsb

using namespace fmsb;

extern "C" int fmsb_conv1d_fwd(const void* x, long long ldx, const void* w, const void* bias, const void* halo,
                               const int* seq_start, void* y, long long ldy, void* pre_out, int T, int C, int K, int dtype,
                               cudaStream_t stream) {
  if (T <= 0) return 0;
  if (K != 4) return -2;
  const long long total = (long long)T * C;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == 1)
    conv1d_fwd_kernel<__nv_bfloat16, 4><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, (const __nv_bfloat16*)bias, (const __nv_bfloat16*)halo, seq_start, (__nv_bfloat16*)y, ldy, (__nv_bfloat16*)pre_out, T, C);
  else if (dtype == 0)
    conv1d_fwd_kernel<__half, 4><<<blocks, 256, 0, stream>>>((const __half*)x, ldx, (const __half*)w, (const __half*)bias, (const __half*)halo, seq_start, (__half*)y, ldy, (__half*)pre_out, T, C);
  else
    return -2;
  return (int)cudaGetLastError();
}

extern "C" int fmsb_conv1d_bwd(const void* dy, long long lddy, const void* pre, const void* w, const int* seq_start,
                               const int* seq_end, void* dx, long long lddx, float* dpre_out, void* dhalo, int T, int C,
                               int K, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (K != 4) return -2;
  const long long total = (long long)(T + K - 1) * C;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == 1)
    conv1d_bwd_kernel<__nv_bfloat16, 4><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)dy, lddy, (const __nv_bfloat16*)pre, (const __nv_bfloat16*)w, seq_start, seq_end, (__nv_bfloat16*)dx, lddx, dpre_out, (__nv_bfloat16*)dhalo, T, C);
  else if (dtype == 0)
    conv1d_bwd_kernel<__half, 4><<<blocks, 256, 0, stream>>>((const __half*)dy, lddy, (const __half*)pre, (const __half*)w, seq_start, seq_end, (__half*)dx, lddx, dpre_out, (__half*)dhalo, T, C);
  else
    return -2;
  return (int)cudaGetLastError();
}

extern "C" int fmsb_ssd_make_g(const void* cb, const float* L, const float* dt, void* g, int nc, int nh, int G, int Q,
                               int dtype, cudaStream_t stream) {
  const long long total = (long long)nc * nh * Q * Q;
  if (total <= 0) return 0;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == 1) ssd_make_g_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)cb, L, dt, (__nv_bfloat16*)g, nc, nh, G, Q);
  else if (dtype == 0) ssd_make_g_kernel<__half><<<blocks, 256, 0, stream>>>((const __half*)cb, L, dt, (__half*)g, nc, nh, G, Q);
  else return -2;
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
                                  float* dS, float* dh0, float* dLtot_partial, int nc, int nh, int PN, int dtype,
                                  cudaStream_t stream) {
  const long long total = (long long)nh * PN;
  if (total <= 0) return 0;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == 1) ssd_state_bwd_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(dhprev_direct, dhT, Ltot, (const __nv_bfloat16*)hprev, dS, dh0, dLtot_partial, nc, nh, PN);
  else if (dtype == 0) ssd_state_bwd_kernel<__half><<<blocks, 256, 0, stream>>>(dhprev_direct, dhT, Ltot, (const __half*)hprev, dS, dh0, dLtot_partial, nc, nh, PN);
  else return -2;
  return (int)cudaGetLastError();
}
