// Bandwidth-bound pieces of the chunked Mamba2 SSD scan for sm_100a: everything between the batched tcgen05
// GEMMs of ops/mamba.py that touches a [chunks, heads, Q, Q] or a [T, heads, P] tensor.  (The reference delegates
// the scan to the external mamba_ssm package, fms_acceleration_mcp/utils/utils.py:17-24,64-80.)
//
//   ssd_make_g2      G[c,h,t,s] = CB[c,g(h),t,s] exp(L_t - L_s) dt_s  (s <= t)         16-byte loads and stores
//   ssd_dcb          dCB[c,g,t,s] = sum_{h in g} dG[c,h,t,s] exp(L_t - L_s) dt_s (s <= t), heads summed in fp32 registers
//   ssd_rowscale     out[t,h,:] = x[t,h,:] * w[t,h]
//   ssd_fwd_combine  y = y_intra + exp(L) y_inter + D x
//   ssd_bwd_combine  dx = D dy + dxw wgt + dx_intra, and the five per-(t,h) dot products the gradients of
//                    dt, A and D are made of
//   ssd_addscaled / ssd_rowdot   the entering-state correction of context parallelism and its decay gradient
//
// The backward needs sum_s dG o G (per row) and sum_t dG o G (per column).  Because dG = dy x^T and
// y_intra = G x, dx_intra = G^T dy, those are dy . y_intra and x . dx_intra per (t, h): no pass over a Q x Q
// tensor is needed for them.
//
// L and dt arrive twice: token-major [T, heads] for the [T, heads, P] kernels and chunk-major [chunks, heads, Q]
// ("Lt", "dtt") for the Q x Q kernels, so both kinds of kernel read them with unit stride.
#include "common.cuh"

namespace fmsb {
namespace ssd {

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]);
template <>
__device__ __forceinline__ void unpack8<__nv_bfloat16>(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __bfloat1622float2(h[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}
template <>
__device__ __forceinline__ void unpack8<__half>(const uint4& u, float (&f)[8]) {
  const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __half22float2(h[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}
template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&f)[8]);
template <>
__device__ __forceinline__ uint4 pack8<__nv_bfloat16>(const float (&f)[8]) {
  return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}
template <>
__device__ __forceinline__ uint4 pack8<__half>(const float (&f)[8]) {
  return make_uint4(pack_f16x2(f[0], f[1]), pack_f16x2(f[2], f[3]), pack_f16x2(f[4], f[5]), pack_f16x2(f[6], f[7]));
}
__device__ __forceinline__ void ld8f(const float* p, float (&f)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
  f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

constexpr int G2_ROWS = 64;  // rows of one (chunk, head) tile per CTA in ssd_make_g2

// grid (ceil(Q / G2_ROWS), nh, nc), block 256; CB [nc*G, Q, Q]; Lt, dtt [nc, nh, Q]; out [nc*nh, Q, Q].
// Q % 8 == 0 and (Q / 8) divides 256, so a thread keeps the same 8 columns for all its rows and holds their
// L_s and dt_s in registers.
template <typename T>
__global__ void __launch_bounds__(256) ssd_make_g2_kernel(const T* __restrict__ cb, const float* __restrict__ Lt,
                                                          const float* __restrict__ dtt, T* __restrict__ g, int nh,
                                                          int G, int Q) {
  const int c = blockIdx.z, h = blockIdx.y, t0 = blockIdx.x * G2_ROWS;
  const long long lbase = ((long long)c * nh + h) * Q;
  const int vpr = Q >> 3, rpp = 256 / vpr;  // vectors per row, rows per pass of the block
  const int s0 = (threadIdx.x % vpr) << 3, r0 = threadIdx.x / vpr;
  const int t_end = min(Q, t0 + G2_ROWS);
  float ls[8], ds[8], wj[8];
  bool split = false;
  if (s0 < t_end) {
    ld8f(Lt + lbase + s0, ls);
    ld8f(dtt + lbase + s0, ds);
    // exp(L_t - L_s) = exp(L_t - L_s0) * exp(L_s0 - L_s): one exponential per row and thread instead of eight, the
    // column factors (times dt_s) are formed once.  Only while the decay across the thread's eight columns is
    // moderate (exponent below 60: no overflow of the column factor, no underflow of the row factor that matters);
    // otherwise every element takes its own exponential.
    split = fabsf(ls[0] - ls[7]) < 60.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) wj[j] = split ? __expf(ls[0] - ls[j]) * ds[j] : 0.f;
  }
  const int gi = h / (nh / G);
  const T* cbt = cb + ((long long)c * G + gi) * Q * Q;
  T* gt = g + ((long long)c * nh + h) * Q * Q;
#pragma unroll 4
  for (int t = t0 + r0; t < t_end; t += rpp) {
    uint4 out = make_uint4(0u, 0u, 0u, 0u);
    if (s0 <= t) {
      const uint4 u = *reinterpret_cast<const uint4*>(cbt + (long long)t * Q + s0);
      const float lt = __ldg(Lt + lbase + t);
      float f[8];
      unpack8<T>(u, f);
      if (split) {
        const float e = __expf(lt - ls[0]);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = (s0 + j <= t) ? f[j] * e * wj[j] : 0.f;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = (s0 + j <= t) ? f[j] * __expf(lt - ls[j]) * ds[j] : 0.f;
      }
      out = pack8<T>(f);
    }
    *reinterpret_cast<uint4*>(gt + (long long)t * Q + s0) = out;
  }
}

// dCB[c, g, t, s] = sum_{h in g} dG[c, h, t, s] exp(L_t - L_s) dt_s  (s <= t).
// grid (ceil(Q / rpp), G, n), block 256, rpp = 256 / (Q / 8): a thread owns 8 columns of one row and sums the heads
// of the group in fp32 registers; dG [n*nh, Q, Q] (16-bit), out [n*G, Q, Q].  Heads are taken two at a time: their L
// and dt (Q values each) pass through shared memory, double-buffered, and the next pair's dG vectors and L/dt values
// are loaded before the current pair's arithmetic, so a thread has two 16-byte loads and up to 16 scalars in
// flight and the CTAs are small enough for several to share an SM.  Q <= 1024.
template <typename T>
__global__ void __launch_bounds__(256, 4) ssd_dcb_kernel(const T* __restrict__ dG, const float* __restrict__ Lt,
                                                       const float* __restrict__ dtt, T* __restrict__ dcb, int nh,
                                                       int G, int Q) {
  __shared__ __align__(16) float sL[2][2][1024];
  __shared__ __align__(16) float sD[2][2][1024];
  const int c = blockIdx.z, gi = blockIdx.y;
  const int vpr = Q >> 3, rpp = 256 / vpr;
  const int s0 = (threadIdx.x % vpr) << 3;
  const int t = blockIdx.x * rpp + threadIdx.x / vpr;
  const int hpg = nh / G;
  const bool on = t < Q && s0 <= t;
  const long long base0 = ((long long)c * nh + gi * hpg) * Q;  // L/dt offset of the group's first head
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  // first pair into buffer 0
  for (int i = threadIdx.x; i < Q; i += 256) {
    sL[0][0][i] = Lt[base0 + i];
    sD[0][0][i] = dtt[base0 + i];
    if (hpg > 1) {
      sL[0][1][i] = Lt[base0 + Q + i];
      sD[0][1][i] = dtt[base0 + Q + i];
    }
  }
  uint4 u0 = make_uint4(0u, 0u, 0u, 0u), u1 = u0;
  if (on) {
    u0 = *reinterpret_cast<const uint4*>(dG + (base0 + t) * Q + s0);
    if (hpg > 1) u1 = *reinterpret_cast<const uint4*>(dG + (base0 + Q + t) * Q + s0);
  }
  for (int h0 = 0; h0 < hpg; h0 += 2) {
    const int buf = (h0 >> 1) & 1;
    __syncthreads();  // buffer `buf` is complete; nobody still reads the other one
    const bool have1 = h0 + 1 < hpg;                  // this pair has a second head
    const bool more0 = h0 + 2 < hpg, more1 = h0 + 3 < hpg;  // heads of the next pair
    const long long nbase = base0 + (long long)(h0 + 2) * Q;
    float nl[2][4], nd[2][4];
    uint4 n0 = make_uint4(0u, 0u, 0u, 0u), n1 = n0;
    if (more0) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int i = threadIdx.x + k * 256;
        if (i < Q) {
          nl[0][k] = Lt[nbase + i];
          nd[0][k] = dtt[nbase + i];
          if (more1) {
            nl[1][k] = Lt[nbase + Q + i];
            nd[1][k] = dtt[nbase + Q + i];
          }
        }
      }
      if (on) {
        n0 = *reinterpret_cast<const uint4*>(dG + (nbase + t) * Q + s0);
        if (more1) n1 = *reinterpret_cast<const uint4*>(dG + (nbase + Q + t) * Q + s0);
      }
    }
    if (on) {
      float ls[8], ds[8], f[8];
      ld8f(&sL[buf][0][s0], ls);
      ld8f(&sD[buf][0][s0], ds);
      const float l0 = sL[buf][0][t];
      unpack8<T>(u0, f);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (s0 + j <= t) acc[j] += f[j] * __expf(l0 - ls[j]) * ds[j];
      if (have1) {
        ld8f(&sL[buf][1][s0], ls);
        ld8f(&sD[buf][1][s0], ds);
        const float l1 = sL[buf][1][t];
        unpack8<T>(u1, f);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (s0 + j <= t) acc[j] += f[j] * __expf(l1 - ls[j]) * ds[j];
      }
    }
    if (more0) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int i = threadIdx.x + k * 256;
        if (i < Q) {
          sL[buf ^ 1][0][i] = nl[0][k];
          sD[buf ^ 1][0][i] = nd[0][k];
          if (more1) {
            sL[buf ^ 1][1][i] = nl[1][k];
            sD[buf ^ 1][1][i] = nd[1][k];
          }
        }
      }
      u0 = n0;
      u1 = n1;
    }
  }
  if (t < Q) *reinterpret_cast<uint4*>(dcb + (((long long)c * G + gi) * Q + t) * Q + s0) = pack8<T>(acc);
}

// out[row, :] = x[row, :] * w[row]   rows = T*nh, P % 8 == 0
template <typename T>
__global__ void ssd_rowscale_kernel(const T* __restrict__ x, const float* __restrict__ w, T* __restrict__ out,
                                    long long n_vec, int vpr) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= n_vec) return;
  const float sc = w[i / vpr];
  float f[8];
  unpack8<T>(*reinterpret_cast<const uint4*>(x + i * 8), f);
#pragma unroll
  for (int j = 0; j < 8; ++j) f[j] *= sc;
  *reinterpret_cast<uint4*>(out + i * 8) = pack8<T>(f);
}

// y[row, :] = y_intra[row, :] + exp(L[row]) * y_inter[row, :] + D[row % nh] * x[row, :]
template <typename T>
__global__ void ssd_fwd_combine_kernel(const float* __restrict__ y_intra, const float* __restrict__ y_inter,
                                       const T* __restrict__ x, const float* __restrict__ L, const float* __restrict__ D,
                                       T* __restrict__ y, long long n_vec, int vpr, int nh) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= n_vec) return;
  const long long row = i / vpr;
  const float e = __expf(L[row]), d = D[(int)(row % nh)];
  float a[8], b[8], xv[8];
  ld8f(y_intra + i * 8, a);
  ld8f(y_inter + i * 8, b);
  unpack8<T>(*reinterpret_cast<const uint4*>(x + i * 8), xv);
#pragma unroll
  for (int j = 0; j < 8; ++j) a[j] = a[j] + e * b[j] + d * xv[j];
  *reinterpret_cast<uint4*>(y + i * 8) = pack8<T>(a);
}

// One (t, h) row of P = 8 * vpr values per TPR lanes (TPR = power of two >= vpr, <= 32).
//   dx      = D dy + dxw wgt + dx_intra
//   red[0]  = dy . x              (dD, summed over t by the caller)
//   red[1]  = exp(L) dy . y_inter (dL through the inter-chunk term)
//   red[2]  = dxw . x             (d of the chunk-state weight)
//   red[3]  = dy . y_intra        (row sums of dG o G)
//   red[4]  = x . dx_intra        (column sums of dG o G)
template <typename T, int TPR>
__global__ void __launch_bounds__(256) ssd_bwd_combine_kernel(
    const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ y_inter, const float* __restrict__ dxw,
    const float* __restrict__ dx_intra, const float* __restrict__ y_intra, const float* __restrict__ L,
    const float* __restrict__ wgt, const float* __restrict__ D, T* __restrict__ dx, float* __restrict__ red,
    long long rows, int vpr, int nh) {
  const long long gt = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long row = gt / TPR;
  const int v = (int)(gt % TPR);
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f, s4 = 0.f;
  const bool live = row < rows && v < vpr;
  if (live) {
    const long long off = (row * vpr + v) * 8;
    const float d = D[(int)(row % nh)], w = wgt[row];
    float dyv[8], xv[8], yi[8], xw[8], di[8], ya[8], o[8];
    unpack8<T>(*reinterpret_cast<const uint4*>(dy + off), dyv);
    unpack8<T>(*reinterpret_cast<const uint4*>(x + off), xv);
    ld8f(y_inter + off, yi);
    ld8f(dxw + off, xw);
    ld8f(dx_intra + off, di);
    ld8f(y_intra + off, ya);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      o[j] = d * dyv[j] + xw[j] * w + di[j];
      s0 += dyv[j] * xv[j];
      s1 += dyv[j] * yi[j];
      s2 += xw[j] * xv[j];
      s3 += dyv[j] * ya[j];
      s4 += xv[j] * di[j];
    }
    *reinterpret_cast<uint4*>(dx + off) = pack8<T>(o);
  }
#pragma unroll
  for (int m = TPR >> 1; m > 0; m >>= 1) {
    s0 += __shfl_xor_sync(0xffffffffu, s0, m);
    s1 += __shfl_xor_sync(0xffffffffu, s1, m);
    s2 += __shfl_xor_sync(0xffffffffu, s2, m);
    s3 += __shfl_xor_sync(0xffffffffu, s3, m);
    s4 += __shfl_xor_sync(0xffffffffu, s4, m);
  }
  if (row < rows && v == 0) {
    red[row] = s0;
    red[rows + row] = __expf(L[row]) * s1;
    red[2 * rows + row] = s2;
    red[3 * rows + row] = s3;
    red[4 * rows + row] = s4;
  }
}

// out[row, :] = a[row, :] + exp(L[row]) * v[row, :]      (a, out 16-bit; v fp32)
template <typename T>
__global__ void ssd_addscaled_kernel(const T* __restrict__ a, const float* __restrict__ v, const float* __restrict__ L,
                                     T* __restrict__ out, long long n_vec, int vpr) {
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= n_vec) return;
  const float e = __expf(L[i / vpr]);
  float f[8], g[8];
  unpack8<T>(*reinterpret_cast<const uint4*>(a + i * 8), f);
  ld8f(v + i * 8, g);
#pragma unroll
  for (int j = 0; j < 8; ++j) f[j] += e * g[j];
  *reinterpret_cast<uint4*>(out + i * 8) = pack8<T>(f);
}

// red[row] = exp(L[row]) * sum_p a[row, p] * v[row, p]    (a 16-bit, v fp32); TPR lanes per row
template <typename T, int TPR>
__global__ void __launch_bounds__(256) ssd_rowdot_kernel(const T* __restrict__ a, const float* __restrict__ v,
                                                         const float* __restrict__ L, float* __restrict__ red,
                                                         long long rows, int vpr) {
  const long long gt = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long row = gt / TPR;
  const int k = (int)(gt % TPR);
  float acc = 0.f;
  if (row < rows && k < vpr) {
    const long long off = (row * vpr + k) * 8;
    float f[8], g[8];
    unpack8<T>(*reinterpret_cast<const uint4*>(a + off), f);
    ld8f(v + off, g);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += f[j] * g[j];
  }
#pragma unroll
  for (int m = TPR >> 1; m > 0; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
  if (row < rows && k == 0) red[row] = __expf(L[row]) * acc;
}

}  // namespace ssd
}  // namespace fmsb

using namespace fmsb;
using namespace fmsb::ssd;

extern "C" int fmsb_ssd_make_g2(const void* cb, const float* Lt, const float* dtt, void* g, int nc, int nh, int G, int Q,
                                int dtype, cudaStream_t stream) {
  if (nc <= 0) return 0;
  if (Q % 8 != 0 || 256 % (Q / 8) != 0 || nh % G != 0 || nc > 65535 || nh > 65535) return -2;
  const dim3 grid((Q + G2_ROWS - 1) / G2_ROWS, nh, nc);
  if (dtype == 1)
    ssd_make_g2_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)cb, Lt, dtt, (__nv_bfloat16*)g, nh, G, Q);
  else if (dtype == 0)
    ssd_make_g2_kernel<__half><<<grid, 256, 0, stream>>>((const __half*)cb, Lt, dtt, (__half*)g, nh, G, Q);
  else
    return -2;
  return (int)cudaGetLastError();
}

extern "C" int fmsb_ssd_dcb(const void* dG, const float* Lt, const float* dtt, void* dcb, int nc, int nh, int G, int Q,
                            int dtype, cudaStream_t stream) {
  if (nc <= 0) return 0;
  if (Q % 8 != 0 || 256 % (Q / 8) != 0 || Q > 1024 || nh % G != 0 || nc > 65535 || G > 65535) return -2;
  const int rows_per_cta = 256 / (Q / 8);
  const dim3 grid((Q + rows_per_cta - 1) / rows_per_cta, G, nc);
  if (dtype == 1)
    ssd_dcb_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)dG, Lt, dtt, (__nv_bfloat16*)dcb, nh, G, Q);
  else if (dtype == 0)
    ssd_dcb_kernel<__half><<<grid, 256, 0, stream>>>((const __half*)dG, Lt, dtt, (__half*)dcb, nh, G, Q);
  else
    return -2;
  return (int)cudaGetLastError();
}

extern "C" int fmsb_ssd_rowscale(const void* x, const float* w, void* out, long long rows, int P, int dtype,
                                 cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (P % 8 != 0) return -2;
  const int vpr = P / 8;
  const long long n_vec = rows * vpr;
  const unsigned blocks = (unsigned)((n_vec + 255) / 256);
  if (dtype == 1)
    ssd_rowscale_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, w, (__nv_bfloat16*)out, n_vec, vpr);
  else if (dtype == 0)
    ssd_rowscale_kernel<__half><<<blocks, 256, 0, stream>>>((const __half*)x, w, (__half*)out, n_vec, vpr);
  else
    return -2;
  return (int)cudaGetLastError();
}

extern "C" int fmsb_ssd_fwd_combine(const float* y_intra, const float* y_inter, const void* x, const float* L,
                                    const float* D, void* y, long long rows, int P, int nh, int dtype,
                                    cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (P % 8 != 0) return -2;
  const int vpr = P / 8;
  const long long n_vec = rows * vpr;
  const unsigned blocks = (unsigned)((n_vec + 255) / 256);
  if (dtype == 1)
    ssd_fwd_combine_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(y_intra, y_inter, (const __nv_bfloat16*)x, L, D, (__nv_bfloat16*)y, n_vec, vpr, nh);
  else if (dtype == 0)
    ssd_fwd_combine_kernel<__half><<<blocks, 256, 0, stream>>>(y_intra, y_inter, (const __half*)x, L, D, (__half*)y, n_vec, vpr, nh);
  else
    return -2;
  return (int)cudaGetLastError();
}

template <typename T>
static int launch_bwd_combine(const void* dy, const void* x, const float* y_inter, const float* dxw,
                              const float* dx_intra, const float* y_intra, const float* L, const float* wgt,
                              const float* D, void* dx, float* red, long long rows, int P, int nh, cudaStream_t stream) {
  const int vpr = P / 8;
  int tpr = 1;
  while (tpr < vpr) tpr <<= 1;
  if (tpr > 32) return -2;
  const long long threads = rows * tpr;
  const unsigned blocks = (unsigned)((threads + 255) / 256);
#define FMSB_BC(TPR_)                                                                                              \
  case TPR_:                                                                                                       \
    ssd_bwd_combine_kernel<T, TPR_><<<blocks, 256, 0, stream>>>((const T*)dy, (const T*)x, y_inter, dxw, dx_intra, \
                                                                y_intra, L, wgt, D, (T*)dx, red, rows, vpr, nh);   \
    break;
  switch (tpr) {
    FMSB_BC(1) FMSB_BC(2) FMSB_BC(4) FMSB_BC(8) FMSB_BC(16) FMSB_BC(32)
    default: return -2;
  }
#undef FMSB_BC
  return (int)cudaGetLastError();
}

extern "C" int fmsb_ssd_bwd_combine(const void* dy, const void* x, const float* y_inter, const float* dxw,
                                    const float* dx_intra, const float* y_intra, const float* L, const float* wgt,
                                    const float* D, void* dx, float* red, long long rows, int P, int nh, int dtype,
                                    cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (P % 8 != 0) return -2;
  if (dtype == 1)
    return launch_bwd_combine<__nv_bfloat16>(dy, x, y_inter, dxw, dx_intra, y_intra, L, wgt, D, dx, red, rows, P, nh, stream);
  if (dtype == 0)
    return launch_bwd_combine<__half>(dy, x, y_inter, dxw, dx_intra, y_intra, L, wgt, D, dx, red, rows, P, nh, stream);
  return -2;
}

extern "C" int fmsb_ssd_addscaled(const void* a, const float* v, const float* L, void* out, long long rows, int P,
                                  int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (P % 8 != 0) return -2;
  const int vpr = P / 8;
  const long long n_vec = rows * vpr;
  const unsigned blocks = (unsigned)((n_vec + 255) / 256);
  if (dtype == 1)
    ssd_addscaled_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)a, v, L, (__nv_bfloat16*)out, n_vec, vpr);
  else if (dtype == 0)
    ssd_addscaled_kernel<__half><<<blocks, 256, 0, stream>>>((const __half*)a, v, L, (__half*)out, n_vec, vpr);
  else
    return -2;
  return (int)cudaGetLastError();
}

template <typename T>
static int launch_rowdot(const void* a, const float* v, const float* L, float* red, long long rows, int P,
                         cudaStream_t stream) {
  const int vpr = P / 8;
  int tpr = 1;
  while (tpr < vpr) tpr <<= 1;
  if (tpr > 32) return -2;
  const unsigned blocks = (unsigned)((rows * tpr + 255) / 256);
#define FMSB_RD(TPR_)                                                                                    \
  case TPR_:                                                                                             \
    ssd_rowdot_kernel<T, TPR_><<<blocks, 256, 0, stream>>>((const T*)a, v, L, red, rows, vpr);           \
    break;
  switch (tpr) {
    FMSB_RD(1) FMSB_RD(2) FMSB_RD(4) FMSB_RD(8) FMSB_RD(16) FMSB_RD(32)
    default: return -2;
  }
#undef FMSB_RD
  return (int)cudaGetLastError();
}

extern "C" int fmsb_ssd_rowdot(const void* a, const float* v, const float* L, float* red, long long rows, int P,
                               int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (P % 8 != 0) return -2;
  if (dtype == 1) return launch_rowdot<__nv_bfloat16>(a, v, L, red, rows, P, stream);
  if (dtype == 0) return launch_rowdot<__half>(a, v, L, red, rows, P, stream);
  return -2;
}
