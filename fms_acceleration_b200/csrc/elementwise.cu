// Bandwidth-bound fused ops for sm_100a: RMSNorm (+residual add) forward/backward, rotary
// embedding with explicit position ids, SwiGLU / GEGLU forward/backward.
//
// Reference semantics (file paths inside the reference project):
//   RMSNorm   fms_acceleration_foak/kernels/unsloth/rms_layernorm.py:21-128  (fp32 accumulate,
//             inv_rms saved; gemma variant uses W+1; the reference has no dW, here it is optional)
//   RoPE      fms_acceleration_foak/kernels/unsloth/rope_embedding.py:20-72   (rotate halves; the
//             reference derives the position from row % seqlen, which is wrong for packed
//             batches; this kernel takes position ids)
//   SwiGLU    fms_acceleration_foak/fused_ops/unsloth_lora/swiglu.py:20-98
//   GEGLU     fms_acceleration_foak/fused_ops/unsloth_lora/geglu.py:20-202
//
// All kernels use 16-byte vector accesses; rows must be multiples of 8 elements and 16-byte
// aligned.  dtype code: 0 = fp16, 1 = bf16.
#include "common.cuh"

namespace fmsb {

template <typename T>
struct Vec8 {
  uint4 u;
  __device__ __forceinline__ void load(const T* p) { u = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ void store(T* p) const { *reinterpret_cast<uint4*>(p) = u; }
  __device__ __forceinline__ void to_float(float (&f)[8]) const;
  __device__ __forceinline__ void from_float(const float (&f)[8]);
};
template <>
__device__ __forceinline__ void Vec8<__nv_bfloat16>::to_float(float (&f)[8]) const {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 v = __bfloat1622float2(h[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}
template <>
__device__ __forceinline__ void Vec8<__half>::to_float(float (&f)[8]) const {
  const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 v = __half22float2(h[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}
template <>
__device__ __forceinline__ void Vec8<__nv_bfloat16>::from_float(const float (&f)[8]) {
  u.x = pack_bf16x2(f[0], f[1]);
  u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]);
  u.w = pack_bf16x2(f[6], f[7]);
}
template <>
__device__ __forceinline__ void Vec8<__half>::from_float(const float (&f)[8]) {
  u.x = pack_f16x2(f[0], f[1]);
  u.y = pack_f16x2(f[2], f[3]);
  u.z = pack_f16x2(f[4], f[5]);
  u.w = pack_f16x2(f[6], f[7]);
}

template <typename T>
__device__ __forceinline__ float round_to(float v);
template <>
__device__ __forceinline__ float round_to<__nv_bfloat16>(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}
template <>
__device__ __forceinline__ float round_to<__half>(float v) {
  return __half2float(__float2half_rn(v));
}

constexpr int NORM_THREADS = 256;
constexpr int NORM_MAXV = 4;  // vectors of 8 cached per thread -> fast path up to H = 8192

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < NORM_THREADS / 32; ++i) t += red[i];
  return t;
}

// ---------------------------------------------------------------------------------------------------------------
// Row-in-registers RMSNorm for the common row widths (H = 1024 ... 8192): one warp (or 2, 4 or 8 warps, WPR) keeps
// its row packed in registers (VPL 16-byte vectors per lane), reduces with shuffles (plus one 64-thread named barrier
// for a pair) and never meets a block-wide barrier, so the warps of a CTA stream independent rows and an SM has 16 or
// more rows in flight.  The block-per-row kernels below had one or two rows in flight per CTA around two
// __syncthreads each and stopped at 0.57 (forward) / 0.67 (backward) of the copy bandwidth.
// ---------------------------------------------------------------------------------------------------------------
constexpr int NORM_WARPS = 8;

// sum over the WPR warps that share a row; `red` is double-buffered by `parity` (a warp cannot run two barriers ahead
// of its partner, so the buffer written two sums ago is free)
template <int WPR>
__device__ __forceinline__ float row_sum(float v, float (*red)[NORM_WARPS], int& parity) {
  v = warp_sum(v);
  if (WPR == 1) return v;
  const int warp = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0) red[parity][warp] = v;
  asm volatile("bar.sync %0, %1;" ::"r"(1 + warp / WPR), "n"(WPR * 32) : "memory");
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < WPR; ++i) t += red[parity][warp / WPR * WPR + i];
  parity ^= 1;
  return t;
}

template <typename T, int VPL, int WPR>
__global__ void __launch_bounds__(NORM_WARPS * 32, 2)
rmsnorm_fwd_rows_kernel(const T* __restrict__ x, const T* __restrict__ residual, const T* __restrict__ w,
                        T* __restrict__ y, T* __restrict__ h_out, float* __restrict__ inv_rms, int rows, float eps,
                        int gemma) {
  constexpr int H = VPL * 256 * WPR;
  constexpr int RPC = NORM_WARPS / WPR;  // rows per CTA and trip
  __shared__ float red[2][NORM_WARPS];
  int parity = 0;
  const int warp = threadIdx.x >> 5;
  const int col0 = ((warp % WPR) * 32 + (threadIdx.x & 31)) * 8;  // this lane's first element; vectors 256 * WPR apart
  for (int row = blockIdx.x * RPC + warp / WPR; row < rows; row += gridDim.x * RPC) {
    const long long base = (long long)row * H + col0;
    Vec8<T> c[VPL];
#pragma unroll
    for (int j = 0; j < VPL; ++j) c[j].load(x + base + j * (256 * WPR));
    if (residual != nullptr) {
#pragma unroll
      for (int j = 0; j < VPL; ++j) {
        Vec8<T> r;
        float a[8], b[8];
        r.load(residual + base + j * (256 * WPR));
        c[j].to_float(a);
        r.to_float(b);
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] += b[i];
        c[j].from_float(a);  // the new residual stream, rounded to the storage type as the next layer will read it
        if (h_out != nullptr) c[j].store(h_out + base + j * (256 * WPR));
      }
    }
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      float a[8];
      c[j].to_float(a);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += a[i] * a[i];
    }
    ss = row_sum<WPR>(ss, red, parity);
    const float inv = rsqrtf(ss / (float)H + eps);
    if (col0 == 0 && inv_rms != nullptr) inv_rms[row] = inv;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      Vec8<T> wv, o;
      float a[8], wf[8], out[8];
      wv.load(w + col0 + j * (256 * WPR));
      wv.to_float(wf);
      c[j].to_float(a);
#pragma unroll
      for (int i = 0; i < 8; ++i) out[i] = gemma ? a[i] * inv * (wf[i] + 1.f) : round_to<T>(a[i] * inv) * wf[i];
      o.from_float(out);
      o.store(y + base + j * (256 * WPR));
    }
  }
}

// dx = inv/H * (H * dy*w - xhat * sum(dy*w*xhat)) [+ dres_in].  WITH_DW: every lane also sums dy * xhat over its rows;
// the warps of a CTA fold their sums in shared memory and the CTA writes ONE partial row dw_partial[blockIdx.x, :].
template <typename T, int VPL, int WPR, bool WITH_DW>
__global__ void __launch_bounds__(NORM_WARPS * 32, 2)
rmsnorm_bwd_rows_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
                        const float* __restrict__ inv_rms, const T* __restrict__ dres_in, T* __restrict__ dx,
                        float* __restrict__ dw_partial, int rows, int gemma) {
  constexpr int H = VPL * 256 * WPR;
  constexpr int RPC = NORM_WARPS / WPR;
  __shared__ float red[2][NORM_WARPS];
  __shared__ float dwred[WITH_DW ? RPC * H : 1];
  int parity = 0;
  const int warp = threadIdx.x >> 5;
  const int col0 = ((warp % WPR) * 32 + (threadIdx.x & 31)) * 8;
  const float wadd = gemma ? 1.f : 0.f;
  float dwacc[WITH_DW ? VPL : 1][8];
#pragma unroll
  for (int j = 0; j < (WITH_DW ? VPL : 1); ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) dwacc[j][i] = 0.f;
  for (int row = blockIdx.x * RPC + warp / WPR; row < rows; row += gridDim.x * RPC) {
    const long long base = (long long)row * H + col0;
    Vec8<T> xc[VPL], dc[VPL];
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      xc[j].load(x + base + j * (256 * WPR));
      dc[j].load(dy + base + j * (256 * WPR));
    }
    const float inv = inv_rms[row];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      Vec8<T> wv;
      float xf[8], df[8], wf[8];
      wv.load(w + col0 + j * (256 * WPR));
      wv.to_float(wf);
      xc[j].to_float(xf);
      dc[j].to_float(df);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float xh = xf[i] * inv;
        dot += df[i] * (wf[i] + wadd) * xh;
        if (WITH_DW) dwacc[WITH_DW ? j : 0][i] += df[i] * xh;
      }
    }
    dot = row_sum<WPR>(dot, red, parity);
    const float c = dot / (float)H;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      Vec8<T> wv, o;
      float xf[8], df[8], wf[8], out[8];
      wv.load(w + col0 + j * (256 * WPR));
      wv.to_float(wf);
      xc[j].to_float(xf);
      dc[j].to_float(df);
#pragma unroll
      for (int i = 0; i < 8; ++i) out[i] = inv * (df[i] * (wf[i] + wadd) - xf[i] * inv * c);
      if (dres_in != nullptr) {
        Vec8<T> rv;
        float rf[8];
        rv.load(dres_in + base + j * (256 * WPR));
        rv.to_float(rf);
#pragma unroll
        for (int i = 0; i < 8; ++i) out[i] += rf[i];
      }
      o.from_float(out);
      o.store(dx + base + j * (256 * WPR));
    }
  }
  if (WITH_DW) {
#pragma unroll
    for (int j = 0; j < (WITH_DW ? VPL : 1); ++j) {
      float* dst = dwred + (warp / WPR) * H + col0 + j * (256 * WPR);
      *reinterpret_cast<float4*>(dst) = make_float4(dwacc[j][0], dwacc[j][1], dwacc[j][2], dwacc[j][3]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(dwacc[j][4], dwacc[j][5], dwacc[j][6], dwacc[j][7]);
    }
    __syncthreads();
    for (int col = threadIdx.x; col < H; col += NORM_WARPS * 32) {
      float t = 0.f;
#pragma unroll
      for (int r = 0; r < RPC; ++r) t += dwred[r * H + col];
      dw_partial[(long long)blockIdx.x * H + col] = t;
    }
  }
}

// y = rms_norm(x [+ residual]) * (w [+1]);  optional h_out = x + residual (the new residual stream)
template <typename T>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ residual, const T* __restrict__ w,
                   T* __restrict__ y, T* __restrict__ h_out, float* __restrict__ inv_rms, int rows, int H,
                   float eps, int gemma) {
  __shared__ float red[NORM_THREADS / 32];
  const int nvec = H / 8;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + (long long)row * H;
    float cache[NORM_MAXV][8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NORM_MAXV; ++j) {
      const int v = threadIdx.x + j * NORM_THREADS;
      if (v < nvec) {
        Vec8<T> a;
        a.load(xr + v * 8);
        a.to_float(cache[j]);
        if (residual != nullptr) {
          Vec8<T> b;
          float rb[8];
          b.load(residual + (long long)row * H + v * 8);
          b.to_float(rb);
#pragma unroll
          for (int i = 0; i < 8; ++i) cache[j][i] = round_to<T>(cache[j][i] + rb[i]);
          if (h_out != nullptr) {
            Vec8<T> o;
            o.from_float(cache[j]);
            o.store(h_out + (long long)row * H + v * 8);
          }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += cache[j][i] * cache[j][i];
      }
    }
    const float tot = block_sum(ss, red);
    const float inv = rsqrtf(tot / (float)H + eps);
    if (threadIdx.x == 0 && inv_rms != nullptr) inv_rms[row] = inv;
#pragma unroll
    for (int j = 0; j < NORM_MAXV; ++j) {
      const int v = threadIdx.x + j * NORM_THREADS;
      if (v < nvec) {
        Vec8<T> wv;
        float wf[8], out[8];
        wv.load(w + v * 8);
        wv.to_float(wf);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (gemma) {
            out[i] = cache[j][i] * inv * (wf[i] + 1.f);
          } else {
            out[i] = round_to<T>(cache[j][i] * inv) * wf[i];
          }
        }
        Vec8<T> o;
        o.from_float(out);
        o.store(y + (long long)row * H + v * 8);
      }
    }
  }
}

// dx = inv/H * (H * dy*w - xhat * sum(dy*w*xhat)) [+ dres_in];   dw_partial[block] += dy * xhat
// MAXV vectors of 8 are cached per thread (2 covers H <= 4096 with a third of the registers of 4); the weight-gradient
// accumulators exist only when WITH_DW, so the common frozen-norm case runs several CTAs per SM.
template <typename T, int MAXV, bool WITH_DW>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
                   const float* __restrict__ inv_rms, const T* __restrict__ dres_in, T* __restrict__ dx,
                   float* __restrict__ dw_partial, int rows, int H, int gemma) {
  __shared__ float red[NORM_THREADS / 32];
  const int nvec = H / 8;
  float dwacc[WITH_DW ? MAXV : 1][8];
#pragma unroll
  for (int j = 0; j < (WITH_DW ? MAXV : 1); ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) dwacc[j][i] = 0.f;
  float wf[MAXV][8];
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int v = threadIdx.x + j * NORM_THREADS;
    if (v < nvec) {
      Vec8<T> wv;
      wv.load(w + v * 8);
      wv.to_float(wf[j]);
      if (gemma) {
#pragma unroll
        for (int i = 0; i < 8; ++i) wf[j][i] += 1.f;
      }
    }
  }
  // Rows are software-pipelined: the 16-byte loads of the NEXT row (x, dy and the incoming residual gradient) are
  // issued before this row's block-wide reduction, so a CTA always has two rows' worth of loads in flight.
  Vec8<T> xn[MAXV], dyn[MAXV], rn[MAXV];
  auto fetch = [&](int row) {
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int v = threadIdx.x + j * NORM_THREADS;
      if (v < nvec) {
        xn[j].load(x + (long long)row * H + v * 8);
        dyn[j].load(dy + (long long)row * H + v * 8);
        if (dres_in != nullptr) rn[j].load(dres_in + (long long)row * H + v * 8);
      }
    }
  };
  if ((int)blockIdx.x < rows) fetch(blockIdx.x);
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const float inv = inv_rms[row];
    float xh[MAXV][8], g[MAXV][8], rf[MAXV][8];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int v = threadIdx.x + j * NORM_THREADS;
      if (v < nvec) {
        float dyf[8];
        xn[j].to_float(xh[j]);
        dyn[j].to_float(dyf);
        if (dres_in != nullptr) rn[j].to_float(rf[j]);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xh[j][i] *= inv;
          g[j][i] = dyf[i] * wf[j][i];
          dot += g[j][i] * xh[j][i];
          if (WITH_DW) dwacc[WITH_DW ? j : 0][i] += dyf[i] * xh[j][i];
        }
      }
    }
    if (row + (int)gridDim.x < rows) fetch(row + gridDim.x);
    const float tot = block_sum(dot, red);
    const float c = tot / (float)H;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      const int v = threadIdx.x + j * NORM_THREADS;
      if (v < nvec) {
        float out[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) out[i] = inv * (g[j][i] - xh[j][i] * c);
        if (dres_in != nullptr) {
#pragma unroll
          for (int i = 0; i < 8; ++i) out[i] += rf[j][i];
        }
        Vec8<T> o;
        o.from_float(out);
        o.store(dx + (long long)row * H + v * 8);
      }
    }
  }
  if (WITH_DW && dw_partial != nullptr) {
#pragma unroll
    for (int j = 0; j < (WITH_DW ? MAXV : 1); ++j) {
      const int v = threadIdx.x + j * NORM_THREADS;
      if (v < nvec) {
        float* dst = dw_partial + (long long)blockIdx.x * H + v * 8;
        *reinterpret_cast<float4*>(dst) = make_float4(dwacc[j][0], dwacc[j][1], dwacc[j][2], dwacc[j][3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(dwacc[j][4], dwacc[j][5], dwacc[j][6], dwacc[j][7]);
      }
    }
  }
}

// out[c] = sum_b partial[b, c].  Block (32, 8): 32 neighbouring columns, the rows dealt over the 8 row lanes and
// folded in shared memory.
__global__ void colsum_kernel(const float* __restrict__ partial, float* __restrict__ out, int nblocks, int H) {
  __shared__ float red[8][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  float s = 0.f;
  if (c < H) {
#pragma unroll 4
    for (int b = threadIdx.y; b < nblocks; b += 8) s += partial[(long long)b * H + c];
  }
  red[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && c < H) {
    float t = 0.f;
#pragma unroll
    for (int y = 0; y < 8; ++y) t += red[y][threadIdx.x];
    out[c] = t;
  }
}

// Walks the [rows, I / 8] grid of 16-byte vectors with a grid-sized stride using 32-bit adds only: the stride's
// (rows, vectors) decomposition is formed once per thread.
struct VecWalk {
  int r, c, dr, dc, vpr;
  __device__ __forceinline__ VecWalk(int vec_per_row) : vpr(vec_per_row) {
    const long long first = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    r = (int)(first / vpr);
    c = (int)(first % vpr);
    dr = (int)(stride / vpr);
    dc = (int)(stride % vpr);
  }
  __device__ __forceinline__ void next() {
    r += dr;
    c += dc;
    if (c >= vpr) {
      c -= vpr;
      r += 1;
    }
  }
};

// Rotary embedding on a packed [T, row_stride] buffer holding n_heads heads of size d starting
// at column 0 (e.g. the q|k part of a fused qkv projection).  cos/sin: [max_pos, d/2] fp32.
// sign = +1 forward, -1 backward.  In place.
template <typename T>
__global__ void rope_kernel(T* __restrict__ qk, const int* __restrict__ pos, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, int T_tokens, int n_heads, int d,
                            long long row_stride, float sign) {
  const int half = d / 2;
  const int vec_per_head = half / 8;
  // (token, vector within the token's heads) by 32-bit adds; the head comes from one small 32-bit division
  for (VecWalk it(n_heads * vec_per_head); it.r < T_tokens; it.next()) {
    const int h = it.c / vec_per_head;
    const int v = it.c - h * vec_per_head;
    const long long t = it.r;
    const int p = pos[t];
    T* base = qk + t * row_stride + (long long)h * d + v * 8;
    Vec8<T> a, b;
    float x1[8], x2[8], o1[8], o2[8];
    a.load(base);
    b.load(base + half);
    a.to_float(x1);
    b.to_float(x2);
    const float4* cp = reinterpret_cast<const float4*>(cos_t + (long long)p * half + v * 8);
    const float4* sp = reinterpret_cast<const float4*>(sin_t + (long long)p * half + v * 8);
    float c[8], s[8];
    *reinterpret_cast<float4*>(c) = cp[0];
    *reinterpret_cast<float4*>(c + 4) = cp[1];
    *reinterpret_cast<float4*>(s) = sp[0];
    *reinterpret_cast<float4*>(s + 4) = sp[1];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float sn = s[i] * sign;
      o1[i] = x1[i] * c[i] - x2[i] * sn;
      o2[i] = x2[i] * c[i] + x1[i] * sn;
    }
    a.from_float(o1);
    b.from_float(o2);
    a.store(base);
    b.store(base + half);
  }
}

// activation codes: 0 = SwiGLU (silu), 1 = GEGLU exact (erf), 2 = GEGLU tanh approximation.  The code is a template
// parameter and the sigmoid uses the approximate reciprocal: with a run-time switch, a full-precision division per
// element and a 64-bit division per vector these kernels were bound by instruction issue (0.70 of the copy bandwidth),
// not by memory.
template <int ACT>
__device__ __forceinline__ float act_fwd(float e) {
  if (ACT == 0) return e * __fdividef(1.f, 1.f + __expf(-e));
  if (ACT == 1) return 0.5f * e * (1.f + erff(e * 0.70710678118654752f));
  const float k = 0.7978845608028654f;
  return 0.5f * e * (1.f + tanhf(k * e * (1.f + 0.044715f * e * e)));
}
// activation and its derivative together (the backward needs both)
template <int ACT>
__device__ __forceinline__ void act_both(float e, float& f, float& df) {
  if (ACT == 0) {
    const float s = __fdividef(1.f, 1.f + __expf(-e));
    f = e * s;
    df = s * (1.f + e * (1.f - s));
    return;
  }
  if (ACT == 1) {
    const float cdf = 0.5f * (1.f + erff(e * 0.70710678118654752f));
    f = e * cdf;
    df = cdf + e * 0.3989422804014327f * __expf(-0.5f * e * e);
    return;
  }
  const float k = 0.7978845608028654f;
  const float u = k * e * (1.f + 0.044715f * e * e);
  const float th = tanhf(u);
  f = 0.5f * e * (1.f + th);
  df = 0.5f * (1.f + th) + 0.5f * e * (1.f - th * th) * k * (1.f + 3.f * 0.044715f * e * e);
}


// h[t, i] = act(e[t, i]) * g[t, i]    e, g, h: row strides in elements
template <typename T, int ACT>
__global__ void __launch_bounds__(256)
glu_fwd_kernel(const T* __restrict__ e, const T* __restrict__ g, T* __restrict__ h, int rows, int I, long long se,
               long long sg, long long sh, const int* __restrict__ rows_dev) {
  // rows_dev (optional): the number of rows actually in use, known only on the device (the filled part of a
  // fixed-capacity mixture-of-experts buffer); never more than `rows`
  if (rows_dev != nullptr) rows = min(rows, *rows_dev);
  for (VecWalk it(I / 8); it.r < rows; it.next()) {
    const int c = it.c * 8;
    Vec8<T> a, b;
    float ef[8], gf[8], out[8];
    a.load(e + it.r * se + c);
    b.load(g + it.r * sg + c);
    a.to_float(ef);
    b.to_float(gf);
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = round_to<T>(act_fwd<ACT>(ef[i])) * gf[i];
    Vec8<T> o;
    o.from_float(out);
    o.store(h + it.r * sh + c);
  }
}

// Given dh, e, g:  de = dh * g * act'(e),  dg = dh * act(e); optionally also h = act(e) * g.
// de/dg may alias e/g (the in-place scheme of the reference).
template <typename T, int ACT>
__global__ void __launch_bounds__(256)
glu_bwd_kernel(const T* __restrict__ dh, const T* e, const T* g, T* de, T* dg, T* __restrict__ h_out, int rows, int I,
               long long sdh, long long se, long long sg, long long sde, long long sdg, long long sh,
               const int* __restrict__ rows_dev) {
  if (rows_dev != nullptr) rows = min(rows, *rows_dev);
  for (VecWalk it(I / 8); it.r < rows; it.next()) {
    const int c = it.c * 8;
    Vec8<T> a, b, d;
    float ef[8], gf[8], df[8], o1[8], o2[8], o3[8];
    a.load(e + it.r * se + c);
    b.load(g + it.r * sg + c);
    d.load(dh + it.r * sdh + c);
    a.to_float(ef);
    b.to_float(gf);
    d.to_float(df);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float f, fp;
      act_both<ACT>(ef[i], f, fp);
      o1[i] = df[i] * gf[i] * fp;
      o2[i] = df[i] * f;
      o3[i] = f * gf[i];
    }
    Vec8<T> w1, w2;
    w1.from_float(o1);
    w2.from_float(o2);
    w1.store(de + it.r * sde + c);
    w2.store(dg + it.r * sdg + c);
    if (h_out != nullptr) {
      Vec8<T> w3;
      w3.from_float(o3);
      w3.store(h_out + it.r * sh + c);
    }
  }
}

// y = a + b (residual add), 16-bit
template <typename T>
__global__ void add_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ y, long long n8) {
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < n8;
       idx += (long long)gridDim.x * blockDim.x) {
    Vec8<T> va, vb;
    float fa[8], fb[8];
    va.load(a + idx * 8);
    vb.load(b + idx * 8);
    va.to_float(fa);
    vb.to_float(fb);
#pragma unroll
    for (int i = 0; i < 8; ++i) fa[i] += fb[i];
    va.from_float(fa);
    va.store(y + idx * 8);
  }
}

// AdamW with decoupled weight decay on one parameter tensor, the arithmetic of torch's fused implementation: fp32
// math per element, one rounding per stored value.  p, g, m, v have the same element type; 16-byte accesses.
//   p <- p (1 - lr wd);  m <- m + (1 - b1)(g s - m);  v <- b2 v + (1 - b2)(g s)^2;
//   p <- p - (lr / c1) m / (sqrt(v) / sqrt(c2) + eps)        c1 = 1 - b1^t, c2 = 1 - b2^t, s = grad_scale
template <typename T>
__global__ void __launch_bounds__(256)
adamw_kernel(T* __restrict__ p, const T* __restrict__ g, T* __restrict__ m, T* __restrict__ v, long long n, float lr,
             float b1, float b2, float eps, float wd, float c1, float c2, float grad_scale) {
  constexpr int V = 16 / sizeof(T);
  const long long nvec = n / V;
  const float decay = 1.f - lr * wd, step = lr / c1, rs2 = rsqrtf(c2);
  auto upd = [&](float& pf, float gf, float& mf, float& vf) {
    gf *= grad_scale;
    pf *= decay;
    mf += (1.f - b1) * (gf - mf);
    vf = b2 * vf + (1.f - b2) * gf * gf;
    pf -= step * mf / (sqrtf(vf) * rs2 + eps);
  };
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    if constexpr (sizeof(T) == 4) {
      float4 pv = reinterpret_cast<float4*>(p)[i], mv = reinterpret_cast<float4*>(m)[i], vv = reinterpret_cast<float4*>(v)[i];
      const float4 gv = reinterpret_cast<const float4*>(g)[i];
      upd(pv.x, gv.x, mv.x, vv.x); upd(pv.y, gv.y, mv.y, vv.y); upd(pv.z, gv.z, mv.z, vv.z); upd(pv.w, gv.w, mv.w, vv.w);
      reinterpret_cast<float4*>(p)[i] = pv; reinterpret_cast<float4*>(m)[i] = mv; reinterpret_cast<float4*>(v)[i] = vv;
    } else {
      Vec8<T> pv, gv, mv, vv;
      float pf[8], gf[8], mf[8], vf[8];
      pv.load(p + i * 8); gv.load(g + i * 8); mv.load(m + i * 8); vv.load(v + i * 8);
      pv.to_float(pf); gv.to_float(gf); mv.to_float(mf); vv.to_float(vf);
#pragma unroll
      for (int k = 0; k < 8; ++k) upd(pf[k], gf[k], mf[k], vf[k]);
      pv.from_float(pf); mv.from_float(mf); vv.from_float(vf);
      pv.store(p + i * 8); mv.store(m + i * 8); vv.store(v + i * 8);
    }
  }
  // tail (fewer than one vector) by the first threads of the grid
  const long long t = nvec * V + blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (t < n) {
    float pf, gf, mf, vf;
    if constexpr (sizeof(T) == 4) {
      pf = p[t]; gf = g[t]; mf = m[t]; vf = v[t];
      upd(pf, gf, mf, vf);
      p[t] = pf; m[t] = mf; v[t] = vf;
    } else if constexpr (std::is_same<T, __nv_bfloat16>::value) {
      pf = __bfloat162float(p[t]); gf = __bfloat162float(g[t]); mf = __bfloat162float(m[t]); vf = __bfloat162float(v[t]);
      upd(pf, gf, mf, vf);
      p[t] = __float2bfloat16_rn(pf); m[t] = __float2bfloat16_rn(mf); v[t] = __float2bfloat16_rn(vf);
    } else {
      pf = __half2float(p[t]); gf = __half2float(g[t]); mf = __half2float(m[t]); vf = __half2float(v[t]);
      upd(pf, gf, mf, vf);
      p[t] = __float2half_rn(pf); m[t] = __float2half_rn(mf); v[t] = __float2half_rn(vf);
    }
  }
}

// One resident wave of a grid-stride kernel: SMs x CTAs that fit per SM (asked of the runtime once per kernel).  A grid
// of a fixed 16 CTAs per SM ran as 2.67 waves of equal CTAs on kernels that fit 6 per SM, i.e. a third wave at a third
// of the machine.
template <typename K>
static int wave_grid(K kernel, int threads, long long work_items, int* cache) {
  if (*cache <= 0) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, 0) != cudaSuccess || per_sm < 1) per_sm = 4;
    *cache = per_sm * 148;
  }
  long long b = (work_items + threads - 1) / threads;
  if (b > *cache) b = *cache;
  return b < 1 ? 1 : (int)b;
}

static inline int grid_for(long long work_items, int threads, int cap_blocks) {
  long long b = (work_items + threads - 1) / threads;
  if (b > cap_blocks) b = cap_blocks;
  if (b < 1) b = 1;
  return (int)b;
}

}  // namespace fmsb

using namespace fmsb;

// row widths served by the row-in-registers kernels (the block-per-row kernels take every other width)
static bool norm_rows_ok(int H) {
  return H == 1024 || H == 1536 || H == 2048 || H == 2560 || H == 4096 || H == 5120 || H == 8192;
}
static int norm_rows_grid(int rows, int wpr) {
  const int rpc = NORM_WARPS / wpr;
  const int need = (rows + rpc - 1) / rpc;
  return need < 148 * 8 ? need : 148 * 8;
}

extern "C" int fmsb_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* h_out,
                                float* inv_rms, int rows, int H, float eps, int gemma, int dtype,
                                cudaStream_t stream) {
  if (H % 8 != 0 || H > 8 * NORM_THREADS * NORM_MAXV) return -2;
  if (rows <= 0) return 0;
  if (norm_rows_ok(H)) {
#define FMSB_NORM_FWD_R(T, VPL, WPR)                                                                            \
  rmsnorm_fwd_rows_kernel<T, VPL, WPR><<<norm_rows_grid(rows, WPR), NORM_WARPS * 32, 0, stream>>>(              \
      (const T*)x, (const T*)residual, (const T*)w, (T*)y, (T*)h_out, inv_rms, rows, eps, gemma)
#define FMSB_NORM_FWD_RT(T)                                     \
  switch (H) {                                                  \
    case 1024: FMSB_NORM_FWD_R(T, 4, 1); break;                 \
    case 1536: FMSB_NORM_FWD_R(T, 6, 1); break;                 \
    case 2048: FMSB_NORM_FWD_R(T, 4, 2); break;                 \
    case 2560: FMSB_NORM_FWD_R(T, 5, 2); break;                 \
    case 5120: FMSB_NORM_FWD_R(T, 5, 4); break;                 \
    case 8192: FMSB_NORM_FWD_R(T, 4, 8); break;                 \
    default: FMSB_NORM_FWD_R(T, 8, 2); break;                   \
  }
    if (dtype == 1) { FMSB_NORM_FWD_RT(__nv_bfloat16) } else { FMSB_NORM_FWD_RT(__half) }
#undef FMSB_NORM_FWD_RT
#undef FMSB_NORM_FWD_R
    return (int)cudaGetLastError();
  }
  const int grid = rows < 148 * 8 ? rows : 148 * 8;
  if (dtype == 1)
    rmsnorm_fwd_kernel<__nv_bfloat16><<<grid, NORM_THREADS, 0, stream>>>(
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)residual, (const __nv_bfloat16*)w, (__nv_bfloat16*)y,
        (__nv_bfloat16*)h_out, inv_rms, rows, H, eps, gemma);
  else
    rmsnorm_fwd_kernel<__half><<<grid, NORM_THREADS, 0, stream>>>((const __half*)x, (const __half*)residual,
                                                                  (const __half*)w, (__half*)y, (__half*)h_out,
                                                                  inv_rms, rows, H, eps, gemma);
  return (int)cudaGetLastError();
}

// dw_partial: [n_partial_blocks, H] fp32 scratch (may be null: no weight gradient);
// the launch uses exactly n_partial_blocks CTAs when dw_partial is given.
extern "C" int fmsb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* inv_rms,
                                const void* dres_in, void* dx, float* dw_partial, float* dw, int n_partial_blocks,
                                int rows, int H, int gemma, int dtype, cudaStream_t stream) {
  if (H % 8 != 0 || H > 8 * NORM_THREADS * NORM_MAXV) return -2;
  if (rows <= 0) return 0;
  if (norm_rows_ok(H)) {
    const bool with_dw = dw_partial != nullptr;
    if (with_dw && n_partial_blocks <= 0) return -2;
    int rgrid = 0;
#define FMSB_NORM_BWD_R(T, VPL, WPR)                                                                              \
  rgrid = norm_rows_grid(rows, WPR);                                                                              \
  if (with_dw) {                                                                                                  \
    if (rgrid > n_partial_blocks) rgrid = n_partial_blocks; /* one partial row per CTA */                         \
    rmsnorm_bwd_rows_kernel<T, VPL, WPR, true><<<rgrid, NORM_WARPS * 32, 0, stream>>>(                            \
        (const T*)dy, (const T*)x, (const T*)w, inv_rms, (const T*)dres_in, (T*)dx, dw_partial, rows, gemma);     \
  } else {                                                                                                        \
    rmsnorm_bwd_rows_kernel<T, VPL, WPR, false><<<rgrid, NORM_WARPS * 32, 0, stream>>>(                           \
        (const T*)dy, (const T*)x, (const T*)w, inv_rms, (const T*)dres_in, (T*)dx, nullptr, rows, gemma);        \
  }
#define FMSB_NORM_BWD_RT(T)                                     \
  switch (H) {                                                  \
    case 1024: FMSB_NORM_BWD_R(T, 4, 1); break;                 \
    case 1536: FMSB_NORM_BWD_R(T, 3, 2); break;                 \
    case 2048: FMSB_NORM_BWD_R(T, 4, 2); break;                 \
    case 2560: FMSB_NORM_BWD_R(T, 5, 2); break;                 \
    case 5120: FMSB_NORM_BWD_R(T, 5, 4); break;                 \
    case 8192: FMSB_NORM_BWD_R(T, 4, 8); break;                 \
    default: FMSB_NORM_BWD_R(T, 4, 4); break;                   \
  }
    if (dtype == 1) { FMSB_NORM_BWD_RT(__nv_bfloat16) } else { FMSB_NORM_BWD_RT(__half) }
#undef FMSB_NORM_BWD_RT
#undef FMSB_NORM_BWD_R
    if (with_dw && dw != nullptr) colsum_kernel<<<(H + 31) / 32, dim3(32, 8), 0, stream>>>(dw_partial, dw, rgrid, H);
    return (int)cudaGetLastError();
  }
  // without a weight gradient the kernel is light on registers: several CTAs per SM, 8 waves of rows each
  int grid = rows < 148 * 8 ? rows : 148 * 8;
  if (dw_partial != nullptr) {
    if (n_partial_blocks <= 0) return -2;
    grid = n_partial_blocks;
  }
  // vectors of 8 cached per thread: the fewer, the more CTAs (rows in flight) an SM holds
  const int maxv = H <= 8 * NORM_THREADS ? 1 : (H <= 8 * NORM_THREADS * 2 ? 2 : 4);
#define FMSB_NORM_BWD(T, MAXV, DW)                                                                                  \
  rmsnorm_bwd_kernel<T, MAXV, DW><<<grid, NORM_THREADS, 0, stream>>>((const T*)dy, (const T*)x, (const T*)w, inv_rms, \
                                                                     (const T*)dres_in, (T*)dx, dw_partial, rows, H, gemma)
#define FMSB_NORM_BWD_T(T)                                                                     \
  if (dw_partial != nullptr) {                                                                 \
    if (maxv == 1) FMSB_NORM_BWD(T, 1, true); else if (maxv == 2) FMSB_NORM_BWD(T, 2, true);   \
    else FMSB_NORM_BWD(T, 4, true);                                                            \
  } else {                                                                                     \
    if (maxv == 1) FMSB_NORM_BWD(T, 1, false); else if (maxv == 2) FMSB_NORM_BWD(T, 2, false); \
    else FMSB_NORM_BWD(T, 4, false);                                                           \
  }
  if (dtype == 1) { FMSB_NORM_BWD_T(__nv_bfloat16) } else { FMSB_NORM_BWD_T(__half) }
#undef FMSB_NORM_BWD_T
#undef FMSB_NORM_BWD
  if (dw_partial != nullptr && dw != nullptr) {
    colsum_kernel<<<(H + 31) / 32, dim3(32, 8), 0, stream>>>(dw_partial, dw, grid, H);
  }
  return (int)cudaGetLastError();
}

extern "C" int fmsb_rope(void* qk, const int* pos, const float* cos_t, const float* sin_t, int T_tokens,
                         int n_heads, int d, long long row_stride, float sign, int dtype, cudaStream_t stream) {
  if (d % 16 != 0 || row_stride % 8 != 0) return -2;
  if (T_tokens <= 0 || n_heads <= 0) return 0;
  const long long total = (long long)T_tokens * n_heads * (d / 16);
  const int grid = grid_for(total, 256, 148 * 16);
  if (dtype == 1)
    rope_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((__nv_bfloat16*)qk, pos, cos_t, sin_t, T_tokens, n_heads, d,
                                                         row_stride, sign);
  else
    rope_kernel<__half><<<grid, 256, 0, stream>>>((__half*)qk, pos, cos_t, sin_t, T_tokens, n_heads, d, row_stride,
                                                  sign);
  return (int)cudaGetLastError();
}

extern "C" int fmsb_glu_fwd(const void* e, const void* g, void* h, int rows, int I, long long se, long long sg,
                            long long sh, int act, int dtype, const int* rows_dev, cudaStream_t stream) {
  if (I % 8 != 0 || se % 8 || sg % 8 || sh % 8) return -2;
  if (rows <= 0) return 0;
  if (act < 0 || act > 2) return -2;
  static int waves[2][3];
#define FMSB_GLU_FWD(T, ACT)                                                                                      \
  glu_fwd_kernel<T, ACT><<<wave_grid(glu_fwd_kernel<T, ACT>, 256, (long long)rows * (I / 8), &waves[dtype == 1][ACT]), \
                           256, 0, stream>>>((const T*)e, (const T*)g, (T*)h, rows, I, se, sg, sh, rows_dev)
#define FMSB_GLU_FWD_T(T) \
  if (act == 0) FMSB_GLU_FWD(T, 0); else if (act == 1) FMSB_GLU_FWD(T, 1); else FMSB_GLU_FWD(T, 2);
  if (dtype == 1) { FMSB_GLU_FWD_T(__nv_bfloat16) } else { FMSB_GLU_FWD_T(__half) }
#undef FMSB_GLU_FWD_T
#undef FMSB_GLU_FWD
  return (int)cudaGetLastError();
}

extern "C" int fmsb_glu_bwd(const void* dh, const void* e, const void* g, void* de, void* dg, void* h_out, int rows,
                            int I, long long sdh, long long se, long long sg, long long sde, long long sdg,
                            long long sh, int act, int dtype, const int* rows_dev, cudaStream_t stream) {
  if (I % 8 != 0 || sdh % 8 || se % 8 || sg % 8 || sde % 8 || sdg % 8 || sh % 8) return -2;
  if (rows <= 0) return 0;
  if (act < 0 || act > 2) return -2;
  static int waves[2][3];
#define FMSB_GLU_BWD(T, ACT)                                                                                      \
  glu_bwd_kernel<T, ACT><<<wave_grid(glu_bwd_kernel<T, ACT>, 256, (long long)rows * (I / 8), &waves[dtype == 1][ACT]), \
                           256, 0, stream>>>((const T*)dh, (const T*)e, (const T*)g, (T*)de, (T*)dg, (T*)h_out, rows,  \
                                             I, sdh, se, sg, sde, sdg, sh, rows_dev)
#define FMSB_GLU_BWD_T(T) \
  if (act == 0) FMSB_GLU_BWD(T, 0); else if (act == 1) FMSB_GLU_BWD(T, 1); else FMSB_GLU_BWD(T, 2);
  if (dtype == 1) { FMSB_GLU_BWD_T(__nv_bfloat16) } else { FMSB_GLU_BWD_T(__half) }
#undef FMSB_GLU_BWD_T
#undef FMSB_GLU_BWD
  return (int)cudaGetLastError();
}

extern "C" int fmsb_add(const void* a, const void* b, void* y, long long n, int dtype, cudaStream_t stream) {
  if (n % 8 != 0) return -2;
  if (n <= 0) return 0;
  const int grid = grid_for(n / 8, 256, 148 * 16);
  if (dtype == 1)
    add_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
                                                        (__nv_bfloat16*)y, n / 8);
  else
    add_kernel<__half><<<grid, 256, 0, stream>>>((const __half*)a, (const __half*)b, (__half*)y, n / 8);
  return (int)cudaGetLastError();
}

// One AdamW step on a tensor of n elements (dtype 0 fp16, 1 bf16, 2 fp32 for p, g, m and v alike; all four 16-byte
// aligned).  c1 = 1 - beta1^t and c2 = 1 - beta2^t are formed by the caller; grad_scale multiplies the gradient first
// (clipping coefficient, 1 / accumulation steps).
extern "C" int fmsb_adamw(void* p, const void* g, void* m, void* v, long long n, float lr, float b1, float b2, float eps,
                          float wd, float c1, float c2, float grad_scale, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(m) |
       reinterpret_cast<uintptr_t>(v)) & 15u)
    return -2;
  if (c1 <= 0.f || c2 <= 0.f) return -2;
  static int waves[3];
  const int per = dtype == 2 ? 4 : 8;
  const long long items = n / per + 1;
#define FMSB_ADAMW(T, SLOT)                                                                                      \
  adamw_kernel<T><<<wave_grid(adamw_kernel<T>, 256, items, &waves[SLOT]), 256, 0, stream>>>(                     \
      (T*)p, (const T*)g, (T*)m, (T*)v, n, lr, b1, b2, eps, wd, c1, c2, grad_scale)
  if (dtype == 1) FMSB_ADAMW(__nv_bfloat16, 1);
  else if (dtype == 0) FMSB_ADAMW(__half, 0);
  else if (dtype == 2) FMSB_ADAMW(float, 2);
  else return -2;
#undef FMSB_ADAMW
  return (int)cudaGetLastError();
}
