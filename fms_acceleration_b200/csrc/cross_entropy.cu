// Cross-entropy kernels for sm_100a.
//
// Reference semantics (paths inside the reference project):
//   fms_acceleration_foak/kernels/unsloth/cross_entropy_loss.py:22-187  forward saves logsumexp,
//       loss = lse - x[label], 0 for label == -100; backward writes dloss * (softmax - onehot)
//       in place over the logits.  The reference splits vocabularies above 65536 into chunks and
//       combines with torch.logsumexp; this kernel runs an online logsumexp over any vocabulary
//       size in one launch.
//   fms_acceleration_foak/fused_ops/liger_ce/cross_entropy.py:32-179    online softmax, loss AND
//       gradient computed in the forward, label smoothing, mean/sum reduction via a scale.
//
// One CTA per row.  dtype of the logits: 0 = fp16, 1 = bf16, 2 = fp32.
#include "common.cuh"

namespace fmsb {

constexpr int CE_THREADS = 512;

template <typename T>
__device__ __forceinline__ float ld_as_float(const T* p);
template <>
__device__ __forceinline__ float ld_as_float<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ld_as_float<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <>
__device__ __forceinline__ float ld_as_float<__half>(const __half* p) { return __half2float(*p); }

template <typename T>
__device__ __forceinline__ void st_from_float(T* p, float v);
template <>
__device__ __forceinline__ void st_from_float<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void st_from_float<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ void st_from_float<__half>(__half* p, float v) { *p = __float2half_rn(v); }

// elements per 16-byte vector
template <typename T>
struct VecN { static constexpr int n = 16 / sizeof(T); };

template <typename T>
__device__ __forceinline__ void load_vec(const T* p, float* f) {
  constexpr int n = VecN<T>::n;
  uint4 u = *reinterpret_cast<const uint4*>(p);
  const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
  for (int i = 0; i < n; ++i) f[i] = ld_as_float<T>(e + i);
}
template <typename T>
__device__ __forceinline__ void store_vec(T* p, const float* f) {
  constexpr int n = VecN<T>::n;
  uint4 u;
  T* e = reinterpret_cast<T*>(&u);
#pragma unroll
  for (int i = 0; i < n; ++i) st_from_float<T>(e + i, f[i]);
  *reinterpret_cast<uint4*>(p) = u;
}

struct MaxSum {
  float m, s, t;  // running max, sum of exp(x - m), plain sum of x (for label smoothing)
};
__device__ __forceinline__ MaxSum combine(MaxSum a, MaxSum b) {
  MaxSum r;
  r.m = fmaxf(a.m, b.m);
  r.s = (a.m == -INFINITY ? 0.f : a.s * __expf(a.m - r.m)) + (b.m == -INFINITY ? 0.f : b.s * __expf(b.m - r.m));
  r.t = a.t + b.t;
  return r;
}

// loss[row], lse[row]; when WRITE_GRAD the logits row is overwritten with
//   grad_scale(row) * (softmax - (1-eps)*onehot - eps/V),   grad_scale = *scale_ptr * row_scale[row]
// (either factor may be absent = 1).  Rows with label == ignore_index get loss 0 and zero gradient.
template <typename T, bool WRITE_GRAD>
__global__ void __launch_bounds__(CE_THREADS)
ce_kernel(T* logits, long long row_stride, const long long* __restrict__ labels, float* __restrict__ loss,
          float* __restrict__ lse_out, const float* __restrict__ scale_ptr, const float* __restrict__ row_scale,
          int V, int ignore_index, float label_smoothing) {
  __shared__ MaxSum red[CE_THREADS / 32];
  __shared__ MaxSum total;
  const int row = blockIdx.x;
  T* x = logits + (long long)row * row_stride;
  const long long label = labels[row];
  constexpr int n = VecN<T>::n;
  const bool vec_ok = ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
  const int nvec = vec_ok ? V / n : 0;

  if (label == ignore_index) {
    if (threadIdx.x == 0) {
      loss[row] = 0.f;
      if (lse_out != nullptr) lse_out[row] = 0.f;
    }
    if (WRITE_GRAD) {
      float z[n];
#pragma unroll
      for (int i = 0; i < n; ++i) z[i] = 0.f;
      for (int v = threadIdx.x; v < nvec; v += CE_THREADS) store_vec<T>(x + v * n, z);
      for (int i = nvec * n + threadIdx.x; i < V; i += CE_THREADS) st_from_float<T>(x + i, 0.f);
    }
    return;
  }

  MaxSum acc{-INFINITY, 0.f, 0.f};
  // four 16-byte loads in flight per thread, then one running-maximum update for the four vectors together
  constexpr int U = 4;
  for (int v0 = threadIdx.x; v0 < nvec; v0 += CE_THREADS * U) {
    uint4 raw[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int v = v0 + u * CE_THREADS;
      if (v < nvec) raw[u] = *reinterpret_cast<const uint4*>(x + v * n);
    }
    float f[U][n];
    float mx = -INFINITY;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const bool ok = v0 + u * CE_THREADS < nvec;
      const T* e = reinterpret_cast<const T*>(&raw[u]);
#pragma unroll
      for (int i = 0; i < n; ++i) {
        f[u][i] = ok ? ld_as_float<T>(e + i) : -INFINITY;
        mx = fmaxf(mx, f[u][i]);
      }
    }
    const float nm = fmaxf(acc.m, mx);
    float s = acc.m == -INFINITY ? 0.f : acc.s * __expf(acc.m - nm);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const bool ok = v0 + u * CE_THREADS < nvec;
#pragma unroll
      for (int i = 0; i < n; ++i) {
        s += __expf(f[u][i] - nm);  // exp(-inf) = 0 for the slots beyond the row
        if (ok) acc.t += f[u][i];
      }
    }
    acc.m = nm;
    acc.s = s;
  }
  for (int i = nvec * n + threadIdx.x; i < V; i += CE_THREADS) {
    const float f = ld_as_float<T>(x + i);
    const float nm = fmaxf(acc.m, f);
    acc.s = (acc.m == -INFINITY ? 0.f : acc.s * __expf(acc.m - nm)) + __expf(f - nm);
    acc.m = nm;
    acc.t += f;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxSum other;
    other.m = __shfl_xor_sync(0xffffffffu, acc.m, o);
    other.s = __shfl_xor_sync(0xffffffffu, acc.s, o);
    other.t = __shfl_xor_sync(0xffffffffu, acc.t, o);
    acc = combine(acc, other);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = acc;
  __syncthreads();
  if (warp == 0) {
    MaxSum a = lane < CE_THREADS / 32 ? red[lane] : MaxSum{-INFINITY, 0.f, 0.f};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      MaxSum other;
      other.m = __shfl_xor_sync(0xffffffffu, a.m, o);
      other.s = __shfl_xor_sync(0xffffffffu, a.s, o);
      other.t = __shfl_xor_sync(0xffffffffu, a.t, o);
      a = combine(a, other);
    }
    if (lane == 0) total = a;
  }
  __syncthreads();
  const float lse = total.m + __logf(total.s);
  const float xy = ld_as_float<T>(x + label);
  if (threadIdx.x == 0) {
    float l = lse - xy;
    if (label_smoothing > 0.f) {
      const float smooth = lse - total.t / (float)V;
      l = (1.f - label_smoothing) * l + label_smoothing * smooth;
    }
    loss[row] = l;
    if (lse_out != nullptr) lse_out[row] = lse;
  }
  if (WRITE_GRAD) {
    __syncthreads();  // x[label] has been read by everyone before it is overwritten
    float sc = 1.f;
    if (scale_ptr != nullptr) sc *= *scale_ptr;
    if (row_scale != nullptr) sc *= row_scale[row];
    const float eps_v = label_smoothing / (float)V;
    for (int v = threadIdx.x; v < nvec; v += CE_THREADS) {
      float f[n];
      load_vec<T>(x + v * n, f);
#pragma unroll
      for (int i = 0; i < n; ++i) {
        float g = __expf(f[i] - lse) - eps_v;
        if ((long long)(v * n + i) == label) g -= (1.f - label_smoothing);
        f[i] = g * sc;
      }
      store_vec<T>(x + v * n, f);
    }
    for (int i = nvec * n + threadIdx.x; i < V; i += CE_THREADS) {
      float g = __expf(ld_as_float<T>(x + i) - lse) - eps_v;
      if ((long long)i == label) g -= (1.f - label_smoothing);
      st_from_float<T>(x + i, g * sc);
    }
  }
}

// Separate backward: dst[row] = dloss[row] * (exp(src[row] - lse[row]) - onehot); dst may be src (in place, as the
// reference does) or another matrix (no clone of the logits is needed for an out-of-place gradient).  16-byte loads
// and stores when both rows are aligned; grid (rows, chunks of the vocabulary).
template <typename T>
__global__ void __launch_bounds__(256)
ce_bwd_kernel(const T* src, long long src_stride, T* dst, long long dst_stride, const long long* __restrict__ labels,
              const float* __restrict__ lse, const float* __restrict__ dloss, long long dloss_stride, int V,
              int ignore_index) {
  constexpr int n = VecN<T>::n;
  const int row = blockIdx.x;
  const T* x = src + (long long)row * src_stride;
  T* y = dst + (long long)row * dst_stride;
  const long long label = labels[row];
  const float l = lse[row];
  const bool dead = label == ignore_index;
  const float d = dead ? 0.f : dloss[row * dloss_stride];
  const bool vec_ok = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
  const int nvec = vec_ok ? V / n : 0;
  // four vectors per thread and trip: the loads go out together
  constexpr int U = 4;
  const int stride = gridDim.y * blockDim.x;
  for (int v0 = blockIdx.y * blockDim.x + threadIdx.x; v0 < nvec; v0 += stride * U) {
    uint4 raw[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int v = v0 + u * stride;
      raw[u] = (!dead && v < nvec) ? *reinterpret_cast<const uint4*>(x + v * n) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int v = v0 + u * stride;
      if (v >= nvec) continue;
      float f[n];
      const T* e = reinterpret_cast<const T*>(&raw[u]);
#pragma unroll
      for (int i = 0; i < n; ++i) {
        float g = 0.f;
        if (!dead) {
          g = __expf(ld_as_float<T>(e + i) - l);
          if ((long long)(v * n + i) == label) g -= 1.f;
          g *= d;
        }
        f[i] = g;
      }
      store_vec<T>(y + v * n, f);
    }
  }
  for (int i = nvec * n + blockIdx.y * blockDim.x + threadIdx.x; i < V; i += gridDim.y * blockDim.x) {
    float g = 0.f;
    if (!dead) {
      g = __expf(ld_as_float<T>(x + i) - l);
      if ((long long)i == label) g -= 1.f;
      g *= d;
    }
    st_from_float<T>(y + i, g);
  }
}

// out[0] = number of labels != ignore_index ; out[1] = 1 / max(count, 1)
__global__ void count_valid_kernel(const long long* __restrict__ labels, long long n, int ignore_index,
                                   float* __restrict__ out) {
  __shared__ float red[32];
  float c = 0.f;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) c += labels[i] != ignore_index ? 1.f : 0.f;
  c = warp_sum(c);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < blockDim.x / 32 ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) {
      out[0] = t;
      out[1] = 1.f / fmaxf(t, 1.f);
    }
  }
}

}  // namespace fmsb

using namespace fmsb;

extern "C" int fmsb_ce(void* logits, long long row_stride, const long long* labels, float* loss, float* lse,
                       const float* scale_ptr, const float* row_scale, int rows, int V, int ignore_index,
                       float label_smoothing, int write_grad, int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
#define CE_LAUNCH(T)                                                                                            \
  if (write_grad)                                                                                               \
    ce_kernel<T, true><<<rows, CE_THREADS, 0, stream>>>((T*)logits, row_stride, labels, loss, lse, scale_ptr,   \
                                                        row_scale, V, ignore_index, label_smoothing);           \
  else                                                                                                          \
    ce_kernel<T, false><<<rows, CE_THREADS, 0, stream>>>((T*)logits, row_stride, labels, loss, lse, scale_ptr,  \
                                                         row_scale, V, ignore_index, label_smoothing);
  if (dtype == 0) {
    CE_LAUNCH(__half)
  } else if (dtype == 1) {
    CE_LAUNCH(__nv_bfloat16)
  } else if (dtype == 2) {
    CE_LAUNCH(float)
  } else {
    return -2;
  }
#undef CE_LAUNCH
  return (int)cudaGetLastError();
}

extern "C" int fmsb_ce_bwd(const void* logits, long long row_stride, void* dlogits, long long d_stride,
                           const long long* labels, const float* lse, const float* dloss, long long dloss_stride,
                           int rows, int V, int ignore_index, int dtype, cudaStream_t stream) {
  if (rows <= 0) return 0;
  // 256 threads x 4 vectors of 16 bytes per trip, about four trips per thread: CTAs long enough to amortise the
  // row's label / lse / dloss look-ups
  const int per_vec = dtype == 2 ? 4 : 8;
  int chunks = (V / per_vec + 4095) / 4096;
  if (chunks < 1) chunks = 1;
  if (chunks > 65535) chunks = 65535;
  dim3 grid(rows, chunks);
  if (dtype == 0)
    ce_bwd_kernel<__half><<<grid, 256, 0, stream>>>((const __half*)logits, row_stride, (__half*)dlogits, d_stride,
                                                    labels, lse, dloss, dloss_stride, V, ignore_index);
  else if (dtype == 1)
    ce_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)logits, row_stride,
                                                           (__nv_bfloat16*)dlogits, d_stride, labels, lse, dloss,
                                                           dloss_stride, V, ignore_index);
  else if (dtype == 2)
    ce_bwd_kernel<float><<<grid, 256, 0, stream>>>((const float*)logits, row_stride, (float*)dlogits, d_stride, labels,
                                                   lse, dloss, dloss_stride, V, ignore_index);
  else
    return -2;
  return (int)cudaGetLastError();
}

extern "C" int fmsb_count_valid(const long long* labels, long long n, int ignore_index, float* out,
                                cudaStream_t stream) {
  count_valid_kernel<<<1, 1024, 0, stream>>>(labels, n, ignore_index, out);
  return (int)cudaGetLastError();
}
