// RMSNorm backward for callers that cannot allocate device memory: the partial sums of the weight gradient are
// kept in a scratch array that is compiled into the library instead of one supplied by the caller.  See
// no_alloc.h for the contract.  This entry point has no counterpart in the reference project.
#include "no_alloc.h"

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstring>

#include "common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kMaxVec = FMSB_NOALLOC_MAX_H / 8 / kThreads;  // 16-byte vectors cached per thread (= 4)

// The scratch itself.  In host code this name is only a handle for the runtime's symbol table, NOT a device
// address; the launcher below asks the runtime for the real address once per device.
static __device__ __align__(256) float g_dw_partial[FMSB_NOALLOC_PARTIAL_ROWS * FMSB_NOALLOC_MAX_H];

thread_local char t_last_error[256] = "";

void set_error(const char* fmt, long long a = 0, long long b = 0) { snprintf(t_last_error, sizeof(t_last_error), fmt, a, b); }

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&f)[8]);
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __bfloat1622float2(h[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}
template <>
__device__ __forceinline__ void load8<__half>(const __half* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __half22float2(h[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&f)[8]);
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  u.x = fmsb::pack_bf16x2(f[0], f[1]);
  u.y = fmsb::pack_bf16x2(f[2], f[3]);
  u.z = fmsb::pack_bf16x2(f[4], f[5]);
  u.w = fmsb::pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}
template <>
__device__ __forceinline__ void store8<__half>(__half* p, const float (&f)[8]) {
  uint4 u;
  u.x = fmsb::pack_f16x2(f[0], f[1]);
  u.y = fmsb::pack_f16x2(f[2], f[3]);
  u.z = fmsb::pack_f16x2(f[4], f[5]);
  u.w = fmsb::pack_f16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

// One CTA walks rows blockIdx.x, blockIdx.x + gridDim.x, ...; it writes its partial dw into row blockIdx.x of
// `partial` (row stride FMSB_NOALLOC_MAX_H).
template <typename T>
__global__ void __launch_bounds__(kThreads)
rmsnorm_bwd_noalloc_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
                           const float* __restrict__ inv_rms, const T* __restrict__ dres_in, T* __restrict__ dx,
                           float* __restrict__ partial, int rows, int H, int gemma) {
  __shared__ float red[kThreads / 32];
  const int nvec = H / 8;
  float wf[kMaxVec][8], dwacc[kMaxVec][8];
#pragma unroll
  for (int j = 0; j < kMaxVec; ++j) {
    const int v = threadIdx.x + j * kThreads;
#pragma unroll
    for (int i = 0; i < 8; ++i) dwacc[j][i] = 0.f;
    if (v < nvec) {
      load8<T>(w + v * 8, wf[j]);
      if (gemma) {
#pragma unroll
        for (int i = 0; i < 8; ++i) wf[j][i] += 1.f;
      }
    }
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const float inv = inv_rms[row];
    float xh[kMaxVec][8], g[kMaxVec][8];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxVec; ++j) {
      const int v = threadIdx.x + j * kThreads;
      if (v < nvec) {
        float dyf[8];
        load8<T>(x + (long long)row * H + v * 8, xh[j]);
        load8<T>(dy + (long long)row * H + v * 8, dyf);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xh[j][i] *= inv;
          g[j][i] = dyf[i] * wf[j][i];
          dot += g[j][i] * xh[j][i];
          dwacc[j][i] += dyf[i] * xh[j][i];
        }
      }
    }
    dot = fmsb::warp_sum(dot);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = dot;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < kThreads / 32; ++i) tot += red[i];
    const float c = tot / (float)H;
#pragma unroll
    for (int j = 0; j < kMaxVec; ++j) {
      const int v = threadIdx.x + j * kThreads;
      if (v < nvec) {
        float out[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) out[i] = inv * (g[j][i] - xh[j][i] * c);
        if (dres_in != nullptr) {
          float rf[8];
          load8<T>(dres_in + (long long)row * H + v * 8, rf);
#pragma unroll
          for (int i = 0; i < 8; ++i) out[i] += rf[i];
        }
        store8<T>(dx + (long long)row * H + v * 8, out);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < kMaxVec; ++j) {
    const int v = threadIdx.x + j * kThreads;
    if (v < nvec) {
      float* dst = partial + (long long)blockIdx.x * FMSB_NOALLOC_MAX_H + v * 8;
      *reinterpret_cast<float4*>(dst) = make_float4(dwacc[j][0], dwacc[j][1], dwacc[j][2], dwacc[j][3]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(dwacc[j][4], dwacc[j][5], dwacc[j][6], dwacc[j][7]);
    }
  }
}

__global__ void colsum_noalloc_kernel(const float* __restrict__ partial, float* __restrict__ dw, int nblocks, int H) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float s = 0.f;
  for (int b = 0; b < nblocks; ++b) s += partial[(long long)b * FMSB_NOALLOC_MAX_H + c];
  dw[c] = s;
}

// Device address of the scratch array, looked up once per device (with that device current).
constexpr int kMaxDevices = 64;
std::atomic<float*> g_scratch_addr[kMaxDevices] = {};

int scratch_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return FMSB_NOALLOC_ERR_SETUP;
  if (g_scratch_addr[dev].load(std::memory_order_acquire) == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_dw_partial);
    if (e != cudaSuccess || p == nullptr) {
      set_error("cudaGetSymbolAddress for the built-in scratch failed on device %lld (CUDA error %lld)", dev, (long long)e);
      return e != cudaSuccess ? (int)e : FMSB_NOALLOC_ERR_SETUP;
    }
    g_scratch_addr[dev].store(p, std::memory_order_release);  // every thread that looks it up stores the same value
  }
  *out = g_scratch_addr[dev].load(std::memory_order_acquire);
  return 0;
}

}  // namespace

extern "C" const char* fmsb_noalloc_last_error(void) { return t_last_error; }

extern "C" int fmsb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* inv_rms,
                                        const void* dres_in, void* dx, float* dw, int rows, int H, int gemma, int dtype,
                                        cudaStream_t stream) {
  t_last_error[0] = '\0';
  if (dy == nullptr || x == nullptr || w == nullptr || inv_rms == nullptr || dx == nullptr || dw == nullptr ||
      rows < 0 || H <= 0 || H % 8 != 0 || (dtype != 0 && dtype != 1)) {
    set_error("bad argument (null pointer, H not a positive multiple of 8, or dtype not 0/1): rows=%lld H=%lld", rows, H);
    return FMSB_NOALLOC_ERR_BAD_ARG;
  }
  // the kernels move 16 bytes per access on every row-sized operand; a pointer off that boundary would fault
  // on the device, so it is refused here instead
  const void* const vec_ptrs[] = {dy, x, w, dres_in, dx};
  for (const void* q : vec_ptrs) {
    if ((reinterpret_cast<uintptr_t>(q) & 15u) != 0) {
      set_error("dy, x, w, dres_in and dx must be 16-byte aligned (rows=%lld H=%lld)", rows, H);
      return FMSB_NOALLOC_ERR_BAD_ARG;
    }
  }
  if (((reinterpret_cast<uintptr_t>(inv_rms) | reinterpret_cast<uintptr_t>(dw)) & 3u) != 0) {
    set_error("inv_rms and dw must be 4-byte aligned (rows=%lld H=%lld)", rows, H);
    return FMSB_NOALLOC_ERR_BAD_ARG;
  }
  if (H > FMSB_NOALLOC_MAX_H) {
    set_error("row width H=%lld exceeds the built-in scratch (at most %lld elements per row)", H, FMSB_NOALLOC_MAX_H);
    return FMSB_NOALLOC_ERR_TOO_LARGE;
  }
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  if (rows == 0) {
    // still define dw: no rows contribute
    cudaError_t e = cudaMemsetAsync(dw, 0, sizeof(float) * H, stream);
    return (int)e;
  }
  const int grid = rows < FMSB_NOALLOC_PARTIAL_ROWS ? rows : FMSB_NOALLOC_PARTIAL_ROWS;
  if (dtype == 1)
    rmsnorm_bwd_noalloc_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(
        (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, inv_rms,
        (const __nv_bfloat16*)dres_in, (__nv_bfloat16*)dx, scratch, rows, H, gemma);
  else
    rmsnorm_bwd_noalloc_kernel<__half><<<grid, kThreads, 0, stream>>>((const __half*)dy, (const __half*)x,
                                                                      (const __half*)w, inv_rms, (const __half*)dres_in,
                                                                      (__half*)dx, scratch, rows, H, gemma);
  colsum_noalloc_kernel<<<(H + 255) / 256, 256, 0, stream>>>(scratch, dw, grid, H);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) set_error("kernel launch failed (CUDA error %lld)", (long long)e);
  return (int)e;
}
