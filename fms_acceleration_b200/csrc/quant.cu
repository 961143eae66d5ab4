// 4-bit blockwise (NF4 / FP4, optional double quantisation of the block scales) and GPTQ
// 2/4/8-bit weight formats: quantise, dequantise.
//
// What these replace in the reference project:
//   the bitsandbytes C library calls in fms_acceleration_foak/fused_ops/unsloth_lora/utils.py:86-141
//     (cdequantize_blockwise_fp32 on the 8-bit block scales, `+ offset`, then
//      cdequantize_blockwise_{fp16,bf16}_nf4 on the packed weights) and the quantise-at-load
//      done by bitsandbytes for fms_acceleration_peft/framework_plugin_bnb.py:143-158;
//   the Triton dequant_kernel_248 in
//     fms_acceleration_foak/fused_ops/unsloth_lora/gptq/triton/kernels.py:53-122 and
//     fms_acceleration_peft/gptqmodel/nn_modules/triton_utils/dequant.py:36-100.
//
// 4-bit blockwise layout: the tensor is flattened; each run of `blocksize` (a multiple of 32)
// values shares one scale absmax = max|w|; value i is stored as the index of the code-book entry
// nearest to w/absmax; two indices per byte, the earlier element in the high nibble.  With
// double quantisation the fp32 scales have their mean (`offset`) removed and are themselves
// stored as 8-bit indices into a 256-entry code book with one fp32 scale per 256 block scales.
#include "common.cuh"

namespace fmsb {

// ---------------------------------------------------------------------------- quantise 4-bit
template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }

// one warp per block of `blocksize` values
template <typename T>
__global__ void quant4_kernel(const T* __restrict__ w, long long n, const float* __restrict__ code16, int blocksize,
                              uint8_t* __restrict__ packed, float* __restrict__ absmax) {
  __shared__ float code[16];
  if (threadIdx.x < 16) code[threadIdx.x] = code16[threadIdx.x];
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const long long warp_global = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const long long nblocks = (n + blocksize - 1) / blocksize;
  for (long long b = warp_global; b < nblocks; b += nwarps) {
    const long long base = b * blocksize;
    float mx = 0.f;
    for (int i = lane; i < blocksize; i += 32) {
      const long long idx = base + i;
      if (idx < n) mx = fmaxf(mx, fabsf(to_f<T>(w[idx])));
    }
    mx = warp_max(mx);
    if (lane == 0) absmax[b] = mx;
    const float inv = mx > 0.f ? 1.f / mx : 0.f;
    // each lane packs pairs (2 values -> 1 byte)
    for (int pair = lane; pair < blocksize / 2; pair += 32) {
      uint32_t byte = 0;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const long long idx = base + 2 * pair + h;
        const float v = idx < n ? to_f<T>(w[idx]) * inv : 0.f;
        int best = 0;
        float bd = fabsf(v - code[0]);
#pragma unroll
        for (int c = 1; c < 16; ++c) {
          const float d = fabsf(v - code[c]);
          if (d < bd) {
            bd = d;
            best = c;
          }
        }
        byte |= (uint32_t)best << (h == 0 ? 4 : 0);
      }
      const long long pidx = (base >> 1) + pair;
      if (2 * pidx < n) packed[pidx] = (uint8_t)byte;
    }
  }
}

// 8-bit blockwise quantisation of (v - offset) against a sorted 256-entry code book; one CTA of
// 256 threads per block of 256 values.
__global__ void quant8_kernel(const float* __restrict__ v, long long n, float offset, const float* __restrict__ code256,
                              uint8_t* __restrict__ q, float* __restrict__ absmax2) {
  __shared__ float code[256];
  __shared__ float red[8];
  code[threadIdx.x] = code256[threadIdx.x];
  const long long idx = blockIdx.x * 256LL + threadIdx.x;
  const float x = idx < n ? v[idx] - offset : 0.f;
  float mx = warp_max(fabsf(x));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) mx = fmaxf(mx, red[i]);
  if (threadIdx.x == 0) absmax2[blockIdx.x] = mx;
  if (idx >= n) return;
  const float t = mx > 0.f ? x / mx : 0.f;
  // binary search for the nearest entry of the sorted code book
  int lo = 0, hi = 255;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (code[mid] <= t) lo = mid; else hi = mid;
  }
  q[idx] = (uint8_t)((fabsf(code[hi] - t) < fabsf(t - code[lo])) ? hi : lo);
}

// ---------------------------------------------------------------------------- dequantise 4-bit
// Per trip a warp expands 512 packed bytes into 2 KB.  Lane l takes the four 4-byte words at l*4 + {0, 128, 256, 384}
// of the warp's bytes and writes the four 16-byte results at l*16 + {0, 512, 1024, 1536}, so every load instruction
// covers 128 contiguous bytes and every store instruction 512.  (A lane that expands 16 contiguous bytes writes its 64
// output bytes with four stores that are 64 bytes apart from the neighbouring lane's: 16 cache lines per store
// instruction, four times the requests the same bytes need.)  The 256-entry code book of the double-quantised scales
// sits in shared memory.
template <typename T>
__global__ void __launch_bounds__(256)
dequant4_warp_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ absmax,
                     const uint8_t* __restrict__ absmax_q, const float* __restrict__ code256,
                     const float* __restrict__ absmax2, float offset, const float* __restrict__ code16, int blocksize,
                     int block_shift, long long n, T* __restrict__ out) {
  __shared__ float code[16];
  __shared__ float code2[256];
  if (threadIdx.x < 16) code[threadIdx.x] = code16[threadIdx.x];
  if (absmax_q != nullptr) code2[threadIdx.x] = code256[threadIdx.x];
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  const long long trips = (n + 1023) / 1024;
  for (long long t = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5); t < trips; t += nwarps) {
    const long long e_warp = t * 1024;
    uint32_t word[4];
    float scale[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const long long e0 = e_warp + (k * 32 + lane) * 8;
      word[k] = 0u;
      scale[k] = 0.f;
      if (e0 < n) {
        word[k] = *reinterpret_cast<const uint32_t*>(packed + (e0 >> 1));
        const long long b = block_shift >= 0 ? (e0 >> block_shift) : e0 / blocksize;
        scale[k] = absmax_q != nullptr ? code2[absmax_q[b]] * absmax2[b >> 8] + offset : absmax[b];
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const long long e0 = e_warp + (k * 32 + lane) * 8;
      if (e0 >= n) continue;
      uint4 o;
      uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int bi = 0; bi < 4; ++bi) {
        const uint32_t byte = (word[k] >> (8 * bi)) & 0xff;
        const float hi = code[byte >> 4] * scale[k];
        const float lo = code[byte & 15] * scale[k];
        ow[bi] = std::is_same<T, __nv_bfloat16>::value ? pack_bf16x2(hi, lo) : pack_f16x2(hi, lo);
      }
      *reinterpret_cast<uint4*>(out + e0) = o;
    }
  }
}

// ---------------------------------------------------------------------------- GPTQ dequantise
// qweight int32 [in*bits/32, out] packs consecutive input rows along the bit positions;
// qzeros int32 [groups, out*bits/32] packs along the output columns; scales [groups, out];
// g_idx int32 [in] (may be null: group = row / group_size).  Output W[in, out]:
//   W[r, c] = scales[g, c] * (field(qweight[r / per, c], r % per) - (field(qzeros[g, c / per], c % per) + zero_offset))
template <typename T>
__global__ void gptq_dequant_kernel(const int* __restrict__ qweight, const T* __restrict__ scales,
                                    const int* __restrict__ qzeros, const int* __restrict__ g_idx, int in_features,
                                    int out_features, int bits, int group_size, int zero_offset,
                                    T* __restrict__ out, long long ldo) {
  const int per = 32 / bits;
  const uint32_t mask = (1u << bits) - 1u;
  const long long total = (long long)in_features * out_features;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(idx / out_features);
    const int c = (int)(idx % out_features);
    const int g = g_idx != nullptr ? g_idx[r] : r / group_size;
    const uint32_t qw = (uint32_t)qweight[(long long)(r / per) * out_features + c];
    const uint32_t qz = (uint32_t)qzeros[(long long)g * (out_features / per) + c / per];
    const int wv = (int)((qw >> ((r % per) * bits)) & mask);
    const int zv = (int)((qz >> ((c % per) * bits)) & mask) + zero_offset;
    const float s = to_f<T>(scales[(long long)g * out_features + c]);
    const float v = s * (float)(wv - zv);
    const long long o = (long long)r * ldo + c;
    if (std::is_same<T, __nv_bfloat16>::value)
      reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(v);
    else
      reinterpret_cast<__half*>(out)[o] = __float2half_rn(v);
  }
}

// Vectorised form used whenever out_features % 8 == 0: one thread expands one packed word row (32/BITS input rows)
// of 8 consecutive output columns: 8 coalesced int32 loads, then 32/BITS coalesced 16-byte stores.  Every packed
// word is read once (the scalar kernel above reads it 32/BITS times and stores 2 bytes at a time).
template <typename T, int BITS>
__global__ void gptq_dequant_vec_kernel(const int* __restrict__ qweight, const T* __restrict__ scales,
                                        const int* __restrict__ qzeros, const int* __restrict__ g_idx,
                                        int in_features, int out_features, int group_size, int zero_offset,
                                        T* __restrict__ out, long long ldo) {
  constexpr int PER = 32 / BITS;
  constexpr uint32_t MASK = (1u << BITS) - 1u;
  const int cgroups = out_features / 8;
  const long long total = (long long)(in_features / PER) * cgroups;
  const int zwords = out_features / PER;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int pr = (int)(idx / cgroups);
    const int c0 = (int)(idx % cgroups) * 8;
    const uint4 qa = *reinterpret_cast<const uint4*>(qweight + (long long)pr * out_features + c0);
    const uint4 qb = *reinterpret_cast<const uint4*>(qweight + (long long)pr * out_features + c0 + 4);
    const uint32_t qw[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
    const int r0 = pr * PER;
    int g_prev = -1;
    float sc[8], zs[8];  // scale and scale * zero per column for the current group
#pragma unroll 1
    for (int j = 0; j < PER; ++j) {
      const int r = r0 + j;
      const int g = g_idx != nullptr ? g_idx[r] : r / group_size;
      if (g != g_prev) {
        g_prev = g;
        const uint4 sv = *reinterpret_cast<const uint4*>(scales + (long long)g * out_features + c0);
        const T* sp = reinterpret_cast<const T*>(&sv);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int c = c0 + i;
          const uint32_t qz = (uint32_t)qzeros[(long long)g * zwords + c / PER];
          const int zv = (int)((qz >> ((c % PER) * BITS)) & MASK) + zero_offset;
          sc[i] = to_f<T>(sp[i]);
          zs[i] = (float)zv;
        }
      }
      float v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = sc[i] * ((float)((qw[i] >> (j * BITS)) & MASK) - zs[i]);
      uint4 o;
      if (std::is_same<T, __nv_bfloat16>::value) {
        o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
        o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
      } else {
        o.x = pack_f16x2(v[0], v[1]); o.y = pack_f16x2(v[2], v[3]);
        o.z = pack_f16x2(v[4], v[5]); o.w = pack_f16x2(v[6], v[7]);
      }
      *reinterpret_cast<uint4*>(out + (long long)r * ldo + c0) = o;
    }
  }
}

template <typename T>
static int gptq_launch_vec(const int* qweight, const T* scales, const int* qzeros, const int* g_idx, int in_features,
                           int out_features, int bits, int group_size, int zero_offset, T* out, long long ldo,
                           cudaStream_t stream) {
  const int per = 32 / bits;
  const long long total = (long long)(in_features / per) * (out_features / 8);
  long long ctas = (total + 255) / 256;
  if (ctas > 148 * 32) ctas = 148 * 32;
  if (bits == 4)
    gptq_dequant_vec_kernel<T, 4><<<(int)ctas, 256, 0, stream>>>(qweight, scales, qzeros, g_idx, in_features,
                                                                out_features, group_size, zero_offset, out, ldo);
  else if (bits == 8)
    gptq_dequant_vec_kernel<T, 8><<<(int)ctas, 256, 0, stream>>>(qweight, scales, qzeros, g_idx, in_features,
                                                                out_features, group_size, zero_offset, out, ldo);
  else
    gptq_dequant_vec_kernel<T, 2><<<(int)ctas, 256, 0, stream>>>(qweight, scales, qzeros, g_idx, in_features,
                                                                out_features, group_size, zero_offset, out, ldo);
  return (int)cudaGetLastError();
}

}  // namespace fmsb

using namespace fmsb;

extern "C" int fmsb_quant4(const void* w, long long n, const float* code16, int blocksize, void* packed,
                           float* absmax, int dtype, cudaStream_t stream) {
  if (blocksize % 32 != 0 || n % 2 != 0) return -2;
  if (n <= 0) return 0;
  const long long nblocks = (n + blocksize - 1) / blocksize;
  long long ctas = (nblocks + 7) / 8;
  if (ctas > 148 * 32) ctas = 148 * 32;
  if (dtype == 0)
    quant4_kernel<__half><<<(int)ctas, 256, 0, stream>>>((const __half*)w, n, code16, blocksize, (uint8_t*)packed,
                                                         absmax);
  else if (dtype == 1)
    quant4_kernel<__nv_bfloat16><<<(int)ctas, 256, 0, stream>>>((const __nv_bfloat16*)w, n, code16, blocksize,
                                                                (uint8_t*)packed, absmax);
  else if (dtype == 2)
    quant4_kernel<float><<<(int)ctas, 256, 0, stream>>>((const float*)w, n, code16, blocksize, (uint8_t*)packed,
                                                        absmax);
  else
    return -2;
  return (int)cudaGetLastError();
}

extern "C" int fmsb_quant8_blockwise(const float* v, long long n, float offset, const float* code256, void* q,
                                     float* absmax2, cudaStream_t stream) {
  if (n <= 0) return 0;
  quant8_kernel<<<(int)((n + 255) / 256), 256, 0, stream>>>(v, n, offset, code256, (uint8_t*)q, absmax2);
  return (int)cudaGetLastError();
}

// absmax_q == nullptr: plain fp32 block scales in `absmax`; otherwise double-quantised scales.
extern "C" int fmsb_dequant4(const void* packed, const float* absmax, const void* absmax_q, const float* code256,
                             const float* absmax2, float offset, const float* code16, int blocksize, long long n,
                             void* out, int dtype, cudaStream_t stream) {
  if (blocksize % 32 != 0 || n % 32 != 0) return -2;
  if (n <= 0) return 0;
  if (dtype != 0 && dtype != 1) return -2;
  // shift for the usual power-of-two block sizes, a division otherwise
  int block_shift = -1;
  if ((blocksize & (blocksize - 1)) == 0) {
    block_shift = 0;
    while ((1 << block_shift) < blocksize) ++block_shift;
  }
  static int wave[2];
  int& per_wave = wave[dtype];
  if (per_wave <= 0) {
    int per_sm = 0;
    cudaError_t e = dtype == 1 ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, dequant4_warp_kernel<__nv_bfloat16>, 256, 0)
                               : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, dequant4_warp_kernel<__half>, 256, 0);
    per_wave = (e == cudaSuccess && per_sm > 0 ? per_sm : 4) * 148;
  }
  long long ctas = ((n + 1023) / 1024 + 7) / 8;  // eight warps per CTA, 1024 values per warp and trip
  if (ctas > per_wave) ctas = per_wave;
  if (dtype == 1)
    dequant4_warp_kernel<__nv_bfloat16><<<(int)ctas, 256, 0, stream>>>((const uint8_t*)packed, absmax,
                                                                       (const uint8_t*)absmax_q, code256, absmax2,
                                                                       offset, code16, blocksize, block_shift, n,
                                                                       (__nv_bfloat16*)out);
  else
    dequant4_warp_kernel<__half><<<(int)ctas, 256, 0, stream>>>((const uint8_t*)packed, absmax,
                                                                (const uint8_t*)absmax_q, code256, absmax2, offset,
                                                                code16, blocksize, block_shift, n, (__half*)out);
  return (int)cudaGetLastError();
}

extern "C" int fmsb_gptq_dequant(const int* qweight, const void* scales, const int* qzeros, const int* g_idx,
                                 int in_features, int out_features, int bits, int group_size, int zero_offset,
                                 void* out, long long ldo, int dtype, cudaStream_t stream) {
  if (!(bits == 2 || bits == 4 || bits == 8)) return -2;
  if (out_features % (32 / bits) != 0 || in_features % (32 / bits) != 0) return -2;
  const long long total = (long long)in_features * out_features;
  if (total <= 0) return 0;
  // (v - z) * s in the vector kernel equals s * (v - z) of the scalar one: one fp32 product of the same operands
  if (ldo < out_features) return -2;
  const bool aligned = ((uintptr_t)qweight % 16 == 0) && ((uintptr_t)scales % 16 == 0) && ((uintptr_t)out % 16 == 0) &&
                       (ldo % 8 == 0);
  if (out_features % 8 == 0 && aligned && (dtype == 0 || dtype == 1)) {
    if (dtype == 1)
      return gptq_launch_vec<__nv_bfloat16>(qweight, (const __nv_bfloat16*)scales, qzeros, g_idx, in_features,
                                            out_features, bits, group_size, zero_offset, (__nv_bfloat16*)out, ldo, stream);
    return gptq_launch_vec<__half>(qweight, (const __half*)scales, qzeros, g_idx, in_features, out_features, bits,
                                   group_size, zero_offset, (__half*)out, ldo, stream);
  }
  long long ctas = (total + 255) / 256;
  if (ctas > 148 * 32) ctas = 148 * 32;
  if (dtype == 1)
    gptq_dequant_kernel<__nv_bfloat16><<<(int)ctas, 256, 0, stream>>>(qweight, (const __nv_bfloat16*)scales, qzeros,
                                                                      g_idx, in_features, out_features, bits,
                                                                      group_size, zero_offset, (__nv_bfloat16*)out, ldo);
  else if (dtype == 0)
    gptq_dequant_kernel<__half><<<(int)ctas, 256, 0, stream>>>(qweight, (const __half*)scales, qzeros, g_idx,
                                                               in_features, out_features, bits, group_size,
                                                               zero_offset, (__half*)out, ldo);
  else
    return -2;
  return (int)cudaGetLastError();
}
