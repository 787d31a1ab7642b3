// FP8 (E4M3) weight preparation: per-row quantisation of BF16 matrices and the matching
// dequantisation.  Run once when the model is loaded, not on the decode path.  No
// counterpart in the reference (its quantisation entry points are absent,
// csrc/quantization_kernels.cu:7-13).
#include <cuda_fp8.h>

#include "common.cuh"

namespace b200moe {

constexpr int kQuantThreads = 256;
constexpr float kE4m3Max = 448.0f;

__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) {
  return __uint_as_float(bits16 << 16);
}

// One block per row: max |w| over the row, scale = max / 448, then every element is
// divided by the scale (IEEE division, so a host restatement reproduces it bit for bit)
// and rounded to E4M3, nearest-even, saturating.
__global__ void __launch_bounds__(kQuantThreads)
fp8_quantize_rows_kernel(const uint4* __restrict__ w, uint4* __restrict__ q,
                         float* __restrict__ scale_out, int cols) {
  __shared__ float s_max[kQuantThreads / 32];
  __shared__ float s_scale;
  const size_t row = blockIdx.x;
  const int vecs = cols / 8;  // 8 BF16 per 16-byte load
  const uint4* src = w + row * vecs;

  float amax = 0.0f;
  for (int v = threadIdx.x; v < vecs; v += kQuantThreads) {
    const uint4 x = __ldg(src + v);
    const uint32_t words[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      amax = fmaxf(amax, fabsf(bf16_bits_to_float(words[i] & 0xFFFFu)));
      amax = fmaxf(amax, fabsf(bf16_bits_to_float(words[i] >> 16)));
    }
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
  if ((threadIdx.x & 31) == 0) s_max[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = 0.0f;
    for (int i = 0; i < kQuantThreads / 32; ++i) m = fmaxf(m, s_max[i]);
    const float scale = m > 0.0f ? __fdiv_rn(m, kE4m3Max) : 1.0f;
    s_scale = scale;
    scale_out[row] = scale;
  }
  __syncthreads();
  const float scale = s_scale;

  // 16 elements (two 16-byte loads) -> 16 bytes
  uint4* dst = q + row * (cols / 16);
  for (int v = threadIdx.x; v < cols / 16; v += kQuantThreads) {
    uint32_t out[4];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const uint4 x = __ldg(src + 2 * v + half);
      const uint32_t words[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
      for (int pair = 0; pair < 2; ++pair) {
        uint32_t packed = 0;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const uint32_t word = words[2 * pair + i];
          const float lo = __fdiv_rn(bf16_bits_to_float(word & 0xFFFFu), scale);
          const float hi = __fdiv_rn(bf16_bits_to_float(word >> 16), scale);
          const uint32_t b0 = __nv_cvt_float_to_fp8(lo, __NV_SATFINITE, __NV_E4M3);
          const uint32_t b1 = __nv_cvt_float_to_fp8(hi, __NV_SATFINITE, __NV_E4M3);
          packed |= (b0 | (b1 << 8)) << (16 * i);
        }
        out[2 * half + pair] = packed;
      }
    }
    dst[v] = make_uint4(out[0], out[1], out[2], out[3]);
  }
}

// Dequantisation for inspection and tests (the GEMM kernels feed the E4M3 bytes to the tensor
// core as they are): byte -> BF16 of the same value by a bit placement and one packed multiply
// (e4m3x4_to_bf16x4), exact for every byte value, then the row scale in FP32.
__device__ __forceinline__ uint32_t scale_pair(uint32_t pair, float scale) {
  const float lo = bf16_bits_to_float(pair & 0xFFFFu) * scale;
  const float hi = bf16_bits_to_float(pair >> 16) * scale;
  const __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&r);
}

__global__ void __launch_bounds__(kQuantThreads)
fp8_dequantize_rows_kernel(const uint4* __restrict__ q, const float* __restrict__ scale,
                           uint4* __restrict__ out, int cols) {
  const size_t row = blockIdx.x;
  const float s = scale ? scale[row] : 1.0f;
  const uint4* src = q + row * (cols / 16);
  uint4* dst = out + row * (cols / 8);
  for (int v = threadIdx.x; v < cols / 16; v += kQuantThreads) {
    const uint4 x = __ldg(src + v);
    const uint32_t words[4] = {x.x, x.y, x.z, x.w};
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) e4m3x4_to_bf16x4(words[i], o[2 * i], o[2 * i + 1]);
    if (scale) {
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = scale_pair(o[i], s);
    }
    dst[2 * v] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[2 * v + 1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

cudaError_t launch_fp8_quantize_rows(const void* w, long long rows, int cols, uint8_t* q,
                                     float* scale, cudaStream_t stream) {
  fp8_quantize_rows_kernel<<<(unsigned)rows, kQuantThreads, 0, stream>>>(
      static_cast<const uint4*>(w), reinterpret_cast<uint4*>(q), scale, cols);
  return cudaGetLastError();
}

cudaError_t launch_fp8_dequantize_rows(const uint8_t* q, const float* scale, long long rows,
                                       int cols, void* out, cudaStream_t stream) {
  fp8_dequantize_rows_kernel<<<(unsigned)rows, kQuantThreads, 0, stream>>>(
      reinterpret_cast<const uint4*>(q), scale, static_cast<uint4*>(out), cols);
  return cudaGetLastError();
}

}  // namespace b200moe
