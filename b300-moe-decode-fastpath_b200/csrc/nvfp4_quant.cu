// NVFP4 data preparation: expert weights -> packed E2M1 + block scales (once, at load time),
// and token rows -> E2M1 planes with fixed scales (every forward).
//
// No counterpart in the reference, whose NVFP4 backend is a stub that always fails
// (csrc/quantization_kernels.cu:7-13) and names what a real one needs (:3-6): a 4-bit E2M1
// payload and two levels of scales.  The format is the published one:
//   value = tensor_scale (FP32, one per expert matrix)
//         * block_scale  (unsigned E4M3, one per 16 consecutive elements along K)
//         * element      (E2M1: 0, 0.5, 1, 1.5, 2, 3, 4, 6 and their negatives),
// two elements per byte, the even one in the low nibble.
//
// Block scales are stored in the order the tensor core's scale-factor copy consumes
// (tcgen05.cp 32x128b.warpx4): tiles of 128 rows x 4 scales (64 elements of K), 512 bytes
// each, byte (r % 32) * 16 + (r / 32) * 4 + k for row r and scale k of the tile, so one
// plain bulk copy brings a pipeline stage's scales into shared memory ready for the copy.
//
// The block-scaled MMA needs E2M1 on both sides, so the token rows are held as four E2M1
// planes in fixed point: with a power-of-two row scale t that puts max |row| / t into
// [2, 4), plane p rounds what planes 0..p-1 left over, divided by t * 8^-p, to E2M1:
//   x ~= t * (e0 + e1 / 8 + e2 / 64 + e3 / 512),   |x - that| <= t * 2^-10 <= max |row| * 2^-11.
// Every residual is at most 4 in its plane's unit, where the E2M1 grid is at most 1 apart,
// so each plane removes three bits; all of it is exact FP32 arithmetic.  The scale of a plane
// is the same for every block of every row, so the scale factors of the token operand are
// constants that the GEMM kernels put into tensor memory once (they are never stored).
#include <cuda_fp8.h>

#include "common.cuh"

namespace b200moe {

constexpr int kNvfp4Block = 16;
constexpr int kNvfp4RowThreads = 128;   // token-row kernels: one thread per 8 elements of a chunk

__device__ __forceinline__ float e4m3_value(uint32_t code) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)code, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

// E2M1 code of x: round to nearest, ties to the even mantissa bit, saturating at 6.
__device__ __forceinline__ uint32_t e2m1_code(float x) {
  const float m = fabsf(x);
  const uint32_t idx = (uint32_t)(m > 0.25f) + (uint32_t)(m >= 0.75f) + (uint32_t)(m > 1.25f) +
                       (uint32_t)(m >= 1.75f) + (uint32_t)(m > 2.5f) + (uint32_t)(m >= 3.5f) +
                       (uint32_t)(m > 5.0f);
  return idx | ((__float_as_uint(x) >> 28) & 8u);
}
__device__ __forceinline__ float e2m1_value(uint32_t code) {
  // magnitudes 0, 0.5, 1, 1.5, 2, 3, 4, 6: from index 2 on, 2^(i / 2 - 1) * (1 + (i & 1) / 2),
  // written straight into the exponent and the top mantissa bit
  const uint32_t i = code & 7u;
  const uint32_t bits = i < 2u ? (i ? 0x3F000000u : 0u) : (((126u + (i >> 1)) << 23) | ((i & 1u) << 22));
  return __uint_as_float(bits | ((code & 8u) << 28));
}

// Byte offset of scale `sf_index` (= k / 16) of row `r` inside one matrix's swizzled scale
// array with `k_tiles` = ceil(K / 64) tiles per row tile.
__device__ __forceinline__ size_t swizzled_sf_offset(int r, int sf_index, int k_tiles) {
  const int row_tile = r >> 7, rr = r & 127, k_tile = sf_index >> 2, k = sf_index & 3;
  return ((size_t)row_tile * k_tiles + k_tile) * 512 + (size_t)(rr & 31) * 16 + (rr >> 5) * 4 + k;
}

// ---- weights ---------------------------------------------------------------------------
// max |w| of every expert matrix (bit pattern; non-negative floats order like their bits)
__global__ void __launch_bounds__(256)
nvfp4_amax_kernel(const __nv_bfloat16* __restrict__ w, long long per_expert, uint32_t* amax) {
  const int expert = blockIdx.y;
  const uint4* src = reinterpret_cast<const uint4*>(w + (size_t)expert * per_expert);
  const long long vecs = per_expert / 8;
  float m = 0.0f;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < vecs;
       v += (long long)gridDim.x * blockDim.x) {
    const uint4 x = __ldg(src + v);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  m = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(m)));
  if ((threadIdx.x & 31) == 0 && m > 0.0f) atomicMax(amax + expert, __float_as_uint(m));
}

// One thread per block of 16 elements.  `halves` = 2 for the gate+up matrix, whose gate and
// up halves ([rows] each) have separate scale tilings so that a 128-row tile of either
// starts a scale tile; 1 otherwise.
__global__ void __launch_bounds__(256)
nvfp4_quantize_kernel(const __nv_bfloat16* __restrict__ w, const uint32_t* __restrict__ amax,
                      int rows, int cols, int halves, uint8_t* __restrict__ packed,
                      uint8_t* __restrict__ sf, float* __restrict__ tensor_scale) {
  const int expert = blockIdx.y;
  const int blocks_per_row = cols / kNvfp4Block;
  const long long total = (long long)halves * rows * blocks_per_row;
  const float top = __uint_as_float(amax[expert]);
  const float g = top > 0.0f ? __fdiv_rn(top, 2688.0f) : 1.0f;  // 6 * 448
  if (blockIdx.x == 0 && threadIdx.x == 0) tensor_scale[expert] = g;
  const int k_tiles = (cols + 63) / 64;
  const size_t sf_per_half = (size_t)((rows + 127) / 128) * k_tiles * 512;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int b = (int)(i % blocks_per_row);
    const long long row_all = i / blocks_per_row;             // row inside [halves * rows]
    const int half = (int)(row_all / rows), r = (int)(row_all % rows);
    const __nv_bfloat16* src = w + ((size_t)expert * halves * rows + row_all) * cols + (size_t)b * 16;
    float v[16];
    const uint4 x0 = __ldg(reinterpret_cast<const uint4*>(src));
    const uint4 x1 = __ldg(reinterpret_cast<const uint4*>(src) + 1);
    const __nv_bfloat162* h0 = reinterpret_cast<const __nv_bfloat162*>(&x0);
    const __nv_bfloat162* h1 = reinterpret_cast<const __nv_bfloat162*>(&x1);
    float block_max = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = __bfloat1622float2(h0[j]), c = __bfloat1622float2(h1[j]);
      v[2 * j] = a.x; v[2 * j + 1] = a.y; v[8 + 2 * j] = c.x; v[8 + 2 * j + 1] = c.y;
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) block_max = fmaxf(block_max, fabsf(v[j]));
    const float target = __fdiv_rn(__fdiv_rn(block_max, 6.0f), g);
    const uint32_t code = __nv_cvt_float_to_fp8(target, __NV_SATFINITE, __NV_E4M3);
    const float denom = __fmul_rn(g, e4m3_value(code));
    uint32_t lo = 0u, hi = 0u;
    if (denom > 0.0f) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        lo |= e2m1_code(__fdiv_rn(v[j], denom)) << (4 * j);
        hi |= e2m1_code(__fdiv_rn(v[8 + j], denom)) << (4 * j);
      }
    }
    const size_t out_row = (size_t)expert * halves * rows + row_all;
    *reinterpret_cast<uint2*>(packed + out_row * (cols / 2) + (size_t)b * 8) = make_uint2(lo, hi);
    sf[((size_t)expert * halves + half) * sf_per_half + swizzled_sf_offset(r, b, k_tiles)] =
        (uint8_t)code;
  }
}

// ---- token rows ------------------------------------------------------------------------
// Block-wide maximum of a non-negative float; every thread gets the result.
__device__ __forceinline__ float nv_block_max(float v, float* tmp) {
  v = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(v)));
  if ((threadIdx.x & 31) == 0) tmp[threadIdx.x >> 5] = v;
  __syncthreads();
  float m = 0.0f;
  for (int i = 0; i < kNvfp4RowThreads / 32; ++i) m = fmaxf(m, tmp[i]);
  __syncthreads();
  return m;
}

// power of two t with max|row| / t in [2, 4); 1 for an all-zero row (and never below 2^-100,
// so that t / 8 and t * 8^-3 stay normal numbers)
__device__ __forceinline__ float row_scale_pow2(float amax) {
  if (!(amax > 0.0f)) return 1.0f;
  int e;
  frexpf(amax, &e);
  return ldexpf(1.0f, max(e - 2, -100));
}

// 8 values -> kNvfp4Planes planes of 4 packed bytes each.
__device__ __forceinline__ void octet_to_planes(float (&res)[8], float t, uint8_t* planes,
                                                size_t plane_stride, size_t data_offset) {
  float step = t;
#pragma unroll
  for (int p = 0; p < kNvfp4Planes; ++p) {
    // round(residual / step) to E2M1 without dividing: step is a power of two, so the seven
    // midpoints times step are exact and the comparisons decide exactly
    const float m025 = 0.25f * step, m075 = 0.75f * step, m125 = 1.25f * step,
                m175 = 1.75f * step, m250 = 2.5f * step, m350 = 3.5f * step, m500 = 5.0f * step;
    uint32_t word = 0u;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float m = fabsf(res[j]);
      const uint32_t idx = (uint32_t)(m > m025) + (uint32_t)(m >= m075) + (uint32_t)(m > m125) +
                           (uint32_t)(m >= m175) + (uint32_t)(m > m250) + (uint32_t)(m >= m350) +
                           (uint32_t)(m > m500);
      const uint32_t q = idx | ((__float_as_uint(res[j]) >> 28) & 8u);
      word |= q << (4 * j);
      res[j] = __fsub_rn(res[j], __fmul_rn(e2m1_value(q), step));
    }
    *reinterpret_cast<uint32_t*>(planes + p * plane_stride + data_offset) = word;
    step *= 0.125f;
  }
}

__device__ __forceinline__ void bf16x8_to_float(const uint4& x, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 v = __bfloat1622float2(h[j]);
    f[2 * j] = v.x;
    f[2 * j + 1] = v.y;
  }
}

// Gather for the NVFP4 path: permuted_hidden[p, :] = hidden[permutation[p] / K, :] as in
// gather_rows_kernel, plus the row's planes and row scale in scratch.  One block per (row,
// chunk of 1024 columns): every block reads the whole row for its maximum (8 KB, from L2
// after the first) and converts its own chunk, one thread per 8 columns.
__global__ void __launch_bounds__(kNvfp4RowThreads)
gather_rows_nvfp4_kernel(const uint4* __restrict__ hidden, const int64_t* __restrict__ permutation,
                         uint4* __restrict__ out, uint8_t* __restrict__ planes,
                         float* __restrict__ row_scale, int num_assign, int num_tokens,
                         int top_k, int hidden_size, int rows_cap,
                         unsigned long long* __restrict__ trace) {
  __shared__ float s_tmp[kNvfp4RowThreads / 32];
  pdl_wait();
  pdl_launch_dependents();
  trace_start(trace, kTraceGather);
  const int row = blockIdx.x;
  const int vec_per_row = hidden_size / 8;
  const int own = blockIdx.y * kNvfp4RowThreads + threadIdx.x;
  const int64_t a = permutation[row];
  const bool valid = a >= 0 && a < (int64_t)num_assign && (a / top_k) < (int64_t)num_tokens;
  const uint4* src = hidden + (valid ? (size_t)(a / top_k) * vec_per_row : 0);
  float amax = 0.0f;
  uint4 mine = make_uint4(0u, 0u, 0u, 0u);
  for (int v = threadIdx.x; v < vec_per_row; v += kNvfp4RowThreads) {
    // this block's chunk comes round in turn blockIdx.y of this loop
    uint4 x = make_uint4(0u, 0u, 0u, 0u);
    if (valid) x = __ldg(src + v);
    if (v == own) mine = x;
    float f[8];
    bf16x8_to_float(x, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
  }
  amax = nv_block_max(amax, s_tmp);
  const float t = row_scale_pow2(amax);
  if (threadIdx.x == 0 && blockIdx.y == 0) row_scale[row] = t;
  if (own < vec_per_row) {
    out[(size_t)row * vec_per_row + own] = mine;
    float res[8];
    bf16x8_to_float(mine, res);
    octet_to_planes(res, t, planes, (size_t)rows_cap * (hidden_size / 2),
                    (size_t)row * (hidden_size / 2) + (size_t)own * 4);
  }
  trace_end(trace, kTraceGather);
}

// Between the two NVFP4 GEMMs: activation rows (hi + lo BF16 halves) -> planes and a row
// scale, in the bytes the gathered rows' planes occupied.  The gate+up epilogue left the
// maximum |activation| of every (row, 128-column tile); the row scale only needs their
// maximum, so the chunks of a row are independent: one block per (row, 1024 columns), one
// thread per 8 columns.
__global__ void __launch_bounds__(kNvfp4RowThreads)
act_planes_nvfp4_kernel(const uint4* __restrict__ act_hi, const uint4* __restrict__ act_lo,
                        const float* __restrict__ tile_amax, uint8_t* __restrict__ planes,
                        float* __restrict__ row_scale, int inter, int rows_cap) {
  __shared__ float s_tmp[kNvfp4RowThreads / 32];
  // the down grid may become resident and prefetch weight tiles now; it waits for this
  // grid's completion before it touches the planes
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const int vec_per_row = inter / 8;
  const int own = blockIdx.y * kNvfp4RowThreads + threadIdx.x;
  // the activations are requested before the maximum is known
  uint4 xh = make_uint4(0u, 0u, 0u, 0u), xl = xh;
  if (own < vec_per_row) {
    xh = act_hi[(size_t)row * vec_per_row + own];
    xl = act_lo[(size_t)row * vec_per_row + own];
  }
  const int tiles = (inter + 127) / 128;
  float amax = 0.0f;
  for (int i = threadIdx.x; i < tiles; i += kNvfp4RowThreads)
    amax = fmaxf(amax, tile_amax[(size_t)row * tiles + i]);
  amax = nv_block_max(amax, s_tmp);
  const float t = row_scale_pow2(amax);
  if (threadIdx.x == 0 && blockIdx.y == 0) row_scale[row] = t;
  if (own >= vec_per_row) return;
  float hi[8], lo[8], res[8];
  bf16x8_to_float(xh, hi);
  bf16x8_to_float(xl, lo);
#pragma unroll
  for (int j = 0; j < 8; ++j) res[j] = __fadd_rn(hi[j], lo[j]);
  octet_to_planes(res, t, planes, (size_t)rows_cap * (inter / 2),
                  (size_t)row * (inter / 2) + (size_t)own * 4);
}

// Standalone row -> planes conversion of FP32 rows (tests of the plane rule).
__global__ void __launch_bounds__(kNvfp4RowThreads)
rows_to_planes_nvfp4_kernel(const float* __restrict__ rows, uint8_t* __restrict__ planes,
                            float* __restrict__ row_scale, int cols, int rows_cap) {
  __shared__ float s_tmp[kNvfp4RowThreads / 32];
  const int row = blockIdx.x;
  const float* src = rows + (size_t)row * cols;
  float amax = 0.0f;
  for (int c = threadIdx.x; c < cols; c += kNvfp4RowThreads) amax = fmaxf(amax, fabsf(src[c]));
  amax = nv_block_max(amax, s_tmp);
  const float t = row_scale_pow2(amax);
  if (threadIdx.x == 0 && blockIdx.y == 0) row_scale[row] = t;
  const int own = blockIdx.y * kNvfp4RowThreads + threadIdx.x;
  if (own >= cols / 8) return;
  float res[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) res[j] = src[own * 8 + j];
  octet_to_planes(res, t, planes, (size_t)rows_cap * (cols / 2),
                  (size_t)row * (cols / 2) + (size_t)own * 4);
}

// ---- launchers -------------------------------------------------------------------------
cudaError_t launch_nvfp4_quantize(const void* w, int experts, int rows, int cols, int halves,
                                  uint8_t* packed, uint8_t* sf, float* tensor_scale,
                                  uint32_t* amax_scratch, cudaStream_t stream) {
  cudaError_t err = cudaMemsetAsync(amax_scratch, 0, sizeof(uint32_t) * experts, stream);
  if (err != cudaSuccess) return err;
  const long long per_expert = (long long)halves * rows * cols;
  const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(w);
  nvfp4_amax_kernel<<<dim3(296, experts), 256, 0, stream>>>(src, per_expert, amax_scratch);
  nvfp4_quantize_kernel<<<dim3(592, experts), 256, 0, stream>>>(src, amax_scratch, rows, cols,
                                                               halves, packed, sf, tensor_scale);
  return cudaGetLastError();
}

static cudaError_t launch_rows_pdl(const void* func, int rows, int chunks, void** args, bool pdl,
                                   cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(rows, chunks);
  cfg.blockDim = dim3(kNvfp4RowThreads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelExC(&cfg, func, args);
}

cudaError_t launch_gather_nvfp4(const void* hidden, const int64_t* permutation, void* out,
                                uint8_t* planes, float* row_scale, int num_assign,
                                int num_tokens, int top_k, int hidden_size, int rows_cap,
                                unsigned long long* trace, bool pdl, cudaStream_t stream) {
  const uint4* h = static_cast<const uint4*>(hidden);
  uint4* o = static_cast<uint4*>(out);
  void* args[] = {&h, &permutation, &o, &planes, &row_scale, &num_assign,
                  &num_tokens, &top_k, &hidden_size, &rows_cap, &trace};
  const int chunks = (hidden_size / 8 + kNvfp4RowThreads - 1) / kNvfp4RowThreads;
  return launch_rows_pdl(reinterpret_cast<const void*>(&gather_rows_nvfp4_kernel), num_assign,
                         chunks, args, pdl, stream);
}

cudaError_t launch_act_planes_nvfp4(const void* act_hi, const void* act_lo,
                                    const float* tile_amax, uint8_t* planes, float* row_scale,
                                    int num_assign, int inter, int rows_cap, bool pdl,
                                    cudaStream_t stream) {
  const uint4* hi = static_cast<const uint4*>(act_hi);
  const uint4* lo = static_cast<const uint4*>(act_lo);
  void* args[] = {&hi, &lo, &tile_amax, &planes, &row_scale, &inter, &rows_cap};
  const int chunks = (inter / 8 + kNvfp4RowThreads - 1) / kNvfp4RowThreads;
  return launch_rows_pdl(reinterpret_cast<const void*>(&act_planes_nvfp4_kernel), num_assign,
                         chunks, args, pdl, stream);
}

cudaError_t launch_rows_to_planes_nvfp4(const float* rows, int num_rows, int cols,
                                        uint8_t* planes, float* row_scale,
                                        cudaStream_t stream) {
  const int chunks = (cols / 8 + kNvfp4RowThreads - 1) / kNvfp4RowThreads;
  rows_to_planes_nvfp4_kernel<<<dim3(num_rows, chunks), kNvfp4RowThreads, 0, stream>>>(
      rows, planes, row_scale, cols, num_rows);
  return cudaGetLastError();
}

}  // namespace b200moe
