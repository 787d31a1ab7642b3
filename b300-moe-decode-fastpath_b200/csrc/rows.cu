// Stage 2 (gather) and stage 5 (combine): the two row-moving kernels either
// side of the grouped GEMMs.  Both are pure HBM traffic and use 16-byte
// accesses throughout.
#include <cuda_fp8.h>

#include "common.cuh"

namespace b200moe {

constexpr int kRowThreads = 256;

// permuted_hidden[p, :] = hidden[permutation[p] / K, :]
// Same contract as the reference gather (csrc/permutation_kernels.cu:25-50): a
// row whose mapping is outside [0, A) is zero-filled.
__global__ void __launch_bounds__(kRowThreads)
gather_rows_kernel(const uint4* __restrict__ hidden, const int64_t* __restrict__ permutation,
                   uint4* __restrict__ out, int num_assign, int num_tokens, int top_k,
                   int vec_per_row, unsigned long long* __restrict__ trace) {
  // The gate+up grid may start once every block here has passed its wait, that is, once
  // the routing kernel has completed: it reads the schedule as soon as it starts.
  pdl_wait();
  pdl_launch_dependents();
  trace_start(trace, kTraceGather);
  const int row = blockIdx.x;
  const int64_t a = permutation[row];
  const bool valid = a >= 0 && a < (int64_t)num_assign && (a / top_k) < (int64_t)num_tokens;
  const uint4* src = hidden + (valid ? (size_t)(a / top_k) * vec_per_row : 0);
  uint4* dst = out + (size_t)row * vec_per_row;
  for (int v = threadIdx.x; v < vec_per_row; v += kRowThreads) {
    uint4 x = make_uint4(0u, 0u, 0u, 0u);
    if (valid) x = __ldg(src + v);
    dst[v] = x;
  }
  trace_end(trace, kTraceGather);
}

__device__ __forceinline__ uint4 pack_bf16x8(const float (&f)[8]) {
  uint4 p;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&p);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return p;
}

// out[t, :] = bf16( sum_k float(w[t,k]) * row(reverse_mapping[t*K+k]) ), where
// row(p) = sum over the split-K slices of the down projection, slice 0 first.
// FP32 accumulation in slot order; weights used as supplied; rows whose
// mapping is invalid are skipped (csrc/combine_kernels.cu:39-47).  One thread
// owns eight consecutive hidden columns.
__global__ void __launch_bounds__(128)
combine_rows_kernel(const int64_t* __restrict__ reverse_mapping,
                    const __nv_bfloat16* __restrict__ weights, const float* __restrict__ partials,
                    const int32_t* __restrict__ sched, uint4* __restrict__ out,
                    uint4* __restrict__ expert_out, int num_assign, int top_k, int hidden,
                    size_t slice_elems, int f32_out, unsigned long long* __restrict__ trace) {
  pdl_wait();
  pdl_launch_dependents();
  trace_start(trace, kTraceCombine);
  const int token = blockIdx.x;
  const int col = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (col >= hidden) return;
  const int splits = sched[kSchedDownSplits];

  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;

  // Slot metadata first (independent loads), then per slot all split-K slices at once:
  // the loads of one slot are issued back to back and only the additions are ordered.
  int64_t rows[8];
  float wts[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    rows[k] = -1;
    wts[k] = 0.0f;
    if (k < top_k) {
      rows[k] = reverse_mapping[token * top_k + k];
      wts[k] = __bfloat162float(weights[token * top_k + k]);
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    if (k >= top_k) break;
    const int64_t row = rows[k];
    if (row < 0 || row >= (int64_t)num_assign) continue;
    const float w = wts[k];
    const float* src = partials + (size_t)row * hidden + col;
    float4 lo[kDownSplitMax], hi[kDownSplitMax];
#pragma unroll
    for (int s = 0; s < kDownSplitMax; ++s) {
      if (s < splits) {
        lo[s] = *reinterpret_cast<const float4*>(src + (size_t)s * slice_elems);
        hi[s] = *reinterpret_cast<const float4*>(src + (size_t)s * slice_elems + 4);
      }
    }
    float v[8] = {lo[0].x, lo[0].y, lo[0].z, lo[0].w, hi[0].x, hi[0].y, hi[0].z, hi[0].w};
#pragma unroll
    for (int s = 1; s < kDownSplitMax; ++s) {
      if (s < splits) {
        v[0] += lo[s].x; v[1] += lo[s].y; v[2] += lo[s].z; v[3] += lo[s].w;
        v[4] += hi[s].x; v[5] += hi[s].y; v[6] += hi[s].z; v[7] += hi[s].w;
      }
    }
    if (expert_out) expert_out[((size_t)row * hidden + col) >> 3] = pack_bf16x8(v);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = fmaf(v[i], w, acc[i]);
  }
  if (f32_out) {
    // unrounded sums, for callers that add partial outputs of several ranks
    float4* o = reinterpret_cast<float4*>(reinterpret_cast<float*>(out) +
                                          (size_t)token * hidden + col);
    o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
  } else {
    out[((size_t)token * hidden + col) >> 3] = pack_bf16x8(acc);
  }
  trace_end(trace, kTraceCombine);
}

// The same combine for calls of few assignments, where its latency and not its bytes count:
// kGroup (a power of two >= top_k) consecutive lanes share eight consecutive hidden columns
// of one token.  Lane k of the group fetches slot k (its routing weight, its row's split-K
// slices, all in flight at once), sums the slices and stores the BF16 expert row; the
// group's first lane then collects the sums with shuffles and adds them in slot order.  The
// arithmetic is exactly the one of combine_rows_kernel, but the slots' trips to L2 overlap
// instead of following one another (top_k = 8, one token: 5.4 -> 2.1 us).  With many tokens
// the extra lanes and shuffles cost more than the latency they hide (top_k = 2, 64 tokens:
// 2.9 -> 6.2 us), so the host uses it for T * top_k <= kSlotCombineMaxAssign only.
constexpr int kSlotCombineMaxAssign = 64;

template <int kGroup>
__global__ void __launch_bounds__(128)
combine_rows_slots_kernel(const int64_t* __restrict__ reverse_mapping,
                    const __nv_bfloat16* __restrict__ weights, const float* __restrict__ partials,
                    const int32_t* __restrict__ sched, uint4* __restrict__ out,
                    uint4* __restrict__ expert_out, int num_assign, int top_k, int hidden,
                    size_t slice_elems, int f32_out, unsigned long long* __restrict__ trace) {
  pdl_wait();
  pdl_launch_dependents();
  trace_start(trace, kTraceCombine);
  const int token = blockIdx.x;
  const int k = threadIdx.x & (kGroup - 1);                              // this lane's slot
  const int col = (int)((blockIdx.y * blockDim.x + threadIdx.x) / kGroup) * 8;   // the group's columns
  const bool in_range = col < hidden;
  const int splits = sched[kSchedDownSplits];

  int64_t row = -1;
  float w = 0.0f;
  if (in_range && k < top_k) {
    row = reverse_mapping[token * top_k + k];
    w = __bfloat162float(weights[token * top_k + k]);
  }
  const bool ok = row >= 0 && row < (int64_t)num_assign;
  float v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = 0.0f;
  if (ok) {
    const float* src = partials + (size_t)row * hidden + col;
    float4 lo[kDownSplitMax], hi[kDownSplitMax];
#pragma unroll
    for (int s = 0; s < kDownSplitMax; ++s) {
      if (s < splits) {
        lo[s] = *reinterpret_cast<const float4*>(src + (size_t)s * slice_elems);
        hi[s] = *reinterpret_cast<const float4*>(src + (size_t)s * slice_elems + 4);
      }
    }
    v[0] = lo[0].x; v[1] = lo[0].y; v[2] = lo[0].z; v[3] = lo[0].w;
    v[4] = hi[0].x; v[5] = hi[0].y; v[6] = hi[0].z; v[7] = hi[0].w;
#pragma unroll
    for (int s = 1; s < kDownSplitMax; ++s) {
      if (s < splits) {
        v[0] += lo[s].x; v[1] += lo[s].y; v[2] += lo[s].z; v[3] += lo[s].w;
        v[4] += hi[s].x; v[5] += hi[s].y; v[6] += hi[s].z; v[7] += hi[s].w;
      }
    }
    if (expert_out) expert_out[((size_t)row * hidden + col) >> 3] = pack_bf16x8(v);
  }

  // the group's first lane adds the slots in order
  const unsigned full = 0xffffffffu;
  const int leader = (int)(threadIdx.x & 31) & ~(kGroup - 1);
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
#pragma unroll
  for (int kk = 0; kk < kGroup; ++kk) {
    const float wk = __shfl_sync(full, w, leader + kk);
    const int okk = __shfl_sync(full, (int)ok, leader + kk);
    float vk[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) vk[i] = __shfl_sync(full, v[i], leader + kk);
    if (okk) {
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = fmaf(vk[i], wk, acc[i]);
    }
  }
  if (k == 0 && in_range) {
    if (f32_out) {
      // unrounded sums, for callers that add partial outputs of several ranks
      float4* o = reinterpret_cast<float4*>(reinterpret_cast<float*>(out) +
                                            (size_t)token * hidden + col);
      o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    } else {
      out[((size_t)token * hidden + col) >> 3] = pack_bf16x8(acc);
    }
  }
  trace_end(trace, kTraceCombine);
}

// Legacy combine: out[t, :] = bf16( sum_k float(w[t,k]) * float(rows[map[t*K+k], :]) ) on BF16
// expert rows, FP32 accumulation in slot order, rows with an invalid mapping skipped
// (csrc/combine_cuda.cu:23-52).
__global__ void __launch_bounds__(128)
combine_bf16_rows_kernel(const uint4* __restrict__ expert_rows,
                         const int64_t* __restrict__ assignment_to_permuted,
                         const __nv_bfloat16* __restrict__ weights, uint4* __restrict__ out,
                         int num_assign, int top_k, int hidden) {
  const int token = blockIdx.x;
  const int col = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (col >= hidden) return;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
  for (int k = 0; k < top_k; ++k) {
    const int a = token * top_k + k;
    const int64_t row = assignment_to_permuted[a];
    if (row < 0 || row >= (int64_t)num_assign) continue;
    const float w = __bfloat162float(weights[a]);
    const uint4 packed = __ldg(expert_rows + (((size_t)row * hidden + col) >> 3));
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&packed);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 v = __bfloat1622float2(h[i]);
      acc[2 * i] = fmaf(v.x, w, acc[2 * i]);
      acc[2 * i + 1] = fmaf(v.y, w, acc[2 * i + 1]);
    }
  }
  out[((size_t)token * hidden + col) >> 3] = pack_bf16x8(acc);
}

// ---------------------------------------------------------------------------
// FP8-weight path: token rows as E4M3 planes plus a scale per row.
//
// r = x / s, then
//   p0 = e4m3(r), p1 = e4m3((r - p0) * 16), p2 = e4m3(((r - p0) * 16 - p1) * 16),
// every rounding to nearest-even, saturating; x ~= s * (p0 + p1/16 + p2/256).
// Hidden rows (BF16): s = the power of two that puts max|row| / s into [128, 256), two
// planes, exact.  Activation rows: s = max|row| / 448 (1 for an all-zero row), three planes.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float e4m3_to_float(uint32_t code) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)code, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

__device__ __forceinline__ void split_e4m3x3(float r, uint32_t& c0, uint32_t& c1, uint32_t& c2) {
  c0 = __nv_cvt_float_to_fp8(r, __NV_SATFINITE, __NV_E4M3);
  const float r1 = (r - e4m3_to_float(c0)) * 16.0f;
  c1 = __nv_cvt_float_to_fp8(r1, __NV_SATFINITE, __NV_E4M3);
  const float r2 = (r1 - e4m3_to_float(c1)) * 16.0f;
  c2 = __nv_cvt_float_to_fp8(r2, __NV_SATFINITE, __NV_E4M3);
}

// Block-wide maximum of a non-negative float; every thread gets the result.
__device__ __forceinline__ float block_max(float v, float* tmp) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, d));
  if ((threadIdx.x & 31) == 0) tmp[threadIdx.x >> 5] = v;
  __syncthreads();
  float m = 0.0f;
  for (int i = 0; i < kRowThreads / 32; ++i) m = fmaxf(m, tmp[i]);
  __syncthreads();
  return m;
}

// Eight consecutive values of one row -> eight bytes in each of the kPlanes planes.
template <int kPlanes>
__device__ __forceinline__ void store_planes8(const float (&r)[8], uint8_t* plane0,
                                              size_t plane_stride, size_t offset) {
  uint32_t lo[3] = {0u, 0u, 0u}, hi[3] = {0u, 0u, 0u};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    uint32_t c[3];
    split_e4m3x3(r[i], c[0], c[1], c[2]);
#pragma unroll
    for (int pl = 0; pl < kPlanes; ++pl) {
      if (i < 4) lo[pl] |= c[pl] << (8 * i);
      else hi[pl] |= c[pl] << (8 * (i - 4));
    }
  }
#pragma unroll
  for (int pl = 0; pl < kPlanes; ++pl)
    *reinterpret_cast<uint2*>(plane0 + pl * plane_stride + offset) = make_uint2(lo[pl], hi[pl]);
}

// Gather for the FP8-weight path: the BF16 row goes to permuted_hidden as in
// gather_rows_kernel, and its planes and scale go to scratch.  The row is BF16 (eight
// significant bits), so with a power-of-two scale -- the division is then exact -- two
// planes of four bits each hold it exactly (values below 2^-12 of the row maximum run into
// the second plane's subnormal step: their error stays under 2^-21 of that maximum).  Also clears the row's activation
// maximum, which the gate+up kernel accumulates next.
__global__ void __launch_bounds__(kRowThreads)
gather_rows_fp8_kernel(const uint4* __restrict__ hidden, const int64_t* __restrict__ permutation,
                       uint4* __restrict__ out, uint8_t* __restrict__ planes,
                       float* __restrict__ row_scale, uint32_t* __restrict__ act_amax,
                       int num_assign, int num_tokens, int top_k, int hidden_size, int rows_cap,
                       unsigned long long* __restrict__ trace) {
  __shared__ float s_tmp[kRowThreads / 32];
  pdl_wait();
  pdl_launch_dependents();
  trace_start(trace, kTraceGather);
  const int row = blockIdx.x;
  const int vec_per_row = hidden_size / 8;
  const int64_t a = permutation[row];
  const bool valid = a >= 0 && a < (int64_t)num_assign && (a / top_k) < (int64_t)num_tokens;
  const uint4* src = hidden + (valid ? (size_t)(a / top_k) * vec_per_row : 0);
  uint4* dst = out + (size_t)row * vec_per_row;
  float amax = 0.0f;
  for (int v = threadIdx.x; v < vec_per_row; v += kRowThreads) {
    uint4 x = make_uint4(0u, 0u, 0u, 0u);
    if (valid) x = __ldg(src + v);
    dst[v] = x;
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  amax = block_max(amax, s_tmp);
  // power of two with max|x| / scale in [128, 256): frexp gives amax = f * 2^e, f in [0.5, 1)
  float scale = 1.0f;
  if (amax > 0.0f) {
    int e;
    frexpf(amax, &e);
    scale = ldexpf(1.0f, e - 8);
  }
  if (threadIdx.x == 0) {
    row_scale[row] = scale;
    act_amax[row] = 0u;
  }
  const size_t plane_stride = (size_t)rows_cap * hidden_size;
  for (int v = threadIdx.x; v < vec_per_row; v += kRowThreads) {
    uint4 x = make_uint4(0u, 0u, 0u, 0u);
    if (valid) x = __ldg(src + v);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x);
    float r[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      r[2 * i] = __fdiv_rn(f.x, scale);
      r[2 * i + 1] = __fdiv_rn(f.y, scale);
    }
    store_planes8<kFp8PlanesHidden>(r, planes, plane_stride,
                                    (size_t)row * hidden_size + (size_t)v * 8);
  }
  trace_end(trace, kTraceGather);
}

// Between the two FP8 GEMMs: activation rows (hi + lo BF16 halves, maximum already known)
// -> three planes and a scale per row, into the bytes the gathered rows occupied.  One
// block per (row, chunk of 8 * kRowThreads columns): the row maximum is known, so chunks
// are independent.
__global__ void __launch_bounds__(kRowThreads)
act_planes_fp8_kernel(const uint4* __restrict__ act_hi, const uint4* __restrict__ act_lo,
                      const uint32_t* __restrict__ act_amax, uint8_t* __restrict__ planes,
                      float* __restrict__ row_scale, int inter, int rows_cap) {
  // Let the down grid become resident and prefetch its weight tiles now; it waits for this
  // grid's completion before it touches the planes, and the schedule it reads first has
  // been final since the routing kernel completed, several grids ago.
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const int vec_per_row = inter / 8;
  const float amax = __uint_as_float(act_amax[row]);
  const float scale = amax > 0.0f ? __fdiv_rn(amax, 448.0f) : 1.0f;
  if (threadIdx.x == 0 && blockIdx.y == 0) row_scale[row] = scale;
  const int v = blockIdx.y * kRowThreads + threadIdx.x;
  if (v >= vec_per_row) return;
  const size_t plane_stride = (size_t)rows_cap * inter;
  const uint4 xh = act_hi[(size_t)row * vec_per_row + v];
  const uint4 xl = act_lo[(size_t)row * vec_per_row + v];
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&xh);
  const __nv_bfloat162* l = reinterpret_cast<const __nv_bfloat162*>(&xl);
  float r[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 fh = __bfloat1622float2(h[i]), fl = __bfloat1622float2(l[i]);
    r[2 * i] = __fdiv_rn(fh.x + fl.x, scale);
    r[2 * i + 1] = __fdiv_rn(fh.y + fl.y, scale);
  }
  store_planes8<kFp8Planes>(r, planes, plane_stride, (size_t)row * inter + (size_t)v * 8);
}

cudaError_t launch_combine_bf16(const void* expert_rows, const int64_t* assignment_to_permuted,
                                const void* weights, void* out, int num_tokens, int top_k,
                                int hidden_size, cudaStream_t stream) {
  const dim3 grid(num_tokens, (hidden_size / 8 + 127) / 128);
  combine_bf16_rows_kernel<<<grid, 128, 0, stream>>>(
      static_cast<const uint4*>(expert_rows), assignment_to_permuted,
      static_cast<const __nv_bfloat16*>(weights), static_cast<uint4*>(out),
      num_tokens * top_k, top_k, hidden_size);
  return cudaGetLastError();
}

static cudaError_t launch_with_pdl(const void* func, dim3 grid, dim3 block, void** args,
                                   bool pdl, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelExC(&cfg, func, args);
}

cudaError_t launch_gather(const void* hidden, const int64_t* permutation, void* out,
                          int num_assign, int num_tokens, int top_k, int hidden_size,
                          unsigned long long* trace, bool pdl, cudaStream_t stream) {
  int vec_per_row = hidden_size / 8;
  const uint4* h = static_cast<const uint4*>(hidden);
  uint4* o = static_cast<uint4*>(out);
  void* args[] = {&h, &permutation, &o, &num_assign, &num_tokens, &top_k, &vec_per_row, &trace};
  return launch_with_pdl(reinterpret_cast<const void*>(&gather_rows_kernel), dim3(num_assign),
                         dim3(kRowThreads), args, pdl, stream);
}

cudaError_t launch_combine(const int64_t* reverse_mapping, const void* weights,
                           const float* partials, const int32_t* sched, void* out,
                           void* expert_out, int num_tokens, int top_k, int hidden_size,
                           size_t slice_elems, bool f32_out, unsigned long long* trace, bool pdl,
                           cudaStream_t stream) {
  int num_assign = num_tokens * top_k;
  const __nv_bfloat16* w = static_cast<const __nv_bfloat16*>(weights);
  uint4* o = static_cast<uint4*>(out);
  uint4* eo = static_cast<uint4*>(expert_out);
  int f32 = f32_out ? 1 : 0;
  void* args[] = {&reverse_mapping, &w, &partials, &sched, &o, &eo, &num_assign, &top_k,
                  &hidden_size, &slice_elems, &f32, &trace};
  const int vecs = hidden_size / 8;
  if (num_assign <= kSlotCombineMaxAssign && top_k > 1) {
    // few assignments: one lane per slot, so that the slots' loads overlap
    const int group = top_k <= 2 ? 2 : (top_k <= 4 ? 4 : 8);
    const void* kernel = group == 2 ? reinterpret_cast<const void*>(&combine_rows_slots_kernel<2>)
                         : group == 4 ? reinterpret_cast<const void*>(&combine_rows_slots_kernel<4>)
                                      : reinterpret_cast<const void*>(&combine_rows_slots_kernel<8>);
    dim3 grid(num_tokens, (vecs * group + 127) / 128);
    return launch_with_pdl(kernel, grid, dim3(128), args, pdl, stream);
  }
  dim3 grid(num_tokens, (vecs + 127) / 128);
  return launch_with_pdl(reinterpret_cast<const void*>(&combine_rows_kernel), grid, dim3(128),
                         args, pdl, stream);
}

cudaError_t launch_gather_fp8(const void* hidden, const int64_t* permutation, void* out,
                              uint8_t* planes, float* row_scale, uint32_t* act_amax,
                              int num_assign, int num_tokens, int top_k, int hidden_size,
                              int rows_cap, unsigned long long* trace, bool pdl,
                              cudaStream_t stream) {
  const uint4* h = static_cast<const uint4*>(hidden);
  uint4* o = static_cast<uint4*>(out);
  void* args[] = {&h, &permutation, &o, &planes, &row_scale, &act_amax, &num_assign, &num_tokens,
                  &top_k, &hidden_size, &rows_cap, &trace};
  return launch_with_pdl(reinterpret_cast<const void*>(&gather_rows_fp8_kernel),
                         dim3(num_assign), dim3(kRowThreads), args, pdl, stream);
}

cudaError_t launch_act_planes_fp8(const void* act_hi, const void* act_lo,
                                  const uint32_t* act_amax, uint8_t* planes, float* row_scale,
                                  int num_assign, int inter, int rows_cap, bool pdl,
                                  cudaStream_t stream) {
  const uint4* hi = static_cast<const uint4*>(act_hi);
  const uint4* lo = static_cast<const uint4*>(act_lo);
  void* args[] = {&hi, &lo, &act_amax, &planes, &row_scale, &inter, &rows_cap};
  const int chunks = (inter / 8 + kRowThreads - 1) / kRowThreads;
  return launch_with_pdl(reinterpret_cast<const void*>(&act_planes_fp8_kernel),
                         dim3(num_assign, chunks), dim3(kRowThreads), args, pdl, stream);
}

}  // namespace b200moe
