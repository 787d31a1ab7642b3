// Router front end: top-k over the router logits and a softmax over the selected
// logits, one warp per token.  It restates what the reference does with two
// PyTorch calls in front of the layer (baseline/routing.py:48-55: torch.topk, then
// softmax of the selected logits in FP32, cast back to the logits' dtype) and what its
// benchmark counts inside routing_us / total_us (benchmark/benchmark_goal_1b.py:464).
// Selected experts come out in descending logit order; among equal logits the lower
// expert id wins; a NaN logit ranks above every number, as torch.topk ranks it, and a row
// of NaN or -inf still yields top_k distinct ids in [0, E).
#include "common.cuh"

namespace b200moe {

constexpr int kRouterWarps = 4;

template <typename T>
__device__ __forceinline__ float logit_to_float(T v);
template <>
__device__ __forceinline__ float logit_to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float logit_to_float<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}

template <typename T>
__global__ void __launch_bounds__(kRouterWarps * 32)
router_topk_kernel(const T* __restrict__ logits, int num_tokens, int num_experts, int top_k,
                   int64_t* __restrict__ ids, __nv_bfloat16* __restrict__ weights_bf16,
                   float* __restrict__ weights_f32) {
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int token = blockIdx.x * kRouterWarps + (threadIdx.x >> 5);
  if (token >= num_tokens) return;

  // each lane keeps experts lane, lane+32, ... (at most 8 for E <= 256)
  float v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < num_experts ? logit_to_float(logits[(size_t)token * num_experts + e]) : -INFINITY;
  }
  // Selection key: the logit's bits mapped to an unsigned order (NaN above every number,
  // as torch.topk ranks it; -inf still above nothing), then the lower expert id; 0 marks
  // an entry that is taken or does not exist.  Every slot therefore gets an id in [0, E)
  // as long as top_k <= E, whatever the logits hold.
  unsigned long long key[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int e = lane + 32 * i;
    const uint32_t bits = __float_as_uint(v[i]);
    uint32_t order = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
    if (v[i] != v[i]) order = 0xFFFFFFFFu;
    key[i] = e < num_experts ? ((unsigned long long)order << 32) | (uint32_t)(0x7fffffff - e) : 0ull;
  }
  float sel[8];
  float denom = 0.0f;
  for (int k = 0; k < top_k; ++k) {
    unsigned long long best = 0ull;
#pragma unroll
    for (int i = 0; i < 8; ++i) best = key[i] > best ? key[i] : best;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, d);
      best = other > best ? other : best;
    }
    const int best_e = 0x7fffffff - (int)(uint32_t)(best & 0xFFFFFFFFull);
    float value = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (lane + 32 * i == best_e) {
        value = v[i];
        key[i] = 0ull;  // taken
      }
    }
    // the owner lane holds the logit; everyone needs it for the softmax
    value = __shfl_sync(0xffffffffu, value, best_e & 31);
    if (lane == 0) ids[(size_t)token * top_k + k] = best_e;
    sel[k] = value;
  }
  // softmax over the selected logits; sel[0] is the maximum
  const float top = sel[0];
  for (int k = 0; k < top_k; ++k) {
    sel[k] = expf(sel[k] - top);
    denom += sel[k];
  }
  if (lane == 0) {
    for (int k = 0; k < top_k; ++k) {
      const float w = sel[k] / denom;
      if (weights_bf16) weights_bf16[(size_t)token * top_k + k] = __float2bfloat16_rn(w);
      if (weights_f32) weights_f32[(size_t)token * top_k + k] = w;
    }
  }
}

cudaError_t launch_router_topk(const void* logits, bool logits_f32, int num_tokens,
                               int num_experts, int top_k, int64_t* ids, void* weights_bf16,
                               float* weights_f32, cudaStream_t stream) {
  const dim3 grid((num_tokens + kRouterWarps - 1) / kRouterWarps), block(kRouterWarps * 32);
  if (logits_f32) {
    router_topk_kernel<float><<<grid, block, 0, stream>>>(
        static_cast<const float*>(logits), num_tokens, num_experts, top_k, ids,
        static_cast<__nv_bfloat16*>(weights_bf16), weights_f32);
  } else {
    router_topk_kernel<__nv_bfloat16><<<grid, block, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(logits), num_tokens, num_experts, top_k, ids,
        static_cast<__nv_bfloat16*>(weights_bf16), weights_f32);
  }
  return cudaGetLastError();
}

}  // namespace b200moe
