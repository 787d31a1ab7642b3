// Expert-parallel combine over NVLink peer memory: one kernel that signals this
// rank's partial output as ready, waits (bounded) for every peer's signal, then
// reads all ranks' FP32 partial outputs with plain peer loads, adds them in rank
// order and rounds once to BF16.  It is the fused counterpart of "all-reduce the
// partial outputs, then cast": no library collective, one launch, and the sum
// order is fixed (rank 0 first), so every rank computes bit-identical rows.
//
// Memory used across GPUs (all allocated as peer-mapped symmetric buffers by the
// caller): each rank's partial buffer FP32 [T,H] and each rank's flag array
// uint32[world].  Rank r publishes epoch e by storing e into flags[r] of every
// rank (release, system scope) after its local combine kernel has completed;
// a reader acquires flags[j] >= e before touching rank j's partial buffer.
// Only plain loads/stores touch peer memory: no TMA, no multimem.
#include "common.cuh"

namespace b200moe {

constexpr int kMaxEpWorld = 8;

struct EpReduceParams {
  const float* partial[kMaxEpWorld];   // peer-mapped FP32 [T,H] of every rank
  uint32_t* flags[kMaxEpWorld];        // peer-mapped uint32[world] of every rank
  uint4* output;                        // BF16 [T,H] of this rank
  uint32_t* status;                     // this rank's status word (may be null)
  int world, rank, hidden;
  uint32_t epoch;
  unsigned long long wait_limit_ns;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(128)
ep_reduce_kernel(const EpReduceParams p) {
  __shared__ int s_ready;
  pdl_wait();  // this rank's local combine (previous kernel) has completed
  pdl_launch_dependents();

  // Publish: one block tells every rank (itself included) that epoch `epoch` of this
  // rank's partial buffer is complete.
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x < p.world) {
    __threadfence_system();
    st_release_sys(p.flags[threadIdx.x] + p.rank, p.epoch);
  }

  // Wait, bounded: this rank's own flag array must show the epoch for every rank.
  if (threadIdx.x == 0) s_ready = 1;
  __syncthreads();
  if (threadIdx.x < p.world) {
    const uint32_t* flag = p.flags[p.rank] + threadIdx.x;
    const uint64_t t0 = global_timer_ns();
    // epochs only grow; compare with wrap-around in mind
    while ((int32_t)(ld_acquire_sys(flag) - p.epoch) < 0) {
      if (global_timer_ns() - t0 > p.wait_limit_ns) {
        s_ready = 0;
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  if (!s_ready) {
    // A peer never arrived: report it and leave the output untouched.
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, B200MOE_STATUS_PEER_TIMEOUT);
    return;
  }

  const int token = blockIdx.x;
  const int col = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (col >= p.hidden) return;
  const size_t at = (size_t)token * p.hidden + col;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
#pragma unroll
  for (int r = 0; r < kMaxEpWorld; ++r) {
    if (r < p.world) {
      const float4 lo = *reinterpret_cast<const float4*>(p.partial[r] + at);
      const float4 hi = *reinterpret_cast<const float4*>(p.partial[r] + at + 4);
      acc[0] += lo.x; acc[1] += lo.y; acc[2] += lo.z; acc[3] += lo.w;
      acc[4] += hi.x; acc[5] += hi.y; acc[6] += hi.z; acc[7] += hi.w;
    }
  }
  uint4 packed;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
  p.output[at >> 3] = packed;
}

cudaError_t launch_ep_reduce(const void* const* partial_ptrs, void* const* flag_ptrs, int world,
                             int rank, int num_tokens, int hidden, uint32_t epoch,
                             unsigned long long wait_limit_ns, void* output, uint32_t* status,
                             bool pdl, cudaStream_t stream) {
  EpReduceParams p = {};
  for (int r = 0; r < world; ++r) {
    p.partial[r] = static_cast<const float*>(partial_ptrs[r]);
    p.flags[r] = static_cast<uint32_t*>(flag_ptrs[r]);
  }
  p.output = static_cast<uint4*>(output);
  p.status = status;
  p.world = world;
  p.rank = rank;
  p.hidden = hidden;
  p.epoch = epoch;
  p.wait_limit_ns = wait_limit_ns;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(num_tokens, (hidden / 8 + 127) / 128);
  cfg.blockDim = dim3(128);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, ep_reduce_kernel, p);
}

// ---------------------------------------------------------------------------
// Expert-parallel dispatch of sharded tokens: every rank stores its T/N token rows,
// expert ids and routing weights into slot `rank` of every rank's gathered buffers
// (peer stores over NVLink), and the block that finishes last publishes the epoch into
// flags[rank] of every rank.  The consumer is the routing kernel of the same forward,
// which waits (bounded) until its own flag array shows the epoch for every rank.
// One launch replaces three all-gathers.
// ---------------------------------------------------------------------------
struct EpPushParams {
  const uint4* hidden;        // this rank's [T_local, H] bf16 as 16-byte vectors
  const int64_t* ids;         // this rank's [T_local, K]
  const uint16_t* weights;    // this rank's [T_local, K] bf16 bit patterns
  uint4* hidden_dst[kMaxEpWorld];     // slot `rank` inside rank r's gathered hidden buffer
  int64_t* ids_dst[kMaxEpWorld];
  uint16_t* weights_dst[kMaxEpWorld];
  uint32_t* flags[kMaxEpWorld];       // rank r's dispatch flag array uint32[world]
  unsigned int* block_counter;        // local, zero between launches
  int world, rank;
  int hidden_vecs, id_count;          // T_local*H/8 vectors, T_local*K ids (= weights)
  uint32_t epoch;
};

__global__ void __launch_bounds__(256)
ep_push_kernel(const EpPushParams p) {
  __shared__ int s_is_last;
  pdl_launch_dependents();
  const int stride = gridDim.x * blockDim.x;
  const int first = blockIdx.x * blockDim.x + threadIdx.x;
  for (int v = first; v < p.hidden_vecs; v += stride) {
    const uint4 x = __ldg(p.hidden + v);
#pragma unroll
    for (int r = 0; r < kMaxEpWorld; ++r)
      if (r < p.world) p.hidden_dst[r][v] = x;
  }
  for (int i = first; i < p.id_count; i += stride) {
    const int64_t id = p.ids[i];
    const uint16_t w = p.weights[i];
#pragma unroll
    for (int r = 0; r < kMaxEpWorld; ++r) {
      if (r < p.world) {
        p.ids_dst[r][i] = id;
        p.weights_dst[r][i] = w;
      }
    }
  }
  // The last block to get here knows that every block's stores were issued and fenced.
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int done = atomicAdd(p.block_counter, 1u);
    s_is_last = (done == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (s_is_last) {
    if (threadIdx.x == 0) *p.block_counter = 0u;
    if (threadIdx.x < p.world) {
      __threadfence_system();
      st_release_sys(p.flags[threadIdx.x] + p.rank, p.epoch);
    }
  }
}

cudaError_t launch_ep_push(const void* hidden, const int64_t* ids, const void* weights,
                           void* const* hidden_dst, void* const* ids_dst,
                           void* const* weights_dst, void* const* flag_ptrs,
                           unsigned int* block_counter, int world, int rank, int tokens_local,
                           int top_k, int hidden_size, uint32_t epoch, cudaStream_t stream) {
  EpPushParams p = {};
  p.hidden = static_cast<const uint4*>(hidden);
  p.ids = ids;
  p.weights = static_cast<const uint16_t*>(weights);
  for (int r = 0; r < world; ++r) {
    p.hidden_dst[r] = static_cast<uint4*>(hidden_dst[r]);
    p.ids_dst[r] = static_cast<int64_t*>(ids_dst[r]);
    p.weights_dst[r] = static_cast<uint16_t*>(weights_dst[r]);
    p.flags[r] = static_cast<uint32_t*>(flag_ptrs[r]);
  }
  p.block_counter = block_counter;
  p.world = world;
  p.rank = rank;
  p.hidden_vecs = tokens_local * (hidden_size / 8);
  p.id_count = tokens_local * top_k;
  p.epoch = epoch;
  int blocks = (p.hidden_vecs + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 64) blocks = 64;
  ep_push_kernel<<<blocks, 256, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace b200moe
