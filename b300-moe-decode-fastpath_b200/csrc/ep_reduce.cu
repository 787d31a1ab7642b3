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
  const int token = blockIdx.x;
  const int col = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  if (!s_ready) {
    // A peer never arrived: report it; the rows read as zeros, never as stale memory.
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, B200MOE_STATUS_PEER_TIMEOUT);
    if (col < p.hidden)
      p.output[((size_t)token * p.hidden + col) >> 3] = make_uint4(0u, 0u, 0u, 0u);
    return;
  }
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
// Combine and cross-rank reduce in one kernel.  Replaces the pair "combine kernel
// (FP32 partial output) + ep_reduce_kernel" of an expert-parallel forward:
//
//  1. every block computes this rank's weighted sum for its (token, 1024 columns) from the
//     split-K slices of the down projection, exactly as the combine kernel does, keeps it
//     in registers and -- only if this rank owns an expert of the token -- stores it to
//     this rank's peer-mapped partial buffer;
//  2. the block that finishes last publishes the epoch into flags[rank] of every rank;
//  3. blocks of the tokens this rank must output wait (bounded) until every rank has
//     published, then add the partial rows of the ranks that own an expert of the token,
//     in rank order (their own from registers, the others with plain peer loads), and
//     round once to BF16.  Which ranks those are follows from the token's expert ids,
//     which every rank holds: a token routed to K experts reads at most K rows instead of
//     `world`.
//
// Waiting for every rank (not only the owners) costs nothing -- a rank without work
// publishes early -- and keeps the ranks within one forward of each other, which is what
// makes two alternating partial buffers enough.  Blocks of one grid wait for other GPUs,
// never for each other; the host uses this kernel only while the whole grid is resident at
// once (what the occupancy calculation allows), so the publishing block of every rank
// always gets to run.
// ---------------------------------------------------------------------------
struct EpCombineParams {
  const int64_t* reverse_mapping;   // [T*K] local rows, -1 for other ranks' assignments
  const __nv_bfloat16* weights;     // [T,K]
  const float* slices;              // [splits][rows_cap][H] of the down projection
  const int32_t* sched;
  uint4* expert_out;                // [rows_cap,H] bf16 or null
  const int64_t* ids;               // [T,K] global expert ids
  float* partial[kMaxEpWorld];      // every rank's FP32 [T,H] partial buffer
  uint32_t* flags[kMaxEpWorld];
  unsigned int* block_counter;      // local, zero between launches
  uint4* output;                    // BF16 [out_tokens, H]
  uint32_t* status;
  size_t slice_elems;
  int num_assign, top_k, hidden, experts_per_rank;
  int world, rank, first_token, out_tokens;
  uint32_t epoch;
  unsigned long long wait_limit_ns;
  unsigned long long* trace;
};

__global__ void __launch_bounds__(128, 4)
ep_combine_reduce_kernel(const EpCombineParams p) {
  __shared__ int s_flag;
  pdl_wait();  // the down projection of this rank has completed
  pdl_launch_dependents();
  trace_start(p.trace, kTraceCombine);
  const int token = blockIdx.x;
  const int col = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  const bool active = col < p.hidden;
  const int splits = p.sched[kSchedDownSplits];

  // ---- 1. this rank's share of the token --------------------------------------------
  // Slot metadata first (independent loads), then per slot all split-K slices at once: the
  // loads of one slot are issued back to back and only the additions are ordered.
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
  int64_t rows[8], ids[8];
  float wts[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    rows[k] = -1;
    ids[k] = -1;
    wts[k] = 0.0f;
    if (k < p.top_k) {
      rows[k] = p.reverse_mapping[token * p.top_k + k];
      ids[k] = p.ids[token * p.top_k + k];
      wts[k] = __bfloat162float(p.weights[token * p.top_k + k]);
    }
  }
  bool contributes = false;
  unsigned owners = 0u;  // ranks that own an expert of this token
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    if (ids[k] >= 0 && ids[k] < (int64_t)p.world * p.experts_per_rank)
      owners |= 1u << (int)(ids[k] / p.experts_per_rank);
    if (rows[k] >= 0 && rows[k] < (int64_t)p.num_assign) contributes = true;
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    if (k >= p.top_k) break;
    const int64_t row = rows[k];
    if (row < 0 || row >= (int64_t)p.num_assign || !active) continue;
    const float* src = p.slices + (size_t)row * p.hidden + col;
    float4 lo[kDownSplitMax], hi[kDownSplitMax];
#pragma unroll
    for (int s = 0; s < kDownSplitMax; ++s) {
      if (s < splits) {
        lo[s] = *reinterpret_cast<const float4*>(src + (size_t)s * p.slice_elems);
        hi[s] = *reinterpret_cast<const float4*>(src + (size_t)s * p.slice_elems + 4);
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
    if (p.expert_out) {
      uint4 packed;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
      for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      p.expert_out[((size_t)row * p.hidden + col) >> 3] = packed;
    }
    const float w = wts[k];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = fmaf(v[i], w, acc[i]);
  }
  const size_t at = (size_t)token * p.hidden + col;
  if (active && contributes) {
    float4* o = reinterpret_cast<float4*>(p.partial[p.rank] + at);
    o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }

  // ---- 2. the last block of the grid publishes the epoch -----------------------------
  // One system-scope fence per block: the block barrier orders every thread's stores
  // before thread 0's fence, which then covers them all (a fence per thread costs
  // several microseconds with a few hundred blocks fencing at once).
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int total = gridDim.x * gridDim.y;
    s_flag = (atomicAdd(p.block_counter, 1u) == total - 1u) ? 1 : 0;
  }
  __syncthreads();
  if (s_flag) {
    if (threadIdx.x == 0) *p.block_counter = 0u;
    if (threadIdx.x < p.world) {
      __threadfence_system();
      st_release_sys(p.flags[threadIdx.x] + p.rank, p.epoch);
    }
  }

  // ---- 3. tokens this rank outputs ---------------------------------------------------
  if (token < p.first_token || token >= p.first_token + p.out_tokens) return;
  __syncthreads();
  if (threadIdx.x == 0) s_flag = 1;
  __syncthreads();
  if (threadIdx.x < p.world && threadIdx.x != p.rank) {
    const uint32_t* flag = p.flags[p.rank] + threadIdx.x;
    const uint64_t t0 = global_timer_ns();
    while ((int32_t)(ld_acquire_sys(flag) - p.epoch) < 0) {
      if (global_timer_ns() - t0 > p.wait_limit_ns) {
        s_flag = 0;
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  const size_t out_at = ((size_t)(token - p.first_token) * p.hidden + col) >> 3;
  if (!s_flag) {
    // A peer never arrived: report it; the rows read as zeros, never as stale memory.
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, B200MOE_STATUS_PEER_TIMEOUT);
    if (active) p.output[out_at] = make_uint4(0u, 0u, 0u, 0u);
    return;
  }
  if (!active) return;
  // all peer rows are requested before the first addition; the sum itself is in rank order
  float4 plo[kMaxEpWorld], phi[kMaxEpWorld];
#pragma unroll
  for (int r = 0; r < kMaxEpWorld; ++r) {
    plo[r] = phi[r] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (r < p.world && r != p.rank && ((owners >> r) & 1u)) {
      plo[r] = *reinterpret_cast<const float4*>(p.partial[r] + at);
      phi[r] = *reinterpret_cast<const float4*>(p.partial[r] + at + 4);
    }
  }
  float sum[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) sum[i] = 0.0f;
#pragma unroll
  for (int r = 0; r < kMaxEpWorld; ++r) {
    if (r < p.world && ((owners >> r) & 1u)) {
      if (r == p.rank) {
#pragma unroll
        for (int i = 0; i < 8; ++i) sum[i] += acc[i];
      } else {
        sum[0] += plo[r].x; sum[1] += plo[r].y; sum[2] += plo[r].z; sum[3] += plo[r].w;
        sum[4] += phi[r].x; sum[5] += phi[r].y; sum[6] += phi[r].z; sum[7] += phi[r].w;
      }
    }
  }
  uint4 packed;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(sum[2 * i], sum[2 * i + 1]);
  p.output[out_at] = packed;
  trace_end(p.trace, kTraceCombine);
}

// Blocks of ep_combine_reduce_kernel that are resident at once on the current device
// (occupancy x SM count), 0 when it cannot be found out.  Asked once per device.
int ep_combine_reduce_resident_blocks(int sm_count) {
  static int per_sm[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (per_sm[dev] == 0) {
    int blocks = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, ep_combine_reduce_kernel, 128,
                                                      0) != cudaSuccess)
      return 0;
    per_sm[dev] = blocks > 0 ? blocks : -1;
  }
  return per_sm[dev] > 0 ? per_sm[dev] * sm_count : 0;
}

cudaError_t launch_ep_combine_reduce(const int64_t* reverse_mapping, const void* weights,
                                     const float* slices, const int32_t* sched,
                                     void* expert_out, const int64_t* ids,
                                     const void* const* partial_ptrs, void* const* flag_ptrs,
                                     unsigned int* block_counter, void* output,
                                     uint32_t* status, size_t slice_elems, int num_tokens,
                                     int top_k, int hidden, int experts_per_rank, int world,
                                     int rank, int first_token, int out_tokens, uint32_t epoch,
                                     unsigned long long wait_limit_ns, unsigned long long* trace,
                                     bool pdl, cudaStream_t stream) {
  EpCombineParams p = {};
  p.reverse_mapping = reverse_mapping;
  p.weights = static_cast<const __nv_bfloat16*>(weights);
  p.slices = slices;
  p.sched = sched;
  p.expert_out = static_cast<uint4*>(expert_out);
  p.ids = ids;
  for (int r = 0; r < world; ++r) {
    p.partial[r] = static_cast<float*>(const_cast<void*>(partial_ptrs[r]));
    p.flags[r] = static_cast<uint32_t*>(flag_ptrs[r]);
  }
  p.block_counter = block_counter;
  p.output = static_cast<uint4*>(output);
  p.status = status;
  p.slice_elems = slice_elems;
  p.num_assign = num_tokens * top_k;
  p.top_k = top_k;
  p.hidden = hidden;
  p.experts_per_rank = experts_per_rank;
  p.world = world;
  p.rank = rank;
  p.first_token = first_token;
  p.out_tokens = out_tokens;
  p.epoch = epoch;
  p.wait_limit_ns = wait_limit_ns;
  p.trace = trace;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(num_tokens, (hidden / 8 + 127) / 128);
  cfg.blockDim = dim3(128);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, ep_combine_reduce_kernel, p);
}

// ---------------------------------------------------------------------------
// Combine and cross-rank reduce by PUSHING flagged rows (the low-latency variant).
//
// ep_combine_reduce_kernel above pays a chain of long-latency steps after the combine:
// system fence, counter, fence, flag store over NVLink, the peers' polls, then a read over
// NVLink.  Here every 4-byte value travels with its own 4-byte flag in one 8-byte word
// (single-copy atomic), so no fence and no separate flag are needed:
//
//  1. as above: this rank's weighted sum for (token, 1024 columns), kept in registers;
//  2. if the rank owns an expert of the token, the block stores {value, epoch} words
//     straight into the inbox of every rank that outputs the token (all ranks when tokens
//     are replicated, one rank when they are sharded), slot [parity][this rank][token];
//  3. blocks of tokens this rank outputs poll their OWN inbox (local memory) for the rows
//     of the other owners until every word carries this epoch, add in rank order (their
//     own from registers) and round once to BF16.
//
// A block never waits for another block of its grid, and it pushes before it waits.
// Inboxes alternate by epoch parity.  A slot is rewritten two epochs later; before pushing
// to a rank the block checks that rank's progress word (every rank stores its epoch into
// progress[rank] of all ranks when its kernel starts, i.e. after its previous forward has
// completed), which in steady state is long since there.  All waits are bounded; a wait
// that runs out zeroes the rows and sets B200MOE_STATUS_PEER_TIMEOUT.
// ---------------------------------------------------------------------------
struct EpPushCombineParams {
  const int64_t* reverse_mapping;
  const __nv_bfloat16* weights;
  const float* slices;
  const int32_t* sched;
  uint4* expert_out;
  const int64_t* ids;
  uint4* inbox[kMaxEpWorld];        // every rank's inbox: [2][world][cap_tokens][H] words of 8 bytes
  uint32_t* progress[kMaxEpWorld];  // every rank's progress array uint32[world]
  uint4* output;
  uint32_t* status;
  size_t slice_elems;
  size_t rank_stride;               // cap_tokens * H words between two source ranks' slots
  int num_assign, top_k, hidden, experts_per_rank;
  int world, rank, first_token, out_tokens;
  int tokens_per_rank;              // sharded tokens: rank t / tokens_per_rank outputs token t; 0: all do
  uint32_t epoch;
  unsigned long long wait_limit_ns;
  unsigned long long* trace;
};

__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_volatile_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

__global__ void __launch_bounds__(128, 4)
ep_combine_push_kernel(const EpPushCombineParams p) {
  __shared__ int s_ok;
  pdl_wait();  // the down projection of this rank has completed
  pdl_launch_dependents();
  trace_start(p.trace, kTraceCombine);
  const int token = blockIdx.x;
  // A block covers 1024 columns, a warp 256 of them, and a lane the four column PAIRS
  // base + 64 j + 2 lane (j = 0..3): every 16-byte {value, epoch, value, epoch} store of a
  // warp then lands in one contiguous 512-byte run, so the stores cross NVLink as full
  // 128-byte writes instead of 32 separate 16-byte ones (a lane that owned 8 adjacent
  // columns wrote at a 64-byte stride: ~8 us more at T = 64).
  const int warp_base = blockIdx.y * 1024 + (threadIdx.x >> 5) * 256 + 2 * (threadIdx.x & 31);
  int cols[4];
  bool on[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    cols[j] = warp_base + 64 * j;
    on[j] = cols[j] < p.hidden;
  }
  const int splits = p.sched[kSchedDownSplits];
  // this rank has begun epoch `epoch`: its previous forward, and every read that forward
  // made of this rank's inbox, is complete
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x < p.world)
    st_relaxed_sys(p.progress[threadIdx.x] + p.rank, p.epoch);
  // ranks that output this token, as a mask
  unsigned targets = p.tokens_per_rank > 0 ? 1u << (token / p.tokens_per_rank)
                                           : (p.world >= 32 ? 0xffffffffu : (1u << p.world) - 1u);
  targets &= ~(1u << p.rank);
  // how far each target has got (checked in step 2): the load goes out together with the
  // loads of step 1 instead of after them; the word only ever grows, so an early value
  // that already passes is as good as a late one
  const bool watches = threadIdx.x < p.world && ((targets >> threadIdx.x) & 1u);
  uint32_t progress_seen = p.epoch;
  if (watches) progress_seen = ld_relaxed_sys(p.progress[p.rank] + threadIdx.x);

  // ---- 1. this rank's share of the token (as in ep_combine_reduce_kernel) ------------
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
  int64_t rows[8], ids[8];
  float wts[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    rows[k] = -1;
    ids[k] = -1;
    wts[k] = 0.0f;
    if (k < p.top_k) {
      rows[k] = p.reverse_mapping[token * p.top_k + k];
      ids[k] = p.ids[token * p.top_k + k];
      wts[k] = __bfloat162float(p.weights[token * p.top_k + k]);
    }
  }
  bool contributes = false;
  unsigned owners = 0u;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    if (ids[k] >= 0 && ids[k] < (int64_t)p.world * p.experts_per_rank)
      owners |= 1u << (int)(ids[k] / p.experts_per_rank);
    if (rows[k] >= 0 && rows[k] < (int64_t)p.num_assign) contributes = true;
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    if (k >= p.top_k) break;
    const int64_t row = rows[k];
    if (row < 0 || row >= (int64_t)p.num_assign) continue;
    const float* src = p.slices + (size_t)row * p.hidden;
    float2 part[kDownSplitMax][4];
#pragma unroll
    for (int s = 0; s < kDownSplitMax; ++s) {
      if (s < splits) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          part[s][j] = on[j] ? *reinterpret_cast<const float2*>(src + (size_t)s * p.slice_elems +
                                                                 cols[j])
                             : make_float2(0.0f, 0.0f);
      }
    }
    float v[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[2 * j] = part[0][j].x;
      v[2 * j + 1] = part[0][j].y;
    }
#pragma unroll
    for (int s = 1; s < kDownSplitMax; ++s) {
      if (s < splits) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          v[2 * j] += part[s][j].x;
          v[2 * j + 1] += part[s][j].y;
        }
      }
    }
    if (p.expert_out) {
      __nv_bfloat162* out_row =
          reinterpret_cast<__nv_bfloat162*>(p.expert_out) + (((size_t)row * p.hidden) >> 1);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (on[j]) out_row[cols[j] >> 1] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
    }
    const float w = wts[k];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = fmaf(v[i], w, acc[i]);
  }

  // ---- 2. push this rank's row to the ranks that output the token --------------------
  const uint64_t t0 = global_timer_ns();
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (contributes && watches) {
    // the slot was last used two epochs ago: wait (normally not at all) until the target
    // has begun the previous epoch
    const uint32_t* word = p.progress[p.rank] + threadIdx.x;
    while ((int32_t)(progress_seen - (p.epoch - 1u)) < 0) {
      if (global_timer_ns() - t0 > p.wait_limit_ns) {
        s_ok = 0;
        break;
      }
      __nanosleep(32);
      progress_seen = ld_relaxed_sys(word);
    }
  }
  __syncthreads();
  // words of 8 bytes: word index of (slot rank r, token, column) inside one parity half;
  // a column pair is one 16-byte vector (every term of the index is even)
  const size_t parity_base = (size_t)(p.epoch & 1u) * p.world * p.rank_stride;
  const size_t at = (size_t)token * p.hidden;
  if (contributes && s_ok) {
    const size_t word = parity_base + (size_t)p.rank * p.rank_stride + at;
#pragma unroll
    for (int r = 0; r < kMaxEpWorld; ++r) {
      if (r < p.world && ((targets >> r) & 1u)) {
        uint4* dst = p.inbox[r] + (word >> 1);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (on[j])
            dst[cols[j] >> 1] = make_uint4(__float_as_uint(acc[2 * j]), p.epoch,
                                           __float_as_uint(acc[2 * j + 1]), p.epoch);
      }
    }
  }

  // ---- 3. tokens this rank outputs ---------------------------------------------------
  if (token < p.first_token || token >= p.first_token + p.out_tokens) return;
  __nv_bfloat162* out_row = reinterpret_cast<__nv_bfloat162*>(p.output) +
                            (((size_t)(token - p.first_token) * p.hidden) >> 1);
  float sum[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) sum[i] = 0.0f;
  bool ok = s_ok != 0;
#pragma unroll
  for (int r = 0; r < kMaxEpWorld; ++r) {
    if (r >= p.world || !((owners >> r) & 1u)) continue;
    if (r == p.rank) {
#pragma unroll
      for (int i = 0; i < 8; ++i) sum[i] += acc[i];
      continue;
    }
    const uint4* src = p.inbox[p.rank] + ((parity_base + (size_t)r * p.rank_stride + at) >> 1);
    uint4 w[4];
    uint32_t spins = 0;
    while (ok) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        w[j] = on[j] ? ld_volatile_v4(src + (cols[j] >> 1)) : make_uint4(0u, p.epoch, 0u, p.epoch);
      bool all = true;
#pragma unroll
      for (int j = 0; j < 4; ++j) all = all && w[j].y == p.epoch && w[j].w == p.epoch;
      if (all) break;
      if ((++spins & 15u) == 0u && global_timer_ns() - t0 > p.wait_limit_ns) ok = false;
    }
    if (ok) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        sum[2 * j] += __uint_as_float(w[j].x);
        sum[2 * j + 1] += __uint_as_float(w[j].z);
      }
    }
  }
  // a wait that ran out anywhere in the block: the whole block's rows read as zeros
  if (!ok) s_ok = 0;
  __syncthreads();
  if (!s_ok) {
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, B200MOE_STATUS_PEER_TIMEOUT);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (on[j]) out_row[cols[j] >> 1] = __floats2bfloat162_rn(0.0f, 0.0f);
    return;
  }
#pragma unroll
  for (int j = 0; j < 4; ++j)
    if (on[j]) out_row[cols[j] >> 1] = __floats2bfloat162_rn(sum[2 * j], sum[2 * j + 1]);
  trace_end(p.trace, kTraceCombine);
}

int ep_combine_push_resident_blocks(int sm_count) {
  static int per_sm[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (per_sm[dev] == 0) {
    int blocks = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, ep_combine_push_kernel, 128, 0) !=
        cudaSuccess)
      return 0;
    per_sm[dev] = blocks > 0 ? blocks : -1;
  }
  return per_sm[dev] > 0 ? per_sm[dev] * sm_count : 0;
}

cudaError_t launch_ep_combine_push(const int64_t* reverse_mapping, const void* weights,
                                   const float* slices, const int32_t* sched, void* expert_out,
                                   const int64_t* ids, void* const* inbox_ptrs,
                                   void* const* progress_ptrs, void* output, uint32_t* status,
                                   size_t slice_elems, int cap_tokens, int num_tokens, int top_k,
                                   int hidden, int experts_per_rank, int world, int rank,
                                   int first_token, int out_tokens, int tokens_per_rank,
                                   uint32_t epoch, unsigned long long wait_limit_ns,
                                   unsigned long long* trace, bool pdl, cudaStream_t stream) {
  EpPushCombineParams p = {};
  p.reverse_mapping = reverse_mapping;
  p.weights = static_cast<const __nv_bfloat16*>(weights);
  p.slices = slices;
  p.sched = sched;
  p.expert_out = static_cast<uint4*>(expert_out);
  p.ids = ids;
  for (int r = 0; r < world; ++r) {
    p.inbox[r] = static_cast<uint4*>(inbox_ptrs[r]);
    p.progress[r] = static_cast<uint32_t*>(progress_ptrs[r]);
  }
  p.output = static_cast<uint4*>(output);
  p.status = status;
  p.slice_elems = slice_elems;
  p.rank_stride = (size_t)cap_tokens * hidden;
  p.num_assign = num_tokens * top_k;
  p.top_k = top_k;
  p.hidden = hidden;
  p.experts_per_rank = experts_per_rank;
  p.world = world;
  p.rank = rank;
  p.first_token = first_token;
  p.out_tokens = out_tokens;
  p.tokens_per_rank = tokens_per_rank;
  p.epoch = epoch;
  p.wait_limit_ns = wait_limit_ns;
  p.trace = trace;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(num_tokens, (hidden / 8 + 127) / 128);
  cfg.blockDim = dim3(128);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, ep_combine_push_kernel, p);
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
