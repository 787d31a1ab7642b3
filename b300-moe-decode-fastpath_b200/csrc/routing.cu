// Stage 1: routing metadata in one launch of one thread block.
//
// Computes what the reference builds with three fills, three kernels and a
// copy (csrc/routing_kernels.cu:24-139, fastpath/b300_moe.py:652-653):
//   counts[e]          = #{a : id[a] == e}
//   offsets            = [0, cumsum(counts)]   (empty experts: equal adjacent offsets)
//   permutation        = stable argsort of the flattened ids
//   reverse_mapping    = its inverse
// and, in the same launch, the segment schedule both grouped GEMMs read, so no
// host synchronisation is needed to size their work.
//
// Stability: assignments are visited in increasing order, one block-width (at
// most 1024) per round; in a round, a warp owns 32 consecutive assignments, a lane's rank among equal
// ids in its warp is the number of lower lanes with the same id, and warps are
// ordered by a per-expert running cursor.  Rows of one expert therefore keep
// increasing assignment ids, which is torch.argsort(stable=True).
#include <mutex>

#include "common.cuh"

namespace b200moe {

constexpr int kRoutingThreads = 1024;   // most threads per block; small calls launch fewer
constexpr int kRoutingWarps = kRoutingThreads / 32;

// Exclusive scan of one int per thread over the whole block.  `total` receives
// the block sum in every thread.  `tmp` is kRoutingWarps ints of shared memory.
__device__ __forceinline__ int block_exclusive_scan(int v, int* tmp, int& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int num_warps = blockDim.x >> 5;
  int inc = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    int n = __shfl_up_sync(0xffffffffu, inc, d);
    if (lane >= d) inc += n;
  }
  if (lane == 31) tmp[warp] = inc;
  __syncthreads();
  int base = 0, sum = 0;
  for (int w = 0; w < num_warps; ++w) {
    int t = tmp[w];
    if (w < warp) base += t;
    sum += t;
  }
  __syncthreads();
  total = sum;
  return base + inc - v;
}

__global__ void __launch_bounds__(kRoutingThreads, 1)
routing_kernel(const int64_t* __restrict__ ids, const __nv_bfloat16* __restrict__ weights,
               int num_assign, int top_k, int num_experts, int64_t* __restrict__ counts,
               int64_t* __restrict__ offsets, int64_t* __restrict__ reverse_mapping,
               int64_t* __restrict__ permutation, int32_t* __restrict__ offsets_i32,
               int64_t* __restrict__ perm_tokens, int64_t* __restrict__ perm_experts,
               __nv_bfloat16* __restrict__ perm_weights, int32_t* __restrict__ sched,
               uint32_t* __restrict__ status, int down_tiles, int down_kblocks, int target_ctas,
               int seg_rows, int id_base, int foreign_ids_allowed, unsigned long long* __restrict__ trace,
               const uint32_t* __restrict__ wait_flags, int wait_world, uint32_t wait_epoch,
               unsigned long long wait_limit_ns, int wait_at_end,
               uint4* __restrict__ zero_rows, int zero_row_vecs) {
  __shared__ int s_cnt[B200MOE_MAX_EXPERTS];
  __shared__ int s_cursor[B200MOE_MAX_EXPERTS];
  extern __shared__ int s_whist[];  // [warps of this launch][num_experts]
  __shared__ int s_tmp[kRoutingWarps];
  __shared__ int s_bad;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int threads = blockDim.x, num_warps = blockDim.x >> 5;
  __shared__ int s_peers_ready;

  // Expert parallel with sharded tokens: the ids, weights and token rows of the other
  // ranks arrive by peer stores; wait (bounded) until every rank has published this
  // forward's epoch.  If a peer never arrives the call routes nothing and reports it.
  if (wait_flags) {
    if (tid == 0) s_peers_ready = 1;
    __syncthreads();
    if (tid < wait_world) {
      const uint64_t t0 = global_timer_ns();
      while (true) {
        uint32_t seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(wait_flags + tid) : "memory");
        if ((int32_t)(seen - wait_epoch) >= 0) break;
        if (global_timer_ns() - t0 > wait_limit_ns) {
          s_peers_ready = 0;
          break;
        }
        __nanosleep(64);
      }
    }
    __syncthreads();
    if (!s_peers_ready) {
      // route nothing: every assignment is marked dropped, so the combine adds nothing
      for (int a = tid; a < num_assign; a += threads) {
        reverse_mapping[a] = -1;
        permutation[a] = -1;
      }
      num_assign = 0;
    }
  }

  // Everything the next kernel needs from this one is written before this grid
  // completes, and it waits for completion; let its launch overlap this one.
  pdl_launch_dependents();

  if (tid < B200MOE_MAX_EXPERTS) s_cnt[tid] = 0;
  if (tid == 0) {
    s_bad = 0;
    // the status word describes the forward this launch begins
    *status = (wait_flags && !s_peers_ready) ? B200MOE_STATUS_PEER_TIMEOUT : 0u;
    if (trace) {
      // end times of the forward that begins; in small-call order the gate+up kernel runs
      // in front of this one and its stamps belong to this forward already
      for (int k = 0; k < kTraceKernels; ++k)
        if (!(wait_at_end && k == kTraceGateUp)) trace[2 * k + 1] = 0ull;
      trace[2 * kTraceRouting] = global_timer_ns();
    }
  }
  __syncthreads();

  // The routing weight of this thread's first assignment is only copied (pass 2); asking
  // for it now lets its memory latency overlap the histogram and the scans.
  __nv_bfloat16 first_weight = __float2bfloat16(0.0f);
  if (perm_weights && weights && tid < num_assign) first_weight = weights[tid];

  // Pass 1: histogram.  Ids outside [0, E) are not counted (the reference
  // ignores them the same way, csrc/routing_kernels.cu:33) and are reported.
  for (int a = tid; a < num_assign; a += threads) {
    const int64_t e = ids[a] - id_base;
    if (e >= 0 && e < (int64_t)num_experts) {
      atomicAdd(&s_cnt[(int)e], 1);
    } else {
      s_bad = 1;
    }
  }
  __syncthreads();

  const bool is_expert = tid < num_experts;
  const int my_cnt = is_expert ? s_cnt[tid] : 0;
  int n_valid;
  const int my_off = block_exclusive_scan(my_cnt, s_tmp, n_valid);
  const int my_chunks = (my_cnt + seg_rows - 1) / seg_rows;
  int n_seg;
  const int my_seg = block_exclusive_scan(my_chunks, s_tmp, n_seg);
  const int n_active = __syncthreads_count(my_cnt > 0);

  if (is_expert) {
    counts[tid] = my_cnt;
    offsets[tid + 1] = my_off + my_cnt;
    offsets_i32[tid] = my_off + my_cnt;
    s_cursor[tid] = my_off;
    for (int c = 0; c < my_chunks; ++c) {
      int32_t* seg = sched + kSchedHeaderWords + kSchedSegWords * (my_seg + c);
      const int done = c * seg_rows;
      seg[0] = tid;
      seg[1] = my_off + done;
      seg[2] = min(seg_rows, my_cnt - done);
      seg[3] = 0;
    }
  }
  if (tid == 0) {
    offsets[0] = 0;
    // Split-K factor of the down projection: when few (segment, tile) units
    // exist, cut K so that about `target_ctas` blocks stream weights at once.
    // (a negative `target_ctas` is a factor forced by the caller, for tuning sweeps)
    const int splits = down_splits_for(n_seg, n_valid, down_tiles, down_kblocks, target_ctas);
    sched[kSchedNumSegments] = n_seg;
    sched[kSchedNumActive] = n_active;
    sched[kSchedNumValidRows] = n_valid;
    sched[kSchedDownSplits] = splits;
    sched[kSchedSegRows] = seg_rows;
    sched[5] = 0;
    sched[6] = 0;
    sched[7] = 0;
  }
  __syncthreads();

  // Pass 2: stable placement, one block-width of assignments per round.
  for (int base = 0; base < num_assign; base += threads) {
    for (int i = tid; i < num_warps * num_experts; i += threads) s_whist[i] = 0;
    __syncthreads();

    const int a = base + tid;
    int64_t e64 = -1;
    if (a < num_assign) e64 = ids[a] - id_base;
    const bool valid = (a < num_assign) && e64 >= 0 && e64 < (int64_t)num_experts;
    const int e = valid ? (int)e64 : -1;
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    if (valid && rank == 0) s_whist[warp * num_experts + e] = __popc(peers);
    __syncthreads();

    if (is_expert) {
      int run = s_cursor[tid];
      for (int w = 0; w < num_warps; ++w) {
        const int t = s_whist[w * num_experts + tid];
        s_whist[w * num_experts + tid] = run;
        run += t;
      }
      s_cursor[tid] = run;
    }
    __syncthreads();

    if (valid) {
      const int p = s_whist[warp * num_experts + e] + rank;
      reverse_mapping[a] = p;
      permutation[p] = a;
      if (perm_tokens) perm_tokens[p] = a / top_k;
      if (perm_experts) perm_experts[p] = e;
      if (perm_weights && weights) perm_weights[p] = base == 0 ? first_weight : weights[a];
    } else if (a < num_assign) {
      reverse_mapping[a] = -1;
    }
    __syncthreads();
  }

  // Rows past the valid ones exist only when some id was out of range: mark
  // them invalid so the gather zero-fills them and nothing reads stale indices.
  if (s_bad) {
    for (int p = n_valid + tid; p < num_assign; p += threads) {
      permutation[p] = -1;
      if (perm_tokens) perm_tokens[p] = -1;
      if (perm_experts) perm_experts[p] = -1;
      if (perm_weights) perm_weights[p] = __float2bfloat16(0.0f);
    }
    // On an expert-parallel rank, ids outside the local range are other ranks' experts.
    if (tid == 0 && !foreign_ids_allowed) atomicOr(status, B200MOE_STATUS_BAD_EXPERT_ID);
    // A forward in small-call order has no gather kernel: the rows past the valid ones,
    // which that kernel zero-fills, are cleared here.
    if (zero_rows) {
      const size_t first = (size_t)n_valid * zero_row_vecs;
      const size_t count = (size_t)(num_assign - n_valid) * zero_row_vecs;
      for (size_t v = tid; v < count; v += threads) zero_rows[first + v] = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  trace_end(trace, kTraceRouting);
  // Small-call order: the kernel in front of this one is the gate+up GEMM, and the kernel
  // behind it waits for this grid alone.  Leaving only once gate+up has completed makes
  // "routing complete" imply "gate+up complete" for everything that follows.
  if (wait_at_end) pdl_wait();
}

cudaError_t launch_routing(const int64_t* ids, const void* weights, int num_assign, int top_k,
                           int num_experts, int64_t* counts, int64_t* offsets,
                           int64_t* reverse_mapping, int64_t* permutation, int32_t* offsets_i32,
                           int64_t* perm_tokens, int64_t* perm_experts, void* perm_weights,
                           int32_t* sched, uint32_t* status, int down_tiles, int down_kblocks,
                           int target_ctas, int seg_rows, int id_base, bool foreign_ids_allowed,
                           const uint32_t* wait_flags, int wait_world, uint32_t wait_epoch,
                           unsigned long long wait_limit_ns, bool after_gate_up, bool pdl,
                           bool after_dispatch, void* zero_rows, int zero_row_vecs,
                           cudaStream_t stream) {
  // One thread per expert and per assignment of a round, in whole warps; fewer warps make
  // the block-wide barriers of a decode-sized call cheaper.
  int threads = num_assign > num_experts ? num_assign : num_experts;
  threads = (threads + 31) / 32 * 32;
  if (threads > kRoutingThreads) threads = kRoutingThreads;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1);
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = sizeof(int) * (size_t)(threads / 32) * num_experts;  // <= 32 KB
  cfg.stream = stream;
  // `after_gate_up`: small-call order, this kernel follows the gate+up GEMM in the stream
  // and runs beside it (programmatic dependent launch); see the end of the kernel.
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  // `after_dispatch`: the kernel in front is this step's dispatch of sharded tokens, whose
  // flags this kernel waits for anyway (its own rank's included), so it need not wait for
  // that kernel's completion, only for the flags.
  cfg.numAttrs = ((after_gate_up && pdl) || (after_dispatch && wait_flags != nullptr)) ? 1 : 0;
  return cudaLaunchKernelEx(
      &cfg, routing_kernel, ids, static_cast<const __nv_bfloat16*>(weights), num_assign, top_k,
      num_experts, counts, offsets, reverse_mapping, permutation, offsets_i32, perm_tokens,
      perm_experts, static_cast<__nv_bfloat16*>(perm_weights), sched, status, down_tiles,
      down_kblocks, target_ctas, seg_rows, id_base, foreign_ids_allowed ? 1 : 0,
      reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(status) + kTraceOffsetBytes),
      wait_flags, wait_world, wait_epoch, wait_limit_ns, after_gate_up ? 1 : 0,
      static_cast<uint4*>(zero_rows), zero_row_vecs);
}

// ---------------------------------------------------------------------------
// Routing for callers that must not allocate.
//
// The routing kernel needs a few KB of device scratch (status word + segment
// schedule).  Hosts that gave all device memory to their own arena, or that sit
// behind a plugin interface with a "no allocation after initialisation" rule,
// cannot supply one with cudaMalloc.  For them the
// scratch lives in this translation unit, inside the loaded module: every GPU
// that loads the library holds kStaticRoutingScratchBytes until the process ends.
//
// `g_static_routing_scratch` is a device symbol.  In host code its name is only a
// stand-in, so the device address is looked up once per device with
// cudaGetSymbolAddress (with that device current) and cached.
// ---------------------------------------------------------------------------
constexpr int kStaticRoutingMaxAssignments = B200MOE_STATIC_ROUTING_MAX_ASSIGNMENTS;
constexpr size_t kStaticRoutingScratchBytes = 8192;
static_assert(kStatusBytes + sizeof(int32_t) * (kSchedHeaderWords +
                                                (size_t)kSchedSegWords *
                                                    (B200MOE_MAX_EXPERTS +
                                                     kStaticRoutingMaxAssignments / kSegRows + 1)) <=
                  kStaticRoutingScratchBytes,
              "static routing scratch too small for its stated maximum");

static __device__ __align__(256) unsigned char g_static_routing_scratch[kStaticRoutingScratchBytes];

namespace {
constexpr int kStaticMaxDevices = 64;
std::mutex g_static_mutex;
void* g_static_scratch_addr[kStaticMaxDevices] = {};
}  // namespace

// Returns the device address of the static scratch on the current device.
static cudaError_t static_routing_scratch(void** out) {
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= kStaticMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_scratch_addr[dev] == nullptr) {
    void* addr = nullptr;
    err = cudaGetSymbolAddress(&addr, g_static_routing_scratch);
    if (err != cudaSuccess) return err;
    g_static_scratch_addr[dev] = addr;
  }
  *out = g_static_scratch_addr[dev];
  return cudaSuccess;
}

cudaError_t launch_routing_static(const int64_t* ids, const void* weights, int num_assign,
                                  int top_k, int num_experts, int64_t* counts, int64_t* offsets,
                                  int64_t* reverse_mapping, int64_t* permutation,
                                  int32_t* offsets_i32, int64_t* perm_tokens,
                                  int64_t* perm_experts, void* perm_weights, int down_tiles,
                                  int down_kblocks, int target_ctas, cudaStream_t stream) {
  void* base = nullptr;
  cudaError_t err = static_routing_scratch(&base);
  if (err != cudaSuccess) return err;
  unsigned char* b = static_cast<unsigned char*>(base);
  // The kernel clears the status word and rewrites every schedule entry it
  // later reports as used, so nothing of the previous call survives.
  return launch_routing(ids, weights, num_assign, top_k, num_experts, counts, offsets,
                        reverse_mapping, permutation, offsets_i32, perm_tokens, perm_experts,
                        perm_weights, reinterpret_cast<int32_t*>(b + kStatusBytes),
                        reinterpret_cast<uint32_t*>(b), down_tiles, down_kblocks, target_ctas,
                        kSegRows, 0, false, nullptr, 0, 0u, 0ull, false, false, false, nullptr,
                        0, stream);
}

}  // namespace b200moe
