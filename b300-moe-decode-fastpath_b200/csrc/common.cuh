// Shared definitions for the sm_100a MoE decode kernels: scratch layout,
// schedule format, and thin inline-PTX wrappers (mbarrier, TMA, tcgen05, PDL).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/b200moe.h"

namespace b200moe {

// ---------------------------------------------------------------------------
// Schedule built on the device by the routing kernel, read by both GEMMs and
// by the combine kernel.  A "segment" is a run of at most kSegRows consecutive
// expert-major rows that belong to one expert; it is the N (token) extent of
// one tcgen05 accumulator tile.
// ---------------------------------------------------------------------------
constexpr int kSegRows = 128;        // max token rows per segment (MMA N <= 128)
constexpr int kSegRowsFp8 = 64;      // ... when the weights are FP8: the token operand is held as
                                     // two to three planes per row, so 64 rows already make
                                     // an MMA of N = 192 and a 24 KB share of every stage
constexpr int kDownSplitMax = 8;     // max split-K factor of the down projection
constexpr int kSchedHeaderWords = 8;
constexpr int kSchedSegWords = 4;    // {expert, row_start, n_rows, reserved}
enum SchedWord {
  kSchedNumSegments = 0,
  kSchedNumActive = 1,      // experts with at least one row
  kSchedNumValidRows = 2,   // rows with an in-range expert id
  kSchedDownSplits = 3,     // split-K factor chosen for the down projection
  kSchedSegRows = 4,        // segment length this schedule was built with
};

// Split-K factor of the down projection for `units` (segment, tile) work units, each of
// `kblocks` K blocks and on average `rows16` token rows (rounded up to a multiple of 16),
// when `resident` blocks fit on the GPU at once.  Cost model fitted to measurements, in
// units of one full wave of unsplit blocks: full waves each take 1/s; the last, partial
// wave of r blocks cannot go faster than ~0.67 of a full wave however few blocks it has (a
// block alone on its SM streams ~33 GB/s against a fair share of ~22), nor than ~0.75 once
// some SMs hold two blocks and others one; every extra split adds fixed work per block
// (start-up, and an epilogue and token tiles that grow with the rows).
// Above four waves of units the tail no longer matters and nothing is split.  Shared by
// the routing kernel (which decides) and the host (which sizes the grid for the worst case).
__host__ __device__ inline int choose_down_splits(int units, int resident, int kblocks,
                                                  int rows16) {
  if (units <= 0 || units >= 4 * resident) return 1;
  int max_splits = kblocks / 4;
  if (max_splits > kDownSplitMax) max_splits = kDownSplitMax;
  if (max_splits < 1) max_splits = 1;
  // start-up and drain of a block cost about as much as streaming 4.7 K blocks; the
  // epilogue and the token tiles add about one more per 16 rows
  const float fixed = 4.7f + (float)(rows16 - 16) * (1.0f / 16.0f);
  int splits = 1;
  float best = 3.0e38f;
  for (int s = 1; s <= max_splits; ++s) {
    const int n = units * s;
    const int full = n / resident;
    const int rest = n - full * resident;
    float tail = 0.0f;
    if (rest > 0) {
      tail = (float)rest / (float)resident;
      const float floor_ = 2 * rest > resident ? 0.75f : 0.67f;
      if (tail < floor_) tail = floor_;
    }
    float cost = ((float)full + tail) / (float)s;
    cost *= 1.0f + fixed * (float)s / (float)kblocks;
    if (cost < best * 0.995f) {
      best = cost;
      splits = s;
    }
  }
  return splits;
}

// Average rows per segment, rounded up to a multiple of 16 and capped at 128: the argument
// of the cost model above.
__host__ __device__ inline int rows16_of(int rows, int segments) {
  if (segments <= 0) return 16;
  int avg = (rows + segments - 1) / segments;
  avg = (avg + 15) / 16 * 16;
  return avg < 16 ? 16 : (avg > 128 ? 128 : avg);
}

// The factor the routing kernel publishes for a call with `n_seg` segments and `n_valid`
// rows.  `request` is the number of resident blocks to aim at, or minus a forced factor.
// One function for every place that must arrive at the same number: the routing kernel,
// down-projection blocks that derive their unit from the expert ids, and the host.
__host__ __device__ inline int down_splits_for(int n_seg, int n_valid, int down_tiles,
                                               int down_kblocks, int request) {
  int splits = request < 0 ? -request
                           : choose_down_splits(n_seg * down_tiles, request, down_kblocks,
                                                rows16_of(n_valid, n_seg));
  if (splits > kDownSplitMax) splits = kDownSplitMax;
  if (splits > down_kblocks) splits = down_kblocks;
  return splits < 1 ? 1 : splits;
}

// Calls with at most this many assignments (T * top_k) can run in "small-call" order: one
// warp holds every expert id of the call in its lanes, so a GEMM block finds its work unit
// with a few warp votes instead of waiting for the routing kernel.
constexpr int kSmallCallMaxAssign = 32;

// What a GEMM launch needs to run in small-call order (host side).
struct SmallCall {
  const int64_t* ids;         // [num_assign] expert ids of the call
  int num_assign, num_experts, id_base, top_k;
  const void* hidden;         // gate+up: [T, H] rows to fetch and to copy to permuted_hidden
  void* permuted_hidden;
  int split_request;          // down: what the routing kernel is given
};

constexpr size_t kScratchAlign = 256;
constexpr size_t kStatusBytes = 256;  // status word lives in the first 256 bytes

__host__ __device__ inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

__host__ __device__ inline int max_segments(int rows, int experts) {
  int active = rows < experts ? rows : experts;
  return active + rows / 16 + 1;  // sized for the shortest segment length any path uses
}

// Byte offsets of the private scratch region for `rows_cap` expert-major rows.
struct ScratchLayout {
  size_t status;     // uint32
  size_t sched;      // int32[kSchedHeaderWords + kSchedSegWords * max_segments]
  size_t act_lo;     // bf16 [rows_cap, I]   low-order halves of the SwiGLU activations
  size_t partials;   // fp32 [kDownSplitMax, rows_cap, H]
  // FP8-weight path only: the token operand of both GEMMs as three E4M3 planes per row
  // (first the gathered hidden rows [3][rows_cap][H], later, in the same bytes, the
  // activations [3][rows_cap][I]) and the per-row scales that go with them
  size_t q_planes;   // uint8 [3, rows_cap, max(H, I)]
  size_t x_scale;    // fp32 [rows_cap]
  size_t a_scale;    // fp32 [rows_cap]
  size_t a_amax;     // uint32 [rows_cap]  bit pattern of max |activation| per row
  size_t total;
};

constexpr int kNvfp4Planes = 4;      // E2M1 planes per token row of the NVFP4-weight path
constexpr int kSegRowsNvfp4 = 64;    // its longest segment: four planes of 64 rows, N = 64 per MMA
constexpr int kFp8Planes = 3;        // activation rows of the down projection
constexpr int kFp8PlanesHidden = 2;  // BF16 hidden rows of gate+up: exact with a power-of-two scale

__host__ __device__ inline ScratchLayout scratch_layout(int rows_cap, int experts, int hidden,
                                                        int inter) {
  ScratchLayout l;
  l.status = 0;
  l.sched = kStatusBytes;
  size_t sched_bytes =
      sizeof(int32_t) * (kSchedHeaderWords + (size_t)kSchedSegWords * max_segments(rows_cap, experts));
  l.act_lo = align_up(l.sched + sched_bytes, kScratchAlign);
  l.partials = align_up(l.act_lo + (size_t)rows_cap * inter * sizeof(__nv_bfloat16), kScratchAlign);
  l.q_planes = align_up(l.partials + (size_t)kDownSplitMax * rows_cap * hidden * sizeof(float),
                        kScratchAlign);
  const size_t widest = (size_t)(hidden > inter ? hidden : inter);
  l.x_scale = align_up(l.q_planes + (size_t)kFp8Planes * rows_cap * widest, kScratchAlign);
  l.a_scale = align_up(l.x_scale + (size_t)rows_cap * sizeof(float), kScratchAlign);
  l.a_amax = align_up(l.a_scale + (size_t)rows_cap * sizeof(float), kScratchAlign);
  l.total = align_up(l.a_amax + (size_t)rows_cap * sizeof(uint32_t), kScratchAlign);
  return l;
}

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------


__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Timeline of one forward, kept in the status area of the scratch region: for kernel k,
// word 2k = time block 0 started, word 2k+1 = time the last block finished
// (%globaltimer, ns).  The routing kernel clears the end times when it starts.
constexpr int kTraceKernels = 8;
constexpr size_t kTraceOffsetBytes = 64;
enum TraceKernel {
  kTraceRouting = 0, kTraceGather = 1, kTraceGateUp = 2, kTraceDown = 3, kTraceCombine = 4,
  kTraceEpReduce = 5, kTraceGateUpFirstData = 6, kTraceDownFirstData = 7,
};
__device__ __forceinline__ void trace_start(unsigned long long* t, int k) {
  if (t && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) t[2 * k] = global_timer_ns();
}
__device__ __forceinline__ void trace_end(unsigned long long* t, int k) {
  if (t && threadIdx.x == 0) atomicMax(&t[2 * k + 1], (unsigned long long)global_timer_ns());
}

// Routing of a small call (num_assign <= 32) held in the lanes of one warp: lane a owns
// assignment a.  Restates the routing kernel's rules for this size -- ids outside
// [id_base, id_base + num_experts) are dropped, every expert with rows is exactly one
// segment, segments are ordered by expert id, rows of an expert keep increasing assignment
// ids -- so a block that uses it agrees with the schedule the routing kernel writes.
struct SmallRouteLane {
  int expert;         // this lane's expert (local id), -1 when the lane has no valid assignment
  unsigned members;   // lanes that hold the same expert
  int rows_before;    // valid assignments whose expert id is lower = first row of this expert
  int segs_before;    // active experts with a lower id = this expert's segment index
  int n_seg, n_valid; // of the whole call
};
__device__ __forceinline__ SmallRouteLane small_route_scan(const int64_t* __restrict__ ids,
                                                           int num_assign, int num_experts,
                                                           int id_base) {
  const unsigned full = 0xffffffffu;
  const int lane = threadIdx.x & 31;
  long long e64 = -1;
  if (lane < num_assign) e64 = (long long)ids[lane] - (long long)id_base;
  const bool valid = lane < num_assign && e64 >= 0 && e64 < (long long)num_experts;
  SmallRouteLane r;
  r.expert = valid ? (int)e64 : -1;
  r.members = __match_any_sync(full, r.expert);
  const bool first = valid && (r.members & ((1u << lane) - 1u)) == 0u;
  const unsigned firsts = __ballot_sync(full, first);
  r.n_valid = __popc(__ballot_sync(full, valid));
  r.n_seg = __popc(firsts);
  r.rows_before = 0;
  r.segs_before = 0;
  for (int j = 0; j < num_assign; ++j) {
    const int ej = __shfl_sync(full, r.expert, j);
    if (ej >= 0 && ej < r.expert) {
      r.rows_before += 1;
      r.segs_before += (int)((firsts >> j) & 1u);
    }
  }
  return r;
}
// The segment with index `seg`: {expert, first row, rows, member lanes}; false when the call
// has fewer segments.  Every lane of the warp gets the same answer.
__device__ __forceinline__ bool small_route_pick(const SmallRouteLane& r, int seg, int& expert,
                                                 int& row_start, int& n_rows,
                                                 unsigned& members) {
  const unsigned full = 0xffffffffu;
  const int lane = threadIdx.x & 31;
  const bool first = r.expert >= 0 && (r.members & ((1u << lane) - 1u)) == 0u;
  const unsigned who = __ballot_sync(full, first && r.segs_before == seg);
  if (who == 0u) return false;
  const int src = __ffs(who) - 1;
  expert = __shfl_sync(full, r.expert, src);
  row_start = __shfl_sync(full, r.rows_before, src);
  members = __shfl_sync(full, r.members, src);
  n_rows = __popc(members);
  return true;
}

// Programmatic dependent launch: wait until the grids this one depends on have
// completed and their writes are visible.  A no-op when the kernel was not
// launched with the programmatic-serialization attribute.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait: gives up after `limit_ns` of wall time or when another thread
// of the block has already given up (`*abort_flag != 0`).  Returns false then.
constexpr uint64_t kPipeWaitLimitNs = 200000000ull;  // 200 ms
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity,
                                                  volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 63u) == 0u) {
      if (*abort_flag) return false;
      if (global_timer_ns() - t0 > kPipeWaitLimitNs) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

// TMA tiled loads into this CTA only, completion on an mbarrier of this CTA.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(dst),
      "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// Same, with an L2 eviction-priority hint (streamed-once weights: evict first).
__device__ __forceinline__ void tma_load_3d_hint(uint32_t dst, const CUtensorMap* map,
                                                 uint32_t bar, int c0, int c1, int c2,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      ".L2::cache_hint [%0], [%1, {%3, %4, %5}], [%2], %6;" ::"r"(dst),
      "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d_hint(uint32_t dst, const CUtensorMap* map,
                                                 uint32_t bar, int c0, int c1, int c2, int c3,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      ".L2::cache_hint [%0], [%1, {%3, %4, %5, %6}], [%2], %7;" ::"r"(dst),
      "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "l"(policy)
      : "memory");
}
// Untiled bulk copy global -> shared memory of this CTA (both 16-byte aligned, size a
// multiple of 16 bytes), completion on an mbarrier of this CTA.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes,
                                          uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// tcgen05: tensor memory management, MMA issue, completion, loads.
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result_addr, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_result_addr),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, BF16 inputs, FP32 accumulate, issued by ONE thread.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on an mbarrier once all MMAs issued so far by this thread have completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns: thread l of the warp gets lane (base+l).
__device__ __forceinline__ void tmem_ld_16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor for a K-major BF16 operand tile whose rows are
// 128 bytes (64 elements) and were written by TMA with the 128-byte swizzle:
// 8-row x 128-byte atoms, consecutive atoms 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_smem_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);   // start address, bits [0,14)
  d |= (uint64_t)0 << 16;                         // leading byte offset (unused: one atom along K)
  d |= (uint64_t)(1024u >> 4) << 32;              // stride byte offset between 8-row atoms
  d |= (uint64_t)1 << 46;                         // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;                         // layout: 128-byte swizzle
  return d;
}
// 32-bit instruction descriptor: BF16 x BF16 -> FP32, both operands K-major, M=128.
__device__ __forceinline__ uint32_t umma_idesc_bf16_m128(uint32_t n) {
  return (1u << 4)             // accumulator format FP32
         | (1u << 7)           // A format BF16
         | (1u << 10)          // B format BF16
         | ((n >> 3) << 17)    // N / 8
         | ((128u >> 4) << 24);  // M / 16
}

// D[tmem] (+)= A[smem] * B[smem]^T with 8-bit floating-point inputs (formats in the
// instruction descriptor), FP32 accumulate, K = 32 per instruction, issued by ONE thread.
__device__ __forceinline__ void umma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Instruction descriptor: E4M3 x E4M3 -> FP32, both operands K-major, M=128.
__device__ __forceinline__ uint32_t umma_idesc_e4m3_m128(uint32_t n) {
  return (1u << 4)             // accumulator format FP32
         | (0u << 7)           // A format E4M3
         | (0u << 10)          // B format E4M3
         | ((n >> 3) << 17)    // N / 8
         | ((128u >> 4) << 24);  // M / 16
}

// Block-scaled FP4: D[tmem] (+)= (A * scale_a)[smem] * (B * scale_b)[smem]^T with E2M1
// elements, one unsigned-E4M3 scale per 16 elements along K held in tensor memory, FP32
// accumulate, K = 64 per instruction, issued by ONE thread.
__device__ __forceinline__ void umma_nvfp4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                           uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], "
      "p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
// Instruction descriptor of the block-scaled kinds: E2M1 x E2M1, both operands K-major,
// unsigned-E4M3 scales, M = 128, K = 64.
__device__ __forceinline__ uint32_t umma_idesc_nvfp4_m128(uint32_t n) {
  return (1u << 7)             // A format E2M1
         | (1u << 10)          // B format E2M1
         | ((n >> 3) << 17)    // N / 8
         | (0u << 23)          // scale format: unsigned E4M3
         | ((128u >> 4) << 24);  // M / 16
}
// Scale factors shared memory -> tensor memory: 32 rows of 16 bytes (one 128-row x 4-scale
// tile) land in 4 consecutive columns, lane l / column c holding the four scales of row
// c * 32 + l, replicated into all four lane quarters.
__device__ __forceinline__ void tmem_copy_scales(uint32_t dst_tmem, uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);   // start address
  d |= (uint64_t)(128u >> 4) << 32;               // 8-row x 16-byte atoms are 128 bytes apart
  d |= (uint64_t)1 << 46;                         // descriptor version; no swizzle
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(dst_tmem), "l"(d)
               : "memory");
}

// Four E4M3 bytes (K order k0..k3 from the low byte up) -> two packed BF16 pairs (k0,k1)
// and (k2,k3).  An E4M3 byte s.eeee.mmm placed at BF16 bits [15] and [10:4] reads as the
// same value times 2^-120 (a BF16 subnormal where the E4M3 exponent field is zero); one
// packed multiply by 2^120 restores it exactly.  Bytes 0x7F/0xFF (E4M3 NaN, never
// produced by the quantiser here) come out as +-480.
__device__ __forceinline__ void e4m3x4_to_bf16x4(uint32_t w, uint32_t& p01, uint32_t& p23) {
  const uint32_t y0 = __byte_perm(w, 0u, 0x1404);  // (b0 << 8) | (b1 << 24)
  const uint32_t y1 = __byte_perm(w, 0u, 0x3424);  // (b2 << 8) | (b3 << 24)
  const uint32_t r0 = (y0 & 0x80008000u) | ((y0 >> 4) & 0x07F007F0u);
  const uint32_t r1 = (y1 & 0x80008000u) | ((y1 >> 4) & 0x07F007F0u);
  const uint32_t two120 = 0x7B807B80u;             // BF16 2^120, twice
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(p01) : "r"(r0), "r"(two120));
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(p23) : "r"(r1), "r"(two120));
}

}  // namespace b200moe
