// Stages 3 and 4: the two grouped BF16 GEMMs, written for the decode regime
// where the expert weights are streamed from HBM once and the token count per
// expert is tiny.
//
// Operand roles are swapped relative to the textbook layout: the WEIGHT tile is
// the 128-row "A" operand of tcgen05.mma and the expert's token rows are the
// "N" dimension (16..128 columns of the accumulator).  Both operands are
// K-major in global memory already ([.., 2I, H], [.., H, I], [rows, H],
// [rows, I]), so TMA brings 64-element (128-byte) K slices straight into the
// 128-byte-swizzled shared-memory layout the MMA reads; nothing is transposed.
// Accumulator element (lane m, column j) = weight row m . token row j.
//
// One thread block = one work unit = (segment, 128-row weight tile[, K split]).
// Units are decoded from the schedule the routing kernel left in device memory;
// blocks whose unit does not exist return at once, so the host launches a grid
// sized for the worst case without ever reading the routing result back.  Two
// blocks fit on an SM (<= 109 KB of pipeline stages and <= 256 TMEM columns
// each), which keeps ~200 KB of TMA loads in flight per SM.
//
// Warp roles (192 threads): warp 0 = TMA producer (one lane), warp 1 = TMEM
// allocation + MMA issue (one lane), warps 2..5 = epilogue (each owns the 32
// TMEM lanes its warp id modulo 4 selects).
//
// gate+up (stage 3): each pipeline stage holds a 128-row gate tile and the
// matching 128-row up tile (one 4-D TMA box over [E][2][I][H]) plus the token
// rows; two accumulators (gate, up) share the token operand, so the epilogue
// computes silu(g) * u in FP32 thread-locally and stores it as a BF16 high
// part plus a BF16 low-order remainder.
//
// down (stage 4): each stage holds one 128-row weight tile and the high and low
// activation rows, one after the other; one MMA per K step over both computes
// W . hi and W . lo into two accumulators.  The epilogue adds them and stores FP32
// rows into this block's split-K slice.
//
// A call with at most 32 assignments runs in "small-call" order: gate+up is the
// first kernel of the forward, its blocks derive their unit from the expert ids
// and fetch their token rows from hidden_states themselves, and the routing
// kernel runs beside it.
#include "common.cuh"

namespace b200moe {

constexpr int kGemmThreads = 192;
constexpr int kMaxStages = 8;
constexpr uint32_t kMaxStageBudget = 220u * 1024u;        // one block per SM
constexpr int kTileM = 128;   // weight rows per unit
constexpr int kTileK = 64;    // elements per pipeline stage along K (128 bytes)
constexpr uint64_t kAbortDrainNs = 1000000ull;
constexpr uint64_t kHandoverWaitNs = 200000000ull;   // a down block's wait for its segment's rows

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// orders earlier generic-proxy accesses (here: other blocks' stores, acquired through a
// flag) before this thread's later async-proxy accesses (TMA loads from global memory)
__device__ __forceinline__ void fence_proxy_async_global() {
  asm volatile("fence.proxy.async;" ::: "memory");
}

struct GemmParams {
  const int32_t* sched;
  uint32_t* status;
  __nv_bfloat16* act_hi;   // gate+up output [rows_cap, I]
  __nv_bfloat16* act_lo;   // gate+up output [rows_cap, I]
  float* partials;         // down output [splits][rows_cap][H]
  int m_total;             // weight rows per expert matrix: I (gate+up) or H (down)
  int k_total;             // reduction length: H (gate+up) or I (down)
  int m_tiles;             // ceil(m_total / 128)
  int rows_cap;
  int sched_cap;           // segment entries the schedule array holds
  // Regular order inside one forward: gate+up blocks count their finished tiles per segment
  // in the schedule entry's fourth word, and a down block waits for its own segment's count
  // instead of the whole gate+up grid (see "segment hand-over" below).
  int overlap;
  // small calls (<= kSmallCallMaxAssign assignments): every block derives its unit from
  // the call's expert ids and does not read the schedule before its dependency wait
  int small;
  const int64_t* ids;      // [num_assign]
  int num_assign, num_experts, id_base, top_k;
  int split_request;       // down: what the routing kernel is given to choose the split-K factor
  // small gate+up: blocks load their token rows from hidden_states themselves, and the
  // blocks of tile 0 also write them to permuted_hidden (the gather of this call)
  const uint4* hidden;
  uint4* permuted_hidden;
  int hidden_vecs;         // H / 8
  unsigned long long* trace;
  uint32_t stage_budget;   // bytes of shared memory the stage ring may use
  int evict_first;         // stream the weight tiles with an L2 evict-first hint
};

template <bool kGateUp>
__global__ void __launch_bounds__(kGemmThreads, 2)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ CUtensorMap map_b0,
                    const __grid_constant__ CUtensorMap map_b1, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t s_full[kMaxStages];
  __shared__ __align__(8) uint64_t s_empty[kMaxStages];
  __shared__ __align__(8) uint64_t s_acc;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  __shared__ int s_tokens[kSmallCallMaxAssign];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // Prologue that does not depend on earlier kernels.
  if (threadIdx.x == 0) {
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(smem_u32(&s_full[s]), 1);
      mbar_init(smem_u32(&s_empty[s]), 1);
    }
    mbar_init(smem_u32(&s_acc), 1);
    s_abort = 0;
    fence_mbar_init();
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_b0);
    prefetch_tensormap(&map_b1);
  }
  __syncthreads();  // s_abort and the barriers are initialised before any thread uses them

  // ---- find this block's unit --------------------------------------------------
  // Regular order (routing, gather, gate+up, down, combine): the schedule is final before
  // either GEMM grid can start -- gather lets gate+up start only after its own wait for
  // the routing kernel, and down starts after every gate+up block has passed its wait --
  // so blocks read it first and prefetch weight tiles before their own dependency wait.
  //
  // Small-call order (gate+up, routing, down, combine): gate+up is the first kernel of the
  // forward and needs nothing from the routing kernel, which runs beside it.  Its blocks
  // wait for whatever preceded the forward (the inputs are then final and the previous
  // forward has released the activation buffers), derive their unit from the expert ids
  // held in one warp, and fetch their token rows from hidden_states themselves.  The
  // routing kernel leaves only after gate+up has completed, so that the completion of
  // routing, which is what down waits for, implies both.  Down blocks derive their unit
  // the same way (the ids are inputs of the call, nothing an earlier kernel of this
  // forward writes), prefetch weights, wait, and then compare with the schedule.
  int unit = blockIdx.x;
  int split = 0, n_split = 1;
  int expert = 0, row_start = 0, n_rows = 0;
  const int tiles = p.m_tiles;
  unsigned members = 0u;
  const int kblocks = (p.k_total + kTileK - 1) / kTileK;
  if (p.small) {
    if (kGateUp) {
      pdl_wait();
      pdl_launch_dependents();  // the routing kernel may start now
    }
    const SmallRouteLane route = small_route_scan(p.ids, p.num_assign, p.num_experts, p.id_base);
    if (!kGateUp) {
      n_split = down_splits_for(route.n_seg, route.n_valid, p.m_tiles, kblocks, p.split_request);
      split = unit % n_split;
      unit /= n_split;
    }
    if (!small_route_pick(route, unit / tiles, expert, row_start, n_rows, members)) {
      // No such unit in this call.  A down block still leaves only after its dependency
      // is resolved: the combine kernel waits for this grid alone and reads what the
      // routing kernel wrote.
      if (!kGateUp) pdl_wait();
      return;
    }
    if (kGateUp && warp == 0 && ((members >> lane) & 1u))
      s_tokens[__popc(members & ((1u << lane) - 1u))] = lane / p.top_k;
  } else {
    // header {segments, active, valid rows, splits} and the segment entry are 16 bytes
    // each; gate+up knows its segment index without the header, so both loads go out
    // together (the index is clamped to the array and checked against the count after).
    const int4 header = *reinterpret_cast<const int4*>(p.sched);
    const int n_seg = header.x;
    if (!kGateUp) {
      n_split = header.w;
      split = unit % n_split;
      unit /= n_split;
    }
    const int seg = unit / tiles;
    const int4 entry = *reinterpret_cast<const int4*>(
        p.sched + kSchedHeaderWords + kSchedSegWords * min(seg, p.sched_cap - 1));
    if (seg >= n_seg) return;
    expert = entry.x;
    row_start = entry.y;
    n_rows = entry.z;
  }
  const int tile = unit % tiles;
  const int n_mma = (n_rows + 15) & ~15;  // accumulator columns: 16..128
  trace_start(p.trace, kGateUp ? kTraceGateUp : kTraceDown);
  const bool direct = kGateUp && p.small != 0;  // token rows come straight from hidden_states

  int kb0 = 0, num_kb = kblocks;
  if (!kGateUp) {
    const int per = kblocks / n_split, rem = kblocks % n_split;
    kb0 = split * per + min(split, rem);
    num_kb = per + (split < rem ? 1 : 0);
  }

  // ---- shared-memory pipeline geometry ---------------------------------------
  constexpr uint32_t a_bytes = kGateUp ? 2u * kTileM * 128u : kTileM * 128u;
  const uint32_t b_bytes = (uint32_t)n_mma * 128u * (kGateUp ? 1u : 2u);
  const uint32_t stage_bytes = a_bytes + b_bytes;
  // bytes one stage receives: row-by-row loads bring only the real rows
  const uint32_t stage_tx = direct ? a_bytes + (uint32_t)n_rows * 128u : stage_bytes;
  const int num_stages = min((int)(p.stage_budget / stage_bytes), kMaxStages);
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

  const uint64_t weight_policy = p.evict_first ? l2_policy_evict_first() : 0ull;
  auto load_weights = [&](uint32_t dst, uint32_t bar, int kc) {
    if (kGateUp) {
      // one box over [E][2][I][H]: the gate rows of the tile, then the matching up rows
      if (p.evict_first) tma_load_4d_hint(dst, &map_w, bar, kc, tile * kTileM, 0, expert, weight_policy);
      else tma_load_4d(dst, &map_w, bar, kc, tile * kTileM, 0, expert);
    } else {
      if (p.evict_first) tma_load_3d_hint(dst, &map_w, bar, kc, tile * kTileM, expert, weight_policy);
      else tma_load_3d(dst, &map_w, bar, kc, tile * kTileM, expert);
    }
  };

  auto load_tokens = [&](uint32_t b_dst, uint32_t bar, int kc) {
    if (direct) {
      // map_b1 describes hidden_states [T, H] with one-row boxes
      for (int r = 0; r < n_rows; ++r)
        tma_load_2d(b_dst + (uint32_t)r * 128u, &map_b1, bar, kc, s_tokens[r]);
    } else {
      for (int r = 0; r < n_mma; r += 16) {
        tma_load_2d(b_dst + (uint32_t)r * 128u, &map_b0, bar, kc, row_start + r);
        if (!kGateUp)
          tma_load_2d(b_dst + (uint32_t)(n_mma + r) * 128u, &map_b1, bar, kc, row_start + r);
      }
    }
  };

  // ---- weight prefetch: fill the first stages' weight tiles while the previous
  // kernel is still finishing; the token rows of those stages follow after the wait
  // (a small-call gate+up block has waited already and loads both at once).
  const int prefetched = min(num_stages, num_kb);
  if (warp == 0) {
    __syncwarp();  // s_tokens, written by this warp
    if (lane == 0) {
      for (int i = 0; i < prefetched; ++i) {
        const uint32_t bar = smem_u32(&s_full[i]);
        const uint32_t a_dst = smem_base + (uint32_t)i * stage_bytes;
        const int kc = (kb0 + i) * kTileK;
        mbar_expect_tx(bar, stage_tx);
        load_weights(a_dst, bar, kc);
        if (direct) load_tokens(a_dst + a_bytes, bar, kc);
      }
    }
  }

  // ---- tensor memory (allocated before the dependency wait: one step less between the
  // wait's return and the first token load) ----------------------------------------
  const uint32_t cols_needed = (uint32_t)n_mma * 2u;  // gate and up, or high and low halves
  uint32_t tmem_cols = 32;
  while (tmem_cols < cols_needed) tmem_cols <<= 1;
  if (warp == 1) {
    tmem_alloc(smem_u32(&s_tmem_base), tmem_cols);
    tmem_relinquish();
  }

  // ---- the dependency wait ------------------------------------------------------
  // Segment hand-over (regular order, p.overlap): a down block does not wait for the whole
  // gate+up grid.  This grid is launched once every gate+up block has started (each
  // executes launch_dependents right after its own wait), i.e. into the slots that free up
  // during gate+up's last, partial wave; the blocks of early segments, whose activations are
  // complete by then, stream their weights under that tail instead of idling until the
  // last gate+up block has finished.  Only the thread that loads activations waits, on its
  // segment's tile count (bounded).  No deadlock is possible even without the bound: every
  // gate+up block is resident or finished before the first down block exists.
  const bool handover = !kGateUp && p.overlap != 0 && p.small == 0;
  if (handover) {
    pdl_launch_dependents();
  } else if (!(kGateUp && p.small)) {
    pdl_wait();
    pdl_launch_dependents();
  }

  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = s_tmem_base;
  volatile int* abort_flag = &s_abort;

  if (warp == 0) {
    // ===== TMA producer =====
    if (lane == 0) {
      bool rows_ready = true;
      if (handover) {
        // all gate+up tiles of this segment have stored their activations: acquire the
        // count, then order those generic-proxy writes before this thread's TMA reads
        const int* done = p.sched + kSchedHeaderWords + kSchedSegWords * (unit / tiles) + 3;
        const int need = (p.k_total + kTileM - 1) / kTileM;   // gate+up tiles = ceil(I / 128)
        const uint64_t t0 = global_timer_ns();
        while (ld_acquire_gpu(done) < need) {
          if (*abort_flag || global_timer_ns() - t0 > kHandoverWaitNs) {
            rows_ready = false;
            *abort_flag = 1;
            break;
          }
        }
        fence_proxy_async_global();
      }
      for (int i = 0; rows_ready && i < num_kb; ++i) {
        const int s = i % num_stages;
        const uint32_t round = (uint32_t)(i / num_stages);
        if (i >= num_stages &&
            !mbar_wait_bounded(smem_u32(&s_empty[s]), (round - 1u) & 1u, abort_flag))
          break;
        const uint32_t bar = smem_u32(&s_full[s]);
        const uint32_t a_dst = smem_base + (uint32_t)s * stage_bytes;
        const uint32_t b_dst = a_dst + a_bytes;
        const int kc = (kb0 + i) * kTileK;
        if (i >= prefetched) {
          mbar_expect_tx(bar, stage_tx);
          load_weights(a_dst, bar, kc);
        }
        if (i >= prefetched || !direct) load_tokens(b_dst, bar, kc);
      }
    }
  } else if (warp == 1) {
    // ===== MMA issuer =====
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16_m128((uint32_t)n_mma);
      const uint32_t idesc_down = umma_idesc_bf16_m128((uint32_t)(2 * n_mma));
      bool ok = true;
      for (int i = 0; i < num_kb; ++i) {
        const int s = i % num_stages;
        const uint32_t round = (uint32_t)(i / num_stages);
        if (!mbar_wait_bounded(smem_u32(&s_full[s]), round & 1u, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        if (i == 0 && p.trace && blockIdx.x == 0)
          p.trace[2 * (kGateUp ? kTraceGateUpFirstData : kTraceDownFirstData)] = global_timer_ns();
        const uint32_t a_addr = smem_base + (uint32_t)s * stage_bytes;
        const uint32_t b_addr = a_addr + a_bytes;
        const uint64_t a0 = umma_smem_desc_sw128(a_addr);
        const uint64_t b0 = umma_smem_desc_sw128(b_addr);
        if (kGateUp) {
          const uint64_t a1 = umma_smem_desc_sw128(a_addr + kTileM * 128u);  // up tile
#pragma unroll
          for (int k = 0; k < kTileK / 16; ++k) {
            const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
            // advancing 16 BF16 elements along K = 32 bytes = 2 descriptor units
            umma_bf16(tmem, a0 + 2u * k, b0 + 2u * k, idesc, acc);
            umma_bf16(tmem + (uint32_t)n_mma, a1 + 2u * k, b0 + 2u * k, idesc, acc);
          }
        } else {
          // The low halves follow the high halves in the stage: one K-major operand of
          // 2 * n_mma rows, so a single MMA per K step fills both accumulators (columns
          // [0, n_mma) from the high halves, [n_mma, 2 n_mma) from the low ones).
#pragma unroll
          for (int k = 0; k < kTileK / 16; ++k) {
            const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
            umma_bf16(tmem, a0 + 2u * k, b0 + 2u * k, idesc_down, acc);
          }
        }
        umma_commit(smem_u32(&s_empty[s]));  // frees the stage once these MMAs have read it
      }
      if (ok && num_kb > 0) umma_commit(smem_u32(&s_acc));  // accumulators complete
    }
  } else {
    // ===== epilogue warps =====
    const int quarter = warp & 3;
    // Small call: this forward has no gather kernel; the blocks of tile 0 copy their rows
    // to permuted_hidden while the main loop runs (16-byte loads and stores).
    if (direct && tile == 0 && p.permuted_hidden != nullptr) {
      const int t = (int)threadIdx.x - 64;
      for (int r = 0; r < n_rows; ++r) {
        const uint4* src = p.hidden + (size_t)s_tokens[r] * p.hidden_vecs;
        uint4* dst = p.permuted_hidden + (size_t)(row_start + r) * p.hidden_vecs;
        for (int v = t; v < p.hidden_vecs; v += 128) dst[v] = __ldg(src + v);
      }
    }
    // Small-call down: the routing kernel's schedule is authoritative; a block whose own
    // derivation disagreed with it would have streamed the wrong tiles (never observed;
    // reported, and the block then writes nothing).  Checked here, by the warps that idle
    // during the main loop, so that the two loads do not stand between the dependency wait
    // and the producer's first token loads.
    bool unit_agrees = true;
    if (!kGateUp && p.small) {
      const int4 header = *reinterpret_cast<const int4*>(p.sched);
      const int4 entry = *reinterpret_cast<const int4*>(
          p.sched + kSchedHeaderWords + kSchedSegWords * min(unit / tiles, p.sched_cap - 1));
      unit_agrees = header.w == n_split && entry.x == expert && entry.y == row_start &&
                    entry.z == n_rows;
      if (!unit_agrees) *abort_flag = 1;
    }
    // ----- TMEM -> registers -> global -----
    bool have_acc = num_kb > 0;
    if (have_acc) have_acc = mbar_wait_bounded(smem_u32(&s_acc), 0u, abort_flag);
    have_acc = have_acc && unit_agrees;
    have_acc = __all_sync(0xffffffffu, have_acc);  // tcgen05.ld needs the whole warp
    if ((have_acc || num_kb == 0) && unit_agrees) {
      // A block that gave up writes nothing; the status word reports it.
      const int m = tile * kTileM + quarter * 32 + lane;  // weight row of this thread
      const bool m_ok = m < p.m_total;
      tc_fence_after_sync();
      const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
      for (int c0 = 0; c0 < n_mma; c0 += 16) {
        uint32_t g[16], u[16];
        if (num_kb > 0) {
          tmem_ld_16(lane_base + (uint32_t)c0, g);
          tmem_ld_16(lane_base + (uint32_t)(n_mma + c0), u);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) g[j] = u[j] = 0u;
        }
        if (kGateUp) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (m_ok && c0 + j < n_rows) {
              const float gate = __uint_as_float(g[j]);
              const float up = __uint_as_float(u[j]);
              const float act = gate / (1.0f + __expf(-gate)) * up;
              const __nv_bfloat16 hi = __float2bfloat16_rn(act);
              const __nv_bfloat16 lo = __float2bfloat16_rn(act - __bfloat162float(hi));
              const size_t o = (size_t)(row_start + c0 + j) * p.m_total + m;
              p.act_hi[o] = hi;
              p.act_lo[o] = lo;
            }
          }
        } else {
          float* dst = p.partials + (size_t)split * p.rows_cap * p.m_total;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (m_ok && c0 + j < n_rows)
              dst[(size_t)(row_start + c0 + j) * p.m_total + m] =
                  __uint_as_float(g[j]) + __uint_as_float(u[j]);  // W.hi + W.lo
          }
        }
      }
    }
  }

  // ---- teardown -----------------------------------------------------------------
  __syncwarp();
  if (*abort_flag) {
    // Some wait ran out.  Give copies and MMAs still in flight time to land
    // before shared and tensor memory are released.
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < kAbortDrainNs) {
    }
  }
  // segment hand-over: every thread's activation stores are ordered before the count
  if (kGateUp && p.overlap != 0 && p.small == 0 && warp >= 2) __threadfence();
  tc_fence_before_sync();
  __syncthreads();
  if (kGateUp && p.overlap != 0 && p.small == 0 && threadIdx.x == 0 && !*abort_flag) {
    // release: the other threads' stores happen before this fence through the barrier
    __threadfence();
    atomicAdd(const_cast<int*>(p.sched) + kSchedHeaderWords + kSchedSegWords * (unit / tiles) + 3, 1);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicOr(p.status, B200MOE_STATUS_PIPE_TIMEOUT);
  trace_end(p.trace, kGateUp ? kTraceGateUp : kTraceDown);
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem, tmem_cols);
  }
}

// Tuning knobs (b200moe_tune): process-wide, meant for benchmarking sweeps.
int g_gemm_stage_kb = 108;
int g_gemm_evict_first = 0;
// Shared memory of one block's stage ring.  Normally two blocks share an SM.  A grid that
// cannot put more than one block on an SM anyway (`grid <= sm_count`, known on the host from
// the worst-case unit count) gets the whole SM per block: with so few blocks the bytes in
// flight, not HBM, bound the stream, and a ring twice as deep doubles them.
constexpr uint32_t kLoneBlockStageBudget = 216u * 1024u;
static uint32_t gemm_stage_budget(int grid, int sm_count) {
  uint32_t b = (uint32_t)g_gemm_stage_kb * 1024u;
  if (g_gemm_stage_kb == 108 && sm_count > 0 && grid <= sm_count) b = kLoneBlockStageBudget;
  if (b < 48u * 1024u) b = 48u * 1024u;
  if (b > kMaxStageBudget) b = kMaxStageBudget;
  return b;
}

template <bool kGateUp>
static cudaError_t launch_gemm(const CUtensorMap& map_w, const CUtensorMap& map_b0,
                               const CUtensorMap& map_b1, const GemmParams& params, int grid,
                               bool pdl, cudaStream_t stream) {
  static bool attr_set[64] = {};
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= 64 || !attr_set[dev]) {
    err = cudaFuncSetAttribute(grouped_gemm_kernel<kGateUp>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)(kMaxStageBudget + 1024u));
    if (err != cudaSuccess) return err;
    if (dev >= 0 && dev < 64) attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = params.stage_budget + 1024u;  // + slack to align to 1024
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, grouped_gemm_kernel<kGateUp>, map_w, map_b0, map_b1, params);
}

cudaError_t launch_gate_up(const CUtensorMap& map_w, const CUtensorMap& map_x,
                           const CUtensorMap* map_hidden, const int32_t* sched, int sched_cap,
                           uint32_t* status, void* act_hi, void* act_lo, int inter, int hidden,
                           int rows_cap, int grid, const SmallCall* small, int overlap,
                           int sm_count, bool pdl, cudaStream_t stream) {
  GemmParams p = {};
  p.overlap = overlap;
  if (small != nullptr && map_hidden != nullptr) {
    p.small = 1;
    p.ids = small->ids;
    p.num_assign = small->num_assign;
    p.num_experts = small->num_experts;
    p.id_base = small->id_base;
    p.top_k = small->top_k;
    p.hidden = static_cast<const uint4*>(small->hidden);
    p.permuted_hidden = static_cast<uint4*>(small->permuted_hidden);
    p.hidden_vecs = hidden / 8;
  }
  p.trace = reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(status) +
                                                  kTraceOffsetBytes);
  p.stage_budget = gemm_stage_budget(grid, sm_count);
  p.evict_first = g_gemm_evict_first;
  p.sched = sched;
  p.sched_cap = sched_cap;
  p.status = status;
  p.act_hi = static_cast<__nv_bfloat16*>(act_hi);
  p.act_lo = static_cast<__nv_bfloat16*>(act_lo);
  p.partials = nullptr;
  p.m_total = inter;
  p.k_total = hidden;
  p.m_tiles = (inter + kTileM - 1) / kTileM;
  p.rows_cap = rows_cap;
  return launch_gemm<true>(map_w, map_x, p.small ? *map_hidden : map_x, p, grid, pdl, stream);
}

cudaError_t launch_down(const CUtensorMap& map_w, const CUtensorMap& map_hi,
                        const CUtensorMap& map_lo, const int32_t* sched, int sched_cap,
                        uint32_t* status, float* partials, int hidden, int inter, int rows_cap,
                        int grid, const SmallCall* small, int overlap, int sm_count, bool pdl,
                        cudaStream_t stream) {
  GemmParams p = {};
  p.overlap = overlap;
  if (small != nullptr) {
    p.small = 1;
    p.ids = small->ids;
    p.num_assign = small->num_assign;
    p.num_experts = small->num_experts;
    p.id_base = small->id_base;
    p.top_k = small->top_k;
    p.split_request = small->split_request;
  }
  p.stage_budget = gemm_stage_budget(grid, sm_count);
  p.evict_first = g_gemm_evict_first;
  p.trace = reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(status) +
                                                  kTraceOffsetBytes);
  p.sched = sched;
  p.sched_cap = sched_cap;
  p.status = status;
  p.act_hi = nullptr;
  p.act_lo = nullptr;
  p.partials = partials;
  p.m_total = hidden;
  p.k_total = inter;
  p.m_tiles = (hidden + kTileM - 1) / kTileM;
  p.rows_cap = rows_cap;
  return launch_gemm<false>(map_w, map_hi, map_lo, p, grid, pdl, stream);
}

}  // namespace b200moe
