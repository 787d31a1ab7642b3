// Stages 3 and 4 with NVFP4 expert weights, on the block-scaled tensor-core kind
// tcgen05.mma kind::mxf4nvf4 (E2M1 elements, one unsigned-E4M3 scale per 16 elements of K
// applied inside the instruction, FP32 accumulate).
//
// No counterpart in the reference: its NVFP4 backend always fails
// (csrc/quantization_kernels.cu:7-13, fastpath/b300_moe.py:571-596).  Expert weights are
// 0.5625 bytes per element (packed E2M1 + scales) instead of 2: the weight stream that
// bounds decode shrinks 3.5x.
//
// The instruction wants E2M1 on both sides, so -- as in the FP8-weight kernels -- the small
// operand is what gets converted: every token row is held as four E2M1 planes in fixed
// point, x ~= t * (e0 + e1 / 8 + e2 / 64 + e3 / 512) (nvfp4_quant.cu).  The planes of a step
// lie one after another in shared memory, so Q consecutive planes form one K-major operand of
// Q x rows rows: one MMA of N = Q x rows fills Q accumulators at once, and the remaining
// planes accumulate into the same columns with further MMAs.  The scale of a plane
// (8, 1, 1/8, 1/64; the epilogue multiplies by t / 8) is the same for every block of K, so
// the token operand's scale factors are constants: their tiles are written to tensor memory
// once, before the main loop.  The epilogue adds the Q accumulators and applies t and the
// weight tensor's FP32 scale.
//
// What bounds this kernel is not arithmetic but the number of tensor-core instructions:
// measured on a B200, one block-scaled MMA of N <= 64 holds the issuing thread ~56 ns and
// one scale copy to tensor memory ~37 ns, against ~90 ns that the 4 KB of weights one MMA
// consumes take to arrive at a block's share of HBM.  Hence: as many planes per MMA as
// tensor memory allows (N up to 128), and no per-stage token-scale copies at all.
//
// Weight scales are stored pre-arranged in 512-byte tiles (128 rows x 4 scales) and reach
// shared memory with one bulk copy per step; the issuing thread copies every tile to tensor
// memory (tcgen05.cp) right before the MMAs that use it, into one of two column sets that
// alternate, so the copies of one step run under the MMAs of the one before; copies and MMAs
// of one thread execute in issue order.
//
// Two rings in shared memory.  A weight slot holds one 128-row tile over 256 elements of K
// (16 KB) and its scales (2 KB); the gate tile and the up tile of a step are separate slots,
// so the ring is cut finely: five slots = 90 KB of weights in flight per block, two blocks
// per SM.  A token slot holds the planes of a step (4 x rows x 128 bytes) and serves both
// tiles of the step.  Same structure as the other GEMM kernels otherwise: one block =
// (segment of <= 64 rows, 128-row weight tile[, K split]); warp 0 = TMA producer, warp 1 =
// TMEM allocation + MMA issue, warps 2..5 = epilogue, warp 6 = second MMA issuer; every wait
// bounded.
#include "common.cuh"

namespace b200moe {

constexpr int kFThreads = 224;                     // warp 6: second MMA issuer of gate+up
constexpr int kFStageK = 256;                      // E2M1 elements per step along K
constexpr int kFTileM = 128;
constexpr int kFMaxSlots = 8;
constexpr uint32_t kFTileBytes = kFTileM * 128u;   // one weight tile of a step: 16 KB
constexpr uint32_t kFSfTile = 512u;                // scales of 128 rows x 64 elements of K
constexpr uint32_t kFSfaBytes = 4u * kFSfTile;     // one weight tile's scales of a step
constexpr uint32_t kFSlotBytes = kFTileBytes + kFSfaBytes;
// planes one MMA covers for a segment of n_mma (16, 32, 48 or 64) accumulator columns:
// gate+up keeps two accumulator sets (N <= 64 each), down one (N <= 128)
__host__ __device__ inline int nvfp4_planes_per_mma(int n_mma, bool gate_up) {
  if (gate_up) return n_mma <= 16 ? 4 : (n_mma <= 32 ? 2 : 1);
  return n_mma <= 32 ? 4 : 2;
}
// unsigned-E4M3 codes of the plane scales 8, 1, 1/8, 1/64
__device__ __forceinline__ uint32_t nvfp4_plane_scale_code(int plane) {
  return 0x50u - 0x18u * (uint32_t)plane;
}
constexpr uint64_t kFAbortDrainNs = 1000000ull;

// Development aid, compiled out of the product: with -DB200MOE_STAGE_TRACE block 0 of each
// kernel stamps (%globaltimer) when every ring slot became free (event 0), its weights (1)
// and token planes (2) had landed and its MMAs were issued (3), when the accumulators were
// complete (6, 0), the epilogue done (6, 4) and the block finished (6, 1); (7, 0..1) are the
// block's start and its return from the wait for the previous kernel.
// b200moe_debug_stage_trace() copies the stamps out.  The instruction costs quoted at the
// top of this file were measured this way.
#ifdef B200MOE_STAGE_TRACE
constexpr int kStageTraceEvents = 8, kStageTraceSlots = 64;
__device__ unsigned long long g_stage_trace[2][kStageTraceEvents][kStageTraceSlots];
#define STAGE_STAMP(event, i)                                                          \
  do {                                                                                 \
    if (blockIdx.x == 0 && (i) < kStageTraceSlots)                                     \
      g_stage_trace[kGateUp ? 1 : 0][event][i] = global_timer_ns();                    \
  } while (0)
#else
#define STAGE_STAMP(event, i) do { } while (0)
#endif

struct FGemmParams {
  const int32_t* sched;
  uint32_t* status;
  __nv_bfloat16* act_hi;      // gate+up output [rows_cap, I]
  __nv_bfloat16* act_lo;
  float* tile_amax;           // gate+up output [rows_cap][m_tiles]: max |act| of the row in the tile
  float* partials;            // down output [splits][rows_cap][H]
  const uint8_t* sfa;         // weight scales, 512-byte tiles: [E][(2)][m_tiles][k_tiles]
  const float* tensor_scale;  // [E]
  const float* token_scale;   // [rows_cap]: the rows' power-of-two scales t
  int m_total;                // I (gate+up) or H (down)
  int k_total;                // H (gate+up) or I (down)
  int m_tiles;
  int rows_cap;
  int sched_cap;
  unsigned long long* trace;
  uint32_t stage_budget;
  int prefetch_slots;         // weight slots filled before the wait for the previous kernel
  int issuers;                // gate+up: 1 = one thread issues both tiles' MMAs, 2 = one each
};

__device__ __forceinline__ void epilogue_warps_sync() {
  asm volatile("bar.sync 1, 128;" ::: "memory");
}

template <bool kGateUp>
__global__ void __launch_bounds__(kFThreads, 2)
grouped_gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap map_w,
                          const __grid_constant__ CUtensorMap map_b, const FGemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t s_a_full[kFMaxSlots];    // a weight tile and its scales
  __shared__ __align__(8) uint64_t s_a_empty[kFMaxSlots];
  __shared__ __align__(8) uint64_t s_b_full[kFMaxSlots];    // the token planes of a step
  __shared__ __align__(8) uint64_t s_b_empty[kFMaxSlots];
  __shared__ __align__(8) uint64_t s_acc;
  __shared__ __align__(8) uint64_t s_sfb_ready;             // token-scale tiles are in tensor memory
  __shared__ __align__(16) uint8_t s_sfb[4 * kFSfTile];     // the constant token-scale tiles
  __shared__ float s_token_scale[kSegRowsNvfp4];
  __shared__ float s_row_max[4][kSegRowsNvfp4];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // ---- this block's unit (the schedule is final before this grid can start) ----------
  int unit = blockIdx.x;
  int split = 0, n_split = 1;
  const int4 header = *reinterpret_cast<const int4*>(p.sched);
  const int n_seg = header.x;
  if (!kGateUp) {
    n_split = header.w;
    split = unit % n_split;
    unit /= n_split;
  }
  const int seg = unit / p.m_tiles;
  const int4 entry = *reinterpret_cast<const int4*>(
      p.sched + kSchedHeaderWords + kSchedSegWords * min(seg, p.sched_cap - 1));
  if (seg >= n_seg) return;
  const int expert = entry.x;
  const int row_start = entry.y;
  const int n_rows = entry.z;
  const int tile = unit % p.m_tiles;
  const int n_mma = (n_rows + 15) & ~15;   // accumulator columns per plane: 16..64
  trace_start(p.trace, kGateUp ? kTraceGateUp : kTraceDown);
  if (threadIdx.x == 0) STAGE_STAMP(7, 0);

  // Two issuing threads (warps 1 and 6): issuing one block-scaled MMA holds a thread for
  // longer than the tensor core works on it, so two threads with separate accumulators issue
  // in parallel.  gate+up: one thread per weight tile (gate, up) of every step.  down: the
  // threads take alternate steps into two accumulator sets that the epilogue adds -- for
  // segments of at most 32 rows, with two sets of 64 columns (32 rows: two planes per MMA
  // and two passes instead of four planes in one).
  const int issuers = p.issuers == 2 && (kGateUp || n_mma <= 32) ? 2 : 1;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kFMaxSlots; ++s) {
      mbar_init(smem_u32(&s_a_full[s]), 1);
      mbar_init(smem_u32(&s_a_empty[s]), 1);
      mbar_init(smem_u32(&s_b_full[s]), 1);
      // gate+up: both issuers read a step's token planes; down: the step's own issuer does
      mbar_init(smem_u32(&s_b_empty[s]), kGateUp ? (uint32_t)issuers : 1u);
    }
    mbar_init(smem_u32(&s_acc), (uint32_t)issuers);
    mbar_init(smem_u32(&s_sfb_ready), 1);
    s_abort = 0;
    fence_mbar_init();
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_b);
  }
  __syncthreads();

  const int kblocks = (p.k_total + kFStageK - 1) / kFStageK;
  const int k_tiles = (p.k_total + 63) / 64;   // scale tiles along K
  int kb0 = 0, num_kb = kblocks;
  if (!kGateUp) {
    const int per = kblocks / n_split, rem = kblocks % n_split;
    kb0 = split * per + min(split, rem);
    num_kb = per + (split < rem ? 1 : 0);
  }

  // ---- shared memory: the weight ring, then the token ring -------------------------------
  constexpr int kSets = kGateUp ? 2 : 1;   // gate and up tiles, or the one down tile
  const uint32_t plane_bytes = (uint32_t)n_mma * 128u;
  const uint32_t b_bytes = kNvfp4Planes * plane_bytes;
  const int q_planes = (!kGateUp && issuers == 2 && n_mma == 32)
                           ? 2
                           : nvfp4_planes_per_mma(n_mma, kGateUp);   // planes per MMA
  const int passes = kNvfp4Planes / q_planes;                  // MMAs per weight tile and 64 elements of K
  // gate+up: two token slots serve any number of weight slots; down: one token slot per step
  const int n_b = kGateUp ? 2 : min((int)(p.stage_budget / (kFSlotBytes + b_bytes)), kFMaxSlots);
  const int n_a = kGateUp ? min((int)((p.stage_budget - 2u * b_bytes) / kFSlotBytes), kFMaxSlots)
                          : n_b;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t b_base = smem_base + (uint32_t)n_a * kFSlotBytes;
  volatile int* abort_flag = &s_abort;
  if (n_a < 2 || n_b < 2 || n_mma > kSegRowsNvfp4) {
    // a schedule with segments longer than this kernel supports: a caller error; report
    if (threadIdx.x == 0) atomicOr(p.status, B200MOE_STATUS_PIPE_TIMEOUT);
    return;
  }
  const int num_h = kSets * num_kb;   // weight tiles this block consumes, in ring order

  // scale tiles of K the step that starts at element kc holds (the last step may be short)
  auto groups_at = [&](int kc) { return min(4, k_tiles - kc / 64); };
  auto a_tx = [&](int kc) { return kFTileBytes + (uint32_t)groups_at(kc) * kFSfTile; };
  auto load_weights = [&](uint32_t dst, uint32_t bar, int set, int kc) {
    // one box over [E][2][I][H / 2 bytes] (set 0 = gate rows, 1 = the matching up rows) or
    // over [E][H][I / 2 bytes]; coordinates of the innermost dimension are in bytes
    if (kGateUp) tma_load_4d(dst, &map_w, bar, kc / 2, tile * kFTileM, set, expert);
    else tma_load_3d(dst, &map_w, bar, kc / 2, tile * kFTileM, expert);
    const size_t tile_index =
        kGateUp ? ((size_t)(expert * 2 + set) * p.m_tiles + tile) : ((size_t)expert * p.m_tiles + tile);
    bulk_load(dst + kFTileBytes, p.sfa + (tile_index * k_tiles + kc / 64) * kFSfTile,
              (uint32_t)groups_at(kc) * kFSfTile, bar);
  };

  // Weight prefetch: fill the ring with weight tiles and scales while the previous kernel is
  // still finishing; the token planes follow after the wait.
  const int prefetched = min(min(n_a, num_h), p.prefetch_slots);
  if (threadIdx.x == 0) {
    for (int h = 0; h < prefetched; ++h) {
      const uint32_t bar = smem_u32(&s_a_full[h]);
      const int kc = (kb0 + h / kSets) * kFStageK;
      mbar_expect_tx(bar, a_tx(kc));
      load_weights(smem_base + (uint32_t)h * kFSlotBytes, bar, h % kSets, kc);
    }
  }

  // ---- tensor memory: accumulators, two sets of weight-scale columns, token scales -------
  const uint32_t set_cols = (uint32_t)(q_planes * n_mma);   // accumulator columns of one set
  const int acc_sets = kGateUp ? kSets : issuers;            // gate and up tiles, or one set per issuer
  const uint32_t acc_cols = (uint32_t)acc_sets * set_cols;
  constexpr uint32_t kSfaCols = 2u * 16u;                  // 4 tiles x 4 columns, twice
  const uint32_t sfb_cols = (uint32_t)passes * 4u;
  uint32_t tmem_cols = 32;
  while (tmem_cols < acc_cols + kSfaCols + sfb_cols) tmem_cols <<= 1;
  if (warp == 1) {
    tmem_alloc(smem_u32(&s_tmem_base), tmem_cols);
    tmem_relinquish();
  }
  float w_scale = 0.0f;
  if (warp >= 2 && warp < 6) {
    // Token-scale tiles, one per pass: row r = (plane % q_planes) * n_mma + n of the pass's
    // operand carries its plane's scale four times, at byte (r % 32) * 16 + (r / 32) * 4.
    const int r = (int)threadIdx.x - 64;   // 0..127
    for (int pass = 0; pass < passes; ++pass) {
      const uint32_t code =
          r < q_planes * n_mma ? nvfp4_plane_scale_code(pass * q_planes + r / n_mma) : 0u;
      *reinterpret_cast<uint32_t*>(s_sfb + pass * kFSfTile + (r & 31) * 16 + (r >> 5) * 4) =
          code * 0x01010101u;
    }
    if (r < kSegRowsNvfp4) {
#pragma unroll
      for (int q = 0; q < 4; ++q) s_row_max[q][r] = 0.0f;
    }
    w_scale = 0.125f * p.tensor_scale[expert];   // weights are the caller's: readable before the wait
  }
  pdl_wait();
  pdl_launch_dependents();
  if (threadIdx.x == 0) STAGE_STAMP(7, 1);
  // the tensor-memory copy reads the token-scale tiles through the async proxy
  if (warp >= 2 && warp < 6) fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp >= 2 && warp < 6) {
    // the rows' scales (written by the previous kernel) are only needed by the epilogue: they
    // are fetched here, under the main loop, and not in front of the barrier above, which
    // would keep the producer from requesting the token planes for the length of this load
    const int r = (int)threadIdx.x - 64;
    if (r < kSegRowsNvfp4) s_token_scale[r] = r < n_rows ? p.token_scale[row_start + r] : 0.0f;
  }
  const uint32_t tmem = s_tmem_base;
  const uint32_t tmem_sfa = tmem + acc_cols;
  const uint32_t tmem_sfb = tmem_sfa + kSfaCols;

  if (warp == 0) {
    // ===== TMA producer =====
    if (lane == 0) {
      for (int h = 0; h < num_h; ++h) {
        const int i = h / kSets, set = h % kSets;
        const int sa = h % n_a;
        const int kc = (kb0 + i) * kFStageK;
        if (h >= n_a &&
            !mbar_wait_bounded(smem_u32(&s_a_empty[sa]), (uint32_t)(h / n_a - 1) & 1u, abort_flag))
          break;
        STAGE_STAMP(0, h);
        if (h >= prefetched) {
          const uint32_t bar = smem_u32(&s_a_full[sa]);
          mbar_expect_tx(bar, a_tx(kc));
          load_weights(smem_base + (uint32_t)sa * kFSlotBytes, bar, set, kc);
        }
        if (set == 0) {
          const int sb = i % n_b;
          if (i >= n_b &&
              !mbar_wait_bounded(smem_u32(&s_b_empty[sb]), (uint32_t)(i / n_b - 1) & 1u, abort_flag))
            break;
          const uint32_t bar = smem_u32(&s_b_full[sb]);
          const uint32_t dst = b_base + (uint32_t)sb * b_bytes;
          mbar_expect_tx(bar, b_bytes);
          for (int pl = 0; pl < kNvfp4Planes; ++pl)
            for (int r = 0; r < n_mma; r += 16)
              tma_load_3d(dst + (uint32_t)pl * plane_bytes + (uint32_t)r * 128u, &map_b, bar,
                          kc / 2, row_start + r, pl);
        }
      }
    }
  } else if (warp == 1 || warp == 6) {
    // ===== scale copies + MMA issue =====
    const int me = warp == 1 ? 0 : 1;   // issuer 0: every tile, or the gate tiles; 1: the up tiles
    if (lane == 0 && me < issuers) {
      const uint32_t idesc = umma_idesc_nvfp4_m128(set_cols);
      bool ok = true;
      if (me == 0) {
        for (int pass = 0; pass < passes; ++pass)
          tmem_copy_scales(tmem_sfb + (uint32_t)(pass * 4), smem_u32(s_sfb) + (uint32_t)pass * kFSfTile);
        if (issuers == 2) umma_commit(smem_u32(&s_sfb_ready));
      } else {
        ok = mbar_wait_bounded(smem_u32(&s_sfb_ready), 0u, abort_flag);
        tc_fence_after_sync();
      }
      for (int h = me; h < num_h && ok; h += issuers) {
        const int i = h / kSets, set = h % kSets;
        const int sa = h % n_a, sb = i % n_b;
        if (!mbar_wait_bounded(smem_u32(&s_a_full[sa]), (uint32_t)(h / n_a) & 1u, abort_flag)) {
          ok = false;
          break;
        }
        STAGE_STAMP(1, h);
        // the token planes of the step: the thread that issues a step's first tile waits; a
        // second issuer has to see them as well before its own first read
        if ((set == 0 || issuers == 2) &&
            !mbar_wait_bounded(smem_u32(&s_b_full[sb]), (uint32_t)(i / n_b) & 1u, abort_flag)) {
          ok = false;
          break;
        }
        STAGE_STAMP(2, h);
        tc_fence_after_sync();
        if (h == 0 && p.trace && blockIdx.x == 0)
          p.trace[2 * (kGateUp ? kTraceGateUpFirstData : kTraceDownFirstData)] = global_timer_ns();
        const int groups = groups_at((kb0 + i) * kFStageK);
        const uint32_t a_addr = smem_base + (uint32_t)sa * kFSlotBytes;
        const uint32_t b_addr = b_base + (uint32_t)sb * b_bytes;
        const uint32_t sfa_t = tmem_sfa + (uint32_t)(h & 1) * 16u;
        for (int g = 0; g < groups; ++g)
          tmem_copy_scales(sfa_t + (uint32_t)(g * 4), a_addr + kFTileBytes + (uint32_t)g * kFSfTile);
        const uint64_t a_desc = umma_smem_desc_sw128(a_addr);
        const uint32_t d_tmem = tmem + (uint32_t)(kGateUp ? set : me) * set_cols;
        const bool first_step = kGateUp ? i == 0 : h < issuers;   // of this accumulator set
        for (int g = 0; g < groups; ++g) {
          for (int pass = 0; pass < passes; ++pass) {
            // the pass's q_planes planes are one operand of q_planes * n_mma rows;
            // 64 E2M1 elements along K = 32 bytes = 2 descriptor units
            const uint64_t b_desc =
                umma_smem_desc_sw128(b_addr + (uint32_t)(pass * q_planes) * plane_bytes) + 2u * g;
            umma_nvfp4(d_tmem, a_desc + 2u * g, b_desc, idesc, sfa_t + (uint32_t)(g * 4),
                       tmem_sfb + (uint32_t)(pass * 4), (!first_step || g > 0 || pass > 0) ? 1u : 0u);
          }
        }
        umma_commit(smem_u32(&s_a_empty[sa]));
        if (set == kSets - 1 || issuers == 2) umma_commit(smem_u32(&s_b_empty[sb]));
        STAGE_STAMP(3, h);
      }
      if (ok && num_kb > 0) {
        // an issuer that had no step of its own (a block with a single step) has nothing
        // in flight: it arrives directly
        if (me < num_h) umma_commit(smem_u32(&s_acc));
        else mbar_arrive(smem_u32(&s_acc));
      }
    }
  } else {
    // ===== epilogue (warps 2..5) =====
    const int quarter = warp & 3;
    const int et = (int)threadIdx.x - 64;
    const int m = tile * kFTileM + quarter * 32 + lane;   // weight row of this thread
    const bool m_ok = m < p.m_total;
    epilogue_warps_sync();   // s_token_scale is complete
    bool have_acc = true;
    if (num_kb > 0) have_acc = mbar_wait_bounded(smem_u32(&s_acc), 0u, abort_flag);
    have_acc = __all_sync(0xffffffffu, have_acc);   // tcgen05.ld needs the whole warp
    if (threadIdx.x == 64) STAGE_STAMP(6, 0);
    // A block that gave up writes nothing; the status word reports it.
    if (have_acc) {
      tc_fence_after_sync();
      const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
      for (int c0 = 0; c0 < n_mma; c0 += 16) {
        // the q_planes accumulators of a weight tile, added up
        float g[16], u[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) g[j] = u[j] = 0.0f;
        if (num_kb > 0) {
          // down with two issuers: the second set exists only if that issuer had a step
          const int sets_to_add = kGateUp ? 1 : min(issuers, num_h);
          for (int a_set = 0; a_set < sets_to_add; ++a_set) {
            for (int q = 0; q < q_planes; ++q) {
              uint32_t a[16], b[16];
              tmem_ld_16(lane_base + (uint32_t)a_set * set_cols + (uint32_t)(q * n_mma + c0), a);
              if (kGateUp) tmem_ld_16(lane_base + set_cols + (uint32_t)(q * n_mma + c0), b);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                g[j] += __uint_as_float(a[j]);
                if (kGateUp) u[j] += __uint_as_float(b[j]);
              }
            }
          }
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const bool real = m_ok && c0 + j < n_rows;
          const float scale = s_token_scale[c0 + j] * w_scale;
          if (kGateUp) {
            float mag = 0.0f;
            if (real) {
              const float gate = g[j] * scale;
              const float up = u[j] * scale;
              const float act = gate / (1.0f + __expf(-gate)) * up;
              const __nv_bfloat16 hi = __float2bfloat16_rn(act);
              const __nv_bfloat16 lo = __float2bfloat16_rn(act - __bfloat162float(hi));
              const size_t o = (size_t)(row_start + c0 + j) * p.m_total + m;
              p.act_hi[o] = hi;
              p.act_lo[o] = lo;
              // what the plane kernel reads back is hi + lo
              mag = fabsf(__bfloat162float(hi) + __bfloat162float(lo));
            }
            // the row's max |activation| (non-negative floats order like their bit patterns)
            const uint32_t warp_max = __reduce_max_sync(0xffffffffu, __float_as_uint(mag));
            if (lane == 0) s_row_max[quarter][c0 + j] = __uint_as_float(warp_max);
          } else if (real) {
            float* dst = p.partials + (size_t)split * p.rows_cap * p.m_total;
            dst[(size_t)(row_start + c0 + j) * p.m_total + m] = g[j] * scale;
          }
        }
      }
    }
    if (kGateUp) {
      // this tile's max |activation| of every row: the plane kernel takes the maximum over
      // the tiles (plain stores; every (row, tile) of a valid row has exactly one writer)
      epilogue_warps_sync();
      if (have_acc && et < n_rows)
        p.tile_amax[(size_t)(row_start + et) * p.m_tiles + tile] =
            fmaxf(fmaxf(s_row_max[0][et], s_row_max[1][et]), fmaxf(s_row_max[2][et], s_row_max[3][et]));
    }
    if (threadIdx.x == 64) STAGE_STAMP(6, 4);
  }

  // ---- teardown -----------------------------------------------------------------------
  __syncwarp();
  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < kFAbortDrainNs) {
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicOr(p.status, B200MOE_STATUS_PIPE_TIMEOUT);
  trace_end(p.trace, kGateUp ? kTraceGateUp : kTraceDown);
  if (threadIdx.x == 0) STAGE_STAMP(6, 1);
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem, tmem_cols);
  }
}

// Two blocks per SM in general (107 KB of rings + 4 KB of static shared memory each); for
// grids of at most one block per SM a block gets the whole SM and a ring up to eight slots deep.
constexpr uint32_t kFStageBudget = 107u * 1024u;
constexpr uint32_t kFLoneBlockStageBudget = 216u * 1024u;

template <bool kGateUp>
static cudaError_t launch_nvfp4(const CUtensorMap& map_w, const CUtensorMap& map_b,
                                const FGemmParams& params, int grid, bool pdl,
                                cudaStream_t stream) {
  static bool attr_set[64] = {};
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= 64 || !attr_set[dev]) {
    err = cudaFuncSetAttribute(grouped_gemm_nvfp4_kernel<kGateUp>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)(kFLoneBlockStageBudget + 1024u));
    if (err != cudaSuccess) return err;
    if (dev >= 0 && dev < 64) attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kFThreads);
  cfg.dynamicSmemBytes = params.stage_budget + 1024u;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, grouped_gemm_nvfp4_kernel<kGateUp>, map_w, map_b, params);
}

static FGemmParams nvfp4_params(const int32_t* sched, int sched_cap, uint32_t* status,
                                const uint8_t* sfa, const float* tensor_scale,
                                const float* token_scale, int m_total, int k_total, int rows_cap,
                                int grid, int sm_count, int prefetch_slots, int issuers) {
  FGemmParams p = {};
  p.sched = sched;
  p.sched_cap = sched_cap;
  p.status = status;
  p.sfa = sfa;
  p.tensor_scale = tensor_scale;
  p.token_scale = token_scale;
  p.m_total = m_total;
  p.k_total = k_total;
  p.m_tiles = (m_total + kFTileM - 1) / kFTileM;
  p.rows_cap = rows_cap;
  p.trace = reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(status) +
                                                  kTraceOffsetBytes);
  const bool lone = sm_count > 0 && grid <= sm_count;
  p.stage_budget = lone ? kFLoneBlockStageBudget : kFStageBudget;
  p.prefetch_slots = prefetch_slots;
  p.issuers = issuers;
  return p;
}

cudaError_t launch_gate_up_nvfp4(const CUtensorMap& map_w, const CUtensorMap& map_x,
                                 const int32_t* sched, int sched_cap, uint32_t* status,
                                 void* act_hi, void* act_lo, float* tile_amax,
                                 const uint8_t* sfa, const float* tensor_scale,
                                 const float* token_scale, int inter, int hidden, int rows_cap,
                                 int grid, int sm_count, int prefetch_slots, int issuers,
                                 bool pdl, cudaStream_t stream) {
  FGemmParams p = nvfp4_params(sched, sched_cap, status, sfa, tensor_scale, token_scale, inter,
                               hidden, rows_cap, grid, sm_count, prefetch_slots, issuers);
  p.act_hi = static_cast<__nv_bfloat16*>(act_hi);
  p.act_lo = static_cast<__nv_bfloat16*>(act_lo);
  p.tile_amax = tile_amax;
  return launch_nvfp4<true>(map_w, map_x, p, grid, pdl, stream);
}

cudaError_t launch_down_nvfp4(const CUtensorMap& map_w, const CUtensorMap& map_act,
                              const int32_t* sched, int sched_cap, uint32_t* status,
                              float* partials, const uint8_t* sfa, const float* tensor_scale,
                              const float* token_scale, int hidden, int inter, int rows_cap,
                              int grid, int sm_count, int prefetch_slots, int issuers, bool pdl,
                              cudaStream_t stream) {
  FGemmParams p = nvfp4_params(sched, sched_cap, status, sfa, tensor_scale, token_scale, hidden,
                               inter, rows_cap, grid, sm_count, prefetch_slots, issuers);
  p.partials = partials;
  return launch_nvfp4<false>(map_w, map_act, p, grid, pdl, stream);
}

}  // namespace b200moe

#ifdef B200MOE_STAGE_TRACE
extern "C" int b200moe_debug_stage_trace(unsigned long long* host_out) {
  return (int)cudaMemcpyFromSymbol(host_out, b200moe::g_stage_trace,
                                   sizeof(b200moe::g_stage_trace));
}
#endif
