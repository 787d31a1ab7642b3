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
// operand is what gets converted: every token row is held as four E2M1 planes with their own
// block scales, x ~= t * sum_p scale_p * element_p (nvfp4_quant.cu).  The planes of a stage
// lie one after another in shared memory, so Q consecutive planes form one K-major operand of
// Q x rows rows: one MMA of N = Q x rows <= 64 fills Q accumulators at once (Q = 4 for up to
// 16 rows, 2 up to 32, 1 beyond), and the remaining planes accumulate into the same columns
// with further MMAs.  Tensor memory therefore holds at most 64 accumulator columns per
// weight tile whatever the segment length, few instructions are issued per byte streamed
// (a kernel issuing one MMA per plane was bound by instruction issue, not by HBM), and the
// epilogue adds the Q accumulators and applies t and the weight tensor's FP32 scale.
//
// Scales live in tensor memory while an MMA runs.  Weight scales are stored pre-arranged in
// 512-byte tiles (128 rows x 4 scales) and reach shared memory with one bulk copy per stage;
// token scales are stored plainly ([plane][row][K / 16]) and the four epilogue warps, idle
// during the main loop, arrange each stage's tiles in shared memory (a segment starts at an
// arbitrary row, which a fixed global tiling could not follow).  The issuing thread copies
// every tile to tensor memory (tcgen05.cp) right before the MMAs that use it; copies and
// MMAs of one thread execute in issue order.
//
// Same structure as the other GEMM kernels otherwise: one block = (segment of <= 64 rows,
// 128-row weight tile[, K split]); warp 0 = TMA producer, warp 1 = TMEM allocation + MMA
// issue, warps 2..5 = scale arranging, then epilogue; two blocks per SM; every wait bounded.
// A pipeline stage covers 256 elements of K: 128 bytes per row, the 128-byte swizzle.
#include "common.cuh"

namespace b200moe {

constexpr int kFThreads = 192;
constexpr int kFStageK = 256;                      // E2M1 elements per stage along K
constexpr int kFTileM = 128;
constexpr int kFMaxStages = 4;
constexpr uint32_t kFTileBytes = kFTileM * 128u;   // one weight tile of a stage: 16 KB
constexpr uint32_t kFSfTile = 512u;                // scales of 128 rows x 64 elements of K
constexpr uint32_t kFSfaBytes = 4u * kFSfTile;     // one weight tile's scales of a stage
// planes one MMA covers for a segment of n_mma (16, 32, 48 or 64) accumulator columns
__host__ __device__ inline int nvfp4_planes_per_mma(int n_mma) {
  return n_mma <= 16 ? 4 : (n_mma <= 32 ? 2 : 1);
}
constexpr uint64_t kFAbortDrainNs = 1000000ull;

struct FGemmParams {
  const int32_t* sched;
  uint32_t* status;
  __nv_bfloat16* act_hi;      // gate+up output [rows_cap, I]
  __nv_bfloat16* act_lo;
  uint32_t* act_amax;         // gate+up output [rows_cap]: bit pattern of max |act| per row
  float* partials;            // down output [splits][rows_cap][H]
  const uint8_t* sfa;         // weight scales, 512-byte tiles: [E][(2)][m_tiles][k_tiles]
  const float* tensor_scale;  // [E]
  const uint8_t* sfb;         // token scales [planes][rows_cap][k_total / 16]
  const float* token_scale;   // [rows_cap]
  int m_total;                // I (gate+up) or H (down)
  int k_total;                // H (gate+up) or I (down)
  int m_tiles;
  int rows_cap;
  int sched_cap;
  unsigned long long* trace;
  uint32_t stage_budget;
};

template <bool kGateUp>
__global__ void __launch_bounds__(kFThreads, 2)
grouped_gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap map_w,
                          const __grid_constant__ CUtensorMap map_b, const FGemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t s_full[kFMaxStages];   // weights, weight scales, token planes
  __shared__ __align__(8) uint64_t s_sfb[kFMaxStages];    // token scales arranged
  __shared__ __align__(8) uint64_t s_empty[kFMaxStages];
  __shared__ __align__(8) uint64_t s_acc;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kFMaxStages; ++s) {
      mbar_init(smem_u32(&s_full[s]), 1);
      mbar_init(smem_u32(&s_sfb[s]), 4);   // one arrival per epilogue warp
      mbar_init(smem_u32(&s_empty[s]), 1);
    }
    mbar_init(smem_u32(&s_acc), 1);
    s_abort = 0;
    fence_mbar_init();
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_b);
  }
  __syncthreads();

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
  const int n_mma = (n_rows + 15) & ~15;   // accumulator columns: 16..64
  trace_start(p.trace, kGateUp ? kTraceGateUp : kTraceDown);

  const int kblocks = (p.k_total + kFStageK - 1) / kFStageK;
  const int k_tiles = (p.k_total + 63) / 64;   // scale tiles along K
  int kb0 = 0, num_kb = kblocks;
  if (!kGateUp) {
    const int per = kblocks / n_split, rem = kblocks % n_split;
    kb0 = split * per + min(split, rem);
    num_kb = per + (split < rem ? 1 : 0);
  }

  // ---- shared-memory stage: weights | weight scales | token planes | token scales ------
  constexpr int kSets = kGateUp ? 2 : 1;   // gate and up tiles, or the one down tile
  constexpr uint32_t kABytes = kSets * kFTileBytes;
  constexpr uint32_t kSfaStage = kSets * kFSfaBytes;
  const uint32_t plane_bytes = (uint32_t)n_mma * 128u;
  const uint32_t b_bytes = kNvfp4Planes * plane_bytes;
  const int q_planes = nvfp4_planes_per_mma(n_mma);   // planes per MMA
  const int passes = kNvfp4Planes / q_planes;         // MMAs per weight tile and 64 elements of K
  const uint32_t sfb_bytes = (uint32_t)passes * 4u * kFSfTile;   // one scale tile per pass and K group
  const uint32_t stage_bytes = kABytes + kSfaStage + b_bytes + sfb_bytes;
  const int num_stages = min((int)(p.stage_budget / stage_bytes), kFMaxStages);
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_ptr = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile int* abort_flag = &s_abort;
  if (num_stages < 2 || n_mma > kSegRowsNvfp4) {
    // a schedule with segments longer than this kernel supports: a caller error; report
    if (threadIdx.x == 0) atomicOr(p.status, B200MOE_STATUS_PIPE_TIMEOUT);
    return;
  }

  // scale tiles of K the stage that starts at element kc holds (the last stage may be short)
  auto groups_at = [&](int kc) { return min(4, k_tiles - kc / 64); };
  // weight-scale tiles of this block's rows: set 0 = the (gate) tile, set 1 = the up tile
  auto sfa_src = [&](int set, int kc) {
    const size_t tile_index =
        kGateUp ? ((size_t)(expert * 2 + set) * p.m_tiles + tile) : ((size_t)expert * p.m_tiles + tile);
    return p.sfa + (tile_index * k_tiles + kc / 64) * kFSfTile;
  };
  auto load_weights = [&](uint32_t dst, uint32_t bar, int kc) {
    // data: one box over [E][2][I][H / 2 bytes] (gate rows, then the matching up rows), or
    // over [E][H][I / 2 bytes]; coordinates of the innermost dimension are in bytes
    if (kGateUp) tma_load_4d(dst, &map_w, bar, kc / 2, tile * kFTileM, 0, expert);
    else tma_load_3d(dst, &map_w, bar, kc / 2, tile * kFTileM, expert);
    const uint32_t bytes = (uint32_t)groups_at(kc) * kFSfTile;
    for (int set = 0; set < kSets; ++set)
      bulk_load(dst + kABytes + (uint32_t)set * kFSfaBytes, sfa_src(set, kc), bytes, bar);
  };
  auto stage_tx = [&](int kc) {
    return kABytes + (uint32_t)(kSets * groups_at(kc)) * kFSfTile + b_bytes;
  };
  auto load_tokens = [&](uint32_t b_dst, uint32_t bar, int kc) {
    for (int pl = 0; pl < kNvfp4Planes; ++pl)
      for (int r = 0; r < n_mma; r += 16)
        tma_load_3d(b_dst + (uint32_t)pl * plane_bytes + (uint32_t)r * 128u, &map_b, bar, kc / 2,
                    row_start + r, pl);
  };

  // Weight prefetch: fill the first stages' weight tiles and scales while the previous
  // kernel is still finishing; the token planes of those stages follow after the wait.
  const int prefetched = min(num_stages, num_kb);
  if (threadIdx.x == 0) {
    for (int i = 0; i < prefetched; ++i) {
      const uint32_t bar = smem_u32(&s_full[i]);
      const int kc = (kb0 + i) * kFStageK;
      mbar_expect_tx(bar, stage_tx(kc));
      load_weights(smem_base + (uint32_t)i * stage_bytes, bar, kc);
    }
  }
  pdl_wait();
  pdl_launch_dependents();

  // ---- tensor memory: accumulators, then the scale columns ------------------------------
  const uint32_t set_cols = (uint32_t)(q_planes * n_mma);   // accumulator columns per weight tile
  const uint32_t acc_cols = kSets * set_cols;
  constexpr uint32_t kSfaCols = kSets * 16u;              // 4 tiles x 4 columns per weight tile
  const uint32_t kSfbCols = (uint32_t)passes * 16u;
  uint32_t tmem_cols = 32;
  while (tmem_cols < acc_cols + kSfaCols + kSfbCols) tmem_cols <<= 1;
  if (warp == 1) {
    tmem_alloc(smem_u32(&s_tmem_base), tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = s_tmem_base;
  const uint32_t tmem_sfa = tmem + acc_cols;
  const uint32_t tmem_sfb = tmem_sfa + kSfaCols;

  if (warp == 0) {
    // ===== TMA producer =====
    if (lane == 0) {
      for (int i = 0; i < num_kb; ++i) {
        const int s = i % num_stages;
        const uint32_t round = (uint32_t)(i / num_stages);
        if (i >= num_stages &&
            !mbar_wait_bounded(smem_u32(&s_empty[s]), (round - 1u) & 1u, abort_flag))
          break;
        const uint32_t bar = smem_u32(&s_full[s]);
        const uint32_t a_dst = smem_base + (uint32_t)s * stage_bytes;
        const int kc = (kb0 + i) * kFStageK;
        if (i >= prefetched) {
          mbar_expect_tx(bar, stage_tx(kc));
          load_weights(a_dst, bar, kc);
        }
        load_tokens(a_dst + kABytes + kSfaStage, bar, kc);
      }
    }
  } else if (warp == 1) {
    // ===== scale copies + MMA issue =====
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_nvfp4_m128(set_cols);
      bool ok = true;
      for (int i = 0; i < num_kb; ++i) {
        const int s = i % num_stages;
        const uint32_t parity = (uint32_t)(i / num_stages) & 1u;
        if (!mbar_wait_bounded(smem_u32(&s_full[s]), parity, abort_flag) ||
            !mbar_wait_bounded(smem_u32(&s_sfb[s]), parity, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        if (i == 0 && p.trace && blockIdx.x == 0)
          p.trace[2 * (kGateUp ? kTraceGateUpFirstData : kTraceDownFirstData)] = global_timer_ns();
        const int kc = (kb0 + i) * kFStageK;
        const int groups = groups_at(kc);
        const uint32_t a_addr = smem_base + (uint32_t)s * stage_bytes;
        const uint32_t sfa_addr = a_addr + kABytes;
        const uint32_t b_addr = sfa_addr + kSfaStage;
        const uint32_t sfb_addr = b_addr + b_bytes;
        for (int g = 0; g < groups; ++g) {
          for (int set = 0; set < kSets; ++set)
            tmem_copy_scales(tmem_sfa + (uint32_t)(set * 16 + g * 4),
                             sfa_addr + (uint32_t)set * kFSfaBytes + (uint32_t)g * kFSfTile);
          for (int pass = 0; pass < passes; ++pass)
            tmem_copy_scales(tmem_sfb + (uint32_t)((pass * 4 + g) * 4),
                             sfb_addr + (uint32_t)(pass * 4 + g) * kFSfTile);
        }
        const uint64_t a0 = umma_smem_desc_sw128(a_addr);
        const uint64_t a1 = umma_smem_desc_sw128(a_addr + kFTileBytes);   // up tile
        for (int g = 0; g < groups; ++g) {
          for (int pass = 0; pass < passes; ++pass) {
            // the pass's q_planes planes are one operand of q_planes * n_mma rows;
            // 64 E2M1 elements along K = 32 bytes = 2 descriptor units
            const uint64_t b =
                umma_smem_desc_sw128(b_addr + (uint32_t)(pass * q_planes) * plane_bytes) + 2u * g;
            const uint32_t acc = (i > 0 || g > 0 || pass > 0) ? 1u : 0u;
            const uint32_t sfb_t = tmem_sfb + (uint32_t)((pass * 4 + g) * 4);
            umma_nvfp4(tmem, a0 + 2u * g, b, idesc, tmem_sfa + (uint32_t)(g * 4), sfb_t, acc);
            if (kGateUp)
              umma_nvfp4(tmem + set_cols, a1 + 2u * g, b, idesc, tmem_sfa + (uint32_t)(16 + g * 4),
                         sfb_t, acc);
          }
        }
        umma_commit(smem_u32(&s_empty[s]));
      }
      if (ok && num_kb > 0) umma_commit(smem_u32(&s_acc));
    }
  } else {
    // ===== token scales of every stage, then the epilogue =====
    // One item = (plane, row of the segment): its 16 scales of a stage are four words, one
    // per K group.  The planes of one pass share a scale tile: the item is row
    // r = (plane % q_planes) * n_mma + n of its pass's operand, and its word goes to byte
    // (r % 32) * 16 + (r / 32) * 4 of that pass's tile of the K group.  At most two items
    // per thread.  The words of the NEXT stage are requested before this stage's
    // slot is waited for, so the global-memory latency stays off the pipeline's path.
    const int et = (int)threadIdx.x - 64;   // 0..127
    const int sf_per_row = p.k_total / 16;
    const int items = kNvfp4Planes * n_mma;
    auto fetch = [&](int i, uint32_t (&w)[2][4]) {
      const int kc = (kb0 + i) * kFStageK;
#pragma unroll
      for (int it = 0; it < 2; ++it) {
        const int item = et + it * 128;
        const int pl = item / n_mma, n = item % n_mma;
        const bool real = item < items && n < n_rows;
        const uint32_t* src = reinterpret_cast<const uint32_t*>(
            p.sfb + ((size_t)pl * p.rows_cap + row_start + n) * sf_per_row);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int word = kc / 64 + g;   // scale tile along K = word of the row
          w[it][g] = (real && word < k_tiles) ? __ldg(src + word) : 0u;
        }
      }
    };
    uint32_t cur[2][4], nxt[2][4];
    if (num_kb > 0) fetch(0, cur);
    bool alive = true;
    for (int i = 0; i < num_kb && alive; ++i) {
      const int s = i % num_stages;
      const uint32_t round = (uint32_t)(i / num_stages);
      if (i + 1 < num_kb) fetch(i + 1, nxt);
      if (i >= num_stages)
        alive = mbar_wait_bounded(smem_u32(&s_empty[s]), (round - 1u) & 1u, abort_flag);
      alive = __all_sync(0xffffffffu, alive);
      if (!alive) break;
      uint8_t* sfb_s = smem_ptr + (size_t)s * stage_bytes + kABytes + kSfaStage + b_bytes;
#pragma unroll
      for (int it = 0; it < 2; ++it) {
        const int item = et + it * 128;
        if (item >= items) continue;
        const int pl = item / n_mma, n = item % n_mma;
        const int pass = pl / q_planes, r = (pl % q_planes) * n_mma + n;
#pragma unroll
        for (int g = 0; g < 4; ++g)
          *reinterpret_cast<uint32_t*>(sfb_s + (size_t)(pass * 4 + g) * kFSfTile + (r & 31) * 16 +
                                       (r >> 5) * 4) = cur[it][g];
      }
      fence_proxy_async_smem();   // the tensor-memory copy reads through the async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&s_sfb[s]));
#pragma unroll
      for (int it = 0; it < 2; ++it)
#pragma unroll
        for (int g = 0; g < 4; ++g) cur[it][g] = nxt[it][g];
    }

    const int quarter = warp & 3;
    const int m = tile * kFTileM + quarter * 32 + lane;   // weight row of this thread
    const bool m_ok = m < p.m_total;
    bool have_acc = true;
    if (num_kb > 0) have_acc = mbar_wait_bounded(smem_u32(&s_acc), 0u, abort_flag);
    have_acc = __all_sync(0xffffffffu, have_acc);   // tcgen05.ld needs the whole warp
    // A block that gave up writes nothing; the status word reports it.
    if (have_acc) {
      tc_fence_after_sync();
      const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
      const float w_scale = p.tensor_scale[expert];
      for (int c0 = 0; c0 < n_mma; c0 += 16) {
        // the q_planes accumulators of a weight tile, added up
        float g[16], u[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) g[j] = u[j] = 0.0f;
        if (num_kb > 0) {
          for (int q = 0; q < q_planes; ++q) {
            uint32_t a[16], b[16];
            tmem_ld_16(lane_base + (uint32_t)(q * n_mma + c0), a);
            if (kGateUp) tmem_ld_16(lane_base + set_cols + (uint32_t)(q * n_mma + c0), b);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              g[j] += __uint_as_float(a[j]);
              if (kGateUp) u[j] += __uint_as_float(b[j]);
            }
          }
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const bool real = m_ok && c0 + j < n_rows;
          const float scale = c0 + j < n_rows ? p.token_scale[row_start + c0 + j] * w_scale : 0.0f;
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
            if (lane == 0 && c0 + j < n_rows && warp_max != 0u)
              atomicMax(p.act_amax + row_start + c0 + j, warp_max);
          } else if (real) {
            float* dst = p.partials + (size_t)split * p.rows_cap * p.m_total;
            dst[(size_t)(row_start + c0 + j) * p.m_total + m] = g[j] * scale;
          }
        }
      }
    }
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
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem, tmem_cols);
  }
}

// Two blocks per SM while two stages of the longest possible segment fit into half an SM's
// shared memory (16 rows: two 46 KB gate+up or three 28 KB down stages); otherwise, and for
// grids of at most one block per SM, a block gets the whole SM (a stage of a 64-row segment
// is 76 KB for gate+up).
constexpr uint32_t kFStageBudget = 111u * 1024u;
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
                                const uint8_t* sfb, const float* token_scale, int m_total,
                                int k_total, int rows_cap, int max_rows, bool gate_up, int grid,
                                int sm_count) {
  FGemmParams p = {};
  p.sched = sched;
  p.sched_cap = sched_cap;
  p.status = status;
  p.sfa = sfa;
  p.tensor_scale = tensor_scale;
  p.sfb = sfb;
  p.token_scale = token_scale;
  p.m_total = m_total;
  p.k_total = k_total;
  p.m_tiles = (m_total + kFTileM - 1) / kFTileM;
  p.rows_cap = rows_cap;
  p.trace = reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(status) +
                                                  kTraceOffsetBytes);
  // the longest segment this call can have, as accumulator columns
  int n_mma = max_rows < kSegRowsNvfp4 ? max_rows : kSegRowsNvfp4;
  n_mma = (n_mma + 15) & ~15;
  const uint32_t stage = (gate_up ? 2u : 1u) * (kFTileBytes + kFSfaBytes) +
                         kNvfp4Planes * (uint32_t)n_mma * 128u +
                         (uint32_t)(kNvfp4Planes / nvfp4_planes_per_mma(n_mma)) * 4u * kFSfTile;
  const bool lone = (sm_count > 0 && grid <= sm_count) || 2u * stage > kFStageBudget;
  p.stage_budget = lone ? kFLoneBlockStageBudget : kFStageBudget;
  return p;
}

cudaError_t launch_gate_up_nvfp4(const CUtensorMap& map_w, const CUtensorMap& map_x,
                                 const int32_t* sched, int sched_cap, uint32_t* status,
                                 void* act_hi, void* act_lo, uint32_t* act_amax,
                                 const uint8_t* sfa,
                                 const float* tensor_scale, const uint8_t* sfb,
                                 const float* token_scale, int inter, int hidden, int rows_cap,
                                 int max_rows, int grid, int sm_count, bool pdl,
                                 cudaStream_t stream) {
  FGemmParams p = nvfp4_params(sched, sched_cap, status, sfa, tensor_scale, sfb, token_scale,
                               inter, hidden, rows_cap, max_rows, true, grid, sm_count);
  p.act_hi = static_cast<__nv_bfloat16*>(act_hi);
  p.act_lo = static_cast<__nv_bfloat16*>(act_lo);
  p.act_amax = act_amax;
  return launch_nvfp4<true>(map_w, map_x, p, grid, pdl, stream);
}

cudaError_t launch_down_nvfp4(const CUtensorMap& map_w, const CUtensorMap& map_act,
                              const int32_t* sched, int sched_cap, uint32_t* status,
                              float* partials, const uint8_t* sfa, const float* tensor_scale,
                              const uint8_t* sfb, const float* token_scale, int hidden, int inter,
                              int rows_cap, int max_rows, int grid, int sm_count, bool pdl,
                              cudaStream_t stream) {
  FGemmParams p = nvfp4_params(sched, sched_cap, status, sfa, tensor_scale, sfb, token_scale,
                               hidden, inter, rows_cap, max_rows, false, grid, sm_count);
  p.partials = partials;
  return launch_nvfp4<false>(map_w, map_act, p, grid, pdl, stream);
}

}  // namespace b200moe
