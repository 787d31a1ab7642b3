// Stages 3 and 4 with FP8 (E4M3) expert weights, on tcgen05.mma kind::f8f6f4.
//
// No counterpart in the reference, which lists quantised expert weights as future work
// (docs/goal_1b_report.md:313-314).  The layer is bound by streaming each active expert's
// weights once, so storing them as one E4M3 byte per element (plus an FP32 scale per
// weight row) halves the time of both GEMMs.
//
// The tensor core has no FP8 x BF16 mode, and converting the weight stream in shared
// memory costs more than the bytes it saves (measured: slower than the BF16 kernels).
// So the weights go from TMA straight into the MMA, and the small operand -- the token
// rows -- is what gets converted, once per row and not once per weight byte: every row r
// is held as E4M3 planes and a scale s_r,
//     x[r, k] ~= s_r * (p0[r,k] + p1[r,k] / 16 [+ p2[r,k] / 256]).
// The hidden rows of gate+up are BF16 (eight significant bits): with a power-of-two scale
// two planes hold them exactly.  The activation rows of the down projection carry sixteen
// bits (high + low BF16 halves): three planes keep twelve relative to the row maximum.
// The planes of a stage lie one after another in shared memory, i.e. they are one K-major
// operand of planes x rows rows, so ONE MMA per K step fills one FP32 accumulator per plane
// in tensor memory; the epilogue adds them with their weights and applies s_r and the
// weight row's scale.
//
// Same structure as the BF16 kernels otherwise: one block = (segment of <= 64 rows, weight
// tile[, K split]); warp 0 = TMA producer, warp 1 = TMEM allocation + MMA issue, warps 2..5
// = epilogue; two blocks per SM; every wait bounded.
//
// gate+up: a stage holds 128 gate rows and the 128 matching up rows (one 4-D TMA box over
// [E][2][I][H], 32 KB) and two MMAs per K step fill a gate and an up accumulator set, so
// SwiGLU is thread-local as in the BF16 kernel.  Besides the hi/lo BF16 activations the
// epilogue records each row's max |activation| (atomicMax on the bit pattern), from which
// the rows are re-quantised into planes for the down projection.
#include "common.cuh"

namespace b200moe {

constexpr int kQThreads = 192;
constexpr int kQStageK = 128;   // E4M3 elements (= bytes) per pipeline stage along K
constexpr int kQTileM = 128;
constexpr int kQMaxStages = 8;
constexpr uint32_t kQTileBytes = kQTileM * kQStageK;  // one 128-row weight tile of a stage: 16 KB
constexpr uint64_t kQAbortDrainNs = 1000000ull;

struct QGemmParams {
  const int32_t* sched;
  uint32_t* status;
  __nv_bfloat16* act_hi;      // gate+up output [rows_cap, I]
  __nv_bfloat16* act_lo;
  uint32_t* act_amax;         // gate+up output [rows_cap]: bit pattern of max |act| per row
  float* partials;            // down output [splits][rows_cap][H]
  const float* row_scale;     // weights: gate+up [E, 2I]; down [E, H]
  const float* token_scale;   // planes: [rows_cap]
  int m_total;                // I (gate+up) or H (down)
  int k_total;                // H (gate+up) or I (down)
  int m_tiles;                // ceil(I / 128) (gate+up) or ceil(H / 128) (down)
  int rows_cap;
  int sched_cap;              // segment entries the schedule array holds
  unsigned long long* trace;
  uint32_t stage_budget;
};

template <bool kGateUp>
__global__ void __launch_bounds__(kQThreads, 2)
grouped_gemm_fp8_kernel(const __grid_constant__ CUtensorMap map_w,
                        const __grid_constant__ CUtensorMap map_b, const QGemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t s_full[kQMaxStages];
  __shared__ __align__(8) uint64_t s_empty[kQMaxStages];
  __shared__ __align__(8) uint64_t s_acc;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  __shared__ float s_token_scale[kSegRowsFp8];
  __shared__ float s_row_max[4][kSegRowsFp8];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kQMaxStages; ++s) {
      mbar_init(smem_u32(&s_full[s]), 1);
      mbar_init(smem_u32(&s_empty[s]), 1);
    }
    mbar_init(smem_u32(&s_acc), 1);
    s_abort = 0;
    fence_mbar_init();
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_b);
  }

  // ---- this block's unit (the schedule is final before this grid can start) ----------
  int unit = blockIdx.x;
  int split = 0, n_split = 1;
  // header {segments, active, valid rows, splits} and the segment entry are 16 bytes each;
  // gate+up knows its segment index without the header, so both loads go out together (the
  // index is clamped to the array; blocks past the last segment leave right after)
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
  const int n_mma = (n_rows + 15) & ~15;  // accumulator columns per plane: 16..64
  trace_start(p.trace, kGateUp ? kTraceGateUp : kTraceDown);

  const int kblocks = (p.k_total + kQStageK - 1) / kQStageK;
  int kb0 = 0, num_kb = kblocks;
  if (!kGateUp) {
    const int per = kblocks / n_split, rem = kblocks % n_split;
    kb0 = split * per + min(split, rem);
    num_kb = per + (split < rem ? 1 : 0);
  }

  // ---- shared-memory pipeline geometry ----------------------------------------------
  constexpr int kPlanes = kGateUp ? kFp8PlanesHidden : kFp8Planes;
  constexpr uint32_t kABytes = kGateUp ? 2u * kQTileBytes : kQTileBytes;  // gate + up tiles
  const uint32_t plane_bytes = (uint32_t)n_mma * 128u;
  const uint32_t stage_bytes = kABytes + (uint32_t)kPlanes * plane_bytes;
  const int num_stages = min((int)(p.stage_budget / stage_bytes), kQMaxStages);
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  volatile int* abort_flag = &s_abort;
  if (num_stages < 2 || n_mma > kSegRowsFp8) {
    // a schedule with segments longer than this kernel supports: a caller error; report
    if (threadIdx.x == 0) atomicOr(p.status, B200MOE_STATUS_PIPE_TIMEOUT);
    return;
  }

  auto load_weights = [&](uint32_t dst, uint32_t bar, int kc) {
    if (kGateUp) tma_load_4d(dst, &map_w, bar, kc, tile * kQTileM, 0, expert);
    else tma_load_3d(dst, &map_w, bar, kc, tile * kQTileM, expert);
  };
  auto load_tokens = [&](uint32_t b_dst, uint32_t bar, int kc) {
    for (int pl = 0; pl < kPlanes; ++pl)
      for (int r = 0; r < n_mma; r += 16)
        tma_load_3d(b_dst + (uint32_t)pl * plane_bytes + (uint32_t)r * 128u, &map_b, bar, kc,
                    row_start + r, pl);
  };

  // Weight prefetch: fill the first stages' weight tiles while the previous kernel is
  // still finishing; the token planes of those stages follow after the dependency wait.
  const int prefetched = min(num_stages, num_kb);
  if (threadIdx.x == 0) {
    for (int i = 0; i < prefetched; ++i) {
      const uint32_t bar = smem_u32(&s_full[i]);
      mbar_expect_tx(bar, stage_bytes);
      load_weights(smem_base + (uint32_t)i * stage_bytes, bar, (kb0 + i) * kQStageK);
    }
  }
  // ---- tensor memory: one accumulator of n_mma columns per plane (gate and up: each);
  // allocated before the dependency wait ------------------------------------------------
  constexpr int kAccSets = kGateUp ? 2 : 1;
  uint32_t tmem_cols = 32;
  while (tmem_cols < (uint32_t)(kAccSets * kPlanes * n_mma)) tmem_cols <<= 1;
  if (warp == 1) {
    tmem_alloc(smem_u32(&s_tmem_base), tmem_cols);
    tmem_relinquish();
  }
  pdl_wait();
  pdl_launch_dependents();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = s_tmem_base;

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
        const int kc = (kb0 + i) * kQStageK;
        if (i >= prefetched) {
          mbar_expect_tx(bar, stage_bytes);
          load_weights(a_dst, bar, kc);
        }
        load_tokens(a_dst + kABytes, bar, kc);
      }
    }
  } else if (warp == 1) {
    // ===== MMA issuer =====
    if (lane == 0) {
      // The planes of a stage are one K-major operand of kPlanes * n_mma rows: a single MMA
      // per K step (and weight tile) fills all of a set's accumulators, plane pl in columns
      // [pl * n_mma, (pl + 1) * n_mma) of the set.
      const uint32_t idesc = umma_idesc_e4m3_m128((uint32_t)(kPlanes * n_mma));
      bool ok = true;
      for (int i = 0; i < num_kb; ++i) {
        const int s = i % num_stages;
        if (!mbar_wait_bounded(smem_u32(&s_full[s]), (uint32_t)(i / num_stages) & 1u,
                               abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        if (i == 0 && p.trace && blockIdx.x == 0)
          p.trace[2 * (kGateUp ? kTraceGateUpFirstData : kTraceDownFirstData)] = global_timer_ns();
        const uint32_t a_addr = smem_base + (uint32_t)s * stage_bytes;
        const uint64_t a0 = umma_smem_desc_sw128(a_addr);
        const uint64_t a1 = umma_smem_desc_sw128(a_addr + kQTileBytes);  // up tile (gate+up only)
        const uint64_t b0 = umma_smem_desc_sw128(a_addr + kABytes);
#pragma unroll
        for (int k = 0; k < kQStageK / 32; ++k) {
          // 32 one-byte elements along K = 32 bytes = 2 descriptor units
          const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
          umma_f8(tmem, a0 + 2u * k, b0 + 2u * k, idesc, acc);
          if (kGateUp)
            umma_f8(tmem + (uint32_t)(kPlanes * n_mma), a1 + 2u * k, b0 + 2u * k, idesc, acc);
        }
        umma_commit(smem_u32(&s_empty[s]));
      }
      if (ok && num_kb > 0) umma_commit(smem_u32(&s_acc));
    }
  } else {
    // ===== epilogue: TMEM -> registers -> scales -> global =====
    const int quarter = warp & 3;
    const int trow = quarter * 32 + lane;  // accumulator lane = weight row of the tile
    const int m = tile * kQTileM + trow;
    const bool m_ok = m < p.m_total;
    // Everything the epilogue needs from global memory is fetched now, under the main loop:
    // a load issued after the accumulators are complete would queue behind the weight
    // prefetch of the next kernel's blocks, which become resident at about that time.
    const int et = (int)threadIdx.x - 64;   // 0..127
    float scale0 = 0.0f, scale1 = 0.0f;     // gate and up row scales, or the down row scale
    if (m_ok) {
      if (kGateUp) {
        scale0 = p.row_scale[(size_t)expert * 2 * p.m_total + m];
        scale1 = p.row_scale[(size_t)expert * 2 * p.m_total + p.m_total + m];
      } else {
        scale0 = p.row_scale[(size_t)expert * p.m_total + m];
      }
    }
    if (et < kSegRowsFp8) {
      s_token_scale[et] = et < n_rows ? p.token_scale[row_start + et] : 0.0f;
#pragma unroll
      for (int q = 0; q < 4; ++q) s_row_max[q][et] = 0.0f;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");   // the four epilogue warps
    bool have_acc = true;
    if (num_kb > 0) have_acc = mbar_wait_bounded(smem_u32(&s_acc), 0u, abort_flag);
    have_acc = __all_sync(0xffffffffu, have_acc);  // tcgen05.ld needs the whole warp
    // A block that gave up writes nothing; the status word reports it.
    if (have_acc) {
      tc_fence_after_sync();
      const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
      // weighted sum of one set's plane accumulators for 16 columns starting at c0, times
      // the token rows' scales
      auto load_columns = [&](int set, int c0, float (&out)[16]) {
        if (num_kb > 0) {
          uint32_t a[kPlanes][16];
#pragma unroll
          for (int pl = 0; pl < kPlanes; ++pl)
            tmem_ld_16(lane_base + (uint32_t)((set * kPlanes + pl) * n_mma + c0), a[pl]);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float v = __uint_as_float(a[0][j]) + __uint_as_float(a[1][j]) * 0.0625f;
            if (kPlanes > 2) v += __uint_as_float(a[kPlanes - 1][j]) * 0.00390625f;
            out[j] = v * s_token_scale[c0 + j];
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) out[j] = 0.0f;
        }
      };
      if (kGateUp) {
        const float gate_scale = scale0, up_scale = scale1;
        float g[16], u[16];
        for (int c0 = 0; c0 < n_mma; c0 += 16) {
          load_columns(0, c0, g);
          load_columns(1, c0, u);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float mag = 0.0f;
            if (m_ok && c0 + j < n_rows) {
              const float gate = g[j] * gate_scale;
              const float up = u[j] * up_scale;
              const float act = gate / (1.0f + __expf(-gate)) * up;
              const __nv_bfloat16 hi = __float2bfloat16_rn(act);
              const __nv_bfloat16 lo = __float2bfloat16_rn(act - __bfloat162float(hi));
              const size_t o = (size_t)(row_start + c0 + j) * p.m_total + m;
              p.act_hi[o] = hi;
              p.act_lo[o] = lo;
              // what the next kernel reads back is hi + lo
              mag = fabsf(__bfloat162float(hi) + __bfloat162float(lo));
            }
            // non-negative floats order like their bit patterns
            const uint32_t warp_max = __reduce_max_sync(0xffffffffu, __float_as_uint(mag));
            if (lane == 0) s_row_max[quarter][c0 + j] = __uint_as_float(warp_max);
          }
        }
      } else {
        const float scale = scale0;
        float* dst = p.partials + (size_t)split * p.rows_cap * p.m_total;
        float v[16];
        for (int c0 = 0; c0 < n_mma; c0 += 16) {
          load_columns(0, c0, v);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if (m_ok && c0 + j < n_rows)
              dst[(size_t)(row_start + c0 + j) * p.m_total + m] = v[j] * scale;
          }
        }
      }
    }
    if (kGateUp) {
      // one atomic per block and row (one per warp made 448 same-address atomics per row
      // at T = 1, all at the end of the launch)
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (have_acc && et < n_rows) {
        const float mx = fmaxf(fmaxf(s_row_max[0][et], s_row_max[1][et]),
                               fmaxf(s_row_max[2][et], s_row_max[3][et]));
        if (mx > 0.0f) atomicMax(p.act_amax + row_start + et, __float_as_uint(mx));
      }
    }
  }

  // ---- teardown -----------------------------------------------------------------------
  __syncwarp();
  if (*abort_flag) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < kQAbortDrainNs) {
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

constexpr uint32_t kQStageBudget = 110u * 1024u;  // 16 rows: three 36 KB (gate+up) or five 22 KB (down) stages; with 1.4 KB of static shared memory two blocks fit an SM
// a grid of at most one block per SM gets the whole SM's shared memory per block (deeper
// ring: more bytes in flight when few blocks stream)
constexpr uint32_t kQLoneBlockStageBudget = 216u * 1024u;

template <bool kGateUp>
static cudaError_t launch_fp8(const CUtensorMap& map_w, const CUtensorMap& map_b,
                              const QGemmParams& params, int grid, bool pdl,
                              cudaStream_t stream) {
  static bool attr_set[64] = {};
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= 64 || !attr_set[dev]) {
    err = cudaFuncSetAttribute(grouped_gemm_fp8_kernel<kGateUp>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)(kQLoneBlockStageBudget + 1024u));
    if (err != cudaSuccess) return err;
    if (dev >= 0 && dev < 64) attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kQThreads);
  cfg.dynamicSmemBytes = params.stage_budget + 1024u;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, grouped_gemm_fp8_kernel<kGateUp>, map_w, map_b, params);
}

static QGemmParams fp8_params(const int32_t* sched, int sched_cap, uint32_t* status, const float* row_scale,
                              const float* token_scale, int m_total, int k_total, int m_tiles,
                              int rows_cap, int grid, int sm_count) {
  QGemmParams p = {};
  p.sched = sched;
  p.sched_cap = sched_cap;
  p.status = status;
  p.row_scale = row_scale;
  p.token_scale = token_scale;
  p.m_total = m_total;
  p.k_total = k_total;
  p.m_tiles = m_tiles;
  p.rows_cap = rows_cap;
  p.trace = reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(status) +
                                                  kTraceOffsetBytes);
  p.stage_budget = (sm_count > 0 && grid <= sm_count) ? kQLoneBlockStageBudget : kQStageBudget;
  return p;
}

cudaError_t launch_gate_up_fp8(const CUtensorMap& map_w, const CUtensorMap& map_x,
                               const int32_t* sched, int sched_cap, uint32_t* status,
                               void* act_hi, void* act_lo, uint32_t* act_amax, const float* row_scale,
                               const float* token_scale, int inter, int hidden, int rows_cap,
                               int grid, int sm_count, bool pdl, cudaStream_t stream) {
  QGemmParams p = fp8_params(sched, sched_cap, status, row_scale, token_scale, inter, hidden,
                             (inter + 127) / 128, rows_cap, grid, sm_count);
  p.act_hi = static_cast<__nv_bfloat16*>(act_hi);
  p.act_lo = static_cast<__nv_bfloat16*>(act_lo);
  p.act_amax = act_amax;
  return launch_fp8<true>(map_w, map_x, p, grid, pdl, stream);
}

cudaError_t launch_down_fp8(const CUtensorMap& map_w, const CUtensorMap& map_act,
                            const int32_t* sched, int sched_cap, uint32_t* status, float* partials,
                            const float* row_scale, const float* token_scale, int hidden,
                            int inter, int rows_cap, int grid, int sm_count, bool pdl,
                            cudaStream_t stream) {
  QGemmParams p = fp8_params(sched, sched_cap, status, row_scale, token_scale, hidden, inter,
                             (hidden + 127) / 128, rows_cap, grid, sm_count);
  p.partials = partials;
  return launch_fp8<false>(map_w, map_act, p, grid, pdl, stream);
}

}  // namespace b200moe
