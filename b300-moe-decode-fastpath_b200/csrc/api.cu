// extern "C" entry points of libb200moe.so (declared in include/b200moe.h):
// argument checks, TMA tensor-map encoding, grid sizing and kernel launches.
// Host code here never allocates device memory, never synchronises and never
// reads device memory.
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <mutex>

#include <cudaTypedefs.h>

#include "common.cuh"

namespace b200moe {

// kernels / launchers defined in the other translation units
cudaError_t launch_routing(const int64_t* ids, const void* weights, int num_assign, int top_k,
                           int num_experts, int64_t* counts, int64_t* offsets,
                           int64_t* reverse_mapping, int64_t* permutation, int32_t* offsets_i32,
                           int64_t* perm_tokens, int64_t* perm_experts, void* perm_weights,
                           int32_t* sched, uint32_t* status, int down_tiles, int down_kblocks,
                           int target_ctas, int seg_rows, int id_base, bool foreign_ids_allowed,
                           const uint32_t* wait_flags, int wait_world, uint32_t wait_epoch,
                           unsigned long long wait_limit_ns, bool after_gate_up, bool pdl,
                           bool after_dispatch, void* zero_rows, int zero_row_vecs,
                           cudaStream_t stream);
cudaError_t launch_ep_push(const void* hidden, const int64_t* ids, const void* weights,
                           void* const* hidden_dst, void* const* ids_dst,
                           void* const* weights_dst, void* const* flag_ptrs,
                           unsigned int* block_counter, int world, int rank, int tokens_local,
                           int top_k, int hidden_size, uint32_t epoch, cudaStream_t stream);
cudaError_t launch_routing_static(const int64_t* ids, const void* weights, int num_assign,
                                  int top_k, int num_experts, int64_t* counts, int64_t* offsets,
                                  int64_t* reverse_mapping, int64_t* permutation,
                                  int32_t* offsets_i32, int64_t* perm_tokens,
                                  int64_t* perm_experts, void* perm_weights, int down_tiles,
                                  int down_kblocks, int target_ctas, cudaStream_t stream);
cudaError_t launch_gather(const void* hidden, const int64_t* permutation, void* out,
                          int num_assign, int num_tokens, int top_k, int hidden_size,
                          unsigned long long* trace, bool pdl, cudaStream_t stream);
cudaError_t launch_combine(const int64_t* reverse_mapping, const void* weights,
                           const float* partials, const int32_t* sched, void* out,
                           void* expert_out, int num_tokens, int top_k, int hidden_size,
                           size_t slice_elems, bool f32_out, unsigned long long* trace, bool pdl,
                           cudaStream_t stream);
cudaError_t launch_gate_up(const CUtensorMap& map_w, const CUtensorMap& map_x,
                           const CUtensorMap* map_hidden, const int32_t* sched, int sched_cap,
                           uint32_t* status, void* act_hi, void* act_lo, int inter, int hidden,
                           int rows_cap, int grid, const SmallCall* small, int overlap,
                           int sm_count, bool pdl, cudaStream_t stream);
cudaError_t launch_down(const CUtensorMap& map_w, const CUtensorMap& map_hi,
                        const CUtensorMap& map_lo, const int32_t* sched, int sched_cap,
                        uint32_t* status, float* partials, int hidden, int inter, int rows_cap,
                        int grid, const SmallCall* small, int overlap, int sm_count, bool pdl,
                        cudaStream_t stream);

cudaError_t launch_gate_up_fp8(const CUtensorMap& map_w, const CUtensorMap& map_x,
                               const int32_t* sched, int sched_cap, uint32_t* status,
                               void* act_hi, void* act_lo, uint32_t* act_amax,
                               const float* row_scale,
                               const float* token_scale, int inter, int hidden, int rows_cap,
                               int grid, int sm_count, bool pdl, cudaStream_t stream);
cudaError_t launch_down_fp8(const CUtensorMap& map_w, const CUtensorMap& map_act,
                            const int32_t* sched, int sched_cap, uint32_t* status,
                            float* partials,
                            const float* row_scale, const float* token_scale, int hidden,
                            int inter, int rows_cap, int grid, int sm_count, bool pdl,
                            cudaStream_t stream);
cudaError_t launch_gather_fp8(const void* hidden, const int64_t* permutation, void* out,
                              uint8_t* planes, float* row_scale, uint32_t* act_amax,
                              int num_assign, int num_tokens, int top_k, int hidden_size,
                              int rows_cap, unsigned long long* trace, bool pdl,
                              cudaStream_t stream);
cudaError_t launch_act_planes_fp8(const void* act_hi, const void* act_lo,
                                  const uint32_t* act_amax, uint8_t* planes, float* row_scale,
                                  int num_assign, int inter, int rows_cap, bool pdl,
                                  cudaStream_t stream);
cudaError_t launch_fp8_quantize_rows(const void* w, long long rows, int cols, uint8_t* q,
                                     float* scale, cudaStream_t stream);
cudaError_t launch_fp8_dequantize_rows(const uint8_t* q, const float* scale, long long rows,
                                       int cols, void* out, cudaStream_t stream);

cudaError_t launch_nvfp4_quantize(const void* w, int experts, int rows, int cols, int halves,
                                  uint8_t* packed, uint8_t* sf, float* tensor_scale,
                                  uint32_t* amax_scratch, cudaStream_t stream);
cudaError_t launch_gather_nvfp4(const void* hidden, const int64_t* permutation, void* out,
                                uint8_t* planes, float* row_scale, int num_assign,
                                int num_tokens, int top_k, int hidden_size, int rows_cap,
                                unsigned long long* trace, bool pdl, cudaStream_t stream);
cudaError_t launch_act_planes_nvfp4(const void* act_hi, const void* act_lo,
                                    const float* tile_amax, uint8_t* planes, float* row_scale,
                                    int num_assign, int inter, int rows_cap, bool pdl,
                                    cudaStream_t stream);
cudaError_t launch_rows_to_planes_nvfp4(const float* rows, int num_rows, int cols,
                                        uint8_t* planes, float* row_scale,
                                        cudaStream_t stream);
cudaError_t launch_gate_up_nvfp4(const CUtensorMap& map_w, const CUtensorMap& map_x,
                                 const int32_t* sched, int sched_cap, uint32_t* status,
                                 void* act_hi, void* act_lo, float* tile_amax,
                                 const uint8_t* sfa, const float* tensor_scale,
                                 const float* token_scale, int inter, int hidden, int rows_cap,
                                 int grid, int sm_count, int prefetch_slots, int issuers,
                                 bool pdl, cudaStream_t stream);
cudaError_t launch_down_nvfp4(const CUtensorMap& map_w, const CUtensorMap& map_act,
                              const int32_t* sched, int sched_cap, uint32_t* status,
                              float* partials, const uint8_t* sfa, const float* tensor_scale,
                              const float* token_scale, int hidden, int inter, int rows_cap,
                              int grid, int sm_count, int prefetch_slots, int issuers, bool pdl,
                              cudaStream_t stream);

cudaError_t launch_combine_bf16(const void* expert_rows, const int64_t* assignment_to_permuted,
                                const void* weights, void* out, int num_tokens, int top_k,
                                int hidden_size, cudaStream_t stream);
cudaError_t launch_ep_reduce(const void* const* partial_ptrs, void* const* flag_ptrs, int world,
                             int rank, int num_tokens, int hidden, uint32_t epoch,
                             unsigned long long wait_limit_ns, void* output, uint32_t* status,
                             bool pdl, cudaStream_t stream);

cudaError_t launch_ep_combine_reduce(const int64_t* reverse_mapping, const void* weights,
                                     const float* slices, const int32_t* sched,
                                     void* expert_out, const int64_t* ids,
                                     const void* const* partial_ptrs, void* const* flag_ptrs,
                                     unsigned int* block_counter, void* output,
                                     uint32_t* status, size_t slice_elems, int num_tokens,
                                     int top_k, int hidden, int experts_per_rank, int world,
                                     int rank, int first_token, int out_tokens, uint32_t epoch,
                                     unsigned long long wait_limit_ns, unsigned long long* trace,
                                     bool pdl, cudaStream_t stream);

int ep_combine_reduce_resident_blocks(int sm_count);
int ep_combine_push_resident_blocks(int sm_count);
cudaError_t launch_ep_combine_push(const int64_t* reverse_mapping, const void* weights,
                                   const float* slices, const int32_t* sched, void* expert_out,
                                   const int64_t* ids, void* const* inbox_ptrs,
                                   void* const* progress_ptrs, void* output, uint32_t* status,
                                   size_t slice_elems, int cap_tokens, int num_tokens, int top_k,
                                   int hidden, int experts_per_rank, int world, int rank,
                                   int first_token, int out_tokens, int tokens_per_rank,
                                   uint32_t epoch, unsigned long long wait_limit_ns,
                                   unsigned long long* trace, bool pdl, cudaStream_t stream);
cudaError_t launch_router_topk(const void* logits, bool logits_f32, int num_tokens,
                               int num_experts, int top_k, int64_t* ids, void* weights_bf16,
                               float* weights_f32, cudaStream_t stream);

extern int g_gemm_stage_kb;
extern int g_gemm_evict_first;

namespace {

int g_l2_promotion = 2;  // 0 none, 1 128 B, 2 256 B
int g_down_target = 0;   // blocks the down projection's split-K aims at (0: 2 per SM)

int g_gemm_overlap = -1;    // BF16 forward: down takes over from gate+up segment by segment (-1: rule)
int g_nvfp4_prefetch = 8;   // NVFP4 GEMMs: weight slots requested before the wait for the previous kernel
int g_nvfp4_issuers = 2;    // NVFP4 gate+up: threads issuing MMAs (1 or 2)
int g_fp8_seg_rows = kSegRowsFp8;  // segment length of the FP8-weight path (16, 32, 48 or 64)
int g_down_splits = 0;   // forced split-K factor of the down projection (0: chosen on the device)
int g_small_call_max = -1;  // most assignments that run in small-call order (0: never; -1: default rule)

int down_target(int sm_count) { return g_down_target > 0 ? g_down_target : 2 * sm_count; }
// what the routing kernel receives: the target, or minus the forced split factor
int down_split_request(int sm_count) {
  return g_down_splits > 0 ? -g_down_splits : down_target(sm_count);
}

constexpr int kMaxDevices = 64;
// The NVFP4 kernels are compiled in and pass their parity tests on a B200 (tests/test_gpu_nvfp4.py).
// With 0 the capability probe answers 0 and b300_moe_forward(backend="cutlass_nvfp4") fails
// loudly, as the reference's backend of that name always does.
constexpr int kNvfp4Ready = 1;

struct DeviceInfo {
  bool probed = false;
  int cc_major = 0, cc_minor = 0, sm_count = 0;
};
DeviceInfo g_devices[kMaxDevices];
std::mutex g_mutex;
PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
bool g_encode_probed = false;

// Properties of the current device, probed once per device.
int current_device_info(DeviceInfo* out) {
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return (int)err;
  if (dev < 0 || dev >= kMaxDevices) return B200MOE_E_ARCH;
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceInfo& info = g_devices[dev];
  if (!info.probed) {
    err = cudaDeviceGetAttribute(&info.cc_major, cudaDevAttrComputeCapabilityMajor, dev);
    if (err != cudaSuccess) return (int)err;
    err = cudaDeviceGetAttribute(&info.cc_minor, cudaDevAttrComputeCapabilityMinor, dev);
    if (err != cudaSuccess) return (int)err;
    err = cudaDeviceGetAttribute(&info.sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (err != cudaSuccess) return (int)err;
    info.probed = true;
  }
  *out = info;
  // The cubin is sm_100a: architecture-specific, it runs on CC 10.0 only.
  if (info.cc_major != 10 || info.cc_minor != 0) return B200MOE_E_ARCH;
  return 0;
}

int resolve_encoder() {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_encode_probed) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (err == cudaSuccess && q == cudaDriverEntryPointSuccess)
      g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
    g_encode_probed = true;
  }
  return g_encode ? 0 : B200MOE_E_DRIVER;
}

// Tensor map of BF16 (or, with `bytes`, one-byte) elements, innermost dimension first,
// 128-byte swizzle, zero fill outside the tensor.  `dims`/`box` have `rank` entries.
int encode_map(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
               const uint32_t* box, bool bytes) {
  int rc = resolve_encoder();
  if (rc) return rc;
  cuuint64_t gdim[5];
  cuuint64_t gstride[4];
  cuuint32_t bdim[5];
  cuuint32_t estride[5];
  uint64_t stride = bytes ? 1 : sizeof(__nv_bfloat16);
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estride[i] = 1;
    stride *= dims[i];
    if (i + 1 < rank) gstride[i] = stride;
  }
  const CUtensorMapL2promotion promotion =
      g_l2_promotion == 0 ? CU_TENSOR_MAP_L2_PROMOTION_NONE
                          : (g_l2_promotion == 1 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B
                                                 : CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
  CUresult r = g_encode(map, bytes ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                        (cuuint32_t)rank,
                        const_cast<void*>(base), gdim, gstride, bdim, estride,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        promotion, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : B200MOE_E_DRIVER;
}

int encode_bf16_map(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                    const uint32_t* box) {
  return encode_map(map, base, rank, dims, box, false);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// `local_experts`: `experts` is one rank's share of a larger layer, so top_k may exceed it.
int check_shape(int tokens, int top_k, int experts, int hidden, int inter,
                bool local_experts = false) {
  if (tokens < 1 || hidden < 1 || inter < 1 || experts < 1) return B200MOE_E_SHAPE;
  if (!(top_k == 1 || top_k == 2 || top_k == 4 || top_k == 8)) return B200MOE_E_SHAPE;
  if (experts > B200MOE_MAX_EXPERTS || (top_k > experts && !local_experts))
    return B200MOE_E_SHAPE;
  if ((long long)tokens * top_k > (1ll << 24)) return B200MOE_E_SHAPE;
  if (hidden % 8 || inter % 8) return B200MOE_E_ALIGN;
  return 0;
}

// Upper bound on the number of segments `rows` assignments can produce.
int segment_bound(int rows, int experts, int seg_rows = kSegRows) {
  return (rows < experts ? rows : experts) + rows / seg_rows;
}

bool fp8_weights(const B200MoeArgs* a) { return (a->flags & B200MOE_FLAG_FP8_WEIGHTS) != 0; }
bool nvfp4_weights(const B200MoeArgs* a) { return (a->flags & B200MOE_FLAG_NVFP4_WEIGHTS) != 0; }


int tiles128(int n) { return (n + 127) / 128; }

struct Scratch {
  uint32_t* status;
  int32_t* sched;
  void* act_lo;
  float* partials;
  uint8_t* q_planes;   // FP8-weight path: token operand as three E4M3 planes
  float* x_scale;
  float* a_scale;
  uint32_t* a_amax;
};

// NVFP4 path: the token planes and the per-tile activation maxima share the scratch bytes of
// the FP8 path's planes (4 planes of W / 2 bytes per row, then one float per row and 128
// columns of I, with W = max(H, I): at most 2.04 of the 3 bytes per element that region holds).
float* nvfp4_tile_amax(const Scratch& s, int rows_cap, int hidden, int inter) {
  const size_t widest = (size_t)(hidden > inter ? hidden : inter);
  return reinterpret_cast<float*>(s.q_planes + 2 * (size_t)rows_cap * widest);
}

int carve_scratch(void* scratch, size_t scratch_bytes, int rows_cap, int experts, int hidden,
                  int inter, Scratch* out) {
  if (!scratch) return B200MOE_E_NULL;
  if (reinterpret_cast<uintptr_t>(scratch) % kScratchAlign) return B200MOE_E_ALIGN;
  const ScratchLayout l = scratch_layout(rows_cap, experts, hidden, inter);
  if (scratch_bytes < l.total) return B200MOE_E_SCRATCH;
  char* b = static_cast<char*>(scratch);
  out->status = reinterpret_cast<uint32_t*>(b + l.status);
  out->sched = reinterpret_cast<int32_t*>(b + l.sched);
  out->act_lo = b + l.act_lo;
  out->partials = reinterpret_cast<float*>(b + l.partials);
  out->q_planes = reinterpret_cast<uint8_t*>(b + l.q_planes);
  out->x_scale = reinterpret_cast<float*>(b + l.x_scale);
  out->a_scale = reinterpret_cast<float*>(b + l.a_scale);
  out->a_amax = reinterpret_cast<uint32_t*>(b + l.a_amax);
  return 0;
}

// Grid of the down projection.  The routing kernel picks the split-K factor from the number
// of segments and rows it finds, so the grid is sized for the worst case over every possible
// segment count and row average.  Remembered per thread: a decode loop asks for the same geometry every step.
int down_grid(int bound, int tiles, int kblocks, int sm_count) {
  if (g_down_splits > 0) return bound * tiles * g_down_splits;
  struct Memo { int bound, tiles, kblocks, target, grid; };
  constexpr int kMemo = 16;  // a decode loop cycles through a handful of token counts
  static thread_local Memo memo[kMemo] = {};
  static thread_local int next = 0;
  const int target = down_target(sm_count);
  for (int i = 0; i < kMemo; ++i) {
    const Memo& m = memo[i];
    if (m.grid > 0 && m.bound == bound && m.tiles == tiles && m.kblocks == kblocks &&
        m.target == target)
      return m.grid;
  }
  int worst = bound * tiles;
  // the model never splits at or above four waves of units: segment counts beyond that
  // cannot raise the bound above bound * tiles
  const int last = std::min(bound, 4 * target / (tiles > 0 ? tiles : 1) + 1);
  for (int segs = 1; segs <= last; ++segs) {
    for (int rows16 = 16; rows16 <= kSegRows; rows16 += 16) {
      const int n = segs * tiles * choose_down_splits(segs * tiles, target, kblocks, rows16);
      if (n > worst) worst = n;
    }
  }
  memo[next] = {bound, tiles, kblocks, target, worst};
  next = (next + 1) % kMemo;
  return worst;
}

// `after_gate_up`: the forward runs in small-call order (see b200moe_forward).
int do_routing(const B200MoeArgs* a, const Scratch& s, const DeviceInfo& dev,
               cudaStream_t stream, bool after_gate_up = false, bool pdl = false) {
  const bool local = (a->flags & B200MOE_FLAG_LOCAL_EXPERTS) != 0;
  return (int)launch_routing(a->expert_indices, a->expert_weights, a->num_tokens * a->top_k,
                             a->top_k, a->num_experts, a->expert_counts, a->expert_offsets,
                             a->reverse_mapping, a->permutation, a->expert_offsets_i32,
                             a->permuted_token_indices, a->permuted_expert_indices,
                             a->permuted_weights, s.sched, s.status, tiles128(a->hidden_size),
                             nvfp4_weights(a) ? (a->intermediate_size + 255) / 256
                             : fp8_weights(a) ? (a->intermediate_size + 127) / 128
                                              : (a->intermediate_size + 63) / 64,
                             down_split_request(dev.sm_count),
                             nvfp4_weights(a) ? kSegRowsNvfp4
                             : fp8_weights(a) ? g_fp8_seg_rows : kSegRows,
                             local ? a->expert_id_base : 0, local,
                             static_cast<const uint32_t*>(a->ep_wait_flags), a->ep_world,
                             a->ep_epoch,
                             (a->ep_wait_limit_us ? (unsigned long long)a->ep_wait_limit_us
                                                  : 1000000ull) * 1000ull,
                             after_gate_up, pdl,
                             (a->flags & B200MOE_FLAG_EP_AFTER_PUSH) != 0 &&
                                 (a->flags & B200MOE_FLAG_PDL) != 0,
                             after_gate_up ? a->permuted_hidden : nullptr, a->hidden_size / 8,
                             stream);
}

int do_gate_up(const void* x, const void* w, int rows_cap, int assignments, int experts,
               int hidden, int inter, void* act_hi, const Scratch& s, const SmallCall* small,
               bool overlap, const DeviceInfo& dev, bool pdl, cudaStream_t stream) {
  CUtensorMap map_w, map_x, map_hidden;
  {
    const uint64_t dims[4] = {(uint64_t)hidden, (uint64_t)inter, 2, (uint64_t)experts};
    const uint32_t box[4] = {64, 128, 2, 1};  // 128 gate rows + the 128 matching up rows
    int rc = encode_bf16_map(&map_w, w, 4, dims, box);
    if (rc) return rc;
  }
  const int grid = segment_bound(assignments, experts) * tiles128(inter);
  {
    const uint64_t dims[2] = {(uint64_t)hidden, (uint64_t)rows_cap};
    const uint32_t box[2] = {64, 16};
    int rc = encode_bf16_map(&map_x, x, 2, dims, box);
    if (rc) return rc;
  }
  if (small) {
    // hidden_states [T,H] with one-row boxes: the blocks fetch their token rows from here
    const uint64_t dims[2] = {(uint64_t)hidden, (uint64_t)(assignments / small->top_k)};
    const uint32_t box[2] = {64, 1};
    int rc = encode_bf16_map(&map_hidden, small->hidden, 2, dims, box);
    if (rc) return rc;
  }
  return (int)launch_gate_up(map_w, map_x, small ? &map_hidden : nullptr, s.sched,
                             max_segments(rows_cap, experts), s.status, act_hi, s.act_lo, inter,
                             hidden, rows_cap, grid, small, overlap ? 1 : 0, dev.sm_count, pdl,
                             stream);
}

int do_down(const void* act_hi, const void* w, int rows_cap, int assignments, int experts,
            int hidden, int inter, const Scratch& s, const SmallCall* small, bool overlap,
            const DeviceInfo& dev, bool pdl, cudaStream_t stream) {
  CUtensorMap map_w, map_hi, map_lo;
  {
    const uint64_t dims[3] = {(uint64_t)inter, (uint64_t)hidden, (uint64_t)experts};
    const uint32_t box[3] = {64, 128, 1};
    int rc = encode_bf16_map(&map_w, w, 3, dims, box);
    if (rc) return rc;
  }
  const uint64_t dims[2] = {(uint64_t)inter, (uint64_t)rows_cap};
  const uint32_t box[2] = {64, 16};
  int rc = encode_bf16_map(&map_hi, act_hi, 2, dims, box);
  if (rc) return rc;
  rc = encode_bf16_map(&map_lo, s.act_lo, 2, dims, box);
  if (rc) return rc;
  const int grid = down_grid(segment_bound(assignments, experts), tiles128(hidden),
                             (inter + 63) / 64, dev.sm_count);
  return (int)launch_down(map_w, map_hi, map_lo, s.sched, max_segments(rows_cap, experts),
                          s.status, s.partials, hidden, inter, rows_cap, grid, small,
                          overlap ? 1 : 0, dev.sm_count, pdl, stream);
}

// FP8 weights: one-byte tensor maps of the weights and of the token planes.
int encode_plane_map(CUtensorMap* map, const uint8_t* planes, int cols, int rows_cap,
                     int num_planes) {
  const uint64_t dims[3] = {(uint64_t)cols, (uint64_t)rows_cap, (uint64_t)num_planes};
  const uint32_t box[3] = {128, 16, 1};
  return encode_map(map, planes, 3, dims, box, true);
}

int do_gate_up_fp8(const void* w, const float* row_scale, int rows_cap, int assignments,
                   int experts, int hidden, int inter, void* act_hi, const Scratch& s,
                   const DeviceInfo& dev, bool pdl, cudaStream_t stream) {
  CUtensorMap map_w, map_x;
  {
    const uint64_t dims[4] = {(uint64_t)hidden, (uint64_t)inter, 2, (uint64_t)experts};
    const uint32_t box[4] = {128, 128, 2, 1};  // 128 gate rows + the 128 matching up rows
    int rc = encode_map(&map_w, w, 4, dims, box, true);
    if (rc) return rc;
  }
  int rc = encode_plane_map(&map_x, s.q_planes, hidden, rows_cap, kFp8PlanesHidden);
  if (rc) return rc;
  const int grid = segment_bound(assignments, experts, g_fp8_seg_rows) * tiles128(inter);
  return (int)launch_gate_up_fp8(map_w, map_x, s.sched, max_segments(rows_cap, experts),
                                 s.status, act_hi, s.act_lo, s.a_amax,
                                 row_scale, s.x_scale, inter, hidden, rows_cap, grid,
                                 dev.sm_count, pdl, stream);
}

int do_down_fp8(const void* act_hi, const void* w, const float* row_scale, int rows_cap,
                int assignments, int experts, int hidden, int inter, const Scratch& s,
                const DeviceInfo& dev, bool pdl, cudaStream_t stream) {
  CUtensorMap map_w, map_act;
  {
    const uint64_t dims[3] = {(uint64_t)inter, (uint64_t)hidden, (uint64_t)experts};
    const uint32_t box[3] = {128, 128, 1};
    int rc = encode_map(&map_w, w, 3, dims, box, true);
    if (rc) return rc;
  }
  int rc = encode_plane_map(&map_act, s.q_planes, inter, rows_cap, kFp8Planes);
  if (rc) return rc;
  const int grid = down_grid(segment_bound(assignments, experts, g_fp8_seg_rows),
                             tiles128(hidden), (inter + 127) / 128, dev.sm_count);
  // the activation rows become planes (in the bytes the gathered rows occupied), then the GEMM
  rc = (int)launch_act_planes_fp8(act_hi, s.act_lo, s.a_amax, s.q_planes, s.a_scale, assignments,
                                  inter, rows_cap, pdl, stream);
  if (rc) return rc;
  return (int)launch_down_fp8(map_w, map_act, s.sched, max_segments(rows_cap, experts),
                              s.status, s.partials, row_scale,
                              s.a_scale, hidden, inter, rows_cap, grid, dev.sm_count, pdl,
                              stream);
}

// NVFP4 weights: byte tensor maps of the packed weights (two elements per byte) and of the
// token planes; scales travel outside the tensor maps.
int do_gate_up_nvfp4(const B200MoeArgs* a, const Scratch& s, int assignments,
                     const DeviceInfo& dev, bool pdl, cudaStream_t stream) {
  const int hidden = a->hidden_size, inter = a->intermediate_size, experts = a->num_experts;
  CUtensorMap map_w, map_x;
  {
    const uint64_t dims[4] = {(uint64_t)hidden / 2, (uint64_t)inter, 2, (uint64_t)experts};
    const uint32_t box[4] = {128, 128, 1, 1};  // 128 gate rows or the 128 matching up rows
    int rc = encode_map(&map_w, a->gate_up_weight, 4, dims, box, true);
    if (rc) return rc;
  }
  int rc = encode_plane_map(&map_x, s.q_planes, hidden / 2, a->rows_cap, kNvfp4Planes);
  if (rc) return rc;
  const int grid = segment_bound(assignments, experts, kSegRowsNvfp4) * tiles128(inter);
  return (int)launch_gate_up_nvfp4(
      map_w, map_x, s.sched, max_segments(a->rows_cap, experts), s.status, a->swiglu_output,
      s.act_lo, nvfp4_tile_amax(s, a->rows_cap, hidden, inter),
      static_cast<const uint8_t*>(a->gate_up_block_scale), a->gate_up_scale, s.x_scale, inter,
      hidden, a->rows_cap, grid, dev.sm_count, g_nvfp4_prefetch, g_nvfp4_issuers, pdl, stream);
}

int do_down_nvfp4(const B200MoeArgs* a, const Scratch& s, int assignments, const DeviceInfo& dev,
                  bool pdl, cudaStream_t stream) {
  const int hidden = a->hidden_size, inter = a->intermediate_size, experts = a->num_experts;
  CUtensorMap map_w, map_act;
  {
    const uint64_t dims[3] = {(uint64_t)inter / 2, (uint64_t)hidden, (uint64_t)experts};
    const uint32_t box[3] = {128, 128, 1};
    int rc = encode_map(&map_w, a->down_weight, 3, dims, box, true);
    if (rc) return rc;
  }
  int rc = encode_plane_map(&map_act, s.q_planes, inter / 2, a->rows_cap, kNvfp4Planes);
  if (rc) return rc;
  const int grid = down_grid(segment_bound(assignments, experts, kSegRowsNvfp4),
                             tiles128(hidden), (inter + 255) / 256, dev.sm_count);
  // the activation rows become planes (in the bytes the gathered rows' planes occupied)
  rc = (int)launch_act_planes_nvfp4(a->swiglu_output, s.act_lo,
                                    nvfp4_tile_amax(s, a->rows_cap, hidden, inter), s.q_planes,
                                    s.a_scale, assignments, inter, a->rows_cap, pdl, stream);
  if (rc) return rc;
  return (int)launch_down_nvfp4(map_w, map_act, s.sched, max_segments(a->rows_cap, experts),
                                s.status, s.partials,
                                static_cast<const uint8_t*>(a->down_block_scale), a->down_scale,
                                s.a_scale, hidden, inter, a->rows_cap, grid, dev.sm_count,
                                g_nvfp4_prefetch, g_nvfp4_issuers, pdl, stream);
}

// geometry and pointers the NVFP4 path needs on top of the common checks
int check_nvfp4(const B200MoeArgs* a) {
  if (!a->gate_up_scale || !a->down_scale || !a->gate_up_block_scale || !a->down_block_scale)
    return B200MOE_E_NULL;
  if (a->hidden_size % 64 || a->intermediate_size % 64) return B200MOE_E_ALIGN;
  if (!aligned16(a->gate_up_block_scale) || !aligned16(a->down_block_scale))
    return B200MOE_E_ALIGN;
  if (fp8_weights(a)) return B200MOE_E_SHAPE;
  return 0;
}

unsigned long long* trace_of(const Scratch& s) {
  return reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(s.status) +
                                               kTraceOffsetBytes);
}

struct Ctx {
  DeviceInfo dev;
  Scratch s;
  int assignments;
  bool pdl;
  cudaStream_t stream;
};

// Checks shared by every stage: geometry, device, scratch region.
int prepare(const B200MoeArgs* a, void* stream, Ctx* c) {
  if (!a) return B200MOE_E_NULL;
  int rc = check_shape(a->num_tokens, a->top_k, a->num_experts, a->hidden_size,
                       a->intermediate_size, (a->flags & B200MOE_FLAG_LOCAL_EXPERTS) != 0);
  if (rc) return rc;
  if ((a->flags & B200MOE_FLAG_LOCAL_EXPERTS) && a->expert_id_base < 0) return B200MOE_E_SHAPE;
  if (a->ep_wait_flags && (a->ep_world < 1 || a->ep_world > B200MOE_EP_MAX_WORLD))
    return B200MOE_E_SHAPE;
  c->assignments = a->num_tokens * a->top_k;
  if (a->rows_cap < c->assignments) return B200MOE_E_SHAPE;
  rc = current_device_info(&c->dev);
  if (rc) return rc;
  rc = carve_scratch(a->scratch, a->scratch_bytes, a->rows_cap, a->num_experts, a->hidden_size,
                     a->intermediate_size, &c->s);
  if (rc) return rc;
  c->pdl = (a->flags & B200MOE_FLAG_PDL) != 0;
  c->stream = static_cast<cudaStream_t>(stream);
  return 0;
}

int stage_routing(const B200MoeArgs* a, const Ctx& c, bool after_gate_up = false,
                  bool pdl = false) {
  if (!a->expert_indices || !a->expert_counts || !a->expert_offsets || !a->expert_offsets_i32 ||
      !a->permutation || !a->reverse_mapping)
    return B200MOE_E_NULL;
  return do_routing(a, c.s, c.dev, c.stream, after_gate_up, pdl);
}

// Small-call order applies to BF16 weights, device-resident per-step tensors and ids that
// are in place when the forward is enqueued (not pushed by peers during it).
// Default rule: T * top_k <= 32 and top_k <= 4.  With top_k = 8 the same number of
// assignments means four times as many one-row segments, each of whose blocks repeats the
// routing vote and whose first tile copies a row: measured 0-3 us slower than the five-launch
// order (H = I = 2880 and H = 7168 / I = 2048 layers, T = 1...4), against 1-4 us faster for
// top_k = 2.
bool small_call(const B200MoeArgs* a, int assignments) {
  int most = kSmallCallMaxAssign;
  if (g_small_call_max >= 0) most = g_small_call_max < most ? g_small_call_max : most;
  else if (a->top_k > 4) return false;
  return assignments <= most && !fp8_weights(a) && !nvfp4_weights(a) &&
         a->ep_wait_flags == nullptr &&
         (a->flags & B200MOE_FLAG_HOST_IO) == 0;
}

SmallCall small_call_of(const B200MoeArgs* a, const Ctx& c) {
  SmallCall sc;
  sc.ids = a->expert_indices;
  sc.num_assign = c.assignments;
  sc.num_experts = a->num_experts;
  sc.id_base = (a->flags & B200MOE_FLAG_LOCAL_EXPERTS) ? a->expert_id_base : 0;
  sc.top_k = a->top_k;
  sc.hidden = a->hidden_states;
  sc.permuted_hidden = a->permuted_hidden;
  sc.split_request = down_split_request(c.dev.sm_count);
  return sc;
}

int stage_gather(const B200MoeArgs* a, const Ctx& c, bool pdl) {
  if (!a->hidden_states || !a->permutation || !a->permuted_hidden) return B200MOE_E_NULL;
  if (!aligned16(a->hidden_states) || !aligned16(a->permuted_hidden)) return B200MOE_E_ALIGN;
  if (nvfp4_weights(a)) {
    if (a->hidden_size % 64 || a->intermediate_size % 64) return B200MOE_E_ALIGN;
    return (int)launch_gather_nvfp4(
        a->hidden_states, a->permutation, a->permuted_hidden, c.s.q_planes, c.s.x_scale,
        c.assignments, a->num_tokens, a->top_k, a->hidden_size, a->rows_cap, trace_of(c.s), pdl,
        c.stream);
  }
  if (fp8_weights(a))
    return (int)launch_gather_fp8(a->hidden_states, a->permutation, a->permuted_hidden,
                                  c.s.q_planes, c.s.x_scale, c.s.a_amax, c.assignments,
                                  a->num_tokens, a->top_k, a->hidden_size, a->rows_cap,
                                  trace_of(c.s), pdl, c.stream);
  return (int)launch_gather(a->hidden_states, a->permutation, a->permuted_hidden, c.assignments,
                            a->num_tokens, a->top_k, a->hidden_size, trace_of(c.s), pdl, c.stream);
}

int stage_gate_up(const B200MoeArgs* a, const Ctx& c, bool pdl, const SmallCall* small = nullptr,
                  bool overlap = false) {
  if (!a->permuted_hidden || !a->gate_up_weight || !a->swiglu_output) return B200MOE_E_NULL;
  if (!aligned16(a->permuted_hidden) || !aligned16(a->gate_up_weight) ||
      !aligned16(a->swiglu_output))
    return B200MOE_E_ALIGN;
  if (nvfp4_weights(a)) {
    int rc = check_nvfp4(a);
    return rc ? rc : do_gate_up_nvfp4(a, c.s, c.assignments, c.dev, pdl, c.stream);
  }
  if (fp8_weights(a)) {
    if (!a->gate_up_scale) return B200MOE_E_NULL;
    if (a->hidden_size % 16 || a->intermediate_size % 16) return B200MOE_E_ALIGN;
    return do_gate_up_fp8(a->gate_up_weight, a->gate_up_scale, a->rows_cap, c.assignments,
                          a->num_experts, a->hidden_size, a->intermediate_size,
                          a->swiglu_output, c.s, c.dev, pdl, c.stream);
  }
  return do_gate_up(a->permuted_hidden, a->gate_up_weight, a->rows_cap, c.assignments,
                    a->num_experts, a->hidden_size, a->intermediate_size, a->swiglu_output, c.s,
                    small, overlap, c.dev, pdl, c.stream);
}

int stage_down(const B200MoeArgs* a, const Ctx& c, bool pdl, const SmallCall* small = nullptr,
               bool overlap = false) {
  if (!a->swiglu_output || !a->down_weight) return B200MOE_E_NULL;
  if (!aligned16(a->swiglu_output) || !aligned16(a->down_weight)) return B200MOE_E_ALIGN;
  if (nvfp4_weights(a)) {
    int rc = check_nvfp4(a);
    return rc ? rc : do_down_nvfp4(a, c.s, c.assignments, c.dev, pdl, c.stream);
  }
  if (fp8_weights(a)) {
    if (!a->down_scale) return B200MOE_E_NULL;
    if (a->hidden_size % 16 || a->intermediate_size % 16) return B200MOE_E_ALIGN;
    return do_down_fp8(a->swiglu_output, a->down_weight, a->down_scale, a->rows_cap,
                       c.assignments, a->num_experts, a->hidden_size, a->intermediate_size, c.s,
                       c.dev, pdl, c.stream);
  }
  return do_down(a->swiglu_output, a->down_weight, a->rows_cap, c.assignments, a->num_experts,
                 a->hidden_size, a->intermediate_size, c.s, small, overlap, c.dev, pdl, c.stream);
}

int stage_combine(const B200MoeArgs* a, const Ctx& c, bool pdl) {
  if (!a->reverse_mapping || !a->expert_weights || !a->output) return B200MOE_E_NULL;
  if (!aligned16(a->output) || (a->expert_output && !aligned16(a->expert_output)))
    return B200MOE_E_ALIGN;
  return (int)launch_combine(a->reverse_mapping, a->expert_weights, c.s.partials, c.s.sched,
                             a->output, a->expert_output, a->num_tokens, a->top_k,
                             a->hidden_size, (size_t)a->rows_cap * a->hidden_size,
                             (a->flags & B200MOE_FLAG_F32_OUTPUT) != 0, trace_of(c.s), pdl,
                             c.stream);
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" {

int b200moe_abi_version(void) { return B200MOE_ABI_VERSION; }

int b200moe_build_info(char* json, size_t cap) {
  char buf[768];
  int n = snprintf(
      buf, sizeof(buf),
      "{\"goal\": \"1B\", \"compiled_architecture\": \"sm_100a\", "
      "\"wrapper_compiled_architecture\": \"sm_100a\", \"uses_fallback\": false, "
      "\"bf16_grouped_gemm_provider\": \"b200moe tcgen05 grouped GEMM (in-tree, hand-written)\", "
      "\"bf16_provider_implementation\": \"tcgen05.mma kind::f16, TMEM accumulators, TMA 128B-swizzle loads\", "
      "\"cutlass_version\": null, \"cuda_runtime_version\": %d, \"nvfp4_compiled\": %s, "
      "\"fp8_weights_compiled\": true, "
      "\"abi_version\": %d, \"segment_rows\": %d, \"down_split_max\": %d}",
      (int)CUDART_VERSION, kNvfp4Ready ? "true" : "false", B200MOE_ABI_VERSION, kSegRows,
      kDownSplitMax);
  if (json && cap > 0) {
    size_t c = (size_t)n < cap - 1 ? (size_t)n : cap - 1;
    memcpy(json, buf, c);
    json[c] = '\0';
  }
  return n;
}

const char* b200moe_error_string(int code) {
  switch (code) {
    case 0: return "success";
    case B200MOE_E_NULL: return "a required pointer is NULL";
    case B200MOE_E_SHAPE: return "unsupported shape (T>=1, K in {1,2,4,8}, K<=E<=256)";
    case B200MOE_E_ALIGN: return "pointers must be 16-byte aligned and H, I divisible by 8";
    case B200MOE_E_SCRATCH: return "scratch region is smaller than b200moe_scratch_bytes()";
    case B200MOE_E_DRIVER: return "cuTensorMapEncodeTiled unavailable or failed";
    case B200MOE_E_ARCH: return "device is not compute capability 10.0 (sm_100a)";
    case B200MOE_E_UNSUPPORTED: return "not implemented (NVFP4 is never substituted by BF16)";
    case B200MOE_E_LIMIT:
      return "the call exceeds a fixed limit of this entry point (b200moe_routing_static: "
             "4096 assignments; b200moe_ep_combine_reduce with B200MOE_FLAG_EP_PUSH: a grid "
             "that is resident at once)";
    default: break;
  }
  if (code > 0) return cudaGetErrorString((cudaError_t)code);
  return "unknown b200moe error";
}

int b200moe_scratch_bytes(int max_tokens, int top_k, int num_experts, int hidden_size,
                          int intermediate_size, size_t* bytes) {
  if (!bytes) return B200MOE_E_NULL;
  int rc = check_shape(max_tokens, top_k, num_experts, hidden_size, intermediate_size);
  if (rc) return rc;
  *bytes = scratch_layout(max_tokens * top_k, num_experts, hidden_size, intermediate_size).total;
  return 0;
}

int b200moe_status_ptr(void* scratch, size_t scratch_bytes, uint32_t** status) {
  if (!scratch || !status) return B200MOE_E_NULL;
  if (scratch_bytes < kStatusBytes) return B200MOE_E_SCRATCH;
  *status = reinterpret_cast<uint32_t*>(scratch);
  return 0;
}

int b200moe_nvfp4_available(void) { return kNvfp4Ready; }

int b200moe_nvfp4_scale_bytes(int rows, int cols, int halves, size_t* bytes_per_expert) {
  if (!bytes_per_expert) return B200MOE_E_NULL;
  if (rows < 1 || cols < 64 || (halves != 1 && halves != 2)) return B200MOE_E_SHAPE;
  if (cols % 64) return B200MOE_E_ALIGN;
  *bytes_per_expert = (size_t)halves * ((rows + 127) / 128) * ((cols + 63) / 64) * 512;
  return 0;
}

int b200moe_nvfp4_quantize(const void* weights_bf16, int num_experts, int rows, int cols,
                           int halves, uint8_t* packed_out, uint8_t* block_scale_out,
                           float* tensor_scale_out, uint32_t* amax_scratch, void* stream) {
  if (!weights_bf16 || !packed_out || !block_scale_out || !tensor_scale_out || !amax_scratch)
    return B200MOE_E_NULL;
  if (num_experts < 1 || num_experts > B200MOE_MAX_EXPERTS || rows < 1 || cols < 64 ||
      (halves != 1 && halves != 2))
    return B200MOE_E_SHAPE;
  if (cols % 64 || !aligned16(weights_bf16) || !aligned16(packed_out) ||
      !aligned16(block_scale_out))
    return B200MOE_E_ALIGN;
  DeviceInfo dev;
  int rc = current_device_info(&dev);
  if (rc) return rc;
  return (int)launch_nvfp4_quantize(weights_bf16, num_experts, rows, cols, halves, packed_out,
                                    block_scale_out, tensor_scale_out, amax_scratch,
                                    static_cast<cudaStream_t>(stream));
}

int b200moe_nvfp4_rows_to_planes(const float* rows_f32, int num_rows, int cols, uint8_t* planes,
                                 float* row_scale, void* stream) {
  if (!rows_f32 || !planes || !row_scale) return B200MOE_E_NULL;
  if (num_rows < 1 || cols < 16) return B200MOE_E_SHAPE;
  if (cols % 16 || !aligned16(planes)) return B200MOE_E_ALIGN;
  DeviceInfo dev;
  int rc = current_device_info(&dev);
  if (rc) return rc;
  return (int)launch_rows_to_planes_nvfp4(rows_f32, num_rows, cols, planes, row_scale,
                                          static_cast<cudaStream_t>(stream));
}

int b200moe_router_topk(const void* logits, int logits_are_f32, int num_tokens, int num_experts,
                        int top_k, int64_t* expert_indices, void* weights_bf16,
                        float* weights_f32, void* stream) {
  if (!logits || !expert_indices) return B200MOE_E_NULL;
  if (num_tokens < 1 || num_experts < 1 || num_experts > B200MOE_MAX_EXPERTS || top_k < 1 ||
      top_k > 8 || top_k > num_experts)
    return B200MOE_E_SHAPE;
  DeviceInfo dev;
  int rc = current_device_info(&dev);
  if (rc) return rc;
  return (int)launch_router_topk(logits, logits_are_f32 != 0, num_tokens, num_experts, top_k,
                                 expert_indices, weights_bf16, weights_f32,
                                 static_cast<cudaStream_t>(stream));
}

int b200moe_fp8_quantize_rows(const void* weights_bf16, long long rows, int cols, uint8_t* q_out,
                              float* scale_out, void* stream) {
  if (!weights_bf16 || !q_out || !scale_out) return B200MOE_E_NULL;
  if (rows < 1 || rows > 0x7fffffffll || cols < 16) return B200MOE_E_SHAPE;
  if (cols % 16 || !aligned16(weights_bf16) || !aligned16(q_out)) return B200MOE_E_ALIGN;
  DeviceInfo dev;
  int rc = current_device_info(&dev);
  if (rc) return rc;
  return (int)launch_fp8_quantize_rows(weights_bf16, rows, cols, q_out, scale_out,
                                       static_cast<cudaStream_t>(stream));
}

int b200moe_fp8_dequantize_rows(const uint8_t* q, const float* scale, long long rows, int cols,
                                void* out_bf16, void* stream) {
  if (!q || !out_bf16) return B200MOE_E_NULL;
  if (rows < 1 || rows > 0x7fffffffll || cols < 16) return B200MOE_E_SHAPE;
  if (cols % 16 || !aligned16(q) || !aligned16(out_bf16)) return B200MOE_E_ALIGN;
  DeviceInfo dev;
  int rc = current_device_info(&dev);
  if (rc) return rc;
  return (int)launch_fp8_dequantize_rows(q, scale, rows, cols, out_bf16,
                                         static_cast<cudaStream_t>(stream));
}

int b200moe_tune(int knob, int value) {
  switch (knob) {
    case B200MOE_TUNE_STAGE_KB:
      if (value < 48 || value > 220) return B200MOE_E_SHAPE;
      g_gemm_stage_kb = value;
      return 0;
    case B200MOE_TUNE_L2_PROMOTION:
      if (value < 0 || value > 2) return B200MOE_E_SHAPE;
      g_l2_promotion = value;
      return 0;
    case B200MOE_TUNE_EVICT_FIRST:
      g_gemm_evict_first = value ? 1 : 0;
      return 0;
    case B200MOE_TUNE_DOWN_TARGET:
      if (value < 0 || value > 4096) return B200MOE_E_SHAPE;
      g_down_target = value;
      return 0;
    case B200MOE_TUNE_DOWN_SPLITS:
      if (value < 0 || value > kDownSplitMax) return B200MOE_E_SHAPE;
      g_down_splits = value;
      return 0;
    case B200MOE_TUNE_FP8_SEG_ROWS:
      if (value < 16 || value > kSegRowsFp8 || value % 16) return B200MOE_E_SHAPE;
      g_fp8_seg_rows = value;
      return 0;
    case B200MOE_TUNE_SMALL_CALL_MAX:
      if (value < -1 || value > kSmallCallMaxAssign) return B200MOE_E_SHAPE;
      g_small_call_max = value;
      return 0;
    case B200MOE_TUNE_GEMM_OVERLAP:
      if (value < -1 || value > 1) return B200MOE_E_SHAPE;
      g_gemm_overlap = value;
      return 0;
    case B200MOE_TUNE_NVFP4_PREFETCH:
      if (value < 0 || value > 8) return B200MOE_E_SHAPE;
      g_nvfp4_prefetch = value;
      return 0;
    case B200MOE_TUNE_NVFP4_ISSUERS:
      if (value < 1 || value > 2) return B200MOE_E_SHAPE;
      g_nvfp4_issuers = value;
      return 0;
    default:
      return B200MOE_E_SHAPE;
  }
}

int b200moe_routing(const B200MoeArgs* a, void* stream) {
  Ctx c;
  int rc = prepare(a, stream, &c);
  return rc ? rc : stage_routing(a, c);
}

int b200moe_routing_static(const B200MoeArgs* a, void* stream) {
  if (!a) return B200MOE_E_NULL;
  if (!a->expert_indices || !a->expert_counts || !a->expert_offsets || !a->expert_offsets_i32 ||
      !a->permutation || !a->reverse_mapping)
    return B200MOE_E_NULL;
  int rc = check_shape(a->num_tokens, a->top_k, a->num_experts, a->hidden_size,
                       a->intermediate_size);
  if (rc) return rc;
  const long long assignments = (long long)a->num_tokens * a->top_k;
  if (assignments > B200MOE_STATIC_ROUTING_MAX_ASSIGNMENTS) return B200MOE_E_LIMIT;
  DeviceInfo dev;
  rc = current_device_info(&dev);
  if (rc) return rc;
  return (int)launch_routing_static(
      a->expert_indices, a->expert_weights, (int)assignments, a->top_k, a->num_experts,
      a->expert_counts, a->expert_offsets, a->reverse_mapping, a->permutation,
      a->expert_offsets_i32, a->permuted_token_indices, a->permuted_expert_indices,
      a->permuted_weights, tiles128(a->hidden_size), (a->intermediate_size + 63) / 64,
      2 * dev.sm_count, static_cast<cudaStream_t>(stream));
}

int b200moe_gather(const B200MoeArgs* a, void* stream) {
  Ctx c;
  int rc = prepare(a, stream, &c);
  return rc ? rc : stage_gather(a, c, false);
}

int b200moe_gate_up_swiglu(const B200MoeArgs* a, void* stream) {
  Ctx c;
  int rc = prepare(a, stream, &c);
  return rc ? rc : stage_gate_up(a, c, false);
}

int b200moe_down(const B200MoeArgs* a, void* stream) {
  Ctx c;
  int rc = prepare(a, stream, &c);
  return rc ? rc : stage_down(a, c, false);
}

int b200moe_combine(const B200MoeArgs* a, void* stream) {
  Ctx c;
  int rc = prepare(a, stream, &c);
  return rc ? rc : stage_combine(a, c, false);
}

int b200moe_ep_reduce(const B200MoeEpReduceArgs* a, void* stream) {
  if (!a || !a->partial_ptrs || !a->flag_ptrs || !a->output) return B200MOE_E_NULL;
  if (a->world < 1 || a->world > B200MOE_EP_MAX_WORLD || a->rank < 0 || a->rank >= a->world ||
      a->num_tokens < 1 || a->hidden_size < 8)
    return B200MOE_E_SHAPE;
  if (a->hidden_size % 8 || !aligned16(a->output)) return B200MOE_E_ALIGN;
  for (int r = 0; r < a->world; ++r) {
    if (!a->partial_ptrs[r] || !a->flag_ptrs[r]) return B200MOE_E_NULL;
    if (!aligned16(a->partial_ptrs[r])) return B200MOE_E_ALIGN;
  }
  DeviceInfo dev;
  int rc = current_device_info(&dev);
  if (rc) return rc;
  const unsigned long long limit_ns =
      (a->wait_limit_us ? (unsigned long long)a->wait_limit_us : 1000000ull) * 1000ull;
  return (int)launch_ep_reduce(a->partial_ptrs, a->flag_ptrs, a->world, a->rank, a->num_tokens,
                               a->hidden_size, a->epoch, limit_ns, a->output, a->status,
                               (a->flags & B200MOE_FLAG_PDL) != 0,
                               static_cast<cudaStream_t>(stream));
}

int b200moe_ep_push_max_blocks(int* blocks) {
  if (!blocks) return B200MOE_E_NULL;
  DeviceInfo dev;
  int rc = current_device_info(&dev);
  if (rc) return rc;
  *blocks = ep_combine_push_resident_blocks(dev.sm_count);
  return 0;
}

int b200moe_ep_combine_reduce(const B200MoeArgs* a, const B200MoeEpReduceArgs* e, void* stream) {
  if (!e || !e->flag_ptrs || !e->output) return B200MOE_E_NULL;
  const bool push = (e->flags & B200MOE_FLAG_EP_PUSH) != 0;
  if (push ? !e->inbox_ptrs : (!e->partial_ptrs || !e->block_counter)) return B200MOE_E_NULL;
  Ctx c;
  int rc = prepare(a, stream, &c);
  if (rc) return rc;
  if (!a->reverse_mapping || !a->expert_weights || !a->expert_indices) return B200MOE_E_NULL;
  if (e->world < 1 || e->world > B200MOE_EP_MAX_WORLD || e->rank < 0 || e->rank >= e->world ||
      e->num_tokens < 1 || e->first_token < 0 ||
      e->first_token + e->num_tokens > a->num_tokens || e->hidden_size != a->hidden_size)
    return B200MOE_E_SHAPE;
  if (!aligned16(e->output) || (a->expert_output && !aligned16(a->expert_output)))
    return B200MOE_E_ALIGN;
  for (int r = 0; r < e->world; ++r) {
    const void* data = push ? e->inbox_ptrs[r] : e->partial_ptrs[r];
    if (!data || !e->flag_ptrs[r]) return B200MOE_E_NULL;
    if (!aligned16(data)) return B200MOE_E_ALIGN;
  }
  const unsigned long long limit_ns =
      (e->wait_limit_us ? (unsigned long long)e->wait_limit_us : 1000000ull) * 1000ull;
  const bool pdl = (e->flags & B200MOE_FLAG_PDL) != 0;
  const int chunks = (a->hidden_size / 8 + 127) / 128;
  const size_t slice_elems = (size_t)a->rows_cap * a->hidden_size;
  if (push) {
    if (e->inbox_cap_tokens < a->num_tokens || e->epoch == 0u) return B200MOE_E_SHAPE;
    if (e->tokens_per_rank < 0 ||
        (e->tokens_per_rank > 0 && (long long)e->tokens_per_rank * e->world < a->num_tokens))
      return B200MOE_E_SHAPE;
    // blocks push before they wait and never wait for their own grid; the grid must still
    // be resident at once so that every rank's pushing blocks get to run
    if ((long long)a->num_tokens * chunks > (long long)ep_combine_push_resident_blocks(c.dev.sm_count))
      return B200MOE_E_LIMIT;
    return (int)launch_ep_combine_push(
        a->reverse_mapping, a->expert_weights, c.s.partials, c.s.sched, a->expert_output,
        a->expert_indices, e->inbox_ptrs, e->flag_ptrs, e->output, e->status, slice_elems,
        e->inbox_cap_tokens, a->num_tokens, a->top_k, a->hidden_size, a->num_experts, e->world,
        e->rank, e->first_token, e->num_tokens, e->tokens_per_rank, e->epoch, limit_ns,
        trace_of(c.s), pdl, c.stream);
  }
  // The fused kernel's blocks wait for other GPUs while the publishing block of their own
  // grid may not have run yet, so it is used only while the whole grid is resident at once
  // (what the occupancy calculation says fits; kernels that share the GPU for a while --
  // the tail of the down projection -- delay blocks but do not depend on them).
  if ((long long)a->num_tokens * chunks <= (long long)ep_combine_reduce_resident_blocks(c.dev.sm_count))
    return (int)launch_ep_combine_reduce(
        a->reverse_mapping, a->expert_weights, c.s.partials, c.s.sched, a->expert_output,
        a->expert_indices, e->partial_ptrs, e->flag_ptrs, e->block_counter, e->output,
        e->status, slice_elems, a->num_tokens, a->top_k, a->hidden_size, a->num_experts,
        e->world, e->rank, e->first_token, e->num_tokens, e->epoch, limit_ns, trace_of(c.s),
        pdl, c.stream);
  // Larger calls: the combine kernel writes this rank's FP32 partial output, then the
  // reduce kernel (whose blocks never depend on blocks of their own grid) adds the ranks'.
  rc = (int)launch_combine(a->reverse_mapping, a->expert_weights, c.s.partials, c.s.sched,
                           const_cast<void*>(e->partial_ptrs[e->rank]), a->expert_output,
                           a->num_tokens, a->top_k, a->hidden_size, slice_elems, true,
                           trace_of(c.s), pdl, c.stream);
  if (rc) return rc;
  const void* shifted[B200MOE_EP_MAX_WORLD];
  for (int r = 0; r < e->world; ++r)
    shifted[r] = static_cast<const char*>(e->partial_ptrs[r]) +
                 (size_t)e->first_token * a->hidden_size * sizeof(float);
  return (int)launch_ep_reduce(shifted, e->flag_ptrs, e->world, e->rank, e->num_tokens,
                               a->hidden_size, e->epoch, limit_ns, e->output, e->status, pdl,
                               c.stream);
}

static size_t dispatch_scratch_need(int rows_cap, int experts) {
  return kStatusBytes +
         sizeof(int32_t) * (kSchedHeaderWords + (size_t)kSchedSegWords * max_segments(rows_cap, experts));
}

int b200moe_dispatch_scratch_bytes(int rows_cap, int num_experts, size_t* bytes) {
  if (!bytes) return B200MOE_E_NULL;
  if (rows_cap < 1 || num_experts < 1 || num_experts > B200MOE_MAX_EXPERTS) return B200MOE_E_SHAPE;
  *bytes = dispatch_scratch_need(rows_cap, num_experts);
  return 0;
}

int b200moe_dispatch(const B200MoeArgs* a, void* stream) {
  if (!a) return B200MOE_E_NULL;
  if (!a->hidden_states || !a->expert_indices || !a->expert_counts || !a->expert_offsets ||
      !a->expert_offsets_i32 || !a->permutation || !a->reverse_mapping || !a->permuted_hidden ||
      !a->scratch)
    return B200MOE_E_NULL;
  int rc = check_shape(a->num_tokens, a->top_k, a->num_experts, a->hidden_size, 8,
                       (a->flags & B200MOE_FLAG_LOCAL_EXPERTS) != 0);
  if (rc) return rc;
  const int assignments = a->num_tokens * a->top_k;
  if (a->rows_cap < assignments) return B200MOE_E_SHAPE;
  if (!aligned16(a->hidden_states) || !aligned16(a->permuted_hidden)) return B200MOE_E_ALIGN;
  if (reinterpret_cast<uintptr_t>(a->scratch) % kScratchAlign) return B200MOE_E_ALIGN;
  const size_t need = dispatch_scratch_need(a->rows_cap, a->num_experts);
  if (a->scratch_bytes < need) return B200MOE_E_SCRATCH;
  Ctx c;
  rc = current_device_info(&c.dev);
  if (rc) return rc;
  char* b = static_cast<char*>(a->scratch);
  c.s.status = reinterpret_cast<uint32_t*>(b);
  c.s.sched = reinterpret_cast<int32_t*>(b + kStatusBytes);
  c.s.act_lo = nullptr;
  c.s.partials = nullptr;
  c.assignments = assignments;
  c.pdl = (a->flags & B200MOE_FLAG_PDL) != 0;
  c.stream = static_cast<cudaStream_t>(stream);
  if ((rc = stage_routing(a, c))) return rc;
  return stage_gather(a, c, c.pdl);
}

int b200moe_combine_bf16(const void* expert_rows, const int64_t* assignment_to_permuted,
                         const void* routing_weights, int num_tokens, int top_k, int hidden_size,
                         void* output, void* stream) {
  if (!expert_rows || !assignment_to_permuted || !routing_weights || !output)
    return B200MOE_E_NULL;
  if (num_tokens < 1 || hidden_size < 8 ||
      !(top_k == 1 || top_k == 2 || top_k == 4 || top_k == 8))
    return B200MOE_E_SHAPE;
  if (hidden_size % 8 || !aligned16(expert_rows) || !aligned16(output)) return B200MOE_E_ALIGN;
  DeviceInfo dev;
  int rc = current_device_info(&dev);
  if (rc) return rc;
  return (int)launch_combine_bf16(expert_rows, assignment_to_permuted, routing_weights, output,
                                  num_tokens, top_k, hidden_size,
                                  static_cast<cudaStream_t>(stream));
}

int b200moe_ep_push(const B200MoeEpPushArgs* a, void* stream) {
  if (!a || !a->hidden_states || !a->expert_indices || !a->expert_weights || !a->hidden_dst ||
      !a->indices_dst || !a->weights_dst || !a->flag_ptrs || !a->block_counter)
    return B200MOE_E_NULL;
  if (a->world < 1 || a->world > B200MOE_EP_MAX_WORLD || a->rank < 0 || a->rank >= a->world ||
      a->tokens_local < 1 || a->top_k < 1 || a->hidden_size < 8)
    return B200MOE_E_SHAPE;
  if (a->hidden_size % 8 || !aligned16(a->hidden_states)) return B200MOE_E_ALIGN;
  for (int r = 0; r < a->world; ++r) {
    if (!a->hidden_dst[r] || !a->indices_dst[r] || !a->weights_dst[r] || !a->flag_ptrs[r])
      return B200MOE_E_NULL;
    if (!aligned16(a->hidden_dst[r])) return B200MOE_E_ALIGN;
  }
  DeviceInfo dev;
  int rc = current_device_info(&dev);
  if (rc) return rc;
  return (int)launch_ep_push(a->hidden_states, a->expert_indices, a->expert_weights,
                             a->hidden_dst, a->indices_dst, a->weights_dst, a->flag_ptrs,
                             a->block_counter, a->world, a->rank, a->tokens_local, a->top_k,
                             a->hidden_size, a->epoch, static_cast<cudaStream_t>(stream));
}

int b200moe_forward(const B200MoeArgs* a, void* stream) {
  Ctx c;
  int rc = prepare(a, stream, &c);
  if (rc) return rc;
  // All pointer checks first, so a contract error launches nothing at all.
  const bool skip_combine = (a->flags & B200MOE_FLAG_SKIP_COMBINE) != 0;
  if (!a->hidden_states || !a->expert_indices || !a->expert_weights || !a->gate_up_weight ||
      !a->down_weight || !a->expert_counts || !a->expert_offsets || !a->expert_offsets_i32 ||
      !a->permutation || !a->reverse_mapping || !a->permuted_hidden || !a->swiglu_output ||
      (!a->output && !skip_combine))
    return B200MOE_E_NULL;
  if (!aligned16(a->hidden_states) || !aligned16(a->gate_up_weight) ||
      !aligned16(a->down_weight) || !aligned16(a->permuted_hidden) ||
      !aligned16(a->swiglu_output) || (!skip_combine && !aligned16(a->output)) ||
      (a->expert_output && !aligned16(a->expert_output)))
    return B200MOE_E_ALIGN;
  if (fp8_weights(a)) {
    if (!a->gate_up_scale || !a->down_scale) return B200MOE_E_NULL;
    if (a->hidden_size % 16 || a->intermediate_size % 16) return B200MOE_E_ALIGN;
  }
  if (nvfp4_weights(a) && (rc = check_nvfp4(a))) return rc;
  if (small_call(a, c.assignments)) {
    // Small-call order: the gate+up GEMM first (its blocks need nothing from the routing
    // kernel and also do the gather), the routing kernel beside it, then down and combine.
    const SmallCall sc = small_call_of(a, c);
    if ((rc = stage_gate_up(a, c, c.pdl, &sc))) return rc;
    if ((rc = stage_routing(a, c, true, c.pdl))) return rc;
    if ((rc = stage_down(a, c, c.pdl, &sc))) return rc;
    return skip_combine ? 0 : stage_combine(a, c, c.pdl);
  }
  // Inside one forward with dependent launches the down projection can take over segment by
  // segment from gate+up (BF16 weights; the quantised paths have a plane pass in between).
  // After such a hand-over the down blocks of the LAST segment run alone, each at what one
  // block can pull from HBM, so it pays only where those blocks are short: I <= H (a down
  // block then streams at most a quarter of a gate+up block's bytes).  Measured: H = 7168,
  // I = 2048, 64 experts: 580 -> 557, 838 -> 817, 844 -> 825 us at T = 8 / 32 / 64;
  // H = I = 2880: 1-2 us of 90-95; Mixtral shape (I = 3.5 H): 0 to +8 us, hence the rule.
  const bool overlap_wanted = g_gemm_overlap < 0 ? a->intermediate_size <= a->hidden_size
                                                 : g_gemm_overlap != 0;
  const bool overlap = c.pdl && overlap_wanted && !fp8_weights(a) && !nvfp4_weights(a);
  if ((rc = stage_routing(a, c))) return rc;
  if ((rc = stage_gather(a, c, c.pdl))) return rc;
  if ((rc = stage_gate_up(a, c, c.pdl, nullptr, overlap))) return rc;
  if ((rc = stage_down(a, c, c.pdl, nullptr, overlap))) return rc;
  return skip_combine ? 0 : stage_combine(a, c, c.pdl);
}

}  // extern "C"
