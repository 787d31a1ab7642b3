/*
 * b200moe.h -- C ABI of libb200moe.so: the explicitly routed SwiGLU MoE decode
 * layer as hand-written sm_100a kernels.
 *
 * Every entry point takes plain device pointers, sizes and an explicit CUDA
 * stream (passed as void* so that C callers need no CUDA headers).  Nothing
 * here allocates device memory, synchronises the stream or reads device memory
 * back to the host unless the comment of the function says so.
 *
 * Return value convention:
 *    0  work was enqueued on the stream
 *   <0  B200MOE_E_* : argument/contract error found on the host, nothing launched
 *   >0  a cudaError_t reported by the CUDA runtime or driver
 *
 * Conditions that can only be seen on the device (an expert id outside
 * [0, E), a pipeline wait that ran out) never trap: they set bits in the
 * caller-provided 32-bit status word and the offending row is dropped.
 *
 * Index conventions (same as the reference, csrc/moe_fastpath.h:9-12):
 *   assignment a = token * top_k + slot          (token-major, slot-minor)
 *   permutation[p]     = a   expert-major row -> assignment  ("permuted_to_assignment")
 *   reverse_mapping[a] = p   assignment -> expert-major row  ("assignment_to_permuted")
 */
#ifndef B200MOE_H_
#define B200MOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200MOE_ABI_VERSION 5

/* host-side contract errors */
#define B200MOE_E_NULL        (-1)  /* a required pointer is NULL */
#define B200MOE_E_SHAPE       (-2)  /* T, K, E, H or I outside the supported range */
#define B200MOE_E_ALIGN       (-3)  /* pointer not 16-byte aligned, or H/I not a multiple of 8 */
#define B200MOE_E_SCRATCH     (-4)  /* scratch region smaller than b200moe_scratch_bytes() */
#define B200MOE_E_DRIVER      (-5)  /* cuTensorMapEncodeTiled could not be resolved / failed */
#define B200MOE_E_ARCH        (-6)  /* current device is not compute capability 10.0 */
#define B200MOE_E_UNSUPPORTED (-7)  /* feature is declared but not implemented (NVFP4) */
#define B200MOE_E_LIMIT       (-8)  /* the call exceeds a fixed limit of the entry point */

/* bits of the device status word */
#define B200MOE_STATUS_BAD_EXPERT_ID  0x1u  /* some expert id was outside [0, E); its row was dropped */
#define B200MOE_STATUS_PIPE_TIMEOUT   0x2u  /* a bounded mbarrier wait inside a GEMM gave up */
#define B200MOE_STATUS_PEER_TIMEOUT   0x4u  /* a bounded wait on an expert-parallel peer flag gave up */

#define B200MOE_MAX_EXPERTS   256   /* same limit as the reference, csrc/routing_kernels.cu:107 */

/* most assignments (T * top_k) b200moe_routing_static() accepts */
#define B200MOE_STATIC_ROUTING_MAX_ASSIGNMENTS 4096

/* flags of B200MoeArgs.flags */
#define B200MOE_FLAG_PDL      0x1u  /* launch kernels 2..5 with programmatic dependent launch */
/* Expert-parallel rank: this call owns experts [expert_id_base, expert_id_base + num_experts)
 * of a larger layer.  Ids outside that range belong to other ranks: their rows are dropped
 * silently (reverse_mapping == -1, no status bit) and contribute nothing to the output. */
#define B200MOE_FLAG_LOCAL_EXPERTS 0x2u
/* `output` is FP32 [T,H]: the combine stores the unrounded sums, so that partial outputs
 * of several ranks can be added before the single BF16 rounding. */
#define B200MOE_FLAG_F32_OUTPUT    0x4u
/* Expert weights are FP8: gate_up_weight / down_weight point to E4M3 bytes ([E,2I,H] and
 * [E,H,I], one byte per element, produced by b200moe_fp8_quantize_rows) and gate_up_scale /
 * down_scale hold one FP32 scale per weight row.  Activations, accumulation and output are
 * as in the BF16 path.  Needs H and I divisible by 16.  No counterpart in the reference,
 * which names quantised expert weights as future work (docs/goal_1b_report.md:313-314);
 * the "cutlass_nvfp4" name keeps failing loudly (b200moe_nvfp4_available() == 0). */
#define B200MOE_FLAG_FP8_WEIGHTS   0x8u
/* hidden_states, expert_indices, expert_weights and output live in pinned host memory that
 * the kernels read and write over PCIe.  b200moe_forward then keeps the regular kernel order
 * (routing, gather, gate+up, down, combine) whatever the size of the call. */
#define B200MOE_FLAG_HOST_IO       0x10u
/* b200moe_forward stops after the down projection: the caller combines the rows itself
 * (b200moe_ep_combine_reduce on an expert-parallel rank).  `output` is not used. */
#define B200MOE_FLAG_SKIP_COMBINE  0x20u
/* Expert weights are NVFP4: gate_up_weight / down_weight point to packed E2M1 elements
 * ([E,2I,H/2] and [E,H,I/2] bytes, two elements per byte, the even one in the low nibble),
 * gate_up_block_scale / down_block_scale to their unsigned-E4M3 block scales (one per 16
 * elements of the reduction dimension, in 512-byte tiles of 128 rows x 4 scales), and
 * gate_up_scale / down_scale to one FP32 scale per expert matrix; all three are produced by
 * b200moe_nvfp4_quantize.  weight = tensor scale * block scale * element.  Activations,
 * accumulation and output are as in the BF16 path.  Needs H and I divisible by 64.  This is
 * what the reference's "cutlass_nvfp4" backend names and never had
 * (csrc/quantization_kernels.cu:3-13).  Not combined with B200MOE_FLAG_FP8_WEIGHTS. */
#define B200MOE_FLAG_NVFP4_WEIGHTS 0x80u
/* With ep_wait_flags and B200MOE_FLAG_PDL: the kernel in front of this call in its stream is
 * the b200moe_ep_push of the same step, launched without any launch attribute.  The routing
 * kernel, which waits for every rank's dispatch flag (this rank's own included) before it
 * reads anything the dispatch writes, may then start while that kernel is still running
 * (programmatic dependent launch) instead of after its completion.  Only for that
 * situation: with any other kernel in front, the routing kernel could overwrite what an
 * earlier forward's last kernel still reads. */
#define B200MOE_FLAG_EP_AFTER_PUSH 0x100u
/* With B200MOE_FLAG_FP8_WEIGHTS the staged entry points keep their meaning, with two
 * details: b200moe_gather also writes the gathered rows as E4M3 planes into scratch, which
 * b200moe_gate_up_swiglu consumes; b200moe_down first turns the activation rows into planes
 * in the same scratch bytes (one extra launch inside the call), so after it the planes of
 * stage 2 are gone and stage 3 cannot be repeated without repeating stage 2. */

/* ABI version of the loaded library (== B200MOE_ABI_VERSION it was built with). */
int b200moe_abi_version(void);

/*
 * Writes a NUL-terminated JSON object describing the build into `json`
 * (at most `cap` bytes) and returns the length that was needed.  Keys mirror
 * the reference's build_info() dict (csrc/bindings.cpp:63-85):
 * compiled_architecture ("sm_100a"), uses_fallback (false),
 * bf16_grouped_gemm_provider, cuda_runtime_version, nvfp4_compiled (false), ...
 */
int b200moe_build_info(char* json, size_t cap);

/* Human-readable text for a negative B200MOE_E_* code; cudaGetErrorString for positive ones. */
const char* b200moe_error_string(int code);

/*
 * Bytes of private scratch the layer needs, beyond the reference's twelve
 * public workspace buffers, for up to `max_tokens` tokens: the FP32 split-K
 * partial rows of the down projection, the low-order halves of the SwiGLU
 * activations, the device-built segment schedule and the status word.
 * Replaces the hidden allocations ATen's grouped GEMM makes per call in the
 * reference (csrc/grouped_gemm_sm103.cu:47-52).
 */
int b200moe_scratch_bytes(int max_tokens, int top_k, int num_experts,
                          int hidden_size, int intermediate_size, size_t* bytes);

/*
 * Arguments of the layer.  Every stage entry point takes the same struct, so
 * the scratch region is carved identically by all of them; each stage reads
 * only the fields its comment names.
 */
typedef struct B200MoeArgs {
  /* inputs */
  const void*    hidden_states;      /* [T,H]     bf16 */
  const int64_t* expert_indices;     /* [T,K]     int64 */
  const void*    expert_weights;     /* [T,K]     bf16 */
  const void*    gate_up_weight;     /* [E,2I,H]  bf16, gate rows first */
  const void*    down_weight;        /* [E,H,I]   bf16 */
  int32_t num_tokens, top_k, num_experts, hidden_size, intermediate_size;
  int32_t rows_cap;                  /* rows of the permuted_* buffers (>= T*K) */
  /* reference workspace buffers (fastpath/b300_moe.py:182-195) */
  int64_t* expert_counts;            /* [E]   */
  int64_t* expert_offsets;           /* [E+1] */
  int32_t* expert_offsets_i32;       /* [E]   cumulative END offsets */
  int64_t* permutation;              /* [rows_cap] */
  int64_t* reverse_mapping;          /* [rows_cap] */
  int64_t* permuted_token_indices;   /* [rows_cap] or NULL */
  int64_t* permuted_expert_indices;  /* [rows_cap] or NULL */
  void*    permuted_weights;         /* [rows_cap] bf16 or NULL */
  void*    permuted_hidden;          /* [rows_cap,H] bf16 */
  void*    swiglu_output;            /* [rows_cap,I] bf16 */
  void*    expert_output;            /* [rows_cap,H] bf16 or NULL */
  /* private scratch, b200moe_scratch_bytes() for rows_cap / top_k tokens, 256-byte aligned */
  void*    scratch;
  size_t   scratch_bytes;
  /* result */
  void*    output;                   /* [T,H] bf16 (fp32 with B200MOE_FLAG_F32_OUTPUT) */
  uint32_t flags;                    /* B200MOE_FLAG_* */
  int32_t  expert_id_base;           /* first global expert id of this rank (B200MOE_FLAG_LOCAL_EXPERTS) */
  /* Expert parallel with sharded tokens: when ep_wait_flags is non-NULL the routing kernel
   * first waits (at most ep_wait_limit_us, 0 = 1 s) until ep_wait_flags[r] >= ep_epoch for
   * r < ep_world, i.e. until every rank's b200moe_ep_push of this forward has landed. */
  const void* ep_wait_flags;         /* uint32[ep_world] on this device, or NULL */
  int32_t  ep_world;
  uint32_t ep_epoch;
  uint32_t ep_wait_limit_us;
  /* B200MOE_FLAG_FP8_WEIGHTS only: dequantised weight = E4M3 value * scale of its row */
  const float* gate_up_scale;        /* [E, 2I] fp32   (NVFP4: [E] fp32, one per expert matrix) */
  const float* down_scale;           /* [E, H]  fp32   (NVFP4: [E] fp32) */
  /* B200MOE_FLAG_NVFP4_WEIGHTS only: block scales as b200moe_nvfp4_quantize lays them out */
  const void* gate_up_block_scale;   /* [E][2][ceil(I/128)][H/64][512] bytes */
  const void* down_block_scale;      /* [E][ceil(H/128)][I/64][512] bytes */
} B200MoeArgs;

/*
 * Stage 1 -- routing metadata.  Replaces routing_metadata_out_cuda
 * (csrc/routing_kernels.cu:79-139) plus the int32 offsets copy
 * (fastpath/b300_moe.py:652-653): histogram, exclusive scan (empty experts
 * keep equal adjacent offsets), stable expert-major permutation and its exact
 * inverse, in one launch.  Also fills permuted_token_indices /
 * permuted_expert_indices / permuted_weights when those pointers are non-NULL,
 * and builds, on the device and with no host synchronisation, the segment
 * schedule the two GEMMs consume.  Clears the status word.
 * Reads: expert_indices, expert_weights.  Writes: the routing buffers, scratch.
 */
int b200moe_routing(const B200MoeArgs* args, void* stream);

/*
 * Stage 1 for callers that cannot allocate device memory.  It has no
 * counterpart in the reference.
 *
 * Some hosts of this library are not allowed to call cudaMalloc when they need
 * routing metadata: an inference server that gave all device memory to its own
 * arena at start-up, or a plugin whose interface forbids allocation after
 * initialisation.  This
 * entry point computes the same counts / offsets / permutation /
 * reverse_mapping (and, when the pointers are non-NULL, the permuted_* arrays)
 * as b200moe_routing, but keeps the few KB of scratch the kernel needs in a
 * fixed 8 KiB array inside the library.  Every GPU that loads the library holds
 * those 8 KiB until the process exits.  args->scratch and args->scratch_bytes
 * are ignored; inputs and outputs are still the caller's buffers.
 *
 * Limits and rules:
 *  - T * top_k must not exceed B200MOE_STATIC_ROUTING_MAX_ASSIGNMENTS (4096);
 *    larger calls return B200MOE_E_LIMIT and launch nothing.
 *  - It calls no cudaMalloc, cudaFree or other allocating routine.
 *  - The first call on each device looks up the array's device address (one
 *    cudaGetSymbolAddress, with that device current).  Make that first call
 *    before any stream capture begins.
 *  - All calls on one device share the one array: calls that may overlap on the
 *    GPU (different streams, different threads) race and must be ordered by the
 *    caller.  Each call clears the state it needs, so back-to-back calls on one
 *    stream are independent of one another.
 *  - The segment schedule stays inside the library, so the GEMM stages cannot
 *    follow this entry point; it serves callers that need the routing tensors.
 *    An expert id outside [0, E) shows up as reverse_mapping == -1 for that
 *    assignment and as a shorter count total (the status word lives in the
 *    library's array, so B200MOE_STATUS_BAD_EXPERT_ID cannot be read back).
 *  - Fields it does not read: scratch, scratch_bytes, flags (in particular
 *    B200MOE_FLAG_LOCAL_EXPERTS and B200MOE_FLAG_FP8_WEIGHTS), expert_id_base,
 *    ep_wait_flags / ep_world / ep_epoch / ep_wait_limit_us.  It always routes the
 *    global id range [0, num_experts) with 128-row segments.
 */
int b200moe_routing_static(const B200MoeArgs* args, void* stream);

/*
 * Stage 2 -- gather.  Replaces permute_out_cuda (csrc/permutation_kernels.cu:72-110):
 * permuted_hidden[p, :] = hidden_states[permutation[p] / K, :] with 16-byte
 * loads and stores; rows whose mapping is invalid are zero-filled exactly like
 * the reference kernel (csrc/permutation_kernels.cu:41-48).
 */
int b200moe_gather(const B200MoeArgs* args, void* stream);

/*
 * Stage 3 -- grouped gate+up GEMM with SwiGLU in the epilogue.  Replaces
 * grouped_gemm_bf16_out_cuda on the [E,2I,H] weight (csrc/grouped_gemm_sm103.cu:21-53)
 * followed by swiglu_out_cuda (csrc/moe_fastpath.cu:24-71):
 *   act[p, i] = silu(x_p . Wgate[e(p), i, :]) * (x_p . Wup[e(p), i, :])
 * accumulated and activated in FP32 (tcgen05 MMA, TMEM accumulators), written
 * as a BF16 high part into swiglu_output and a BF16 low-order remainder into
 * the scratch region, so the down projection sees the FP32 value to ~2^-17.
 * Must run after stage 1 on the same scratch region.
 */
int b200moe_gate_up_swiglu(const B200MoeArgs* args, void* stream);

/*
 * Stage 4 -- grouped down GEMM.  Replaces grouped_gemm_bf16_out_cuda on the
 * [E,H,I] weight (csrc/grouped_gemm_sm103.cu:21-53).  Consumes the high/low
 * activation pair and writes FP32 rows (split-K partial slices, summed in a
 * fixed order by stage 5) into the scratch region.
 */
int b200moe_down(const B200MoeArgs* args, void* stream);

/*
 * Stage 5 -- combine.  Replaces combine_out_cuda (csrc/combine_kernels.cu:55-93):
 *   output[t, :] = bf16( sum_k float(w[t,k]) * row(reverse_mapping[t*K+k]) )
 * FP32 accumulation in slot order, weights used exactly as supplied
 * (unnormalised, negative, zero); invalid rows are skipped like the
 * reference kernel (csrc/combine_kernels.cu:44).  row() is the fixed-order sum
 * of the split-K slices stage 4 wrote.  When expert_output is non-NULL the
 * BF16-rounded expert rows are stored there too, which is what the reference
 * keeps in its expert_output buffer.
 */
int b200moe_combine(const B200MoeArgs* args, void* stream);

/*
 * Stages 1 + 2 on their own: the legacy "dispatch" operation.  Replaces dispatch_cuda
 * (csrc/dispatch_cuda.cu:24-201, bound as fastpath._C.dispatch and used by
 * fastpath/ops.py:150-178): counts, offsets, both mappings and the gathered rows.
 * Needs only the head of a scratch region (status words + schedule), 256-byte aligned;
 * b200moe_dispatch_scratch_bytes gives its size for rows_cap rows and E experts.
 * intermediate_size, swiglu_output, the weights and output are not read.
 */
int b200moe_dispatch(const B200MoeArgs* args, void* stream);
int b200moe_dispatch_scratch_bytes(int rows_cap, int num_experts, size_t* bytes);

/*
 * The legacy "combine" operation on BF16 expert rows.  Replaces combine_cuda
 * (csrc/combine_cuda.cu:23-141, fastpath/ops.py:242-271):
 *   output[t, :] = bf16( sum_k float(w[t,k]) * float(expert_rows[map[t*K+k], :]) )
 * FP32 accumulation in slot order; entries of the mapping outside [0, T*K) are skipped.
 */
int b200moe_combine_bf16(const void* expert_rows /*[T*K,H] bf16*/,
                         const int64_t* assignment_to_permuted /*[T*K]*/,
                         const void* routing_weights /*[T,K] bf16*/, int num_tokens, int top_k,
                         int hidden_size, void* output /*[T,H] bf16*/, void* stream);

/*
 * The whole layer: stages 1..5 enqueued back to back on `stream` by one call.
 * Replaces _call_compiled_bf16 (fastpath/b300_moe.py:620-760).  No allocation,
 * no synchronisation, no host read-back.
 *
 * Kernel order.  Regular: routing, gather, gate+up, down, combine.  A BF16 call with at
 * most 32 assignments (T * top_k) runs in small-call order instead: the gate+up GEMM is
 * the first kernel -- every block finds its work unit from expert_indices with a few warp
 * votes, fetches its token rows from hidden_states itself and, for the first tile of each
 * expert, also writes them to permuted_hidden -- the routing kernel runs beside it, and
 * down and combine follow.  Results and every output buffer are the same in both orders;
 * small-call order takes the routing and gather launches off the critical path.
 */
int b200moe_forward(const B200MoeArgs* args, void* stream);

/*
 * Expert-parallel combine over NVLink peer memory.  No counterpart in the
 * reference, which has no multi-GPU code (README.md:206-207).
 *
 * After its local b200moe_forward (B200MOE_FLAG_LOCAL_EXPERTS |
 * B200MOE_FLAG_F32_OUTPUT, output = this rank's partial buffer), every rank calls
 * this once per layer call with the same `epoch` (1, 2, 3, ...).  The kernel
 * publishes the epoch into flags[rank] of every rank, waits until its own flag
 * array shows the epoch for all ranks (at most wait_limit_us, then
 * B200MOE_STATUS_PEER_TIMEOUT is set in *status and the output is left
 * untouched), then adds the `world` FP32 partial outputs in rank order with plain
 * peer loads and stores BF16 [T,H].
 *
 *   partial_ptrs[world]  device pointers, valid on THIS device, to every rank's
 *                        FP32 [num_tokens, hidden_size] partial buffer
 *   flag_ptrs[world]     device pointers, valid on THIS device, to every rank's
 *                        uint32[world] flag array (zero before the first epoch)
 * Both arrays are read on the host.  Callers alternate two partial buffers by
 * epoch parity so a fast rank never overwrites a buffer a slow rank still reads.
 */
typedef struct B200MoeEpReduceArgs {
  const void* const* partial_ptrs;
  void* const*       flag_ptrs;
  int32_t  world, rank, num_tokens, hidden_size;
  uint32_t epoch;
  uint32_t wait_limit_us;            /* 0 selects the default of 1 s */
  void*    output;                   /* [T,H] bf16 */
  uint32_t* status;                  /* device status word, or NULL */
  uint32_t flags;                    /* B200MOE_FLAG_PDL */
  /* b200moe_ep_combine_reduce only */
  int32_t  first_token;              /* first of the num_tokens rows this rank outputs */
  unsigned int* block_counter;       /* one zero-initialised uint32 in this device's memory */
  /* b200moe_ep_combine_reduce with B200MOE_FLAG_EP_PUSH only */
  void* const* inbox_ptrs;           /* every rank's inbox, valid on THIS device (see below) */
  int32_t  inbox_cap_tokens;         /* tokens one inbox slot holds (>= layer->num_tokens) */
  int32_t  tokens_per_rank;          /* sharded tokens: rank t / tokens_per_rank outputs token t;
                                        0: tokens are replicated, every rank outputs all */
} B200MoeEpReduceArgs;

#define B200MOE_EP_MAX_WORLD 8

int b200moe_ep_reduce(const B200MoeEpReduceArgs* args, void* stream);

/*
 * Stage 5 of an expert-parallel rank: combine and cross-rank reduce in ONE kernel.  No
 * counterpart in the reference.  Follows a b200moe_forward with B200MOE_FLAG_LOCAL_EXPERTS |
 * B200MOE_FLAG_SKIP_COMBINE on the same `layer` arguments (expert_indices holding the
 * GLOBAL ids of all layer->num_tokens tokens, num_experts the experts of this rank).
 *
 * Every block computes this rank's routing-weighted sum for its token from the down
 * projection's FP32 rows (as b200moe_combine does), stores it to this rank's partial
 * buffer only if the rank owns an expert of the token, and the last block publishes
 * `epoch` into flags[rank] of every rank.  Blocks of the rows this rank outputs
 * (first_token .. first_token + num_tokens) then wait, bounded as in b200moe_ep_reduce,
 * until every rank has published, add the partial rows of the ranks that own an expert of
 * the token in rank order -- found from the token's ids, so a token routed to K experts
 * reads at most K rows instead of `world` -- and round once to BF16.  On a timeout the rows
 * are written as zeros and B200MOE_STATUS_PEER_TIMEOUT is set.
 *
 * partial_ptrs[r] is the start of rank r's FP32 [layer->num_tokens, H] buffer (not offset by
 * first_token).  Calls whose grid (T * ceil(H / 1024) blocks) exceeds what the GPU holds at
 * once run as the two separate kernels instead, with the same result.
 */
int b200moe_ep_combine_reduce(const B200MoeArgs* layer, const B200MoeEpReduceArgs* ep,
                              void* stream);

/*
 * B200MOE_FLAG_EP_PUSH in ep->flags selects the low-latency variant of
 * b200moe_ep_combine_reduce: instead of publishing one flag per rank and letting the peers
 * read its partial rows, every block stores its row straight into the inbox of each rank that
 * outputs the token, each 4-byte value together with the 4-byte epoch in one 8-byte word, so
 * that no fence and no flag round trip separate the combine from the peers' sums; receivers
 * poll their own memory.  partial_ptrs and block_counter are not used.
 *   inbox_ptrs[r]   rank r's inbox: 2 * world * inbox_cap_tokens * H words of 8 bytes, zero
 *                   before the first epoch, laid out [epoch parity][source rank][token][H]
 *   flag_ptrs[r]    rank r's uint32[world] array; here it carries progress: every rank stores
 *                   its epoch there when its kernel starts, and a rank waits (bounded) for the
 *                   target's previous epoch before it reuses an inbox slot
 *   epoch           1, 2, 3, ... (never 0), the same on every rank for one layer call
 * One layer instance uses either this variant or the other for all its calls.  The grid
 * (T * ceil(H / 1024) blocks) must be resident at once: larger calls return B200MOE_E_LIMIT
 * (b200moe_ep_push_max_blocks gives the bound for the current device).
 */
#define B200MOE_FLAG_EP_PUSH 0x40u
int b200moe_ep_push_max_blocks(int* blocks);

/*
 * Expert-parallel dispatch of sharded tokens over NVLink peer memory.  No counterpart
 * in the reference.  Every rank holds T/N tokens; one launch stores this rank's token
 * rows, expert ids and routing weights into slot `rank` of every rank's gathered
 * buffers (plain peer stores) and then publishes `epoch` into flags[rank] of every rank.
 * The consumer is the b200moe_forward of the same layer call with ep_wait_flags set.
 *   hidden_dst[r] / indices_dst[r] / weights_dst[r]   device pointers, valid on THIS device,
 *       to where this rank's shard goes inside rank r's gathered [T,H] / [T,K] / [T,K] buffers
 *   flag_ptrs[r]      rank r's dispatch flag array uint32[world]
 *   block_counter     one zero-initialised uint32 in this device's memory
 * The pointer arrays are read on the host.  Alternate two sets of gathered buffers by
 * epoch parity so a fast rank never overwrites what a slow rank still reads.
 */
typedef struct B200MoeEpPushArgs {
  const void*    hidden_states;      /* [T_local,H] bf16 */
  const int64_t* expert_indices;     /* [T_local,K] */
  const void*    expert_weights;     /* [T_local,K] bf16 */
  void* const*   hidden_dst;
  void* const*   indices_dst;
  void* const*   weights_dst;
  void* const*   flag_ptrs;
  unsigned int*  block_counter;
  int32_t  world, rank, tokens_local, top_k, hidden_size;
  uint32_t epoch;
} B200MoeEpPushArgs;

int b200moe_ep_push(const B200MoeEpPushArgs* args, void* stream);

/*
 * Device address of the 32-bit status word inside a scratch region, so a
 * caller can copy it back when it chooses to synchronise.  Replaces the
 * device-side assert the reference uses for out-of-range ids
 * (fastpath/reference.py:99-103), which would poison the CUDA context.
 */
int b200moe_status_ptr(void* scratch, size_t scratch_bytes, uint32_t** status);

/*
 * NVFP4 capability probe.  Mirrors nvfp4_grouped_gemm_available_cuda
 * (csrc/quantization_kernels.cu:7-13), which always answers 0; here it answers 1: the
 * block-scaled FP4 grouped GEMMs are compiled in.  BF16 is never substituted for NVFP4.
 */
int b200moe_nvfp4_available(void);

/*
 * NVFP4 weight preparation, run once when the model is loaded.  No counterpart in the
 * reference.  `weights_bf16` is [num_experts][halves * rows][cols] BF16 (halves = 2 for the
 * gate+up matrix with rows = I, whose gate and up halves get separate scale tilings; 1 for
 * the down matrix with rows = H; cols is the reduction dimension, a multiple of 64).  Per
 * expert matrix: tensor_scale = max|w| / (6 * 448) (1 when all zero); per block of 16
 * elements: block_scale = E4M3(max|block| / 6 / tensor_scale), round to nearest even;
 * element = E2M1(w / (tensor_scale * block_scale)), round to nearest even, saturating.
 *   packed_out        [num_experts][halves * rows][cols / 2] bytes
 *   block_scale_out   num_experts * b200moe_nvfp4_scale_bytes(rows, cols, halves) bytes, zeroed
 *                     by the caller (rows of a partial last tile stay zero)
 *   tensor_scale_out  [num_experts] fp32
 *   amax_scratch      [num_experts] uint32 of device scratch
 */
int b200moe_nvfp4_scale_bytes(int rows, int cols, int halves, size_t* bytes_per_expert);
int b200moe_nvfp4_quantize(const void* weights_bf16, int num_experts, int rows, int cols,
                           int halves, uint8_t* packed_out, uint8_t* block_scale_out,
                           float* tensor_scale_out, uint32_t* amax_scratch, void* stream);
/*
 * The rule by which the NVFP4 kernels hold a token row, exposed for tests: FP32 rows
 * [num_rows][cols] -> four E2M1 planes [4][num_rows][cols / 2] bytes and one power-of-two
 * FP32 scale t per row (max |row| / t in [2, 4)), with
 * row ~= t * (plane0 + plane1 / 8 + plane2 / 64 + plane3 / 512); every plane rounds what the
 * planes before it left over, so |row - that| <= t / 1024.
 */
int b200moe_nvfp4_rows_to_planes(const float* rows_f32, int num_rows, int cols, uint8_t* planes,
                                 float* row_scale, void* stream);

/*
 * FP8 (E4M3) weight preparation, run once when the model is loaded.  No counterpart in the
 * reference.  Row r of a [rows, cols] BF16 matrix (rows = E*2I or E*H, cols = H or I) gets
 * scale[r] = max|w[r,:]| / 448 (1 when the row is all zero) and
 * q[r,c] = E4M3(round-to-nearest-even, saturating)(float(w[r,c]) / scale[r]).
 * b200moe_fp8_dequantize_rows writes bf16(E4M3 value * scale[r]) (scale == NULL: the bare
 * E4M3 values, which BF16 holds exactly); it is for inspection and tests, the GEMM kernels
 * feed the E4M3 bytes to the tensor core as they are.
 * cols must be a multiple of 16; pointers 16-byte aligned.
 */
int b200moe_fp8_quantize_rows(const void* weights_bf16, long long rows, int cols,
                              uint8_t* q_out, float* scale_out, void* stream);
int b200moe_fp8_dequantize_rows(const uint8_t* q, const float* scale, long long rows, int cols,
                                void* out_bf16, void* stream);

/*
 * Router front end (the step in front of the layer).  Replaces the two PyTorch
 * calls of topk_routing (baseline/routing.py:48-55), which the reference's
 * benchmark counts in routing_us and total_us (benchmark/benchmark_goal_1b.py:464,
 * 530-533): per token the top_k largest router logits in descending order
 * (lower expert id first among equal logits), then a softmax over those k
 * logits computed in FP32.
 *   logits            [T,E] bf16, or fp32 when logits_are_f32 != 0;  E <= 256
 *   expert_indices    [T,K] int64 out
 *   weights_bf16      [T,K] bf16 out or NULL
 *   weights_f32       [T,K] fp32 out or NULL
 */
int b200moe_router_topk(const void* logits, int logits_are_f32, int num_tokens, int num_experts,
                        int top_k, int64_t* expert_indices, void* weights_bf16,
                        float* weights_f32, void* stream);

/*
 * Process-wide tuning knobs of the grouped GEMMs, for benchmarking sweeps.  No
 * counterpart in the reference (its GEMMs are library calls with no knobs).
 * Not thread-safe against concurrent forwards; results never depend on them.
 *   B200MOE_TUNE_STAGE_KB      shared memory of the TMA stage ring per block,
 *                              48..220 KB (default 108: two blocks per SM;
 *                              above 113 one block per SM with a deeper ring)
 *   B200MOE_TUNE_L2_PROMOTION  TMA L2 promotion of all tensor maps: 0 none,
 *                              1 = 128 B, 2 = 256 B (default)
 *   B200MOE_TUNE_EVICT_FIRST   1: weight tiles are loaded with an L2
 *                              evict-first hint (default 0)
 *   B200MOE_TUNE_SMALL_CALL_MAX  most assignments (T * top_k) for which b200moe_forward
 *                              uses small-call order, for every top_k (0..32; 0 = never);
 *                              -1 = the default rule: T * top_k <= 32 and top_k <= 4
 *   B200MOE_TUNE_DOWN_SPLITS   force the split-K factor of the down projection (1..8;
 *                              0 = chosen on the device from the routing result)
 *   B200MOE_TUNE_FP8_SEG_ROWS  longest segment of the FP8-weight path: 16, 32, 48 or 64 rows
 *                              (default 64; shorter segments leave more shared memory to
 *                              the weight stream and re-read weights of longer experts)
 *   B200MOE_TUNE_DOWN_TARGET   number of blocks the split-K of the down projection aims
 *                              at when few (segment, tile) units exist (0 = default)
 *   B200MOE_TUNE_GEMM_OVERLAP  1: inside b200moe_forward (regular order, BF16, dependent
 *                              launches) a down block waits for the gate+up tiles of its own
 *                              segment only; 0: for the whole gate+up grid; -1 (default):
 *                              1 where intermediate_size <= hidden_size, else 0
 *   B200MOE_TUNE_NVFP4_PREFETCH  NVFP4 GEMMs: weight slots a block requests before it waits
 *                              for the previous kernel (0..8, default 8 = the whole ring)
 *   B200MOE_TUNE_NVFP4_ISSUERS  NVFP4 GEMMs: 1 = one thread issues every MMA of a block;
 *                              2 (default) = two threads: gate+up one per weight tile, down
 *                              alternate K steps (segments of at most 32 rows)
 */
#define B200MOE_TUNE_STAGE_KB     1
#define B200MOE_TUNE_L2_PROMOTION 2
#define B200MOE_TUNE_EVICT_FIRST  3
#define B200MOE_TUNE_SMALL_CALL_MAX 4
#define B200MOE_TUNE_DOWN_TARGET  5
#define B200MOE_TUNE_DOWN_SPLITS  6
#define B200MOE_TUNE_FP8_SEG_ROWS 7
#define B200MOE_TUNE_NVFP4_PREFETCH 8
#define B200MOE_TUNE_NVFP4_ISSUERS 9
#define B200MOE_TUNE_GEMM_OVERLAP 10
int b200moe_tune(int knob, int value);

#ifdef __cplusplus
}
#endif
#endif /* B200MOE_H_ */
