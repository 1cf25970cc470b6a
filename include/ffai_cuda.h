/*
 * ffai_cuda.h — C ABI of libffai_cuda: the sparse mixture-of-experts feed-forward
 * block of FFAI (router → dispatch → grouped expert products → combine) over MLX
 * affine-quantized weights, implemented as hand-written CUDA for sm_100a.
 *
 * The reference (thewafflehaus/FFAI) has no FFI boundary for this path: the block
 * is called in-process through Swift methods.  Every entry point below therefore
 * cites the Swift method (path within the FFAI project, file:line) whose work it
 * replaces.  All signatures are plain C: pointers, sizes, an opaque handle, and a
 * `void*` that carries a `cudaStream_t`.
 *
 * Conventions
 *   - Activations are bf16 (uint16_t bit patterns), row-major, contiguous.
 *   - Packed weights are uint32 words in the MLX affine layout: a row of `in`
 *     values at `bits` bits is `in*bits/32` little-endian words holding one
 *     contiguous LSB-first bit stream (value i occupies stream bits
 *     [i*bits, (i+1)*bits)); `w = scale*q + bias` with one bf16 scale and one
 *     bf16 bias per `group_size` input values.
 *     (FFAI: Sources/FFAI/Layers.swift:133-189, Ops/QuantizedOpsValidation.swift:52-57,
 *      bit layout pinned by Tests/FFAITests/Ops/QuantizedOpsTests.swift:33-124.)
 *   - Every function returns an `ffai_status`; nothing traps.  The reference
 *     traps via `precondition` (e.g. Sources/FFAI/Ops/Ops.swift:4588-4615); each
 *     such precondition maps to FFAI_ERR_INVALID_ARG here.
 *   - One handle may be used by one stream at a time (the reference's threading
 *     contract, Sources/FFAI/Models/MoELayer.swift:311-318).
 *   - There is no CPU fallback: without a CUDA device every compute entry point
 *     returns FFAI_ERR_CUDA.
 */
#ifndef FFAI_CUDA_H
#define FFAI_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define FFAI_API __attribute__((visibility("default")))
#else
#define FFAI_API
#endif

#define FFAI_CUDA_ABI_VERSION 1
#define FFAI_MAX_TOP_K 32
#define FFAI_MAX_EXPERTS 1024

typedef enum ffai_status {
    FFAI_OK = 0,
    FFAI_ERR_INVALID_ARG = 1, /* a reference `precondition` would have failed   */
    FFAI_ERR_UNSUPPORTED = 2, /* valid request, not implemented for this shape   */
    FFAI_ERR_CUDA = 3,        /* a CUDA runtime/driver call failed               */
    FFAI_ERR_NOT_READY = 4,   /* forward before set_weights                      */
    FFAI_ERR_NCCL = 5,        /* expert-parallel exchange failed                 */
    FFAI_ERR_DEVICE_CHECK = 6 /* a bounded device-side wait or check gave up     */
} ffai_status;

/* MoEGatingMode — Sources/FFAI/Models/MoELayer.swift:71-78 */
typedef enum ffai_gating_mode {
    FFAI_GATING_SOFTMAX_THEN_TOPK = 0,
    FFAI_GATING_TOPK_THEN_SOFTMAX = 1,
    /* NemotronHMoELayer routing (Sources/FFAI/Models/Text/NemotronHText.swift:844-867): scores =
     * sigmoid(logits); selection on scores + expert_bias (e_score_correction_bias; ties to the lower
     * index); combine weights are the raw sigmoids of the selected, divided by (their sum + 1e-20) when
     * top_k > 1 and norm_topk_prob, then multiplied by routed_scaling_factor. */
    FFAI_GATING_SIGMOID_TOPK = 2
} ffai_gating_mode;

/* Expert activation.
 *   SWIGLU          silu(gate)*up                 Sources/FFAI/Ops/Ops.swift:6400-6452
 *   CLAMPED_SWIGLU  g=min(gate,L); u=clamp(up,-L,L);
 *                   (u+1) * g / (1+exp(-alpha*g))  Sources/FFAI/Models/Text/GPTOSSText.swift:1414-1431
 *   GELU_GLU        gelu_tanh(gate)*up             Sources/FFAI/Ops/OpsFused.swift:55-87
 *   RELU2           relu(up)^2: experts WITHOUT a gate projection (NemotronHExpert,
 *                   Sources/FFAI/Models/Text/NemotronHText.swift:741-763; Ops.relu, Ops.swift:209-212);
 *                   gate_proj (and shared_gate_proj) are not read and may be null; a shared expert has
 *                   the same form
 */
typedef enum ffai_activation {
    FFAI_ACT_SWIGLU = 0,
    FFAI_ACT_CLAMPED_SWIGLU = 1,
    FFAI_ACT_GELU_GLU = 2,
    FFAI_ACT_RELU2 = 3
} ffai_activation;

/* Storage type of a dense-or-quantized projection (router, shared-expert gate). */
typedef enum ffai_linear_kind {
    FFAI_LINEAR_NONE = 0,
    FFAI_LINEAR_F32 = 1,   /* Linear, fp32 weight  — Sources/FFAI/Layers.swift:24-130 */
    FFAI_LINEAR_BF16 = 2,  /* Linear, bf16 weight                                      */
    FFAI_LINEAR_AFFINE = 3 /* QuantizedLinear      — Sources/FFAI/Layers.swift:133-289 */
} ffai_linear_kind;

typedef enum ffai_mem_location {
    FFAI_MEM_HOST = 0,  /* library allocates device memory and copies          */
    FFAI_MEM_DEVICE = 1 /* library borrows the device pointers (no copy); the   */
                        /* caller keeps them alive until destroy/set_weights   */
} ffai_mem_location;

/*
 * Layer description.  One struct covers MoELayer (MoELayer.swift:319-498),
 * GPTOSSMoELayer (GPTOSSText.swift:1302-1337) and Qwen35MoEFFN
 * (Qwen3xText.swift:870-926).  Zero-initialise, set `struct_size`, fill in.
 */
typedef struct ffai_moe_config {
    uint32_t struct_size;      /* = sizeof(ffai_moe_config) */
    int32_t hidden;            /* H, multiple of 64                                   */
    int32_t intermediate;      /* I, multiple of 64                                   */
    int32_t n_experts;         /* E (global count, also under expert parallelism)     */
    int32_t top_k;             /* 1..min(E, FFAI_MAX_TOP_K)                           */
    int32_t gating_mode;       /* ffai_gating_mode                                    */
    int32_t norm_topk_prob;    /* MoERouter.normTopKProb, MoELayer.swift:92-95        */
    int32_t router_expert_bias;/* 1: post-softmax additive bias (LFM2), :97-103       */
    int32_t activation;        /* ffai_activation                                     */
    float swiglu_limit;        /* L  (GPT-OSS swiglu_limit, GPTOSSText.swift:120)      */
    float swiglu_alpha;        /* alpha (1.702, GPTOSSText.swift:959)                  */
    int32_t router_kind;       /* ffai_linear_kind                                    */
    int32_t router_bits;       /* AFFINE only: 2,3,4,5,6,8                            */
    int32_t router_group_size; /* AFFINE only: 32,64,128                              */
    int32_t router_has_bias;   /* GPTOSSBiasedLinear, GPTOSSText.swift:341-362        */
    int32_t router_logits_bf16;/* 1: logits are rounded to bf16 before top-k, as the  */
                               /* reference's bf16 logits tensor is (MoELayer.swift:540,572) */
    int32_t expert_bits;       /* 3,4,5,6,8 (2 accepted)                              */
    int32_t expert_group_size; /* 32,64,128                                           */
    int32_t expert_row_bias;   /* 1: per-row projection bias b_g,b_u,b_d (GPT-OSS)    */
    int32_t shared_intermediate;/* 0: no shared expert                                */
    int32_t shared_bits;
    int32_t shared_group_size;
    int32_t shared_gate_kind;  /* ffai_linear_kind; NONE: shared output added         */
                               /* unconditionally (MoELayer.swift:621-624); otherwise  */
                               /* scaled by sigmoid(gate·x) (Qwen3xText.swift:1013-1035) */
    int32_t shared_gate_bits;
    int32_t shared_gate_group_size;
    int32_t max_tokens;        /* largest T a forward call may pass                   */
    int32_t ep_rank;           /* expert parallelism: this rank, 0 when ep_world<=1   */
    int32_t ep_world;          /* 0 or 1: single GPU                                  */
    int32_t prefill_weight_cache; /* bf16 copy of the routed experts (2 bytes per weight, beside the  */
                               /* packed ones) that the tensor-core prefill path reads without a   */
                               /* dequant stage: 0 automatic (kept when max_tokens*top_k/n_experts */
                               /* >= 32 and the copy is at most 4 GiB), 1 never, 2 always.  Decode   */
                               /* batches always stream the packed weights.                         */
    float router_logit_scale;  /* the logits are multiplied by this (fp32) before top-k / softmax; 0 means 1.   */
                               /* Gemma 4 folds hidden^-0.5 into the logits here (Gemma4Text.swift:937-943). */
    float routed_scaling_factor; /* FFAI_GATING_SIGMOID_TOPK: factor on the combine weights; 0 means 1          */
                               /* (NemotronHText.swift:263, 866).                                             */
    int32_t reserved[5];
} ffai_moe_config;

/* One stacked quantized projection: weight [n, out, in*bits/32] u32,
 * scales/biases [n, out, in/group] bf16, optional row bias [n, out] bf16.
 * (StackedInt4Experts, MoELayer.swift:347-391; n = 1 for the shared expert.) */
typedef struct ffai_qproj {
    const uint32_t* weight;
    const uint16_t* scales;
    const uint16_t* biases;
    const uint16_t* row_bias; /* nullable */
} ffai_qproj;

/* A dense or quantized [out, in] projection (router; shared-expert gate). */
typedef struct ffai_linear {
    const void* weight;       /* f32 / bf16 [out,in], or u32 [out, in*bits/32]  */
    const uint16_t* scales;   /* AFFINE only */
    const uint16_t* biases;   /* AFFINE only */
    const uint16_t* bias;     /* nullable projection bias [out], bf16           */
} ffai_linear;

typedef struct ffai_moe_weights {
    uint32_t struct_size;     /* = sizeof(ffai_moe_weights) */
    int32_t location;         /* ffai_mem_location, applies to every pointer    */
    ffai_linear router;       /* [E, H]                                         */
    const float* router_expert_bias; /* [E] fp32, nullable                      */
    ffai_qproj gate_proj;     /* [E_local, I, H]                                 */
    ffai_qproj up_proj;       /* [E_local, I, H]                                 */
    ffai_qproj down_proj;     /* [E_local, H, I]                                 */
    ffai_qproj shared_gate_proj; /* [1, I_s, H]                                  */
    ffai_qproj shared_up_proj;   /* [1, I_s, H]                                  */
    ffai_qproj shared_down_proj; /* [1, H, I_s]                                  */
    ffai_linear shared_gate;  /* [1, H]                                         */
    const float* router_per_expert_scale; /* nullable [E] f32: combine weight of a slot *= scale[its expert] */
                                          /* (Gemma 4 router.per_expert_scale, Gemma4Text.swift:944-949)     */
} ffai_moe_weights;

/* Optional per-call routing/dispatch outputs (device pointers for
 * ffai_moe_forward, host pointers for ffai_moe_forward_host; any may be NULL). */
typedef struct ffai_moe_debug {
    uint32_t* indices;  /* [T, k]   selected experts, value-desc / index-asc     */
    float* weights;     /* [T, k]   combine weights                              */
    float* logits;      /* [T, E]   router logits as seen by top-k               */
    uint32_t* counts;   /* [E]      rows per expert                              */
    uint32_t* offsets;  /* [E+1]    exclusive scan of counts                     */
    uint32_t* perm;     /* [T*k]    sorted position -> token*k+slot              */
    uint32_t* inv_perm; /* [T*k]    token*k+slot -> sorted position              */
} ffai_moe_debug;

typedef struct ffai_moe_layer ffai_moe_layer; /* opaque */

/* Library / device probes. */
FFAI_API int ffai_cuda_abi_version(void);
/* Number of visible CUDA devices; 0 without a GPU (never an error). */
FFAI_API int ffai_cuda_device_count(void);
FFAI_API const char* ffai_status_string(int status);

/*
 * Lifecycle.
 * create   replaces MoELayer.init / MoERouter.init (MoELayer.swift:105-124, 440-498),
 *          GPTOSSMoELayer.init (GPTOSSText.swift:1311-1325), Qwen35MoEFFN.init.
 *          Allocates all workspace for `max_tokens` on the current CUDA device.
 * set_weights  replaces the borrowed-tensor hand-off of Qwen35Hybrid.buildMoE /
 *          tryLoadStackedInt4 (Qwen3xText.swift:598-739).
 * destroy  frees everything the library allocated.
 */
FFAI_API int ffai_moe_create(const ffai_moe_config* config, ffai_moe_layer** out_layer);
FFAI_API int ffai_moe_set_weights(ffai_moe_layer* layer, const ffai_moe_weights* weights);
FFAI_API int ffai_moe_destroy(ffai_moe_layer* layer);
FFAI_API const char* ffai_moe_last_error(const ffai_moe_layer* layer);

/*
 * forward — replaces MoELayer.decode (MoELayer.swift:530-634, T = 1),
 * MoELayer.decodeMany (:677-969), GPTOSSMoELayer.decode (GPTOSSText.swift:1340-1392)
 * and Qwen35MoEFFN.forward / forwardMany (Qwen3xText.swift:928-1103).
 *   x, out, residual: device bf16 [T, H]; residual nullable; out complete when
 *   `stream` reaches the end of the call.  No allocation.  No host synchronisation on one GPU and
 *   under expert parallelism over peer memory; expert parallelism over NCCL waits for the stream once
 *   per call (NCCL takes the exchange sizes from the host).
 */
FFAI_API int ffai_moe_forward(ffai_moe_layer* layer, const uint16_t* x, int32_t n_tokens,
                     uint16_t* out, const uint16_t* residual,
                     const ffai_moe_debug* debug, void* cuda_stream);

/* Same call with HOST buffers: copies x (and residual) to the device, runs
 * forward, copies out (and debug outputs) back, and waits.  This is what a
 * caller holding host tensors uses, as the reference's callers do with
 * shared-storage MTLBuffers (Sources/FFAI/Device.swift:23-64). */
FFAI_API int ffai_moe_forward_host(ffai_moe_layer* layer, const uint16_t* x, int32_t n_tokens,
                          uint16_t* out, const uint16_t* residual,
                          const ffai_moe_debug* debug);

/* As ffai_moe_forward / ffai_moe_forward_host, with the router reading its own input rows x_router
 * [T, hidden] while the experts (and the shared expert) read x: Gemma 4 normalises the two branches
 * differently (Gemma4Text.swift:929-933, 957).  x_router == NULL means x. */
FFAI_API int ffai_moe_forward_split(ffai_moe_layer* layer, const uint16_t* x, const uint16_t* x_router, int32_t n_tokens,
                                    uint16_t* out, const uint16_t* residual, const ffai_moe_debug* debug, void* stream);
FFAI_API int ffai_moe_forward_host_split(ffai_moe_layer* layer, const uint16_t* x, const uint16_t* x_router, int32_t n_tokens,
                                         uint16_t* out, const uint16_t* residual, const ffai_moe_debug* debug);

/* Expert parallelism: attach an initialised ncclComm_t (one rank per GPU) before
 * the first forward when config.ep_world > 1.  No reference counterpart (the
 * reference is single-device). */
FFAI_API int ffai_moe_set_nccl_comm(ffai_moe_layer* layer, void* nccl_comm);

/* Expert-parallel plumbing (no reference counterpart).  Rank 0 makes an id, the host code hands the 128
 * bytes to every rank (any transport), each rank creates its communicator with its GPU current and
 * attaches it with ffai_moe_set_nccl_comm.  NCCL is looked up at run time; single-GPU use needs none. */
FFAI_API int ffai_ep_get_unique_id(uint8_t out_id[128]);
FFAI_API int ffai_ep_comm_create(const uint8_t id[128], int32_t rank, int32_t world, void** out_comm);
FFAI_API int ffai_ep_comm_destroy(void* comm);
/* Exchange over peer memory instead of NCCL (one process per GPU on one node, every GPU reachable over
 * NVLink): each rank exports three of its buffers as CUDA IPC handles, the host code hands every
 * rank's blob to every rank (rank order, any transport), each rank imports.  From then on a step
 * makes no NCCL call and no host synchronisation: the row gather stores straight into the owners'
 * buffers, the combine loads result rows from them, three flag barriers (time-limited) order the
 * phases.  Needs the 4-bit expert kernels (or the bf16 weight cache); all ranks call forward for every
 * step, with the same max_tokens.  No reference counterpart. */
#define FFAI_EP_EXPORT_BYTES 192
FFAI_API int ffai_moe_ep_export(ffai_moe_layer* layer, uint8_t out_blob[FFAI_EP_EXPORT_BYTES]);
FFAI_API int ffai_moe_ep_import(ffai_moe_layer* layer, const uint8_t* blobs /* [ep_world][FFAI_EP_EXPORT_BYTES] */);
/* Unmaps the peers' buffers (after the last step; before any rank destroys its layer, so that no
 * exported buffer is freed while a peer still maps it).  The step counter that the flag barriers carry keeps
 * running over a release and a later import, so flags left from earlier steps can never satisfy a new wait;
 * ranks that import again must do so together, with layers that have run the same number of steps. */
FFAI_API int ffai_moe_ep_release(ffai_moe_layer* layer);
/* A rank that sits out one step of the peer-memory exchange (it learned on the host that the step is void for
 * it) advances its step counter with this call instead of forward, so that it meets the others again at the
 * next step.  The ranks that did run the step see their barriers give up after the wait limit (option
 * "ep_wait_ms"), get FFAI_ERR_DEVICE_CHECK from ffai_moe_check_device_status / ffai_moe_forward_host, and discard
 * that step's output.  No reference counterpart. */
FFAI_API int ffai_moe_ep_skip_step(ffai_moe_layer* layer);
/* The layout the peer-memory exchange derives on the device, computed on the host by the same code (for
 * tests; needs no GPU): from counts_matrix[world][n_experts] (rows every rank sends to every expert),
 * local_offsets[n_experts/world + 1] = row ranges of `rank`'s own experts in its row buffer, and
 * send_base[n_experts] = where `rank`'s rows for each expert start in the owner's row buffer. */
FFAI_API int ffai_ep_peer_layout(const uint32_t* counts_matrix, int32_t world, int32_t n_experts, int32_t rank,
                                 uint32_t* local_offsets, uint32_t* send_base);
/* Host-side plan of one exchange from the per-(source rank, local expert) row counts
 * recv_counts[world][e_local]: where each source's rows start in the receive buffer
 * (rank_offsets[world+1]), the expert-contiguous layout after regrouping (local_offsets[e_local+1]),
 * and the start of every (source, expert) segment in both (seg_src, seg_dst, [world*e_local]).
 * Returns the number of rows received.  Integer arithmetic only; needs no GPU. */
FFAI_API uint32_t ffai_ep_plan_exchange(const uint32_t* recv_counts, int32_t world, int32_t e_local,
                                        uint32_t* rank_offsets, uint32_t* local_offsets,
                                        uint32_t* seg_src, uint32_t* seg_dst);

/* Execution options, replacing the reference's FFAI_MOE_* environment switches
 * (Sources/FFAI/Models/MoELayer.swift:486-497).  Names:
 *   "path"         0 automatic, 1 CUDA-core grouped GEMV only, 2 tcgen05 grouped GEMM whenever possible,
 *                  3 streaming decode kernels whenever possible
 *   "tc_min_rows"  smallest T*k that takes the tcgen05 path under "path" = 0 (0: default)
 *   "tc_weights"   tcgen05 path reads 0 automatic (the bf16 weight cache when the layer keeps one, except gate/up
 *                  with at most 160 routed rows per expert), 1 always the packed weights, 2 always the cache
 *   "host_chunks"  host entry points: 0 = a batch of 4096 tokens or more goes through in up to 3 chunks whose copies
 *                  overlap the compute (same bits: tokens are independent), 1 = always as one piece, 2..4 = at
 *                  most that many chunks
 *   "ksplit"       cp.async decode kernels: slices of the reduction axis per 16-row block (0 automatic, 1, 2, 4)
 *   "decode"       decode kernels: 0 automatic, 1 cp.async rings, 2 bulk-copy streams
 *   "decode_team"  bulk-copy streams: warps that share one 16-row block (0 automatic, 1, 4, 16)
 *   "nt2_cost"     bulk-copy streams: schedule weight of a block with more than 8 rows, 8 = as one with fewer (8..32)
 *   "overlap"      shared expert on a second stream beside router, plan and row exchange (default 1; 0: one stream)
 *   "pdl"          decode chain launched as programmatic dependent launches (default 1; 0: plain launches)
 *   "ep_wait_ms"   limit of a barrier wait of the peer-memory exchange, milliseconds (default 2000)
 *   "timeline"     1: the gate/up tcgen05 kernel records its device timeline (builds with FFAI_G100_TIMELINE only) */
FFAI_API int ffai_moe_set_option(ffai_moe_layer* layer, const char* name, int32_t value);

/* Profiling aid for the tcgen05 grouped GEMM (the device-side counterpart of the reference's
 * signpost intervals, Sources/FFAI/Telemetry/Profiling.swift:76-117).  After
 * ffai_moe_set_option(layer, "timeline", 1), CTA 0 of the gate/up kernel records its SM clock at
 * fixed points of each warp role for its first 96 k-blocks; this call waits for the device and
 * copies the 5 x 96 x 4 table ([role][k block][event], 0 = not reached) into `out`. */
FFAI_API int ffai_moe_read_timeline(ffai_moe_layer* layer, int64_t* out, int32_t capacity);

/* Waits for the device and reports whether any kernel of this handle raised its error word
 * (a bounded device-side wait that expired): FFAI_OK or FFAI_ERR_DEVICE_CHECK.  The word is
 * cleared by the call.  ffai_moe_forward_host performs this check itself. */
FFAI_API int ffai_moe_check_device_status(ffai_moe_layer* layer);

/* Device time of the stages of the most recent forward on this handle, in
 * milliseconds (CUDA events recorded on the call's stream when timing is on).
 * Names mirror the reference's stages: router, plan, gather, gate_up, down,
 * combine, shared, exchange.  Replaces the signpost phases of
 * Sources/FFAI/Telemetry/Profiling.swift:76-117. */
#define FFAI_N_STAGES 8
FFAI_API int ffai_moe_set_stage_timing(ffai_moe_layer* layer, int enabled);
FFAI_API int ffai_moe_get_stage_ms(ffai_moe_layer* layer, float out_ms[FFAI_N_STAGES]);
/* Number of kernels the most recent forward launched. */
FFAI_API int ffai_moe_last_launch_count(const ffai_moe_layer* layer);

/* ───────────────────────── operator-level entry points ─────────────────────────
 * Thin wrappers over the same kernels the layer uses, shaped like the
 * reference's `Ops.*` so its unit tests can be restated one-for-one.  All
 * pointers are DEVICE pointers; `stream` is a cudaStream_t.                     */

/* Ops.dequantGemv — Sources/FFAI/Ops/Ops.swift:1489-1693.
 * out[o] = sum_i (scales[o,i/gs]*q[o,i] + biases[o,i/gs]) * x[i]; x, out bf16. */
FFAI_API int ffai_op_dequant_gemv(const uint16_t* x, const uint32_t* weight,
                         const uint16_t* scales, const uint16_t* biases,
                         uint16_t* out, int32_t out_dim, int32_t in_dim,
                         int32_t bits, int32_t group_size, void* stream);

/* Ops.dequantGemvInt4ExpertIndexed — Ops.swift:2444-2519: the expert slab is
 * chosen on the device from expert_index[0] in a stacked [E,out,in*bits/32]. */
FFAI_API int ffai_op_dequant_gemv_expert_indexed(const uint16_t* x, const uint32_t* weight,
                                        const uint16_t* scales, const uint16_t* biases,
                                        const uint32_t* expert_index, uint16_t* out,
                                        int32_t n_experts, int32_t out_dim, int32_t in_dim,
                                        int32_t bits, int32_t group_size, void* stream);

/* MoERouter.route (MoELayer.swift:140-205) and Ops.moeRouterTopKMany
 * (Ops.swift:2598-2661): logits fp32 [T,E] -> indices u32 [T,k], weights fp32 [T,k].
 * expert_bias nullable [E]. */
FFAI_API int ffai_op_moe_router_topk(const float* logits, uint32_t* indices, float* weights,
                            int32_t n_tokens, int32_t n_experts, int32_t k,
                            int32_t gating_mode, int32_t norm_topk_prob,
                            const float* expert_bias, void* stream);

/* Plan build of MoELayer.decodeMany (MoELayer.swift:752-792), made a stable
 * counting sort by (expert, token, slot).  workspace: device, at least
 * ffai_op_moe_plan_workspace_bytes(n_tokens*k, E) bytes. */
FFAI_API size_t ffai_op_moe_plan_workspace_bytes(int32_t n_rows, int32_t n_experts);
FFAI_API int ffai_op_moe_plan(const uint32_t* indices, int32_t n_tokens, int32_t k,
                     int32_t n_experts, uint32_t* counts, uint32_t* offsets,
                     uint32_t* perm, uint32_t* inv_perm, void* workspace, void* stream);

/* Dispatch plan for callers that must not allocate.  No counterpart in the reference.
 *
 * Same inputs, outputs and results as ffai_op_moe_plan, but the caller passes no workspace and the
 * call never touches the CUDA allocator (no cudaMalloc / cudaFree, no allocating library routine):
 * the per-block histograms live in a fixed array inside the library's device image
 * (FFAI_PLAN_STATIC_MAX_ROWS / 1024 blocks x FFAI_MAX_EXPERTS counters = 512 KiB, held by every GPU
 * that loads the library until the process exits).  It is meant for hosts that own all device
 * memory themselves and forbid a plug-in to allocate once serving has started - an inference
 * server with a pre-sized arena, or code running where an allocator call would block or fail.
 *
 * Limits: n_tokens * k <= FFAI_PLAN_STATIC_MAX_ROWS and n_experts <= FFAI_MAX_EXPERTS, otherwise
 * FFAI_ERR_INVALID_ARG.  The first call on each device looks up the address of the array (with that
 * device current); make that first call before starting any stream capture.  All calls on a
 * device share the one array, which keeps the previous call's contents: every counter a call reads
 * is rewritten by that call first, so nothing needs clearing, but two calls that overlap on the
 * GPU (different streams) race on it - serialise them. */
#define FFAI_PLAN_STATIC_MAX_ROWS 131072
FFAI_API int ffai_op_moe_plan_static(const uint32_t* indices, int32_t n_tokens, int32_t k,
                                     int32_t n_experts, uint32_t* counts, uint32_t* offsets,
                                     uint32_t* perm, uint32_t* inv_perm, void* stream);

/* Ops.gather — Ops.swift:308-346: out[m,:] = table[ids[m],:], bf16 rows. */
FFAI_API int ffai_op_gather_rows(const uint16_t* table, const uint32_t* ids, uint16_t* out,
                        int32_t n_rows, int32_t row_len, void* stream);

/* Ops.moeGatherDequantGemmInt4 (+Bm8/Bm64Mpp/M1) — Ops.swift:4553-4708, 4912-5201,
 * 6499-6585: out[m,n] = sum_k dequant(W[indices[m]])[n,k] * x[m,k]; rows sorted by
 * expert; x,out bf16; any supported bit width. */
FFAI_API int ffai_op_moe_gather_dequant_gemm(const uint16_t* x, const uint32_t* weight,
                                    const uint16_t* scales, const uint16_t* biases,
                                    const uint32_t* indices, uint16_t* out,
                                    int32_t m_total, int32_t n_out, int32_t k_in,
                                    int32_t n_experts, int32_t bits, int32_t group_size,
                                    void* stream);

/* Ops.swiglu (Ops.swift:6400-6452), GPT-OSS clamped form, Ops.fusedGateGelu. */
FFAI_API int ffai_op_glu_activation(const uint16_t* gate, const uint16_t* up, uint16_t* out,
                           int64_t n, int32_t activation, float limit, float alpha,
                           void* stream);

/* Ops.moeUnpermute — Ops.swift:5030-5110:
 * out[t,:] = sum_s weights[t,s] * expert_out[inv_perm[t*k+s],:], slot order. */
FFAI_API int ffai_op_moe_unpermute(const uint16_t* expert_out, const uint32_t* inv_perm,
                          const float* weights, uint16_t* out, int32_t n_tokens,
                          int32_t hidden, int32_t k, void* stream);

/* Reading a block's weights from a .safetensors file (host code; no GPU needed).  The file is mapped
 * read-only and ffai_moe_weights is filled with HOST pointers into the mapping, valid until
 * ffai_st_close; hand it to ffai_moe_set_weights (which copies to the device) before closing.
 * Replaces the reference's loader path for the block (Loader/SafeTensors.swift:377-396; stacked triplets
 * Qwen3xText.swift:605-650, Gemma4Text.swift:540-554; bit widths derived per tensor from the shapes,
 * Layers.swift:340-363).  ffai_st_moe_weights takes the group sizes from `config` (expert_group_size
 * must be set; router / shared ones default to it), and fills in from the file: n_experts, hidden,
 * intermediate, the bit widths, the router kind and bias flag, the shared expert's sizes.  Routing
 * mode, activation, top_k and max_tokens stay the caller's.  GPT-OSS checkpoints (MXFP4 experts) go
 * through ffai_st_tensor + ffai_op_mxfp4_to_affine_int4 instead. */
typedef struct ffai_st_file ffai_st_file;
enum { FFAI_ST_SWITCH_MLP = 0,   /* <prefix>.switch_mlp.{gate,up,down}_proj.*, router <prefix>.gate.*             */
       FFAI_ST_SWITCH_GLU = 1 }; /* <prefix>.experts.switch_glu.*, router <prefix>.router.proj.* (+ per_expert_scale) */
FFAI_API int ffai_st_open(const char* path, ffai_st_file** out_file);
FFAI_API void ffai_st_close(ffai_st_file* file);
FFAI_API const char* ffai_st_last_error(const ffai_st_file* file);
FFAI_API int ffai_st_tensor(const ffai_st_file* file, const char* name, const void** data, uint64_t* n_bytes,
                            char dtype[8], int64_t shape[8], int32_t* n_dims);
FFAI_API int32_t ffai_st_derive_bits(int64_t weight_packed_cols, int64_t scale_cols, int32_t group_size);
FFAI_API int ffai_st_moe_weights(ffai_st_file* file, const char* prefix, int32_t scheme, ffai_moe_config* config,
                                 ffai_moe_weights* out_weights);

/* Weight preparation (rows either side of the block).
 * ffai_op_mxfp4_to_affine_int4: the load-time transcode of GPT-OSS experts
 *   (GPTOSSText.swift:1071-1244, a host loop there): per group of 32 fp4 (e2m1) codes and one e8m0
 *   scale byte, fit an affine 16-level grid to the group's own min/max and remap the codes nibble for
 *   nibble.  packed: n_groups*4 words; out_weight the same size (bits 4, group size 32); scales and
 *   biases bf16, one per group.  Bit-identical to the host version.
 * ffai_op_affine_quantize: MLX affine quantization of a [rows, in_dim] bf16 matrix into the packed
 *   layout this library reads (QuantizedOps.swift:229-388); bits in {2,3,4,5,6,8}, gs in {32,64,128}. */
/* The step in front of the block (Ops.addAndRmsNorm, Ops.swift:658-760; called right before the MoE
 * block in GPTOSSText.swift:700-716): residual_out = a + b, normed_out = RMSNorm(a + b) * weight, rows of
 * n bf16 (n a multiple of 8; no upper limit, unlike the reference's 4096), fp32 arithmetic inside.
 * With b = NULL it is the plain row-wise RMSNorm (Ops.rmsNorm / Ops.rmsNormRows, Ops.swift:515-578): the norm a
 * Gemma 4 block applies to the router's input rows and to the experts' input rows (Gemma4Text.swift:932-960)
 * before ffai_moe_forward_split; residual_out may then be NULL. */
FFAI_API int ffai_op_add_rmsnorm(const uint16_t* a, const uint16_t* b, const uint16_t* weight, float eps,
                                 int32_t n_rows, int32_t n, uint16_t* residual_out, uint16_t* normed_out, void* stream);
FFAI_API int ffai_op_mxfp4_to_affine_int4(const uint32_t* packed, const uint8_t* e8m0, int64_t n_groups,
                                          uint32_t* out_weight, uint16_t* out_scales, uint16_t* out_biases,
                                          void* stream);
FFAI_API int ffai_op_affine_quantize(const uint16_t* w, int64_t rows, int32_t in_dim, int32_t bits, int32_t gs,
                                     uint32_t* out_weight, uint16_t* out_scales, uint16_t* out_biases, void* stream);

/* Ops.sigmoidScalarFMA / sigmoidScalarFMAResidual — Ops.swift:6255-6334,
 * OpsFused.swift:699-753, batched over rows:
 * out[t,:] = [residual[t,:] +] base[t,:] + sigmoid(gate[t]) * value[t,:]. */
FFAI_API int ffai_op_sigmoid_scalar_fma(const uint16_t* gate, const uint16_t* value,
                               const uint16_t* base, const uint16_t* residual,
                               uint16_t* out, int32_t n_rows, int32_t hidden, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FFAI_CUDA_H */
