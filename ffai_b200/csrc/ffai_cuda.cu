// libffai_cuda — C ABI over the sm_100a MoE kernels.  See include/ffai_cuda.h.
#include "../../include/ffai_cuda.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <vector>

#include "combine.cuh"
#include "common.cuh"
#include "expert_gemv.cuh"
#include "ep.cuh"
#include "expert_mma_decode.cuh"
#include "expert_stream_decode.cuh"
#include "plan.cuh"
#include "router.cuh"
#include "safetensors.hpp"
#include "tc_path.cuh"
#include "weight_prep.cuh"

using namespace ffai;

// ───────────────────────────── layer object ─────────────────────────────

struct ffai_moe_layer {
    ffai_moe_config cfg{};
    int device = -1;
    int e_local = 0;  // experts held by this rank
    bool weights_set = false;
    ffai_moe_weights w{};  // device pointers
    std::vector<void*> owned_weights;
    std::vector<void*> owned_ws;
    std::vector<void*> owned_pinned;

    // workspace (device)
    float* logits = nullptr;        // [T,E]
    uint32_t* indices = nullptr;    // [T,k]
    float* rweights = nullptr;      // [T,k]
    uint32_t* counts = nullptr;     // [E]
    uint32_t* offsets = nullptr;    // [E+1]
    uint32_t* perm = nullptr;       // [M]
    uint32_t* inv_perm = nullptr;   // [M]
    uint32_t* block_hist = nullptr; // [nblocks,E]
    float* router_partials = nullptr;  // [H/64][T][E] chunk sums of the split batched router (when it fits 256 MiB)
    size_t router_partials_cap = 0;    // in floats
    uint32_t* tickets = nullptr;    // [min(T,96)] per-token arrival counters of the small-batch router (self-resetting)
    float* inner = nullptr;         // [M,I]
    float* y = nullptr;             // [M,H]
    float* sh_inner = nullptr;      // [T,Is]
    float* sh_y = nullptr;          // [T,H]
    float* sh_gate = nullptr;       // [T]

    // tensor-core path (tcgen05 grouped GEMM): bf16 staging buffers, schedules, tensor maps
    bool tc_ok = false;              // tensor maps encoded, buffers allocated
    int n_sms = 0;
    int opt_path = 0;                // 0 auto, 1 CUDA-core GEMV, 2 tcgen05 grouped GEMM, 3 register-streaming decode
    int opt_tc_min_rows = 0;         // auto: smallest T*k routed through the tensor-core path
    int opt_ksplit = 0;              // streaming kernels: 0 automatic, else 1, 2 or 4 reduction slices
    long long* timeline = nullptr;   // device buffer for the gate/up kernel's CTA-0 timeline (option "timeline")
    uint16_t* xg = nullptr;          // [M,H]  expert-contiguous input rows (8-run permuted)
    uint16_t* inner_bf = nullptr;    // [M,I]  activation output (8-run permuted)
    uint16_t* y_bf = nullptr;        // [M,H]
    float* xsum = nullptr;           // [M, H/64]  64-run sums of xg rows
    uint16_t* x_tok = nullptr;       // [T, H] token rows, 8-run permuted (streaming kernels read them through perm)
    float* xsum_tok = nullptr;       // [T, H/64 rounded up to 4] their 64-run sums
    uint32_t* expert_order = nullptr; // [E] experts by descending row count, written with the fused small-batch plan
    float* router_f32 = nullptr;     // quantized router expanded to fp32 (owned with the weights)
    float* inner_parts = nullptr;    // [M, I/16]  16-run sums of inner rows, written by the gate/up streaming kernel
    float* inner_sum = nullptr;      // [M, I/64]  64-run sums of inner rows
    const uint16_t* router_x = nullptr;  // set for the duration of a split forward: the router's own input rows
    uint16_t* dev_xr = nullptr;          // host-buffer entry point: device copy of the router input
    bool no_gate = false;            // experts without a gate projection (relu(up)^2): CUDA-core GEMV kernels only
    bool mma_ok = false;             // register-streaming decode kernels usable (4-bit, group 64/128)
    uint8_t* st_gate_up = nullptr;   // bulk-copy streams of the decode kernels: gate and up interleaved per 64-run, ...
    uint8_t* st_down = nullptr;      // ... and down (re-tiled copies of the packed experts, owned with the weights)
    int opt_decode = 0;              // decode kernels: 0 automatic, 1 per-lane cp.async rings, 2 bulk-copy streams
    int opt_overlap = 1;             // shared expert on a second stream beside router / plan / exchange (0: one stream)
    cudaStream_t aux_stream = nullptr;
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    int opt_pdl = 1;                 // decode chain: programmatic dependent launches (0: plain launches)
    int opt_decode_team = 0;         // bulk-copy streams: warps per 16-row block (0 automatic, 1, 4, 16)
    int opt_nt2_cost = 12;           // bulk-copy streams: schedule weight of an item with more than 8 rows (8 = as one with fewer)
    uint32_t* sb_gate = nullptr;     // repacked (scale | bias << 16) words of the expert projections
    uint32_t* sb_up = nullptr;
    uint32_t* sb_down = nullptr;
    uint32_t* tile_offsets = nullptr;    // [E+1]
    uint16_t* sh_x = nullptr;        // [T,H]  shared expert input (8-run permuted)
    uint16_t* exp_wbf[3] = {nullptr, nullptr, nullptr}; // routed experts expanded to bf16 (prefill weight cache): gate, up, down
    bool cache_planned = false;
    int opt_tc_weights = 0;          // tensor-core path reads: 0 the bf16 cache when there is one, 1 always the packed weights
    uint16_t* sh_wbf[3] = {nullptr, nullptr, nullptr};  // shared expert expanded to bf16 (bit widths other than 4): gate, up, down
    uint16_t* sh_inner_bf = nullptr; // [T,Is]
    uint32_t* sh_sched = nullptr;    // offsets[2] + tile_offsets[2]
    uint32_t* error_word = nullptr;
    CUtensorMap tm_gate{}, tm_up{}, tm_down{}, tm_sh_gate{}, tm_sh_up{}, tm_sh_down{};
    CUtensorMap tm_xg{}, tm_inner{}, tm_sh_x{}, tm_sh_inner{};  // activation maps: 64 k x 128-row boxes

    // expert parallelism (ep_world > 1): Mx = rows that may arrive here = world * max_tokens * top_k
    size_t mx_rows = 0;              // capacity of xg / inner / y in rows (== M when single GPU)
    uint16_t* ep_send_x = nullptr;   // [M,H]   my rows sorted by (global) expert, ready to leave
    uint16_t* ep_recv_x = nullptr;   // [Mx,H]  rows as they arrive, source-rank order
    float* ep_ret_y = nullptr;       // [Mx,H]  expert outputs back in arrival order
    float* ep_home_y = nullptr;      // [M,H]   my rows' outputs, in my sorted order
    uint32_t* ep_recv_counts = nullptr;  // [world][E_local] rows per (source, local expert)
    uint32_t* ep_plan_dev = nullptr;     // local_offsets[E_local+1] | seg_src | seg_dst  (each world*E_local)
    // exchange over peer memory (CUDA IPC): control window, peers' windows / row buffers / result buffers
    uint32_t* ep_win = nullptr;          // flags + counts matrix (exported)
    uint16_t* ep_y_bf = nullptr;         // [mx_rows, H] bf16 results of this rank's experts (exported; peers pull from it)
    uint32_t* ep_send_base = nullptr;    // [E] base of this rank's rows for expert e in the owner's row buffer
    ep::PeerPtrs ep_peer_win{}, ep_peer_rows{}, ep_peer_y{};
    std::vector<void*> ep_opened;        // IPC mappings to close
    bool ep_peer_on = false;
    const uint32_t* ep_rows_dev = nullptr;   // set while the experts run on rows whose count only the device knows
    uint32_t ep_epoch = 0;               // step counter of the peer exchange; never reset, so flags of earlier steps stay behind it
    uint64_t ep_wait_ns = ep::EP_WAIT_LIMIT_NS;   // limit of a peer barrier wait (option "ep_wait_ms")
    uint32_t* ep_pin = nullptr;          // pinned: recv_counts | offsets[E+1] | plan upload staging

    // host-buffer entry point
    cudaStream_t own_stream = nullptr;
    cudaStream_t h2d_stream = nullptr, d2h_stream = nullptr;   // host entry point, chunked form: copies beside the compute stream
    cudaEvent_t ev_in[4] = {}, ev_out[4] = {};
    int opt_host_chunks = 0;         // host entry point: 0 = large batches go through in up to 3 chunks, 1 = always whole, 2..4 = at most that many
    uint16_t* pin_x = nullptr;
    uint16_t* pin_out = nullptr;
    uint16_t* pin_res = nullptr;
    uint16_t* dev_x = nullptr;
    uint16_t* dev_out = nullptr;
    uint16_t* dev_res = nullptr;
    void* pin_dbg = nullptr;
    size_t pin_dbg_bytes = 0;

    // stage timing
    bool timing = false;
    cudaEvent_t ev[FFAI_N_STAGES][3][2]{};  // [stage][segment][begin/end]
    bool ev_made = false;
    int ev_segments[FFAI_N_STAGES]{};
    int launches = 0;
    void* nccl_comm = nullptr;
    std::string err;
};

namespace {

int fail(ffai_moe_layer* L, int status, const char* fmt, ...) {
    if (L) {
        char buf[512];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        L->err = buf;
    }
    return status;
}

#define CUDA_TRY(L, expr)                                                                   \
    do {                                                                                    \
        cudaError_t _e = (expr);                                                            \
        if (_e != cudaSuccess)                                                              \
            return fail((L), FFAI_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
    } while (0)

bool valid_bits(int b) { return b == 2 || b == 3 || b == 4 || b == 5 || b == 6 || b == 8; }
bool valid_gs(int g) { return g == 32 || g == 64 || g == 128; }
bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename T>
int ws_alloc(ffai_moe_layer* L, T** out, size_t count) {
    void* p = nullptr;
    if (count == 0) count = 1;
    CUDA_TRY(L, cudaMalloc(&p, count * sizeof(T)));
    L->owned_ws.push_back(p);
    *out = static_cast<T*>(p);
    return FFAI_OK;
}

size_t qproj_weight_bytes(int n, int out_dim, int in_dim, int bits) {
    return (size_t)n * out_dim * (size_t)(in_dim * bits / 32) * 4;
}
size_t qproj_group_bytes(int n, int out_dim, int in_dim, int gs) {
    return (size_t)n * out_dim * (size_t)(in_dim / gs) * 2;
}

int upload(ffai_moe_layer* L, const void* src, size_t bytes, int location, const void** dst) {
    *dst = nullptr;
    if (!src) return FFAI_OK;
    if (location == FFAI_MEM_DEVICE) {
        *dst = src;
        return FFAI_OK;
    }
    void* p = nullptr;
    CUDA_TRY(L, cudaMalloc(&p, bytes ? bytes : 1));
    L->owned_weights.push_back(p);
    CUDA_TRY(L, cudaMemcpy(p, src, bytes, cudaMemcpyHostToDevice));
    *dst = p;
    return FFAI_OK;
}

int upload_qproj(ffai_moe_layer* L, const ffai_qproj& src, int n, int out_dim, int in_dim, int bits,
                 int gs, int location, ffai_qproj* dst, const char* name) {
    if (!src.weight || !src.scales || !src.biases)
        return fail(L, FFAI_ERR_INVALID_ARG, "%s: weight/scales/biases must be non-null", name);
    int rc;
    if ((rc = upload(L, src.weight, qproj_weight_bytes(n, out_dim, in_dim, bits), location,
                     (const void**)&dst->weight)))
        return rc;
    if ((rc = upload(L, src.scales, qproj_group_bytes(n, out_dim, in_dim, gs), location,
                     (const void**)&dst->scales)))
        return rc;
    if ((rc = upload(L, src.biases, qproj_group_bytes(n, out_dim, in_dim, gs), location,
                     (const void**)&dst->biases)))
        return rc;
    if ((rc = upload(L, src.row_bias, (size_t)n * out_dim * 2, location, (const void**)&dst->row_bias)))
        return rc;
    if (!aligned16(dst->weight) || !aligned16(dst->scales) || !aligned16(dst->biases))
        return fail(L, FFAI_ERR_INVALID_ARG, "%s: device pointers must be 16-byte aligned", name);
    return FFAI_OK;
}

int upload_linear(ffai_moe_layer* L, const ffai_linear& src, int kind, int out_dim, int in_dim,
                  int bits, int gs, int location, ffai_linear* dst, const char* name) {
    if (!src.weight) return fail(L, FFAI_ERR_INVALID_ARG, "%s: weight must be non-null", name);
    size_t wbytes = 0;
    if (kind == FFAI_LINEAR_F32) wbytes = (size_t)out_dim * in_dim * 4;
    else if (kind == FFAI_LINEAR_BF16) wbytes = (size_t)out_dim * in_dim * 2;
    else wbytes = qproj_weight_bytes(1, out_dim, in_dim, bits);
    int rc;
    if ((rc = upload(L, src.weight, wbytes, location, &dst->weight))) return rc;
    if (kind == FFAI_LINEAR_AFFINE) {
        if (!src.scales || !src.biases)
            return fail(L, FFAI_ERR_INVALID_ARG, "%s: affine projection needs scales and biases", name);
        if ((rc = upload(L, src.scales, qproj_group_bytes(1, out_dim, in_dim, gs), location,
                         (const void**)&dst->scales)))
            return rc;
        if ((rc = upload(L, src.biases, qproj_group_bytes(1, out_dim, in_dim, gs), location,
                         (const void**)&dst->biases)))
            return rc;
    }
    if ((rc = upload(L, src.bias, (size_t)out_dim * 2, location, (const void**)&dst->bias))) return rc;
    if (!aligned16(dst->weight))
        return fail(L, FFAI_ERR_INVALID_ARG, "%s: device pointers must be 16-byte aligned", name);
    return FFAI_OK;
}

void free_list(std::vector<void*>& v) {
    for (void* p : v) cudaFree(p);
    v.clear();
}

// ───────────────────────────── launch helpers ─────────────────────────────

#define BITS_SWITCH(bits, ...)                                  \
    switch (bits) {                                             \
        case 2: { constexpr int B = 2; __VA_ARGS__; } break;    \
        case 3: { constexpr int B = 3; __VA_ARGS__; } break;    \
        case 4: { constexpr int B = 4; __VA_ARGS__; } break;    \
        case 5: { constexpr int B = 5; __VA_ARGS__; } break;    \
        case 6: { constexpr int B = 6; __VA_ARGS__; } break;    \
        case 8: { constexpr int B = 8; __VA_ARGS__; } break;    \
        default: return FFAI_ERR_INVALID_ARG;                   \
    }

// Launch with or without the programmatic-stream-serialization attribute (the kernel then calls pdl_wait before it
// reads anything its predecessor in the stream writes).
template <typename... KArgs, typename... Args>
cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl, Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename TIn, typename TOut, bool FUSED>
int launch_grouped_gemv(const GemvParams& p, int bits, const TIn* in, TOut* out, int expert_slots,
                        cudaStream_t st) {
    if (p.N <= 0 || p.n_rows <= 0) return FFAI_OK;
    dim3 grid((p.N + 3) / 4, expert_slots), block(128);
    BITS_SWITCH(bits, (grouped_gemv_kernel<B, TIn, TOut, FUSED><<<grid, block, 0, st>>>(p, in, out)));
    return cudaGetLastError() == cudaSuccess ? FFAI_OK : FFAI_ERR_CUDA;
}

template <int KIND>
int launch_router_kind(const RouterParams& p, const uint16_t* x, int T, uint32_t* idx, float* w,
                       float* logits, cudaStream_t st) {
    const int nchunks = (p.hidden + 63) / 64;
    const size_t smem = ((size_t)p.n_experts * nchunks + 2 * (size_t)p.n_experts) * sizeof(float);
    if (smem > 200 * 1024) return FFAI_ERR_UNSUPPORTED;
    const int work = p.n_experts * nchunks;
    int threads = work >= 512 ? 512 : ((work + 31) / 32) * 32;
    if (threads < 32) threads = 32;
    if (KIND == FFAI_LINEAR_AFFINE) {
        BITS_SWITCH(p.bits, {
            auto k = router_token_kernel<KIND, B>;
            if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            k<<<T, threads, smem, st>>>(p, x, T, idx, w, logits);
        });
    } else {
        auto k = router_token_kernel<KIND, 4>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        k<<<T, threads, smem, st>>>(p, x, T, idx, w, logits);
    }
    return cudaGetLastError() == cudaSuccess ? FFAI_OK : FFAI_ERR_CUDA;
}

template <int KIND, int BITS>
void launch_router_tiled(const RouterParams& p, const uint16_t* x, int T, float* logits, float* partials, int n_sms,
                         cudaStream_t st) {
    const int eb = (p.n_experts + 63) / 64;
    const unsigned z = partials ? p.hidden / 64 : 1;
    // smallest token tile whose grid still gives every SM a block
    if (((T + 63) / 64) * eb * (int)z >= n_sms) {
        router_logits_tiled_kernel<KIND, BITS, 64><<<dim3((T + 63) / 64, eb, z), 256, 0, st>>>(p, x, T, logits, partials);
    } else if (((T + 31) / 32) * eb * (int)z >= n_sms) {
        router_logits_tiled_kernel<KIND, BITS, 32><<<dim3((T + 31) / 32, eb, z), 128, 0, st>>>(p, x, T, logits, partials);
    } else {
        router_logits_tiled_kernel<KIND, BITS, 16><<<dim3((T + 15) / 16, eb, z), 64, 0, st>>>(p, x, T, logits, partials);
    }
}

// Many tokens: tiled projection, then one warp per token routes.  When the un-split grid would leave SMs
// idle and the chunk-sum buffer is available, the hidden axis is split over blockIdx.z (one 64-wide chunk
// per block) and the chunk sums are added in order by the routing kernel.  Returns launches or -1.
int launch_router_batched(const RouterParams& p, const uint16_t* x, int T, uint32_t* idx, float* w,
                          float* logits, float* partials, size_t partials_capacity, int n_sms, cudaStream_t st) {
    const int n_chunks = p.hidden / 64;
    // 128-token x 64-expert tiles with the next chunk's loads in flight behind the arithmetic (dense weights; a
    // quantized router arrives here expanded to fp32).  Long chunks give every SM a tile; mid-sized ones split the
    // hidden axis into ranges of chunks as well and leave the ordered sum of the chunks to the routing kernel.
    if ((p.kind == FFAI_LINEAR_F32 || p.kind == FFAI_LINEAR_BF16) && p.hidden % 64 == 0 && T >= 256) {
        const int tiles = ((T + RB_TOK - 1) / RB_TOK) * ((p.n_experts + RB_EXP - 1) / RB_EXP);
        int z = 1, per = n_chunks;
        float* part = nullptr;
        // measured at 256 experts: 128 tiles take 156 us un-split (one block per SM) against 169 us split three ways
        // with their 134 MB of chunk sums; 64 tiles take 87 us split and would take the same 156 us un-split
        if (tiles * 4 < n_sms * 3) {
            if (partials && (size_t)T * p.n_experts * n_chunks <= partials_capacity) {
                z = std::min(n_chunks, (2 * n_sms + tiles - 1) / tiles);
                per = (n_chunks + z - 1) / z;
                z = (n_chunks + per - 1) / per;
                part = partials;
            } else {
                z = 0;   // no room for the chunk sums: the smaller tiles below
            }
        }
        if (z > 0) {
            const dim3 grid((T + RB_TOK - 1) / RB_TOK, (p.n_experts + RB_EXP - 1) / RB_EXP, z);
            static SmemOptIn opt1, opt2;
            bool ok;
            if (p.kind == FFAI_LINEAR_F32) {
                ok = opt1.ensure(router_logits_big_kernel<1>, RB_SMEM);
                if (ok) router_logits_big_kernel<1><<<grid, 256, RB_SMEM, st>>>(p, x, T, logits, part, per);
            } else {
                ok = opt2.ensure(router_logits_big_kernel<2>, RB_SMEM);
                if (ok) router_logits_big_kernel<2><<<grid, 256, RB_SMEM, st>>>(p, x, T, logits, part, per);
            }
            if (ok) {
                const int warps = 4;
                const size_t smem = (size_t)warps * 2 * p.n_experts * sizeof(float);
                if (part) route_from_partials_kernel<<<(T + warps - 1) / warps, warps * 32, smem, st>>>(p, part, n_chunks, T, idx, w, logits);
                else route_only_kernel<<<(T + warps - 1) / warps, warps * 32, smem, st>>>(p, logits, T, idx, w);
                return cudaGetLastError() == cudaSuccess ? 2 : -1;
            }
        }
    }
    const bool few_blocks = ((T + 63) / 64) * ((p.n_experts + 63) / 64) < 4 * n_sms;
    if (!(partials && few_blocks && (size_t)T * p.n_experts * n_chunks <= partials_capacity)) partials = nullptr;
    switch (p.kind) {
        case FFAI_LINEAR_F32: launch_router_tiled<1, 4>(p, x, T, logits, partials, n_sms, st); break;
        case FFAI_LINEAR_BF16: launch_router_tiled<2, 4>(p, x, T, logits, partials, n_sms, st); break;
        case FFAI_LINEAR_AFFINE:
            BITS_SWITCH(p.bits, (launch_router_tiled<3, B>(p, x, T, logits, partials, n_sms, st)));
            break;
        default: return -1;
    }
    const int warps = 4;
    const size_t smem = (size_t)warps * 2 * p.n_experts * sizeof(float);
    if (partials)
        route_from_partials_kernel<<<(T + warps - 1) / warps, warps * 32, smem, st>>>(p, partials, n_chunks, T, idx, w, logits);
    else
        route_only_kernel<<<(T + warps - 1) / warps, warps * 32, smem, st>>>(p, logits, T, idx, w);
    return cudaGetLastError() == cudaSuccess ? 2 : -1;
}

// Few tokens, dense router weights: staged rows + last-block routing.  Returns 0, or -1 when the
// shape does not fit (the caller then uses router_token_kernel).
template <int KIND>
int launch_router_rows(const RouterParams& p, const uint16_t* x, int T, uint32_t* idx, float* w, float* logits,
                       uint32_t* tickets, const PlanOut& plan, uint16_t* x_perm8, float* x_sum64, int sum_pitch, cudaStream_t st) {
    const int wbytes = KIND == 1 ? 4 : 2;
    // rows per block: 8, or fewer while the grid would leave most SMs without a block (a one-token step reads the
    // router's weights through E / rows blocks only)
    int rpb = ROUTER_ROWS;
    while (rpb > 1 && ((p.n_experts + rpb - 1) / rpb) * T < 64) rpb >>= 1;
    const size_t smem = (size_t)rpb * p.hidden * wbytes + (size_t)p.hidden * 2 +
                        (size_t)rpb * (p.hidden / 64) * 4 + 2 * (size_t)p.n_experts * 4;
    if (smem > 200 * 1024 || p.hidden % 64 || T > ROUTER_BATCH_TICKET) return -1;
    auto k = router_rows_kernel<KIND>;
    static SmemOptIn opt_in;
    if (smem > 48 * 1024 && !opt_in.ensure(k, (int)smem)) return -1;
    dim3 grid((p.n_experts + rpb - 1) / rpb, T);
    k<<<grid, 256, smem, st>>>(p, x, T, idx, w, logits, tickets, plan, x_perm8, x_sum64, sum_pitch, rpb);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int launch_router(const RouterParams& p, const uint16_t* x, int T, uint32_t* idx, float* w,
                  float* logits, cudaStream_t st) {
    switch (p.kind) {
        case FFAI_LINEAR_F32: return launch_router_kind<FFAI_LINEAR_F32>(p, x, T, idx, w, logits, st);
        case FFAI_LINEAR_BF16: return launch_router_kind<FFAI_LINEAR_BF16>(p, x, T, idx, w, logits, st);
        case FFAI_LINEAR_AFFINE: return launch_router_kind<FFAI_LINEAR_AFFINE>(p, x, T, idx, w, logits, st);
    }
    return FFAI_ERR_INVALID_ARG;
}

// returns number of launches, or -1 on error
// When tile_offsets is given and the one-block form ran, *tiles_done is set and tile_offsets holds the
// token-tile schedule for tile_rows rows per tile.
int launch_plan(const uint32_t* indices, int n_rows, int E, uint32_t* counts, uint32_t* offsets,
                uint32_t* perm, uint32_t* inv_perm, uint32_t* block_hist, cudaStream_t st,
                int tile_rows = 0, uint32_t* tile_offsets = nullptr, bool* tiles_done = nullptr) {
    if (n_rows <= PLAN_ENTRIES_PER_WARP) {
        plan_small_kernel<<<1, 32, 2 * E * sizeof(uint32_t), st>>>(indices, n_rows, E, counts, offsets,
                                                                  perm, inv_perm);
        return cudaGetLastError() == cudaSuccess ? 1 : -1;
    }
    const int nb = plan_num_blocks(n_rows);
    if (nb <= PLAN_BLOCK_MAX_WARPS) {
        const int run_len = plan_block_run_len(n_rows);
        const int n_warps = (n_rows + run_len - 1) / run_len;
        const size_t lean_smem = plan_block_smem(n_warps, E, 0), staged_smem = plan_block_smem(n_warps, E, n_rows);
        const bool staged = staged_smem <= 200 * 1024;
        const size_t block_smem = staged ? staged_smem : lean_smem;
        static SmemOptIn opt_in;
        if (block_smem <= 200 * 1024 && (block_smem <= 48 * 1024 || opt_in.ensure(plan_block_kernel, (int)block_smem))) {
            const PlanOut o{counts, offsets, perm, inv_perm, nullptr};
            const bool tiles = tile_offsets != nullptr && tile_rows > 0;
            plan_block_kernel<<<1, n_warps * 32, block_smem, st>>>(indices, n_rows, E, run_len, o, tile_rows,
                                                                   tiles ? tile_offsets : nullptr, staged ? 1 : 0);
            if (tiles && tiles_done) *tiles_done = true;
            return cudaGetLastError() == cudaSuccess ? 1 : -1;
        }
    }
    plan_count_kernel<<<nb, 32, E * sizeof(uint32_t), st>>>(indices, n_rows, E, block_hist);
    const bool tiles3 = tile_offsets != nullptr && tile_rows > 0;
    plan_scan_kernel<<<1, 256, (E + 1) * sizeof(uint32_t), st>>>(block_hist, nb, E, counts, offsets, tile_rows,
                                                                tiles3 ? tile_offsets : nullptr);
    if (tiles3 && tiles_done) *tiles_done = true;
    plan_scatter_kernel<<<nb, 32, E * sizeof(uint32_t), st>>>(indices, n_rows, E, block_hist, perm, inv_perm);
    return cudaGetLastError() == cudaSuccess ? 3 : -1;
}

template <bool FUSED, int NT, int KSPLIT, bool G32>
void launch_mma_decode_k(const dmma::Params& p, int n_experts, cudaStream_t st, bool pdl) {
    using WS = dmma::WarpStage<FUSED, G32>;
    auto k = dmma::grouped_mma_decode_kernel<FUSED, NT, KSPLIT, G32>;
    const int smem = WS::smem_bytes(p.K / 64, KSPLIT);
    static SmemOptIn opt_in;
    opt_in.ensure(k, smem);   // a failure shows as a launch error, which the caller reports
    const int rbw = 4 / KSPLIT;
    const int row_blocks = (FUSED && p.pair) ? (p.N + 31) / 32 : p.N / 16;   // 16-row blocks, or 32-row pairs
    dim3 grid((row_blocks + rbw - 1) / rbw, n_experts);
    launch_kernel(k, grid, dim3(128), (size_t)smem, st, pdl, p);
}

template <bool FUSED, bool G32>
void launch_mma_decode_g(const dmma::Params& p, int n_experts, int nt, int ksplit, cudaStream_t st, bool pdl) {
    if (nt == 2) {
        if (ksplit == 4) launch_mma_decode_k<FUSED, 2, 4, G32>(p, n_experts, st, pdl);
        else if (ksplit == 2) launch_mma_decode_k<FUSED, 2, 2, G32>(p, n_experts, st, pdl);
        else launch_mma_decode_k<FUSED, 2, 1, G32>(p, n_experts, st, pdl);
    } else {
        if (ksplit == 4) launch_mma_decode_k<FUSED, 1, 4, G32>(p, n_experts, st, pdl);
        else if (ksplit == 2) launch_mma_decode_k<FUSED, 1, 2, G32>(p, n_experts, st, pdl);
        else launch_mma_decode_k<FUSED, 1, 1, G32>(p, n_experts, st, pdl);
    }
}

// nt: 8-row activation tiles per pass (1 or 2); ksplit: slices of the reduction axis per 16-row block (1, 2, 4);
// the group size (p.group_size) picks the 32-run variant
template <bool FUSED>
void launch_mma_decode(const dmma::Params& p, int n_experts, int nt, int ksplit, cudaStream_t st, bool pdl = false) {
    if (p.group_size == 32) launch_mma_decode_g<FUSED, true>(p, n_experts, nt, ksplit, st, pdl);
    else launch_mma_decode_g<FUSED, false>(p, n_experts, nt, ksplit, st, pdl);
}

// Bulk-copy streamed decode kernels.  team: warps that share one 16-row block (4, or 16 for the smallest batches).
// Returns false when the shape does not fit the kernel's shared memory (the caller then uses the cp.async kernels).
template <bool FUSED, int TEAM, int CPU, int DEPTH>
bool launch_stream_decode_t(const dstr::Params& p, int n_sms, cudaStream_t st, bool pdl) {
    using LY = dstr::Layout<FUSED, TEAM, CPU, DEPTH>;
    const int smem = LY::total(p.n_experts, p.K);
    if (smem > 227 * 1024) return false;
    auto k = dstr::stream_decode_kernel<FUSED, TEAM, CPU, DEPTH>;
    static SmemOptIn opt_in;
    if (!opt_in.ensure(k, smem)) return false;
    return launch_kernel(k, dim3(n_sms), dim3(dstr::THREADS), (size_t)smem, st, pdl, p) == cudaSuccess;
}
template <bool FUSED>
bool launch_stream_decode(const dstr::Params& p, int team, int n_sms, cudaStream_t st, bool pdl) {
    constexpr int CPU2 = FUSED ? 1 : 2;
    if (team == 16) return launch_stream_decode_t<FUSED, 16, 1, 5>(p, n_sms, st, pdl) || launch_stream_decode_t<FUSED, 16, 1, 3>(p, n_sms, st, pdl);
    if (team == 4) return launch_stream_decode_t<FUSED, 4, CPU2, 5>(p, n_sms, st, pdl) || launch_stream_decode_t<FUSED, 4, CPU2, 3>(p, n_sms, st, pdl);
    return launch_stream_decode_t<FUSED, 1, CPU2, 6>(p, n_sms, st, pdl) || launch_stream_decode_t<FUSED, 1, CPU2, 3>(p, n_sms, st, pdl);
}

// dense [1,H] projection per token (shared-expert gate stored as f32 / bf16)
template <typename TW>
__global__ void dense_rowdot_kernel(const TW* __restrict__ w, const uint16_t* __restrict__ x,
                                    float* __restrict__ out, int n_tokens, int hidden) {
    const int warps = blockDim.x / 32;
    const int t = blockIdx.x * warps + threadIdx.x / 32;
    if (t >= n_tokens) return;
    const int lane = threadIdx.x & 31;
    float acc = 0.0f;
    for (int k = lane; k < hidden; k += 32) {
        float wv;
        if (sizeof(TW) == 4) wv = ((const float*)w)[k];
        else wv = bf16_bits_to_f32(((const uint16_t*)w)[k]);
        acc = fmaf(wv, bf16_bits_to_f32(x[(size_t)t * hidden + k]), acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) out[t] = acc;
}

// A quantized router expanded to fp32 once at load time: w = fma(scale, q, bias), the value the
// quantized projection uses for every product (FFAI Layers.swift:201-210), so the dense fp32 router
// kernels give the same logits bit for bit and the per-use unpacking disappears (E*H*4 bytes).
template <int BITS>
__global__ void expand_router_f32_kernel(const uint32_t* __restrict__ weight, const uint16_t* __restrict__ scales,
                                         const uint16_t* __restrict__ biases, float* __restrict__ out,
                                         int rows, int K, int group_size) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)rows * K) return;
    const size_t row = i / K;
    const int k = (int)(i - row * K);
    const uint32_t* w = weight + row * ((size_t)K * BITS / 32);
    const size_t g = row * (K / group_size) + k / group_size;
    out[i] = __fmaf_rn(bf16_bits_to_f32(scales[g]), (float)unpack_at<BITS>(w, k), bf16_bits_to_f32(biases[g]));
}

// One projection expanded to bf16 as the tensor-core kernel's operand tiles: w = fma(q, scale, bias) rounded
// once, every 8-run stored as 0,4,1,5,2,6,3,7 (one 16-byte chunk).  The cache is tile-major: for every
// (expert, block of 128 rows, 64-k block) the 16 KB operand tile sits contiguously and already 128-byte
// swizzled (row r of the block at r * 128 bytes, chunk c at ((c ^ (r & 7)) * 16)), so the kernel's weight
// producer brings a tile in with one contiguous bulk copy.  blocks_per_expert may exceed ceil(n_out / 128):
// rows past n_out stay zero (the buffer is cleared first).  One thread per 8-run.  Runs once, at load time.
template <int BITS>
__global__ void expand_to_bf16_tiles_kernel(const uint32_t* __restrict__ weight, const uint16_t* __restrict__ scales,
                                            const uint16_t* __restrict__ biases, uint16_t* __restrict__ out,
                                            size_t rows, int n_out, int blocks_per_expert, int K, int group_size) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int runs = K / 8;
    if (i >= rows * runs) return;
    const size_t row = i / runs;
    const int run = (int)(i - row * runs);
    const uint32_t* w = weight + row * ((size_t)K * BITS / 32);
    const int gpr = K / group_size;
    const float s = bf16_bits_to_f32(scales[row * gpr + (run * 8) / group_size]);
    const float b = bf16_bits_to_f32(biases[row * gpr + (run * 8) / group_size]);
    uint16_t v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = f32_to_bf16_bits(fmaf((float)unpack_at<BITS>(w, run * 8 + j), s, b));
    uint4 o;
    o.x = (uint32_t)v[0] | ((uint32_t)v[4] << 16);
    o.y = (uint32_t)v[1] | ((uint32_t)v[5] << 16);
    o.z = (uint32_t)v[2] | ((uint32_t)v[6] << 16);
    o.w = (uint32_t)v[3] | ((uint32_t)v[7] << 16);
    const size_t e = row / n_out;
    const int rp = (int)(row - e * n_out);
    const int rb = rp >> 7, r = rp & 127, kb = run >> 3, c = run & 7;
    const size_t tile = (e * blocks_per_expert + rb) * (size_t)(K / 64) + kb;
    uint8_t* dst = reinterpret_cast<uint8_t*>(out) + tile * 16384 + (size_t)r * 128 + (size_t)((c ^ (r & 7)) << 4);
    *reinterpret_cast<uint4*>(dst) = o;
}

// 128-row blocks per expert in a tile-major cache: a gate/up stage takes block m of each projection, a down
// stage takes blocks 2m and 2m+1, so down rounds its count up to an even number (the extra block stays zero).
int cache_blocks(int n_out, bool fused) { return fused ? (n_out + 127) / 128 : 2 * ((n_out + 255) / 256); }

// Size in bytes of a tile-major cache.
size_t cache_tiles_bytes(size_t n_groups, int blocks_per_expert, int K) {
    return n_groups * blocks_per_expert * (size_t)(K / 64) * 16384;
}

int launch_expand_to_bf16(const ffai_qproj& q, uint16_t* out, size_t n_groups, int n_out, int blocks_per_expert, int K,
                          int bits, int gs) {
    const size_t rows = n_groups * n_out;
    const size_t n = rows * (K / 8);
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (cudaMemset(out, 0, cache_tiles_bytes(n_groups, blocks_per_expert, K)) != cudaSuccess) return FFAI_ERR_CUDA;
    switch (bits) {
        case 2: expand_to_bf16_tiles_kernel<2><<<blocks, 256>>>(q.weight, q.scales, q.biases, out, rows, n_out, blocks_per_expert, K, gs); break;
        case 3: expand_to_bf16_tiles_kernel<3><<<blocks, 256>>>(q.weight, q.scales, q.biases, out, rows, n_out, blocks_per_expert, K, gs); break;
        case 4: expand_to_bf16_tiles_kernel<4><<<blocks, 256>>>(q.weight, q.scales, q.biases, out, rows, n_out, blocks_per_expert, K, gs); break;
        case 5: expand_to_bf16_tiles_kernel<5><<<blocks, 256>>>(q.weight, q.scales, q.biases, out, rows, n_out, blocks_per_expert, K, gs); break;
        case 6: expand_to_bf16_tiles_kernel<6><<<blocks, 256>>>(q.weight, q.scales, q.biases, out, rows, n_out, blocks_per_expert, K, gs); break;
        case 8: expand_to_bf16_tiles_kernel<8><<<blocks, 256>>>(q.weight, q.scales, q.biases, out, rows, n_out, blocks_per_expert, K, gs); break;
        default: return FFAI_ERR_INVALID_ARG;
    }
    return cudaGetLastError() == cudaSuccess ? FFAI_OK : FFAI_ERR_CUDA;
}

// [1,H] affine-quantized projection per token (the shared expert's sigmoid gate): one warp per token,
// fp32 accumulation, lanes take 8-runs round robin, fixed-shape warp reduction.
template <int BITS>
__global__ void affine_rowdot_kernel(const uint32_t* __restrict__ w, const uint16_t* __restrict__ scales,
                                     const uint16_t* __restrict__ biases, const uint16_t* __restrict__ x,
                                     float* __restrict__ out, int n_tokens, int hidden, int group_size) {
    const int warps = blockDim.x / 32;
    const int t = blockIdx.x * warps + threadIdx.x / 32;
    if (t >= n_tokens) return;
    const int lane = threadIdx.x & 31;
    const uint16_t* xr = x + (size_t)t * hidden;
    float acc = 0.0f;
    for (int k0 = lane * 8; k0 < hidden; k0 += 256) {
        const float s = bf16_bits_to_f32(scales[k0 / group_size]);
        const float b = bf16_bits_to_f32(biases[k0 / group_size]);
        const uint4 xv = *reinterpret_cast<const uint4*>(xr + k0);
        const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float wv = fmaf((float)unpack_at<BITS>(w, k0 + j), s, b);
            const float xf = (j & 1) ? bf16hi(xw[j >> 1]) : bf16lo(xw[j >> 1]);
            acc = fmaf(wv, xf, acc);
        }
    }
    acc = warp_sum(acc);
    if (lane == 0) out[t] = acc;
}

int launch_affine_rowdot(const ffai_linear& g, int bits, int gs, const uint16_t* x, float* out, int T, int H, cudaStream_t st) {
    const uint32_t* w = (const uint32_t*)g.weight;
    const unsigned blocks = (unsigned)((T + 3) / 4);
    switch (bits) {
        case 2: affine_rowdot_kernel<2><<<blocks, 128, 0, st>>>(w, g.scales, g.biases, x, out, T, H, gs); break;
        case 3: affine_rowdot_kernel<3><<<blocks, 128, 0, st>>>(w, g.scales, g.biases, x, out, T, H, gs); break;
        case 4: affine_rowdot_kernel<4><<<blocks, 128, 0, st>>>(w, g.scales, g.biases, x, out, T, H, gs); break;
        case 5: affine_rowdot_kernel<5><<<blocks, 128, 0, st>>>(w, g.scales, g.biases, x, out, T, H, gs); break;
        case 6: affine_rowdot_kernel<6><<<blocks, 128, 0, st>>>(w, g.scales, g.biases, x, out, T, H, gs); break;
        case 8: affine_rowdot_kernel<8><<<blocks, 128, 0, st>>>(w, g.scales, g.biases, x, out, T, H, gs); break;
        default: return FFAI_ERR_INVALID_ARG;
    }
    return cudaGetLastError() == cudaSuccess ? FFAI_OK : FFAI_ERR_CUDA;
}

enum Stage { ST_ROUTER = 0, ST_PLAN, ST_GATHER, ST_GATE_UP, ST_DOWN, ST_COMBINE, ST_SHARED, ST_EXCHANGE };

// A stage may run in up to three segments per forward (the exchange does).
void stage_begin(ffai_moe_layer* L, int stage, cudaStream_t st) {
    if (!L->timing || L->ev_segments[stage] >= 3) return;
    cudaEventRecord(L->ev[stage][L->ev_segments[stage]][0], st);
}
void stage_end(ffai_moe_layer* L, int stage, cudaStream_t st) {
    if (!L->timing || L->ev_segments[stage] >= 3) return;
    cudaEventRecord(L->ev[stage][L->ev_segments[stage]][1], st);
    L->ev_segments[stage] += 1;
}

int validate_config(const ffai_moe_config* c, ffai_moe_layer* L) {
    if (c->struct_size != sizeof(ffai_moe_config))
        return fail(L, FFAI_ERR_INVALID_ARG, "config.struct_size %u != %zu", c->struct_size, sizeof(ffai_moe_config));
    if (c->hidden <= 0 || c->hidden % 64) return fail(L, FFAI_ERR_INVALID_ARG, "hidden must be a positive multiple of 64");
    if (c->intermediate <= 0 || c->intermediate % 64) return fail(L, FFAI_ERR_INVALID_ARG, "intermediate must be a positive multiple of 64");
    // MoERouter.init preconditions, MoELayer.swift:109-118
    if (c->n_experts <= 0 || c->n_experts > FFAI_MAX_EXPERTS) return fail(L, FFAI_ERR_INVALID_ARG, "n_experts must be in 1..%d", FFAI_MAX_EXPERTS);
    if (c->top_k <= 0 || c->top_k > c->n_experts || c->top_k > FFAI_MAX_TOP_K)
        return fail(L, FFAI_ERR_INVALID_ARG, "top_k (%d) must be in 1..min(n_experts=%d, %d)", c->top_k, c->n_experts, FFAI_MAX_TOP_K);
    if (c->gating_mode < FFAI_GATING_SOFTMAX_THEN_TOPK || c->gating_mode > FFAI_GATING_SIGMOID_TOPK)
        return fail(L, FFAI_ERR_INVALID_ARG, "unknown gating_mode %d", c->gating_mode);
    if (c->activation < 0 || c->activation > FFAI_ACT_RELU2) return fail(L, FFAI_ERR_INVALID_ARG, "unknown activation %d", c->activation);
    if (c->router_kind < FFAI_LINEAR_F32 || c->router_kind > FFAI_LINEAR_AFFINE) return fail(L, FFAI_ERR_INVALID_ARG, "unknown router_kind %d", c->router_kind);
    if (c->router_kind == FFAI_LINEAR_AFFINE && (!valid_bits(c->router_bits) || !valid_gs(c->router_group_size)))
        return fail(L, FFAI_ERR_INVALID_ARG, "router bits/group_size (%d/%d) unsupported", c->router_bits, c->router_group_size);
    if (!valid_bits(c->expert_bits) || !valid_gs(c->expert_group_size))
        return fail(L, FFAI_ERR_INVALID_ARG, "expert bits/group_size (%d/%d) unsupported", c->expert_bits, c->expert_group_size);
    if (c->shared_intermediate < 0 || c->shared_intermediate % 64) return fail(L, FFAI_ERR_INVALID_ARG, "shared_intermediate must be a multiple of 64");
    if (c->shared_intermediate > 0) {
        if (!valid_bits(c->shared_bits) || !valid_gs(c->shared_group_size))
            return fail(L, FFAI_ERR_INVALID_ARG, "shared bits/group_size (%d/%d) unsupported", c->shared_bits, c->shared_group_size);
        if (c->shared_gate_kind < FFAI_LINEAR_NONE || c->shared_gate_kind > FFAI_LINEAR_AFFINE)
            return fail(L, FFAI_ERR_INVALID_ARG, "unknown shared_gate_kind %d", c->shared_gate_kind);
        if (c->shared_gate_kind == FFAI_LINEAR_AFFINE && (!valid_bits(c->shared_gate_bits) || !valid_gs(c->shared_gate_group_size)))
            return fail(L, FFAI_ERR_INVALID_ARG, "shared gate bits/group_size unsupported");
    }
    if (c->max_tokens <= 0) return fail(L, FFAI_ERR_INVALID_ARG, "max_tokens must be positive");
    if ((int64_t)c->max_tokens * c->top_k > (int64_t)1 << 30) return fail(L, FFAI_ERR_INVALID_ARG, "max_tokens*top_k too large");
    const int world = c->ep_world <= 1 ? 1 : c->ep_world;
    if (c->n_experts % world) return fail(L, FFAI_ERR_INVALID_ARG, "n_experts must divide evenly over ep_world");
    if (c->ep_rank < 0 || c->ep_rank >= world) return fail(L, FFAI_ERR_INVALID_ARG, "ep_rank out of range");
    return FFAI_OK;
}

}  // namespace

// ───────────────────────────── probes ─────────────────────────────

extern "C" FFAI_API int ffai_cuda_abi_version(void) { return FFAI_CUDA_ABI_VERSION; }

extern "C" FFAI_API int ffai_cuda_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

extern "C" FFAI_API const char* ffai_status_string(int status) {
    switch (status) {
        case FFAI_OK: return "ok";
        case FFAI_ERR_INVALID_ARG: return "invalid argument";
        case FFAI_ERR_UNSUPPORTED: return "unsupported";
        case FFAI_ERR_CUDA: return "CUDA error";
        case FFAI_ERR_NOT_READY: return "weights not set";
        case FFAI_ERR_NCCL: return "NCCL error";
        case FFAI_ERR_DEVICE_CHECK: return "device-side check failed";
    }
    return "unknown status";
}

// ───────────────────────────── lifecycle ─────────────────────────────

extern "C" FFAI_API int ffai_moe_create(const ffai_moe_config* config, ffai_moe_layer** out_layer) {
    if (!config || !out_layer) return FFAI_ERR_INVALID_ARG;
    *out_layer = nullptr;
    ffai_moe_layer* L = new (std::nothrow) ffai_moe_layer();
    if (!L) return FFAI_ERR_CUDA;
    int rc = validate_config(config, L);
    if (rc != FFAI_OK) {
        // hand the object back so the caller can read the message, but mark it unusable
        L->cfg = ffai_moe_config{};
        *out_layer = L;
        return rc;
    }
    L->cfg = *config;
    const ffai_moe_config& c = L->cfg;
    const int world = c.ep_world <= 1 ? 1 : c.ep_world;
    L->e_local = c.n_experts / world;
    L->no_gate = c.activation == FFAI_ACT_RELU2;
    *out_layer = L;
    if (ffai_cuda_device_count() <= 0) return fail(L, FFAI_ERR_CUDA, "no CUDA device available (there is no CPU fallback)");
    CUDA_TRY(L, cudaGetDevice(&L->device));

    const size_t T = c.max_tokens, K = c.top_k, E = c.n_experts, H = c.hidden, I = c.intermediate;
    const size_t M = T * K;
    const size_t Mx = M * (size_t)world;   // rows that can arrive at this rank under expert parallelism
    L->mx_rows = Mx;
    if ((rc = ws_alloc(L, &L->logits, T * E))) return rc;
    if ((rc = ws_alloc(L, &L->indices, M))) return rc;
    if ((rc = ws_alloc(L, &L->rweights, M))) return rc;
    if ((rc = ws_alloc(L, &L->counts, E))) return rc;
    if ((rc = ws_alloc(L, &L->offsets, E + 1))) return rc;
    if ((rc = ws_alloc(L, &L->perm, M))) return rc;
    if ((rc = ws_alloc(L, &L->inv_perm, M))) return rc;
    if ((rc = ws_alloc(L, &L->block_hist, (size_t)plan_num_blocks((int)M) * E))) return rc;
    if (T >= 96 && T * E * (H / 64) * sizeof(float) <= (size_t)256 << 20) {
        L->router_partials_cap = T * E * (H / 64);
        if ((rc = ws_alloc(L, &L->router_partials, L->router_partials_cap))) return rc;
    }
    if ((rc = ws_alloc(L, &L->expert_order, E))) return rc;
    if ((rc = ws_alloc(L, &L->tickets, ROUTER_TICKETS))) return rc;
    CUDA_TRY(L, cudaMemset(L->tickets, 0, ROUTER_TICKETS * sizeof(uint32_t)));
    if ((rc = ws_alloc(L, &L->inner, Mx * I))) return rc;
    if ((rc = ws_alloc(L, &L->y, Mx * H))) return rc;
    if (world > 1) {
        const size_t El = L->e_local, W = world;
        if ((rc = ws_alloc(L, &L->ep_send_x, M * H))) return rc;
        if ((rc = ws_alloc(L, &L->ep_recv_x, Mx * H))) return rc;
        if ((rc = ws_alloc(L, &L->ep_ret_y, Mx * H))) return rc;
        if ((rc = ws_alloc(L, &L->ep_home_y, M * H))) return rc;
        if ((rc = ws_alloc(L, &L->ep_recv_counts, W * El))) return rc;
        if ((rc = ws_alloc(L, &L->ep_plan_dev, (El + 1) + 2 * W * El))) return rc;
        if (W > (size_t)ep::EP_MAX_WORLD) return fail(L, FFAI_ERR_INVALID_ARG, "ep_world %zu exceeds %d", W, ep::EP_MAX_WORLD);
        // exported to the peers: a whole 2 MiB granule of its own, so the mapping a peer opens holds nothing else
        const size_t win_words = std::max(ep::win_words((int)W, (int)E), (size_t)(2u << 20) / sizeof(uint32_t));
        if ((rc = ws_alloc(L, &L->ep_win, win_words))) return rc;
        CUDA_TRY(L, cudaMemset(L->ep_win, 0, win_words * sizeof(uint32_t)));
        if ((rc = ws_alloc(L, &L->ep_send_base, E))) return rc;
        if ((rc = ws_alloc(L, &L->ep_y_bf, Mx * H))) return rc;
        void* pin = nullptr;
        CUDA_TRY(L, cudaMallocHost(&pin, sizeof(uint32_t) * (W * El + (E + 1) + (El + 1) + 2 * W * El)));
        L->owned_pinned.push_back(pin);
        L->ep_pin = static_cast<uint32_t*>(pin);
    }
    if (c.shared_intermediate > 0) {
        if ((rc = ws_alloc(L, &L->sh_inner, T * c.shared_intermediate))) return rc;
        if ((rc = ws_alloc(L, &L->sh_y, T * H))) return rc;
        if ((rc = ws_alloc(L, &L->sh_gate, T))) return rc;
    }
    if ((rc = ws_alloc(L, &L->error_word, 1))) return rc;
    CUDA_TRY(L, cudaMemset(L->error_word, 0, 4));
    CUDA_TRY(L, cudaDeviceGetAttribute(&L->n_sms, cudaDevAttrMultiProcessorCount, L->device));
    int cc_major = 0;
    CUDA_TRY(L, cudaDeviceGetAttribute(&cc_major, cudaDevAttrComputeCapabilityMajor, L->device));
    // 4-bit experts: bf16 staging buffers shared by the register-streaming decode kernels and the
    // tcgen05 grouped GEMM.  The tcgen05 path also needs every reduction length to hold at least one
    // 256-k packed TMA box.
    const bool tc_shapes = H >= 256 && I >= 256 && (c.shared_intermediate == 0 || c.shared_intermediate >= 256);
    const bool want_tc = cc_major == 10 && tc_shapes && !L->no_gate;
    {
        const double cache_bytes = 3.0 * (double)L->e_local * H * I * 2.0;
        const bool prefill_sized = (double)T * K / E >= 32.0;
        L->cache_planned = want_tc && c.prefill_weight_cache != 1 &&
                           (c.prefill_weight_cache == 2 || (prefill_sized && cache_bytes <= 4.0 * 1073741824.0));
    }
    if (c.expert_bits == 4 || (want_tc && (c.shared_intermediate > 0 || L->cache_planned))) {
        const size_t Mp = Mx < 128 ? 128 : Mx, Tp = T < 128 ? 128 : T;  // at least one full TMA box of rows
        if ((rc = ws_alloc(L, &L->xg, Mp * H))) return rc;
        if ((rc = ws_alloc(L, &L->inner_bf, Mp * I))) return rc;
        // 64-run sums, row pitch rounded up to 4 floats (16-byte rows for cp.async), + one spare row
        if ((rc = ws_alloc(L, &L->xsum, (Mx + 1) * (size_t)((H / 32 + 3) & ~3)))) return rc;
        if ((rc = ws_alloc(L, &L->inner_sum, (Mx + 1) * (size_t)((I / 32 + 3) & ~3)))) return rc;
        if ((rc = ws_alloc(L, &L->inner_parts, (Mx + 1) * (size_t)(I / 16)))) return rc;
        if ((rc = ws_alloc(L, &L->x_tok, (T + 1) * H))) return rc;
        if ((rc = ws_alloc(L, &L->xsum_tok, (T + 1) * (size_t)((H / 32 + 3) & ~3)))) return rc;
        L->mma_ok = c.expert_bits == 4 && !L->no_gate;   // every group size the format allows (32, 64, 128)
        if (want_tc) {
            if (world == 1 && (rc = ws_alloc(L, &L->y_bf, M * H))) return rc;
            if ((rc = ws_alloc(L, &L->tile_offsets, E + 1))) return rc;
            if (c.shared_intermediate > 0) {
                if ((rc = ws_alloc(L, &L->sh_x, Tp * H))) return rc;
                if ((rc = ws_alloc(L, &L->sh_inner_bf, Tp * c.shared_intermediate))) return rc;
                if ((rc = ws_alloc(L, &L->sh_sched, 4))) return rc;
            }
        }
    }
    if (world > 1 && !L->xg && (rc = ws_alloc(L, &L->xg, Mx * H))) return rc;  // regrouped rows for the GEMV path
    return FFAI_OK;
}

extern "C" FFAI_API int ffai_moe_set_weights(ffai_moe_layer* L, const ffai_moe_weights* w) {
    if (!L || !w) return FFAI_ERR_INVALID_ARG;
    if (L->cfg.struct_size == 0) return fail(L, FFAI_ERR_INVALID_ARG, "layer was not created successfully");
    if (w->struct_size != sizeof(ffai_moe_weights))
        return fail(L, FFAI_ERR_INVALID_ARG, "weights.struct_size %u != %zu", w->struct_size, sizeof(ffai_moe_weights));
    if (w->location != FFAI_MEM_HOST && w->location != FFAI_MEM_DEVICE)
        return fail(L, FFAI_ERR_INVALID_ARG, "unknown weights.location %d", w->location);
    const ffai_moe_config& c = L->cfg;
    CUDA_TRY(L, cudaSetDevice(L->device));
    free_list(L->owned_weights);
    L->sh_wbf[0] = L->sh_wbf[1] = L->sh_wbf[2] = nullptr;
    L->exp_wbf[0] = L->exp_wbf[1] = L->exp_wbf[2] = nullptr;
    L->weights_set = false;
    L->w = ffai_moe_weights{};
    int rc;
    const int loc = w->location;
    if ((rc = upload_linear(L, w->router, c.router_kind, c.n_experts, c.hidden, c.router_bits,
                            c.router_group_size, loc, &L->w.router, "router")))
        return rc;
    L->router_f32 = nullptr;
    if (c.router_kind == FFAI_LINEAR_AFFINE) {
        void* buf = nullptr;
        const size_t n = (size_t)c.n_experts * c.hidden;
        CUDA_TRY(L, cudaMalloc(&buf, n * sizeof(float)));
        L->owned_weights.push_back(buf);
        L->router_f32 = static_cast<float*>(buf);
        const unsigned blocks = (unsigned)((n + 255) / 256);
        const uint32_t* rw = static_cast<const uint32_t*>(L->w.router.weight);
        BITS_SWITCH(c.router_bits, (expand_router_f32_kernel<B><<<blocks, 256>>>(rw, L->w.router.scales, L->w.router.biases, L->router_f32,
                                                                                c.n_experts, c.hidden, c.router_group_size)));
        CUDA_TRY(L, cudaGetLastError());
        CUDA_TRY(L, cudaDeviceSynchronize());
    }
    if (c.router_has_bias && !w->router.bias) return fail(L, FFAI_ERR_INVALID_ARG, "router_has_bias set but router.bias is null");
    if (!c.router_has_bias) L->w.router.bias = nullptr;
    if (c.router_expert_bias) {
        if (!w->router_expert_bias) return fail(L, FFAI_ERR_INVALID_ARG, "router_expert_bias set but pointer is null");
        if ((rc = upload(L, w->router_expert_bias, (size_t)c.n_experts * 4, loc, (const void**)&L->w.router_expert_bias))) return rc;
    }
    if (w->router_per_expert_scale)
        if ((rc = upload(L, w->router_per_expert_scale, (size_t)c.n_experts * 4, loc, (const void**)&L->w.router_per_expert_scale))) return rc;
    const int El = L->e_local;
    if (!L->no_gate && (rc = upload_qproj(L, w->gate_proj, El, c.intermediate, c.hidden, c.expert_bits, c.expert_group_size, loc, &L->w.gate_proj, "gate_proj"))) return rc;
    if ((rc = upload_qproj(L, w->up_proj, El, c.intermediate, c.hidden, c.expert_bits, c.expert_group_size, loc, &L->w.up_proj, "up_proj"))) return rc;
    if ((rc = upload_qproj(L, w->down_proj, El, c.hidden, c.intermediate, c.expert_bits, c.expert_group_size, loc, &L->w.down_proj, "down_proj"))) return rc;
    if (c.expert_row_bias && ((!L->no_gate && !w->gate_proj.row_bias) || !w->up_proj.row_bias || !w->down_proj.row_bias))
        return fail(L, FFAI_ERR_INVALID_ARG, "expert_row_bias set but a row_bias pointer is null");
    if (!c.expert_row_bias) L->w.gate_proj.row_bias = L->w.up_proj.row_bias = L->w.down_proj.row_bias = nullptr;
    if (c.shared_intermediate > 0) {
        const int Is = c.shared_intermediate;
        if (!L->no_gate && (rc = upload_qproj(L, w->shared_gate_proj, 1, Is, c.hidden, c.shared_bits, c.shared_group_size, loc, &L->w.shared_gate_proj, "shared_gate_proj"))) return rc;
        if ((rc = upload_qproj(L, w->shared_up_proj, 1, Is, c.hidden, c.shared_bits, c.shared_group_size, loc, &L->w.shared_up_proj, "shared_up_proj"))) return rc;
        if ((rc = upload_qproj(L, w->shared_down_proj, 1, c.hidden, Is, c.shared_bits, c.shared_group_size, loc, &L->w.shared_down_proj, "shared_down_proj"))) return rc;
        L->w.shared_gate_proj.row_bias = L->w.shared_up_proj.row_bias = L->w.shared_down_proj.row_bias = nullptr;
        if (c.shared_gate_kind != FFAI_LINEAR_NONE)
            if ((rc = upload_linear(L, w->shared_gate, c.shared_gate_kind, 1, c.hidden, c.shared_gate_bits, c.shared_gate_group_size, loc, &L->w.shared_gate, "shared_gate"))) return rc;
    }
    // tensor maps for the tcgen05 path
    L->tc_ok = false;
    if (L->tile_offsets) {
        using namespace g100;
        uint64_t Mcap = L->mx_rows, Tcap = (uint64_t)c.max_tokens;
        if (Mcap < 128) Mcap = 128;
        if (Tcap < 128) Tcap = 128;
        bool ok = true;
        if (c.expert_bits == 4) {
            ok = ok && make_weight_map(&L->tm_gate, L->w.gate_proj.weight, (uint64_t)El * c.intermediate, c.hidden / 8);
            ok = ok && make_weight_map(&L->tm_up, L->w.up_proj.weight, (uint64_t)El * c.intermediate, c.hidden / 8);
            ok = ok && make_weight_map(&L->tm_down, L->w.down_proj.weight, (uint64_t)El * c.hidden, c.intermediate / 8);
            ok = ok && make_act_map(&L->tm_xg, L->xg, Mcap, c.hidden, BM);
            ok = ok && make_act_map(&L->tm_inner, L->inner_bf, Mcap, c.intermediate, BM);
        }
        if (L->cache_planned) {
            const ffai_qproj* q[3] = {&L->w.gate_proj, &L->w.up_proj, &L->w.down_proj};
            const int n_out[3] = {c.intermediate, c.intermediate, c.hidden};
            const int kk[3] = {c.hidden, c.hidden, c.intermediate};
            for (int i = 0; i < 3; ++i) {
                const int blocks = cache_blocks(n_out[i], i < 2);
                void* buf = nullptr;
                CUDA_TRY(L, cudaMalloc(&buf, cache_tiles_bytes((size_t)El, blocks, kk[i])));
                L->owned_weights.push_back(buf);
                L->exp_wbf[i] = static_cast<uint16_t*>(buf);
                if ((rc = launch_expand_to_bf16(*q[i], L->exp_wbf[i], (size_t)El, n_out[i], blocks, kk[i], c.expert_bits, c.expert_group_size)))
                    return fail(L, rc, "expanding the experts to bf16 failed");
            }
            CUDA_TRY(L, cudaDeviceSynchronize());
            if (c.expert_bits != 4) {
                ok = ok && make_act_map(&L->tm_xg, L->xg, Mcap, c.hidden, BM);
                ok = ok && make_act_map(&L->tm_inner, L->inner_bf, Mcap, c.intermediate, BM);
            }
        }
        if (L->sh_x) {
            const int Is = c.shared_intermediate;
            if (c.shared_bits == 4) {
                ok = ok && make_weight_map(&L->tm_sh_gate, L->w.shared_gate_proj.weight, Is, c.hidden / 8);
                ok = ok && make_weight_map(&L->tm_sh_up, L->w.shared_up_proj.weight, Is, c.hidden / 8);
                ok = ok && make_weight_map(&L->tm_sh_down, L->w.shared_down_proj.weight, c.hidden, Is / 8);
            } else {
                // other bit widths: expand the one shared expert to bf16 once (2 bytes per weight) and let the
                // tensor-core kernel read it without a dequant stage
                const ffai_qproj* q[3] = {&L->w.shared_gate_proj, &L->w.shared_up_proj, &L->w.shared_down_proj};
                const int n_out[3] = {Is, Is, c.hidden};
                const int kk[3] = {c.hidden, c.hidden, Is};
                for (int i = 0; i < 3; ++i) {
                    const int blocks = cache_blocks(n_out[i], i < 2);
                    void* buf = nullptr;
                    CUDA_TRY(L, cudaMalloc(&buf, cache_tiles_bytes(1, blocks, kk[i])));
                    L->owned_weights.push_back(buf);
                    L->sh_wbf[i] = static_cast<uint16_t*>(buf);
                    if ((rc = launch_expand_to_bf16(*q[i], L->sh_wbf[i], 1, n_out[i], blocks, kk[i], c.shared_bits, c.shared_group_size)))
                        return fail(L, rc, "expanding the shared expert to bf16 failed");
                }
                CUDA_TRY(L, cudaDeviceSynchronize());
            }
            ok = ok && make_act_map(&L->tm_sh_x, L->sh_x, Tcap, c.hidden, BM);
            ok = ok && make_act_map(&L->tm_sh_inner, L->sh_inner_bf, Tcap, Is, BM);
        }
        if (!ok) return fail(L, FFAI_ERR_CUDA, "cuTensorMapEncodeTiled failed");
        L->tc_ok = true;
    }
    // scale/bias words repacked for the streaming decode kernels (owned copies, freed with the weights)
    L->sb_gate = L->sb_up = L->sb_down = nullptr;
    if (L->mma_ok) {
        auto repack = [&](const ffai_qproj& q, int N, int K, uint32_t** out) -> int {
            const int run = c.expert_group_size == 32 ? 32 : 64;
            const size_t total = (size_t)El * N * (K / run);
            void* p = nullptr;
            CUDA_TRY(L, cudaMalloc(&p, total * 4));
            L->owned_weights.push_back(p);
            *out = static_cast<uint32_t*>(p);
            dmma::repack_scale_bias_kernel<<<(unsigned)((total + 255) / 256), 256>>>(q.scales, q.biases, *out, El, N, K, c.expert_group_size, run);
            CUDA_TRY(L, cudaGetLastError());
            return FFAI_OK;
        };
        if ((rc = repack(L->w.gate_proj, c.intermediate, c.hidden, &L->sb_gate))) return rc;
        if ((rc = repack(L->w.up_proj, c.intermediate, c.hidden, &L->sb_up))) return rc;
        if ((rc = repack(L->w.down_proj, c.hidden, c.intermediate, &L->sb_down))) return rc;
        CUDA_TRY(L, cudaDeviceSynchronize());
    }
    // re-tiled streams for the bulk-copy decode kernels (group 64 / 128; same bytes as the packed experts + scale words)
    L->st_gate_up = L->st_down = nullptr;
    if (L->mma_ok && c.expert_group_size != 32) {
        const size_t H = c.hidden, I = c.intermediate;
        const size_t gu_cells = (size_t)El * (I / 16) * (H / 64), dn_cells = (size_t)El * (H / 16) * (I / 64);
        if (gu_cells < (1u << 31) && dn_cells < (1u << 31)) {
            void* a = nullptr;
            void* b = nullptr;
            CUDA_TRY(L, cudaMalloc(&a, gu_cells * 2 * dstr::CELL));
            L->owned_weights.push_back(a);
            CUDA_TRY(L, cudaMalloc(&b, dn_cells * dstr::CELL));
            L->owned_weights.push_back(b);
            dstr::retile_stream_kernel<<<(unsigned)gu_cells, 96>>>(L->w.gate_proj.weight, L->w.gate_proj.scales, L->w.gate_proj.biases,
                                                                   L->w.up_proj.weight, L->w.up_proj.scales, L->w.up_proj.biases,
                                                                   static_cast<uint8_t*>(a), (int)I, (int)H, c.expert_group_size);
            dstr::retile_stream_kernel<<<(unsigned)dn_cells, 64>>>(L->w.down_proj.weight, L->w.down_proj.scales, L->w.down_proj.biases,
                                                                   nullptr, nullptr, nullptr, static_cast<uint8_t*>(b), (int)H, (int)I,
                                                                   c.expert_group_size);
            CUDA_TRY(L, cudaGetLastError());
            CUDA_TRY(L, cudaDeviceSynchronize());
            L->st_gate_up = static_cast<uint8_t*>(a);
            L->st_down = static_cast<uint8_t*>(b);
        }
    }
    L->weights_set = true;
    return FFAI_OK;
}

extern "C" FFAI_API int ffai_moe_destroy(ffai_moe_layer* L) {
    if (!L) return FFAI_OK;
    if (L->device >= 0) cudaSetDevice(L->device);
    for (void* p : L->ep_opened) cudaIpcCloseMemHandle(p);
    free_list(L->owned_weights);
    free_list(L->owned_ws);
    for (void* p : L->owned_pinned) cudaFreeHost(p);
    if (L->ev_made)
        for (auto& a : L->ev) for (auto& b : a) for (auto& e : b) cudaEventDestroy(e);
    if (L->own_stream) cudaStreamDestroy(L->own_stream);
    if (L->h2d_stream) {
        cudaStreamDestroy(L->h2d_stream);
        cudaStreamDestroy(L->d2h_stream);
        for (auto& e : L->ev_in) cudaEventDestroy(e);
        for (auto& e : L->ev_out) cudaEventDestroy(e);
    }
    if (L->aux_stream) { cudaStreamDestroy(L->aux_stream); cudaEventDestroy(L->ev_fork); cudaEventDestroy(L->ev_join); }
    delete L;
    return FFAI_OK;
}

extern "C" FFAI_API const char* ffai_moe_last_error(const ffai_moe_layer* L) { return L ? L->err.c_str() : ""; }

extern "C" FFAI_API int ffai_moe_set_nccl_comm(ffai_moe_layer* L, void* comm) {
    if (!L) return FFAI_ERR_INVALID_ARG;
    L->nccl_comm = comm;
    return FFAI_OK;
}

extern "C" FFAI_API int ffai_moe_ep_export(ffai_moe_layer* L, uint8_t out_blob[FFAI_EP_EXPORT_BYTES]) {
    if (!L || !out_blob) return FFAI_ERR_INVALID_ARG;
    if (L->cfg.ep_world <= 1 || !L->ep_win) return fail(L, FFAI_ERR_INVALID_ARG, "layer was not created with ep_world > 1");
    static_assert(3 * sizeof(cudaIpcMemHandle_t) == FFAI_EP_EXPORT_BYTES, "export blob size");
    CUDA_TRY(L, cudaSetDevice(L->device));
    cudaIpcMemHandle_t h[3];
    CUDA_TRY(L, cudaIpcGetMemHandle(&h[0], L->ep_win));
    CUDA_TRY(L, cudaIpcGetMemHandle(&h[1], L->xg));
    CUDA_TRY(L, cudaIpcGetMemHandle(&h[2], L->ep_y_bf));
    memcpy(out_blob, h, sizeof(h));
    return FFAI_OK;
}

extern "C" FFAI_API int ffai_moe_ep_import(ffai_moe_layer* L, const uint8_t* blobs) {
    if (!L || !blobs) return FFAI_ERR_INVALID_ARG;
    const int W = L->cfg.ep_world, me = L->cfg.ep_rank;
    if (W <= 1 || !L->ep_win) return fail(L, FFAI_ERR_INVALID_ARG, "layer was not created with ep_world > 1");
    if (L->ep_peer_on) return fail(L, FFAI_ERR_INVALID_ARG, "peer buffers were already imported");
    CUDA_TRY(L, cudaSetDevice(L->device));
    for (int r = 0; r < W; ++r) {
        if (r == me) {
            L->ep_peer_win.p[r] = L->ep_win; L->ep_peer_rows.p[r] = L->xg; L->ep_peer_y.p[r] = L->ep_y_bf;
            continue;
        }
        cudaIpcMemHandle_t h[3];
        memcpy(h, blobs + (size_t)r * FFAI_EP_EXPORT_BYTES, sizeof(h));
        void* ptr[3] = {nullptr, nullptr, nullptr};
        for (int i = 0; i < 3; ++i) {
            CUDA_TRY(L, cudaIpcOpenMemHandle(&ptr[i], h[i], cudaIpcMemLazyEnablePeerAccess));
            L->ep_opened.push_back(ptr[i]);
        }
        L->ep_peer_win.p[r] = ptr[0]; L->ep_peer_rows.p[r] = ptr[1]; L->ep_peer_y.p[r] = ptr[2];
    }
    L->ep_peer_on = true;   // the step counter keeps running: the flags a peer left in this window are all behind it
    return FFAI_OK;
}

extern "C" FFAI_API int ffai_ep_peer_layout(const uint32_t* counts_matrix, int32_t world, int32_t n_experts, int32_t rank,
                                            uint32_t* local_offsets, uint32_t* send_base) {
    if (!counts_matrix || !local_offsets || !send_base || world < 1 || n_experts < world || n_experts % world || rank < 0 || rank >= world)
        return FFAI_ERR_INVALID_ARG;
    const int el = n_experts / world;
    for (int e = 0; e < n_experts; ++e) send_base[e] = ep::peer_send_base(counts_matrix, n_experts, el, rank, world, e);
    for (int i = 0; i <= el; ++i) local_offsets[i] = ep::peer_local_offset(counts_matrix, n_experts, el, rank, world, i);
    return FFAI_OK;
}

extern "C" FFAI_API int ffai_moe_ep_release(ffai_moe_layer* L) {
    if (!L) return FFAI_ERR_INVALID_ARG;
    CUDA_TRY(L, cudaSetDevice(L->device));
    CUDA_TRY(L, cudaDeviceSynchronize());
    for (void* p : L->ep_opened) cudaIpcCloseMemHandle(p);
    L->ep_opened.clear();
    L->ep_peer_on = false;
    return FFAI_OK;
}

extern "C" FFAI_API int ffai_moe_ep_skip_step(ffai_moe_layer* L) {
    if (!L) return FFAI_ERR_INVALID_ARG;
    if (!L->ep_peer_on) return fail(L, FFAI_ERR_INVALID_ARG, "no peer buffers are imported");
    L->ep_epoch += 1;
    return FFAI_OK;
}

extern "C" FFAI_API int ffai_ep_get_unique_id(uint8_t out_id[128]) {
    if (!out_id) return FFAI_ERR_INVALID_ARG;
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId size");
    if (!ep::nccl().ok) return FFAI_ERR_NCCL;
    ncclUniqueId id;
    if (ep::nccl().GetUniqueId(&id) != ncclSuccess) return FFAI_ERR_NCCL;
    memcpy(out_id, &id, 128);
    return FFAI_OK;
}

extern "C" FFAI_API int ffai_ep_comm_create(const uint8_t id_bytes[128], int32_t rank, int32_t world, void** out_comm) {
    if (!id_bytes || !out_comm || world < 1 || rank < 0 || rank >= world) return FFAI_ERR_INVALID_ARG;
    if (!ep::nccl().ok) return FFAI_ERR_NCCL;
    ncclUniqueId id;
    memcpy(&id, id_bytes, 128);
    ncclComm_t comm = nullptr;
    if (ep::nccl().CommInitRank(&comm, world, id, rank) != ncclSuccess) return FFAI_ERR_NCCL;
    *out_comm = comm;
    return FFAI_OK;
}

extern "C" FFAI_API int ffai_ep_comm_destroy(void* comm) {
    if (!comm) return FFAI_OK;
    if (!ep::nccl().ok) return FFAI_ERR_NCCL;
    return ep::nccl().CommDestroy(static_cast<ncclComm_t>(comm)) == ncclSuccess ? FFAI_OK : FFAI_ERR_NCCL;
}

extern "C" FFAI_API uint32_t ffai_ep_plan_exchange(const uint32_t* recv_counts, int32_t world, int32_t e_local,
                                                   uint32_t* rank_offsets, uint32_t* local_offsets,
                                                   uint32_t* seg_src, uint32_t* seg_dst) {
    if (!recv_counts || !rank_offsets || !local_offsets || !seg_src || !seg_dst || world < 1 || e_local < 1) return 0;
    return ep::plan_exchange(recv_counts, world, e_local, rank_offsets, local_offsets, seg_src, seg_dst);
}

extern "C" FFAI_API int ffai_moe_set_option(ffai_moe_layer* L, const char* name, int32_t value) {
    if (!L || !name) return FFAI_ERR_INVALID_ARG;
    if (!strcmp(name, "path")) {
        if (value < 0 || value > 3) return fail(L, FFAI_ERR_INVALID_ARG, "option path must be 0..3");
        L->opt_path = value;
        return FFAI_OK;
    }
    if (!strcmp(name, "tc_min_rows")) {
        if (value < 0) return fail(L, FFAI_ERR_INVALID_ARG, "option tc_min_rows must be >= 0");
        L->opt_tc_min_rows = value;
        return FFAI_OK;
    }
    if (!strcmp(name, "host_chunks")) {
        if (value < 0 || value > 4) return fail(L, FFAI_ERR_INVALID_ARG, "host_chunks must be 0 (automatic), 1 (never split) or 2..4 chunks");
        L->opt_host_chunks = value;
        return FFAI_OK;
    }
    if (!strcmp(name, "tc_weights")) {
        if (value < 0 || value > 2) return fail(L, FFAI_ERR_INVALID_ARG, "tc_weights must be 0 (automatic), 1 (packed) or 2 (cache when present)");
        L->opt_tc_weights = value;
        return FFAI_OK;
    }
    if (!strcmp(name, "ksplit")) {
        if (value != 0 && value != 1 && value != 2 && value != 4) return fail(L, FFAI_ERR_INVALID_ARG, "option ksplit must be 0, 1, 2 or 4");
        L->opt_ksplit = value;
        return FFAI_OK;
    }
    if (!strcmp(name, "ep_wait_ms")) {
        if (value < 1 || value > 60000) return fail(L, FFAI_ERR_INVALID_ARG, "option ep_wait_ms must be in 1..60000");
        L->ep_wait_ns = (uint64_t)value * 1000000ull;
        return FFAI_OK;
    }
    if (!strcmp(name, "decode")) {
        if (value < 0 || value > 2) return fail(L, FFAI_ERR_INVALID_ARG, "option decode must be 0 (automatic), 1 (cp.async rings) or 2 (bulk-copy streams)");
        L->opt_decode = value;
        return FFAI_OK;
    }
    if (!strcmp(name, "overlap")) {
        L->opt_overlap = value != 0;
        return FFAI_OK;
    }
    if (!strcmp(name, "pdl")) {
        L->opt_pdl = value != 0;
        return FFAI_OK;
    }
    if (!strcmp(name, "decode_team")) {
        if (value != 0 && value != 1 && value != 4 && value != 16) return fail(L, FFAI_ERR_INVALID_ARG, "option decode_team must be 0, 1, 4 or 16");
        L->opt_decode_team = value;
        return FFAI_OK;
    }
    if (!strcmp(name, "nt2_cost")) {
        if (value < 8 || value > 32) return fail(L, FFAI_ERR_INVALID_ARG, "option nt2_cost must be in 8..32");
        L->opt_nt2_cost = value;
        return FFAI_OK;
    }
    if (!strcmp(name, "timeline")) {
        if (value && !L->timeline) {
            int rc = ws_alloc(L, &L->timeline, (size_t)g100::TL_ROLES * g100::TL_SLOTS * g100::TL_EVENTS);
            if (rc) return rc;
        }
        if (!value) L->timeline = nullptr;
        return FFAI_OK;
    }
    return fail(L, FFAI_ERR_INVALID_ARG, "unknown option %s", name);
}

extern "C" FFAI_API int ffai_moe_read_timeline(ffai_moe_layer* L, int64_t* out, int32_t capacity) {
    if (!L || !out) return FFAI_ERR_INVALID_ARG;
    const int n = g100::TL_ROLES * g100::TL_SLOTS * g100::TL_EVENTS;
    if (!L->timeline || capacity < n) return fail(L, FFAI_ERR_INVALID_ARG, "timeline not enabled or capacity < %d", n);
    CUDA_TRY(L, cudaSetDevice(L->device));
    CUDA_TRY(L, cudaDeviceSynchronize());
    CUDA_TRY(L, cudaMemcpy(out, L->timeline, sizeof(long long) * n, cudaMemcpyDeviceToHost));
    return FFAI_OK;
}

extern "C" FFAI_API int ffai_moe_check_device_status(ffai_moe_layer* L) {
    if (!L) return FFAI_ERR_INVALID_ARG;
    if (!L->error_word) return FFAI_OK;
    CUDA_TRY(L, cudaSetDevice(L->device));
    CUDA_TRY(L, cudaDeviceSynchronize());
    uint32_t word = 0;
    CUDA_TRY(L, cudaMemcpy(&word, L->error_word, 4, cudaMemcpyDeviceToHost));
    if (word) {
        CUDA_TRY(L, cudaMemset(L->error_word, 0, 4));
        return fail(L, FFAI_ERR_DEVICE_CHECK, "a kernel gave up a bounded wait (code %u)", word);
    }
    return FFAI_OK;
}

extern "C" FFAI_API int ffai_moe_set_stage_timing(ffai_moe_layer* L, int enabled) {
    if (!L) return FFAI_ERR_INVALID_ARG;
    if (enabled && !L->ev_made) {
        for (auto& a : L->ev) for (auto& b : a) for (auto& e : b) CUDA_TRY(L, cudaEventCreate(&e));
        L->ev_made = true;
    }
    L->timing = enabled != 0;
    return FFAI_OK;
}

extern "C" FFAI_API int ffai_moe_get_stage_ms(ffai_moe_layer* L, float out_ms[FFAI_N_STAGES]) {
    if (!L || !out_ms) return FFAI_ERR_INVALID_ARG;
    for (int i = 0; i < FFAI_N_STAGES; ++i) out_ms[i] = 0.0f;
    if (!L->ev_made) return FFAI_OK;
    for (int i = 0; i < FFAI_N_STAGES; ++i)
        for (int s = 0; s < L->ev_segments[i]; ++s) {
            float ms = 0.0f;
            CUDA_TRY(L, cudaEventSynchronize(L->ev[i][s][1]));
            CUDA_TRY(L, cudaEventElapsedTime(&ms, L->ev[i][s][0], L->ev[i][s][1]));
            out_ms[i] += ms;
        }
    return FFAI_OK;
}

extern "C" FFAI_API int ffai_moe_last_launch_count(const ffai_moe_layer* L) { return L ? L->launches : 0; }

// ───────────────────────────── forward ─────────────────────────────

namespace {

RouterParams router_params(const ffai_moe_layer* L) {
    const ffai_moe_config& c = L->cfg;
    RouterParams p{};
    p.weight = L->w.router.weight;
    p.scales = L->w.router.scales;
    p.biases = L->w.router.biases;
    p.bias = L->w.router.bias;
    p.expert_bias = c.router_expert_bias ? L->w.router_expert_bias : nullptr;
    p.kind = c.router_kind;
    if (L->router_f32) {   // quantized router: its fp32 expansion through the dense kernels (same bits, no per-use unpacking)
        p.weight = L->router_f32;
        p.kind = FFAI_LINEAR_F32;
    }
    p.bits = c.router_bits;
    p.group_size = c.router_group_size;
    p.hidden = c.hidden;
    p.n_experts = c.n_experts;
    p.top_k = c.top_k;
    p.gating_mode = c.gating_mode;
    p.norm_topk_prob = c.norm_topk_prob;
    p.logits_bf16 = c.router_logits_bf16;
    p.logit_scale = c.router_logit_scale != 0.0f ? c.router_logit_scale : 1.0f;
    p.per_expert_scale = L->w.router_per_expert_scale;
    p.routed_scaling = c.routed_scaling_factor != 0.0f ? c.routed_scaling_factor : 1.0f;
    return p;
}

GemvParams gemv_params(const ffai_qproj& a, const ffai_qproj* b, int N, int K, int gs, int n_experts) {
    GemvParams p{};
    p.weight = a.weight; p.scales = a.scales; p.biases = a.biases; p.row_bias = a.row_bias;
    if (b) { p.weight2 = b->weight; p.scales2 = b->scales; p.biases2 = b->biases; p.row_bias2 = b->row_bias; }
    p.N = N; p.K = K; p.group_size = gs; p.n_experts = n_experts;
    p.in_row_div = 1;
    return p;
}

int copy_debug(ffai_moe_layer* L, const ffai_moe_debug* d, int T, cudaStream_t st, cudaMemcpyKind kind) {
    if (!d) return FFAI_OK;
    const ffai_moe_config& c = L->cfg;
    const size_t M = (size_t)T * c.top_k, E = c.n_experts;
    if (d->indices) CUDA_TRY(L, cudaMemcpyAsync(d->indices, L->indices, M * 4, kind, st));
    if (d->weights) CUDA_TRY(L, cudaMemcpyAsync(d->weights, L->rweights, M * 4, kind, st));
    if (d->logits) CUDA_TRY(L, cudaMemcpyAsync(d->logits, L->logits, (size_t)T * E * 4, kind, st));
    if (d->counts) CUDA_TRY(L, cudaMemcpyAsync(d->counts, L->counts, E * 4, kind, st));
    if (d->offsets) CUDA_TRY(L, cudaMemcpyAsync(d->offsets, L->offsets, (E + 1) * 4, kind, st));
    if (d->perm) CUDA_TRY(L, cudaMemcpyAsync(d->perm, L->perm, M * 4, kind, st));
    if (d->inv_perm) CUDA_TRY(L, cudaMemcpyAsync(d->inv_perm, L->inv_perm, M * 4, kind, st));
    return FFAI_OK;
}


// ───────────────────────────── expert parallelism ─────────────────────────────

#define NCCL_TRY(L, expr)                                                                        \
    do {                                                                                         \
        ncclResult_t _r = (expr);                                                                \
        if (_r != ncclSuccess)                                                                   \
            return fail((L), FFAI_ERR_NCCL, "%s failed: %s", #expr,                              \
                        ep::nccl().GetErrorString ? ep::nccl().GetErrorString(_r) : "nccl error"); \
    } while (0)

// All-to-all of byte ranges: rank d gets send[off_s[d], +len_s[d]); rank s's range lands at recv[off_r[s], +len_r[s]).
int ep_all_to_all(ffai_moe_layer* L, const uint8_t* send, const size_t* off_s, const size_t* len_s, uint8_t* recv,
                  const size_t* off_r, const size_t* len_r, cudaStream_t st) {
    ep::NcclApi& n = ep::nccl();
    ncclComm_t comm = static_cast<ncclComm_t>(L->nccl_comm);
    const int W = L->cfg.ep_world, me = L->cfg.ep_rank;
    NCCL_TRY(L, n.GroupStart());
    for (int d = 0; d < W; ++d) {
        if (d == me) continue;
        if (len_s[d]) NCCL_TRY(L, n.Send(send + off_s[d], len_s[d], ncclUint8, d, comm, st));
        if (len_r[d]) NCCL_TRY(L, n.Recv(recv + off_r[d], len_r[d], ncclUint8, d, comm, st));
    }
    NCCL_TRY(L, n.GroupEnd());
    if (len_s[me]) CUDA_TRY(L, cudaMemcpyAsync(recv + off_r[me], send + off_s[me], len_s[me], cudaMemcpyDeviceToDevice, st));
    return FFAI_OK;
}

// The two grouped GEMMs of the tensor-core path, from the bf16 weight cache when the layer keeps one,
// else from the packed 4-bit weights with the in-kernel dequant stage.
int tc_group_rows(const ffai_moe_layer*) { return g100::BM; }
bool tc_reads_cache(const ffai_moe_layer* L) { return L->exp_wbf[0] && (L->opt_tc_weights != 1 || L->cfg.expert_bits != 4); }
bool tc_possible(const ffai_moe_layer* L) { return L->tc_ok && (L->cfg.expert_bits == 4 || L->exp_wbf[0]); }
// Gate/up with few rows per expert goes over the packed weights even when the layer keeps a cache: an expert
// then has one or two token tiles, the dequant stage runs once or twice per weight tile, and the 4x smaller
// weight read wins (cfg3: 160 us packed against 170 us cached; at 256 rows per expert the cache wins, 300
// against 339 us).  Down keeps the cache: its reduction axis is short and the packed pipeline's start-up per
// item weighs more.
int tc_gate_up(ffai_moe_layer* L, const g100::Params& p, double rows_per_expert, cudaStream_t st) {
    const bool packed_pays = L->cfg.expert_bits == 4 && L->opt_tc_weights == 0 && rows_per_expert <= 160.0;
    if (tc_reads_cache(L) && !packed_pays) {
        g100::Params pc = p;
        pc.wcache = L->exp_wbf[0]; pc.wcache2 = L->exp_wbf[1]; pc.cache_blocks = cache_blocks(p.n_out, true);
        return g100::launch_grouped_gemm<true, uint16_t, true>(L->tm_xg, L->tm_xg, L->tm_xg, pc, L->n_sms, st);
    }
    return g100::launch_grouped_gemm<true, uint16_t>(L->tm_gate, L->tm_up, L->tm_xg, p, L->n_sms, st);
}
template <typename TOut>
int tc_down(ffai_moe_layer* L, const g100::Params& p, cudaStream_t st) {
    if (tc_reads_cache(L)) {
        g100::Params pc = p;
        pc.wcache = L->exp_wbf[2]; pc.wcache2 = nullptr; pc.cache_blocks = cache_blocks(p.n_out, false);
        return g100::launch_grouped_gemm<false, TOut, true>(L->tm_inner, L->tm_inner, L->tm_inner, pc, L->n_sms, st);
    }
    return g100::launch_grouped_gemm<false, TOut>(L->tm_down, L->tm_down, L->tm_inner, p, L->n_sms, st);
}

// Whether rows travel 8-run permuted (the layout both 4-bit kernels read).  Every rank must agree, so
// the rule looks only at the layer's configuration and options.
bool ep_rows_perm8(const ffai_moe_layer* L) { return (L->mma_ok || tc_possible(L)) && L->opt_path != 1; }

// Routed experts over rows that are already expert-contiguous in L->xg (bf16; 8-run permuted when the layer's
// experts are 4-bit with group 64/128, plain otherwise).  Output: fp32 rows in L->y.
int run_experts_on_rows(ffai_moe_layer* L, int n_rows, int n_exp, const uint32_t* offsets_dev, cudaStream_t st) {
    const ffai_moe_config& c = L->cfg;
    const int H = c.hidden, I = c.intermediate;
    if (n_rows <= 0) return FFAI_OK;
    const double rpe = (double)n_rows / n_exp;
    const bool can_tc = tc_possible(L);
    bool use_mma = false, use_tc = false;
    if (ep_rows_perm8(L)) {   // the rows arrived 8-run permuted: the streaming or the tensor-core kernels must take them
        if (L->opt_path == 3) use_tc = !L->mma_ok;
        else if (L->opt_path == 2) use_tc = can_tc;
        else use_tc = can_tc && (rpe > 16.0 || !L->mma_ok);
        if (!L->mma_ok) use_tc = true;
        if (!can_tc) use_tc = false;
        use_mma = !use_tc;
    }
    if (use_mma) {
        using namespace dmma;
        const int xp_h = (H / 32 + 3) & ~3, xp_i = (I / 32 + 3) & ~3;
        if (L->ep_rows_dev)
            ep::sum64_rows_counted_kernel<<<(unsigned)((L->mx_rows + 7) / 8), 256, 0, st>>>(L->xg, L->xsum, L->ep_rows_dev, H, xp_h);
        else
            sum64_rows_kernel<<<(n_rows + 7) / 8, 256, 0, st>>>(L->xg, L->xsum, n_rows, H, xp_h);
        Params p{};
        p.group_size = c.expert_group_size;
        p.offsets = offsets_dev;
        p.activation = c.activation; p.limit = c.swiglu_limit; p.alpha = c.swiglu_alpha;
        const int nt = rpe > 4.0 ? 2 : 1;
        const int ksplit = L->opt_ksplit > 0 ? L->opt_ksplit : (n_rows <= 4 ? 2 : 1);
        stage_begin(L, ST_GATE_UP, st);
        p.w1 = L->w.gate_proj.weight; p.s1 = L->w.gate_proj.scales; p.b1 = L->w.gate_proj.biases; p.rb1 = L->w.gate_proj.row_bias;
        p.w2 = L->w.up_proj.weight; p.s2 = L->w.up_proj.scales; p.b2 = L->w.up_proj.biases; p.rb2 = L->w.up_proj.row_bias;
        p.sb1 = L->sb_gate; p.sb2 = L->sb_up;
        p.N = I; p.K = H; p.x = L->xg; p.xsum = L->xsum; p.xsum_pitch = xp_h; p.out = L->inner_bf;
        p.out_parts = L->inner_parts;
        launch_mma_decode<true>(p, n_exp, nt, ksplit, st);
        stage_end(L, ST_GATE_UP, st);
        stage_begin(L, ST_DOWN, st);
        p.w1 = L->w.down_proj.weight; p.s1 = L->w.down_proj.scales; p.b1 = L->w.down_proj.biases; p.rb1 = L->w.down_proj.row_bias;
        p.w2 = nullptr; p.s2 = nullptr; p.b2 = nullptr; p.rb2 = nullptr;
        p.sb1 = L->sb_down; p.sb2 = nullptr;
        p.N = H; p.K = I; p.x = L->inner_bf; p.xsum = nullptr; p.xsum_parts = L->inner_parts; p.xsum_pitch = xp_i; p.out = L->y;
        if (L->ep_peer_on) { p.out = L->ep_y_bf; p.out_bf16 = 1; }
        p.out_parts = nullptr;
        // group 32: 32 rows per warp through the two-projection kernel (measured 9 % faster there; no gain at group 64)
        p.pair = c.expert_group_size == 32;
        if (p.pair) launch_mma_decode<true>(p, n_exp, nt, ksplit, st);
        else launch_mma_decode<false>(p, n_exp, nt, ksplit, st);
        stage_end(L, ST_DOWN, st);
        L->launches += 3;
    } else if (use_tc) {
        using namespace g100;
        tile_schedule_kernel<<<1, 32, 0, st>>>(offsets_dev, n_exp, tc_group_rows(L), L->tile_offsets);
        Params p{};
        p.n_experts = n_exp; p.group_size = c.expert_group_size;
        p.offsets = offsets_dev; p.tile_offsets = L->tile_offsets;
        p.activation = c.activation; p.limit = c.swiglu_limit; p.alpha = c.swiglu_alpha;
        p.error_word = L->error_word;
        stage_begin(L, ST_GATE_UP, st);
        p.scales = L->w.gate_proj.scales; p.biases = L->w.gate_proj.biases; p.row_bias = L->w.gate_proj.row_bias;
        p.scales2 = L->w.up_proj.scales; p.biases2 = L->w.up_proj.biases; p.row_bias2 = L->w.up_proj.row_bias;
        if (c.expert_group_size != 32) { p.sb = L->sb_gate; p.sb2 = L->sb_up; }
        p.n_out = I; p.K = H; p.m_tiles = (I + BN / 2 - 1) / (BN / 2);
        p.out = L->inner_bf; p.out_ld = I; p.out_permute8 = 1;
        if (tc_gate_up(L, p, rpe, st))
            return fail(L, FFAI_ERR_CUDA, "gate/up grouped GEMM launch failed");
        stage_end(L, ST_GATE_UP, st);
        stage_begin(L, ST_DOWN, st);
        p.scales = L->w.down_proj.scales; p.biases = L->w.down_proj.biases; p.row_bias = L->w.down_proj.row_bias;
        p.scales2 = nullptr; p.biases2 = nullptr; p.row_bias2 = nullptr;
        p.sb = c.expert_group_size != 32 ? L->sb_down : nullptr; p.sb2 = nullptr;
        p.n_out = H; p.K = I; p.m_tiles = (H + BN - 1) / BN;
        p.out = L->y; p.out_ld = H; p.out_permute8 = 0;
        if (L->ep_peer_on) p.out = L->ep_y_bf;
        if (L->ep_peer_on ? tc_down<uint16_t>(L, p, st) : tc_down<float>(L, p, st))
            return fail(L, FFAI_ERR_CUDA, "down grouped GEMM launch failed");
        stage_end(L, ST_DOWN, st);
        L->launches += 3;
    } else {
        int rc;
        GemvParams p = L->no_gate ? gemv_params(L->w.up_proj, nullptr, I, H, c.expert_group_size, n_exp)
                                  : gemv_params(L->w.gate_proj, &L->w.up_proj, I, H, c.expert_group_size, n_exp);
        p.offsets = offsets_dev;
        p.n_rows = n_rows;
        p.activation = c.activation; p.limit = c.swiglu_limit; p.alpha = c.swiglu_alpha;
        p.post_relu2 = L->no_gate;
        stage_begin(L, ST_GATE_UP, st);
        if ((rc = L->no_gate ? launch_grouped_gemv<uint16_t, float, false>(p, c.expert_bits, L->xg, L->inner, n_exp, st)
                             : launch_grouped_gemv<uint16_t, float, true>(p, c.expert_bits, L->xg, L->inner, n_exp, st))) return fail(L, rc, "gate/up launch failed");
        stage_end(L, ST_GATE_UP, st);
        stage_begin(L, ST_DOWN, st);
        GemvParams d = gemv_params(L->w.down_proj, nullptr, H, I, c.expert_group_size, n_exp);
        d.offsets = offsets_dev;
        d.n_rows = n_rows;
        if ((rc = launch_grouped_gemv<float, float, false>(d, c.expert_bits, L->inner, L->y, n_exp, st))) return fail(L, rc, "down launch failed");
        stage_end(L, ST_DOWN, st);
        L->launches += 2;
    }
    return cudaGetLastError() == cudaSuccess ? FFAI_OK : fail(L, FFAI_ERR_CUDA, "expert kernels launch failed");
}

// The routed experts under expert parallelism: exchange counts, dispatch rows, compute, return rows.
// On return L->ep_home_y holds, in this rank's sorted-row order, the fp32 expert outputs of its own rows.
int forward_experts_ep(ffai_moe_layer* L, const uint16_t* x, int T, cudaStream_t st) {
    const ffai_moe_config& c = L->cfg;
    const int H = c.hidden, E = c.n_experts, K = c.top_k, W = c.ep_world, me = c.ep_rank, El = L->e_local;
    const int M = T * K;
    if (!L->nccl_comm || !ep::nccl().ok) return fail(L, FFAI_ERR_NCCL, "expert parallelism needs ffai_moe_set_nccl_comm first");
    int rc;
    // rows leave sorted by (expert, token, slot); 8-run permuted when the 4-bit kernels will consume them
    stage_begin(L, ST_GATHER, st);
    if (M == 0) { /* nothing leaves this rank */ }
    else if (ep_rows_perm8(L)) g100::gather_rows_perm8_kernel<<<(M + 7) / 8, 256, 0, st>>>(x, L->perm, K, L->ep_send_x, M, H);
    else gather_rows_kernel<<<(M + 7) / 8, 256, 0, st>>>(x, L->perm, K, L->ep_send_x, M, H);
    L->launches += 1;
    stage_end(L, ST_GATHER, st);

    stage_begin(L, ST_EXCHANGE, st);
    // 1. counts: rank d learns how many of my rows go to each of its experts
    std::vector<size_t> so(W), sl(W), ro(W), rl(W);
    for (int d = 0; d < W; ++d) { so[d] = (size_t)d * El * 4; sl[d] = (size_t)El * 4; ro[d] = (size_t)d * El * 4; rl[d] = (size_t)El * 4; }
    if ((rc = ep_all_to_all(L, (const uint8_t*)L->counts, so.data(), sl.data(), (uint8_t*)L->ep_recv_counts, ro.data(), rl.data(), st))) return rc;
    uint32_t* h_rc = L->ep_pin;                 // [W*El]
    uint32_t* h_off = h_rc + (size_t)W * El;     // [E+1]
    uint32_t* h_plan = h_off + (E + 1);          // local_offsets[El+1] | seg_src[W*El] | seg_dst[W*El]
    CUDA_TRY(L, cudaMemcpyAsync(h_rc, L->ep_recv_counts, sizeof(uint32_t) * W * El, cudaMemcpyDeviceToHost, st));
    CUDA_TRY(L, cudaMemcpyAsync(h_off, L->offsets, sizeof(uint32_t) * (E + 1), cudaMemcpyDeviceToHost, st));
    CUDA_TRY(L, cudaStreamSynchronize(st));      // the one host round trip of the exchange: NCCL needs sizes on the host
    // 2. plan
    std::vector<uint32_t> rank_off(W + 1);
    uint32_t* local_off = h_plan;
    uint32_t* seg_src = h_plan + (El + 1);
    uint32_t* seg_dst = seg_src + (size_t)W * El;
    const uint32_t n_recv = ep::plan_exchange(h_rc, W, El, rank_off.data(), local_off, seg_src, seg_dst);
    if (n_recv > L->mx_rows) return fail(L, FFAI_ERR_INVALID_ARG, "expert-parallel receive of %u rows exceeds capacity %zu", n_recv, L->mx_rows);
    CUDA_TRY(L, cudaMemcpyAsync(L->ep_plan_dev, h_plan, sizeof(uint32_t) * ((El + 1) + 2 * (size_t)W * El), cudaMemcpyHostToDevice, st));
    const uint32_t* d_local_off = L->ep_plan_dev;
    const uint32_t* d_seg_src = L->ep_plan_dev + (El + 1);
    const uint32_t* d_seg_dst = d_seg_src + (size_t)W * El;
    // 3. dispatch rows
    const size_t xrow = (size_t)H * 2, yrow = (size_t)H * 4;
    for (int d = 0; d < W; ++d) {
        so[d] = (size_t)h_off[d * El] * xrow;
        sl[d] = (size_t)(h_off[(d + 1) * El] - h_off[d * El]) * xrow;
        ro[d] = (size_t)rank_off[d] * xrow;
        rl[d] = (size_t)(rank_off[d + 1] - rank_off[d]) * xrow;
    }
    if ((rc = ep_all_to_all(L, (const uint8_t*)L->ep_send_x, so.data(), sl.data(), (uint8_t*)L->ep_recv_x, ro.data(), rl.data(), st))) return rc;
    // 4. regroup the per-source segments of each local expert (ascending source rank)
    if (n_recv) {
        ep::copy_segments_kernel<<<dim3(W * El, 8), 256, 0, st>>>((const uint8_t*)L->ep_recv_x, (uint8_t*)L->xg, d_seg_src, d_seg_dst, L->ep_recv_counts, (int)xrow);
        L->launches += 1;
    }
    stage_end(L, ST_EXCHANGE, st);

    if ((rc = run_experts_on_rows(L, (int)n_recv, El, d_local_off, st))) return rc;

    stage_begin(L, ST_EXCHANGE, st);
    if (n_recv) {
        ep::copy_segments_kernel<<<dim3(W * El, 8), 256, 0, st>>>((const uint8_t*)L->y, (uint8_t*)L->ep_ret_y, d_seg_dst, d_seg_src, L->ep_recv_counts, (int)yrow);
        L->launches += 1;
    }
    // 5. results travel back along the same segments
    for (int d = 0; d < W; ++d) {
        const size_t s_off = so[d] / xrow, s_rows = sl[d] / xrow, r_off = ro[d] / xrow, r_rows = rl[d] / xrow;
        so[d] = r_off * yrow; sl[d] = r_rows * yrow;   // what I received from d goes back to d
        ro[d] = s_off * yrow; rl[d] = s_rows * yrow;   // what I sent to d comes back into my sorted order
    }
    if ((rc = ep_all_to_all(L, (const uint8_t*)L->ep_ret_y, so.data(), sl.data(), (uint8_t*)L->ep_home_y, ro.data(), rl.data(), st))) return rc;
    stage_end(L, ST_EXCHANGE, st);
    (void)me;
    return FFAI_OK;
}

// The routed experts under expert parallelism with the exchange over peer memory: no NCCL call and no
// host synchronisation inside the step.  On return the result rows are in their owners' result
// buffers; the combine pulls them (combine_peer_kernel).
int forward_experts_ep_peer(ffai_moe_layer* L, const uint16_t* x, int T, cudaStream_t st) {
    const ffai_moe_config& c = L->cfg;
    const int H = c.hidden, E = c.n_experts, K = c.top_k, W = c.ep_world, me = c.ep_rank, El = L->e_local;
    const int M = T * K;
    if (!ep_rows_perm8(L)) return fail(L, FFAI_ERR_UNSUPPORTED, "the peer-memory exchange needs the 4-bit or cached-bf16 expert kernels");
    const uint32_t epoch = ++L->ep_epoch;
    int rc;
    stage_begin(L, ST_EXCHANGE, st);
    uint32_t* local_off = L->ep_plan_dev;
    ep::ep_publish_and_layout_kernel<<<1, 256, 2 * E * sizeof(uint32_t), st>>>(L->counts, E, El, me, W, L->ep_peer_win, epoch, L->ep_wait_ns,
                                                                                local_off, L->ep_send_base, (uint32_t)L->mx_rows, L->error_word);
    stage_end(L, ST_EXCHANGE, st);
    // the dispatch is the row gather with its stores going to the owners' buffers: timed as the gather stage,
    // so the exchange stage shows what the counts, the layout and the barriers cost by themselves
    stage_begin(L, ST_GATHER, st);
    if (M > 0)
        ep::ep_dispatch_kernel<<<(M + 7) / 8, 256, 0, st>>>(x, L->perm, L->indices, L->offsets, L->ep_send_base, K, El, M, H,
                                                            L->ep_peer_rows, (uint32_t)L->mx_rows, L->error_word);
    stage_end(L, ST_GATHER, st);
    stage_begin(L, ST_EXCHANGE, st);
    ep::ep_barrier_kernel<<<1, 32, 0, st>>>(1, me, W, L->ep_peer_win, epoch, L->ep_wait_ns, L->error_word);
    L->launches += M > 0 ? 3 : 2;
    stage_end(L, ST_EXCHANGE, st);
    if (cudaGetLastError() != cudaSuccess) return fail(L, FFAI_ERR_CUDA, "exchange kernels launch failed");

    // the row count is known on the device only: kernels take their ranges from local_off; the path is
    // chosen for a balanced share
    L->ep_rows_dev = local_off + El;
    // hint for the kernel choice: this rank's own row count, but not below a small batch (a rank with few or no
    // tokens of its own may still receive many rows)
    if ((rc = run_experts_on_rows(L, M > 64 ? M : 64, El, local_off, st))) return rc;
    L->ep_rows_dev = nullptr;

    stage_begin(L, ST_EXCHANGE, st);
    ep::ep_barrier_kernel<<<1, 32, 0, st>>>(2, me, W, L->ep_peer_win, epoch, L->ep_wait_ns, L->error_word);
    L->launches += 1;
    stage_end(L, ST_EXCHANGE, st);
    return FFAI_OK;
}

int forward_device(ffai_moe_layer* L, const uint16_t* x, int T, uint16_t* out, const uint16_t* residual,
                   cudaStream_t st) {
    const ffai_moe_config& c = L->cfg;
    const int H = c.hidden, I = c.intermediate, E = c.n_experts, K = c.top_k;
    const int M = T * K;
    int rc;
    L->launches = 0;
    for (auto& n : L->ev_segments) n = 0;
    if (T == 0) {   // expert parallelism only: no rows of its own, but its experts serve the other ranks
        CUDA_TRY(L, cudaMemsetAsync(L->counts, 0, sizeof(uint32_t) * E, st));
        CUDA_TRY(L, cudaMemsetAsync(L->offsets, 0, sizeof(uint32_t) * (E + 1), st));
        return L->ep_peer_on ? forward_experts_ep_peer(L, x, 0, st) : forward_experts_ep(L, x, 0, st);
    }

    // The shared expert reads only the layer's input.  With a prefill-sized batch (or under expert parallelism) it runs
    // on a second stream beside router, plan, gather and the row exchange, which leave most of the GPU idle; the
    // combine waits for it.  With stage events on, everything stays on one stream so the stage times mean something.
    const float* sh_y = nullptr;
    const float* sh_gate = nullptr;
    const bool tc_shared = L->tc_ok && L->sh_x && L->opt_path != 1 && L->opt_path != 3 && (L->opt_path == 2 || T >= 16);
    auto run_shared = [&](cudaStream_t ss) -> int {
    if (c.shared_intermediate > 0) {
            const int Is = c.shared_intermediate;
            if (tc_shared) {
                using namespace g100;
                single_group_schedule_kernel<<<1, 32, 0, ss>>>(T, tc_group_rows(L), L->sh_sched);
                gather_rows_perm8_kernel<<<(T + 7) / 8, 256, 0, ss>>>(x, nullptr, 1, L->sh_x, T, H);
                Params p{};
                p.n_experts = 1; p.group_size = c.shared_group_size;
                p.offsets = L->sh_sched; p.tile_offsets = L->sh_sched + 2;
                p.activation = FFAI_ACT_SWIGLU;
                p.error_word = L->error_word;
                p.scales = L->w.shared_gate_proj.scales; p.biases = L->w.shared_gate_proj.biases;
                p.scales2 = L->w.shared_up_proj.scales; p.biases2 = L->w.shared_up_proj.biases;
                p.n_out = Is; p.K = H; p.m_tiles = (Is + BN / 2 - 1) / (BN / 2);
                p.out = L->sh_inner_bf; p.out_ld = Is; p.out_permute8 = 1;
                const bool wbf = L->sh_wbf[0] != nullptr;
                if (wbf) { p.wcache = L->sh_wbf[0]; p.wcache2 = L->sh_wbf[1]; p.cache_blocks = cache_blocks(Is, true); }
                if (wbf ? launch_grouped_gemm<true, uint16_t, true>(L->tm_sh_x, L->tm_sh_x, L->tm_sh_x, p, L->n_sms, ss)
                        : launch_grouped_gemm<true, uint16_t>(L->tm_sh_gate, L->tm_sh_up, L->tm_sh_x, p, L->n_sms, ss))
                    return fail(L, FFAI_ERR_CUDA, "shared gate/up grouped GEMM launch failed");
                p.scales = L->w.shared_down_proj.scales; p.biases = L->w.shared_down_proj.biases;
                p.scales2 = nullptr; p.biases2 = nullptr;
                p.n_out = H; p.K = Is; p.m_tiles = (H + BN - 1) / BN;
                p.out = L->sh_y; p.out_ld = H; p.out_permute8 = 0;
                if (wbf) { p.wcache = L->sh_wbf[2]; p.wcache2 = nullptr; p.cache_blocks = cache_blocks(H, false); }
                if (wbf ? launch_grouped_gemm<false, float, true>(L->tm_sh_inner, L->tm_sh_inner, L->tm_sh_inner, p, L->n_sms, ss)
                        : launch_grouped_gemm<false, float>(L->tm_sh_down, L->tm_sh_down, L->tm_sh_inner, p, L->n_sms, ss))
                    return fail(L, FFAI_ERR_CUDA, "shared down grouped GEMM launch failed");
                L->launches += 4;
            } else {
                GemvParams p = L->no_gate ? gemv_params(L->w.shared_up_proj, nullptr, Is, H, c.shared_group_size, 1)
                                          : gemv_params(L->w.shared_gate_proj, &L->w.shared_up_proj, Is, H, c.shared_group_size, 1);
                p.n_rows = T;
                p.activation = FFAI_ACT_SWIGLU;
                p.post_relu2 = L->no_gate;   // beside gate-less experts the shared expert has their form (NemotronHText.swift:885-891)
                if ((rc = L->no_gate ? launch_grouped_gemv<uint16_t, float, false>(p, c.shared_bits, x, L->sh_inner, 1, ss)
                                     : launch_grouped_gemv<uint16_t, float, true>(p, c.shared_bits, x, L->sh_inner, 1, ss)))
                    return fail(L, rc, "shared gate/up launch failed");
                GemvParams d = gemv_params(L->w.shared_down_proj, nullptr, H, Is, c.shared_group_size, 1);
                d.n_rows = T;
                if ((rc = launch_grouped_gemv<float, float, false>(d, c.shared_bits, L->sh_inner, L->sh_y, 1, ss)))
                    return fail(L, rc, "shared down launch failed");
                L->launches += 2;
            }
            sh_y = L->sh_y;
            if (c.shared_gate_kind == FFAI_LINEAR_AFFINE) {
                if ((rc = launch_affine_rowdot(L->w.shared_gate, c.shared_gate_bits, c.shared_gate_group_size, x, L->sh_gate, T, H, ss)))
                    return fail(L, rc, "shared gate launch failed");
                L->launches += 1;
                sh_gate = L->sh_gate;
            } else if (c.shared_gate_kind == FFAI_LINEAR_F32) {
                dense_rowdot_kernel<float><<<(T + 3) / 4, 128, 0, ss>>>((const float*)L->w.shared_gate.weight, x, L->sh_gate, T, H);
                L->launches += 1;
                sh_gate = L->sh_gate;
            } else if (c.shared_gate_kind == FFAI_LINEAR_BF16) {
                dense_rowdot_kernel<uint16_t><<<(T + 3) / 4, 128, 0, ss>>>((const uint16_t*)L->w.shared_gate.weight, x, L->sh_gate, T, H);
                L->launches += 1;
                sh_gate = L->sh_gate;
            }
        }
        return FFAI_OK;
    };
    const bool shared_beside = c.shared_intermediate > 0 && L->opt_overlap && !L->timing && (T >= 96 || c.ep_world > 1);
    if (shared_beside) {
        if (!L->aux_stream) {
            CUDA_TRY(L, cudaStreamCreateWithFlags(&L->aux_stream, cudaStreamNonBlocking));
            CUDA_TRY(L, cudaEventCreateWithFlags(&L->ev_fork, cudaEventDisableTiming));
            CUDA_TRY(L, cudaEventCreateWithFlags(&L->ev_join, cudaEventDisableTiming));
        }
        CUDA_TRY(L, cudaEventRecord(L->ev_fork, st));
        CUDA_TRY(L, cudaStreamWaitEvent(L->aux_stream, L->ev_fork, 0));
        if ((rc = run_shared(L->aux_stream))) return rc;
        CUDA_TRY(L, cudaEventRecord(L->ev_join, L->aux_stream));
    }

    // stage 0: router (projection + bias + top-k + softmax)
    stage_begin(L, ST_ROUTER, st);
    RouterParams rp = router_params(L);
    // small batches: the router kernel's last block also builds the dispatch plan
    const PlanOut fused_plan = (M <= PLAN_ENTRIES_PER_WARP) ? PlanOut{L->counts, L->offsets, L->perm, L->inv_perm, L->expert_order} : PlanOut{nullptr, nullptr, nullptr, nullptr, nullptr};
    bool plan_done = false, tiles_done = false;
    // 4-bit streaming kernels read per-token rows through the permutation: the rows (8-run permuted) and their
    // 64-run sums are written once per token, by the router kernel when it is the small-batch one
    const uint16_t* xr = L->router_x ? L->router_x : x;   // the router's input rows (its own under a split forward)
    uint16_t* tok_x = (L->mma_ok && c.ep_world <= 1 && xr == x) ? L->x_tok : nullptr;
    const int xp_tok = (H / 32 + 3) & ~3;
    bool tok_rows_done = false;
    if (T >= 96) {
        int nr = launch_router_batched(rp, xr, T, L->indices, L->rweights, L->logits, L->router_partials,
                                       L->router_partials_cap, L->n_sms, st);
        if (nr < 0) return fail(L, FFAI_ERR_CUDA, "router launch failed: %s", cudaGetErrorString(cudaGetLastError()));
        L->launches += nr;
    } else if ((rp.kind == FFAI_LINEAR_F32 && launch_router_rows<1>(rp, xr, T, L->indices, L->rweights, L->logits, L->tickets, fused_plan, tok_x, L->xsum_tok, xp_tok, st) == 0) ||
               (rp.kind == FFAI_LINEAR_BF16 && launch_router_rows<2>(rp, xr, T, L->indices, L->rweights, L->logits, L->tickets, fused_plan, tok_x, L->xsum_tok, xp_tok, st) == 0)) {
        L->launches += 1;
        plan_done = fused_plan.perm != nullptr;
        tok_rows_done = tok_x != nullptr;
    } else {
        if ((rc = launch_router(rp, xr, T, L->indices, L->rweights, L->logits, st)))
            return fail(L, rc, "router launch failed: %s", cudaGetErrorString(cudaGetLastError()));
        L->launches += 1;
    }
    stage_end(L, ST_ROUTER, st);

    // stage 1: dispatch plan
    stage_begin(L, ST_PLAN, st);
    if (!plan_done) {
        int nl = launch_plan(L->indices, M, E, L->counts, L->offsets, L->perm, L->inv_perm, L->block_hist, st,
                             tc_group_rows(L), L->tile_offsets, &tiles_done);
        if (nl < 0) return fail(L, FFAI_ERR_CUDA, "plan launch failed: %s", cudaGetErrorString(cudaGetLastError()));
        L->launches += nl;
    }
    stage_end(L, ST_PLAN, st);

    const bool ep_on = c.ep_world > 1;
    if (ep_on) {
        if ((rc = L->ep_peer_on ? forward_experts_ep_peer(L, x, T, st) : forward_experts_ep(L, x, T, st))) return rc;
    }
    // Path choice for the routed experts:
    //   register-streaming mma kernels  4-bit, few rows per expert (decode): bound by HBM
    //   tcgen05 grouped GEMM            4-bit, many rows per expert (prefill): bound by the tensor cores
    //   CUDA-core grouped GEMV          any bit width / group size, and shapes the others do not take
    const double rows_per_expert = (double)M / E;
    const bool can_tc = tc_possible(L);
    bool mma_experts = false, tc_experts = false, decode_pdl = false;
    if (ep_on) { /* done above */ }
    else if (L->opt_path == 3) mma_experts = L->mma_ok;
    else if (L->opt_path == 2) tc_experts = can_tc;
    else if (L->opt_path == 0) {
        if (L->mma_ok && (rows_per_expert <= 16.0 || !can_tc)) mma_experts = rows_per_expert <= 48.0;
        if (!mma_experts && can_tc) tc_experts = M >= (L->opt_tc_min_rows > 0 ? L->opt_tc_min_rows : 64);
        if (!mma_experts && !tc_experts && L->mma_ok && rows_per_expert <= 48.0) mma_experts = true;
    }

    if (mma_experts) {
        using namespace dmma;
        stage_begin(L, ST_GATHER, st);
        const int xp_h = (H / 32 + 3) & ~3, xp_i = (I / 32 + 3) & ~3;
        if (!tok_rows_done) {   // one row per token (not per routed row); the kernels follow the permutation themselves
            gather_perm8_sum64_kernel<<<(T + 7) / 8, 256, 0, st>>>(x, nullptr, 1, L->x_tok, L->xsum_tok, T, H, xp_h);
            L->launches += 1;
        }
        stage_end(L, ST_GATHER, st);

        // Which decode kernels: the bulk-copy streamed ones (a warp owns a 16-row block; the batch sizes where they
        // measure faster on the GPT-OSS shape: more than 8 and at most 160 routed rows), else the cp.async ring kernels.
        const bool stream = L->st_gate_up && (L->opt_decode == 2 || (L->opt_decode == 0 && M > 8 && M <= 160));
        // Programmatic dependent launches down the decode chain (gate/up after the router, down after gate/up, the
        // combine after down): a kernel's blocks start as its predecessor's retire.  Stage events between the
        // launches would serialise them again, so the chain is plain when timing is on.
        const bool pdl = L->opt_pdl && !L->timing;
        decode_pdl = pdl;
        bool streamed = false;
        if (stream) {
            dstr::Params q{};
            q.n_experts = E; q.offsets = L->offsets; q.order = plan_done ? L->expert_order : nullptr;
            q.activation = c.activation; q.limit = c.swiglu_limit; q.alpha = c.swiglu_alpha;
            q.nt2_cost = L->opt_nt2_cost; q.error_word = L->error_word;
            // warps that share one 16-row block: one, unless the batch is so small that whole items are too few for the grid
            const int team = L->opt_decode_team ? L->opt_decode_team : (M <= 8 ? 4 : 1);
            stage_begin(L, ST_GATE_UP, st);
            q.wt = L->st_gate_up; q.rb1 = L->w.gate_proj.row_bias; q.rb2 = L->w.up_proj.row_bias;
            q.N = I; q.K = H; q.x = L->x_tok; q.row_src = L->perm; q.row_div = K; q.xsum = L->xsum_tok; q.xsum_pitch = xp_h;
            q.out = L->inner_bf; q.out_parts = L->inner_parts;
            q.tables_ready = 0;
            streamed = launch_stream_decode<true>(q, team, L->n_sms, st, pdl);
            stage_end(L, ST_GATE_UP, st);
            if (streamed) {
                stage_begin(L, ST_DOWN, st);
                q.wt = L->st_down; q.rb1 = L->w.down_proj.row_bias; q.rb2 = nullptr;
                q.N = H; q.K = I; q.x = L->inner_bf; q.row_src = nullptr; q.row_div = 1; q.xsum = nullptr; q.xsum_parts = L->inner_parts;
                q.out = L->y; q.out_parts = nullptr;
                q.tables_ready = 1;   // routing tables were written before the gate/up kernel started
                streamed = launch_stream_decode<false>(q, team, L->n_sms, st, pdl);
                stage_end(L, ST_DOWN, st);
                if (!streamed) return fail(L, FFAI_ERR_UNSUPPORTED, "down projection does not fit the streamed decode kernel");
                L->launches += 2;
            }
            if (cudaGetLastError() != cudaSuccess) return fail(L, FFAI_ERR_CUDA, "decode kernels launch failed");
        }
        if (!streamed) {
        Params p{};
        p.group_size = c.expert_group_size;
        p.offsets = L->offsets;
        p.order = plan_done ? L->expert_order : nullptr;   // longest experts first shortens the tail of the grid
        p.activation = c.activation; p.limit = c.swiglu_limit; p.alpha = c.swiglu_alpha;
        const int nt = rows_per_expert > 4.0 ? 2 : 1;  // 16 activation rows per pass instead of 8
        // few routed rows -> few active experts -> slice the reduction axis to keep every SM busy
        const int ksplit = L->opt_ksplit > 0 ? L->opt_ksplit : (M <= 4 ? 2 : 1);

        stage_begin(L, ST_GATE_UP, st);
        p.w1 = L->w.gate_proj.weight; p.s1 = L->w.gate_proj.scales; p.b1 = L->w.gate_proj.biases; p.rb1 = L->w.gate_proj.row_bias;
        p.w2 = L->w.up_proj.weight; p.s2 = L->w.up_proj.scales; p.b2 = L->w.up_proj.biases; p.rb2 = L->w.up_proj.row_bias;
        p.sb1 = L->sb_gate; p.sb2 = L->sb_up;
        p.N = I; p.K = H; p.x = L->x_tok; p.xsum = L->xsum_tok; p.xsum_pitch = xp_h; p.out = L->inner_bf;
        p.row_src = L->perm; p.row_div = K;
        p.out_parts = L->inner_parts;
        launch_mma_decode<true>(p, E, nt, ksplit, st, pdl);
        p.row_src = nullptr; p.row_div = 1;
        L->launches += 1;
        stage_end(L, ST_GATE_UP, st);

        stage_begin(L, ST_DOWN, st);
        p.w1 = L->w.down_proj.weight; p.s1 = L->w.down_proj.scales; p.b1 = L->w.down_proj.biases; p.rb1 = L->w.down_proj.row_bias;
        p.w2 = nullptr; p.s2 = nullptr; p.b2 = nullptr; p.rb2 = nullptr;
        p.sb1 = L->sb_down; p.sb2 = nullptr;
        p.N = H; p.K = I; p.x = L->inner_bf; p.xsum = nullptr; p.xsum_parts = L->inner_parts; p.xsum_pitch = xp_i; p.out = L->y;
        p.out_parts = nullptr;
        // group 32: 32 rows per warp through the two-projection kernel (measured 9 % faster there; no gain at group 64)
        p.pair = c.expert_group_size == 32;
        if (p.pair) launch_mma_decode<true>(p, E, nt, ksplit, st, pdl);
        else launch_mma_decode<false>(p, E, nt, ksplit, st, pdl);
        L->launches += 1;
        stage_end(L, ST_DOWN, st);
        if (cudaGetLastError() != cudaSuccess) return fail(L, FFAI_ERR_CUDA, "decode kernels launch failed");
        }
    } else
    if (tc_experts) {
        using namespace g100;
        stage_begin(L, ST_GATHER, st);
        if (!tiles_done) {
            tile_schedule_kernel<<<1, 32, 0, st>>>(L->offsets, E, tc_group_rows(L), L->tile_offsets);
            L->launches += 1;
        }
        gather_rows_perm8_kernel<<<(M + 7) / 8, 256, 0, st>>>(x, L->perm, K, L->xg, M, H);
        L->launches += 1;
        stage_end(L, ST_GATHER, st);

        Params p{};
        p.n_experts = E; p.group_size = c.expert_group_size;
        p.offsets = L->offsets; p.tile_offsets = L->tile_offsets;
        p.activation = c.activation; p.limit = c.swiglu_limit; p.alpha = c.swiglu_alpha;
        p.error_word = L->error_word;
        p.timeline = L->timeline;
        if (L->timeline) cudaMemsetAsync(L->timeline, 0, sizeof(long long) * g100::TL_ROLES * g100::TL_SLOTS * g100::TL_EVENTS, st);

        stage_begin(L, ST_GATE_UP, st);
        p.scales = L->w.gate_proj.scales; p.biases = L->w.gate_proj.biases; p.row_bias = L->w.gate_proj.row_bias;
        p.scales2 = L->w.up_proj.scales; p.biases2 = L->w.up_proj.biases; p.row_bias2 = L->w.up_proj.row_bias;
        if (c.expert_group_size != 32) { p.sb = L->sb_gate; p.sb2 = L->sb_up; }
        p.n_out = I; p.K = H; p.m_tiles = (I + BN / 2 - 1) / (BN / 2);
        p.out = L->inner_bf; p.out_ld = I; p.out_permute8 = 1;
        if (tc_gate_up(L, p, rows_per_expert, st))
            return fail(L, FFAI_ERR_CUDA, "gate/up grouped GEMM launch failed: %s", cudaGetErrorString(cudaGetLastError()));
        L->launches += 1;
        stage_end(L, ST_GATE_UP, st);

        stage_begin(L, ST_DOWN, st);
        p.timeline = nullptr;
        p.scales = L->w.down_proj.scales; p.biases = L->w.down_proj.biases; p.row_bias = L->w.down_proj.row_bias;
        p.scales2 = nullptr; p.biases2 = nullptr; p.row_bias2 = nullptr;
        p.sb = c.expert_group_size != 32 ? L->sb_down : nullptr; p.sb2 = nullptr;
        p.n_out = H; p.K = I; p.m_tiles = (H + BN - 1) / BN;
        p.out = L->y_bf; p.out_ld = H; p.out_permute8 = 0;
        if (tc_down<uint16_t>(L, p, st))
            return fail(L, FFAI_ERR_CUDA, "down grouped GEMM launch failed: %s", cudaGetErrorString(cudaGetLastError()));
        L->launches += 1;
        stage_end(L, ST_DOWN, st);
    } else if (!ep_on) {
        // gate/up products + activation -> inner[M, I]; rows are read through the permutation
        stage_begin(L, ST_GATE_UP, st);
        {
            GemvParams p = L->no_gate ? gemv_params(L->w.up_proj, nullptr, I, H, c.expert_group_size, E)
                                      : gemv_params(L->w.gate_proj, &L->w.up_proj, I, H, c.expert_group_size, E);
            p.offsets = L->offsets;
            p.in_row_ids = L->perm;
            p.in_row_div = K;
            p.n_rows = M;
            p.activation = c.activation; p.limit = c.swiglu_limit; p.alpha = c.swiglu_alpha;
            p.post_relu2 = L->no_gate;
            if ((rc = L->no_gate ? launch_grouped_gemv<uint16_t, float, false>(p, c.expert_bits, x, L->inner, E, st)
                                 : launch_grouped_gemv<uint16_t, float, true>(p, c.expert_bits, x, L->inner, E, st)))
                return fail(L, rc, "gate/up launch failed: %s", cudaGetErrorString(cudaGetLastError()));
            L->launches += 1;
        }
        stage_end(L, ST_GATE_UP, st);
        // down product -> y[M, H]
        stage_begin(L, ST_DOWN, st);
        {
            GemvParams p = gemv_params(L->w.down_proj, nullptr, H, I, c.expert_group_size, E);
            p.offsets = L->offsets;
            p.n_rows = M;
            if ((rc = launch_grouped_gemv<float, float, false>(p, c.expert_bits, L->inner, L->y, E, st)))
                return fail(L, rc, "down launch failed: %s", cudaGetErrorString(cudaGetLastError()));
            L->launches += 1;
        }
        stage_end(L, ST_DOWN, st);
    }

    // shared expert (when it did not run beside the rest)
    stage_begin(L, ST_SHARED, st);
    if (shared_beside) {
        CUDA_TRY(L, cudaStreamWaitEvent(st, L->ev_join, 0));
    } else if ((rc = run_shared(st))) {
        return rc;
    }
    stage_end(L, ST_SHARED, st);
    stage_begin(L, ST_COMBINE, st);
    if (ep_on && L->ep_peer_on)
        ep::combine_peer_kernel<<<T, 256, 0, st>>>(L->ep_peer_y, L->inv_perm, L->indices, L->offsets, L->ep_send_base, L->e_local,
                                                   L->rweights, K, sh_y, sh_gate, residual, out, H, (uint32_t)L->mx_rows, L->error_word);
    else if (ep_on)
        combine_kernel<float, float><<<T, 256, 0, st>>>(L->ep_home_y, L->inv_perm, L->rweights, K, sh_y, sh_gate, residual, out, H);
    else if (tc_experts)
        combine_kernel<uint16_t, float><<<T, 256, 0, st>>>(L->y_bf, L->inv_perm, L->rweights, K, sh_y, sh_gate, residual, out, H);
    else if (launch_kernel(combine_kernel<float, float>, dim3(T), dim3(256), 0, st, decode_pdl && !sh_y, (const float*)L->y, (const uint32_t*)L->inv_perm,
                           (const float*)L->rweights, K, sh_y, sh_gate, residual, out, H) != cudaSuccess)
        return fail(L, FFAI_ERR_CUDA, "combine launch failed");
    L->launches += 1;
    stage_end(L, ST_COMBINE, st);
    if (cudaGetLastError() != cudaSuccess) return fail(L, FFAI_ERR_CUDA, "combine launch failed");
    return FFAI_OK;
}

int check_forward_args(ffai_moe_layer* L, const void* x, int T, const void* out) {
    if (!L) return FFAI_ERR_INVALID_ARG;
    if (L->cfg.struct_size == 0) return fail(L, FFAI_ERR_INVALID_ARG, "layer was not created successfully");
    if (!L->weights_set) return fail(L, FFAI_ERR_NOT_READY, "forward called before set_weights");
    if (T < 0) return fail(L, FFAI_ERR_INVALID_ARG, "n_tokens must be >= 0");
    if (T > L->cfg.max_tokens) return fail(L, FFAI_ERR_INVALID_ARG, "n_tokens %d exceeds max_tokens %d", T, L->cfg.max_tokens);
    if (T > 0 && (!x || !out)) return fail(L, FFAI_ERR_INVALID_ARG, "x and out must be non-null");
    return FFAI_OK;
}

}  // namespace

extern "C" FFAI_API int ffai_moe_forward(ffai_moe_layer* L, const uint16_t* x, int32_t T, uint16_t* out,
                                const uint16_t* residual, const ffai_moe_debug* debug, void* stream) {
    int rc = check_forward_args(L, x, T, out);
    if (rc) return rc;
    if (T == 0 && L->cfg.ep_world <= 1) return FFAI_OK;   // an expert-parallel rank without tokens still serves its experts
    if (!aligned16(x) || !aligned16(out) || (residual && !aligned16(residual)))
        return fail(L, FFAI_ERR_INVALID_ARG, "x/out/residual must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if ((rc = forward_device(L, x, T, out, residual, st))) return rc;
    return copy_debug(L, debug, T, st, cudaMemcpyDeviceToDevice);
}

extern "C" FFAI_API int ffai_moe_forward_split(ffai_moe_layer* L, const uint16_t* x, const uint16_t* x_router, int32_t T,
                                               uint16_t* out, const uint16_t* residual, const ffai_moe_debug* debug, void* stream) {
    if (!L) return FFAI_ERR_INVALID_ARG;
    if (x_router && !aligned16(x_router)) return fail(L, FFAI_ERR_INVALID_ARG, "x_router must be 16-byte aligned");
    L->router_x = x_router;
    const int rc = ffai_moe_forward(L, x, T, out, residual, debug, stream);
    L->router_x = nullptr;
    return rc;
}

extern "C" FFAI_API int ffai_moe_forward_host(ffai_moe_layer* L, const uint16_t* x, int32_t T, uint16_t* out,
                                              const uint16_t* residual, const ffai_moe_debug* debug);

// How many chunks the host entry point cuts a batch into (1 = not at all).  Only batches whose chunks still take
// the tensor-core path with every expert holding more than one decode batch of rows are cut, so a chunk runs the
// kernels the whole batch would; not under expert parallelism (ranks must take the same steps), not with debug
// outputs or stage timing.
int host_chunks(const ffai_moe_layer* L, int T, const ffai_moe_debug* debug) {
    const ffai_moe_config& c = L->cfg;
    if (L->opt_host_chunks == 1 || c.ep_world > 1 || debug || L->timing || L->opt_path == 1 || L->opt_path == 3) return 1;
    if (!L->tc_ok || !(c.expert_bits == 4 || L->exp_wbf[0])) return 1;
    // measured on the 256-expert layer at 8192 tokens: 2.20 ms whole, 1.88 in two chunks, 1.86 in three, 2.00 in four
    // (smaller chunks fill the 128-row token tiles of the grouped GEMM less well)
    int n = T / 2048;
    const int cap = L->opt_host_chunks > 1 ? L->opt_host_chunks : 3;
    if (n > cap) n = cap;
    if (n < 2) return 1;
    const int per = (((T + n - 1) / n) + 127) & ~127;
    const double rows_per_expert = (double)per * c.top_k / c.n_experts;
    return rows_per_expert >= 48.0 ? n : 1;
}

extern "C" FFAI_API int ffai_moe_forward_host_split(ffai_moe_layer* L, const uint16_t* x, const uint16_t* x_router, int32_t T,
                                                    uint16_t* out, const uint16_t* residual, const ffai_moe_debug* debug) {
    int rc = check_forward_args(L, x, T, out);
    if (rc) return rc;
    if (!x_router || T == 0) return ffai_moe_forward_host(L, x, T, out, residual, debug);
    CUDA_TRY(L, cudaSetDevice(L->device));
    if (!L->dev_xr && (rc = ws_alloc(L, &L->dev_xr, (size_t)L->cfg.max_tokens * L->cfg.hidden))) return rc;
    CUDA_TRY(L, cudaMemcpy(L->dev_xr, x_router, (size_t)T * L->cfg.hidden * 2, cudaMemcpyHostToDevice));
    L->router_x = L->dev_xr;
    rc = ffai_moe_forward_host(L, x, T, out, residual, debug);
    L->router_x = nullptr;
    return rc;
}

extern "C" FFAI_API int ffai_moe_forward_host(ffai_moe_layer* L, const uint16_t* x, int32_t T, uint16_t* out,
                                     const uint16_t* residual, const ffai_moe_debug* debug) {
    int rc = check_forward_args(L, x, T, out);
    if (rc) return rc;
    if (T == 0 && L->cfg.ep_world <= 1) return FFAI_OK;
    const ffai_moe_config& c = L->cfg;
    CUDA_TRY(L, cudaSetDevice(L->device));
    const size_t cap = (size_t)c.max_tokens * c.hidden * 2;
    if (!L->own_stream) {
        CUDA_TRY(L, cudaStreamCreateWithFlags(&L->own_stream, cudaStreamNonBlocking));
        void* p;
        CUDA_TRY(L, cudaMallocHost(&p, cap)); L->owned_pinned.push_back(p); L->pin_x = (uint16_t*)p;
        CUDA_TRY(L, cudaMallocHost(&p, cap)); L->owned_pinned.push_back(p); L->pin_out = (uint16_t*)p;
        CUDA_TRY(L, cudaMallocHost(&p, cap + 16)); L->owned_pinned.push_back(p); L->pin_res = (uint16_t*)p;
        if ((rc = ws_alloc(L, &L->dev_x, cap / 2))) return rc;
        if ((rc = ws_alloc(L, &L->dev_out, cap / 2))) return rc;
        if ((rc = ws_alloc(L, &L->dev_res, cap / 2))) return rc;
    }
    cudaStream_t st = L->own_stream;
    const size_t bytes = (size_t)T * c.hidden * 2;
    // Page-locked caller buffers are copied from directly; pageable ones are staged through the handle's
    // pinned buffers so the transfers are asynchronous DMA either way.
    auto is_pinned = [](const void* p) {
        cudaPointerAttributes a;
        if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return false; }
        return a.type == cudaMemoryTypeHost;
    };
    const bool x_pinned = is_pinned(x), out_pinned = is_pinned(out);
    const bool chunked = host_chunks(L, T, debug) > 1;
    if (bytes == 0) {
        // nothing to stage
    } else if (chunked) {
        if (!x_pinned) memcpy(L->pin_x, x, bytes);   // the copies themselves are issued per chunk below
    } else if (x_pinned) {
        CUDA_TRY(L, cudaMemcpyAsync(L->dev_x, x, bytes, cudaMemcpyHostToDevice, st));
    } else {
        memcpy(L->pin_x, x, bytes);
        CUDA_TRY(L, cudaMemcpyAsync(L->dev_x, L->pin_x, bytes, cudaMemcpyHostToDevice, st));
    }
    const uint16_t* dres = nullptr;
    if (residual && bytes) {
        if (chunked) {
            if (!is_pinned(residual)) memcpy(L->pin_res, residual, bytes);
        } else if (is_pinned(residual)) {
            CUDA_TRY(L, cudaMemcpyAsync(L->dev_res, residual, bytes, cudaMemcpyHostToDevice, st));
        } else {
            memcpy(L->pin_res, residual, bytes);
            CUDA_TRY(L, cudaMemcpyAsync(L->dev_res, L->pin_res, bytes, cudaMemcpyHostToDevice, st));
        }
        dres = L->dev_res;
    }
    const int n_chunks = host_chunks(L, T, debug);
    if (n_chunks > 1) {
        // A large batch goes through in chunks: tokens are independent (routing, experts and combine are all
        // per token and a chunk takes the same kernels as the whole batch), so the result is the same bits,
        // and chunk i's experts run while chunk i+1 uploads and chunk i-1 downloads.
        if (!L->h2d_stream) {
            CUDA_TRY(L, cudaStreamCreateWithFlags(&L->h2d_stream, cudaStreamNonBlocking));
            CUDA_TRY(L, cudaStreamCreateWithFlags(&L->d2h_stream, cudaStreamNonBlocking));
            for (auto& e : L->ev_in) CUDA_TRY(L, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
            for (auto& e : L->ev_out) CUDA_TRY(L, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        }
        const int per = (((T + n_chunks - 1) / n_chunks) + 127) & ~127;
        const uint16_t* xsrc = x_pinned ? x : L->pin_x;
        const uint16_t* rsrc = residual ? (is_pinned(residual) ? residual : L->pin_res) : nullptr;
        uint16_t* odst = out_pinned ? out : L->pin_out;
        const uint16_t* router_rows = L->router_x;
        int launches = 0;
        for (int i = 0; i < n_chunks; ++i) {
            const int t0 = i * per, ti = std::min(per, T - t0);
            const size_t off = (size_t)t0 * c.hidden, nb = (size_t)ti * c.hidden * 2;
            CUDA_TRY(L, cudaMemcpyAsync(L->dev_x + off, xsrc + off, nb, cudaMemcpyHostToDevice, L->h2d_stream));
            if (rsrc) CUDA_TRY(L, cudaMemcpyAsync(L->dev_res + off, rsrc + off, nb, cudaMemcpyHostToDevice, L->h2d_stream));
            CUDA_TRY(L, cudaEventRecord(L->ev_in[i], L->h2d_stream));
        }
        for (int i = 0; i < n_chunks; ++i) {
            const int t0 = i * per, ti = std::min(per, T - t0);
            const size_t off = (size_t)t0 * c.hidden, nb = (size_t)ti * c.hidden * 2;
            CUDA_TRY(L, cudaStreamWaitEvent(st, L->ev_in[i], 0));
            if (router_rows) L->router_x = router_rows + off;
            rc = forward_device(L, L->dev_x + off, ti, L->dev_out + off, rsrc ? L->dev_res + off : nullptr, st);
            L->router_x = router_rows;
            if (rc) return rc;
            launches += L->launches;
            CUDA_TRY(L, cudaEventRecord(L->ev_out[i], st));
            CUDA_TRY(L, cudaStreamWaitEvent(L->d2h_stream, L->ev_out[i], 0));
            CUDA_TRY(L, cudaMemcpyAsync(odst + off, L->dev_out + off, nb, cudaMemcpyDeviceToHost, L->d2h_stream));
        }
        L->launches = launches;
    } else {
        if ((rc = forward_device(L, L->dev_x, T, L->dev_out, dres, st))) return rc;
        if (bytes) CUDA_TRY(L, cudaMemcpyAsync(out_pinned ? out : L->pin_out, L->dev_out, bytes, cudaMemcpyDeviceToHost, st));
        if ((rc = copy_debug(L, debug, T, st, cudaMemcpyDeviceToHost))) return rc;
    }
    uint32_t* pin_err = reinterpret_cast<uint32_t*>(L->pin_res + cap / 2);
    CUDA_TRY(L, cudaMemcpyAsync(pin_err, L->error_word, 4, cudaMemcpyDeviceToHost, st));
    CUDA_TRY(L, cudaStreamSynchronize(st));
    if (n_chunks > 1) CUDA_TRY(L, cudaStreamSynchronize(L->d2h_stream));
    if (*pin_err) {
        cudaMemsetAsync(L->error_word, 0, 4, st);
        return fail(L, FFAI_ERR_DEVICE_CHECK, "a kernel gave up a bounded wait (code %u)", *pin_err);
    }
    if (!out_pinned && bytes) memcpy(out, L->pin_out, bytes);
    return FFAI_OK;
}


// ───────────────────────────── safetensors -> ffai_moe_weights ─────────────────────────────

struct ffai_st_file {
    ffai::st::File* f = nullptr;
    std::string error;
};

extern "C" FFAI_API int ffai_st_open(const char* path, ffai_st_file** out) {
    if (!path || !out) return FFAI_ERR_INVALID_ARG;
    ffai_st_file* h = new (std::nothrow) ffai_st_file();
    if (!h) return FFAI_ERR_CUDA;
    h->f = ffai::st::open_file(path, &h->error);
    *out = h;
    return h->f ? FFAI_OK : FFAI_ERR_INVALID_ARG;
}

extern "C" FFAI_API void ffai_st_close(ffai_st_file* h) {
    if (!h) return;
    ffai::st::close_file(h->f);
    delete h;
}

extern "C" FFAI_API const char* ffai_st_last_error(const ffai_st_file* h) { return h ? h->error.c_str() : "null handle"; }

extern "C" FFAI_API int ffai_st_tensor(const ffai_st_file* h, const char* name, const void** data, uint64_t* n_bytes,
                                       char dtype[8], int64_t shape[8], int32_t* n_dims) {
    if (!h || !h->f || !name) return FFAI_ERR_INVALID_ARG;
    const ffai::st::Tensor* t = ffai::st::find(h->f, name);
    if (!t) return FFAI_ERR_INVALID_ARG;
    if (data) *data = h->f->data + t->begin;
    if (n_bytes) *n_bytes = t->end - t->begin;
    if (dtype) { memset(dtype, 0, 8); strncpy(dtype, t->dtype.c_str(), 7); }
    if (n_dims) *n_dims = (int32_t)t->shape.size();
    if (shape) for (size_t i = 0; i < t->shape.size() && i < 8; ++i) shape[i] = t->shape[i];
    return FFAI_OK;
}

extern "C" FFAI_API int32_t ffai_st_derive_bits(int64_t weight_packed_cols, int64_t scale_cols, int32_t group_size) {
    const int64_t in_features = scale_cols * group_size;   // Layers.swift:348-363
    if (in_features <= 0 || (32 * weight_packed_cols) % in_features) return 0;
    return (int32_t)((32 * weight_packed_cols) / in_features);
}

namespace {
int st_fail(ffai_st_file* h, const std::string& msg) {
    h->error = msg;
    return FFAI_ERR_INVALID_ARG;
}

// One stacked quantized projection <base>.{weight,scales,biases}: shapes [n, out, in*bits/32] and [n, out, in/gs].
int st_qproj(ffai_st_file* h, const std::string& base, int gs, ffai_qproj* q, int64_t* n, int64_t* out_dim, int64_t* in_dim, int* bits) {
    const ffai::st::Tensor* w = ffai::st::find(h->f, base + ".weight");
    const ffai::st::Tensor* s = ffai::st::find(h->f, base + ".scales");
    const ffai::st::Tensor* b = ffai::st::find(h->f, base + ".biases");
    if (!w || !s || !b) return st_fail(h, "missing " + base + ".{weight,scales,biases}");
    if (w->dtype != "U32") return st_fail(h, base + ".weight is not U32");
    if (s->dtype != "BF16" || b->dtype != "BF16") return st_fail(h, base + ": scales/biases must be BF16");
    if (w->shape.size() < 2 || s->shape != b->shape || s->shape.size() != w->shape.size()) return st_fail(h, base + ": shapes do not match");
    const size_t r = w->shape.size();
    const int64_t wcols = w->shape[r - 1], scols = s->shape[r - 1];
    const int bt = ffai_st_derive_bits(wcols, scols, gs);
    if (!valid_bits(bt)) return st_fail(h, base + ": shapes do not describe an affine-quantized tensor at this group size");
    for (size_t i = 0; i + 1 < r; ++i)
        if (w->shape[i] != s->shape[i]) return st_fail(h, base + ": leading dimensions differ");
    // pointers into the mapping are handed out typed: the payload offsets must keep their natural alignment
    if ((reinterpret_cast<uintptr_t>(h->f->data + w->begin) & 3u) || (reinterpret_cast<uintptr_t>(h->f->data + s->begin) & 1u) ||
        (reinterpret_cast<uintptr_t>(h->f->data + b->begin) & 1u))
        return st_fail(h, base + ": tensor data is not aligned to its element size");
    if (r > 3) return st_fail(h, base + ": more than three dimensions");
    *n = r == 3 ? w->shape[0] : 1;
    *out_dim = w->shape[r - 2];
    *in_dim = scols * gs;
    *bits = bt;
    q->weight = reinterpret_cast<const uint32_t*>(h->f->data + w->begin);
    q->scales = reinterpret_cast<const uint16_t*>(h->f->data + s->begin);
    q->biases = reinterpret_cast<const uint16_t*>(h->f->data + b->begin);
    q->row_bias = nullptr;
    return FFAI_OK;
}

// A router / gate projection <base>.weight [+ .scales/.biases]: dense F32 / BF16, or affine.
int st_linear(ffai_st_file* h, const std::string& base, int gs, ffai_linear* lin, int* kind, int* bits, int64_t* out_dim, int64_t* in_dim) {
    const ffai::st::Tensor* w = ffai::st::find(h->f, base + ".weight");
    if (!w || w->shape.size() != 2) return st_fail(h, "missing or non-2-D " + base + ".weight");
    *lin = ffai_linear{};
    if (reinterpret_cast<uintptr_t>(h->f->data + w->begin) & (w->dtype == "BF16" ? 1u : 3u))
        return st_fail(h, base + ".weight is not aligned to its element size");
    lin->weight = h->f->data + w->begin;
    *out_dim = w->shape[0];
    if (w->dtype == "F32") { *kind = FFAI_LINEAR_F32; *bits = 0; *in_dim = w->shape[1]; }
    else if (w->dtype == "BF16") { *kind = FFAI_LINEAR_BF16; *bits = 0; *in_dim = w->shape[1]; }
    else if (w->dtype == "U32") {
        const ffai::st::Tensor* s = ffai::st::find(h->f, base + ".scales");
        const ffai::st::Tensor* b = ffai::st::find(h->f, base + ".biases");
        if (!s || !b || s->shape.size() != 2) return st_fail(h, base + ": packed weight without scales/biases");
        if (s->dtype != "BF16" || b->dtype != "BF16" || s->shape != b->shape || s->shape[0] != w->shape[0])
            return st_fail(h, base + ": scales/biases must be BF16 with the weight's row count");
        if ((reinterpret_cast<uintptr_t>(h->f->data + s->begin) & 1u) || (reinterpret_cast<uintptr_t>(h->f->data + b->begin) & 1u))
            return st_fail(h, base + ": scales/biases are not aligned to their element size");
        *bits = ffai_st_derive_bits(w->shape[1], s->shape[1], gs);
        if (!valid_bits(*bits)) return st_fail(h, base + ": shapes do not describe an affine-quantized tensor at this group size");
        *kind = FFAI_LINEAR_AFFINE;
        *in_dim = s->shape[1] * gs;
        lin->scales = reinterpret_cast<const uint16_t*>(h->f->data + s->begin);
        lin->biases = reinterpret_cast<const uint16_t*>(h->f->data + b->begin);
    } else return st_fail(h, base + ".weight has an unsupported dtype " + w->dtype);
    if (const ffai::st::Tensor* bias = ffai::st::find(h->f, base + ".bias"))
        if (bias->dtype == "BF16" && bias->end - bias->begin == (uint64_t)w->shape[0] * 2 &&
            !(reinterpret_cast<uintptr_t>(h->f->data + bias->begin) & 1u))
            lin->bias = reinterpret_cast<const uint16_t*>(h->f->data + bias->begin);
    return FFAI_OK;
}
}  // namespace

extern "C" FFAI_API int ffai_st_moe_weights(ffai_st_file* h, const char* prefix, int32_t scheme, ffai_moe_config* cfg,
                                            ffai_moe_weights* out) {
    if (!h || !h->f || !prefix || !cfg || !out) return FFAI_ERR_INVALID_ARG;
    if (scheme != FFAI_ST_SWITCH_MLP && scheme != FFAI_ST_SWITCH_GLU) return st_fail(h, "unknown naming scheme");
    const std::string p = prefix;
    const std::string ex = p + (scheme == FFAI_ST_SWITCH_MLP ? ".switch_mlp" : ".experts.switch_glu");
    const std::string router = p + (scheme == FFAI_ST_SWITCH_MLP ? ".gate" : ".router.proj");
    if (!valid_gs(cfg->expert_group_size)) return st_fail(h, "config.expert_group_size must be 32, 64 or 128");
    *out = ffai_moe_weights{};
    out->struct_size = sizeof(ffai_moe_weights);
    out->location = FFAI_MEM_HOST;
    int rc, bits[3];
    int64_t n[3], od[3], id[3];
    if ((rc = st_qproj(h, ex + ".gate_proj", cfg->expert_group_size, &out->gate_proj, &n[0], &od[0], &id[0], &bits[0]))) return rc;
    if ((rc = st_qproj(h, ex + ".up_proj", cfg->expert_group_size, &out->up_proj, &n[1], &od[1], &id[1], &bits[1]))) return rc;
    if ((rc = st_qproj(h, ex + ".down_proj", cfg->expert_group_size, &out->down_proj, &n[2], &od[2], &id[2], &bits[2]))) return rc;
    if (n[0] != n[1] || n[0] != n[2] || od[0] != od[1] || id[0] != id[1] || od[2] != id[0] || id[2] != od[0])
        return st_fail(h, "gate/up/down shapes are inconsistent");
    if (bits[0] != bits[1] || bits[0] != bits[2]) return st_fail(h, "gate/up/down use different bit widths (not supported in one block)");
    cfg->n_experts = (int32_t)n[0];
    cfg->intermediate = (int32_t)od[0];
    cfg->hidden = (int32_t)id[0];
    cfg->expert_bits = bits[0];
    int64_t ro, ri;
    const int rgs = cfg->router_group_size ? cfg->router_group_size : cfg->expert_group_size;
    if ((rc = st_linear(h, router, rgs, &out->router, &cfg->router_kind, &cfg->router_bits, &ro, &ri))) return rc;
    if (ro != n[0] || ri != id[0]) return st_fail(h, "router shape does not match the experts");
    cfg->router_group_size = cfg->router_kind == FFAI_LINEAR_AFFINE ? rgs : 0;
    cfg->router_has_bias = out->router.bias != nullptr;
    if (const ffai::st::Tensor* t = ffai::st::find(h->f, p + ".router.per_expert_scale"))
        if (t->dtype == "F32" && t->end - t->begin == (uint64_t)n[0] * 4)
            out->router_per_expert_scale = reinterpret_cast<const float*>(h->f->data + t->begin);
    // optional shared expert (Qwen3xText.swift:626-650): <prefix>.shared_expert.* and <prefix>.shared_expert_gate
    cfg->shared_intermediate = 0;
    if (ffai::st::find(h->f, p + ".shared_expert.gate_proj.weight")) {
        const int sgs = cfg->shared_group_size ? cfg->shared_group_size : cfg->expert_group_size;
        int sb[3];
        int64_t sn[3], so[3], si[3];
        if ((rc = st_qproj(h, p + ".shared_expert.gate_proj", sgs, &out->shared_gate_proj, &sn[0], &so[0], &si[0], &sb[0]))) return rc;
        if ((rc = st_qproj(h, p + ".shared_expert.up_proj", sgs, &out->shared_up_proj, &sn[1], &so[1], &si[1], &sb[1]))) return rc;
        if ((rc = st_qproj(h, p + ".shared_expert.down_proj", sgs, &out->shared_down_proj, &sn[2], &so[2], &si[2], &sb[2]))) return rc;
        if (si[0] != id[0] || so[2] != id[0] || so[0] != so[1] || si[2] != so[0] || sb[0] != sb[1] || sb[0] != sb[2])
            return st_fail(h, "shared expert shapes are inconsistent");
        cfg->shared_intermediate = (int32_t)so[0];
        cfg->shared_bits = sb[0];
        cfg->shared_group_size = sgs;
        cfg->shared_gate_kind = FFAI_LINEAR_NONE;
        if (ffai::st::find(h->f, p + ".shared_expert_gate.weight")) {
            int64_t go, gi;
            const int ggs = cfg->shared_gate_group_size ? cfg->shared_gate_group_size : sgs;
            if ((rc = st_linear(h, p + ".shared_expert_gate", ggs, &out->shared_gate, &cfg->shared_gate_kind, &cfg->shared_gate_bits, &go, &gi))) return rc;
            if (go != 1 || gi != id[0]) return st_fail(h, "shared_expert_gate must be [1, hidden]");
            cfg->shared_gate_group_size = cfg->shared_gate_kind == FFAI_LINEAR_AFFINE ? ggs : 0;
        }
    }
    return FFAI_OK;
}

// ───────────────────────────── operator-level entry points ─────────────────────────────

namespace {
int op_check_quant(int bits, int gs, int in_dim) {
    if (!valid_bits(bits) || !valid_gs(gs)) return FFAI_ERR_INVALID_ARG;
    if (in_dim <= 0 || in_dim % 32 || in_dim % gs) return FFAI_ERR_INVALID_ARG;  // Ops.swift:4610-4615
    return FFAI_OK;
}
int need_device() { return ffai_cuda_device_count() > 0 ? FFAI_OK : FFAI_ERR_CUDA; }
}  // namespace

extern "C" FFAI_API int ffai_op_dequant_gemv(const uint16_t* x, const uint32_t* weight, const uint16_t* scales,
                                    const uint16_t* biases, uint16_t* out, int32_t out_dim,
                                    int32_t in_dim, int32_t bits, int32_t gs, void* stream) {
    if (!x || !weight || !scales || !biases || !out || out_dim <= 0) return FFAI_ERR_INVALID_ARG;
    int rc = op_check_quant(bits, gs, in_dim);
    if (rc) return rc;
    if ((rc = need_device())) return rc;
    ffai_qproj q{weight, scales, biases, nullptr};
    GemvParams p = gemv_params(q, nullptr, out_dim, in_dim, gs, 1);
    p.n_rows = 1;
    return launch_grouped_gemv<uint16_t, uint16_t, false>(p, bits, x, out, 1, (cudaStream_t)stream);
}

extern "C" FFAI_API int ffai_op_dequant_gemv_expert_indexed(const uint16_t* x, const uint32_t* weight,
                                                   const uint16_t* scales, const uint16_t* biases,
                                                   const uint32_t* expert_index, uint16_t* out,
                                                   int32_t n_experts, int32_t out_dim, int32_t in_dim,
                                                   int32_t bits, int32_t gs, void* stream) {
    if (!x || !weight || !scales || !biases || !out || !expert_index || out_dim <= 0 || n_experts <= 0)
        return FFAI_ERR_INVALID_ARG;
    int rc = op_check_quant(bits, gs, in_dim);
    if (rc) return rc;
    if ((rc = need_device())) return rc;
    ffai_qproj q{weight, scales, biases, nullptr};
    GemvParams p = gemv_params(q, nullptr, out_dim, in_dim, gs, n_experts);
    p.n_rows = 1;
    p.expert_index = expert_index;
    return launch_grouped_gemv<uint16_t, uint16_t, false>(p, bits, x, out, 1, (cudaStream_t)stream);
}

extern "C" FFAI_API int ffai_op_moe_router_topk(const float* logits, uint32_t* indices, float* weights,
                                       int32_t T, int32_t E, int32_t k, int32_t gating_mode,
                                       int32_t norm, const float* expert_bias, void* stream) {
    if (!logits || !indices || !weights || T <= 0) return FFAI_ERR_INVALID_ARG;
    if (E <= 0 || E > FFAI_MAX_EXPERTS || k <= 0 || k > E || k > FFAI_MAX_TOP_K) return FFAI_ERR_INVALID_ARG;
    if (gating_mode < 0 || gating_mode > FFAI_GATING_SIGMOID_TOPK) return FFAI_ERR_INVALID_ARG;
    int rc;
    if ((rc = need_device())) return rc;
    RouterParams p{};
    p.n_experts = E; p.top_k = k; p.gating_mode = gating_mode; p.norm_topk_prob = norm;
    p.routed_scaling = 1.0f;
    p.expert_bias = expert_bias;
    const int warps = 4;
    route_only_kernel<<<(T + warps - 1) / warps, warps * 32, (size_t)warps * 2 * E * sizeof(float),
                        (cudaStream_t)stream>>>(p, logits, T, indices, weights);
    return cudaGetLastError() == cudaSuccess ? FFAI_OK : FFAI_ERR_CUDA;
}

extern "C" FFAI_API size_t ffai_op_moe_plan_workspace_bytes(int32_t n_rows, int32_t n_experts) {
    if (n_rows <= 0 || n_experts <= 0) return 0;
    return (size_t)plan_num_blocks(n_rows) * n_experts * sizeof(uint32_t);
}

extern "C" FFAI_API int ffai_op_moe_plan(const uint32_t* indices, int32_t T, int32_t k, int32_t E,
                                uint32_t* counts, uint32_t* offsets, uint32_t* perm,
                                uint32_t* inv_perm, void* workspace, void* stream) {
    if (!indices || !counts || !offsets || !perm || !inv_perm || T <= 0 || k <= 0) return FFAI_ERR_INVALID_ARG;
    if (E <= 0 || E > FFAI_MAX_EXPERTS) return FFAI_ERR_INVALID_ARG;
    if ((int64_t)T * k > PLAN_ENTRIES_PER_WARP && !workspace) return FFAI_ERR_INVALID_ARG;
    int rc;
    if ((rc = need_device())) return rc;
    return launch_plan(indices, T * k, E, counts, offsets, perm, inv_perm, (uint32_t*)workspace,
                       (cudaStream_t)stream) < 0 ? FFAI_ERR_CUDA : FFAI_OK;
}

// ── plan without allocation ──
// Per-block histograms of the three-pass plan, resident in the library's device image.  In host
// code this name is only a handle for cudaGetSymbolAddress; kernels get the looked-up address.
static __device__ __align__(256) uint32_t g_plan_static_hist[(FFAI_PLAN_STATIC_MAX_ROWS / PLAN_ENTRIES_PER_WARP) * FFAI_MAX_EXPERTS];

namespace {
constexpr int kMaxDevices = 64;
uint32_t* g_plan_static_ptr[kMaxDevices] = {};
std::mutex g_plan_static_mutex;

// Address of the array on the current device, looked up once per device.
int plan_static_scratch(uint32_t** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return FFAI_ERR_CUDA;
    std::lock_guard<std::mutex> lock(g_plan_static_mutex);
    if (!g_plan_static_ptr[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_plan_static_hist) != cudaSuccess || !p) {
            cudaGetLastError();
            return FFAI_ERR_CUDA;
        }
        g_plan_static_ptr[dev] = static_cast<uint32_t*>(p);
    }
    *out = g_plan_static_ptr[dev];
    return FFAI_OK;
}
}  // namespace

extern "C" FFAI_API int ffai_op_moe_plan_static(const uint32_t* indices, int32_t T, int32_t k, int32_t E,
                                                uint32_t* counts, uint32_t* offsets, uint32_t* perm,
                                                uint32_t* inv_perm, void* stream) {
    if (!indices || !counts || !offsets || !perm || !inv_perm || T <= 0 || k <= 0) return FFAI_ERR_INVALID_ARG;
    if (E <= 0 || E > FFAI_MAX_EXPERTS) return FFAI_ERR_INVALID_ARG;
    if ((int64_t)T * k > FFAI_PLAN_STATIC_MAX_ROWS) return FFAI_ERR_INVALID_ARG;
    int rc;
    if ((rc = need_device())) return rc;
    uint32_t* scratch = nullptr;
    if ((rc = plan_static_scratch(&scratch))) return rc;
    return launch_plan(indices, T * k, E, counts, offsets, perm, inv_perm, scratch, (cudaStream_t)stream) < 0
               ? FFAI_ERR_CUDA : FFAI_OK;
}

extern "C" FFAI_API int ffai_op_gather_rows(const uint16_t* table, const uint32_t* ids, uint16_t* out,
                                   int32_t n_rows, int32_t row_len, void* stream) {
    if (!table || !ids || !out || n_rows <= 0 || row_len <= 0 || row_len % 8) return FFAI_ERR_INVALID_ARG;
    int rc;
    if ((rc = need_device())) return rc;
    gather_rows_kernel<<<(n_rows + 3) / 4, 128, 0, (cudaStream_t)stream>>>(table, ids, 1, out, n_rows, row_len);
    return cudaGetLastError() == cudaSuccess ? FFAI_OK : FFAI_ERR_CUDA;
}

extern "C" FFAI_API int ffai_op_moe_gather_dequant_gemm(const uint16_t* x, const uint32_t* weight,
                                               const uint16_t* scales, const uint16_t* biases,
                                               const uint32_t* indices, uint16_t* out, int32_t m_total,
                                               int32_t n_out, int32_t k_in, int32_t n_experts,
                                               int32_t bits, int32_t gs, void* stream) {
    if (!x || !weight || !scales || !biases || !indices || !out) return FFAI_ERR_INVALID_ARG;
    if (m_total <= 0 || n_out <= 0 || n_experts <= 0 || n_experts > FFAI_MAX_EXPERTS) return FFAI_ERR_INVALID_ARG;
    int rc = op_check_quant(bits, gs, k_in);
    if (rc) return rc;
    if ((rc = need_device())) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    uint32_t* offsets = nullptr;
    if (cudaMallocAsync((void**)&offsets, (size_t)(n_experts + 1) * 4, st) != cudaSuccess) return FFAI_ERR_CUDA;
    offsets_from_sorted_ids_kernel<<<(n_experts + 1 + 127) / 128, 128, 0, st>>>(indices, m_total, n_experts, offsets);
    ffai_qproj q{weight, scales, biases, nullptr};
    GemvParams p = gemv_params(q, nullptr, n_out, k_in, gs, n_experts);
    p.offsets = offsets;
    p.n_rows = m_total;
    rc = launch_grouped_gemv<uint16_t, uint16_t, false>(p, bits, x, out, n_experts, st);
    cudaFreeAsync(offsets, st);
    return rc;
}

extern "C" FFAI_API int ffai_op_glu_activation(const uint16_t* gate, const uint16_t* up, uint16_t* out,
                                      int64_t n, int32_t activation, float limit, float alpha,
                                      void* stream) {
    if (!gate || !up || !out || n <= 0 || activation < 0 || activation > FFAI_ACT_GELU_GLU) return FFAI_ERR_INVALID_ARG;
    int rc;
    if ((rc = need_device())) return rc;
    glu_activation_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(gate, up, out, n, activation, limit, alpha);
    return cudaGetLastError() == cudaSuccess ? FFAI_OK : FFAI_ERR_CUDA;
}

extern "C" FFAI_API int ffai_op_moe_unpermute(const uint16_t* expert_out, const uint32_t* inv_perm,
                                     const float* weights, uint16_t* out, int32_t T, int32_t hidden,
                                     int32_t k, void* stream) {
    if (!expert_out || !inv_perm || !weights || !out || T <= 0 || hidden <= 0 || hidden % 4) return FFAI_ERR_INVALID_ARG;
    if (k <= 0 || k > FFAI_MAX_TOP_K) return FFAI_ERR_INVALID_ARG;
    int rc;
    if ((rc = need_device())) return rc;
    combine_kernel<uint16_t, float><<<T, 256, 0, (cudaStream_t)stream>>>(expert_out, inv_perm, weights, k, nullptr, nullptr, nullptr, out, hidden);
    return cudaGetLastError() == cudaSuccess ? FFAI_OK : FFAI_ERR_CUDA;
}

extern "C" FFAI_API int ffai_op_add_rmsnorm(const uint16_t* a, const uint16_t* b, const uint16_t* weight, float eps,
                                            int32_t n_rows, int32_t n, uint16_t* residual_out, uint16_t* normed_out, void* stream) {
    if (!a || !weight || !normed_out || n_rows <= 0 || n <= 0 || n % 4) return FFAI_ERR_INVALID_ARG;
    if (b && !residual_out) return FFAI_ERR_INVALID_ARG;   // the sum is the caller's next residual: it must have a home
    if (!aligned16(a) || (b && !aligned16(b)) || (residual_out && !aligned16(residual_out)) || !aligned16(normed_out) || (n % 8))
        return FFAI_ERR_INVALID_ARG;
    int rc;
    if ((rc = need_device())) return rc;
    prep::add_rmsnorm_kernel<<<n_rows, 256, 0, (cudaStream_t)stream>>>(a, b, weight, eps, n, residual_out, normed_out);
    return cudaGetLastError() == cudaSuccess ? FFAI_OK : FFAI_ERR_CUDA;
}

extern "C" FFAI_API int ffai_op_mxfp4_to_affine_int4(const uint32_t* packed, const uint8_t* e8m0, int64_t n_groups,
                                                     uint32_t* out_weight, uint16_t* out_scales, uint16_t* out_biases,
                                                     void* stream) {
    if (!packed || !e8m0 || !out_weight || !out_scales || !out_biases || n_groups <= 0) return FFAI_ERR_INVALID_ARG;
    if (!aligned16(packed) || !aligned16(out_weight)) return FFAI_ERR_INVALID_ARG;
    int rc;
    if ((rc = need_device())) return rc;
    const unsigned blocks = (unsigned)((n_groups + 255) / 256);
    prep::mxfp4_to_affine4_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const uint4*>(packed), e8m0, (long)n_groups, reinterpret_cast<uint4*>(out_weight), out_scales, out_biases);
    return cudaGetLastError() == cudaSuccess ? FFAI_OK : FFAI_ERR_CUDA;
}

extern "C" FFAI_API int ffai_op_affine_quantize(const uint16_t* w, int64_t rows, int32_t in_dim, int32_t bits, int32_t gs,
                                                uint32_t* out_weight, uint16_t* out_scales, uint16_t* out_biases, void* stream) {
    if (!w || !out_weight || !out_scales || !out_biases || rows <= 0) return FFAI_ERR_INVALID_ARG;
    int rc = op_check_quant(bits, gs, in_dim);
    if (rc) return rc;
    if ((rc = need_device())) return rc;
    const long n_groups = (long)rows * (in_dim / gs);
    const unsigned blocks = (unsigned)((n_groups + 127) / 128);
    cudaStream_t st = (cudaStream_t)stream;
    switch (bits) {
        case 2: prep::affine_quantize_kernel<2><<<blocks, 128, 0, st>>>(w, n_groups, gs, out_weight, out_scales, out_biases); break;
        case 3: prep::affine_quantize_kernel<3><<<blocks, 128, 0, st>>>(w, n_groups, gs, out_weight, out_scales, out_biases); break;
        case 4: prep::affine_quantize_kernel<4><<<blocks, 128, 0, st>>>(w, n_groups, gs, out_weight, out_scales, out_biases); break;
        case 5: prep::affine_quantize_kernel<5><<<blocks, 128, 0, st>>>(w, n_groups, gs, out_weight, out_scales, out_biases); break;
        case 6: prep::affine_quantize_kernel<6><<<blocks, 128, 0, st>>>(w, n_groups, gs, out_weight, out_scales, out_biases); break;
        case 8: prep::affine_quantize_kernel<8><<<blocks, 128, 0, st>>>(w, n_groups, gs, out_weight, out_scales, out_biases); break;
        default: return FFAI_ERR_INVALID_ARG;
    }
    return cudaGetLastError() == cudaSuccess ? FFAI_OK : FFAI_ERR_CUDA;
}

extern "C" FFAI_API int ffai_op_sigmoid_scalar_fma(const uint16_t* gate, const uint16_t* value,
                                          const uint16_t* base, const uint16_t* residual,
                                          uint16_t* out, int32_t n_rows, int32_t hidden, void* stream) {
    if (!gate || !value || !base || !out || n_rows <= 0 || hidden <= 0) return FFAI_ERR_INVALID_ARG;
    int rc;
    if ((rc = need_device())) return rc;
    sigmoid_scalar_fma_kernel<<<n_rows, 256, 0, (cudaStream_t)stream>>>(gate, value, base, residual, out, hidden);
    return cudaGetLastError() == cudaSuccess ? FFAI_OK : FFAI_ERR_CUDA;
}
