// Router: projection + bias + top-k + softmax/renormalise, fused in one kernel.
//
// Replaces, per token: the router GEMV (FFAI Layers.swift:78-84 / :201-210,
// GPTOSSText.swift:341-362), the device->host sync and MoERouter.route
// (MoELayer.swift:140-296) or GPTOSSMoELayer's sort (GPTOSSText.swift:1346-1361),
// and Ops.moeRouterTopKMany (Ops.swift:2598-2661).
//
// Accumulation order of a logit is fixed so that top-k is reproducible to the
// bit: the hidden axis is cut into 64-wide chunks; inside a chunk products are
// folded in ascending k with fused multiply-add starting from 0; chunk sums are
// then added in ascending chunk order.  Top-k orders by (value desc, index asc).
#pragma once
#include "common.cuh"
#include "plan.cuh"

namespace ffai {

struct RouterParams {
    const void* weight;        // f32 / bf16 [E,H] or u32 [E, H*bits/32]
    const uint16_t* scales;    // affine only
    const uint16_t* biases;    // affine only
    const uint16_t* bias;      // nullable projection bias [E], bf16
    const float* expert_bias;  // nullable post-softmax bias [E]
    int kind;                  // ffai_linear_kind: 1 f32, 2 bf16, 3 affine
    int bits, group_size;
    int hidden, n_experts, top_k;
    int gating_mode, norm_topk_prob;
    int logits_bf16;
    float logit_scale;               // logits are multiplied by this before routing (1 unless the model says otherwise)
    const float* per_expert_scale;   // nullable [E]: combine weight *= scale[expert]
    float routed_scaling;            // sigmoid routing: factor on the combine weights (1 unless the model says otherwise)
};

// One 64-wide chunk of dot(x[t], W[e]) in ascending k with fused multiply-add.
template <int KIND, int BITS>
FFAI_DEVINL float router_chunk_dot(const RouterParams& p, const uint16_t* __restrict__ xrow, int e,
                                   int k0, int k1) {
    float acc = 0.0f;
    const int H = p.hidden;
    if (KIND == 1) {
        const float* w = (const float*)p.weight + (size_t)e * H;
        if (k1 - k0 == 64) {
            // all loads of the chunk first, then the dependent chain: one memory latency per chunk, not eight
            uint4 xv[8];
            float4 wv[16];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                xv[j] = *(const uint4*)(xrow + k0 + 8 * j);
                wv[2 * j] = *(const float4*)(w + k0 + 8 * j);
                wv[2 * j + 1] = *(const float4*)(w + k0 + 8 * j + 4);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float4 w0 = wv[2 * j], w1 = wv[2 * j + 1];
                acc = __fmaf_rn(bf16lo(xv[j].x), w0.x, acc); acc = __fmaf_rn(bf16hi(xv[j].x), w0.y, acc);
                acc = __fmaf_rn(bf16lo(xv[j].y), w0.z, acc); acc = __fmaf_rn(bf16hi(xv[j].y), w0.w, acc);
                acc = __fmaf_rn(bf16lo(xv[j].z), w1.x, acc); acc = __fmaf_rn(bf16hi(xv[j].z), w1.y, acc);
                acc = __fmaf_rn(bf16lo(xv[j].w), w1.z, acc); acc = __fmaf_rn(bf16hi(xv[j].w), w1.w, acc);
            }
        } else {
            for (int k = k0; k < k1; ++k) acc = __fmaf_rn(bf16_bits_to_f32(xrow[k]), w[k], acc);
        }
    } else if (KIND == 2) {
        const uint16_t* w = (const uint16_t*)p.weight + (size_t)e * H;
        if (k1 - k0 == 64) {
            uint4 xv[8], wv[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                xv[j] = *(const uint4*)(xrow + k0 + 8 * j);
                wv[j] = *(const uint4*)(w + k0 + 8 * j);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                acc = __fmaf_rn(bf16lo(xv[j].x), bf16lo(wv[j].x), acc); acc = __fmaf_rn(bf16hi(xv[j].x), bf16hi(wv[j].x), acc);
                acc = __fmaf_rn(bf16lo(xv[j].y), bf16lo(wv[j].y), acc); acc = __fmaf_rn(bf16hi(xv[j].y), bf16hi(wv[j].y), acc);
                acc = __fmaf_rn(bf16lo(xv[j].z), bf16lo(wv[j].z), acc); acc = __fmaf_rn(bf16hi(xv[j].z), bf16hi(wv[j].z), acc);
                acc = __fmaf_rn(bf16lo(xv[j].w), bf16lo(wv[j].w), acc); acc = __fmaf_rn(bf16hi(xv[j].w), bf16hi(wv[j].w), acc);
            }
        } else {
            for (int k = k0; k < k1; ++k)
                acc = __fmaf_rn(bf16_bits_to_f32(xrow[k]), bf16_bits_to_f32(w[k]), acc);
        }
    } else {
        // affine: w = fma(scale, q, bias), one scale/bias per group_size values
        const uint32_t* w = (const uint32_t*)p.weight + (size_t)e * (H * BITS / 32);
        const int gpr = H / p.group_size;
        for (int k = k0; k < k1; k += 32) {  // H is a multiple of 32; a 32-run lies in one group
            const int g = k / p.group_size;
            const float s = bf16_bits_to_f32(p.scales[(size_t)e * gpr + g]);
            const float b = bf16_bits_to_f32(p.biases[(size_t)e * gpr + g]);
            uint32_t words[BITS + 1];
            const uint32_t* src = w + (k / 32) * BITS;
#pragma unroll
            for (int i = 0; i < BITS; ++i) words[i] = src[i];
            words[BITS] = 0;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                float q = small_uint_to_float(unpack_at<BITS>(words, j));
                float wv = __fmaf_rn(s, q, b);
                acc = __fmaf_rn(bf16_bits_to_f32(xrow[k + j]), wv, acc);
            }
        }
    }
    return acc;
}

// Warp-wide arg-best by (value desc, index asc).
FFAI_DEVINL void warp_argbest(float& v, int& i) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
        float ov = __shfl_xor_sync(0xFFFFFFFFu, v, m);
        int oi = __shfl_xor_sync(0xFFFFFFFFu, i, m);
        bool take = (oi >= 0) && (i < 0 || ov > v || (ov == v && oi < i));
        if (take) { v = ov; i = oi; }
    }
}

// Top-k of vals[0..E) in shared memory by one warp; selected indices (in
// selection order) returned lane-wise: lane j < k holds index j.  `taken` is a
// per-lane bit mask over the lane's strided elements (e = lane + 32*j).
FFAI_DEVINL void warp_topk(const float* vals, int E, int k, int lane, int& my_idx, float& my_val) {
    uint32_t taken = 0;
    my_idx = -1;
    my_val = 0.0f;
    for (int r = 0; r < k; ++r) {
        float bv = 0.0f;
        int bi = -1;
        for (int j = 0, e = lane; e < E; ++j, e += 32) {
            if (taken & (1u << j)) continue;
            float v = vals[e];
            if (bi < 0 || v > bv) { bv = v; bi = e; }
        }
        warp_argbest(bv, bi);
        if (bi >= 0 && (bi & 31) == lane) taken |= 1u << (bi >> 5);
        if (lane == r) { my_idx = bi; my_val = bv; }
    }
}

// Routing of one token by one warp, given its logits in shared memory.
// `scratch` is E floats of shared memory (used by the general softmax path).
FFAI_DEVINL void route_token_warp(const RouterParams& p, float* logits_s, float* scratch, int lane,
                                  uint32_t* idx_out, float* w_out) {
    const int E = p.n_experts, K = p.top_k;
    int my_idx;
    float my_val;
    if (p.logit_scale != 1.0f && p.logit_scale != 0.0f) {   // (0: unset) Gemma 4: hidden^-0.5 folded into the logits (Gemma4Text.swift:937-943)
        for (int e = lane; e < E; e += 32) logits_s[e] = __fmul_rn(logits_s[e], p.logit_scale);
        __syncwarp();
    }
    if (p.gating_mode == 2) {
        // NemotronH routing (NemotronHText.swift:844-867): sigmoid scores; selection on score + bias; weights are the
        // raw sigmoids of the selected, over (their sum + 1e-20) when k > 1 and renormalising, times the scaling factor
        for (int e = lane; e < E; e += 32) {
            const float sg = __fdiv_rn(1.0f, __fadd_rn(1.0f, det_expf(-logits_s[e])));
            logits_s[e] = sg;
            scratch[e] = p.expert_bias ? __fadd_rn(sg, p.expert_bias[e]) : sg;
        }
        __syncwarp();
        warp_topk(scratch, E, K, lane, my_idx, my_val);
        float w = (lane < K) ? logits_s[my_idx] : 0.0f;
        if (K > 1 && p.norm_topk_prob) {
            float sum = 0.0f;
            for (int j = 0; j < K; ++j) sum = __fadd_rn(sum, __shfl_sync(0xFFFFFFFFu, w, j));
            sum = __fadd_rn(sum, 1e-20f);
            w = __fdiv_rn(w, sum);
        }
        w = __fmul_rn(w, p.routed_scaling);
        if (p.per_expert_scale && lane < K) w = __fmul_rn(w, p.per_expert_scale[my_idx]);
        if (lane < K) { idx_out[lane] = (uint32_t)my_idx; w_out[lane] = w; }
        return;
    }
    const bool fast = (p.gating_mode == 1) ||
                      (p.gating_mode == 0 && p.norm_topk_prob && p.expert_bias == nullptr);
    if (fast) {
        // top-k of the logits, softmax over the picked (MoELayer.swift:146-172, 197-203)
        warp_topk(logits_s, E, K, lane, my_idx, my_val);
        float vmax = __shfl_sync(0xFFFFFFFFu, my_val, 0);  // selection order is value-desc
        float ex = (lane < K) ? det_expf(__fsub_rn(my_val, vmax)) : 0.0f;
        float sum = 0.0f;
        for (int j = 0; j < K; ++j) sum = __fadd_rn(sum, __shfl_sync(0xFFFFFFFFu, ex, j));
        float w = (sum > 0.0f) ? __fdiv_rn(ex, sum) : __fdiv_rn(1.0f, (float)K);
        if (p.per_expert_scale && lane < K) w = __fmul_rn(w, p.per_expert_scale[my_idx]);
        if (lane < K) { idx_out[lane] = (uint32_t)my_idx; w_out[lane] = w; }
        return;
    }
    // general softmax-then-top-k (MoELayer.swift:174-195)
    float vmax = -INFINITY;
    for (int e = lane; e < E; e += 32) vmax = fmaxf(vmax, logits_s[e]);
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) vmax = fmaxf(vmax, __shfl_xor_sync(0xFFFFFFFFu, vmax, m));
    for (int e = lane; e < E; e += 32) scratch[e] = det_expf(__fsub_rn(logits_s[e], vmax));
    __syncwarp();
    float sum = 0.0f;
    for (int e = 0; e < E; ++e) sum = __fadd_rn(sum, scratch[e]);  // ascending order, every lane
    const bool degenerate = !(sum > 0.0f);
    for (int e = lane; e < E; e += 32) {
        float g = degenerate ? __fdiv_rn(1.0f, (float)E) : __fdiv_rn(scratch[e], sum);
        if (p.expert_bias) g = __fadd_rn(g, p.expert_bias[e]);
        scratch[e] = g;
    }
    __syncwarp();
    warp_topk(scratch, E, K, lane, my_idx, my_val);
    float w = my_val;
    if (p.norm_topk_prob) {
        float s2 = 0.0f;
        for (int j = 0; j < K; ++j) s2 = __fadd_rn(s2, __shfl_sync(0xFFFFFFFFu, my_val, j));
        if (s2 > 0.0f) w = __fdiv_rn(my_val, s2);
    }
    if (p.per_expert_scale && lane < K) w = __fmul_rn(w, p.per_expert_scale[my_idx]);
    if (lane < K) { idx_out[lane] = (uint32_t)my_idx; w_out[lane] = w; }
}

// One block per token.  Threads walk (expert, chunk) pairs; chunk sums land in
// shared memory; one thread per expert adds them in ascending chunk order; warp 0
// routes.  Dynamic shared memory: E*nchunks + 2*E floats.
template <int KIND, int BITS>
__global__ void __launch_bounds__(512)
router_token_kernel(RouterParams p, const uint16_t* __restrict__ x, int n_tokens,
                    uint32_t* __restrict__ indices, float* __restrict__ weights,
                    float* __restrict__ logits_out) {
    extern __shared__ float smem[];
    const int H = p.hidden, E = p.n_experts;
    const int nchunks = (H + 63) / 64;
    float* partial = smem;                 // [E][nchunks]
    float* logits_s = smem + E * nchunks;  // [E]
    float* scratch = logits_s + E;         // [E]
    const int t = blockIdx.x;
    if (t >= n_tokens) return;
    const uint16_t* xrow = x + (size_t)t * H;
    const int total = E * nchunks;
    for (int i = threadIdx.x; i < total; i += blockDim.x) {
        const int e = i / nchunks, c = i - e * nchunks;
        const int k0 = c * 64, k1 = min(k0 + 64, H);
        partial[i] = router_chunk_dot<KIND, BITS>(p, xrow, e, k0, k1);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        float total_e = 0.0f;
        for (int c = 0; c < nchunks; ++c) total_e = __fadd_rn(total_e, partial[e * nchunks + c]);
        if (p.logits_bf16) total_e = bf16_round(total_e);
        if (p.bias) {
            total_e = __fadd_rn(total_e, bf16_bits_to_f32(p.bias[e]));
            if (p.logits_bf16) total_e = bf16_round(total_e);
        }
        logits_s[e] = total_e;
        if (logits_out) logits_out[(size_t)t * E + e] = total_e;
    }
    __syncthreads();
    if (threadIdx.x < 32)
        route_token_warp(p, logits_s, scratch, threadIdx.x, indices + (size_t)t * p.top_k,
                         weights + (size_t)t * p.top_k);
}

// Small-batch router for dense (fp32 / bf16) weights: grid (ceil(E / ROWS), T), 256 threads.
// A block stages ROWS weight rows and the token's activation row in shared memory with coalesced
// 16-byte asynchronous copies (the per-(expert, chunk) work items of router_token_kernel made every
// lane touch its own 128-byte line: tag-lookup bound on one SM), then each thread folds one
// (expert, chunk) pair from shared memory in the fixed order, one thread per expert adds the chunk
// sums, and the last block to finish a token (a ticket counter that resets itself) routes it.
// With a destination for it, block 0 of a token also writes the token's row in the order the 4-bit
// expert kernels read (every 8-run as 0,4,1,5,2,6,3,7) and the fp32 sum of every 32-run, from the
// copy it staged anyway.
// With a plan destination, the block that routes the last token of the batch (a second ticket, in
// the last slot of the ticket array) also builds the dispatch plan, which saves a launch per step.
// Shared-memory rows are stored with the 16-byte pieces of each 64-value line XOR-swizzled by the
// line index, so threads that read consecutive lines hit distinct banks.
constexpr int ROUTER_ROWS = 8;                // most weight rows a block stages (fewer when the batch is tiny, so that the grid still covers the SMs)
constexpr int ROUTER_TICKETS = 96;             // per-token tickets; the last slot counts routed tokens of the batch
constexpr int ROUTER_BATCH_TICKET = ROUTER_TICKETS - 1;

template <int KIND>  // 1: fp32 weights, 2: bf16 weights
__global__ void __launch_bounds__(256)
router_rows_kernel(RouterParams p, const uint16_t* __restrict__ x, int n_tokens,
                   uint32_t* __restrict__ indices, float* __restrict__ weights,
                   float* __restrict__ logits_out, uint32_t* __restrict__ tickets, PlanOut plan,
                   uint16_t* __restrict__ x_perm8, float* __restrict__ x_sum64, int sum_pitch, int rows_per_block) {
    constexpr int WBYTES = KIND == 1 ? 4 : 2;
    constexpr int LINE16 = 64 * WBYTES / 16;   // 16-byte pieces per 64-value line of a weight row
    extern __shared__ __align__(16) uint8_t rsm[];
    const int H = p.hidden, E = p.n_experts;
    const int nchunks = H / 64;
    const int t = blockIdx.y;
    const int e0 = blockIdx.x * rows_per_block;
    const int rows = min(rows_per_block, E - e0);
    uint8_t* wsm = rsm;                                          // [ROWS][H * WBYTES]
    uint8_t* xsm = wsm + (size_t)rows_per_block * H * WBYTES;    // [H * 2]
    float* partial = reinterpret_cast<float*>(xsm + (size_t)H * 2);  // [ROWS][nchunks]
    float* lsm = partial + rows_per_block * nchunks;             // [2 * E] (routing, last block only)
    __shared__ uint32_t ticket_s;
    const uint32_t wsm_u = (uint32_t)__cvta_generic_to_shared(wsm), xsm_u = (uint32_t)__cvta_generic_to_shared(xsm);

    // stage: weight rows (rows * nchunks * LINE16 pieces) and the activation row (nchunks * 8 pieces)
    const uint8_t* wsrc = reinterpret_cast<const uint8_t*>(p.weight) + (size_t)e0 * H * WBYTES;
    const int wpieces = rows * nchunks * LINE16;
    for (int i = threadIdx.x; i < wpieces; i += blockDim.x) {
        const int line = i / LINE16, j = i - line * LINE16;      // line = row * nchunks + chunk
        const uint32_t dst = wsm_u + (uint32_t)(line * LINE16 + (j ^ (line & 7))) * 16;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(wsrc + (size_t)i * 16) : "memory");
    }
    const uint8_t* xsrc = reinterpret_cast<const uint8_t*>(x + (size_t)t * H);
    for (int i = threadIdx.x; i < nchunks * 8; i += blockDim.x) {
        const int line = i >> 3, j = i & 7;
        const uint32_t dst = xsm_u + (uint32_t)(line * 8 + (j ^ (line & 7))) * 16;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(xsrc + (size_t)i * 16) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();

    if (x_perm8 && blockIdx.x == 0) {
        // 16-byte piece i of the row (8 values): permuted copy + its share of the 32-run sum; the four
        // pieces of a run sit in four consecutive lanes
        uint4* d = reinterpret_cast<uint4*>(x_perm8 + (size_t)t * H);
        for (int i0 = 0; i0 < nchunks * 8; i0 += blockDim.x) {
            const int i = i0 + threadIdx.x;
            float part = 0.0f;
            if (i < nchunks * 8) {
                const int line = i >> 3, j = i & 7;
                const uint4 v = *reinterpret_cast<const uint4*>(xsm + (size_t)(line * 8 + (j ^ (line & 7))) * 16);
                uint4 o;
                o.x = __byte_perm(v.x, v.z, 0x5410);
                o.y = __byte_perm(v.x, v.z, 0x7632);
                o.z = __byte_perm(v.y, v.w, 0x5410);
                o.w = __byte_perm(v.y, v.w, 0x7632);
                d[i] = o;
                part = ((bf16lo(v.x) + bf16hi(v.x)) + (bf16lo(v.y) + bf16hi(v.y))) +
                       ((bf16lo(v.z) + bf16hi(v.z)) + (bf16lo(v.w) + bf16hi(v.w)));
            }
            part += __shfl_xor_sync(0xFFFFFFFFu, part, 1);
            part += __shfl_xor_sync(0xFFFFFFFFu, part, 2);
            if ((threadIdx.x & 3) == 0 && i < nchunks * 8) x_sum64[(size_t)t * sum_pitch + (i >> 2)] = part;
        }
    }

    // one (row, chunk) pair per thread: 64 fused multiply-adds in ascending k
    for (int i = threadIdx.x; i < rows * nchunks; i += blockDim.x) {
        const int c = i % nchunks;
        const int line = i;                                      // row * nchunks + chunk
        float acc = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint4 xv = *reinterpret_cast<const uint4*>(xsm + (size_t)(c * 8 + (j ^ (c & 7))) * 16);
            const float xf[8] = {bf16lo(xv.x), bf16hi(xv.x), bf16lo(xv.y), bf16hi(xv.y),
                                 bf16lo(xv.z), bf16hi(xv.z), bf16lo(xv.w), bf16hi(xv.w)};
            if (KIND == 1) {
                const float4 w0 = *reinterpret_cast<const float4*>(wsm + (size_t)(line * LINE16 + ((2 * j) ^ (line & 7))) * 16);
                const float4 w1 = *reinterpret_cast<const float4*>(wsm + (size_t)(line * LINE16 + ((2 * j + 1) ^ (line & 7))) * 16);
                acc = __fmaf_rn(xf[0], w0.x, acc); acc = __fmaf_rn(xf[1], w0.y, acc);
                acc = __fmaf_rn(xf[2], w0.z, acc); acc = __fmaf_rn(xf[3], w0.w, acc);
                acc = __fmaf_rn(xf[4], w1.x, acc); acc = __fmaf_rn(xf[5], w1.y, acc);
                acc = __fmaf_rn(xf[6], w1.z, acc); acc = __fmaf_rn(xf[7], w1.w, acc);
            } else {
                const uint4 wv = *reinterpret_cast<const uint4*>(wsm + (size_t)(line * LINE16 + (j ^ (line & 7))) * 16);
                acc = __fmaf_rn(xf[0], bf16lo(wv.x), acc); acc = __fmaf_rn(xf[1], bf16hi(wv.x), acc);
                acc = __fmaf_rn(xf[2], bf16lo(wv.y), acc); acc = __fmaf_rn(xf[3], bf16hi(wv.y), acc);
                acc = __fmaf_rn(xf[4], bf16lo(wv.z), acc); acc = __fmaf_rn(xf[5], bf16hi(wv.z), acc);
                acc = __fmaf_rn(xf[6], bf16lo(wv.w), acc); acc = __fmaf_rn(xf[7], bf16hi(wv.w), acc);
            }
        }
        partial[i] = acc;
    }
    __syncthreads();
    if (threadIdx.x < rows) {
        const int e = e0 + threadIdx.x;
        float total = 0.0f;
        for (int c = 0; c < nchunks; ++c) total = __fadd_rn(total, partial[threadIdx.x * nchunks + c]);
        if (p.logits_bf16) total = bf16_round(total);
        if (p.bias) {
            total = __fadd_rn(total, bf16_bits_to_f32(p.bias[e]));
            if (p.logits_bf16) total = bf16_round(total);
        }
        logits_out[(size_t)t * E + e] = total;
    }
    // last block of this token routes it
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) ticket_s = atomicAdd(&tickets[t], 1u);
    __syncthreads();
    if (ticket_s != gridDim.x - 1) return;
    __threadfence();
    for (int e = threadIdx.x; e < E; e += blockDim.x) lsm[e] = __ldcg(logits_out + (size_t)t * E + e);
    if (threadIdx.x == 0) tickets[t] = 0;  // ready for the next call
    __syncthreads();
    if (threadIdx.x < 32) {
        route_token_warp(p, lsm, lsm + E, threadIdx.x, indices + (size_t)t * p.top_k, weights + (size_t)t * p.top_k);
        if (plan.perm) {
            __syncwarp();
            __threadfence();                       // this token's indices are visible before the batch ticket moves
            uint32_t done = 0;
            if (threadIdx.x == 0) done = atomicAdd(&tickets[ROUTER_BATCH_TICKET], 1u);
            done = __shfl_sync(0xFFFFFFFFu, done, 0);
            if (done == (uint32_t)n_tokens - 1) {  // every token of the batch is routed
                if (threadIdx.x == 0) tickets[ROUTER_BATCH_TICKET] = 0;
                __threadfence();
                uint32_t* hist = reinterpret_cast<uint32_t*>(lsm);
                plan_small_warp(indices, n_tokens * p.top_k, E, plan, hist, hist + E, threadIdx.x);
            }
        }
    }
}

// Batched router projection for many tokens: a TB-token x 64-expert tile per block (TB = 64, 32 or
// 16, chosen so the grid covers the SMs), 4x4 outputs
// per thread, the hidden axis walked one 64-wide chunk at a time.  Inside a chunk every output
// folds its products in ascending k with fused multiply-add from 0; the chunk sum is then added
// to the running total — the same order as router_token_kernel, so both give identical bits.
// Replaces the batched gate projection of MoELayer.decodeMany (FFAI MoELayer.swift:690,
// Layers.swift:101-130, 217-287).
template <int KIND, int BITS, int TB>
__global__ void __launch_bounds__(TB * 4)
router_logits_tiled_kernel(RouterParams p, const uint16_t* __restrict__ x, int n_tokens,
                           float* __restrict__ logits_out, float* __restrict__ partials) {
    constexpr int EB = 64, LD = 68, NTHR = TB * 4;  // LD: padded row length of the transposed tiles
    // Column swizzle of the transposed tiles: row r of k-line k sits at column r ^ (((k >> 3) & 7) << 2).  A warp
    // that stages 4 rows x 8 sixteen-byte pieces then writes 32 different banks (unswizzled it would hit 4), and
    // a thread's 4 consecutive rows stay one aligned float4.
    auto swz = [](int k) { return ((k >> 3) & 7) << 2; };
    __shared__ __align__(16) float xs[64 * LD];   // [k][token]
    __shared__ __align__(16) float ws[64 * LD];   // [k][expert]
    const int H = p.hidden, E = p.n_experts;
    const int t0 = blockIdx.x * TB, e0 = blockIdx.y * EB;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float total[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) total[i][j] = 0.0f;

    // partials != nullptr: blockIdx.z selects one chunk; its sums go to partials[chunk][token][expert]
    // and route_from_partials_kernel adds the chunks in ascending order (same bits, more blocks).
    const int kbeg = partials ? (int)blockIdx.z * 64 : 0;
    const int kend = partials ? kbeg + 64 : H;
    for (int k0 = kbeg; k0 < kend; k0 += 64) {
        // stage the chunk: 64x64 activations and 64x64 weights, both as fp32, transposed
        for (int i = threadIdx.x; i < TB * 8; i += NTHR) {
            const int row = i >> 3, c8 = (i & 7) * 8;
            const int t = t0 + row;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (t < n_tokens) v = *(const uint4*)(x + (size_t)t * H + k0 + c8);
            const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                xs[(c8 + 2 * j) * LD + (row ^ swz(c8))] = bf16lo(w4[j]);
                xs[(c8 + 2 * j + 1) * LD + (row ^ swz(c8))] = bf16hi(w4[j]);
            }
        }
        if (KIND == 1) {
            const float* w = (const float*)p.weight;
            for (int i = threadIdx.x; i < 64 * 16; i += NTHR) {
                const int row = i >> 4, c4 = (i & 15) * 4;
                const int e = e0 + row;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (e < E) v = *(const float4*)(w + (size_t)e * H + k0 + c4);
                const int col = row ^ swz(c4);
                ws[(c4 + 0) * LD + col] = v.x; ws[(c4 + 1) * LD + col] = v.y;
                ws[(c4 + 2) * LD + col] = v.z; ws[(c4 + 3) * LD + col] = v.w;
            }
        } else if (KIND == 2) {
            const uint16_t* w = (const uint16_t*)p.weight;
            for (int i = threadIdx.x; i < 64 * 8; i += NTHR) {
                const int row = i >> 3, c8 = (i & 7) * 8;
                const int e = e0 + row;
                uint4 v = make_uint4(0, 0, 0, 0);
                if (e < E) v = *(const uint4*)(w + (size_t)e * H + k0 + c8);
                const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    ws[(c8 + 2 * j) * LD + (row ^ swz(c8))] = bf16lo(w4[j]);
                    ws[(c8 + 2 * j + 1) * LD + (row ^ swz(c8))] = bf16hi(w4[j]);
                }
            }
        } else {
            // affine: one thread unpacks a 32-run of one expert row (w = fma(scale, q, bias))
            const uint32_t* w = (const uint32_t*)p.weight;
            const int gpr = H / p.group_size;
            for (int i = threadIdx.x; i < 64 * 2; i += NTHR) {
                const int row = i >> 1, h32 = (i & 1) * 32;
                const int e = e0 + row;
                if (e < E) {
                    const int k = k0 + h32;
                    const int g = k / p.group_size;
                    const float sc = bf16_bits_to_f32(p.scales[(size_t)e * gpr + g]);
                    const float bi = bf16_bits_to_f32(p.biases[(size_t)e * gpr + g]);
                    uint32_t words[BITS + 1];
                    const uint32_t* src = w + (size_t)e * (H * BITS / 32) + (k / 32) * BITS;
#pragma unroll
                    for (int j = 0; j < BITS; ++j) words[j] = src[j];
                    words[BITS] = 0;
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        ws[(h32 + j) * LD + (row ^ swz(h32 + j))] = __fmaf_rn(sc, small_uint_to_float(unpack_at<BITS>(words, j)), bi);
                } else {
                    for (int j = 0; j < 32; ++j) ws[(h32 + j) * LD + (row ^ swz(h32 + j))] = 0.0f;
                }
            }
        }
        __syncthreads();
        float part[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) part[i][j] = 0.0f;
#pragma unroll 8
        for (int k = 0; k < 64; ++k) {
            const float4 xv = *(const float4*)(xs + k * LD + ((ty * 4) ^ swz(k)));
            const float4 wv = *(const float4*)(ws + k * LD + ((tx * 4) ^ swz(k)));
            const float xa[4] = {xv.x, xv.y, xv.z, xv.w};
            const float wa[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) part[i][j] = __fmaf_rn(xa[i], wa[j], part[i][j]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) total[i][j] = __fadd_rn(total[i][j], part[i][j]);
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int t = t0 + ty * 4 + i;
        if (t >= n_tokens) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int e = e0 + tx * 4 + j;
            if (e >= E) continue;
            float v = total[i][j];
            if (partials) {  // 0 + chunk sum is the chunk sum: exact
                partials[((size_t)blockIdx.z * n_tokens + t) * E + e] = v;
                continue;
            }
            if (p.logits_bf16) v = bf16_round(v);
            if (p.bias) {
                v = __fadd_rn(v, bf16_bits_to_f32(p.bias[e]));
                if (p.logits_bf16) v = bf16_round(v);
            }
            logits_out[(size_t)t * E + e] = v;
        }
    }
}

// Batched router projection for long prefill chunks: a 128-token x 64-expert tile per block of 256 threads, 8 x 4
// outputs per thread, the hidden axis walked one 64-wide chunk at a time.  The global loads of chunk c+1 are issued
// before the arithmetic of chunk c and parked in registers, so their latency hides behind 64 k-steps of fused
// multiply-adds.  The running totals live in shared memory (touched once per chunk), which leaves the registers to
// the 32 chunk accumulators and the parked loads.  Accumulation order is the fixed one (inside a chunk: ascending k
// from 0 with fused multiply-add; chunk sums added in ascending order), so the logits equal those of every other
// router kernel bit for bit.  KIND: 1 fp32 weights, 2 bf16 weights.
constexpr int RB_TOK = 128, RB_EXP = 64, RB_XLD = 132, RB_WLD = 68;
constexpr int RB_SMEM = (64 * (RB_XLD + RB_WLD) + 32 * 256) * 4;

// With `partials` the hidden axis is also split over blockIdx.z into ranges of `chunks_per_z` chunks: a block then
// writes the sum of every chunk of its range to partials[chunk][token][expert] instead of keeping totals, and
// route_from_partials_kernel adds the chunks in ascending order (same bits, enough blocks for mid-sized batches).
template <int KIND>
__global__ void __launch_bounds__(256, 2)
router_logits_big_kernel(RouterParams p, const uint16_t* __restrict__ x, int n_tokens, float* __restrict__ logits_out,
                         float* __restrict__ partials, int chunks_per_z) {
    extern __shared__ __align__(16) float rbsm[];
    float* xs = rbsm;                          // [64 k][RB_XLD]
    float* ws = rbsm + 64 * RB_XLD;            // [64 k][RB_WLD]
    float* tot = ws + 64 * RB_WLD + threadIdx.x;   // [32 outputs][256 threads]
    auto swz = [](int k) { return ((k >> 3) & 7) << 2; };
    const int H = p.hidden, E = p.n_experts;
    const int t0 = blockIdx.x * RB_TOK, e0 = blockIdx.y * RB_EXP;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    constexpr int WV = KIND == 1 ? 4 : 2;      // 16-byte pieces of weights per thread and chunk

    uint4 xr[4];
    uint4 wr[WV];
    auto load_chunk = [&](int k0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int id = threadIdx.x + 256 * i, row = id >> 3, c8 = (id & 7) * 8;
            const int t = t0 + row;
            xr[i] = t < n_tokens ? *reinterpret_cast<const uint4*>(x + (size_t)t * H + k0 + c8) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int i = 0; i < WV; ++i) {
            const int id = threadIdx.x + 256 * i;
            if (KIND == 1) {
                const int row = id >> 4, c4 = (id & 15) * 4;
                const int e = e0 + row;
                wr[i] = e < E ? *reinterpret_cast<const uint4*>((const float*)p.weight + (size_t)e * H + k0 + c4) : make_uint4(0, 0, 0, 0);
            } else {
                const int row = id >> 3, c8 = (id & 7) * 8;
                const int e = e0 + row;
                wr[i] = e < E ? *reinterpret_cast<const uint4*>((const uint16_t*)p.weight + (size_t)e * H + k0 + c8) : make_uint4(0, 0, 0, 0);
            }
        }
    };
    auto store_chunk = [&]() {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int id = threadIdx.x + 256 * i, row = id >> 3, c8 = (id & 7) * 8;
            const uint32_t w4[4] = {xr[i].x, xr[i].y, xr[i].z, xr[i].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                xs[(c8 + 2 * j) * RB_XLD + (row ^ swz(c8))] = bf16lo(w4[j]);
                xs[(c8 + 2 * j + 1) * RB_XLD + (row ^ swz(c8))] = bf16hi(w4[j]);
            }
        }
#pragma unroll
        for (int i = 0; i < WV; ++i) {
            const int id = threadIdx.x + 256 * i;
            if (KIND == 1) {
                const int row = id >> 4, c4 = (id & 15) * 4;
                const int col = row ^ swz(c4);
                ws[(c4 + 0) * RB_WLD + col] = __uint_as_float(wr[i].x); ws[(c4 + 1) * RB_WLD + col] = __uint_as_float(wr[i].y);
                ws[(c4 + 2) * RB_WLD + col] = __uint_as_float(wr[i].z); ws[(c4 + 3) * RB_WLD + col] = __uint_as_float(wr[i].w);
            } else {
                const int row = id >> 3, c8 = (id & 7) * 8;
                const uint32_t w4[4] = {wr[i].x, wr[i].y, wr[i].z, wr[i].w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    ws[(c8 + 2 * j) * RB_WLD + (row ^ swz(c8))] = bf16lo(w4[j]);
                    ws[(c8 + 2 * j + 1) * RB_WLD + (row ^ swz(c8))] = bf16hi(w4[j]);
                }
            }
        }
    };

#pragma unroll
    for (int i = 0; i < 32; ++i) tot[i * 256] = 0.0f;

    const int all_chunks = H / 64;
    const int c_begin = partials ? (int)blockIdx.z * chunks_per_z : 0;
    const int n_chunks = partials ? min(all_chunks, c_begin + chunks_per_z) : all_chunks;   // end of this block's range
    if (c_begin >= n_chunks) return;
    load_chunk(c_begin * 64);
    for (int c = c_begin; c < n_chunks; ++c) {
        store_chunk();
        __syncthreads();
        if (c + 1 < n_chunks) load_chunk((c + 1) * 64);
        float part[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) part[i][j] = 0.0f;
#pragma unroll 8
        for (int k = 0; k < 64; ++k) {
            const float4 xa = *reinterpret_cast<const float4*>(xs + k * RB_XLD + ((ty * 8) ^ swz(k)));
            const float4 xc = *reinterpret_cast<const float4*>(xs + k * RB_XLD + ((ty * 8 + 4) ^ swz(k)));
            const float4 wv = *reinterpret_cast<const float4*>(ws + k * RB_WLD + ((tx * 4) ^ swz(k)));
            const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xc.x, xc.y, xc.z, xc.w};
            const float wa[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) part[i][j] = __fmaf_rn(xv[i], wa[j], part[i][j]);
        }
        if (partials) {
            float* dst = partials + (size_t)c * n_tokens * E;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int t = t0 + ty * 8 + i, e = e0 + tx * 4;
                if (t >= n_tokens) continue;
                if (e + 3 < E && (E & 3) == 0) {
                    *reinterpret_cast<float4*>(dst + (size_t)t * E + e) = make_float4(part[i][0], part[i][1], part[i][2], part[i][3]);
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (e + j < E) dst[(size_t)t * E + e + j] = part[i][j];
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) tot[(i * 4 + j) * 256] = __fadd_rn(tot[(i * 4 + j) * 256], part[i][j]);
        }
        __syncthreads();   // the tiles are read: the next chunk may overwrite them
    }
    if (partials) return;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int t = t0 + ty * 8 + i;
        if (t >= n_tokens) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int e = e0 + tx * 4 + j;
            if (e >= E) continue;
            float v = tot[(i * 4 + j) * 256];
            if (p.logits_bf16) v = bf16_round(v);
            if (p.bias) {
                v = __fadd_rn(v, bf16_bits_to_f32(p.bias[e]));
                if (p.logits_bf16) v = bf16_round(v);
            }
            logits_out[(size_t)t * E + e] = v;
        }
    }
}

// Second half of the chunk-split projection: one warp per token adds the chunk sums of every expert in
// ascending chunk order (the fixed order), applies rounding and bias, and routes.
__global__ void route_from_partials_kernel(RouterParams p, const float* __restrict__ partials, int n_chunks,
                                           int n_tokens, uint32_t* __restrict__ indices,
                                           float* __restrict__ weights, float* __restrict__ logits_out) {
    extern __shared__ float smem[];
    const int E = p.n_experts;
    const int warps = blockDim.x / 32;
    const int warp = threadIdx.x / 32, lane = threadIdx.x & 31;
    const int t = blockIdx.x * warps + warp;
    float* logits_s = smem + (size_t)warp * 2 * E;
    float* scratch = logits_s + E;
    if (t >= n_tokens) return;
    auto finish = [&](int e, float total) {
        if (p.logits_bf16) total = bf16_round(total);
        if (p.bias) {
            total = __fadd_rn(total, bf16_bits_to_f32(p.bias[e]));
            if (p.logits_bf16) total = bf16_round(total);
        }
        logits_s[e] = total;
        if (logits_out) logits_out[(size_t)t * E + e] = total;
    };
    if ((E & 3) == 0) {
        // a lane owns four consecutive experts; eight chunk loads are issued before the first add so the
        // (ordered) additions do not wait for one memory latency each
        constexpr int U = 8;
        for (int e = lane * 4; e < E; e += 128) {
            float4 total = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int c0 = 0; c0 < n_chunks; c0 += U) {
                float4 v[U];
#pragma unroll
                for (int u = 0; u < U; ++u)
                    if (c0 + u < n_chunks) v[u] = __ldg(reinterpret_cast<const float4*>(partials + ((size_t)(c0 + u) * n_tokens + t) * E + e));
#pragma unroll
                for (int u = 0; u < U; ++u)
                    if (c0 + u < n_chunks) {
                        total.x = __fadd_rn(total.x, v[u].x); total.y = __fadd_rn(total.y, v[u].y);
                        total.z = __fadd_rn(total.z, v[u].z); total.w = __fadd_rn(total.w, v[u].w);
                    }
            }
            finish(e, total.x); finish(e + 1, total.y); finish(e + 2, total.z); finish(e + 3, total.w);
        }
    } else {
        for (int e = lane; e < E; e += 32) {
            float total = 0.0f;
            for (int c = 0; c < n_chunks; ++c) total = __fadd_rn(total, partials[((size_t)c * n_tokens + t) * E + e]);
            finish(e, total);
        }
    }
    __syncwarp();
    route_token_warp(p, logits_s, scratch, lane, indices + (size_t)t * p.top_k, weights + (size_t)t * p.top_k);
}

// Routing only (logits already computed): one warp per token.
__global__ void route_only_kernel(RouterParams p, const float* __restrict__ logits, int n_tokens,
                                  uint32_t* __restrict__ indices, float* __restrict__ weights) {
    extern __shared__ float smem[];
    const int E = p.n_experts;
    const int warps = blockDim.x / 32;
    const int warp = threadIdx.x / 32, lane = threadIdx.x & 31;
    const int t = blockIdx.x * warps + warp;
    float* logits_s = smem + (size_t)warp * 2 * E;
    float* scratch = logits_s + E;
    if (t >= n_tokens) return;
    for (int e = lane; e < E; e += 32) logits_s[e] = logits[(size_t)t * E + e];
    __syncwarp();
    route_token_warp(p, logits_s, scratch, lane, indices + (size_t)t * p.top_k,
                     weights + (size_t)t * p.top_k);
}

}  // namespace ffai
