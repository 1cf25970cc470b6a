// Grouped dequant-GEMV on CUDA cores, any supported bit width (2,3,4,5,6,8).
//
// Replaces the reference's per-projection GEMV family: Ops.dequantGemv (FFAI
// Ops.swift:1489-1693), dequantGemvInt4ExpertIndexed[Many] (:2444-2587), the
// scalar grouped kernel moeGatherDequantGemmInt4M1 (:6499-6585) and, with the
// activation fused, Ops.swiglu (:6400-6452) / the GPT-OSS host activation loop
// (GPTOSSText.swift:1421-1431).
//
// One warp owns one output row of one expert and walks the rows routed to that
// expert four at a time, so a packed weight row is unpacked once per four
// tokens.  A lane handles 32 consecutive input values per step (BITS words of
// the packed row) and uses  sum_j (s*q_j + b)*x_j = s*sum_j q_j*x_j + b*sum_j x_j.
// fp32 accumulation throughout.
#pragma once
#include "common.cuh"

namespace ffai {

constexpr int GEMV_TT = 4;  // rows of activations per pass over a weight row

struct GemvParams {
    const uint32_t* weight;    // [E, N, K*bits/32]
    const uint16_t* scales;    // [E, N, K/gs]
    const uint16_t* biases;    // [E, N, K/gs]
    const uint16_t* row_bias;  // nullable [E, N]
    // second projection (fused gate/up): same shapes
    const uint32_t* weight2;
    const uint16_t* scales2;
    const uint16_t* biases2;
    const uint16_t* row_bias2;
    int N, K, group_size;
    int n_experts;
    const uint32_t* offsets;       // [E+1] row ranges per expert; nullptr: one expert, rows [0,n_rows)
    const uint32_t* row_expert;    // nullable [n_rows]: expert of each row (rows sorted by expert)
    const uint32_t* expert_index;  // nullable [1]: single expert chosen on the device
    const uint32_t* in_row_ids;    // nullable: input row of position p is in_row_ids[p] / in_row_div
    int in_row_div;
    int n_rows;
    int activation;
    float limit, alpha;
    int post_relu2;                // one-projection launches: out = relu(W x + b)^2 (experts without a gate projection)
};

template <typename TIn>
FFAI_DEVINL void load32(const TIn* p, float* v);

template <>
FFAI_DEVINL void load32<uint16_t>(const uint16_t* p, float* v) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint4 u = *(const uint4*)(p + i * 8);
        v[i * 8 + 0] = bf16lo(u.x); v[i * 8 + 1] = bf16hi(u.x);
        v[i * 8 + 2] = bf16lo(u.y); v[i * 8 + 3] = bf16hi(u.y);
        v[i * 8 + 4] = bf16lo(u.z); v[i * 8 + 5] = bf16hi(u.z);
        v[i * 8 + 6] = bf16lo(u.w); v[i * 8 + 7] = bf16hi(u.w);
    }
}
template <>
FFAI_DEVINL void load32<float>(const float* p, float* v) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float4 u = *(const float4*)(p + i * 4);
        v[i * 4 + 0] = u.x; v[i * 4 + 1] = u.y; v[i * 4 + 2] = u.z; v[i * 4 + 3] = u.w;
    }
}

FFAI_DEVINL void store_out(float* p, float v) { *p = v; }
FFAI_DEVINL void store_out(uint16_t* p, float v) { *p = f32_to_bf16_bits(v); }

template <int BITS>
FFAI_DEVINL void load_unpack32(const uint32_t* __restrict__ src, float* q) {
    uint32_t words[BITS + 1];
    if (BITS == 4) {
        uint4 u = *(const uint4*)src;
        words[0] = u.x; words[1] = u.y; words[2] = u.z; words[3] = u.w;
    } else if (BITS == 8) {
        uint4 u = *(const uint4*)src, v = *(const uint4*)(src + 4);
        words[0] = u.x; words[1] = u.y; words[2] = u.z; words[3] = u.w;
        words[4] = v.x; words[5] = v.y; words[6] = v.z; words[7] = v.w;
    } else {
#pragma unroll
        for (int i = 0; i < BITS; ++i) words[i] = src[i];
    }
    words[BITS] = 0;
#pragma unroll
    for (int j = 0; j < 32; ++j) q[j] = small_uint_to_float(unpack_at<BITS>(words, j));
}

// grid: (ceil(N / warps_per_block), n_expert_slots); block: warps_per_block*32.
// FUSED: out[p, n] = act(gate[p,n], up[p,n]); otherwise out[p, n] = W[e][n]·in[p] (+row_bias).
template <int BITS, typename TIn, typename TOut, bool FUSED>
__global__ void __launch_bounds__(128)
grouped_gemv_kernel(GemvParams p, const TIn* __restrict__ in, TOut* __restrict__ out) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * (blockDim.x >> 5) + warp;
    if (n >= p.N) return;
    int e = blockIdx.y;
    int row0 = 0, row1 = p.n_rows;
    if (p.offsets) {
        row0 = (int)p.offsets[e];
        row1 = (int)p.offsets[e + 1];
    } else if (p.expert_index) {
        e = (int)p.expert_index[0];
        if (e >= p.n_experts) return;
    }
    if (row0 >= row1) return;

    const int K = p.K, gs = p.group_size;
    const int wrow = K * BITS / 32, gpr = K / gs;
    const size_t r = (size_t)e * p.N + n;
    const uint32_t* w1 = p.weight + r * wrow;
    const uint16_t* s1 = p.scales + r * gpr;
    const uint16_t* b1 = p.biases + r * gpr;
    const uint32_t* w2 = FUSED ? p.weight2 + r * wrow : nullptr;
    const uint16_t* s2 = FUSED ? p.scales2 + r * gpr : nullptr;
    const uint16_t* b2 = FUSED ? p.biases2 + r * gpr : nullptr;
    const int nsteps = K / 32;

    for (int t0 = row0; t0 < row1; t0 += GEMV_TT) {
        const TIn* xin[GEMV_TT];
#pragma unroll
        for (int tt = 0; tt < GEMV_TT; ++tt) {
            int pos = min(t0 + tt, row1 - 1);
            size_t irow = p.in_row_ids ? (size_t)(p.in_row_ids[pos] / (uint32_t)p.in_row_div) : (size_t)pos;
            xin[tt] = in + irow * K;
        }
        float acc1[GEMV_TT], acc2[GEMV_TT];
#pragma unroll
        for (int tt = 0; tt < GEMV_TT; ++tt) { acc1[tt] = 0.0f; acc2[tt] = 0.0f; }

        for (int st = lane; st < nsteps; st += 32) {
            const int k0 = st * 32;
            const int g = k0 / gs;
            float q1[32], q2[32];
            load_unpack32<BITS>(w1 + st * BITS, q1);
            const float sc1 = bf16_bits_to_f32(s1[g]), bi1 = bf16_bits_to_f32(b1[g]);
            float sc2 = 0.0f, bi2 = 0.0f;
            if (FUSED) {
                load_unpack32<BITS>(w2 + st * BITS, q2);
                sc2 = bf16_bits_to_f32(s2[g]);
                bi2 = bf16_bits_to_f32(b2[g]);
            }
#pragma unroll
            for (int tt = 0; tt < GEMV_TT; ++tt) {
                if (t0 + tt < row1) {
                    float xv[32];
                    load32<TIn>(xin[tt] + k0, xv);
                    float d1 = 0.0f, d2 = 0.0f, sx = 0.0f;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        d1 = fmaf(q1[j], xv[j], d1);
                        if (FUSED) d2 = fmaf(q2[j], xv[j], d2);
                        sx += xv[j];
                    }
                    acc1[tt] = fmaf(sc1, d1, fmaf(bi1, sx, acc1[tt]));
                    if (FUSED) acc2[tt] = fmaf(sc2, d2, fmaf(bi2, sx, acc2[tt]));
                }
            }
        }
#pragma unroll
        for (int tt = 0; tt < GEMV_TT; ++tt) {
            float a1 = warp_sum(acc1[tt]);
            float a2 = FUSED ? warp_sum(acc2[tt]) : 0.0f;
            if (lane == 0 && t0 + tt < row1) {
                if (p.row_bias) a1 += bf16_bits_to_f32(p.row_bias[r]);
                float v = a1;
                if (FUSED) {
                    if (p.row_bias2) a2 += bf16_bits_to_f32(p.row_bias2[r]);
                    v = glu_activation(a1, a2, p.activation, p.limit, p.alpha);
                } else if (p.post_relu2) {
                    v = fmaxf(v, 0.0f);
                    v = v * v;
                }
                store_out(out + (size_t)(t0 + tt) * p.N + n, v);
            }
        }
    }
}

// Rows sorted by expert given as a per-row expert id (the reference's
// `indices[m]` argument, Ops.swift:4561-4571): build row ranges per expert.
__global__ void offsets_from_sorted_ids_kernel(const uint32_t* __restrict__ ids, int n_rows,
                                               int n_experts, uint32_t* __restrict__ offsets) {
    // offsets[e] = first row whose id >= e  (lower bound), offsets[E] = n_rows
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e > n_experts) return;
    int lo = 0, hi = n_rows;
    while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (ids[mid] < (uint32_t)e) lo = mid + 1; else hi = mid;
    }
    offsets[e] = (uint32_t)lo;
}

// Elementwise activation: Ops.swiglu / clamped / fusedGateGelu, bf16 in and out, fp32 math.
__global__ void glu_activation_kernel(const uint16_t* __restrict__ gate, const uint16_t* __restrict__ up,
                                      uint16_t* __restrict__ out, int64_t n, int activation,
                                      float limit, float alpha) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    out[i] = f32_to_bf16_bits(glu_activation(bf16_bits_to_f32(gate[i]), bf16_bits_to_f32(up[i]),
                                             activation, limit, alpha));
}

}  // namespace ffai
