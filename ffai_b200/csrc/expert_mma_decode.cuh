// Decode-regime grouped 4-bit dequant products: weights stream straight from HBM into
// registers, one warp per 16 weight rows, no shared memory and no cross-warp handshakes.
//
// Replaces, for small batches, the reference's per-expert GEMV chain
// (Ops.dequantGemvInt4ExpertIndexedMany, FFAI Ops.swift:2529-2587; the fused
// moeDownSwigluAccumInt4Chain8, OpsFused.swift:545-697; MoELayer.decodeGPURouter,
// MoELayer.swift:1167-1341) and GPT-OSS's three-sync-per-expert loop
// (GPTOSSText.swift:1399-1445).
//
// A warp owns 16 consecutive output rows of one expert (for gate/up: the 16 gate rows and
// the 16 up rows, so the activation is applied in registers) and walks the reduction axis
// one 64-value group at a time.  Per group a lane loads two packed words per row it
// touches (8-byte loads; a warp covers 8 rows x 32 contiguous bytes), turns each word into
// four bf16 pairs holding 128+q exactly ((q | 0x4300) is the bf16 128+q), and feeds them to
// mma.sync.m16n8k16 as the A operand; the B operand is the 8 (or 16) activation rows routed
// to this expert, read through L1.  The tensor core is only the dot-product engine here:
// the kernel is bound by HBM.  After each group the fp32 partial is folded in with the
// group's scale and bias:
//     sum_k (s*q_k + b) x_k = s * sum_k (128+q_k) x_k + (b - 128 s) * sum_k x_k,
// where sum_k x_k per (row of activations, group) is precomputed by the kernel that wrote
// the activations.  fp32 accumulation throughout; weights are never rounded.
//
// K order: the unpack yields the nibble pairs (0,4),(1,5),(2,6),(3,7) of a word, so the
// activation rows are stored with every 8-run in the order 0,4,1,5,2,6,3,7 (done by the
// kernels that write them); the dot product does not see the permutation.
#pragma once
#include "common.cuh"

namespace ffai {
namespace dmma {

struct Params {
    const uint32_t* w1;    // [E, N, K/8]
    const uint16_t* s1;    // [E, N, K/gs]
    const uint16_t* b1;
    const uint16_t* rb1;   // nullable [E, N]
    const uint32_t* w2;    // second projection (fused gate/up)
    const uint16_t* s2;
    const uint16_t* b2;
    const uint16_t* rb2;
    int N, K, group_size;  // group_size 64 or 128
    const uint32_t* offsets;  // [E+1] rows per expert in the sorted row space
    const uint16_t* x;        // [rows, K] bf16, 8-run permuted
    const float* xsum;        // [rows, K/64] sum of each 64-run of x
    void* out;                // FUSED: bf16 [rows, N] 8-run permuted;  else fp32 [rows, N]
    int activation;
    float limit, alpha;
};

FFAI_DEVINL void mma_bf16_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// One packed word -> 4 bf16 pairs (128+n0,128+n4), (128+n1,128+n5), (128+n2,128+n6), (128+n3,128+n7).
FFAI_DEVINL void unpack_word_128(uint32_t w, uint32_t* o) {
    o[0] = (w & 0x000F000Fu) | 0x43004300u;
    o[1] = ((w >> 4) & 0x000F000Fu) | 0x43004300u;
    o[2] = ((w >> 8) & 0x000F000Fu) | 0x43004300u;
    o[3] = ((w >> 12) & 0x000F000Fu) | 0x43004300u;
}

FFAI_DEVINL uint2 ld_stream_u2(const uint32_t* p) {
    uint2 v;
    asm volatile("ld.global.cs.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

FFAI_DEVINL int permute8_col(int n) {
    const int k = n & 7;
    return (n & ~7) | (((k & 3) << 1) | (k >> 2));
}

// grid: (ceil(N/16 / 4), E); block: 128 threads = 4 warps, each warp one 16-row block.
// NT: activation rows handled per pass over the weights, in units of 8.
template <bool FUSED, int NT>
__global__ void __launch_bounds__(128)
grouped_mma_decode_kernel(const Params p) {
    constexpr int NP = FUSED ? 2 : 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int e = blockIdx.y;
    const int rb = blockIdx.x * 4 + warp;
    if (rb * 16 >= p.N) return;
    const int row0 = (int)p.offsets[e], cnt = (int)p.offsets[e + 1] - row0;
    if (cnt <= 0) return;

    const int K = p.K, wpr = K / 8, gpr = K / p.group_size, n64 = K / 64;
    const int gshift = p.group_size == 128 ? 1 : 0;  // 64-run index -> scale group index
    const size_t rlo = (size_t)e * p.N + rb * 16 + g, rhi = rlo + 8;
    const uint32_t* wp[NP][2];
    const uint16_t* sp[NP][2];
    const uint16_t* bp[NP][2];
    wp[0][0] = p.w1 + rlo * wpr + 2 * t; wp[0][1] = p.w1 + rhi * wpr + 2 * t;
    sp[0][0] = p.s1 + rlo * gpr; sp[0][1] = p.s1 + rhi * gpr;
    bp[0][0] = p.b1 + rlo * gpr; bp[0][1] = p.b1 + rhi * gpr;
    if (FUSED) {
        wp[NP - 1][0] = p.w2 + rlo * wpr + 2 * t; wp[NP - 1][1] = p.w2 + rhi * wpr + 2 * t;
        sp[NP - 1][0] = p.s2 + rlo * gpr; sp[NP - 1][1] = p.s2 + rhi * gpr;
        bp[NP - 1][0] = p.b2 + rlo * gpr; bp[NP - 1][1] = p.b2 + rhi * gpr;
    }

    for (int tok0 = 0; tok0 < cnt; tok0 += 8 * NT) {
        // activation row read by this lane as B operand (column g of each 8-wide tile), and the
        // two rows whose results this lane holds (columns 2t, 2t+1); clamped, masked at the store
        const uint16_t* xrow[NT];
        const float* sxa[NT];
        const float* sxb[NT];
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const int last = cnt - 1;
            xrow[j] = p.x + (size_t)(row0 + min(tok0 + 8 * j + g, last)) * K + 16 * t;
            sxa[j] = p.xsum + (size_t)(row0 + min(tok0 + 8 * j + 2 * t, last)) * n64;
            sxb[j] = p.xsum + (size_t)(row0 + min(tok0 + 8 * j + 2 * t + 1, last)) * n64;
        }
        float tot[NT][NP][4];
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int q = 0; q < NP; ++q)
#pragma unroll
                for (int i = 0; i < 4; ++i) tot[j][q][i] = 0.0f;

        // software pipeline: packed words of the next group are in flight while this one is consumed
        uint2 wnext[NP][2];
#pragma unroll
        for (int q = 0; q < NP; ++q) { wnext[q][0] = ld_stream_u2(wp[q][0]); wnext[q][1] = ld_stream_u2(wp[q][1]); }

        for (int G = 0; G < n64; ++G) {
            uint2 wcur[NP][2];
#pragma unroll
            for (int q = 0; q < NP; ++q) { wcur[q][0] = wnext[q][0]; wcur[q][1] = wnext[q][1]; }
            if (G + 1 < n64) {
#pragma unroll
                for (int q = 0; q < NP; ++q) {
                    wnext[q][0] = ld_stream_u2(wp[q][0] + (G + 1) * 8);
                    wnext[q][1] = ld_stream_u2(wp[q][1] + (G + 1) * 8);
                }
            }
            // scale and (bias - 128*scale) of the two rows this lane's results belong to
            float sc[NP][2], bm[NP][2];
            const int gi = G >> gshift;
#pragma unroll
            for (int q = 0; q < NP; ++q)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const float s = bf16_bits_to_f32(__ldg(sp[q][h] + gi));
                    const float b = bf16_bits_to_f32(__ldg(bp[q][h] + gi));
                    sc[q][h] = s;
                    bm[q][h] = fmaf(-128.0f, s, b);
                }
            // A fragments: [projection][word 0/1][row lo/hi][pair 0..3]
            uint32_t af[NP][2][2][4];
#pragma unroll
            for (int q = 0; q < NP; ++q)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    unpack_word_128(wcur[q][h].x, af[q][0][h]);
                    unpack_word_128(wcur[q][h].y, af[q][1][h]);
                }
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const uint4 x0 = __ldg(reinterpret_cast<const uint4*>(xrow[j] + G * 64));
                const uint4 x1 = __ldg(reinterpret_cast<const uint4*>(xrow[j] + G * 64 + 8));
                const uint32_t xb[2][4] = {{x0.x, x0.y, x0.z, x0.w}, {x1.x, x1.y, x1.z, x1.w}};
                const float sx0 = __ldg(sxa[j] + G), sx1 = __ldg(sxb[j] + G);
#pragma unroll
                for (int q = 0; q < NP; ++q) {
                    float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int w = 0; w < 2; ++w)
#pragma unroll
                        for (int hp = 0; hp < 2; ++hp) {
                            // k-slots (2t,2t+1) <- pair 2hp, (2t+8,2t+9) <- pair 2hp+1 of word w
                            const uint32_t a[4] = {af[q][w][0][2 * hp], af[q][w][1][2 * hp],
                                                   af[q][w][0][2 * hp + 1], af[q][w][1][2 * hp + 1]};
                            mma_bf16_16816(c, a, xb[w][2 * hp], xb[w][2 * hp + 1]);
                        }
                    tot[j][q][0] = fmaf(sc[q][0], c[0], fmaf(bm[q][0], sx0, tot[j][q][0]));
                    tot[j][q][1] = fmaf(sc[q][0], c[1], fmaf(bm[q][0], sx1, tot[j][q][1]));
                    tot[j][q][2] = fmaf(sc[q][1], c[2], fmaf(bm[q][1], sx0, tot[j][q][2]));
                    tot[j][q][3] = fmaf(sc[q][1], c[3], fmaf(bm[q][1], sx1, tot[j][q][3]));
                }
            }
        }

        // results: value i -> (row g + 8*(i>>1), activation row tok0 + 8j + 2t + (i&1))
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int tok = tok0 + 8 * j + 2 * t + (i & 1);
                if (tok >= cnt) continue;
                const int n = rb * 16 + g + 8 * (i >> 1);
                const size_t rr = (size_t)e * p.N + n;
                float v = tot[j][0][i];
                if (p.rb1) v += bf16_bits_to_f32(p.rb1[rr]);
                if (FUSED) {
                    float u = tot[j][NP - 1][i];
                    if (p.rb2) u += bf16_bits_to_f32(p.rb2[rr]);
                    v = glu_activation(v, u, p.activation, p.limit, p.alpha);
                    reinterpret_cast<uint16_t*>(p.out)[(size_t)(row0 + tok) * p.N + permute8_col(n)] = f32_to_bf16_bits(v);
                } else {
                    reinterpret_cast<float*>(p.out)[(size_t)(row0 + tok) * p.N + n] = v;
                }
            }
    }
}

// Gather rows into expert-sorted order with the 8-run permutation, and write the sum of every
// 64-run (fp32).  One warp per output row.  ids nullable (identity), id_div as in Ops.gather use.
__global__ void gather_perm8_sum64_kernel(const uint16_t* __restrict__ table, const uint32_t* __restrict__ ids,
                                          int id_div, uint16_t* __restrict__ out, float* __restrict__ sums,
                                          int n_rows, int row_len) {
    const int warps = blockDim.x / 32;
    const int row = blockIdx.x * warps + threadIdx.x / 32;
    if (row >= n_rows) return;
    const int lane = threadIdx.x & 31;
    const uint32_t src = ids ? ids[row] / (uint32_t)id_div : (uint32_t)row;
    const uint4* s = (const uint4*)(table + (size_t)src * row_len);
    uint4* d = (uint4*)(out + (size_t)row * row_len);
    const int chunks = row_len / 8;  // 16-byte chunks; 8 chunks per 64-run
    for (int i0 = 0; i0 < chunks; i0 += 32) {
        const int i = i0 + lane;
        float part = 0.0f;
        if (i < chunks) {
            const uint4 v = s[i];
            uint4 o;
            o.x = __byte_perm(v.x, v.z, 0x5410);
            o.y = __byte_perm(v.x, v.z, 0x7632);
            o.z = __byte_perm(v.y, v.w, 0x5410);
            o.w = __byte_perm(v.y, v.w, 0x7632);
            d[i] = o;
            part = ((bf16lo(v.x) + bf16hi(v.x)) + (bf16lo(v.y) + bf16hi(v.y))) +
                   ((bf16lo(v.z) + bf16hi(v.z)) + (bf16lo(v.w) + bf16hi(v.w)));
        }
        // 8 consecutive lanes hold one 64-run: fixed-shape tree over them
        part += __shfl_xor_sync(0xFFFFFFFFu, part, 1);
        part += __shfl_xor_sync(0xFFFFFFFFu, part, 2);
        part += __shfl_xor_sync(0xFFFFFFFFu, part, 4);
        if ((lane & 7) == 0 && i < chunks) sums[(size_t)row * (row_len / 64) + (i >> 3)] = part;
    }
}

// Sum of every 64-run of rows that are already stored 8-run permuted (the sum does not depend
// on the order inside a run).  One warp per row.
__global__ void sum64_rows_kernel(const uint16_t* __restrict__ rows, float* __restrict__ sums, int n_rows,
                                  int row_len) {
    const int warps = blockDim.x / 32;
    const int row = blockIdx.x * warps + threadIdx.x / 32;
    if (row >= n_rows) return;
    const int lane = threadIdx.x & 31;
    const uint4* s = (const uint4*)(rows + (size_t)row * row_len);
    const int chunks = row_len / 8;
    for (int i0 = 0; i0 < chunks; i0 += 32) {
        const int i = i0 + lane;
        float part = 0.0f;
        if (i < chunks) {
            const uint4 v = s[i];
            part = ((bf16lo(v.x) + bf16hi(v.x)) + (bf16lo(v.y) + bf16hi(v.y))) +
                   ((bf16lo(v.z) + bf16hi(v.z)) + (bf16lo(v.w) + bf16hi(v.w)));
        }
        part += __shfl_xor_sync(0xFFFFFFFFu, part, 1);
        part += __shfl_xor_sync(0xFFFFFFFFu, part, 2);
        part += __shfl_xor_sync(0xFFFFFFFFu, part, 4);
        if ((lane & 7) == 0 && i < chunks) sums[(size_t)row * (row_len / 64) + (i >> 3)] = part;
    }
}

}  // namespace dmma
}  // namespace ffai
