// Decode-regime grouped 4-bit dequant products: packed weights stream from HBM through a
// cp.async-staged shared-memory ring (16-byte asynchronous copies, three 256-k stages in
// flight) into registers, one warp per 16 weight rows; the only synchronisation is one
// __syncthreads per stage.
//
// Replaces, for small batches, the reference's per-expert GEMV chain
// (Ops.dequantGemvInt4ExpertIndexedMany, FFAI Ops.swift:2529-2587; the fused
// moeDownSwigluAccumInt4Chain8, OpsFused.swift:545-697; MoELayer.decodeGPURouter,
// MoELayer.swift:1167-1341) and GPT-OSS's three-sync-per-expert loop
// (GPTOSSText.swift:1399-1445).
//
// A warp owns 16 consecutive output rows of one expert (for gate/up: the 16 gate rows and
// the 16 up rows, so the activation is applied in registers) and walks the reduction axis
// one 64-value group at a time.  Per group a lane reads two packed words per row it
// touches from the staged tile, turns each word into
// four bf16 pairs holding 128+q exactly ((q | 0x4300) is the bf16 128+q), and feeds them to
// mma.sync.m16n8k16 as the A operand; the B operand is the 8 (or 16) activation rows routed
// to this expert, staged alongside.  The tensor core is only the dot-product engine here:
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
    const float* xsum;        // [rows, xsum_pitch] sum of each 64-run of x; pitch = K/64 rounded up to 4
    int xsum_pitch;
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

FFAI_DEVINL void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
FFAI_DEVINL void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
FFAI_DEVINL void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Shared-memory staging geometry.  A stage is 256 k: per weight row 128 bytes (pitch 160 so the
// 8-byte fragment reads of eight rows fall in distinct banks), per activation row 512 bytes
// (pitch 528 for the 16-byte fragment reads).
constexpr int STG_K = 256;                 // k per stage
constexpr int STG_GROUPS = STG_K / 64;     // 64-runs per stage
constexpr int W_PITCH = 160;
constexpr int X_PITCH = 528;
constexpr int WARPS = 4;                   // warps per CTA, 16 weight rows each
constexpr int DEPTH = 3;                   // stages in flight

template <bool FUSED, int NT>
struct StageLayout {
    static constexpr int NP = FUSED ? 2 : 1;
    static constexpr int W_BYTES = WARPS * NP * 16 * W_PITCH;   // packed weight rows of the whole CTA
    static constexpr int X_BYTES = NT * 8 * X_PITCH;            // activation rows shared by the CTA
    static constexpr int S_BYTES = NT * 8 * 16;                 // their 64-run sums: 4 floats per row
    static constexpr int STAGE = W_BYTES + X_BYTES + S_BYTES;
    static constexpr int TOTAL = DEPTH * STAGE;
};

// grid: (ceil(N / 64), E); block: 128 threads = 4 warps; warp w owns rows [64*bx + 16*w, +16) of expert by.
// The four warps share the expert, hence the activation rows: weights and activations are staged by the
// whole CTA with cp.async (16-byte asynchronous copies, DEPTH stages in flight, one __syncthreads per stage).
// NT: activation rows handled per pass over the weights, in units of 8.
template <bool FUSED, int NT>
__global__ void __launch_bounds__(128)
grouped_mma_decode_kernel(const Params p) {
    using SL = StageLayout<FUSED, NT>;
    constexpr int NP = SL::NP;
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int e = blockIdx.y;
    const int row0 = (int)p.offsets[e], cnt = (int)p.offsets[e + 1] - row0;
    if (cnt <= 0) return;
    const int cta_row = blockIdx.x * 64;           // first weight row (within the expert) of this CTA
    const int K = p.K, wpr = K / 8, gpr = K / p.group_size, n64 = K / 64;
    const int n_stages = (K + STG_K - 1) / STG_K;
    const int gshift = p.group_size == 128 ? 1 : 0;  // 64-run index -> scale group index
    const int rb_row = cta_row + warp * 16;        // this warp's first row
    const bool warp_active = rb_row < p.N;         // N is a multiple of 16
    const size_t rlo = (size_t)e * p.N + (warp_active ? rb_row : 0) + g, rhi = rlo + 8;
    const uint16_t* sp[NP][2];
    const uint16_t* bp[NP][2];
    sp[0][0] = p.s1 + rlo * gpr; sp[0][1] = p.s1 + rhi * gpr;
    bp[0][0] = p.b1 + rlo * gpr; bp[0][1] = p.b1 + rhi * gpr;
    if (FUSED) {
        sp[NP - 1][0] = p.s2 + rlo * gpr; sp[NP - 1][1] = p.s2 + rhi * gpr;
        bp[NP - 1][0] = p.b2 + rlo * gpr; bp[NP - 1][1] = p.b2 + rhi * gpr;
    }
    const int rows_in_cta = min(64, p.N - cta_row);  // multiple of 16

    for (int tok0 = 0; tok0 < cnt; tok0 += 8 * NT) {
        const int ntok = min(8 * NT, cnt - tok0);
        // issue the asynchronous copies of one stage: CTA-wide, 16 bytes per copy
        auto issue_stage = [&](int st) {
            if (st < n_stages) {
                const uint32_t dst = sbase + (st % DEPTH) * SL::STAGE;
                const int kbytes_w = min(STG_K, K - st * STG_K) / 2;   // valid packed bytes per row in this stage
                const int kbytes_x = kbytes_w * 4;                     // valid activation bytes per row
                // weights: NP * 64 rows x 8 chunks
                for (int c = threadIdx.x; c < NP * 64 * 8; c += 128) {
                    const int col = c & 7, r = (c >> 3) & 63, q = c >> 9;
                    if (r < rows_in_cta) {
                        const uint32_t* base = q ? p.w2 : p.w1;
                        const uint8_t* src = reinterpret_cast<const uint8_t*>(base + ((size_t)e * p.N + cta_row + r) * wpr) +
                                             st * (STG_K / 2) + col * 16;
                        const uint32_t d = dst + (((r >> 4) * NP + q) * 16 + (r & 15)) * W_PITCH + col * 16;
                        const int valid = kbytes_w - col * 16;
                        if (valid > 0) cp_async16(d, src, 16);
                    }
                }
                // activations: ntok rows x 32 chunks
                for (int c = threadIdx.x; c < ntok * 32; c += 128) {
                    const int col = c & 31, r = c >> 5;
                    const uint8_t* src = reinterpret_cast<const uint8_t*>(p.x + (size_t)(row0 + tok0 + r) * K) +
                                         st * (STG_K * 2) + col * 16;
                    const uint32_t d = dst + SL::W_BYTES + r * X_PITCH + col * 16;
                    if (col * 16 < kbytes_x) cp_async16(d, src, 16);
                }
                // 64-run sums of those rows: 4 floats per row
                if (threadIdx.x < ntok)
                    cp_async16(dst + SL::W_BYTES + SL::X_BYTES + threadIdx.x * 16,
                               p.xsum + (size_t)(row0 + tok0 + threadIdx.x) * p.xsum_pitch + st * STG_GROUPS, 16);
            }
            cp_async_commit();
        };

        float tot[NT][NP][4];
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int q = 0; q < NP; ++q)
#pragma unroll
                for (int i = 0; i < 4; ++i) tot[j][q][i] = 0.0f;

        __syncthreads();  // every warp is done with the previous pass's stages
#pragma unroll
        for (int st = 0; st < DEPTH - 1; ++st) issue_stage(st);
        // (scale | bias << 16) of stages st and st+1, alternating slots
        uint32_t sb_cur[NP][2], sb_nxt[NP][2];
        auto fetch_sb = [&](int st, uint32_t (*dst)[2]) {
            const int Gm = min(st * STG_GROUPS + t, n64 - 1) >> gshift;
#pragma unroll
            for (int q = 0; q < NP; ++q)
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    dst[q][h] = (uint32_t)__ldg(sp[q][h] + Gm) | ((uint32_t)__ldg(bp[q][h] + Gm) << 16);
        };
        fetch_sb(0, sb_cur);
        fetch_sb(1, sb_nxt);

        for (int st = 0; st < n_stages; ++st) {
            cp_async_wait<DEPTH - 2>();   // stage st has landed (this thread's copies)
            __syncthreads();              // ... and everyone else's; stage st-1 is free again
            issue_stage(st + DEPTH - 1);
            if (warp_active) {
                const uint8_t* stage = smem + (st % DEPTH) * SL::STAGE;
                const uint8_t* wst = stage + warp * NP * 16 * W_PITCH;
                const uint8_t* xst = stage + SL::W_BYTES;
                const float* sst = reinterpret_cast<const float*>(xst + SL::X_BYTES);
                const int groups = min(STG_GROUPS, n64 - st * STG_GROUPS);
                // scale / bias: lane (g, t) holds 64-run st*4+t of its two rows (shared by shuffle below);
                // the values of the stage after next are fetched now, so the loads never stall the warp
                uint32_t sbv[NP][2], sbn[NP][2];
                fetch_sb(st + 2, sbn);
#pragma unroll
                for (int q = 0; q < NP; ++q)
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        sbv[q][h] = sb_cur[q][h];
                        sb_cur[q][h] = sb_nxt[q][h];
                        sb_nxt[q][h] = sbn[q][h];
                    }
                float s_l[NP][2], b_l[NP][2];
#pragma unroll
                for (int q = 0; q < NP; ++q)
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        s_l[q][h] = __uint_as_float(sbv[q][h] << 16);
                        b_l[q][h] = __uint_as_float(sbv[q][h] & 0xFFFF0000u);
                    }
                for (int Gi = 0; Gi < groups; ++Gi) {
                    const int src_lane = (lane & ~3) | Gi;
                    float sc[NP][2], bm[NP][2];
#pragma unroll
                    for (int q = 0; q < NP; ++q)
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const float s = __shfl_sync(0xFFFFFFFFu, s_l[q][h], src_lane);
                            const float b = __shfl_sync(0xFFFFFFFFu, b_l[q][h], src_lane);
                            sc[q][h] = s;
                            bm[q][h] = fmaf(-128.0f, s, b);
                        }
                    // A fragments: [projection][word 0/1][row lo/hi][pair 0..3]
                    uint32_t af[NP][2][2][4];
#pragma unroll
                    for (int q = 0; q < NP; ++q)
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const uint2 wv = *reinterpret_cast<const uint2*>(wst + (q * 16 + g + 8 * h) * W_PITCH + Gi * 32 + t * 8);
                            unpack_word_128(wv.x, af[q][0][h]);
                            unpack_word_128(wv.y, af[q][1][h]);
                        }
#pragma unroll
                    for (int j = 0; j < NT; ++j) {
                        const uint8_t* xr = xst + (8 * j + g) * X_PITCH + Gi * 128 + t * 32;
                        const uint4 x0 = *reinterpret_cast<const uint4*>(xr);
                        const uint4 x1 = *reinterpret_cast<const uint4*>(xr + 16);
                        const uint32_t xb[2][4] = {{x0.x, x0.y, x0.z, x0.w}, {x1.x, x1.y, x1.z, x1.w}};
                        const float sx0 = sst[(8 * j + 2 * t) * 4 + Gi], sx1 = sst[(8 * j + 2 * t + 1) * 4 + Gi];
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
            }
        }
        cp_async_wait<0>();

        // results: value i -> (row g + 8*(i>>1), activation row tok0 + 8j + 2t + (i&1))
        if (warp_active) {
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int tok = tok0 + 8 * j + 2 * t + (i & 1);
                    if (tok >= cnt) continue;
                    const int n = rb_row + g + 8 * (i >> 1);
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
}

// Gather rows into expert-sorted order with the 8-run permutation, and write the sum of every
// 64-run (fp32).  One warp per output row.  ids nullable (identity), id_div as in Ops.gather use.
__global__ void gather_perm8_sum64_kernel(const uint16_t* __restrict__ table, const uint32_t* __restrict__ ids,
                                          int id_div, uint16_t* __restrict__ out, float* __restrict__ sums,
                                          int n_rows, int row_len, int sum_pitch) {
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
        if ((lane & 7) == 0 && i < chunks) sums[(size_t)row * sum_pitch + (i >> 3)] = part;
    }
}

// Sum of every 64-run of rows that are already stored 8-run permuted (the sum does not depend
// on the order inside a run).  One warp per row.
__global__ void sum64_rows_kernel(const uint16_t* __restrict__ rows, float* __restrict__ sums, int n_rows,
                                  int row_len, int sum_pitch) {
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
        if ((lane & 7) == 0 && i < chunks) sums[(size_t)row * sum_pitch + (i >> 3)] = part;
    }
}

}  // namespace dmma
}  // namespace ffai
