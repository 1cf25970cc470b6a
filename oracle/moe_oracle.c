/*
 * moe_oracle.c — CPU oracle for the sparse-MoE block.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker, never the product: only the test-suite, the smoke
 * check and the CPU-baseline leg of the benchmark load it.  The CUDA library
 * does not link, call or fall back to anything here.
 *
 * It is a scalar restatement, in plain C, of the arithmetic the FFAI reference
 * performs on this path.  The reference's kernels live in an un-vendored
 * sibling project (thewafflehaus/metaltile, branch `dev`, no pinned revision),
 * so the arithmetic is taken from the reference's Swift host code and from the
 * CPU oracles embedded in its own unit tests; each function cites the file and
 * lines (paths within the FFAI project) it follows.
 *
 * Parity pins: tests/test_oracle_golden.py checks this file against every
 * known-answer case the reference's tests hold for the path (router cases,
 * bit-packing helpers, per-bit-width GEMV cases, the grouped-GEMM integer-hash
 * cases, unpermute, the 4-expert top-2 layer).  Unpinned in the reference and
 * therefore here: the GPU router's tie order (we use the CPU router's), the
 * summation order inside GEMV/GEMM kernels, and the affine quantizer's rounding.
 *
 * Two deliberate, documented choices where the reference leaves freedom:
 *   1. Router logits are accumulated in a fixed order (64-wide chunks, fused
 *      multiply-add inside a chunk, chunk sums added in ascending order) so the
 *      CUDA router can reproduce them bit-for-bit and top-k is exact.
 *   2. The softmax uses orc_expf below, a fixed sequence of IEEE operations,
 *      instead of libm's expf, so combine weights are reproducible bit-for-bit
 *      (it agrees with expf to 2 ulp; the reference's tests allow 1e-4).
 *
 * Build: gcc -O2 -ffp-contract=off -mfma -fopenmp -shared -fPIC (see Makefile).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "../include/ffai_cuda.h"

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_EXPORT __attribute__((visibility("default")))

/* ───────────────────────────── bf16 ───────────────────────────── */

/* Sources/FFAI/Tensor.swift:145-150 (round to nearest even on the bit pattern). */
ORC_EXPORT uint16_t orc_f32_to_bf16(float f) {
    uint32_t bits;
    memcpy(&bits, &f, 4);
    uint32_t rounded = bits + 0x7FFFu + ((bits >> 16) & 1u);
    return (uint16_t)(rounded >> 16);
}

/* Sources/FFAI/Tensor.swift:107-113. */
ORC_EXPORT float orc_bf16_to_f32(uint16_t b) {
    uint32_t bits = ((uint32_t)b) << 16;
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

static inline float bf16r(float f) { return orc_bf16_to_f32(orc_f32_to_bf16(f)); }

/* ───────────────────────────── packing ───────────────────────────── */

/* MLX affine bit stream: value i of a row occupies stream bits [i*b, (i+1)*b),
 * words little-endian, LSB first.  Equivalent to every pack helper in
 * Tests/FFAITests/Ops/QuantizedOpsTests.swift:33-124 (pack8, pack4Bytes,
 * pack16Twobit, pack16Sixbit, pack32Threebit, pack32Fivebit). */
ORC_EXPORT uint32_t orc_unpack(const uint32_t* row, int bits, int64_t i) {
    int64_t bit = i * bits;
    int64_t word = bit >> 5;
    int sh = (int)(bit & 31);
    uint64_t v = row[word];
    if (sh + bits > 32) v |= ((uint64_t)row[word + 1]) << 32;
    return (uint32_t)((v >> sh) & ((1u << bits) - 1u));
}

/* Inverse of orc_unpack: n values -> n*bits/32 words (n*bits must be a multiple of 32). */
ORC_EXPORT void orc_pack(const uint32_t* q, int64_t n, int bits, uint32_t* out) {
    int64_t words = n * bits / 32;
    memset(out, 0, (size_t)words * 4);
    for (int64_t i = 0; i < n; ++i) {
        int64_t bit = i * bits;
        int64_t word = bit >> 5;
        int sh = (int)(bit & 31);
        uint64_t v = ((uint64_t)(q[i] & ((1u << bits) - 1u))) << sh;
        out[word] |= (uint32_t)v;
        if (sh + bits > 32) out[word + 1] |= (uint32_t)(v >> 32);
    }
}

/* ───────────────────────────── exp ───────────────────────────── */

/* Fixed-sequence e^x for x <= ~88: n = rint(x*log2e); r = x - n*ln2 (two-step,
 * fused); degree-7 Taylor polynomial by Horner with fused multiply-add; scale
 * by 2^n through the exponent field.  Every step is a correctly rounded IEEE
 * operation, so any conforming implementation gives the same bits. */
ORC_EXPORT float orc_expf(float x) {
    if (!(x > -87.0f)) return 0.0f;
    if (x > 88.0f) x = 88.0f;
    float n = rintf(x * 1.44269504088896341f);
    float r = fmaf(n, -0.693145751953125f, x);
    r = fmaf(n, -1.42860682030941723e-6f, r);
    float p = 1.0f / 5040.0f;
    p = fmaf(p, r, 1.0f / 720.0f);
    p = fmaf(p, r, 1.0f / 120.0f);
    p = fmaf(p, r, 1.0f / 24.0f);
    p = fmaf(p, r, 1.0f / 6.0f);
    p = fmaf(p, r, 0.5f);
    p = fmaf(p, r, 1.0f);
    p = fmaf(p, r, 1.0f);
    int32_t e = (int32_t)n + 127;
    uint32_t sbits = ((uint32_t)e) << 23;
    float s;
    memcpy(&s, &sbits, 4);
    return p * s;
}

/* ───────────────────────────── router ───────────────────────────── */

/* MoERouter.softmax — Sources/FFAI/Models/MoELayer.swift:210-219
 * (GPTOSSText.swift:1449-1457 is the same function). */
static void softmax_small(const float* x, int n, float* out) {
    float maxv = x[0];
    for (int i = 1; i < n; ++i)
        if (x[i] > maxv) maxv = x[i];
    float sum = 0.0f;
    for (int i = 0; i < n; ++i) {
        out[i] = orc_expf(x[i] - maxv);
        sum = sum + out[i];
    }
    if (!(sum > 0.0f)) {
        for (int i = 0; i < n; ++i) out[i] = 1.0f / (float)n;
        return;
    }
    for (int i = 0; i < n; ++i) out[i] = out[i] / sum;
}

/* MoERouter.topKIndices — MoELayer.swift:223-296.  The reference keeps a
 * k-heap; its contract is "k largest, ordered value-desc then index-asc", which
 * repeated selection states directly (GPTOSSText.swift:1355-1358 sorts by the
 * same key). */
static void topk_indices(const float* x, int n, int k, int32_t* idx) {
    uint8_t* taken = (uint8_t*)calloc((size_t)n, 1);
    for (int j = 0; j < k; ++j) {
        int best = -1;
        for (int i = 0; i < n; ++i) {
            if (taken[i]) continue;
            if (best < 0 || x[i] > x[best]) best = i; /* strict > keeps the lower index on ties */
        }
        taken[best] = 1;
        idx[j] = best;
    }
    free(taken);
}

/* NemotronHMoELayer routing — Sources/FFAI/Models/Text/NemotronHText.swift:844-867: sigmoid of every logit,
 * selection on sigmoid + bias (order: value desc, index asc), weights = raw sigmoid of the selected, divided by
 * (their sum + 1e-20) when k > 1 and norm_topk_prob, times the routed scaling factor.  fp32 throughout, as the
 * reference's Float arrays. */
static void route_sigmoid(const float* logits, int n_experts, int k, int norm_topk_prob, const float* expert_bias,
                          float routed_scaling, int32_t* indices, float* weights) {
    float* orig = (float*)malloc(sizeof(float) * (size_t)n_experts);
    float* sel = (float*)malloc(sizeof(float) * (size_t)n_experts);
    for (int e = 0; e < n_experts; ++e) {
        orig[e] = 1.0f / (1.0f + orc_expf(-logits[e]));
        sel[e] = expert_bias ? orig[e] + expert_bias[e] : orig[e];
    }
    topk_indices(sel, n_experts, k, indices);
    for (int j = 0; j < k; ++j) weights[j] = orig[indices[j]];
    if (k > 1 && norm_topk_prob) {
        float sum = 0.0f;
        for (int j = 0; j < k; ++j) sum = sum + weights[j];
        sum = sum + 1e-20f;
        for (int j = 0; j < k; ++j) weights[j] = weights[j] / sum;
    }
    for (int j = 0; j < k; ++j) weights[j] = weights[j] * routed_scaling;
    free(orig); free(sel);
}

/* MoERouter.route — MoELayer.swift:140-205 (three branches, kept as written); routed_scaling applies to the
 * sigmoid mode only. */
ORC_EXPORT void orc_route_scaled(const float* logits, int n_experts, int k, int gating_mode,
                                 int norm_topk_prob, const float* expert_bias, float routed_scaling,
                                 int32_t* indices, float* weights);
ORC_EXPORT void orc_route(const float* logits, int n_experts, int k, int gating_mode,
                          int norm_topk_prob, const float* expert_bias, int32_t* indices,
                          float* weights) {
    orc_route_scaled(logits, n_experts, k, gating_mode, norm_topk_prob, expert_bias, 1.0f, indices, weights);
}
ORC_EXPORT void orc_route_scaled(const float* logits, int n_experts, int k, int gating_mode,
                                 int norm_topk_prob, const float* expert_bias, float routed_scaling,
                                 int32_t* indices, float* weights) {
    float picked[FFAI_MAX_TOP_K];
    if (gating_mode == FFAI_GATING_SIGMOID_TOPK) {
        route_sigmoid(logits, n_experts, k, norm_topk_prob, expert_bias, routed_scaling, indices, weights);
        return;
    }
    if ((gating_mode == FFAI_GATING_SOFTMAX_THEN_TOPK && norm_topk_prob && !expert_bias) ||
        gating_mode == FFAI_GATING_TOPK_THEN_SOFTMAX) {
        topk_indices(logits, n_experts, k, indices);
        for (int j = 0; j < k; ++j) picked[j] = logits[indices[j]];
        softmax_small(picked, k, weights);
        return;
    }
    float* gated = (float*)malloc(sizeof(float) * (size_t)n_experts);
    softmax_small(logits, n_experts, gated);
    if (expert_bias)
        for (int e = 0; e < n_experts; ++e) gated[e] = gated[e] + expert_bias[e];
    topk_indices(gated, n_experts, k, indices);
    for (int j = 0; j < k; ++j) weights[j] = gated[indices[j]];
    if (norm_topk_prob) {
        float sum = 0.0f;
        for (int j = 0; j < k; ++j) sum = sum + weights[j];
        if (sum > 0.0f)
            for (int j = 0; j < k; ++j) weights[j] = weights[j] / sum;
    }
    free(gated);
}

/* One weight of a dense-or-quantized [out,in] projection as fp32. */
static inline float linear_weight(const ffai_linear* lin, int kind, int bits, int gs,
                                  int64_t in_dim, int64_t o, int64_t i) {
    if (kind == FFAI_LINEAR_F32) return ((const float*)lin->weight)[o * in_dim + i];
    if (kind == FFAI_LINEAR_BF16)
        return orc_bf16_to_f32(((const uint16_t*)lin->weight)[o * in_dim + i]);
    const uint32_t* row = ((const uint32_t*)lin->weight) + o * (in_dim * bits / 32);
    int64_t g = o * (in_dim / gs) + i / gs;
    float q = (float)orc_unpack(row, bits, i);
    return fmaf(orc_bf16_to_f32(lin->scales[g]), q, orc_bf16_to_f32(lin->biases[g]));
}

/* Router projection (Layers.swift:78-84 dense, :201-210 quantized) in the fixed
 * chunk order described in the header comment, plus GPTOSSBiasedLinear's bias
 * (GPTOSSText.swift:341-362: a separate add in the activation dtype). */
ORC_EXPORT void orc_router_logits(const ffai_moe_config* c, const ffai_linear* router,
                                  const uint16_t* x, int n_tokens, float* logits) {
    const int H = c->hidden, E = c->n_experts;
#pragma omp parallel for schedule(static)
    for (int t = 0; t < n_tokens; ++t) {
        for (int e = 0; e < E; ++e) {
            float total = 0.0f;
            for (int k0 = 0; k0 < H; k0 += 64) {
                int k1 = k0 + 64 < H ? k0 + 64 : H;
                float p = 0.0f;
                for (int k = k0; k < k1; ++k) {
                    float w = linear_weight(router, c->router_kind, c->router_bits,
                                            c->router_group_size, H, e, k);
                    p = fmaf(orc_bf16_to_f32(x[(int64_t)t * H + k]), w, p);
                }
                total = total + p;
            }
            if (c->router_logits_bf16) total = bf16r(total);
            if (c->router_has_bias && router->bias) {
                total = total + orc_bf16_to_f32(router->bias[e]);
                if (c->router_logits_bf16) total = bf16r(total);
            }
            logits[(int64_t)t * E + e] = total;
        }
    }
}

/* ───────────────────────────── plan ───────────────────────────── */

/* Plan build of MoELayer.decodeMany — MoELayer.swift:752-792: tuples appended
 * token-major then slot, ordered by expert.  Swift's sort is not contractually
 * stable; the order kept here is the stable one (expert, token, slot). */
ORC_EXPORT void orc_plan(const uint32_t* indices, int n_tokens, int k, int n_experts,
                         uint32_t* counts, uint32_t* offsets, uint32_t* perm,
                         uint32_t* inv_perm) {
    int64_t m = (int64_t)n_tokens * k;
    for (int e = 0; e < n_experts; ++e) counts[e] = 0;
    for (int64_t i = 0; i < m; ++i) counts[indices[i]]++;
    offsets[0] = 0;
    for (int e = 0; e < n_experts; ++e) offsets[e + 1] = offsets[e] + counts[e];
    uint32_t* cursor = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)n_experts);
    for (int e = 0; e < n_experts; ++e) cursor[e] = offsets[e];
    for (int64_t i = 0; i < m; ++i) {
        uint32_t pos = cursor[indices[i]]++;
        perm[pos] = (uint32_t)i;
        inv_perm[i] = pos;
    }
    free(cursor);
}

/* ───────────────────────────── dequant products ───────────────────────────── */

/* Dequantise one packed row to fp32: w = scale*q + bias, as the reference's test
 * oracles do (MoEBgemmBm64MppTests.swift:100-106 `s * q + b`;
 * QuantizedOpsTests.swift:150-156 `(qv * s + b)`).  Separate multiply and add. */
static void dequant_row(const uint32_t* row, const uint16_t* scales, const uint16_t* biases,
                        int bits, int gs, int in_dim, float* w) {
    for (int g = 0; g < in_dim / gs; ++g) {
        float s = orc_bf16_to_f32(scales[g]);
        float b = orc_bf16_to_f32(biases[g]);
        for (int j = 0; j < gs; ++j) {
            int i = g * gs + j;
            float q = (float)orc_unpack(row, bits, i);
            w[i] = s * q + b;
        }
    }
}

/* fp32 accumulate in ascending k — MoEBgemmBm64MppTests.swift:95-110 (`acc += w * x`). */
static inline float dot_seq(const float* w, const float* x, int n) {
    float acc = 0.0f;
    for (int i = 0; i < n; ++i) acc += w[i] * x[i];
    return acc;
}

/* Ops.dequantGemv — CPU reference of QuantizedOpsTests.swift:143-158 and the
 * 3/5/6/8-bit cases (:195-438).  x fp32 in, out fp32. */
ORC_EXPORT void orc_dequant_gemv(const float* x, const uint32_t* weight, const uint16_t* scales,
                                 const uint16_t* biases, float* out, int out_dim, int in_dim,
                                 int bits, int gs) {
    float* w = (float*)malloc(sizeof(float) * (size_t)in_dim);
    for (int o = 0; o < out_dim; ++o) {
        dequant_row(weight + (int64_t)o * (in_dim * bits / 32), scales + (int64_t)o * (in_dim / gs),
                    biases + (int64_t)o * (in_dim / gs), bits, gs, in_dim, w);
        out[o] = dot_seq(w, x, in_dim);
    }
    free(w);
}

/* m1Oracle — MoEBgemmBm64MppTests.swift:82-114: per-row expert from indices[r],
 * stacked [E, N, K*bits/32] weights; generalised from 4-bit to any width. */
ORC_EXPORT void orc_gather_dequant_gemm(const float* x, const uint32_t* weight,
                                        const uint16_t* scales, const uint16_t* biases,
                                        const uint32_t* indices, float* out, int m_total,
                                        int n_out, int k_in, int n_experts, int bits, int gs) {
    (void)n_experts;
    int64_t wrow = (int64_t)k_in * bits / 32, grow = k_in / gs;
#pragma omp parallel
    {
        float* w = (float*)malloc(sizeof(float) * (size_t)k_in);
#pragma omp for schedule(dynamic, 8)
        for (int n = 0; n < n_out; ++n) {
            int64_t last_e = -1;
            for (int r = 0; r < m_total; ++r) {
                int64_t e = indices[r];
                if (e != last_e) {
                    dequant_row(weight + (e * n_out + n) * wrow, scales + (e * n_out + n) * grow,
                                biases + (e * n_out + n) * grow, bits, gs, k_in, w);
                    last_e = e;
                }
                out[(int64_t)r * n_out + n] = dot_seq(w, x + (int64_t)r * k_in, k_in);
            }
        }
        free(w);
    }
}

/* Activation on one (gate, up) pair. */
ORC_EXPORT float orc_glu(float g, float u, int activation, float limit, float alpha) {
    if (activation == FFAI_ACT_CLAMPED_SWIGLU) {
        /* GPTOSSMoELayer.runExpert host loop — GPTOSSText.swift:1421-1431. */
        if (g > limit) g = limit;
        if (u > limit) u = limit;
        if (u < -limit) u = -limit;
        float glu = g / (1.0f + expf(-alpha * g));
        return glu * (u + 1.0f);
    }
    if (activation == FFAI_ACT_GELU_GLU) {
        /* Ops.fusedGateGelu — OpsFused.swift:55-87: tanh-approximate GELU(gate)*up. */
        float inner = 0.7978845608028654f * (g + 0.044715f * g * g * g);
        return 0.5f * g * (1.0f + tanhf(inner)) * u;
    }
    /* MoELayerTests.swift:127-131 / Ops.swiglu Ops.swift:6400-6410: silu(g)*u in fp32. */
    float silu = g * (1.0f / (1.0f + expf(-g)));
    return silu * u;
}

/* Ops.moeUnpermute — Ops.swift:5030-5042; test case OpsSpecialPathTests.swift:1081-1124. */
ORC_EXPORT void orc_unpermute(const float* expert_out, const uint32_t* inv_perm,
                              const float* weights, float* out, int n_tokens, int hidden, int k) {
    for (int t = 0; t < n_tokens; ++t)
        for (int h = 0; h < hidden; ++h) {
            float acc = 0.0f;
            for (int s = 0; s < k; ++s)
                acc += weights[t * k + s] * expert_out[(int64_t)inv_perm[t * k + s] * hidden + h];
            out[(int64_t)t * hidden + h] = acc;
        }
}

/* ───────────────────────────── whole layer ───────────────────────────── */

typedef struct {
    const ffai_qproj* p;
    int bits, gs, out_dim, in_dim;
} proj_view;

static void proj_row(const proj_view* v, int64_t e, int o, float* w) {
    int64_t wrow = (int64_t)v->in_dim * v->bits / 32, grow = v->in_dim / v->gs;
    int64_t r = e * v->out_dim + o;
    dequant_row(v->p->weight + r * wrow, v->p->scales + r * grow, v->p->biases + r * grow, v->bits,
                v->gs, v->in_dim, w);
}

static inline float proj_bias(const proj_view* v, int64_t e, int o) {
    return v->p->row_bias ? orc_bf16_to_f32(v->p->row_bias[e * v->out_dim + o]) : 0.0f;
}

/* One SwiGLU-style expert over `cnt` input rows (fp32 copies of bf16 rows):
 * MoELayer.swiGLU — MoELayer.swift:1146-1155 (gate/up GEMV, activation, down GEMV),
 * GPTOSSMoELayer.runExpert — GPTOSSText.swift:1399-1445 (adds the row biases).
 * xs: [cnt][in]; ys: [cnt][H].  round_stages reproduces the reference's rounding
 * to the activation dtype at every tensor boundary. */
static void run_expert(const ffai_moe_config* c, const proj_view* pg, const proj_view* pu,
                       const proj_view* pd, int64_t e, const float* const* xs, float* const* ys,
                       int cnt, int round_stages) {
    const int H = pu->in_dim, I = pu->out_dim;
    /* experts without a gate projection (NemotronHExpert.forward, NemotronHText.swift:756-762): relu(up)^2 */
    const int no_gate = c->activation == FFAI_ACT_RELU2;
    float* wg = (float*)malloc(sizeof(float) * (size_t)(H > I ? H : I));
    float* wu = (float*)malloc(sizeof(float) * (size_t)H);
    float* inner = (float*)malloc(sizeof(float) * (size_t)cnt * I);
    for (int n = 0; n < I; ++n) {
        if (no_gate) {
            proj_row(pu, e, n, wu);
            float bu = proj_bias(pu, e, n);
            for (int r = 0; r < cnt; ++r) {
                float u = dot_seq(wu, xs[r], H);
                if (round_stages) u = bf16r(u);
                if (pu->p->row_bias) { u = u + bu; if (round_stages) u = bf16r(u); }
                float a = u > 0.0f ? u : 0.0f;
                if (round_stages) a = bf16r(a);
                a = a * a;
                if (round_stages) a = bf16r(a);
                inner[(int64_t)r * I + n] = a;
            }
            continue;
        }
        proj_row(pg, e, n, wg);
        proj_row(pu, e, n, wu);
        float bg = proj_bias(pg, e, n), bu = proj_bias(pu, e, n);
        for (int r = 0; r < cnt; ++r) {
            float g = dot_seq(wg, xs[r], H);
            float u = dot_seq(wu, xs[r], H);
            if (round_stages) { g = bf16r(g); u = bf16r(u); }
            if (pg->p->row_bias) { g = g + bg; if (round_stages) g = bf16r(g); }
            if (pu->p->row_bias) { u = u + bu; if (round_stages) u = bf16r(u); }
            float a = orc_glu(g, u, c->activation, c->swiglu_limit, c->swiglu_alpha);
            if (round_stages) a = bf16r(a);
            inner[(int64_t)r * I + n] = a;
        }
    }
    for (int h = 0; h < pd->out_dim; ++h) {
        proj_row(pd, e, h, wg);
        float bd = proj_bias(pd, e, h);
        for (int r = 0; r < cnt; ++r) {
            float y = dot_seq(wg, inner + (int64_t)r * I, I);
            if (round_stages) y = bf16r(y);
            if (pd->p->row_bias) { y = y + bd; if (round_stages) y = bf16r(y); }
            ys[r][h] = y;
        }
    }
    free(wg); free(wu); free(inner);
}

/*
 * The whole block.  Follows, in order:
 *   MoELayer.decode        MoELayer.swift:530-634 (router, route, per-expert SwiGLU,
 *                          weight*out then running add in slot order, shared expert)
 *   MoELayer.decodeMany    MoELayer.swift:677-969 (plan, gather, grouped products, unpermute)
 *   GPTOSSMoELayer.decode  GPTOSSText.swift:1340-1392
 *   Qwen35MoEFFN.forward   Qwen3xText.swift:928-1038 (sigmoid-gated shared expert, residual)
 * weights: HOST pointers.  token_mask (nullable, [T]): expert outputs are computed only
 * for tokens with a non-zero mask; routing and the plan always cover all tokens.
 * out_f32 (nullable) receives the un-rounded fp32 result, out_bf16 (nullable) the rounded one.
 */
ORC_EXPORT int orc_moe_forward_split(const ffai_moe_config* c, const ffai_moe_weights* w,
                                     const uint16_t* x, const uint16_t* x_router, int n_tokens, float* out_f32,
                                     uint16_t* out_bf16, const uint16_t* residual,
                                     const ffai_moe_debug* dbg, const uint8_t* token_mask,
                                     int round_stages, int n_threads);

ORC_EXPORT int orc_moe_forward(const ffai_moe_config* c, const ffai_moe_weights* w,
                               const uint16_t* x, int n_tokens, float* out_f32,
                               uint16_t* out_bf16, const uint16_t* residual,
                               const ffai_moe_debug* dbg, const uint8_t* token_mask,
                               int round_stages, int n_threads) {
    return orc_moe_forward_split(c, w, x, x, n_tokens, out_f32, out_bf16, residual, dbg, token_mask, round_stages, n_threads);
}

/* x_router: the rows the router reads (Gemma 4 normalises the router input and the expert input
 * differently, Gemma4Text.swift:929-933, 957); the logits are scaled by router_logit_scale before
 * routing (:937-943) and each combine weight by router_per_expert_scale[expert] (:944-949). */
ORC_EXPORT int orc_moe_forward_split(const ffai_moe_config* c, const ffai_moe_weights* w,
                                     const uint16_t* x, const uint16_t* x_router, int n_tokens, float* out_f32,
                                     uint16_t* out_bf16, const uint16_t* residual,
                                     const ffai_moe_debug* dbg, const uint8_t* token_mask,
                                     int round_stages, int n_threads) {
    const int H = c->hidden, I = c->intermediate, E = c->n_experts, K = c->top_k, T = n_tokens;
    if (T <= 0) return 0;
#ifdef _OPENMP
    if (n_threads > 0) omp_set_num_threads(n_threads);
#else
    (void)n_threads;
#endif
    const int64_t M = (int64_t)T * K;
    float* logits = (float*)malloc(sizeof(float) * (size_t)T * E);
    uint32_t* indices = (uint32_t*)malloc(4 * (size_t)M);
    float* rw = (float*)malloc(4 * (size_t)M);
    uint32_t* counts = (uint32_t*)malloc(4 * (size_t)E);
    uint32_t* offsets = (uint32_t*)malloc(4 * (size_t)(E + 1));
    uint32_t* perm = (uint32_t*)malloc(4 * (size_t)M);
    uint32_t* inv_perm = (uint32_t*)malloc(4 * (size_t)M);

    orc_router_logits(c, &w->router, x_router ? x_router : x, T, logits);
    const float logit_scale = c->router_logit_scale != 0.0f ? c->router_logit_scale : 1.0f;
    float* scaled = logit_scale != 1.0f ? (float*)malloc(sizeof(float) * (size_t)T * E) : NULL;
    if (scaled)
        for (int64_t i = 0; i < (int64_t)T * E; ++i) scaled[i] = logits[i] * logit_scale;
#pragma omp parallel for schedule(static)
    for (int t = 0; t < T; ++t) {
        int32_t idx[FFAI_MAX_TOP_K];
        orc_route_scaled((scaled ? scaled : logits) + (int64_t)t * E, E, K, c->gating_mode, c->norm_topk_prob,
                         c->router_expert_bias ? w->router_expert_bias : NULL,
                         c->routed_scaling_factor != 0.0f ? c->routed_scaling_factor : 1.0f, idx, rw + (int64_t)t * K);
        for (int s = 0; s < K; ++s) {
            indices[(int64_t)t * K + s] = (uint32_t)idx[s];
            if (w->router_per_expert_scale) rw[(int64_t)t * K + s] *= w->router_per_expert_scale[idx[s]];
        }
    }
    free(scaled);
    orc_plan(indices, T, K, E, counts, offsets, perm, inv_perm);
    if (dbg) {
        if (dbg->logits) memcpy(dbg->logits, logits, sizeof(float) * (size_t)T * E);
        if (dbg->indices) memcpy(dbg->indices, indices, 4 * (size_t)M);
        if (dbg->weights) memcpy(dbg->weights, rw, 4 * (size_t)M);
        if (dbg->counts) memcpy(dbg->counts, counts, 4 * (size_t)E);
        if (dbg->offsets) memcpy(dbg->offsets, offsets, 4 * (size_t)(E + 1));
        if (dbg->perm) memcpy(dbg->perm, perm, 4 * (size_t)M);
        if (dbg->inv_perm) memcpy(dbg->inv_perm, inv_perm, 4 * (size_t)M);
    }
    if (!out_f32 && !out_bf16) {
        free(logits); free(indices); free(rw); free(counts); free(offsets); free(perm); free(inv_perm);
        return 0;
    }

    /* fp32 copies of the (bf16) input rows. */
    float* xf = (float*)malloc(sizeof(float) * (size_t)T * H);
    for (int64_t i = 0; i < (int64_t)T * H; ++i) xf[i] = orc_bf16_to_f32(x[i]);
    float* y = (float*)calloc((size_t)M * H, sizeof(float)); /* expert outputs at sorted positions */

    proj_view pg = {&w->gate_proj, c->expert_bits, c->expert_group_size, I, H};
    proj_view pu = {&w->up_proj, c->expert_bits, c->expert_group_size, I, H};
    proj_view pd = {&w->down_proj, c->expert_bits, c->expert_group_size, H, I};

#pragma omp parallel for schedule(dynamic, 1)
    for (int e = 0; e < E; ++e) {
        int cnt = 0;
        const float** xs = (const float**)malloc(sizeof(float*) * (counts[e] + 1));
        float** ys = (float**)malloc(sizeof(float*) * (counts[e] + 1));
        for (uint32_t p = offsets[e]; p < offsets[e + 1]; ++p) {
            int t = (int)(perm[p] / (uint32_t)K);
            if (token_mask && !token_mask[t]) continue;
            xs[cnt] = xf + (int64_t)t * H;
            ys[cnt] = y + (int64_t)p * H;
            cnt++;
        }
        if (cnt) run_expert(c, &pg, &pu, &pd, e, xs, ys, cnt, round_stages);
        free(xs); free(ys);
    }

    /* Shared expert (MoELayer.swift:621-624; Qwen3xText.swift:939-1036). */
    float* sh = NULL;
    float* sgate = NULL;
    if (c->shared_intermediate > 0) {
        sh = (float*)calloc((size_t)T * H, sizeof(float));
        proj_view sg = {&w->shared_gate_proj, c->shared_bits, c->shared_group_size, c->shared_intermediate, H};
        proj_view su = {&w->shared_up_proj, c->shared_bits, c->shared_group_size, c->shared_intermediate, H};
        proj_view sd = {&w->shared_down_proj, c->shared_bits, c->shared_group_size, H, c->shared_intermediate};
        ffai_moe_config cs = *c;
        /* the shared expert is a plain SwiGLU MLP, or, beside gate-less experts, of their form (NemotronHText.swift:885-891) */
        cs.activation = c->activation == FFAI_ACT_RELU2 ? FFAI_ACT_RELU2 : FFAI_ACT_SWIGLU;
        int nthr = 1;
#ifdef _OPENMP
        nthr = omp_get_max_threads();
#endif
        /* split the token list into slices, one run_expert call per slice */
        int slices = nthr * 4 < T ? nthr * 4 : T;
#pragma omp parallel for schedule(dynamic, 1)
        for (int sl = 0; sl < slices; ++sl) {
            int t0 = (int)((int64_t)T * sl / slices), t1 = (int)((int64_t)T * (sl + 1) / slices);
            const float** xs = (const float**)malloc(sizeof(float*) * (size_t)(t1 - t0 + 1));
            float** ys = (float**)malloc(sizeof(float*) * (size_t)(t1 - t0 + 1));
            int cnt = 0;
            for (int t = t0; t < t1; ++t) {
                if (token_mask && !token_mask[t]) continue;
                xs[cnt] = xf + (int64_t)t * H;
                ys[cnt] = sh + (int64_t)t * H;
                cnt++;
            }
            if (cnt) run_expert(&cs, &sg, &su, &sd, 0, xs, ys, cnt, round_stages);
            free(xs); free(ys);
        }
        if (c->shared_gate_kind != FFAI_LINEAR_NONE) {
            sgate = (float*)malloc(sizeof(float) * (size_t)T);
            for (int t = 0; t < T; ++t) {
                float acc = 0.0f;
                for (int k = 0; k < H; ++k)
                    acc += linear_weight(&w->shared_gate, c->shared_gate_kind, c->shared_gate_bits,
                                         c->shared_gate_group_size, H, 0, k) * xf[(int64_t)t * H + k];
                if (round_stages) acc = bf16r(acc);
                sgate[t] = acc;
            }
        }
    }

    /* Combine: slot order (MoELayer.swift:601-617; Ops.moeUnpermute Ops.swift:5030-5042),
     * then the shared expert, then the optional residual
     * (sigmoidScalarFMAResidual, OpsFused.swift:699-753). */
#pragma omp parallel for schedule(static)
    for (int t = 0; t < T; ++t) {
        if (token_mask && !token_mask[t]) {
            for (int h = 0; h < H; ++h) {
                if (out_f32) out_f32[(int64_t)t * H + h] = 0.0f;
                if (out_bf16) out_bf16[(int64_t)t * H + h] = 0;
            }
            continue;
        }
        float sig = 1.0f;
        if (sgate) sig = 1.0f / (1.0f + expf(-sgate[t]));
        for (int h = 0; h < H; ++h) {
            float acc = 0.0f;
            for (int s = 0; s < K; ++s) {
                float wt = rw[(int64_t)t * K + s];
                float yv = y[(int64_t)inv_perm[(int64_t)t * K + s] * H + h];
                if (round_stages) {
                    float scaled = bf16r(bf16r(wt) * yv);
                    acc = (s == 0) ? scaled : bf16r(acc + scaled);
                } else {
                    acc += wt * yv;
                }
            }
            if (sh) {
                float sv = sh[(int64_t)t * H + h];
                acc = acc + sig * sv;
                if (round_stages) acc = bf16r(acc);
            }
            if (residual) acc = acc + orc_bf16_to_f32(residual[(int64_t)t * H + h]);
            if (out_f32) out_f32[(int64_t)t * H + h] = acc;
            if (out_bf16) out_bf16[(int64_t)t * H + h] = orc_f32_to_bf16(acc);
        }
    }

    free(xf); free(y); free(sh); free(sgate);
    free(logits); free(indices); free(rw); free(counts); free(offsets); free(perm); free(inv_perm);
    return 0;
}

ORC_EXPORT int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ───────────────────────── weight preparation (next rows) ───────────────────────── */

/* MXFP4 -> affine int4, group 32, as GPT-OSS checkpoints are transcoded at load time
 * (GPTOSSText.swift:943-956 constants, :1150-1226 the per-group fit).  Per group of 32 fp4 codes
 * (16 bytes, low nibble first) and one e8m0 byte:
 *   micro = 2^(e8m0 - 127); lo, hi = min / max of the code values (scan order: bytes ascending, low
 *   nibble then high nibble; strict comparisons, so the first zero met decides the sign of a zero
 *   minimum); bias = lo * micro; scale = (hi - lo) * micro / 15 (0 for a flat group);
 *   q = clamp(round_half_away(((value - lo) * (micro * (1 / scale)))), 0, 15), nibble for nibble.
 * Scale and bias are stored as bf16 (round to nearest even). */
static const float MXFP4_LUT[16] = {+0.0f, +0.5f, +1.0f, +1.5f, +2.0f, +3.0f, +4.0f, +6.0f,
                                    -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

ORC_EXPORT void orc_mxfp4_to_affine4(const uint8_t* packed, const uint8_t* e8m0, int64_t n_groups, uint8_t* out_packed,
                          uint16_t* out_scales, uint16_t* out_biases) {
#pragma omp parallel for schedule(static)
    for (int64_t g = 0; g < n_groups; ++g) {
        const float micro = (float)exp2((double)((int)e8m0[g] - 127));
        const uint8_t* src = packed + g * 16;
        float lo = 1e30f, hi = -1e30f;
        for (int b = 0; b < 16; ++b) {
            const float v0 = MXFP4_LUT[src[b] & 0x0F], v1 = MXFP4_LUT[src[b] >> 4];
            if (v0 < lo) lo = v0;
            if (v0 > hi) hi = v0;
            if (v1 < lo) lo = v1;
            if (v1 > hi) hi = v1;
        }
        const float aff_bias = lo * micro;
        const float span = (hi - lo) * micro;
        const float aff_scale = span > 0.0f ? span / 15.0f : 0.0f;
        const float inv_scale = aff_scale > 0.0f ? 1.0f / aff_scale : 0.0f;
        out_scales[g] = orc_f32_to_bf16(aff_scale);
        out_biases[g] = orc_f32_to_bf16(aff_bias);
        const float code_scale = micro * inv_scale;
        for (int b = 0; b < 16; ++b) {
            int q0 = (int)roundf((MXFP4_LUT[src[b] & 0x0F] - lo) * code_scale);
            int q1 = (int)roundf((MXFP4_LUT[src[b] >> 4] - lo) * code_scale);
            if (q0 < 0) q0 = 0;
            if (q0 > 15) q0 = 15;
            if (q1 < 0) q1 = 0;
            if (q1 > 15) q1 = 15;
            out_packed[g * 16 + b] = (uint8_t)(q0 | (q1 << 4));
        }
    }
}

/* MLX affine quantization of one [rows, K] matrix, bits in {2,3,4,5,6,8}, group size gs
 * (wrapper and shape rules: QuantizedOps.swift:229-388, QuantizedOpsValidation.swift:132-146).
 * The reference's kernel body is in the un-vendored metaltile project; what follows is MLX's published
 * affine_quantize (the algorithm the reference's format comes from), which the reference's own
 * tests constrain only through round-trip error bounds (QuantizedOpsAffineTests.swift:19-381):
 *   n = 2^bits - 1; scale = max((max - min) / n, 1e-7); the edge with the larger magnitude is kept
 *   exact: side = |min| > |max|; scale = side ? scale : -scale; edge = side ? min : max;
 *   q0 = round(edge / scale); if q0 != 0 { scale = edge / q0; bias = edge } else bias = 0;
 *   q = min(round((w - bias) / scale), n)   (fp32 scale and bias; bf16 copies are stored)
 * Values are packed LSB first.  Input and scale/bias are bf16 bit patterns. */
ORC_EXPORT void orc_affine_quantize(const uint16_t* w, int64_t rows, int K, int bits, int gs, uint32_t* out_packed,
                         uint16_t* out_scales, uint16_t* out_biases) {
    const int gpr = K / gs;
    const int64_t words_per_row = (int64_t)K * bits / 32;
    const float n_bins = (float)((1 << bits) - 1);
    memset(out_packed, 0, (size_t)(rows * words_per_row) * 4);
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        for (int g = 0; g < gpr; ++g) {
            const uint16_t* src = w + r * K + (int64_t)g * gs;
            float w_min = INFINITY, w_max = -INFINITY;
            for (int i = 0; i < gs; ++i) {
                const float v = orc_bf16_to_f32(src[i]);
                w_min = fminf(w_min, v);
                w_max = fmaxf(w_max, v);
            }
            float scale = fmaxf((w_max - w_min) / n_bins, 1e-7f);
            const int side = fabsf(w_min) > fabsf(w_max);
            scale = side ? scale : -scale;
            const float edge = side ? w_min : w_max;
            const float q0 = roundf(edge / scale);
            float bias = 0.0f;
            if (q0 != 0.0f) {
                scale = edge / q0;
                bias = edge;
            }
            out_scales[r * gpr + g] = orc_f32_to_bf16(scale);
            out_biases[r * gpr + g] = orc_f32_to_bf16(bias);
            for (int i = 0; i < gs; ++i) {
                const float v = orc_bf16_to_f32(src[i]);
                float q = roundf((v - bias) / scale);
                if (q > n_bins) q = n_bins;
                if (!(q >= 0.0f)) q = 0.0f;
                const uint32_t qi = (uint32_t)q;
                const int64_t bit = (int64_t)(g * gs + i) * bits;
                uint32_t* row = out_packed + r * words_per_row;
                row[bit >> 5] |= qi << (bit & 31);
                if ((bit & 31) + bits > 32) row[(bit >> 5) + 1] |= qi >> (32 - (bit & 31));
            }
        }
    }
}

/* residual = a + b; normed = (a + b) / sqrt(mean((a + b)^2) + eps) * weight, per row of n values.
 * Follows the CPU check of the reference's own test (OpsTests.swift:1042-1052): the sum of squares is
 * accumulated sequentially in float, the norm uses the unrounded sum.  bf16 bit patterns in and out.
 * b = NULL: the plain RMSNorm y = x / rms(x) * weight (LayersTests.swift:101-128 holds its CPU check). */
ORC_EXPORT void orc_add_rmsnorm(const uint16_t* a, const uint16_t* b, const uint16_t* weight, float eps, int n_rows, int n,
                                uint16_t* residual_out, uint16_t* normed_out, float* normed_f32) {
    for (int r = 0; r < n_rows; ++r) {
        float ssq = 0.0f;
        for (int d = 0; d < n; ++d) {
            const float s = orc_bf16_to_f32(a[(size_t)r * n + d]) + (b ? orc_bf16_to_f32(b[(size_t)r * n + d]) : 0.0f);
            ssq += s * s;
        }
        const float rms = sqrtf(ssq / (float)n + eps);
        for (int d = 0; d < n; ++d) {
            const float s = orc_bf16_to_f32(a[(size_t)r * n + d]) + (b ? orc_bf16_to_f32(b[(size_t)r * n + d]) : 0.0f);
            const float v = s / rms * orc_bf16_to_f32(weight[d]);
            if (residual_out) residual_out[(size_t)r * n + d] = orc_f32_to_bf16(s);
            normed_out[(size_t)r * n + d] = orc_f32_to_bf16(v);
            if (normed_f32) normed_f32[(size_t)r * n + d] = v;
        }
    }
}
