// Weight preparation on the GPU: the MXFP4 -> affine-int4 transcode GPT-OSS checkpoints need, and the
// MLX affine quantizer.  Both are streaming, HBM-bound kernels; both replace host loops of the reference.
#pragma once
#include "common.cuh"

namespace ffai {
namespace prep {

// fp4 (e2m1) code -> value (0, .5, 1, 1.5, 2, 3, 4, 6; the top bit is the sign: FFAI GPTOSSText.swift:948-953),
// built from the code's fields: exponent field 0 is the subnormal pair {0, 0.5}.
FFAI_DEVINL float mxfp4_value(uint32_t code) {
    const uint32_t ex = (code >> 1) & 3u, man = code & 1u;
    const uint32_t mag = ex ? (((ex + 126u) << 23) | (man << 22)) : (man ? 0x3F000000u : 0u);
    return __uint_as_float(mag | ((code & 8u) << 28));
}

// One thread per group of 32 codes (16 bytes in, 16 bytes + two bf16 out): the per-group min/max fit
// and nibble-for-nibble remap of the reference's load-time transcode
// (FFAI GPTOSSText.swift:1150-1226; there a host loop over ~20 billion codes per checkpoint).
// Same operations in the same order in fp32, so every output bit matches the host version:
// scan order bytes ascending, low nibble first, strict comparisons.  Scale bytes whose power of two
// leaves the fp32 range (the reference traps on them) are not given a meaning here either.
__global__ void __launch_bounds__(256)
mxfp4_to_affine4_kernel(const uint4* __restrict__ packed, const uint8_t* __restrict__ e8m0,
                        long n_groups, uint4* __restrict__ out_packed,
                        uint16_t* __restrict__ out_scales, uint16_t* __restrict__ out_biases) {
    const long g = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= n_groups) return;
    const uint32_t eb = e8m0[g];
    // 2^(e - 127): e = 0 is the subnormal 2^-127, e = 255 overflows to +inf, as the host table does
    const float micro = eb == 0 ? __uint_as_float(0x00400000u) : __uint_as_float(eb << 23);
    const uint4 src = packed[g];
    const uint32_t w[4] = {src.x, src.y, src.z, src.w};
    float v[32];
    float lo = 1e30f, hi = -1e30f;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int n = 0; n < 8; ++n) {   // nibble n of word i = byte n/2, low nibble first
            const float x = mxfp4_value((w[i] >> (4 * n)) & 15u);
            v[i * 8 + n] = x;
            if (x < lo) lo = x;
            if (x > hi) hi = x;
        }
    const float aff_bias = __fmul_rn(lo, micro);
    const float span = __fmul_rn(__fsub_rn(hi, lo), micro);
    const float aff_scale = span > 0.0f ? __fdiv_rn(span, 15.0f) : 0.0f;
    const float inv_scale = aff_scale > 0.0f ? __fdiv_rn(1.0f, aff_scale) : 0.0f;
    out_scales[g] = f32_to_bf16_bits(aff_scale);
    out_biases[g] = f32_to_bf16_bits(aff_bias);
    const float code_scale = __fmul_rn(micro, inv_scale);
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t acc = 0;
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            // values are >= 0 here, so round-half-away is floor(t + 0.5) unless the sum itself rounds up:
            // use the exact library rounding to stay bit-identical
            int q = (int)roundf(__fmul_rn(__fsub_rn(v[i * 8 + n], lo), code_scale));
            q = min(max(q, 0), 15);
            acc |= (uint32_t)q << (4 * n);
        }
        o[i] = acc;
    }
    out_packed[g] = make_uint4(o[0], o[1], o[2], o[3]);
}

// MLX affine quantization, one thread per group of GS values of a [rows, K] bf16 matrix (the reference's
// wrapper: FFAI QuantizedOps.swift:229-388).  The edge of larger magnitude is represented exactly;
// fp32 scale and bias quantize, their bf16 roundings are stored.  Codes are packed LSB first into the
// group's own words (GS * BITS is a multiple of 32 for every allowed pair), 16-byte loads of the input.
template <int BITS>
__global__ void __launch_bounds__(128)
affine_quantize_kernel(const uint16_t* __restrict__ w, long n_groups, int group_size, uint32_t* __restrict__ out_packed,
                       uint16_t* __restrict__ out_scales, uint16_t* __restrict__ out_biases) {
    const long g = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= n_groups) return;
    const uint4* src = reinterpret_cast<const uint4*>(w + g * group_size);
    const int chunks = group_size / 8;               // 16-byte pieces: 4, 8 or 16
    float w_min = INFINITY, w_max = -INFINITY;
    for (int c = 0; c < chunks; ++c) {
        const uint4 u = __ldg(src + c);
        const uint32_t p[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float a = bf16lo(p[i]), b = bf16hi(p[i]);
            w_min = fminf(w_min, fminf(a, b));
            w_max = fmaxf(w_max, fmaxf(a, b));
        }
    }
    const float n_bins = (float)((1 << BITS) - 1);
    float scale = fmaxf(__fdiv_rn(__fsub_rn(w_max, w_min), n_bins), 1e-7f);
    const bool side = fabsf(w_min) > fabsf(w_max);
    scale = side ? scale : -scale;
    const float edge = side ? w_min : w_max;
    const float q0 = roundf(__fdiv_rn(edge, scale));
    float bias = 0.0f;
    if (q0 != 0.0f) {
        scale = __fdiv_rn(edge, q0);
        bias = edge;
    }
    out_scales[g] = f32_to_bf16_bits(scale);
    out_biases[g] = f32_to_bf16_bits(bias);
    uint32_t* dst = out_packed + g * (group_size * BITS / 32);
    uint64_t acc = 0;
    int filled = 0;
    for (int c = 0; c < chunks; ++c) {
        const uint4 u = __ldg(src + c);              // second pass over the group: L1 / L2 hits
        const uint32_t p[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float x = (i & 1) ? bf16hi(p[i >> 1]) : bf16lo(p[i >> 1]);
            float q = roundf(__fdiv_rn(__fsub_rn(x, bias), scale));
            if (q > n_bins) q = n_bins;
            if (!(q >= 0.0f)) q = 0.0f;
            acc |= (uint64_t)(uint32_t)q << filled;
            filled += BITS;
            if (filled >= 32) {
                *dst++ = (uint32_t)acc;
                acc >>= 32;
                filled -= 32;
            }
        }
    }
}

// The step in front of the block: residual = a + b, normed = RMSNorm(a + b) * weight, one pass
// (FFAI Ops.addAndRmsNorm, Ops.swift:658-760; GPT-OSS calls it right before the MoE block,
// GPTOSSText.swift:700-716).  bf16 in and out; the sum, the mean of squares and the scaling are fp32
// and the norm is taken from the unrounded sum, as in the reference's CPU check
// (OpsTests.swift:1042-1052).  One block per row; a thread owns 4 consecutive positions per step.
__global__ void __launch_bounds__(256)
add_rmsnorm_kernel(const uint16_t* __restrict__ a, const uint16_t* __restrict__ b, const uint16_t* __restrict__ weight,
                   float eps, int n, uint16_t* __restrict__ residual_out, uint16_t* __restrict__ normed_out) {
    const size_t row = blockIdx.x;
    const uint16_t* ar = a + row * n;
    const uint16_t* br = b ? b + row * n : nullptr;   // no second addend: a plain RMSNorm of a
    __shared__ float red[8];
    float ssq = 0.0f;
    for (int h = threadIdx.x * 4; h < n; h += blockDim.x * 4) {
        const uint2 ua = *reinterpret_cast<const uint2*>(ar + h);
        const uint2 ub = br ? *reinterpret_cast<const uint2*>(br + h) : make_uint2(0u, 0u);
        const float s0 = bf16lo(ua.x) + bf16lo(ub.x), s1 = bf16hi(ua.x) + bf16hi(ub.x);
        const float s2 = bf16lo(ua.y) + bf16lo(ub.y), s3 = bf16hi(ua.y) + bf16hi(ub.y);
        ssq += (s0 * s0 + s1 * s1) + (s2 * s2 + s3 * s3);
    }
    ssq = warp_sum(ssq);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ssq;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) total += red[w];
    const float inv_rms = 1.0f / sqrtf(total / (float)n + eps);
    for (int h = threadIdx.x * 4; h < n; h += blockDim.x * 4) {
        const uint2 ua = *reinterpret_cast<const uint2*>(ar + h);
        const uint2 ub = br ? *reinterpret_cast<const uint2*>(br + h) : make_uint2(0u, 0u);
        const uint2 uw = *reinterpret_cast<const uint2*>(weight + h);
        const float s0 = bf16lo(ua.x) + bf16lo(ub.x), s1 = bf16hi(ua.x) + bf16hi(ub.x);
        const float s2 = bf16lo(ua.y) + bf16lo(ub.y), s3 = bf16hi(ua.y) + bf16hi(ub.y);
        uint2 r, o;
        r.x = (uint32_t)f32_to_bf16_bits(s0) | ((uint32_t)f32_to_bf16_bits(s1) << 16);
        r.y = (uint32_t)f32_to_bf16_bits(s2) | ((uint32_t)f32_to_bf16_bits(s3) << 16);
        o.x = (uint32_t)f32_to_bf16_bits(s0 * inv_rms * bf16lo(uw.x)) | ((uint32_t)f32_to_bf16_bits(s1 * inv_rms * bf16hi(uw.x)) << 16);
        o.y = (uint32_t)f32_to_bf16_bits(s2 * inv_rms * bf16lo(uw.y)) | ((uint32_t)f32_to_bf16_bits(s3 * inv_rms * bf16hi(uw.y)) << 16);
        if (residual_out) *reinterpret_cast<uint2*>(residual_out + row * n + h) = r;
        *reinterpret_cast<uint2*>(normed_out + row * n + h) = o;
    }
}

}  // namespace prep
}  // namespace ffai
