// Shared device helpers for libffai_cuda (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ffai {

#define FFAI_DEVINL __device__ __forceinline__

// The opt-in shared-memory size of a kernel is a per-device attribute.  One of these per kernel
// instantiation (a function-local static) remembers the largest size set on each device, so a
// process that drives several GPUs sets it on each of them.
struct SmemOptIn {
    int set[64] = {};
    template <typename K>
    bool ensure(K kernel, int bytes) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
        if (bytes <= set[dev]) return true;
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return false;
        set[dev] = bytes;
        return true;
    }
};

// Programmatic dependent launch (a kernel launched with the programmatic-stream-serialization attribute may start
// while its predecessor in the stream is still running): `pdl_wait` blocks until the predecessor has completed and
// its memory is visible; everything before it must not read what the predecessor writes.  `pdl_launch_dependents`
// lets the successor's blocks be scheduled as this kernel's blocks retire.  Both are no-ops in a plain launch.
FFAI_DEVINL void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
FFAI_DEVINL void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// bf16 bit pattern <-> fp32.  Same rule as FFAI's Tensor.swift:107-113,145-150
// (round to nearest even on the bit pattern).
FFAI_DEVINL float bf16_bits_to_f32(uint16_t b) { return __uint_as_float(((uint32_t)b) << 16); }
FFAI_DEVINL uint16_t f32_to_bf16_bits(float f) {
    uint32_t bits = __float_as_uint(f);
    uint32_t rounded = bits + 0x7FFFu + ((bits >> 16) & 1u);
    return (uint16_t)(rounded >> 16);
}
FFAI_DEVINL float bf16_round(float f) { return bf16_bits_to_f32(f32_to_bf16_bits(f)); }

// Two bf16 values packed in one 32-bit word -> two floats (low half first).
FFAI_DEVINL float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
FFAI_DEVINL float bf16hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// e^x as a fixed sequence of correctly rounded IEEE operations (round-to-int,
// two-step Cody-Waite reduction with fused multiply-add, degree-7 Horner
// polynomial, exponent-field scaling).  Any conforming implementation that runs
// the same sequence produces the same bits, which is what makes the combine
// weights reproducible between host and device.
FFAI_DEVINL float det_expf(float x) {
    if (!(x > -87.0f)) return 0.0f;
    if (x > 88.0f) x = 88.0f;
    float n = rintf(__fmul_rn(x, 1.44269504088896341f));
    float r = __fmaf_rn(n, -0.693145751953125f, x);
    r = __fmaf_rn(n, -1.42860682030941723e-6f, r);
    float p = 1.0f / 5040.0f;
    p = __fmaf_rn(p, r, 1.0f / 720.0f);
    p = __fmaf_rn(p, r, 1.0f / 120.0f);
    p = __fmaf_rn(p, r, 1.0f / 24.0f);
    p = __fmaf_rn(p, r, 1.0f / 6.0f);
    p = __fmaf_rn(p, r, 0.5f);
    p = __fmaf_rn(p, r, 1.0f);
    p = __fmaf_rn(p, r, 1.0f);
    int e = (int)n + 127;
    float s = __uint_as_float(((uint32_t)e) << 23);
    return __fmul_rn(p, s);
}

// Value i of an LSB-first bit stream of BITS-bit values held in `w` (little-endian
// words; the MLX affine layout).  `w` must hold the words the value touches.
template <int BITS>
FFAI_DEVINL uint32_t unpack_at(const uint32_t* w, int i) {
    const int bit = i * BITS;
    const int word = bit >> 5;
    const int sh = bit & 31;
    uint32_t lo = w[word];
    if (sh + BITS > 32) {
        uint32_t hi = w[word + 1];
        return __funnelshift_r(lo, hi, sh) & ((1u << BITS) - 1u);
    }
    return (lo >> sh) & ((1u << BITS) - 1u);
}

// Small unsigned integer -> float without the slow integer convert: OR the value
// into the mantissa of 2^23 and subtract 2^23 (exact for q < 2^23).
FFAI_DEVINL float small_uint_to_float(uint32_t q) {
    return __uint_as_float(0x4B000000u | q) - 8388608.0f;
}

// The same activations with the kind fixed at compile time, for loops that branch once outside.
template <int ACT>
FFAI_DEVINL float glu_activation_t(float g, float u, float limit, float alpha) {
    if (ACT == 1) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return __fdividef(g, 1.0f + __expf(-alpha * g)) * (u + 1.0f);
    }
    if (ACT == 2) {
        const float inner = 0.7978845608028654f * (g + 0.044715f * g * g * g);
        return 0.5f * g * (1.0f + tanhf(inner)) * u;
    }
    return __fdividef(g, 1.0f + __expf(-g)) * u;
}

// Epilogue variants with one special-function instruction per element: sigmoid(z) = 0.5 + 0.5 tanh(z/2)
// with the hardware tanh (relative error about 2^-11, far below the bf16 rounding of the result).
FFAI_DEVINL float tanh_fast(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
template <int ACT>
FFAI_DEVINL float glu_activation_fast(float g, float u, float limit, float alpha) {
    if (ACT == 1) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        const float hg = 0.5f * g;
        return fmaf(hg, tanh_fast(alpha * hg), hg) * (u + 1.0f);
    }
    if (ACT == 2) {
        const float inner = 0.7978845608028654f * (g + 0.044715f * g * g * g);
        const float hg = 0.5f * g;
        return fmaf(hg, tanh_fast(inner), hg) * u;
    }
    const float hg = 0.5f * g;
    return fmaf(hg, tanh_fast(hg), hg) * u;
}

FFAI_DEVINL float warp_sum(float v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, m);
    return v;
}

// Expert activation on one (gate, up) pair; fp32 math with the fast exponential and reciprocal
// (a few ulp; the epilogue that calls this shares issue slots with the dequant warps).
//   0 SwiGLU          silu(g)*u                      (FFAI Ops.swift:6400-6452)
//   1 clamped SwiGLU  GPT-OSS host loop              (FFAI GPTOSSText.swift:1421-1431)
//   2 GELU-GLU        tanh-approximate gelu(g)*u     (FFAI OpsFused.swift:55-87)
FFAI_DEVINL float glu_activation(float g, float u, int activation, float limit, float alpha) {
    if (activation == 1) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        float glu = __fdividef(g, 1.0f + __expf(-alpha * g));
        return glu * (u + 1.0f);
    }
    if (activation == 2) {
        float inner = 0.7978845608028654f * (g + 0.044715f * g * g * g);
        return 0.5f * g * (1.0f + tanhf(inner)) * u;
    }
    float silu = __fdividef(g, 1.0f + __expf(-g));
    return silu * u;
}

}  // namespace ffai
