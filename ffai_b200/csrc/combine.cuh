// Weighted combine: a fixed-order per-token reduction over the k expert outputs,
// plus the (optionally sigmoid-gated) shared expert and the optional residual,
// with a single rounding to bf16 at the end.
//
// Replaces Ops.moeUnpermute (FFAI Ops.swift:5030-5110), the mul/add chain of the
// CPU-router path (MoELayer.swift:601-617), the shared-expert add (:621-624) and
// Ops.sigmoidScalarFMA[Residual] (Ops.swift:6255-6334, OpsFused.swift:699-753).
// Slot order is the router's order (value desc, index asc), so the sum is the
// same whatever the launch geometry.
#pragma once
#include "common.cuh"

namespace ffai {

FFAI_DEVINL float4 load4(const float* p) { return *(const float4*)p; }
FFAI_DEVINL float4 load4(const uint16_t* p) {
    uint2 u = *(const uint2*)p;
    return make_float4(bf16lo(u.x), bf16hi(u.x), bf16lo(u.y), bf16hi(u.y));
}

// One block per token; a thread owns 4 consecutive hidden positions.
template <typename TY, typename TS>
__global__ void __launch_bounds__(256)
combine_kernel(const TY* __restrict__ y, const uint32_t* __restrict__ inv_perm,
               const float* __restrict__ weights, int k, const TS* __restrict__ shared_y,
               const float* __restrict__ shared_gate_logit, const uint16_t* __restrict__ residual,
               uint16_t* __restrict__ out, int hidden) {
    const int t = blockIdx.x;
    __shared__ uint32_t pos_s[32];
    __shared__ float w_s[32];
    __shared__ float sig_s;
    pdl_wait();
    if (threadIdx.x < k) {
        pos_s[threadIdx.x] = inv_perm[(size_t)t * k + threadIdx.x];
        w_s[threadIdx.x] = weights[(size_t)t * k + threadIdx.x];
    }
    if (threadIdx.x == 0) {
        float sig = 1.0f;
        if (shared_gate_logit) sig = 1.0f / (1.0f + __expf(-shared_gate_logit[t]));
        sig_s = sig;
    }
    __syncthreads();
    for (int h = threadIdx.x * 4; h < hidden; h += blockDim.x * 4) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s = 0; s < k; ++s) {
            const float w = w_s[s];
            const float4 v = load4(y + (size_t)pos_s[s] * hidden + h);
            acc.x += w * v.x; acc.y += w * v.y; acc.z += w * v.z; acc.w += w * v.w;
        }
        if (shared_y) {
            const float sig = sig_s;
            const float4 v = load4(shared_y + (size_t)t * hidden + h);
            acc.x += sig * v.x; acc.y += sig * v.y; acc.z += sig * v.z; acc.w += sig * v.w;
        }
        if (residual) {
            const float4 v = load4(residual + (size_t)t * hidden + h);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        uint2 o;
        o.x = (uint32_t)f32_to_bf16_bits(acc.x) | ((uint32_t)f32_to_bf16_bits(acc.y) << 16);
        o.y = (uint32_t)f32_to_bf16_bits(acc.z) | ((uint32_t)f32_to_bf16_bits(acc.w) << 16);
        *(uint2*)(out + (size_t)t * hidden + h) = o;
    }
}

// out[t,:] = [residual[t,:] +] base[t,:] + sigmoid(gate[t]) * value[t,:], all bf16.
__global__ void sigmoid_scalar_fma_kernel(const uint16_t* __restrict__ gate,
                                          const uint16_t* __restrict__ value,
                                          const uint16_t* __restrict__ base,
                                          const uint16_t* __restrict__ residual,
                                          uint16_t* __restrict__ out, int hidden) {
    const int t = blockIdx.x;
    const float sig = 1.0f / (1.0f + __expf(-bf16_bits_to_f32(gate[t])));
    for (int h = threadIdx.x; h < hidden; h += blockDim.x) {
        const size_t i = (size_t)t * hidden + h;
        float v = bf16_bits_to_f32(base[i]) + sig * bf16_bits_to_f32(value[i]);
        if (residual) v += bf16_bits_to_f32(residual[i]);
        out[i] = f32_to_bf16_bits(v);
    }
}

}  // namespace ffai
