// Token dispatch plan: per-expert histogram, exclusive prefix scan, and a
// deterministic (stable) scatter of the T*k (token, slot) entries into
// expert-contiguous order.
//
// Replaces the host-side plan build of MoELayer.decodeMany (FFAI
// MoELayer.swift:752-792: tuple list, sort by expert, invPerm) and the four
// host->device copies that follow it (:826-839, :912-935).  The order is the
// stable one — by (expert, token, slot) — and does not depend on the order in
// which blocks or atomics execute: each warp owns a contiguous run of entries,
// ranks them with warp match operations in entry order, and block bases come
// from a scan over per-warp histograms.
#pragma once
#include "common.cuh"

namespace ffai {

constexpr int PLAN_ENTRIES_PER_WARP = 1024;  // entries ranked by one warp (one block)

// Workspace: block_hist [nblocks][E] u32.
__host__ __device__ inline int plan_num_blocks(int n_rows) {
    return (n_rows + PLAN_ENTRIES_PER_WARP - 1) / PLAN_ENTRIES_PER_WARP;
}

// Pass 1: histogram of each block's run.  Integer adds commute, so shared-memory
// atomics are deterministic here.
__global__ void plan_count_kernel(const uint32_t* __restrict__ indices, int n_rows, int n_experts,
                                  uint32_t* __restrict__ block_hist) {
    extern __shared__ uint32_t hist[];
    for (int e = threadIdx.x; e < n_experts; e += 32) hist[e] = 0;
    __syncwarp();
    const int base = blockIdx.x * PLAN_ENTRIES_PER_WARP;
    const int end = min(base + PLAN_ENTRIES_PER_WARP, n_rows);
    for (int i = base + threadIdx.x; i < end; i += 32) {
        uint32_t e = indices[i];
        if (e < (uint32_t)n_experts) atomicAdd(&hist[e], 1u);
    }
    __syncwarp();
    for (int e = threadIdx.x; e < n_experts; e += 32)
        block_hist[(size_t)blockIdx.x * n_experts + e] = hist[e];
}

// Pass 2 (one block): per expert, running sum over blocks -> block bases;
// totals -> counts; exclusive scan over experts -> offsets; bases made absolute.
__global__ void plan_scan_kernel(uint32_t* __restrict__ block_hist, int n_blocks, int n_experts,
                                 uint32_t* __restrict__ counts, uint32_t* __restrict__ offsets) {
    extern __shared__ uint32_t totals[];  // [E+1]
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
        uint32_t run = 0;
        for (int b = 0; b < n_blocks; ++b) {
            uint32_t c = block_hist[(size_t)b * n_experts + e];
            block_hist[(size_t)b * n_experts + e] = run;
            run += c;
        }
        totals[e] = run;
        counts[e] = run;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t run = 0;
        for (int e = 0; e < n_experts; ++e) {
            uint32_t c = totals[e];
            totals[e] = run;
            offsets[e] = run;
            run += c;
        }
        offsets[n_experts] = run;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
        const uint32_t off = totals[e];
        for (int b = 0; b < n_blocks; ++b) block_hist[(size_t)b * n_experts + e] += off;
    }
}

// Pass 3: each warp ranks its run in entry order.
__global__ void plan_scatter_kernel(const uint32_t* __restrict__ indices, int n_rows, int n_experts,
                                    const uint32_t* __restrict__ block_base,
                                    uint32_t* __restrict__ perm, uint32_t* __restrict__ inv_perm) {
    extern __shared__ uint32_t cursor[];  // [E]
    const int lane = threadIdx.x;
    for (int e = lane; e < n_experts; e += 32)
        cursor[e] = block_base[(size_t)blockIdx.x * n_experts + e];
    __syncwarp();
    const int base = blockIdx.x * PLAN_ENTRIES_PER_WARP;
    const int end = min(base + PLAN_ENTRIES_PER_WARP, n_rows);
    for (int i0 = base; i0 < end; i0 += 32) {
        const int i = i0 + lane;
        const bool valid = i < end;
        uint32_t e = valid ? indices[i] : 0xFFFFFFFFu;
        if (valid && e >= (uint32_t)n_experts) e = 0xFFFFFFFEu;  // corrupt id: dropped
        const uint32_t peers = __match_any_sync(0xFFFFFFFFu, e);
        const uint32_t rank = __popc(peers & ((1u << lane) - 1u));
        uint32_t pos = 0;
        const bool real = valid && e < (uint32_t)n_experts;
        if (real) pos = cursor[e] + rank;
        __syncwarp();
        if (real && rank == 0) cursor[e] += __popc(peers);
        __syncwarp();
        if (real) {
            perm[pos] = (uint32_t)i;
            inv_perm[i] = pos;
        }
    }
}

// Where a plan goes (all device pointers).
struct PlanOut {
    uint32_t* counts;    // [E]
    uint32_t* offsets;   // [E+1]
    uint32_t* perm;      // [n_rows]
    uint32_t* inv_perm;  // [n_rows]
    uint32_t* order;     // nullable [E]: experts by descending row count (ties: ascending index), for kernels that
                         // want their longest work items scheduled first
};

// The whole plan by one warp, for small row counts (decode): histogram, exclusive scan, stable scatter.
// hist and cursor: n_experts words of shared memory each.  indices are read past L1 (they may have
// been written by other blocks of the same launch).  n_rows <= PLAN_ENTRIES_PER_WARP.
FFAI_DEVINL void plan_small_warp(const uint32_t* indices, int n_rows, int n_experts, const PlanOut& o,
                                 uint32_t* hist, uint32_t* cursor, int lane) {
    for (int e = lane; e < n_experts; e += 32) hist[e] = 0;
    __syncwarp();
    for (int i = lane; i < n_rows; i += 32) {
        uint32_t e = __ldcg(indices + i);
        if (e < (uint32_t)n_experts) atomicAdd(&hist[e], 1u);
    }
    __syncwarp();
    // exclusive scan over experts, 32 at a time
    uint32_t carry = 0;
    for (int e0 = 0; e0 < n_experts; e0 += 32) {
        const int e = e0 + lane;
        const uint32_t c = (e < n_experts) ? hist[e] : 0u;
        uint32_t incl = c;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            uint32_t v = __shfl_up_sync(0xFFFFFFFFu, incl, d);
            if (lane >= d) incl += v;
        }
        if (e < n_experts) {
            o.counts[e] = c;
            o.offsets[e] = carry + incl - c;
            cursor[e] = carry + incl - c;
        }
        carry += __shfl_sync(0xFFFFFFFFu, incl, 31);
    }
    if (lane == 0) o.offsets[n_experts] = carry;
    __syncwarp();
    if (o.order) {   // rank of expert e = experts with more rows, or as many and a smaller index (E^2 / 32 compares per lane)
        for (int e = lane; e < n_experts; e += 32) {
            const uint32_t c = hist[e];
            int rank = 0;
            for (int f = 0; f < n_experts; ++f) {
                const uint32_t d = hist[f];
                rank += (d > c) || (d == c && f < e);
            }
            o.order[rank] = (uint32_t)e;
        }
    }
    for (int i0 = 0; i0 < n_rows; i0 += 32) {
        const int i = i0 + lane;
        const bool valid = i < n_rows;
        uint32_t e = valid ? __ldcg(indices + i) : 0xFFFFFFFFu;
        if (valid && e >= (uint32_t)n_experts) e = 0xFFFFFFFEu;
        const uint32_t peers = __match_any_sync(0xFFFFFFFFu, e);
        const uint32_t rank = __popc(peers & ((1u << lane) - 1u));
        const bool real = valid && e < (uint32_t)n_experts;
        uint32_t pos = 0;
        if (real) pos = cursor[e] + rank;
        __syncwarp();
        if (real && rank == 0) cursor[e] += __popc(peers);
        __syncwarp();
        if (real) {
            o.perm[pos] = (uint32_t)i;
            o.inv_perm[i] = pos;
        }
    }
}

// Single-launch variant for small row counts (decode): one warp does all three passes.
__global__ void plan_small_kernel(const uint32_t* __restrict__ indices, int n_rows, int n_experts,
                                  uint32_t* __restrict__ counts, uint32_t* __restrict__ offsets,
                                  uint32_t* __restrict__ perm, uint32_t* __restrict__ inv_perm) {
    extern __shared__ uint32_t sm[];  // hist[E], cursor[E]
    const PlanOut o{counts, offsets, perm, inv_perm, nullptr};
    plan_small_warp(indices, n_rows, n_experts, o, sm, sm + n_experts, threadIdx.x);
}

// Ops.gather (FFAI Ops.swift:308-346) specialised to the dispatch: row `pos` of the
// expert-contiguous buffer is the input row of token perm[pos]/k.  One warp per
// row, 16-byte copies; row_len is a multiple of 8 bf16.
__global__ void gather_rows_kernel(const uint16_t* __restrict__ table, const uint32_t* __restrict__ ids,
                                   int id_div, uint16_t* __restrict__ out, int n_rows, int row_len) {
    const int warps = blockDim.x / 32;
    const int row = blockIdx.x * warps + threadIdx.x / 32;
    if (row >= n_rows) return;
    const int lane = threadIdx.x & 31;
    const uint32_t src = ids[row] / (uint32_t)id_div;
    const uint4* s = (const uint4*)(table + (size_t)src * row_len);
    uint4* d = (uint4*)(out + (size_t)row * row_len);
    for (int i = lane; i < row_len / 8; i += 32) d[i] = s[i];
}

}  // namespace ffai
