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

// Pass 2 (one block): per expert, totals over blocks -> counts; exclusive scans over experts (rows and, when
// tile_offsets is given, token tiles of tile_rows rows) by one warp with shuffles; then per expert the running
// sum over blocks, offset by the expert's base -> absolute block bases.  The loads of a pass are issued in
// batches before anything that depends on them, so a pass costs a few memory round trips, not one per block.
__global__ void plan_scan_kernel(uint32_t* __restrict__ block_hist, int n_blocks, int n_experts,
                                 uint32_t* __restrict__ counts, uint32_t* __restrict__ offsets,
                                 int tile_rows, uint32_t* __restrict__ tile_offsets) {
    extern __shared__ uint32_t totals[];  // [E+1]
    constexpr int BATCH = 16;
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
        uint32_t run = 0;
        for (int b0 = 0; b0 < n_blocks; b0 += BATCH) {
            uint32_t c[BATCH];
#pragma unroll
            for (int j = 0; j < BATCH; ++j) c[j] = b0 + j < n_blocks ? block_hist[(size_t)(b0 + j) * n_experts + e] : 0u;
#pragma unroll
            for (int j = 0; j < BATCH; ++j) run += c[j];
        }
        totals[e] = run;
        counts[e] = run;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        uint32_t carry = 0, tcarry = 0;
        for (int e0 = 0; e0 < n_experts; e0 += 32) {
            const int e = e0 + lane;
            const uint32_t c = (e < n_experts) ? totals[e] : 0u;
            const uint32_t t = tile_offsets ? (c + tile_rows - 1) / tile_rows : 0u;
            uint32_t incl = c, tincl = t;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const uint32_t v = __shfl_up_sync(0xFFFFFFFFu, incl, d);
                const uint32_t tv = __shfl_up_sync(0xFFFFFFFFu, tincl, d);
                if (lane >= d) { incl += v; tincl += tv; }
            }
            if (e < n_experts) {
                totals[e] = carry + incl - c;
                offsets[e] = carry + incl - c;
                if (tile_offsets) tile_offsets[e] = tcarry + tincl - t;
            }
            carry += __shfl_sync(0xFFFFFFFFu, incl, 31);
            tcarry += __shfl_sync(0xFFFFFFFFu, tincl, 31);
        }
        if (lane == 0) {
            offsets[n_experts] = carry;
            if (tile_offsets) tile_offsets[n_experts] = tcarry;
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
        uint32_t run = totals[e];
        for (int b0 = 0; b0 < n_blocks; b0 += BATCH) {
            uint32_t c[BATCH];
#pragma unroll
            for (int j = 0; j < BATCH; ++j) c[j] = b0 + j < n_blocks ? block_hist[(size_t)(b0 + j) * n_experts + e] : 0u;
#pragma unroll
            for (int j = 0; j < BATCH; ++j) {
                if (b0 + j < n_blocks) block_hist[(size_t)(b0 + j) * n_experts + e] = run;
                run += c[j];
            }
        }
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
    // Stable scatter, 32 entries at a time.  Lanes with the same expert find each other by OR-ing their lane
    // bit into the expert's word (hist, free again after the ranking above); the next 32 ids are in flight
    // while this group is placed.
    __syncwarp();
    for (int e = lane; e < n_experts; e += 32) hist[e] = 0;
    __syncwarp();
    const uint32_t below = (1u << lane) - 1u;
    uint32_t e_next = (lane < n_rows) ? __ldcg(indices + lane) : 0xFFFFFFFFu;
    for (int i0 = 0; i0 < n_rows; i0 += 32) {
        const int i = i0 + lane;
        const uint32_t e = e_next;
        e_next = (i + 32 < n_rows) ? __ldcg(indices + i + 32) : 0xFFFFFFFFu;
        const bool real = e < (uint32_t)n_experts;   // padding and corrupt ids are dropped
        if (real) atomicOr(&hist[e], 1u << lane);
        __syncwarp();
        const uint32_t peers = real ? hist[e] : 0u;
        const uint32_t pos = real ? cursor[e] + __popc(peers & below) : 0u;
        __syncwarp();
        if (real && (peers & below) == 0u) {
            cursor[e] += __popc(peers);
            hist[e] = 0u;
        }
        __syncwarp();
        if (real) {
            o.perm[pos] = (uint32_t)i;
            o.inv_perm[i] = pos;
        }
    }
}

// Medium row counts (a prefill chunk): the three passes in ONE block of up to 32 warps.  Each warp owns a
// contiguous run of run_len entries (a multiple of 32, at most PLAN_ENTRIES_PER_WARP); the stable order
// does not depend on how the entries are cut into runs, so the permutation equals the three-launch one.
// Lanes that hold the same expert find each other through a per-warp word per expert that they OR their
// lane bit into (commutative, so deterministic); this is several times cheaper than a warp match when
// most lanes hold different experts.  Shared memory: hist[warps][E] + base[E] + mask[warps][E] words, and with
// stage_perm another n_rows words: the permutation is then assembled in shared memory and written out in
// order, because one SM retires scattered 4-byte global stores at about one per clock.
// When tile_offsets is given it also receives the prefix sum of ceil(count / tile_rows) (the grouped
// GEMM's token-tile schedule).
constexpr int PLAN_BLOCK_MAX_WARPS = 32;

__host__ __device__ inline int plan_block_run_len(int n_rows) {
    const int per_warp = (n_rows + PLAN_BLOCK_MAX_WARPS - 1) / PLAN_BLOCK_MAX_WARPS;
    return ((per_warp + 31) / 32) * 32;
}
__host__ __device__ inline size_t plan_block_smem(int n_warps, int n_experts, int staged_rows) {
    return ((size_t)(2 * n_warps + 1) * n_experts + (size_t)staged_rows) * sizeof(uint32_t);
}

__global__ void __launch_bounds__(PLAN_BLOCK_MAX_WARPS * 32)
plan_block_kernel(const uint32_t* __restrict__ indices, int n_rows, int n_experts, int run_len, PlanOut o,
                  int tile_rows, uint32_t* __restrict__ tile_offsets, int stage_perm) {
    extern __shared__ uint32_t sm[];
    __shared__ uint32_t n_placed_s;
    const int n_warps = blockDim.x / 32;
    const int warp = threadIdx.x / 32, lane = threadIdx.x & 31;
    uint32_t* hist = sm + (size_t)warp * n_experts;                       // this warp's histogram, then its cursors
    uint32_t* base = sm + (size_t)n_warps * n_experts;                    // [E] totals, then expert offsets
    uint32_t* mask = sm + (size_t)(n_warps + 1 + warp) * n_experts;       // this warp's lane sets per expert
    uint32_t* perm_out = stage_perm ? sm + (size_t)(2 * n_warps + 1) * n_experts : o.perm;
    for (int i = threadIdx.x; i < (2 * n_warps + 1) * n_experts; i += blockDim.x) sm[i] = 0;
    __syncthreads();
    const int begin = warp * run_len;
    const int end = min(begin + run_len, n_rows);
    // the warp's whole run sits in registers: one round trip to memory instead of one per 32 entries
    constexpr int PER_LANE = PLAN_ENTRIES_PER_WARP / 32;
    uint32_t ev[PER_LANE];
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) {
        const int i = begin + j * 32 + lane;
        ev[j] = (i < end) ? indices[i] : 0xFFFFFFFFu;   // ids out of range (padding or corrupt) are dropped
    }
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j)
        if (ev[j] < (uint32_t)n_experts) atomicAdd(&hist[ev[j]], 1u);
    __syncthreads();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {   // running sum over warps, per expert
        uint32_t run = 0;
        for (int w = 0; w < n_warps; ++w) {
            const uint32_t c = sm[(size_t)w * n_experts + e];
            sm[(size_t)w * n_experts + e] = run;
            run += c;
        }
        base[e] = run;
        o.counts[e] = run;
    }
    __syncthreads();
    if (warp == 0) {   // exclusive scans over experts, 32 at a time: rows and token tiles
        uint32_t carry = 0, tcarry = 0;
        for (int e0 = 0; e0 < n_experts; e0 += 32) {
            const int e = e0 + lane;
            const uint32_t c = (e < n_experts) ? base[e] : 0u;
            const uint32_t t = tile_offsets ? (c + tile_rows - 1) / tile_rows : 0u;
            uint32_t incl = c, tincl = t;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const uint32_t v = __shfl_up_sync(0xFFFFFFFFu, incl, d);
                const uint32_t tv = __shfl_up_sync(0xFFFFFFFFu, tincl, d);
                if (lane >= d) { incl += v; tincl += tv; }
            }
            if (e < n_experts) {
                o.offsets[e] = carry + incl - c;
                base[e] = carry + incl - c;
                if (tile_offsets) tile_offsets[e] = tcarry + tincl - t;
            }
            carry += __shfl_sync(0xFFFFFFFFu, incl, 31);
            tcarry += __shfl_sync(0xFFFFFFFFu, tincl, 31);
        }
        if (lane == 0) {
            o.offsets[n_experts] = carry;
            n_placed_s = carry;
            if (tile_offsets) tile_offsets[n_experts] = tcarry;
        }
    }
    __syncthreads();
    for (int e = lane; e < n_experts; e += 32) hist[e] += base[e];
    __syncwarp();
    const uint32_t below = (1u << lane) - 1u;
#pragma unroll
    for (int j = 0; j < PER_LANE; ++j) {   // stable scatter of this warp's run, 32 entries at a time
        if (begin + j * 32 >= end) break;
        const uint32_t e = ev[j];
        const bool real = e < (uint32_t)n_experts;
        if (real) atomicOr(&mask[e], 1u << lane);
        __syncwarp();
        const uint32_t peers = real ? mask[e] : 0u;
        const uint32_t pos = real ? hist[e] + __popc(peers & below) : 0u;
        __syncwarp();
        if (real && (peers & below) == 0u) {   // the lowest lane of each expert advances its cursor
            hist[e] += __popc(peers);
            mask[e] = 0u;
        }
        __syncwarp();
        if (real) {
            const uint32_t i = (uint32_t)(begin + j * 32 + lane);
            perm_out[pos] = i;
            o.inv_perm[i] = pos;
        }
    }
    if (stage_perm) {
        __syncthreads();
        const uint32_t n_placed = n_placed_s;
        for (uint32_t i = threadIdx.x; i < n_placed; i += blockDim.x) o.perm[i] = perm_out[i];
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
