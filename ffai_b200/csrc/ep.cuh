// Expert parallelism across the GPUs of one node: tokens stay data-parallel (each rank routes its own
// rows), experts are sharded E/G per rank in contiguous blocks, and two all-to-all exchanges over NCCL
// (NVLink / NVSwitch) move activation rows to the ranks that own their experts and results back.
//
// The reference has no counterpart (single device; "dispatch" is a host sort plus one gather,
// FFAI MoELayer.swift:752-774, 843).  Order is kept deterministic: rows leave a rank sorted by
// (expert, token, slot); a receiving rank regroups the per-source segments of each of its experts in
// ascending source-rank order; results travel back along the same segments, so the sender finds its
// rows where the single-GPU path would have produced them and the combine is unchanged.
//
// NCCL is resolved at run time (dlopen) so that single-GPU users need no NCCL at all.
#pragma once
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>
#include <stdint.h>

#include "common.cuh"

namespace ffai {
namespace ep {

struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    bool ok = false;
};

inline NcclApi& nccl() {
    static NcclApi api;
    static bool tried = false;
    if (!tried) {
        tried = true;
        // prefer a copy that is already mapped into the process (e.g. the one a host framework loaded)
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
        if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (h) {
            api.GetUniqueId = (decltype(api.GetUniqueId))dlsym(h, "ncclGetUniqueId");
            api.CommInitRank = (decltype(api.CommInitRank))dlsym(h, "ncclCommInitRank");
            api.CommDestroy = (decltype(api.CommDestroy))dlsym(h, "ncclCommDestroy");
            api.Send = (decltype(api.Send))dlsym(h, "ncclSend");
            api.Recv = (decltype(api.Recv))dlsym(h, "ncclRecv");
            api.GroupStart = (decltype(api.GroupStart))dlsym(h, "ncclGroupStart");
            api.GroupEnd = (decltype(api.GroupEnd))dlsym(h, "ncclGroupEnd");
            api.GetErrorString = (decltype(api.GetErrorString))dlsym(h, "ncclGetErrorString");
            api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.Send && api.Recv &&
                     api.GroupStart && api.GroupEnd;
        }
    }
    return api;
}

// Host-side plan of one exchange, from the per-(source rank, local expert) row counts.
//   recv_counts   [world][e_local]
//   rank_offsets  [world+1]   where the rows of each source start in the receive buffer (source order)
//   local_offsets [e_local+1] rows per local expert after regrouping (expert-contiguous order)
//   seg_src/seg_dst [world*e_local]  start of segment (s, e) in the receive buffer / regrouped buffer
// Returns the total number of received rows.  Pure integer arithmetic: runs (and is tested) without a GPU.
inline uint32_t plan_exchange(const uint32_t* recv_counts, int world, int e_local, uint32_t* rank_offsets,
                              uint32_t* local_offsets, uint32_t* seg_src, uint32_t* seg_dst) {
    uint32_t run = 0;
    for (int s = 0; s < world; ++s) {
        rank_offsets[s] = run;
        for (int e = 0; e < e_local; ++e) {
            seg_src[s * e_local + e] = run;
            run += recv_counts[s * e_local + e];
        }
    }
    rank_offsets[world] = run;
    uint32_t run2 = 0;
    for (int e = 0; e < e_local; ++e) {
        local_offsets[e] = run2;
        for (int s = 0; s < world; ++s) {
            seg_dst[s * e_local + e] = run2;
            run2 += recv_counts[s * e_local + e];
        }
    }
    local_offsets[e_local] = run2;
    return run;
}

// Copy row segments: segment i moves seg_rows[i] rows of row_bytes bytes from src + seg_from[i] rows to
// dst + seg_to[i] rows.  One block per (segment, 8-row slice); 16-byte copies.
__global__ void copy_segments_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                     const uint32_t* __restrict__ seg_from, const uint32_t* __restrict__ seg_to,
                                     const uint32_t* __restrict__ seg_rows, int row_bytes) {
    const int seg = blockIdx.x;
    const uint32_t rows = seg_rows[seg];
    const int warps = blockDim.x / 32, warp = threadIdx.x / 32, lane = threadIdx.x & 31;
    const int chunks = row_bytes / 16;
    for (uint32_t r = blockIdx.y * warps + warp; r < rows; r += gridDim.y * warps) {
        const uint4* s = reinterpret_cast<const uint4*>(src + (size_t)(seg_from[seg] + r) * row_bytes);
        uint4* d = reinterpret_cast<uint4*>(dst + (size_t)(seg_to[seg] + r) * row_bytes);
        for (int i = lane; i < chunks; i += 32) d[i] = s[i];
    }
}

}  // namespace ep
}  // namespace ffai
