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

// ───────────────────── exchange over peer memory (no NCCL, no host round trip) ─────────────────────
//
// Every rank exports three allocations to the others (CUDA IPC; one process per GPU): its row buffer
// (rows it will compute on, expert-contiguous), its result buffer, and a small control window that
// holds the counts matrix [world][n_experts] and the barrier flags.  Per step, all on the stream:
//   publish   every rank stores its per-expert row counts into row `rank` of every peer's matrix; barrier 0
//   layout    every rank derives, from the same matrix, where each (source, expert) segment lives in each
//             receiver's row buffer: its own expert offsets, and the base of its own segments elsewhere
//   dispatch  the gather writes each routed row (8-run permuted) straight into its owner's row buffer
//             over NVLink; barrier 1
//   experts   unchanged kernels over the local rows; barrier 2
//   combine   each token pulls its k result rows from the owners' result buffers while it sums them
// so the gather is fused with the dispatch and the combine with the return.  A barrier is a flag per
// (barrier, source rank) holding the step number, written into every peer's window and polled locally
// with a time limit; on expiry the kernel records an error word and returns.
constexpr int EP_MAX_WORLD = 16;
constexpr int EP_BARRIERS = 3;
constexpr uint64_t EP_WAIT_LIMIT_NS = 2000000000ull;   // default limit of a barrier wait (a per-layer option overrides it)
enum : uint32_t { EP_ERR_BARRIER_TIMEOUT = 16, EP_ERR_CAPACITY = 17 };

struct PeerPtrs {
    void* p[EP_MAX_WORLD];
};

// control window, in 32-bit words: flags[EP_BARRIERS][EP_MAX_WORLD], then the counts matrix [world][n_experts]
__host__ __device__ __forceinline__ uint32_t* win_flags(void* win, int barrier) { return static_cast<uint32_t*>(win) + barrier * EP_MAX_WORLD; }
__host__ __device__ __forceinline__ uint32_t* win_matrix(void* win) { return static_cast<uint32_t*>(win) + EP_BARRIERS * EP_MAX_WORLD; }
inline size_t win_words(int world, int n_experts) { return (size_t)EP_BARRIERS * EP_MAX_WORLD + (size_t)world * n_experts; }

// Tell every peer this rank reached `barrier` of step `epoch`, then wait (bounded) for all of them.
// Called by one block; threads 0..world-1 take one peer each.  Writes before the call are made
// visible system-wide first.
FFAI_DEVINL void peer_barrier(const PeerPtrs& win, int me, int world, int barrier, uint32_t epoch, uint64_t limit_ns, uint32_t* error_word) {
    __threadfence_system();
    __syncthreads();
    if ((int)threadIdx.x < world) {
        volatile uint32_t* theirs = win_flags(win.p[threadIdx.x], barrier) + me;
        *theirs = epoch;
        volatile uint32_t* mine = win_flags(win.p[me], barrier) + threadIdx.x;
        uint64_t t0 = 0;
        for (uint32_t spin = 0;; ++spin) {
            if ((int32_t)(*mine - epoch) >= 0) break;
            if ((spin & 255u) == 255u) {
                uint64_t now;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                if (t0 == 0) t0 = now;
                else if (now - t0 > limit_ns) {
                    atomicExch(error_word, EP_ERR_BARRIER_TIMEOUT);
                    break;
                }
            }
        }
    }
    __syncthreads();
    __threadfence_system();
}

__global__ void __launch_bounds__(32)
ep_barrier_kernel(int barrier, int me, int world, PeerPtrs win, uint32_t epoch, uint64_t limit_ns, uint32_t* error_word) {
    peer_barrier(win, me, world, barrier, epoch, limit_ns, error_word);
}

// From the counts matrix [world][n_experts] (identical on every rank after barrier 0): where rank `me`'s rows
// for expert e start in the row buffer of the rank that owns e.  Rows are grouped by expert, and inside an
// expert by ascending source rank - the layout plan_exchange gives the NCCL mode.  Host and device share
// these two functions; the host copy is exported for tests.
__host__ __device__ inline uint32_t peer_send_base(const uint32_t* matrix, int n_experts, int e_local, int me, int world, int e) {
    const int first = (e / e_local) * e_local;   // first expert of the owner
    uint32_t base = 0;
    for (int ee = first; ee < e; ++ee)
        for (int s = 0; s < world; ++s) base += matrix[(size_t)s * n_experts + ee];
    for (int s = 0; s < me; ++s) base += matrix[(size_t)s * n_experts + e];
    return base;
}
// ... and where the rows of rank `me`'s own expert el (0..e_local; e_local gives the total) start in its buffer.
__host__ __device__ inline uint32_t peer_local_offset(const uint32_t* matrix, int n_experts, int e_local, int me, int world, int el) {
    uint32_t run = 0;
    for (int ee = 0; ee < el; ++ee)
        for (int s = 0; s < world; ++s) run += matrix[(size_t)s * n_experts + me * e_local + ee];
    return run;
}

//   local_off[e_local+1]  row ranges of this rank's experts in its own row buffer (all sources, ascending rank)
//   send_base[n_experts]  where this rank's rows for expert e start in the owner's row buffer
// Offsets are clamped to the row buffer's capacity (and the error word raised) so that a matrix left half-updated
// by a barrier that gave up cannot send the expert kernels past the buffer.
FFAI_DEVINL void ep_layout_block(const uint32_t* __restrict__ matrix, int n_experts, int e_local, int me, int world,
                                 uint32_t* __restrict__ local_off, uint32_t* __restrict__ send_base, uint32_t capacity,
                                 uint32_t* error_word) {
    // The same numbers as peer_send_base / peer_local_offset, by prefix sums: per expert the rows of all sources,
    // an exclusive scan of those totals inside every owner's range (one warp per owner at a time, 32 experts per
    // round), plus the rows of the sources below this rank.  (Evaluating the two functions per expert walks up
    // to e_local * world matrix words in a dependent chain per thread: 50 us at 256 experts.)
    extern __shared__ uint32_t lay_sm[];     // [n_experts] totals, then [n_experts] exclusive scans
    uint32_t* tot = lay_sm;
    uint32_t* excl = lay_sm + n_experts;
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
        uint32_t t = 0;
        for (int s = 0; s < world; ++s) t += __ldcg(matrix + (size_t)s * n_experts + e);   // written by the peers: read from L2
        tot[e] = t;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    for (int owner = warp; owner < world; owner += n_warps) {
        uint32_t carry = 0;
        for (int e0 = 0; e0 < e_local; e0 += 32) {
            const int el = e0 + lane;
            const uint32_t c = el < e_local ? tot[owner * e_local + el] : 0u;
            uint32_t incl = c;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const uint32_t v = __shfl_up_sync(0xFFFFFFFFu, incl, d);
                if (lane >= d) incl += v;
            }
            if (el < e_local) excl[owner * e_local + el] = carry + incl - c;
            carry += __shfl_sync(0xFFFFFFFFu, incl, 31);
        }
        if (owner == me && lane == 0) {
            uint32_t v = carry;              // all rows this rank's experts receive
            if (v > capacity) {
                v = capacity;
                atomicExch(error_word, EP_ERR_CAPACITY);
            }
            local_off[e_local] = v;
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) {
        uint32_t below = 0;
        for (int s = 0; s < me; ++s) below += __ldcg(matrix + (size_t)s * n_experts + e);
        send_base[e] = excl[e] + below;
    }
    for (int el = threadIdx.x; el < e_local; el += blockDim.x) {
        uint32_t v = excl[me * e_local + el];
        if (v > capacity) {
            v = capacity;
            atomicExch(error_word, EP_ERR_CAPACITY);
        }
        local_off[el] = v;
    }
}

// Counts to every peer, barrier 0, then the layout - one launch (one block of 256 threads, 2 * n_experts words of
// dynamic shared memory).
__global__ void __launch_bounds__(256)
ep_publish_and_layout_kernel(const uint32_t* __restrict__ counts, int n_experts, int e_local, int me, int world, PeerPtrs win,
                             uint32_t epoch, uint64_t limit_ns, uint32_t* __restrict__ local_off,
                             uint32_t* __restrict__ send_base, uint32_t capacity, uint32_t* error_word) {
    for (int d = 0; d < world; ++d) {
        uint32_t* row = win_matrix(win.p[d]) + (size_t)me * n_experts;
        for (int e = threadIdx.x; e < n_experts; e += blockDim.x) row[e] = counts[e];
    }
    peer_barrier(win, me, world, 0, epoch, limit_ns, error_word);
    ep_layout_block(win_matrix(win.p[me]), n_experts, e_local, me, world, local_off, send_base, capacity, error_word);
}

// Gather fused with the dispatch: sorted row r of this rank (token perm[r]/k, expert indices[perm[r]])
// is written, 8-run permuted, into the row buffer of the rank that owns the expert.  One warp per row.
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const uint16_t* __restrict__ x, const uint32_t* __restrict__ perm, const uint32_t* __restrict__ indices,
                   const uint32_t* __restrict__ offsets, const uint32_t* __restrict__ send_base, int k, int e_local,
                   int n_rows, int hidden, PeerPtrs rows_of, uint32_t capacity, uint32_t* error_word) {
    const int warps = blockDim.x / 32;
    const int r = blockIdx.x * warps + threadIdx.x / 32;
    if (r >= n_rows) return;
    const int lane = threadIdx.x & 31;
    const uint32_t pe = perm[r];
    const uint32_t e = indices[pe];
    const uint32_t pos = send_base[e] + ((uint32_t)r - offsets[e]);
    if (pos >= capacity) {
        if (lane == 0) atomicExch(error_word, EP_ERR_CAPACITY);
        return;
    }
    const uint4* s = reinterpret_cast<const uint4*>(x + (size_t)(pe / (uint32_t)k) * hidden);
    uint4* d = reinterpret_cast<uint4*>(static_cast<uint16_t*>(rows_of.p[e / (uint32_t)e_local]) + (size_t)pos * hidden);
    // four 16-byte pieces per lane in flight: all loads first, then the (possibly remote) stores
    const int chunks = hidden / 8;
    for (int i0 = 0; i0 < chunks; i0 += 128) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * 32 + lane;
            if (i < chunks) v[u] = s[i];
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * 32 + lane;
            if (i < chunks) {
                uint4 o;
                o.x = __byte_perm(v[u].x, v[u].z, 0x5410);
                o.y = __byte_perm(v[u].x, v[u].z, 0x7632);
                o.z = __byte_perm(v[u].y, v[u].w, 0x5410);
                o.w = __byte_perm(v[u].y, v[u].w, 0x7632);
                d[i] = o;
            }
        }
    }
}

// Combine fused with the return: as combine_kernel<bf16, float>, but slot s of token t reads its
// result row (bf16: half the bytes over NVLink) from the owner of its expert.  One block per token; a thread owns 4 hidden positions.
__global__ void __launch_bounds__(256)
combine_peer_kernel(PeerPtrs y_of, const uint32_t* __restrict__ inv_perm, const uint32_t* __restrict__ indices,
                    const uint32_t* __restrict__ offsets, const uint32_t* __restrict__ send_base, int e_local,
                    const float* __restrict__ weights, int k, const float* __restrict__ shared_y,
                    const float* __restrict__ shared_gate_logit, const uint16_t* __restrict__ residual,
                    uint16_t* __restrict__ out, int hidden, uint32_t capacity, uint32_t* error_word) {
    const int t = blockIdx.x;
    __shared__ const uint16_t* row_s[32];
    __shared__ float w_s[32];
    __shared__ float sig_s;
    if ((int)threadIdx.x < k) {
        const size_t slot = (size_t)t * k + threadIdx.x;
        const uint32_t e = indices[slot];
        uint32_t pos = send_base[e] + (inv_perm[slot] - offsets[e]);
        float w = weights[slot];
        if (pos >= capacity) {   // only after a barrier gave up: the row is left out, the error word says so
            atomicExch(error_word, EP_ERR_CAPACITY);
            pos = 0;
            w = 0.0f;
        }
        row_s[threadIdx.x] = static_cast<const uint16_t*>(y_of.p[e / (uint32_t)e_local]) + (size_t)pos * hidden;
        w_s[threadIdx.x] = w;
    }
    if (threadIdx.x == 0) {
        float sig = 1.0f;
        if (shared_gate_logit) sig = 1.0f / (1.0f + __expf(-shared_gate_logit[t]));
        sig_s = sig;
    }
    __syncthreads();
    // a thread owns 8 consecutive hidden positions; the (remote) rows of up to 8 slots are loaded before the first use
    for (int h = threadIdx.x * 8; h < hidden; h += blockDim.x * 8) {
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
        for (int s0 = 0; s0 < k; s0 += 8) {
            uint4 u[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (s0 + j < k) u[j] = *reinterpret_cast<const uint4*>(row_s[s0 + j] + h);
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (s0 + j < k) {   // slot order: the sum does not depend on the launch geometry
                    const float w = w_s[s0 + j];
                    acc[0] += w * bf16lo(u[j].x); acc[1] += w * bf16hi(u[j].x); acc[2] += w * bf16lo(u[j].y); acc[3] += w * bf16hi(u[j].y);
                    acc[4] += w * bf16lo(u[j].z); acc[5] += w * bf16hi(u[j].z); acc[6] += w * bf16lo(u[j].w); acc[7] += w * bf16hi(u[j].w);
                }
        }
        if (shared_y) {
            const float sig = sig_s;
            const float4 v0 = *reinterpret_cast<const float4*>(shared_y + (size_t)t * hidden + h);
            const float4 v1 = *reinterpret_cast<const float4*>(shared_y + (size_t)t * hidden + h + 4);
            acc[0] += sig * v0.x; acc[1] += sig * v0.y; acc[2] += sig * v0.z; acc[3] += sig * v0.w;
            acc[4] += sig * v1.x; acc[5] += sig * v1.y; acc[6] += sig * v1.z; acc[7] += sig * v1.w;
        }
        if (residual) {
            const uint4 r = *reinterpret_cast<const uint4*>(residual + (size_t)t * hidden + h);
            acc[0] += bf16lo(r.x); acc[1] += bf16hi(r.x); acc[2] += bf16lo(r.y); acc[3] += bf16hi(r.y);
            acc[4] += bf16lo(r.z); acc[5] += bf16hi(r.z); acc[6] += bf16lo(r.w); acc[7] += bf16hi(r.w);
        }
        uint4 o;
        o.x = (uint32_t)f32_to_bf16_bits(acc[0]) | ((uint32_t)f32_to_bf16_bits(acc[1]) << 16);
        o.y = (uint32_t)f32_to_bf16_bits(acc[2]) | ((uint32_t)f32_to_bf16_bits(acc[3]) << 16);
        o.z = (uint32_t)f32_to_bf16_bits(acc[4]) | ((uint32_t)f32_to_bf16_bits(acc[5]) << 16);
        o.w = (uint32_t)f32_to_bf16_bits(acc[6]) | ((uint32_t)f32_to_bf16_bits(acc[7]) << 16);
        *reinterpret_cast<uint4*>(out + (size_t)t * hidden + h) = o;
    }
}

// 32-run sums of the first *n_rows_dev rows (the count lives on the device); grid sized for the capacity.
__global__ void sum64_rows_counted_kernel(const uint16_t* __restrict__ rows, float* __restrict__ sums,
                                          const uint32_t* __restrict__ n_rows_dev, int row_len, int sum_pitch) {
    const int warps = blockDim.x / 32;
    const int row = blockIdx.x * warps + threadIdx.x / 32;
    if (row >= (int)*n_rows_dev) return;
    const int lane = threadIdx.x & 31;
    const uint4* s = reinterpret_cast<const uint4*>(rows + (size_t)row * row_len);
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
        if ((lane & 3) == 0 && i < chunks) sums[(size_t)row * sum_pitch + (i >> 2)] = part;
    }
}

}  // namespace ep
}  // namespace ffai
