// Decode-regime grouped 4-bit dequant products, bulk-copy streamed (group size 64 or 128).
//
// Replaces, for small batches, the reference's per-expert GEMV chain
// (Ops.dequantGemvInt4ExpertIndexedMany, FFAI Ops.swift:2529-2587; the fused
// moeDownSwigluAccumInt4Chain8, OpsFused.swift:545-697; MoELayer.decodeGPURouter,
// MoELayer.swift:1167-1341) and GPT-OSS's three-sync-per-expert loop
// (GPTOSSText.swift:1399-1445).  Same arithmetic as expert_mma_decode.cuh:
//     sum_k (s*q_k + b) x_k = s * sum_k (128+q_k) x_k + (b - 128 s) * sum_k x_k
// per 64-run, (128+q) exact in bf16, mma.sync.m16n8k16 as the dot engine, fp32 everywhere else.
//
// What differs is how the operands reach the registers.  At load time the packed words and the
// (scale | bias << 16) words of every 16-row block are re-tiled into one contiguous stream per
// (expert, block) in the order the MMA fragments want them:
//     cell  = 16 rows x 64 k:  512 B of packed words, lane l's four words at l*16 (rows g = l/4 and
//             g+8, words 2t and 2t+1 of the run, t = l%4), then 64 B of scale words ([g][row half])
//     unit  = what one bulk copy moves: gate/up launches: the gate cell and the up cell of one 64-run
//             (1152 B); one-projection launches: CPU consecutive cells (CPU x 576 B)
// A warp streams the units of its items through its own ring of DEPTH slots with cp.async.bulk +
// mbarrier complete_tx issued by one lane: no per-lane copy instructions, no address arithmetic per
// stage, one 16-byte shared-memory read per lane and cell, and no barrier of any kind inside the
// stream.  The grid is persistent (one CTA of 16 warps per SM).  The (expert, pass, block) items are
// split over the CTAs in contiguous ranges of equal cost, so a CTA stays on one or two experts; the
// activation rows of the expert passes in its range (at most 16 rows at a time) are brought into
// shared memory once, by bulk copies, with their 64-run sums beside them.  Inside a CTA, teams of
// TEAM warps take the items round robin.  TEAM = 1: a warp owns an item from start to end.  TEAM > 1
// (the smallest batches, where items are too few for 2368 warps): the warps of a team split the
// reduction axis and add their partials in a fixed order through shared memory.  Weight copies for
// the next item are in flight while the current one finishes.
//
// Every wait on an mbarrier is bounded; on expiry the warp records an error word, stops streaming,
// keeps meeting the CTA's barriers, and drains (bounded) the copies it still has in flight.
#pragma once
#include <type_traits>

#include "common.cuh"
#include "expert_mma_decode.cuh"

namespace ffai {
namespace dstr {

constexpr int CELL_W = 512;               // packed words of a cell
constexpr int CELL_SB = 64;               // scale words of a cell
constexpr int CELL = CELL_W + CELL_SB;    // 576
constexpr int SLOT = 2 * CELL;            // ring slot: the largest unit
constexpr int WARPS = 16;
constexpr int THREADS = WARPS * 32;
constexpr int XROWS = 16;                 // activation rows resident in shared memory at a time
constexpr int MAX_SEGS = 16;              // expert passes resident at a time (each holds at least one row)
constexpr uint32_t WAIT_TRIES = 1u << 22; // bounded wait: tries of up to ~1 us each
enum : uint32_t { ERR_STREAM_TIMEOUT = 32 };

struct Params {
    const uint8_t* wt;        // re-tiled stream: [E][N/16][units][unit bytes]
    const uint16_t* rb1;      // nullable row bias [E, N] (first projection)
    const uint16_t* rb2;      // nullable (second projection of a gate/up launch)
    int N, K;
    int n_experts;
    const uint32_t* offsets;  // [E+1] rows per expert in the sorted row space
    const uint32_t* order;    // nullable [E]: experts by descending row count; identity when null
    const uint16_t* x;        // [rows, K] bf16, 8-run permuted
    const uint32_t* row_src;  // nullable: sorted row r reads x (and xsum) at row row_src[r] / row_div
    int row_div;
    const float* xsum;        // [rows, xsum_pitch] sums of 32-runs of x (two per cell)
    int xsum_pitch;
    const float* xsum_parts;  // alternative (when non-null): [rows, K/16] sums of 16-runs (four per cell)
    float* out_parts;         // gate/up, nullable: [rows, N/16] sum of each block's 16 rounded outputs per row
    void* out;                // gate/up: bf16 [rows, N] 8-run permuted;  else fp32 [rows, N] (bf16 when out_bf16)
    int out_bf16;
    int activation;
    float limit, alpha;
    int nt2_cost;             // cost of an item with more than 8 rows relative to 8 for one with fewer (>= 8)
    int tables_ready;         // 1: offsets / order were written two or more kernels back (a programmatic dependent launch
                              // may build its schedule and start streaming weights before the kernel before it has ended)
    uint32_t* error_word;
};

FFAI_DEVINL uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
FFAI_DEVINL void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
FFAI_DEVINL void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
FFAI_DEVINL bool mbar_test_wait(uint32_t bar, uint32_t parity) {   // one look, no suspension
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}
FFAI_DEVINL bool mbar_try_wait(uint32_t bar, uint32_t parity) {    // may suspend the thread up to ~1 us
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(1000u)
        : "memory");
    return done != 0;
}
// Bounded wait; false when the limit expires.
FFAI_DEVINL bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    if (mbar_test_wait(bar, parity)) return true;
    for (uint32_t tries = 0; tries < WAIT_TRIES; ++tries)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// Contiguous global -> shared copy; the mbarrier receives the byte count on completion.
FFAI_DEVINL void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
FFAI_DEVINL void team_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Expert passes whose rows are resident in shared memory (one "group"), built by thread 0.
struct SegTable {
    int n;                         // segments in the group
    int group_end;                 // first item after the group
    int n_rows;                    // buffer rows in use
    int first[MAX_SEGS];           // item of block 0 of the segment's pass (may lie before the CTA's range)
    int end[MAX_SEGS];             // first item after the segment, clipped to the CTA's range
    int expert[MAX_SEGS];
    int row0[MAX_SEGS];            // first sorted row of the expert
    int cnt[MAX_SEGS];             // rows of the expert
    int tok0[MAX_SEGS];            // first row of the pass within the expert
    int base[MAX_SEGS];            // first buffer row of the segment (even)
    int src_row[XROWS];            // buffer row -> sorted row, or -1
};

// grid: one CTA per SM (persistent), 512 threads.  Dynamic shared memory, in order: mbarriers [WARPS][DEPTH] + 1
// and the segment table (2 KiB), rings [WARPS][DEPTH][SLOT], activation rows [16][2 K + 16], their 64-run sums
// [cells + 1][16], schedule tables (2 (E+1) + E words), per-team partial buffers [teams][TEAM-1][16 x 32 floats].
template <bool FUSED, int TEAM, int CPU, int DEPTH>
struct Layout {
    static constexpr int TEAMS = WARPS / TEAM;
    static constexpr int UNIT = FUSED ? 2 * CELL : CPU * CELL;
    static constexpr int CELLS_PER_UNIT = FUSED ? 1 : CPU;
    static constexpr int RED_PER_WARP = 16 * 32 * 4;   // 2 tiles x NP x 4 values per lane, at most 16
    static_assert(WARPS * DEPTH * 8 + 8 + sizeof(SegTable) <= 2048, "barrier and table area");
    __host__ __device__ static int x_pitch(int K) { return 2 * K + 16; }   // an odd number of 16-byte pieces: conflict-free fragment reads
    __host__ __device__ static int table() { return WARPS * DEPTH * 8 + 8; }
    __host__ __device__ static int rings() { return 2048; }
    __host__ __device__ static int xrows() { return rings() + WARPS * DEPTH * SLOT; }
    __host__ __device__ static int xs(int K) { return xrows() + XROWS * x_pitch(K); }
    __host__ __device__ static int sched(int K) { return xs(K) + (K / 64 + 1) * 64; }
    __host__ __device__ static int red(int E, int K) { return (sched(K) + (3 * E + 2) * 4 + 15) & ~15; }
    __host__ __device__ static int total(int E, int K) { return red(E, K) + (TEAM > 1 ? TEAMS * (TEAM - 1) * RED_PER_WARP : 0); }
};

FFAI_DEVINL uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
FFAI_DEVINL uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.b32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}

// One cell against the B fragments in xc: unpack, MMAs, fold into tot[tile][value].  wa / sa: shared-window addresses
// of this lane's packed words and scale words of the cell; xsa: of its 64-run sums (8-byte pairs, 32 bytes apart per tile).
template <int NT>
FFAI_DEVINL void compute_cell(uint32_t wa, uint32_t sa, const uint4 (*xc)[2], uint32_t xsa,
                              uint32_t mask, uint32_t expo, float (*tot)[4]) {
    const uint4 wv = lds128(wa);          // row g: x, y;  row g+8: z, w
    const uint2 sbv = lds64(sa);          // rows g, g+8
    float sc[2], bm[2];
    sc[0] = __uint_as_float(sbv.x << 16); sc[1] = __uint_as_float(sbv.y << 16);
    bm[0] = fmaf(-128.0f, sc[0], __uint_as_float(sbv.x & 0xFFFF0000u));
    bm[1] = fmaf(-128.0f, sc[1], __uint_as_float(sbv.y & 0xFFFF0000u));
    uint32_t af[2][2][4];   // [word][row half][pair]
    dmma::unpack_word_128r(wv.x, af[0][0], mask, expo);
    dmma::unpack_word_128r(wv.y, af[1][0], mask, expo);
    dmma::unpack_word_128r(wv.z, af[0][1], mask, expo);
    dmma::unpack_word_128r(wv.w, af[1][1], mask, expo);
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const uint2 sxb = lds64(xsa + 32 * j);
        const float2 sx = make_float2(__uint_as_float(sxb.x), __uint_as_float(sxb.y));
        const uint32_t xb[2][4] = {{xc[j][0].x, xc[j][0].y, xc[j][0].z, xc[j][0].w},
                                   {xc[j][1].x, xc[j][1].y, xc[j][1].z, xc[j][1].w}};
        float c[4];
#pragma unroll
        for (int w = 0; w < 2; ++w)
#pragma unroll
            for (int hp = 0; hp < 2; ++hp) {
                // k-slots (2t,2t+1) <- pair 2hp, (2t+8,2t+9) <- pair 2hp+1 of word w
                const uint32_t a[4] = {af[w][0][2 * hp], af[w][1][2 * hp], af[w][0][2 * hp + 1], af[w][1][2 * hp + 1]};
                if (w == 0 && hp == 0) dmma::mma_bf16_16816_zero(c, a, xb[w][2 * hp], xb[w][2 * hp + 1]);
                else dmma::mma_bf16_16816(c, a, xb[w][2 * hp], xb[w][2 * hp + 1]);
            }
        tot[j][0] = fmaf(sc[0], c[0], fmaf(bm[0], sx.x, tot[j][0]));
        tot[j][1] = fmaf(sc[0], c[1], fmaf(bm[0], sx.y, tot[j][1]));
        tot[j][2] = fmaf(sc[1], c[2], fmaf(bm[1], sx.x, tot[j][2]));
        tot[j][3] = fmaf(sc[1], c[3], fmaf(bm[1], sx.y, tot[j][3]));
    }
}

template <bool FUSED, int TEAM, int CPU, int DEPTH>
__global__ void __launch_bounds__(THREADS, 1)
stream_decode_kernel(const Params p) {
    using L = Layout<FUSED, TEAM, CPU, DEPTH>;
    constexpr int NP = FUSED ? 2 : 1;
    constexpr int TEAMS = L::TEAMS;
    constexpr int UNIT = L::UNIT;
    constexpr int CPUNIT = L::CELLS_PER_UNIT;
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int team = warp / TEAM, slice = warp % TEAM;
    const int E = p.n_experts, K = p.K;
    const int n_cells = K / 64, n_rb = p.N / 16;
    const int n_units = (n_cells + CPUNIT - 1) / CPUNIT;
    const uint32_t block_bytes = (uint32_t)(n_cells * NP * CELL);   // stream of one (expert, 16-row block)
    const int x_pitch = L::x_pitch(K);

    const uint32_t bar0 = smem_u32(smem) + warp * DEPTH * 8;
    const uint32_t xbar = smem_u32(smem) + WARPS * DEPTH * 8;
    SegTable* seg = reinterpret_cast<SegTable*>(smem + L::table());
    uint8_t* ring = smem + L::rings() + warp * DEPTH * SLOT;
    const uint32_t ring_u = smem_u32(ring);
    uint8_t* x_sm = smem + L::xrows();
    float* xs_sm = reinterpret_cast<float*>(smem + L::xs(K));
    uint32_t* pre_items = reinterpret_cast<uint32_t*>(smem + L::sched(K));   // [E+1]
    uint32_t* pre_cost = pre_items + (E + 1);                                // [E+1]
    uint32_t* ord_expert = pre_cost + (E + 1);                               // [E]
    float* red = TEAM > 1 ? reinterpret_cast<float*>(smem + L::red(E, K)) + (size_t)team * (TEAM - 1) * (L::RED_PER_WARP / 4) : nullptr;

    if (lane == 0)
        for (int d = 0; d < DEPTH; ++d) mbar_init(bar0 + d * 8, 1);
    if (threadIdx.x == 0) mbar_init(xbar, 1);
    if (!p.tables_ready) pdl_wait();   // the routing tables come from the kernel right before this one
    // schedule tables: one warp scans the experts in hand-out order
    if (warp == 0) {
        uint32_t run_i = 0, run_c = 0;
        for (int o0 = 0; o0 < E; o0 += 32) {
            const int o = o0 + lane;
            uint32_t items = 0, cost = 0;
            if (o < E) {
                const uint32_t e = p.order ? p.order[o] : (uint32_t)o;
                const uint32_t cnt = p.offsets[e + 1] - p.offsets[e];
                items = ((cnt + 15) / 16) * (uint32_t)n_rb;
                cost = items * (cnt > 8 ? (uint32_t)p.nt2_cost : 8u);
                ord_expert[o] = e;
            }
            uint32_t si = items, sc = cost;   // inclusive warp scan
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const uint32_t vi = __shfl_up_sync(0xFFFFFFFFu, si, d), vc = __shfl_up_sync(0xFFFFFFFFu, sc, d);
                if (lane >= d) { si += vi; sc += vc; }
            }
            if (o < E) { pre_items[o] = run_i + si - items; pre_cost[o] = run_c + sc - cost; }
            run_i += __shfl_sync(0xFFFFFFFFu, si, 31);
            run_c += __shfl_sync(0xFFFFFFFFu, sc, 31);
        }
        if (lane == 0) { pre_items[E] = run_i; pre_cost[E] = run_c; }
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();

    // this CTA's item range: the cost axis cut into gridDim.x equal parts, a cut mapped to the first item at or after it
    auto item_at = [&](uint32_t cut) -> int {
        int lo = 0, hi = E;   // last expert position whose cost prefix is <= cut
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (pre_cost[mid] <= cut) lo = mid; else hi = mid;
        }
        const uint32_t items = pre_items[lo + 1] - pre_items[lo];
        if (items == 0) return (int)pre_items[lo + 1];
        const uint32_t w = (pre_cost[lo + 1] - pre_cost[lo]) / items;
        return (int)min(pre_items[lo] + (cut - pre_cost[lo] + w - 1) / w, pre_items[lo + 1]);
    };
    const uint64_t total_cost = pre_cost[E];
    const int item_begin = item_at((uint32_t)(total_cost * blockIdx.x / gridDim.x));
    const int item_end = blockIdx.x + 1 == gridDim.x ? (int)pre_items[E]
                                                     : item_at((uint32_t)(total_cost * (blockIdx.x + 1) / gridDim.x));

    uint32_t mask, expo;
    asm volatile("mov.u32 %0, 0x000F000F;" : "=r"(mask));
    asm volatile("mov.u32 %0, 0x43004300;" : "=r"(expo));

    // This warp's share of an item: units [u_begin, u_end) of the block's stream.
    const int per = (n_units + TEAM - 1) / TEAM;
    const int u_begin = min(slice * per, n_units), u_end = min(u_begin + per, n_units);
    const int my_units = u_end - u_begin;
    const uint32_t last_bytes = (uint32_t)(min(CPUNIT, n_cells - (u_end - 1) * CPUNIT) * NP * CELL);   // of the warp's last unit

    // The copy engine of this warp: walks the team's items (item_begin + team, + TEAMS, ...) and this warp's units
    // inside each, DEPTH copies ahead of the arithmetic, across item and group boundaries.  It refills the slot the
    // arithmetic has just left, so one slot cursor serves both.
    int p_item = item_begin + team - TEAMS, p_ord = 0, p_left = 0;
    const uint8_t* p_src = nullptr;
    bool failed = false;             // a bounded wait expired: stop streaming, keep meeting the barriers
    auto produce = [&](uint32_t slot_addr, uint32_t bar) {   // one unit into the given slot, if any is left
        if (p_left == 0) {
            if (my_units == 0 || failed) return;
            p_item += TEAMS;
            if (p_item >= item_end) { p_item = item_end; return; }
            while (p_item >= (int)pre_items[p_ord + 1]) ++p_ord;
            const int rb = (p_item - (int)pre_items[p_ord]) % n_rb;
            p_src = p.wt + ((size_t)ord_expert[p_ord] * n_rb + rb) * block_bytes + (size_t)u_begin * UNIT;
            p_left = my_units;
        }
        if (lane == 0) {
            const uint32_t bytes = p_left == 1 ? last_bytes : (uint32_t)UNIT;
            mbar_expect_tx(bar, bytes);
            bulk_load(slot_addr, p_src, bytes, bar);
        }
        p_src += UNIT;
        --p_left;
    };
#pragma unroll 1
    for (int d = 0; d < DEPTH; ++d) produce(ring_u + d * SLOT, bar0 + d * 8);

    // The weights are in flight; the activation rows (and their sums) come from the kernel before this one.
    if (p.tables_ready) pdl_wait();
    pdl_launch_dependents();
    uint32_t c_off = 0, c_bar = bar0, c_phase = 0;   // slot cursor: byte offset into the ring, its mbarrier, the phase bit to wait for
    uint32_t x_phase = 0;
    int g_ord = 0;                      // expert cursor of the group builder (thread 0)
    const uint32_t lane16 = lane * 16, g8 = g * 8;
#pragma unroll 1
    for (int it = item_begin; it < item_end;) {
        // ── group: the expert passes from item `it` on whose rows fit the buffer together ──
        __syncthreads();                               // everybody is done with the previous group's rows, sums and table
        if (threadIdx.x == 0) {
            int n = 0, rows = 0, cur = it;
            for (int r = 0; r < XROWS; ++r) seg->src_row[r] = -1;
            while (cur < item_end && n < MAX_SEGS) {
                while (cur >= (int)pre_items[g_ord + 1]) ++g_ord;
                const int e = (int)ord_expert[g_ord];
                const int pass = (cur - (int)pre_items[g_ord]) / n_rb;
                const int first = (int)pre_items[g_ord] + pass * n_rb;
                const int row0 = (int)p.offsets[e], cnt = (int)p.offsets[e + 1] - row0;
                const int here = min(16, cnt - pass * 16);
                if (rows + here > XROWS) break;
                seg->first[n] = first; seg->end[n] = min(item_end, first + n_rb);
                seg->expert[n] = e; seg->row0[n] = row0; seg->cnt[n] = cnt; seg->tok0[n] = pass * 16; seg->base[n] = rows;
                for (int r = 0; r < here; ++r) seg->src_row[rows + r] = row0 + pass * 16 + r;
                rows += (here + 1) & ~1;               // bases stay even: a lane reads the sums of two rows at once
                cur = seg->end[n];
                ++n;
            }
            seg->n = n; seg->group_end = cur; seg->n_rows = rows;
        }
        __syncthreads();
        const int group_end = seg->group_end;
        if (warp == 0) {
            int my_src = lane < XROWS ? seg->src_row[lane] : -1;
            const uint32_t n_live = __popc(__ballot_sync(0xFFFFFFFFu, my_src >= 0));
            if (lane == 0) mbar_expect_tx(xbar, n_live * (uint32_t)(2 * K));
            __syncwarp();
            if (my_src >= 0) {
                const size_t sr = p.row_src ? (size_t)(__ldg(p.row_src + my_src) / (uint32_t)p.row_div) : (size_t)my_src;
                bulk_load(smem_u32(x_sm) + lane * x_pitch, p.x + sr * K, (uint32_t)(2 * K), xbar);
            }
        }
        // 64-run sums of the resident rows -> shared memory [cell][buffer row]; unused rows read as zero
        for (int i = threadIdx.x; i < n_cells * XROWS; i += THREADS) {
            const int r = i / n_cells, R = i - r * n_cells;
            const int src = seg->src_row[r];
            float v = 0.0f;
            if (src >= 0) {
                if (p.xsum_parts) {
                    const float4 q4 = __ldg(reinterpret_cast<const float4*>(p.xsum_parts + (size_t)src * (K / 16)) + R);
                    v = (q4.x + q4.y) + (q4.z + q4.w);
                } else {
                    const size_t sr = p.row_src ? (size_t)(__ldg(p.row_src + src) / (uint32_t)p.row_div) : (size_t)src;
                    const float2 q2 = __ldg(reinterpret_cast<const float2*>(p.xsum + sr * p.xsum_pitch) + R);
                    v = q2.x + q2.y;
                }
            }
            xs_sm[R * XROWS + r] = v;
        }
        __syncthreads();
        if (!failed && !mbar_wait_bounded(xbar, x_phase)) failed = true;
        x_phase ^= 1u;

        // ── this team's items of the group ──
        int si = 0;   // segment cursor
#pragma unroll 1
        for (int item = it + ((team - (it - item_begin)) % TEAMS + TEAMS) % TEAMS; item < group_end; item += TEAMS) {
            while (item >= seg->end[si]) ++si;
            const int e = seg->expert[si], row0 = seg->row0[si], cnt = seg->cnt[si], tok0 = seg->tok0[si], base = seg->base[si];
            const int rb = item - seg->first[si];
            const int rows_here = min(16, cnt - tok0);
            const bool two = rows_here > 8;

            float tot[NP][2][4];   // [projection][8-row tile][value]
#pragma unroll
            for (int q = 0; q < NP; ++q)
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int i = 0; i < 4; ++i) tot[q][j][i] = 0.0f;

            // B-operand rows of this lane (column g of each 8-wide tile), clamped to the last row of the pass; shared-window
            // addresses, so that every access below is one load at [lane base + warp-uniform offset + constant]
            uint32_t xl[2];
#pragma unroll
            for (int j = 0; j < 2; ++j)
                xl[j] = smem_u32(x_sm) + (base + min(8 * j + g, rows_here - 1)) * x_pitch + 32 * t + u_begin * CPUNIT * 128;
            const uint32_t xsl = smem_u32(xs_sm) + (base + 2 * t + u_begin * CPUNIT * XROWS) * 4;
            const uint32_t wl = ring_u + lane16, sl = ring_u + CELL_W + g8;

            auto run_units = [&](auto nt_tag) {
                constexpr int NT = decltype(nt_tag)::value;
#pragma unroll 1
                for (int u = 0; u < my_units; ++u) {
                    if (!mbar_test_wait(c_bar, c_phase)) {
                        if (!mbar_wait_bounded(c_bar, c_phase)) { failed = true; break; }
                    }
                    const bool second = CPUNIT > 1 && (u + 1 < my_units || last_bytes == (uint32_t)UNIT);
                    const uint32_t xo = (uint32_t)u * (CPUNIT * 128), so = (uint32_t)u * (CPUNIT * XROWS * 4);
#pragma unroll
                    for (int cI = 0; cI < CPUNIT; ++cI) {
                        if (cI > 0 && !second) break;
                        uint4 xc[NT][2];
#pragma unroll
                        for (int j = 0; j < NT; ++j) {
                            xc[j][0] = lds128(xl[j] + xo + cI * 128);
                            xc[j][1] = lds128(xl[j] + xo + cI * 128 + 16);
                        }
#pragma unroll
                        for (int q = 0; q < NP; ++q)
                            compute_cell<NT>(wl + c_off + (cI * NP + q) * CELL, sl + c_off + (cI * NP + q) * CELL, xc,
                                             xsl + so + cI * (XROWS * 4), mask, expo, tot[q]);
                    }
                    __syncwarp();   // every lane has used what it read from the slot
                    produce(ring_u + c_off, c_bar);   // refill it with the unit DEPTH ahead
                    c_off += SLOT; c_bar += 8;
                    if (c_off == DEPTH * SLOT) { c_off = 0; c_bar = bar0; c_phase ^= 1u; }
                }
            };
            if (!failed) {
                if (two) run_units(std::integral_constant<int, 2>{});
                else run_units(std::integral_constant<int, 1>{});
            }

            if (TEAM > 1) {
                // fixed-order sum of the team's slices: slices 1.. park their partials, slice 0 adds them in order
                float* my = red + (size_t)(slice > 0 ? slice - 1 : 0) * (L::RED_PER_WARP / 4);
                if (slice > 0) {
#pragma unroll
                    for (int q = 0; q < NP; ++q)
#pragma unroll
                        for (int j = 0; j < 2; ++j)
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                if (j == 0 || two) my[((q * 2 + j) * 4 + i) * 32 + lane] = tot[q][j][i];
                }
                team_barrier(1 + team, TEAM * 32);
                if (slice == 0) {
                    for (int o = 1; o < TEAM; ++o) {
                        const float* theirs = red + (size_t)(o - 1) * (L::RED_PER_WARP / 4);
#pragma unroll
                        for (int q = 0; q < NP; ++q)
#pragma unroll
                            for (int j = 0; j < 2; ++j)
#pragma unroll
                                for (int i = 0; i < 4; ++i)
                                    if (j == 0 || two) tot[q][j][i] += theirs[((q * 2 + j) * 4 + i) * 32 + lane];
                    }
                }
                team_barrier(1 + team, TEAM * 32);   // the partials are read: the next item may overwrite them
                if (slice != 0) continue;
            }
            if (failed) continue;

            // results: value i -> (row g + 8*(i>>1), activation row tok0 + 8j + 2t + (i&1))
            const int rb_row = rb * 16;
            float rsum[2][2];
#pragma unroll
            for (int j = 0; j < 2; ++j) rsum[j][0] = rsum[j][1] = 0.0f;
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int tok = tok0 + 8 * j + 2 * t + (i & 1);
                    if (tok >= cnt || (j == 1 && !two)) continue;
                    const int n = rb_row + g + 8 * (i >> 1);
                    const size_t rr = (size_t)e * p.N + n;
                    float v = tot[0][j][i];
                    if (p.rb1) v += bf16_bits_to_f32(p.rb1[rr]);
                    if (FUSED) {
                        float u = tot[NP - 1][j][i];
                        if (p.rb2) u += bf16_bits_to_f32(p.rb2[rr]);
                        v = glu_activation(v, u, p.activation, p.limit, p.alpha);
                        const uint16_t vb = f32_to_bf16_bits(v);
                        reinterpret_cast<uint16_t*>(p.out)[(size_t)(row0 + tok) * p.N + dmma::permute8_col(n)] = vb;
                        rsum[j][i & 1] += bf16_bits_to_f32(vb);
                    } else if (p.out_bf16) {
                        reinterpret_cast<uint16_t*>(p.out)[(size_t)(row0 + tok) * p.N + n] = f32_to_bf16_bits(v);
                    } else {
                        reinterpret_cast<float*>(p.out)[(size_t)(row0 + tok) * p.N + n] = v;
                    }
                }
            if (FUSED && p.out_parts) {
                // sum over the block's 16 output rows (the lanes that share t), fixed butterfly; lanes g == 0 write
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        float v = rsum[j][h];
                        v += __shfl_xor_sync(0xFFFFFFFFu, v, 4);
                        v += __shfl_xor_sync(0xFFFFFFFFu, v, 8);
                        v += __shfl_xor_sync(0xFFFFFFFFu, v, 16);
                        const int tok = tok0 + 8 * j + 2 * t + h;
                        if (g == 0 && tok < cnt && (j == 0 || two)) p.out_parts[(size_t)(row0 + tok) * (p.N / 16) + rb] = v;
                    }
            }
        }
        it = group_end;
    }

    if (failed) {
        if (lane == 0 && p.error_word) atomicExch(p.error_word, (uint32_t)ERR_STREAM_TIMEOUT);
        // copies this warp still has in flight land in its ring: give every slot (in ring order from the cursor) a
        // bounded wait for the phase a pending copy would complete, before the CTA may exit
        for (int d = 0; d < DEPTH; ++d) {
            uint32_t tries = 0;
            while (!mbar_try_wait(c_bar, c_phase) && ++tries < 2048u) {}
            c_off += SLOT; c_bar += 8;
            if (c_off == DEPTH * SLOT) { c_off = 0; c_bar = bar0; c_phase ^= 1u; }
        }
    }
}

// Load-time re-tiling of one stacked projection pair (gate and up) or of one projection into the stream layout
// described at the top.  One block per (expert, 16-row block, cell); thread c writes 16-byte chunk c.
//   out[((e*n_rb + rb)*n_cells + cell) * NP*576 + proj*576 + {0: packed words, 512: scale words}],  NP = 2 for gate/up
__global__ void retile_stream_kernel(const uint32_t* __restrict__ w1, const uint16_t* __restrict__ s1, const uint16_t* __restrict__ b1,
                                     const uint32_t* __restrict__ w2, const uint16_t* __restrict__ s2, const uint16_t* __restrict__ b2,
                                     uint8_t* __restrict__ out, int N, int K, int group_size) {
    const int np = w2 != nullptr ? 2 : 1;
    const int n_cells = K / 64, wpr = K / 8, gpr = K / group_size;
    const size_t cell_id = blockIdx.x;       // (e*n_rb + rb)*n_cells + cell
    const int cell = (int)(cell_id % n_cells);
    const size_t row0 = (cell_id / n_cells) * 16;   // e*N + rb*16
    const int c = threadIdx.x;               // chunk: proj * 36 + {0..31: words of lane c, 32..35: scale words}
    if (c >= np * 36) return;
    const int proj = c / 36, cc = c - proj * 36;
    const uint32_t* w = proj ? w2 : w1;
    const uint16_t* s = proj ? s2 : s1;
    const uint16_t* b = proj ? b2 : b1;
    uint8_t* dst = out + cell_id * (size_t)(np * CELL) + proj * CELL;
    if (cc < 32) {
        const int gg = cc >> 2, tt = cc & 3;
        const uint32_t* lo = w + (row0 + gg) * wpr + cell * 8 + 2 * tt;
        const uint32_t* hi = w + (row0 + gg + 8) * wpr + cell * 8 + 2 * tt;
        *reinterpret_cast<uint4*>(dst + cc * 16) = make_uint4(lo[0], lo[1], hi[0], hi[1]);
    } else {
        const int j = cc - 32;   // entries 4j..4j+3 = rows (g = 2j, +0), (2j, +8), (2j+1, +0), (2j+1, +8)
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int gg = 2 * j + (i >> 1), h = i & 1;
            const size_t src = (row0 + gg + 8 * h) * gpr + (size_t)(cell * 64 / group_size);
            o[i] = (uint32_t)s[src] | ((uint32_t)b[src] << 16);
        }
        *reinterpret_cast<uint4*>(dst + CELL_W + j * 16) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

}  // namespace dstr
}  // namespace ffai
