// Grouped 4-bit dequant GEMM for sm_100a: TMA -> shared memory -> in-SMEM dequant ->
// tcgen05.mma with TMEM accumulators -> fused activation epilogue.
//
// Replaces the reference's grouped int4 matmuls over expert-sorted rows
// (Ops.moeGatherDequantGemmInt4 and its Bm8 / Bm64Mpp tiles, FFAI Ops.swift:4553-4708,
// 4912-5201) together with Ops.swiglu between them (Ops.swift:6400-6452):
//     out[row, n] = sum_k (scale[e,n,k/gs] * q[e,n,k] + bias[e,n,k/gs]) * x[row, k],   e = expert of row.
//
// Orientation: the activation rows routed to an expert are the M side of the MMA (128 rows per
// tile, one TMEM lane each); the weight rows are the N side, 256 per instruction - for gate/up the
// 128 gate rows and the 128 matching up rows of the expert, so one tcgen05.mma (128 x 256 x 16)
// feeds both halves of the activation and a thread of the epilogue finds gate and up of one output
// element in its own TMEM lane.  (Measured with the device timeline: one tcgen05.mma costs its
// issuing thread 80-100 clk whatever its N; only N = 256 keeps the tensor pipe busy that long.)
//
// Warp roles in a 768-thread CTA (persistent; work items are (expert, 128 routed rows, weight-row tile)):
//   warp 0       producer of weights.  Packed 4-bit: two TMA boxes of [128 rows x 128 B] (256 k) per stage,
//                128-byte swizzle, ring "W".  bf16 weights (WBF16: expanded once at load time into tile-major,
//                pre-swizzled 16 KB tiles): two contiguous bulk copies per 64 k straight into the operand ring "B".
//   warp 2       TMA producer of activations: [128 rows x 128 B] per 64 k, 128-byte swizzle, ring "X"
//   warp 3       scheduler: finds the expert, row range and weight tile of each of the CTA's work items (a 32-way
//                search over the tile prefix sums) and hands them to every other role through a small ring in
//                shared memory, so no role waits on a chain of global loads at an item boundary
//   warp 1       MMA issuer (one thread): 4 x tcgen05.mma (M128 N256 K16) per 64 k; owns TMEM
//                (two accumulators of 256 columns, so the epilogue of a tile overlaps the next tile)
//   warps 4-19   dequant (packed weights only): two groups of 256 threads that take alternate 64-k blocks,
//                thread = weight row; unpack 4-bit to bf16 (w = fma(q, scale, bias) rounded once), store into
//                the 128-byte-swizzled K-major operand tile, ring "B"
//   warps 20-23  epilogue: tcgen05.ld 8 or 16 columns at a time with the next chunk's load in flight,
//                bias + activation (one special-function op per element), 16-byte stores
// Every mbarrier wait is bounded (about one second); on expiry the kernel raises an error
// word, stops issuing work, waits (bounded) for its own copies in flight, frees TMEM and returns.
//
// K order: a 4-bit word holds 8 consecutive k.  The unpack yields the pairs (0,4),(1,5),(2,6),(3,7),
// so operand tiles keep every 8-run in the order 0,4,1,5,2,6,3,7.  The activation side is written
// in the same order by its producer (the row gather, or the previous GEMM's epilogue), which makes
// the permutation invisible to the dot product.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace ffai {
namespace g100 {

constexpr int BM = 128;        // activation rows per tile (the MMA's M: one TMEM lane each)
constexpr int BN = 256;        // weight rows per tile (the MMA's N: one fp32 TMEM column each)
constexpr int BK = 64;         // k per MMA stage (one 128-byte swizzle row of bf16)
constexpr int KS = 256;        // k per packed-weight TMA box (one 128-byte row of 4-bit values)
constexpr int SUB = KS / BK;   // MMA stages per packed-weight stage
constexpr int SPF = 4;         // 64-k blocks of scale words a dequant thread fetches ahead
constexpr int THREADS = 768;   // 24 warps
constexpr int W_WARP = 0;      // packed-weight TMA producer
constexpr int MMA_WARP = 1;    // MMA issuer, owns TMEM
constexpr int X_WARP = 2;      // activation TMA producer
constexpr int SCHED_WARP = 3;  // work-item scheduler: resolves (expert, rows, weight tile) ahead of the other roles
constexpr int NSCHED = 8;      // work items the scheduler may run ahead
constexpr int DEQ_WARP0 = 4;   // first of the dequant warps
constexpr int N_DEQ_WARPS = 16;
constexpr int EPI_WARP0 = 20;  // four epilogue warps, warp % 4 = TMEM lane quadrant
constexpr uint64_t WAIT_LIMIT_NS = 1000000000ull;

enum : uint32_t { ERR_NONE = 0, ERR_WAIT_TIMEOUT = 1 };

struct Params {
    const uint16_t* scales;    // [E, n_out, K/gs]
    const uint16_t* biases;
    const uint16_t* row_bias;  // nullable [E, n_out]
    const uint16_t* scales2;   // second projection (fused gate/up)
    const uint16_t* biases2;
    const uint16_t* row_bias2;
    const uint16_t* wcache;    // WBF16: the projection's tile-major bf16 cache, [E, cache_blocks, K/64] tiles of 16 KB
    const uint16_t* wcache2;   // WBF16, fused gate/up: the up projection's cache
    int cache_blocks;          // 128-row blocks per expert in a cache
    const uint32_t* sb;        // nullable: (scale | bias << 16) words re-tiled [E, n_out/16, K/64, 16] (group 64 or 128)
    const uint32_t* sb2;
    int n_out;                 // output rows per expert
    int K;
    int group_size;
    int n_experts;
    const uint32_t* offsets;       // [E+1] row ranges per expert in the sorted row space
    const uint32_t* tile_offsets;  // [E+1] prefix sum of token tiles per expert
    int m_tiles;                   // ceil(n_out / 128)
    int activation;
    float limit, alpha;
    void* out;                 // [rows, out_ld]
    int out_ld;
    int out_permute8;          // 1: store column n at (n & ~7) | {0,2,4,6,1,3,5,7}[n & 7]
    uint32_t* error_word;
    long long* timeline;       // nullable: CTA 0 records clock64() per role / k block / event (TL_* layout)
};

// Timeline layout: [role][k-block index < TL_SLOTS][event < TL_EVENTS].
constexpr int TL_ROLES = 5, TL_SLOTS = 96, TL_EVENTS = 4;
enum { TL_WPROD = 0, TL_XPROD = 1, TL_MMA = 2, TL_DEQ = 3, TL_EPI = 4 };
#ifndef FFAI_G100_TIMELINE
#define FFAI_G100_TIMELINE 0   // 1: compile the timeline marks in (profiling builds); 0: they vanish
#endif
FFAI_DEVINL void tl_mark(const Params& p, int role, int idx, int ev) {
#if FFAI_G100_TIMELINE
    if (p.timeline && blockIdx.x == 0 && idx < TL_SLOTS)
        p.timeline[(role * TL_SLOTS + idx) * TL_EVENTS + ev] = clock64();
#else
    (void)p; (void)role; (void)idx; (void)ev;
#endif
}

// ───────────────────────── PTX wrappers ─────────────────────────

FFAI_DEVINL uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

FFAI_DEVINL uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

FFAI_DEVINL void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
FFAI_DEVINL void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
FFAI_DEVINL void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
FFAI_DEVINL bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(20000u)   // the thread may stay suspended up to 20 us per try; it wakes when the phase completes
        : "memory");
    return done != 0;
}
// Bounded wait.  Returns false when the limit expires or another thread of the CTA gave up.
// Waiting threads are suspended by the hardware inside try_wait (time hint), so they take no issue slots.
template <int SLEEP_NS>
FFAI_DEVINL bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    uint64_t t0 = 0;
    for (uint32_t spin = 1;; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 7u) == 0) {  // the slow checks, once per 8 tries (each try may sleep up to 20 us)
            if (*abort_flag) return false;
            const uint64_t now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > WAIT_LIMIT_NS) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}

// Ring position: stage index and phase bit, advanced without division.
struct RingPos {
    int stage;
    uint32_t phase;
    FFAI_DEVINL void advance(int depth) {
        if (++stage == depth) { stage = 0; phase ^= 1u; }
    }
};

FFAI_DEVINL void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
// Contiguous bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), completion on the mbarrier.
FFAI_DEVINL void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
FFAI_DEVINL void prefetch_tmap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

FFAI_DEVINL void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
FFAI_DEVINL void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
FFAI_DEVINL void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
FFAI_DEVINL void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

FFAI_DEVINL void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
FFAI_DEVINL void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
FFAI_DEVINL void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]^T, bf16 inputs, fp32 accumulate.
FFAI_DEVINL void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// mbarrier arrives once all tcgen05 operations issued so far by this thread have completed.
FFAI_DEVINL void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

FFAI_DEVINL void tmem_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
FFAI_DEVINL void tmem_ld8(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
        : "r"(taddr)
        : "memory");
}
template <int N>
FFAI_DEVINL void tmem_ld_n(uint32_t taddr, uint32_t* r) {
    if (N == 8) tmem_ld8(taddr, r); else tmem_ld16(taddr, r);
}
FFAI_DEVINL void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major operand tile in shared memory, 128-byte swizzle: rows of 128 bytes (64 bf16),
// 8-row groups 1024 bytes apart.  Descriptor fields (sm_100 shared-memory matrix descriptor):
// start>>4 [0,14), leading byte offset>>4 [16,30) (unused for swizzled K-major), stride byte
// offset>>4 [32,46) = 1024>>4, version 1 at [46,48), swizzle mode 2 (128 B) at [61,64).
FFAI_DEVINL uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// kind::f16 instruction descriptor: D fp32 (bit 4), A bf16 (bit 7), B bf16 (bit 10), both
// K-major (bits 15, 16 clear), N>>3 at [17,23), M>>4 at [24,29).
FFAI_DEVINL uint32_t make_idesc_bf16(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// One packed word (8 x 4-bit) -> 8 bf16 weights in the order 0,4,1,5,2,6,3,7 as 4 packed pairs.
// (q | 0x4300) is the bf16 value 128+q exactly; subtracting 128 is exact; the fused
// multiply-add rounds scale*q+bias to bf16 once.
FFAI_DEVINL uint4 dequant_word_bf16(uint32_t w, __nv_bfloat162 s2, __nv_bfloat162 b2) {
    const __nv_bfloat162 k128 = __floats2bfloat162_rn(128.0f, 128.0f);
    uint32_t t[4];
    t[0] = (w & 0x000F000Fu) | 0x43004300u;
    // right shifts as high halves of multiplies: they issue on the FMA pipe instead of the half-rate ALU pipe
    t[1] = (__umulhi(w, 1u << 28) & 0x000F000Fu) | 0x43004300u;
    t[2] = (__umulhi(w, 1u << 24) & 0x000F000Fu) | 0x43004300u;
    t[3] = (__umulhi(w, 1u << 20) & 0x000F000Fu) | 0x43004300u;
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __nv_bfloat162 q = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&t[i]), k128);
        __nv_bfloat162 v = __hfma2(q, s2, b2);
        o[i] = *reinterpret_cast<uint32_t*>(&v);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

// Two floats -> packed bf16 pair (lo, hi), round to nearest even, one convert instruction.
FFAI_DEVINL uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

FFAI_DEVINL int permute8_store_col(int n) {
    // k 0..7 live at positions 0,2,4,6,1,3,5,7 of their 8-run
    const int k = n & 7;
    return (n & ~7) | (((k & 3) << 1) | (k >> 2));
}

// A work item is (expert, token tile of up to 128 routed rows, weight-row tile).  Consecutive items share
// the rows so the activation tiles stay hot in L2 across the CTAs that work on one expert.
// n_cols_valid counts the item's rows (1..128).
struct TileCoord {
    int expert, row_begin, n_cols_valid, m_tile;
};

// The scheduler warp's search: the last e in [0, n_experts) with tile_offsets[e] <= g, 32 candidates per round.
FFAI_DEVINL int find_group_warp(const uint32_t* __restrict__ tile_offsets, int n_experts, int g, int lane) {
    int lo = 0, n = n_experts;
    while (n > 1) {
        const int step = (n + 31) >> 5;
        const int idx = lo + lane * step;
        const bool le = idx < lo + n && (int)__ldg(tile_offsets + idx) <= g;
        const int c = __popc(__ballot_sync(0xFFFFFFFFu, le));   // monotone: lanes 0..c-1 hold values <= g (c >= 1)
        const int nlo = lo + (c - 1) * step;
        n = min(step, lo + n - nlo);
        lo = nlo;
    }
    return lo;
}

// A role's view of the scheduler ring: wait for the next item's coordinates, copy them, release the slot.
struct ItemFeed {
    uint32_t full0, empty0, coords0;   // shared-window addresses
    uint32_t i;
    // whole_warp: every lane of the warp calls (and reads); lane 0 releases the slot once all have read
    FFAI_DEVINL bool take(TileCoord& c, volatile uint32_t* abort_flag, bool whole_warp) {
        const uint32_t slot = i % NSCHED, phase = (i / NSCHED) & 1u;
        ++i;
        if (!mbar_wait<32>(full0 + 8u * slot, phase, abort_flag)) return false;
        uint32_t a, b, d, e;
        asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(a), "=r"(b), "=r"(d), "=r"(e) : "r"(coords0 + 16u * slot));
        c.expert = (int)a; c.row_begin = (int)b; c.n_cols_valid = (int)d; c.m_tile = (int)e;
        if (whole_warp) {
            __syncwarp();
            if ((threadIdx.x & 31) == 0) mbar_arrive(empty0 + 8u * slot);
        } else {
            mbar_arrive(empty0 + 8u * slot);
        }
        return true;
    }
};

// Ring depths.  Both TMA-fed rings must hold enough 64-k stages to cover the latency of a bulk copy
// (a few thousand cycles) at one stage per ~540 cycles of tensor-pipe time, or the MMA issuer idles.
//   packed weights: operand ring 3 x 32 KB (filled by the dequant warps), packed ring 2 x 32 KB, activations 4 x 16 KB
//                   (a packed ring of 4 x 16 KB with 64-byte unswizzled boxes measured slower)
//   bf16 weights:   operand ring 4 x 32 KB (filled by TMA), no packed ring, activations 5 x 16 KB
template <bool WBF16>
struct SmemLayout {
    static constexpr int B_STAGE = BN * BK * 2;            // 32 KB: 256 weight rows x 64 k, bf16
#ifndef FFAI_G100_NB_PACKED
#define FFAI_G100_NB_PACKED 3
#define FFAI_G100_NX_PACKED 4
#define FFAI_G100_NB_BF16 4
#define FFAI_G100_NX_BF16 5
#endif
    static constexpr int NB = WBF16 ? FFAI_G100_NB_BF16 : FFAI_G100_NB_PACKED;   // operand ring
    static constexpr int W_STAGE = BN * (KS / 2);          // 32 KB: 256 weight rows x 256 k, packed 4-bit
    static constexpr int NW = WBF16 ? 0 : 2;               // packed-weight ring (256-k super blocks)
    static constexpr int X_TILE = BM * BK * 2;             // 16 KB: 128 activation rows x 64 k
    static constexpr int NX = WBF16 ? FFAI_G100_NX_BF16 : FFAI_G100_NX_PACKED;   // activation ring
    static constexpr int OFF_B = 0;
    static constexpr int OFF_W = OFF_B + NB * B_STAGE;
    static constexpr int OFF_X = OFF_W + NW * W_STAGE;
    static constexpr int OFF_BAR = OFF_X + NX * X_TILE;
    static constexpr int N_BARS = 2 * NW + 2 * NX + 2 * NB + 4 + 2 * NSCHED;
    static constexpr int OFF_SCHED = OFF_BAR + N_BARS * 8 + 16;     // NSCHED x 16 bytes of item coordinates
    static constexpr int N_ITEM_READERS = 3 + (WBF16 ? 0 : N_DEQ_WARPS) + 4;   // warps that take every work item
    static constexpr int TOTAL = OFF_SCHED + NSCHED * 16 + 1024;    // + alignment slack
    static constexpr int TMEM_COLS = 2 * BN;               // two accumulators of 256 fp32 columns
    static_assert(TOTAL <= 227 * 1024, "shared memory limit");
};

// One CTA tile: 128 activation rows (the MMA's M, one TMEM lane each) x 256 weight rows (the MMA's N).
// FUSED:  the 256 weight rows are 128 gate rows and the 128 matching up rows of one expert;
//         out[row, n] = act(Wg[e][n]·x[row] + bg, Wu[e][n]·x[row] + bu), bf16, optionally 8-run permuted
// !FUSED: 256 consecutive rows of one projection;  out[row, n] = W[e][n]·x[row] + b, TOut
// WBF16: the weights are already bf16 operand tiles (tile-major cache, 8-runs permuted like the
//         activations, 128-byte swizzle applied): the weight producer copies them straight into the operand
//         ring and the dequant warps have nothing to do.  Used for projections that were expanded once at load time
//         (bit widths other than 4).
template <bool FUSED, typename TOut, bool WBF16>
__global__ void __launch_bounds__(THREADS, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_w2,
                    const __grid_constant__ CUtensorMap tm_x, const Params p) {
    using L = SmemLayout<WBF16>;
    constexpr int NB = L::NB;
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment for the swizzled tiles
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar0 = sbase + L::OFF_BAR;
    auto w_full = [&](int s) { return bar0 + 8u * s; };
    auto w_empty = [&](int s) { return bar0 + 8u * (L::NW + s); };
    auto x_full = [&](int s) { return bar0 + 8u * (2 * L::NW + s); };
    auto x_empty = [&](int s) { return bar0 + 8u * (2 * L::NW + L::NX + s); };
    auto b_full = [&](int s) { return bar0 + 8u * (2 * L::NW + 2 * L::NX + s); };
    auto b_empty = [&](int s) { return bar0 + 8u * (2 * L::NW + 2 * L::NX + NB + s); };
    auto acc_full = [&](int b) { return bar0 + 8u * (2 * L::NW + 2 * L::NX + 2 * NB + b); };
    auto acc_empty = [&](int b) { return bar0 + 8u * (2 * L::NW + 2 * L::NX + 2 * NB + 2 + b); };
    auto s_full = [&](int s) { return bar0 + 8u * (2 * L::NW + 2 * L::NX + 2 * NB + 4 + s); };
    auto s_empty = [&](int s) { return bar0 + 8u * (2 * L::NW + 2 * L::NX + 2 * NB + 4 + NSCHED + s); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + L::OFF_BAR + L::N_BARS * 8);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KB = p.K / BK;                 // 64-k blocks
    const int SB = (KB + SUB - 1) / SUB;     // 256-k super blocks
    const int total_tiles = (int)p.tile_offsets[p.n_experts] * p.m_tiles;
    constexpr int ROWS_PER_TILE = FUSED ? BN / 2 : BN;   // output rows of one projection covered by a tile

    if (threadIdx.x == 0) {
        for (int s = 0; s < L::NW; ++s) { mbar_init(w_full(s), 1); mbar_init(w_empty(s), N_DEQ_WARPS); }
        for (int s = 0; s < L::NX; ++s) { mbar_init(x_full(s), 1); mbar_init(x_empty(s), 1); }
        for (int s = 0; s < NB; ++s) { mbar_init(b_full(s), WBF16 ? 1 : N_DEQ_WARPS / 2); mbar_init(b_empty(s), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full(b), 1); mbar_init(acc_empty(b), 4); }
        for (int s = 0; s < NSCHED; ++s) { mbar_init(s_full(s), 1); mbar_init(s_empty(s), L::N_ITEM_READERS); }
        *abort_flag = 0;
        fence_barrier_init();
        if (!WBF16) {
            prefetch_tmap(&tm_w);
            if (FUSED) prefetch_tmap(&tm_w2);
        }
        prefetch_tmap(&tm_x);
    }
    if (warp == MMA_WARP) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), L::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    ItemFeed feed{s_full(0), s_empty(0), sbase + (uint32_t)L::OFF_SCHED, 0u};

    if (warp == W_WARP && WBF16) {
        // ───────────── producer, bf16 weights: two contiguous 16 KB tiles per 64 k, into the operand ring ─────────────
        // The cache holds every (expert, 128-row block, 64-k block) tile contiguously and already swizzled, so a
        // tile is one bulk copy of consecutive bytes: full DRAM pages instead of 128 rows of 128 bytes 4 KB apart.
        if (lane == 0) {
            RingPos bp{0, 0};
            uint32_t issued = 0;
            bool ok = true;
            constexpr uint32_t TILE = BM * BK * 2;   // 16 KB
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                TileCoord c;
                if (!feed.take(c, abort_flag, false)) { ok = false; break; }
                const size_t blk = (size_t)c.expert * p.cache_blocks + (FUSED ? c.m_tile : 2 * c.m_tile);
                const uint8_t* src0 = reinterpret_cast<const uint8_t*>(p.wcache) + blk * KB * TILE;
                const uint8_t* src1 = FUSED ? reinterpret_cast<const uint8_t*>(p.wcache2) + blk * KB * TILE
                                            : src0 + (size_t)KB * TILE;   // the next 128-row block of the projection
                for (int kb = 0; kb < KB; ++kb) {
                    if (!mbar_wait<64>(b_empty(bp.stage), bp.phase ^ 1, abort_flag)) { ok = false; break; }
                    const uint32_t stage = sbase + L::OFF_B + bp.stage * L::B_STAGE;
                    mbar_arrive_expect_tx(b_full(bp.stage), L::B_STAGE);
                    bulk_load_1d(stage, src0 + (size_t)kb * TILE, TILE, b_full(bp.stage));
                    bulk_load_1d(stage + L::B_STAGE / 2, src1 + (size_t)kb * TILE, TILE, b_full(bp.stage));
                    bp.advance(NB);
                    ++issued;
                }
            }
            if (!ok) {
                const uint32_t first = issued > (uint32_t)NB ? issued - NB : 0;
                for (uint32_t j = first; j < issued; ++j) {
                    const uint64_t t0 = global_timer_ns();
                    while (!mbar_try_wait(b_full(j % NB), (j / NB) & 1) && global_timer_ns() - t0 < 2000000ull) {}
                }
            }
        }
    } else if (warp == W_WARP) {
        // ───────────── TMA producer, packed weights: two 128-row x 128-byte boxes per 256 k ─────────────
        if (lane == 0) {
            RingPos wp{0, 0};
            uint32_t issued = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                TileCoord c;
                if (!feed.take(c, abort_flag, false)) { ok = false; break; }
                const int wrow = c.expert * p.n_out + c.m_tile * ROWS_PER_TILE;
                for (int sb = 0; sb < SB; ++sb) {
                    tl_mark(p, TL_WPROD, (int)issued, 0);
                    if (!mbar_wait<64>(w_empty(wp.stage), wp.phase ^ 1, abort_flag)) { ok = false; break; }
                    tl_mark(p, TL_WPROD, (int)issued, 1);
                    const uint32_t stage = sbase + L::OFF_W + wp.stage * L::W_STAGE;
                    mbar_arrive_expect_tx(w_full(wp.stage), L::W_STAGE);
                    tma_load_2d(stage, &tm_w, sb * (KS / 8), wrow, w_full(wp.stage));
                    if (FUSED) tma_load_2d(stage + L::W_STAGE / 2, &tm_w2, sb * (KS / 8), wrow, w_full(wp.stage));
                    else tma_load_2d(stage + L::W_STAGE / 2, &tm_w, sb * (KS / 8), wrow + BN / 2, w_full(wp.stage));
                    wp.advance(L::NW);
                    ++issued;
                }
            }
            if (!ok) {
                // copies already issued still land in this CTA's shared memory: wait for them (bounded, 2 ms each)
                constexpr uint32_t NWd = L::NW > 0 ? L::NW : 1;   // (this branch is never taken without a packed ring)
                const uint32_t first = issued > NWd ? issued - NWd : 0;
                for (uint32_t j = first; j < issued; ++j) {
                    const uint64_t t0 = global_timer_ns();
                    while (!mbar_try_wait(w_full(j % NWd), (j / NWd) & 1) && global_timer_ns() - t0 < 2000000ull) {}
                }
            }
        }
    } else if (warp == X_WARP) {
        // ───────────── TMA producer, activations: 128 rows x 128 bytes per 64 k ─────────────
        if (lane == 0) {
            RingPos xp{0, 0};
            uint32_t issued = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                TileCoord c;
                if (!feed.take(c, abort_flag, false)) { ok = false; break; }
                for (int kb = 0; kb < KB; ++kb) {
                    if (!mbar_wait<32>(x_empty(xp.stage), xp.phase ^ 1, abort_flag)) { ok = false; break; }
                    mbar_arrive_expect_tx(x_full(xp.stage), L::X_TILE);
                    tma_load_2d(sbase + L::OFF_X + xp.stage * L::X_TILE, &tm_x, kb * BK, c.row_begin, x_full(xp.stage));
                    xp.advance(L::NX);
                    ++issued;
                }
            }
            if (!ok) {
                const uint32_t first = issued > (uint32_t)L::NX ? issued - L::NX : 0;
                for (uint32_t j = first; j < issued; ++j) {
                    const uint64_t t0 = global_timer_ns();
                    while (!mbar_try_wait(x_full(j % L::NX), (j / L::NX) & 1) && global_timer_ns() - t0 < 2000000ull) {}
                }
            }
        }
    } else if (warp == MMA_WARP) {
        // ───────────── MMA issuer: 4 x (128 x 256 x 16) per 64 k ─────────────
        if (lane == 0) {
            RingPos xp{0, 0}, bp{0, 0};
            uint32_t tcount = 0;
            int gk = 0;
            bool ok = true;
            const uint32_t idesc = make_idesc_bf16(BM, BN);
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                TileCoord c;
                if (!feed.take(c, abort_flag, false)) { ok = false; break; }
                // the item accumulates in TMEM buffer tcount & 1
                if (!mbar_wait<32>(acc_empty(tcount & 1), ((tcount >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
                const uint32_t d0 = tmem_base + (uint32_t)((tcount & 1) * BN);
                tc_fence_after();
                for (int kb = 0; kb < KB && ok; ++kb, ++gk) {
                    tl_mark(p, TL_MMA, gk, 2);
                    if (!mbar_wait<0>(b_full(bp.stage), bp.phase, abort_flag)) { ok = false; break; }
                    if (!mbar_wait<0>(x_full(xp.stage), xp.phase, abort_flag)) { ok = false; break; }
                    tl_mark(p, TL_MMA, gk, 0);
                    tc_fence_after();
                    const uint64_t bd0 = make_kmajor_sw128_desc(sbase + L::OFF_B + bp.stage * L::B_STAGE);
                    const uint64_t ad0 = make_kmajor_sw128_desc(sbase + L::OFF_X + xp.stage * L::X_TILE);
#pragma unroll
                    for (int k16 = 0; k16 < BK / 16; ++k16) {
                        // advancing 16 k inside the swizzled row = +32 bytes = +2 in the (addr >> 4) field
                        umma_bf16(d0, ad0 + 2 * k16, bd0 + 2 * k16, idesc, (kb | k16) != 0 ? 1u : 0u);
                    }
                    tl_mark(p, TL_MMA, gk, 1);
                    umma_commit(x_empty(xp.stage));
                    umma_commit(b_empty(bp.stage));
                    tl_mark(p, TL_MMA, gk, 3);
                    xp.advance(L::NX);
                    bp.advance(NB);
                }
                if (ok) umma_commit(acc_full(tcount & 1));
                ++tcount;
            }
        }
    } else if (!WBF16 && warp >= DEQ_WARP0 && warp < DEQ_WARP0 + N_DEQ_WARPS) {
        // ───────────── dequant: two groups of 8 warps, a group takes every other 64-k block ─────────────
        // Thread = one weight row of the 256-row stage; in a block of its group it turns the row's 8 packed words
        // (two 16-byte reads) into 64 bf16 (eight 16-byte stores).  Eight consecutive rows per quarter-warp, so the
        // reads of the 128-byte-swizzled packed tile and the stores into the 128-byte-swizzled operand tile
        // touch eight distinct chunk columns: no bank conflicts either way.  Per word: 4 logic ops (mask and
        // exponent held in registers so each pair is one instruction), 3 shifts, 4 subtract-128 and 4 fused
        // multiply-adds on bf16 pairs.  The two groups work on different operand stages at the same time, so
        // one group's waits and fences overlap the other group's arithmetic; blocks are counted over the CTA's
        // whole run, so the alternation carries across work items whatever K is.
        const int dw = warp - DEQ_WARP0;
        const uint32_t grp = (uint32_t)dw >> 3;
        const int r = (dw & 7) * 32 + lane;                         // 0..255
        const int gpr = p.K / p.group_size;
        const int gshift = p.group_size == 32 ? 5 : (p.group_size == 64 ? 6 : 7);
        const bool second = FUSED && r >= BN / 2;                   // the up projection's half of the tile
        const uint16_t* sbase_ptr = second ? p.scales2 : p.scales;
        const uint16_t* bbase_ptr = second ? p.biases2 : p.biases;
        const uint32_t* sbw_ptr = second ? p.sb2 : p.sb;            // nullable: repacked (scale | bias << 16) words
        const int r_in_proj = FUSED ? (r & (BN / 2 - 1)) : r;
        uint32_t mask, expo;
        asm volatile("mov.u32 %0, 0x000F000F;" : "=r"(mask));
        asm volatile("mov.u32 %0, 0x43004300;" : "=r"(expo));       // also the bf16 pair (128, 128)
        // shared-window addresses of this thread's row in stage 0 of both rings; a 16-byte piece c of the row
        // sits at ((c << 4) ^ swz) in either ring
        const uint32_t w_row0 = sbase + L::OFF_W + r * (KS / 2);
        const uint32_t b_row0 = sbase + L::OFF_B + r * 128;
        const uint32_t swz = (uint32_t)(r & 7) << 4;
        RingPos wp{0, 0}, bp{0, 0};
        if (grp) bp.advance(NB);                                    // the group's first block is block grp of the run
        uint32_t blocks_before = 0;                                 // 64-k blocks of the work items so far
        bool ok = true;
        int gk = 0;
        const bool tl_on = (warp == DEQ_WARP0 && lane == 0);
        // Where a row's scales and biases live, for one work item.
        struct RowScales {
            const uint16_t *sp, *bq;
            const uint32_t* sw;
            int j0;   // the group's blocks of a packed stage are j0 and j0 + 2
        };
        auto row_scales = [&](const TileCoord& c, uint32_t blocks_before_item) {
            int prow = c.m_tile * ROWS_PER_TILE + r_in_proj;        // row within the expert's projection
            if (prow >= p.n_out) prow = p.n_out - 1;                // rows past the projection: zero-filled by TMA, masked at store
            const long grow = (long)c.expert * p.n_out + prow;
            RowScales rs;
            rs.sp = sbase_ptr + grow * gpr;
            rs.bq = bbase_ptr + grow * gpr;
            rs.sw = sbw_ptr ? sbw_ptr + (((size_t)c.expert * (p.n_out >> 4) + (prow >> 4)) * KB) * 16 + (prow & 15) : nullptr;
            rs.j0 = (int)((grp ^ blocks_before_item) & 1u);
            return rs;
        };
        // (scale | bias << 16) of both 32-k halves of the group's two blocks of a packed stage, fetched one packed
        // stage ahead - across work items too: the first stage of the next item is fetched during the last
        // stage of this one, so no item starts by waiting for its scales.
        uint32_t nxt[2][2];
        auto fetch_scales = [&](const RowScales& rs, int kb0) {
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {
                const int kb = min(kb0 + rs.j0 + 2 * jj, KB - 1);
                if (rs.sw) {
                    nxt[jj][0] = __ldg(rs.sw + (size_t)kb * 16);
                    nxt[jj][1] = nxt[jj][0];
                } else {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int g = (kb * BK + h * 32) >> gshift;
                        nxt[jj][h] = (uint32_t)rs.sp[g] | ((uint32_t)rs.bq[g] << 16);
                    }
                }
            }
        };
        TileCoord c_next;
        bool have_next = blockIdx.x < total_tiles && feed.take(c_next, abort_flag, true);
        RowScales rs_next{};
        if (have_next) {
            rs_next = row_scales(c_next, 0u);
            fetch_scales(rs_next, 0);
        }
        for (int tile = blockIdx.x; tile < total_tiles && ok && have_next; tile += gridDim.x) {
            const RowScales rs = rs_next;
            const int j0 = rs.j0;
            have_next = tile + (int)gridDim.x < total_tiles && feed.take(c_next, abort_flag, true);
            if (have_next) rs_next = row_scales(c_next, blocks_before + (uint32_t)KB);
            else if (tile + (int)gridDim.x < total_tiles) ok = false;   // gave up waiting for the scheduler
            for (int kb0 = 0; kb0 < KB && ok; kb0 += SUB) {
                uint32_t cur[2][2];
#pragma unroll
                for (int jj = 0; jj < 2; ++jj) { cur[jj][0] = nxt[jj][0]; cur[jj][1] = nxt[jj][1]; }
                if (kb0 + SUB < KB) fetch_scales(rs, kb0 + SUB);
                else if (have_next) fetch_scales(rs_next, 0);
                const int nblk = min(SUB, KB - kb0);
                if (j0 < nblk) {
                    if (!mbar_wait<0>(w_full(wp.stage), wp.phase, abort_flag)) { ok = false; break; }
                    const uint32_t w_row = w_row0 + wp.stage * L::W_STAGE;
#pragma unroll
                    for (int jj = 0; jj < 2; ++jj) {
                        const int j = j0 + 2 * jj;
                        if (j >= nblk) break;
                        if (tl_on) tl_mark(p, TL_DEQ, gk, 0);
                        uint32_t w8[8];
                        asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];"
                                     : "=r"(w8[0]), "=r"(w8[1]), "=r"(w8[2]), "=r"(w8[3]) : "r"(w_row + (((uint32_t)(2 * j) << 4) ^ swz)));
                        asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];"
                                     : "=r"(w8[4]), "=r"(w8[5]), "=r"(w8[6]), "=r"(w8[7]) : "r"(w_row + (((uint32_t)(2 * j + 1) << 4) ^ swz)));
                        if (!mbar_wait<0>(b_empty(bp.stage), bp.phase ^ 1, abort_flag)) { ok = false; break; }
                        if (tl_on) tl_mark(p, TL_DEQ, gk, 1);
                        const uint32_t b_row = b_row0 + bp.stage * L::B_STAGE;
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const uint32_t sbv = cur[jj][h];
                            const uint32_t s2 = __byte_perm(sbv, sbv, 0x1010), b2 = __byte_perm(sbv, sbv, 0x3232);
#pragma unroll
                            for (int q4 = 0; q4 < 4; ++q4) {
                                const uint32_t w = w8[h * 4 + q4];
                                uint32_t o[4];
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    uint32_t t, q;
                                    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(t) : "r"(i == 0 ? w : (w >> (4 * i))), "r"(mask), "r"(expo));
                                    asm("sub.bf16x2 %0, %1, %2;" : "=r"(q) : "r"(t), "r"(expo));
                                    asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(o[i]) : "r"(q), "r"(s2), "r"(b2));
                                }
                                asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};"
                                             ::"r"(b_row + (((uint32_t)(h * 4 + q4) << 4) ^ swz)), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]) : "memory");
                            }
                        }
                        if (tl_on) tl_mark(p, TL_DEQ, gk, 2);
                        fence_proxy_async_smem();  // generic-proxy stores -> visible to the tensor core's async proxy
                        __syncwarp();
                        if (lane == 0) mbar_arrive(b_full(bp.stage));
                        if (tl_on) tl_mark(p, TL_DEQ, gk, 3);
                        ++gk;
                        bp.advance(NB);
                        bp.advance(NB);
                    }
                    if (!ok) break;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(w_empty(wp.stage));  // this warp is done with the packed stage (or has no block in it)
                wp.advance(L::NW);
            }
            blocks_before += (uint32_t)KB;
        }
    } else if (warp >= EPI_WARP0) {
        // ───────────── epilogue: thread = activation row (TMEM lane), walks the 256 accumulator columns ─────────────
        const int q = warp & 3;  // TMEM lane quadrant this warp may read
        uint32_t tcount = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            TileCoord c;
            if (!feed.take(c, abort_flag, true)) break;
            const int buf = tcount & 1;
            const uint32_t acc_ph = (tcount >> 1) & 1;
            if (warp == EPI_WARP0 && lane == 0) tl_mark(p, TL_EPI, (int)tcount, 0);
            if (!mbar_wait<256>(acc_full(buf), acc_ph, abort_flag)) { ok = false; break; }
            if (warp == EPI_WARP0 && lane == 0) tl_mark(p, TL_EPI, (int)tcount, 1);
            tc_fence_after();
            const int tok = q * 32 + lane;                      // activation row within the tile
            const bool tok_ok = tok < c.n_cols_valid;
            const int n0 = c.m_tile * ROWS_PER_TILE;            // first output row of the tile
            const uint32_t t0 = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN);
            const size_t ebase = (size_t)c.expert * p.n_out;
            uint8_t* orow = reinterpret_cast<uint8_t*>(p.out) + (size_t)(c.row_begin + tok) * p.out_ld * sizeof(TOut);
            // One chunk of CH accumulator columns: bias, activation, pack, 16-byte stores.  CH = 8 for gate/up
            // (two accumulator halves are read per output column, so 8 keeps both register sets small), else 16.
            constexpr int CH = FUSED ? 8 : 16;
            auto finish_chunk = [&](int c0, uint32_t* a, uint32_t* b) {
                if (!tok_ok || n0 + c0 >= p.n_out) return;      // n_out is a multiple of 16: a chunk is all in or all out
                float v[CH];
#pragma unroll
                for (int j = 0; j < CH; ++j) {
                    v[j] = __uint_as_float(a[j]);
                    if (p.row_bias) v[j] += bf16_bits_to_f32(p.row_bias[ebase + n0 + c0 + j]);
                }
                if (FUSED) {
                    float u[CH];
#pragma unroll
                    for (int j = 0; j < CH; ++j) {
                        u[j] = __uint_as_float(b[j]);
                        if (p.row_bias2) u[j] += bf16_bits_to_f32(p.row_bias2[ebase + n0 + c0 + j]);
                    }
                    // one branch per chunk, outside the element loop: with the kind tested per element the
                    // compiler predicates all three bodies and every element pays for all of them
                    if (p.activation == 1) {
#pragma unroll
                        for (int j = 0; j < CH; ++j) v[j] = glu_activation_fast<1>(v[j], u[j], p.limit, p.alpha);
                    } else if (p.activation == 2) {
#pragma unroll
                        for (int j = 0; j < CH; ++j) v[j] = glu_activation_fast<2>(v[j], u[j], p.limit, p.alpha);
                    } else {
#pragma unroll
                        for (int j = 0; j < CH; ++j) v[j] = glu_activation_fast<0>(v[j], u[j], p.limit, p.alpha);
                    }
                }
                if (sizeof(TOut) == 2) {
                    // 8 bf16 per 16-byte store; with the 8-run permutation, run positions hold k = 0,4,1,5,2,6,3,7
                    uint32_t w8[CH / 2];
#pragma unroll
                    for (int h8 = 0; h8 < CH / 8; ++h8)
#pragma unroll
                        for (int pp = 0; pp < 4; ++pp)
                            w8[h8 * 4 + pp] = p.out_permute8 ? pack_bf16x2(v[h8 * 8 + pp], v[h8 * 8 + pp + 4])
                                                             : pack_bf16x2(v[h8 * 8 + 2 * pp], v[h8 * 8 + 2 * pp + 1]);
                    uint4* dst = reinterpret_cast<uint4*>(orow + (size_t)(n0 + c0) * 2);
#pragma unroll
                    for (int i = 0; i < CH / 8; ++i) dst[i] = make_uint4(w8[4 * i], w8[4 * i + 1], w8[4 * i + 2], w8[4 * i + 3]);
                } else {
                    float4* dst = reinterpret_cast<float4*>(orow + (size_t)(n0 + c0) * 4);
#pragma unroll
                    for (int i = 0; i < CH / 4; ++i) dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                }
            };
            // Two register sets: the TMEM loads of the next chunk are in flight while this one is finished.
            // (tcgen05.wait::ld waits for every outstanding load, so the next load is issued right after it.)
            uint32_t a0[CH], b0[CH], a1[CH], b1[CH];
            tmem_ld_n<CH>(t0, a0);
            if (FUSED) tmem_ld_n<CH>(t0 + BN / 2, b0);
            for (int c0 = 0; c0 < ROWS_PER_TILE; c0 += 2 * CH) {
                tmem_ld_wait();
                tmem_ld_n<CH>(t0 + c0 + CH, a1);
                if (FUSED) tmem_ld_n<CH>(t0 + BN / 2 + c0 + CH, b1);
                finish_chunk(c0, a0, b0);
                tmem_ld_wait();
                if (c0 + 2 * CH < ROWS_PER_TILE) {
                    tmem_ld_n<CH>(t0 + c0 + 2 * CH, a0);
                    if (FUSED) tmem_ld_n<CH>(t0 + BN / 2 + c0 + 2 * CH, b0);
                }
                finish_chunk(c0 + CH, a1, b1);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty(buf));
            if (warp == EPI_WARP0 && lane == 0) tl_mark(p, TL_EPI, (int)tcount, 2);
            ++tcount;
        }
    } else if (warp == SCHED_WARP) {
        // ───────────── scheduler: coordinates of the CTA's work items, up to NSCHED items ahead ─────────────
        bool ok = true;
        uint32_t i = 0;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++i) {
            const uint32_t slot = i % NSCHED, phase = (i / NSCHED) & 1u;
            if (!mbar_wait<64>(s_empty(slot), phase ^ 1u, abort_flag)) { ok = false; break; }
            const int g = tile / p.m_tiles;
            const int e = find_group_warp(p.tile_offsets, p.n_experts, g, lane);
            if (lane == 0) {
                const int nt = g - (int)__ldg(p.tile_offsets + e);
                const int row_begin = (int)__ldg(p.offsets + e) + nt * BM;
                const int n_valid = min(BM, (int)__ldg(p.offsets + e + 1) - row_begin);
                asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};"
                             ::"r"(sbase + (uint32_t)L::OFF_SCHED + 16u * slot), "r"(e), "r"(row_begin), "r"(n_valid),
                               "r"(tile - g * p.m_tiles) : "memory");
                mbar_arrive(s_full(slot));   // release: the readers' wait acquires the coordinates
            }
            __syncwarp();
        }
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag && p.error_word) atomicExch(p.error_word, (uint32_t)ERR_WAIT_TIMEOUT);
    if (warp == MMA_WARP) {
        tc_fence_after();
        tmem_dealloc(tmem_base, L::TMEM_COLS);
    }
}

// Token tiles per expert and their prefix sum (one warp, 32 experts per round).
__global__ void tile_schedule_kernel(const uint32_t* __restrict__ offsets, int n_experts, int ntok,
                                     uint32_t* __restrict__ tile_offsets) {
    const int lane = threadIdx.x & 31;
    if (threadIdx.x >= 32) return;
    uint32_t carry = 0;
    for (int e0 = 0; e0 < n_experts; e0 += 32) {
        const int e = e0 + lane;
        const uint32_t t = e < n_experts ? (offsets[e + 1] - offsets[e] + ntok - 1) / ntok : 0u;
        uint32_t incl = t;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t v = __shfl_up_sync(0xFFFFFFFFu, incl, d);
            if (lane >= d) incl += v;
        }
        if (e < n_experts) tile_offsets[e] = carry + incl - t;
        carry += __shfl_sync(0xFFFFFFFFu, incl, 31);
    }
    if (lane == 0) tile_offsets[n_experts] = carry;
}

// Schedule of a single group of n_rows rows (the shared expert): sched = {0, n_rows, 0, n_tiles}.
__global__ void single_group_schedule_kernel(int n_rows, int ntok, uint32_t* __restrict__ sched) {
    if (threadIdx.x == 0) {
        sched[0] = 0;
        sched[1] = (uint32_t)n_rows;
        sched[2] = 0;
        sched[3] = (uint32_t)((n_rows + ntok - 1) / ntok);
    }
}

// Row gather into the expert-contiguous buffer with every 8-run stored in the order
// 0,4,1,5,2,6,3,7 (the order the 4-bit unpack produces).  One warp per row.
__global__ void gather_rows_perm8_kernel(const uint16_t* __restrict__ table, const uint32_t* __restrict__ ids,
                                         int id_div, uint16_t* __restrict__ out, int n_rows, int row_len) {
    const int warps = blockDim.x / 32;
    const int row = blockIdx.x * warps + threadIdx.x / 32;
    if (row >= n_rows) return;
    const int lane = threadIdx.x & 31;
    const uint32_t src = ids ? ids[row] / (uint32_t)id_div : (uint32_t)row;
    const uint4* s = (const uint4*)(table + (size_t)src * row_len);
    uint4* d = (uint4*)(out + (size_t)row * row_len);
    for (int i = lane; i < row_len / 8; i += 32) {
        const uint4 v = s[i];
        uint4 o;
        o.x = __byte_perm(v.x, v.z, 0x5410);
        o.y = __byte_perm(v.x, v.z, 0x7632);
        o.z = __byte_perm(v.y, v.w, 0x5410);
        o.w = __byte_perm(v.y, v.w, 0x7632);
        d[i] = o;
    }
}

}  // namespace g100
}  // namespace ffai
