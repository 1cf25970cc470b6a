// Decode-regime grouped 4-bit dequant products: packed weights stream from HBM through
// per-warp cp.async-staged shared-memory rings (16-byte asynchronous copies, three 128-k
// stages in flight per warp) into registers, one warp per 16 weight rows; warps do not
// synchronise with each other inside the stream.
//
// Replaces, for small batches, the reference's per-expert GEMV chain
// (Ops.dequantGemvInt4ExpertIndexedMany, FFAI Ops.swift:2529-2587; the fused
// moeDownSwigluAccumInt4Chain8, OpsFused.swift:545-697; MoELayer.decodeGPURouter,
// MoELayer.swift:1167-1341) and GPT-OSS's three-sync-per-expert loop
// (GPTOSSText.swift:1399-1445).
//
// A warp owns 16 consecutive output rows of one expert (for gate/up: the 16 gate rows and
// the 16 up rows, so the activation is applied in registers) and walks the reduction axis
// one 64-value group at a time.  Per group a lane reads two packed words per row it
// touches from the staged tile, turns each word into
// four bf16 pairs holding 128+q exactly ((q | 0x4300) is the bf16 128+q), and feeds them to
// mma.sync.m16n8k16 as the A operand; the B operand is the 8 (or 16) activation rows routed
// to this expert, staged alongside.  The tensor core is only the dot-product engine here:
// the kernel is bound by HBM.  After each group the fp32 partial is folded in with the
// group's scale and bias:
//     sum_k (s*q_k + b) x_k = s * sum_k (128+q_k) x_k + (b - 128 s) * sum_k x_k,
// where sum_k x_k per (row of activations, group) is precomputed by the kernel that wrote
// the activations.  fp32 accumulation throughout; weights are never rounded.
//
// K order: the unpack yields the nibble pairs (0,4),(1,5),(2,6),(3,7) of a word, so the
// activation rows are stored with every 8-run in the order 0,4,1,5,2,6,3,7 (done by the
// kernels that write them); the dot product does not see the permutation.
#pragma once
#include "common.cuh"

namespace ffai {
namespace dmma {

struct Params {
    const uint32_t* w1;    // [E, N, K/8]
    const uint16_t* s1;    // [E, N, K/gs]
    const uint16_t* b1;
    const uint16_t* rb1;   // nullable [E, N]
    const uint32_t* w2;    // second projection (fused gate/up)
    const uint16_t* s2;
    const uint16_t* b2;
    const uint16_t* rb2;
    const uint32_t* sb1;   // repacked (scale | bias << 16): [E, N/16, K/64, 16]  (see repack_scale_bias_kernel)
    const uint32_t* sb2;
    int N, K, group_size;  // group_size 64 or 128
    const uint32_t* offsets;  // [E+1] rows per expert in the sorted row space
    const uint32_t* order;    // nullable [E]: expert handled by grid row y (longest first); identity when null
    const uint16_t* x;        // [rows, K] bf16, 8-run permuted
    const uint32_t* row_src;  // nullable: sorted row r reads x (and xsum) at row row_src[r] / row_div instead of r
    int row_div;              //           (the dispatch permutation over per-token rows: no gathered copy is made)
    const float* xsum;        // [rows, xsum_pitch] sum of each 64-run of x; pitch = K/64 rounded up to 4
    int xsum_pitch;
    const float* xsum_parts;  // alternative to xsum (when non-null): [rows, K/16] sums of 16-runs, four per 64-run,
                              // as written by the gate/up kernel; added in ascending order
    float* out_parts;         // FUSED, nullable: [rows, N/16] sum of each warp's 16 rounded outputs per activation row
    void* out;                // FUSED: bf16 [rows, N] 8-run permuted;  else fp32 [rows, N] (bf16 when out_bf16)
    int out_bf16;             // !FUSED or pair: store bf16 in plain column order instead of fp32
    int pair;                 // FUSED instantiation used for ONE projection: a warp owns 32 consecutive rows, the
                              // "second projection" being rows +16 of the first (w2/s2/b2/rb2/sb2 unused); no
                              // activation, both halves stored.  Halves the activation reads per weight byte.
    int activation;
    float limit, alpha;
};

FFAI_DEVINL void mma_bf16_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Row of x / xsum that sorted row r reads.
FFAI_DEVINL size_t src_row(const Params& p, int r) {
    return p.row_src ? (size_t)(__ldg(p.row_src + r) / (uint32_t)p.row_div) : (size_t)r;
}

FFAI_DEVINL int permute8_col(int n) {
    const int k = n & 7;
    return (n & ~7) | (((k & 3) << 1) | (k >> 2));
}

FFAI_DEVINL void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
FFAI_DEVINL void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
FFAI_DEVINL void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// First MMA of a group: accumulator starts from zero (lets the compiler use the zero register).
FFAI_DEVINL void mma_bf16_16816_zero(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.0f));
}

// Per-warp staging geometry.  A stage is 128 k (two 64-runs): per weight row 64 packed bytes, the four
// 16-byte columns of a row XOR-swizzled with bit 1 of the row index (so the 8-byte fragment reads of a
// half warp fall in 32 distinct banks), followed by the packed (scale | bias << 16) words of the
// stage, 16 rows x 2 runs per projection.
constexpr int STG_RUNS = 2;
constexpr int W_PITCH = 64;
#ifndef FFAI_DM_DEPTH_FUSED
#define FFAI_DM_DEPTH_FUSED 3
#endif
#ifndef FFAI_DM_DEPTH_PLAIN
#define FFAI_DM_DEPTH_PLAIN 4
#endif
#ifndef FFAI_DM_MIN_BLOCKS
#define FFAI_DM_MIN_BLOCKS 4
#endif

// Runs of 64-run sums kept in shared memory per pass: whole stages, plus one stage that the look-ahead may touch.
// (With group size 32 the sums are kept per 32-run: twice as many entries.)
__host__ __device__ inline int xs_sm_runs(int n64) { return ((n64 + STG_RUNS - 1) / STG_RUNS + 1) * STG_RUNS; }

// Block-shared activation ring (kernels without a split reduction axis): per stage 16 rows x 256 bytes
// (128 k), rows padded to 272 bytes so the 16-byte fragment reads of a quarter warp hit distinct banks.
constexpr int X_PITCH = 272;
constexpr int X_STAGE = 16 * X_PITCH;

// G32: quantization groups of 32 (two scale words per row and 64-run instead of one).
template <bool FUSED, bool G32 = false>
struct WarpStage {
    static constexpr int NP = FUSED ? 2 : 1;
    static constexpr int SBW = G32 ? 2 : 1;            // scale words per row and 64-run
    static constexpr int DEPTH = FUSED ? FFAI_DM_DEPTH_FUSED : FFAI_DM_DEPTH_PLAIN;   // ring slots per warp; DEPTH-1 stages in flight
    static constexpr int W_BYTES = NP * 16 * W_PITCH;
    static constexpr int SB_BYTES = NP * STG_RUNS * 64 * SBW;
    static constexpr int STAGE = W_BYTES + SB_BYTES;
    static constexpr int PER_WARP = DEPTH * STAGE;
    static constexpr int TOTAL = 4 * PER_WARP;
    static constexpr int X_RING = DEPTH * X_STAGE;
    // dynamic shared memory of a launch: weight rings, [activation ring], 64-run sums
    static int smem_bytes(int n64, int ksplit) { return TOTAL + (ksplit == 1 ? X_RING : 0) + xs_sm_runs(n64) * 64 * SBW; }
};

// (w & mask) | expo with both constants held in registers: with immediates the compiler has to emit two
// logic instructions per pair (one immediate operand per instruction), which doubles the load on the
// half-rate pipe that bounds the kernel.
FFAI_DEVINL uint32_t and_or(uint32_t w, uint32_t mask, uint32_t expo) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(w), "r"(mask), "r"(expo));
    return r;
}
// One packed word -> 4 bf16 pairs (128+n0,128+n4), (128+n1,128+n5), (128+n2,128+n6), (128+n3,128+n7).
FFAI_DEVINL void unpack_word_128r(uint32_t w, uint32_t* o, uint32_t mask, uint32_t expo) {
    o[0] = and_or(w, mask, expo);
    o[1] = and_or(w >> 4, mask, expo);
    o[2] = and_or(w >> 8, mask, expo);
    o[3] = and_or(w >> 12, mask, expo);
}
// 16-byte asynchronous copy that reads `bytes` (16 or 0) from the source and zero-fills the rest.
FFAI_DEVINL void cp_async16_zfill(uint32_t dst, const void* src, uint32_t bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}

// What a warp knows about its slice of the weights; does not change between passes over the activations.
template <bool FUSED>
struct WarpJob {
    const uint8_t* wsrc[WarpStage<FUSED, false>::NP * 2];  // this lane's 16-byte column of the rows it copies, at the slice start
    const uint8_t* sbsrc;                           // this lane's chunk of scale words, at the slice start
    bool sb_lane;                                   // lane copies scale words
    uint32_t wdst;                                  // shared-memory address of this lane's first weight chunk in slot 0
    uint32_t sbdst;                                 // ... of its scale chunk in slot 0
    int n_runs;                                     // 64-runs in the slice
    int G0;                                         // first run of the slice
    bool second_ok;                                 // pair mode: the warp's second 16 rows exist (else they are zero-filled)
    bool sb_second;                                 // this lane's scale chunk belongs to the second projection / half
};

// One 64-run of a stage: scale words, A fragments from the staged packed rows, MMAs against the B
// fragments in xc, fold into tot.
//   group 64/128: a lane's two packed words are k 16t..16t+15 of the run (one 8-byte read); one fold per run
//   group 32:     word 0 is k 8t..8t+7 of the first half, word 1 the same of the second half (two 4-byte
//                 reads), so the two MMAs of a word stay inside one quantization group; one fold per half
// rd: this lane's byte offsets into a weight row of the stage ([Gi] for group 64, [2 Gi + word] for group 32);
// xs: the lane's 64-run sums for this run (16 floats per run; per 32-run with group 32).
template <bool FUSED, int NT, bool G32, int Gi>
FFAI_DEVINL void compute_run(const uint8_t* stage, const uint32_t* rd, const uint4 (*xc)[2], const float* xs,
                             uint32_t mask, uint32_t expo, int g, float (*tot)[WarpStage<FUSED, G32>::NP][4]) {
    using WS = WarpStage<FUSED, G32>;
    constexpr int NP = WS::NP;
    constexpr int SBW = WS::SBW;
    float2 sx[SBW][NT];
#pragma unroll
    for (int hf = 0; hf < SBW; ++hf)
#pragma unroll
        for (int j = 0; j < NT; ++j) sx[hf][j] = *reinterpret_cast<const float2*>(xs + hf * 16 + 8 * j);
#pragma unroll
    for (int q = 0; q < NP; ++q) {
        // scale and (bias - 128*scale) of the two rows this lane's results belong to
        float sc[SBW][2], bm[SBW][2];
#pragma unroll
        for (int hf = 0; hf < SBW; ++hf)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t v = *reinterpret_cast<const uint32_t*>(
                    stage + WS::W_BYTES + q * (STG_RUNS * 64 * SBW) + (Gi * SBW + hf) * 64 + (g + 8 * h) * 4);
                const float s = __uint_as_float(v << 16), b = __uint_as_float(v & 0xFFFF0000u);
                sc[hf][h] = s;
                bm[hf][h] = fmaf(-128.0f, s, b);
            }
        // A fragments: [word 0/1][row lo/hi][pair 0..3]
        uint32_t af[2][2][4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            if (G32) {
                const uint32_t w0 = *reinterpret_cast<const uint32_t*>(stage + (q * 16 + 8 * h) * W_PITCH + rd[2 * Gi]);
                const uint32_t w1 = *reinterpret_cast<const uint32_t*>(stage + (q * 16 + 8 * h) * W_PITCH + rd[2 * Gi + 1]);
                unpack_word_128r(w0, af[0][h], mask, expo);
                unpack_word_128r(w1, af[1][h], mask, expo);
            } else {
                const uint2 wv = *reinterpret_cast<const uint2*>(stage + (q * 16 + 8 * h) * W_PITCH + rd[Gi]);
                unpack_word_128r(wv.x, af[0][h], mask, expo);
                unpack_word_128r(wv.y, af[1][h], mask, expo);
            }
        }
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const uint32_t xb[2][4] = {{xc[j][0].x, xc[j][0].y, xc[j][0].z, xc[j][0].w},
                                       {xc[j][1].x, xc[j][1].y, xc[j][1].z, xc[j][1].w}};
            float c[4];
#pragma unroll
            for (int w = 0; w < 2; ++w) {
#pragma unroll
                for (int hp = 0; hp < 2; ++hp) {
                    // k-slots (2t,2t+1) <- pair 2hp, (2t+8,2t+9) <- pair 2hp+1 of word w
                    const uint32_t a[4] = {af[w][0][2 * hp], af[w][1][2 * hp], af[w][0][2 * hp + 1], af[w][1][2 * hp + 1]};
                    if ((G32 || w == 0) && hp == 0) mma_bf16_16816_zero(c, a, xb[w][2 * hp], xb[w][2 * hp + 1]);
                    else mma_bf16_16816(c, a, xb[w][2 * hp], xb[w][2 * hp + 1]);
                }
                if (G32 || w == 1) {
                    const int hf = G32 ? w : 0;
                    tot[j][q][0] = fmaf(sc[hf][0], c[0], fmaf(bm[hf][0], sx[hf][j].x, tot[j][q][0]));
                    tot[j][q][1] = fmaf(sc[hf][0], c[1], fmaf(bm[hf][0], sx[hf][j].y, tot[j][q][1]));
                    tot[j][q][2] = fmaf(sc[hf][1], c[2], fmaf(bm[hf][1], sx[hf][j].x, tot[j][q][2]));
                    tot[j][q][3] = fmaf(sc[hf][1], c[3], fmaf(bm[hf][1], sx[hf][j].y, tot[j][q][3]));
                }
            }
        }
    }
}

// This lane's byte offsets into a weight row of a stage (see compute_run).
template <bool G32>
FFAI_DEVINL void weight_read_offsets(int g, int t, uint32_t* rd) {
    const uint32_t swz = ((g >> 1) & 1) << 1;                     // 16-byte columns are XOR-swizzled with bit 1 of the row
    if (G32) {
#pragma unroll
        for (int i = 0; i < 4; ++i) rd[i] = g * W_PITCH + (((uint32_t)i ^ swz) << 4) + 4 * t;   // i = 2 Gi + word
    } else {
        const uint32_t rd0 = g * W_PITCH + (t & 1) * 8 + ((((uint32_t)t >> 1) ^ swz) << 4);
        rd[0] = rd0;
        rd[1] = rd0 ^ 32u;
    }
}

// One pass over the weights of a warp's 16-row block for up to 8*NT activation rows.
// All stages have the same shape: the second run of an odd tail (and every stage issued past the
// end) is copied with zero source bytes, so its weights and scale words read as zero and add nothing;
// its activations are read from the last real run (finite values).
template <bool FUSED, int NT, bool G32>
FFAI_DEVINL void decode_pass(const Params& p, const WarpJob<FUSED>& job, uint8_t* wsm, const float* xs_sm,
                             int row0, int cnt, int tok0, int lane, float (*tot)[WarpStage<FUSED, G32>::NP][4]) {
    using WS = WarpStage<FUSED, G32>;
    constexpr int NP = WS::NP;
    constexpr int DEPTH = WS::DEPTH;
    constexpr int SBW = WS::SBW;
    const int g = lane >> 2, t = lane & 3;
    const int K = p.K;
    const int n_runs = job.n_runs;
    const int n_stages = (n_runs + STG_RUNS - 1) / STG_RUNS;
    uint32_t mask, expo;
    asm volatile("mov.u32 %0, 0x000F000F;" : "=r"(mask));
    asm volatile("mov.u32 %0, 0x43004300;" : "=r"(expo));

    // B-operand rows of this lane (column g of each 8-wide tile), clamped to the last valid row; the lane's
    // k range inside a run: 16t.. (one 32-byte piece) or, with group 32, 8t.. of each half (two 16-byte pieces)
    const uint8_t* xrow[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j)
        xrow[j] = reinterpret_cast<const uint8_t*>(p.x + src_row(p, row0 + min(tok0 + 8 * j + g, cnt - 1)) * K + (G32 ? 8 : 16) * t) +
                  (size_t)job.G0 * 128;
    const uint32_t x_last = (uint32_t)(n_runs > 0 ? n_runs - 1 : 0) * 128u;

#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int q = 0; q < NP; ++q)
#pragma unroll
            for (int i = 0; i < 4; ++i) tot[j][q][i] = 0.0f;

    const uint32_t col_run = (uint32_t)(lane & 3) >> 1;          // which run of a stage this lane's weight column belongs to
    const uint32_t sb_run = G32 ? (uint32_t)(lane & 15) >> 3 : (uint32_t)(lane & 7) >> 2;   // ... and its scale chunk
    uint32_t issue_off = 0;                                      // byte offset of the next stage in the source rows
    uint32_t issue_slot = 0;                                     // byte offset of the ring slot it goes to
    int issue_rem = n_runs;                                      // runs not yet issued (may go negative)
    auto issue_stage = [&]() {
        const uint32_t szw = (int)col_run < issue_rem ? 16u : 0u;
#pragma unroll
        for (int i = 0; i < NP * 2; ++i)
            cp_async16_zfill(job.wdst + issue_slot + i * 8 * W_PITCH, job.wsrc[i] + issue_off, (i >= 2 && !job.second_ok) ? 0u : szw);
        if (job.sb_lane)
            cp_async16_zfill(job.sbdst + issue_slot, job.sbsrc + issue_off * (2 * SBW),
                             ((int)sb_run < issue_rem && !(job.sb_second && !job.second_ok)) ? 16u : 0u);
        cp_async_commit();
        issue_off += 64;
        issue_rem -= STG_RUNS;
        issue_slot = issue_slot == (DEPTH - 1) * WS::STAGE ? 0u : issue_slot + WS::STAGE;
    };

    __syncwarp();
#pragma unroll
    for (int st = 0; st < DEPTH - 1; ++st) issue_stage();

    uint4 xbuf[STG_RUNS][NT][2];
    auto fetch_x = [&](uint32_t off, uint4 (*xd)[2]) {
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const uint4* src = reinterpret_cast<const uint4*>(xrow[j] + off);
            xd[j][0] = __ldg(src);
            xd[j][1] = __ldg(src + (G32 ? 4 : 1));
        }
    };
    uint32_t x_off = 0;
    if (n_runs > 0) fetch_x(0, xbuf[0]);   // a warp without a slice must not touch the row at all

    uint32_t use_slot = 0;
    uint32_t rd[4];
    weight_read_offsets<G32>(g, t, rd);
    const float* xs_run = xs_sm + job.G0 * 16 * SBW + 2 * t;     // 16 floats (one per activation row of the pass) per (half) run
    for (int st = 0; st < n_stages; ++st) {
        cp_async_wait<DEPTH - 2>();   // this lane's copies of the stage have landed
        __syncwarp();                 // ... and the other lanes'; the slot of the previous stage is free again
        issue_stage();
        const uint8_t* stage = wsm + use_slot;
        use_slot = use_slot == (DEPTH - 1) * WS::STAGE ? 0u : use_slot + WS::STAGE;
        // run 0 of the stage: its activations are in set 0; start fetching run 1's into set 1, and so on
        x_off = min(x_off + 128u, x_last);
        fetch_x(x_off, xbuf[1]);
        compute_run<FUSED, NT, G32, 0>(stage, rd, xbuf[0], xs_run, mask, expo, g, tot);
        x_off = min(x_off + 128u, x_last);
        fetch_x(x_off, xbuf[0]);
        compute_run<FUSED, NT, G32, 1>(stage, rd, xbuf[1], xs_run + 16 * SBW, mask, expo, g, tot);
        xs_run += STG_RUNS * 16 * SBW;
    }
    cp_async_wait<0>();
}

// The same pass with the activation rows staged once per CTA: the four warps of a CTA work on the same
// expert, the same rows and (no split) the same 128-k stage, so the rows travel from L2 once per CTA
// instead of once per warp.  All threads copy (weights into their warp's ring, activations into the
// shared ring) and meet at one barrier per stage, which both publishes the stage and frees the slot
// of the previous one.  The loop count is the CTA's (n64), so warps without rows still take part.
template <bool FUSED, int NT, bool G32>
FFAI_DEVINL void decode_pass_shared(const Params& p, const WarpJob<FUSED>& job, uint8_t* wsm, uint8_t* xring,
                                    const float* xs_sm, int row0, int cnt, int tok0, int n64, int lane,
                                    float (*tot)[WarpStage<FUSED, G32>::NP][4]) {
    using WS = WarpStage<FUSED, G32>;
    constexpr int NP = WS::NP;
    constexpr int DEPTH = WS::DEPTH;
    constexpr int SBW = WS::SBW;
    const int g = lane >> 2, t = lane & 3;
    const int K = p.K;
    const int n_stages = (n64 + STG_RUNS - 1) / STG_RUNS;
    uint32_t mask, expo;
    asm volatile("mov.u32 %0, 0x000F000F;" : "=r"(mask));
    asm volatile("mov.u32 %0, 0x43004300;" : "=r"(expo));

    // activation chunks this thread copies per stage: chunk c = tid + 128 i -> row c / 16, 16-byte column c % 16
    const uint8_t* xsrc[NT];
    uint32_t xdst[NT];
    const uint32_t xcol_run = (threadIdx.x & 15) >> 3;
    {
        const uint32_t xring_u32 = (uint32_t)__cvta_generic_to_shared(xring);
#pragma unroll
        for (int i = 0; i < NT; ++i) {
            const int c = threadIdx.x + 128 * i, row = c >> 4, col = c & 15;
            xsrc[i] = reinterpret_cast<const uint8_t*>(p.x + src_row(p, row0 + min(tok0 + row, cnt - 1)) * K) + col * 16;
            xdst[i] = xring_u32 + row * X_PITCH + col * 16;
        }
    }

#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int q = 0; q < NP; ++q)
#pragma unroll
            for (int i = 0; i < 4; ++i) tot[j][q][i] = 0.0f;

    const uint32_t col_run = (uint32_t)(lane & 3) >> 1;
    const uint32_t sb_run = G32 ? (uint32_t)(lane & 15) >> 3 : (uint32_t)(lane & 7) >> 2;
    uint32_t issue_off = 0, issue_slot = 0, issue_xslot = 0;
    int issue_rem = job.n_runs;       // this warp's weight runs not yet issued (0 for a warp without rows)
    int issue_rem_x = n64;            // the CTA's activation runs not yet issued
    auto issue_stage = [&]() {
        const uint32_t szw = (int)col_run < issue_rem ? 16u : 0u;
#pragma unroll
        for (int i = 0; i < NP * 2; ++i)
            cp_async16_zfill(job.wdst + issue_slot + i * 8 * W_PITCH, job.wsrc[i] + issue_off, (i >= 2 && !job.second_ok) ? 0u : szw);
        if (job.sb_lane)
            cp_async16_zfill(job.sbdst + issue_slot, job.sbsrc + issue_off * (2 * SBW),
                             ((int)sb_run < issue_rem && !(job.sb_second && !job.second_ok)) ? 16u : 0u);
        const uint32_t szx = (int)xcol_run < issue_rem_x ? 16u : 0u;
#pragma unroll
        for (int i = 0; i < NT; ++i) cp_async16_zfill(xdst[i] + issue_xslot, xsrc[i] + issue_off * 4, szx);
        cp_async_commit();
        issue_off += 64;
        issue_rem -= STG_RUNS;
        issue_rem_x -= STG_RUNS;
        issue_slot = issue_slot == (DEPTH - 1) * WS::STAGE ? 0u : issue_slot + WS::STAGE;
        issue_xslot = issue_xslot == (DEPTH - 1) * X_STAGE ? 0u : issue_xslot + X_STAGE;
    };

#pragma unroll
    for (int st = 0; st < DEPTH - 1; ++st) issue_stage();

    uint32_t use_slot = 0, use_xslot = 0;
    uint32_t rd[4];
    weight_read_offsets<G32>(g, t, rd);
    const uint32_t xrd = g * X_PITCH + t * (G32 ? 16 : 32);   // the lane's k range inside a run (see decode_pass)
    constexpr int X2 = G32 ? 64 : 16;                         // byte distance of its second 16-byte piece
    const float* xs_run = xs_sm + 2 * t;
    for (int st = 0; st < n_stages; ++st) {
        cp_async_wait<DEPTH - 2>();   // this thread's copies of the stage have landed
        __syncthreads();              // ... and everybody's; the slots of the previous stage are free again
        issue_stage();
        const uint8_t* stage = wsm + use_slot;
        const uint8_t* xstage = xring + use_xslot + xrd;
        use_slot = use_slot == (DEPTH - 1) * WS::STAGE ? 0u : use_slot + WS::STAGE;
        use_xslot = use_xslot == (DEPTH - 1) * X_STAGE ? 0u : use_xslot + X_STAGE;
        uint4 xc[NT][2];
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            xc[j][0] = *reinterpret_cast<const uint4*>(xstage + j * 8 * X_PITCH);
            xc[j][1] = *reinterpret_cast<const uint4*>(xstage + j * 8 * X_PITCH + X2);
        }
        compute_run<FUSED, NT, G32, 0>(stage, rd, xc, xs_run, mask, expo, g, tot);
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            xc[j][0] = *reinterpret_cast<const uint4*>(xstage + j * 8 * X_PITCH + 128);
            xc[j][1] = *reinterpret_cast<const uint4*>(xstage + j * 8 * X_PITCH + 128 + X2);
        }
        compute_run<FUSED, NT, G32, 1>(stage, rd, xc, xs_run + 16 * SBW, mask, expo, g, tot);
        xs_run += STG_RUNS * 16 * SBW;
    }
    cp_async_wait<0>();
}

// grid: (ceil(N / 16 / (4 / KSPLIT)), E); block: 128 threads = 4 warps.
// Warp w works on 16-row block (w / KSPLIT) of the CTA and on the (w % KSPLIT)-th slice of the
// reduction axis; with KSPLIT > 1 the slices are summed in a fixed order through shared memory at
// the end (tiny batches: more warps in flight per active expert).  Every warp streams its own packed
// rows and scale words through its own cp.async ring (16-byte asynchronous copies, DEPTH stages of
// 128 k in flight) and synchronises with nobody inside the stream.
// NT: most activation rows handled per pass over the weights, in units of 8; a pass with 8 rows or
// fewer left runs the one-tile body whatever NT is.
// Shared memory: the rings, then 16 floats per 64-run (rounded up to whole stages, plus one stage)
// holding the 64-run sums of the pass's activation rows, transposed so a lane reads its two rows at once.
template <bool FUSED, int NT, int KSPLIT, bool G32>
__global__ void __launch_bounds__(128, FFAI_DM_MIN_BLOCKS)
grouped_mma_decode_kernel(const Params p) {
    using WS = WarpStage<FUSED, G32>;
    constexpr int NP = WS::NP;
    constexpr int SBW = WS::SBW;
    constexpr int RBW = 4 / KSPLIT;  // 16-row blocks per CTA
    extern __shared__ __align__(16) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    pdl_wait();                 // the routing tables and the activation rows come from the kernels before this one
    pdl_launch_dependents();
    const int e = p.order ? (int)p.order[blockIdx.y] : (int)blockIdx.y;
    const int row0 = (int)p.offsets[e], cnt = (int)p.offsets[e + 1] - row0;
    if (cnt <= 0) return;
    const int K = p.K, wpr = K / 8, n64 = K / 64;
    const bool pair = FUSED && p.pair;                 // one projection, 32 rows per warp (see Params::pair)
    const int rb = blockIdx.x * RBW + warp / KSPLIT;   // 16-row (pair: 32-row) block within the expert
    const int ks = warp % KSPLIT;
    const int rb_row = rb * (pair ? 32 : 16);
    const bool warp_active = rb_row < p.N;             // N is a multiple of 16
    const int per = (n64 + KSPLIT - 1) / KSPLIT;
    const int G0 = min(ks * per, n64), G1 = min(G0 + per, n64);

    uint8_t* wsm = smem + warp * WS::PER_WARP;
    uint8_t* xring = smem + WS::TOTAL;   // present only without a split reduction axis
    float* xs_sm = reinterpret_cast<float*>(smem + WS::TOTAL + (KSPLIT == 1 ? WS::X_RING : 0));
    const int xs_runs = xs_sm_runs(n64) * SBW;   // entries of the sums table: per 64-run, or per 32-run with group 32

    WarpJob<FUSED> job;
    job.n_runs = warp_active ? G1 - G0 : 0;
    job.G0 = G0;
    job.second_ok = !pair || rb_row + 16 < p.N;
    {
        const int col = lane & 3;
#pragma unroll
        for (int i = 0; i < NP * 2; ++i) {
            const int ridx = (lane >> 2) + 8 * i;  // 0 .. NP*16-1
            const uint32_t* base = (ridx >= 16 && !pair) ? p.w2 : p.w1;
            const int half_rows = (ridx >= 16 && pair && job.second_ok) ? 16 : 0;   // second half of a pair: the next 16 rows
            const size_t row = (size_t)e * p.N + (warp_active ? rb_row : 0) + half_rows + (ridx & 15);
            job.wsrc[i] = reinterpret_cast<const uint8_t*>(base + row * wpr) + G0 * 32 + col * 16;
        }
        // scale words of a stage: per projection 8 (16 with group 32) 16-byte chunks; lane -> (projection, chunk)
        constexpr int SB_CHUNKS = 8 * SBW;
        const int sb_q = lane / SB_CHUNKS;  // projection whose scale words this lane copies (valid when < NP)
        const int sb_c = lane % SB_CHUNKS;
        job.sb_lane = sb_q < NP;
        job.sb_second = sb_q == 1;
        // 16-row block whose scale words this lane copies: in pair mode the warp's two halves are blocks 2 rb, 2 rb + 1
        const int sb_blk = !warp_active ? 0 : (pair ? 2 * rb + ((sb_q == 1 && job.second_ok) ? 1 : 0) : rb);
        job.sbsrc = reinterpret_cast<const uint8_t*>(
            ((sb_q == 1 && FUSED && !pair) ? p.sb2 : p.sb1) + (((size_t)e * (p.N / 16) + sb_blk) * (n64 * SBW) + G0 * SBW) * 16) + sb_c * 16;
        const uint32_t wsm_u32 = (uint32_t)__cvta_generic_to_shared(wsm);
        job.wdst = wsm_u32 + (lane >> 2) * W_PITCH + ((col ^ (((lane >> 3) & 1) << 1)) << 4);
        job.sbdst = wsm_u32 + WS::W_BYTES + (sb_q & (NP - 1)) * (STG_RUNS * 64 * SBW) + sb_c * 16;
    }

    for (int tok0 = 0; tok0 < cnt; tok0 += 8 * NT) {
        // 64-run sums of the pass's activation rows -> shared memory, [run][row]; rows past the end and
        // the padding runs read as zero
        __syncthreads();   // the previous pass (or the reduction below) is done with shared memory
        // p.xsum holds sums of 32-runs (two per 64-run); p.xsum_parts sums of 16-runs (four per 64-run)
        for (int i = threadIdx.x; i < xs_runs * 16; i += 128) {
            const int r = i / xs_runs, R = i - r * xs_runs;   // R: 64-run index, or 32-run index with group 32
            float v = 0.0f;
            if (tok0 + r < cnt && R < n64 * SBW) {
                if (p.xsum_parts) {
                    const float* q = p.xsum_parts + (size_t)(row0 + tok0 + r) * (K / 16);
                    if (G32) {
                        const float2 q2 = __ldg(reinterpret_cast<const float2*>(q) + R);
                        v = q2.x + q2.y;
                    } else {
                        const float4 q4 = __ldg(reinterpret_cast<const float4*>(q) + R);
                        v = (q4.x + q4.y) + (q4.z + q4.w);
                    }
                } else {
                    const float* q = p.xsum + src_row(p, row0 + tok0 + r) * p.xsum_pitch;
                    if (G32) {
                        v = __ldg(q + R);
                    } else {
                        const float2 q2 = __ldg(reinterpret_cast<const float2*>(q) + R);
                        v = q2.x + q2.y;
                    }
                }
            }
            xs_sm[R * 16 + r] = v;
        }
        __syncthreads();

        float tot[NT][NP][4];
        if (NT == 1 || cnt - tok0 <= 8) {
            if (KSPLIT == 1) decode_pass_shared<FUSED, 1, G32>(p, job, wsm, xring, xs_sm, row0, cnt, tok0, n64, lane, tot);
            else decode_pass<FUSED, 1, G32>(p, job, wsm, xs_sm, row0, cnt, tok0, lane, tot);
#pragma unroll
            for (int j = 1; j < NT; ++j)
#pragma unroll
                for (int q = 0; q < NP; ++q)
#pragma unroll
                    for (int i = 0; i < 4; ++i) tot[j][q][i] = 0.0f;
        } else {
            if (KSPLIT == 1) decode_pass_shared<FUSED, NT, G32>(p, job, wsm, xring, xs_sm, row0, cnt, tok0, n64, lane, tot);
            else decode_pass<FUSED, NT, G32>(p, job, wsm, xs_sm, row0, cnt, tok0, lane, tot);
        }

        if (KSPLIT > 1) {
            // fixed-order sum of the reduction slices: slices 1.. park their partials, slice 0 adds them in order
            __syncthreads();  // every warp is out of its ring: reuse the start of shared memory
            float* red = reinterpret_cast<float*>(smem);
            constexpr int PER_WARP_VALS = NT * NP * 4 * 32;
            if (ks > 0) {
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int q = 0; q < NP; ++q)
#pragma unroll
                        for (int i = 0; i < 4; ++i) red[warp * PER_WARP_VALS + ((j * NP + q) * 4 + i) * 32 + lane] = tot[j][q][i];
            }
            __syncthreads();
            if (ks == 0) {
                for (int o = 1; o < KSPLIT; ++o)
#pragma unroll
                    for (int j = 0; j < NT; ++j)
#pragma unroll
                        for (int q = 0; q < NP; ++q)
#pragma unroll
                            for (int i = 0; i < 4; ++i) tot[j][q][i] += red[(warp + o) * PER_WARP_VALS + ((j * NP + q) * 4 + i) * 32 + lane];
            }
        }

        // results: value i -> (row g + 8*(i>>1), activation row tok0 + 8j + 2t + (i&1))
        if (FUSED && pair) {
            if (warp_active && ks == 0) {
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int q = 0; q < NP; ++q)
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int tok = tok0 + 8 * j + 2 * t + (i & 1);
                            if (tok >= cnt || (q == 1 && !job.second_ok)) continue;
                            const int n = rb_row + 16 * q + g + 8 * (i >> 1);
                            float v = tot[j][q][i];
                            if (p.rb1) v += bf16_bits_to_f32(p.rb1[(size_t)e * p.N + n]);
                            if (p.out_bf16) reinterpret_cast<uint16_t*>(p.out)[(size_t)(row0 + tok) * p.N + n] = f32_to_bf16_bits(v);
                            else reinterpret_cast<float*>(p.out)[(size_t)(row0 + tok) * p.N + n] = v;
                        }
            }
        } else
        if (warp_active && ks == 0) {
            float rsum[NT][2];   // FUSED: this lane's two rows' share of sum over the warp's 16 outputs, per activation row
#pragma unroll
            for (int j = 0; j < NT; ++j) rsum[j][0] = rsum[j][1] = 0.0f;
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int tok = tok0 + 8 * j + 2 * t + (i & 1);
                    if (tok >= cnt) continue;
                    const int n = rb_row + g + 8 * (i >> 1);
                    const size_t rr = (size_t)e * p.N + n;
                    float v = tot[j][0][i];
                    if (p.rb1) v += bf16_bits_to_f32(p.rb1[rr]);
                    if (FUSED) {
                        float u = tot[j][NP - 1][i];
                        if (p.rb2) u += bf16_bits_to_f32(p.rb2[rr]);
                        v = glu_activation(v, u, p.activation, p.limit, p.alpha);
                        const uint16_t vb = f32_to_bf16_bits(v);
                        reinterpret_cast<uint16_t*>(p.out)[(size_t)(row0 + tok) * p.N + permute8_col(n)] = vb;
                        rsum[j][i & 1] += bf16_bits_to_f32(vb);
                    } else if (p.out_bf16) {
                        reinterpret_cast<uint16_t*>(p.out)[(size_t)(row0 + tok) * p.N + n] = f32_to_bf16_bits(v);
                    } else {
                        reinterpret_cast<float*>(p.out)[(size_t)(row0 + tok) * p.N + n] = v;
                    }
                }
            if (FUSED && p.out_parts) {
                // sum over the warp's 16 output rows (the lanes that share t), fixed butterfly; lanes g == 0 write
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        float v = rsum[j][h];
                        v += __shfl_xor_sync(0xFFFFFFFFu, v, 4);
                        v += __shfl_xor_sync(0xFFFFFFFFu, v, 8);
                        v += __shfl_xor_sync(0xFFFFFFFFu, v, 16);
                        const int tok = tok0 + 8 * j + 2 * t + h;
                        if (g == 0 && tok < cnt) p.out_parts[(size_t)(row0 + tok) * (p.N / 16) + rb] = v;
                    }
            }
        }
    }
}

// Scale and bias of a stacked projection repacked for the streaming kernels:
//   out[((e * N/16 + rb) * K/run + G) * 16 + r] = scale | bias << 16   of row rb*16 + r, run G
// (run = 64 for group sizes 64 and 128, 32 for group size 32)
// so that the 16 rows of a block are contiguous per run and a warp's stage is one 128-byte copy.
__global__ void repack_scale_bias_kernel(const uint16_t* __restrict__ scales, const uint16_t* __restrict__ biases,
                                         uint32_t* __restrict__ out, int n_experts, int N, int K, int group_size, int run) {
    const size_t total = (size_t)n_experts * N * (K / run);
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int r = (int)(i & 15);
    const size_t rest = i >> 4;
    const int nr = K / run;
    const int G = (int)(rest % nr);
    const size_t blk = rest / nr;  // e * N/16 + rb
    const size_t row = blk * 16 + r;  // e * N + rb*16 + r
    const int gpr = K / group_size;
    const size_t src = row * gpr + (size_t)(G * run / group_size);
    out[i] = (uint32_t)scales[src] | ((uint32_t)biases[src] << 16);
}

// Gather rows into expert-sorted order with the 8-run permutation, and write the sum of every
// 32-run (fp32; a 64-run's sum is the sum of its two halves).  One warp per output row.  ids nullable (identity), id_div as in Ops.gather use.
__global__ void gather_perm8_sum64_kernel(const uint16_t* __restrict__ table, const uint32_t* __restrict__ ids,
                                          int id_div, uint16_t* __restrict__ out, float* __restrict__ sums,
                                          int n_rows, int row_len, int sum_pitch) {
    const int warps = blockDim.x / 32;
    const int row = blockIdx.x * warps + threadIdx.x / 32;
    if (row >= n_rows) return;
    const int lane = threadIdx.x & 31;
    const uint32_t src = ids ? ids[row] / (uint32_t)id_div : (uint32_t)row;
    const uint4* s = (const uint4*)(table + (size_t)src * row_len);
    uint4* d = (uint4*)(out + (size_t)row * row_len);
    const int chunks = row_len / 8;  // 16-byte chunks; 8 chunks per 64-run
    for (int i0 = 0; i0 < chunks; i0 += 32) {
        const int i = i0 + lane;
        float part = 0.0f;
        if (i < chunks) {
            const uint4 v = s[i];
            uint4 o;
            o.x = __byte_perm(v.x, v.z, 0x5410);
            o.y = __byte_perm(v.x, v.z, 0x7632);
            o.z = __byte_perm(v.y, v.w, 0x5410);
            o.w = __byte_perm(v.y, v.w, 0x7632);
            d[i] = o;
            part = ((bf16lo(v.x) + bf16hi(v.x)) + (bf16lo(v.y) + bf16hi(v.y))) +
                   ((bf16lo(v.z) + bf16hi(v.z)) + (bf16lo(v.w) + bf16hi(v.w)));
        }
        // 4 consecutive lanes hold one 32-run: fixed-shape tree over them
        part += __shfl_xor_sync(0xFFFFFFFFu, part, 1);
        part += __shfl_xor_sync(0xFFFFFFFFu, part, 2);
        if ((lane & 3) == 0 && i < chunks) sums[(size_t)row * sum_pitch + (i >> 2)] = part;
    }
}

// Sum of every 64-run of rows that are already stored 8-run permuted (the sum does not depend
// on the order inside a run).  One warp per row.
__global__ void sum64_rows_kernel(const uint16_t* __restrict__ rows, float* __restrict__ sums, int n_rows,
                                  int row_len, int sum_pitch) {
    const int warps = blockDim.x / 32;
    const int row = blockIdx.x * warps + threadIdx.x / 32;
    if (row >= n_rows) return;
    const int lane = threadIdx.x & 31;
    const uint4* s = (const uint4*)(rows + (size_t)row * row_len);
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

}  // namespace dmma
}  // namespace ffai
