// Fused neighbourhood-attention backward on tcgen05 tensor cores (sm_100a).
//
// Two launches of one kernel template, neither materialises P or dS in memory:
//   * query side: rows = a box of 128 queries, columns = chunks of the key box.
//     S = Q K^T, dP = dO V^T (tensor cores, TMEM); threads turn them into
//     dS = P (dP - delta) * scale with P = exp2(S*scale*log2e - lse*log2e); dQ += dS K.
//   * key side: rows = a box of 128 keys, columns = chunks of the box of queries that
//     attend to them (the inverse neighbourhood, a contiguous range per axis), for
//     every query head of the GQA group.  S^T = K Q^T, dP^T = V dO^T;
//     dV += P^T dO, dK += dS^T Q.  Per-column lse / delta are staged in shared memory
//     by a helper warp.
// The row accumulators live in TMEM for the whole tile, so dK/dV are reduced in a
// fixed order: results are bit-reproducible, no atomics.
//
// Chunks are 64 columns wide so that, up to head dim 64, a CTA needs only 256 TMEM columns and 102 KB of
// shared memory: two CTAs share an SM and one computes while the other waits for its MMAs or loads.  At head
// dim 128 one CTA owns the SM's 512 columns; the 128 spare ones hold a second S / dP buffer, so that the
// products of chunk g + 1 run while the threads work on chunk g.  The grid is persistent (CTAs walk the
// tiles), so barriers, TMEM and the column-stage ring are set up once and the next tile's loads run ahead.
// Warps: 8 compute warps (two per TMEM lane quadrant, each owns half of the chunk's columns), two MMA-issuing
// warps (independent streams: dP / acc1 and S / acc2), one helper warp (per-axis tables one tile ahead, the
// TMA loads, column statistics on the key side).
// TMEM: S [0,64)  dP [64,128)  acc1 [128,128+D)  acc2 [128+D,128+2D); head dim 128: second S [384,448) and
// dP [448,512).  The 16-bit P and dS that feed the accumulating MMAs overwrite the first half of the S / dP
// columns of the piece they were computed from (same warp, after it has read them).
#include "tc_kernels.cuh"

#include "simt_kernels.cuh"
#include "tc_plan.cuh"
#include "tc_rowtile.cuh"

#include <type_traits>

#ifndef NATTEN_ABL
#define NATTEN_ABL 0
#endif

namespace natten {

using namespace tc;
using namespace tcplan;
using namespace rowtile;

// Optional clock stamps of one CTA's pipeline events (development builds only: -DNATTEN_TRACE).
#ifdef NATTEN_TRACE
__device__ long long g_trace_bwd[2 * 16 * 512];
#define STAMP(id)                                                                                   \
    do {                                                                                            \
        if (blockIdx.x == 7 && lane == 0 && tn < 255) {                                             \
            long long* tr_ = g_trace_bwd + (kKeySide ? 16 * 512 : 0) + warp * 512;                  \
            tr_[2 * tn] = (id);                                                                     \
            tr_[2 * tn + 1] = clock64();                                                            \
            ++tn;                                                                                   \
        }                                                                                           \
    } while (0)
#else
#define STAMP(id) do { } while (0)
#endif

namespace {

constexpr int kStages = 3;
constexpr int kComputeWarps = 8;
constexpr int kThreads = (kComputeWarps + 3) * 32;    // + MMA issue, helper (tables, statistics), loader
constexpr uint32_t kColS = 0, kColDP = 64, kColA1 = 128;   // acc2 follows acc1 (64 or 128 columns each)
constexpr int kRowHalf = kTileRows * 128;   // bytes of one [128 x 64] 16-bit block of a row tile
constexpr int kColHalf = kCols * 128;       // bytes of one [64 x 64] 16-bit block of a column tile

template <int DH>
struct SmemB {
    static constexpr int kHalves = DH / 64;
    static constexpr int kTile = kRowHalf * kHalves;             // row tile  [128 x DH]
    static constexpr int kColTile = kColHalf * kHalves;          // column tile [64 x DH]
    static constexpr int kR1 = 0;
    static constexpr int kR2 = kR1 + kTile;
    static constexpr int kC1 = kR2 + kTile;                     // [kStages]
    static constexpr int kC2 = kC1 + kStages * kColTile;        // [kStages]
    static constexpr int kStats = kC2 + kStages * kColTile;     // [kStages][2][64] float
    static constexpr int kTab = kStats + kStages * 512;         // [2] tables: axis entries, then a TileHead
    static constexpr int kTabBytes = kAxisEntries * 16 + 96;
    static constexpr int kBar = kTab + 2 * kTabBytes;
    static constexpr int kStage = (kBar + 256 + 1023) & ~1023;   // output staging: a row tile [128 x DH] 16-bit, swizzled like the loads
    static constexpr int kTotal = kStage + kTile;
    static constexpr uint32_t kTmemCols = DH == 64 ? 256 : 512;
    static constexpr uint32_t kColA2 = kColA1 + DH;
};

// Persistent kernel: every CTA walks the work items blockIdx.x, blockIdx.x + gridDim.x, ...;
// barriers, TMEM and the column-stage ring live for the whole launch, so the next tile's
// rows and first column chunks are already on their way while this tile's accumulators are
// written out.  Barrier phases run on across tiles (g = chunks processed so far).
// kInner: innermost chunk extent when it is 16 or 32 (separable row / column masks, packed
// 16-bit arithmetic), 0 = any geometry (per-column validity words).
template <int DH, bool BF16, bool kKeySide, int kInner>
__global__ void __launch_bounds__(kThreads, (DH == 64 ? 2 : 1))
tc_bwd_kernel(const __grid_constant__ CUtensorMap tmR1, const __grid_constant__ CUtensorMap tmR2,
              const __grid_constant__ CUtensorMap tmC1, const __grid_constant__ CUtensorMap tmC2,
              const __grid_constant__ CUtensorMap tmE1, const __grid_constant__ CUtensorMap tmE2,
              const __grid_constant__ CUtensorMap tmO1, const __grid_constant__ CUtensorMap tmO2,
              const __grid_constant__ TcParams P, const float* __restrict__ lse,
              const float* __restrict__ delta, uint16_t* __restrict__ out1, uint16_t* __restrict__ out2)
{
    using Smem = SmemB<DH>;
    constexpr int kTile = Smem::kTile, kColTile = Smem::kColTile, CH = DH / 2;
    constexpr uint32_t kTmemCols = Smem::kTmemCols, kColA2 = Smem::kColA2;
    extern __shared__ __align__(1024) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef NATTEN_TRACE
    int tn = 0;
#endif
    const int quad = warp & 3, piece = (warp >> 2) & 1;      // compute warps: TMEM lane quadrant, 32-column piece
    const int prior_abort = *reinterpret_cast<volatile int*>(P.status);   // loaded early, used at barrier set-up
    const unsigned nwork = kKeySide ? P.work_kv : P.work_q;

    // ---- shared memory, barriers, TMEM --------------------------------------
    const uint32_t sbase = smem_u32(smem);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Smem::kBar + 192);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Smem::kBar + 200);
    const uint32_t bar_row = sbase + Smem::kBar + 0;          // row tiles landed
    const uint32_t bar_col = sbase + Smem::kBar + 8;          // [kStages] C1, C2 landed
    const uint32_t bar_stats = sbase + Smem::kBar + 40;       // [kStages] column lse / delta staged
    const uint32_t bar_s = sbase + Smem::kBar + 72;           // S and dP of the chunk are in TMEM
    const uint32_t bar_sp = sbase + Smem::kBar + 80;          // threads consumed S/dP, wrote P/dS
    const uint32_t bar_free = sbase + Smem::kBar + 96;        // [kStages] accumulating MMAs of the stage's chunk finished
    const uint32_t bar_tab_full = sbase + Smem::kBar + 128;   // [2] row table written
    const uint32_t bar_tab_empty = sbase + Smem::kBar + 144;  // [2] row table read by every compute thread and the MMA warp
    const uint32_t bar_rowfree = sbase + Smem::kBar + 176;    // every S / dP product of the tile finished: the row tiles are free
    // At head dim 128 one CTA owns all 512 TMEM columns and 128 of them are spare: S and dP get a second buffer
    // ([384,448) and [448,512), used by the odd chunks), so the products of chunk g + 1 run while the threads work
    // on chunk g.  Each buffer has its own bar_s / bar_sp, completed once per two chunks.
    constexpr bool kTwoBuf = DH == 128;
    const uint32_t bar_s1 = sbase + Smem::kBar + 160, bar_sp1 = sbase + Smem::kBar + 168;
    auto buf_cols = [&](unsigned g) -> uint32_t { return (kTwoBuf && (g & 1u)) ? 384u : 0u; };
    auto bar_s_of = [&](unsigned g) -> uint32_t { return (kTwoBuf && (g & 1u)) ? bar_s1 : bar_s; };
    auto bar_sp_of = [&](unsigned g) -> uint32_t { return (kTwoBuf && (g & 1u)) ? bar_sp1 : bar_sp; };
    auto par_of = [&](unsigned g) -> uint32_t { return kTwoBuf ? ((g >> 1) & 1u) : (g & 1u); };
    float* stats = reinterpret_cast<float*>(smem + Smem::kStats);

    if (warp == kComputeWarps) {
        if (lane == 0) {
            *abort_flag = ((sbase & 1023u) || prior_abort) ? 1 : 0;
            mbar_init(bar_row, 1);
            for (int s = 0; s < kStages; ++s) {
                mbar_init(bar_col + 8 * s, 1);
                mbar_init(bar_stats + 8 * s, 32);
                mbar_init(bar_free + 8 * s, kKeySide ? 2 : 1);      // one commit per MMA stream that accumulates
            }
            mbar_init(bar_s, 2);                 // one commit per MMA stream
            mbar_init(bar_sp, kComputeWarps * 32);
            mbar_init(bar_s1, 2);
            mbar_init(bar_sp1, kComputeWarps * 32);
            for (int i = 0; i < 2; ++i) { mbar_init(bar_tab_full + 8 * i, 32); mbar_init(bar_tab_empty + 8 * i, kComputeWarps * 32 + 2); }
            mbar_init(bar_rowfree, 2);
            mbar_init_fence();
            fence_async_smem();
        }
        __syncwarp();
        tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    // next work item of this CTA with anything to do for the tensor cores
    auto next_active = [&](unsigned w, BwdTile& X) {
        for (; w < nwork; w += gridDim.x) {
            bwd_tile_setup<kKeySide>(P, w, X);
            if (X.active) break;
        }
        return w;
    };

    if (warp == kComputeWarps || warp == kComputeWarps + 2) {
        // =====================================================================
        // MMA issue: one thread in each of two warps.  A single thread gets a tcgen05.mma out every ~65
        // cycles whatever its N, so the chunk's products are split into two independent streams:
        //   first  (warp 8):  acc1 += dS x C1   then   dP(next) = R2 x C2^T     (both touch the dP columns)
        //   second (warp 10): acc2 += P x C2    then   S(next)  = R1 x C1^T     (both touch the S columns; acc2 on
        //                                                                        the key side only)
        // Each stream is ordered by its own issue order; the streams share no TMEM columns.  Every barrier that
        // tracks the products takes one commit from each stream.
        // =====================================================================
        // The whole warp runs the loop (warp-uniform code); the tensor-core instructions execute on one elected lane.
        const uint32_t leader = elect_one();
        if (!*abort_flag) {
            const bool second = warp != kComputeWarps;
            constexpr uint32_t idesc_kk = instr_desc(BF16 ? 1 : 0, kCols, 0, 0);    // both operands K-major
            constexpr uint32_t idesc_acc = instr_desc(BF16 ? 1 : 0, DH, 0, 1);      // A from TMEM, B MN-major
            const uint64_t dR = smem_desc(sbase + (second ? Smem::kR1 : Smem::kR2), 16, 1024);
            const uint32_t col_tiles = second ? Smem::kC1 : Smem::kC2;             // column tiles of this stream's S / dP
            const uint32_t acc_tiles = second ? Smem::kC2 : Smem::kC1;             // ... and of its accumulating product
            const uint32_t col_out = second ? kColS : kColDP;                      // TMEM columns of S | dP (and of P | dS)
            const bool has_acc = !second || kKeySide;
            auto issue_s_dp = [&](unsigned g, int cc, const TileHead& X) {
                const int s = g % kStages;
                if (P.extents && cc < X.nbox) {      // rows of the column tile past the sample's extent -> zeros
                    int r = cc % X.nchunks;
                    const int c2 = r % X.nc[2]; r /= X.nc[2];
                    const int c1 = r % X.nc[1], c0 = r / X.nc[1];
                    const int box0[3] = {X.boxlo[0] + chunk_coord(P, 0, c0, 0), X.boxlo[1] + chunk_coord(P, 1, c1, 0),
                                         X.boxlo[2] + chunk_coord(P, 2, c2, 0)};
                    uint8_t* tile = smem + col_tiles + s * kColTile;     // the other stream zeroes the other tile
                    if (leader) zero_rows_past_extent(P, box0, X.Lp, kCols, Smem::kHalves, kColHalf, tile, tile);
                    __syncwarp();
                }
                const uint64_t dC = smem_desc(sbase + col_tiles + s * kColTile, 16, 1024);
                tc_fence_after();
                // 32 bytes per k-step inside a 64-channel block; blocks are kRowHalf / kColHalf apart
#pragma unroll
                for (int ks = 0; ks < DH / 16; ++ks)
                    mma_ss_e(tmem + col_out + buf_cols(g), dR + (((ks / 4) * kRowHalf + (ks % 4) * 32) >> 4),
                             dC + (((ks / 4) * kColHalf + (ks % 4) * 32) >> 4), idesc_kk, ks > 0, leader);
                mma_commit_e(bar_s_of(g), leader);
                if (cc + 1 == X.total) mma_commit_e(bar_rowfree, leader);      // the tile's last read of this stream's row tile
            };
            // k-step ks covers columns 16*ks..16*ks+15 of the chunk; their 16-bit pairs sit in the first 8 of
            // those columns (16-column inner rows) or in the first 16 TMEM columns of the 32-column piece
            // they came from.  The column tile is read MN-major: 16 rows (2048 bytes) per k-step, the second
            // 64-channel block kColHalf further.
            auto pair_col = [](int ks) { return kInner == 16 ? 16 * ks : 32 * (ks / 2) + 8 * (ks % 2); };
            auto issue_acc = [&](unsigned g, bool accumulate) {
                const int s = g % kStages;
                if (has_acc) {
                    const uint64_t dC = smem_desc(sbase + acc_tiles + s * kColTile, kColHalf, 1024);
                    tc_fence_after();
#pragma unroll
                    for (int ks = 0; ks < kCols / 16; ++ks)
                        mma_ts_e(tmem + (second ? kColA2 : kColA1), tmem + col_out + buf_cols(g) + pair_col(ks), dC + 128 * ks, idesc_acc,
                                 (accumulate || ks > 0) ? 1u : 0u, leader);
                }
                if (has_acc) mma_commit_e(bar_free + 8 * s, leader);     // the stage's column tiles (and statistics) may be replaced
            };

            unsigned g = 0, tileno = 0, item = 0;
            bool ok = true;
            for (unsigned work = blockIdx.x; work < nwork && ok; work += gridDim.x, ++item) {
                const unsigned slot = item & 1;
                ok = mbar_wait(bar_tab_full + 8 * slot, (item >> 1) & 1, abort_flag, P.wait_budget);
                if (!ok) break;
                const TileHead T = *reinterpret_cast<const TileHead*>(smem + Smem::kTab + slot * Smem::kTabBytes + kAxisEntries * 16);
                __syncwarp();                    // every lane has read the head
                if (leader) mbar_arrive(bar_tab_empty + 8 * slot);
                if (!T.active) continue;
                STAMP(190);
                ok = mbar_wait(bar_row, tileno & 1, abort_flag, P.wait_budget);
                STAMP(191);
                ok = ok && mbar_wait(bar_col + 8 * (g % kStages), (g / kStages) & 1, abort_flag, P.wait_budget);
                if (!ok) break;
                STAMP(192);
                issue_s_dp(g, 0, T);
                for (int cc = 0; cc < T.total && ok; ++cc, ++g) {
                    STAMP(200 + cc);
                    if (kTwoBuf && cc + 1 < T.total) {
                        // two buffers: the next chunk's products go into the other buffer, whose P / dS were read
                        // by products this warp issued earlier, so they need not wait for the threads
                        ok = mbar_wait(bar_col + 8 * ((g + 1) % kStages), ((g + 1) / kStages) & 1, abort_flag, P.wait_budget);
                        if (!ok) break;
                        issue_s_dp(g + 1, cc + 1, T);
                    }
                    ok = mbar_wait(bar_sp_of(g), par_of(g), abort_flag, P.wait_budget);               // S/dP consumed, P/dS stored
                    if (!ok) break;
                    STAMP(210);
                    issue_acc(g, cc > 0);                                    // reads P/dS ...
                    STAMP(215);
                    if (!kTwoBuf && cc + 1 < T.total) {
                        ok = mbar_wait(bar_col + 8 * ((g + 1) % kStages), ((g + 1) / kStages) & 1, abort_flag, P.wait_budget);
                        if (!ok) break;
                        STAMP(216);
                        issue_s_dp(g + 1, cc + 1, T);                                // ... before the next S/dP overwrite them
                    }
                    STAMP(220);
                }
                ++tileno;
            }
        }
    } else if (warp == kComputeWarps + 1) {
        // =====================================================================
        // helper warp: row tables one tile ahead; the loads (lane 0: row tiles, then the ring of column tiles,
        // as far ahead of the tensor cores as the stages allow); on the key side also the column statistics
        // (lse*log2e and delta of the chunk's queries) that go with each column tile
        // =====================================================================
        bool ok = !*abort_flag;
        unsigned g = 0;
        // table of work item `work` (the item-th of this CTA) into slot item & 1
        auto write_table = [&](unsigned work, unsigned item, const BwdTile& X) {
            const unsigned slot = item & 1;
            if (item >= 2) ok = ok && mbar_wait(bar_tab_empty + 8 * slot, ((item >> 1) - 1) & 1, abort_flag, P.wait_budget);
            uint8_t* tab = smem + Smem::kTab + slot * Smem::kTabBytes;
            AxisEntry* ent = reinterpret_cast<AxisEntry*>(tab);
            int base = 0;
#pragma unroll
            for (int a = 0; a < 3; ++a) {
                for (int i = lane; i < P.tile[a]; i += 32) {
                    const int xa = X.origin[a] + i;
                    AxisEntry en;
                    en.pa = X.rg[a] + P.dil[a] * xa;
                    en.flags = (xa < X.Lp[a] ? 1 : 0) | (en.pa < P.L[a] ? 2 : 0);
                    int fa = 0, ea = 0;
                    if (X.active) {
                        if (kKeySide) {
                            int qlo, qhi;
                            inverse_range(xa, X.Lp[a], P.K[a], P.causal[a], qlo, qhi);
                            fa = qlo - X.boxlo[a];
                            ea = qhi + 1 - X.boxlo[a];
                        } else {
                            const int first = P.causal[a] ? xa - (P.K[a] - 1) : ws1(xa, X.Lp[a], P.K[a]);
                            fa = (first > 0 ? first : 0) - X.boxlo[a];
                            ea = (first + P.K[a] < X.Lp[a] ? first + P.K[a] : X.Lp[a]) - X.boxlo[a];
                        }
                    }
                    en.f = (short)fa;
                    en.e = (short)ea;
                    en.pad = 0;
                    ent[base + i] = en;
                }
                base += P.tile[a];
            }
            if (lane == 0) {
                TileHead* hd = reinterpret_cast<TileHead*>(tab + kAxisEntries * 16);
                hd->active = X.active ? 1 : 0;
                hd->total = X.total;
                hd->nbox = X.nbox;
                hd->nchunks = X.nchunks;
                hd->b = X.b;
                hd->hy = X.hy;
                hd->rg0 = (short)X.rg[0]; hd->rg1 = (short)X.rg[1]; hd->rg2 = (short)X.rg[2];
                hd->origin0 = (short)X.origin[0]; hd->origin1 = (short)X.origin[1]; hd->origin2 = (short)X.origin[2];
#pragma unroll
                for (int a = 0; a < 3; ++a) { hd->nc[a] = X.nc[a]; hd->boxlo[a] = X.boxlo[a]; hd->Lp[a] = X.Lp[a]; }
            }
            mbar_arrive(bar_tab_full + 8 * slot);
        };
        auto issue_rows = [&](const BwdTile& X) {
            const int hx = X.hy * DH;
            mbar_expect_tx(bar_row, 2 * kTile);
#pragma unroll
            for (int hf = 0; hf < Smem::kHalves; ++hf) {
                tma_load_heads(sbase + Smem::kR1 + hf * kRowHalf, &tmR1, bar_row, P, DH, hx + 64 * hf, X.rg[2] + P.dil[2] * X.origin[2],
                            X.rg[1] + P.dil[1] * X.origin[1], X.rg[0] + P.dil[0] * X.origin[0], X.b);
                tma_load_heads(sbase + Smem::kR2 + hf * kRowHalf, &tmR2, bar_row, P, DH, hx + 64 * hf, X.rg[2] + P.dil[2] * X.origin[2],
                            X.rg[1] + P.dil[1] * X.origin[1], X.rg[0] + P.dil[0] * X.origin[0], X.b);
            }
        };
        BwdTile T, Tn;
        unsigned item = 0, tiles = 0;
        if (blockIdx.x < nwork) {
            bwd_tile_setup<kKeySide>(P, blockIdx.x, T);
            write_table(blockIdx.x, 0, T);
        }
        for (unsigned work = blockIdx.x; work < nwork; work += gridDim.x, ++item) {
            const unsigned wn = work + gridDim.x;
            STAMP(390);
            if (wn < nwork) {                    // the next item's table first: it is needed before this tile ends
                bwd_tile_setup<kKeySide>(P, wn, Tn);
                write_table(wn, item + 1, Tn);
            }
            STAMP(395);
            if (T.active) {
                // the row tiles are free once the previous tile's last S / dP products have finished
                if (tiles > 0) ok = ok && mbar_wait(bar_rowfree, (tiles - 1) & 1, abort_flag, P.wait_budget);
                STAMP(398);
                if (lane == 0 && ok) issue_rows(T);
                ++tiles;
                int ci[3] = {0, 0, 0}, hc = T.hy * P.group;
                const int head_kv = kKeySide ? T.hy : T.hy / P.group;
                for (int cc = 0; cc < T.total; ++cc, ++g) {
                    const int s = g % kStages;
                    STAMP(400 + cc);
                    // key side: the chunk's column statistics are fetched before the wait for the stage, so that
                    // their latency is not part of what follows it
                    float raw_lse[kCols / 32], raw_delta[kCols / 32];
                    if (kKeySide) {
#pragma unroll
                        for (int k = 0; k < kCols / 32; ++k) {
                            const int j = lane + 32 * k;
                            const int j2 = j & (P.cb[2] - 1);
                            const int j1 = (j >> P.cb2_log) & (P.cb[1] - 1);
                            const int j0 = j >> (P.cb2_log + P.cb1_log);
                            const int q0 = T.boxlo[0] + chunk_coord(P, 0, ci[0], j0);
                            const int q1 = T.boxlo[1] + chunk_coord(P, 1, ci[1], j1);
                            const int q2 = T.boxlo[2] + chunk_coord(P, 2, ci[2], j2);
                            const bool inside = ok && q0 >= 0 && q0 < T.Lp[0] && q1 >= 0 && q1 < T.Lp[1] && q2 >= 0 && q2 < T.Lp[2];
                            raw_lse[k] = 0.f;
                            raw_delta[k] = 0.f;
                            if (inside) {
                                const long long pflat = ((long long)(T.rg[0] + P.dil[0] * q0) * P.L[1] + (T.rg[1] + P.dil[1] * q1)) * P.L[2]
                                                        + (T.rg[2] + P.dil[2] * q2);
                                const long long row = ((long long)T.b * P.ltot + pflat) * P.Hq + hc;
                                raw_lse[k] = lse[row];
                                raw_delta[k] = delta[row];
                            }
                        }
                    }
                    if (g >= (unsigned)kStages) ok = ok && mbar_wait(bar_free + 8 * s, ((g / kStages) - 1) & 1, abort_flag, P.wait_budget);
                    STAMP(410);
                    if (lane == 0 && ok) {
                        const uint32_t bar = bar_col + 8 * s;
                        mbar_expect_tx(bar, 2 * kColTile);
                        if (cc < T.nbox) {
                            int X[3];
#pragma unroll
                            for (int a = 0; a < 3; ++a) X[a] = T.rg[a] + P.dil[a] * (T.boxlo[a] + chunk_coord(P, a, ci[a], 0));
                            // query side: columns are keys (kv head); key side: columns are queries (query head)
                            const int hx = (kKeySide ? hc : head_kv) * DH;
#pragma unroll
                            for (int hf = 0; hf < Smem::kHalves; ++hf) {
                                tma_load_heads(sbase + Smem::kC1 + s * kColTile + hf * kColHalf, &tmC1, bar, P, DH, hx + 64 * hf, X[2], X[1], X[0], T.b);
                                tma_load_heads(sbase + Smem::kC2 + s * kColTile + hf * kColHalf, &tmC2, bar, P, DH, hx + 64 * hf, X[2], X[1], X[0], T.b);
                            }
                        } else {                             // additional tokens (rows past n_extra are zero-filled)
                            const int e0 = (cc - T.nbox) * kCols;
#pragma unroll
                            for (int hf = 0; hf < Smem::kHalves; ++hf) {
                                tma_load_heads(sbase + Smem::kC1 + s * kColTile + hf * kColHalf, &tmE1, bar, P, DH, head_kv * DH + 64 * hf, e0, 0, 0, T.b);
                                tma_load_heads(sbase + Smem::kC2 + s * kColTile + hf * kColHalf, &tmE2, bar, P, DH, head_kv * DH + 64 * hf, e0, 0, 0, T.b);
                            }
                        }
                    }
                    __syncwarp();
                    if (!kKeySide) {
                        if (cc < T.nbox && ++ci[2] == T.nc[2]) { ci[2] = 0; if (++ci[1] == T.nc[1]) { ci[1] = 0; ++ci[0]; } }
                        continue;
                    }
                    float* st = stats + s * 128;
#pragma unroll
                    for (int k = 0; k < kCols / 32; ++k) {               // negated, pre-scaled addends
                        st[lane + 32 * k] = -raw_lse[k] * 1.4426950408889634f;
                        st[kCols + lane + 32 * k] = -raw_delta[k] * P.scale;
                    }
                    mbar_arrive(bar_stats + 8 * s);
                    if (++ci[2] == T.nc[2]) { ci[2] = 0; if (++ci[1] == T.nc[1]) { ci[1] = 0; if (++ci[0] == T.nc[0]) { ci[0] = 0; ++hc; } } }
                }
            }
            T = Tn;
        }
    } else {
        // =====================================================================
        // compute warps: thread = (row, 32-column piece)
        // =====================================================================
        const uint32_t trow = tmem + (static_cast<uint32_t>(quad * 32) << 16);
        bool ok = true;
        unsigned g = 0;                          // chunks processed so far (all tiles)
        constexpr int kPairs = kInner > 0 ? kInner / 2 : 1;
        unsigned item = 0;
        for (unsigned work = blockIdx.x; work < nwork; work += gridDim.x, ++item) {
            // ---- this thread's row, from the helper warp's table ----
            const unsigned slot = item & 1;
            ok = mbar_wait(bar_tab_full + 8 * slot, (item >> 1) & 1, abort_flag, P.wait_budget) && ok;
            const uint8_t* tab = smem + Smem::kTab + slot * Smem::kTabBytes;
            STAMP(300);
            const TileHead T = *reinterpret_cast<const TileHead*>(tab + kAxisEntries * 16);
            int f[3], e[3];
            bool valid_row = true, in_tensor = true;
            long long pflat = 0;
            {
                int ri[3];
                row_offsets(P, quad * 32 + lane, ri);
                const AxisEntry* ent = reinterpret_cast<const AxisEntry*>(tab);
                int base = 0;
#pragma unroll
                for (int a = 0; a < 3; ++a) {
                    const AxisEntry en = ent[base + ri[a]];
                    base += P.tile[a];
                    f[a] = en.f;
                    e[a] = en.e;
                    valid_row = valid_row && (en.flags & 1);
                    in_tensor = in_tensor && (en.flags & 2);
                    pflat = pflat * P.L[a] + en.pa;
                }
            }
            mbar_arrive(bar_tab_empty + 8 * slot);
            STAMP(301);
            if (!valid_row) { e[0] = f[0]; e[1] = f[1]; e[2] = f[2]; }
            const long long out_row = ((long long)T.b * P.ltot + pflat) * (kKeySide ? P.Hkv : P.Hq) + T.hy;
            // query side: the row's lse and delta; scaled where they are first used, so that the loads' latency
            // runs under the set-up of the first chunk and the wait for its scores
            float raw_lse = 0.f, raw_delta = 0.f;
            if (!kKeySide && valid_row && in_tensor && T.active && ok) {
                raw_lse = lse[out_row];
                raw_delta = delta[out_row];
            }
            STAMP(302);
            if (!T.active) {                     // padding rows get zero gradients
                if (in_tensor) {
#pragma unroll
                    for (int which = 0; which < (kKeySide ? 2 : 1); ++which) {
                        uint4* o = reinterpret_cast<uint4*>((which == 0 ? out1 : out2) + out_row * P.dreal + piece * CH);
#pragma unroll
                        for (int i = 0; i < CH / 8; ++i)
                            if (piece * CH + 8 * i < P.dreal) o[i] = make_uint4(0, 0, 0, 0);
                    }
                }
                continue;
            }
            const int nbox = T.nbox;
            // Chunk columns of this warp's half h, and where its 16-bit pairs go.  With 16-column inner rows a
            // chunk is four rows: the warp takes rows piece and piece + 2, so that the two warps of a lane
            // quadrant share a row's window evenly when the chunk rows are interleaved; the pairs of a row
            // overwrite the first 8 of its own 16 columns.  Otherwise the warp takes 32 adjacent columns whose
            // pairs fill the first 16 of them.
            auto col0 = [&](int h) { return kInner == 16 ? 16 * (piece + 2 * h) : 32 * piece + 16 * h; };
            auto dst0 = [&](int h) { return kInner == 16 ? 16 * (piece + 2 * h) : 32 * piece + 8 * h; };
            int ci[3] = {0, 0, 0};               // chunk index per axis, advanced without divisions
            const bool line = line_chunks(P);    // chunks are runs of the innermost axis (1-D windows): cheap validity words
            uint32_t colmask[kPairs];            // separable geometry: 16-bit lane masks per column pair
            bool cols_any = false;
            int cached_c2 = -1;
            // 16-column inner rows, one chunk along the innermost axis, at most 16 chunks in the box: which of a
            // chunk's four rows lie inside this thread's range is worked out once per tile from the row's side
            // (every row of the range lands in one row of one chunk), four bits per chunk.
            bool mapped = false;
            unsigned long long rowmap = 0ull;
            int cl = 0;                          // chunk of the box (wraps with every query head on the key side)
            if (kInner == 16 && T.nc[2] == 1 && T.nchunks <= 16) {
                mapped = true;
                for (int x0 = f[0]; x0 < e[0]; ++x0) {
                    int c0, j0;
                    if (P.il[0] == 1) { c0 = x0 >> P.cb0_log; j0 = x0 & (P.cb[0] - 1); }
                    else { j0 = (int)fast_div((unsigned)x0, P.il_mul[0]); c0 = x0 - j0 * P.il[0]; }
                    for (int x1 = f[1]; x1 < e[1]; ++x1) {
                        int c1, j1;
                        if (P.il[1] == 1) { c1 = x1 >> P.cb1_log; j1 = x1 & (P.cb[1] - 1); }
                        else { j1 = (int)fast_div((unsigned)x1, P.il_mul[1]); c1 = x1 - j1 * P.il[1]; }
                        rowmap |= 1ull << (4 * (c0 * T.nc[1] + c1) + (j0 << P.cb1_log) + j1);
                    }
                }
            }
            for (int cc = 0; cc < T.total; ++cc, ++g) {
                // ---- validity of this warp's two 16-column halves for this thread's row ----
                // half h covers chunk columns col0(h) .. col0(h)+15; bits [16h, 16h+16) of `word` belong to it
                uint32_t word = 0u;                  // generic geometry / additional tokens: one bit per column
                uint32_t rowmask[2] = {0u, 0u};      // separable geometry: all-ones / zero per inner row
                bool mine[2] = {false, false};
                const bool extra = !kKeySide && cc >= nbox;      // additional tokens: first n_extra columns, every live row
                if (extra) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t w = valid_row ? (low_bits(P.n_extra - ((cc - nbox) * kCols + col0(h))) & 0xFFFFu) : 0u;
                        word |= w << (16 * h);
                        mine[h] = w != 0u;
                    }
                } else if (kInner > 0) {
                    // columns of this chunk inside the row's window, per axis (chunks may be interleaved)
                    if (ci[2] != cached_c2) {        // the column masks only change with the innermost chunk index
                        cached_c2 = ci[2];
                        int lo2, hi2;
                        chunk_range(P, 2, ci[2], f[2], e[2], lo2, hi2);
#pragma unroll
                        for (int i = 0; i < kPairs; ++i)
                            colmask[i] = ((2 * i >= lo2 && 2 * i < hi2) ? 0x0000FFFFu : 0u) |
                                         ((2 * i + 1 >= lo2 && 2 * i + 1 < hi2) ? 0xFFFF0000u : 0u);
                        cols_any = hi2 > lo2;
                    }
                    if (mapped) {
                        const uint32_t bits = (uint32_t)(rowmap >> (4 * cl)) & 15u;
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const bool rok = (bits >> (piece + 2 * h)) & 1u;
                            rowmask[h] = rok ? 0xFFFFFFFFu : 0u;
                            mine[h] = rok && cols_any;
                        }
                    } else {
                        int lo0, hi0, lo1, hi1;
                        chunk_range(P, 0, ci[0], f[0], e[0], lo0, hi0);
                        chunk_range(P, 1, ci[1], f[1], e[1], lo1, hi1);
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const int jj = col0(h);
                            const int j1 = (jj >> P.cb2_log) & (P.cb[1] - 1);
                            const int j0 = jj >> (P.cb2_log + P.cb1_log);
                            const bool rok = j0 >= lo0 && j0 < hi0 && j1 >= lo1 && j1 < hi1;
                            rowmask[h] = rok ? 0xFFFFFFFFu : 0u;
                            mine[h] = rok && cols_any;
                        }
                    }
                } else {
                    if (line) {
                        word = line_word(P, piece, ci, f, e);
                    } else {
                        int jl[3], jh[3];
#pragma unroll
                        for (int a = 0; a < 3; ++a) chunk_range(P, a, ci[a], f[a], e[a], jl[a], jh[a]);
                        word = piece_word_ranges(P, piece, jl, jh);
                    }
                    mine[0] = (word & 0xFFFFu) != 0u;
                    mine[1] = (word >> 16) != 0u;
                }
#if NATTEN_ABL == 2
                const bool any[2] = {false, false};
#else
                const bool any[2] = {__any_sync(0xffffffffu, mine[0]) != 0, __any_sync(0xffffffffu, mine[1]) != 0};
#endif
                const bool separable = kInner > 0 && !extra;
                const bool full = !separable && __all_sync(0xffffffffu, word == 0xffffffffu);
                STAMP(310 + ((any[0] || any[1]) ? 1 : 0));
                ok = ok && mbar_wait(bar_s_of(g), par_of(g), abort_flag, P.wait_budget);      // also: the P/dS this buffer held were consumed
                const uint32_t tbuf = trow + buf_cols(g);
                if (kKeySide) ok = ok && mbar_wait(bar_stats + 8 * (g % kStages), (g / kStages) & 1, abort_flag, P.wait_budget);
                tc_fence_after();
                STAMP(320);
                const float row_lse2 = -raw_lse * 1.4426950408889634f, row_delta = -raw_delta * P.scale;   // negated, pre-scaled addends
                const uint64_t scale_log2_2 = pack2(P.scale_log2, P.scale_log2), scale_2 = pack2(P.scale, P.scale);
#pragma unroll
                for (int half = 0; half < 2; ++half) {               // 16 columns at a time
                    uint32_t pk_p[8], pk_ds[8];
                    if (any[half]) {
                        const float* stp = stats + (g % kStages) * 128 + col0(half);
                        const float4* st4 = reinterpret_cast<const float4*>(stp);
                        uint32_t s[16], dp[16];
                        tmem_ld16(tbuf + kColS + col0(half), s);
                        tmem_ld16(tbuf + kColDP + col0(half), dp);
                        tmem_ld_wait();
                        if (separable || full) {
                            // P = 2^(s*c - lse2), dS = P * (dP*scale - delta*scale); fp32, rounded once each
#pragma unroll
                            for (int g4 = 0; g4 < 4; ++g4) {             // four columns at a time
                                float nl[4], nd[4];
                                if (kKeySide) {
                                    const float4 a = st4[g4], d = st4[kCols / 4 + g4];
                                    nl[0] = a.x; nl[1] = a.y; nl[2] = a.z; nl[3] = a.w;
                                    nd[0] = d.x; nd[1] = d.y; nd[2] = d.z; nd[3] = d.w;
                                } else {
#pragma unroll
                                    for (int u = 0; u < 4; ++u) { nl[u] = row_lse2; nd[u] = row_delta; }
                                }
#pragma unroll
                                for (int h2 = 0; h2 < 2; ++h2) {
                                    const int pl = 2 * g4 + h2, j = 2 * pl;      // pair / column inside the half
                                    // two columns per instruction: packed fp32 fma / mul
                                    const uint64_t x = fma2(pack2(__uint_as_float(s[j]), __uint_as_float(s[j + 1])), scale_log2_2,
                                                            pack2(nl[2 * h2], nl[2 * h2 + 1]));
                                    const float p0 = fast_exp2(lo_of(x)), p1 = fast_exp2(hi_of(x));
                                    const uint64_t gg = fma2(pack2(__uint_as_float(dp[j]), __uint_as_float(dp[j + 1])), scale_2,
                                                             pack2(nd[2 * h2], nd[2 * h2 + 1]));
                                    const uint64_t ds2 = mul2(pack2(p0, p1), gg);
                                    uint32_t dd = cvt_pack<BF16>(lo_of(ds2), hi_of(ds2));
                                    if (separable) dd = dd & colmask[(8 * half + pl) % kPairs] & rowmask[kInner == 16 ? half : 0];
                                    pk_ds[pl] = dd;
                                    if (kKeySide) {
                                        uint32_t pp = cvt_pack<BF16>(p0, p1);
                                        if (separable) pp = pp & colmask[(8 * half + pl) % kPairs] & rowmask[kInner == 16 ? half : 0];
                                        pk_p[pl] = pp;
                                    }
                                }
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                float pv[2], dsv[2];
#pragma unroll
                                for (int u = 0; u < 2; ++u) {
                                    const int j = 2 * i + u;
                                    const float nl = kKeySide ? stp[j] : row_lse2;
                                    const float nd = kKeySide ? stp[kCols + j] : row_delta;
                                    const bool on = (word >> (16 * half + j)) & 1u;
                                    const float p = on ? fast_exp2(fmaf(__uint_as_float(s[j]), P.scale_log2, nl)) : 0.f;
                                    pv[u] = p;
                                    dsv[u] = p * fmaf(__uint_as_float(dp[j]), P.scale, nd);
                                }
                                pk_p[i] = pack16(pv[0], pv[1], BF16);
                                pk_ds[i] = pack16(dsv[0], dsv[1], BF16);
                            }
                        }
                    } else {                             // nothing valid in this half: the MMA must read zeros
#pragma unroll
                        for (int i = 0; i < 8; ++i) { pk_p[i] = 0u; pk_ds[i] = 0u; }
                    }
                    // the pairs overwrite columns this warp has already read (or will not read)
                    tmem_st8(tbuf + kColDP + dst0(half), pk_ds);
                    if (kKeySide) tmem_st8(tbuf + kColS + dst0(half), pk_p);
                }
                tmem_st_wait();
                tc_fence_before();
                mbar_arrive(bar_sp_of(g));
                STAMP(330);
                // next chunk (innermost axis fastest; wraps to the next query head on the key side)
                if (mapped) {
                    if (++cl == T.nchunks) cl = 0;
                } else if (++ci[2] == T.nc[2]) {
                    ci[2] = 0;
                    if (++ci[1] == T.nc[1]) {
                        ci[1] = 0;
                        if (++ci[0] == T.nc[0]) ci[0] = 0;
                    }
                }
            }

            // ---- accumulators -> global: this warp owns 32 of the 64 channels ----
            STAMP(340);
            ok = ok && mbar_wait(bar_free + 8 * ((g - 1) % kStages), ((g - 1) / kStages) & 1, abort_flag, P.wait_budget);   // the last chunk's accumulating products
            tc_fence_after();
            STAMP(350);
            // The accumulators leave through shared memory and a bulk tensor store: every thread converts its
            // 32 channels of its row and writes them into a [128 x DH] tile laid out like the row tiles the loads
            // bring in (128-byte rows, 16-byte chunks swizzled by the row); one thread then hands the tile to the
            // TMA unit, which writes it out in the background (rows outside the tensor are clipped) while the
            // threads go on.  The tile is reused only after that thread has seen the store finish reading it.
            const bool live = valid_row && ok;
            const int row = quad * 32 + lane;
#pragma unroll
            for (int which = 0; which < (kKeySide ? 2 : 1); ++which) {
                if (warp == 0 && lane == 0) tma_store_wait_read();               // the previous store has let go of the tile
                asm volatile("bar.sync 1, 256;" ::: "memory");
#pragma unroll
                for (int part = 0; part < CH / 32; ++part) {
                    uint32_t a[32];
                    tmem_ld32(trow + (which == 0 ? kColA1 : kColA2) + CH * piece + 32 * part, a);
                    tmem_ld_wait();
                    const int ch = CH * piece + 32 * part;                   // first of this thread's 32 channels
                    uint8_t* blk = smem + Smem::kStage + (ch >> 6) * kRowHalf + row * 128;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t w[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            w[j] = live ? pack16(__uint_as_float(a[8 * c + 2 * j]), __uint_as_float(a[8 * c + 2 * j + 1]), BF16) : 0u;
                        const int chunk = ((ch & 63) >> 3) + c;
                        *reinterpret_cast<uint4*>(blk + ((chunk ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
                fence_async_smem();                                          // the TMA unit reads through the async proxy
                asm volatile("bar.sync 1, 256;" ::: "memory");
                if (warp == 0 && lane == 0 && ok && NATTEN_ABL != 1) {
                    const CUtensorMap* map = which == 0 ? &tmO1 : &tmO2;
#pragma unroll
                    for (int hf = 0; hf < Smem::kHalves; ++hf)
                        tma_store_heads(map, sbase + Smem::kStage + hf * kRowHalf, P, DH, T.hy * DH + 64 * hf,
                                        T.rg2 + P.dil[2] * T.origin2, T.rg1 + P.dil[1] * T.origin1, T.rg0 + P.dil[0] * T.origin0, T.b);
                    tma_store_commit();
                }
            }
            // the next tile's first accumulating MMA is issued only after every thread has passed here
            tc_fence_before();
            STAMP(360);
        }
    }

    if (warp == 0 && lane == 0) tma_store_wait_all();     // bulk stores of the last tiles
    if (*abort_flag) abort_grace_sleep();       // loads of a wait that gave up may still be landing
    tc_fence_before();
    __syncthreads();
    if (warp == kComputeWarps) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
        if (lane == 0 && *abort_flag) atomicExch(P.status, 1);
    }
}

// delta[row] = sum_d out[row,d]*dout[row,d] - dlse[row]      (kPer threads per row, 16 bytes each, kPer the
// power of two >= D/8; every thread takes kDeltaRows rows a grid-width apart, so that eight 16-byte loads
// are in flight).  blockIdx.y picks a slab of `slab_rows` consecutive rows; with per-sample lengths of a 1-D
// problem (lens != nullptr) a slab is one sample, row = position * heads + head inside it, and the rows past
// the sample's length are not read: nothing attends from them, their delta is 0.
constexpr int kDeltaRows = 4;
template <int kPer, bool BF16, bool kLens>
__global__ void __launch_bounds__(256)
tc_delta_kernel(const uint16_t* __restrict__ out, const uint16_t* __restrict__ dout,
                const float* __restrict__ dlse, float* __restrict__ delta, long long slab_rows, long long row_step, int D,
                const int* __restrict__ lens, int heads)
{
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long local0 = t / kPer;
    const int part = (int)(t % kPer);
    const bool mine = 8 * part < D;
    long long live_rows = slab_rows;
    if constexpr (kLens) {   // this slab's rows are rows 0 .. slab_rows-1 from here on
        const long long base = (long long)blockIdx.y * slab_rows;
        out += base * D;
        dout += base * D;
        delta += base;
        if (dlse) dlse += base;
        live_rows = (long long)lens[blockIdx.y] * heads;
        live_rows = live_rows < slab_rows ? live_rows : slab_rows;
    }
    uint4 a[kDeltaRows], g[kDeltaRows];
#pragma unroll
    for (int r = 0; r < kDeltaRows; ++r) {
        const long long local = local0 + r * row_step;
        a[r] = make_uint4(0, 0, 0, 0);
        g[r] = make_uint4(0, 0, 0, 0);
        if (local < live_rows && mine) {
            a[r] = reinterpret_cast<const uint4*>(out + local * D)[part];
            g[r] = reinterpret_cast<const uint4*>(dout + local * D)[part];
        }
    }
#pragma unroll
    for (int r = 0; r < kDeltaRows; ++r) {
        const long long local = local0 + r * row_step;
        const uint32_t aw[4] = {a[r].x, a[r].y, a[r].z, a[r].w}, gw[4] = {g[r].x, g[r].y, g[r].z, g[r].w};
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 x, y;
            if (BF16) {
                x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&aw[i]));
                y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gw[i]));
            } else {
                x = __half22float2(*reinterpret_cast<const __half2*>(&aw[i]));
                y = __half22float2(*reinterpret_cast<const __half2*>(&gw[i]));
            }
            acc += x.x * y.x + x.y * y.y;
        }
#pragma unroll
        for (int o = 1; o < kPer; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (local < slab_rows && part == 0) delta[local] = (!kLens || local < live_rows) ? acc - (dlse ? dlse[local] : 0.f) : 0.f;
    }
}

// Output stride > 1: only every stride-th position is a query.  The backward kernels keep their
// unit-stride geometry and get full-resolution copies of dout, lse and delta instead: at a query position
// the caller's row, elsewhere dout = 0, delta = 0 and lse = 1e30, so that the recomputed probability of such
// a row is exp(s - 1e30) = 0 and it contributes exactly nothing (its dq row comes out as zeros, which is
// what the operator defines for positions that are not queries).
struct Expanded {
    const Geo* original;           // the caller's (strided) geometry
    void* dout_full;               // [B, *L, Hq, D]
    float *lse_full, *delta_full;  // [B, *L, Hq]
};

__global__ void __launch_bounds__(256)
expand_strided_kernel(const __grid_constant__ Geo g, const uint4* __restrict__ dout, const float* __restrict__ lse,
                      const float* __restrict__ delta, uint4* __restrict__ dout_full, float* __restrict__ lse_full,
                      float* __restrict__ delta_full, long long total, int vecs)
{
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int vec = (int)(i % vecs);
    const long long row = i / vecs;                    // (b * ltot + p) * Hq + h
    const int h = (int)(row % g.Hq);
    long long p = (row / g.Hq) % g.ltot;
    const long long b = row / g.Hq / g.ltot;
    bool query = true;
    long long oflat = 0, mul = 1;
    for (int a = g.rank - 1; a >= 0; --a) {
        const int pos = (int)(p % g.L[a]);
        p /= g.L[a];
        if (pos % g.st[a] != 0) query = false;
        oflat += (long long)(pos / g.st[a]) * mul;
        mul *= g.O[a];
    }
    const long long orow = (b * g.otot + oflat) * g.Hq + h;
    dout_full[i] = query ? dout[orow * vecs + vec] : make_uint4(0, 0, 0, 0);
    if (vec == 0) {
        lse_full[row] = query ? lse[orow] : 1e30f;
        delta_full[row] = query ? delta[orow] : 0.f;
    }
}

template <int DH, bool BF16>
int launch_bwd(int dtype, const Geo& g, const Plan& plan, const void* q, const void* k, const void* v,
               const void* ek, const void* ev, void* dek, void* dev, const void* out, const void* lse, const void* dout, const void* dlse, void* dq, void* dk,
               void* dv, float* delta, cudaStream_t s, const Expanded* ex = nullptr)
{
    const TcParams& p = plan.p;
    // With an output stride the kernels run on the unit-stride geometry `g` over full-resolution copies of
    // dout / lse / delta (see expand_strided_kernel); the caller's arrays are only read to build them.
    const void* dout_k = ex ? ex->dout_full : dout;
    const float* lse_k = ex ? ex->lse_full : (const float*)lse;
    const float* delta_k = ex ? ex->delta_full : delta;
    const long long dos[3] = {g.ltot * g.Hq * g.Dv, (long long)g.Hq * g.Dv, g.Dv};   // dout is contiguous
    CUtensorMap q_tile, do_tile, k_chunk, v_chunk, k_tile, v_tile, q_chunk, do_chunk, ek_chunk, ev_chunk;
    const bool bf = BF16;
    using Smem = SmemB<DH>;
    if (!encode_map(&q_tile, q, bf, p, g.Hq, g.D, g.qs, plan.box_q) ||
        !encode_map(&do_tile, dout_k, bf, p, g.Hq, g.D, dos, plan.box_q) ||
        !encode_map(&k_chunk, k, bf, p, g.Hkv, g.D, g.ks, plan.box_kv, false, /*interleaved=*/true) ||
        !encode_map(&v_chunk, v, bf, p, g.Hkv, g.D, g.vs, plan.box_kv, false, true) ||
        !encode_map(&k_tile, k, bf, p, g.Hkv, g.D, g.ks, plan.box_q) ||
        !encode_map(&v_tile, v, bf, p, g.Hkv, g.D, g.vs, plan.box_q) ||
        !encode_map(&q_chunk, q, bf, p, g.Hq, g.D, g.qs, plan.box_kv, false, true) ||
        !encode_map(&do_chunk, dout_k, bf, p, g.Hq, g.D, dos, plan.box_kv, false, true))
        return -2;
    // outputs: contiguous [B, *L, H, D]; stored as row tiles
    CUtensorMap dq_tile, dk_tile, dv_tile;
    const long long dqs[3] = {g.ltot * g.Hq * g.D, (long long)g.Hq * g.D, g.D};
    const long long dks[3] = {g.ltot * g.Hkv * g.D, (long long)g.Hkv * g.D, g.D};
    if (!encode_map(&dq_tile, dq, bf, p, g.Hq, g.D, dqs, plan.box_q) ||
        !encode_map(&dk_tile, dk, bf, p, g.Hkv, g.D, dks, plan.box_q) ||
        !encode_map(&dv_tile, dv, bf, p, g.Hkv, g.D, dks, plan.box_q))
        return -2;
    ek_chunk = k_chunk; ev_chunk = v_chunk;      // placeholders when there are no additional tokens
    if (g.n_extra > 0 && (!encode_extra_map(&ek_chunk, ek, bf, g.B, g.n_extra, g.Hkv, g.D, kCols, p.split_heads) ||
                          !encode_extra_map(&ev_chunk, ev, bf, g.B, g.n_extra, g.Hkv, g.D, kCols, p.split_heads)))
        return -2;
    // delta only once nothing can send this call to the other kernel family any more
    const Geo& go = ex ? *ex->original : g;      // geometry of out / dout / lse as the caller holds them
    {
        const long long qrows = (long long)go.B * go.otot * go.Hq;
        // per-sample lengths of a 1-D problem without output stride: one slab of rows per sample, rows past its
        // length are skipped; otherwise the whole tensor is one slab
        const int* lens = (go.extents && go.rank == 1 && go.otot == go.ltot && go.B <= 65535) ? go.extents : nullptr;
        const long long slab_rows = lens ? go.otot * go.Hq : qrows;
        const unsigned slabs = lens ? (unsigned)go.B : 1u;
        // rows handled per pass of the grid: a whole number of blocks, a quarter of a slab's rows each
        auto run_delta = [&](auto per) {
            constexpr int kPer = decltype(per)::value;
            const long long rows_per_block = 256 / kPer;
            const long long blocks = ((slab_rows + kDeltaRows - 1) / kDeltaRows + rows_per_block - 1) / rows_per_block;
            if (lens)
                tc_delta_kernel<kPer, BF16, true><<<dim3((unsigned)blocks, slabs), 256, 0, s>>>(
                    (const uint16_t*)out, (const uint16_t*)dout, (const float*)dlse, delta, slab_rows, blocks * rows_per_block, g.D,
                    lens, go.Hq);
            else
                tc_delta_kernel<kPer, BF16, false><<<(unsigned)blocks, 256, 0, s>>>(
                    (const uint16_t*)out, (const uint16_t*)dout, (const float*)dlse, delta, slab_rows, blocks * rows_per_block, g.D,
                    nullptr, go.Hq);
        };
        if (g.D <= 32) run_delta(std::integral_constant<int, 4>{});
        else if (g.D <= 64) run_delta(std::integral_constant<int, 8>{});
        else run_delta(std::integral_constant<int, 16>{});
    }
    tc_count_launch();
    if (ex) {                                    // scatter dout / lse / delta onto the full-resolution grid
        const long long rows_full = (long long)g.B * g.ltot * g.Hq;
        const int vecs = g.D / 8;
        const long long total = rows_full * vecs;
        expand_strided_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(
            *ex->original, (const uint4*)dout, (const float*)lse, delta, (uint4*)ex->dout_full, ex->lse_full,
            ex->delta_full, total, vecs);
        tc_count_launch();
    }

    int ngroups = 1;
    for (int a = 0; a < 3; ++a) ngroups *= p.dil[a];
    const dim3 grid_q(persistent_grid(p.work_q, DH == 64 ? 2 : 1));
    const dim3 grid_k(persistent_grid(p.work_kv, DH == 64 ? 2 : 1));
    auto launch = [&](auto inner) {
        constexpr int kInner = decltype(inner)::value;
        ensure_dynamic_smem((const void*)tc_bwd_kernel<DH, BF16, false, kInner>, Smem::kTotal);
        ensure_dynamic_smem((const void*)tc_bwd_kernel<DH, BF16, true, kInner>, Smem::kTotal);
        tc_bwd_kernel<DH, BF16, false, kInner><<<grid_q, kThreads, Smem::kTotal, s>>>(
            q_tile, do_tile, k_chunk, v_chunk, ek_chunk, ev_chunk, dq_tile, dq_tile, p, lse_k, delta_k, (uint16_t*)dq, nullptr);
        tc_count_launch();
        tc_bwd_kernel<DH, BF16, true, kInner><<<grid_k, kThreads, Smem::kTotal, s>>>(
            k_tile, v_tile, q_chunk, do_chunk, ek_chunk, ev_chunk, dk_tile, dv_tile, p, lse_k, delta_k, (uint16_t*)dk, (uint16_t*)dv);
        tc_count_launch();
    };
    if (p.cb[2] == 16) launch(std::integral_constant<int, 16>{});
    else if (p.cb[2] == 32) launch(std::integral_constant<int, 32>{});
    else launch(std::integral_constant<int, 0>{});
    cudaError_t err = cudaGetLastError();
    // The additional tokens' own gradients sum over every query of the sample: SIMT kernel.
    if (err == cudaSuccess && g.n_extra > 0)
        err = simt_fused_bwd_extra(dtype, go, q, ek, ev, lse, delta, dout, dek, dev,
                                   reinterpret_cast<unsigned char*>(delta) + simt_delta_bytes(go, 4), s);
    return err == cudaSuccess ? 0 : (int)err;
}

} // namespace

namespace {
size_t align256(size_t n) { return (n + 255) & ~(size_t)255; }
bool has_stride(const Geo& g)
{
    for (int a = 0; a < g.rank; ++a)
        if (g.st[a] != 1) return true;
    return false;
}
} // namespace

int tc_fused_bwd(int dtype, const Geo& g_in, const void* q, const void* k, const void* v, const void* ek,
                 const void* ev, const void* out, const void* lse, const void* dout, const void* dlse,
                 void* dq, void* dk, void* dv, void* dek, void* dev, void* workspace, cudaStream_t s)
{
    if (!tc_eligible(dtype, g_in, q, k, v, /*allow_stride=*/true)) return -2;
    if (g_in.n_extra > 0 && ((reinterpret_cast<uintptr_t>(ek) | reinterpret_cast<uintptr_t>(ev)) & 15u)) return -2;
    if ((reinterpret_cast<uintptr_t>(dout) | reinterpret_cast<uintptr_t>(dq) | reinterpret_cast<uintptr_t>(dk) |
         reinterpret_cast<uintptr_t>(dv)) & 15u)
        return -2;
    const bool strided = has_stride(g_in);
    Geo g = g_in;
    Expanded ex;
    if (strided) {                               // unit-stride geometry over full-resolution copies
        for (int a = 0; a < 3; ++a) { g.st[a] = 1; g.O[a] = g.L[a]; }
        g.otot = g.ltot;
        unsigned char* base = static_cast<unsigned char*>(workspace) + simt_delta_bytes(g_in, 4) +
                              simt_extra_partial_bytes(dtype, g_in);
        const size_t rows_full = (size_t)g.B * (size_t)g.ltot * (size_t)g.Hq;
        ex.original = &g_in;
        ex.delta_full = reinterpret_cast<float*>(base);
        ex.lse_full = reinterpret_cast<float*>(base + align256(rows_full * 4));
        ex.dout_full = base + 2 * align256(rows_full * 4);
    }
    Plan plan;
    if (!make_plan(g, plan, kCols, /*with_stride=*/false, /*interleave=*/true)) return -2;
    plan.p.status = status_ptr();
    if (!plan.p.status) return -2;
    if (g.B == 0) return 0;
    if (g.Hq > 65535 || g.B > 65535) return -2;
    float* delta = reinterpret_cast<float*>(workspace);
    const Expanded* exp = strided ? &ex : nullptr;
    if (g.D <= 64)
        return dtype == 2 ? launch_bwd<64, true>(dtype, g, plan, q, k, v, ek, ev, dek, dev, out, lse, dout, dlse, dq, dk, dv, delta, s, exp)
                          : launch_bwd<64, false>(dtype, g, plan, q, k, v, ek, ev, dek, dev, out, lse, dout, dlse, dq, dk, dv, delta, s, exp);
    return dtype == 2 ? launch_bwd<128, true>(dtype, g, plan, q, k, v, ek, ev, dek, dev, out, lse, dout, dlse, dq, dk, dv, delta, s, exp)
                      : launch_bwd<128, false>(dtype, g, plan, q, k, v, ek, ev, dek, dev, out, lse, dout, dlse, dq, dk, dv, delta, s, exp);
}

// Scratch of the strided backward (full-resolution delta, lse and dout); sized for every 16-bit strided
// problem, whichever kernel family ends up serving it.
size_t tc_bwd_workspace_bytes(int dtype, const Geo& g)
{
    if ((dtype != 1 && dtype != 2) || !has_stride(g)) return 0;
    const size_t rows_full = (size_t)g.B * (size_t)g.ltot * (size_t)g.Hq;
    return 2 * align256(rows_full * 4) + align256(rows_full * (size_t)g.D * 2);
}

#ifdef NATTEN_TRACE
extern "C" int natten_trace_read_bwd(long long* host, int clear)
{
    cudaError_t e = cudaMemcpyFromSymbol(host, g_trace_bwd, sizeof(g_trace_bwd));
    if (e == cudaSuccess && clear) {
        static long long zeros[2 * 16 * 512] = {0};
        e = cudaMemcpyToSymbol(g_trace_bwd, zeros, sizeof(g_trace_bwd));
    }
    return (int)e;
}
#endif

} // namespace natten
