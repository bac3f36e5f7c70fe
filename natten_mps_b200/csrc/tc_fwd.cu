// Fused neighbourhood-attention forward on tcgen05 tensor cores (sm_100a).
//
// One CTA handles a box of 128 queries of one (batch, head): the union of their
// neighbourhoods is a box of keys, walked in chunks of 128 keys.  Per chunk
//   S = Q K^T      tcgen05.mma, operands staged by TMA (128-byte swizzle), accumulator in TMEM
//   P = exp2(S*scale*log2e - max)   softmax warps, one query row per thread, read S from TMEM,
//                                   apply the window mask, write P (16-bit) back to TMEM
//   O += P V       tcgen05.mma with A = P from TMEM, B = V tile read MN-major
// O stays in TMEM for the whole tile: the stabiliser of the stored probabilities only moves
// when a chunk's maximum exceeds it by more than 2^8 (then O and the row sum are rescaled in
// place), so there is no register accumulator.  One extra warp issues every TMA load and MMA.
// Geometry (rank, window, dilation, causal axes, per-sample extents) is runtime data; masks
// are built per 32-column piece from per-row box ranges.  Dilation is handled as independent
// sub-grids, loaded through the tensor map's element strides.
//
// TMEM columns per CTA (256):  S [0,128)  P [128,192)  O [192,256).
// Shared memory per CTA: Q 16 KB + 3 stages x (K 16 KB + V 16 KB) = 112 KB -> two CTAs per SM.
#include "tc_kernels.cuh"

#include "tc_plan.cuh"

#include <type_traits>

namespace natten {

using namespace tc;
using namespace tcplan;

namespace {

constexpr int kThreads = 288;            // 8 softmax warps + 1 TMA/MMA warp
constexpr uint32_t kColS = 0, kColP = 128;      // S: 128 columns, P: 64; O follows (64 or 128 columns)

// Shared-memory map (dynamic, base must be 1024-byte aligned).
template <int DH>
struct SmemMap {
    static constexpr int kHalves = DH / 64;                       // 64-channel blocks (one swizzle row each)
    static constexpr int kStages = DH == 64 ? 3 : 2;
    static constexpr int kHalf = kTileRows * 128;                 // bytes of one [128 x 64] 16-bit block
    static constexpr int kTile = kHalf * kHalves;                 // bytes of one [128 x DH] 16-bit tile
    static constexpr int kQ = 0;
    static constexpr int kK = kQ + kTile;
    static constexpr int kV = kK + kStages * kTile;
    static constexpr int kBar = kV + kStages * kTile;
    // barriers: q, kv_full[3], s_full, sp_ready, o_full  (8 bytes each) + tmem ptr + abort flag,
    // then 512 bytes for the two column halves to exchange their row maxima
    static constexpr int kTotal = kBar + 128 + 512;
    static constexpr uint32_t kTmemCols = DH == 64 ? 256 : 512;
    static constexpr uint32_t kColO = DH == 64 ? 192 : 256;
};

__device__ __forceinline__ int tc_window_start(int p, int L, int K) { return window_start(p, L, K, 1); }

// kInner: innermost chunk extent when it is 16 or 32 (separable row / column masks),
// 0 = any geometry (per-column validity words from piece_word).
template <int DH, bool BF16, int kInner>
__global__ void __launch_bounds__(kThreads, (DH == 64 ? 2 : 1))
tc_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
              const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmEK,
              const __grid_constant__ CUtensorMap tmEV, const __grid_constant__ TcParams P,
              uint16_t* __restrict__ out, float* __restrict__ lse)
{
    using SM = SmemMap<DH>;
    constexpr int kStages = SM::kStages;
    constexpr int CH = DH / 2;                 // output channels per softmax thread
    // One CTA per SM (D = 128) has the registers to keep a chunk's scores: they are read from TMEM once
    // and the next Q K^T is issued as soon as every thread holds them.  D = 64 reads them twice.
    constexpr bool kKeepScores = DH == 128;
    constexpr uint32_t kColO = SM::kColO, kTmemCols = SM::kTmemCols;
    extern __shared__ __align__(1024) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.y, b = blockIdx.z, hk = h / P.group;
    const int quad = warp & 3, team = (warp >> 2) & 1;        // softmax warps: TMEM lane quadrant, column half
    const int prior_abort = *reinterpret_cast<volatile int*>(P.status);   // loaded early, used at barrier set-up

    // ---- CTA geometry -------------------------------------------------------
    // origin[] counts queries of the dilation group; query i of an axis sits at sub-grid index
    // x0 + sx * i (every index when the output stride is 1).
    int rg[3], origin[3], Lp[3], lo[3], nc[3], x0[3], sx[3], nq[3], nqf[3];
    bool cta_active = cta_geometry(P, blockIdx.x, b, rg, origin, Lp);
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        sx[a] = P.qstep[a];
        x0[a] = P.qx0[a][rg[a]];
        const int lpf = (P.L[a] - rg[a] + P.dil[a] - 1) / P.dil[a];          // sub-grid length of the whole tensor
        if (x0[a] < 0) {                         // no output position falls into this dilation group
            nq[a] = 0;
            nqf[a] = 0;
            x0[a] = 0;
        } else if (sx[a] == 1) {
            nq[a] = Lp[a];
            nqf[a] = rg[a] < P.L[a] ? lpf : 0;
        } else {
            nq[a] = (x0[a] >= 0 && x0[a] < Lp[a]) ? (Lp[a] - x0[a] + sx[a] - 1) / sx[a] : 0;
            nqf[a] = (x0[a] >= 0 && x0[a] < lpf) ? (lpf - x0[a] + sx[a] - 1) / sx[a] : 0;
        }
        if (origin[a] >= nq[a]) cta_active = false;
    }
    int nnb = 1;                             // chunks of the neighbourhood box
    if (cta_active) {
#pragma unroll
        for (int a = 0; a < 3; ++a) {
            const int lastq = origin[a] + P.tile[a] - 1 < nq[a] - 1 ? origin[a] + P.tile[a] - 1 : nq[a] - 1;
            const int xf = x0[a] + sx[a] * origin[a], xl = x0[a] + sx[a] * lastq;
            lo[a] = P.causal[a] ? xf - (P.K[a] - 1) : tc_window_start(xf, Lp[a], P.K[a]);
            const int hi = P.causal[a] ? xl : tc_window_start(xl, Lp[a], P.K[a]) + P.K[a] - 1;
            nc[a] = chunks_along(P, a, hi - lo[a] + 1);       // chunks this tile really needs
            nnb *= nc[a];
        }
    }
    const int nch = nnb + ((P.n_extra + kChunk - 1) >> 7);   // then the additional tokens, 128 per chunk

    if (!cta_active) {                       // nothing to attend: rows that exist in the output are zero
        if (warp < 8) {
            int qi[3];
            row_offsets(P, quad * 32 + lane, qi);
            bool inside = true;
            long long oflat = 0;
#pragma unroll
            for (int a = 0; a < 3; ++a) {
                const int qa = origin[a] + qi[a];
                if (qa >= nqf[a]) inside = false;
                const int pa = rg[a] + P.dil[a] * (x0[a] + sx[a] * qa);
                oflat = oflat * P.O[a] + (P.st[a] == 1 ? pa : pa / P.st[a]);
            }
            if (inside) {
                const long long orow = ((long long)b * P.otot + oflat) * P.Hq + h;
                uint4* o4 = reinterpret_cast<uint4*>(out + orow * P.dreal + team * CH);
#pragma unroll
                for (int i = 0; i < CH / 8; ++i)
                    if (team * CH + 8 * i < P.dreal) o4[i] = make_uint4(0, 0, 0, 0);
                if (team == 0) lse[orow] = 0.f;
            }
        }
        return;
    }

    // ---- shared memory, barriers, TMEM --------------------------------------
    const uint32_t sbase = smem_u32(smem);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::kBar + 64);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SM::kBar + 72);
    uint16_t* xmax = reinterpret_cast<uint16_t*>(smem + SM::kBar + 128);      // [2][128] partial row maxima (bf16 bits)
    const uint32_t bar_q = sbase + SM::kBar + 0;
    const uint32_t bar_kv = sbase + SM::kBar + 8;       // [3]
    const uint32_t bar_s = sbase + SM::kBar + 32;
    const uint32_t bar_sp = sbase + SM::kBar + 40;
    const uint32_t bar_o = sbase + SM::kBar + 48;
    const uint32_t bar_sr = sbase + SM::kBar + 56;      // (kKeepScores) every softmax thread holds S(c) in registers

    // The issuing warp sets up the barriers, allocates TMEM and starts the first loads right away,
    // so they are in flight while the softmax warps are still working out their row geometry.
    int ld[3] = {0, 0, 0};                       // chunk counters of the next load
    int loaded = 0;
    auto issue_kv = [&]() {
        const int s = loaded % kStages;
        const uint32_t bar = bar_kv + 8 * s;
        mbar_expect_tx(bar, 2 * SM::kTile);
        if (loaded < nnb) {
            int X[3];
#pragma unroll
            for (int a = 0; a < 3; ++a) X[a] = rg[a] + P.dil[a] * (lo[a] + ld[a] * P.cb[a]);
#pragma unroll
            for (int hf = 0; hf < SM::kHalves; ++hf) {
                tma_load_heads(sbase + SM::kK + s * SM::kTile + hf * SM::kHalf, &tmK, bar, P, DH, hk * DH + 64 * hf, X[2], X[1], X[0], b);
                tma_load_heads(sbase + SM::kV + s * SM::kTile + hf * SM::kHalf, &tmV, bar, P, DH, hk * DH + 64 * hf, X[2], X[1], X[0], b);
            }
            if (++ld[2] == nc[2]) { ld[2] = 0; if (++ld[1] == nc[1]) { ld[1] = 0; ++ld[0]; } }
        } else {                                 // additional tokens (rows past n_extra are zero-filled)
            const int e0 = (loaded - nnb) * kChunk;
#pragma unroll
            for (int hf = 0; hf < SM::kHalves; ++hf) {
                tma_load_heads(sbase + SM::kK + s * SM::kTile + hf * SM::kHalf, &tmEK, bar, P, DH, hk * DH + 64 * hf, e0, 0, 0, b);
                tma_load_heads(sbase + SM::kV + s * SM::kTile + hf * SM::kHalf, &tmEV, bar, P, DH, hk * DH + 64 * hf, e0, 0, 0, b);
            }
        }
        ++loaded;
    };
    if (warp == 8) {
        if (lane == 0) {
            // swizzled tiles need a 1024-byte aligned base; once any CTA has given up, the rest bail out
            *abort_flag = ((sbase & 1023u) || prior_abort) ? 1 : 0;
            mbar_init(bar_q, 1);
            for (int s = 0; s < kStages; ++s) mbar_init(bar_kv + 8 * s, 1);
            mbar_init(bar_s, 1);
            mbar_init(bar_sp, 256);
            mbar_init(bar_o, 1);
            mbar_init(bar_sr, 256);
            mbar_init_fence();
            fence_async_smem();
            if (!*abort_flag) {
                mbar_expect_tx(bar_q, SM::kTile + (P.inject == 1 ? 16u : 0u));
#pragma unroll
                for (int hf = 0; hf < SM::kHalves; ++hf)
                    tma_load_heads(sbase + SM::kQ + hf * SM::kHalf, &tmQ, bar_q, P, DH, h * DH + 64 * hf,
                                rg[2] + P.dil[2] * (x0[2] + sx[2] * origin[2]), rg[1] + P.dil[1] * (x0[1] + sx[1] * origin[1]),
                                rg[0] + P.dil[0] * (x0[0] + sx[0] * origin[0]), b);
                for (int c = 0; c < nch && c < kStages; ++c) issue_kv();
            }
        }
        __syncwarp();
        tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    }
    // ---- per-thread query row (softmax warps) -------------------------------
    int f[3] = {0, 0, 0}, e[3] = {0, 0, 0};
    bool valid_q = false, in_tensor = false;
    long long out_row = 0;
    if (warp < 8) {
        int qi[3];
        row_offsets(P, quad * 32 + lane, qi);
        valid_q = true; in_tensor = true;
        long long oflat = 0;
#pragma unroll
        for (int a = 0; a < 3; ++a) {
            const int qa = origin[a] + qi[a];                 // query count along the axis
            const int xq = x0[a] + sx[a] * qa;                // its sub-grid index
            const int pa = rg[a] + P.dil[a] * xq;             // its position in the tensor
            if (qa >= nq[a]) valid_q = false;
            if (qa >= nqf[a]) in_tensor = false;
            oflat = oflat * P.O[a] + (P.st[a] == 1 ? pa : pa / P.st[a]);
            if (cta_active) {
                const int first = P.causal[a] ? xq - (P.K[a] - 1) : tc_window_start(xq, Lp[a], P.K[a]);
                f[a] = (first > 0 ? first : 0) - lo[a];
                e[a] = (first + P.K[a] < Lp[a] ? first + P.K[a] : Lp[a]) - lo[a];
            }
        }
        if (!valid_q) { e[0] = f[0]; e[1] = f[1]; e[2] = f[2]; }
        out_row = (((long long)b * P.otot + oflat) * P.Hq + h);
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 8) {
        // =====================================================================
        // TMA + MMA issue: the warp runs the loop converged, the tensor-core instructions execute on an
        // elected lane (a thread issuing alone from a divergent branch pays for every operand it moves into
        // the uniform registers those instructions take)
        // =====================================================================
        const uint32_t leader = elect_one();
        if (!*abort_flag) {
            constexpr uint32_t idesc_qk = instr_desc(BF16 ? 1 : 0, kChunk, 0, 0);
            constexpr uint32_t idesc_pv = instr_desc(BF16 ? 1 : 0, DH, 0, 1);
            const uint64_t dq0 = smem_desc(sbase + SM::kQ, 16, 1024);
            int qc[3] = {0, 0, 0};                   // chunk index per axis of the next Q K^T (per-sample extents only)
            auto issue_qk = [&](int c) {
                if (P.extents && c < nnb) {
                    const int box0[3] = {lo[0] + qc[0] * P.cb[0], lo[1] + qc[1] * P.cb[1], lo[2] + qc[2] * P.cb[2]};
                    if (leader)
                        zero_rows_past_extent(P, box0, Lp, kChunk, SM::kHalves, SM::kHalf,
                                              smem + SM::kK + (c % kStages) * SM::kTile, smem + SM::kV + (c % kStages) * SM::kTile);
                    __syncwarp();
                    if (++qc[2] == nc[2]) { qc[2] = 0; if (++qc[1] == nc[1]) { qc[1] = 0; ++qc[0]; } }
                }
                const uint64_t dk0 = smem_desc(sbase + SM::kK + (c % kStages) * SM::kTile, 16, 1024);
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < DH / 16; ++ks) {       // 32 bytes per k-step inside a 64-channel block
                    const uint32_t off = ((ks / 4) * SM::kHalf + (ks % 4) * 32) >> 4;
                    mma_ss_e(tmem + kColS, dq0 + off, dk0 + off, idesc_qk, ks > 0, leader);
                }
                mma_commit_e(bar_s, leader);
            };
            auto issue_pv = [&](int c) {
                // V read MN-major: 16 key rows per k-step, the second 64-channel block sits kHalf bytes further.
                // O stays in TMEM for the whole tile: every chunk after the first adds to it.
                const uint64_t dv0 = smem_desc(sbase + SM::kV + (c % kStages) * SM::kTile, SM::kHalf, 1024);
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < kChunk / 16; ++ks)
                    mma_ts_e(tmem + kColO, tmem + kColP + 8 * ks, dv0 + 128 * ks, idesc_pv, c > 0 || ks > 0, leader);
                mma_commit_e(bar_o, leader);
            };
            bool ok = mbar_wait(bar_q, 0, abort_flag, P.wait_budget);
            ok = ok && mbar_wait(bar_kv, 0, abort_flag, P.wait_budget);
            if (ok) issue_qk(0);
            for (int c = 0; c < nch && ok; ++c) {
                if (kKeepScores) {       // S(c) sits in the threads' registers: the next scores may overwrite it
                    ok = mbar_wait(bar_sr, c & 1, abort_flag, P.wait_budget);
                    if (!ok) break;
                    if (c + 1 < nch) {
                        ok = mbar_wait(bar_kv + 8 * ((c + 1) % kStages), ((c + 1) / kStages) & 1, abort_flag, P.wait_budget);
                        if (!ok) break;
                        issue_qk(c + 1);
                    }
                }
                ok = mbar_wait(bar_sp, c & 1, abort_flag, P.wait_budget);           // S(c) consumed, P(c) stored
                if (!ok) break;
                if (!kKeepScores && c + 1 < nch) {                   // next scores first: the threads wait for them
                    ok = mbar_wait(bar_kv + 8 * ((c + 1) % kStages), ((c + 1) / kStages) & 1, abort_flag, P.wait_budget);
                    if (!ok) break;
                    issue_qk(c + 1);
                }
                issue_pv(c);
                if (c + kStages < nch) {
                    ok = mbar_wait(bar_o, c & 1, abort_flag, P.wait_budget);        // stage c % kStages is free again
                    if (!ok) break;
                    if (leader) issue_kv();
                    __syncwarp();
                }
            }
        }
    } else {
        // =====================================================================
        // softmax warps: thread = (query row, 64-column half of the chunk, 32 output channels)
        // =====================================================================
        const uint32_t trow = tmem + (static_cast<uint32_t>(quad * 32) << 16);
        const int row = quad * 32 + lane;
        bool ok = true;
        // O accumulates in TMEM over the tile's chunks.  m is the stabiliser the stored
        // probabilities use; it only moves (and O, l are rescaled) when a chunk's maximum
        // exceeds it by more than 2^8, so probabilities stay below 256.
        float m = -INFINITY, l = 0.f;
        int ci[3] = {0, 0, 0};
        uint32_t colbits = 0u;               // separable geometry: valid columns of one inner row
        int cached_c2 = -1;

        for (int c = 0; c < nch; ++c) {
            // ---- validity words of this thread's two 32-column pieces ----
            uint32_t words[2];
            if (c >= nnb) {                // additional tokens: every live row sees the first n_extra columns
#pragma unroll
                for (int pc = 0; pc < 2; ++pc)
                    words[pc] = valid_q ? low_bits(P.n_extra - ((c - nnb) * kChunk + 64 * team + 32 * pc)) : 0u;
            } else if constexpr (kInner > 0) {
                if (ci[2] != cached_c2) {
                    cached_c2 = ci[2];
                    int lo2 = f[2] - ci[2] * kInner, hi2 = e[2] - ci[2] * kInner;
                    lo2 = lo2 > 0 ? lo2 : 0;
                    hi2 = hi2 < kInner ? hi2 : kInner;
                    colbits = hi2 > lo2 ? (low_bits(hi2 - lo2) << lo2) : 0u;
                }
#pragma unroll
                for (int pc = 0; pc < 2; ++pc) {
                    uint32_t w = 0u;
#pragma unroll
                    for (int t = 0; t < 32 / kInner; ++t) {
                        const int jj = 64 * team + 32 * pc + t * kInner;
                        const int j1 = (jj >> P.cb2_log) & (P.cb[1] - 1);
                        const int j0 = jj >> (P.cb2_log + P.cb1_log);
                        const int i0 = ci[0] * P.cb[0] + j0, i1 = ci[1] * P.cb[1] + j1;
                        if (i0 >= f[0] && i0 < e[0] && i1 >= f[1] && i1 < e[1]) w |= colbits << (t * kInner);
                    }
                    words[pc] = w;
                }
            } else {
#pragma unroll
                for (int pc = 0; pc < 2; ++pc) words[pc] = piece_word(P, ci, 2 * team + pc, f, e);
            }

            ok = ok && mbar_wait(bar_s, c & 1, abort_flag, P.wait_budget);
            tc_fence_after();
            const bool any[2] = {__any_sync(0xffffffffu, words[0] != 0u) != 0, __any_sync(0xffffffffu, words[1] != 0u) != 0};
            uint32_t s0[kKeepScores ? 32 : 1], s1[kKeepScores ? 32 : 1];      // the chunk's scores (kKeepScores)
            float mc = -INFINITY;
            if constexpr (kKeepScores) {
                if (any[0]) tmem_ld32(trow + kColS + 64 * team, s0);
                if (any[1]) tmem_ld32(trow + kColS + 64 * team + 32, s1);
                tmem_ld_wait();
                // columns outside the row's neighbourhood become -inf once, here
                auto masked_max = [&](uint32_t (&s)[kKeepScores ? 32 : 1], uint32_t w) {
                    float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            if (!((w >> (i + j)) & 1u)) s[i + j] = 0xff800000u;
                        m0 = fmaxf(m0, __uint_as_float(s[i]));
                        m1 = fmaxf(m1, __uint_as_float(s[i + 1]));
                        m2 = fmaxf(m2, __uint_as_float(s[i + 2]));
                        m3 = fmaxf(m3, __uint_as_float(s[i + 3]));
                    }
                    mc = fmaxf(mc, fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)));
                };
                if (any[0]) masked_max(s0, words[0]);
                if (any[1]) masked_max(s1, words[1]);
            } else {
                // ---- pass 1: maximum over the valid columns of this half ----
#pragma unroll
                for (int pc = 0; pc < 2; ++pc) {
                    if (!any[pc]) continue;
                    uint32_t s[32];
                    tmem_ld32(trow + kColS + 64 * team + 32 * pc, s);
                    tmem_ld_wait();
                    float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {        // guarded maxima: one predicate and one max per column
                        if ((words[pc] >> i) & 1u) m0 = fmaxf(m0, __uint_as_float(s[i]));
                        if ((words[pc] >> (i + 1)) & 1u) m1 = fmaxf(m1, __uint_as_float(s[i + 1]));
                        if ((words[pc] >> (i + 2)) & 1u) m2 = fmaxf(m2, __uint_as_float(s[i + 2]));
                        if ((words[pc] >> (i + 3)) & 1u) m3 = fmaxf(m3, __uint_as_float(s[i + 3]));
                    }
                    mc = fmaxf(mc, fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)));
                }
            }
            if (!ok) mc = -INFINITY;
            {
                // Both halves must use one maximum.  Each publishes its own rounded up to bf16
                // (any value >= the true maximum works as the stabiliser) and takes the larger.
                uint32_t bits = __float_as_uint(mc);
                bits = (mc >= 0.f) ? ((bits + 0xFFFFu) & 0xFFFF0000u) : (bits & 0xFFFF0000u);
                xmax[team * 128 + row] = static_cast<uint16_t>(bits >> 16);
                asm volatile("bar.sync %0, 64;" ::"r"(1 + quad) : "memory");
                const uint32_t other = static_cast<uint32_t>(xmax[(1 - team) * 128 + row]) << 16;
                mc = fmaxf(__uint_as_float(bits), __uint_as_float(other));
            }
            if constexpr (kKeepScores) {
                // S(c) is in registers and the partner's maximum has been read: the next scores may
                // land (they are what lets this thread overwrite its exchange slot again).
                tc_fence_before();
                mbar_arrive(bar_sr);
            }

            // ---- P(c-1) V has finished: P may be rewritten, O may be rescaled ----
            if (c > 0) {
                ok = ok && mbar_wait(bar_o, (c - 1) & 1, abort_flag, P.wait_budget);
                tc_fence_after();
            }
            bool grow = false;
            if (mc > -INFINITY) {
                if (m == -INFINITY) m = mc;
                else grow = (mc - m) * P.scale_log2 > 8.f;
            }
            if (__any_sync(0xffffffffu, grow)) {          // rare: both halves of a row decide alike
                const float fac = grow ? fast_exp2((m - mc) * P.scale_log2) : 1.f;
#pragma unroll 1
                for (int part = 0; part < CH / 16; ++part) {
                    uint32_t o[16];
                    tmem_ld16(trow + kColO + CH * team + 16 * part, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * fac);
                    tmem_st16(trow + kColO + CH * team + 16 * part, o);
                }
                l *= fac;
                if (grow) m = mc;
            }
            const float mb = (m == -INFINITY) ? 0.f : m * P.scale_log2;

            // ---- probabilities -> TMEM (16-bit pairs), row sum of this half ----
            float r0 = 0.f, r1 = 0.f;
#pragma unroll
            for (int pc = 0; pc < 2; ++pc) {
                uint32_t packed[16];
                if (any[pc]) {
                    if constexpr (kKeepScores) {
                        const uint32_t (&s)[kKeepScores ? 32 : 1] = pc == 0 ? s0 : s1;
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const float p0 = fast_exp2(fmaf(__uint_as_float(s[2 * i]), P.scale_log2, -mb));
                            const float p1 = fast_exp2(fmaf(__uint_as_float(s[2 * i + 1]), P.scale_log2, -mb));
                            r0 += p0;
                            r1 += p1;
                            packed[i] = cvt_pack<BF16>(p0, p1);
                        }
                    } else {                                         // pass 2 over TMEM
                        uint32_t s[32];
                        tmem_ld32(trow + kColS + 64 * team + 32 * pc, s);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            float p0 = fast_exp2(fmaf(__uint_as_float(s[2 * i]), P.scale_log2, -mb));
                            float p1 = fast_exp2(fmaf(__uint_as_float(s[2 * i + 1]), P.scale_log2, -mb));
                            if (!((words[pc] >> (2 * i)) & 1u)) p0 = 0.f;
                            if (!((words[pc] >> (2 * i + 1)) & 1u)) p1 = 0.f;
                            r0 += p0;
                            r1 += p1;
                            packed[i] = cvt_pack<BF16>(p0, p1);
                        }
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) packed[i] = 0u;
                }
                tmem_st16(trow + kColP + 32 * team + 16 * pc, packed);
            }
            l += ok ? r0 + r1 : 0.f;
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(bar_sp);
            if (++ci[2] == nc[2]) { ci[2] = 0; if (++ci[1] == nc[1]) { ci[1] = 0; ++ci[0]; } }
        }

        // ---- combine the two halves' sums while the last P V runs, then normalise and write out ----
        // Every Q K^T has finished and no load is in flight, so the first K stage can carry the sums.
        {
            float* xsum = reinterpret_cast<float*>(smem + SM::kK);
            xsum[team * 128 + row] = l;
            asm volatile("bar.sync %0, 64;" ::"r"(1 + quad) : "memory");
            l += xsum[(1 - team) * 128 + row];
        }
        ok = ok && mbar_wait(bar_o, (nch - 1) & 1, abort_flag, P.wait_budget);
        tc_fence_after();
        {
            const bool live = valid_q && ok;
#pragma unroll
            for (int part = 0; part < CH / 32; ++part) {
                uint32_t o[32];
                tmem_ld32(trow + kColO + CH * team + 32 * part, o);
                tmem_ld_wait();
                const float inv = (live && l > 0.f) ? 1.f / l : 0.f;
                if (in_tensor) {
                    uint4* o4 = reinterpret_cast<uint4*>(out + out_row * P.dreal + team * CH + 32 * part);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if (team * CH + 32 * part + 8 * i >= P.dreal) break;      // padded channels are not part of the output
                        uint32_t w[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            w[j] = cvt_pack<BF16>(__uint_as_float(o[8 * i + 2 * j]) * inv, __uint_as_float(o[8 * i + 2 * j + 1]) * inv);
                        o4[i] = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
            // natural-log lse of scale * logits
            if (in_tensor && team == 0)
                lse[out_row] = (live && l > 0.f) ? (m * P.scale_log2 + log2f(l)) * 0.6931471805599453f : 0.f;
        }
    }

    if (*abort_flag) abort_grace_sleep();       // loads of a wait that gave up may still be landing
    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
        if (lane == 0 && *abort_flag) atomicExch(P.status, 1);
    }
}

} // namespace

int tc_fused_fwd(int dtype, const Geo& g, const void* q, const void* k, const void* v, const void* ek,
                 const void* ev, void* out, void* lse, cudaStream_t s)
{
    if (!tc_eligible(dtype, g, q, k, v, /*allow_stride=*/true)) return -2;
    if (g.n_extra > 0 && ((reinterpret_cast<uintptr_t>(ek) | reinterpret_cast<uintptr_t>(ev)) & 15u)) return -2;
    Plan plan;
    if (!make_plan(g, plan, kChunk, /*with_stride=*/true)) return -2;
    const bool bf16 = dtype == 2;
    CUtensorMap mq, mk, mv, mek, mev;
    if (!encode_map(&mq, q, bf16, plan.p, g.Hq, g.D, g.qs, plan.box_q, /*query_lattice=*/true) ||
        !encode_map(&mk, k, bf16, plan.p, g.Hkv, g.D, g.ks, plan.box_kv) ||
        !encode_map(&mv, v, bf16, plan.p, g.Hkv, g.Dv, g.vs, plan.box_kv))
        return -2;
    mek = mk; mev = mv;                      // placeholders when there are no additional tokens
    if (g.n_extra > 0 && (!encode_extra_map(&mek, ek, bf16, g.B, g.n_extra, g.Hkv, g.D, kChunk, plan.p.split_heads) ||
                          !encode_extra_map(&mev, ev, bf16, g.B, g.n_extra, g.Hkv, g.Dv, kChunk, plan.p.split_heads)))
        return -2;
    plan.p.status = status_ptr();
    if (!plan.p.status) return -2;
    int ngroups = 1;
    for (int a = 0; a < 3; ++a) ngroups *= plan.p.grp_n[a];     // dilation groups that hold queries
    const dim3 grid((unsigned)(plan.p.ntiles * ngroups), (unsigned)g.Hq, (unsigned)g.B);
    if (grid.x == 0 || g.B == 0) return 0;
    if (g.Hq > 65535 || g.B > 65535) return -2;
    cudaError_t err;
    auto launch = [&](auto dh, auto bf, auto inner) {
        constexpr int kDh = decltype(dh)::value;
        constexpr bool kBf = decltype(bf)::value;
        constexpr int kInner = decltype(inner)::value;
        using SM = SmemMap<kDh>;
        ensure_dynamic_smem((const void*)tc_fwd_kernel<kDh, kBf, kInner>, SM::kTotal);
        tc_fwd_kernel<kDh, kBf, kInner><<<grid, kThreads, SM::kTotal, s>>>(mq, mk, mv, mek, mev, plan.p, (uint16_t*)out, (float*)lse);
    };
    auto by_inner = [&](auto dh, auto bf) {
        if (plan.p.cb[2] == 16) launch(dh, bf, std::integral_constant<int, 16>{});
        else if (plan.p.cb[2] == 32) launch(dh, bf, std::integral_constant<int, 32>{});
        else launch(dh, bf, std::integral_constant<int, 0>{});
    };
    auto by_type = [&](auto dh) {
        if (bf16) by_inner(dh, std::true_type{});
        else by_inner(dh, std::false_type{});
    };
    if (g.D <= 64) by_type(std::integral_constant<int, 64>{});
    else by_type(std::integral_constant<int, 128>{});
    err = cudaGetLastError();
    tc_count_launch();
    return err == cudaSuccess ? 0 : (int)err;
}

static unsigned long long g_tc_launches = 0;
void tc_count_launch() { ++g_tc_launches; }
unsigned long long tc_launch_count() { return g_tc_launches; }

} // namespace natten
